/* Testing aids of libmolla_sample_testing.so: the same library compiled with
 * -DMOLLA_SAMPLE_TESTING. None of them has a counterpart in the reference, and none exists in
 * libmolla_sample.so: the production kernels carry no profiling stamps and take no experiment
 * switches. The three switches are process-wide and not thread-safe: set, call, reset. */
#ifndef MOLLA_SAMPLE_TESTING_H
#define MOLLA_SAMPLE_TESTING_H

#include "molla_sample.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Experiment switches of the row kernels. Streaming kernel: bit 1 no last-use hint on the second
 * pass over a row, bit 2 no keep hint on list traffic, bit 3 no help from idle blocks. Both
 * kernels: bit 4 pretends, after the row has arrived, that one warp's bounded wait ran out
 * (nothing is withheld and nothing is left waiting): the row must come back with
 * MOLLA_ROW_LOAD_TIMEOUT, token -1 and its sampler state untouched. 0 = production behaviour. */
void molla_sample_debug_knobs(int32_t knobs);

/* When given a device buffer of B x 32 int64, later calls record clock64() stamps at the phase
 * boundaries of each row (NULL switches it off again). */
void molla_sample_debug_profile(void *d_stamps);

/* When given a device buffer of B x cap int32, later calls write, for every row sampled with
 * 1 < top_k < 128, the ids that survive top-k (`_top_k`, sample.mojo:485-490) in descending
 * probability, padded with -1 (NULL switches it off again). */
void molla_sample_debug_topk(void *d_ids, int32_t cap);

#ifdef __cplusplus
}
#endif
#endif /* MOLLA_SAMPLE_TESTING_H */
