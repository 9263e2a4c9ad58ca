// The launch of the one-row-per-cluster kernel (molla_cluster.cu), called by the entry points
// in molla_sample.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

struct BatchArgs;

constexpr int MOLLA_CLUSTER_DECLINED = 1;  // the vocabulary is too wide for a cluster, or the device cannot hold one

// Enqueues the sampling of `a.B` rows on `st`. `d_workspace` is the caller's workspace (the row
// order is written behind its first 256 bytes). Returns MOLLA_OK, MOLLA_CLUSTER_DECLINED (nothing
// was launched) or a MOLLA_ERR_* code with its message in `err`.
int molla_cluster_launch(const BatchArgs &a, void *d_workspace, cudaStream_t st, char *err, size_t errlen);
