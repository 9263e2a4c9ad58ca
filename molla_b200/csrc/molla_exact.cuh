// Device functions shared by the sampling kernels: the exact sequential fp32 sum, the search
// over value bins, the sorted walk and typical-p. Everything here works on a thread block of NT
// threads and on a context object `c` with members tid, lane, warp, status and `A`, a pointer to
// the block's scratch in shared memory (the member names used below). The sizes NBINS and NC
// can be set per translation unit before this file is included.
#pragma once
#include <type_traits>

#include "molla_device.cuh"
#include "../../include/molla_sample.h"

using namespace molla;

// Everything a launch needs: the same structure in every translation unit of the library.
struct BatchArgs {
    const float *logits; long long row_stride; int B, V;
    const float *temperature; const int *top_k; const float *top_p; const float *min_p;
    const float *typical_p; const float *repeat_penalty; const float *frequency_penalty;
    const float *presence_penalty; const unsigned char *window_on;
    const unsigned long long *seed; const unsigned long long *drawn;
    const long long *hist; const int *hist_off;
    const long long *bias_ids; const float *bias_vals; const int *bias_off;
    int *tokens; unsigned int *row_status; float *diag;
    float *penalised;  // optional dump [B x V]
    int penalised_only;
    int R;                       // floats per warp region (multiple of 4)
    int *row_counter;            // scratch: next row to hand out (zeroed before the launch)
    const int *order;            // scratch: rows by decreasing cost (NULL = as given)
    unsigned long long *wlist;   // scratch: per CTA, 2 x 16 x R list entries
#ifdef MOLLA_SAMPLE_TESTING
    long long *prof;             // optional [B x 32] clock64 stamps per row
    int knobs;                   // experiment switches (0 = production behaviour)
    int *topk_out; int topk_cap; // optional [B x cap] ids of the sorted head after top-k
#endif
    // thread blocks that ran out of rows help the ones still converting a long list (HelpSlot)
    void *help;                  // [grid] HelpSlot, one per thread block, or nullptr
    unsigned int *help_tables;   // [grid x HELP_TABLE_WORDS]
    int *rows_done;              // rows finished so far (zeroed before the launch)
    // decode-step form: which row of the logit block each batch row reads, which slot of the
    // per-stream arrays (settings and state) it uses, the final-logit softcap, and the state
    const int *rows;             // [B] or nullptr (row r reads logit row r)
    const int *slot;             // [B] or nullptr (row r uses slot r)
    float softcap;               // 0 = none
    long long *ring;             // [slots x ring_cap] token windows, or nullptr (windows come from hist)
    int ring_cap;
    int *ring_head, *ring_filled;
    const int *ring_len;         // [slots] repeat_last_n of every slot (0 = penalties off)
    unsigned long long *drawn_rw;  // [slots] draw counters, advanced by one per pick
    const long long *stop_token;   // [slots] or nullptr
    unsigned char *stopped;        // [B] or nullptr: the pick was the slot's stop token
    // vocab-sharded form: this GPU holds columns [col0, col0 + V) of a vocabulary of Vg
    int n_logit_rows, n_slots;   // bounds of rows[] and slot[] values (0 = not given)
    const unsigned int *mask; long long mask_stride;  // grammar mask: bit t of row r's words = token t allowed (nullptr = all)
    // one row per thread-block cluster: blocks per cluster, logits per block, logits per thread
    int G, Vc, L;
    int mode;                    // 0 whole pipeline; 1, 2, 3 the stages around the two all-gathers
    int col0, Vg;
    float *sa_out;               // stage 1 out: [B x SA_WORDS] summary of the slice
    const float *sb_in;          // stages 2, 3 in: [B x 4] global max, head threshold, sum bound before the slice, global argmax
    unsigned long long *sb_list; int *sb_count; int list_cap;     // stage 2 out: the slice's list
    const unsigned long long *sc_list; const int *sc_count; int world;  // stage 3 in: [world][B][cap], [world][B]
};

namespace {

#ifndef MOLLA_NBINS_LOG2
#define MOLLA_NBINS_LOG2 11
#endif
#ifndef MOLLA_NC
#define MOLLA_NC 2048
#endif
constexpr int NBINS_LOG2 = MOLLA_NBINS_LOG2;
constexpr int NBINS = 1 << NBINS_LOG2;   // histogram bins over the top bits of a value in [0, 1]
constexpr int BIN_SHIFT = 30 - NBINS_LOG2;  // 2048 bins: sign + 8 exponent + 4 mantissa bits
constexpr int BIN_SHIFT2 = BIN_SHIFT > NBINS_LOG2 ? BIN_SHIFT - NBINS_LOG2 : 0;  // a crowded bin split again: the next bits
constexpr int BPT = NBINS / NT;      // bins per thread in the bin search
constexpr int NC = MOLLA_NC;         // candidate-list capacity (gathered bins)
constexpr int HEADC = 1024;          // head-list capacity
constexpr int HEAD_NEED = 128;       // the sorted head covers top-k + 1 up to this many
constexpr int HSLOTS = 2048;         // hash slots for penalised / biased tokens
constexpr int PATCH_MAX = 1024;      // window + bias entries per row
constexpr short SUS = -32768;        // chunk that must be replayed sequentially
constexpr int TOPN_MAX = 20;
constexpr float REL_MARGIN = 17.6f;  // > 25 ln 2 = 17.33: this far below ln(running sum) nothing can matter
constexpr int ORDER_CAP = 4096;      // rows whose order is sorted by cost
static_assert(NBINS % NT == 0 && NC % NT == 0 && HEADC <= NC, "table sizes must be multiples of the block size");
static_assert((1 << BIN_SHIFT2) <= NBINS, "the third level of the bin search looks at single values");

// The testing build (-DMOLLA_SAMPLE_TESTING) carries experiment switches and profiling stamps;
// the production build has neither.
#ifdef MOLLA_SAMPLE_TESTING
#define MOLLA_KNOB(a, bit) (((a).knobs & (bit)) != 0)
#else
#define MOLLA_KNOB(a, bit) false
#endif

// Tell the compiler which address space a pointer is in (functions it does not inline would
// otherwise use generic loads, stores and atomics on shared memory).
#define IN_SHARED(ptr) __builtin_assume(__isShared(ptr))


enum { EV_NONE = 0, EV_CUT = 1, EV_DRAW = 2, EV_LIMIT = 3, EV_EXHAUSTED = 4, EV_DEGENERATE = 5 };

// ---- block collectives (NT threads) ----------------------------------------------
template <class CX>
__device__ __forceinline__ void block_argmax(CX &c, float &v, int &i) {
    warp_argmax(v, i);
    __syncthreads();
    if (c.lane == 0) { c.A->wsf[c.warp] = v; c.A->wsi[c.warp] = i; }
    __syncthreads();
    float bv = c.A->wsf[0];
    int bi = c.A->wsi[0];
#pragma unroll
    for (int w = 1; w < NWARP; w++) {
        float ov = c.A->wsf[w];
        int oi = c.A->wsi[w];
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    v = bv; i = bi;
}

// bitonic sort, descending, of n2 (power of two) keys in shared memory
__device__ void bitonic_desc(unsigned long long *k, int n2, int tid) {
    IN_SHARED(k);
    // A warp's 32 consecutive pair indices cover 64 consecutive keys whenever the stride is at
    // most 16, the same 64 for every such stride: those stages only need the warp to agree.
    bool local = false;  // the previous stage was such a stage
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1, ls = 31 - __clz(size >> 1); stride > 0; stride >>= 1, ls--) {
            if (local && stride <= 16) __syncwarp(); else __syncthreads();
            local = stride <= 16 && !(size == 2);
            for (int i = tid; i < (n2 >> 1); i += NT) {
                int pos = ((i >> ls) << (ls + 1)) + (i & (stride - 1));  // strides are powers of two: no division
                int par = pos + stride;
                bool desc = ((pos & size) == 0);
                unsigned long long x = k[pos], y = k[par];
                if ((x < y) == desc) { k[pos] = y; k[par] = x; }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ unsigned int fkey(float f) {  // order-preserving key of a float
    unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(unsigned int k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ int key_idx(unsigned long long k) {
    return (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull));
}
__device__ __forceinline__ float key_val(unsigned long long k) {
    return __uint_as_float((unsigned int)(k >> 32));
}
__device__ __forceinline__ unsigned long long make_key(unsigned int ebits, int idx) {
    return ((unsigned long long)ebits << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)idx);
}

__device__ __forceinline__ int hslot(int tok) { return (int)(((unsigned int)tok * 2654435761u) >> 21); }

// =============================================================================
// The exact sequential fp32 sum of the list's values, in list (= vocabulary) order.
// =============================================================================
// Every thread owns L consecutive entries. From approximate prefix sums each chunk
// guesses the binade(s) the true running sum can be in when it reaches the chunk (a
// margin of 2^-12 covers the rounding drift of the true sum) and adds up its terms'
// integer contributions for that binade (`pa`) and, when the guess straddles a power
// of two, for the next one (`pb`). Chunks holding a rounding tie, a term >= sum/4, or
// a span of more than two binades are replayed term by term. Thread 0 then carries
// the exact sum across the list from those tables (`p1_walk`), optionally stopping at
// the first entry whose running sum exceeds a target.
struct Walker {
    float s; int found; int at; int slow;
    int nsim = 0, nel = 0;  // replays and entries replayed (diagnostics)
};

// value accessors (shared memory): a list of (value bits << 32 | ~id) keys, or bare value bits
struct ValKeys {
    const unsigned long long *p;
    __device__ __forceinline__ float operator()(int i) const { IN_SHARED(p); return __uint_as_float((unsigned int)(p[i] >> 32)); }
};
struct ValBits {
    const unsigned int *p;
    __device__ __forceinline__ float operator()(int i) const { IN_SHARED(p); return __uint_as_float(p[i]); }
};

template <bool LOCATE, class V>
__device__ __forceinline__ void p1_sim_t(V lst, int i0, int i1, float target, Walker &w) {
    float s = w.s;
    int i = i0;
    for (; i + 8 <= i1; i += 8) {  // the loads do not depend on the running sum: fetch eight, then add
        float v[8];
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = lst(i + q);
#pragma unroll
        for (int q = 0; q < 8; q++) {
            s = __fadd_rn(s, v[q]);
            if (LOCATE && !w.found && target < s) { w.found = 1; w.at = i + q; }
        }
        if (LOCATE && w.found) { w.s = s; return; }
    }
    if (i < i1) {
        // the last few in one batch as well (their loads would otherwise wait for one another);
        // what lies past the end is read from inside the range and not added
        const int rem = i1 - i;
        float v[8];
#pragma unroll
        for (int q = 0; q < 7; q++) v[q] = lst(q < rem ? i + q : i);
#pragma unroll
        for (int q = 0; q < 7; q++) {
            if (q < rem) {
                s = __fadd_rn(s, v[q]);
                if (LOCATE && !w.found && target < s) { w.found = 1; w.at = i + q; }
            }
        }
    }
    w.s = s;
}

template <class V>
__device__ __forceinline__ void p1_sim(V lst, int i0, int i1, bool locate, float target, Walker &w) {
    w.nsim++; w.nel += i1 - i0;
    if (locate) p1_sim_t<true>(lst, i0, i1, target, w);
    else p1_sim_t<false>(lst, i0, i1, target, w);
}

// this thread's estimate of the sum of its own L entries
template <class V>
__device__ __forceinline__ float p1_csum(V lst, int n, int L, int tid) {
    const int i0 = min(n, tid * L), i1 = min(n, (tid + 1) * L);
    // only an estimate is needed here: four partial sums shorten the dependency chain
    float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;
    int i = i0;
    for (; i + 4 <= i1; i += 4) {
        c0 = __fadd_rn(c0, lst(i)); c1 = __fadd_rn(c1, lst(i + 1)); c2 = __fadd_rn(c2, lst(i + 2)); c3 = __fadd_rn(c3, lst(i + 3));
    }
    for (; i < i1; i++) c0 = __fadd_rn(c0, lst(i));
    return __fadd_rn(__fadd_rn(c0, c1), __fadd_rn(c2, c3));
}

// The tables for the walk, given every thread's estimate `csum` and the estimated sum `sst` of
// everything before its entries.
__device__ __forceinline__ unsigned long long seg_pack(int t0, short j, unsigned char dual, bool nonempty) {
    return (unsigned long long)(unsigned int)t0 | ((unsigned long long)(unsigned short)j << 16) |
           ((unsigned long long)dual << 32) | ((unsigned long long)(nonempty ? 1u : 0u) << 40);
}

template <class CX, class V>
__device__ void p1_tables(CX &c, V lst, int n, int L, float csum, double sst) {
    auto *A = c.A;
    IN_SHARED(A);
    const float EPS = 1.0f / 4096.0f;
    const int i0 = min(n, c.tid * L), i1 = min(n, (c.tid + 1) * L);
    short ja = SUS;
    unsigned char dual = 0;
    float da = 0.0f, db = 0.0f;
    const float lo = (float)(sst * (1.0 - (double)EPS));
    const float hi = (float)((sst + (double)csum) * (1.0 + (double)EPS));
    // (a warp whose lanes disagree would run both loops below one after the other: it runs the
    // two-binade loop for all of them instead; a lane that needs one binade ignores the second sum)
    const bool usable = lo > 0.0f && i1 > i0 && fexpo(hi) <= fexpo(lo) + 1 && fexpo(lo) >= -100 && fexpo(hi) <= 100;
    const bool any_two = __any_sync(0xffffffffu, usable && fexpo(hi) == fexpo(lo) + 1);
    if (lo > 0.0f && i1 > i0) {
        const int jl = fexpo(lo), j2 = fexpo(hi);
        if (j2 <= jl + 1 && jl >= -100 && j2 <= 100) {
            bool bad = false;
            const bool two = (j2 == jl + 1);
            const float C1 = __fmul_rn(1.5f, fpow2(jl)), h1 = fpow2(jl - 24), b1 = fpow2(jl - 1);
            const float C2 = __fmul_rn(1.5f, fpow2(jl + 1)), h2 = fpow2(jl - 23);
            // the terms are multiples of the binade's unit and their sum stays below 2^24 units, so
            // these additions are exact in any order: two accumulators each
            float da1 = 0.0f, db1 = 0.0f;
            auto term = [&](int i, float &xa, float &xb) {
                const float v = lst(i);
                const float q = __fsub_rn(__fadd_rn(v, C1), C1);
                const float r = __fsub_rn(v, q);
                bad |= (fabsf(r) == h1) | (v >= b1);
                xa = __fadd_rn(xa, q);
                const float q2 = __fsub_rn(__fadd_rn(v, C2), C2);
                const float r2 = __fsub_rn(v, q2);
                bad |= two & (fabsf(r2) == h2);
                xb = __fadd_rn(xb, q2);
            };
            auto term1 = [&](int i, float &xa) {  // the guess lies inside one binade
                const float v = lst(i);
                const float q = __fsub_rn(__fadd_rn(v, C1), C1);
                const float r = __fsub_rn(v, q);
                bad |= (fabsf(r) == h1) | (v >= b1);
                xa = __fadd_rn(xa, q);
            };
            int i = i0;
            if (any_two) {
                for (; i + 2 <= i1; i += 2) { term(i, da, db); term(i + 1, da1, db1); }
                if (i < i1) term(i, da, db);
                da = __fadd_rn(da, da1); db = __fadd_rn(db, db1);
            } else {
                float da2 = 0.0f, da3 = 0.0f;
                for (; i + 4 <= i1; i += 4) { term1(i, da); term1(i + 1, da1); term1(i + 2, da2); term1(i + 3, da3); }
                for (; i < i1; i++) term1(i, da);
                da = __fadd_rn(__fadd_rn(da, da1), __fadd_rn(da2, da3));
            }
            if (!bad) { ja = (short)jl; dual = two ? 1 : 0; }
        }
    }
    if (ja == SUS) { da = 0.0f; db = 0.0f; dual = 0; }
    A->u.p1.csum[c.tid] = (i1 > i0) ? csum : 0.0f;
    A->u.p1.ja[c.tid] = ja;
    A->u.p1.dual[c.tid] = dual;
    double pa, pb, ta, tb;
    block_excl_scan2((double)da, (double)(dual ? db : da), A->wsd, pa, pb, ta, tb);
    A->u.p1.pa[c.tid] = pa;
    A->u.p1.pb[c.tid] = pb;
    if (c.tid == NT - 1) { A->u.p1.pa[NT] = ta; A->u.p1.pb[NT] = tb; }
    __syncthreads();
    // Segment list: chunks where (binade guess, dual, replay) changes. A chunk of zeros adds
    // nothing in any binade: it joins the segment before it whatever its own guess was, so a
    // sparse row has few segments. `prev` is the last chunk before this one that is not empty.
    const bool nonempty = (i1 > i0) && csum != 0.0f;
    int prev = -1;
    {
        const unsigned int ne = __ballot_sync(0xffffffffu, nonempty);
        if (c.lane == 0) A->wsi[c.warp] = ne ? (c.warp * 32 + 31 - __clz((int)ne)) : -1;  // (block_excl_scan2 is done with wsd, not wsi)
        __syncthreads();
        const unsigned int below = ne & ((1u << c.lane) - 1u);
        if (below) prev = c.warp * 32 + 31 - __clz((int)below);
        else
            for (int w = c.warp - 1; w >= 0 && prev < 0; w--) prev = A->wsi[w];
        __syncthreads();
    }
    bool start = (c.tid == 0);
    if (nonempty && !start) {
        start = ja == SUS || prev < 0;
        if (!start) {
            const short pj = A->u.p1.ja[prev];
            start = pj == SUS || pj != ja || A->u.p1.dual[prev] != dual;
        }
    }
    const unsigned int bal = __ballot_sync(0xffffffffu, start);
    int wtot;
    int wex = block_excl_scan<int>(c.lane == 0 ? __popc(bal) : 0, A->wsi, &wtot);
    wex = __shfl_sync(0xffffffffu, wex, 0);
    // a segment's first chunk, its binade guess and flags in one word, so that the walk needs one
    // load per segment (and can fetch the next one ahead); the list ends with a word for chunk NT
    if (start) A->u.p1.segd[wex + __popc(bal & ((1u << c.lane) - 1u))] = seg_pack(c.tid, ja, dual, nonempty);
    if (c.tid == 0) { A->nseg = wtot; A->u.p1.segd[wtot] = seg_pack(NT, SUS, 0, false); }
    __syncthreads();
}

template <class CX, class V>
__device__ void p1_build(CX &c, V lst, int n, int L, double sbase) {
    auto *A = c.A;
    IN_SHARED(A);
    const float csum = p1_csum(lst, n, L, c.tid);
    double tot;
    const double sst = sbase + block_excl_scan<double>((double)csum, A->wsd, &tot);
    p1_tables(c, lst, n, L, csum, sst);
}

__device__ __forceinline__ double dpow2(int j) {  // 2^j as a double, -1022 <= j <= 1023
    return __longlong_as_double((long long)(j + 1023) << 52);
}

// thread 0 only; continues from the state in `w`
template <class CX, class V>
__device__ void p1_walk(CX &c, V lst, int n, int L, bool locate, float target, Walker &w) {
    auto *A = c.A;
    IN_SHARED(A);
    const int nseg = A->nseg;
    const double *PA = A->u.p1.pa, *PB = A->u.p1.pb;
    // One thread runs this and waits for every load it needs: the words and table entries of the
    // next segment are fetched while this one is worked on.
    unsigned long long nd = A->u.p1.segd[0], ndn = A->u.p1.segd[nseg > 0 ? 1 : 0];
    double npa0 = PA[(int)(nd & 0xffffu)], npb0 = PB[(int)(nd & 0xffffu)];
    double npa1 = PA[(int)(ndn & 0xffffu)], npb1 = PB[(int)(ndn & 0xffffu)];
    for (int si = 0; si < nseg && !(locate && w.found); si++) {
        const unsigned long long d = nd, dn = ndn;
        const double pa0 = npa0, pa1 = npa1, pb0 = npb0, pb1 = npb1;
        {
            const unsigned long long dnn = A->u.p1.segd[min(si + 2, nseg)];  // (the list has an end word)
            nd = ndn; ndn = dnn;
            npa0 = npa1; npb0 = npb1;
            npa1 = PA[(int)(dnn & 0xffffu)]; npb1 = PB[(int)(dnn & 0xffffu)];
        }
        const int t0 = (int)(d & 0xffffu), t1 = (int)(dn & 0xffffu);
        const int j = (int)(short)(unsigned short)(d >> 16);
        const int e0 = min(n, t0 * L), e1 = min(n, t1 * L);
        if (e1 <= e0) break;  // chunks past the end of the list are empty
        if (j == SUS) {
            // (the chunks behind t0 in this segment hold zeros only)
            if ((d >> 40) & 1u) p1_sim(lst, e0, min(e1, min(n, (t0 + 1) * L)), locate, target, w);
            continue;
        }
        const bool dual = ((d >> 32) & 0xffu) != 0;
        if (pa1 == pa0 && pb1 == pb0) continue;  // every term rounds to nothing in either binade
        bool ok = false;
        if (w.s > 0.0f) {
            const int js = fexpo(w.s);
            const double sd = (double)w.s;
            // step over chunks [ta, tb) with table P, valid while the sum stays below lim
            auto bulk = [&](const double *P, int ta, int tb, double lim, bool whole = false, double diff = 0.0) -> bool {
                double sn = (double)w.s + (whole ? diff : (P[tb] - P[ta]));
                if (!(sn < lim)) return false;
                if (locate && target < (float)sn) {
                    int lo_ = ta, hi_ = tb - 1;  // first chunk whose end value exceeds the target
                    while (lo_ < hi_) {
                        int mid = (lo_ + hi_) >> 1;
                        if (target < (float)((double)w.s + (P[mid + 1] - P[ta]))) hi_ = mid;
                        else lo_ = mid + 1;
                    }
                    w.s = (float)((double)w.s + (P[lo_] - P[ta]));
                    p1_sim(lst, min(n, lo_ * L), min(n, (lo_ + 1) * L), true, target, w);
                    return true;
                }
                w.s = (float)sn;
                return true;
            };
            if (!dual) {
                if (js == j) ok = bulk(PA, t0, t1, dpow2(j + 1), true, pa1 - pa0);
            } else if (js == j + 1) {
                ok = bulk(PB, t0, t1, dpow2(j + 2), true, pb1 - pb0);
            } else if (js == j) {
                const double lim = dpow2(j + 1);
                if (sd + (pa1 - pa0) < lim) {
                    ok = bulk(PA, t0, t1, lim, true, pa1 - pa0);
                } else {
                    // the running sum leaves binade j inside this segment: find the chunk
                    int lo_ = t0, hi_ = t1 - 1;
                    while (lo_ < hi_) {
                        int mid = (lo_ + hi_) >> 1;
                        if (sd + (PA[mid + 1] - pa0) >= lim) hi_ = mid;
                        else lo_ = mid + 1;
                    }
                    const int ts = lo_;
                    bool fine = true;
                    if (ts > t0) fine = bulk(PA, t0, ts, lim);
                    if (fine) {
                        ok = true;
                        if (!(locate && w.found)) {
                            p1_sim(lst, min(n, ts * L), min(n, (ts + 1) * L), locate, target, w);
                            if (!(locate && w.found) && ts + 1 < t1) {
                                if (!(fexpo(w.s) == j + 1 && bulk(PB, ts + 1, t1, dpow2(j + 2)))) {
                                    w.slow = 1;
                                    p1_sim(lst, min(n, (ts + 1) * L), e1, locate, target, w);
                                }
                            }
                        }
                    }
                }
            }
        }
        if (!ok) {
            w.slow = 1;
            p1_sim(lst, e0, e1, locate, target, w);
        }
    }
}

// =============================================================================
// Histogram search: thread t owns bins NBINS-1-BPT*t-i (i < BPT), so a scan over the
// threads runs through the bins in descending order.
// =============================================================================
// A bin's integer mass is kept as two sums, of the low MASS_SPLIT bits of each contribution and of
// the rest: contributions are below 2^27 (32 elements of less than 2^22 units each) and a bin holds
// fewer than 2^20 elements, so neither sum can wrap, and the additions need no return value.
constexpr int MASS_SPLIT = 11;
constexpr unsigned int MASS_LO_MASK = (1u << MASS_SPLIT) - 1u;
struct BinQuery {
    unsigned long long m0, xq;       // mass event: m0 + cum_q >= xq   (xq = ~0 disables)
    unsigned long long pos0, nstop;  // count event: pos0 + cum_c >= nstop (nstop = ~0 disables)
    int specbin;                     // stop at this bin (-1 disables)
    int bin_hi;                      // only bins below this one count (NBINS = all)
    const unsigned int *spec_bits;   // or: stop at any bin whose bit is set here (nullptr = use specbin)
    const unsigned int *hq, *hqh, *hc;  // per bin: integer mass (low MASS_SPLIT bits summed, the rest summed) and count
};

// `bin_load(b, q, n)` gives bin b's integer mass and count (one thread block's tables, or the
// sum over the tables of a cluster's thread blocks).
struct NoAdjust {};
// `adjust(q, eq)` may change the masses of the thread's bins once their sum before the bins (eq)
// is known; it returns whether it did (the same answer in every thread).
template <class CX, class LD, class ADJ>
__device__ void find_event_bin_adj(CX &c, const BinQuery &qy, LD bin_load, ADJ adjust) {
    auto *A = c.A;
    IN_SHARED(A);
    unsigned long long q[BPT], n[BPT], sq = 0, sn = 0;
#pragma unroll
    for (int i = 0; i < BPT; i++) {
        const int b = NBINS - 1 - BPT * c.tid - i;
        const bool live = b < qy.bin_hi;
        q[i] = 0ull; n[i] = 0ull;
        if (live) bin_load(b, q[i], n[i]);
        sq += q[i]; sn += n[i];
    }
    unsigned long long tq, tc;
    unsigned long long eq = block_excl_scan<unsigned long long>(sq, A->wsu, &tq);
    if constexpr (!std::is_same<ADJ, NoAdjust>::value) if (adjust(q, eq)) {
        sq = 0;
#pragma unroll
        for (int i = 0; i < BPT; i++) sq += q[i];
        eq = block_excl_scan<unsigned long long>(sq, A->wsu, &tq);
    }
    const unsigned long long ec = block_excl_scan<unsigned long long>(sn, A->wsu, &tc);
    __syncthreads();
    if (c.tid == 0) { A->evt_thread = 0x7fffffff; A->tot_q = tq; A->tot_c = tc; A->hit_bin = -1; }
    __syncthreads();
    int hit = -1;
    unsigned long long cq = eq, cc = ec, hq_before = 0, hc_before = 0;
#pragma unroll
    for (int i = 0; i < BPT; i++) {
        const int b = NBINS - 1 - BPT * c.tid - i;
        const unsigned long long q1 = cq + q[i], c1 = cc + n[i];
        const bool pr = (qy.xq != ~0ull && qy.m0 + q1 >= qy.xq) || (qy.nstop != ~0ull && qy.pos0 + c1 >= qy.nstop) ||
                        (qy.spec_bits ? (b < qy.bin_hi && ((qy.spec_bits[b >> 5] >> (b & 31)) & 1u)) : (b <= qy.specbin));
        if (pr && hit < 0) { hit = b; hq_before = cq; hc_before = cc; }
        cq = q1; cc = c1;
    }
    if (hit >= 0) atomicMin(&A->evt_thread, c.tid);
    __syncthreads();
    if (A->evt_thread == c.tid) { A->hit_bin = hit; A->hit_qbefore = hq_before; A->hit_cbefore = hc_before; }
    __syncthreads();
}

template <class CX, class LD>
__device__ void find_event_bin_with(CX &c, const BinQuery &qy, LD bin_load) {
    find_event_bin_adj(c, qy, bin_load, NoAdjust{});
}

template <class CX>
__device__ void find_event_bin(CX &c, const BinQuery &qy) {
    find_event_bin_with(c, qy, [&](int b, unsigned long long &q, unsigned long long &n) {
        q = (unsigned long long)qy.hq[b] + ((unsigned long long)qy.hqh[b] << MASS_SPLIT);
        n = qy.hc[b];
    });
}

// Sort the candidate list (descending probability, ascending token id).
template <class CX>
__device__ void sort_cands(CX &c, int n) {
    auto *A = c.A;
    IN_SHARED(A);
    __syncthreads();
    if (n <= NT) {
        // few keys: every key counts the keys above it (they are all different: the token id is part
        // of the key) and goes to that place; no sorting network, two barriers
        const unsigned long long mine = (c.tid < n) ? A->cand[c.tid] : 0ull;
        int rank = 0;
        if (c.tid < n) {
            int j = 0;
            for (; j + 4 <= n; j += 4) {
                const unsigned long long k0 = A->cand[j], k1 = A->cand[j + 1], k2 = A->cand[j + 2], k3 = A->cand[j + 3];
                rank += (k0 > mine ? 1 : 0) + (k1 > mine ? 1 : 0) + (k2 > mine ? 1 : 0) + (k3 > mine ? 1 : 0);
            }
            for (; j < n; j++) rank += A->cand[j] > mine ? 1 : 0;
        }
        __syncthreads();
        if (c.tid < n) A->cand[rank] = mine;
        __syncthreads();
    } else {
        int n2 = 2;
        while (n2 < n) n2 <<= 1;
        for (int i = n + c.tid; i < n2; i += NT) A->cand[i] = 0ull;
        bitonic_desc(A->cand, n2, c.tid);
    }
    for (int i = c.tid; i < n; i += NT) A->pc[i] = key_val(A->cand[i]);
    __syncthreads();
}

// Adds the sorted candidates pc[0..nb) to the running sum `s0` in order, exactly as the
// reference's loops do (sample.mojo:497-506, 585-590), and stops at the first event: the sum
// reaching x_ge, exceeding x_gt, or the count reaching nstop. Where the sum stays in one
// binade the additions are integers and the first event is found with a block scan; a
// candidate that takes the sum across a power of two is added by itself and the scan resumes
// behind it; a rounding tie or a candidate >= sum/4 sends the rest to one thread.
// Results: A->b_event, b_s, b_pos, and for an event b_idx (token), b_p, b_aux (tie).
template <class CX>
__device__ void walk_sorted(CX &c, int nb, float s0, long long pos0, float x_ge, float x_gt, bool counting,
                            long long nstop) {
    auto *A = c.A;
    IN_SHARED(A);
    constexpr int EPT = NC / NT;
    __syncthreads();
    if (c.tid == 0) { A->b_s = s0; A->b_event = EV_NONE; A->b_aux = -1; A->b_idx = 0; }
    __syncthreads();
    for (int round = 0; round < 256; round++) {
        const int st = A->b_idx;      // candidates before st are consumed
        const float s = A->b_s;
        if (A->b_event != EV_NONE || st >= nb) break;
        const bool have_s = s > 0.0f;
        const int j = have_s ? fexpo(s) : 0;
        const bool ok = have_s && j >= -100 && j <= 100;
        const float Cm = __fmul_rn(1.5f, fpow2(j)), halfu = fpow2(j - 24), bigthr = fpow2(j - 1), inv_u = fpow2(23 - j);
        unsigned int q[EPT];
        bool special = !ok;
#pragma unroll
        for (int e = 0; e < EPT; e++) {
            const int i = st + c.tid * EPT + e;
            q[e] = 0u;
            if (i < nb && ok) {
                const float p = A->pc[i];
                const float qf = __fsub_rn(__fadd_rn(p, Cm), Cm);
                const float r = __fsub_rn(p, qf);
                if (fabsf(r) == halfu || p >= bigthr) special = true;
                q[e] = __float2uint_rn(__fmul_rn(qf, inv_u));
            }
        }
        if (__syncthreads_or(special ? 1 : 0)) {
            // one thread, one addition at a time, from st to the first event or the end
            if (c.tid == 0) {
                float acc = s;
                long long pos = pos0 + st;
                int ev = EV_NONE, at = -1;
                for (int i = st; i < nb; i++) {
                    acc = __fadd_rn(acc, A->pc[i]);
                    pos++;
                    if (acc >= x_ge) ev = EV_CUT;
                    else if (x_gt < acc) ev = EV_DRAW;
                    else if (counting && pos >= nstop) ev = EV_LIMIT;
                    if (ev != EV_NONE) { at = i; break; }
                }
                A->b_s = acc; A->b_event = ev; A->b_aux = at; A->b_idx = nb;
            }
            __syncthreads();
            break;
        }
        unsigned long long loc = 0;
#pragma unroll
        for (int e = 0; e < EPT; e++) loc += q[e];
        unsigned long long tot;
        const unsigned long long ex = block_excl_scan<unsigned long long>(loc, A->wsu, &tot);
        const unsigned long long m0 = (unsigned long long)((double)s * (double)inv_u);
        unsigned long long X = 1ull << 24;
        if (x_ge < 3.0e38f) { double t = ceil((double)x_ge * (double)inv_u); if (t < (double)X) X = t <= 0.0 ? 0ull : (unsigned long long)t; }
        if (x_gt < 3.0e38f) { double t = floor((double)x_gt * (double)inv_u) + 1.0; if (t < (double)X) X = t <= 0.0 ? 0ull : (unsigned long long)t; }
        __syncthreads();
        if (c.tid == 0) A->evt_thread = 0x7fffffff;
        __syncthreads();
        unsigned long long m = m0 + ex, mb_first = 0;
        int first = -1;
#pragma unroll
        for (int e = 0; e < EPT; e++) {
            const int i = st + c.tid * EPT + e;
            const unsigned long long mb = m;
            m += q[e];
            if (i < nb && first < 0 && (m >= X || (counting && pos0 + i + 1 >= nstop))) { first = i; mb_first = mb; }
        }
        if (first >= 0) atomicMin(&A->evt_thread, first);
        __syncthreads();
        const int hit = A->evt_thread;
        if (hit == 0x7fffffff) {
            if (c.tid == 0) { A->b_s = (float)((double)(m0 + tot) * (double)fpow2(j - 23)); A->b_idx = nb; }
            __syncthreads();
            break;
        }
        if (first == hit) {
            // the true addition at the candidate the integers point at decides what happened there
            const float sb = (float)((double)mb_first * (double)fpow2(j - 23));
            const float acc = __fadd_rn(sb, A->pc[hit]);
            int ev = EV_NONE;
            if (acc >= x_ge) ev = EV_CUT;
            else if (x_gt < acc) ev = EV_DRAW;
            else if (counting && pos0 + hit + 1 >= nstop) ev = EV_LIMIT;
            A->b_s = acc; A->b_event = ev; A->b_aux = (ev != EV_NONE) ? hit : -1; A->b_idx = hit + 1;
        }
        __syncthreads();
    }
    if (c.tid == 0) {
        const int at = A->b_aux;
        const int consumed = (A->b_event != EV_NONE) ? at + 1 : nb;
        A->b_pos = pos0 + consumed;
        if (A->b_event != EV_NONE) {
            const float p = A->pc[at];
            A->b_idx = key_idx(A->cand[at]); A->b_p = p;
            A->b_aux = ((at > 0 && A->pc[at - 1] == p) || (at + 1 < nb && A->pc[at + 1] == p)) ? 1 : 0;
        }
    }
    __syncthreads();
}

// =============================================================================
// Typical-p (sample.mojo:525-567) on a kept set that lies inside the sorted head: m
// probabilities pc[0..m), descending, ids in hidx. Entropy H = -sum p log p, added up
// in that order in fp32; distance |-log p - H|; stable order by distance; the smallest
// prefix whose probabilities add up to typ; then the draw of sample.mojo:569-594 over
// that prefix in that order. The sums run on one thread (m is at most the head's 1024).
// Results: A->b_idx (token), b_p, b_sum, b_target, b_aux (tie bits).
// =============================================================================
template <class CX>
__device__ void typical_head(CX &c, int m, float typ, float u01) {
    auto *A = c.A;
    IN_SHARED(A);
    float *lg = reinterpret_cast<float *>(A->cand);             // log p
    float *tt = lg + HEADC;                                     // p * log p
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(&A->u);  // HEADC sort keys
    __syncthreads();
    for (int i = c.tid; i < m; i += NT) {
        const float p = A->pc[i];
        const float l = (p > 0.0f) ? logf_pinned(p) : 0.0f;
        lg[i] = l;
        tt[i] = __fmul_rn(p, l);
    }
    __syncthreads();
    if (c.tid == 0) {
        float ent = 0.0f;
        for (int i = 0; i < m; i++)
            if (A->pc[i] > 0.0f) ent = __fsub_rn(ent, tt[i]);
        A->b_s = ent;
    }
    __syncthreads();
    const float ent = A->b_s;
    int n2 = 2;
    while (n2 < m) n2 <<= 1;
    for (int i = c.tid; i < n2; i += NT) {
        unsigned long long key = 0ull;
        if (i < m) {
            const float sur = (A->pc[i] > 0.0f) ? -lg[i] : 0.0f;
            const float d = fabsf(__fsub_rn(sur, ent));
            // descending keys = ascending distance, and among equal distances ascending position (stable)
            key = ((unsigned long long)(~__float_as_uint(d)) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)i);
        }
        keys[i] = key;
    }
    bitonic_desc(keys, n2, c.tid);
    if (c.tid == 0) {
        float s = 0.0f;
        int kept = m;
        for (int j = 0; j < m; j++) {
            const int i = (int)(0xFFFFFFFFu - (unsigned int)(keys[j] & 0xFFFFFFFFull));
            s = __fadd_rn(s, A->pc[i]);
            A->pre[j] = s;
            if (s >= typ) { kept = j + 1; break; }
        }
        const float sum = A->pre[kept - 1];
        int at = kept - 1;
        float target = 0.0f;
        if (sum <= 0.0f) at = 0;  // sample.mojo:583-584
        else {
            target = __fmul_rn(u01, sum);
            for (int j = 0; j < kept; j++)
                if (target < A->pre[j]) { at = j; break; }
        }
        const int i_at = (int)(0xFFFFFFFFu - (unsigned int)(keys[at] & 0xFFFFFFFFull));
        int tie = 0;
        if (A->hidx[i_at] & 0x80000000u) tie |= MOLLA_ROW_CHOSEN_TIE;
        // the last one kept and the first one dropped equally probable: which of them the
        // reference keeps depends on the order its sort left them in
        if (kept < m) {
            const int i_last = (int)(0xFFFFFFFFu - (unsigned int)(keys[kept - 1] & 0xFFFFFFFFull));
            const int i_next = (int)(0xFFFFFFFFu - (unsigned int)(keys[kept] & 0xFFFFFFFFull));
            if (A->pc[i_last] == A->pc[i_next]) tie |= MOLLA_ROW_TOPP_TIE;
        }
        A->b_idx = (int)(A->hidx[i_at] & 0x7fffffffu); A->b_p = A->pc[i_at];
        A->b_sum = sum; A->b_target = target; A->b_aux = tie;
    }
    __syncthreads();
}

}  // namespace
