// The token-sampling kernel and its C ABI (declared in include/molla_sample.h).
//
// One thread-block cluster owns one logit row at a time: the row is fetched from
// HBM exactly once (bulk asynchronous copies into shared memory, one slice per
// CTA of the cluster) and every later pass - penalties, maximum, exponentials,
// the softmax denominator, candidate selection, the top-p cut and the draw -
// reads it from shared / distributed shared memory.
//
// The reference (src/molla/engine/sample.mojo) defines its result through
// *sequential* fp32 sums: the softmax denominator is accumulated in vocabulary
// order (:431-434), the top-p prefix and the draw walk in sorted order
// (:497-506, :580-590). A parallel reduction rounds differently, and a different
// last bit moves the top-p cut and the drawn token. So the kernel reproduces
// those sums bit for bit instead of approximating them:
//   * a running fp32 sum of non-negative terms stays inside one binade
//     [2^j, 2^(j+1)) for long stretches; there `s + a` rounds to a multiple of
//     ulp = 2^(j-23), so every term contributes the integer rne(a/ulp) and the
//     contributions add exactly, in any order (`p1_*` below);
//   * the few places where that fails - the running sum crossing into the next
//     binade, a term that is large against the sum, a rounding tie whose
//     direction depends on the parity of the sum - are found in parallel and
//     replayed sequentially by one thread.
// What cannot be reproduced is the order the reference's unstable heapsort
// (:440-483) leaves equal probabilities in; rows where that order could matter
// are marked in the row status (MOLLA_ROW_*_TIE) and equal probabilities are
// ordered by token id.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/molla_sample.h"
#include "molla_device.cuh"

namespace cg = cooperative_groups;
using namespace molla;

namespace {

constexpr int NBINS = 2048;      // histogram bins over the top bits of exp(v - max) in [0, 1]
constexpr int BIN_SHIFT = 19;    // sign + 8 exponent + 4 mantissa bits
constexpr int NC = 2048;         // candidate-list capacity (head list, gathered bins)
constexpr int HEAD_MAX = 1025;   // the sorted head covers top-k + 1 up to this many
constexpr int HIST_STAGE = 4096; // history ids staged in shared memory
constexpr short SUS = -32768;    // chunk that must be replayed sequentially
constexpr int TOPN_MAX = 20;

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
    int S;             // slice capacity in floats (multiple of 4)
    int L;             // chunk length per thread (odd), L*NT >= S
    int *row_counter;  // workspace: next row to hand out
    long long *prof;   // optional [B x 16] clock64 stamps per row (testing aid)
};

struct Bcast {       // decisions published by CTA 0 to every CTA of the cluster
    float s; unsigned int tau; int event; int idx; float p; long long pos; int aux;
};

struct __align__(16) Aux {
    union {
        struct {
            double pa[NT + 1];
            double pb[NT + 1];
            float csum[NT];
            short ja[NT];
            unsigned char dual[NT];
            unsigned short seg[NT];
        } p1;
        struct {
            unsigned long long hq[NBINS];
            unsigned int hc[NBINS];
        } h;
        int hist_tok[HIST_STAGE];
    } u;
    float cmax[NT];
    unsigned long long cand[NC];
    float pc[NC];
    float pre[NC];
    unsigned int hidx[NC];          // head: token id, bit 31 = equal to a neighbour
    unsigned long long xs[2][16];   // cluster exchange slots, two banks used alternately
    unsigned long long stage;
    double wsd[NWARP + 1];
    unsigned long long wsu[NWARP + 1];
    float wsf[NWARP + 1];
    int wsi[NWARP + 1];
    uint64_t mbar;
    int nseg;
    int ncand;
    int evt_thread;
    int specbin;
    int hit_bin; unsigned long long hit_qbefore; unsigned long long hit_cbefore;
    unsigned long long tot_q; unsigned long long tot_c;
    Bcast bc;
};

#define STAMP(i) do { if (a.prof && c.rank == 0 && c.tid == 0) a.prof[(long long)r * 16 + (i)] = clock64(); } while (0)

enum { EV_NONE = 0, EV_CUT = 1, EV_DRAW = 2, EV_LIMIT = 3, EV_EXHAUSTED = 4, EV_DEGENERATE = 5 };

struct Ctx {
    cg::cluster_group cluster;
    int cs, rank, tid, lane, warp;
    float *row;
    Aux *A;
    int S, L, V, base, nloc;
    int c0, c1;  // this thread's chunk of local indices
    int xph;     // exchange counter (selects the slot bank)
};

// ---- cluster-wide exchange: every CTA publishes one 64-bit value (valid in its
// thread 0), all CTAs read all. Two slot banks alternate so that a fast CTA's
// next exchange cannot overwrite a value a slow CTA has not read yet.
__device__ __forceinline__ const unsigned long long *xchg(Ctx &c, unsigned long long v) {
    Aux *A = c.A;
    const int bank = c.xph & 1;
    c.xph++;
    if (c.tid == 0) A->stage = v;
    __syncthreads();
    if (c.tid < c.cs) {
        Aux *RA = c.cluster.map_shared_rank(A, c.tid);
        RA->xs[bank][c.rank] = A->stage;
    }
    c.cluster.sync();
    return A->xs[bank];
}
__device__ __forceinline__ unsigned long long pack_fi(float f, int i) {
    return ((unsigned long long)__float_as_uint(f) << 32) | (unsigned long long)(unsigned int)i;
}

__device__ __forceinline__ float block_max(Ctx &c, float v) {
    v = warp_max(v);
    __syncthreads();
    if (c.lane == 0) c.A->wsf[c.warp] = v;
    __syncthreads();
    float r = c.A->wsf[0];
#pragma unroll
    for (int w = 1; w < NWARP; w++) r = fmaxf(r, c.A->wsf[w]);
    return r;
}

__device__ __forceinline__ void block_argmax(Ctx &c, float &v, int &i) {
    warp_argmax(v, i);
    __syncthreads();
    if (c.lane == 0) { c.A->wsf[c.warp] = v; c.A->wsi[c.warp] = i; }
    __syncthreads();
    float bv = c.A->wsf[0];
    int bi = c.A->wsi[0];
    for (int w = 1; w < NWARP; w++) {
        float ov = c.A->wsf[w];
        int oi = c.A->wsi[w];
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    v = bv; i = bi;
}

// ---- bitonic sort, descending, of n2 (power of two) keys in shared memory -----
__device__ void bitonic_desc(unsigned long long *k, int n2, int tid) {
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = tid; i < (n2 >> 1); i += NT) {
                int pos = ((i / stride) * stride * 2) + (i % stride);
                int par = pos + stride;
                bool desc = ((pos & size) == 0);
                unsigned long long a = k[pos], b = k[par];
                if ((a < b) == desc) { k[pos] = b; k[par] = a; }
            }
        }
    }
    __syncthreads();
}

// =============================================================================
// P1: the exact sequential fp32 sum of row[0..V) in vocabulary order.
// =============================================================================
// Build: every thread owns a contiguous chunk. From approximate prefix sums each
// chunk guesses the binade(s) the true running sum can be in when it reaches the
// chunk (a margin of 2^-12 covers the rounding drift of the true sum) and adds up
// its terms' integer contributions for that binade (`pa`) and, when the guess
// straddles a power of two, for the next one (`pb`). Chunks holding a rounding
// tie, a term >= sum/4, or a span of more than two binades are left to the
// sequential replay. `csum` (per-thread fp32 chunk sum) is an input.
__device__ void p1_build(Ctx &c, float csum) {
    Aux *A = c.A;
    const float EPS = 1.0f / 4096.0f;
    double tot;
    double ex = block_excl_scan<double>((double)csum, A->wsd, &tot);
    const unsigned long long *xs = xchg(c, (unsigned long long)__double_as_longlong(tot));
    double basesum = 0.0;
    for (int r = 0; r < c.rank; r++) basesum += __longlong_as_double((long long)xs[r]);
    double sst = basesum + ex;
    short ja = SUS;
    unsigned char dual = 0;
    float da = 0.0f, db = 0.0f;
    float lo = (float)(sst * (1.0 - (double)EPS));
    float hi = (float)((sst + (double)csum) * (1.0 + (double)EPS));
    if (lo > 0.0f && c.c1 > c.c0) {
        int jl = fexpo(lo), j2 = fexpo(hi);
        if (j2 <= jl + 1 && jl >= -100 && j2 <= 100) {
            bool bad = false;
            const bool two = (j2 == jl + 1);
            const float C1 = __fmul_rn(1.5f, fpow2(jl)), h1 = fpow2(jl - 24), b1 = fpow2(jl - 1);
            const float C2 = __fmul_rn(1.5f, fpow2(jl + 1)), h2 = fpow2(jl - 23);
            for (int i = c.c0; i < c.c1; i++) {
                float e = c.row[i];
                float q = __fsub_rn(__fadd_rn(e, C1), C1);
                float r = __fsub_rn(e, q);
                bad |= (fabsf(r) == h1) | (e >= b1);
                da = __fadd_rn(da, q);
                if (two) {
                    float q2 = __fsub_rn(__fadd_rn(e, C2), C2);
                    float r2 = __fsub_rn(e, q2);
                    bad |= (fabsf(r2) == h2);
                    db = __fadd_rn(db, q2);
                }
            }
            if (!bad) { ja = (short)jl; dual = two ? 1 : 0; }
        }
    }
    if (c.c1 <= c.c0) { ja = SUS; }  // empty chunk: replay does nothing
    if (ja == SUS) { da = 0.0f; db = 0.0f; dual = 0; }
    A->u.p1.csum[c.tid] = (c.c1 > c.c0) ? csum : 0.0f;
    A->u.p1.ja[c.tid] = ja;
    A->u.p1.dual[c.tid] = dual;
    double t2;
    double pa = block_excl_scan<double>((double)da, A->wsd, &t2);
    A->u.p1.pa[c.tid] = pa;
    if (c.tid == NT - 1) A->u.p1.pa[NT] = t2;
    double pb = block_excl_scan<double>((double)(dual ? db : da), A->wsd, &t2);
    A->u.p1.pb[c.tid] = pb;
    if (c.tid == NT - 1) A->u.p1.pb[NT] = t2;
    __syncthreads();
    // segment list: chunks where (binade guess, dual, replay) changes
    bool start = (c.tid == 0) || ja == SUS || A->u.p1.ja[c.tid - 1] != ja ||
                 A->u.p1.dual[c.tid - 1] != dual;
    unsigned int bal = __ballot_sync(0xffffffffu, start);
    int wcount = __popc(bal);
    int wtot;
    int wex = block_excl_scan<int>(c.lane == 0 ? wcount : 0, A->wsi, &wtot);
    wex = __shfl_sync(0xffffffffu, wex, 0);
    if (start) {
        int pos = wex + __popc(bal & ((1u << c.lane) - 1u));
        A->u.p1.seg[pos] = (unsigned short)c.tid;
    }
    if (c.tid == 0) A->nseg = wtot;
    c.cluster.sync();
}

// Walk (one thread): replays the sum across the whole cluster from the tables
// p1_build left in every CTA's shared memory. With `locate`, stops at the first
// index i whose running sum exceeds `target` (strictly) and returns it.
struct P1Walk {
    float s;
    int found;      // locate mode: index found
    long long idx;  // global vocabulary index
    int slow;       // a fallback replay ran
};

__device__ __forceinline__ void p1_sim(const float *rrow, int i0, int i1, long long gbase,
                                       bool locate, float target, P1Walk &w) {
    float s = w.s;
    int i = i0;
    while (i < i1) {
        float buf[8];
        int n = min(8, i1 - i);
#pragma unroll
        for (int k = 0; k < 8; k++) buf[k] = (k < n) ? rrow[i + k] : 0.0f;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (k < n) {
                s = __fadd_rn(s, buf[k]);
                if (locate && !w.found && target < s) { w.found = 1; w.idx = gbase + i + k; }
            }
        }
        if (locate && w.found) break;
        i += n;
    }
    w.s = s;
}

__device__ void p1_walk(Ctx &c, bool locate, float target, P1Walk &w) {
    w.s = 0.0f; w.found = 0; w.idx = -1; w.slow = 0;
    const int L = c.L;
    for (int r = 0; r < c.cs && !(locate && w.found); r++) {
        Aux *RA = c.cluster.map_shared_rank(c.A, r);
        const float *rrow = c.cluster.map_shared_rank(c.row, r);
        const long long gbase = (long long)r * c.S;
        long long nl = (long long)c.V - gbase;
        const int nloc = (int)(nl < 0 ? 0 : (nl > c.S ? c.S : nl));
        const int nseg = RA->nseg;
        const double *PA = RA->u.p1.pa, *PB = RA->u.p1.pb;
        for (int si = 0; si < nseg && !(locate && w.found); si++) {
            const int t0 = RA->u.p1.seg[si];
            const int t1 = (si + 1 < nseg) ? (int)RA->u.p1.seg[si + 1] : NT;
            const int j = RA->u.p1.ja[t0];
            const int e0 = min(nloc, t0 * L), e1 = min(nloc, t1 * L);
            if (e1 <= e0) continue;
            if (j == SUS) {
                if (RA->u.p1.csum[t0] != 0.0f) p1_sim(rrow, e0, e1, gbase, locate, target, w);
                continue;
            }
            const bool dual = RA->u.p1.dual[t0] != 0;
            const double pa0 = PA[t0], pa1 = PA[t1], pb0 = PB[t0], pb1 = PB[t1];
            if (pa1 == pa0 && pb1 == pb0) continue;  // all terms round to nothing in either binade
            bool ok = false;
            if (w.s > 0.0f) {
                const int js = fexpo(w.s);
                const double sd = (double)w.s;
                // bulk step over chunks [ta, tb) using table P, valid while the sum stays below lim
                auto bulk = [&](const double *P, int ta, int tb, double lim) -> bool {
                    double sn = (double)w.s + (P[tb] - P[ta]);
                    if (!(sn < lim)) return false;
                    if (locate && target < (float)sn) {
                        // first chunk t in [ta, tb) whose end value exceeds the target
                        int lo_ = ta, hi_ = tb - 1;
                        while (lo_ < hi_) {
                            int mid = (lo_ + hi_) >> 1;
                            if (target < (float)((double)w.s + (P[mid + 1] - P[ta]))) hi_ = mid;
                            else lo_ = mid + 1;
                        }
                        w.s = (float)((double)w.s + (P[lo_] - P[ta]));
                        p1_sim(rrow, min(nloc, lo_ * L), min(nloc, (lo_ + 1) * L), gbase, true, target, w);
                        return true;
                    }
                    w.s = (float)sn;
                    return true;
                };
                if (!dual) {
                    if (js == j) ok = bulk(PA, t0, t1, ldexp(1.0, j + 1));
                } else if (js == j + 1) {
                    ok = bulk(PB, t0, t1, ldexp(1.0, j + 2));
                } else if (js == j) {
                    const double lim = ldexp(1.0, j + 1);
                    if (sd + (pa1 - pa0) < lim) {
                        ok = bulk(PA, t0, t1, lim);
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
                        if (fine && !(locate && w.found)) {
                            p1_sim(rrow, min(nloc, ts * L), min(nloc, (ts + 1) * L), gbase, locate, target, w);
                            if (!(locate && w.found) && ts + 1 < t1) {
                                if (fexpo(w.s) == j + 1 && bulk(PB, ts + 1, t1, ldexp(1.0, j + 2))) {
                                } else {
                                    w.slow = 1;
                                    p1_sim(rrow, min(nloc, (ts + 1) * L), e1, gbase, locate, target, w);
                                }
                            }
                            ok = true;
                        } else if (fine) {
                            ok = true;
                        } else {
                            ok = false;  // cannot happen (ts chosen so the prefix stays below lim)
                        }
                    }
                }
            }
            if (!ok) {
                w.slow = 1;
                p1_sim(rrow, e0, e1, gbase, locate, target, w);
            }
        }
    }
}

// =============================================================================
// Histogram search shared by head selection and the descending walk.
// Thread t owns bins NBINS-1-2t and NBINS-2-2t, so a scan over threads runs
// through the bins in descending order. Totals are summed over the cluster's
// CTAs; every CTA computes the same answer.
// =============================================================================
struct BinQuery {
    unsigned long long m0, xq;     // mass event: m0 + cum_q >= xq   (xq = ~0 disables)
    unsigned long long pos0, nstop;  // count event: pos0 + cum_c >= nstop (nstop = ~0 disables)
    int specbin;                   // stop at this bin (-1 disables)
};

__device__ void find_event_bin(Ctx &c, const BinQuery &qy) {
    Aux *A = c.A;
    const int bh = NBINS - 1 - 2 * c.tid, bl = bh - 1;
    unsigned long long qh = 0, ql = 0, ch = 0, cl = 0;
    for (int r = 0; r < c.cs; r++) {
        Aux *RA = c.cluster.map_shared_rank(A, r);
        qh += RA->u.h.hq[bh]; ql += RA->u.h.hq[bl];
        ch += RA->u.h.hc[bh]; cl += RA->u.h.hc[bl];
    }
    unsigned long long tq, tc;
    unsigned long long eq = block_excl_scan<unsigned long long>(qh + ql, A->wsu, &tq);
    unsigned long long ec = block_excl_scan<unsigned long long>(ch + cl, A->wsu, &tc);
    __syncthreads();
    if (c.tid == 0) { A->evt_thread = 0x7fffffff; A->tot_q = tq; A->tot_c = tc; A->hit_bin = -1; }
    __syncthreads();
    auto pred = [&](unsigned long long cq, unsigned long long cc, int bin) -> bool {
        if (qy.xq != ~0ull && qy.m0 + cq >= qy.xq) return true;
        if (qy.nstop != ~0ull && qy.pos0 + cc >= qy.nstop) return true;
        if (bin <= qy.specbin) return true;
        return false;
    };
    const bool ph = pred(eq + qh, ec + ch, bh);
    const bool pl = pred(eq + qh + ql, ec + ch + cl, bl);
    if (ph || pl) atomicMin(&A->evt_thread, c.tid);
    __syncthreads();
    if (A->evt_thread == c.tid) {
        if (ph) { A->hit_bin = bh; A->hit_qbefore = eq; A->hit_cbefore = ec; }
        else { A->hit_bin = bl; A->hit_qbefore = eq + qh; A->hit_cbefore = ec + ch; }
    }
    __syncthreads();
}

// Gather every remaining element of bin `bin` (exp bits below `tau`) into CTA 0's
// candidate list as sortable keys (value bits high, inverted token id low).
__device__ void gather_bin(Ctx &c, int bin_lo, unsigned int tau) {
    Aux *A0 = c.cluster.map_shared_rank(c.A, 0);
    for (int i = c.c0; i < c.c1; i++) {
        unsigned int eb = __float_as_uint(c.row[i]);
        if (eb < tau && (int)(eb >> BIN_SHIFT) >= bin_lo) {
            int pos = atomicAdd(&A0->ncand, 1);
            if (pos < NC)
                A0->cand[pos] = ((unsigned long long)eb << 32) |
                                (unsigned long long)(0xFFFFFFFFu - (unsigned int)(c.base + i));
        }
    }
}

__device__ __forceinline__ int key_idx(unsigned long long k) {
    return (int)(0xFFFFFFFFu - (unsigned int)(k & 0xFFFFFFFFull));
}
__device__ __forceinline__ float key_val(unsigned long long k) {
    return __uint_as_float((unsigned int)(k >> 32));
}

// Sort CTA 0's candidate list (descending value, ascending token id) and turn the
// exponentials into probabilities p = e / Z (sample.mojo:437-438). CTA 0 only.
__device__ void sort_cands(Ctx &c, int n, float Z) {
    Aux *A = c.A;
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    if (n2 < 2) n2 = 2;
    for (int i = n + c.tid; i < n2; i += NT) A->cand[i] = 0ull;
    bitonic_desc(A->cand, n2, c.tid);
    for (int i = c.tid; i < n; i += NT) A->pc[i] = __fdiv_rn(key_val(A->cand[i]), Z);
    __syncthreads();
}

__device__ __forceinline__ void publish(Ctx &c, const Bcast &b) {
    for (int r = 0; r < c.cs; r++) {
        Aux *RA = c.cluster.map_shared_rank(c.A, r);
        RA->bc = b;
    }
}

// =============================================================================
// The descending walk past the sorted head (sample.mojo:492-506 and :580-590 on
// rows whose nucleus is larger than the head). State: exact running sum `s`,
// elements consumed `pos`, and `tau`: everything with exp bits >= tau is consumed.
// Each phase histograms the remaining elements by value bin with their integer
// contributions in the current binade, consumes whole bins up to the first bin
// holding an event (the sum reaching x_ge, exceeding x_gt, leaving the binade, a
// count limit, or an element needing sequential care), then gathers that bin,
// sorts it and adds it element by element.
// =============================================================================
struct Walk {
    float s; long long pos; unsigned int tau;
    int event; int idx; float p; int tie;  // outcome
};

__device__ void descend(Ctx &c, float Z, Walk &w, float x_ge, float x_gt, long long nstop,
                        unsigned int &status) {
    Aux *A = c.A;
    const bool counting = nstop >= 0;
    for (int phase = 0; phase < 4096; phase++) {
        // ---- histogram of what remains
        for (int i = c.tid; i < NBINS; i += NT) { A->u.h.hq[i] = 0ull; A->u.h.hc[i] = 0u; }
        if (c.tid == 0) { A->specbin = -1; if (c.rank == 0) A->ncand = 0; }
        __syncthreads();
        const bool have_s = w.s > 0.0f;
        const int j = have_s ? fexpo(w.s) : 0;
        const bool binade_ok = have_s && j >= -100 && j <= 100;
        const float Cm = __fmul_rn(1.5f, fpow2(j)), halfu = fpow2(j - 24), bigthr = fpow2(j - 1);
        const float inv_u = fpow2(23 - j);
        for (int i = c.c0; i < c.c1; i++) {
            const float e = c.row[i];
            const unsigned int eb = __float_as_uint(e);
            if (eb >= w.tau) continue;
            const int bin = (int)(eb >> BIN_SHIFT);
            if (!binade_ok) {
                atomicAdd(&A->u.h.hc[bin], 1u);
                continue;
            }
            const float p = __fdiv_rn(e, Z);
            const float q = __fsub_rn(__fadd_rn(p, Cm), Cm);
            const float r = __fsub_rn(p, q);
            if (fabsf(r) == halfu || p >= bigthr) {
                atomicMax(&A->specbin, bin);
                if (counting) atomicAdd(&A->u.h.hc[bin], 1u);
                continue;
            }
            const unsigned int qu = __float2uint_rn(__fmul_rn(q, inv_u));
            if (qu) atomicAdd(&A->u.h.hq[bin], (unsigned long long)qu);
            if (counting) atomicAdd(&A->u.h.hc[bin], 1u);
        }
        __syncthreads();
        int specbin = -1;
        {
            const unsigned long long *xs = xchg(c, (unsigned long long)(unsigned int)(A->specbin + 1));
            for (int r = 0; r < c.cs; r++) specbin = max(specbin, (int)(unsigned int)xs[r] - 1);
        }
        // ---- first bin (descending) that holds an event
        BinQuery qy;
        qy.specbin = specbin;
        qy.pos0 = (unsigned long long)w.pos;
        qy.nstop = counting ? (unsigned long long)nstop : ~0ull;
        qy.m0 = 0; qy.xq = ~0ull;
        if (binade_ok) {
            qy.m0 = (unsigned long long)((double)w.s * (double)inv_u);
            unsigned long long xq = 1ull << 24;  // leaving the binade
            if (x_ge < 3.0e38f) {
                double t = ceil((double)x_ge * (double)inv_u);
                if (t < (double)xq) xq = (t <= 0.0) ? 0ull : (unsigned long long)t;
            }
            if (x_gt < 3.0e38f) {
                double t = floor((double)x_gt * (double)inv_u) + 1.0;
                if (t < (double)xq) xq = (t <= 0.0) ? 0ull : (unsigned long long)t;
            }
            qy.xq = xq;
        } else {
            // no usable binade yet (nothing consumed): take the highest non-empty bin
            qy.pos0 = 0; qy.nstop = 1;
        }
        find_event_bin(c, qy);
        const int hb = A->hit_bin;
        if (hb < 0) {
            // nothing left triggers an event: consume everything
            if (binade_ok) w.s = (float)((double)(qy.m0 + A->tot_q) * (double)fpow2(j - 23));
            w.pos += (long long)A->tot_c;
            w.tau = 0;
            w.event = EV_EXHAUSTED;
            c.cluster.sync();
            return;
        }
        const unsigned long long qb = A->hit_qbefore, cb = A->hit_cbefore;
        // ---- gather that bin into CTA 0 and walk it element by element
        {
            Aux *A0 = c.cluster.map_shared_rank(A, 0);
            for (int i = c.c0; i < c.c1; i++) {
                unsigned int eb = __float_as_uint(c.row[i]);
                if (eb < w.tau && (int)(eb >> BIN_SHIFT) == hb) {
                    int pos = atomicAdd(&A0->ncand, 1);
                    if (pos < NC)
                        A0->cand[pos] = ((unsigned long long)eb << 32) |
                                        (unsigned long long)(0xFFFFFFFFu - (unsigned int)(c.base + i));
                }
            }
        }
        c.cluster.sync();
        if (c.rank == 0) {
            const int nb = A->ncand;
            Bcast b;
            b.event = EV_NONE; b.idx = -1; b.p = 0.0f; b.aux = 0;
            if (nb > NC) {
                b.event = EV_DEGENERATE; b.s = w.s; b.pos = w.pos; b.tau = w.tau;
                if (c.tid == 0) publish(c, b);
            } else {
                sort_cands(c, nb, Z);
                if (c.tid == 0) {
                    float s = binade_ok ? (float)((double)(qy.m0 + qb) * (double)fpow2(j - 23)) : w.s;
                    long long pos = w.pos + (counting || !binade_ok ? (long long)cb : 0);
                    for (int i = 0; i < nb; i++) {
                        const float p = A->pc[i];
                        s = __fadd_rn(s, p);
                        pos++;
                        int ev = EV_NONE;
                        if (s >= x_ge) ev = EV_CUT;
                        else if (x_gt < s) ev = EV_DRAW;
                        else if (counting && pos >= nstop) ev = EV_LIMIT;
                        if (ev != EV_NONE) {
                            b.event = ev; b.idx = key_idx(A->cand[i]); b.p = p;
                            bool tie = (i > 0 && A->pc[i - 1] == p) || (i + 1 < nb && A->pc[i + 1] == p);
                            b.aux = tie ? 1 : 0;
                            break;
                        }
                    }
                    b.s = s; b.pos = pos; b.tau = (unsigned int)hb << BIN_SHIFT;
                    publish(c, b);
                }
            }
        }
        c.cluster.sync();
        const Bcast b = A->bc;
        w.s = b.s; w.pos = b.pos; w.tau = b.tau;
        if (b.event == EV_DEGENERATE) { w.event = EV_DEGENERATE; status |= MOLLA_ROW_DEGENERATE; return; }
        if (b.event != EV_NONE) { w.event = b.event; w.idx = b.idx; w.p = b.p; w.tie = b.aux; return; }
        if (phase > 8) status |= MOLLA_ROW_SLOW_PATH;
    }
    w.event = EV_DEGENERATE;
    status |= MOLLA_ROW_DEGENERATE;
}

// =============================================================================
// The kernel: a persistent cluster per row.
// =============================================================================
__global__ void __launch_bounds__(NT, 1) sample_rows_kernel(const __grid_constant__ BatchArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Ctx c{cg::this_cluster()};
    c.cs = (int)c.cluster.num_blocks();
    c.rank = (int)c.cluster.block_rank();
    c.tid = threadIdx.x; c.lane = c.tid & 31; c.warp = c.tid >> 5;
    c.row = reinterpret_cast<float *>(smem_raw);
    c.A = reinterpret_cast<Aux *>(smem_raw + (((size_t)a.S * 4 + 127) / 128) * 128);
    c.S = a.S; c.L = a.L; c.V = a.V;
    Aux *A = c.A;
    const int ncl = gridDim.x / c.cs;
    const int cid = blockIdx.x / c.cs;
    c.base = c.rank * c.S;
    {
        long long nl = (long long)a.V - c.base;
        c.nloc = (int)(nl < 0 ? 0 : (nl > c.S ? c.S : nl));
    }
    c.c0 = min(c.nloc, c.tid * c.L);
    c.c1 = min(c.nloc, (c.tid + 1) * c.L);
    if (c.tid == 0) { mbar_init(&A->mbar, 1); fence_proxy_async(); }
    unsigned int parity = 0;
    c.cluster.sync();

    for (int r = cid; r < a.B; r += ncl) {
        unsigned int status = 0;
        const float T = a.temperature ? a.temperature[r] : 0.0f;
        const int k = a.top_k ? a.top_k[r] : 0;
        const float P = a.top_p ? a.top_p[r] : 1.0f;
        const float minp = a.min_p ? a.min_p[r] : 0.0f;
        const float typ = a.typical_p ? a.typical_p[r] : 1.0f;
        const float rp = a.repeat_penalty ? a.repeat_penalty[r] : 1.0f;
        const float fp = a.frequency_penalty ? a.frequency_penalty[r] : 0.0f;
        const float pp = a.presence_penalty ? a.presence_penalty[r] : 0.0f;
        const bool won = a.window_on ? (a.window_on[r] != 0) : true;
        const int h0 = (a.hist && a.hist_off) ? a.hist_off[r] : 0;
        const int H = (a.hist && a.hist_off) ? (a.hist_off[r + 1] - h0) : 0;
        const int b0 = (a.bias_ids && a.bias_off) ? a.bias_off[r] : 0;
        const int nb = (a.bias_ids && a.bias_off) ? (a.bias_off[r + 1] - b0) : 0;
        // the rules of SamplerConfig.check (sample.mojo:140-154); NaN fails every test
        bool valid = (T >= 0.0f) && (k >= 0) && (P > 0.0f && P <= 1.0f) && (minp >= 0.0f && minp <= 1.0f) &&
                     (typ > 0.0f && typ <= 1.0f) && (rp > 0.0f) && H >= 0 && nb >= 0;
        const bool greedy = !(T > 0.0f);
        if (!a.penalised_only) {
            if (!valid) status |= MOLLA_ROW_INVALID_CONFIG;
            else if (!greedy && (minp > 0.0f || typ < 1.0f)) status |= MOLLA_ROW_UNSUPPORTED;
            if (status) {
                if (c.rank == 0 && c.tid == 0) {
                    a.tokens[r] = -1; a.row_status[r] = status;
                    if (a.diag) { a.diag[4 * r] = a.diag[4 * r + 1] = a.diag[4 * r + 2] = a.diag[4 * r + 3] = 0.0f; }
                }
                continue;
            }
        }
        const bool penalizing = won && H > 0 && (rp != 1.0f || fp != 0.0f || pp != 0.0f);

        STAMP(0);
        // ---- 1. fetch this CTA's slice of the row, once, from HBM
        const float *src = a.logits + (long long)r * a.row_stride + c.base;
        {
            const bool aligned = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0);
            const int nbulk = aligned ? (c.nloc & ~3) : 0;
            if (nbulk > 0) {
                if (c.tid == 0) {
                    fence_proxy_async();
                    mbar_expect_tx(&A->mbar, (uint32_t)nbulk * 4u);
                    const int PIECE = 8192;  // floats per bulk copy (32 KB)
                    for (int o = 0; o < nbulk; o += PIECE) {
                        int n = min(PIECE, nbulk - o);
                        bulk_g2s(c.row + o, src + o, (uint32_t)n * 4u, &A->mbar);
                    }
                }
            }
            for (int i = nbulk + c.tid; i < c.nloc; i += NT) c.row[i] = __ldg(src + i);
            if (nbulk > 0) {
                bool done = false;
                for (int spin = 0; spin < (1 << 22); spin++) {
                    if (mbar_try_wait(&A->mbar, parity)) { done = true; break; }
                }
                if (!done) status |= MOLLA_ROW_LOAD_TIMEOUT;
                parity ^= 1u;
            }
            __syncthreads();
        }

        STAMP(1);
        // ---- 2. logit bias, then penalties, scattered over the window's tokens
        // (sample.mojo:381-417: bias first, each in the reference's operation order)
        if (nb > 0) {
            for (int jx = c.tid; jx < nb; jx += NT) {
                const long long tok = a.bias_ids[b0 + jx];
                if (tok < c.base || tok >= (long long)c.base + c.nloc) continue;
                bool first = true;
                for (int q = 0; q < jx; q++)
                    if (a.bias_ids[b0 + q] == tok) { first = false; break; }
                if (!first) continue;
                float v = c.row[tok - c.base];
                for (int q = 0; q < nb; q++)
                    if (a.bias_ids[b0 + q] == tok) v = __fadd_rn(v, a.bias_vals[b0 + q]);
                c.row[tok - c.base] = v;
            }
            __syncthreads();
        }
        if (penalizing) {
            const bool staged = H <= HIST_STAGE;
            if (staged) {
                for (int h = c.tid; h < H; h += NT) {
                    long long t = a.hist[h0 + h];
                    A->u.hist_tok[h] = (t >= 0 && t < a.V) ? (int)t : -1;
                }
                __syncthreads();
            }
            for (int h = c.tid; h < H; h += NT) {
                long long tok = staged ? (long long)A->u.hist_tok[h] : a.hist[h0 + h];
                if (tok < c.base || tok >= (long long)c.base + c.nloc) continue;
                int n = 0;
                bool first = true;
                if (staged) {
                    const int ti = (int)tok;
                    for (int q = 0; q < H; q++) {
                        if (A->u.hist_tok[q] == ti) { n++; if (q < h) first = false; }
                    }
                } else {
                    for (int q = 0; q < H; q++) {
                        if (a.hist[h0 + q] == tok) { n++; if (q < h) first = false; }
                    }
                }
                if (!first) continue;
                float v = c.row[tok - c.base];
                if (v > 0.0f) v = __fdiv_rn(v, rp);
                else v = __fmul_rn(v, rp);
                v = __fsub_rn(v, __fmul_rn((float)n, fp));
                v = __fsub_rn(v, pp);
                c.row[tok - c.base] = v;
            }
            __syncthreads();
        }
        if (a.penalised) {
            float *dst = a.penalised + (long long)r * a.V + c.base;
            for (int i = c.tid; i < c.nloc; i += NT) dst[i] = c.row[i];
        }
        if (a.penalised_only) { c.cluster.sync(); continue; }

        STAMP(2);
        // ---- 3. maximum and its first index (kernel.mojo:571-585, sample.mojo:342-346)
        float mx = -INFINITY;
        int mi = 0x7fffffff;
        for (int i = c.c0; i < c.c1; i++) {
            float x = c.row[i];
            if (x > mx) { mx = x; mi = c.base + i; }
        }
        if (c.c1 > c.c0 && mi == 0x7fffffff) mi = c.base + c.c0;  // all -inf / NaN guard
        block_argmax(c, mx, mi);
        float xmax; int imax;
        {
            const unsigned long long *xs = xchg(c, pack_fi(mx, mi));
            xmax = __uint_as_float((unsigned int)(xs[0] >> 32)); imax = (int)(unsigned int)xs[0];
            for (int q = 1; q < c.cs; q++) {
                float ov = __uint_as_float((unsigned int)(xs[q] >> 32)); int oi = (int)(unsigned int)xs[q];
                if (ov > xmax || (ov == xmax && oi < imax)) { xmax = ov; imax = oi; }
            }
        }
        STAMP(3);
        const long long n_lim = (k > 0 && k < a.V) ? (long long)k : (long long)a.V;

        int token = -1;
        float dZ = 0.0f, dsum = 0.0f, dtarget = 0.0f, dp = 0.0f;

        if (greedy) {
            token = imax;
        } else {
            // ---- 4. temperature, exponentials (sample.mojo:419-434) and chunk statistics
            const float top = (T == 1.0f) ? xmax : __fdiv_rn(xmax, T);
            float csum = 0.0f, cmx = -1.0f;
            int nties = 0;
            for (int i = c.c0; i < c.c1; i++) {
                float x = c.row[i];
                float v = (T == 1.0f) ? x : __fdiv_rn(x, T);
                float e = expf_pinned(__fsub_rn(v, top));
                c.row[i] = e;
                csum = __fadd_rn(csum, e);
                cmx = fmaxf(cmx, e);
                nties += (e == 1.0f) ? 1 : 0;
            }
            A->cmax[c.tid] = cmx;
            STAMP(4);
            if (n_lim == 1) {
                // top-k of one: the sort's first element is a maximum (sample.mojo:485-490)
                int tot;
                (void)block_excl_scan<int>(nties, A->wsi, &tot);
                const unsigned long long *xs = xchg(c, (unsigned long long)(unsigned int)tot);
                int all = 0;
                for (int q = 0; q < c.cs; q++) all += (int)(unsigned int)xs[q];
                if (all > 1) status |= MOLLA_ROW_TOPK_TIE;
                token = imax;
            } else {
                // ---- 5. the softmax denominator, exactly as the sequential loop rounds it
                p1_build(c, csum);
                STAMP(5);
                if (c.rank == 0 && c.tid == 0) {
                    P1Walk w;
                    p1_walk(c, false, 0.0f, w);
                    Bcast b; b.s = w.s; b.aux = w.slow; b.event = 0; b.idx = 0; b.p = 0; b.pos = 0; b.tau = 0;
                    publish(c, b);
                }
                c.cluster.sync();
                const float Z = A->bc.s;
                STAMP(6);
                if (A->bc.aux) status |= MOLLA_ROW_SLOW_PATH;
                dZ = Z;
                const float u01 = draw01(a.seed ? a.seed[r] : 0ull, a.drawn ? a.drawn[r] : 0ull);
                const bool topp_on = (P < 1.0f) && (n_lim > 1);

                if (!topp_on && n_lim == (long long)a.V) {
                    // ---- 6a. nothing sorted: the draw walks the vocabulary in order
                    // (sample.mojo:365-369, 580-594), over p = e / Z
                    float ps = 0.0f;
                    for (int i = c.c0; i < c.c1; i++) {
                        float p = __fdiv_rn(c.row[i], Z);
                        c.row[i] = p;
                        ps = __fadd_rn(ps, p);
                    }
                    p1_build(c, ps);
                    if (c.rank == 0 && c.tid == 0) {
                        P1Walk w;
                        p1_walk(c, false, 0.0f, w);
                        const float sum = w.s;
                        int slow = w.slow;
                        const float target = __fmul_rn(u01, sum);
                        P1Walk w2;
                        p1_walk(c, true, target, w2);
                        slow |= w2.slow;
                        Bcast b; b.s = sum; b.p = target; b.aux = slow; b.event = 0; b.pos = 0; b.tau = 0;
                        b.idx = w2.found ? (int)w2.idx : (a.V - 1);
                        publish(c, b);
                    }
                    c.cluster.sync();
                    token = A->bc.idx; dsum = A->bc.s; dtarget = A->bc.p;
                    if (A->bc.aux) status |= MOLLA_ROW_SLOW_PATH;
                    if (token >= 0 && c.rank == 0 && c.tid == 0) {
                        const int owner = token / c.S;  // probability of the chosen token (diagnostic)
                        dp = c.cluster.map_shared_rank(c.row, owner)[token - owner * c.S];
                    }
                } else {
                    // ---- 6b. sorted order. Head: the top candidates, sorted, walked exactly.
                    long long need = n_lim + 1;
                    if (need > HEAD_MAX) need = HEAD_MAX;
                    if (need > a.V) need = a.V;
                    // The need-th largest chunk maximum bounds the need-th largest element from
                    // below, so a histogram of the chunk maxima alone gives a safe value threshold.
                    for (int i = c.tid; i < NBINS; i += NT) { A->u.h.hq[i] = 0ull; A->u.h.hc[i] = 0u; }
                    if (c.tid == 0 && c.rank == 0) A->ncand = 0;
                    __syncthreads();
                    if (cmx >= 0.0f) atomicAdd(&A->u.h.hc[__float_as_uint(cmx) >> BIN_SHIFT], 1u);
                    c.cluster.sync();
                    BinQuery qy; qy.m0 = 0; qy.xq = ~0ull; qy.pos0 = 0; qy.nstop = (unsigned long long)need; qy.specbin = -1;
                    find_event_bin(c, qy);
                    int hb = A->hit_bin < 0 ? 0 : A->hit_bin;
                    gather_bin(c, hb, 0xFFFFFFFFu);
                    c.cluster.sync();  // histograms read, candidates gathered
                    int nc = c.cluster.map_shared_rank(A, 0)->ncand;
                    c.cluster.sync();
                    if (nc > NC) {
                        // Too many (flat or tiny rows): count every element per bin and keep the
                        // highest bins that fit the candidate list.
                        for (int i = c.tid; i < NBINS; i += NT) A->u.h.hc[i] = 0u;
                        if (c.tid == 0 && c.rank == 0) A->ncand = 0;
                        __syncthreads();
                        for (int i = c.c0; i < c.c1; i++) atomicAdd(&A->u.h.hc[__float_as_uint(c.row[i]) >> BIN_SHIFT], 1u);
                        c.cluster.sync();
                        qy.nstop = (unsigned long long)NC + 1ull;
                        find_event_bin(c, qy);
                        hb = A->hit_bin < 0 ? 0 : A->hit_bin + 1;
                        if (hb < NBINS) gather_bin(c, hb, 0xFFFFFFFFu);
                        c.cluster.sync();
                        nc = c.cluster.map_shared_rank(A, 0)->ncand;
                        c.cluster.sync();
                        status |= MOLLA_ROW_SLOW_PATH;
                    }
                    STAMP(7);
                    const unsigned int tau_head = (hb >= NBINS) ? 0x7F800000u : ((unsigned int)hb << BIN_SHIFT);
                    // ---- head walk on CTA 0 (sample.mojo:497-506 then :580-590)
                    if (c.rank == 0) {
                        sort_cands(c, nc, Z);
                        for (int i = c.tid; i < nc; i += NT) {
                            const float p = A->pc[i];
                            const bool eq = (i > 0 && A->pc[i - 1] == p) || (i + 1 < nc && A->pc[i + 1] == p);
                            A->hidx[i] = (unsigned int)key_idx(A->cand[i]) | (eq ? 0x80000000u : 0u);
                        }
                        __syncthreads();
                        if (c.tid == 0) {
                            Bcast b; b.event = EV_NONE; b.idx = -1; b.p = 0; b.aux = 0; b.tau = tau_head;
                            float s = 0.0f;
                            long long pos = 0;
                            int cut = -1;  // kept count once known
                            int tie = 0;
                            for (int i = 0; i < nc; i++) {
                                if (pos >= n_lim) break;
                                s = __fadd_rn(s, A->pc[i]);
                                A->pre[i] = s;
                                pos++;
                                if (topp_on && s >= P) {
                                    cut = i + 1;
                                    if (i + 1 < nc && (long long)(i + 1) < n_lim && A->pc[i + 1] == A->pc[i]) tie |= MOLLA_ROW_TOPP_TIE;
                                    break;
                                }
                                if (pos >= n_lim) { cut = i + 1; break; }
                            }
                            if (cut < 0 && nc == a.V) cut = nc;
                            if (n_lim < (long long)a.V && (long long)nc > n_lim && A->pc[n_lim] == A->pc[n_lim - 1])
                                tie |= MOLLA_ROW_TOPK_TIE;
                            b.s = s; b.pos = pos;
                            if (cut > 0) {
                                const float sum = A->pre[cut - 1];
                                const float target = __fmul_rn(u01, sum);
                                int at = cut - 1;
                                for (int i = 0; i < cut; i++)
                                    if (target < A->pre[i]) { at = i; break; }
                                b.event = EV_DRAW; b.idx = (int)(A->hidx[at] & 0x7fffffffu); b.p = A->pc[at];
                                if ((at > 0 && A->pc[at - 1] == A->pc[at]) || (at + 1 < cut && A->pc[at + 1] == A->pc[at]))
                                    tie |= MOLLA_ROW_CHOSEN_TIE;
                                dsum = sum; dtarget = target;
                            }
                            b.aux = tie;
                            publish(c, b);
                        }
                    }
                    c.cluster.sync();
                    const Bcast hbq = A->bc;
                    STAMP(8);
                    status |= (unsigned int)hbq.aux;
                    if (hbq.event == EV_DRAW) {
                        token = hbq.idx; dp = hbq.p;
                    } else {
                        // ---- 7. past the head: the cut walk, then the draw walk
                        Walk cutw; cutw.s = hbq.s; cutw.pos = hbq.pos; cutw.tau = tau_head;
                        cutw.event = EV_NONE; cutw.idx = -1; cutw.p = 0; cutw.tie = 0;
                        const bool limited = n_lim < (long long)a.V;
                        descend(c, Z, cutw, topp_on ? P : 3.4e38f, 3.4e38f, limited ? n_lim : -1, status);
                        if (cutw.event == EV_DEGENERATE) {
                            token = -1;
                        } else {
                            if (cutw.event == EV_CUT && cutw.tie) status |= MOLLA_ROW_TOPP_TIE;
                            if (cutw.event == EV_LIMIT && cutw.tie) status |= MOLLA_ROW_TOPK_TIE;
                            const float sum = cutw.s;
                            const float target = __fmul_rn(u01, sum);
                            dsum = sum; dtarget = target;
                            // is the drawn element in the head?
                            if (c.rank == 0 && c.tid == 0) {
                                Bcast b; b.event = EV_NONE; b.idx = -1; b.p = 0; b.aux = 0; b.s = 0; b.pos = 0; b.tau = 0;
                                int at = -1;
                                for (int i = 0; i < nc; i++)
                                    if (target < A->pre[i]) { at = i; break; }
                                if (at >= 0) {
                                    b.event = EV_DRAW; b.idx = (int)(A->hidx[at] & 0x7fffffffu);
                                    b.p = __fsub_rn(A->pre[at], at > 0 ? A->pre[at - 1] : 0.0f);
                                    if (A->hidx[at] & 0x80000000u) b.aux = MOLLA_ROW_CHOSEN_TIE;
                                }
                                publish(c, b);
                            }
                            c.cluster.sync();
                            const Bcast hd = A->bc;
                            if (hd.event == EV_DRAW) {
                                token = hd.idx; dp = hd.p; status |= (unsigned int)hd.aux;
                            } else {
                                bool resolved = false;
                                if (target < sum) {
                                    Walk dw; dw.s = hbq.s; dw.pos = hbq.pos; dw.tau = tau_head;
                                    dw.event = EV_NONE; dw.idx = -1; dw.p = 0; dw.tie = 0;
                                    descend(c, Z, dw, 3.4e38f, target, -1, status);
                                    if (dw.event == EV_DRAW) {
                                        token = dw.idx; dp = dw.p; resolved = true;
                                        if (dw.tie) status |= MOLLA_ROW_CHOSEN_TIE;
                                    } else if (dw.event == EV_DEGENERATE) {
                                        token = -1; resolved = true;
                                    }
                                }
                                if (!resolved) {
                                    // the walk falls off the end: the last kept candidate (sample.mojo:591-594)
                                    if (cutw.event == EV_CUT || cutw.event == EV_LIMIT) {
                                        token = cutw.idx; dp = cutw.p;
                                    } else {
                                        // everything was kept: the smallest probability, highest id last
                                        float nv = -INFINITY; int ni = 0x7fffffff;
                                        for (int i = c.c0; i < c.c1; i++) {
                                            const float e = -c.row[i];
                                            const int id = 0x7fffffff - (c.base + i);
                                            if (e > nv || (e == nv && id < ni)) { nv = e; ni = id; }
                                        }
                                        block_argmax(c, nv, ni);
                                        const unsigned long long *xs = xchg(c, pack_fi(nv, ni));
                                        float bv = __uint_as_float((unsigned int)(xs[0] >> 32)); int bi = (int)(unsigned int)xs[0];
                                        for (int q = 1; q < c.cs; q++) {
                                            float ov = __uint_as_float((unsigned int)(xs[q] >> 32)); int oi = (int)(unsigned int)xs[q];
                                            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
                                        }
                                        token = 0x7fffffff - bi;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
        STAMP(9);
        if (c.rank == 0 && c.tid == 0) {
            a.tokens[r] = token;
            a.row_status[r] = status;
            if (a.diag) { a.diag[4 * r] = dZ; a.diag[4 * r + 1] = dsum; a.diag[4 * r + 2] = dtarget; a.diag[4 * r + 3] = dp; }
        }
        // the row buffer and the tables are free again only when every CTA is done with them
        c.cluster.sync();
    }
}

// =============================================================================
// Logprobs of the raw logits (sample.mojo:268-293): one CTA per row, the row is
// read twice (second read is an L2 hit for blocks that fit).
// =============================================================================
__global__ void __launch_bounds__(NT, 1) logprob_kernel(const float *logits, long long row_stride, int B, int V,
                                                        const int *tokens, int top_n, float *chosen_lp,
                                                        int *top_ids, float *top_lps, float *full_out) {
    __shared__ float wsf[NWARP + 1];
    __shared__ double wsd[NWARP + 1];
    __shared__ unsigned long long cand[NT];
    __shared__ int ncand;
    __shared__ float s_thr;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int r = blockIdx.x; r < B; r += gridDim.x) {
        const float *z = logits + (long long)r * row_stride;
        // pass 1: maximum and each thread's own maximum
        float tm = -INFINITY;
        for (int i = tid; i < V; i += NT) tm = fmaxf(tm, __ldg(z + i));
        float m = warp_max(tm);
        __syncthreads();
        if (lane == 0) wsf[warp] = m;
        __syncthreads();
        float top = wsf[0];
        for (int w = 1; w < NWARP; w++) top = fmaxf(top, wsf[w]);
        // threshold for the top-N: the N-th largest of the per-thread maxima
        float thr = -INFINITY;
        if (top_n > 0) {
            // order-preserving key of a float
            unsigned int b = __float_as_uint(tm);
            unsigned int key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
            __syncthreads();
            cand[tid] = ((unsigned long long)key << 32) | (unsigned long long)tid;
            bitonic_desc(cand, NT, tid);
            if (tid == 0) {
                int nth = min(top_n, V) - 1;
                unsigned int kk = (unsigned int)(cand[nth] >> 32);
                unsigned int bb = (kk & 0x80000000u) ? (kk & 0x7fffffffu) : ~kk;
                s_thr = __uint_as_float(bb);
                ncand = 0;
            }
            __syncthreads();
            thr = s_thr;
        }
        // pass 2: sum of exp(z - top) accumulated in fp64, candidates for the top-N
        double acc = 0.0;
        for (int i = tid; i < V; i += NT) {
            float x = __ldg(z + i);
            acc += (double)expf_pinned(__fsub_rn(x, top));
            if (top_n > 0 && x >= thr) {
                int pos = atomicAdd(&ncand, 1);
                if (pos < NT) {
                    unsigned int b = __float_as_uint(x);
                    unsigned int key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
                    cand[pos] = ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)i);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        __syncthreads();
        if (lane == 0) wsd[warp] = acc;
        __syncthreads();
        double sum = 0.0;
        for (int w = 0; w < NWARP; w++) sum += wsd[w];
        const float offset = (float)log(sum);
        if (chosen_lp && tokens && tid == 0) {
            int t = tokens[r];
            chosen_lp[r] = (t >= 0 && t < V) ? __fsub_rn(__fsub_rn(__ldg(z + t), top), offset) : 0.0f;
        }
        if (full_out) {
            float *o = full_out + (long long)r * V;
            for (int i = tid; i < V; i += NT) o[i] = __fsub_rn(__fsub_rn(__ldg(z + i), top), offset);
        }
        if (top_n > 0) {
            __syncthreads();
            int n = min(ncand, NT);
            for (int i = n + tid; i < NT; i += NT) cand[i] = 0ull;
            __syncthreads();
            bitonic_desc(cand, NT, tid);
            if (tid < top_n) {
                if (tid < n) {
                    int id = (int)(0xFFFFFFFFu - (unsigned int)(cand[tid] & 0xFFFFFFFFull));
                    top_ids[(long long)r * top_n + tid] = id;
                    top_lps[(long long)r * top_n + tid] = __fsub_rn(__fsub_rn(__ldg(z + id), top), offset);
                } else {
                    top_ids[(long long)r * top_n + tid] = -1;
                    top_lps[(long long)r * top_n + tid] = 0.0f;
                }
            }
        }
        __syncthreads();
    }
}

__global__ void expf_kernel(const float *x, long long n, float *out) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = expf_pinned(x[i]);
}

// =============================================================================
// Host side of the C ABI
// =============================================================================
thread_local char g_err[512] = "";
long long *g_prof = nullptr;

int fail(int code, const char *fmt, const char *detail = "") {
    snprintf(g_err, sizeof(g_err), fmt, detail);
    return code;
}

struct Plan { int cs, S, L, nclusters; size_t smem; };

// Smallest cluster whose CTAs can each hold a slice of the row next to the tables.
int make_plan(int V, int B, Plan &p) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(MOLLA_ERR_CUDA, "cudaGetDevice failed%s");
    int max_optin = 0, sms = 0;
    cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t aux = ((sizeof(Aux) + 127) / 128) * 128 + 128;
    if ((size_t)max_optin <= aux + 4096) return fail(MOLLA_ERR_CUDA, "device shared memory too small%s");
    const long long cap = (((long long)max_optin - (long long)aux) / 4) & ~3ll;
    static const int sizes[] = {1, 2, 4, 8, 16};
    for (int cs : sizes) {
        long long S = (((long long)V + cs - 1) / cs + 3) & ~3ll;
        if (S <= cap) {
            p.cs = cs; p.S = (int)S;
            int L = (int)((S + NT - 1) / NT);
            if ((L & 1) == 0) L += 1;
            p.L = L;
            p.smem = (((size_t)S * 4 + 127) / 128) * 128 + sizeof(Aux);
            cudaError_t e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
            if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "cudaFuncSetAttribute(smem): %s", cudaGetErrorString(e));
            if (cs > 8) {
                e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "cluster size 16 not allowed: %s", cudaGetErrorString(e));
            }
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(cs, 1, 1); cfg.blockDim = dim3(NT, 1, 1); cfg.dynamicSmemBytes = p.smem;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = cs; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.attrs = at; cfg.numAttrs = 1;
            int maxc = 0;
            e = cudaOccupancyMaxActiveClusters(&maxc, sample_rows_kernel, &cfg);
            if (e != cudaSuccess || maxc <= 0) { cudaGetLastError(); maxc = sms / cs > 0 ? sms / cs : 1; }
            p.nclusters = B < maxc ? B : maxc;
            if (p.nclusters < 1) p.nclusters = 1;
            return MOLLA_OK;
        }
    }
    return fail(MOLLA_ERR_VOCAB, "vocabulary too wide for one cluster's shared memory%s");
}

int launch_rows(const BatchArgs &args_in, cudaStream_t st) {
    BatchArgs a = args_in;
    Plan p;
    int rc = make_plan(a.V, a.B, p);
    if (rc != MOLLA_OK) return rc;
    a.S = p.S; a.L = p.L;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.nclusters * p.cs, 1, 1);
    cfg.blockDim = dim3(NT, 1, 1);
    cfg.dynamicSmemBytes = p.smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = p.cs; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_rows_kernel, a);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

}  // namespace

extern "C" {

int32_t molla_sample_abi_version(void) { return MOLLA_SAMPLE_ABI_VERSION; }

const char *molla_sample_last_error(void) { return g_err; }

float molla_sample_draw(uint64_t seed, uint64_t counter) { return draw01(seed, counter); }

int64_t molla_sample_workspace_bytes(int32_t B, int32_t V, int32_t top_n) {
    if (B < 0 || V <= 0 || top_n < 0 || top_n > TOPN_MAX) return fail(MOLLA_ERR_ARGUMENT, "bad shape for the workspace query%s");
    return 256;
}

int32_t molla_sample_batch(const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
                           const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
                           const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
                           const float *d_frequency_penalty, const float *d_presence_penalty,
                           const uint8_t *d_window_on, const uint64_t *d_seed, const uint64_t *d_drawn,
                           const int64_t *d_hist, const int32_t *d_hist_off, const int64_t *d_bias_ids,
                           const float *d_bias_vals, const int32_t *d_bias_off, int32_t top_n,
                           void *d_workspace, int64_t workspace_bytes, void *stream, int32_t *d_tokens,
                           float *d_chosen_logprob, int32_t *d_top_ids, float *d_top_logprobs,
                           uint32_t *d_row_status, float *d_diag) {
    g_err[0] = 0;
    if (!d_logits || !d_tokens || !d_row_status) return fail(MOLLA_ERR_ARGUMENT, "logits, tokens and row status are required%s");
    if (B < 0 || V <= 0 || row_stride < V) return fail(MOLLA_ERR_ARGUMENT, "bad block shape%s");
    if (top_n < 0 || top_n > TOPN_MAX) return fail(MOLLA_ERR_ARGUMENT, "top_n out of range%s");
    if (top_n > 0 && (!d_top_ids || !d_top_logprobs)) return fail(MOLLA_ERR_ARGUMENT, "top_n needs its output arrays%s");
    if ((d_hist == nullptr) != (d_hist_off == nullptr)) return fail(MOLLA_ERR_ARGUMENT, "history ids and offsets go together%s");
    if ((d_bias_ids == nullptr) != (d_bias_off == nullptr) || (d_bias_ids && !d_bias_vals))
        return fail(MOLLA_ERR_ARGUMENT, "bias ids, values and offsets go together%s");
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V, top_n))
        return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.logits = d_logits; a.row_stride = row_stride; a.B = B; a.V = V;
    a.temperature = d_temperature; a.top_k = d_top_k; a.top_p = d_top_p; a.min_p = d_min_p;
    a.typical_p = d_typical_p; a.repeat_penalty = d_repeat_penalty;
    a.frequency_penalty = d_frequency_penalty; a.presence_penalty = d_presence_penalty;
    a.window_on = d_window_on;
    a.seed = (const unsigned long long *)d_seed; a.drawn = (const unsigned long long *)d_drawn;
    a.hist = (const long long *)d_hist; a.hist_off = d_hist_off;
    a.bias_ids = (const long long *)d_bias_ids; a.bias_vals = d_bias_vals; a.bias_off = d_bias_off;
    a.tokens = d_tokens; a.row_status = d_row_status; a.diag = d_diag;
    a.penalised = nullptr; a.penalised_only = 0;
    a.row_counter = (int *)d_workspace;
    a.prof = g_prof;
    int rc = launch_rows(a, st);
    if (rc != MOLLA_OK) return rc;
    if (d_chosen_logprob || top_n > 0) {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int grid = B < sms ? B : sms;
        logprob_kernel<<<grid, NT, 0, st>>>(d_logits, row_stride, B, V, d_tokens, top_n, d_chosen_logprob,
                                            d_top_ids, d_top_logprobs, nullptr);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "logprob launch failed: %s", cudaGetErrorString(e));
    }
    return MOLLA_OK;
}

// ---- host-buffer form ---------------------------------------------------------
namespace {
inline size_t al256(size_t n) { return (n + 255) & ~(size_t)255; }
struct HostLayout {
    size_t logits, f[8], win, seed, drawn, k, hist, hist_off, bias_ids, bias_vals, bias_off;
    size_t tokens, status, chosen, top_ids, top_lps, total;
};
HostLayout host_layout(int B, int V, long long n_hist, long long n_bias, int top_n) {
    HostLayout L;
    size_t o = 256;  // the batched call's own workspace comes first
    L.logits = o; o += al256((size_t)B * V * 4);
    for (int i = 0; i < 8; i++) { L.f[i] = o; o += al256((size_t)B * 4); }
    L.k = o; o += al256((size_t)B * 4);
    L.win = o; o += al256((size_t)B);
    L.seed = o; o += al256((size_t)B * 8);
    L.drawn = o; o += al256((size_t)B * 8);
    L.hist = o; o += al256((size_t)(n_hist > 0 ? n_hist : 1) * 8);
    L.hist_off = o; o += al256((size_t)(B + 1) * 4);
    L.bias_ids = o; o += al256((size_t)(n_bias > 0 ? n_bias : 1) * 8);
    L.bias_vals = o; o += al256((size_t)(n_bias > 0 ? n_bias : 1) * 4);
    L.bias_off = o; o += al256((size_t)(B + 1) * 4);
    L.tokens = o; o += al256((size_t)B * 4);
    L.status = o; o += al256((size_t)B * 4);
    L.chosen = o; o += al256((size_t)B * 4);
    L.top_ids = o; o += al256((size_t)B * (top_n > 0 ? top_n : 1) * 4);
    L.top_lps = o; o += al256((size_t)B * (top_n > 0 ? top_n : 1) * 4);
    L.total = o;
    return L;
}
}  // namespace

int64_t molla_sample_host_workspace_bytes(int32_t B, int32_t V, int64_t n_hist, int64_t n_bias, int32_t top_n) {
    if (B < 0 || V <= 0 || n_hist < 0 || n_bias < 0 || top_n < 0 || top_n > TOPN_MAX)
        return fail(MOLLA_ERR_ARGUMENT, "bad shape for the workspace query%s");
    return (int64_t)host_layout(B, V, n_hist, n_bias, top_n).total;
}

int32_t molla_sample_batch_host(const float *h_logits, int64_t row_stride, int32_t B, int32_t V,
                                const float *temperature, const int32_t *top_k, const float *top_p,
                                const float *min_p, const float *typical_p, const float *repeat_penalty,
                                const float *frequency_penalty, const float *presence_penalty,
                                const uint8_t *window_on, const uint64_t *seed, const uint64_t *drawn,
                                const int64_t *hist, const int32_t *hist_off, const int64_t *bias_ids,
                                const float *bias_vals, const int32_t *bias_off, int32_t top_n,
                                void *d_workspace, int64_t workspace_bytes, void *stream, int32_t *h_tokens,
                                float *h_chosen_logprob, int32_t *h_top_ids, float *h_top_logprobs,
                                uint32_t *h_row_status) {
    g_err[0] = 0;
    if (!h_logits || !h_tokens || !h_row_status || !temperature) return fail(MOLLA_ERR_ARGUMENT, "logits, temperature, tokens and row status are required%s");
    if (B < 0 || V <= 0 || row_stride < V) return fail(MOLLA_ERR_ARGUMENT, "bad block shape%s");
    if (top_n < 0 || top_n > TOPN_MAX || (top_n > 0 && (!h_top_ids || !h_top_logprobs))) return fail(MOLLA_ERR_ARGUMENT, "bad top_n arguments%s");
    if ((hist == nullptr) != (hist_off == nullptr)) return fail(MOLLA_ERR_ARGUMENT, "history ids and offsets go together%s");
    if ((bias_ids == nullptr) != (bias_off == nullptr) || (bias_ids && !bias_vals)) return fail(MOLLA_ERR_ARGUMENT, "bias ids, values and offsets go together%s");
    if (B == 0) return MOLLA_OK;
    // SamplerConfig.check (sample.mojo:140-154) and Sampler.bias (:225-232), before anything is launched
    for (int r = 0; r < B; r++) {
        if (!(temperature[r] >= 0)) return fail(MOLLA_ERR_CONFIG, "a temperature cannot be negative%s");
        if (top_k && top_k[r] < 0) return fail(MOLLA_ERR_CONFIG, "a top-k cannot be negative%s");
        if (top_p && !(top_p[r] > 0 && top_p[r] <= 1)) return fail(MOLLA_ERR_CONFIG, "a top-p has to be above zero and at most one%s");
        if (min_p && !(min_p[r] >= 0 && min_p[r] <= 1)) return fail(MOLLA_ERR_CONFIG, "a min-p has to be between zero and one%s");
        if (typical_p && !(typical_p[r] > 0 && typical_p[r] <= 1)) return fail(MOLLA_ERR_CONFIG, "a typical-p has to be above zero and at most one%s");
        if (repeat_penalty && !(repeat_penalty[r] > 0)) return fail(MOLLA_ERR_CONFIG, "a repetition penalty of zero or less erases a logit%s");
    }
    const long long n_hist = hist_off ? hist_off[B] : 0, n_bias = bias_off ? bias_off[B] : 0;
    for (long long j = 0; j < n_bias; j++)
        if (bias_ids[j] < 0 || bias_ids[j] >= V) return fail(MOLLA_ERR_CONFIG, "a logit bias names a token outside the vocabulary%s");
    const HostLayout L = host_layout(B, V, n_hist, n_bias, top_n);
    if (!d_workspace || workspace_bytes < (int64_t)L.total) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    char *w = (char *)d_workspace;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemsetAsync(w, 0, 256, st);
    if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(w + L.logits, (size_t)V * 4, h_logits, (size_t)row_stride * 4, (size_t)V * 4, (size_t)B, cudaMemcpyHostToDevice, st);
    const float *fsrc[8] = {temperature, top_p, min_p, typical_p, repeat_penalty, frequency_penalty, presence_penalty, nullptr};
    for (int i = 0; i < 7 && e == cudaSuccess; i++)
        if (fsrc[i]) e = cudaMemcpyAsync(w + L.f[i], fsrc[i], (size_t)B * 4, cudaMemcpyHostToDevice, st);
    auto up = [&](size_t off, const void *src, size_t bytes) { if (src && bytes && e == cudaSuccess) e = cudaMemcpyAsync(w + off, src, bytes, cudaMemcpyHostToDevice, st); };
    up(L.k, top_k, (size_t)B * 4); up(L.win, window_on, (size_t)B); up(L.seed, seed, (size_t)B * 8); up(L.drawn, drawn, (size_t)B * 8);
    up(L.hist, hist, (size_t)n_hist * 8); up(L.hist_off, hist_off, (size_t)(B + 1) * 4);
    up(L.bias_ids, bias_ids, (size_t)n_bias * 8); up(L.bias_vals, bias_vals, (size_t)n_bias * 4); up(L.bias_off, bias_off, (size_t)(B + 1) * 4);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "host to device copy failed: %s", cudaGetErrorString(e));
    auto dp = [&](size_t off, const void *src) -> void * { return src ? (void *)(w + off) : nullptr; };
    int rc = molla_sample_batch(
        (const float *)(w + L.logits), V, B, V, (const float *)dp(L.f[0], temperature), (const int32_t *)dp(L.k, top_k),
        (const float *)dp(L.f[1], top_p), (const float *)dp(L.f[2], min_p), (const float *)dp(L.f[3], typical_p),
        (const float *)dp(L.f[4], repeat_penalty), (const float *)dp(L.f[5], frequency_penalty),
        (const float *)dp(L.f[6], presence_penalty), (const uint8_t *)dp(L.win, window_on),
        (const uint64_t *)dp(L.seed, seed), (const uint64_t *)dp(L.drawn, drawn), (const int64_t *)dp(L.hist, hist),
        (const int32_t *)dp(L.hist_off, hist_off), (const int64_t *)dp(L.bias_ids, bias_ids),
        (const float *)dp(L.bias_vals, bias_vals), (const int32_t *)dp(L.bias_off, bias_off), top_n, w, 256, stream,
        (int32_t *)(w + L.tokens), h_chosen_logprob ? (float *)(w + L.chosen) : nullptr,
        top_n > 0 ? (int32_t *)(w + L.top_ids) : nullptr, top_n > 0 ? (float *)(w + L.top_lps) : nullptr,
        (uint32_t *)(w + L.status), nullptr);
    if (rc != MOLLA_OK) return rc;
    e = cudaMemcpyAsync(h_tokens, w + L.tokens, (size_t)B * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_row_status, w + L.status, (size_t)B * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && h_chosen_logprob) e = cudaMemcpyAsync(h_chosen_logprob, w + L.chosen, (size_t)B * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && top_n > 0) {
        e = cudaMemcpyAsync(h_top_ids, w + L.top_ids, (size_t)B * top_n * 4, cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(h_top_logprobs, w + L.top_lps, (size_t)B * top_n * 4, cudaMemcpyDeviceToHost, st);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "device to host copy failed: %s", cudaGetErrorString(e));
    for (int r = 0; r < B; r++)
        if (h_row_status[r] & (MOLLA_ROW_LOAD_TIMEOUT | MOLLA_ROW_DEGENERATE | MOLLA_ROW_INVALID_CONFIG))
            return fail(MOLLA_ERR_DEVICE, "a row reported an error in its status word%s");
    return MOLLA_OK;
}

int32_t molla_sample_penalised(const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
                               const float *d_repeat_penalty, const float *d_frequency_penalty,
                               const float *d_presence_penalty, const uint8_t *d_window_on,
                               const int64_t *d_hist, const int32_t *d_hist_off, const int64_t *d_bias_ids,
                               const float *d_bias_vals, const int32_t *d_bias_off, void *d_workspace,
                               int64_t workspace_bytes, void *stream, float *d_out) {
    g_err[0] = 0;
    if (!d_logits || !d_out) return fail(MOLLA_ERR_ARGUMENT, "logits and output are required%s");
    if (B < 0 || V <= 0 || row_stride < V) return fail(MOLLA_ERR_ARGUMENT, "bad block shape%s");
    if (!d_workspace || workspace_bytes < 256) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.logits = d_logits; a.row_stride = row_stride; a.B = B; a.V = V;
    a.repeat_penalty = d_repeat_penalty; a.frequency_penalty = d_frequency_penalty;
    a.presence_penalty = d_presence_penalty; a.window_on = d_window_on;
    a.hist = (const long long *)d_hist; a.hist_off = d_hist_off;
    a.bias_ids = (const long long *)d_bias_ids; a.bias_vals = d_bias_vals; a.bias_off = d_bias_off;
    a.penalised = d_out; a.penalised_only = 1;
    a.row_counter = (int *)d_workspace;
    return launch_rows(a, (cudaStream_t)stream);
}

int32_t molla_sample_logprobs(const float *d_logits, int64_t row_stride, int32_t B, int32_t V, void *stream,
                              float *d_out) {
    g_err[0] = 0;
    if (!d_logits || !d_out || B < 0 || V <= 0 || row_stride < V) return fail(MOLLA_ERR_ARGUMENT, "bad arguments to logprobs%s");
    if (B == 0) return MOLLA_OK;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = B < sms ? B : sms;
    logprob_kernel<<<grid, NT, 0, (cudaStream_t)stream>>>(d_logits, row_stride, B, V, nullptr, 0, nullptr, nullptr,
                                                          nullptr, d_out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "logprob launch failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

int32_t molla_sample_expf(const float *d_x, int64_t n, void *stream, float *d_out) {
    g_err[0] = 0;
    if (!d_x || !d_out || n < 0) return fail(MOLLA_ERR_ARGUMENT, "bad arguments to expf%s");
    if (n == 0) return MOLLA_OK;
    long long blocks = (n + 255) / 256;
    expf_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(d_x, n, d_out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "expf launch failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

void molla_sample_debug_profile(void *d_stamps) { g_prof = (long long *)d_stamps; }

int32_t molla_sample_sync(void *stream) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "stream synchronize failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

}  // extern "C"
