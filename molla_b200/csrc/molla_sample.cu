// The token-sampling kernel and its C ABI (declared in include/molla_sample.h).
//
// One CTA owns one logit row at a time and streams it twice through shared memory:
// pass A reads it from HBM and finds the maximum; pass B, a moment later, finds the
// same bytes in L2. With one CTA per SM about 150 rows are in flight, which is less
// than the L2 holds, so HBM sees each logit once. In both passes every warp runs its
// own pipeline: it owns a contiguous sixteenth of the row, fetches it piece by piece
// with bulk asynchronous copies (TMA without a tensor map) into its own shared-memory
// slots behind its own mbarriers, and never waits for another warp. Thread blocks that
// run out of rows lend themselves to the blocks still working on a long list (HelpSlot).
//
// The reference (src/molla/engine/sample.mojo) defines its result through
// *sequential* fp32 sums: the softmax denominator is accumulated in vocabulary
// order (:431-434), the top-p prefix and the draw walk in sorted order
// (:497-506, :580-590). A parallel reduction rounds differently, and a different
// last bit moves the top-p cut and the drawn token. So the kernel reproduces
// those sums bit for bit instead of approximating them:
//   * a term smaller than half an ulp of the running sum adds nothing at all. The
//     running sum is never below the largest term before it, so a logit more than
//     17.6 (in temperature-scaled units) below the logarithm of the running sum cannot change
//     any sum and can never be drawn. Pass B drops those (its only per-element work
//     on them is one compare) and leaves the rest as one list, in vocabulary order,
//     of (exp bits, token id) pairs: the "relevant list". Everything after pass B
//     works on that list;
//   * a running fp32 sum of non-negative terms stays inside one binade
//     [2^j, 2^(j+1)) for long stretches; there `s + a` rounds to a multiple of
//     ulp = 2^(j-23), so every term contributes the integer rne(a/ulp) and the
//     contributions add exactly, in any order;
//   * the few places where that fails - the running sum crossing into the next
//     binade, a term that is large against the sum, a rounding tie whose
//     direction depends on the parity of the sum - are found in parallel and
//     replayed sequentially by one thread.
// What cannot be reproduced is the order the reference's unstable heapsort
// (:440-483) leaves equal probabilities in; rows where that order could matter
// are marked in the row status (MOLLA_ROW_*_TIE) and equal probabilities are
// ordered by token id.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/molla_sample.h"
#ifdef MOLLA_SAMPLE_TESTING
#include "../../include/molla_sample_testing.h"
#endif
#include "molla_device.cuh"
#include "molla_exact.cuh"
#include "molla_cluster.h"

using namespace molla;

namespace {

constexpr int LT = 11;               // elements per lane per piece (odd: conflict-free strides)
constexpr int PIECE = 32 * LT;       // 352 floats = 1408 bytes: what one warp fetches at a time
constexpr int NSTAGE = 4;            // pieces in flight per warp
constexpr int MAX_PIECES = 128;      // per warp: V <= 16 * 128 * 352 = 720896
constexpr int STAGE_FLOATS = NWARP * NSTAGE * PIECE;       // 22528 floats = 90112 bytes
constexpr int SLIST_CAP = STAGE_FLOATS / 2;                 // list entries that fit the stage area
constexpr int SA_WORDS = 3 + NWARP + HEAD_NEED + 1;  // max, argmax, ties, region maxima, top thread maxima


struct __align__(16) Aux {
    union {
        struct {
            double pa[NT + 1];
            double pb[NT + 1];
            float csum[NT];
            short ja[NT];
            unsigned char dual[NT];
            unsigned long long segd[NT + 1];  // the walk's segments: first chunk, binade guess, flags
        } p1;
        struct {
            unsigned int hq[NBINS];   // per bin: sum of the low bits of the integer contributions
            unsigned int hqh[NBINS];  // ... and of their high bits
            unsigned int hc[NBINS];
        } h;
        struct {                                 // the streaming passes only
            float pmax[NWARP][MAX_PIECES];       // per warp, per piece: its maximum (pass A)
            unsigned short ppos[NWARP][PIECE];   // per warp: positions of the piece's kept elements
            float rmax[NWARP];                   // per warp: maximum of its region
        } s;
    } u;
    unsigned long long cand[NC];
    float pc[NC];
    float pre[HEADC];
    unsigned int hidx[HEADC];  // head: token id, bit 31 = equal to a neighbour
    int hkey[HSLOTS];
    int hcnt[HSLOTS];
    float hval[HSLOTS];
    uint64_t mbar[NWARP][NSTAGE];
    double wsd[2 * (NWARP + 1)];
    unsigned long long wsu[NWARP + 1];
    float wsf[NWARP + 1];
    int wsi[NWARP + 1];
    int wcnt[NWARP + 1];             // per warp: entries it put on the list
    int woff[NWARP + 1];             // their offsets in the whole list
    int nseg;
    int ncand;
    int cur_row;
    int evt_thread;
    int specbin;
    int hit_bin; unsigned long long hit_qbefore; unsigned long long hit_cbefore;
    unsigned long long tot_q; unsigned long long tot_c;
    float walk_s; int walk_found; int walk_idx; int walk_slow;
    unsigned int spec_bits[NBINS / 32];  // bins holding an element that needs sequential care
    float blk_s[44];                 // exact running sum at the start of every staged block
    float b_s; unsigned int b_tau; int b_event; int b_idx; float b_p; long long b_pos; int b_aux;
    float b_sum; float b_target;
};


struct Ctx {
    int tid, lane, warp;
    float *stage;         // NWARP x NSTAGE x PIECE floats
    unsigned int *bm;     // bitmap of patched tokens
    Aux *A;
    int V, R;
    bool patching;
    const float *src;     // this row in global memory
    bool aligned;
    bool last_read;       // the pass being streamed is the last one over this row: L2 need not keep it
    float softcap;        // final-logit softcap applied to every logit as it is read (0 = none)
    unsigned int status;
    // this warp's region and pipeline
    int rbeg, rlen, npieces;
    unsigned int parbits;
};



// ---- the warp's own pipeline: piece p of its region lands in slot p % NSTAGE --------
__device__ __forceinline__ float *wslot(const Ctx &c, int p) {
    return c.stage + (c.warp * NSTAGE + (p % NSTAGE)) * PIECE;
}
__device__ __forceinline__ int piece_len(const Ctx &c, int p) {
    const int left = c.rlen - p * PIECE;
    return left > PIECE ? PIECE : left;
}
// lane 0 only; the slot is free (a __syncwarp separates its last reader from here)
__device__ __forceinline__ void piece_issue(Ctx &c, int p) {
    if (!c.aligned || p >= c.npieces) return;
    const int nbulk = piece_len(c, p) & ~3;
    if (nbulk <= 0) return;
    uint64_t *bar = &c.A->mbar[c.warp][p % NSTAGE];
    fence_proxy_async();
    mbar_expect_tx(bar, (uint32_t)nbulk * 4u);
    if (c.last_read) bulk_g2s_last_use(wslot(c, p), c.src + c.rbeg + (long long)p * PIECE, (uint32_t)nbulk * 4u, bar);
    else bulk_g2s(wslot(c, p), c.src + c.rbeg + (long long)p * PIECE, (uint32_t)nbulk * 4u, bar);
}
__device__ __forceinline__ void pieces_begin(Ctx &c) {
    __syncwarp();
    if (c.lane == 0)
        for (int p = 0; p < NSTAGE - 1; p++) piece_issue(c, p);
}
// Make piece p readable by the whole warp; returns its slot and length. Requests piece
// p + NSTAGE - 1 into the slot the warp finished with in the previous iteration.
__device__ __forceinline__ const float *piece_acquire(Ctx &c, int p, int &n) {
    n = piece_len(c, p);
    float *slot = wslot(c, p);
    __syncwarp();  // the warp is done with the slot of piece p - 1
    if (c.lane == 0) piece_issue(c, p + NSTAGE - 1);
    const float *g = c.src + c.rbeg + (long long)p * PIECE;
    if (c.aligned) {
        const int nbulk = n & ~3;
        if (nbulk + c.lane < n) slot[nbulk + c.lane] = __ldg(g + nbulk + c.lane);
        if (nbulk > 0) {
            const int s = p % NSTAGE;
            bool done = false;
            for (int spin = 0; spin < (1 << 22); spin++) {
                if (mbar_try_wait(&c.A->mbar[c.warp][s], (c.parbits >> s) & 1u)) { done = true; break; }
            }
            if (!done) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
            c.parbits ^= (1u << s);
        }
    } else {
        for (int i = c.lane; i < n; i += 32) slot[i] = __ldg(g + i);
    }
    __syncwarp();
    return slot;
}

// ---- patched tokens: bitmap over the vocabulary + a small hash of their values -----

__device__ __forceinline__ float patch_lookup(const Aux *A, int tok, float x) {
    int s = hslot(tok);
    for (int probe = 0; probe < HSLOTS; probe++) {
        const int k = A->hkey[s];
        if (k == tok) return A->hval[s];
        if (k < 0) return x;
        s = (s + 1) & (HSLOTS - 1);
    }
    return x;
}
// bit j = 1 where element g0 + j (j < 32) is patched
__device__ __forceinline__ unsigned int patch_mask(const Ctx &c, int g0) {
    if (!c.patching) return 0u;
    const int w = g0 >> 5, sh = g0 & 31;
    const int nwords = (c.V + 31) >> 5;
    const unsigned int lo = c.bm[w];
    const unsigned int hi = (w + 1 < nwords) ? c.bm[w + 1] : 0u;
    return __funnelshift_r(lo, hi, sh);
}
// this lane's LT elements of a piece, with patches applied; past the end: -inf
__device__ __forceinline__ void load_chunk(const Ctx &c, const float *slot, int n, int g0, float (&x)[LT]) {
    const int l0 = c.lane * LT;
    const unsigned int pm = (l0 < n) ? (patch_mask(c, g0) & ((1u << LT) - 1u)) : 0u;
#pragma unroll
    for (int j = 0; j < LT; j++) x[j] = (l0 + j < n) ? slot[l0 + j] : -INFINITY;
    if (c.softcap > 0.0f) {
#pragma unroll
        for (int j = 0; j < LT; j++)
            if (l0 + j < n) x[j] = softcap_pinned(x[j], c.softcap);
    }
    if (pm) {
#pragma unroll
        for (int j = 0; j < LT; j++)
            if (((pm >> j) & 1u) && l0 + j < n) x[j] = patch_lookup(c.A, g0 + j, x[j]);
    }
}

// Block-strided loop over a list with four loads in flight per thread (the lists of hot rows
// live in global memory; one dependent load per iteration would leave the loop latency-bound).
template <class F>
__device__ __forceinline__ void for_list(const unsigned long long *lst, int nl, int tid, F f) {
    int i = tid;
    for (; i + 3 * NT < nl; i += 4 * NT) {
        const unsigned long long k0 = lst[i], k1 = lst[i + NT], k2 = lst[i + 2 * NT], k3 = lst[i + 3 * NT];
        f(i, k0); f(i + NT, k1); f(i + 2 * NT, k2); f(i + 3 * NT, k3);
    }
    for (; i < nl; i += NT) f(i, lst[i]);
}


// A row's list as the later phases see it: a copy in shared memory when it is small, else the
// segments pass B wrote (one per warp, each in vocabulary order, `stride` entries apart).
struct LView {
    const unsigned long long *flat;  // shared-memory copy, or nullptr
    unsigned long long *seg;
    size_t stride;
    const int *woff;                 // NWARP + 1 segment offsets into the whole list
    int n;
    uint64_t keep;                   // L2 policy for loads from a list in global memory
    __device__ __forceinline__ unsigned long long *slot(int v) const {
        if (flat) return const_cast<unsigned long long *>(flat) + v;
        int w = 0;
#pragma unroll
        for (int q = 1; q < NWARP; q++) w += (v >= woff[q]) ? 1 : 0;
        return seg + (size_t)w * stride + (size_t)(v - woff[w]);
    }
    __device__ __forceinline__ unsigned long long at(int v) const { return flat ? *slot(v) : __ldcg(slot(v)); }
    // f(index in the whole list, key) over the entries [v0, v1): the whole block on one segment
    // after the other, 16-byte loads (two entries), eight in flight per thread
    template <class F>
    __device__ __forceinline__ void for_range(int tid, int v0, int v1, F f) const {
        const bool one = flat || stride == 0;
        const int nseg = one ? 1 : NWARP;
        for (int w = 0; w < nseg; w++) {
            const unsigned long long *b = flat ? flat : seg + (size_t)w * stride;
            const int o = one ? 0 : woff[w];
            const int m = one ? n : woff[w + 1] - o;
            const int lo = max(v0 - o, 0), hi = min(v1 - o, m);
            if (hi <= lo) continue;
            const int lo2 = (lo + 1) & ~1, hi2 = hi & ~1;
            if (tid == 0 && (lo & 1)) f(o + lo, b[lo]);
            if (tid == 32 && (hi & 1) && hi - 1 >= lo2) f(o + hi - 1, b[hi - 1]);
            const ulonglong2 *b2 = reinterpret_cast<const ulonglong2 *>(b);
            const int p1 = hi2 >> 1;
            // (every round issues its eight loads before it uses one, the last round included:
            // a range is often only a round or two long)
            for (int i = (lo2 >> 1) + tid; i < p1; i += 8 * NT) {
                ulonglong2 k[8];
#pragma unroll
                for (int q = 0; q < 8; q++)
                    k[q] = (i + q * NT < p1) ? (flat ? b2[i + q * NT] : __ldcg(b2 + i + q * NT)) : make_ulonglong2(0ull, 0ull);
#pragma unroll
                for (int q = 0; q < 8; q++)
                    if (i + q * NT < p1) { f(o + 2 * (i + q * NT), k[q].x); f(o + 2 * (i + q * NT) + 1, k[q].y); }
            }
        }
    }
    // f(index in the whole list, key, where the key lives). A list in segments is walked with one
    // warp per segment (pass B left sixteen of similar length); 16-byte loads, eight in flight.
    template <class F>
    __device__ __forceinline__ void for_each(int tid, F f) const {
        unsigned long long *b;
        int o, m, t, step;
        if (flat || stride == 0) { b = flat ? const_cast<unsigned long long *>(flat) : seg; o = 0; m = n; t = tid; step = NT; }
        else {
            const int w = tid >> 5;
            b = seg + (size_t)w * stride; o = woff[w]; m = woff[w + 1] - o; t = tid & 31; step = 32;
        }
        const ulonglong2 *b2 = reinterpret_cast<const ulonglong2 *>(b);
        const int mp = m >> 1;
        int i = t;
        for (; i + 7 * step < mp; i += 8 * step) {
            ulonglong2 k[8];
#pragma unroll
            for (int q = 0; q < 8; q++) k[q] = flat ? b2[i + q * step] : __ldcg(b2 + i + q * step);
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const int e = 2 * (i + q * step);
                f(o + e, k[q].x, b + e); f(o + e + 1, k[q].y, b + e + 1);
            }
        }
        for (; i < mp; i += step) {
            const ulonglong2 k = flat ? b2[i] : __ldcg(b2 + i);
            f(o + 2 * i, k.x, b + 2 * i); f(o + 2 * i + 1, k.y, b + 2 * i + 1);
        }
        if ((m & 1) && t == 0) f(o + m - 1, b[m - 1], b + m - 1);
    }
};


// The whole list, exactly: in one go when it sits in shared memory, else in blocks of bare
// values staged there (`vals`, VBLK entries) with the exact sum carried from block to block.
// The sum at every block start is remembered, so a second run that only has to find where
// the running sum passes `target` rebuilds a single block.
// Result in A->walk_s (and A->walk_found / A->walk_idx = list position when locating).
constexpr int VBLK = STAGE_FLOATS;  // values per staged block
constexpr int MAX_VBLK = 40;

template <class V>
__device__ void p1_block(Ctx &c, V vals, int n, int base, bool locate, float target) {
    Aux *A = c.A;
    IN_SHARED(A);
    int L = (n + NT - 1) / NT;
    if ((L & 1) == 0) L += 1;
    p1_build(c, vals, n, L, (double)A->walk_s);
    if (c.tid == 0) {
        Walker w; w.s = A->walk_s; w.found = 0; w.at = -1; w.slow = A->walk_slow;
        p1_walk(c, vals, n, L, locate, target, w);
        A->walk_s = w.s; A->walk_slow = w.slow;
        if (w.found) { A->walk_found = 1; A->walk_idx = base + w.at; }
    }
    __syncthreads();
}

__device__ void p1_run(Ctx &c, const LView &lv, unsigned int *vals, bool locate, float target) {
    IN_SHARED(vals);
    Aux *A = c.A;
    IN_SHARED(A);
    __syncthreads();
    if (c.tid == 0) { A->walk_s = 0.0f; A->walk_found = 0; A->walk_idx = -1; }
    __syncthreads();
    if (lv.flat) {
        p1_block(c, ValKeys{lv.flat}, lv.n, 0, locate, target);
        return;
    }
    const int nblk = (lv.n + VBLK - 1) / VBLK;
    int b0 = 0, b1 = nblk;
    if (locate && nblk <= MAX_VBLK) {
        // the block whose end value is the first to exceed the target (sums remembered by the last full run)
        b0 = nblk;
        for (int b = 0; b < nblk; b++)
            if (target < A->blk_s[b + 1]) { b0 = b; break; }
        if (b0 == nblk) return;  // never exceeded
        b1 = b0 + 1;
        __syncthreads();
        if (c.tid == 0) A->walk_s = A->blk_s[b0];
        __syncthreads();
    }
    for (int b = b0; b < b1; b++) {
        const int n = min(VBLK, lv.n - b * VBLK);
        __syncthreads();
        if (!locate && c.tid == 0 && b < MAX_VBLK) A->blk_s[b] = A->walk_s;
        {
            const int o = b * VBLK;
            lv.for_range(c.tid, o, o + n, [&](int v, unsigned long long k) { vals[v - o] = (unsigned int)(k >> 32); });
        }
        __syncthreads();
        if (locate && A->walk_found) break;
        p1_block(c, ValBits{vals}, n, b * VBLK, locate, target);
    }
    if (!locate && c.tid == 0 && nblk <= MAX_VBLK) A->blk_s[nblk] = A->walk_s;
    __syncthreads();
}


// =============================================================================
// The descending walk past the sorted head (sample.mojo:492-506 and :580-590 on rows
// whose nucleus is larger than the head), over the row's relevant list. State: exact
// running sum `s`, elements consumed `pos`, and `tau`: everything with exp bits >= tau
// is consumed. Each phase histograms what remains by value bin with its integer
// contribution in the current binade, consumes whole bins up to the first bin holding
// an event (the sum reaching x_ge, exceeding x_gt, leaving the binade, a count limit,
// or an element needing sequential care), then gathers that bin, sorts it and adds it
// element by element.
// =============================================================================
struct Walk {
    float s; long long pos; unsigned int tau;
    int event; int idx; float p; int tie;
};

// index in list order of the (nth+1)-th entry whose exp bits equal `eb` and lie below `tau`
__device__ int nth_equal(Ctx &c, const LView &lv, unsigned int eb, unsigned int tau, int nth) {
    const int nl = lv.n;
    Aux *A = c.A;
    IN_SHARED(A);
    const int L = (nl + NT - 1) / NT;
    const int i0 = min(nl, c.tid * L), i1 = min(nl, (c.tid + 1) * L);
    int cnt = 0;
    for (int i = i0; i < i1; i++) cnt += ((unsigned int)(lv.at(i) >> 32) == eb && eb < tau) ? 1 : 0;
    int tot;
    const int ex = block_excl_scan<int>(cnt, A->wsi, &tot);
    __syncthreads();
    if (c.tid == 0) A->b_idx = -1;
    __syncthreads();
    if (nth >= ex && nth < ex + cnt) {
        int seen = ex;
        for (int i = i0; i < i1; i++) {
            const unsigned long long kk = lv.at(i);
            if ((unsigned int)(kk >> 32) == eb) {
                if (seen == nth) { A->b_idx = key_idx(kk); break; }
                seen++;
            }
        }
    }
    __syncthreads();
    return A->b_idx;
}

__device__ void descend(Ctx &c, const LView &lv, Walk &w, float x_ge, float x_gt,
                        long long nstop) {
    Aux *A = c.A;
    IN_SHARED(A);
    const bool counting = nstop >= 0;
    // Bins are 2048 ranges of exp bits. A bin holding more than the candidate buffer is split
    // again (level 2: the next 11 bits; level 3: single values); a single value repeated more
    // often than that is added one copy at a time.
    int lvl = 1;
    unsigned int lo = 0u;
    int shift = BIN_SHIFT;
    for (int phase = 0; phase < 8192; phase++) {
        __syncthreads();
        for (int i = c.tid; i < NBINS; i += NT) { A->u.h.hq[i] = 0u; A->u.h.hqh[i] = 0u; A->u.h.hc[i] = 0u; }
        if (c.tid == 0) { A->specbin = -1; A->ncand = 0; }
        __syncthreads();
        const bool have_s = w.s > 0.0f;
        const int j = have_s ? fexpo(w.s) : 0;
        const bool binade_ok = have_s && j >= -100 && j <= 100;
        const float Cm = __fmul_rn(1.5f, fpow2(j)), halfu = fpow2(j - 24), bigthr = fpow2(j - 1);
        const float inv_u = fpow2(23 - j);
        lv.for_each(c.tid, [&](int, unsigned long long key, unsigned long long *) {
            const unsigned int eb = (unsigned int)(key >> 32);
            if (eb >= w.tau || eb < lo) return;
            const int bin = (int)((eb - lo) >> shift);
            if (!binade_ok) { sred_add(&A->u.h.hc[bin], 1u); return; }
            const float p = __uint_as_float(eb);
            const float q = __fsub_rn(__fadd_rn(p, Cm), Cm);
            const float r = __fsub_rn(p, q);
            if (fabsf(r) == halfu || p >= bigthr) {
                sred_max(&A->specbin, bin);
                if (counting) sred_add(&A->u.h.hc[bin], 1u);
                return;
            }
            const unsigned int qu = __float2uint_rn(__fmul_rn(q, inv_u));
            if (qu) {  // two halves, so that neither counter can wrap and no atomic has to return a value
                sred_add(&A->u.h.hq[bin], qu & MASS_LO_MASK);
                if (qu >> MASS_SPLIT) sred_add(&A->u.h.hqh[bin], qu >> MASS_SPLIT);
            }
            if (counting) sred_add(&A->u.h.hc[bin], 1u);
        });
        __syncthreads();
        BinQuery qy;
        qy.specbin = A->specbin; qy.bin_hi = NBINS; qy.spec_bits = nullptr;
        qy.hq = A->u.h.hq; qy.hqh = A->u.h.hqh; qy.hc = A->u.h.hc;
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
            qy.pos0 = 0; qy.nstop = 1;  // nothing consumed yet: take the highest non-empty bin
        }
        find_event_bin(c, qy);
        const int hb = A->hit_bin;
        if (hb < 0) {
            // nothing left in this range triggers an event: consume it whole
            if (binade_ok) w.s = (float)((double)(qy.m0 + A->tot_q) * (double)fpow2(j - 23));
            w.pos += (long long)A->tot_c;
            if (lvl == 1) { w.tau = 0; w.event = EV_EXHAUSTED; return; }
            w.tau = lo; lvl = 1; lo = 0u; shift = BIN_SHIFT;  // back to the coarse bins below this range
            continue;
        }
        const unsigned long long qb = A->hit_qbefore, cb = A->hit_cbefore;
        const unsigned int blo = lo + ((unsigned int)hb << shift);
        const unsigned long long bhi64 = (unsigned long long)lo + ((unsigned long long)(hb + 1) << shift);
        const unsigned int bhi = bhi64 > 0xFFFFFFFFull ? 0xFFFFFFFFu : (unsigned int)bhi64;
        lv.for_each(c.tid, [&](int, unsigned long long key, unsigned long long *) {
            const unsigned int eb = (unsigned int)(key >> 32);
            if (eb < w.tau && eb >= blo && eb < bhi) {
                int pos = satom_add(&A->ncand, 1);
                if (pos < NC) A->cand[pos] = key;
            }
        });
        __syncthreads();
        const int nb = A->ncand;
        // what lies above the bin is consumed without an event either way
        const float s_bin = binade_ok ? (float)((double)(qy.m0 + qb) * (double)fpow2(j - 23)) : w.s;
        const long long pos_bin = w.pos + ((counting || !binade_ok) ? (long long)cb : 0);
        if (nb > NC && lvl < 3) {
            w.s = s_bin; w.pos = pos_bin;
            w.tau = bhi < w.tau ? bhi : w.tau;
            lo = blo; shift = (lvl == 1) ? BIN_SHIFT2 : 0; lvl++;
            c.status |= MOLLA_ROW_SLOW_PATH;
            continue;
        }
        if (nb > NC) {
            // one value, more copies than the buffer holds: add them one at a time (thread 0), then
            // find which copy, in token order, the event fell on
            c.status |= MOLLA_ROW_SLOW_PATH;
            const float pv = __uint_as_float(blo);
            __syncthreads();
            if (c.tid == 0) {
                float s = s_bin;
                long long pos = pos_bin;
                int ev = EV_NONE, at = -1;
                for (int i = 0; i < nb; i++) {
                    s = __fadd_rn(s, pv);
                    pos++;
                    if (s >= x_ge) ev = EV_CUT;
                    else if (x_gt < s) ev = EV_DRAW;
                    else if (counting && pos >= nstop) ev = EV_LIMIT;
                    if (ev != EV_NONE) { at = i; break; }
                }
                A->b_event = ev; A->b_s = s; A->b_pos = pos; A->b_aux = at;
            }
            __syncthreads();
            const int ev = A->b_event, at = A->b_aux;
            w.s = A->b_s; w.pos = A->b_pos;
            if (ev != EV_NONE) {
                const int id = nth_equal(c, lv, blo, w.tau, at);
                w.event = ev; w.idx = id; w.p = pv; w.tie = 1;
                return;
            }
            w.tau = blo;
            continue;
        }
        sort_cands(c, nb);
        walk_sorted(c, nb, s_bin, pos_bin, x_ge, x_gt, counting, nstop);
        if (c.tid == 0) A->b_tau = blo;
        __syncthreads();
        w.s = A->b_s; w.pos = A->b_pos; w.tau = A->b_tau;
        if (A->b_event != EV_NONE) { w.event = A->b_event; w.idx = A->b_idx; w.p = A->b_p; w.tie = A->b_aux; return; }
        if (phase > 8) c.status |= MOLLA_ROW_SLOW_PATH;
    }
    w.event = EV_DEGENERATE;
    c.status |= MOLLA_ROW_DEGENERATE;
}

// =============================================================================
// The same walk for long lists, which live in global memory: every pass over them costs
// tens of microseconds. The pass that turns the list's exponentials into probabilities
// also adds every entry's integer contribution to its value bin, in the units of
// MASS_SETS consecutive binades starting at the one the running sum is in after the head
// (`masses_add`). Those tables serve the cut walk and the draw walk alike (both run
// through the same prefix sums), so a walk costs one filtered pass per bin it has to
// look into: the bin where the sum leaves a binade, and the bin of the event itself.
// =============================================================================
// Value bins: 64 per binade over the 32 binades below 1 (probabilities further down share
// bin 0), so that even a flat row spreads over hundreds of bins.
constexpr int BK_SHIFT = 17;
constexpr int BK_BASE = (127 - 32) << 6;
__device__ __forceinline__ int bk_bin(unsigned int pbits) {
    const int b = (int)(pbits >> BK_SHIFT) - BK_BASE;
    return min(max(b, 0), NBINS - 1);
}
__device__ __forceinline__ unsigned int bk_lo(int bin) {  // smallest value bits of a bin
    return bin <= 0 ? 0u : (unsigned int)(bin + BK_BASE) << BK_SHIFT;
}

constexpr int MASS_SETS = 3;
constexpr int MASS_SET_WORDS = 2 * NBINS + NBINS / 32;  // low sums, high sums, care bits
constexpr int MASS_CK = 4;

struct MassTable {
    unsigned int *cnt;    // [NBINS] entries per bin (shared memory)
    unsigned int *sets;   // MASS_SETS x MASS_SET_WORDS (shared memory)
    int j0;               // set k is in the units of binade j0 + k
    unsigned int tau0;    // only entries with value bits below this are in the tables
    float Cm0, half0, big0;
};
// bins a walk consumed whole: the exact state before and after, for the walk that follows
struct MassCk {
    int n;
    int bin[MASS_CK]; float s_in[MASS_CK], s_out[MASS_CK]; long long pos_in[MASS_CK], pos_out[MASS_CK];
};

__device__ __forceinline__ void masses_begin(Ctx &c, MassTable &mt, int j0, unsigned int tau0) {
    __syncthreads();
    for (int i = c.tid; i < MASS_SETS * MASS_SET_WORDS; i += NT) mt.sets[i] = 0u;
    for (int i = c.tid; i < NBINS; i += NT) mt.cnt[i] = 0u;
    mt.j0 = j0; mt.tau0 = tau0;
    mt.Cm0 = __fmul_rn(1.5f, fpow2(j0)); mt.half0 = fpow2(j0 - 24); mt.big0 = fpow2(j0 - 1);
    __syncthreads();
}

// one entry's contribution to its bin in every set
__device__ __forceinline__ void masses_add(const MassTable &mt, unsigned int pb) {
    if (pb >= mt.tau0) return;
    const int bin = bk_bin(pb);
    sred_add(&mt.cnt[bin], 1u);
    const float v = __uint_as_float(pb);
#pragma unroll
    for (int k = 0; k < MASS_SETS; k++) {
        // v + 1.5 * 2^(j0+k) rounds v to the binade's unit; below 2^(j0+k-1) the rounded multiple
        // sits in the low 22 mantissa bits of that sum
        const float sc = (float)(1 << k);  // exact scalings
        const float Cm = __fmul_rn(mt.Cm0, sc);
        const float t = __fadd_rn(v, Cm);
        const float r = __fsub_rn(v, __fsub_rn(t, Cm));
        const unsigned int tb = __float_as_uint(t);
        unsigned int *set = mt.sets + k * MASS_SET_WORDS;
        if (fabsf(r) == __fmul_rn(mt.half0, sc) || v >= __fmul_rn(mt.big0, sc) || !(tb & 0x400000u)) {
            sred_or(&set[2 * NBINS + (bin >> 5)], 1u << (bin & 31));  // a rounding tie or a large term
        } else {
            const unsigned int q = tb & 0x3fffffu;
            if (q & MASS_LO_MASK) sred_add(&set[bin], q & MASS_LO_MASK);
            if (q >> MASS_SPLIT) sred_add(&set[NBINS + bin], q >> MASS_SPLIT);
        }
    }
}

// =============================================================================
// Help with long lists. The step is as long as its dearest row, and the dearest rows are the
// ones whose list is most of the vocabulary; they are handed out first, so when they reach
// the pass that turns their list into probabilities and bin masses, most other thread blocks
// have run out of rows. Those blocks then take segments of that pass: the owner publishes
// what the pass needs in its HelpSlot, owner and helpers claim segments with an atomic
// counter, a helper converts a segment in place (global memory, L1 bypassed on both sides),
// collects the segment's bin masses in its own shared memory and adds them into the owner's
// table in global memory. The owner never depends on a helper turning up: it claims segments
// itself until none are left and then waits, with a bound, for the ones still in other hands.
// =============================================================================
constexpr int HELP_MASS_WORDS = MASS_SETS * MASS_SET_WORDS + NBINS;    // the sets, then the bin counts
constexpr int HELP_TABLE_WORDS = HELP_MASS_WORDS + 2 * NC;             // ... then a candidate buffer of NC keys
constexpr int HELP_MIN_LIST = 24576;                                  // shorter lists are not worth publishing
struct __align__(256) HelpSlot {
    int open;            // 1 while segments can be claimed
    int claim;           // next segment to hand out
    int done;            // segments finished
    int nunits;
    float Z;
    unsigned int tau_bits;
    int mark_head;
    int j0;
    unsigned int tau0;
    int count[NWARP];    // entries in each segment
    int kind;            // 0: turn a segment into probabilities and bin masses; 1: collect one bin's entries
    int bin;             // kind 1: the bin
    int found;           // kind 1: entries the helpers have put into the owner's global candidate buffer
};

// One segment of a long list: exponentials to probabilities in place, and every entry's
// contribution into `mt` (this block's shared memory). All threads; 16-byte accesses that
// bypass L1 (the segment may have been written, or will be read, by another SM).
__device__ __forceinline__ void convert_segment(Ctx &c, unsigned long long *ks, int m, float Z, unsigned int tau_bits,
                                                bool mark_head, const MassTable &mt) {
    auto one = [&](unsigned long long kk) -> unsigned long long {
        unsigned int pb = __float_as_uint(__fdiv_rn(key_val(kk), Z));
        if (mark_head && (unsigned int)(kk >> 32) >= tau_bits) pb = 0xFFFFFFFFu;  // the head took it in pass B
        masses_add(mt, pb);
        return ((unsigned long long)pb << 32) | (kk & 0xFFFFFFFFull);
    };
    ulonglong2 *k2 = reinterpret_cast<ulonglong2 *>(ks);
    const int mp = m >> 1;
    for (int i = c.tid; i < mp; i += 8 * NT) {
        ulonglong2 k[8];
#pragma unroll
        for (int q = 0; q < 8; q++) k[q] = (i + q * NT < mp) ? __ldcg(k2 + i + q * NT) : make_ulonglong2(0ull, 0ull);
#pragma unroll
        for (int q = 0; q < 8; q++)
            if (i + q * NT < mp) { k[q].x = one(k[q].x); k[q].y = one(k[q].y); __stcg(k2 + i + q * NT, k[q]); }
    }
    if ((m & 1) && c.tid == 0) __stcg(ks + m - 1, one(__ldcg(ks + m - 1)));
}

// The owner's side: publish, work, wait, merge. Returns false if a helper did not report back
// within the bound (the row is then failed; its list may be half converted).
__device__ bool helped_convert(Ctx &c, const BatchArgs &a, unsigned long long *wl_seg, float Z, unsigned int tau_bits,
                               bool mark_head, const MassTable &mt) {
    Aux *A = c.A;
    IN_SHARED(A);
    HelpSlot *hs = static_cast<HelpSlot *>(a.help) + blockIdx.x;
    unsigned int *gt = a.help_tables + (size_t)blockIdx.x * HELP_TABLE_WORDS;
    __syncthreads();
    for (int i = c.tid; i < HELP_MASS_WORDS; i += NT) __stcg(gt + i, 0u);
    if (c.tid < NWARP) hs->count[c.tid] = A->woff[c.tid + 1] - A->woff[c.tid];
    if (c.tid == 0) {
        hs->Z = Z; hs->tau_bits = tau_bits; hs->mark_head = mark_head ? 1 : 0; hs->j0 = mt.j0; hs->tau0 = mt.tau0;
        hs->nunits = NWARP; hs->done = 0; hs->kind = 0;
    }
    __threadfence();
    __syncthreads();
    if (c.tid == 0) { atomicExch(&hs->claim, 0); __threadfence(); atomicExch(&hs->open, 1); }
    for (;;) {
        __syncthreads();
        if (c.tid == 0) A->evt_thread = atomicAdd(&hs->claim, 1);
        __syncthreads();
        const int u = A->evt_thread;
        if (u >= NWARP) break;
        convert_segment(c, wl_seg + (size_t)u * (size_t)a.R, A->woff[u + 1] - A->woff[u], Z, tau_bits, mark_head, mt);
        __threadfence();
        __syncthreads();
        if (c.tid == 0) atomicAdd(&hs->done, 1);
    }
    if (c.tid == 0) {
        int ok = 0;
        for (int spin = 0; spin < (1 << 22); spin++) {
            if (atomicAdd(&hs->done, 0) >= NWARP) { ok = 1; break; }
            __nanosleep(200);
        }
        atomicExch(&hs->open, 0);
        A->evt_thread = ok;
    }
    __syncthreads();
    const bool ok = A->evt_thread != 0;
    __threadfence();
    // what the helpers found: sums add, care bits and nothing else are or-ed
    for (int i = c.tid; i < HELP_MASS_WORDS; i += NT) {
        const unsigned int v = __ldcg(gt + i);
        if (!v) continue;
        if (i >= MASS_SETS * MASS_SET_WORDS) { mt.cnt[i - MASS_SETS * MASS_SET_WORDS] += v; continue; }
        const int k = i / MASS_SET_WORDS, j = i - k * MASS_SET_WORDS;
        unsigned int *set = mt.sets + k * MASS_SET_WORDS;
        if (j >= 2 * NBINS) set[j] |= v; else set[j] += v;
    }
    __syncthreads();
    return ok;
}

// The entries of one segment that lie in value bin `hb` (below tau0), handed to `sink`. All threads.
template <class S>
__device__ __forceinline__ void gather_segment(Ctx &c, const unsigned long long *ks, int m, unsigned int tau0, int hb, S sink) {
    const ulonglong2 *k2 = reinterpret_cast<const ulonglong2 *>(ks);
    const int mp = m >> 1;
    auto one = [&](unsigned long long kk) {
        const unsigned int pb = (unsigned int)(kk >> 32);
        if (pb < tau0 && bk_bin(pb) == hb) sink(kk);
    };
    for (int i = c.tid; i < mp; i += 8 * NT) {
        ulonglong2 k[8];
#pragma unroll
        for (int q = 0; q < 8; q++) k[q] = (i + q * NT < mp) ? __ldcg(k2 + i + q * NT) : make_ulonglong2(~0ull, ~0ull);
#pragma unroll
        for (int q = 0; q < 8; q++) { one(k[q].x); one(k[q].y); }
    }
    if ((m & 1) && c.tid == 0) one(__ldcg(ks + m - 1));
}

// The owner's side of a helped gather: the bin's entries end up in A->cand[0 .. A->ncand).
__device__ bool helped_gather(Ctx &c, const BatchArgs &a, const unsigned long long *wl_seg, unsigned int tau0, int hb) {
    Aux *A = c.A;
    IN_SHARED(A);
    HelpSlot *hs = static_cast<HelpSlot *>(a.help) + blockIdx.x;
    unsigned long long *gc = reinterpret_cast<unsigned long long *>(a.help_tables + (size_t)blockIdx.x * HELP_TABLE_WORDS + HELP_MASS_WORDS);
    __syncthreads();
    if (c.tid < NWARP) hs->count[c.tid] = A->woff[c.tid + 1] - A->woff[c.tid];
    if (c.tid == 0) { hs->tau0 = tau0; hs->bin = hb; hs->kind = 1; hs->found = 0; hs->nunits = NWARP; hs->done = 0; A->ncand = 0; }
    __threadfence();
    __syncthreads();
    if (c.tid == 0) { atomicExch(&hs->claim, 0); __threadfence(); atomicExch(&hs->open, 1); }
    for (;;) {
        __syncthreads();
        if (c.tid == 0) A->evt_thread = atomicAdd(&hs->claim, 1);
        __syncthreads();
        const int u = A->evt_thread;
        if (u >= NWARP) break;
        gather_segment(c, wl_seg + (size_t)u * (size_t)a.R, A->woff[u + 1] - A->woff[u], tau0, hb, [&](unsigned long long kk) {
            const int pos = satom_add(&A->ncand, 1);
            if (pos < NC) A->cand[pos] = kk;
        });
        __syncthreads();
        if (c.tid == 0) atomicAdd(&hs->done, 1);
    }
    if (c.tid == 0) {
        int ok = 0;
        for (int spin = 0; spin < (1 << 22); spin++) {
            if (atomicAdd(&hs->done, 0) >= NWARP) { ok = 1; break; }
            __nanosleep(100);
        }
        atomicExch(&hs->open, 0);
        A->evt_thread = ok;
    }
    __syncthreads();
    const bool ok = A->evt_thread != 0;
    __threadfence();
    const int ng = min(atomicAdd(&hs->found, 0), NC), n0 = A->ncand;
    __syncthreads();
    for (int i = c.tid; i < ng; i += NT)
        if (n0 + i < NC) A->cand[n0 + i] = __ldcg(gc + i);
    __syncthreads();
    if (c.tid == 0) A->ncand = n0 + ng;
    __syncthreads();
    return ok;
}

// A block with no rows left: look for a published pass and take segments of it, until every
// row of the launch is done.
__device__ void help_others(Ctx &c, const BatchArgs &a) {
    Aux *A = c.A;
    IN_SHARED(A);
    const int nslots = (int)gridDim.x;
    MassTable mt;
    mt.cnt = reinterpret_cast<unsigned int *>(A->hval);
    mt.sets = reinterpret_cast<unsigned int *>(c.stage);
    mt.j0 = 0; mt.tau0 = 0u; mt.Cm0 = mt.half0 = mt.big0 = 0.0f;
    if (c.tid == 0) A->ncand = ((int)blockIdx.x + 1) % nslots;  // the slot the scan starts from (shared by the block)
    for (int poll = 0; poll < (1 << 20); poll++) {
        __syncthreads();
        if (c.tid == 0) { A->evt_thread = 0x7fffffff; A->specbin = (*(volatile int *)a.rows_done >= a.B) ? 1 : 0; }
        __syncthreads();
        if (A->specbin) return;
        const int next = A->ncand;
        // every thread looks at one slot; the nearest open one after the slot served last is tried
        for (int sidx = c.tid; sidx < nslots; sidx += NT) {
            if (sidx == (int)blockIdx.x) continue;
            const volatile HelpSlot *hs = static_cast<HelpSlot *>(a.help) + sidx;
            if (hs->open == 1 && hs->claim < NWARP) atomicMin(&A->evt_thread, (sidx - next + nslots) % nslots);
        }
        __syncthreads();
        const int pick = A->evt_thread;
        __syncthreads();
        if (c.tid == 0) {
            int found = -1, unit = 0;
            if (pick != 0x7fffffff) {
                const int sidx = (pick + next) % nslots;
                unit = atomicAdd(&static_cast<HelpSlot *>(a.help)[sidx].claim, 1);
                if (unit < NWARP) { found = sidx; A->ncand = sidx; }
            } else {
                __nanosleep(100);
            }
            A->evt_thread = found; A->specbin = unit;
        }
        __syncthreads();
        const int sidx = A->evt_thread, u = A->specbin;
        if (sidx < 0) continue;
        HelpSlot *hs = static_cast<HelpSlot *>(a.help) + sidx;
        __threadfence();
        unsigned long long *seg = a.wlist + (size_t)sidx * 2 * NWARP * (size_t)a.R + (size_t)u * (size_t)a.R;
        if (__ldcg(&hs->kind) == 1) {
            unsigned long long *gc = reinterpret_cast<unsigned long long *>(a.help_tables + (size_t)sidx * HELP_TABLE_WORDS + HELP_MASS_WORDS);
            gather_segment(c, seg, __ldcg(&hs->count[u]), __ldcg(&hs->tau0), __ldcg(&hs->bin), [&](unsigned long long kk) {
                const int pos = atomicAdd(&hs->found, 1);
                if (pos < NC) __stcg(gc + pos, kk);
            });
            __threadfence();
            __syncthreads();
            if (c.tid == 0) atomicAdd(&hs->done, 1);
            continue;
        }
        const float Z = __ldcg(&hs->Z);
        const unsigned int tau_bits = __ldcg(&hs->tau_bits);
        const bool mark_head = __ldcg(&hs->mark_head) != 0;
        const int m = __ldcg(&hs->count[u]);
        masses_begin(c, mt, __ldcg(&hs->j0), __ldcg(&hs->tau0));
        convert_segment(c, seg, m, Z, tau_bits, mark_head, mt);
        __syncthreads();
        unsigned int *gt = a.help_tables + (size_t)sidx * HELP_TABLE_WORDS;
        for (int i = c.tid; i < HELP_MASS_WORDS; i += NT) {
            unsigned int v;
            if (i >= MASS_SETS * MASS_SET_WORDS) v = mt.cnt[i - MASS_SETS * MASS_SET_WORDS];
            else v = mt.sets[i];
            if (!v) continue;
            const int j = i % MASS_SET_WORDS;
            if (i < MASS_SETS * MASS_SET_WORDS && j >= 2 * NBINS) atomicOr(gt + i, v); else atomicAdd(gt + i, v);
        }
        __threadfence();
        __syncthreads();
        if (c.tid == 0) atomicAdd(&hs->done, 1);
    }
}

// Returns false if it met something it leaves to the general walk (a running sum outside the
// tables' binades, or a bin larger than the candidate buffer); `w` then holds the exact state
// to continue from.
__device__ bool descend_masses(Ctx &c, const BatchArgs &a, bool helped, const LView &lv, const MassTable &mt, MassCk &ck, Walk &w, int &hi, float x_ge, float x_gt,
                               long long nstop) {
    Aux *A = c.A;
    IN_SHARED(A);
    const bool counting = nstop >= 0;
    for (int phase = 0; phase < 8192; phase++) {
        if (hi <= 0) { w.tau = 0; w.event = EV_EXHAUSTED; return true; }
        if (!(w.s > 0.0f)) return false;
        const int j = fexpo(w.s);
        if (j < mt.j0 || j >= mt.j0 + MASS_SETS || j < -100 || j > 100) return false;
        const float inv_u = fpow2(23 - j);
        const unsigned int *set = mt.sets + (j - mt.j0) * MASS_SET_WORDS;
        BinQuery qy;
        qy.specbin = -1; qy.bin_hi = hi; qy.spec_bits = set + 2 * NBINS;
        qy.hq = set; qy.hqh = set + NBINS; qy.hc = mt.cnt;
        qy.pos0 = (unsigned long long)w.pos;
        qy.nstop = counting ? (unsigned long long)nstop : ~0ull;
        qy.m0 = (unsigned long long)((double)w.s * (double)inv_u);
        unsigned long long xq = 1ull << 24;
        if (x_ge < 3.0e38f) { double t = ceil((double)x_ge * (double)inv_u); if (t < (double)xq) xq = (t <= 0.0) ? 0ull : (unsigned long long)t; }
        if (x_gt < 3.0e38f) { double t = floor((double)x_gt * (double)inv_u) + 1.0; if (t < (double)xq) xq = (t <= 0.0) ? 0ull : (unsigned long long)t; }
        qy.xq = xq;
        find_event_bin(c, qy);
        const int hb = A->hit_bin;
        if (hb < 0) {
            w.s = (float)((double)(qy.m0 + A->tot_q) * (double)fpow2(j - 23));
            w.pos += (long long)A->tot_c;
            w.tau = 0; hi = 0;
            w.event = EV_EXHAUSTED;
            return true;
        }
        const unsigned long long qb = A->hit_qbefore, cb = A->hit_cbefore;
        const float s_bin = (float)((double)(qy.m0 + qb) * (double)fpow2(j - 23));
        const long long pos_bin = w.pos + (long long)cb;
        const int nb = (int)mt.cnt[hb];
        if (nb > NC) {  // a crowded bin: the general walk splits it further
            w.s = s_bin; w.pos = pos_bin; w.tau = min(bk_lo(hb + 1), mt.tau0); hi = hb + 1;
            return false;
        }
        // a bin an earlier walk went through whole, from the same state: if this walk's event does
        // not fall inside it either (prefix sums only grow), take the state behind it
        bool skipped = false;
        for (int q = 0; q < ck.n; q++) {
            if (ck.bin[q] == hb && ck.s_in[q] == s_bin && ck.pos_in[q] == pos_bin && !(ck.s_out[q] >= x_ge) &&
                !(x_gt < ck.s_out[q]) && !(counting && ck.pos_out[q] >= nstop)) {
                w.s = ck.s_out[q]; w.pos = ck.pos_out[q]; w.tau = bk_lo(hb); hi = hb;
                skipped = true;
                break;
            }
        }
        if (skipped) continue;
        __syncthreads();
        if (c.tid == 0) A->ncand = 0;
        __syncthreads();
        const unsigned int tau0 = mt.tau0;
        if (helped) {
            if (!helped_gather(c, a, lv.seg, tau0, hb)) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
        } else
        lv.for_each(c.tid, [&](int, unsigned long long key, unsigned long long *) {
            const unsigned int pb = (unsigned int)(key >> 32);
            if (pb < tau0 && bk_bin(pb) == hb) {
                const int pos = satom_add(&A->ncand, 1);
                if (pos < NC) A->cand[pos] = key;
            }
        });
        __syncthreads();
        sort_cands(c, nb);
        walk_sorted(c, nb, s_bin, pos_bin, x_ge, x_gt, counting, nstop);
        w.s = A->b_s; w.pos = A->b_pos; w.tau = bk_lo(hb); hi = hb;
        if (A->b_event != EV_NONE) { w.event = A->b_event; w.idx = A->b_idx; w.p = A->b_p; w.tie = A->b_aux; return true; }
        if (ck.n < MASS_CK) {
            const int q = ck.n++;
            ck.bin[q] = hb; ck.s_in[q] = s_bin; ck.pos_in[q] = pos_bin; ck.s_out[q] = w.s; ck.pos_out[q] = w.pos;
        }
    }
    return false;
}


// Between the two all-gathers of the vocab-sharded form: one thread per row folds the shards'
// stage-1 summaries into what stage 2 needs (the global maximum, the head threshold, a bound on
// the softmax sum before this shard's columns) and answers the rows that need nothing more.
__global__ void shard_merge_kernel(int B, int Vg, int world, int rank, const float *temperature, const int *top_k,
                                   const float *gathered /*[world][B][SA_WORDS]*/, float *global4, int *tokens,
                                   unsigned int *status) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= B) return;
    const float T = temperature ? temperature[r] : 0.0f;
    const int k = top_k ? top_k[r] : 0;
    float xmax = -INFINITY; int imax = 0, eq = 0;
    for (int w = 0; w < world; w++) {
        const float *s = gathered + ((long long)w * B + r) * SA_WORDS;
        if (s[0] > xmax) { xmax = s[0]; imax = __float_as_int(s[1]); eq = __float_as_int(s[2]); }
        else if (s[0] == xmax) eq += __float_as_int(s[2]);
    }
    const bool greedy = !(T > 0.0f);
    const long long n_lim = (k > 0 && k < Vg) ? (long long)k : (long long)Vg;
    long long need = n_lim + 1;
    if (need > HEAD_NEED) need = HEAD_NEED;
    if (need > Vg) need = Vg;
    // the need-th largest of the union of the shards' sorted lists (a merge by one thread)
    int ptr[16];
    for (int w = 0; w < 16; w++) ptr[w] = 0;
    float tau = -INFINITY;
    for (long long step = 0; step < need; step++) {
        float best = -INFINITY; int bw = -1;
        for (int w = 0; w < world; w++) {
            if (ptr[w] >= HEAD_NEED) continue;
            const float v = gathered[((long long)w * B + r) * SA_WORDS + 3 + NWARP + ptr[w]];
            if (bw < 0 || v > best) { best = v; bw = w; }
        }
        if (bw < 0) { tau = -INFINITY; break; }
        tau = best; ptr[bw]++;
    }
    float lb = 0.0f;
    if (!greedy) {
        const float top = (T == 1.0f) ? xmax : __fdiv_rn(xmax, T);
        for (int w = 0; w < rank; w++)
            for (int q = 0; q < NWARP; q++) {
                const float m = gathered[((long long)w * B + r) * SA_WORDS + 3 + q];
                const float v = (T == 1.0f) ? m : __fdiv_rn(m, T);
                lb += expf_pinned(__fsub_rn(v, top));
            }
    }
    global4[4 * r] = xmax; global4[4 * r + 1] = tau; global4[4 * r + 2] = lb; global4[4 * r + 3] = __int_as_float(imax);
    if ((greedy || n_lim == 1) && tokens && status && xmax > -INFINITY) {
        tokens[r] = imax;
        status[r] = (!greedy && eq > 1) ? MOLLA_ROW_TOPK_TIE : 0u;
    }
}

// Rows differ in cost by an order of magnitude (a greedy row is one pass, a hot row keeps
// most of its vocabulary). Handing out the dearest first keeps the last CTAs from running
// long: this small kernel sorts the rows by a cost estimate.
__global__ void __launch_bounds__(NT, 1) order_rows_kernel(const float *temperature, const int *top_k, const int *slot, int B, int *order) {
    __shared__ unsigned long long keys[ORDER_CAP];
    int n2 = 2;
    while (n2 < B) n2 <<= 1;
    for (int i = threadIdx.x; i < n2; i += NT) {
        float cost = -1.0f;
        if (i < B) {
            const int q = slot ? slot[i] : i;
            const float T = temperature ? temperature[q] : 0.0f;
            const int k = top_k ? top_k[q] : 0;
            cost = (T > 0.0f && k != 1) ? T + ((k == 0 || k >= HEAD_NEED) ? 0.25f : 0.0f) : 0.0f;
        }
        keys[i] = ((unsigned long long)fkey(cost) << 32) | (unsigned long long)(0xFFFFu - (unsigned int)(i & 0xFFFF));
    }
    bitonic_desc(keys, n2, threadIdx.x);
    for (int i = threadIdx.x; i < B; i += NT) order[i] = (int)(0xFFFFu - (unsigned int)(keys[i] & 0xFFFFull));
}

// =============================================================================
// The kernel: persistent CTAs, each taking the next row (dearest rows first).
// =============================================================================
__global__ void __launch_bounds__(NT, 1) sample_rows_kernel(const __grid_constant__ BatchArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Ctx c;
    c.tid = threadIdx.x; c.lane = c.tid & 31; c.warp = c.tid >> 5;
    c.stage = reinterpret_cast<float *>(smem_raw);
    c.A = reinterpret_cast<Aux *>(smem_raw + STAGE_FLOATS * 4);
    c.bm = reinterpret_cast<unsigned int *>(smem_raw + STAGE_FLOATS * 4 + ((sizeof(Aux) + 15) / 16) * 16);
    c.V = a.V; c.R = a.R;
    c.parbits = 0;
    Aux *A = c.A;
    IN_SHARED(A);
    if (c.lane == 0) {
        for (int s = 0; s < NSTAGE; s++) mbar_init(&A->mbar[c.warp][s], 1);
        fence_proxy_async();
    }
    __syncthreads();
    {   // this warp's sixteenth of every row
        long long beg = (long long)c.warp * a.R;
        long long len = (long long)a.V - beg;
        c.rbeg = (int)(beg < a.V ? beg : a.V);
        c.rlen = (int)(len < 0 ? 0 : (len > a.R ? a.R : len));
        c.npieces = (c.rlen + PIECE - 1) / PIECE;
    }
    unsigned long long *wl_seg = a.wlist + (size_t)blockIdx.x * 2 * NWARP * (size_t)a.R;   // per-warp segments
    unsigned long long *wl_flat = wl_seg + (size_t)NWARP * (size_t)a.R;                   // contiguous copy
    unsigned long long *slist = reinterpret_cast<unsigned long long *>(c.stage);           // list in shared memory
    const int nwords = (a.V + 31) >> 5;
    const uint64_t keep_policy = MOLLA_KNOB(a, 4) ? l2_normal_policy() : l2_keep_policy();

    bool had_row = false;
    for (;;) {
        __syncthreads();
        if (c.tid == 0) {
            if (had_row && a.rows_done) { __threadfence(); atomicAdd(a.rows_done, 1); }
            int t = atomicAdd(a.row_counter, 1);
            if (a.order && t < a.B) t = a.order[t];
            A->cur_row = t;
        }
        __syncthreads();
        const int r = A->cur_row;
        if (r >= a.B) break;
        had_row = true;
        c.status = 0; c.last_read = false;
        const int q = a.slot ? a.slot[r] : r;  // where this row's settings and state live
        {   // a stale row or slot index: nothing of that row or slot is touched
            const long long lrow = a.rows ? (long long)a.rows[r] : (long long)r;
            const bool idx_ok = (!a.slot || (q >= 0 && (a.n_slots <= 0 || q < a.n_slots))) &&
                                (!a.rows || (lrow >= 0 && (a.n_logit_rows <= 0 || lrow < a.n_logit_rows)));
            if (!idx_ok) {
                if (c.tid == 0 && !a.penalised_only && a.tokens) { a.tokens[r] = -1; a.row_status[r] = MOLLA_ROW_INVALID_CONFIG; }
                continue;
            }
        }
        const float T = a.temperature ? a.temperature[q] : 0.0f;
        const int k = a.top_k ? a.top_k[q] : 0;
        const float P = a.top_p ? a.top_p[q] : 1.0f;
        const float minp = a.min_p ? a.min_p[q] : 0.0f;
        const float typ = a.typical_p ? a.typical_p[q] : 1.0f;
        const float rp = a.repeat_penalty ? a.repeat_penalty[q] : 1.0f;
        const float fp = a.frequency_penalty ? a.frequency_penalty[q] : 0.0f;
        const float pp = a.presence_penalty ? a.presence_penalty[q] : 0.0f;
        const int ring_n = a.ring ? min(max(a.ring_len[q], 0), a.ring_cap) : 0;
        const bool won = a.ring ? (ring_n > 0) : (a.window_on ? (a.window_on[q] != 0) : true);
        const int h0 = (a.hist && a.hist_off) ? a.hist_off[q] : 0;
        // a window kept on the device fills from its first slot (sample.mojo:246-258): the first
        // `filled` entries are the window, whatever the head is
        const long long *histp = a.ring ? a.ring + (size_t)q * (size_t)a.ring_cap : (a.hist ? a.hist + h0 : nullptr);
        const int H = a.ring ? min(max(a.ring_filled[q], 0), ring_n) : ((a.hist && a.hist_off) ? (a.hist_off[q + 1] - h0) : 0);
        const int b0 = (a.bias_ids && a.bias_off) ? a.bias_off[q] : 0;
        const int nb = (a.bias_ids && a.bias_off) ? (a.bias_off[q + 1] - b0) : 0;
        // the rules of SamplerConfig.check (sample.mojo:140-154); NaN fails every test
        const bool valid = (T >= 0.0f) && (k >= 0) && (P > 0.0f && P <= 1.0f) && (minp >= 0.0f && minp <= 1.0f) &&
                           (typ > 0.0f && typ <= 1.0f) && (rp > 0.0f) && H >= 0 && nb >= 0;
        const bool greedy = !(T > 0.0f);
        const bool penalizing = won && H > 0 && (rp != 1.0f || fp != 0.0f || pp != 0.0f);
        const int npatch = (a.mode == 3) ? 0 : (penalizing ? H : 0) + nb;
        if (!a.penalised_only) {
            if (!valid) c.status |= MOLLA_ROW_INVALID_CONFIG;
            // typical-p is done on rows an earlier filter sorted and cut to a set inside the sorted head
            else if (!greedy && typ < 1.0f && !((k > 0 && k < a.Vg) || P < 1.0f)) c.status |= MOLLA_ROW_UNSUPPORTED;
        }
        if (npatch > PATCH_MAX) c.status |= MOLLA_ROW_UNSUPPORTED;
        if (c.status) {
            if (a.mode == 1 && c.tid == 0) { float *o = a.sa_out + (long long)r * SA_WORDS; o[0] = -INFINITY; o[1] = __int_as_float(0); o[2] = __int_as_float(0); }
            if (a.mode == 2 && c.tid == 0) a.sb_count[r] = 0;
            if (c.tid == 0 && !a.penalised_only && a.tokens) {
                a.tokens[r] = -1; a.row_status[r] = c.status;
                if (a.diag) { a.diag[4 * r] = a.diag[4 * r + 1] = a.diag[4 * r + 2] = a.diag[4 * r + 3] = 0.0f; }
            }
            continue;
        }
        c.src = a.logits + (long long)(a.rows ? a.rows[r] : r) * a.row_stride;
        c.softcap = a.softcap;
        c.aligned = ((reinterpret_cast<uintptr_t>(c.src) & 15u) == 0);

        // ---- 1. logit bias and penalties (sample.mojo:381-417) touch at most a window's worth of
        // tokens: their new values go into a hash, a bitmap over the vocabulary marks them.
        c.patching = false;
        if (npatch > 0) {
            for (int i = c.tid; i < nwords; i += NT) c.bm[i] = 0u;
            for (int i = c.tid; i < HSLOTS; i += NT) { A->hkey[i] = -1; A->hcnt[i] = 0; }
            __syncthreads();
            for (int i = c.tid; i < npatch; i += NT) {
                const bool is_bias = i < nb;
                const long long t64 = (is_bias ? a.bias_ids[b0 + i] : histp[i - nb]) - a.col0;
                if (t64 < 0 || t64 >= a.V) continue;
                const int tok = (int)t64;
                int s = hslot(tok);
                for (int probe = 0; probe < HSLOTS; probe++) {
                    const int old = atomicCAS(&A->hkey[s], -1, tok);
                    if (old == -1 || old == tok) { if (!is_bias) atomicAdd(&A->hcnt[s], 1); break; }
                    s = (s + 1) & (HSLOTS - 1);
                }
            }
            __syncthreads();
            for (int s = c.tid; s < HSLOTS; s += NT) {
                const int tok = A->hkey[s];
                if (tok < 0) continue;
                float v = __ldg(c.src + tok);
                if (c.softcap > 0.0f) v = softcap_pinned(v, c.softcap);
                for (int bq = 0; bq < nb; bq++)  // duplicates add up, in the order they were given
                    if (a.bias_ids[b0 + bq] == (long long)tok + a.col0) v = __fadd_rn(v, a.bias_vals[b0 + bq]);
                const int n = A->hcnt[s];
                if (n > 0) {
                    if (v > 0.0f) v = __fdiv_rn(v, rp);
                    else v = __fmul_rn(v, rp);
                    v = __fsub_rn(v, __fmul_rn((float)n, fp));
                    v = __fsub_rn(v, pp);
                }
                A->hval[s] = v;
                atomicOr(&c.bm[tok >> 5], 1u << (tok & 31));
            }
            __syncthreads();
            c.patching = true;
        }

        if (a.penalised) {
            float *dst = a.penalised + (long long)r * a.V;
            pieces_begin(c);
            for (int p = 0; p < c.npieces; p++) {
                int n;
                const float *slot = piece_acquire(c, p, n);
                const int g0 = c.rbeg + p * PIECE + c.lane * LT;
                float x[LT];
                load_chunk(c, slot, n, g0, x);
#pragma unroll
                for (int j = 0; j < LT; j++)
                    if (c.lane * LT + j < n) dst[g0 + j] = x[j];
            }
            if (a.penalised_only) continue;
        }

        // ---- 2. pass A (HBM): the maximum and its first index (kernel.mojo:571-585, sample.mojo:342-346)
        float tmax = -INFINITY;
        int tidx = 0x7fffffff, teq = 0;
        if (a.mode != 3) {
            float rmx = -INFINITY;
            pieces_begin(c);
            for (int p = 0; p < c.npieces; p++) {
                int n;
                const float *slot = piece_acquire(c, p, n);
                const int g0 = c.rbeg + p * PIECE + c.lane * LT;
                float x[LT];
                load_chunk(c, slot, n, g0, x);
                // the chunk's maximum first (a short tree); only a chunk that reaches the running
                // maximum, which is rare after the first few pieces, is looked at element by element
                float cm;
                {
                    float m[LT];
#pragma unroll
                    for (int j = 0; j < LT; j++) m[j] = x[j];
#pragma unroll
                    for (int w = 1; w < LT; w <<= 1)
#pragma unroll
                        for (int j = 0; j + w < LT; j += 2 * w) m[j] = fmaxf(m[j], m[j + w]);
                    cm = m[0];
                }
                if (cm >= tmax) {
                    if (cm > tmax) { tmax = cm; teq = 0; tidx = 0x7fffffff; }
#pragma unroll
                    for (int j = 0; j < LT; j++) {
                        if (x[j] == tmax && c.lane * LT + j < n) {
                            if (tidx == 0x7fffffff) tidx = g0 + j + a.col0;
                            teq++;
                        }
                    }
                }
                if (!greedy || a.mode == 1) {
                    cm = fkey_inv(__reduce_max_sync(0xffffffffu, fkey(cm)));
                    if (c.lane == 0) A->u.s.pmax[c.warp][p] = cm;
                    rmx = fmaxf(rmx, cm);
                }
            }
            if ((!greedy || a.mode == 1) && c.lane == 0) A->u.s.rmax[c.warp] = rmx;
        }
        float xmax = tmax;
        int imax = tidx;
        if (a.mode != 3) block_argmax(c, xmax, imax);
        if (imax == 0x7fffffff) imax = 0;
        if (a.mode == 1) {
            // stage 1 of the sharded form: what the other shards need to know about this slice
            int tot;
            (void)block_excl_scan<int>((tmax == xmax) ? teq : 0, A->wsi, &tot);
            float *o = a.sa_out + (long long)r * SA_WORDS;
            __syncthreads();
            A->cand[c.tid] = ((unsigned long long)fkey(tmax) << 32) | (unsigned long long)c.tid;
            bitonic_desc(A->cand, NT, c.tid);
            if (c.tid < HEAD_NEED) o[3 + NWARP + c.tid] = fkey_inv((unsigned int)(A->cand[c.tid] >> 32));
            if (c.tid < NWARP) o[3 + c.tid] = A->u.s.rmax[c.tid];
            if (c.tid == 0) { o[0] = xmax; o[1] = __int_as_float(imax); o[2] = __int_as_float(tot); o[SA_WORDS - 1] = 0.0f; }
            continue;
        }
        if (a.mode >= 2) { xmax = a.sb_in[4 * r]; imax = __float_as_int(a.sb_in[4 * r + 3]); }
        const long long n_lim = (k > 0 && k < a.Vg) ? (long long)k : (long long)a.Vg;
        if (a.mode >= 2 && (greedy || n_lim == 1)) {  // the first all-gather already answered these rows
            if (a.mode == 2 && c.tid == 0) a.sb_count[r] = 0;
            continue;
        }
        int token = -1;
        float dZ = 0.0f, dsum = 0.0f, dtarget = 0.0f, dp = 0.0f;

        if (greedy) {
            token = imax;
        } else if (n_lim == 1) {
            // top-k of one: the sort's first element is a maximum (sample.mojo:485-490)
            int tot;
            (void)block_excl_scan<int>((tmax == xmax) ? teq : 0, A->wsi, &tot);
            if (tot > 1) c.status |= MOLLA_ROW_TOPK_TIE;
            token = imax;
        } else {
            const float top = (T == 1.0f) ? xmax : __fdiv_rn(xmax, T);
            const bool topp_on = (P < 1.0f) && (n_lim > 1);
            const bool pure = !topp_on && n_lim == (long long)a.Vg;
            const float u01 = draw01(a.seed ? a.seed[q] : 0ull, a.drawn ? a.drawn[q] : 0ull);
            const bool filter_ok = fabsf(top) < 1.0e5f;
            long long need = n_lim + 1;
            if (need > HEAD_NEED) need = HEAD_NEED;
            if (need > a.Vg) need = a.Vg;
            const bool p3row = !pure && (n_lim + 1 > HEAD_NEED);

            // The head of the sorted order holds the `need` largest. The need-th largest of the threads'
            // own maxima bounds the need-th largest element from below, so everything at or above it is
            // kept for the head whether or not it can matter to a sum.
            float tau_x = INFINITY;
            unsigned int tau_bits = 1u;
            if (!pure) {
                __syncthreads();
                if (a.mode >= 2) {
                    tau_x = a.sb_in[4 * r + 1];
                } else {
                    A->cand[c.tid] = ((unsigned long long)fkey(tmax) << 32) | (unsigned long long)c.tid;
                    bitonic_desc(A->cand, NT, c.tid);
                    tau_x = fkey_inv((unsigned int)(A->cand[need - 1] >> 32));
                }
                const float tv = (T == 1.0f) ? tau_x : __fdiv_rn(tau_x, T);
                const unsigned int tb_ = __float_as_uint(expf_pinned(__fsub_rn(tv, top)));
                tau_bits = tb_ > 1u ? tb_ : 1u;
                __syncthreads();
            }

            // ---- 3. pass B (L2): keep what can matter, in vocabulary order, with its exponential
            // (temperature and softmax numerator, sample.mojo:419-434)
            // A lower bound on the running sum at every piece: each earlier piece adds at least the
            // exponential of its own maximum. What is below half an ulp of that bound is dropped.
            const bool head_in_pass = (a.mode == 0) && !pure;  // the head's candidates are picked up on the way
            if (c.tid == 0) A->ncand = 0;
            if (a.mode != 3) {
            {
                const int maxp = (a.R + PIECE - 1) / PIECE;
                for (int idx = c.tid; idx < NWARP * maxp; idx += NT) {
                    const int w = idx / maxp, p = idx - w * maxp;
                    long long rl = (long long)a.V - (long long)w * a.R;
                    const int rlen = (int)(rl < 0 ? 0 : (rl > a.R ? a.R : rl));
                    if (p * PIECE < rlen) {
                        const float x = A->u.s.pmax[w][p];
                        const float v = (T == 1.0f) ? x : __fdiv_rn(x, T);
                        A->u.s.pmax[w][p] = expf_pinned(__fsub_rn(v, top));
                    }
                }
                __syncthreads();
                float rs = 0.0f;
                for (int p = c.lane; p < c.npieces; p += 32) rs += A->u.s.pmax[c.warp][p];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) rs += __shfl_xor_sync(0xffffffffu, rs, o);
                if (c.lane == 0) A->u.s.rmax[c.warp] = rs;
                __syncthreads();
            }
            float lb = (a.mode == 2) ? a.sb_in[4 * r + 2] : 0.0f;  // bound on the sum of everything before this warp's current piece
            for (int w = 0; w < c.warp; w++) lb += A->u.s.rmax[w];
            int base = 0;
            unsigned long long *myseg = wl_seg + (size_t)c.warp * (size_t)a.R;
            c.last_read = !MOLLA_KNOB(a, 2);
            pieces_begin(c);
            for (int p = 0; p < c.npieces; p++) {
                int n;
                float *slot = const_cast<float *>(piece_acquire(c, p, n));
                const int g0 = c.rbeg + p * PIECE + c.lane * LT;
                float x[LT];
                load_chunk(c, slot, n, g0, x);
                // below top - 105 the exponential is exactly zero whatever came before
                const float thr_rel = (filter_ok && lb > 0.0f) ? T * (top + logf(0.9f * lb) - REL_MARGIN) : -INFINITY;
                const float thr_zero = filter_ok ? T * (top - 105.0f) : -INFINITY;
                const float thr = fminf(fmaxf(thr_rel, thr_zero), tau_x);
                int cnt = 0;
#pragma unroll
                for (int j = 0; j < LT; j++) cnt += (c.lane * LT + j < n && x[j] >= thr) ? 1 : 0;
                const int incl = warp_incl_scan(cnt, c.lane);
                const int total = __shfl_sync(0xffffffffu, incl, 31);
                int off = incl - cnt;
                __syncwarp();  // every lane has its elements in registers: compact in place
#pragma unroll
                for (int j = 0; j < LT; j++) {
                    if (c.lane * LT + j < n && x[j] >= thr) {
                        slot[off] = x[j];
                        A->u.s.ppos[c.warp][off] = (unsigned short)(c.lane * LT + j);
                        off++;
                    }
                }
                __syncwarp();
                {
                    const int gbase = a.col0 + c.rbeg + p * PIECE;
                    auto value = [&](int i) -> float {
                        const float xx = slot[i];
                        const float v = (T == 1.0f) ? xx : __fdiv_rn(xx, T);
                        return expf_pinned(__fsub_rn(v, top));
                    };
                    auto emit = [&](int i, float e) {
                        const unsigned long long key = make_key(__float_as_uint(e), gbase + (int)A->u.s.ppos[c.warp][i]);
                        stg_keep(myseg + base + i, key, keep_policy);
                        if (head_in_pass && __float_as_uint(e) >= tau_bits) {
                            const int pos = satom_add(&A->ncand, 1);
                            if (pos < HEADC) A->cand[pos] = key;
                        }
                    };
                    int i = c.lane;
                    for (; i + 96 < total; i += 128) {  // four independent evaluations in flight
                        const float e0 = value(i), e1 = value(i + 32), e2 = value(i + 64), e3 = value(i + 96);
                        emit(i, e0); emit(i + 32, e1); emit(i + 64, e2); emit(i + 96, e3);
                    }
                    for (; i < total; i += 32) emit(i, value(i));
                }
                base += total;
                lb += A->u.s.pmax[c.warp][p];
            }

            if (c.lane == 0) A->wcnt[c.warp] = base;
            } else if (c.tid < NWARP) {
                // stage 3: the segments are the shards' lists, already in vocabulary order
                int n = (c.tid < a.world) ? a.sc_count[(long long)c.tid * a.B + r] : 0;
                A->wcnt[c.tid] = n < 0 ? 0 : (n > a.list_cap ? a.list_cap : n);
            }
            __syncthreads();
            // offsets of the warps' segments in the whole list
            if (c.tid == 0) {
                int o = 0;
                for (int w = 0; w < NWARP; w++) { A->woff[w] = o; o += A->wcnt[w]; }
                A->woff[NWARP] = o;
            }
            __syncthreads();
            const int nl = A->woff[NWARP];
            {
                // gather the warps' segments into one array: shared memory if it fits, else global
                unsigned long long *dstl = (nl <= SLIST_CAP) ? slist : wl_flat;
                if (a.mode == 2) dstl = a.sb_list + (long long)r * a.list_cap;  // the slice's list goes to the all-gather
                // a long list of the ordinary form stays where pass B wrote it (the view walks the segments)
                const bool stays = (a.mode == 0 && nl > SLIST_CAP);
                const int nmove = (stays || (a.mode == 2 && nl > a.list_cap)) ? 0 : nl;
                auto fetch = [&](int v) -> unsigned long long {
                    int w = 0;
#pragma unroll
                    for (int q = 1; q < NWARP; q++) w += (v >= A->woff[q]) ? 1 : 0;
                    if (a.mode == 3) return a.sc_list[((size_t)w * a.B + r) * (size_t)a.list_cap + (size_t)(v - A->woff[w])];
                    return wl_seg[(size_t)w * (size_t)a.R + (size_t)(v - A->woff[w])];
                };
                int i = c.tid;
                for (; i + 3 * NT < nmove; i += 4 * NT) {
                    const unsigned long long k0 = fetch(i), k1 = fetch(i + NT), k2 = fetch(i + 2 * NT), k3 = fetch(i + 3 * NT);
                    dstl[i] = k0; dstl[i + NT] = k1; dstl[i + 2 * NT] = k2; dstl[i + 3 * NT] = k3;
                }
                for (; i < nmove; i += NT) dstl[i] = fetch(i);
            }
            __syncthreads();
            if (a.mode == 3 && c.tid == 0) {
                for (int w = 0; w < a.world; w++) {
                    const int n = a.sc_count[(long long)w * a.B + r];
                    if (n < 0 || n > a.list_cap) c.status |= MOLLA_ROW_SHARD_OVERFLOW;
                }
            }
            if (a.mode == 2) {
                if (c.tid == 0) a.sb_count[r] = (nl > a.list_cap) ? -1 : nl;  // -1: the slice's list outgrew the exchange buffer
                continue;
            }
            LView lv;
            lv.n = nl; lv.woff = A->woff; lv.keep = keep_policy;
            if (nl <= SLIST_CAP) { lv.flat = slist; lv.seg = nullptr; lv.stride = 0; }
            else if (a.mode == 0) { lv.flat = nullptr; lv.seg = wl_seg; lv.stride = (size_t)a.R; }
            else {  // stage 3: the shards' lists were copied into one global array
                if (c.tid <= NWARP) A->woff[c.tid] = (c.tid == 0) ? 0 : nl;
                __syncthreads();
                lv.flat = nullptr; lv.seg = wl_flat; lv.stride = 0;
            }

            // ---- 4. the softmax denominator, exactly as the sequential loop rounds it
            if (c.tid == 0) A->walk_slow = 0;
            unsigned int *vstage = reinterpret_cast<unsigned int *>(c.stage);
            p1_run(c, lv, vstage, false, 0.0f);
            const float Z = A->walk_s;
            if (A->walk_slow) c.status |= MOLLA_ROW_SLOW_PATH;
            dZ = Z;

            // probabilities p = e / Z (sample.mojo:437-438). The head's candidates came out of pass B
            // and are converted on their own; the list itself is converted (once, in place) only for
            // rows that have to walk it.
            const unsigned int tau_p = __float_as_uint(__fdiv_rn(__uint_as_float(tau_bits), Z));
            const unsigned int tau_pb = tau_p > 1u ? tau_p : 1u;

            // min-p (sample.mojo:508-523): candidates below `largest probability * min_p` go; what is
            // left keeps its order. The largest probability is exp(0) / Z. On a sorted row the survivors
            // are a prefix, so the filter is one more bound on how many the walk may keep; on an
            // unsorted row the others' probabilities become zero, which no running sum can see.
            long long n_use = n_lim;
            const bool typ_on = typ < 1.0f;
            unsigned int minp_pbits = 0u;   // probability bits of the floor (0: off)
            if (minp > 0.0f) {
                const float p_top = __fdiv_rn(expf_pinned(__fsub_rn(top, top)), Z);
                const float floor_p = __fmul_rn(p_top, minp);
                minp_pbits = __float_as_uint(floor_p);
                // everything pass B dropped has a probability below 2.2e-8: a floor under that could
                // keep candidates the list no longer holds
                if (!(floor_p >= 2.2e-8f)) {
                    c.status |= MOLLA_ROW_UNSUPPORTED;
                } else if (!pure) {
                    // the smallest exponential whose probability reaches the floor (e / Z is monotone in e)
                    unsigned int lo_b = 0u, hi_b = 0x3F800000u;  // fdiv(hi) >= floor: p_top itself is e = 1
                    for (int it = 0; it < 32 && lo_b < hi_b; it++) {
                        const unsigned int mid = lo_b + ((hi_b - lo_b) >> 1);
                        if (__fdiv_rn(__uint_as_float(mid), Z) >= floor_p) hi_b = mid; else lo_b = mid + 1u;
                    }
                    const unsigned int e_floor = hi_b;
                    int cnt_ge = 0;
                    lv.for_each(c.tid, [&](int, unsigned long long kk, unsigned long long *) { cnt_ge += ((unsigned int)(kk >> 32) >= e_floor) ? 1 : 0; });
                    int n_ge;
                    (void)block_excl_scan<int>(cnt_ge, A->wsi, &n_ge);
                    __syncthreads();
                    if (n_ge < 1) n_ge = 1;  // never empties
                    if ((long long)n_ge < n_use) n_use = n_ge;
                }
            }
            if (c.status & MOLLA_ROW_UNSUPPORTED) {
                if (c.tid == 0) {
                    a.tokens[r] = -1; a.row_status[r] = c.status;
                    if (a.diag) { a.diag[4 * r] = Z; a.diag[4 * r + 1] = a.diag[4 * r + 2] = a.diag[4 * r + 3] = 0.0f; }
                }
                continue;
            }
            bool mark_head = head_in_pass;  // the head was taken in pass B: its entries are consumed
            bool mass_on = false;  // set: the conversion pass also fills the bin mass tables
            MassTable mt;
            mt.cnt = nullptr; mt.sets = nullptr; mt.j0 = 0; mt.tau0 = 0u; mt.Cm0 = mt.half0 = mt.big0 = 0.0f;
            auto convert_list = [&](bool gather_head) {
                __syncthreads();
                if (gather_head && c.tid == 0) A->ncand = 0;
                __syncthreads();
                lv.for_each(c.tid, [&](int, unsigned long long kk, unsigned long long *where) {
                    unsigned int pb = __float_as_uint(__fdiv_rn(key_val(kk), Z));
                    // entries the head took in pass B (by their exponential) are marked as consumed
                    if (!gather_head && mark_head && (unsigned int)(kk >> 32) >= tau_bits) pb = 0xFFFFFFFFu;
                    if (pure && pb < minp_pbits) pb = 0u;
                    const unsigned long long nk = ((unsigned long long)pb << 32) | (kk & 0xFFFFFFFFull);
                    if (lv.flat) *where = nk; else stg_keep(where, nk, keep_policy);
                    if (mass_on) masses_add(mt, pb);
                    if (gather_head && pb >= tau_pb) {
                        const int pos = atomicAdd(&A->ncand, 1);
                        if (pos < HEADC) A->cand[pos] = nk;
                    }
                });
                __syncthreads();
            };
            bool list_is_p = false;
            if (pure || !head_in_pass) { convert_list(!pure); list_is_p = true; }
            else {
                __syncthreads();
                const int nh = min(A->ncand, HEADC);
                for (int i = c.tid; i < nh; i += NT) {
                    const unsigned long long kk = A->cand[i];
                    A->cand[i] = ((unsigned long long)__float_as_uint(__fdiv_rn(key_val(kk), Z)) << 32) | (kk & 0xFFFFFFFFull);
                }
                __syncthreads();
            }

            if (pure) {
                // ---- 5a. nothing sorted: the draw walks the vocabulary in order (sample.mojo:365-369,
                // 580-594): the same exact-sum machinery on the list of probabilities
                __syncthreads();
                p1_run(c, lv, vstage, false, 0.0f);
                const float sum = A->walk_s;
                const float target = __fmul_rn(u01, sum);
                p1_run(c, lv, vstage, true, target);
                if (c.tid == 0) {
                    A->b_sum = sum; A->b_target = target;
                    A->b_event = A->walk_found;
                    A->b_idx = A->walk_found ? key_idx(lv.at(A->walk_idx)) : imax;
                    A->b_aux = A->walk_slow;
                }
                __syncthreads();
                token = A->b_idx; dsum = A->b_sum; dtarget = A->b_target;
                if (A->b_aux) c.status |= MOLLA_ROW_SLOW_PATH;
                if (!A->b_event) {
                    // the walk fell off the end: the reference returns the last token of the vocabulary,
                    // whether or not it could matter to any sum
                    token = a.Vg - 1;
                    if (minp_pbits) {  // ... the last one min-p left
                        int last = -1;
                        lv.for_each(c.tid, [&](int, unsigned long long kk, unsigned long long *) {
                            if ((unsigned int)(kk >> 32) >= minp_pbits) last = max(last, key_idx(kk));
                        });
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
                        __syncthreads();
                        if (c.lane == 0) A->wsi[c.warp] = last;
                        __syncthreads();
                        for (int w = 0; w < NWARP; w++) last = max(last, A->wsi[w]);
                        __syncthreads();
                        token = last >= 0 ? last : imax;
                    }
                }
            } else {
                // ---- 5b. sorted order. The head: the need largest, sorted, walked exactly
                // (sample.mojo:497-506, :580-590). The need-th largest of the threads' own maxima
                // bounds the need-th largest element from below.
                int nc = A->ncand;
                unsigned int tau_head = head_in_pass ? 0xFFFFFFFFu : tau_pb;
                bool head_overflow = false;
                if (nc > HEADC) {
                    // more equal-or-larger values than the head holds (flat or heavily tied rows):
                    // no head, the descending walk takes everything from the top
                    nc = 0; tau_head = 0xFFFFFFFFu; head_overflow = true; mark_head = false;
                    c.status |= MOLLA_ROW_SLOW_PATH;
                }
                {
                    sort_cands(c, nc);
                    for (int i = c.tid; i < nc; i += NT) {
                        const float p = A->pc[i];
                        const bool eq = (i > 0 && A->pc[i - 1] == p) || (i + 1 < nc && A->pc[i + 1] == p);
                        A->hidx[i] = (unsigned int)key_idx(A->cand[i]) | (eq ? 0x80000000u : 0u);
                    }
                    __syncthreads();
#ifdef MOLLA_SAMPLE_TESTING
                    if (a.topk_out) {
                        for (int i = c.tid; i < a.topk_cap; i += NT)
                            a.topk_out[(long long)r * a.topk_cap + i] =
                                (i < nc && (long long)i < n_use) ? (int)(A->hidx[i] & 0x7fffffffu) : -1;
                    }
#endif
                    if (c.tid == 0) {
                        float s = 0.0f;
                        long long pos = 0;
                        int cut = -1, tie = 0;
                        for (int i = 0; i < nc; i++) {
                            if (pos >= n_use) break;
                            s = __fadd_rn(s, A->pc[i]);
                            A->pre[i] = s;
                            pos++;
                            if (topp_on && s >= P) {
                                cut = i + 1;
                                if (i + 1 < nc && (long long)(i + 1) < n_use && A->pc[i + 1] == A->pc[i]) tie |= MOLLA_ROW_TOPP_TIE;
                                break;
                            }
                            if (pos >= n_use) { cut = i + 1; break; }
                        }
                        if (cut < 0 && !p3row && !head_overflow) cut = nc;  // everything that can matter is in the head
                        if (n_use < (long long)a.Vg && (long long)nc > n_use && A->pc[n_use] == A->pc[n_use - 1])
                            tie |= MOLLA_ROW_TOPK_TIE;
                        A->b_s = s; A->b_pos = pos; A->b_event = EV_NONE; A->b_idx = -1; A->b_p = 0.0f;
                        if (typ_on) {
                            A->ncand = cut;  // the typical-p filter takes over from here
                        } else if (cut > 0) {
                            const float sum = A->pre[cut - 1];
                            const float target = __fmul_rn(u01, sum);
                            int at = cut - 1;
                            for (int i = 0; i < cut; i++)
                                if (target < A->pre[i]) { at = i; break; }
                            A->b_event = EV_DRAW; A->b_idx = (int)(A->hidx[at] & 0x7fffffffu); A->b_p = A->pc[at];
                            if ((at > 0 && A->pc[at - 1] == A->pc[at]) || (at + 1 < cut && A->pc[at + 1] == A->pc[at]))
                                tie |= MOLLA_ROW_CHOSEN_TIE;
                            A->b_sum = sum; A->b_target = target;
                        }
                        A->b_aux = tie;
                    }
                    __syncthreads();
                    c.status |= (unsigned int)A->b_aux;
                    const float head_s = A->b_s;
                    const long long head_pos = A->b_pos;
                    if (typ_on) {
                        const int m = A->ncand;
                        if (m <= 0) {
                            c.status |= MOLLA_ROW_UNSUPPORTED;  // what the earlier filters left reaches past the head
                        } else {
                            typical_head(c, m, typ, u01);
                            token = A->b_idx; dp = A->b_p; dsum = A->b_sum; dtarget = A->b_target;
                            c.status |= (unsigned int)A->b_aux;
                        }
                    } else if (A->b_event == EV_DRAW) {
                        token = A->b_idx; dp = A->b_p; dsum = A->b_sum; dtarget = A->b_target;
                    } else {
                        // ---- 6. past the head: the cut walk, then the draw walk
                        // long lists (global memory) are first sorted into their value bins
                        // long lists (global memory): per-bin integer masses come out of the conversion pass
                        MassCk ck;
                        ck.n = 0;
                        mt.cnt = reinterpret_cast<unsigned int *>(A->hval);
                        mt.sets = reinterpret_cast<unsigned int *>(c.stage);  // idle while the list is a global view
                        const bool use_mt = (a.mode == 0) && !lv.flat && !list_is_p && head_s > 0.0f;
                        if (use_mt) { masses_begin(c, mt, fexpo(head_s), tau_head); mass_on = true; }
                        const bool help_on = use_mt && a.help && nl >= HELP_MIN_LIST && !MOLLA_KNOB(a, 8);
                        if (help_on) {
                            // a long list: blocks that have run out of rows take segments of this pass
                            if (!helped_convert(c, a, wl_seg, Z, tau_bits, mark_head, mt)) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
                            list_is_p = true;
                        }
                        if (!list_is_p) { convert_list(false); list_is_p = true; }
                        mass_on = false;
                        __syncthreads();
                        Walk cutw; cutw.s = head_s; cutw.pos = head_pos; cutw.tau = tau_head;
                        cutw.event = EV_NONE; cutw.idx = -1; cutw.p = 0; cutw.tie = 0;
                        const bool limited = n_use < (long long)a.Vg;
                        {
                            int hi = NBINS;
                            const bool done = use_mt && descend_masses(c, a, help_on, lv, mt, ck, cutw, hi, topp_on ? P : 3.4e38f, 3.4e38f, limited ? n_use : -1);
                            if (!done) descend(c, lv, cutw, topp_on ? P : 3.4e38f, 3.4e38f, limited ? n_use : -1);
                        }
                        if (cutw.event != EV_DEGENERATE) {
                            if (cutw.event == EV_CUT && cutw.tie) c.status |= MOLLA_ROW_TOPP_TIE;
                            if (cutw.event == EV_LIMIT && cutw.tie) c.status |= MOLLA_ROW_TOPK_TIE;
                            const float sum = cutw.s;
                            const float target = __fmul_rn(u01, sum);
                            dsum = sum; dtarget = target;
                            __syncthreads();
                            if (c.tid == 0) {  // is the drawn element in the head?
                                int at = -1;
                                for (int i = 0; i < nc; i++)
                                    if (target < A->pre[i]) { at = i; break; }
                                A->b_event = EV_NONE;
                                if (at >= 0) {
                                    A->b_event = EV_DRAW; A->b_idx = (int)(A->hidx[at] & 0x7fffffffu);
                                    A->b_p = __fsub_rn(A->pre[at], at > 0 ? A->pre[at - 1] : 0.0f);
                                    A->b_aux = (A->hidx[at] & 0x80000000u) ? MOLLA_ROW_CHOSEN_TIE : 0;
                                }
                            }
                            __syncthreads();
                            if (A->b_event == EV_DRAW) {
                                token = A->b_idx; dp = A->b_p; c.status |= (unsigned int)A->b_aux;
                            } else {
                                bool resolved = false;
                                if (target < sum) {
                                    __syncthreads();
                                    Walk dw; dw.s = head_s; dw.pos = head_pos; dw.tau = tau_head;
                                    dw.event = EV_NONE; dw.idx = -1; dw.p = 0; dw.tie = 0;
                                    bool ddone = false;
                                    if (use_mt) {
                                        int hi = NBINS;
                                        ddone = descend_masses(c, a, help_on, lv, mt, ck, dw, hi, 3.4e38f, target, -1);
                                    }
                                    if (!ddone) descend(c, lv, dw, 3.4e38f, target, -1);
                                    if (dw.event == EV_DRAW) {
                                        token = dw.idx; dp = dw.p; resolved = true;
                                        if (dw.tie) c.status |= MOLLA_ROW_CHOSEN_TIE;
                                    } else if (dw.event == EV_DEGENERATE) {
                                        resolved = true;
                                    }
                                }
                                if (!resolved) {
                                    // the walk falls off the end: the last kept candidate (sample.mojo:591-594)
                                    if (cutw.event == EV_CUT || cutw.event == EV_LIMIT) {
                                        token = cutw.idx; dp = cutw.p;
                                    } else {
                                        // everything listed was kept: its smallest value, highest id last
                                        // (keys order by value, then by inverted id)
                                        unsigned long long best = ~0ull;
                                        lv.for_each(c.tid, [&](int, unsigned long long kk, unsigned long long *) { best = kk < best ? kk : best; });
#pragma unroll
                                        for (int o = 16; o > 0; o >>= 1) {
                                            unsigned long long ob = __shfl_xor_sync(0xffffffffu, best, o);
                                            best = ob < best ? ob : best;
                                        }
                                        __syncthreads();
                                        if (c.lane == 0) A->wsu[c.warp] = best;
                                        __syncthreads();
                                        best = A->wsu[0];
                                        for (int w = 1; w < NWARP; w++) best = A->wsu[w] < best ? A->wsu[w] : best;
                                        token = nl > 0 ? key_idx(best) : imax;
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
        // a bounded wait that ran out in any warp fails the row; a failed row keeps its sampler state
        if (MOLLA_KNOB(a, 16) && c.warp == 3) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
        if (__syncthreads_or((c.status & MOLLA_ROW_LOAD_TIMEOUT) ? 1 : 0)) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
        if (c.status & (MOLLA_ROW_LOAD_TIMEOUT | MOLLA_ROW_DEGENERATE | MOLLA_ROW_INVALID_CONFIG | MOLLA_ROW_UNSUPPORTED | MOLLA_ROW_SHARD_OVERFLOW | MOLLA_ROW_EMPTY)) token = -1;
        if (c.tid == 0) {
            a.tokens[r] = token;
            a.row_status[r] = c.status;
            if (a.ring && token >= 0) {  // `_took` (sample.mojo:361-363): observe, then one more draw used
                if (ring_n > 0) {        // `observe` (:246-258)
                    const int hd = a.ring_head[q];
                    const int at = (hd >= 0 && hd < ring_n) ? hd : 0;
                    a.ring[(size_t)q * (size_t)a.ring_cap + at] = (long long)token;
                    a.ring_head[q] = (at + 1) % ring_n;
                    const int f = a.ring_filled[q];
                    a.ring_filled[q] = f < ring_n ? f + 1 : ring_n;
                }
                a.drawn_rw[q] += 1ull;
                if (a.stopped) a.stopped[r] = (a.stop_token && a.stop_token[q] == (long long)token) ? 1 : 0;
            }
            if (a.diag) { a.diag[4 * r] = dZ; a.diag[4 * r + 1] = dsum; a.diag[4 * r + 2] = dtarget; a.diag[4 * r + 3] = dp; }
        }
    }
    if (a.help && !MOLLA_KNOB(a, 8)) help_others(c, a);  // no rows left: lend a hand to the blocks still on a long list
}

// =============================================================================
// Logprobs of the raw logits (sample.mojo:268-293): one CTA per row, the row is
// read twice (second read is an L2 hit for blocks that fit).
// =============================================================================
__global__ void __launch_bounds__(NT, 1) logprob_kernel(const float *logits, long long row_stride, int B, int V,
                                                        const int *tokens, int top_n, float *chosen_lp,
                                                        int *top_ids, float *top_lps, float *full_out,
                                                        const int *rows, int n_logit_rows, float softcap) {
    __shared__ float wsf[NWARP + 1];
    __shared__ int wsi[NWARP + 1];
    __shared__ double wsd[NWARP + 1];
    __shared__ unsigned long long cand[NT];
    __shared__ int ncand;
    __shared__ float s_thr;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int r = blockIdx.x; r < B; r += gridDim.x) {
        const long long lrow = rows ? (long long)rows[r] : (long long)r;
        if (rows && (lrow < 0 || (n_logit_rows > 0 && lrow >= n_logit_rows))) {
            // a stale row index: nothing is read; the row's sampling call has reported it
            if (chosen_lp && tid == 0) chosen_lp[r] = 0.0f;
            for (int i = tid; i < top_n; i += NT) { top_ids[(long long)r * top_n + i] = -1; top_lps[(long long)r * top_n + i] = 0.0f; }
            continue;
        }
        const float *z = logits + lrow * row_stride;
        auto cap1 = [&](float x) -> float { return softcap > 0.0f ? softcap_pinned(x, softcap) : x; };
        auto at = [&](int i) -> float { return cap1(__ldg(z + i)); };
        // rows that start on a 16-byte boundary are read four logits at a time
        const bool vec = ((reinterpret_cast<uintptr_t>(z) & 15u) == 0);
        const int n4 = vec ? (V >> 2) : 0;
        const float4 *z4 = reinterpret_cast<const float4 *>(z);
        // pass 1: maximum and each thread's own maximum
        float tm = -INFINITY;
        for (int i = tid; i < n4; i += NT) {
            const float4 x = __ldg(z4 + i);
            tm = fmaxf(fmaxf(tm, fmaxf(cap1(x.x), cap1(x.y))), fmaxf(cap1(x.z), cap1(x.w)));
        }
        for (int i = 4 * n4 + tid; i < V; i += NT) tm = fmaxf(tm, at(i));
        float m = warp_max(tm);
        __syncthreads();
        if (lane == 0) wsf[warp] = m;
        __syncthreads();
        float top = wsf[0];
        for (int w = 1; w < NWARP; w++) top = fmaxf(top, wsf[w]);
        // threshold for the top-N: the N-th largest of the per-thread maxima (at least N logits reach it)
        float thr = -INFINITY;
        if (top_n > 0) {
            __syncthreads();
            cand[tid] = ((unsigned long long)fkey(tm) << 32) | (unsigned long long)tid;
            bitonic_desc(cand, NT, tid);
            if (tid == 0) {
                const int nth = min(min(top_n, V), NT) - 1;
                s_thr = fkey_inv((unsigned int)(cand[nth] >> 32));
                ncand = 0;
            }
            __syncthreads();
            thr = s_thr;
        }
        // pass 2: sum of exp(z - top) accumulated in fp64, candidates for the top-N
        double acc = 0.0;
        auto one = [&](float x, int i) {
            acc += (double)expf_pinned(__fsub_rn(x, top));
            if (top_n > 0 && x >= thr) {
                const int pos = atomicAdd(&ncand, 1);
                if (pos < NT) cand[pos] = ((unsigned long long)fkey(x) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned int)i);
            }
        };
        for (int i = tid; i < n4; i += NT) {
            const float4 x = __ldg(z4 + i);
            one(cap1(x.x), 4 * i); one(cap1(x.y), 4 * i + 1); one(cap1(x.z), 4 * i + 2); one(cap1(x.w), 4 * i + 3);
        }
        for (int i = 4 * n4 + tid; i < V; i += NT) one(at(i), i);
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
            chosen_lp[r] = (t >= 0 && t < V) ? __fsub_rn(__fsub_rn(at(t), top), offset) : 0.0f;
        }
        if (full_out) {
            float *o = full_out + (long long)r * V;
            for (int i = tid; i < V; i += NT) o[i] = __fsub_rn(__fsub_rn(at(i), top), offset);
        }
        if (top_n > 0) {
            __syncthreads();
            const int n = ncand;
            if (n <= NT) {
                for (int i = n + tid; i < NT; i += NT) cand[i] = 0ull;
                __syncthreads();
                bitonic_desc(cand, NT, tid);
                if (tid < top_n) {
                    if (tid < n) {
                        int id = (int)(0xFFFFFFFFu - (unsigned int)(cand[tid] & 0xFFFFFFFFull));
                        top_ids[(long long)r * top_n + tid] = id;
                        top_lps[(long long)r * top_n + tid] = __fsub_rn(__fsub_rn(at(id), top), offset);
                    } else {
                        top_ids[(long long)r * top_n + tid] = -1;
                        top_lps[(long long)r * top_n + tid] = 0.0f;
                    }
                }
            } else {
                // More logits at or above the threshold than the buffer holds (a flat or heavily
                // quantised row): the N largest one after the other, each the first in the order
                // (value descending, index ascending) behind the one before it. A pass per pick.
                float lastv = INFINITY;
                int lasti = -1;
                for (int k = 0; k < top_n; k++) {
                    float bv = -INFINITY;
                    int bi = 0x7fffffff;
                    for (int i = tid; i < V; i += NT) {
                        const float x = at(i);
                        const bool behind = x < lastv || (x == lastv && i > lasti);
                        if (behind && (x > bv || (x == bv && i < bi))) { bv = x; bi = i; }
                    }
                    warp_argmax(bv, bi);
                    __syncthreads();
                    if (lane == 0) { wsf[warp] = bv; wsi[warp] = bi; }
                    __syncthreads();
                    bv = wsf[0]; bi = wsi[0];
                    for (int w = 1; w < NWARP; w++)
                        if (wsf[w] > bv || (wsf[w] == bv && wsi[w] < bi)) { bv = wsf[w]; bi = wsi[w]; }
                    const bool found = bi != 0x7fffffff;
                    if (tid == 0) {
                        top_ids[(long long)r * top_n + k] = found ? bi : -1;
                        top_lps[(long long)r * top_n + k] = found ? __fsub_rn(__fsub_rn(bv, top), offset) : 0.0f;
                    }
                    lastv = bv; lasti = bi;
                    if (!found) lastv = -INFINITY;
                }
            }
        }
        __syncthreads();
    }
}

__global__ void expf_kernel(const float *x, long long n, float *out) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = (x[i] <= 0.0f) ? expf_pinned_nonpos(x[i]) : expf_pinned(x[i]);  // both forms are in use
}

__global__ void logf_kernel(const float *x, long long n, float *out) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = logf_pinned(x[i]);
}

// =============================================================================
// Host side of the C ABI
// =============================================================================
thread_local char g_err[512] = "";

// Scratch of the entry point that allocates nothing. It lives in the library's device image:
// every GPU that loads the library sets these bytes aside until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MOLLA_NOALLOC_SCRATCH_BYTES];
constexpr int NOALLOC_MAX_DEVICES = 64;
void *g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};  // device address of the array, per device ordinal
#ifdef MOLLA_SAMPLE_TESTING
long long *g_prof = nullptr;
int g_knobs = 0;
int *g_topk = nullptr;
int g_topk_cap = 0;
#define MOLLA_SET_TESTING_ARGS(a) do { (a).prof = g_prof; (a).knobs = g_knobs; (a).topk_out = g_topk; (a).topk_cap = g_topk_cap; } while (0)
#else
#define MOLLA_SET_TESTING_ARGS(a) do { } while (0)
#endif

int fail(int code, const char *fmt, const char *detail = "") {
    snprintf(g_err, sizeof(g_err), fmt, detail);
    return code;
}

int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    return sms;
}

size_t smem_bytes(int V) {
    return (size_t)STAGE_FLOATS * 4 + ((sizeof(Aux) + 15) / 16) * 16 + (size_t)((V + 31) / 32) * 4 + 16;
}

int region_floats(int V) { return (((V + NWARP - 1) / NWARP) + 3) & ~3; }

// scratch layout: [row counter and finished-rows counter, 256 bytes][row order][per CTA: 16 per-warp
// list segments + one contiguous copy, each entry an (exp bits, token id) pair]
constexpr size_t WS_HEADER = 256 + (size_t)ORDER_CAP * 4;
// ... and behind the lists, for the ordinary entry points, one HelpSlot and one bin-mass table
// per CTA
size_t help_bytes(size_t ctas) { return ctas * (sizeof(HelpSlot) + (size_t)HELP_TABLE_WORDS * 4); }
size_t batch_workspace_bytes(int B, int V, int sms) {
    const size_t ctas = (size_t)(B < sms ? B : sms);
    return WS_HEADER + ctas * 2 * (size_t)NWARP * (size_t)region_floats(V) * 8 + help_bytes(ctas);
}

int launch_rows(const BatchArgs &args_in, void *d_workspace, cudaStream_t st, int max_ctas = 0x7fffffff, bool with_help = false) {
    BatchArgs a = args_in;
    const int sms = sm_count();
    if (sms <= 0) return fail(MOLLA_ERR_CUDA, "cannot query the device%s");
    int dev = 0, max_optin = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&max_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    const size_t smem = smem_bytes(a.V);
    a.R = region_floats(a.V);
    if (a.mode == 0) { a.Vg = a.V; a.col0 = 0; }
    if (smem > (size_t)max_optin || (a.R + PIECE - 1) / PIECE > MAX_PIECES)
        return fail(MOLLA_ERR_VOCAB, "vocabulary too wide for the shared-memory bitmap and tile table%s");
    cudaError_t e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "cudaFuncSetAttribute(smem): %s", cudaGetErrorString(e));
    a.row_counter = (int *)d_workspace;
    a.wlist = (unsigned long long *)((char *)d_workspace + WS_HEADER);
    e = cudaMemsetAsync(d_workspace, 0, 256, st);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "workspace clear failed: %s", cudaGetErrorString(e));
    int grid = a.B < sms ? a.B : sms;
    if (grid > max_ctas) grid = max_ctas;
    a.rows_done = (int *)d_workspace + 2;
    a.help = nullptr; a.help_tables = nullptr;
    if (with_help && a.mode == 0 && grid > 1) {
        const size_t ctas = (size_t)(a.B < sms ? a.B : sms);
        char *hb = (char *)d_workspace + WS_HEADER + ctas * 2 * (size_t)NWARP * (size_t)a.R * 8;
        a.help = hb;
        a.help_tables = (unsigned int *)(hb + ctas * sizeof(HelpSlot));
        e = cudaMemsetAsync(hb, 0, ctas * sizeof(HelpSlot), st);
        if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "workspace clear failed: %s", cudaGetErrorString(e));
    }
    a.order = nullptr;
    if (!a.penalised_only && a.B > grid && a.B <= ORDER_CAP && a.temperature) {
        int *order = (int *)((char *)d_workspace + 256);
        order_rows_kernel<<<1, NT, 0, st>>>(a.temperature, a.top_k, a.slot, a.B, order);
        a.order = order;
    }
    sample_rows_kernel<<<grid, NT, smem, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

// The ordinary entry points' launch: the cluster kernel when the vocabulary fits a cluster, else
// the streaming kernel with its lists in the workspace.
int launch_sampling(const BatchArgs &args_in, void *d_workspace, cudaStream_t st) {
    const int rc = molla_cluster_launch(args_in, d_workspace, st, g_err, sizeof(g_err));
    if (rc != MOLLA_CLUSTER_DECLINED) return rc;
    if (args_in.mask) return fail(MOLLA_ERR_VOCAB, "a grammar mask is only done for vocabularies a thread-block cluster can hold%s");
    return launch_rows(args_in, d_workspace, st, 0x7fffffff, true);
}

}  // namespace

extern "C" {

int32_t molla_sample_abi_version(void) { return MOLLA_SAMPLE_ABI_VERSION; }

const char *molla_sample_last_error(void) { return g_err; }

float molla_sample_draw(uint64_t seed, uint64_t counter) { return draw01(seed, counter); }

int64_t molla_sample_workspace_bytes(int32_t B, int32_t V, int32_t top_n) {
    if (B < 0 || V <= 0 || top_n < 0 || top_n > TOPN_MAX) return fail(MOLLA_ERR_ARGUMENT, "bad shape for the workspace query%s");
    const int sms = sm_count();
    if (sms <= 0) return fail(MOLLA_ERR_CUDA, "cannot query the device%s");
    return (int64_t)batch_workspace_bytes(B, V, sms);
}

int32_t molla_sample_batch_masked(const uint32_t *d_mask, int64_t mask_stride_words,
                                  const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
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
    if (d_mask && mask_stride_words < (V + 31) / 32) return fail(MOLLA_ERR_ARGUMENT, "a row of the mask has fewer bits than the vocabulary%s");
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V, top_n))
        return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.logits = d_logits; a.row_stride = row_stride; a.B = B; a.V = V;
    a.mask = d_mask; a.mask_stride = mask_stride_words;
    a.temperature = d_temperature; a.top_k = d_top_k; a.top_p = d_top_p; a.min_p = d_min_p;
    a.typical_p = d_typical_p; a.repeat_penalty = d_repeat_penalty;
    a.frequency_penalty = d_frequency_penalty; a.presence_penalty = d_presence_penalty;
    a.window_on = d_window_on;
    a.seed = (const unsigned long long *)d_seed; a.drawn = (const unsigned long long *)d_drawn;
    a.hist = (const long long *)d_hist; a.hist_off = d_hist_off;
    a.bias_ids = (const long long *)d_bias_ids; a.bias_vals = d_bias_vals; a.bias_off = d_bias_off;
    a.tokens = d_tokens; a.row_status = d_row_status; a.diag = d_diag;
    a.penalised = nullptr; a.penalised_only = 0;
    MOLLA_SET_TESTING_ARGS(a);
    int rc = launch_sampling(a, d_workspace, st);
    if (rc != MOLLA_OK) return rc;
    if (d_chosen_logprob || top_n > 0) {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int grid = B < sms ? B : sms;
        logprob_kernel<<<grid, NT, 0, st>>>(d_logits, row_stride, B, V, d_tokens, top_n, d_chosen_logprob,
                                            d_top_ids, d_top_logprobs, nullptr, nullptr, 0, 0.0f);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "logprob launch failed: %s", cudaGetErrorString(e));
    }
    return MOLLA_OK;
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
    return molla_sample_batch_masked(nullptr, 0, d_logits, row_stride, B, V, d_temperature, d_top_k, d_top_p, d_min_p,
                                     d_typical_p, d_repeat_penalty, d_frequency_penalty, d_presence_penalty, d_window_on,
                                     d_seed, d_drawn, d_hist, d_hist_off, d_bias_ids, d_bias_vals, d_bias_off, top_n,
                                     d_workspace, workspace_bytes, stream, d_tokens, d_chosen_logprob, d_top_ids,
                                     d_top_logprobs, d_row_status, d_diag);
}

int32_t molla_sample_decode_step(const float *d_logits, int64_t row_stride, int32_t n_logit_rows, int32_t V,
                                 const int32_t *d_rows, const int32_t *d_slots, int32_t B, int32_t n_slots,
                                 float final_softcap, const float *d_temperature, const int32_t *d_top_k,
                                 const float *d_top_p, const float *d_min_p, const float *d_typical_p,
                                 const float *d_repeat_penalty, const float *d_frequency_penalty,
                                 const float *d_presence_penalty, const uint64_t *d_seed, uint64_t *d_drawn,
                                 int64_t *d_ring, int32_t ring_cap, int32_t *d_ring_head, int32_t *d_ring_filled,
                                 const int32_t *d_ring_len, const int64_t *d_stop_token, const int64_t *d_bias_ids,
                                 const float *d_bias_vals, const int32_t *d_bias_off, int32_t top_n,
                                 void *d_workspace, int64_t workspace_bytes, void *stream, int32_t *d_tokens,
                                 uint8_t *d_stopped, float *d_chosen_logprob, int32_t *d_top_ids,
                                 float *d_top_logprobs, uint32_t *d_row_status) {
    g_err[0] = 0;
    if (!d_logits || !d_tokens || !d_row_status) return fail(MOLLA_ERR_ARGUMENT, "logits, tokens and row status are required%s");
    if (B < 0 || V <= 0 || row_stride < V || n_logit_rows < 0 || n_slots < 0) return fail(MOLLA_ERR_ARGUMENT, "bad block shape%s");
    if (!d_rows && B > n_logit_rows) return fail(MOLLA_ERR_ARGUMENT, "more rows asked for than the block holds%s");
    if (!d_slots && B > n_slots) return fail(MOLLA_ERR_ARGUMENT, "more rows than sampler slots%s");
    if (!(final_softcap >= 0.0f)) return fail(MOLLA_ERR_ARGUMENT, "a softcap cannot be negative%s");
    if (!d_drawn || !d_ring || !d_ring_head || !d_ring_filled || !d_ring_len || ring_cap <= 0)
        return fail(MOLLA_ERR_ARGUMENT, "the sampler state (draw counters and windows) is required%s");
    if (ring_cap > PATCH_MAX) return fail(MOLLA_ERR_ARGUMENT, "windows longer than 1024 tokens are not supported%s");
    if (top_n < 0 || top_n > TOPN_MAX) return fail(MOLLA_ERR_ARGUMENT, "top_n out of range%s");
    if (top_n > 0 && (!d_top_ids || !d_top_logprobs)) return fail(MOLLA_ERR_ARGUMENT, "top_n needs its output arrays%s");
    if ((d_bias_ids == nullptr) != (d_bias_off == nullptr) || (d_bias_ids && !d_bias_vals))
        return fail(MOLLA_ERR_ARGUMENT, "bias ids, values and offsets go together%s");
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V, top_n))
        return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.logits = d_logits; a.row_stride = row_stride; a.B = B; a.V = V;
    a.rows = d_rows; a.slot = d_slots; a.softcap = final_softcap;
    a.temperature = d_temperature; a.top_k = d_top_k; a.top_p = d_top_p; a.min_p = d_min_p;
    a.typical_p = d_typical_p; a.repeat_penalty = d_repeat_penalty;
    a.frequency_penalty = d_frequency_penalty; a.presence_penalty = d_presence_penalty;
    a.seed = (const unsigned long long *)d_seed; a.drawn = (const unsigned long long *)d_drawn;
    a.drawn_rw = (unsigned long long *)d_drawn;
    a.ring = (long long *)d_ring; a.ring_cap = ring_cap; a.ring_head = d_ring_head; a.ring_filled = d_ring_filled;
    a.ring_len = d_ring_len; a.stop_token = (const long long *)d_stop_token; a.stopped = d_stopped;
    a.bias_ids = (const long long *)d_bias_ids; a.bias_vals = d_bias_vals; a.bias_off = d_bias_off;
    a.tokens = d_tokens; a.row_status = d_row_status;
    a.n_logit_rows = n_logit_rows; a.n_slots = n_slots;
    MOLLA_SET_TESTING_ARGS(a);
    if (d_stopped) {
        cudaError_t e0 = cudaMemsetAsync(d_stopped, 0, (size_t)B, st);
        if (e0 != cudaSuccess) return fail(MOLLA_ERR_CUDA, "clearing the stop flags failed: %s", cudaGetErrorString(e0));
    }
    int rc = launch_sampling(a, d_workspace, st);
    if (rc != MOLLA_OK) return rc;
    if (d_chosen_logprob || top_n > 0) {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int grid = B < sms ? B : sms;
        logprob_kernel<<<grid, NT, 0, st>>>(d_logits, row_stride, B, V, d_tokens, top_n, d_chosen_logprob,
                                            d_top_ids, d_top_logprobs, nullptr, d_rows, n_logit_rows, final_softcap);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "logprob launch failed: %s", cudaGetErrorString(e));
    }
    return MOLLA_OK;
}

int32_t molla_sample_batch_noalloc(const float *d_logits, int64_t row_stride, int32_t B, int32_t V,
                                   const float *d_temperature, const int32_t *d_top_k, const float *d_top_p,
                                   const float *d_min_p, const float *d_typical_p, const float *d_repeat_penalty,
                                   const float *d_frequency_penalty, const float *d_presence_penalty,
                                   const uint8_t *d_window_on, const uint64_t *d_seed, const uint64_t *d_drawn,
                                   const int64_t *d_hist, const int32_t *d_hist_off, const int64_t *d_bias_ids,
                                   const float *d_bias_vals, const int32_t *d_bias_off, int32_t top_n, void *stream,
                                   int32_t *d_tokens, float *d_chosen_logprob, int32_t *d_top_ids,
                                   float *d_top_logprobs, uint32_t *d_row_status) {
    g_err[0] = 0;
    if (!d_logits || !d_tokens || !d_row_status) return fail(MOLLA_ERR_ARGUMENT, "logits, tokens and row status are required%s");
    if (B < 0 || V <= 0 || row_stride < V) return fail(MOLLA_ERR_ARGUMENT, "bad block shape%s");
    if (top_n < 0 || top_n > TOPN_MAX) return fail(MOLLA_ERR_ARGUMENT, "top_n out of range%s");
    if (top_n > 0 && (!d_top_ids || !d_top_logprobs)) return fail(MOLLA_ERR_ARGUMENT, "top_n needs its output arrays%s");
    if ((d_hist == nullptr) != (d_hist_off == nullptr)) return fail(MOLLA_ERR_ARGUMENT, "history ids and offsets go together%s");
    if ((d_bias_ids == nullptr) != (d_bias_off == nullptr) || (d_bias_ids && !d_bias_vals))
        return fail(MOLLA_ERR_ARGUMENT, "bias ids, values and offsets go together%s");
    if (V > MOLLA_NOALLOC_MAX_VOCAB)
        return fail(MOLLA_ERR_WORKSPACE, "the built-in scratch holds rows of at most MOLLA_NOALLOC_MAX_VOCAB logits%s");
    if (B > MOLLA_NOALLOC_MAX_ROWS)
        return fail(MOLLA_ERR_WORKSPACE, "the built-in scratch serves at most MOLLA_NOALLOC_MAX_ROWS rows per call%s");
    if (B == 0) return MOLLA_OK;
    // how many CTAs' lists the fixed array holds for this vocabulary (at least one, by the limit above)
    const size_t per_cta = 2 * (size_t)NWARP * (size_t)region_floats(V) * 8;
    const size_t room = (size_t)MOLLA_NOALLOC_SCRATCH_BYTES - WS_HEADER;
    const int max_ctas = (int)(room / per_cta);
    if (max_ctas < 1) return fail(MOLLA_ERR_WORKSPACE, "the built-in scratch is too small for this vocabulary%s");
    // Set-up, once per device: in host code the array's name is only a handle. The address the
    // kernels can use comes from cudaGetSymbolAddress with that device current.
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(MOLLA_ERR_ARGUMENT, "device ordinal out of range%s");
    if (!g_noalloc_addr[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) return fail(MOLLA_ERR_CUDA, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_noalloc_addr[dev] = ptr;
    }
    void *ws = g_noalloc_addr[dev];
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
    a.tokens = d_tokens; a.row_status = d_row_status; a.diag = nullptr;
    // launch_rows clears the row counter at the head of the scratch (the one part that must start
    // at zero); the row order and the lists behind it are written before they are read
    int rc = launch_rows(a, ws, st, max_ctas);
    if (rc != MOLLA_OK) return rc;
    if (d_chosen_logprob || top_n > 0) {
        int sms = 148;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int grid = B < sms ? B : sms;
        logprob_kernel<<<grid, NT, 0, st>>>(d_logits, row_stride, B, V, d_tokens, top_n, d_chosen_logprob,
                                            d_top_ids, d_top_logprobs, nullptr, nullptr, 0, 0.0f);
        e = cudaGetLastError();
        if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "logprob launch failed: %s", cudaGetErrorString(e));
    }
    return MOLLA_OK;
}

// ---- vocab-sharded form ------------------------------------------------------------
namespace {
BatchArgs shard_args(const float *d_logits, int64_t row_stride, int32_t B, int32_t V, const float *t, const int32_t *k,
                     const float *p, const float *minp, const float *typ, const float *rp, const float *fp,
                     const float *pp, const uint8_t *won, const uint64_t *seed, const uint64_t *drawn,
                     const int64_t *hist, const int32_t *hist_off, const int64_t *bias_ids, const float *bias_vals,
                     const int32_t *bias_off) {
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.logits = d_logits; a.row_stride = row_stride; a.B = B; a.V = V;
    a.temperature = t; a.top_k = k; a.top_p = p; a.min_p = minp; a.typical_p = typ; a.repeat_penalty = rp;
    a.frequency_penalty = fp; a.presence_penalty = pp; a.window_on = won;
    a.seed = (const unsigned long long *)seed; a.drawn = (const unsigned long long *)drawn;
    a.hist = (const long long *)hist; a.hist_off = hist_off;
    a.bias_ids = (const long long *)bias_ids; a.bias_vals = bias_vals; a.bias_off = bias_off;
    return a;
}
}  // namespace

int32_t molla_sample_shard_summary_words(void) { return SA_WORDS; }

int32_t molla_sample_shard_stage_a(const float *d_logits, int64_t row_stride, int32_t B, int32_t V_local, int32_t col0,
                                   int32_t V_global, const float *d_temperature, const int32_t *d_top_k,
                                   const float *d_top_p, const float *d_min_p, const float *d_typical_p,
                                   const float *d_repeat_penalty, const float *d_frequency_penalty,
                                   const float *d_presence_penalty, const uint8_t *d_window_on, const int64_t *d_hist,
                                   const int32_t *d_hist_off, const int64_t *d_bias_ids, const float *d_bias_vals,
                                   const int32_t *d_bias_off, void *d_workspace, int64_t workspace_bytes, void *stream,
                                   float *d_summary) {
    g_err[0] = 0;
    if (!d_logits || !d_summary || B < 0 || V_local <= 0 || row_stride < V_local || col0 < 0 ||
        (long long)col0 + V_local > V_global)
        return fail(MOLLA_ERR_ARGUMENT, "bad arguments to the sharded stage 1%s");
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V_local, 0)) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    BatchArgs a = shard_args(d_logits, row_stride, B, V_local, d_temperature, d_top_k, d_top_p, d_min_p, d_typical_p,
                             d_repeat_penalty, d_frequency_penalty, d_presence_penalty, d_window_on, nullptr, nullptr,
                             d_hist, d_hist_off, d_bias_ids, d_bias_vals, d_bias_off);
    a.mode = 1; a.col0 = col0; a.Vg = V_global; a.sa_out = d_summary;
    return launch_rows(a, d_workspace, (cudaStream_t)stream);
}

int32_t molla_sample_shard_merge(int32_t B, int32_t V_global, int32_t world, int32_t rank, const float *d_temperature,
                                 const int32_t *d_top_k, const float *d_gathered_summaries, void *stream,
                                 float *d_global, int32_t *d_tokens, uint32_t *d_row_status) {
    g_err[0] = 0;
    if (B < 0 || V_global <= 0 || world < 1 || world > NWARP || rank < 0 || rank >= world || !d_gathered_summaries || !d_global)
        return fail(MOLLA_ERR_ARGUMENT, "bad arguments to the sharded merge (at most 16 shards)%s");
    if (B == 0) return MOLLA_OK;
    shard_merge_kernel<<<(B + 127) / 128, 128, 0, (cudaStream_t)stream>>>(B, V_global, world, rank, d_temperature, d_top_k,
                                                                       d_gathered_summaries, d_global, d_tokens, d_row_status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "merge launch failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

int32_t molla_sample_shard_stage_b(const float *d_logits, int64_t row_stride, int32_t B, int32_t V_local, int32_t col0,
                                   int32_t V_global, const float *d_temperature, const int32_t *d_top_k,
                                   const float *d_top_p, const float *d_min_p, const float *d_typical_p,
                                   const float *d_repeat_penalty, const float *d_frequency_penalty,
                                   const float *d_presence_penalty, const uint8_t *d_window_on, const int64_t *d_hist,
                                   const int32_t *d_hist_off, const int64_t *d_bias_ids, const float *d_bias_vals,
                                   const int32_t *d_bias_off, const float *d_global, int32_t list_cap, void *d_workspace,
                                   int64_t workspace_bytes, void *stream, uint64_t *d_list, int32_t *d_count) {
    g_err[0] = 0;
    if (!d_logits || !d_global || !d_list || !d_count || B < 0 || V_local <= 0 || row_stride < V_local || list_cap < 1 ||
        col0 < 0 || (long long)col0 + V_local > V_global)
        return fail(MOLLA_ERR_ARGUMENT, "bad arguments to the sharded stage 2%s");
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V_local, 0)) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    BatchArgs a = shard_args(d_logits, row_stride, B, V_local, d_temperature, d_top_k, d_top_p, d_min_p, d_typical_p,
                             d_repeat_penalty, d_frequency_penalty, d_presence_penalty, d_window_on, nullptr, nullptr,
                             d_hist, d_hist_off, d_bias_ids, d_bias_vals, d_bias_off);
    a.mode = 2; a.col0 = col0; a.Vg = V_global; a.sb_in = d_global;
    a.sb_list = (unsigned long long *)d_list; a.sb_count = d_count; a.list_cap = list_cap;
    return launch_rows(a, d_workspace, (cudaStream_t)stream);
}

int32_t molla_sample_shard_stage_c(int32_t B, int32_t V_global, const float *d_temperature, const int32_t *d_top_k,
                                   const float *d_top_p, const float *d_min_p, const float *d_typical_p,
                                   const uint64_t *d_seed, const uint64_t *d_drawn, const float *d_global, int32_t world,
                                   int32_t list_cap, const uint64_t *d_lists, const int32_t *d_counts, void *d_workspace,
                                   int64_t workspace_bytes, void *stream, int32_t *d_tokens, uint32_t *d_row_status,
                                   float *d_diag) {
    g_err[0] = 0;
    if (!d_global || !d_lists || !d_counts || !d_tokens || !d_row_status || B < 0 || V_global <= 0 || world < 1 ||
        world > NWARP || list_cap < 1)
        return fail(MOLLA_ERR_ARGUMENT, "bad arguments to the sharded stage 3 (at most 16 shards)%s");
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V_global, 0)) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    BatchArgs a = shard_args(nullptr, V_global, B, V_global, d_temperature, d_top_k, d_top_p, d_min_p, d_typical_p, nullptr,
                             nullptr, nullptr, nullptr, d_seed, d_drawn, nullptr, nullptr, nullptr, nullptr, nullptr);
    a.mode = 3; a.col0 = 0; a.Vg = V_global; a.sb_in = d_global; a.world = world; a.list_cap = list_cap;
    a.sc_list = (const unsigned long long *)d_lists; a.sc_count = d_counts;
    a.tokens = d_tokens; a.row_status = d_row_status; a.diag = d_diag;
    return launch_rows(a, d_workspace, (cudaStream_t)stream);
}

// ---- host-buffer form ---------------------------------------------------------
namespace {
constexpr int CL_MAX_DEVICES_HOST = 64;
// The library's own copy stream and events for the host-buffer form, one set per device and per
// calling thread (calls from different threads never share them).
struct CopyLane {
    cudaStream_t stream = nullptr;
    cudaEvent_t ready = nullptr;
    cudaEvent_t arrived[8] = {};
    bool ok = false;
};
CopyLane *copy_lane() {
    static thread_local CopyLane lanes[CL_MAX_DEVICES_HOST];
    static thread_local bool tried[CL_MAX_DEVICES_HOST] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= CL_MAX_DEVICES_HOST) return nullptr;
    CopyLane &l = lanes[dev];
    if (!tried[dev]) {
        tried[dev] = true;
        bool ok = cudaStreamCreateWithFlags(&l.stream, cudaStreamNonBlocking) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&l.ready, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; i < 8 && ok; i++) ok = cudaEventCreateWithFlags(&l.arrived[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) (void)cudaGetLastError();
        l.ok = ok;
    }
    return l.ok ? &l : nullptr;
}
inline size_t al256(size_t n) { return (n + 255) & ~(size_t)255; }
struct HostLayout {
    size_t logits, f[8], win, seed, drawn, k, hist, hist_off, bias_ids, bias_vals, bias_off;
    size_t tokens, status, chosen, top_ids, top_lps, total, inner;
};
HostLayout host_layout(int B, int V, long long n_hist, long long n_bias, int top_n, int sms) {
    HostLayout L;
    size_t o = al256(batch_workspace_bytes(B, V, sms));  // the batched call's own workspace comes first
    L.inner = o;
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
    const int sms = sm_count();
    if (sms <= 0) return fail(MOLLA_ERR_CUDA, "cannot query the device%s");
    return (int64_t)host_layout(B, V, n_hist, n_bias, top_n, sms).total;
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
    // the ragged windows and bias lists: offsets that start at zero and never go back
    for (int pass = 0; pass < 2; pass++) {
        const int32_t *off = pass ? bias_off : hist_off;
        if (!off) continue;
        if (off[0] != 0) return fail(MOLLA_ERR_ARGUMENT, "an offset array has to start at zero%s");
        for (int r = 0; r < B; r++)
            if (off[r + 1] < off[r]) return fail(MOLLA_ERR_ARGUMENT, "an offset array has to be non-decreasing%s");
    }
    const long long n_hist = hist_off ? hist_off[B] : 0, n_bias = bias_off ? bias_off[B] : 0;
    for (long long j = 0; j < n_bias; j++)
        if (bias_ids[j] < 0 || bias_ids[j] >= V) return fail(MOLLA_ERR_CONFIG, "a logit bias names a token outside the vocabulary%s");
    const int sms = sm_count();
    if (sms <= 0) return fail(MOLLA_ERR_CUDA, "cannot query the device%s");
    const HostLayout L = host_layout(B, V, n_hist, n_bias, top_n, sms);
    if (!d_workspace || workspace_bytes < (int64_t)L.total) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    char *w = (char *)d_workspace;
    cudaStream_t st = (cudaStream_t)stream;
    // A large block goes up in pieces on a stream of the library's own (one per device, made on first
    // use) while the pieces that have arrived are sampled on the caller's stream; a small one in one go.
    constexpr int MAXPIECE = 8;
    int npiece = 1;
    if ((size_t)B * V * 4 >= ((size_t)32 << 20) && B >= 2 * MAXPIECE) npiece = MAXPIECE;
    CopyLane *lane = npiece > 1 ? copy_lane() : nullptr;
    if (!lane) npiece = 1;
    cudaError_t e = cudaSuccess;
    if (npiece == 1)
        e = cudaMemcpy2DAsync(w + L.logits, (size_t)V * 4, h_logits, (size_t)row_stride * 4, (size_t)V * 4, (size_t)B, cudaMemcpyHostToDevice, st);
    const float *fsrc[8] = {temperature, top_p, min_p, typical_p, repeat_penalty, frequency_penalty, presence_penalty, nullptr};
    for (int i = 0; i < 7 && e == cudaSuccess; i++)
        if (fsrc[i]) e = cudaMemcpyAsync(w + L.f[i], fsrc[i], (size_t)B * 4, cudaMemcpyHostToDevice, st);
    auto up = [&](size_t off, const void *src, size_t bytes) { if (src && bytes && e == cudaSuccess) e = cudaMemcpyAsync(w + off, src, bytes, cudaMemcpyHostToDevice, st); };
    up(L.k, top_k, (size_t)B * 4); up(L.win, window_on, (size_t)B); up(L.seed, seed, (size_t)B * 8); up(L.drawn, drawn, (size_t)B * 8);
    up(L.hist, hist, (size_t)n_hist * 8); up(L.hist_off, hist_off, (size_t)(B + 1) * 4);
    up(L.bias_ids, bias_ids, (size_t)n_bias * 8); up(L.bias_vals, bias_vals, (size_t)n_bias * 4); up(L.bias_off, bias_off, (size_t)(B + 1) * 4);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "host to device copy failed: %s", cudaGetErrorString(e));
    // rows [r0, r1) of the block on the device: per-row arrays advance by r0 elements (the window and
    // bias offsets are absolute, so their arrays only shift)
    auto dp = [&](size_t off, const void *src, size_t elem, int r0) -> void * { return src ? (void *)(w + off + elem * (size_t)r0) : nullptr; };
    auto sample_rows = [&](int r0, int r1) -> int {
        return molla_sample_batch(
            (const float *)(w + L.logits) + (size_t)r0 * V, V, r1 - r0, V, (const float *)dp(L.f[0], temperature, 4, r0),
            (const int32_t *)dp(L.k, top_k, 4, r0), (const float *)dp(L.f[1], top_p, 4, r0), (const float *)dp(L.f[2], min_p, 4, r0),
            (const float *)dp(L.f[3], typical_p, 4, r0), (const float *)dp(L.f[4], repeat_penalty, 4, r0),
            (const float *)dp(L.f[5], frequency_penalty, 4, r0), (const float *)dp(L.f[6], presence_penalty, 4, r0),
            (const uint8_t *)dp(L.win, window_on, 1, r0), (const uint64_t *)dp(L.seed, seed, 8, r0),
            (const uint64_t *)dp(L.drawn, drawn, 8, r0), (const int64_t *)dp(L.hist, hist, 8, 0),
            (const int32_t *)dp(L.hist_off, hist_off, 4, r0), (const int64_t *)dp(L.bias_ids, bias_ids, 8, 0),
            (const float *)dp(L.bias_vals, bias_vals, 4, 0), (const int32_t *)dp(L.bias_off, bias_off, 4, r0), top_n, w,
            (int64_t)L.inner, stream, (int32_t *)(w + L.tokens) + r0, h_chosen_logprob ? (float *)(w + L.chosen) + r0 : nullptr,
            top_n > 0 ? (int32_t *)(w + L.top_ids) + (size_t)r0 * top_n : nullptr,
            top_n > 0 ? (float *)(w + L.top_lps) + (size_t)r0 * top_n : nullptr, (uint32_t *)(w + L.status) + r0, nullptr);
    };
    int rc = MOLLA_OK;
    if (npiece == 1) {
        rc = sample_rows(0, B);
    } else {
        // the copies start once everything queued on the caller's stream so far is done (the workspace may still be in use)
        e = cudaEventRecord(lane->ready, st);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(lane->stream, lane->ready, 0);
        for (int c = 0; c < npiece && e == cudaSuccess; c++) {
            const int r0 = (int)((long long)B * c / npiece), r1 = (int)((long long)B * (c + 1) / npiece);
            e = cudaMemcpy2DAsync(w + L.logits + (size_t)r0 * V * 4, (size_t)V * 4, h_logits + (size_t)r0 * row_stride,
                                  (size_t)row_stride * 4, (size_t)V * 4, (size_t)(r1 - r0), cudaMemcpyHostToDevice, lane->stream);
            if (e == cudaSuccess) e = cudaEventRecord(lane->arrived[c], lane->stream);
        }
        if (e != cudaSuccess) { cudaStreamSynchronize(lane->stream); return fail(MOLLA_ERR_CUDA, "host to device copy failed: %s", cudaGetErrorString(e)); }
        for (int c = 0; c < npiece && rc == MOLLA_OK; c++) {
            const int r0 = (int)((long long)B * c / npiece), r1 = (int)((long long)B * (c + 1) / npiece);
            e = cudaStreamWaitEvent(st, lane->arrived[c], 0);
            if (e != cudaSuccess) { rc = fail(MOLLA_ERR_CUDA, "waiting for a piece of the block failed: %s", cudaGetErrorString(e)); break; }
            rc = sample_rows(r0, r1);
        }
        if (rc != MOLLA_OK) cudaStreamSynchronize(lane->stream);  // no copy of this call outlives it
    }
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
    // a row the library did not answer (token -1) fails the call, as `pick` would have raised
    for (int r = 0; r < B; r++) {
        if (h_row_status[r] & MOLLA_ROW_UNSUPPORTED)
            return fail(MOLLA_ERR_DEVICE, "a row asked for a filter combination the library does not do yet (MOLLA_ROW_UNSUPPORTED)%s");
        if (h_row_status[r] & (MOLLA_ROW_LOAD_TIMEOUT | MOLLA_ROW_DEGENERATE | MOLLA_ROW_INVALID_CONFIG | MOLLA_ROW_SHARD_OVERFLOW | MOLLA_ROW_EMPTY))
            return fail(MOLLA_ERR_DEVICE, "a row reported an error in its status word%s");
    }
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
    if (!d_workspace || workspace_bytes < molla_sample_workspace_bytes(B, V, 0)) return fail(MOLLA_ERR_WORKSPACE, "workspace missing or too small%s");
    if (B == 0) return MOLLA_OK;
    BatchArgs a;
    memset(&a, 0, sizeof(a));
    a.logits = d_logits; a.row_stride = row_stride; a.B = B; a.V = V;
    a.repeat_penalty = d_repeat_penalty; a.frequency_penalty = d_frequency_penalty;
    a.presence_penalty = d_presence_penalty; a.window_on = d_window_on;
    a.hist = (const long long *)d_hist; a.hist_off = d_hist_off;
    a.bias_ids = (const long long *)d_bias_ids; a.bias_vals = d_bias_vals; a.bias_off = d_bias_off;
    a.penalised = d_out; a.penalised_only = 1;
    return launch_rows(a, d_workspace, (cudaStream_t)stream);
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
                                                          nullptr, d_out, nullptr, 0, 0.0f);
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

int32_t molla_sample_logf(const float *d_x, int64_t n, void *stream, float *d_out) {
    g_err[0] = 0;
    if (!d_x || !d_out || n < 0) return fail(MOLLA_ERR_ARGUMENT, "bad arguments to logf%s");
    if (n == 0) return MOLLA_OK;
    long long blocks = (n + 255) / 256;
    logf_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(d_x, n, d_out);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "logf launch failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

#ifdef MOLLA_SAMPLE_TESTING
void molla_sample_debug_profile(void *d_stamps) { g_prof = (long long *)d_stamps; }
void molla_sample_debug_knobs(int32_t k) { g_knobs = k; }
void molla_sample_debug_topk(void *d_ids, int32_t cap) { g_topk = (int *)d_ids; g_topk_cap = d_ids ? cap : 0; }
#endif

int32_t molla_sample_sync(void *stream) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return fail(MOLLA_ERR_CUDA, "stream synchronize failed: %s", cudaGetErrorString(e));
    return MOLLA_OK;
}

}  // extern "C"
