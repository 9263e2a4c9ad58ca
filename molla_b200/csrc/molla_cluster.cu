// The row kernel of the ordinary entry points: one logit row per thread-block cluster.
//
// A row of up to 8 x 38400 logits is split into contiguous column ranges, one per thread block
// of the cluster, and every block keeps its range in shared memory from the moment the bulk
// copies (TMA without a tensor map, never multicast) land until the row's token is known. HBM
// sees every logit once and no pass after the first touches global memory: bias and penalties
// are written into the resident range, the maximum is taken from it, the exponentials replace
// the logits in place (what cannot matter to any sum becomes zero, which adds nothing to a
// sequential fp32 sum), and the exact softmax denominator, the sorted head and the walks past
// it all read shared memory. The range's position is the token id, so nothing carries indices.
//
// What the blocks of a cluster have to tell each other (the range maxima, a lower bound of the
// running sum before each range, the threads' maxima for the head threshold, the estimated
// range sums, the exact running sum handed from range to range, the head's candidates, the
// bin tables of a walk) goes through distributed shared memory between cluster barriers. All
// blocks of a cluster take the same branches: every decision is made from values all of them
// hold.
//
// The device functions this kernel shares with the streaming kernel (the exact sum, the bin
// search, the sorted walk, typical-p) come from molla_exact.cuh.
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdio.h>

#include "molla_exact.cuh"
#include "molla_cluster.h"

namespace cg = cooperative_groups;

namespace {

constexpr int CL_MAX_G = 8;                  // thread blocks per cluster at most (the portable limit)
constexpr int CL_LMAX = 75;                  // logits per thread at most (odd: conflict-free strides)
constexpr int CL_CAPF = NT * CL_LMAX;        // logits per thread block at most: 38400 (150 KB)
constexpr int CL_PIECE = 4096;               // floats per bulk copy
constexpr int CL_HEADC = 2048;                // candidates of the sorted head at most (the buffers of a gathered bin hold as many)
constexpr int CL_HEAD_NEED = 1026;            // the sorted head covers top-k + 1 up to this many: a top-k up to 1025 never walks
constexpr int TIE_CAP = 64;                   // rounding ties a walk resolves by parity; more send it the slow way
constexpr int TBINS = NT;                    // bins of the threads' maxima by distance below the row's maximum
constexpr float TRES = (float)(NT / 32);     // bins per unit of logit: the bins cover 32 units

// Profiling stamps exist in the testing build only (per row 32 slots of clock readings and counts).
#ifdef MOLLA_SAMPLE_TESTING
#define CSTAMP(i) do { if (a.prof && leader && c.tid == 0) a.prof[(long long)r * 32 + (i)] = clock64(); } while (0)
#define CPROF_SLOTS(cond, first) ((a.prof && (cond)) ? a.prof + (long long)r * 32 + (first) : nullptr)
#else
#define CSTAMP(i) do { } while (0)
#define CPROF_SLOTS(cond, first) nullptr
#endif

struct __align__(16) AuxC {
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
            unsigned int hq[NBINS];
            unsigned int hqh[NBINS];
            unsigned int hc[NBINS];
        } h;
    } u;
    unsigned long long cand[NC];   // first the hash of the patched tokens, then the head / a bin's candidates
    float pc[NC];
    float pre[CL_HEADC];
    unsigned int hidx[CL_HEADC];
    double wsd[2 * (NWARP + 1)];
    unsigned long long wsu[NWARP + 1];
    float wsf[NWARP + 1];
    int wsi[NWARP + 1];
    int nseg, ncand, evt_thread, specbin, hit_bin;
    unsigned long long hit_qbefore, hit_cbefore, tot_q, tot_c;
    float walk_s; int walk_found, walk_idx, walk_slow;
    float b_s; unsigned int b_tau; int b_event; int b_idx; float b_p; long long b_pos; int b_aux;
    float b_sum; float b_target;
    uint64_t mbar;
    unsigned int thist[TBINS];           // the threads' maxima by distance below the block's maximum
    // what the blocks of the cluster write into each other (slot = the writer's rank)
    float x1_max[CL_MAX_G]; int x1_idx[CL_MAX_G]; int x1_eq[CL_MAX_G]; unsigned int x1_status[CL_MAX_G];
    float x2_total[CL_MAX_G];
    double x3_tot[CL_MAX_G]; int x3_n[CL_MAX_G];
    int x4_n[CL_MAX_G]; unsigned long long x5_key[CL_MAX_G];
    float ch_s; int ch_found, ch_at, ch_slow;   // the exact sum on its way from range to range
    int ch_flag;                                 // which hand-over of the row has arrived (the writer releases, thread 0 acquires)
    // elements of a walk that would round on a tie: their keys, bins, the mass before them
    long long rx[8];          // words fetched from the leader for the whole block
    int ngath, ngath_over;   // a bin's entries collected by this block; blocks whose own buffer overflowed (leader's)
    int ntie[2]; unsigned long long tkey[TIE_CAP]; int tbin[TIE_CAP]; unsigned int tpq_lo[TIE_CAP], tpq_hi[TIE_CAP]; unsigned long long tpqm[TIE_CAP], tabove[TIE_CAP], tc[TIE_CAP];
    unsigned int tbits[NBINS / 32];
    int r_kind; int r_idx; float r_s; long long r_pos; unsigned int r_status;  // the leader's word after the head
};

struct CtxC {
    int tid, lane, warp;
    AuxC *A;
    unsigned int status;
};

struct ClWalk {
    float s; long long pos; unsigned int tau;
    int event; int idx; float p; int tie;
};

struct ClGeo {          // where this thread block stands
    int G, rank, c0, nloc, L;
};

// The exact sequential fp32 sum of the cluster's row (values `bits`, zero = absent), in vocabulary
// order: every block builds the tables of its range from an estimate of the sum before it, then
// the exact running sum travels from range to range. With `locate`, stops at the first entry
// whose running sum exceeds `target`; its token id is returned in `at`.
struct ClSum { float s; int found; int at; int slow; bool timeout; };

// cluster-scope release / acquire of one word of (possibly another block's) shared memory
__device__ __forceinline__ void st_release_cluster(int *p, int v) {
    asm volatile("st.release.cluster.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_cluster(const int *p) {
    int v;
    asm volatile("ld.acquire.cluster.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// `epoch` counts the sums of a row (the same in every block): the hand-over from range to range
// is a word released into the next block's shared memory, on which only that block's thread 0
// waits (with a bound); everybody else waits once, at the cluster barrier after the last range.
__device__ ClSum cluster_exact_sum(cg::cluster_group &cl, CtxC &c, const ClGeo &g, const unsigned int *bits,
                                   bool locate, float target, int &epoch, long long *stamps = nullptr, long long *stamps2 = nullptr) {
    AuxC *A = c.A;
    IN_SHARED(A);
    IN_SHARED(bits);
    ValBits vals{bits};
    epoch++;
    __syncthreads();
    const float csum = p1_csum(vals, g.nloc, g.L, c.tid);
    double tot;
    const double ex = block_excl_scan<double>((double)csum, A->wsd, &tot);
    if (c.tid < g.G) cl.map_shared_rank(A, c.tid)->x3_tot[g.rank] = tot;
    cl.sync();
    double sbase = 0.0;
    for (int h = 0; h < g.rank; h++) sbase += A->x3_tot[h];
    if (stamps && c.tid == 0) stamps[0] = clock64();
    p1_tables(c, vals, g.nloc, g.L, csum, sbase + ex);
    if (stamps && c.tid == 0) stamps[1] = clock64();
    if (c.tid == 0) {
        Walker w;
        int timed_out = 0;
        if (g.rank == 0) { w.s = 0.0f; w.found = 0; w.at = -1; w.slow = 0; }
        else {
            bool here = false;
            for (int spin = 0; spin < (1 << 22); spin++)
                if (ld_acquire_cluster(&A->ch_flag) == epoch) { here = true; break; }
            if (!here) timed_out = 4;
            w.s = A->ch_s; w.found = A->ch_found; w.at = A->ch_at; w.slow = A->ch_slow;
        }
        if (!(locate && w.found)) {
            const long long tw0 = clock64();
            p1_walk(c, vals, g.nloc, g.L, locate, target, w);
            if (w.found) w.at += g.c0;
            if (stamps2) { stamps2[g.rank] = clock64() - tw0; stamps2[4 + g.rank] = w.nsim * 100000ll + w.nel; stamps2[8 + g.rank] = A->nseg; }
        }
        w.slow |= timed_out;
        if (g.rank + 1 < g.G) {
            AuxC *nx = cl.map_shared_rank(A, g.rank + 1);
            nx->ch_s = w.s; nx->ch_found = w.found; nx->ch_at = w.at; nx->ch_slow = w.slow;
            st_release_cluster(&nx->ch_flag, epoch);
        } else {
            for (int o = 0; o < g.G; o++) {
                AuxC *ox = cl.map_shared_rank(A, o);
                ox->ch_s = w.s; ox->ch_found = w.found; ox->ch_at = w.at; ox->ch_slow = w.slow;
            }
        }
    }
    cl.sync();
    ClSum out;
    out.s = A->ch_s; out.found = A->ch_found; out.at = A->ch_at; out.slow = A->ch_slow & 1; out.timeout = (A->ch_slow & 4) != 0;
    return out;
}

// Token id of the (nth+1)-th entry, in vocabulary order, whose bits equal `eb` (eb below tau).
__device__ int cluster_nth_equal(cg::cluster_group &cl, CtxC &c, const ClGeo &g, const unsigned int *bits,
                                 unsigned int eb, int nth) {
    AuxC *A = c.A;
    IN_SHARED(A);
    IN_SHARED(bits);
    const int i0 = min(g.nloc, c.tid * g.L), i1 = min(g.nloc, (c.tid + 1) * g.L);
    int cnt = 0;
    for (int i = i0; i < i1; i++) cnt += (bits[i] == eb) ? 1 : 0;
    int tot;
    const int ex = block_excl_scan<int>(cnt, A->wsi, &tot);
    if (c.tid < g.G) cl.map_shared_rank(A, c.tid)->x4_n[g.rank] = tot;
    if (c.tid == 0) A->r_idx = -1;
    cl.sync();
    int base = 0;
    for (int h = 0; h < g.rank; h++) base += A->x4_n[h];
    if (nth >= base + ex && nth < base + ex + cnt) {
        int seen = base + ex;
        for (int i = i0; i < i1; i++) {
            if (bits[i] == eb) {
                if (seen == nth) {
                    for (int o = 0; o < g.G; o++) cl.map_shared_rank(A, o)->r_idx = g.c0 + i;
                    break;
                }
                seen++;
            }
        }
    }
    cl.sync();
    return A->r_idx;
}

// A few words of the leader's memory for the whole block: threads 0..n-1 fetch one each into
// `A->rx` (a load from another block's memory by every thread would queue up there).
template <class F>
__device__ __forceinline__ void fetch_from_leader(CtxC &c, int n, F word) {
    __syncthreads();
    if (c.tid < n) c.A->rx[c.tid] = word(c.tid);
    __syncthreads();
}

// The descending walk past the sorted head (sample.mojo:492-506 and :580-590) over the cluster's
// row of probabilities. State as in `descend`: exact running sum, elements consumed, and tau:
// everything with probability bits >= tau is consumed. Every phase histograms what remains by
// value bin (each block its range; the tables are added up across the cluster as they are
// read), consumes whole bins up to the first one holding an event, gathers that bin into the
// leader's candidate buffer, and the leader sorts it and adds it element by element.
//
// An element whose addition would be a rounding tie (its value is an odd multiple of half the
// running sum's unit) rounds up or down with the parity of the sum before it. Such elements do
// not stop a phase: they are listed, a second pass adds up what precedes each of them inside
// its own bin, and one thread then resolves them from the top down, each from the exact integer
// sum before it; their contributions go into their bins' masses before the event is searched.
// Where a walk's last phase began. The draw walk adds up the same elements in the same order as
// the cut walk before it, so when its target is not reached before that point it starts there,
// on the bin tables that are still standing (merged, at the leader), and skips the passes that
// built them.
struct ClResume {
    int valid;
    float s; long long pos; unsigned int tau;
    int lvl; unsigned int lo; int shift; int tie_mode; int ntie;
};

__device__ void descend_cluster(cg::cluster_group &cl, CtxC &c, const ClGeo &g, const unsigned int *bits,
                                ClWalk &w, float x_ge, float x_gt, long long nstop, ClResume &rs, bool try_resume,
                                long long *dbg = nullptr) {
    AuxC *A = c.A;
    IN_SHARED(A);
    IN_SHARED(bits);
    AuxC *lead = cl.map_shared_rank(A, 0);
    const bool leader = g.rank == 0;
    const bool counting = nstop >= 0;
    int lvl = 1;
    unsigned int lo = 0u;
    int shift = BIN_SHIFT;
    bool tie_mode = true;
    // (every block holds the same `rs`: its fields are values all blocks computed alike)
    const bool resumed = try_resume && rs.valid && !counting && x_ge >= 3.0e38f && !(x_gt < rs.s);
    if (resumed) {
        w.s = rs.s; w.pos = rs.pos; w.tau = rs.tau;
        lvl = rs.lvl; lo = rs.lo; shift = rs.shift; tie_mode = rs.tie_mode != 0;
    }
    if (c.tid == 0) { A->ntie[0] = 0; A->ntie[1] = 0; }
    for (int phase = 0; phase < 8192; phase++) {
        const bool reuse = resumed && phase == 0;  // this phase's tables stand already
        cl.sync();  // nobody still reads the tables or the leader's results of the phase before
        long long tp0 = clock64();
#define DT(k) do { if (dbg && c.tid == 0) { const long long t_ = clock64(); dbg[k] += t_ - tp0; tp0 = t_; } } while (0)
        if (!reuse) {
            for (int i = c.tid; i < NBINS; i += NT) { A->u.h.hq[i] = 0u; A->u.h.hqh[i] = 0u; A->u.h.hc[i] = 0u; }
            for (int i = c.tid; i < NBINS / 32; i += NT) A->tbits[i] = 0u;
            rs.valid = 1; rs.s = w.s; rs.pos = w.pos; rs.tau = w.tau;
            rs.lvl = lvl; rs.lo = lo; rs.shift = shift; rs.tie_mode = tie_mode ? 1 : 0; rs.ntie = 0;
        }
        if (c.tid == 0) {
            if (!reuse) A->specbin = -1;
            A->ncand = 0; A->ngath = 0; A->ngath_over = 0; A->ntie[(phase + 1) & 1] = 0;  // the other blocks add to this phase's counter already
        }
        __syncthreads();
        const bool have_s = w.s > 0.0f;
        const int j = have_s ? fexpo(w.s) : 0;
        const bool binade_ok = have_s && j >= -100 && j <= 100;
        const float Cm = __fmul_rn(1.5f, fpow2(j)), halfu = fpow2(j - 24), bigthr = fpow2(j - 1);
        const float inv_u = fpow2(23 - j);
        const unsigned int cm_bits = __float_as_uint(Cm);
        const bool ties_listed = tie_mode && lvl == 1 && binade_ok;
        int ntie = rs.ntie;
        if (!reuse) {
        // Every thread's elements four at a time. The common case (an element that simply adds its
        // mass to its bin) runs without a branch; elements that need care and rounding ties are rare
        // and a warp turns to them only when one of its lanes has met one.
        const int ntie_slot = phase & 1;
        const unsigned int wtau = w.tau;
        const int nloc = g.nloc;
        const bool count_all = counting || !binade_ok;
        for (int i0 = c.tid - c.lane; i0 < nloc; i0 += 4 * NT) {  // (the same trips for all lanes of a warp)
            const int i4 = i0 + c.lane;
            unsigned int ebs[4];
            bool rare = false;
#pragma unroll
            for (int u = 0; u < 4; u++) ebs[u] = (i4 + u * NT < nloc) ? bits[i4 + u * NT] : 0u;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const unsigned int eb = ebs[u];
                const bool live = eb != 0u && eb < wtau && eb >= lo;
                const int bin = (int)((eb - lo) >> shift);
                const float p = __uint_as_float(eb);
                const float tq = __fadd_rn(p, Cm);
                const float q = __fsub_rn(tq, Cm);
                const float rr = __fsub_rn(p, q);
                const bool special = (fabsf(rr) == halfu) || (p >= bigthr);
                // q in units: below bigthr, p + Cm stays in Cm's binade, whose unit is the sum's, so
                // the difference of the two bit patterns is the count (a conversion would issue at
                // a quarter of the rate)
                const unsigned int qu = __float_as_uint(tq) - cm_bits;
                if (live && count_all) sred_add(&A->u.h.hc[bin], 1u);
                const bool plain = live && binade_ok && !special;
                if (plain) sred_add(&A->u.h.hq[bin], qu & MASS_LO_MASK);
                if (plain && (qu >> MASS_SPLIT)) sred_add(&A->u.h.hqh[bin], qu >> MASS_SPLIT);
                rare |= live && binade_ok && special;
            }
            if (__any_sync(0xffffffffu, rare)) {
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const unsigned int eb = ebs[u];
                    if (!(eb != 0u && eb < wtau && eb >= lo)) continue;
                    const int bin = (int)((eb - lo) >> shift);
                    const float p = __uint_as_float(eb);
                    const float q = __fsub_rn(__fadd_rn(p, Cm), Cm);
                    const bool tie = fabsf(__fsub_rn(p, q)) == halfu;
                    if ((p >= bigthr) || (tie && !ties_listed)) { sred_max(&A->specbin, bin); continue; }
                    if (tie) {
                        const int pos = atomicAdd(&lead->ntie[ntie_slot], 1);
                        if (pos < TIE_CAP) { lead->tkey[pos] = make_key(eb, g.c0 + i4 + u * NT); lead->tbin[pos] = bin; }
                    }
                }
            }
        }
        cl.sync();
        fetch_from_leader(c, 1, [&](int) { return (long long)lead->ntie[ntie_slot]; });
        ntie = ties_listed ? (int)A->rx[0] : 0;
        rs.ntie = ntie;
        if (dbg && c.tid == 0) { dbg[0] += 1; dbg[1] += ntie; }
        DT(3);
        if (ntie > TIE_CAP) { tie_mode = false; c.status |= MOLLA_ROW_SLOW_PATH; continue; }  // too many: they stop phases instead
        if (ntie > 0) {
            // what precedes each listed element inside its own bin (descending value, then ascending id)
            if (c.tid < ntie) {
                const int b = lead->tbin[c.tid];
                A->tkey[c.tid] = lead->tkey[c.tid]; A->tbin[c.tid] = b; A->tpq_lo[c.tid] = 0u; A->tpq_hi[c.tid] = 0u;
                sred_or(&A->tbits[b >> 5], 1u << (b & 31));
            }
            __syncthreads();
            // the bins that hold a listed element span a short range: a compare against it keeps
            // nearly every element out of the slower path
            int tb_lo = NBINS, tb_hi = -1;
            for (int t = 0; t < ntie; t++) { tb_lo = min(tb_lo, A->tbin[t]); tb_hi = max(tb_hi, A->tbin[t]); }
            const unsigned int tb_span = (unsigned int)(tb_hi - tb_lo);

            const unsigned int wtau2 = w.tau;
            for (int i0 = c.tid - c.lane; i0 < g.nloc; i0 += 4 * NT) {
                const int i4 = i0 + c.lane;
                unsigned int ebs[4];
                bool near = false;
#pragma unroll
                for (int u = 0; u < 4; u++) ebs[u] = (i4 + u * NT < g.nloc) ? bits[i4 + u * NT] : 0u;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const unsigned int eb = ebs[u];
                    const int bin = (int)((eb - lo) >> shift);
                    near |= eb != 0u && eb < wtau2 && eb >= lo && (unsigned int)(bin - tb_lo) <= tb_span;
                }
                if (!__any_sync(0xffffffffu, near)) continue;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const unsigned int eb = ebs[u];
                    if (eb == 0u || eb >= wtau2 || eb < lo) continue;
                    const int bin = (int)((eb - lo) >> shift);
                    if (!((A->tbits[bin >> 5] >> (bin & 31)) & 1u)) continue;
                    const float p = __uint_as_float(eb);
                    const float tq = __fadd_rn(p, Cm);
                    const float q = __fsub_rn(tq, Cm);
                    const float rr = __fsub_rn(p, q);
                    if (fabsf(rr) == halfu || p >= bigthr) continue;
                    const unsigned int qu = __float_as_uint(tq) - cm_bits;
                    const unsigned long long key = make_key(eb, g.c0 + i4 + u * NT);
                    for (int t = 0; t < ntie; t++)
                        if (A->tbin[t] == bin && key > A->tkey[t] && qu) {  // two halves, as in the bin tables
                            sred_add(&A->tpq_lo[t], qu & MASS_LO_MASK);
                            if (qu >> MASS_SPLIT) sred_add(&A->tpq_hi[t], qu >> MASS_SPLIT);
                        }
                }
            }
            cl.sync();
        }
        }  // (!reuse)
        DT(4);
        // The leader adds the other blocks' tables to its own (whole rows of bins at a time, so that
        // the loads from the other blocks' memory are few and wide), searches the event bin and
        // tells everybody.
        BinQuery qy;
        qy.bin_hi = NBINS; qy.spec_bits = nullptr;
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
        if (!reuse && g.G > 1) {
            // every block adds up its share of the bins over all blocks (few, wide loads from the
            // other blocks' memory, spread over all of them) and puts the sums into the leader's tables
            uint4 *mine = reinterpret_cast<uint4 *>(&A->u.h);
            uint4 *dst = reinterpret_cast<uint4 *>(&lead->u.h);
            constexpr int NV = 3 * NBINS / 4;  // the three tables, four bins at a time
            const int per = (NV + g.G - 1) / g.G;
            const int v_hi = min(NV, (g.rank + 1) * per);
            for (int v0 = g.rank * per + c.tid; v0 < v_hi; v0 += NT) {
                uint4 acc = mine[v0];
                for (int o = 0; o < g.G; o++) {
                    if (o == g.rank) continue;
                    const uint4 x = reinterpret_cast<const uint4 *>(&cl.map_shared_rank(A, o)->u.h)[v0];
                    acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
                }
                dst[v0] = acc;
            }
            if (!leader && c.tid == 0 && A->specbin >= 0) atomicMax(&lead->specbin, A->specbin);
            cl.sync();
        }
        if (leader) {
            if (reuse) {
                if (c.tid < ntie) A->tc[c.tid] = 0ull;
                __syncthreads();
            } else {
                if (c.tid < ntie) {
                    unsigned long long s_ = 0ull;
                    for (int o = 0; o < g.G; o++) {
                        const AuxC *ox = cl.map_shared_rank(A, o);
                        s_ += (unsigned long long)ox->tpq_lo[c.tid] + ((unsigned long long)ox->tpq_hi[c.tid] << MASS_SPLIT);
                    }
                    A->tpqm[c.tid] = s_; A->tc[c.tid] = 0ull;
                }
                __syncthreads();
            }
            qy.specbin = A->specbin;
            find_event_bin_adj(c, qy,
                [&](int b, unsigned long long &q, unsigned long long &n) {
                    q = (unsigned long long)qy.hq[b] + ((unsigned long long)qy.hqh[b] << MASS_SPLIT);
                    n = qy.hc[b];
                },
                [&](unsigned long long (&q)[BPT], unsigned long long eq) -> bool {
                    if (ntie == 0) return false;
                    // the mass before each listed element: the bins above its own (the thread that
                    // owns the bin knows), what precedes it inside the bin (added up over the blocks)
                    unsigned long long run = eq;
#pragma unroll
                    for (int i = 0; i < BPT; i++) {
                        const int b = NBINS - 1 - BPT * c.tid - i;
                        for (int t = 0; t < ntie; t++)
                            if (A->tbin[t] == b) A->tabove[t] = run;
                        run += q[i];
                    }
                    __syncthreads();
                    if (c.tid == 0) {
                        // from the top down (what lies below an event never matters: the walk stops there)
                        unsigned long long done = 0ull, carried = 0ull;
                        for (int round = 0; round < ntie; round++) {
                            int best = -1;
                            for (int t = 0; t < ntie; t++)
                                if (!((done >> t) & 1ull) && (best < 0 || A->tkey[t] > A->tkey[best])) best = t;
                            done |= 1ull << best;
                            const float p = key_val(A->tkey[best]);
                            const float qf = __fsub_rn(__fadd_rn(p, Cm), Cm);
                            unsigned long long k = (unsigned long long)__float2uint_rn(__fmul_rn(qf, inv_u));
                            if (qf > p) k -= 1ull;  // the multiple of the unit below p
                            const unsigned long long mb = qy.m0 + A->tabove[best] + A->tpqm[best] + carried;
                            if (qy.xq != ~0ull && mb >= qy.xq) break;
                            const unsigned long long ct = k + ((mb + k) & 1ull);
                            A->tc[best] = ct;
                            carried += ct;
                            if (qy.xq != ~0ull && mb + ct >= qy.xq) break;
                        }
                    }
                    __syncthreads();
#pragma unroll
                    for (int i = 0; i < BPT; i++) {
                        const int b = NBINS - 1 - BPT * c.tid - i;
                        for (int t = 0; t < ntie; t++)
                            if (A->tbin[t] == b) q[i] += A->tc[t];
                    }
                    return true;
                });
            if (c.tid < g.G && c.tid > 0) {
                AuxC *ox = cl.map_shared_rank(A, c.tid);
                ox->hit_bin = A->hit_bin; ox->hit_qbefore = A->hit_qbefore; ox->hit_cbefore = A->hit_cbefore;
                ox->tot_q = A->tot_q; ox->tot_c = A->tot_c;
            }
        }
        cl.sync();
        DT(5);
        const int hb = A->hit_bin;
        if (hb < 0) {
            // nothing left in this range triggers an event: consume it whole
            if (binade_ok) w.s = (float)((double)(qy.m0 + A->tot_q) * (double)fpow2(j - 23));
            w.pos += (long long)A->tot_c;
            if (lvl == 1) { w.tau = 0; w.event = EV_EXHAUSTED; cl.sync(); return; }
            w.tau = lo; lvl = 1; lo = 0u; shift = BIN_SHIFT;  // back to the coarse bins below this range
            continue;
        }
        const unsigned long long qb = A->hit_qbefore, cb = A->hit_cbefore;
        const unsigned int blo = lo + ((unsigned int)hb << shift);
        const unsigned long long bhi64 = (unsigned long long)lo + ((unsigned long long)(hb + 1) << shift);
        const unsigned int bhi = bhi64 > 0xFFFFFFFFull ? 0xFFFFFFFFu : (unsigned int)bhi64;
        // The bin's entries: every block collects its own (in the space of the candidates' values),
        // reserves room at the leader with one addition to the leader's counter and copies them over.
        unsigned long long *mybuf = reinterpret_cast<unsigned long long *>(A->pc);
        constexpr int MYCAP = NC / 2;
        const unsigned int gtau = w.tau < bhi ? w.tau : bhi;  // the bin's entries: blo <= value < gtau, and not zero (an absent element)
        for (int i0 = c.tid - c.lane; i0 < g.nloc; i0 += 4 * NT) {  // (the same trips for all lanes of a warp)
            const int i4 = i0 + c.lane;
            unsigned int ebs[4];
            bool any = false;
#pragma unroll
            for (int u = 0; u < 4; u++) ebs[u] = (i4 + u * NT < g.nloc) ? bits[i4 + u * NT] : 0u;
#pragma unroll
            for (int u = 0; u < 4; u++) any |= ebs[u] != 0u && ebs[u] >= blo && ebs[u] < gtau;
            if (!__any_sync(0xffffffffu, any)) continue;  // one bin of 2048: most warps pass most elements by
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const unsigned int eb = ebs[u];
                if (eb != 0u && eb >= blo && eb < gtau) {
                    const int pos = satom_add(&A->ngath, 1);
                    if (pos < MYCAP) mybuf[pos] = make_key(eb, g.c0 + i4 + u * NT);
                }
            }
        }
        __syncthreads();
        const int mine = A->ngath;
        if (c.tid == 0) {
            A->evt_thread = atomicAdd(&lead->ncand, mine);  // (a word that is idle here; the leader's `specbin` has to survive for a resumed walk)
            if (mine > MYCAP) atomicAdd(&lead->ngath_over, 1);  // more than this block could hold: the bin is split further
        }
        __syncthreads();
        const int cbase = A->evt_thread;
        if (mine <= MYCAP && cbase + mine <= NC)
            for (int i = c.tid; i < mine; i += NT) lead->cand[cbase + i] = mybuf[i];
        cl.sync();
        fetch_from_leader(c, 2, [&](int i) { return (long long)(i == 0 ? lead->ncand : lead->ngath_over); });
        const int nb = (int)A->rx[0];
        const bool crowded = nb > NC || A->rx[1] > 0;
        DT(6);
        if (dbg && c.tid == 0) dbg[2] = nb;
        // what lies above the bin is consumed without an event either way
        const float s_bin = binade_ok ? (float)((double)(qy.m0 + qb) * (double)fpow2(j - 23)) : w.s;
        const long long pos_bin = w.pos + ((counting || !binade_ok) ? (long long)cb : 0);
        if (crowded && lvl < 3) {
            w.s = s_bin; w.pos = pos_bin;
            w.tau = bhi < w.tau ? bhi : w.tau;
            lo = blo; shift = (lvl == 1) ? BIN_SHIFT2 : 0; lvl++;
            c.status |= MOLLA_ROW_SLOW_PATH;
            continue;
        }
        if (crowded) {
            // one value, more copies than the buffer holds: add them one at a time (the leader's
            // thread 0), then find which copy, in token order, the event fell on
            c.status |= MOLLA_ROW_SLOW_PATH;
            const float pv = __uint_as_float(blo);
            if (g.rank == 0 && c.tid == 0) {
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
            cl.sync();
            fetch_from_leader(c, 4, [&](int i) {
                return i == 0 ? (long long)lead->b_event : i == 1 ? (long long)lead->b_aux
                     : i == 2 ? (long long)__float_as_int(lead->b_s) : lead->b_pos; });
            const int ev = (int)A->rx[0], at = (int)A->rx[1];
            w.s = __int_as_float((int)A->rx[2]); w.pos = A->rx[3];
            if (ev != EV_NONE) {
                const int id = cluster_nth_equal(cl, c, g, bits, blo, at);
                w.event = ev; w.idx = id; w.p = pv; w.tie = 1;
                return;
            }
            w.tau = blo;
            continue;
        }
        if (g.rank == 0) {
            sort_cands(c, nb);
            walk_sorted(c, nb, s_bin, pos_bin, x_ge, x_gt, counting, nstop);
        }
        cl.sync();
        DT(7);
        fetch_from_leader(c, 6, [&](int i) {
            return i == 0 ? (long long)lead->b_event : i == 1 ? (long long)lead->b_aux
                 : i == 2 ? (long long)__float_as_int(lead->b_s) : i == 3 ? lead->b_pos
                 : i == 4 ? (long long)lead->b_idx : (long long)__float_as_int(lead->b_p); });
        w.s = __int_as_float((int)A->rx[2]); w.pos = A->rx[3]; w.tau = blo;
        const int ev = (int)A->rx[0];
        if (ev != EV_NONE) {
            w.event = ev; w.idx = (int)A->rx[4]; w.p = __int_as_float((int)A->rx[5]); w.tie = (int)A->rx[1];
            cl.sync();  // the leader's results are read before anyone moves on
            return;
        }
        if (phase > 8) c.status |= MOLLA_ROW_SLOW_PATH;
    }
    w.event = EV_DEGENERATE;
    c.status |= MOLLA_ROW_DEGENERATE;
}

__global__ void __launch_bounds__(NT, 1) sample_rows_cluster_kernel(const __grid_constant__ BatchArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    cg::cluster_group cl = cg::this_cluster();
    CtxC c;
    c.tid = threadIdx.x; c.lane = c.tid & 31; c.warp = c.tid >> 5; c.status = 0;
    float *rowbuf = reinterpret_cast<float *>(smem_raw);
    unsigned int *rowbits = reinterpret_cast<unsigned int *>(smem_raw);
    AuxC *A = reinterpret_cast<AuxC *>(smem_raw + (size_t)CL_CAPF * 4);
    c.A = A;
    IN_SHARED(A);
    IN_SHARED(rowbuf);
    IN_SHARED(rowbits);
    ClGeo g;
    g.G = a.G; g.rank = (int)cl.block_rank(); g.L = a.L;
    g.c0 = g.rank * a.Vc;
    g.nloc = max(0, min(a.Vc, a.V - g.c0));
    const int row_i = (int)blockIdx.x / g.G;
    const int r = a.order ? a.order[row_i] : row_i;
    const bool leader = g.rank == 0;
    AuxC *lead = cl.map_shared_rank(A, 0);

    // ---- settings (the same in every block of the cluster)
    const int q = a.slot ? a.slot[r] : r;
    const long long lrow = a.rows ? (long long)a.rows[r] : (long long)r;
    const bool idx_ok = (!a.slot || (q >= 0 && (a.n_slots <= 0 || q < a.n_slots))) &&
                        (!a.rows || (lrow >= 0 && (a.n_logit_rows <= 0 || lrow < a.n_logit_rows)));
    if (!idx_ok) {  // a stale row or slot index: nothing of that row or slot is touched
        if (leader && c.tid == 0) { a.tokens[r] = -1; a.row_status[r] = MOLLA_ROW_INVALID_CONFIG; }
        return;
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
    const long long *histp = a.ring ? a.ring + (size_t)q * (size_t)a.ring_cap : (a.hist ? a.hist + h0 : nullptr);
    const int H = a.ring ? min(max(a.ring_filled[q], 0), ring_n) : ((a.hist && a.hist_off) ? (a.hist_off[q + 1] - h0) : 0);
    const int b0 = (a.bias_ids && a.bias_off) ? a.bias_off[q] : 0;
    const int nb = (a.bias_ids && a.bias_off) ? (a.bias_off[q + 1] - b0) : 0;
    // the rules of SamplerConfig.check (sample.mojo:140-154); NaN fails every test
    const bool valid = (T >= 0.0f) && (k >= 0) && (P > 0.0f && P <= 1.0f) && (minp >= 0.0f && minp <= 1.0f) &&
                       (typ > 0.0f && typ <= 1.0f) && (rp > 0.0f) && H >= 0 && nb >= 0;
    const bool greedy = !(T > 0.0f);
    const bool penalizing = won && H > 0 && (rp != 1.0f || fp != 0.0f || pp != 0.0f);
    const int npatch = (penalizing ? H : 0) + nb;
    if (!valid) c.status |= MOLLA_ROW_INVALID_CONFIG;
    // typical-p is done on rows an earlier filter sorted and cut to a set inside the sorted head
    else if (!greedy && typ < 1.0f && !((k > 0 && k < a.V) || P < 1.0f)) c.status |= MOLLA_ROW_UNSUPPORTED;
    if (npatch > PATCH_MAX) c.status |= MOLLA_ROW_UNSUPPORTED;

    float dZ = 0.0f, dsum = 0.0f, dtarget = 0.0f, dp = 0.0f;
    int token = -1;
    // the end of every row: the leader's thread 0 writes the answer and does `_took`
    auto finish = [&]() {
        if (!(leader && c.tid == 0)) return;
#ifdef MOLLA_SAMPLE_TESTING
        if (a.prof) {
            unsigned long long gt;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
            a.prof[(long long)r * 32 + 11] = (long long)gt; a.prof[(long long)r * 32 + 9] = clock64();
        }
#endif
        if (c.status & (MOLLA_ROW_LOAD_TIMEOUT | MOLLA_ROW_DEGENERATE | MOLLA_ROW_INVALID_CONFIG | MOLLA_ROW_UNSUPPORTED | MOLLA_ROW_EMPTY)) token = -1;
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
    };
    if (c.status) { finish(); return; }

    CSTAMP(0);
#ifdef MOLLA_SAMPLE_TESTING
    if (a.prof && leader && c.tid == 0) {
        unsigned long long gt;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt));
        a.prof[(long long)r * 32 + 10] = (long long)gt; a.prof[(long long)r * 32 + 12] = blockIdx.x;
    }
#endif
    // ---- 1. this block's range of the row, HBM -> shared memory
    const float *src = a.logits + lrow * a.row_stride + g.c0;
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0);
    const int nbulk = aligned ? (g.nloc & ~3) : 0;
    if (c.tid == 0) {
        mbar_init(&A->mbar, 1);
        fence_proxy_async();
        if (nbulk > 0) {
            mbar_expect_tx(&A->mbar, (uint32_t)nbulk * 4u);
            for (int o = 0; o < nbulk; o += CL_PIECE)
                bulk_g2s_last_use(rowbuf + o, src + o, (uint32_t)min(CL_PIECE, nbulk - o) * 4u, &A->mbar);
        }
    }
    // meanwhile: the tokens a bias or a penalty touches (sample.mojo:381-417), those of this range.
    // A small hash (keys and window counts) in the space the candidates use later.
    int *hkey = reinterpret_cast<int *>(A->cand);
    int *hcnt = hkey + HSLOTS;
    if (npatch > 0) {
        for (int i = c.tid; i < HSLOTS; i += NT) { hkey[i] = -1; hcnt[i] = 0; }
        __syncthreads();
        for (int i = c.tid; i < npatch; i += NT) {
            const bool is_bias = i < nb;
            const long long t64 = (is_bias ? a.bias_ids[b0 + i] : histp[i - nb]) - (long long)g.c0;
            if (t64 < 0 || t64 >= g.nloc) continue;
            const int tok = (int)t64;
            int s = hslot(tok);
            for (int probe = 0; probe < HSLOTS; probe++) {
                const int old = atomicCAS(&hkey[s], -1, tok);
                if (old == -1 || old == tok) { if (!is_bias) atomicAdd(&hcnt[s], 1); break; }
                s = (s + 1) & (HSLOTS - 1);
            }
        }
    }
    // what the bulk copies do not bring: the ragged end, or all of a row that is not 16-byte aligned
    for (int i = nbulk + c.tid; i < g.nloc; i += NT) rowbuf[i] = __ldg(src + i);
    for (int i = g.nloc + c.tid; i < NT * g.L; i += NT) rowbuf[i] = -INFINITY;
    __syncthreads();  // the barrier is initialised before anyone waits on it
    if (nbulk > 0) {
        bool done = false;
        for (int spin = 0; spin < (1 << 22); spin++) {
            if (mbar_try_wait(&A->mbar, 0u)) { done = true; break; }
        }
        if (!done) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
    }
    if (MOLLA_KNOB(a, 16) && c.warp == 3) c.status |= MOLLA_ROW_LOAD_TIMEOUT;  // testing build: one warp reports a wait that ran out
    if (__syncthreads_or((c.status & MOLLA_ROW_LOAD_TIMEOUT) ? 1 : 0)) c.status |= MOLLA_ROW_LOAD_TIMEOUT;
    CSTAMP(1);
    if (a.softcap > 0.0f) {
        for (int i = c.tid; i < g.nloc; i += NT) rowbuf[i] = softcap_pinned(rowbuf[i], a.softcap);
        __syncthreads();
    }
    if (a.mask) {
        // `_mask` (sample.mojo:371-379): what the grammar forbids is no candidate at all. A logit of
        // -inf is exactly that here: it wins no maximum, takes no bias or penalty that could bring it
        // back, its exponential is zero, and zeros are absent from every sum, count and walk.
        const unsigned int *mrow = a.mask + (long long)r * a.mask_stride;
        for (int i = c.tid; i < g.nloc; i += NT) {
            const int t = g.c0 + i;
            if (!((__ldg(mrow + (t >> 5)) >> (t & 31)) & 1u)) rowbuf[i] = -INFINITY;
        }
        __syncthreads();
    }
    if (npatch > 0) {
        for (int s = c.tid; s < HSLOTS; s += NT) {
            const int tok = hkey[s];
            if (tok < 0) continue;
            float v = rowbuf[tok];
            for (int bq = 0; bq < nb; bq++)  // duplicates add up, in the order they were given
                if (a.bias_ids[b0 + bq] == (long long)tok + g.c0) v = __fadd_rn(v, a.bias_vals[b0 + bq]);
            const int n = hcnt[s];
            if (n > 0) {
                if (v > 0.0f) v = __fdiv_rn(v, rp);
                else v = __fmul_rn(v, rp);
                v = __fsub_rn(v, __fmul_rn((float)n, fp));
                v = __fsub_rn(v, pp);
            }
            rowbuf[tok] = v;
        }
        __syncthreads();
    }

    CSTAMP(2);
    // ---- 2. the maximum and its first index (kernel.mojo:571-585, sample.mojo:342-346)
    const long long n_lim = (k > 0 && k < a.V) ? (long long)k : (long long)a.V;
    const bool sampled = !greedy && n_lim > 1;  // rows that need more than the maximum
    const bool topp_on = (P < 1.0f) && (n_lim > 1);
    const bool pure = !topp_on && n_lim == (long long)a.V;
    const int i0 = c.tid * g.L;
    float tmax;
    int tj;
    {
        // four interleaved runs over the thread's range, each keeping its first maximum
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
        int j0 = 0, j1 = 1, j2 = 2, j3 = 3;
        int j = 0;
        for (; j + 4 <= g.L; j += 4) {
            const float x0 = rowbuf[i0 + j], x1 = rowbuf[i0 + j + 1], x2 = rowbuf[i0 + j + 2], x3 = rowbuf[i0 + j + 3];
            if (x0 > m0) { m0 = x0; j0 = j; }
            if (x1 > m1) { m1 = x1; j1 = j + 1; }
            if (x2 > m2) { m2 = x2; j2 = j + 2; }
            if (x3 > m3) { m3 = x3; j3 = j + 3; }
        }
        for (; j < g.L; j++) {
            const float x0 = rowbuf[i0 + j];
            if (x0 > m0) { m0 = x0; j0 = j; }
        }
        tmax = m0; tj = j0;
        if (m1 > tmax || (m1 == tmax && j1 < tj)) { tmax = m1; tj = j1; }
        if (m2 > tmax || (m2 == tmax && j2 < tj)) { tmax = m2; tj = j2; }
        if (m3 > tmax || (m3 == tmax && j3 < tj)) { tmax = m3; tj = j3; }
    }
    float cmax = tmax;
    int cidx = g.c0 + i0 + tj;
    block_argmax(c, cmax, cidx);
    int ceq = 0;
    if (!greedy && n_lim == 1) {
        // only a top-k of one asks how many share the maximum (the sort's first element is one of them)
        int e = 0;
        for (int j = 0; j < g.L; j++) e += (i0 + j < g.nloc && rowbuf[i0 + j] == cmax) ? 1 : 0;
        (void)block_excl_scan<int>(e, A->wsi, &ceq);
    }
    // A lower bound of the running sum before every thread's range: each range adds at least the
    // exponential of its own maximum. Relative to this block's maximum for now; the others' are
    // not known yet.
    float et = 0.0f, eex = 0.0f, etot = 0.0f;
    if (sampled) {
        if (i0 < g.nloc && tmax > -INFINITY) {
            const float d = __fsub_rn(tmax, cmax);
            et = expf_pinned((T == 1.0f) ? d : __fdiv_rn(d, T));
        }
        eex = block_excl_scan<float>(et, A->wsf, &etot);
        if (!pure) {
            // the head's threshold comes from the threads' maxima: how many lie how far below the maximum
            A->thist[c.tid] = 0u;
            __syncthreads();
            if (i0 < g.nloc) {
                const float dd = __fmul_rn(__fsub_rn(cmax, tmax), TRES);
                const int b = (dd >= 0.0f && dd < (float)(TBINS - 1)) ? (int)dd : TBINS - 1;
                sred_add(&A->thist[b], 1u);
            }
        }
    }
    __syncthreads();
    if (c.tid < g.G) {
        AuxC *ox = cl.map_shared_rank(A, c.tid);
        ox->x1_max[g.rank] = cmax; ox->x1_idx[g.rank] = cidx; ox->x1_eq[g.rank] = ceq; ox->x1_status[g.rank] = c.status;
        ox->x2_total[g.rank] = etot;
    }
    if (c.tid == 0) { A->ncand = 0; A->evt_thread = 0x7fffffff; A->ch_flag = 0; }
    CSTAMP(13);
    cl.sync();
    float xmax = -INFINITY;
    int imax = 0x7fffffff, eqs = 0;
    for (int o = 0; o < g.G; o++) {
        c.status |= A->x1_status[o];
        const float m = A->x1_max[o];
        if (m > xmax) { xmax = m; imax = A->x1_idx[o]; eqs = A->x1_eq[o]; }
        else if (m == xmax) { imax = min(imax, A->x1_idx[o]); eqs += A->x1_eq[o]; }
    }
    if (imax == 0x7fffffff) imax = 0;
    if (c.status & MOLLA_ROW_LOAD_TIMEOUT) { finish(); return; }
    if (a.mask && !(xmax > -INFINITY)) { c.status |= MOLLA_ROW_EMPTY; finish(); return; }  // every candidate was filtered out

    CSTAMP(3);
    if (greedy) { token = imax; finish(); return; }
    if (n_lim == 1) {
        // top-k of one: the sort's first element is a maximum (sample.mojo:485-490)
        if (eqs > 1) c.status |= MOLLA_ROW_TOPK_TIE;
        token = imax; finish(); return;
    }

    const float top = (T == 1.0f) ? xmax : __fdiv_rn(xmax, T);
    const float u01 = draw01(a.seed ? a.seed[q] : 0ull, a.drawn ? a.drawn[q] : 0ull);
    const bool filter_ok = fabsf(top) < 1.0e5f;
    // how many the sorted head has to cover: top-k + 1 where a top-k is set (up to CL_HEAD_NEED: such
    // rows finish in the head), a fixed number where the nucleus alone ends the row
    const bool open_row = n_lim == (long long)a.V;
    long long need = open_row ? (long long)HEAD_NEED : n_lim + 1;
    if (need > CL_HEAD_NEED) need = CL_HEAD_NEED;
    if (need > a.V) need = a.V;
    const bool p3row = !pure && (open_row ? (n_lim + 1 > HEAD_NEED) : (n_lim + 1 > CL_HEAD_NEED));

    // ---- 3. the bound relative to the row's maximum, and the head's threshold: a value that at
    // least `need` of the threads' maxima reach bounds the need-th largest element from below.
    float lb;
    {
        float lbbase = 0.0f, mine = 0.0f;
        for (int o = 0; o <= g.rank; o++) {
            const float d = __fsub_rn(A->x1_max[o], xmax);
            const float f = (A->x1_max[o] > -INFINITY) ? expf_pinned((T == 1.0f) ? d : __fdiv_rn(d, T)) : 0.0f;
            if (o < g.rank) lbbase += A->x2_total[o] * f; else mine = f;
        }
        lb = lbbase + eex * mine;
    }
    float tau_x = INFINITY;
    unsigned int tau_bits = 1u;
    if (!pure) {
        // thread t adds up, over the blocks, the counts of bin t of distance below the row's maximum
        // (a block's own bins are shifted by its maximum's distance, rounded up)
        int cnt = 0;
        for (int o = 0; o < g.G; o++) {
            const float dd = __fmul_rn(__fsub_rn(xmax, A->x1_max[o]), TRES);
            if (!(dd >= 0.0f && dd < (float)TBINS)) continue;
            const int lb_ = c.tid - (int)ceilf(dd);
            if (lb_ >= 0 && lb_ < TBINS - 1) cnt += (int)cl.map_shared_rank(A, o)->thist[lb_];
        }
        int tot;
        const int ex = block_excl_scan<int>(cnt, A->wsi, &tot);
        if ((long long)ex < need && (long long)(ex + cnt) >= need) A->evt_thread = c.tid;
        __syncthreads();
        const int gb = A->evt_thread;
        tau_x = (gb < TBINS - 1 && fabsf(xmax) < 65536.0f) ? __fsub_rn(xmax, __fmul_rn((float)(gb + 2), 1.0f / TRES)) : -INFINITY;
        const float tv = (T == 1.0f) ? tau_x : __fdiv_rn(tau_x, T);
        const unsigned int tb_ = __float_as_uint(expf_pinned(__fsub_rn(tv, top)));
        tau_bits = tb_ > 1u ? tb_ : 1u;
    }
    // what is below half an ulp of the bound is dropped; below top - 105 the exponential is
    // exactly zero whatever came before
    float mythr;
    {
        const float thr_rel = (filter_ok && lb > 0.0f) ? T * (top + logf(0.9f * lb) - REL_MARGIN) : -INFINITY;
        const float thr_zero = filter_ok ? T * (top - 105.0f) : -INFINITY;
        mythr = fminf(fmaxf(thr_rel, thr_zero), tau_x);
    }

    CSTAMP(4);
    // ---- 4. the second pass, in place: the exponential (temperature and softmax numerator,
    // sample.mojo:419-434) of what can matter, zero for the rest. Where a row's sum is still small
    // (its first columns) nearly everything matters, later almost nothing: the warps go through
    // the range in interleaved tiles, so that no warp is left alone with the dense stretch, and
    // evaluate what they keep in full warps.
    {
        static_assert(offsetof(AuxC, hidx) == offsetof(AuxC, pre) + sizeof(A->pre), "the head's candidates rely on this layout");
        static_assert(offsetof(AuxC, cand) == sizeof(A->u) && offsetof(AuxC, pc) == offsetof(AuxC, cand) + sizeof(A->cand) &&
                      sizeof(A->u) + sizeof(A->cand) >= (size_t)(NT + 4) * (CL_LMAX + 1),
                      "the threads' lists use the idle space of the tables and the candidates");
        static_assert(sizeof(A->pc) >= NWARP * CL_LMAX * sizeof(float) && sizeof(A->pre) >= NT * sizeof(float), "bounds per thread and per tile");
        unsigned long long *hcand = reinterpret_cast<unsigned long long *>(A->pre);  // CL_HEADC keys over pre + hidx
        auto value = [&](float xx) -> float {
            const float v = (T == 1.0f) ? xx : __fdiv_rn(xx, T);
            return expf_pinned_nonpos(__fsub_rn(v, top));  // no logit of the row exceeds its maximum
        };
        auto take = [&](unsigned int ebits, int i_block) {  // the head's candidates are picked up on the way
            if (!pure && ebits >= tau_bits) {
                const int pos = satom_add(&A->ncand, 1);
                if (pos < CL_HEADC) hcand[pos] = make_key(ebits, g.c0 + i_block);
            }
        };
        // Warp w takes the 32-wide tiles w, w + 16, w + 32, ... of the range, so the dense stretch
        // is spread evenly over all threads. A tile tests its elements against the lowest bound of
        // the threads it overlaps (keeping more than necessary is always right). Every thread notes
        // the tiles in which it keeps its element in a list of its own and evaluates the list
        // afterwards, four at a time: the lists of a warp's lanes are about equally long, and no
        // conversion, population count, bit search or atomic (all of which issue at a fraction of
        // the rate of the rest) is needed to build them.
        unsigned char *klist = reinterpret_cast<unsigned char *>(&A->u);  // [entry][thread], over u + cand
        float *thr_t = A->pc;  // a bound per tile
        {
            float *thr_s = A->pre;  // every thread's bound
            thr_s[c.tid] = mythr;
            __syncthreads();
            // (x / L without a division: exact for x < 2^32 / L, and x stays below NT * L)
            const unsigned int l_magic = (unsigned int)((0x100000000ull + (unsigned long long)g.L - 1ull) / (unsigned long long)g.L);
            for (int t = c.tid; t < NWARP * g.L; t += NT) {
                const int o0 = (int)__umulhi((unsigned int)(32 * t), l_magic), o1 = min(NT - 1, (int)__umulhi((unsigned int)(32 * t + 31), l_magic));
                float m = thr_s[o0];
                for (int o = o0 + 1; o <= o1; o++) m = fminf(m, thr_s[o]);
                thr_t[t] = m;
            }
            __syncthreads();
        }
        CSTAMP(16);
        constexpr int KSTRIDE = NT + 4;  // bytes per list entry row: rows start one bank apart
        int cnt = 0;
        {
            unsigned char *kp = klist + c.tid;  // where this thread's next entry goes
            auto take_tile = [&](int k, int p, float x, float th) {
                // no branch: the entry is written in any case and stays only if the element is kept
                const bool keep = x >= th;
                *kp = (unsigned char)k;
                kp += keep ? KSTRIDE : 0;
                cnt += keep ? 1 : 0;
                rowbuf[p] = keep ? x : 0.0f;
            };
            int k = 0;
            for (; k + 4 <= g.L; k += 4) {  // four tiles' loads ahead of their stores
                int p[4];
                float x[4], th[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int t = (k + u) * NWARP + c.warp;
                    p[u] = (t << 5) + c.lane;
                    x[u] = rowbuf[p[u]];
                    th[u] = thr_t[t];
                }
#pragma unroll
                for (int u = 0; u < 4; u++) take_tile(k + u, p[u], x[u], th[u]);
            }
            for (; k < g.L; k++) {
                const int t = k * NWARP + c.warp;
                const int p = (t << 5) + c.lane;
                take_tile(k, p, rowbuf[p], thr_t[t]);
            }
        }
        CSTAMP(18);
        const int base = (c.warp << 5) + c.lane;
        auto entry = [&](int i) { return (((int)klist[i * KSTRIDE + c.tid] * NWARP) << 5) + base; };
        int i = 0;
        for (; i + 4 <= cnt; i += 4) {  // (no predicates in here: they would turn into branches around every evaluation)
            int pos[4];
            float y[4];
#pragma unroll
            for (int u = 0; u < 4; u++) pos[u] = entry(i + u);
#pragma unroll
            for (int u = 0; u < 4; u++) y[u] = value(rowbuf[pos[u]]);
#pragma unroll
            for (int u = 0; u < 4; u++) { rowbuf[pos[u]] = y[u]; take(__float_as_uint(y[u]), pos[u]); }
        }
        for (; i < cnt; i++) {
            const int pos = entry(i);
            const float y = value(rowbuf[pos]);
            rowbuf[pos] = y;
            take(__float_as_uint(y), pos);
        }
        __syncthreads();
        CSTAMP(17);
        // the head's candidates to where the head looks for them
        const int nh = min(A->ncand, CL_HEADC);
        unsigned long long mine[(CL_HEADC + NT - 1) / NT];
#pragma unroll
        for (int u = 0; u < (CL_HEADC + NT - 1) / NT; u++) mine[u] = (c.tid + u * NT < nh) ? hcand[c.tid + u * NT] : 0ull;
        __syncthreads();
#pragma unroll
        for (int u = 0; u < (CL_HEADC + NT - 1) / NT; u++)
            if (c.tid + u * NT < nh) A->cand[c.tid + u * NT] = mine[u];
    }
    __syncthreads();
    CSTAMP(5);
    // how many candidates for the head every block holds
    if (c.tid < g.G) cl.map_shared_rank(A, c.tid)->x3_n[g.rank] = A->ncand;

    // ---- 5. the softmax denominator, exactly as the sequential loop rounds it
    int epoch = 0;
    const ClSum zs = cluster_exact_sum(cl, c, g, rowbits, false, 0.0f, epoch, CPROF_SLOTS(leader, 14), CPROF_SLOTS(!p3row, 20));
    const float Z = zs.s;
    if (zs.slow) c.status |= MOLLA_ROW_SLOW_PATH;
    if (zs.timeout) { c.status |= MOLLA_ROW_LOAD_TIMEOUT; finish(); return; }  // (the same word in every block)
    dZ = Z;

    CSTAMP(6);
    const unsigned int tau_p = __float_as_uint(__fdiv_rn(__uint_as_float(tau_bits), Z));
    const unsigned int tau_pb = tau_p > 1u ? tau_p : 1u;
    (void)tau_pb;

    // min-p (sample.mojo:508-523): see the note at the same place in sample_rows_kernel
    long long n_use = n_lim;
    const bool typ_on = typ < 1.0f;
    unsigned int minp_pbits = 0u;
    if (minp > 0.0f) {
        const float p_top = __fdiv_rn(expf_pinned(__fsub_rn(top, top)), Z);
        const float floor_p = __fmul_rn(p_top, minp);
        minp_pbits = __float_as_uint(floor_p);
        if (!(floor_p >= 2.2e-8f)) {
            c.status |= MOLLA_ROW_UNSUPPORTED;
        } else if (!pure) {
            unsigned int lo_b = 0u, hi_b = 0x3F800000u;
            for (int it = 0; it < 32 && lo_b < hi_b; it++) {
                const unsigned int mid = lo_b + ((hi_b - lo_b) >> 1);
                if (__fdiv_rn(__uint_as_float(mid), Z) >= floor_p) hi_b = mid; else lo_b = mid + 1u;
            }
            const unsigned int e_floor = hi_b;
            int cnt_ge = 0;
            for (int i = c.tid; i < g.nloc; i += NT) cnt_ge += (rowbits[i] >= e_floor && rowbits[i] != 0u) ? 1 : 0;
            int n_ge_loc;
            (void)block_excl_scan<int>(cnt_ge, A->wsi, &n_ge_loc);
            if (c.tid < g.G) cl.map_shared_rank(A, c.tid)->x4_n[g.rank] = n_ge_loc;
            cl.sync();
            long long n_ge = 0;
            for (int o = 0; o < g.G; o++) n_ge += A->x4_n[o];
            if (n_ge < 1) n_ge = 1;  // never empties
            if (n_ge < n_use) n_use = n_ge;
        }
    }
    if (c.status & MOLLA_ROW_UNSUPPORTED) { finish(); return; }

    if (pure) {
        // ---- 6a. nothing sorted: the draw walks the vocabulary in order (sample.mojo:365-369,
        // 580-594): probabilities p = e / Z (:437-438), what min-p drops becomes zero
        for (int i = c.tid; i < g.nloc; i += NT) {
            const unsigned int eb = rowbits[i];
            if (eb == 0u) continue;
            unsigned int pb = __float_as_uint(__fdiv_rn(__uint_as_float(eb), Z));
            if (pb < minp_pbits) pb = 0u;
            rowbits[i] = pb;
        }
        const ClSum s1 = cluster_exact_sum(cl, c, g, rowbits, false, 0.0f, epoch);
        const float sum = s1.s;
        const float target = __fmul_rn(u01, sum);
        const ClSum s2 = cluster_exact_sum(cl, c, g, rowbits, true, target, epoch);
        if (s1.slow || s2.slow) c.status |= MOLLA_ROW_SLOW_PATH;
        if (s1.timeout || s2.timeout) { c.status |= MOLLA_ROW_LOAD_TIMEOUT; finish(); return; }
        dsum = sum; dtarget = target;
        if (s2.found) token = s2.at;
        else {
            // the walk fell off the end: the reference returns the last token of the vocabulary,
            // whether or not it could matter to any sum ... or the last one min-p left
            token = a.V - 1;
            if (minp_pbits) {
                int last = -1;
                for (int i = c.tid; i < g.nloc; i += NT)
                    if (rowbits[i] >= minp_pbits && rowbits[i] != 0u) last = max(last, g.c0 + i);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
                __syncthreads();
                if (c.lane == 0) A->wsi[c.warp] = last;
                __syncthreads();
                if (c.tid < g.G) {
                    int m = -1;
                    for (int w = 0; w < NWARP; w++) m = max(m, A->wsi[w]);
                    cl.map_shared_rank(A, c.tid)->x4_n[g.rank] = m;
                }
                cl.sync();
                last = -1;
                for (int o = 0; o < g.G; o++) last = max(last, A->x4_n[o]);
                token = last >= 0 ? last : imax;
            }
        }
        finish();
        return;
    }

    CSTAMP(7);
    // ---- 6b. sorted order. The head's candidates go to the leader as probabilities.
    int nc_tot = 0, cbase = 0;
    bool head_overflow = false;
    for (int o = 0; o < g.G; o++) {
        const int n = A->x3_n[o];
        if (o < g.rank) cbase += n;
        nc_tot += n;
        if (n > CL_HEADC) head_overflow = true;
    }
    if (nc_tot > CL_HEADC) head_overflow = true;
    if (!head_overflow) {
        const int mine = A->x3_n[g.rank];
        for (int i = c.tid; i < mine; i += NT) {
            const unsigned long long kk = A->cand[i];
            const unsigned long long nk = ((unsigned long long)__float_as_uint(__fdiv_rn(key_val(kk), Z)) << 32) | (kk & 0xFFFFFFFFull);
            if (leader) A->cand[i] = nk; else lead->cand[cbase + i] = nk;
        }
    }
    cl.sync();
    int nc = head_overflow ? 0 : nc_tot;
    unsigned int tau_head = 0xFFFFFFFFu;
    if (head_overflow) c.status |= MOLLA_ROW_SLOW_PATH;  // no head: the descending walk takes everything from the top
    if (leader) {
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
            int cut = -1, tie = 0;
            bool by_mass = false;
            // the prefix sums of the sorted head (sample.mojo:497-506), eight loads ahead of the
            // additions; at most n_use elements are added
            const int lim = (int)((long long)nc < n_use ? (long long)nc : n_use);
            int i = 0;
            while (i < lim && cut < 0) {
                float v[8];
                const int m = min(8, lim - i);
#pragma unroll
                for (int q = 0; q < 8; q++) v[q] = (q < m) ? A->pc[i + q] : 0.0f;
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    if (q < m && cut < 0) {
                        s = __fadd_rn(s, v[q]);
                        A->pre[i + q] = s;
                        if (topp_on && s >= P) { cut = i + q + 1; by_mass = true; }
                    }
                }
                i += m;
            }
            const long long pos = (cut >= 0) ? (long long)cut : (long long)lim;
            if (by_mass) {
                if (cut < nc && (long long)cut < n_use && A->pc[cut] == A->pc[cut - 1]) tie |= MOLLA_ROW_TOPP_TIE;
            } else if (lim > 0 && (long long)lim >= n_use) {
                cut = lim;  // the count limit
            }
            if (cut < 0 && !p3row && !head_overflow) cut = nc;  // everything that can matter is in the head
            if (n_use < (long long)a.V && (long long)nc > n_use && A->pc[n_use] == A->pc[n_use - 1])
                tie |= MOLLA_ROW_TOPK_TIE;
            A->b_s = s; A->b_pos = pos; A->b_event = EV_NONE; A->b_idx = -1; A->b_p = 0.0f;
            if (typ_on) {
                A->ncand = cut;  // the typical-p filter takes over from here
            } else if (cut > 0) {
                const float sum = A->pre[cut - 1];
                const float target = __fmul_rn(u01, sum);
                int at = cut - 1;
                for (int i0 = 0; i0 < cut && at == cut - 1; i0 += 8) {
                    float v[8];
#pragma unroll
                    for (int q = 0; q < 8; q++) v[q] = (i0 + q < cut) ? A->pre[i0 + q] : 0.0f;
#pragma unroll
                    for (int q = 7; q >= 0; q--)
                        if (i0 + q < cut && target < v[q]) at = i0 + q;  // the first one wins
                }
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
        int kind = 1;  // 0: the row is finished; 1: past the head
        if (typ_on) {
            const int m = A->ncand;
            if (m <= 0 || m > HEADC) {
                c.status |= MOLLA_ROW_UNSUPPORTED;  // what the earlier filters left reaches past the head, or is wider than the filter's scratch
            } else {
                typical_head(c, m, typ, u01);
                token = A->b_idx; dp = A->b_p; dsum = A->b_sum; dtarget = A->b_target;
                c.status |= (unsigned int)A->b_aux;
            }
            kind = 0;
        } else if (A->b_event == EV_DRAW) {
            token = A->b_idx; dp = A->b_p; dsum = A->b_sum; dtarget = A->b_target;
            kind = 0;
        }
        __syncthreads();
        if (c.tid < g.G) {
            AuxC *ox = cl.map_shared_rank(A, c.tid);
            ox->r_kind = kind; ox->r_s = head_s; ox->r_pos = head_pos; ox->r_status = c.status;
        }
    }
    cl.sync();
    if (A->r_kind == 0) { finish(); return; }
    c.status |= A->r_status;
    const float head_s = A->r_s;
    const long long head_pos = A->r_pos;

    CSTAMP(8);
    // ---- 7. past the head: the cut walk, then the draw walk, over the probabilities
    // (sample.mojo:437-438); what the head took is consumed
    for (int i = c.tid; i < g.nloc; i += NT) {
        const unsigned int eb = rowbits[i];
        if (eb == 0u) continue;
        unsigned int pb = __float_as_uint(__fdiv_rn(__uint_as_float(eb), Z));
        if (!head_overflow && eb >= tau_bits) pb = 0u;
        rowbits[i] = pb;
    }
    __syncthreads();
    // One call site for both walks (the walk is most of this kernel's code, and what a row runs
    // through has to stay in the instruction cache): leg 0 is the cut walk, leg 1 the draw walk.
    const bool limited = n_use < (long long)a.V;
    ClWalk w;
    ClResume resume;
    resume.valid = 0;
    int cut_event = EV_NONE, cut_idx = -1;
    float cut_p = 0.0f, sum = 0.0f, target = 0.0f;
    bool settled = false;    // the token is known, or the row is degenerate
    bool resolved = false;
    for (int leg = 0; leg < 2; leg++) {
        w.s = head_s; w.pos = head_pos; w.tau = tau_head;
        w.event = EV_NONE; w.idx = -1; w.p = 0; w.tie = 0;
        const bool cut_round = leg == 0;
        descend_cluster(cl, c, g, rowbits, w, (cut_round && topp_on) ? P : 3.4e38f, cut_round ? 3.4e38f : target,
                        (cut_round && limited) ? n_use : -1, resume, !cut_round, cut_round ? CPROF_SLOTS(leader, 20) : nullptr);
        if (!cut_round) {
            if (w.event == EV_DRAW) {
                token = w.idx; dp = w.p; resolved = true;
                if (w.tie) c.status |= MOLLA_ROW_CHOSEN_TIE;
            } else if (w.event == EV_DEGENERATE) {
                resolved = true;
            }
            break;
        }
        cut_event = w.event; cut_idx = w.idx; cut_p = w.p;
        if (cut_event == EV_DEGENERATE) { settled = true; break; }
        if (cut_event == EV_CUT && w.tie) c.status |= MOLLA_ROW_TOPP_TIE;
        if (cut_event == EV_LIMIT && w.tie) c.status |= MOLLA_ROW_TOPK_TIE;
        sum = w.s;
        target = __fmul_rn(u01, sum);
        dsum = sum; dtarget = target;
        cl.sync();
        if (leader) {  // is the drawn element in the head? (the first prefix sum above the target)
            if (c.tid == 0) A->evt_thread = 0x7fffffff;
            __syncthreads();
            for (int i = c.tid; i < nc; i += NT)
                if (target < A->pre[i]) { atomicMin(&A->evt_thread, i); break; }
            __syncthreads();
        }
        if (leader && c.tid == 0) {
            const int at = (A->evt_thread == 0x7fffffff) ? -1 : A->evt_thread;
            int ev = EV_NONE, idx = -1, aux = 0;
            float pv = 0.0f;
            if (at >= 0) {
                ev = EV_DRAW; idx = (int)(A->hidx[at] & 0x7fffffffu);
                pv = __fsub_rn(A->pre[at], at > 0 ? A->pre[at - 1] : 0.0f);
                aux = (A->hidx[at] & 0x80000000u) ? MOLLA_ROW_CHOSEN_TIE : 0;
            }
            for (int o = 0; o < g.G; o++) {
                AuxC *ox = cl.map_shared_rank(A, o);
                ox->r_kind = ev; ox->r_idx = idx; ox->r_s = pv; ox->r_status = (unsigned int)aux;
            }
        }
        cl.sync();
        if (A->r_kind == EV_DRAW) {
            token = A->r_idx; dp = A->r_s; c.status |= A->r_status;
            settled = true;
            break;
        }
        if (!(target < sum)) break;
    }
    if (!settled) {
        {
            if (!resolved) {
                // the walk falls off the end: the last kept candidate (sample.mojo:591-594)
                if (cut_event == EV_CUT || cut_event == EV_LIMIT) {
                    token = cut_idx; dp = cut_p;
                } else {
                    // everything listed was kept: its smallest value, highest id last
                    unsigned long long best = ~0ull;
                    for (int i = c.tid; i < g.nloc; i += NT) {
                        const unsigned int pb = rowbits[i];
                        if (pb == 0u) continue;
                        const unsigned long long kk = make_key(pb, g.c0 + i);
                        best = kk < best ? kk : best;
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        unsigned long long ob = __shfl_xor_sync(0xffffffffu, best, o);
                        best = ob < best ? ob : best;
                    }
                    __syncthreads();
                    if (c.lane == 0) A->wsu[c.warp] = best;
                    __syncthreads();
                    if (c.tid < g.G) {
                        unsigned long long m = A->wsu[0];
                        for (int v = 1; v < NWARP; v++) m = A->wsu[v] < m ? A->wsu[v] : m;
                        cl.map_shared_rank(A, c.tid)->x5_key[g.rank] = m;
                    }
                    cl.sync();
                    best = ~0ull;
                    for (int o = 0; o < g.G; o++) best = A->x5_key[o] < best ? A->x5_key[o] : best;
                    token = (best != ~0ull) ? key_idx(best) : imax;
                }
            }
        }
    }
    finish();
}

// Rows by decreasing cost estimate (a greedy row is one pass over its logits, a warm row with a
// wide nucleus keeps most of its vocabulary): clusters start in grid order, and the dearest rows
// should not be the last to start. One thread per row counts the rows that come before it.
__global__ void __launch_bounds__(1024, 1) order_rows_rank_kernel(const float *temperature, const int *top_k, const int *slot, int B, int *order) {
    __shared__ float cost[ORDER_CAP];
    for (int i = threadIdx.x; i < B; i += blockDim.x) {
        const int q = slot ? slot[i] : i;
        const float T = temperature ? temperature[q] : 0.0f;
        const int k = top_k ? top_k[q] : 0;
        cost[i] = (T > 0.0f && k != 1) ? T + ((k == 0 || k >= CL_HEAD_NEED) ? 0.25f : 0.0f) : 0.0f;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < B; i += blockDim.x) {
        const float ci = cost[i];
        int rank = 0;
        for (int j = 0; j < B; j++) {
            const float cj = cost[j];
            rank += (cj > ci || (cj == ci && j < i)) ? 1 : 0;
        }
        order[rank] = i;
    }
}

// How a vocabulary of V logits is laid over a cluster: blocks per cluster (0 = too wide), logits
// per block (a multiple of four: bulk copies start on 16-byte boundaries) and logits per thread
// (odd: conflict-free shared-memory strides).
struct ClusterShape { int G, Vc, L; };

// The smallest cluster that holds the row; for a batch so small that larger clusters of all
// its rows are still resident together (a lone decode stream, a few rows per GPU), the largest
// such cluster: the passes over the row shorten with the range, and nobody waits for an SM.
ClusterShape cluster_shape(int V, int B, int sms) {
    ClusterShape best{0, 0, 0};
    for (int G = 1; G <= CL_MAX_G; G *= 2) {
        const int Vc = ((((V + G - 1) / G) + 3) / 4) * 4;
        int L = (Vc + NT - 1) / NT;
        if ((L & 1) == 0) L += 1;
        if (L > CL_LMAX) continue;
        if (best.G == 0) { best = ClusterShape{G, Vc, L}; continue; }
        // (clusters do not fill every SM: leave the same margin the resident-cluster count shows)
        if ((long long)B * G * 9 <= (long long)sms * 8 && L >= 9) best = ClusterShape{G, Vc, L};
    }
    return best;
}

constexpr size_t CL_SMEM = (size_t)CL_CAPF * 4 + ((sizeof(AuxC) + 15) / 16) * 16;
constexpr int CL_MAX_DEVICES = 64;

void cluster_config(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *at, unsigned int blocks, int G, cudaStream_t st) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3(blocks); cfg.blockDim = dim3(NT);
    cfg.dynamicSmemBytes = CL_SMEM; cfg.stream = st;
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)G; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
}

// Whether this device can hold a cluster of G of the kernel's blocks (asked once per device and size).
bool cluster_fits(int dev, int G) {
    static int known[CL_MAX_DEVICES][CL_MAX_G + 1] = {};  // 0 unknown, 1 yes, -1 no
    if (dev < 0 || dev >= CL_MAX_DEVICES) return false;
    if (known[dev][G]) return known[dev][G] > 0;
    bool ok = cudaFuncSetAttribute(sample_rows_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CL_SMEM) == cudaSuccess;
    if (ok) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute at[1];
        cluster_config(cfg, at, (unsigned)G, G, nullptr);
        int n = 0;
        ok = cudaOccupancyMaxActiveClusters(&n, sample_rows_cluster_kernel, &cfg) == cudaSuccess && n > 0;
    }
    if (!ok) (void)cudaGetLastError();
    known[dev][G] = ok ? 1 : -1;
    return ok;
}

}  // namespace

int molla_cluster_launch(const BatchArgs &args_in, void *d_workspace, cudaStream_t st, char *err, size_t errlen) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MOLLA_CLUSTER_DECLINED;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    ClusterShape cs = cluster_shape(args_in.V, args_in.B, sms);
    if (cs.G != 0 && !cluster_fits(dev, cs.G)) cs = cluster_shape(args_in.V, 1 << 30, sms);  // the smallest cluster then
    if (cs.G == 0 || !cluster_fits(dev, cs.G)) return MOLLA_CLUSTER_DECLINED;
    BatchArgs a = args_in;
    a.G = cs.G; a.Vc = cs.Vc; a.L = cs.L;
    a.Vg = a.V; a.col0 = 0; a.mode = 0;
    a.order = nullptr;
    // clusters start in grid order: when not all rows can start at once, the dearest go first
    if (a.B * cs.G > sms && a.B <= ORDER_CAP && a.temperature) {
        int *order = (int *)((char *)d_workspace + 256);
        order_rows_rank_kernel<<<1, 1024, 0, st>>>(a.temperature, a.top_k, a.slot, a.B, order);
        a.order = order;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[1];
    cluster_config(cfg, at, (unsigned)a.B * (unsigned)cs.G, cs.G, st);
    const cudaError_t e = cudaLaunchKernelEx(&cfg, sample_rows_cluster_kernel, a);
    if (e != cudaSuccess) {
        snprintf(err, errlen, "kernel launch failed: %s", cudaGetErrorString(e));
        return MOLLA_ERR_CUDA;
    }
    return MOLLA_OK;
}
