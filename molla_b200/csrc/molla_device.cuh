// Device-side building blocks shared by the sampling kernels: the pinned fp32
// exponential, the counter-based PRNG, warp/block reductions and scans, and the
// mbarrier / bulk-copy wrappers. sm_100a only.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace molla {

constexpr int NT = 512;      // threads per CTA
constexpr int NWARP = NT / 32;

// ---- PRNG: the reference's splitmix64 finaliser and counter-based draw
// (src/molla/engine/sample.mojo:49-71), bit for bit. --------------------------
__host__ __device__ inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline float draw01(uint64_t seed, uint64_t counter) {
    uint64_t h = mix64(seed ^ mix64(counter + 0x9E3779B97F4A7C15ull));
    return (float)(int64_t)(h >> 40) * (1.0f / 16777216.0f);  // exact: a 24-bit integer times 2^-24
}

// ---- exp(x) in fp32 from fused multiply-adds only: 2^n * exp(r) with
// n = rint(x*log2 e), r = x - n*ln2 (two-piece ln2) and a degree-7 Taylor
// polynomial in Horner form. The CPU checker evaluates the same sequence, so the
// two agree bit for bit; the result is within 1 ulp of the exact exponential.
// It stands in for `exp` of the Mojo standard library (sample.mojo:40,290,433).
__device__ __forceinline__ float scale2(float v, int n) {
    if (n >= -126) return __fmul_rn(v, __int_as_float((n + 127) << 23));
    float a = __int_as_float((n + 64 + 127) << 23);
    float b = __int_as_float((-64 + 127) << 23);
    return __fmul_rn(__fmul_rn(v, a), b);
}
__device__ __forceinline__ float expf_pinned(float x) {
    if (x != x) return x;
    if (x > 88.72284f) return __int_as_float(0x7f800000);
    if (x < -104.0f) return 0.0f;
    const float LOG2E = 1.442695040888963f;
    const float LN2_HI = 0.693145751953125f;
    const float LN2_LO = 1.428606765330187e-06f;
    const float MAGIC = 12582912.0f;
    float t = __fmaf_rn(x, LOG2E, MAGIC);
    float nf = __fsub_rn(t, MAGIC);
    float r = __fmaf_rn(nf, -LN2_HI, x);
    r = __fmaf_rn(nf, -LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int n = (int)nf;
    if (n > 127) return __fmul_rn(scale2(p, n - 64), 18446744073709551616.0f);
    return scale2(p, n);
}

// The same exponential for arguments that cannot be positive (a scaled logit minus the row's
// maximum), without a branch: identical bits to expf_pinned for every x <= 0, NaN included.
// The scaling by 2^n goes through 2^(n+64) * 2^-64 for every n: the first factor never
// rounds, the second rounds once where the result is subnormal, as scale2 does.
__device__ __forceinline__ float expf_pinned_nonpos(float x) {
    const float LOG2E = 1.442695040888963f;
    const float LN2_HI = 0.693145751953125f;
    const float LN2_LO = 1.428606765330187e-06f;
    const float MAGIC = 12582912.0f;
    const float xc = fmaxf(x, -128.0f);  // below -104 the answer is zero anyway; keeps n in range
    float t = __fmaf_rn(xc, LOG2E, MAGIC);
    float nf = __fsub_rn(t, MAGIC);
    float r = __fmaf_rn(nf, -LN2_HI, xc);
    r = __fmaf_rn(nf, -LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    // n sits in the low bits of t (t and MAGIC share a binade whose unit is 1): no conversion,
    // which would issue at a quarter of the rate
    const int n = __float_as_int(t) - __float_as_int(MAGIC);
    const float a = __int_as_float((n + 64 + 127) << 23);
    const float res = __fmul_rn(__fmul_rn(p, a), __int_as_float((-64 + 127) << 23));
    return (x < -104.0f) ? 0.0f : ((x != x) ? x : res);
}

// The typical-p filter's logarithm: the same operations in the same order as the CPU oracle's
// molla_oracle_logf, each rounded once, so the bits agree. Within 2 ulp of the true logarithm.
__device__ __forceinline__ float logf_pinned(float x) {
    if (x != x || x < 0.0f) return __int_as_float(0x7fc00000);
    if (x == 0.0f) return __int_as_float(0xff800000);
    if (x == __int_as_float(0x7f800000)) return x;
    unsigned int u = __float_as_uint(x);
    int e = 0;
    if (u < 0x00800000u) { u = __float_as_uint(__fmul_rn(x, 16777216.0f)); e = -24; }
    e += (int)(u >> 23) - 127;
    float m = __uint_as_float((u & 0x007fffffu) | 0x3f800000u);
    if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
    const float f = __fsub_rn(m, 1.0f);
    const float s = __fdiv_rn(f, __fadd_rn(2.0f, f));
    const float z = __fmul_rn(s, s);
    float R = 2.0f / 11.0f;
    R = __fmaf_rn(R, z, 2.0f / 9.0f);
    R = __fmaf_rn(R, z, 2.0f / 7.0f);
    R = __fmaf_rn(R, z, 2.0f / 5.0f);
    R = __fmaf_rn(R, z, 2.0f / 3.0f);
    R = __fmul_rn(R, z);
    const float lm = __fmaf_rn(-s, __fsub_rn(f, R), f);
    const float LN2_HI = 0.693145751953125f;
    const float LN2_LO = 1.428606765330187e-06f;
    const float dk = (float)e;
    return __fmaf_rn(dk, LN2_HI, __fmaf_rn(dk, LN2_LO, lm));
}

// The final-logit softcap `cap * tanh(x / cap)` as the reference's device kernel evaluates it
// (src/molla/nn/gpu_ops.mojo:302-317 with `_tanh`, :607-623: one exponential of a non-positive
// argument), on the pinned exponential.
__device__ __forceinline__ float softcap_pinned(float x, float cap) {
    const float t = __fdiv_rn(x, cap);
    const float v = (t >= 0.0f) ? t : -t;
    const float e = expf_pinned(__fmul_rn(-2.0f, v));
    const float r = __fdiv_rn(__fsub_rn(1.0f, e), __fadd_rn(1.0f, e));
    return __fmul_rn(cap, (t >= 0.0f) ? r : -r);
}

__device__ __forceinline__ int fexpo(float x) {  // floor(log2 x) of a positive normal float
    return (int)((__float_as_uint(x) >> 23) & 0xFF) - 127;
}
__device__ __forceinline__ float fpow2(int j) {  // 2^j, -126 <= j <= 127
    return __int_as_float((j + 127) << 23);
}

// ---- warp / block collectives -------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// (value, index) argmax, ties to the lower index (src/molla/nn/kernel.mojo:571-585)
__device__ __forceinline__ void warp_argmax(float &v, int &i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}
template <class T>
__device__ __forceinline__ T warp_incl_scan(T v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T y = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += y;
    }
    return v;
}
// Exclusive scan over the NT threads of a CTA; `ws` is NWARP elements of shared
// scratch. Every thread gets its exclusive prefix and the block total.
template <class T>
__device__ __forceinline__ T block_excl_scan(T v, T *ws, T *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = warp_incl_scan(v, lane);
    __syncthreads();  // ws may still be read by an earlier call
    if (lane == 31) ws[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        T w = lane < NWARP ? ws[lane] : T(0);
        T wi = warp_incl_scan(w, lane);
        if (lane < NWARP) ws[lane] = wi - w;
        if (lane == NWARP - 1) ws[NWARP] = wi;
    }
    __syncthreads();
    T out = ws[warp] + (inc - v);
    *total = ws[NWARP];
    return out;
}

// Exclusive scan of two doubles at once (one pass of barriers for both).
__device__ __forceinline__ void block_excl_scan2(double a, double b, double *ws /* 2*(NWARP+1) */, double &ea,
                                                 double &eb, double &ta, double &tb) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    double ia = warp_incl_scan(a, lane), ib = warp_incl_scan(b, lane);
    __syncthreads();
    if (lane == 31) { ws[warp] = ia; ws[NWARP + 1 + warp] = ib; }
    __syncthreads();
    if (warp == 0) {
        double wa = lane < NWARP ? ws[lane] : 0.0, wb = lane < NWARP ? ws[NWARP + 1 + lane] : 0.0;
        double sa = warp_incl_scan(wa, lane), sb = warp_incl_scan(wb, lane);
        if (lane < NWARP) { ws[lane] = sa - wa; ws[NWARP + 1 + lane] = sb - wb; }
        if (lane == NWARP - 1) { ws[NWARP] = sa; ws[2 * NWARP + 1] = sb; }
    }
    __syncthreads();
    ea = ws[warp] + (ia - a); eb = ws[NWARP + 1 + warp] + (ib - b);
    ta = ws[NWARP]; tb = ws[2 * NWARP + 1];
}

// ---- mbarrier + bulk copy (TMA without a tensor map, never multicast) ---------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// The same copy, telling L2 that the lines will not be read again (their last use).
__device__ __forceinline__ void bulk_g2s_last_use(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Loads and stores of data that is read again soon (a row's list between its passes): L2 is
// asked to keep these lines in preference to the streamed logits.
__device__ __forceinline__ uint64_t l2_keep_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ uint64_t l2_normal_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ ulonglong2 ldg_keep(const ulonglong2 *p, uint64_t policy) {
    ulonglong2 v;
    asm volatile("ld.global.L2::cache_hint.v2.u64 {%0, %1}, [%2], %3;" : "=l"(v.x), "=l"(v.y) : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ void stg_keep(unsigned long long *p, unsigned long long v, uint64_t policy) {
    asm volatile("st.global.L2::cache_hint.u64 [%0], %1, %2;" ::"l"(p), "l"(v), "l"(policy) : "memory");
}

// Atomics on shared memory through a pointer whose address space the compiler cannot see
// (it would otherwise fall back to generic-address atomics, which are far slower).
__device__ __forceinline__ void sred_add(unsigned int *p, unsigned int v) {
    asm volatile("red.shared.add.u32 [%0], %1;" ::"r"((unsigned int)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void sred_or(unsigned int *p, unsigned int v) {
    asm volatile("red.shared.or.b32 [%0], %1;" ::"r"((unsigned int)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void sred_max(int *p, int v) {
    asm volatile("red.shared.max.s32 [%0], %1;" ::"r"((unsigned int)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ int satom_add(int *p, int v) {
    int old;
    asm volatile("atom.shared.add.u32 %0, [%1], %2;" : "=r"(old) : "r"((unsigned int)__cvta_generic_to_shared(p)), "r"(v) : "memory");
    return old;
}

}  // namespace molla
