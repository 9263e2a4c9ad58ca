/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A scalar CPU restatement of molla's token sampler, used only as the checker
 * for the CUDA library (parity tests, the smoke test, and the CPU-baseline leg
 * of the benchmark). Nothing in the shipped library links, loads or calls it.
 *
 * What it follows, by file:line in the reference project (tamnd/molla 0.5.7):
 *   src/molla/engine/sample.mojo:49-71    _mix / draw (counter-based PRNG)
 *   src/molla/engine/sample.mojo:128-154  greedy / penalizing / check
 *   src/molla/engine/sample.mojo:260-266  count_of (linear scan of the window)
 *   src/molla/engine/sample.mojo:268-293  logprobs
 *   src/molla/engine/sample.mojo:295-359  pick (stage order)
 *   src/molla/engine/sample.mojo:365-594  _load .. _choose (every filter)
 *   src/molla/nn/kernel.mojo:571-585      argmax (ties to the lower index)
 *   src/molla/nn/tensor.mojo:270-296      Buffer row-major addressing
 *
 * Arithmetic is fp32 where the reference says Float32 and fp64 where it says
 * Float64, every operation separately rounded (build with -ffp-contract=off),
 * the heapsort is the reference's own (its tie order is part of the result),
 * and every sum is sequential in the reference's order.
 *
 * PARITY PINNING. The reference is Mojo and no Mojo toolchain exists where this
 * is built, so the restatement is pinned against (a) every numeric property the
 * reference's own tests state (tests/test_sample.mojo, tests/test_gpu_ops.mojo
 * :365-407) and (b) known answers of `draw` derived from an independent Python
 * restatement. The reference commits no golden token sequences. One dependency
 * lies outside the reference tree: `exp`/`log` from the Mojo standard library
 * (package mojo 1.0.0). Its last-ulp behaviour is unpinned; this oracle uses
 * the fp32 `molla_oracle_expf` below (fused-multiply-add polynomial, <= 1 ulp
 * from the correctly rounded result) so that the CPU and the GPU evaluate the
 * same function bit for bit; `exp_mode = 1` switches to libm's expf to measure
 * how much that choice matters.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- PRNG: sample.mojo:49-71 ------------------------------------------- */

uint64_t molla_oracle_mix(uint64_t value) {
    uint64_t z = value;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

float molla_oracle_draw(uint64_t seed, uint64_t counter) {
    uint64_t h = molla_oracle_mix(seed ^ molla_oracle_mix(counter + 0x9E3779B97F4A7C15ull));
    return (float)(int64_t)(h >> 40) / (float)(1 << 24);
}

/* ---- the pinned fp32 exponential ---------------------------------------
 * exp(x) = 2^n * exp(r), n = rint(x*log2(e)), r = x - n*ln2 (two-piece ln2),
 * exp(r) by a degree-7 Taylor polynomial evaluated with fmaf in Horner form.
 * Only fmaf, add, multiply and exact power-of-two scaling are used, so any
 * IEEE-754 machine that evaluates these in fp32 gets identical bits. */
static inline float scale2(float v, int n) {
    /* v * 2^n with one rounding at most (only when the result is subnormal) */
    if (n >= -126) {
        union { uint32_t u; float f; } s;
        s.u = (uint32_t)(n + 127) << 23;
        return v * s.f;
    }
    union { uint32_t u; float f; } a, b;
    a.u = (uint32_t)(n + 64 + 127) << 23; /* exact: v*2^(n+64) is normal */
    b.u = (uint32_t)(-64 + 127) << 23;
    return (v * a.f) * b.f;
}

float molla_oracle_expf(float x) {
    if (x != x) return x;
    if (x > 88.72284f) return INFINITY;
    if (x < -104.0f) return 0.0f;
    const float LOG2E = 1.442695040888963f;
    const float LN2_HI = 0.693145751953125f;       /* 0x3f317200 */
    const float LN2_LO = 1.428606765330187e-06f;   /* ln2 - LN2_HI */
    const float MAGIC = 12582912.0f;               /* 1.5 * 2^23 */
    float t = fmaf(x, LOG2E, MAGIC);
    float nf = t - MAGIC;
    float r = fmaf(nf, -LN2_HI, x);
    r = fmaf(nf, -LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int n = (int)nf;
    if (n > 127) { /* 2^128 does not exist as a float: split the scale */
        return scale2(p, n - 64) * 18446744073709551616.0f;
    }
    return scale2(p, n);
}

static inline float exp_sel(float x, int mode) {
    return mode == 1 ? expf(x) : molla_oracle_expf(x);
}

/* The natural logarithm the typical-p filter uses (sample.mojo:541,550 call the Mojo
 * standard library's `log`, whose bits are not available here): fp32, x = 2^e * m with m in
 * [sqrt(1/2), sqrt(2)), f = m - 1, s = f / (2 + f), log m = f - s * (f - R(s^2)) with the
 * odd series of atanh for R. Only add, multiply, divide and fmaf, each rounded once, so the
 * CUDA kernel (`logf_pinned`) returns the same bits. Within 2 ulp of the true logarithm. */
float molla_oracle_logf(float x) {
    if (x != x || x < 0.0f) return NAN;
    if (x == 0.0f) return -INFINITY;
    if (x == INFINITY) return x;
    union { float f; uint32_t u; } v;
    v.f = x;
    int e = 0;
    if (v.u < 0x00800000u) { v.f = x * 16777216.0f; e = -24; }  /* subnormal: scale up, exactly */
    e += (int)(v.u >> 23) - 127;
    v.u = (v.u & 0x007fffffu) | 0x3f800000u;                    /* m in [1, 2) */
    if (v.f > 1.41421354f) { v.f = v.f * 0.5f; e += 1; }
    const float f = v.f - 1.0f;                                 /* exact */
    const float s = f / (2.0f + f);
    const float z = s * s;
    float R = 2.0f / 11.0f;
    R = fmaf(R, z, 2.0f / 9.0f);
    R = fmaf(R, z, 2.0f / 7.0f);
    R = fmaf(R, z, 2.0f / 5.0f);
    R = fmaf(R, z, 2.0f / 3.0f);
    R = R * z;
    const float lm = fmaf(-s, f - R, f);
    const float LN2_HI = 0.693145751953125f;       /* 0x3f317200: e * LN2_HI is exact for |e| < 2^9 */
    const float LN2_LO = 1.428606765330187e-06f;   /* ln2 - LN2_HI */
    const float dk = (float)e;
    return fmaf(dk, LN2_HI, fmaf(dk, LN2_LO, lm));
}

/* The final-logit softcap of Gemma-style models as the reference's device kernel computes it
 * (src/molla/nn/gpu_ops.mojo:302-317: x = cap * _tanh(x / cap); _tanh :607-623 through one
 * exponential of a non-positive argument), on the pinned exponential. */
void molla_oracle_softcap(const float *x, int64_t n, float cap, float *out) {
    for (int64_t i = 0; i < n; i++) {
        float t = x[i] / cap;
        float v = t >= 0 ? t : -t;
        float e = molla_oracle_expf(-2.0f * v);
        float r = (1.0f - e) / (1.0f + e);
        out[i] = cap * (t >= 0 ? r : -r);
    }
}

static inline float log_sel(float x, int mode) {
    return mode == 1 ? logf(x) : molla_oracle_logf(x);
}

void molla_oracle_logf_array(const float *x, int64_t n, float *out) {
    for (int64_t i = 0; i < n; i++) out[i] = molla_oracle_logf(x[i]);
}

/* ---- argmax: kernel.mojo:571-585 ---------------------------------------- */

int64_t molla_oracle_argmax(const float *x, int64_t at, int64_t n) {
    if (n <= 0) return -1;
    int64_t best = 0;
    for (int64_t i = 1; i < n; i++)
        if (x[at + i] > x[at + best]) best = i;
    return best;
}

/* ---- logprobs: sample.mojo:268-293 -------------------------------------- */

void molla_oracle_logprobs(const float *z, int64_t n, float *out, int exp_mode) {
    float top = z[0];
    for (int64_t i = 1; i < n; i++)
        if (z[i] > top) top = z[i];
    double sum = 0.0;
    for (int64_t i = 0; i < n; i++) sum += (double)exp_sel(z[i] - top, exp_mode);
    float offset = (float)log(sum);
    for (int64_t i = 0; i < n; i++) out[i] = z[i] - top - offset;
}

/* The N largest raw logits, ties to the lower index (the argmax convention),
 * with their logprobs. The reference has no top-N routine; this is the
 * definition the north star gives in terms of `logprobs`. */
void molla_oracle_top_logprobs(const float *z, int64_t n, int top_n, int32_t *ids, float *lps,
                               int exp_mode) {
    float top = z[0];
    for (int64_t i = 1; i < n; i++)
        if (z[i] > top) top = z[i];
    double sum = 0.0;
    for (int64_t i = 0; i < n; i++) sum += (double)exp_sel(z[i] - top, exp_mode);
    float offset = (float)log(sum);
    for (int j = 0; j < top_n; j++) {
        int64_t best = -1;
        for (int64_t i = 0; i < n; i++) {
            int taken = 0;
            for (int q = 0; q < j; q++)
                if (ids[q] == (int32_t)i) { taken = 1; break; }
            if (taken) continue;
            if (best < 0 || z[i] > z[best]) best = i;
        }
        if (best < 0) { ids[j] = -1; lps[j] = 0.0f; continue; }
        ids[j] = (int32_t)best;
        lps[j] = z[best] - top - offset;
    }
}

/* ---- the sampler: sample.mojo:157-594 ----------------------------------- */

typedef struct {
    int64_t vocab;
    int64_t *ids;
    float *vals;
    int64_t kept;
    /* config */
    float temperature, top_p, min_p, typical_p;
    float repeat_penalty, frequency_penalty, presence_penalty;
    int64_t top_k;
    uint64_t seed, drawn;
    /* window and bias (borrowed) */
    const int64_t *recent; int64_t filled; int window_on;
    const int64_t *bias_ids; const float *bias_vals; int64_t nbias;
    int exp_mode;
    int faithful_cost;
    int sorted; /* diagnostic: has a sort run */
    const uint32_t *mask; /* grammar mask of the row: bit t set = token t allowed (NULL = all) */
} sampler_t;

static int cfg_greedy(const sampler_t *s) { return s->temperature <= 0; }

static int cfg_penalizing(const sampler_t *s) {
    if (!s->window_on) return 0;
    return s->repeat_penalty != 1.0f || s->frequency_penalty != 0.0f ||
           s->presence_penalty != 0.0f;
}

static int64_t count_of(const sampler_t *s, int64_t token) {
    int64_t n = 0;
    for (int64_t i = 0; i < s->filled; i++)
        if (s->recent[i] == token) n++;
    return n;
}

static void swap_(sampler_t *s, int64_t a, int64_t b) {
    float v = s->vals[a]; s->vals[a] = s->vals[b]; s->vals[b] = v;
    int64_t i = s->ids[a]; s->ids[a] = s->ids[b]; s->ids[b] = i;
}

static void sift_(sampler_t *s, int64_t at, int64_t n) {
    int64_t root = at;
    for (;;) {
        int64_t child = root * 2 + 1;
        if (child >= n) return;
        if (child + 1 < n && s->vals[child + 1] > s->vals[child]) child += 1;
        if (s->vals[root] >= s->vals[child]) return;
        swap_(s, root, child);
        root = child;
    }
}

static void sort_(sampler_t *s) {
    int64_t n = s->kept;
    for (int64_t start = n / 2 - 1; start >= 0; start--) sift_(s, start, n);
    for (int64_t end = n - 1; end > 0; end--) {
        swap_(s, 0, end);
        sift_(s, 0, end);
    }
    int64_t i = 0, j = n - 1;
    while (i < j) { swap_(s, i, j); i++; j--; }
    s->sorted = 1;
}

static void bias_(sampler_t *s) {
    if (s->nbias <= 0) return;
    if (s->faithful_cost) {
        for (int64_t i = 0; i < s->kept; i++) {
            int64_t t = s->ids[i];
            for (int64_t j = 0; j < s->nbias; j++)
                if (s->bias_ids[j] == t) s->vals[i] += s->bias_vals[j];
        }
    } else { /* same additions in the same order, reached by index */
        for (int64_t j = 0; j < s->nbias; j++) {
            int64_t t = s->bias_ids[j];
            if (t >= 0 && t < s->kept) s->vals[t] += s->bias_vals[j];
        }
    }
}

static void penalise_one(sampler_t *s, int64_t i, int64_t n) {
    float v = s->vals[i];
    if (v > 0) v /= s->repeat_penalty;
    else v *= s->repeat_penalty;
    float fn = (float)n * s->frequency_penalty;
    v -= fn;
    v -= s->presence_penalty;
    s->vals[i] = v;
}

static void penalise_(sampler_t *s) {
    if (!cfg_penalizing(s)) return;
    if (s->faithful_cost) {
        for (int64_t i = 0; i < s->kept; i++) {
            int64_t n = count_of(s, s->ids[i]);
            if (n == 0) continue;
            penalise_one(s, i, n);
        }
    } else { /* same result: visit each distinct window token once */
        for (int64_t a = 0; a < s->filled; a++) {
            int64_t t = s->recent[a];
            if (t < 0 || t >= s->kept) continue;
            int first = 1;
            for (int64_t b = 0; b < a; b++)
                if (s->recent[b] == t) { first = 0; break; }
            if (!first) continue;
            penalise_one(s, t, count_of(s, t));
        }
    }
}

static void temperature_(sampler_t *s) {
    float t = s->temperature;
    if (t == 1.0f) return;
    for (int64_t i = 0; i < s->kept; i++) s->vals[i] /= t;
}

static float softmax_(sampler_t *s) {
    float top = s->vals[0];
    for (int64_t i = 1; i < s->kept; i++)
        if (s->vals[i] > top) top = s->vals[i];
    float sum = 0.0f;
    for (int64_t i = 0; i < s->kept; i++) {
        s->vals[i] = exp_sel(s->vals[i] - top, s->exp_mode);
        sum += s->vals[i];
    }
    if (sum <= 0) return sum;
    for (int64_t i = 0; i < s->kept; i++) s->vals[i] /= sum;
    return sum;
}

#define FLAG_TOPK_TIE 1u      /* p[k-1] == p[k]: which token made the cut is the sort's choice */
#define FLAG_TOPP_TIE 2u      /* the top-p cut splits a run of equal probabilities */
#define FLAG_CHOSEN_TIE 4u    /* the chosen token shares its probability with another kept one */
#define FLAG_CDF_EDGE 8u      /* |target - acc_i| < 1e-6 * sum at the nearest boundary */
#define FLAG_KEPT_TIE 16u     /* some two kept candidates share a probability */

static void top_k_(sampler_t *s, uint32_t *flags) {
    int64_t k = s->top_k;
    if (k <= 0 || k >= s->kept) return;
    sort_(s);
    if (s->vals[k - 1] == s->vals[k]) *flags |= FLAG_TOPK_TIE;
    s->kept = k;
}

static void top_p_(sampler_t *s, uint32_t *flags) {
    float p = s->top_p;
    if (p >= 1.0f || s->kept <= 1) return;
    int64_t before = s->kept;
    sort_(s);
    float sum = 0.0f;
    for (int64_t i = 0; i < s->kept; i++) {
        sum += s->vals[i];
        if (sum >= p) {
            if (i + 1 < before && s->vals[i] == s->vals[i + 1]) *flags |= FLAG_TOPP_TIE;
            s->kept = i + 1;
            return;
        }
    }
}

static void min_p_(sampler_t *s) {
    float floor_ = s->min_p;
    if (floor_ <= 0 || s->kept <= 1) return;
    float top = s->vals[0];
    for (int64_t i = 1; i < s->kept; i++)
        if (s->vals[i] > top) top = s->vals[i];
    float cut = top * floor_;
    int64_t write = 0;
    for (int64_t i = 0; i < s->kept; i++) {
        if (s->vals[i] >= cut) { swap_(s, write, i); write++; }
    }
    if (write > 0) s->kept = write;
}

static void typical_(sampler_t *s) {
    float p = s->typical_p;
    if (p >= 1.0f || s->kept <= 1) return;
    float entropy = 0.0f;
    for (int64_t i = 0; i < s->kept; i++)
        if (s->vals[i] > 0) entropy -= s->vals[i] * log_sel(s->vals[i], s->exp_mode);
    float *distance = (float *)malloc(sizeof(float) * (size_t)s->kept);
    for (int64_t i = 0; i < s->kept; i++) {
        float surprise = 0.0f;
        if (s->vals[i] > 0) surprise = -log_sel(s->vals[i], s->exp_mode);
        float d = surprise - entropy;
        distance[i] = d >= 0 ? d : -d;
    }
    for (int64_t i = 1; i < s->kept; i++) {
        int64_t j = i;
        while (j > 0 && distance[j - 1] > distance[j]) {
            float d = distance[j - 1]; distance[j - 1] = distance[j]; distance[j] = d;
            swap_(s, j - 1, j);
            j--;
        }
    }
    free(distance);
    float sum = 0.0f;
    for (int64_t i = 0; i < s->kept; i++) {
        sum += s->vals[i];
        if (sum >= p) { s->kept = i + 1; return; }
    }
}

typedef struct {
    float z_sum;      /* the softmax denominator (sequential fp32) */
    float keep_sum;   /* sum of the kept probabilities in _choose */
    float target;     /* draw * keep_sum */
    float chosen_p;   /* probability of the chosen token */
    int64_t kept_topk, kept_final, chosen_pos;
    uint32_t flags;
} diag_t;

static int64_t choose_(sampler_t *s, diag_t *d) {
    if (s->kept <= 0) return -1;
    float sum = 0.0f;
    for (int64_t i = 0; i < s->kept; i++) sum += s->vals[i];
    d->keep_sum = sum;
    if (sum <= 0) { d->chosen_pos = 0; return s->ids[0]; }
    float target = molla_oracle_draw(s->seed, s->drawn) * sum;
    d->target = target;
    float acc = 0.0f;
    int64_t at = s->kept - 1;
    float near_ = INFINITY;
    int found = 0;
    for (int64_t i = 0; i < s->kept; i++) {
        acc += s->vals[i];
        float gap = fabsf(target - acc);
        if (i + 1 < s->kept && gap < near_) near_ = gap;
        if (!found && target < acc) { at = i; found = 1; }
    }
    if (near_ < 1e-6f * sum) d->flags |= FLAG_CDF_EDGE;
    d->chosen_pos = at;
    d->chosen_p = s->vals[at];
    /* tie diagnostics over the kept set */
    for (int64_t i = 0; i < s->kept; i++)
        if (i != at && s->vals[i] == s->vals[at]) { d->flags |= FLAG_CHOSEN_TIE; break; }
    if (s->sorted) {
        for (int64_t i = 0; i + 1 < s->kept; i++)
            if (s->vals[i] == s->vals[i + 1]) { d->flags |= FLAG_KEPT_TIE; break; }
    }
    return s->ids[at];
}

/* pick(): sample.mojo:295-359. `penalised_out`, when given, receives the row
 * after bias and penalties and before temperature (vocabulary order). */
static int64_t pick_(sampler_t *s, const float *row, float *penalised_out, diag_t *d,
                     int32_t *kept_ids_out, int64_t kept_ids_cap) {
    memset(d, 0, sizeof(*d));
    s->sorted = 0;
    if (cfg_greedy(s) && !cfg_penalizing(s) && s->nbias <= 0 && !s->mask) {
        if (penalised_out) memcpy(penalised_out, row, sizeof(float) * (size_t)s->vocab);
        return molla_oracle_argmax(row, 0, s->vocab);
    }
    for (int64_t i = 0; i < s->vocab; i++) { s->ids[i] = i; s->vals[i] = row[i]; }
    s->kept = s->vocab;
    if (s->mask) {
        /* `_mask` (sample.mojo:371-379) is where a grammar drops the tokens it forbids, first of
         * all filters; the reference ships it empty. Dropping = the candidate is gone: what is
         * left keeps its order. Nothing left: "every candidate was filtered out" (:578-579). */
        int64_t w = 0;
        for (int64_t i = 0; i < s->vocab; i++)
            if ((s->mask[i >> 5] >> (i & 31)) & 1u) { s->ids[w] = i; s->vals[w] = row[i]; w++; }
        s->kept = w;
        if (w == 0) return -1;
    }
    bias_(s);
    penalise_(s);
    if (penalised_out) memcpy(penalised_out, s->vals, sizeof(float) * (size_t)s->vocab);
    if (cfg_greedy(s)) {
        int64_t best = 0;
        for (int64_t i = 1; i < s->kept; i++)
            if (s->vals[i] > s->vals[best]) best = i;
        return s->ids[best];
    }
    temperature_(s);
    d->z_sum = softmax_(s);
    top_k_(s, &d->flags);
    d->kept_topk = s->kept;
    if (kept_ids_out) {
        int64_t n = s->kept < kept_ids_cap ? s->kept : kept_ids_cap;
        if (s->sorted)
            for (int64_t i = 0; i < n; i++) kept_ids_out[i] = (int32_t)s->ids[i];
    }
    top_p_(s, &d->flags);
    min_p_(s);
    typical_(s);
    d->kept_final = s->kept;
    return choose_(s, d);
}

/*
 * Batched driver: row r of `logits` (row-major, `row_stride` floats between
 * rows) is sampled with the r-th entry of every per-row array, exactly as the
 * decode loop calls `streams[i].sampler.pick(self.logits, r)` once per answered
 * row (src/molla/engine/batch.mojo:509-511). The window of row r is
 * hist[hist_off[r] .. hist_off[r+1]) (the filled part of the ring; order does
 * not matter to count_of). `window_on[r]` is repeat_last_n > 0.
 *
 * Outputs other than `tokens` are optional (NULL to skip).
 * Returns 0, or -1 on a bad argument.
 */
int molla_oracle_pick_batch_masked(
    const uint32_t *mask, int64_t mask_stride_words,
    const float *logits, int64_t row_stride, int32_t B, int32_t V,
    const float *temperature, const int32_t *top_k, const float *top_p, const float *min_p,
    const float *typical_p, const float *repeat_penalty, const float *frequency_penalty,
    const float *presence_penalty, const uint8_t *window_on, const uint64_t *seed,
    const uint64_t *drawn, const int64_t *hist, const int32_t *hist_off, const int64_t *bias_ids,
    const float *bias_vals, const int32_t *bias_off, int32_t exp_mode, int32_t faithful_cost,
    int32_t nthreads,
    int32_t *tokens, float *penalised, float *z_sum, float *keep_sum, float *target,
    float *chosen_p, int32_t *kept_topk, int32_t *kept_final, uint32_t *flags,
    int32_t *kept_ids, int32_t kept_ids_cap) {
    if (!logits || !tokens || B < 0 || V <= 0) return -1;
    if (nthreads < 1) nthreads = 1;
#ifdef _OPENMP
#pragma omp parallel num_threads(nthreads)
#endif
    {
        sampler_t s;
        memset(&s, 0, sizeof(s));
        s.vocab = V;
        s.ids = (int64_t *)malloc(sizeof(int64_t) * (size_t)V);
        s.vals = (float *)malloc(sizeof(float) * (size_t)V);
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1)
#endif
        for (int32_t r = 0; r < B; r++) {
            s.temperature = temperature[r];
            s.top_k = top_k ? top_k[r] : 0;
            s.top_p = top_p ? top_p[r] : 1.0f;
            s.min_p = min_p ? min_p[r] : 0.0f;
            s.typical_p = typical_p ? typical_p[r] : 1.0f;
            s.repeat_penalty = repeat_penalty ? repeat_penalty[r] : 1.0f;
            s.frequency_penalty = frequency_penalty ? frequency_penalty[r] : 0.0f;
            s.presence_penalty = presence_penalty ? presence_penalty[r] : 0.0f;
            s.seed = seed ? seed[r] : 0;
            s.drawn = drawn ? drawn[r] : 0;
            if (hist && hist_off) {
                s.recent = hist + hist_off[r];
                s.filled = hist_off[r + 1] - hist_off[r];
            } else { s.recent = NULL; s.filled = 0; }
            s.window_on = window_on ? window_on[r] : (s.filled > 0);
            if (bias_ids && bias_off) {
                s.bias_ids = bias_ids + bias_off[r];
                s.bias_vals = bias_vals + bias_off[r];
                s.nbias = bias_off[r + 1] - bias_off[r];
            } else { s.bias_ids = NULL; s.bias_vals = NULL; s.nbias = 0; }
            s.exp_mode = exp_mode;
            s.faithful_cost = faithful_cost;
            s.mask = mask ? mask + (int64_t)r * mask_stride_words : NULL;
            if (s.mask) s.faithful_cost = 1; /* the shortcuts index candidates by token id */
            diag_t d;
            int64_t tok = pick_(&s, logits + (int64_t)r * row_stride,
                                penalised ? penalised + (int64_t)r * V : NULL, &d,
                                kept_ids ? kept_ids + (int64_t)r * kept_ids_cap : NULL,
                                kept_ids_cap);
            tokens[r] = (int32_t)tok;
            if (z_sum) z_sum[r] = d.z_sum;
            if (keep_sum) keep_sum[r] = d.keep_sum;
            if (target) target[r] = d.target;
            if (chosen_p) chosen_p[r] = d.chosen_p;
            if (kept_topk) kept_topk[r] = (int32_t)d.kept_topk;
            if (kept_final) kept_final[r] = (int32_t)d.kept_final;
            if (flags) flags[r] = d.flags;
        }
        free(s.ids);
        free(s.vals);
    }
    return 0;
}

/* Batched logprob outputs: chosen-token logprob and the top-N, from the raw row. */
int molla_oracle_pick_batch(
    const float *logits, int64_t row_stride, int32_t B, int32_t V,
    const float *temperature, const int32_t *top_k, const float *top_p, const float *min_p,
    const float *typical_p, const float *repeat_penalty, const float *frequency_penalty,
    const float *presence_penalty, const uint8_t *window_on, const uint64_t *seed,
    const uint64_t *drawn, const int64_t *hist, const int32_t *hist_off, const int64_t *bias_ids,
    const float *bias_vals, const int32_t *bias_off, int32_t exp_mode, int32_t faithful_cost,
    int32_t nthreads,
    int32_t *tokens, float *penalised, float *z_sum, float *keep_sum, float *target,
    float *chosen_p, int32_t *kept_topk, int32_t *kept_final, uint32_t *flags,
    int32_t *kept_ids, int32_t kept_ids_cap) {
    return molla_oracle_pick_batch_masked(NULL, 0, logits, row_stride, B, V, temperature, top_k, top_p, min_p,
                                          typical_p, repeat_penalty, frequency_penalty, presence_penalty, window_on,
                                          seed, drawn, hist, hist_off, bias_ids, bias_vals, bias_off, exp_mode,
                                          faithful_cost, nthreads, tokens, penalised, z_sum, keep_sum, target, chosen_p,
                                          kept_topk, kept_final, flags, kept_ids, kept_ids_cap);
}

int molla_oracle_logprobs_batch(const float *logits, int64_t row_stride, int32_t B, int32_t V,
                                const int32_t *tokens, int32_t top_n, int32_t exp_mode,
                                int32_t nthreads, float *chosen_lp, int32_t *top_ids,
                                float *top_lps) {
    if (!logits || B < 0 || V <= 0 || top_n < 0) return -1;
    if (nthreads < 1) nthreads = 1;
#ifdef _OPENMP
#pragma omp parallel for num_threads(nthreads) schedule(dynamic, 1)
#endif
    for (int32_t r = 0; r < B; r++) {
        const float *z = logits + (int64_t)r * row_stride;
        float top = z[0];
        for (int64_t i = 1; i < V; i++)
            if (z[i] > top) top = z[i];
        double sum = 0.0;
        for (int64_t i = 0; i < V; i++) sum += (double)exp_sel(z[i] - top, exp_mode);
        float offset = (float)log(sum);
        if (chosen_lp && tokens) chosen_lp[r] = z[tokens[r]] - top - offset;
        if (top_n > 0 && top_ids && top_lps) {
            int32_t *ids = top_ids + (int64_t)r * top_n;
            float *lps = top_lps + (int64_t)r * top_n;
            for (int j = 0; j < top_n; j++) {
                int64_t best = -1;
                for (int64_t i = 0; i < V; i++) {
                    int taken = 0;
                    for (int q = 0; q < j; q++)
                        if (ids[q] == (int32_t)i) { taken = 1; break; }
                    if (taken) continue;
                    if (best < 0 || z[i] > z[best]) best = i;
                }
                if (best < 0) { ids[j] = -1; lps[j] = 0.0f; continue; }
                ids[j] = (int32_t)best;
                lps[j] = z[best] - top - offset;
            }
        }
    }
    return 0;
}

int molla_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
