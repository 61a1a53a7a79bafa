/*
 * TEST INFRASTRUCTURE - CPU oracle for the Gefen hot path. Not part of the product: only tests,
 * the smoke check and the cpu_baseline leg of bench.py load this library.
 *
 * A plain-C restatement of the arithmetic of the reference's CUDA kernels, one function per
 * kernel, each citing the reference lines it follows. The reference kernels are plain fp32/fp64
 * scalar arithmetic, so they can be restated exactly; what the source does not fix is how nvcc
 * contracts a*b+c*d into FMAs. `contract` selects that:
 *   0 = every operation rounded separately (the literal source),
 *   1 = fma(a, b, c*d) for sums of two products and fma(-a, b, p) for p - a*b, which is what
 *       nvcc -O3 (fmad on, the reference's build flags, kernels/_build_notice.py:410-411) emits.
 * Compile with -ffp-contract=off so that the compiler adds no contraction of its own.
 *
 * Pinning: compared on a B200 with the reference's own kernels built from its sources
 * (oracle/build_ref.py) and, for fp32, with the reference's PyTorch CPU path through the golden
 * fixtures in tests/golden.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define DT_F32 0
#define DT_F16 1
#define DT_BF16 2
#define DT_F64 3

static int g_contract = 1;
static int g_p1_variant = 0;   /* which product the period-1 second-moment update fuses, see below */
static int g_p1_m_variant = 1; /* which product the period-1 momentum update fuses: measured on a B200 against the
                                  reference build, that kernel fuses (1-beta1)*g, unlike the other step kernels */
void oracle_set_period1_m_variant(int v) { g_p1_m_variant = v; }
void oracle_set_contraction(int mode) { g_contract = mode; }
void oracle_set_period1_variant(int v) { g_p1_variant = v; }
int oracle_get_contraction(void) { return g_contract; }

/* ---------------------------------------------------------------- dtype helpers */
static inline float bf16_to_f32(uint16_t h) {
    union { uint32_t u; float f; } c; c.u = ((uint32_t)h) << 16; return c.f;
}
static inline uint16_t f32_to_bf16(float f) {   /* round to nearest even, NaN kept quiet */
    union { uint32_t u; float f; } c; c.f = f;
    if ((c.u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((c.u >> 16) | 0x0040u);
    const uint32_t lsb = (c.u >> 16) & 1u;
    c.u += 0x7fffu + lsb;
    return (uint16_t)(c.u >> 16);
}
static inline float f16_to_f32(uint16_t h) { _Float16 x; memcpy(&x, &h, 2); return (float)x; }
static inline uint16_t f32_to_f16(float f) { _Float16 x = (_Float16)f; uint16_t h; memcpy(&h, &x, 2); return h; }

static inline float load_as_float(const void* base, int64_t i, int dt) {
    switch (dt) {
        case DT_F32: return ((const float*)base)[i];
        case DT_F16: return f16_to_f32(((const uint16_t*)base)[i]);
        case DT_BF16: return bf16_to_f32(((const uint16_t*)base)[i]);
        default: return (float)((const double*)base)[i];
    }
}
static inline void store_from_float(void* base, int64_t i, int dt, float v) {
    switch (dt) {
        case DT_F32: ((float*)base)[i] = v; break;
        case DT_F16: ((uint16_t*)base)[i] = f32_to_f16(v); break;
        case DT_BF16: ((uint16_t*)base)[i] = f32_to_bf16(v); break;
        default: ((double*)base)[i] = (double)v; break;
    }
}
static inline float round_to(int dt, float v) {
    if (dt == DT_BF16) return bf16_to_f32(f32_to_bf16(v));
    if (dt == DT_F16) return f16_to_f32(f32_to_f16(v));
    return v;
}

static inline float two_products(float a, float b, float c, float d) {   /* a*b + c*d */
    return g_contract ? fmaf(a, b, c * d) : a * b + c * d;
}
static inline float sub_product(float p, float a, float b) {             /* p - a*b */
    return g_contract ? fmaf(-a, b, p) : p - a * b;
}
static inline float acc_square(float acc, float x) {                     /* acc + x*x */
    return g_contract ? fmaf(x, x, acc) : acc + x * x;
}

/* reference: choose_threads, automatic_gefen_fused_kernel.cu:409-418 */
static int choose_threads(int64_t period) {
    int threads = 32;
    while (threads < period && threads < 256) threads <<= 1;
    return threads;
}

/* reference: nearest_codebook_index, automatic_gefen_fused_kernel.cu:59-90 */
int oracle_nearest_index(float x, const float* cb, int k) {
    int left = 0, right = k;
    while (left < right) {
        const int mid = left + (right - left) / 2;
        if (cb[mid] < x) left = mid + 1; else right = mid;
    }
    int r = left;
    if (r < 0) r = 0; else if (r >= k) r = k - 1;
    int l = r - 1;
    if (l < 0) l = 0;
    const float dl = fabsf(x - cb[l]);
    const float dr = fabsf(x - cb[r]);
    return dl <= dr ? l : r;
}

void oracle_nearest_indices(const float* x, int64_t n, const float* cb, int k, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = (uint8_t)oracle_nearest_index(x[i], cb, k);
}

/* reference: automatic_vmean_update_kernel, automatic_vmean_kernel.cu:12-51.
 * Thread-strided partial sums followed by the stride-halving tree, as the kernel does. */
void oracle_vmean_update(void* vmean, int v_dt, const void* g, int g_dt, int64_t nb, int64_t period, double beta2_d) {
    const float beta2 = (float)beta2_d;
    const int T = choose_threads(period);
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        float part[256];
        for (int t = 0; t < T; ++t) {
            float s = 0.0f;
            for (int64_t off = t; off < period; off += T) {
                const float gv = load_as_float(g, b * period + off, g_dt);
                s = acc_square(s, gv);
            }
            part[t] = s;
        }
        for (int stride = T / 2; stride > 0; stride >>= 1)
            for (int t = 0; t < stride; ++t) part[t] += part[t + stride];
        const float mean_sq = part[0] / (float)period;
        const float prev = load_as_float(vmean, b, v_dt);
        store_from_float(vmean, b, v_dt, two_products(beta2, prev, 1.0f - beta2, mean_sq));
    }
}

/* The per-block body shared by the fused update kernels.
 * mode 0: from_vmean (automatic_gefen_fused_kernel.cu:239-318)
 * mode 1: precomputed stepsize (:92-167)
 * mode 2: GefenMuon momentum, dense output to `p` (:169-237) */
static void fused_block(int mode, void* p, const void* g, int s_dt, uint8_t* codes, void* mag, int mag_dt,
                        const void* v, int v_dt, const float* stepsize, const float* cb, int k, int64_t period,
                        int64_t b, float beta1, float lr, float bc1, float bc2, float eps) {
    const int64_t start = b * period;
    const float old_mag = load_as_float(mag, b, mag_dt);
    float step = 0.0f;
    if (mode == 0) {
        const float corrected = load_as_float(v, b, v_dt) / bc2;
        step = (1.0f / bc1) / (sqrtf(corrected) + eps);
    } else if (mode == 1) {
        step = stepsize[b];
    }
    float absmax = 0.0f;
    for (int64_t i = 0; i < period; ++i) {
        const float cur = old_mag * cb[codes[start + i]];
        const float u = two_products(beta1, cur, 1.0f - beta1, load_as_float(g, start + i, s_dt));
        const float a = fabsf(u);
        if (a > absmax) absmax = a;
    }
    store_from_float(mag, b, mag_dt, absmax);
    for (int64_t i = 0; i < period; ++i) {
        const float cur = old_mag * cb[codes[start + i]];
        const float u = two_products(beta1, cur, 1.0f - beta1, load_as_float(g, start + i, s_dt));
        float x = 0.0f;
        if (absmax > 0.0f) x = u / absmax;
        const int q = oracle_nearest_index(x, cb, k);
        codes[start + i] = (uint8_t)q;
        if (mode == 2) {
            store_from_float(p, start + i, s_dt, cb[q] * absmax);
        } else if (lr != 0.0f) {
            const float qv = cb[q] * absmax;
            store_from_float(p, start + i, s_dt, sub_product(load_as_float(p, start + i, s_dt), qv * step, lr));
        }
    }
}

void oracle_fused_update_from_vmean(void* p, const void* g, int s_dt, uint8_t* codes, void* mag, int mag_dt,
                                    const void* v, int v_dt, const float* cb, int k, int64_t nb, int64_t period,
                                    double beta1, double lr, double bc1, double bc2, double eps) {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b)
        fused_block(0, p, g, s_dt, codes, mag, mag_dt, v, v_dt, NULL, cb, k, period, b, (float)beta1, (float)lr,
                    (float)bc1, (float)bc2, (float)eps);
}

void oracle_fused_update(void* p, const void* g, int s_dt, uint8_t* codes, void* mag, int mag_dt,
                         const float* stepsize, const float* cb, int k, int64_t nb, int64_t period, double beta1,
                         double lr) {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b)
        fused_block(1, p, g, s_dt, codes, mag, mag_dt, NULL, 0, stepsize, cb, k, period, b, (float)beta1, (float)lr,
                    1.0f, 1.0f, 0.0f);
}

void oracle_muon_momentum(const void* g, int s_dt, uint8_t* codes, void* mag, int mag_dt, const float* cb, int k,
                          void* out, int64_t nb, int64_t period, double beta1) {
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b)
        fused_block(2, out, g, s_dt, codes, mag, mag_dt, NULL, 0, NULL, cb, k, period, b, (float)beta1, 0.0f, 1.0f,
                    1.0f, 0.0f);
}

static inline float p1_momentum(float beta1, float cur, float g) {
    if (!g_contract || g_p1_m_variant == 2) return beta1 * cur + (1.0f - beta1) * g;
    if (g_p1_m_variant == 1) return fmaf(1.0f - beta1, g, beta1 * cur);
    return fmaf(beta1, cur, (1.0f - beta1) * g);
}

/* reference: automatic_gefen_period1_update_kernel, automatic_gefen_fused_kernel.cu:320-407 */
void oracle_period1_update(void* p, const void* g, int s_dt, uint8_t* codes, void* mag, int mag_dt, void* v, int v_dt,
                           const float* cb, int k, int64_t numel, int64_t divisor, double beta1_d, double beta2_d,
                           double lr_d, double bc1_d, double bc2_d, double eps_d) {
    const float beta1 = (float)beta1_d, beta2 = (float)beta2_d, lr = (float)lr_d;
    const float bc1 = (float)bc1_d, bc2 = (float)bc2_d, eps = (float)eps_d;
    const int64_t nb = numel / divisor;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; ++b) {
        const int64_t start = b * divisor;
        const float old_mag = load_as_float(mag, b, mag_dt);
        float absmax = 0.0f;
        for (int64_t i = start; i < start + divisor; ++i) {
            const float gv = load_as_float(g, i, s_dt);
            const float prev = load_as_float(v, i, v_dt);
            /* beta2*prev + ((1-beta2)*g)*g */
            float nv;
            if (!g_contract) nv = beta2 * prev + (1.0f - beta2) * gv * gv;
            else if (g_p1_variant == 0) nv = fmaf(beta2, prev, ((1.0f - beta2) * gv) * gv);
            else nv = fmaf((1.0f - beta2) * gv, gv, beta2 * prev);
            store_from_float(v, i, v_dt, nv);
            const float u = p1_momentum(beta1, old_mag * cb[codes[i]], gv);
            const float a = fabsf(u);
            if (a > absmax) absmax = a;
        }
        store_from_float(mag, b, mag_dt, absmax);
        for (int64_t i = start; i < start + divisor; ++i) {
            const float gv = load_as_float(g, i, s_dt);
            const float u = p1_momentum(beta1, old_mag * cb[codes[i]], gv);
            float x = 0.0f;
            if (absmax > 0.0f) x = u / absmax;
            const int q = oracle_nearest_index(x, cb, k);
            codes[i] = (uint8_t)q;
            const float corrected = load_as_float(v, i, v_dt) / bc2;
            const float step = (1.0f / bc1) / (sqrtf(corrected) + eps);
            const float qv = cb[q] * absmax;
            store_from_float(p, i, s_dt, sub_product(load_as_float(p, i, s_dt), qv * step, lr));
        }
    }
}

/* Decoupled weight decay as torch applies it before the kernel: p.mul_(1 - lr*wd) in the
 * parameter dtype, the scalar rounded to float first (reference: gefen.py:1280-1281). */
void oracle_weight_decay(void* p, int s_dt, int64_t numel, double lr, double wd) {
    const double scale = 1.0 - lr * wd;
    if (s_dt == DT_F64) {
        double* pd = (double*)p;
        for (int64_t i = 0; i < numel; ++i) pd[i] *= scale;
        return;
    }
    const float m = (float)scale;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < numel; ++i) store_from_float(p, i, s_dt, load_as_float(p, i, s_dt) * m);
}

/* reference: gefen_exact_histogram_kernel, exact_histogram_fused_kernel.cu:17-85 */
void oracle_histogram(const void* g, int dt, int64_t numel, int64_t period, int64_t* counts, int bins) {
    const int64_t nb = numel / period;
    const float scale = 0.5f * (float)bins;
    for (int64_t b = 0; b < nb; ++b) {
        float absmax = 0.0f;
        for (int64_t i = 0; i < period; ++i) {
            const float a = fabsf(load_as_float(g, b * period + i, dt));
            if (a > absmax) absmax = a;
        }
        for (int64_t i = 0; i < period; ++i) {
            const float gv = load_as_float(g, b * period + i, dt);
            float x = 0.0f;
            if (absmax > 0.0f) x = gv / absmax;
            int bin = (int)floorf((x + 1.0f) * scale);
            if (bin < 0) bin = 0; else if (bin >= bins) bin = bins - 1;
            counts[bin] += 1;
        }
    }
}

/* reference: average_adjacent_log_block_mean_difference_kernel + host division,
 * period_variance_kernel.cu:108-165, :392-395. Returns the score; *invalid gets the count of
 * non-positive log inputs (the reference raises when it is non-zero). The order of the fp64
 * additions is the kernel's per-thread one followed by a plain left-to-right sum over pairs
 * (the kernel's atomics have no fixed order). */
double oracle_adjacent_log_score(const void* values, int dt, int64_t numel, int64_t period, int squared, double eps,
                                 double* invalid) {
    const int64_t nb = numel / period;
    double* means = (double*)malloc(sizeof(double) * (size_t)nb);
    double bad = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : bad)
    for (int64_t b = 0; b < nb; ++b) {
        double s = 0.0;
        for (int64_t i = 0; i < period; ++i) {
            const double raw = (double)load_as_float(values, b * period + i, dt);
            const double x = (squared ? raw : raw * raw) + eps;
            if (x <= 0.0) bad += 1.0; else s += log(x);
        }
        means[b] = s / (double)period;
    }
    double total = 0.0;
    for (int64_t b = 0; b + 1 < nb; ++b) total += fabs(means[b + 1] - means[b]);
    free(means);
    *invalid = bad;
    return total / (double)(nb - 1);
}

/* The same score for several candidate periods of one tensor, as the reference's period search asks
 * for them one after the other (partitioning.py:259-268). The logarithm of an element does not depend
 * on the period, so it is taken once into a scratch array; every block sum then adds the same values
 * in the same left-to-right order as oracle_adjacent_log_score, which makes the scores bit-identical
 * to calling that function per period (a CPU test holds the two against each other). Returns 0, or
 * -1 when the scratch array cannot be allocated. */
int oracle_adjacent_log_scores_many(const void* values, int dt, int64_t numel, const int64_t* periods, int n_periods,
                                    int squared, double eps, double* scores, double* invalid) {
    double* logs = (double*)malloc(sizeof(double) * (size_t)(numel > 0 ? numel : 1));
    if (logs == NULL) return -1;
    double bad = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : bad)
    for (int64_t i = 0; i < numel; ++i) {
        const double raw = (double)load_as_float(values, i, dt);
        const double x = (squared ? raw : raw * raw) + eps;
        if (x <= 0.0) { bad += 1.0; logs[i] = 0.0; } else logs[i] = log(x);
    }
    for (int k = 0; k < n_periods; ++k) {
        const int64_t period = periods[k];
        const int64_t nb = numel / period;
        double* means = (double*)malloc(sizeof(double) * (size_t)(nb > 0 ? nb : 1));
        if (means == NULL) { free(logs); return -1; }
#pragma omp parallel for schedule(static)
        for (int64_t b = 0; b < nb; ++b) {
            double s = 0.0;
            const double* src = logs + b * period;
            for (int64_t i = 0; i < period; ++i) s += src[i];
            means[b] = s / (double)period;
        }
        double total = 0.0;
        for (int64_t b = 0; b + 1 < nb; ++b) total += fabs(means[b + 1] - means[b]);
        free(means);
        scores[k] = total / (double)(nb - 1);
    }
    free(logs);
    *invalid = bad;
    return 0;
}

/* reference: average_within_block_variance_kernel / ..._coefficient_of_variation_kernel,
 * period_variance_kernel.cu:13-106 (fp32 sums per block). stats: [sum_var] or [sum_cov, n_pos, n_neg]. */
void oracle_block_moments(const void* values, int dt, int64_t numel, int64_t period, int squared, int cov,
                          double* stats) {
    const int64_t nb = numel / period;
    for (int64_t b = 0; b < nb; ++b) {
        float sx = 0.0f, sx2 = 0.0f;
        for (int64_t i = 0; i < period; ++i) {
            const float v = load_as_float(values, b * period + i, dt);
            const float x = squared ? v : v * v;
            sx += x;
            sx2 = acc_square(sx2, x);
        }
        const float mean = sx / (float)period;
        float var = sx2 / (float)period;
        var -= mean * mean;
        if (var < 0.0f) var = 0.0f;
        if (!cov) stats[0] += (double)var;
        else if (mean < 0.0f) stats[2] += 1.0;
        else if (mean > 0.0f) { stats[0] += (double)(sqrtf(var) / mean); stats[1] += 1.0; }
    }
}

/* reference: gefen_lloyd_accumulate_kernel, lloyd_max_fused_kernel.cu:50-118 (sums in fp64 here
 * to give an order-free yardstick for the fp32 atomics of the kernels) */
void oracle_lloyd_accumulate(const void* g, int dt, int64_t numel, int64_t period, const float* cb, int k,
                             double* sums, int64_t* counts) {
    const int64_t nb = numel / period;
    for (int64_t b = 0; b < nb; ++b) {
        float absmax = 0.0f;
        for (int64_t i = 0; i < period; ++i) {
            const float a = fabsf(load_as_float(g, b * period + i, dt));
            if (a > absmax) absmax = a;
        }
        for (int64_t i = 0; i < period; ++i) {
            const float gv = load_as_float(g, b * period + i, dt);
            float x = 0.0f;
            if (absmax > 0.0f) x = gv / absmax;
            const int e = oracle_nearest_index(x, cb, k);
            sums[e] += (double)x;
            counts[e] += 1;
        }
    }
}

/* reference: gefen_lloyd_mse_kernel, lloyd_max_fused_kernel.cu:120-195 (fp64 accumulation) */
void oracle_lloyd_mse(const void* g, int dt, int64_t numel, int64_t period, const float* old_cb, const float* new_cb,
                      int k, double* out2) {
    const int64_t nb = numel / period;
    double en = 0.0, eo = 0.0;
    for (int64_t b = 0; b < nb; ++b) {
        float absmax = 0.0f;
        for (int64_t i = 0; i < period; ++i) {
            const float a = fabsf(load_as_float(g, b * period + i, dt));
            if (a > absmax) absmax = a;
        }
        for (int64_t i = 0; i < period; ++i) {
            const float gv = load_as_float(g, b * period + i, dt);
            float x = 0.0f;
            if (absmax > 0.0f) x = gv / absmax;
            const float err = x - new_cb[oracle_nearest_index(x, old_cb, k)];
            en += (double)(err * err);
            const float oe = err * absmax;
            eo += (double)(oe * oe);
        }
    }
    out2[0] = en;
    out2[1] = eo;
}

/* reference: _run_exact_dp_numba / _run_exact_dp_python, quantization.py:92-203.
 * prefix_* hold num_points+1 doubles. Writes the K centres unsorted; returns 0 on success. */
int oracle_exact_dp(const double* pw, const double* pwx, const double* pwx2, int num_points, int K, int force,
                    float* codebook) {
    const int64_t n1 = (int64_t)num_points + 1;
    double* prev = (double*)malloc(sizeof(double) * (size_t)n1);
    double* cur = (double*)malloc(sizeof(double) * (size_t)n1);
    int* back = (int*)malloc(sizeof(int) * (size_t)(n1 * (K + 1)));
    if (!prev || !cur || !back) return -1;
    for (int64_t i = 0; i < n1; ++i) prev[i] = INFINITY;
    prev[0] = 0.0;
    for (int c = 1; c <= K; ++c) {
        for (int64_t i = 0; i < n1; ++i) cur[i] = INFINITY;
#pragma omp parallel for schedule(dynamic, 16)
        for (int e = c; e <= num_points; ++e) {
            double best = INFINITY;
            int best_s = -1;
            for (int s = c; s <= e; ++s) {
                const double sw = pw[e] - pw[s - 1];
                const double swx = pwx[e] - pwx[s - 1];
                const double swx2 = pwx2[e] - pwx2[s - 1];
                double cost;
                if (force && c == 1) { const double fc = -1.0; cost = swx2 - 2.0 * fc * swx + fc * fc * sw; }
                else if (force && c == K) { const double fc = 1.0; cost = swx2 - 2.0 * fc * swx + fc * fc * sw; }
                else cost = swx2 - (swx * swx) / sw;
                const double cand = prev[s - 1] + cost;
                if (cand < best) { best = cand; best_s = s; }
            }
            cur[e] = best;
            back[(int64_t)c * n1 + e] = best_s;
        }
        double* t = prev; prev = cur; cur = t;
    }
    int e = num_points;
    int rc = 0;
    for (int c = K; c >= 1; --c) {
        const int s = back[(int64_t)c * n1 + e];
        if (s < 1) { rc = -2; break; }
        if (force && c == 1) codebook[c - 1] = -1.0f;
        else if (force && c == K) codebook[c - 1] = 1.0f;
        else codebook[c - 1] = (float)((pwx[e] - pwx[s - 1]) / (pw[e] - pw[s - 1]));
        e = s - 1;
    }
    free(prev); free(cur); free(back);
    return rc;
}
