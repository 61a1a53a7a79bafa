// One-off calibration kernels: the exact integer histogram of block-normalised gradients, the
// block-period scores and the Lloyd-Max accumulation / MSE kernels.
//
// Reference behaviour:
//   histogram   kernels/exact_histogram_fused_kernel.cu:17-85
//   scores      kernels/period_variance_kernel.cu:13-165 and the host post-ops at :242, :311-317, :392-395
//   Lloyd-Max   kernels/lloyd_max_fused_kernel.cu:50-195
//
// All of them are one read of the gradient from HBM (the reference reads it twice per kernel and,
// for the adjacent-log score, twice per candidate period). A warp owns a block; the second look at
// a block's elements, where one is needed, comes from L1.
#include "common.cuh"

#include <algorithm>
#include <vector>

namespace gefen {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

static int persistent_grid(long long groups, int groups_per_cta, int ctas_per_sm) {
    long long ctas = (groups + groups_per_cta - 1) / groups_per_cta;
    const long long cap = static_cast<long long>(sm_count()) * ctas_per_sm;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return static_cast<int>(ctas);
}

// NaN-ignoring max |g| over one block, by one warp (GROUP=32) or one CTA (GROUP=256).
template <typename S, int GROUP>
__device__ __forceinline__ float block_absmax(const S* g, long long period, int tig, float* red) {
    float m = 0.0f;
    for (long long i = tig; i < period; i += GROUP) m = fmaxf(m, fabsf(ScalarIO<S>::load(g + i)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (GROUP > 32) {
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
        __syncthreads();
        m = red[0];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) m = fmaxf(m, red[w]);
    }
    return m;
}

// ------------------------------------------------------------------------------- vector access
// Eight consecutive elements (16 bytes of a 2-byte type, 32 bytes of fp32) as floats; the pointer is
// 16-byte aligned. Calibration reads every block twice: the second look hits L1.
template <typename S> __device__ __forceinline__ void load8(const S* p, float (&f)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
template <> __device__ __forceinline__ void load8<__half>(const __half* p, float (&f)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}
template <> __device__ __forceinline__ void load8<double>(const double* p, float (&f)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(p[i]);
}

// NaN-ignoring max |v| over the eight elements at p, folded into m (fmaxf semantics, as block_absmax).
template <typename S> __device__ __forceinline__ float absmax8(const S* p, float m) {
    float f[8];
    load8<S>(p, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
    return m;
}
// bf16: two elements per instruction on the packed pipe (max of two bf16 values is exact; NaN loses).
template <> __device__ __forceinline__ float absmax8<__nv_bfloat16>(const __nv_bfloat16* p, float m) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const __nv_bfloat162 b = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    const __nv_bfloat162 c = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw.z));
    const __nv_bfloat162 d = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&raw.w));
    const __nv_bfloat162 top = __hmax2(__hmax2(a, b), __hmax2(c, d));
    return fmaxf(m, fmaxf(__low2float(top), __high2float(top)));
}

// x = v / absmax as the reference divides (IEEE), through the block's reciprocal where that is exact.
struct BlockDivider {
    float absmax, rinv;
    bool fast, nonzero;
    __device__ __forceinline__ explicit BlockDivider(float a) : absmax(a) {
        nonzero = a > 0.0f;
        fast = div_range_ok(a);
        rinv = fast ? 1.0f / a : 0.0f;
    }
    __device__ __forceinline__ float operator()(float v) const {
        if (fast) return div_by_block_constant(v, absmax, rinv);
        return nonzero ? v / absmax : 0.0f;
    }
    // The two cases apart, for loops that decide once per block which one they need (the choice is the same
    // for every element of a block; a test per element costs a branch per element).
    __device__ __forceinline__ float quick(float v) const { return div_by_block_constant(v, absmax, rinv); }
    __device__ __forceinline__ float careful(float v) const { return nonzero ? v / absmax : 0.0f; }
};

// ------------------------------------------------------------------------------- histogram
// bin = clamp(floor((g/absmax + 1) * bins/2), 0, bins-1); counts are integers and therefore
// independent of the order of accumulation. One warp per block (VEC: 128-bit loads, eight elements
// per lane and access) or one CTA per very long block. Every element is one shared-memory atomic
// on the CTA's histogram: the values of a block are bell-shaped over a few hundred bins, so the
// lanes of a warp rarely meet in one bin, and the hardware serialises those that do.
template <typename S, int GROUP, bool VEC, bool POW2>
__global__ void __launch_bounds__(kThreads) histogram_kernel(const S* __restrict__ g, long long period,
                                                             long long num_blocks, int bins,
                                                             unsigned long long* __restrict__ counts) {
    __shared__ unsigned int hist[4096 + 1];   // one spare counter for x == 1 (see below)
    __shared__ float red[kWarps];
    for (int i = threadIdx.x; i <= bins; i += kThreads) hist[i] = 0u;
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int tig = GROUP == 32 ? lane : static_cast<int>(threadIdx.x);
    const long long group0 = GROUP == 32 ? static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5)
                                         : static_cast<long long>(blockIdx.x);
    const long long stride = GROUP == 32 ? static_cast<long long>(gridDim.x) * kWarps : static_cast<long long>(gridDim.x);
    const float scale = 0.5f * static_cast<float>(bins);
    const int last_bin = bins - 1;
    unsigned long long since_flush = 0;

    for (long long b = group0; b < num_blocks; b += stride) {
        const S* gb = g + b * period;
        if (VEC) {   // GROUP == 32, period a multiple of 8, 16-byte aligned blocks
            const int nchunks = static_cast<int>(period >> 3);
            float m = 0.0f;
            for (int c = lane; c < nchunks; c += 32) m = absmax8<S>(gb + 8 * c, m);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const BlockDivider divide(m);
            auto second_look = [&](auto quotient) {
                for (int c = lane; c < nchunks; c += 32) {
                    float f[8];
                    load8<S>(gb + 8 * c, f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // |x| <= 1 (or x is NaN), so (x + 1) * scale lies in [0, bins]: the floor is a truncation,
                        // NaN maps to bin 0, and x == 1 lands in the spare counter hist[bins], folded into the
                        // last bin at the end (the reference's upper clamp). With a power-of-two scale the sum and
                        // the product round as one fused multiply-add does (scaling by 2^k commutes with rounding).
                        const float x = quotient(f[i]);
                        const float y = POW2 ? fmaf(x, scale, scale) : (x + 1.0f) * scale;
                        atomicAdd(&hist[__float2uint_rz(y)], 1u);
                    }
                }
            };
            // (measured: deciding the kind of division once per block pays for 2-byte elements, 0.485 -> 0.518 of the
            // copy bandwidth on bf16; for fp32 the per-element form is the faster one, 0.684 against 0.589)
            if (sizeof(S) != 2) second_look([&](float v) { return divide(v); });
            else if (divide.fast) second_look([&](float v) { return divide.quick(v); });
            else second_look([&](float v) { return divide.careful(v); });
        } else {
            const float absmax = block_absmax<S, GROUP>(gb, period, tig, red);
            for (long long i = tig; i < period; i += GROUP) {
                const float v = ScalarIO<S>::load(gb + i);
                float x = 0.0f;
                if (absmax > 0.0f) x = v / absmax;
                int bin = static_cast<int>(floorf((x + 1.0f) * scale));
                bin = bin < 0 ? 0 : (bin > last_bin ? last_bin : bin);
                atomicAdd(&hist[bin], 1u);
            }
        }
        since_flush += static_cast<unsigned long long>(period);
        if (GROUP > 32 && since_flush > 0x7fffffffull) {  // keep the 32-bit counters from wrapping
            __syncthreads();
            for (int i = threadIdx.x; i < bins; i += kThreads) {
                if (hist[i]) { atomicAdd(&counts[i], static_cast<unsigned long long>(hist[i])); hist[i] = 0u; }
            }
            __syncthreads();
            since_flush = 0;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) { hist[last_bin] += hist[bins]; hist[bins] = 0u; }
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += kThreads) {
        if (hist[i]) atomicAdd(&counts[i], static_cast<unsigned long long>(hist[i]));
    }
}

// ------------------------------------------------------------------------------- period scores
// Sum over one block of log(x + eps) in fp64, x = v*v in fp64 unless the input is already squared
// (reference: period_variance_kernel.cu:124-139). `invalid` counts non-positive log inputs.
template <typename S, bool SQUARED>
__device__ __forceinline__ double log_term(const S* p, double eps, unsigned long long& invalid) {
    const double raw = static_cast<double>(ScalarIO<S>::load(p));
    const double x = (SQUARED ? raw : raw * raw) + eps;
    if (x <= 0.0) { ++invalid; return 0.0; }
    return log(x);
}

// period >= 64: one warp per block. period < 64: one thread per block.
template <typename S, bool SQUARED>
__global__ void __launch_bounds__(kThreads) block_logsum_kernel(const S* __restrict__ values, long long period,
                                                                long long num_blocks, double eps,
                                                                double* __restrict__ sums,
                                                                unsigned long long* __restrict__ invalid_out) {
    unsigned long long invalid = 0;
    if (period >= 64) {
        const int lane = threadIdx.x & 31;
        const long long w0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
        const long long stride = static_cast<long long>(gridDim.x) * kWarps;
        for (long long b = w0; b < num_blocks; b += stride) {
            const S* vb = values + b * period;
            double acc = 0.0;
            for (long long i = lane; i < period; i += 32) acc += log_term<S, SQUARED>(vb + i, eps, invalid);
            acc = warp_sum(acc);
            if (lane == 0) sums[b] = acc;
        }
    } else {
        const long long t0 = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
        const long long stride = static_cast<long long>(gridDim.x) * kThreads;
        for (long long b = t0; b < num_blocks; b += stride) {
            const S* vb = values + b * period;
            double acc = 0.0;
            for (long long i = 0; i < period; ++i) acc += log_term<S, SQUARED>(vb + i, eps, invalid);
            sums[b] = acc;
        }
    }
    if (invalid) atomicAdd(invalid_out, invalid);
}

// partial[c] = sum over this CTA's slice of |S[j+1]/P - S[j]/P|, fixed order => reproducible.
__global__ void __launch_bounds__(kThreads) adjacent_diff_partial_kernel(const double* __restrict__ sums,
                                                                         long long num_pairs, double period,
                                                                         double* __restrict__ partial) {
    __shared__ double red[kWarps];
    const long long per_cta = (num_pairs + gridDim.x - 1) / gridDim.x;
    const long long begin = static_cast<long long>(blockIdx.x) * per_cta;
    long long end = begin + per_cta;
    if (end > num_pairs) end = num_pairs;
    double acc = 0.0;
    for (long long j = begin + threadIdx.x; j < end; j += kThreads) {
        const double cur = sums[j] / period;
        const double nxt = sums[j + 1] / period;
        acc += fabs(nxt - cur);
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kWarps; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}

__global__ void adjacent_diff_final_kernel(const double* __restrict__ partial, int n_partial, double num_pairs,
                                           const unsigned long long* __restrict__ invalid,
                                           double* __restrict__ stats) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < n_partial; ++i) t += partial[i];
        stats[0] = t / num_pairs;
        stats[1] = static_cast<double>(*invalid);
    }
}

// out[j] = sum of `ratio` consecutive entries of in[], added left to right: the block sums of period
// p from those of a divisor q of p (ratio = p / q). Logs are taken once per element, not once per
// candidate period.
__global__ void __launch_bounds__(kThreads) regroup_sums_kernel(const double* __restrict__ in, long long ratio,
                                                                long long num_out, double* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    if (ratio >= 64) {
        const long long w0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
        const long long stride = static_cast<long long>(gridDim.x) * kWarps;
        for (long long j = w0; j < num_out; j += stride) {
            const double* src = in + j * ratio;
            double acc = 0.0;
            for (long long i = lane; i < ratio; i += 32) acc += src[i];
            acc = warp_sum(acc);
            if (lane == 0) out[j] = acc;
        }
    } else {
        const long long t0 = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
        const long long stride = static_cast<long long>(gridDim.x) * kThreads;
        for (long long j = t0; j < num_out; j += stride) {
            const double* src = in + j * ratio;
            double acc = 0.0;
            for (long long i = 0; i < ratio; ++i) acc += src[i];
            out[j] = acc;
        }
    }
}

// ---- the same three kernels for all candidate periods of a scan at once (blockIdx.y = candidate): a scan of 72
// candidates is then a dozen launches instead of two hundred. The arithmetic per candidate, and therefore every
// score, is that of the single-candidate kernels above: an output of the regrouping depends on no launch
// parameter, and the partial sums are cut by the candidate's own number of partials, not by the grid.
struct ScanCandidate {
    long long src;        // offset (in doubles from the scratch base) of the sums this candidate is regrouped from
    long long dst;        // offset of its own sums
    long long ratio;      // period / parent period; 0: the sums are the base sums themselves, nothing to regroup
    long long nb;         // blocks of this period
    long long partial;    // offset of its partial sums (n_partial doubles)
    double period;
    int n_partial;
    int stats;            // index of its pair of outputs
};

__global__ void __launch_bounds__(kThreads) regroup_sums_batch_kernel(double* __restrict__ scratch,
                                                                      const ScanCandidate* __restrict__ table, int first) {
    const ScanCandidate c = table[first + blockIdx.y];
    if (c.ratio == 0) return;
    const double* in = scratch + c.src;
    double* out = scratch + c.dst;
    const long long ratio = c.ratio, num_out = c.nb;
    const int lane = threadIdx.x & 31;
    if (ratio >= 64) {
        const long long w0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
        const long long stride = static_cast<long long>(gridDim.x) * kWarps;
        for (long long j = w0; j < num_out; j += stride) {
            const double* src = in + j * ratio;
            double acc = 0.0;
            for (long long i = lane; i < ratio; i += 32) acc += src[i];
            acc = warp_sum(acc);
            if (lane == 0) out[j] = acc;
        }
    } else {
        const long long t0 = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
        const long long stride = static_cast<long long>(gridDim.x) * kThreads;
        for (long long j = t0; j < num_out; j += stride) {
            const double* src = in + j * ratio;
            double acc = 0.0;
            for (long long i = 0; i < ratio; ++i) acc += src[i];
            out[j] = acc;
        }
    }
}

__global__ void __launch_bounds__(kThreads) adjacent_diff_partial_batch_kernel(double* __restrict__ scratch,
                                                                               const ScanCandidate* __restrict__ table) {
    __shared__ double red[kWarps];
    const ScanCandidate c = table[blockIdx.y];
    if (static_cast<int>(blockIdx.x) >= c.n_partial) return;
    const double* sums = scratch + c.dst;
    const long long num_pairs = c.nb - 1;
    const double period = c.period;
    const long long per_cta = (num_pairs + c.n_partial - 1) / c.n_partial;
    const long long begin = static_cast<long long>(blockIdx.x) * per_cta;
    long long end = begin + per_cta;
    if (end > num_pairs) end = num_pairs;
    double acc = 0.0;
    for (long long j = begin + threadIdx.x; j < end; j += kThreads) {
        const double cur = sums[j] / period;
        const double nxt = sums[j + 1] / period;
        acc += fabs(nxt - cur);
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kWarps; ++w) t += red[w];
        scratch[c.partial + blockIdx.x] = t;
    }
}

__global__ void adjacent_diff_final_batch_kernel(const double* __restrict__ scratch, const ScanCandidate* __restrict__ table,
                                                 const unsigned long long* __restrict__ invalid,
                                                 double* __restrict__ stats) {
    if (threadIdx.x != 0) return;
    const ScanCandidate c = table[blockIdx.x];
    const double* partial = scratch + c.partial;
    double t = 0.0;
    for (int i = 0; i < c.n_partial; ++i) t += partial[i];
    stats[2 * c.stats] = t / static_cast<double>(c.nb - 1);
    stats[2 * c.stats + 1] = static_cast<double>(*invalid);
}

// Mean within-block variance / coefficient of variation of x (= v or v*v), fp32 sums
// (reference: period_variance_kernel.cu:13-106). One warp per block.
template <typename S, bool SQUARED, bool COV>
__global__ void __launch_bounds__(kThreads) block_moment_kernel(const S* __restrict__ values, long long period,
                                                                long long num_blocks, double* __restrict__ stats) {
    const int lane = threadIdx.x & 31;
    const long long w0 = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const long long stride = static_cast<long long>(gridDim.x) * kWarps;
    for (long long b = w0; b < num_blocks; b += stride) {
        const S* vb = values + b * period;
        float sx = 0.0f, sx2 = 0.0f;
        for (long long i = lane; i < period; i += 32) {
            const float v = ScalarIO<S>::load(vb + i);
            const float x = SQUARED ? v : v * v;
            sx += x;
            sx2 = fmaf(x, x, sx2);
        }
        sx = warp_sum(sx);
        sx2 = warp_sum(sx2);
        if (lane == 0) {
            const float mean = sx / static_cast<float>(period);
            float var = sx2 / static_cast<float>(period);
            var -= mean * mean;
            if (var < 0.0f) var = 0.0f;
            if (!COV) {
                atomicAdd(stats, static_cast<double>(var));
            } else if (mean < 0.0f) {
                atomicAdd(stats + 2, 1.0);
            } else if (mean > 0.0f) {
                atomicAdd(stats, static_cast<double>(sqrtf(var) / mean));
                atomicAdd(stats + 1, 1.0);
            }
        }
    }
}

// ------------------------------------------------------------------------------- Lloyd-Max
// Both kernels assign every normalised value to its codebook entry with the rule of the step kernels
// (nearest entry, left on ties; reference: lloyd_max_fused_kernel.cu:16-48), through the codebook
// workspace staged in shared memory: one table read and one compare per value, the binary search
// over the thresholds only for the few undecidable cells.
struct LloydTables {
    const float* cb;
    const float* thr;
    const unsigned char* lut;
    int k;
    __device__ __forceinline__ int entry(float x) const {
        // the table covers [-1, 1]; values outside it (non-finite gradients) take the exact rule
        if (!(fabsf(x) <= 1.0f)) return entry_exact(x, thr, cb, k);
        bool slow;
        const int e = lut_query(x, lut, &slow);
        return slow ? entry_exact(x, thr, cb, k) : e;
    }
};

__device__ __forceinline__ LloydTables stage_lloyd_tables(const unsigned char* ws, unsigned char* smem) {
    const uint4* src = reinterpret_cast<const uint4*>(ws);
    uint4* dst = reinterpret_cast<uint4*>(smem);
    for (int i = threadIdx.x; i < GEFEN_B200_CODEBOOK_WS_BYTES / 16; i += blockDim.x) dst[i] = src[i];
    __syncthreads();
    LloydTables t;
    t.cb = reinterpret_cast<const float*>(smem + kWsCodebookOff);
    t.thr = reinterpret_cast<const float*>(smem + kWsThresholdOff);
    t.lut = smem + kWsLutOff;
    t.k = reinterpret_cast<const int*>(smem + kWsMetaOff)[0];
    return t;
}

// (x + 1) * 2^24 rounded to an integer in [0, 2^25] for |x| <= 1 (non-finite values, which only non-finite
// gradients produce, count as x = 0 in the sum; their count is still taken).
__device__ __forceinline__ unsigned int lloyd_fixed(float x) {
    const float scaled = x * 16777216.0f;
    const int q = (fabsf(scaled) <= 16777216.0f) ? __float2int_rn(scaled) : 0;
    return static_cast<unsigned int>(q + 16777216);
}

// E-step: per codebook entry, the sum of the normalised values assigned to it and their count
// (reference: lloyd_max_fused_kernel.cu:50-118). Sums are fp32 atomics (order-dependent in the
// reference too); counts are exact.
template <typename S, int GROUP, bool VEC>
__global__ void __launch_bounds__(kThreads) lloyd_accumulate_kernel(const S* __restrict__ g, long long period,
                                                                    long long num_blocks, const unsigned char* ws,
                                                                    int k, float* __restrict__ sums,
                                                                    unsigned long long* __restrict__ counts) {
    __shared__ __align__(16) unsigned char tables[GEFEN_B200_CODEBOOK_WS_BYTES];
    // Per-entry sums are kept in shared memory in fixed point, as the 64-bit sum of (x + 1) * 2^24 in two 32-bit
    // words: float and 64-bit additions to shared memory are compare-and-swap loops, 32-bit integer ones are
    // native. An element costs one add to the low word (whose returned old value tells a carry, which then
    // goes to the high word: once per ~128 elements of an entry) and one to the count; the offset count * 2^24
    // comes off at the flush. The sum does not depend on the order of the additions, values of magnitude 2^-1
    // or more are exact and smaller ones are within 2^-25.
    __shared__ unsigned int slo[kMaxCodebook];
    __shared__ unsigned int shi[kMaxCodebook];
    __shared__ unsigned int scnt[kMaxCodebook];
    __shared__ float red[kWarps];
    slo[threadIdx.x] = 0u;
    shi[threadIdx.x] = 0u;
    scnt[threadIdx.x] = 0u;
    auto add = [&](int e, float x) {
        const unsigned int v = lloyd_fixed(x);
        const unsigned int old = atomicAdd(&slo[e], v);
        if (old + v < old) atomicAdd(&shi[e], 1u);
        atomicAdd(&scnt[e], 1u);
    };
    auto flush = [&]() {   // every thread of the CTA, between two __syncthreads
        if (threadIdx.x < k && scnt[threadIdx.x]) {
            const unsigned long long raw = (static_cast<unsigned long long>(shi[threadIdx.x]) << 32) | slo[threadIdx.x];
            const long long fixed = static_cast<long long>(raw) - (static_cast<long long>(scnt[threadIdx.x]) << 24);
            atomicAdd(&sums[threadIdx.x], static_cast<float>(static_cast<double>(fixed) * (1.0 / 16777216.0)));
            atomicAdd(&counts[threadIdx.x], static_cast<unsigned long long>(scnt[threadIdx.x]));
            slo[threadIdx.x] = shi[threadIdx.x] = scnt[threadIdx.x] = 0u;
        }
    };
    const LloydTables t = stage_lloyd_tables(ws, tables);
    const int lane = threadIdx.x & 31;
    const int tig = GROUP == 32 ? lane : static_cast<int>(threadIdx.x);
    const long long group0 = GROUP == 32 ? static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5)
                                         : static_cast<long long>(blockIdx.x);
    const long long stride = GROUP == 32 ? static_cast<long long>(gridDim.x) * kWarps : static_cast<long long>(gridDim.x);
    unsigned long long since_flush = 0;
    for (long long b = group0; b < num_blocks; b += stride) {
        const S* gb = g + b * period;
        if (VEC) {
            const int nchunks = static_cast<int>(period >> 3);
            float m = 0.0f;
            for (int c = lane; c < nchunks; c += 32) {
                float f[8];
                load8<S>(gb + 8 * c, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const BlockDivider divide(m);
            auto second_look = [&](auto quotient) {
                for (int c = lane; c < nchunks; c += 32) {
                    float f[8];
                    load8<S>(gb + 8 * c, f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float x = quotient(f[i]);
                        add(t.entry(x), x);
                    }
                }
            };
            if (divide.fast) second_look([&](float v) { return divide.quick(v); });
            else second_look([&](float v) { return divide.careful(v); });
        } else {
            const float absmax = block_absmax<S, GROUP>(gb, period, tig, red);
            for (long long i = tig; i < period; i += GROUP) {
                const float v = ScalarIO<S>::load(gb + i);
                float x = 0.0f;
                if (absmax > 0.0f) x = v / absmax;
                add(t.entry(x), x);
            }
        }
        since_flush += static_cast<unsigned long long>(period);
        if (GROUP > 32 && since_flush > 0x7fffffffull) {   // keep the 32-bit counts from wrapping
            __syncthreads();
            flush();
            __syncthreads();
            since_flush = 0;
        }
    }
    __syncthreads();
    flush();
}

// Logging MSE of assigning with the old codebook and reconstructing with the new one
// (reference: lloyd_max_fused_kernel.cu:120-195).
template <typename S, int GROUP, bool VEC>
__global__ void __launch_bounds__(kThreads) lloyd_mse_kernel(const S* __restrict__ g, long long period,
                                                             long long num_blocks, const unsigned char* old_ws,
                                                             const float* __restrict__ new_codebook, int k,
                                                             float* __restrict__ mse_norm, float* __restrict__ mse_orig) {
    __shared__ __align__(16) unsigned char tables[GEFEN_B200_CODEBOOK_WS_BYTES];
    __shared__ float ncb[kMaxCodebook];
    __shared__ float red[kWarps];
    __shared__ float red2[2][kWarps];
    ncb[threadIdx.x] = new_codebook[threadIdx.x < k ? threadIdx.x : k - 1];
    const LloydTables t = stage_lloyd_tables(old_ws, tables);
    const int lane = threadIdx.x & 31;
    const int tig = GROUP == 32 ? lane : static_cast<int>(threadIdx.x);
    const long long group0 = GROUP == 32 ? static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5)
                                         : static_cast<long long>(blockIdx.x);
    const long long stride = GROUP == 32 ? static_cast<long long>(gridDim.x) * kWarps : static_cast<long long>(gridDim.x);
    float en = 0.0f, eo = 0.0f;
    for (long long b = group0; b < num_blocks; b += stride) {
        const S* gb = g + b * period;
        if (VEC) {
            const int nchunks = static_cast<int>(period >> 3);
            float m = 0.0f;
            for (int c = lane; c < nchunks; c += 32) {
                float f[8];
                load8<S>(gb + 8 * c, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            const BlockDivider divide(m);
            auto second_look = [&](auto quotient) {
                for (int c = lane; c < nchunks; c += 32) {
                    float f[8];
                    load8<S>(gb + 8 * c, f);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float x = quotient(f[i]);
                        const float err = x - ncb[t.entry(x)];
                        en = fmaf(err, err, en);
                        const float oe = err * m;
                        eo = fmaf(oe, oe, eo);
                    }
                }
            };
            if (divide.fast) second_look([&](float v) { return divide.quick(v); });
            else second_look([&](float v) { return divide.careful(v); });
        } else {
            const float absmax = block_absmax<S, GROUP>(gb, period, tig, red);
            for (long long i = tig; i < period; i += GROUP) {
                const float v = ScalarIO<S>::load(gb + i);
                float x = 0.0f;
                if (absmax > 0.0f) x = v / absmax;
                const float err = x - ncb[t.entry(x)];
                en = fmaf(err, err, en);
                const float oe = err * absmax;
                eo = fmaf(oe, oe, eo);
            }
        }
    }
    en = warp_sum(en);
    eo = warp_sum(eo);
    if (lane == 0) { red2[0][threadIdx.x >> 5] = en; red2[1][threadIdx.x >> 5] = eo; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = 0.0f, c = 0.0f;
        for (int w = 0; w < kWarps; ++w) { a += red2[0][w]; c += red2[1][w]; }
        atomicAdd(mse_norm, a);
        atomicAdd(mse_orig, c);
    }
}

// ------------------------------------------------------------------------------- host side
static int check_flat(const void* values, int dtype, int64_t numel, int64_t period) {
    GEFEN_CHECK_ARG(values != nullptr || numel == 0, "Expected a non-null tensor.");
    GEFEN_CHECK_ARG(is_float_dtype(dtype), "Expected a floating-point tensor.");
    GEFEN_CHECK_ARG(period > 0, "Expected a positive period.");
    GEFEN_CHECK_ARG(numel >= 0 && numel % period == 0, "Expected tensor length to be divisible by period.");
    return GEFEN_B200_OK;
}

#define GEFEN_DISPATCH_S(dtype, ...)                                                       \
    switch (dtype) {                                                                       \
        case GEFEN_B200_F32: { using S = float; __VA_ARGS__; } break;                      \
        case GEFEN_B200_F16: { using S = __half; __VA_ARGS__; } break;                     \
        case GEFEN_B200_BF16: { using S = __nv_bfloat16; __VA_ARGS__; } break;             \
        default: { using S = double; __VA_ARGS__; } break;                                 \
    }

constexpr int kMaxPartials = 1024;
static int partials_for(int64_t pairs) {
    int n_partial = static_cast<int>((pairs + 4095) / 4096);
    if (n_partial > kMaxPartials) n_partial = kMaxPartials;
    if (n_partial < 1) n_partial = 1;
    return n_partial;
}

static int launch_block_logsums(const void* values, int dtype, int64_t numel, int64_t period, bool squared, double eps,
                                double* sums, unsigned long long* invalid, cudaStream_t stream) {
    const int64_t nb = numel / period;
    const int grid = period >= 64 ? persistent_grid(nb, kWarps, 8) : persistent_grid(nb, kThreads, 8);
    GEFEN_DISPATCH_S(dtype, {
        if (squared)
            block_logsum_kernel<S, true><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(values), period, nb, eps, sums, invalid);
        else
            block_logsum_kernel<S, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(values), period, nb, eps, sums, invalid);
    });
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

// score = mean over adjacent pairs of |S[j+1]/P - S[j]/P|; `partial` holds kMaxPartials doubles.
static int launch_adjacent_score(const double* sums, int64_t nb, int64_t period, const unsigned long long* invalid,
                                 double* partial, double* stats, cudaStream_t stream) {
    const int64_t pairs = nb - 1;
    const int n_partial = partials_for(pairs);
    adjacent_diff_partial_kernel<<<n_partial, kThreads, 0, stream>>>(sums, pairs, static_cast<double>(period), partial);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    adjacent_diff_final_kernel<<<1, 32, 0, stream>>>(partial, n_partial, static_cast<double>(pairs), invalid, stats);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

static int adjacent_score(const void* values, int dtype, int64_t numel, int64_t period, bool squared, double eps,
                          double* stats, double* block_sums, cudaStream_t stream) {
    const int64_t nb = numel / period;
    unsigned long long* invalid = reinterpret_cast<unsigned long long*>(block_sums + nb);
    double* partial = block_sums + nb + 1;
    GEFEN_CHECK_CUDA(cudaMemsetAsync(invalid, 0, sizeof(unsigned long long), stream));
    int rc = launch_block_logsums(values, dtype, numel, period, squared, eps, block_sums, invalid, stream);
    if (rc != GEFEN_B200_OK) return rc;
    return launch_adjacent_score(block_sums, nb, period, invalid, partial, stats, stream);
}

static int64_t gcd64(int64_t a, int64_t b) { while (b) { const int64_t t = a % b; a = b; b = t; } return a; }

// Plan of the hierarchical scan: the base period (gcd of all candidates), and for every candidate
// the largest smaller candidate (or the base) that divides it. Offsets index one scratch array:
// [invalid | partials | base sums | sums of candidate 0 | sums of candidate 1 | ...].
struct ScanPlan {
    int64_t base;
    std::vector<int> order;        // candidate indices by ascending period
    std::vector<int> parent;       // per candidate: index of the parent candidate, -1 = base
    std::vector<int64_t> offset;   // per candidate: offset of its sums (== base offset if period == base)
    std::vector<int> level;        // per candidate: regrouping steps between the base sums and its own
    std::vector<int> n_partial;    // per candidate: partial sums of its score
    std::vector<int64_t> partial;  // per candidate: offset of those
    int64_t table_offset;          // the device copy of the candidates' descriptors
    int64_t base_offset;
    int64_t total;
};


static ScanPlan make_scan_plan(int64_t numel, const int64_t* periods, int n) {
    ScanPlan plan;
    plan.base = 0;
    for (int i = 0; i < n; ++i) plan.base = gcd64(plan.base, periods[i]);
    plan.order.resize(n);
    for (int i = 0; i < n; ++i) plan.order[i] = i;
    std::sort(plan.order.begin(), plan.order.end(), [&](int x, int y) { return periods[x] < periods[y]; });
    plan.parent.assign(n, -1);
    plan.offset.assign(n, 0);
    plan.base_offset = 1 + kMaxPartials;
    int64_t cursor = plan.base_offset + numel / plan.base;
    for (int oi = 0; oi < n; ++oi) {
        const int i = plan.order[oi];
        if (periods[i] == plan.base) { plan.offset[i] = plan.base_offset; continue; }
        for (int oj = oi - 1; oj >= 0; --oj) {
            const int j = plan.order[oj];
            if (periods[j] < periods[i] && periods[i] % periods[j] == 0) { plan.parent[i] = j; break; }
        }
        plan.offset[i] = cursor;
        cursor += numel / periods[i];
    }
    plan.level.assign(n, 0);
    plan.n_partial.assign(n, 1);
    plan.partial.assign(n, 0);
    for (int oi = 0; oi < n; ++oi) {   // ascending periods: a parent comes before its children
        const int i = plan.order[oi];
        plan.level[i] = periods[i] == plan.base ? 0 : (plan.parent[i] < 0 ? 1 : plan.level[plan.parent[i]] + 1);
        plan.n_partial[i] = partials_for(numel / periods[i] - 1);
        plan.partial[i] = cursor;
        cursor += plan.n_partial[i];
    }
    plan.table_offset = cursor;
    cursor += (static_cast<int64_t>(n) * static_cast<int64_t>(sizeof(ScanCandidate)) + 7) / 8;
    plan.total = cursor;
    return plan;
}

}  // namespace gefen

using namespace gefen;

extern "C" {

int gefen_b200_exact_histogram(const void* grad_flat, int grad_dtype, int64_t numel, int64_t period,
                               int64_t* bin_counts, int histogram_bins, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(bin_counts != nullptr, "Expected a non-null bin_counts.");
    GEFEN_CHECK_ARG(histogram_bins >= 1 && histogram_bins <= 4096, "Expected histogram size in [1, 4096].");
    GEFEN_CHECK_ARG(period > 0, "Expected period to be positive.");
    GEFEN_CHECK_ARG(grad_flat != nullptr || numel == 0, "Expected a non-null grad_flat.");
    GEFEN_CHECK_ARG(is_float_dtype(grad_dtype), "Unsupported gradient dtype tag %d.", grad_dtype);
    GEFEN_CHECK_ARG(numel >= 0 && numel % period == 0, "Expected grad_flat.numel() to be divisible by period.");
    const int64_t nb = numel / period;
    if (nb == 0) return GEFEN_B200_OK;
    unsigned long long* counts = reinterpret_cast<unsigned long long*>(bin_counts);
    // a warp's 32-bit counters cannot wrap: a CTA of the warp-per-block form sees at most 2^31 elements
    if (period <= 8192) {
        const int grid = persistent_grid(nb, kWarps, 6);
        const bool vec = period % 8 == 0 && aligned16(grad_flat) && grad_dtype != GEFEN_B200_F64 &&
                         numel / grid < 0x7fffffffll;
        const bool pow2 = (histogram_bins & (histogram_bins - 1)) == 0 && histogram_bins >= 2;
        if (vec && pow2) {
            GEFEN_DISPATCH_S(grad_dtype, histogram_kernel<S, 32, true, true><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, histogram_bins, counts));
        } else if (vec) {
            GEFEN_DISPATCH_S(grad_dtype, histogram_kernel<S, 32, true, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, histogram_bins, counts));
        } else {
            GEFEN_DISPATCH_S(grad_dtype, histogram_kernel<S, 32, false, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, histogram_bins, counts));
        }
    } else {
        const int grid = persistent_grid(nb, 1, 6);
        GEFEN_DISPATCH_S(grad_dtype, histogram_kernel<S, 256, false, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, histogram_bins, counts));
    }
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_average_within_block_variance(const void* values, int dtype, int64_t numel, int64_t period,
                                             int input_is_squared, double* stats, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_flat(values, dtype, numel, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(stats != nullptr, "Expected a non-null stats buffer.");
    GEFEN_CHECK_CUDA(cudaMemsetAsync(stats, 0, sizeof(double), stream));
    const int64_t nb = numel / period;
    if (nb == 0) return GEFEN_B200_OK;
    const int grid = persistent_grid(nb, kWarps, 8);
    GEFEN_DISPATCH_S(dtype, {
        if (input_is_squared) block_moment_kernel<S, true, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(values), period, nb, stats);
        else block_moment_kernel<S, false, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(values), period, nb, stats);
    });
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_average_within_block_coefficient_of_variation(const void* values, int dtype, int64_t numel,
                                                             int64_t period, int input_is_squared, double* stats,
                                                             void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_flat(values, dtype, numel, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(stats != nullptr, "Expected a non-null stats buffer.");
    GEFEN_CHECK_CUDA(cudaMemsetAsync(stats, 0, 3 * sizeof(double), stream));
    const int64_t nb = numel / period;
    if (nb == 0) return GEFEN_B200_OK;
    const int grid = persistent_grid(nb, kWarps, 8);
    GEFEN_DISPATCH_S(dtype, {
        if (input_is_squared) block_moment_kernel<S, true, true><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(values), period, nb, stats);
        else block_moment_kernel<S, false, true><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(values), period, nb, stats);
    });
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int64_t gefen_b200_period_scratch_doubles(int64_t numel, int64_t period) {
    if (period <= 0 || numel < 0) return 0;
    return numel / period + 1 + kMaxPartials;
}

int gefen_b200_average_adjacent_log_block_mean_difference(const void* values, int dtype, int64_t numel,
                                                          int64_t period, int input_is_squared, double epsilon,
                                                          double* stats, double* block_sums, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_flat(values, dtype, numel, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(epsilon > 0.0, "Expected a positive epsilon.");
    GEFEN_CHECK_ARG(numel / period >= 2, "Expected at least two blocks to compare adjacent block means.");
    GEFEN_CHECK_ARG(stats != nullptr && block_sums != nullptr, "Expected non-null stats and block_sums.");
    return adjacent_score(values, dtype, numel, period, input_is_squared != 0, epsilon, stats, block_sums, stream);
}

int64_t gefen_b200_period_scan_scratch_doubles(int64_t numel, const int64_t* host_periods, int n_periods) {
    if (numel <= 0 || n_periods <= 0 || host_periods == nullptr) return 0;
    for (int i = 0; i < n_periods; ++i)
        if (host_periods[i] <= 0 || numel % host_periods[i] != 0) return 0;
    return make_scan_plan(numel, host_periods, n_periods).total;
}

int gefen_b200_period_scan(const void* values, int dtype, int64_t numel, int input_is_squared, double epsilon,
                           const int64_t* host_periods, int n_periods, double* stats, double* scratch,
                           void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(n_periods >= 0, "Expected a non-negative number of periods.");
    if (n_periods == 0) return GEFEN_B200_OK;
    GEFEN_CHECK_ARG(host_periods != nullptr && stats != nullptr && scratch != nullptr,
                    "Expected non-null periods, stats and scratch.");
    GEFEN_CHECK_ARG(epsilon > 0.0, "Expected a positive epsilon.");
    for (int i = 0; i < n_periods; ++i) {
        int rc = check_flat(values, dtype, numel, host_periods[i]);
        if (rc != GEFEN_B200_OK) return rc;
        GEFEN_CHECK_ARG(numel / host_periods[i] >= 2, "Expected at least two blocks for period %lld.",
                        static_cast<long long>(host_periods[i]));
    }
    const ScanPlan plan = make_scan_plan(numel, host_periods, n_periods);
    unsigned long long* invalid = reinterpret_cast<unsigned long long*>(scratch);
    GEFEN_CHECK_CUDA(cudaMemsetAsync(invalid, 0, sizeof(unsigned long long), stream));
    // the only pass over the tensor: log sums at the base granularity
    int rc = launch_block_logsums(values, dtype, numel, plan.base, input_is_squared != 0, epsilon,
                                  scratch + plan.base_offset, invalid, stream);
    if (rc != GEFEN_B200_OK) return rc;
    // the candidates in the order of their launches: by regrouping level (a parent is one level above its
    // children), so that each level is one launch over a run of the table
    std::vector<int> exec(plan.order);
    std::stable_sort(exec.begin(), exec.end(), [&](int x, int y) { return plan.level[x] < plan.level[y]; });
    std::vector<ScanCandidate> table(n_periods);
    int max_level = 0, max_partial = 1;
    for (int e = 0; e < n_periods; ++e) {
        const int i = exec[e];
        const int64_t p = host_periods[i];
        ScanCandidate& c = table[e];
        const int64_t q = plan.parent[i] < 0 ? plan.base : host_periods[plan.parent[i]];
        c.src = plan.parent[i] < 0 ? plan.base_offset : plan.offset[plan.parent[i]];
        c.dst = plan.offset[i];
        c.ratio = p == plan.base ? 0 : p / q;
        c.nb = numel / p;
        c.partial = plan.partial[i];
        c.period = static_cast<double>(p);
        c.n_partial = plan.n_partial[i];
        c.stats = i;
        max_level = std::max(max_level, plan.level[i]);
        max_partial = std::max(max_partial, c.n_partial);
    }
    ScanCandidate* dev_table = reinterpret_cast<ScanCandidate*>(scratch + plan.table_offset);
    GEFEN_CHECK_CUDA(cudaMemcpyAsync(dev_table, table.data(), sizeof(ScanCandidate) * n_periods, cudaMemcpyHostToDevice, stream));
    for (int level = 1; level <= max_level; ++level) {
        int first = -1, count = 0;
        int64_t most = 1;
        for (int e = 0; e < n_periods; ++e) {
            if (plan.level[exec[e]] != level) continue;
            if (first < 0) first = e;
            ++count;
            const int64_t groups = table[e].ratio >= 64 ? (table[e].nb + kWarps - 1) / kWarps : (table[e].nb + kThreads - 1) / kThreads;
            most = std::max(most, groups);
        }
        if (count == 0) continue;
        const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
        const dim3 grid(static_cast<unsigned>(std::min(most, cap)), static_cast<unsigned>(count));
        regroup_sums_batch_kernel<<<grid, kThreads, 0, stream>>>(scratch, dev_table, first);
        GEFEN_CHECK_CUDA(cudaGetLastError());
    }
    adjacent_diff_partial_batch_kernel<<<dim3(static_cast<unsigned>(max_partial), static_cast<unsigned>(n_periods)), kThreads, 0,
                                         stream>>>(scratch, dev_table);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    adjacent_diff_final_batch_kernel<<<n_periods, 32, 0, stream>>>(scratch, dev_table, invalid, stats);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_lloyd_accumulate(const void* grad_flat, int grad_dtype, int64_t numel, int64_t period,
                                const float* codebook, int codebook_size, const void* codebook_ws, float* sums,
                                int64_t* counts, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_flat(grad_flat, grad_dtype, numel, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(sums != nullptr && counts != nullptr, "Expected non-null sums and counts.");
    const void* ws = nullptr;
    rc = resolve_codebook_ws(codebook, codebook_size, codebook_ws, stream, &ws);
    if (rc != GEFEN_B200_OK) return rc;
    const int64_t nb = numel / period;
    if (nb == 0) return GEFEN_B200_OK;
    unsigned long long* cnt = reinterpret_cast<unsigned long long*>(counts);
    const unsigned char* wsb = static_cast<const unsigned char*>(ws);
    GEFEN_CHECK_ARG(aligned16(ws), "Expected a 16-byte aligned codebook workspace.");
    if (period <= 8192) {
        const int grid = persistent_grid(nb, kWarps, 4);
        if (period % 8 == 0 && aligned16(grad_flat) && grad_dtype != GEFEN_B200_F64) {
            GEFEN_DISPATCH_S(grad_dtype, lloyd_accumulate_kernel<S, 32, true><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, wsb, codebook_size, sums, cnt));
        } else {
            GEFEN_DISPATCH_S(grad_dtype, lloyd_accumulate_kernel<S, 32, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, wsb, codebook_size, sums, cnt));
        }
    } else {
        const int grid = persistent_grid(nb, 1, 4);
        GEFEN_DISPATCH_S(grad_dtype, lloyd_accumulate_kernel<S, 256, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, wsb, codebook_size, sums, cnt));
    }
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_lloyd_mse(const void* grad_flat, int grad_dtype, int64_t numel, int64_t period,
                         const float* old_codebook, const float* new_codebook, int codebook_size,
                         const void* old_codebook_ws, float* mse_normalized_sum, float* mse_original_sum,
                         void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    int rc = check_flat(grad_flat, grad_dtype, numel, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(new_codebook != nullptr && mse_normalized_sum != nullptr && mse_original_sum != nullptr,
                    "Expected non-null new_codebook and outputs.");
    const void* ws = nullptr;
    rc = resolve_codebook_ws(old_codebook, codebook_size, old_codebook_ws, stream, &ws);
    if (rc != GEFEN_B200_OK) return rc;
    const int64_t nb = numel / period;
    if (nb == 0) return GEFEN_B200_OK;
    const unsigned char* wsb = static_cast<const unsigned char*>(ws);
    GEFEN_CHECK_ARG(aligned16(ws), "Expected a 16-byte aligned codebook workspace.");
    if (period <= 8192) {
        const int grid = persistent_grid(nb, kWarps, 4);
        if (period % 8 == 0 && aligned16(grad_flat) && grad_dtype != GEFEN_B200_F64) {
            GEFEN_DISPATCH_S(grad_dtype, lloyd_mse_kernel<S, 32, true><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, wsb, new_codebook, codebook_size, mse_normalized_sum, mse_original_sum));
        } else {
            GEFEN_DISPATCH_S(grad_dtype, lloyd_mse_kernel<S, 32, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, wsb, new_codebook, codebook_size, mse_normalized_sum, mse_original_sum));
        }
    } else {
        const int grid = persistent_grid(nb, 1, 4);
        GEFEN_DISPATCH_S(grad_dtype, lloyd_mse_kernel<S, 256, false><<<grid, kThreads, 0, stream>>>(static_cast<const S*>(grad_flat), period, nb, wsb, new_codebook, codebook_size, mse_normalized_sum, mse_original_sum));
    }
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

}  // extern "C"
