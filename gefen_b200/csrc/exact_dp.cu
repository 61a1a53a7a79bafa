// Exact 1-D k-means by dynamic programming, stage-parallel on the device in fp64.
//
// Same recurrence, same fp64 expressions and the same tie rule as the reference's numba kernel
// (quantization.py:92-145): dp[e][c] = min over s in [c, e] of dp[s-1][c-1] + cost(s, e), the FIRST
// minimum in ascending s winning (strict `<`). Every candidate is an independent expression, so
// evaluating the candidates of one stage in parallel and reducing with "smaller value, then
// smaller s" gives bit-identical tables. Arithmetic uses the _rn intrinsics so that nothing is
// contracted into FMAs (numba does not contract either).
#include "common.cuh"

namespace gefen {

constexpr int kDpThreads = 256;

__device__ __forceinline__ double segment_cost(const double* pw, const double* pwx, const double* pwx2, int s, int e,
                                               int mode) {
    const double sw = __dsub_rn(pw[e], pw[s - 1]);
    const double swx = __dsub_rn(pwx[e], pwx[s - 1]);
    const double swx2 = __dsub_rn(pwx2[e], pwx2[s - 1]);
    if (mode != 0) {
        // forced centre fc = -1 (mode 1) or +1 (mode 2):
        // (swx2 - (2.0*fc)*swx) + (fc*fc)*sw, evaluated left to right as in the reference.
        const double fc = mode == 1 ? -1.0 : 1.0;
        const double a = __dsub_rn(swx2, __dmul_rn(__dmul_rn(2.0, fc), swx));
        return __dadd_rn(a, __dmul_rn(__dmul_rn(fc, fc), sw));
    }
    return __dsub_rn(swx2, __ddiv_rn(__dmul_rn(swx, swx), sw));
}

// One CTA per end index e. dp_prev = dp[.][c-1], dp_cur = dp[.][c].
__global__ void __launch_bounds__(kDpThreads) dp_stage_kernel(const double* __restrict__ pw, const double* __restrict__ pwx,
                                                              const double* __restrict__ pwx2, int num_points, int c,
                                                              int mode, const double* __restrict__ dp_prev,
                                                              double* __restrict__ dp_cur, int* __restrict__ backtrack,
                                                              int first_end) {
    __shared__ double red_v[kDpThreads / 32];
    __shared__ int red_i[kDpThreads / 32];
    const int e = first_end + static_cast<int>(blockIdx.x);
    if (e > num_points) return;
    if (e < c) {
        if (threadIdx.x == 0) { dp_cur[e] = INFINITY; backtrack[e] = -1; }
        return;
    }
    double best = INFINITY;
    int best_s = -1;
    for (int s = c + static_cast<int>(threadIdx.x); s <= e; s += kDpThreads) {
        const double cand = __dadd_rn(dp_prev[s - 1], segment_cost(pw, pwx, pwx2, s, e, mode));
        if (cand < best) { best = cand; best_s = s; }
    }
    // reduce: smaller value wins, on equal values the smaller start index (-1 = no candidate)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const double ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int os = __shfl_xor_sync(0xffffffffu, best_s, o);
        if (os >= 0 && (best_s < 0 || ov < best || (ov == best && os < best_s))) { best = ov; best_s = os; }
    }
    if ((threadIdx.x & 31) == 0) { red_v[threadIdx.x >> 5] = best; red_i[threadIdx.x >> 5] = best_s; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kDpThreads / 32; ++w) {
            const double ov = red_v[w];
            const int os = red_i[w];
            if (os >= 0 && (best_s < 0 || ov < best || (ov == best && os < best_s))) { best = ov; best_s = os; }
        }
        dp_cur[e] = best;
        backtrack[e] = best_s;
    }
}

__global__ void dp_init_kernel(double* dp0, int num_points) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= num_points) dp0[i] = (i == 0) ? 0.0 : INFINITY;
}

// Walks the backtrack table from (num_points, K) and emits the centres (reference :132-145).
__global__ void dp_backtrack_kernel(const double* __restrict__ pw, const double* __restrict__ pwx, int num_points,
                                    int num_codebooks, int force, const int* __restrict__ backtrack,
                                    float* __restrict__ codebook, int* __restrict__ status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int e = num_points;
    for (int c = num_codebooks; c >= 1; --c) {
        const int s = backtrack[static_cast<long long>(c) * (num_points + 1) + e];
        if (s < 1) { *status = 1; return; }
        if (force && c == 1) codebook[c - 1] = -1.0f;
        else if (force && c == num_codebooks) codebook[c - 1] = 1.0f;
        else {
            const double sw = __dsub_rn(pw[e], pw[s - 1]);
            const double swx = __dsub_rn(pwx[e], pwx[s - 1]);
            codebook[c - 1] = static_cast<float>(__ddiv_rn(swx, sw));
        }
        e = s - 1;
    }
    *status = 0;
}

}  // namespace gefen

using namespace gefen;

extern "C" {

int64_t gefen_b200_exact_dp_scratch_bytes(int num_points, int num_codebooks) {
    if (num_points < 1 || num_codebooks < 1) return 0;
    const int64_t n1 = static_cast<int64_t>(num_points) + 1;
    // two dp columns, the backtrack table, one status word (padded)
    return 2 * n1 * 8 + (static_cast<int64_t>(num_codebooks) + 1) * n1 * 4 + 16;
}

int gefen_b200_exact_dp(const double* prefix_w, const double* prefix_wx, const double* prefix_wx2, int num_points,
                        int num_codebooks, int force_endpoints, void* dp_scratch, float* codebook_out, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(prefix_w && prefix_wx && prefix_wx2 && dp_scratch && codebook_out, "Expected non-null arguments.");
    GEFEN_CHECK_ARG(num_points >= 1, "Cannot run exact DP on an empty histogram.");
    GEFEN_CHECK_ARG(num_codebooks >= 1 && num_codebooks <= num_points,
                    "Expected 1 <= num_codebooks <= num_points (the padded path is handled by the caller).");
    GEFEN_CHECK_ARG((reinterpret_cast<uintptr_t>(dp_scratch) & 7u) == 0, "Expected 8-byte aligned scratch.");
    const int64_t n1 = static_cast<int64_t>(num_points) + 1;
    double* dp_a = static_cast<double*>(dp_scratch);
    double* dp_b = dp_a + n1;
    int* backtrack = reinterpret_cast<int*>(dp_b + n1);
    int* status = backtrack + (static_cast<int64_t>(num_codebooks) + 1) * n1;
    dp_init_kernel<<<static_cast<int>((n1 + 255) / 256), 256, 0, stream>>>(dp_a, num_points);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    double* prev = dp_a;
    double* cur = dp_b;
    for (int c = 1; c <= num_codebooks; ++c) {
        int mode = 0;
        if (force_endpoints && c == 1) mode = 1;
        else if (force_endpoints && c == num_codebooks) mode = 2;
        // only dp[num_points][K] is read from the last stage
        const int first_end = (c == num_codebooks) ? num_points : 0;
        const int n_ends = num_points - first_end + 1;
        dp_stage_kernel<<<n_ends, kDpThreads, 0, stream>>>(prefix_w, prefix_wx, prefix_wx2, num_points, c, mode, prev, cur,
                                                          backtrack + static_cast<int64_t>(c) * n1, first_end);
        GEFEN_CHECK_CUDA(cudaGetLastError());
        double* t = prev; prev = cur; cur = t;
    }
    dp_backtrack_kernel<<<1, 32, 0, stream>>>(prefix_w, prefix_wx, num_points, num_codebooks, force_endpoints ? 1 : 0,
                                              backtrack, codebook_out, status);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

}  // extern "C"
