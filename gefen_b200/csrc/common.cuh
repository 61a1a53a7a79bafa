// Host/device helpers shared by the translation units of libgefen_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/gefen_b200.h"
#include "quant_core.h"

namespace gefen {

// ------------------------------------------------------------------ error reporting (host)
void set_last_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t err, const char* what);

#define GEFEN_CHECK_ARG(cond, ...)                                   \
    do {                                                             \
        if (!(cond)) return ::gefen::fail(GEFEN_B200_EINVAL, __VA_ARGS__); \
    } while (0)

#define GEFEN_CHECK_CUDA(expr)                                        \
    do {                                                              \
        cudaError_t err__ = (expr);                                   \
        if (err__ != cudaSuccess) return ::gefen::cuda_fail(err__, #expr); \
    } while (0)

inline bool is_state_dtype(int d) {
    return d == GEFEN_B200_F32 || d == GEFEN_B200_F16 || d == GEFEN_B200_BF16;
}
inline bool is_float_dtype(int d) { return d >= GEFEN_B200_F32 && d <= GEFEN_B200_F64; }
inline int dtype_size(int d) {
    return d == GEFEN_B200_F32 ? 4 : d == GEFEN_B200_F64 ? 8 : 2;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();  // SMs of the current device (cached per device)

// Layout of the per-codebook workspace (GEFEN_B200_CODEBOOK_WS_BYTES).
constexpr int kWsCodebookOff = 0;      // 256 floats, tail padded with the last entry
constexpr int kWsThresholdOff = 1024;  // 256 floats, tail padded with +inf
constexpr int kWsMetaOff = 2048;       // 4 ints: codebook size, number of undecidable table cells, 0, 0
constexpr int kWsLutOff = 2064;        // kLutBytes of 8-byte entries
static_assert(kWsLutOff + kLutBytes == GEFEN_B200_CODEBOOK_WS_BYTES, "workspace size");

// Returns a workspace for `codebook`: the caller's if given, else the library-owned one of the
// current device, rebuilt on `stream` (see codebook_lut.cu).
int resolve_codebook_ws(const float* codebook, int codebook_size, const void* caller_ws,
                        cudaStream_t stream, const void** ws_out);
// Enqueues the kernel that fills `ws` (device, GEFEN_B200_CODEBOOK_WS_BYTES) from `codebook`.
int launch_codebook_prepare(const float* codebook, int codebook_size, void* ws, cudaStream_t stream);

// ------------------------------------------------------------------ device helpers
#if defined(__CUDACC__)

// Optimizer-state scalars (magnitude, vmean) have a run-time dtype: one per block, so a branch
// is cheaper than multiplying the template instantiations by nine as the reference does
// (automatic_gefen_fused_kernel.cu:767-829).
__device__ __forceinline__ float load_state(const void* base, int64_t idx, int dtype) {
    if (dtype == GEFEN_B200_F32) return static_cast<const float*>(base)[idx];
    if (dtype == GEFEN_B200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    return __half2float(static_cast<const __half*>(base)[idx]);
}
// Stores `value` rounded to `dtype` and returns the rounded value as float (what a later read
// of the state would see).
__device__ __forceinline__ float store_state(void* base, int64_t idx, int dtype, float value) {
    if (dtype == GEFEN_B200_F32) {
        static_cast<float*>(base)[idx] = value;
        return value;
    }
    if (dtype == GEFEN_B200_BF16) {
        const __nv_bfloat16 r = __float2bfloat16_rn(value);
        static_cast<__nv_bfloat16*>(base)[idx] = r;
        return __bfloat162float(r);
    }
    const __half r = __float2half_rn(value);
    static_cast<__half*>(base)[idx] = r;
    return __half2float(r);
}

template <typename S> struct ScalarIO;
template <> struct ScalarIO<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct ScalarIO<double> {
    static __device__ __forceinline__ float load(const double* p) { return static_cast<float>(*p); }
    static __device__ __forceinline__ void store(double* p, float v) { *p = static_cast<double>(v); }
    static __device__ __forceinline__ float round(float v) { return v; }
};
template <> struct ScalarIO<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct ScalarIO<__half> {
    static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
    static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
    static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};

// max(|a|, b) that keeps a NaN once seen, so that one reduction tells "block has a NaN/Inf".
__device__ __forceinline__ float max_abs_nan(float acc, float v) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(acc), "f"(fabsf(v)));
    return r;
}

__device__ __forceinline__ float warp_max_nan(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, o);
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(v) : "f"(v), "f"(other));
    }
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- bulk (TMA) copy of a contiguous, 16-byte aligned global range into shared memory,
// completion on an mbarrier; every wait is bounded.
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                              uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Returns false if the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = 4000000u) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < limit; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

#endif  // __CUDACC__

}  // namespace gefen
