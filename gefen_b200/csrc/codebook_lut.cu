// Error plumbing of the C ABI and the codebook workspace builder.
//
// The workspace turns "nearest codebook entry, left on ties" (reference:
// kernels/automatic_gefen_fused_kernel.cu:59-90) into data the step kernels can stage into
// shared memory with one bulk copy: the padded codebook, the 255 exact decision thresholds and
// a 4097-cell table over [-1, 1] that resolves an element with one 8-byte read and one compare.
#include "common.cuh"

#include <mutex>
#include <string.h>

namespace gefen {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t err, const char* what) {
    snprintf(g_last_error, sizeof(g_last_error), "CUDA error %d (%s) in %s", static_cast<int>(err),
             cudaGetErrorString(err), what);
    return GEFEN_B200_ECUDA;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// One CTA of 256 threads. Thread i < k-1 bisects threshold i; then all threads fill the cells.
__global__ void __launch_bounds__(256) codebook_prepare_kernel(const float* __restrict__ codebook, int k,
                                                               unsigned char* __restrict__ ws) {
    __shared__ float cb[kMaxCodebook];
    __shared__ float thr[kMaxCodebook];
    __shared__ int tcell[kMaxCodebook];
    __shared__ int any_slow;
    const int t = threadIdx.x;
    if (t == 0) any_slow = 0;
    cb[t] = codebook[t < k ? t : k - 1];
    __syncthreads();
    thr[t] = (t < k - 1) ? entry_threshold(t, cb, k) : INFINITY;
    tcell[t] = lut_threshold_cell(thr[t]);
    __syncthreads();
    float* ws_cb = reinterpret_cast<float*>(ws + kWsCodebookOff);
    float* ws_thr = reinterpret_cast<float*>(ws + kWsThresholdOff);
    uint32_t* ws_lut = reinterpret_cast<uint32_t*>(ws + kWsLutOff);
    ws_cb[t] = cb[t];
    ws_thr[t] = thr[t];
    int slow = 0;
    for (int cell = t; cell < kLutBytes / 8; cell += blockDim.x) {
        uint32_t w0 = 0x7f800000u, w1 = 0u;  // padding entries: +inf threshold, nothing below
        if (cell <= kLutCells) lut_build_cell(cell, tcell, thr, k - 1, cb[k - 1], &w0, &w1);
        ws_lut[2 * cell] = w0;
        ws_lut[2 * cell + 1] = w1;
        if (w1 & kLutSlowBit) ++slow;
    }
    if (slow) atomicAdd(&any_slow, slow);
    __syncthreads();
    if (t == 0) {
        int* meta = reinterpret_cast<int*>(ws + kWsMetaOff);
        meta[0] = k;
        meta[1] = any_slow;
        meta[2] = 0;
        meta[3] = 0;
    }
}

static int launch_prepare(const float* codebook, int k, void* ws, cudaStream_t stream) {
    codebook_prepare_kernel<<<1, 256, 0, stream>>>(codebook, k, static_cast<unsigned char*>(ws));
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int launch_codebook_prepare(const float* codebook, int codebook_size, void* ws, cudaStream_t stream) {
    return launch_prepare(codebook, codebook_size, ws, stream);
}

// Library-owned workspaces, one per device, for callers of the reference-shaped entry points
// that pass no workspace. Rebuilt before every use, on the caller's stream.
static std::mutex g_ws_mutex;
static void* g_device_ws[64];

int resolve_codebook_ws(const float* codebook, int codebook_size, const void* caller_ws,
                        cudaStream_t stream, const void** ws_out) {
    GEFEN_CHECK_ARG(codebook != nullptr, "Expected a codebook pointer.");
    GEFEN_CHECK_ARG(codebook_size >= 1 && codebook_size <= kMaxCodebook,
                    "Expected codebook to have between 1 and 256 entries, got %d.", codebook_size);
    if (caller_ws != nullptr) {
        GEFEN_CHECK_ARG(aligned16(caller_ws), "Expected codebook_ws to be 16-byte aligned.");
        *ws_out = caller_ws;
        return GEFEN_B200_OK;
    }
    int dev = 0;
    GEFEN_CHECK_CUDA(cudaGetDevice(&dev));
    GEFEN_CHECK_ARG(dev >= 0 && dev < 64, "Unsupported device ordinal %d.", dev);
    void* ws = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_ws_mutex);
        if (g_device_ws[dev] == nullptr) {
            GEFEN_CHECK_CUDA(cudaMalloc(&g_device_ws[dev], GEFEN_B200_CODEBOOK_WS_BYTES));
        }
        ws = g_device_ws[dev];
    }
    const int rc = launch_prepare(codebook, codebook_size, ws, stream);
    if (rc != GEFEN_B200_OK) return rc;
    *ws_out = ws;
    return GEFEN_B200_OK;
}

}  // namespace gefen

extern "C" {

const char* gefen_b200_last_error(void) { return gefen::g_last_error; }

int gefen_b200_version(void) { return 1; }

int gefen_b200_codebook_prepare(const float* codebook, int codebook_size, void* workspace, void* stream) {
    using namespace gefen;
    GEFEN_CHECK_ARG(codebook != nullptr && workspace != nullptr, "Expected non-null codebook and workspace.");
    GEFEN_CHECK_ARG(codebook_size >= 1 && codebook_size <= kMaxCodebook,
                    "Expected codebook to have between 1 and 256 entries, got %d.", codebook_size);
    GEFEN_CHECK_ARG(aligned16(workspace), "Expected workspace to be 16-byte aligned.");
    return launch_prepare(codebook, codebook_size, workspace, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
