/*
 * gefen_b200 — C ABI of the B200 (sm_100a) implementation of the Gefen optimizer-step hot path.
 *
 * This header is the drop-in boundary. It replaces the pybind11 module of the reference
 * (kernels/gefen_cuda_binding.cpp:107-217, eleven functions taking at::Tensor) with plain
 * `extern "C"` entry points taking raw device pointers, sizes, dtype tags and a CUDA stream.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer unless its name starts with `host_`;
 *  - tensors are contiguous; the caller owns every buffer; in-place outputs as in the reference;
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream, which is what the
 *    reference launches on);
 *  - work is enqueued on `stream` for the CURRENT device; nothing synchronises unless stated;
 *  - return value: 0 on success, a negative GEFEN_B200_E* code otherwise; the text of the last
 *    error of the calling thread is available from gefen_b200_last_error();
 *  - nothing throws, nothing falls back to the CPU.
 */
#ifndef GEFEN_B200_H_
#define GEFEN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype tags (params/grads accept all four, optimizer-state scalars the first three) */
#define GEFEN_B200_F32 0
#define GEFEN_B200_F16 1
#define GEFEN_B200_BF16 2
#define GEFEN_B200_F64 3

#define GEFEN_B200_OK 0
#define GEFEN_B200_EINVAL (-1)   /* bad argument (reference: std::invalid_argument -> ValueError) */
#define GEFEN_B200_ECUDA (-2)    /* CUDA runtime error (reference: C10_CUDA_KERNEL_LAUNCH_CHECK) */
#define GEFEN_B200_ERUNTIME (-3) /* data-dependent failure (reference: std::runtime_error) */
#define GEFEN_B200_EUNSUPPORTED (-4)

/* Bytes of the per-codebook workspace filled by gefen_b200_codebook_prepare:
 * 256 padded codebook floats, 256 decision thresholds, 16 bytes of metadata and the
 * 4097-entry lookup table (8 bytes per entry, padded). */
#define GEFEN_B200_CODEBOOK_WS_BYTES 34848

/* flags of gefen_b200_step_tensor_t.flags */
#define GEFEN_B200_STEP_FUSE_VMEAN 1u   /* update vmean from the gradient inside the step kernel */
#define GEFEN_B200_STEP_WEIGHT_DECAY 2u /* p <- round(p * wd_mul) before the update */
#define GEFEN_B200_STEP_PERIOD1 4u      /* per-element vmean; `period` is the magnitude block */
#define GEFEN_B200_STEP_MUON 8u         /* write the dequantised momentum to `p`, no Adam update */
#define GEFEN_B200_STEP_NESTEROV 16u    /* with MUON: p <- round(round(m*beta1) + (1-beta1)*g) */
#define GEFEN_B200_STEP_PACKED 32u      /* codes are 4-bit, two per byte over the whole tensor, low nibble first */

const char* gefen_b200_last_error(void);
int gefen_b200_version(void);

/* Derives from a sorted codebook (<= 256 floats) the tables the kernels stage into shared
 * memory. Must be re-run when the codebook contents change. `workspace` holds
 * GEFEN_B200_CODEBOOK_WS_BYTES, 16-byte aligned. No counterpart in the reference, whose kernels
 * binary-search the codebook in global memory (automatic_gefen_fused_kernel.cu:59-90). */
int gefen_b200_codebook_prepare(const float* codebook, int codebook_size, void* workspace,
                                void* stream);

/* Replaces automatic_vmean_update_cuda (gefen_cuda_binding.cpp:59-63;
 * automatic_vmean_kernel.cu:66-158): vmean[b] = beta2*vmean[b] + (1-beta2)*mean(grad[b,:]^2). */
int gefen_b200_automatic_vmean_update(void* vmean, int vmean_dtype, const void* grad_view,
                                      int grad_dtype, int64_t num_blocks, int64_t period,
                                      double beta2, void* stream);

/* Replaces automatic_gefen_fused_update_from_vmean_cuda (gefen_cuda_binding.cpp:18-31;
 * automatic_gefen_fused_kernel.cu:676-833). `codebook_ws` may be NULL, in which case a
 * library-owned per-device workspace is (re)built on `stream` before the step. */
int gefen_b200_automatic_gefen_fused_update_from_vmean(
    void* p, const void* grad_view, int param_dtype, uint8_t* m_sign, void* m_magnitude,
    int magnitude_dtype, const void* vmean, int vmean_dtype, const float* codebook,
    int codebook_size, const void* codebook_ws, int packed_indices, int64_t num_blocks,
    int64_t period, double beta1, double lr, double bias_correction_1, double bias_correction_2,
    double eps, void* stream);

/* The step above for callers that are not allowed to allocate device memory: processes whose
 * whole card already belongs to another allocator, runtimes with a fixed memory plan, hooks that
 * promise to stay away from the allocator. It has no counterpart in the reference. Instead of a
 * caller-provided or lazily cudaMalloc'ed codebook workspace it uses a fixed array inside the
 * library image (GEFEN_B200_CODEBOOK_WS_BYTES on every GPU that loads the library, for the life of
 * the process), sized for the largest codebook the kernels accept: 256 entries; larger codebooks
 * are rejected with GEFEN_B200_EINVAL. Inputs and outputs are the caller's, as above. The first
 * call on a device looks the array's address up (cudaGetSymbolAddress), so make that first call
 * before starting any stream capture. The array is rewritten from `codebook` on `stream` at every
 * call; calls that can overlap on one GPU share it and race. No cudaMalloc/cudaFree is issued. */
int gefen_b200_automatic_gefen_fused_update_from_vmean_static_ws(
    void* p, const void* grad_view, int param_dtype, uint8_t* m_sign, void* m_magnitude,
    int magnitude_dtype, const void* vmean, int vmean_dtype, const float* codebook,
    int codebook_size, int packed_indices, int64_t num_blocks, int64_t period, double beta1,
    double lr, double bias_correction_1, double bias_correction_2, double eps, void* stream);

/* Replaces automatic_gefen_fused_update_cuda (gefen_cuda_binding.cpp:6-16;
 * automatic_gefen_fused_kernel.cu:556-674): same as above with a precomputed fp32 stepsize[nb]. */
int gefen_b200_automatic_gefen_fused_update(
    void* p, const void* grad_view, int param_dtype, uint8_t* m_sign, void* m_magnitude,
    int magnitude_dtype, const float* stepsize, const float* codebook, int codebook_size,
    const void* codebook_ws, int packed_indices, int64_t num_blocks, int64_t period, double beta1,
    double lr, void* stream);

/* Replaces automatic_gefen_period1_update_cuda (gefen_cuda_binding.cpp:33-47;
 * automatic_gefen_fused_kernel.cu:835-1000): per-element vmean, one magnitude per
 * `period_one_divisor` elements. */
int gefen_b200_automatic_gefen_period1_update(
    void* p, const void* grad_flat, int param_dtype, uint8_t* m_sign, void* m_magnitude,
    int magnitude_dtype, void* vmean, int vmean_dtype, const float* codebook, int codebook_size,
    const void* codebook_ws, int64_t total_numel, int64_t period_one_divisor, double beta1,
    double beta2, double lr, double bias_correction_1, double bias_correction_2, double eps,
    void* stream);

/* Replaces automatic_gefen_muon_momentum_cuda (gefen_cuda_binding.cpp:49-57;
 * automatic_gefen_fused_kernel.cu:1002-1103): momentum_update <- dequantised new momentum. */
int gefen_b200_automatic_gefen_muon_momentum(
    const void* grad_view, int grad_dtype, uint8_t* m_sign, void* m_magnitude, int magnitude_dtype,
    const float* codebook, int codebook_size, const void* codebook_ws, void* momentum_update,
    int packed_indices, int64_t num_blocks, int64_t period, double beta1, void* stream);

/* One launch for many tensors (no counterpart in the reference, which launches 2-3 kernels per
 * tensor from Python, gefen.py:1208-1333). The host table is copied into `device_table`
 * (n_tensors * sizeof(gefen_b200_step_tensor_t) bytes, caller-owned) on `stream`. Keep
 * host_table in pageable memory, or do not touch a pinned one until the copy has run: the
 * library writes first_block and reserved_ into it and the copy reads it later. All tensors of
 * one call share param_dtype. Fuses the vmean update, the weight-decay pre-multiply and the
 * step. */
typedef struct gefen_b200_step_tensor {
    void* p;            /* params, or the dense momentum output with GEFEN_B200_STEP_MUON */
    const void* g;      /* gradients, same dtype as p */
    uint8_t* codes;     /* m_codebook, one uint8 per element */
    void* mag;          /* m_magnitude [num_blocks] */
    void* v;            /* vmean [num_blocks] (per element with GEFEN_B200_STEP_PERIOD1) */
    int64_t first_block; /* filled by the library */
    int64_t num_blocks;
    int64_t period;     /* elements per magnitude block */
    float beta1, beta2, lr, bc1, bc2, eps, wd_mul; /* already rounded to float as the reference does */
    uint32_t flags;
    int32_t mag_dtype, v_dtype;
    int32_t reserved_[2];
} gefen_b200_step_tensor_t;

#define GEFEN_B200_MAX_PEERS 7

int gefen_b200_multi_tensor_step(gefen_b200_step_tensor_t* host_table, void* device_table,
                                 int n_tensors, int param_dtype, const void* codebook_ws,
                                 void* stream);
/* The same launch for a rank of a ZeRO-1 group whose parameter (and gradient) buffers, one per GPU,
 * are all mapped into this process (peer access). Two collectives ride on the kernel's own
 * accesses over NVLink:
 *  - all-gather: every updated parameter is stored to this GPU's buffer and to the same position of
 *    `n_peers` (<= GEFEN_B200_MAX_PEERS) other buffers; peer_deltas[r] = (peer r's parameter buffer
 *    base) - (this GPU's) in bytes, multiples of 16. Nothing is loaded from a peer for this.
 *  - reduce-scatter (n_grad_srcs > 0): the gradient of an element is grad_scale * (sum over the
 *    n_grad_srcs (<= GEFEN_B200_MAX_PEERS + 1) gradient buffers, fp32, in the order given: use rank
 *    order, with 0 for this rank's own buffer), rounded to the gradient dtype; grad_deltas[r] =
 *    (rank r's gradient buffer base) - (this GPU's) in bytes. The local gradient buffer is not
 *    modified. Not with GEFEN_B200_F64.
 * The caller orders the ranks with a barrier or collective on the same stream before the launch
 * (every rank's gradients are final and nobody still reads the old parameters) and after it (all
 * launches have finished: parameters complete, gradients free to be overwritten). The dense
 * momentum written with GEFEN_B200_STEP_MUON stays local. No counterpart in the reference, which
 * has no collective (gefen.py:1208-1333 runs per process). */
int gefen_b200_multi_tensor_step_peers(gefen_b200_step_tensor_t* host_table, void* device_table,
                                       int n_tensors, int param_dtype, const void* codebook_ws,
                                       const int64_t* peer_deltas, int n_peers,
                                       const int64_t* grad_deltas, int n_grad_srcs, double grad_scale,
                                       void* stream);
/* The same launch when the ranks' buffers are also bound to an NVLink multicast object (NVSwitch), as
 * symmetric-memory allocators provide it. *_multicast_delta = (multicast address of the buffer) -
 * (this GPU's address of it) in bytes, multiples of 16, 0 = not used:
 *  - param_multicast_delta: the staged kernel writes every updated parameter chunk with ONE multimem.st,
 *    which the switch delivers to every rank's copy (this GPU's included), instead of a local store plus
 *    n_peers peer stores: 1/N of the egress of the unicast all-gather;
 *  - grad_multicast_delta: the staged kernel reads every gradient chunk with ONE multimem.ld_reduce (the
 *    switch adds the ranks' copies, fp32 accumulation, one rounding to the gradient dtype), scales by
 *    grad_scale and rounds, instead of n_grad_srcs peer loads: 1/N of the ingress of the unicast
 *    reduce-scatter. The order of the switch's additions is not the rank order of the peer-load path.
 * The kernels for short, odd or unaligned blocks keep using the per-rank offsets, which must therefore be
 * given as well. Ordering between ranks is the caller's, as for gefen_b200_multi_tensor_step_peers. No
 * counterpart in the reference. */
int gefen_b200_multi_tensor_step_multicast(gefen_b200_step_tensor_t* host_table, void* device_table,
                                           int n_tensors, int param_dtype, const void* codebook_ws,
                                           const int64_t* peer_deltas, int n_peers,
                                           const int64_t* grad_deltas, int n_grad_srcs, double grad_scale,
                                           int64_t param_multicast_delta, int64_t grad_multicast_delta,
                                           void* stream);
/* dst[i] = round(scale * sum over ranks of src[i]) with the sum formed by the switch (one
 * multimem.ld_reduce per 16 bytes): what the staged kernel sees of a gradient range when it reads through
 * grad_multicast_delta, written to local memory. numel a multiple of 8, both pointers 16-byte aligned;
 * fp32, fp16 or bf16. For checks of the fused path; no counterpart in the reference. */
int gefen_b200_multicast_sum(void* dst, const void* src_multicast, int dtype, int64_t numel, double scale,
                             void* stream);
/* sizeof(gefen_b200_step_tensor_t) as compiled, for binding-side layout checks. */
int gefen_b200_step_tensor_size(void);
/* Kernel class the library would use for one table entry: 1 = vectorised staged path with one block per
 * warp pass, 2 = the same path with several blocks (of up to 1024 elements) per warp pass,
 * 0 = generic warp-per-block, -1 = generic CTA-per-block. Rows of equal
 * class that are adjacent in the table share one launch. */
int gefen_b200_step_tensor_class(const gefen_b200_step_tensor_t* host_entry, int param_dtype);

/* Error status of the step kernels on the CURRENT device. Every wait inside them is bounded; a CTA
 * whose wait for its staged tables runs out leaves without doing its share of the step and raises
 * bit 0 of a status word. This call synchronises the device, writes the word to *host_status and,
 * with clear != 0, resets it. Non-zero means that a step since the last clear was incomplete. The
 * reference has no counterpart: its kernels do not wait on anything (errors there are exceptions
 * from C10_CUDA_KERNEL_LAUNCH_CHECK). */
int gefen_b200_step_status(int* host_status, int clear);
/* Test hook: the number of polls the step kernels grant the table staging (negative = default).
 * With 0 the wait runs out at once, the kernels return without touching their tensors and the
 * status word is set; nothing faults or hangs. Process-wide, not thread-safe. */
int gefen_b200_debug_set_stage_spin_limit(int64_t limit);

/* Replaces gefen_exact_histogram_cuda (gefen_cuda_binding.cpp:65-69;
 * exact_histogram_fused_kernel.cu:131-160): bin_counts[bin] += #elements, int64, exact. */
int gefen_b200_exact_histogram(const void* grad_flat, int grad_dtype, int64_t numel,
                               int64_t period, int64_t* bin_counts, int histogram_bins,
                               void* stream);

/* Replace average_within_block_variance_cuda, average_within_block_coefficient_of_variation_cuda
 * and average_adjacent_log_block_mean_difference_cuda (gefen_cuda_binding.cpp:71-88;
 * period_variance_kernel.cu:178-396). The reference allocates and returns a device double and
 * synchronises to raise its data-dependent errors; here the raw accumulators go to caller-owned
 * device memory (zeroed by the call) and the Python wrapper applies the reference's post-ops
 * after its single device-to-host read:
 *   variance: stats[0] = sum over blocks of the block variance      -> sqrt(stats[0] / nb)
 *   cov     : stats[0] = sum of sqrt(var)/mean, stats[1] = #blocks with mean > 0,
 *             stats[2] = #blocks with mean < 0                       -> stats[0] / stats[1]
 *   adjacent: stats[0] = mean over adjacent block pairs of |mean log difference| (already
 *             divided by nb-1), stats[1] = number of elements whose log input was <= 0
 * `block_sums` is device scratch of gefen_b200_period_scratch_doubles(numel, period) doubles. */
int gefen_b200_average_within_block_variance(const void* values, int dtype, int64_t numel,
                                             int64_t period, int input_is_squared, double* stats,
                                             void* stream);
int gefen_b200_average_within_block_coefficient_of_variation(const void* values, int dtype,
                                                             int64_t numel, int64_t period,
                                                             int input_is_squared, double* stats,
                                                             void* stream);
int64_t gefen_b200_period_scratch_doubles(int64_t numel, int64_t period);
int gefen_b200_average_adjacent_log_block_mean_difference(const void* values, int dtype,
                                                          int64_t numel, int64_t period,
                                                          int input_is_squared, double epsilon,
                                                          double* stats, double* block_sums,
                                                          void* stream);

/* All candidate periods of one tensor in one call with no host synchronisation in between
 * (replaces the per-divisor launch + .item() loop of partitioning.py:259-268). The logarithm is
 * taken ONCE per element: block sums are formed at the gcd of the candidate periods and every
 * candidate's sums are regrouped from those of its largest already-computed divisor. stats holds
 * 2 * n_periods doubles: stats[2*i] = score of host_periods[i], stats[2*i+1] = the number of
 * elements whose log input was <= 0. `scratch` must hold
 * gefen_b200_period_scan_scratch_doubles(numel, host_periods, n_periods) doubles. */
int64_t gefen_b200_period_scan_scratch_doubles(int64_t numel, const int64_t* host_periods,
                                               int n_periods);
int gefen_b200_period_scan(const void* values, int dtype, int64_t numel, int input_is_squared,
                           double epsilon, const int64_t* host_periods, int n_periods,
                           double* stats, double* scratch, void* stream);

/* Replace gefen_lloyd_accumulate_cuda and gefen_lloyd_mse_cuda (gefen_cuda_binding.cpp:90-105;
 * lloyd_max_fused_kernel.cu:244-356). */
int gefen_b200_lloyd_accumulate(const void* grad_flat, int grad_dtype, int64_t numel,
                                int64_t period, const float* codebook, int codebook_size,
                                const void* codebook_ws, float* sums, int64_t* counts,
                                void* stream);
int gefen_b200_lloyd_mse(const void* grad_flat, int grad_dtype, int64_t numel, int64_t period,
                         const float* old_codebook, const float* new_codebook, int codebook_size,
                         const void* old_codebook_ws, float* mse_normalized_sum,
                         float* mse_original_sum, void* stream);

/* Exact 1-D k-means dynamic programme on the device in fp64 (replaces the numba kernel of
 * quantization.py:92-145). prefix_* are device arrays of num_points+1 doubles (prefix sums of
 * w, w*x, w*x^2 in the reference's order). `dp_scratch` holds
 * gefen_b200_exact_dp_scratch_bytes(num_points, num_codebooks) bytes. Writes num_codebooks
 * UNSORTED float32 centres to `codebook_out` (the caller sorts, as quantization.py:257 does). */
int64_t gefen_b200_exact_dp_scratch_bytes(int num_points, int num_codebooks);
int gefen_b200_exact_dp(const double* prefix_w, const double* prefix_wx, const double* prefix_wx2,
                        int num_points, int num_codebooks, int force_endpoints, void* dp_scratch,
                        float* codebook_out, void* stream);

/* The end of a GefenMuon step for one matrix (replaces the two torch kernels of gefen_muon.py:326-329):
 *   p <- round(p * wd_mul)          (skipped when wd_mul == 1; wd_mul = 1 - lr * weight_decay)
 *   p <- round(p + alpha * update)  (alpha = -adjusted_lr; update = the orthogonalised momentum)
 * in one pass, p and update of the same dtype (fp32, fp16 or bf16). With n_peers > 0 every updated
 * parameter is also stored to the same position of the peers' parameter buffers (peer_deltas as for
 * gefen_b200_multi_tensor_step_peers): the all-gather of a ZeRO-1 group rides on the kernel. */
int gefen_b200_muon_apply(void* p, const void* update, int dtype, int64_t numel, double wd_mul, double alpha,
                          const int64_t* peer_deltas, int n_peers, void* stream);

/* bf16 GEMM on the tcgen05 tensor cores for GefenMuon's Newton-Schulz iteration (replaces the
 * torch.addmm / `@` calls, i.e. cuBLAS, of gefen_muon.py:39-47):
 *   D[M,N] = alpha * A[M,K] * B[N,K]^T + beta * C[M,N], and Dt[N,M] = D^T when dt != NULL.
 * All matrices bf16 row-major with leading dimensions in elements; A and B 16-byte aligned with
 * lda, ldb multiples of 8. fp32 accumulation, one rounding to bf16. `status` (device int, may be
 * NULL) is set to 1 if a bounded wait inside the kernel ran out. `symmetric` != 0 promises that
 * the result is symmetric (M == N, e.g. A == B, C symmetric): only the tiles touching the upper
 * triangle are computed and every element is also written to its mirror position. */
int gefen_b200_ns_gemm_tn(const void* a, const void* b, const void* c, void* d, void* dt, int M,
                          int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd,
                          int64_t lddt, double alpha, double beta, int symmetric, int* status,
                          void* stream);
/* Same with B given as [K, N] row-major (an MN-major tensor-core operand):
 *   D[M,N] = alpha * A[M,K] * B[K,N] + beta * C[M,N]. */
int gefen_b200_ns_gemm_nn(const void* a, const void* b, const void* c, void* d, int M, int N,
                          int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, double alpha,
                          double beta, int* status, void* stream);
/* Both operands given K-first: A as [K, M] and B as [K, N], row-major:
 *   D[M,N] = alpha * A^T * B + beta * C  (the Gram matrix Y^T Y of a tall Y without a transpose). */
int gefen_b200_ns_gemm_tt(const void* a, const void* b, const void* c, void* d, int M, int N,
                          int K, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, double alpha,
                          double beta, int symmetric, int* status, void* stream);

/* `steps` Newton-Schulz iterations (reference: gefen_muon.py:38-47) of one already normalised bf16
 * matrix [rows, cols] (row-major, contiguous, dimensions multiples of 8), enqueued as 3 * steps
 * GEMMs: G = X X^T, B = b G + c G G, X <- a X + B X on the wide orientation, or the mirrored form
 * (Y^T Y, Y B) for rows > cols, so no transpose is ever materialised. x0 holds the input; the
 * iterates alternate between x0 and x1 and the result is in x0 when steps is even, else in x1.
 * gram and poly are [min(rows,cols)]^2 bf16 scratch. */
int gefen_b200_newton_schulz(void* x0, void* x1, void* gram, void* poly, int rows, int cols,
                             int steps, double a, double b, double c, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GEFEN_B200_H_ */
