// The steady-state Gefen step on sm_100a.
//
// What one block (`period` consecutive elements sharing a magnitude and a second moment) goes
// through, in the reference's arithmetic (kernels/automatic_gefen_fused_kernel.cu:239-318 for the
// AdamW form, :320-407 for period 1, :169-237 for GefenMuon; kernels/automatic_vmean_kernel.cu:12-51
// for the second moment; gefen.py:1280-1281 for the decoupled weight decay):
//
//   m_i   = beta1 * (mag * cb[code_i]) + (1 - beta1) * g_i              (fp32)
//   mag'  = max_i |m_i|            stored rounded to the state dtype
//   code' = nearest codebook entry of m_i / mag'   (IEEE divide by the un-rounded fp32 mag')
//   p_i  -= cb[code'_i] * mag' * step * lr,   step = (1/bc1) / (sqrt(v/bc2) + eps)
//
// Two kernels:
//  * step_vec_kernel  - the fast path, in two kinds that are compiled and launched separately: one warp
//    owns one block, or several blocks when they are not longer than 1024 elements (see
//    lanes_per_block). Codes and gradients are read once
//    (128-bit loads), the updated momenta wait in the warp's slice of shared memory while the
//    block's absmax is reduced with shuffles, then they are re-encoded and the parameters updated:
//    codes, gradients and params cross HBM exactly once (8 B/element in bf16, 14 B/element in
//    fp32). Codebook, thresholds and the quantisation table arrive in shared memory by one bulk
//    (TMA) copy per CTA. No __syncthreads after set-up; the loops are short so the code stays in
//    the instruction cache.
//  * step_generic_kernel - any period, alignment and dtype (fp64 included), period-1 tensors and
//    4-bit packed codes: two passes with scalar accesses, the second pass re-reading from L1/L2.
// Both take their tensors from a descriptor table (one launch for many tensors); a single-tensor
// call passes a one-row table inside the kernel parameters. For data-parallel ranks whose buffers
// are mapped into each other's address space the kernels can also store every updated parameter
// to the peers' copies (the all-gather) and average the gradients over the peers' copies while
// reading them (the reduce-scatter): see StepLaunch.
#include "common.cuh"

#include <mutex>
#include <stdlib.h>

namespace gefen {

// fp32 contraction choices. They reproduce what nvcc emits for the reference source when it is
// compiled with its own flags (-O3, fmad on): a*b + c*d becomes fma(a, b, c*d) and p - a*b becomes
// fma(-a, b, p); checked on a B200 against the reference's own kernels. The CPU oracle makes the
// same choices explicitly.
__device__ __forceinline__ float ema_update(float beta, float cur, float omb, float g) {
    return fmaf(beta, cur, omb * g);
}
// In the reference's period-1 kernel (automatic_gefen_fused_kernel.cu:360, :392) nvcc fuses the other
// product of the same expression; measured against the reference build, bit-identical with this form.
__device__ __forceinline__ float ema_update_period1(float beta, float cur, float omb, float g) {
    return fmaf(omb, g, beta * cur);
}

struct StepLaunch {
    const gefen_b200_step_tensor_t* table;  // device table, or nullptr: the row in the kernel params
    int n_tensors;
    int stage_floats;                       // fast path: floats of staging per warp (>= max period)
    long long total_blocks;
    const unsigned char* ws;                // codebook workspace
    const float* stepsize;                  // optional precomputed per-block step (single tensor only)
    // ZeRO-1 with the all-gather fused in: every updated parameter is also stored into the same
    // place of n_peers other GPUs' parameter buffers (byte distance from this GPU's buffer to
    // theirs in this process's address space; plain peer stores over NVLink, no loads).
    int n_peers;
    long long peer_delta[GEFEN_B200_MAX_PEERS];
    // ... and with the reduce-scatter fused in: the gradient of an element is grad_scale times the
    // sum over n_grad_srcs buffers (byte distances from this GPU's gradient buffer, rank order, 0
    // for this rank itself), rounded to the gradient dtype. 0 sources: gradients are used as they are.
    int n_grad_srcs;
    float grad_scale;
    long long grad_delta[GEFEN_B200_MAX_PEERS + 1];
    // NVLink multicast (NVSwitch) mappings of the ranks' buffers, as byte distances from this GPU's own
    // buffer; 0 = not used. grad_mc_delta: the staged kernel reads every gradient chunk with one
    // multimem.ld_reduce (the switch adds the ranks' copies, fp32 accumulation) instead of n_grad_srcs
    // peer loads. param_mc_delta: every updated parameter chunk leaves with one multimem.st that the
    // switch delivers to all ranks' copies, this GPU's included, instead of a local store plus n_peers
    // peer stores.
    long long grad_mc_delta;
    long long param_mc_delta;
    // iteration limit of the wait for the staged tables (g_stage_spin_limit on the host)
    unsigned int spin_limit;
};

// Set (never cleared by a kernel) when a bounded wait ran out and the CTA left without doing its
// share of the step: bit 0 = the table staging of a step kernel. Read and cleared by
// gefen_b200_step_status on the host.
__device__ int g_step_status;

template <typename T> __device__ __forceinline__ T* peer_ptr(T* p, long long delta) {
    return reinterpret_cast<T*>(reinterpret_cast<uintptr_t>(p) + delta);
}

constexpr int kSmemWs = GEFEN_B200_CODEBOOK_WS_BYTES;
constexpr int kMaxSmem = 227 * 1024;
// The fast path reads the codebook twice per element with data-dependent indices. One copy per
// lane (entry e of lane c at word 32*e + c, a 128-byte row per entry) makes every such read
// conflict-free, against the ~3.5-way conflict of a single 1 KB table.
constexpr int kRepCopies = 32;
constexpr int kSmemRep = kMaxCodebook * kRepCopies * 4;

struct SmemView {
    const float* cb;             // 256, padded with the last entry
    const float* thr;            // 256, padded with +inf
    const unsigned char* lut;    // kLutBytes
    const float* rep;            // fast path only: kRepCopies interleaved copies of cb, offset by the lane's copy
    int k;                       // true codebook size
};

// Stages the workspace with one bulk copy. Returns false (uniformly for the CTA) if the copy did
// not land within `spin_limit` polls of its barrier; the status word is raised then, and the CTA
// still gives the copy a second, long bounded wait before it returns, so that it does not leave
// while a copy into its shared memory is in flight.
constexpr unsigned int kStageDrainLimit = 4000000u;
__device__ __forceinline__ bool stage_tables(const unsigned char* ws, unsigned char* smem, SmemView& view,
                                             unsigned int spin_limit) {
    __shared__ uint64_t bar;
    __shared__ int ok;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_expect_tx(&bar, kSmemWs);
        bulk_copy_g2s(smem, ws, kSmemWs, &bar);
        ok = mbar_wait_bounded(&bar, 0, spin_limit) ? 1 : 0;
        if (!ok) {
            atomicOr(&g_step_status, 1);
            mbar_wait_bounded(&bar, 0, kStageDrainLimit);
        }
    }
    __syncthreads();
    view.cb = reinterpret_cast<const float*>(smem + kWsCodebookOff);
    view.thr = reinterpret_cast<const float*>(smem + kWsThresholdOff);
    view.lut = smem + kWsLutOff;
    view.rep = nullptr;
    view.k = 1;
    if (!ok) return false;
    view.k = reinterpret_cast<const int*>(smem + kWsMetaOff)[0];
    return true;
}

__device__ __forceinline__ float adam_step_size(float v, float bc1, float bc2, float eps) {
    const float corrected = v / bc2;
    return (1.0f / bc1) / (sqrtf(corrected) + eps);
}

// Finds the row that owns global block `gb` (rows sorted by first_block).
__device__ __forceinline__ int find_tensor(const gefen_b200_step_tensor_t* table, int n, long long gb) {
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (table[mid].first_block <= gb) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// --------------------------------------------------------------------------- vector IO
// A "chunk" is 8 consecutive elements: 8 code bytes, 16 B of bf16/f16 or 32 B of fp32. Everything is
// read once per step: the loads carry the streaming (evict-first) hint.
// 16-byte accesses to a multicast address: the store reaches every GPU's copy, the load returns the
// element-wise sum of all copies (added in the switch, fp32 accumulation for the 2-byte types).
__device__ __forceinline__ void multimem_store16(void* mc_addr, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}
template <typename S> __device__ __forceinline__ uint4 multimem_load_sum16(const void* mc_addr);
template <> __device__ __forceinline__ uint4 multimem_load_sum16<__nv_bfloat16>(const void* mc_addr) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
    return v;
}
template <> __device__ __forceinline__ uint4 multimem_load_sum16<__half>(const void* mc_addr) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
    return v;
}
template <> __device__ __forceinline__ uint4 multimem_load_sum16<float>(const void* mc_addr) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
    return v;
}

template <typename S> struct Chunk;
template <> struct Chunk<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load_sum(const void* mc_base, long long chunk) {
        raw = multimem_load_sum16<__nv_bfloat16>(reinterpret_cast<const uint4*>(mc_base) + chunk);
    }
    __device__ __forceinline__ void store_all(void* mc_base, long long chunk) const {
        multimem_store16(reinterpret_cast<uint4*>(mc_base) + chunk, raw);
    }
    __device__ __forceinline__ void load(const void* base, long long chunk) {
        raw = __ldcs(reinterpret_cast<const uint4*>(base) + chunk);
    }
    __device__ __forceinline__ void store(void* base, long long chunk) const {
        reinterpret_cast<uint4*>(base)[chunk] = raw;
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    __device__ __forceinline__ void pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        raw = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Chunk<__half> {
    uint4 raw;
    __device__ __forceinline__ void load_sum(const void* mc_base, long long chunk) {
        raw = multimem_load_sum16<__half>(reinterpret_cast<const uint4*>(mc_base) + chunk);
    }
    __device__ __forceinline__ void store_all(void* mc_base, long long chunk) const {
        multimem_store16(reinterpret_cast<uint4*>(mc_base) + chunk, raw);
    }
    __device__ __forceinline__ void load(const void* base, long long chunk) {
        raw = __ldcs(reinterpret_cast<const uint4*>(base) + chunk);
    }
    __device__ __forceinline__ void store(void* base, long long chunk) const {
        reinterpret_cast<uint4*>(base)[chunk] = raw;
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
    __device__ __forceinline__ void pack(const float (&f)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        raw = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Chunk<float> {
    float4 lo, hi;
    __device__ __forceinline__ void load_sum(const void* mc_base, long long chunk) {
        const uint4 a = multimem_load_sum16<float>(reinterpret_cast<const uint4*>(mc_base) + 2 * chunk);
        const uint4 b = multimem_load_sum16<float>(reinterpret_cast<const uint4*>(mc_base) + 2 * chunk + 1);
        lo = make_float4(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w));
        hi = make_float4(__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w));
    }
    __device__ __forceinline__ void store_all(void* mc_base, long long chunk) const {
        multimem_store16(reinterpret_cast<uint4*>(mc_base) + 2 * chunk,
                         make_uint4(__float_as_uint(lo.x), __float_as_uint(lo.y), __float_as_uint(lo.z), __float_as_uint(lo.w)));
        multimem_store16(reinterpret_cast<uint4*>(mc_base) + 2 * chunk + 1,
                         make_uint4(__float_as_uint(hi.x), __float_as_uint(hi.y), __float_as_uint(hi.z), __float_as_uint(hi.w)));
    }
    __device__ __forceinline__ void load(const void* base, long long chunk) {
        lo = __ldcs(reinterpret_cast<const float4*>(base) + 2 * chunk);
        hi = __ldcs(reinterpret_cast<const float4*>(base) + 2 * chunk + 1);
    }
    __device__ __forceinline__ void store(void* base, long long chunk) const {
        __stcs(reinterpret_cast<float4*>(base) + 2 * chunk, lo);   // measured: streaming stores pay for fp32 only
        __stcs(reinterpret_cast<float4*>(base) + 2 * chunk + 1, hi);
    }
    __device__ __forceinline__ void unpack(float (&f)[8]) const {
        f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w;
        f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
    }
    __device__ __forceinline__ void pack(const float (&f)[8]) {
        lo = make_float4(f[0], f[1], f[2], f[3]);
        hi = make_float4(f[4], f[5], f[6], f[7]);
    }
};

// Pulls the lines of this warp's NEXT block towards L2 while the current block is being worked on,
// so that its loads later pay an L2 hit instead of a DRAM round trip (shared memory takes almost
// all of L1, and the registers are busy: a hint costs neither).
__device__ __forceinline__ void prefetch_l2_range(const void* base, long long bytes, int lane) {
    const char* p = static_cast<const char*>(base);
    for (long long off = static_cast<long long>(lane) * 128; off < bytes; off += 32 * 128) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
    }
}

// The updated momenta of chunk c, from the warp's staging slice.
__device__ __forceinline__ void staged_momenta(const float4* stage_a, const float4* stage_b, int c, float (&m)[8]) {
    const float4 ma = stage_a[c], mb = stage_b[c];
    m[0] = ma.x; m[1] = ma.y; m[2] = ma.z; m[3] = ma.w;
    m[4] = mb.x; m[5] = mb.y; m[6] = mb.z; m[7] = mb.w;
}

// --------------------------------------------------------------------------- fast path
// lut_query_fast with the table's shared-memory address folded into the rounding constant: the low mantissa
// bits of fma(x, 16384, magic) are then the address of x's table entry itself (the address is a multiple of
// eight, so the cell, the value with its low three bits cleared, is the same one) and the query needs no add.
__device__ __forceinline__ float lut_magic(const unsigned char* lut) {
    return 12582912.0f + 16384.0f + static_cast<float>(static_cast<uint32_t>(__cvta_generic_to_shared(lut)));
}
__device__ __forceinline__ uint32_t lut_query_shared(float x, float magic) {
    const uint32_t addr = __float_as_uint(fmaf(x, 16384.0f, magic)) & 0x3FFF8u;
    uint32_t thr_bits, below;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(thr_bits), "=r"(below) : "r"(addr));
    return below + (x > __uint_as_float(thr_bits) ? 1u : 0u);
}

// Lanes that share one block, a power of two, so that a warp works on 32 / lanes blocks at once. A lane takes
// several chunks of its block, which keeps as many loads in flight and shares the per-block work (reductions,
// step size, reciprocal, descriptor reads) between more elements: about eight chunks per lane for blocks of
// more than 256 elements, as in a 2048-element block (8 lanes for 512 elements, 16 for 1024, all 32 from 1032
// elements on; measured on 512-element blocks: 0.43 ms -> 0.32 ms per 134 M elements), up to four for 136 to
// 256 elements (8 lanes; 256-element bf16 blocks: 0.25 -> 0.50 of the copy bandwidth against one chunk per
// lane), two below that (bf16, 128 / 64 / 32 elements: 0.23 -> 0.37 / 0.36 / 0.35; four per lane there puts the
// staging slices of a warp's blocks on the same shared-memory banks and is slower for 2-byte elements).
__host__ __device__ __forceinline__ int lanes_per_block(long long period) {
    const long long nchunks = period >> 3;
    const long long want = nchunks > 32 ? (nchunks + 7) >> 3 : (nchunks > 16 ? (nchunks + 3) >> 2 : (nchunks + 1) >> 1);
    int lanes = 1;
    while (lanes < 32 && lanes < want) lanes <<= 1;
    return lanes;
}
// Elements of one work unit of a tensor (what a warp stages at a time).
__host__ __device__ __forceinline__ long long unit_elements(long long period) {
    return period * (32 / lanes_per_block(period));
}
// Work units (one warp pass each) of a tensor on the fast path.
__host__ __device__ __forceinline__ long long vec_units(long long num_blocks, long long period) {
    const int group = 32 / lanes_per_block(period);
    return (num_blocks + group - 1) / group;
}

// Reductions over aligned groups of `lanes` lanes (a power of two); every lane of the warp calls them.
__device__ __forceinline__ float group_max_nan(float v, int lanes) {
    for (int o = lanes >> 1; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, o);
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(v) : "f"(v), "f"(other));
    }
    return v;
}
__device__ __forceinline__ float group_max(float v, int lanes) {
    for (int o = lanes >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float group_sum(float v, int lanes) {
    for (int o = lanes >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// First pass over U chunks of one lane (chunks c0, c0 + LANES, ...): all loads first, then the
// moment update, the running absmax and sum of squares, and the staging of the updated momenta.
// SUMMED: g_blk is the multicast address of the block's gradients; a load returns the sum over the ranks,
// which is scaled by `scale` and rounded to the gradient dtype as a reduce-scatter into it would leave it.
template <typename S, int U, bool GUARD, bool SUMMED>
__device__ __forceinline__ void first_pass_group(const S* g_blk, const uint2* codes_in, float4* stage_a, float4* stage_b,
                                                 const float* rep, int c0, int LANES, int nchunks, float old_mag,
                                                 float beta1, float omb1, float scale, float& absmax, float& sumsq) {
    uint2 craw[U];
    Chunk<S> graw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = c0 + LANES * u;
        if (!GUARD || c < nchunks) {
            craw[u] = __ldcs(codes_in + c);
            if (SUMMED) graw[u].load_sum(g_blk, c);
            else graw[u].load(g_blk, c);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int c = c0 + LANES * u;
        if (!GUARD || c < nchunks) {
            float g[8], m[8];
            graw[u].unpack(g);
            if (SUMMED) {
#pragma unroll
                for (int i = 0; i < 8; ++i) g[i] *= scale;
                Chunk<S> rounded;
                rounded.pack(g);
                rounded.unpack(g);
            }
            const uint32_t cw[2] = {craw[u].x, craw[u].y};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t code = __byte_perm(cw[i >> 2], 0u, 0x4440u + (i & 3));   // byte i & 3, zero-extended
                const float cur = old_mag * rep[code * kRepCopies];
                m[i] = ema_update(beta1, cur, omb1, g[i]);
                absmax = max_abs_nan(absmax, m[i]);
                sumsq = fmaf(g[i], g[i], sumsq);
            }
            stage_a[c] = make_float4(m[0], m[1], m[2], m[3]);
            stage_b[c] = make_float4(m[4], m[5], m[6], m[7]);
        }
    }
}

// First pass of a block whose gradient is averaged over up to NSRC buffers. kSlots 16-byte (fp32:
// 32-byte) loads per lane are in flight at a time: U chunks x a batch of BS sources; the sources of
// a chunk are added batch after batch, in the order given.
// EXACT: there are exactly NSRC sources (no test per source).
template <typename S, int NSRC, bool EXACT = false>
__device__ __forceinline__ void reduce_pass(const StepLaunch& L, const S* g_blk, const uint2* codes_in, float4* stage_a,
                                            float4* stage_b, const float* rep, int lane, int LANES, int nchunks,
                                            float old_mag, float beta1, float omb1, float& absmax, float& sumsq) {
    constexpr int kSlots = sizeof(S) == 2 ? 4 : 2;
    constexpr int BS = NSRC < kSlots ? NSRC : kSlots;
    constexpr int U = kSlots / BS;
    const int n_src = EXACT ? NSRC : L.n_grad_srcs;
    const float scale = L.grad_scale;
    for (int c0 = lane; c0 < nchunks; c0 += LANES * U) {
        float acc[U][8];
        uint2 craw[U];   // the codes travel with the first batch of gradient loads
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
            if (c0 + LANES * u < nchunks) craw[u] = __ldcs(codes_in + c0 + LANES * u);
        }
#pragma unroll
        for (int r0 = 0; r0 < NSRC; r0 += BS) {
            if (r0 < n_src) {
                Chunk<S> src[U * BS];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int c = c0 + LANES * u;
#pragma unroll
                    for (int r = 0; r < BS; ++r)
                        if (c < nchunks && r0 + r < n_src) src[u * BS + r].load(peer_ptr(g_blk, L.grad_delta[r0 + r]), c);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int c = c0 + LANES * u;
#pragma unroll
                    for (int r = 0; r < BS; ++r) {
                        if (c < nchunks && r0 + r < n_src) {
                            float part[8];
                            src[u * BS + r].unpack(part);
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[u][i] += part[i];
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + LANES * u;
            if (c < nchunks) {
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[u][i] *= scale;
                Chunk<S> rounded;
                rounded.pack(acc[u]);
                float g[8], m[8];
                rounded.unpack(g);
                const uint32_t cw[2] = {craw[u].x, craw[u].y};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const uint32_t code = __byte_perm(cw[i >> 2], 0u, 0x4440u + (i & 3));   // byte i & 3, zero-extended
                    const float cur = old_mag * rep[code * kRepCopies];
                    m[i] = ema_update(beta1, cur, omb1, g[i]);
                    absmax = max_abs_nan(absmax, m[i]);
                    sumsq = fmaf(g[i], g[i], sumsq);
                }
                stage_a[c] = make_float4(m[0], m[1], m[2], m[3]);
                stage_b[c] = make_float4(m[4], m[5], m[6], m[7]);
            }
        }
    }
}

// The re-encode and update loop of the common case (finite block, Gefen update of the parameters) with
// everything that is fixed per launch or per tensor decided at compile time, so that the loop body carries no
// branch but the rare one into the exact quantiser: WD = the decoupled weight decay of the reference's
// separate multiply, STORE = 0 this GPU's copy only, 1 peer stores as well, 2 one multicast store.
// The parameters of the next chunk are fetched while this one is encoded.
template <typename S, bool WD, int STORE>
__device__ __forceinline__ void second_pass_common(const StepLaunch& L, const SmemView& s, const float* rep,
                                                   const float4* stage_a, const float4* stage_b, uint2* codes_out,
                                                   S* p_blk, Chunk<S> pnext, int lane, int LANES, int nchunks,
                                                   float absmax, float rinv, float step, float lr, float wd_mul) {
    const float neg_step = -step;
    const float magic = lut_magic(s.lut);
    for (int c = lane; c < nchunks; c += LANES) {
        Chunk<S> praw = pnext;
        if (c + LANES < nchunks) pnext.load(p_blk, c + LANES);
        float m[8];
        staged_momenta(stage_a, stage_b, c, m);
        uint32_t code[8];
        uint32_t any = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x = div_by_block_constant(m[i], absmax, rinv);
            code[i] = lut_query_shared(x, magic);
            any |= code[i];
        }
        if (any & kLutSlowBit) {   // rare: a cell with two thresholds, or values above the last entry
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (code[i] & kLutSlowBit) {
                    const float x = div_by_block_constant(m[i], absmax, rinv);
                    code[i] = static_cast<uint32_t>(entry_exact(x, s.thr, s.cb, s.k));
                }
            }
        }
        uint2 cw;
        cw.x = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
        cw.y = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
        codes_out[c] = cw;
        float pv[8];
        praw.unpack(pv);
        if (WD) {
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] *= wd_mul;
            Chunk<S> rounded;       // the separate multiply of the reference rounds to the parameter dtype
            rounded.pack(pv);
            rounded.unpack(pv);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float q = rep[code[i] * kRepCopies] * absmax;
            pv[i] = fmaf(q * neg_step, lr, pv[i]);   // = fma(-(q * step), lr, p)
        }
        praw.pack(pv);
        if (STORE == 2) {
            praw.store_all(peer_ptr(p_blk, L.param_mc_delta), c);   // every rank's copy, this one included
        } else {
            praw.store(p_blk, c);
            if (STORE == 1) {
                const int n_peers = L.n_peers;
                for (int r = 0; r < n_peers; ++r) praw.store(peer_ptr(p_blk, L.peer_delta[r]), c);
            }
        }
    }
}

// The same loop for GefenMuon's momentum step (finite block): the dequantised new momentum, Nesterov-blended
// with the gradient when asked (torch: m.mul_(momentum).add_(g, alpha=1-momentum) on the rounded momentum,
// reference gefen_muon.py:312-314; alpha travels in the descriptor's beta2), goes where the Gefen step keeps
// the parameters. The gradient chunk of the next iteration is requested while this one is encoded.
template <typename S, bool NESTEROV>
__device__ __forceinline__ void second_pass_muon(const SmemView& s, const float* rep, const float4* stage_a,
                                                 const float4* stage_b, uint2* codes_out, const S* g_blk, S* out_blk,
                                                 int lane, int LANES, int nchunks, float absmax, float rinv,
                                                 float beta1, float alpha) {
    const float magic = lut_magic(s.lut);
    Chunk<S> gnext;
    if (NESTEROV && lane < nchunks) gnext.load(g_blk, lane);
    for (int c = lane; c < nchunks; c += LANES) {
        Chunk<S> graw = gnext;
        if (NESTEROV && c + LANES < nchunks) gnext.load(g_blk, c + LANES);
        float m[8];
        staged_momenta(stage_a, stage_b, c, m);
        uint32_t code[8];
        uint32_t any = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x = div_by_block_constant(m[i], absmax, rinv);
            code[i] = lut_query_shared(x, magic);
            any |= code[i];
        }
        if (any & kLutSlowBit) {   // rare: a cell with two thresholds, or values above the last entry
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (code[i] & kLutSlowBit) {
                    const float x = div_by_block_constant(m[i], absmax, rinv);
                    code[i] = static_cast<uint32_t>(entry_exact(x, s.thr, s.cb, s.k));
                }
            }
        }
        uint2 cw;
        cw.x = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
        cw.y = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
        codes_out[c] = cw;
        float q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = rep[code[i] * kRepCopies] * absmax;
        if (NESTEROV) {
            float g[8];
            graw.unpack(g);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float m1 = ScalarIO<S>::round(ScalarIO<S>::round(q[i]) * beta1);
                q[i] = fmaf(alpha, g[i], m1);
            }
        }
        Chunk<S> out;
        out.pack(q);
        out.store(out_blk, c);
    }
}

// One warp, one unit: 32 / LANES consecutive blocks of t.period = 8 * nchunks elements, LANES lanes
// each (LANES = lanes_per_block(t.period), uniform over the warp; FULL fixes it to 32 at compile
// time, for blocks of more than 1024 elements). A block's slice of `stage` holds period floats: the first halves of all chunks, then the
// second halves, so that the 128-bit shared accesses of a full warp are conflict-free.
// The descriptor lives in global or parameter memory, which the stores below might alias as far as
// the compiler can tell: everything the loops need from it is copied into locals first.
// GSRC: where the gradients come from: 0 = this GPU's buffer, 1 = averaged over the ranks' buffers with peer
// loads, 2 = summed by the switch through the multicast mapping (StepLaunch::grad_mc_delta).
template <typename S, int GSRC, bool FULL>
__device__ __forceinline__ void warp_block_step(const gefen_b200_step_tensor_t& t, long long unit, const StepLaunch& L,
                                                const SmemView& s, float* stage, int warp_lane) {
    const float* const stepsize = L.stepsize;
    const int n_peers = L.n_peers;
    const long long param_mc = L.param_mc_delta;
    const int period = static_cast<int>(t.period);     // at most kFastMaxPeriod
    const int LANES = FULL ? 32 : lanes_per_block(period);
    const int lane = warp_lane & (LANES - 1);          // lane within the block's group
    const int member = warp_lane >> (31 - __clz(LANES));   // which block of the unit
    const long long b = unit * (32 / LANES) + member;
    const bool valid = b < t.num_blocks;               // the last unit of a tensor may be short
    const int nchunks = valid ? (period >> 3) : 0;
    stage += member * period;
    const long long elem0 = b * static_cast<long long>(period);
    const uint2* const codes_in = reinterpret_cast<const uint2*>(t.codes + elem0);
    uint2* const codes_out = reinterpret_cast<uint2*>(t.codes + elem0);
    const S* const g_blk = static_cast<const S*>(t.g) + elem0;   // chunk c of the block = 8 elements at g_blk + 8 c
    S* const p_blk = static_cast<S*>(t.p) + elem0;
    const uint32_t flags = t.flags;
    const bool muon = (flags & GEFEN_B200_STEP_MUON) != 0;

    const float beta1 = t.beta1;
    const float omb1 = 1.0f - beta1;
    const float old_mag = valid ? load_state(t.mag, b, t.mag_dtype) : 0.0f;
    float4* const stage_a = reinterpret_cast<float4*>(stage);
    float4* const stage_b = stage_a + (period >> 3);
    const float* rep = s.rep;  // this lane's copy of the codebook: entry e at rep[e * kRepCopies]

    // Everything the block needs from HBM besides codes and gradients is requested now, so that its
    // latency overlaps the first pass: the second moment and, where the registers allow it (2-byte
    // types), the first chunk of parameters.
    constexpr bool kEarlyParams = sizeof(S) == 2;
    const float lr = t.lr;
    const float wd_mul = t.wd_mul;
    const float nesterov_alpha = t.beta2;
    const bool do_update = muon || lr != 0.0f;
    const bool load_p = !muon && do_update;
    float v_in = 1.0f;
    if (!muon && valid) v_in = stepsize != nullptr ? stepsize[b] : load_state(t.v, b, t.v_dtype);
    Chunk<S> pnext;
    if (kEarlyParams && load_p && lane < nchunks) pnext.load(p_blk, lane);

    // ---- pass over codes and gradients (the only read of both)
    float absmax = 0.0f;
    float sumsq = 0.0f;
    if (GSRC == 2) {
        constexpr int U = 4;
        const S* const g_sum = peer_ptr(g_blk, L.grad_mc_delta);
        for (int c0 = lane; c0 < nchunks; c0 += LANES * U)
            first_pass_group<S, U, true, true>(g_sum, codes_in, stage_a, stage_b, rep, c0, LANES, nchunks, old_mag, beta1, omb1,
                                               L.grad_scale, absmax, sumsq);
    } else if (GSRC == 1) {
        // The gradient of this block is the average over the ranks' buffers (this GPU's and the
        // peers', read over NVLink), summed in fp32 in rank order and rounded to the gradient dtype,
        // as a reduce-scatter into that dtype would leave it.
        const int n_src = L.n_grad_srcs;
        if (n_src == 2) reduce_pass<S, 2, true>(L, g_blk, codes_in, stage_a, stage_b, rep, lane, LANES, nchunks, old_mag, beta1, omb1, absmax, sumsq);
        else if (n_src < 2) reduce_pass<S, 2>(L, g_blk, codes_in, stage_a, stage_b, rep, lane, LANES, nchunks, old_mag, beta1, omb1, absmax, sumsq);
        else if (n_src == 4) reduce_pass<S, 4, true>(L, g_blk, codes_in, stage_a, stage_b, rep, lane, LANES, nchunks, old_mag, beta1, omb1, absmax, sumsq);
        else if (n_src < 4) reduce_pass<S, 4>(L, g_blk, codes_in, stage_a, stage_b, rep, lane, LANES, nchunks, old_mag, beta1, omb1, absmax, sumsq);
        else reduce_pass<S, 8>(L, g_blk, codes_in, stage_a, stage_b, rep, lane, LANES, nchunks, old_mag, beta1, omb1, absmax, sumsq);
    } else {
        // up to four chunks in flight per lane (blocks of up to 256 elements have one chunk per lane). With the
        // kernels of the two block kinds compiled apart, four fit the registers of both (measured on blocks of
        // 512 / 1024 bf16 elements: 0.549 -> 0.599 / 0.566 -> 0.620 of the copy bandwidth against one in flight)
        constexpr int U = (sizeof(S) == 4 && !FULL) ? 2 : 4;   // (fp32 blocks that share a warp: see vec_max_threads)
        // (a separate loop without bounds tests for the complete groups was measured: slower, it
        // costs registers)
        for (int c0 = lane; c0 < nchunks; c0 += LANES * U)
            first_pass_group<S, U, true, false>(g_blk, codes_in, stage_a, stage_b, rep, c0, LANES, nchunks, old_mag, beta1, omb1,
                                                1.0f, absmax, sumsq);
    }
    absmax = group_max_nan(absmax, LANES);

    // ---- second moment (optionally fused) and the step size
    float step = 0.0f;
    if (!muon) {
        if (stepsize != nullptr) {
            step = v_in;
        } else {
            float v = v_in;
            if (flags & GEFEN_B200_STEP_FUSE_VMEAN) {
                const float mean_sq = group_sum(sumsq, LANES) / static_cast<float>(period);
                const float nv = fmaf(t.beta2, v_in, (1.0f - t.beta2) * mean_sq);
                v = 0.0f;
                if (lane == 0 && valid) v = store_state(t.v, b, t.v_dtype, nv);
                v = __shfl_sync(0xffffffffu, v, warp_lane & ~(LANES - 1));
            }
            step = adam_step_size(v, t.bc1, t.bc2, t.eps);
        }
    }
    __syncwarp();  // staged momenta are visible to the whole warp; every lane has read the old magnitude

    // ---- rare: a NaN or Inf in the block. The reference's max ignores NaN; redo it that way and
    // let the exact (threshold) quantiser handle non-finite quotients.
    bool exact_path = false;
    if (__any_sync(0xffffffffu, !(absmax <= 3.0e38f))) {   // warp-uniform: the reduction below shuffles
        float mx = 0.0f;
        for (int c = lane; c < nchunks; c += LANES) {
            float m[8];
            staged_momenta(stage_a, stage_b, c, m);
#pragma unroll
            for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(m[i]));
        }
        absmax = group_max(mx, LANES);
        exact_path = true;
    }
    if (lane == 0 && valid) store_state(t.mag, b, t.mag_dtype, absmax);

    const bool nonzero = absmax > 0.0f;
    const bool fastdiv = !exact_path && div_range_ok(absmax);
    const float rinv = fastdiv ? 1.0f / absmax : 0.0f;
    const bool wd = (flags & GEFEN_B200_STEP_WEIGHT_DECAY) != 0;
    const bool nesterov = (flags & GEFEN_B200_STEP_NESTEROV) != 0;

    // ---- re-encode and update; the parameters of the next chunk are fetched while this one is encoded
    if (!kEarlyParams && load_p && lane < nchunks) pnext.load(p_blk, lane);
    // The common case takes the loop that was compiled for it (the conditions are uniform over the warp: they
    // come from the launch and the tensor's descriptor, and a warp's blocks go one way together).
    if (__all_sync(0xffffffffu, fastdiv || !valid) && !muon && do_update) {
        const int store = param_mc != 0 ? 2 : (n_peers > 0 ? 1 : 0);
#define GEFEN_SECOND_PASS(WD_, STORE_)                                                                                      \
    second_pass_common<S, WD_, STORE_>(L, s, rep, stage_a, stage_b, codes_out, p_blk, pnext, lane, LANES, nchunks, absmax, \
                                       rinv, step, lr, wd_mul)
        if (store == 0) { if (wd) GEFEN_SECOND_PASS(true, 0); else GEFEN_SECOND_PASS(false, 0); }
        else if (store == 1) { if (wd) GEFEN_SECOND_PASS(true, 1); else GEFEN_SECOND_PASS(false, 1); }
        else { if (wd) GEFEN_SECOND_PASS(true, 2); else GEFEN_SECOND_PASS(false, 2); }
#undef GEFEN_SECOND_PASS
        __syncwarp();  // the staging slice is free for this warp's next block
        return;
    }
    if (GSRC == 0 && muon && __all_sync(0xffffffffu, fastdiv || !valid)) {
        if (nesterov) second_pass_muon<S, true>(s, rep, stage_a, stage_b, codes_out, g_blk, p_blk, lane, LANES, nchunks, absmax,
                                                rinv, beta1, nesterov_alpha);
        else second_pass_muon<S, false>(s, rep, stage_a, stage_b, codes_out, g_blk, p_blk, lane, LANES, nchunks, absmax, rinv,
                                        beta1, nesterov_alpha);
        __syncwarp();  // the staging slice is free for this warp's next block
        return;
    }
    // Everything else (lr == 0, blocks that are all zero or hold NaN or Inf, magnitudes outside the range of the
    // reciprocal, GefenMuon's momentum over averaged gradients): the general loop.
    for (int c = lane; c < nchunks; c += LANES) {
        Chunk<S> praw = pnext;
        if (load_p && c + LANES < nchunks) pnext.load(p_blk, c + LANES);
        float m[8];
        staged_momenta(stage_a, stage_b, c, m);
        uint32_t code[8];
        float q[8];
        if (fastdiv) {
            uint32_t any = 0u;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float x = div_by_block_constant(m[i], absmax, rinv);
                code[i] = lut_query_fast(x, s.lut);
                any |= code[i];
            }
            if (any & kLutSlowBit) {   // rare: a cell with two thresholds, or values above the last entry
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (code[i] & kLutSlowBit) {
                        const float x = div_by_block_constant(m[i], absmax, rinv);
                        code[i] = static_cast<uint32_t>(entry_exact(x, s.thr, s.cb, s.k));
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = rep[code[i] * kRepCopies] * absmax;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float x = 0.0f;
                if (nonzero) x = m[i] / absmax;
                code[i] = static_cast<uint32_t>(entry_exact(x, s.thr, s.cb, s.k));
                q[i] = s.cb[code[i]] * absmax;
            }
        }
        uint2 cw;
        cw.x = __byte_perm(__byte_perm(code[0], code[1], 0x0040), __byte_perm(code[2], code[3], 0x0040), 0x5410);
        cw.y = __byte_perm(__byte_perm(code[4], code[5], 0x0040), __byte_perm(code[6], code[7], 0x0040), 0x5410);
        codes_out[c] = cw;
        if (muon) {
            if (nesterov) {
                // torch: m.mul_(momentum).add_(g, alpha=1-momentum) on the rounded momentum
                // (reference: gefen_muon.py:312-314); alpha travels in t.beta2.
                Chunk<S> g2;
                g2.load(g_blk, c);
                float g[8];
                g2.unpack(g);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float m1 = ScalarIO<S>::round(ScalarIO<S>::round(q[i]) * beta1);
                    q[i] = fmaf(nesterov_alpha, g[i], m1);
                }
            }
            Chunk<S> out;
            out.pack(q);
            out.store(p_blk, c);
        } else if (do_update) {
            float pv[8];
            praw.unpack(pv);
            if (wd) {
#pragma unroll
                for (int i = 0; i < 8; ++i) pv[i] *= wd_mul;
                Chunk<S> rounded;       // the separate multiply of the reference rounds to the parameter dtype
                rounded.pack(pv);
                rounded.unpack(pv);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] = fmaf(-(q[i] * step), lr, pv[i]);
            praw.pack(pv);
            if (param_mc != 0) {
                praw.store_all(peer_ptr(p_blk, param_mc), c);   // every rank's copy, this one included
            } else {
                praw.store(p_blk, c);
                for (int r = 0; r < n_peers; ++r) praw.store(peer_ptr(p_blk, L.peer_delta[r]), c);
            }
        }
    }
    __syncwarp();  // the staging slice is free for this warp's next block
}

// Warps per CTA of the staged kernel: twenty for 2-byte types (96 registers per thread), sixteen for
// fp32, whose wider chunks need the full 128.
// The variant that averages gradients over NVLink holds more loads in flight per thread and is not
// bound by occupancy: sixteen warps of 128 registers for every type.
// fp32 tensors whose blocks share a warp are bound by the latency of their loads: there twenty warps of 96
// registers with two chunks in flight beat sixteen of 128 with four (measured on 768-element blocks: 0.725
// against 0.703 of the copy bandwidth).
template <typename S, int GSRC, bool FULL> __host__ __device__ constexpr int vec_max_threads() {
    if (sizeof(S) == 4 && GSRC == 0 && !FULL) return 640;
    return (sizeof(S) == 2 && GSRC != 1) ? 640 : 512;
}

// GSRC: see warp_block_step. FULL: every tensor of the launch has whole-warp blocks (lanes_per_block == 32);
// otherwise none has. The two kinds are separate kernels so that each is compiled (registers, code size) for
// its own loop structure.
template <typename S, int GSRC, bool FULL>
__global__ void __launch_bounds__(vec_max_threads<S, GSRC, FULL>(), 1) step_vec_kernel(const __grid_constant__ StepLaunch L,
                                                           const __grid_constant__ gefen_b200_step_tensor_t single) {
    extern __shared__ __align__(128) unsigned char smem[];
    SmemView s;
    if (!stage_tables(L.ws, smem, s, L.spin_limit)) return;
    const gefen_b200_step_tensor_t* table = L.table != nullptr ? L.table : &single;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int warps = blockDim.x >> 5;
    {
        float* rep = reinterpret_cast<float*>(smem + kSmemWs);
        for (int i = threadIdx.x; i < kMaxCodebook * kRepCopies; i += blockDim.x) rep[i] = s.cb[i / kRepCopies];
        s.rep = rep + (lane & (kRepCopies - 1));
        __syncthreads();
    }
    float* stage = reinterpret_cast<float*>(smem + kSmemWs + kSmemRep) + static_cast<size_t>(warp) * L.stage_floats;
    const long long warp_global = static_cast<long long>(blockIdx.x) * warps + warp;
    const long long warp_stride = static_cast<long long>(gridDim.x) * warps;
    const gefen_b200_step_tensor_t* __restrict__ tp = table;
    // On this path first_block and total_blocks count work units (see vec_units), not blocks.
    long long t_first = tp->first_block, t_count = vec_units(tp->num_blocks, tp->period);
    for (long long gb = warp_global; gb < L.total_blocks; gb += warp_stride) {
        if (gb < t_first || gb >= t_first + t_count) {
            tp = table + find_tensor(table, L.n_tensors, gb);
            t_first = tp->first_block;
            t_count = vec_units(tp->num_blocks, tp->period);
        }
        const gefen_b200_step_tensor_t& t = *tp;
        const long long nb_local = gb - t_first;
        const long long next = nb_local + warp_stride;
        // same tensor: hint the next block of this warp (measured: pays for 2-byte dtypes with long blocks only)
        const long long unit_elems = unit_elements(t.period);
        if (GSRC == 0 && sizeof(S) == 2 && unit_elems >= 1024 && next + 1 < t_count) {   // (not a ragged last unit)
            const long long elem0 = next * unit_elems;
            prefetch_l2_range(t.codes + elem0, unit_elems, lane);
            prefetch_l2_range(static_cast<const char*>(t.g) + elem0 * sizeof(S), unit_elems * sizeof(S), lane);
            if (!(t.flags & GEFEN_B200_STEP_MUON))
                prefetch_l2_range(static_cast<const char*>(t.p) + elem0 * sizeof(S), unit_elems * sizeof(S), lane);
        }
        warp_block_step<S, GSRC, FULL>(t, nb_local, L, s, stage, lane);
    }
}

// One gradient element as the step sees it: the local value, or the rounded average over the
// ranks' buffers (see StepLaunch::grad_delta).
template <typename S>
__device__ __forceinline__ float gradient_element(const S* g, const StepLaunch& L) {
    if (L.n_grad_srcs == 0) return ScalarIO<S>::load(g);
    float acc = 0.0f;
    for (int r = 0; r < L.n_grad_srcs; ++r) acc += ScalarIO<S>::load(peer_ptr(g, L.grad_delta[r]));
    return ScalarIO<S>::round(acc * L.grad_scale);
}

// --------------------------------------------------------------------------- generic path
// GROUP = 32: one warp per block; GROUP = 256: one CTA per block. Two passes, scalar accesses.
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <typename S, int GROUP>
__global__ void __launch_bounds__(kThreads) step_generic_kernel(const __grid_constant__ StepLaunch L,
                                                                const __grid_constant__ gefen_b200_step_tensor_t single) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float red_max[kWarps];
    __shared__ float red_sum[kWarps];
    SmemView s;
    if (!stage_tables(L.ws, smem, s, L.spin_limit)) return;
    const gefen_b200_step_tensor_t* table = L.table != nullptr ? L.table : &single;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int tig = (GROUP == 32) ? lane : static_cast<int>(threadIdx.x);
    const long long group_global = (GROUP == 32) ? static_cast<long long>(blockIdx.x) * kWarps + warp
                                                 : static_cast<long long>(blockIdx.x);
    const long long group_stride = (GROUP == 32) ? static_cast<long long>(gridDim.x) * kWarps
                                                 : static_cast<long long>(gridDim.x);

    for (long long gb = group_global; gb < L.total_blocks; gb += group_stride) {
        const gefen_b200_step_tensor_t* tp = table + find_tensor(table, L.n_tensors, gb);
        const int period = static_cast<int>(tp->period);
        const uint32_t flags = tp->flags;
        // 4-bit codes with an odd period: blocks 2k and 2k + 1 share the byte between them (and with no other
        // block), so the pair is one unit of work and its two blocks are taken one after the other by the same
        // threads; see paired_units.
        const int halves = ((flags & GEFEN_B200_STEP_PACKED) != 0 && (period & 1) != 0) ? 2 : 1;
        for (int half = 0; half < halves; ++half) {
        const long long b = (gb - tp->first_block) * halves + half;
        if (b >= tp->num_blocks) break;
        const long long start = b * period;
        const bool muon = (flags & GEFEN_B200_STEP_MUON) != 0;
        const bool period1 = (flags & GEFEN_B200_STEP_PERIOD1) != 0;
        const bool fuse_v = (flags & GEFEN_B200_STEP_FUSE_VMEAN) != 0;
        const bool wd = (flags & GEFEN_B200_STEP_WEIGHT_DECAY) != 0;
        const bool nesterov = (flags & GEFEN_B200_STEP_NESTEROV) != 0;
        const S* g = static_cast<const S*>(tp->g) + start;
        S* prm = static_cast<S*>(tp->p) + start;
        // 4-bit codes (reference: automatic_gefen_fused_kernel.cu:14-57): two per byte over the whole
        // tensor, low nibble first. A thread owns a byte and the (one or two) elements of this block in it: no
        // atomics (the reference uses atomicCAS). lead = 1: the block starts on the high nibble of its first
        // byte, whose low nibble belongs to the block before; likewise the last byte's high nibble may belong
        // to the block after. Such bytes are rewritten with the other block's nibble kept.
        const bool packed = (flags & GEFEN_B200_STEP_PACKED) != 0;
        const int per = packed ? 2 : 1;
        const int lead = packed ? static_cast<int>(start & 1) : 0;
        uint8_t* codes = tp->codes + (packed ? start / 2 : start);
        void* mag_ptr = tp->mag;
        void* v_ptr = tp->v;
        const int mag_dtype = tp->mag_dtype, v_dtype = tp->v_dtype;
        const float beta1 = tp->beta1;
        const float omb1 = 1.0f - beta1;
        const float beta2 = tp->beta2;
        const float omb2 = 1.0f - beta2;
        const float lr = tp->lr, bc1 = tp->bc1, bc2 = tp->bc2, eps = tp->eps, wd_mul = tp->wd_mul;
        const float old_mag = load_state(mag_ptr, b, mag_dtype);

        // pass 1: NaN-ignoring absmax of the updated momentum (the reference's `>` test), sum g^2;
        // period-1 tensors update their per-element second moment here
        // (reference: automatic_gefen_fused_kernel.cu:350-366).
        float absmax = 0.0f, sumsq = 0.0f;
        for (int i0 = tig * per - lead; i0 < period; i0 += GROUP * per) {
            const uint32_t byte = codes[packed ? (i0 + lead) / 2 : i0];
            for (int e = 0; e < per; ++e) {
                const int i = i0 + e;
                if (i < 0 || i >= period) continue;   // the neighbouring block's nibble
                const uint32_t old_code = packed ? ((byte >> (4 * e)) & 0xFu) : byte;
                const float gi = gradient_element(g + i, L);
                if (period1) {
                    const float prev = load_state(v_ptr, start + i, v_dtype);
                    store_state(v_ptr, start + i, v_dtype, fmaf(beta2, prev, (omb2 * gi) * gi));
                }
                const float cur = old_mag * s.cb[old_code];
                const float u = period1 ? ema_update_period1(beta1, cur, omb1, gi) : ema_update(beta1, cur, omb1, gi);
                absmax = fmaxf(absmax, fabsf(u));
                sumsq = fmaf(gi, gi, sumsq);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) absmax = fmaxf(absmax, __shfl_xor_sync(0xffffffffu, absmax, o));
        sumsq = warp_sum(sumsq);
        if (GROUP > 32) {
            __syncthreads();  // previous iteration's readers are done with red_*
            if (lane == 0) { red_max[warp] = absmax; red_sum[warp] = sumsq; }
            __syncthreads();
            absmax = red_max[0];
            sumsq = red_sum[0];
#pragma unroll
            for (int w = 1; w < kWarps; ++w) { absmax = fmaxf(absmax, red_max[w]); sumsq += red_sum[w]; }
        }

        float step = 0.0f;
        if (!muon && !period1) {
            if (L.stepsize != nullptr) {
                step = L.stepsize[b];
            } else {
                float v = load_state(v_ptr, b, v_dtype);
                float nv = 0.0f;
                if (fuse_v) {
                    nv = fmaf(beta2, v, omb2 * (sumsq / static_cast<float>(period)));
                    // every thread computes the same rounded value; one thread stores it below
                    if (v_dtype == GEFEN_B200_F32) v = nv;
                    else if (v_dtype == GEFEN_B200_BF16) v = __bfloat162float(__float2bfloat16_rn(nv));
                    else v = __half2float(__float2half_rn(nv));
                }
                step = adam_step_size(v, bc1, bc2, eps);
                if (fuse_v) {
                    if (GROUP > 32) __syncthreads(); else __syncwarp();  // everyone has read the old vmean
                    if (tig == 0) store_state(v_ptr, b, v_dtype, nv);
                }
            }
        }
        if (GROUP > 32) __syncthreads(); else __syncwarp();  // old magnitude was read by everyone
        if (tig == 0) store_state(mag_ptr, b, mag_dtype, absmax);
        const bool do_update = muon || period1 || lr != 0.0f;

        // pass 2: re-encode and update
        for (int i0 = tig * per - lead; i0 < period; i0 += GROUP * per) {
            const uint32_t byte = codes[packed ? (i0 + lead) / 2 : i0];
            uint32_t new_byte = 0u;
            for (int e = 0; e < per; ++e) {
            const int i = i0 + e;
            if (i < 0 || i >= period) {   // the neighbouring block's nibble stays
                new_byte |= byte & (0xFu << (4 * e));
                continue;
            }
            const uint32_t old_code = packed ? ((byte >> (4 * e)) & 0xFu) : byte;
            const float gi = gradient_element(g + i, L);
            const float cur = old_mag * s.cb[old_code];
            const float u = period1 ? ema_update_period1(beta1, cur, omb1, gi) : ema_update(beta1, cur, omb1, gi);
            float x = 0.0f;
            if (absmax > 0.0f) x = u / absmax;
            const uint32_t code = static_cast<uint32_t>(entry_exact(x, s.thr, s.cb, s.k));
            new_byte |= packed ? ((code & 0xFu) << (4 * e)) : code;
            const float q = s.cb[code] * absmax;
            if (muon) {
                float out = q;
                if (nesterov) out = fmaf(beta2, gi, ScalarIO<S>::round(ScalarIO<S>::round(q) * beta1));
                ScalarIO<S>::store(prm + i, out);
            } else if (do_update) {
                float st = step;
                if (period1) st = adam_step_size(load_state(v_ptr, start + i, v_dtype), bc1, bc2, eps);
                float pi = ScalarIO<S>::load(prm + i);
                if (wd) pi = ScalarIO<S>::round(pi * wd_mul);
                const float updated = fmaf(-(q * st), lr, pi);
                ScalarIO<S>::store(prm + i, updated);
                for (int r = 0; r < L.n_peers; ++r) ScalarIO<S>::store(peer_ptr(prm + i, L.peer_delta[r]), updated);
            }
            }
            codes[packed ? (i0 + lead) / 2 : i0] = static_cast<uint8_t>(new_byte);
        }
        if (halves > 1) {   // the pair's second block reads the shared byte after this block has written it
            if (GROUP > 32) __syncthreads(); else __syncwarp();
        }
        }
    }
}

// --------------------------------------------------------------------------- vmean only
// vmean[b] = beta2*vmean[b] + (1-beta2)*mean(g[b,:]^2) (reference: automatic_vmean_kernel.cu:12-51).
// One warp per block, fp32 accumulation.
template <typename S>
__global__ void __launch_bounds__(kThreads) vmean_kernel(void* __restrict__ vmean, int v_dtype, const S* __restrict__ g,
                                                         long long num_blocks, long long period, float beta2) {
    const int lane = threadIdx.x & 31;
    const long long warp_global = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
    const long long warp_stride = static_cast<long long>(gridDim.x) * kWarps;
    const bool vec = (sizeof(S) == 2) && (period % 8 == 0) && ((reinterpret_cast<uintptr_t>(g) & 15u) == 0);
    for (long long b = warp_global; b < num_blocks; b += warp_stride) {
        const S* gb = g + b * period;
        float sum = 0.0f;
        if (vec) {
            const uint4* g4 = reinterpret_cast<const uint4*>(gb);
            for (long long c = lane; c < period / 8; c += 32) {
                const uint4 raw = g4[c];
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const S* h = reinterpret_cast<const S*>(&w[i]);
                    const float a = ScalarIO<S>::load(h), c2 = ScalarIO<S>::load(h + 1);
                    sum = fmaf(a, a, sum);
                    sum = fmaf(c2, c2, sum);
                }
            }
        } else {
            for (long long i = lane; i < period; i += 32) {
                const float a = ScalarIO<S>::load(gb + i);
                sum = fmaf(a, a, sum);
            }
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            const float mean_sq = sum / static_cast<float>(period);
            const float prev = load_state(vmean, b, v_dtype);
            store_state(vmean, b, v_dtype, fmaf(beta2, prev, (1.0f - beta2) * mean_sq));
        }
    }
}

// --------------------------------------------------------------------------- multicast sum
// dst[i] = round(scale * sum over the ranks of src[i]), the sum formed by the switch: the gradient the
// staged kernel sees when it reads through the multicast mapping, written out for checks.
template <typename S>
__global__ void __launch_bounds__(kThreads) multicast_sum_kernel(void* __restrict__ dst, const void* __restrict__ src_mc,
                                                                 long long chunks, float scale) {
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (long long c = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; c < chunks; c += stride) {
        Chunk<S> v;
        v.load_sum(src_mc, c);
        float f[8];
        v.unpack(f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= scale;
        v.pack(f);
        v.store(dst, c);
    }
}

// --------------------------------------------------------------------------- GefenMuon apply
// p <- round(p * wd_mul) ; p <- round(p + alpha * u)   (reference: gefen_muon.py:326-329, torch's mul_ and
// add_(update, alpha=-adjusted_lr): each rounds to the parameter dtype), one pass over p and u instead of
// two kernels, and - for ZeRO-1 ranks whose parameter buffers are mapped into each other - the updated
// parameters also stored to the peers' copies (the all-gather).
template <typename S>
__global__ void __launch_bounds__(kThreads) muon_apply_kernel(S* __restrict__ p, const S* __restrict__ u, long long numel,
                                                              float wd_mul, bool decay, float alpha, bool vec,
                                                              const __grid_constant__ StepLaunch L) {
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    const long long tid = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    const long long chunks = vec ? numel >> 3 : 0;
    for (long long c = tid; c < chunks; c += stride) {
        Chunk<S> pr, ur;
        pr.load(p, c);
        ur.load(u, c);
        float pv[8], uv[8];
        pr.unpack(pv);
        ur.unpack(uv);
        if (decay) {
#pragma unroll
            for (int i = 0; i < 8; ++i) pv[i] *= wd_mul;
            pr.pack(pv);
            pr.unpack(pv);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) pv[i] = fmaf(alpha, uv[i], pv[i]);
        pr.pack(pv);
        pr.store(p, c);
        for (int r = 0; r < L.n_peers; ++r) pr.store(peer_ptr(p, L.peer_delta[r]), c);
    }
    for (long long i = chunks * 8 + tid; i < numel; i += stride) {
        float pv = ScalarIO<S>::load(p + i);
        if (decay) pv = ScalarIO<S>::round(pv * wd_mul);
        pv = fmaf(alpha, ScalarIO<S>::load(u + i), pv);
        ScalarIO<S>::store(p + i, pv);
        for (int r = 0; r < L.n_peers; ++r) ScalarIO<S>::store(peer_ptr(p + i, L.peer_delta[r]), pv);
    }
}

// --------------------------------------------------------------------------- host dispatch
static int grid_for(long long groups_needed, int groups_per_cta, int ctas_per_sm) {
    long long ctas = (groups_needed + groups_per_cta - 1) / groups_per_cta;
    const long long cap = static_cast<long long>(sm_count()) * ctas_per_sm;
    if (ctas > cap) ctas = cap;
    if (ctas < 1) ctas = 1;
    return static_cast<int>(ctas);
}

constexpr int kFastMaxPeriod = 8192;
constexpr int kStaticSmemSlack = 256;   // static __shared__ of the kernels (counted against the per-CTA limit)
constexpr int kCtaReservedSmem = 1024;  // what the hardware sets aside per resident CTA (not part of the limit)

// Per-device launch configuration (cudaFuncSetAttribute) is done once per kernel and device, under
// this lock; device ordinals beyond the table are refused with a clear error.
constexpr int kMaxDevices = 64;
static std::mutex g_config_mutex;
static int current_device(int* dev) {
    GEFEN_CHECK_CUDA(cudaGetDevice(dev));
    GEFEN_CHECK_ARG(*dev >= 0 && *dev < kMaxDevices, "Unsupported device ordinal %d (at most %d devices).", *dev, kMaxDevices);
    return GEFEN_B200_OK;
}

static int env_int(const char* name) {
    const char* e = getenv(name);
    const int v = e != nullptr ? atoi(e) : 0;
    return v < 0 ? 0 : v;
}
// GEFEN_B200_STEP_WARPS=n caps the warps per CTA of the staged kernel (for measurements; read once).
static int warps_override() {
    static const int cached = env_int("GEFEN_B200_STEP_WARPS");
    return cached;
}

// Iteration limit of the step kernels' wait for their staged tables. gefen_b200_debug_set_stage_spin_limit
// lowers it so that a test can watch the time-out path (status word, kernel returns) without a fault.
constexpr unsigned int kDefaultStageSpinLimit = 4000000u;
static unsigned int g_stage_spin_limit = kDefaultStageSpinLimit;

template <typename S, int GSRC, bool FULL>
static int launch_vec_variant(StepLaunch L, const gefen_b200_step_tensor_t& single, long long max_period,
                              cudaStream_t stream) {
    static bool configured[kMaxDevices];
    auto kernel = step_vec_kernel<S, GSRC, FULL>;
    {
        int dev = 0;
        const int rc = current_device(&dev);
        if (rc != GEFEN_B200_OK) return rc;
        std::lock_guard<std::mutex> lock(g_config_mutex);
        if (!configured[dev]) {
            GEFEN_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem - kStaticSmemSlack));
            configured[dev] = true;
        }
    }
    // a warp stages one unit: one long block, or the 32 / lanes shorter blocks that share the warp
    // (max_period: the largest unit of the launch, see unit_elements)
    const long long stage_bytes = (max_period > 256 ? max_period : 256) * 4;
    int max_warps = vec_max_threads<S, GSRC, FULL>() / 32;
    if (warps_override() > 0 && warps_override() < max_warps) max_warps = warps_override();
    int warps = static_cast<int>((kMaxSmem - kStaticSmemSlack - kSmemWs - kSmemRep) / stage_bytes);
    if (warps > max_warps) warps = max_warps;
    if (warps < 1) return fail(GEFEN_B200_EINVAL, "internal: period %lld too large for the staged path", max_period);
    if (L.total_blocks < warps) warps = static_cast<int>(L.total_blocks);
    const int smem = kSmemWs + kSmemRep + static_cast<int>(stage_bytes) * warps;
    int ctas_per_sm = (kMaxSmem + kCtaReservedSmem) / (smem + kStaticSmemSlack + kCtaReservedSmem);
    if (ctas_per_sm > 2) ctas_per_sm = 2;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    L.stage_floats = static_cast<int>(stage_bytes / 4);
    const int grid = grid_for(L.total_blocks, warps, ctas_per_sm);
    kernel<<<grid, warps * 32, smem, stream>>>(L, single);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

template <typename S, bool FULL>
static int launch_vec(StepLaunch L, const gefen_b200_step_tensor_t& single, long long max_period, cudaStream_t stream) {
    if (L.grad_mc_delta != 0) return launch_vec_variant<S, 2, FULL>(L, single, max_period, stream);
    if (L.n_grad_srcs > 0) return launch_vec_variant<S, 1, FULL>(L, single, max_period, stream);
    return launch_vec_variant<S, 0, FULL>(L, single, max_period, stream);
}

template <typename S>
static int launch_generic(bool cta_per_block, const StepLaunch& L, const gefen_b200_step_tensor_t& single,
                          cudaStream_t stream) {
    constexpr int smem = kSmemWs;
    static bool configured[kMaxDevices];
    {
        int dev = 0;
        const int rc = current_device(&dev);
        if (rc != GEFEN_B200_OK) return rc;
        std::lock_guard<std::mutex> lock(g_config_mutex);
        if (!configured[dev]) {
            GEFEN_CHECK_CUDA(cudaFuncSetAttribute(step_generic_kernel<S, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            GEFEN_CHECK_CUDA(cudaFuncSetAttribute(step_generic_kernel<S, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            configured[dev] = true;
        }
    }
    if (cta_per_block) {
        const int grid = grid_for(L.total_blocks, 1, 3);
        step_generic_kernel<S, 256><<<grid, kThreads, smem, stream>>>(L, single);
    } else {
        const int grid = grid_for(L.total_blocks, kWarps, 3);
        step_generic_kernel<S, 32><<<grid, kThreads, smem, stream>>>(L, single);
    }
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

// Class of a tensor: 1 = vectorised staged path with whole-warp blocks, 2 = the same path with several blocks
// per warp pass (blocks of up to 1024 elements), 0 = generic warp per block, -1 = generic CTA per block.
static int tensor_class(const gefen_b200_step_tensor_t& t, int dtype) {
    const bool vec_dtype = dtype == GEFEN_B200_F32 || dtype == GEFEN_B200_BF16 || dtype == GEFEN_B200_F16;
    const bool period1 = (t.flags & GEFEN_B200_STEP_PERIOD1) != 0;
    const bool packed = (t.flags & GEFEN_B200_STEP_PACKED) != 0;
    if (vec_dtype && !period1 && !packed && t.period % 8 == 0 && t.period <= kFastMaxPeriod && aligned16(t.g) && aligned16(t.p) &&
        (reinterpret_cast<uintptr_t>(t.codes) & 7u) == 0) {
        return lanes_per_block(t.period) == 32 ? 1 : 2;
    }
    return t.period > 2048 ? -1 : 0;
}
// Units of a tensor in its launch's index space: passes of a warp on the staged path, blocks elsewhere.
// (4-bit codes with an odd period: a pair of blocks is one unit, see step_generic_kernel)
static long long class_units(const gefen_b200_step_tensor_t& t, int cls) {
    if (cls >= 1) return vec_units(t.num_blocks, t.period);
    const bool paired = (t.flags & GEFEN_B200_STEP_PACKED) != 0 && (t.period & 1) != 0;
    return paired ? (t.num_blocks + 1) / 2 : t.num_blocks;
}

static int launch_class(int cls, int dtype, const StepLaunch& L, const gefen_b200_step_tensor_t& single,
                        long long max_period, cudaStream_t stream) {
    if (cls == 1) {
        if (dtype == GEFEN_B200_BF16) return launch_vec<__nv_bfloat16, true>(L, single, max_period, stream);
        if (dtype == GEFEN_B200_F16) return launch_vec<__half, true>(L, single, max_period, stream);
        return launch_vec<float, true>(L, single, max_period, stream);
    }
    if (cls == 2) {
        if (dtype == GEFEN_B200_BF16) return launch_vec<__nv_bfloat16, false>(L, single, max_period, stream);
        if (dtype == GEFEN_B200_F16) return launch_vec<__half, false>(L, single, max_period, stream);
        return launch_vec<float, false>(L, single, max_period, stream);
    }
    const bool cta = cls < 0;
    switch (dtype) {
        case GEFEN_B200_F32: return launch_generic<float>(cta, L, single, stream);
        case GEFEN_B200_F16: return launch_generic<__half>(cta, L, single, stream);
        case GEFEN_B200_BF16: return launch_generic<__nv_bfloat16>(cta, L, single, stream);
        case GEFEN_B200_F64: return launch_generic<double>(cta, L, single, stream);
    }
    return fail(GEFEN_B200_EINVAL, "Unsupported parameter dtype tag %d.", dtype);
}

static int check_common(const void* g, uint8_t* codes, void* mag, int mag_dtype, int param_dtype,
                        int packed_indices, long long num_blocks, long long period) {
    GEFEN_CHECK_ARG(g != nullptr && codes != nullptr && mag != nullptr, "Expected non-null tensor pointers.");
    GEFEN_CHECK_ARG(is_float_dtype(param_dtype), "Unsupported parameter/gradient dtype tag %d.", param_dtype);
    GEFEN_CHECK_ARG(is_state_dtype(mag_dtype),
                    "Expected m_magnitude to have dtype float32, float16, or bfloat16.");
    GEFEN_CHECK_ARG(num_blocks >= 0 && period > 0, "Expected a positive period and a non-negative block count.");
    GEFEN_CHECK_ARG(period <= 0x7FFFFFFFLL, "Period %lld is too large.", period);
    (void)packed_indices;   // any period: with an odd one, pairs of blocks share a byte and are stepped together
    return GEFEN_B200_OK;
}

static int run_single(gefen_b200_step_tensor_t& t, int param_dtype, const float* stepsize, const float* codebook,
                      int codebook_size, const void* codebook_ws, cudaStream_t stream) {
    if (t.num_blocks == 0) return GEFEN_B200_OK;
    const void* ws = nullptr;
    const int rc = resolve_codebook_ws(codebook, codebook_size, codebook_ws, stream, &ws);
    if (rc != GEFEN_B200_OK) return rc;
    t.first_block = 0;
    StepLaunch L;
    L.table = nullptr;
    L.n_tensors = 1;
    L.stage_floats = 0;
    const int cls = tensor_class(t, param_dtype);
    L.total_blocks = class_units(t, cls);
    L.ws = static_cast<const unsigned char*>(ws);
    L.stepsize = stepsize;
    L.n_peers = 0;
    L.n_grad_srcs = 0;
    L.grad_scale = 1.0f;
    L.grad_mc_delta = 0;
    L.param_mc_delta = 0;
    L.spin_limit = g_stage_spin_limit;
    return launch_class(cls, param_dtype, L, t, cls >= 1 ? unit_elements(t.period) : t.period, stream);
}

}  // namespace gefen

using namespace gefen;

extern "C" {

int gefen_b200_automatic_vmean_update(void* vmean, int vmean_dtype, const void* grad_view, int grad_dtype,
                                      int64_t num_blocks, int64_t period, double beta2, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(vmean != nullptr && grad_view != nullptr, "Expected non-null vmean and grad_view.");
    GEFEN_CHECK_ARG(is_state_dtype(vmean_dtype), "Expected vmean to have dtype float32, float16, or bfloat16.");
    GEFEN_CHECK_ARG(is_float_dtype(grad_dtype), "Unsupported gradient dtype tag %d.", grad_dtype);
    GEFEN_CHECK_ARG(period > 0, "Expected grad_view to have a positive period.");
    GEFEN_CHECK_ARG(num_blocks >= 0, "Expected a non-negative block count.");
    if (num_blocks == 0) return GEFEN_B200_OK;
    const int grid = grid_for(num_blocks, kWarps, 8);
    const float b2 = static_cast<float>(beta2);
    switch (grad_dtype) {
        case GEFEN_B200_F32:
            vmean_kernel<float><<<grid, kThreads, 0, stream>>>(vmean, vmean_dtype, static_cast<const float*>(grad_view), num_blocks, period, b2);
            break;
        case GEFEN_B200_F16:
            vmean_kernel<__half><<<grid, kThreads, 0, stream>>>(vmean, vmean_dtype, static_cast<const __half*>(grad_view), num_blocks, period, b2);
            break;
        case GEFEN_B200_BF16:
            vmean_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(vmean, vmean_dtype, static_cast<const __nv_bfloat16*>(grad_view), num_blocks, period, b2);
            break;
        default:
            vmean_kernel<double><<<grid, kThreads, 0, stream>>>(vmean, vmean_dtype, static_cast<const double*>(grad_view), num_blocks, period, b2);
            break;
    }
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_automatic_gefen_fused_update_from_vmean(
    void* p, const void* grad_view, int param_dtype, uint8_t* m_sign, void* m_magnitude, int magnitude_dtype,
    const void* vmean, int vmean_dtype, const float* codebook, int codebook_size, const void* codebook_ws,
    int packed_indices, int64_t num_blocks, int64_t period, double beta1, double lr, double bias_correction_1,
    double bias_correction_2, double eps, void* stream) {
    int rc = check_common(grad_view, m_sign, m_magnitude, magnitude_dtype, param_dtype, packed_indices, num_blocks, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(p != nullptr && vmean != nullptr, "Expected non-null p and vmean.");
    GEFEN_CHECK_ARG(is_state_dtype(vmean_dtype), "Expected vmean to have dtype float32, float16, or bfloat16.");
    GEFEN_CHECK_ARG(bias_correction_1 > 0.0, "Expected bias_correction_1 to be positive.");
    GEFEN_CHECK_ARG(bias_correction_2 > 0.0, "Expected bias_correction_2 to be positive.");
    GEFEN_CHECK_ARG(eps >= 0.0, "Expected eps to be non-negative.");
    gefen_b200_step_tensor_t t = {};
    t.p = p; t.g = grad_view; t.codes = m_sign; t.mag = m_magnitude; t.v = const_cast<void*>(vmean);
    t.num_blocks = num_blocks; t.period = period;
    t.beta1 = static_cast<float>(beta1); t.lr = static_cast<float>(lr);
    t.bc1 = static_cast<float>(bias_correction_1); t.bc2 = static_cast<float>(bias_correction_2);
    t.eps = static_cast<float>(eps); t.wd_mul = 1.0f; t.flags = packed_indices ? GEFEN_B200_STEP_PACKED : 0u;
    t.mag_dtype = magnitude_dtype; t.v_dtype = vmean_dtype;
    return run_single(t, param_dtype, nullptr, codebook, codebook_size, codebook_ws, static_cast<cudaStream_t>(stream));
}

int gefen_b200_automatic_gefen_fused_update(
    void* p, const void* grad_view, int param_dtype, uint8_t* m_sign, void* m_magnitude, int magnitude_dtype,
    const float* stepsize, const float* codebook, int codebook_size, const void* codebook_ws, int packed_indices,
    int64_t num_blocks, int64_t period, double beta1, double lr, void* stream) {
    int rc = check_common(grad_view, m_sign, m_magnitude, magnitude_dtype, param_dtype, packed_indices, num_blocks, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(p != nullptr && stepsize != nullptr, "Expected non-null p and stepsize.");
    gefen_b200_step_tensor_t t = {};
    t.p = p; t.g = grad_view; t.codes = m_sign; t.mag = m_magnitude; t.v = nullptr;
    t.num_blocks = num_blocks; t.period = period;
    t.beta1 = static_cast<float>(beta1); t.lr = static_cast<float>(lr);
    t.bc1 = 1.0f; t.bc2 = 1.0f; t.eps = 0.0f; t.wd_mul = 1.0f; t.flags = packed_indices ? GEFEN_B200_STEP_PACKED : 0u;
    t.mag_dtype = magnitude_dtype; t.v_dtype = GEFEN_B200_F32;
    return run_single(t, param_dtype, stepsize, codebook, codebook_size, codebook_ws, static_cast<cudaStream_t>(stream));
}

int gefen_b200_automatic_gefen_period1_update(
    void* p, const void* grad_flat, int param_dtype, uint8_t* m_sign, void* m_magnitude, int magnitude_dtype,
    void* vmean, int vmean_dtype, const float* codebook, int codebook_size, const void* codebook_ws,
    int64_t total_numel, int64_t period_one_divisor, double beta1, double beta2, double lr,
    double bias_correction_1, double bias_correction_2, double eps, void* stream) {
    GEFEN_CHECK_ARG(period_one_divisor > 0, "Expected period_one_divisor to be positive.");
    GEFEN_CHECK_ARG(total_numel >= 0 && total_numel % period_one_divisor == 0,
                    "Expected period_one_divisor to divide total_numel.");
    const int64_t num_blocks = total_numel / period_one_divisor;
    int rc = check_common(grad_flat, m_sign, m_magnitude, magnitude_dtype, param_dtype, 0, num_blocks, period_one_divisor);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(p != nullptr && vmean != nullptr, "Expected non-null p and vmean.");
    GEFEN_CHECK_ARG(is_state_dtype(vmean_dtype), "Expected vmean to have dtype float32, float16, or bfloat16.");
    GEFEN_CHECK_ARG(bias_correction_1 > 0.0, "Expected bias_correction_1 to be positive.");
    GEFEN_CHECK_ARG(bias_correction_2 > 0.0, "Expected bias_correction_2 to be positive.");
    GEFEN_CHECK_ARG(eps >= 0.0, "Expected eps to be non-negative.");
    gefen_b200_step_tensor_t t = {};
    t.p = p; t.g = grad_flat; t.codes = m_sign; t.mag = m_magnitude; t.v = vmean;
    t.num_blocks = num_blocks; t.period = period_one_divisor;
    t.beta1 = static_cast<float>(beta1); t.beta2 = static_cast<float>(beta2); t.lr = static_cast<float>(lr);
    t.bc1 = static_cast<float>(bias_correction_1); t.bc2 = static_cast<float>(bias_correction_2);
    t.eps = static_cast<float>(eps); t.wd_mul = 1.0f; t.flags = GEFEN_B200_STEP_PERIOD1;
    t.mag_dtype = magnitude_dtype; t.v_dtype = vmean_dtype;
    return run_single(t, param_dtype, nullptr, codebook, codebook_size, codebook_ws, static_cast<cudaStream_t>(stream));
}

int gefen_b200_automatic_gefen_muon_momentum(
    const void* grad_view, int grad_dtype, uint8_t* m_sign, void* m_magnitude, int magnitude_dtype,
    const float* codebook, int codebook_size, const void* codebook_ws, void* momentum_update, int packed_indices,
    int64_t num_blocks, int64_t period, double beta1, void* stream) {
    int rc = check_common(grad_view, m_sign, m_magnitude, magnitude_dtype, grad_dtype, packed_indices, num_blocks, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(momentum_update != nullptr, "Expected a non-null momentum_update.");
    gefen_b200_step_tensor_t t = {};
    t.p = momentum_update; t.g = grad_view; t.codes = m_sign; t.mag = m_magnitude; t.v = nullptr;
    t.num_blocks = num_blocks; t.period = period;
    t.beta1 = static_cast<float>(beta1); t.lr = 0.0f; t.bc1 = 1.0f; t.bc2 = 1.0f; t.wd_mul = 1.0f;
    t.flags = GEFEN_B200_STEP_MUON | (packed_indices ? GEFEN_B200_STEP_PACKED : 0u);
    t.mag_dtype = magnitude_dtype; t.v_dtype = GEFEN_B200_F32;
    return run_single(t, grad_dtype, nullptr, codebook, codebook_size, codebook_ws, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// The same step for callers that must not allocate device memory.
//
// Who needs it: code that runs after all device memory has been handed to another owner (a
// framework's caching allocator holding the whole card, a fixed memory plan of an inference or
// training runtime), and code on paths where an allocation is simply not allowed to happen
// (latency-critical loops, library hooks that promise not to touch the allocator). The regular
// entry point, when it is given no codebook workspace, allocates one per device with cudaMalloc on
// first use; this one keeps that workspace in a fixed array inside the library image instead.
//
// The array costs GEFEN_B200_CODEBOOK_WS_BYTES (34 848 bytes) of device memory on every GPU that
// loads the library, until the process exits. It is sized for the largest codebook the kernels
// accept, 256 entries; a larger codebook is rejected. Every call rewrites the whole array from the
// codebook it is given, on the caller's stream, before the step kernel reads it, so nothing has to
// be cleared and consecutive calls on one stream are independent; calls that may run concurrently
// on the same GPU (different streams) share the array and would race on it.
static __device__ __align__(256) unsigned char g_static_codebook_ws[GEFEN_B200_CODEBOOK_WS_BYTES];

// In host code the array's name is only a handle: the device address comes from the runtime, once
// per device, with that device current.
static std::mutex g_static_ws_mutex;
static void* g_static_ws_address[kMaxDevices];

static int static_codebook_ws(void** out) {
    int dev = 0;
    const int rc_dev = current_device(&dev);
    if (rc_dev != GEFEN_B200_OK) return rc_dev;
    std::lock_guard<std::mutex> lock(g_static_ws_mutex);
    if (g_static_ws_address[dev] == nullptr) {
        void* address = nullptr;
        GEFEN_CHECK_CUDA(cudaGetSymbolAddress(&address, g_static_codebook_ws));
        g_static_ws_address[dev] = address;
    }
    *out = g_static_ws_address[dev];
    return GEFEN_B200_OK;
}

int gefen_b200_automatic_gefen_fused_update_from_vmean_static_ws(
    void* p, const void* grad_view, int param_dtype, uint8_t* m_sign, void* m_magnitude, int magnitude_dtype,
    const void* vmean, int vmean_dtype, const float* codebook, int codebook_size, int packed_indices,
    int64_t num_blocks, int64_t period, double beta1, double lr, double bias_correction_1,
    double bias_correction_2, double eps, void* stream) {
    GEFEN_CHECK_ARG(codebook != nullptr, "Expected a codebook pointer.");
    GEFEN_CHECK_ARG(codebook_size >= 1 && codebook_size <= kMaxCodebook,
                    "The built-in workspace holds tables for at most 256 codebook entries, got %d.", codebook_size);
    // every argument is checked before the shared array is touched: a refused call leaves it as it was
    int rc = check_common(grad_view, m_sign, m_magnitude, magnitude_dtype, param_dtype, packed_indices, num_blocks, period);
    if (rc != GEFEN_B200_OK) return rc;
    GEFEN_CHECK_ARG(p != nullptr && vmean != nullptr, "Expected non-null p and vmean.");
    GEFEN_CHECK_ARG(is_state_dtype(vmean_dtype), "Expected vmean to have dtype float32, float16, or bfloat16.");
    GEFEN_CHECK_ARG(bias_correction_1 > 0.0, "Expected bias_correction_1 to be positive.");
    GEFEN_CHECK_ARG(bias_correction_2 > 0.0, "Expected bias_correction_2 to be positive.");
    GEFEN_CHECK_ARG(eps >= 0.0, "Expected eps to be non-negative.");
    if (num_blocks == 0) return GEFEN_B200_OK;
    void* ws = nullptr;
    rc = static_codebook_ws(&ws);
    if (rc != GEFEN_B200_OK) return rc;
    rc = launch_codebook_prepare(codebook, codebook_size, ws, static_cast<cudaStream_t>(stream));
    if (rc != GEFEN_B200_OK) return rc;
    return gefen_b200_automatic_gefen_fused_update_from_vmean(
        p, grad_view, param_dtype, m_sign, m_magnitude, magnitude_dtype, vmean, vmean_dtype, codebook, codebook_size,
        ws, packed_indices, num_blocks, period, beta1, lr, bias_correction_1, bias_correction_2, eps, stream);
}

int gefen_b200_step_tensor_size(void) { return static_cast<int>(sizeof(gefen_b200_step_tensor_t)); }

int gefen_b200_step_tensor_class(const gefen_b200_step_tensor_t* host_entry, int param_dtype) {
    if (host_entry == nullptr) return -2;
    return tensor_class(*host_entry, param_dtype);
}

int gefen_b200_multicast_sum(void* dst, const void* src_multicast, int dtype, int64_t numel, double scale, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(dst != nullptr && src_multicast != nullptr, "Expected non-null buffers.");
    GEFEN_CHECK_ARG(dtype == GEFEN_B200_F32 || dtype == GEFEN_B200_F16 || dtype == GEFEN_B200_BF16,
                    "The multicast sum supports fp32, fp16 and bf16.");
    GEFEN_CHECK_ARG(numel >= 0 && numel % 8 == 0 && aligned16(dst) && aligned16(src_multicast),
                    "Expected 16-byte aligned buffers and a multiple of 8 elements.");
    if (numel == 0) return GEFEN_B200_OK;
    const long long chunks = numel / 8;
    const int grid = grid_for(chunks, kThreads, 4);
    const float sc = static_cast<float>(scale);
    if (dtype == GEFEN_B200_BF16) multicast_sum_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(dst, src_multicast, chunks, sc);
    else if (dtype == GEFEN_B200_F16) multicast_sum_kernel<__half><<<grid, kThreads, 0, stream>>>(dst, src_multicast, chunks, sc);
    else multicast_sum_kernel<float><<<grid, kThreads, 0, stream>>>(dst, src_multicast, chunks, sc);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_muon_apply(void* p, const void* update, int dtype, int64_t numel, double wd_mul, double alpha,
                          const int64_t* peer_deltas, int n_peers, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(p != nullptr && update != nullptr, "Expected non-null p and update.");
    GEFEN_CHECK_ARG(dtype == GEFEN_B200_F32 || dtype == GEFEN_B200_F16 || dtype == GEFEN_B200_BF16,
                    "The GefenMuon apply supports fp32, fp16 and bf16 parameters.");
    GEFEN_CHECK_ARG(numel >= 0, "Expected a non-negative element count.");
    GEFEN_CHECK_ARG(n_peers >= 0 && n_peers <= GEFEN_B200_MAX_PEERS, "Expected between 0 and %d peers, got %d.",
                    GEFEN_B200_MAX_PEERS, n_peers);
    GEFEN_CHECK_ARG(n_peers == 0 || peer_deltas != nullptr, "Expected peer offsets for %d peers.", n_peers);
    for (int r = 0; r < n_peers; ++r)
        GEFEN_CHECK_ARG(peer_deltas[r] % 16 == 0, "Peer offset %d is not a multiple of 16 bytes.", r);
    if (numel == 0) return GEFEN_B200_OK;
    StepLaunch L = {};
    L.n_peers = n_peers;
    for (int r = 0; r < n_peers; ++r) L.peer_delta[r] = peer_deltas[r];
    const bool vec = aligned16(p) && aligned16(update);
    const bool decay = wd_mul != 1.0;
    const int grid = grid_for((numel + 7) / 8, kThreads, 8);
    const float wm = static_cast<float>(wd_mul), a = static_cast<float>(alpha);
    if (dtype == GEFEN_B200_BF16)
        muon_apply_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(update), numel, wm, decay, a, vec, L);
    else if (dtype == GEFEN_B200_F16)
        muon_apply_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<__half*>(p), static_cast<const __half*>(update), numel, wm, decay, a, vec, L);
    else
        muon_apply_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<float*>(p), static_cast<const float*>(update), numel, wm, decay, a, vec, L);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

int gefen_b200_step_status(int* host_status, int clear) {
    GEFEN_CHECK_ARG(host_status != nullptr, "Expected a host pointer for the status.");
    int value = 0;
    GEFEN_CHECK_CUDA(cudaMemcpyFromSymbol(&value, g_step_status, sizeof(int)));   // synchronises the device
    if (value != 0 && clear) {
        const int zero = 0;
        GEFEN_CHECK_CUDA(cudaMemcpyToSymbol(g_step_status, &zero, sizeof(int)));
    }
    *host_status = value;
    return GEFEN_B200_OK;
}

int gefen_b200_debug_set_stage_spin_limit(int64_t limit) {
    g_stage_spin_limit = (limit < 0 || limit > 0xFFFFFFFFll) ? kDefaultStageSpinLimit : static_cast<unsigned int>(limit);
    return GEFEN_B200_OK;
}

int gefen_b200_multi_tensor_step(gefen_b200_step_tensor_t* host_table, void* device_table, int n_tensors,
                                 int param_dtype, const void* codebook_ws, void* stream_) {
    return gefen_b200_multi_tensor_step_peers(host_table, device_table, n_tensors, param_dtype, codebook_ws, nullptr, 0,
                                              nullptr, 0, 1.0, stream_);
}

int gefen_b200_multi_tensor_step_peers(gefen_b200_step_tensor_t* host_table, void* device_table, int n_tensors,
                                       int param_dtype, const void* codebook_ws, const int64_t* peer_deltas,
                                       int n_peers, const int64_t* grad_deltas, int n_grad_srcs, double grad_scale,
                                       void* stream_) {
    return gefen_b200_multi_tensor_step_multicast(host_table, device_table, n_tensors, param_dtype, codebook_ws, peer_deltas,
                                                  n_peers, grad_deltas, n_grad_srcs, grad_scale, 0, 0, stream_);
}

int gefen_b200_multi_tensor_step_multicast(gefen_b200_step_tensor_t* host_table, void* device_table, int n_tensors,
                                           int param_dtype, const void* codebook_ws, const int64_t* peer_deltas,
                                           int n_peers, const int64_t* grad_deltas, int n_grad_srcs, double grad_scale,
                                           int64_t param_multicast_delta, int64_t grad_multicast_delta, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(param_multicast_delta % 16 == 0 && grad_multicast_delta % 16 == 0,
                    "Multicast offsets must be multiples of 16 bytes.");
    GEFEN_CHECK_ARG(grad_multicast_delta == 0 || n_grad_srcs > 0,
                    "Summing gradients through the multicast mapping also needs the per-rank gradient offsets "
                    "(the kernels for short or odd blocks read the ranks' buffers directly).");
    GEFEN_CHECK_ARG(param_multicast_delta == 0 || n_peers > 0,
                    "Storing parameters through the multicast mapping also needs the per-rank parameter offsets.");
    GEFEN_CHECK_ARG((param_multicast_delta == 0 && grad_multicast_delta == 0) || param_dtype != GEFEN_B200_F64,
                    "The multicast paths support fp32, fp16 and bf16.");
    GEFEN_CHECK_ARG(n_grad_srcs >= 0 && n_grad_srcs <= GEFEN_B200_MAX_PEERS + 1,
                    "Expected between 0 and %d gradient buffers, got %d.", GEFEN_B200_MAX_PEERS + 1, n_grad_srcs);
    GEFEN_CHECK_ARG(n_grad_srcs == 0 || grad_deltas != nullptr, "Expected offsets for %d gradient buffers.", n_grad_srcs);
    for (int r = 0; r < n_grad_srcs; ++r)
        GEFEN_CHECK_ARG(grad_deltas[r] % 16 == 0, "Gradient buffer offset %d is not a multiple of 16 bytes.", r);
    GEFEN_CHECK_ARG(n_grad_srcs == 0 || param_dtype != GEFEN_B200_F64, "Gradient averaging supports fp32, fp16 and bf16.");
    GEFEN_CHECK_ARG(n_peers >= 0 && n_peers <= GEFEN_B200_MAX_PEERS, "Expected between 0 and %d peers, got %d.",
                    GEFEN_B200_MAX_PEERS, n_peers);
    GEFEN_CHECK_ARG(n_peers == 0 || peer_deltas != nullptr, "Expected peer offsets for %d peers.", n_peers);
    for (int r = 0; r < n_peers; ++r)
        GEFEN_CHECK_ARG(peer_deltas[r] % 16 == 0, "Peer offset %d is not a multiple of 16 bytes.", r);
    GEFEN_CHECK_ARG(n_tensors >= 0, "Expected a non-negative tensor count.");
    if (n_tensors == 0) return GEFEN_B200_OK;
    GEFEN_CHECK_ARG(host_table != nullptr && device_table != nullptr && codebook_ws != nullptr,
                    "Expected non-null tables and codebook workspace.");
    GEFEN_CHECK_ARG(aligned16(codebook_ws) && aligned16(device_table), "Expected 16-byte aligned workspace and table.");
    GEFEN_CHECK_ARG(is_float_dtype(param_dtype), "Unsupported parameter dtype tag %d.", param_dtype);
    // Tensors are launched in maximal runs of rows that share a kernel class (staged vector path,
    // generic warp, generic CTA); callers that keep equal classes adjacent get one launch per
    // class. Rows are never reordered.
    for (int i = 0; i < n_tensors; ++i) {
        gefen_b200_step_tensor_t& t = host_table[i];
        GEFEN_CHECK_ARG(t.g != nullptr && t.codes != nullptr && t.mag != nullptr && t.p != nullptr,
                        "Tensor %d of the table has a null pointer.", i);
        GEFEN_CHECK_ARG(t.period > 0 && t.period <= 0x7FFFFFFFLL && t.num_blocks >= 0,
                        "Tensor %d of the table has a bad period or block count.", i);
        GEFEN_CHECK_ARG(is_state_dtype(t.mag_dtype) && is_state_dtype(t.v_dtype),
                        "Tensor %d of the table has a bad state dtype.", i);
        GEFEN_CHECK_ARG((t.flags & GEFEN_B200_STEP_MUON) || t.v != nullptr, "Tensor %d has a null vmean.", i);
        GEFEN_CHECK_ARG(!(t.flags & GEFEN_B200_STEP_PACKED) || !(t.flags & GEFEN_B200_STEP_PERIOD1),
                        "Tensor %d: 4-bit codes are not defined for period-1 tensors.", i);
        GEFEN_CHECK_ARG(n_grad_srcs == 0 || !(t.flags & GEFEN_B200_STEP_MUON),
                        "Tensor %d: the momentum-only step does not average gradients over ranks.", i);
        t.reserved_[0] = tensor_class(t, param_dtype);
    }
    for (int begin = 0; begin < n_tensors;) {
        int end = begin;
        long long first = 0;
        while (end < n_tensors && host_table[end].reserved_[0] == host_table[begin].reserved_[0]) {
            host_table[end].first_block = first;   // in work units on the staged path, in blocks elsewhere
            first += class_units(host_table[end], host_table[end].reserved_[0]);
            ++end;
        }
        host_table[begin].reserved_[1] = end - begin;  // run length, read back below
        begin = end;
    }
    GEFEN_CHECK_CUDA(cudaMemcpyAsync(device_table, host_table, sizeof(gefen_b200_step_tensor_t) * n_tensors,
                                     cudaMemcpyHostToDevice, stream));
    for (int begin = 0; begin < n_tensors;) {
        const int run = host_table[begin].reserved_[1];
        const gefen_b200_step_tensor_t& last = host_table[begin + run - 1];
        const long long total = last.first_block + class_units(last, last.reserved_[0]);
        long long max_period = 0;   // largest staging need of a warp: the elements of one unit on the staged path
        for (int i = begin; i < begin + run; ++i) {
            const long long need = host_table[begin].reserved_[0] >= 1 ? unit_elements(host_table[i].period) : host_table[i].period;
            max_period = need > max_period ? need : max_period;
        }
        if (total > 0) {
            StepLaunch L;
            L.table = static_cast<const gefen_b200_step_tensor_t*>(device_table) + begin;
            L.n_tensors = run;
            L.stage_floats = 0;
            L.total_blocks = total;
            L.ws = static_cast<const unsigned char*>(codebook_ws);
            L.stepsize = nullptr;
            L.n_peers = n_peers;
            for (int r = 0; r < n_peers; ++r) L.peer_delta[r] = peer_deltas[r];
            L.n_grad_srcs = n_grad_srcs;
            L.grad_scale = static_cast<float>(grad_scale);
            for (int r = 0; r < n_grad_srcs; ++r) L.grad_delta[r] = grad_deltas[r];
            L.grad_mc_delta = grad_multicast_delta;
            L.param_mc_delta = param_multicast_delta;
            L.spin_limit = g_stage_spin_limit;
            const int rc = launch_class(host_table[begin].reserved_[0], param_dtype, L, host_table[begin], max_period, stream);
            if (rc != GEFEN_B200_OK) return rc;
        }
        begin += run;
    }
    return GEFEN_B200_OK;
}

}  // extern "C"
