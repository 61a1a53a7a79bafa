// bf16 GEMM on the 5th-generation tensor cores for GefenMuon's Newton-Schulz iteration
// (reference: gefen_muon.py:16-51, where the three products per iteration are torch.addmm / `@`,
// i.e. cuBLAS):
//
//     D[M,N] = alpha * A[M,K] * B[N,K]^T + beta * C[M,N]        (bf16 in/out, fp32 accumulation)
//
// and optionally Dt[N,M] = D^T in the same pass. Both operands are K-major (row-major with K
// contiguous), which covers every product of the iteration once X and X^T are both kept:
//     G  = X X^T               A = B = X
//     Bm = b*G + c*G*G         A = B = C = G      (G is symmetric, so G*G = G*G^T)
//     X' = a*X + Bm*X          A = Bm, B = X^T, C = X, Dt receives X'^T for the next iteration
//
// Structure (128 x BN output tiles, 6 warps; one tile per CTA, or - PERSIST - one CTA per SM that
// walks over tiles with two accumulator buffers in TMEM, so that the epilogue of a tile runs while
// the tensor cores already work on the next one):
//   warp 4  : TMA producer. cp.async.bulk.tensor 2-D loads of 128x64 (A) and BNx64 (B) bf16 boxes,
//             128-byte swizzle, into a STAGES-deep shared-memory ring, completion on mbarriers.
//   warp 5  : allocates TMEM and issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN, K=16)
//             from one thread; tcgen05.commit releases ring slots and finally signals the epilogue.
//   warps 0-3: epilogue. tcgen05.ld of the fp32 accumulators (lane = row), alpha/beta, bf16 stores.
// Every mbarrier wait is bounded: on a time-out the CTA raises a flag in global memory, the
// roles drain, TMEM is released and the kernel returns.
#include "common.cuh"

#include <stdio.h>
#include <stdlib.h>

#include <cuda.h>
#include <map>
#include <mutex>
#include <tuple>

namespace gefen {

constexpr int kBM = 128;
constexpr int kBK = 64;                 // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;
constexpr uint32_t kSpinLimit = 20000000u;

struct GemmArgs {
    const __nv_bfloat16* c;
    __nv_bfloat16* d;
    __nv_bfloat16* dt;
    int M, N, K;
    long long ldc, ldd, lddt;
    float alpha, beta;
    int n_tiles;     // PERSIST: number of tiles to compute (see tile_coords)
    int symmetric;   // the result is known to be symmetric (M == N): compute the tiles that touch the upper
                     // triangle only and write every element above the diagonal to its mirror position too
    int* status;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < kSpinLimit; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((it & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile whose rows are 128 bytes
// apart: 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100),
// layout type 2 (SWIZZLE_128B). The leading byte offset is not used by swizzled K-major layouts.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>(1) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

// MN-major operand ([K rows][MN contiguous] in memory), 128-byte swizzle: the tile is stored as
// groups of 64 MN-elements (one 128-byte row per K index, 8-row swizzle atoms 1024 bytes apart =
// stride byte offset); successive 64-element groups are `group_bytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_major_sw128(uint32_t smem_addr, uint32_t group_bytes) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>(group_bytes >> 4) << 16;
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;
    desc |= static_cast<uint64_t>(1) << 46;
    desc |= static_cast<uint64_t>(2) << 61;
    return desc;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Tile t of the persistent schedule: row-major over the tiles that are computed (all of them, or for
// a symmetric result those that reach the upper triangle: n0 + bn > m0).
__host__ __device__ inline bool tile_coords(int M, int N, int bn, int symmetric, long long t, int* m0, int* n0) {
    const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + bn - 1) / bn;
    if (!symmetric) {
        if (t >= static_cast<long long>(tiles_m) * tiles_n) return false;
        *m0 = static_cast<int>(t / tiles_n) * kBM;
        *n0 = static_cast<int>(t % tiles_n) * bn;
        return true;
    }
    for (int mi = 0; mi < tiles_m; ++mi) {
        const int row0 = mi * kBM;
        const int first = row0 >= bn ? (row0 - bn) / bn + 1 : 0;
        const int cnt = tiles_n - first;
        if (t < cnt) {
            *m0 = row0;
            *n0 = (first + static_cast<int>(t)) * bn;
            return true;
        }
        t -= cnt;
    }
    return false;
}

// B_MN = false: B is [N, K] row-major (K-major operand). B_MN = true: B is [K, N] row-major
// (MN-major operand), i.e. D = alpha * A * B + beta * C without any transposed copy of B.
// A_MN: likewise A given as [K, M] row-major (D = alpha * A^T * B ...), used for the Gram matrix of a
// tall matrix, Y^T Y, without transposing Y.
// Variants whose ring is at most 96 KB run two CTAs per SM: the epilogue of one overlaps the main
// loop of the other (each holds BN <= 256 of the 512 TMEM columns).
template <int BN, int STAGES, bool A_MN, bool B_MN, bool PERSIST>
__global__ void __launch_bounds__(kGemmThreads, (STAGES * (kBM + BN) * kBK * 2 <= 96 * 1024) ? 2 : 1) ns_gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                     const __grid_constant__ CUtensorMap map_b,
                                                                     const __grid_constant__ GemmArgs args) {
    constexpr int kABytes = kBM * kBK * 2;
    constexpr int kBBytes = BN * kBK * 2;
    constexpr int kStageBytes = kABytes + kBBytes;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    __shared__ uint64_t full_bar[STAGES];
    __shared__ uint64_t empty_bar[STAGES];
    __shared__ uint64_t acc_full[2];    // accumulator buffer complete (MMA -> epilogue)
    __shared__ uint64_t acc_empty[2];   // accumulator buffer drained (4 epilogue warps -> MMA); PERSIST only
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    constexpr int kTmemCols = PERSIST ? 2 * BN : BN;
    const int k_blocks = (args.K + kBK - 1) / kBK;
    if (!PERSIST && args.symmetric && static_cast<int>(blockIdx.x) * BN + BN <= static_cast<int>(blockIdx.y) * kBM)
        return;   // tile entirely below the diagonal: its mirror image computes it
    // li-th tile of this CTA
    auto my_tile = [&](int li, int* m0, int* n0) -> bool {
        if (!PERSIST) {
            *m0 = blockIdx.y * kBM;
            *n0 = blockIdx.x * BN;
            return li == 0;
        }
        const long long t = static_cast<long long>(blockIdx.x) + static_cast<long long>(li) * gridDim.x;
        return t < args.n_tiles && tile_coords(args.M, args.N, BN, args.symmetric, t, m0, n0);
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        fence_mbar_init();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;

    if (warp == 4) {
        // ---------------- producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            uint32_t it = 0;   // k-blocks issued so far, over all tiles: ring slot and phase
            bool ok = true;
            int m0, n0;
            for (int li = 0; ok && my_tile(li, &m0, &n0); ++li)
            for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t parity = ((it / STAGES) & 1) ^ 1;
                if (!wait_or_abort(&empty_bar[s], parity, &abort_flag)) { ok = false; break; }
                mbar_expect_tx(&full_bar[s], kStageBytes);
                unsigned char* a_dst = smem + s * kStageBytes;
                if (!A_MN) {
                    tma_load_2d(a_dst, &map_a, kb * kBK, m0, &full_bar[s]);
                } else {
#pragma unroll
                    for (int j = 0; j < kBM / 64; ++j)
                        tma_load_2d(a_dst + j * (kBK * 128), &map_a, m0 + 64 * j, kb * kBK, &full_bar[s]);
                }
                if (!B_MN) {
                    tma_load_2d(a_dst + kABytes, &map_b, kb * kBK, n0, &full_bar[s]);
                } else {
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)   // 64 K-rows x 64 N-columns per box
                        tma_load_2d(a_dst + kABytes + j * (kBK * 128), &map_b, n0 + 64 * j, kb * kBK, &full_bar[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        // ---------------- MMA issuer
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (A_MN ? (1u << 15) : 0u) | (B_MN ? (1u << 16) : 0u) |
                                       (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
            bool ok = true;
            uint32_t it = 0;
            int m0, n0;
            for (int li = 0; ok && my_tile(li, &m0, &n0); ++li) {
            const int buf = PERSIST ? (li & 1) : 0;
            const uint32_t tmem_acc = tmem_base + static_cast<uint32_t>(buf * BN);
            if (PERSIST) {   // the epilogue has drained this buffer (passes at once for the first two tiles)
                ok = wait_or_abort(&acc_empty[buf], ((li >> 1) & 1) ^ 1, &abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
                const int s = it % STAGES;
                const uint32_t parity = (it / STAGES) & 1;
                ok = wait_or_abort(&full_bar[s], parity, &abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(smem + s * kStageBytes);
                const uint64_t desc_a = A_MN ? umma_desc_mn_major_sw128(a_addr, kBK * 128) : umma_desc_k_major_sw128(a_addr);
                const uint64_t desc_b = B_MN ? umma_desc_mn_major_sw128(a_addr + kABytes, kBK * 128)
                                             : umma_desc_k_major_sw128(a_addr + kABytes);
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) {
                    // K-major: 16 bf16 along K = 32 bytes inside the swizzle row (+2 in the address field);
                    // MN-major: 16 K-rows of 128 bytes = 2048 bytes (+128)
                    umma_bf16(tmem_acc, desc_a + (A_MN ? 128 : 2) * k, desc_b + (B_MN ? 128 : 2) * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);   // the slot is free once these MMAs have read it
            }
            umma_commit(&acc_full[buf]);      // accumulators complete (or abandoned)
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warp w owns TMEM lanes (rows) 32w .. 32w+31
        int m0, n0;
        for (int li = 0; my_tile(li, &m0, &n0); ++li) {
        const int buf = PERSIST ? (li & 1) : 0;
        const int row = m0 + warp * 32 + lane;
        const bool row_ok = row < args.M;
        // C does not depend on the accumulators: the first chunk's row segment is fetched while the main
        // loop runs, and chunk j+1's while chunk j is converted and stored.
        const bool use_c = row_ok && args.beta != 0.0f;
        const __nv_bfloat16* crow_base = use_c ? args.c + static_cast<long long>(row) * args.ldc : nullptr;
        const bool c_vec = use_c && ((reinterpret_cast<uintptr_t>(crow_base) & 15u) == 0) && (args.ldc % 8 == 0) && (n0 % 8 == 0);
        uint4 cnext[4];
        auto fetch_c = [&](int j) {
            const int col0 = n0 + j * 32;
            if (c_vec && col0 + 32 <= args.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) cnext[q] = reinterpret_cast<const uint4*>(crow_base + col0)[q];
            }
        };
        fetch_c(0);
        const bool ok = wait_or_abort(&acc_full[buf], PERSIST ? ((li >> 1) & 1) : 0, &abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!ok || abort_flag) break;
        {
#pragma unroll 2
            for (int j = 0; j < BN / 32; ++j) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(buf * BN + j * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                      "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                      "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                uint4 ccur[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) ccur[q] = cnext[q];
                if (j + 1 < BN / 32) fetch_c(j + 1);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int col0 = n0 + j * 32;
                if (col0 >= args.N) continue;
                const bool full_cols = col0 + 32 <= args.N;
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = args.alpha * __uint_as_float(r[i]);
                if (use_c) {
                    const __nv_bfloat16* crow = crow_base + col0;
                    if (full_cols && c_vec) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 raw = ccur[q];
                            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                v[q * 8 + 2 * e] = fmaf(args.beta, __uint_as_float(w[e] << 16), v[q * 8 + 2 * e]);
                                v[q * 8 + 2 * e + 1] = fmaf(args.beta, __uint_as_float(w[e] & 0xFFFF0000u), v[q * 8 + 2 * e + 1]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < args.N) v[i] = fmaf(args.beta, __bfloat162float(crow[i]), v[i]);
                    }
                }
                if (row_ok) {
                    __nv_bfloat16* drow = args.d + static_cast<long long>(row) * args.ldd + col0;
                    if (args.symmetric && col0 < row) {
                        // chunk crosses or lies left of the diagonal: only the elements with column >= row
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < args.N && col0 + i >= row) drow[i] = __float2bfloat16_rn(v[i]);
                    } else if (full_cols && ((reinterpret_cast<uintptr_t>(drow) & 15u) == 0)) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * e], v[q * 8 + 2 * e + 1]);
                                w[e] = *reinterpret_cast<const uint32_t*>(&h);
                            }
                            reinterpret_cast<uint4*>(drow)[q] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < args.N) drow[i] = __float2bfloat16_rn(v[i]);
                    }
                    if (args.dt != nullptr) {
                        // transposed copy: for a fixed column the lanes of a warp write consecutive addresses
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < args.N)
                                args.dt[static_cast<long long>(col0 + i) * args.lddt + row] = __float2bfloat16_rn(v[i]);
                    }
                }
                if (args.symmetric) {
                    // mirror: element (row, c) with c > row also goes to (c, row)
                    const int warp_row0 = m0 + warp * 32;
                    if (col0 > warp_row0 + 31 && warp_row0 + 31 < args.M && full_cols) {
                        // the whole chunk is right of every row of this warp (warp-uniform): lanes pair up so
                        // that each store carries two consecutive rows of one column (4 bytes)
                        const bool odd = (lane & 1) != 0;
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float send = odd ? v[i] : v[i + 1];
                            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                            const float lo = odd ? recv : v[i];          // value of the even row
                            const float hi = odd ? v[i + 1] : recv;      // value of the odd row
                            const int c = col0 + i + (odd ? 1 : 0);
                            const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                            *reinterpret_cast<__nv_bfloat162*>(args.d + static_cast<long long>(c) * args.ldd + (row & ~1)) = h;
                        }
                    } else if (row_ok && col0 + 31 > row) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < args.N && col0 + i > row)
                                args.d[static_cast<long long>(col0 + i) * args.ldd + row] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
        }
        if (PERSIST) {   // this warp has read its rows of the buffer: one arrival per warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (threadIdx.x == 0 && abort_flag && args.status != nullptr) atomicExch(args.status, 1);
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        }
    });
    return fn;
}

// [rows, cols] bf16 row-major with leading dimension ld (elements); box = 64 (inner) x box_rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long k, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(GEFEN_B200_ECUDA, "cuTensorMapEncodeTiled is not available from the driver.");
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t elem[2] = {1, 1};
    const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(GEFEN_B200_ECUDA, "cuTensorMapEncodeTiled failed with code %d.", static_cast<int>(rc));
    return GEFEN_B200_OK;
}

// Tiles a launch computes (see tile_coords).
static int count_tiles(int M, int N, int bn, int symmetric) {
    const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + bn - 1) / bn;
    if (!symmetric) return tiles_m * tiles_n;
    int total = 0;
    for (int mi = 0; mi < tiles_m; ++mi) {
        const int row0 = mi * kBM;
        total += tiles_n - (row0 >= bn ? (row0 - bn) / bn + 1 : 0);
    }
    return total;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, bool PERSIST>
static int launch_gemm_variant(const CUtensorMap& ma, const CUtensorMap& mb, GemmArgs args, cudaStream_t stream) {
    constexpr int smem = STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 1024;
    static bool configured[64];
    int dev = 0;
    GEFEN_CHECK_CUDA(cudaGetDevice(&dev));
    auto kernel = ns_gemm_tn_kernel<BN, STAGES, A_MN, B_MN, PERSIST>;
    if (dev < 64 && !configured[dev]) {
        GEFEN_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured[dev] = true;
    }
    args.n_tiles = count_tiles(args.M, args.N, BN, args.symmetric);
    dim3 grid((args.N + BN - 1) / BN, (args.M + kBM - 1) / kBM);
    if (PERSIST) grid = dim3(args.n_tiles < sm_count() ? args.n_tiles : sm_count(), 1);
    kernel<<<grid, kGemmThreads, smem, stream>>>(ma, mb, args);
    GEFEN_CHECK_CUDA(cudaGetLastError());
    return GEFEN_B200_OK;
}

// More tiles than SMs: one persistent CTA per SM with two accumulator buffers, so that a tile's
// epilogue overlaps the next tile's main loop. Otherwise one CTA per tile.
// GEFEN_B200_NS_PERSIST=0/1 forces the choice (measurements).
template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& args, cudaStream_t stream) {
    static int forced = -2;
    if (forced == -2) {
        const char* e = getenv("GEFEN_B200_NS_PERSIST");
        forced = e == nullptr ? -1 : (e[0] == '0' ? 0 : 1);
    }
    bool persist = count_tiles(args.M, args.N, BN, args.symmetric) > sm_count();
    if (forced >= 0) persist = forced == 1;
    if constexpr (STAGES * (kBM + BN) * kBK * 2 > 96 * 1024) {   // the two-CTAs-per-SM variants stay one tile per CTA
        if (persist) return launch_gemm_variant<BN, STAGES, A_MN, B_MN, true>(ma, mb, args, stream);
    }
    return launch_gemm_variant<BN, STAGES, A_MN, B_MN, false>(ma, mb, args, stream);
}

}  // namespace gefen

using namespace gefen;

static int ns_gemm(const void* a, bool a_is_km, const void* b, bool b_is_kn, const void* c, void* d, void* dt, int M, int N, int K,
                   int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, int64_t lddt, double alpha, double beta,
                   int symmetric, int* status, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    GEFEN_CHECK_ARG(a != nullptr && b != nullptr && d != nullptr, "Expected non-null A, B and D.");
    GEFEN_CHECK_ARG(M > 0 && N > 0 && K > 0, "Expected positive GEMM sizes.");
    GEFEN_CHECK_ARG(beta == 0.0 || c != nullptr, "Expected C when beta != 0.");
    GEFEN_CHECK_ARG(!symmetric || (M == N && ldd % 2 == 0 && (reinterpret_cast<uintptr_t>(d) & 3u) == 0 && dt == nullptr),
                    "A symmetric result needs M == N, an even leading dimension and no transposed output.");
    GEFEN_CHECK_ARG(aligned16(a) && aligned16(b) && lda % 8 == 0 && ldb % 8 == 0 && lda >= (a_is_km ? M : K) &&
                        ldb >= (b_is_kn ? N : K),
                    "Expected 16-byte aligned A and B with leading dimensions that are multiples of 8 elements.");
    GEFEN_CHECK_ARG(ldd >= N && (c == nullptr || ldc >= N) && (dt == nullptr || lddt >= M), "Bad leading dimension.");
    // 128 x 256 tiles have the better arithmetic intensity; 128 x 128 tiles are used for small problems
    // that would leave most SMs without a tile (measured: for 2048-wide outputs the wider tile wins
    // even when a symmetric result computes only 72 of them)
    int bn = (N >= 2048 || (static_cast<long long>((M + 127) / 128) * ((N + 255) / 256)) >= sm_count()) ? 256 : 128;
    // GEFEN_B200_NS_TILE=<bn>x<stages> picks a variant by hand (measurements): 256x4, 256x2, 128x6, 128x3
    static int forced_bn = -1, forced_stages = 0;
    if (forced_bn < 0) {
        forced_bn = 0;
        const char* e = getenv("GEFEN_B200_NS_TILE");
        if (e != nullptr) sscanf(e, "%dx%d", &forced_bn, &forced_stages);
    }
    if (forced_bn == 256 || forced_bn == 128) bn = forced_bn;
    const bool shallow = forced_stages == 2 || forced_stages == 3;
    CUtensorMap ma, mb;
    int rc = a_is_km ? make_map(&ma, a, K, M, lda, kBK) : make_map(&ma, a, M, K, lda, kBM);
    if (rc != GEFEN_B200_OK) return rc;
    rc = b_is_kn ? make_map(&mb, b, K, N, ldb, kBK) : make_map(&mb, b, N, K, ldb, bn);
    if (rc != GEFEN_B200_OK) return rc;
    GemmArgs args;
    args.c = static_cast<const __nv_bfloat16*>(c);
    args.d = static_cast<__nv_bfloat16*>(d);
    args.dt = static_cast<__nv_bfloat16*>(dt);
    args.M = M; args.N = N; args.K = K;
    args.ldc = ldc; args.ldd = ldd; args.lddt = lddt;
    args.alpha = static_cast<float>(alpha);
    args.beta = static_cast<float>(beta);
    args.symmetric = symmetric;
    args.status = status;
    if (a_is_km && b_is_kn) {
        if (shallow) return bn == 256 ? launch_gemm<256, 2, true, true>(ma, mb, args, stream)
                                      : launch_gemm<128, 3, true, true>(ma, mb, args, stream);
        if (bn == 256) return launch_gemm<256, 4, true, true>(ma, mb, args, stream);
        return launch_gemm<128, 6, true, true>(ma, mb, args, stream);
    }
    if (a_is_km) return fail(GEFEN_B200_EUNSUPPORTED, "A given as [K, M] is only combined with B given as [K, N].");
    if (b_is_kn) {
        if (shallow) return bn == 256 ? launch_gemm<256, 2, false, true>(ma, mb, args, stream)
                                      : launch_gemm<128, 3, false, true>(ma, mb, args, stream);
        if (bn == 256) return launch_gemm<256, 4, false, true>(ma, mb, args, stream);
        return launch_gemm<128, 6, false, true>(ma, mb, args, stream);
    }
    if (shallow) return bn == 256 ? launch_gemm<256, 2, false, false>(ma, mb, args, stream)
                                  : launch_gemm<128, 3, false, false>(ma, mb, args, stream);
    if (bn == 256) return launch_gemm<256, 4, false, false>(ma, mb, args, stream);
    return launch_gemm<128, 6, false, false>(ma, mb, args, stream);
}

// The whole Newton-Schulz iteration of one matrix, enqueued from native code (fifteen GEMM launches
// for five steps) so that the host cost per product is a tensor-map encode and a launch.
static int enqueue_newton_schulz(void* x0, void* x1, void* gram, void* poly, int rows, int cols, int steps, double a,
                                 double b, double c, int* status, void* stream) {
    const int m = rows < cols ? rows : cols;
    void* cur = x0;
    void* nxt = x1;
    for (int it = 0; it < steps; ++it) {
        int rc;
        if (rows <= cols) {
            // G = X X^T ; B = b G + c G G ; X' = a X + B X
            rc = ns_gemm(cur, false, cur, false, nullptr, gram, nullptr, m, m, cols, cols, cols, 0, m, 0, 1.0, 0.0, 1, status, stream);
            if (rc != GEFEN_B200_OK) return rc;
            rc = ns_gemm(gram, false, gram, false, gram, poly, nullptr, m, m, m, m, m, m, m, 0, c, b, 1, status, stream);
            if (rc != GEFEN_B200_OK) return rc;
            rc = ns_gemm(poly, false, cur, true, cur, nxt, nullptr, rows, cols, m, m, cols, cols, cols, 0, 1.0, a, 0, status, stream);
            if (rc != GEFEN_B200_OK) return rc;
        } else {
            // G = Y^T Y ; B = b G + c G G ; Y' = a Y + Y B
            rc = ns_gemm(cur, true, cur, true, nullptr, gram, nullptr, m, m, rows, cols, cols, 0, m, 0, 1.0, 0.0, 1, status, stream);
            if (rc != GEFEN_B200_OK) return rc;
            rc = ns_gemm(gram, false, gram, false, gram, poly, nullptr, m, m, m, m, m, m, m, 0, c, b, 1, status, stream);
            if (rc != GEFEN_B200_OK) return rc;
            rc = ns_gemm(cur, false, poly, true, cur, nxt, nullptr, rows, cols, m, cols, m, cols, cols, 0, 1.0, a, 0, status, stream);
            if (rc != GEFEN_B200_OK) return rc;
        }
        void* t = cur; cur = nxt; nxt = t;
    }
    return GEFEN_B200_OK;
}

// The chain is the same fifteen launches whenever buffers, shape and coefficients repeat (an optimizer
// calls it for every matrix of a shape with the same scratch buffers, every step): from the second
// identical call on it is replayed as one CUDA graph, which shortens the gaps between the dependent
// launches. The first call runs eagerly (it also configures the kernels); the capture happens on a
// private stream in thread-local mode, and the graph is launched into the caller's stream.
// GEFEN_B200_NS_GRAPH=0 keeps every call eager.
namespace {
struct ChainKey {
    int dev, rows, cols, steps;
    void *x0, *x1, *gram, *poly, *status;
    double a, b, c;
    bool operator<(const ChainKey& o) const {
        return std::tie(dev, rows, cols, steps, x0, x1, gram, poly, status, a, b, c) <
               std::tie(o.dev, o.rows, o.cols, o.steps, o.x0, o.x1, o.gram, o.poly, o.status, o.a, o.b, o.c);
    }
};
std::mutex g_chain_mutex;
std::map<ChainKey, cudaGraphExec_t> g_chain_graphs;   // nullptr: seen once, not captured yet
cudaStream_t g_capture_stream[64];
constexpr size_t kMaxChainGraphs = 64;
}  // namespace

extern "C" int gefen_b200_newton_schulz(void* x0, void* x1, void* gram, void* poly, int rows, int cols, int steps,
                                        double a, double b, double c, int* status, void* stream) {
    GEFEN_CHECK_ARG(x0 && x1 && gram && poly, "Expected non-null buffers.");
    GEFEN_CHECK_ARG(rows > 0 && cols > 0 && rows % 8 == 0 && cols % 8 == 0, "Expected dimensions that are multiples of 8.");
    GEFEN_CHECK_ARG(steps >= 0 && steps < 100, "Number of steps must be less than 100.");
    static int use_graphs = -1;
    if (use_graphs < 0) {
        const char* e = getenv("GEFEN_B200_NS_GRAPH");
        use_graphs = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    int dev = 0;
    GEFEN_CHECK_CUDA(cudaGetDevice(&dev));
    if (!use_graphs || steps == 0 || dev < 0 || dev >= 64)
        return enqueue_newton_schulz(x0, x1, gram, poly, rows, cols, steps, a, b, c, status, stream);

    const ChainKey key{dev, rows, cols, steps, x0, x1, gram, poly, status, a, b, c};
    std::lock_guard<std::mutex> lock(g_chain_mutex);
    auto it = g_chain_graphs.find(key);
    if (it == g_chain_graphs.end()) {
        if (g_chain_graphs.size() >= kMaxChainGraphs) {   // callers whose buffers keep moving: start over
            for (auto& kv : g_chain_graphs)
                if (kv.second != nullptr) cudaGraphExecDestroy(kv.second);
            g_chain_graphs.clear();
        }
        g_chain_graphs[key] = nullptr;
        return enqueue_newton_schulz(x0, x1, gram, poly, rows, cols, steps, a, b, c, status, stream);
    }
    if (it->second == nullptr) {
        if (g_capture_stream[dev] == nullptr)
            GEFEN_CHECK_CUDA(cudaStreamCreateWithFlags(&g_capture_stream[dev], cudaStreamNonBlocking));
        cudaStream_t cs = g_capture_stream[dev];
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        bool ok = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if (ok) {
            const int rc = enqueue_newton_schulz(x0, x1, gram, poly, rows, cols, steps, a, b, c, status, cs);
            const cudaError_t end = cudaStreamEndCapture(cs, &graph);
            ok = rc == GEFEN_B200_OK && end == cudaSuccess && graph != nullptr;
        }
        if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
        if (graph != nullptr) cudaGraphDestroy(graph);
        if (!ok) {   // leave this chain eager for good
            cudaGetLastError();
            g_chain_graphs.erase(it);
            use_graphs = 0;
            return enqueue_newton_schulz(x0, x1, gram, poly, rows, cols, steps, a, b, c, status, stream);
        }
        it->second = exec;
    }
    GEFEN_CHECK_CUDA(cudaGraphLaunch(it->second, static_cast<cudaStream_t>(stream)));
    return GEFEN_B200_OK;
}

extern "C" int gefen_b200_ns_gemm_tn(const void* a, const void* b, const void* c, void* d, void* dt, int M, int N, int K,
                                     int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, int64_t lddt, double alpha,
                                     double beta, int symmetric, int* status, void* stream) {
    return ns_gemm(a, false, b, false, c, d, dt, M, N, K, lda, ldb, ldc, ldd, lddt, alpha, beta, symmetric, status, stream);
}

extern "C" int gefen_b200_ns_gemm_nn(const void* a, const void* b, const void* c, void* d, int M, int N, int K,
                                     int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, double alpha, double beta,
                                     int* status, void* stream) {
    return ns_gemm(a, false, b, true, c, d, nullptr, M, N, K, lda, ldb, ldc, ldd, 0, alpha, beta, 0, status, stream);
}

extern "C" int gefen_b200_ns_gemm_tt(const void* a, const void* b, const void* c, void* d, int M, int N, int K,
                                     int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, double alpha, double beta,
                                     int symmetric, int* status, void* stream) {
    return ns_gemm(a, true, b, true, c, d, nullptr, M, N, K, lda, ldb, ldc, ldd, 0, alpha, beta, symmetric, status, stream);
}
