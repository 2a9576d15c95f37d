// out[M, N] = x[M, K] w[N, K]^T (+ bias) in bfloat16 on the fifth-generation tensor cores:
// TMA brings 128 x 64 tiles of both operands into a four-stage, 128-byte-swizzled shared
// memory ring; one thread issues tcgen05.mma (128 x 128 x 16 per instruction) with the
// float32 accumulator in tensor memory; four warps read the accumulator back with
// tcgen05.ld, add the bias, round once and store. It stands where the reference calls
// F.linear on many tokens (mercury/model/qwen2.py:42, :64-69).
//
// One CTA computes one 128 x 128 tile of the output (cta_group::1, no cluster, no
// multicast). Roles: thread 0 of warp 0 produces (TMA), thread 0 of warp 1 issues the MMAs,
// all four warps run the epilogue. Every wait on an mbarrier is bounded: a wait that runs
// out sets the error word the host passes in and the CTA stops issuing work, waits
// (bounded again) for the copies it has in flight, frees its tensor memory and returns.
//
// Sizes: K a multiple of 8 (a TMA row stride is a multiple of 16 bytes), any M and N
// (edges are zero-filled by TMA on the way in and masked on the way out); operands must be
// 16-byte aligned.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace mb {

constexpr int TC_BM = 128, TC_BK = 64;
constexpr long long TC_WAIT_CYCLES = 2000000000ll;             // about a second of SM clocks

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

// Bounded wait for the phase with the given parity; false (and the error word set) if it
// never came.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error, int code) {
    const uint32_t addr = smem_u32(bar);
    const long long start = clock64();
    while (clock64() - start < TC_WAIT_CYCLES) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    atomicExch(error, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Shared-memory operand descriptor: K-major tile of rows x 64 bfloat16 as TMA leaves it with
// 128-byte swizzle (rows 128 bytes apart, groups of 8 rows 1024 bytes apart).
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset: next 8-row group
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // 128-byte swizzle
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M x N tile.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// OUT_F32: float32 output rows instead of bfloat16. TC_BN: columns of the output tile (the N
// of the MMA, also the tensor-memory columns held); TC_STAGES: depth of the operand ring.
template <bool OUT_F32, int TC_BN, int TC_STAGES>
__global__ void __launch_bounds__(128)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __nv_bfloat16* __restrict__ bias, void* __restrict__ out, int M, int N,
                    int K, int* __restrict__ error) {
    grid_dependency_sync();
    constexpr int TC_STAGE_BYTES = (TC_BM + TC_BN) * TC_BK * 2;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the dynamic window is only 16-byte aligned by contract: round up to the swizzle atom
    unsigned char* tiles =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[TC_STAGES], empty_bar[TC_STAGES], accum_bar;
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * TC_BN;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmem_base_slot)),
                     "r"((uint32_t)TC_BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_base_slot;

    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads of both operands, one k-block per stage
        int issued = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
            const int s = kb % TC_STAGES;
            const uint32_t phase = (kb / TC_STAGES) & 1;
            if (!mbar_wait(&empty_bar[s], phase ^ 1, error, 1)) break;
            unsigned char* a_tile = tiles + s * TC_STAGE_BYTES;
            unsigned char* b_tile = a_tile + TC_BM * TC_BK * 2;
            mbar_expect_tx(&full_bar[s], TC_STAGE_BYTES);
            tma_load_2d(a_tile, &map_x, kb * TC_BK, m0, &full_bar[s]);
            tma_load_2d(b_tile, &map_w, kb * TC_BK, n0, &full_bar[s]);
            issued = kb + 1;
        }
        // if the consumer gave up, still wait (bounded) for what was issued and not consumed
        if (*reinterpret_cast<volatile int*>(error) != 0) {
            for (int kb = issued > TC_STAGES ? issued - TC_STAGES : 0; kb < issued; ++kb)
                mbar_wait(&full_bar[kb % TC_STAGES], (kb / TC_STAGES) & 1, error, 4);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc = umma_idesc(TC_BM, TC_BN);
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int s = kb % TC_STAGES;
            const uint32_t phase = (kb / TC_STAGES) & 1;
            ok = mbar_wait(&full_bar[s], phase, error, 2);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned char* a_tile = tiles + s * TC_STAGE_BYTES;
            const unsigned char* b_tile = a_tile + TC_BM * TC_BK * 2;
            const uint64_t adesc = umma_desc(a_tile), bdesc = umma_desc(b_tile);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; ++k) {
                // 16 bfloat16 = 32 bytes further along K inside the swizzled row
                umma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                          (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
        }
        umma_commit(&accum_bar);          // the accumulator is complete once all MMAs are done
    }

    // ---- epilogue: all four warps, warp w owns accumulator lanes (rows) 32w .. 32w+31
    __syncwarp();
    const bool ready = mbar_wait(&accum_bar, 0, error, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int m = m0 + warp * 32 + lane;
    // tcgen05.ld is warp-wide: take the decision for the whole warp
    const bool go = __all_sync(0xffffffffu, ready && *reinterpret_cast<volatile int*>(error) == 0);
    if (go) {
#pragma unroll 1
        for (int c0 = 0; c0 < TC_BN; c0 += 32) {
            uint32_t r[32];
            tmem_load_32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
            if (m < M) {
                if (OUT_F32) {
                    float* row = reinterpret_cast<float*>(out) + (int64_t)m * N + n0 + c0;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = n0 + c0 + j;
                        if (n < N) row[j] = __uint_as_float(r[j]) + (bias ? __bfloat162float(bias[n]) : 0.f);
                    }
                } else {
                    __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(out) + (int64_t)m * N + n0 + c0;
                    if (n0 + c0 + 32 <= N && (N % 8) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 q;
                            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int n = n0 + c0 + j + 2 * e;
                                const float b0 = bias ? __bfloat162float(bias[n]) : 0.f;
                                const float b1 = bias ? __bfloat162float(bias[n + 1]) : 0.f;
                                h2[e] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) + b0,
                                                              __uint_as_float(r[j + 2 * e + 1]) + b1);
                            }
                            *reinterpret_cast<uint4*>(row + j) = q;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int n = n0 + c0 + j;
                            if (n < N)
                                row[j] = __float2bfloat16_rn(__uint_as_float(r[j]) +
                                                             (bias ? __bfloat162float(bias[n]) : 0.f));
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d),
                     "r"((uint32_t)TC_BN)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------
// The persistent variant: one CTA per SM walks output tiles of 128 x 256; a producer warp
// keeps the four-stage operand ring full across tile boundaries, an MMA warp alternates
// between two 256-column accumulators in tensor memory, and four epilogue warps drain one
// accumulator while the MMAs fill the other, so the epilogue costs no tensor-core time.
// EPI 0: bfloat16 out (+ bias); 1: float32 out (+ bias); 2: SiLU gate: the B tile is 128
// gate rows followed by the 128 matching up rows of a packed [2 * width, K] matrix, and the
// output [M, width] is silu(gate) * up (mercury/model/qwen2.py:42), so the packed
// projection is never written out.
constexpr int TP_BN = 256, TP_STAGES = 4;
constexpr int TP_STAGE_BYTES = (TC_BM + TP_BN) * TC_BK * 2;   // 48 KB
constexpr int TP_THREADS = 192;

template <int EPI>
__global__ void __launch_bounds__(TP_THREADS)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_x,
                               const __grid_constant__ CUtensorMap map_w,
                               const __nv_bfloat16* __restrict__ bias, void* __restrict__ out, int M,
                               int N, int K, int width, int* __restrict__ error) {
    grid_dependency_sync();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* tiles =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[TP_STAGES], empty_bar[TP_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    // EPI 2 walks tiles of 128 result columns (each needs 128 gate + 128 up rows of w)
    const int n_cols = EPI == 2 ? width : N;
    const int tile_cols = EPI == 2 ? 128 : TP_BN;
    const int tiles_n = (n_cols + tile_cols - 1) / tile_cols;
    const int tiles_m = (M + TC_BM - 1) / TC_BM;
    const int num_tiles = tiles_n * tiles_m;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TP_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);     // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile / tiles_n) * TC_BM, n0 = (tile % tiles_n) * tile_cols;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TP_STAGES;
                    const uint32_t phase = (it / TP_STAGES) & 1;
                    ok = mbar_wait(&empty_bar[s], phase ^ 1, error, 1);
                    if (!ok) break;
                    unsigned char* a_tile = tiles + s * TP_STAGE_BYTES;
                    unsigned char* b_tile = a_tile + TC_BM * TC_BK * 2;
                    mbar_expect_tx(&full_bar[s], TP_STAGE_BYTES);
                    tma_load_2d(a_tile, &map_x, kb * TC_BK, m0, &full_bar[s]);
                    if (EPI == 2) {
                        // the w map has boxes of 128 rows: gate rows, then the up rows
                        tma_load_2d(b_tile, &map_w, kb * TC_BK, n0, &full_bar[s]);
                        tma_load_2d(b_tile + 128 * TC_BK * 2, &map_w, kb * TC_BK, width + n0,
                                    &full_bar[s]);
                    } else {
                        tma_load_2d(b_tile, &map_w, kb * TC_BK, n0, &full_bar[s]);
                    }
                }
            }
            if (!ok) {
                // wait (bounded) for what is still in flight before the CTA may exit
                for (int s = 0; s < TP_STAGES; ++s) mbar_wait(&full_bar[s], 0, error, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer
            const uint32_t idesc = umma_idesc(TC_BM, TP_BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
                ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, error, 5);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * TP_BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % TP_STAGES;
                    const uint32_t phase = (it / TP_STAGES) & 1;
                    ok = mbar_wait(&full_bar[s], phase, error, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned char* a_tile = tiles + s * TP_STAGE_BYTES;
                    const unsigned char* b_tile = a_tile + TC_BM * TC_BK * 2;
                    const uint64_t adesc = umma_desc(a_tile), bdesc = umma_desc(b_tile);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(&empty_bar[s]);
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---- epilogue warps 2..5: warp w may touch accumulator lanes 32 * (w % 4) ..
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
            ok = mbar_wait(&acc_full[acc], acc_phase, error, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m0 = (tile / tiles_n) * TC_BM, n0 = (tile % tiles_n) * tile_cols;
            const int m = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * TP_BN + ((uint32_t)(quarter * 32) << 16);
            if (EPI == 2) {
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t g[32], u[32];
                    tmem_load_32(taddr + (uint32_t)c0, g);
                    tmem_load_32(taddr + (uint32_t)(128 + c0), u);
                    if (m < M) {
                        __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(out) + (int64_t)m * width + n0 + c0;
                        const bool fast = n0 + c0 + 32 <= width && (width % 8) == 0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 q;
                            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float v[2];
#pragma unroll
                                for (int z = 0; z < 2; ++z) {
                                    // as the separate kernels do: gate and up rounded to bfloat16 first
                                    const float gv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(g[j + 2 * e + z])));
                                    const float uv = __bfloat162float(__float2bfloat16_rn(__uint_as_float(u[j + 2 * e + z])));
                                    // the result is rounded to bfloat16: the fast exponential and
                                    // division are far inside that rounding
                                    v[z] = __fdividef(gv, 1.f + __expf(-gv)) * uv;
                                }
                                h2[e] = __floats2bfloat162_rn(v[0], v[1]);
                            }
                            if (fast) {
                                *reinterpret_cast<uint4*>(row + j) = q;
                            } else {
                                const __nv_bfloat16* q16 = reinterpret_cast<const __nv_bfloat16*>(&q);
                                for (int e = 0; e < 8; ++e)
                                    if (n0 + c0 + j + e < width) row[j + e] = q16[e];
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < TP_BN; c0 += 32) {
                    if (n0 + c0 >= N) break;
                    uint32_t r[32];
                    tmem_load_32(taddr + (uint32_t)c0, r);
                    if (m < M) {
                        if (EPI == 1) {
                            float* row = reinterpret_cast<float*>(out) + (int64_t)m * N + n0 + c0;
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int n = n0 + c0 + j;
                                if (n < N) row[j] = __uint_as_float(r[j]) + (bias ? __bfloat162float(bias[n]) : 0.f);
                            }
                        } else {
                            __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(out) + (int64_t)m * N + n0 + c0;
                            const bool fast = n0 + c0 + 32 <= N && (N % 8) == 0;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 q;
                                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int n = n0 + c0 + j + 2 * e;
                                    const float b0 = (bias && n < N) ? __bfloat162float(bias[n]) : 0.f;
                                    const float b1 = (bias && n + 1 < N) ? __bfloat162float(bias[n + 1]) : 0.f;
                                    h2[e] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) + b0,
                                                                  __uint_as_float(r[j + 2 * e + 1]) + b1);
                                }
                                if (fast) {
                                    *reinterpret_cast<uint4*>(row + j) = q;
                                } else {
                                    const __nv_bfloat16* q16 = reinterpret_cast<const __nv_bfloat16*>(&q);
                                    for (int e = 0; e < 8; ++e)
                                        if (n0 + c0 + j + e < N) row[j + e] = q16[e];
                                }
                            }
                        }
                    }
                }
            }
            // this accumulator may be overwritten once all four warps have read it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc]))
                             : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                     : "memory");
    }
}

// ------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) !=
                cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// A [rows, K] bfloat16 row-major matrix as tiles of box_rows x 64 with 128-byte swizzle.
// Encoding a map costs microseconds on the host and the same few matrices come back every
// step, so encoded maps are kept (a map depends only on address, sizes and box).
struct MapKey {
    const void* base;
    int rows, K, box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        h ^= std::hash<long long>()(((long long)k.rows << 32) ^ ((long long)k.K << 8) ^ k.box_rows) +
             0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};

static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex guard;
    const MapKey key{base, rows, K, box_rows};
    {
        std::lock_guard<std::mutex> lock(guard);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *map = it->second;
            return true;
        }
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(guard);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *map;
    return true;
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_gemm_tcgen05_supports(int M, int N, int K) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0;
}

template <bool OUT_F32, int BN, int STAGES>
static int launch_tcgen05(const void* x, const void* w, const void* bias, void* out, int M, int N,
                          int K, int* error, cudaStream_t s) {
    CUtensorMap map_x, map_w;
    if (!make_map(&map_x, x, M, K, TC_BM) || !make_map(&map_w, w, N, K, BN)) return MB_ERR_LAUNCH;
    const size_t smem = (size_t)STAGES * (TC_BM + BN) * TC_BK * 2 + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<OUT_F32, BN, STAGES>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + TC_BM - 1) / TC_BM);
    if (grid.y > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    MB_LAUNCH((gemm_tcgen05_kernel<OUT_F32, BN, STAGES>), grid, 128, smem, s, map_x, map_w,
              (const __nv_bfloat16*)bias, out, M, N, K, error);
    return launch_status();
}

// x: [M, K], w: [N, K], bias: [N] or null, all bfloat16; out: [M, N] bfloat16 (out_f32 = 0)
// or float32 (out_f32 = 1). `error`: one int on the device, zero before the call; nonzero
// afterwards means a bounded wait inside the kernel ran out (1 producer, 2 MMA issuer,
// 3 epilogue) and the output is not valid. `tile`: 0 picks the tile by shape; 1 = 128 x 128
// with a three-stage ring (two CTAs per SM), 2 = 128 x 256 with a four-stage ring.
MB_EXPORT int mb_gemm_tcgen05(const void* x, const void* w, const void* bias, void* out, int out_f32,
                              int M, int N, int K, int* error, int tile, void* stream) {
    if (!mb_gemm_tcgen05_supports(M, N, K)) return MB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return MB_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (tile == 0) {
        const long long wide_ctas = (long long)((N + 255) / 256) * ((M + 127) / 128);
        tile = wide_ctas >= 148 ? 2 : 1;
    }
    if (tile == 2)
        return out_f32 ? launch_tcgen05<true, 256, 4>(x, w, bias, out, M, N, K, error, s)
                       : launch_tcgen05<false, 256, 4>(x, w, bias, out, M, N, K, error, s);
    return out_f32 ? launch_tcgen05<true, 128, 3>(x, w, bias, out, M, N, K, error, s)
                   : launch_tcgen05<false, 128, 3>(x, w, bias, out, M, N, K, error, s);
}

template <int EPI>
static int launch_persistent(const void* x, const void* w, const void* bias, void* out, int M, int N,
                             int K, int width, int* error, cudaStream_t s) {
    CUtensorMap map_x, map_w;
    const int w_rows = EPI == 2 ? 2 * width : N;
    if (!make_map(&map_x, x, M, K, TC_BM) || !make_map(&map_w, w, w_rows, K, EPI == 2 ? 128 : TP_BN))
        return MB_ERR_LAUNCH;
    const size_t smem = (size_t)TP_STAGES * TP_STAGE_BYTES + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<EPI>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    const int n_cols = EPI == 2 ? width : N;
    const int tile_cols = EPI == 2 ? 128 : TP_BN;
    const long long tiles = (long long)((n_cols + tile_cols - 1) / tile_cols) * ((M + TC_BM - 1) / TC_BM);
    const int grid = (int)(tiles < sms ? tiles : sms);
    MB_LAUNCH((gemm_tcgen05_persistent_kernel<EPI>), grid, TP_THREADS, smem, s, map_x, map_w,
              (const __nv_bfloat16*)bias, out, M, N, K, width, error);
    return launch_status();
}

// The persistent kernel. mode 0: bfloat16 out [M, N] (+ bias); 1: float32 out (+ bias);
// 2: w is a packed [2 * N, K] gate/up matrix and out is silu(x gate^T) * (x up^T), [M, N]
// bfloat16 (N a multiple of 8). `error` as for mb_gemm_tcgen05 (5: the MMA issuer gave up
// waiting for an accumulator).
MB_EXPORT int mb_gemm_tcgen05_persistent(const void* x, const void* w, const void* bias, void* out,
                                         int mode, int M, int N, int K, int* error, void* stream) {
    if (!mb_gemm_tcgen05_supports(M, N, K)) return MB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return MB_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == 0) return launch_persistent<0>(x, w, bias, out, M, N, K, 0, error, s);
    if (mode == 1) return launch_persistent<1>(x, w, bias, out, M, N, K, 0, error, s);
    if (mode == 2) {
        if (N % 8) return MB_ERR_UNSUPPORTED_SIZE;
        return launch_persistent<2>(x, w, nullptr, out, M, 2 * N, K, N, error, s);
    }
    return MB_ERR_BAD_DTYPE;
}
