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
#include "tcgen05.cuh"

namespace mb {

// OUT_F32: float32 output rows instead of bfloat16. TC_BN: columns of the output tile (the N
// of the MMA, also the tensor-memory columns held); TC_STAGES: depth of the operand ring.
template <bool OUT_F32, int TC_BN, int TC_STAGES>
__global__ void __launch_bounds__(128)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __nv_bfloat16* __restrict__ bias, void* __restrict__ out, int M, int N,
                    int K, int* __restrict__ error, long long wait_limit, int withheld_kb) {
    // wait_limit: SM clocks after which a wait gives up. withheld_kb: -1, or (to try the
    // giving-up path) the k-block whose bytes are announced to the barrier and never sent.
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
            if (!mbar_wait(&empty_bar[s], phase ^ 1, error, 1, wait_limit)) break;
            unsigned char* a_tile = tiles + s * TC_STAGE_BYTES;
            unsigned char* b_tile = a_tile + TC_BM * TC_BK * 2;
            mbar_expect_tx(&full_bar[s], TC_STAGE_BYTES);
            if (kb != withheld_kb) {
                tma_load_2d(a_tile, &map_x, kb * TC_BK, m0, &full_bar[s]);
                tma_load_2d(b_tile, &map_w, kb * TC_BK, n0, &full_bar[s]);
            }
            issued = kb + 1;
        }
        // if the consumer gave up, still wait (bounded) for what was issued and not consumed
        if (*reinterpret_cast<volatile int*>(error) != 0) {
            for (int kb = issued > TC_STAGES ? issued - TC_STAGES : 0; kb < issued; ++kb)
                mbar_wait(&full_bar[kb % TC_STAGES], (kb / TC_STAGES) & 1, error, 4, wait_limit);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc = umma_idesc(TC_BM, TC_BN);
        bool ok = true;
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
            const int s = kb % TC_STAGES;
            const uint32_t phase = (kb / TC_STAGES) & 1;
            ok = mbar_wait(&full_bar[s], phase, error, 2, wait_limit);
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
    const bool ready = mbar_wait(&accum_bar, 0, error, 3, wait_limit);
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

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_gemm_tcgen05_supports(int M, int N, int K) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0;
}

template <bool OUT_F32, int BN, int STAGES>
static int launch_tcgen05(const void* x, const void* w, const void* bias, void* out, int M, int N,
                          int K, int* error, cudaStream_t s, long long wait_limit = TC_WAIT_CYCLES,
                          int withheld_kb = -1) {
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
              (const __nv_bfloat16*)bias, out, M, N, K, error, wait_limit, withheld_kb);
    return launch_status();
}

// The giving-up path of the bounded waits, run on purpose: the product as mb_gemm_tcgen05
// computes it (128 x 128 tiles, bfloat16 out), except that the bytes of k-block 0 are
// announced to their barrier and never sent, and every wait gives up after `wait_cycles` SM
// clocks instead of about a second. Each block's MMA issuer runs out of patience, sets
// `error`, the other roles see it or run out themselves, copies in flight are waited for,
// tensor memory is freed, and the kernel returns: `out` is left as it was and the context
// stays usable. For tests of that path only.
MB_EXPORT int mb_gemm_tcgen05_withheld(const void* x, const void* w, void* out, int M, int N, int K,
                                       int* error, long long wait_cycles, void* stream) {
    if (!mb_gemm_tcgen05_supports(M, N, K) || wait_cycles <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) return MB_ERR_ALIGNMENT;
    return launch_tcgen05<false, 128, 3>(x, w, nullptr, out, M, N, K, error, (cudaStream_t)stream,
                                         wait_cycles, 0);
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
