// The many-token bfloat16 product on pairs of SMs: out[M, N] = x[M, K] w[N, K]^T with one of
// the epilogues below. Two CTAs of a thread-block cluster share one tcgen05.mma of 256 rows
// (cta_group::2): each CTA brings its own 128 rows of x and its own half of the w rows of the
// tile into its shared memory by TMA, one thread of the even CTA issues the MMAs for both,
// and each CTA finds its 128 rows of the accumulator in its own tensor memory. A CTA thus
// loads 128 + BN/2 operand rows per 128 x BN outputs where a lone CTA loads 128 + BN: the
// products of a prompt step are bound by the operand traffic from L2, not by the tensor
// pipe. No load is multicast: every TMA copy lands in the shared memory of the CTA that
// issued it and only its completion is counted on the even CTA's barrier.
//
// Persistent: the pairs walk the output tiles; a producer warp per CTA keeps the operand
// ring full across tile boundaries, the MMA thread alternates between two accumulators in
// tensor memory, and four epilogue warps per CTA drain one accumulator while the MMAs fill
// the other. Every mbarrier wait is bounded; a wait that runs out sets the error word, the
// roles stop, both CTAs meet at the closing cluster barrier, free their tensor memory and
// return.
//
// Epilogues (EPI), each after an optional row scale 1/rms of the input rows, which commutes
// with the product (the input is then the float32 stream times the norm weight, and the
// sums of squares of the stream's rows come in pieces per row, as the kernel that updated
// the stream left them; mercury/model/layers.py:14-30 is the norm this finishes):
//   0  bfloat16 out (+ bias)                           (mercury/model/qwen2.py:64-69)
//   2  silu(gate) * up for w = [gate rows; up rows]     (mercury/model/qwen2.py:42)
//   3  added into the float32 stream h[M, N]; with `next_w` it also leaves bfloat16(h * next_w)
//      and the row's sum of squares over this tile's columns for the product after the next
//      norm (mercury/model/qwen2.py:91-99: residual add, then the next RMSNorm)
#include "tcgen05.cuh"

namespace mb {

// Two warps may read each quarter of the accumulator's rows; they share its columns, chunk of
// 32 by chunk (with four epilogue warps a 128 x 256 tile took longer to drain than its MMAs
// take at 14 k-blocks).
constexpr int GP_EPI_GROUPS = 2;
constexpr int GP_THREADS = 64 + 128 * GP_EPI_GROUPS;
constexpr int GP_RING_BYTES = 192 * 1024;

struct PairEpilogue {
    const __nv_bfloat16* bias;      // [N] or null
    const float* ss_part;           // [M, ss_tiles] sums of squares of the input's stream rows, or null
    int ss_tiles;
    float ss_eps;
    int ss_k;                       // length of a stream row
    float* h;                       // EPI 3: the stream
    const __nv_bfloat16* next_w;    // EPI 3: weight of the norm that follows, or null
    __nv_bfloat16* next_x;          // EPI 3: [M, N]
    float* next_ss;                 // EPI 3: [M, tiles along N]
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// the address of the same shared-memory object in the CTA `rank` of the cluster
__device__ __forceinline__ uint32_t peer_address(const void* p, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
    return a;
}

__device__ __forceinline__ void cluster_meet() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// A TMA copy into this CTA's shared memory whose bytes are counted on a barrier that may
// lie in the other CTA of the pair (`bar` is a shared::cluster address). Not a multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One arrival, once the MMAs issued so far are done, on the barrier at this offset in both
// CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"((uint16_t)3)
        : "memory");
}

__device__ __forceinline__ void arrive_at(uint32_t cluster_address) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address)
                 : "memory");
}

// BN: columns of a pair's output tile (each CTA brings BN / 2 rows of w). For EPI 2 the tile
// is 128 result columns: 128 gate rows in the even CTA, the matching up rows in the odd one.
template <int EPI, int BN>
__global__ void __launch_bounds__(GP_THREADS)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 PairEpilogue ep, void* __restrict__ out, int M, int N, int K, int width,
                 int* __restrict__ error) {
    grid_dependency_sync();
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = (BN / 2) * TC_BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int STAGES = GP_RING_BYTES / STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // (the same rounding in both CTAs: the pair's MMAs address both memories by one offset)
    unsigned char* tiles =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;
    const int n_cols = EPI == 2 ? width : N;
    constexpr int TILE_COLS = EPI == 2 ? BN / 2 : BN;
    const int tiles_n = (n_cols + TILE_COLS - 1) / TILE_COLS;
    const int tiles_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
    const int num_tiles = tiles_n * tiles_m;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);      // even CTA: its producer's arrival; bytes of both
            mbar_init(&empty_bar[s], 1);     // a commit of the pair's MMAs
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 8 * GP_EPI_GROUPS);   // even CTA: the epilogue warps of both CTAs
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_meet();     // the other CTA's barriers exist before anything is counted on them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (both CTAs): this CTA's rows of x and of w for every k-block
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
                const int m0 = (tile / tiles_n) * 2 * TC_BM + (int)rank * TC_BM;
                const int n0 = (tile % tiles_n) * TILE_COLS;
                const int w_row = EPI == 2 ? (rank ? width + n0 : n0) : n0 + (int)rank * (BN / 2);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    ok = mbar_wait(&empty_bar[s], phase ^ 1, error, 1);
                    if (!ok) break;
                    unsigned char* a_tile = tiles + s * STAGE_BYTES;
                    unsigned char* b_tile = a_tile + A_BYTES;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
                    const uint32_t bar = peer_address(&full_bar[s], 0);
                    tma_load_2d_pair(a_tile, &map_x, kb * TC_BK, m0, bar);
                    tma_load_2d_pair(b_tile, &map_w, kb * TC_BK, w_row, bar);
                }
            }
            if (!ok && rank == 0) {
                // wait (bounded) for what may still be in flight before the CTAs may exit
                for (int s = 0; s < STAGES; ++s) mbar_wait(&full_bar[s], 0, error, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer of the pair
            const uint32_t idesc = umma_idesc(2 * TC_BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
                const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
                ok = mbar_wait(&acc_empty[acc], acc_phase ^ 1, error, 5);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phase = (it / STAGES) & 1;
                    ok = mbar_wait(&full_bar[s], phase, error, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned char* a_tile = tiles + s * STAGE_BYTES;
                    const uint64_t adesc = umma_desc(a_tile), bdesc = umma_desc(a_tile + A_BYTES);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16_pair(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty_bar[s]);
                }
                if (ok) umma_commit_pair(&acc_full[acc]);
            }
        }
    } else {
        // ---- epilogue warps from 2 on (both CTAs): warp w may touch accumulator lanes 32 (w % 4) ..
        const int quarter = warp & 3, group = (warp - 2) >> 2;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
            const uint32_t acc = local & 1, acc_phase = (local >> 1) & 1;
            ok = mbar_wait(&acc_full[acc], acc_phase, error, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int tile_n = tile % tiles_n;
            const int m0 = (tile / tiles_n) * 2 * TC_BM + (int)rank * TC_BM, n0 = tile_n * TILE_COLS;
            const int m = m0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
            float rs = 1.f;
            if (ep.ss_part && m < M) {
                float sum = 0.f;
                for (int t = 0; t < ep.ss_tiles; ++t) sum += ep.ss_part[(int64_t)m * ep.ss_tiles + t];
                rs = rsqrtf(sum / (float)ep.ss_k + ep.ss_eps);
            }
            if (EPI == 2) {
#pragma unroll 1
                for (int c0 = 32 * group; c0 < BN / 2; c0 += 32 * GP_EPI_GROUPS) {
                    if (n0 + c0 >= width) break;
                    uint32_t g[32], u[32];
                    tmem_load_32_async(taddr + (uint32_t)c0, g);
                    tmem_load_32_async(taddr + (uint32_t)(BN / 2 + c0), u);
                    tmem_wait_ld();
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
                                    const float gv = __bfloat162float(
                                        __float2bfloat16_rn(__uint_as_float(g[j + 2 * e + z]) * rs));
                                    const float uv = __bfloat162float(
                                        __float2bfloat16_rn(__uint_as_float(u[j + 2 * e + z]) * rs));
                                    // (the result is rounded to bfloat16: the fast exponential and
                                    // division are far inside that rounding)
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
            } else if (EPI == 3) {
                float sq = 0.f;
#pragma unroll 1
                for (int c0 = 32 * group; c0 < BN; c0 += 32 * GP_EPI_GROUPS) {
                    if (n0 + c0 >= N) break;
                    uint32_t r[32];
                    tmem_load_32(taddr + (uint32_t)c0, r);
                    if (m < M) {
                        float* hrow = ep.h + (int64_t)m * N + n0 + c0;
                        if (n0 + c0 + 32 <= N && (N % 8) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                float4 a = *reinterpret_cast<const float4*>(hrow + j);
                                float4 b = *reinterpret_cast<const float4*>(hrow + j + 4);
                                float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                                for (int e = 0; e < 8; ++e) {
                                    v[e] += __uint_as_float(r[j + e]) * rs +
                                            (ep.bias ? __bfloat162float(ep.bias[n0 + c0 + j + e]) : 0.f);
                                    sq += v[e] * v[e];
                                }
                                *reinterpret_cast<float4*>(hrow + j) = make_float4(v[0], v[1], v[2], v[3]);
                                *reinterpret_cast<float4*>(hrow + j + 4) = make_float4(v[4], v[5], v[6], v[7]);
                                if (ep.next_w) {
                                    const uint4 wq = *reinterpret_cast<const uint4*>(ep.next_w + n0 + c0 + j);
                                    const __nv_bfloat16* w8 = reinterpret_cast<const __nv_bfloat16*>(&wq);
                                    uint4 q;
                                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                                    for (int e = 0; e < 4; ++e)
                                        h2[e] = __floats2bfloat162_rn(v[2 * e] * __bfloat162float(w8[2 * e]),
                                                                      v[2 * e + 1] * __bfloat162float(w8[2 * e + 1]));
                                    *reinterpret_cast<uint4*>(ep.next_x + (int64_t)m * N + n0 + c0 + j) = q;
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const int n = n0 + c0 + j;
                                if (n >= N) continue;
                                const float v = hrow[j] + __uint_as_float(r[j]) * rs +
                                                (ep.bias ? __bfloat162float(ep.bias[n]) : 0.f);
                                hrow[j] = v;
                                sq += v * v;
                                if (ep.next_w)
                                    ep.next_x[(int64_t)m * N + n] =
                                        __float2bfloat16_rn(v * __bfloat162float(ep.next_w[n]));
                            }
                        }
                    }
                }
                if (ep.next_ss && m < M)
                    ep.next_ss[(int64_t)m * (tiles_n * GP_EPI_GROUPS) + tile_n * GP_EPI_GROUPS + group] = sq;
            } else {
#pragma unroll 1
                for (int c0 = 32 * group; c0 < BN; c0 += 32 * GP_EPI_GROUPS) {
                    if (n0 + c0 >= N) break;
                    uint32_t r[32];
                    tmem_load_32(taddr + (uint32_t)c0, r);
                    if (m < M) {
                        __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(out) + (int64_t)m * N + n0 + c0;
                        const bool fast = n0 + c0 + 32 <= N && (N % 8) == 0;
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 q;
                            __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int n = n0 + c0 + j + 2 * e;
                                const float b0 = (ep.bias && n < N) ? __bfloat162float(ep.bias[n]) : 0.f;
                                const float b1 = (ep.bias && n + 1 < N) ? __bfloat162float(ep.bias[n + 1]) : 0.f;
                                h2[e] = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) * rs + b0,
                                                              __uint_as_float(r[j + 2 * e + 1]) * rs + b1);
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
            // this accumulator may be overwritten once the epilogue warps of both CTAs have read it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) arrive_at(peer_address(&acc_empty[acc], 0));
        }
    }
    // Neither CTA may leave, or give its tensor memory back, while the other may still read
    // its shared memory (the pair's MMAs) or count on its barriers.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_meet();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                     : "memory");
    }
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_gemm_pair_supports(int M, int N, int K) {
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && N % 8 == 0;
}

static int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

// Column tiles of a product of modes 0 and 3 (the second extent of next_ss): tiles of 256
// columns when those give every pair of SMs a tile, of 128 otherwise.
static bool pair_wide(int M, int N) {
    const long long wide = (long long)((N + 255) / 256) * ((M + 2 * TC_BM - 1) / (2 * TC_BM));
    return N > 128 && wide >= sm_count() / 2;
}

MB_EXPORT int mb_gemm_pair_tiles(int M, int N) {
    return GP_EPI_GROUPS * (pair_wide(M, N) ? (N + 255) / 256 : (N + 127) / 128);
}

template <int EPI, int BN>
static int launch_pair(const void* x, const void* w, const PairEpilogue& ep, void* out, int M, int N,
                       int K, int width, int* error, cudaStream_t s) {
    CUtensorMap map_x, map_w;
    const int w_rows = EPI == 2 ? 2 * width : N;
    if (!make_map(&map_x, x, M, K, TC_BM) || !make_map(&map_w, w, w_rows, K, BN / 2)) return MB_ERR_LAUNCH;
    const size_t smem = (size_t)GP_RING_BYTES + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(gemm_pair_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    const int sms = sm_count();
    const int n_cols = EPI == 2 ? width : N;
    const int tile_cols = EPI == 2 ? BN / 2 : BN;
    const long long tiles = (long long)((n_cols + tile_cols - 1) / tile_cols) * ((M + 2 * TC_BM - 1) / (2 * TC_BM));
    const int pairs = (int)(tiles < sms / 2 ? tiles : sms / 2);
    MB_LAUNCH_CLUSTER((gemm_pair_kernel<EPI, BN>), dim3(2 * pairs), GP_THREADS, smem, s, 2, 1, 1, map_x,
                      map_w, ep, out, M, N, K, width, error);
    return launch_status();
}

// x: [M, K], w: [N, K] (mode 2: [2 N, K], gate rows then up rows), bias: [N] or null, all
// bfloat16. mode 0: out [M, N] bfloat16; 2: out [M, N] = silu(x gate^T) * (x up^T); 3: h[M, N]
// float32 += the product, and with next_w also next_x [M, N] = bfloat16(h * next_w) and
// next_ss [M, tiles] (tiles = mb_gemm_pair_tiles(M, N)), the sums of squares of h's rows per
// column tile. ss_part [M, ss_tiles]: sums of squares of the stream rows that x was made of
// (x = stream * norm weight): the result rows are scaled by rsqrt(sum / ss_k + ss_eps).
// `error`: one int on the device, zero before the call; nonzero afterwards means a bounded
// wait inside the kernel ran out (1 producer, 2 and 5 MMA issuer, 3 epilogue) and the
// output is not valid.
MB_EXPORT int mb_gemm_pair(const void* x, const void* w, const void* bias, void* out, int mode, int M,
                           int N, int K, const float* ss_part, int ss_tiles, float ss_eps, int ss_k,
                           float* h, const void* next_w, void* next_x, float* next_ss, int* error,
                           void* stream) {
    if (!mb_gemm_pair_supports(M, N, K)) return MB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)h | (uintptr_t)next_x |
         (uintptr_t)next_w) & 15)
        return MB_ERR_ALIGNMENT;
    if (mode == 3 && !h) return MB_ERR_UNSUPPORTED_SIZE;
    if (next_w && (mode != 3 || !next_x || !next_ss)) return MB_ERR_UNSUPPORTED_SIZE;
    if (ss_part && (ss_tiles <= 0 || ss_k <= 0)) return MB_ERR_UNSUPPORTED_SIZE;
    PairEpilogue ep;
    ep.bias = (const __nv_bfloat16*)bias;
    ep.ss_part = ss_part;
    ep.ss_tiles = ss_tiles;
    ep.ss_eps = ss_eps;
    ep.ss_k = ss_k;
    ep.h = h;
    ep.next_w = (const __nv_bfloat16*)next_w;
    ep.next_x = (__nv_bfloat16*)next_x;
    ep.next_ss = next_ss;
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == 2) return launch_pair<2, 256>(x, w, ep, out, M, 2 * N, K, N, error, s);
    // narrow outputs: tiles of 128 columns, so that more pairs have one
    const bool narrow = !pair_wide(M, N);
    if (mode == 0)
        return narrow ? launch_pair<0, 128>(x, w, ep, out, M, N, K, 0, error, s)
                      : launch_pair<0, 256>(x, w, ep, out, M, N, K, 0, error, s);
    if (mode == 3)
        return narrow ? launch_pair<3, 128>(x, w, ep, out, M, N, K, 0, error, s)
                      : launch_pair<3, 256>(x, w, ep, out, M, N, K, 0, error, s);
    return MB_ERR_BAD_DTYPE;
}
