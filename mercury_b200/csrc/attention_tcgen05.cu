// Paged attention of prompt portions on the fifth-generation tensor cores (bfloat16, head
// size 64): scores and the probability-weighted values are tcgen05.mma products with their
// accumulators in tensor memory; queries, keys and values arrive by TMA, keys and values one
// cache page per copy straight from the pages the block table names.
//
// Same contract as the other attention kernels (ragged batch, causal by absolute position,
// optional window; mercury/model/attention.py:77-101 is the reference's gather-and-SDPA
// version). A CTA takes floor(128 / group) query tokens of one sequence and one KV head: the
// (token, head of the group) pairs are the 128 rows of the MMA, one row per accumulator
// lane and per softmax thread. Per tile of 128 keys:
//   producer (warp 4)  TMA of up to 128/page_size key pages and value pages
//   MMA      (warp 5)  S = Q K^T (128 x 128 x 64) into tensor memory
//   softmax  (warps 0-3, one thread per row)  tcgen05.ld of the row, mask, running maximum,
//            2^x, probabilities rounded to bfloat16 into a swizzled shared-memory tile
//   MMA                O_tile = P V (128 x 64 x 128), V used as stored (MN-major operand)
//   softmax            O = O * correction + O_tile in registers (float32)
// Two CTAs fit on an SM (80 KB of shared memory, 256 tensor-memory columns each), so one
// CTA's MMAs run under the other's softmax. Every mbarrier wait is bounded; a wait that
// runs out sets the error word and the CTA winds down (frees its tensor memory, returns).
#include "tcgen05.cuh"

namespace mb {

constexpr int TA_D = 64;             // head size
constexpr int TA_ROWS = 128;         // MMA M: query rows per CTA
constexpr int TA_KEYS = 128;         // keys per tile
constexpr int TA_THREADS = 192;

__device__ __forceinline__ float ta_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// MN-major B operand (values as stored: [key][d], d contiguous, 128-byte swizzle).
__device__ __forceinline__ uint64_t umma_desc_mn(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;               // one 64-element block along N: offset unused
    d |= (uint64_t)(1024 >> 4) << 32;     // next group of 8 keys
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(TA_THREADS)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const int* __restrict__ table,
                         int max_pages, const int* __restrict__ q_start,
                         const int* __restrict__ kv_len_of, __nv_bfloat16* __restrict__ out, int n_q,
                         int n_kv, int page_size, float scale, int window, int tiles_per_seq,
                         int* __restrict__ error) {
    grid_dependency_sync();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;                       // 128 rows x 128 B
    unsigned char* k_s = q_s + TA_ROWS * 128;        // 128 keys x 128 B
    unsigned char* v_s = k_s + TA_KEYS * 128;        // 128 keys x 128 B
    unsigned char* p_s = v_s + TA_KEYS * 128;        // 2 x (128 rows x 128 B): keys 0-63, 64-127
    __shared__ uint64_t q_full, kv_full, s_ready, p_ready, o_ready;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int page_ok[TA_KEYS];                 // per key of the tile: 1 if its page was copied

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = n_q / n_kv;
    const int tok_per_tile = TA_ROWS / group;
    const int seq = blockIdx.x / tiles_per_seq;
    const int tile = tiles_per_seq - 1 - (blockIdx.x - seq * tiles_per_seq);   // heavy tiles first
    const int kvh = blockIdx.y;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    const int tok0 = tile * tok_per_tile;
    if (tok0 >= q_len) return;
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;
    int tok_max = tok0 + tok_per_tile - 1;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok0, p_max = first_pos + tok_max;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / TA_KEYS;
    const int t_hi = p_max / TA_KEYS + 1;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        mbar_init(&kv_full, 1);
        mbar_init(&s_ready, 1);
        mbar_init(&p_ready, 4);
        mbar_init(&o_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmem_base_slot)),
                     "r"(256u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_base_slot;            // 128 columns of scores
    const uint32_t tmem_o = tmem_base_slot + TA_KEYS;  // 64 columns of P.V

    if (warp == 4) {
        // ---------------------------------------------------------------- producer
        // page ids of a tile are looked up by the whole warp, copies issued by lane 0
        if (lane == 0) {
            mbar_expect_tx(&q_full, (uint32_t)(group * tok_per_tile * 128));
            tma_load_4d(q_s, &map_q, 0, 0, kvh, q_begin + tok0, &q_full);
        }
        const int pages_per_tile = TA_KEYS / page_size;
        bool ok = true;
        for (int kt = t_lo; kt < t_hi && ok; ++kt) {
            const int i = kt - t_lo;
            if (i > 0) ok = mbar_wait(&o_ready, (uint32_t)((i - 1) & 1), error, 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            // lanes 0 .. pages_per_tile-1 each look one page up
            int page = -1;
            if (lane < pages_per_tile) {
                const int key0 = kt * TA_KEYS + lane * page_size;
                if (key0 < kv_len) page = table[(int64_t)seq * max_pages + key0 / page_size];
            }
            for (int k = lane; k < TA_KEYS; k += 32) {
                const int pg = __shfl_sync(0xffffffffu, page, k / page_size);
                page_ok[k] = pg >= 0 && kt * TA_KEYS + k < kv_len;
            }
            const unsigned valid = __ballot_sync(0xffffffffu, page >= 0);
            __syncwarp();
            if (lane == 0) {
                const int copies = __popc(valid);
                mbar_expect_tx(&kv_full, (uint32_t)(copies * 2 * page_size * 128));
            }
            __syncwarp();
            if (page >= 0) {
                const int row = (page * n_kv + kvh) * page_size;
                tma_load_2d(k_s + lane * page_size * 128, &map_k, 0, row, &kv_full);
                tma_load_2d(v_s + lane * page_size * 128, &map_v, 0, row, &kv_full);
            }
        }
    } else if (warp == 5) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(TA_ROWS, TA_KEYS);
            const uint32_t idesc_o = umma_idesc(TA_ROWS, TA_D) | (1u << 16);   // B is MN-major
            bool ok = mbar_wait(&q_full, 0, error, 2);
            for (int kt = t_lo; kt < t_hi && ok; ++kt) {
                const uint32_t parity = (uint32_t)((kt - t_lo) & 1);
                ok = mbar_wait(&kv_full, parity, error, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t qd = umma_desc(q_s), kd = umma_desc(k_s);
#pragma unroll
                for (int k = 0; k < TA_D / 16; ++k)
                    umma_bf16(tmem_s, qd + (uint64_t)(2 * k), kd + (uint64_t)(2 * k), idesc_s, k > 0);
                umma_commit(&s_ready);
                ok = mbar_wait(&p_ready, parity, error, 5);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t vd = umma_desc_mn(v_s);
#pragma unroll
                for (int k = 0; k < TA_KEYS / 16; ++k) {
                    const uint64_t pd = umma_desc(p_s + (k / 4) * (TA_ROWS * 128)) + (uint64_t)(2 * (k % 4));
                    umma_bf16(tmem_o, pd, vd + (uint64_t)(k * (2048 >> 4)), idesc_o, k > 0);
                }
                umma_commit(&o_ready);
            }
        }
    } else {
        // ---------------------------------------------------------------- softmax: row = thread
        const int r = warp * 32 + lane;
        const int tok = tok0 + r / group;
        const int hg = r % group;
        const bool row_ok = r < group * tok_per_tile && tok < q_len;
        const int pos = first_pos + tok;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const float scale2 = scale * 1.4426950408889634f;
        float o[TA_D];
#pragma unroll
        for (int c = 0; c < TA_D; ++c) o[c] = 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int kt = t_lo; kt < t_hi; ++kt) {
            const uint32_t parity = (uint32_t)((kt - t_lo) & 1);
            ok = mbar_wait(&s_ready, parity, error, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int key0 = kt * TA_KEYS;
            // does every key of the tile count for this row, and is every key real?
            const bool plain = row_ok && key0 + TA_KEYS - 1 <= pos && key0 + TA_KEYS <= kv_len &&
                               (window <= 0 || key0 > pos - window);
            // pass 1: the row's maximum over the tile
            float m_new = m;
#pragma unroll 1
            for (int c0 = 0; c0 < TA_KEYS; c0 += 32) {
                uint32_t sv[32];
                tmem_load_32(tmem_s + lane_addr + (uint32_t)c0, sv);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int key = key0 + c0 + j;
                    bool seen = plain;
                    if (!plain) {
                        seen = row_ok && key <= pos && key < kv_len && page_ok[c0 + j];
                        if (window > 0) seen = seen && key > pos - window;
                    }
                    if (seen) m_new = fmaxf(m_new, __uint_as_float(sv[j]) * scale2);
                }
            }
            const float corr = m_new > -INFINITY ? ta_exp2(m - m_new) : 1.f;
            m = m_new;
            l *= corr;
            // pass 2: probabilities, rounded to bfloat16, into the swizzled P tile
#pragma unroll 1
            for (int c0 = 0; c0 < TA_KEYS; c0 += 32) {
                uint32_t sv[32];
                tmem_load_32(tmem_s + lane_addr + (uint32_t)c0, sv);
                unsigned char* prow = p_s + (c0 / 64) * (TA_ROWS * 128) + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 packed;
                    uint32_t* pw = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        float p2[2];
#pragma unroll
                        for (int z = 0; z < 2; ++z) {
                            const int j = q4 * 8 + e * 2 + z;
                            const int key = key0 + c0 + j;
                            bool seen = plain;
                            if (!plain) {
                                seen = row_ok && key <= pos && key < kv_len && page_ok[c0 + j];
                                if (window > 0) seen = seen && key > pos - window;
                            }
                            const float p = (seen && m > -INFINITY)
                                                ? ta_exp2(__uint_as_float(sv[j]) * scale2 - m)
                                                : 0.f;
                            l += p;
                            p2[z] = p;
                        }
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(p2[0], p2[1]);
                        pw[e] = *reinterpret_cast<uint32_t*>(&h2);
                    }
                    const int chunk = (c0 % 64) / 8 + q4;          // 16-byte chunk inside the 128-byte row
                    *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) * 16)) = packed;
                }
            }
            // a value row that was not copied, or lies beyond the sequence, must not reach the
            // MMA as it is (0 * NaN): thread r clears key r of the tile
            if (!page_ok[r]) {
                uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(v_s + r * 128 + c * 16) = zero;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_ready)) : "memory");
            ok = mbar_wait(&o_ready, parity, error, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c0 = 0; c0 < TA_D; c0 += 32) {
                uint32_t ov[32];
                tmem_load_32(tmem_o + lane_addr + (uint32_t)c0, ov);
#pragma unroll
                for (int j = 0; j < 32; ++j) o[c0 + j] = o[c0 + j] * corr + __uint_as_float(ov[j]);
            }
            // the next tile's P.V may overwrite tmem_o only after this read: ordered by the
            // p_ready arrival of the next tile, which comes after it in program order
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        if (ok && row_ok) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + ((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * TA_D;
#pragma unroll
            for (int c = 0; c < TA_D; c += 8) {
                uint4 q;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    h2[e] = __floats2bfloat162_rn(o[c + 2 * e] * inv, o[c + 2 * e + 1] * inv);
                *reinterpret_cast<uint4*>(dst + c) = q;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_slot),
                     "r"(256u)
                     : "memory");
    }
}

}  // namespace mb

using namespace mb;

// Whether the tensor-memory attention takes this problem: bfloat16, head size 64, pages of 8
// to 128 tokens, groups of at most 128 query heads per KV head, row strides that TMA accepts.
MB_EXPORT int mb_attention_tcgen05_supports(int d, int page_size, int n_q, int n_kv, int q_row_stride) {
    if (d != TA_D || n_kv <= 0 || n_q % n_kv) return 0;
    const int group = n_q / n_kv;
    if (group > TA_ROWS) return 0;
    if (page_size < 8 || page_size > TA_KEYS || (page_size & (page_size - 1))) return 0;
    return q_row_stride % 8 == 0;
}

// qkv: [tokens, q_row_stride] bfloat16 with the rotated queries first; k_pages / v_pages:
// [num_pages, n_kv, page_size, 64]; out: [tokens, n_q * 64]. `error` as for mb_gemm_tcgen05
// (codes 1 producer, 2 and 5 MMA issuer, 3 and 4 softmax).
MB_EXPORT int mb_paged_attention_tcgen05(const void* qkv, int q_row_stride, const void* k_pages,
                                         const void* v_pages, int num_pages, const int* table,
                                         int max_pages, const int* q_start, const int* kv_len,
                                         void* out, int tokens, int num_seqs, int max_q_len, int n_q,
                                         int n_kv, int d, int page_size, float scale, int window,
                                         int* error, void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_attention_tcgen05_supports(d, page_size, n_q, n_kv, q_row_stride)) return MB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) & 15) return MB_ERR_ALIGNMENT;
    const int group = n_q / n_kv;
    const int tok_per_tile = TA_ROWS / group;
    CUtensorMap map_q, map_k, map_v;
    {
        // queries: [D, group, n_kv, tokens]
        cuuint64_t dims[4] = {(cuuint64_t)TA_D, (cuuint64_t)group, (cuuint64_t)n_kv, (cuuint64_t)tokens};
        cuuint64_t strides[3] = {(cuuint64_t)TA_D * 2, (cuuint64_t)group * TA_D * 2, (cuuint64_t)q_row_stride * 2};
        cuuint32_t box[4] = {(cuuint32_t)TA_D, (cuuint32_t)group, 1u, (cuuint32_t)tok_per_tile};
        if (!make_map_nd(&map_q, qkv, 4, dims, strides, box)) return MB_ERR_LAUNCH;
    }
    {
        const cuuint64_t rows = (cuuint64_t)num_pages * n_kv * page_size;
        cuuint64_t dims[2] = {(cuuint64_t)TA_D, rows};
        cuuint64_t strides[1] = {(cuuint64_t)TA_D * 2};
        cuuint32_t box[2] = {(cuuint32_t)TA_D, (cuuint32_t)page_size};
        if (!make_map_nd(&map_k, k_pages, 2, dims, strides, box) ||
            !make_map_nd(&map_v, v_pages, 2, dims, strides, box))
            return MB_ERR_LAUNCH;
    }
    const size_t smem = (size_t)(TA_ROWS + 2 * TA_KEYS + 2 * TA_ROWS) * 128 + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    const int tiles_per_seq = (max_q_len + tok_per_tile - 1) / tok_per_tile;
    dim3 grid(num_seqs * tiles_per_seq, n_kv);
    if (n_kv > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    MB_LAUNCH((attention_tcgen05_kernel), grid, TA_THREADS, smem, (cudaStream_t)stream, map_q, map_k, map_v,
              table, max_pages, q_start, kv_len, (__nv_bfloat16*)out, n_q, n_kv, page_size, scale, window,
              tiles_per_seq, error);
    return launch_status();
}
