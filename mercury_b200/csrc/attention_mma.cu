// Paged attention in bfloat16 on the tensor cores (mma.sync m16n8k16), for head sizes 64
// and 128: the serving path of prompt portions and of decode tokens.
//
// Same contract as the CUDA-core kernel in attention_simt.cu (ragged batch, block tables,
// causal mask by absolute position, optional window, optional split over keys merged by
// attention_combine_kernel); other head sizes are left to that kernel.
//
// The (query token, head of the group) pairs of one sequence and one KV head are laid out
// as rows, so the query heads that share a KV head also share each key tile. A warp owns
// 16 rows; a block has NWARPS warps (4 for prompt portions, 1 for decode-like batches,
// where the split over keys provides the parallelism). Keys are walked in tiles of 64
// aligned to absolute positions, brought in by 16-byte cp.async copies straight from the
// pages into a two-stage, XOR-swizzled shared-memory ring. Scores, the running maximum and
// sum, and the output accumulate in float32; probabilities are rounded to bfloat16 for the
// P.V product (the usual flash-attention arrangement).
#include "tcgen05.cuh"

namespace mb {

constexpr int MMA_BN = 64;  // keys per tile

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zeroed
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(addr), "l"(gmem),
                 "r"(bytes));
}

// 2^x by the special-function unit (ex2.approx: relative error about 2^-22, far below the
// bfloat16 rounding that follows); 2^-inf = 0.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32)
attention_mma_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                     const __nv_bfloat16* __restrict__ k_pages,
                     const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ table,
                     int max_pages, const int* __restrict__ q_start,
                     const int* __restrict__ kv_len_of, __nv_bfloat16* __restrict__ out,
                     float* __restrict__ part_acc, float* __restrict__ part_ml, int n_q, int n_kv,
                     int page_size, float scale, int window, int tiles_per_seq, int num_splits) {
    grid_dependency_sync();
    constexpr int ROWS = NWARPS * 16;
    constexpr int CH = D / 8;        // 16-byte chunks per row
    constexpr int THREADS = NWARPS * 32;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [ROWS][D]
    __nv_bfloat16* k_s = q_s + ROWS * D;                              // [2][MMA_BN][D]
    __nv_bfloat16* v_s = k_s + 2 * MMA_BN * D;                        // [2][MMA_BN][D]

    const int seq = blockIdx.x / tiles_per_seq;
    // later row tiles see more keys: hand them out first
    const int tile = tiles_per_seq - 1 - (blockIdx.x - seq * tiles_per_seq);
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int group = n_q / n_kv;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    const int row0 = tile * ROWS;
    if (row0 >= q_len * group) return;
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // ---- queries of this block's rows -> shared (swizzled) -> A fragments
    for (int idx = tid; idx < ROWS * CH; idx += THREADS) {
        const int r = idx / CH, c = idx - r * CH;
        const int row = row0 + r;
        const int tok = row / group, hg = row - tok * group;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (tok < q_len)
            val = *reinterpret_cast<const uint4*>(qkv + (int64_t)(q_begin + tok) * q_row_stride +
                                                  (kvh * group + hg) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + r * D + ((c ^ (r & 7)) * 8)) = val;
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = ks * 2 + (lane >> 4);
        ldmatrix_x4(qf[ks], q_s + r * D + ((c ^ (r & 7)) * 8));
    }

    // ---- rows of this thread: g and g + 8 of the warp's 16
    const int g = lane >> 2, t4 = lane & 3;
    int pos[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = row0 + warp * 16 + g + h * 8;
        const int tok = row / group;
        row_ok[h] = tok < q_len;
        pos[h] = first_pos + tok;
    }

    // first and last position among the rows of this warp (for whole-tile tests)
    const int wrow0 = row0 + warp * 16;
    const bool warp_rows_ok = (wrow0 + 15) / group < q_len;
    const int warp_pos_min = first_pos + wrow0 / group;
    const int warp_pos_max = first_pos + (wrow0 + 15) / group;

    // ---- key tiles of this block
    const int tok_min = row0 / group;
    int tok_max = (row0 + ROWS - 1) / group;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok_min, p_max = first_pos + tok_max;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / MMA_BN;
    int t_hi = p_max / MMA_BN + 1;
    if (num_splits > 1) {
        const int per = (t_hi - t_lo + num_splits - 1) / num_splits;
        t_lo = t_lo + split * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }

    auto load_tile = [&](int stage, int kt) {
        __nv_bfloat16* kd = k_s + stage * MMA_BN * D;
        __nv_bfloat16* vd = v_s + stage * MMA_BN * D;
        for (int idx = tid; idx < MMA_BN * CH; idx += THREADS) {
            const int j = idx / CH, c = idx - j * CH;
            const int key = kt * MMA_BN + j;
            int page = -1;
            if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
            const bool valid = page >= 0;
            const int64_t at =
                valid ? (((int64_t)page * n_kv + kvh) * page_size + (key % page_size)) * D + c * 8 : 0;
            const int sw = (c ^ (j & 7)) * 8;
            cp_async_16(kd + j * D + sw, k_pages + at, valid);
            cp_async_16(vd + j * D + sw, v_pages + at, valid);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float scale2 = scale * 1.4426950408889634f;  // scores in units of log2(e)

    if (t_lo < t_hi) load_tile(0, t_lo);
    for (int kt = t_lo; kt < t_hi; ++kt) {
        const int stage = (kt - t_lo) & 1;
        if (kt + 1 < t_hi) {
            load_tile(stage ^ 1, kt + 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        const __nv_bfloat16* kt_s = k_s + stage * MMA_BN * D;
        const __nv_bfloat16* vt_s = v_s + stage * MMA_BN * D;

        // S = Q K^T : 16 rows x 64 keys per warp
        float s[MMA_BN / 8][4];
#pragma unroll
        for (int i = 0; i < MMA_BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int n2 = 0; n2 < MMA_BN / 16; ++n2) {
                uint32_t b[4];
                const int j = n2 * 16 + (lane & 7) + (lane >> 4) * 8;
                const int c = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(b, kt_s + j * D + ((c ^ (j & 7)) * 8));
                mma_bf16(s[2 * n2], qf[ks], b[0], b[1]);
                mma_bf16(s[2 * n2 + 1], qf[ks], b[2], b[3]);
            }
        }

        // mask, scale, online softmax (float32). A tile that every row of the warp sees
        // whole (all its keys at or before the warp's first position, inside every window)
        // needs no per-element test.
        float m_new[2] = {m[0], m[1]};
        const int tile_first = kt * MMA_BN, tile_last = tile_first + MMA_BN - 1;
        const bool whole = warp_rows_ok && tile_last <= warp_pos_min && tile_last < kv_len &&
                           (window <= 0 || tile_first > warp_pos_max - window);
        if (whole) {
#pragma unroll
            for (int nt = 0; nt < MMA_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    s[nt][e] *= scale2;
                    m_new[e >> 1] = fmaxf(m_new[e >> 1], s[nt][e]);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < MMA_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int h = e >> 1;
                    const int key = tile_first + nt * 8 + 2 * t4 + (e & 1);
                    bool seen = row_ok[h] && key <= pos[h] && key < kv_len;
                    if (window > 0) seen = seen && key > pos[h] - window;
                    s[nt][e] = seen ? s[nt][e] * scale2 : -INFINITY;
                    m_new[h] = fmaxf(m_new[h], s[nt][e]);
                }
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
            corr[h] = m_new[h] > -INFINITY ? fast_exp2(m[h] - m_new[h]) : 1.f;
            m[h] = m_new[h];
            l[h] *= corr[h];
        }
#pragma unroll
        for (int nt = 0; nt < MMA_BN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const float p = m[h] > -INFINITY ? fast_exp2(s[nt][e] - m[h]) : 0.f;
                s[nt][e] = p;
                l[h] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }

        // O += P V
#pragma unroll
        for (int kk = 0; kk < MMA_BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int d2 = 0; d2 < D / 16; ++d2) {
                uint32_t b[4];
                const int j = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = d2 * 2 + (lane >> 4);
                ldmatrix_x4_trans(b, vt_s + j * D + ((c ^ (j & 7)) * 8));
                mma_bf16(o[2 * d2], a, b[0], b[1]);
                mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();  // everyone is done with this stage before it is refilled
    }

    // ---- finish: per-thread partial sums of l over the quad, then write
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_ok[h]) continue;
        const int row = row0 + warp * 16 + g + h * 8;
        const int tok = row / group, hg = row - tok * group;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + kvh * group + hg;
        if (num_splits == 1) {
            const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(out + flat * D + i * 8 + 2 * t4) = v;
            }
        } else {
            const int64_t at = flat * num_splits + split;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                float2 v = make_float2(o[i][2 * h], o[i][2 * h + 1]);
                *reinterpret_cast<float2*>(part_acc + at * D + i * 8 + 2 * t4) = v;
            }
            if (t4 == 0) {
                // the merge kernel works with natural-log maxima
                part_ml[at * 2] = m[h] * 0.6931471805599453f;
                part_ml[at * 2 + 1] = l[h];
            }
        }
    }
}

// Decode-like batches: at most 16 rows per (sequence, KV head), so one m16 tile of queries.
// The four warps of a block share each 64-key tile, 16 keys per warp, and merge their
// running (max, sum, output) through shared memory at the end; with one warp alone the
// kernel is bound by the latency of its own instruction stream. When `counters` is given,
// the block that finishes last among the splits of a (sequence, KV head) merges them and
// writes the output itself, which saves the separate merge launch; the merge walks the
// splits in index order, so the result does not depend on which block came last.
template <int D>
__global__ void __launch_bounds__(128)
attention_decode_kernel(const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                        const __nv_bfloat16* __restrict__ k_pages,
                        const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ table,
                        int max_pages, const int* __restrict__ q_start,
                        const int* __restrict__ kv_len_of, __nv_bfloat16* __restrict__ out,
                        float* __restrict__ part_acc, float* __restrict__ part_ml,
                        int* __restrict__ counters, int n_q, int n_kv, int page_size, float scale,
                        int window, int num_splits) {
    constexpr int CH = D / 8;
    constexpr int STAGES = 3;
    // Before waiting for the kernel in front (which stores this step's keys): ask L2 for the
    // keys and values of this block's tiles. Lengths and block tables were copied to the
    // device before the step began, and all but the newest key are from earlier steps.
    {
        const int seq_ = blockIdx.x, kvh_ = blockIdx.y;
        const int q_len_ = q_start[seq_ + 1] - q_start[seq_];
        if (q_len_ > 0 && (threadIdx.x & 1) == 0) {
            const int kv_len_ = kv_len_of[seq_];
            int lo = 0;
            if (window > 0 && kv_len_ - q_len_ - window + 1 > 0) lo = (kv_len_ - q_len_ - window + 1) / MMA_BN;
            int hi = (kv_len_ - 1) / MMA_BN + 1;
            if (num_splits > 1) {
                const int per = (hi - lo + num_splits - 1) / num_splits;
                lo = lo + (int)blockIdx.z * per;
                if (lo + per < hi) hi = lo + per;
            }
            for (int kt = lo; kt < hi; ++kt) {
                const int key = kt * MMA_BN + (threadIdx.x >> 1);
                if (key >= kv_len_) continue;
                const int page = table_page(table, seq_, max_pages, key / page_size);
                if (page < 0) continue;
                const int64_t at = (((int64_t)page * n_kv + kvh_) * page_size + (key % page_size)) * D;
                for (int b = 0; b < D * 2; b += 128) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(k_pages + at) + b));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char*>(v_pages + at) + b));
                }
            }
        }
    }
    grid_dependency_sync();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);      // [16][D]
    __nv_bfloat16* k_s = q_s + 16 * D;                                    // [STAGES][64][D]
    __nv_bfloat16* v_s = k_s + STAGES * MMA_BN * D;                       // [STAGES][64][D]
    float* o_red = reinterpret_cast<float*>(k_s);                         // [4][16][D], after the loop
    __shared__ float ml_red[4][16][2];
    __shared__ int last_flag;

    const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int group = n_q / n_kv;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    if (q_len <= 0) return;
    const int rows = q_len * group;          // <= 16
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;

    for (int idx = tid; idx < 16 * CH; idx += 128) {
        const int r = idx / CH, c = idx - r * CH;
        const int tok = r / group, hg = r - tok * group;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r < rows)
            val = *reinterpret_cast<const uint4*>(qkv + (int64_t)(q_begin + tok) * q_row_stride +
                                                  (kvh * group + hg) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + r * D + ((c ^ (r & 7)) * 8)) = val;
    }

    int pos[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + h * 8;
        row_ok[h] = r < rows;
        pos[h] = first_pos + r / group;
    }
    const int p_min = first_pos, p_max = kv_len - 1;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / MMA_BN;
    int t_hi = p_max / MMA_BN + 1;
    if (num_splits > 1) {
        const int per = (t_hi - t_lo + num_splits - 1) / num_splits;
        t_lo = t_lo + split * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }

    // each thread copies half a key row of K and of V: one table lookup per tile
    const int lj = tid >> 1, lc0 = (tid & 1) * (CH / 2);
    auto load_tile = [&](int stage, int kt) {
        const int key = kt * MMA_BN + lj;
        int page = -1;
        if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
        const bool valid = page >= 0;
        const int64_t at =
            valid ? (((int64_t)page * n_kv + kvh) * page_size + (key % page_size)) * D : 0;
        __nv_bfloat16* kd = k_s + (stage * MMA_BN + lj) * D;
        __nv_bfloat16* vd = v_s + (stage * MMA_BN + lj) * D;
#pragma unroll
        for (int c = 0; c < CH / 2; ++c) {
            const int sw = ((lc0 + c) ^ (lj & 7)) * 8;
            cp_async_16(kd + sw, k_pages + at + (lc0 + c) * 8, valid);
            cp_async_16(vd + sw, v_pages + at + (lc0 + c) * 8, valid);
        }
    };

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float scale2 = scale * 1.4426950408889634f;

    // prologue: STAGES - 1 tiles in flight (empty groups keep the accounting uniform)
#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (t_lo + st < t_hi) load_tile(st, t_lo + st);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = ks * 2 + (lane >> 4);
        ldmatrix_x4(qf[ks], q_s + r * D + ((c ^ (r & 7)) * 8));
    }

    for (int kt = t_lo; kt < t_hi; ++kt) {
        const int it = kt - t_lo;
        const int stage = it % STAGES;
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
        __syncthreads();   // tile kt has landed for everyone; tile kt-1's stage is free
        if (kt + STAGES - 1 < t_hi) load_tile((it + STAGES - 1) % STAGES, kt + STAGES - 1);
        asm volatile("cp.async.commit_group;\n" ::);
        const __nv_bfloat16* kt_s = k_s + stage * MMA_BN * D;
        const __nv_bfloat16* vt_s = v_s + stage * MMA_BN * D;

        // this warp's 16 keys of the tile
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t b[4];
            const int j = warp * 16 + (lane & 7) + (lane >> 4) * 8;
            const int c = ks * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b, kt_s + j * D + ((c ^ (j & 7)) * 8));
            mma_bf16(s[0], qf[ks], b[0], b[1]);
            mma_bf16(s[1], qf[ks], b[2], b[3]);
        }
        float m_new[2] = {m[0], m[1]};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int key = kt * MMA_BN + warp * 16 + nt * 8 + 2 * t4 + (e & 1);
                bool seen = row_ok[h] && key <= pos[h] && key < kv_len;
                if (window > 0) seen = seen && key > pos[h] - window;
                s[nt][e] = seen ? s[nt][e] * scale2 : -INFINITY;
                m_new[h] = fmaxf(m_new[h], s[nt][e]);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
            corr[h] = m_new[h] > -INFINITY ? fast_exp2(m[h] - m_new[h]) : 1.f;
            m[h] = m_new[h];
            l[h] *= corr[h];
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const float p = m[h] > -INFINITY ? fast_exp2(s[nt][e] - m[h]) : 0.f;
                s[nt][e] = p;
                l[h] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= corr[0];
            o[i][1] *= corr[0];
            o[i][2] *= corr[1];
            o[i][3] *= corr[1];
        }
        uint32_t a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int d2 = 0; d2 < D / 16; ++d2) {
            uint32_t b[4];
            const int j = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int c = d2 * 2 + (lane >> 4);
            ldmatrix_x4_trans(b, vt_s + j * D + ((c ^ (j & 7)) * 8));
            mma_bf16(o[2 * d2], a, b[0], b[1]);
            mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();   // every warp is done with the key tiles: their memory becomes o_red

    // ---- merge the four warps (each saw a quarter of the keys)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        if (t4 == 0) {
            ml_red[warp][g + h * 8][0] = m[h];
            ml_red[warp][g + h * 8][1] = l[h];
        }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + h * 8;
        float big = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) big = fmaxf(big, ml_red[w][r][0]);
        const float mine = m[h] > -INFINITY ? fast_exp2(m[h] - big) : 0.f;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            float2 v = make_float2(o[i][2 * h] * mine, o[i][2 * h + 1] * mine);
            *reinterpret_cast<float2*>(o_red + (warp * 16 + r) * D + i * 8 + 2 * t4) = v;
        }
    }
    __syncthreads();
    // 128 threads: thread -> (row = tid / 8, 8 threads across D)
    {
        const int r = tid >> 3;
        const int tok = r / group, hg = r - tok * group;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + kvh * group + hg;
        float big = -INFINITY, sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) big = fmaxf(big, ml_red[w][r][0]);
#pragma unroll
        for (int w = 0; w < 4; ++w)
            if (ml_red[w][r][0] > -INFINITY) sum += ml_red[w][r][1] * fast_exp2(ml_red[w][r][0] - big);
        if (r < rows) {
            for (int c = (tid & 7); c < D; c += 8) {
                const float v = o_red[(0 * 16 + r) * D + c] + o_red[(1 * 16 + r) * D + c] +
                                o_red[(2 * 16 + r) * D + c] + o_red[(3 * 16 + r) * D + c];
                if (num_splits == 1)
                    out[flat * D + c] = __float2bfloat16_rn(sum > 0.f ? v / sum : 0.f);
                else
                    part_acc[(flat * num_splits + split) * D + c] = v;
            }
            if (num_splits > 1 && (tid & 7) == 0) {
                part_ml[(flat * num_splits + split) * 2] = big * 0.6931471805599453f;
                part_ml[(flat * num_splits + split) * 2 + 1] = sum;
            }
        }
    }
    if (num_splits == 1 || counters == nullptr) return;

    // ---- the last block of this (sequence, KV head) merges the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int ticket = atomicAdd(&counters[seq * n_kv + kvh], 1);
        last_flag = ticket == num_splits - 1;
        if (last_flag) counters[seq * n_kv + kvh] = 0;   // ready for the next launch
    }
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    // weights of the splits per row, then the weighted sum with independent loads
    float* wz = o_red;                      // [16][64] reuses the tile memory once more
    const int r = tid >> 3, j = tid & 7;
    const int tok = r / group, hg = r - tok * group;
    const int64_t flat = (int64_t)(q_begin + (r < rows ? tok : 0)) * n_q + kvh * group +
                         (r < rows ? hg : 0);
    __syncthreads();                        // o_red is no longer read by anyone
    for (int z = j; z < num_splits; z += 8)
        wz[r * 64 + z] = __ldcg(part_ml + (flat * num_splits + z) * 2);
    __syncthreads();
    float big = -INFINITY;
    for (int z = 0; z < num_splits; ++z) big = fmaxf(big, wz[r * 64 + z]);
    __syncthreads();
    for (int z = j; z < num_splits; z += 8) {
        const float mz = wz[r * 64 + z];
        const float lz = __ldcg(part_ml + (flat * num_splits + z) * 2 + 1);
        wz[r * 64 + z] = mz > -INFINITY ? expf(mz - big) : 0.f;
        wz[16 * 64 + r * 64 + z] = mz > -INFINITY ? lz * expf(mz - big) : 0.f;
    }
    __syncthreads();
    if (r >= rows) return;
    float denom = 0.f;
    for (int z = 0; z < num_splits; ++z) denom += wz[16 * 64 + r * 64 + z];
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    // thread j of a row owns columns [j * D/8, (j + 1) * D/8)
    constexpr int COLS = D / 8;
    float acc[COLS];
#pragma unroll
    for (int c = 0; c < COLS; ++c) acc[c] = 0.f;
#pragma unroll 4
    for (int z = 0; z < num_splits; ++z) {
        const float w = wz[r * 64 + z];
        const float4* src =
            reinterpret_cast<const float4*>(part_acc + (flat * num_splits + z) * D + j * COLS);
#pragma unroll
        for (int c4 = 0; c4 < COLS / 4; ++c4) {
            const float4 v = __ldcg(src + c4);
            acc[4 * c4] += w * v.x;
            acc[4 * c4 + 1] += w * v.y;
            acc[4 * c4 + 2] += w * v.z;
            acc[4 * c4 + 3] += w * v.w;
        }
    }
#pragma unroll
    for (int c = 0; c < COLS; c += 2)
        *reinterpret_cast<__nv_bfloat162*>(out + flat * D + j * COLS + c) =
            __floats2bfloat162_rn(acc[c] * inv, acc[c + 1] * inv);
}

// The decode kernel once more, for up to eight key ranges per (sequence, KV head): the
// blocks of one (sequence, KV head) form a thread-block cluster. Two things take the keys
// off the critical path of a captured decode step. (1) Everything a block needs of the
// cache except the tile with the newest key is copied into shared memory BEFORE the block
// waits for the kernel in front (which writes only the newest key and the queries), so that
// after the wait only the queries, and in one block of the cluster one tile, are fetched.
// (2) The ranges are merged through distributed shared memory: each block finishes a share
// of the rows. With head size 64 every block writes its (maximum, sum, output) of a row
// into the shared memory of the block that finishes the row, and after one cluster barrier
// each block works from its own memory and leaves. With head size 128 (where that landing
// area would cost the second block per SM) every block keeps its result, and after a cluster
// barrier each block reads its rows from all the others' memories; a second barrier keeps
// the memories alive meanwhile. Nothing goes through global memory, and there is no ticket.
// FED: the key and value tiles come by TMA (one copy per page, 128-byte swizzle, which is the
// layout the fragments are read in) issued by lanes of warp 0 and awaited on one mbarrier per
// stage, instead of 16 bytes per thread and instruction. For blocks that walk many tiles
// (large batches) the per-thread copies were the limit: issuing a tile's 8 cp.async took a
// thread 780 of the 2080 cycles a tile took. Head size 64, pages of 8 tokens or more.
// TWO: the step's query rows (tokens x heads of the group) are more than 8 and take a second
// column tile of the transposed products.
// STG: stages of 64 keys in shared memory (not FED). Head size 128 has three when two blocks
// are to share an SM and five when the blocks are few: five tiles are what a block of a small
// batch walks at 2048-token contexts, and with all of them in shared memory before the kernel
// in front is done nothing is copied inside the loop (16 copies of 16 bytes per thread and
// tile there: some 2000 cycles a tile).
template <int D, bool FED, bool TWO, int STG>
__global__ void __launch_bounds__(FED ? 160 : 128)
attention_decode_cluster_kernel(const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v,
                                const __nv_bfloat16* __restrict__ qkv, int q_row_stride,
                                const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages,
                                const int* __restrict__ table, int max_pages,
                                const int* __restrict__ q_start, const int* __restrict__ kv_len_of,
                                __nv_bfloat16* __restrict__ out, int n_q, int n_kv, int page_size,
                                float scale, int window, const float* __restrict__ cos_t,
                                const float* __restrict__ sin_t, int raw, int store,
                                int* __restrict__ error) {
    // raw: q, k and v in `qkv` are the projection as it came out of the product (bias added,
    // not rotated, nothing stored): this kernel rotates the queries as it loads them, and the
    // block whose key range holds this step's positions rotates the new keys, writes them and
    // the new values into the pages (if `store`) and into its own tiles. The product in front
    // then needs no block per head, and every tile of the pages can be copied before the wait.
    constexpr int CH = D / 8;
    // (FED: STG counts half stages, see below)
    constexpr int STAGES = FED ? 4 : STG;
    __nv_bfloat16* k_pages_out = const_cast<__nv_bfloat16*>(k_pages);
    __nv_bfloat16* v_pages_out = const_cast<__nv_bfloat16*>(v_pages);
    __shared__ __align__(16) __nv_bfloat16 new_k[16][D]; // this step's keys, rotated
    __shared__ __align__(16) __nv_bfloat16 new_v[16][D];
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // (TMA's swizzle goes by the address: the tiles then start on a 1024-byte boundary)
    unsigned char* smem_base = FED ? reinterpret_cast<unsigned char*>(
                                         (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023)
                                   : smem_raw;
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_base);     // [16][D]
    // FED: STG half stages of 32 keys, two per consumer warp, or one where two blocks of head
    // size 128 are to fit an SM; a head of 128 features lies as two sub-tiles of 64, each
    // 128-byte swizzled, the form in which TMA leaves a box of 64 features
    constexpr int HALF = MMA_BN / 2, HDEPTH = FED ? STG / 4 : 1, HSTAGES = 4 * HDEPTH;
    constexpr bool SUBTILED = FED && D > 64;
    constexpr int KV_ELEMS = FED ? HSTAGES * HALF * D : STAGES * MMA_BN * D;
    __nv_bfloat16* k_s = q_s + 16 * D;                                    // [STAGES][64][D]
    __nv_bfloat16* v_s = k_s + KV_ELEMS;                                  // [STAGES][64][D]
    // where row j, 16-byte piece c of a key (or value) tile lies
    auto piece_at = [&](const __nv_bfloat16* tile, int j, int c) -> const __nv_bfloat16* {
        if (SUBTILED) return tile + (c >> 3) * (HALF * 64) + j * 64 + (((c & 7) ^ (j & 7)) * 8);
        return tile + j * D + ((c ^ (j & 7)) * 8);
    };
    // (rows of D + 4 floats: the warps write their pieces of O^T column by column, and with
    // this stride the 32 lanes of a store fall into 32 banks)
    constexpr int OR = D + 4;
    float* o_red = reinterpret_cast<float*>(k_s);                         // [4][16][OR], after the loop
    float* o_part = o_red + 4 * 16 * OR;                                  // [16][D], this block's result
    // where the other blocks leave their results for this block's rows (head size 64 only):
    // [range][row of this block][D], then [range][row of this block][maximum, sum]; no
    // other use, since a block that is done early writes here while this one still runs
    constexpr bool PUSH = D == 64;
    float* land_o = reinterpret_cast<float*>(v_s + KV_ELEMS);
    float* land_ml = land_o + 16 * D;
    __shared__ float ml_red[4][16][2];
    __shared__ float ml_part[16][2];                                      // row maximum (log2 units), sum
    // The block table of this block's key range, a window of it at a time: a table entry
    // read from global memory inside the key loop puts a trip to L2 in front of every tile's
    // copies (with 16 tiles per block that trip, not the copies, set the kernel's time).
    constexpr int PAGE_WINDOW = 256;
    __shared__ int page_s[PAGE_WINDOW];
    __shared__ uint64_t tile_full[HSTAGES];      // FED: a half stage's copies have landed
    __shared__ uint64_t tile_free[HSTAGES];      // FED: its warp has read it
    __shared__ uint32_t tile_pages[HSTAGES];     // FED: which of its pages were there
    __shared__ int fed_error;                    // FED: a wait gave up (never read by the host:
                                                 // the block then leaves its rows unwritten)

    uint32_t split, num_splits;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(split));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(num_splits));
    const int seq = blockIdx.x, kvh = blockIdx.y;
    const int group = n_q / n_kv;
    // lengths and block tables were copied to the device before the step began
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    if (q_len <= 0) return;                  // the same for every block of the cluster
    const int rows = q_len * group;          // <= 16
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int p_min = first_pos, p_max = kv_len - 1;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / MMA_BN;
    int t_hi = p_max / MMA_BN + 1;
    // tiles that hold a key of this step: written by the kernel in front
    const int t_new = first_pos / MMA_BN;
    {
        const int per = (t_hi - t_lo + (int)num_splits - 1) / (int)num_splits;
        t_lo = t_lo + (int)split * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }
    const int n_tiles = t_hi > t_lo ? t_hi - t_lo : 0;

    // tiles [window_lo, window_lo + window_tiles) have their table entries in page_s
    // (pages of 2 or more tokens: at least 8 tiles, which covers the stages filled up front;
    // pages larger than a tile share an entry between tiles, two entries are kept spare)
    // (a page holds a power of two of tokens: shifts and masks, since an integer division
    // costs a thread some hundred cycles and the tile loop had four of them per tile)
    const int page_shift = 31 - __clz(page_size), page_mask = page_size - 1;
    const int window_tiles = page_size >= MMA_BN ? PAGE_WINDOW - 2 : PAGE_WINDOW >> (6 - page_shift);
    int window_lo = t_lo;
    auto fill_window = [&](int first_tile) {
        window_lo = first_tile;
        const int base = (first_tile * MMA_BN) >> page_shift;
        // (FED: by the threads that load neither queries nor new keys, so that all three
        // trips to L2 are under way at once)
        for (int e = FED ? tid - 96 : tid; e < PAGE_WINDOW; e += (FED ? 64 : 128)) {
            if (e < 0) continue;
            const int column = base + e;
            page_s[e] = (column < max_pages && ((int64_t)column << page_shift) < kv_len)
                            ? table_page(table, seq, max_pages, column) : -1;
        }
    };
    // FED: this form is never launched ahead of the kernel in front (large batches are not
    // captured with dependent launch), so nothing is gained by putting work before the wait:
    // it waits first, and then queries, new keys and the block table are fetched side by side
    // by different warps, with one barrier of the block before the loop instead of two.
    if (FED) grid_dependency_sync();
    fill_window(t_lo);
    if (FED && tid == 0) {
        for (int st = 0; st < HSTAGES; ++st) {
            mbar_init(&tile_full[st], 1);   // the arrival that announces the bytes
            mbar_init(&tile_free[st], 1);   // lane 0 of the warp that read it
        }
        fed_error = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (!FED) __syncthreads();

    // each thread copies half a key row of K and of V
    const int lj = tid >> 1, lc0 = (tid & 1) * (CH / 2);
    // FED: a copy brings `box` keys (a page, or 64 keys of a larger one)
    const int box = FED ? (page_size < HALF ? page_size : HALF) : (page_size < MMA_BN ? page_size : MMA_BN);
    const int box_shift = 31 - __clz(box);
    auto load_tile = [&](int stage, int kt) {
        if (FED) return;     // (the producer warp's copies: fetch_round below)
        const int key = kt * MMA_BN + lj;
        int page = -1;
        if (key < kv_len && !(raw && key >= first_pos))
            page = page_s[(key >> page_shift) - ((window_lo * MMA_BN) >> page_shift)];
        const bool valid = page >= 0;
        const int64_t at =
            valid ? ((((int64_t)page * n_kv + kvh) << page_shift) + (key & page_mask)) * D : 0;
        __nv_bfloat16* kd = k_s + (stage * MMA_BN + lj) * D;
        __nv_bfloat16* vd = v_s + (stage * MMA_BN + lj) * D;
#pragma unroll
        for (int c = 0; c < CH / 2; ++c) {
            const int sw = ((lc0 + c) ^ (lj & 7)) * 8;
            cp_async_16(kd + sw, k_pages + at + (lc0 + c) * 8, valid);
            cp_async_16(vd + sw, v_pages + at + (lc0 + c) * 8, valid);
        }
    };

    // FED: the producer warp's copies of a round of half tiles (32 keys each; half tile h of the
    // block belongs to consumer warp h % 4, whose two half stages alternate, and round r is
    // the half tiles 4 r .. 4 r + 3). One lane per page (or half page) and half tile: a copy
    // costs its warp some hundred cycles however many lanes issue it, so a round goes out in
    // one instruction per tensor. `reuse`: wait until each stage's warp has read what was there.
    const int keys_end = kv_len < t_hi * MMA_BN ? kv_len : t_hi * MMA_BN;
    const int n_half = FED && keys_end > t_lo * MMA_BN ? (keys_end - t_lo * MMA_BN + HALF - 1) / HALF : 0;
    auto fetch_round = [&](int r, bool reuse) -> bool {
        const int copies_shift = 5 - box_shift;              // copies per half tile: 1, 2 or 4
        const int w = lane >> copies_shift, piece = lane & ((1 << copies_shift) - 1);
        const int h = 4 * r + w;
        const bool active = w < 4 && h < n_half;
        const int hs = (w & 3) + 4 * (r % HDEPTH);
        bool ok = true;
        if (active && reuse)
            ok = mbar_wait(&tile_free[hs], (uint32_t)((r / HDEPTH - 1) & 1), error ? error : &fed_error, 8);
        if (!__all_sync(0xffffffffu, ok)) return false;
        int page = -1, row = 0;
        if (active) {
            const int key0 = t_lo * MMA_BN + h * HALF + (piece << box_shift);
            if (key0 < kv_len) {
                const int column = key0 >> page_shift;
                const int e = column - ((window_lo * MMA_BN) >> page_shift);
                // (beyond the window of the table in shared memory: from the table itself)
                page = e < PAGE_WINDOW ? page_s[e]
                                       : (column < max_pages ? table_page(table, seq, max_pages, column) : -1);
            }
            if (page >= 0) row = ((page * n_kv + kvh) << page_shift) + (key0 & page_mask);
        }
        const unsigned valid = __ballot_sync(0xffffffffu, page >= 0);
        if (active && piece == 0) {
            const unsigned mine = (valid >> (w << copies_shift)) & ((1u << (1 << copies_shift)) - 1u);
            tile_pages[hs] = mine;
            // (a copy brings `box` keys of 2 D bytes, of K and of V)
            mbar_expect_tx(&tile_full[hs], (uint32_t)(__popc(mine) << box_shift) * (4u * D));
        }
        __syncwarp();
        if (page >= 0) {
#pragma unroll
            for (int sb = 0; sb < D / 64; ++sb) {
                const int to = hs * HALF * D + sb * (HALF * 64) + (piece << box_shift) * 64;
                tma_load_2d(k_s + to, &map_k, sb * 64, row, &tile_full[hs]);
                tma_load_2d(v_s + to, &map_v, sb * 64, row, &tile_full[hs]);
            }
        }
        return true;
    };

    // ---- before the wait: the first STAGES tiles, one copy group each (an empty group for a
    // tile that is not there or holds keys of this step)
#pragma unroll
    for (int st = 0; st < STAGES; ++st) {
        const int kt = t_lo + st;
        if (!FED && kt < t_hi && (kt < t_new || raw)) load_tile(st, kt);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    // raw: which piece of this step's keys and values this thread will turn and store (threads
    // other than the ones that load the queries, where there are any: the two loads then
    // travel together), and its page, looked up now
    constexpr int HC = CH / 2;             // 16-byte pieces in half a head
    const int new_idx = (tid + 128 - (16 * HC) % 128) % 128;
    int new_tok = 0, new_c = 0, new_page = -1;
    bool new_mine = false;
    if (raw && tid < 128 && new_idx < q_len * HC) {
        new_tok = new_idx / HC;
        new_c = new_idx - new_tok * HC;
        const int key = first_pos + new_tok, kt = key / MMA_BN;
        new_mine = kt >= t_lo && kt < t_hi;
        if (new_mine && store) new_page = table_page(table, seq, max_pages, key >> page_shift);
    }
    if (!FED) grid_dependency_sync();

    // ---- after it: the queries, and the tiles of the first STAGES that had to wait
    if (!raw) {
        for (int idx = tid; idx < 16 * CH; idx += 128) {
            const int r = idx / CH, c = idx - r * CH;
            const int tok = r / group, hg = r - tok * group;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (r < rows)
                val = *reinterpret_cast<const uint4*>(qkv + (int64_t)(q_begin + tok) * q_row_stride +
                                                      (kvh * group + hg) * D + c * 8);
            *reinterpret_cast<uint4*>(q_s + r * D + ((c ^ (r & 7)) * 8)) = val;
        }
#pragma unroll
        for (int st = 0; st < STAGES; ++st) {
            const int kt = t_lo + st;
            if (!FED && kt < t_hi && kt >= t_new) load_tile(st, kt);
        }
    } else {
        // (the angles are read beside the values they turn: the same trip to L2)
        const bool rotate = cos_t != nullptr;
        // eight pairs (i, i + D/2) at a time: 16 bytes of each half of the head, rotated in
        // float32 with the angles of the token's position, rounded once
        auto turn8 = [&](const __nv_bfloat16* head, int pos_of, int c, uint4& lo, uint4& hi) {
            lo = *reinterpret_cast<const uint4*>(head + c * 8);
            hi = *reinterpret_cast<const uint4*>(head + D / 2 + c * 8);
            if (!rotate) return;
            pos_of = checked_position(pos_of);
            const float4* cs = reinterpret_cast<const float4*>(cos_t + (int64_t)pos_of * (D / 2) + c * 8);
            const float4* sn = reinterpret_cast<const float4*>(sin_t + (int64_t)pos_of * (D / 2) + c * 8);
            const float4 c0 = cs[0], c1 = cs[1], s0 = sn[0], s1 = sn[1];
            const float cc[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float ss[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&lo);
            __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&hi);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float x = __bfloat162float(a[e]), y = __bfloat162float(b[e]);
                a[e] = __float2bfloat16_rn(x * cc[e] - y * ss[e]);
                b[e] = __float2bfloat16_rn(y * cc[e] + x * ss[e]);
            }
        };
        for (int idx = tid; idx < 16 * HC; idx += 128) {
            const int r = idx / HC, c = idx - r * HC;
            const int tok = r / group, hg = r - tok * group;
            uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
            if (r < rows)
                turn8(qkv + (int64_t)(q_begin + tok) * q_row_stride + (kvh * group + hg) * D,
                      first_pos + tok, c, lo, hi);
            *reinterpret_cast<uint4*>(q_s + r * D + ((c ^ (r & 7)) * 8)) = lo;
            *reinterpret_cast<uint4*>(q_s + r * D + (((c + HC) ^ (r & 7)) * 8)) = hi;
        }
        // this step's keys and values, if their tiles are this block's: rotated keys and the
        // values into shared memory (they are put into their tiles when those come up) and
        // into the pages
        if (new_mine) {
            const int tok = new_tok, c = new_c;
            const int key = first_pos + tok;
            const __nv_bfloat16* src = qkv + (int64_t)(q_begin + tok) * q_row_stride + (n_q + kvh) * D;
            uint4 klo, khi;
            turn8(src, key, c, klo, khi);
            const uint4 vlo = *reinterpret_cast<const uint4*>(src + n_kv * D + c * 8);
            const uint4 vhi = *reinterpret_cast<const uint4*>(src + n_kv * D + D / 2 + c * 8);
            *reinterpret_cast<uint4*>(&new_k[tok][c * 8]) = klo;
            *reinterpret_cast<uint4*>(&new_k[tok][D / 2 + c * 8]) = khi;
            *reinterpret_cast<uint4*>(&new_v[tok][c * 8]) = vlo;
            *reinterpret_cast<uint4*>(&new_v[tok][D / 2 + c * 8]) = vhi;
            if (store) {
                const int page = new_page;
                if (page >= 0) {
                    const int64_t at = ((((int64_t)page * n_kv + kvh) << page_shift) + (key & page_mask)) * D;
                    *reinterpret_cast<uint4*>(k_pages_out + at + c * 8) = klo;
                    *reinterpret_cast<uint4*>(k_pages_out + at + D / 2 + c * 8) = khi;
                    *reinterpret_cast<uint4*>(v_pages_out + at + c * 8) = vlo;
                    *reinterpret_cast<uint4*>(v_pages_out + at + D / 2 + c * 8) = vhi;
                }
            }
        }
    }
    asm volatile("cp.async.commit_group;\n" ::);

    // The products run transposed: S^T = K Q^T and O^T = V^T P^T, keys (or the head's
    // dimensions) along the 16 rows of an MMA and the step's query rows along its 8 columns.
    // A decode step of a group of up to 8 query heads then needs one column tile where the
    // untransposed form spent a 16-row tile on 7 rows, and mma.sync is the scarce unit here:
    // an m16n8k16 issues about every 40 cycles per scheduler on this GPU, so a 64-key tile cost
    // a warp some 700 cycles of MMAs alone. A thread holds, of a 16 x 8 piece, rows g and g + 8
    // (keys) and columns 2 t4 and 2 t4 + 1 (query rows).
    constexpr bool two = TWO;                // a second column tile of query rows
    int pos[2][2];
    bool row_ok[2][2];
#pragma unroll
    for (int nr = 0; nr < 2; ++nr) {
#pragma unroll
        for (int z = 0; z < 2; ++z) {
            const int r = nr * 8 + 2 * t4 + z;
            row_ok[nr][z] = r < rows;
            pos[nr][z] = first_pos + r / group;
        }
    }
    float o[D / 16][2][4];                   // O^T: [dimension tile][row tile]
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
#pragma unroll
        for (int nr = 0; nr < 2; ++nr) o[i][nr][0] = o[i][nr][1] = o[i][nr][2] = o[i][nr][3] = 0.f;
    }
    float m[2][2] = {{-INFINITY, -INFINITY}, {-INFINITY, -INFINITY}}, l[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    const float scale2 = scale * 1.4426950408889634f;

    // no more tiles than stages: every tile was asked for before the wait (or, a tile with
    // this step's keys that the kernel in front writes, right after it) and none is refilled,
    // so one wait and the barrier below stand for the per-tile ones
    const bool resident = !FED && n_tiles <= STAGES;
    if (resident) asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();
    if (FED && warp == 4) {
        // the first rounds (the block table and the barriers are there now)
        for (int r = 0; r < HDEPTH && 4 * r < n_half; ++r) fetch_round(r, false);
    }
    uint32_t qf[D / 16][4];                  // Q as the B operand: [0], [1] rows 0..7, [2], [3] rows 8..15
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int r = (lane & 7) + (lane >> 4) * 8;
        const int c = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(qf[ks], q_s + r * D + ((c ^ (r & 7)) * 8));
    }

    // scores of the 16 keys from row `j0` of a tile on
    auto unit_scores = [&](const __nv_bfloat16* kt_s, int j0, float (&sc)[2][4]) {
#pragma unroll
        for (int nr = 0; nr < 2; ++nr) sc[nr][0] = sc[nr][1] = sc[nr][2] = sc[nr][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t a[4];
            const int j = j0 + (lane & 15);
            const int c = ks * 2 + (lane >> 4);
            ldmatrix_x4(a, piece_at(kt_s, j, c));
            mma_bf16(sc[0], a, qf[ks][0], qf[ks][1]);
            if (two) mma_bf16(sc[1], a, qf[ks][2], qf[ks][3]);
        }
    };
    // scale and mask the unit's scores (keys from `key_lo` on) and raise `top` to their maxima.
    // Every key of the 16 is seen by every row when the newest of them is no later than the
    // earliest position of the step, real, and inside every row's window (rows beyond the
    // step's are zeros and go nowhere): then nothing is masked one by one.
    auto unit_mask = [&](float (&sc)[2][4], int key_lo, float (&top)[2][2]) {
        const bool plain = key_lo + 15 <= first_pos && key_lo + 15 < kv_len &&
                           (window <= 0 || key_lo > p_max - window);
#pragma unroll
        for (int nr = 0; nr < 2; ++nr) {
            if (nr == 1 && !two) continue;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int z = e & 1;
                bool seen = true;
                if (!plain) {
                    const int key = key_lo + g + (e >> 1) * 8;
                    seen = row_ok[nr][z] && key <= pos[nr][z] && key < kv_len;
                    if (window > 0) seen = seen && key > pos[nr][z] - window;
                }
                sc[nr][e] = seen ? sc[nr][e] * scale2 : -INFINITY;
                top[nr][z] = fmaxf(top[nr][z], sc[nr][e]);
            }
        }
    };
    // the maxima of a row over the keys of all lanes that hold it (lanes of one t4)
    auto across_keys_max = [&](float (&top)[2][2]) {
#pragma unroll
        for (int nr = 0; nr < 2; ++nr) {
            if (nr == 1 && !two) continue;
#pragma unroll
            for (int z = 0; z < 2; ++z) {
                top[nr][z] = fmaxf(top[nr][z], __shfl_xor_sync(0xffffffffu, top[nr][z], 4));
                top[nr][z] = fmaxf(top[nr][z], __shfl_xor_sync(0xffffffffu, top[nr][z], 8));
                top[nr][z] = fmaxf(top[nr][z], __shfl_xor_sync(0xffffffffu, top[nr][z], 16));
            }
        }
    };
    // probabilities on the rows' maxima, their sums, and O^T += V^T P^T for the unit
    auto unit_values = [&](float (&sc)[2][4], const __nv_bfloat16* vt_s, int j0) {
        uint32_t pt[2][2];
#pragma unroll
        for (int nr = 0; nr < 2; ++nr) {
            if (nr == 1 && !two) continue;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int z = e & 1;
                const float p = m[nr][z] > -INFINITY ? fast_exp2(sc[nr][e] - m[nr][z]) : 0.f;
                sc[nr][e] = p;
                l[nr][z] += p;
            }
            // P^T as the B operand: the 8 x 8 pieces [keys][rows] turned into [rows][keys]
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const uint32_t piece = pack_bf16(sc[nr][2 * half], sc[nr][2 * half + 1]);
                asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(pt[nr][half]) : "r"(piece));
            }
        }
#pragma unroll
        for (int d2 = 0; d2 < D / 16; ++d2) {
            uint32_t a[4];
            const int j = j0 + (lane & 7) + (lane >> 4) * 8;
            const int c = d2 * 2 + ((lane >> 3) & 1);
            ldmatrix_x4_trans(a, piece_at(vt_s, j, c));
            mma_bf16(o[d2][0], a, pt[0][0], pt[0][1]);
            if (two) mma_bf16(o[d2][1], a, pt[1][0], pt[1][1]);
        }
    };

    if (resident) {
        // Every tile is in shared memory. The warps then share the keys by runs instead of
        // every warp taking a quarter of every tile: a warp takes n_tiles consecutive units
        // of 16 keys, computes all its scores, goes through the softmax once and then through
        // P V, so that its MMAs are independent chains and nothing is rescaled.
        if (raw && t_new < t_hi) {
            // this step's keys and values take their rows of their tiles (the copies left zeros)
            for (int idx = tid; idx < q_len * CH; idx += 128) {
                const int tok = idx / CH, c = idx - tok * CH;
                const int key = first_pos + tok, kt = key / MMA_BN;
                if (kt < t_lo || kt >= t_hi) continue;
                const int row = key % MMA_BN;
                const int sw = (c ^ (row & 7)) * 8;
                *reinterpret_cast<uint4*>(k_s + ((kt - t_lo) * MMA_BN + row) * D + sw) =
                    *reinterpret_cast<const uint4*>(&new_k[tok][c * 8]);
                *reinterpret_cast<uint4*>(v_s + ((kt - t_lo) * MMA_BN + row) * D + sw) =
                    *reinterpret_cast<const uint4*>(&new_v[tok][c * 8]);
            }
            __syncthreads();
        }
        constexpr int UPW = STAGES;          // units per warp: n_tiles of them, at most STAGES
        const int u_lo = warp * n_tiles;
        float sc[UPW][2][4];
#pragma unroll
        for (int u = 0; u < UPW; ++u) {
#pragma unroll
            for (int nr = 0; nr < 2; ++nr) sc[u][nr][0] = sc[u][nr][1] = sc[u][nr][2] = sc[u][nr][3] = 0.f;
        }
        // (slice of the head by slice, all units in each: consecutive MMAs are independent)
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t a[UPW][4];
#pragma unroll
            for (int u = 0; u < UPW; ++u) {
                if (u < n_tiles) {
                    const int unit = u_lo + u;
                    const int j = (unit & 3) * 16 + (lane & 15);
                    const int c = ks * 2 + (lane >> 4);
                    ldmatrix_x4(a[u], piece_at(k_s + (unit >> 2) * MMA_BN * D, j, c));
                }
            }
#pragma unroll
            for (int u = 0; u < UPW; ++u) {
                if (u < n_tiles) {
                    mma_bf16(sc[u][0], a[u], qf[ks][0], qf[ks][1]);
                    if (two) mma_bf16(sc[u][1], a[u], qf[ks][2], qf[ks][3]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UPW; ++u) {
            if (u < n_tiles)
                unit_mask(sc[u], (t_lo + ((u_lo + u) >> 2)) * MMA_BN + ((u_lo + u) & 3) * 16, m);
        }
        across_keys_max(m);
#pragma unroll
        for (int u = 0; u < UPW; ++u) {
            if (u < n_tiles) {
                const int unit = u_lo + u;
                unit_values(sc[u], v_s + (unit >> 2) * MMA_BN * D, (unit & 3) * 16);
            }
        }
    }

    if (FED && warp == 4) {
        // ---- the producer warp: a round's half tiles go into their half stages as soon as the
        // warps that own the stages have read what was there (two rounds earlier)
        for (int r = HDEPTH; 4 * r < n_half; ++r)
            if (!fetch_round(r, true)) break;
    } else if (FED) {
        // ---- Many tiles per block: every consumer warp walks half tiles of its own (warp w
        // takes the block's half tiles w, w + 4, ...) through two half stages of its own. It
        // waits for its half tile, goes through the two units of 16 keys side by side and hands
        // the half stage back to the producer warp, so that no barrier of the block stands in
        // the loop, the copies are nobody's detour, and while a warp waits the others work.
        for (int h = warp; h < n_half; h += 4) {
            const int hs = warp + 4 * ((h >> 2) % HDEPTH);
            const int key_base = t_lo * MMA_BN + h * HALF;
            // (bounded like every mbarrier wait of this library; a wait that gives up sets
            // the error word and the warp goes on with whatever the stage holds)
            mbar_wait(&tile_full[hs], (uint32_t)(((h >> 2) / HDEPTH) & 1), error ? error : &fed_error, 8);
            __nv_bfloat16* kt_s = k_s + hs * HALF * D;
            __nv_bfloat16* vt_s = v_s + hs * HALF * D;
            if (raw && key_base + HALF > first_pos) {
                // this step's keys and values take their rows of the half tile
                for (int idx = lane; idx < q_len * CH; idx += 32) {
                    const int tok = idx / CH, c = idx - tok * CH;
                    const int row = first_pos + tok - key_base;
                    if (row < 0 || row >= HALF) continue;
                    *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(piece_at(kt_s, row, c))) =
                        *reinterpret_cast<const uint4*>(&new_k[tok][c * 8]);
                    *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(piece_at(vt_s, row, c))) =
                        *reinterpret_cast<const uint4*>(&new_v[tok][c * 8]);
                }
            }
            // A copy brings whole pages and nothing for a page that is not there: value rows
            // beyond the sequence or of a missing page are cleared before P V meets them
            // (0 x NaN).
            if (key_base + HALF > kv_len || tile_pages[hs] != (1u << (HALF >> box_shift)) - 1u) {
                const int key = key_base + lane;
                const bool there = key < kv_len && ((tile_pages[hs] >> (lane >> box_shift)) & 1u);
                if (!there) {
                    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int c = 0; c < CH; ++c)
                        *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(piece_at(vt_s, lane, c))) = zero;
                }
            }
            __syncwarp();
            float sc[2][2][4];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int nr = 0; nr < 2; ++nr) sc[u][nr][0] = sc[u][nr][1] = sc[u][nr][2] = sc[u][nr][3] = 0.f;
            }
            // (slice of the head by slice, both units in each: consecutive MMAs are independent)
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[2][4];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int j = u * 16 + (lane & 15);
                    const int c = ks * 2 + (lane >> 4);
                    ldmatrix_x4(a[u], piece_at(kt_s, j, c));
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    mma_bf16(sc[u][0], a[u], qf[ks][0], qf[ks][1]);
                    if (two) mma_bf16(sc[u][1], a[u], qf[ks][2], qf[ks][3]);
                }
            }
            float m_new[2][2] = {{m[0][0], m[0][1]}, {m[1][0], m[1][1]}};
#pragma unroll
            for (int u = 0; u < 2; ++u) unit_mask(sc[u], key_base + u * 16, m_new);
            across_keys_max(m_new);
            // the running sums and the output move to a new maximum only when some row has one
            if (__any_sync(0xffffffffu, m_new[0][0] > m[0][0] || m_new[0][1] > m[0][1] ||
                                            m_new[1][0] > m[1][0] || m_new[1][1] > m[1][1])) {
#pragma unroll
                for (int nr = 0; nr < 2; ++nr) {
                    float corr[2];
#pragma unroll
                    for (int z = 0; z < 2; ++z) {
                        corr[z] = m_new[nr][z] > -INFINITY ? fast_exp2(m[nr][z] - m_new[nr][z]) : 1.f;
                        m[nr][z] = m_new[nr][z];
                        l[nr][z] *= corr[z];
                    }
#pragma unroll
                    for (int i = 0; i < D / 16; ++i) {
                        o[i][nr][0] *= corr[0];
                        o[i][nr][1] *= corr[1];
                        o[i][nr][2] *= corr[0];
                        o[i][nr][3] *= corr[1];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) unit_values(sc[u], vt_s, u * 16);
            // the half tile has been read (its fragments are in registers and used) and the
            // rows this warp wrote are ordered before the copy that will overwrite them
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tile_free[hs])) : "memory");
        }
    }

    // Copy groups in the order they were committed: tiles 0 .. STAGES-1, the late group, then
    // one refill per iteration from the second on. A tile of this step's keys may sit in the
    // late group: it waits for everything; any other tile is older than the newest
    // STAGES - 2 groups when its turn comes.
    for (int it = 0; it < n_tiles && !resident && !FED; ++it) {
        const int kt = t_lo + it;
        const int stage = it % STAGES;
        {
            if (kt >= t_new && !raw) {
                asm volatile("cp.async.wait_group 0;\n" ::);
            } else {
                asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
            }
            __syncthreads();   // tile `it` has landed for everyone; the stage of tile it-1 is free
        }
        auto refill = [&]() {
            const int next = it - 1 + STAGES;
            if (next < n_tiles && t_lo + next >= window_lo + window_tiles) {
                // the window has been used up: everyone is past the barrier above, so nobody
                // reads it any more; the next stretch of the table takes its place
                fill_window(t_lo + next);
                __syncthreads();
            }
            if (next < n_tiles) load_tile((it - 1) % STAGES, t_lo + next);
            asm volatile("cp.async.commit_group;\n" ::);
        };
        if (it >= 1) refill();
        __nv_bfloat16* kt_s = k_s + stage * MMA_BN * D;
        __nv_bfloat16* vt_s = v_s + stage * MMA_BN * D;
        if (raw && kt >= t_new) {
            // this step's keys and values take their rows of the tile (the copy left zeros)
            for (int idx = tid; idx < q_len * CH; idx += 128) {
                const int tok = idx / CH, c = idx - tok * CH;
                const int key = first_pos + tok;
                if (key / MMA_BN != kt) continue;
                const int row = key % MMA_BN;
                const int sw = (c ^ (row & 7)) * 8;
                *reinterpret_cast<uint4*>(kt_s + row * D + sw) =
                    *reinterpret_cast<const uint4*>(&new_k[tok][c * 8]);
                *reinterpret_cast<uint4*>(vt_s + row * D + sw) =
                    *reinterpret_cast<const uint4*>(&new_v[tok][c * 8]);
            }
            __syncthreads();
        }

        // this warp's 16 keys of the tile
        float sc[2][4];
        unit_scores(kt_s, warp * 16, sc);
        float m_new[2][2] = {{m[0][0], m[0][1]}, {m[1][0], m[1][1]}};
        unit_mask(sc, kt * MMA_BN + warp * 16, m_new);
        across_keys_max(m_new);
        // the running sums and the output move to a new maximum only when some row of the
        // warp has one (after the first tiles that is rare)
        if (__any_sync(0xffffffffu, m_new[0][0] > m[0][0] || m_new[0][1] > m[0][1] ||
                                        m_new[1][0] > m[1][0] || m_new[1][1] > m[1][1])) {
#pragma unroll
            for (int nr = 0; nr < 2; ++nr) {
                float corr[2];
#pragma unroll
                for (int z = 0; z < 2; ++z) {
                    corr[z] = m_new[nr][z] > -INFINITY ? fast_exp2(m[nr][z] - m_new[nr][z]) : 1.f;
                    m[nr][z] = m_new[nr][z];
                    l[nr][z] *= corr[z];
                }
#pragma unroll
                for (int i = 0; i < D / 16; ++i) {
                    o[i][nr][0] *= corr[0];
                    o[i][nr][1] *= corr[1];
                    o[i][nr][2] *= corr[0];
                    o[i][nr][3] *= corr[1];
                }
            }
        }
        unit_values(sc, vt_s, warp * 16);
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    __syncthreads();   // every warp is done with the key tiles: their memory becomes o_red

    // ---- merge the four warps (each saw a quarter of the keys)
    if (!FED || warp < 4) {
#pragma unroll
    for (int nr = 0; nr < 2; ++nr) {
#pragma unroll
        for (int z = 0; z < 2; ++z) {
            l[nr][z] += __shfl_xor_sync(0xffffffffu, l[nr][z], 4);
            l[nr][z] += __shfl_xor_sync(0xffffffffu, l[nr][z], 8);
            l[nr][z] += __shfl_xor_sync(0xffffffffu, l[nr][z], 16);
            if (g == 0) {
                ml_red[warp][nr * 8 + 2 * t4 + z][0] = m[nr][z];
                ml_red[warp][nr * 8 + 2 * t4 + z][1] = l[nr][z];
            }
        }
    }
    // (each warp's output goes in as it is, on its own maximum; the weights that bring the
    // four onto the common maximum are applied where they are summed)
#pragma unroll
    for (int nr = 0; nr < 2; ++nr) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                o_red[(warp * 16 + nr * 8 + 2 * t4 + (e & 1)) * OR + i * 16 + g + (e >> 1) * 8] = o[i][nr][e];
        }
    }
    }
    __syncthreads();
    // 128 threads: thread -> (row = tid / 8, 8 threads across D)
    if (!FED || tid < 128) {
        const int r = tid >> 3;
        const int tok = r / group, hg = r - tok * group;
        float big = -INFINITY, sum = 0.f;
        float wgt[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) big = fmaxf(big, ml_red[w][r][0]);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            wgt[w] = ml_red[w][r][0] > -INFINITY ? fast_exp2(ml_red[w][r][0] - big) : 0.f;
            sum += ml_red[w][r][1] * wgt[w];
        }
        if (PUSH && num_splits > 1) {
            // row r is finished by block r / per_block: its landing slot for this range
            const int per_block = (16 + (int)num_splits - 1) / (int)num_splits;
            const uint32_t owner = (uint32_t)(r / per_block);
            const int slot = (int)split * per_block + (r - (int)owner * per_block);
            uint32_t dst_o, dst_ml;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                         : "=r"(dst_o)
                         : "r"((uint32_t)__cvta_generic_to_shared(land_o + slot * D)), "r"(owner));
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                         : "=r"(dst_ml)
                         : "r"((uint32_t)__cvta_generic_to_shared(land_ml + slot * 2)), "r"(owner));
            if (r < rows) {
                for (int c4 = (tid & 7); c4 < D / 4; c4 += 8) {
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float4 u = *reinterpret_cast<const float4*>(o_red + (w * 16 + r) * OR + 4 * c4);
                        v.x += wgt[w] * u.x;
                        v.y += wgt[w] * u.y;
                        v.z += wgt[w] * u.z;
                        v.w += wgt[w] * u.w;
                    }
                    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst_o + 16 * c4),
                                 "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                                 : "memory");
                }
                if ((tid & 7) == 0)
                    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(dst_ml), "f"(big), "f"(sum)
                                 : "memory");
            }
        } else {
            for (int c = (tid & 7); c < D; c += 8) {
                const float v = wgt[0] * o_red[(0 * 16 + r) * OR + c] + wgt[1] * o_red[(1 * 16 + r) * OR + c] +
                                wgt[2] * o_red[(2 * 16 + r) * OR + c] + wgt[3] * o_red[(3 * 16 + r) * OR + c];
                if (num_splits == 1) {
                    if (r < rows)
                        out[((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * D + c] =
                            __float2bfloat16_rn(sum > 0.f ? v / sum : 0.f);
                } else {
                    o_part[r * D + c] = v;
                }
            }
            if ((tid & 7) == 0) {
                ml_part[r][0] = big;
                ml_part[r][1] = sum;
            }
        }
    }
    if (num_splits == 1) return;

    if (PUSH) {
        // ---- the ranges have met in the memory of the blocks that finish them: after the
        // barrier (the writes above are released by the arrival) nobody touches another
        // block's memory again, so a block may leave as soon as its own rows are out
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int per_block = (16 + (int)num_splits - 1) / (int)num_splits;
        const int r_first = (int)split * per_block;
        for (int e = tid; e < per_block * D && tid < 128; e += 128) {
            const int r_local = e / D, c = e % D;
            const int r = r_first + r_local;
            if (r >= rows) continue;
            float mz[8], vz[8], lz[8];
            float big = -INFINITY;
#pragma unroll
            for (int z = 0; z < 8; ++z) {
                mz[z] = -INFINITY;
                vz[z] = lz[z] = 0.f;
                if (z < (int)num_splits) {
                    const int slot = z * per_block + r_local;
                    mz[z] = land_ml[slot * 2];
                    lz[z] = land_ml[slot * 2 + 1];
                    vz[z] = land_o[slot * D + c];
                }
            }
#pragma unroll
            for (int z = 0; z < 8; ++z) big = fmaxf(big, mz[z]);
            float acc = 0.f, denom = 0.f;
#pragma unroll
            for (int z = 0; z < 8; ++z) {
                const float w = mz[z] > -INFINITY ? fast_exp2(mz[z] - big) : 0.f;
                acc += w * vz[z];
                denom += w * lz[z];
            }
            const int tok = r / group, hg = r - tok * group;
            out[((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * D + c] =
                __float2bfloat16_rn(denom > 0.f ? acc / denom : 0.f);
        }
        return;
    }

    // ---- the ranges meet: every block finishes its share of the rows from all the blocks
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    {
        const int per_block = (16 + (int)num_splits - 1) / (int)num_splits;
        const int r_first = (int)split * per_block;
        const uint32_t local_o = (uint32_t)__cvta_generic_to_shared(o_part);
        const uint32_t local_ml = (uint32_t)__cvta_generic_to_shared(&ml_part[0][0]);
        for (int e = tid; e < per_block * D && tid < 128; e += 128) {
            const int r = r_first + e / D, c = e % D;
            if (r >= rows) continue;
            float mz[8], vz[8], lz[8];
            float big = -INFINITY;
#pragma unroll
            for (uint32_t z = 0; z < 8; ++z) {
                mz[z] = -INFINITY;
                vz[z] = lz[z] = 0.f;
                if (z < num_splits) {
                    uint32_t remote_o, remote_ml;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_o) : "r"(local_o), "r"(z));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_ml) : "r"(local_ml), "r"(z));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(mz[z]) : "r"(remote_ml + 8 * r) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(lz[z]) : "r"(remote_ml + 8 * r + 4) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(vz[z]) : "r"(remote_o + 4 * (r * D + c)) : "memory");
                }
            }
#pragma unroll
            for (int z = 0; z < 8; ++z) big = fmaxf(big, mz[z]);
            float acc = 0.f, denom = 0.f;
#pragma unroll
            for (int z = 0; z < 8; ++z) {
                const float w = mz[z] > -INFINITY ? fast_exp2(mz[z] - big) : 0.f;
                acc += w * vz[z];
                denom += w * lz[z];
            }
            const int tok = r / group, hg = r - tok * group;
            out[((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * D + c] =
                __float2bfloat16_rn(denom > 0.f ? acc / denom : 0.f);
        }
    }
    // nobody leaves (and gives its shared memory up) while another block may still read it
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

static int device_sms() {
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (sms <= 0) sms = 148;
    }
    return sms;
}

template <int D, bool FED, bool TWO, int STG>
int launch_attention_decode_cluster(const void* qkv, int q_row_stride, const void* k_pages,
                                    const void* v_pages, const int* table, int max_pages,
                                    const int* q_start, const int* kv_len, void* out, int n_q, int n_kv,
                                    int page_size, float scale, int window, int num_seqs, int cluster,
                                    const float* cos_t, const float* sin_t, int raw, int store,
                                    int num_pages, int* error, cudaStream_t s) {
    constexpr int STAGES = FED ? 4 : STG;
    CUtensorMap map_k, map_v;
    memset(&map_k, 0, sizeof(map_k));
    memset(&map_v, 0, sizeof(map_v));
    if (FED) {
        const cuuint64_t rows = (cuuint64_t)num_pages * n_kv * page_size;
        cuuint64_t dims[2] = {(cuuint64_t)D, rows};
        cuuint64_t strides[1] = {(cuuint64_t)D * 2};
        // (a copy brings a page, or 32 keys of a larger one: the kernel's half tiles)
        cuuint32_t box[2] = {64u, (cuuint32_t)(page_size < MMA_BN / 2 ? page_size : MMA_BN / 2)};
        if (!make_map_nd(&map_k, k_pages, 2, dims, strides, box) ||
            !make_map_nd(&map_v, v_pages, 2, dims, strides, box))
            return MB_ERR_LAUNCH;
    }
    // queries and key/value stages; with head size 64 also the landing area of the merge
    // (FED: and room to start the tiles on a 1024-byte boundary)
    // (FED: STG half stages of 32 keys, as in the kernel)
    const size_t kv_elems = FED ? (size_t)STG * (MMA_BN / 2) * D : (size_t)STAGES * MMA_BN * D;
    const size_t smem = (size_t)(16 * D + 2 * kv_elems) * sizeof(__nv_bfloat16) +
                        (D == 64 ? (size_t)(16 * D + 16 * 2) * sizeof(float) : 0) + (FED ? 1024 : 0);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(attention_decode_cluster_kernel<D, FED, TWO, STG>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    typedef __nv_bfloat16 bf;
    cudaLaunchConfig_t config = launch_config(dim3(num_seqs, n_kv, cluster), FED ? 160 : 128, smem, s);
    cudaLaunchAttribute attrs[2];
    int num_attrs = 0;
    if (config.numAttrs) attrs[num_attrs++] = config.attrs[0];
    if (cluster > 1) {
        attrs[num_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[num_attrs].val.clusterDim.x = 1;
        attrs[num_attrs].val.clusterDim.y = 1;
        attrs[num_attrs].val.clusterDim.z = (unsigned)cluster;
        ++num_attrs;
    }
    config.attrs = attrs;
    config.numAttrs = num_attrs;
    cudaLaunchKernelEx(&config, attention_decode_cluster_kernel<D, FED, TWO, STG>, map_k, map_v, (const bf*)qkv,
                       q_row_stride, (const bf*)k_pages, (const bf*)v_pages, table, max_pages, q_start,
                       kv_len, (bf*)out, n_q, n_kv, page_size, scale, window, cos_t, sin_t, raw, store,
                       error);
    return launch_status();
}

template <int D>
int launch_attention_decode(const void* qkv, int q_row_stride, const void* k_pages,
                            const void* v_pages, const int* table, int max_pages, const int* q_start,
                            const int* kv_len, void* out, float* part_acc, float* part_ml,
                            int* counters, int n_q, int n_kv, int page_size, float scale, int window,
                            int num_seqs, int num_splits, cudaStream_t s) {
    const size_t smem = (size_t)(16 * D + 2 * 3 * MMA_BN * D) * sizeof(__nv_bfloat16);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(attention_decode_kernel<D>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    dim3 grid(num_seqs, n_kv, num_splits);
    typedef __nv_bfloat16 bf;
    MB_LAUNCH((attention_decode_kernel<D>), grid, 128, smem, s, 
        (const bf*)qkv, q_row_stride, (const bf*)k_pages, (const bf*)v_pages, table, max_pages,
        q_start, kv_len, (bf*)out, part_acc, part_ml, counters, n_q, n_kv, page_size, scale, window,
        num_splits);
    return launch_status();
}

template <int D, int NWARPS>
int launch_attention_mma(const void* qkv, int q_row_stride, const void* k_pages, const void* v_pages,
                         const int* table, int max_pages, const int* q_start, const int* kv_len,
                         void* out, float* part_acc, float* part_ml, int n_q, int n_kv,
                         int page_size, float scale, int window, int num_seqs, int max_q_len,
                         int num_splits, cudaStream_t s) {
    constexpr int ROWS = NWARPS * 16;
    const size_t smem = (size_t)(ROWS * D + 4 * MMA_BN * D) * sizeof(__nv_bfloat16);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(attention_mma_kernel<D, NWARPS>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    const int group = n_q / n_kv;
    const int tiles_per_seq = (max_q_len * group + ROWS - 1) / ROWS;
    dim3 grid(num_seqs * tiles_per_seq, n_kv, num_splits);
    typedef __nv_bfloat16 bf;
    MB_LAUNCH((attention_mma_kernel<D, NWARPS>), grid, NWARPS * 32, smem, s, 
        (const bf*)qkv, q_row_stride, (const bf*)k_pages, (const bf*)v_pages, table, max_pages,
        q_start, kv_len, (bf*)out, part_acc, part_ml, n_q, n_kv, page_size, scale, window,
        tiles_per_seq, num_splits);
    return launch_status();
}

}  // namespace mb

using namespace mb;

// 1 if this kernel takes the head size (bfloat16 only), else 0: the caller then uses the
// CUDA-core kernel.
MB_EXPORT int mb_attention_mma_supports(int d) { return d == 64 || d == 128; }

// Whether a decode-like step should hand the cluster kernel the bare projections (`raw`: it
// then rotates the queries and rotates and stores the new keys itself) instead of running the
// fused q/k/v kernel in front of it. Measured inside the captured decode step on B200: head
// size 64, batch 8, 0.671 -> 0.660 ms per step; head size 128 (since its tiles are all in shared
// memory before the wait and the new keys are put in there): 1.5B sizes batch 8 1.552 -> 1.544,
// batch 16 2.18 -> 2.07, 7B sizes batch 8 3.93 -> 3.73. The answer is a property of this
// kernel, asked for here.
MB_EXPORT int mb_attention_decode_raw_pays(int d) { return d == 64 || d == 128; }

// Decode-like batches (at most 16 rows per sequence and KV head) with the key ranges of a
// (sequence, KV head) as one cluster of `cluster` blocks (1, 2, 4 or 8): no scratch, no
// counters, one launch. bfloat16, head sizes 64 and 128. With `raw` the q/k/v rows are the
// bare projection: the kernel rotates with `cos_t` / `sin_t` ([positions, d/2], null = no
// rotation, the whole head otherwise) and, with `store`, writes this step's keys and values
// into the pages itself.
MB_EXPORT int mb_paged_attention_decode_cluster(const void* qkv, int q_row_stride, const void* k_pages,
                                                const void* v_pages, const int* table, int max_pages,
                                                const int* q_start, const int* kv_len, void* out,
                                                int tokens, int num_seqs, int max_q_len, int n_q,
                                                int n_kv, int d, int page_size, float scale, int window,
                                                int cluster, const float* cos_t, const float* sin_t,
                                                int raw, int store, int num_pages, int* error,
                                                void* stream) {
    // num_pages > 0 (with the pages' count) and `error` (a zeroed word on the device) select
    // the TMA-fed form (pages of 8 to 64 tokens): for blocks that walk many key tiles each
    // (large batches). 0: the copies are 16 bytes per thread, as the small batches want them,
    // whose tiles are all in flight before the kernel in front is done.
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_attention_mma_supports(d) || n_kv <= 0 || n_q % n_kv) return MB_ERR_UNSUPPORTED_SIZE;
    // (pages of one token would leave the kernel's window of the block table shorter than
    // the tiles it fills up front)
    if (page_size < 2 || (page_size & (page_size - 1))) return MB_ERR_UNSUPPORTED_SIZE;
    if (q_row_stride % 8) return MB_ERR_ALIGNMENT;
    if (max_q_len * (n_q / n_kv) > 16 || n_kv > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    if (cluster != 1 && cluster != 2 && cluster != 4 && cluster != 8) return MB_ERR_UNSUPPORTED_SIZE;
    // bare projections are only taken by the call that also stores the new keys: a layer that
    // reads another layer's cache must find this step's keys in the pages
    if (raw && !store) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const bool fed = num_pages > 0 && error != nullptr && page_size >= 8 &&
                     page_size <= MMA_BN && (((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) == 0;
    // (the longest portion bounds every sequence's rows: one column tile of 8 rows, or two)
    const bool two = max_q_len * (n_q / n_kv) > 8;
#define MB_DC_LAUNCH(D_, FED_, TWO_, STG_)                                                            \
    launch_attention_decode_cluster<D_, FED_, TWO_, STG_>(qkv, q_row_stride, k_pages, v_pages, table, max_pages, \
                                                    q_start, kv_len, out, n_q, n_kv, page_size, scale, \
                                                    window, num_seqs, cluster, cos_t, sin_t, raw, store, \
                                                    FED_ ? num_pages : 0, FED_ ? error : nullptr, s)
    // (TMA-fed: eight half stages at head size 64, four at 128, where eight would leave an SM
    // to one block: measured at 1.5B sizes with no more blocks than SMs, 8 sequences, 1.32 ms per
    // step with four and 1.44 with eight)
    if (fed && d == 64) return two ? MB_DC_LAUNCH(64, true, true, 8) : MB_DC_LAUNCH(64, true, false, 8);
    if (fed) return two ? MB_DC_LAUNCH(128, true, true, 4) : MB_DC_LAUNCH(128, true, false, 4);
    if (d == 64) return two ? MB_DC_LAUNCH(64, false, true, 5) : MB_DC_LAUNCH(64, false, false, 5);
    // head size 128: five stages (164 KB, one block per SM) while the blocks are at most half
    // the SMs. Measured on B200 inside the captured decode step at 1.5B sizes: batch 1 (16
    // blocks) 1.29 ms with three stages, 1.17 with five; batch 8 (128 blocks) 1.49 with three,
    // 1.54 with five (a block that needs an SM to itself is placed later while blocks of the
    // kernel in front are still there)
    if (2ll * num_seqs * n_kv * cluster <= device_sms())
        return two ? MB_DC_LAUNCH(128, false, true, 5) : MB_DC_LAUNCH(128, false, false, 5);
    return two ? MB_DC_LAUNCH(128, false, true, 3) : MB_DC_LAUNCH(128, false, false, 3);
#undef MB_DC_LAUNCH
}

// Same arguments as mb_paged_attention_simt; bfloat16 only. Scratch as there.
MB_EXPORT int mb_paged_attention_mma(const void* qkv, int q_row_stride, const void* k_pages,
                                     const void* v_pages, const int* table, int max_pages,
                                     const int* q_start, const int* kv_len, const int* seq_of_token,
                                     void* out, float* scratch, long long scratch_floats, int tokens,
                                     int num_seqs, int max_q_len, int n_q, int n_kv, int d,
                                     int page_size, float scale, int window, int num_splits,
                                     int* counters, void* stream) {
    // counters: num_seqs * n_kv zeroed ints (left zeroed) to let the last split block merge
    // in the same launch; null selects the separate merge kernel.
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_attention_mma_supports(d) || n_kv <= 0 || n_q % n_kv) return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || (page_size & (page_size - 1))) return MB_ERR_UNSUPPORTED_SIZE;
    if (q_row_stride % 8) return MB_ERR_ALIGNMENT;
    if (num_splits < 1) num_splits = 1;
    if (n_kv > 65535 || num_splits > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    float* part_acc = nullptr;
    float* part_ml = nullptr;
    if (num_splits > 1) {
        const long long need = (long long)tokens * n_q * num_splits * (d + 2);
        if (!scratch || scratch_floats < need) return MB_ERR_SCRATCH;
        part_acc = scratch;
        part_ml = scratch + (int64_t)tokens * n_q * num_splits * d;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int group = n_q / n_kv;
    const bool small = max_q_len * group <= 16;  // decode-like: one warp of rows per block
    int rc;
    if (small) {
        if (num_splits > 64) counters = nullptr;   // the in-kernel merge holds 64 splits
        if (d == 64)
            rc = launch_attention_decode<64>(qkv, q_row_stride, k_pages, v_pages, table, max_pages,
                                             q_start, kv_len, out, part_acc, part_ml, counters, n_q,
                                             n_kv, page_size, scale, window, num_seqs, num_splits, s);
        else
            rc = launch_attention_decode<128>(qkv, q_row_stride, k_pages, v_pages, table, max_pages,
                                              q_start, kv_len, out, part_acc, part_ml, counters, n_q,
                                              n_kv, page_size, scale, window, num_seqs, num_splits,
                                              s);
        if (rc != MB_OK || num_splits == 1 || counters != nullptr) return rc;
        return launch_attention_combine(part_acc, part_ml, seq_of_token, out, tokens, n_q, d,
                                        num_splits, MB_BF16, s);
    }
#define MB_MMA_CASE(DD, NW)                                                                       \
    rc = launch_attention_mma<DD, NW>(qkv, q_row_stride, k_pages, v_pages, table, max_pages,      \
                                      q_start, kv_len, out, part_acc, part_ml, n_q, n_kv,         \
                                      page_size, scale, window, num_seqs, max_q_len, num_splits, s)
    if (d == 64) {
        MB_MMA_CASE(64, 4);
    } else {
        MB_MMA_CASE(128, 4);
    }
#undef MB_MMA_CASE
    if (rc != MB_OK || num_splits == 1) return rc;
    return launch_attention_combine(part_acc, part_ml, seq_of_token, out, tokens, n_q, d, num_splits,
                                    MB_BF16, s);
}
