// Embedding lookup, residual-add + RMSNorm, SiLU gate, rotary encoding + page store.
//
// All arithmetic is float32; storage is float32 or bfloat16 (the template parameter T is
// the activation type; weights carry a run-time dtype flag, because a checkpoint tensor
// stored in 32-bit stays 32-bit even in the bfloat16 engine).
#include "common.cuh"

namespace mb {

// ---------------------------------------------------------------------------- embedding
// out[t, :] = table[ids[t], :], written into the float32 residual stream.
// mercury/model/qwen2.py:109 (nn.Embedding, no scaling).
__global__ void embed_kernel(const int* __restrict__ ids, const void* __restrict__ table,
                             int table_dtype, float* __restrict__ out, int hidden, int vocab) {
    grid_dependency_sync();
    const int t = blockIdx.x;
    int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
#ifdef MB_BOUNDS_CHECK
    if (!ok && threadIdx.x == 0) check_report(MB_CHECK_TOKEN, id, vocab);
#endif
    const int64_t base = (int64_t)(ok ? id : 0) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[(int64_t)t * hidden + c] = ok ? load_as_float(table, base + c, table_dtype) : 0.f;
}

// Token ids that were not known on the host when the step was put together (the step was
// launched while the step before was still running): ids[t] = sampled[from[t]] where
// from[t] >= 0, taken from the tokens the step before has sampled on the device.
__global__ void patch_tokens_kernel(int* __restrict__ ids, const int* __restrict__ from,
                                    const int* __restrict__ sampled, int tokens) {
    grid_dependency_sync();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < tokens && from[t] >= 0) ids[t] = sampled[from[t]];
}

// ---------------------------------------------------------------------------- norm
// One block per row. x = h + delta (float32); when `rows` is null the sum is stored back
// as the new residual (mercury/model/qwen2.py:27-28); y = x * rsqrt(mean(x^2) + eps) * w
// (mercury/model/qwen2.py:29-31). With `rows` only the listed rows are read, nothing is
// stored back, and output row r holds the norm of input row rows[r].
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                   const void* __restrict__ weight, int weight_dtype,
                                   T* __restrict__ out, const int* __restrict__ rows,
                                   int hidden, float eps) {
    grid_dependency_sync();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = (int64_t)(rows ? rows[r] : r) * hidden;
    const int64_t dst = (int64_t)r * hidden;
    float ss = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float x = h[src + c];
        if (delta) {
            x += to_float(delta[src + c]);
            if (!rows) h[src + c] = x;
        }
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float x = h[src + c];
        if (delta && rows) x += to_float(delta[src + c]);
        out[dst + c] = from_float<T>(x * rstd * load_as_float(weight, c, weight_dtype));
    }
}

// ---------------------------------------------------------------------------- SiLU gate
// out[t, i] = silu(gate_up[t, i]) * gate_up[t, width + i], silu(z) = z / (1 + exp(-z))
// (mercury/model/qwen2.py:42).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int64_t total,
                              int width) {
    grid_dependency_sync();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / width;
        const int c = (int)(i - t * width);
        const float g = to_float(gate_up[t * 2 * width + c]);
        const float u = to_float(gate_up[t * 2 * width + width + c]);
        out[i] = from_float<T>(g / (1.f + expf(-g)) * u);
    }
}

// ---------------------------------------------------------------------------- rotary + store
// One block per token. The q heads are rotated in place; the k heads are rotated and
// stored into the token's page slot; the v heads are copied there
// (mercury/model/rope.py:11-17 for the rotation, mercury/model/attention.py:35-45 and
// mercury/runner.py:25-34 for the slot). cos/sin: float32 [positions, rot/2]; a null
// `cos` means no rotation. Tokens of sequence -1 are padding and are skipped, and a page
// entry of -1 (given back) is never written.
// qkv row: [n_q * d | n_kv * d | n_kv * d]. Pages: [page][kv head][slot in page][d].
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, int rot,
                                  const int* __restrict__ positions,
                                  const int* __restrict__ seq_of_token,
                                  const int* __restrict__ table, int max_pages,
                                  T* __restrict__ k_pages, T* __restrict__ v_pages,
                                  int n_q, int n_kv, int d, int page_size, int store) {
    grid_dependency_sync();
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int pos = checked_position(positions[t]);
    const int half = rot / 2;
    const int64_t row = (int64_t)t * (n_q + 2 * n_kv) * d;
    int64_t slot = -1;
    if (store) {
        const int page = table_page(table, seq, max_pages, pos / page_size);
        if (page >= 0) slot = (int64_t)page * n_kv * page_size + pos % page_size;
    }
    // rotated heads: q and k. One work item = one (head, pair or pass-through feature).
    const int per_head = d - half;  // `half` pairs + (d - rot) untouched features
    const int rotated_heads = n_q + n_kv;
    for (int w = threadIdx.x; w < rotated_heads * per_head; w += blockDim.x) {
        const int head = w / per_head;
        const int i = w - head * per_head;
        T* x = qkv + row + (int64_t)head * d;
        T* dst = nullptr;
        if (head >= n_q && slot >= 0)
            dst = k_pages + (slot + (int64_t)(head - n_q) * page_size) * d;
        if (i < half) {
            float a = to_float(x[i]), b = to_float(x[i + half]);
            if (cos_t) {
                const float c = cos_t[(int64_t)pos * half + i], s = sin_t[(int64_t)pos * half + i];
                const float ra = a * c - b * s, rb = b * c + a * s;
                a = ra;
                b = rb;
            }
            const T ta = from_float<T>(a), tb = from_float<T>(b);
            x[i] = ta;
            x[i + half] = tb;
            if (dst) {
                dst[i] = ta;
                dst[i + half] = tb;
            }
        } else if (dst) {
            dst[i + half] = x[i + half];
        }
    }
    if (slot >= 0) {
        const T* v = qkv + row + (int64_t)(n_q + n_kv) * d;
        for (int w = threadIdx.x; w < n_kv * d; w += blockDim.x) {
            const int head = w / d, i = w - head * d;
            v_pages[(slot + (int64_t)head * page_size) * d + i] = v[w];
        }
    }
}

// bfloat16, width a multiple of 8: eight features per thread through 16-byte accesses.
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up,
                                     __nv_bfloat16* __restrict__ out, int tokens, int width) {
    grid_dependency_sync();
    const int chunks = width / 8;
    const int64_t total = (int64_t)tokens * chunks;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / chunks;
        const int c = (int)(i - t * chunks) * 8;
        const uint4 gq = *reinterpret_cast<const uint4*>(gate_up + t * 2 * width + c);
        const uint4 uq = *reinterpret_cast<const uint4*>(gate_up + t * 2 * width + width + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gq);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uq);
        uint4 oq;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&oq);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x,
                                          g.y / (1.f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * width + c) = oq;
    }
}

// bfloat16 activations and weight, hidden a multiple of 4 and at most 4 * ITEMS * threads:
// each row is read once, kept in registers between the sum of squares and the scaling.
template <int ITEMS>
__global__ void add_rmsnorm_bf16_regs_kernel(float* __restrict__ h,
                                             const __nv_bfloat16* __restrict__ delta,
                                             const __nv_bfloat16* __restrict__ weight,
                                             __nv_bfloat16* __restrict__ out,
                                             const int* __restrict__ rows, int hidden, float eps) {
    grid_dependency_sync();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int64_t src = (int64_t)(rows ? rows[r] : r) * hidden;
    const int64_t dst = (int64_t)r * hidden;
    float4 x[ITEMS];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        x[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < hidden) {
            x[it] = *reinterpret_cast<const float4*>(h + src + c);
            if (delta) {
                const uint2 dq = *reinterpret_cast<const uint2*>(delta + src + c);
                const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dq.x));
                const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dq.y));
                x[it].x += d0.x;
                x[it].y += d0.y;
                x[it].z += d1.x;
                x[it].w += d1.y;
                if (!rows) *reinterpret_cast<float4*>(h + src + c) = x[it];
            }
            ss += x[it].x * x[it].x + x[it].y * x[it].y + x[it].z * x[it].z + x[it].w * x[it].w;
        }
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < hidden) {
            const uint2 wq = *reinterpret_cast<const uint2*>(weight + c);
            const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wq.x));
            const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wq.y));
            uint2 oq;
            *reinterpret_cast<__nv_bfloat162*>(&oq.x) =
                __floats2bfloat162_rn(x[it].x * rstd * w0.x, x[it].y * rstd * w0.y);
            *reinterpret_cast<__nv_bfloat162*>(&oq.y) =
                __floats2bfloat162_rn(x[it].z * rstd * w1.x, x[it].w * rstd * w1.y);
            *reinterpret_cast<uint2*>(out + dst + c) = oq;
        }
    }
}

// The same for many rows (prompt steps): one warp per row, eight rows per block, so that the
// sum of squares needs shuffles only and each thread has a row's worth of loads in flight.
// hidden a multiple of 4 and at most 128 * ITEMS.
template <int ITEMS>
__global__ void __launch_bounds__(256)
add_rmsnorm_bf16_warp_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                             const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out,
                             int count, int hidden, float eps) {
    grid_dependency_sync();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= count) return;
    const int64_t at = (int64_t)r * hidden;
    float4 x[ITEMS];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int c = (it * 32 + lane) * 4;
        x[it] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < hidden) x[it] = *reinterpret_cast<const float4*>(h + at + c);
    }
    if (delta) {
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int c = (it * 32 + lane) * 4;
            if (c < hidden) {
                const uint2 dq = *reinterpret_cast<const uint2*>(delta + at + c);
                const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dq.x));
                const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dq.y));
                x[it].x += d0.x;
                x[it].y += d0.y;
                x[it].z += d1.x;
                x[it].w += d1.y;
                *reinterpret_cast<float4*>(h + at + c) = x[it];
            }
        }
    }
#pragma unroll
    for (int it = 0; it < ITEMS; ++it)
        ss += x[it].x * x[it].x + x[it].y * x[it].y + x[it].z * x[it].z + x[it].w * x[it].w;
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
        const int c = (it * 32 + lane) * 4;
        if (c < hidden) {
            const uint2 wq = *reinterpret_cast<const uint2*>(weight + c);
            const float2 w0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wq.x));
            const float2 w1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wq.y));
            uint2 oq;
            *reinterpret_cast<__nv_bfloat162*>(&oq.x) =
                __floats2bfloat162_rn(x[it].x * rstd * w0.x, x[it].y * rstd * w0.y);
            *reinterpret_cast<__nv_bfloat162*>(&oq.y) =
                __floats2bfloat162_rn(x[it].z * rstd * w1.x, x[it].w * rstd * w1.y);
            *reinterpret_cast<uint2*>(out + at + c) = oq;
        }
    }
}

// bfloat16, the whole head rotated, head size a multiple of 16: one thread per (token, head,
// run of eight pairs), through 16-byte accesses (a thread holds features [8j, 8j+8) of the
// first half and the matching eight of the second half).
__global__ void rope_store_bf16_kernel(__nv_bfloat16* __restrict__ qkv,
                                       const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ seq_of_token,
                                       const int* __restrict__ table, int max_pages,
                                       __nv_bfloat16* __restrict__ k_pages,
                                       __nv_bfloat16* __restrict__ v_pages, int tokens, int n_q,
                                       int n_kv, int d, int page_size, int store) {
    grid_dependency_sync();
    const int heads = n_q + 2 * n_kv;
    const int half = d / 2, runs = half / 8;
    const int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (int64_t)tokens * heads * runs) return;
    const int run = (int)(item % runs);
    const int head = (int)((item / runs) % heads);
    const int t = (int)(item / ((int64_t)runs * heads));
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int pos = checked_position(positions[t]);
    const int i = run * 8;
    __nv_bfloat16* x = qkv + (int64_t)t * heads * d + (int64_t)head * d;
    __nv_bfloat16* dst = nullptr;
    if (head >= n_q && store) {
        const int page = table_page(table, seq, max_pages, pos / page_size);
        if (page >= 0) {
            const bool is_k = head < n_q + n_kv;
            const int kvh = is_k ? head - n_q : head - n_q - n_kv;
            dst = (is_k ? k_pages : v_pages) +
                  (((int64_t)page * n_kv + kvh) * page_size + pos % page_size) * d;
        }
    }
    if (head >= n_q + n_kv) {                    // a value head: copy
        if (dst) {
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(x + i);
            *reinterpret_cast<uint4*>(dst + i + half) = *reinterpret_cast<const uint4*>(x + i + half);
        }
        return;
    }
    {
        uint4 aq = *reinterpret_cast<const uint4*>(x + i);
        uint4 bq = *reinterpret_cast<const uint4*>(x + i + half);
        if (cos_t) {
            __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&aq);
            __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&bq);
            const float* cp = cos_t + (int64_t)pos * half + i;
            const float* sp = sin_t + (int64_t)pos * half + i;
            const float4 c0 = *reinterpret_cast<const float4*>(cp), c1 = *reinterpret_cast<const float4*>(cp + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(sp), s1 = *reinterpret_cast<const float4*>(sp + 4);
            const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(a2[e]), b = __bfloat1622float2(b2[e]);
                a2[e] = __floats2bfloat162_rn(a.x * cs[2 * e] - b.x * sn[2 * e],
                                              a.y * cs[2 * e + 1] - b.y * sn[2 * e + 1]);
                b2[e] = __floats2bfloat162_rn(b.x * cs[2 * e] + a.x * sn[2 * e],
                                              b.y * cs[2 * e + 1] + a.y * sn[2 * e + 1]);
            }
        }
        *reinterpret_cast<uint4*>(x + i) = aq;
        *reinterpret_cast<uint4*>(x + i + half) = bq;
        if (dst) {
            *reinterpret_cast<uint4*>(dst + i) = aq;
            *reinterpret_cast<uint4*>(dst + i + half) = bq;
        }
    }
}

}  // namespace mb

namespace mb {
int g_dependent_launch = 0;
#ifdef MB_BOUNDS_CHECK
__device__ int mb_check_limit[4] = {0, 0, 0, 0};
__device__ int mb_check_word[4] = {0, 0, 0, 0};
#endif
}

using namespace mb;

// 1: launch every kernel with the programmatic-serialization attribute (see common.cuh).
MB_EXPORT void mb_set_dependent_launch(int enabled) { g_dependent_launch = enabled ? 1 : 0; }

// 1 if this library is the checked build (see common.cuh), else 0.
MB_EXPORT int mb_check_enabled() {
#ifdef MB_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}

// Checked build: the limits that indices are compared with from now on (pages of the pool
// whose tables the next kernels read, rows of the rotation tables; 0 = not checked). Ordered
// with the kernels of `stream`. A no-op in the ordinary build.
MB_EXPORT int mb_check_set_limits(int pages, int positions, void* stream) {
#ifdef MB_BOUNDS_CHECK
    const int limits[4] = {pages, positions, 0, 0};
    if (cudaMemcpyToSymbolAsync(mb_check_limit, limits, sizeof(limits), 0, cudaMemcpyHostToDevice,
                                (cudaStream_t)stream) != cudaSuccess)
        return MB_ERR_LAUNCH;
#else
    (void)pages, (void)positions, (void)stream;
#endif
    return MB_OK;
}

// Checked build: copies the status word (kind, value, limit, count) to `out` (4 ints on the
// host) after everything on `stream` has run, and clears it. Zeros in the ordinary build.
MB_EXPORT int mb_check_read(int* out, void* stream) {
    out[0] = out[1] = out[2] = out[3] = 0;
#ifdef MB_BOUNDS_CHECK
    cudaStream_t s = (cudaStream_t)stream;
    if (cudaMemcpyFromSymbolAsync(out, mb_check_word, 4 * sizeof(int), 0, cudaMemcpyDeviceToHost, s) !=
            cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess)
        return MB_ERR_LAUNCH;
    const int zeros[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbolAsync(mb_check_word, zeros, sizeof(zeros), 0, cudaMemcpyHostToDevice, s) !=
        cudaSuccess)
        return MB_ERR_LAUNCH;
#else
    (void)stream;
#endif
    return MB_OK;
}

MB_EXPORT int mb_embed(const int* ids, const void* table, int table_dtype, float* out, int tokens,
                       int hidden, int vocab, void* stream) {
    if (tokens <= 0) return MB_OK;
    MB_LAUNCH((embed_kernel), tokens, 256, 0, (cudaStream_t)stream, ids, table, table_dtype, out, hidden,
                                                            vocab);
    return launch_status();
}

MB_EXPORT int mb_patch_tokens(int* ids, const int* from, const int* sampled, int tokens, void* stream) {
    if (tokens <= 0) return MB_OK;
    MB_LAUNCH((patch_tokens_kernel), (tokens + 127) / 128, 128, 0, (cudaStream_t)stream, ids, from, sampled,
              tokens);
    return launch_status();
}

MB_EXPORT int mb_add_rmsnorm(float* h, const void* delta, const void* weight, int weight_dtype,
                             void* out, const int* rows, int count, int hidden, float eps,
                             int dtype, void* stream) {
    if (count <= 0) return MB_OK;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((add_rmsnorm_kernel<float>), count, threads, 0, s, 
            h, (const float*)delta, weight, weight_dtype, (float*)out, rows, hidden, eps);
    else if (dtype == MB_BF16 && weight_dtype == MB_BF16 && hidden % 4 == 0 && hidden <= 8192) {
        typedef __nv_bfloat16 bf;
        // many whole rows: a warp per row (the block-per-row kernels are for the few rows of
        // a decode step, where a row's latency counts, and for picked rows)
        if (rows == nullptr && count >= 256 && hidden <= 2048) {
            const int blocks = (count + 7) / 8;
            if (hidden <= 1024)
                MB_LAUNCH((add_rmsnorm_bf16_warp_kernel<8>), blocks, 256, 0, s, h, (const bf*)delta,
                          (const bf*)weight, (bf*)out, count, hidden, eps);
            else
                MB_LAUNCH((add_rmsnorm_bf16_warp_kernel<16>), blocks, 256, 0, s, h, (const bf*)delta,
                          (const bf*)weight, (bf*)out, count, hidden, eps);
        } else if (hidden <= 1024)
            MB_LAUNCH((add_rmsnorm_bf16_regs_kernel<2>), count, 128, 0, s, 
                h, (const bf*)delta, (const bf*)weight, (bf*)out, rows, hidden, eps);
        else if (hidden <= 4096)
            MB_LAUNCH((add_rmsnorm_bf16_regs_kernel<4>), count, 256, 0, s, 
                h, (const bf*)delta, (const bf*)weight, (bf*)out, rows, hidden, eps);
        else
            MB_LAUNCH((add_rmsnorm_bf16_regs_kernel<8>), count, 256, 0, s, 
                h, (const bf*)delta, (const bf*)weight, (bf*)out, rows, hidden, eps);
    } else if (dtype == MB_BF16)
        MB_LAUNCH((add_rmsnorm_kernel<__nv_bfloat16>), count, threads, 0, s, 
            h, (const __nv_bfloat16*)delta, weight, weight_dtype, (__nv_bfloat16*)out, rows, hidden,
            eps);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

MB_EXPORT int mb_swiglu(const void* gate_up, void* out, int tokens, int width, int dtype,
                        void* stream) {
    const int64_t total = (int64_t)tokens * width;
    if (total <= 0) return MB_OK;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((swiglu_kernel<float>), blocks, 256, 0, s, (const float*)gate_up, (float*)out, total, width);
    else if (dtype == MB_BF16 && width % 8 == 0) {
        const int64_t work = total / 8;
        const int grid = (int)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
        MB_LAUNCH((swiglu_bf16x8_kernel), grid, 256, 0, s, (const __nv_bfloat16*)gate_up,
                                                  (__nv_bfloat16*)out, tokens, width);
    } else if (dtype == MB_BF16)
        MB_LAUNCH((swiglu_kernel<__nv_bfloat16>), blocks, 256, 0, s, 
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, total, width);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

MB_EXPORT int mb_rope_store(void* qkv, const float* cos_t, const float* sin_t, int rot,
                            const int* positions, const int* seq_of_token, const int* table,
                            int max_pages, void* k_pages, void* v_pages, int tokens, int n_q,
                            int n_kv, int d, int page_size, int store, int dtype, void* stream) {
    if (tokens <= 0) return MB_OK;
    if (rot < 0 || rot > d || (rot & 1)) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        MB_LAUNCH((rope_store_kernel<float>), tokens, 256, 0, s, 
            (float*)qkv, cos_t, sin_t, rot, positions, seq_of_token, table, max_pages,
            (float*)k_pages, (float*)v_pages, n_q, n_kv, d, page_size, store);
    else if (dtype == MB_BF16 && d % 16 == 0 && (rot == d || rot == 0)) {
        const long long items = (long long)tokens * (n_q + 2 * n_kv) * (d / 16);
        const int blocks = (int)((items + 255) / 256);
        MB_LAUNCH((rope_store_bf16_kernel), blocks, 256, 0, s, (__nv_bfloat16*)qkv,
                  rot ? cos_t : nullptr, sin_t, positions, seq_of_token, table, max_pages,
                  (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, tokens, n_q, n_kv, d, page_size,
                  store);
    }
    else if (dtype == MB_BF16)
        MB_LAUNCH((rope_store_kernel<__nv_bfloat16>), tokens, 256, 0, s, 
            (__nv_bfloat16*)qkv, cos_t, sin_t, rot, positions, seq_of_token, table, max_pages,
            (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, n_q, n_kv, d, page_size, store);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}
