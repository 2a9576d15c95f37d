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
    const int t = blockIdx.x;
    int id = ids[t];
    const bool ok = id >= 0 && id < vocab;
    const int64_t base = (int64_t)(ok ? id : 0) * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[(int64_t)t * hidden + c] = ok ? load_as_float(table, base + c, table_dtype) : 0.f;
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
    const int t = blockIdx.x;
    const int seq = seq_of_token[t];
    if (seq < 0) return;
    const int pos = positions[t];
    const int half = rot / 2;
    const int64_t row = (int64_t)t * (n_q + 2 * n_kv) * d;
    int64_t slot = -1;
    if (store) {
        const int page = table[(int64_t)seq * max_pages + pos / page_size];
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

template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        out[i] = from_float<TO>(to_float(in[i]));
}

}  // namespace mb

using namespace mb;

MB_EXPORT int mb_embed(const int* ids, const void* table, int table_dtype, float* out, int tokens,
                       int hidden, int vocab, void* stream) {
    if (tokens <= 0) return MB_OK;
    embed_kernel<<<tokens, 256, 0, (cudaStream_t)stream>>>(ids, table, table_dtype, out, hidden,
                                                            vocab);
    return launch_status();
}

MB_EXPORT int mb_add_rmsnorm(float* h, const void* delta, const void* weight, int weight_dtype,
                             void* out, const int* rows, int count, int hidden, float eps,
                             int dtype, void* stream) {
    if (count <= 0) return MB_OK;
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MB_F32)
        add_rmsnorm_kernel<float><<<count, threads, 0, s>>>(
            h, (const float*)delta, weight, weight_dtype, (float*)out, rows, hidden, eps);
    else if (dtype == MB_BF16)
        add_rmsnorm_kernel<__nv_bfloat16><<<count, threads, 0, s>>>(
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
        swiglu_kernel<float><<<blocks, 256, 0, s>>>((const float*)gate_up, (float*)out, total, width);
    else if (dtype == MB_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(
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
        rope_store_kernel<float><<<tokens, 256, 0, s>>>(
            (float*)qkv, cos_t, sin_t, rot, positions, seq_of_token, table, max_pages,
            (float*)k_pages, (float*)v_pages, n_q, n_kv, d, page_size, store);
    else if (dtype == MB_BF16)
        rope_store_kernel<__nv_bfloat16><<<tokens, 256, 0, s>>>(
            (__nv_bfloat16*)qkv, cos_t, sin_t, rot, positions, seq_of_token, table, max_pages,
            (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, n_q, n_kv, d, page_size, store);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

MB_EXPORT int mb_convert(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                         void* stream) {
    if (n <= 0) return MB_OK;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == MB_BF16 && out_dtype == MB_F32)
        convert_kernel<<<blocks, 256, 0, s>>>((const __nv_bfloat16*)in, (float*)out, (int64_t)n);
    else if (in_dtype == MB_F32 && out_dtype == MB_BF16)
        convert_kernel<<<blocks, 256, 0, s>>>((const float*)in, (__nv_bfloat16*)out, (int64_t)n);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}
