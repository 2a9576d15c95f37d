// Paged attention on the CUDA cores: the float32 path of the engine, and the fallback of
// the bfloat16 engine for head sizes its tensor-core kernels refuse.
//
// One kernel covers prompt portions and decode tokens alike. A step's batch is ragged:
// sequence s owns the query tokens q_start[s] .. q_start[s+1]-1 of the batch; after this
// step it has kv_len[s] keys, so its i-th query token sits at position
// kv_len[s] - q_len + i. Keys and values are read in place from the pages that the
// sequence's block table names (no gather copy as in mercury/model/attention.py:63-64,
// :88-89). Key j is seen from position p iff j <= p (mercury/model/attention.py:97-99)
// and, with a window, j > p - window; the softmax runs online in float32 with the true
// expf. Query head h reads KV head h / (n_q / n_kv) (mercury/model/attention.py:26-29).
//
// Work split: the (query token, head of the group) pairs of one sequence and one KV head
// are laid out as rows; a block of 8 warps takes 16 consecutive rows, each warp two of
// them. Keys are walked in tiles of 32 aligned to absolute positions 0, 32, 64, ..., one
// key per lane for the scores and 32 features per lane for the weighted sum, so a row's
// arithmetic does not depend on how the batch was cut. With num_splits > 1 the key tiles
// are divided over gridDim.z and each split leaves (max, sum, weighted values) in scratch
// for `attention_combine_kernel`.
#include "common.cuh"

namespace mb {

constexpr int ATT_ROWS = 16;     // rows per block
constexpr int ATT_WARPS = 8;
constexpr int ATT_RPW = ATT_ROWS / ATT_WARPS;  // rows per warp
constexpr int ATT_KEYS = 32;     // keys per tile

template <typename T, int NC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_kernel(const T* __restrict__ qkv, int q_row_stride, const T* __restrict__ k_pages,
                       const T* __restrict__ v_pages, const int* __restrict__ table, int max_pages,
                       const int* __restrict__ q_start, const int* __restrict__ kv_len_of,
                       T* __restrict__ out, float* __restrict__ part_acc,
                       float* __restrict__ part_ml, int n_q, int n_kv, int d, int page_size,
                       float scale, int window, int tiles_per_seq, int num_splits) {
    grid_dependency_sync();
    extern __shared__ float smem[];
    const int seq = blockIdx.x / tiles_per_seq;
    const int tile = blockIdx.x - seq * tiles_per_seq;
    const int kvh = blockIdx.y;
    const int split = blockIdx.z;
    const int group = n_q / n_kv;
    const int q_begin = q_start[seq];
    const int q_len = q_start[seq + 1] - q_begin;
    const int row0 = tile * ATT_ROWS;
    if (row0 >= q_len * group) return;
    const int kv_len = kv_len_of[seq];
    const int first_pos = kv_len - q_len;

    float* q_s = smem;                                   // [ATT_ROWS][d]
    float* k_s = q_s + ATT_ROWS * d;                     // [ATT_KEYS][d + 1]
    float* v_s = k_s + ATT_KEYS * (d + 1);               // [ATT_KEYS][d]
    int* page_s = reinterpret_cast<int*>(v_s + ATT_KEYS * d);  // [ATT_KEYS]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // queries of this block's rows, float32
    for (int idx = tid; idx < ATT_ROWS * d; idx += blockDim.x) {
        const int r = idx / d, c = idx - r * d;
        const int row = row0 + r;
        const int tok = row / group, hg = row - tok * group;
        float v = 0.f;
        if (tok < q_len)
            v = to_float(qkv[(int64_t)(q_begin + tok) * q_row_stride + (kvh * group + hg) * d + c]);
        q_s[idx] = v;
    }

    // positions of this warp's rows
    int row_pos[ATT_RPW];
    bool row_ok[ATT_RPW];
#pragma unroll
    for (int rr = 0; rr < ATT_RPW; ++rr) {
        const int row = row0 + warp * ATT_RPW + rr;
        const int tok = row / group;
        row_ok[rr] = tok < q_len;
        row_pos[rr] = first_pos + tok;
    }

    // key tiles this block has to look at
    const int tok_min = row0 / group;
    int tok_max = (row0 + ATT_ROWS - 1) / group;
    if (tok_max > q_len - 1) tok_max = q_len - 1;
    const int p_min = first_pos + tok_min, p_max = first_pos + tok_max;
    int t_lo = 0;
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / ATT_KEYS;
    int t_hi = p_max / ATT_KEYS + 1;
    if (num_splits > 1) {
        const int per = (t_hi - t_lo + num_splits - 1) / num_splits;
        t_lo = t_lo + split * per;
        if (t_lo + per < t_hi) t_hi = t_lo + per;
    }

    float m[ATT_RPW], l[ATT_RPW], acc[ATT_RPW][NC];
#pragma unroll
    for (int rr = 0; rr < ATT_RPW; ++rr) {
        m[rr] = -INFINITY;
        l[rr] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[rr][c] = 0.f;
    }

    for (int kt = t_lo; kt < t_hi; ++kt) {
        __syncthreads();  // the previous tile is consumed (and q_s is complete)
        if (tid < ATT_KEYS) {
            const int key = kt * ATT_KEYS + tid;
            int page = -1;
            if (key < kv_len) page = table_page(table, seq, max_pages, key / page_size);
            page_s[tid] = page;
        }
        __syncthreads();
        for (int idx = tid; idx < ATT_KEYS * d; idx += blockDim.x) {
            const int j = idx / d, c = idx - j * d;
            const int page = page_s[j];
            float kv = 0.f, vv = 0.f;
            if (page >= 0) {
                const int key = kt * ATT_KEYS + j;
                const int64_t at =
                    (((int64_t)page * n_kv + kvh) * page_size + (key % page_size)) * d + c;
                kv = to_float(k_pages[at]);
                vv = to_float(v_pages[at]);
            }
            k_s[j * (d + 1) + c] = kv;
            v_s[idx] = vv;
        }
        __syncthreads();

        // scores of this lane's key against the warp's rows
        float s[ATT_RPW];
#pragma unroll
        for (int rr = 0; rr < ATT_RPW; ++rr) s[rr] = 0.f;
        const float* krow = k_s + lane * (d + 1);
        const float* qrow = q_s + warp * ATT_RPW * d;
        for (int c = 0; c < d; ++c) {
            const float kv = krow[c];
#pragma unroll
            for (int rr = 0; rr < ATT_RPW; ++rr) s[rr] = fmaf(qrow[rr * d + c], kv, s[rr]);
        }
        const int key = kt * ATT_KEYS + lane;
        const bool key_ok = page_s[lane] >= 0;
#pragma unroll
        for (int rr = 0; rr < ATT_RPW; ++rr) {
            bool seen = row_ok[rr] && key_ok && key <= row_pos[rr];
            if (window > 0) seen = seen && key > row_pos[rr] - window;
            const float sc = seen ? s[rr] * scale : -INFINITY;
            const float m_new = fmaxf(m[rr], warp_max(sc));
            float p = 0.f, corr = 1.f;
            if (m_new > -INFINITY) {
                p = seen ? expf(sc - m_new) : 0.f;
                corr = expf(m[rr] - m_new);  // exp(-inf) = 0 on the first seen tile
            }
            l[rr] = l[rr] * corr + warp_sum(p);
            m[rr] = m_new;
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[rr][c] *= corr;
            for (int j = 0; j < ATT_KEYS; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int dim = lane + 32 * c;
                    if (dim < d) acc[rr][c] = fmaf(pj, v_s[j * d + dim], acc[rr][c]);
                }
            }
        }
    }

#pragma unroll
    for (int rr = 0; rr < ATT_RPW; ++rr) {
        if (!row_ok[rr]) continue;
        const int row = row0 + warp * ATT_RPW + rr;
        const int tok = row / group, hg = row - tok * group;
        const int64_t flat = (int64_t)(q_begin + tok) * n_q + kvh * group + hg;
        if (num_splits == 1) {
            const float inv = l[rr] > 0.f ? 1.f / l[rr] : 0.f;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int dim = lane + 32 * c;
                if (dim < d) out[flat * d + dim] = from_float<T>(acc[rr][c] * inv);
            }
        } else {
            const int64_t at = flat * num_splits + split;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int dim = lane + 32 * c;
                if (dim < d) part_acc[at * d + dim] = acc[rr][c];
            }
            if (lane == 0) {
                part_ml[at * 2] = m[rr];
                part_ml[at * 2 + 1] = l[rr];
            }
        }
    }
}

// Merge the splits of one (token, head): out = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M).
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc,
                                         const float* __restrict__ part_ml,
                                         const int* __restrict__ seq_of_token, T* __restrict__ out,
                                         int n_q, int d, int num_splits) {
    grid_dependency_sync();
    const int tok = blockIdx.x, head = blockIdx.y;
    const int64_t flat = (int64_t)tok * n_q + head;
    if (seq_of_token[tok] < 0) {
        for (int c = threadIdx.x; c < d; c += blockDim.x) out[flat * d + c] = from_float<T>(0.f);
        return;
    }
    float big = -INFINITY;
    for (int z = 0; z < num_splits; ++z) big = fmaxf(big, part_ml[(flat * num_splits + z) * 2]);
    float denom = 0.f;
    for (int z = 0; z < num_splits; ++z) {
        const float mz = part_ml[(flat * num_splits + z) * 2];
        if (mz > -INFINITY) denom += part_ml[(flat * num_splits + z) * 2 + 1] * expf(mz - big);
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = 0.f;
        for (int z = 0; z < num_splits; ++z) {
            const float mz = part_ml[(flat * num_splits + z) * 2];
            if (mz > -INFINITY) v += part_acc[(flat * num_splits + z) * d + c] * expf(mz - big);
        }
        out[flat * d + c] = from_float<T>(v * inv);
    }
}

template <typename T, int NC>
int launch_attention(const void* qkv, int q_row_stride, const void* k_pages, const void* v_pages,
                     const int* table, int max_pages, const int* q_start, const int* kv_len,
                     void* out, float* part_acc, float* part_ml, int n_q, int n_kv, int d,
                     int page_size, float scale, int window, int num_seqs, int tiles_per_seq,
                     int num_splits, cudaStream_t s) {
    const size_t smem = (size_t)(ATT_ROWS * d + ATT_KEYS * (d + 1) + ATT_KEYS * d) * sizeof(float) +
                        ATT_KEYS * sizeof(int);
    static bool raised = false;  // one flag per instantiation
    if (smem > 48 * 1024 && !raised) {
        if (cudaFuncSetAttribute(paged_attention_kernel<T, NC>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    dim3 grid(num_seqs * tiles_per_seq, n_kv, num_splits);
    MB_LAUNCH((paged_attention_kernel<T, NC>), grid, ATT_WARPS * 32, smem, s, 
        (const T*)qkv, q_row_stride, (const T*)k_pages, (const T*)v_pages, table, max_pages, q_start,
        kv_len, (T*)out, part_acc, part_ml, n_q, n_kv, d, page_size, scale, window, tiles_per_seq,
        num_splits);
    return launch_status();
}

template <typename T>
int dispatch_attention(int nc, const void* qkv, int q_row_stride, const void* k_pages,
                       const void* v_pages, const int* table, int max_pages, const int* q_start,
                       const int* kv_len, void* out, float* part_acc, float* part_ml, int n_q,
                       int n_kv, int d, int page_size, float scale, int window, int num_seqs,
                       int tiles_per_seq, int num_splits, cudaStream_t s) {
#define MB_ATT_CASE(N)                                                                           \
    case N:                                                                                      \
        return launch_attention<T, N>(qkv, q_row_stride, k_pages, v_pages, table, max_pages,     \
                                      q_start, kv_len, out, part_acc, part_ml, n_q, n_kv, d,     \
                                      page_size, scale, window, num_seqs, tiles_per_seq,         \
                                      num_splits, s)
    switch (nc) {
        MB_ATT_CASE(1);
        MB_ATT_CASE(2);
        MB_ATT_CASE(3);
        MB_ATT_CASE(4);
        MB_ATT_CASE(5);
        MB_ATT_CASE(6);
        MB_ATT_CASE(7);
        MB_ATT_CASE(8);
    }
#undef MB_ATT_CASE
    return MB_ERR_UNSUPPORTED_SIZE;
}

// Launch the merge of `num_splits` partial results per (token, head); shared by every
// attention kernel that splits keys. dtype: MB_F32 or MB_BF16 output.
int launch_attention_combine(const float* part_acc, const float* part_ml, const int* seq_of_token,
                             void* out, int tokens, int n_q, int d, int num_splits, int dtype,
                             cudaStream_t s) {
    if (n_q > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    dim3 grid(tokens, n_q);
    if (dtype == MB_F32)
        MB_LAUNCH((attention_combine_kernel<float>), grid, 64, 0, s, part_acc, part_ml, seq_of_token,
                                                            (float*)out, n_q, d, num_splits);
    else if (dtype == MB_BF16)
        MB_LAUNCH((attention_combine_kernel<__nv_bfloat16>), grid, 64, 0, s, 
            part_acc, part_ml, seq_of_token, (__nv_bfloat16*)out, n_q, d, num_splits);
    else
        return MB_ERR_BAD_DTYPE;
    return launch_status();
}

}  // namespace mb

using namespace mb;

// Scratch the split path needs, in floats: tokens * n_q * num_splits * (d + 2).
MB_EXPORT long long mb_attention_scratch_floats(int tokens, int n_q, int d, int num_splits) {
    return num_splits <= 1 ? 0 : (long long)tokens * n_q * num_splits * (d + 2);
}

// max_q_len: the most query tokens one sequence has in this batch (sizes the grid).
// scratch: float32 buffer of at least mb_attention_scratch_floats() (may be null when
// num_splits is 1). Head sizes up to 256 are taken; anything else is refused.
MB_EXPORT int mb_paged_attention_simt(const void* qkv, int q_row_stride, const void* k_pages,
                                      const void* v_pages, const int* table, int max_pages,
                                      const int* q_start, const int* kv_len,
                                      const int* seq_of_token, void* out, float* scratch,
                                      long long scratch_floats, int tokens, int num_seqs,
                                      int max_q_len, int n_q, int n_kv, int d, int page_size,
                                      float scale, int window, int num_splits, int dtype,
                                      void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (d <= 0 || d > 256 || n_kv <= 0 || n_q % n_kv) return MB_ERR_UNSUPPORTED_SIZE;
    if (page_size <= 0 || (page_size & (page_size - 1))) return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits < 1) num_splits = 1;
    if (n_kv > 65535 || num_splits > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    const int group = n_q / n_kv;
    const int tiles_per_seq = (max_q_len * group + ATT_ROWS - 1) / ATT_ROWS;
    float* part_acc = nullptr;
    float* part_ml = nullptr;
    if (num_splits > 1) {
        if (!scratch || scratch_floats < mb_attention_scratch_floats(tokens, n_q, d, num_splits))
            return MB_ERR_SCRATCH;
        part_acc = scratch;
        part_ml = scratch + (int64_t)tokens * n_q * num_splits * d;
    }
    const int nc = (d + 31) / 32;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (dtype == MB_F32)
        rc = dispatch_attention<float>(nc, qkv, q_row_stride, k_pages, v_pages, table, max_pages,
                                       q_start, kv_len, out, part_acc, part_ml, n_q, n_kv, d,
                                       page_size, scale, window, num_seqs, tiles_per_seq,
                                       num_splits, s);
    else if (dtype == MB_BF16)
        rc = dispatch_attention<__nv_bfloat16>(nc, qkv, q_row_stride, k_pages, v_pages, table,
                                               max_pages, q_start, kv_len, out, part_acc, part_ml,
                                               n_q, n_kv, d, page_size, scale, window, num_seqs,
                                               tiles_per_seq, num_splits, s);
    else
        return MB_ERR_BAD_DTYPE;
    if (rc != MB_OK || num_splits == 1) return rc;
    return launch_attention_combine(part_acc, part_ml, seq_of_token, out, tokens, n_q, d,
                                    num_splits, dtype, s);
}

// ------------------------------------------------------------------------------------------
// The variant for callers that cannot allocate: see no_alloc.h. The partial results of the
// key splits live in this file-scope array instead of a buffer handed in by the caller.
#include "no_alloc.h"

static __device__ __align__(256) float g_static_scratch[MB_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_scratch_address[kMaxDevices] = {};  // device address of the array, per device
}  // namespace

MB_EXPORT int mb_paged_attention_static(const void* qkv, int q_row_stride, const void* k_pages,
                                        const void* v_pages, const int* table, int max_pages,
                                        const int* q_start, const int* kv_len,
                                        const int* seq_of_token, void* out, int tokens,
                                        int num_seqs, int max_q_len, int n_q, int n_kv, int d,
                                        int page_size, float scale, int window, int num_splits,
                                        int dtype, void* stream) {
    if (num_splits < 1) num_splits = 1;
    if (tokens < 0 || n_q <= 0 || d <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    if (num_splits == 1)
        // One split keeps its results in registers and writes the output directly: nothing
        // of the array is used, so its size sets no limit and its address is not needed.
        return mb_paged_attention_simt(qkv, q_row_stride, k_pages, v_pages, table, max_pages,
                                       q_start, kv_len, seq_of_token, out, nullptr, 0, tokens,
                                       num_seqs, max_q_len, n_q, n_kv, d, page_size, scale, window,
                                       1, dtype, stream);
    const long long need = (long long)tokens * n_q * num_splits * (d + 2);
    if (need > MB_STATIC_SCRATCH_FLOATS) return MB_ERR_SCRATCH;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
        return MB_ERR_LAUNCH;
    if (g_static_scratch_address[device] == nullptr) {
        // In host code `g_static_scratch` is only a handle for the symbol; the address the
        // kernels need comes from the runtime, for the device that is current now. Two
        // threads making their first call at once both look the address up and both store
        // the same value: a race without consequence.
        float* address = nullptr;
        if (cudaGetSymbolAddress((void**)&address, g_static_scratch) != cudaSuccess ||
            address == nullptr)
            return MB_ERR_LAUNCH;
        g_static_scratch_address[device] = address;
    }
    // The split kernel writes every (row, split) pair that the merge kernel reads, so the
    // array needs no clearing between calls.
    return mb_paged_attention_simt(qkv, q_row_stride, k_pages, v_pages, table, max_pages, q_start,
                                   kv_len, seq_of_token, out, g_static_scratch_address[device],
                                   MB_STATIC_SCRATCH_FLOATS, tokens, num_seqs, max_q_len, n_q, n_kv,
                                   d, page_size, scale, window, num_splits, dtype, stream);
}
