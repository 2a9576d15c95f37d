// Token choice on the device: argmax, and temperature / top-p sampling by inverse CDF.
//
// Rules (mercury/sampling.py:17-35, mercury/request.py:21-23): a row with temperature <= 0
// is greedy (here: the lowest index among equal maxima); otherwise probabilities are
// softmax(logits / max(T, 1e-5)) in float32; with top_p < 1 a token stays iff the tokens
// strictly more probable than it hold at most top_p of the mass (the token that crosses the
// threshold stays, mercury/sampling.py:9-10; equal probabilities stay or go together);
// the draw is the first index, in index order, whose cumulative kept mass exceeds
// u * (kept mass), with u in [0, 1) supplied by the caller per row. The reference draws with
// torch.multinomial from one shared generator instead (mercury/sampling.py:34).
#include "common.cuh"

namespace mb {

constexpr int SAMPLE_THREADS = 1024;

__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    grid_dependency_sync();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (int64_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        best_v[warp] = bv;
        best_i[warp] = bi;
    }
    __syncthreads();
    if (warp == 0) {
        const int warps = blockDim.x >> 5;
        bv = lane < warps ? best_v[lane] : -INFINITY;
        bi = lane < warps ? best_i[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Large vocabularies: a row is cut into `parts` slices, one block each, which leave their
// (maximum, lowest index of it) in `partial`; argmax_merge_kernel picks the winner. One
// block per row cannot pull a 600 KB row fast enough to stay out of a decode step's way.
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, float* __restrict__ partial_v,
                      int* __restrict__ partial_i, int vocab, int parts) {
    grid_dependency_sync();
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    const int r = blockIdx.y, part = blockIdx.x;
    const float* row = logits + (int64_t)r * vocab;
    const int per = (((vocab + parts - 1) / parts) + 3) & ~3;      // a multiple of four floats
    const int begin = part * per < vocab ? part * per : vocab;
    const int end = begin + per < vocab ? begin + per : vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    };
    if ((vocab & 3) == 0 && (per & 3) == 0) {
        // 16 bytes per load and four loads in flight per thread (the slice of a row is a few
        // thousand floats: with one float per load the kernel waited for memory trip by trip)
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int b4 = begin >> 2, e4 = end >> 2;
        for (int i0 = b4 + threadIdx.x; i0 < e4; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * blockDim.x;
                v[u] = i < e4 ? row4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = (i0 + u * (int)blockDim.x) << 2;
                take(v[u].x, i);
                take(v[u].y, i + 1);
                take(v[u].z, i + 2);
                take(v[u].w, i + 3);
            }
        }
    } else {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) take(row[i], i);
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        take(ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        best_v[warp] = bv;
        best_i[warp] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) {
                bv = best_v[w];
                bi = best_i[w];
            }
        partial_v[r * parts + part] = bv;
        partial_i[r * parts + part] = bi;
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ partial_v,
                                    const int* __restrict__ partial_i, int* __restrict__ out,
                                    int parts) {
    grid_dependency_sync();
    const int r = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int p = threadIdx.x; p < parts; p += 32) {
        const float v = partial_v[r * parts + p];
        const int i = partial_i[r * parts + p];
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

// One block per row. Each thread owns a contiguous run of the vocabulary so that prefix
// sums follow index order.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ out, int vocab) {
    grid_dependency_sync();
    __shared__ float scratch[33];
    __shared__ float sums[SAMPLE_THREADS];
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (int64_t)r * vocab;
    const float temp = temperature[r];
    const int tid = threadIdx.x;

    // greedy rows: same rule as argmax_kernel
    float bv = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) bv = fmaxf(bv, row[i]);
    const float top = block_max(bv, scratch);
    if (temp <= 0.f) {
        if (tid == 0) chosen = 0x7fffffff;
        __syncthreads();
        int bi = 0x7fffffff;
        for (int i = tid; i < vocab; i += blockDim.x)
            if (row[i] == top && i < bi) bi = i;
        if (bi != 0x7fffffff) atomicMin(&chosen, bi);
        __syncthreads();
        if (tid == 0) out[r] = chosen == 0x7fffffff ? 0 : chosen;
        return;
    }
    const float inv_t = 1.f / fmaxf(temp, 1e-5f);
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int begin = tid * per;
    const int end = begin + per < vocab ? begin + per : vocab;

    // unnormalised weights e_i = exp((x_i - max) / T); total mass
    float mine = 0.f;
    for (int i = begin; i < end; ++i) mine += expf((row[i] - top) * inv_t);
    const float total = block_sum(mine, scratch);

    // top-p: the smallest weight w* such that the mass strictly above w* is <= top_p * total;
    // tokens with e_i >= w* stay. Bisection over the bit patterns of positive floats, which
    // are ordered like their values.
    float keep_from = 0.f;
    const float p_keep = top_p[r];
    if (p_keep < 1.f) {
        const float limit = p_keep * total;
        unsigned lo = 0u, hi = 0x3f800000u;  // weights lie in (0, 1]; mass above 1.0 is 0
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo) / 2;
            const float t = __uint_as_float(mid);
            float above = 0.f;
            for (int i = begin; i < end; ++i) {
                const float e = expf((row[i] - top) * inv_t);
                above += e > t ? e : 0.f;
            }
            above = block_sum(above, scratch);
            if (above <= limit) hi = mid; else lo = mid + 1;
        }
        keep_from = __uint_as_float(lo);
    }

    // inverse CDF over the kept tokens, in index order
    mine = 0.f;
    for (int i = begin; i < end; ++i) {
        const float e = expf((row[i] - top) * inv_t);
        mine += e >= keep_from ? e : 0.f;
    }
    sums[tid] = mine;
    if (tid == 0) chosen = 0x7fffffff;
    __syncthreads();
    // exclusive prefix of the per-thread sums, left to right (index order), by one warp
    if (tid < 32) {
        const int chunk = blockDim.x / 32;
        float run = 0.f;
        for (int j = 0; j < chunk; ++j) run += sums[tid * chunk + j];
        float incl = run;
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (tid >= o) incl += up;
        }
        float base = incl - run;
        for (int j = 0; j < chunk; ++j) {
            const float v = sums[tid * chunk + j];
            sums[tid * chunk + j] = base;
            base += v;
        }
        if (tid == 31) scratch[0] = incl;
    }
    __syncthreads();
    const float kept_total = scratch[0];
    const float target = uniform[r] * kept_total;
    float cum = sums[tid];
    int last_kept = -1;
    for (int i = begin; i < end; ++i) {
        const float e = expf((row[i] - top) * inv_t);
        if (e >= keep_from) {
            cum += e;
            last_kept = i;
            if (cum > target) {
                atomicMin(&chosen, i);
                break;
            }
        }
    }
    __syncthreads();
    // rounding may leave the target just above the last cumulative sum: take the last kept token
    __shared__ int fallback;
    if (tid == 0) fallback = -1;
    __syncthreads();
    if (chosen == 0x7fffffff && last_kept >= 0) atomicMax(&fallback, last_kept);
    __syncthreads();
    if (tid == 0) out[r] = chosen != 0x7fffffff ? chosen : (fallback >= 0 ? fallback : 0);
}

}  // namespace mb

using namespace mb;

// `scratch`: room for rows * 64 floats and rows * 64 ints (8 bytes per slot), or null to use
// the one-block-per-row kernel.
MB_EXPORT int mb_argmax(const float* logits, int* out, int rows, int vocab, void* scratch,
                        void* stream) {
    if (rows <= 0) return MB_OK;
    if (vocab <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    if (scratch && vocab >= 16384 && rows <= 65535) {
        const int parts = 64;
        float* pv = reinterpret_cast<float*>(scratch);
        int* pi = reinterpret_cast<int*>(pv + (size_t)rows * parts);
        MB_LAUNCH((argmax_partial_kernel), dim3(parts, rows), 256, 0, (cudaStream_t)stream, logits, pv,
                  pi, vocab, parts);
        MB_LAUNCH((argmax_merge_kernel), rows, 32, 0, (cudaStream_t)stream, (const float*)pv,
                  (const int*)pi, out, parts);
        return launch_status();
    }
    MB_LAUNCH((argmax_kernel), rows, SAMPLE_THREADS, 0, (cudaStream_t)stream, logits, out, vocab);
    return launch_status();
}

MB_EXPORT int mb_sample(const float* logits, const float* temperature, const float* top_p,
                        const float* uniform, int* out, int rows, int vocab, void* stream) {
    if (rows <= 0) return MB_OK;
    if (vocab <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    MB_LAUNCH((sample_kernel), rows, SAMPLE_THREADS, 0, (cudaStream_t)stream, logits, temperature, top_p,
                                                                    uniform, out, vocab);
    return launch_status();
}
