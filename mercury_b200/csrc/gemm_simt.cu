// out[M, N] = x[M, K] * w[N, K]^T (+ bias[N]) on the CUDA cores with float32 FMAs.
//
// This is the product of the true 32-bit path (no tensor-core mode rounds its operands)
// and the fallback of the bfloat16 engine for shapes and dtypes its tensor-core kernels
// refuse. It stands where the reference calls F.linear (mercury/model/qwen2.py:42,
// :64-69, :149-150). Each output element is accumulated over k in ascending order by one
// thread, so a row's result does not depend on which other rows are in the batch.
//
// Tiling: a block of 256 threads computes a 64 x 64 tile, each thread a 4 x 4 patch, over
// K in steps of 16 staged through shared memory; edges are zero-filled.
#include "common.cuh"

namespace mb {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const void* __restrict__ bias,
                 int bias_dtype, TO* __restrict__ out, int M, int N, int K) {
    grid_dependency_sync();
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tr = (tid / 16) * 4, tc = (tid % 16) * 4;
    float acc[4][4] = {};
    // staging: 64 rows x 16 k per operand = 1024 elements, 4 per thread
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int m = m0 + lrow, n = n0 + lrow;
            xs[lk + j][lrow] = (m < M && k < K) ? to_float(x[(int64_t)m * K + k]) : 0.f;
            ws[lk + j][lrow] = (n < N && k < K) ? to_float(w[(int64_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][tr + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tc + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tr + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tc + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += load_as_float(bias, n, bias_dtype);
            out[(int64_t)m * N + n] = from_float<TO>(v);
        }
    }
}

template <typename TX, typename TW, typename TO>
int launch_gemm(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int M,
                int N, int K, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return MB_ERR_UNSUPPORTED_SIZE;
    MB_LAUNCH((gemm_simt_kernel<TX, TW, TO>), grid, 256, 0, s, (const TX*)x, (const TW*)w, bias, bias_dtype,
                                                     (TO*)out, M, N, K);
    return launch_status();
}

}  // namespace mb

using namespace mb;

// dtypes: MB_F32 or MB_BF16 for each of x, w, bias and out.
MB_EXPORT int mb_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias,
                           int bias_dtype, void* out, int out_dtype, int M, int N, int K,
                           void* stream) {
    if (M <= 0 || N <= 0) return MB_OK;
    if (K <= 0) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
    const int key = x_dtype * 4 + w_dtype * 2 + out_dtype;
    switch (key) {
        case 0: return launch_gemm<float, float, float>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 1: return launch_gemm<float, float, bf>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 2: return launch_gemm<float, bf, float>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 3: return launch_gemm<float, bf, bf>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 4: return launch_gemm<bf, float, float>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 5: return launch_gemm<bf, float, bf>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 6: return launch_gemm<bf, bf, float>(x, w, bias, bias_dtype, out, M, N, K, s);
        case 7: return launch_gemm<bf, bf, bf>(x, w, bias, bias_dtype, out, M, N, K, s);
    }
    return MB_ERR_BAD_DTYPE;
}
