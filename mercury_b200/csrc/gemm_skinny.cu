// Products with few rows of activations (decode steps): out[t, n] = sum_k x[t, k] w[n, k],
// for up to 16 tokens, bfloat16 operands, float32 accumulation, on the tensor cores
// (mma.sync m16n8k16) with the roles swapped: 16 weight rows are the M side of the MMA and
// 8 tokens its N side, so that no tensor-core work is wasted on padding tokens.
//
// Such a product is bound by the time to stream the weight matrix once from HBM, and for
// the small matrices of a layer by latency, so the kernel is laid out to have every byte
// of the matrix in flight at once: a warp owns 16 weight rows over a share of K and reads
// them with 16-byte loads straight into MMA fragments (the k order inside a 32-wide chunk
// is permuted identically for weights and activations, which leaves dot products
// unchanged); the activations are small and come through L1. Warps that split K meet in
// shared memory, where the epilogue runs:
//   plain    (+ bias) -> bfloat16 or float32 rows            (LM head)
//   residual (+ bias) added into the float32 residual stream (o-proj, down-proj), each
//            element by the one thread that owns it
//   swiglu   silu(gate) * up for paired gate/up row tiles    (mercury/model/qwen2.py:42)
//   rope     bias, rotary encoding of q and k, q written back, k and v stored into the
//            token's cache page (mercury/model/rope.py:11-17, mercury/model/attention.py:35-45)
// The activations may also be given as the float32 residual stream plus an RMSNorm weight:
// then every block first computes the rows' 1/rms itself (the stream is a few KB) and
// builds the normalised bfloat16 activations on the fly, which saves the norm's own launch
// (mercury/model/qwen2.py:29-31 for the formula).
// Sizes it takes: K a multiple of 32, N a multiple of 16, at most 16 tokens (eight per
// block, the second eight in a block further along z); the callers fall back to the general
// kernels otherwise.
#include "tcgen05.cuh"

namespace mb {

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Where the activations of a product come from: bfloat16 rows `x`, or (norm_w != null) the
// float32 stream `h` to be normalised with `norm_w`; `rows` optionally picks the rows.
struct SkinnyInput {
    const __nv_bfloat16* x;
    const float* h;
    const __nv_bfloat16* norm_w;
    const int* rows;
    float eps;
    // deferred RMSNorm scale: x holds stream * norm weight (not yet divided by the rms), and
    // ss_part[tok * ss_tiles + j] the sums of squares of the stream's 16-column tiles, left
    // by the product that updated the stream; 1/rms multiplies this product's result rows
    const float* ss_part;
    int ss_tiles;
    float ss_eps;
    int ss_k;
};

// 1/rms of each row from the partial sums of squares, into scale_s[T] (ones without them).
__device__ __forceinline__ void skinny_row_scale(const SkinnyInput& in, int T, float* scale_s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int tok = warp; tok < T; tok += warps) {
        float ss = 0.f;
        if (in.ss_part) {
            for (int j = lane; j < in.ss_tiles; j += 32) ss += in.ss_part[(int64_t)tok * in.ss_tiles + j];
            ss = warp_sum(ss);
        }
        if (lane == 0) scale_s[tok] = in.ss_part ? rsqrtf(ss / (float)in.ss_k + in.ss_eps) : 1.f;
    }
}

// 1/rms of each of the T rows of the stream, by the whole block, into rstd_s[T].
__device__ __forceinline__ void skinny_row_rstd(const SkinnyInput& in, int T, int K, float* rstd_s) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int tok = warp; tok < T; tok += warps) {
        const float* row = in.h + (int64_t)(in.rows ? in.rows[tok] : tok) * K;
        float ss = 0.f;
        for (int k = lane * 4; k < K; k += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + k);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = warp_sum(ss);
        if (lane == 0) rstd_s[tok] = rsqrtf(ss / (float)K + in.eps);
    }
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One warp: rows [n0, n0+16) of w against tokens [0, 8*NT) over chunks [c_begin, c_end)
// of 32 k each. acc[nt] holds (row g, tokens 2t, 2t+1) and (row g+8, tokens 2t, 2t+1).
// Loads are issued four chunks ahead of their use, so a warp whose share of K is four
// chunks or fewer pays one trip to memory.
template <int NT, bool NORM>
__device__ __forceinline__ void skinny_mainloop(const SkinnyInput& in, const float* rstd_s,
                                                const __nv_bfloat16* __restrict__ w, int n0, int T,
                                                int K, int c_begin, int c_end, float (&acc)[NT][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const __nv_bfloat16* wa = w + (int64_t)(n0 + g) * K + 8 * t4;
    const __nv_bfloat16* wb = w + (int64_t)(n0 + g + 8) * K + 8 * t4;
    const __nv_bfloat16* xr[NT];
    const float* hr[NT];
    float rs[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        int tok = nt * 8 + g;
        if (tok > T - 1) tok = T - 1;  // padding tokens read a real row; their columns are dropped
        if (NORM) {
            hr[nt] = in.h + (int64_t)(in.rows ? in.rows[tok] : tok) * K + 8 * t4;
            rs[nt] = rstd_s[tok];
        } else {
            xr[nt] = in.x + (int64_t)tok * K + 8 * t4;
        }
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int c0 = c_begin; c0 < c_end; c0 += 4) {
        uint4 a[4], b[4], xv[4][NT];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = c0 + j;
            const bool ok = c < c_end;
            a[j] = ok ? __ldg(reinterpret_cast<const uint4*>(wa + c * 32)) : zero;
            b[j] = ok ? __ldg(reinterpret_cast<const uint4*>(wb + c * 32)) : zero;
            if (NORM) {
                uint4 nq = zero;
                if (ok) nq = __ldg(reinterpret_cast<const uint4*>(in.norm_w + c * 32 + 8 * t4));
                const __nv_bfloat162* n2 = reinterpret_cast<const __nv_bfloat162*>(&nq);
                const float2 w0 = __bfloat1622float2(n2[0]), w1 = __bfloat1622float2(n2[1]);
                const float2 w2 = __bfloat1622float2(n2[2]), w3 = __bfloat1622float2(n2[3]);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
                    if (ok) {
                        lo = *reinterpret_cast<const float4*>(hr[nt] + c * 32);
                        hi = *reinterpret_cast<const float4*>(hr[nt] + c * 32 + 4);
                    }
                    const float r = rs[nt];
                    xv[j][nt].x = pack2(lo.x * r * w0.x, lo.y * r * w0.y);
                    xv[j][nt].y = pack2(lo.z * r * w1.x, lo.w * r * w1.y);
                    xv[j][nt].z = pack2(hi.x * r * w2.x, hi.y * r * w2.y);
                    xv[j][nt].w = pack2(hi.z * r * w3.x, hi.w * r * w3.y);
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt)
                    xv[j][nt] = ok ? *reinterpret_cast<const uint4*>(xr[nt] + c * 32) : zero;
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma_bf16_16816(acc[nt], a[j].x, b[j].x, a[j].y, b[j].y, xv[j][nt].x, xv[j][nt].y);
                mma_bf16_16816(acc[nt], a[j].z, b[j].z, a[j].w, b[j].w, xv[j][nt].z, xv[j][nt].w);
            }
        }
    }
}

constexpr int SKINNY_PREFETCH_CHUNKS = 8;   // 512 bytes of each weight row

// Ask L2 for this warp's share of the weight rows. Issued before the kernel waits for its
// predecessor (weights do not depend on it), so that with programmatic dependent launch the
// weight stream overlaps the tail of the kernel before.
__device__ __forceinline__ void skinny_prefetch_weights(const __nv_bfloat16* __restrict__ w, int n0,
                                                        int K, int c_begin, int c_end) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    // one 128-byte line holds two chunks of a row: lanes with t4 == 0 cover the even chunks
    if (t4 != 0) return;
    const __nv_bfloat16* wa = w + (int64_t)(n0 + g) * K;
    const __nv_bfloat16* wb = w + (int64_t)(n0 + g + 8) * K;
    // a long share is not asked for in full: every resident block doing so would push more
    // through L2 than it holds (the loads of the main loop stream the rest)
    if (c_end > c_begin + SKINNY_PREFETCH_CHUNKS) c_end = c_begin + SKINNY_PREFETCH_CHUNKS;
    for (int c = c_begin; c < c_end; c += 2) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(wa + c * 32));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(wb + c * 32));
    }
}

// K may also be shared between the blocks of a thread-block cluster (`slices` along y): block
// `slice` walks its part of K, leaves its sums in the shared memory of the cluster's first
// block, and after one cluster barrier the first block alone runs the epilogue. A product
// with few row tiles and a long K (down-proj, q/k/v) so gets more SMs to pull its weights.
__device__ __forceinline__ void cluster_rank_size(uint32_t& rank, uint32_t& size) {
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(size));
}

__device__ __forceinline__ void cluster_store_to_first(float* local_slot, float v) {
    uint32_t remote;
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(local_slot);
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// This block's part [s0, s1) of the K chunks and, inside it, this warp's share.
__device__ __forceinline__ void skinny_share(int chunks, uint32_t slice, uint32_t slices, int ks, int ksplit,
                                             int& c_begin, int& c_end) {
    const int per_slice = (chunks + (int)slices - 1) / (int)slices;
    const int s0 = (int)slice * per_slice;
    const int s1 = s0 + per_slice < chunks ? s0 + per_slice : chunks;
    const int per = (s1 - s0 + ksplit - 1) / ksplit;
    c_begin = s0 + ks * per;
    c_end = c_begin + per < s1 ? c_begin + per : s1;
    if (c_begin > c_end) c_begin = c_end;
}

// Every warp leaves its 16 x (8 NT) partial tile in shared memory: red[warp][row][token].
template <int NT>
__device__ __forceinline__ void store_partial(float* red, const float (&acc)[NT][4]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t4 = lane & 3;
    float* mine = red + warp * 16 * (8 * NT);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mine[g * (8 * NT) + nt * 8 + 2 * t4] = acc[nt][0];
        mine[g * (8 * NT) + nt * 8 + 2 * t4 + 1] = acc[nt][1];
        mine[(g + 8) * (8 * NT) + nt * 8 + 2 * t4] = acc[nt][2];
        mine[(g + 8) * (8 * NT) + nt * 8 + 2 * t4 + 1] = acc[nt][3];
    }
}

// A block holds `rowt` row tiles of 16 weight rows, each shared by `ksplit` warps that
// split K between them (rowt * ksplit warps in all, warp = tile * ksplit + share).
// EPI: 0 = bfloat16 out, 1 = float32 out, 2 = swiglu (bfloat16 out; the row tiles of a
// block alternate gate / up, and `half_n` is the width of the result), 3 = added into the
// float32 rows of `out`.
// Threads a block of this kernel may have: eight tokens per block leave room for 1024 (the
// gated form is built for three blocks of 448 per SM); sixteen tokens per block keep twice
// the activation fragments and sums in registers and get half the threads.
constexpr int skinny_max_threads(int NT, int EPI, bool NORM) {
    return NT == 2 ? 512 : (NORM ? 512 : (EPI == 2 ? 448 : 1024));
}

template <int NT, int EPI, bool NORM>
__global__ void __launch_bounds__(skinny_max_threads(NT, EPI, NORM), (NT == 1 && EPI == 2 && !NORM) ? 3 : 1)
skinny_gemm_kernel(SkinnyInput in_all,
                                   const __nv_bfloat16* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ bias, void* __restrict__ out_all,
                                   int T_all, int N, int K, int half_n, int rowt, int ksplit,
                                   const __nv_bfloat16* __restrict__ next_norm_w,
                                   __nv_bfloat16* __restrict__ next_x_all,
                                   float* __restrict__ next_ss_all, int h_stable) {
    constexpr int TOK = 8 * NT;
    // Tokens beyond the first TOK belong to the blocks further along z: block z takes tokens
    // [z TOK, z TOK + TOK), with every pointer that is indexed by token moved there.
    SkinnyInput in = in_all;
    const int t0 = blockIdx.z * TOK;
    const int T = T_all - t0 < TOK ? T_all - t0 : TOK;
    if (in.x) in.x += (int64_t)t0 * K;
    if (in.rows) in.rows += t0;
    else if (in.h) in.h += (int64_t)t0 * K;
    if (in.ss_part) in.ss_part += (int64_t)t0 * in.ss_tiles;
    void* out = EPI == 0 ? (void*)(reinterpret_cast<__nv_bfloat16*>(out_all) + (int64_t)t0 * N)
              : EPI == 2 ? (void*)(reinterpret_cast<__nv_bfloat16*>(out_all) + (int64_t)t0 * half_n)
                         : (void*)(reinterpret_cast<float*>(out_all) + (int64_t)t0 * N);
    __nv_bfloat16* next_x = next_x_all ? next_x_all + (int64_t)t0 * N : nullptr;
    float* next_ss = next_ss_all ? next_ss_all + (int64_t)t0 * (N / 16) : nullptr;
    extern __shared__ float red[];  // [rowt * ksplit][16][TOK]
    __shared__ float rstd_s[TOK];
    __shared__ float scale_s[TOK];
    const int warp = threadIdx.x >> 5;
    const int rt = warp / ksplit, ks = warp - rt * ksplit;
    int n0;  // first weight row of this warp's tile
    if (EPI == 2) {
        const int pair = blockIdx.x * (rowt / 2) + rt / 2;
        n0 = (rt & 1) * half_n + pair * 16;
    } else {
        n0 = (blockIdx.x * rowt + rt) * 16;
    }
    const int limit = EPI == 2 ? ((rt & 1) + 1) * half_n : N;
    uint32_t slice, slices;
    cluster_rank_size(slice, slices);
    int c_begin, c_end;
    skinny_share(K / 32, slice, slices, ks, ksplit, c_begin, c_end);
    if (n0 < limit) skinny_prefetch_weights(w, n0, K, c_begin, c_end);
    // The stream element this thread will add to (EPI 3, one element per thread when the
    // block has at least 16 TOK threads per tile): read before the wait when the caller says
    // that the kernel in front does not write the stream.
    // Bias and the next norm's weight of that element are weights: read before the wait too.
    float h_early = 0.f, bias_early = 0.f, next_w_early = 0.f;
    const bool one_each = EPI != 2 && (int)blockDim.x >= rowt * 16 * TOK;
    const bool early = EPI == 3 && h_stable && one_each;
    if (one_each) {
        const int idx = threadIdx.x;
        if (idx < rowt * 16 * TOK) {
            const int r = idx % 16, tok = (idx / 16) % TOK, tile = idx / (16 * TOK);
            const int n = (blockIdx.x * rowt + tile) * 16 + r;
            if (tok < T && n < N) {
                if (early) h_early = reinterpret_cast<const float*>(out)[(int64_t)tok * N + n];
                if (bias) bias_early = __bfloat162float(bias[n]);
                if (EPI == 3 && next_norm_w) next_w_early = __bfloat162float(next_norm_w[n]);
            }
        }
    }
    grid_dependency_sync();
    skinny_row_scale(in, T, scale_s);     // read after the barrier that follows the product
    if (NORM) {
        skinny_row_rstd(in, T, K, rstd_s);
        __syncthreads();
    }
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    if (n0 < limit) skinny_mainloop<NT, NORM>(in, rstd_s, w, n0, T, K, c_begin, c_end, acc);
    if (EPI == 2 && next_norm_w != nullptr && blockIdx.z == 0) {
        // The gated form has no next norm: its two spare arguments name the matrix of the
        // product behind it (`h_stable` lines of 128 bytes from `next_norm_w` on). This
        // kernel's own weights are in by now, so L2 is asked for those lines here: they travel
        // while this kernel reduces, stores and leaves, and the product behind (whose blocks
        // of 1024 threads cannot be resident beside these) finds them there.
        const char* ahead = reinterpret_cast<const char*>(next_norm_w);
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < h_stable;
             i += (long long)gridDim.x * blockDim.x)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(ahead + i * 128));
    }
    store_partial<NT>(red, acc);
    __syncthreads();

    // gathered[j][idx]: the sums of the cluster's block j + 1, in the first block's memory
    float* gathered = red + rowt * ksplit * 16 * TOK;
    if (EPI != 2 && slices > 1) {
        if (slice != 0) {
            for (int idx = threadIdx.x; idx < rowt * 16 * TOK; idx += blockDim.x) {
                const int r = idx % 16, tok = (idx / 16) % TOK, tile = idx / (16 * TOK);
                float v = 0.f;
                for (int k = 0; k < ksplit; ++k) v += red[(tile * ksplit + k) * 16 * TOK + r * TOK + tok];
                cluster_store_to_first(gathered + (slice - 1) * rowt * 16 * TOK + idx, v);
            }
        }
        cluster_barrier();
        if (slice != 0) return;
    }

    if (EPI == 2) {
        // element (pair tile p, row r, token): silu(gate) * up
        for (int idx = threadIdx.x; idx < (rowt / 2) * 16 * TOK; idx += blockDim.x) {
            const int r = idx % 16, tok = (idx / 16) % TOK, p = idx / (16 * TOK);
            const int n = (blockIdx.x * (rowt / 2) + p) * 16 + r;
            if (tok >= T || n >= half_n) continue;
            float gate = 0.f, up = 0.f;
            for (int k = 0; k < ksplit; ++k) {
                gate += red[((2 * p) * ksplit + k) * 16 * TOK + r * TOK + tok];
                up += red[((2 * p + 1) * ksplit + k) * 16 * TOK + r * TOK + tok];
            }
            // the separate kernels round gate and up to bfloat16 between product and gate
            gate = __bfloat162float(__float2bfloat16_rn(gate * scale_s[tok]));
            up = __bfloat162float(__float2bfloat16_rn(up * scale_s[tok]));
            reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * half_n + n] =
                __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
    } else {
        // (the loop bound and the block size are multiples of 32: whole warps run it, and
        // the 16 rows of one (tile, token) sit in one half-warp)
        for (int idx = threadIdx.x; idx < rowt * 16 * TOK; idx += blockDim.x) {
            const int r = idx % 16, tok = (idx / 16) % TOK, tile = idx / (16 * TOK);
            const int tile_global = blockIdx.x * rowt + tile;
            const int n = tile_global * 16 + r;
            const bool live = tok < T && n < N;
            float v = 0.f;
            for (int k = 0; k < ksplit; ++k) v += red[(tile * ksplit + k) * 16 * TOK + r * TOK + tok];
            for (uint32_t j = 1; j < slices; ++j) v += gathered[(j - 1) * rowt * 16 * TOK + idx];
            v *= scale_s[tok < T ? tok : 0];
            if (bias && live) v += one_each ? bias_early : __bfloat162float(bias[n]);
            float sq = 0.f;
            if (live) {
                if (EPI == 0) {
                    reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
                } else if (EPI == 3) {
                    float* at = reinterpret_cast<float*>(out) + (int64_t)tok * N + n;
                    const float updated = (early ? h_early : *at) + v;
                    *at = updated;
                    if (next_norm_w) {
                        // for the product after the next norm: the stream times that norm's
                        // weight, and this tile's share of the row's sum of squares
                        next_x[(int64_t)tok * N + n] = __float2bfloat16_rn(
                            updated * (one_each ? next_w_early : __bfloat162float(next_norm_w[n])));
                        sq = updated * updated;
                    }
                } else {
                    reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
                }
            }
            if (EPI == 3 && next_norm_w) {
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (r == 0 && tok < T && tile_global * 16 < N)
                    next_ss[(int64_t)tok * (N / 16) + tile_global] = sq;
            }
        }
    }
}

// The same product for matrices that are bound by HBM alone (tens of megabytes and more):
// the weights do not come by per-thread loads but by TMA. Every warp owns a ring of
// SKINNY_FED_STAGES boxes of 16 rows x 64 k (2 KB, 128-byte swizzle) of its own row tile and
// K share, filled by copies that its first lane issues and waits for on the warp's own
// mbarriers; the ring is filled before the kernel waits for the one in front. A warp keeps
// 8 KB in flight without holding a register for it, 16 warps 128 KB per SM, which is what
// the per-thread loads above could not: they stream at 3.6 TB/s, this at the rate of a TMA
// copy. The fragments are read from shared memory in the same permuted-k order as above
// (16 bytes per lane: the swizzle keeps the eight rows of a quarter-warp apart), the
// activations still come through L1, and the epilogues are those of skinny_gemm_kernel.
// K a multiple of 64; at most 16 warps per block; eight tokens per block, more along z.
constexpr int SKINNY_FED_STAGES = 4;

template <int EPI, int NT>
__global__ void __launch_bounds__(512)
skinny_fed_kernel(const __grid_constant__ CUtensorMap wmap, SkinnyInput in_all,
                  const __nv_bfloat16* __restrict__ bias, void* __restrict__ out_all, int T_all, int N,
                  int K, int half_n, int rowt, int ksplit,
                  const __nv_bfloat16* __restrict__ next_norm_w, __nv_bfloat16* __restrict__ next_x_all,
                  float* __restrict__ next_ss_all, int* __restrict__ error) {
    constexpr int TOK = 8 * NT;
    constexpr int STG = SKINNY_FED_STAGES;
    SkinnyInput in = in_all;
    const int t0 = blockIdx.z * TOK;
    const int T = T_all - t0 < TOK ? T_all - t0 : TOK;
    if (in.x) in.x += (int64_t)t0 * K;
    if (in.ss_part) in.ss_part += (int64_t)t0 * in.ss_tiles;
    void* out = EPI == 0 ? (void*)(reinterpret_cast<__nv_bfloat16*>(out_all) + (int64_t)t0 * N)
              : EPI == 2 ? (void*)(reinterpret_cast<__nv_bfloat16*>(out_all) + (int64_t)t0 * half_n)
                         : (void*)(reinterpret_cast<float*>(out_all) + (int64_t)t0 * N);
    __nv_bfloat16* next_x = next_x_all ? next_x_all + (int64_t)t0 * N : nullptr;
    float* next_ss = next_ss_all ? next_ss_all + (int64_t)t0 * (N / 16) : nullptr;

    extern __shared__ __align__(1024) unsigned char fed_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(fed_raw) + 1023) & ~(uintptr_t)1023);   // [warps][STG][2048]
    float* red = reinterpret_cast<float*>(ring + (size_t)rowt * ksplit * STG * 2048);  // [warps][16][TOK]
    __shared__ uint64_t full[16][STG];
    __shared__ float scale_s[TOK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int rt = warp / ksplit, ks = warp - rt * ksplit;
    int n0;
    if (EPI == 2) {
        const int pair = blockIdx.x * (rowt / 2) + rt / 2;
        n0 = (rt & 1) * half_n + pair * 16;
    } else {
        n0 = (blockIdx.x * rowt + rt) * 16;
    }
    const int limit = EPI == 2 ? ((rt & 1) + 1) * half_n : N;
    // this warp's boxes of 64 k
    const int boxes_all = K / 64;
    const int per = (boxes_all + ksplit - 1) / ksplit;
    const int b_begin = ks * per < boxes_all ? ks * per : boxes_all;
    const int b_end = b_begin + per < boxes_all ? b_begin + per : boxes_all;
    const int boxes = n0 < limit ? b_end - b_begin : 0;
    unsigned char* mine = ring + (size_t)warp * STG * 2048;
    if (lane == 0) {
        for (int st = 0; st < STG; ++st) mbar_init(&full[warp][st], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int st = 0; st < STG && st < boxes; ++st) {
            mbar_expect_tx(&full[warp][st], 2048u);
            tma_load_2d(mine + st * 2048, &wmap, (b_begin + st) * 64, n0, &full[warp][st]);
        }
    }
    __syncwarp();
    grid_dependency_sync();
    skinny_row_scale(in, T, scale_s);     // read after the barrier that follows the product

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    {
        const __nv_bfloat16* xr[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            int tok = nt * 8 + g;
            if (tok > T - 1) tok = T - 1;      // padding tokens read a real row; their columns are dropped
            xr[nt] = in.x + (int64_t)tok * K + 8 * t4;
        }
        const uint32_t sw = (uint32_t)(g & 7);
        bool ok = true;
        for (int b = 0; b < boxes; ++b) {
            const int st = b % STG;
            // the activations of this box: asked for before the wait for its weights
            uint4 x0[NT], x1[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                x0[nt] = *reinterpret_cast<const uint4*>(xr[nt] + (int64_t)(b_begin + b) * 64);
                x1[nt] = *reinterpret_cast<const uint4*>(xr[nt] + (int64_t)(b_begin + b) * 64 + 32);
            }
            ok = mbar_wait(&full[warp][st], (uint32_t)((b / STG) & 1), error, 7);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const unsigned char* box = mine + st * 2048;
            // rows g and g + 8, 16-byte piece t4 of the first and of the second 32 k
            const uint4 a0 = *reinterpret_cast<const uint4*>(box + g * 128 + (((uint32_t)t4) ^ sw) * 16);
            const uint4 b0 = *reinterpret_cast<const uint4*>(box + (g + 8) * 128 + (((uint32_t)t4) ^ sw) * 16);
            const uint4 a1 = *reinterpret_cast<const uint4*>(box + g * 128 + (((uint32_t)(4 + t4)) ^ sw) * 16);
            const uint4 b1 = *reinterpret_cast<const uint4*>(box + (g + 8) * 128 + (((uint32_t)(4 + t4)) ^ sw) * 16);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                mma_bf16_16816(acc[nt], a0.x, b0.x, a0.y, b0.y, x0[nt].x, x0[nt].y);
                mma_bf16_16816(acc[nt], a0.z, b0.z, a0.w, b0.w, x0[nt].z, x0[nt].w);
                mma_bf16_16816(acc[nt], a1.x, b1.x, a1.y, b1.y, x1[nt].x, x1[nt].y);
                mma_bf16_16816(acc[nt], a1.z, b1.z, a1.w, b1.w, x1[nt].z, x1[nt].w);
            }
            __syncwarp();      // every lane has used what it read of the box: fill it again
            if (lane == 0 && b + STG < boxes) {
                mbar_expect_tx(&full[warp][st], 2048u);
                tma_load_2d(mine + st * 2048, &wmap, (b_begin + b + STG) * 64, n0, &full[warp][st]);
            }
        }
    }
    {
        float* part = red + warp * 16 * TOK;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            part[g * TOK + nt * 8 + 2 * t4] = acc[nt][0];
            part[g * TOK + nt * 8 + 2 * t4 + 1] = acc[nt][1];
            part[(g + 8) * TOK + nt * 8 + 2 * t4] = acc[nt][2];
            part[(g + 8) * TOK + nt * 8 + 2 * t4 + 1] = acc[nt][3];
        }
    }
    __syncthreads();

    if (EPI == 2) {
        for (int idx = threadIdx.x; idx < (rowt / 2) * 16 * TOK; idx += blockDim.x) {
            const int r = idx % 16, tok = (idx / 16) % TOK, p = idx / (16 * TOK);
            const int n = (blockIdx.x * (rowt / 2) + p) * 16 + r;
            if (tok >= T || n >= half_n) continue;
            float gate = 0.f, up = 0.f;
            for (int k = 0; k < ksplit; ++k) {
                gate += red[((2 * p) * ksplit + k) * 16 * TOK + r * TOK + tok];
                up += red[((2 * p + 1) * ksplit + k) * 16 * TOK + r * TOK + tok];
            }
            gate = __bfloat162float(__float2bfloat16_rn(gate * scale_s[tok]));
            up = __bfloat162float(__float2bfloat16_rn(up * scale_s[tok]));
            reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * half_n + n] =
                __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
        }
    } else {
        for (int idx = threadIdx.x; idx < rowt * 16 * TOK; idx += blockDim.x) {
            const int r = idx % 16, tok = (idx / 16) % TOK, tile = idx / (16 * TOK);
            const int tile_global = blockIdx.x * rowt + tile;
            const int n = tile_global * 16 + r;
            const bool live = tok < T && n < N;
            float v = 0.f;
            for (int k = 0; k < ksplit; ++k) v += red[(tile * ksplit + k) * 16 * TOK + r * TOK + tok];
            v *= scale_s[tok < T ? tok : 0];
            if (bias && live) v += __bfloat162float(bias[n]);
            float sq = 0.f;
            if (live) {
                if (EPI == 0) {
                    reinterpret_cast<__nv_bfloat16*>(out)[(int64_t)tok * N + n] = __float2bfloat16_rn(v);
                } else if (EPI == 3) {
                    float* at = reinterpret_cast<float*>(out) + (int64_t)tok * N + n;
                    const float updated = *at + v;
                    *at = updated;
                    if (next_norm_w) {
                        next_x[(int64_t)tok * N + n] =
                            __float2bfloat16_rn(updated * __bfloat162float(next_norm_w[n]));
                        sq = updated * updated;
                    }
                } else {
                    reinterpret_cast<float*>(out)[(int64_t)tok * N + n] = v;
                }
            }
            if (EPI == 3 && next_norm_w) {
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                if (r == 0 && tok < T && tile_global * 16 < N)
                    next_ss[(int64_t)tok * (N / 16) + tile_global] = sq;
            }
        }
    }
}

// One block per head of the packed q/k/v projection: D/16 row tiles, each shared by
// `ksplit` warps. After the product: bias, rotation of q and k heads (pairs i, i + D/2),
// q written to the qkv buffer, k and v written to the token's slot of the cache page.
// Where each token goes (position, page), the bias and the rotation angles are fetched
// before the kernel waits for the one in front.
template <int NT, int D, bool NORM>
__global__ void __launch_bounds__(NORM ? 512 : 1024) skinny_qkv_rope_kernel(SkinnyInput in,
                                       const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ bias,
                                       __nv_bfloat16* __restrict__ qkv,
                                       const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t,
                                       const int* __restrict__ positions,
                                       const int* __restrict__ seq_of_token,
                                       const int* __restrict__ table, int max_pages,
                                       __nv_bfloat16* __restrict__ k_pages,
                                       __nv_bfloat16* __restrict__ v_pages, int T, int K, int n_q,
                                       int n_kv, int page_size, int store, int ksplit) {
    constexpr int ROWT = D / 16;
    uint32_t slice, slices;
    cluster_rank_size(slice, slices);
    int c_begin, c_end;
    {
        const int w_ = threadIdx.x >> 5;
        const int rt_ = w_ / ksplit, ks_ = w_ - rt_ * ksplit;
        skinny_share(K / 32, slice, slices, ks_, ksplit, c_begin, c_end);
        skinny_prefetch_weights(w, blockIdx.x * D + rt_ * 16, K, c_begin, c_end);
    }
    constexpr int TOK = 8 * NT;
    extern __shared__ float red[];          // [ROWT * ksplit][16][TOK]
    float* val = red + ROWT * ksplit * 16 * TOK;  // [TOK][D]
    __shared__ int tok_pos[TOK];
    __shared__ int tok_page[TOK];           // -2: padding token, -1: no page
    __shared__ float rstd_s[TOK];
    __shared__ float scale_s[TOK];
    __shared__ float bias_s[D];
    __shared__ float cos_s[TOK][D / 2], sin_s[TOK][D / 2];
    const int head = blockIdx.x;  // 0..n_q-1 q heads, then k heads, then v heads
    // Positions, block tables, bias and rotation angles do not depend on the kernel in front
    // (they were on the device before the step began): all of them are fetched before the
    // wait, so that after it only the activations are missing.
    if (threadIdx.x < TOK) {
        const int tok = threadIdx.x;
        int pos = 0, page = -2;
        if (tok < T) {
            const int seq = seq_of_token[tok];
            if (seq >= 0) {
                pos = checked_position(positions[tok]);
                page = (store && head >= n_q) ? table_page(table, seq, max_pages, pos / page_size) : -1;
            }
        }
        tok_pos[tok] = pos;
        tok_page[tok] = page;
    }
    for (int r = threadIdx.x; r < D; r += blockDim.x)
        bias_s[r] = bias ? __bfloat162float(bias[head * D + r]) : 0.f;
    if (cos_t && head < n_q + n_kv) {
        for (int idx = threadIdx.x; idx < TOK * (D / 2); idx += blockDim.x) {
            const int i = idx % (D / 2), tok = idx / (D / 2);
            int pos = 0;
            if (tok < T && seq_of_token[tok] >= 0) pos = checked_position(positions[tok]);
            cos_s[tok][i] = cos_t[(int64_t)pos * (D / 2) + i];
            sin_s[tok][i] = sin_t[(int64_t)pos * (D / 2) + i];
        }
    }
    grid_dependency_sync();
    skinny_row_scale(in, T, scale_s);
    if (NORM) {
        skinny_row_rstd(in, T, K, rstd_s);
        __syncthreads();
    }
    const int warp = threadIdx.x >> 5;
    const int rt = warp / ksplit, ks = warp - rt * ksplit;
    const int n0 = head * D + rt * 16;
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    skinny_mainloop<NT, NORM>(in, rstd_s, w, n0, T, K, c_begin, c_end, acc);
    store_partial<NT>(red, acc);
    __syncthreads();
    // gathered[j][idx]: the sums of the cluster's block j + 1, in the first block's memory
    float* gathered = val + TOK * D;
    if (slices > 1) {
        if (slice != 0) {
            for (int idx = threadIdx.x; idx < D * TOK; idx += blockDim.x) {
                const int r = idx % D, tok = idx / D;
                const int tile = r / 16, rr = r % 16;
                float v = 0.f;
                for (int k = 0; k < ksplit; ++k) v += red[(tile * ksplit + k) * 16 * TOK + rr * TOK + tok];
                cluster_store_to_first(gathered + (slice - 1) * D * TOK + idx, v);
            }
        }
        cluster_barrier();
        if (slice != 0) return;
    }
    for (int idx = threadIdx.x; idx < D * TOK; idx += blockDim.x) {
        const int r = idx % D, tok = idx / D;
        const int tile = r / 16, rr = r % 16;
        float v = 0.f;
        for (int k = 0; k < ksplit; ++k) v += red[(tile * ksplit + k) * 16 * TOK + rr * TOK + tok];
        for (uint32_t j = 1; j < slices; ++j) v += gathered[(j - 1) * D * TOK + idx];
        v *= scale_s[tok < T ? tok : 0];
        v += bias_s[r];
        // the separate kernels round the projection to bfloat16 before rotating it
        val[tok * D + r] = __bfloat162float(__float2bfloat16_rn(v));
    }
    __syncthreads();
    const int total_heads = n_q + 2 * n_kv;
    const bool is_v = head >= n_q + n_kv;
    const bool is_k = head >= n_q && !is_v;
    for (int idx = threadIdx.x; idx < (D / 2) * TOK; idx += blockDim.x) {
        const int i = idx % (D / 2), tok = idx / (D / 2);
        const int page = tok_page[tok];
        if (page == -2) continue;
        const int pos = tok_pos[tok];
        float a = val[tok * D + i], b = val[tok * D + i + D / 2];
        if (!is_v && cos_t) {
            const float c = cos_s[tok][i], s = sin_s[tok][i];
            const float ra = a * c - b * s, rb = b * c + a * s;
            a = ra;
            b = rb;
        }
        const __nv_bfloat16 ta = __float2bfloat16_rn(a), tb = __float2bfloat16_rn(b);
        if (!is_k && !is_v) {
            __nv_bfloat16* q = qkv + (int64_t)tok * total_heads * D + head * D;
            q[i] = ta;
            q[i + D / 2] = tb;
        } else if (page >= 0) {
            const int kvh = is_k ? head - n_q : head - n_q - n_kv;
            __nv_bfloat16* dst = (is_k ? k_pages : v_pages) +
                                 (((int64_t)page * n_kv + kvh) * page_size + pos % page_size) * D;
            dst[i] = ta;
            dst[i + D / 2] = tb;
        }
    }
}

// How many warps share the K of one row tile: enough that no warp walks more than about
// four chunks while the device is not yet full, never fewer than two chunks per warp.
static int pick_ksplit(int tiles, int chunks, int max_ksplit) {
    int want = (148 * 32) / (tiles > 0 ? tiles : 1);
    if (want > max_ksplit) want = max_ksplit;
    if (want > chunks / 2) want = chunks / 2;
    return want < 1 ? 1 : want;
}

// Blocks of a cluster that share K: a product with few blocks and a long K is cut so that
// more SMs pull its weights. 0 = decide here; tests and tuning runs set it.
static int g_slices_plain = 0, g_slices_qkv = 0;
// Matrices of at least this many elements go to the TMA-fed kernel (0 = never).
static long long g_fed_min_elements = 12ll * 1024 * 1024;
// (the gated product: measured slower than the other kernel at 2 x 8960 x 1536)
static long long g_fed_min_gated = 64ll * 1024 * 1024;

static int pick_slices(int blocks, int chunks, int forced) {
    if (forced > 0) return forced;
    int slices = 1;
    while (slices < 4 && blocks * slices * 2 <= 148 && chunks / (slices * 2) >= 16) slices *= 2;
    return slices;
}

// Dynamic shared memory beyond 48 KB has to be asked for once per kernel (and again only
// when a larger amount is needed).
template <typename KernelT>
static int raise_smem(KernelT kernel, size_t bytes) {
    // per kernel (instantiations of one template share their function type, so the amount
    // already asked for is kept by address). The kernels also hold up to 12 KB of static
    // shared memory, and the 48 KB that need no asking cover both kinds together.
    static std::unordered_map<const void*, size_t> raised;
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    size_t& have = raised[reinterpret_cast<const void*>(kernel)];
    if (have == 0) have = 32 * 1024;
    if (bytes <= have) return MB_OK;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) !=
        cudaSuccess)
        return MB_ERR_UNSUPPORTED_SIZE;
    have = bytes;
    return MB_OK;
}

}  // namespace mb

using namespace mb;

// From how many weight elements on a few-token product takes the TMA-fed kernel (0 = never).
MB_EXPORT int mb_gemm_skinny_set_fed_min(long long elements) {
    g_fed_min_elements = elements;
    return MB_OK;
}

// Force the number of blocks that share K in the plain and in the q/k/v few-token products
// (1, 2 or 4; 0 = let the library decide).
MB_EXPORT int mb_gemm_skinny_set_slices(int plain, int qkv) {
    const bool ok = (plain == 0 || plain == 1 || plain == 2 || plain == 4) &&
                    (qkv == 0 || qkv == 1 || qkv == 2 || qkv == 4);
    if (!ok) return MB_ERR_UNSUPPORTED_SIZE;
    g_slices_plain = plain;
    g_slices_qkv = qkv;
    return MB_OK;
}

// At most 16 tokens: a block takes 8 or 16 of them and uses its weight fragments for each.
// (32 tokens per block, and 33 to 64 tokens as two groups of blocks that both stream the
// matrix, were built and measured at the 0.5B widths: a decode step of 32 sequences took 1.49 ms
// against 1.18 ms with the library product and separate norm and gate kernels, one of 64
// took 2.33 against 1.40. Each warp's MMAs then repeat per token tile while the weights no
// longer bound the time, so beyond 16 tokens the library product is the better tool.)
MB_EXPORT int mb_gemm_skinny_supports(int T, int N, int K) {
    return T >= 1 && T <= 16 && K > 0 && K % 32 == 0 && N > 0 && N % 16 == 0;
}

// Tokens per block in units of eight for a product of T tokens.
static int skinny_nt(int T) { return T <= 8 ? 1 : 2; }

#define MB_SK_NT_SWITCH(NTV, ...)                            \
    if (NTV <= 1) { constexpr int NT = 1; __VA_ARGS__ }        \
    else { constexpr int NT = 2; __VA_ARGS__ }

static SkinnyInput skinny_input(const void* x, const float* h, const void* norm_w, const int* rows,
                                float eps, const float* ss_part, int ss_tiles, float ss_eps,
                                int ss_k) {
    SkinnyInput in;
    in.x = (const __nv_bfloat16*)x;
    in.h = h;
    in.norm_w = (const __nv_bfloat16*)norm_w;
    in.rows = rows;
    in.eps = eps;
    in.ss_part = ss_part;
    in.ss_tiles = ss_tiles;
    in.ss_eps = ss_eps;
    in.ss_k = ss_k;
    return in;
}

#define MB_SK_LAUNCH_GEMM(EPI_)                                                                  \
    do {                                                                                         \
        if (norm_w) {                                                                            \
            rc = raise_smem(skinny_gemm_kernel<NT, EPI_, true>, smem);                           \
            if (rc == MB_OK)                                                                     \
                MB_LAUNCH_CLUSTER((skinny_gemm_kernel<NT, EPI_, true>), dim3(blocks, slices, groups), threads, \
                          smem, s, 1, slices, 1, in,                                            \
                          (const bf*)w, (const bf*)bias, out, T, N, K, half_n, rowt, ksplit,     \
                          (const bf*)next_w, (bf*)next_x, next_ss, h_stable);                    \
        } else {                                                                                 \
            rc = raise_smem(skinny_gemm_kernel<NT, EPI_, false>, smem);                          \
            if (rc == MB_OK)                                                                     \
                MB_LAUNCH_CLUSTER((skinny_gemm_kernel<NT, EPI_, false>), dim3(blocks, slices, groups), threads, \
                          smem, s, 1, slices, 1, in,                                            \
                          (const bf*)w, (const bf*)bias, out, T, N, K, half_n, rowt, ksplit,     \
                          (const bf*)next_w, (bf*)next_x, next_ss, h_stable);                    \
        }                                                                                        \
    } while (0)

// The TMA-fed form of the product, for large matrices. pairs > 0 selects the gated form (w
// holds 2 * pairs * 16 rows, gate rows first). Returns MB_ERR_UNSUPPORTED_SIZE if the shape is
// not for it (the caller then takes the other kernel).
static int launch_fed(const SkinnyInput& in, const void* w, const void* bias, void* out, int mode, int T,
                      int N, int K, int pairs, const void* next_w, void* next_x, float* next_ss,
                      int* error, cudaStream_t s) {
    typedef __nv_bfloat16 bf;
    if (K % 64 || in.norm_w != nullptr || error == nullptr || ((uintptr_t)w & 15)) return MB_ERR_UNSUPPORTED_SIZE;
    const int rows_total = pairs > 0 ? 2 * pairs * 16 : N;
    CUtensorMap map;
    if (!make_map(&map, w, rows_total, K, 16)) return MB_ERR_UNSUPPORTED_SIZE;
    const int tiles = rows_total / 16;
    const int boxes = K / 64;
    // about sixteen warps per SM over the whole device; a warp walks two boxes at least
    // blocks of eight warps (three of them on an SM: one block's start and end overlap the
    // others' streaming)
    // blocks, where the matrix has tiles enough; with few tiles and a long K a tile gets a
    // block of up to sixteen warps of its own)
    int ksplit = (148 * 16) / tiles;
    const int most = pairs > 0 ? 8 : 16;
    if (ksplit > most) ksplit = most;
    if (ksplit > boxes / 2) ksplit = boxes / 2;
    if (ksplit < 1) ksplit = 1;
    int rowt, blocks;
    if (pairs > 0) {
        const int per_block = 4 / ksplit > 0 ? 4 / ksplit : 1;
        rowt = 2 * per_block;
        blocks = (pairs + per_block - 1) / per_block;
    } else {
        rowt = 8 / ksplit > 0 ? 8 / ksplit : 1;
        blocks = (tiles + rowt - 1) / rowt;
    }
    const int warps = rowt * ksplit;
    const int threads = warps * 32;
    const int nt = T > 8 ? 2 : 1;      // sixteen tokens per block where there are more than eight
    const size_t smem = (size_t)warps * (SKINNY_FED_STAGES * 2048 + 16 * 8 * nt * sizeof(float)) + 1024;
    const int groups = (T + 8 * nt - 1) / (8 * nt);
    const int half_n = pairs > 0 ? pairs * 16 : 0;
    int rc;
#define MB_FED_(EPI_, NT_)                                                                        \
    do {                                                                                          \
        rc = raise_smem(skinny_fed_kernel<EPI_, NT_>, smem);                                      \
        if (rc == MB_OK)                                                                          \
            MB_LAUNCH((skinny_fed_kernel<EPI_, NT_>), dim3(blocks, 1, groups), threads, smem, s,  \
                      map, in, (const bf*)bias, out, T, N, K, half_n, rowt, ksplit,               \
                      (const bf*)next_w, (bf*)next_x, next_ss, error);                            \
    } while (0)
#define MB_FED(EPI_)                                                                              \
    do {                                                                                          \
        if (nt == 1) MB_FED_(EPI_, 1);                                                            \
        else MB_FED_(EPI_, 2);                                                                    \
    } while (0)
    if (pairs > 0) MB_FED(2);
    else if (mode == 0) MB_FED(0);
    else if (mode == 1) MB_FED(1);
    else MB_FED(3);
#undef MB_FED_
#undef MB_FED
    return rc != MB_OK ? rc : launch_status();
}

// The activations are either `x` (bfloat16 [T, K]) or, when `norm_w` is given, the float32
// stream `h` [*, K] normalised with `norm_w` and `eps`, rows picked by `rows` if not null.
// mode: 0 = bfloat16 out, 1 = float32 out, 3 = add into the float32 rows of `out`.
// bias may be null. A third form of input: `ss_part` given means x is a stream already
// multiplied by a norm weight and ss_part [T, ss_tiles] holds its sums of squares per
// 16-column tile; the result rows are multiplied by rsqrt(sum / ss_k + ss_eps).
// With mode 3 and `next_w` given the product leaves exactly that for the product after the
// next norm: next_x [T, N] = bfloat16(updated stream * next_w) and next_ss [T, N / 16].
// `h_stable` (mode 3) says that the kernel launched just before this one does not write
// `out`: the stream is then read before the wait for that kernel.
MB_EXPORT int mb_gemm_skinny(const void* x, const float* h, const void* norm_w, const int* rows,
                             float eps, const float* ss_part, int ss_tiles, float ss_eps, int ss_k,
                             const void* w, const void* bias, void* out, int mode, int T, int N,
                             int K, const void* next_w, void* next_x, float* next_ss, int h_stable,
                             int* error, void* stream) {
    if (next_w && (mode != 3 || !next_x || !next_ss)) return MB_ERR_UNSUPPORTED_SIZE;
    if (!mb_gemm_skinny_supports(T, N, K)) return MB_ERR_UNSUPPORTED_SIZE;
    if (mode != 0 && mode != 1 && mode != 3) return MB_ERR_BAD_DTYPE;
    typedef __nv_bfloat16 bf;
    cudaStream_t s = (cudaStream_t)stream;
    const SkinnyInput in = skinny_input(x, h, norm_w, rows, eps, ss_part, ss_tiles, ss_eps, ss_k);
    // large matrices: weights by TMA (`error` as for mb_gemm_tcgen05, code 7; null: never)
    if (g_fed_min_elements > 0 && (long long)N * K >= g_fed_min_elements && T <= 16) {
        const int rc_fed = launch_fed(in, w, bias, out, mode, T, N, K, 0, next_w, next_x, next_ss, error, s);
        if (rc_fed != MB_ERR_UNSUPPORTED_SIZE) return rc_fed;
    }
    const int nt = skinny_nt(T);
    const int tiles = N / 16;
    // (blocks if K were not shared: one per row tile once a tile has 8 warps or more)
    const int slices = norm_w ? 1 : pick_slices(tiles, K / 32, g_slices_plain);
    const int ksplit = pick_ksplit(tiles * slices, (K / 32 + slices - 1) / slices,
                                   (nt == 2 || norm_w) ? 16 : 32);
    const int rowt = ksplit >= 8 ? 1 : 8 / ksplit;
    const int blocks = (tiles + rowt - 1) / rowt;
    const int threads = rowt * ksplit * 32;
    const int half_n = 0;
    int rc = MB_OK;
    // 8 or 16 tokens per block (a block of 16 has fewer threads, see skinny_max_threads:
    // sixteen tokens in a 1024-thread block spilled)
    const int groups = (T + 8 * nt - 1) / (8 * nt);
    MB_SK_NT_SWITCH(nt, {
        const size_t smem = (size_t)rowt * (ksplit + slices - 1) * 16 * 8 * NT * sizeof(float);
        if (mode == 0) MB_SK_LAUNCH_GEMM(0);
        else if (mode == 1) MB_SK_LAUNCH_GEMM(1);
        else MB_SK_LAUNCH_GEMM(3);
    })
    return rc != MB_OK ? rc : launch_status();
}

// w: [2 * width, K] with the gate rows first; out: [T, width] bfloat16. Input as above.
MB_EXPORT int mb_gemm_skinny_swiglu(const void* x, const float* h, const void* norm_w,
                                    const int* rows, float eps, const float* ss_part, int ss_tiles,
                                    float ss_eps, int ss_k, const void* w, void* out, int T,
                                    int width, int K, const void* ahead, long long ahead_bytes,
                                    int* error, void* stream) {
    // ahead, ahead_bytes: the matrix that the product behind this one will stream (or null):
    // L2 is asked for it once this product's own weights are in
    if (!mb_gemm_skinny_supports(T, width, K)) return MB_ERR_UNSUPPORTED_SIZE;
    typedef __nv_bfloat16 bf;
    cudaStream_t s = (cudaStream_t)stream;
    const SkinnyInput in = skinny_input(x, h, norm_w, rows, eps, ss_part, ss_tiles, ss_eps, ss_k);
    if (T <= 16 && g_fed_min_elements > 0 && 2ll * width * K >= (g_fed_min_elements > g_fed_min_gated || g_fed_min_elements < 1024 ? g_fed_min_elements : g_fed_min_gated)) {
        const int rc_fed = launch_fed(in, w, nullptr, out, 0, T, 2 * width, K, width / 16, nullptr, nullptr,
                                      nullptr, error, s);
        if (rc_fed != MB_ERR_UNSUPPORTED_SIZE) return rc_fed;
    }
    const int nt = skinny_nt(T);
    const int pairs = width / 16;
    // (at most 14 warps: the gated kernel is built for three blocks of 448 threads per SM, so
    // that all its blocks are resident beside the blocks of the kernel in front)
    const int ksplit = pick_ksplit(2 * pairs, K / 32, 7);
    const int pairs_per_block = ksplit >= 4 ? 1 : 4 / ksplit;
    const int rowt = 2 * pairs_per_block;
    const int blocks = (pairs + pairs_per_block - 1) / pairs_per_block;
    const int threads = rowt * ksplit * 32;
    const int N = 2 * width, half_n = width;
    const void* bias = nullptr;
    const bool look_ahead = ahead != nullptr && ahead_bytes >= 128 && ahead_bytes / 128 < (1ll << 30);
    const int h_stable = look_ahead ? (int)(ahead_bytes / 128) : 0;   // (EPI 2: lines to ask L2 for)
    const void* next_w = look_ahead ? ahead : nullptr;                // (EPI 2: where they start)
    void* next_x = nullptr;
    float* next_ss = nullptr;
    const int slices = 1;
    int rc = MB_OK;
    const int groups = (T + 8 * nt - 1) / (8 * nt);
    MB_SK_NT_SWITCH(nt, {
        const size_t smem = (size_t)rowt * ksplit * 16 * 8 * NT * sizeof(float);
        MB_SK_LAUNCH_GEMM(2);
    })
    return rc != MB_OK ? rc : launch_status();
}

MB_EXPORT int mb_gemm_skinny_qkv_supports(int T, int K, int d, int rot) {
    return T >= 1 && T <= 16 && K > 0 && K % 32 == 0 && (d == 64 || d == 128) && (rot == d || rot == 0);
}

#define MB_SK_LAUNCH_QKV(DD, NORM_)                                                              \
    do {                                                                                         \
        rc = raise_smem(skinny_qkv_rope_kernel<NT, DD, NORM_>, smem);                            \
        if (rc == MB_OK)                                                                         \
            MB_LAUNCH_CLUSTER((skinny_qkv_rope_kernel<NT, DD, NORM_>), dim3(heads, slices), threads,  \
                      smem, s, 1, slices, 1, in,                                                \
                      (const bf*)w, (const bf*)bias, (bf*)qkv, c, sin_t, positions, seq_of_token, \
                      table, max_pages, (bf*)k_pages, (bf*)v_pages, T, K, n_q, n_kv, page_size,  \
                      store, ksplit);                                                            \
    } while (0)

// The packed q/k/v projection of a few tokens with bias, rotation and cache store fused.
// Input as for mb_gemm_skinny (rows is not used here).
MB_EXPORT int mb_gemm_skinny_qkv_rope(const void* x, const float* h, const void* norm_w, float eps,
                                      const float* ss_part, int ss_tiles, float ss_eps, int ss_k,
                                      const void* w, const void* bias, void* qkv,
                                      const float* cos_t, const float* sin_t, int rot,
                                      const int* positions, const int* seq_of_token,
                                      const int* table, int max_pages, void* k_pages, void* v_pages,
                                      int T, int K, int n_q, int n_kv, int d, int page_size,
                                      int store, void* stream) {
    if (!mb_gemm_skinny_qkv_supports(T, K, d, rot)) return MB_ERR_UNSUPPORTED_SIZE;
    typedef __nv_bfloat16 bf;
    cudaStream_t s = (cudaStream_t)stream;
    const SkinnyInput in = skinny_input(x, h, norm_w, nullptr, eps, ss_part, ss_tiles, ss_eps, ss_k);
    const int nt = (T + 7) / 8;
    const int heads = n_q + 2 * n_kv;
    const int rowt = d / 16;
    const int slices = norm_w ? 1 : pick_slices(heads, K / 32, g_slices_qkv);
    const int ksplit = pick_ksplit(heads * rowt * slices, (K / 32 + slices - 1) / slices,
                                   (norm_w ? 16 : 32) / rowt);
    const int threads = rowt * ksplit * 32;
    const float* c = rot ? cos_t : nullptr;
    int rc = MB_OK;
    MB_SK_NT_SWITCH(nt, {
        const size_t smem = ((size_t)rowt * ksplit * 16 + (size_t)d * slices) * 8 * NT * sizeof(float);
        if (d == 64) {
            if (norm_w) MB_SK_LAUNCH_QKV(64, true); else MB_SK_LAUNCH_QKV(64, false);
        } else {
            if (norm_w) MB_SK_LAUNCH_QKV(128, true); else MB_SK_LAUNCH_QKV(128, false);
        }
    })
    return rc != MB_OK ? rc : launch_status();
}
