// Shared helpers of the sm_100a kernels: storage types, error codes, reductions.
//
// Every entry point is `extern "C"`, takes raw device pointers, sizes and the stream to
// launch on, and returns 0 or one of the MB_ERR_* codes below when it refuses a size
// (the Python wrapper turns the code into an exception that names the limit).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MB_OK 0
#define MB_ERR_UNSUPPORTED_SIZE 1   // a size outside what the kernel was written for
#define MB_ERR_BAD_DTYPE 2          // a dtype flag the entry point does not know
#define MB_ERR_LAUNCH 3             // the launch itself failed (cudaGetLastError)
#define MB_ERR_ALIGNMENT 4          // a pointer or stride breaks an alignment rule
#define MB_ERR_SCRATCH 5            // the scratch buffer given is too small

// dtype flags of the C interface
#define MB_F32 0
#define MB_BF16 1

#define MB_EXPORT extern "C" __attribute__((visibility("default")))

namespace mb {

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Load element i of an array whose dtype is only known at run time.
__device__ __forceinline__ float load_as_float(const void* p, int64_t i, int dtype) {
    return dtype == MB_F32 ? reinterpret_cast<const float*>(p)[i]
                           : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds
// 33 floats of shared memory. The order of the additions is fixed by the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ---- the checked build ---------------------------------------------------------------
// Compiled with -DMB_BOUNDS_CHECK (kernels/build.py: build(bounds_check=True); selected at
// run time by MERCURY_B200_BOUNDS_CHECK=1) every index that a kernel takes from the step's
// device buffers is compared with its limit before it is used: block-table columns, page
// numbers, positions (rows of the rotation tables), token ids. A bad index is recorded in a
// status word (the first one wins; a counter keeps the total), the access is skipped as if
// the page had been given back, and the kernel goes on: no trap, the context stays usable.
// The host sets the limits with mb_check_set_limits and reads the word with mb_check_read.
// In the ordinary build all of this compiles to the plain loads.
#ifdef MB_BOUNDS_CHECK
extern __device__ int mb_check_limit[4];   // [0] pages of the pool, [1] rows of the rotation tables
extern __device__ int mb_check_word[4];    // [0] kind of the first bad index, [1] its value, [2] the limit, [3] how many
__device__ __forceinline__ void check_report(int kind, int value, int limit) {
    if (atomicCAS(&mb_check_word[0], 0, kind) == 0) {
        mb_check_word[1] = value;
        mb_check_word[2] = limit;
    }
    atomicAdd(&mb_check_word[3], 1);
}
#endif
#define MB_CHECK_PAGE 1       // a page number beyond the pool
#define MB_CHECK_COLUMN 2     // a block-table column beyond the table's width
#define MB_CHECK_POSITION 3   // a position beyond the rotation tables
#define MB_CHECK_TOKEN 4      // a token id outside the vocabulary
#define MB_CHECK_SEQUENCE 5   // a sequence number beyond the batch

// The page of block-table column `column` of sequence `seq` (-1: given back, or refused).
__device__ __forceinline__ int table_page(const int* __restrict__ table, int seq, int max_pages,
                                          int column) {
#ifdef MB_BOUNDS_CHECK
    if (column < 0 || column >= max_pages) {
        check_report(MB_CHECK_COLUMN, column, max_pages);
        return -1;
    }
    const int page = table[(int64_t)seq * max_pages + column];
    if (page >= mb_check_limit[0] && mb_check_limit[0] > 0) {
        check_report(MB_CHECK_PAGE, page, mb_check_limit[0]);
        return -1;
    }
    return page;
#else
    return table[(int64_t)seq * max_pages + column];
#endif
}

// A position that indexes the rotation tables (0 when refused).
__device__ __forceinline__ int checked_position(int pos) {
#ifdef MB_BOUNDS_CHECK
    if (pos < 0 || (mb_check_limit[1] > 0 && pos >= mb_check_limit[1])) {
        check_report(MB_CHECK_POSITION, pos, mb_check_limit[1]);
        return 0;
    }
#endif
    return pos;
}

// defined in attention_simt.cu
int launch_attention_combine(const float* part_acc, const float* part_ml, const int* seq_of_token,
                             void* out, int tokens, int n_q, int d, int num_splits, int dtype,
                             cudaStream_t s);

// ---- programmatic dependent launch -----------------------------------------------------
// Every kernel of this library starts with grid_dependency_sync(): when the launch carries
// the programmatic-serialization attribute, the kernel may be scheduled while its
// predecessor in the stream is still draining, and this call is where it waits for the
// predecessor's memory to be complete; without the attribute it does nothing. Right after
// it the kernel lets its own successor be scheduled. This hides most of the launch latency
// between the many small kernels of a decode step.
// What a kernel does before this call must not depend on the kernel in front (weights,
// block tables, positions are fine) and must not take a resource that the kernel in front
// may still be waiting for: above all, tensor memory is allocated only after it, or blocks
// of the kernel in front that are not yet placed could wait for tensor memory for ever.
__device__ __forceinline__ void grid_dependency_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// set by mb_set_dependent_launch (elementwise.cu)
extern int g_dependent_launch;

inline cudaLaunchConfig_t launch_config(dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    static cudaLaunchAttribute attribute = [] {
        cudaLaunchAttribute a = {};
        a.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        a.val.programmaticStreamSerializationAllowed = 1;
        return a;
    }();
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    config.attrs = &attribute;
    config.numAttrs = g_dependent_launch ? 1 : 0;
    return config;
}

// MB_LAUNCH((kernel<T>), grid, block, smem, stream, args...)
#define MB_LAUNCH(kernel, grid, block, smem, stream, ...)                              \
    do {                                                                               \
        cudaLaunchConfig_t config_ = mb::launch_config(grid, block, smem, stream);     \
        cudaLaunchKernelEx(&config_, kernel, __VA_ARGS__);                             \
    } while (0)

// The same with the blocks grouped into thread-block clusters of (cx, cy, cz).
#define MB_LAUNCH_CLUSTER(kernel, grid, block, smem, stream, cx, cy, cz, ...)                     \
    do {                                                                                          \
        cudaLaunchConfig_t config_ = mb::launch_config(grid, block, smem, stream);                \
        cudaLaunchAttribute attrs_[2];                                                            \
        int count_ = 0;                                                                           \
        if (config_.numAttrs) attrs_[count_++] = config_.attrs[0];                                \
        if ((cx) * (cy) * (cz) > 1) {                                                             \
            attrs_[count_].id = cudaLaunchAttributeClusterDimension;                              \
            attrs_[count_].val.clusterDim.x = (unsigned)(cx);                                     \
            attrs_[count_].val.clusterDim.y = (unsigned)(cy);                                     \
            attrs_[count_].val.clusterDim.z = (unsigned)(cz);                                     \
            ++count_;                                                                             \
        }                                                                                         \
        config_.attrs = attrs_;                                                                   \
        config_.numAttrs = count_;                                                                \
        cudaLaunchKernelEx(&config_, kernel, __VA_ARGS__);                                        \
    } while (0)

inline int launch_status() {
    return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

}  // namespace mb
