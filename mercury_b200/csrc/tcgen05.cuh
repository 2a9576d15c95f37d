// Device helpers for TMA, mbarriers, tcgen05.mma and tensor memory, and the host-side cache
// of encoded tensor maps, shared by the product and the attention kernels of sm_100a.
#pragma once

#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace mb {

constexpr int TC_BM = 128, TC_BK = 64;
constexpr long long TC_WAIT_CYCLES = 2000000000ll;             // about a second of SM clocks

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

// Bounded wait for the phase with the given parity; false (and the error word set) if it
// never came. try_wait itself suspends the thread for a while when the phase is not there
// yet (a suspend-time hint changed nothing measurable); the clock is read only now and then.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error, int code,
                                          long long limit = TC_WAIT_CYCLES) {
    const uint32_t addr = smem_u32(bar);
    long long start = 0;
    for (int round = 0;; ++round) {
#pragma unroll 1
        for (int poll = 0; poll < 32; ++poll) {
            uint32_t done;
            asm volatile(
                "{\n"
                ".reg .pred p;\n"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                "selp.u32 %0, 1, 0, p;\n"
                "}\n"
                : "=r"(done)
                : "r"(addr), "r"(parity)
                : "memory");
            if (done) return true;
        }
        if (round == 0) start = clock64();
        else if (clock64() - start > limit) break;
    }
    atomicExch(error, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2,
                                            int c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Shared-memory operand descriptor: K-major tile of rows x 64 bfloat16 as TMA leaves it with
// 128-byte swizzle (rows 128 bytes apart, groups of 8 rows 1024 bytes apart).
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);  // start address, 16-byte units
    d |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset: next 8-row group
    d |= (uint64_t)1 << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                            // 128-byte swizzle
    return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M x N tile.
__device__ __forceinline__ uint32_t umma_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same load without the wait, for several loads in flight; the registers may be read
// only after tmem_wait_ld().
__device__ __forceinline__ void tmem_load_32_async(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 32 columns from registers to tensor memory (complete after tmem_wait_st()).
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, "
        "%21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
          "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
          "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
          "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}


// ------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) !=
                cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// A [rows, K] bfloat16 row-major matrix as tiles of box_rows x 64 with 128-byte swizzle.
// Encoding a map costs microseconds on the host and the same few matrices come back every
// step, so encoded maps are kept (a map depends only on address, sizes and box).
struct MapKey {
    const void* base;
    int rows, K, box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && K == o.K && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        h ^= std::hash<long long>()(((long long)k.rows << 32) ^ ((long long)k.K << 8) ^ k.box_rows) +
             0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
        return h;
    }
};

static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex guard;
    const MapKey key{base, rows, K, box_rows};
    {
        std::lock_guard<std::mutex> lock(guard);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *map = it->second;
            return true;
        }
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(guard);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *map;
    return true;
}


// A general tiled map: `rank` dimensions of bfloat16, innermost first; `strides` in bytes for
// dimensions 1 .. rank-1; 128-byte swizzle (the innermost box extent must be 64 elements).
struct MapKeyN {
    const void* base;
    unsigned long long v[12];
    bool operator==(const MapKeyN& o) const {
        if (base != o.base) return false;
        for (int i = 0; i < 12; ++i)
            if (v[i] != o.v[i]) return false;
        return true;
    }
};
struct MapKeyNHash {
    size_t operator()(const MapKeyN& k) const {
        size_t h = std::hash<const void*>()(k.base);
        for (int i = 0; i < 12; ++i) h = h * 1099511628211ull ^ std::hash<unsigned long long>()(k.v[i]);
        return h;
    }
};

static bool make_map_nd(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims,
                        const cuuint64_t* strides, const cuuint32_t* box) {
    static std::unordered_map<MapKeyN, CUtensorMap, MapKeyNHash> cache;
    static std::mutex guard;
    MapKeyN key;
    key.base = base;
    for (int i = 0; i < 12; ++i) key.v[i] = 0;
    for (int i = 0; i < rank; ++i) {
        key.v[i] = dims[i];
        key.v[4 + i] = box[i];
        if (i + 1 < rank) key.v[8 + i] = strides[i];
    }
    key.v[11] = (unsigned long long)rank;
    {
        std::lock_guard<std::mutex> lock(guard);
        auto it = cache.find(key);
        if (it != cache.end()) {
            *map = it->second;
            return true;
        }
    }
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    cuuint32_t elem[4] = {1, 1, 1, 1};
    if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides,
           box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    std::lock_guard<std::mutex> lock(guard);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *map;
    return true;
}

}  // namespace mb
