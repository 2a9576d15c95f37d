// Paged attention of prompt portions on the fifth-generation tensor cores, head sizes 64
// and 128 (bfloat16): scores and the probability-weighted values are tcgen05.mma products
// with their accumulators in tensor memory; queries, keys and values arrive by TMA, keys and
// values straight from the pages the block table names; the probabilities never leave
// tensor memory.
//
// Same contract as the other attention kernels (ragged batch, causal by absolute position,
// optional window; mercury/model/attention.py:77-101 is the reference's gather-and-SDPA
// version). A CTA takes floor(128 / group) query tokens of one sequence and one KV head: the
// (token, head of the group) pairs are the 128 rows of the MMA, one row per accumulator
// lane. Keys are walked in tiles of 128, one CTA per SM:
//   producers (warp 8 the keys and the queries, warp 10 the values)  TMA of the tile's
//            pages into rings of four (head size 64) or two (128) stages; a head of 128
//            features lies as two sub-tiles of 64, each 128-byte swizzled. A stage's keys are
//            handed back as soon as the scores that read them are done, its values after
//            P V. The block table is read a window of 256 entries at a time, so that no trip
//            to global memory stands between a free stage and its copies.
//   MMA      (warp 9)  S(i+1) = Q K(i+1)^T is issued before P(i) V(i): scores and
//            probabilities are double-buffered in tensor memory (2 x 128 + 2 x 64 columns)
//            beside the output (64 or 128 columns), and the softmax of tile i+1 finds its
//            scores waiting. O += P(i) V(i) reads P FROM tensor memory (the A operand of the
//            MMA) and V from shared memory as it lies in the pages.
//   softmax  (warps 0-7, two threads per row: warps w and w + 4 share the rows of tensor-
//            memory lane quarter w, 64 keys and half of the output columns each)  one trip
//            to tensor memory for the thread's 64 scores, mask, 2^x relative to the maximum
//            in use, the probabilities packed to bfloat16 into the tile's P columns, and the
//            maximum of the thread's keys on the side; the two threads of a row then compare
//            notes on a named barrier of their own. Nothing goes through shared memory but
//            that one number. The maximum that the probabilities and the output are relative
//            to is only raised when a tile exceeds it by more than 2^8: the two warps then
//            rescale their columns of O in tensor memory and do the tile again (its scores
//            are still there). Rows of the MMA that are no rows of the problem (two of 128
//            with seven heads to a group) are cleared once and run the same code as the
//            others: a lane on a path of its own holds its whole warp back in every tile.
// What sets the kernel's time is the softmax of the heaviest row tile (2^x runs at 16 a
// cycle and SM), so the row tiles are launched heaviest first.
// Launched as thread-block clusters of 2 or 4 CTAs, the CTAs of a cluster share one row tile
// and split its key tiles between them; each leaves its (maximum, sum, unnormalised output)
// in its own shared memory and the first CTA of the cluster merges them through distributed
// shared memory. Every mbarrier wait is bounded; a wait that runs out sets the error word
// and the CTA winds down (frees its tensor memory, returns).
#include "tcgen05.cuh"

namespace mb {

constexpr int TB_ROWS = 128;         // MMA M: query rows per CTA
constexpr int TB_KEYS = 128;         // keys per tile
constexpr int TB_THREADS = 352;      // 8 softmax warps, key producer, MMA issuer, value producer
constexpr float TB_RAISE = 8.f;      // log2 of how far a tile may exceed the maximum in use

__device__ __forceinline__ float tb_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// MN-major B operand (values as stored: [key][64 features], features contiguous, 128-byte
// swizzle; 8 keys are 1024 bytes).
__device__ __forceinline__ uint64_t tb_desc_mn(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;               // one 64-element block along N: offset unused
    d |= (uint64_t)(1024 >> 4) << 32;     // next group of 8 keys
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// D[tmem] (+)= A[tmem] . B[smem]: the A operand (128 rows x 16 bfloat16, two to a column,
// row = lane) is read from tensor memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc,
                                                 uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int D>
__global__ void __launch_bounds__(TB_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const int* __restrict__ table,
                     int max_pages, const int* __restrict__ q_start, const int* __restrict__ kv_len_of,
                     __nv_bfloat16* __restrict__ out, int n_q, int n_kv, int page_size, float scale,
                     int window, int tiles_per_seq, int* __restrict__ error) {
    constexpr int SUBS = D / 64;                       // 64-feature sub-tiles of a head
    constexpr int S_BUFS = 2;                          // score (and probability) buffers in tensor memory
    constexpr int TB_STAGES = D == 64 ? 4 : 2;         // key/value tiles in flight
    constexpr int SUB_BYTES = TB_KEYS * 128;           // one sub-tile: 128 rows x 128 bytes
    constexpr int TILE_BYTES = SUBS * SUB_BYTES;       // one K (or V, or Q) tile
    constexpr uint32_t TMEM_COLS = 512u;               // 2 x 128 scores, 2 x 64 probabilities, D output
    grid_dependency_sync();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base =
        reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = base;                              // [SUBS][128 rows][128 B]
    unsigned char* kv_s = q_s + TILE_BYTES;                 // [stage][K tile, V tile]
    __shared__ uint64_t q_full, k_full[TB_STAGES], k_free[TB_STAGES], v_full[TB_STAGES], v_free[TB_STAGES],
        s_ready[2], p_ready[2], o_ready[2];
    __shared__ uint32_t tmem_base_slot;
    // per tile in flight, one bit per copy (a page, or 128 keys of a larger one): was it there?
    // (twice as many entries as stages: a stage's keys are handed back when its scores are
    // done, which is when the softmax threads only begin to look at the entry)
    __shared__ uint32_t copied[2 * TB_STAGES];
    __shared__ float row_xch[3][2][TB_ROWS];         // [first tile, tile parity][half][row]: maxima, sums
    // the pages of this CTA's key tiles, a window of them at a time (producer warp only): a
    // table entry fetched from global memory when a stage comes free would put a trip to L2
    // in front of every tile's copies
    constexpr int PAGE_WINDOW = 256;
    __shared__ int page_win[2][PAGE_WINDOW];         // one window for each of the two producers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = n_q / n_kv;
    const int tok_per_tile = TB_ROWS / group;
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
    if (window > 0 && p_min - window + 1 > 0) t_lo = (p_min - window + 1) / TB_KEYS;
    // the key tiles of this row tile, cut evenly over the CTAs of the cluster
    uint32_t cl_rank, cl_size;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cl_rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(cl_size));
    const int tiles_all = p_max / TB_KEYS + 1 - t_lo;
    const int tiles_per_cta = (tiles_all + (int)cl_size - 1) / (int)cl_size;
    const int t_first = t_lo + (int)cl_rank * tiles_per_cta;
    int n_tiles = t_lo + tiles_all - t_first;
    if (n_tiles > tiles_per_cta) n_tiles = tiles_per_cta;
    if (n_tiles < 0) n_tiles = 0;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < TB_STAGES; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_free[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_ready[i], 1);
            mbar_init(&p_ready[i], 8);       // one arrival per softmax warp
            // P V of tile i commits to o_ready[i & 1]: a wait for tile i finds that barrier
            // either in the phase of tile i or just past it (tile i - 2 is known to be complete
            // when the scores of tile i have arrived, tile i + 2 cannot start before P(i + 2)
            // exists), so the parity of the wait is never ambiguous although most phases are
            // never waited for
            mbar_init(&o_ready[i], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // The query rows beyond group * tok_per_tile (two of 128 with seven heads to a group) are
    // no part of the TMA box: they are cleared once, so that their scores are zeros rather
    // than whatever the memory held, and their threads can run the same code as every other
    // row (a lane on a path of its own would hold its whole warp back in every tile).
    for (int idx = threadIdx.x; idx < (TB_ROWS - group * tok_per_tile) * SUBS * 8; idx += TB_THREADS) {
        const int row = group * tok_per_tile + idx / (SUBS * 8), piece = idx % (SUBS * 8);
        *reinterpret_cast<uint4*>(q_s + (piece / 8) * SUB_BYTES + row * 128 + (piece % 8) * 16) =
            make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&tmem_base_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = tmem_base_slot;                                    // S_BUFS x 128 columns of scores
    const uint32_t tmem_p = tmem_base_slot + S_BUFS * TB_KEYS;                 // S_BUFS x 64 columns of probabilities
    const uint32_t tmem_o = tmem_base_slot + S_BUFS * (TB_KEYS + TB_KEYS / 2); // D columns of output

    // a copy brings `box` keys: a whole page, or 128 keys of a larger one
    const int box = page_size < TB_KEYS ? page_size : TB_KEYS;
    const int box_shift = 31 - __clz(box);
    if (warp == 8 || warp == 10) {
        // ------------------------------------------- producers: warp 8 the keys (and the
        // queries), warp 10 the values. A stage's keys are free again as soon as the scores
        // that read them are done, its values after P V; each warp issues its own copies
        // (a copy costs its issuing thread some 60 cycles, 8 to 32 of them per tile).
        const bool keys = warp == 8;
        uint64_t* full = keys ? k_full : v_full;
        uint64_t* freed = keys ? k_free : v_free;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        int* window = page_win[keys ? 0 : 1];
        if (keys && lane == 0 && n_tiles > 0) {
            mbar_expect_tx(&q_full, (uint32_t)(group * tok_per_tile * D * 2));
#pragma unroll
            for (int s = 0; s < SUBS; ++s)
                tma_load_4d(q_s + s * SUB_BYTES, &map_q, s * 64, 0, kvh, q_begin + tok0, &q_full);
        }
        const int copies = TB_KEYS / box;                 // at most 16 (pages of 8)
        const int win_tiles = PAGE_WINDOW / copies;
        int win_lo = t_first;
        auto fill_window = [&](int first_tile) {
            win_lo = first_tile;
            __syncwarp();
            for (int e = lane; e < PAGE_WINDOW; e += 32) {
                const int key0 = first_tile * TB_KEYS + e * box;
                window[e] = key0 < kv_len ? table_page(table, seq, max_pages, key0 / page_size) : -1;
            }
            __syncwarp();
        };
        if (n_tiles > 0) fill_window(t_first);
        bool ok = true;
        for (int i = 0; i < n_tiles; ++i) {
            const int st = i % TB_STAGES, kt = t_first + i;
            if (kt >= win_lo + win_tiles) fill_window(kt);
            // lanes 0 .. copies-1 each take one page of the tile
            int page = -1, row = 0;
            if (lane < copies) {
                const int key0 = kt * TB_KEYS + lane * box;
                page = window[(kt - win_lo) * copies + lane];
                if (page >= 0) row = (page * n_kv + kvh) * page_size + key0 % page_size;
            }
            const unsigned valid = __ballot_sync(0xffffffffu, page >= 0);
            if (i >= TB_STAGES) {
                ok = mbar_wait(&freed[st], (uint32_t)((i / TB_STAGES - 1) & 1), error, 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            if (lane == 0) {
                if (keys) copied[i % (2 * TB_STAGES)] = valid;   // read by the softmax threads behind s_ready
                mbar_expect_tx(&full[st], (uint32_t)(__popc(valid) * box * D * 2));
            }
            __syncwarp();
            if (page >= 0) {
                unsigned char* dst = kv_s + st * 2 * TILE_BYTES + (keys ? 0 : TILE_BYTES) + lane * box * 128;
#pragma unroll
                for (int s = 0; s < SUBS; ++s) tma_load_2d(dst + s * SUB_BYTES, map, s * 64, row, &full[st]);
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(TB_ROWS, TB_KEYS);
            const uint32_t idesc_o = umma_idesc(TB_ROWS, 64) | (1u << 16);   // B is MN-major
            bool ok = n_tiles > 0 && mbar_wait(&q_full, 0, error, 2);
            // S(i) = Q K(i)^T into score buffer i % S_BUFS
            auto issue_scores = [&](int i) -> bool {
                const int st = i % TB_STAGES;
                if (!mbar_wait(&k_full[st], (uint32_t)((i / TB_STAGES) & 1), error, 2)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int s = 0; s < SUBS; ++s) {
                    const uint64_t qd = umma_desc(q_s + s * SUB_BYTES);
                    const uint64_t kd = umma_desc(kv_s + st * 2 * TILE_BYTES + s * SUB_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tmem_s + (uint32_t)((i % S_BUFS) * TB_KEYS), qd + (uint64_t)(2 * k),
                                  kd + (uint64_t)(2 * k), idesc_s, (s > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&s_ready[i % S_BUFS]);
                umma_commit(&k_free[st]);          // the keys are free once these scores are done
                return true;
            };
            if (ok) ok = issue_scores(0);
            for (int i = 0; i < n_tiles && ok; ++i) {
                // two score buffers: the scores of the next tile go first, into the buffer the
                // softmax of tile i - 1 has finished with (it handed P(i - 1) over before this
                // point); one buffer: they go as soon as the softmax of tile i has read its own
                if (S_BUFS == 2 && i + 1 < n_tiles) ok = issue_scores(i + 1);
                if (!ok) break;
                const int buf = i % S_BUFS;
                ok = mbar_wait(&p_ready[buf], (uint32_t)((i / S_BUFS) & 1), error, 5);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (S_BUFS == 1 && i + 1 < n_tiles) ok = issue_scores(i + 1);
                if (!ok) break;
                const int st = i % TB_STAGES;
                ok = mbar_wait(&v_full[st], (uint32_t)((i / TB_STAGES) & 1), error, 2);
                if (!ok) break;
                const unsigned char* v_tile = kv_s + st * 2 * TILE_BYTES + TILE_BYTES;
                const uint32_t p_at = tmem_p + (uint32_t)(buf * (TB_KEYS / 2));
#pragma unroll
                for (int k = 0; k < TB_KEYS / 16; ++k) {
#pragma unroll
                    for (int s = 0; s < SUBS; ++s)
                        umma_bf16_a_tmem(tmem_o + (uint32_t)(s * 64), p_at + (uint32_t)(8 * k),
                                         tb_desc_mn(v_tile + s * SUB_BYTES) + (uint64_t)(k * (2048 >> 4)),
                                         idesc_o, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&o_ready[i & 1]);       // O holds tiles 0 .. i
                umma_commit(&v_free[st]);
            }
        }
    } else {
        // ------------------------------------------------------- softmax: two threads per row
        // Warps w and w + 4 share the rows of tensor-memory lane quarter w: each takes 64 of a
        // tile's 128 keys and half of the output columns. The two meet once per tile on a
        // named barrier of their own (64 threads), to agree on the row's maximum; the meeting
        // is a plain barrier, so a warp whose bounded wait ran out still goes through every
        // tile's meetings (and does nothing else), or its partner would wait for ever.
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;
        const int tok = tok0 + r / group;
        const int hg = r % group;
        const bool row_ok = r < group * tok_per_tile && tok < q_len;
        const int pos = first_pos + tok;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const int c_half = half * (TB_KEYS / 2);            // first key of a tile that is this thread's
        const float scale2 = scale * 1.4426950408889634f;
        auto meet = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); };
        // m: the maximum that O and l are relative to (log2 units); l: this thread's keys only
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        const uint32_t my_o = tmem_o + lane_addr + (uint32_t)(half * (D / 2));
        for (int i = 0; i < n_tiles; ++i) {
            const int st = i % TB_STAGES, kt = t_first + i, buf = i % S_BUFS;
            if (ok) {
                ok = mbar_wait(&s_ready[buf], (uint32_t)((i / S_BUFS) & 1), error, 3);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (!ok) {
                if (i == 0) meet();
                meet();
                continue;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t my_s = tmem_s + lane_addr + (uint32_t)(buf * TB_KEYS + c_half);
            const uint32_t my_p = tmem_p + lane_addr + (uint32_t)(buf * (TB_KEYS / 2) + c_half / 2);
            const int key0 = kt * TB_KEYS + c_half;
            // does every key of the tile count for this row, and is every key real? (A row
            // that is no row of the problem takes the same path: its numbers are finite and
            // go nowhere.)
            const bool plain = kt * TB_KEYS + TB_KEYS - 1 <= pos && (kt + 1) * TB_KEYS <= kv_len &&
                               (window <= 0 || kt * TB_KEYS > pos - window);
            const uint32_t landed = copied[i % (2 * TB_STAGES)];   // which pages of the tile were there
            // this thread's 64 scores of the row in one trip to tensor memory (two loads in
            // flight); a key that does not count becomes -inf
            auto load_scores = [&](uint32_t (&sa)[32], uint32_t (&sb)[32]) {
                tmem_load_32_async(my_s, sa);
                tmem_load_32_async(my_s + 32u, sb);
                tmem_wait_ld();
                if (!plain) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int ka = key0 + j, kb = ka + 32;
                        bool seen_a = row_ok && ka <= pos && ka < kv_len && ((landed >> ((c_half + j) >> box_shift)) & 1u);
                        bool seen_b = row_ok && kb <= pos && kb < kv_len && ((landed >> ((c_half + 32 + j) >> box_shift)) & 1u);
                        if (window > 0) {
                            seen_a = seen_a && ka > pos - window;
                            seen_b = seen_b && kb > pos - window;
                        }
                        sa[j] = seen_a ? sa[j] : 0xff800000u;
                        sb[j] = seen_b ? sb[j] : 0xff800000u;
                    }
                }
            };
            // The probabilities of this thread's keys relative to `shift`, rounded to bfloat16,
            // two to a column, into the tile's P columns; returns their sum and leaves their
            // maximum (log2 units) in `m_mine`. A row that has seen no key yet (m = -inf)
            // gets zeros: (-inf) * scale2 - 0 = -inf, 2^-inf = 0.
            auto emit = [&](float shift, float& m_mine) -> float {
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t sa[32], sb[32], packed[32];
                load_scores(sa, sb);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float a0 = __uint_as_float(sa[2 * j]), a1 = __uint_as_float(sa[2 * j + 1]);
                    const float b0 = __uint_as_float(sb[2 * j]), b1 = __uint_as_float(sb[2 * j + 1]);
                    mx[j & 3] = fmaxf(mx[j & 3], fmaxf(fmaxf(a0, a1), fmaxf(b0, b1)));
                    const float p0 = tb_exp2(a0 * scale2 - shift), p1 = tb_exp2(a1 * scale2 - shift);
                    const float p2 = tb_exp2(b0 * scale2 - shift), p3 = tb_exp2(b1 * scale2 - shift);
                    sum[j & 3] += (p0 + p1) + (p2 + p3);
                    __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
                    packed[j] = *reinterpret_cast<uint32_t*>(&lo);         // keys 2j, 2j + 1 of this half
                    packed[16 + j] = *reinterpret_cast<uint32_t*>(&hi);    // keys 32 + 2j, 32 + 2j + 1
                }
                tmem_store_32(my_p, packed);
                m_mine = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * scale2;
                return (sum[0] + sum[1]) + (sum[2] + sum[3]);
            };
            if (i == 0) {
                // the first tile: the row's maximum first (a pass over the scores alone)
                uint32_t sa[32], sb[32];
                load_scores(sa, sb);
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    mx = fmaxf(mx, fmaxf(__uint_as_float(sa[j]), __uint_as_float(sb[j])));
                row_xch[2][half][r] = mx * scale2;
                meet();
                m = fmaxf(mx * scale2, row_xch[2][half ^ 1][r]);
            }
            // One pass: the probabilities relative to the maximum in use, and the maximum of
            // this thread's keys beside them; the two threads of a row then compare notes. Only
            // when some row of the warp outgrew its maximum by more than 2^8 is the tile done
            // again (by both warps of the quarter: they see the same rows and the same
            // maxima): every row moves to its exact maximum and the warps rescale their
            // columns of O, once P(i-1) V(i-1) is in. Short of that a stale maximum changes
            // nothing but the scale of intermediate values.
            float m_mine;
            float added = emit(m > -INFINITY ? m : 0.f, m_mine);
            row_xch[i & 1][half][r] = m_mine;
            meet();
            const float m_tile = fmaxf(m_mine, row_xch[i & 1][half ^ 1][r]);
            if (__any_sync(0xffffffffu, m_tile > m + TB_RAISE)) {
                const float m_new = fmaxf(m, m_tile);
                const float factor = m > -INFINITY ? tb_exp2(m - m_new) : 1.f;
                m = m_new;
                l *= factor;
                if (i > 0) {
                    ok = mbar_wait(&o_ready[(i - 1) & 1], (uint32_t)(((i - 1) >> 1) & 1), error, 4);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) continue;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                    for (int c0 = 0; c0 < D / 2; c0 += 32) {
                        uint32_t ov[32];
                        tmem_load_32(my_o + (uint32_t)c0, ov);
#pragma unroll
                        for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * factor);
                        tmem_store_32(my_o + (uint32_t)c0, ov);
                    }
                }
                added = emit(m > -INFINITY ? m : 0.f, m_mine);
            }
            l += added;
            // a value row that was not copied, or lies beyond the sequence, must not reach the
            // MMA as it is (0 * NaN): the threads of the first half each clear one key of the
            // tile, once the tile's copies have landed (a copy brings whole pages, rows beyond
            // the sequence included)
            if (half == 0 && !(((landed >> (r >> box_shift)) & 1u) && kt * TB_KEYS + r < kv_len)) {
                mbar_wait(&v_full[st], (uint32_t)((i / TB_STAGES) & 1), error, 3);
#pragma unroll
                for (int s = 0; s < SUBS; ++s) {
                    unsigned char* v_row = kv_s + st * 2 * TILE_BYTES + TILE_BYTES + s * SUB_BYTES + r * 128;
                    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(v_row + c * 16) = zero;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tmem_wait_st();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&p_ready[buf])) : "memory");
        }
        // the output: all tiles are in once the last P V has been committed
        if (ok && n_tiles > 0) {
            ok = mbar_wait(&o_ready[(n_tiles - 1) & 1], (uint32_t)(((n_tiles - 1) >> 1) & 1), error, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        // the row's sum: both halves
        row_xch[2][half][r] = l;
        meet();
        l += row_xch[2][half ^ 1][r];
        if (cl_size == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16* dst = out + ((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * D + half * (D / 2);
#pragma unroll 1
            for (int c0 = 0; c0 < D / 2; c0 += 32) {
                uint32_t ov[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) ov[c] = 0u;
                if (ok && n_tiles > 0) tmem_load_32(my_o + (uint32_t)c0, ov);    // the whole warp
                if (ok && row_ok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 q;
                        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            h2[e] = __floats2bfloat162_rn(__uint_as_float(ov[c + 2 * e]) * inv,
                                                          __uint_as_float(ov[c + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = q;
                    }
                }
            }
        } else {
            // this CTA's share of the keys, for the merge below: the key/value ring is free
            // (every tile loaded was consumed); four columns of a row lie together and the
            // rows of a column group follow each other, so that a warp writes whole lines
            float4* merge_o = reinterpret_cast<float4*>(kv_s);                          // [D / 4][128 rows]
            float* merge_ml = reinterpret_cast<float*>(merge_o + (D / 4) * TB_ROWS);    // [m, l][128]
#pragma unroll 1
            for (int c0 = 0; c0 < D / 2; c0 += 32) {
                uint32_t ov[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) ov[c] = 0u;
                if (ok && n_tiles > 0) tmem_load_32(my_o + (uint32_t)c0, ov);
#pragma unroll
                for (int c = 0; c < 32; c += 4)
                    merge_o[((half * (D / 2) + c0 + c) / 4) * TB_ROWS + r] =
                        make_float4(__uint_as_float(ov[c]), __uint_as_float(ov[c + 1]),
                                    __uint_as_float(ov[c + 2]), __uint_as_float(ov[c + 3]));
            }
            if (half == 0) {
                merge_ml[r] = ok ? m : -INFINITY;
                merge_ml[TB_ROWS + r] = ok ? l : 0.f;
            }
        }
    }
    if (cl_size > 1) {
        // Every thread of every CTA of the cluster comes here (a CTA without key tiles too).
        __syncthreads();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        if (cl_rank == 0 && warp < 8) {
            const int quarter = warp & 3, half = warp >> 2;
            const int r = quarter * 32 + lane;
            const int tok = tok0 + r / group, hg = r % group;
            const bool row_ok = r < group * tok_per_tile && tok < q_len;
            const int col0 = half * (D / 2);
            const uint32_t local_o = smem_u32(kv_s);
            const uint32_t local_ml = local_o + D * TB_ROWS * 4;
            uint32_t remote_o[4];
            float weight[4], l_of[4];
            float m_all = -INFINITY, l_all = 0.f;
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
                weight[k] = -INFINITY;
                l_of[k] = 0.f;
                remote_o[k] = local_o;
                if (k < cl_size) {
                    uint32_t remote_ml;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_o[k]) : "r"(local_o), "r"(k));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_ml) : "r"(local_ml), "r"(k));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(weight[k]) : "r"(remote_ml + 4 * r) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(l_of[k]) : "r"(remote_ml + 4 * (TB_ROWS + r)) : "memory");
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) m_all = fmaxf(m_all, weight[k]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                weight[k] = weight[k] > -INFINITY ? tb_exp2(weight[k] - m_all) : 0.f;
                l_all += l_of[k] * weight[k];
            }
            if (row_ok) {
                const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
                __nv_bfloat16* dst = out + ((int64_t)(q_begin + tok) * n_q + kvh * group + hg) * D;
#pragma unroll 1
                for (int c = col0; c < col0 + D / 2; c += 8) {
                    // all loads of these eight columns first, then the sums
                    float4 part[4][2];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
#pragma unroll
                        for (int g4 = 0; g4 < 2; ++g4) {
                            part[k][g4] = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (weight[k] != 0.f) {    // a CTA without keys for this row is skipped
                                const uint32_t at = remote_o[k] + 16u * (uint32_t)((c / 4 + g4) * TB_ROWS + r);
                                asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(part[k][g4].x), "=f"(part[k][g4].y),
                                               "=f"(part[k][g4].z), "=f"(part[k][g4].w)
                                             : "r"(at)
                                             : "memory");
                            }
                        }
                    }
                    float acc[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
#pragma unroll
                        for (int g4 = 0; g4 < 2; ++g4) {
                            acc[4 * g4 + 0] += part[k][g4].x * weight[k];
                            acc[4 * g4 + 1] += part[k][g4].y * weight[k];
                            acc[4 * g4 + 2] += part[k][g4].z * weight[k];
                            acc[4 * g4 + 3] += part[k][g4].w * weight[k];
                        }
                    }
                    uint4 q;
                    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        h2[e] = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
                    *reinterpret_cast<uint4*>(dst + c) = q;
                }
            }
        }
        // nobody leaves (and gives its shared memory up) before the merge has read it
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_slot),
                     "r"(TMEM_COLS)
                     : "memory");
    }
}

}  // namespace mb

using namespace mb;

// Whether the tensor-memory attention takes this problem: bfloat16, head size 64 or 128,
// pages of 8 to 128 tokens, groups of at most 128 query heads per KV head, row strides that
// TMA accepts.
MB_EXPORT int mb_attention_tcgen05_supports(int d, int page_size, int n_q, int n_kv, int q_row_stride) {
    if ((d != 64 && d != 128) || n_kv <= 0 || n_q % n_kv) return 0;
    const int group = n_q / n_kv;
    if (group > TB_ROWS) return 0;
    if (page_size < 8 || page_size > 128 || (page_size & (page_size - 1))) return 0;
    return q_row_stride % 8 == 0;
}

template <int D>
static int launch_attention_tcgen05(const void* qkv, int q_row_stride, const void* k_pages, const void* v_pages,
                      int num_pages, const int* table, int max_pages, const int* q_start,
                      const int* kv_len, void* out, int tokens, int num_seqs, int max_q_len, int n_q,
                      int n_kv, int page_size, float scale, int window, int cluster, int* error,
                      cudaStream_t stream) {
    const int group = n_q / n_kv;
    const int tok_per_tile = TB_ROWS / group;
    CUtensorMap map_q, map_k, map_v;
    {
        // queries: [D, group, n_kv, tokens], copied 64 features at a time
        cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)group, (cuuint64_t)n_kv, (cuuint64_t)tokens};
        cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)group * D * 2, (cuuint64_t)q_row_stride * 2};
        cuuint32_t box[4] = {64u, (cuuint32_t)group, 1u, (cuuint32_t)tok_per_tile};
        if (!make_map_nd(&map_q, qkv, 4, dims, strides, box)) return MB_ERR_LAUNCH;
    }
    {
        const cuuint64_t rows = (cuuint64_t)num_pages * n_kv * page_size;
        cuuint64_t dims[2] = {(cuuint64_t)D, rows};
        cuuint64_t strides[1] = {(cuuint64_t)D * 2};
        cuuint32_t box[2] = {64u, (cuuint32_t)(page_size < TB_KEYS ? page_size : TB_KEYS)};
        if (!make_map_nd(&map_k, k_pages, 2, dims, strides, box) ||
            !make_map_nd(&map_v, v_pages, 2, dims, strides, box))
            return MB_ERR_LAUNCH;
    }
    // queries, four (head size 64) or two (128) stages of keys and values, and room to round
    // the start up to 1024 bytes
    constexpr int stages = D == 64 ? 4 : 2;
    const size_t smem = (size_t)(1 + 2 * stages) * (D / 64) * TB_KEYS * 128 + 1024;
    static bool raised = false;
    if (!raised) {
        if (cudaFuncSetAttribute(attention_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return MB_ERR_UNSUPPORTED_SIZE;
        raised = true;
    }
    const int tiles_per_seq = (max_q_len + tok_per_tile - 1) / tok_per_tile;
    // the CTAs of a cluster lie along z and share (row tile, KV head)
    dim3 grid(num_seqs * tiles_per_seq, n_kv, cluster);
    cudaLaunchConfig_t config = launch_config(grid, TB_THREADS, smem, stream);
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
    cudaLaunchKernelEx(&config, attention_tcgen05_kernel<D>, map_q, map_k, map_v, table, max_pages, q_start,
                       kv_len, (__nv_bfloat16*)out, n_q, n_kv, page_size, scale, window, tiles_per_seq,
                       error);
    return launch_status();
}

// qkv: [tokens, q_row_stride] bfloat16 with the rotated queries first; k_pages / v_pages:
// [num_pages, n_kv, page_size, d]; out: [tokens, n_q * d]. `error` as for mb_gemm_tcgen05
// (codes 1 producer, 2 and 5 MMA issuer, 3 and 4 softmax). `cluster` (1, 2 or 4) is the
// number of CTAs that share a row tile and split its keys.
MB_EXPORT int mb_paged_attention_tcgen05(const void* qkv, int q_row_stride, const void* k_pages,
                                     const void* v_pages, int num_pages, const int* table,
                                     int max_pages, const int* q_start, const int* kv_len, void* out,
                                     int tokens, int num_seqs, int max_q_len, int n_q, int n_kv, int d,
                                     int page_size, float scale, int window, int cluster, int* error,
                                     void* stream) {
    if (tokens <= 0 || num_seqs <= 0 || max_q_len <= 0) return MB_OK;
    if (!mb_attention_tcgen05_supports(d, page_size, n_q, n_kv, q_row_stride)) return MB_ERR_UNSUPPORTED_SIZE;
    if (((uintptr_t)qkv | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) & 15) return MB_ERR_ALIGNMENT;
    if (n_kv > 65535 || (cluster != 1 && cluster != 2 && cluster != 4)) return MB_ERR_UNSUPPORTED_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 64)
        return launch_attention_tcgen05<64>(qkv, q_row_stride, k_pages, v_pages, num_pages, table, max_pages, q_start,
                              kv_len, out, tokens, num_seqs, max_q_len, n_q, n_kv, page_size, scale,
                              window, cluster, error, s);
    return launch_attention_tcgen05<128>(qkv, q_row_stride, k_pages, v_pages, num_pages, table, max_pages, q_start,
                           kv_len, out, tokens, num_seqs, max_q_len, n_q, n_kv, page_size, scale, window,
                           cluster, error, s);
}
