// Causal grouped-query attention of prompt portions over the paged bfloat16 cache on the
// 5th-generation tensor cores (tcgen05), sm_100a, for head sizes 64 and 128.
//
// One CTA owns 128 query rows -- (token, query head of one KV head) pairs of one segment, as
// in the mma.sync kernel -- and walks the keys of its request in 64-key tiles (one page of one
// KV head each), lowest first:
//
//   S  = Q K^T     tcgen05.mma, A = Q [128 x hd] and B = K [64 x hd] from shared memory (K-major,
//                  128-byte swizzle), D = S [128 x 64] fp32 in tensor memory
//   softmax        four warps, one query row per thread (tcgen05.ld gives a thread its row, so
//                  the row maximum and sum need no shuffles): scale, causal/window mask,
//                  P = 2^(S - m) rounded to bfloat16 and stored back (tcgen05.st) into the columns
//                  of tensor memory the scores came from
//   O += P V       tcgen05.mma, A = P [128 x 64] read from tensor memory, B = V [64 keys x hd] exactly
//                  as TMA left it (the head dimension contiguous: an MN-major operand), D = O
//                  [128 x hd] fp32, which accumulates in tensor memory over all key tiles
//
// m is the maximum the exponents are taken against.  It is moved to the row's true running
// maximum only when that has grown by more than 2^8 since m was set; then the row's O in tensor
// memory and its sum are scaled by 2^(m_old - m_new).  Until then P is at most 2^8, which
// bfloat16 holds with the same relative precision, and O / sum comes out the same.  So the
// softmax warps' loop is: load S, maximum, exponentials, store P -- no pass over O per tile.
//
// The scores of tile j+1 are computed (into a second S buffer) while the softmax of tile j runs,
// and P lives in its own tile's buffer, so neither the tensor core nor the softmax warps wait for
// the other; P never passes through shared memory (no proxy fence, no shared-memory traffic).
//
// A CTA takes two work items (row tile, KV head): the heaviest and the lightest that are left,
// which evens out what the causal mask makes uneven.
//
// Roles: warp 0 = TMA producer (K and V boxes of a page into a ring of stages), warp 1 = tensor
// memory allocator and MMA issuer, warps 2..5 = softmax and output.  Several CTAs share an SM,
// so one CTA's exponentials overlap another's matrix products.
//
// Pages past a request's last key may hold anything.  Keys beyond a row's position are masked
// by selection (never by arithmetic), and the rows of the last V tile beyond the tile's last
// visible key are cleared in shared memory, so that 0 * garbage cannot reach the output.
//
// Every wait on an mbarrier is bounded: after the limit the CTA raises the library's status
// word, every role stops waiting, the CTA frees its tensor memory and returns.
#include "tcgen05.cuh"

using namespace fwb;
using namespace fwb::tc5;

namespace {

constexpr int ROWS = 128;        // query rows per CTA (UMMA M)
constexpr int KEYS = 64;         // keys per tile == page size
constexpr int SOFTMAX_WARPS = 4;   // one per quarter of the TMEM lanes, one query row per thread
constexpr int THREADS = 64 + 32 * SOFTMAX_WARPS;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int LEAD = 2;                 // the scores run this many key tiles ahead of PV
constexpr float RESCALE_STEP = 8.0f;   // O is rescaled when a row's maximum has grown by more than 2^8

template <int HD>
struct Layout {
    static constexpr int BOXES = HD / 64;                    // 64-element (128-byte) column blocks
    static constexpr int Q_BOX = ROWS * 128;
    static constexpr int Q_BYTES = BOXES * Q_BOX;
    static constexpr int KV_BOX = KEYS * 128;
    static constexpr int KV_BYTES = BOXES * KV_BOX;          // one K or one V tile
    static constexpr int STAGES = 4;                         // ring slots, each one K tile and one V tile
    static constexpr int DATA = Q_BYTES + 2 * STAGES * KV_BYTES;
    static constexpr int SMEM = DATA + 1024 + 256;           // alignment slack + barriers
    static constexpr int S_COLS = 2 * KEYS;                  // two S buffers at column 0, PV behind them
    static constexpr int TMEM_COLS = 256;
};

struct AttnParams {
    const __nv_bfloat16* q;      // [T][nh*hd]
    __nv_bfloat16* out;          // [T][nh*hd]
    const int* positions;        // [T]
    const int* seg_start;        // [S+1]
    const int* tile_seg;         // [n_tiles]
    const int* tile_tok0;        // [n_tiles]
    const int* block_table;      // [S][max_pages]
    int max_pages, nh, nkv, group, tokens_per_tile, window, n_row_tiles;
    int items_per_cta;           // 2: CTA c takes items c and n-1-c; 1: one item each (few items)
    float scale_log2;            // softmax scale * log2(e)
    int* status;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Makes this thread's ordinary shared-memory writes visible to the tensor core and TMA.
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 2^x on the special-function unit (relative error 2^-22; results below 2^-126 are 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One work item: a row tile (up to 128 / group tokens of one segment) and a KV head.
struct Item {
    int tok0, kvh, rows, pos_first, pos_last, tile_begin, n_tiles;
    const int* table;
};

__device__ __forceinline__ Item load_item(const AttnParams& prm, int w) {
    Item it;
    const int tile_index = prm.n_row_tiles - 1 - w / prm.nkv;
    it.kvh = w % prm.nkv;
    const int seg = prm.tile_seg[tile_index];
    it.tok0 = prm.tile_tok0[tile_index];
    int n_tok = prm.seg_start[seg + 1] - it.tok0;
    if (n_tok > prm.tokens_per_tile) n_tok = prm.tokens_per_tile;
    it.rows = n_tok * prm.group;
    it.pos_first = prm.positions[it.tok0];
    it.pos_last = prm.positions[it.tok0 + n_tok - 1];
    const int lo_block = prm.window > 0 ? (it.pos_first - prm.window + 1 > 0 ? it.pos_first - prm.window + 1 : 0) : 0;
    it.tile_begin = lo_block / KEYS;
    it.n_tiles = it.pos_last / KEYS + 1 - it.tile_begin;
    it.table = prm.block_table + (size_t)seg * prm.max_pages;
    return it;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// A x B with A (P, bfloat16 pairs in 32-bit columns) read from tensor memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int HD>
__global__ void __launch_bounds__(THREADS, HD == 64 ? 2 : 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k,
                                 const __grid_constant__ CUtensorMap map_v, const AttnParams prm) {
    using L = Layout<HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_s = base;
    uint8_t* k_s = q_s + L::Q_BYTES;
    uint8_t* v_s = k_s + L::STAGES * L::KV_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(base + L::DATA);
    uint64_t* empty = full + L::STAGES;
    uint64_t* q_ready = empty + L::STAGES;
    uint64_t* s_ready = q_ready + 1;                       // [2]: one per S buffer
    uint64_t* p_ready = s_ready + 2;                       // [2]: P of a tile is in its S buffer
    uint64_t* pv_ready = p_ready + 2;                      // [2]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pv_ready + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < L::STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(q_ready, SOFTMAX_WARPS);
        for (int b = 0; b < 2; ++b) {
            mbar_init(&s_ready[b], 1);
            mbar_init(&p_ready[b], SOFTMAX_WARPS);
            mbar_init(&pv_ready[b], 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, L::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    // q, the cache pages and the batch arrays all come from earlier in the stream
    pdl_wait();

    // Work items are (row tile, KV head) pairs, counted from the heaviest: under a causal mask the
    // last row tiles of a prompt walk the most keys.  CTA c takes item c and item n-1-c, the
    // heaviest left and the lightest left, so every CTA walks about the same number of key tiles.
    const int n_items = prm.n_row_tiles * prm.nkv;
    // (With fewer items than a wave of such pairs would hold, every CTA takes one item: half
    // the walk per CTA and twice the CTAs.)
    const int second_item = prm.items_per_cta == 2 ? n_items - 1 - (int)blockIdx.x : -1;
    const int n_local = second_item > (int)blockIdx.x ? 2 : 1;
    // Barrier phases and ring slots follow a count g of key tiles that runs on over both items.
    // The barriers between the softmax warps and the MMA issuer come in pairs used by alternate
    // tiles (g & 1), each completing once per two tiles: a waiter can then never be a whole
    // phase pair behind, whoever runs ahead.

    if (warp == 0) {
        if (lane == 0) {
            // Step t of an item brings K tile t and V tile t - LEAD into one ring slot under one
            // barrier: they are what the MMA issuer needs next at the same moment (scores run
            // LEAD tiles ahead of PV), and the slot is free again after that one visit.
            int u = 0;                                     // steps so far, over both items
            bool ok = true;
            for (int it = 0; it < n_local && ok; ++it) {
                const Item item = load_item(prm, it == 0 ? (int)blockIdx.x : second_item);
                for (int t = 0; t < item.n_tiles + LEAD; ++t, ++u) {
                    const int s = u % L::STAGES;
                    if (u >= L::STAGES) ok = mbar_wait(&empty[s], ((u / L::STAGES) - 1) & 1, abort_flag, 11, prm.status);
                    if (!ok) break;
                    const bool has_k = t < item.n_tiles, has_v = t >= LEAD;
                    mbar_expect_tx(&full[s], ((has_k ? 1 : 0) + (has_v ? 1 : 0)) * L::KV_BYTES);
                    if (has_k) {
                        const int row = (item.table[item.tile_begin + t] * prm.nkv + item.kvh) * KEYS;
#pragma unroll
                        for (int b = 0; b < L::BOXES; ++b)
                            tma_load_2d(k_s + (size_t)s * L::KV_BYTES + b * L::KV_BOX, &map_k, &full[s], b * 64, row);
                    }
                    if (has_v) {
                        const int row = (item.table[item.tile_begin + t - LEAD] * prm.nkv + item.kvh) * KEYS;
#pragma unroll
                        for (int b = 0; b < L::BOXES; ++b)
                            tma_load_2d(v_s + (size_t)s * L::KV_BYTES + b * L::KV_BOX, &map_v, &full[s], b * 64, row);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc_mn(ROWS, KEYS);
            constexpr uint32_t idesc_pv = make_idesc_mn(ROWS, HD) | IDESC_B_MN_MAJOR;
            const uint32_t tmem_pv = tmem_base + L::S_COLS;
            const uint32_t q_addr = smem_u32(q_s);
            bool ok = true;
            // S of tile g goes to buffer g & 1, so that the softmax of one tile runs while the
            // tensor core already computes the scores of the next.  One thread issues everything,
            // so a commit also covers every product issued before it: when S of tile g is ready,
            // PV of tile g-2 has read its P, which lay in the buffer S and P of tile g use.
            auto wait_step = [&](int u) {
                const int s = u % L::STAGES;
                ok = ok && mbar_wait(&full[s], (u / L::STAGES) & 1, abort_flag, 13, prm.status);
                tc_fence_after();
                return s;
            };
            auto issue_qk = [&](int g, int s) {
                const uint32_t k_addr = smem_u32(k_s + (size_t)s * L::KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < HD / UMMA_K; ++kk) {
                    const uint64_t a = make_smem_desc(q_addr + (kk >> 2) * L::Q_BOX) + 2 * (kk & 3);
                    const uint64_t b = make_smem_desc(k_addr + (kk >> 2) * L::KV_BOX) + 2 * (kk & 3);
                    umma_bf16(tmem_base + (g & 1) * KEYS, a, b, idesc_qk, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_ready[g & 1]);
            };
            int g0 = 0, u = 0;
            for (int it = 0; it < n_local && ok; ++it) {
                const Item item = load_item(prm, it == 0 ? (int)blockIdx.x : second_item);
                ok = mbar_wait(q_ready, it & 1, abort_flag, 12, prm.status);
                for (int t = 0; t < LEAD && ok; ++t, ++u) {           // the steps that bring no V yet
                    const int s = wait_step(u);
                    if (!ok) break;
                    if (t < item.n_tiles) issue_qk(g0 + t, s);
                    umma_commit(&empty[s]);
                }
                for (int j = 0; j < item.n_tiles && ok; ++j, ++u) {
                    const int g = g0 + j;
                    // the softmax of tile j has also taken S of tile j out of its buffer
                    ok = mbar_wait(&p_ready[g & 1], (g >> 1) & 1, abort_flag, 15, prm.status);
                    const int s = wait_step(u);
                    if (!ok) break;
                    const uint32_t v_addr = smem_u32(v_s + (size_t)s * L::KV_BYTES);
#pragma unroll
                    for (int kk = 0; kk < KEYS / UMMA_K; ++kk) {
                        // 16 keys further: two 8-row groups of 1024 bytes
                        const uint64_t b = make_smem_desc_mn_major(v_addr + kk * 2048, L::KV_BOX);
                        const uint32_t acc = (j > 0 || kk > 0) ? 1u : 0u;               // O accumulates over the item's tiles
                        // P of tile g lies in the first 32 columns of its S buffer: 16 keys = 8 columns
                        umma_bf16_a_tmem(tmem_pv, tmem_base + (g & 1) * KEYS + kk * 8, b, idesc_pv, acc);
                    }
                    umma_commit(&pv_ready[g & 1]);
                    if (j + LEAD < item.n_tiles) issue_qk(g + LEAD, s);
                    umma_commit(&empty[s]);
                }
                g0 += item.n_tiles;
            }
        }
    } else {
        const int quarter = warp & 3;                      // the TMEM lanes this warp may read
        const int row = quarter * 32 + lane;
        const int swz = row & 7;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t o_addr = lane_addr + L::S_COLS;
        bool ok = true;
        int g0 = 0, u0 = 0;
        for (int it = 0; it < n_local && ok; ++it) {
            const Item item = load_item(prm, it == 0 ? (int)blockIdx.x : second_item);
            const bool valid = row < item.rows;
            const int tok = item.tok0 + (valid ? row / prm.group : 0);
            const int head = item.kvh * prm.group + (valid ? row % prm.group : 0);
            const int pos = prm.positions[tok];
            const int hi = valid ? pos : -1;               // a row without a token sees no key
            const int lo = prm.window > 0 ? (pos - prm.window + 1 > 0 ? pos - prm.window + 1 : 0) : 0;
            {
                // every matrix product that read the previous item's Q has completed: that item's
                // O has been taken
                const __nv_bfloat16* q_row = prm.q + ((size_t)tok * prm.nh + head) * HD;
#pragma unroll
                for (int c = 0; c < HD / 8; ++c) {
                    const uint4 v = valid ? *reinterpret_cast<const uint4*>(q_row + c * 8) : make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(q_s + (c >> 3) * L::Q_BOX + row * 128 + (((c & 7) ^ swz) << 4)) = v;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(q_ready);
            }
            // m: the maximum the exponents are taken against.  It follows the true running maximum
            // only when that has moved by more than RESCALE_STEP (in base 2), so P stays below
            // 2^RESCALE_STEP and O, which accumulates in tensor memory, is rescaled rarely.
            float m = -INFINITY, l = 0.0f;
            // the highest lower bound of the keys any row of this item may see
            const int lo_max = prm.window > 0 ? (item.pos_last - prm.window + 1 > 0 ? item.pos_last - prm.window + 1 : 0) : 0;
            for (int j = 0; j < item.n_tiles; ++j) {
                const int g = g0 + j, key0 = (item.tile_begin + j) * KEYS, buf = g & 1;
                ok = mbar_wait(&s_ready[buf], (g >> 1) & 1, abort_flag, 16, prm.status);
                ok = __all_sync(0xffffffffu, ok);          // tcgen05.ld needs the whole warp
                if (!ok) break;
                tc_fence_after();
                float sc[KEYS];
                tmem_ld64(lane_addr + buf * KEYS, sc);
                tc_fence_before();                         // S is out of its buffer before this warp says that P is ready
                // a tile every row sees whole needs no mask (rows without a token are never stored)
                const bool whole = key0 >= lo_max && key0 + KEYS - 1 <= item.pos_first;
                if (!whole) {
#pragma unroll
                    for (int i = 0; i < KEYS; ++i) {
                        const int key = key0 + i;
                        sc[i] = (key >= lo && key <= hi) ? sc[i] : -INFINITY;
                    }
                }
                // four interleaved chains each for the maximum and the sum: a fixed order, a quarter of the latency
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < KEYS; ++i) mx[i & 3] = fmaxf(mx[i & 3], sc[i]);
                const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * prm.scale_log2;
                const bool moved = tile_max > m + RESCALE_STEP;          // also: the row's first keys (m = -inf)
                float factor = 1.0f;
                if (moved) {
                    factor = ex2(m - tile_max);                          // 2^(-inf) = 0 for the first keys
                    m = tile_max;
                    l *= factor;
                }
                if (j > 0 && __any_sync(0xffffffffu, moved)) {
                    // every PV so far has landed in O; scale this warp's rows (by exactly 1 where nothing moved)
                    ok = mbar_wait(&pv_ready[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag, 18, prm.status);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        float v[32];
                        tmem_ld32(o_addr + c0, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] *= factor;
                        tmem_st32(o_addr + c0, v);
                    }
                    tc_fence_before();
                }
                const float zero = m == -INFINITY ? 0.0f : m;            // a row that has seen no key yet
                float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                uint32_t packed[KEYS / 2];
#pragma unroll
                for (int i = 0; i < KEYS; i += 2) {
                    const float p0 = ex2(fmaf(sc[i], prm.scale_log2, -zero));         // masked: 2^(-inf) = 0
                    const float p1 = ex2(fmaf(sc[i + 1], prm.scale_log2, -zero));
                    sum[i & 3] += p0;
                    sum[(i + 1) & 3] += p1;
                    packed[i >> 1] = pack2(p0, p1);
                }
                l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
                // P goes back into the columns its scores came from (bfloat16 pairs in the first 32 of
                // the buffer's 64 columns): the PV product reads it from tensor memory.  The buffer's
                // last reader, PV of the tile before the last, had completed when this tile's S was
                // ready, and PV of this tile is issued before the scores of tile g + 2 overwrite it
                float as_bits[KEYS / 2];
#pragma unroll
                for (int i = 0; i < KEYS / 2; ++i) as_bits[i] = __uint_as_float(packed[i]);
                tmem_st32(lane_addr + buf * KEYS, as_bits);
                tc_fence_before();
                const int seen = item.pos_last - key0 + 1;                // keys of this tile anybody may see
                if (seen < KEYS) {
                    // only the last tile: clear the V rows beyond it (whole 128-byte rows of every box)
                    const int u = u0 + j + LEAD, s = u % L::STAGES;   // the step that brought this V tile
                    ok = mbar_wait(&full[s], (u / L::STAGES) & 1, abort_flag, 17, prm.status);
                    uint8_t* v_tile = v_s + (size_t)s * L::KV_BYTES;
                    const int chunks = (KEYS - seen) * 8;
                    for (int b = 0; b < L::BOXES; ++b)
                        for (int i = threadIdx.x - 64; i < chunks; i += 32 * SOFTMAX_WARPS)
                            *reinterpret_cast<uint4*>(v_tile + b * L::KV_BOX + seen * 128 + i * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                if (seen < KEYS) fence_proxy_async();        // the cleared V rows, for the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_ready[buf]);
            }
            // O / l: the item's last PV has landed
            if (ok) {
                const int last = g0 + item.n_tiles - 1;
                ok = mbar_wait(&pv_ready[last & 1], (last >> 1) & 1, abort_flag, 20, prm.status);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                tc_fence_after();
                const float inv = 1.0f / l;
                __nv_bfloat16* dst = prm.out + ((size_t)tok * prm.nh + head) * HD;
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    float v[32];
                    tmem_ld32(o_addr + c0, v);
                    if (valid && !*abort_flag) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint4 packed;
                            packed.x = pack2(v[8 * c + 0] * inv, v[8 * c + 1] * inv);
                            packed.y = pack2(v[8 * c + 2] * inv, v[8 * c + 3] * inv);
                            packed.z = pack2(v[8 * c + 4] * inv, v[8 * c + 5] * inv);
                            packed.w = pack2(v[8 * c + 6] * inv, v[8 * c + 7] * inv);
                            *reinterpret_cast<uint4*>(dst + c0 + c * 8) = packed;
                        }
                    }
                }
                tc_fence_before();
            }
            g0 += item.n_tiles;
            u0 += item.n_tiles + LEAD;
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

template <int HD>
int launch(const CUtensorMap& map_k, const CUtensorMap& map_v, const AttnParams& prm, int n_tiles,
           cudaStream_t stream) {
    using L = Layout<HD>;
    auto kernel = attention_prefill_tcgen05_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int n_items = n_tiles * prm.nkv;
    fwb::pdl(kernel, dim3(prm.items_per_cta == 2 ? (n_items + 1) / 2 : n_items), THREADS, L::SMEM, stream)(
        map_k, map_v, prm);
    return fwb_launch_status();
}

}  // namespace

// Shapes this kernel takes; everything else runs the mma.sync kernel.
FWB_API int fwb_attention_prefill_tcgen05_accepts(int nh, int nkv, int hd, int page_size) {
    return (hd == 64 || hd == 128) && page_size == KEYS && nkv > 0 && nh % nkv == 0 && nh / nkv <= ROWS;
}

// q, out: [T][nh*hd] bf16.  k_pool, v_pool: [num_pages][nkv][64][hd] bf16.  tile_seg, tile_tok0:
// [n_tiles]; a tile holds up to `tokens_per_tile` (<= 128 / group) consecutive tokens of one segment.
FWB_API int fwb_attention_prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool,
                                          const int* positions, const int* seg_start, const int* tile_seg,
                                          const int* tile_tok0, const int* block_table, int max_pages,
                                          int page_size, int num_pages, void* out, int n_tiles, int nh,
                                          int nkv, int hd, int tokens_per_tile, int window, float scale,
                                          cudaStream_t stream) {
    if (n_tiles <= 0) return FWB_OK;
    if (!q || !k_pool || !v_pool || !positions || !seg_start || !tile_seg || !tile_tok0 || !block_table || !out)
        return FWB_BAD_ARGUMENT;
    if (!fwb_attention_prefill_tcgen05_accepts(nh, nkv, hd, page_size)) return FWB_UNSUPPORTED;
    const int group = nh / nkv;
    if (tokens_per_tile < 1 || tokens_per_tile * group > ROWS || num_pages <= 0) return FWB_BAD_ARGUMENT;
    if ((((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) != 0) return FWB_UNSUPPORTED;
    const long pool_rows = (long)num_pages * nkv * KEYS;
    if (pool_rows > 2147483647L || (long)n_tiles * nkv > 2147483647L) return FWB_TOO_LARGE;
    CUtensorMap map_k, map_v;
    if (!make_map(&map_k, k_pool, pool_rows, hd, KEYS)) return FWB_UNSUPPORTED;
    if (!make_map(&map_v, v_pool, pool_rows, hd, KEYS)) return FWB_UNSUPPORTED;
    AttnParams prm;
    prm.q = static_cast<const __nv_bfloat16*>(q);
    prm.out = static_cast<__nv_bfloat16*>(out);
    prm.positions = positions;
    prm.seg_start = seg_start;
    prm.tile_seg = tile_seg;
    prm.tile_tok0 = tile_tok0;
    prm.block_table = block_table;
    prm.max_pages = max_pages;
    prm.nh = nh;
    prm.nkv = nkv;
    prm.group = group;
    prm.tokens_per_tile = tokens_per_tile;
    prm.window = window;
    prm.n_row_tiles = n_tiles;
    // one CTA per SM is resident (the tiles fill shared memory): pairs of items even out the causal
    // triangle when there are waves of them; up to one wave of single items, single items finish sooner
    prm.items_per_cta = (long)n_tiles * nkv <= 148 ? 1 : 2;
    prm.scale_log2 = scale * LOG2E;
    prm.status = status_word();
    return hd == 64 ? launch<64>(map_k, map_v, prm, n_tiles, stream)
                    : launch<128>(map_k, map_v, prm, n_tiles, stream);
}
