// Causal grouped-query attention over the paged bfloat16 cache on tensor cores
// (mma.sync m16n8k16, fp32 accumulation and fp32 softmax), for head sizes 16..128.
//
// The rows of a tile are (query token, query head of one KV head) pairs, so the query heads
// that share a KV head also share every K/V tile that is loaded: a page of keys is read
// once per group, not once per query head.
//
//   prefill kernel: one CTA = one tile of 64 rows (64/group tokens x group heads) of one
//       segment and one KV head; 4 warps x 16 rows; walks the keys in 64-key tiles (one
//       page tile each) with an online softmax, K and V staged in shared memory by cp.async,
//       double buffered.
//   decode kernel:  one CTA = one token, one KV head, one slice of the context ("split");
//       the group's heads are the (padded) 16 rows, the 4 warps take 16 keys each of every
//       64-key tile; warps and then splits are merged with the usual (max, sum, acc) rule --
//       splits through a small fp32 scratch buffer and a second kernel, or inside the kernel as a
//       cluster.  At head sizes 64 and 128 the K and V tiles come by TMA: a (page, KV head) tile of
//       the pool is one box of a tensor map (two at head size 128), one thread asks for it and an
//       mbarrier says when it has landed; the 128-byte swizzle the copy leaves is what the
//       ldmatrix addresses undo.  Other head sizes are copied by cp.async into padded rows.
//
// Key tiles start at multiples of 64 and are visited in ascending order, whatever the cut.
#include "qk_head.cuh"
#include "tcgen05.cuh"

using namespace fwb;

namespace {

constexpr int KEYS = 64;            // keys per tile == page size
constexpr int WARPS = 4;
// Scores are kept in base 2: s * scale * log2(e), so the softmax exponentials are single ex2
// operations (fp32, relative error 2^-22); running maxima and the partial results of context
// slices live in the same domain.
constexpr float LOG2E = 1.4426950408889634f;
int g_decode_tma = 1;               // test switch: 0 sends head sizes 64 and 128 down the cp.async way too
int g_decode_tma_stages = 0;        // test switch: ring depth of the TMA way (0: chosen by the launcher)
constexpr int MAX_TMA_STAGES = 8;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Ring depth of the decode kernel when the launch is small (few CTAs: each should have more of
// its slice in flight); as deep as leaves three CTAs to an SM.  Large launches keep two stages
// and twice the CTAs per SM (measured at batch 8 and 64: the deep ring is 1 to 5 % slower there,
// at batch 1 it is 2.6 % faster).
template <int HD> constexpr int decode_stages() { return HD <= 64 ? 4 : (HD <= 96 ? 3 : 2); }

template <int HD>
struct Smem {
    static constexpr int ROW = HD + 8;                     // bf16 elements; +16 bytes: no bank conflicts
    static constexpr int TILE = KEYS * ROW;                // one K or V tile
    static constexpr int BYTES = 2 * 2 * TILE * 2;         // 2 stages x (K, V) x bf16
};

// Where 8 channels (one 16-byte chunk) of a key lie in a tile.  Padded rows (cp.async), or what a
// TMA box of [64 keys][64 channels] with the 128-byte swizzle leaves: rows of 128 bytes whose chunks
// are XOR-ed with the row number mod 8; a head of 128 channels is two such boxes, one after the other.
template <int HD, bool SWZ>
__device__ __forceinline__ const __nv_bfloat16* tile_at(const __nv_bfloat16* tile, int key, int chunk) {
    if (!SWZ) return tile + key * Smem<HD>::ROW + chunk * 8;
    return tile + (chunk >> 3) * (KEYS * 64) + key * 64 + (((chunk & 7) ^ (key & 7)) << 3);
}

// Copy one (page, kv head) tile of K and of V into shared memory (whole CTA).
template <int HD>
__device__ __forceinline__ void load_tile(__nv_bfloat16* ks, __nv_bfloat16* vs,
                                          const __nv_bfloat16* __restrict__ k_pool,
                                          const __nv_bfloat16* __restrict__ v_pool, size_t src) {
    constexpr int CHUNKS = HD / 8;                         // 16-byte chunks per row
    for (int i = threadIdx.x; i < KEYS * CHUNKS; i += WARPS * 32) {
        const int r = i / CHUNKS, c = i - r * CHUNKS;
        cp_async16(ks + r * Smem<HD>::ROW + c * 8, k_pool + src + (size_t)r * HD + c * 8);
        cp_async16(vs + r * Smem<HD>::ROW + c * 8, v_pool + src + (size_t)r * HD + c * 8);
    }
}

// Rows of a V tile past the last key anybody may see hold whatever the page held before
// (or nothing yet); their probabilities are exactly 0, but 0 * garbage must stay 0, so the
// rows are cleared.  Called by the whole CTA between two barriers.
template <int HD, bool SWZ = false>
__device__ __forceinline__ void clear_v_rows(__nv_bfloat16* vs, int first_row) {
    constexpr int CHUNKS = HD / 8;
    for (int i = threadIdx.x; i < (KEYS - first_row) * CHUNKS; i += WARPS * 32) {
        const int r = first_row + i / CHUNKS, c = i % CHUNKS;
        *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(tile_at<HD, SWZ>(vs, r, c))) = make_uint4(0u, 0u, 0u, 0u);
    }
}

// One warp: S[16 x NK*8] += Q[16 x HD] * K[keys][HD]^T for the keys that start at `key0`.
template <int HD, int NT, bool SWZ = false>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const uint32_t (&qf)[HD / 16][4],
                                        const __nv_bfloat16* ks, int key0, int lane) {
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[n][j] = 0.0f;
    // ldmatrix.x4: matrices (keys 0-7, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 0-7), (keys 8-15, d 8-15)
    const int mat = lane >> 3, r = lane & 7;
    const int key_off = (mat >> 1) * 8 + r, d_off = (mat & 1) * 8;
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, tile_at<HD, SWZ>(ks, key0 + n * 8 + key_off, 2 * k + (d_off >> 3)));
            mma_bf16(s[n], qf[k], b[0], b[1]);
            mma_bf16(s[n + 1], qf[k], b[2], b[3]);
        }
    }
}

// One warp: O[16 x HD] += P[16 x NT*8] * V[keys][HD], P taken from the score registers.
template <int HD, int NT, bool SWZ = false>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const float (&p)[NT][4],
                                        const __nv_bfloat16* vs, int key0, int lane) {
    // ldmatrix.x4.trans: matrices (keys 0-7, d 0-7), (keys 8-15, d 0-7), (keys 0-7, d 8-15), (keys 8-15, d 8-15)
    const int mat = lane >> 3, r = lane & 7;
    const int key_off = (mat & 1) * 8 + r, d_off = (mat >> 1) * 8;
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
        a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
        a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
        a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
        for (int n = 0; n < HD / 8; n += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, tile_at<HD, SWZ>(vs, key0 + kk * 16 + key_off, n + (d_off >> 3)));
            mma_bf16(o[n], a, b[0], b[1]);
            mma_bf16(o[n + 1], a, b[2], b[3]);
        }
    }
}

// Scale, mask and online-softmax one row pair (rows g and g+8 of the warp's 16) over NT*8 keys.
// key index of s[n][j]: key_base + n*8 + 2*t + (j&1); row of s[n][j]: g + 8*(j>>1).
template <int HD, int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&o)[HD / 8][4], float (&m)[2],
                                               float (&l)[2], int key_base, const int (&lo)[2],
                                               const int (&hi)[2], float scale, int lane) {
    const int t = lane & 3;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int key = key_base + n * 8 + 2 * t + (j & 1);
            const int h = j >> 1;
            const float v = (key >= lo[h] && key <= hi[h]) ? s[n][j] * scale : -INFINITY;   // scale has log2(e) folded in
            s[n][j] = v;
            mx[h] = fmaxf(mx[h], v);
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float corr[2], sum[2] = {0.0f, 0.0f}, base[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float m_new = fmaxf(m[h], mx[h]);
        base[h] = m_new == -INFINITY ? 0.0f : m_new;       // a row that has seen no key yet
        corr[h] = exp2f(m[h] - base[h]);                   // 2^(-inf) = 0
        m[h] = m_new;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int h = j >> 1;
            const float p = exp2f(s[n][j] - base[h]);      // masked: 2^(-inf) = 0
            s[n][j] = p;
            sum[h] += p;
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
        l[h] = l[h] * corr[h] + sum[h];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        o[n][0] *= corr[0];
        o[n][1] *= corr[0];
        o[n][2] *= corr[1];
        o[n][3] *= corr[1];
    }
}

// Q fragments of 16 rows: row r of the warp reads HD bf16 at q_rows[r] (nullptr: a zero row).
template <int HD>
__device__ __forceinline__ void load_q(uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* row_lo,
                                       const __nv_bfloat16* row_hi, int lane) {
    const int t = lane & 3;
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
        const int d = k * 16 + 2 * t;
        qf[k][0] = row_lo ? *reinterpret_cast<const uint32_t*>(row_lo + d) : 0u;
        qf[k][1] = row_hi ? *reinterpret_cast<const uint32_t*>(row_hi + d) : 0u;
        qf[k][2] = row_lo ? *reinterpret_cast<const uint32_t*>(row_lo + d + 8) : 0u;
        qf[k][3] = row_hi ? *reinterpret_cast<const uint32_t*>(row_hi + d + 8) : 0u;
    }
}

// ------------------------------------------------------------------ prefill
// tile_seg[b], tile_tok0[b]: segment and first token (global index) of row tile b.
template <int HD>
__global__ void __launch_bounds__(WARPS * 32, HD <= 64 ? 4 : 2)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ positions,
                         const int* __restrict__ seg_start, const int* __restrict__ tile_seg,
                         const int* __restrict__ tile_tok0, const int* __restrict__ block_table,
                         int max_pages, __nv_bfloat16* __restrict__ out, int nh, int nkv, int group,
                         int tokens_per_tile, int window, float scale) {
    fwb::pdl_entry();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // the last tiles of a prompt walk the most keys: they go first, so that the launch does not
    // end on a few long CTAs
    const int tile_index = gridDim.x - 1 - blockIdx.x;
    const int seg = tile_seg[tile_index], tok0 = tile_tok0[tile_index], kvh = blockIdx.y;
    const int seg_end = seg_start[seg + 1];
    int n_tok = seg_end - tok0;
    if (n_tok > tokens_per_tile) n_tok = tokens_per_tile;
    const int rows = n_tok * group;                         // valid rows of this tile (<= 64)
    const int* table = block_table + (size_t)seg * max_pages;

    // the two rows this thread owns inside its warp's 16: r = warp*16 + g (+8)
    int tok[2], head[2], lo[2], hi[2];
    const __nv_bfloat16* qrow[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + g + 8 * h;
        const bool valid = r < rows;
        tok[h] = tok0 + (valid ? r / group : 0);
        head[h] = kvh * group + (valid ? r % group : 0);
        const int pos = positions[tok[h]];
        hi[h] = valid ? pos : -1;                           // an invalid row sees no key
        lo[h] = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
        qrow[h] = valid ? q + ((size_t)tok[h] * nh + head[h]) * HD : nullptr;
    }
    uint32_t qf[HD / 16][4];
    load_q<HD>(qf, qrow[0], qrow[1], lane);

    // keys this CTA walks: from the lowest key any row may see to the position of its last token
    const int pos_first = positions[tok0], pos_last = positions[tok0 + n_tok - 1];
    const int lo_block = window > 0 ? (pos_first - window + 1 > 0 ? pos_first - window + 1 : 0) : 0;
    const int tile_begin = lo_block / KEYS, tile_end = pos_last / KEYS + 1;

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[n][j] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    auto stage_k = [&](int s) { return smem + s * 2 * Smem<HD>::TILE; };
    auto stage_v = [&](int s) { return smem + s * 2 * Smem<HD>::TILE + Smem<HD>::TILE; };
    auto issue = [&](int tile, int s) {
        const size_t src = ((size_t)table[tile] * nkv + kvh) * KEYS * HD;
        load_tile<HD>(stage_k(s), stage_v(s), k_pool, v_pool, src);
        cp_async_commit();
    };
    issue(tile_begin, 0);
    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int s = (tile - tile_begin) & 1;
        if (tile + 1 < tile_end) {
            issue(tile + 1, s ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (pos_last - tile * KEYS + 1 < KEYS) {
            clear_v_rows<HD>(stage_v(s), pos_last - tile * KEYS + 1);
            __syncthreads();
        }
        // a warp whose rows all lie before this tile's first key has nothing to do in it
        const int warp_hi = __reduce_max_sync(0xffffffffu, hi[0] > hi[1] ? hi[0] : hi[1]);
        if (warp_hi >= tile * KEYS) {
            float sc[8][4];
            qk_tile<HD, 8>(sc, qf, stage_k(s), 0, lane);
            softmax_update<HD, 8>(sc, o, m, l, tile * KEYS, lo, hi, scale, lane);
            pv_tile<HD, 8>(o, sc, stage_v(s), 0, lane);
        }
        __syncthreads();                                    // the stage may be overwritten next
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (hi[h] < 0) continue;
        const float inv = 1.0f / l[h];
        __nv_bfloat16* dst = out + ((size_t)tok[h] * nh + head[h]) * HD;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
    }
}

// ------------------------------------------------------------------ decode
// The decode kernel may do the step's q/k norm, rotation and page write itself (a step of single
// tokens only): it then reads the rows of the fused q|k|v projection instead of finished queries.
struct FusedQkv {
    const __nv_bfloat16* qkv;    // [T][(nh + 2 nkv_in) HD]; null: `q` holds finished queries
    const float* wq;             // [HD] head-norm weights (unused when !use_norm)
    const float* wk;
    const float2* table;         // [positions][rot / 2] (cos, sin)
    __nv_bfloat16* k_pool;       // where the token's key and value go (nkv_in > 0)
    __nv_bfloat16* v_pool;
    int nkv_in;                  // KV heads in the qkv row (0: this layer reads another layer's cache)
    int rot, pairing, use_norm;
    float eps;
};

// The fused form's prologue (not inlined: its registers are not the main loop's): norm and turn the
// queries of this KV head's group into `own_q` [group][HD]; in the slice that holds the token's own
// position also its key and value, into `own_kv` [2][HD] and into the pools at `cache_at` (for the
// steps to come).  hd/8 adjacent lanes own a head, as in the kernel that does this for whole steps.
template <int HD>
__device__ __noinline__ void fused_heads(const FusedQkv& fused, int tok, int pos, int kvh, int nh, int nkv, int group,
                                         bool owns_token, size_t cache_at, __nv_bfloat16* own_q,
                                         __nv_bfloat16* own_kv) {
    constexpr int G = HD / 8, PER_WARP = 32 / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane / G, gl = lane - sub * G;
    const int heads_in = nh + 2 * fused.nkv_in;
    const __nv_bfloat16* row = fused.qkv + (size_t)tok * heads_in * HD;
    const float2* cs = fused.table + (size_t)pos * (fused.rot / 2);
    const int n_slots = group + (owns_token ? 2 : 0);
    for (int slot0 = warp * PER_WARP; slot0 < n_slots; slot0 += WARPS * PER_WARP) {
        const int slot = slot0 + sub;
        const bool valid = sub < PER_WARP && slot < n_slots;
        const int kind = slot < group ? 0 : (slot == group ? 1 : 2);
        const int h = kind == 0 ? kvh * group + slot : (kind == 1 ? nh + kvh : nh + fused.nkv_in + kvh);
        float v[8];
        if (valid) {
            load8(row + (size_t)h * HD + gl * 8, v);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        head_norm_rope8(v, valid, kind, sub, gl, G, HD, fused.rot, fused.pairing, fused.use_norm, fused.eps,
                        fused.wq, fused.wk, cs);
        if (!valid) continue;
        if (kind == 0) {
            store8(own_q + slot * HD + gl * 8, v);
        } else {
            store8(own_kv + (kind - 1) * HD + gl * 8, v);
            store8((kind == 1 ? fused.k_pool : fused.v_pool) + cache_at + gl * 8, v);
        }
    }
}

// grid (splits, nkv, T).  A split covers `tiles_per_split` key tiles; with splits == 1 the
// result goes straight to `out`, else (acc, max, sum) go to the scratch buffers:
//   part_o[t][kvh][split][group][HD] fp32 (not normalised), part_ml[t][kvh][split][group][2].
//
// TMA: the tiles are boxes of the tensor maps `map_k` / `map_v` over the pools seen as
// [pages * nkv * 64 keys][HD] (head sizes 64 and 128; the maps are not read otherwise).  Thread 0
// asks for a tile's boxes and arms the stage's mbarrier with their bytes; every thread waits on that
// barrier itself (bounded: after the limit the library's status word is raised and nobody waits again).
// FUSED: the form that norms, turns and stores its own token's heads (an instantiation of its own: the
// plain form carries none of its registers, shared memory or branches).
template <int HD, bool CLUSTER, bool DEEP, bool TMA, bool FUSED>
__global__ void __launch_bounds__(WARPS * 32, (TMA && HD <= 64) ? 5 : 1)   // five CTAs an SM: what the slicing rule counts on
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, const int* __restrict__ positions,
                        const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                        int max_pages, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int nh, int nkv, int group, int tiles_per_split,
                        int window, float scale, int* status, int tma_stages, const FusedQkv fused) {
    fwb::pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t smem_dynamic[];
    // the swizzle of a TMA box counts rows from a 1024-byte boundary
    uint8_t* smem_raw = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dynamic) + 1023) & ~uintptr_t(1023))
                            : smem_dynamic;
    __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __shared__ float merge_ml[WARPS][16][2];
    __shared__ uint64_t full_bar[MAX_TMA_STAGES];
    __shared__ int abort_flag;
    __shared__ __align__(16) __nv_bfloat16 own_q[FUSED ? 16 * HD : 8];    // fused form: the group's queries, normed and turned
    __shared__ __align__(16) __nv_bfloat16 own_kv[FUSED ? 2 * HD : 8];    // ... and the token's own key and value
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, splits = gridDim.x, kvh = blockIdx.y, tok = blockIdx.z;
    // positions, segments and block tables were uploaded before the step's first kernel started,
    // and every key tile but the token's last one was written by earlier steps: the first tile
    // of a slice that does not hold the token itself is fetched before the wait for the previous
    // kernel (which writes this step's keys and the queries)
    const int pos = positions[tok];
    const int lo_key = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
    const int* table = block_table + (size_t)tok_seg[tok] * max_pages;
    const int first_tile = lo_key / KEYS, last_tile = pos / KEYS;
    const int tile_begin = first_tile + split * tiles_per_split;
    int tile_end = tile_begin + tiles_per_split;
    if (tile_end > last_tile + 1) tile_end = last_tile + 1;

    // cp.async: two stages, or the deep ring; TMA: as many as the launcher found room for
    const int DECODE_STAGES = TMA ? tma_stages : (DEEP ? decode_stages<HD>() : 2);
    constexpr int TILE = TMA ? KEYS * HD : Smem<HD>::TILE;  // elements of one K or V tile in shared memory
    // A ring of DECODE_STAGES key/value tiles: a slice of eight tiles has half of its bytes in
    // flight from the start (two stages left the memory pipe waiting on every tile's round trip).
    auto stage_k = [&](int s) { return smem + s * 2 * TILE; };
    auto stage_v = [&](int s) { return smem + s * 2 * TILE + TILE; };
    if (TMA) {
        if (threadIdx.x == 0) {
            for (int s = 0; s < DECODE_STAGES; ++s) tc5::mbar_init(&full_bar[s], 1);
            abort_flag = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    }
    auto issue = [&](int tile, int s) {
        if (TMA) {
            if (threadIdx.x == 0 && tile < tile_end) {
                // the stage was read (and, in a token's last tile, cleared) through ordinary loads and stores
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tc5::mbar_expect_tx(&full_bar[s], 2 * TILE * 2);
                const int row = (table[tile] * nkv + kvh) * KEYS;
#pragma unroll
                for (int x = 0; x < HD / 64; ++x) {
                    tc5::tma_load_2d(stage_k(s) + x * KEYS * 64, &map_k, &full_bar[s], x * 64, row);
                    tc5::tma_load_2d(stage_v(s) + x * KEYS * 64, &map_v, &full_bar[s], x * 64, row);
                }
            }
            return;
        }
        if (tile < tile_end) {
            const size_t src = ((size_t)table[tile] * nkv + kvh) * KEYS * HD;
            load_tile<HD>(stage_k(s), stage_v(s), k_pool, v_pool, src);
        }
        cp_async_commit();                                  // an empty group keeps the count in step
    };
    // every tile but the token's own last one was written by earlier steps: those among the first
    // DECODE_STAGES - 1 are fetched before the wait for the previous kernel
    int issued = 0;
    while (issued < DECODE_STAGES - 1 && tile_begin + issued < tile_end && tile_begin + issued < last_tile) {
        issue(tile_begin + issued, issued);
        ++issued;
    }
    fwb::pdl_wait();

    constexpr bool fuse = FUSED;
    // the slice that holds the token's own position also norms, turns and stores its key and value
    const bool owns_token = fuse && fused.nkv_in > 0 && last_tile >= tile_begin && last_tile < tile_end;
    if constexpr (fuse) {
        fused_heads<HD>(fused, tok, pos, kvh, nh, nkv, group, owns_token,
                        owns_token ? (((size_t)table[last_tile] * nkv + kvh) * KEYS + (size_t)(pos % KEYS)) * HD : 0,
                        own_q, own_kv);
        __syncthreads();
    }
    // rows 0..group-1 are the group's query heads; the rest are padding
    const __nv_bfloat16* q_rows = fuse ? own_q : q + ((size_t)tok * nh + kvh * group) * HD;
    const __nv_bfloat16* qrow0 = g < group ? q_rows + (size_t)g * HD : nullptr;
    const __nv_bfloat16* qrow1 = g + 8 < group ? q_rows + (size_t)(g + 8) * HD : nullptr;
    uint32_t qf[HD / 16][4];
    load_q<HD>(qf, qrow0, qrow1, lane);
    const int lo[2] = {lo_key, lo_key};
    const int hi[2] = {g < group ? pos : -1, g + 8 < group ? pos : -1};

    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[n][j] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    for (; issued < DECODE_STAGES - 1; ++issued) issue(tile_begin + issued, issued);
    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int s = (tile - tile_begin) % DECODE_STAGES;
        // the slot this tile's successor-but-two goes to was read in the iteration before this one
        issue(tile + DECODE_STAGES - 1, (tile - tile_begin + DECODE_STAGES - 1) % DECODE_STAGES);
        if (TMA) {
            // the tile's bytes have landed when its barrier's phase completes; a thread that has
            // seen that may read them
            tc5::mbar_wait(&full_bar[s], (uint32_t)((tile - tile_begin) / DECODE_STAGES) & 1u, &abort_flag, 21, status);
        } else {
            cp_async_wait<(DEEP ? decode_stages<HD>() : 2) - 1>();
            __syncthreads();
        }
        if (tile == last_tile && (owns_token || pos - tile * KEYS + 1 < KEYS)) {
            if (owns_token && threadIdx.x < 2 * (HD / 8)) {
                // the page row of the token itself: what this CTA has just computed (the copy in the
                // pool may or may not have been seen by the tile's load)
                const int which = threadIdx.x / (HD / 8), c = threadIdx.x % (HD / 8);
                __nv_bfloat16* tile_base = which ? stage_v(s) : stage_k(s);
                *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(tile_at<HD, TMA>(tile_base, pos % KEYS, c))) =
                    *reinterpret_cast<const uint4*>(own_kv + which * HD + c * 8);
            }
            if (pos - tile * KEYS + 1 < KEYS) clear_v_rows<HD, TMA>(stage_v(s), pos - tile * KEYS + 1);
            __syncthreads();
        }
        float sc[2][4];                                     // this warp's 16 keys of the tile
        qk_tile<HD, 2, TMA>(sc, qf, stage_k(s), warp * 16, lane);
        softmax_update<HD, 2>(sc, o, m, l, tile * KEYS + warp * 16, lo, hi, scale, lane);
        pv_tile<HD, 2, TMA>(o, sc, stage_v(s), warp * 16, lane);
        __syncthreads();
    }

    // ---- merge the four warps (each saw a quarter of the keys) through shared memory
    float* merge_o = reinterpret_cast<float*>(smem_raw);    // [WARPS][16][HD] fp32, stages are free now
    float* cta_o = merge_o + WARPS * 16 * HD;               // [16][HD]: this CTA's result (CLUSTER)
    float* cta_ml = cta_o + 16 * HD;                        // [16][2]
    if (t == 0) {
        merge_ml[warp][g][0] = m[0];
        merge_ml[warp][g][1] = l[0];
        merge_ml[warp][g + 8][0] = m[1];
        merge_ml[warp][g + 8][1] = l[1];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        float* row0 = merge_o + ((size_t)warp * 16 + g) * HD + n * 8 + 2 * t;
        float* row1 = merge_o + ((size_t)warp * 16 + g + 8) * HD + n * 8 + 2 * t;
        row0[0] = o[n][0];
        row0[1] = o[n][1];
        row1[0] = o[n][2];
        row1[1] = o[n][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < group * HD; i += WARPS * 32) {
        const int r = i / HD, d = i - r * HD;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, merge_ml[w][r][0]);
        const float base = mm == -INFINITY ? 0.0f : mm;
        float acc = 0.0f, ll = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float c = exp2f(merge_ml[w][r][0] - base);
            acc += c * merge_o[((size_t)w * 16 + r) * HD + d];
            ll += c * merge_ml[w][r][1];
        }
        if (splits == 1) {
            out[((size_t)tok * nh + kvh * group + r) * HD + d] = __float2bfloat16_rn(acc / ll);
        } else if (CLUSTER) {
            cta_o[r * HD + d] = acc;
            if (d == 0) {
                cta_ml[r * 2] = mm;
                cta_ml[r * 2 + 1] = ll;
            }
        } else {
            const size_t at = (((size_t)tok * nkv + kvh) * splits + split) * group + r;
            part_o[at * HD + d] = acc;
            if (d == 0) {
                part_ml[at * 2] = mm;
                part_ml[at * 2 + 1] = ll;
            }
        }
    }
    if (CLUSTER && splits > 1) {
        // The slices of one (token, KV head) form a thread-block cluster: every CTA left its
        // (acc, max, sum) in its own shared memory; each then merges a share of the outputs over
        // all slices, read through distributed shared memory in slice order.
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const uint32_t o_base = static_cast<uint32_t>(__cvta_generic_to_shared(cta_o));
        const uint32_t ml_base = static_cast<uint32_t>(__cvta_generic_to_shared(cta_ml));
        auto peer = [](uint32_t local, uint32_t rank) {
            uint32_t remote;
            float v;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
            asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
            return v;
        };
        for (int i = split * (WARPS * 32) + threadIdx.x; i < group * HD; i += splits * WARPS * 32) {
            const int r = i / HD, d = i - r * HD;
            float ms[8], ls[8], os[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const bool on = s < splits;
                ms[s] = on ? peer(ml_base + (uint32_t)(r * 2) * 4, s) : -INFINITY;
                ls[s] = on ? peer(ml_base + (uint32_t)(r * 2 + 1) * 4, s) : 0.0f;
                os[s] = on ? peer(o_base + (uint32_t)(r * HD + d) * 4, s) : 0.0f;
            }
            float mm = -INFINITY;
#pragma unroll
            for (int s = 0; s < 8; ++s) mm = fmaxf(mm, ms[s]);
            float acc = 0.0f, ll = 0.0f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const float c = exp2f(ms[s] - mm);          // a slice without keys: 2^(-inf) = 0
                acc += c * os[s];
                ll += c * ls[s];
            }
            out[((size_t)tok * nh + kvh * group + r) * HD + d] = __float2bfloat16_rn(acc / ll);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // nobody leaves while a peer reads
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
}

// grid (nkv, T), block 128: sum the splits in ascending order.  The loads of eight splits are
// issued together (they do not depend on one another), then combined one after the other.
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ out, int nh, int nkv, int group, int hd,
                                       int splits) {
    fwb::pdl_entry();
    const int kvh = blockIdx.x, tok = blockIdx.y;
    const size_t base_at = ((size_t)tok * nkv + kvh) * splits;
    for (int i = threadIdx.x; i < group * hd; i += blockDim.x) {
        const int r = i / hd, d = i - r * hd;
        float mm = -INFINITY;
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float m8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                m8[j] = s0 + j < splits ? part_ml[((base_at + s0 + j) * group + r) * 2] : -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) mm = fmaxf(mm, m8[j]);
        }
        float acc = 0.0f, ll = 0.0f;
        for (int s0 = 0; s0 < splits; s0 += 8) {
            float m8[8], l8[8], o8[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool on = s0 + j < splits;
                const size_t at = (base_at + s0 + j) * group + r;
                m8[j] = on ? part_ml[at * 2] : -INFINITY;
                l8[j] = on ? part_ml[at * 2 + 1] : 0.0f;
                o8[j] = on ? part_o[at * hd + d] : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float c = exp2f(m8[j] - mm);          // a split without keys: 2^(-inf) = 0
                acc += c * o8[j];
                ll += c * l8[j];
            }
        }
        out[((size_t)tok * nh + kvh * group + r) * hd + d] = __float2bfloat16_rn(acc / ll);
    }
}

template <typename K>
int opt_in_smem(K kernel, size_t bytes) {
    // these kernels live on shared memory, not L1: ask for the largest carve-out so that as many
    // CTAs as the registers allow are resident
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (bytes <= 48 * 1024) return FWB_OK;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return e == cudaSuccess ? FWB_OK : (int)e;
}

template <int HD>
int launch_prefill(const void* q, const void* k_pool, const void* v_pool, const int* positions,
                   const int* seg_start, const int* tile_seg, const int* tile_tok0, const int* block_table,
                   int max_pages, void* out, int n_tiles, int nh, int nkv, int tokens_per_tile, int window,
                   float scale, cudaStream_t stream) {
    auto kernel = attention_prefill_kernel<HD>;
    int st = opt_in_smem(kernel, Smem<HD>::BYTES);
    if (st != FWB_OK) return st;
    using bf = __nv_bfloat16;
    fwb::pdl(kernel, dim3(n_tiles, nkv), WARPS * 32, Smem<HD>::BYTES, stream)(
        (const bf*)q, (const bf*)k_pool, (const bf*)v_pool, positions, seg_start, tile_seg, tile_tok0,
        block_table, max_pages, (bf*)out, nh, nkv, nh / nkv, tokens_per_tile, window, scale * LOG2E);
    return fwb_launch_status();
}

template <int HD, bool TMA>
int launch_decode_as(const CUtensorMap& map_k, const CUtensorMap& map_v, const void* q, const void* k_pool,
                     const void* v_pool, const int* positions, const int* tok_seg, const int* block_table,
                     int max_pages, void* out, float* part_o, float* part_ml, int T, int nh, int nkv, int splits,
                     int tiles_per_split, int window, float scale, bool in_cluster, const FusedQkv& fused,
                     cudaStream_t stream) {
    constexpr size_t merge_bytes = (size_t)(WARPS + 1) * 16 * HD * 4 + 16 * 2 * 4;
    // few CTAs (at most three per SM): the deep ring; else two stages and more CTAs per SM
    const bool deep = (long)splits * nkv * T <= 3 * 148;
    // TMA tiles are not padded, but start on a 1024-byte boundary
    constexpr size_t tile_bytes = TMA ? (size_t)KEYS * HD * 2 : (size_t)Smem<HD>::TILE * 2;
    constexpr size_t slack = TMA ? 1024 : 0;
    constexpr size_t shallow_ring = 2 * 2 * tile_bytes, deep_ring = decode_stages<HD>() * 2 * tile_bytes;
    constexpr size_t shallow_bytes = (shallow_ring > merge_bytes ? shallow_ring : merge_bytes) + slack;
    constexpr size_t deep_bytes = (deep_ring > merge_bytes ? deep_ring : merge_bytes) + slack;
    size_t bytes = deep ? deep_bytes : shallow_bytes;
    int stages = 0;
    if (TMA) {
        // as deep a ring as lets the CTAs that share an SM all fit (registers allow five at head size
        // 64, three at 128), and no deeper than a slice is long: a CTA more on an SM is worth more
        // than a stage more in the ring (8 x 4,096 keys: 15.4 us with three stages, 21.7 with four).
        // (Six CTAs an SM, with the registers capped at 80, were slower: 64 x 4,096 keys 90 -> 94 us.)
        const long ctas = (long)splits * nkv * T;
        const long most = HD <= 64 ? 5 : 3;
        long resident = (ctas + 147) / 148;
        resident = resident < 1 ? 1 : (resident > most ? most : resident);
        const size_t room = (size_t)(220 * 1024) / (size_t)resident - slack;
        stages = (int)(room / (2 * tile_bytes));
        stages = stages > MAX_TMA_STAGES ? MAX_TMA_STAGES : stages;
        stages = stages > tiles_per_split ? tiles_per_split : stages;
        stages = stages < 2 ? 2 : stages;
        if (g_decode_tma_stages >= 2 && g_decode_tma_stages <= MAX_TMA_STAGES) stages = g_decode_tma_stages;
        const size_t ring = (size_t)stages * 2 * tile_bytes;
        bytes = (ring > merge_bytes ? ring : merge_bytes) + slack;
    }
    int* status = tc5::status_word();
    using bf = __nv_bfloat16;
    if (splits > 1 && in_cluster) {
        // the slices of a (token, KV head) as a cluster: merged through distributed shared memory
        const bool fuse = fused.qkv != nullptr;
        auto kernel = fuse ? (deep ? attention_decode_kernel<HD, true, true, TMA, true> : attention_decode_kernel<HD, true, false, TMA, true>)
                           : (deep ? attention_decode_kernel<HD, true, true, TMA, false> : attention_decode_kernel<HD, true, false, TMA, false>);
        int st = opt_in_smem(kernel, bytes);
        if (st != FWB_OK) return st;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(splits, nkv, T);
        config.blockDim = dim3(WARPS * 32);
        config.dynamicSmemBytes = bytes;
        config.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attr;
        config.numAttrs = pdl_enabled() ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&config, kernel, map_k, map_v, (const bf*)q, (const bf*)k_pool,
                                           (const bf*)v_pool, positions, tok_seg, block_table, max_pages, (bf*)out,
                                           (float*)nullptr, (float*)nullptr, nh, nkv, nh / nkv,
                                           tiles_per_split, window, scale * LOG2E, status, stages, fused);
        return e == cudaSuccess ? fwb_launch_status() : (int)e;
    }
    const bool fuse = fused.qkv != nullptr;
    auto kernel = fuse ? (deep ? attention_decode_kernel<HD, false, true, TMA, true> : attention_decode_kernel<HD, false, false, TMA, true>)
                       : (deep ? attention_decode_kernel<HD, false, true, TMA, false> : attention_decode_kernel<HD, false, false, TMA, false>);
    int st = opt_in_smem(kernel, bytes);
    if (st != FWB_OK) return st;
    fwb::pdl(kernel, dim3(splits, nkv, T), WARPS * 32, bytes, stream)(
        map_k, map_v, (const bf*)q, (const bf*)k_pool, (const bf*)v_pool, positions, tok_seg, block_table, max_pages,
        (bf*)out, part_o, part_ml, nh, nkv, nh / nkv, tiles_per_split, window, scale * LOG2E, status, stages, fused);
    st = fwb_launch_status();
    if (st != FWB_OK || splits == 1) return st;
    fwb::pdl(attention_merge_kernel, dim3(nkv, T), 128, 0, stream)(part_o, part_ml, (bf*)out, nh, nkv, nh / nkv, HD,
                                                             splits);
    return fwb_launch_status();
}

// `num_pages` > 0 (the pools' first extent) lets head sizes 64 and 128 take their tiles by TMA.
template <int HD>
int launch_decode(const void* q, const void* k_pool, const void* v_pool, const int* positions,
                  const int* tok_seg, const int* block_table, int max_pages, int num_pages, void* out,
                  float* part_o, float* part_ml, int T, int nh, int nkv, int splits, int tiles_per_split,
                  int window, float scale, bool in_cluster, const FusedQkv& fused, cudaStream_t stream) {
    CUtensorMap map_k, map_v;
    memset(&map_k, 0, sizeof(map_k));
    memset(&map_v, 0, sizeof(map_v));
    if constexpr (HD == 64 || HD == 128) {
        const long pool_rows = (long)num_pages * nkv * KEYS;
        const bool aligned = ((((uintptr_t)k_pool) | ((uintptr_t)v_pool)) & 15) == 0;
        if (g_decode_tma && num_pages > 0 && aligned && pool_rows <= 2147483647L &&
            tc5::make_map(&map_k, k_pool, pool_rows, HD, KEYS) && tc5::make_map(&map_v, v_pool, pool_rows, HD, KEYS))
            return launch_decode_as<HD, true>(map_k, map_v, q, k_pool, v_pool, positions, tok_seg, block_table,
                                              max_pages, out, part_o, part_ml, T, nh, nkv, splits, tiles_per_split,
                                              window, scale, in_cluster, fused, stream);
    }
    return launch_decode_as<HD, false>(map_k, map_v, q, k_pool, v_pool, positions, tok_seg, block_table, max_pages,
                                       out, part_o, part_ml, T, nh, nkv, splits, tiles_per_split, window, scale,
                                       in_cluster, fused, stream);
}

bool shape_ok(int nh, int nkv, int hd, int page_size) {
    return nh > 0 && nkv > 0 && nh % nkv == 0 && nh / nkv <= 16 && hd >= 16 && hd <= 128 && hd % 16 == 0 &&
           page_size == KEYS && nkv <= 65535;
}

}  // namespace

#define FWB_HD_SWITCH(hd, CALL)                  \
    switch (hd) {                                \
        case 16: return CALL(16);                \
        case 32: return CALL(32);                \
        case 48: return CALL(48);                \
        case 64: return CALL(64);                \
        case 80: return CALL(80);                \
        case 96: return CALL(96);                \
        case 112: return CALL(112);              \
        case 128: return CALL(128);              \
        default: return FWB_UNSUPPORTED;         \
    }

// Prompt portions (and anything else): q, out [T][nh*hd] bf16; pools [pages][nkv][64][hd] bf16.
// tile_seg, tile_tok0: [n_tiles], a tile holds up to `tokens_per_tile` = 64 / group consecutive
// tokens of one segment.
FWB_API int fwb_attention_prefill_mma(const void* q, const void* k_pool, const void* v_pool,
                                      const int* positions, const int* seg_start, const int* tile_seg,
                                      const int* tile_tok0, const int* block_table, int max_pages,
                                      int page_size, void* out, int n_tiles, int nh, int nkv, int hd,
                                      int tokens_per_tile, int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return FWB_OK;
    if (!q || !k_pool || !v_pool || !positions || !seg_start || !tile_seg || !tile_tok0 || !block_table || !out)
        return FWB_BAD_ARGUMENT;
    if (!shape_ok(nh, nkv, hd, page_size)) return FWB_UNSUPPORTED;
    if (tokens_per_tile < 1 || tokens_per_tile * (nh / nkv) > 64) return FWB_BAD_ARGUMENT;
#define CALL(HD)                                                                                          \
    launch_prefill<HD>(q, k_pool, v_pool, positions, seg_start, tile_seg, tile_tok0, block_table, max_pages, \
                       out, n_tiles, nh, nkv, tokens_per_tile, window, scale, stream)
    FWB_HD_SWITCH(hd, CALL)
#undef CALL
}

// Decode tokens: one query token each.  The slices of the context are merged either inside the
// kernel (`merge_in_cluster` != 0, splits <= 8: the slices form a thread-block cluster; best
// while the launch has few CTAs) or by a second kernel through scratch: part_o needs
// T*nkv*splits*group*hd floats and part_ml T*nkv*splits*group*2 floats.  num_pages: the pools'
// first extent (0: unknown, no TMA).
FWB_API int fwb_attention_decode_mma(const void* q, const void* k_pool, const void* v_pool,
                                     const int* positions, const int* tok_seg, const int* block_table,
                                     int max_pages, int page_size, int num_pages, void* out, float* part_o,
                                     float* part_ml, int T, int nh, int nkv, int hd, int splits,
                                     int tiles_per_split, int window, float scale, int merge_in_cluster,
                                     cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!q || !k_pool || !v_pool || !positions || !tok_seg || !block_table || !out) return FWB_BAD_ARGUMENT;
    if (!shape_ok(nh, nkv, hd, page_size) || T > 65535) return FWB_UNSUPPORTED;
    const bool in_cluster = merge_in_cluster != 0 && splits <= 8;
    if (splits < 1 || tiles_per_split < 1 || (splits > 1 && !in_cluster && (!part_o || !part_ml))) return FWB_BAD_ARGUMENT;
    FusedQkv fused;
    memset(&fused, 0, sizeof(fused));
#define CALL(HD)                                                                                          \
    launch_decode<HD>(q, k_pool, v_pool, positions, tok_seg, block_table, max_pages, num_pages, out, part_o,  \
                      part_ml, T, nh, nkv, splits, tiles_per_split, window, scale, in_cluster, fused, stream)
    FWB_HD_SWITCH(hd, CALL)
#undef CALL
}

// The same for a step of single tokens only, with the q/k head norm, the rotation and the page write
// done by the attention kernel itself: qkv [T][(nh + 2 nkv_in) hd] bf16 is the fused projection
// (nkv_in = nkv, or 0 for a layer that reads another layer's cache and writes none), wq / wk [hd] fp32
// the head-norm weights (use_norm), table [positions][rot / 2] (cos, sin) pairs, pairing 0 half-split /
// 1 interleaved.  Each CTA norms and turns the queries of its KV head's group; the slice that holds a
// token's own position does the same to its key, copies its value, stores both into the pools for the
// steps to come and into its own tile of shared memory.  The arithmetic is that of fwb_qk_norm_rope's
// bfloat16 form (one function): the same bits.  Needs rot % 16 == 0 and 16-byte aligned rows.
FWB_API int fwb_attention_decode_fused(const void* qkv, int nkv_in, const float* wq, const float* wk,
                                       const void* table, int rot, float eps, int use_norm, int pairing,
                                       void* k_pool, void* v_pool, const int* positions, const int* tok_seg,
                                       const int* block_table, int max_pages, int page_size, int num_pages,
                                       void* out, float* part_o, float* part_ml, int T, int nh, int nkv, int hd,
                                       int splits, int tiles_per_split, int window, float scale,
                                       int merge_in_cluster, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!qkv || !table || !k_pool || !v_pool || !positions || !tok_seg || !block_table || !out) return FWB_BAD_ARGUMENT;
    if (!shape_ok(nh, nkv, hd, page_size) || T > 65535) return FWB_UNSUPPORTED;
    if (nkv_in != 0 && nkv_in != nkv) return FWB_BAD_ARGUMENT;
    if (use_norm && (!wq || (nkv_in > 0 && !wk))) return FWB_BAD_ARGUMENT;
    if (rot < 0 || rot > hd || (rot & 15) || (pairing != 0 && pairing != 1)) return FWB_UNSUPPORTED;
    if ((((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) != 0) return FWB_UNSUPPORTED;
    const bool in_cluster = merge_in_cluster != 0 && splits <= 8;
    if (splits < 1 || tiles_per_split < 1 || (splits > 1 && !in_cluster && (!part_o || !part_ml))) return FWB_BAD_ARGUMENT;
    FusedQkv fused;
    fused.qkv = static_cast<const __nv_bfloat16*>(qkv);
    fused.wq = wq;
    fused.wk = wk;
    fused.table = static_cast<const float2*>(table);
    fused.k_pool = static_cast<__nv_bfloat16*>(k_pool);
    fused.v_pool = static_cast<__nv_bfloat16*>(v_pool);
    fused.nkv_in = nkv_in;
    fused.rot = rot;
    fused.pairing = pairing;
    fused.use_norm = use_norm;
    fused.eps = eps;
#define CALL(HD)                                                                                                \
    launch_decode<HD>(nullptr, k_pool, v_pool, positions, tok_seg, block_table, max_pages, num_pages, out, part_o, \
                      part_ml, T, nh, nkv, splits, tiles_per_split, window, scale, in_cluster, fused, stream)
    FWB_HD_SWITCH(hd, CALL)
#undef CALL
}

// Test switch: whether head sizes 64 and 128 take their key and value tiles by TMA (the default) or by
// cp.async like the other head sizes, and how deep the TMA way's ring is (0: the launcher's choice).
// All give the same bits: the arithmetic does not change.
FWB_API int fwb_attention_decode_set_tma(int on, int stages) {
    g_decode_tma = on ? 1 : 0;
    g_decode_tma_stages = stages;
    return FWB_OK;
}
