// Causal grouped-query attention over the paged cache, plain SIMT, fp32 arithmetic.
//
// One block per (query token, KV head).  The block walks the keys that the token may
// see, lo..pos (lo = max(0, pos-window+1) with a window, else 0), in tiles of 32
// positions that start at multiples of 32, stages each K and V tile in shared memory
// once, and lets its warps run an online softmax for the query heads of that KV head.
// A tile never straddles a page (the page size is a multiple of 32).  The walk and the
// reduction order depend only on the token's own position, never on how the batch was
// cut, so the result for a token is the same in a whole prompt, in a portion, or as a
// single decoded token.
//
// This kernel is the attention of the 32-bit path, and the fallback of the bfloat16
// path for head sizes or group sizes the tensor-core kernels refuse.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int WARPS = 4;
constexpr int TILE = 32;
constexpr int MAX_HPW = 4;   // query heads per warp  -> group size <= 16
constexpr int MAX_DPL = 8;   // head channels per lane -> head size <= 256

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const TQ* __restrict__ q, const TC* __restrict__ k_pool,
                      const TC* __restrict__ v_pool, const int* __restrict__ positions,
                      const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                      int max_pages, int page_size, TO* __restrict__ out, int nh, int nkv, int hd,
                      int window, float scale) {
    fwb::pdl_entry();
    extern __shared__ float smem[];
    const int group = nh / nkv;
    float* qs = smem;                         // [group][hd]
    float* ks = qs + group * hd;              // [TILE][hd+1]
    float* vs = ks + TILE * (hd + 1);         // [TILE][hd]
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int* table = block_table + (size_t)tok_seg[t] * max_pages;
    const int lo = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;

    for (int i = threadIdx.x; i < group * hd; i += blockDim.x)
        qs[i] = to_f32<TQ>(q[((size_t)t * nh + (size_t)kvh * group) * hd + i]);

    float m[MAX_HPW], l[MAX_HPW], acc[MAX_HPW][MAX_DPL];
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
        m[a] = -INFINITY;
        l[a] = 0.0f;
#pragma unroll
        for (int d = 0; d < MAX_DPL; ++d) acc[a][d] = 0.0f;
    }

    for (int base = (lo / TILE) * TILE; base <= pos; base += TILE) {
        __syncthreads();
        const int page = table[base / page_size];
        const size_t src = (((size_t)page * nkv + kvh) * page_size + (base % page_size)) * hd;
        const int valid = pos - base + 1 < TILE ? pos - base + 1 : TILE;   // rows of the tile in use
        for (int i = threadIdx.x; i < TILE * hd; i += blockDim.x) {
            const int r = i / hd, c = i - r * hd;
            const bool live = r < valid;
            ks[r * (hd + 1) + c] = live ? to_f32<TC>(k_pool[src + i]) : 0.0f;
            vs[i] = live ? to_f32<TC>(v_pool[src + i]) : 0.0f;
        }
        __syncthreads();
        const int kpos = base + lane;
        const bool seen = kpos >= lo && kpos <= pos;
#pragma unroll
        for (int a = 0; a < MAX_HPW; ++a) {
            const int g = warp + a * WARPS;
            if (g >= group) break;
            const float* qh = qs + g * hd;
            const float* kr = ks + lane * (hd + 1);
            float s = 0.0f;
            for (int d = 0; d < hd; ++d) s = fmaf(qh[d], kr[d], s);
            s = seen ? s * scale : -INFINITY;
            const float tile_max = warp_max(s);
            if (tile_max == -INFINITY) continue;   // nothing visible in this tile (warp-uniform)
            const float m_new = fmaxf(m[a], tile_max);
            const float p = seen ? expf(s - m_new) : 0.0f;
            const float corr = expf(m[a] - m_new);  // m[a] == -inf gives 0
            l[a] = l[a] * corr + warp_sum(p);
            m[a] = m_new;
#pragma unroll
            for (int d = 0; d < MAX_DPL; ++d) acc[a][d] *= corr;
            for (int j = 0; j < valid; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
                for (int d = 0; d < MAX_DPL; ++d) {
                    const int c = lane + 32 * d;
                    if (c < hd) acc[a][d] = fmaf(pj, vs[j * hd + c], acc[a][d]);
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < MAX_HPW; ++a) {
        const int g = warp + a * WARPS;
        if (g >= group) break;
        const float inv = 1.0f / l[a];
        TO* dst = out + ((size_t)t * nh + (size_t)kvh * group + g) * hd;
#pragma unroll
        for (int d = 0; d < MAX_DPL; ++d) {
            const int c = lane + 32 * d;
            if (c < hd) dst[c] = from_f32<TO>(acc[a][d] * inv);
        }
    }
}

}  // namespace

// q, out: [T][nh*hd].  k_pool, v_pool: [pages][nkv][page_size][hd].  positions, tok_seg: [T].
// block_table: [S][max_pages].  The keys of every position <= a token's own must
// already be in the cache (this step's included).  Dtype flags: 0 fp32, 1 bf16.
FWB_API int fwb_attention_simt(const void* q, int q_bf16, const void* k_pool, const void* v_pool,
                               int cache_bf16, const int* positions, const int* tok_seg,
                               const int* block_table, int max_pages, int page_size, void* out,
                               int out_bf16, int T, int nh, int nkv, int hd, int window, float scale,
                               cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!q || !k_pool || !v_pool || !positions || !tok_seg || !block_table || !out)
        return FWB_BAD_ARGUMENT;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || max_pages <= 0) return FWB_BAD_ARGUMENT;
    if (page_size <= 0 || page_size % TILE != 0) return FWB_UNSUPPORTED;
    const int group = nh / nkv;
    if (group > WARPS * MAX_HPW || hd > 32 * MAX_DPL || nkv > 65535) return FWB_UNSUPPORTED;
    const size_t smem = ((size_t)group * hd + (size_t)TILE * (2 * hd + 1)) * sizeof(float);
    using bf = __nv_bfloat16;
    dim3 grid(T, nkv);
#define FWB_ATTN(TQ, TC, TO)                                                                      \
    do {                                                                                          \
        auto kernel = attention_simt_kernel<TQ, TC, TO>;                                          \
        if (smem > 48 * 1024) {                                                                   \
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                      \
            if (e != cudaSuccess) return (int)e;                                                  \
        }                                                                                         \
        fwb::pdl(kernel, grid, WARPS * 32, smem, stream)((const TQ*)q, (const TC*)k_pool,               \
                                                   (const TC*)v_pool, positions, tok_seg,         \
                                                   block_table, max_pages, page_size, (TO*)out,   \
                                                   nh, nkv, hd, window, scale);                   \
    } while (0)
    if (!q_bf16 && !cache_bf16 && !out_bf16) FWB_ATTN(float, float, float);
    else if (q_bf16 && cache_bf16 && out_bf16) FWB_ATTN(bf, bf, bf);
    else return FWB_UNSUPPORTED;
#undef FWB_ATTN
    return fwb_launch_status();
}
