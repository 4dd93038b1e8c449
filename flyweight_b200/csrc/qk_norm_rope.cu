// Per-head RMSNorm of q and k, rotary position encoding from a table, and the write
// of k and v into the paged cache, in one pass over the fused q|k|v projection.
//
//   qkv[t] = [ q: nh*hd | k: nkv*hd | v: nkv*hd ]
//   q^ = rope(rmsnorm_hd(q_head) * wq),  k^ = rope(rmsnorm_hd(k_head) * wk),  v unchanged
//   rope over the first `rot` channels of a head, pair i of rot/2 turning by table[pos][i]:
//       a' = a*cos - b*sin,  b' = b*cos + a*sin
//   with (a, b) = channels (i, i+rot/2) for half-split pairing (0), (2i, 2i+1) for interleaved (1)
//   K[page][kvh][off][:] = k^,  V[page][kvh][off][:] = v   with page = block_table[seg][pos/P],
//                                                          off = pos % P
// Norm, angle lookup and rotation are fp32; only the stores round to the cache type.
// With nkv_in == 0 the launch handles queries only (a layer that reads another
// layer's cache writes none of its own).
#include "common.cuh"
#include "qk_head.cuh"

using namespace fwb;

namespace {

constexpr int MAX_HD = 512;
constexpr int WARPS = 4;

template <typename TI, typename TQ, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_kernel(const TI* __restrict__ qkv, const float* __restrict__ wq,
                    const float* __restrict__ wk, const float2* __restrict__ table,
                    const int* __restrict__ positions, const int* __restrict__ tok_seg,
                    const int* __restrict__ block_table, int max_pages, int page_size,
                    TQ* __restrict__ q_out, TC* __restrict__ k_pool, TC* __restrict__ v_pool, int nh,
                    int nkv, int hd, int rot, float eps, int use_norm, int pairing) {
    fwb::pdl_entry();
    extern __shared__ float smem[];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* buf = smem + warp * hd;
    const int pos = positions[t];
    const int row_width = (nh + 2 * nkv) * hd;
    const TI* row = qkv + (size_t)t * row_width;
    const float2* cs = table + (size_t)pos * (rot / 2);
    size_t cache_base = 0;
    if (nkv > 0) {
        const int page = block_table[(size_t)tok_seg[t] * max_pages + pos / page_size];
        cache_base = ((size_t)page * nkv) * page_size * hd + (size_t)(pos % page_size) * hd;
    }
    const int heads = nh + 2 * nkv;
    for (int h = blockIdx.y * WARPS + warp; h < heads; h += gridDim.y * WARPS) {
        const TI* src = row + (size_t)h * hd;
        if (h >= nh + nkv) {  // v: copy
            const int kvh = h - nh - nkv;
            TC* dst = v_pool + cache_base + (size_t)kvh * page_size * hd;
            for (int i = lane; i < hd; i += 32) dst[i] = from_f32<TC>(to_f32<TI>(src[i]));
            continue;
        }
        const bool is_q = h < nh;
        const float* w = is_q ? wq : wk;
        float ss = 0.0f;
        for (int i = lane; i < hd; i += 32) {
            const float v = to_f32<TI>(src[i]);
            buf[i] = v;
            ss += v * v;
        }
        ss = warp_sum(ss);
        const float inv = use_norm ? rsqrtf(ss / (float)hd + eps) : 1.0f;
        __syncwarp();
        const int half = rot / 2;
        if (is_q) {
            TQ* dst = q_out + ((size_t)t * nh + h) * hd;
            for (int i = lane; i < half; i += 32) {
                const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
                const float a = use_norm ? (buf[ia] * inv) * w[ia] : buf[ia];
                const float b = use_norm ? (buf[ib] * inv) * w[ib] : buf[ib];
                const float2 c = cs[i];
                dst[ia] = from_f32<TQ>(a * c.x - b * c.y);
                dst[ib] = from_f32<TQ>(b * c.x + a * c.y);
            }
            for (int i = rot + lane; i < hd; i += 32)
                dst[i] = from_f32<TQ>(use_norm ? (buf[i] * inv) * w[i] : buf[i]);
        } else {
            TC* dst = k_pool + cache_base + (size_t)(h - nh) * page_size * hd;
            for (int i = lane; i < half; i += 32) {
                const int ia = pairing ? 2 * i : i, ib = pairing ? 2 * i + 1 : i + half;
                const float a = use_norm ? (buf[ia] * inv) * w[ia] : buf[ia];
                const float b = use_norm ? (buf[ib] * inv) * w[ib] : buf[ib];
                const float2 c = cs[i];
                dst[ia] = from_f32<TC>(a * c.x - b * c.y);
                dst[ib] = from_f32<TC>(b * c.x + a * c.y);
            }
            for (int i = rot + lane; i < hd; i += 32)
                dst[i] = from_f32<TC>(use_norm ? (buf[i] * inv) * w[i] : buf[i]);
        }
        __syncwarp();
    }
}

// All-bfloat16 form: hd/8 adjacent lanes own one head, 8 contiguous channels each (one 16-byte
// load and store per lane), so a warp works on 32/(hd/8) heads at a time.  The sum of squares
// goes over the lanes of a head in lane order; the rotation partner (i +- rot/2) sits
// rot/16 lanes away and is fetched with shuffles.  Needs hd % 8 == 0, hd <= 256, rot % 16 == 0.
__global__ void __launch_bounds__(WARPS * 32)
qk_norm_rope_bf16x8_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ wq,
                           const float* __restrict__ wk, const float2* __restrict__ table,
                           const int* __restrict__ positions, const int* __restrict__ tok_seg,
                           const int* __restrict__ block_table, int max_pages, int page_size,
                           __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_pool,
                           __nv_bfloat16* __restrict__ v_pool, int nh, int nkv, int hd, int rot, float eps,
                           int use_norm, int pairing) {
    fwb::pdl_entry();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = hd >> 3, per_warp = 32 / G;
    const int sub = lane / G, gl = lane - sub * G;
    const int pos = positions[t];
    const int heads = nh + 2 * nkv;
    const __nv_bfloat16* row = qkv + (size_t)t * heads * hd;
    const float2* cs = table + (size_t)pos * (rot / 2);
    size_t cache_base = 0;
    if (nkv > 0) {
        const int page = block_table[(size_t)tok_seg[t] * max_pages + pos / page_size];
        cache_base = ((size_t)page * nkv) * page_size * hd + (size_t)(pos % page_size) * hd;
    }
    const int block_warps = blockDim.x >> 5;
    for (int h0 = (blockIdx.y * block_warps + warp) * per_warp; h0 < heads; h0 += gridDim.y * block_warps * per_warp) {
        const int h = h0 + sub;
        const bool valid = sub < per_warp && h < heads;
        float v[8];
        if (valid) {
            load8(row + (size_t)h * hd + gl * 8, v);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        const bool is_v = h >= nh + nkv, is_q = h < nh;
        head_norm_rope8(v, valid, is_q ? 0 : (is_v ? 2 : 1), sub, gl, G, hd, rot, pairing, use_norm, eps, wq, wk, cs);
        if (!valid) continue;
        __nv_bfloat16* dst;
        if (is_q) dst = q_out + ((size_t)t * nh + h) * hd;
        else if (!is_v) dst = k_pool + cache_base + (size_t)(h - nh) * page_size * hd;
        else dst = v_pool + cache_base + (size_t)(h - nh - nkv) * page_size * hd;
        store8(dst + gl * 8, v);
    }
}

}  // namespace

// qkv: [T][(nh+2*nkv)*hd] fp32 or bf16.  wq, wk: [hd] fp32 (ignored when use_norm == 0).
// table: [max_pos][rot/2] float2 (cos, sin).  positions, tok_seg: [T].
// pairing: 0 half-split (i, i+rot/2), 1 interleaved (2i, 2i+1).
// block_table: [S][max_pages] page ids.  q_out: [T][nh*hd].  k_pool, v_pool:
// [pages][nkv][page_size][hd].  Dtype flags: 0 fp32, 1 bf16.
FWB_API int fwb_qk_norm_rope(const void* qkv, int in_bf16, const float* wq, const float* wk,
                             const void* table, const int* positions, const int* tok_seg,
                             const int* block_table, int max_pages, int page_size, void* q_out,
                             int q_bf16, void* k_pool, void* v_pool, int cache_bf16, int T, int nh,
                             int nkv, int hd, int rot, float eps, int use_norm, int pairing,
                             cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!qkv || !table || !positions || !q_out || nh <= 0 || nkv < 0) return FWB_BAD_ARGUMENT;
    if (nkv > 0 && (!tok_seg || !block_table || !k_pool || !v_pool || page_size <= 0 || max_pages <= 0))
        return FWB_BAD_ARGUMENT;
    if (use_norm && (!wq || (nkv > 0 && !wk))) return FWB_BAD_ARGUMENT;
    if (hd <= 0 || hd > MAX_HD || (hd & 1) || rot < 0 || rot > hd || (rot & 1)) return FWB_UNSUPPORTED;
    if (pairing != 0 && pairing != 1) return FWB_UNSUPPORTED;
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    // one warp per head; few tokens (decode) spread their heads over several blocks
    const int head_blocks = T >= 256 ? 1 : (nh + 2 * nkv + WARPS - 1) / WARPS;
    if (T > 2147483647 / 1 || head_blocks > 65535) return FWB_TOO_LARGE;
    const dim3 grid(T, head_blocks);
    using bf = __nv_bfloat16;
#define FWB_QK(TI, TQ, TC)                                                                        \
    fwb::pdl(qk_norm_rope_kernel<TI, TQ, TC>, grid, WARPS * 32, smem, stream)(                             \
        (const TI*)qkv, wq, wk, (const float2*)table, positions, tok_seg, block_table, max_pages, \
        page_size, (TQ*)q_out, (TC*)k_pool, (TC*)v_pool, nh, nkv, hd, rot, eps, use_norm, pairing)
    const int key = (in_bf16 ? 4 : 0) | (q_bf16 ? 2 : 0) | (cache_bf16 ? 1 : 0);
    const bool aligned = (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0;
    if (key == 7 && (hd & 7) == 0 && hd <= 256 && (rot & 15) == 0 && aligned) {
        const int per_block = WARPS * (32 / (hd >> 3));
        const dim3 vgrid(T, T >= 256 ? 1 : (nh + 2 * nkv + per_block - 1) / per_block);
        fwb::pdl(qk_norm_rope_bf16x8_kernel, vgrid, WARPS * 32, 0, stream)(
            (const __nv_bfloat16*)qkv, wq, wk, (const float2*)table, positions, tok_seg, block_table,
            max_pages, page_size, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, nh,
            nkv, hd, rot, eps, use_norm, pairing);
        return fwb_launch_status();
    }
    switch (key) {
        case 0: FWB_QK(float, float, float); break;
        case 3: FWB_QK(float, bf, bf); break;
        case 7: FWB_QK(bf, bf, bf); break;
        default: return FWB_UNSUPPORTED;
    }
#undef FWB_QK
    return fwb_launch_status();
}
