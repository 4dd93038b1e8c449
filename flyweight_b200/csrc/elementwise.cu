// Embedding gather, RMSNorm (with the residual sum folded in), SiLU-gate product
// and dtype casts.  All arithmetic is fp32; T only names the storage type.
#include "common.cuh"

using namespace fwb;

// ------------------------------------------------------------------ embedding
// out[t][:] = scale * table[ids[t]][:] widened to fp32 (scale 1: the row as it is; some
// architectures multiply the embedding by sqrt(H)).  An id outside [0, V) writes
// zeros and raises *bad (the host refuses such ids before upload; this is the
// second fence).
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ out, int T, int H, int V, int* bad, float scale) {
    fwb::pdl_entry();
    const int t = blockIdx.y;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0 && blockIdx.x == 0 && bad) atomicExch(bad, 1);
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < H; c += gridDim.x * blockDim.x)
        out[(size_t)t * H + c] = ok ? scale * to_f32<TW>(table[(size_t)id * H + c]) : 0.0f;
}

// bfloat16 table, H a multiple of 8: a thread widens 8 adjacent entries (one 16-byte load, two
// 16-byte stores); one block per token.
__global__ void embed_bf16x8_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V, int* bad, float scale) {
    fwb::pdl_entry();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0 && bad) atomicExch(bad, 1);
    const __nv_bfloat16* row = table + (size_t)(ok ? id : 0) * H;
    float* dst = out + (size_t)t * H;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        float4 lo = make_float4(0, 0, 0, 0), hi = lo;
        if (ok) {
            const uint4 v = *reinterpret_cast<const uint4*>(row + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
            const float2 e = __bfloat1622float2(h[2]), f = __bfloat1622float2(h[3]);
            lo = make_float4(scale * a.x, scale * a.y, scale * b.x, scale * b.y);
            hi = make_float4(scale * e.x, scale * e.y, scale * f.x, scale * f.y);
        }
        *reinterpret_cast<float4*>(dst + c) = lo;
        *reinterpret_cast<float4*>(dst + c + 4) = hi;
    }
}

FWB_API int fwb_embed(const void* table, int table_bf16, const int* ids, float* out, int T, int H,
                      int V, int* bad, float scale, cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!table || !ids || !out || H <= 0 || V <= 0 || T > 65535) return FWB_BAD_ARGUMENT;
    if (table_bf16 && (H & 7) == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
        const int threads = H / 8 < 256 ? ((H / 8 + 31) / 32) * 32 : 256;
        fwb::pdl(embed_bf16x8_kernel, T, threads, 0, stream)((const __nv_bfloat16*)table, ids, out, H, V, bad, scale);
        return fwb_launch_status();
    }
    dim3 grid((H + 255) / 256 > 64 ? 64 : (H + 255) / 256, T);
    if (table_bf16)
        fwb::pdl(embed_kernel<__nv_bfloat16>, grid, 256, 0, stream)(
            (const __nv_bfloat16*)table, ids, out, T, H, V, bad, scale);
    else
        fwb::pdl(embed_kernel<float>, grid, 256, 0, stream)((const float*)table, ids, out, T, H, V, bad, scale);
    return fwb_launch_status();
}

// ------------------------------------------------------------------ RMSNorm
// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] + delta[s]     (the residual sum, fp32; without `rows` it is stored back to x)
//   out[r] = (v * rsqrt(mean(v^2) + eps)) * w
// With `rows` the launch gathers: x is left as it is (a row may be asked for twice).
// One block per row; the sum of squares is reduced in an order fixed by the block
// size, so a row's result does not depend on which other rows are in the batch.
template <typename TO>
__global__ void rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                               const float* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int H, float eps) {
    fwb::pdl_entry();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + s * H;
    const float* dr = delta ? delta + s * H : nullptr;
    const bool store = dr && !rows;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (dr) v += dr[c];
        if (store) xr[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)r * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = xr[c];
        if (dr && !store) v += dr[c];
        orow[c] = from_f32<TO>((v * inv) * w[c]);
    }
}

// The same operation for rows that fit the registers of one block (H a multiple of 4, at most
// VEC float4 per thread): every load of the row is in flight at once and the row is read once.
template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ w,
                   TO* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    fwb::pdl_launch_dependents();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int n4 = H >> 2;
    float4 wv[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {           // the weight is nobody's output: load it early
        const int c = threadIdx.x + i * 256;
        wv[i] = c < n4 ? reinterpret_cast<const float4*>(w)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    fwb::pdl_wait();
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float4* xr = reinterpret_cast<float4*>(x + s * H);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + s * H) : nullptr;
    const bool store = dr && !rows;
    float4 v[VEC];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = threadIdx.x + i * 256;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (dr) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const int c = threadIdx.x + i * 256;
            if (c < n4) {
                const float4 d = dr[c];
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                if (store) xr[c] = v[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    ss = block_sum(ss, scratch);
    const float inv = rsqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)r * H;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int c = threadIdx.x + i * 256;
        if (c >= n4) continue;
        const float a = (v[i].x * inv) * wv[i].x, b = (v[i].y * inv) * wv[i].y;
        const float cc = (v[i].z * inv) * wv[i].z, d = (v[i].w * inv) * wv[i].w;
        if (sizeof(TO) == 4) {
            reinterpret_cast<float4*>(orow)[c] = make_float4(a, b, cc, d);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(orow)[c] = packed;
        }
    }
}

FWB_API int fwb_rmsnorm(float* x, const float* delta, const float* w, void* out, int out_bf16,
                        const int* rows, int R, int H, float eps, cudaStream_t stream) {
    if (R <= 0) return FWB_OK;
    if (!x || !w || !out || H <= 0) return FWB_BAD_ARGUMENT;
    const bool aligned = ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
                         (!delta || ((uintptr_t)delta & 15) == 0);
    if ((H & 3) == 0 && H >= 512 && H <= 4 * 256 * 4 && aligned) {
        using bf = __nv_bfloat16;
        const int vec = (H / 4 + 255) / 256;
#define FWB_NORM(V)                                                                                     \
    if (out_bf16) fwb::pdl(rmsnorm_vec_kernel<bf, V>, R, 256, 0, stream)(x, delta, w, (bf*)out, rows, H, eps); \
    else fwb::pdl(rmsnorm_vec_kernel<float, V>, R, 256, 0, stream)(x, delta, w, (float*)out, rows, H, eps)
        if (vec == 1) { FWB_NORM(1); } else if (vec == 2) { FWB_NORM(2); } else if (vec == 3) { FWB_NORM(3); } else { FWB_NORM(4); }
#undef FWB_NORM
        return fwb_launch_status();
    }
    const int threads = H >= 1024 ? 256 : (H >= 256 ? 128 : 64);
    if (out_bf16)
        fwb::pdl(rmsnorm_kernel<__nv_bfloat16>, R, threads, 0, stream)(x, delta, w, (__nv_bfloat16*)out,
                                                                rows, H, eps);
    else
        fwb::pdl(rmsnorm_kernel<float>, R, threads, 0, stream)(x, delta, w, (float*)out, rows, H, eps);
    return fwb_launch_status();
}

// x += delta (fp32), for a residual that no norm follows.
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ delta, size_t n) {
    fwb::pdl_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        x[i] += delta[i];
}

FWB_API int fwb_add(float* x, const float* delta, long long n, cudaStream_t stream) {
    if (n <= 0) return FWB_OK;
    if (!x || !delta) return FWB_BAD_ARGUMENT;
    const int blocks = (int)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256);
    fwb::pdl(add_kernel, blocks, 256, 0, stream)(x, delta, (size_t)n);
    return fwb_launch_status();
}

// ------------------------------------------------------------------ SiLU gate
// gu is [T][2F] with the gate in columns [0,F) and the up projection in [F,2F);
// out[t][f] = silu(gate) * up.
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, TO* __restrict__ out, int T, int F) {
    fwb::pdl_entry();
    const size_t n = (size_t)T * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / F, f = i - t * F;
        const float g = to_f32<TI>(gu[t * 2 * F + f]);
        const float u = to_f32<TI>(gu[t * 2 * F + F + f]);
        out[i] = from_f32<TO>(silu_f32(g) * u);
    }
}

FWB_API int fwb_silu_mul(const void* gu, int in_bf16, void* out, int out_bf16, int T, int F,
                         cudaStream_t stream) {
    if (T <= 0) return FWB_OK;
    if (!gu || !out || F <= 0) return FWB_BAD_ARGUMENT;
    const size_t n = (size_t)T * F;
    const int blocks = (int)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256);
    if (in_bf16 && out_bf16)
        fwb::pdl(silu_mul_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream)(
            (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F);
    else if (!in_bf16 && out_bf16)
        fwb::pdl(silu_mul_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream)(
            (const float*)gu, (__nv_bfloat16*)out, T, F);
    else if (!in_bf16 && !out_bf16)
        fwb::pdl(silu_mul_kernel<float, float>, blocks, 256, 0, stream)((const float*)gu, (float*)out, T, F);
    else
        return FWB_UNSUPPORTED;
    return fwb_launch_status();
}

// ------------------------------------------------------------------ casts
template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
    fwb::pdl_entry();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<TO>(to_f32<TI>(in[i]));
}

FWB_API int fwb_cast(const void* in, int in_bf16, void* out, int out_bf16, long long n,
                     cudaStream_t stream) {
    if (n <= 0) return FWB_OK;
    if (!in || !out || in_bf16 == out_bf16) return FWB_BAD_ARGUMENT;
    const int blocks = (int)((n + 255) / 256 > 8192 ? 8192 : (n + 255) / 256);
    if (in_bf16)
        fwb::pdl(cast_kernel<__nv_bfloat16, float>, blocks, 256, 0, stream)((const __nv_bfloat16*)in,
                                                                       (float*)out, (size_t)n);
    else
        fwb::pdl(cast_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream)((const float*)in,
                                                                       (__nv_bfloat16*)out, (size_t)n);
    return fwb_launch_status();
}

// ------------------------------------------------------------------ logit soft-cap
// x = cap * tanh(x / cap), in place on fp32 (a head whose logits are squashed into (-cap, cap)).
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
    fwb::pdl_entry();
    const float inv = 1.0f / cap;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] * inv);
}

FWB_API int fwb_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n <= 0) return FWB_OK;
    if (!x || !(cap > 0.0f)) return FWB_BAD_ARGUMENT;
    const long long blocks = (n + 255) / 256;
    fwb::pdl(softcap_kernel, (int)(blocks > 4096 ? 4096 : blocks), 256, 0, stream)(x, n, cap);
    return fwb_launch_status();
}

// ------------------------------------------------------------------ token ids that were still on the device
// token_ids[dst[i]] = source[src[i]]: a step that was planned before the step in front of it was
// read gets the ids that step sampled straight from the sampler's output.
__global__ void patch_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ dst,
                                    const int* __restrict__ source, const int* __restrict__ src, int n) {
    fwb::pdl_entry();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) token_ids[dst[i]] = source[src[i]];
}

FWB_API int fwb_patch_tokens(int* token_ids, const int* dst, const int* source, const int* src, int n,
                             cudaStream_t stream) {
    if (n <= 0) return FWB_OK;
    if (!token_ids || !dst || !source || !src) return FWB_BAD_ARGUMENT;
    fwb::pdl(patch_tokens_kernel, (n + 127) / 128, 128, 0, stream)(token_ids, dst, source, src, n);
    return fwb_launch_status();
}
