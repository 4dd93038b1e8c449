// Gated short convolution over a ragged batch of segments, with the per-request
// rolling state read and advanced in the same launch.
//
//   p[t] = [ B | C | x ]  (3*H columns, produced by in_proj)
//   u    = B * x                                  (per token, per channel)
//   y[c] = bias[c] + sum_{k<L} taps[c][k] * u[j-(L-1)+k]     (j = index inside the segment;
//                                                  u at negative j comes from the state)
//   z    = C * y
//   state[slot][c][0..L-2] <- the last L-1 values of (state ++ u[0..n-1]), oldest first
//
// The filter is a FIR, so tokens are independent once the first L-1 of a segment have
// the state.  The launch has two kinds of blocks: "body" threads own one (token,
// channel) with j >= L-1 and never touch the state; "head" threads own one (segment,
// channel): they read the old state once, produce the first min(n, L-1) outputs and
// write the new state.  Nothing else reads or writes that state entry, so there is no
// ordering problem inside the launch, however the batch was cut.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int MAX_TAPS = 16;

template <typename TP, typename TZ>
__global__ void shortconv_kernel(const TP* __restrict__ p, const float* __restrict__ taps,
                                 const float* __restrict__ bias, float* __restrict__ state,
                                 const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                                 const int* __restrict__ tok_seg, TZ* __restrict__ z, int T, int S,
                                 int H, int L, int body_blocks, size_t slot_stride) {
    fwb::pdl_entry();
    const int ld = 3 * H;
    if ((int)blockIdx.x < body_blocks) {
        const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (idx >= (size_t)T * H) return;
        const int t = (int)(idx / H), c = (int)(idx - (size_t)t * H);
        const int j = t - seg_start[tok_seg[t]];
        if (j < L - 1) return;  // a head thread produces this one
        float y = bias ? bias[c] : 0.0f;
        for (int k = 0; k < L; ++k) {
            const TP* row = p + (size_t)(t - (L - 1) + k) * ld;
            y = fmaf(taps[c * L + k], to_f32<TP>(row[c]) * to_f32<TP>(row[2 * H + c]), y);
        }
        z[idx] = from_f32<TZ>(to_f32<TP>(p[(size_t)t * ld + H + c]) * y);
        return;
    }
    const size_t idx = (size_t)(blockIdx.x - body_blocks) * blockDim.x + threadIdx.x;
    if (idx >= (size_t)S * H) return;
    const int s = (int)(idx / H), c = (int)(idx - (size_t)s * H);
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    float* st = state + (size_t)seg_slot[s] * slot_stride + (size_t)c * (L - 1);
    // hist[0..L-2] = state (oldest first), hist[L-1..] = u of the first tokens.
    float hist[2 * MAX_TAPS];
    float w[MAX_TAPS];
    for (int k = 0; k < L; ++k) w[k] = taps[c * L + k];
    for (int k = 0; k < L - 1; ++k) hist[k] = st[k];
    const int first = n < L - 1 ? n : L - 1;
    for (int j = 0; j < first; ++j) {
        const TP* row = p + (size_t)(t0 + j) * ld;
        hist[L - 1 + j] = to_f32<TP>(row[c]) * to_f32<TP>(row[2 * H + c]);
        float y = bias ? bias[c] : 0.0f;
        for (int k = 0; k < L; ++k) y = fmaf(w[k], hist[j + k], y);
        z[(size_t)(t0 + j) * H + c] = from_f32<TZ>(to_f32<TP>(row[H + c]) * y);
    }
    if (n >= L - 1) {
        for (int k = 0; k < L - 1; ++k) {
            const TP* row = p + (size_t)(t0 + n - (L - 1) + k) * ld;
            st[k] = to_f32<TP>(row[c]) * to_f32<TP>(row[2 * H + c]);
        }
    } else {
        // shorter than the state: shift by n, the new values are hist[L-1 .. L-1+n)
        for (int k = 0; k < L - 1; ++k) st[k] = hist[k + n];
    }
}

// The bfloat16 form of the same launch with body threads that own 8 adjacent channels of one
// token: every load is one 16-byte vector, the B*x products of a tap are formed once per
// 8 outputs.  Head threads are the scalar ones above (there are S*H of them, few).
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// Head work of the bfloat16 launches: thread idx owns (segment, channel): the first L-1 outputs
// of the segment and the state.
__device__ __forceinline__ void conv_head_bf16(const __nv_bfloat16* __restrict__ p, const float* __restrict__ taps,
                                               const float* __restrict__ bias, float* __restrict__ state,
                                               const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                                               __nv_bfloat16* __restrict__ z, int S, int H, int L, size_t idx,
                                               size_t slot_stride) {
    const int ld = 3 * H;
    if (idx >= (size_t)S * H) return;
    const int s = (int)(idx / H), c = (int)(idx - (size_t)s * H);
    const int t0 = seg_start[s], n = seg_start[s + 1] - t0;
    float* st = state + (size_t)seg_slot[s] * slot_stride + (size_t)c * (L - 1);
    float hist[2 * MAX_TAPS];
    float w[MAX_TAPS];
    for (int k = 0; k < L; ++k) w[k] = taps[c * L + k];
    for (int k = 0; k < L - 1; ++k) hist[k] = st[k];
    const int first = n < L - 1 ? n : L - 1;
    for (int j = 0; j < first; ++j) {
        const __nv_bfloat16* row = p + (size_t)(t0 + j) * ld;
        hist[L - 1 + j] = __bfloat162float(row[c]) * __bfloat162float(row[2 * H + c]);
        float y = bias ? bias[c] : 0.0f;
        for (int k = 0; k < L; ++k) y = fmaf(w[k], hist[j + k], y);
        z[(size_t)(t0 + j) * H + c] = __float2bfloat16_rn(__bfloat162float(row[H + c]) * y);
    }
    if (n >= L - 1) {
        for (int k = 0; k < L - 1; ++k) {
            const __nv_bfloat16* row = p + (size_t)(t0 + n - (L - 1) + k) * ld;
            st[k] = __bfloat162float(row[c]) * __bfloat162float(row[2 * H + c]);
        }
    } else {
        for (int k = 0; k < L - 1; ++k) st[k] = hist[k + n];
    }
}

__global__ void shortconv_bf16x8_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ taps,
                                        const float* __restrict__ bias, float* __restrict__ state,
                                        const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                                        const int* __restrict__ tok_seg, __nv_bfloat16* __restrict__ z,
                                        int T, int S, int H, int L, int body_blocks, size_t slot_stride) {
    fwb::pdl_entry();
    const int ld = 3 * H;
    if ((int)blockIdx.x < body_blocks) {
        const int groups = H >> 3;
        const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (idx >= (size_t)T * groups) return;
        const int t = (int)(idx / groups), c = (int)(idx - (size_t)t * groups) * 8;
        const int j = t - seg_start[tok_seg[t]];
        if (j < L - 1) return;  // a head thread produces this one
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = bias ? bias[c + i] : 0.0f;
        for (int k = 0; k < L; ++k) {
            const __nv_bfloat16* row = p + (size_t)(t - (L - 1) + k) * ld;
            float b[8], x[8];
            unpack8(*reinterpret_cast<const uint4*>(row + c), b);
            unpack8(*reinterpret_cast<const uint4*>(row + 2 * H + c), x);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = fmaf(taps[(c + i) * L + k], b[i] * x[i], y[i]);
        }
        float g[8];
        unpack8(*reinterpret_cast<const uint4*>(p + (size_t)t * ld + H + c), g);
        uint4 out;
        __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(g[2 * i] * y[2 * i], g[2 * i + 1] * y[2 * i + 1]);
        *reinterpret_cast<uint4*>(z + (size_t)t * H + c) = out;
        return;
    }
    conv_head_bf16(p, taps, bias, state, seg_start, seg_slot, z, S, H, L,
                   (size_t)(blockIdx.x - body_blocks) * blockDim.x + threadIdx.x, slot_stride);
}

// Prompt-sized bfloat16 launches: a body thread owns 8 adjacent channels over a run of
// consecutive tokens and slides the window of B*x products through registers, so each row of p
// is loaded once per run instead of once per tap.  Products that precede the run are reloaded
// at its start; a run that crosses into another segment carries products of the previous
// segment only into outputs with j < L-1, which the head threads own.  The sum runs in the
// same order as everywhere else: bias, then taps oldest first.
template <int L, int RUN>
__global__ void __launch_bounds__(128)
shortconv_bf16_run_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ taps,
                          const float* __restrict__ bias, float* __restrict__ state,
                          const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                          const int* __restrict__ tok_seg, __nv_bfloat16* __restrict__ z, int T, int S,
                          int H, int body_blocks, size_t slot_stride) {
    fwb::pdl_entry();
    const int ld = 3 * H;
    if ((int)blockIdx.x < body_blocks) {
        const int groups = H >> 3;
        constexpr int run = RUN;
        const int runs = (T + run - 1) / run;
        const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        if (idx >= (size_t)runs * groups) return;
        const int r = (int)(idx / groups), c = (int)(idx - (size_t)r * groups) * 8;
        const int t0 = r * run, t1 = min(T, t0 + run);
        float w[L][8], b0[8], hist[L - 1][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            b0[i] = bias ? bias[c + i] : 0.0f;
#pragma unroll
            for (int k = 0; k < L; ++k) w[k][i] = taps[(c + i) * L + k];
        }
#pragma unroll
        for (int k = 0; k < L - 1; ++k) {
            const int t = t0 - (L - 1) + k;
            if (t >= 0) {
                const __nv_bfloat16* row = p + (size_t)t * ld;
                float b[8], x[8];
                unpack8(*reinterpret_cast<const uint4*>(row + c), b);
                unpack8(*reinterpret_cast<const uint4*>(row + 2 * H + c), x);
#pragma unroll
                for (int i = 0; i < 8; ++i) hist[k][i] = b[i] * x[i];
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) hist[k][i] = 0.0f;
            }
        }
        // every load of the run goes out before the first product is formed
        uint4 vb[RUN], vx[RUN], vc[RUN];
        int first[RUN];
#pragma unroll
        for (int i = 0; i < RUN; ++i) {
            const int t = t0 + i < T ? t0 + i : T - 1;
            const __nv_bfloat16* row = p + (size_t)t * ld;
            vb[i] = *reinterpret_cast<const uint4*>(row + c);
            vx[i] = *reinterpret_cast<const uint4*>(row + 2 * H + c);
            vc[i] = *reinterpret_cast<const uint4*>(row + H + c);
            first[i] = seg_start[tok_seg[t]];
        }
#pragma unroll
        for (int i = 0; i < RUN; ++i) {
            const int t = t0 + i;
            if (t >= t1) break;
            float b[8], x[8], u[8];
            unpack8(vb[i], b);
            unpack8(vx[i], x);
#pragma unroll
            for (int k = 0; k < 8; ++k) u[k] = b[k] * x[k];
            if (t - first[i] >= L - 1) {
                float g[8], y[8];
                unpack8(vc[i], g);
#pragma unroll
                for (int k8 = 0; k8 < 8; ++k8) {
                    y[k8] = b0[k8];
#pragma unroll
                    for (int k = 0; k < L - 1; ++k) y[k8] = fmaf(w[k][k8], hist[k][k8], y[k8]);
                    y[k8] = fmaf(w[L - 1][k8], u[k8], y[k8]);
                }
                uint4 out;
                __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    o[k] = __floats2bfloat162_rn(g[2 * k] * y[2 * k], g[2 * k + 1] * y[2 * k + 1]);
                *reinterpret_cast<uint4*>(z + (size_t)t * H + c) = out;
            }
#pragma unroll
            for (int k8 = 0; k8 < 8; ++k8) {
#pragma unroll
                for (int k = 0; k + 1 < L - 1; ++k) hist[k][k8] = hist[k + 1][k8];
                hist[L - 2][k8] = u[k8];
            }
        }
        return;
    }
    conv_head_bf16(p, taps, bias, state, seg_start, seg_slot, z, S, H, L,
                   (size_t)(blockIdx.x - body_blocks) * blockDim.x + threadIdx.x, slot_stride);
}

}  // namespace

// p: [T][3H] (fp32 or bf16); taps: [H][L] fp32; bias: [H] fp32 or null;
// state: fp32 [H][L-1] per slot, slots `state_slot_stride` floats apart; seg_start: [S+1]; seg_slot: [S]; tok_seg: [T];
// z: [T][H] (fp32 or bf16).
FWB_API int fwb_shortconv(const void* p, int p_bf16, const float* taps, const float* bias,
                          float* state, const int* seg_start, const int* seg_slot,
                          const int* tok_seg, void* z, int z_bf16, int T, int S, int H, int L,
                          long long state_slot_stride, cudaStream_t stream) {
    if (T <= 0 || S <= 0) return FWB_OK;
    if (!p || !taps || !state || !seg_start || !seg_slot || !tok_seg || !z || H <= 0)
        return FWB_BAD_ARGUMENT;
    if (L < 2 || L > MAX_TAPS) return FWB_UNSUPPORTED;
    if (state_slot_stride < (long long)H * (L - 1)) return FWB_BAD_ARGUMENT;
    const size_t slot_stride = (size_t)state_slot_stride;
    const int threads = 128;
    if (p_bf16 && z_bf16 && (H & 7) == 0 && ((uintptr_t)p & 15) == 0 && ((uintptr_t)z & 15) == 0) {
        const int head = (int)(((size_t)S * H + threads - 1) / threads);
        if (T >= 256 && L >= 2 && L <= 4) {
            constexpr int run = 4;
            const int body = (int)(((size_t)((T + run - 1) / run) * (H >> 3) + threads - 1) / threads);
#define FWB_CONV_RUN(LL)                                                                          \
    fwb::pdl(shortconv_bf16_run_kernel<LL, run>, body + head, threads, 0, stream)(                \
        (const __nv_bfloat16*)p, taps, bias, state, seg_start, seg_slot, tok_seg, (__nv_bfloat16*)z, T, S, \
        H, body, slot_stride)
            if (L == 2) FWB_CONV_RUN(2);
            else if (L == 3) FWB_CONV_RUN(3);
            else FWB_CONV_RUN(4);
#undef FWB_CONV_RUN
            return fwb_launch_status();
        }
        const int body = (int)(((size_t)T * (H >> 3) + threads - 1) / threads);
        fwb::pdl(shortconv_bf16x8_kernel, body + head, threads, 0, stream)(
            (const __nv_bfloat16*)p, taps, bias, state, seg_start, seg_slot, tok_seg, (__nv_bfloat16*)z, T, S,
            H, L, body, slot_stride);
        return fwb_launch_status();
    }
    const int body_blocks = (int)(((size_t)T * H + threads - 1) / threads);
    const int head_blocks = (int)(((size_t)S * H + threads - 1) / threads);
    const int blocks = body_blocks + head_blocks;
    using bf = __nv_bfloat16;
#define FWB_CONV(TP, TZ)                                                                          \
    fwb::pdl(shortconv_kernel<TP, TZ>, blocks, threads, 0, stream)(                                     \
        (const TP*)p, taps, bias, state, seg_start, seg_slot, tok_seg, (TZ*)z, T, S, H, L,        \
        body_blocks, slot_stride)
    if (p_bf16 && z_bf16) FWB_CONV(bf, bf);
    else if (!p_bf16 && z_bf16) FWB_CONV(float, bf);
    else if (!p_bf16 && !z_bf16) FWB_CONV(float, float);
    else return FWB_UNSUPPORTED;
#undef FWB_CONV
    return fwb_launch_status();
}
