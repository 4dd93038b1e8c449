// One head's share of the fused q/k norm + rotation, for kernels in which hd/8 adjacent lanes own a
// head and every lane eight contiguous channels of it (bfloat16 in, fp32 arithmetic).  Shared by the
// kernel that transforms a whole step's q|k|v rows and by the decode attention kernel, which does the
// same to its own token's heads in its prologue: one function, so both give the same bits.
#pragma once
#include "common.cuh"

namespace fwb {

__device__ __forceinline__ void load8(const __nv_bfloat16* src, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(src);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ void store8(__nv_bfloat16* dst, const float (&f)[8]) {
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(dst) = out;
}

// v: the lane's eight channels (zeros where !valid), transformed in place.  kind: 0 query, 1 key,
// 2 value (left as it is).  The warp's lanes sub*G .. sub*G + G-1 hold one head (gl = lane - sub*G);
// every lane of the warp must call this (shuffles with the full mask).  The sum of squares goes over
// the lanes of the head in lane order; the rotation partner (i +- rot/2) sits rot/16 lanes away.
// cs: the (cos, sin) pairs of the token's position.  Needs rot % 16 == 0.
__device__ __forceinline__ void head_norm_rope8(float (&v)[8], bool valid, int kind, int sub, int gl, int G, int hd,
                                                int rot, int pairing, int use_norm, float eps,
                                                const float* __restrict__ wq, const float* __restrict__ wk,
                                                const float2* __restrict__ cs) {
    const int lane = threadIdx.x & 31;
    const int half_lanes = rot >> 4, rot_lanes = rot >> 3;
    const int partner = gl < half_lanes ? lane + half_lanes : (gl < rot_lanes ? lane - half_lanes : lane);
    const bool is_v = kind == 2, is_q = kind == 0;
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    float total = 0.0f;
    for (int j = 0; j < G; ++j) total += __shfl_sync(0xffffffffu, ss, (sub * G + j) & 31);
    if (use_norm && !is_v) {
        const float inv = rsqrtf(total / (float)hd + eps);
        const float* w = (is_q ? wq : wk) + gl * 8;
        if (valid) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (v[i] * inv) * w[i];
        }
    }
    float other[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) other[i] = __shfl_sync(0xffffffffu, v[i], partner);
    if (!valid) return;
    if (!is_v && gl < rot_lanes && pairing) {
        // interleaved pairs lie side by side in this lane's eight channels
        const float2* c = cs + gl * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 a = c[j];
            const float x0 = v[2 * j], x1 = v[2 * j + 1];
            v[2 * j] = x0 * a.x - x1 * a.y;
            v[2 * j + 1] = x1 * a.x + x0 * a.y;
        }
    } else if (!is_v && gl < rot_lanes) {
        const bool low = gl < half_lanes;
        const float2* c = cs + (low ? gl : gl - half_lanes) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 a = c[i];
            v[i] = low ? v[i] * a.x - other[i] * a.y : v[i] * a.x + other[i] * a.y;
        }
    }
}

}  // namespace fwb
