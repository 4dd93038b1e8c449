// Y[M][N] = X[M][K] * W[N][K]^T (+ addend), plain SIMT with fp32 FMA accumulation.
//
// This is the true 32-bit matrix product of the engine (no tensor-core mode of any
// kind), and the fallback of the bfloat16 path for shapes the tensor-core kernel
// refuses.  Any M, N, K >= 1.  Each output element is one accumulator that walks
// k = 0..K-1 in ascending order, so the value at [m][n] does not depend on M or on
// which other rows share the launch.
#include "common.cuh"

using namespace fwb;

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ X, const TW* __restrict__ W, TY* __restrict__ Y,
                 const float* __restrict__ addend, int M, int N, int K, int ldx, int ldy) {
    fwb::pdl_entry();
    __shared__ float xs[TK][TM + 4];
    __shared__ float ws[TK][TN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    const int lrow = tid / 4, lk = (tid % 4) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int m = m0 + lrow, n = n0 + lrow;
            xs[lk + j][lrow] = (m < M && k < K) ? to_f32<TX>(X[(size_t)m * ldx + k]) : 0.0f;
            ws[lk + j][lrow] = (n < N && k < K) ? to_f32<TW>(W[(size_t)n * K + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][tm + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tn + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (addend) v += addend[(size_t)m * ldy + n];
            Y[(size_t)m * ldy + n] = from_f32<TY>(v);
        }
    }
}

template <typename TX, typename TW, typename TY>
int launch(const void* X, const void* W, void* Y, const float* addend, int M, int N, int K, int ldx,
           int ldy, cudaStream_t stream) {
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    if (grid.y > 65535) return FWB_TOO_LARGE;
    fwb::pdl(gemm_simt_kernel<TX, TW, TY>, grid, 256, 0, stream)((const TX*)X, (const TW*)W, (TY*)Y,
                                                           addend, M, N, K, ldx, ldy);
    return fwb_launch_status();
}

}  // namespace

// Dtype flags: 0 = float32, 1 = bfloat16.  `addend` (fp32, same layout as a fp32 Y,
// may alias Y) is added before the store; it needs y_bf16 == 0.
FWB_API int fwb_gemm_simt(const void* X, int x_bf16, const void* W, int w_bf16, void* Y, int y_bf16,
                          const float* addend, int M, int N, int K, int ldx, int ldy,
                          cudaStream_t stream) {
    if (M <= 0 || N <= 0) return FWB_OK;
    if (!X || !W || !Y || K <= 0 || ldx < K || ldy < N) return FWB_BAD_ARGUMENT;
    if (addend && y_bf16) return FWB_UNSUPPORTED;
    using bf = __nv_bfloat16;
    const int key = (x_bf16 ? 4 : 0) | (w_bf16 ? 2 : 0) | (y_bf16 ? 1 : 0);
    switch (key) {
        case 0: return launch<float, float, float>(X, W, Y, addend, M, N, K, ldx, ldy, stream);
        case 2: return launch<float, bf, float>(X, W, Y, addend, M, N, K, ldx, ldy, stream);
        case 4: return launch<bf, float, float>(X, W, Y, addend, M, N, K, ldx, ldy, stream);
        case 6: return launch<bf, bf, float>(X, W, Y, addend, M, N, K, ldx, ldy, stream);
        case 7: return launch<bf, bf, bf>(X, W, Y, addend, M, N, K, ldx, ldy, stream);
        case 5: return launch<bf, float, bf>(X, W, Y, addend, M, N, K, ldx, ldy, stream);
        default: return FWB_UNSUPPORTED;
    }
}
