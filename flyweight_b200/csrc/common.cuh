// Shared device helpers for the flyweight_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FWB_API extern "C" __attribute__((visibility("default")))

// Status codes returned by every host launcher.  0 = launched; a positive value
// is a cudaError_t from the launch; negative values are refusals made on the
// host before anything ran.
enum FwbStatus : int {
    FWB_OK = 0,
    FWB_BAD_ARGUMENT = -1,     // a size, stride or pointer the kernel cannot take
    FWB_UNSUPPORTED = -2,      // a combination the kernel was not written for
    FWB_TOO_LARGE = -3,        // beyond a stated maximum
};

static inline int fwb_launch_status() {
    cudaError_t err = cudaPeekAtLastError();
    return err == cudaSuccess ? FWB_OK : static_cast<int>(err);
}

namespace fwb {

// ---- programmatic dependent launch ------------------------------------------------
// Every kernel of the library is launched with programmatic stream serialisation: the next
// kernel in the stream may be scheduled while this one still runs, and does its set-up
// (shared-memory barriers, tensor-memory allocation, weight prefetch) in that shadow.
// pdl_wait() returns once the previous kernel has completed and its writes are visible; no
// kernel reads or writes anything another kernel touches before it.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_entry() {
    pdl_launch_dependents();
    pdl_wait();
}

inline bool& pdl_enabled() {
    static bool enabled = true;
    return enabled;
}

template <typename Kernel>
struct PdlLauncher {
    Kernel kernel;
    dim3 grid, block;
    size_t smem;
    cudaStream_t stream;
    template <typename... Args>
    void operator()(Args... args) const {
        cudaLaunchConfig_t config = {};
        config.gridDim = grid;
        config.blockDim = block;
        config.dynamicSmemBytes = smem;
        config.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attr;
        config.numAttrs = pdl_enabled() ? 1 : 0;
        cudaLaunchKernelEx(&config, kernel, args...);   // errors surface through fwb_launch_status()
    }
};
template <typename Kernel>
PdlLauncher<Kernel> pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream) {
    return PdlLauncher<Kernel>{kernel, grid, block, smem, stream};
}

// ---- element access: everything is computed in fp32, stored as T --------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch`
// holds 33 floats of shared memory.  The order of additions is fixed by the
// block size alone, so equal inputs give equal sums.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        float t = lane < warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// silu(g) = g * sigmoid(g), sigmoid split by sign so neither branch overflows.
__device__ __forceinline__ float silu_f32(float g) {
    const float e = expf(-fabsf(g));
    const float sig = g >= 0.0f ? 1.0f / (1.0f + e) : e / (1.0f + e);
    return g * sig;
}

}  // namespace fwb
