// The allocation-free greedy sampler declared in flyweight_b200_no_alloc.h.
//
// A variant of the split argmax of sampling.cu: the same slicing of a row over several
// blocks and the same "last block to arrive reduces the row" step, but the slice maxima and
// the arrival counters live in a file-scope __device__ array instead of buffers that the
// caller (or torch) allocates.  It has no counterpart in yairpatch/flyweight.
#include <mutex>
#include <stdio.h>

#include "common.cuh"
#include "flyweight_b200_no_alloc.h"

namespace {

constexpr int CHUNKS = 64;                       // slices per row
constexpr int MAX_ROWS = FWB_NO_ALLOC_MAX_ROWS;
constexpr int MAX_DEVICES = 64;

// Scratch, one copy per GPU that loads the library: slice maxima, then arrival counters.
struct Scratch {
    unsigned long long partial[MAX_ROWS * CHUNKS];   // 128 KiB
    int counters[MAX_ROWS];                          //   1 KiB
};
static __device__ __align__(256) Scratch g_scratch;

// In host code `g_scratch` is only a handle for the symbol, not a device address; the address
// is looked up once per device and cached here.
Scratch* g_scratch_address[MAX_DEVICES] = {};
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int fail(int code, const char* text) {
    snprintf(g_error, sizeof(g_error), "%s", text);
    return code;
}

__device__ __forceinline__ unsigned long long make_key(float v, int id) {
    unsigned bits = 0u;
    if (v == v) {                                 // NaN keeps 0: it loses against everything
        bits = __float_as_uint(v + 0.0f);         // -0 becomes +0: equal values, equal keys
        bits = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    }
    return ((unsigned long long)bits << 32) | (unsigned long long)(0xffffffffu - (unsigned)id);
}

__device__ unsigned long long block_max(unsigned long long v, unsigned long long* shared) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    __syncthreads();
    if (lane == 0) shared[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned long long t = lane < (int)(blockDim.x >> 5) ? shared[lane] : 0ull;
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
            t = other > t ? other : t;
        }
        if (lane == 0) shared[32] = t;
    }
    __syncthreads();
    return shared[32];
}

__global__ void __launch_bounds__(256)
argmax_no_alloc_kernel(const float* __restrict__ logits, int V, int* __restrict__ out, Scratch* scratch) {
    __shared__ unsigned long long shared[33];
    __shared__ int last;
    const int r = blockIdx.y, chunk = blockIdx.x;
    const float* row = logits + (size_t)r * V;
    const int per = (V + CHUNKS - 1) / CHUNKS;
    const int begin = chunk * per, end = begin + per < V ? begin + per : V;
    unsigned long long best = 0ull;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const unsigned long long key = make_key(row[i], i);
        best = key > best ? key : best;
    }
    best = block_max(best, shared);
    if (threadIdx.x == 0) {
        scratch->partial[r * CHUNKS + chunk] = best;
        __threadfence();
        last = atomicAdd(&scratch->counters[r], 1) == CHUNKS - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    best = 0ull;
    for (int i = threadIdx.x; i < CHUNKS; i += blockDim.x) {
        const unsigned long long key = *(volatile unsigned long long*)&scratch->partial[r * CHUNKS + i];
        best = key > best ? key : best;
    }
    best = block_max(best, shared);
    if (threadIdx.x == 0) out[r] = (int)(0xffffffffu - (unsigned)(best & 0xffffffffull));
}

// The device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(Scratch** address) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return fail((int)err, "cudaGetDevice failed");
    if (device < 0 || device >= MAX_DEVICES) return fail(FWB_TOO_LARGE, "device index beyond 63");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_address[device]) {
        void* found = nullptr;
        err = cudaGetSymbolAddress(&found, g_scratch);
        if (err != cudaSuccess || !found) {
            return fail(err != cudaSuccess ? (int)err : FWB_BAD_ARGUMENT,
                        "cudaGetSymbolAddress could not find the scratch array on this device");
        }
        g_scratch_address[device] = static_cast<Scratch*>(found);
    }
    *address = g_scratch_address[device];
    return FWB_OK;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int fwb_argmax_no_alloc(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
    if (!logits || !out) return fail(FWB_BAD_ARGUMENT, "logits and out must be device pointers");
    if (rows <= 0 || vocab <= 0) return fail(FWB_BAD_ARGUMENT, "rows and vocab must be positive");
    if (rows > MAX_ROWS || vocab > FWB_NO_ALLOC_MAX_VOCAB) {
        snprintf(g_error, sizeof(g_error),
                 "fwb_argmax_no_alloc serves at most %d rows of %d entries (asked: %d x %d); "
                 "use fwb_argmax with scratch of your own", MAX_ROWS, FWB_NO_ALLOC_MAX_VOCAB, rows, vocab);
        return FWB_TOO_LARGE;
    }
    if (stream) {
        // the scratch address below is that of the current device: the stream must live there
        int current = -1, of_stream = -1;
        if (cudaGetDevice(&current) == cudaSuccess && cudaStreamGetDevice(stream, &of_stream) == cudaSuccess &&
            current != of_stream) {
            snprintf(g_error, sizeof(g_error),
                     "the stream belongs to device %d but device %d is current; make the stream's device "
                     "current before the call", of_stream, current);
            return FWB_BAD_ARGUMENT;
        }
    }
    Scratch* scratch = nullptr;
    int status = scratch_for_current_device(&scratch);
    if (status != FWB_OK) return status;
    // The array keeps what the last call left (also a call that was cut short): the counters of
    // the rows in use start from zero on every call.  The slice maxima are all rewritten.
    cudaError_t err = cudaMemsetAsync(scratch->counters, 0, sizeof(int) * rows, stream);
    if (err != cudaSuccess) return fail((int)err, "clearing the arrival counters failed");
    argmax_no_alloc_kernel<<<dim3(CHUNKS, rows), 256, 0, stream>>>(logits, vocab, out, scratch);
    err = cudaPeekAtLastError();
    if (err != cudaSuccess) return fail((int)err, cudaGetErrorString(err));
    return FWB_OK;
}

extern "C" __attribute__((visibility("default")))
const char* fwb_no_alloc_last_error(void) { return g_error; }
