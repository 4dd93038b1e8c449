// Sampling on the device: greedy argmax, and temperature sampling with top-k, top-p,
// min-p and repetition / presence / frequency penalties.
//
// Order of operations (it decides which token a given uniform number picks):
//   candidates = the top_k largest logits, sorted descending, ties to the lower id
//                (top_k == 0: the whole vocabulary);
//   penalties on candidates that occur among the request's recent tokens:
//                l = l > 0 ? l / rep : l * rep;  l -= presence;  l -= frequency * count;
//                then sorted again;
//   temperature 0: the first candidate;
//   else p_i = exp(l_i / t - l_0 / t) in double; keep the shortest prefix whose share of
//                the total mass reaches top_p; of that, keep the prefix with
//                p_i >= min_p * p_0; draw with one uniform number u: the first i with
//                u * kept_mass <= p_0 + ... + p_i.
//
// A logit and its id are packed into one 64-bit key, (ordered float bits << 32) |
// (0xffffffff - id), so that "larger key" means "larger logit, or equal logit and lower
// id", all keys are distinct, and selection and sorting need no tie rules of their own.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;
constexpr int SMALL_K = 1024;     // candidates that fit the shared-memory path
constexpr int MAX_RECENT = 256;

__device__ __forceinline__ unsigned ordered_bits(float v) {
    if (v != v) return 0u;                       // NaN sorts last
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unordered_bits(unsigned o) {
    const unsigned b = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
    return __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long make_key(float logit, int id) {
    return ((unsigned long long)ordered_bits(logit) << 32) | (unsigned long long)(0xffffffffu - (unsigned)id);
}
__device__ __forceinline__ int key_id(unsigned long long key) {
    return (int)(0xffffffffu - (unsigned)(key & 0xffffffffull));
}
__device__ __forceinline__ float key_logit(unsigned long long key) {
    return unordered_bits((unsigned)(key >> 32));
}

__device__ unsigned long long block_max_key(unsigned long long v, unsigned long long* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned long long t = lane < (blockDim.x >> 5) ? scratch[lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
            t = other > t ? other : t;
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ------------------------------------------------------------------ greedy
__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out) {
    fwb::pdl_entry();
    __shared__ unsigned long long scratch[33];
    const float* row = logits + (size_t)blockIdx.x * V;
    unsigned long long best = 0ull;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const unsigned long long key = make_key(row[i], i);
        best = key > best ? key : best;
    }
    best = block_max_key(best, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] = key_id(best);
}

// The same over `chunks` blocks per row: every block writes the best key of its slice, and the
// block that finds itself last for its row (a self-resetting counter) reduces the slices.  The
// maximum of distinct keys does not depend on the order, so the result is the same every time.
// partial: [R][chunks] keys; counters: [R] ints, zero before the first launch and left zero.
__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int V, int* __restrict__ out,
                    unsigned long long* __restrict__ partial, int* __restrict__ counters) {
    fwb::pdl_entry();
    __shared__ unsigned long long scratch[33];
    __shared__ int last;
    const int r = blockIdx.y, chunk = blockIdx.x, chunks = gridDim.x;
    const float* row = logits + (size_t)r * V;
    const int per = (V + chunks - 1) / chunks;
    const int begin = chunk * per, end = begin + per < V ? begin + per : V;
    unsigned long long best = 0ull;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const unsigned long long key = make_key(row[i], i);
        best = key > best ? key : best;
    }
    best = block_max_key(best, scratch);
    if (threadIdx.x == 0) {
        partial[(size_t)r * chunks + chunk] = best;
        __threadfence();
        last = atomicAdd(&counters[r], 1) == chunks - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    best = 0ull;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) {
        const unsigned long long key = *(volatile unsigned long long*)&partial[(size_t)r * chunks + i];
        best = key > best ? key : best;
    }
    best = block_max_key(best, scratch);
    if (threadIdx.x == 0) {
        out[r] = key_id(best);
        counters[r] = 0;
    }
}

// Descending bitonic sort of n (a power of two) keys by the whole block.
__device__ void bitonic_sort_desc(unsigned long long* keys, int n) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool descending = (i & size) == 0;
                    const unsigned long long a = keys[i], b = keys[j];
                    if ((a < b) == descending) {
                        keys[i] = b;
                        keys[j] = a;
                    }
                }
            }
        }
    }
    __syncthreads();
}

struct RowParams {
    float temperature;
    int top_k;
    float top_p;
    float min_p;
    float repetition_penalty;
    float presence_penalty;
    float frequency_penalty;
    int n_recent;
};

// The draw over `n` sorted candidates (keys descending).  One thread; double arithmetic.
// `probs` is scratch for n doubles.
__device__ int draw_sorted(const unsigned long long* keys, int n, const RowParams& prm, double u,
                           double* probs) {
    if (!(prm.temperature > 0.0f) || n == 1) return key_id(keys[0]);
    const double t = (double)prm.temperature;
    const double maximum = (double)key_logit(keys[0]) / t;
    double total = 0.0;
    for (int i = 0; i < n; ++i) {
        const double scaled = (double)key_logit(keys[i]) / t;
        const double p = isfinite(scaled) ? exp(scaled - maximum) : 0.0;
        probs[i] = p;
        total += p;
    }
    if (!(total > 0.0) || !isfinite(total)) return key_id(keys[0]);
    int keep = n;
    if (prm.top_p < 1.0f) {
        double cumulative = 0.0;
        for (int i = 0; i < n; ++i) {
            cumulative += probs[i] / total;
            if (cumulative >= (double)prm.top_p) {
                keep = i + 1;
                break;
            }
        }
    }
    if (prm.min_p > 0.0f) {
        const double floor_p = (double)prm.min_p * probs[0];
        int kept = 1;
        while (kept < keep && probs[kept] >= floor_p) ++kept;
        keep = kept;
    }
    double kept_total = 0.0;
    for (int i = 0; i < keep; ++i) kept_total += probs[i];
    const double threshold = u * kept_total;
    double cumulative = 0.0;
    for (int i = 0; i < keep; ++i) {
        cumulative += probs[i];
        if (threshold <= cumulative) return key_id(keys[i]);
    }
    return key_id(keys[keep - 1]);
}

// One block per row.  Rows whose candidate count is <= SMALL_K are finished here; rows
// that need more are finished by sample_large_kernel (they are marked in `out` by -1).
__global__ void __launch_bounds__(THREADS)
sample_small_kernel(const float* __restrict__ logits, int V, const RowParams* __restrict__ params,
                    const double* __restrict__ uniform, const int* __restrict__ recent,
                    int recent_stride, int* __restrict__ out) {
    fwb::pdl_entry();
    __shared__ unsigned long long keys[SMALL_K];
    __shared__ unsigned long long scratch[33];
    __shared__ double probs[SMALL_K];
    __shared__ int hist[256];
    __shared__ unsigned long long prefix_s;
    __shared__ int remaining_s, count_s;
    const int r = blockIdx.x;
    const RowParams prm = params[r];
    const float* row = logits + (size_t)r * V;
    const bool penalize = prm.n_recent > 0 && (prm.repetition_penalty != 1.0f ||
                          prm.presence_penalty != 0.0f || prm.frequency_penalty != 0.0f);
    int k = prm.top_k > 0 ? (prm.top_k < V ? prm.top_k : V) : V;
    if ((!(prm.temperature > 0.0f) && !penalize) || k == 1) {
        unsigned long long best = 0ull;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const unsigned long long key = make_key(row[i], i);
            best = key > best ? key : best;
        }
        best = block_max_key(best, scratch);
        if (threadIdx.x == 0) out[r] = key_id(best);
        return;
    }
    if (k > SMALL_K) {
        if (threadIdx.x == 0) out[r] = -1;
        return;
    }
    // radix select: the k-th largest key, 8 bits at a time from the top
    if (threadIdx.x == 0) {
        prefix_s = 0ull;
        remaining_s = k;
    }
    for (int pass = 0; pass < 8; ++pass) {
        const int shift = 56 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
        __syncthreads();
        const unsigned long long prefix = prefix_s;
        const unsigned long long mask = pass == 0 ? 0ull : (~0ull << (shift + 8));
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const unsigned long long key = make_key(row[i], i);
            if ((key & mask) == prefix) atomicAdd(&hist[(int)((key >> shift) & 0xffull)], 1);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int remaining = remaining_s;
            int digit = 255;
            for (; digit > 0; --digit) {
                if (hist[digit] >= remaining) break;
                remaining -= hist[digit];
            }
            prefix_s = prefix | ((unsigned long long)digit << shift);
            remaining_s = remaining;
        }
        __syncthreads();
    }
    const unsigned long long kth = prefix_s;     // keys are distinct: exactly k keys are >= kth
    int padded = 1;
    while (padded < k) padded <<= 1;
    for (int i = threadIdx.x; i < padded; i += blockDim.x) keys[i] = 0ull;
    if (threadIdx.x == 0) count_s = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const unsigned long long key = make_key(row[i], i);
        if (key >= kth) {
            const int at = atomicAdd(&count_s, 1);
            if (at < SMALL_K) keys[at] = key;
        }
    }
    __syncthreads();
    bitonic_sort_desc(keys, padded);
    if (penalize) {
        const int* rec = recent + (size_t)r * recent_stride;
        for (int i = threadIdx.x; i < k; i += blockDim.x) {
            const int id = key_id(keys[i]);
            int occurrences = 0;
            for (int j = 0; j < prm.n_recent; ++j) occurrences += rec[j] == id;
            if (occurrences) {
                float logit = key_logit(keys[i]);
                if (prm.repetition_penalty != 1.0f)
                    logit = logit > 0.0f ? logit / prm.repetition_penalty
                                         : logit * prm.repetition_penalty;
                logit -= prm.presence_penalty;
                logit -= prm.frequency_penalty * (float)occurrences;
                keys[i] = make_key(logit, id);
            }
        }
        __syncthreads();
        bitonic_sort_desc(keys, padded);
    }
    if (threadIdx.x == 0) out[r] = draw_sorted(keys, k, prm, uniform[r], probs);
}

// Rows that the small kernel left (out[r] == -1): sort the whole row in global scratch.
// keys: [R][Vpad] (Vpad = power of two >= V), probs: [R][Vpad] doubles.
__global__ void __launch_bounds__(THREADS)
sample_large_kernel(const float* __restrict__ logits, int V, int Vpad,
                    const RowParams* __restrict__ params, const double* __restrict__ uniform,
                    unsigned long long* __restrict__ keys_all, double* __restrict__ probs_all,
                    int* __restrict__ out) {
    fwb::pdl_entry();
    const int r = blockIdx.x;
    if (out[r] != -1) return;
    const RowParams prm = params[r];
    const float* row = logits + (size_t)r * V;
    unsigned long long* keys = keys_all + (size_t)r * Vpad;
    for (int i = threadIdx.x; i < Vpad; i += blockDim.x) keys[i] = i < V ? make_key(row[i], i) : 0ull;
    bitonic_sort_desc(keys, Vpad);
    const int k = prm.top_k > 0 ? (prm.top_k < V ? prm.top_k : V) : V;
    if (threadIdx.x == 0) out[r] = draw_sorted(keys, k, prm, uniform[r], probs_all + (size_t)r * Vpad);
}

}  // namespace

// With scratch (partial: R*chunks keys of 8 bytes, counters: R zeroed ints) a row is cut into
// `chunks` slices that run as separate blocks; without it one block scans a row.
FWB_API int fwb_argmax(const float* logits, int R, int V, int* out, void* partial, int* counters,
                       int chunks, cudaStream_t stream) {
    if (R <= 0) return FWB_OK;
    if (!logits || !out || V <= 0) return FWB_BAD_ARGUMENT;
    if (partial && counters && chunks > 1 && R <= 65535) {
        fwb::pdl(argmax_split_kernel, dim3(chunks, R), 256, 0, stream)(
            logits, V, out, (unsigned long long*)partial, counters);
        return fwb_launch_status();
    }
    fwb::pdl(argmax_kernel, R, THREADS, 0, stream)(logits, V, out);
    return fwb_launch_status();
}

// params: [R] records of 8 x 4 bytes {temperature f32, top_k i32, top_p f32, min_p f32,
// repetition f32, presence f32, frequency f32, n_recent i32}; uniform: [R] doubles in [0,1);
// recent: [R][recent_stride] token ids (only the first n_recent of a row are read).
// keys_scratch / probs_scratch: [R][Vpad] each, needed only if some row keeps more than
// 1024 candidates (pass null to refuse such rows).
FWB_API int fwb_sample(const float* logits, int R, int V, const void* params, const double* uniform,
                       const int* recent, int recent_stride, int* out, void* keys_scratch,
                       double* probs_scratch, int Vpad, int need_large, cudaStream_t stream) {
    if (R <= 0) return FWB_OK;
    if (!logits || !out || !params || !uniform || V <= 0) return FWB_BAD_ARGUMENT;
    if (recent_stride > MAX_RECENT || (recent_stride > 0 && !recent)) return FWB_BAD_ARGUMENT;
    fwb::pdl(sample_small_kernel, R, THREADS, 0, stream)(logits, V, (const RowParams*)params, uniform,
                                                   recent, recent_stride, out);
    int status = fwb_launch_status();
    if (status != FWB_OK || !need_large) return status;
    if (!keys_scratch || !probs_scratch || Vpad < V || (Vpad & (Vpad - 1))) return FWB_BAD_ARGUMENT;
    fwb::pdl(sample_large_kernel, R, THREADS, 0, stream)(logits, V, Vpad, (const RowParams*)params, uniform,
                                                   (unsigned long long*)keys_scratch, probs_scratch,
                                                   out);
    return fwb_launch_status();
}
