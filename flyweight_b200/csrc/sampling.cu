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
    const unsigned b = __float_as_uint(v + 0.0f);    // -0 becomes +0: equal values get equal bits
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
    const bool vectorised = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    const int quads = vectorised ? V >> 2 : 0;
    unsigned long long best = 0ull;
#pragma unroll 4
    for (int qd = threadIdx.x; qd < quads; qd += blockDim.x) {
        const float4 l4 = reinterpret_cast<const float4*>(row)[qd];
        const float l[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned long long key = make_key(l[j], 4 * qd + j);
            best = key > best ? key : best;
        }
    }
    for (int i = 4 * quads + threadIdx.x; i < V; i += blockDim.x) {
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

// Inclusive prefix sums of a[0 .. 2 * blockDim.x) in place (every thread owns two neighbours);
// `warp_totals` holds one word per warp.  All threads call it.
__device__ void block_prefix_sums(unsigned long long* a, unsigned long long* warp_totals) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, warps = blockDim.x >> 5;
    const unsigned long long x0 = a[2 * t], x1 = a[2 * t + 1];
    unsigned long long s = x0 + x1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long v = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += v;
    }
    if (lane == 31) warp_totals[warp] = s;
    __syncthreads();
    if (warp == 0) {
        unsigned long long v = lane < warps ? warp_totals[lane] : 0ull;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long w = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += w;
        }
        if (lane < warps) warp_totals[lane] = v;
    }
    __syncthreads();
    const unsigned long long before = (warp ? warp_totals[warp - 1] : 0ull) + (s - (x0 + x1));
    a[2 * t] = before + x0;
    a[2 * t + 1] = before + x0 + x1;
    __syncthreads();
}

// The first index of the non-decreasing a[0 .. n) with a[index] >= target (n if there is none).
__device__ int first_reaching(const unsigned long long* a, int n, unsigned long long target) {
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (a[mid] >= target) hi = mid;
        else lo = mid + 1;
    }
    return lo;
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

// The draw over `n` sorted candidates (keys descending), double arithmetic.  The exponentials
// are formed by the whole block (`fill_probs`, then a barrier), the running sums by one thread
// in candidate order, which is what makes a draw reproducible to the last bit.
__device__ void fill_probs(const unsigned long long* keys, int n, const RowParams& prm, double* probs) {
    if (!(prm.temperature > 0.0f)) return;
    const double t = (double)prm.temperature;
    const double maximum = (double)key_logit(keys[0]) / t;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const double scaled = (double)key_logit(keys[i]) / t;
        probs[i] = isfinite(scaled) ? exp(scaled - maximum) : 0.0;
    }
}

__device__ int draw_sorted(const unsigned long long* keys, int n, const RowParams& prm, double u,
                           const double* probs) {
    if (!(prm.temperature > 0.0f) || n == 1) return key_id(keys[0]);
    double total = 0.0;
    for (int i = 0; i < n; ++i) total += probs[i];
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

// ------------------------------------------------------------------ the sampling kernel
// A row is worked on by a thread-block cluster of CLUSTER CTAs; CTA c owns every CLUSTER-th group
// of four logits.  Nothing is sorted except the (at most 1024) candidates of a top-k row.
//
// "The k-th largest key" and "the first candidate, in descending order, at which the running
// mass reaches T" are the same question -- the largest key x with weight{keys > x} < T <=
// weight{keys >= x} -- and x is found digit by digit from the top, eight bits a pass: every CTA
// makes a histogram of weight per digit over its share of the row (weight 1 for top-k, the
// probability mass for top-p and for the draw), the CTAs read one another's histograms through
// distributed shared memory, and all of them take the same step down.  Masses are 64-bit fixed
// point (p * 2^40 with p = exp((l - l0)/t) in double, p0 = 1), so every sum is an exact integer
// whatever the order of addition: the draw is reproducible.  Against the sequential double sums
// of the definition the kept prefix and the drawn token can differ only when a threshold falls
// within ~2^-40 of the boundary between two candidates.
// CLUSTER (8, 4, 2 or 1) is chosen on the host by the number of rows: eight CTAs a row answer a
// few rows soonest; with hundreds of rows the clusters would queue for the SMs in many rounds, each
// bound by its barriers, and fewer CTAs a row keep every row in flight at once.
constexpr int CTA_THREADS = 512;
constexpr int LIST_CAP = 2048;                   // shortlist entries a CTA keeps (16 KB)
constexpr int CTA_WARPS = CTA_THREADS / 32;
constexpr double MASS_ONE = 1099511627776.0;     // 2^40
constexpr int LEVELS = 7;                        // mass levels 2^38, 2^36 ... 2^26 (a quarter ... 2^-14 of the first candidate's)

__device__ __forceinline__ unsigned cluster_cta_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned peer_address(const void* local, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote)
                 : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ unsigned long long peer_load_u64(const void* local, unsigned rank) {
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(peer_address(local, rank)));
    return v;
}

// What a CTA keeps in shared memory for the walks and the reductions.
struct Shared {
    unsigned long long total[2][256];              // this CTA's histogram of the pass (peers read it); passes alternate
    unsigned long long per_warp[CTA_WARPS][256];   // one histogram per warp, summed into `total`
    unsigned long long all[256];                   // the cluster's histogram
    unsigned long long slot[2];                    // this CTA's share of a cluster-wide sum or maximum; calls alternate
    unsigned turn;                                 // which of the two a reduction writes next
    unsigned members[256];                         // pass 3 only: how many members fell into a digit ...
    unsigned long long largest[256];               // ... and the largest key among them
    unsigned long long pick[2];                    // digits chosen so far, what is left of the target
    unsigned settled;                              // pass 3 found the one key with the chosen logit
    unsigned long long scratch[33];
    unsigned long long keys[SMALL_K];              // the candidates of a top-k row (rank 0 sorts and draws)
    double probs[SMALL_K];
    unsigned count;
    // top-k rows: once a pass has narrowed the k-th key down to a bucket with few members, this
    // CTA's members of that bucket are kept here and the later passes walk them instead of the row
    unsigned long long list[LIST_CAP];
    unsigned list_count;
    unsigned list_state;                           // 0: walking the row, 1: walking the lists, 2: a list overflowed (row again)
    unsigned long long bucket_members;             // members of the bucket the last pass chose (cluster-wide)
    unsigned done;                                 // rank 0: the row's token has been drawn from the sorted candidates
    unsigned attempt;                              // the 1,024 largest candidates may hold the top-p prefix
    unsigned long long level_all[2 * LEVELS + 2];  // `level` summed over the cluster
    unsigned long long level[2 * LEVELS + 2];      // of a sample of this CTA's candidates: how many weigh at least each mass level and their mass; the sample's size and mass
};

// Sum (or maximum) over the cluster of one value per thread.
template <int CLUSTER, bool MAXIMUM>
__device__ unsigned long long cluster_reduce(unsigned long long v, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = MAXIMUM ? (other > v ? other : v) : v + other;
    }
    __syncthreads();
    if (lane == 0) sh.scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned long long t = lane < CTA_WARPS ? sh.scratch[lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
            t = MAXIMUM ? (other > t ? other : t) : t + other;
        }
        if (lane == 0) sh.slot[sh.turn & 1] = t;
    }
    // One barrier is enough: this slot is written again two reductions from now, and before that
    // every CTA passes the barrier of the next reduction, which a peer reaches only after this read.
    cluster_barrier();
    const unsigned which = sh.turn & 1;
    unsigned long long part[CLUSTER];
#pragma unroll
    for (unsigned r = 0; r < CLUSTER; ++r) part[r] = peer_load_u64(&sh.slot[which], r);
    unsigned long long all = 0ull;
#pragma unroll
    for (unsigned r = 0; r < CLUSTER; ++r) all = MAXIMUM ? (part[r] > all ? part[r] : all) : all + part[r];
    __syncthreads();
    if (threadIdx.x == 0) sh.turn = which + 1;
    __syncthreads();
    return all;
}

// Calls f(logit, index, mass) for every element of the row this CTA owns: groups of four logits
// (one 16-byte load, several loads in flight), dealt round robin to the CTAs of the cluster.
template <int CLUSTER, bool WITH_MASS, typename F>
__device__ __forceinline__ void sweep(const float* __restrict__ row, const unsigned long long* __restrict__ mass,
                                      int V, unsigned rank, F f) {
    const bool vectorised = (reinterpret_cast<uintptr_t>(row) & 15) == 0 &&
                            (!WITH_MASS || (reinterpret_cast<uintptr_t>(mass) & 15) == 0);
    const int quads = vectorised ? V >> 2 : 0;
#pragma unroll 2
    for (int qd = rank * CTA_THREADS + threadIdx.x; qd < quads; qd += CLUSTER * CTA_THREADS) {
        const float4 l4 = reinterpret_cast<const float4*>(row)[qd];
        ulonglong2 ma = make_ulonglong2(0ull, 0ull), mb = ma;
        if (WITH_MASS) {
            ma = reinterpret_cast<const ulonglong2*>(mass)[2 * qd];
            mb = reinterpret_cast<const ulonglong2*>(mass)[2 * qd + 1];
        }
        f(l4.x, 4 * qd, ma.x);
        f(l4.y, 4 * qd + 1, ma.y);
        f(l4.z, 4 * qd + 2, mb.x);
        f(l4.w, 4 * qd + 3, mb.y);
    }
    for (int i = 4 * quads + rank * CTA_THREADS + threadIdx.x; i < V; i += CLUSTER * CTA_THREADS)
        f(row[i], i, WITH_MASS ? mass[i] : 0ull);
}

// The same walk with loops that all lanes of a warp run the same number of times: f(valid, logit,
// index) is called by every lane in every turn (valid: the lane has an element), so f may use
// warp-wide primitives with the full mask.
template <int CLUSTER, typename F>
__device__ __forceinline__ void sweep_together(const float* __restrict__ row, int V, unsigned rank, F f) {
    const bool vectorised = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    const int quads = vectorised ? V >> 2 : 0;
#pragma unroll 2
    for (int base = rank * CTA_THREADS; base < quads; base += CLUSTER * CTA_THREADS) {
        const int qd = base + threadIdx.x;
        const bool valid = qd < quads;
        const float4 l4 = valid ? reinterpret_cast<const float4*>(row)[qd] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        f(valid, l4.x, 4 * qd);
        f(valid, l4.y, 4 * qd + 1);
        f(valid, l4.z, 4 * qd + 2);
        f(valid, l4.w, 4 * qd + 3);
    }
    for (int base = 4 * quads + rank * CTA_THREADS; base < V; base += CLUSTER * CTA_THREADS) {
        const int i = base + threadIdx.x;
        const bool valid = i < V;
        f(valid, valid ? row[i] : 0.0f, i);
    }
}

// The largest key x among the row's members with weight{members > x} < target <= weight{members >= x}.
// Members: keys >= low_cut whose mass is >= floor_mass; COUNT: every member weighs 1 (mass unused).
// 1 <= target <= the members' weight.  Every CTA of the cluster returns the same key.
//
// SHORTLIST (top-k rows, COUNT): as soon as the bucket a pass chose has few members (cluster-wide, at
// most LIST_CAP / 2 a CTA on average), one more walk over the row puts every CTA's members of that
// bucket on its list and sends the keys ABOVE the bucket -- fewer than `target` of them, candidates
// for certain -- straight to rank 0's candidate array (keys_at_0 / count_at_0, which rank 0 has
// emptied before); the remaining passes walk the lists.  sh.list_state says afterwards whether the
// lists hold the bucket (1) or the row has to be walked for the candidates as before (0, 2).
template <int CLUSTER, bool COUNT, bool SHORTLIST = false>
__device__ unsigned long long descend(const float* __restrict__ row, int V, const unsigned long long* __restrict__ mass,
                                      unsigned long long low_cut, unsigned long long floor_mass,
                                      unsigned long long target, unsigned rank, Shared& sh,
                                      unsigned keys_at_0 = 0u, unsigned count_at_0 = 0u) {
    __syncthreads();
    if (threadIdx.x == 0) {
        sh.pick[0] = 0ull;
        sh.pick[1] = target;
        sh.list_state = 0u;
        sh.list_count = 0u;
    }
    unsigned long long* mine = sh.per_warp[threadIdx.x >> 5];
    for (int pass = 0; pass < 8; ++pass) {
        const int shift = 56 - 8 * pass;
        for (int i = threadIdx.x; i < CTA_WARPS * 256; i += CTA_THREADS) (&sh.per_warp[0][0])[i] = 0ull;
        if (pass == 3)
            for (int i = threadIdx.x; i < 256; i += CTA_THREADS) {
                sh.members[i] = 0u;
                sh.largest[i] = 0ull;
            }
        __syncthreads();
        const unsigned long long prefix = sh.pick[0];
        const unsigned long long mask = pass == 0 ? 0ull : (~0ull << (shift + 8));
        if (COUNT) {
            // Counting members (every weight 1): the lanes of a warp that hold the same digit are
            // found with one match and their leader adds their number, so that thirty-two lanes never
            // queue for one word of the histogram.  (In a first pass a few digits hold nearly every
            // key: with one atomic a lane it took six times as long as a plain walk over the row.)
            auto count_one = [&](bool valid, unsigned long long key) {
                const bool member = valid && (key & mask) == prefix && key >= low_cut;
                const int digit = member ? (int)((key >> shift) & 0xffull) : -1;
                const unsigned same = __match_any_sync(0xffffffffu, digit);
                if (!member) return;
                const bool leader = (int)(__ffs(same) - 1) == (int)(threadIdx.x & 31);
                if (pass == 3) {                     // few keys share 24 bits of a logit
                    if (leader) atomicAdd(&sh.members[digit], (unsigned)__popc(same));
                    atomicMax(&sh.largest[digit], key);
                }
                if (leader) atomicAdd(&mine[digit], (unsigned long long)__popc(same));
            };
            if (SHORTLIST && sh.list_state == 1u) {
                const unsigned n_list = sh.list_count;
                for (unsigned base = 0; base < n_list; base += CTA_THREADS) {
                    const unsigned i = base + threadIdx.x;
                    count_one(i < n_list, i < n_list ? sh.list[i] : 0ull);
                }
            } else {
                sweep_together<CLUSTER>(row, V, rank, [&](bool valid, float logit, int i) {
                    count_one(valid, make_key(logit, i));
                });
            }
        } else {
            // Masses: in the first pass nearly all keys share two or three digits (the sign and the
            // top of the exponent): a thread keeps four digits' sums in registers and touches the
            // histogram only when a fifth digit turns up.  (Adding the masses of equal digits inside
            // the warp first, as the counts are, was slower: two integer reductions a key.)
            int held[4] = {-1, -1, -1, -1};
            unsigned long long sums[4] = {0ull, 0ull, 0ull, 0ull};
            int victim = 0;
            sweep<CLUSTER, true>(row, mass, V, rank, [&](float logit, int i, unsigned long long m) {
                const unsigned long long key = make_key(logit, i);
                if ((key & mask) != prefix || key < low_cut || m < floor_mass) return;
                const int digit = (int)((key >> shift) & 0xffull);
                if (pass == 3) {
                    atomicAdd(&sh.members[digit], 1u);
                    atomicMax(&sh.largest[digit], key);
                }
                bool hit = false;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (held[c] == digit) {
                        sums[c] += m;
                        hit = true;
                    }
                if (!hit) {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c == victim) {
                            if (held[c] >= 0) atomicAdd(&mine[held[c]], sums[c]);
                            held[c] = digit;
                            sums[c] = m;
                        }
                    victim = (victim + 1) & 3;
                }
            });
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (held[c] >= 0) atomicAdd(&mine[held[c]], sums[c]);
        }
        __syncthreads();
        for (int d = threadIdx.x; d < 256; d += CTA_THREADS) {
            unsigned long long all = 0ull;
#pragma unroll
            for (int w = 0; w < CTA_WARPS; ++w) all += sh.per_warp[w][d];
            sh.total[pass & 1][d] = all;
        }
        // one barrier a pass: the histogram of pass p is written again in pass p+2, after the
        // barrier of pass p+1, which a peer reaches only when it has read pass p's
        cluster_barrier();
        for (int d = threadIdx.x; d < 256; d += CTA_THREADS) {
            // all peers' words are requested before the first is used: one round trip, not eight
            unsigned long long part[CLUSTER];
#pragma unroll
            for (unsigned r = 0; r < CLUSTER; ++r) part[r] = peer_load_u64(&sh.total[pass & 1][d], r);
            unsigned long long all = 0ull;
#pragma unroll
            for (unsigned r = 0; r < CLUSTER; ++r) all += part[r];
            sh.all[d] = all;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // the digit at which the running weight, from digit 255 down, reaches what is left of
            // the target: a lane adds up eight digits, a scan over the lanes finds the lane, the
            // lane its digit
            const int lane = threadIdx.x;
            const unsigned long long left = sh.pick[1];
            unsigned long long eight = 0ull;
#pragma unroll
            for (int j = 0; j < 8; ++j) eight += sh.all[255 - 8 * lane - j];
            unsigned long long upto = eight;               // inclusive, lanes 0..lane
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned long long other = __shfl_up_sync(0xffffffffu, upto, o);
                if (lane >= o) upto += other;
            }
            const unsigned crossed = __ballot_sync(0xffffffffu, upto >= left);
            const int owner = crossed ? __ffs(crossed) - 1 : 31;
            if (lane == owner) {
                unsigned long long rest = left - (upto - eight);
                int digit = 255 - 8 * lane;
                for (int j = 0; j < 7; ++j, --digit) {
                    if (sh.all[digit] >= rest) break;
                    rest -= sh.all[digit];
                }
                sh.pick[0] = prefix | ((unsigned long long)digit << shift);
                sh.pick[1] = rest;
                sh.settled = 0u;
                sh.bucket_members = sh.all[digit];
                if (pass == 3) {
                    // the logit is settled.  If one key has it (nearly always), that is the answer
                    // and the four passes over the id bits are not needed.
                    unsigned count = 0u;
                    unsigned long long top = 0ull;
                    for (unsigned r = 0; r < CLUSTER; ++r) {
                        unsigned c;
                        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(c) : "r"(peer_address(&sh.members[digit], r)));
                        const unsigned long long k = peer_load_u64(&sh.largest[digit], r);
                        count += c;
                        top = k > top ? k : top;
                    }
                    if (count == 1u) {
                        sh.pick[0] = top;
                        sh.settled = 1u;
                    }
                }
            }
        }
        __syncthreads();                            // pick is set
        if (pass == 3 && sh.settled) break;
        if (SHORTLIST && sh.list_state == 0u && pass < 3 &&
            sh.bucket_members <= (unsigned long long)(CLUSTER * (LIST_CAP / 2))) {
            // few members left: every CTA lists its own, the keys above the bucket go to rank 0
            const unsigned long long chosen = sh.pick[0];
            const unsigned long long bucket_mask = ~0ull << shift;
            unsigned over = 0u;
            sweep<CLUSTER, false>(row, nullptr, V, rank, [&](float logit, int i, unsigned long long) {
                const unsigned long long key = make_key(logit, i);
                if ((key & bucket_mask) == chosen) {
                    const unsigned at = atomicAdd(&sh.list_count, 1u);
                    if (at < (unsigned)LIST_CAP) sh.list[at] = key;
                    else over = 1u;
                } else if (key > chosen) {          // a digit above the chosen one: fewer than `target` such keys
                    unsigned at;
                    asm volatile("atom.shared::cluster.add.u32 %0, [%1], 1;" : "=r"(at) : "r"(count_at_0) : "memory");
                    if (at < (unsigned)SMALL_K)
                        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(keys_at_0 + at * 8u), "l"(key) : "memory");
                }
            });
            const unsigned long long any_over = cluster_reduce<CLUSTER, true>((unsigned long long)over, sh);
            if (threadIdx.x == 0) sh.list_state = any_over ? 2u : 1u;
            __syncthreads();
        }
    }
    // the walk's last histogram may still be read by a peer: the next walk or reduction of this
    // kernel starts with writes to other words and passes a cluster barrier before it returns here
    return sh.pick[0];
}

// Grid (CLUSTER, R), cluster (CLUSTER, 1, 1).  mass_all: [R][Vpad] 64-bit words of scratch, needed
// by rows with more than SMALL_K candidates (null: such rows are refused on the host).
template <int CLUSTER>
__global__ void __launch_bounds__(CTA_THREADS)
sample_kernel(const float* __restrict__ logits, int V, int Vpad, const RowParams* __restrict__ params,
              const double* __restrict__ uniform, const int* __restrict__ recent, int recent_stride,
              unsigned long long* __restrict__ mass_all, int* __restrict__ out) {
    fwb::pdl_entry();
    extern __shared__ __align__(16) unsigned char shared_raw[];
    Shared& sh = *reinterpret_cast<Shared*>(shared_raw);
    unsigned long long* keys = sh.keys;
    double* probs = sh.probs;
    const unsigned rank = cluster_cta_rank();
    const int r = blockIdx.y;
    if (threadIdx.x == 0) sh.turn = 0u;
    __syncthreads();
    const RowParams prm = params[r];
    const float* row = logits + (size_t)r * V;
    const int k = prm.top_k > 0 ? (prm.top_k < V ? prm.top_k : V) : V;
    // a row with more than SMALL_K candidates arrives with its penalties already applied to its
    // logits (fwb_penalize_rows), so its history is not looked at here
    const bool penalize = k <= SMALL_K && prm.n_recent > 0 &&
                          (prm.repetition_penalty != 1.0f || prm.presence_penalty != 0.0f ||
                           prm.frequency_penalty != 0.0f);

    const bool greedy_row = (!(prm.temperature > 0.0f) && !penalize) || k == 1;
    unsigned long long best = 0ull;
    if (greedy_row || k > SMALL_K) {                // (a sorted candidate list knows its own maximum)
        sweep<CLUSTER, false>(row, nullptr, V, rank, [&](float logit, int i, unsigned long long) {
            const unsigned long long key = make_key(logit, i);
            best = key > best ? key : best;
        });
        best = cluster_reduce<CLUSTER, true>(best, sh);
    }
    if (greedy_row) {
        if (rank == 0 && threadIdx.x == 0) out[r] = key_id(best);
        cluster_barrier();                          // no CTA leaves while a peer still reads its shared memory
        return;
    }

    if (k <= SMALL_K) {
        // the candidates are the k largest keys: find the k-th, gather them in rank 0, sort, draw
        if (rank == 0) {
            for (int i = threadIdx.x; i < SMALL_K; i += CTA_THREADS) keys[i] = 0ull;
            if (threadIdx.x == 0) sh.count = 0u;
        }
        cluster_barrier();                          // rank 0's array is empty before anybody sends to it
        const unsigned keys_at_0 = peer_address(keys, 0), count_at_0 = peer_address(&sh.count, 0);
        const unsigned long long kth = descend<CLUSTER, true, true>(row, V, nullptr, 0ull, 0ull, (unsigned long long)k,
                                                                    rank, sh, keys_at_0, count_at_0);
        auto candidate = [&](unsigned long long key) {
            if (key < kth) return;                  // keys are distinct: exactly k keys pass in all
            unsigned at;
            asm volatile("atom.shared::cluster.add.u32 %0, [%1], 1;" : "=r"(at) : "r"(count_at_0) : "memory");
            if (at < (unsigned)SMALL_K)
                asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(keys_at_0 + at * 8u), "l"(key) : "memory");
        };
        if (sh.list_state == 1u) {
            // the keys above the bucket are at rank 0 already; the rest of the candidates are on the lists
            const unsigned n_list = sh.list_count;
            for (unsigned i = threadIdx.x; i < n_list; i += CTA_THREADS) candidate(sh.list[i]);
        } else {
            if (sh.list_state == 2u) {              // a list overflowed: what was sent to rank 0 is sent again below
                cluster_barrier();
                if (rank == 0 && threadIdx.x == 0) sh.count = 0u;
                cluster_barrier();
            }
            sweep<CLUSTER, false>(row, nullptr, V, rank, [&](float logit, int i, unsigned long long) {
                candidate(make_key(logit, i));
            });
        }
        cluster_barrier();
        if (rank != 0) return;
        int padded = 1;
        while (padded < k) padded <<= 1;
        bitonic_sort_desc(keys, padded);
        if (penalize) {
            const int* rec = recent + (size_t)r * recent_stride;
            for (int i = threadIdx.x; i < k; i += CTA_THREADS) {
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
        __syncthreads();
        fill_probs(keys, k, prm, probs);
        __syncthreads();
        if (threadIdx.x == 0) out[r] = draw_sorted(keys, k, prm, uniform[r], probs);
        return;
    }

    // more than SMALL_K candidates (the whole vocabulary among them): no sort at all
    unsigned long long* mass = mass_all + (size_t)r * Vpad;
    unsigned long long low_cut = 0ull;
    if (k < V) low_cut = descend<CLUSTER, true>(row, V, nullptr, 0ull, 0ull, (unsigned long long)k, rank, sh);
    const double t = (double)prm.temperature;
    const double maximum = (double)key_logit(best) / t;
    unsigned long long mine = 0ull;
    constexpr int LEVEL_WORDS = 2 * LEVELS + 2;
    if (threadIdx.x < LEVEL_WORDS) sh.level[threadIdx.x] = 0ull;
    __syncthreads();
    const bool estimate = prm.top_p < 1.0f;
    sweep<CLUSTER, false>(row, nullptr, V, rank, [&](float logit, int i, unsigned long long) {
        unsigned long long m = 0ull;
        if (make_key(logit, i) >= low_cut) {
            const double scaled = (double)logit / t;
            const double p = isfinite(scaled) ? exp(scaled - maximum) : 0.0;
            m = (unsigned long long)llrint(p * MASS_ONE);
        }
        mass[i] = m;                                // read again only by this CTA, in the same order
        mine += m;
    });
    if (estimate && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // Of every eighth group of 128 masses this CTA has just written (each thread reads its own
        // back): how many weigh at least 2^38, 2^36 ... 2^26 and what those weigh together -- an
        // estimate, enough to tell further down a row whose top-p prefix will not lie inside its
        // 1,024 largest candidates.  (A walk of its own: kept beside the masses above, these sums
        // cost the registers that let two CTAs share an SM.)
        unsigned level_count[LEVELS];
        unsigned long long level_mass[LEVELS];
#pragma unroll
        for (int j = 0; j < LEVELS; ++j) {
            level_count[j] = 0u;
            level_mass[j] = 0ull;
        }
        unsigned seen = 0u;
        unsigned long long seen_mass = 0ull;
        const int quads = V >> 2;
        int turn = threadIdx.x >> 5;
        for (int qd = rank * CTA_THREADS + threadIdx.x; qd < quads; qd += CLUSTER * CTA_THREADS, ++turn) {
            if (turn & 7) continue;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const unsigned long long m = mass[4 * qd + e];
                ++seen;
                seen_mass += m;
                const unsigned top = (unsigned)(m >> 26);   // m <= 2^40
#pragma unroll
                for (int j = 0; j < LEVELS; ++j)
                    if (top >= (1u << (12 - 2 * j))) {
                        ++level_count[j];
                        level_mass[j] += m;
                    }
            }
        }
        if (__any_sync(0xffffffffu, seen != 0u)) {
            auto add_up = [&](unsigned long long v, int word) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if ((threadIdx.x & 31) == 0 && v) atomicAdd(&sh.level[word], v);
            };
#pragma unroll
            for (int j = 0; j < LEVELS; ++j) {
                add_up(level_count[j], 2 * j);
                add_up(level_mass[j], 2 * j + 1);
            }
            add_up(seen, 2 * LEVELS);
            add_up(seen_mass, 2 * LEVELS + 1);
        }
    }
    // (the barriers inside the reduction put these sums before the peers' reads below)
    const unsigned long long total = cluster_reduce<CLUSTER, false>(mine, sh);     // >= 2^40: the first candidate weighs 1
    // Can the 1,024 largest candidates reach top_p of the total?  None weighs more than the first
    // one's 2^40, so not if that asks for more than 1,024 * 2^40.  And with n candidates at or above
    // a level L, the candidates outside the 1,024 largest weigh at least (mass below L) + (n - 1024) L
    // (for n < 1,024: the 1,024 largest take fewer than 1,024 - n from below L); if that, as estimated
    // from the sample, is more than top_p leaves over, the row goes straight to the walks further down.
    // Either way the same token is drawn: this only chooses the shorter way.
    bool prefix_may_be_short = false;
    if (estimate) {
        const double wanted = ceil((double)prm.top_p * (double)total);
        prefix_may_be_short = wanted <= (double)SMALL_K * MASS_ONE;
        // one thread a word fetches the peers' sums; thread 0 decides for the CTA (every CTA of the
        // cluster adds the same integers and decides alike)
        if (threadIdx.x < LEVEL_WORDS) {
            unsigned long long sum = 0ull;
#pragma unroll
            for (unsigned c = 0; c < CLUSTER; ++c) sum += peer_load_u64(&sh.level[threadIdx.x], c);
            sh.level_all[threadIdx.x] = sum;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned long long* word = sh.level_all;
            unsigned may = prefix_may_be_short ? 1u : 0u;
            if (word[2 * LEVELS] > 0ull) {
                const double scale = (double)V / (double)word[2 * LEVELS];
                const double left_over = (double)total - wanted;
                for (int j = 0; j < LEVELS; ++j) {
                    const double level = (double)(1ull << (38 - 2 * j));
                    const double n = scale * (double)word[2 * j];
                    const double below = scale * (double)(word[2 * LEVELS + 1] - word[2 * j + 1]);
                    if (below + (n - (double)SMALL_K) * level > left_over) may = 0u;
                }
            }
            sh.attempt = may;
        }
        __syncthreads();
        prefix_may_be_short = sh.attempt != 0u;
    }
    if (prm.top_p < 1.0f && prefix_may_be_short && CTA_THREADS * 2 == SMALL_K) {
        // The prefix that top_p keeps is, for any row that is not nearly flat, far shorter than
        // 1,024 candidates.  So: gather the 1,024 largest keys (two or three walks with the
        // shortlist), sort them, give them the same fixed-point masses, add those up in order --
        // if they reach top_p of the row's total, the cut, the min_p floor and the draw are all
        // inside them and the row is done after five walks instead of a dozen.  The same integers
        // in the same comparisons as below, so the same token.  If they do not reach it, go on below.
        if (rank == 0) {
            for (int i = threadIdx.x; i < SMALL_K; i += CTA_THREADS) keys[i] = 0ull;
            if (threadIdx.x == 0) {
                sh.count = 0u;
                sh.done = 0u;
            }
        }
        cluster_barrier();
        const unsigned keys_at_0 = peer_address(keys, 0), count_at_0 = peer_address(&sh.count, 0);
        const unsigned long long last = descend<CLUSTER, true, true>(row, V, nullptr, low_cut, 0ull,
                                                                     (unsigned long long)SMALL_K, rank, sh,
                                                                     keys_at_0, count_at_0);
        auto candidate = [&](unsigned long long key) {
            if (key < last) return;
            unsigned at;
            asm volatile("atom.shared::cluster.add.u32 %0, [%1], 1;" : "=r"(at) : "r"(count_at_0) : "memory");
            if (at < (unsigned)SMALL_K)
                asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(keys_at_0 + at * 8u), "l"(key) : "memory");
        };
        if (sh.list_state == 1u) {
            const unsigned n_list = sh.list_count;
            for (unsigned i = threadIdx.x; i < n_list; i += CTA_THREADS) candidate(sh.list[i]);
        } else {
            if (sh.list_state == 2u) {
                cluster_barrier();
                if (rank == 0 && threadIdx.x == 0) sh.count = 0u;
                cluster_barrier();
            }
            sweep<CLUSTER, false>(row, nullptr, V, rank, [&](float logit, int i, unsigned long long) {
                candidate(make_key(logit, i));
            });
        }
        cluster_barrier();
        if (rank == 0) {
            bitonic_sort_desc(keys, SMALL_K);
            unsigned long long* sums = reinterpret_cast<unsigned long long*>(probs);
            for (int i = threadIdx.x; i < SMALL_K; i += CTA_THREADS) {
                const double scaled = (double)key_logit(keys[i]) / t;
                const double p = isfinite(scaled) ? exp(scaled - maximum) : 0.0;
                sums[i] = (unsigned long long)llrint(p * MASS_ONE);
            }
            __syncthreads();
            block_prefix_sums(sums, sh.scratch);
            if (threadIdx.x == 0) {
                unsigned long long target = (unsigned long long)ceil((double)prm.top_p * (double)total);
                target = target < 1ull ? 1ull : (target > total ? total : target);
                if (sums[SMALL_K - 1] >= target) {
                    int keep = first_reaching(sums, SMALL_K, target) + 1;
                    if (prm.min_p > 0.0f) {
                        const unsigned long long floor_mass = (unsigned long long)ceil((double)prm.min_p * MASS_ONE);
                        int kept = 1;                  // the first candidate weighs 2^40: it stays
                        while (kept < keep && sums[kept] - sums[kept - 1] >= floor_mass) ++kept;
                        keep = kept;
                    }
                    const unsigned long long kept_mass = sums[keep - 1];
                    unsigned long long draw = (unsigned long long)ceil(uniform[r] * (double)kept_mass);
                    draw = draw < 1ull ? 1ull : (draw > kept_mass ? kept_mass : draw);
                    out[r] = key_id(keys[first_reaching(sums, keep, draw)]);
                    sh.done = 1u;
                }
            }
        }
        cluster_barrier();                          // rank 0 has decided
        unsigned done;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(done) : "r"(peer_address(&sh.done, 0)));
        cluster_barrier();                          // no CTA leaves while a peer still reads its shared memory
        if (done) return;
    }
    if (prm.top_p < 1.0f) {
        // the shortest prefix whose mass reaches top_p of the total
        unsigned long long target = (unsigned long long)ceil((double)prm.top_p * (double)total);
        target = target < 1ull ? 1ull : (target > total ? total : target);
        const unsigned long long cut = descend<CLUSTER, false>(row, V, mass, low_cut, 0ull, target, rank, sh);
        low_cut = cut > low_cut ? cut : low_cut;
    }
    // min_p: of that prefix, the candidates that weigh at least min_p of the first
    unsigned long long floor_mass = 0ull;
    if (prm.min_p > 0.0f) floor_mass = (unsigned long long)ceil((double)prm.min_p * MASS_ONE);
    unsigned long long kept_mine = 0ull;
    sweep<CLUSTER, true>(row, mass, V, rank, [&](float logit, int i, unsigned long long m) {
        if (make_key(logit, i) >= low_cut && m >= floor_mass) kept_mine += m;
    });
    const unsigned long long kept = cluster_reduce<CLUSTER, false>(kept_mine, sh);
    unsigned long long target = (unsigned long long)ceil(uniform[r] * (double)kept);
    target = target < 1ull ? 1ull : (target > kept ? kept : target);
    const unsigned long long drawn = descend<CLUSTER, false>(row, V, mass, low_cut, floor_mass, target, rank, sh);
    if (rank == 0 && threadIdx.x == 0) out[r] = key_id(drawn);
    cluster_barrier();                              // no CTA leaves while a peer still reads its shared memory
}

// Rows that keep more than SMALL_K candidates (the whole vocabulary among them) are never sorted,
// so their penalties cannot act on a sorted candidate list.  For those rows the penalties are
// applied to the row's logits themselves, over the whole vocabulary and before any cut, which is
// the order of flyweight's host sampler (src/flyweight/v2.py:1497-1518); the sampler then sees
// the row without a history.  One block per row; the thread that holds the first occurrence of
// a token id in the history applies all of that id's penalties.
__global__ void __launch_bounds__(MAX_RECENT)
penalize_rows_kernel(float* __restrict__ logits, int V, const RowParams* __restrict__ params,
                     const int* __restrict__ recent, int recent_stride) {
    fwb::pdl_entry();
    const int r = blockIdx.x;
    const RowParams prm = params[r];
    const int k = prm.top_k > 0 ? (prm.top_k < V ? prm.top_k : V) : V;
    if (prm.n_recent <= 0 || k <= SMALL_K) return;
    const int* rec = recent + (size_t)r * recent_stride;
    const int j = threadIdx.x;
    if (j >= prm.n_recent) return;
    const int id = rec[j];
    if (id < 0 || id >= V) return;
    int occurrences = 0;
    for (int i = 0; i < prm.n_recent; ++i) {
        if (rec[i] != id) continue;
        if (i < j) return;                          // an earlier thread owns this id
        ++occurrences;
    }
    float logit = logits[(size_t)r * V + id];
    if (prm.repetition_penalty != 1.0f)
        logit = logit > 0.0f ? logit / prm.repetition_penalty : logit * prm.repetition_penalty;
    logit -= prm.presence_penalty;
    logit -= prm.frequency_penalty * (float)occurrences;
    logits[(size_t)r * V + id] = logit;
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

namespace {
int g_sample_cluster = 0;

template <int CLUSTER>
int launch_sample(const float* logits, int R, int V, int Vpad, const void* params, const double* uniform,
                  const int* recent, int recent_stride, void* keys_scratch, int* out, cudaStream_t stream) {
    auto kernel = sample_kernel<CLUSTER>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Shared));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(CLUSTER, R);
    config.blockDim = dim3(CTA_THREADS);
    config.dynamicSmemBytes = sizeof(Shared);
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = fwb::pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, logits, V, Vpad, (const RowParams*)params, uniform,
                                       recent, recent_stride, (unsigned long long*)keys_scratch, out);
    return e == cudaSuccess ? fwb_launch_status() : (int)e;
}
}  // namespace

// params: [R] records of 8 x 4 bytes {temperature f32, top_k i32, top_p f32, min_p f32,
// repetition f32, presence f32, frequency f32, n_recent i32}; uniform: [R] doubles in [0,1);
// recent: [R][recent_stride] token ids (only the first n_recent of a row are read).
// keys_scratch: [R][Vpad] 64-bit words, needed only if some row keeps more than 1024 candidates
// (`need_large`); probs_scratch is not used any more.
FWB_API int fwb_sample(const float* logits, int R, int V, const void* params, const double* uniform,
                       const int* recent, int recent_stride, int* out, void* keys_scratch,
                       double* probs_scratch, int Vpad, int need_large, cudaStream_t stream) {
    (void)probs_scratch;
    if (R <= 0) return FWB_OK;
    if (!logits || !out || !params || !uniform || V <= 0) return FWB_BAD_ARGUMENT;
    if (recent_stride > MAX_RECENT || (recent_stride > 0 && !recent)) return FWB_BAD_ARGUMENT;
    if (need_large && (!keys_scratch || Vpad < V)) return FWB_BAD_ARGUMENT;
    if (V > (1 << 23)) return FWB_TOO_LARGE;      // the fixed-point masses of a row must fit 64 bits
    if (R > 65535) return FWB_TOO_LARGE;
    // as many CTAs a row as keep all rows on the GPU at once (two CTAs fit an SM), eight at most
    int cluster = g_sample_cluster;
    if (cluster <= 0) {
        cluster = 8;
        while (cluster > 1 && (long long)R * cluster > 2 * 148) cluster >>= 1;
        // rows that walk the whole vocabulary a dozen times are better off shared by two CTAs even
        // when the rows alone would fill the GPU (512 rows: 1.21 -> 1.04 ms)
        if (need_large && cluster < 2) cluster = 2;
    }
    switch (cluster) {
        case 8: return launch_sample<8>(logits, R, V, Vpad, params, uniform, recent, recent_stride, keys_scratch, out, stream);
        case 4: return launch_sample<4>(logits, R, V, Vpad, params, uniform, recent, recent_stride, keys_scratch, out, stream);
        case 2: return launch_sample<2>(logits, R, V, Vpad, params, uniform, recent, recent_stride, keys_scratch, out, stream);
        default: return launch_sample<1>(logits, R, V, Vpad, params, uniform, recent, recent_stride, keys_scratch, out, stream);
    }
}

// CTAs a row for the sampling kernel: 8, 4, 2 or 1 (0: chosen by the number of rows).  For tests
// and measurements; every choice draws the same tokens.
FWB_API int fwb_sample_set_cluster(int ctas) {
    if (ctas != 0 && ctas != 1 && ctas != 2 && ctas != 4 && ctas != 8) return FWB_BAD_ARGUMENT;
    g_sample_cluster = ctas;
    return FWB_OK;
}

// In place on a copy of the logits that the caller owns: the penalties of every row that keeps
// more than 1024 candidates (see penalize_rows_kernel).  Same params and recent arrays as
// fwb_sample, which is then called with those rows' histories emptied.
FWB_API int fwb_penalize_rows(float* logits, int R, int V, const void* params, const int* recent,
                              int recent_stride, cudaStream_t stream) {
    if (R <= 0 || recent_stride <= 0) return FWB_OK;
    if (!logits || !params || !recent || V <= 0) return FWB_BAD_ARGUMENT;
    if (recent_stride > MAX_RECENT) return FWB_BAD_ARGUMENT;
    if (R > 65535) return FWB_TOO_LARGE;
    fwb::pdl(penalize_rows_kernel, R, MAX_RECENT, 0, stream)(logits, V, (const RowParams*)params, recent,
                                                             recent_stride);
    return fwb_launch_status();
}
