// The native step executor: one call runs the forward pass of a whole step.
//
// A *plan* is the model's forward pass as a short list of operations over fixed device
// buffers, built once per model from Python (every part of the model adds its operations;
// see flyweight_b200/engine/plan.py).  `fwb_plan_run` then takes one step's batch -- its int32
// arrays in pinned host memory and a few counts -- uploads the arrays and launches every
// kernel of the step from C++: no Python between launches, no allocation, no tensor objects.
// (flyweight's engine cycle is one C call too: native/include/flyweight_v2.h:1002.)
//
// Operations are semantic (norm + product, product + residual sum, short convolution, rotary
// + page write, attention, ...).  Which kernel serves one -- the tcgen05 product on single
// CTAs, on CTA pairs or with a split K, with the norm folded in or the sum in the epilogue, the
// SIMT product of the 32-bit path; the decode, tcgen05 or mma.sync attention kernel -- depends
// on the number of tokens in the step and is decided here, per step, by the same rules as
// the Python dispatch in flyweight_b200/kernels/tensorcore.py and attention.py (the two are
// compared bit for bit in the tests).
#include <stdint.h>
#include <string.h>

#include <vector>

#include "common.cuh"

// ---- the launchers of the other source files --------------------------------------------
extern "C" {
int fwb_embed(const void*, int, const int*, float*, int, int, int, int*, float, cudaStream_t);
int fwb_rmsnorm(float*, const float*, const float*, void*, int, const int*, int, int, float, cudaStream_t);
int fwb_silu_mul(const void*, int, void*, int, int, int, cudaStream_t);
int fwb_softcap(float*, long long, float, cudaStream_t);
int fwb_patch_tokens(int*, const int*, const int*, const int*, int, cudaStream_t);
int fwb_gemm_simt(const void*, int, const void*, int, void*, int, const float*, int, int, int, int, int,
                  cudaStream_t);
int fwb_gemm_tcgen05(const void*, const void*, void*, const float*, int, int, int, int, int, int, int, int,
                     int, int, int, cudaStream_t);
int fwb_gemm_tcgen05_normed(const float*, const float*, const int*, float, const void*, void*, int, int, int,
                            int, int, int, int, int, int, int, cudaStream_t);
int fwb_gemm_tcgen05_pair(const void*, const void*, void*, int, int, int, int, int, int, int, int,
                          cudaStream_t);
int fwb_shortconv(const void*, int, const float*, const float*, float*, const int*, const int*, const int*,
                  void*, int, int, int, int, int, long long, cudaStream_t);
int fwb_qk_norm_rope(const void*, int, const float*, const float*, const void*, const int*, const int*,
                     const int*, int, int, void*, int, void*, void*, int, int, int, int, int, int, float, int,
                     int, cudaStream_t);
int fwb_attention_simt(const void*, int, const void*, const void*, int, const int*, const int*, const int*,
                       int, int, void*, int, int, int, int, int, int, float, cudaStream_t);
int fwb_attention_prefill_mma(const void*, const void*, const void*, const int*, const int*, const int*,
                              const int*, const int*, int, int, void*, int, int, int, int, int, int, float,
                              cudaStream_t);
int fwb_attention_prefill_tcgen05(const void*, const void*, const void*, const int*, const int*, const int*,
                                  const int*, const int*, int, int, int, void*, int, int, int, int, int, int,
                                  float, cudaStream_t);
int fwb_attention_decode_mma(const void*, const void*, const void*, const int*, const int*, const int*, int,
                             int, int, void*, float*, float*, int, int, int, int, int, int, int, float, int,
                             cudaStream_t);
}

namespace {

constexpr int SM_COUNT = 148;
constexpr int EPI_F32 = 0, EPI_BF16 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3;

// ---- switches (tests turn paths on and off; the Python setters keep both sides equal) ---
enum Option {
    OPT_TENSORCORE = 0,        // tcgen05 products at all
    OPT_FORCED_SPLITS = 1,     // > 0: the split-K factor of decode-sized products is pinned
    OPT_PAIRS = 2,             // prompt-sized products on CTA pairs
    OPT_MID_SIZE_SPLIT = 3,    // 128-token tiles with a split K for narrow products with a long K
    OPT_FUSE_NORM = 4,         // norms folded into the product that follows
    OPT_ADD_IN_PLACE = 5,      // residual sums in the product's epilogue
    OPT_FUSE_ALWAYS = 6,       // ... at every decode-sized token count (default: from 16 tokens)
    OPT_ATTENTION_MMA = 7,     // tensor-core attention kernels at all
    OPT_FORCE_TILED = 8,       // single decode tokens through the tiled attention kernel
    OPT_ATTENTION_TCGEN05 = 9, // prompt portions through the tcgen05 attention kernel
    OPT_MIXED_SPLIT = 10,      // decoding requests at the head of a mixed step through the decode kernel
    OPT_COUNT = 11,
};
int g_option[OPT_COUNT] = {1, 0, 1, 1, 1, 1, 0, 1, 0, 1, 1};
constexpr int FUSE_FROM_TOKENS = 16;
constexpr int CLUSTER_MERGE_CTAS = 1024;

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

// ---- rules of the tensor-core products (kernels/tensorcore.py has the measurements) ------
int decode_tile(int M, int N) {
    if (M <= 16) return 16;
    if (M <= 32 || ceil_div(N, 128) < SM_COUNT) return 32;
    return 64;
}

int splits_for(int M, int N, int K, int accumulators) {
    const int bn = decode_tile(M, N);
    const int tiles = ceil_div(N, 128) * ceil_div(M, bn);
    const int k_blocks = ceil_div(K, 64);
    const int budget = accumulators == 2 ? 256 : 400;
    const int limit = accumulators == 2 ? 4 : 8;
    if (accumulators == 2 && M > 32) return 1;
    int splits = 1;
    while (splits < limit && tiles * splits * 2 <= budget && k_blocks >= splits * 8) splits *= 2;
    return splits;
}

int ring_depth(int M, int N, int splits, int accumulators) {
    const int bn = decode_tile(M, N);
    const int stage = accumulators * 16384 + bn * 128;
    const int ctas = ceil_div(N, 128) * ceil_div(M, bn) * splits;
    const int per_sm = ceil_div(ctas, SM_COUNT) > 1 ? ceil_div(ctas, SM_COUNT) : 1;
    const int fit = ((227 * 1024) / per_sm - 2048) / stage;
    int depth = (accumulators == 2 && bn <= 16) ? 3 : 4;
    if (fit < depth) depth = fit;
    if (depth > 8) depth = 8;
    return depth < 2 ? 2 : depth;
}

int pick_splits(int M, int N, int K) {
    if (g_option[OPT_FORCED_SPLITS] > 0) return M <= 64 ? g_option[OPT_FORCED_SPLITS] : 1;
    if (M > 64) return 1;
    return splits_for(M, N, K, 1);
}

// 65 to 512 tokens: the cost model of kernels/tensorcore.py (mid_size_choice), in hundredths of a
// microsecond.  Returns true for CTA pairs, else sets the token tile and the slices of K.
constexpr int MID_FROM = 65, MID_TO = 512;
bool mid_size_choice(int M, int N, int K, int accumulators, bool pair_ok, int& tile_out, int& splits_out) {
    static const int tiles[3] = {64, 128, 256};
    static const int block_cost[2][3] = {{38, 38, 42}, {63, 58, 84}};
    const int k_blocks = ceil_div(K, 64), feature_tiles = ceil_div(N, 128);
    long best = -1;
    bool pair = false;
    for (int ti = 0; ti < 3; ++ti) {
        const int tile = tiles[ti];
        if (tile == 256 && M <= 128) continue;
        for (int splits = 1; splits <= 4; splits *= 2) {
            if (splits > 1 && (tile > 128 || accumulators == 2 || g_option[OPT_FORCED_SPLITS] > 0 ||
                               k_blocks < 4 * splits))
                continue;
            const int ctas = feature_tiles * ceil_div(M, tile) * splits;
            const int waves = ceil_div(ctas, SM_COUNT);
            if (splits > 1 && waves > 1) continue;
            long cost = 310 + (long)block_cost[accumulators - 1][ti] * ceil_div(k_blocks, splits) * waves;
            if (splits > 1) cost += tile == 128 ? (splits == 2 ? 360 : 260) : (splits == 2 ? 390 : 310);
            if (best < 0 || cost < best) {
                best = cost;
                tile_out = tile;
                splits_out = splits;
            }
        }
    }
    if (pair_ok) {
        const int pairs = ceil_div(N, 256) * ceil_div(M, 256);
        const long cost = 310 + 36L * k_blocks * ceil_div(pairs, SM_COUNT / 2);
        if (cost < best) pair = true;
    }
    return pair;
}

int wave_cut(int M, int F) {
    const int token_tiles = ceil_div(M, 256), feature_tiles = ceil_div(F, 128);
    const int ctas = token_tiles * feature_tiles;
    const int whole = ctas / SM_COUNT, left = ctas - whole * SM_COUNT;
    if (whole == 0 || left == 0 || left > 0.75 * SM_COUNT) return 0;
    const int cut = (whole * SM_COUNT) / token_tiles, rest = feature_tiles - cut;
    if (cut <= 0 || rest <= 0 || rest * ceil_div(M, 128) > SM_COUNT) return 0;
    return cut;
}

int pair_wave_cut(int M, int N) {
    const int slots = SM_COUNT / 2, token_tiles = ceil_div(M, 256);
    const int pairs = ceil_div(N, 512) * token_tiles;
    const int whole = pairs / slots, left = pairs - whole * slots;
    if (whole == 0 || left == 0 || left > 0.75 * slots) return 0;
    const int cut = (whole * slots) / token_tiles, rest = N - cut * 512;
    if (cut <= 0 || rest <= 0 || ceil_div(rest, 256) * token_tiles > slots) return 0;
    return cut;
}

bool tc_accepts(const void* x, const void* w, int M, int K) {
    return g_option[OPT_TENSORCORE] && K % 8 == 0 && K >= 8 && aligned16(x) && aligned16(w) && M <= 65535 * 16;
}

bool normed_accepts(int M, int K, const void* w, int accumulators, int N) {
    if (!(g_option[OPT_TENSORCORE] && g_option[OPT_FUSE_NORM]) || M > 64 || K % 8 || !aligned16(w)) return false;
    if (M < FUSE_FROM_TOKENS && !g_option[OPT_FUSE_ALWAYS]) return false;
    const int splits = g_option[OPT_FORCED_SPLITS] > 0 ? g_option[OPT_FORCED_SPLITS]
                                                        : splits_for(M, N, K, accumulators);
    return ceil_div(K, 64) <= 8 * splits;
}

bool adds_in_place(const void* x, const void* w, int M, int K) {
    return g_option[OPT_ADD_IN_PLACE] && (M >= FUSE_FROM_TOKENS || g_option[OPT_FUSE_ALWAYS]) &&
           tc_accepts(x, w, M, K) && M <= 128;
}

struct Launches {
    int count = 0;
    int status = FWB_OK;
    void add(int s, int n = 1) {
        if (status == FWB_OK && s != FWB_OK) status = s;
        count += n;
    }
    bool ok() const { return status == FWB_OK; }
};

const char* offset(const void* base, long long elements, int bytes) {
    return (const char*)base + elements * bytes;
}

// x [M][K] bf16 @ w[N][K]^T -> out [M][N] (fp32 or bf16); addend fp32 (may be `out` itself).
void tc_gemm(Launches& L, const void* x, const void* w, void* out, int out_bf16, const float* addend, int M,
             int N, int K, cudaStream_t stream) {
    const bool in_place = addend && (const void*)addend == out;
    const int epilogue = addend ? EPI_ADD_F32 : (out_bf16 ? EPI_BF16 : EPI_F32);
    const bool pair_ok = g_option[OPT_PAIRS] && M > 128 && !addend && !in_place && N >= 256;
    int splits = 0, stages = 0, tile_tokens = 0;
    bool pair = false, wide = false;
    if (g_option[OPT_MID_SIZE_SPLIT] && M >= MID_FROM && M <= MID_TO) {
        pair = mid_size_choice(M, N, K, 1, pair_ok, tile_tokens, splits);
    } else if (pair_ok) {
        pair = true;
        wide = ceil_div(N, 256) * ceil_div(M, 256) > SM_COUNT / 2;
    }
    if (pair) {
        const int cut = wide ? pair_wave_cut(M, N) : 0;
        const int out_bytes = out_bf16 ? 2 : 4;
        if (cut) {
            const int first = cut * 512;
            L.add(fwb_gemm_tcgen05_pair(x, w, out, M, first, K, N, N, epilogue, 0, 1, stream));
            L.add(fwb_gemm_tcgen05_pair(x, offset(w, (long long)first * K, 2), (void*)offset(out, first, out_bytes),
                                        M, N - first, K, N - first, N, epilogue, 0, 0, stream));
            return;
        }
        L.add(fwb_gemm_tcgen05_pair(x, w, out, M, N, K, N, N, epilogue, 0, wide ? 1 : 0, stream));
        return;
    }
    if (!splits) splits = pick_splits(M, N, K);
    if (M <= 64) {
        stages = ring_depth(M, N, splits, 1);
        tile_tokens = decode_tile(M, N);
    }
    L.add(fwb_gemm_tcgen05(x, w, out, addend, M, N, K, N, N, epilogue, 0, splits, stages, tile_tokens, -1, stream));
}

// silu(x @ gate^T) * (x @ up^T) for w = [gate rows | up rows] ([2F][K]) -> out [M][F] bf16.
void tc_swiglu(Launches& L, const void* x, const void* w, void* out, int M, int F, int K, cudaStream_t stream) {
    int splits = 1, stages = 0, tile_tokens = 0;
    if (M <= 64) {
        splits = g_option[OPT_FORCED_SPLITS] > 0 ? g_option[OPT_FORCED_SPLITS] : splits_for(M, F, K, 2);
        stages = ring_depth(M, F, splits, 2);
        tile_tokens = decode_tile(M, F);
    }
    const bool mid = g_option[OPT_MID_SIZE_SPLIT] && M >= MID_FROM && M <= MID_TO;
    if (mid) mid_size_choice(M, F, K, 2, false, tile_tokens, splits);
    const int cut = (M > 128 && splits == 1 && !stages && !tile_tokens && !mid) ? wave_cut(M, F) : 0;
    if (cut) {
        const int first = cut * 128;
        L.add(fwb_gemm_tcgen05(x, w, out, nullptr, M, first, K, 2 * F, F, EPI_SWIGLU_BF16, F, 1, 0, 256, -1, stream));
        L.add(fwb_gemm_tcgen05(x, offset(w, (long long)first * K, 2), (void*)offset(out, first, 2), nullptr, M,
                               F - first, K, 2 * F - first, F, EPI_SWIGLU_BF16, F, 1, 0, 128, -1, stream));
        return;
    }
    L.add(fwb_gemm_tcgen05(x, w, out, nullptr, M, F, K, 2 * F, F, EPI_SWIGLU_BF16, F, splits, stages, tile_tokens,
                           -1, stream));
}

// The product the model uses, from activations that are already there (kernels/ops.py: linear).
void linear(Launches& L, const void* x, int x_bf16, const void* w, int w_bf16, void* out, int out_bf16,
            const float* addend, int M, int N, int K, cudaStream_t stream) {
    if (w_bf16 && x_bf16 && tc_accepts(x, w, M, K) && !(addend && out_bf16)) {
        tc_gemm(L, x, w, out, out_bf16, addend, M, N, K, stream);
        return;
    }
    L.add(fwb_gemm_simt(x, x_bf16, w, w_bf16, out, out_bf16, addend, M, N, K, K, N, stream));
}

// ---- operations of a plan -----------------------------------------------------------------
enum OpKind { OP_EMBED, OP_NORM_LINEAR, OP_LINEAR_RESIDUAL, OP_SHORTCONV, OP_QK_ROPE, OP_ATTENTION, OP_SOFTCAP };
// ids of the step's int32 arrays (their offsets into the uploaded block come with every step)
enum MetaArray { META_TOKEN_IDS, META_POSITIONS, META_TOK_SEG, META_SEG_START, META_SEG_SLOT, META_SEG_POS0,
                 META_LOGIT_ROWS, META_TILE_SEG_A, META_TILE_TOK0_A, META_TILE_SEG_B, META_TILE_TOK0_B,
                 META_PATCH_DST, META_PATCH_SRC, META_BLOCK_TABLE0 };
constexpr int MAX_GROUPS = 8;
constexpr int META_COUNT = META_BLOCK_TABLE0 + MAX_GROUPS;

struct Op {
    int kind = 0;
    // buffers (device pointers fixed when the plan is built)
    void* in = nullptr;          // activations in
    void* out = nullptr;         // activations out
    float* x = nullptr;          // the fp32 residual stream
    float* delta = nullptr;      // a residual delta not yet added (written or read, see `pending`)
    void* scratch = nullptr;     // normalised rows; gate|up of an unfused SwiGLU after them
    void* scratch2 = nullptr;
    const void* w = nullptr;     // matrix
    const float* v0 = nullptr;   // norm weight | taps | q norm
    const float* v1 = nullptr;   // bias | k norm
    const void* table = nullptr; // rotary table | embedding table
    void* pool_k = nullptr;      // K pages | conv state
    void* pool_v = nullptr;
    float* part_o = nullptr;     // scratch of the split decode attention
    float* part_ml = nullptr;
    int* flag = nullptr;         // the embedding's bad-token flag
    int w_bf16 = 0, epilogue = 0, on_logit_rows = 0, out_bf16 = 0;
    int N = 0, K = 0;            // product: out features, in features (SwiGLU: N = F)
    int nh = 0, nkv = 0, hd = 0, rot = 0, pairing = 0, use_norm = 0, window = 0, group = 0, taps = 0;
    int page_size = 0, num_pages = 0, vocab = 0;
    long long stride = 0;
    float eps = 0.0f, scale = 1.0f;
};

constexpr int STAGING = 4;

struct Plan {
    int act_bf16 = 1;
    std::vector<Op> ops;
    int failed_op = -1;
    long long launches = 0;
    // pinned staging for the step's int32 arrays: the host may prepare step k+1 while the copy of
    // step k is still in flight, so a small ring, each slot guarded by an event
    int* staging[STAGING] = {};
    cudaEvent_t copied[STAGING] = {};
    size_t staging_words = 0;
    int turn = 0;
};

int stage(Plan& plan, const int* words, size_t count, int** pinned) {
    if (count > plan.staging_words) {
        cudaError_t e = cudaDeviceSynchronize();                    // nothing reads the old slots any more
        if (e != cudaSuccess) return (int)e;
        for (int i = 0; i < STAGING; ++i) {
            if (plan.staging[i]) cudaFreeHost(plan.staging[i]);
            plan.staging[i] = nullptr;
        }
        size_t grown = plan.staging_words ? plan.staging_words : 4096;
        while (grown < count) grown *= 2;
        for (int i = 0; i < STAGING; ++i) {
            e = cudaHostAlloc((void**)&plan.staging[i], grown * sizeof(int), cudaHostAllocDefault);
            if (e != cudaSuccess) return (int)e;
            if (!plan.copied[i]) {
                e = cudaEventCreateWithFlags(&plan.copied[i], cudaEventDisableTiming);
                if (e != cudaSuccess) return (int)e;
            }
        }
        plan.staging_words = grown;
    }
    const int turn = plan.turn;
    plan.turn = (turn + 1) % STAGING;
    cudaError_t e = cudaEventSynchronize(plan.copied[turn]);       // the copy that last read this slot is done
    if (e != cudaSuccess) return (int)e;
    memcpy(plan.staging[turn], words, count * sizeof(int));
    *pinned = plan.staging[turn];
    return turn;
}

}  // namespace

// One step's batch, filled by the caller for every run.
struct FwbStep {
    const int* meta_host;       // the int32 arrays of the step, packed, in ordinary host memory
    int* meta_dev;              // where they go on the device
    int meta_words;
    int upload;                 // 1: copy meta_host to meta_dev first (through pinned staging that the
                                // plan keeps); 0: the caller has put the arrays on the device itself
    int offsets[META_COUNT];    // where each array starts inside the block (words)
    int T, S, R;                // tokens, segments, wanted logit rows
    int width[MAX_GROUPS];      // block-table width of each page group
    int max_segment;            // the longest segment
    int leading_singles;        // one-token segments at the head of the batch
    int tokens_per_tile[2];     // of the two attention tile lists (A: 128 rows, B: 64 rows) ...
    int n_tiles[2];             // ... and how many tiles each holds
    void* logits;               // [R][vocab] fp32 out
    const int* patch_source;    // n_patch > 0: token ids on the device (the sampler's output of the step
    int n_patch;                // before) that go into token_ids[patch_dst[i]] from patch_source[patch_src[i]]
};

namespace {

const int* meta(const FwbStep& step, int id) { return step.meta_dev + step.offsets[id]; }

void run_norm_linear(Launches& L, const Op& op, const FwbStep& step, bool& pending, int act_bf16,
                     cudaStream_t stream) {
    const int M = op.on_logit_rows ? step.R : step.T;
    if (M <= 0) return;
    const int* rows = op.on_logit_rows ? meta(step, META_LOGIT_ROWS) : nullptr;
    void* out = op.on_logit_rows && op.out == nullptr ? step.logits : op.out;
    const bool swiglu = op.epilogue == EPI_SWIGLU_BF16;
    const int accumulators = swiglu ? 2 : 1;
    if (!pending && op.w_bf16 && act_bf16 && normed_accepts(M, op.K, op.w, accumulators, op.N)) {
        // the norm, the product (both products and silu(g)*u) in one kernel
        int splits, stages, tile_tokens;
        if (swiglu) {
            splits = g_option[OPT_FORCED_SPLITS] > 0 ? g_option[OPT_FORCED_SPLITS] : splits_for(M, op.N, op.K, 2);
        } else {
            splits = pick_splits(M, op.N, op.K);
        }
        stages = ring_depth(M, op.N, splits, accumulators);
        tile_tokens = decode_tile(M, op.N);
        L.add(fwb_gemm_tcgen05_normed(op.x, op.v0, rows, op.eps, op.w, out, M, op.N, op.K,
                                      swiglu ? 2 * op.N : op.N, op.N, op.epilogue, swiglu ? op.N : 0, splits,
                                      stages, tile_tokens, stream));
        return;
    }
    // the norm kernel first (it also adds a pending delta into the residual), into scratch rows
    const int h_bf16 = op.w_bf16 ? 1 : 0;
    L.add(fwb_rmsnorm(op.x, pending ? op.delta : nullptr, op.v0, op.scratch, h_bf16, rows, M, op.K, op.eps, stream));
    pending = false;
    if (swiglu) {
        if (op.w_bf16 && tc_accepts(op.scratch, op.w, M, op.K)) {
            tc_swiglu(L, op.scratch, op.w, out, M, op.N, op.K, stream);
        } else {
            linear(L, op.scratch, h_bf16, op.w, op.w_bf16, op.scratch2, act_bf16, nullptr, M, 2 * op.N, op.K, stream);
            L.add(fwb_silu_mul(op.scratch2, act_bf16, out, act_bf16, M, op.N, stream));
        }
        return;
    }
    linear(L, op.scratch, h_bf16, op.w, op.w_bf16, out, op.out_bf16, nullptr, M, op.N, op.K, stream);
}

void run_linear_residual(Launches& L, const Op& op, const FwbStep& step, bool& pending, int act_bf16,
                         cudaStream_t stream) {
    const int M = step.T;
    if (op.w_bf16 && act_bf16 && adds_in_place(op.in, op.w, M, op.K)) {
        tc_gemm(L, op.in, op.w, op.x, 0, op.x, M, op.N, op.K, stream);      // x += in @ w^T in the epilogue
        pending = false;
        return;
    }
    linear(L, op.in, act_bf16, op.w, op.w_bf16, op.delta, 0, nullptr, M, op.N, op.K, stream);
    pending = true;
}

void decode_splits(int n_tokens, int n_kv, int max_tiles, int head_dim, int& splits, int& tiles_per_split,
                   bool& in_cluster) {
    // the same rule as kernels/attention.py: decode_splits (the measurements are quoted there): as many
    // slices as keep every CTA resident at once, of 8 to 128 tiles; else the fewest that fill the SMs'
    // last round to 85 %
    const long pairs = (long)n_tokens * n_kv > 1 ? (long)n_tokens * n_kv : 1;
    const long resident = (long)SM_COUNT * (head_dim <= 64 ? 5 : 3);
    int least = 1;
    while (least * 128 < max_tiles && least < 64) least *= 2;
    int choice = 0;
    for (int s = least; s <= 64 && pairs * s <= resident && (s == least || s * 8 <= max_tiles); s *= 2) choice = s;
    if (!choice)
        for (int s = least; s <= 64; s *= 2) {
            const long ctas = pairs * s;
            const long rounds = (ctas + resident - 1) / resident;
            if ((double)ctas >= 0.85 * (double)(rounds * resident)) {
                choice = s;
                break;
            }
        }
    if (!choice) choice = least;
    tiles_per_split = ceil_div(max_tiles, choice);
    splits = ceil_div(max_tiles, tiles_per_split);
    in_cluster = splits > 1 && splits <= 8 && pairs * splits <= CLUSTER_MERGE_CTAS;
}

void run_decode_attention(Launches& L, const Op& op, const FwbStep& step, const int* table, int width,
                          int n_tokens, cudaStream_t stream) {
    int splits, tiles_per_split;
    bool in_cluster;
    decode_splits(n_tokens, op.nkv, width, op.hd, splits, tiles_per_split, in_cluster);
    const bool merged_in_kernel = in_cluster && splits > 1 && splits <= 8;
    const bool scratch = splits > 1 && !merged_in_kernel;
    L.add(fwb_attention_decode_mma(op.in, op.pool_k, op.pool_v, meta(step, META_POSITIONS), meta(step, META_TOK_SEG),
                                   table, width, op.page_size, op.num_pages, op.out, scratch ? op.part_o : nullptr,
                                   scratch ? op.part_ml : nullptr, n_tokens, op.nh, op.nkv, op.hd, splits,
                                   tiles_per_split, op.window, op.scale, merged_in_kernel ? 1 : 0, stream),
          scratch ? 2 : 1);
}

void run_attention(Launches& L, const Op& op, const FwbStep& step, int act_bf16, cudaStream_t stream) {
    const int T = step.T;
    const int width = step.width[op.group];
    const int* table = meta(step, META_BLOCK_TABLE0 + op.group);
    const bool mma_shape = op.nh % op.nkv == 0 && op.nh / op.nkv <= 16 && op.hd >= 16 && op.hd <= 128 &&
                           op.hd % 16 == 0 && op.page_size == 64;
    if (g_option[OPT_ATTENTION_MMA] && act_bf16 && mma_shape) {
        const bool force_tiled = g_option[OPT_FORCE_TILED] != 0;
        if (step.max_segment == 1 && !force_tiled) {
            run_decode_attention(L, op, step, table, width, T, stream);
            return;
        }
        const int group = op.nh / op.nkv;
        int first = 0;
        if (step.leading_singles && !force_tiled && g_option[OPT_MIXED_SPLIT]) {
            first = step.leading_singles;
            run_decode_attention(L, op, step, table, width, first, stream);
        }
        const bool tcgen05_shape = (op.hd == 64 || op.hd == 128) && op.page_size == 64 && op.nkv > 0 &&
                                   op.nh % op.nkv == 0 && group <= 128;
        // tile list A holds 128-row tiles, list B 64-row tiles; both skip the leading singles
        // exactly when the decode kernel took them
        if (g_option[OPT_ATTENTION_TCGEN05] && !force_tiled && tcgen05_shape && 2 * step.max_segment * group >= 128) {
            L.add(fwb_attention_prefill_tcgen05(op.in, op.pool_k, op.pool_v, meta(step, META_POSITIONS),
                                                meta(step, META_SEG_START), meta(step, META_TILE_SEG_A),
                                                meta(step, META_TILE_TOK0_A), table, width, op.page_size,
                                                op.num_pages, op.out, step.n_tiles[0], op.nh, op.nkv, op.hd,
                                                step.tokens_per_tile[0], op.window, op.scale, stream));
            return;
        }
        L.add(fwb_attention_prefill_mma(op.in, op.pool_k, op.pool_v, meta(step, META_POSITIONS),
                                        meta(step, META_SEG_START), meta(step, META_TILE_SEG_B),
                                        meta(step, META_TILE_TOK0_B), table, width, op.page_size, op.out,
                                        step.n_tiles[1], op.nh, op.nkv, op.hd, step.tokens_per_tile[1], op.window,
                                        op.scale, stream));
        return;
    }
    L.add(fwb_attention_simt(op.in, act_bf16, op.pool_k, op.pool_v, act_bf16, meta(step, META_POSITIONS),
                             meta(step, META_TOK_SEG), table, width, op.page_size, op.out, act_bf16, T, op.nh,
                             op.nkv, op.hd, op.window, op.scale, stream));
}

}  // namespace

// ---- the C interface ------------------------------------------------------------------------
FWB_API int fwb_set_option(int option, int value) {
    if (option < 0 || option >= OPT_COUNT) return FWB_BAD_ARGUMENT;
    g_option[option] = value;
    return FWB_OK;
}

FWB_API int fwb_get_option(int option) {
    return option < 0 || option >= OPT_COUNT ? -1 : g_option[option];
}

FWB_API void* fwb_plan_create(int act_bf16) {
    Plan* plan = new Plan();
    plan->act_bf16 = act_bf16 ? 1 : 0;
    return plan;
}

FWB_API int fwb_plan_destroy(void* handle) {
    Plan* plan = static_cast<Plan*>(handle);
    if (!plan) return FWB_OK;
    for (int i = 0; i < STAGING; ++i) {
        if (plan->copied[i]) {
            cudaEventSynchronize(plan->copied[i]);
            cudaEventDestroy(plan->copied[i]);
        }
        if (plan->staging[i]) cudaFreeHost(plan->staging[i]);
    }
    delete plan;
    return FWB_OK;
}

FWB_API int fwb_plan_size(void* handle) {
    return handle ? (int)static_cast<Plan*>(handle)->ops.size() : -1;
}

// x[T][H] = scale * table[token_ids]
FWB_API int fwb_plan_embed(void* handle, const void* table, int table_bf16, float* x, int H, int vocab,
                           float scale, int* bad_flag) {
    if (!handle || !table || !x) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_EMBED;
    op.table = table;
    op.w_bf16 = table_bf16;
    op.x = x;
    op.K = H;
    op.vocab = vocab;
    op.scale = scale;
    op.flag = bad_flag;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

// out = epilogue( rmsnorm(x [+ delta, if one is pending]) @ w^T ).  epilogue 0: fp32 [.][N], 1: bf16 [.][N],
// 3: SwiGLU, w = [gate | up] ([2N][K]) -> [.][N] in the activation dtype.  on_logit_rows: only the rows
// the step wants logits at (then out may be null: the step's logits buffer).  scratch: [rows][K] in
// the matrix dtype; scratch2: [rows][2N] activations (SwiGLU without the fused kernel only).
FWB_API int fwb_plan_norm_linear(void* handle, float* x, float* delta, const float* norm_w, float eps,
                                 const void* w, int w_bf16, int N, int K, int epilogue, int on_logit_rows,
                                 void* out, void* scratch, void* scratch2) {
    if (!handle || !x || !norm_w || !w || !scratch || N <= 0 || K <= 0) return FWB_BAD_ARGUMENT;
    if (!out && !on_logit_rows) return FWB_BAD_ARGUMENT;
    if (epilogue != EPI_F32 && epilogue != EPI_BF16 && epilogue != EPI_SWIGLU_BF16) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_NORM_LINEAR;
    op.x = x;
    op.delta = delta;
    op.v0 = norm_w;
    op.eps = eps;
    op.w = w;
    op.w_bf16 = w_bf16;
    op.N = N;
    op.K = K;
    op.epilogue = epilogue;
    op.out_bf16 = epilogue == EPI_BF16;
    op.on_logit_rows = on_logit_rows;
    op.out = out;
    op.scratch = scratch;
    op.scratch2 = scratch2;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

// x += in @ w^T: in the product's epilogue when the step's size has that form, else the product
// goes to `delta` and stays pending until the next norm (or the end of the plan) adds it.
FWB_API int fwb_plan_linear_residual(void* handle, const void* in, const void* w, int w_bf16, int N, int K,
                                     float* x, float* delta) {
    if (!handle || !in || !w || !x || !delta || N <= 0 || K <= 0) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_LINEAR_RESIDUAL;
    op.in = const_cast<void*>(in);
    op.w = w;
    op.w_bf16 = w_bf16;
    op.N = N;
    op.K = K;
    op.x = x;
    op.delta = delta;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

FWB_API int fwb_plan_shortconv(void* handle, const void* p, const float* taps, const float* bias, float* state,
                               long long slot_stride, void* z, int H, int L) {
    if (!handle || !p || !taps || !state || !z) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_SHORTCONV;
    op.in = const_cast<void*>(p);
    op.v0 = taps;
    op.v1 = bias;
    op.pool_k = state;
    op.stride = slot_stride;
    op.out = z;
    op.K = H;
    op.taps = L;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

FWB_API int fwb_plan_qk_rope(void* handle, const void* qkv, const float* q_norm, const float* k_norm,
                             const void* table, void* q_out, void* k_pool, void* v_pool, int group,
                             int page_size, int nh, int nkv_in, int hd, int rot, int pairing, float eps,
                             int use_norm) {
    if (!handle || !qkv || !table || !q_out || group < 0 || group >= MAX_GROUPS) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_QK_ROPE;
    op.in = const_cast<void*>(qkv);
    op.v0 = q_norm;
    op.v1 = k_norm;
    op.table = table;
    op.out = q_out;
    op.pool_k = k_pool;
    op.pool_v = v_pool;
    op.group = group;
    op.page_size = page_size;
    op.nh = nh;
    op.nkv = nkv_in;
    op.hd = hd;
    op.rot = rot;
    op.pairing = pairing;
    op.eps = eps;
    op.use_norm = use_norm;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

FWB_API int fwb_plan_attention(void* handle, const void* q, void* k_pool, void* v_pool, void* out, int group,
                               int page_size, int num_pages, int nh, int nkv, int hd, int window, float scale,
                               float* part_o, float* part_ml) {
    if (!handle || !q || !k_pool || !v_pool || !out || group < 0 || group >= MAX_GROUPS) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_ATTENTION;
    op.in = const_cast<void*>(q);
    op.pool_k = k_pool;
    op.pool_v = v_pool;
    op.out = out;
    op.group = group;
    op.page_size = page_size;
    op.num_pages = num_pages;
    op.nh = nh;
    op.nkv = nkv;
    op.hd = hd;
    op.window = window;
    op.scale = scale;
    op.part_o = part_o;
    op.part_ml = part_ml;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

FWB_API int fwb_plan_softcap(void* handle, float cap, int vocab) {
    if (!handle || !(cap > 0.0f)) return FWB_BAD_ARGUMENT;
    Op op;
    op.kind = OP_SOFTCAP;
    op.scale = cap;
    op.vocab = vocab;
    static_cast<Plan*>(handle)->ops.push_back(op);
    return FWB_OK;
}

// Run one step.  Returns 0, or the status of the first launcher that refused or failed
// (`fwb_plan_failed_op` then says which operation of the plan it was).  `launches` (may be null)
// receives the number of kernels launched.
FWB_API int fwb_plan_run(void* handle, const void* step_ptr, int* launches, cudaStream_t stream) {
    if (!handle || !step_ptr) return FWB_BAD_ARGUMENT;
    Plan& plan = *static_cast<Plan*>(handle);
    const FwbStep& step = *static_cast<const FwbStep*>(step_ptr);
    if (step.T <= 0 || step.S <= 0 || !step.meta_dev) return FWB_BAD_ARGUMENT;
    if (step.upload) {
        if (!step.meta_host || step.meta_words <= 0) return FWB_BAD_ARGUMENT;
        int* pinned = nullptr;
        const int turn = stage(plan, step.meta_host, (size_t)step.meta_words, &pinned);
        if (turn < 0 || !pinned) return turn < 0 ? turn : FWB_BAD_ARGUMENT;
        cudaError_t e = cudaMemcpyAsync(step.meta_dev, pinned, sizeof(int) * (size_t)step.meta_words,
                                        cudaMemcpyHostToDevice, stream);
        if (e == cudaSuccess) e = cudaEventRecord(plan.copied[turn], stream);
        if (e != cudaSuccess) return (int)e;
    }
    Launches L;
    if (step.n_patch > 0) {
        if (!step.patch_source) return FWB_BAD_ARGUMENT;
        L.add(fwb_patch_tokens(step.meta_dev + step.offsets[META_TOKEN_IDS], meta(step, META_PATCH_DST),
                               step.patch_source, meta(step, META_PATCH_SRC), step.n_patch, stream));
    }
    bool pending = false;                   // a delta written by the last product, not yet in x
    const int act_bf16 = plan.act_bf16;
    plan.failed_op = -1;
    for (size_t i = 0; i < plan.ops.size() && L.ok(); ++i) {
        const Op& op = plan.ops[i];
        switch (op.kind) {
            case OP_EMBED:
                L.add(fwb_embed(op.table, op.w_bf16, meta(step, META_TOKEN_IDS), op.x, step.T, op.K, op.vocab,
                                op.flag, op.scale, stream));
                break;
            case OP_NORM_LINEAR:
                run_norm_linear(L, op, step, pending, act_bf16, stream);
                break;
            case OP_LINEAR_RESIDUAL:
                run_linear_residual(L, op, step, pending, act_bf16, stream);
                break;
            case OP_SHORTCONV:
                L.add(fwb_shortconv(op.in, act_bf16, op.v0, op.v1, (float*)op.pool_k, meta(step, META_SEG_START),
                                    meta(step, META_SEG_SLOT), meta(step, META_TOK_SEG), op.out, act_bf16, step.T,
                                    step.S, op.K, op.taps, op.stride, stream));
                break;
            case OP_QK_ROPE:
                L.add(fwb_qk_norm_rope(op.in, act_bf16, op.v0, op.v1, op.table, meta(step, META_POSITIONS),
                                       meta(step, META_TOK_SEG),
                                       op.nkv ? meta(step, META_BLOCK_TABLE0 + op.group) : nullptr,
                                       op.nkv ? step.width[op.group] : 0, op.nkv ? op.page_size : 0, op.out, act_bf16,
                                       op.pool_k, op.pool_v, act_bf16, step.T, op.nh, op.nkv, op.hd, op.rot, op.eps,
                                       op.use_norm, op.pairing, stream));
                break;
            case OP_ATTENTION:
                run_attention(L, op, step, act_bf16, stream);
                break;
            case OP_SOFTCAP:
                if (step.R > 0)
                    L.add(fwb_softcap((float*)step.logits, (long long)step.R * op.vocab, op.scale, stream));
                break;
            default:
                L.add(FWB_BAD_ARGUMENT, 0);
        }
        if (!L.ok()) plan.failed_op = (int)i;
    }
    plan.launches += L.count;
    if (launches) *launches = L.count;
    return L.status;
}

FWB_API int fwb_plan_failed_op(void* handle) {
    return handle ? static_cast<Plan*>(handle)->failed_op : -1;
}
