// bfloat16 matrix product for prompt-sized steps on CTA PAIRS (tcgen05 cta_group::2), sm_100a.
//
//   Y[t][f] = sum_k X[t][k] * W[f][k]
//
// Two CTAs of a cluster work on one tile of 256 features x 256 tokens per accumulator: each CTA
// holds 128 of the features (its half of operand A) and 128 of the tokens (its half of operand
// B) in shared memory, the leader CTA issues one tcgen05.mma.cta_group::2 (M = 256, N = 256,
// K = 16) that reads both halves of both operands, and each CTA's tensor memory receives the
// accumulator rows of its own 128 features for all 256 tokens.  Against the single-CTA kernel a
// CTA loads and reads half of the activations per MMA: that kernel's tensor pipe waits on shared-
// memory bandwidth (TMA fill plus operand reads exceed 128 B/clk), this one's does not.
//
// Per stage: both CTAs' producers fill their own shared memory by TMA (plain tile loads of this
// GPU's memory, one destination each) whose completion bytes are all counted on the LEADER's
// "full" barrier (the cta_group::2 form of the load allows the barrier to live in the pair's other
// CTA); the leader's MMA thread waits for that one barrier, issues the MMAs and commits with a
// cluster-wide arrive that frees the stage in both CTAs.  The last commit raises "accumulator ready" in both CTAs, whose epilogue
// warps then read their own tensor memory.
//
// Accumulators per CTA: 1 (plain), or 2 = SwiGLU (gate rows f, up rows F + f -> silu(g) * u) or
// wide (a second block of 256 features).  Launched with programmatic stream serialisation like
// every kernel of the library; every mbarrier wait is bounded.
#include "tcgen05.cuh"

using namespace fwb;
using namespace fwb::tc5;

namespace {

constexpr int EPI_WARPS = 16;          // four per quarter of the TMEM lanes
constexpr int THREADS = 64 + 32 * EPI_WARPS;   // warp 0 producer, warp 1 MMA, then the epilogue warps
constexpr int BN = 256;                // tokens per tile (128 per CTA in shared memory)
constexpr int HALF_N = BN / 2;
constexpr int PAIR_M = 2 * BM;         // features per pair and accumulator
constexpr int SMEM_BUDGET = 225 * 1024;

enum PairEpilogue : int { PAIR_F32 = 0, PAIR_BF16 = 1, PAIR_SWIGLU_BF16 = 3, PAIR_F32_WIDE = 4, PAIR_BF16_WIDE = 5 };
constexpr bool pair_wide(int epi) { return epi == PAIR_F32_WIDE || epi == PAIR_BF16_WIDE; }
constexpr int pair_accumulators(int epi) { return (epi == PAIR_SWIGLU_BF16 || pair_wide(epi)) ? 2 : 1; }

template <int NACC>
struct PairTile {
    static constexpr int A_BYTES = BM * BK * 2;             // 16 KiB: this CTA's 128 features
    static constexpr int B_BYTES = HALF_N * BK * 2;         // 16 KiB: this CTA's 128 tokens
    static constexpr int STAGE_BYTES = NACC * A_BYTES + B_BYTES;
    static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES > 8 ? 8 : SMEM_BUDGET / STAGE_BYTES;
    static constexpr int COLS = BN * NACC;
    static constexpr int TMEM_COLS = COLS <= 256 ? 256 : 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512;
};

struct PairParams {
    void* y;
    int M, N, K, ldy;
    int up_row_offset;
    int token_tiles;
    int* status;
};

__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive (once all MMAs issued so far have completed) on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"(mask)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* holder, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// One arrival on the barrier at the same offset in CTA `rank` of the cluster.
// Cluster-window address of `ptr`'s offset in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_addr(const void* ptr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(ptr)), "r"(rank));
    return remote;
}
// TMA tile load into this CTA's shared memory whose bytes are counted on a barrier that may live
// in the other CTA of the pair (given by its cluster-window address).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 const PairParams prm) {
    constexpr int NACC = pair_accumulators(EPI);
    constexpr bool WIDE = pair_wide(EPI);
    using T = PairTile<NACC>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + T::STAGES * T::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + T::STAGES;
    uint64_t* acc_bar = empty_bar + T::STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                // 0 = leader
    const int pair = blockIdx.x >> 1;
    // token tiles are the fast index: pairs that run together share weight tiles in L2
    const int tok0 = (pair % prm.token_tiles) * BN;
    const int feat_pair0 = (pair / prm.token_tiles) * (WIDE ? 2 * PAIR_M : PAIR_M);
    const int feat0 = feat_pair0 + (int)rank * BM;                       // this CTA's rows, accumulator 0
    const int feat1 = WIDE ? feat0 + PAIR_M : prm.up_row_offset + feat0;  // accumulator 1
    const int my_tok0 = tok0 + (int)rank * HALF_N;                       // this CTA's half of operand B
    const int n_kb = (prm.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T::STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_holder, T::TMEM_COLS);   // the same warp in both CTAs
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // both CTAs' barriers exist before anybody signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // every load of the pair reports to the leader's barrier of its stage; the leader arms it
            // with the bytes of both CTAs
            const int ahead = n_kb < T::STAGES ? n_kb : T::STAGES;
            for (int i = 0; i < ahead; ++i) {            // weights first: nothing in the stream writes them
                uint8_t* stage = tiles + (size_t)i * T::STAGE_BYTES;
                const uint32_t bar = cluster_addr(&full_bar[i], 0);
                if (rank == 0) mbar_expect_tx(&full_bar[i], 2 * T::STAGE_BYTES);
                tma_load_2d_pair(stage, &map_w, bar, i * BK, feat0);
                if (NACC == 2) tma_load_2d_pair(stage + T::A_BYTES, &map_w, bar, i * BK, feat1);
            }
            pdl_wait();
            for (int i = 0; i < ahead; ++i)
                tma_load_2d_pair(tiles + (size_t)i * T::STAGE_BYTES + NACC * T::A_BYTES, &map_x,
                                 cluster_addr(&full_bar[i], 0), i * BK, my_tok0);
            for (int i = ahead; i < n_kb; ++i) {
                const int s = i % T::STAGES;
                const uint32_t round = i / T::STAGES;
                if (!mbar_wait(&empty_bar[s], (round - 1) & 1, abort_flag, 11, prm.status)) break;
                uint8_t* stage = tiles + (size_t)s * T::STAGE_BYTES;
                const uint32_t bar = cluster_addr(&full_bar[s], 0);
                if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * T::STAGE_BYTES);
                tma_load_2d_pair(stage, &map_w, bar, i * BK, feat0);
                if (NACC == 2) tma_load_2d_pair(stage + T::A_BYTES, &map_w, bar, i * BK, feat1);
                tma_load_2d_pair(stage + NACC * T::A_BYTES, &map_x, bar, i * BK, my_tok0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_mn(PAIR_M, BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % T::STAGES;
                ok = mbar_wait_cluster(&full_bar[s], (i / T::STAGES) & 1, abort_flag, 13, prm.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t stage = smem_u32(tiles + (size_t)s * T::STAGE_BYTES);
                const uint64_t b_desc = make_smem_desc(stage + NACC * T::A_BYTES);
#pragma unroll
                for (int a = 0; a < NACC; ++a) {
                    const uint64_t a_desc = make_smem_desc(stage + a * T::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem_base + a * BN, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                       (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit_pair(&empty_bar[s]);         // frees the stage in both CTAs
            }
            umma_commit_pair(acc_bar);                   // accumulators complete, in both CTAs
        }
    }
    __syncwarp();

    // ---------------------------------------------------------------- epilogue (both CTAs)
    if (warp >= 2) {
        pdl_wait();
        bool ready = n_kb > 0 ? mbar_wait(acc_bar, 0, abort_flag, 15, prm.status) : true;
        ready = ready && !*abort_flag;
        ready = __all_sync(0xffffffffu, ready);
        tc_fence_after();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int f = feat0 + row;
        if (ready) {
            // the warps of a quarter of the TMEM lanes share the 256 token columns
            constexpr int PER_GROUP = BN / (EPI_WARPS / 4);
            const int c_begin = ((warp - 2) >> 2) * PER_GROUP;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_begin + PER_GROUP; c0 += 16) {
                float g[16], u[16];
                if (n_kb > 0) {
                    tmem_ld16(lane_addr + c0, g);
                    if (NACC == 2) tmem_ld16(lane_addr + BN + c0, u);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int t = tok0 + c0 + j;
                    if (t >= prm.M || f >= prm.N) continue;
                    const size_t at = (size_t)t * prm.ldy + f;
                    if (EPI == PAIR_F32) reinterpret_cast<float*>(prm.y)[at] = g[j];
                    else if (EPI == PAIR_BF16) reinterpret_cast<__nv_bfloat16*>(prm.y)[at] = __float2bfloat16_rn(g[j]);
                    else if (EPI == PAIR_SWIGLU_BF16)
                        reinterpret_cast<__nv_bfloat16*>(prm.y)[at] = __float2bfloat16_rn(silu_fast(g[j]) * u[j]);
                    else if (EPI == PAIR_F32_WIDE) {
                        reinterpret_cast<float*>(prm.y)[at] = g[j];
                        if (f + PAIR_M < prm.N) reinterpret_cast<float*>(prm.y)[at + PAIR_M] = u[j];
                    } else {
                        reinterpret_cast<__nv_bfloat16*>(prm.y)[at] = __float2bfloat16_rn(g[j]);
                        if (f + PAIR_M < prm.N)
                            reinterpret_cast<__nv_bfloat16*>(prm.y)[at + PAIR_M] = __float2bfloat16_rn(u[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither CTA frees tensor memory or leaves while the other still works
    if (warp == 1) tmem_dealloc_pair(tmem_base, T::TMEM_COLS);
}

template <int EPI>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const PairParams& prm, int pairs,
           cudaStream_t stream) {
    using T = PairTile<pair_accumulators(EPI)>;
    auto kernel = gemm_pair_kernel<EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * pairs, 1, 1);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = T::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, map_w, map_x, prm);
    return e == cudaSuccess ? fwb_launch_status() : (int)e;
}

}  // namespace

// X: [M][K] bf16, W: [w_rows][K] bf16, Y: [M][ldy] fp32 (epilogue 0) or bf16 (1, 3).
// epilogue: 0 = fp32, 1 = bf16, 3 = SwiGLU (N = F, up rows at up_row_offset).  `wide` gives a
// CTA pair two blocks of 256 features (plain epilogues only).  K % 8 == 0, bases 16-byte aligned.
FWB_API int fwb_gemm_tcgen05_pair(const void* X, const void* W, void* Y, int M, int N, int K, int w_rows,
                                  int ldy, int epilogue, int up_row_offset, int wide, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return FWB_OK;
    if (!X || !W || !Y || K <= 0 || ldy < N) return FWB_BAD_ARGUMENT;
    if ((K & 7) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return FWB_UNSUPPORTED;
    if (epilogue == PAIR_SWIGLU_BF16 && (up_row_offset < N || w_rows < up_row_offset + N)) return FWB_BAD_ARGUMENT;
    if (epilogue != PAIR_SWIGLU_BF16 && w_rows < N) return FWB_BAD_ARGUMENT;
    if (epilogue == PAIR_F32 && wide) epilogue = PAIR_F32_WIDE;
    else if (epilogue == PAIR_BF16 && wide) epilogue = PAIR_BF16_WIDE;
    PairParams prm;
    prm.y = Y;
    prm.M = M;
    prm.N = N;
    prm.K = K;
    prm.ldy = ldy;
    prm.up_row_offset = up_row_offset;
    prm.token_tiles = (M + BN - 1) / BN;
    prm.status = status_word();
    const int features_per_pair = pair_wide(epilogue) ? 2 * PAIR_M : PAIR_M;
    const long pairs = (long)prm.token_tiles * ((N + features_per_pair - 1) / features_per_pair);
    if (pairs * 2 > 2147483647L) return FWB_TOO_LARGE;
    CUtensorMap map_w, map_x;
    if (!make_map(&map_w, W, w_rows, K, BM)) return FWB_UNSUPPORTED;
    if (!make_map(&map_x, X, M, K, HALF_N)) return FWB_UNSUPPORTED;
    switch (epilogue) {
        case PAIR_F32: return launch<PAIR_F32>(map_w, map_x, prm, (int)pairs, stream);
        case PAIR_BF16: return launch<PAIR_BF16>(map_w, map_x, prm, (int)pairs, stream);
        case PAIR_SWIGLU_BF16: return launch<PAIR_SWIGLU_BF16>(map_w, map_x, prm, (int)pairs, stream);
        case PAIR_F32_WIDE: return launch<PAIR_F32_WIDE>(map_w, map_x, prm, (int)pairs, stream);
        case PAIR_BF16_WIDE: return launch<PAIR_BF16_WIDE>(map_w, map_x, prm, (int)pairs, stream);
        default: return FWB_UNSUPPORTED;
    }
}
