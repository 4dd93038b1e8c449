// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05), sm_100a.
//
//   Y[t][f] = sum_k X[t][k] * W[f][k]        X: [M tokens][K], W: [N features][K], both K-major
//
// The weight matrix is the MMA's A operand and the activations its B operand ("swap-AB"):
// a CTA owns 128 features x BN tokens, the accumulator D[128 x BN] lives in tensor memory
// with one feature per TMEM lane and one token per column.  With BN = 16..64 the kernel is a
// weight streamer for decode (every weight byte is read once, the few tokens ride along);
// with BN = 256 it is the ordinary 128x256 tile for prefill.  One kernel, five BN.
//
// Roles inside a CTA (192 or 576 threads): warp 0 = TMA producer (one elected lane issues
// cp.async.bulk.tensor loads of 128B-swizzled [rows x 64] boxes into a ring of stages),
// warp 1 = TMEM allocator and MMA issuer (one elected lane issues tcgen05.mma, K = 16 per
// instruction, four per stage, and commits stages back to the producer), warps 2..5 or 2..17 =
// epilogue (tcgen05.ld of their lane quarter, then the fused epilogue and the store).
//
// Split-K without atomics or scratch in global memory: grid.z CTAs that share an output
// tile form a thread-block cluster; each accumulates its slice of K in its own TMEM, parks
// the partial tile in its own shared memory, and after a cluster barrier every CTA sums a
// share of the columns over all peers through distributed shared memory, in rank order --
// so the result does not depend on which CTA ran first.
//
// Epilogues: store fp32 / store bf16 / add an fp32 addend (the residual) and store fp32 /
// SwiGLU: two accumulators (gate rows f, up rows F+f of the same matrix), silu(g)*u as bf16.
//
// The kernel is launched with programmatic stream serialisation: it may start while the kernel
// before it still runs, sets up its barriers and tensor memory and requests its first ring of
// WEIGHT tiles (which nothing in the stream writes) in that shadow, and touches activations,
// addend and output only after griddepcontrol.wait.
//
// NORMED forms (token tiles <= 64): the activations are not a bf16 matrix but the fp32 residual
// stream and an RMSNorm weight.  The four epilogue warps, idle until the accumulator is ready,
// build the B tiles themselves: bf16(x * w) straight into the swizzled ring slot, and the sum of
// squares of each token's row on the way.  The accumulator is multiplied by rsqrt(mean + eps) in the
// epilogue -- (W (x*w)) * r = W (x*w*r) -- so the norm costs no kernel and no pass over memory.
// With split K each CTA sums the squares of its slice and the cluster adds them in rank order.
//
// Every wait on an mbarrier is bounded: after the limit the CTA raises the library's status
// word, stops waiting everywhere, still meets its cluster barriers, frees its TMEM and
// returns.
#include "tcgen05.cuh"

using namespace fwb;
using namespace fwb::tc5;

namespace {
__device__ int g_gemm_status = 0;
}

namespace fwb {
namespace tc5 {
int* status_word() {
    static int* address = nullptr;
    if (!address) {
        void* found = nullptr;
        if (cudaGetSymbolAddress(&found, g_gemm_status) == cudaSuccess) address = static_cast<int*>(found);
    }
    return address;
}
}  // namespace tc5
}  // namespace fwb

namespace {

// Epilogue warps: four for decode-sized token tiles (little to store, and several CTAs share an
// SM), sixteen -- four per quarter of the TMEM lanes -- for prompt-sized tiles, where the stores
// of 128 x 256 (x2) values would otherwise leave the tensor pipe idle for a fifth of the time.
constexpr int epi_warps(int bn) { return bn >= 128 ? 16 : 4; }
constexpr int threads_for(int bn) { return 64 + 32 * epi_warps(bn); }   // + producer and MMA warps
constexpr int SMEM_BUDGET = 200 * 1024;

// The WIDE forms give a CTA two adjacent 128-feature tiles (two accumulators over the same
// token tile): per MMA the activations are read from L2 once for 256 features, which is what
// keeps the tensor pipe fed at prefill sizes.
enum Epilogue : int { EPI_F32 = 0, EPI_BF16 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU_BF16 = 3,
                      EPI_F32_WIDE = 4, EPI_BF16_WIDE = 5 };
constexpr bool epi_wide(int epi) { return epi == EPI_F32_WIDE || epi == EPI_BF16_WIDE; }
constexpr int epi_accumulators(int epi) { return (epi == EPI_SWIGLU_BF16 || epi_wide(epi)) ? 2 : 1; }


template <int BN, int NACC>
struct Tile {
    static constexpr int A_BYTES = BM * BK * 2;                 // 16 KiB per accumulator
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = NACC * A_BYTES + B_BYTES;
    static constexpr int RAW_STAGES = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int MAX_STAGES = RAW_STAGES > 8 ? 8 : RAW_STAGES;
    // the default ring keeps a CTA under ~110 KiB so that two fit an SM (the next kernel's CTAs
    // can then be resident and prefetch weights while this kernel still runs)
    static constexpr int DEFAULT_STAGES = MAX_STAGES > 6 ? 6 : MAX_STAGES;
    static constexpr int COLS = BN * NACC;                      // TMEM columns in use
    static constexpr int TMEM_COLS = COLS <= 32 ? 32 : (COLS <= 64 ? 64 : (COLS <= 128 ? 128 : (COLS <= 256 ? 256 : 512)));
    static constexpr int PARTIAL_BYTES = (BN <= 64 || NACC == 1) ? COLS * BM * 4 : 0;   // fp32 partial tile for split-K
    static constexpr int data_bytes(int stages) {
        return stages * STAGE_BYTES > PARTIAL_BYTES ? stages * STAGE_BYTES : PARTIAL_BYTES;
    }
    // + alignment slack, barriers (256 bytes) and one float per token for the sums of squares
    static constexpr int smem_bytes(int stages) { return data_bytes(stages) + 1024 + 512; }
};

struct Params {
    void* y;               // [M][ldy] fp32 or bf16
    const float* addend;   // [M][ldy] fp32 or null
    int M, N, K;           // tokens, features (of one accumulator), reduction
    int ldy;
    int up_row_offset;     // SwiGLU: rows of the up projection start here in W
    int k_blocks_per_split;
    int stages;            // depth of the shared-memory ring (<= Tile::MAX_STAGES)
    int* status;           // the library's status word (see tc5::status_word)
    // NORMED forms: rows of the fp32 residual [.][K] (row t, or norm_rows[t]), the norm's weight [K], eps
    const float* norm_x;
    const float* norm_w;
    const int* norm_rows;
    float norm_eps;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// NORMED forms, run by the 128 threads of the four epilogue warps: for every 64-wide block of
// this CTA's K slice, write bf16(x[t][k] * w[k]) for the tile's tokens into the ring slot's B
// tile (128-byte rows, 16-byte chunks XOR-swizzled by row: what TMA would have left) and arrive
// on the slot's barrier; add up x^2 per token.  A thread owns chunk c = thread & 7 of token
// rows thread >> 3, + 16, ...; the sums of the eight chunk lanes of a row are added by shuffles,
// so sum_sq[r] is this CTA's share for token r, summed in an order fixed by K and the split.
// Loads of up to GROUP blocks are in flight together: a decode step's slice is one group.
template <int BN, int NACC>
__device__ __forceinline__ void produce_normed_tiles(const Params& prm, uint8_t* tiles, uint64_t* full_bar,
                                                     uint64_t* empty_bar, volatile int* abort_flag,
                                                     float* sum_sq, int STAGES, int kb_begin, int n_kb,
                                                     int tok0) {
    using T = Tile<BN, NACC>;
    constexpr int PASSES = BN / 16;
    constexpr int GROUP = BN == 16 ? 4 : (BN == 32 ? 2 : 1);
    const int et = (int)threadIdx.x - 64, lane = et & 31;
    const int c = et & 7, r0 = et >> 3;
    const float* rows[PASSES];
    float sq[PASSES];
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        const int t = tok0 + r0 + 16 * p;
        rows[p] = t < prm.M ? prm.norm_x + (size_t)(prm.norm_rows ? prm.norm_rows[t] : t) * prm.K : nullptr;
        sq[p] = 0.0f;
    }
    bool ok = true;
    // tiles [announced, upto) are written: one fence for all of them, then their barriers
    int announced = 0;
    auto announce = [&](int upto) {
        if (upto <= announced) return;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the tensor core
        __syncwarp();
        if (lane == 0)
            for (int k = announced; k < upto; ++k) mbar_arrive(&full_bar[k % STAGES]);
        announced = upto;
    };
    for (int i0 = 0; i0 < n_kb && ok; i0 += GROUP) {
        float4 xv[GROUP][PASSES][2], wv[GROUP][2];
#pragma unroll
        for (int gi = 0; gi < GROUP; ++gi) {
            const int k = (kb_begin + i0 + gi) * BK + c * 8;
            const bool in = i0 + gi < n_kb && k < prm.K;           // K is a multiple of 8: a chunk is whole or absent
            wv[gi][0] = in ? *reinterpret_cast<const float4*>(prm.norm_w + k) : make_float4(0, 0, 0, 0);
            wv[gi][1] = in ? *reinterpret_cast<const float4*>(prm.norm_w + k + 4) : make_float4(0, 0, 0, 0);
#pragma unroll
            for (int p = 0; p < PASSES; ++p) {
                const bool on = in && rows[p];
                xv[gi][p][0] = on ? *reinterpret_cast<const float4*>(rows[p] + k) : make_float4(0, 0, 0, 0);
                xv[gi][p][1] = on ? *reinterpret_cast<const float4*>(rows[p] + k + 4) : make_float4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int gi = 0; gi < GROUP; ++gi) {
            const int i = i0 + gi;
            if (i >= n_kb) break;
            const int s = i % STAGES;
            if (i >= STAGES) {
                // the slot comes free only after tiles already written here have been announced
                announce(i);
                ok = mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abort_flag, 4, prm.status);
            }
            if (!ok) break;
            uint8_t* b_tile = tiles + (size_t)s * T::STAGE_BYTES + NACC * T::A_BYTES;
#pragma unroll
            for (int p = 0; p < PASSES; ++p) {
                const float4 a = xv[gi][p][0], b = xv[gi][p][1], wa = wv[gi][0], wb = wv[gi][1];
                sq[p] = fmaf(a.x, a.x, sq[p]); sq[p] = fmaf(a.y, a.y, sq[p]);
                sq[p] = fmaf(a.z, a.z, sq[p]); sq[p] = fmaf(a.w, a.w, sq[p]);
                sq[p] = fmaf(b.x, b.x, sq[p]); sq[p] = fmaf(b.y, b.y, sq[p]);
                sq[p] = fmaf(b.z, b.z, sq[p]); sq[p] = fmaf(b.w, b.w, sq[p]);
                uint4 packed;
                __nv_bfloat162 h;
                h = __floats2bfloat162_rn(a.x * wa.x, a.y * wa.y); packed.x = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(a.z * wa.z, a.w * wa.w); packed.y = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(b.x * wb.x, b.y * wb.y); packed.z = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(b.z * wb.z, b.w * wb.w); packed.w = *reinterpret_cast<uint32_t*>(&h);
                const int r = r0 + 16 * p;
                *reinterpret_cast<uint4*>(b_tile + r * 128 + ((c ^ (r & 7)) << 4)) = packed;
            }
        }
        if (ok) announce(i0 + GROUP < n_kb ? i0 + GROUP : n_kb);
    }
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
        float v = sq[p];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (c == 0) sum_sq[r0 + 16 * p] = v;
    }
    // all four warps' sums are in place before anybody's epilogue reads them (and, with split K,
    // before the cluster barrier that precedes the peers' reads)
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <int BN, int EPI, bool NORMED>
__global__ void __launch_bounds__(threads_for(BN), 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const Params prm) {
    constexpr int NACC = epi_accumulators(EPI);
    constexpr bool WIDE = epi_wide(EPI);
    using T = Tile<BN, NACC>;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int STAGES = prm.stages;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(tiles + T::data_bytes(STAGES));
    uint64_t* empty_bar = full_bar + T::MAX_STAGES;
    uint64_t* acc_bar = empty_bar + T::MAX_STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    float* sum_sq = reinterpret_cast<float*>(tiles + T::data_bytes(STAGES) + 256);   // [BN], NORMED only

    pdl_launch_dependents();     // the next kernel may set itself up in this one's shadow
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // token tiles are the fast grid dimension: CTAs that run together share weight tiles, and
    // a wave's weights plus all the activations fit the L2 cache
    const int feat0 = blockIdx.y * (WIDE ? 2 * BM : BM), tok0 = blockIdx.x * BN;
    const int second_tile_row = WIDE ? feat0 + BM : prm.up_row_offset + feat0;   // accumulator 1's rows of W
    const int splits = gridDim.z;
    const int total_kb = (prm.K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * prm.k_blocks_per_split;
    int kb_end = kb_begin + prm.k_blocks_per_split;
    if (kb_end > total_kb) kb_end = total_kb;
    const int n_kb = kb_end > kb_begin ? kb_end - kb_begin : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], NORMED ? 1 + epi_warps(BN) : 1);   // + the warps that write the B tile
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(tmem_holder, T::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            // Weights do not depend on the kernel before this one: the first ring of weight
            // tiles is requested before waiting for it, the activations after.
            const int ahead = n_kb < STAGES ? n_kb : STAGES;
            for (int i = 0; i < ahead; ++i) {
                uint8_t* stage = tiles + (size_t)i * T::STAGE_BYTES;
                mbar_expect_tx(&full_bar[i], NORMED ? NACC * T::A_BYTES : T::STAGE_BYTES);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(stage, &map_w, &full_bar[i], k, feat0);
                if (NACC == 2) tma_load_2d(stage + T::A_BYTES, &map_w, &full_bar[i], k, second_tile_row);
            }
            pdl_wait();
            if (!NORMED)
                for (int i = 0; i < ahead; ++i)
                    tma_load_2d(tiles + (size_t)i * T::STAGE_BYTES + NACC * T::A_BYTES, &map_x, &full_bar[i],
                                (kb_begin + i) * BK, tok0);
            for (int i = ahead; i < n_kb; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                if (!mbar_wait(&empty_bar[s], (round - 1) & 1, abort_flag, 1, prm.status)) break;
                uint8_t* stage = tiles + (size_t)s * T::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], NORMED ? NACC * T::A_BYTES : T::STAGE_BYTES);
                const int k = (kb_begin + i) * BK;
                tma_load_2d(stage, &map_w, &full_bar[s], k, feat0);
                if (NACC == 2) tma_load_2d(stage + T::A_BYTES, &map_w, &full_bar[s], k, second_tile_row);
                if (!NORMED) tma_load_2d(stage + NACC * T::A_BYTES, &map_x, &full_bar[s], k, tok0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BN);
            bool ok = true;
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t round = i / STAGES;
                ok = mbar_wait(&full_bar[s], round & 1, abort_flag, 2, prm.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t stage = smem_u32(tiles + (size_t)s * T::STAGE_BYTES);
                const uint64_t b_desc = make_smem_desc(stage + NACC * T::A_BYTES);
#pragma unroll
                for (int a = 0; a < NACC; ++a) {
                    const uint64_t a_desc = make_smem_desc(stage + a * T::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements = 32 bytes = 2 descriptor units along K inside the swizzle row
                        umma_bf16(tmem_base + a * BN, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                  (i > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(&empty_bar[s]);       // the stage is free once these MMAs have read it
            }
            umma_commit(acc_bar);                 // arrives when every MMA above has completed
        }
    }
    __syncwarp();

    // ---------------------------------------------------------------- epilogue
    const bool epi_warp = warp >= 2;
    // sixteen epilogue warps: four per quarter of the TMEM lanes (a warp may only read the quarter
    // its index selects); with one slice of K they split the token columns between them, which
    // keeps several warps per scheduler busy during the stores instead of one
    const int column_group = (warp - 2) >> 2;
    const int quarter = warp & 3;                  // the TMEM lanes this warp may read
    const int row = quarter * 32 + lane;           // feature inside the tile
    bool acc_ready = true;
    if (epi_warp) {
        pdl_wait();              // the addend is read and Y written only after the previous kernel
        if constexpr (NORMED) produce_normed_tiles<BN, NACC>(prm, tiles, full_bar, empty_bar, abort_flag, sum_sq, STAGES,
                                                   kb_begin, n_kb, tok0);
        if (n_kb > 0) acc_ready = mbar_wait(acc_bar, 0, abort_flag, 3, prm.status);
        acc_ready = acc_ready && !*abort_flag;
        acc_ready = __all_sync(0xffffffffu, acc_ready);   // tcgen05.ld needs the whole warp
        tc_fence_after();
    }
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int f = feat0 + row;

    auto finish = [&](int col, float g, float u, float r) {
        // col: token inside the tile; g: accumulator 0; u: accumulator 1 (SwiGLU only);
        // r: the token's rsqrt(mean square + eps) (NORMED only)
        const int t = tok0 + col;
        if (t >= prm.M || f >= prm.N) return;
        if (NORMED) {
            g *= r;
            u *= r;
        }
        const size_t at = (size_t)t * prm.ldy + f;
        if (EPI == EPI_F32) reinterpret_cast<float*>(prm.y)[at] = g;
        else if (EPI == EPI_F32_WIDE) {
            reinterpret_cast<float*>(prm.y)[at] = g;
            if (f + BM < prm.N) reinterpret_cast<float*>(prm.y)[at + BM] = u;
        } else if (EPI == EPI_BF16_WIDE) {
            reinterpret_cast<__nv_bfloat16*>(prm.y)[at] = __float2bfloat16_rn(g);
            if (f + BM < prm.N) reinterpret_cast<__nv_bfloat16*>(prm.y)[at + BM] = __float2bfloat16_rn(u);
        } else if (EPI == EPI_ADD_F32) reinterpret_cast<float*>(prm.y)[at] = g + (splits > 1 ? u : prm.addend[at]);
        else if (EPI == EPI_BF16) reinterpret_cast<__nv_bfloat16*>(prm.y)[at] = __float2bfloat16_rn(g);
        else reinterpret_cast<__nv_bfloat16*>(prm.y)[at] = __float2bfloat16_rn(silu_fast(g) * u);
    };

    if (splits == 1) {
        if (epi_warp && acc_ready) {
            constexpr int GROUPS = epi_warps(BN) / 4;
            constexpr int PER_GROUP = BN / GROUPS >= 16 ? BN / GROUPS : 16;
            const int c_begin = column_group * PER_GROUP;
            const int c_end = c_begin + PER_GROUP < BN ? c_begin + PER_GROUP : BN;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 16) {
                float g[16], u[16];
                if (n_kb > 0) {
                    tmem_ld16(lane_addr + c0, g);
                    if (NACC == 2) tmem_ld16(lane_addr + BN + c0, u);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    finish(c0 + j, g[j], NACC == 2 ? u[j] : 0.0f,
                           NORMED ? rsqrtf(sum_sq[c0 + j] / (float)prm.K + prm.norm_eps) : 1.0f);
            }
        }
    } else {
        // park the partial tile in shared memory: partial[col][row], fp32 (the pipeline's stages
        // are free: every MMA that read them has completed).  With sixteen epilogue warps each
        // quarter of the rows is shared by four warps, a quarter of the columns each.
        constexpr int GROUPS = epi_warps(BN) / 4;
        float* partial = reinterpret_cast<float*>(tiles);
        if (epi_warp) {
#pragma unroll 1
            for (int c0 = column_group * 16; c0 < T::COLS; c0 += 16 * GROUPS) {
                float v[16];
                if (n_kb > 0 && acc_ready) tmem_ld16(lane_addr + c0, v);
                else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) partial[(c0 + j) * BM + row] = v[j];
            }
        }
        tc_fence_before();
        cluster_sync_all();
        if (epi_warp) {
            // Column c of the tile is merged by rank c % splits, and among that rank's warps by
            // column group (c / splits) % GROUPS.  A thread (one feature row) asks every peer for its
            // values of BATCH columns before it uses the first -- one round trip through distributed
            // shared memory for all of them -- and adds them in rank order, as every cut of the work does.
            const uint32_t rank = cluster_rank();
            const uint32_t base = smem_u32(partial);
            constexpr int BATCH = BN >= 64 ? 4 : 2;
            const int col_step = splits * GROUPS;
#pragma unroll 1
            for (int col0 = (int)rank + column_group * splits; col0 < BN; col0 += col_step * BATCH) {
                float pg[BATCH][8], pu[BATCH][8], ps[BATCH][8], add[BATCH];
#pragma unroll
                for (int b = 0; b < BATCH; ++b) {
                    const int col = col0 + b * col_step;
                    const bool live = col < BN;
                    add[b] = 0.0f;
                    if (EPI == EPI_ADD_F32 && live && tok0 + col < prm.M && f < prm.N)
                        add[b] = prm.addend[(size_t)(tok0 + col) * prm.ldy + f];
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const bool on = live && r < splits;
                        pg[b][r] = on ? ld_dsmem_f32(base + (uint32_t)((col * BM + row) * 4), (uint32_t)r) : 0.0f;
                        pu[b][r] = (on && NACC == 2)
                                       ? ld_dsmem_f32(base + (uint32_t)(((BN + col) * BM + row) * 4), (uint32_t)r) : 0.0f;
                        ps[b][r] = (on && NORMED) ? ld_dsmem_f32(smem_u32(sum_sq) + (uint32_t)(col * 4), (uint32_t)r) : 0.0f;
                    }
                }
#pragma unroll
                for (int b = 0; b < BATCH; ++b) {
                    const int col = col0 + b * col_step;
                    if (col >= BN) break;
                    float g = 0.0f, u = 0.0f, sq = 0.0f;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {            // + 0 beyond the last rank: exact
                        g += pg[b][r];
                        u += pu[b][r];
                        sq += ps[b][r];
                    }
                    if (EPI == EPI_ADD_F32) u = add[b];
                    if (!*abort_flag)
                        finish(col, g, u, NORMED ? rsqrtf(sq / (float)prm.K + prm.norm_eps) : 1.0f);
                }
            }
        }
        cluster_sync_all();                        // nobody leaves while a peer still reads it
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, T::TMEM_COLS);
}

// ------------------------------------------------------------------ host side
template <int BN, int EPI, bool NORMED = false>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, Params prm, int splits,
           cudaStream_t stream) {
    constexpr int NACC = epi_accumulators(EPI);
    using T = Tile<BN, NACC>;
    auto kernel = gemm_tcgen05_kernel<BN, EPI, NORMED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             T::smem_bytes(T::MAX_STAGES));
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    if (prm.stages <= 0) prm.stages = T::DEFAULT_STAGES;
    if (prm.stages > T::MAX_STAGES) prm.stages = T::MAX_STAGES;
    if (prm.stages < 2) prm.stages = 2;
    cudaLaunchConfig_t config = {};
    constexpr int FEATURES = epi_wide(EPI) ? 2 * BM : BM;
    config.gridDim = dim3((prm.M + BN - 1) / BN, (prm.N + FEATURES - 1) / FEATURES, splits);
    config.blockDim = dim3(threads_for(BN));
    config.dynamicSmemBytes = T::smem_bytes(prm.stages);
    config.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&config, kernel, map_w, map_x, prm);
    return e == cudaSuccess ? fwb_launch_status() : (int)e;
}

// The NORMED forms exist for decode-sized token tiles and the epilogues that follow a norm.
template <int BN>
int launch_normed(int epi, const CUtensorMap& map_w, const Params& prm, int splits, cudaStream_t stream) {
    switch (epi) {
        case EPI_F32: return launch<BN, EPI_F32, true>(map_w, map_w, prm, splits, stream);
        case EPI_BF16: return launch<BN, EPI_BF16, true>(map_w, map_w, prm, splits, stream);
        case EPI_SWIGLU_BF16: return launch<BN, EPI_SWIGLU_BF16, true>(map_w, map_w, prm, splits, stream);
        default: return FWB_UNSUPPORTED;
    }
}

template <int BN>
int launch_epi(int epi, const CUtensorMap& map_w, const CUtensorMap& map_x, const Params& prm, int splits,
               cudaStream_t stream) {
    switch (epi) {
        case EPI_F32: return launch<BN, EPI_F32>(map_w, map_x, prm, splits, stream);
        case EPI_BF16: return launch<BN, EPI_BF16>(map_w, map_x, prm, splits, stream);
        case EPI_ADD_F32: return launch<BN, EPI_ADD_F32>(map_w, map_x, prm, splits, stream);
        case EPI_SWIGLU_BF16: return launch<BN, EPI_SWIGLU_BF16>(map_w, map_x, prm, splits, stream);
        case EPI_F32_WIDE: return launch<BN, EPI_F32_WIDE>(map_w, map_x, prm, splits, stream);
        case EPI_BF16_WIDE: return launch<BN, EPI_BF16_WIDE>(map_w, map_x, prm, splits, stream);
        default: return FWB_UNSUPPORTED;
    }
}

}  // namespace

// X: [M][K] bf16; W: [rows][K] bf16 (rows = N, or >= up_row_offset + N for SwiGLU);
// Y: [M][ldy] (fp32 for epilogues 0 and 2, bf16 for 1 and 3).  `splits` (1..8) CTAs share the
// K range of a tile as a cluster; with splits > 1 the token tile must be <= 128 wide (64 for SwiGLU).
// `stages` sets the depth of the shared-memory ring (0: the default).  `tile_tokens` (0: by M)
// may ask for a smaller token tile than M would pick (more CTAs); `wide` gives a CTA two feature tiles.
// K must be a multiple of 8 (TMA strides are multiples of 16 bytes) and both base
// pointers 16-byte aligned; anything else is refused.
FWB_API int fwb_gemm_tcgen05(const void* X, const void* W, void* Y, const float* addend, int M, int N,
                             int K, int w_rows, int ldy, int epilogue, int up_row_offset, int splits,
                             int stages, int tile_tokens, int wide, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return FWB_OK;
    if (!X || !W || !Y || K <= 0 || ldy < N) return FWB_BAD_ARGUMENT;
    if ((K & 7) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return FWB_UNSUPPORTED;
    if (epilogue == EPI_ADD_F32 && !addend) return FWB_BAD_ARGUMENT;
    if (epilogue == EPI_SWIGLU_BF16 && (up_row_offset < N || w_rows < up_row_offset + N)) return FWB_BAD_ARGUMENT;
    if (epilogue != EPI_SWIGLU_BF16 && w_rows < N) return FWB_BAD_ARGUMENT;
    if (splits < 1 || splits > 8) return FWB_BAD_ARGUMENT;
    int bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
    if (tile_tokens == 16 || tile_tokens == 32 || tile_tokens == 64 || tile_tokens == 128 || tile_tokens == 256) {
        if (tile_tokens < bn) bn = tile_tokens;                            // a smaller tile: more CTAs
    } else if (tile_tokens != 0) {
        return FWB_BAD_ARGUMENT;
    }
    const int bn_eff = bn;
    // a full token tile and enough features: two 128-feature tiles per CTA (all 512 TMEM columns)
    // (`wide`: 1 = yes, 0 = no, -1 = when single tiles would not fit the GPU in one wave; measured
    // at 2,048 tokens on B200: 2048-feature products are faster narrow, 3072 and up faster wide)
    const long narrow_ctas = (long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    const bool go_wide = wide == 1 || (wide < 0 && bn == 256 && narrow_ctas > 148);
    if (go_wide && bn >= 128 && N >= 2 * BM && splits == 1) {
        if (epilogue == EPI_F32) epilogue = EPI_F32_WIDE;
        else if (epilogue == EPI_BF16) epilogue = EPI_BF16_WIDE;
    }
    // the slices' partial tiles are parked in the ring's shared memory (columns x 128 rows of fp32,
    // which the ring is sized for): token tiles up to 128 split, with one accumulator (256-token
    // tiles were measured too: a cluster of CTAs that each fill an SM gains nothing over the pairs)
    if (splits > 1 && (bn_eff > 128 || (bn_eff == 128 && epi_accumulators(epilogue) == 2))) return FWB_UNSUPPORTED;
    if ((N + BM - 1) / BM > 65535) return FWB_TOO_LARGE;
    const int total_kb = (K + BK - 1) / BK;
    if (splits > total_kb) splits = total_kb;
    Params prm;
    prm.y = Y;
    prm.addend = addend;
    prm.M = M;
    prm.N = N;
    prm.K = K;
    prm.ldy = ldy;
    prm.up_row_offset = up_row_offset;
    prm.k_blocks_per_split = (total_kb + splits - 1) / splits;
    prm.stages = stages;
    prm.status = status_word();
    prm.norm_x = nullptr;
    prm.norm_w = nullptr;
    prm.norm_rows = nullptr;
    prm.norm_eps = 0.0f;
    CUtensorMap map_w, map_x;
    if (!make_map(&map_w, W, w_rows, K, BM)) return FWB_UNSUPPORTED;
    if (!make_map(&map_x, X, M, K, bn_eff)) return FWB_UNSUPPORTED;
    switch (bn_eff) {
        case 16: return launch_epi<16>(epilogue, map_w, map_x, prm, splits, stream);
        case 32: return launch_epi<32>(epilogue, map_w, map_x, prm, splits, stream);
        case 64: return launch_epi<64>(epilogue, map_w, map_x, prm, splits, stream);
        case 128: return launch_epi<128>(epilogue, map_w, map_x, prm, splits, stream);
        default: return launch_epi<256>(epilogue, map_w, map_x, prm, splits, stream);
    }
}

// The same product with the RMSNorm that precedes it folded in: the activations are rows of the
// fp32 residual `x_res` ([.][K]; row t of the product reads row `rows[t]`, or row t when `rows`
// is null), normalised with weight `norm_w` [K] and `eps`:
//     Y[t][f] = sum_k W[f][k] * bf16(x[t][k] * norm_w[k])  *  rsqrt(mean_k x[t][k]^2 + eps)
// Token tiles of at most 64 (M <= 64 or tile_tokens <= 64); epilogues 0 (fp32), 1 (bf16), 3 (SwiGLU).
FWB_API int fwb_gemm_tcgen05_normed(const float* x_res, const float* norm_w, const int* rows, float eps,
                                    const void* W, void* Y, int M, int N, int K, int w_rows, int ldy,
                                    int epilogue, int up_row_offset, int splits, int stages,
                                    int tile_tokens, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return FWB_OK;
    if (!x_res || !norm_w || !W || !Y || K <= 0 || ldy < N) return FWB_BAD_ARGUMENT;
    if ((K & 7) || ((uintptr_t)W & 15) || ((uintptr_t)x_res & 15) || ((uintptr_t)norm_w & 15)) return FWB_UNSUPPORTED;
    if (epilogue == EPI_SWIGLU_BF16 && (up_row_offset < N || w_rows < up_row_offset + N)) return FWB_BAD_ARGUMENT;
    if (epilogue != EPI_SWIGLU_BF16 && w_rows < N) return FWB_BAD_ARGUMENT;
    if (splits < 1 || splits > 8) return FWB_BAD_ARGUMENT;
    int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    if (tile_tokens == 16 || tile_tokens == 32 || tile_tokens == 64) {
        if (tile_tokens < bn) bn = tile_tokens;
    } else if (tile_tokens != 0) {
        return FWB_BAD_ARGUMENT;
    }
    if ((N + BM - 1) / BM > 65535) return FWB_TOO_LARGE;
    const int total_kb = (K + BK - 1) / BK;
    if (splits > total_kb) splits = total_kb;
    Params prm;
    prm.y = Y;
    prm.addend = nullptr;
    prm.M = M;
    prm.N = N;
    prm.K = K;
    prm.ldy = ldy;
    prm.up_row_offset = up_row_offset;
    prm.k_blocks_per_split = (total_kb + splits - 1) / splits;
    prm.stages = stages;
    prm.status = status_word();
    prm.norm_x = x_res;
    prm.norm_w = norm_w;
    prm.norm_rows = rows;
    prm.norm_eps = eps;
    CUtensorMap map_w;
    if (!make_map(&map_w, W, w_rows, K, BM)) return FWB_UNSUPPORTED;
    switch (bn) {
        case 16: return launch_normed<16>(epilogue, map_w, prm, splits, stream);
        case 32: return launch_normed<32>(epilogue, map_w, prm, splits, stream);
        default: return launch_normed<64>(epilogue, map_w, prm, splits, stream);
    }
}

// Reads and clears the status word that a wait which gave up leaves behind (0 = none).
// Synchronises the device.
FWB_API int fwb_gemm_tcgen05_status() {
    int value = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&value, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    if (value) cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    return value;
}

// The two words a health check reads -- the status word above (not cleared here) and the
// embedding's bad-token flag -- copied to pinned host memory behind the work queued on `stream`,
// so that a caller who waits for that work anyway learns of a failure without a wait of its own.
FWB_API int fwb_health_peek_async(int* pinned_host, const int* bad_token_flag, cudaStream_t stream) {
    int* word = status_word();
    if (!word || !pinned_host) return FWB_BAD_ARGUMENT;
    pinned_host[1] = 0;
    cudaError_t e = cudaMemcpyAsync(pinned_host, word, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess && bad_token_flag)
        e = cudaMemcpyAsync(pinned_host + 1, bad_token_flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
    return e == cudaSuccess ? FWB_OK : (int)e;
}

namespace {
// One thread waits, with a short limit, on a barrier that nobody will ever arrive on: the wait
// must give up, leave its code in the status word and let the kernel end normally.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned limit, int code) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(&bar, 0, &abort_flag, code, status, limit);
}
}  // namespace

// Exercises the path a stuck pipeline takes, without sticking anything: returns once the kernel
// has given up (a few thousand polls); afterwards fwb_gemm_tcgen05_status() returns `code`.
FWB_API int fwb_selftest_bounded_wait(int code, cudaStream_t stream) {
    bounded_wait_selftest_kernel<<<1, 1, 0, stream>>>(status_word(), 4096u, code);
    return fwb_launch_status();
}

// Programmatic dependent launch for every kernel of the library: 1 = on (default), 0 = off.
FWB_API int fwb_set_pdl(int enabled) {
    fwb::pdl_enabled() = enabled != 0;
    return FWB_OK;
}
