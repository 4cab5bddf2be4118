// bf16 GEMM for sm_100a on the 5th-generation tensor cores:
//   D[M,N] = A[M,K] * B_T[N,K]^T,  fp32 accumulation in TMEM, f32 or bf16 output.
// One kernel template covers the three reference entry points
//   build_gemm          (1-SM MMA, 128x256 tile per CTA)
//   build_gemm_2sm      (cta_group::2 MMA, 256x256 tile per 2-CTA cluster)
//   build_grouped_gemm  (G independent problems stacked along the row axis)
// (examples/blackwell/gemm_highperf_blackwell.py:69-313, :902-1246,
//  examples/blackwell/grouped_gemm.py:61-289).
//
// Structure (what differs from the reference's kernels and why):
//   * persistent: one CTA (or CTA pair) per SM walks a static list of output
//     tiles, so barrier setup, TMEM allocation and pipeline fill are paid once
//     per SM instead of once per tile;
//   * warp specialised: warp 0 = TMA producer, warp 1 = MMA issuer (+ TMEM
//     owner), warps 2-5 = epilogue.  Producer and issuer are single threads;
//   * the accumulator is double buffered in TMEM (2 x BN fp32 columns, the
//     whole 512 when BN = 256), so the epilogue of tile i overlaps the main loop
//     of tile i+1;
//   * shared-memory ring slots are released by tcgen05.commit, i.e. when the
//     MMAs that read them have retired, never right after issue;
//   * the epilogue goes TMEM -> registers -> swizzled shared memory -> TMA
//     store, one 32-row x 128-byte box per warp, so every global write is a full
//     128-byte line;
//   * tiles are rasterised in bands of `band` M-tiles so that the ~148 tiles in
//     flight share A and B panels through L2;
//   * tensor maps are kernel parameters (__grid_constant__), encoded per launch;
//   * every mbarrier wait is bounded and reports through a status word.
//
// 2-SM protocol: both CTAs of a pair load their own 128 rows of A and their own
// BN/2 rows of B_T with cta_group::2 TMA loads that signal the leader's "full"
// barrier; the leader (cluster rank 0) issues the M=256 MMAs, which read both
// CTAs' shared memory and write both CTAs' TMEM; it releases a ring slot with
// two commits, one to its own "empty" barrier and one to the peer's (address
// from mapa); epilogue warps of both CTAs arrive on the leader's "tmem empty"
// barrier.  No copy in this file is multicast.
#include "common.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <atomic>

namespace pb200 {
namespace {

using namespace ptx;

constexpr int BM = 128;          // rows per CTA tile (TMEM lanes)
constexpr int BK = 64;           // bf16 elements per k-tile = one 128-byte swizzle row
constexpr int UMMA_K = 16;       // K per tcgen05.mma for 16-bit operands
static_assert(BK / UMMA_K == 4, "the MMA issuer is written out for four MMAs per k-tile");
constexpr int kThreads = 192;    // 6 warps
constexpr int kEpiWarps = 4;
constexpr int kStageRows = 32;   // rows per epilogue store box (one warp)
constexpr int kStageBytes = kStageRows * 128;  // 4 KiB, swizzle-128B image
constexpr uint32_t kDebugDirectStore = 1u << 16;  // create flag: bypass the TMA-store epilogue
constexpr uint32_t kForceNarrowTile = 1u << 18;   // create flag: 2-SM kernels always use the 256 x 256 tile
constexpr uint32_t kForceWideTile = 1u << 19;     // create flag: 2-SM kernels use the 512 x 256 tile whenever M % 512 == 0

struct GemmShape {
    int tiles_m;      // tiles along M per group (a tile is BM*CTA_GROUP rows)
    int tiles_n;
    int k_tiles;
    int groups;
    int rows_per_group_a;   // M  (row offset of group g in A and D is g*M)
    int rows_per_group_b;   // N  (row offset of group g in B_T is g*N)
    int band;               // M-tiles per raster band
    int n_total;            // leading dimension of D (elements)
    int n_experts;          // variable-size grouped GEMM: number of experts (0 = fixed-size problem)
    int up_row_off;         // EPI 1: row offset of an expert's "up" weights inside its block of B_T (= F)
    int act;                // EPI 3: 0 none, 1 relu, 2 gelu (erf form), 3 silu
    int has_bias;           // EPI 3: aux points at bias[N] (f32)
};

// EPI = 3: D = act(accumulator + bias[column]).
__device__ __forceinline__ float bias_act(float x, int act) {
    switch (act) {
        case 1: return fmaxf(x, 0.0f);
        case 2: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
        case 3: return __fdividef(x, 1.0f + __expf(-x));
        default: return x;
    }
}
// v[0..31] += bias[col .. col+31] (the same 32 values for every lane: broadcast loads), then act.
__device__ __forceinline__ void apply_bias_act(uint32_t (&v)[32], const float* __restrict__ bias, int col,
                                               const GemmShape& shape) {
    if (shape.has_bias) {
        const float4* bp = reinterpret_cast<const float4*>(bias + col);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float4 b = __ldg(bp + j);
            v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + b.x);
            v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + b.y);
            v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + b.z);
            v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + b.w);
        }
    }
    if (shape.act) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(bias_act(__uint_as_float(v[i]), shape.act));
    }
}

template <int BN, int CTA_GROUP, int WIDE = 0>
struct SmemPlan {
    static constexpr int kBRows = BN / CTA_GROUP;            // rows of B_T this CTA loads
    static constexpr int kABytes = BM * BK * 2 * (1 + WIDE); // 16 KiB per 128-row block of A
    static constexpr int kBBytes = kBRows * BK * 2;
    static constexpr int kStage = kABytes + kBBytes;
    // Store boxes in flight per epilogue warp.  Three or four (with one ring stage fewer) measured
    // within 0.5 % of two at 8192^3, so the ring keeps the shared memory.
    static constexpr int kEpiBufs = 2;
    static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kStageBytes;   // 32 KiB with two buffers per warp
    static constexpr int kBarBytes = 1024;
    static constexpr int kBudget = 227 * 1024 - 1024;        // minus alignment slack
    static constexpr int kStagesMax = (kBudget - kEpiBytes - kBarBytes) / kStage;
    static constexpr int kStages = kStagesMax > 8 ? 8 : kStagesMax;
    static constexpr int kTotal = kStages * kStage + kEpiBytes + kBarBytes + 1024;
    static constexpr uint32_t kTxBytes = (uint32_t)kStage * CTA_GROUP;
};

// tile index -> (group, m-tile, n-tile).  Within a group, tiles are numbered
// band by band: a band is `band` consecutive M-tiles, walked M-fastest.
__device__ __forceinline__ void tile_coords(const GemmShape& s, int t, int& g, int& tm, int& tn) {
    const int per_group = s.tiles_m * s.tiles_n;
    g = t / per_group;
    int r = t - g * per_group;
    const int band_tiles = s.band * s.tiles_n;
    const int b = r / band_tiles;
    r -= b * band_tiles;
    const int m0 = b * s.band;
    const int width = min(s.band, s.tiles_m - m0);
    tn = r / width;
    tm = m0 + (r - tn * width);
}

// Destinations of the "push" variant (EPI = 2): every finished tile is stored to the same
// coordinates of `n` extra [M, N] regions besides D.  The regions may be another GPU's memory
// mapped into this process (peer access over NVLink): with one region per rank, all at this
// rank's row offset of a gathered buffer, the all-gather of D happens tile by tile under the
// main loop of the following tiles.  The stores are plain (non-multicast) TMA stores.
constexpr int kMaxPushDest = 8;
struct PushMaps {
    CUtensorMap m[kMaxPushDest - 1];
    int n;
};
struct NoPush {};
template <int EPI> struct PushParam { using type = NoPush; };
template <> struct PushParam<2> { using type = PushMaps; };

// EPI = 0: D = accumulator.  EPI = 1 (grouped, 1-SM): the 256 accumulator columns of a tile are
// 128 "gate" columns followed by the matching 128 "up" columns of one expert, and the kernel
// writes silu(gate) * up (128 columns) -- the MoE up-projection with its activation fused.
//
// WIDE = 1: a tile is two row blocks of A (2 x 256 rows for 2-SM, 2 x 128 for 1-SM) against one
// block of B_T.
// The two accumulators take the whole TMEM (2 x 256 columns), so there is no second buffer for
// the next tile; in exchange every B tile fetched from L2 feeds twice the math (96 KiB per
// k-tile and CTA pair for 512 x 256 outputs instead of 128 KiB), which is what the kernel pays
// for in power at large sizes.  The epilogue drains the first accumulator, then the second; the
// next tile's MMAs into an accumulator start as soon as that one is drained.
template <int BN, int CTA_GROUP, typename OutT, bool DIRECT, int EPI = 0, int WIDE = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
            const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_d,
            OutT* __restrict__ d_ptr, GemmShape shape, int* status, int kernel_id,
            const int* __restrict__ expert_offsets,
            const __grid_constant__ typename PushParam<EPI>::type push) {
    using Plan = SmemPlan<BN, CTA_GROUP, WIDE>;
    static_assert(WIDE == 0 || (BN == 256 && EPI != 1), "the wide tile is a 256-column variant of the dense kernels");
    static_assert(EPI != 3 || (BN == 256 && !DIRECT), "the bias/activation epilogue is a dense, TMA-store variant");
    constexpr int kSub = 1 + WIDE;                            // 256-row blocks of A per tile
    constexpr int kStages = Plan::kStages;
    constexpr int kChunkCols = 128 / (int)sizeof(OutT);     // columns per 128-byte store row
    constexpr int kOutCols = EPI == 1 ? BN / 2 : BN;        // output columns per tile
    constexpr int kChunks = kOutCols / kChunkCols;
    static_assert(EPI != 2 || (BN == 256 && !DIRECT), "the push epilogue is a 256-column, TMA-store variant");
    static_assert(EPI != 1 || (BN == 256 && CTA_GROUP == 1 && !DIRECT), "the fused SwiGLU epilogue is a 1-SM, 256-column, TMA-store variant");
    constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    constexpr uint32_t kIdesc = make_idesc_f16(BM * CTA_GROUP, BN);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t s_a = smem_base;
    const uint32_t s_b = s_a + kStages * Plan::kABytes;
    const uint32_t s_epi = s_b + kStages * Plan::kBBytes;
    const uint32_t s_bar = s_epi + Plan::kEpiBytes;
    const uint32_t bar_full = s_bar;                       // [kStages]
    const uint32_t bar_empty = bar_full + 8 * kStages;     // [kStages]
    const uint32_t bar_tfull = bar_empty + 8 * kStages;    // [2]
    const uint32_t bar_tempty = bar_tfull + 16;            // [2]
    const uint32_t s_tmem_slot = bar_tempty + 16;
    const uint32_t s_abort = s_tmem_slot + 8;
    volatile uint32_t* tmem_slot_gen = (volatile uint32_t*)(smem_gen + (s_tmem_slot - smem_base));
    volatile int* abort_gen = (volatile int*)(smem_gen + (s_abort - smem_base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = CTA_GROUP == 2 ? cluster_ctarank() : 0u;
    const bool is_leader = cta_rank == 0;
    const int unit = CTA_GROUP == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;      // tile walker id
    const int n_units = CTA_GROUP == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    // Variable-size grouped GEMM: A and D are one stack of row blocks, expert e owning rows
    // [expert_offsets[e], expert_offsets[e+1]) (multiples of BM, so no tile straddles two experts);
    // only the row blocks below expert_offsets[n_experts] exist, and only the B tile depends on e.
    // (reads expert_offsets: only after pdl_wait)
    auto count_tiles = [&]() {
        return shape.n_experts > 0
            ? (min(__ldg(expert_offsets + shape.n_experts), shape.tiles_m * BM) / BM) * shape.tiles_n
            : shape.groups * shape.tiles_m * shape.tiles_n;
    };

    WaitCtx ctx{status, abort_gen, kernel_id};

    // TMA producer (thread 0), written as a resumable routine: with one CTA per tile walker
    // (CTA_GROUP == 1) the first ring-full of loads is issued before the CTA-wide set-up barrier,
    // so that the first tiles are in flight while TMEM is being allocated; the rest follows below.
    int p_tile = unit, p_kt = 0, p_stage = 0, p_row_a = 0, p_row_b = 0, p_tiles = 0;
    uint32_t p_phase = 0;
    bool p_ok = true;
    const uint32_t full_leader = CTA_GROUP == 2 ? map_to_cta(bar_full, 0) : bar_full;
    auto produce = [&](int max_loads) {
        for (int n = 0; n < max_loads && p_ok && p_tile < p_tiles; ++n) {
            if (p_kt == 0) {
                int g, tm, tn;
                tile_coords(shape, p_tile, g, tm, tn);
                p_row_a = g * shape.rows_per_group_a + (tm * CTA_GROUP * kSub + (int)cta_rank) * BM;
                if (shape.n_experts > 0) {
                    // which expert owns this row block (a handful of cached 4-byte loads per tile)
                    while (g + 1 < shape.n_experts && __ldg(expert_offsets + g + 1) <= p_row_a) ++g;
                }
                p_row_b = shape.n_experts > 0 ? g * shape.rows_per_group_b + tn * BN : EPI == 1 ? g * shape.rows_per_group_b + tn * (BN / 2)
                                              : g * shape.rows_per_group_b + tn * BN + (int)cta_rank * Plan::kBRows;
            }
            if (!(p_ok = mbar_wait(bar_empty + 8 * p_stage, p_phase ^ 1u, ctx, 1))) break;
            const uint32_t dst_a = s_a + p_stage * Plan::kABytes;
            const uint32_t dst_b = s_b + p_stage * Plan::kBBytes;
            if (CTA_GROUP == 1) {
                mbar_arrive_expect_tx(bar_full + 8 * p_stage, Plan::kTxBytes);
                tma_load_2d(dst_a, &tmap_a, bar_full + 8 * p_stage, p_kt * BK, p_row_a);
                if (WIDE) tma_load_2d(dst_a + BM * BK * 2, &tmap_a, bar_full + 8 * p_stage, p_kt * BK, p_row_a + BM);
                if (EPI == 1) {
                    // 128 gate rows, then the 128 up rows of the same feature block
                    tma_load_2d(dst_b, &tmap_b, bar_full + 8 * p_stage, p_kt * BK, p_row_b);
                    tma_load_2d(dst_b + (BN / 2) * BK * 2, &tmap_b, bar_full + 8 * p_stage, p_kt * BK, p_row_b + shape.up_row_off);
                } else {
                    tma_load_2d(dst_b, &tmap_b, bar_full + 8 * p_stage, p_kt * BK, p_row_b);
                }
            } else {
                if (is_leader) mbar_arrive_expect_tx(bar_full + 8 * p_stage, Plan::kTxBytes);
                tma_load_2d_pair(dst_a, &tmap_a, full_leader + 8 * p_stage, p_kt * BK, p_row_a);
                if (WIDE) tma_load_2d_pair(dst_a + BM * BK * 2, &tmap_a, full_leader + 8 * p_stage, p_kt * BK, p_row_a + CTA_GROUP * BM);
                tma_load_2d_pair(dst_b, &tmap_b, full_leader + 8 * p_stage, p_kt * BK, p_row_b);
            }
            if (++p_stage == kStages) { p_stage = 0; p_phase ^= 1u; }
            if (++p_kt == shape.k_tiles) { p_kt = 0; p_tile += n_units; }
        }
    };

    if (threadIdx.x == 0) {
        *abort_gen = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull + 8 * b, 1);
            mbar_init(bar_tempty + 8 * b, kEpiWarps * CTA_GROUP);
        }
        fence_mbarrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        if (!DIRECT) prefetch_tmap(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc<CTA_GROUP>(s_tmem_slot, kTmemCols);
        tmem_relinquish<CTA_GROUP>();
    }
    pdl_launch_dependents();
    if (CTA_GROUP == 1 && threadIdx.x == 0) {
        // The full barriers were initialised by this very thread, and only the MMA thread waits on
        // them (after the barrier below), so the first loads need not wait for the other warps.
        pdl_wait();
        p_tiles = count_tiles();
        produce(kStages);
    }
    tc_fence_before_sync();
    if (CTA_GROUP == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;
    // Set-up above overlaps the previous kernel's tail; global memory is touched only below.
    pdl_wait();
    const int n_tiles = count_tiles();

    if (warp == 0) {
        // ------------------------- TMA producer -------------------------
        if (lane == 0) {
            p_tiles = n_tiles;
            produce(0x7fffffff);
        }
    } else if (warp == 1) {
        // ------------------------- MMA issuer ---------------------------
        if (lane == 0 && is_leader) {
            // This thread is the serial resource of the kernel (it shares its scheduler with an
            // epilogue warp, and four MMAs retire every 512 clocks), so its loop carries running
            // barrier addresses and running descriptor low words instead of recomputing them; only
            // the 14-bit start-address field of a descriptor ever changes, and that is in the low word.
            int stage = 0; uint32_t phase = 0;
            const uint32_t empty_peer0 = CTA_GROUP == 2 ? map_to_cta(bar_empty, 1) : 0u;
            const uint32_t tfull_peer = CTA_GROUP == 2 ? map_to_cta(bar_tfull, 1) : 0u;
            const uint64_t da0 = make_desc_kmajor_sw128(s_a), db0 = make_desc_kmajor_sw128(s_b);
            const uint32_t a_hi = (uint32_t)(da0 >> 32), b_hi = (uint32_t)(db0 >> 32);
            const uint32_t a_lo0 = (uint32_t)da0, b_lo0 = (uint32_t)db0;
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            uint32_t full_cur = bar_full, empty_cur = bar_empty, empty_peer = empty_peer0;
            bool ok = true;
            int local = 0;
            for (int t = unit; t < n_tiles && ok; t += n_units, ++local) {
                // Narrow tile: accumulators alternate between the two TMEM buffers.  Wide tile: every
                // tile uses both (rows 0-255 in the first, 256-511 in the second).
                const int buf = WIDE ? 0 : (local & 1);
                const uint32_t acc_phase = WIDE ? ((uint32_t)local & 1u) : ((uint32_t)(local >> 1) & 1u);
                if (!(ok = mbar_wait(bar_tempty + 8 * buf, acc_phase ^ 1u, ctx, 2))) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kt = 0; kt < shape.k_tiles; ++kt) {
                    if (!(ok = mbar_wait(full_cur, phase, ctx, 3))) break;
                    tc_fence_after_sync();
                    // +32 bytes along K inside the 128-byte swizzle row = +2 in the encoded address.
                    umma_f16_ss_lohi<CTA_GROUP>(d_tmem, a_lo, a_hi, b_lo, b_hi, kIdesc, kt != 0 ? 1u : 0u);
                    umma_f16_ss_lohi<CTA_GROUP>(d_tmem, a_lo + 2, a_hi, b_lo + 2, b_hi, kIdesc, 1u);
                    umma_f16_ss_lohi<CTA_GROUP>(d_tmem, a_lo + 4, a_hi, b_lo + 4, b_hi, kIdesc, 1u);
                    umma_f16_ss_lohi<CTA_GROUP>(d_tmem, a_lo + 6, a_hi, b_lo + 6, b_hi, kIdesc, 1u);
                    if (WIDE) {
                        if (kt == shape.k_tiles - 1) {
                            // the first accumulator is complete: its drain overlaps the last MMAs of the second
                            umma_commit<CTA_GROUP>(bar_tfull);
                            if (CTA_GROUP == 2) umma_commit<CTA_GROUP>(tfull_peer);
                        }
                        if (kt == 0) {
                            if (!(ok = mbar_wait(bar_tempty + 8, acc_phase ^ 1u, ctx, 5))) break;
                            tc_fence_after_sync();
                        }
                        constexpr uint32_t kA1 = (uint32_t)(BM * BK * 2) >> 4;    // second A block of the stage
                        const uint32_t d1 = tmem_base + (uint32_t)BN;
                        umma_f16_ss_lohi<CTA_GROUP>(d1, a_lo + kA1, a_hi, b_lo, b_hi, kIdesc, kt != 0 ? 1u : 0u);
                        umma_f16_ss_lohi<CTA_GROUP>(d1, a_lo + kA1 + 2, a_hi, b_lo + 2, b_hi, kIdesc, 1u);
                        umma_f16_ss_lohi<CTA_GROUP>(d1, a_lo + kA1 + 4, a_hi, b_lo + 4, b_hi, kIdesc, 1u);
                        umma_f16_ss_lohi<CTA_GROUP>(d1, a_lo + kA1 + 6, a_hi, b_lo + 6, b_hi, kIdesc, 1u);
                    }
                    umma_commit<CTA_GROUP>(empty_cur);
                    if (CTA_GROUP == 2) umma_commit<CTA_GROUP>(empty_peer);
                    if (++stage == kStages) {
                        stage = 0; phase ^= 1u;
                        a_lo = a_lo0; b_lo = b_lo0; full_cur = bar_full; empty_cur = bar_empty; empty_peer = empty_peer0;
                    } else {
                        a_lo += Plan::kABytes >> 4; b_lo += Plan::kBBytes >> 4;
                        full_cur += 8; empty_cur += 8; empty_peer += 8;
                    }
                }
                if (!ok) break;
                if (WIDE) {
                    umma_commit<CTA_GROUP>(bar_tfull + 8);
                    if (CTA_GROUP == 2) umma_commit<CTA_GROUP>(tfull_peer + 8);
                } else {
                    umma_commit<CTA_GROUP>(bar_tfull + 8 * buf);
                    if (CTA_GROUP == 2) umma_commit<CTA_GROUP>(tfull_peer + 8 * buf);
                }
            }
        }
    } else {
        // ------------------------- epilogue (warps 2..5) -----------------
        const int q = warp & 3;                         // TMEM lane quarter this warp may read
        const int ew = warp - 2;                        // staging buffer owner index
        const uint32_t stage_buf = s_epi + (uint32_t)(ew * Plan::kEpiBufs) * kStageBytes;
        const uint32_t tempty_leader = CTA_GROUP == 2 ? map_to_cta(bar_tempty, 0) : bar_tempty;
        bool ok = true;
        int local = 0;
        int flip = 0;
        for (int t = unit; t < n_tiles && ok; t += n_units, ++local) {
            int g, tm, tn;
            tile_coords(shape, t, g, tm, tn);
            const int col0 = tn * kOutCols;
#pragma unroll 1
            for (int sub = 0; sub < kSub && ok; ++sub) {
            const int buf = WIDE ? sub : (local & 1);
            const uint32_t acc_phase = WIDE ? ((uint32_t)local & 1u) : ((uint32_t)(local >> 1) & 1u);
            const int row0 = g * shape.rows_per_group_a + ((tm * kSub + sub) * CTA_GROUP + (int)cta_rank) * BM + q * 32;
            ok = mbar_wait(bar_tfull + 8 * buf, acc_phase, ctx, 4);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
#pragma unroll 1
            for (int c = 0; c < kChunks; ++c) {
                uint32_t v[32];
                if (EPI == 1) {
                    // silu(gate) * up on kChunkCols columns: gate at column x, up at column 128 + x
#pragma unroll
                    for (int h = 0; h < kChunkCols / 32; ++h) {
                        uint32_t gt[32], up[32];
                        tmem_ld_32x32b_x32(t_row + (uint32_t)(c * kChunkCols + h * 32), gt);
                        tmem_ld_32x32b_x32(t_row + (uint32_t)(BN / 2 + c * kChunkCols + h * 32), up);
                        tmem_ld_wait();
                        if (sizeof(OutT) == 4) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const float gg = __uint_as_float(gt[i]);
                                v[i] = __float_as_uint(__fdividef(gg, 1.0f + __expf(-gg)) * __uint_as_float(up[i]));
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float g0 = __uint_as_float(gt[2 * i]), g1 = __uint_as_float(gt[2 * i + 1]);
                                __nv_bfloat162 pk = __floats2bfloat162_rn(
                                    __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(up[2 * i]),
                                    __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(up[2 * i + 1]));
                                v[h * 16 + i] = *reinterpret_cast<uint32_t*>(&pk);
                            }
                        }
                    }
                } else if (sizeof(OutT) == 4) {
                    tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
                    if (EPI == 3) apply_bias_act(v, reinterpret_cast<const float*>(expert_offsets), col0 + c * 32, shape);
                } else {
                    uint32_t lo[32], hi[32];
                    tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 64), lo);
                    tmem_ld_32x32b_x32(t_row + (uint32_t)(c * 64 + 32), hi);
                    tmem_ld_wait();
                    if (EPI == 3) {
                        apply_bias_act(lo, reinterpret_cast<const float*>(expert_offsets), col0 + c * 64, shape);
                        apply_bias_act(hi, reinterpret_cast<const float*>(expert_offsets), col0 + c * 64 + 32, shape);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1]));
                        v[i] = *reinterpret_cast<uint32_t*>(&p);
                        __nv_bfloat162 r = __floats2bfloat162_rn(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1]));
                        v[16 + i] = *reinterpret_cast<uint32_t*>(&r);
                    }
                }
                if (c == kChunks - 1) {
                    // All TMEM reads of this accumulator are done: hand it back to the MMA issuer.
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if (CTA_GROUP == 2) mbar_arrive_cluster(tempty_leader + 8 * buf);
                        else mbar_arrive(bar_tempty + 8 * buf);
                    }
                }
                if (DIRECT) {
                    OutT* dst = d_ptr + (size_t)(row0 + lane) * shape.n_total + col0 + c * kChunkCols;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        reinterpret_cast<uint4*>(dst)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
                    const uint32_t sb = stage_buf + (uint32_t)flip * kStageBytes;
                    // The store that last read this buffer was issued kEpiBufs chunks ago.
                    if (lane == 0) tma_store_wait_read<Plan::kEpiBufs - 1>();
                    __syncwarp();
                    const uint32_t row_addr = sb + (uint32_t)lane * 128u;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        st_shared_v4(row_addr + (uint32_t)((j ^ (lane & 7)) << 4),
                                     v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_d, sb, col0 + c * kChunkCols, row0);
                        if constexpr (EPI == 2) {
                            for (int i = 0; i < push.n; ++i)
                                tma_store_2d(&push.m[i], sb, col0 + c * kChunkCols, row0);
                        }
                        tma_store_commit();
                    }
                    flip = flip + 1 == Plan::kEpiBufs ? 0 : flip + 1;
                }
            }
            }   // sub
        }
        // Shared memory must outlive the stores' reads; the writes themselves complete with the grid.
        // The push variant waits for completion: a barrier kernel on the same stream follows it.
        if (!DIRECT && lane == 0) {
            if (EPI == 2) tma_store_wait_all<0>(); else tma_store_wait_read<0>();
        }
    }

    // ------------------------- teardown --------------------------------------
    tc_fence_before_sync();
    if (CTA_GROUP == 2) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc<CTA_GROUP>(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
int pick_bn(int64_t n) {
    if (n % 256 == 0) return 256;
    if (n % 128 == 0) return 128;
    if (n % 64 == 0) return 64;
    return 0;
}

// dims of the push kernel: {n_dest, cta_group, M, N, K}
//
// The 2-SM entry point runs a problem whose 128 x 256 tiles fit the SMs in ONE wave, but fill
// more than half of them, on the 1-SM shape: with one tile per CTA a pair buys no operand reuse
// worth its cluster set-up and tear-down (2048^3: 16.4 us against 18.3 us).  Every output element
// is the same fp32 sum over K in the same order either way, so the result bits do not change.
// tile="narrow" / "wide" (and the direct-store debug path) keep the pair shape.
int cta_group_of(const Record& r) {
    if (r.kernel_id == PB200_K_GEMM_PUSH) return (int)r.dims[1];
    if (r.kernel_id != PB200_K_GEMM_2SM) return 1;
    if (r.flags & (kForceNarrowTile | kForceWideTile | kDebugDirectStore)) return 2;
    if (r.n_dims >= 3) {
        const int64_t M = r.dims[r.n_dims - 3], N = r.dims[r.n_dims - 2];
        const int64_t tiles = (M / BM) * (N / 256);
        const int64_t sms = sm_count();
        if (M % BM == 0 && N % 256 == 0 && tiles <= sms && 2 * tiles > sms) return 1;
    }
    return 2;
}

constexpr uint32_t kForceBn256 = 1u << 20;        // create flag: the grouped kernel keeps 256-column tiles

// Tile width.  A fixed-size grouped problem whose 128 x 256 tiles would leave more than half of the
// SMs idle runs on 128 x 128 tiles, one per CTA on twice as many SMs (measured at G=4, M=2048,
// N=256, K=2048: 13.9 us against 15.3 us).  With more tiles than that the wider tile wins: the
// N=128 MMA needs 128 B/clk of shared-memory reads and runs below the N=256 rate.
int choose_bn(const Record& r) {
    const int64_t N = r.dims[r.n_dims - 2];
    const int bn = pick_bn(N);
    if (bn != 256 || r.kernel_id != PB200_K_GROUPED_GEMM || (r.flags & (kForceBn256 | kDebugDirectStore))) return bn;
    const int64_t tiles = r.dims[0] * (r.dims[1] / BM) * (N / 256);
    return 2 * tiles <= sm_count() ? 128 : 256;
}

bool is_grouped(int32_t kid) {
    return kid == PB200_K_GROUPED_GEMM || kid == PB200_K_GROUPED_GEMM_SWIGLU || kid == PB200_K_GROUPED_GEMM_VARLEN;
}

template <int BN, int CTA_GROUP, typename OutT, bool DIRECT, int EPI = 0, int WIDE = 0>
int launch_variant(const Record& r, cudaStream_t stream, void** p, const GemmShape& shape, char* err) {
    using Plan = SmemPlan<BN, CTA_GROUP, WIDE>;
    auto kernel = gemm_kernel<BN, CTA_GROUP, OutT, DIRECT, EPI, WIDE>;
    static std::atomic<uint64_t> attr_set{0};   // bit per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!(attr_set.load(std::memory_order_relaxed) & (1ull << (dev & 63)))) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kTotal);
        if (e != cudaSuccess) { set_err(err, "cudaFuncSetAttribute(smem=%d): %s", Plan::kTotal, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
        attr_set.fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
    }
    const bool varlen = r.kernel_id == PB200_K_GROUPED_GEMM_VARLEN;
    const int64_t G = is_grouped(r.kernel_id) && !varlen ? r.dims[0] : 1;     // varlen: M is already the stacked total
    const int64_t M = r.dims[r.n_dims - 3], N = r.dims[r.n_dims - 2], K = r.dims[r.n_dims - 1];
    const int64_t n_experts = varlen ? r.dims[0] : 0;
    void* out_ptr = p[varlen || (r.flags & PB200_F_BIAS) ? 3 : 2];
    // EPI 1: dims carry F; B_T holds 2F rows per expert (gate rows, then up rows), D has F columns.
    const int64_t b_rows = EPI == 1 ? 2 * N : varlen ? n_experts * N : N;
    const uint32_t b_box_rows = EPI == 1 ? (uint32_t)(BN / 2) : (uint32_t)Plan::kBRows;
    CUtensorMap ta, tb, td;
    {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)(G * M)};
        uint64_t str[1] = {(uint64_t)K * 2};
        uint32_t box[2] = {BK, BM};
        int rc = make_tensor_map(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p[0], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    }
    {
        uint64_t dims[2] = {(uint64_t)K, (uint64_t)(G * b_rows)};
        uint64_t str[1] = {(uint64_t)K * 2};
        uint32_t box[2] = {BK, b_box_rows};
        int rc = make_tensor_map(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p[1], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    }
    {
        uint64_t dims[2] = {(uint64_t)N, (uint64_t)(G * M)};
        uint64_t str[1] = {(uint64_t)N * sizeof(OutT)};
        uint32_t box[2] = {128 / sizeof(OutT), kStageRows};
        int rc = make_tensor_map(&td, sizeof(OutT) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                 2, out_ptr, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(r.geom.grid[0], 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = Plan::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTA_GROUP;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // programmatic dependent launch: see pdl_wait() in the kernel
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    OutT* d_ptr = (OutT*)out_ptr;
    typename PushParam<EPI>::type push{};
    if constexpr (EPI == 2) {
        push.n = (int)r.dims[0] - 1;
        for (int i = 0; i < push.n; ++i) {
            uint64_t dims[2] = {(uint64_t)N, (uint64_t)M};
            uint64_t str[1] = {(uint64_t)N * sizeof(OutT)};
            uint32_t box[2] = {128 / sizeof(OutT), kStageRows};
            int rc = make_tensor_map(&push.m[i], sizeof(OutT) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                     2, p[3 + i], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
            if (rc) return rc;
        }
    }
    const bool with_bias = EPI == 3 && (r.flags & PB200_F_BIAS);
    const int* expert_offsets = varlen || with_bias ? (const int*)p[2] : nullptr;   // aux pointer: offsets or bias
    int* status = device_status_ptr();
    int kid = r.kernel_id;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, td, d_ptr, shape, status, kid, expert_offsets, push);
    if (e != cudaSuccess) {
        set_err(err, "gemm launch failed (BN=%d cta_group=%d grid=%u smem=%d): %s", BN, CTA_GROUP, r.geom.grid[0],
                Plan::kTotal, cudaGetErrorString(e));
        return CTA_GROUP == 2 ? PB200_ERR_CLUSTER : PB200_ERR_LAUNCH;
    }
    return PB200_OK;
}

// Whether a dense problem runs on double-height tiles (512 x 256 per CTA pair, 256 x 256 per CTA).
// Measured faster at 4096^3 and 8192^3 (+2..8 %) and slower when they leave SMs without a tile
// (2048^3): they halve the number of tiles, so they are taken only when there is at least one
// full wave of them and the last wave stays about as full as with single-height tiles.
bool use_wide_tile(const Record& r, int64_t units) {
    if (is_grouped(r.kernel_id)) return false;
    if (r.flags & kForceNarrowTile) return false;
    if ((r.flags & kDebugDirectStore) && r.kernel_id == PB200_K_GEMM_PUSH) return false;
    const int64_t M = r.dims[r.n_dims - 3], N = r.dims[r.n_dims - 2];
    const int cg = cta_group_of(r);
    if (M % (2 * cg * BM) != 0) return false;
    if (r.flags & kForceWideTile) return true;
    if (units < 1) units = 1;
    const int64_t narrow = (M / (cg * BM)) * (N / 256), wide = narrow / 2;
    const double eff_n = (double)narrow / (double)(((narrow + units - 1) / units) * units);
    const double eff_w = (double)wide / (double)(((wide + units - 1) / units) * units);
    return wide >= units && eff_w >= eff_n - 0.04;
}

GemmShape make_shape(const Record& r, int bn, int cta_group, bool wide = false) {
    const bool varlen = r.kernel_id == PB200_K_GROUPED_GEMM_VARLEN;
    const int64_t G = is_grouped(r.kernel_id) && !varlen ? r.dims[0] : 1;
    const int64_t M = r.dims[r.n_dims - 3], N = r.dims[r.n_dims - 2], K = r.dims[r.n_dims - 1];
    const bool swiglu = r.kernel_id == PB200_K_GROUPED_GEMM_SWIGLU;
    GemmShape s;
    s.n_experts = varlen ? (int)r.dims[0] : 0;
    s.tiles_m = (int)(M / (BM * cta_group * (wide ? 2 : 1)));
    s.tiles_n = swiglu ? (int)(N / 128) : (int)(N / bn);
    s.k_tiles = (int)(K / BK);
    s.groups = (int)G;
    s.rows_per_group_a = (int)M;
    s.rows_per_group_b = swiglu ? (int)(2 * N) : (int)N;
    s.up_row_off = swiglu ? (int)N : 0;
    s.has_bias = (r.flags & PB200_F_BIAS) ? 1 : 0;
    s.act = (int)((r.flags & PB200_F_ACT_MASK) >> 4);
    int band = (int)r.dims[7];            // stored by plan_gemm
    s.band = band < 1 ? 1 : (band > s.tiles_m ? s.tiles_m : band);
    if (wide && (int)r.dims[6] == 0) s.band = s.band > 8 ? 8 : s.band;   // default band: 8 wide row blocks
    if (varlen) s.band = 1;     // row blocks in order, so that the active ones are a prefix of the tile list
    s.n_total = (int)N;
    return s;
}

}  // namespace

// dims: {M,N,K} (+ optional band) for the dense kernels, {G,M,N,K} (+ optional band) for grouped.
int plan_gemm(Record& r, char* err) {
    const bool grouped = is_grouped(r.kernel_id);
    const bool swiglu = r.kernel_id == PB200_K_GROUPED_GEMM_SWIGLU;
    const bool push = r.kernel_id == PB200_K_GEMM_PUSH;
    const int need = push ? 5 : grouped ? 4 : 3;
    if (push && r.n_dims >= 2) {
        if (r.dims[0] < 1 || r.dims[0] > kMaxPushDest) { set_err(err, "destination count must be in [1, %d]", kMaxPushDest); return PB200_ERR_BAD_SHAPE; }
        if (r.dims[1] != 1 && r.dims[1] != 2) { set_err(err, "cta_group must be 1 or 2"); return PB200_ERR_BAD_SHAPE; }
    }
    if (r.n_dims != need && r.n_dims != need + 1) {
        set_err(err, "gemm kernel %d needs %d dims (+1 optional raster band), got %d", r.kernel_id, need, r.n_dims);
        return PB200_ERR_BAD_SHAPE;
    }
    int64_t band = 16;
    const bool band_given = r.n_dims == need + 1;
    if (band_given) { band = r.dims[need]; r.n_dims = need; }
    if (band < 1) { set_err(err, "raster band must be at least 1"); return PB200_ERR_BAD_SHAPE; }
    r.dims[7] = band;
    r.dims[6] = band_given ? 1 : 0;
    const bool varlen = r.kernel_id == PB200_K_GROUPED_GEMM_VARLEN;
    const int64_t G = grouped && !varlen ? r.dims[0] : 1;
    if (varlen && (r.dims[0] < 1 || r.dims[0] > 65536)) { set_err(err, "expert count must be in [1, 65536]"); return PB200_ERR_BAD_SHAPE; }
    const int64_t M = r.dims[need - 3], N = r.dims[need - 2], K = r.dims[need - 1];
    const int cta_group = cta_group_of(r);
    if ((r.flags & (PB200_F_BIAS | PB200_F_ACT_MASK)) && r.kernel_id != PB200_K_GEMM_1SM && r.kernel_id != PB200_K_GEMM_2SM) {
        set_err(err, "bias / activation flags apply to the dense GEMM kernels only");
        return PB200_ERR_BAD_SHAPE;
    }
    if ((r.flags & (PB200_F_BIAS | PB200_F_ACT_MASK)) && (r.flags & kDebugDirectStore)) {
        set_err(err, "the direct-store debug path has no bias / activation epilogue");
        return PB200_ERR_BAD_SHAPE;
    }
    if (G < 1 || M < 1 || N < 1 || K < 1) { set_err(err, "G, M, N, K must be positive"); return PB200_ERR_BAD_SHAPE; }
    const int m_unit = r.kernel_id == PB200_K_GEMM_2SM ? 2 * BM : BM * cta_group;     // the 2-SM entry keeps its rule on every shape
    if (M % m_unit != 0) { set_err(err, "M=%lld must be divisible by %d", (long long)M, m_unit); return PB200_ERR_BAD_SHAPE; }
    if (K % BK != 0) { set_err(err, "K=%lld must be divisible by %d", (long long)K, BK); return PB200_ERR_BAD_SHAPE; }
    if (swiglu && N % 128 != 0) { set_err(err, "F=%lld must be divisible by 128", (long long)N); return PB200_ERR_BAD_SHAPE; }
    const int bn = swiglu ? 256 : choose_bn(r);
    if (bn == 0 || (!grouped && bn != 256)) {
        set_err(err, "N=%lld must be divisible by %d", (long long)N, grouped ? 64 : 256);
        return PB200_ERR_BAD_SHAPE;
    }
    if (G * M > 0x7fffffffLL || G * N > 0x7fffffffLL || K > 0x7fffffffLL) { set_err(err, "extent exceeds 2^31-1"); return PB200_ERR_BAD_SHAPE; }
    const int64_t tiles = G * (M / (BM * cta_group)) * (swiglu ? N / 128 : N / bn);
    int64_t units = sm_count() / cta_group;
    if (units > tiles) units = tiles;
    pb200_geometry& g = r.geom;
    g.grid[0] = (uint32_t)(units * cta_group); g.grid[1] = g.grid[2] = 1;
    g.block[0] = kThreads; g.block[1] = g.block[2] = 1;
    g.cluster[0] = (uint32_t)cta_group; g.cluster[1] = g.cluster[2] = 1;
    const bool wide = bn == 256 && use_wide_tile(r, sm_count() / cta_group);
    g.smem_bytes = bn == 256 ? (cta_group == 2 ? (wide ? SmemPlan<256, 2, 1>::kTotal : SmemPlan<256, 2>::kTotal)
                                               : (wide ? SmemPlan<256, 1, 1>::kTotal : SmemPlan<256, 1>::kTotal))
                 : bn == 128 ? SmemPlan<128, 1>::kTotal : SmemPlan<64, 1>::kTotal;
    g.n_inputs = varlen || (r.flags & PB200_F_BIAS) ? 3 : 2; g.n_outputs = push ? (uint32_t)r.dims[0] : 1;
    return PB200_OK;
}

int launch_gemm(const Record& r, cudaStream_t stream, void** p, char* err) {
    const int64_t N = r.dims[r.n_dims - 2];
    const bool swiglu = r.kernel_id == PB200_K_GROUPED_GEMM_SWIGLU;
    const int bn = swiglu ? 256 : choose_bn(r);
    const int cta_group = cta_group_of(r);
    const bool bf16_out = (r.flags & PB200_F_OUT_BF16) != 0;
    const bool direct = (r.flags & kDebugDirectStore) != 0;
    Record rr = r;
    // The grid was planned without a device; clamp it to this device's SM count.
    {
        const int64_t units = sm_count() / cta_group;
        if ((int64_t)rr.geom.grid[0] > units * cta_group) rr.geom.grid[0] = (uint32_t)(units * cta_group);
    }
    const bool wide = !swiglu && bn == 256 && use_wide_tile(rr, sm_count() / cta_group);
    GemmShape shape = make_shape(rr, bn, cta_group, wide);
    if (wide) {
#define PB200_WIDE_CASE(CG_, EPI_)                                                                       \
        return bf16_out ? launch_variant<256, CG_, __nv_bfloat16, false, EPI_, 1>(rr, stream, p, shape, err) \
                        : launch_variant<256, CG_, float, false, EPI_, 1>(rr, stream, p, shape, err);
        if (r.kernel_id == PB200_K_GEMM_PUSH) {
            if (cta_group == 2) { PB200_WIDE_CASE(2, 2) }
            PB200_WIDE_CASE(1, 2)
        }
        if (r.flags & (PB200_F_BIAS | PB200_F_ACT_MASK)) {
            if (cta_group == 2) { PB200_WIDE_CASE(2, 3) }
            PB200_WIDE_CASE(1, 3)
        }
        if (direct) {
            if (cta_group == 2)
                return bf16_out ? launch_variant<256, 2, __nv_bfloat16, true, 0, 1>(rr, stream, p, shape, err)
                                : launch_variant<256, 2, float, true, 0, 1>(rr, stream, p, shape, err);
            return bf16_out ? launch_variant<256, 1, __nv_bfloat16, true, 0, 1>(rr, stream, p, shape, err)
                            : launch_variant<256, 1, float, true, 0, 1>(rr, stream, p, shape, err);
        }
        if (cta_group == 2) { PB200_WIDE_CASE(2, 0) }
        PB200_WIDE_CASE(1, 0)
#undef PB200_WIDE_CASE
    }
    if (swiglu)
        return bf16_out ? launch_variant<256, 1, __nv_bfloat16, false, 1>(rr, stream, p, shape, err)
                        : launch_variant<256, 1, float, false, 1>(rr, stream, p, shape, err);
    if (r.kernel_id == PB200_K_GEMM_PUSH) {
        if (cta_group == 2)
            return bf16_out ? launch_variant<256, 2, __nv_bfloat16, false, 2>(rr, stream, p, shape, err)
                            : launch_variant<256, 2, float, false, 2>(rr, stream, p, shape, err);
        return bf16_out ? launch_variant<256, 1, __nv_bfloat16, false, 2>(rr, stream, p, shape, err)
                        : launch_variant<256, 1, float, false, 2>(rr, stream, p, shape, err);
    }
    if (r.flags & (PB200_F_BIAS | PB200_F_ACT_MASK)) {
        if (cta_group == 2)
            return bf16_out ? launch_variant<256, 2, __nv_bfloat16, false, 3>(rr, stream, p, shape, err)
                            : launch_variant<256, 2, float, false, 3>(rr, stream, p, shape, err);
        return bf16_out ? launch_variant<256, 1, __nv_bfloat16, false, 3>(rr, stream, p, shape, err)
                        : launch_variant<256, 1, float, false, 3>(rr, stream, p, shape, err);
    }
#define PB200_GEMM_CASE(BN_, CG_)                                                                       \
    if (bn == BN_ && cta_group == CG_) {                                                                \
        if (bf16_out) return direct ? launch_variant<BN_, CG_, __nv_bfloat16, true>(rr, stream, p, shape, err)  \
                                    : launch_variant<BN_, CG_, __nv_bfloat16, false>(rr, stream, p, shape, err); \
        return direct ? launch_variant<BN_, CG_, float, true>(rr, stream, p, shape, err)               \
                      : launch_variant<BN_, CG_, float, false>(rr, stream, p, shape, err);             \
    }
    PB200_GEMM_CASE(256, 1)
    PB200_GEMM_CASE(256, 2)
    PB200_GEMM_CASE(128, 1)
    PB200_GEMM_CASE(64, 1)
#undef PB200_GEMM_CASE
    set_err(err, "no gemm variant for BN=%d cta_group=%d", bn, cta_group);
    return PB200_ERR_BAD_SHAPE;
}

}  // namespace pb200
