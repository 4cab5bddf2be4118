// Flash-attention backward for sm_100a on tcgen05 tensor cores.
//   given Q, K, V, O, dO (bf16) and the forward's row statistic lse (f32):
//     P  = exp(scale * Q K^T - lse)            (recomputed, never stored)
//     dV = P^T dO        dP = dO V^T        dS = P o (dP - delta),  delta_i = sum_c O_ic dO_ic
//     dQ = scale * dS K  dK = scale * dS^T Q
// The reference ships the autograd hook for such a pair (pyptx/torch_support.py:446-519) and keeps
// the row statistics of its forward in registers (examples/hopper/experimental/
// flash_attention_hopper.py:205-256); it has no backward kernel.  The arithmetic follows the
// forward here: bf16 operands, fp32 accumulation, P and dS rounded to bf16 before they become
// MMA operands.
//
// ONE kernel template in three modes, plus a whole-tile fused kernel for head_dim <= 64 (further
// down).  The default is a fused pass (MODE 2 at head_dim > 64): five MMAs per tile pair, dQ summed
// over key tiles with fp32 reductions into a scratch buffer (not bit-reproducible).
// With PB200_F_DETERMINISTIC two passes run instead (MODE 0, then MODE 1), so that no gradient needs
// atomics and the result is bit-reproducible, at seven MMAs per tile pair (S and dP formed twice):
//   MODE 0 (dK, dV): a CTA owns 128 keys (K, V tiles stay in shared memory) and streams the query
//          tiles (Q, dO).  Scores are computed transposed, S^T = K Q^T and dP^T = V dO^T, so that
//          keys are TMEM lanes and P^T / dS^T can be fed back as the TMEM A operand of
//          dV += P^T dO and dK += dS^T Q (Q and dO tiles consumed as MN-major B operands).
//   MODE 1 (dQ):     a CTA owns 128 queries (Q, dO stay) and streams K, V: S = Q K^T, dP = dO V^T,
//          dS as the TMEM A operand of dQ += dS K.
//   MODE 2 (dK, dV, dQ): MODE 0 with dQ^T = K^T dS^T formed per tile pair; see the kernel's comment.
//   warp 0      TMA producer (stationary pair once, streamed pairs through a ring)
//   warp 1      MMA issuer (single thread)
//   warps 4-7   score math for streamed columns 0-63    (one TMEM lane per thread)
//   warps 8-11  score math for streamed columns 64-127
// TMEM: X1 (S) | X2 (dP) | acc A | acc B, 128 columns each.  The two math warpgroups ping-pong: each
// owns one 64-row half of every streamed tile, with its own score MMAs (N = 64), its own barriers
// and its own half of the S / dP columns, so that while one warpgroup does its score math the tensor
// core runs the other's MMAs.  P overwrites the head of a warpgroup's own S columns, dS the same of
// dP, so no warpgroup writes where the other still reads, and the next scores of a half follow the
// MMAs that read its P and dS (MMAs of one thread execute in issue order).
// A small row kernel first writes delta and lse * log2(e) into scratch, padded to whole tiles
// (padding rows get lse = +inf, i.e. P = 0).  Every mbarrier wait is bounded.
#include "common.cuh"
#include "fmha_math.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <cmath>

namespace pb200 {
namespace {

using namespace ptx;

constexpr int kTile = 128;            // rows of a stationary tile = rows of a streamed tile
constexpr int kBwdThreads = 384;
constexpr int kBwdLaunchRegs = 168;     // registers per thread at launch (65536 / 384, multiple of 8)
constexpr int kBwdRegsIssue = 88;       // TMA / MMA warpgroup after setmaxnreg
constexpr int kBwdRegsMath = 208;       // the two score-math warpgroups
static_assert(kBwdRegsIssue * 128 + kBwdRegsMath * 256 <= kBwdLaunchRegs * kBwdThreads,
              "setmaxnreg may only hand around the registers the CTA was launched with");
#ifndef PB200_BWD_FMA_EXP_PAIRS
#define PB200_BWD_FMA_EXP_PAIRS 0       // of every 8 score pairs, how many take the FMA-pipe exp2 (0..3 measured within 3 %)
#endif

struct BwdParams {
    int bh, s_q, s_kv, sq_pad;
    int causal, causal_offset;        // query i sees keys j <= i + offset
    float scale, scale_log2;
    int hd;                            // head dimension of the tensors (multiple of 8, <= HD)
};

template <int HD, bool FUSED>
struct BwdSmem {
    static constexpr int kStages = HD == 64 ? 3 : 2;
    static constexpr int kTileBytes = kTile * HD * 2;
    static constexpr int kDsBytes = kTile * 128;                        // dS^T of one warpgroup: 128 keys x 64 queries, bf16
    static constexpr int kOffStat = 0;                                  // two stationary tiles
    static constexpr int kOffRing = 2 * kTileBytes;                     // kStages x two streamed tiles
    static constexpr int kOffDs = kOffRing + kStages * 2 * kTileBytes;  // fused pass: dS^T of both warpgroups
    static constexpr int kOffBar = kOffDs + (FUSED ? 2 * kDsBytes : 0);
    static constexpr int kOffStats = kOffBar + 256;                     // key-stationary passes: lse2 / delta of the streamed queries
    static constexpr int kStatSets = FUSED ? 1 : 2;                     // buffers per warpgroup
    static constexpr int kTotal = kOffStats + kStatSets * 2 * 128 * 4 + 1024;
    static_assert(kTotal <= 227 * 1024, "shared memory budget exceeded");
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);      // .x = a in the low half
    return *reinterpret_cast<uint32_t*>(&v);
}

// 32 accumulator columns of one row -> global (the first cols_here of them exist), scaled.
template <typename OutT>
__device__ __forceinline__ void store_row_chunk(OutT* dst, const uint32_t (&o)[32], int cols_here, float mul) {
    if (sizeof(OutT) == 4) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (4 * i < cols_here)
                reinterpret_cast<float4*>(dst)[i] =
                    make_float4(__uint_as_float(o[4 * i]) * mul, __uint_as_float(o[4 * i + 1]) * mul,
                                __uint_as_float(o[4 * i + 2]) * mul, __uint_as_float(o[4 * i + 3]) * mul);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (8 * i < cols_here)
                reinterpret_cast<uint4*>(dst)[i] =
                    make_uint4(pack_bf16(__uint_as_float(o[8 * i]) * mul, __uint_as_float(o[8 * i + 1]) * mul),
                               pack_bf16(__uint_as_float(o[8 * i + 2]) * mul, __uint_as_float(o[8 * i + 3]) * mul),
                               pack_bf16(__uint_as_float(o[8 * i + 4]) * mul, __uint_as_float(o[8 * i + 5]) * mul),
                               pack_bf16(__uint_as_float(o[8 * i + 6]) * mul, __uint_as_float(o[8 * i + 7]) * mul));
    }
}

// delta[bh, i] = sum_c O[bh, i, c] * dO[bh, i, c];  lse2[bh, i] = lse[bh, i] * log2(e).
// One warp per row; rows in [s_q, sq_pad) are written as (0, +inf).
__global__ void __launch_bounds__(256)
fmha_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                     const float* __restrict__ lse, float* __restrict__ delta, float* __restrict__ lse2,
                     int bh, int s_q, int sq_pad, int hd) {
    const int warp = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (warp >= bh * sq_pad) return;
    const int b = warp / sq_pad, i = warp - b * sq_pad;
    if (i >= s_q) {
        if (lane == 0) { delta[warp] = 0.f; lse2[warp] = INFINITY; }
        return;
    }
    const size_t row = ((size_t)b * s_q + i) * hd;
    float acc = 0.f;
    for (int c = lane * 8; c < hd; c += 256) {          // hd is a multiple of 8: 16-byte loads
        const uint4 a = *reinterpret_cast<const uint4*>(o + row + c);
        const uint4 g = *reinterpret_cast<const uint4*>(d_o + row + c);
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pg = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 fa = __bfloat1622float2(pa[k]), fg = __bfloat1622float2(pg[k]);
            acc = fmaf(fa.x, fg.x, acc);
            acc = fmaf(fa.y, fg.y, acc);
        }
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (lane == 0) {
        delta[warp] = acc;
        lse2[warp] = lse[(size_t)b * s_q + i] * 1.4426950408889634f;
    }
}

// dQ[bh, i, c] = scale * dq_acc[bh, i, c] for i < s_q, c < hd (dq_acc rows are HD_TILE floats, sq_pad rows per head).
template <typename OutT>
__global__ void __launch_bounds__(256)
fmha_bwd_dq_finish_kernel(const float* __restrict__ dq_acc, OutT* __restrict__ dq, int bh, int s_q, int sq_pad,
                          int hd, int hd_tile, float scale) {
    const int quads = hd >> 2;                            // hd is a multiple of 8
    const size_t n = (size_t)bh * s_q * quads;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const int c4 = (int)(idx % quads);
        const size_t rowi = idx / quads;
        const int i = (int)(rowi % s_q);
        const size_t b = rowi / s_q;
        const float4 v = *reinterpret_cast<const float4*>(dq_acc + (b * sq_pad + i) * hd_tile + 4 * c4);
        OutT* dst = dq + rowi * hd + 4 * c4;
        if (sizeof(OutT) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
        } else {
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(v.x * scale, v.y * scale), pack_bf16(v.z * scale, v.w * scale));
        }
    }
}

// MODE 0: stationary = (K, V), streamed = (Q, dO), outputs dV (acc A) and dK (acc B).
// MODE 1: stationary = (Q, dO), streamed = (K, V), output dQ (acc B).
// MODE 2: MODE 0 plus dQ in the same pass (five MMAs per tile pair).  dS^T goes to shared memory
//         instead of TMEM: it is the K-major A operand of dK += dS^T Q and the MN-major B operand of
//         dQ^T = K^T dS^T (K tile as MN-major A, M = head_dim padded to 128 lanes, N = the
//         warpgroup's 64 queries), which lands in the warpgroup's own dP columns once dP has been
//         read.  The warpgroup reads it back (lane = head-dim index, column = query) and adds it
//         to an fp32 accumulation buffer dq_acc[bh][sq_pad][HD] with red.global.add: coalesced
//         128-byte rows, no ordering between key tiles, so dQ is not bit-reproducible from run to
//         run.  A row kernel scales and rounds dq_acc afterwards.
template <int HD, int MODE, typename OutT>
__global__ void __launch_bounds__(kBwdThreads, 1)
fmha_bwd_kernel(const __grid_constant__ CUtensorMap tmap_s1, const __grid_constant__ CUtensorMap tmap_s2,
                const __grid_constant__ CUtensorMap tmap_m1, const __grid_constant__ CUtensorMap tmap_m2,
                const float* __restrict__ lse2, const float* __restrict__ delta,
                OutT* __restrict__ out_a, OutT* __restrict__ out_b, float* __restrict__ dq_acc, BwdParams prm, int* status) {
    constexpr bool kFused = MODE == 2;
    static_assert(!kFused || HD == 128, "head_dim <= 64 takes the whole-tile fused kernel below");
    constexpr bool kKeyStat = MODE != 1;           // keys stationary, queries streamed
    using L = BwdSmem<HD, kFused>;
    constexpr int kStages = L::kStages;
    constexpr int kDBlocks = HD / 64;
    constexpr int kHalf = kTile / 2;                                             // streamed rows per warpgroup
    constexpr uint32_t kIdescX = make_idesc_f16(kTile, kHalf, true, 0, 0);      // both operands K-major
    constexpr uint32_t kIdescAcc = make_idesc_f16(kTile, HD, true, 0, 1);       // B operand MN-major
    constexpr uint32_t kIdescDq = make_idesc_f16(kTile, kHalf, true, 1, 1);     // both operands MN-major

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t s_stat = base + L::kOffStat, s_ring = base + L::kOffRing;
    const uint32_t bars = base + L::kOffBar;
    const uint32_t bar_stat = bars;                       // [1]
    const uint32_t bar_full = bars + 8;                   // [kStages]
    const uint32_t bar_empty = bar_full + 8 * kStages;    // [kStages]
    const uint32_t bar_xfull = bar_empty + 8 * kStages;   // [2] S and dP of a warpgroup's half tile are in TMEM
    const uint32_t bar_pready = bar_xfull + 16;           // [2] its P and dS are written (4 warps)
    const uint32_t bar_outfull = bar_pready + 16;         // [1] accumulators complete
    const uint32_t bar_dqfull = bar_outfull + 8;          // [2] fused: dQ^T of a warpgroup's half tile is in TMEM
    const uint32_t bar_dqfree = bar_dqfull + 16;          // [2] fused: ... and has been read (4 warps)
    float* stats_gen = reinterpret_cast<float*>(gen + L::kOffStats);    // [parity][warpgroup][64 lse2 | 64 delta]
    const uint32_t s_ds = base + L::kOffDs;
    const uint32_t s_tmem_slot = bar_dqfree + 16;
    const uint32_t s_abort = s_tmem_slot + 8;
    volatile uint32_t* tmem_slot_gen = (volatile uint32_t*)(gen + (s_tmem_slot - base));
    volatile int* abort_gen = (volatile int*)(gen + (s_abort - base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Stationary tile: MODE 0 counts key tiles (tile 0 meets every query tile under the causal mask),
    // MODE 1 query tiles from the last (which meets every key tile) down: heaviest first.  Causal
    // launches deal the tiles out heaviest-first across a group of heads at a time (CTAs start in
    // linear block order, x fastest), so that the grid ends on light tiles; groups of 16 heads keep
    // the operands of the CTAs in flight inside L2.
    constexpr int kHeadGroup = 16;
    int bh = (int)blockIdx.y;
    int heavy_rank = (int)blockIdx.x;                   // 0 = heaviest
    if (prm.causal) {
        const int n_st = (int)gridDim.x;
        const int lin = (int)blockIdx.x + n_st * (int)blockIdx.y;
        const int grp = lin / (n_st * kHeadGroup);
        const int rem = lin - grp * (n_st * kHeadGroup);
        const int heads_here = min(kHeadGroup, (int)gridDim.y - grp * kHeadGroup);
        heavy_rank = rem / heads_here;
        bh = grp * kHeadGroup + rem % heads_here;
    }
    const int st = kKeyStat ? heavy_rank : (int)gridDim.x - 1 - heavy_rank;
    const int st0 = st * kTile;
    // Range of streamed tiles [m_begin, m_end).
    int m_begin = 0, m_end;
    if (kKeyStat) {
        m_end = (prm.s_q + kTile - 1) / kTile;
        if (prm.causal) m_begin = min(max(st0 - prm.causal_offset, 0) / kTile, m_end);   // first query that sees key st0
    } else {
        m_end = (prm.s_kv + kTile - 1) / kTile;
        if (prm.causal) m_end = min(m_end, max((st0 + kTile - 1 + prm.causal_offset) / kTile + 1, 1));
    }
    const int n_iter = m_end - m_begin;

    WaitCtx ctx{status, abort_gen, PB200_K_FLASH_ATTN_BWD};

    if (threadIdx.x == 0) {
        *abort_gen = 0;
        mbar_init(bar_stat, 1);
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int w = 0; w < 2; ++w) {
            mbar_init(bar_xfull + 8 * w, 1); mbar_init(bar_pready + 8 * w, 4);
            mbar_init(bar_dqfull + 8 * w, 1); mbar_init(bar_dqfree + 8 * w, 4);
        }
        mbar_init(bar_outfull, 1);
        fence_mbarrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_s1); prefetch_tmap(&tmap_s2); prefetch_tmap(&tmap_m1); prefetch_tmap(&tmap_m2);
    }
    if (warp == 1) {
        tmem_alloc<1>(s_tmem_slot, 512);
        tmem_relinquish<1>();
    }
    pdl_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_wait();      // set-up above overlaps the previous kernel's tail; global memory is touched only below
    const uint32_t tmem_base = *tmem_slot_gen;
    const uint32_t tmem_x1 = tmem_base, tmem_x2 = tmem_base + 128u;
    const uint32_t tmem_acc_a = tmem_base + 256u, tmem_acc_b = tmem_base + 384u;
    // dQ^T of warpgroup w (fused pass): over its own dP^T columns
    const uint32_t tmem_dq[2] = {tmem_x2, tmem_x2 + (uint32_t)(kTile / 2)};

    if (warp < 4) {
    reg_dealloc<kBwdRegsIssue>();
    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0 && n_iter > 0) {
            mbar_arrive_expect_tx(bar_stat, (uint32_t)(2 * L::kTileBytes));
            for (int db = 0; db < kDBlocks; ++db) {
                tma_load_3d(s_stat + db * (kTile * 128), &tmap_s1, bar_stat, db * 64, st0, bh);
                tma_load_3d(s_stat + L::kTileBytes + db * (kTile * 128), &tmap_s2, bar_stat, db * 64, st0, bh);
            }
            int stage = 0; uint32_t phase = 0;
            for (int it = 0; it < n_iter; ++it) {
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, ctx, 11)) break;
                const uint32_t dst = s_ring + stage * 2 * L::kTileBytes;
                mbar_arrive_expect_tx(bar_full + 8 * stage, (uint32_t)(2 * L::kTileBytes));
                for (int db = 0; db < kDBlocks; ++db) {
                    tma_load_3d(dst + db * (kTile * 128), &tmap_m1, bar_full + 8 * stage, db * 64, (m_begin + it) * kTile, bh);
                    tma_load_3d(dst + L::kTileBytes + db * (kTile * 128), &tmap_m2, bar_full + 8 * stage, db * 64,
                                (m_begin + it) * kTile, bh);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0 && n_iter > 0) {
            bool ok = mbar_wait(bar_stat, 0, ctx, 21);
            const uint64_t sd = make_desc_kmajor_sw128(s_stat);
            const uint64_t md = make_desc_kmajor_sw128(s_ring);
            const uint64_t bd = make_smem_desc(s_ring, kTile * 128, 1024, 2);       // streamed tile as MN-major B
            const uint32_t s_lo = (uint32_t)sd, s_hi = (uint32_t)(sd >> 32);
            const uint32_t m_lo = (uint32_t)md, m_hi = (uint32_t)(md >> 32);
            const uint32_t b_lo = (uint32_t)bd, b_hi = (uint32_t)(bd >> 32);
            constexpr uint32_t kTileDesc = (uint32_t)(L::kTileBytes >> 4);
            // X_t[:, 64 w ..] = stationary tile t . (rows 64 w .. of streamed tile t)^T, contraction over head_dim
            auto issue_x = [&](int w, int stage) {
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    const uint32_t a = s_lo + (uint32_t)t * kTileDesc;
                    const uint32_t b = m_lo + (uint32_t)(stage * 2 + t) * kTileDesc + (uint32_t)(w * ((kHalf * 128) >> 4));
                    const uint32_t d = (t == 0 ? tmem_x1 : tmem_x2) + (uint32_t)(w * kHalf);
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k) {
                        const uint32_t off = (uint32_t)((k >> 2) * (kTile * 8) + (k & 3) * 2);
                        umma_f16_ss_lohi(d, a + off, s_hi, b + off, m_hi, kIdescX, k != 0 ? 1u : 0u);
                    }
                }
            };
            // acc += (P or dS of warpgroup w, from TMEM) . rows 64 w .. of streamed tile t: contraction
            // over those 64 rows.  The operand sits at the head of the warpgroup's own 64 columns.
            auto issue_acc = [&](uint32_t acc, uint32_t a_tmem, int t, int w, int stage, bool first) {
                const uint32_t b = b_lo + (uint32_t)(stage * 2 + t) * kTileDesc + (uint32_t)(w * ((kHalf * 128) >> 4));
#pragma unroll
                for (int k = 0; k < kHalf / 16; ++k)
                    umma_f16_ts_lohi(acc, a_tmem + (uint32_t)(w * kHalf + k * 8), b + (uint32_t)(k * 128), b_hi,
                                     kIdescAcc, (first && k == 0) ? 0u : 1u);
            };
            // fused pass: dK += dS^T_w Q_w with dS^T from shared memory (K-major A: one 128-byte row per key)
            const uint64_t dsk = make_desc_kmajor_sw128(s_ds);
            const uint64_t dsm = make_smem_desc(s_ds, kTile * 128, 1024, 2);         // the same bytes as MN-major B
            const uint64_t ktd = make_smem_desc(s_stat, kTile * 128, 1024, 2);       // K tile as MN-major A (M = head_dim)
            auto issue_dk_ss = [&](int w, int stage, bool first) {
                const uint32_t a = (uint32_t)dsk + (uint32_t)(w * (L::kDsBytes >> 4));
                const uint32_t b = b_lo + (uint32_t)(stage * 2) * kTileDesc + (uint32_t)(w * ((kHalf * 128) >> 4));
#pragma unroll
                for (int k = 0; k < kHalf / 16; ++k)
                    umma_f16_ss_lohi(tmem_acc_b, a + (uint32_t)(k * 2), (uint32_t)(dsk >> 32), b + (uint32_t)(k * 128), b_hi,
                                     kIdescAcc, (first && k == 0) ? 0u : 1u);
            };
            // dQ^T_w = K^T dS^T_w: contraction over the 128 keys, 16 per step (2048 bytes in both operands)
            auto issue_dq = [&](int w) {
                const uint32_t b = (uint32_t)dsm + (uint32_t)(w * (L::kDsBytes >> 4));
#pragma unroll
                for (int k = 0; k < kTile / 16; ++k)
                    umma_f16_ss_lohi(tmem_dq[w], (uint32_t)ktd + (uint32_t)(k * 128), (uint32_t)(ktd >> 32),
                                     b + (uint32_t)(k * 128), (uint32_t)(dsm >> 32), kIdescDq, k != 0 ? 1u : 0u);
            };
            int stage = 0; uint32_t phase = 0;
            if (ok) ok = mbar_wait(bar_full, 0, ctx, 22);
            if (ok) {
                tc_fence_after_sync();
                issue_x(0, 0); umma_commit<1>(bar_xfull);
                issue_x(1, 0); umma_commit<1>(bar_xfull + 8);
            }
            for (int it = 0; it < n_iter && ok; ++it) {
                int nstage = stage + 1; uint32_t nphase = phase;
                if (nstage == kStages) { nstage = 0; nphase ^= 1u; }
                const bool more = it + 1 < n_iter;
                if (more && !(ok = mbar_wait(bar_full + 8 * nstage, nphase, ctx, 24))) break;
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    if (!(ok = mbar_wait(bar_pready + 8 * w, (uint32_t)it & 1u, ctx, 23))) break;
                    tc_fence_after_sync();
                    // Fused: dQ^T first, so that the warpgroup reads it while dV and dK run and the next dP^T
                    // of this half (which overwrites it) is not held up (+2.5 % against dV, dK, dQ^T).
                    if (kFused) { issue_dq(w); umma_commit<1>(bar_dqfull + 8 * w); }
                    if (kKeyStat) issue_acc(tmem_acc_a, tmem_x1, 1, w, stage, it == 0 && w == 0);     // dV += P^T dO
                    if (kFused) {
                        issue_dk_ss(w, stage, it == 0 && w == 0);
                    } else {
                        issue_acc(tmem_acc_b, tmem_x2, 0, w, stage, it == 0 && w == 0);                // dK += dS^T Q  /  dQ += dS K
                    }
                    if (w == 1) umma_commit<1>(bar_empty + 8 * stage);
                    if (!kFused && more) { issue_x(w, nstage); umma_commit<1>(bar_xfull + 8 * w); }
                }
                if (!ok) break;
                if (kFused && more) {
                    // the next dP^T of a half overwrites its dQ^T: wait until the warpgroup has read it
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        if (!(ok = mbar_wait(bar_dqfree + 8 * w, (uint32_t)it & 1u, ctx, 25))) break;
                        tc_fence_after_sync();
                        issue_x(w, nstage); umma_commit<1>(bar_xfull + 8 * w);
                    }
                }
                stage = nstage; phase = nphase;
            }
            if (ok) umma_commit<1>(bar_outfull);
        }
    }
    } else {
        reg_alloc<kBwdRegsMath>();
        // ------------------------------- score math + epilogue -----------------------
        const int wg = (warp - 4) >> 2;                  // which 64 streamed columns
        const int q4 = warp & 3;                         // TMEM lane quarter
        const int row_in_tile = q4 * 32 + lane;
        const int srow = st0 + row_in_tile;              // key (MODE 0) or query (MODE 1) of this thread
        const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
        const uint32_t col0 = (uint32_t)(wg * 64);
        const uint32_t tx1 = tmem_x1 + lane_off + col0, tx2 = tmem_x2 + lane_off + col0;
        const float* lse2_bh = lse2 + (size_t)bh * prm.sq_pad;
        const float* delta_bh = delta + (size_t)bh * prm.sq_pad;
        float my_lse2 = 0.f, my_delta = 0.f;
        if (!kKeyStat) { my_lse2 = lse2_bh[srow]; my_delta = delta_bh[srow]; }     // srow < sq_pad always
        bool ok = true;
        const int wg_tid = (int)threadIdx.x - 128 - wg * 128;      // 0..127 inside the warpgroup
        for (int it = 0; it < n_iter && ok; ++it) {
            const int m0 = (m_begin + it) * kTile + wg * 64;      // first streamed row of this thread's columns
            // MODE 0: the columns are queries, so every thread needs the same 64 (lse2, delta) pairs.
            // The warpgroup stages them in shared memory (one value per thread, fetched before the
            // wait for the scores; two buffers by iteration parity) and reads them back as broadcasts.
            // (The fused pass has one buffer: its refill below follows the wait for dQ^T, which the
            // MMA thread only produces after all four warps have finished their score math.)
            float* stats = stats_gen + ((kFused ? 0 : (it & 1) * 2) + wg) * 128;
            if (kKeyStat) {
                if (!kFused || it == 0)
                    stats[wg_tid] = wg_tid < 64 ? __ldg(lse2_bh + m0 + wg_tid) : __ldg(delta_bh + m0 + wg_tid - 64);
                named_barrier_sync(1 + wg, 128);
            }
            ok = mbar_wait(bar_xfull + 8 * wg, (uint32_t)it & 1u, ctx, 31);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            // Causal: key <= query + offset.  MODE 0: row = key, column = query; MODE 1 the other way.
            // Whole-tile shortcut: no element of these 64 columns is hidden when the smallest query
            // of the pairing still sees the largest key.
            bool masked = false;
            if (prm.causal) {
                if (kKeyStat) masked = st0 + q4 * 32 + 31 > m0 + prm.causal_offset;
                else masked = m0 + 63 > st0 + q4 * 32 + prm.causal_offset;
            }
            // All 64 columns of S and dP at once: four TMEM loads in flight, one wait.
            uint32_t sx[64], dp[64];
            tmem_ld_32x32b_x32(tx1, *reinterpret_cast<uint32_t(*)[32]>(&sx[0]));
            tmem_ld_32x32b_x32(tx1 + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sx[32]));
            tmem_ld_32x32b_x32(tx2, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
            tmem_ld_32x32b_x32(tx2 + 32u, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
            tmem_ld_wait();
            reg_fence(sx); reg_fence(dp);
            uint32_t pp[32], ds[32];
            // Per pair of columns: one FFMA2 (score -> exponent), two exponentials (MUFU, or the
            // FMA-pipe form for some pairs), one FADD2 (dP - delta), one FMUL2, two packs.
#pragma unroll
            for (int c2 = 0; c2 < 32; ++c2) {
                float nl0, nl1, nd0, nd1;
                if (kKeyStat) {
                    const float2 lv = reinterpret_cast<const float2*>(stats)[c2];
                    const float2 dv = reinterpret_cast<const float2*>(stats + 64)[c2];
                    nl0 = -lv.x; nl1 = -lv.y; nd0 = -dv.x; nd1 = -dv.y;
                } else {
                    nl0 = nl1 = -my_lse2; nd0 = nd1 = -my_delta;
                }
                float t0, t1, p0, p1, u0, u1, g0, g1;
                fma2v(t0, t1, __uint_as_float(sx[2 * c2]), __uint_as_float(sx[2 * c2 + 1]), prm.scale_log2, prm.scale_log2, nl0, nl1);
                if ((c2 & 7) < PB200_BWD_FMA_EXP_PAIRS) exp2_fma_pair(p0, p1, t0, t1);
                else { p0 = fast_exp2(t0); p1 = fast_exp2(t1); }
                if (masked) {
                    const int mrow = m0 + 2 * c2;                 // streamed row (query in MODE 0, key in MODE 1)
                    if (kKeyStat ? (srow > mrow + prm.causal_offset) : (mrow > srow + prm.causal_offset)) p0 = 0.f;
                    if (kKeyStat ? (srow > mrow + 1 + prm.causal_offset) : (mrow + 1 > srow + prm.causal_offset)) p1 = 0.f;
                }
                add2v(u0, u1, __uint_as_float(dp[2 * c2]), __uint_as_float(dp[2 * c2 + 1]), nd0, nd1);
                mul2v(g0, g1, p0, p1, u0, u1);
                pp[c2] = pack_bf16(p0, p1);
                ds[c2] = pack_bf16(g0, g1);
            }
            // P over the head of this warpgroup's own S columns, dS over the head of its dP columns.
            if (kKeyStat) tmem_st_32x32b_x32(tx1, pp);
            if (kFused) {
                // dS^T row of this key: 64 queries = 128 bytes = one row of the SWIZZLE_128B image
                const uint32_t rowp = s_ds + (uint32_t)(wg * L::kDsBytes) + (uint32_t)row_in_tile * 128u;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    st_shared_v4(rowp + (((uint32_t)j ^ (uint32_t)(row_in_tile & 7)) << 4), ds[4 * j], ds[4 * j + 1], ds[4 * j + 2], ds[4 * j + 3]);
                fence_proxy_async_smem();
            } else {
                tmem_st_32x32b_x32(tx2, ds);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pready + 8 * wg);
            if (kFused) {
                const bool more = it + 1 < n_iter;
                float next_stat = 0.f;
                if (more) next_stat = wg_tid < 64 ? __ldg(lse2_bh + m0 + kTile + wg_tid) : __ldg(delta_bh + m0 + kTile + wg_tid - 64);
                ok = mbar_wait(bar_dqfull + 8 * wg, (uint32_t)it & 1u, ctx, 33);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                uint32_t dq[64];
                const uint32_t tdq = tmem_dq[wg] + lane_off;
                tmem_ld_32x32b_x32(tdq, *reinterpret_cast<uint32_t(*)[32]>(&dq[0]));
                tmem_ld_32x32b_x32(tdq + 32u, *reinterpret_cast<uint32_t(*)[32]>(&dq[32]));
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_dqfree + 8 * wg);
                stats[wg_tid] = next_stat;
                // lane = head-dim index, column = query: one coalesced 128-byte row segment per column
                if (row_in_tile < HD) {
                    float* dst = dq_acc + ((size_t)bh * prm.sq_pad + m0) * HD + row_in_tile;
#pragma unroll
                    for (int c = 0; c < 64; ++c) atomicAdd(dst + (size_t)c * HD, __uint_as_float(dq[c]));
                }
            }
        }
        // A warp that gave up leaves its share of the warpgroup's barrier behind, so that the others,
        // which may already wait there for the next tile, reach their own next bounded wait and see
        // the abort flag instead of waiting for this warp for ever.
        if (kKeyStat && !ok) named_barrier_arrive(1 + wg, 128);
        // epilogue: accumulators -> global, one row per thread, each warpgroup half of head_dim
        if (ok && n_iter > 0) {
            ok = mbar_wait(bar_outfull, 0, ctx, 41);
            ok = __all_sync(0xffffffffu, ok);
        }
        const int s_rows = kKeyStat ? prm.s_kv : prm.s_q;
        const bool row_exists = srow < s_rows;
        const size_t row_off = ((size_t)bh * s_rows + srow) * prm.hd;
#pragma unroll 1
        for (int which = (kKeyStat ? 0 : 1); which < 2; ++which) {
            OutT* dst = (which == 0 ? out_a : out_b) + row_off;
            const uint32_t acc = (which == 0 ? tmem_acc_a : tmem_acc_b) + lane_off;
            const float mul = which == 0 ? 1.0f : prm.scale;
#pragma unroll 1
            for (int c = wg * (HD / 64); c < (wg + 1) * (HD / 64); ++c) {       // 32-column chunks of this warpgroup
                uint32_t o[32];
                if (ok && n_iter > 0) {
                    tc_fence_after_sync();
                    tmem_ld_32x32b_x32(acc + (uint32_t)(c * 32), o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;                      // a tile that nothing attends to
                }
                if (!ok || !row_exists || c * 32 >= prm.hd) continue;
                const int cols_here = prm.hd - c * 32;
                if (sizeof(OutT) == 4) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (4 * i < cols_here)
                            reinterpret_cast<float4*>(dst + c * 32)[i] =
                                make_float4(__uint_as_float(o[4 * i]) * mul, __uint_as_float(o[4 * i + 1]) * mul,
                                            __uint_as_float(o[4 * i + 2]) * mul, __uint_as_float(o[4 * i + 3]) * mul);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (8 * i < cols_here)
                            reinterpret_cast<uint4*>(dst + c * 32)[i] =
                                make_uint4(pack_bf16(__uint_as_float(o[8 * i]) * mul, __uint_as_float(o[8 * i + 1]) * mul),
                                           pack_bf16(__uint_as_float(o[8 * i + 2]) * mul, __uint_as_float(o[8 * i + 3]) * mul),
                                           pack_bf16(__uint_as_float(o[8 * i + 4]) * mul, __uint_as_float(o[8 * i + 5]) * mul),
                                           pack_bf16(__uint_as_float(o[8 * i + 6]) * mul, __uint_as_float(o[8 * i + 7]) * mul));
                }
            }
        }
    }

    // ------------------------------- teardown ---------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, 512);
    }
}

// ---------------------------------------------------------------------------------------------
// Fused pass at head_dim <= 64, whole-tile form.  A tcgen05.mma of N = 64 or 128 (K = 16) costs the
// issuing thread and the tensor pipe about the same ~65 clocks here, so the half-tile MMAs of the
// template above (48 per tile pair at head_dim 64) are replaced by whole-tile ones where the
// operands allow (S^T, dP^T, dQ^T with N = 128: 32 per tile pair), and TMEM has room for it:
//   S^T/P^T 128 | dP^T 128 | dV 64 | dK 64 | dQ^T 128 columns.
// dQ^T has columns of its own, so nothing waits for it to be read except the next dQ^T; dS^T is
// double-buffered in shared memory (two SWIZZLE_128B images [128 keys][64 queries] per buffer, one
// per warpgroup), so the warpgroups write tile i's while the MMAs still read tile i-1's.
//   MMA order per query tile i: dV(i), S^T(i+1), dP^T(i+1), dK(i), dQ^T(i)
//   warpgroup per tile i: exponentials -> P^T to TMEM; dS^T to shared memory; then, off the MMA
//   thread's critical path, dQ^T(i-1) from TMEM into dq_acc with red.global.add.
// The two warpgroups work in step on the two 64-query halves of the same tile; the tensor pipe is
// kept busy by the order above (the next scores are issued before this tile's dK and dQ^T).
template <int HD>
struct FusedSmem {
    static_assert(HD == 64, "the whole-tile fused pass is the head_dim <= 64 kernel");
    static constexpr int kStages = 3;
    static constexpr int kTileBytes = kTile * HD * 2;
    static constexpr int kDsBytes = kTile * 128;                        // dS^T of one warpgroup: 128 keys x 64 queries, bf16
    static constexpr int kOffStat = 0;                                  // K, V
    static constexpr int kOffRing = 2 * kTileBytes;                     // kStages x (Q, dO)
    static constexpr int kOffDs = kOffRing + kStages * 2 * kTileBytes;
    static constexpr int kStageBytes = 64 * HD * 4;                     // dQ staging of one warpgroup: 64 queries x head_dim fp32
    static constexpr int kOffStage = kOffDs + 2 * 2 * kDsBytes;         // (dS^T: two buffers x two warpgroups)
    static constexpr int kOffBar = kOffStage + 2 * kStageBytes;
    static constexpr int kOffStats = kOffBar + 256;                     // [warpgroup][64 lse2 | 64 delta]
    static constexpr int kTotal = kOffStats + 2 * 128 * 4 + 1024;
    static_assert(kTotal <= 227 * 1024, "shared memory budget exceeded");
};

template <int HD, typename OutT>
__global__ void __launch_bounds__(kBwdThreads, 1)
fmha_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                      const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                      const float* __restrict__ lse2, const float* __restrict__ delta,
                      OutT* __restrict__ out_dv, OutT* __restrict__ out_dk, float* __restrict__ dq_acc,
                      BwdParams prm, int* status) {
    using L = FusedSmem<HD>;
    constexpr int kStages = L::kStages;
    constexpr int kDBlocks = HD / 64;
    constexpr int kHalf = kTile / 2;
    constexpr uint32_t kIdescX = make_idesc_f16(kTile, kTile, true, 0, 0);      // both operands K-major
    constexpr uint32_t kIdescAcc = make_idesc_f16(kTile, HD, true, 0, 1);       // B operand MN-major
    constexpr uint32_t kIdescDq = make_idesc_f16(kTile, kTile, true, 1, 1);     // both operands MN-major
    // Both warpgroups take their exponentials at the same time here, so the MUFU is the limit of that
    // phase: 2 of every 8 score pairs use the FMA-pipe form (+3 %; 3 of 8 is slower again).
    constexpr int kFmaExpPairs = 2;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t s_stat = base + L::kOffStat, s_ring = base + L::kOffRing, s_ds = base + L::kOffDs;
    const uint32_t bars = base + L::kOffBar;
    const uint32_t bar_stat = bars;                       // K, V have landed
    const uint32_t bar_full = bars + 8;                   // [kStages]
    const uint32_t bar_empty = bar_full + 8 * kStages;    // [kStages]
    const uint32_t bar_sfull = bar_empty + 8 * kStages;   // S^T is in TMEM
    const uint32_t bar_dpfull = bar_sfull + 8;            // dP^T is in TMEM
    const uint32_t bar_pready = bar_dpfull + 8;           // P^T and dS^T are written (8 warps)
    const uint32_t bar_dqfull = bar_pready + 8;           // dQ^T is in TMEM
    const uint32_t bar_dqfree = bar_dqfull + 8;           // ... and has been read (8 warps)
    const uint32_t bar_outfull = bar_dqfree + 8;          // dV, dK complete
    const uint32_t s_tmem_slot = bar_outfull + 8;
    const uint32_t s_abort = s_tmem_slot + 8;
    float* stats_gen = reinterpret_cast<float*>(gen + L::kOffStats);
    volatile uint32_t* tmem_slot_gen = (volatile uint32_t*)(gen + (s_tmem_slot - base));
    volatile int* abort_gen = (volatile int*)(gen + (s_abort - base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Causal launches deal the key tiles out heaviest-first (tile 0 meets every query tile) across a
    // group of 16 heads at a time, as the two-pass kernel does.
    constexpr int kHeadGroup = 16;
    int bh = (int)blockIdx.y;
    int st = (int)blockIdx.x;
    if (prm.causal) {
        const int n_st = (int)gridDim.x;
        const int lin = (int)blockIdx.x + n_st * (int)blockIdx.y;
        const int grp = lin / (n_st * kHeadGroup);
        const int rem = lin - grp * (n_st * kHeadGroup);
        const int heads_here = min(kHeadGroup, (int)gridDim.y - grp * kHeadGroup);
        st = rem / heads_here;
        bh = grp * kHeadGroup + rem % heads_here;
    }
    const int st0 = st * kTile;
    const int m_end = (prm.s_q + kTile - 1) / kTile;
    const int m_begin = prm.causal ? min(max(st0 - prm.causal_offset, 0) / kTile, m_end) : 0;   // first query tile that sees key st0
    const int n_iter = m_end - m_begin;

    WaitCtx ctx{status, abort_gen, PB200_K_FLASH_ATTN_BWD};

    if (threadIdx.x == 0) {
        *abort_gen = 0;
        mbar_init(bar_stat, 1);
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_sfull, 1); mbar_init(bar_dpfull, 1); mbar_init(bar_pready, 8);
        mbar_init(bar_dqfull, 1); mbar_init(bar_dqfree, 8); mbar_init(bar_outfull, 1);
        fence_mbarrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do);
    }
    if (warp == 1) {
        tmem_alloc<1>(s_tmem_slot, 512);
        tmem_relinquish<1>();
    }
    pdl_launch_dependents();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    pdl_wait();
    const uint32_t tmem_base = *tmem_slot_gen;
    const uint32_t tmem_x1 = tmem_base, tmem_x2 = tmem_base + 128u;
    const uint32_t tmem_dv = tmem_base + 256u, tmem_dk = tmem_base + 320u, tmem_dq = tmem_base + 384u;

    if (warp < 4) {
    reg_dealloc<kBwdRegsIssue>();
    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0 && n_iter > 0) {
            mbar_arrive_expect_tx(bar_stat, (uint32_t)(2 * L::kTileBytes));
            for (int db = 0; db < kDBlocks; ++db) {
                tma_load_3d(s_stat + db * (kTile * 128), &tmap_k, bar_stat, db * 64, st0, bh);
                tma_load_3d(s_stat + L::kTileBytes + db * (kTile * 128), &tmap_v, bar_stat, db * 64, st0, bh);
            }
            int stage = 0; uint32_t phase = 0;
            for (int it = 0; it < n_iter; ++it) {
                if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, ctx, 11)) break;
                const uint32_t dst = s_ring + stage * 2 * L::kTileBytes;
                mbar_arrive_expect_tx(bar_full + 8 * stage, (uint32_t)(2 * L::kTileBytes));
                for (int db = 0; db < kDBlocks; ++db) {
                    tma_load_3d(dst + db * (kTile * 128), &tmap_q, bar_full + 8 * stage, db * 64, (m_begin + it) * kTile, bh);
                    tma_load_3d(dst + L::kTileBytes + db * (kTile * 128), &tmap_do, bar_full + 8 * stage, db * 64,
                                (m_begin + it) * kTile, bh);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0 && n_iter > 0) {
            bool ok = mbar_wait(bar_stat, 0, ctx, 21);
            const uint64_t sd = make_desc_kmajor_sw128(s_stat);                      // K, V as K-major A
            const uint64_t md = make_desc_kmajor_sw128(s_ring);                      // Q, dO as K-major B
            const uint64_t bd = make_smem_desc(s_ring, kTile * 128, 1024, 2);        // Q, dO as MN-major B
            const uint64_t ktd = make_smem_desc(s_stat, kTile * 128, 1024, 2);       // K as MN-major A (M = head_dim)
            const uint64_t dsk = make_desc_kmajor_sw128(s_ds);                       // dS^T as K-major A
            const uint64_t dsm = make_smem_desc(s_ds, L::kDsBytes, 1024, 2);         // dS^T as MN-major B, N = 128 queries
            const uint32_t s_lo = (uint32_t)sd, s_hi = (uint32_t)(sd >> 32);
            const uint32_t m_lo = (uint32_t)md, m_hi = (uint32_t)(md >> 32);
            const uint32_t b_lo = (uint32_t)bd, b_hi = (uint32_t)(bd >> 32);
            constexpr uint32_t kTileDesc = (uint32_t)(L::kTileBytes >> 4);
            // X = stationary tile t . (streamed tile t)^T, contraction over head_dim: S^T (t = 0) or dP^T (t = 1)
            auto issue_x = [&](int t, int stage) {
                const uint32_t a = s_lo + (uint32_t)t * kTileDesc;
                const uint32_t b = m_lo + (uint32_t)(stage * 2 + t) * kTileDesc;
                const uint32_t d = t == 0 ? tmem_x1 : tmem_x2;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint32_t off = (uint32_t)((k >> 2) * (kTile * 8) + (k & 3) * 2);
                    umma_f16_ss_lohi(d, a + off, s_hi, b + off, m_hi, kIdescX, k != 0 ? 1u : 0u);
                }
            };
            // dV += P^T_w dO_w: P^T of warpgroup w from TMEM (head of its 64 columns), contraction over its 64 queries
            auto issue_dv = [&](int w, int stage, bool first) {
                const uint32_t b = b_lo + (uint32_t)(stage * 2 + 1) * kTileDesc + (uint32_t)(w * ((kHalf * 128) >> 4));
#pragma unroll
                for (int k = 0; k < kHalf / 16; ++k)
                    umma_f16_ts_lohi(tmem_dv, tmem_x1 + (uint32_t)(w * kHalf + k * 8), b + (uint32_t)(k * 128), b_hi,
                                     kIdescAcc, (first && k == 0) ? 0u : 1u);
            };
            // dK += dS^T_w Q_w: dS^T from shared memory (one 128-byte row of 64 queries per key)
            auto issue_dk = [&](int w, int stage, int buf, bool first) {
                const uint32_t a = (uint32_t)dsk + (uint32_t)((buf * 2 + w) * (L::kDsBytes >> 4));
                const uint32_t b = b_lo + (uint32_t)(stage * 2) * kTileDesc + (uint32_t)(w * ((kHalf * 128) >> 4));
#pragma unroll
                for (int k = 0; k < kHalf / 16; ++k)
                    umma_f16_ss_lohi(tmem_dk, a + (uint32_t)(k * 2), (uint32_t)(dsk >> 32), b + (uint32_t)(k * 128), b_hi,
                                     kIdescAcc, (first && k == 0) ? 0u : 1u);
            };
            // dQ^T = K^T dS^T: contraction over the 128 keys, 16 per step (2048 bytes in both operands)
            auto issue_dq = [&](int buf) {
                const uint32_t b = (uint32_t)dsm + (uint32_t)(buf * 2 * (L::kDsBytes >> 4));
#pragma unroll
                for (int k = 0; k < kTile / 16; ++k)
                    umma_f16_ss_lohi(tmem_dq, (uint32_t)ktd + (uint32_t)(k * 128), (uint32_t)(ktd >> 32),
                                     b + (uint32_t)(k * 128), (uint32_t)(dsm >> 32), kIdescDq, k != 0 ? 1u : 0u);
            };
            int stage = 0; uint32_t phase = 0;
            if (ok) ok = mbar_wait(bar_full, 0, ctx, 22);
            if (ok) {
                tc_fence_after_sync();
                issue_x(0, 0); umma_commit<1>(bar_sfull);
                issue_x(1, 0); umma_commit<1>(bar_dpfull);
            }
            for (int it = 0; it < n_iter && ok; ++it) {
                int nstage = stage + 1; uint32_t nphase = phase;
                if (nstage == kStages) { nstage = 0; nphase ^= 1u; }
                const bool more = it + 1 < n_iter;
                const uint32_t par = (uint32_t)it & 1u;
                if (!(ok = mbar_wait(bar_pready, par, ctx, 23))) break;
                tc_fence_after_sync();
                issue_dv(0, stage, it == 0); issue_dv(1, stage, false);
                if (more) {
                    // S^T of the next query tile overwrites P^T, which the dV MMAs above read (issue order);
                    // dP^T of this tile has been read by the warpgroups (they have arrived)
                    if (!(ok = mbar_wait(bar_full + 8 * nstage, nphase, ctx, 24))) break;
                    tc_fence_after_sync();
                    issue_x(0, nstage); umma_commit<1>(bar_sfull);
                    issue_x(1, nstage); umma_commit<1>(bar_dpfull);
                }
                issue_dk(0, stage, (int)par, it == 0); issue_dk(1, stage, (int)par, false);
                umma_commit<1>(bar_empty + 8 * stage);
                if (it > 0) {       // the previous dQ^T must have been read
                    if (!(ok = mbar_wait(bar_dqfree, (uint32_t)(it - 1) & 1u, ctx, 25))) break;
                    tc_fence_after_sync();
                }
                issue_dq((int)par); umma_commit<1>(bar_dqfull);
                stage = nstage; phase = nphase;
            }
            if (ok) umma_commit<1>(bar_outfull);
        }
    }
    } else {
        reg_alloc<kBwdRegsMath>();
        // ------------------------------- score math + epilogue -----------------------
        const int wg = (warp - 4) >> 2;                  // which 64 queries of the streamed tile
        const int q4 = warp & 3;                         // TMEM lane quarter
        const int row_in_tile = q4 * 32 + lane;
        const int srow = st0 + row_in_tile;              // key of this thread
        const uint32_t lane_off = (uint32_t)(q4 * 32) << 16;
        const uint32_t col0 = (uint32_t)(wg * 64);
        const uint32_t tx1 = tmem_x1 + lane_off + col0, tx2 = tmem_x2 + lane_off + col0;
        const float* lse2_bh = lse2 + (size_t)bh * prm.sq_pad;
        const float* delta_bh = delta + (size_t)bh * prm.sq_pad;
        const int wg_tid = (int)threadIdx.x - 128 - wg * 128;      // 0..127 inside the warpgroup
        float* stats = stats_gen + wg * 128;             // 64 lse2 | 64 delta of this warpgroup's queries
        bool ok = true;
        // Thread t < 64 of the warpgroup carries lse2 of query t, thread t >= 64 delta of query t - 64:
        // fetched one tile ahead, stored where no warp can still be reading the previous tile's
        // (lse2 after the barrier that follows the exponentials, delta after the one that opens a tile).
        const float* stat_src = (wg_tid < 64 ? lse2_bh : delta_bh - 64) + wg * 64 + wg_tid;
        float nxt = 0.f;
        if (n_iter > 0) {
            if (wg_tid < 64) stats[wg_tid] = __ldg(stat_src + m_begin * kTile);
            else nxt = __ldg(stat_src + m_begin * kTile);
        }
        // dQ^T of query tile itq: TMEM -> registers -> fp32 rows in the warpgroup's staging buffer -> dq_acc
        // by a bulk reduction of the TMA engine (cp.reduce.async.bulk .add.f32, 16 KB).  lane = head-dim
        // index, column = query: a warp stores 128 contiguous bytes per query (lanes past head_dim hold
        // nothing).  Issuing the 64 red.global.add per thread instead kept both warpgroups' LSU path busy
        // for ~1200 clk per tile in their serial path; the engine has the same throughput but costs the
        // warps only the staging stores.
        const uint32_t tdq = tmem_dq + lane_off + col0;
        const uint32_t s_stage = base + L::kOffStage + (uint32_t)(wg * L::kStageBytes);
        auto move_dq = [&](int itq) -> bool {
            bool good = mbar_wait(bar_dqfull, (uint32_t)itq & 1u, ctx, 33);
            good = __all_sync(0xffffffffu, good);
            if (!good) return false;
            tc_fence_after_sync();
            uint32_t dq[64];
            tmem_ld_32x32b_x32(tdq, *reinterpret_cast<uint32_t(*)[32]>(&dq[0]));
            tmem_ld_32x32b_x32(tdq + 32u, *reinterpret_cast<uint32_t(*)[32]>(&dq[32]));
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_dqfree);
            if (wg_tid == 0) bulk_wait_read0();           // the previous reduction has read the staging buffer
            named_barrier_sync(1 + wg, 128);
            if (row_in_tile < HD) {
#pragma unroll
                for (int c = 0; c < 64; ++c) st_shared_b32(s_stage + (uint32_t)(c * HD + row_in_tile) * 4u, dq[c]);
            }
            fence_proxy_async_smem();
            named_barrier_sync(1 + wg, 128);
            if (wg_tid == 0) {
                bulk_reduce_add_f32(dq_acc + ((size_t)bh * prm.sq_pad + (m_begin + itq) * kTile + wg * 64) * HD, s_stage,
                                    (uint32_t)L::kStageBytes);
                bulk_commit_group();
            }
            return true;
        };
        for (int it = 0; it < n_iter && ok; ++it) {
            const int m0 = (m_begin + it) * kTile + wg * 64;      // first query of this thread's columns
            const uint32_t par = (uint32_t)it & 1u;
            const bool more = it + 1 < n_iter;
            named_barrier_sync(1 + wg, 128);                      // lse2 of this tile is visible; delta of the previous one is no longer read
            if (wg_tid >= 64) stats[wg_tid] = nxt;
            if (more) nxt = __ldg(stat_src + (m_begin + it + 1) * kTile);
            ok = mbar_wait(bar_sfull, par, ctx, 31);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            // Causal: key <= query + offset.  No element of these 64 columns is hidden for this warp
            // when its largest key is still seen by the smallest query.
            const bool masked = prm.causal && (st0 + q4 * 32 + 31 > m0 + prm.causal_offset);
            uint32_t sx[64];
            tmem_ld_32x32b_x32(tx1, *reinterpret_cast<uint32_t(*)[32]>(&sx[0]));
            tmem_ld_32x32b_x32(tx1 + 32u, *reinterpret_cast<uint32_t(*)[32]>(&sx[32]));
            tmem_ld_wait();
            reg_fence(sx);
            // P^T = exp2(S^T scale - lse2[query]): per pair of columns one FFMA2 and two exponentials; kept in fp32
            // (in place) for dS, rounded to bf16 for the dV operand.
            {
                uint32_t pp[32];
#pragma unroll
                for (int c2 = 0; c2 < 32; ++c2) {
                    const float2 lv = reinterpret_cast<const float2*>(stats)[c2];
                    float t0, t1, p0, p1;
                    fma2v(t0, t1, __uint_as_float(sx[2 * c2]), __uint_as_float(sx[2 * c2 + 1]), prm.scale_log2, prm.scale_log2, -lv.x, -lv.y);
                    if ((c2 & 7) < kFmaExpPairs) exp2_fma_pair(p0, p1, t0, t1);
                    else { p0 = fast_exp2(t0); p1 = fast_exp2(t1); }
                    if (masked) {
                        const int mq = m0 + 2 * c2;
                        if (srow > mq + prm.causal_offset) p0 = 0.f;
                        if (srow > mq + 1 + prm.causal_offset) p1 = 0.f;
                    }
                    sx[2 * c2] = __float_as_uint(p0); sx[2 * c2 + 1] = __float_as_uint(p1);
                    pp[c2] = pack_bf16(p0, p1);
                }
                tmem_st_32x32b_x32(tx1, pp);             // over the head of this warp's own S^T columns
            }
            ok = mbar_wait(bar_dpfull, par, ctx, 32);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            uint32_t dp[64];
            tmem_ld_32x32b_x32(tx2, *reinterpret_cast<uint32_t(*)[32]>(&dp[0]));
            tmem_ld_32x32b_x32(tx2 + 32u, *reinterpret_cast<uint32_t(*)[32]>(&dp[32]));
            tmem_ld_wait();
            reg_fence(dp);
            named_barrier_sync(1 + wg, 128);                      // every warp is past its exponentials: lse2 may be replaced
            if (wg_tid < 64 && more) stats[wg_tid] = nxt;
            // dS^T = P^T o (dP^T - delta[query]) -> this key's row of the warpgroup's SWIZZLE_128B image in
            // buffer it & 1 (its previous readers, the dK and dQ^T MMAs of tile it - 2, retired before the
            // dQ^T barrier this warp passed at the end of tile it - 1)
            const uint32_t rowp = s_ds + (uint32_t)((par * 2 + wg) * L::kDsBytes) + (uint32_t)row_in_tile * 128u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t ds[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c2 = 4 * j + i;
                    const float2 dv = reinterpret_cast<const float2*>(stats + 64)[c2];
                    float u0, u1, g0, g1;
                    add2v(u0, u1, __uint_as_float(dp[2 * c2]), __uint_as_float(dp[2 * c2 + 1]), -dv.x, -dv.y);
                    mul2v(g0, g1, __uint_as_float(sx[2 * c2]), __uint_as_float(sx[2 * c2 + 1]), u0, u1);
                    ds[i] = pack_bf16(g0, g1);
                }
                st_shared_v4(rowp + (((uint32_t)j ^ (uint32_t)(row_in_tile & 7)) << 4), ds[0], ds[1], ds[2], ds[3]);
            }
            fence_proxy_async_smem();
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pready);
            // off the MMA thread's critical path: the previous tile's dQ^T
            if (it > 0 && !(ok = move_dq(it - 1))) break;
        }
        if (ok && n_iter > 0) ok = move_dq(n_iter - 1);
        if (wg_tid == 0) bulk_wait_all();                // the reductions must have completed before the CTA exits
        if (!ok) named_barrier_arrive(1 + wg, 128);      // see the template above: nobody may wait for this warp for ever
        // epilogue: dV, dK -> global, one key row per thread, each warpgroup half of head_dim
        if (ok && n_iter > 0) {
            ok = mbar_wait(bar_outfull, 0, ctx, 41);
            ok = __all_sync(0xffffffffu, ok);
        }
        const bool row_exists = srow < prm.s_kv;
        const size_t row_off = ((size_t)bh * prm.s_kv + srow) * prm.hd;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            OutT* dst = (which == 0 ? out_dv : out_dk) + row_off;
            const uint32_t acc = (which == 0 ? tmem_dv : tmem_dk) + lane_off;
            const float mul = which == 0 ? 1.0f : prm.scale;
#pragma unroll 1
            for (int c = wg * (HD / 64); c < (wg + 1) * (HD / 64); ++c) {
                uint32_t o[32];
                if (ok && n_iter > 0) {
                    tc_fence_after_sync();
                    tmem_ld_32x32b_x32(acc + (uint32_t)(c * 32), o);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;                      // a key tile that no query attends to
                }
                if (!ok || !row_exists || c * 32 >= prm.hd) continue;
                store_row_chunk(dst + c * 32, o, prm.hd - c * 32, mul);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, 512);
    }
}


int tile_map(CUtensorMap* m, const void* p, int64_t hd, int64_t rows, int64_t bh, char* err) {
    uint64_t dims[3] = {(uint64_t)hd, (uint64_t)rows, (uint64_t)bh};
    uint64_t str[2] = {(uint64_t)hd * 2, (uint64_t)rows * hd * 2};
    uint32_t box[3] = {64, kTile, 1};
    return make_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
}

template <int HD, int MODE, typename OutT>
int launch_pass(const CUtensorMap& s1, const CUtensorMap& s2, const CUtensorMap& m1, const CUtensorMap& m2,
                const float* lse2, const float* delta, void* out_a, void* out_b, float* dq_acc, const BwdParams& prm,
                int tiles, cudaStream_t stream, char* err) {
    using L = BwdSmem<HD, MODE == 2>;
    auto kernel = fmha_bwd_kernel<HD, MODE, OutT>;
    static std::atomic<uint64_t> attr_set{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!(attr_set.load(std::memory_order_relaxed) & (1ull << (dev & 63)))) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
        if (e != cudaSuccess) { set_err(err, "cudaFuncSetAttribute(smem=%d): %s", L::kTotal, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
        attr_set.fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
    }
    dim3 grid((unsigned)tiles, (unsigned)prm.bh, 1);
    cudaError_t e = launch_with_pdl(kernel, grid, dim3(kBwdThreads), L::kTotal, stream, s1, s2, m1, m2, lse2, delta,
                                    (OutT*)out_a, (OutT*)out_b, dq_acc, prm, device_status_ptr());
    if (e != cudaSuccess) { set_err(err, "attention backward launch failed (HD=%d mode=%d): %s", HD, MODE, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    return PB200_OK;
}

template <int HD, typename OutT>
int launch_fused(const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tq, const CUtensorMap& tdo,
                 const float* lse2, const float* delta, void* dv, void* dk, float* dq_acc, const BwdParams& prm, int tiles,
                 cudaStream_t stream, char* err) {
    using L = FusedSmem<HD>;
    auto kernel = fmha_bwd_fused_kernel<HD, OutT>;
    static std::atomic<uint64_t> attr_set{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!(attr_set.load(std::memory_order_relaxed) & (1ull << (dev & 63)))) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
        if (e != cudaSuccess) { set_err(err, "cudaFuncSetAttribute(smem=%d): %s", L::kTotal, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
        attr_set.fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
    }
    dim3 grid((unsigned)tiles, (unsigned)prm.bh, 1);
    cudaError_t e = launch_with_pdl(kernel, grid, dim3(kBwdThreads), L::kTotal, stream, tk, tv, tq, tdo, lse2, delta,
                                    (OutT*)dv, (OutT*)dk, dq_acc, prm, device_status_ptr());
    if (e != cudaSuccess) { set_err(err, "attention backward launch failed (HD=%d fused): %s", HD, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    return PB200_OK;
}

template <int HD, typename OutT>
int launch_bwd(const Record& r, cudaStream_t stream, void** p, char* err) {
    const int64_t BH = r.dims[0], SQ = r.dims[1], SKV = r.dims[2], hd = r.dims[3];
    BwdParams prm;
    prm.bh = (int)BH; prm.s_q = (int)SQ; prm.s_kv = (int)SKV;
    prm.sq_pad = (int)((SQ + kTile - 1) / kTile * kTile);
    prm.causal = (r.flags & PB200_F_CAUSAL) ? 1 : 0;
    prm.causal_offset = (int)(SKV - SQ);
    prm.scale = (float)r.fparams[0];
    prm.scale_log2 = (float)(r.fparams[0] * 1.4426950408889634);
    prm.hd = (int)hd;
    // buffers: q, k, v, o, lse, do | dq, dk, dv | scratch (delta, then lse2; sq_pad floats per head each)
    CUtensorMap tq, tk, tv, tdo;
    if (int rc = tile_map(&tq, p[0], hd, SQ, BH, err)) return rc;
    if (int rc = tile_map(&tk, p[1], hd, SKV, BH, err)) return rc;
    if (int rc = tile_map(&tv, p[2], hd, SKV, BH, err)) return rc;
    if (int rc = tile_map(&tdo, p[5], hd, SQ, BH, err)) return rc;
    float* delta = (float*)p[9];
    float* lse2 = delta + (size_t)BH * prm.sq_pad;
    float* dq_acc = lse2 + (size_t)BH * prm.sq_pad;          // fused pass only
    const bool fused = !(r.flags & PB200_F_DETERMINISTIC);
    const int rows = (int)(BH * prm.sq_pad);
    if (fused) {
        cudaError_t e = cudaMemsetAsync(dq_acc, 0, (size_t)rows * HD * sizeof(float), stream);
        if (e != cudaSuccess) { set_err(err, "attention backward: clearing the dQ accumulator failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    }
    fmha_bwd_prep_kernel<<<(rows + 7) / 8, 256, 0, stream>>>((const __nv_bfloat16*)p[3], (const __nv_bfloat16*)p[5],
                                                            (const float*)p[4], delta, lse2, (int)BH, (int)SQ, prm.sq_pad, (int)hd);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, "attention backward (row pass) launch failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    const int kv_tiles = (int)((SKV + kTile - 1) / kTile), q_tiles = (int)((SQ + kTile - 1) / kTile);
    if (fused) {
        int rc;
        if constexpr (HD == 64) rc = launch_fused<64, OutT>(tk, tv, tq, tdo, lse2, delta, p[8], p[7], dq_acc, prm, kv_tiles, stream, err);
        else rc = launch_pass<HD, 2, OutT>(tk, tv, tq, tdo, lse2, delta, p[8], p[7], dq_acc, prm, kv_tiles, stream, err);
        if (rc) return rc;
        const size_t quads = (size_t)BH * SQ * (hd / 4);
        const unsigned blocks = (unsigned)std::min<size_t>((quads + 255) / 256, 148 * 16);
        fmha_bwd_dq_finish_kernel<OutT><<<blocks, 256, 0, stream>>>(dq_acc, (OutT*)p[6], (int)BH, (int)SQ, prm.sq_pad, (int)hd, HD, prm.scale);
        e = cudaGetLastError();
        if (e != cudaSuccess) { set_err(err, "attention backward (dQ row pass) launch failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
        return PB200_OK;
    }
    if (int rc = launch_pass<HD, 0, OutT>(tk, tv, tq, tdo, lse2, delta, p[8], p[7], nullptr, prm, kv_tiles, stream, err)) return rc;   // dV, dK
    return launch_pass<HD, 1, OutT>(tq, tdo, tk, tv, lse2, delta, nullptr, p[6], nullptr, prm, q_tiles, stream, err);                 // dQ
}

}  // namespace

// dims = {batch*heads, S_q, S_kv, head_dim}; fparams = {sm_scale} (0 -> 1/sqrt(head_dim))
int plan_attention_bwd(Record& r, char* err) {
    if (r.n_dims != 4) { set_err(err, "attention backward needs dims = {batch*heads, S_q, S_kv, head_dim}, got %d dims", r.n_dims); return PB200_ERR_BAD_SHAPE; }
    const int64_t BH = r.dims[0], SQ = r.dims[1], SKV = r.dims[2], HD = r.dims[3];
    if (BH < 1 || SQ < 1 || SKV < 1) { set_err(err, "batch*heads, S_q, S_kv must be positive"); return PB200_ERR_BAD_SHAPE; }
    if (HD < 8 || HD > 128 || HD % 8 != 0) { set_err(err, "head_dim=%lld must be a multiple of 8 in [8, 128]", (long long)HD); return PB200_ERR_BAD_SHAPE; }
    if (SQ > 0x7fffffffLL / 256 || SKV > 0x7fffffffLL / 256) { set_err(err, "sequence length too large"); return PB200_ERR_BAD_SHAPE; }
    if ((r.flags & PB200_F_CAUSAL) && SKV < SQ) { set_err(err, "causal attention needs S_kv >= S_q"); return PB200_ERR_BAD_SHAPE; }
    if (BH > 65535) { set_err(err, "batch*heads=%lld exceeds 65535", (long long)BH); return PB200_ERR_BAD_SHAPE; }
    if (r.n_fparams < 1 || r.fparams[0] == 0.0) { r.fparams[0] = 1.0 / std::sqrt((double)HD); r.n_fparams = 1; }
    pb200_geometry& g = r.geom;
    const int64_t sq_pad = (SQ + kTile - 1) / kTile * kTile;
    // geometry of the dK/dV pass (the dQ pass has one CTA per query tile)
    g.grid[0] = (uint32_t)((SKV + kTile - 1) / kTile); g.grid[1] = (uint32_t)BH; g.grid[2] = 1;
    g.block[0] = kBwdThreads; g.block[1] = g.block[2] = 1;
    g.cluster[0] = g.cluster[1] = g.cluster[2] = 1;
    const bool fused = !(r.flags & PB200_F_DETERMINISTIC);
    g.smem_bytes = HD <= 64 ? (fused ? FusedSmem<64>::kTotal : BwdSmem<64, false>::kTotal)
                            : (fused ? BwdSmem<128, true>::kTotal : BwdSmem<128, false>::kTotal);
    g.n_inputs = 6; g.n_outputs = 3;
    // delta and lse * log2(e) per padded query; the fused pass adds the fp32 dQ accumulator (rows of the tile's head_dim)
    g.scratch_bytes = (uint64_t)(2 * BH * sq_pad * sizeof(float)) +
                      (fused ? (uint64_t)(BH * sq_pad * (HD <= 64 ? 64 : 128) * sizeof(float)) : 0);
    return PB200_OK;
}

int launch_attention_bwd(const Record& r, cudaStream_t stream, void** p, char* err) {
    const int64_t HD = r.dims[3];
    const bool bf16_out = (r.flags & PB200_F_OUT_BF16) != 0;
    if (HD <= 64) return bf16_out ? launch_bwd<64, __nv_bfloat16>(r, stream, p, err) : launch_bwd<64, float>(r, stream, p, err);
    return bf16_out ? launch_bwd<128, __nv_bfloat16>(r, stream, p, err) : launch_bwd<128, float>(r, stream, p, err);
}

}  // namespace pb200
