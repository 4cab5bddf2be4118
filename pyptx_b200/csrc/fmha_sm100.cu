// Flash-attention forward for sm_100a on tcgen05 tensor cores.
//   O[bh, i, :] = softmax_j(scale * Q[bh, i, :] . K[bh, j, :]  (+ causal mask)) . V[bh, j, :]
// bf16 operands, fp32 scores / statistics / accumulator, P rounded to bf16 before the
// second product -- the arithmetic of the reference's algorithm
// (examples/hopper/experimental/flash_attention_hopper.py:158-256: scores, running max,
// alpha rescale, P -> bf16, acc += P V, final 1/l), re-designed for Blackwell, with the
// batch*head dimension, head_dim 128 and the causal mask the reference lacks.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles that ping-pong:
// while the softmax warps of one tile work, the tensor core runs the other tile's MMAs.
//   warp 0      TMA producer: Q once, then K and V tiles of 128 keys through 2-3 stage rings
//   warp 1      MMA issuer (single thread): S_t = Q_t K^T into TMEM, O_t += P_t V
//   warps 4-7   softmax for tile 0 (one query row per thread, TMEM lane = row)
//   warps 8-11  softmax for tile 1
// TMEM (512 columns): S0 | S1 | O0 | O1, 128 columns each.  P overwrites the first 64
// columns of its S in place (two bf16 per column) and is consumed by the MMA directly
// from TMEM, so P never touches shared memory.  A template switch keeps P in swizzled
// shared memory instead (head_dim 64 only) as a cross-check of the TMEM-operand path.
// V (keys x head_dim, head_dim contiguous) and, when the caller passes the reference's
// transposed K (head_dim x keys), K are consumed as MN-major B operands.
// The accumulator is rescaled lazily: the running reference maximum only moves when the
// true maximum has grown by more than 2^8, which keeps P within bf16/fp32 range and makes
// the TMEM round trip of O rare; the final division by l makes the result independent of it.
// Every mbarrier wait is bounded and reports through the status word.
#include "common.cuh"
#include "fmha_math.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

#include <atomic>
#include <cmath>

namespace pb200 {
namespace {

using namespace ptx;

constexpr int kQTile = 128;       // query rows per tile (TMEM lanes)
constexpr int kKvTile = 128;      // keys per K/V tile
constexpr int kFmhaThreads = 384; // 3 warpgroups: {TMA, MMA, 2 idle}, softmax tile 0, softmax tile 1
constexpr uint32_t kDebugPSmem = 1u << 17;   // create flag: keep P in shared memory (head_dim 64)
constexpr float kRescaleThreshold = 8.0f;    // log2 units
constexpr int kRegsIssue = 88;               // registers per thread of the TMA / MMA warpgroup after setmaxnreg
constexpr int kRegsSoftmax = 208;            // ... of the two softmax warpgroups
#ifndef PB200_FMHA_SPLIT_P
#define PB200_FMHA_SPLIT_P 1
#endif
#ifndef PB200_FMA_EXP_PAIRS
#define PB200_FMA_EXP_PAIRS 1
#endif
#ifndef PB200_FMA_EXP_PAIRS_D64
#define PB200_FMA_EXP_PAIRS_D64 1
#endif
// Of every 8 score pairs, how many take the FMA-pipe exp2 (by tile width: the narrower tile has
// half the MMA time per exponential, so the MUFU unit is further from balance there).
template <int HD> constexpr int kFmaExpPairsOf8 = HD == 64 ? PB200_FMA_EXP_PAIRS_D64 : PB200_FMA_EXP_PAIRS;

struct FmhaParams {
    int bh;            // batch * heads
    int s_q;
    int s_kv;
    int causal;
    int k_transposed;
    float scale_log2;  // sm_scale * log2(e)
    int causal_offset; // s_kv - s_q: query i sees keys j <= i + offset
    int hd;            // head dimension of the tensors in global memory (multiple of 8, <= HD)
};

template <int HD, bool P_SMEM>
struct FmhaSmem {
#ifndef PB200_FMHA_STAGES_D64
#define PB200_FMHA_STAGES_D64 3
#endif
    static constexpr int kStages = HD == 64 ? PB200_FMHA_STAGES_D64 : 2;
    static constexpr int kQBytes = kQTile * HD * 2;          // per tile
    static constexpr int kKvBytes = kKvTile * HD * 2;        // per stage, K or V
    static constexpr int kPBytes = P_SMEM ? kQTile * kKvTile * 2 : 0;   // per tile
    static constexpr int kOffQ = 0;
    static constexpr int kOffK = kOffQ + 2 * kQBytes;
    static constexpr int kOffV = kOffK + kStages * kKvBytes;
    static constexpr int kOffP = kOffV + kStages * kKvBytes;
    static constexpr int kOffBar = kOffP + 2 * kPBytes;
    static constexpr int kTotal = kOffBar + 512 + 1024;
    static_assert(kTotal <= 227 * 1024, "shared memory budget exceeded");
};

// 32 raw scores -> 16 packed bf16 pairs of P = 2^(s * scale - m), row sums into sum4.  Per pair of
// scores: one FFMA2, two exponentials (MUFU, or the FMA-pipe form for FMA_OF8 of every 8 pairs),
// one FADD2, one pack.
template <int FMA_OF8>
__device__ __forceinline__ void exp_chunk(const uint32_t (&v)[32], uint32_t* packed, float (&sum4)[4],
                                          float scale_log2, float neg_m) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float t0, t1;
        fma2(t0, t1, __uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]), scale_log2, neg_m);
        float p0, p1;
        if ((i & 7) < FMA_OF8) exp2_fma_pair(p0, p1, t0, t1);   // compile-time choice per pair
        else { p0 = fast_exp2(t0); p1 = fast_exp2(t1); }
        add2(sum4[2 * (i & 1)], sum4[2 * (i & 1) + 1], p0, p1);
        __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);        // .x = p0 in the low half
        packed[i] = *reinterpret_cast<uint32_t*>(&b);
    }
}

#ifndef PB200_FMHA_SETMAXNREG
#define PB200_FMHA_SETMAXNREG 1
#endif
#ifndef PB200_FMHA_SPEC_MAX
#define PB200_FMHA_SPEC_MAX 1
#endif

// MSPEC: masked tiles (diagonal, ragged) take a speculative path of their own.  It pays wherever masked
// tiles are frequent (causal) and, at head_dim 64, also changes the register allocation of the
// whole softmax loop for the better (no spills: +6 % without any mask); at head_dim 128 its presence
// costs an unmasked launch 1.4 %, so non-causal launches there use the instantiation without it.
template <int HD, typename OutT, bool P_SMEM, bool MSPEC>
__global__ void __launch_bounds__(kFmhaThreads, 1)
fmha_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v,
                OutT* __restrict__ out, float* __restrict__ lse, FmhaParams prm, int* status) {
    using L = FmhaSmem<HD, P_SMEM>;
    constexpr int kStages = L::kStages;
    constexpr int kDBlocks = HD / 64;                  // 64-element (128-byte) blocks along head_dim
    constexpr uint32_t kIdescS = make_idesc_f16(kQTile, kKvTile, true, 0, 0);
    constexpr uint32_t kIdescS_T = make_idesc_f16(kQTile, kKvTile, true, 0, 1);   // K given transposed
    constexpr uint32_t kIdescPV = make_idesc_f16(kQTile, HD, true, 0, 1);         // V is MN-major

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t s_q = base + L::kOffQ, s_k = base + L::kOffK, s_v = base + L::kOffV, s_p = base + L::kOffP;
    const uint32_t bars = base + L::kOffBar;
    const uint32_t bar_q = bars;                        // [1]
    const uint32_t bar_kfull = bars + 8;                // [kStages]
    const uint32_t bar_kempty = bar_kfull + 8 * kStages;
    const uint32_t bar_vfull = bar_kempty + 8 * kStages;
    const uint32_t bar_vempty = bar_vfull + 8 * kStages;
    const uint32_t bar_sfull = bar_vempty + 8 * kStages;   // [2]
    const uint32_t bar_pfull = bar_sfull + 16;             // [2]
    const uint32_t bar_ofull = bar_pfull + 16;             // [2]
    const uint32_t bar_pvdone = bar_ofull + 16;            // [2] (split-P only)
    const uint32_t s_tmem_slot = bar_pvdone + 16;
    const uint32_t s_abort = s_tmem_slot + 8;
    volatile uint32_t* tmem_slot_gen = (volatile uint32_t*)(gen + (s_tmem_slot - base));
    volatile int* abort_gen = (volatile int*)(gen + (s_abort - base));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_qblocks = (int)gridDim.x;
    // Causal: a query block's cost grows with its row index, and CTAs start in linear block order
    // (x fastest).  Blocks are therefore dealt out heaviest first across a GROUP of heads at a
    // time -- within a group all heads' last blocks, then all their second-to-last ones, ... --
    // so that what runs at the end of the grid is light blocks, not one head's heaviest.  Groups
    // of kHeadGroup heads keep the K/V working set of the CTAs in flight inside L2.
#ifndef PB200_FMHA_HEAD_GROUP
#define PB200_FMHA_HEAD_GROUP 16
#endif
    constexpr int kHeadGroup = PB200_FMHA_HEAD_GROUP;
    int qblock = n_qblocks - 1 - (int)blockIdx.x;
    int bh = (int)blockIdx.y;
    if (prm.causal) {
        const int lin = (int)blockIdx.x + n_qblocks * (int)blockIdx.y;
        const int grp = lin / (n_qblocks * kHeadGroup);
        const int rem = lin - grp * (n_qblocks * kHeadGroup);
        const int heads_here = min(kHeadGroup, (int)gridDim.y - grp * kHeadGroup);
        qblock = n_qblocks - 1 - rem / heads_here;
        bh = grp * kHeadGroup + rem % heads_here;
    }
    const int q0 = qblock * 2 * kQTile;
    const bool has_t1 = q0 + kQTile < prm.s_q;
    // Number of K/V tiles each query tile visits.
    int n_kv[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        int n = (prm.s_kv + kKvTile - 1) / kKvTile;     // the last tile may be partial: TMA fills it with zeros
        if (prm.causal) {
            const int last_key = q0 + t * kQTile + kQTile - 1 + prm.causal_offset;   // of the tile's last row
            n = min(n, max(last_key / kKvTile + 1, 1));
        }
        n_kv[t] = n;
    }
    if (!has_t1) n_kv[1] = 0;
    const int n_iter = max(n_kv[0], n_kv[1]);

    WaitCtx ctx{status, abort_gen, PB200_K_FLASH_ATTN};

    if (threadIdx.x == 0) {
        *abort_gen = 0;
        mbar_init(bar_q, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_kfull + 8 * s, 1); mbar_init(bar_kempty + 8 * s, 1);
            mbar_init(bar_vfull + 8 * s, 1); mbar_init(bar_vempty + 8 * s, 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(bar_sfull + 8 * t, 1);
            mbar_init(bar_pfull + 8 * t, 4);     // one arrival per softmax warp
            mbar_init(bar_ofull + 8 * t, 1);
            mbar_init(bar_pvdone + 8 * t, 1);
        }
        fence_mbarrier_init();
        fence_proxy_async_smem();
        prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
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
    const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128u};
    const uint32_t tmem_o[2] = {tmem_base + 256u, tmem_base + 384u};
    // Head dimension 64 leaves 64 free columns behind each O: P gets columns of its own there, so
    // that the next S of a tile no longer has to wait for the P V product that reads P (with P
    // aliased over S it must), and S(j+1) is issued ahead of P(j) V(j).
    constexpr bool kSplitP = PB200_FMHA_SPLIT_P && HD == 64 && !P_SMEM;
    const uint32_t tmem_p[2] = {kSplitP ? tmem_o[0] + 64u : tmem_s[0], kSplitP ? tmem_o[1] + 64u : tmem_s[1]};

    // Registers move from the TMA / MMA warpgroup (two single-thread roles) to the softmax
    // warpgroups; each setmaxnreg sits at the head of its own branch so that the compiler sees which
    // budget governs which code.  A CTA can only hand around the registers it was launched with
    // (168 per thread here): an increase beyond what the decrease released would block for ever.
    static_assert(kRegsIssue * 128 + kRegsSoftmax * 256 <= 168 * kFmhaThreads, "setmaxnreg budget exceeds the launch allocation");
    if (warp < 4) {
#if PB200_FMHA_SETMAXNREG
    reg_dealloc<kRegsIssue>();
#endif
    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            const int n_tiles = has_t1 ? 2 : 1;
            mbar_arrive_expect_tx(bar_q, (uint32_t)(n_tiles * L::kQBytes));
            for (int t = 0; t < n_tiles; ++t)
                for (int db = 0; db < kDBlocks; ++db)
                    tma_load_3d(s_q + t * L::kQBytes + db * (kQTile * 128), &tmap_q, bar_q, db * 64, q0 + t * kQTile, bh);
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int j = 0; j < n_iter && ok; ++j) {
                if (!(ok = mbar_wait(bar_kempty + 8 * stage, phase ^ 1u, ctx, 11))) break;
                mbar_arrive_expect_tx(bar_kfull + 8 * stage, (uint32_t)L::kKvBytes);
                if (!prm.k_transposed) {
                    for (int db = 0; db < kDBlocks; ++db)
                        tma_load_3d(s_k + stage * L::kKvBytes + db * (kKvTile * 128), &tmap_k, bar_kfull + 8 * stage,
                                    db * 64, j * kKvTile, bh);
                } else {
                    // K_t[bh][HD][s_kv]: two boxes of 64 keys x HD rows
                    for (int nb = 0; nb < kKvTile / 64; ++nb)
                        tma_load_3d(s_k + stage * L::kKvBytes + nb * (HD * 128), &tmap_k, bar_kfull + 8 * stage,
                                    j * kKvTile + nb * 64, 0, bh);
                }
                if (!(ok = mbar_wait(bar_vempty + 8 * stage, phase ^ 1u, ctx, 12))) break;
                mbar_arrive_expect_tx(bar_vfull + 8 * stage, (uint32_t)L::kKvBytes);
                for (int db = 0; db < kDBlocks; ++db)
                    tma_load_3d(s_v + stage * L::kKvBytes + db * (kKvTile * 128), &tmap_v, bar_vfull + 8 * stage,
                                db * 64, j * kKvTile, bh);
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------
        if (lane == 0) {
            bool ok = mbar_wait(bar_q, 0, ctx, 21);
            // The issuing thread is the serial resource of this kernel: it shares its scheduler with
            // two busy softmax warps, and a 128x128x16 MMA retires every 64 clocks.  Descriptors are
            // therefore built once; their high word is constant and every per-MMA change stays inside
            // the 14-bit start-address field of the low word, so an MMA costs one 32-bit add per operand.
            // One thread issues for both tiles on purpose: the fixed order PV0 S0 PV1 S1 keeps the two
            // tiles half a period apart, so one tile's softmax always overlaps the other tile's MMAs.
            const bool kt = prm.k_transposed != 0;
            const uint32_t idesc_s = kt ? kIdescS_T : kIdescS;
            const uint64_t qd0 = make_desc_kmajor_sw128(s_q), qd1 = make_desc_kmajor_sw128(s_q + L::kQBytes);
            const uint64_t kd0 = kt ? make_smem_desc(s_k, HD * 128, 1024, 2) : make_desc_kmajor_sw128(s_k);
            const uint64_t vd0 = make_smem_desc(s_v, kKvTile * 128, 1024, 2);
            const uint64_t pd0 = make_desc_kmajor_sw128(s_p), pd1 = make_desc_kmajor_sw128(s_p + L::kPBytes);
            const uint32_t q_lo[2] = {(uint32_t)qd0, (uint32_t)qd1}, q_hi = (uint32_t)(qd0 >> 32);
            const uint32_t p_lo[2] = {(uint32_t)pd0, (uint32_t)pd1}, p_hi = (uint32_t)(pd0 >> 32);
            const uint32_t k_lo0 = (uint32_t)kd0, k_hi = (uint32_t)(kd0 >> 32);
            const uint32_t v_lo0 = (uint32_t)vd0, v_hi = (uint32_t)(vd0 >> 32);
            uint32_t k_step[HD / 16];     // K-major: 32 bytes per step inside a 64-wide block; transposed: 16 rows
#pragma unroll
            for (int k = 0; k < HD / 16; ++k)
                k_step[k] = kt ? (uint32_t)(k * 128) : (uint32_t)((k >> 2) * (kKvTile * 8) + (k & 3) * 2);
            // S_t(j) = Q_t . K(j)^T : HD/16 MMAs of K = 16.
            auto issue_s = [&](int t, int kstage) {
                const uint32_t kl = k_lo0 + (uint32_t)(kstage * (L::kKvBytes >> 4));
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    umma_f16_ss_lohi(tmem_s[t], q_lo[t] + (uint32_t)((k >> 2) * (kQTile * 8) + (k & 3) * 2), q_hi,
                                     kl + k_step[k], k_hi, idesc_s, k != 0 ? 1u : 0u);
            };
            // O_t += P_t . V(j) : 128/16 MMAs of K = 16.
            auto issue_pv = [&](int t, int vstage, bool first) {
                const uint32_t vl = v_lo0 + (uint32_t)(vstage * (L::kKvBytes >> 4));
#pragma unroll
                for (int k = 0; k < kKvTile / 16; ++k) {
                    const uint32_t acc = (first && k == 0) ? 0u : 1u;
                    if (P_SMEM)
                        umma_f16_ss_lohi(tmem_o[t], p_lo[t] + (uint32_t)((k >> 2) * (kQTile * 8) + (k & 3) * 2), p_hi,
                                         vl + (uint32_t)(k * 128), v_hi, kIdescPV, acc);
                    else
                        umma_f16_ts_lohi(tmem_o[t], tmem_p[t] + (uint32_t)(k * 8), vl + (uint32_t)(k * 128), v_hi, kIdescPV, acc);
                }
            };
            int kstage = 0; uint32_t kphase = 0;     // ring position of K(j+1) being consumed by S
            int vstage = 0; uint32_t vphase = 0;     // ring position of V(j)
            if (ok && n_iter > 0) {
                ok = mbar_wait(bar_kfull + 8 * kstage, kphase, ctx, 22);
                if (ok) {
                    tc_fence_after_sync();
                    issue_s(0, kstage); umma_commit<1>(bar_sfull + 0);
                    if (n_kv[1] > 0) { issue_s(1, kstage); umma_commit<1>(bar_sfull + 8); }
                    umma_commit<1>(bar_kempty + 8 * kstage);
                    if (++kstage == kStages) { kstage = 0; kphase ^= 1u; }
                }
            }
            for (int j = 0; j < n_iter && ok; ++j) {
                const uint32_t jpar = (uint32_t)j & 1u;
                const bool more = j + 1 < n_iter;
                if (!(ok = mbar_wait(bar_vfull + 8 * vstage, vphase, ctx, 23))) break;
                if (more && !(ok = mbar_wait(bar_kfull + 8 * kstage, kphase, ctx, 24))) break;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j < n_kv[t]) {
                        if (!(ok = mbar_wait(bar_pfull + 8 * t, jpar, ctx, 25 + t))) break;
                        tc_fence_after_sync();
                        if (kSplitP) {
                            if (j + 1 < n_kv[t]) { issue_s(t, kstage); umma_commit<1>(bar_sfull + 8 * t); }
                            issue_pv(t, vstage, j == 0);
                            if (j + 1 < n_kv[t]) umma_commit<1>(bar_pvdone + 8 * t);
                            else umma_commit<1>(bar_ofull + 8 * t);
                        } else {
                            issue_pv(t, vstage, j == 0);
                            if (j + 1 < n_kv[t]) { issue_s(t, kstage); umma_commit<1>(bar_sfull + 8 * t); }
                            else umma_commit<1>(bar_ofull + 8 * t);
                        }
                    }
                }
                if (!ok) break;
                umma_commit<1>(bar_vempty + 8 * vstage);
                if (++vstage == kStages) { vstage = 0; vphase ^= 1u; }
                if (more) {
                    umma_commit<1>(bar_kempty + 8 * kstage);
                    if (++kstage == kStages) { kstage = 0; kphase ^= 1u; }
                }
            }
        }
    }
    } else {
#if PB200_FMHA_SETMAXNREG
        reg_alloc<kRegsSoftmax>();
#endif
        // ------------------------------- softmax + epilogue --------------------------
        const int t = (warp - 4) >> 2;                   // query tile of this warp group
        const int q = warp & 3;                          // TMEM lane quarter
        const int row_in_tile = q * 32 + lane;
        const int row = q0 + t * kQTile + row_in_tile;   // query index inside this (batch, head)
        const uint32_t lane_off = (uint32_t)(q * 32) << 16;
        const uint32_t ts = tmem_s[t] + lane_off;
        const uint32_t to = tmem_o[t] + lane_off;
        const uint32_t tp = tmem_p[t] + lane_off;
        const int n = n_kv[t];
        float m_used = -INFINITY;     // reference maximum currently baked into O and l (log2 units)
        float l = 0.f;
        bool ok = true;
        for (int j = 0; j < n && ok; ++j) {
            ok = mbar_wait(bar_sfull + 8 * t, (uint32_t)j & 1u, ctx, 31 + t);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const int key0 = j * kKvTile;
            // Largest key index this row may see: the causal bound and the end of the sequence.
            const int last_visible = prm.causal ? min(row + prm.causal_offset, prm.s_kv - 1) : prm.s_kv - 1;
            // Tiles that cross the diagonal (for any row of this warp) or the end of K/V take the masked path.
            const bool diag = (prm.causal && (key0 + kKvTile - 1 > q0 + t * kQTile + q * 32 + prm.causal_offset)) ||
                              (key0 + kKvTile > prm.s_kv);
            // Fast path (every unmasked tile; masked ones have a variant of their own further down, and a
            // masked FIRST tile takes the exact path): the exponentials are taken against the reference
            // maximum already in use (first tile: an estimate), without a maximum pass and so without its
            // serial dependency.  P stays in registers until the row sums say it is valid:
            // every P <= 2^8 is implied by a tile sum <= 2^8, which is the lazy-rescale invariant.  A
            // larger sum (the running maximum moved, or many scores sit just below 2^8) sends the
            // whole warp to the exact path below, which reads S again (nothing was stored yet).
            // On a masked tile every 32-key chunk is, for the 32 rows of this warp, wholly visible,
            // wholly hidden, or mixed: only mixed chunks pay for per-element masking, hidden ones
            // are not evaluated at all (on an aligned diagonal tile: q visible, 1 mixed, 3 - q hidden).
            const int row_lo = q0 + t * kQTile + q * 32;
            const int vis_lo = prm.causal ? min(row_lo + prm.causal_offset, prm.s_kv - 1) : prm.s_kv - 1;        // first row of the warp
            const int vis_hi = prm.causal ? min(row_lo + 31 + prm.causal_offset, prm.s_kv - 1) : prm.s_kv - 1;   // last row
            auto chunk_class = [&](int c) {          // 0 visible, 1 mixed, 2 hidden
                const int kc = key0 + c * 32;
                return !diag || kc + 31 <= vis_lo ? 0 : kc > vis_hi ? 2 : 1;
            };
            bool slow = diag || !PB200_FMHA_SPEC_MAX;
            bool forced = false;
            uint32_t packed[kKvTile / 2];
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
            if (!slow) {
                uint32_t v0[32], v1[32];
                tmem_ld_32x32b_x32(ts, v0);
                tmem_ld_32x32b_x32(ts + 32u, v1);
                tmem_ld_wait();
                reg_fence(v0); reg_fence(v1);
                if (j == 0) {
                    // First tile: O and l are empty, so any reference maximum is valid as long as no P
                    // exceeds 2^8, which the sum check below verifies.  The maximum of the row's first 64
                    // scores stands in for the row maximum (the exact path follows if it was too low).
                    float e0 = -INFINITY, e1 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        e0 = fmax3(e0, __uint_as_float(v0[i]), __uint_as_float(v0[i + 1]));
                        e1 = fmax3(e1, __uint_as_float(v1[i]), __uint_as_float(v1[i + 1]));
                    }
                    m_used = fmaxf(e0, e1) * prm.scale_log2;
                }
                const float neg_m = -m_used;
                exp_chunk<kFmaExpPairsOf8<HD>>(v0, &packed[0], sum4, prm.scale_log2, neg_m);
                tmem_ld_32x32b_x32(ts + 64u, v0);
                exp_chunk<kFmaExpPairsOf8<HD>>(v1, &packed[16], sum4, prm.scale_log2, neg_m);
                tmem_ld_32x32b_x32(ts + 96u, v1);
                tmem_ld_wait();
                reg_fence(v0); reg_fence(v1);
                exp_chunk<kFmaExpPairsOf8<HD>>(v0, &packed[32], sum4, prm.scale_log2, neg_m);
                exp_chunk<kFmaExpPairsOf8<HD>>(v1, &packed[48], sum4, prm.scale_log2, neg_m);
                const float tile_sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                slow = __any_sync(0xffffffffu, !(tile_sum <= 256.0f));
                forced = slow;
            } else if (MSPEC && PB200_FMHA_SPEC_MAX && diag && j > 0) {
                // A masked tile with a reference maximum in hand: the same speculation, chunk by chunk
                // (a block of its own, so that the unmasked path above keeps its schedule).
                const float neg_m = -m_used;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int cls = chunk_class(c);
                    if (cls == 2) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) packed[16 * c + i] = 0u;
                        continue;
                    }
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(ts + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
                    reg_fence(v);
                    if (cls == 0) {
                        exp_chunk<kFmaExpPairsOf8<HD>>(v, &packed[16 * c], sum4, prm.scale_log2, neg_m);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * i]), prm.scale_log2, neg_m));
                            float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), prm.scale_log2, neg_m));
                            if (key0 + c * 32 + 2 * i > last_visible) p0 = 0.f;
                            if (key0 + c * 32 + 2 * i + 1 > last_visible) p1 = 0.f;
                            sum4[i & 3] += p0 + p1;
                            __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                            packed[16 * c + i] = *reinterpret_cast<uint32_t*>(&b);
                        }
                    }
                }
                const float tile_sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
                slow = __any_sync(0xffffffffu, !(tile_sum <= 256.0f));
                forced = slow;
            }
            if (kSplitP && j > 0) {
                // P(j-1) V(j-1) must have retired before O is rescaled or P is overwritten
                ok = mbar_wait(bar_pvdone + 8 * t, (uint32_t)(j - 1) & 1u, ctx, 35 + t);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
            }
            if (!slow) {
                if (P_SMEM) {
                    const uint32_t rowp = s_p + t * L::kPBytes + (uint32_t)row_in_tile * 128u;
#pragma unroll
                    for (int c8 = 0; c8 < 16; ++c8)      // 16-byte chunks of 8 keys: 8 per 64-key block
                        st_shared_v4(rowp + (uint32_t)(c8 >> 3) * (kQTile * 128) + (((uint32_t)(c8 & 7) ^ (uint32_t)(row_in_tile & 7)) << 4),
                                     packed[4 * c8], packed[4 * c8 + 1], packed[4 * c8 + 2], packed[4 * c8 + 3]);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        tmem_st_32x32b_x16(tp + (uint32_t)(c * 16), *reinterpret_cast<uint32_t(*)[16]>(&packed[c * 16]));
                }
            } else {
                sum4[0] = sum4[1] = sum4[2] = sum4[3] = 0.f;
                // The whole score row (128 fp32) comes out of TMEM once: four loads in flight, one wait.
                uint32_t sc[kKvTile];
#pragma unroll
                for (int c = 0; c < kKvTile / 32; ++c)
                    tmem_ld_32x32b_x32(ts + (uint32_t)(c * 32), *reinterpret_cast<uint32_t(*)[32]>(&sc[c * 32]));
                tmem_ld_wait();
                reg_fence(sc);
                // row maximum of the raw scores: four independent chains of 3-input max
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int c = 0; c < kKvTile / 32; ++c) {
                    const int cls = chunk_class(c);
                    if (cls == 0) {
#pragma unroll
                        for (int i = c * 32; i < c * 32 + 32; i += 8) {
                            mx4[0] = fmax3(mx4[0], __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
                            mx4[1] = fmax3(mx4[1], __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
                            mx4[2] = fmax3(mx4[2], __uint_as_float(sc[i + 4]), __uint_as_float(sc[i + 5]));
                            mx4[3] = fmax3(mx4[3], __uint_as_float(sc[i + 6]), __uint_as_float(sc[i + 7]));
                        }
                    } else if (cls == 1) {
#pragma unroll
                        for (int i = c * 32; i < c * 32 + 32; ++i)
                            if (key0 + i <= last_visible) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sc[i]));
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                const float m_new = fmaxf(m_used, mx * prm.scale_log2);
                if (j == 0) {
                    m_used = m_new;
                } else if (__any_sync(0xffffffffu, m_new - m_used > (forced ? 0.0f : kRescaleThreshold))) {
                    const float alpha = fast_exp2(m_used - m_new);     // 1 for lanes whose maximum did not move
                    m_used = m_new;
                    l *= alpha;
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        uint32_t o[32];
                        tmem_ld_32x32b_x32(to + (uint32_t)(c * 32), o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32b_x32(to + (uint32_t)(c * 32), o);
                    }
                    tmem_st_wait();
                }
                // P = exp2(S * scale - m_used): the scores are read again in two halves of 64 (two loads in
                // flight per wait), exponentiated, summed and written back as bf16 P to TMEM (or shared memory).
                const float neg_m = -m_used;
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    uint32_t v[64];
                    tmem_ld_32x32b_x32(ts + (uint32_t)(h * 64), *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
                    tmem_ld_32x32b_x32(ts + (uint32_t)(h * 64 + 32), *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
                    tmem_ld_wait();
                    reg_fence(v);
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int c = h * 2 + cc;          // 32-key chunk index
                        uint32_t pk[16];
                        const int cls = chunk_class(c);
                        if (cls == 0) {
                            // no mask: per pair of scores one FFMA2, two EX2, one FADD2, one pack
                            exp_chunk<kFmaExpPairsOf8<HD>>(*reinterpret_cast<uint32_t(*)[32]>(&v[cc * 32]), pk, sum4, prm.scale_log2, neg_m);
                        } else if (cls == 1) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                float p0 = fast_exp2(fmaf(__uint_as_float(v[cc * 32 + 2 * i]), prm.scale_log2, neg_m));
                                float p1 = fast_exp2(fmaf(__uint_as_float(v[cc * 32 + 2 * i + 1]), prm.scale_log2, neg_m));
                                if (key0 + c * 32 + 2 * i > last_visible) p0 = 0.f;
                                if (key0 + c * 32 + 2 * i + 1 > last_visible) p1 = 0.f;
                                sum4[i & 3] += p0 + p1;
                                __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
                                pk[i] = *reinterpret_cast<uint32_t*>(&b);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i) pk[i] = 0u;      // P = 0 for keys no row of this warp sees
                        }
                        if (P_SMEM) {
                            // K-major SWIZZLE_128B image: 64-key blocks of [128 rows][128 bytes]
                            const uint32_t rowp = s_p + t * L::kPBytes + (uint32_t)h * (kQTile * 128) + (uint32_t)row_in_tile * 128u;
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                const uint32_t chunk = (uint32_t)(cc * 4 + jj);
                                st_shared_v4(rowp + ((chunk ^ (uint32_t)(row_in_tile & 7)) << 4),
                                             pk[4 * jj], pk[4 * jj + 1], pk[4 * jj + 2], pk[4 * jj + 3]);
                            }
                        } else {
                            tmem_st_32x32b_x16(tp + (uint32_t)(c * 16), pk);
                        }
                    }
                }
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l += sum;
            if (P_SMEM) fence_proxy_async_smem(); else tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pfull + 8 * t);
        }
        // epilogue: O / l -> global, one row per thread
        if (ok && n > 0) {
            ok = mbar_wait(bar_ofull + 8 * t, 0, ctx, 41 + t);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && n > 0) {
            tc_fence_after_sync();
            const float inv = 1.0f / l;
            // The tensors' head dimension may be smaller than the tile's (see launch_fmha): rows are
            // prm.hd apart and only the first prm.hd columns exist.
            OutT* dst = out + ((size_t)bh * prm.s_q + row) * prm.hd;
            const bool row_exists = row < prm.s_q;          // a partial last query tile computes padding rows
            // log-sum-exp of the scaled scores (natural log), for callers that run a backward pass:
            // m_used is in log2 units and l = sum 2^(x - m_used).
            if (lse != nullptr && row_exists)
                lse[(size_t)bh * prm.s_q + row] = (m_used + log2f(l)) * 0.6931471805599453f;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
                uint32_t o[32];
                tmem_ld_32x32b_x32(to + (uint32_t)(c * 32), o);
                tmem_ld_wait();
                if (!row_exists || c * 32 >= prm.hd) continue;
                const int cols_here = prm.hd - c * 32;        // multiple of 8; >= 32 for a full chunk
                if (sizeof(OutT) == 4) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (4 * i < cols_here)
                            reinterpret_cast<float4*>(dst + c * 32)[i] =
                                make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                            __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
                } else {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv);
                        pk[i] = *reinterpret_cast<uint32_t*>(&b);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (8 * i < cols_here)
                            reinterpret_cast<uint4*>(dst + c * 32)[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
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

template <int HD, typename OutT, bool P_SMEM, bool MSPEC>
int launch_fmha(const Record& r, cudaStream_t stream, void** p, char* err) {
    using L = FmhaSmem<HD, P_SMEM>;
    auto kernel = fmha_fwd_kernel<HD, OutT, P_SMEM, MSPEC>;
    static std::atomic<uint64_t> attr_set{0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!(attr_set.load(std::memory_order_relaxed) & (1ull << (dev & 63)))) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
        if (e != cudaSuccess) { set_err(err, "cudaFuncSetAttribute(smem=%d): %s", L::kTotal, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
        attr_set.fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
    }
    const int64_t BH = r.dims[0], SQ = r.dims[1], SKV = r.dims[2];
    // Head dimension of the tensors.  The kernel's tiles are HD (64 or 128) wide; a smaller head
    // dimension keeps the 64-element boxes, and TMA fills the columns (rows, for K given
    // transposed) past the tensor's extent with zeros: zero columns of Q and K add nothing to
    // Q K^T, zero columns of V give zero columns of O, which the epilogue does not store.
    const int64_t hd = r.dims[3];
    const bool kt = (r.flags & PB200_F_K_TRANSPOSED) != 0;
    CUtensorMap tq, tk, tv;
    {
        uint64_t dims[3] = {(uint64_t)hd, (uint64_t)SQ, (uint64_t)BH};
        uint64_t str[2] = {(uint64_t)hd * 2, (uint64_t)SQ * hd * 2};
        uint32_t box[3] = {64, kQTile, 1};
        int rc = make_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p[0], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    }
    if (!kt) {
        uint64_t dims[3] = {(uint64_t)hd, (uint64_t)SKV, (uint64_t)BH};
        uint64_t str[2] = {(uint64_t)hd * 2, (uint64_t)SKV * hd * 2};
        uint32_t box[3] = {64, kKvTile, 1};
        int rc = make_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p[1], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    } else {
        uint64_t dims[3] = {(uint64_t)SKV, (uint64_t)hd, (uint64_t)BH};
        uint64_t str[2] = {(uint64_t)SKV * 2, (uint64_t)SKV * hd * 2};
        uint32_t box[3] = {64, (uint32_t)HD, 1};
        int rc = make_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p[1], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    }
    {
        uint64_t dims[3] = {(uint64_t)hd, (uint64_t)SKV, (uint64_t)BH};
        uint64_t str[2] = {(uint64_t)hd * 2, (uint64_t)SKV * hd * 2};
        uint32_t box[3] = {64, kKvTile, 1};
        int rc = make_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, p[2], dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B, err);
        if (rc) return rc;
    }
    FmhaParams prm;
    prm.bh = (int)BH; prm.s_q = (int)SQ; prm.s_kv = (int)SKV;
    prm.causal = (r.flags & PB200_F_CAUSAL) ? 1 : 0;
    prm.k_transposed = kt ? 1 : 0;
    prm.scale_log2 = (float)(r.fparams[0] * 1.4426950408889634);
    prm.causal_offset = (int)(SKV - SQ);
    prm.hd = (int)hd;
    dim3 grid(r.geom.grid[0], r.geom.grid[1], 1);
    float* lse = (r.flags & PB200_F_RETURN_LSE) ? (float*)p[4] : nullptr;
    cudaError_t e = launch_with_pdl(kernel, grid, dim3(kFmhaThreads), L::kTotal, stream, tq, tk, tv, (OutT*)p[3], lse, prm,
                                    device_status_ptr());
    if (e != cudaSuccess) { set_err(err, "attention launch failed (HD=%d smem=%d): %s", HD, L::kTotal, cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    return PB200_OK;
}

}  // namespace

// dims = {batch*heads, S_q, S_kv, head_dim}; fparams = {sm_scale} (0 -> 1/sqrt(head_dim))
int plan_attention(Record& r, char* err) {
    if (r.n_dims != 4) { set_err(err, "attention needs dims = {batch*heads, S_q, S_kv, head_dim}, got %d dims", r.n_dims); return PB200_ERR_BAD_SHAPE; }
    const int64_t BH = r.dims[0], SQ = r.dims[1], SKV = r.dims[2], HD = r.dims[3];
    if (BH < 1 || SQ < 1 || SKV < 1) { set_err(err, "batch*heads, S_q, S_kv must be positive"); return PB200_ERR_BAD_SHAPE; }
    if (HD < 8 || HD > 128 || HD % 8 != 0) { set_err(err, "head_dim=%lld must be a multiple of 8 in [8, 128]", (long long)HD); return PB200_ERR_BAD_SHAPE; }
    const int tile_hd = HD <= 64 ? 64 : 128;
    if ((r.flags & PB200_F_K_TRANSPOSED) && SKV % 8 != 0) {
        set_err(err, "S_kv=%lld must be divisible by 8 when K is given transposed (16-byte row pitch)", (long long)SKV);
        return PB200_ERR_BAD_SHAPE;
    }
    if (SQ > 0x7fffffffLL / 256 || SKV > 0x7fffffffLL / 256) { set_err(err, "sequence length too large"); return PB200_ERR_BAD_SHAPE; }
    if ((r.flags & PB200_F_CAUSAL) && SKV < SQ) { set_err(err, "causal attention needs S_kv >= S_q"); return PB200_ERR_BAD_SHAPE; }
    if (BH > 65535) { set_err(err, "batch*heads=%lld exceeds 65535", (long long)BH); return PB200_ERR_BAD_SHAPE; }
    if ((r.flags & kDebugPSmem) && tile_hd != 64) { set_err(err, "the shared-memory P variant exists for head_dim 64 only"); return PB200_ERR_BAD_SHAPE; }
    if (r.n_fparams < 1 || r.fparams[0] == 0.0) { r.fparams[0] = 1.0 / std::sqrt((double)HD); r.n_fparams = 1; }
    pb200_geometry& g = r.geom;
    g.grid[0] = (uint32_t)((SQ + 2 * kQTile - 1) / (2 * kQTile)); g.grid[1] = (uint32_t)BH; g.grid[2] = 1;
    g.block[0] = kFmhaThreads; g.block[1] = g.block[2] = 1;
    g.cluster[0] = g.cluster[1] = g.cluster[2] = 1;
    g.smem_bytes = tile_hd == 64 ? ((r.flags & kDebugPSmem) ? FmhaSmem<64, true>::kTotal : FmhaSmem<64, false>::kTotal)
                            : FmhaSmem<128, false>::kTotal;
    g.n_inputs = 3; g.n_outputs = (r.flags & PB200_F_RETURN_LSE) ? 2 : 1;
    return PB200_OK;
}

int launch_attention(const Record& r, cudaStream_t stream, void** p, char* err) {
    const int64_t HD = r.dims[3];
    const bool bf16_out = (r.flags & PB200_F_OUT_BF16) != 0;
    const bool p_smem = (r.flags & kDebugPSmem) != 0;
    if (HD <= 64) {
        if (p_smem) return bf16_out ? launch_fmha<64, __nv_bfloat16, true, true>(r, stream, p, err) : launch_fmha<64, float, true, true>(r, stream, p, err);
        return bf16_out ? launch_fmha<64, __nv_bfloat16, false, true>(r, stream, p, err) : launch_fmha<64, float, false, true>(r, stream, p, err);
    }
    if (r.flags & PB200_F_CAUSAL)
        return bf16_out ? launch_fmha<128, __nv_bfloat16, false, true>(r, stream, p, err) : launch_fmha<128, float, false, true>(r, stream, p, err);
    return bf16_out ? launch_fmha<128, __nv_bfloat16, false, false>(r, stream, p, err) : launch_fmha<128, float, false, false>(r, stream, p, err);
}

}  // namespace pb200
