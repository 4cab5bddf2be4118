// Backward kernels of the row-wise f32 ops for sm_100a: RMSNorm, LayerNorm, SwiGLU.
//
// The reference ships no backward kernels; its autograd hook
// (pyptx/torch_support.py:446-519, differentiable_kernel) pairs a forward kernel with a
// user-supplied backward one.  These are the backward halves for that hook, HBM-bound like
// the forward kernels and built on the same skeleton (row in registers, 128-bit coalesced
// accesses, warp-shuffle + one shared-memory exchange per reduction).
//
// RMSNorm   y = x * r * w,  r = rsqrt(mean(x^2) + eps)
//   dx = r * (w*dy - xhat * mean(xhat * w*dy)),  xhat = x * r;   dw = sum_rows dy * xhat
// LayerNorm y = xhat * w + b,  xhat = (x - mu) * r
//   dx = r * (w*dy - mean(w*dy) - xhat * mean(xhat * w*dy));   dw = sum_rows dy * xhat;  db = sum_rows dy
// SwiGLU    out = g * s * u,  s = sigmoid(g)
//   dg = dout * u * s * (1 + g * (1 - s));   du = dout * g * s
//
// The column sums dw / db go through SCRATCH memory: a persistent grid of P CTAs walks the
// rows, every thread keeps the partial sums of its own columns in registers, each CTA writes
// one partial row to scratch[P][N] (two planes for LayerNorm), and a second small kernel
// folds the P rows.  This is deterministic (no atomics) and costs P*N*4 bytes of traffic
// against 3*B*N*4 for the main pass.  The scratch buffer is supplied by the caller as one
// extra trailing pointer (its size is part of the handle's geometry).
#include "common.cuh"
#include "ptx.cuh"

#include <atomic>

namespace pb200 {
namespace {

constexpr int kWarp = 32;

__device__ __forceinline__ float4 ld_stream4(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream4(float4* p, const float4& v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Two block-wide sums with one barrier (see block_reduce in row_kernels.cu for the slot rule).
template <int THREADS>
__device__ __forceinline__ void block_sum2(float& a, float& b, float2* slot) {
    constexpr int NW = THREADS / kWarp;
    a = warp_sum(a);
    b = warp_sum(b);
    if (NW == 1) return;
    if ((threadIdx.x & (kWarp - 1)) == 0) slot[threadIdx.x / kWarp] = make_float2(a, b);
    __syncthreads();
    float2 r = slot[0];
#pragma unroll
    for (int i = 1; i < NW; ++i) { r.x += slot[i].x; r.y += slot[i].y; }
    a = r.x;
    b = r.y;
}

// The same for a CTA of many warps: every warp reads the per-warp partials once (lane i takes warp
// i's) and folds them with shuffles, instead of every thread reading all of them.  All warps run
// the same tree, so every thread ends with the same bits.
template <int THREADS>
__device__ __forceinline__ void block_sum2_tree(float& a, float& b, float2* slot) {
    constexpr int NW = THREADS / kWarp;
    const int lane = threadIdx.x & (kWarp - 1);
    a = warp_sum(a);
    b = warp_sum(b);
    if (lane == 0) slot[threadIdx.x / kWarp] = make_float2(a, b);
    __syncthreads();
    const float2 v = lane < NW ? slot[lane] : make_float2(0.f, 0.f);
    a = warp_sum(v.x);
    b = warp_sum(v.y);
}

// MODE 0 = RMSNorm, 1 = LayerNorm.  partial_w / partial_b: [gridDim.x][4*n4] f32.
// A CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; each thread owns VPT float4 columns.
// Its running column sums (dw, db) live in shared memory, not registers: that keeps the kernel
// at 64 registers, so two 512-thread CTAs share an SM and one loads while the other reduces.
constexpr int bwd_min_ctas(int threads) { return threads >= 1024 ? 1 : 1024 / threads; }
template <int THREADS, int VPT, int MODE>
__global__ void __launch_bounds__(THREADS, bwd_min_ctas(THREADS))
norm_bwd_kernel(const float4* __restrict__ x, const float4* __restrict__ w, const float4* __restrict__ dy,
                float4* __restrict__ dx, float4* __restrict__ partial_w, float4* __restrict__ partial_b,
                int rows, int n4, float inv_n, float eps) {
    __shared__ float2 red[3][kWarp];
    extern __shared__ float4 acc_smem[];              // [MODE + 1][THREADS * VPT]
    float4* acc_w = acc_smem;
    float4* acc_b = acc_smem + THREADS * VPT;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        acc_w[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (MODE == 1) acc_b[idx] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    int flip = 0;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        // w (64 KiB at most) is re-read where it is used: L1 serves it after the first row, and
        // holding it would cost the registers that let two CTAs share an SM.
        const float4* xr = x + (size_t)row * n4;
        const float4* gr = dy + (size_t)row * n4;
        float4* dr = dx + (size_t)row * n4;
        float4 xv[VPT], gv[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            const bool in = idx < n4;
            xv[i] = in ? ld_stream4(xr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            gv[i] = in ? ld_stream4(gr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // first moments: sum x (LayerNorm only) and sum w*dy
        float s_x = 0.f, s_wdy = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (MODE == 1) {
                const int idx = threadIdx.x + i * THREADS;
                const float4 wq = idx < n4 ? __ldg(w + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
                s_x += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w);
                s_wdy += wq.x * gv[i].x + wq.y * gv[i].y + wq.z * gv[i].z + wq.w * gv[i].w;
            }
        }
        if (MODE == 1) {        // RMSNorm needs neither the mean of x nor the mean of w*dy
            block_sum2<THREADS>(s_x, s_wdy, red[flip]);
            flip = flip == 2 ? 0 : flip + 1;
        }
        const float mu = MODE == 1 ? s_x * inv_n : 0.f;
        // second moments: sum (x-mu)^2 and sum (x-mu) * w*dy
        float s_xx = 0.f, s_xwdy = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                const float4 wq = __ldg(w + idx);
                const float cx = xv[i].x - mu, cy = xv[i].y - mu, cz = xv[i].z - mu, cw = xv[i].w - mu;
                s_xx += cx * cx + cy * cy + cz * cz + cw * cw;
                s_xwdy += cx * wq.x * gv[i].x + cy * wq.y * gv[i].y + cz * wq.z * gv[i].z + cw * wq.w * gv[i].w;
            }
        }
        block_sum2<THREADS>(s_xx, s_xwdy, red[flip]);
        flip = flip == 2 ? 0 : flip + 1;
        const float r = rsqrtf(s_xx * inv_n + eps);
        const float c1 = s_xwdy * r * inv_n;                    // mean(xhat * w*dy)
        const float c2 = MODE == 1 ? s_wdy * inv_n : 0.f;       // mean(w*dy)
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                const float hx = (xv[i].x - mu) * r, hy = (xv[i].y - mu) * r, hz = (xv[i].z - mu) * r, hw = (xv[i].w - mu) * r;
                const float4 wq = __ldg(w + idx);
                float4 o;
                o.x = r * (wq.x * gv[i].x - c2 - hx * c1);
                o.y = r * (wq.y * gv[i].y - c2 - hy * c1);
                o.z = r * (wq.z * gv[i].z - c2 - hz * c1);
                o.w = r * (wq.w * gv[i].w - c2 - hw * c1);
                st_stream4(dr + idx, o);
                float4 aw = acc_w[idx];
                aw.x += gv[i].x * hx; aw.y += gv[i].y * hy; aw.z += gv[i].z * hz; aw.w += gv[i].w * hw;
                acc_w[idx] = aw;
                if (MODE == 1) {
                    float4 ab = acc_b[idx];
                    ab.x += gv[i].x; ab.y += gv[i].y; ab.z += gv[i].z; ab.w += gv[i].w;
                    acc_b[idx] = ab;
                }
            }
        }
    }
    // this CTA's partial column sums -> scratch
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (idx < n4) {
            partial_w[(size_t)blockIdx.x * n4 + idx] = acc_w[idx];
            if (MODE == 1) partial_b[(size_t)blockIdx.x * n4 + idx] = acc_b[idx];
        }
    }
}

// The same pass for rows of 4097 .. 8192 columns (the benchmark's 8192 among them), shaped for
// streaming: ONE 1024-thread CTA per SM, VPT <= 2 float4 columns per thread, so that within 64
// registers a thread holds its slice of w for the whole kernel (instead of three cached re-reads
// per row) and, next to the row it works on, the NEXT row's x and dy, whose loads are issued before
// the reductions of the current row.  HBM then always has a row in flight per SM while the
// barrier-separated phases of the current one run.  (Measured alternatives that were not faster:
// w in shared memory to make room for both column sums in registers, and LayerNorm's four row sums
// in one shifted pass with a single barrier.)
#ifndef PB200_RMS_ACC_REGS
#define PB200_RMS_ACC_REGS 0      // RMSNorm's single column sum in registers measured 3 % slower than in shared memory
#endif
#ifndef PB200_LN_BOTH_REGS
#define PB200_LN_BOTH_REGS 0       // both LayerNorm sums in registers spill (64-register limit at 1024 threads): 45 % slower
#endif
// does the streaming kernel keep dw's column sum in shared memory?
constexpr bool stream_acc_in_smem(int mode) { return mode == 0 ? !PB200_RMS_ACC_REGS : !PB200_LN_BOTH_REGS; }
template <int VPT, int MODE>
__global__ void __launch_bounds__(1024, 1)
norm_bwd_stream_kernel(const float4* __restrict__ x, const float4* __restrict__ w, const float4* __restrict__ dy,
                       float4* __restrict__ dx, float4* __restrict__ partial_w, float4* __restrict__ partial_b,
                       int rows, int n4, float inv_n, float eps) {
    constexpr int THREADS = 1024;
    constexpr bool kAccWInRegs = MODE == 0 ? PB200_RMS_ACC_REGS : PB200_LN_BOTH_REGS;
    constexpr bool kBoth = MODE == 1 && PB200_LN_BOTH_REGS;
    __shared__ float2 red[3][kWarp];
    extern __shared__ float4 acc_smem[];              // LayerNorm: [THREADS * VPT] column sums of dy * xhat
    float4* acc_w = acc_smem;
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    ptx::pdl_launch_dependents();
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (!kAccWInRegs) acc_w[idx] = zero4;
    }
    ptx::pdl_wait();
    float4 wv[VPT], xv[VPT], gv[VPT];
    // LayerNorm keeps db's column sum in registers and dw's in shared memory: both in registers do not
    // fit in 64, and each sum kept in shared memory costs 64 KiB of read-modify-write per row in the
    // unit (L1 / shared memory) that also moves the rows: with both there the kernel ran at 0.76 of
    // the copy bandwidth, with one 0.83.
    float4 ab[VPT], aw2[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) { ab[i] = zero4; aw2[i] = zero4; }
    int row = blockIdx.x;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        const bool in = idx < n4;
        wv[i] = in ? __ldg(w + idx) : zero4;
        xv[i] = in && row < rows ? ld_stream4(x + (size_t)row * n4 + idx) : zero4;
        gv[i] = in && row < rows ? ld_stream4(dy + (size_t)row * n4 + idx) : zero4;
    }
    int flip = 0;
    for (; row < rows; row += gridDim.x) {
        // next row first: its loads fly while this row is reduced, scaled and stored
        const int nrow = row + (int)gridDim.x;
        float4 xn[VPT], gn[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            const bool in = idx < n4 && nrow < rows;
            xn[i] = in ? ld_stream4(x + (size_t)nrow * n4 + idx) : zero4;
            gn[i] = in ? ld_stream4(dy + (size_t)nrow * n4 + idx) : zero4;
        }
        float mu = 0.f, c2 = 0.f;
        if (MODE == 1) {        // RMSNorm needs neither the mean of x nor the mean of w*dy
            float s_x = 0.f, s_wdy = 0.f;
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                s_x += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w);
                s_wdy += wv[i].x * gv[i].x + wv[i].y * gv[i].y + wv[i].z * gv[i].z + wv[i].w * gv[i].w;
            }
            block_sum2_tree<THREADS>(s_x, s_wdy, red[flip]);
            flip = flip == 2 ? 0 : flip + 1;
            mu = s_x * inv_n;
            c2 = s_wdy * inv_n;                               // mean(w*dy)
        }
        float s_xx = 0.f, s_xwdy = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            if (threadIdx.x + i * THREADS < n4) {             // padding columns must not see -mu
                const float cx = xv[i].x - mu, cy = xv[i].y - mu, cz = xv[i].z - mu, cw = xv[i].w - mu;
                s_xx += cx * cx + cy * cy + cz * cz + cw * cw;
                s_xwdy += cx * wv[i].x * gv[i].x + cy * wv[i].y * gv[i].y + cz * wv[i].z * gv[i].z + cw * wv[i].w * gv[i].w;
            }
        }
        block_sum2_tree<THREADS>(s_xx, s_xwdy, red[flip]);
        flip = flip == 2 ? 0 : flip + 1;
        const float r = rsqrtf(s_xx * inv_n + eps);
        const float c1 = s_xwdy * r * inv_n;                    // mean(xhat * w*dy)
        float4* dr = dx + (size_t)row * n4;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                const float hx = (xv[i].x - mu) * r, hy = (xv[i].y - mu) * r, hz = (xv[i].z - mu) * r, hw = (xv[i].w - mu) * r;
                float4 o;
                o.x = r * (wv[i].x * gv[i].x - c2 - hx * c1);
                o.y = r * (wv[i].y * gv[i].y - c2 - hy * c1);
                o.z = r * (wv[i].z * gv[i].z - c2 - hz * c1);
                o.w = r * (wv[i].w * gv[i].w - c2 - hw * c1);
                st_stream4(dr + idx, o);
                if (kBoth) {
                    aw2[i].x += gv[i].x * hx; aw2[i].y += gv[i].y * hy; aw2[i].z += gv[i].z * hz; aw2[i].w += gv[i].w * hw;
                } else if (kAccWInRegs) {
                    ab[i].x += gv[i].x * hx; ab[i].y += gv[i].y * hy; ab[i].z += gv[i].z * hz; ab[i].w += gv[i].w * hw;
                } else {
                    float4 aw = acc_w[idx];
                    aw.x += gv[i].x * hx; aw.y += gv[i].y * hy; aw.z += gv[i].z * hz; aw.w += gv[i].w * hw;
                    acc_w[idx] = aw;
                }
                if (MODE == 1) { ab[i].x += gv[i].x; ab[i].y += gv[i].y; ab[i].z += gv[i].z; ab[i].w += gv[i].w; }
            }
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) { xv[i] = xn[i]; gv[i] = gn[i]; }
    }
    // this CTA's partial column sums -> scratch
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * THREADS;
        if (idx < n4) {
            partial_w[(size_t)blockIdx.x * n4 + idx] = kBoth ? aw2[i] : kAccWInRegs ? ab[i] : acc_w[idx];
            if (MODE == 1) partial_b[(size_t)blockIdx.x * n4 + idx] = ab[i];
        }
    }
}

// out[c] = sum_p partial[p][c]; blockIdx.y selects the plane (dw, then db).  A CTA folds 32
// float4 columns with 32 part-lanes: lane j adds parts j, j+32, ... in order, then one warp adds
// the 32 lane sums in order, so the result depends on `parts` alone, not on timing.  (A column per
// thread with one serial loop over all parts took as long as the backward pass itself.)
__global__ void __launch_bounds__(1024)
fold_partials_kernel(const float4* __restrict__ partial, float4* __restrict__ out_w, float4* __restrict__ out_b,
                     int parts, int n4) {
    __shared__ float4 lane_sum[32][32];
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();                 // the partial rows come from the kernel launched just before
    const int c = threadIdx.x & 31, j = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + c;
    const float4* src = partial + (size_t)blockIdx.y * parts * n4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < n4) {
        for (int p = j; p < parts; p += 32) {
            const float4 v = src[(size_t)p * n4 + col];
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
    }
    lane_sum[j][c] = a;
    __syncthreads();
    if (j == 0 && col < n4) {
        float4 t = lane_sum[0][c];
#pragma unroll
        for (int k = 1; k < 32; ++k) {
            const float4 v = lane_sum[k][c];
            t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w;
        }
        (blockIdx.y == 0 ? out_w : out_b)[col] = t;
    }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const float4* __restrict__ gate, const float4* __restrict__ up, const float4* __restrict__ dout,
                  float4* __restrict__ dgate, float4* __restrict__ dup, size_t total4) {
    constexpr int UNROLL = 2;
    const size_t tile = (size_t)256 * UNROLL;
    for (size_t base = (size_t)blockIdx.x * tile; base < total4; base += (size_t)gridDim.x * tile) {
        float4 g[UNROLL], u[UNROLL], d[UNROLL];
#pragma unroll
        for (int i = 0; i < UNROLL; ++i) {
            const size_t idx = base + threadIdx.x + (size_t)i * 256;
            if (idx < total4) { g[i] = ld_stream4(gate + idx); u[i] = ld_stream4(up + idx); d[i] = ld_stream4(dout + idx); }
        }
#pragma unroll
        for (int i = 0; i < UNROLL; ++i) {
            const size_t idx = base + threadIdx.x + (size_t)i * 256;
            if (idx < total4) {
                float4 og, ou;
                auto one = [](float gg, float uu, float dd, float& dg, float& du) {
                    const float s = 1.0f / (1.0f + expf(-gg));
                    du = dd * gg * s;
                    dg = dd * uu * s * (1.0f + gg * (1.0f - s));
                };
                one(g[i].x, u[i].x, d[i].x, og.x, ou.x);
                one(g[i].y, u[i].y, d[i].y, og.y, ou.y);
                one(g[i].z, u[i].z, d[i].z, og.z, ou.z);
                one(g[i].w, u[i].w, d[i].w, og.w, ou.w);
                st_stream4(dgate + idx, og);
                st_stream4(dup + idx, ou);
            }
        }
    }
}

struct BwdConfig { int threads; int vpt; };
// Smallest register-resident configuration that covers a row; rows beyond 16384 columns are not supported.
// 1024-thread configurations run norm_bwd_stream_kernel (one CTA per SM, next row prefetched).
bool pick_bwd_config(int64_t n4, BwdConfig& c) {
    const BwdConfig table[] = {{32, 1}, {32, 2}, {64, 2}, {128, 2}, {128, 4}, {256, 4}, {1024, 2}, {512, 8}};
    for (const BwdConfig& t : table)
        if ((int64_t)t.threads * t.vpt >= n4) { c = t; return true; }
    return false;
}
size_t bwd_acc_bytes(const BwdConfig& c, int mode) {
    if (c.threads == 1024) return stream_acc_in_smem(mode) ? (size_t)c.threads * c.vpt * sizeof(float4) : 0;   // streaming kernel
    return (size_t)(mode + 1) * c.threads * c.vpt * sizeof(float4);
}

// CTAs of the persistent grid: two per SM where two fit (threads and the shared-memory column
// sums), else one, so that no CTA waits for a slot.
int bwd_parts(int64_t rows, int64_t n4, int mode) {
    BwdConfig c{256, 4};
    pick_bwd_config(n4, c);
    const bool two = c.threads < 1024 && 2 * c.threads <= 2048 && 2 * bwd_acc_bytes(c, mode) <= 200 * 1024;
    const int64_t p = (two ? 2 : 1) * (int64_t)sm_count();
    return (int)(rows < p ? rows : p);
}

template <int THREADS, int VPT>
void launch_norm(int mode, int parts, cudaStream_t s, const float4* x, const float4* w, const float4* dy, float4* dx,
                 float4* pw, float4* pb, int rows, int n4, float inv_n, float eps) {
    const size_t smem = (size_t)(mode + 1) * THREADS * VPT * sizeof(float4);
    if (smem > 48 * 1024) {
        // opt in once per kernel and device (a host-side attribute, no allocation)
        static std::atomic<uint64_t> done[2];
        int dev = 0;
        cudaGetDevice(&dev);
        if (!(done[mode].load(std::memory_order_relaxed) & (1ull << (dev & 63)))) {
            if (mode == 0) cudaFuncSetAttribute(norm_bwd_kernel<THREADS, VPT, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            else cudaFuncSetAttribute(norm_bwd_kernel<THREADS, VPT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            done[mode].fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
        }
    }
    if (mode == 0) norm_bwd_kernel<THREADS, VPT, 0><<<parts, THREADS, smem, s>>>(x, w, dy, dx, pw, pb, rows, n4, inv_n, eps);
    else norm_bwd_kernel<THREADS, VPT, 1><<<parts, THREADS, smem, s>>>(x, w, dy, dx, pw, pb, rows, n4, inv_n, eps);
}

template <int VPT>
void launch_norm_stream(int mode, int parts, cudaStream_t s, const float4* x, const float4* w, const float4* dy, float4* dx,
                        float4* pw, float4* pb, int rows, int n4, float inv_n, float eps) {
    const size_t smem = stream_acc_in_smem(mode) ? (size_t)1024 * VPT * sizeof(float4) : 0;
    if (smem > 48 * 1024) {
        static std::atomic<uint64_t> done[2];
        int dev = 0;
        cudaGetDevice(&dev);
        if (!(done[mode].load(std::memory_order_relaxed) & (1ull << (dev & 63)))) {
            if (mode == 0) cudaFuncSetAttribute(norm_bwd_stream_kernel<VPT, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            else cudaFuncSetAttribute(norm_bwd_stream_kernel<VPT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            done[mode].fetch_or(1ull << (dev & 63), std::memory_order_relaxed);
        }
    }
    if (mode == 0) launch_with_pdl(norm_bwd_stream_kernel<VPT, 0>, dim3(parts), dim3(1024), smem, s, x, w, dy, dx, pw, pb, rows, n4, inv_n, eps);
    else launch_with_pdl(norm_bwd_stream_kernel<VPT, 1>, dim3(parts), dim3(1024), smem, s, x, w, dy, dx, pw, pb, rows, n4, inv_n, eps);
}

}  // namespace

// Shared by the generic entry (scratch from the caller) and the allocation-free entry (static scratch).
int enqueue_norm_bwd(int mode, int rows, int n, float eps, int parts, cudaStream_t s, const void* x, const void* w,
                     const void* dy, void* dx, void* dw, void* db, void* scratch, char* err) {
    const int n4 = n / 4;
    BwdConfig c;
    if (!pick_bwd_config(n4, c)) { set_err(err, "backward norm kernels support at most 16384 columns, got %d", n); return PB200_ERR_BAD_SHAPE; }
    float4* pw = (float4*)scratch;
    float4* pb = pw + (size_t)parts * n4;
    const float inv_n = 1.0f / (float)n;
#define PB200_BWD_CASE(T, V) \
    if (c.threads == T && c.vpt == V) launch_norm<T, V>(mode, parts, s, (const float4*)x, (const float4*)w, (const float4*)dy, \
                                                        (float4*)dx, pw, pb, rows, n4, inv_n, eps); else
    PB200_BWD_CASE(32, 1) PB200_BWD_CASE(32, 2) PB200_BWD_CASE(64, 2) PB200_BWD_CASE(128, 2)
    PB200_BWD_CASE(128, 4) PB200_BWD_CASE(256, 4) PB200_BWD_CASE(512, 8)
    if (c.threads == 1024) launch_norm_stream<2>(mode, parts, s, (const float4*)x, (const float4*)w, (const float4*)dy,
                                                 (float4*)dx, pw, pb, rows, n4, inv_n, eps);
#undef PB200_BWD_CASE
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess)
        e = launch_with_pdl(fold_partials_kernel, dim3((n4 + 31) / 32, mode == 1 ? 2 : 1), dim3(1024), 0, s,
                            (const float4*)pw, (float4*)dw, (float4*)db, parts, n4);
    if (e != cudaSuccess) { set_err(err, "backward norm launch failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    return PB200_OK;
}

size_t norm_bwd_scratch_bytes(int mode, int parts, int n) { return (size_t)(mode == 1 ? 2 : 1) * parts * n * sizeof(float); }

int plan_row_bwd(Record& r, char* err) {
    if (r.n_dims != 2) { set_err(err, "backward row kernel needs dims = {rows, cols}, got %d dims", r.n_dims); return PB200_ERR_BAD_SHAPE; }
    const int64_t rows = r.dims[0], n = r.dims[1];
    if (rows <= 0 || n <= 0 || rows > 0x7fffffffLL) { set_err(err, "rows=%lld cols=%lld out of range", (long long)rows, (long long)n); return PB200_ERR_BAD_SHAPE; }
    if (n % 4 != 0) { set_err(err, "cols=%lld must be divisible by 4 (128-bit vector access)", (long long)n); return PB200_ERR_BAD_SHAPE; }
    pb200_geometry& g = r.geom;
    g.grid[1] = g.grid[2] = 1; g.block[1] = g.block[2] = 1;
    g.cluster[0] = g.cluster[1] = g.cluster[2] = 1;
    g.smem_bytes = 0;
    g.scratch_bytes = 0;
    g.n_inputs = 3;
    if (r.kernel_id == PB200_K_SWIGLU_BWD) {
        const int64_t total4 = rows * n / 4;
        int64_t ctas = (total4 + 511) / 512;
        if (ctas > 0x7fffffffLL) ctas = 0x7fffffffLL;
        g.grid[0] = (uint32_t)ctas; g.block[0] = 256; g.n_outputs = 2;
        return PB200_OK;
    }
    BwdConfig c;
    if (!pick_bwd_config(n / 4, c)) { set_err(err, "backward norm kernels support at most 16384 columns, got %lld", (long long)n); return PB200_ERR_BAD_SHAPE; }
    const int mode = r.kernel_id == PB200_K_LAYER_NORM_BWD ? 1 : 0;
    const int parts = bwd_parts(rows, n / 4, mode);
    r.dims[7] = parts;            // fixed at create time: the scratch size depends on it
    g.grid[0] = (uint32_t)parts; g.block[0] = (uint32_t)c.threads;
    g.smem_bytes = (uint32_t)(3 * kWarp * sizeof(float2) + bwd_acc_bytes(c, mode));
    g.n_outputs = mode == 1 ? 3 : 2;
    g.scratch_bytes = norm_bwd_scratch_bytes(mode, parts, (int)n);
    return PB200_OK;
}

// buffers: x, w, dy | dx, dw [, db] | scratch          (SwiGLU: gate, up, dout | dgate, dup)
int launch_row_bwd(const Record& r, cudaStream_t s, void** p, char* err) {
    const int rows = (int)r.dims[0], n = (int)r.dims[1];
    if (r.kernel_id == PB200_K_SWIGLU_BWD) {
        swiglu_bwd_kernel<<<r.geom.grid[0], 256, 0, s>>>((const float4*)p[0], (const float4*)p[1], (const float4*)p[2],
                                                         (float4*)p[3], (float4*)p[4], (size_t)rows * (n / 4));
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { set_err(err, "swiglu backward launch failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
        return PB200_OK;
    }
    const int mode = r.kernel_id == PB200_K_LAYER_NORM_BWD ? 1 : 0;
    void* db = mode == 1 ? p[5] : nullptr;
    void* scratch = mode == 1 ? p[6] : p[5];
    return enqueue_norm_bwd(mode, rows, n, (float)r.fparams[0], (int)r.dims[7], s, p[0], p[1], p[2], p[3], p[4], db, scratch, err);
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward for hosts that hand a kernel library no memory to work in.
//
// Some callers may not allocate device memory where they call us: an inference server whose
// memory plan is fixed when the model is loaded, a plugin slot of a larger engine that gives
// the plugin its tensors and nothing else, a process that lives inside a fixed share of a
// GPU.  For them cudaMalloc on the request path is either forbidden outright or would stall
// the device and break the owner's accounting, and they have no allocator of their own to
// lend us.  The regular backward entry needs a scratch buffer from the caller; this one
// brings its own, a fixed array that is part of the loaded library image.
//
// Limits and rules that follow from a shared, fixed array:
//   * kStaticScratchBytes (4 MiB) per GPU stay reserved from the moment the library is
//     loaded on that GPU until the process exits, whether or not this entry is ever called;
//   * the partial-sum rows must fit: the grid is capped at kStaticScratchBytes / (4 * cols)
//     CTAs (128 at 8192 columns, 64 at 16384), so very wide rows run with fewer CTAs than
//     the regular entry would use, and cols above kStaticMaxCols are rejected;
//   * every call on a GPU uses the same array.  Nothing in it has to start at zero (each call
//     overwrites every word it later reads), so no clearing is done, but two calls that can
//     run at the same time on one GPU (different streams, or different host threads) would
//     overwrite each other's partial sums: callers must order them, e.g. on one stream;
//   * the first call on each GPU looks up the array's device address (cudaGetSymbolAddress,
//     which may initialise the CUDA context); make that first call during start-up, outside
//     any stream capture.  Later calls only enqueue two kernels.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 4u << 20;
constexpr int kStaticMaxCols = 16384;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

namespace {
constexpr int kMaxDev = 64;
std::atomic<float*> g_static_scratch_ptr[kMaxDev];

// Device address of g_static_scratch on the current device.  The array's name is only a
// host-side handle here; the kernels need the address the runtime reports for it.
int static_scratch_address(float** out, char* err) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDev) {
        set_err(err, "no usable current CUDA device (%s)", e == cudaSuccess ? "index out of range" : cudaGetErrorString(e));
        return PB200_ERR_NO_CUDA;
    }
    float* p = g_static_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        void* addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess || !addr) {
            set_err(err, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
            return PB200_ERR_NO_CUDA;
        }
        p = (float*)addr;
        g_static_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return PB200_OK;
}
}  // namespace

}  // namespace pb200

extern "C" PB200_API int pb200_rms_norm_bwd_static(int64_t rows, int64_t cols, double eps, uint64_t stream,
                                                    const void* x, const void* w, const void* dy,
                                                    void* dx, void* dw, char* err_out) {
    using namespace pb200;
    if (err_out) err_out[0] = 0;
    if (rows <= 0 || rows > 0x7fffffffLL || cols <= 0 || cols % 4 != 0) {
        set_err(err_out, "rows=%lld must be positive and cols=%lld a positive multiple of 4", (long long)rows, (long long)cols);
        return PB200_ERR_BAD_SHAPE;
    }
    if (cols > kStaticMaxCols) {
        set_err(err_out, "cols=%lld exceeds the %d columns the built-in %zu-byte scratch is sized for; "
                         "use PB200_K_RMS_NORM_BWD with caller-provided scratch", (long long)cols, kStaticMaxCols,
                kStaticScratchBytes);
        return PB200_ERR_BAD_SHAPE;
    }
    const void* ptrs[5] = {x, w, dy, dx, dw};
    for (int i = 0; i < 5; ++i)
        if (!ptrs[i] || ((uintptr_t)ptrs[i] & 15u)) {
            set_err(err_out, "buffer %d (%p) is NULL or not 16-byte aligned", i, ptrs[i]);
            return PB200_ERR_MISALIGNED;
        }
    float* scratch = nullptr;
    int rc = static_scratch_address(&scratch, err_out);
    if (rc != PB200_OK) return rc;
    // as many partial rows as fit, never more than the regular entry would use
    int64_t parts = (int64_t)(kStaticScratchBytes / sizeof(float)) / cols;
    const int64_t want = 2 * (int64_t)sm_count();
    if (parts > want) parts = want;
    if (parts > rows) parts = rows;
    return enqueue_norm_bwd(0, (int)rows, (int)cols, (float)eps, (int)parts, (cudaStream_t)(uintptr_t)stream,
                            x, w, dy, dx, dw, nullptr, scratch, err_out);
}
