// Row-wise f32 kernels for sm_100a: RMSNorm, LayerNorm, SwiGLU (silu(g)*u), softmax.
//
// These are HBM-bound (0.25-0.5 flop per byte), so the design is about bytes in
// flight, not arithmetic:
//   * one CTA owns one row at a time and keeps the whole row in registers
//     (x is read from HBM exactly once; the second pass runs out of registers);
//   * every global access is a 128-bit vector, consecutive lanes touch
//     consecutive 16-byte segments (fully coalesced 512-byte warp requests);
//   * all of a thread's loads are issued before the first use, so a CTA of
//     256 threads x 8 float4 has 32 KiB outstanding, and 6-8 resident CTAs per
//     SM cover the HBM latency-bandwidth product;
//   * row reductions are warp shuffles plus one shared-memory exchange
//     (one __syncthreads per reduction, no serial tail);
//   * inputs are read with the streaming/no-allocate path and outputs written
//     with streaming stores, since nothing is reused.
//
// Math follows the reference kernels' formulas
// (examples/hopper/rms_norm.py:105-162, layer_norm.py:120-215,
//  swiglu.py:100-140, softmax.py:100-170) with two deliberate changes that
// tighten accuracy to 1e-5 relative of an fp32 CPU evaluation: full-precision
// rsqrtf, division and (in SwiGLU) expf instead of the .approx instructions
// (softmax keeps ex2.approx on an exactly computed x - max, whose error stays
// near 1e-6), and a two-pass variance (sum of squared deviations from the mean,
// taken over registers) instead of E[x^2]-mean^2.
#include "common.cuh"
#include "ptx.cuh"

#include <cuda_bf16.h>

namespace pb200 {
namespace {

constexpr int kWarp = 32;

__device__ __forceinline__ float4 ld_stream(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(float4* p, const float4& v) {
    asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// Four results to element index 4*idx4 of an f32 or bf16 array (bf16 = the fused output cast).
template <typename OutT>
__device__ __forceinline__ void store4(void* base, size_t idx4, const float4& v) {
    if (sizeof(OutT) == 4) {
        st_stream(reinterpret_cast<float4*>(base) + idx4, v);
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        asm volatile("st.global.cs.v2.b32 [%0], {%1, %2};"
                     :: "l"(reinterpret_cast<uint2*>(base) + idx4), "r"(*reinterpret_cast<uint32_t*>(&lo)),
                        "r"(*reinterpret_cast<uint32_t*>(&hi)) : "memory");
    }
}

constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = kWarp / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide reduction with a single barrier: each warp publishes its partial,
// then every thread folds all partials itself.  `slot` must alternate between
// two buffers on consecutive calls so that a warp that races ahead to the next
// reduction cannot overwrite partials that a slower warp has not read yet.
template <int THREADS, bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float* slot) {
    constexpr int NW = THREADS / kWarp;
    v = IS_MAX ? warp_max(v) : warp_sum(v);
    if (NW == 1) return v;
    if ((threadIdx.x & (kWarp - 1)) == 0) slot[threadIdx.x / kWarp] = v;
    __syncthreads();
    float r = slot[0];
#pragma unroll
    for (int i = 1; i < NW; ++i) r = IS_MAX ? fmaxf(r, slot[i]) : r + slot[i];
    return r;
}

// ---------------------------------------------------------------------------
// RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w
// ---------------------------------------------------------------------------
// Programmatic dependent launch (see ptx.cuh): about 2 us of launch latency between two 20 us kernels.
__device__ __forceinline__ void pdl_prologue() {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
}

template <int THREADS, int VPT, typename OutT>
__global__ void __launch_bounds__(THREADS)
rms_norm_kernel(const float4* __restrict__ x, const float4* __restrict__ w,
                void* __restrict__ y, int rows, int n4, float inv_n, float eps) {
    pdl_prologue();
    __shared__ float red[2][kWarp];
    int flip = 0;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* xr = x + (size_t)row * n4;
        const size_t row4 = (size_t)row * n4;
        float4 v[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            v[i] = idx < n4 ? ld_stream(xr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i)
            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        float tot = block_reduce<THREADS, false>(ss, red[flip]);
        flip ^= 1;
        float rstd = rsqrtf(tot * inv_n + eps);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                float4 g = __ldg(w + idx);
                float4 o;
                o.x = v[i].x * rstd * g.x;
                o.y = v[i].y * rstd * g.y;
                o.z = v[i].z * rstd * g.z;
                o.w = v[i].w * rstd * g.w;
                store4<OutT>(y, row4 + idx, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// LayerNorm: y = (x - mean) * rsqrt(var + eps) * w + b, var over registers
// ---------------------------------------------------------------------------
template <int THREADS, int VPT, typename OutT>
__global__ void __launch_bounds__(THREADS)
layer_norm_kernel(const float4* __restrict__ x, const float4* __restrict__ w,
                  const float4* __restrict__ b, void* __restrict__ y,
                  int rows, int n4, float inv_n, float eps) {
    pdl_prologue();
    __shared__ float red[2][kWarp];
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* xr = x + (size_t)row * n4;
        const size_t row4 = (size_t)row * n4;
        float4 v[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            v[i] = idx < n4 ? ld_stream(xr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        float mean = block_reduce<THREADS, false>(s, red[0]) * inv_n;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                float dx = v[i].x - mean, dy = v[i].y - mean, dz = v[i].z - mean, dw = v[i].w - mean;
                q += dx * dx + dy * dy + dz * dz + dw * dw;
            }
        }
        float var = block_reduce<THREADS, false>(q, red[1]) * inv_n;
        float rstd = rsqrtf(var + eps);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                float4 g = __ldg(w + idx);
                float4 c = __ldg(b + idx);
                float4 o;
                o.x = (v[i].x - mean) * rstd * g.x + c.x;
                o.y = (v[i].y - mean) * rstd * g.y + c.y;
                o.z = (v[i].z - mean) * rstd * g.z + c.z;
                o.w = (v[i].w - mean) * rstd * g.w + c.w;
                store4<OutT>(y, row4 + idx, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Softmax: y = exp(x - max) / sum(exp(x - max))
// ---------------------------------------------------------------------------
template <int THREADS, int VPT, typename OutT>
__global__ void __launch_bounds__(THREADS)
softmax_kernel(const float4* __restrict__ x, void* __restrict__ y, int rows, int n4) {
    pdl_prologue();
    __shared__ float red[2][kWarp];
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* xr = x + (size_t)row * n4;
        const size_t row4 = (size_t)row * n4;
        float4 v[VPT];
        const float ninf = -INFINITY;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            v[i] = idx < n4 ? ld_stream(xr + idx) : make_float4(ninf, ninf, ninf, ninf);
        }
        float m = ninf;
#pragma unroll
        for (int i = 0; i < VPT; ++i) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        m = block_reduce<THREADS, true>(m, red[0]);
        // exp(x - m) as 2^((x - m) * log2(e)): one subtract, one multiply and one MUFU op per
        // element.  (x - m) is exact to 1 ulp, so the relative error stays near 1e-6 for the
        // |x - m| < 40 range that still contributes to the sum.
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            v[i].x = exp2_approx((v[i].x - m) * kLog2e);
            v[i].y = exp2_approx((v[i].y - m) * kLog2e);
            v[i].z = exp2_approx((v[i].z - m) * kLog2e);
            v[i].w = exp2_approx((v[i].w - m) * kLog2e);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        s = block_reduce<THREADS, false>(s, red[1]);
        const float inv = __frcp_rn(s);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            int idx = threadIdx.x + i * THREADS;
            if (idx < n4) {
                float4 o;
                o.x = v[i].x * inv;
                o.y = v[i].y * inv;
                o.z = v[i].z * inv;
                o.w = v[i].w * inv;
                store4<OutT>(y, row4 + idx, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Rows too long for the register-resident kernels: three streaming passes.
// The second and third pass re-read the row, which a 126 MB L2 serves.
// MODE 0 = RMSNorm, 1 = LayerNorm, 2 = softmax.
// ---------------------------------------------------------------------------
template <int MODE, typename OutT>
__global__ void __launch_bounds__(1024)
long_row_kernel(const float4* __restrict__ x, const float4* __restrict__ w,
                const float4* __restrict__ b, void* __restrict__ y,
                int rows, int n4, float inv_n, float eps) {
    pdl_prologue();
    constexpr int THREADS = 1024;
    __shared__ float red[2][kWarp];
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const float4* xr = x + (size_t)row * n4;
        const size_t row4 = (size_t)row * n4;
        float a = MODE == 2 ? -INFINITY : 0.f;
        for (int idx = threadIdx.x; idx < n4; idx += THREADS) {
            float4 t = xr[idx];
            if (MODE == 0) a += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
            if (MODE == 1) a += (t.x + t.y) + (t.z + t.w);
            if (MODE == 2) a = fmaxf(a, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
        }
        float first = block_reduce<THREADS, MODE == 2>(a, red[0]);
        float second = 0.f;
        if (MODE != 0) {
            float mean = first * inv_n;
            float q = 0.f;
            for (int idx = threadIdx.x; idx < n4; idx += THREADS) {
                float4 t = xr[idx];
                if (MODE == 1) {
                    float dx = t.x - mean, dy = t.y - mean, dz = t.z - mean, dw = t.w - mean;
                    q += dx * dx + dy * dy + dz * dz + dw * dw;
                } else {
                    q += (expf(t.x - first) + expf(t.y - first)) + (expf(t.z - first) + expf(t.w - first));
                }
            }
            second = block_reduce<THREADS, false>(q, red[1]);
        }
        for (int idx = threadIdx.x; idx < n4; idx += THREADS) {
            float4 t = xr[idx];
            float4 o;
            if (MODE == 0) {
                float rstd = rsqrtf(first * inv_n + eps);
                float4 g = __ldg(w + idx);
                o.x = t.x * rstd * g.x; o.y = t.y * rstd * g.y; o.z = t.z * rstd * g.z; o.w = t.w * rstd * g.w;
            } else if (MODE == 1) {
                float mean = first * inv_n;
                float rstd = rsqrtf(second * inv_n + eps);
                float4 g = __ldg(w + idx);
                float4 c = __ldg(b + idx);
                o.x = (t.x - mean) * rstd * g.x + c.x; o.y = (t.y - mean) * rstd * g.y + c.y;
                o.z = (t.z - mean) * rstd * g.z + c.z; o.w = (t.w - mean) * rstd * g.w + c.w;
            } else {
                o.x = expf(t.x - first) / second; o.y = expf(t.y - first) / second;
                o.z = expf(t.z - first) / second; o.w = expf(t.w - first) / second;
            }
            store4<OutT>(y, row4 + idx, o);
        }
        __syncthreads();  // red[] is reused by the next row
    }
}

// ---------------------------------------------------------------------------
// SwiGLU: out = silu(gate) * up = gate / (1 + exp(-gate)) * up, flat over M*F.
// Each thread keeps UNROLL independent 16-byte loads per operand in flight.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float silu_mul(float g, float u) {
    return g / (1.0f + expf(-g)) * u;
}

template <int THREADS, int UNROLL, typename OutT>
__global__ void __launch_bounds__(THREADS)
swiglu_kernel(const float4* __restrict__ gate, const float4* __restrict__ up,
              void* __restrict__ out, size_t total4) {
    pdl_prologue();
    const size_t tile = (size_t)THREADS * UNROLL;
    for (size_t base = (size_t)blockIdx.x * tile; base < total4; base += (size_t)gridDim.x * tile) {
        float4 g[UNROLL], u[UNROLL];
#pragma unroll
        for (int i = 0; i < UNROLL; ++i) {
            size_t idx = base + threadIdx.x + (size_t)i * THREADS;
            if (idx < total4) { g[i] = ld_stream(gate + idx); u[i] = ld_stream(up + idx); }
        }
#pragma unroll
        for (int i = 0; i < UNROLL; ++i) {
            size_t idx = base + threadIdx.x + (size_t)i * THREADS;
            if (idx < total4) {
                float4 o;
                o.x = silu_mul(g[i].x, u[i].x);
                o.y = silu_mul(g[i].y, u[i].y);
                o.z = silu_mul(g[i].z, u[i].z);
                o.w = silu_mul(g[i].w, u[i].w);
                store4<OutT>(out, idx, o);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Host side: pick a (THREADS, VPT) instantiation that covers N with the row in
// registers, and a grid that is one CTA per row (the hardware block scheduler
// balances the rows over the SMs; the per-CTA row loop only matters when the
// row count exceeds the grid limit).
// ---------------------------------------------------------------------------
struct RowConfig { int threads; int vpt; };

// `threads` > 0 asks for that CTA size (a tuning override carried in dims[2]); the smallest
// float4-per-thread count that covers the row is chosen for it.
RowConfig pick_row_config(int64_t n4, int threads = 0) {
    if (threads == 128 || threads == 256 || threads == 512 || threads == 1024) {
        for (int vpt : {1, 2, 4, 8, 16})
            if ((int64_t)threads * vpt >= n4) return {threads, vpt};
    }
    // Default: 8 float4 per thread (32 KiB per 256-thread CTA in flight).
    const RowConfig table[] = {
        {32, 1}, {32, 2}, {32, 4}, {64, 4}, {128, 4}, {128, 8}, {256, 8}, {512, 8}, {1024, 8},
    };
    for (const RowConfig& c : table)
        if ((int64_t)c.threads * c.vpt >= n4) return c;
    return {1024, 0};  // long-row kernel
}

// Return code of this thread's last cudaLaunchKernelEx (launch_row reads it after the dispatch).
thread_local cudaError_t t_launch_rc = cudaSuccess;

// Launch with the programmatic-serialization attribute (see pdl_prologue).
template <typename... KArgs, typename... Args>
void launch_pdl(void (*kernel)(KArgs...), dim3 grid, int threads, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3((unsigned)threads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    t_launch_rc = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <int THREADS, int VPT, typename OutT>
void launch_typed(int kid, dim3 grid, cudaStream_t s, void** p, int rows, int n4, float inv_n, float eps) {
    if (kid == PB200_K_RMS_NORM)
        launch_pdl(rms_norm_kernel<THREADS, VPT, OutT>, grid, THREADS, s,
                   (const float4*)p[0], (const float4*)p[1], p[2], rows, n4, inv_n, eps);
    else if (kid == PB200_K_LAYER_NORM)
        launch_pdl(layer_norm_kernel<THREADS, VPT, OutT>, grid, THREADS, s,
                   (const float4*)p[0], (const float4*)p[1], (const float4*)p[2], p[3], rows, n4, inv_n, eps);
    else
        launch_pdl(softmax_kernel<THREADS, VPT, OutT>, grid, THREADS, s, (const float4*)p[0], p[1], rows, n4);
}
template <int THREADS, int VPT>
void launch_one(int kid, bool bf16_out, dim3 grid, cudaStream_t s, void** p, int rows, int n4, float inv_n, float eps) {
    if (bf16_out) launch_typed<THREADS, VPT, __nv_bfloat16>(kid, grid, s, p, rows, n4, inv_n, eps);
    else launch_typed<THREADS, VPT, float>(kid, grid, s, p, rows, n4, inv_n, eps);
}

template <typename OutT>
void launch_long(int kid, dim3 grid, cudaStream_t s, void** p, int rows, int n4, float inv_n, float eps) {
    if (kid == PB200_K_RMS_NORM)
        launch_pdl(long_row_kernel<0, OutT>, grid, 1024, s, (const float4*)p[0], (const float4*)p[1], (const float4*)nullptr, p[2], rows, n4, inv_n, eps);
    else if (kid == PB200_K_LAYER_NORM)
        launch_pdl(long_row_kernel<1, OutT>, grid, 1024, s, (const float4*)p[0], (const float4*)p[1], (const float4*)p[2], p[3], rows, n4, inv_n, eps);
    else
        launch_pdl(long_row_kernel<2, OutT>, grid, 1024, s, (const float4*)p[0], (const float4*)nullptr, (const float4*)nullptr, p[1], rows, n4, inv_n, eps);
}
template <int UNROLL>
void launch_swiglu(bool bf16_out, dim3 grid, cudaStream_t s, void** p, size_t total4) {
    if (bf16_out)
        launch_pdl(swiglu_kernel<256, UNROLL, __nv_bfloat16>, grid, 256, s, (const float4*)p[0], (const float4*)p[1], p[2], total4);
    else
        launch_pdl(swiglu_kernel<256, UNROLL, float>, grid, 256, s, (const float4*)p[0], (const float4*)p[1], p[2], total4);
}

constexpr int kSwigluThreads = 256;
constexpr int kSwigluUnroll = 2;

}  // namespace

int plan_row(Record& r, char* err) {
    // dims = {rows, cols} plus an optional tuning word: CTA size for the row kernels (128 / 256 /
    // 512 / 1024), float4 pairs in flight per thread for SwiGLU (2 / 4 / 8; default 2).  0 or absent = default.
    if (r.n_dims != 2 && r.n_dims != 3) { set_err(err, "row kernel needs dims = {rows, cols}, got %d dims", r.n_dims); return PB200_ERR_BAD_SHAPE; }
    const int tune = r.n_dims == 3 ? (int)r.dims[2] : 0;
    r.dims[7] = tune;
    r.n_dims = 2;
    const int64_t rows = r.dims[0], n = r.dims[1];
    if (rows <= 0 || n <= 0) { set_err(err, "rows=%lld cols=%lld must be positive", (long long)rows, (long long)n); return PB200_ERR_BAD_SHAPE; }
    if (n % 4 != 0) { set_err(err, "cols=%lld must be divisible by 4 (128-bit vector access)", (long long)n); return PB200_ERR_BAD_SHAPE; }
    if (rows > 0x7fffffffLL || n > 0x7fffffffLL) { set_err(err, "rows/cols exceed 2^31-1"); return PB200_ERR_BAD_SHAPE; }
    pb200_geometry& g = r.geom;
    g.grid[1] = g.grid[2] = 1; g.block[1] = g.block[2] = 1;
    g.cluster[0] = g.cluster[1] = g.cluster[2] = 1;
    g.smem_bytes = 0;
    g.n_outputs = 1;
    if (r.kernel_id == PB200_K_SWIGLU) {
        const int64_t total4 = rows * n / 4;
        const int unroll = (tune == 4 || tune == 8) ? tune : kSwigluUnroll;
        const int64_t tile = (int64_t)kSwigluThreads * unroll;
        int64_t ctas = (total4 + tile - 1) / tile;
        if (ctas > 0x7fffffffLL) ctas = 0x7fffffffLL;
        g.grid[0] = (uint32_t)ctas; g.block[0] = kSwigluThreads;
        g.n_inputs = 2;
        return PB200_OK;
    }
    RowConfig c = pick_row_config(n / 4, tune);
    g.grid[0] = (uint32_t)rows; g.block[0] = (uint32_t)c.threads;
    g.smem_bytes = 2 * kWarp * sizeof(float);
    g.n_inputs = r.kernel_id == PB200_K_RMS_NORM ? 2 : r.kernel_id == PB200_K_LAYER_NORM ? 3 : 1;
    return PB200_OK;
}

int launch_row(const Record& r, cudaStream_t s, void** p, char* err) {
    const int rows = (int)r.dims[0];
    const int n = (int)r.dims[1];
    const int n4 = n / 4;
    const float inv_n = 1.0f / (float)n;
    const float eps = (float)r.fparams[0];
    dim3 grid(r.geom.grid[0]);
    const bool bf16_out = (r.flags & PB200_F_OUT_BF16) != 0;
    t_launch_rc = cudaSuccess;
    if (r.kernel_id == PB200_K_SWIGLU) {
        const int tune = (int)r.dims[7];
        const size_t total4 = (size_t)rows * n4;
        if (tune == 4) launch_swiglu<4>(bf16_out, grid, s, p, total4);
        else if (tune == 8) launch_swiglu<8>(bf16_out, grid, s, p, total4);
        else launch_swiglu<kSwigluUnroll>(bf16_out, grid, s, p, total4);
    } else {
        RowConfig c = pick_row_config(n4, (int)r.dims[7]);
        const int kid = r.kernel_id;
#define PB200_ROW_CASE(T, V) \
        if (c.threads == T && c.vpt == V) launch_one<T, V>(kid, bf16_out, grid, s, p, rows, n4, inv_n, eps); else
        PB200_ROW_CASE(32, 1) PB200_ROW_CASE(32, 2) PB200_ROW_CASE(32, 4) PB200_ROW_CASE(64, 4)
        PB200_ROW_CASE(128, 4) PB200_ROW_CASE(128, 8) PB200_ROW_CASE(256, 8) PB200_ROW_CASE(512, 8)
        PB200_ROW_CASE(1024, 8)
        PB200_ROW_CASE(128, 1) PB200_ROW_CASE(128, 2) PB200_ROW_CASE(128, 16)
        PB200_ROW_CASE(256, 1) PB200_ROW_CASE(256, 2) PB200_ROW_CASE(256, 4) PB200_ROW_CASE(256, 16)
        PB200_ROW_CASE(512, 1) PB200_ROW_CASE(512, 2) PB200_ROW_CASE(512, 4) PB200_ROW_CASE(512, 16)
        PB200_ROW_CASE(1024, 1) PB200_ROW_CASE(1024, 2) PB200_ROW_CASE(1024, 4) PB200_ROW_CASE(1024, 16)
        {
            if (bf16_out) launch_long<__nv_bfloat16>(kid, grid, s, p, rows, n4, inv_n, eps);
            else launch_long<float>(kid, grid, s, p, rows, n4, inv_n, eps);
        }
#undef PB200_ROW_CASE
    }
    cudaError_t e = cudaGetLastError();
    if (t_launch_rc != cudaSuccess) e = t_launch_rc;
    if (e != cudaSuccess) { set_err(err, "row kernel launch failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    return PB200_OK;
}

}  // namespace pb200
