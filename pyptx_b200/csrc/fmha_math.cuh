// Arithmetic helpers shared by the attention forward and backward kernels: MUFU and FMA-pipe
// exponentials, the packed f32x2 forms of fma / add, and a three-input max.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace pb200 {
namespace {

__device__ __forceinline__ float fast_exp2(float x) {
    // Not volatile on purpose: the compiler must be free to batch the FMAs of a chunk ahead of
    // its exponentials; a volatile asm pins every ex2 behind its own FMA and serialises the chunk.
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// max of three (one instruction on sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// (a0, a1) * scale + bias on the packed-f32x2 path: one FFMA2 for two scores.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float scale, float bias) {
    asm("{\n.reg .b64 a, s, b, d;\n"
        "mov.b64 a, {%2, %3};\nmov.b64 s, {%4, %4};\nmov.b64 b, {%5, %5};\n"
        "fma.rn.f32x2 d, a, s, b;\nmov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(scale), "f"(bias));
}
// General packed forms: (d0, d1) = (a0, a1) * (b0, b1) + (c0, c1) and (d0, d1) = (a0, a1) + (b0, b1).
__device__ __forceinline__ void fma2v(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n.reg .b64 a, b, c, d;\n"
        "mov.b64 a, {%2, %3};\nmov.b64 b, {%4, %5};\nmov.b64 c, {%6, %7};\n"
        "fma.rn.f32x2 d, a, b, c;\nmov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add2v(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n.reg .b64 a, b, d;\n"
        "mov.b64 a, {%2, %3};\nmov.b64 b, {%4, %5};\n"
        "add.rn.f32x2 d, a, b;\nmov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// 2^x for two arguments on the FMA pipe instead of the MUFU unit, which is the scarcer resource
// of this kernel (16 exponentials per clock per SM against 8192 MMA flops).  Round-to-nearest
// split x = n + f with the 1.5*2^23 trick, cubic minimax for 2^f on [-0.5, 0.5] (relative error
// 1.0e-4, far below the bf16 rounding of P), n added into the exponent field.  The argument is
// clamped to [-126, 127]: below, the result underflows to ~0 as it should; above, it saturates near
// 2^127 instead of wrapping into the sign bit, so that a caller's overflow check still fires.
__device__ __forceinline__ void exp2_fma_pair(float& r0, float& r1, float x0, float x1) {
    constexpr float kMagic = 12582912.0f;
    x0 = fminf(fmaxf(x0, -126.0f), 127.0f);
    x1 = fminf(fmaxf(x1, -126.0f), 127.0f);
    float t0, t1, n0, n1, f0, f1, p0, p1;
    add2v(t0, t1, x0, x1, kMagic, kMagic);
    add2v(n0, n1, t0, t1, -kMagic, -kMagic);
    add2v(f0, f1, x0, x1, -n0, -n1);
    fma2v(p0, p1, f0, f1, 0.05500892f, 0.05500892f, 0.24221097f, 0.24221097f);
    fma2v(p0, p1, p0, p1, f0, f1, 0.69328290f, 0.69328290f);
    fma2v(p0, p1, p0, p1, f0, f1, 1.0f, 1.0f);
    r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
    r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}
// (acc0, acc1) += (p0, p1): one FADD2.
__device__ __forceinline__ void add2(float& acc0, float& acc1, float p0, float p1) {
    asm("{\n.reg .b64 a, p;\n"
        "mov.b64 a, {%0, %1};\nmov.b64 p, {%2, %3};\n"
        "add.rn.f32x2 a, a, p;\nmov.b64 {%0, %1}, a;\n}"
        : "+f"(acc0), "+f"(acc1) : "f"(p0), "f"(p1));
}

// (d0, d1) = (a0, a1) * (b0, b1): one FMUL2.
__device__ __forceinline__ void mul2v(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n.reg .b64 a, b, d;\n"
        "mov.b64 a, {%2, %3};\nmov.b64 b, {%4, %5};\n"
        "mul.rn.f32x2 d, a, b;\nmov.b64 {%0, %1}, d;\n}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

}  // namespace
}  // namespace pb200
