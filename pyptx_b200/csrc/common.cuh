// Internal declarations shared by the C-ABI front end (abi.cu) and the
// kernel translation units.  Nothing here is part of the public ABI.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/pyptx_b200.h"

namespace pb200 {

// One registry entry: the static description of a launch.
struct Record {
    int32_t  kernel_id = 0;
    int64_t  dims[8]   = {0, 0, 0, 0, 0, 0, 0, 0};
    int      n_dims    = 0;
    double   fparams[4] = {0, 0, 0, 0};
    int      n_fparams = 0;
    uint64_t flags     = 0;
    pb200_geometry geom{};
};

inline void set_err(char* err_out, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
inline void set_err(char* err_out, const char* fmt, ...) {
    if (!err_out) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_out, PB200_ERR_LEN, fmt, ap);
    va_end(ap);
}

// Per-kernel-family hooks.  `plan_*` validates the shape and fills the launch
// geometry at create time (host only, no CUDA call); `launch_*` enqueues the
// kernel.  Both return a PB200_* code.
int plan_row(Record& r, char* err);
int launch_row(const Record& r, cudaStream_t stream, void** ptrs, char* err);

int plan_gemm(Record& r, char* err);
int launch_gemm(const Record& r, cudaStream_t stream, void** ptrs, char* err);

int plan_row_bwd(Record& r, char* err);
int launch_row_bwd(const Record& r, cudaStream_t stream, void** ptrs, char* err);
// Backward norm pass + fold of the partial column sums, with the scratch given explicitly.
int enqueue_norm_bwd(int mode, int rows, int n, float eps, int parts, cudaStream_t s, const void* x, const void* w,
                     const void* dy, void* dx, void* dw, void* db, void* scratch, char* err);
size_t norm_bwd_scratch_bytes(int mode, int parts, int n);

int plan_peer_barrier(Record& r, char* err);
int launch_peer_barrier(const Record& r, cudaStream_t stream, void** ptrs, char* err);

int plan_attention(Record& r, char* err);
int launch_attention(const Record& r, cudaStream_t stream, void** ptrs, char* err);

int plan_attention_bwd(Record& r, char* err);
int launch_attention_bwd(const Record& r, cudaStream_t stream, void** ptrs, char* err);

// Device-side status word (defined in abi.cu's translation unit of the same
// library; each .cu that needs it reaches it through report_timeout()).
// Layout: [0] = code (0 ok), [1] = kernel id, [2] = wait site, [3] = block id.
constexpr int kStatusWords = 4;

// Number of SMs of the current device, cached per device.  Returns 148 (the
// B200 count) when no device is visible so that planning works on a CPU box.
int sm_count();

// Resolves cuTensorMapEncodeTiled through the runtime (no link-time libcuda).
// Returns nullptr when the driver is not present.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// Encodes a row-major tensor of `rank` dims (dims[0] innermost) with the given
// box and swizzle.  strides_bytes has rank-1 entries (dim 1 .. rank-1).
int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle, char* err);

// Address of the device status words on the current device (host-callable).
int* device_status_ptr();

// Launch with the programmatic-stream-serialization attribute: the kernel's CTAs may be scheduled
// while the previous kernel of the stream drains; the kernel itself waits (ptx::pdl_wait) before it
// touches global memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_with_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream,
                            Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace pb200
