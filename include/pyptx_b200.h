/*
 * pyptx_b200 -- C ABI of the B200 (sm_100a) kernel library.
 *
 * This header is the drop-in boundary.  It plays the role that the launch
 * shim plays in the reference project: a process-local registry of
 * "handles", and one generic launch entry that takes raw device pointers
 * in inputs-then-outputs order plus a CUDA stream.
 *
 * Differences from the reference shim, by design:
 *   - a handle names an ahead-of-time compiled kernel + its static shape,
 *     not a JIT-loaded CUfunction; nothing is compiled at run time;
 *   - TMA descriptors are encoded on the host per launch and passed to the
 *     kernel by value, so no device slot is patched and two launches with
 *     different pointers never race;
 *   - every device-side wait is bounded; a wait that gives up records a
 *     status word that pb200_device_status() returns.
 *
 * Conventions (same as the reference shim, pyptx/_shim/pyptx_launch.cc:316-467):
 *   - functions return 0 on success and a negative code on failure;
 *   - `err_out`, when not NULL, points at a caller-owned buffer of at least
 *     PB200_ERR_LEN bytes that receives a NUL-terminated message;
 *   - nothing throws or aborts across this boundary;
 *   - launches are asynchronous on `stream`; the library never synchronises
 *     on the launch path and allocates no device memory.
 *
 * All pointers given to pb200_launch_raw must be device pointers on the
 * current CUDA device, 16-byte aligned, to contiguous row-major arrays.
 */
#ifndef PYPTX_B200_H_
#define PYPTX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PB200_ERR_LEN 128

#if defined(__GNUC__)
#define PB200_API __attribute__((visibility("default")))
#else
#define PB200_API
#endif

/* ---- error codes (0..-8 mirror pyptx/_shim/pyptx_launch.cc:316-467) ---- */
#define PB200_OK                    0
#define PB200_ERR_NO_CUDA          -1  /* CUDA runtime / driver not usable        */
#define PB200_ERR_UNKNOWN_HANDLE   -2  /* handle not in the registry              */
#define PB200_ERR_NO_TMA_API       -3  /* cuTensorMapEncodeTiled not resolvable   */
#define PB200_ERR_ARG_COUNT        -4  /* wrong number of buffer pointers         */
#define PB200_ERR_TMA_ENCODE       -5  /* tensor-map encode failed                */
#define PB200_ERR_LAUNCH           -7  /* kernel launch failed                    */
#define PB200_ERR_CLUSTER          -8  /* cluster launch unsupported              */
#define PB200_ERR_BAD_SHAPE        -9  /* shape / option rejected at create time  */
#define PB200_ERR_MISALIGNED      -10  /* a buffer pointer is NULL or not 16-B aligned */
#define PB200_ERR_DEVICE_TIMEOUT  -11  /* a bounded device-side wait gave up      */
#define PB200_ERR_BAD_KERNEL      -12  /* unknown kernel id                       */
#define PB200_ERR_WRONG_DEVICE    -13  /* a buffer lives on another GPU or in pageable host memory */

/* ---- kernel ids: each names one reference entry point ------------------ */
/* build_rms_norm            examples/blackwell/rms_norm.py:26 (body examples/hopper/rms_norm.py:63-182)
 *   dims = {B, N}            fparams = {eps}
 *   buffers: x[B,N] f32, w[N] f32 -> y[B,N] f32                                   */
#define PB200_K_RMS_NORM       1
/* build_layer_norm          examples/blackwell/layer_norm.py:32 (body examples/hopper/layer_norm.py:57-225)
 *   dims = {B, N}            fparams = {eps}
 *   buffers: x[B,N], w[N], b[N] f32 -> y[B,N] f32                                 */
#define PB200_K_LAYER_NORM     2
/* build_fused_silu_mul      examples/blackwell/swiglu.py:32 (body examples/hopper/swiglu.py:48-156)
 *   dims = {M, F}
 *   buffers: gate[M,F], up[M,F] f32 -> out[M,F] f32                               */
#define PB200_K_SWIGLU         3
/* build_softmax             examples/hopper/softmax.py:49-182
 *   dims = {B, N}
 *   buffers: x[B,N] f32 -> y[B,N] f32                                             */
#define PB200_K_SOFTMAX        4
/* build_gemm                examples/blackwell/gemm_highperf_blackwell.py:69-313
 *   dims = {M, N, K}         flags: PB200_F_OUT_BF16
 *   buffers: A[M,K] bf16, B_T[N,K] bf16 -> D[M,N] f32 (or bf16)                   */
#define PB200_K_GEMM_1SM       5
/* build_gemm_2sm            examples/blackwell/gemm_highperf_blackwell.py:902-1246
 *   same dims / buffers as PB200_K_GEMM_1SM; M must divide by 256                 */
#define PB200_K_GEMM_2SM       6
/* build_grouped_gemm        examples/blackwell/grouped_gemm.py:61-289
 *   dims = {G, M, N, K}      flags: PB200_F_OUT_BF16
 *   buffers: A[G*M,K] bf16, B_T[G*N,K] bf16 -> C[G*M,N] f32 (or bf16)             */
#define PB200_K_GROUPED_GEMM   7
/* build_flash_attention_hopper  examples/hopper/experimental/flash_attention_hopper.py:44-465
 *   dims = {batch*heads, M_q, N_seq, head_dim}   fparams = {sm_scale}
 *   flags: PB200_F_CAUSAL, PB200_F_OUT_BF16, PB200_F_K_TRANSPOSED, PB200_F_RETURN_LSE
 *   buffers: Q[BH,M_q,d] bf16, K[BH,N_seq,d] bf16 (or K_t[BH,d,N_seq] with
 *            PB200_F_K_TRANSPOSED, the reference's layout), V[BH,N_seq,d] bf16
 *            -> O[BH,M_q,d] f32 (or bf16)                                         */
#define PB200_K_FLASH_ATTN     8

/* Fused MoE up-projection: out[g] = silu(A[g] W_gate[g]^T) * (A[g] W_up[g]^T).  The two products it
 * fuses are build_grouped_gemm (examples/blackwell/grouped_gemm.py:61-289) followed by
 * build_fused_silu_mul (examples/blackwell/swiglu.py:32); the reference has no fused entry point.
 *   dims = {G, M, F, K}      flags: PB200_F_OUT_BF16
 *   buffers: A[G*M,K] bf16, W_T[G*2F,K] bf16 (per expert: F gate rows, then F up rows)
 *            -> out[G*M,F] f32 (or bf16)                                            */
#define PB200_K_GROUPED_GEMM_SWIGLU 9

/* Grouped GEMM with per-expert row counts, the follow-up the reference names
 * (examples/hopper/grouped_gemm.py:15-17) but does not ship.
 *   dims = {G, M_total, N, K}   flags: PB200_F_OUT_BF16
 *   buffers: A[M_total,K] bf16, B_T[G*N,K] bf16, offsets[G+1] int32 (device; offsets[0] = 0,
 *            non-decreasing multiples of 128, offsets[G] <= M_total; expert e owns rows
 *            [offsets[e], offsets[e+1])) -> C[M_total,N] f32 (or bf16); rows at or beyond
 *            offsets[G] are not written                                              */
#define PB200_K_GROUPED_GEMM_VARLEN 10

/* Backward halves of the row ops, for the reference's autograd hook differentiable_kernel
 * (pyptx/torch_support.py:446-519); the reference ships no backward kernels of its own.
 *   PB200_K_RMS_NORM_BWD    dims = {B, N}  fparams = {eps}
 *       buffers: x[B,N], w[N], dy[B,N] f32 -> dx[B,N], dw[N] f32            + scratch
 *   PB200_K_LAYER_NORM_BWD  dims = {B, N}  fparams = {eps}
 *       buffers: x[B,N], w[N], dy[B,N] f32 -> dx[B,N], dw[N], db[N] f32     + scratch
 *   PB200_K_SWIGLU_BWD      dims = {M, F}
 *       buffers: gate[M,F], up[M,F], dout[M,F] f32 -> dgate[M,F], dup[M,F] f32
 * "+ scratch": these kernels need pb200_geometry.scratch_bytes of device memory for partial
 * column sums; the caller passes it as one extra pointer after the outputs (contents are
 * overwritten, nothing has to be cleared).  N <= 16384.                                  */
#define PB200_K_RMS_NORM_BWD   11
#define PB200_K_LAYER_NORM_BWD 12
#define PB200_K_SWIGLU_BWD     13

/* Multi-GPU extensions (one process per GPU, buffers mapped between the GPUs of a node by the
 * caller, e.g. through torch's symmetric memory).  The reference is single-device and has no
 * counterpart for either.
 *   PB200_K_GEMM_PUSH   the dense GEMM with its result stored to n_dest regions at once
 *       dims = {n_dest (1..8), cta_group (1|2), M, N, K}   flags: PB200_F_OUT_BF16
 *       buffers: A[M,K] bf16, B_T[N,K] bf16 -> n_dest pointers, each an [M,N] row-major f32
 *                (or bf16) region; regions may be peer-mapped memory of other GPUs.  With one
 *                region per rank, all at this rank's row offset of a gathered buffer, the
 *                all-gather of D rides on the epilogue's TMA stores (none of them multicast).
 *                A peer sees the data after the stream-ordered barrier below.
 *   PB200_K_PEER_BARRIER   flag barrier across the ranks of a node, stream-ordered and bounded
 *       dims = {world (1..8), rank}   fparams = {timeout in seconds, default 10}
 *       buffers: world pointers, entry p = rank p's 64-byte flag block (16 uint32, zero before
 *                the first call, mapped on every rank).  On expiry the kernel returns and
 *                pb200_device_status() reports PB200_ERR_DEVICE_TIMEOUT.                       */
#define PB200_K_GEMM_PUSH      14
#define PB200_K_PEER_BARRIER   15
/* Attention backward: the half that pairs with PB200_K_FLASH_ATTN (built with PB200_F_RETURN_LSE)
 * under the reference's autograd hook differentiable_kernel (pyptx/torch_support.py:446-519); the
 * reference has no backward kernel.  Row statistics as its forward keeps them
 * (examples/hopper/experimental/flash_attention_hopper.py:205-256), here read from lse.
 *   dims = {batch*heads, S_q, S_kv, head_dim}   fparams = {sm_scale (0 -> 1/sqrt(head_dim))}
 *   flags: PB200_F_CAUSAL, PB200_F_OUT_BF16 (dtype of dQ, dK, dV; default f32), PB200_F_DETERMINISTIC
 *   buffers: Q[BH,S_q,d], K[BH,S_kv,d], V[BH,S_kv,d], O[BH,S_q,d] bf16, lse[BH,S_q] f32, dO[BH,S_q,d] bf16
 *            -> dQ[BH,S_q,d], dK[BH,S_kv,d], dV[BH,S_kv,d], then scratch (geometry.scratch_bytes)
 *   The scratch needs no initialisation: the call writes its row statistics there and (default form)
 *   clears the fp32 dQ accumulator it keeps there with a stream-ordered memset.                      */
#define PB200_K_FLASH_ATTN_BWD 16

/* ---- create-time flags -------------------------------------------------- */
#define PB200_F_OUT_BF16       (1ull << 0)  /* round the output to bf16            */
#define PB200_F_CAUSAL         (1ull << 1)  /* attention: lower-triangular mask    */
#define PB200_F_K_TRANSPOSED   (1ull << 2)  /* attention: K given as (d, N_seq)    */
/* Dense GEMM epilogue (PB200_K_GEMM_1SM / _2SM): D = act(A B_T^T + bias).  The reference's GEMMs
 * have a plain store epilogue (examples/blackwell/gemm_highperf_blackwell.py:283-311); these fuse
 * the bias add / activation a caller would otherwise run as a second pass over D.             */
#define PB200_F_BIAS           (1ull << 3)  /* third input: bias[N] f32, added per column  */
#define PB200_F_ACT_RELU       (1ull << 4)
#define PB200_F_ACT_GELU       (2ull << 4)  /* 0.5 x (1 + erf(x / sqrt 2))                 */
#define PB200_F_ACT_SILU       (3ull << 4)
#define PB200_F_ACT_MASK       (3ull << 4)
/* Attention: second output lse[BH, S_q] f32 = log(sum_j exp(scale * q_i . k_j)) over the visible keys,
 * the row statistic a backward pass needs (the reference's kernel keeps it in registers only,
 * examples/hopper/experimental/flash_attention_hopper.py:213-256).                              */
#define PB200_F_RETURN_LSE     (1ull << 6)
/* attention backward: the two-pass form (dQ in a pass of its own, no atomics, bit-reproducible);
 * the default forms dQ in the dK/dV pass and accumulates it across key tiles with fp32 atomics */
#define PB200_F_DETERMINISTIC  (1ull << 7)

/* Launch geometry of a handle, as the reference's Kernel object exposes it
 * (pyptx/kernel.py:402-447: grid, block, cluster, smem). */
typedef struct pb200_geometry {
    uint32_t grid[3];
    uint32_t block[3];
    uint32_t cluster[3];
    uint32_t smem_bytes;
    uint32_t n_inputs;
    uint32_t n_outputs;
    uint64_t scratch_bytes;   /* > 0: one scratch pointer of this size follows the outputs */
} pb200_geometry;

/* Registers a (kernel, static shape, options) record and returns a handle
 * > 0, or a negative error code.  Replaces pyptx_shim_register_launch +
 * pyptx_shim_add_scalar_param + pyptx_shim_add_tma_spec
 * (pyptx/_shim/pyptx_launch.cc:239-285): geometry, scalar parameters and
 * tensor-map layouts all follow from (kernel_id, dims, fparams, flags). */
PB200_API int64_t pb200_create(int32_t kernel_id,
                     const int64_t* dims, size_t n_dims,
                     const double* fparams, size_t n_fparams,
                     uint64_t flags, char* err_out);

/* Launches the kernel behind `handle` on `stream` (a cudaStream_t / CUstream
 * passed as an integer).  `buffer_ptrs` holds n_buffers device pointers:
 * the inputs in spec order, then the outputs, then (only for handles whose geometry reports
 * scratch_bytes > 0) one scratch buffer of that size.
 * Replaces pyptx_shim_launch_raw (pyptx/_shim/pyptx_launch.cc:484-492);
 * same argument list, same return convention.  The caller makes the buffers' device current; the
 * first launch of a handle (every launch with PB200_CHECK_POINTERS=1 in the environment) verifies
 * it and returns PB200_ERR_WRONG_DEVICE otherwise. */
PB200_API int pb200_launch_raw(int64_t handle, uint64_t stream,
                     void** buffer_ptrs, size_t n_buffers, char* err_out);

/* Fills `out` with the launch geometry of `handle`.
 * Counterpart of the Kernel.grid/.block/.cluster/.smem accessors
 * (pyptx/kernel.py:402-447). */
PB200_API int pb200_geometry_of(int64_t handle, pb200_geometry* out);

/* Registry maintenance: pyptx_shim_has_handle, pyptx_shim_registry_size,
 * pyptx_shim_clear_registry (pyptx/_shim/pyptx_launch.cc:287-301). */
PB200_API int    pb200_has_handle(int64_t handle);
PB200_API size_t pb200_registry_size(void);
PB200_API void   pb200_clear_registry(void);
PB200_API int    pb200_destroy(int64_t handle);

/* Synchronises the current device and returns the device-side status word:
 * 0 if no bounded wait has given up since the last call, else
 * PB200_ERR_DEVICE_TIMEOUT with a description in err_out.  Reading clears it.
 * The reference has no counterpart: its device waits are unbounded
 * (pyptx/ptx.py:2311-2337). */
PB200_API int pb200_device_status(char* err_out);

/* RMSNorm backward that brings its own scratch memory.  It has no counterpart in the reference.
 * For hosts that may not allocate device memory on the path that calls this library (a serving
 * process with a memory plan fixed at load time, a plugin slot that receives its tensors and
 * nothing else) and therefore cannot supply the scratch buffer PB200_K_RMS_NORM_BWD asks for.
 * Computes dx[rows,cols] and dw[cols] from x[rows,cols], w[cols], dy[rows,cols] (f32, 16-byte
 * aligned device pointers on the current device) and enqueues on `stream`; it calls no
 * allocation routine.  The scratch is a 4 MiB array inside the library image: it is held on every
 * GPU that loads the library, cols may not exceed 16384 (rejected with PB200_ERR_BAD_SHAPE), all
 * calls on one GPU share it, so calls that could overlap on the GPU must be ordered by the caller,
 * and the first call on each GPU resolves the array's address -- make it at start-up, before any
 * stream capture. */
PB200_API int pb200_rms_norm_bwd_static(int64_t rows, int64_t cols, double eps, uint64_t stream,
                                        const void* x, const void* w, const void* dy,
                                        void* dx, void* dw, char* err_out);

/* Host-side evaluation of the encodings the matrix kernels use, exported so
 * that tests can pin them to the reference's known answers.
 *   pb200_encode_idesc      tcgen05 instruction descriptor, kind::f16, f32 accumulate
 *                           (pyptx/ptx.py:3312-3366; tests/test_typed_wrappers.py:407-425)
 *   pb200_encode_smem_desc  shared-memory matrix descriptor; layout 0/2/4/6 = none/128B/64B/32B
 *                           (pyptx/ptx.py:3368-3459; tests/test_typed_wrappers.py:427-438)
 *   pb200_swizzle128        byte offset -> swizzled byte offset, Swizzle<3,4,3>
 *                           (pyptx/smem.py:476-492) */
PB200_API uint32_t pb200_encode_idesc(int32_t m, int32_t n, int32_t bf16_inputs,
                                      int32_t a_mn_major, int32_t b_mn_major);
PB200_API uint64_t pb200_encode_smem_desc(uint32_t smem_addr, uint32_t leading_bytes,
                                          uint32_t stride_bytes, uint32_t layout);
PB200_API uint32_t pb200_swizzle128(uint32_t byte_offset);

/* Library version and the architecture the kernels were compiled for. */
PB200_API const char* pb200_version(void);
PB200_API const char* pb200_arch(void);

#ifdef __cplusplus
}
#endif
#endif /* PYPTX_B200_H_ */
