// C-ABI front end: handle registry, argument validation, dispatch.
//
// Plays the role of the reference's launch shim
// (pyptx/_shim/pyptx_launch.cc:236-301 registry, :316-467 launch core,
// :484-492 raw entry) for ahead-of-time compiled sm_100a kernels.
//
// Threading: the registry is guarded by a shared mutex; a launch copies its
// record under a shared lock and enqueues outside it (the reference copies
// under a plain mutex, pyptx_launch.cc:330-343).  Error text goes to the
// caller's buffer, never to shared state.
#include "common.cuh"
#include "ptx.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdlib>
#include <mutex>
#include <shared_mutex>
#include <unordered_map>

namespace pb200 {

// Device-side status words.  Kernels receive the address as a parameter
// (device_status_ptr()) and only write on a wait that gave up.
__device__ int g_device_status[kStatusWords];

namespace {

std::shared_mutex g_mu;
std::unordered_map<int64_t, Record> g_registry;
std::atomic<int64_t> g_next_handle{1};

constexpr int kMaxDevices = 64;
std::atomic<int>  g_sm_count[kMaxDevices];
std::atomic<int*> g_status_ptr[kMaxDevices];

int current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return -1; }
    return dev;
}

bool is_row(int32_t k) {
    return k == PB200_K_RMS_NORM || k == PB200_K_LAYER_NORM || k == PB200_K_SWIGLU || k == PB200_K_SOFTMAX;
}
bool is_row_bwd(int32_t k) {
    return k == PB200_K_RMS_NORM_BWD || k == PB200_K_LAYER_NORM_BWD || k == PB200_K_SWIGLU_BWD;
}
bool is_gemm(int32_t k) {
    return k == PB200_K_GEMM_1SM || k == PB200_K_GEMM_2SM || k == PB200_K_GROUPED_GEMM ||
           k == PB200_K_GROUPED_GEMM_SWIGLU || k == PB200_K_GROUPED_GEMM_VARLEN || k == PB200_K_GEMM_PUSH;
}

// Handles whose buffers were already checked against the current device.
std::mutex g_checked_mu;
std::unordered_map<int64_t, bool> g_checked;

// "Assert the current device owns the buffers" of the reference's launch path
// (pyptx/torch_support.py:189-195 switches to the tensors' device before the launch; the raw entry
// trusts its caller).  A pointer that belongs to another GPU, or plain pageable host memory, would
// fault inside the kernel, so the raw entry looks at every buffer on the first launch of a handle,
// and on every launch when PB200_CHECK_POINTERS=1 is set in the environment.  Kernels that address
// peer memory on purpose (the push GEMM's outputs, the peer barrier's flag blocks) are exempt there.
int check_buffer_devices(const Record& r, int64_t handle, void** ptrs, size_t n, char* err) {
    static const bool always = [] { const char* e = getenv("PB200_CHECK_POINTERS"); return e && e[0] == '1'; }();
    if (!always) {
        std::lock_guard<std::mutex> lk(g_checked_mu);
        if (g_checked.count(handle)) return PB200_OK;
    }
    if (r.kernel_id == PB200_K_PEER_BARRIER) return PB200_OK;
    const int dev = current_device();
    if (dev < 0) { set_err(err, "no current CUDA device"); return PB200_ERR_NO_CUDA; }
    const size_t n_check = r.kernel_id == PB200_K_GEMM_PUSH ? (size_t)r.geom.n_inputs : n;
    for (size_t i = 0; i < n_check; ++i) {
        cudaPointerAttributes a{};
        if (cudaPointerGetAttributes(&a, ptrs[i]) != cudaSuccess) { cudaGetLastError(); continue; }
        if (a.type == cudaMemoryTypeUnregistered) {
            set_err(err, "buffer %zu (%p) is not device-accessible memory", i, ptrs[i]);
            return PB200_ERR_WRONG_DEVICE;
        }
        if (a.type == cudaMemoryTypeDevice && a.device != dev) {
            set_err(err, "buffer %zu (%p) lives on device %d, the current device is %d", i, ptrs[i], a.device, dev);
            return PB200_ERR_WRONG_DEVICE;
        }
    }
    if (!always) {
        std::lock_guard<std::mutex> lk(g_checked_mu);
        g_checked[handle] = true;
    }
    return PB200_OK;
}

}  // namespace

int sm_count() {
    int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return 148;
    int n = g_sm_count[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 148;
    }
    g_sm_count[dev].store(n, std::memory_order_relaxed);
    return n;
}

int* device_status_ptr() {
    int dev = current_device();
    if (dev < 0 || dev >= kMaxDevices) return nullptr;
    int* p = g_status_ptr[dev].load(std::memory_order_acquire);
    if (p) return p;
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_device_status) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    g_status_ptr[dev].store((int*)addr, std::memory_order_release);
    return (int*)addr;
}

EncodeTiledFn encode_tiled_fn() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
        else
            cudaGetLastError();
    });
    return fn;
}

int make_tensor_map(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle, char* err) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) { set_err(err, "cuTensorMapEncodeTiled is not available from this driver"); return PB200_ERR_NO_TMA_API; }
    cuuint64_t gdim[5]; cuuint64_t gstr[4]; cuuint32_t bx[5]; cuuint32_t es[5];
    for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
    CUresult rc = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        set_err(err, "cuTensorMapEncodeTiled failed (CUresult %d) rank=%d dim0=%llu box0=%u", (int)rc, rank,
                (unsigned long long)dims[0], box[0]);
        return PB200_ERR_TMA_ENCODE;
    }
    return PB200_OK;
}

}  // namespace pb200

using namespace pb200;

extern "C" {

PB200_API int64_t pb200_create(int32_t kernel_id, const int64_t* dims, size_t n_dims,
                     const double* fparams, size_t n_fparams, uint64_t flags, char* err_out) {
    if (err_out) err_out[0] = 0;
    Record r;
    r.kernel_id = kernel_id;
    if (n_dims > 8 || (n_dims > 0 && !dims)) { set_err(err_out, "n_dims=%zu out of range", n_dims); return PB200_ERR_BAD_SHAPE; }
    if (n_fparams > 4 || (n_fparams > 0 && !fparams)) { set_err(err_out, "n_fparams=%zu out of range", n_fparams); return PB200_ERR_BAD_SHAPE; }
    r.n_dims = (int)n_dims;
    for (size_t i = 0; i < n_dims; ++i) r.dims[i] = dims[i];
    r.n_fparams = (int)n_fparams;
    for (size_t i = 0; i < n_fparams; ++i) r.fparams[i] = fparams[i];
    r.flags = flags;
    int rc;
    if (is_row(kernel_id)) rc = plan_row(r, err_out);
    else if (is_row_bwd(kernel_id)) rc = plan_row_bwd(r, err_out);
    else if (is_gemm(kernel_id)) rc = plan_gemm(r, err_out);
    else if (kernel_id == PB200_K_FLASH_ATTN) rc = plan_attention(r, err_out);
    else if (kernel_id == PB200_K_FLASH_ATTN_BWD) rc = plan_attention_bwd(r, err_out);
    else if (kernel_id == PB200_K_PEER_BARRIER) rc = plan_peer_barrier(r, err_out);
    else { set_err(err_out, "unknown kernel id %d", kernel_id); return PB200_ERR_BAD_KERNEL; }
    if (rc != PB200_OK) return rc;
    int64_t h = g_next_handle.fetch_add(1);
    std::unique_lock<std::shared_mutex> lk(g_mu);
    g_registry.emplace(h, r);
    return h;
}

PB200_API int pb200_launch_raw(int64_t handle, uint64_t stream, void** buffer_ptrs, size_t n_buffers, char* err_out) {
    if (err_out) err_out[0] = 0;
    Record r;
    {
        std::shared_lock<std::shared_mutex> lk(g_mu);
        auto it = g_registry.find(handle);
        if (it == g_registry.end()) {
            set_err(err_out, "unknown handle %lld", (long long)handle);
            return PB200_ERR_UNKNOWN_HANDLE;
        }
        r = it->second;
    }
    const size_t want = (size_t)r.geom.n_inputs + r.geom.n_outputs + (r.geom.scratch_bytes ? 1 : 0);
    if (n_buffers != want || !buffer_ptrs) {
        set_err(err_out, "kernel %d takes %zu buffers (%u inputs + %u outputs%s), got %zu", r.kernel_id, want,
                r.geom.n_inputs, r.geom.n_outputs, r.geom.scratch_bytes ? " + 1 scratch" : "", n_buffers);
        return PB200_ERR_ARG_COUNT;
    }
    for (size_t i = 0; i < n_buffers; ++i) {
        uintptr_t a = (uintptr_t)buffer_ptrs[i];
        if (a == 0 || (a & 15u) != 0) {
            set_err(err_out, "buffer %zu (%p) is NULL or not 16-byte aligned", i, buffer_ptrs[i]);
            return PB200_ERR_MISALIGNED;
        }
    }
    if (int rc = check_buffer_devices(r, handle, buffer_ptrs, n_buffers, err_out)) return rc;
    cudaStream_t s = (cudaStream_t)(uintptr_t)stream;
    if (is_row(r.kernel_id)) return launch_row(r, s, buffer_ptrs, err_out);
    if (is_row_bwd(r.kernel_id)) return launch_row_bwd(r, s, buffer_ptrs, err_out);
    if (is_gemm(r.kernel_id)) return launch_gemm(r, s, buffer_ptrs, err_out);
    if (r.kernel_id == PB200_K_PEER_BARRIER) return launch_peer_barrier(r, s, buffer_ptrs, err_out);
    if (r.kernel_id == PB200_K_FLASH_ATTN_BWD) return launch_attention_bwd(r, s, buffer_ptrs, err_out);
    return launch_attention(r, s, buffer_ptrs, err_out);
}

PB200_API int pb200_geometry_of(int64_t handle, pb200_geometry* out) {
    if (!out) return PB200_ERR_ARG_COUNT;
    std::shared_lock<std::shared_mutex> lk(g_mu);
    auto it = g_registry.find(handle);
    if (it == g_registry.end()) return PB200_ERR_UNKNOWN_HANDLE;
    *out = it->second.geom;
    return PB200_OK;
}

PB200_API int pb200_has_handle(int64_t handle) {
    std::shared_lock<std::shared_mutex> lk(g_mu);
    return g_registry.count(handle) ? 1 : 0;
}

PB200_API size_t pb200_registry_size(void) {
    std::shared_lock<std::shared_mutex> lk(g_mu);
    return g_registry.size();
}

PB200_API void pb200_clear_registry(void) {
    std::unique_lock<std::shared_mutex> lk(g_mu);
    g_registry.clear();
    std::lock_guard<std::mutex> lk2(g_checked_mu);
    g_checked.clear();
}

PB200_API int pb200_destroy(int64_t handle) {
    std::unique_lock<std::shared_mutex> lk(g_mu);
    {
        std::lock_guard<std::mutex> lk2(g_checked_mu);
        g_checked.erase(handle);
    }
    return g_registry.erase(handle) ? PB200_OK : PB200_ERR_UNKNOWN_HANDLE;
}

PB200_API int pb200_device_status(char* err_out) {
    if (err_out) err_out[0] = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { set_err(err_out, "cudaDeviceSynchronize: %s", cudaGetErrorString(e)); return PB200_ERR_NO_CUDA; }
    int host[kStatusWords] = {0, 0, 0, 0};
    e = cudaMemcpyFromSymbol(host, g_device_status, sizeof(host));
    if (e != cudaSuccess) { set_err(err_out, "cudaMemcpyFromSymbol: %s", cudaGetErrorString(e)); return PB200_ERR_NO_CUDA; }
    if (host[0] == 0) return PB200_OK;
    int zero[kStatusWords] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_device_status, zero, sizeof(zero));
    set_err(err_out, "device wait gave up: kernel %d, wait site %d, block %d", host[1], host[2], host[3]);
    return PB200_ERR_DEVICE_TIMEOUT;
}

PB200_API uint32_t pb200_encode_idesc(int32_t m, int32_t n, int32_t bf16_inputs, int32_t a_mn_major, int32_t b_mn_major) {
    return ptx::make_idesc_f16(m, n, bf16_inputs != 0, a_mn_major != 0, b_mn_major != 0);
}
PB200_API uint64_t pb200_encode_smem_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes, uint32_t layout) {
    return ptx::make_smem_desc(smem_addr, leading_bytes, stride_bytes, layout);
}
PB200_API uint32_t pb200_swizzle128(uint32_t byte_offset) { return ptx::swizzle128(byte_offset); }

PB200_API const char* pb200_version(void) { return "0.1.0"; }
PB200_API const char* pb200_arch(void) { return "sm_100a"; }

}  // extern "C"
