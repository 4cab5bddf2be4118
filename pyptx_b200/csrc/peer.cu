// Flag barrier between the GPUs of one node, for buffers that ranks write into each other's
// memory (the push epilogue of the GEMM): stream-ordered, no host involvement, bounded.
//
// Every rank owns one 64-byte flag block in memory that all ranks have mapped (peer access):
//   words 0..7   arrival counters, word p written by rank p
//   word  8      this rank's own call counter (only its owner touches it)
// A barrier call on rank r increments r's counter to e, stores e into word r of every rank's
// block (release, system scope), then waits until every word of its own block has reached e
// (acquire, system scope).  All ranks call the barrier the same number of times, so the
// counters agree without passing an epoch from the host, which keeps the launch replayable
// from a CUDA graph.  The blocks must be zero before the first call.
//
// The wait is bounded: after `timeout` seconds the waiting thread records
// (PB200_ERR_DEVICE_TIMEOUT, kernel id, peer, rank) in the device status word and returns, so
// a peer that never arrives leaves this GPU's context usable.  The kernels of different ranks
// wait on one another and must therefore run on different GPUs.
//
// The reference has no multi-GPU path (its kernels are single-device); this file has no
// counterpart there.
#include "common.cuh"

namespace pb200 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kCounterWord = 8;

struct FlagBlocks {
    uint32_t* block[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(32, 1)
peer_barrier_kernel(FlagBlocks flags, int world, int rank, uint64_t timeout_ns, int* status, int kernel_id) {
    __shared__ uint32_t epoch_s;
    uint32_t* mine = flags.block[rank];
    if (threadIdx.x == 0) {
        const uint32_t e = mine[kCounterWord] + 1u;
        mine[kCounterWord] = e;
        epoch_s = e;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    const int p = (int)threadIdx.x;
    if (p >= world) return;
    // Everything this GPU wrote before the barrier (earlier kernels of the stream included)
    // is ordered before the flag by the release at system scope.
    __threadfence_system();
    st_release_sys(flags.block[p] + rank, epoch);
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine + p) - epoch) < 0) {
        __nanosleep(64);
        if ((++spins & 255u) == 0 && global_timer_ns() - t0 > timeout_ns) {
            if (status != nullptr && atomicCAS(status, 0, PB200_ERR_DEVICE_TIMEOUT) == 0) {
                status[1] = kernel_id;
                status[2] = p;
                status[3] = rank;
            }
            break;
        }
    }
}

}  // namespace

// dims = {world, rank}; fparams = {timeout in seconds (default 10)}.
int plan_peer_barrier(Record& r, char* err) {
    if (r.n_dims != 2) { set_err(err, "peer barrier needs dims {world, rank}, got %d dims", r.n_dims); return PB200_ERR_BAD_SHAPE; }
    const int64_t world = r.dims[0], rank = r.dims[1];
    if (world < 1 || world > kMaxRanks) { set_err(err, "world=%lld must be in [1, %d]", (long long)world, kMaxRanks); return PB200_ERR_BAD_SHAPE; }
    if (rank < 0 || rank >= world) { set_err(err, "rank=%lld outside [0, %lld)", (long long)rank, (long long)world); return PB200_ERR_BAD_SHAPE; }
    if (r.n_fparams < 1) { r.fparams[0] = 10.0; r.n_fparams = 1; }
    if (!(r.fparams[0] > 0.0) || r.fparams[0] > 600.0) { set_err(err, "timeout must be in (0, 600] seconds"); return PB200_ERR_BAD_SHAPE; }
    pb200_geometry& g = r.geom;
    g.grid[0] = g.grid[1] = g.grid[2] = 1;
    g.block[0] = 32; g.block[1] = g.block[2] = 1;
    g.cluster[0] = g.cluster[1] = g.cluster[2] = 1;
    g.smem_bytes = 0;
    g.n_inputs = (uint32_t)world;       // one flag block per rank, in rank order
    g.n_outputs = 0;
    return PB200_OK;
}

int launch_peer_barrier(const Record& r, cudaStream_t stream, void** p, char* err) {
    FlagBlocks f{};
    const int world = (int)r.dims[0];
    for (int i = 0; i < world; ++i) f.block[i] = (uint32_t*)p[i];
    const uint64_t timeout_ns = (uint64_t)(r.fparams[0] * 1e9);
    int* status = device_status_ptr();
    // Without the status word a timed-out wait could not be reported: refuse to launch.
    if (status == nullptr) { set_err(err, "peer barrier: the device status word is not available on this device"); return PB200_ERR_NO_CUDA; }
    peer_barrier_kernel<<<1, 32, 0, stream>>>(f, world, (int)r.dims[1], timeout_ns, status, r.kernel_id);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, "peer barrier launch failed: %s", cudaGetErrorString(e)); return PB200_ERR_LAUNCH; }
    return PB200_OK;
}

}  // namespace pb200
