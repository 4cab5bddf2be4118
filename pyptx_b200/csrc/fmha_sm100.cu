// Flash-attention forward for sm_100a (placeholder until the tcgen05 kernel lands).
#include "common.cuh"

namespace pb200 {
int plan_attention(Record&, char* err) { set_err(err, "flash attention is not built yet"); return PB200_ERR_BAD_KERNEL; }
int launch_attention(const Record&, cudaStream_t, void**, char* err) { set_err(err, "flash attention is not built yet"); return PB200_ERR_BAD_KERNEL; }
}  // namespace pb200
