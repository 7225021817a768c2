// Grouped expert GEMM on the tensor cores (placeholder until the tcgen05 kernel lands: the fp32-FMA kernel serves).
#include "common.cuh"
namespace pg {
bool moe_gemm_tc_supported(int, int, const int32_t*, int, int, int) { return false; }
int moe_gemm_tc(void*, int, const void*, int, const int32_t*, const void*, const int32_t*, int, int, int, int, int, int,
                cudaStream_t) { set_error("moe_gemm_tc: not built"); return PG_ERR_INVALID; }
}  // namespace pg
