#include "kdnn_common.cuh"
namespace kdnn {
cudaError_t moe_route_launch(const void*, size_t, size_t, size_t, int, const void*, int, int, float, int, int32_t*, float*, cudaStream_t) { return cudaErrorNotSupported; }
size_t moe_workspace_bytes(size_t, size_t, size_t, size_t, size_t) { return 256; }
cudaError_t moe_ffn_launch(const void*, size_t, size_t, int, const kdnn_b200_weight_table*, const kdnn_b200_weight_table*, const kdnn_b200_weight_table*, const int32_t*, const float*, size_t, void*, size_t, int, size_t, size_t, void*, cudaStream_t) { return cudaErrorNotSupported; }
int moe_take_status() { return 0; }
}
