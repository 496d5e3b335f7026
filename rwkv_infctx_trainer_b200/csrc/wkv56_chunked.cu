// Chunked tensor-core v5/v6 kernels (placeholder until the tcgen05 path lands).
#include "wkv_common.cuh"
namespace wkv {
bool chunked_supported(const wkv_args_t *, bool) { return false; }
size_t chunked_forward_workspace(const wkv_args_t *, bool) { return 0; }
size_t chunked_backward_workspace(const wkv_args_t *, bool) { return 0; }
int chunked_forward(const wkv_args_t *, bool, cudaStream_t) { return WKV_ERR_UNSUPPORTED; }
int chunked_backward(const wkv_args_t *, bool, cudaStream_t) { return WKV_ERR_UNSUPPORTED; }
}  // namespace wkv
