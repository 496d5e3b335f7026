// Shared helpers of the WKV kernels: element-type traits and argument checks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/wkv_b200.h"

namespace wkv {

constexpr int HEAD = 64;  // head size N compiled in (RWKV-v6/src/model.py:313)

template <typename F> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float ld(const float *p) { return *p; }
    static __device__ __forceinline__ void st(float *p, float x) { *p = x; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float ld(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void st(__nv_bfloat16 *p, float x) { *p = __float2bfloat16_rn(x); }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float ld(const __half *p) { return __half2float(*p); }
    static __device__ __forceinline__ void st(__half *p, float x) { *p = __float2half_rn(x); }
};

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? WKV_OK : WKV_ERR_LAUNCH; }

// Programmatic dependent launch.  A kernel launched through launch_chained() may be scheduled
// while the kernel before it in the stream is still running, which hides its launch latency
// behind that kernel's last CTAs.  pdl_wait() returns once every earlier kernel of the stream
// has finished and its writes are visible: it is the first statement of every kernel launched
// this way, in every thread, before anything touches global memory -- and before any tensor
// memory is allocated, so that a waiting CTA never holds what a CTA of the earlier kernel still
// needs.  pdl_trigger() lets the next kernel be scheduled once every CTA of this one has called
// it or left.  Both are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline int launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...) == cudaSuccess ? WKV_OK : WKV_ERR_LAUNCH;
}

// scalar (token-serial) v5/v6 kernels, wkv56_scalar.cu
size_t scalar_backward_workspace(const wkv_args_t *a);
int scalar_forward(const wkv_args_t *a, bool per_token_w, cudaStream_t s);
int scalar_backward(const wkv_args_t *a, bool per_token_w, cudaStream_t s);

// chunked tensor-core v5/v6 kernels, wkv56_chunked.cu
bool chunked_supported(const wkv_args_t *a, bool per_token_w);
size_t chunked_forward_workspace(const wkv_args_t *a, bool per_token_w);
size_t chunked_backward_workspace(const wkv_args_t *a, bool per_token_w);

}  // namespace wkv
