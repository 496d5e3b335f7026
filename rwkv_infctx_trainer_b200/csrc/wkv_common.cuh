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

// scalar (token-serial) v5/v6 kernels, wkv56_scalar.cu
size_t scalar_backward_workspace(const wkv_args_t *a);
int scalar_forward(const wkv_args_t *a, bool per_token_w, cudaStream_t s);
int scalar_backward(const wkv_args_t *a, bool per_token_w, cudaStream_t s);

// chunked tensor-core v5/v6 kernels, wkv56_chunked.cu
bool chunked_supported(const wkv_args_t *a, bool per_token_w);
size_t chunked_forward_workspace(const wkv_args_t *a, bool per_token_w);
size_t chunked_backward_workspace(const wkv_args_t *a, bool per_token_w);

}  // namespace wkv
