// TEST INFRASTRUCTURE ONLY.  extern "C" doorway to the RWKV-infctx-trainer
// project's own v6 state launchers
// (RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu:295-308), compiled unchanged
// next to this file by oracle/build.py.  Valid for B == 1 only: those kernels
// index the state without the batch row.
#include "ATen/ATen.h"
typedef at::BFloat16 bf16;

void cuda_forward(int B, int T, int C, int H, bf16 *r, bf16 *k, bf16 *v, float *w, bf16 *u,
                  bf16 *z, bf16 *y);
void cuda_backward(int B, int T, int C, int H, bf16 *r, bf16 *k, bf16 *v, float *w, bf16 *u,
                   bf16 *z, bf16 *gy, bf16 *gr, bf16 *gk, bf16 *gv, bf16 *gw, bf16 *gu, bf16 *gz);

extern "C" void ref_wkv6_forward(int B, int T, int C, int H, void *r, void *k, void *v, float *w,
                                 void *u, void *s, void *y) {
    cuda_forward(B, T, C, H, (bf16 *)r, (bf16 *)k, (bf16 *)v, w, (bf16 *)u, (bf16 *)s, (bf16 *)y);
}

extern "C" void ref_wkv6_backward(int B, int T, int C, int H, void *r, void *k, void *v, float *w,
                                  void *u, void *s, void *gy, void *gr, void *gk, void *gv,
                                  void *gw, void *gu, void *gs) {
    cuda_backward(B, T, C, H, (bf16 *)r, (bf16 *)k, (bf16 *)v, w, (bf16 *)u, (bf16 *)s,
                  (bf16 *)gy, (bf16 *)gr, (bf16 *)gk, (bf16 *)gv, (bf16 *)gw, (bf16 *)gu,
                  (bf16 *)gs);
}
