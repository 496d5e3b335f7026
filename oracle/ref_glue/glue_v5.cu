// TEST INFRASTRUCTURE ONLY.  extern "C" doorway to the RWKV-infctx-trainer
// project's own v5 launchers (RWKV-v5/src/module/cuda/wkv5_cuda.cu:348-383),
// compiled unchanged next to this file by oracle/build.py.
#include "ATen/ATen.h"
typedef at::BFloat16 bf16;
typedef float fp32;

void cuda_forward_bf16(int B, int T, int C, int H, float *state, bf16 *r, bf16 *k, bf16 *v,
                       float *w, bf16 *u, bf16 *y);
void cuda_forward_fp32(int B, int T, int C, int H, float *state, fp32 *r, fp32 *k, fp32 *v,
                       float *w, fp32 *u, fp32 *y);
void cuda_backward_bf16(int B, int T, int C, int H, float *state, bf16 *r, bf16 *k, bf16 *v,
                        float *w, float *ww, bf16 *u, bf16 *gy, bf16 *gr, bf16 *gk, bf16 *gv,
                        bf16 *gw, bf16 *gu);
void cuda_backward_fp32(int B, int T, int C, int H, float *state, fp32 *r, fp32 *k, fp32 *v,
                        float *w, float *ww, fp32 *u, fp32 *gy, fp32 *gr, fp32 *gk, fp32 *gv,
                        fp32 *gw, fp32 *gu);

extern "C" void ref_wkv5_forward(int is_bf16, int B, int T, int C, int H, float *state, void *r,
                                 void *k, void *v, float *w, void *u, void *y) {
    if (is_bf16)
        cuda_forward_bf16(B, T, C, H, state, (bf16 *)r, (bf16 *)k, (bf16 *)v, w, (bf16 *)u, (bf16 *)y);
    else
        cuda_forward_fp32(B, T, C, H, state, (fp32 *)r, (fp32 *)k, (fp32 *)v, w, (fp32 *)u, (fp32 *)y);
}

extern "C" void ref_wkv5_backward(int is_bf16, int B, int T, int C, int H, float *state, void *r,
                                  void *k, void *v, float *w, float *ww, void *u, void *gy,
                                  void *gr, void *gk, void *gv, void *gw, void *gu) {
    if (is_bf16)
        cuda_backward_bf16(B, T, C, H, state, (bf16 *)r, (bf16 *)k, (bf16 *)v, w, ww, (bf16 *)u,
                           (bf16 *)gy, (bf16 *)gr, (bf16 *)gk, (bf16 *)gv, (bf16 *)gw, (bf16 *)gu);
    else
        cuda_backward_fp32(B, T, C, H, state, (fp32 *)r, (fp32 *)k, (fp32 *)v, w, ww, (fp32 *)u,
                           (fp32 *)gy, (fp32 *)gr, (fp32 *)gk, (fp32 *)gv, (fp32 *)gw, (fp32 *)gu);
}
