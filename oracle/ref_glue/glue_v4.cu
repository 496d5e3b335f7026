// TEST INFRASTRUCTURE ONLY.  extern "C" doorway to the RWKV-infctx-trainer
// project's own v4 launchers (RWKV-v4neo/cuda/wkv_cuda_bf16.cu:160-172), which
// are compiled unchanged next to this file by oracle/build.py.  Declarations
// below restate those launchers' signatures; nothing else is taken from them.
#include "ATen/ATen.h"
typedef at::BFloat16 bf16;

void cuda_forward(int B, int T, int C, float *w, bf16 *u, bf16 *k, bf16 *v, float *last_state,
                  bf16 *y, float *new_state);
void cuda_backward(int B, int T, int C, float *w, bf16 *u, bf16 *k, bf16 *v, float *last_state,
                   bf16 *gy, float *gnew_state, bf16 *gw, bf16 *gu, bf16 *gk, bf16 *gv,
                   float *glast_state);

extern "C" void ref_wkv4_forward(int B, int T, int C, float *w, void *u, void *k, void *v,
                                 float *last_state, void *y, float *new_state) {
    cuda_forward(B, T, C, w, (bf16 *)u, (bf16 *)k, (bf16 *)v, last_state, (bf16 *)y, new_state);
}

extern "C" void ref_wkv4_backward(int B, int T, int C, float *w, void *u, void *k, void *v,
                                  float *last_state, void *gy, float *gnew_state, void *gw,
                                  void *gu, void *gk, void *gv, float *glast_state) {
    cuda_backward(B, T, C, w, (bf16 *)u, (bf16 *)k, (bf16 *)v, last_state, (bf16 *)gy, gnew_state,
                  (bf16 *)gw, (bf16 *)gu, (bf16 *)gk, (bf16 *)gv, glast_state);
}
