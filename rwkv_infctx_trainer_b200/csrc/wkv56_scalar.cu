// Token-serial fp32 kernels for the v5/v6 WKV recurrence (any element type,
// any T): the exact path behind the fp32 entry points and the fallback for
// shapes the tensor-core kernels do not take.
//
// One CTA per (batch, head).  Forward: thread j owns state column S[:,j] in
// registers.  Backward: one forward sweep (threads 0..63 own state rows) emits
// gr and stashes q_t[k] = r_t[k] * sum_v S_t[k,v] gy_t[v]; one reverse sweep
// carries D = dL/dS both row-owned (threads 0..63: gk, gw) and column-owned
// (threads 64..127: gv).  The decay gradient uses
//   E_t = sum_v S_t[k,v] D_t[k,v],  E_t = E_{t+1} + q_t - p_t,
//   dL/d(log w_t) = E_{t+1} - p_t,  p_t[k] = k_t[k] * sum_v D_{t+1}[k,v] v_t[v],
// which needs only per-token scalars from the forward sweep (the fp32 [B,T,C]
// workspace) instead of every intermediate state.
//
// Same math as RWKV-v5/src/module/cuda/wkv5_cuda.cu:129-340 and
// RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu:6-293, plus what those lack:
// per-batch state, state_out, gstate_out -> gstate_in.
#include "wkv_common.cuh"

namespace wkv {
namespace {

constexpr int N = HEAD;

// log-decay (<= 0) of channel c at token t from either encoding
template <typename F, bool PER_TOKEN>
__device__ __forceinline__ float load_logw(const void *w, int w_kind, size_t tok_off, int c) {
    if (PER_TOKEN) {
        if (w_kind == WKV_W_RAW) return -expf(Elem<F>::ld((const F *)w + tok_off + c));
        return ((const float *)w)[tok_off + c];
    } else {
        const float x = ((const float *)w)[c];
        return w_kind == WKV_W_RAW ? -expf(x) : x;
    }
}

__device__ __forceinline__ size_t state_idx(int layout, int key, int val) {
    return layout == WKV_STATE_KV ? (size_t)key * N + val : (size_t)val * N + key;
}

template <typename F, bool PER_TOKEN>
__global__ void __launch_bounds__(N)
k_scalar_fwd(int T, int H, int w_kind, int layout, const F *__restrict__ r,
             const F *__restrict__ k, const F *__restrict__ v, const void *__restrict__ w,
             const F *__restrict__ u, const float *state_in, F *__restrict__ y,
             float *state_out) {
    const int bh = blockIdx.x, b = bh / H, h = bh % H, j = threadIdx.x, C = H * N;
    __shared__ float sr[N], sk[N], sw[N], su[N];
    float S[N];
    const size_t sbase = (size_t)bh * N * N;
#pragma unroll
    for (int i = 0; i < N; i++) S[i] = state_in ? state_in[sbase + state_idx(layout, i, j)] : 0.f;
    su[j] = Elem<F>::ld(u + h * N + j);
    if (!PER_TOKEN) sw[j] = expf(load_logw<F, false>(w, w_kind, 0, h * N + j));
    for (int t = 0; t < T; t++) {
        const size_t o = ((size_t)b * T + t) * C + (size_t)h * N;
        __syncthreads();
        sr[j] = Elem<F>::ld(r + o + j);
        sk[j] = Elem<F>::ld(k + o + j);
        if (PER_TOKEN) sw[j] = expf(load_logw<F, true>(w, w_kind, o, j));
        const float vj = Elem<F>::ld(v + o + j);
        __syncthreads();
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < N; i++) {
            const float kv = sk[i] * vj;
            acc += sr[i] * (su[i] * kv + S[i]);
            S[i] = sw[i] * S[i] + kv;
        }
        Elem<F>::st(y + o + j, acc);
    }
    if (state_out) {
#pragma unroll
        for (int i = 0; i < N; i++) state_out[sbase + state_idx(layout, i, j)] = S[i];
    }
}

template <typename F, bool PER_TOKEN>
__global__ void __launch_bounds__(2 * N)
k_scalar_bwd(int T, int H, int w_kind, int layout, const F *__restrict__ r,
             const F *__restrict__ k, const F *__restrict__ v, const void *__restrict__ w,
             const F *__restrict__ u, const float *__restrict__ state_in,
             const F *__restrict__ gy, const float *__restrict__ gstate_out,
             F *__restrict__ gr, F *__restrict__ gk, F *__restrict__ gv, void *gw_out,
             float *__restrict__ gu, float *gstate_in, float *__restrict__ q_ws) {
    const int bh = blockIdx.x, b = bh / H, h = bh % H, tid = threadIdx.x, C = H * N;
    const int i = tid & (N - 1);
    const bool row_owner = tid < N;
    __shared__ float sr[N], sk[N], sv[N], sg[N], sw[N], slw[N], su[N];
    float M[N];  // S row (forward sweep), then D row or D column (reverse sweep)
    const size_t sbase = (size_t)bh * N * N;
    if (row_owner) {
        su[i] = Elem<F>::ld(u + h * N + i);
        if (!PER_TOKEN) {
            slw[i] = load_logw<F, false>(w, w_kind, 0, h * N + i);
            sw[i] = expf(slw[i]);
        }
#pragma unroll
        for (int j = 0; j < N; j++) M[j] = state_in ? state_in[sbase + state_idx(layout, i, j)] : 0.f;
    }
    float gu_acc = 0.f;
    // ---- forward sweep: gr, gu, q_t
    for (int t = 0; t < T; t++) {
        const size_t o = ((size_t)b * T + t) * C + (size_t)h * N;
        __syncthreads();
        if (row_owner) {
            sk[i] = Elem<F>::ld(k + o + i);
            sv[i] = Elem<F>::ld(v + o + i);
            if (PER_TOKEN) sw[i] = expf(load_logw<F, true>(w, w_kind, o, i));
        } else {
            sg[i] = Elem<F>::ld(gy + o + i);
        }
        __syncthreads();
        if (row_owner) {
            const float ri = Elem<F>::ld(r + o + i);
            float vg = 0.f, sgy = 0.f;
#pragma unroll
            for (int j = 0; j < N; j++) {
                vg += sv[j] * sg[j];
                sgy += M[j] * sg[j];
                M[j] = sw[i] * M[j] + sk[i] * sv[j];
            }
            Elem<F>::st(gr + o + i, su[i] * sk[i] * vg + sgy);
            q_ws[o + i] = ri * sgy;
            gu_acc += ri * sk[i] * vg;
        }
    }
    // ---- junction: E_T = sum_v S_T[k,v] D_T[k,v]; load D_T (row- and column-owned)
    float E = 0.f;
    if (row_owner) {
#pragma unroll
        for (int j = 0; j < N; j++) {
            const float d = gstate_out ? gstate_out[sbase + state_idx(layout, i, j)] : 0.f;
            E += M[j] * d;
            M[j] = d;
        }
        gu[(size_t)b * C + h * N + i] = gu_acc;
    } else {
#pragma unroll
        for (int j = 0; j < N; j++) M[j] = gstate_out ? gstate_out[sbase + state_idx(layout, j, i)] : 0.f;
    }
    float gw_acc = 0.f;
    // ---- reverse sweep: gk, gv, gw, D
    for (int t = T - 1; t >= 0; t--) {
        const size_t o = ((size_t)b * T + t) * C + (size_t)h * N;
        __syncthreads();
        if (row_owner) {
            sr[i] = Elem<F>::ld(r + o + i);
            sk[i] = Elem<F>::ld(k + o + i);
            if (PER_TOKEN) {
                slw[i] = load_logw<F, true>(w, w_kind, o, i);
                sw[i] = expf(slw[i]);
            }
        } else {
            sv[i] = Elem<F>::ld(v + o + i);
            sg[i] = Elem<F>::ld(gy + o + i);
        }
        __syncthreads();
        if (row_owner) {  // thread owns D[i, :]
            float vg = 0.f, dv = 0.f;
#pragma unroll
            for (int j = 0; j < N; j++) {
                vg += sv[j] * sg[j];
                dv += M[j] * sv[j];
                M[j] = sr[i] * sg[j] + sw[i] * M[j];
            }
            Elem<F>::st(gk + o + i, su[i] * sr[i] * vg + dv);
            const float p = sk[i] * dv;
            const float g = (E - p) * slw[i];  // d/dx with log w = -exp(x)
            E += q_ws[o + i] - p;
            if (PER_TOKEN) Elem<F>::st((F *)gw_out + o + i, g);
            else gw_acc += g;
        } else {  // thread owns D[:, i]
            float acc = 0.f, urk = 0.f;
#pragma unroll
            for (int j = 0; j < N; j++) {
                urk += su[j] * sr[j] * sk[j];
                acc += M[j] * sk[j];
                M[j] = sr[j] * sg[i] + sw[j] * M[j];
            }
            Elem<F>::st(gv + o + i, acc + urk * sg[i]);
        }
    }
    if (row_owner) {
        if (!PER_TOKEN) ((float *)gw_out)[(size_t)b * C + h * N + i] = gw_acc;
        if (gstate_in) {
#pragma unroll
            for (int j = 0; j < N; j++) gstate_in[sbase + state_idx(layout, i, j)] = M[j];
        }
    }
}

template <typename F, bool PT>
int launch_fwd(const wkv_args_t *a, cudaStream_t s) {
    k_scalar_fwd<F, PT><<<a->B * a->H, N, 0, s>>>(
        a->T, a->H, a->w_kind, a->state_layout, (const F *)a->r, (const F *)a->k, (const F *)a->v,
        a->w, (const F *)a->u, a->state_in, (F *)a->y, a->state_out);
    return launch_status();
}

template <typename F, bool PT>
int launch_bwd(const wkv_args_t *a, cudaStream_t s) {
    k_scalar_bwd<F, PT><<<a->B * a->H, 2 * N, 0, s>>>(
        a->T, a->H, a->w_kind, a->state_layout, (const F *)a->r, (const F *)a->k, (const F *)a->v,
        a->w, (const F *)a->u, a->state_in, (const F *)a->gy, a->gstate_out, (F *)a->gr,
        (F *)a->gk, (F *)a->gv, a->gw, a->gu, a->gstate_in, (float *)a->workspace);
    return launch_status();
}

}  // namespace

size_t scalar_backward_workspace(const wkv_args_t *a) {
    return (size_t)a->B * a->T * a->H * a->N * sizeof(float);
}

int scalar_forward(const wkv_args_t *a, bool pt, cudaStream_t s) {
    switch (a->dtype) {
        case WKV_F32: return pt ? launch_fwd<float, true>(a, s) : launch_fwd<float, false>(a, s);
        case WKV_BF16: return pt ? launch_fwd<__nv_bfloat16, true>(a, s) : launch_fwd<__nv_bfloat16, false>(a, s);
        case WKV_F16: return pt ? launch_fwd<__half, true>(a, s) : launch_fwd<__half, false>(a, s);
    }
    return WKV_ERR_DTYPE;
}

int scalar_backward(const wkv_args_t *a, bool pt, cudaStream_t s) {
    switch (a->dtype) {
        case WKV_F32: return pt ? launch_bwd<float, true>(a, s) : launch_bwd<float, false>(a, s);
        case WKV_BF16: return pt ? launch_bwd<__nv_bfloat16, true>(a, s) : launch_bwd<__nv_bfloat16, false>(a, s);
        case WKV_F16: return pt ? launch_bwd<__half, true>(a, s) : launch_bwd<__half, false>(a, s);
    }
    return WKV_ERR_DTYPE;
}

}  // namespace wkv
