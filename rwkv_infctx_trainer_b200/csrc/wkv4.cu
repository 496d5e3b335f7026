// v4 WKV (aa/bb/pp state): log-space-stabilised scan over T, forward and backward
// with the (p,q,o) state and its (gp,gq,go) gradient carried across segments.
//
// Math: RWKV-v4neo/cuda/wkv_cuda_bf16.cu:7-53 (forward), :55-158 (backward).
// Differences in execution: one of the two exponentials of every max-shifted
// pair is exp(0), so each pair costs one exp; the backward keeps no per-thread
// T-sized arrays -- a forward sweep writes the state at the start of every
// TILE tokens to the workspace and the reverse sweep recomputes one tile at a
// time into registers; T is a run-time argument.
#include "wkv_common.cuh"

namespace wkv {
namespace {

constexpr float MIN_VALUE = -1e38f;
constexpr int TILE = 16;
constexpr int THREADS = 128;

// (A,B) = (exp(a-m), exp(b-m)), m = max(a,b): one exp.
__device__ __forceinline__ void exp_pair(float a, float b, float &A, float &Bv, float &m) {
    const float d = a - b;
    const float e = __expf(-fabsf(d));
    const bool ge = d >= 0.f;
    A = ge ? 1.f : e;
    Bv = ge ? e : 1.f;
    m = ge ? a : b;
}

template <typename F>
__global__ void __launch_bounds__(THREADS)
k_v4_fwd(int B, int T, int C, const float *__restrict__ w_, const F *__restrict__ u_,
         const F *__restrict__ k_, const F *__restrict__ v_, const float *__restrict__ state_in,
         F *__restrict__ y_, float *__restrict__ state_out) {
    const int idx = blockIdx.x * THREADS + threadIdx.x;
    if (idx >= B * C) return;
    const int b = idx / C, c = idx % C;
    const float w = w_[c], u = Elem<F>::ld(u_ + c);
    const size_t off = (size_t)b * T * C + c, so = (size_t)idx * 3;
    float p = 0.f, q = 0.f, o = MIN_VALUE;
    if (state_in) { p = state_in[so]; q = state_in[so + 1]; o = state_in[so + 2]; }
    for (int t = 0; t < T; t++) {
        const float kk = Elem<F>::ld(k_ + off + (size_t)t * C);
        const float vv = Elem<F>::ld(v_ + off + (size_t)t * C);
        float A, E, m;
        exp_pair(o, u + kk, A, E, m);
        Elem<F>::st(y_ + off + (size_t)t * C, __fdividef(A * p + E * vv, A * q + E));
        exp_pair(w + o, kk, A, E, m);
        p = A * p + E * vv; q = A * q + E; o = m;
    }
    if (state_out) { state_out[so] = p; state_out[so + 1] = q; state_out[so + 2] = o; }
}

template <typename F>
__global__ void __launch_bounds__(THREADS)
k_v4_bwd(int B, int T, int C, const float *__restrict__ w_, const F *__restrict__ u_,
         const F *__restrict__ k_, const F *__restrict__ v_, const float *__restrict__ state_in,
         const F *__restrict__ gy_, const float *__restrict__ gstate_out, float *__restrict__ gw_,
         float *__restrict__ gu_, F *__restrict__ gk_, F *__restrict__ gv_,
         float *__restrict__ gstate_in, float *__restrict__ ws) {
    const int idx = blockIdx.x * THREADS + threadIdx.x;
    if (idx >= B * C) return;
    const int b = idx / C, c = idx % C;
    const float w = w_[c], u = Elem<F>::ld(u_ + c);
    const size_t off = (size_t)b * T * C + c, so = (size_t)idx * 3;
    const int ntile = (T + TILE - 1) / TILE;
    // workspace [B][ntile][3][C]
    float *ck = ws + (size_t)b * ntile * 3 * C + c;
    float p = 0.f, q = 0.f, o = MIN_VALUE;
    if (state_in) { p = state_in[so]; q = state_in[so + 1]; o = state_in[so + 2]; }
    float gw = 0.f, gu = 0.f, dpdw = 0.f, dqdw = 0.f;
    for (int t = 0; t < T; t++) {
        if (t % TILE == 0) {
            float *c3 = ck + (size_t)(t / TILE) * 3 * C;
            c3[0] = p; c3[C] = q; c3[2 * C] = o;
        }
        const float kk = Elem<F>::ld(k_ + off + (size_t)t * C);
        const float vv = Elem<F>::ld(v_ + off + (size_t)t * C);
        const float g = Elem<F>::ld(gy_ + off + (size_t)t * C);
        float A, E, m;
        exp_pair(o, u + kk, A, E, m);
        const float iden = __fdividef(1.f, A * q + E);
        const float y = (A * p + E * vv) * iden;
        gw += g * (dpdw - dqdw * y) * iden * A;
        gu += g * (vv - y) * E * iden;
        exp_pair(w + o, kk, A, E, m);
        dpdw = A * (p + dpdw); dqdw = A * (q + dqdw);
        p = A * p + E * vv; q = A * q + E; o = m;
    }
    float gp = 0.f, gq = 0.f, go = MIN_VALUE;
    if (gstate_out) {
        gp = gstate_out[so]; gq = gstate_out[so + 1]; go = gstate_out[so + 2];
        if (gp == 0.f && gq == 0.f) go = MIN_VALUE;
        gw += (gp * dpdw + gq * dqdw) * __expf(o + go);
    }
    for (int tile = ntile - 1; tile >= 0; tile--) {
        const int t0 = tile * TILE;
        const float *c3 = ck + (size_t)tile * 3 * C;
        p = c3[0]; q = c3[C]; o = c3[2 * C];
        float ys[TILE], zs[TILE], ze[TILE];
#pragma unroll
        for (int j = 0; j < TILE; j++) {
            if (t0 + j < T) {
                const float kk = Elem<F>::ld(k_ + off + (size_t)(t0 + j) * C);
                const float vv = Elem<F>::ld(v_ + off + (size_t)(t0 + j) * C);
                float A, E, m;
                exp_pair(o, u + kk, A, E, m);
                const float iden = __fdividef(1.f, A * q + E);
                ys[j] = (A * p + E * vv) * iden; zs[j] = iden; ze[j] = kk + u - m;
                exp_pair(w + o, kk, A, E, m);
                p = A * p + E * vv; q = A * q + E; o = m;
            }
        }
#pragma unroll
        for (int j = TILE - 1; j >= 0; j--) {
            if (t0 + j < T) {
                const size_t ii = off + (size_t)(t0 + j) * C;
                const float kk = Elem<F>::ld(k_ + ii), vv = Elem<F>::ld(v_ + ii);
                const float g = Elem<F>::ld(gy_ + ii);
                const float gz = g * zs[j];
                float A = gz * __expf(ze[j]);
                float E = __expf(kk + go);
                Elem<F>::st(gk_ + ii, A * (vv - ys[j]) + E * (gp * vv + gq));
                Elem<F>::st(gv_ + ii, A + E * gp);
                float m;
                exp_pair(w + go, ze[j] - kk - u, A, E, m);
                E *= gz;
                gp = A * gp + E; gq = A * gq - E * ys[j]; go = m;
            }
        }
    }
    if (gstate_in) { gstate_in[so] = gp; gstate_in[so + 1] = gq; gstate_in[so + 2] = go; }
    gw_[idx] = gw * w;
    gu_[idx] = gu;
}

template <typename F>
int fwd(int B, int T, int C, const float *w, const void *u, const void *k, const void *v,
        const float *si, void *y, float *so, cudaStream_t s) {
    const int n = B * C;
    k_v4_fwd<F><<<(n + THREADS - 1) / THREADS, THREADS, 0, s>>>(
        B, T, C, w, (const F *)u, (const F *)k, (const F *)v, si, (F *)y, so);
    return launch_status();
}

template <typename F>
int bwd(int B, int T, int C, const float *w, const void *u, const void *k, const void *v,
        const float *si, const void *gy, const float *gso, float *gw, float *gu, void *gk,
        void *gv, float *gsi, float *ws, cudaStream_t s) {
    const int n = B * C;
    k_v4_bwd<F><<<(n + THREADS - 1) / THREADS, THREADS, 0, s>>>(
        B, T, C, w, (const F *)u, (const F *)k, (const F *)v, si, (const F *)gy, gso, gw, gu,
        (F *)gk, (F *)gv, gsi, ws);
    return launch_status();
}

// segments shorter than this run on the one-thread-per-chain kernels above
constexpr int PAR_MIN_T = 128;

size_t serial_backward_workspace(int B, int T, int C) {
    if (B <= 0 || T <= 0 || C <= 0) return 0;
    const size_t ntile = (size_t)(T + TILE - 1) / TILE;
    return (size_t)B * ntile * 3 * C * sizeof(float);
}

}  // namespace

// time-parallel kernels, wkv4_par.cu
size_t v4_par_forward_workspace(int B, int T, int C);
size_t v4_par_backward_workspace(int B, int T, int C);
size_t v4_par_ckpt_bytes(int B, int T, int C);
int v4_par_forward(int B, int T, int C, int dtype, const float *w, const void *u, const void *k, const void *v,
                   const float *si, void *y, float *so, float *ws, float *ckpt, cudaStream_t s);
int v4_par_backward(int B, int T, int C, int dtype, const float *w, const void *u, const void *k, const void *v,
                    const float *si, const void *gy, const float *gso, float *gw, float *gu, void *gk, void *gv,
                    float *gsi, float *ws, const float *ckpt, cudaStream_t s);
}  // namespace wkv

using namespace wkv;

extern "C" size_t wkv4_forward_workspace(int B, int T, int C) {
    if (B <= 0 || C <= 0 || T < PAR_MIN_T) return 0;
    return v4_par_forward_workspace(B, T, C);
}

extern "C" size_t wkv4_state_ckpt_bytes(int B, int T, int C) {
    if (B <= 0 || C <= 0 || T < PAR_MIN_T) return 0;
    return v4_par_ckpt_bytes(B, T, C);
}

extern "C" int wkv4_forward(int B, int T, int C, int dtype, const float *w, const void *u,
                            const void *k, const void *v, const float *state_in, void *y,
                            float *state_out, void *workspace, size_t workspace_bytes, void *stream) {
    return wkv4_forward_ckpt(B, T, C, dtype, w, u, k, v, state_in, y, state_out, workspace, workspace_bytes,
                             nullptr, 0, stream);
}

extern "C" int wkv4_forward_ckpt(int B, int T, int C, int dtype, const float *w, const void *u,
                                 const void *k, const void *v, const float *state_in, void *y,
                                 float *state_out, void *workspace, size_t workspace_bytes,
                                 void *state_ckpt, size_t state_ckpt_bytes, void *stream) {
    if (B < 0 || T < 0 || C < 0) return WKV_ERR_SHAPE;
    if (B == 0 || C == 0) return WKV_OK;
    if (!w || !u) return WKV_ERR_NULL;
    if (T > 0 && (!k || !v || !y)) return WKV_ERR_NULL;
    if (dtype != WKV_F32 && dtype != WKV_BF16 && dtype != WKV_F16) return WKV_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    if (T >= PAR_MIN_T) {
        if (!workspace || workspace_bytes < wkv4_forward_workspace(B, T, C)) return WKV_ERR_WORKSPACE;
        if (state_ckpt && state_ckpt_bytes < wkv4_state_ckpt_bytes(B, T, C)) return WKV_ERR_WORKSPACE;
        return v4_par_forward(B, T, C, dtype, w, u, k, v, state_in, y, state_out, (float *)workspace,
                              (float *)state_ckpt, s);
    }
    switch (dtype) {
        case WKV_F32: return fwd<float>(B, T, C, w, u, k, v, state_in, y, state_out, s);
        case WKV_BF16: return fwd<__nv_bfloat16>(B, T, C, w, u, k, v, state_in, y, state_out, s);
        case WKV_F16: return fwd<__half>(B, T, C, w, u, k, v, state_in, y, state_out, s);
    }
    return WKV_ERR_DTYPE;
}

extern "C" size_t wkv4_backward_workspace(int B, int T, int C) {
    if (B <= 0 || T <= 0 || C <= 0) return 0;
    const size_t a = serial_backward_workspace(B, T, C);
    const size_t b = T >= PAR_MIN_T ? v4_par_backward_workspace(B, T, C) : 0;
    return a > b ? a : b;
}

extern "C" int wkv4_backward(int B, int T, int C, int dtype, const float *w, const void *u,
                             const void *k, const void *v, const float *state_in, const void *gy,
                             const float *gstate_out, float *gw, float *gu, void *gk, void *gv,
                             float *gstate_in, void *workspace, size_t workspace_bytes,
                             void *stream) {
    return wkv4_backward_ckpt(B, T, C, dtype, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in,
                              workspace, workspace_bytes, nullptr, 0, stream);
}

extern "C" int wkv4_backward_ckpt(int B, int T, int C, int dtype, const float *w, const void *u,
                                  const void *k, const void *v, const float *state_in, const void *gy,
                                  const float *gstate_out, float *gw, float *gu, void *gk, void *gv,
                                  float *gstate_in, void *workspace, size_t workspace_bytes,
                                  const void *state_ckpt, size_t state_ckpt_bytes, void *stream) {
    if (B < 0 || T < 0 || C < 0) return WKV_ERR_SHAPE;
    if (B == 0 || C == 0) return WKV_OK;
    if (!w || !u || !gw || !gu) return WKV_ERR_NULL;
    if (T > 0 && (!k || !v || !gy || !gk || !gv)) return WKV_ERR_NULL;
    const size_t need = wkv4_backward_workspace(B, T, C);
    if (need && (!workspace || workspace_bytes < need)) return WKV_ERR_WORKSPACE;
    if (dtype != WKV_F32 && dtype != WKV_BF16 && dtype != WKV_F16) return WKV_ERR_DTYPE;
    cudaStream_t s = (cudaStream_t)stream;
    float *ws = (float *)workspace;
    if (T >= PAR_MIN_T) {
        if (state_ckpt && state_ckpt_bytes < wkv4_state_ckpt_bytes(B, T, C)) return WKV_ERR_WORKSPACE;
        return v4_par_backward(B, T, C, dtype, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws,
                               (const float *)state_ckpt, s);
    }
    switch (dtype) {
        case WKV_F32:
            return bwd<float>(B, T, C, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws, s);
        case WKV_BF16:
            return bwd<__nv_bfloat16>(B, T, C, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws, s);
        case WKV_F16:
            return bwd<__half>(B, T, C, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws, s);
    }
    return WKV_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Backward without a caller-provided workspace.
//
// Some hosts of this library cannot hand it scratch memory: a foreign-language
// binding that was given its tensors by another framework and owns no device
// allocator, or a training loop whose device memory is planned up front and
// which must not call cudaMalloc in the middle of a step (cudaMalloc also
// synchronises the device).  For them the tile-start states that
// wkv4_backward keeps in its workspace live here, in a fixed array inside the
// library image.  Every GPU that loads the library holds these bytes until the
// process exits.
namespace {

constexpr size_t kStaticScratchBytes = (size_t)32 << 20;  // 32 MiB
static __device__ __align__(256) unsigned char g_v4_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void *g_scratch_addr[kMaxDevices];  // device address of the array, per device ordinal
bool g_scratch_known[kMaxDevices];

// In host code `g_v4_static_scratch` names a host-side shadow, not device
// memory; the device address has to be asked for, on the device in question.
// The answer is remembered per device ordinal.  It belongs to the device's
// primary context (the one the runtime API uses): after cudaDeviceReset, or with
// another context made current through the driver API, it is no longer valid --
// this entry point is for processes that do neither.
int static_scratch_address(void **out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return WKV_ERR_LAUNCH;
    if (!__atomic_load_n(&g_scratch_known[dev], __ATOMIC_ACQUIRE)) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_v4_static_scratch) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return WKV_ERR_LAUNCH;
        }
        g_scratch_addr[dev] = p;
        __atomic_store_n(&g_scratch_known[dev], true, __ATOMIC_RELEASE);
    }
    *out = g_scratch_addr[dev];
    return WKV_OK;
}

}  // namespace

extern "C" size_t wkv4_backward_static_limit(void) { return kStaticScratchBytes; }

extern "C" int wkv4_backward_static(int B, int T, int C, int dtype, const float *w, const void *u,
                                    const void *k, const void *v, const float *state_in,
                                    const void *gy, const float *gstate_out, float *gw, float *gu,
                                    void *gk, void *gv, float *gstate_in, void *stream) {
    if (B < 0 || T < 0 || C < 0) return WKV_ERR_SHAPE;
    if (B == 0 || C == 0) return WKV_OK;
    if (!w || !u || !gw || !gu) return WKV_ERR_NULL;
    if (T > 0 && (!k || !v || !gy || !gk || !gv)) return WKV_ERR_NULL;
    if (dtype != WKV_F32 && dtype != WKV_BF16 && dtype != WKV_F16) return WKV_ERR_DTYPE;
    if (wkv4_backward_workspace(B, T, C) > kStaticScratchBytes) return WKV_ERR_TOO_LARGE;
    void *scratch = nullptr;
    const int err = static_scratch_address(&scratch);
    if (err != WKV_OK) return err;
    cudaStream_t s = (cudaStream_t)stream;
    float *ws = (float *)scratch;
    // Nothing in the scratch has to start at zero: both kernel families write every word of it
    // that they later read (tile-start states; piece summaries, scanned states and partial sums).
    if (T >= PAR_MIN_T)   // the same time-parallel kernels wkv4_backward runs, on the built-in array
        return v4_par_backward(B, T, C, dtype, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws,
                               nullptr, s);
    switch (dtype) {
        case WKV_F32:
            return bwd<float>(B, T, C, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws, s);
        case WKV_BF16:
            return bwd<__nv_bfloat16>(B, T, C, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws, s);
        default:
            return bwd<__half>(B, T, C, w, u, k, v, state_in, gy, gstate_out, gw, gu, gk, gv, gstate_in, ws, s);
    }
}
