// Elementwise neighbours of the WKV op in the v5/v6 time-mix block, fused so that every
// [B,T,C] tensor crosses HBM once per pass:
//
//   lnx_gate   out = GroupNorm_heads(y) * g      (RWKV-v6/src/module/TimeMix.py:296-298,
//              RWKV-v5/src/module/TimeMix.py:318-320: x = ln_x(x.view(-1,C)).view(B,T,C); x = x * g)
//              GroupNorm with one group per head: per token and head, the 64 channels are
//              normalised (biased variance, eps), then scaled and shifted per channel.
//   ddlerp     the five data-dependent token-shift mixes of v6
//              (RWKV-v6/src/module/TimeMix.py:262-273):  x_i = x + (x_prev - x) * (maa_i + m_i)
//
// All are HBM-bound: a thread owns 8 consecutive channels (one 16-byte access per tensor), the 8
// lanes that share a head exchange their sums by shuffles, accumulation is fp32, parameter
// gradients are reduced in a fixed order (per-CTA partials, then one fold): no atomics.
#include "wkv_common.cuh"

namespace wkv {
namespace {

constexpr int TPB = 256;

__device__ __forceinline__ void unpack8(const uint4 &q, float *f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint4 pack8(const float *f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
// sum over the 8 lanes that hold one head's 64 channels
__device__ __forceinline__ float head_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}
__device__ __forceinline__ void load8f(const float *p, float *f) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Work split shared by the kernels: the C channels are cut into column blocks of 256 (a warp's
// 32 lanes x 8 channels = 4 heads); blockIdx.x = column block + ncb * token slot; the 8 warps of
// a CTA take tokens slot*8 + warp, slot*8 + warp + stride, ...  A thread therefore always owns the
// same 8 channels, which keeps its parameters and its parameter-gradient sums in registers.
struct Split {
    int ncb, nslot;
};

__global__ void __launch_bounds__(TPB)
k_lnx_gate_fwd(int tokens, int C, Split sp, const uint4 *__restrict__ y, const uint4 *__restrict__ g,
               const float *__restrict__ gamma, const float *__restrict__ beta, float eps, uint4 *__restrict__ out) {
    const int cb = blockIdx.x % sp.ncb, slot = blockIdx.x / sp.ncb, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = cb * 256 + lane * 8;
    // (lanes past the last channel stay in the loop with zeros: the shuffles below name all 32 lanes)
    const bool live = c0 < C;
    float ga[8], be[8];
#pragma unroll
    for (int q = 0; q < 8; q++) { ga[q] = 0.f; be[q] = 0.f; }
    if (live) {
        load8f(gamma + c0, ga);
        load8f(beta + c0, be);
    }
    const int stride = sp.nslot * 8, row16 = C / 8;
    for (int t = slot * 8 + warp; t < tokens; t += stride) {
        const size_t i = (size_t)t * row16 + (c0 >> 3);
        float yv[8], gv[8];
        const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
        unpack8(live ? y[i] : zero4, yv);
        unpack8(live ? g[i] : zero4, gv);
        float s = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) s += yv[q];
        const float mean = head_sum(s) * (1.f / 64.f);
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < 8; q++) { yv[q] -= mean; v += yv[q] * yv[q]; }
        const float rstd = rsqrtf(head_sum(v) * (1.f / 64.f) + eps);
        float o[8];
#pragma unroll
        for (int q = 0; q < 8; q++) o[q] = (yv[q] * rstd * ga[q] + be[q]) * gv[q];
        if (live) out[i] = pack8(o);
    }
}

// gy, gg and per-CTA partial sums of the gradients of gamma and beta ([nslot, 2, C])
__global__ void __launch_bounds__(TPB)
k_lnx_gate_bwd(int tokens, int C, Split sp, const uint4 *__restrict__ y, const uint4 *__restrict__ g,
               const float *__restrict__ gamma, const float *__restrict__ beta, float eps,
               const uint4 *__restrict__ gout, uint4 *__restrict__ gy, uint4 *__restrict__ gg,
               float *__restrict__ part) {
    __shared__ float red[8][2][256];
    const int cb = blockIdx.x % sp.ncb, slot = blockIdx.x / sp.ncb, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = cb * 256 + lane * 8;
    const bool live = c0 < C;
    float ga[8], be[8], dga[8], dbe[8];
#pragma unroll
    for (int q = 0; q < 8; q++) { dga[q] = 0.f; dbe[q] = 0.f; ga[q] = 0.f; be[q] = 0.f; }
    {
        // (every lane runs the loop, lanes past the last channel on zeros: the shuffles name all 32 lanes)
        if (live) {
            load8f(gamma + c0, ga);
            load8f(beta + c0, be);
        }
        const int stride = sp.nslot * 8, row16 = C / 8;
        for (int t = slot * 8 + warp; t < tokens; t += stride) {
            const size_t i = (size_t)t * row16 + (c0 >> 3);
            float yv[8], gv[8], go[8];
            const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
            unpack8(live ? y[i] : zero4, yv);
            unpack8(live ? g[i] : zero4, gv);
            unpack8(live ? gout[i] : zero4, go);
            float s = 0.f;
#pragma unroll
            for (int q = 0; q < 8; q++) s += yv[q];
            const float mean = head_sum(s) * (1.f / 64.f);
            float v = 0.f;
#pragma unroll
            for (int q = 0; q < 8; q++) { yv[q] -= mean; v += yv[q] * yv[q]; }
            const float rstd = rsqrtf(head_sum(v) * (1.f / 64.f) + eps);
            float dg[8], dy[8], s1 = 0.f, s2 = 0.f;
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float xh = yv[q] * rstd;               // normalised value
                const float dln = go[q] * gv[q];             // gradient at the GroupNorm output
                dg[q] = go[q] * (xh * ga[q] + be[q]);
                dga[q] += dln * xh;
                dbe[q] += dln;
                dy[q] = dln * ga[q];                         // gradient at the normalised value
                s1 += dy[q];
                s2 += dy[q] * xh;
                yv[q] = xh;
            }
            const float m1 = head_sum(s1) * (1.f / 64.f), m2 = head_sum(s2) * (1.f / 64.f);
#pragma unroll
            for (int q = 0; q < 8; q++) dy[q] = rstd * (dy[q] - m1 - yv[q] * m2);
            if (live) {
                gy[i] = pack8(dy);
                gg[i] = pack8(dg);
            }
        }
    }
    // the CTA's 8 warps hold partial sums for the same 256 channels: fold them in warp order
#pragma unroll
    for (int q = 0; q < 8; q++) { red[warp][0][lane * 8 + q] = dga[q]; red[warp][1][lane * 8 + q] = dbe[q]; }
    __syncthreads();
    const int c = cb * 256 + threadIdx.x;
    if (c < C) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) { a += red[w][0][threadIdx.x]; b += red[w][1][threadIdx.x]; }
        part[((size_t)slot * 2) * C + c] = a;
        part[((size_t)slot * 2 + 1) * C + c] = b;
    }
}

__global__ void __launch_bounds__(TPB)
k_fold_params(const float *__restrict__ part, int nslot, int C, float *__restrict__ ggamma, float *__restrict__ gbeta) {
    const int c = blockIdx.x * TPB + threadIdx.x;
    if (c >= C) return;
    float a = 0.f, b = 0.f;
    for (int s = 0; s < nslot; s++) { a += part[((size_t)s * 2) * C + c]; b += part[((size_t)s * 2 + 1) * C + c]; }
    ggamma[c] = a;
    gbeta[c] = b;
}

// x_i = x + (x_prev - x) * (maa_i + m_i) for n mixes; x_prev of a row's first token is `shift` (the
// last token of the previous segment).  m: [n, tokens, C] (NULL: no data-dependent part).
template <int NMIX>
__global__ void __launch_bounds__(TPB)
k_ddlerp_fwd(int B, int T, int C, const uint4 *__restrict__ x, const uint4 *__restrict__ shift,
             const float *__restrict__ maa, const uint4 *__restrict__ m, uint4 *__restrict__ out) {
    const int row16 = C / 8;
    const size_t total = (size_t)B * T * row16, tokens = (size_t)B * T;
    for (size_t i = (size_t)blockIdx.x * TPB + threadIdx.x; i < total; i += (size_t)gridDim.x * TPB) {
        const size_t tok = i / row16;
        const int c8 = (int)(i - tok * row16), t = (int)(tok % T), b = (int)(tok / T);
        float xv[8], pv[8];
        unpack8(x[i], xv);
        unpack8(t > 0 ? x[i - row16] : shift[(size_t)b * row16 + c8], pv);
#pragma unroll
        for (int q = 0; q < 8; q++) pv[q] -= xv[q];
#pragma unroll
        for (int n = 0; n < NMIX; n++) {
            float a[8], mv[8], o[8];
            load8f(maa + (size_t)n * C + c8 * 8, a);
            if (m) {
                unpack8(m[(size_t)n * tokens * row16 + i], mv);
#pragma unroll
                for (int q = 0; q < 8; q++) a[q] += mv[q];
            }
#pragma unroll
            for (int q = 0; q < 8; q++) o[q] = xv[q] + pv[q] * a[q];
            out[(size_t)n * tokens * row16 + i] = pack8(o);
        }
    }
}

// Backward of the mixes: with d = x_prev - x and a_i = maa_i + m_i,
//   gm_i = gout_i * d,   gmaa_i = sum over tokens of gm_i,
//   gx_t = sum_i gout_i,t (1 - a_i,t)  +  sum_i gout_i,t+1 a_i,t+1     (the second term: token t is
//   the predecessor of t+1; for a row's last token it comes from the next segment, `gshift_in`),
//   gshift_out = sum_i gout_i,0 a_i,0   (gradient w.r.t. `shift`).
// A thread walks the tokens of one (batch row, 8-channel column) so that the t+1 term is carried in
// registers; rows x columns give B*C/8 threads... too few for small B, so T is also cut into pieces
// and the carry of a piece is recomputed from the first token of the next piece.
template <int NMIX>
__global__ void __launch_bounds__(TPB)
k_ddlerp_bwd(int B, int T, int C, int piece, const uint4 *__restrict__ x, const uint4 *__restrict__ shift,
             const float *__restrict__ maa, const uint4 *__restrict__ m, const uint4 *__restrict__ gout,
             const uint4 *__restrict__ gshift_in, uint4 *__restrict__ gx, uint4 *__restrict__ gm,
             uint4 *__restrict__ gshift_out, float *__restrict__ part) {
    const int row16 = C / 8, npiece = (T + piece - 1) / piece;
    const size_t tokens = (size_t)B * T;
    const size_t id = (size_t)blockIdx.x * TPB + threadIdx.x;
    const size_t nthr = (size_t)B * npiece * row16;
    float acc[NMIX][8];
#pragma unroll
    for (int n = 0; n < NMIX; n++)
#pragma unroll
        for (int q = 0; q < 8; q++) acc[n][q] = 0.f;
    const int c8 = (int)(id % row16);
    if (id < nthr) {
        const int pc = (int)((id / row16) % npiece), b = (int)(id / ((size_t)row16 * npiece));
        const int t0 = pc * piece, t1 = min(T, t0 + piece);
        float mz[NMIX][8];
#pragma unroll
        for (int n = 0; n < NMIX; n++) load8f(maa + (size_t)n * C + c8 * 8, mz[n]);
        // carry: what token t1 (the first token after the piece) sends back to token t1-1
        float carry[8];
        if (t1 < T) {
            const size_t j = ((size_t)b * T + t1) * row16 + c8;
#pragma unroll
            for (int q = 0; q < 8; q++) carry[q] = 0.f;
#pragma unroll
            for (int n = 0; n < NMIX; n++) {
                float go[8], mv[8];
                unpack8(gout[(size_t)n * tokens * row16 + j], go);
                if (m) unpack8(m[(size_t)n * tokens * row16 + j], mv);
#pragma unroll
                for (int q = 0; q < 8; q++) carry[q] += go[q] * (mz[n][q] + (m ? mv[q] : 0.f));
            }
        } else if (gshift_in) {
            unpack8(gshift_in[(size_t)b * row16 + c8], carry);
        } else {
#pragma unroll
            for (int q = 0; q < 8; q++) carry[q] = 0.f;
        }
        for (int t = t1 - 1; t >= t0; t--) {
            const size_t i = ((size_t)b * T + t) * row16 + c8;
            float xv[8], pv[8], gxv[8], nxt[8];
            unpack8(x[i], xv);
            unpack8(t > 0 ? x[i - row16] : shift[(size_t)b * row16 + c8], pv);
#pragma unroll
            for (int q = 0; q < 8; q++) { pv[q] -= xv[q]; gxv[q] = carry[q]; nxt[q] = 0.f; }
#pragma unroll
            for (int n = 0; n < NMIX; n++) {
                float go[8], mv[8], gmv[8];
                unpack8(gout[(size_t)n * tokens * row16 + i], go);
                if (m) unpack8(m[(size_t)n * tokens * row16 + i], mv);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float a = mz[n][q] + (m ? mv[q] : 0.f);
                    gmv[q] = go[q] * pv[q];
                    acc[n][q] += gmv[q];
                    gxv[q] += go[q] * (1.f - a);
                    nxt[q] += go[q] * a;
                }
                if (gm) gm[(size_t)n * tokens * row16 + i] = pack8(gmv);
            }
            gx[i] = pack8(gxv);
#pragma unroll
            for (int q = 0; q < 8; q++) carry[q] = nxt[q];
        }
        if (t0 == 0 && gshift_out) gshift_out[(size_t)b * row16 + c8] = pack8(carry);
    }
    // partial sums of gmaa per thread: [B*npiece, NMIX, C], folded by k_fold_maa
    if (id < nthr) {
        const size_t rowp = id / row16;
#pragma unroll
        for (int n = 0; n < NMIX; n++) {
            float4 *dst = reinterpret_cast<float4 *>(part + (rowp * NMIX + n) * C + c8 * 8);
            dst[0] = make_float4(acc[n][0], acc[n][1], acc[n][2], acc[n][3]);
            dst[1] = make_float4(acc[n][4], acc[n][5], acc[n][6], acc[n][7]);
        }
    }
}

__global__ void __launch_bounds__(TPB)
k_fold_maa(const float *__restrict__ part, int rows, int nmix, int C, float *__restrict__ gmaa) {
    const int i = blockIdx.x * TPB + threadIdx.x;
    if (i >= nmix * C) return;
    float a = 0.f;
    for (int r = 0; r < rows; r++) a += part[(size_t)r * nmix * C + i];
    gmaa[i] = a;
}

Split make_split(int tokens, int C) {
    Split sp;
    sp.ncb = (C + 255) / 256;
    int sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int want = (sms * 8 + sp.ncb - 1) / sp.ncb;           // about 8 CTAs per SM
    const int most = (tokens + 7) / 8;
    sp.nslot = want < most ? want : most;
    if (sp.nslot < 1) sp.nslot = 1;
    return sp;
}
constexpr int DDLERP_PIECE = 64;

}  // namespace
}  // namespace wkv

using namespace wkv;

extern "C" {

int wkv_lnx_gate_forward(int tokens, int H, const void *y, const void *g, const float *gamma, const float *beta,
                         float eps, void *out, void *stream) {
    if (tokens < 0 || H < 0) return WKV_ERR_SHAPE;
    if (tokens == 0 || H == 0) return WKV_OK;
    if (!y || !g || !gamma || !beta || !out) return WKV_ERR_NULL;
    for (const void *p : {y, g, (const void *)gamma, (const void *)beta, (const void *)out})
        if (!aligned16(p)) return WKV_ERR_ALIGN;
    const int C = H * HEAD;
    const Split sp = make_split(tokens, C);
    k_lnx_gate_fwd<<<sp.ncb * sp.nslot, TPB, 0, (cudaStream_t)stream>>>(tokens, C, sp, (const uint4 *)y, (const uint4 *)g,
                                                                      gamma, beta, eps, (uint4 *)out);
    return launch_status();
}

size_t wkv_lnx_gate_backward_workspace(int tokens, int H) {
    if (tokens <= 0 || H <= 0) return 0;
    return (size_t)make_split(tokens, H * HEAD).nslot * 2 * H * HEAD * sizeof(float);
}

int wkv_lnx_gate_backward(int tokens, int H, const void *y, const void *g, const float *gamma, const float *beta,
                          float eps, const void *gout, void *gy, void *gg, float *ggamma, float *gbeta,
                          void *workspace, size_t workspace_bytes, void *stream) {
    if (tokens < 0 || H < 0) return WKV_ERR_SHAPE;
    if (H == 0) return WKV_OK;
    if (!ggamma || !gbeta) return WKV_ERR_NULL;
    const int C = H * HEAD;
    cudaStream_t s = (cudaStream_t)stream;
    if (tokens == 0) {
        if (cudaMemsetAsync(ggamma, 0, C * sizeof(float), s) != cudaSuccess ||
            cudaMemsetAsync(gbeta, 0, C * sizeof(float), s) != cudaSuccess)
            return WKV_ERR_LAUNCH;
        return WKV_OK;
    }
    if (!y || !g || !gamma || !beta || !gout || !gy || !gg) return WKV_ERR_NULL;
    for (const void *p : {y, g, (const void *)gamma, (const void *)beta, gout, (const void *)gy, (const void *)gg})
        if (!aligned16(p)) return WKV_ERR_ALIGN;
    if (!workspace || workspace_bytes < wkv_lnx_gate_backward_workspace(tokens, H)) return WKV_ERR_WORKSPACE;
    const Split sp = make_split(tokens, C);
    k_lnx_gate_bwd<<<sp.ncb * sp.nslot, TPB, 0, s>>>(tokens, C, sp, (const uint4 *)y, (const uint4 *)g, gamma, beta, eps,
                                                     (const uint4 *)gout, (uint4 *)gy, (uint4 *)gg, (float *)workspace);
    k_fold_params<<<(C + TPB - 1) / TPB, TPB, 0, s>>>((const float *)workspace, sp.nslot, C, ggamma, gbeta);
    return launch_status();
}

int wkv_ddlerp_forward(int B, int T, int C, int nmix, const void *x, const void *shift, const float *maa,
                       const void *m, void *out, void *stream) {
    if (B < 0 || T < 0 || C < 0 || C % 8 != 0) return WKV_ERR_SHAPE;
    if (nmix != 1 && nmix != 3 && nmix != 4 && nmix != 5) return WKV_ERR_UNSUPPORTED;
    if (B == 0 || T == 0 || C == 0) return WKV_OK;
    if (!x || !shift || !maa || !out) return WKV_ERR_NULL;
    for (const void *p : {x, shift, (const void *)maa, (const void *)out})
        if (!aligned16(p)) return WKV_ERR_ALIGN;
    if (m && !aligned16(m)) return WKV_ERR_ALIGN;
    const size_t total = (size_t)B * T * (C / 8);
    size_t blocks = (total + TPB - 1) / TPB;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (nmix == 5)
        k_ddlerp_fwd<5><<<(unsigned)blocks, TPB, 0, (cudaStream_t)stream>>>(B, T, C, (const uint4 *)x, (const uint4 *)shift,
                                                                           maa, (const uint4 *)m, (uint4 *)out);
    else if (nmix == 4)
        k_ddlerp_fwd<4><<<(unsigned)blocks, TPB, 0, (cudaStream_t)stream>>>(B, T, C, (const uint4 *)x, (const uint4 *)shift,
                                                                           maa, (const uint4 *)m, (uint4 *)out);
    else if (nmix == 3)
        k_ddlerp_fwd<3><<<(unsigned)blocks, TPB, 0, (cudaStream_t)stream>>>(B, T, C, (const uint4 *)x, (const uint4 *)shift,
                                                                           maa, (const uint4 *)m, (uint4 *)out);
    else
        k_ddlerp_fwd<1><<<(unsigned)blocks, TPB, 0, (cudaStream_t)stream>>>(B, T, C, (const uint4 *)x, (const uint4 *)shift,
                                                                           maa, (const uint4 *)m, (uint4 *)out);
    return launch_status();
}

size_t wkv_ddlerp_backward_workspace(int B, int T, int C, int nmix) {
    if (B <= 0 || T <= 0 || C <= 0) return 0;
    const size_t npiece = (T + DDLERP_PIECE - 1) / DDLERP_PIECE;
    return (size_t)B * npiece * nmix * C * sizeof(float);
}

int wkv_ddlerp_backward(int B, int T, int C, int nmix, const void *x, const void *shift, const float *maa, const void *m,
                        const void *gout, const void *gshift_in, void *gx, void *gm, void *gshift_out, float *gmaa,
                        void *workspace, size_t workspace_bytes, void *stream) {
    if (B < 0 || T < 0 || C < 0 || C % 8 != 0) return WKV_ERR_SHAPE;
    if (nmix != 1 && nmix != 3 && nmix != 4 && nmix != 5) return WKV_ERR_UNSUPPORTED;
    if (!gmaa) return WKV_ERR_NULL;
    cudaStream_t s = (cudaStream_t)stream;
    if (B == 0 || T == 0 || C == 0) {
        if (C > 0 && cudaMemsetAsync(gmaa, 0, (size_t)nmix * C * sizeof(float), s) != cudaSuccess) return WKV_ERR_LAUNCH;
        return WKV_OK;
    }
    if (!x || !shift || !maa || !gout || !gx) return WKV_ERR_NULL;
    if (m && !gm) return WKV_ERR_NULL;
    for (const void *p : {x, shift, (const void *)maa, gout, (const void *)gx})
        if (!aligned16(p)) return WKV_ERR_ALIGN;
    if (!workspace || workspace_bytes < wkv_ddlerp_backward_workspace(B, T, C, nmix)) return WKV_ERR_WORKSPACE;
    const int npiece = (T + DDLERP_PIECE - 1) / DDLERP_PIECE;
    const size_t nthr = (size_t)B * npiece * (C / 8);
    const unsigned blocks = (unsigned)((nthr + TPB - 1) / TPB);
    if (nmix == 5)
        k_ddlerp_bwd<5><<<blocks, TPB, 0, s>>>(B, T, C, DDLERP_PIECE, (const uint4 *)x, (const uint4 *)shift, maa,
                                               (const uint4 *)m, (const uint4 *)gout, (const uint4 *)gshift_in, (uint4 *)gx,
                                               (uint4 *)gm, (uint4 *)gshift_out, (float *)workspace);
    else if (nmix == 4)
        k_ddlerp_bwd<4><<<blocks, TPB, 0, s>>>(B, T, C, DDLERP_PIECE, (const uint4 *)x, (const uint4 *)shift, maa,
                                               (const uint4 *)m, (const uint4 *)gout, (const uint4 *)gshift_in, (uint4 *)gx,
                                               (uint4 *)gm, (uint4 *)gshift_out, (float *)workspace);
    else if (nmix == 3)
        k_ddlerp_bwd<3><<<blocks, TPB, 0, s>>>(B, T, C, DDLERP_PIECE, (const uint4 *)x, (const uint4 *)shift, maa,
                                               (const uint4 *)m, (const uint4 *)gout, (const uint4 *)gshift_in, (uint4 *)gx,
                                               (uint4 *)gm, (uint4 *)gshift_out, (float *)workspace);
    else
        k_ddlerp_bwd<1><<<blocks, TPB, 0, s>>>(B, T, C, DDLERP_PIECE, (const uint4 *)x, (const uint4 *)shift, maa,
                                               (const uint4 *)m, (const uint4 *)gout, (const uint4 *)gshift_in, (uint4 *)gx,
                                               (uint4 *)gm, (uint4 *)gshift_out, (float *)workspace);
    k_fold_maa<<<(nmix * C + TPB - 1) / TPB, TPB, 0, s>>>((const float *)workspace, B * npiece, nmix, C, gmaa);
    return launch_status();
}

}  // extern "C"
