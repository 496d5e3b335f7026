// v4 WKV, parallel over time.
//
// One thread per (batch, channel) chain leaves a B200 mostly idle (B*C chains, each a
// dependent chain over T).  The state recurrence is linear in (p, q) with a constant decay
// per step, so T is cut into segments of SEG tokens that are processed independently:
//
//   forward   1. k_seg_summary   each segment's (p,q,o) from an empty state
//             2. k_seg_scan      per chain, fold the summaries: state at every segment start
//             3. k_seg_forward   each segment from its true start state -> y
//   backward  1-2 as above (segment-start states)
//             3. k_seg_rsummary  each segment's reverse accumulation (gp,gq,go) from an empty
//                                incoming gradient (needs the forward quantities of the segment)
//             4. k_seg_rscan     per chain, fold them in reverse: (gp,gq,go) at every segment end
//             5. k_seg_backward  each segment with its start state and end gradient -> gk, gv and
//                                per-segment partial gw, gu
//             6. k_seg_reduce    sum the partials over the segments in a fixed order
//
// Per-segment arithmetic is the math of RWKV-v4neo/cuda/wkv_cuda_bf16.cu:7-158; folding two
// pieces a (earlier, n tokens after it) and b:  o' = o_a + n*w;  m = max(o', o_b);
// (p,q) = e^{o'-m}(p_a,q_a) + e^{o_b-m}(p_b,q_b);  o = m  -- the same max-shift the kernel uses
// token by token.  Threads of a warp hold consecutive channels: every access is coalesced.
#include "wkv_common.cuh"

namespace wkv {
namespace {

constexpr float MIN_VALUE = -1e38f;
constexpr int SEG = 64;     // tokens per segment
constexpr int TILE = 4;     // tokens recomputed at a time inside a segment (register stash).  Small on purpose:
                            // the backward kernels are bound by latency at low occupancy, and 4-token tiles need 72-96
                            // registers where 16-token tiles needed 128-168 (measured: 1.21 -> 1.09 ms on the v4 workload)
constexpr int THREADS = 128;

__device__ __forceinline__ void exp_pair(float a, float b, float &A, float &Bv, float &m) {
    const float d = a - b;
    const float e = __expf(-fabsf(d));
    const bool ge = d >= 0.f;
    A = ge ? 1.f : e;
    Bv = ge ? e : 1.f;
    m = ge ? a : b;
}

struct Dims {
    int B, T, C, nseg;
};

// thread -> (b, seg, c); c fastest so that a warp reads consecutive channels
__device__ __forceinline__ bool locate(const Dims &d, int &b, int &seg, int &c, int &t0, int &len) {
    const long long idx = (long long)blockIdx.x * THREADS + threadIdx.x;
    if (idx >= (long long)d.B * d.nseg * d.C) return false;
    c = (int)(idx % d.C);
    seg = (int)((idx / d.C) % d.nseg);
    b = (int)(idx / ((long long)d.C * d.nseg));
    t0 = seg * SEG;
    len = min(SEG, d.T - t0);
    return true;
}
// summaries / segment states: [B][nseg][3][C]
__device__ __forceinline__ size_t sidx(const Dims &d, int b, int seg, int c) {
    return ((size_t)(b * d.nseg + seg) * 3) * d.C + c;
}

template <typename F>
__global__ void __launch_bounds__(THREADS)
k_seg_summary(Dims d, const float *__restrict__ w_, const F *__restrict__ k_, const F *__restrict__ v_,
              float *__restrict__ loc) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate(d, b, seg, c, t0, len)) return;
    const float w = w_[c];
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    float p = 0.f, q = 0.f, o = MIN_VALUE;
    // loads of 8 tokens go out together, then the dependent chain runs over them
    for (int t8 = 0; t8 < len; t8 += 8) {
        float kk[8], vv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool in = t8 + j < len;
            kk[j] = in ? Elem<F>::ld(k_ + off + (size_t)(t8 + j) * d.C) : 0.f;
            vv[j] = in ? Elem<F>::ld(v_ + off + (size_t)(t8 + j) * d.C) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (t8 + j < len) {
                float A, E, m;
                exp_pair(w + o, kk[j], A, E, m);
                p = A * p + E * vv[j]; q = A * q + E; o = m;
            }
        }
    }
    const size_t s = sidx(d, b, seg, c);
    loc[s] = p; loc[s + d.C] = q; loc[s + 2 * (size_t)d.C] = o;
}

// per chain: state at the start of every segment, and the final state
__global__ void __launch_bounds__(THREADS)
k_seg_scan(Dims d, const float *__restrict__ w_, const float *__restrict__ state_in,
           const float *__restrict__ loc, float *__restrict__ st, float *__restrict__ state_out) {
    pdl_wait();
    pdl_trigger();
    const int idx = blockIdx.x * THREADS + threadIdx.x;
    if (idx >= d.B * d.C) return;
    const int b = idx / d.C, c = idx % d.C;
    const float w = w_[c];
    float p = 0.f, q = 0.f, o = MIN_VALUE;
    if (state_in) { p = state_in[(size_t)idx * 3]; q = state_in[(size_t)idx * 3 + 1]; o = state_in[(size_t)idx * 3 + 2]; }
    // (the summaries of 8 pieces are fetched together: the chain is short, the loads are what takes time)
    for (int s8 = 0; s8 < d.nseg; s8 += 8) {
        float lp[8], lq[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool in = s8 + j < d.nseg;
            const size_t s = sidx(d, b, in ? s8 + j : s8, c);
            lp[j] = in ? loc[s] : 0.f; lq[j] = in ? loc[s + d.C] : 0.f; lo[j] = in ? loc[s + 2 * (size_t)d.C] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int seg = s8 + j;
            if (seg < d.nseg) {
                const size_t s = sidx(d, b, seg, c);
                st[s] = p; st[s + d.C] = q; st[s + 2 * (size_t)d.C] = o;
                const int len = min(SEG, d.T - seg * SEG);
                float A, E, m;
                exp_pair(o + len * w, lo[j], A, E, m);
                p = A * p + E * lp[j]; q = A * q + E * lq[j]; o = m;
            }
        }
    }
    if (state_out) { state_out[(size_t)idx * 3] = p; state_out[(size_t)idx * 3 + 1] = q; state_out[(size_t)idx * 3 + 2] = o; }
}

// What forward leaves for backward (optional): at the start of every CK-token tile of every piece the
// state (p,q,o) and its derivative w.r.t. the decay accumulated since the piece start (dpdw,dqdw) --
// [B][nseg][SEG/CK][5][C] floats, 2.5 bytes per token-channel.  With it neither backward pass needs its
// forward sweep over the piece (which is there only to find the tile-start values).
constexpr int CK = 8;
constexpr int NCK = SEG / CK;
__device__ __forceinline__ size_t cidx(const Dims &d, int b, int seg, int tile, int c) {
    return (((size_t)(b * d.nseg + seg) * NCK + tile) * 5) * d.C + c;
}

template <typename F>
__global__ void __launch_bounds__(THREADS)
k_seg_forward(Dims d, const float *__restrict__ w_, const F *__restrict__ u_, const F *__restrict__ k_,
              const F *__restrict__ v_, const float *__restrict__ st, F *__restrict__ y_, float *__restrict__ ck) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate(d, b, seg, c, t0, len)) return;
    const float w = w_[c], u = Elem<F>::ld(u_ + c);
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    const size_t s = sidx(d, b, seg, c);
    float p = st[s], q = st[s + d.C], o = st[s + 2 * (size_t)d.C];
    float dpdw = 0.f, dqdw = 0.f;
    for (int t8 = 0; t8 < len; t8 += 8) {
        if (ck) {      // (8 = CK: every load batch starts a tile)
            const size_t i = cidx(d, b, seg, t8 / CK, c);
            ck[i] = p; ck[i + d.C] = q; ck[i + 2 * (size_t)d.C] = o;
            ck[i + 3 * (size_t)d.C] = dpdw; ck[i + 4 * (size_t)d.C] = dqdw;
        }
        float kk[8], vv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool in = t8 + j < len;
            kk[j] = in ? Elem<F>::ld(k_ + off + (size_t)(t8 + j) * d.C) : 0.f;
            vv[j] = in ? Elem<F>::ld(v_ + off + (size_t)(t8 + j) * d.C) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (t8 + j < len) {
                float A, E, m;
                exp_pair(o, u + kk[j], A, E, m);
                Elem<F>::st(y_ + off + (size_t)(t8 + j) * d.C, __fdividef(A * p + E * vv[j], A * q + E));
                exp_pair(w + o, kk[j], A, E, m);
                if (ck) { dpdw = A * (p + dpdw); dqdw = A * (q + dqdw); }
                p = A * p + E * vv[j]; q = A * q + E; o = m;
            }
        }
    }
}

// One segment backward.  FINAL = false: only the reverse accumulation from an empty incoming
// gradient (the segment's reverse summary).  FINAL = true: with the true incoming gradient,
// writing gk, gv and the segment's gw, gu.
template <typename F, bool FINAL>
__global__ void __launch_bounds__(THREADS)
k_seg_backward(Dims d, const float *__restrict__ w_, const F *__restrict__ u_, const F *__restrict__ k_,
               const F *__restrict__ v_, const F *__restrict__ gy_, const float *__restrict__ st,
               const float *__restrict__ gend, float *__restrict__ rloc, F *__restrict__ gk_,
               F *__restrict__ gv_, float *__restrict__ gw_part, float *__restrict__ gu_part) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate(d, b, seg, c, t0, len)) return;
    const float w = w_[c], u = Elem<F>::ld(u_ + c);
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    const size_t s = sidx(d, b, seg, c);
    constexpr int NT = SEG / TILE;
    float cp[NT], cq[NT], co[NT];   // state at the start of every tile of the segment
    float p = st[s], q = st[s + d.C], o = st[s + 2 * (size_t)d.C];
    float gw = 0.f, gu = 0.f, dpdw = 0.f, dqdw = 0.f;
    // every tile: its loads go out together (independent of the recurrence), then the chain runs.
    // The tile loops stay rolled: unrolled, the compiler hoists the loads of all four tiles and
    // runs out of registers; the 12 tile-start values then live in (L1-resident) local memory.
#pragma unroll 1
    for (int tile = 0; tile < NT; tile++) {
        cp[tile] = p; cq[tile] = q; co[tile] = o;
        if (tile * TILE < len) {
            float kk[TILE], vv[TILE], gg[TILE];
#pragma unroll
            for (int j = 0; j < TILE; j++) {
                const int t = tile * TILE + j;
                const bool in = t < len;
                kk[j] = in ? Elem<F>::ld(k_ + off + (size_t)t * d.C) : 0.f;
                vv[j] = in ? Elem<F>::ld(v_ + off + (size_t)t * d.C) : 0.f;
                gg[j] = (FINAL && in) ? Elem<F>::ld(gy_ + off + (size_t)t * d.C) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < TILE; j++) {
                if (tile * TILE + j < len) {
                    float A, E, m;
                    if (FINAL) {
                        exp_pair(o, u + kk[j], A, E, m);
                        const float iden = __fdividef(1.f, A * q + E);
                        const float y = (A * p + E * vv[j]) * iden;
                        gw += gg[j] * (dpdw - dqdw * y) * iden * A;
                        gu += gg[j] * (vv[j] - y) * E * iden;
                    }
                    exp_pair(w + o, kk[j], A, E, m);
                    if (FINAL) { dpdw = A * (p + dpdw); dqdw = A * (q + dqdw); }
                    p = A * p + E * vv[j]; q = A * q + E; o = m;
                }
            }
        }
    }
    float gp = 0.f, gq = 0.f, go = MIN_VALUE;
    if (FINAL) {
        gp = gend[s]; gq = gend[s + d.C]; go = gend[s + 2 * (size_t)d.C];
        gw += (gp * dpdw + gq * dqdw) * __expf(o + go);
    }
#pragma unroll 1
    for (int tile = NT - 1; tile >= 0; tile--) {
        if (tile * TILE < len) {
            p = cp[tile]; q = cq[tile]; o = co[tile];
            float kk[TILE], vv[TILE], gg[TILE];
#pragma unroll
            for (int j = 0; j < TILE; j++) {
                const int t = tile * TILE + j;
                const bool in = t < len;
                kk[j] = in ? Elem<F>::ld(k_ + off + (size_t)t * d.C) : 0.f;
                vv[j] = in ? Elem<F>::ld(v_ + off + (size_t)t * d.C) : 0.f;
                gg[j] = in ? Elem<F>::ld(gy_ + off + (size_t)t * d.C) : 0.f;
            }
            float ys[TILE], zs[TILE], ze[TILE];
#pragma unroll
            for (int j = 0; j < TILE; j++) {
                if (tile * TILE + j < len) {
                    float A, E, m;
                    exp_pair(o, u + kk[j], A, E, m);
                    const float iden = __fdividef(1.f, A * q + E);
                    ys[j] = (A * p + E * vv[j]) * iden; zs[j] = iden; ze[j] = kk[j] + u - m;
                    exp_pair(w + o, kk[j], A, E, m);
                    p = A * p + E * vv[j]; q = A * q + E; o = m;
                }
            }
#pragma unroll
            for (int j = TILE - 1; j >= 0; j--) {
                const int t = tile * TILE + j;
                if (t < len) {
                    const size_t ii = off + (size_t)t * d.C;
                    const float gz = gg[j] * zs[j];
                    float A, E, m;
                    if (FINAL) {
                        A = gz * __expf(ze[j]);
                        E = __expf(kk[j] + go);
                        Elem<F>::st(gk_ + ii, A * (vv[j] - ys[j]) + E * (gp * vv[j] + gq));
                        Elem<F>::st(gv_ + ii, A + E * gp);
                    }
                    exp_pair(w + go, ze[j] - kk[j] - u, A, E, m);
                    E *= gz;
                    gp = A * gp + E; gq = A * gq - E * ys[j]; go = m;
                }
            }
        }
    }
    if (FINAL) {
        gw_part[(size_t)(b * d.nseg + seg) * d.C + c] = gw * w;
        gu_part[(size_t)(b * d.nseg + seg) * d.C + c] = gu;
    } else {
        rloc[s] = gp; rloc[s + d.C] = gq; rloc[s + 2 * (size_t)d.C] = go;
    }
}

// The same two passes when the forward call left its tile checkpoints: no forward sweep.  Tiles of CK
// tokens are taken in reverse; each starts from its checkpoint, recomputes y, 1/denominator and the
// exponent for its tokens (FINAL: and adds the tile's share of gw, gu, whose running derivatives
// dpdw, dqdw come from the checkpoint too), then runs the reverse recurrence over them.
template <typename F, bool FINAL>
__global__ void __launch_bounds__(THREADS)
k_seg_backward_ck(Dims d, const float *__restrict__ w_, const F *__restrict__ u_, const F *__restrict__ k_,
                  const F *__restrict__ v_, const F *__restrict__ gy_, const float *__restrict__ ck,
                  const float *__restrict__ gend, float *__restrict__ rloc, F *__restrict__ gk_,
                  F *__restrict__ gv_, float *__restrict__ gw_part, float *__restrict__ gu_part) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate(d, b, seg, c, t0, len)) return;
    const float w = w_[c], u = Elem<F>::ld(u_ + c);
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    const size_t s = sidx(d, b, seg, c);
    float gw = 0.f, gu = 0.f;
    float gp = 0.f, gq = 0.f, go = MIN_VALUE;
    if (FINAL) { gp = gend[s]; gq = gend[s + d.C]; go = gend[s + 2 * (size_t)d.C]; }
    const int last = (len - 1) / CK;
#pragma unroll 1
    for (int tile = last; tile >= 0; tile--) {
        const size_t ci = cidx(d, b, seg, tile, c);
        float p = ck[ci], q = ck[ci + d.C], o = ck[ci + 2 * (size_t)d.C];
        float dpdw = 0.f, dqdw = 0.f;
        if (FINAL) { dpdw = ck[ci + 3 * (size_t)d.C]; dqdw = ck[ci + 4 * (size_t)d.C]; }
        float kk[CK], vv[CK], gg[CK];
#pragma unroll
        for (int j = 0; j < CK; j++) {
            const int t = tile * CK + j;
            const bool in = t < len;
            kk[j] = in ? Elem<F>::ld(k_ + off + (size_t)t * d.C) : 0.f;
            vv[j] = in ? Elem<F>::ld(v_ + off + (size_t)t * d.C) : 0.f;
            gg[j] = in ? Elem<F>::ld(gy_ + off + (size_t)t * d.C) : 0.f;
        }
        float ys[CK], zs[CK], ze[CK];
#pragma unroll
        for (int j = 0; j < CK; j++) {
            if (tile * CK + j < len) {
                float A, E, m;
                exp_pair(o, u + kk[j], A, E, m);
                const float iden = __fdividef(1.f, A * q + E);
                ys[j] = (A * p + E * vv[j]) * iden; zs[j] = iden; ze[j] = kk[j] + u - m;
                if (FINAL) {
                    gw += gg[j] * (dpdw - dqdw * ys[j]) * iden * A;
                    gu += gg[j] * (vv[j] - ys[j]) * E * iden;
                }
                exp_pair(w + o, kk[j], A, E, m);
                if (FINAL) { dpdw = A * (p + dpdw); dqdw = A * (q + dqdw); }
                p = A * p + E * vv[j]; q = A * q + E; o = m;
            }
        }
        // the piece's end: what the incoming gradient sees of the decay through the whole piece
        if (FINAL && tile == last) gw += (gp * dpdw + gq * dqdw) * __expf(o + go);
#pragma unroll
        for (int j = CK - 1; j >= 0; j--) {
            const int t = tile * CK + j;
            if (t < len) {
                const size_t ii = off + (size_t)t * d.C;
                const float gz = gg[j] * zs[j];
                float A, E, m;
                if (FINAL) {
                    A = gz * __expf(ze[j]);
                    E = __expf(kk[j] + go);
                    Elem<F>::st(gk_ + ii, A * (vv[j] - ys[j]) + E * (gp * vv[j] + gq));
                    Elem<F>::st(gv_ + ii, A + E * gp);
                }
                exp_pair(w + go, ze[j] - kk[j] - u, A, E, m);
                E *= gz;
                gp = A * gp + E; gq = A * gq - E * ys[j]; go = m;
            }
        }
    }
    if (FINAL) {
        gw_part[(size_t)(b * d.nseg + seg) * d.C + c] = gw * w;
        gu_part[(size_t)(b * d.nseg + seg) * d.C + c] = gu;
    } else {
        rloc[s] = gp; rloc[s + d.C] = gq; rloc[s + 2 * (size_t)d.C] = go;
    }
}

// ---------------------------------------------------------------------------
// The same three hot kernels with TWO adjacent channels per thread (used whenever C is even).  These
// kernels are bound by latency, so what counts is the bytes each access in flight carries: with a
// channel pair per thread every k, v, gy, y, gk, gv access is 4 bytes per lane for 16-bit types
// (128 bytes per warp instead of 64) and 8 bytes for fp32, half as many threads run the same number
// of chains, and every thread has two independent chains to interleave.  Measured on the v4
// workload: bf16 1.07 -> 0.93 ms, fp32 1.00 -> 0.86 ms.
template <typename F> struct Pair;
template <> struct Pair<__nv_bfloat16> {
    static __device__ __forceinline__ float2 ld(const __nv_bfloat16 *p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
    }
    static __device__ __forceinline__ void st(__nv_bfloat16 *p, float a, float b) {
        *reinterpret_cast<__nv_bfloat162 *>(p) = __floats2bfloat162_rn(a, b);
    }
};
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 ld(const float *p) { return *reinterpret_cast<const float2 *>(p); }
    static __device__ __forceinline__ void st(float *p, float a, float b) { *reinterpret_cast<float2 *>(p) = make_float2(a, b); }
};
template <> struct Pair<__half> {
    static __device__ __forceinline__ float2 ld(const __half *p) {
        return __half22float2(*reinterpret_cast<const __half2 *>(p));
    }
    static __device__ __forceinline__ void st(__half *p, float a, float b) {
        *reinterpret_cast<__half2 *>(p) = __floats2half2_rn(a, b);
    }
};

// thread -> (b, seg, channel pair c, c+1)
__device__ __forceinline__ bool locate2(const Dims &d, int &b, int &seg, int &c, int &t0, int &len) {
    const long long idx = (long long)blockIdx.x * THREADS + threadIdx.x;
    const int half = d.C / 2;
    if (idx >= (long long)d.B * d.nseg * half) return false;
    c = 2 * (int)(idx % half);
    seg = (int)((idx / half) % d.nseg);
    b = (int)(idx / ((long long)half * d.nseg));
    t0 = seg * SEG;
    len = min(SEG, d.T - t0);
    return true;
}

template <typename F>
__global__ void __launch_bounds__(THREADS)
k_seg_summary2(Dims d, const float *__restrict__ w_, const F *__restrict__ k_, const F *__restrict__ v_,
               float *__restrict__ loc) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate2(d, b, seg, c, t0, len)) return;
    const float w[2] = {w_[c], w_[c + 1]};
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    float p[2] = {0.f, 0.f}, q[2] = {0.f, 0.f}, o[2] = {MIN_VALUE, MIN_VALUE};
    for (int t8 = 0; t8 < len; t8 += 8) {
        float2 kk[8], vv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool in = t8 + j < len;
            kk[j] = in ? Pair<F>::ld(k_ + off + (size_t)(t8 + j) * d.C) : make_float2(0.f, 0.f);
            vv[j] = in ? Pair<F>::ld(v_ + off + (size_t)(t8 + j) * d.C) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (t8 + j < len) {
                const float kj[2] = {kk[j].x, kk[j].y}, vj[2] = {vv[j].x, vv[j].y};
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    float A, E, m;
                    exp_pair(w[n] + o[n], kj[n], A, E, m);
                    p[n] = A * p[n] + E * vj[n]; q[n] = A * q[n] + E; o[n] = m;
                }
            }
        }
    }
    const size_t s = sidx(d, b, seg, c);
    *reinterpret_cast<float2 *>(loc + s) = make_float2(p[0], p[1]);
    *reinterpret_cast<float2 *>(loc + s + d.C) = make_float2(q[0], q[1]);
    *reinterpret_cast<float2 *>(loc + s + 2 * (size_t)d.C) = make_float2(o[0], o[1]);
}

template <typename F>
__global__ void __launch_bounds__(THREADS)
k_seg_forward2(Dims d, const float *__restrict__ w_, const F *__restrict__ u_, const F *__restrict__ k_,
               const F *__restrict__ v_, const float *__restrict__ st, F *__restrict__ y_, float *__restrict__ ck) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate2(d, b, seg, c, t0, len)) return;
    const float w[2] = {w_[c], w_[c + 1]};
    const float2 u2 = Pair<F>::ld(u_ + c);
    const float u[2] = {u2.x, u2.y};
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    const size_t s = sidx(d, b, seg, c);
    float p[2], q[2], o[2], dpdw[2] = {0.f, 0.f}, dqdw[2] = {0.f, 0.f};
    {
        const float2 a = *reinterpret_cast<const float2 *>(st + s), e = *reinterpret_cast<const float2 *>(st + s + d.C),
                     f = *reinterpret_cast<const float2 *>(st + s + 2 * (size_t)d.C);
        p[0] = a.x; p[1] = a.y; q[0] = e.x; q[1] = e.y; o[0] = f.x; o[1] = f.y;
    }
    for (int t8 = 0; t8 < len; t8 += 8) {
        if (ck) {
            const size_t i = cidx(d, b, seg, t8 / CK, c);
            *reinterpret_cast<float2 *>(ck + i) = make_float2(p[0], p[1]);
            *reinterpret_cast<float2 *>(ck + i + d.C) = make_float2(q[0], q[1]);
            *reinterpret_cast<float2 *>(ck + i + 2 * (size_t)d.C) = make_float2(o[0], o[1]);
            *reinterpret_cast<float2 *>(ck + i + 3 * (size_t)d.C) = make_float2(dpdw[0], dpdw[1]);
            *reinterpret_cast<float2 *>(ck + i + 4 * (size_t)d.C) = make_float2(dqdw[0], dqdw[1]);
        }
        float2 kk[8], vv[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool in = t8 + j < len;
            kk[j] = in ? Pair<F>::ld(k_ + off + (size_t)(t8 + j) * d.C) : make_float2(0.f, 0.f);
            vv[j] = in ? Pair<F>::ld(v_ + off + (size_t)(t8 + j) * d.C) : make_float2(0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (t8 + j < len) {
                const float kj[2] = {kk[j].x, kk[j].y}, vj[2] = {vv[j].x, vv[j].y};
                float yo[2];
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    float A, E, m;
                    exp_pair(o[n], u[n] + kj[n], A, E, m);
                    yo[n] = __fdividef(A * p[n] + E * vj[n], A * q[n] + E);
                    exp_pair(w[n] + o[n], kj[n], A, E, m);
                    if (ck) { dpdw[n] = A * (p[n] + dpdw[n]); dqdw[n] = A * (q[n] + dqdw[n]); }
                    p[n] = A * p[n] + E * vj[n]; q[n] = A * q[n] + E; o[n] = m;
                }
                Pair<F>::st(y_ + off + (size_t)(t8 + j) * d.C, yo[0], yo[1]);
            }
        }
    }
}

template <typename F, bool FINAL>
__global__ void __launch_bounds__(THREADS)
k_seg_backward_ck2(Dims d, const float *__restrict__ w_, const F *__restrict__ u_, const F *__restrict__ k_,
                   const F *__restrict__ v_, const F *__restrict__ gy_, const float *__restrict__ ck,
                   const float *__restrict__ gend, float *__restrict__ rloc, F *__restrict__ gk_,
                   F *__restrict__ gv_, float *__restrict__ gw_part, float *__restrict__ gu_part) {
    pdl_wait();
    pdl_trigger();
    int b, seg, c, t0, len;
    if (!locate2(d, b, seg, c, t0, len)) return;
    const float w[2] = {w_[c], w_[c + 1]};
    const float2 u2 = Pair<F>::ld(u_ + c);
    const float u[2] = {u2.x, u2.y};
    const size_t off = ((size_t)b * d.T + t0) * d.C + c;
    const size_t s = sidx(d, b, seg, c);
    auto ld2 = [](const float *p, float (&x)[2]) { const float2 a = *reinterpret_cast<const float2 *>(p); x[0] = a.x; x[1] = a.y; };
    float gw[2] = {0.f, 0.f}, gu[2] = {0.f, 0.f};
    float gp[2] = {0.f, 0.f}, gq[2] = {0.f, 0.f}, go[2] = {MIN_VALUE, MIN_VALUE};
    if (FINAL) { ld2(gend + s, gp); ld2(gend + s + d.C, gq); ld2(gend + s + 2 * (size_t)d.C, go); }
    const int last = (len - 1) / CK;
#pragma unroll 1
    for (int tile = last; tile >= 0; tile--) {
        const size_t ci = cidx(d, b, seg, tile, c);
        float p[2], q[2], o[2], dpdw[2] = {0.f, 0.f}, dqdw[2] = {0.f, 0.f};
        ld2(ck + ci, p); ld2(ck + ci + d.C, q); ld2(ck + ci + 2 * (size_t)d.C, o);
        if (FINAL) { ld2(ck + ci + 3 * (size_t)d.C, dpdw); ld2(ck + ci + 4 * (size_t)d.C, dqdw); }
        float2 kk[CK], vv[CK], gg[CK];
#pragma unroll
        for (int j = 0; j < CK; j++) {
            const int t = tile * CK + j;
            const bool in = t < len;
            kk[j] = in ? Pair<F>::ld(k_ + off + (size_t)t * d.C) : make_float2(0.f, 0.f);
            vv[j] = in ? Pair<F>::ld(v_ + off + (size_t)t * d.C) : make_float2(0.f, 0.f);
            gg[j] = in ? Pair<F>::ld(gy_ + off + (size_t)t * d.C) : make_float2(0.f, 0.f);
        }
        float ys[CK][2], zs[CK][2], ze[CK][2];
#pragma unroll
        for (int j = 0; j < CK; j++) {
            if (tile * CK + j < len) {
                const float kj[2] = {kk[j].x, kk[j].y}, vj[2] = {vv[j].x, vv[j].y}, gj[2] = {gg[j].x, gg[j].y};
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    float A, E, m;
                    exp_pair(o[n], u[n] + kj[n], A, E, m);
                    const float iden = __fdividef(1.f, A * q[n] + E);
                    ys[j][n] = (A * p[n] + E * vj[n]) * iden; zs[j][n] = iden; ze[j][n] = kj[n] + u[n] - m;
                    if (FINAL) {
                        gw[n] += gj[n] * (dpdw[n] - dqdw[n] * ys[j][n]) * iden * A;
                        gu[n] += gj[n] * (vj[n] - ys[j][n]) * E * iden;
                    }
                    exp_pair(w[n] + o[n], kj[n], A, E, m);
                    if (FINAL) { dpdw[n] = A * (p[n] + dpdw[n]); dqdw[n] = A * (q[n] + dqdw[n]); }
                    p[n] = A * p[n] + E * vj[n]; q[n] = A * q[n] + E; o[n] = m;
                }
            }
        }
        if (FINAL && tile == last) {
#pragma unroll
            for (int n = 0; n < 2; n++) gw[n] += (gp[n] * dpdw[n] + gq[n] * dqdw[n]) * __expf(o[n] + go[n]);
        }
#pragma unroll
        for (int j = CK - 1; j >= 0; j--) {
            const int t = tile * CK + j;
            if (t < len) {
                const size_t ii = off + (size_t)t * d.C;
                const float kj[2] = {kk[j].x, kk[j].y}, vj[2] = {vv[j].x, vv[j].y}, gj[2] = {gg[j].x, gg[j].y};
                float ok[2], ov[2];
#pragma unroll
                for (int n = 0; n < 2; n++) {
                    const float gz = gj[n] * zs[j][n];
                    float A, E, m;
                    if (FINAL) {
                        A = gz * __expf(ze[j][n]);
                        E = __expf(kj[n] + go[n]);
                        ok[n] = A * (vj[n] - ys[j][n]) + E * (gp[n] * vj[n] + gq[n]);
                        ov[n] = A + E * gp[n];
                    }
                    exp_pair(w[n] + go[n], ze[j][n] - kj[n] - u[n], A, E, m);
                    E *= gz;
                    gp[n] = A * gp[n] + E; gq[n] = A * gq[n] - E * ys[j][n]; go[n] = m;
                }
                if (FINAL) {
                    Pair<F>::st(gk_ + ii, ok[0], ok[1]);
                    Pair<F>::st(gv_ + ii, ov[0], ov[1]);
                }
            }
        }
    }
    if (FINAL) {
        const size_t gi = (size_t)(b * d.nseg + seg) * d.C + c;
        *reinterpret_cast<float2 *>(gw_part + gi) = make_float2(gw[0] * w[0], gw[1] * w[1]);
        *reinterpret_cast<float2 *>(gu_part + gi) = make_float2(gu[0], gu[1]);
    } else {
        *reinterpret_cast<float2 *>(rloc + s) = make_float2(gp[0], gp[1]);
        *reinterpret_cast<float2 *>(rloc + s + d.C) = make_float2(gq[0], gq[1]);
        *reinterpret_cast<float2 *>(rloc + s + 2 * (size_t)d.C) = make_float2(go[0], go[1]);
    }
}

// per chain, in reverse: incoming gradient at the end of every segment, and the chain's glast_state
__global__ void __launch_bounds__(THREADS)
k_seg_rscan(Dims d, const float *__restrict__ w_, const float *__restrict__ gstate_out,
            const float *__restrict__ rloc, float *__restrict__ gend, float *__restrict__ gstate_in) {
    pdl_wait();
    pdl_trigger();
    const int idx = blockIdx.x * THREADS + threadIdx.x;
    if (idx >= d.B * d.C) return;
    const int b = idx / d.C, c = idx % d.C;
    const float w = w_[c];
    float gp = 0.f, gq = 0.f, go = MIN_VALUE;
    if (gstate_out) {
        gp = gstate_out[(size_t)idx * 3]; gq = gstate_out[(size_t)idx * 3 + 1]; go = gstate_out[(size_t)idx * 3 + 2];
        if (gp == 0.f && gq == 0.f) go = MIN_VALUE;
    }
    for (int s8 = d.nseg - 1; s8 >= 0; s8 -= 8) {
        float lp[8], lq[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const bool in = s8 - j >= 0;
            const size_t s = sidx(d, b, in ? s8 - j : 0, c);
            lp[j] = in ? rloc[s] : 0.f; lq[j] = in ? rloc[s + d.C] : 0.f; lo[j] = in ? rloc[s + 2 * (size_t)d.C] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int seg = s8 - j;
            if (seg >= 0) {
                const size_t s = sidx(d, b, seg, c);
                gend[s] = gp; gend[s + d.C] = gq; gend[s + 2 * (size_t)d.C] = go;
                const int len = min(SEG, d.T - seg * SEG);
                float A, E, m;
                exp_pair(go + len * w, lo[j], A, E, m);
                gp = A * gp + E * lp[j]; gq = A * gq + E * lq[j]; go = m;
            }
        }
    }
    if (gstate_in) { gstate_in[(size_t)idx * 3] = gp; gstate_in[(size_t)idx * 3 + 1] = gq; gstate_in[(size_t)idx * 3 + 2] = go; }
}

__global__ void __launch_bounds__(THREADS)
k_seg_reduce(Dims d, const float *__restrict__ gw_part, const float *__restrict__ gu_part,
             float *__restrict__ gw, float *__restrict__ gu) {
    pdl_wait();
    pdl_trigger();
    const int idx = blockIdx.x * THREADS + threadIdx.x;
    if (idx >= d.B * d.C) return;
    const int b = idx / d.C, c = idx % d.C;
    float a = 0.f, e = 0.f;
#pragma unroll 8
    for (int seg = 0; seg < d.nseg; seg++) {
        a += gw_part[(size_t)(b * d.nseg + seg) * d.C + c];
        e += gu_part[(size_t)(b * d.nseg + seg) * d.C + c];
    }
    gw[idx] = a;
    gu[idx] = e;
}

inline unsigned blocks(long long n) { return (unsigned)((n + THREADS - 1) / THREADS); }

// `ckpt` (or NULL): where the piece-start states go instead of the workspace, for the backward call to reuse
template <typename F>
int par_fwd(Dims d, const float *w, const void *u, const void *k, const void *v, const float *si, void *y,
            float *so, float *ws, float *ckpt, cudaStream_t s) {
    const size_t n3 = (size_t)d.B * d.nseg * 3 * d.C;
    float *loc = ws, *st = ws + n3;
    const long long nthr = (long long)d.B * d.nseg * d.C;
    int err = WKV_OK;
    if constexpr (sizeof(F) >= 2) {
        if (d.C % 2 == 0) {      // a channel pair per thread (every dtype)
            err |= launch_chained(k_seg_summary2<F>, dim3(blocks(nthr / 2)), dim3(THREADS), 0, s, d, w,
                                  (const F *)k, (const F *)v, loc);
            err |= launch_chained(k_seg_scan, dim3(blocks((long long)d.B * d.C)), dim3(THREADS), 0, s, d, w, si,
                                  loc, st, so);
            err |= launch_chained(k_seg_forward2<F>, dim3(blocks(nthr / 2)), dim3(THREADS), 0, s, d, w,
                                  (const F *)u, (const F *)k, (const F *)v, st, (F *)y, ckpt);
            return err ? WKV_ERR_LAUNCH : WKV_OK;
        }
    }
    err |= launch_chained(k_seg_summary<F>, dim3(blocks(nthr)), dim3(THREADS), 0, s, d, w, (const F *)k,
                          (const F *)v, loc);
    err |= launch_chained(k_seg_scan, dim3(blocks((long long)d.B * d.C)), dim3(THREADS), 0, s, d, w, si, loc, st,
                          so);
    err |= launch_chained(k_seg_forward<F>, dim3(blocks(nthr)), dim3(THREADS), 0, s, d, w, (const F *)u,
                          (const F *)k, (const F *)v, st, (F *)y, ckpt);
    return err ? WKV_ERR_LAUNCH : WKV_OK;
}

template <typename F>
int par_bwd(Dims d, const float *w, const void *u, const void *k, const void *v, const float *si,
            const void *gy, const float *gso, float *gw, float *gu, void *gk, void *gv, float *gsi, float *ws,
            const float *ckpt, cudaStream_t s) {
    const size_t n3 = (size_t)d.B * d.nseg * 3 * d.C, n1 = (size_t)d.B * d.nseg * d.C;
    float *loc = ws, *stw = loc + n3, *rloc = stw + n3, *gend = rloc + n3, *gwp = gend + n3, *gup = gwp + n1;
    const long long nthr = (long long)d.B * d.nseg * d.C;
    const unsigned nb = blocks(nthr), nc = blocks((long long)d.B * d.C);
    int err = WKV_OK;
    if constexpr (sizeof(F) >= 2) {
        if (ckpt && d.C % 2 == 0) {      // tile checkpoints and a channel pair per thread
            const unsigned nb2 = blocks(nthr / 2);
            err |= launch_chained(k_seg_backward_ck2<F, false>, dim3(nb2), dim3(THREADS), 0, s, d, w, (const F *)u,
                                  (const F *)k, (const F *)v, (const F *)gy, ckpt, nullptr, rloc, nullptr, nullptr,
                                  nullptr, nullptr);
            err |= launch_chained(k_seg_rscan, dim3(nc), dim3(THREADS), 0, s, d, w, gso, rloc, gend, gsi);
            err |= launch_chained(k_seg_backward_ck2<F, true>, dim3(nb2), dim3(THREADS), 0, s, d, w, (const F *)u,
                                  (const F *)k, (const F *)v, (const F *)gy, ckpt, gend, nullptr, (F *)gk, (F *)gv,
                                  gwp, gup);
            err |= launch_chained(k_seg_reduce, dim3(nc), dim3(THREADS), 0, s, d, gwp, gup, gw, gu);
            return err ? WKV_ERR_LAUNCH : WKV_OK;
        }
    }
    if (ckpt) {
        // the forward call left its tile checkpoints: neither pass needs a forward sweep
        err |= launch_chained(k_seg_backward_ck<F, false>, dim3(nb), dim3(THREADS), 0, s, d, w, (const F *)u,
                              (const F *)k, (const F *)v, (const F *)gy, ckpt, nullptr, rloc, nullptr, nullptr,
                              nullptr, nullptr);
        err |= launch_chained(k_seg_rscan, dim3(nc), dim3(THREADS), 0, s, d, w, gso, rloc, gend, gsi);
        err |= launch_chained(k_seg_backward_ck<F, true>, dim3(nb), dim3(THREADS), 0, s, d, w, (const F *)u,
                              (const F *)k, (const F *)v, (const F *)gy, ckpt, gend, nullptr, (F *)gk, (F *)gv, gwp,
                              gup);
    } else {
        // rebuild the piece-start states, then the two passes with their own forward sweeps
        err |= launch_chained(k_seg_summary<F>, dim3(nb), dim3(THREADS), 0, s, d, w, (const F *)k, (const F *)v,
                              loc);
        err |= launch_chained(k_seg_scan, dim3(nc), dim3(THREADS), 0, s, d, w, si, loc, stw, nullptr);
        err |= launch_chained(k_seg_backward<F, false>, dim3(nb), dim3(THREADS), 0, s, d, w, (const F *)u,
                              (const F *)k, (const F *)v, (const F *)gy, stw, nullptr, rloc, nullptr, nullptr,
                              nullptr, nullptr);
        err |= launch_chained(k_seg_rscan, dim3(nc), dim3(THREADS), 0, s, d, w, gso, rloc, gend, gsi);
        err |= launch_chained(k_seg_backward<F, true>, dim3(nb), dim3(THREADS), 0, s, d, w, (const F *)u,
                              (const F *)k, (const F *)v, (const F *)gy, stw, gend, nullptr, (F *)gk, (F *)gv, gwp,
                              gup);
    }
    err |= launch_chained(k_seg_reduce, dim3(nc), dim3(THREADS), 0, s, d, gwp, gup, gw, gu);
    return err ? WKV_ERR_LAUNCH : WKV_OK;
}

}  // namespace

size_t v4_par_forward_workspace(int B, int T, int C) {
    const size_t nseg = (size_t)(T + SEG - 1) / SEG;
    return 2 * (size_t)B * nseg * 3 * C * sizeof(float);
}
size_t v4_par_backward_workspace(int B, int T, int C) {
    const size_t nseg = (size_t)(T + SEG - 1) / SEG;
    return (4 * 3 + 2) * (size_t)B * nseg * C * sizeof(float);
}

size_t v4_par_ckpt_bytes(int B, int T, int C) {
    return (size_t)B * ((T + SEG - 1) / SEG) * NCK * 5 * C * sizeof(float);
}

int v4_par_forward(int B, int T, int C, int dtype, const float *w, const void *u, const void *k, const void *v,
                   const float *si, void *y, float *so, float *ws, float *ckpt, cudaStream_t s) {
    const Dims d{B, T, C, (T + SEG - 1) / SEG};
    switch (dtype) {
        case WKV_F32: return par_fwd<float>(d, w, u, k, v, si, y, so, ws, ckpt, s);
        case WKV_BF16: return par_fwd<__nv_bfloat16>(d, w, u, k, v, si, y, so, ws, ckpt, s);
        case WKV_F16: return par_fwd<__half>(d, w, u, k, v, si, y, so, ws, ckpt, s);
    }
    return WKV_ERR_DTYPE;
}

int v4_par_backward(int B, int T, int C, int dtype, const float *w, const void *u, const void *k, const void *v,
                    const float *si, const void *gy, const float *gso, float *gw, float *gu, void *gk, void *gv,
                    float *gsi, float *ws, const float *ckpt, cudaStream_t s) {
    const Dims d{B, T, C, (T + SEG - 1) / SEG};
    switch (dtype) {
        case WKV_F32: return par_bwd<float>(d, w, u, k, v, si, gy, gso, gw, gu, gk, gv, gsi, ws, ckpt, s);
        case WKV_BF16: return par_bwd<__nv_bfloat16>(d, w, u, k, v, si, gy, gso, gw, gu, gk, gv, gsi, ws, ckpt, s);
        case WKV_F16: return par_bwd<__half>(d, w, u, k, v, si, gy, gso, gw, gu, gk, gv, gsi, ws, ckpt, s);
    }
    return WKV_ERR_DTYPE;
}

}  // namespace wkv
