// Shared pieces of the chunked tensor-core WKV kernels: tile helpers and the per-chunk
// decay bookkeeping (cumulative log-decay and the reference points that keep every
// operand scale factor inside the bf16/fp32 exponent range).
#pragma once
#include "sm100_primitives.cuh"
#include "tma_host.cuh"
#include "wkv_common.cuh"

namespace wkv {
namespace chunked {

using namespace sm100;

constexpr int CH = 64;            // tokens per chunk
constexpr int HB = 32;            // tokens per block
constexpr float LW_FLOOR = -5.298317367f;  // log(0.005)

struct __align__(16) Tile { unsigned char b[TILE_BYTES]; };

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void unpack8(const uint4 &q, float *f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float *f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
__device__ __forceinline__ uint4 ld_tile(const Tile &t, int row, int chunk) {
    return *reinterpret_cast<const uint4 *>(t.b + tile_off(row, chunk));
}
__device__ __forceinline__ void st_tile(Tile &t, int row, int chunk, const uint4 &v) {
    *reinterpret_cast<uint4 *>(t.b + tile_off(row, chunk)) = v;
}

// ---------------------------------------------------------------------------
// Per-chunk operand preparation.  Thread layout (128 threads): 16-byte column
// `cc` = 2*warp + (lane>>4) (8 channels), token group tg = lane & 15 (4 tokens).
// Everything a thread computes concerns tokens 4*tg..4*tg+3 of channels 8*cc..+7.
struct Prep {
    float c[4][8];    // inclusive cumulative log-decay
    float lw[4][8];   // per-token log-decay (floored), 0 for tokens past the segment end
    float m0[8], m1[8], e0[8], e1[8];
};

// lw filled by the caller; computes the chunk-wide cumulative sums by a local scan
// plus a 16-lane segmented warp scan, then the four reference values.
__device__ __forceinline__ void prep_scan(Prep &p, int lane) {
    const int tg = lane & 15;
#pragma unroll
    for (int ch = 0; ch < 8; ch++) {
        p.c[0][ch] = p.lw[0][ch];
#pragma unroll
        for (int i = 1; i < 4; i++) p.c[i][ch] = p.c[i - 1][ch] + p.lw[i][ch];
        float tot = p.c[3][ch];
#pragma unroll
        for (int off = 1; off < 16; off <<= 1) {
            const float o = __shfl_up_sync(0xffffffffu, tot, off, 16);
            if (tg >= off) tot += o;
        }
        const float excl = tot - p.c[3][ch];
#pragma unroll
        for (int i = 0; i < 4; i++) p.c[i][ch] += excl;
        // inclusive sums at tokens 15, 31, 47, 63 live in lanes tg = 3, 7, 11, 15
        p.m0[ch] = __shfl_sync(0xffffffffu, p.c[3][ch], 3, 16);
        p.e0[ch] = __shfl_sync(0xffffffffu, p.c[3][ch], 7, 16);
        p.m1[ch] = __shfl_sync(0xffffffffu, p.c[3][ch], 11, 16);
        p.e1[ch] = __shfl_sync(0xffffffffu, p.c[3][ch], 15, 16);
    }
}


}  // namespace chunked

// chunk-start states of a segment as bf16 [B*H, nchunk+1, 64, 64] (key rows, value columns),
// written by the forward kernel; y is not produced when `y` in `a` is NULL
int chunked_forward_impl(const wkv_args_t *a, bool per_token_w, void *state_ckpt, cudaStream_t s);

}  // namespace wkv
