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
// Per-chunk decay bookkeeping.  Thread layout of the operand passes (128 threads):
//   warp  = 2*blk + cch     blk: which 32-token block of the chunk, cch: upper/lower 4
//                           of the 8 16-byte columns of a tile row
//   lane  = 4*tgl + ccl     tgl: group of 4 consecutive tokens inside the block (0..7),
//                           ccl: column inside the group of 4
// so a thread owns tokens 32*blk + 4*tgl .. +3 of channels 8*(4*cch+ccl) .. +7.  With the
// 128-byte swizzle every 8 consecutive lanes then touch 8 different 16-byte bank groups:
// the tile loads and stores are free of bank conflicts.
//
// All decay arithmetic is done in the log2 domain (one ex2 per exponential, no
// extra multiply): l2 = log2(decay) per token, c = running sum of l2 from the start
// of the thread's block, cp = c - l2.  Scale factors of neighbouring tokens differ by
// exactly one token's decay, so a thread evaluates one exponential per factor
// for its first (or last) token and walks to the others by multiplying with the
// per-token decay w = 2^{l2}.  Everything a block needs from the other block is that
// block's total, exchanged through shared memory.
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float L2_FLOOR = LW_FLOOR * LOG2E;

// log2 of the (floored) decay from the two encodings of the decay tensor; `live` tells
// whether the decay is above the floor (the floor passes no gradient)
__device__ __forceinline__ float log2_decay(float x, int w_kind, bool &live) {
    const float l2 = w_kind == WKV_W_RAW ? -exp2f(x * LOG2E) * LOG2E : x * LOG2E;
    live = l2 >= L2_FLOOR;
    return fmaxf(l2, L2_FLOOR);
}

template <int NCH>
struct DecayT {
    float w[4][NCH];   // decay of each of the thread's 4 tokens (1 past the segment end)
    float cp0[NCH];    // log2-decay accumulated from the block start to before the thread's first token
    float c3[NCH];     // ... up to and including its last token
    float m[NCH];      // ... up to and including token 15 of the block (the block midpoint reference)
    float e[NCH];      // the whole block
};
using Decay = DecayT<8>;

// In: l2[i][ch] per-token log2-decay.  Out: l2 holds the block-local inclusive sums c
// (local scan + scan over the 8 threads that share a column, which sit 4 lanes apart).
template <int NCH>
__device__ __forceinline__ void decay_scan(float (&l2)[4][NCH], int lane, DecayT<NCH> &D) {
    const int tgl = lane >> 2, ccl = lane & 3;
#pragma unroll
    for (int ch = 0; ch < NCH; ch++) {
#pragma unroll
        for (int i = 0; i < 4; i++) D.w[i][ch] = exp2f(l2[i][ch]);
        const float first = l2[0][ch];
#pragma unroll
        for (int i = 1; i < 4; i++) l2[i][ch] += l2[i - 1][ch];
        float tot = l2[3][ch];
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) {
            const float o = __shfl_up_sync(0xffffffffu, tot, 4 * off);
            if (tgl >= off) tot += o;
        }
        const float excl = tot - l2[3][ch];
#pragma unroll
        for (int i = 0; i < 4; i++) l2[i][ch] += excl;
        D.cp0[ch] = l2[0][ch] - first;
        D.c3[ch] = l2[3][ch];
        D.m[ch] = __shfl_sync(0xffffffffu, l2[3][ch], ccl + 12);   // tgl = 3: token 15 of the block
        D.e[ch] = __shfl_sync(0xffffffffu, l2[3][ch], ccl + 28);   // tgl = 7: token 31
    }
}

// Operand-pass layout for kernels with eight compute warps (256 threads):
//   warp w owns tokens 8w .. 8w+7 of the chunk (so warps 0..3 are block 0, warps 4..7 block 1);
//   lane = 16*r + 2*cc + hf:  tokens 8w + 4r .. +3,  channels 8*cc + 4*hf .. +3,
// i.e. a thread owns 4 tokens x 4 channels and reads or writes 8 bytes of a tile row at a time.
// The 16 lanes of a half-warp then cover one whole 128-byte row: free of bank conflicts.
//
// In: l2[i][ch] per-token log2-decay.  Out: l2 holds the block-local inclusive sums c; D as in
// decay_scan; other_l2 = log2-decay total of the other block.  The totals of the eight warps go
// through `wtot` ([8][CH] floats of shared memory); `sync(pred)` is the barrier of the 256 threads,
// returning the OR of `pred` over them.
//
// Returns true when the chunk is "mild": no 8 consecutive tokens decay by more than 2^-30 in any
// channel, so that the whole chunk can be factored around ONE reference point, the end of block 0
// (both halves then stay within 2^+-120), and the separate treatment of the pairs across the two
// blocks is not needed.
constexpr float MILD_L2_PER_8 = -30.f;
template <class Sync>
__device__ __forceinline__ bool decay_scan8(float (&l2)[4][4], int warp, int lane, float *wtot, DecayT<4> &D,
                                            float (&other_l2)[4], Sync sync) {
    const int r = lane >> 4, ch0 = (lane & 15) * 4, blk = warp >> 2, wb = warp & 3;
    float tot[4], first[4];
    bool steep = false;
#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
#pragma unroll
        for (int i = 0; i < 4; i++) D.w[i][ch] = exp2f(l2[i][ch]);
        first[ch] = l2[0][ch];
#pragma unroll
        for (int i = 1; i < 4; i++) l2[i][ch] += l2[i - 1][ch];
        const float o = __shfl_xor_sync(0xffffffffu, l2[3][ch], 16);
        tot[ch] = l2[3][ch] + o;
        steep |= tot[ch] < MILD_L2_PER_8;
        if (r) {
#pragma unroll
            for (int i = 0; i < 4; i++) l2[i][ch] += o;
        }
    }
    if (r) *reinterpret_cast<float4 *>(wtot + warp * CH + ch0) = make_float4(tot[0], tot[1], tot[2], tot[3]);
    const bool mild = !sync(steep);
    const float *own = wtot + 4 * blk * CH + ch0, *oth = wtot + 4 * (blk ^ 1) * CH + ch0;
    float base[4] = {0.f, 0.f, 0.f, 0.f}, m[4], e[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const float4 a4 = *reinterpret_cast<const float4 *>(own + q * CH);
        const float4 b4 = *reinterpret_cast<const float4 *>(oth + q * CH);
        const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            if (q == 0) { m[ch] = a[ch]; other_l2[ch] = b[ch]; }
            else if (q == 1) { m[ch] += a[ch]; e[ch] = m[ch]; other_l2[ch] += b[ch]; }     // m: through token 15 of the block
            else { e[ch] += a[ch]; other_l2[ch] += b[ch]; }                                // e: the whole block
            if (wb > q) base[ch] += a[ch];
        }
    }
#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
#pragma unroll
        for (int i = 0; i < 4; i++) l2[i][ch] += base[ch];
        D.cp0[ch] = l2[0][ch] - first[ch];
        D.c3[ch] = l2[3][ch];
        D.m[ch] = m[ch];
        D.e[ch] = e[ch];
    }
    return mild;
}

// The same quantities for a static per-channel decay (v5) and a chunk with all 64 tokens in range:
// every token of channel ch decays by lw[ch] (log2), so nothing has to be scanned or exchanged.
// w[ch] = 2^{lw[ch]}; tok0 = first of the thread's 4 tokens (0..63).
__device__ __forceinline__ void decay_static(const float (&lw)[4], const float (&w)[4], int tok0, float (&l2)[4][4],
                                             DecayT<4> &D, float (&other_l2)[4]) {
    const float t0 = (float)(tok0 & (HB - 1));
#pragma unroll
    for (int ch = 0; ch < 4; ch++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            D.w[i][ch] = w[ch];
            l2[i][ch] = (t0 + (float)(i + 1)) * lw[ch];
        }
        D.cp0[ch] = t0 * lw[ch];
        D.c3[ch] = l2[3][ch];
        D.m[ch] = 16.f * lw[ch];
        D.e[ch] = 32.f * lw[ch];
        other_l2[ch] = D.e[ch];
    }
}

// 8-byte halves of a 16-byte tile chunk (4 bf16)
__device__ __forceinline__ void unpack4(const uint2 &q, float *f) {
    f[0] = __uint_as_float(q.x << 16); f[1] = __uint_as_float(q.x & 0xFFFF0000u);
    f[2] = __uint_as_float(q.y << 16); f[3] = __uint_as_float(q.y & 0xFFFF0000u);
}
__device__ __forceinline__ uint2 pack4(const float *f) { return make_uint2(pack2(f[0], f[1]), pack2(f[2], f[3])); }
__device__ __forceinline__ uint2 ld_tile4(const Tile &t, int row, int chunk, int half) {
    return *reinterpret_cast<const uint2 *>(t.b + tile_off(row, chunk) + 8 * half);
}
__device__ __forceinline__ void st_tile4(Tile &t, int row, int chunk, int half, const uint2 &v) {
    *reinterpret_cast<uint2 *>(t.b + tile_off(row, chunk) + 8 * half) = v;
}

// What the forward kernel hands to the backward kernels (wkv_args_t.state_ckpt):
//   sck     bf16 [B*H, nchunk+1, 64, 64]  state at the start of every chunk (key rows, value columns)
//   rhat    bf16 [B, T, C]                r_t * (decay accumulated from the chunk start to before t)
//   dchunk  fp32 [B*H, nchunk, 64]        decay of each whole chunk per key channel
//   mild    u8   [B*H * nchunk]           1 = the chunk is mild (see decay_scan8), 0 = steep: which build of
//                                         the per-chunk backward kernel the chunk needs
struct CkptLayout {
    size_t sck, rhat, dchunk, mild, total;
};
inline CkptLayout ckpt_layout(int B, int T, int H) {
    const size_t n = (size_t)(T + CH - 1) / CH, bh = (size_t)B * H;
    auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
    CkptLayout L;
    L.sck = 0;
    L.rhat = al(bh * (n + 1) * 64 * 64 * 2);
    L.dchunk = L.rhat + al((size_t)B * T * H * 64 * 2);
    L.mild = L.dchunk + al(bh * n * 64 * 4);
    L.total = L.mild + al(bh * n);
    return L;
}

// Time groups (see the head of wkv56_chunked.cu): G groups of L consecutive chunks per chain.
struct GroupPlan {
    int G, L;
};
constexpr int SAVE_EVERY = 8;     // chunks between two saved fp32 states (wkv_args_t.group_states)
// requested: 0 = decide from the number of chains and the device's SM count, 1 = never split,
// > 1 = that many groups (at most one per chunk)
GroupPlan plan_groups(int BH, int nchunk, int requested);
GroupPlan plan_forward(const wkv_args_t *a);

// Scratch of the time-group passes, for `units` = chains * G (all fp32, state matrices [key,value]):
//   gU      [units, 64, 64]  what a group adds to the state (gradient) starting from zero
//   gD      [units, 64]      decay of the whole group per key channel
//   gstart  [units, 64, 64]  state (gradient) a group starts from
struct GroupLayout {
    size_t gU, gD, gstart, total;
};
GroupLayout group_layout(size_t units);
int launch_group_scan(const void *group_ws, int BH, int G, const float *init, float *final_out, int layout,
                      bool reverse, cudaStream_t stream);

}  // namespace chunked

// What only the wait-timeout self-test changes: how many polls a device-side wait makes before it
// gives up, and one TMA load that is deliberately never issued (kernel: 0 forward, 1 dS scan,
// 2 per-chunk backward; skip_load: local chunk / step index, -1 = none).
struct ChunkedTest {
    uint32_t wait_limit = 4000000u;
    int kernel = -1;
    int skip_load = -1;
};

int device_sm_count();
size_t chunked_group_states_bytes(const wkv_args_t *a);
// v6 with the fp32 ew = -exp(x) encoding: bytes of, and conversion into, a bf16 x tensor (a no-op otherwise)
size_t chunked_wconv_bytes(const wkv_args_t *a, bool per_token_w);
int chunked_convert_w(wkv_args_t *a, bool per_token_w, void *scratch, cudaStream_t s);
int selftest_wait(int *status, uint32_t limit, cudaStream_t s);

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device property of a kernel: set it on
// the first launch on each device only (`done` is the call site's own per-device record)
template <class K>
inline bool set_max_smem_once(K kern, int bytes, unsigned char (&done)[64]) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return false;
    if (dev >= 0 && dev < 64 && __atomic_load_n(&done[dev], __ATOMIC_ACQUIRE)) return true;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
    if (dev >= 0 && dev < 64) __atomic_store_n(&done[dev], (unsigned char)1, __ATOMIC_RELEASE);
    return true;
}

// `state_ckpt` (laid out as chunked::CkptLayout, or NULL) receives what the backward kernels
// reuse from the forward pass; y is not produced when `y` in `a` is NULL; `group_ws` is
// chunked::group_layout() bytes of scratch, used when the chains are split into time groups
int chunked_forward_impl(const wkv_args_t *a, bool per_token_w, void *state_ckpt, void *group_ws,
                         const ChunkedTest &tst, cudaStream_t s);
int chunked_forward(const wkv_args_t *a, bool per_token_w, const ChunkedTest &tst, cudaStream_t s);
int chunked_backward(const wkv_args_t *a, bool per_token_w, const ChunkedTest &tst, cudaStream_t s);

}  // namespace wkv
