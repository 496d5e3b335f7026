// Chunked tensor-core kernels for the v5/v6 WKV recurrence (bf16 I/O, fp32 state).
//
// Time is cut into chunks of 64 tokens, each chunk into two blocks of 32.  With
// c_t the inclusive running sum of the log-decay inside a chunk and cp_t = c_{t-1}:
//   scores  A[t,s] = sum_k r_t[k] k_s[k] e^{cp_t[k]-c_s[k]}  (s<t),  A[t,t] = sum_k r_t u k_t
//   y       = A V + (r e^{cp}) S_in
//   S_out   = diag(e^{c_63}) S_in + (k e^{c_63-c})^T V
// (the chunked form of RWKV-v6/src/module/rwkv_inner.py:48-113).  Every factor that
// multiplies an MMA operand is kept inside the bf16/fp32 exponent range: pairs inside
// a 32-token block are factored around the block's midpoint (as rwkv_inner.py:88-90
// does for its 128-token chunks in fp64), pairs across the two blocks around the end
// of the first block (both factors <= 1).  For that to hold for any input the decay
// is floored at 0.005 -- the floor rwkv_inner.py:40-45 applies.
//
// All contractions run on tcgen05.mma (M=64, bf16 operands in 128-byte-swizzled
// shared-memory tiles, fp32 accumulators in tensor memory); input tiles arrive by
// TMA; the fp32 state lives in tensor memory for the whole segment.
#include <cstdlib>

#include "wkv56_chunked.cuh"

namespace wkv {
namespace {

using namespace sm100;
using namespace chunked;

// ---------------------------------------------------------------------------
// Forward: one CTA per (batch, head), serial over the chunks of the segment.
struct FwdSmem {
    Tile in[2][4];     // per stage: r, k, v, w  (r,k,w are overwritten in place by
                       // r*fr, k*fk, r*e^{cp})
    Tile x, khat[2], atil, sbf;   // khat is double-buffered: chunk j+1 is prepared while the
                                  // state update of chunk j still reads khat of chunk j
    float dpart[8][CH];
    float dvec[CH];
    float btot[2][CH];     // log2-decay total of each 32-token block, per channel
    uint64_t load_bar[2];
    uint64_t mma_bar;
    uint32_t tmem_base;
};

struct FwdParams {
    int T, H, nchunk, layout, w_kind, state_only;
    const __nv_bfloat16 *u;
    const float *wvec;        // v5: per-channel decay parameter [H*64]
    const float *state_in;
    float *state_out;
    __nv_bfloat16 *y;
    __nv_bfloat16 *ckpt;      // [B,H,nchunk+1,64,64] chunk-start states, or NULL
    float *dchunk;            // [B*H,nchunk,64] decay of each whole chunk, or NULL; with it the
                              // kernel also stores r e^{cp} of every chunk through map_rh
    int *status;
    long long *timeline;      // optional debug aid: clock stamps of one mid-sequence step of one CTA
};

// Tensor-memory columns.  An M=64 accumulator fills lanes 0..15 of each 32-lane quarter ("lo");
// a second one can sit in lanes 16..31 ("hi") of the same columns, which lets both halves of a
// warp work on one token row: score columns 0..31 / y columns 0..31 in lo, 32..63 in hi.
//   S       lo   0.. 31   state[key, value 0..31]      hi  0.. 31   state[key, value 32..63]
//   A1a     lo  32.. 63   same-block scores, columns (s) 0..31
//   A2      lo  64.. 95   cross-block scores (rows 32..63, columns 0..31)
//   A1b     hi  64.. 95   same-block scores, columns (s) 32..63
//   Y       lo  96..127   y[:, 0..31]                  hi 96..127   y[:, 32..63]
enum { COL_S = 0, COL_A1A = 32, COL_A2 = 64, COL_Y = 96, FWD_TMEM_COLS = 128 };

template <bool PER_TOKEN>
__global__ void __launch_bounds__(128, 2)
k_chunk_fwd(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_w,
            const __grid_constant__ CUtensorMap map_rh, const FwdParams P) {
    extern __shared__ unsigned char smem_raw[];
    FwdSmem &s = *reinterpret_cast<FwdSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int bh = blockIdx.x, b = bh / P.H, h = bh % P.H, C = P.H * 64;
    const bool active = (lane & 16) == 0;          // lo half-warp: owns an accumulator row in lanes 0..15
    const int row = warp * 16 + (lane & 15);       // that row
    const uint32_t lane_base = (uint32_t)(warp * 32);
    // operand-pass coordinates (see wkv56_chunked.cuh)
    const int blk = warp >> 1, cc = 4 * (warp & 1) + (lane & 3), tgl = lane >> 2, tok0 = 32 * blk + 4 * tgl;
    const int n = P.nchunk;
    const bool full = P.state_only == 0;

    if (tid == 0) {
        mbar_init(&s.load_bar[0], 1); mbar_init(&s.load_bar[1], 1);
        mbar_init(&s.mma_bar, 4);   // lane 0 of every warp issues a share of each MMA group and commits
        fence_mbar_init();
        prefetch_tmap(&map_r); prefetch_tmap(&map_k); prefetch_tmap(&map_v);
        if (PER_TOKEN) prefetch_tmap(&map_w);
    }
    if (warp == 0) { tmem_alloc(&s.tmem_base, FWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s.tmem_base, tm_hi = tm + (16u << 16);

    auto issue_load = [&](int j) {
        const int st = j & 1;
        const uint32_t bytes = (PER_TOKEN ? 4 : 3) * TILE_BYTES;
        mbar_expect_tx(&s.load_bar[st], bytes);
        tma_load_3d(&s.in[st][0], &map_r, &s.load_bar[st], h * 64, j * CH, b);
        tma_load_3d(&s.in[st][1], &map_k, &s.load_bar[st], h * 64, j * CH, b);
        tma_load_3d(&s.in[st][2], &map_v, &s.load_bar[st], h * 64, j * CH, b);
        if (PER_TOKEN) tma_load_3d(&s.in[st][3], &map_w, &s.load_bar[st], h * 64, j * CH, b);
    };
    if (tid == 0 && n > 0) issue_load(0);

    // state -> tensor memory (row = key channel, column = value channel); tcgen05.ld/st are
    // warp-wide, lanes 16..31 of a warp touch the unused upper half of the quarter
    const size_t sbase = (size_t)bh * 64 * 64;
    const int vcol0 = active ? 0 : 32;             // value columns this thread holds of state row `row`
    {
        float v[32];
#pragma unroll
        for (int q = 0; q < 32; q++) {
            const int vc = vcol0 + q;
            const size_t idx = P.layout == WKV_STATE_KV ? (size_t)row * 64 + vc : (size_t)vc * 64 + row;
            v[q] = P.state_in ? P.state_in[sbase + idx] : 0.f;
        }
        tmem_st16(tmem_addr(tm, lane_base, COL_S), v);
        tmem_st16(tmem_addr(tm, lane_base, COL_S + 16), v + 16);
    }
    tmem_st_wait();

    // per-thread constants of the 8 channels this thread prepares
    float uu[8], lwc[8];
    {
        const uint4 q = *reinterpret_cast<const uint4 *>(P.u + h * 64 + cc * 8);
        unpack8(q, uu);
        if (!PER_TOKEN) {
#pragma unroll
            for (int ch = 0; ch < 8; ch++) {
                bool live;
                lwc[ch] = log2_decay(P.wvec[h * 64 + cc * 8 + ch], P.w_kind, live);
            }
        }
    }

    // Operand pass for chunk j: scaled r/k tiles in place in stage j&1, x, khat[j&1], the
    // score-diagonal partials and the chunk decay.  Contains one __syncthreads.
    auto prep = [&](int j) {
        Tile *in = s.in[j & 1];
        Tile &khat = s.khat[j & 1];
        float c[4][8];
        Decay D;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int t = tok0 + i;
            const bool valid = j * CH + t < P.T;
            if (PER_TOKEN) {
                float x[8];
                unpack8(ld_tile(in[3], t, cc), x);
#pragma unroll
                for (int ch = 0; ch < 8; ch++) {
                    bool live;
                    const float l2 = log2_decay(x[ch], P.w_kind, live);
                    c[i][ch] = valid ? l2 : 0.f;
                }
            } else {
#pragma unroll
                for (int ch = 0; ch < 8; ch++) c[i][ch] = valid ? lwc[ch] : 0.f;
            }
        }
        decay_scan(c, lane, D);
        if (tgl == 7) {
#pragma unroll
            for (int ch = 0; ch < 8; ch++) s.btot[blk][cc * 8 + ch] = D.e[ch];
        }
        __syncthreads();
        float other[8];          // 2^{total of the other block}
#pragma unroll
        for (int ch = 0; ch < 8; ch++) other[ch] = exp2f(s.btot[blk ^ 1][cc * 8 + ch]);
        if (blk == 0 && tgl == 7) {
#pragma unroll
            for (int ch = 0; ch < 8; ch++) {
                const float d = exp2f(D.e[ch]) * other[ch];
                s.dvec[cc * 8 + ch] = d;
                if (P.dchunk) P.dchunk[((size_t)bh * n + j) * 64 + cc * 8 + ch] = d;
            }
        }
        // r-side operands, walking forward over the thread's tokens:
        //   fa = 2^{cp - m};  fb = 2^{cp}   (cp counted from the block start)
        //   block 0: rhat = r fb                 block 1: x = r fb, rhat = x 2^{total of block 0}
        float fa[8], fb[8];
#pragma unroll
        for (int ch = 0; ch < 8; ch++) {
            fa[ch] = exp2f(D.cp0[ch] - D.m[ch]);
            fb[ch] = exp2f(D.cp0[ch]);
        }
        if (full) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = tok0 + i;
                float r[8], k[8], rt[8], rh[8], xx[8];
                unpack8(ld_tile(in[0], t, cc), r);
                unpack8(ld_tile(in[1], t, cc), k);
                float dsum = 0.f;
#pragma unroll
                for (int ch = 0; ch < 8; ch++) {
                    rt[ch] = r[ch] * fa[ch];
                    xx[ch] = r[ch] * fb[ch];
                    rh[ch] = blk ? xx[ch] * other[ch] : xx[ch];
                    dsum += r[ch] * uu[ch] * k[ch];
                    fa[ch] *= D.w[i][ch];
                    fb[ch] *= D.w[i][ch];
                }
                st_tile(in[0], t, cc, pack8(rt));
                st_tile(in[3], t, cc, pack8(rh));
                if (blk) st_tile(s.x, t, cc, pack8(xx));
                s.dpart[cc][t] = dsum;
            }
        } else if (P.dchunk) {
            // state-only pass on behalf of a backward call: r e^{cp} alone
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = tok0 + i;
                float r[8], rh[8];
                unpack8(ld_tile(in[0], t, cc), r);
#pragma unroll
                for (int ch = 0; ch < 8; ch++) {
                    const float xx = r[ch] * fb[ch];
                    rh[ch] = blk ? xx * other[ch] : xx;
                    fb[ch] *= D.w[i][ch];
                }
                st_tile(in[3], t, cc, pack8(rh));
            }
        }
        // k-side operands, walking backward:
        //   fa = 2^{m - c};  fb = 2^{e - c}   (e = total of the thread's block)
        //   block 0: x = k fb, khat = x 2^{total of block 1}      block 1: khat = k fb
#pragma unroll
        for (int ch = 0; ch < 8; ch++) {
            fa[ch] = exp2f(D.m[ch] - D.c3[ch]);
            fb[ch] = exp2f(D.e[ch] - D.c3[ch]);
        }
#pragma unroll
        for (int i = 3; i >= 0; i--) {
            const int t = tok0 + i;
            float k[8], kt[8], kh[8], xx[8];
            unpack8(ld_tile(in[1], t, cc), k);
#pragma unroll
            for (int ch = 0; ch < 8; ch++) {
                kt[ch] = k[ch] * fa[ch];
                xx[ch] = k[ch] * fb[ch];
                kh[ch] = blk ? xx[ch] : xx[ch] * other[ch];
                fa[ch] *= D.w[i][ch];
                fb[ch] *= D.w[i][ch];
            }
            if (full) {
                st_tile(in[1], t, cc, pack8(kt));
                if (!blk) st_tile(s.x, t, cc, pack8(xx));
            }
            st_tile(khat, t, cc, pack8(kh));
        }
    };

    uint32_t mma_phase = 0;
    int fail = 0;        // a bounded wait ran out (carried through the next barrier)
    int aborted = 0;
    int issued = n > 0 ? 0 : -1, landed = -1;   // TMA loads issued / seen complete

    // prologue: operands of chunk 0
    if (n > 0) {
        if (mbar_wait(&s.load_bar[0], 0)) landed = 0; else fail = 1;
        prep(0);
        if (n > 1) {
            if (tid == 0) issue_load(1);
            issued = 1;
        }
    }
    fence_async_smem();
    tc_fence_before();
    if (__syncthreads_or(fail)) aborted = 1;

    // Software pipeline: while the tensor core runs y/state of chunk j, the CUDA cores prepare
    // the operands of chunk j+1.
    for (int j = 0; j < n && !aborted; j++) {
        const int st = j & 1;
        Tile *in = s.in[st];
        const bool stamp = P.timeline != nullptr && tid == 0 && blockIdx.x == gridDim.x / 2 && j == n / 2;
        if (stamp) P.timeline[0] = clock64();
        // r e^{cp} of this chunk goes out for the backward pass (read again by the state product below)
        if (tid == 0 && P.dchunk) {
            tma_store_3d(&map_rh, &in[3], h * 64, j * CH, b);
            tma_store_commit();
        }

        // (A) scores: A1 = Rt Kt^T (same-block halves), A2 = X X[0:32]^T.  A tcgen05.mma is
        // issued by one thread and costs it ~100 cycles of descriptor arithmetic, so the three
        // accumulators go out from three warps at once; every warp's lane 0 commits.
        if (lane == 0 && full) {
            tc_fence_after();
            const uint32_t id32 = make_idesc(64, 32, false, false);
            if (warp == 0) {
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(tm + COL_A1A, desc_kmajor(&in[0], 0, k), desc_kmajor(&in[1], 0, k), id32, k > 0);
            } else if (warp == 1) {
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(tm_hi + COL_A2, desc_kmajor(&in[0], 0, k), desc_kmajor(&in[1], 32, k), id32, k > 0);
            } else if (warp == 2) {
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(tm + COL_A2, desc_kmajor(&s.x, 0, k), desc_kmajor(&s.x, 0, k), id32, k > 0);
            }
            mma_commit(&s.mma_bar);
        }
        // (B) meanwhile: snapshot the state as bf16 (operand of rhat*S, checkpoint) and decay it;
        // each half-warp holds 32 of the 64 value columns of its state row
        {
            float v[32];
            tmem_ld16(tmem_addr(tm, lane_base, COL_S), v);
            tmem_ld16(tmem_addr(tm, lane_base, COL_S + 16), v + 16);
            tmem_ld_wait();
            const float d = s.dvec[row];
            uint4 q[4];
#pragma unroll
            for (int c8 = 0; c8 < 4; c8++) {
                q[c8] = pack8(v + 8 * c8);
                st_tile(s.sbf, row, (vcol0 >> 3) + c8, q[c8]);
            }
            if (P.ckpt) {
                uint4 *dst = reinterpret_cast<uint4 *>(P.ckpt + (((size_t)bh * (n + 1) + j) * 64 + row) * 64 + vcol0);
#pragma unroll
                for (int c8 = 0; c8 < 4; c8++) dst[c8] = q[c8];
            }
#pragma unroll
            for (int c = 0; c < 32; c++) v[c] *= d;
            tmem_st16(tmem_addr(tm, lane_base, COL_S), v);
            tmem_st16(tmem_addr(tm, lane_base, COL_S + 16), v + 16);
        }
        tmem_st_wait();
        if (stamp) P.timeline[1] = clock64();
        // (C) mask pass: lo lanes own columns 0..31 of token row t, hi lanes columns 32..63
        if (full) {
            if (!mbar_wait(&s.mma_bar, mma_phase)) fail = 1;
            mma_phase ^= 1;
            tc_fence_after();
            const int t = row;
            const int col0 = active ? 0 : 32;
            float a[32];
            // rows 0..31 (warps 0,1): A1a for the lo half, nothing to read for the hi half;
            // rows 32..63 (warps 2,3): A2 (lo) and A1b (hi) share their columns
            const int src = warp < 2 ? COL_A1A : COL_A2;
            tmem_ld16(tmem_addr(tm, lane_base, src), a);
            tmem_ld16(tmem_addr(tm, lane_base, src + 16), a + 16);
            tmem_ld_wait();
            float diag = 0.f;
#pragma unroll
            for (int q = 0; q < 8; q++) diag += s.dpart[q][t];
            const bool cross = t >= HB && active;          // A2 block: every entry is kept
            const bool empty = t < HB && !active;          // upper-right block: all zero
#pragma unroll
            for (int q = 0; q < 32; q++) {
                const int sx = col0 + q;
                float val = a[q];
                if (!cross) val = sx < t ? val : (sx == t ? diag : 0.f);
                if (empty) val = 0.f;
                a[q] = val;
            }
#pragma unroll
            for (int c8 = 0; c8 < 4; c8++) st_tile(s.atil, t, (col0 >> 3) + c8, pack8(a + 8 * c8));
        }
        if (stamp) P.timeline[2] = clock64();
        fence_async_smem();
        tc_fence_before();
        if (__syncthreads_or(fail)) { aborted = 1; break; }

        // (D) y = Atil V + Rhat Sbf (value columns 0..31 -> lo lanes, 32..63 -> hi lanes) ;
        //     S = d*S + Khat^T V
        if (lane == 0) {
            tc_fence_after();
            if (warp < 2 && full) {
                const uint32_t id_km32 = make_idesc(64, 32, false, true);
                const uint32_t d = (warp ? tm_hi : tm) + COL_Y;
                const uint64_t off = warp ? 4 : 0;   // +64 bytes along the contiguous dim
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(d, desc_kmajor(&s.atil, 0, k), desc_mnmajor(&in[2], 0, k) + off, id_km32, k > 0);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(d, desc_kmajor(&in[3], 0, k), desc_mnmajor(&s.sbf, 0, k) + off, id_km32, true);
            } else if (warp >= 2) {
                const uint32_t id_mm32 = make_idesc(64, 32, true, true);
                const uint32_t d = (warp == 3 ? tm_hi : tm) + COL_S;
                const uint64_t off = warp == 3 ? 4 : 0;
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(d, desc_mnmajor(&s.khat[st], 0, k), desc_mnmajor(&in[2], 0, k) + off, id_mm32, true);
            }
            mma_commit(&s.mma_bar);
        }
        if (stamp) P.timeline[3] = clock64();
        // (E) operands of the next chunk while the tensor core works
        if (j + 1 < n) {
            if (mbar_wait(&s.load_bar[(j + 1) & 1], (uint32_t)(((j + 1) >> 1) & 1))) landed = j + 1; else fail = 1;
            prep(j + 1);
        }
        if (stamp) P.timeline[4] = clock64();
        // (F) y of this chunk
        if (!mbar_wait(&s.mma_bar, mma_phase)) fail = 1;
        mma_phase ^= 1;
        tc_fence_after();
        if (stamp) P.timeline[5] = clock64();
        if (full) {
            const int t = j * CH + row;
            float yv[32];
            tmem_ld16(tmem_addr(tm, lane_base, COL_Y), yv);
            tmem_ld16(tmem_addr(tm, lane_base, COL_Y + 16), yv + 16);
            tmem_ld_wait();
            if (t < P.T) {
                uint4 *dst = reinterpret_cast<uint4 *>(P.y + ((size_t)b * P.T + t) * C + h * 64 + (active ? 0 : 32));
#pragma unroll
                for (int c8 = 0; c8 < 4; c8++) dst[c8] = pack8(yv + 8 * c8);
            }
        }
        if (stamp) P.timeline[6] = clock64();
        fence_async_smem();
        tc_fence_before();
        if (__syncthreads_or(fail)) { aborted = 1; break; }
        // stage j&1 is free now (its last reader was the MMA group that just completed)
        if (j + 2 < n) {
            if (tid == 0) {
                tma_store_wait_read();     // the store above has read its tile of this stage
                issue_load(j + 2);
            }
            issued = j + 2;
        }
        if (stamp) P.timeline[7] = clock64();
    }

    // after a failed wait: let TMA loads that were issued land (bounded), so that the CTA
    // never exits under one
    if (aborted) {
        for (int q = landed + 1; q <= issued; q++) mbar_wait(&s.load_bar[q & 1], (uint32_t)((q >> 1) & 1));
    }
    tc_fence_after();
    {
        float v[32];
        tmem_ld16(tmem_addr(tm, lane_base, COL_S), v);
        tmem_ld16(tmem_addr(tm, lane_base, COL_S + 16), v + 16);
        tmem_ld_wait();
        if (!aborted && P.state_out) {
#pragma unroll
            for (int q = 0; q < 32; q++) {
                const int vc = vcol0 + q;
                const size_t idx = P.layout == WKV_STATE_KV ? (size_t)row * 64 + vc : (size_t)vc * 64 + row;
                P.state_out[sbase + idx] = v[q];
            }
        }
        if (!aborted && P.ckpt) {
            uint4 *dst = reinterpret_cast<uint4 *>(P.ckpt + (((size_t)bh * (n + 1) + n) * 64 + row) * 64 + vcol0);
#pragma unroll
            for (int c8 = 0; c8 < 4; c8++) dst[c8] = pack8(v + 8 * c8);
        }
    }
    if (aborted && P.status && tid == 0) atomicOr(P.status, 1);
    if (tid == 0) tma_store_wait_read();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tm, FWD_TMEM_COLS);
}

static_assert(sizeof(FwdSmem) + 1024 <= 115712, "two CTAs per SM need <= 113 KiB each");

}  // namespace

// ---------------------------------------------------------------------------
// host side

bool chunked_supported(const wkv_args_t *a, bool per_token_w) {
    if (a->dtype != WKV_BF16 || a->N != 64 || a->T <= 0) return false;
    if (per_token_w && a->w_kind != WKV_W_RAW) return false;  // fp32 ew tensor: scalar path
    return true;
}

// workspace layout: [0,256) status words ; then what the call needs
size_t chunked_forward_workspace(const wkv_args_t *, bool) { return 256; }

int chunked_forward_impl(const wkv_args_t *a, bool per_token_w, void *state_ckpt, cudaStream_t stream) {
    const int B = a->B, T = a->T, H = a->H, C = H * 64;
    CUtensorMap mr, mk, mv, mw;
    if (!make_btc_map(&mr, a->r, B, T, C) || !make_btc_map(&mk, a->k, B, T, C) ||
        !make_btc_map(&mv, a->v, B, T, C))
        return WKV_ERR_LAUNCH;
    if (per_token_w) {
        if (!make_btc_map(&mw, a->w, B, T, C)) return WKV_ERR_LAUNCH;
    } else {
        mw = mr;
    }
    FwdParams p;
    p.T = T; p.H = H; p.nchunk = (T + CH - 1) / CH; p.layout = a->state_layout; p.w_kind = a->w_kind;
    p.state_only = a->y == nullptr;
    p.u = (const __nv_bfloat16 *)a->u;
    p.wvec = per_token_w ? nullptr : (const float *)a->w;
    p.state_in = a->state_in; p.state_out = a->state_out;
    p.y = (__nv_bfloat16 *)a->y;
    const CkptLayout CL = ckpt_layout(B, T, H);
    CUtensorMap mrh = mr;
    p.ckpt = nullptr; p.dchunk = nullptr;
    if (state_ckpt) {
        char *ck = (char *)state_ckpt;
        p.ckpt = (__nv_bfloat16 *)(ck + CL.sck);
        p.dchunk = (float *)(ck + CL.dchunk);
        if (!make_btc_map(&mrh, ck + CL.rhat, B, T, C)) return WKV_ERR_LAUNCH;
    }
    p.status = (int *)a->workspace;
    p.timeline = getenv("WKV_B200_TIMELINE") ? (long long *)((char *)a->workspace + 64) : nullptr;
    const size_t smem = sizeof(FwdSmem) + 1024;
    auto kern = per_token_w ? k_chunk_fwd<true> : k_chunk_fwd<false>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return WKV_ERR_LAUNCH;
    kern<<<B * H, 128, smem, stream>>>(mr, mk, mv, mw, mrh, p);
    return launch_status();
}

int chunked_forward(const wkv_args_t *a, bool per_token_w, cudaStream_t stream) {
    if (cudaMemsetAsync(a->workspace, 0, 256, stream) != cudaSuccess) return WKV_ERR_LAUNCH;
    return chunked_forward_impl(a, per_token_w, a->state_ckpt, stream);
}

}  // namespace wkv
