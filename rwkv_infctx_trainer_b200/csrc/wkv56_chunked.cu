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
// TMA; the fp32 state is carried in registers by the compute warps (the tensor core
// only forms each chunk's own contribution to it).
//
// Time groups.  A segment's chunks are a serial chain per (batch, head).  When there are
// too few chains to fill the device the chain is cut into G groups of consecutive
// chunks and the forward runs as three launches:
//   A. per (chain, group), from a zero state: the group's own contribution U_g and the
//      decay d_g of the whole group (no y, no scores -- a "summary" pass);
//   B. k_group_scan: S_start[g+1] = d_g * S_start[g] + U_g, elementwise over the groups;
//   C. per (chain, group), from S_start[g]: the full pass.
// With G = 1 only C runs, from the caller's state.

#include "wkv56_chunked.cuh"

namespace wkv {
namespace {

using namespace sm100;
using namespace chunked;

// ---------------------------------------------------------------------------
// Forward: one CTA per (batch, head), serial over the chunks of the segment.
//
// Nine warps.  Warp 8 (one lane) feeds the machine: TMA loads, every tcgen05.mma, the TMA
// store of r e^{cp}.  Warps 0..7 do the CUDA-core work of a chunk -- operand pass, state
// update, mask pass, y epilogue -- and meet only on a named barrier of their own.  The fp32
// state lives in registers (thread = key row, 16 value columns); the tensor core forms only
// the chunk's own contribution U_j = khat_j^T V_j, which does not depend on the state, so the
// serial chain per chunk is one fused multiply-add per state element.
struct FwdSmem {
    Tile in[2][4];     // per stage: r, k, v, w  (r,k,w are overwritten in place by
                       // r*fr, k*fk, r*e^{cp})
    Tile x, khat[2], atil, sbf;   // khat is double-buffered: chunk j+1 is prepared while the
                                  // state product of chunk j may still read khat of chunk j
    float dpart[4][CH];    // score-diagonal partials per token
    float dvec[2][CH];     // decay of the whole chunk per key channel, by chunk parity
    float wtot[8][CH];     // log2-decay total of each warp's 8 tokens, per channel
    __align__(16) float uf[CH];   // the head's bonus u in fp32
    uint64_t load_bar[2];  // TMA: a stage has landed
    uint64_t ops_bar[2];   // compute warps -> feeder: the operands of a chunk are in place (by chunk parity:
                           // in a state-only pass the compute warps may run a chunk ahead of the feeder)
    uint64_t yrdy_bar;     // compute warps -> feeder: masked scores and bf16 state are in place
    uint64_t score_bar;    // tensor core: scores of a chunk
    uint64_t u_bar[2];     // tensor core: state product of a chunk, by chunk parity
    uint64_t y_bar;        // tensor core: y of a chunk
    uint32_t tmem_base;
    int abort_flag;        // set by any thread whose bounded wait ran out; ends every other wait
    int mild_flag[2];      // compute warps -> feeder, by chunk parity: the chunk is mild (see decay_scan8)
};

struct FwdParams {
    int T, H, nchunk, layout, w_kind;
    int G, L;                 // time groups per chain, chunks per group (the last group may be shorter)
    const __nv_bfloat16 *u;
    const float *wvec;        // v5: per-channel decay parameter [H*64]
    const float *state_in;    // G == 1: the caller's state (layout `layout`)
    const float *gstart;      // G > 1, pass C: [B*H*G, 64, 64] state at the start of every group ([key,value])
    float *state_out;         // written by the CTA whose group ends the segment
    float *gU;                // pass A: [B*H*G, 64, 64] state a group builds from zero ([key,value])
    float *gD;                // pass A: [B*H*G, 64] decay of a whole group per key channel
    float *gsave;             // or NULL: [B*H, ceil(nchunk/Lsave), 64, 64] fp32 state at the start of every
    int Lsave;                // Lsave-th chunk ([key,value]), for a later call that restarts from them
    __nv_bfloat16 *y;
    __nv_bfloat16 *ckpt;      // [B,H,nchunk+1,64,64] chunk-start states, or NULL
    float *dchunk;            // [B*H,nchunk,64] decay of each whole chunk, or NULL; with it the
                              // kernel also stores r e^{cp} of every chunk through map_rh
    unsigned char *mildflag;  // with dchunk: [B*H*nchunk], 1 = the chunk is mild
    int *status;
    uint32_t wait_limit;      // polls before a wait gives up
    int skip_load;            // -1; a local chunk index leaves that chunk's TMA load out (wait-timeout test)
};

// Tensor-memory columns.  An M=64 accumulator fills lanes 0..15 of each 32-lane quarter ("lo");
// a second one can sit in lanes 16..31 ("hi") of the same columns.
//   U[q]    lo  32q..32q+31  khat^T V [key, value 0..31]  hi: [key, value 32..63]   (q = chunk parity)
//   A1a     lo  64.. 95   same-block scores, columns (s) 0..31
//   A2      lo  96..127   cross-block scores (rows 32..63, columns 0..31)
//   A1b     hi  96..127   same-block scores, columns (s) 32..63
//   Y       lo 128..159   y[:, 0..31]                  hi 128..159   y[:, 32..63]
enum { COL_U = 0, COL_A1A = 64, COL_A2 = 96, COL_Y = 128, FWD_TMEM_COLS = 256 };
constexpr int FWD_THREADS = 288;

// barrier of the 256 compute threads that also ORs a predicate over them
__device__ __forceinline__ bool compute_sync_or(bool pred) {
    uint32_t any;
    asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, 1, 256, q;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(any) : "r"((uint32_t)pred) : "memory");
    return any != 0;
}
// barrier of the 256 compute threads
__device__ __forceinline__ void compute_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// MODE: what the launch is for (compiled separately so that the full pass does not carry the others' state)
enum { FWD_FULL = 0,      // y, state_out and, when asked for, the hand-over to the backward pass
       FWD_STATES = 1,    // backward without a hand-over: chunk-start states, r e^{cp}, chunk decays only
       FWD_SUMMARY = 2 }; // pass A of the time-group scheme
template <bool PER_TOKEN, int MODE>
__global__ void __launch_bounds__(FWD_THREADS, 2)
k_chunk_fwd(const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_k,
            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_w,
            const __grid_constant__ CUtensorMap map_rh, const FwdParams P) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles want a 1024-byte aligned base.  The padding is added to the __shared__ array
    // itself (not to an integer copy of its address), so the compiler still knows that everything
    // behind `s` is shared memory and uses shared-memory loads and stores for the tiles.
    FwdSmem &s = *reinterpret_cast<FwdSmem *>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // tells the compiler it is uniform across the warp
    // this CTA's group of chunks: global chunk index = j0 + local index, n of them
    // (grid: x = group, y = chain)
    const int grp = blockIdx.x, bh = blockIdx.y, unit = bh * P.G + grp;
    const int b = bh / P.H, h = bh % P.H, C = P.H * 64;
    const int j0 = grp * P.L, n = min(P.L, P.nchunk - j0);
    constexpr bool full = MODE == FWD_FULL, summary = MODE == FWD_SUMMARY;

    if (tid == 0) {
        mbar_init(&s.load_bar[0], 1); mbar_init(&s.load_bar[1], 1);
        mbar_init(&s.ops_bar[0], 1); mbar_init(&s.ops_bar[1], 1); mbar_init(&s.yrdy_bar, 1);
        mbar_init(&s.score_bar, 1); mbar_init(&s.u_bar[0], 1); mbar_init(&s.u_bar[1], 1); mbar_init(&s.y_bar, 1);
        s.abort_flag = 0;
        fence_mbar_init();
    }
    if (full && tid >= 64 && tid < 64 + CH) s.uf[tid - 64] = __bfloat162float(P.u[h * 64 + tid - 64]);
    if (warp == 0) { tmem_alloc(&s.tmem_base, FWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s.tmem_base, tm_hi = tm + (16u << 16);
    int fail = 0;

    if (warp == 8) {
        // ------------------------------------------------------------------ feeder
        if (lane == 0) {
            prefetch_tmap(&map_r); prefetch_tmap(&map_k); prefetch_tmap(&map_v);
            if (PER_TOKEN) prefetch_tmap(&map_w);
            // (local chunk c; P.skip_load names a chunk whose load is left out: the host-side fault
            // injection of the wait-timeout test, -1 in normal use)
            int issued = -1;
            auto issue_load = [&](int c) {
                if (c == P.skip_load) return;
                const int st = c & 1, t0 = (j0 + c) * CH;
                mbar_expect_tx(&s.load_bar[st], (PER_TOKEN ? 4 : 3) * TILE_BYTES);
                tma_load_3d(&s.in[st][0], &map_r, &s.load_bar[st], h * 64, t0, b);
                tma_load_3d(&s.in[st][1], &map_k, &s.load_bar[st], h * 64, t0, b);
                tma_load_3d(&s.in[st][2], &map_v, &s.load_bar[st], h * 64, t0, b);
                if (PER_TOKEN) tma_load_3d(&s.in[st][3], &map_w, &s.load_bar[st], h * 64, t0, b);
                issued = c;
            };
            for (int c = 0; c < 2 && c < n; c++) issue_load(c);
            // descriptors: a tile's descriptor plus (byte offset >> 4) addresses inside it
            const uint64_t d_x = make_desc(smem_u32(&s.x)), d_atil = make_desc(smem_u32(&s.atil)),
                           d_sbf = make_desc(smem_u32(&s.sbf));
            constexpr uint64_t KSTEP = 32 >> 4;            // K-major: 16 elements along the row
            constexpr uint64_t MSTEP = (16 * 128) >> 4;    // MN-major: 16 rows
            constexpr uint64_t ROW32 = (32 * 128) >> 4;    // rows 32..63 of a tile
            constexpr uint64_t HI = 64 >> 4;               // the upper 32 of 64 contiguous elements
            const uint32_t id32 = make_idesc(64, 32, false, false), id_mm32 = make_idesc(64, 32, true, true),
                           id_km32 = make_idesc(64, 32, false, true);
            int pending = -1;   // last chunk whose products may still be running
            for (int c = 0; c < n; c++) {
                const int st = c & 1;
                const uint64_t d_r = make_desc(smem_u32(&s.in[st][0])), d_k = make_desc(smem_u32(&s.in[st][1])),
                               d_v = make_desc(smem_u32(&s.in[st][2])), d_rh = make_desc(smem_u32(&s.in[st][3])),
                               d_kh = make_desc(smem_u32(&s.khat[st]));
                if (!mbar_wait_or_abort(&s.ops_bar[c & 1], (uint32_t)((c >> 1) & 1), &s.abort_flag, P.wait_limit)) { fail = 1; break; }
                tc_fence_after();
                // the per-chunk backward kernel comes in two builds: tell it which one this chunk needs
                // (written from here: this lane has time, the compute warps do not)
                if (P.dchunk)
                    P.mildflag[bh * P.nchunk + j0 + c] = *reinterpret_cast<volatile int *>(&s.mild_flag[c & 1]) != 0;
                if (full) {
                    // scores: A1 = Rt Kt^T (column halves), A2 = X X[0:32]^T.  In a mild chunk Rt and Kt are
                    // scaled around one point, A1's rows 32..63 of columns 0..31 ARE the cross-block scores:
                    // that half goes where A2 would have gone and A2 is not formed.
                    const bool mild = *reinterpret_cast<volatile int *>(&s.mild_flag[c & 1]) != 0;
                    const uint32_t a1a = tm + (mild ? COL_A2 : COL_A1A);
#pragma unroll
                    for (int k = 0; k < 4; k++) mma_ss(a1a, d_r + k * KSTEP, d_k + k * KSTEP, id32, k > 0);
#pragma unroll
                    for (int k = 0; k < 4; k++) mma_ss(tm_hi + COL_A2, d_r + k * KSTEP, d_k + ROW32 + k * KSTEP, id32, k > 0);
                    if (!mild) {
#pragma unroll
                        for (int k = 0; k < 4; k++) mma_ss(tm + COL_A2, d_x + k * KSTEP, d_x + k * KSTEP, id32, k > 0);
                    }
                    mma_commit(&s.score_bar);
                }
                // U = Khat^T V  (value columns 0..31 -> lo lanes, 32..63 -> hi lanes)
#pragma unroll
                for (int hf = 0; hf < 2; hf++)
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        mma_ss((hf ? tm_hi : tm) + COL_U + 32 * (c & 1), d_kh + k * MSTEP, d_v + k * MSTEP + (hf ? HI : 0),
                               id_mm32, k > 0);
                mma_commit(&s.u_bar[c & 1]);
                pending = c;
                // r e^{cp} of this chunk goes out for the backward pass
                if (P.dchunk) {
                    tma_store_3d(&map_rh, &s.in[st][3], h * 64, (j0 + c) * CH, b);
                    tma_store_commit();
                }
                if (full) {
                    if (!mbar_wait_or_abort(&s.yrdy_bar, (uint32_t)(c & 1), &s.abort_flag, P.wait_limit)) { fail = 1; break; }
                    tc_fence_after();
                    // y = Atil V + Rhat Sbf  (value columns 0..31 -> lo lanes, 32..63 -> hi lanes)
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        const uint32_t d = (hf ? tm_hi : tm) + COL_Y;
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            mma_ss(d, d_atil + k * KSTEP, d_v + k * MSTEP + (hf ? HI : 0), id_km32, k > 0);
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            mma_ss(d, d_rh + k * KSTEP, d_sbf + k * MSTEP + (hf ? HI : 0), id_km32, true);
                    }
                    mma_commit(&s.y_bar);
                }
                // the stage is free for chunk c+2 when every product of chunk c is done (the last
                // commit covers all earlier ones of this thread) and the store has read its tile
                if (c + 2 < n) {
                    uint64_t *last = full ? &s.y_bar : &s.u_bar[c & 1];
                    const uint32_t par = full ? (uint32_t)(c & 1) : (uint32_t)((c >> 1) & 1);
                    if (!mbar_wait_or_abort(last, par, &s.abort_flag, P.wait_limit)) { fail = 1; break; }
                    pending = -1;
                    tma_store_wait_read();
                    issue_load(c + 2);
                }
            }
            if (fail) {
                atomicExch(&s.abort_flag, 1);
                if (P.status) atomicOr(P.status, 1);
                // let whatever is in flight finish before shared and tensor memory go away
                // (the last load issued on each of the two stages; earlier phases of a barrier are over)
                for (int q = issued > 0 ? issued - 1 : 0; q <= issued; q++)
                    if (q != P.skip_load) mbar_wait(&s.load_bar[q & 1], (uint32_t)((q >> 1) & 1), 200000u);
                if (pending >= 0) {
                    mbar_wait(&s.u_bar[pending & 1], (uint32_t)((pending >> 1) & 1), 200000u);
                    if (full) mbar_wait(&s.score_bar, (uint32_t)(pending & 1), 200000u);
                }
            }
            tma_store_wait_read();
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ compute warps
        const int wg = warp >> 2, w4 = warp & 3;
        const bool lo = (lane & 16) == 0;
        const int row = w4 * 16 + (lane & 15);         // accumulator row: key channel (state) or token (scores, y)
        const uint32_t lane_base = (uint32_t)(w4 * 32);
        // operand-pass coordinates (see decay_scan8 in wkv56_chunked.cuh): 4 tokens x 4 channels per thread
        const int blk = warp >> 2, cc = (lane & 15) >> 1, hf = lane & 1, tok0 = 8 * warp + 4 * (lane >> 4);
        const int ch0 = cc * 8 + 4 * hf;
        const int vcol0 = (lo ? 0 : 32) + 16 * wg;     // 16 columns of the row this thread holds

        const size_t sbase = (size_t)bh * 64 * 64;
        float S[16];
#pragma unroll
        for (int q = 0; q < 16; q++) {
            const int vc = vcol0 + q;
            const size_t idx = P.layout == WKV_STATE_KV ? (size_t)row * 64 + vc : (size_t)vc * 64 + row;
            if (P.gstart) S[q] = P.gstart[(size_t)unit * 4096 + row * 64 + vc];
            else S[q] = (P.state_in && !summary) ? P.state_in[sbase + idx] : 0.f;
        }
        float dprod = 1.f;      // summary pass: decay of the whole group for key channel `row`
        float lwc[4], wc[4];
        bool steep_static = false;
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            bool live;
            lwc[ch] = PER_TOKEN ? 0.f : log2_decay(P.wvec[h * 64 + ch0 + ch], P.w_kind, live);
            wc[ch] = exp2f(lwc[ch]);
            steep_static |= 8.f * lwc[ch] < MILD_L2_PER_8;
        }
        // static decay: whether the head's chunks are mild is known once and for all
        const bool mild_static = PER_TOKEN ? false : !compute_sync_or(steep_static);

        // Operand pass for chunk j: scaled r/k tiles in place in stage j&1, x, khat[j&1], the
        // score-diagonal partials and the chunk decay.  Contains one barrier of the compute warps.
        auto prep = [&](int j) -> bool {          // j: local chunk index
            const int jg = j0 + j;
            Tile *in = s.in[j & 1];
            Tile &khat = s.khat[j & 1];
            float c[4][4];
            DecayT<4> D;
            float other_l2[4];
            bool mild;
            if (!PER_TOKEN && (jg + 1) * CH <= P.T) {
                // static decay, whole chunk in range: closed form, nothing to scan or exchange
                decay_static(lwc, wc, tok0, c, D, other_l2);
                mild = mild_static;
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int t = tok0 + i;
                    const bool valid = jg * CH + t < P.T;
                    if (PER_TOKEN) {
                        float x[4];
                        unpack4(ld_tile4(in[3], t, cc, hf), x);
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            bool live;
                            const float l2 = log2_decay(x[ch], P.w_kind, live);
                            c[i][ch] = valid ? l2 : 0.f;
                        }
                    } else {
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) c[i][ch] = valid ? lwc[ch] : 0.f;
                    }
                }
                mild = decay_scan8(c, warp, lane, &s.wtot[0][0], D, other_l2, [](bool p) { return compute_sync_or(p); });
            }
            if (tid == 0) s.mild_flag[j & 1] = mild;
            // The warp reconverges here before it touches the r and k tiles.  The barrier also keeps the
            // tile loads below the decay scan: hoisted above it they push the pass over the 96 registers
            // that two 288-thread CTAs per SM allow, and it spills inside the serial loop.
            __syncwarp();
            // the bonus u of the thread's 4 channels (read again for every chunk: registers are scarce here)
            float uu[4];
            if (full) {
                const float4 u4 = *reinterpret_cast<const float4 *>(s.uf + ch0);
                uu[0] = u4.x; uu[1] = u4.y; uu[2] = u4.z; uu[3] = u4.w;
            }
            float other[4];          // 2^{total of the other block}
#pragma unroll
            for (int ch = 0; ch < 4; ch++) other[ch] = exp2f(other_l2[ch]);
            if (warp == 0 && lane < 16) {
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    const float d = exp2f(D.e[ch]) * other[ch];
                    s.dvec[j & 1][ch0 + ch] = d;
                    if (P.dchunk) P.dchunk[((size_t)bh * P.nchunk + jg) * 64 + ch0 + ch] = d;
                }
            }
            if (mild) {
                // One reference point (the end of block 0) for the whole chunk.  With it the state-term
                // factors are the score factors times a per-channel constant:
                //   block 0:  rt = r 2^{cp - e0},  rhat = rt 2^{e0};   kt = k 2^{e0 - c},  khat = kt 2^{total of block 1}
                //   block 1:  rt = r 2^{cp},       rhat = rt 2^{e0};   kt = k 2^{-c},      khat = kt 2^{total of block 1}
                // (cp, c counted from the thread's block start) -- one running factor per side instead of two.
                float fa[4], cr[4], ck[4];
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    const float own = exp2f(D.e[ch]);
                    cr[ch] = blk ? other[ch] : own;
                    ck[ch] = blk ? own : other[ch];
                    fa[ch] = exp2f(D.cp0[ch] - (blk ? 0.f : D.e[ch]));
                }
                if (full) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int t = tok0 + i;
                        float r[4], k[4], rt[4], rh[4];
                        unpack4(ld_tile4(in[0], t, cc, hf), r);
                        unpack4(ld_tile4(in[1], t, cc, hf), k);
                        float dsum = 0.f;
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            rt[ch] = r[ch] * fa[ch];
                            rh[ch] = rt[ch] * cr[ch];
                            dsum += r[ch] * uu[ch] * k[ch];
                            fa[ch] *= D.w[i][ch];
                        }
                        st_tile4(in[0], t, cc, hf, pack4(rt));
                        st_tile4(in[3], t, cc, hf, pack4(rh));
                        dsum += __shfl_xor_sync(0xffffffffu, dsum, 1);
                        dsum += __shfl_xor_sync(0xffffffffu, dsum, 2);
                        if ((lane & 3) == 0) s.dpart[(lane & 15) >> 2][t] = dsum;
                    }
                } else if (P.dchunk) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int t = tok0 + i;
                        float r[4], rh[4];
                        unpack4(ld_tile4(in[0], t, cc, hf), r);
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            rh[ch] = r[ch] * fa[ch] * cr[ch];
                            fa[ch] *= D.w[i][ch];
                        }
                        st_tile4(in[3], t, cc, hf, pack4(rh));
                    }
                }
#pragma unroll
                for (int ch = 0; ch < 4; ch++) fa[ch] = exp2f((blk ? 0.f : D.e[ch]) - D.c3[ch]);
#pragma unroll
                for (int i = 3; i >= 0; i--) {
                    const int t = tok0 + i;
                    float k[4], kt[4], kh[4];
                    unpack4(ld_tile4(in[1], t, cc, hf), k);
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        kt[ch] = k[ch] * fa[ch];
                        kh[ch] = kt[ch] * ck[ch];
                        fa[ch] *= D.w[i][ch];
                    }
                    if (full) st_tile4(in[1], t, cc, hf, pack4(kt));
                    st_tile4(khat, t, cc, hf, pack4(kh));
                }
            } else {
                // r-side operands, walking forward over the thread's tokens:
                //   fa = 2^{cp - m};  fb = 2^{cp}   (cp counted from the block start)
                //   block 0: rhat = r fb                 block 1: x = r fb, rhat = x 2^{total of block 0}
                float fa[4], fb[4], ref[4];     // ref: the reference point of the score factors (block-local)
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    ref[ch] = D.m[ch];
                    fa[ch] = exp2f(D.cp0[ch] - ref[ch]);
                    fb[ch] = exp2f(D.cp0[ch]);
                }
                if (full) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int t = tok0 + i;
                        float r[4], k[4], rt[4], rh[4], xx[4];
                        unpack4(ld_tile4(in[0], t, cc, hf), r);
                        unpack4(ld_tile4(in[1], t, cc, hf), k);
                        float dsum = 0.f;
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            rt[ch] = r[ch] * fa[ch];
                            xx[ch] = r[ch] * fb[ch];
                            rh[ch] = blk ? xx[ch] * other[ch] : xx[ch];
                            dsum += r[ch] * uu[ch] * k[ch];
                            fa[ch] *= D.w[i][ch];
                            fb[ch] *= D.w[i][ch];
                        }
                        st_tile4(in[0], t, cc, hf, pack4(rt));
                        st_tile4(in[3], t, cc, hf, pack4(rh));
                        if (blk) st_tile4(s.x, t, cc, hf, pack4(xx));
                        // groups of four lanes pool their channels; four partials per token remain
                        dsum += __shfl_xor_sync(0xffffffffu, dsum, 1);
                        dsum += __shfl_xor_sync(0xffffffffu, dsum, 2);
                        if ((lane & 3) == 0) s.dpart[(lane & 15) >> 2][t] = dsum;
                    }
                } else if (P.dchunk) {
                    // state-only pass on behalf of a backward call: r e^{cp} alone
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int t = tok0 + i;
                        float r[4], rh[4];
                        unpack4(ld_tile4(in[0], t, cc, hf), r);
#pragma unroll
                        for (int ch = 0; ch < 4; ch++) {
                            const float xx = r[ch] * fb[ch];
                            rh[ch] = blk ? xx * other[ch] : xx;
                            fb[ch] *= D.w[i][ch];
                        }
                        st_tile4(in[3], t, cc, hf, pack4(rh));
                    }
                }
                // k-side operands, walking backward:
                //   fa = 2^{m - c};  fb = 2^{e - c}   (e = total of the thread's block)
                //   block 0: x = k fb, khat = x 2^{total of block 1}      block 1: khat = k fb
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    fa[ch] = exp2f(ref[ch] - D.c3[ch]);
                    fb[ch] = exp2f(D.e[ch] - D.c3[ch]);
                }
#pragma unroll
                for (int i = 3; i >= 0; i--) {
                    const int t = tok0 + i;
                    float k[4], kt[4], kh[4], xx[4];
                    unpack4(ld_tile4(in[1], t, cc, hf), k);
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        kt[ch] = k[ch] * fa[ch];
                        xx[ch] = k[ch] * fb[ch];
                        kh[ch] = blk ? xx[ch] : xx[ch] * other[ch];
                        fa[ch] *= D.w[i][ch];
                        fb[ch] *= D.w[i][ch];
                    }
                    if (full) {
                        st_tile4(in[1], t, cc, hf, pack4(kt));
                        if (!blk) st_tile4(s.x, t, cc, hf, pack4(xx));
                    }
                    st_tile4(khat, t, cc, hf, pack4(kh));
                }
            }
            return mild;
        };
        // a wait of a compute thread; running out of patience ends everybody else's waits too
        auto cwait = [&](uint64_t *bar, uint32_t parity) {
            if (mbar_wait_or_abort(bar, parity, &s.abort_flag, P.wait_limit)) return true;
            *reinterpret_cast<volatile int *>(&s.abort_flag) = 1;
            return false;
        };
        // bf16 copy of the state at the start of chunk jn: operand of rhat*S, checkpoint
        // (jn local; the state at the end of a group is the next group's first checkpoint, written there)
        auto publish_state = [&](int jn) {
            const uint4 q0 = pack8(S), q1 = pack8(S + 8);
            if (full && jn < n) {
                st_tile(s.sbf, row, (vcol0 >> 3), q0);
                st_tile(s.sbf, row, (vcol0 >> 3) + 1, q1);
            }
            if (P.gsave && jn < n && (j0 + jn) % P.Lsave == 0) {
                const int nsave = (P.nchunk + P.Lsave - 1) / P.Lsave;
                float4 *dst = reinterpret_cast<float4 *>(
                    P.gsave + ((size_t)bh * nsave + (j0 + jn) / P.Lsave) * 4096 + row * 64 + vcol0);
#pragma unroll
                for (int q = 0; q < 4; q++) dst[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
            }
            if (P.ckpt && (jn < n || j0 + n == P.nchunk)) {
                uint4 *dst = reinterpret_cast<uint4 *>(
                    P.ckpt + (((size_t)bh * (P.nchunk + 1) + j0 + jn) * 64 + row) * 64 + vcol0);
                dst[0] = q0;
                dst[1] = q1;
            }
        };

        // Iteration j works on three chunks at once: operands of chunk j+1, y of chunk j, and the
        // state / masked scores that the y product of chunk j+1 needs.  j = -1 is the prologue.
        bool mild_next = false;      // chunk j+1 is mild
        for (int j = -1; j < n; j++) {
            // (P) operands of chunk j+1
            if (j + 1 < n) {
                if (!cwait(&s.load_bar[(j + 1) & 1], (uint32_t)(((j + 1) >> 1) & 1))) fail = 1;
                mild_next = prep(j + 1);
                fence_async_smem();
                compute_sync();
                if (tid == 0) mbar_arrive(&s.ops_bar[(j + 1) & 1]);
            }
            // (E) y of chunk j
            if (j >= 0 && full) {
                if (!cwait(&s.y_bar, (uint32_t)(j & 1))) fail = 1;
                tc_fence_after();
                float yv[16];
                tmem_ld16(tmem_addr(tm, lane_base, COL_Y + 16 * wg), yv);
                tmem_ld_wait();
                const int t = (j0 + j) * CH + row;
                if (t < P.T) {
                    uint4 *dst = reinterpret_cast<uint4 *>(P.y + ((size_t)b * P.T + t) * C + h * 64 + vcol0);
                    dst[0] = pack8(yv);
                    dst[1] = pack8(yv + 8);
                }
            }
            // (S) state at the start of chunk j+1:  S = d_j S + U_j
            if (j >= 0) {
                if (!cwait(&s.u_bar[j & 1], (uint32_t)((j >> 1) & 1))) fail = 1;
                tc_fence_after();
                float uacc[16];
                tmem_ld16(tmem_addr(tm, lane_base, COL_U + 32 * (j & 1) + 16 * wg), uacc);
                tmem_ld_wait();
                const float d = s.dvec[j & 1][row];
                if (summary) dprod *= d;
#pragma unroll
                for (int q = 0; q < 16; q++) S[q] = fmaf(d, S[q], uacc[q]);
            }
            publish_state(j + 1);
            // (M) masked scores of chunk j+1: lo lanes own columns 0..31 of token row t, hi lanes 32..63;
            // this warp group 16 of them
            if (j + 1 < n && full) {
                if (!cwait(&s.score_bar, (uint32_t)((j + 1) & 1))) fail = 1;
                tc_fence_after();
                const int t = row;
                float a[16];
                // rows 0..31 (w4 0,1): A1a for the lo half, nothing kept for the hi half;
                // rows 32..63 (w4 2,3): A2 (lo) and A1b (hi) share their columns; in a mild chunk A1a sits there too
                tmem_ld16(tmem_addr(tm, lane_base, (w4 < 2 && !mild_next ? COL_A1A : COL_A2) + 16 * wg), a);
                tmem_ld_wait();
                const float diag = (s.dpart[0][t] + s.dpart[1][t]) + (s.dpart[2][t] + s.dpart[3][t]);
                // entries left of local column `lim` are kept, column lim is the diagonal
                const bool cross = t >= HB && lo, empty = t < HB && !lo;
                const int lim = cross ? 99 : (empty ? -1 : (t & 31) - 16 * wg);
#pragma unroll
                for (int q = 0; q < 16; q++) a[q] = q < lim ? a[q] : (q == lim ? diag : 0.f);
                st_tile(s.atil, t, (vcol0 >> 3), pack8(a));
                st_tile(s.atil, t, (vcol0 >> 3) + 1, pack8(a + 8));
            }
            fence_async_smem();
            tc_fence_before();
            {
                // closing barrier of the iteration; a failed wait anywhere ends the loop for everyone
                uint32_t any;
                asm volatile(
                    "{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, 1, 256, q;\nselp.u32 %0, 1, 0, p;\n}"
                    : "=r"(any) : "r"((uint32_t)fail) : "memory");
                if (any) { fail = 1; break; }
            }
            if (j + 1 < n && full && tid == 0) mbar_arrive(&s.yrdy_bar);
        }
        if (fail) {
            if (tid == 0) {
                atomicExch(&s.abort_flag, 1);
                if (P.status) atomicOr(P.status, 1);
            }
        } else if (summary) {
            float4 *dst = reinterpret_cast<float4 *>(P.gU + (size_t)unit * 4096 + row * 64 + vcol0);
#pragma unroll
            for (int q = 0; q < 4; q++) dst[q] = make_float4(S[4 * q], S[4 * q + 1], S[4 * q + 2], S[4 * q + 3]);
            if (vcol0 == 0) P.gD[(size_t)unit * 64 + row] = dprod;
        } else if (P.state_out && j0 + n == P.nchunk) {
#pragma unroll
            for (int q = 0; q < 16; q++) {
                const int vc = vcol0 + q;
                const size_t idx = P.layout == WKV_STATE_KV ? (size_t)row * 64 + vc : (size_t)vc * 64 + row;
                P.state_out[sbase + idx] = S[q];
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tm, FWD_TMEM_COLS);
}

static_assert(sizeof(FwdSmem) + 1024 <= 115712, "two CTAs per SM need <= 113 KiB each");

// Pass B of the time-group scheme: for every chain the elementwise recurrence over its groups,
//   S <- init;  for each group g (forward order, or reverse for the gradient):  starts[g] = S;  S = d_g * S + U_g
// and the final S.  One thread per state element; the loads do not depend on S, so the compiler
// is free to run them ahead.  `init` / `final_out` are in the caller's state layout (NULL init = zeros).
__global__ void __launch_bounds__(256)
k_group_scan(const float *__restrict__ U, const float *__restrict__ dG, const float *__restrict__ init,
             float *__restrict__ starts, float *__restrict__ final_out, int G, int layout, int reverse) {
    pdl_wait();
    pdl_trigger();
    const int idx = blockIdx.x * 256 + threadIdx.x, bh = idx >> 12, e = idx & 4095, row = e >> 6, vc = e & 63;
    const size_t lidx = (size_t)bh * 4096 + (layout == WKV_STATE_KV ? e : vc * 64 + row);
    float S = init ? init[lidx] : 0.f;
#pragma unroll 4
    for (int step = 0; step < G; step++) {
        const size_t u = (size_t)bh * G + (reverse ? G - 1 - step : step);
        starts[u * 4096 + e] = S;
        S = fmaf(dG[u * 64 + row], S, U[u * 4096 + e]);
    }
    if (final_out) final_out[lidx] = S;
}

// Self-test of the bounded waits: one CTA, one mbarrier on which nobody ever arrives.  Warp 0
// waits on it with the plain bounded wait; when that runs out it raises the CTA's abort flag,
// which must end the (much longer) abortable wait of warp 1.  Status bits: 16 = the plain wait
// gave up, 32 = the abortable wait gave up.
__global__ void __launch_bounds__(64) k_selftest_wait(int *status, uint32_t limit) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        if (!mbar_wait(&bar, 0, limit)) {
            if (threadIdx.x == 0) {
                atomicOr(status, 16);
                *reinterpret_cast<volatile int *>(&abort_flag) = 1;
            }
        }
    } else {
        if (!mbar_wait_or_abort(&bar, 0, &abort_flag, limit * 64u) && threadIdx.x == 32) atomicOr(status, 32);
    }
}

}  // namespace

int selftest_wait(int *status, uint32_t limit, cudaStream_t stream) {
    if (limit == 0 || limit > 100000u) return WKV_ERR_SHAPE;     // a test: keep it short
    k_selftest_wait<<<1, 64, 0, stream>>>(status, limit);
    return launch_status();
}

// ---------------------------------------------------------------------------
// host side

bool chunked_supported(const wkv_args_t *a, bool) {
    return a->dtype == WKV_BF16 && a->N == 64 && a->T > 0;
}

// The per-token kernels read the decay activation x as a bf16 [B,T,C] tensor.  A caller that
// holds the fp32 ew = -exp(x) instead (RWKV-v6/src/module/TimeMix.py:49-51) gets x = log(-ew)
// rebuilt in bf16 first.  That is exact when ew was computed from a bf16 x, as that wrapper does
// (the round trip is off by ~1e-7 relative, far inside half a bf16 step); an ew that never was
// a bf16 x is seen at bf16 resolution of x -- the resolution the activation has in bf16 training.
namespace {
__global__ void __launch_bounds__(256) k_ew_to_x(const float4 *__restrict__ ew, uint2 *__restrict__ x, size_t n4) {
    pdl_wait();
    pdl_trigger();
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    const float4 e = ew[i];
    x[i] = make_uint2(pack2(logf(-e.x), logf(-e.y)), pack2(logf(-e.z), logf(-e.w)));
}
}  // namespace

size_t chunked_wconv_bytes(const wkv_args_t *a, bool per_token_w) {
    if (!per_token_w || a->w_kind != WKV_W_NEGEXP) return 0;
    return (((size_t)a->B * a->T * a->H * 64 * 2) + 255) & ~(size_t)255;
}

int chunked_convert_w(wkv_args_t *a, bool per_token_w, void *scratch, cudaStream_t stream) {
    if (!per_token_w || a->w_kind != WKV_W_NEGEXP) return WKV_OK;
    const size_t n4 = (size_t)a->B * a->T * a->H * 16;
    const int err = launch_chained(k_ew_to_x, dim3((unsigned)((n4 + 255) / 256)), dim3(256), 0, stream,
                                   (const float4 *)a->w, (uint2 *)scratch, n4);
    a->w = scratch;
    a->w_kind = WKV_W_RAW;
    return err;
}

int device_sm_count() {
    static int sms[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = __atomic_load_n(&sms[dev], __ATOMIC_RELAXED);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        __atomic_store_n(&sms[dev], n, __ATOMIC_RELAXED);
    }
    return n;
}

namespace chunked {

GroupPlan plan_groups(int BH, int nchunk, int requested) {
    int G = 1;
    if (requested > 0) {
        G = requested < nchunk ? requested : nchunk;
    } else if (nchunk >= 8) {
        // two CTAs of the serial kernels fit on an SM; split only when the chains alone leave
        // most of those slots empty, and keep every group at two chunks or more
        const int slots = 2 * device_sm_count();
        if (BH * 5 < slots * 2) {
            G = slots / BH;
            if (G > nchunk / 2) G = nchunk / 2;
        }
    }
    if (G < 1) G = 1;
    GroupPlan P;
    P.L = (nchunk + G - 1) / G;
    P.G = (nchunk + P.L - 1) / P.L;
    return P;
}

// The plan of a forward call.  A call that saves group states keeps its groups a multiple of the
// saving distance long: a restart then runs, inside every saved group, exactly the operations of
// the call that saved (which is what makes it bit-identical).  A restart's groups are the saved ones.
GroupPlan plan_forward(const wkv_args_t *a) {
    const int n = (a->T + CH - 1) / CH;
    GroupPlan gp = plan_groups(a->B * a->H, n, a->time_groups);
    if (a->group_states && a->group_states_mode == WKV_GROUP_STATES_USE) {
        gp.L = SAVE_EVERY;
        gp.G = (n + SAVE_EVERY - 1) / SAVE_EVERY;
    } else if (a->group_states && a->group_states_mode == WKV_GROUP_STATES_SAVE && gp.G > 1) {
        gp.L = (gp.L + SAVE_EVERY - 1) / SAVE_EVERY * SAVE_EVERY;
        gp.G = (n + gp.L - 1) / gp.L;
    }
    return gp;
}

GroupLayout group_layout(size_t units) {
    auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
    GroupLayout L;
    L.gU = 0;
    L.gD = al(units * 4096 * 4);
    L.gstart = L.gD + al(units * 64 * 4);
    L.total = L.gstart + al(units * 4096 * 4);
    return L;
}

int launch_group_scan(const void *group_ws, int BH, int G, const float *init, float *final_out, int layout,
                      bool reverse, cudaStream_t stream) {
    const GroupLayout GL = group_layout((size_t)BH * G);
    const char *g = (const char *)group_ws;
    return launch_chained(k_group_scan, dim3(BH * 16), dim3(256), 0, stream, (const float *)(g + GL.gU),
                          (const float *)(g + GL.gD), init, (float *)(g + GL.gstart), final_out, G, layout,
                          reverse ? 1 : 0);
}

}  // namespace chunked

// workspace layout: [0,256) status words; then the time-group buffers when the chains are split
size_t chunked_group_states_bytes(const wkv_args_t *a) {
    const size_t n = (a->T + CH - 1) / CH;
    return (size_t)a->B * a->H * ((n + SAVE_EVERY - 1) / SAVE_EVERY) * 4096 * sizeof(float);
}

size_t chunked_forward_workspace(const wkv_args_t *a, bool per_token_w) {
    const GroupPlan gp = plan_forward(a);
    return 256 + (gp.G > 1 ? group_layout((size_t)a->B * a->H * gp.G).total : 0) + chunked_wconv_bytes(a, per_token_w);
}

int chunked_forward_impl(const wkv_args_t *a, bool per_token_w, void *state_ckpt, void *group_ws,
                         const ChunkedTest &tst, cudaStream_t stream) {
    const int B = a->B, T = a->T, H = a->H, C = H * 64, BH = B * H;
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
    // restarting from saved group states: the groups are the saved ones, and only pass C runs
    const bool restart = a->group_states && a->group_states_mode == WKV_GROUP_STATES_USE;
    const GroupPlan gp = plan_forward(a);
    p.G = gp.G; p.L = gp.L;
    p.gsave = (a->group_states && a->group_states_mode == WKV_GROUP_STATES_SAVE) ? (float *)a->group_states : nullptr;
    p.Lsave = SAVE_EVERY;
    p.u = (const __nv_bfloat16 *)a->u;
    p.wvec = per_token_w ? nullptr : (const float *)a->w;
    p.status = (int *)a->workspace;
    p.mildflag = nullptr;
    p.wait_limit = tst.wait_limit;
    p.skip_load = tst.kernel == 0 ? tst.skip_load : -1;
    const size_t smem = sizeof(FwdSmem) + 1024;
    const int mode = a->y == nullptr ? FWD_STATES : FWD_FULL;
    using Kern = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                          const CUtensorMap, const FwdParams);
    static const Kern kerns[2][3] = {
        {k_chunk_fwd<false, FWD_FULL>, k_chunk_fwd<false, FWD_STATES>, k_chunk_fwd<false, FWD_SUMMARY>},
        {k_chunk_fwd<true, FWD_FULL>, k_chunk_fwd<true, FWD_STATES>, k_chunk_fwd<true, FWD_SUMMARY>}};
    static unsigned char attr_done[2][3][64];
    const int pt = per_token_w ? 1 : 0;
    CUtensorMap mrh = mr;

    const GroupLayout GL = group_layout((size_t)BH * gp.G);
    char *g = (char *)group_ws;
    if (gp.G > 1 && !restart) {
        // A: what every group adds to the state, from zero
        if (!set_max_smem_once(kerns[pt][FWD_SUMMARY], (int)smem, attr_done[pt][FWD_SUMMARY])) return WKV_ERR_LAUNCH;
        p.state_in = nullptr; p.gstart = nullptr; p.state_out = nullptr;
        p.gU = (float *)(g + GL.gU); p.gD = (float *)(g + GL.gD);
        p.y = nullptr; p.ckpt = nullptr; p.dchunk = nullptr;
        if (launch_chained(kerns[pt][FWD_SUMMARY], dim3(gp.G, BH), dim3(FWD_THREADS), smem, stream, mr, mk, mv, mw,
                           mrh, p) != WKV_OK)
            return WKV_ERR_LAUNCH;
        // B: the state at the start of every group.  (The state after the segment is left to the last
        // group of pass C, so that a later restart from saved states reproduces it bit for bit.)
        if (launch_group_scan(g, BH, gp.G, a->state_in, nullptr, a->state_layout, false, stream) != WKV_OK)
            return WKV_ERR_LAUNCH;
    }
    // C (or the whole job when the chains are not split)
    if (!set_max_smem_once(kerns[pt][mode], (int)smem, attr_done[pt][mode])) return WKV_ERR_LAUNCH;
    p.state_in = a->state_in;
    p.gstart = restart ? (const float *)a->group_states : gp.G > 1 ? (const float *)(g + GL.gstart) : nullptr;
    p.state_out = a->state_out;      // written by the group that ends the segment
    p.gU = nullptr; p.gD = nullptr;
    p.y = (__nv_bfloat16 *)a->y;
    const CkptLayout CL = ckpt_layout(B, T, H);
    p.ckpt = nullptr; p.dchunk = nullptr;
    if (state_ckpt) {
        char *ck = (char *)state_ckpt;
        p.ckpt = (__nv_bfloat16 *)(ck + CL.sck);
        p.dchunk = (float *)(ck + CL.dchunk);
        p.mildflag = (unsigned char *)(ck + CL.mild);
        if (!make_btc_map(&mrh, ck + CL.rhat, B, T, C)) return WKV_ERR_LAUNCH;
    }
    return launch_chained(kerns[pt][mode], dim3(gp.G, BH), dim3(FWD_THREADS), smem, stream, mr, mk, mv, mw, mrh, p);
}

int chunked_forward(const wkv_args_t *a0, bool per_token_w, const ChunkedTest &tst, cudaStream_t stream) {
    wkv_args_t a = *a0;
    if (cudaMemsetAsync(a.workspace, 0, 256, stream) != cudaSuccess) return WKV_ERR_LAUNCH;
    const size_t conv = chunked_wconv_bytes(&a, per_token_w);
    if (conv) {   // the converted decay tensor sits at the end of the workspace
        const int err = chunked_convert_w(&a, per_token_w, (char *)a.workspace + chunked_forward_workspace(a0, per_token_w) - conv, stream);
        if (err != WKV_OK) return err;
    }
    return chunked_forward_impl(&a, per_token_w, a.state_ckpt, (char *)a.workspace + 256, tst, stream);
}

}  // namespace wkv
