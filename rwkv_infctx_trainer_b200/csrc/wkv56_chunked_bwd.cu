// Chunked tensor-core backward of the v5/v6 WKV recurrence (bf16 I/O, fp32 state).
//
// Three kernels per BPTT segment:
//   1. the forward kernel has left (or, in a state-only mode, now writes) S_j, the state at
//      the start of every 64-token chunk (bf16), the tiles r e^{cp} and the chunk decays d_j;
//   2. k_chunk_dscan runs the reverse recurrence  D_j = d_j D_{j+1} + (r e^{cp})^T gy  with D
//      in registers and only the chunk's own product on the tensor core, writes every D_{j+1}
//      (bf16), E_j = rowsum(S_j * D_j) and the state gradient D_0;
//   3. k_chunk_bwd handles every (batch, head, chunk) independently from S_j and
//      D_{j+1}: recomputes the masked scores A, P = gy v^T, and from them
//         gv = A^T gy + khat D
//         gr = fr*(P~d Kt) + g*(P~x X) + e^{cp}*(gy S^T) + p_tt u k
//         gk = fk*(P~d^T Rt) + g*(P~x^T X) + e^{c_63-c}*(v D^T) + p_tt u r
//      (P~d / P~x = same-block / cross-block part of the strictly lower P; Rt, Kt, X, khat the
//      scaled operands of the forward kernel) with every product on tcgen05.mma, accumulators
//      laid out [token, channel] so that the epilogue works on whole 16-byte tile chunks.
//
// Decay gradient.  dL/d(log w_t)[k] = w_t sum_v S_t[k,v] D_{t+1}[k,v] expands into
//   E_j + sum_{t'<=t} (a_t' + b_t') - b_t,     a = -(qrS + qrI),   b = qkD + qkI,
// where qrS/qkD are the state parts of r*gr and k*gk and qrI/qkI their intra-chunk
// parts.  The sum is a difference of large terms; it is exact only because qrI and qkI
// are built from the SAME bf16-rounded factors (Rt * (P~d Kt) and Kt * (P~d^T Rt)),
// so the common terms cancel to fp32 rounding instead of to bf16 rounding.
//
// Math reference: RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu:70-293 (what the
// gradients are), RWKV-v6/src/module/rwkv_inner.py:48-113 (the chunked form).
#include <type_traits>

#include "wkv56_chunked.cuh"

namespace wkv {
namespace {

using namespace sm100;
using namespace chunked;

// ----------------------------------------------------------------------------
// dS scan

constexpr int DS_STAGES = 3;   // (four stages measured no faster: the kernel is HBM bound)

struct DscanSmem {
    Tile in[DS_STAGES][3];              // r e^{cp} and gy of the step's chunk; S at the chunk's end
    __align__(16) float dvec[DS_STAGES][CH];   // decay of the whole chunk per key channel
    uint64_t load_bar[DS_STAGES];       // TMA: a stage has landed
    uint64_t stage_free[DS_STAGES];     // the four scan warps are done with a stage
    uint64_t mma_bar[2];                // tensor core: a product buffer is complete
    uint64_t prod_free[2];              // the four scan warps have read a product buffer
    uint32_t tmem_base;
};

struct DscanParams {
    int T, H, nchunk, layout;
    int G, L;             // time groups per chain, chunks per group (see wkv56_chunked.cu)
    int summary;          // pass A: zero start, the only outputs are gU / gD
    const float *dchunk;  // [B*H, nchunk, 64] decay of each whole chunk (from the forward kernel)
    const float *gstate_out;   // G == 1: the caller's gradient w.r.t. the state after the segment
    const float *gstart;       // G > 1, pass C: [B*H*G, 64, 64] gradient at the END of every group ([key,value])
    float *gstate_in;          // G == 1 only (with G > 1 the group scan writes it)
    float *gU;                 // pass A: [B*H*G, 64, 64] gradient a group builds from zero
    float *gD;                 // pass A: [B*H*G, 64] decay of a whole group per key channel
    __nv_bfloat16 *dck;  // [B*H, nchunk+1, 64, 64]; entry j+1 = dL/dS at the end of chunk j
    float *e0;           // [B*H, nchunk+1, 64]; entry j = sum_v S_j[k,v] D_j[k,v] at chunk boundary j
    int *status;
    uint32_t wait_limit;
    int skip_load;        // -1; a step index leaves that step's TMA loads out (wait-timeout test)
};

// Reverse scan of the state gradient:  D_j = d_j D_{j+1} + (r e^{cp})^T gy  over the chunks j of a
// segment, step i = 0..n-1 handling chunk j = n-1-i.  The scaled r tiles and the chunk decays
// d_j come from the forward kernel, so a step has no operand pass.
//
// Five warps.  Warp 4 (one lane) feeds the machine: TMA loads DS_STAGES steps ahead, and for every
// step the product U_j = (r e^{cp})^T gy into one of two tensor-memory buffers -- U_j does not
// depend on the carried gradient, so it is ready before the scan gets there.  Warps 0..3 carry
// D in registers (thread = key row, 32 value columns) and run the serial chain,
//   write D_{j+1} (bf16) and E_{j+1} = rowsum(S_{j+1} * D_{j+1});   D_j = d_j D_{j+1} + U_j,
// without ever synchronising with one another: each warp only waits on the barriers of the data
// it consumes and releases buffers back to warp 4.  A closing step i = n writes E_0 and D_0.
// Every wait is bounded; a warp whose wait runs out flags the status word and leaves the loop,
// which makes the waits of the others run out in turn.
//
// With time groups a CTA handles the chunks [j0, j0+n) of its chain: as a summary pass (from a
// zero gradient; no S tiles, no checkpoints, outputs gU / gD) or as the full pass from the
// gradient the group scan computed for the end of its group.  The closing step (E and D at the
// chain's first chunk boundary) belongs to the first group alone.
__global__ void __launch_bounds__(160)
k_chunk_dscan(const __grid_constant__ CUtensorMap map_rh, const __grid_constant__ CUtensorMap map_gy,
              const __grid_constant__ CUtensorMap map_s, const DscanParams P) {
    pdl_wait();
    pdl_trigger();
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles want a 1024-byte aligned base.  The padding is added to the __shared__ array
    // itself (not to an integer copy of its address), so the compiler still knows that everything
    // behind `s` is shared memory and uses shared-memory loads and stores for the tiles.
    DscanSmem &s = *reinterpret_cast<DscanSmem *>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int unit = blockIdx.x, bh = unit / P.G, grp = unit - bh * P.G, b = bh / P.H, h = bh % P.H;
    const int j0 = grp * P.L, n = min(P.L, P.nchunk - j0), N = P.nchunk;
    const bool summary = P.summary != 0;
    const int nsteps = n + ((!summary && grp == 0) ? 1 : 0);    // + the closing step
    const uint32_t LIM = P.wait_limit;

    if (tid == 0) {
        for (int q = 0; q < DS_STAGES; q++) { mbar_init(&s.load_bar[q], 1); mbar_init(&s.stage_free[q], 4); }
        for (int q = 0; q < 2; q++) { mbar_init(&s.mma_bar[q], 1); mbar_init(&s.prod_free[q], 4); }
        fence_mbar_init();
    }
    if (warp == 0) { tmem_alloc(&s.tmem_base, 64); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s.tmem_base;
    auto load_parity = [&](int i) { return (uint32_t)((i / DS_STAGES) & 1); };
    auto prod_parity = [&](int i) { return (uint32_t)((i >> 1) & 1); };
    int fail = 0;

    if (warp == 4) {
        if (lane == 0) {
            int issued = -1, landed = -1, mma_issued = -1;
            auto issue_load = [&](int i) {
                if (i == P.skip_load) return;
                const int st = i % DS_STAGES, j = j0 + n - 1 - i;      // global chunk of step i
                mbar_expect_tx(&s.load_bar[st], (i < n ? 2 * TILE_BYTES + CH * 4 : 0) + (summary ? 0 : TILE_BYTES));
                if (i < n) {
                    tma_load_3d(&s.in[st][0], &map_rh, &s.load_bar[st], h * 64, j * CH, b);
                    tma_load_3d(&s.in[st][1], &map_gy, &s.load_bar[st], h * 64, j * CH, b);
                    bulk_load_1d(s.dvec[st], P.dchunk + ((size_t)bh * N + j) * 64, CH * 4, &s.load_bar[st]);
                }
                if (!summary) tma_load_3d(&s.in[st][2], &map_s, &s.load_bar[st], 0, 0, bh * (N + 1) + j + 1);
                issued = i;
            };
            for (int i = 0; i < DS_STAGES && i < nsteps; i++) issue_load(i);
            const uint32_t id = make_idesc(64, 32, true, true);
            for (int i = 0; i < nsteps && !fail; i++) {
                if (!mbar_wait(&s.load_bar[i % DS_STAGES], load_parity(i), LIM)) { fail = 1; break; }
                landed = i;
                if (i < n) {
                    // buffer i&1 held the product of step i-2
                    if (i >= 2 && !mbar_wait(&s.prod_free[i & 1], prod_parity(i - 2), LIM)) { fail = 1; break; }
                    tc_fence_after();
                    Tile *in = s.in[i % DS_STAGES];
                    // value columns 0..31 into lanes 0..15 of each quarter, 32..63 into lanes 16..31
#pragma unroll
                    for (int hf = 0; hf < 2; hf++)
#pragma unroll
                        for (int k = 0; k < 4; k++)
                            mma_ss(tm + (hf ? (16u << 16) : 0u) + 32u * (i & 1), desc_mnmajor(&in[0], 0, k),
                                   desc_mnmajor(&in[1], 0, k) + (hf ? 4 : 0), id, k > 0);
                    mma_commit(&s.mma_bar[i & 1]);
                    mma_issued = i;
                }
                // the stage of step i-1 goes to step i-1+DS_STAGES as soon as the scan warps are done with it
                if (i >= 1 && i + DS_STAGES - 1 < nsteps) {
                    if (!mbar_wait(&s.stage_free[(i - 1) % DS_STAGES], load_parity(i - 1), LIM)) { fail = 1; break; }
                    issue_load(i + DS_STAGES - 1);
                }
            }
            if (fail) {
                // let everything in flight land before the shared and tensor memory go away
                for (int q = landed + 1; q <= issued; q++)
                    if (q != P.skip_load) mbar_wait(&s.load_bar[q % DS_STAGES], load_parity(q), 200000u);
                if (mma_issued >= 0) mbar_wait(&s.mma_bar[mma_issued & 1], prod_parity(mma_issued), 100000u);
                if (mma_issued >= 1) mbar_wait(&s.mma_bar[(mma_issued - 1) & 1], prod_parity(mma_issued - 1), 100000u);
                if (P.status) atomicOr(P.status, 2);
            }
        }
        __syncwarp();
    } else {
        const bool active = (lane & 16) == 0;
        const int row = warp * 16 + (lane & 15);
        const uint32_t lane_base = (uint32_t)(warp * 32);
        // U[key, value 0..31] sits in lanes 0..15 of each quarter, U[key, value 32..63] in lanes 16..31
        const int vcol0 = active ? 0 : 32;
        const size_t sbase = (size_t)bh * 64 * 64;
        float v[32];     // D, this thread's key row and half of the value columns
#pragma unroll
        for (int q = 0; q < 32; q++) {
            const int vc = vcol0 + q;
            const size_t idx = P.layout == WKV_STATE_KV ? (size_t)row * 64 + vc : (size_t)vc * 64 + row;
            if (P.gstart) v[q] = P.gstart[(size_t)unit * 4096 + row * 64 + vc];
            else v[q] = (P.gstate_out && !summary) ? P.gstate_out[sbase + idx] : 0.f;
        }
        float dprod = 1.f;      // summary pass: decay of the whole group for key channel `row`
        for (int i = 0; i < nsteps; i++) {
            const int st = i % DS_STAGES, j = j0 + n - 1 - i;       // global chunk of step i
            Tile *in = s.in[st];
            if (!mbar_wait(&s.load_bar[st], load_parity(i), LIM)) { fail = 1; break; }
            // with D_{j+1} in hand: its checkpoint and E_{j+1} ...
            if (!summary) {
                float dot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c8 = 0; c8 < 4; c8++) {
                    float sv[8];
                    unpack8(ld_tile(in[2], row, (vcol0 >> 3) + c8), sv);
#pragma unroll
                    for (int q = 0; q < 8; q++) dot[c8] += sv[q] * v[8 * c8 + q];
                }
                float e = (dot[0] + dot[1]) + (dot[2] + dot[3]);
                e += __shfl_xor_sync(0xffffffffu, e, 16);
                if (active) P.e0[((size_t)bh * (N + 1) + (j + 1)) * 64 + row] = e;
            }
            if (i == n) {   // closing step: D_0 is the state gradient
                if (P.gstate_in && P.G == 1) {
#pragma unroll
                    for (int q = 0; q < 32; q++) {
                        const int vc = vcol0 + q;
                        const size_t idx = P.layout == WKV_STATE_KV ? (size_t)row * 64 + vc : (size_t)vc * 64 + row;
                        P.gstate_in[sbase + idx] = v[q];
                    }
                }
                break;
            }
            if (!summary) {
                uint4 *dst = reinterpret_cast<uint4 *>(P.dck + (((size_t)bh * (N + 1) + j + 1) * 64 + row) * 64 + vcol0);
#pragma unroll
                for (int c8 = 0; c8 < 4; c8++) dst[c8] = pack8(v + 8 * c8);
            }
            // ... then D_j = d_j D_{j+1} + U_j
            if (!mbar_wait(&s.mma_bar[i & 1], prod_parity(i), LIM)) { fail = 1; break; }
            tc_fence_after();
            {
                float u[32];
                tmem_ld16(tmem_addr(tm, lane_base, 32 * (i & 1)), u);
                tmem_ld16(tmem_addr(tm, lane_base, 32 * (i & 1) + 16), u + 16);
                tmem_ld_wait();
                const float d = s.dvec[st][row];
                dprod *= d;
#pragma unroll
                for (int q = 0; q < 32; q++) v[q] = fmaf(d, v[q], u[q]);
            }
            // this warp is done with the product buffer and with the stage
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&s.prod_free[i & 1]); mbar_arrive(&s.stage_free[st]); }
        }
        if (fail) {
            if (lane == 0 && P.status) atomicOr(P.status, 2);
        } else if (summary) {
            float4 *dst = reinterpret_cast<float4 *>(P.gU + (size_t)unit * 4096 + row * 64 + vcol0);
#pragma unroll
            for (int q = 0; q < 8; q++) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            if (active) P.gD[(size_t)unit * 64 + row] = dprod;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tm, 64);
}

// ----------------------------------------------------------------------------
// per-chunk gradients

enum { T_R = 0, T_K, T_V, T_W, T_GY, T_S, T_D, N_IN };

// 14 tiles + 1 KiB: two CTAs fit in one SM's shared memory.
struct BwdSmem {
    Tile in[N_IN];             // raw r, k, v, w, gy; S_j, D_{j+1}.  The w slot becomes rows
                               // 0..31 of the cumulative-decay table once w has been read.
    Tile rt, kt, x, khat;      // scaled operands
    Tile atil, ptil;           // masked scores A (with diagonal), P~
    Tile ctab_hi;              // rows 32..63 of the cumulative-decay table
    float ptt[CH];
    float kb[CH];              // decay-gradient constant of the chunk start, per channel
    __align__(16) float uf[CH];   // the head's bonus u in fp32
    uint64_t load_bar;
    uint64_t bar_early;        // P and the state products (need the raw tiles only)
    uint64_t bar_score;        // A1, A2
    uint64_t bar_grad;         // phase 2 except gv
    uint64_t bar_gv;           // gv
    uint32_t tmem_base;
    int not_mine;              // mild-only build: the chunk turned out to be a steep one
};

static_assert(sizeof(BwdSmem) <= 115712, "two CTAs per SM need <= 113 KiB each");

struct BwdParams {
    int T, H, nchunk, w_kind;
    int prefetch_dist;   // CTAs resident on the device at once: that far ahead tiles are pulled into L2
    const __nv_bfloat16 *u;
    const float *wvec;
    const float *e0;  // [B*H, nchunk+1, 64]: sum_v S_j[k,v] D_j[k,v] at chunk boundary j (from the dS scan)
    float *gu_part;   // [B*H, nchunk, 64]
    float *gw_part;   // v5 only: [B*H, nchunk, 64]
    int *status;
    uint32_t wait_limit;
    int skip_load;        // -1; a chunk index whose CTAs leave their TMA loads out (wait-timeout test)
    const unsigned char *mildflag;   // [B*H*nchunk] from the forward kernel: 1 = the chunk is mild
};

// tensor-memory columns; "lo" = lanes 0..15 of each 32-lane quarter, "hi" = lanes 16..31.
// Phase 1: A1 and A2 in lo, P in hi (full 64-column score rows).  The state products of phase 1
// and everything of phase 2 are [token, 32 channels] with channels 0..31 in lo and 32..63 in hi.
enum { C_GSR = 0, C_GSK = 32,                                          // phase 1, read by the epilogue
       C_A1 = 64, C_P = 64, C_A2 = 128,                                // phase 1, read by the mask pass
       C_G1R = 64, C_G2R = 96, C_G1K = 128, C_G2K = 160, C_GV = 192,   // phase 2
       BWD_TMEM_COLS = 256 };

// fp32 cumulative log-decay table c[t][k]: rows 0..31 in `a`, rows 32..63 in `b`, 256 bytes per row;
// the 16-byte column index is XORed with (t & 7) so that 8 consecutive rows of one column fall into
// 8 different bank groups
__device__ __forceinline__ float4 *ctab_ptr4(Tile &a, Tile &b, int t, int col4) {
    return reinterpret_cast<float4 *>((t < 32 ? a.b : b.b) + (t & 31) * 256 + ((col4 ^ (t & 7)) << 4));
}
// channels 8*c8 .. +7 of row t
__device__ __forceinline__ void ld_ctab8(Tile &a, Tile &b, int t, int c8, float *v) {
    const float4 p = *ctab_ptr4(a, b, t, 2 * c8), q = *ctab_ptr4(a, b, t, 2 * c8 + 1);
    v[0] = p.x; v[1] = p.y; v[2] = p.z; v[3] = p.w;
    v[4] = q.x; v[5] = q.y; v[6] = q.z; v[7] = q.w;
}
// Sum of each of 8 values over the 16 lanes of a half-warp.  The lanes exchange halves of the
// vector (8 -> 4 -> 2 -> 1 values); lanes 2i and 2i+1 both end with the total of value i.
__device__ __forceinline__ float halving_sum8(const float *v, int l16) {
    float a4[4], a2[2];
    const bool b3 = l16 & 8, b2 = l16 & 4, b1 = l16 & 2;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float send = b3 ? v[i] : v[4 + i];
        a4[i] = (b3 ? v[4 + i] : v[i]) + __shfl_xor_sync(0xffffffffu, send, 8);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const float send = b2 ? a4[i] : a4[2 + i];
        a2[i] = (b2 ? a4[2 + i] : a4[i]) + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    const float send = b1 ? a2[0] : a2[1];
    float r = (b1 ? a2[1] : a2[0]) + __shfl_xor_sync(0xffffffffu, send, 2);
    r += __shfl_xor_sync(0xffffffffu, r, 1);
    return r;
}

// Eight warps: warps 0..3 and 4..7 share the four 32-lane quarters of tensor memory (warp & 3).
// The two groups split every CUDA-core phase: the operand pass by channels (4 of the 8 channels
// of a tile chunk each), the
// mask pass by score columns, the epilogue by tokens.  The decay-gradient recurrence runs forward
// in both groups; group 1 (tokens 32..63) starts from zero, parks its fp32 values in tensor-memory
// columns it has already consumed and adds the per-channel offset that group 0 publishes when it
// reaches token 31.  (Walking group 1 backward from the chunk-end constant would need no offset,
// but that constant comes from a separately rounded bf16 state and the small residuals of
// strongly decaying channels do not survive the mismatch.)
//
// The body is compiled twice.  MILD_ONLY = true: the chunk is known to be mild (the forward kernel
// said so), every cross-block code path is left out -- a smaller, leaner kernel (96 instead of 125
// registers) that serves every chunk of ordinary data.  MILD_ONLY = false: the general body, run
// only for the chunks the forward kernel listed as steep.
template <bool PER_TOKEN, bool MILD_ONLY>
__device__ __forceinline__ void
bwd_chunk(const CUtensorMap &map_r, const CUtensorMap &map_k, const CUtensorMap &map_v, const CUtensorMap &map_w,
          const CUtensorMap &map_gy, const CUtensorMap &map_s, const CUtensorMap &map_d, const CUtensorMap &map_gr,
          const CUtensorMap &map_gk, const CUtensorMap &map_gv, const CUtensorMap &map_gw, const BwdParams &P,
          const int chunk_id) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    BwdSmem &s = *reinterpret_cast<BwdSmem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // tells the compiler it is uniform across the warp
    const int wg = warp >> 2, w4 = warp & 3;
    const int n = P.nchunk;
    const int bh = chunk_id / n, j = chunk_id % n, b = bh / P.H, h = bh % P.H;
    const bool lo = (lane & 16) == 0;
    const int row = w4 * 16 + (lane & 15);   // accumulator row owned (token in phase 1, channel in phase 2)
    const uint32_t lane_base = (uint32_t)(w4 * 32);

    // the swizzled tiles need a 1024-byte aligned base; refuse to run otherwise
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (tid == 0 && P.status) atomicOr(P.status, 8);
        return;
    }
    const uint32_t LIM = P.wait_limit;
    if (tid == 0) {
        mbar_init(&s.load_bar, 1);
        // lane 0 of every warp commits to every barrier, whether or not it issued a share of the group
        mbar_init(&s.bar_early, 8); mbar_init(&s.bar_score, 8); mbar_init(&s.bar_grad, 8); mbar_init(&s.bar_gv, 8);
        fence_mbar_init();
        if (j != P.skip_load) {
            mbar_expect_tx(&s.load_bar, (PER_TOKEN ? 7 : 6) * TILE_BYTES);
            tma_load_3d(&s.in[T_R], &map_r, &s.load_bar, h * 64, j * CH, b);
            tma_load_3d(&s.in[T_K], &map_k, &s.load_bar, h * 64, j * CH, b);
            tma_load_3d(&s.in[T_V], &map_v, &s.load_bar, h * 64, j * CH, b);
            if (PER_TOKEN) tma_load_3d(&s.in[T_W], &map_w, &s.load_bar, h * 64, j * CH, b);
            tma_load_3d(&s.in[T_GY], &map_gy, &s.load_bar, h * 64, j * CH, b);
            tma_load_3d(&s.in[T_S], &map_s, &s.load_bar, 0, 0, bh * (n + 1) + j);
            tma_load_3d(&s.in[T_D], &map_d, &s.load_bar, 0, 0, bh * (n + 1) + j + 1);
        }
    }
    if (MILD_ONLY && tid == 32) {
        // the CTA that will take this one's place on the SM finds its tiles in L2
        const int nb = chunk_id + P.prefetch_dist;
        if (nb < (int)gridDim.x) {
            const int bh2 = nb / n, j2 = nb % n, b2 = bh2 / P.H, h2 = bh2 % P.H;
            tma_prefetch_l2_3d(&map_r, h2 * 64, j2 * CH, b2);
            tma_prefetch_l2_3d(&map_k, h2 * 64, j2 * CH, b2);
            tma_prefetch_l2_3d(&map_v, h2 * 64, j2 * CH, b2);
            if (PER_TOKEN) tma_prefetch_l2_3d(&map_w, h2 * 64, j2 * CH, b2);
            tma_prefetch_l2_3d(&map_gy, h2 * 64, j2 * CH, b2);
            tma_prefetch_l2_3d(&map_s, 0, 0, bh2 * (n + 1) + j2);
            tma_prefetch_l2_3d(&map_d, 0, 0, bh2 * (n + 1) + j2 + 1);
        }
    }
    // (the flag is read while the loads are in flight: asking first would put a DRAM round trip in front of them)
    if (MILD_ONLY && tid == 64) s.not_mine = P.mildflag[chunk_id] == 0;
    if (tid >= 128 && tid < 128 + CH) s.uf[tid - 128] = __bfloat162float(P.u[h * 64 + tid - 128]);
    if (warp == 0) { tmem_alloc(&s.tmem_base, BWD_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s.tmem_base;
    const uint32_t tm_lo = tm, tm_hi = tm + (16u << 16);
    if (MILD_ONLY && s.not_mine) {
        // a steep chunk: the other kernel computes it.  Let this CTA's loads land, give the tensor memory back.
        if (tid == 0 && chunk_id % P.nchunk != P.skip_load) mbar_wait(&s.load_bar, 0, LIM);
        __syncthreads();
        if (warp == 0) tmem_dealloc(tm, BWD_TMEM_COLS);
        return;
    }

    // operand-pass coordinates (see decay_scan8): 4 tokens x 4 channels per thread, a half-warp per tile row
    const int pblk = warp >> 2, pcc = (lane & 15) >> 1, phf = lane & 1, ptok0 = 8 * warp + 4 * (lane >> 4);
    const int ch0 = pcc * 8 + 4 * phf;
    float lwc[4];
    bool livec[4];
    if (!PER_TOKEN) {
#pragma unroll
        for (int ch = 0; ch < 4; ch++) lwc[ch] = log2_decay(P.wvec[h * 64 + ch0 + ch], P.w_kind, livec[ch]);
    }
    int fail = 0;
    if (!mbar_wait(&s.load_bar, 0, LIM)) fail = 1;

    // The products that need only the raw tiles go to the tensor core before the operand pass
    // (a tcgen05.mma is issued by one thread and costs it ~100 cycles of descriptor arithmetic:
    // the accumulators of a group go out from different warps at once).
    if (lane == 0) {
        const uint32_t id64 = make_idesc(64, 64, false, false), id32 = make_idesc(64, 32, false, false);
        if (!fail) {
            if (warp == 0) {
                // P[t,s] = sum_v gy[t,v] v[s,v]
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(tm_hi + C_P, desc_kmajor(&s.in[T_GY], 0, k), desc_kmajor(&s.in[T_V], 0, k), id64, k > 0);
            } else if (warp < 3) {
                // gr state part: GSr[t, k] = sum_v gy[t,v] S[k,v]; channels 0..31 in lo, 32..63 in hi lanes
                const int hf = warp - 1;
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss((hf ? tm_hi : tm_lo) + C_GSR, desc_kmajor(&s.in[T_GY], 0, k), desc_kmajor(&s.in[T_S], 32 * hf, k), id32, k > 0);
            } else if (warp < 5) {
                // gk state part: GSk[s, k] = sum_v v[s,v] D[k,v]
                const int hf = warp - 3;
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss((hf ? tm_hi : tm_lo) + C_GSK, desc_kmajor(&s.in[T_V], 0, k), desc_kmajor(&s.in[T_D], 32 * hf, k), id32, k > 0);
            }
        }
        mma_commit(&s.bar_early);
    }

    // ---------------------------------------------------------------- operand pass
    // mild chunk (see decay_scan8): one reference point, the end of block 0, for all 64 tokens; the
    // cross-block operands x / P~x and the products A2, G2r, G2k are then not needed
    bool mild = false;
    {
        float c[4][4];
        DecayT<4> D;
        unsigned livebits[4];
        // the warps' decay totals are exchanged through the first bytes of the A~ tile (unused until the mask pass)
        float *wtot = reinterpret_cast<float *>(s.atil.b);
        float other_l2[4], other[4];
        if (!PER_TOKEN && (j + 1) * CH <= P.T) {
            // static decay, whole chunk in range: closed form, nothing to scan or exchange
            float wc[4];
            bool steep = false;
            unsigned lb = 0;
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                wc[ch] = exp2f(lwc[ch]);
                steep |= 8.f * lwc[ch] < MILD_L2_PER_8;
                lb |= (livec[ch] ? 1u : 0u) << ch;
            }
#pragma unroll
            for (int i = 0; i < 4; i++) livebits[i] = lb;
            decay_static(lwc, wc, ptok0, c, D, other_l2);
            mild = __syncthreads_or(steep) == 0;
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int t = ptok0 + i;
                const bool valid = j * CH + t < P.T;
                livebits[i] = 0;
                if (PER_TOKEN) {
                    float x[4];
                    unpack4(ld_tile4(s.in[T_W], t, pcc, phf), x);
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        bool live;
                        const float l2 = log2_decay(x[ch], P.w_kind, live);
                        livebits[i] |= (live ? 1u : 0u) << ch;
                        c[i][ch] = valid ? l2 : 0.f;
                    }
                } else {
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        livebits[i] |= (livec[ch] ? 1u : 0u) << ch;
                        c[i][ch] = valid ? lwc[ch] : 0.f;
                    }
                }
            }
            // (the barrier inside: every w value has been read, so its slot may take the table)
            mild = decay_scan8(c, warp, lane, wtot, D, other_l2, [](bool p) { return __syncthreads_or(p) != 0; });
        }
#pragma unroll
        for (int ch = 0; ch < 4; ch++) other[ch] = exp2f(other_l2[ch]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int t = ptok0 + i;
            float cv[4];      // cumulative log2-decay counted from the chunk start; its lowest mantissa
                              // bit is replaced by the "decay above the floor" flag of the token
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                const float cabs = pblk ? c[i][ch] + other_l2[ch] : c[i][ch];
                cv[ch] = __uint_as_float((__float_as_uint(cabs) & ~1u) | ((livebits[i] >> ch) & 1u));
            }
            *ctab_ptr4(s.in[T_W], s.ctab_hi, t, ch0 >> 2) = make_float4(cv[0], cv[1], cv[2], cv[3]);
        }
        // r-side operands, walking forward:  fa = 2^{cp - m};  block 1 also x = r 2^{cp}  (block-local cp)
        float fa[4], fb[4], ref[4];      // ref: the reference point of the same-block factors (block-local)
#pragma unroll
        for (int ch = 0; ch < 4; ch++) {
            ref[ch] = mild ? (pblk ? 0.f : D.e[ch]) : D.m[ch];
            fa[ch] = exp2f(D.cp0[ch] - ref[ch]);
            fb[ch] = exp2f(D.cp0[ch]);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int t = ptok0 + i;
            float r[4], rt[4], xx[4];
            unpack4(ld_tile4(s.in[T_R], t, pcc, phf), r);
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                rt[ch] = r[ch] * fa[ch];
                fa[ch] *= D.w[i][ch];
            }
            st_tile4(s.rt, t, pcc, phf, pack4(rt));
            if (pblk && !mild) {
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    xx[ch] = r[ch] * fb[ch];
                    fb[ch] *= D.w[i][ch];
                }
                st_tile4(s.x, t, pcc, phf, pack4(xx));
            }
        }
        // k-side operands, walking backward:  fa = 2^{m - c};  fb = 2^{e - c}
        //   block 0: x = k fb, khat = x 2^{total of block 1}      block 1: khat = k fb
        if (mild) {
            // one reference point: khat is kt times a per-channel constant (block 0: kt = k 2^{e0 - c},
            // khat = kt 2^{total of block 1};  block 1: kt = k 2^{-c}, khat = kt 2^{total of block 1})
            float ck[4];
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                fa[ch] = exp2f(ref[ch] - D.c3[ch]);
                ck[ch] = pblk ? exp2f(D.e[ch]) : other[ch];
            }
#pragma unroll
            for (int i = 3; i >= 0; i--) {
                const int t = ptok0 + i;
                float k[4], kt[4], kh[4];
                unpack4(ld_tile4(s.in[T_K], t, pcc, phf), k);
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    kt[ch] = k[ch] * fa[ch];
                    kh[ch] = kt[ch] * ck[ch];
                    fa[ch] *= D.w[i][ch];
                }
                st_tile4(s.kt, t, pcc, phf, pack4(kt));
                st_tile4(s.khat, t, pcc, phf, pack4(kh));
            }
        } else {
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                fa[ch] = exp2f(ref[ch] - D.c3[ch]);
                fb[ch] = exp2f(D.e[ch] - D.c3[ch]);
            }
#pragma unroll
            for (int i = 3; i >= 0; i--) {
                const int t = ptok0 + i;
                float k[4], kt[4], kh[4], xx[4];
                unpack4(ld_tile4(s.in[T_K], t, pcc, phf), k);
#pragma unroll
                for (int ch = 0; ch < 4; ch++) {
                    kt[ch] = k[ch] * fa[ch];
                    xx[ch] = k[ch] * fb[ch];
                    kh[ch] = pblk ? xx[ch] : xx[ch] * other[ch];
                    fa[ch] *= D.w[i][ch];
                    fb[ch] *= D.w[i][ch];
                }
                st_tile4(s.kt, t, pcc, phf, pack4(kt));
                if (!pblk) st_tile4(s.x, t, pcc, phf, pack4(xx));
                st_tile4(s.khat, t, pcc, phf, pack4(kh));
            }
        }
    }
    if (MILD_ONLY) mild = true;      // (what the scan just found as well; as a constant it removes the steep code)
    fence_async_smem();
    tc_fence_before();
    const int abort1 = __syncthreads_or(fail);

    // ------------------------------------------------- phase 1: the scores A1, A2
    if (lane == 0) {
        if (!abort1) {
            tc_fence_after();
            if (warp == 0) {
                const uint32_t id64 = make_idesc(64, 64, false, false);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(tm_lo + C_A1, desc_kmajor(&s.rt, 0, k), desc_kmajor(&s.kt, 0, k), id64, k > 0);
            } else if (warp == 1 && !mild) {
                const uint32_t id32 = make_idesc(64, 32, false, false);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    mma_ss(tm_lo + C_A2, desc_kmajor(&s.x, 0, k), desc_kmajor(&s.x, 0, k), id32, k > 0);
            }
        }
        mma_commit(&s.bar_score);
    }
    // meanwhile: the bonus term of the score diagonal, sum_k r_t u k_t, in the warps whose 16 rows x
    // 32 columns straddle the diagonal; the lo lane takes channels 0..31 of the row, the hi lane 32..63
    const int col0 = 32 * wg;                       // score columns this group masks
    const bool diag_warp = (w4 >= 2) == (wg == 1), cross_warp = wg == 0 && w4 >= 2;
    float diag = 0.f;
    if (diag_warp) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int c8 = (lo ? 0 : 4) + c;
            float a[8], d[8], uq[8];
            unpack8(ld_tile(s.in[T_R], row, c8), a);
            unpack8(ld_tile(s.in[T_K], row, c8), d);
            {
                const float4 u0 = *reinterpret_cast<const float4 *>(s.uf + 8 * c8), u1 = *reinterpret_cast<const float4 *>(s.uf + 8 * c8 + 4);
                uq[0] = u0.x; uq[1] = u0.y; uq[2] = u0.z; uq[3] = u0.w; uq[4] = u1.x; uq[5] = u1.y; uq[6] = u1.z; uq[7] = u1.w;
            }
#pragma unroll
            for (int q = 0; q < 8; q++) diag += a[q] * uq[q] * d[q];
        }
        diag += __shfl_xor_sync(0xffffffffu, diag, 16);
    }
    if (!abort1 && !(mbar_wait(&s.bar_early, 0, LIM) && mbar_wait(&s.bar_score, 0, LIM))) fail = 1;
    tc_fence_after();

    // mask pass: lo lanes build A~ (row t), hi lanes build P~ (row t); this group's 32 columns.
    // P~ is split: its two same-block triangles go to the P~ tile (cross block zero), the
    // cross block (t >= 32, s < 32) to the same rows of the v tile, whose readers are done.
    {
        const int t = row;
        float a[32];
        // columns col0..+31 of A1 (lo lanes) and of P (hi lanes) share their tensor-memory columns
        if (diag_warp || cross_warp) {
            tmem_ld16(tmem_addr(tm, lane_base, C_A1 + col0), a);
            tmem_ld16(tmem_addr(tm, lane_base, C_A1 + col0 + 16), a + 16);
        }
        if (cross_warp && mild) {   // rows 32..63, columns 0..31: every entry kept; A1 holds the cross-block scores too
            tmem_ld_wait();
        } else if (cross_warp) {    // ... A~ takes the cross-block scores from their own product
            float a2[32];
            tmem_ld16(tmem_addr(tm, lane_base, C_A2), a2);
            tmem_ld16(tmem_addr(tm, lane_base, C_A2 + 16), a2 + 16);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 32; q++) a[q] = lo ? a2[q] : a[q];
        } else if (diag_warp) {
            tmem_ld_wait();
            // local row lim = t - col0: columns below it are kept, column lim is the diagonal (the bonus
            // term in A~, p_tt set aside and zero in P~).  Rows 0..15 of the block cannot reach columns
            // 16..31, rows 16..31 keep all of columns 0..15.
            const float dval = lo ? diag : 0.f;
            float pt = 0.f;
            if ((w4 & 1) == 0) {
                const int lim = t - col0;
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    if (q == lim) pt = a[q];
                    a[q] = q < lim ? a[q] : (q == lim ? dval : 0.f);
                    a[16 + q] = 0.f;
                }
            } else {
                const int lim = t - col0 - 16;
#pragma unroll
                for (int q = 0; q < 16; q++) {
                    if (q == lim) pt = a[16 + q];
                    a[16 + q] = q < lim ? a[16 + q] : (q == lim ? dval : 0.f);
                }
            }
            if (!lo) s.ptt[t] = pt;
        } else {                    // upper-right block: nothing survives
#pragma unroll
            for (int q = 0; q < 32; q++) a[q] = 0.f;
        }
        Tile &dst = lo ? s.atil : (cross_warp && !mild ? s.in[T_V] : s.ptil);
#pragma unroll
        for (int c8 = 0; c8 < 4; c8++) st_tile(dst, t, (col0 >> 3) + c8, pack8(a + 8 * c8));
        if (cross_warp && !mild && !lo) {
#pragma unroll
            for (int c8 = 0; c8 < 4; c8++) st_tile(s.ptil, t, c8, make_uint4(0u, 0u, 0u, 0u));
        }
    }
    fence_async_smem();
    tc_fence_before();
    const int abort2 = __syncthreads_or(fail) | abort1;

    // ------------------------------------------------- phase 2: token-major accumulators
    // every accumulator is [token, 32 channels]: channels 0..31 in the lo lanes, 32..63 in the hi lanes
    // gv is needed last: it goes to a barrier of its own, from the two warps that have no gradient
    // product to issue (so that no warp enters the epilogue later than the others).
    if (lane == 0) {
        tc_fence_after();
        const uint32_t id_kn = make_idesc(64, 32, false, true), id_nn = make_idesc(64, 32, true, true);
        const int hf = warp & 1;
        const uint32_t tmh = hf ? tm_hi : tm_lo;
        const uint64_t boff = hf ? 4 : 0;     // +64 bytes: the upper 32 of the 64 contiguous elements
        if (abort2) {
            mma_commit(&s.bar_grad);          // nothing is issued
        } else if (warp == 0 && !mild) {
            // gr intra, across blocks: G2r[t >= 32, k] = sum_{s<32} P~x[t,s] X[s,k]   (rows t < 32 are not read)
#pragma unroll
            for (int hq = 0; hq < 2; hq++)
#pragma unroll
                for (int k = 0; k < 2; k++)
                    mma_ss((hq ? tm_hi : tm_lo) + C_G2R, desc_kmajor(&s.in[T_V], 0, k),
                           desc_mnmajor(&s.x, 0, k) + (hq ? 4 : 0), id_kn, k > 0);
            mma_commit(&s.bar_grad);
        } else if (warp == 1 && !mild) {
            // gk intra, across blocks: G2k[s < 32, k] = sum_{t>=32} P~x[t,s] X[t,k]   (rows s >= 32 are not read)
#pragma unroll
            for (int hq = 0; hq < 2; hq++)
#pragma unroll
                for (int k = 0; k < 2; k++)
                    mma_ss((hq ? tm_hi : tm_lo) + C_G2K, desc_mnmajor(&s.in[T_V], 32, k),
                           desc_mnmajor(&s.x, 32, k) + (hq ? 4 : 0), id_nn, k > 0);
            mma_commit(&s.bar_grad);
        } else if (warp == 2 || warp == 3) {
            // gr intra, same block (mild chunk: the whole chunk): G1r[t,k] = sum_s P~d[t,s] Kt[s,k]
#pragma unroll
            for (int k = 0; k < 4; k++)
                mma_ss(tmh + C_G1R, desc_kmajor(&s.ptil, 0, k), desc_mnmajor(&s.kt, 0, k) + boff, id_kn, k > 0);
            mma_commit(&s.bar_grad);
        } else if (warp == 4 || warp == 5) {
            // gk intra, same block (mild chunk: the whole chunk): G1k[s,k] = sum_t P~d[t,s] Rt[t,k]
#pragma unroll
            for (int k = 0; k < 4; k++)
                mma_ss(tmh + C_G1K, desc_mnmajor(&s.ptil, 0, k), desc_mnmajor(&s.rt, 0, k) + boff, id_nn, k > 0);
            mma_commit(&s.bar_grad);
        } else {
            mma_commit(&s.bar_grad);
        }
        if (!abort2 && warp >= 6) {
            // gv[s, v] = sum_t A~[t,s] gy[t,v] + sum_k khat[s,k] D[k,v]
#pragma unroll
            for (int k = 0; k < 4; k++)
                mma_ss(tmh + C_GV, desc_mnmajor(&s.atil, 0, k), desc_mnmajor(&s.in[T_GY], 0, k) + boff, id_nn, k > 0);
#pragma unroll
            for (int k = 0; k < 4; k++)
                mma_ss(tmh + C_GV, desc_kmajor(&s.khat, 0, k), desc_mnmajor(&s.in[T_D], 0, k) + boff, id_kn, true);
        }
        mma_commit(&s.bar_gv);
    }

    // ------------------------------------------------- epilogue
    // A thread owns token t = row and the 32 channels of its lane half; group 0 is the gr side,
    // group 1 the gk side.  While gv is still being accumulated (from A~, gy, khat, D) only tiles
    // outside that product are touched: gr and gk are staged in place of the scaled operands each
    // thread has just consumed (gr->rt, gk->kt), S and the P~ tile carry the exchange between the
    // groups, the v tile the per-warp sums.  Once gv is done: gv->gy, gw->D.
    Tile &o_gr = s.rt, &o_gk = s.kt, &o_gw = s.in[T_D], &o_gv = s.in[T_GY];
    Tile &ct_lo = s.in[T_W], &ct_hi = s.ctab_hi;
    const int t = row, hh = lane >> 4, l16 = lane & 15;
    const float ptt_t = s.ptt[t];
    const bool tvalid = j * CH + t < P.T;
    // [4][64] totals of the token scan, and [4][64] partial sums for gu / the static gw.  General build:
    // per warp, in the v tile.  Mild-only build: per quarter of the chunk's tokens, in the A~ tile (free
    // once gv is done; the v tile holds part of the a/b exchange there).
    float *wtot = reinterpret_cast<float *>(MILD_ONLY ? s.atil.b : s.in[T_V].b);
    float *gup = wtot + 4 * CH, *gwp = gup + 4 * CH;
    float keep[16];   // (general build) group 0: a_t of its first 16 channels; group 1: b_t of its last 16 channels

    // decay-gradient constant sum_v S[k,v] D[k,v] at the chunk start (consumed after two more barriers)
    if (tid < CH) s.kb[tid] = P.e0[((size_t)bh * (n + 1) + j) * 64 + tid];
    if (!abort2 && !mbar_wait(&s.bar_grad, 0, LIM)) fail = 1;
    tc_fence_after();

    // The decay gradient of token t is  glw_t = K_j + sum_{t'<=t} (a_t' + b_t') - b_t  with
    //   a_t = -(qrS_t + qrI_t)   (gr side),     b_t = qkD_t + qkI_t   (gk side),
    // qrS/qkD the state parts of r*gr and k*gk and qrI/qkI their intra-chunk parts (file header).
    auto side_pass = [&](auto side_tag, auto mild_tag) {
        constexpr bool GR = decltype(side_tag)::value;
        constexpr bool MILD = decltype(mild_tag)::value;      // compiled twice: without / with the cross-block terms
        const bool has2 = !MILD && (GR ? (w4 >= 2) : (w4 < 2));   // the cross-block accumulator covers this token
        const Tile &t_own = GR ? s.rt : s.kt;
        const Tile &t_raw = GR ? s.in[T_R] : s.in[T_K], &t_oth = GR ? s.in[T_K] : s.in[T_R];
        constexpr int cGS = GR ? C_GSR : C_GSK, cG1 = GR ? C_G1R : C_G1K, cG2 = GR ? C_G2R : C_G2K;
        Tile &o_main = GR ? o_gr : o_gk;
        Tile &exch = GR ? s.in[T_S] : s.ptil;                 // what the other group needs from this one
        const int zrow = GR ? t - 1 : t;                      // gr factors use c_{t-1}, gk factors c_t
        const int mrow = MILD ? 31 : (t < HB ? 15 : 47);          // row of the table that holds the reference point
#pragma unroll 1
        for (int bt = 0; bt < 4; bt++) {
            const int c8 = 4 * hh + bt;       // 16-byte column of the bf16 tiles; channels 8*c8 .. +7
            float g1[8], gs[8], g2[8];
            tmem_ld8(tmem_addr(tm, lane_base, cG1 + 8 * bt), g1);
            tmem_ld8(tmem_addr(tm, lane_base, cGS + 8 * bt), gs);
            if (has2) tmem_ld8(tmem_addr(tm, lane_base, cG2 + 8 * bt), g2);
            float own[8], raw[8], oth[8], xx[8], uu[8], z[8], mb[8], e0r[8], e1r[8];
            unpack8(ld_tile(t_own, t, c8), own);
            unpack8(ld_tile(t_raw, t, c8), raw);
            unpack8(ld_tile(t_oth, t, c8), oth);
            {
                const float4 u0 = *reinterpret_cast<const float4 *>(s.uf + 8 * c8), u1 = *reinterpret_cast<const float4 *>(s.uf + 8 * c8 + 4);
                uu[0] = u0.x; uu[1] = u0.y; uu[2] = u0.z; uu[3] = u0.w; uu[4] = u1.x; uu[5] = u1.y; uu[6] = u1.z; uu[7] = u1.w;
            }
            ld_ctab8(ct_lo, ct_hi, mrow, c8, mb);
            if (zrow >= 0) {
                ld_ctab8(ct_lo, ct_hi, zrow, c8, z);
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) z[q] = 0.f;
            }
            if (!GR) ld_ctab8(ct_lo, ct_hi, 63, c8, e1r);
            if (has2) {
                unpack8(ld_tile(s.x, t, c8), xx);
                ld_ctab8(ct_lo, ct_hi, 31, c8, e0r);
            }
            tmem_ld_wait();
            float out[8], ab[8], gue[8];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float f1 = GR ? exp2f(z[q] - mb[q]) : exp2f(mb[q] - z[q]);
                const float fS = GR ? exp2f(z[q]) : exp2f(e1r[q] - z[q]);
                const float sgs = fS * gs[q];
                float o = f1 * g1[q] + sgs + ptt_t * uu[q] * oth[q];
                float qq = own[q] * g1[q] + raw[q] * sgs;
                if (has2) {
                    const float f3 = GR ? exp2f(z[q] - e0r[q]) : exp2f(e0r[q] - z[q]);
                    o += f3 * g2[q];
                    qq += xx[q] * g2[q];
                }
                out[q] = o;
                ab[q] = GR ? -qq : qq;
                if (!GR && !MILD_ONLY) gue[q] = ptt_t * raw[q] * oth[q];
            }
            st_tile(o_main, t, c8, pack8(out));
            if constexpr (MILD_ONLY) {
                // a_t (gr side) / b_t (gk side) of the lane half's 32 channels: one fp32 row of a tile of
                // their own (a: S and P~ tiles, b: v and x tiles -- all consumed by now), read back
                // channel-major by the token scan below
                Tile &dstt = GR ? (hh ? s.ptil : s.in[T_S]) : (hh ? s.x : s.in[T_V]);
                *reinterpret_cast<float4 *>(dstt.b + tile_off(t, 2 * bt)) = make_float4(ab[0], ab[1], ab[2], ab[3]);
                *reinterpret_cast<float4 *>(dstt.b + tile_off(t, 2 * bt + 1)) = make_float4(ab[4], ab[5], ab[6], ab[7]);
                continue;
            }
            const bool mine = GR ? (bt < 2) : (bt >= 2);
            if (mine) {
                if (bt & 1) {
#pragma unroll
                    for (int q = 0; q < 8; q++) keep[8 + q] = ab[q];
                } else {
#pragma unroll
                    for (int q = 0; q < 8; q++) keep[q] = ab[q];
                }
            } else {
                float4 *dst = reinterpret_cast<float4 *>(exch.b + tile_off(t, 4 * hh + 2 * (bt & 1)));
                dst[0] = make_float4(ab[0], ab[1], ab[2], ab[3]);
                *reinterpret_cast<float4 *>(exch.b + tile_off(t, 4 * hh + 2 * (bt & 1) + 1)) =
                    make_float4(ab[4], ab[5], ab[6], ab[7]);
            }
            if (!GR) {
                // gu: sum over this warp's 16 tokens of p_tt r k, by a halving exchange
                const float tot = halving_sum8(gue, l16);
                if ((l16 & 1) == 0) gup[w4 * CH + 8 * c8 + (l16 >> 1)] = tot;
            }
        }
    };
    if (mild) {
        if (wg == 0) side_pass(std::true_type{}, std::true_type{}); else side_pass(std::false_type{}, std::true_type{});
    } else {
        if (wg == 0) side_pass(std::true_type{}, std::false_type{}); else side_pass(std::false_type{}, std::false_type{});
    }
    if (wg == 0) {
        // gv: accumulator [s, v]
        if (!abort2 && !mbar_wait(&s.bar_gv, 0, LIM)) fail = 1;
        tc_fence_after();
        float gv[32];
        tmem_ld16(tmem_addr(tm, lane_base, C_GV), gv);
        tmem_ld16(tmem_addr(tm, lane_base, C_GV + 16), gv + 16);
        tmem_ld_wait();
#pragma unroll
        for (int c8 = 0; c8 < 4; c8++) st_tile(o_gv, t, 4 * hh + c8, pack8(gv + 8 * c8));
    }
    __syncthreads();
    if constexpr (MILD_ONLY) {
        // Token scan, channel-major: thread = one channel c and one quarter q4 of the chunk's tokens.
        // a and b of its 16 tokens come from the exchange tiles (a warp reads 32 consecutive floats of
        // a row: no bank conflict); the exclusive prefix of z = a + b is a serial sum in registers, the
        // quarters meet through `wtot`.  gu's partial sum p_tt r k rides along.
        const int c = tid & 63, q4 = tid >> 6, cl = c & 31;
        const Tile &ta = (c & 32) ? s.ptil : s.in[T_S], &tb = (c & 32) ? s.x : s.in[T_V];
        float av[16], pre[16];
        float run = 0.f, gus = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int tt = 16 * q4 + i;
            const uint32_t off = tile_off(tt, cl >> 2) + (cl & 3) * 4;
            const float a = *reinterpret_cast<const float *>(ta.b + off);
            const float b = *reinterpret_cast<const float *>(tb.b + off);
            av[i] = a;
            pre[i] = run;
            run += a + b;
            const uint32_t boff = tile_off(tt, c >> 3) + (c & 7) * 2;
            const float rr = __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(s.in[T_R].b + boff));
            const float kk = __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(s.in[T_K].b + boff));
            gus = fmaf(s.ptt[tt] * rr, kk, gus);
        }
        wtot[q4 * CH + c] = run;
        gup[q4 * CH + c] = gus;
        __syncthreads();
        float base = s.kb[c];      // the constant of the chunk start plus the earlier quarters' totals
        for (int w = 0; w < q4; w++) base += wtot[w * CH + c];
        if (PER_TOKEN) {
            // times the floored log-decay of the token, zero where the floor was hit (no gradient)
            auto ctab1 = [&](int tt) { return reinterpret_cast<const float *>(ctab_ptr4(ct_lo, ct_hi, tt, c >> 2))[c & 3]; };
            float cprev = q4 ? ctab1(16 * q4 - 1) : 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int tt = 16 * q4 + i;
                const float cc = ctab1(tt);
                const float glw = base + pre[i] + av[i];
                const float o = (__float_as_uint(cc) & 1u) ? glw * (cc - cprev) * LN2 : 0.f;
                cprev = cc;
                *reinterpret_cast<__nv_bfloat16 *>(o_gw.b + tile_off(tt, c >> 3) + (c & 7) * 2) = __float2bfloat16_rn(o);
            }
        } else {
            float tot = 0.f;
#pragma unroll
            for (int i = 0; i < 16; i++)
                if (j * CH + 16 * q4 + i < P.T) tot += base + pre[i] + av[i];
            gwp[q4 * CH + c] = tot;
        }
    } else {
        // the token scan of z = a + b for this thread's 16 channels: 32*hh + 16*wg .. +15
        float bsub[16];
        {
            const Tile &got = wg ? s.in[T_S] : s.ptil;         // what the other group left for this one
    #pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                const float4 o = *reinterpret_cast<const float4 *>(got.b + tile_off(t, 4 * hh + c4));
                const float ov[4] = {o.x, o.y, o.z, o.w};
    #pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int i = 4 * c4 + q;
                    bsub[i] = wg ? keep[i] : ov[q];            // b_t
                    keep[i] += ov[q];                          // z_t
                }
            }
    #pragma unroll
            for (int off = 1; off < 16; off <<= 1) {
    #pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float o = __shfl_up_sync(0xffffffffu, keep[i], off, 16);
                    if (l16 >= off) keep[i] += o;
                }
            }
            if (l16 == 15) {
    #pragma unroll
                for (int c4 = 0; c4 < 4; c4++)
                    *reinterpret_cast<float4 *>(wtot + w4 * CH + 32 * hh + 16 * wg + 4 * c4) =
                        make_float4(keep[4 * c4], keep[4 * c4 + 1], keep[4 * c4 + 2], keep[4 * c4 + 3]);
            }
        }
        __syncthreads();
        {
            const int kb0 = 32 * hh + 16 * wg;                 // first of the 16 channels
            float glw[16];
            // the constant of the chunk start plus the earlier warps' totals
    #pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                float4 o = *reinterpret_cast<const float4 *>(s.kb + kb0 + 4 * c4);
                for (int w = 0; w < w4; w++) {
                    const float4 p = *reinterpret_cast<const float4 *>(wtot + w * CH + kb0 + 4 * c4);
                    o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
                }
                glw[4 * c4] = o.x + keep[4 * c4] - bsub[4 * c4];
                glw[4 * c4 + 1] = o.y + keep[4 * c4 + 1] - bsub[4 * c4 + 1];
                glw[4 * c4 + 2] = o.z + keep[4 * c4 + 2] - bsub[4 * c4 + 2];
                glw[4 * c4 + 3] = o.w + keep[4 * c4 + 3] - bsub[4 * c4 + 3];
            }
            if (PER_TOKEN) {
                // times the floored log-decay of the token, zero where the floor was hit (no gradient)
    #pragma unroll
                for (int c2 = 0; c2 < 2; c2++) {
                    const int c8 = (kb0 >> 3) + c2;
                    float c[8], cp[8];
                    ld_ctab8(ct_lo, ct_hi, t, c8, c);
                    if (t > 0) {
                        ld_ctab8(ct_lo, ct_hi, t - 1, c8, cp);
                    } else {
    #pragma unroll
                        for (int q = 0; q < 8; q++) cp[q] = 0.f;
                    }
                    float o[8];
    #pragma unroll
                    for (int q = 0; q < 8; q++)
                        o[q] = (__float_as_uint(c[q]) & 1u) ? glw[8 * c2 + q] * (c[q] - cp[q]) * LN2 : 0.f;
                    st_tile(o_gw, t, c8, pack8(o));
                }
            } else {
    #pragma unroll
                for (int c2 = 0; c2 < 2; c2++) {
                    float e[8];
    #pragma unroll
                    for (int q = 0; q < 8; q++) e[q] = tvalid ? glw[8 * c2 + q] : 0.f;
                    const float tot = halving_sum8(e, l16);
                    if ((l16 & 1) == 0) gwp[w4 * CH + kb0 + 8 * c2 + (l16 >> 1)] = tot;
                }
            }
        }
    }
    fence_async_smem();
    tc_fence_before();
    const int abort3 = __syncthreads_or(fail) | abort2;
    if (!abort3 && tid == 0) {
        tma_store_3d(&map_gr, &o_gr, h * 64, j * CH, b);
        tma_store_3d(&map_gk, &o_gk, h * 64, j * CH, b);
        tma_store_3d(&map_gv, &o_gv, h * 64, j * CH, b);
        if (PER_TOKEN) tma_store_3d(&map_gw, &o_gw, h * 64, j * CH, b);
        tma_store_commit();
    }
    // per-chunk partials, folded later in a fixed order
    if (tid >= 64 && tid < 128) {
        const int k = tid - 64;
        P.gu_part[((size_t)bh * n + j) * 64 + k] = gup[k] + gup[CH + k] + gup[2 * CH + k] + gup[3 * CH + k];
    } else if (!PER_TOKEN && tid >= 128 && tid < 192) {
        const int k = tid - 128;
        bool live;
        const float lw = log2_decay(P.wvec[h * 64 + k], P.w_kind, live) * LN2;
        const float tot = gwp[k] + gwp[CH + k] + gwp[2 * CH + k] + gwp[3 * CH + k];
        P.gw_part[((size_t)bh * n + j) * 64 + k] = live ? tot * lw : 0.f;
    }
    if (!abort3 && tid == 0) tma_store_wait_read();   // the tiles must outlive the reads of the bulk stores
    if (abort3 && tid == 0) {
        // every warp has arrived on every barrier: whatever was issued is done once they complete
        mbar_wait(&s.bar_early, 0); mbar_wait(&s.bar_score, 0); mbar_wait(&s.bar_grad, 0); mbar_wait(&s.bar_gv, 0);
        if (P.status) atomicOr(P.status, 4);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tm, BWD_TMEM_COLS);
}

#define BWD_MAPS                                                                                              \
    const __grid_constant__ CUtensorMap map_r, const __grid_constant__ CUtensorMap map_k,                    \
        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_w,                \
        const __grid_constant__ CUtensorMap map_gy, const __grid_constant__ CUtensorMap map_s,               \
        const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_gr,               \
        const __grid_constant__ CUtensorMap map_gk, const __grid_constant__ CUtensorMap map_gv,              \
        const __grid_constant__ CUtensorMap map_gw
#define BWD_MAP_ARGS map_r, map_k, map_v, map_w, map_gy, map_s, map_d, map_gr, map_gk, map_gv, map_gw

// one CTA per (batch, head, chunk); CTAs of steep chunks leave early (the other kernel has them)
template <bool PER_TOKEN>
__global__ void __launch_bounds__(256, 2) k_chunk_bwd(BWD_MAPS, const BwdParams P) {
    pdl_wait();
    pdl_trigger();
    bwd_chunk<PER_TOKEN, true>(BWD_MAP_ARGS, P, (int)blockIdx.x);
}

// A fixed, small grid that looks through the mild flags for steep chunks (usually there is none and
// every CTA leaves after one load) and runs the general body on them.  CTA c looks at chunks
// c, c + grid, c + 2 grid, ...: 256 of them per round, one flag per thread.
// One CTA per SM: the general body inside a loop wants more than the 128 registers two CTAs leave.
template <bool PER_TOKEN>
__global__ void __launch_bounds__(256, 1) k_chunk_bwd_steep(BWD_MAPS, const BwdParams P, const int total) {
    pdl_wait();
    pdl_trigger();
    __shared__ unsigned char is_steep[256];
    for (int base = blockIdx.x; base < total; base += 256 * gridDim.x) {
        const int mine = base + threadIdx.x * gridDim.x;
        const bool steep = mine < total && P.mildflag[mine] == 0;
        is_steep[threadIdx.x] = steep ? 1 : 0;
        if (!__syncthreads_or(steep)) continue;
        for (int t = 0; t < 256; t++) {
            if (is_steep[t]) {      // (the same for every thread of the CTA)
                bwd_chunk<PER_TOKEN, false>(BWD_MAP_ARGS, P, base + t * gridDim.x);
                __syncthreads();    // the barriers and the tensor memory of this chunk are done with
            }
        }
        __syncthreads();
    }
}

// sum the per-chunk partials: out[bh*64 + k] = sum_j part[(bh*n + j)*64 + k]
__global__ void k_reduce_partials(const float *__restrict__ part, float *__restrict__ out, int n, int total) {
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int bh = i >> 6, k = i & 63;
    float acc = 0.f;
    for (int j = 0; j < n; j++) acc += part[((size_t)bh * n + j) * 64 + k];
    out[i] = acc;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct BwdLayout {
    size_t status, sck, dck, e0, gu_part, gw_part, groups, wconv, total;
};
BwdLayout bwd_layout(const wkv_args_t *a, bool per_token_w) {
    const size_t n = (a->T + CH - 1) / CH, bh = (size_t)a->B * a->H;
    const GroupPlan gp = plan_groups((int)bh, (int)n, a->time_groups);
    BwdLayout L;
    L.status = 0;
    L.sck = 256;
    L.dck = L.sck + align256(ckpt_layout(a->B, a->T, a->H).total);
    L.e0 = L.dck + align256(bh * (n + 1) * 64 * 64 * 2);
    L.gu_part = L.e0 + align256(bh * (n + 1) * 64 * 4);
    L.gw_part = L.gu_part + align256(bh * n * 64 * 4);
    L.groups = L.gw_part + (per_token_w ? 0 : align256(bh * n * 64 * 4));
    // one region serves the forward re-run (when no hand-over was given) and then the dS scan
    L.wconv = L.groups + (gp.G > 1 ? group_layout(bh * gp.G).total : 0);
    L.total = L.wconv + chunked_wconv_bytes(a, per_token_w);
    return L;
}

}  // namespace

size_t chunked_backward_workspace(const wkv_args_t *a, bool per_token_w) { return bwd_layout(a, per_token_w).total; }

int chunked_backward(const wkv_args_t *a0, bool per_token_w, const ChunkedTest &tst, cudaStream_t stream) {
    wkv_args_t args = *a0;
    wkv_args_t *a = &args;
    const int B = a->B, T = a->T, H = a->H, C = H * 64, n = (T + CH - 1) / CH, BH = B * H;
    const BwdLayout L = bwd_layout(a, per_token_w);
    char *ws = (char *)a->workspace;
    if (cudaMemsetAsync(ws, 0, 256, stream) != cudaSuccess) return WKV_ERR_LAUNCH;
    if (chunked_convert_w(a, per_token_w, ws + L.wconv, stream) != WKV_OK) return WKV_ERR_LAUNCH;
    // what the forward kernel leaves for this call: chunk-start states, r e^{cp}, chunk decays
    char *fwd_ck = a->state_ckpt ? (char *)a->state_ckpt : ws + L.sck;
    const CkptLayout CL = ckpt_layout(B, T, H);
    void *sck = fwd_ck + CL.sck, *dck = ws + L.dck;
    float *gu_part = (float *)(ws + L.gu_part), *gw_part = (float *)(ws + L.gw_part), *e0 = (float *)(ws + L.e0);

    // 1. chunk-start states (unless the forward call handed them over)
    if (!a->state_ckpt) {
        wkv_args_t f = *a;
        f.y = nullptr;
        f.state_out = nullptr;
        f.group_states = nullptr;
        f.group_states_mode = WKV_GROUP_STATES_NONE;
        const int err = chunked_forward_impl(&f, per_token_w, fwd_ck, ws + L.groups, tst, stream);
        if (err != WKV_OK) return err;
    }
    CUtensorMap mr, mk, mv, mw, mgy, ms, md, mgr, mgk, mgv, mgw, mrh;
    bool ok = make_btc_map(&mr, a->r, B, T, C) && make_btc_map(&mk, a->k, B, T, C) &&
              make_btc_map(&mv, a->v, B, T, C) && make_btc_map(&mgy, a->gy, B, T, C) &&
              make_btc_map(&mgr, a->gr, B, T, C) && make_btc_map(&mgk, a->gk, B, T, C) &&
              make_btc_map(&mgv, a->gv, B, T, C) && make_btc_map(&ms, sck, BH * (n + 1), 64, 64) &&
              make_btc_map(&md, dck, BH * (n + 1), 64, 64) && make_btc_map(&mrh, fwd_ck + CL.rhat, B, T, C);
    if (per_token_w) ok = ok && make_btc_map(&mw, a->w, B, T, C) && make_btc_map(&mgw, a->gw, B, T, C);
    else { mw = mr; mgw = mgr; }
    if (!ok) return WKV_ERR_LAUNCH;

    // 2. dS scan (with time groups: summary pass, group scan, full pass)
    {
        const GroupPlan gp = plan_groups(BH, n, a->time_groups);
        const GroupLayout GL = group_layout((size_t)BH * gp.G);
        char *g = ws + L.groups;
        DscanParams p;
        p.T = T; p.H = H; p.nchunk = n; p.layout = a->state_layout;
        p.G = gp.G; p.L = gp.L;
        p.dchunk = (const float *)(fwd_ck + CL.dchunk);
        p.dck = (__nv_bfloat16 *)dck; p.e0 = e0; p.status = (int *)ws;
        p.wait_limit = tst.wait_limit;
        p.skip_load = tst.kernel == 1 ? tst.skip_load : -1;
        const size_t smem = sizeof(DscanSmem) + 1024;
        static unsigned char attr_done[64];
        if (!set_max_smem_once(k_chunk_dscan, (int)smem, attr_done)) return WKV_ERR_LAUNCH;
        if (gp.G > 1) {
            p.summary = 1;
            p.gstate_out = nullptr; p.gstart = nullptr; p.gstate_in = nullptr;
            p.gU = (float *)(g + GL.gU); p.gD = (float *)(g + GL.gD);
            if (launch_chained(k_chunk_dscan, dim3(BH * gp.G), dim3(160), smem, stream, mrh, mgy, ms, p) != WKV_OK)
                return WKV_ERR_LAUNCH;
            if (launch_group_scan(g, BH, gp.G, a->gstate_out, a->gstate_in, a->state_layout, true, stream) != WKV_OK)
                return WKV_ERR_LAUNCH;
        }
        p.summary = 0;
        p.gstate_out = a->gstate_out;
        p.gstart = gp.G > 1 ? (const float *)(g + GL.gstart) : nullptr;
        p.gstate_in = gp.G > 1 ? nullptr : a->gstate_in;
        p.gU = nullptr; p.gD = nullptr;
        if (launch_chained(k_chunk_dscan, dim3(BH * gp.G), dim3(160), smem, stream, mrh, mgy, ms, p) != WKV_OK)
            return WKV_ERR_LAUNCH;
    }
    // 3. per-chunk gradients
    {
        BwdParams p;
        p.T = T; p.H = H; p.nchunk = n; p.w_kind = a->w_kind;
        p.prefetch_dist = 2 * device_sm_count();      // two CTAs of this kernel fit on an SM
        p.u = (const __nv_bfloat16 *)a->u;
        p.wvec = per_token_w ? nullptr : (const float *)a->w;
        p.e0 = e0; p.gu_part = gu_part; p.gw_part = gw_part; p.status = (int *)ws;
        p.wait_limit = tst.wait_limit;
        p.skip_load = tst.kernel == 2 ? tst.skip_load : -1;
        p.mildflag = (const unsigned char *)(fwd_ck + CL.mild);
        const size_t smem = sizeof(BwdSmem);
        auto kern = per_token_w ? k_chunk_bwd<true> : k_chunk_bwd<false>;
        auto kern_steep = per_token_w ? k_chunk_bwd_steep<true> : k_chunk_bwd_steep<false>;
        static unsigned char attr_done[2][2][64];
        const int pt = per_token_w ? 1 : 0;
        if (!set_max_smem_once(kern, (int)smem, attr_done[0][pt]) ||
            !set_max_smem_once(kern_steep, (int)smem, attr_done[1][pt]))
            return WKV_ERR_LAUNCH;
        // every chunk the forward kernel found mild (all of them, on ordinary data) ...
        if (launch_chained(kern, dim3(BH * n), dim3(256), smem, stream, mr, mk, mv, mw, mgy, ms, md, mgr, mgk, mgv,
                           mgw, p) != WKV_OK)
            return WKV_ERR_LAUNCH;
        // ... and the ones it flagged as steep
        const int steep_grid = BH * n < device_sm_count() ? BH * n : device_sm_count();
        if (launch_chained(kern_steep, dim3(steep_grid), dim3(256), smem, stream, mr, mk, mv, mw, mgy, ms, md, mgr,
                           mgk, mgv, mgw, p, BH * n) != WKV_OK)
            return WKV_ERR_LAUNCH;
    }
    // 4. fold the per-chunk partial sums
    {
        const int total = BH * 64;
        if (launch_chained(k_reduce_partials, dim3((total + 255) / 256), dim3(256), 0, stream, (const float *)gu_part,
                           (float *)a->gu, n, total) != WKV_OK)
            return WKV_ERR_LAUNCH;
        if (!per_token_w && launch_chained(k_reduce_partials, dim3((total + 255) / 256), dim3(256), 0, stream,
                                           (const float *)gw_part, (float *)a->gw, n, total) != WKV_OK)
            return WKV_ERR_LAUNCH;
    }
    return WKV_OK;
}

}  // namespace wkv
