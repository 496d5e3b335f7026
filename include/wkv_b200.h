/*
 * wkv_b200 -- C ABI of the B200 (sm_100a) implementation of the RWKV WKV
 * time-mix recurrence: forward and backward, recurrent state and its gradient
 * carried across BPTT segments, for the v4, v5 and v6 variants.
 *
 * Every entry point takes raw device pointers and sizes, launches on the
 * stream it is given (a cudaStream_t passed as void*), allocates nothing and
 * never synchronises.  The caller makes the device that owns the pointers
 * current before the call.  State kept between calls: per-device facts looked
 * up once (SM count, kernel attributes already set), a per-thread cache of the
 * last TMA descriptors built, and -- wkv4_backward_static only -- the device
 * address and contents of its built-in scratch array (see there).  Return value: WKV_OK or
 * one of the WKV_ERR_* codes (wkv_error_string() gives the text); on error
 * nothing was launched.  Nothing ever aborts the process or traps the device.
 *
 * file:line citations name the interface of RWKV-infctx-trainer that each
 * entry point replaces (paths inside that project).
 */
#ifndef WKV_B200_H
#define WKV_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Element type of the activation tensors (r,k,v,u,y,gy,gr,gk,gv,gw). */
enum { WKV_F32 = 0, WKV_BF16 = 1, WKV_F16 = 2 };

enum {
    WKV_OK = 0,
    WKV_ERR_NULL = 1,       /* a required pointer is NULL */
    WKV_ERR_SHAPE = 2,      /* negative size, head size other than 64, C != H*N ... */
    WKV_ERR_DTYPE = 3,      /* unknown element type / decay encoding / state layout */
    WKV_ERR_ALIGN = 4,      /* a pointer is not 16-byte aligned */
    WKV_ERR_WORKSPACE = 5,  /* workspace missing or smaller than *_workspace() says */
    WKV_ERR_LAUNCH = 6,     /* the CUDA runtime refused the launch (cudaGetLastError) */
    WKV_ERR_UNSUPPORTED = 7, /* combination not built (e.g. fast path asked for fp32) */
    WKV_ERR_TOO_LARGE = 8    /* needs more scratch than the built-in array holds */
};

/* How the decay tensor `w` is encoded. */
enum {
    WKV_W_RAW = 0, /* the module parameter/activation x; decay = exp(-exp(x)).
                      v6: [B,T,C] in the activation dtype.  v5: [H,N] fp32. */
    WKV_W_NEGEXP = 1 /* ew = -exp(x), fp32 (what the project's Python wrappers
                        precompute: RWKV-v6/src/module/TimeMix.py:49-51,
                        RWKV-v5/src/module/TimeMix.py:57-60).  Same shapes. */
};

/* Memory layout of the v5/v6 per-head N x N state. */
enum {
    WKV_STATE_KV = 0, /* [B,H,key,value]: rwkv_inner's kv_state
                         (RWKV-v6/src/module/rwkv_inner.py:22) */
    WKV_STATE_VK = 1  /* [B,H,value,key]: the project's CUDA kernels
                         (RWKV-v5/src/module/cuda/wkv5_cuda.cu:142-149) */
};

/* Which implementation runs a v5/v6 call. */
enum {
    WKV_PATH_AUTO = 0,   /* tensor-core chunked kernels when dtype is bf16, else scalar */
    WKV_PATH_SCALAR = 1, /* token-serial fp32 CUDA-core kernels (any dtype, any T) */
    WKV_PATH_CHUNKED = 2 /* tcgen05 chunked kernels (bf16 only) */
};
/* The two paths differ in one documented way.  The chunked kernels floor every per-token
 * decay at 0.005 and pass no gradient to a floored element -- what the project's working
 * path does (w.clamp(0.005), RWKV-v6/src/module/rwkv_inner.py:40-45) and what keeps every
 * operand of the tensor-core products inside the bf16 exponent range.  The token-serial
 * kernels do not floor, like the project's CUDA kernels (wkv6state_cuda_v1.cu, wkv5_cuda.cu).
 * So a bf16 call under WKV_PATH_AUTO follows rwkv_inner on decays below 0.005 (they need
 * x > 1.667), and WKV_PATH_SCALAR follows the CUDA kernels; above the floor they agree.
 * The v6 chunked kernels read the decay activation x in bf16: given WKV_W_NEGEXP they first
 * rebuild x = log(-ew) in bf16 (exact when ew came from a bf16 x, as in TimeMix.py:49-51). */

const char *wkv_error_string(int code);

/* ------------------------------------------------------------------ v4 --
 * Replaces cuda_forward / cuda_backward of RWKV-v4neo/cuda/wkv_cuda_bf16.cu:160-172
 * (called from WKVFunction, RWKV-v4neo/cuda/wkv_op_bf16.cpp:53-56, 76-83).
 *   w          fp32 [C]      = -exp(time_decay)                (wkv_op_bf16.cpp:34)
 *   u,k,v,y    dtype [C] / [B,T,C]   (the project supports bf16 only; fp32 and
 *                                     fp16 are additions)
 *   state_*    fp32 [B,C,3] = (p,q,o); NULL state_in means (0,0,-1e38)
 *   gw,gu      fp32 [B,C] per-batch partials (the caller sums over B as
 *              wkv_op_bf16.cpp:85 does); gw is d/d(time_decay), i.e. already
 *              multiplied by w (wkv_cuda_bf16.cu:156)
 *   gstate_*   fp32 [B,C,3] = (gp,gq,go) in the exponent-scaled convention of
 *              wkv_cuda_bf16.cu:116-152; gstate_out may be NULL (= none)
 * No compile-time limit on T (the project needs T <= Tmax).  Segments of 128 tokens or
 * more are cut into 64-token pieces that run in parallel (piece summaries are folded per
 * channel); that needs the scratch memory wkv4_*_workspace() sizes.
 */
size_t wkv4_forward_workspace(int B, int T, int C);

int wkv4_forward(int B, int T, int C, int dtype, const float *w, const void *u,
                 const void *k, const void *v, const float *state_in, void *y,
                 float *state_out, void *workspace, size_t workspace_bytes, void *stream);

size_t wkv4_backward_workspace(int B, int T, int C);

int wkv4_backward(int B, int T, int C, int dtype, const float *w, const void *u,
                  const void *k, const void *v, const float *state_in,
                  const void *gy, const float *gstate_out, float *gw, float *gu,
                  void *gk, void *gv, float *gstate_in, void *workspace,
                  size_t workspace_bytes, void *stream);

/* Optional hand-over from forward to backward of the same segment (no counterpart in the project,
 * whose backward recomputes everything): wkv4_state_ckpt_bytes() bytes (2.5 per token-channel) that
 * receive, for every 8th token, the state and its derivative w.r.t. the decay.  Backward given the
 * buffer skips rebuilding the states and the forward sweeps of its two passes (three passes over k
 * and v less).  0 bytes / NULL for segments under 128 tokens; NULL is always allowed and
 * makes the _ckpt entry points identical to the plain ones. */
size_t wkv4_state_ckpt_bytes(int B, int T, int C);
int wkv4_forward_ckpt(int B, int T, int C, int dtype, const float *w, const void *u, const void *k,
                      const void *v, const float *state_in, void *y, float *state_out, void *workspace,
                      size_t workspace_bytes, void *state_ckpt, size_t state_ckpt_bytes, void *stream);
int wkv4_backward_ckpt(int B, int T, int C, int dtype, const float *w, const void *u, const void *k,
                       const void *v, const float *state_in, const void *gy, const float *gstate_out,
                       float *gw, float *gu, void *gk, void *gv, float *gstate_in, void *workspace,
                       size_t workspace_bytes, const void *state_ckpt, size_t state_ckpt_bytes,
                       void *stream);

/* wkv4_backward for callers that cannot supply a workspace.  (No counterpart in
 * RWKV-infctx-trainer: its kernels keep their scratch in per-thread arrays.)
 *
 * Who needs it: a host that binds only this C ABI and was handed its tensors
 * by someone else, so it has no device allocator to ask; or a training loop
 * whose device memory is laid out in advance and which may not call cudaMalloc
 * (which also synchronises the device) between steps.
 *
 * Same arguments and results as wkv4_backward minus workspace/workspace_bytes.
 * The tile-start states go to a 32 MiB array that is part of the library image
 * (wkv4_backward_static_limit() returns its size); every GPU that loads the
 * library carries those 32 MiB until the process ends.  The call allocates and
 * frees nothing.  If wkv4_backward_workspace(B,T,C) exceeds the limit it
 * returns WKV_ERR_TOO_LARGE and launches nothing -- split T into shorter
 * segments (the state chains) or use wkv4_backward.
 *
 * The first call on each device looks up the array's device address (one
 * cudaGetSymbolAddress with that device current); make that first call outside
 * any stream capture.  All calls on a device share the one array, which keeps
 * whatever the previous call left there: the kernel needs none of it zeroed,
 * but two calls whose kernels may run at the same time on one GPU (different
 * streams, or different host threads) overwrite each other's states and give
 * wrong gradients.  Issue them on one stream, or order them with events. */
size_t wkv4_backward_static_limit(void);
int wkv4_backward_static(int B, int T, int C, int dtype, const float *w, const void *u,
                         const void *k, const void *v, const float *state_in,
                         const void *gy, const float *gstate_out, float *gw, float *gu,
                         void *gk, void *gv, float *gstate_in, void *stream);

/* -------------------------------------------------------------- v5 / v6 --
 * One argument block serves forward and backward of both variants.
 * C = H*N, N must be 64 (RWKV-v6/src/model.py:313 fixes the head size).
 */
typedef struct wkv_args {
    int B, T, H, N;
    int dtype;        /* WKV_F32 / WKV_BF16 / WKV_F16 */
    int w_kind;       /* WKV_W_RAW / WKV_W_NEGEXP */
    int state_layout; /* WKV_STATE_KV / WKV_STATE_VK (applies to state_* and gstate_*) */
    int path;         /* WKV_PATH_* */
    /* forward inputs */
    const void *r, *k, *v; /* [B,T,C] dtype */
    const void *w;         /* see w_kind */
    const void *u;         /* [H,N] dtype */
    const float *state_in; /* [B,H,N,N] fp32, NULL = zeros */
    /* forward outputs */
    void *y;          /* [B,T,C] dtype */
    float *state_out; /* [B,H,N,N] fp32; may be NULL; may alias state_in */
    /* backward inputs */
    const void *gy;          /* [B,T,C] dtype */
    const float *gstate_out; /* [B,H,N,N] fp32, NULL = zeros */
    /* backward outputs */
    void *gr, *gk, *gv; /* [B,T,C] dtype */
    void *gw;           /* v6: [B,T,C] dtype, gradient w.r.t. x (both w_kinds:
                           the project's kernels multiply by ew too,
                           wkv6state_cuda_v1.cu:290).  v5: [B,C] fp32 per-batch
                           partials of the gradient w.r.t. time_decay */
    float *gu;          /* [B,C] fp32 per-batch partials */
    float *gstate_in;   /* [B,H,N,N] fp32; may be NULL */
    /* scratch */
    void *workspace;
    size_t workspace_bytes;
    /* optional hand-over from forward to backward (chunked path only), wkv56_state_ckpt_bytes()
     * bytes: the state at the start of every 64-token chunk (bf16), r scaled by the decay
     * accumulated since the chunk start (bf16 [B,T,C]) and the decay of every whole chunk.
     * Forward fills it when non-NULL; backward given the same buffer skips recomputing it.
     * The trainer's activation checkpointing re-runs the op's forward anyway
     * (RWKV-v6/src/model.py:660-662); this is the op-level equivalent. */
    void *state_ckpt;
    size_t state_ckpt_bytes;
    /* Chunked path only.  The chunks of a segment form a serial chain per (batch, head); when
     * there are too few chains to fill the GPU (few heads per GPU, batch 1) the chain is cut
     * into this many groups of consecutive chunks that run in parallel (a summary pass per
     * group, a scan over the groups, then the full pass per group).  0 = the library decides
     * from B*H, T and the SM count; 1 = never split; n > 1 = n groups (at most one per chunk).
     * The *_workspace() sizes depend on it: fill it in before asking for them. */
    int time_groups;
    /* Chunked path, forward only: fp32 states for a later re-run of the same forward call (what
     * activation checkpointing does, RWKV-v6/src/model.py:657-665).  wkv56_group_states_bytes()
     * bytes.  WKV_GROUP_STATES_SAVE: the call also stores the state at the start of every 8th
     * chunk (512 tokens) there.  WKV_GROUP_STATES_USE: the call starts every 8-chunk group from the
     * stored state instead of scanning: the groups run in parallel, no serial pass over T, and
     * y, state_out and the hand-over are bit-identical to those of the call that saved them
     * (same inputs). */
    void *group_states;
    size_t group_states_bytes;
    int group_states_mode;
} wkv_args_t;

enum { WKV_GROUP_STATES_NONE = 0, WKV_GROUP_STATES_SAVE = 1, WKV_GROUP_STATES_USE = 2 };
size_t wkv56_group_states_bytes(const wkv_args_t *a);

/* Bytes of wkv_args_t.state_ckpt for these arguments (0 when the call would not run on
 * the chunked kernels). */
size_t wkv56_state_ckpt_bytes(const wkv_args_t *a, int per_token_w);

/* v5: replaces cuda_forward_{bf16,fp16,fp32} / cuda_backward_* of
 * RWKV-v5/src/module/cuda/wkv5_cuda.cu:348-383 (bound in wkv5_op.cpp:88-116),
 * with per-batch state, a state output and the state gradient those lack. */
size_t wkv5_forward_workspace(const wkv_args_t *a);
size_t wkv5_backward_workspace(const wkv_args_t *a);
int wkv5_forward(const wkv_args_t *a, void *stream);
int wkv5_backward(const wkv_args_t *a, void *stream);

/* v6: replaces cuda_forward / cuda_backward of
 * RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu:295-308 (bound in
 * wkv6state_op.cpp:8-22) and of the stateless wkv6_cuda.cu:229-242, with fp32
 * per-batch state, a state output, and the full state gradient. */
size_t wkv6_forward_workspace(const wkv_args_t *a);
size_t wkv6_backward_workspace(const wkv_args_t *a);
int wkv6_forward(const wkv_args_t *a, void *stream);
int wkv6_backward(const wkv_args_t *a, void *stream);

/* 1 if a v5 (per_token_w = 0) / v6 (per_token_w = 1) call with these arguments runs on the
 * chunked tensor-core kernels, 0 if on the token-serial ones.  When it does, the first 4
 * bytes of the workspace hold a status word after the call has completed on the stream:
 * 0 = ok, non-zero = a bounded device-side wait ran out and the results are invalid. */
int wkv56_uses_chunked(const wkv_args_t *a, int per_token_w);

/* ------------------------------------------- neighbours of the op in TimeMix --
 * The elementwise stages on either side of the WKV op, each fused into one pass over its
 * [B,T,C] tensors (bf16 tensors, fp32 parameters and parameter gradients, fp32 arithmetic).
 *
 * wkv_lnx_gate_*: out = ln_x(y) * g of RWKV-v6/src/module/TimeMix.py:296-298 (v5:
 *   RWKV-v5/src/module/TimeMix.py:318-320), ln_x = GroupNorm(H groups of 64 channels, eps),
 *   gamma/beta its weight and bias [C], tokens = B*T.  Backward returns gy, gg and the
 *   parameter gradients ggamma, gbeta [C] (summed over all tokens in a fixed order).
 *
 * wkv_ddlerp_*: the token-shift mixes of RWKV-v6/src/module/TimeMix.py:262-273,
 *   out_i = x + (x_prev - x) * (maa_i + m_i),  i < nmix,  nmix = 1 (the first mix, m = NULL),
 *   5 (xw,xk,xv,xr,xg in the order of m), 4 (the static mixes of the v5 block,
 *   RWKV-v5/src/module/TimeMix.py:293-300, with maa = 1 - time_mix and m = NULL) or 3 (those
 *   of the v4 block, RWKV-v4neo/src/model.py:240-244).
 *   x [B,T,C]; x_prev of a row's first token is
 *   shift [B,C] (last token of the previous segment); maa fp32 [nmix,C]; m, out [nmix,B,T,C].
 *   Backward: gx [B,T,C], gm [nmix,B,T,C] (when m is given), gmaa fp32 [nmix,C], and
 *   gshift_out [B,C] = gradient w.r.t. shift; gshift_in [B,C] (or NULL) = what the next
 *   segment's gshift_out sends back to this segment's last token. */
int wkv_lnx_gate_forward(int tokens, int H, const void *y, const void *g, const float *gamma,
                         const float *beta, float eps, void *out, void *stream);
size_t wkv_lnx_gate_backward_workspace(int tokens, int H);
int wkv_lnx_gate_backward(int tokens, int H, const void *y, const void *g, const float *gamma,
                          const float *beta, float eps, const void *gout, void *gy, void *gg,
                          float *ggamma, float *gbeta, void *workspace, size_t workspace_bytes,
                          void *stream);
int wkv_ddlerp_forward(int B, int T, int C, int nmix, const void *x, const void *shift,
                       const float *maa, const void *m, void *out, void *stream);
size_t wkv_ddlerp_backward_workspace(int B, int T, int C, int nmix);
int wkv_ddlerp_backward(int B, int T, int C, int nmix, const void *x, const void *shift,
                        const float *maa, const void *m, const void *gout, const void *gshift_in,
                        void *gx, void *gm, void *gshift_out, float *gmaa, void *workspace,
                        size_t workspace_bytes, void *stream);

/* Library build identification: "wkv_b200 <n> sm_100a". */
const char *wkv_version(void);

/* ------------------------------------------------------------ self-tests --
 * (No counterpart in RWKV-infctx-trainer: its kernels have no device-side waits.)
 * Every device-side wait of the chunked kernels is bounded: after a number of polls it
 * gives up, the kernel sets its bit in the status word, lets copies and products in
 * flight finish, frees its tensor memory and returns.  These two entry points make that
 * happen on purpose, safely: nothing spins without a bound and nothing traps.
 *
 * wkv_selftest_wait_timeout: one CTA waits on a barrier nobody arrives on, `limit`
 * polls (1..100000); afterwards *status_word (device memory, zeroed by the caller) holds
 * 16 | 32: the plain wait gave up, and the abort flag it raised ended the CTA's other wait.
 *
 * wkv56_selftest_abort: a normal v5/v6 forward (backward_call = 0) or backward call on
 * the chunked kernels in which one kernel (0 forward, 1 dS scan, 2 per-chunk backward)
 * never issues the loads of chunk `skip_chunk`, with every wait cut to `limit` polls.
 * The call returns WKV_OK (the launch succeeded); the status word at the start of the
 * workspace then has bit 1 (forward), 2 (dS scan) or 4 (per-chunk backward) set and the
 * outputs are invalid. */
int wkv_selftest_wait_timeout(int *status_word, unsigned limit, void *stream);
int wkv56_selftest_abort(const wkv_args_t *a, int per_token_w, int backward_call, int kernel,
                         int skip_chunk, unsigned limit, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* WKV_B200_H */
