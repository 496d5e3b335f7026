// C-ABI entry points for v5/v6: argument validation and dispatch between the
// token-serial kernels and the chunked tensor-core kernels.
#include "wkv56_chunked.cuh"
#include "wkv_common.cuh"

using namespace wkv;

namespace {

int check_common(const wkv_args_t *a, bool backward, bool per_token_w) {
    if (!a) return WKV_ERR_NULL;
    if (a->B < 0 || a->T < 0 || a->H < 0) return WKV_ERR_SHAPE;
    if (a->N != HEAD) return WKV_ERR_SHAPE;
    if (a->dtype != WKV_F32 && a->dtype != WKV_BF16 && a->dtype != WKV_F16) return WKV_ERR_DTYPE;
    if (a->w_kind != WKV_W_RAW && a->w_kind != WKV_W_NEGEXP) return WKV_ERR_DTYPE;
    if (a->state_layout != WKV_STATE_KV && a->state_layout != WKV_STATE_VK) return WKV_ERR_DTYPE;
    if (a->path != WKV_PATH_AUTO && a->path != WKV_PATH_SCALAR && a->path != WKV_PATH_CHUNKED)
        return WKV_ERR_DTYPE;
    if (a->time_groups < 0) return WKV_ERR_SHAPE;
    if (a->group_states_mode < WKV_GROUP_STATES_NONE || a->group_states_mode > WKV_GROUP_STATES_USE) return WKV_ERR_DTYPE;
    if (a->group_states && !aligned16(a->group_states)) return WKV_ERR_ALIGN;
    if (a->B == 0 || a->H == 0) return WKV_OK;
    if (!a->u) return WKV_ERR_NULL;
    if (!per_token_w && !a->w) return WKV_ERR_NULL;
    if (a->T > 0) {
        if (!a->r || !a->k || !a->v) return WKV_ERR_NULL;
        if (per_token_w && !a->w) return WKV_ERR_NULL;
        if (!backward && !a->y) return WKV_ERR_NULL;
        if (backward && (!a->gy || !a->gr || !a->gk || !a->gv)) return WKV_ERR_NULL;
        if (backward && per_token_w && !a->gw) return WKV_ERR_NULL;
    }
    if (backward && (!a->gu || (!per_token_w && !a->gw))) return WKV_ERR_NULL;
    const void *ptrs[] = {a->r, a->k, a->v, a->y, a->gy, a->gr, a->gk, a->gv, a->state_in,
                          a->state_out, a->gstate_out, a->gstate_in, a->workspace, a->state_ckpt};
    for (const void *p : ptrs)
        if (p && !aligned16(p)) return WKV_ERR_ALIGN;
    if (per_token_w && a->w && !aligned16(a->w)) return WKV_ERR_ALIGN;
    if (per_token_w && a->gw && !aligned16(a->gw)) return WKV_ERR_ALIGN;
    return WKV_OK;
}

bool use_chunked(const wkv_args_t *a, bool per_token_w, int *err) {
    *err = WKV_OK;
    if (a->path == WKV_PATH_SCALAR) return false;
    const bool ok = chunked_supported(a, per_token_w);
    if (a->path == WKV_PATH_CHUNKED && !ok) *err = WKV_ERR_UNSUPPORTED;
    return ok;
}

size_t fwd_ws(const wkv_args_t *a, bool pt) {
    if (!a || a->B <= 0 || a->H <= 0 || a->T <= 0 || a->N != HEAD) return 0;
    int err;
    return use_chunked(a, pt, &err) ? chunked_forward_workspace(a, pt) : 0;
}

size_t bwd_ws(const wkv_args_t *a, bool pt) {
    if (!a || a->B <= 0 || a->H <= 0 || a->T <= 0 || a->N != HEAD) return 0;
    int err;
    return use_chunked(a, pt, &err) ? chunked_backward_workspace(a, pt) : scalar_backward_workspace(a);
}

int forward(const wkv_args_t *a, bool pt, void *stream, const ChunkedTest &tst = ChunkedTest()) {
    int err = check_common(a, false, pt);
    if (err != WKV_OK) return err;
    if (a->B == 0 || a->H == 0) return WKV_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool ch = use_chunked(a, pt, &err);
    if (err != WKV_OK) return err;
    const size_t need = fwd_ws(a, pt);
    if (need && (!a->workspace || a->workspace_bytes < need)) return WKV_ERR_WORKSPACE;
    if (ch && a->state_ckpt && a->state_ckpt_bytes < wkv56_state_ckpt_bytes(a, pt)) return WKV_ERR_WORKSPACE;
    if (a->group_states && a->group_states_mode != WKV_GROUP_STATES_NONE) {
        if (!ch) return WKV_ERR_UNSUPPORTED;
        if (a->group_states_bytes < wkv56_group_states_bytes(a)) return WKV_ERR_WORKSPACE;
    }
    return ch ? chunked_forward(a, pt, tst, s) : scalar_forward(a, pt, s);
}

int backward(const wkv_args_t *a, bool pt, void *stream, const ChunkedTest &tst = ChunkedTest()) {
    int err = check_common(a, true, pt);
    if (err != WKV_OK) return err;
    if (a->B == 0 || a->H == 0) return WKV_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool ch = use_chunked(a, pt, &err);
    if (err != WKV_OK) return err;
    const size_t need = bwd_ws(a, pt);
    if (need && (!a->workspace || a->workspace_bytes < need)) return WKV_ERR_WORKSPACE;
    if (ch && a->state_ckpt && a->state_ckpt_bytes < wkv56_state_ckpt_bytes(a, pt)) return WKV_ERR_WORKSPACE;
    return ch ? chunked_backward(a, pt, tst, s) : scalar_backward(a, pt, s);
}

}  // namespace

extern "C" {

const char *wkv_error_string(int code) {
    switch (code) {
        case WKV_OK: return "ok";
        case WKV_ERR_NULL: return "a required pointer is NULL";
        case WKV_ERR_SHAPE: return "bad shape (negative size or head size other than 64)";
        case WKV_ERR_DTYPE: return "unknown element type, decay encoding, state layout or path";
        case WKV_ERR_ALIGN: return "a tensor pointer is not 16-byte aligned";
        case WKV_ERR_WORKSPACE: return "workspace missing or too small";
        case WKV_ERR_LAUNCH: return "CUDA launch failed";
        case WKV_ERR_UNSUPPORTED: return "the chunked tensor-core path does not take these arguments";
        case WKV_ERR_TOO_LARGE: return "needs more scratch than the library's built-in array holds";
    }
    return "unknown error code";
}

int wkv56_uses_chunked(const wkv_args_t *a, int per_token_w);

const char *wkv_version(void) { return "wkv_b200 2 sm_100a"; }

size_t wkv56_group_states_bytes(const wkv_args_t *a) {
    if (!a || a->B <= 0 || a->H <= 0 || a->T <= 0 || a->N != HEAD || a->dtype != WKV_BF16) return 0;
    return chunked_group_states_bytes(a);
}

size_t wkv56_state_ckpt_bytes(const wkv_args_t *a, int per_token_w) {
    if (!wkv56_uses_chunked(a, per_token_w)) return 0;
    return chunked::ckpt_layout(a->B, a->T, a->H).total;
}

int wkv56_uses_chunked(const wkv_args_t *a, int per_token_w) {
    if (!a || a->B <= 0 || a->H <= 0 || a->T <= 0 || a->N != HEAD) return 0;
    int err;
    return use_chunked(a, per_token_w != 0, &err) ? 1 : 0;
}

int wkv_selftest_wait_timeout(int *status_word, unsigned limit, void *stream) {
    if (!status_word) return WKV_ERR_NULL;
    return selftest_wait(status_word, limit, (cudaStream_t)stream);
}

int wkv56_selftest_abort(const wkv_args_t *a, int per_token_w, int backward_call, int kernel, int skip_chunk,
                         unsigned limit, void *stream) {
    if (limit == 0 || limit > 100000u || kernel < 0 || kernel > 2 || skip_chunk < 0) return WKV_ERR_SHAPE;
    if (!wkv56_uses_chunked(a, per_token_w)) return WKV_ERR_UNSUPPORTED;
    ChunkedTest tst;
    tst.wait_limit = limit;
    tst.kernel = kernel;
    tst.skip_load = skip_chunk;
    return backward_call ? backward(a, per_token_w != 0, stream, tst) : forward(a, per_token_w != 0, stream, tst);
}

size_t wkv5_forward_workspace(const wkv_args_t *a) { return fwd_ws(a, false); }
size_t wkv5_backward_workspace(const wkv_args_t *a) { return bwd_ws(a, false); }
int wkv5_forward(const wkv_args_t *a, void *stream) { return forward(a, false, stream); }
int wkv5_backward(const wkv_args_t *a, void *stream) { return backward(a, false, stream); }

size_t wkv6_forward_workspace(const wkv_args_t *a) { return fwd_ws(a, true); }
size_t wkv6_backward_workspace(const wkv_args_t *a) { return bwd_ws(a, true); }
int wkv6_forward(const wkv_args_t *a, void *stream) { return forward(a, true, stream); }
int wkv6_backward(const wkv_args_t *a, void *stream) { return backward(a, true, stream); }

}  // extern "C"
