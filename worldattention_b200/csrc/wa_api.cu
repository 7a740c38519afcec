// C-ABI glue: error buffer, version, and the whole-forward entry point wa_hsa_forward, which
// sequences routing -> sparse branch -> compressed branch -> gate/combine on one stream.
// Mirrors hsa_attention, wan/modules/hsa/attention.py:153-259.
#include "wa_common.cuh"
#include "wa_internal.cuh"

namespace wa {
char *last_error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}
unsigned long long &launch_counter() {
    static unsigned long long n = 0;
    return n;
}

// Optional timing of the attention kernel inside wa_hsa_forward (for roofline measurement).
static bool g_profile = false;
static cudaEvent_t g_ev0 = nullptr, g_ev1 = nullptr;
static bool g_ev_valid = false;
static int g_profile_pause = 0;

void profile_pause(bool on) { g_profile_pause += on ? 1 : -1; }

void profile_mark(bool begin, cudaStream_t stream) {
    if (!g_profile || g_profile_pause > 0) return;
    if (!g_ev0) {
        if (cudaEventCreate(&g_ev0) != cudaSuccess || cudaEventCreate(&g_ev1) != cudaSuccess) {
            g_ev0 = g_ev1 = nullptr;
            return;
        }
    }
    cudaEventRecord(begin ? g_ev0 : g_ev1, stream);
    if (!begin) g_ev_valid = true;
}
}  // namespace wa

using namespace wa;

extern "C" int wa_abi_version(void) { return WA_ABI_VERSION; }
extern "C" size_t wa_hsa_params_size(void) { return sizeof(wa_hsa_params); }
extern "C" unsigned long long wa_launch_count(void) { return launch_counter(); }
extern "C" int wa_profile_enable(int on) {
    g_profile = on != 0;
    g_ev_valid = false;
    return 0;
}
extern "C" int wa_profile_attention_ms(float *ms) {
    WA_REQUIRE(ms, WA_ERR_ARG, "wa_profile_attention_ms: null pointer");
    WA_REQUIRE(g_ev_valid, WA_ERR_ARG, "wa_profile_attention_ms: no profiled launch recorded");
    cudaError_t e = cudaEventSynchronize(g_ev1);
    if (e == cudaSuccess) e = cudaEventElapsedTime(ms, g_ev0, g_ev1);
    if (e != cudaSuccess) return fail((int)e, "wa_profile_attention_ms: %s", cudaGetErrorString(e));
    return 0;
}
extern "C" const char *wa_last_error(void) { return last_error_buffer(); }

namespace {

struct Workspace {
    size_t q_pooled, k_pooled, block_attn, index, num, gini, thresholds, counters, kc, vc, sparse, linear, tuned, total;
    int Nq, Nkv, Lc_inline;
};

size_t take(size_t &cursor, size_t bytes) {
    const size_t at = cursor;
    cursor = align_up(cursor + bytes, 256);
    return at;
}

int inline_coarse_len(const wa_hsa_params *p) {
    const int seg = p->proj_segment_len > 0 ? p->proj_segment_len : p->Lkv;
    int total = 0;
    for (int start = 0; start < p->Lkv; start += seg) {
        const int n = p->Lkv - start < seg ? p->Lkv - start : seg;
        const int r = ceil_div(n, p->block_size);
        total += r < p->proj_rank ? r : p->proj_rank;
    }
    return total;
}

Workspace plan(const wa_hsa_params *p) {
    Workspace w{};
    w.Nq = ceil_div(p->Lq, p->block_size);
    w.Nkv = ceil_div(p->Lkv, p->block_size);
    w.Lc_inline = p->Lc > 0 ? 0 : inline_coarse_len(p);
    const size_t bh = (size_t)p->B * p->H;
    size_t c = 0;
    w.q_pooled = take(c, bh * w.Nq * p->D * sizeof(float));
    w.k_pooled = take(c, bh * w.Nkv * p->D * sizeof(float));
    w.block_attn = take(c, bh * w.Nq * w.Nkv * sizeof(float));
    w.index = take(c, bh * w.Nq * w.Nkv * sizeof(int32_t));
    w.num = take(c, bh * w.Nq * sizeof(int32_t));
    w.gini = take(c, bh * w.Nq * sizeof(float));
    w.thresholds = take(c, (size_t)p->H * sizeof(float));
    w.counters = take(c, ((size_t)p->H + 1) * sizeof(int));
    const size_t kvsz = dtype_size(p->k.dtype);
    w.kc = take(c, (size_t)p->B * w.Lc_inline * p->H * p->D * kvsz);
    w.vc = take(c, (size_t)p->B * w.Lc_inline * p->H * p->D * kvsz);
    const size_t tokens = (size_t)p->B * p->Lq * p->H * p->D;
    w.sparse = take(c, tokens * sizeof(__nv_bfloat16));
    w.linear = take(c, tokens * sizeof(float));
    w.tuned = take(c, hsa_sm100_workspace_bytes(p));
    w.total = c;
    return w;
}

int validate(const wa_hsa_params *p) {
    const char *what = "wa_hsa_forward";
    WA_REQUIRE(p, WA_ERR_ARG, "%s: null params", what);
    WA_REQUIRE(p->B > 0 && p->H > 0 && p->D > 0, WA_ERR_ARG, "%s: B, H, D must be positive", what);
    WA_REQUIRE(p->Lq > 0 && p->Lkv > 0, WA_ERR_ARG, "%s: q_len and kv_len must be positive", what);
    WA_REQUIRE(p->block_size > 0, WA_ERR_ARG, "%s: block_size must be positive", what);
    WA_REQUIRE(p->Lc >= 0, WA_ERR_ARG, "%s: negative compressed length", what);
    WA_REQUIRE(valid_dtype(p->q.dtype) && valid_dtype(p->k.dtype) && p->k.dtype == p->v.dtype &&
                   (p->part_sparse || valid_dtype(p->out.dtype)),
               WA_ERR_ARG, "%s: bad or mismatched q/k/v/out dtypes", what);
    if (p->Lc > 0) {
        WA_REQUIRE(p->k_coarse.ptr && p->v_coarse.ptr, WA_ERR_ARG, "%s: compressed cache pointers are null", what);
        WA_REQUIRE(valid_dtype(p->k_coarse.dtype) && p->k_coarse.dtype == p->v_coarse.dtype, WA_ERR_ARG,
                   "%s: bad compressed cache dtype", what);
    } else {
        WA_REQUIRE(p->k_proj && p->v_proj && p->proj_rank > 0 && p->proj_cols > 0 && valid_dtype(p->proj_dtype),
                   WA_ERR_ARG, "%s: projection matrices required when no compressed cache is given", what);
    }
    WA_REQUIRE(!p->gate_w || valid_dtype(p->gate_dtype), WA_ERR_ARG, "%s: bad gate dtype", what);
    return 0;
}

}  // namespace

extern "C" size_t wa_hsa_workspace_bytes(const wa_hsa_params *p) {
    if (!p || p->B <= 0 || p->H <= 0 || p->D <= 0 || p->Lq <= 0 || p->Lkv <= 0 || p->block_size <= 0) return 0;
    return plan(p).total;
}

extern "C" int wa_hsa_status(const wa_hsa_params *p, int *status, void *stream_) {
    int rc = validate(p);
    if (rc) return rc;
    WA_REQUIRE(status && p->workspace, WA_ERR_ARG, "wa_hsa_status: null pointer");
    const Workspace w = plan(p);
    WA_REQUIRE(p->workspace_bytes >= w.total, WA_ERR_WORKSPACE, "wa_hsa_status: workspace too small");
    cudaStream_t stream = (cudaStream_t)stream_;
    cudaError_t e = cudaMemcpyAsync(status, (char *)p->workspace + w.tuned + hsa_sm100_status_offset(p), sizeof(int),
                                    cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail((int)e, "wa_hsa_status: %s", cudaGetErrorString(e));
    return 0;
}

extern "C" int wa_hsa_forward(const wa_hsa_params *p, int *used_tuned, void *stream_) {
    const char *what = "wa_hsa_forward";
    int rc = validate(p);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    const Workspace w = plan(p);
    WA_REQUIRE(p->workspace && p->workspace_bytes >= w.total, WA_ERR_WORKSPACE,
               "%s: workspace of %zu bytes required, got %zu", what, w.total, p->workspace_bytes);
    WA_REQUIRE((uintptr_t)p->workspace % 256 == 0, WA_ERR_ALIGN, "%s: workspace must be 256-byte aligned", what);
    char *ws = (char *)p->workspace;
    float *q_pooled = (float *)(ws + w.q_pooled), *k_pooled = p->k_pooled ? p->k_pooled : (float *)(ws + w.k_pooled);
    const int k_first = p->k_pooled ? p->k_pooled_valid : 0;
    WA_REQUIRE(k_first >= 0 && k_first <= w.Nkv, WA_ERR_ARG, "%s: k_pooled_valid must be in [0, %d], got %d", what, w.Nkv, k_first);
    WA_REQUIRE(!p->k_pooled || (uintptr_t)p->k_pooled % 16 == 0, WA_ERR_ALIGN, "%s: k_pooled must be 16-byte aligned", what);
    float *block_attn = (float *)(ws + w.block_attn);
    int32_t *index = p->index_out ? p->index_out : (int32_t *)(ws + w.index);
    int32_t *num = p->num_out ? p->num_out : (int32_t *)(ws + w.num);
    float *thresholds = p->thresholds_out ? p->thresholds_out : (float *)(ws + w.thresholds);
    float *gini = (float *)(ws + w.gini);
    if (used_tuned) *used_tuned = 0;

    // ---- routing (routing.py:45-118) ---------------------------------------------------------
    WA_REQUIRE(p->H <= 65535 && p->B <= 65535, WA_ERR_UNSUPPORTED, "%s: B, H must be <= 65535", what);
    WA_REQUIRE((p->index_in == nullptr) == (p->num_in == nullptr), WA_ERR_ARG, "%s: index_in and num_in go together", what);
    const bool partial = p->part_sparse != nullptr;
    WA_REQUIRE(!partial || (p->part_linear && p->lse_sparse && p->lse_linear), WA_ERR_ARG,
               "%s: partial-output mode needs all four of part_sparse, part_linear, lse_sparse, lse_linear", what);
    // ---- compressed cache views (attention.py:186-200); the kernel runs after routing ----------
    wa_tensor4 kc = p->k_coarse, vc = p->v_coarse;
    int Lc = p->Lc;
    const bool compress_inline = Lc == 0;
    if (compress_inline) {
        Lc = w.Lc_inline;
        kc.ptr = ws + w.kc; vc.ptr = ws + w.vc;
        kc.dtype = vc.dtype = p->k.dtype;
        kc.stride_h = vc.stride_h = p->D;
        kc.stride_l = vc.stride_l = (int64_t)p->H * p->D;
        kc.stride_b = vc.stride_b = (int64_t)Lc * p->H * p->D;
    }
    const int lin_dtype = vc.dtype;
    const bool tuned = !(p->flags & WA_HSA_FORCE_GENERIC) && hsa_sm100_supported(p, Lc, &kc, &vc);
    WA_REQUIRE(tuned || !(p->flags & WA_HSA_REQUIRE_TUNED), WA_ERR_UNSUPPORTED,
               "%s: shape not covered by the tcgen05 kernel (needs bf16, head_dim 128, block 64 or 128)", what);

    WA_REQUIRE(p->peer_rows == 0 || (tuned && partial && p->B == 1 && p->peer_rows > 0 && p->peer_self >= 0 && p->peer_self < 8 &&
                                     (long long)p->peer_rows * 8 >= p->Lq && p->part_stride > 0 && p->lse_stride_token > 0),
               WA_ERR_ARG, "%s: peer stores need the tcgen05 kernel, packed partial records, B = 1 and at most 8 ranks covering Lq", what);
    if (p->peer_rows > 0)
        for (int d = 0; d < 8; ++d)
            WA_REQUIRE(p->peer_delta[d] % 4 == 0, WA_ERR_ALIGN, "%s: peer_delta[%d] must be a multiple of 4 floats (16 bytes)", what, d);
    WA_REQUIRE(tuned || (p->part_stride == 0 && p->lse_stride_token == 0 && p->lse_stride_head == 0), WA_ERR_UNSUPPORTED,
               "%s: a partial-output layout other than the contiguous one needs the tcgen05 kernel", what);

    bool prepared = false;
    if (p->index_in) {
        index = const_cast<int32_t *>(p->index_in);
        num = const_cast<int32_t *>(p->num_in);
    } else {
        // pooling, then scores + sort + thresholds + counts (+ the tcgen05 kernel's work order) in one launch
        int *counters = (int *)(ws + w.counters);
        if ((rc = pool_launch(&p->q, p->Lq, q_pooled, &p->k, p->Lkv, k_pooled, p->B, p->H, p->D, p->block_size, stream,
                              counters, p->H + 1, k_first, p->status_mirror)))
            return rc;
        SchedJob job{};
        if (tuned) job = hsa_sm100_sched_job(p, ws + w.tuned);
        if ((rc = route_fused_launch(q_pooled, k_pooled, p->B, p->H, w.Nq, w.Nkv, p->D, p->tau_min, p->tau_max,
                                     p->topk_per_head, block_attn, index, num, thresholds, gini, counters, job, stream,
                                     /*whole_order=*/p->index_out != nullptr || p->thresholds_out != nullptr)))
            return rc;
        prepared = tuned;
    }

    if (compress_inline) {
        if ((rc = wa_compress_kv(&p->k, &p->v, &kc, &vc, p->B, p->Lkv, p->H, p->D, p->proj_segment_len,
                                 p->block_size, p->k_proj, p->v_proj, p->proj_dtype, p->proj_rank, p->proj_cols,
                                 stream)))
            return rc;
    }

    // ---- tuned tcgen05 path -------------------------------------------------------------------
    if (tuned) {
        rc = hsa_sm100_launch(p, Lc, &kc, &vc, index, num, w.Nq, w.Nkv, ws + w.tuned, prepared, stream);
        if (rc) return rc;
        if (used_tuned) *used_tuned = 1;
        return 0;
    }

    // ---- generic SIMT path --------------------------------------------------------------------
    if (partial) {
        wa_tensor4 ps{}, pl{};
        ps.ptr = p->part_sparse; pl.ptr = p->part_linear;
        ps.dtype = pl.dtype = WA_F32;
        ps.stride_h = pl.stride_h = p->D;
        ps.stride_l = pl.stride_l = (int64_t)p->H * p->D;
        ps.stride_b = pl.stride_b = (int64_t)p->Lq * p->H * p->D;
        if ((rc = wa_block_sparse_forward(&p->q, &p->k, &p->v, &ps, p->B, p->H, p->Lq, p->Lkv, p->D, p->block_size, index,
                                          num, w.Nkv, nullptr, 1, 0, p->lse_sparse, stream)))
            return rc;
        return wa_linear_branch(&p->q, &kc, &vc, &pl, p->B, p->H, p->Lq, Lc, p->D, 0, p->lse_linear, stream);
    }
    wa_tensor4 sparse{}, linear{};
    sparse.ptr = ws + w.sparse; sparse.dtype = WA_BF16;
    linear.ptr = ws + w.linear; linear.dtype = lin_dtype;
    sparse.stride_h = linear.stride_h = p->D;
    sparse.stride_l = linear.stride_l = (int64_t)p->H * p->D;
    sparse.stride_b = linear.stride_b = (int64_t)p->Lq * p->H * p->D;
    profile_mark(true, stream);
    rc = wa_block_sparse_forward(&p->q, &p->k, &p->v, &sparse, p->B, p->H, p->Lq, p->Lkv, p->D, p->block_size, index,
                                 num, w.Nkv, nullptr, /*round_in=*/1, /*round_out=*/1, nullptr, stream);
    profile_mark(false, stream);
    if (rc) return rc;
    if (!(p->flags & WA_HSA_FORCE_GENERIC) && hsa_sm100_linear_supported(p, Lc, &kc, &vc)) {
        // routing block size other than 128: the sparse branch ran on the SIMT kernel above, but the linear branch
        // does not depend on the block size and takes the tcgen05 kernel (float32 result, as in the fused path)
        linear.dtype = WA_F32;
        if ((rc = hsa_sm100_launch_linear(p, Lc, &kc, &vc, (float *)linear.ptr, ws + w.tuned, stream))) return rc;
    } else if ((rc = wa_linear_branch(&p->q, &kc, &vc, &linear, p->B, p->H, p->Lq, Lc, p->D, lin_dtype == WA_BF16, nullptr,
                                      stream))) {
        return rc;
    }
    return wa_gate_combine(&p->q, &sparse, &linear, &p->out, p->B, p->Lq, p->H, p->D, p->gate_w, p->gate_b,
                           p->gate_dtype, lin_dtype == WA_BF16, stream);
}
