/*
 * worldattention_b200 -- C ABI of the sm_100a HSA / HKV kernels.
 *
 * One shared library (libwa_b200.so), plain C linkage, raw device pointers and sizes only.  The
 * caller owns every buffer (inputs, outputs, workspace); the library allocates no device memory.
 * All launches go to the CUDA stream passed as `stream` (a cudaStream_t cast to void*; NULL is
 * the legacy default stream).  No entry point synchronises the host.
 *
 * Return value of every int function: 0 = success, < 0 = rejected argument (WA_ERR_*), > 0 = a
 * cudaError_t raised by a launch.  `wa_last_error()` returns the message of the calling thread's
 * most recent failure.  Nothing here throws, traps or aborts.
 *
 * Each entry point names the reference interface it stands in for; paths are relative to the
 * WorldAttention project (wan/modules/hsa/..., pipeline/hkv/...).
 */
#ifndef WORLDATTENTION_B200_H_
#define WORLDATTENTION_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WA_ABI_VERSION 3

/* element types */
#define WA_F32 0
#define WA_BF16 1

/* argument errors */
#define WA_ERR_ARG (-1)         /* null pointer, non-positive size, bad dtype            */
#define WA_ERR_UNSUPPORTED (-2) /* shape outside what the kernels implement              */
#define WA_ERR_WORKSPACE (-3)   /* workspace missing or too small                        */
#define WA_ERR_ALIGN (-4)       /* pointer / stride alignment the kernel needs is absent */
#define WA_ERR_DEVICE (-5)      /* device is not sm_100 or driver entry point missing    */

/* flags for wa_hsa_forward */
#define WA_HSA_FORCE_GENERIC 1  /* skip the tcgen05 kernel even when the shape qualifies  */
#define WA_HSA_REQUIRE_TUNED 2  /* fail with WA_ERR_UNSUPPORTED instead of using the generic kernels */

/* A strided view of a `[B, L, H, D]` tensor whose last axis is contiguous.  Strides count
 * elements.  `[B, H, N, D]` tensors are described by swapping stride_l / stride_h. */
typedef struct wa_tensor4 {
    void *ptr;
    int32_t dtype; /* WA_F32 | WA_BF16 */
    int32_t reserved;
    int64_t stride_b, stride_l, stride_h;
} wa_tensor4;

int wa_abi_version(void);
const char *wa_last_error(void);
/* sizeof(wa_hsa_params) as the library was compiled: a binding checks its own mirror of the struct against it. */
size_t wa_hsa_params_size(void);

/* Measurement aids (no reference counterpart).  wa_launch_count: kernels this library has
 * launched in this process.  wa_profile_enable(1) makes wa_hsa_forward bracket its attention
 * kernel (the tcgen05 kernel, or the SIMT sparse kernel on the generic path) with CUDA events on
 * the launch stream; wa_profile_attention_ms waits for the last bracketed launch and returns its
 * duration.  Profiling is off by default and is the only place the library synchronises. */
unsigned long long wa_launch_count(void);
int wa_profile_enable(int on);
int wa_profile_attention_ms(float *ms);

/* ---------------------------------------------------------------------------------------------
 * Routing -- wan/modules/hsa/routing.py
 * ------------------------------------------------------------------------------------------- */

/* block_mean_pool (routing.py:45-61).  Reads the unpadded `[B, L, H, D]` view once and writes
 * float32 `[B, H, ceil(L/block_size), D]`.  Aligned L: mean rounded to the input dtype; ragged L:
 * sum rounded to the input dtype, divided by the real block size in float32. */
int wa_pool_blocks(const wa_tensor4 *x, int B, int L, int H, int D, int block_size, float *pooled,
                   void *stream);

/* block_attention_map (routing.py:64-68).  float32 `[B,H,Nq,D]` x `[B,H,Nkv,D]` ->
 * softmax over Nkv, float32 `[B,H,Nq,Nkv]`; float64 accumulation, one rounding per value. */
int wa_route_scores(const float *q_pooled, const float *k_pooled, int B, int H, int Nq, int Nkv,
                    int D, float *block_attn, void *stream);

/* build_block_routing (routing.py:71-118).  Descending order with equal values by ascending id,
 * Gini -> per-head threshold -> cumulative-mass count.  `fixed_num_per_head` (device `[H]`, may
 * be NULL) replaces the count by min(k_h, Nkv).  `mask` (bytes `[B,H,Nq,Nkv]`) may be NULL.
 * `gini_scratch` is caller-provided device memory of B*H*Nq floats. */
int wa_route_select(const float *block_attn, int B, int H, int Nq, int Nkv, double tau_min,
                    double tau_max, const int32_t *fixed_num_per_head, int32_t *index,
                    int32_t *num, uint8_t *mask, float *thresholds, float *gini_scratch,
                    void *stream);

/* The same selection as wa_route_select for callers that cannot allocate device memory where
 * routing runs (a server that partitions HBM once at start-up, a plugin whose host owns the
 * allocator, code that must avoid the device-wide synchronisation cudaMalloc implies).  It has no
 * counterpart in the reference.  The Gini scratch lives in a device array inside the library:
 * at most WA_ROUTE_SELECT_STATIC_MAX_ROWS rows (B*H*Nq); larger problems are rejected with
 * WA_ERR_UNSUPPORTED.  The library calls no allocation routine here.  The first call on each
 * device looks up the array's device address (one cudaGetSymbolAddress); make that first call
 * before any stream capture.  All calls on a device share the one array and it keeps the last
 * call's contents, so two calls that can overlap on the GPU (different streams) race: serialise
 * them.  Nothing in the array needs clearing between calls. */
#define WA_ROUTE_SELECT_STATIC_MAX_ROWS 65536
int wa_route_select_static(const float *block_attn, int B, int H, int Nq, int Nkv, double tau_min,
                           double tau_max, const int32_t *fixed_num_per_head, int32_t *index,
                           int32_t *num, uint8_t *mask, float *thresholds, void *stream);

/* map_to_index (block_sparse_triton.py:20-57).  Byte mask -> ascending ids (-1 filled) + count. */
int wa_map_to_index(const uint8_t *mask, int B, int H, int Nq, int Nkv, int32_t *index,
                    int32_t *num, void *stream);

/* Restriction of a routing decision to the key blocks [block_lo, block_hi) that one KV shard owns (no reference
 * counterpart: the reference is single-device).  Per row: the selected ids (first num entries of index, clamped to
 * [0, Nkv)) that fall in the range, rebased to the shard, duplicates collapsed, ascending; then the shard's other
 * blocks, ascending, so that every row of local_index [rows, block_hi - block_lo] is a permutation.
 * local_num [rows] = number of selected blocks of the shard.  At most 16384 blocks per shard. */
int wa_route_local_selection(const int32_t *index, const int32_t *num, long long rows, int Nkv, int block_lo,
                             int block_hi, int32_t *local_index, int32_t *local_num, void *stream);

/* Fixed top-k routing over a key cache that is SHARDED across ranks (no reference counterpart).  Step 1, per rank:
 * score the Nloc key blocks this rank owns (k_pooled_local `[B, H, Nloc, D]`, global ids block_lo ...) against every
 * query block and keep the best `kcap` of each row as 64-bit keys that sort ascending into (logit descending, global
 * block id ascending); absent entries are all-ones.  candidates `[B*H*Nq, kcap]`. */
int wa_route_local_candidates(const float *q_pooled, const float *k_pooled_local, int B, int H, int Nq, int Nloc, int D,
                              int block_lo, int kcap, unsigned long long *candidates, void *stream);
/* Step 2, after the ranks have exchanged their candidates (`[W, B*H*Nq, kcap]`, rank-major): per row the k_h =
 * min(topk_per_head[h], Nkv_total) best of all candidates; of those, the blocks in [block_lo, block_hi) go to
 * local_index (rebased to the shard, ascending, rows `index_stride` ints apart) and their number to local_num.
 * Selection is by logit; it equals wa_route_select's fixed-count choice except where distinct logits round to equal
 * probabilities at the k-th place. */
int wa_route_merge_candidates(const unsigned long long *candidates, int W, int B, int H, int Nq, int kcap,
                              const int32_t *topk_per_head, int Nkv_total, int block_lo, int block_hi, int index_stride,
                              int32_t *local_index, int32_t *local_num, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Attention branches -- wan/modules/hsa/block_sparse_torch.py, block_sparse_triton.py,
 * attention.py
 * ------------------------------------------------------------------------------------------- */

/* block_sparse_attention_reference (block_sparse_torch.py:16-64) and the inference branch of
 * block_sparse_attention (block_sparse_triton.py:371-382).  `Lq`/`Lkv` are the real lengths;
 * rows of the last query block beyond Lq are not written.  `index` rows are `index_stride` ints
 * apart; only the first num[b,h,i] entries are read and ids are clamped to [0, Nkv-1].
 * `block_sizes` (device `[Nkv]`) may be NULL, meaning min(block_size, Lkv - id*block_size).
 * Inputs are rounded to bf16 on load when `round_inputs_bf16` (attention.py:225-227); the result
 * is rounded to bf16 when `round_output_bf16`.  `lse` (float32 `[B,H,Lq]`, natural log, -inf for
 * an empty selection) may be NULL.  All-SIMT kernel for any D <= 256. */
int wa_block_sparse_forward(const wa_tensor4 *q, const wa_tensor4 *k, const wa_tensor4 *v,
                            const wa_tensor4 *out, int B, int H, int Lq, int Lkv, int D,
                            int block_size, const int32_t *index, const int32_t *num,
                            int index_stride, const int32_t *block_sizes, int round_inputs_bf16,
                            int round_output_bf16, float *lse, void *stream);

/* compress_kv (attention.py:64-110) on `[B, L, H, D]` views.  out_k/out_v receive
 * `[B, sum_seg rank_seg, H, D]`; `proj_*` are `[proj_rank, proj_cols]` row-major. */
int wa_compress_kv(const wa_tensor4 *k, const wa_tensor4 *v, const wa_tensor4 *out_k,
                   const wa_tensor4 *out_v, int B, int L, int H, int D, int segment_len,
                   int block_size, const void *k_proj, const void *v_proj, int proj_dtype,
                   int proj_rank, int proj_cols, void *stream);

/* The KV-cache write of one forward (causal_model.py:395-413, where the reference first clones the whole layer cache,
 * :294-299) fused with the compression of the segments it completes (causal_model.py:317-326 -> compress_kv): the
 * `n_new` new token rows `[B, n_new, H, D]` are read once, stored at rows [position, position + n_new) of the caches
 * `[B, capacity, H, D]`, and projected into compressed slots position / segment_len * rank ... of `k_coarse` /
 * `v_coarse` `[B, slots, H, D]`.  `position` is a multiple of segment_len (as token_range_to_coarse requires).
 * k_new / v_new may BE those cache rows (the rows were written in place, e.g. by a copy from the host): then nothing
 * is copied and the call only compresses; any other overlap with the caches is not allowed.  bf16, stride_h == D,
 * H*D a multiple of 128, rank <= 32 (WA_ERR_UNSUPPORTED otherwise: copy the rows and call wa_compress_kv).
 * `workspace`: wa_kv_append_workspace_bytes(...) bytes, 256-byte aligned, ZEROED before its first use (every call
 * leaves it ready for the next); calls that share a workspace must not overlap on the GPU.  (On an sm_100 device with
 * 16-byte aligned rows the call runs as a TMA + tcgen05 stream that needs no workspace; the SIMT kernel behind it
 * splits the tokens of a segment over several CTAs and adds their partial sums through the workspace.) */
size_t wa_kv_append_workspace_bytes(int B, int n_new, int H, int D, int segment_len, int block_size, int proj_rank);
int wa_kv_append_compress(const wa_tensor4 *k_new, const wa_tensor4 *v_new, const wa_tensor4 *k_cache,
                          const wa_tensor4 *v_cache, const wa_tensor4 *k_coarse, const wa_tensor4 *v_coarse, int B,
                          int n_new, int position, int H, int D, int segment_len, int block_size, const void *k_proj,
                          const void *v_proj, int proj_dtype, int proj_rank, int proj_cols, void *workspace,
                          size_t workspace_bytes, void *stream);

/* Failure detection for the tcgen05 compress / append stream: every wait inside it is bounded; a wait that ran out
 * leaves its site code in a word inside the library (sticky; 0 = no failure so far).  Waits for the device. */
int wa_compress_status(int *status);

/* _linear_branch (attention.py:113-118): dense softmax attention of q over Lc compressed slots.
 * Output rounded to bf16 when `round_output_bf16`; `lse` as above, may be NULL. */
int wa_linear_branch(const wa_tensor4 *q, const wa_tensor4 *k_coarse, const wa_tensor4 *v_coarse,
                     const wa_tensor4 *out, int B, int H, int Lq, int Lc, int D,
                     int round_output_bf16, float *lse, void *stream);

/* Gate and combine (attention.py:246-259): out = sparse + linear * sigmoid(q W^T + b), or
 * sigmoid(q) when gate_w is NULL.  W is `[D, D]` row-major (nn.Linear weight), b `[D]` or NULL. */
int wa_gate_combine(const wa_tensor4 *q, const wa_tensor4 *sparse, const wa_tensor4 *linear,
                    const wa_tensor4 *out, int B, int L, int H, int D, const void *gate_w,
                    const void *gate_b, int gate_dtype, int round_gate_bf16, void *stream);

/* Merge G shard partials of one branch: out = sum_g exp(lse_g - LSE) out_g (float32, natural
 * log).  `outs` is `[G, rows, D]`, `lses` `[G, rows]`.  Used by the KV-sharded multi-GPU path;
 * the reference has no sharded attention (its softmax, block_sparse_torch.py:62-64, is the G=1
 * case). */
int wa_merge_partials(const float *outs, const float *lses, int G, int64_t rows, int D,
                      float *out, float *lse, void *stream);

/* The same merge for the packed records of the KV-sharded exchange (see wa_hsa_params::part_stride): `recv` holds
 * G x vectors records of `record` floats, [sparse (D) | linear (D) | lse_sparse lse_linear ...], shard-major.  Writes
 * the merged sparse branch rounded to bf16 (attention.py:253 casts it so) and the merged linear branch in float32,
 * both `[vectors, D]`: the inputs of wa_gate_combine. */
int wa_merge_packed(const float *recv, int G, int64_t vectors, int D, int record, void *sparse_out, float *linear_out,
                    void *stream);

/* hsa_attention (attention.py:153-259), the whole forward in one call. */
typedef struct wa_hsa_params {
    int32_t B, H, D, Lq, Lkv, Lc; /* Lc = compressed slots supplied (0: compress inline)       */
    int32_t block_size;
    int32_t proj_segment_len, proj_rank, proj_cols, proj_dtype;
    int32_t gate_dtype; /* dtype of gate_w / gate_b                                            */
    int32_t flags;      /* WA_HSA_*                                                            */
    int32_t reserved;
    double tau_min, tau_max;
    wa_tensor4 q, k, v, k_coarse, v_coarse, out;
    const void *k_proj, *v_proj;         /* `[proj_rank, proj_cols]`; unused when Lc > 0        */
    const void *gate_w, *gate_b;         /* NULL gate_w: gate = sigmoid(q)                      */
    const int32_t *topk_per_head;        /* device `[H]` or NULL (cumulative-mass routing)      */
    int32_t *index_out;                  /* optional `[B,H,Nq,Nkv]`, NULL: kept in workspace    */
    int32_t *num_out;                    /* optional `[B,H,Nq]`                                 */
    float *thresholds_out;               /* optional `[H]`                                      */
    void *workspace;
    size_t workspace_bytes;
    /* Sharded execution (no reference counterpart; the reference is single-device).
     * index_in / num_in: routing decided elsewhere (e.g. globally across key shards) and already
     * restricted to this call's key range; when set, pooling and selection are skipped.
     * part_*: when part_sparse is set the call stops before the gate: it writes the normalised
     * float32 output of each branch `[B, Lq, H, D]` (contiguous) and its natural-log row
     * normaliser `[B, H, Lq]` (-inf where the branch saw no key), for wa_merge_partials. */
    const int32_t *index_in, *num_in;
    float *part_sparse, *part_linear, *lse_sparse, *lse_linear;
    /* Pooled-key cache (no reference counterpart: the reference pools the whole key cache on every call).
     * k_pooled: float32 `[B, H, Nkv, D]` (Nkv = ceil(Lkv / block_size)) that the caller keeps across calls on a
     * growing cache.  Its first k_pooled_valid blocks already hold the block means of k -- blocks that were complete
     * at an earlier call and have not changed since.  The call pools only the blocks from k_pooled_valid on into it
     * and routes on the whole buffer (results are identical to pooling everything).  NULL: the pooled keys live in
     * the workspace and every block is pooled.  Ignored when index_in is set. */
    float *k_pooled;
    int32_t k_pooled_valid, reserved2;
    /* Failure mirror (optional, may be NULL): an int32 the device can write and the host can read without a
     * copy -- page-locked host memory.  When a bounded wait inside the tcgen05 kernel runs out, the site code
     * that wa_hsa_status would return is also stored here, so a caller can poll it at its own synchronisation
     * points instead of paying a device-to-host copy per call.  The library never clears it. */
    int32_t *status_mirror;
    /* Layout of the partial outputs (0 everywhere: the contiguous defaults described above).  part_stride: floats
     * between the vectors of consecutive (token, head) pairs in part_sparse / part_linear (a multiple of 4, >= D), the
     * vector of (b, token, head) starting at ((b * Lq + token) * H + head) * part_stride.  lse_stride_token /
     * lse_stride_head: the normaliser of (b, head, token) sits at (b * Lq + token) * lse_stride_token + head *
     * lse_stride_head.  With part_linear = part_sparse + D, lse_sparse = part_sparse + 2 D, lse_linear = lse_sparse + 1,
     * part_stride = lse_stride_head = 2 D + 4 and lse_stride_token = H * part_stride, a (token, head) becomes ONE
     * record [sparse | linear | lse_s lse_l pad pad] and the rows of a query range one contiguous block: the unit the
     * KV-sharded path exchanges.  tcgen05 kernel only. */
    int64_t part_stride, lse_stride_token, lse_stride_head;
    /* Partial outputs written straight into the buffers of the ranks that merge them (KV-sharded multi-GPU, B = 1, packed
     * records as above).  peer_rows > 0 switches it on: query row t belongs to rank t / peer_rows and is stored as that
     * rank's row peer_self * peer_rows + t % peer_rows, i.e. the record of (t, head) goes to
     * part_sparse + peer_delta[t / peer_rows] + ((peer_self * peer_rows + t % peer_rows) * H + head) * part_stride
     * (likewise part_linear and the normalisers).  peer_delta[r] is the distance IN FLOATS from this rank's buffer to rank
     * r's buffer as mapped into this process (CUDA IPC / peer access; 0 for the rank itself; a multiple of 4, since the
     * records leave in 16-byte stores).  Plain stores over NVLink: the
     * caller orders them against the readers (a collective or an event after the launch).  tcgen05 kernel only. */
    int32_t peer_rows, peer_self;
    int64_t peer_delta[8];
} wa_hsa_params;

/* Bytes of workspace wa_hsa_forward needs for these sizes (pointers in `p` are ignored). */
size_t wa_hsa_workspace_bytes(const wa_hsa_params *p);
/* Returns through *used_tuned (may be NULL) whether the tcgen05 kernel ran. */
int wa_hsa_forward(const wa_hsa_params *p, int *used_tuned, void *stream);
/* Failure detection for the tcgen05 kernel.  Every wait inside it is bounded; a wait that runs
 * out records its site (1..10) in the workspace, the kernel releases its tensor memory and
 * returns.  wa_hsa_status waits for `stream` and copies that flag to *status (0 = the last tuned
 * launch on this workspace completed normally).  `p` must be the params of that launch.  The
 * reference has no counterpart (its kernels cannot time out). */
int wa_hsa_status(const wa_hsa_params *p, int *status, void *stream);

/* ---------------------------------------------------------------------------------------------
 * q/k preparation of the DiT self-attention -- wan/modules/model.py, wan/modules/causal_model.py
 * ------------------------------------------------------------------------------------------- */

/* WanRMSNorm (model.py:70-86) over the H*D values of a token, then causal_rope_apply (causal_model.py:34-62), in one
 * pass.  x / out: `[B, L, H, D]` views of one dtype (float32 or bf16); the L tokens are a (frames, grid_h, grid_w)
 * grid whose first frame is `start_frame`.  norm_weight `[H*D]` (NULL: no normalisation).  freqs: the reference's
 * complex128 table as `[freq_rows, D/2, 2]` doubles (NULL: no rotation); of a head's D/2 pairs the first
 * D/2 - 2 (D/2 / 3) turn with the frame, the next (D/2) / 3 with the row, the last (D/2) / 3 with the column. */
int wa_qk_norm_rope(const wa_tensor4 *x, const wa_tensor4 *out, int B, int L, int H, int D, const void *norm_weight,
                    int weight_dtype, float eps, const double *freqs, int freq_rows, int start_frame, int grid_h,
                    int grid_w, void *stream);
/* The same with the first frame's index read from device memory when the kernel runs, so that a captured launch
 * (CUDA graph of a chunk's forwards) can be replayed at another position of the video. */
int wa_qk_norm_rope_at(const wa_tensor4 *x, const wa_tensor4 *out, int B, int L, int H, int D, const void *norm_weight,
                       int weight_dtype, float eps, const double *freqs, int freq_rows, const int32_t *start_frame_device,
                       int grid_h, int grid_w, void *stream);

/* The element-wise wrappers of a DiT block's sub-layers (wan/modules/causal_model.py:586-659 with WanLayerNorm,
 * wan/modules/model.py:89-103), bf16 rows `[rows, C]`, contiguous.  Frame f of the batch owns rows
 * [f * tokens_per_frame, (f + 1) * tokens_per_frame); its modulation vectors start at `ptr + f * mod_stride` elements.
 *   wa_ln_modulate:    out = LN(x) [* weight + bias], rounded to bf16, then * (1 + scale[f]) + shift[f] (each NULL = absent),
 *                      every step rounded to bf16 as the reference's tensor expressions round it.
 *   wa_gated_residual: out = x + y * gate[f] (gate NULL: x + y).  out may alias x. */
int wa_ln_modulate(const void *x, void *out, long long rows, int C, float eps, const void *weight, const void *bias,
                   const void *scale, const void *shift, long long mod_stride, int tokens_per_frame, void *stream);
int wa_gated_residual(const void *x, const void *y, void *out, long long rows, int C, const void *gate, long long mod_stride,
                      int tokens_per_frame, void *stream);

/* ---------------------------------------------------------------------------------------------
 * HKV retrieval -- pipeline/hkv/retrieval.py, rope.py, cache.py
 * ------------------------------------------------------------------------------------------- */

/* page_key_index + derope_temporal (retrieval.py:50-72, rope.py:70-82).  keys `[B, T, H, D]`;
 * `spans` device int32 `[P, 2]` (start, end) token ranges; `derope` device float `[F, nt, 2]`
 * = complex64 conj-rotation of frame f = t / frame_seq_length (NULL: no rotation).  Writes
 * float32 `[P, H*D]`: mean over the page's tokens, then over the batch. */
int wa_hkv_page_centroids(const wa_tensor4 *keys, int B, int T, int H, int D, const int32_t *spans,
                          int P, const float *derope, int n_frames, int n_temporal,
                          int frame_seq_length, float *page_index, void *stream);

/* score_pages + top-k (retrieval.py:75-89, 105-126).  `page_index` float32 `[P, G*Dg]`, `query`
 * `[G*Dg]`; G = 1 scores whole vectors (the reference), G = H scores each head's slice and
 * selects per head.  scores `[G, P]` = dot / scale (scale <= 0: no division).  top_ids /
 * top_scores `[G, topk]`: highest first, equal scores by lower id. */
int wa_hkv_score_topk(const float *page_index, const float *query, int P, int G, int Dg,
                      float scale, int topk, float *scores, int32_t *top_ids, float *top_scores,
                      void *stream);

/* The same for `layers` page indexes at once (no reference counterpart: the reference scores layer 0 only):
 * page_index `[layers, P, G*Dg]`, query `[G*Dg]` shared by the layers (query_layer_stride = 0) or one per layer
 * (stride in floats); scores `[layers, G, P]`, top_ids / top_scores `[layers, G, topk]`. */
int wa_hkv_score_topk_layers(const float *page_index, const float *query, int layers, int P, int G, int Dg,
                             long long query_layer_stride, float scale, int topk, float *scores, int32_t *top_ids,
                             float *top_scores, void *stream);

/* One page copy of the install step (cache.py:229-246).  `row_elems` contiguous elements per
 * token (H*D for whole-token pages, D for one head), token rows `src_stride` / `dst_stride`
 * elements apart.  `rot` >= 0 selects `rotations[rot]` (shift_temporal_rope, rope.py:50-67) and
 * applies it to the first 2*n_temporal elements of every head_dim-sized group; rot < 0 copies. */
typedef struct wa_page_copy {
    const void *src;
    void *dst;
    int64_t src_stride, dst_stride;
    int32_t n_tokens;
    int32_t rot;
} wa_page_copy;

/* Builds the copy records of a per-head retrieval on the device, where the selected ids are (no reference
 * counterpart: the reference walks Python lists on the host).  top_ids `[layers, heads, topk]` (topk <= 64, -1 =
 * none); page_src `[P]`: device address of each page's first token (layer 0, head 0), 0 = not resident.  Per
 * (layer, head) the resident ids are put in ascending (chronological) order and record r copies page r of that order,
 * head `head` only (head_dim elements per token, token rows src_token_stride / dst_token_stride elements apart),
 * from page_src[id] + layer * src_layer_stride to dst_base + layer * dst_layer_stride + r * page_tokens token rows;
 * rot = r when `rotate` is set, else -1.  Records of absent pages get n_tokens = 0 and are counted in *missing
 * (optional, caller zeroes it).  records `[layers * heads * topk]`.  Strides of layers in bytes. */
int wa_hkv_build_records(const int32_t *top_ids, int layers, int heads, int topk, const long long *page_src, int P,
                         long long src_layer_stride, long long src_token_stride, void *dst_base,
                         long long dst_layer_stride, long long dst_token_stride, int page_tokens, int head_dim,
                         int elem_size, int rotate, wa_page_copy *records, int32_t *missing, void *stream);

/* Promotion of cold pages (the `.to(device)` of cache.py:229-231 for chunks that live in host memory): one
 * asynchronous host-to-device copy per record of the HOST array `host_records` (src = page-locked host memory,
 * dst = device memory, `rot` ignored), queued on `stream` -- the caller's side stream.  A record whose token rows
 * are `row_elems` apart on both sides moves as one block, any other as a two-dimensional copy.  No kernel is
 * launched and nothing waits: record an event on `stream` afterwards and let the install stream wait for it. */
int wa_hkv_promote_pages(const wa_page_copy *host_records, int n, int row_elems, int elem_size, void *stream);

/* `copies` is a device array of `n` records; `rotations` device float `[R, nt, 2]`. */
int wa_hkv_gather_pages(const wa_page_copy *copies, int n, int max_tokens, int row_elems,
                        int head_dim, int dtype, const float *rotations, int n_temporal,
                        void *stream);

#ifdef __cplusplus
}
#endif
#endif /* WORLDATTENTION_B200_H_ */
