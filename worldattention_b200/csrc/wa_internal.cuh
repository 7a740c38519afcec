// Internal (non-ABI) declarations shared between translation units.
#pragma once
#include "wa_common.cuh"

namespace wa {

// Launch preparation of the tcgen05 kernel that can ride on another kernel: the heaviest-first work
// order over all (batch, head, query block) items, the reset of the work counter and failure flag,
// and the bf16 copy of the gate weight.  `order == nullptr` means "nothing to prepare".
struct SchedJob {
    int32_t *order;
    int *work_counter;
    int *error_flag;
    const void *gate_w, *gate_b;
    int gate_dt;
    __nv_bfloat16 *w_out;   // [128 x 128] bf16
    float *b_out;           // [128] float32
    int release_dependents_after_rows;   // timing experiment (WA_B200_PDL=2), see route_row
};

constexpr int SCHED_BINS = 4096;

// Counting sort of the items by selected-block count, heaviest first.  Called by every thread of ONE
// CTA whose size is a power of two between 32 and 1024.
__device__ inline void schedule_items(const int32_t *num, int n_items, int Nkv, int32_t *__restrict__ order,
                                      int *work_counter, int *error_flag) {
    __shared__ int hist[SCHED_BINS];
    __shared__ int warp_tot[32];
    const int T = blockDim.x, tid = threadIdx.x;
    // bins 0..top hold counts top..0 (bin 0 = heaviest); `per` bins per thread, a power of two >= 1
    const int top = min(Nkv, SCHED_BINS - 1);
    int per = 1;
    while (per * T < top + 1) per <<= 1;
    for (int i = tid; i < per * T; i += T) hist[i] = 0;
    if (tid == 0) {
        *work_counter = 0;
        *error_flag = 0;
    }
    __syncthreads();
    // the counts were written by other CTAs of this launch: read them past L1, and only once when they fit in registers
    constexpr int KEEP = 4;
    int bin_of[KEEP];
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
        const int i = tid + u * T;
        bin_of[u] = i < n_items ? top - max(0, min(__ldcg(num + i), top)) : -1;
    }
#pragma unroll
    for (int u = 0; u < KEEP; ++u)
        if (bin_of[u] >= 0) atomicAdd(&hist[bin_of[u]], 1);
    for (int i = tid + KEEP * T; i < n_items; i += T) atomicAdd(&hist[top - max(0, min(__ldcg(num + i), top))], 1);
    __syncthreads();
    // exclusive prefix over the bins: a contiguous run of bins per thread, then a block scan of the run totals
    const int b0 = tid * per;
    int mine = 0;
    for (int i = 0; i < per; ++i) mine += hist[b0 + i];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if ((tid & 31) >= o) incl += v;
    }
    if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        int w = tid < (T >> 5) ? warp_tot[tid] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (tid >= o) w += v;
        }
        warp_tot[tid] = w;
    }
    __syncthreads();
    int base = incl - mine + ((tid >> 5) ? warp_tot[(tid >> 5) - 1] : 0);
    for (int i = 0; i < per; ++i) {
        const int c = hist[b0 + i];
        hist[b0 + i] = base;
        base += c;
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < KEEP; ++u)
        if (bin_of[u] >= 0) order[atomicAdd(&hist[bin_of[u]], 1)] = tid + u * T;
    for (int i = tid + KEEP * T; i < n_items; i += T) order[atomicAdd(&hist[top - max(0, min(__ldcg(num + i), top))], 1)] = i;
}

// Elements [first, first + count) of the gate weight -> bf16 (it is an MMA operand) and of the bias -> float32.
__device__ inline void convert_gate_slice(const SchedJob &job, int first, int count) {
    for (int i = first + threadIdx.x; i < first + count && i < 128 * 128; i += blockDim.x) {
        job.w_out[i] = __float2bfloat16_rn(load_elem(job.gate_w, job.gate_dt, i));
        if (i < 128) job.b_out[i] = job.gate_b ? load_elem(job.gate_b, job.gate_dt, i) : 0.f;
    }
}

// routing (wa_routing.cu): pools x and optionally y in one launch; zeroes `n_zero` ints at `zero` on the way.
// `y_first_block`: the first blocks of y are already pooled in py (rows [0, y_first_block) per batch and head).
int pool_launch(const wa_tensor4 *x, int Lx, float *px, const wa_tensor4 *y, int Ly, float *py, int B, int H, int D,
                int block_size, cudaStream_t stream, int *zero = nullptr, int n_zero = 0, int y_first_block = 0,
                int *status_mirror = nullptr);   // host-visible word that receives a non-zero code if a bounded wait of the TMA kernel runs out

// routing (wa_routing.cu): scores, sort, Gini thresholds and counts in ONE launch (plus `job` when its order is set).
// `sorted` ([rows, Nkv] float32) and `gini` ([rows]) are scratch; `counters` are H + 1 ints that are zero on entry.
int route_fused_launch(const float *q_pooled, const float *k_pooled, int B, int H, int Nq, int Nkv, int D, double tau_min,
                       double tau_max, const int32_t *fixed_num_per_head, float *sorted, int32_t *index, int32_t *num,
                       float *thresholds, float *gini, int *counters, const SchedJob &job, cudaStream_t stream,
                       bool whole_order = true);   // false: only the first num[row] ids of a row are needed (fixed counts)

// optional CUDA-event bracket around the attention kernel (wa_api.cu)
void profile_mark(bool begin, cudaStream_t stream);
void profile_pause(bool on);   // nested launches that must not move the bracket

// tcgen05 fused HSA kernel (wa_hsa_sm100.cu)
size_t hsa_sm100_workspace_bytes(const wa_hsa_params *p);
size_t hsa_sm100_status_offset(const wa_hsa_params *p);   // int32 flag inside the tuned workspace
bool hsa_sm100_supported(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc);
SchedJob hsa_sm100_sched_job(const wa_hsa_params *p, void *workspace);
// `prepared`: the SchedJob of this call has already run on the stream (as part of the routing kernel)
int hsa_sm100_launch(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc,
                     const int32_t *index, const int32_t *num, int Nq, int Nkv, void *workspace,
                     bool prepared, cudaStream_t stream);

// the linear branch alone on the tcgen05 kernel (bf16, head_dim 128; any routing block size): float32 [B, Lq, H, 128]
bool hsa_sm100_linear_supported(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc);
int hsa_sm100_launch_linear(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc, float *linear_out,
                            void *workspace, cudaStream_t stream);

// block-mean pooling as a TMA stream (wa_pool_sm100.cu); y may be null; out_blocks_y = rows per (batch, head) of py
bool pool_sm100_supported(const wa_tensor4 *x, const wa_tensor4 *y, int H, int D, int block_size);
int pool_sm100_launch(const wa_tensor4 *x, int Lx, float *px, const wa_tensor4 *y, int Ly, float *py, int out_blocks_y, int B, int H,
                      int D, int block_size, cudaStream_t stream, int *zero, int n_zero, int *status_mirror);

// compress_kv / KV-cache append as a TMA + tcgen05 stream (wa_compress_sm100.cu)
bool compress_sm100_supported(const wa_tensor4 *k, const wa_tensor4 *v, const wa_tensor4 *ok, const wa_tensor4 *ov,
                              const wa_tensor4 *dst_k, const wa_tensor4 *dst_v, int H, int D, int proj_dtype, int proj_cols,
                              int rank_full, const void *k_proj, const void *v_proj);
int compress_sm100_launch(const wa_tensor4 *k, const wa_tensor4 *v, const wa_tensor4 *ok, const wa_tensor4 *ov,
                          const wa_tensor4 *dst_k, const wa_tensor4 *dst_v, int dst_row0, int B, int L, int H, int D,
                          int segment_len, int block_size, const void *k_proj, const void *v_proj, int proj_rank, int proj_cols,
                          int slot0, int slot_stride, cudaStream_t stream);

}  // namespace wa
