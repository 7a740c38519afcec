// Low-rank sequence projection of K and V (the "compressed cache" of the HSA linear branch).
//
// Stands in for compress_kv, wan/modules/hsa/attention.py:64-110: per segment of `segment_len`
// tokens, out[r, :] = sum_t E[r, t] * x[t, :], r < min(proj_rank, ceil(seg_tokens / block_size)).
// SIMT kernel: one thread per (head, channel) column, the projection tile broadcast from shared
// memory, float32 accumulation.
#include "wa_common.cuh"

namespace wa {

constexpr int CK_THREADS = 128;
constexpr int CK_RMAX = 32;   // ranks accumulated per pass
constexpr int CK_TT = 64;     // tokens per shared-memory projection tile

__global__ void __launch_bounds__(CK_THREADS)
compress_kernel(View4 k, View4 v, void *ok, void *ov, int out_dtype, long long osb, long long osl, long long osh,
                int L, int H, int D, int segment_len, int block_size, const void *pk, const void *pv, int pdt,
                int proj_rank, int proj_cols, int rank_full) {
    __shared__ float es[CK_RMAX][CK_TT];
    const int col = blockIdx.x * CK_THREADS + threadIdx.x;
    const int seg = blockIdx.y;
    const int b = blockIdx.z >> 1, which = blockIdx.z & 1;
    const View4 x = which ? v : k;
    const void *proj = which ? pv : pk;
    void *out = which ? ov : ok;

    const int t0 = seg * segment_len;
    const int n_tok = min(segment_len, L - t0);
    const int rank = min(proj_rank, (n_tok + block_size - 1) / block_size);
    const bool active = col < H * D;
    const int h = active ? col / D : 0, d = active ? col % D : 0;
    const long long xoff = (long long)b * x.sb + (long long)h * x.sh + d;
    const long long ooff = (long long)b * osb + (long long)h * osh + d;

    for (int r0 = 0; r0 < rank; r0 += CK_RMAX) {
        const int nr = min(CK_RMAX, rank - r0);
        float acc[CK_RMAX];
#pragma unroll
        for (int r = 0; r < CK_RMAX; ++r) acc[r] = 0.f;
        for (int tt0 = 0; tt0 < n_tok; tt0 += CK_TT) {
            const int nt = min(CK_TT, n_tok - tt0);
            __syncthreads();
            for (int e = threadIdx.x; e < CK_RMAX * CK_TT; e += CK_THREADS) {
                const int r = e / CK_TT, t = e % CK_TT;
                es[r][t] = (r < nr && t < nt) ? load_elem(proj, pdt, (long long)(r0 + r) * proj_cols + tt0 + t) : 0.f;
            }
            __syncthreads();
            if (active) {
                for (int t = 0; t < nt; ++t) {
                    const float xv = load_elem(x.ptr, x.dtype, xoff + (long long)(t0 + tt0 + t) * x.sl);
#pragma unroll
                    for (int r = 0; r < CK_RMAX; ++r) acc[r] = fmaf(es[r][t], xv, acc[r]);
                }
            }
        }
        if (active) {
#pragma unroll
            for (int r = 0; r < CK_RMAX; ++r)
                if (r < nr)
                    store_elem(out, out_dtype, ooff + (long long)(seg * rank_full + r0 + r) * osl, acc[r]);
        }
    }
}

}  // namespace wa

using namespace wa;

extern "C" int wa_compress_kv(const wa_tensor4 *k, const wa_tensor4 *v, const wa_tensor4 *out_k,
                              const wa_tensor4 *out_v, int B, int L, int H, int D, int segment_len, int block_size,
                              const void *k_proj, const void *v_proj, int proj_dtype, int proj_rank, int proj_cols,
                              void *stream) {
    const char *what = "wa_compress_kv";
    WA_REQUIRE(k && v && out_k && out_v && k->ptr && v->ptr && out_k->ptr && out_v->ptr && k_proj && v_proj,
               WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(valid_dtype(k->dtype) && k->dtype == v->dtype && valid_dtype(out_k->dtype) &&
                   out_k->dtype == out_v->dtype && valid_dtype(proj_dtype),
               WA_ERR_ARG, "%s: bad or mismatched dtypes", what);
    WA_REQUIRE(B > 0 && L > 0 && H > 0 && D > 0 && block_size > 0 && proj_rank > 0 && proj_cols > 0, WA_ERR_ARG,
               "%s: sizes must be positive", what);
    WA_REQUIRE(out_k->stride_b == out_v->stride_b && out_k->stride_l == out_v->stride_l &&
                   out_k->stride_h == out_v->stride_h,
               WA_ERR_ARG, "%s: out_k and out_v must share strides", what);
    if (segment_len <= 0) segment_len = L;
    const int n_seg = ceil_div(L, segment_len);
    const int longest = L < segment_len ? L : segment_len;
    WA_REQUIRE(longest <= proj_cols, WA_ERR_ARG, "%s: segment length %d exceeds projection length %d", what,
               longest, proj_cols);
    const int rank_full = proj_rank < ceil_div(longest, block_size) ? proj_rank : ceil_div(longest, block_size);
    WA_REQUIRE(n_seg <= 65535 && 2 * B <= 65535, WA_ERR_UNSUPPORTED, "%s: too many segments", what);
    dim3 grid(ceil_div(H * D, CK_THREADS), n_seg, 2 * B);
    compress_kernel<<<grid, CK_THREADS, 0, (cudaStream_t)stream>>>(
        make_view(k), make_view(v), out_k->ptr, out_v->ptr, out_k->dtype, out_k->stride_b, out_k->stride_l,
        out_k->stride_h, L, H, D, segment_len, block_size, k_proj, v_proj, proj_dtype, proj_rank, proj_cols,
        rank_full);
    return check_launch(what);
}
