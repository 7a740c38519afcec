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


// ------------------------------------------------------------------------------------------------
// Fast path: bf16, heads contiguous (stride_h == D), rank <= 32.  One CTA per (128 columns, segment,
// K|V, batch); the eight warps take every eighth token, a lane owns four adjacent columns (8-byte
// loads), the projection tile is staged in shared memory as float32 [token][rank] so that four
// ranks come from one 16-byte broadcast load.  Partial sums of the warps are added in warp order.
// ------------------------------------------------------------------------------------------------
constexpr int CF_WARPS = 8;
constexpr int CF_TT = 128;      // tokens per staged projection tile (16 per warp)
constexpr int CF_PF = 8;        // token rows a warp keeps in flight

template <int R>                // padded rank: 16 or 32
__global__ void __launch_bounds__(CF_WARPS * 32)
compress_fast_kernel(const __nv_bfloat16 *__restrict__ k, const __nv_bfloat16 *__restrict__ v, long long xsb, long long xsl,
                     __nv_bfloat16 *__restrict__ ok, __nv_bfloat16 *__restrict__ ov, long long osb, long long osl, int L,
                     int segment_len, int block_size, const void *pk, const void *pv, int pdt, int proj_rank,
                     int proj_cols, int rank_full) {
    __shared__ __align__(16) float es[CF_TT][R];
    __shared__ float red[R][128];
    const int col0 = blockIdx.x * 128;
    const int seg = blockIdx.y;
    const int b = blockIdx.z >> 1, which = blockIdx.z & 1;
    const __nv_bfloat16 *x = (which ? v : k) + (long long)b * xsb + col0;
    const void *proj = which ? pv : pk;
    __nv_bfloat16 *out = (which ? ov : ok) + (long long)b * osb + col0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int t0 = seg * segment_len;
    const int n_tok = min(segment_len, L - t0);
    const int rank = min(proj_rank, (n_tok + block_size - 1) / block_size);

    float acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;

    for (int tt0 = 0; tt0 < n_tok; tt0 += CF_TT) {
        const int nt = min(CF_TT, n_tok - tt0);
        __syncthreads();
        for (int e = threadIdx.x; e < CF_TT * R; e += CF_WARPS * 32) {
            const int r = e / CF_TT, t = e % CF_TT;     // consecutive threads read consecutive tokens of one row
            es[t][r] = (r < rank && t < nt) ? load_elem(proj, pdt, (long long)r * proj_cols + tt0 + t) : 0.f;
        }
        __syncthreads();
        // this warp's tokens of the tile: warp, warp + 8, ...; CF_PF rows are loaded before any is used
        for (int g0 = 0; g0 < CF_TT / CF_WARPS; g0 += CF_PF) {
            uint2 raw[CF_PF];
#pragma unroll
            for (int i = 0; i < CF_PF; ++i) {
                const int t = warp + (g0 + i) * CF_WARPS;
                raw[i] = t < nt ? *reinterpret_cast<const uint2 *>(x + (long long)(t0 + tt0 + t) * xsl + lane * 4)
                                : make_uint2(0u, 0u);
            }
#pragma unroll
            for (int i = 0; i < CF_PF; ++i) {
                const int t = warp + (g0 + i) * CF_WARPS;
                if (t >= nt) break;
                const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[i].x));
                const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[i].y));
#pragma unroll
                for (int r4 = 0; r4 < R; r4 += 4) {
                    const float4 e4 = *reinterpret_cast<const float4 *>(&es[t][r4]);
                    const float ev[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        acc[r4 + u][0] = fmaf(ev[u], x01.x, acc[r4 + u][0]);
                        acc[r4 + u][1] = fmaf(ev[u], x01.y, acc[r4 + u][1]);
                        acc[r4 + u][2] = fmaf(ev[u], x23.x, acc[r4 + u][2]);
                        acc[r4 + u][3] = fmaf(ev[u], x23.y, acc[r4 + u][3]);
                    }
                }
            }
        }
    }
    // ordered reduction over the warps
    for (int w = 0; w < CF_WARPS; ++w) {
        __syncthreads();
        if (warp == w) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (w == 0) red[r][lane * 4 + u] = acc[r][u];
                    else red[r][lane * 4 + u] += acc[r][u];
                }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < rank * 128; e += CF_WARPS * 32) {
        const int r = e / 128, c = e % 128;
        out[(long long)(seg * rank_full + r) * osl + c] = __float2bfloat16_rn(red[r][c]);
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
    const bool fast = k->dtype == WA_BF16 && out_k->dtype == WA_BF16 && k->stride_h == D && v->stride_h == D &&
                      out_k->stride_h == D && (H * D) % 128 == 0 && rank_full <= 32 && k->stride_b == v->stride_b &&
                      k->stride_l == v->stride_l && k->stride_l % 4 == 0 && k->stride_b % 4 == 0 &&
                      ((uintptr_t)k->ptr % 8 == 0) && ((uintptr_t)v->ptr % 8 == 0);
    if (fast) {
        dim3 fgrid(H * D / 128, n_seg, 2 * B);
        if (rank_full <= 16)
            compress_fast_kernel<16><<<fgrid, CF_WARPS * 32, 0, (cudaStream_t)stream>>>(
                (const __nv_bfloat16 *)k->ptr, (const __nv_bfloat16 *)v->ptr, k->stride_b, k->stride_l,
                (__nv_bfloat16 *)out_k->ptr, (__nv_bfloat16 *)out_v->ptr, out_k->stride_b, out_k->stride_l, L,
                segment_len, block_size, k_proj, v_proj, proj_dtype, proj_rank, proj_cols, rank_full);
        else
            compress_fast_kernel<32><<<fgrid, CF_WARPS * 32, 0, (cudaStream_t)stream>>>(
                (const __nv_bfloat16 *)k->ptr, (const __nv_bfloat16 *)v->ptr, k->stride_b, k->stride_l,
                (__nv_bfloat16 *)out_k->ptr, (__nv_bfloat16 *)out_v->ptr, out_k->stride_b, out_k->stride_l, L,
                segment_len, block_size, k_proj, v_proj, proj_dtype, proj_rank, proj_cols, rank_full);
        return check_launch(what);
    }
    dim3 grid(ceil_div(H * D, CK_THREADS), n_seg, 2 * B);
    compress_kernel<<<grid, CK_THREADS, 0, (cudaStream_t)stream>>>(
        make_view(k), make_view(v), out_k->ptr, out_v->ptr, out_k->dtype, out_k->stride_b, out_k->stride_l,
        out_k->stride_h, L, H, D, segment_len, block_size, k_proj, v_proj, proj_dtype, proj_rank, proj_cols,
        rank_full);
    return check_launch(what);
}
