// Low-rank sequence projection of K and V (the "compressed cache" of the HSA linear branch).
//
// Stands in for compress_kv, wan/modules/hsa/attention.py:64-110: per segment of `segment_len`
// tokens, out[r, :] = sum_t E[r, t] * x[t, :], r < min(proj_rank, ceil(seg_tokens / block_size)).
// SIMT kernel: one thread per (head, channel) column, the projection tile broadcast from shared
// memory, float32 accumulation.
#include "wa_common.cuh"
#include "wa_internal.cuh"

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

// ------------------------------------------------------------------------------------------------
// Append + compress in one pass (bf16, heads contiguous, rank <= 32): the new token rows are read ONCE;
// every row is stored at its place in the K/V cache and, from the same registers, accumulated into the
// compressed slots of its segment.  The tokens of a segment are split over SPLIT CTAs so that a chunk of a
// few segments still fills the GPU; a CTA leaves its float32 partial sums in the workspace, and the CTA
// that finishes a (column tile, segment, K|V, batch) group last adds the SPLIT partials in split order --
// a fixed order, whoever arrives last -- rounds to bf16 and resets the group's counter for the next call.
// ------------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(CF_WARPS * 32)
append_compress_kernel(const __nv_bfloat16 *__restrict__ k_new, const __nv_bfloat16 *__restrict__ v_new, long long nsb, long long nsl,
                       __nv_bfloat16 *__restrict__ k_cache, __nv_bfloat16 *__restrict__ v_cache, long long csb, long long csl,
                       int position, __nv_bfloat16 *__restrict__ ok, __nv_bfloat16 *__restrict__ ov, long long osb, long long osl,
                       int slot0, int n_new, int segment_len, int block_size, int split, int tokens_per_split, const void *pk,
                       const void *pv, int pdt, int proj_rank, int proj_cols, int slot_stride, float *__restrict__ partials,
                       int *__restrict__ counters) {
    __shared__ __align__(16) float es[CF_TT][R];
    __shared__ float red[R][128];
    __shared__ int last_flag;
    const int col0 = blockIdx.x * 128;
    const int seg = blockIdx.y / split, part = blockIdx.y % split;
    const int b = blockIdx.z >> 1, which = blockIdx.z & 1;
    const __nv_bfloat16 *x = (which ? v_new : k_new) + (long long)b * nsb + col0;
    __nv_bfloat16 *cache = (which ? v_cache : k_cache) + (long long)b * csb + col0;
    const bool copy = cache + (long long)position * csl != x;   // rows that are in place already are not copied onto themselves
    const void *proj = which ? pv : pk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const int t0 = seg * segment_len;                       // first new token of the segment
    const int seg_tok = min(segment_len, n_new - t0);
    const int rank = min(proj_rank, (seg_tok + block_size - 1) / block_size);
    const int p0 = part * tokens_per_split, p1 = min(seg_tok, p0 + tokens_per_split);   // this CTA's tokens of the segment

    float acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;

    for (int tt0 = p0; tt0 < p1; tt0 += CF_TT) {
        const int nt = min(CF_TT, p1 - tt0);
        __syncthreads();
        for (int e = threadIdx.x; e < CF_TT * R; e += CF_WARPS * 32) {
            const int r = e / CF_TT, t = e % CF_TT;
            es[t][r] = (r < rank && t < nt) ? load_elem(proj, pdt, (long long)r * proj_cols + tt0 + t) : 0.f;
        }
        __syncthreads();
        for (int g0 = 0; g0 < CF_TT / CF_WARPS; g0 += CF_PF) {
            uint2 raw[CF_PF];
#pragma unroll
            for (int i = 0; i < CF_PF; ++i) {
                const int t = warp + (g0 + i) * CF_WARPS;
                raw[i] = t < nt ? *reinterpret_cast<const uint2 *>(x + (long long)(t0 + tt0 + t) * nsl + lane * 4) : make_uint2(0u, 0u);
            }
#pragma unroll
            for (int i = 0; i < CF_PF; ++i) {
                const int t = warp + (g0 + i) * CF_WARPS;
                if (t >= nt) break;
                if (copy) *reinterpret_cast<uint2 *>(cache + (long long)(position + t0 + tt0 + t) * csl + lane * 4) = raw[i];
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
    // group = (batch, K|V, segment, column tile); its SPLIT partials are [split][R][128] floats
    const long long group = ((long long)blockIdx.z * (gridDim.y / split) + seg) * gridDim.x + blockIdx.x;
    float *mine = partials + (group * split + part) * (long long)(R * 128);
    for (int e = threadIdx.x; e < rank * 128; e += CF_WARPS * 32) mine[e] = red[e / 128][e % 128];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_flag = atomicAdd(&counters[group], 1) == split - 1;
    __syncthreads();
    if (!last_flag) return;
    __threadfence();
    __nv_bfloat16 *out = (which ? ov : ok) + (long long)b * osb + col0;
    const float *all = partials + group * split * (long long)(R * 128);
    for (int e = threadIdx.x; e < rank * 128; e += CF_WARPS * 32) {
        float sum = 0.f;
        for (int s = 0; s < split; ++s) sum += __ldcg(all + (long long)s * (R * 128) + e);
        out[(long long)(slot0 + seg * slot_stride + e / 128) * osl + e % 128] = __float2bfloat16_rn(sum);
    }
    if (threadIdx.x == 0) counters[group] = 0;   // ready for the next call on this workspace
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
    // bf16 with contiguous heads on an sm_100 device: the TMA + tcgen05 stream (reads K and V once at HBM speed)
    if (compress_sm100_supported(k, v, out_k, out_v, nullptr, nullptr, H, D, proj_dtype, proj_cols, rank_full, k_proj, v_proj))
        return compress_sm100_launch(k, v, out_k, out_v, nullptr, nullptr, 0, B, L, H, D, segment_len, block_size, k_proj, v_proj,
                                     proj_rank, proj_cols, 0, rank_full, (cudaStream_t)stream);
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

// Workspace of wa_kv_append_compress: counters first (they must be zero before the FIRST call and are left zero by every
// call), then the float32 partial sums.
namespace {
struct AppendPlan {
    int n_seg, split, tokens_per_split, rank_full, slot_stride, tiles;
    size_t counters_bytes, total_bytes;
};
AppendPlan append_plan(int B, int n_new, int H, int D, int segment_len, int block_size, int proj_rank) {
    AppendPlan a{};
    a.n_seg = ceil_div(n_new, segment_len);
    const int longest = n_new < segment_len ? n_new : segment_len;
    a.rank_full = proj_rank < ceil_div(longest, block_size) ? proj_rank : ceil_div(longest, block_size);
    // slots a whole segment occupies in the compressed cache: the cache is laid out for full segments, whatever this call appends
    a.slot_stride = proj_rank < ceil_div(segment_len, block_size) ? proj_rank : ceil_div(segment_len, block_size);
    a.tiles = H * D / 128;
    // enough CTAs for two per SM of a large GPU, but no split shorter than one staged projection tile
    const int groups = a.tiles * a.n_seg * 2 * B;
    int split = groups >= 296 ? 1 : ceil_div(296, groups);
    const int max_split = longest / CF_TT > 0 ? longest / CF_TT : 1;
    if (split > max_split) split = max_split;
    if (split > 16) split = 16;
    a.split = split;
    a.tokens_per_split = ceil_div(ceil_div(longest, split), CF_WARPS) * CF_WARPS;
    a.counters_bytes = align_up((size_t)groups * sizeof(int), 256);
    a.total_bytes = a.counters_bytes + (size_t)groups * split * 32 * 128 * sizeof(float);
    return a;
}
}  // namespace

extern "C" size_t wa_kv_append_workspace_bytes(int B, int n_new, int H, int D, int segment_len, int block_size, int proj_rank) {
    if (B <= 0 || n_new <= 0 || H <= 0 || D <= 0 || block_size <= 0 || proj_rank <= 0) return 0;
    if (segment_len <= 0) segment_len = n_new;
    return append_plan(B, n_new, H, D, segment_len, block_size, proj_rank).total_bytes;
}

extern "C" int wa_kv_append_compress(const wa_tensor4 *k_new, const wa_tensor4 *v_new, const wa_tensor4 *k_cache,
                                     const wa_tensor4 *v_cache, const wa_tensor4 *k_coarse, const wa_tensor4 *v_coarse, int B,
                                     int n_new, int position, int H, int D, int segment_len, int block_size, const void *k_proj,
                                     const void *v_proj, int proj_dtype, int proj_rank, int proj_cols, void *workspace,
                                     size_t workspace_bytes, void *stream) {
    const char *what = "wa_kv_append_compress";
    WA_REQUIRE(k_new && v_new && k_cache && v_cache && k_coarse && v_coarse && k_new->ptr && v_new->ptr && k_cache->ptr &&
                   v_cache->ptr && k_coarse->ptr && v_coarse->ptr && k_proj && v_proj,
               WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(B > 0 && n_new > 0 && H > 0 && D > 0 && block_size > 0 && proj_rank > 0 && proj_cols > 0 && position >= 0, WA_ERR_ARG,
               "%s: sizes must be positive", what);
    if (segment_len <= 0) segment_len = n_new;
    WA_REQUIRE(position % segment_len == 0, WA_ERR_ARG,
               "%s: rows are appended at segment boundaries (position %d, segment length %d)", what, position, segment_len);
    const int longest = n_new < segment_len ? n_new : segment_len;
    WA_REQUIRE(longest <= proj_cols, WA_ERR_ARG, "%s: segment length %d exceeds projection length %d", what, longest, proj_cols);
    WA_REQUIRE(valid_dtype(proj_dtype), WA_ERR_ARG, "%s: bad projection dtype", what);
    const AppendPlan a = append_plan(B, n_new, H, D, segment_len, block_size, proj_rank);
    {   // the TMA + tcgen05 stream: token tiles are read once and leave twice (cache rows, compressed slots); no workspace
        const bool in_place = (char *)k_new->ptr == (char *)k_cache->ptr + (size_t)position * k_cache->stride_l * 2 &&
                              (char *)v_new->ptr == (char *)v_cache->ptr + (size_t)position * v_cache->stride_l * 2 &&
                              k_new->stride_l == k_cache->stride_l && k_new->stride_b == k_cache->stride_b &&
                              v_new->stride_l == v_cache->stride_l && v_new->stride_b == v_cache->stride_b;
        if (k_coarse->stride_b == v_coarse->stride_b && k_coarse->stride_l == v_coarse->stride_l &&
            compress_sm100_supported(k_new, v_new, k_coarse, v_coarse, in_place ? nullptr : k_cache, in_place ? nullptr : v_cache, H, D,
                                     proj_dtype, proj_cols, a.rank_full, k_proj, v_proj))
            return compress_sm100_launch(k_new, v_new, k_coarse, v_coarse, in_place ? nullptr : k_cache, in_place ? nullptr : v_cache,
                                         position, B, n_new, H, D, segment_len, block_size, k_proj, v_proj, proj_rank, proj_cols,
                                         position / segment_len * a.slot_stride, a.slot_stride, (cudaStream_t)stream);
    }
    const wa_tensor4 *views[6] = {k_new, v_new, k_cache, v_cache, k_coarse, v_coarse};
    bool fast = (H * D) % 128 == 0 && a.rank_full <= 32 && a.n_seg * a.split <= 65535 && 2 * B <= 65535;
    for (const wa_tensor4 *t : views)
        fast = fast && t->dtype == WA_BF16 && t->stride_h == D && t->stride_l % 4 == 0 && t->stride_b % 4 == 0 && (uintptr_t)t->ptr % 8 == 0;
    fast = fast && k_new->stride_b == v_new->stride_b && k_new->stride_l == v_new->stride_l && k_cache->stride_b == v_cache->stride_b &&
           k_cache->stride_l == v_cache->stride_l && k_coarse->stride_b == v_coarse->stride_b && k_coarse->stride_l == v_coarse->stride_l;
    WA_REQUIRE(fast, WA_ERR_UNSUPPORTED,
               "%s: needs bf16 tensors with contiguous heads (stride_h == D), H*D a multiple of 128, rank <= 32 and K/V pairs that "
               "share strides; copy the rows and call wa_compress_kv otherwise", what);
    WA_REQUIRE(workspace && workspace_bytes >= a.total_bytes && (uintptr_t)workspace % 256 == 0, WA_ERR_WORKSPACE,
               "%s: a 256-byte aligned workspace of %zu bytes is required (zeroed before its first use)", what, a.total_bytes);
    int *counters = (int *)workspace;
    float *partials = (float *)((char *)workspace + a.counters_bytes);
    const int slot0 = position / segment_len * a.slot_stride;
    dim3 grid(a.tiles, a.n_seg * a.split, 2 * B);
#define WA_APPEND_LAUNCH(R)                                                                                                      \
    append_compress_kernel<R><<<grid, CF_WARPS * 32, 0, (cudaStream_t)stream>>>(                                                 \
        (const __nv_bfloat16 *)k_new->ptr, (const __nv_bfloat16 *)v_new->ptr, k_new->stride_b, k_new->stride_l,                  \
        (__nv_bfloat16 *)k_cache->ptr, (__nv_bfloat16 *)v_cache->ptr, k_cache->stride_b, k_cache->stride_l, position,            \
        (__nv_bfloat16 *)k_coarse->ptr, (__nv_bfloat16 *)v_coarse->ptr, k_coarse->stride_b, k_coarse->stride_l, slot0, n_new,    \
        segment_len, block_size, a.split, a.tokens_per_split, k_proj, v_proj, proj_dtype, proj_rank, proj_cols, a.slot_stride,   \
        partials, counters)
    if (a.rank_full <= 16) WA_APPEND_LAUNCH(16);
    else WA_APPEND_LAUNCH(32);
#undef WA_APPEND_LAUNCH
    return check_launch(what);
}
