// Hierarchical KV cache retrieval on the GPU: page centroids, page scoring + top-k, page install.
//
// Stand-ins for pipeline/hkv/retrieval.py:50-126, pipeline/hkv/rope.py:33-82 and the copy loop of
// pipeline/hkv/cache.py:229-246.  All three are byte-moving, HBM-bound kernels: 128-bit coalesced
// accesses, warp-shuffle reductions, no tensor cores.
#include "wa_common.cuh"

namespace wa {

// ------------------------------------------------------------------------------------------------
// Page centroids with the temporal rotation removed.
// grid (pair tiles, pages); block (CT_TX complex pairs, CT_TY token rows).
// ------------------------------------------------------------------------------------------------
constexpr int CT_TX = 64, CT_TY = 4;

__global__ void __launch_bounds__(CT_TX *CT_TY)
page_centroid_kernel(View4 keys, int B, int H, int D, const int32_t *__restrict__ spans,
                     const float2 *__restrict__ derope, int n_frames, int nt, int frame_seq_length,
                     float *__restrict__ page_index) {
    __shared__ double sre[CT_TY][CT_TX], sim[CT_TY][CT_TX];
    const int page = blockIdx.y;
    const int pair = blockIdx.x * CT_TX + threadIdx.x;   // complex pair within the H*D row
    const int ty = threadIdx.y;
    const int start = spans[2 * page], end = spans[2 * page + 1];
    const int n_tok = max(0, end - start);
    const bool active = pair < (H * D) / 2;
    const int h = active ? (2 * pair) / D : 0;
    const int dpair = active ? ((2 * pair) % D) / 2 : 0;
    const bool rotate = derope != nullptr && dpair < nt;

    double out_re = 0.0, out_im = 0.0;   // running sum over the batch of per-item token means
    for (int b = 0; b < B; ++b) {
        double acc_re = 0.0, acc_im = 0.0;
        if (active) {
            const long long base = (long long)b * keys.sb + (long long)h * keys.sh + 2 * dpair;
            for (int t = start + ty; t < end; t += CT_TY) {
                const long long off = base + (long long)t * keys.sl;
                float a = load_elem(keys.ptr, keys.dtype, off);
                float c = load_elem(keys.ptr, keys.dtype, off + 1);
                if (rotate) {
                    const int f = min(max(t / frame_seq_length, 0), n_frames - 1);
                    const float2 w = derope[(long long)f * nt + dpair];
                    const float re = __fsub_rn(__fmul_rn(a, w.x), __fmul_rn(c, w.y));
                    const float im = __fadd_rn(__fmul_rn(a, w.y), __fmul_rn(c, w.x));
                    a = re;
                    c = im;
                    if (keys.dtype == WA_BF16) {
                        a = bf16_round_f(a);
                        c = bf16_round_f(c);
                    }
                }
                acc_re += (double)a;
                acc_im += (double)c;
            }
        }
        sre[ty][threadIdx.x] = acc_re;
        sim[ty][threadIdx.x] = acc_im;
        __syncthreads();
        if (ty == 0 && active) {
            double r = 0.0, i = 0.0;
            for (int y = 0; y < CT_TY; ++y) {
                r += sre[y][threadIdx.x];
                i += sim[y][threadIdx.x];
            }
            out_re += (double)(float)(r / (double)max(n_tok, 1));
            out_im += (double)(float)(i / (double)max(n_tok, 1));
        }
        __syncthreads();
    }
    if (ty == 0 && active) {
        float *dst = page_index + (long long)page * H * D + 2 * pair;
        dst[0] = (float)(out_re / (double)B);
        dst[1] = (float)(out_im / (double)B);
    }
}

// The same for bf16 keys whose heads lie side by side (stride D, D a multiple of 8, 16-byte aligned rows): a thread owns
// FOUR neighbouring pairs (one 16-byte load per token) and keeps four tokens' loads in flight, so that the kernel streams
// instead of waiting for one 4-byte load per thread at a time (1.4 TB/s).  Same arithmetic per value; the float64 sums
// of a pair are taken token by token within a row group and the row groups are added in order, as above.
constexpr int CV_TX = 64, CV_TY = 4, CV_U = 4;

__global__ void __launch_bounds__(CV_TX *CV_TY)
page_centroid_vec_kernel(const __nv_bfloat16 *__restrict__ keys, long long sb, long long sl, int B, int H, int D,
                         const int32_t *__restrict__ spans, const float2 *__restrict__ derope, int n_frames, int nt,
                         int frame_seq_length, float *__restrict__ page_index) {
    __shared__ double sre[CV_TY][CV_TX][4], sim[CV_TY][CV_TX][4];
    const int page = blockIdx.y, ty = threadIdx.y;
    const int pair0 = (blockIdx.x * CV_TX + threadIdx.x) * 4;      // first of this thread's four pairs within the H*D row
    const int start = spans[2 * page], end = spans[2 * page + 1];
    const int n_tok = max(0, end - start);
    const bool active = pair0 < (H * D) / 2;
    const int dpair0 = active ? ((2 * pair0) % D) / 2 : 0;          // pair index inside the head (the four share a head)

    double out_re[4] = {0.0, 0.0, 0.0, 0.0}, out_im[4] = {0.0, 0.0, 0.0, 0.0};
    for (int b = 0; b < B; ++b) {
        double acc_re[4] = {0.0, 0.0, 0.0, 0.0}, acc_im[4] = {0.0, 0.0, 0.0, 0.0};
        if (active) {
            const __nv_bfloat16 *base = keys + (long long)b * sb + 2 * pair0;
            const bool rotating = derope != nullptr && dpair0 < nt;
            int frame_lo = 0, frame_hi = -1;      // token range of the frame whose factors are in `rot`
            float2 rot[4];
            for (int t0 = start + ty; t0 < end; t0 += CV_TY * CV_U) {
                uint4 v[CV_U];
#pragma unroll
                for (int u = 0; u < CV_U; ++u) {
                    const int t = t0 + u * CV_TY;
                    v[u] = t < end ? *reinterpret_cast<const uint4 *>(base + (long long)t * sl) : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < CV_U; ++u) {
                    const int t = t0 + u * CV_TY;
                    if (t < end) {
                        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                        if (rotating && (t < frame_lo || t >= frame_hi)) {      // a new frame: its rotation factors (rare)
                            const int f = min(max(t / frame_seq_length, 0), n_frames - 1);
                            frame_lo = (t / frame_seq_length) * frame_seq_length;
                            frame_hi = frame_lo + frame_seq_length;
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                rot[e] = dpair0 + e < nt ? derope[(long long)f * nt + dpair0 + e] : make_float2(1.f, 0.f);
                        }
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float x = __uint_as_float(w[e] << 16), y = __uint_as_float(w[e] & 0xffff0000u);
                            if (rotating && dpair0 + e < nt) {
                                const float re = __fsub_rn(__fmul_rn(x, rot[e].x), __fmul_rn(y, rot[e].y));
                                const float im = __fadd_rn(__fmul_rn(x, rot[e].y), __fmul_rn(y, rot[e].x));
                                x = bf16_round_f(re);
                                y = bf16_round_f(im);
                            }
                            acc_re[e] += (double)x;
                            acc_im[e] += (double)y;
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            sre[ty][threadIdx.x][e] = acc_re[e];
            sim[ty][threadIdx.x][e] = acc_im[e];
        }
        __syncthreads();
        if (ty == 0 && active) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                double r = 0.0, i = 0.0;
                for (int y = 0; y < CV_TY; ++y) {
                    r += sre[y][threadIdx.x][e];
                    i += sim[y][threadIdx.x][e];
                }
                out_re[e] += (double)(float)(r / (double)max(n_tok, 1));
                out_im[e] += (double)(float)(i / (double)max(n_tok, 1));
            }
        }
        __syncthreads();
    }
    if (ty == 0 && active) {
        float *dst = page_index + (long long)page * H * D + 2 * pair0;
        float o[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            o[2 * e] = (float)(out_re[e] / (double)B);
            o[2 * e + 1] = (float)(out_im[e] / (double)B);
        }
        *reinterpret_cast<float4 *>(dst) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4 *>(dst + 4) = make_float4(o[4], o[5], o[6], o[7]);
    }
}

// ------------------------------------------------------------------------------------------------
// Page scores and top-k.  One CTA per score group (1 = whole vector, H = per head).
// ------------------------------------------------------------------------------------------------
constexpr int ST_THREADS = 256;

__device__ __forceinline__ unsigned long long rank_key(float s, int id) {
    if (s == 0.0f) s = 0.0f;
    uint32_t u = __float_as_uint(s);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)(~u) << 32) | (unsigned)id;   // ascending key = descending score, ascending id
}

__global__ void __launch_bounds__(ST_THREADS)
score_topk_kernel(const float *__restrict__ page_index, const float *__restrict__ query, int P, int G, int Dg,
                  float scale, int topk, float *__restrict__ scores, int32_t *__restrict__ top_ids,
                  float *__restrict__ top_scores, long long query_layer_stride) {
    __shared__ unsigned long long red[ST_THREADS / 32];
    __shared__ unsigned long long prev_s;
    const int g = blockIdx.x;
    {   // blockIdx.y: one page index per layer (`[layers, P, G*Dg]`), outputs `[layers, G, ...]`
        const long long l = blockIdx.y;
        page_index += l * P * G * Dg;
        query += l * query_layer_stride;
        scores += l * G * P;
        if (top_ids) top_ids += l * G * topk;
        if (top_scores) top_scores += l * G * topk;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *q = query + (long long)g * Dg;
    float *sc = scores + (long long)g * P;

    for (int p = warp; p < P; p += ST_THREADS / 32) {
        const float *row = page_index + ((long long)p * G + g) * Dg;
        double acc = 0.0;
        for (int d = lane; d < Dg; d += 32) acc = fma((double)row[d], (double)q[d], acc);
        acc = warp_sum_d(acc);
        if (lane == 0) {
            float s = (float)acc;
            if (scale > 0.f) s = __fdiv_rn(s, scale);
            sc[p] = s;
        }
    }
    __syncthreads();
    if (topk <= 0) return;

    unsigned long long prev = 0ull;
    bool first = true;
    for (int r = 0; r < topk; ++r) {
        unsigned long long best = 0xFFFFFFFFFFFFFFFFull;
        for (int p = threadIdx.x; p < P; p += ST_THREADS) {
            const unsigned long long key = rank_key(sc[p], p);
            if ((first || key > prev) && key < best) best = key;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other < best ? other : best;
        }
        if (lane == 0) red[warp] = best;
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long bb = red[0];
            for (int w = 1; w < ST_THREADS / 32; ++w) bb = red[w] < bb ? red[w] : bb;
            prev_s = bb;
            const long long o = (long long)g * topk + r;
            if (bb != 0xFFFFFFFFFFFFFFFFull) {
                const int id = (int)(bb & 0xFFFFFFFFull);
                top_ids[o] = id;
                top_scores[o] = sc[id];
            } else {
                top_ids[o] = -1;
                top_scores[o] = -INFINITY;
            }
        }
        __syncthreads();
        prev = prev_s;
        first = false;
        if (prev == 0xFFFFFFFFFFFFFFFFull) {
            // fewer than topk pages: fill the tail
            for (int rr = r + 1 + threadIdx.x; rr < topk; rr += ST_THREADS) {
                top_ids[(long long)g * topk + rr] = -1;
                top_scores[(long long)g * topk + rr] = -INFINITY;
            }
            return;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Page install: strided row copy with an optional per-page temporal rotation of the keys.
// grid (token tiles, records).  16-byte vectors when every address allows it.
// ------------------------------------------------------------------------------------------------
constexpr int GP_THREADS = 256;
constexpr int GP_UNROLL = 4;

template <typename T, int VE>   // VE elements per 16-byte vector
__device__ __forceinline__ void rotate_vec(uint4 &raw, int elem0, int head_dim, int nt, const float2 *rot) {
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < VE; i += 2) {
        const int dpair = ((elem0 + i) % head_dim) >> 1;
        if (dpair < nt) {
            const float2 w = rot[dpair];
            float a, c;
            if (sizeof(T) == 2) {
                a = __bfloat162float(reinterpret_cast<__nv_bfloat16 *>(e)[i]);
                c = __bfloat162float(reinterpret_cast<__nv_bfloat16 *>(e)[i + 1]);
            } else {
                a = reinterpret_cast<float *>(e)[i];
                c = reinterpret_cast<float *>(e)[i + 1];
            }
            const float re = __fsub_rn(__fmul_rn(a, w.x), __fmul_rn(c, w.y));
            const float im = __fadd_rn(__fmul_rn(a, w.y), __fmul_rn(c, w.x));
            if (sizeof(T) == 2) {
                reinterpret_cast<__nv_bfloat16 *>(e)[i] = __float2bfloat16_rn(re);
                reinterpret_cast<__nv_bfloat16 *>(e)[i + 1] = __float2bfloat16_rn(im);
            } else {
                reinterpret_cast<float *>(e)[i] = re;
                reinterpret_cast<float *>(e)[i + 1] = im;
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(GP_THREADS)
gather_pages_kernel(const wa_page_copy *__restrict__ copies, int row_elems, int head_dim,
                    const float2 *__restrict__ rotations, int nt) {
    constexpr int VE = 16 / sizeof(T);
    const wa_page_copy rec = copies[blockIdx.y];
    const T *src = reinterpret_cast<const T *>(rec.src);
    T *dst = reinterpret_cast<T *>(rec.dst);
    const float2 *rot = (rec.rot >= 0 && rotations) ? rotations + (long long)rec.rot * nt : nullptr;
    const bool vec_ok = (row_elems % VE == 0) && (rec.src_stride % VE == 0) && (rec.dst_stride % VE == 0) &&
                        (reinterpret_cast<uintptr_t>(src) % 16 == 0) && (reinterpret_cast<uintptr_t>(dst) % 16 == 0) &&
                        (head_dim % VE == 0 || rot == nullptr);
    if (vec_ok) {
        const int vpr = row_elems / VE;
        const long long total = (long long)rec.n_tokens * vpr;
        const long long base = (long long)blockIdx.x * GP_THREADS * GP_UNROLL + threadIdx.x;
        uint4 buf[GP_UNROLL];
        long long tok[GP_UNROLL];
        int c[GP_UNROLL];
#pragma unroll
        for (int u = 0; u < GP_UNROLL; ++u) {
            const long long e = base + (long long)u * GP_THREADS;
            if (e < total) {
                tok[u] = e / vpr;
                c[u] = (int)(e % vpr) * VE;
                buf[u] = *reinterpret_cast<const uint4 *>(src + tok[u] * rec.src_stride + c[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < GP_UNROLL; ++u) {
            const long long e = base + (long long)u * GP_THREADS;
            if (e < total) {
                if (rot) rotate_vec<T, VE>(buf[u], c[u], head_dim, nt, rot);
                *reinterpret_cast<uint4 *>(dst + tok[u] * rec.dst_stride + c[u]) = buf[u];
            }
        }
    } else {
        // element pairs
        const int ppr = row_elems / 2;
        const long long total = (long long)rec.n_tokens * ppr;
        for (int u = 0; u < GP_UNROLL * 4; ++u) {
            const long long e = ((long long)blockIdx.x * GP_UNROLL * 4 + u) * GP_THREADS + threadIdx.x;
            if (e >= total) break;
            const long long t = e / ppr;
            const int col = (int)(e % ppr) * 2;
            float a = load_elem(src, sizeof(T) == 2 ? WA_BF16 : WA_F32, t * rec.src_stride + col);
            float b = load_elem(src, sizeof(T) == 2 ? WA_BF16 : WA_F32, t * rec.src_stride + col + 1);
            const int dpair = (col % head_dim) >> 1;
            if (rot && dpair < nt) {
                const float2 w = rot[dpair];
                const float re = __fsub_rn(__fmul_rn(a, w.x), __fmul_rn(b, w.y));
                const float im = __fadd_rn(__fmul_rn(a, w.y), __fmul_rn(b, w.x));
                a = re;
                b = im;
            }
            store_elem(dst, sizeof(T) == 2 ? WA_BF16 : WA_F32, t * rec.dst_stride + col, a);
            store_elem(dst, sizeof(T) == 2 ? WA_BF16 : WA_F32, t * rec.dst_stride + col + 1, b);
        }
    }
}

}  // namespace wa

using namespace wa;

extern "C" int wa_hkv_page_centroids(const wa_tensor4 *keys, int B, int T, int H, int D, const int32_t *spans,
                                     int P, const float *derope, int n_frames, int n_temporal,
                                     int frame_seq_length, float *page_index, void *stream) {
    const char *what = "wa_hkv_page_centroids";
    WA_REQUIRE(keys && keys->ptr && spans && page_index, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(valid_dtype(keys->dtype), WA_ERR_ARG, "%s: bad dtype", what);
    WA_REQUIRE(B > 0 && T > 0 && H > 0 && D > 0 && P > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    WA_REQUIRE(D % 2 == 0, WA_ERR_UNSUPPORTED, "%s: head_dim must be even", what);
    WA_REQUIRE(!derope || (n_frames > 0 && n_temporal >= 0 && 2 * n_temporal <= D && frame_seq_length > 0),
               WA_ERR_ARG, "%s: bad rotation table arguments", what);
    WA_REQUIRE(P <= 65535, WA_ERR_UNSUPPORTED, "%s: at most 65535 pages per call", what);
    if (keys->dtype == WA_BF16 && keys->stride_h == D && D % 8 == 0 && (uintptr_t)keys->ptr % 16 == 0 && keys->stride_l % 8 == 0 &&
        keys->stride_b % 8 == 0 && (uintptr_t)page_index % 16 == 0) {
        dim3 vgrid(ceil_div(H * D / 2, CV_TX * 4), P), vblock(CV_TX, CV_TY);
        page_centroid_vec_kernel<<<vgrid, vblock, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16 *)keys->ptr, keys->stride_b, keys->stride_l, B, H, D, spans, reinterpret_cast<const float2 *>(derope),
            n_frames, n_temporal, frame_seq_length, page_index);
        return check_launch(what);
    }
    dim3 grid(ceil_div(H * D / 2, CT_TX), P), block(CT_TX, CT_TY);
    page_centroid_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(
        make_view(keys), B, H, D, spans, reinterpret_cast<const float2 *>(derope), n_frames, n_temporal,
        frame_seq_length, page_index);
    return check_launch(what);
}

extern "C" int wa_hkv_score_topk(const float *page_index, const float *query, int P, int G, int Dg, float scale,
                                 int topk, float *scores, int32_t *top_ids, float *top_scores, void *stream) {
    const char *what = "wa_hkv_score_topk";
    WA_REQUIRE(page_index && query && scores, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(topk <= 0 || (top_ids && top_scores), WA_ERR_ARG, "%s: top-k outputs are null", what);
    WA_REQUIRE(P > 0 && G > 0 && Dg > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    score_topk_kernel<<<G, ST_THREADS, 0, (cudaStream_t)stream>>>(page_index, query, P, G, Dg, scale, topk, scores,
                                                                  top_ids, top_scores, 0);
    return check_launch(what);
}

extern "C" int wa_hkv_score_topk_layers(const float *page_index, const float *query, int layers, int P, int G, int Dg,
                                        long long query_layer_stride, float scale, int topk, float *scores,
                                        int32_t *top_ids, float *top_scores, void *stream) {
    const char *what = "wa_hkv_score_topk_layers";
    WA_REQUIRE(page_index && query && scores, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(topk <= 0 || (top_ids && top_scores), WA_ERR_ARG, "%s: top-k outputs are null", what);
    WA_REQUIRE(layers > 0 && P > 0 && G > 0 && Dg > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    WA_REQUIRE(layers <= 65535, WA_ERR_UNSUPPORTED, "%s: at most 65535 layers", what);
    score_topk_kernel<<<dim3(G, layers), ST_THREADS, 0, (cudaStream_t)stream>>>(page_index, query, P, G, Dg, scale, topk, scores,
                                                                               top_ids, top_scores, query_layer_stride);
    return check_launch(what);
}

namespace wa {
// Copy records for the selected pages of every (layer, head) list, built where the ids are: one warp per list sorts
// its ids (chronological = ascending page id; absent ids last) and writes `topk` records.
__global__ void __launch_bounds__(128)
build_records_kernel(const int32_t *__restrict__ top_ids, int n_lists, int heads, int topk, const long long *__restrict__ page_src,
                     int P, long long src_layer_stride, long long src_token_stride, unsigned long long dst_base,
                     long long dst_layer_stride, long long dst_token_stride, int page_tokens, int head_dim, int elem_size,
                     int rotate, wa_page_copy *__restrict__ records, int32_t *__restrict__ missing) {
    const int list = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (list >= n_lists) return;
    const int layer = list / heads, head = list % heads;
    // up to 64 ids per list: two keys per lane, bitonic sort across the warp (absent / out-of-range ids sort last)
    unsigned int key[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = lane + 32 * u;
        int id = r < topk ? top_ids[(long long)list * topk + r] : -1;
        key[u] = (id >= 0 && id < P && page_src[id] != 0) ? (unsigned)id : 0xFFFFFFFFu;
    }
    for (int k = 2; k <= 64; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            const unsigned int a0 = key[0], a1 = key[1];
            // element i = lane + 32 u; its partner i ^ j is the lane's other register when j = 32
            const unsigned int o0 = j == 32 ? a1 : __shfl_xor_sync(0xffffffffu, a0, j);
            const unsigned int o1 = j == 32 ? a0 : __shfl_xor_sync(0xffffffffu, a1, j);
            const bool min0 = ((lane & j) == 0) == ((lane & k) == 0);
            const bool min1 = (((lane + 32) & j) == 0) == (((lane + 32) & k) == 0);
            key[0] = (o0 < a0) == min0 ? o0 : a0;
            key[1] = (o1 < a1) == min1 ? o1 : a1;
        }
    }
    int absent = 0;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int r = lane + 32 * u;
        if (r < topk) {
            wa_page_copy rec;
            const bool present = key[u] != 0xFFFFFFFFu;
            const unsigned long long src = present ? (unsigned long long)page_src[key[u]] : 0ull;
            rec.src = reinterpret_cast<const void *>(src + (unsigned long long)(layer * src_layer_stride) +
                                                     (unsigned long long)head * head_dim * elem_size);
            rec.dst = reinterpret_cast<void *>(dst_base + (unsigned long long)(layer * dst_layer_stride) +
                                               ((unsigned long long)r * page_tokens * dst_token_stride + (unsigned long long)head * head_dim) *
                                                   elem_size);
            rec.src_stride = src_token_stride;
            rec.dst_stride = dst_token_stride;
            rec.n_tokens = present ? page_tokens : 0;
            rec.rot = rotate ? r : -1;
            records[(long long)list * topk + r] = rec;
            absent += present ? 0 : 1;
        }
    }
    if (missing) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) absent += __shfl_xor_sync(0xffffffffu, absent, o);
        if (lane == 0 && absent) atomicAdd(missing, absent);
    }
}
}  // namespace wa

extern "C" int wa_hkv_build_records(const int32_t *top_ids, int layers, int heads, int topk, const long long *page_src, int P,
                                    long long src_layer_stride, long long src_token_stride, void *dst_base,
                                    long long dst_layer_stride, long long dst_token_stride, int page_tokens, int head_dim,
                                    int elem_size, int rotate, wa_page_copy *records, int32_t *missing, void *stream) {
    const char *what = "wa_hkv_build_records";
    WA_REQUIRE(top_ids && page_src && dst_base && records, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(layers > 0 && heads > 0 && topk > 0 && P > 0 && page_tokens > 0 && head_dim > 0, WA_ERR_ARG,
               "%s: sizes must be positive", what);
    WA_REQUIRE(topk <= 64, WA_ERR_UNSUPPORTED, "%s: at most 64 pages per list, got %d", what, topk);
    WA_REQUIRE(elem_size == 2 || elem_size == 4, WA_ERR_ARG, "%s: element size must be 2 or 4", what);
    const long long n_lists = (long long)layers * heads;
    WA_REQUIRE(n_lists < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many lists", what);
    wa::build_records_kernel<<<(unsigned)((n_lists + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
        top_ids, (int)n_lists, heads, topk, page_src, P, src_layer_stride, src_token_stride, (unsigned long long)dst_base,
        dst_layer_stride, dst_token_stride, page_tokens, head_dim, elem_size, rotate, records, missing);
    return check_launch(what);
}

extern "C" int wa_hkv_gather_pages(const wa_page_copy *copies, int n, int max_tokens, int row_elems, int head_dim,
                                   int dtype, const float *rotations, int n_temporal, void *stream) {
    const char *what = "wa_hkv_gather_pages";
    WA_REQUIRE(copies, WA_ERR_ARG, "%s: null record array", what);
    WA_REQUIRE(valid_dtype(dtype), WA_ERR_ARG, "%s: bad dtype", what);
    WA_REQUIRE(n > 0 && max_tokens > 0 && row_elems > 0 && head_dim > 0, WA_ERR_ARG, "%s: sizes must be positive",
               what);
    WA_REQUIRE(row_elems % 2 == 0 && head_dim % 2 == 0 && row_elems % head_dim == 0, WA_ERR_UNSUPPORTED,
               "%s: row_elems must be a multiple of an even head_dim", what);
    WA_REQUIRE(n <= 65535, WA_ERR_UNSUPPORTED, "%s: at most 65535 records per call", what);
    WA_REQUIRE(2 * n_temporal <= head_dim, WA_ERR_ARG, "%s: temporal band wider than head_dim", what);
    const int ve = dtype == WA_BF16 ? 8 : 4;
    // tiles sized for the vector path; the pair path covers 4x as many (smaller) items per CTA
    const long long vecs = (long long)max_tokens * ceil_div(row_elems, ve);
    const long long tiles = (vecs + GP_THREADS * GP_UNROLL - 1) / (GP_THREADS * GP_UNROLL);
    WA_REQUIRE(tiles < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: page too large", what);
    dim3 grid((unsigned)tiles, n);
    if (dtype == WA_BF16)
        gather_pages_kernel<__nv_bfloat16><<<grid, GP_THREADS, 0, (cudaStream_t)stream>>>(
            copies, row_elems, head_dim, reinterpret_cast<const float2 *>(rotations), n_temporal);
    else
        gather_pages_kernel<float><<<grid, GP_THREADS, 0, (cudaStream_t)stream>>>(
            copies, row_elems, head_dim, reinterpret_cast<const float2 *>(rotations), n_temporal);
    return check_launch(what);
}

// Cold-tier promotion: host-to-device copies of pages that live in page-locked host memory, queued on
// `stream` (the caller's side stream) one cudaMemcpyAsync per page -- two-dimensional when the token rows
// of source and destination are not equally spaced.  Nothing is launched and nothing waits here; the
// caller records an event behind the copies and makes the stream of the install kernel wait for it.
extern "C" int wa_hkv_promote_pages(const wa_page_copy *host_records, int n, int row_elems, int elem_size, void *stream) {
    const char *what = "wa_hkv_promote_pages";
    WA_REQUIRE(host_records || n == 0, WA_ERR_ARG, "%s: null record array", what);
    WA_REQUIRE(n >= 0 && row_elems > 0 && (elem_size == 2 || elem_size == 4), WA_ERR_ARG, "%s: bad sizes", what);
    const size_t row_bytes = (size_t)row_elems * elem_size;
    for (int i = 0; i < n; ++i) {
        const wa_page_copy &r = host_records[i];
        if (r.n_tokens <= 0) continue;
        WA_REQUIRE(r.src && r.dst, WA_ERR_ARG, "%s: record %d has a null address", what, i);
        WA_REQUIRE(r.src_stride >= row_elems && r.dst_stride >= row_elems, WA_ERR_ARG,
                   "%s: record %d: token rows overlap (stride below the row length)", what, i);
        cudaError_t e;
        if (r.src_stride == row_elems && r.dst_stride == row_elems)
            e = cudaMemcpyAsync(r.dst, r.src, row_bytes * r.n_tokens, cudaMemcpyHostToDevice, (cudaStream_t)stream);
        else
            e = cudaMemcpy2DAsync(r.dst, (size_t)r.dst_stride * elem_size, r.src, (size_t)r.src_stride * elem_size, row_bytes,
                                  r.n_tokens, cudaMemcpyHostToDevice, (cudaStream_t)stream);
        if (e != cudaSuccess) return fail((int)e, "%s: copy %d of %d: %s", what, i, n, cudaGetErrorString(e));
    }
    return 0;
}
