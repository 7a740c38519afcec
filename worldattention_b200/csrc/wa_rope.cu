// q/k RMSNorm + causal rotary embedding in one pass over the projected tokens.
//
// Stands in for WanRMSNorm (wan/modules/model.py:70-86) followed by causal_rope_apply
// (wan/modules/causal_model.py:34-62), which the reference runs as separate tensor operations with a Python
// loop over samples and a float64 complex copy of q and of k.  Bandwidth-bound: one warp per token reads the
// H*D values (twice; the second read hits L1/L2), writes them once.  Rounding points follow the reference:
// the normalised value and its product with the weight are each stored in the input dtype, the rotation is a
// float64 complex product stored once in the input dtype.
#include "wa_common.cuh"

namespace wa {

constexpr int RN_WARPS = 8;

template <typename T> __device__ __forceinline__ float2 load_pair(const T *p);
template <> __device__ __forceinline__ float2 load_pair<float>(const float *p) { return *reinterpret_cast<const float2 *>(p); }
template <> __device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16 *p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
}
template <typename T> __device__ __forceinline__ float round_to(float x);
template <> __device__ __forceinline__ float round_to<float>(float x) { return x; }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float x) { return bf16_round_f(x); }
template <typename T> __device__ __forceinline__ void store_pair(T *p, double re, double im);
template <> __device__ __forceinline__ void store_pair<float>(float *p, double re, double im) {
    *reinterpret_cast<float2 *>(p) = make_float2((float)re, (float)im);
}
template <> __device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16 *p, double re, double im) {
    __nv_bfloat162 v;
    v.x = __double2bfloat16(re);
    v.y = __double2bfloat16(im);
    *reinterpret_cast<__nv_bfloat162 *>(p) = v;
}

template <typename T>
__global__ void __launch_bounds__(RN_WARPS * 32)
qk_norm_rope_kernel(const T *__restrict__ x, long long xsb, long long xsl, long long xsh, T *__restrict__ out, long long osb,
                    long long osl, long long osh, long long tokens, int L, int H, int D, const void *__restrict__ weight, int wdt,
                    float eps, const double2 *__restrict__ freqs, int freq_rows, int start_frame, const int *__restrict__ start_frame_dev,
                    int grid_h, int grid_w) {
    if (start_frame_dev) start_frame = max(*start_frame_dev, 0);   // the position lives on the device (replayed launches)
    const long long tok = (long long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5);
    if (tok >= tokens) return;
    const int lane = threadIdx.x & 31;
    const int b = (int)(tok / L), t = (int)(tok % L);
    const T *src = x + (long long)b * xsb + (long long)t * xsl;
    T *dst = out + (long long)b * osb + (long long)t * osl;
    const int c = D >> 1, pairs = H * c;

    float scale = 1.0f;
    if (weight) {
        double acc = 0.0;
        for (int p = lane; p < pairs; p += 32) {
            const float2 v = load_pair<T>(src + (long long)(p / c) * xsh + 2 * (p % c));
            acc += (double)v.x * (double)v.x + (double)v.y * (double)v.y;
        }
        acc = warp_sum_d(acc);
        const float mean_sq = (float)(acc / (double)(H * D));
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
    }
    // position of the token in the (frame, row, column) grid; the three bands of a head's pairs take one each
    const int per_frame = grid_h * grid_w;
    const int frame = min(max(start_frame + t / per_frame, 0), freq_rows - 1);
    const int row = min((t / grid_w) % grid_h, freq_rows - 1), col = min(t % grid_w, freq_rows - 1);
    const int ct = c - 2 * (c / 3), ch = c / 3;
    for (int p = lane; p < pairs; p += 32) {
        const int h = p / c, j = p % c;
        float2 v = load_pair<T>(src + (long long)h * xsh + 2 * j);
        if (weight) {
            const float w0 = load_elem(weight, wdt, (long long)h * D + 2 * j), w1 = load_elem(weight, wdt, (long long)h * D + 2 * j + 1);
            v.x = round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(v.x, scale)), w0));
            v.y = round_to<T>(__fmul_rn(round_to<T>(__fmul_rn(v.y, scale)), w1));
        }
        double re = (double)v.x, im = (double)v.y;
        if (freqs) {
            const int pos = j < ct ? frame : (j < ct + ch ? row : col);
            const double2 f = freqs[(long long)pos * c + j];
            const double a = re, bb = im;
            re = a * f.x - bb * f.y;
            im = a * f.y + bb * f.x;
        }
        store_pair<T>(dst + (long long)h * osh + 2 * j, re, im);
    }
}

// bf16 tokens whose heads lie side by side (stride D): the token's H*D values are read ONCE as 16-byte vectors and
// kept in registers (up to 8 vectors per lane: H*D <= 2048).  Same arithmetic per value as the kernel above.
constexpr int RN_MAX_VEC = 8;

__global__ void __launch_bounds__(RN_WARPS * 32)
qk_norm_rope_rows_kernel(const __nv_bfloat16 *__restrict__ x, long long xsb, long long xsl, __nv_bfloat16 *__restrict__ out,
                         long long osb, long long osl, long long tokens, int L, int H, int D, const void *__restrict__ weight, int wdt,
                         float eps, const double2 *__restrict__ freqs, int freq_rows, int start_frame,
                         const int *__restrict__ start_frame_dev, int grid_h, int grid_w) {
    if (start_frame_dev) start_frame = max(*start_frame_dev, 0);
    const long long tok = (long long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5);
    if (tok >= tokens) return;
    const int lane = threadIdx.x & 31;
    const int b = (int)(tok / L), t = (int)(tok % L);
    const uint4 *src = reinterpret_cast<const uint4 *>(x + (long long)b * xsb + (long long)t * xsl);
    uint4 *dst = reinterpret_cast<uint4 *>(out + (long long)b * osb + (long long)t * osl);
    const int nvec = (H * D) >> 3, c = D >> 1;

    uint4 v[RN_MAX_VEC];
    double acc = 0.0;
#pragma unroll
    for (int i = 0; i < RN_MAX_VEC; ++i) {
        const int j = i * 32 + lane;
        if (j < nvec) {
            v[i] = src[j];
            const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const double lo = (double)__uint_as_float(w[e] << 16), hi = (double)__uint_as_float(w[e] & 0xffff0000u);
                acc += lo * lo + hi * hi;
            }
        }
    }
    float scale = 1.0f;
    if (weight) {
        acc = warp_sum_d(acc);
        const float mean_sq = (float)(acc / (double)(H * D));
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean_sq, eps)));
    }
    const int per_frame = grid_h * grid_w;
    const int frame = min(max(start_frame + t / per_frame, 0), freq_rows - 1);
    const int row = min((t / grid_w) % grid_h, freq_rows - 1), col = min(t % grid_w, freq_rows - 1);
    const int ct = c - 2 * (c / 3), ch = c / 3;
#pragma unroll
    for (int i = 0; i < RN_MAX_VEC; ++i) {
        const int j = i * 32 + lane;
        if (j < nvec) {
            const int elem = j << 3, h = elem / D, pair0 = (elem - h * D) >> 1;      // four pairs of one head
            const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int jp = pair0 + e;
                float vx = __uint_as_float(w[e] << 16), vy = __uint_as_float(w[e] & 0xffff0000u);
                if (weight) {
                    const float w0 = load_elem(weight, wdt, (long long)h * D + 2 * jp), w1 = load_elem(weight, wdt, (long long)h * D + 2 * jp + 1);
                    vx = bf16_round_f(__fmul_rn(bf16_round_f(__fmul_rn(vx, scale)), w0));
                    vy = bf16_round_f(__fmul_rn(bf16_round_f(__fmul_rn(vy, scale)), w1));
                }
                double re = (double)vx, im = (double)vy;
                if (freqs) {
                    const int pos = jp < ct ? frame : (jp < ct + ch ? row : col);
                    const double2 f = freqs[(long long)pos * c + jp];
                    const double a = re, bb = im;
                    re = a * f.x - bb * f.y;
                    im = a * f.y + bb * f.x;
                }
                __nv_bfloat162 r;
                r.x = __double2bfloat16(re);
                r.y = __double2bfloat16(im);
                o[e] = *reinterpret_cast<const uint32_t *>(&r);
            }
            dst[j] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

}  // namespace wa

using namespace wa;

static int qk_norm_rope_launch(const wa_tensor4 *x, const wa_tensor4 *out, int B, int L, int H, int D, const void *norm_weight,
                               int weight_dtype, float eps, const double *freqs, int freq_rows, int start_frame,
                               const int *start_frame_dev, int grid_h, int grid_w, void *stream) {
    const char *what = "wa_qk_norm_rope";
    WA_REQUIRE(x && out && x->ptr && out->ptr, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(valid_dtype(x->dtype) && x->dtype == out->dtype, WA_ERR_ARG, "%s: x and out must share a dtype", what);
    WA_REQUIRE(B > 0 && L > 0 && H > 0 && D > 0 && D % 2 == 0, WA_ERR_ARG, "%s: sizes must be positive and head_dim even", what);
    WA_REQUIRE(!norm_weight || valid_dtype(weight_dtype), WA_ERR_ARG, "%s: bad weight dtype", what);
    WA_REQUIRE(!freqs || (freq_rows > 0 && grid_h > 0 && grid_w > 0 && start_frame >= 0), WA_ERR_ARG,
               "%s: a rotation needs a table and a positive grid", what);
    const int align = x->dtype == WA_BF16 ? 4 : 8;
    WA_REQUIRE((uintptr_t)x->ptr % align == 0 && (uintptr_t)out->ptr % align == 0 && x->stride_h % 2 == 0 && x->stride_l % 2 == 0 &&
                   x->stride_b % 2 == 0 && out->stride_h % 2 == 0 && out->stride_l % 2 == 0 && out->stride_b % 2 == 0,
               WA_ERR_ALIGN, "%s: pairs must be naturally aligned (even strides)", what);
    const long long tokens = (long long)B * L;
    const long long blocks = (tokens + RN_WARPS - 1) / RN_WARPS;
    WA_REQUIRE(blocks < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many tokens", what);
    if (!freqs) grid_h = grid_w = 1;
    const bool rows_in_registers = x->dtype == WA_BF16 && x->stride_h == D && out->stride_h == D && D % 8 == 0 &&
                                   (long long)H * D <= 32 * RN_MAX_VEC * 8 && (uintptr_t)x->ptr % 16 == 0 && (uintptr_t)out->ptr % 16 == 0 &&
                                   x->stride_l % 8 == 0 && x->stride_b % 8 == 0 && out->stride_l % 8 == 0 && out->stride_b % 8 == 0;
    if (rows_in_registers)
        qk_norm_rope_rows_kernel<<<(unsigned)blocks, RN_WARPS * 32, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16 *)x->ptr, x->stride_b, x->stride_l, (__nv_bfloat16 *)out->ptr, out->stride_b, out->stride_l, tokens, L, H,
            D, norm_weight, weight_dtype, eps, (const double2 *)freqs, freq_rows, start_frame, start_frame_dev, grid_h, grid_w);
    else if (x->dtype == WA_BF16)
        qk_norm_rope_kernel<__nv_bfloat16><<<(unsigned)blocks, RN_WARPS * 32, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16 *)x->ptr, x->stride_b, x->stride_l, x->stride_h, (__nv_bfloat16 *)out->ptr, out->stride_b,
            out->stride_l, out->stride_h, tokens, L, H, D, norm_weight, weight_dtype, eps, (const double2 *)freqs, freq_rows,
            start_frame, start_frame_dev, grid_h, grid_w);
    else
        qk_norm_rope_kernel<float><<<(unsigned)blocks, RN_WARPS * 32, 0, (cudaStream_t)stream>>>(
            (const float *)x->ptr, x->stride_b, x->stride_l, x->stride_h, (float *)out->ptr, out->stride_b, out->stride_l,
            out->stride_h, tokens, L, H, D, norm_weight, weight_dtype, eps, (const double2 *)freqs, freq_rows, start_frame,
            start_frame_dev, grid_h, grid_w);
    return check_launch(what);
}

extern "C" int wa_qk_norm_rope(const wa_tensor4 *x, const wa_tensor4 *out, int B, int L, int H, int D, const void *norm_weight,
                               int weight_dtype, float eps, const double *freqs, int freq_rows, int start_frame, int grid_h,
                               int grid_w, void *stream) {
    return qk_norm_rope_launch(x, out, B, L, H, D, norm_weight, weight_dtype, eps, freqs, freq_rows, start_frame, nullptr, grid_h,
                               grid_w, stream);
}

extern "C" int wa_qk_norm_rope_at(const wa_tensor4 *x, const wa_tensor4 *out, int B, int L, int H, int D, const void *norm_weight,
                                  int weight_dtype, float eps, const double *freqs, int freq_rows, const int32_t *start_frame_device,
                                  int grid_h, int grid_w, void *stream) {
    WA_REQUIRE(start_frame_device, WA_ERR_ARG, "wa_qk_norm_rope_at: null position pointer");
    return qk_norm_rope_launch(x, out, B, L, H, D, norm_weight, weight_dtype, eps, freqs, freq_rows, 0, start_frame_device, grid_h,
                               grid_w, stream);
}
