// The element-wise steps around the attention layer in a DiT block, one pass each (bf16 rows).
//
// WanAttentionBlock.forward (wan/modules/causal_model.py:586-659) wraps its three sub-layers in
//     norm(x).unflatten(frames, tokens) * (1 + e_scale) + e_shift          and          x + y.unflatten(...) * e_gate
// where WanLayerNorm (wan/modules/model.py:89-103) computes in float32 and casts back.  Written with tensor
// expressions that is about twelve passes over the activations per sub-layer (casts, broadcasts, temporaries); here it is
// one read and one write.  The reference's rounding points are kept: the normalised value is rounded to bf16, so are
// 1 + e_scale, the product and the sum, and y * e_gate before the residual addition.
#include "wa_common.cuh"

namespace wa {

constexpr int GLUE_WARPS = 8;
constexpr int GLUE_MAX_VEC = 16;   // 16-byte vectors per lane: rows of up to 32 * 16 * 8 = 4096 bf16

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ void unpack8(const uint4 &v, float *f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint4 pack8(const float *f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t *>(&p);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// One warp per row.  out = bf16(bf16(bf16(LN(x) [* w + b]) * bf16(1 + scale[f])) + shift[f]); scale / shift are per
// (batch, frame) vectors `[.., C]` with a row stride of `mod_stride` elements, or null.
__global__ void __launch_bounds__(GLUE_WARPS * 32)
ln_modulate_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ out, long long rows, int C, float eps,
                   const __nv_bfloat16 *__restrict__ weight, const __nv_bfloat16 *__restrict__ bias,
                   const __nv_bfloat16 *__restrict__ scale, const __nv_bfloat16 *__restrict__ shift, long long mod_stride,
                   int tokens_per_frame) {
    const long long row = (long long)blockIdx.x * GLUE_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31, nvec = C >> 3;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + row * C);
    uint4 v[GLUE_MAX_VEC];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; ++i) {
        const int j = i * 32 + lane;
        if (j < nvec) {
            v[i] = src[j];
            float f[8];
            unpack8(v[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += f[e];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / (float)C;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; ++i) {
        const int j = i * 32 + lane;
        if (j < nvec) {
            float f[8];
            unpack8(v[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) sq += (f[e] - mean) * (f[e] - mean);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / (float)C + eps);
    const long long frame = row / tokens_per_frame;
    const uint4 *wv = reinterpret_cast<const uint4 *>(weight), *bv = reinterpret_cast<const uint4 *>(bias);
    const uint4 *sc = scale ? reinterpret_cast<const uint4 *>(scale + frame * mod_stride) : nullptr;
    const uint4 *sh = shift ? reinterpret_cast<const uint4 *>(shift + frame * mod_stride) : nullptr;
    uint4 *dst = reinterpret_cast<uint4 *>(out + row * C);
#pragma unroll
    for (int i = 0; i < GLUE_MAX_VEC; ++i) {
        const int j = i * 32 + lane;
        if (j < nvec) {
            float f[8], a[8];
            unpack8(v[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = (f[e] - mean) * rstd;
            if (wv) {
                unpack8(wv[j], a);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] *= a[e];
            }
            if (bv) {
                unpack8(bv[j], a);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += a[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = bf16r(f[e]);
            if (sc) {
                unpack8(sc[j], a);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = bf16r(f[e] * bf16r(1.f + a[e]));
            }
            if (sh) {
                unpack8(sh[j], a);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] += a[e];
            }
            dst[j] = pack8(f);
        }
    }
}

// out = bf16(x + bf16(y * gate[f])) (gate null: out = bf16(x + y)); eight elements per thread.
__global__ void __launch_bounds__(256)
gated_residual_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ y, __nv_bfloat16 *__restrict__ out,
                      long long rows, int C, const __nv_bfloat16 *__restrict__ gate, long long mod_stride, int tokens_per_frame) {
    const int nvec = C >> 3;
    const long long total = rows * nvec;
    for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
        const long long row = t / nvec;
        const int j = (int)(t - row * nvec);
        float a[8], b[8], g[8];
        unpack8(reinterpret_cast<const uint4 *>(x)[t], a);
        unpack8(reinterpret_cast<const uint4 *>(y)[t], b);
        if (gate) {
            unpack8(reinterpret_cast<const uint4 *>(gate + (row / tokens_per_frame) * mod_stride)[j], g);
#pragma unroll
            for (int e = 0; e < 8; ++e) b[e] = bf16r(b[e] * g[e]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += b[e];
        reinterpret_cast<uint4 *>(out)[t] = pack8(a);
    }
}

static bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace wa

using namespace wa;

extern "C" int wa_ln_modulate(const void *x, void *out, long long rows, int C, float eps, const void *weight, const void *bias,
                              const void *scale, const void *shift, long long mod_stride, int tokens_per_frame, void *stream) {
    const char *what = "wa_ln_modulate";
    WA_REQUIRE(x && out, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(rows >= 0 && C > 0 && tokens_per_frame > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    WA_REQUIRE(C % 8 == 0 && C <= 32 * GLUE_MAX_VEC * 8, WA_ERR_UNSUPPORTED, "%s: row length must be a multiple of 8 and at most %d, got %d",
               what, 32 * GLUE_MAX_VEC * 8, C);
    WA_REQUIRE(aligned16(x) && aligned16(out) && aligned16(weight) && aligned16(bias) && aligned16(scale) && aligned16(shift) &&
                   mod_stride % 8 == 0,
               WA_ERR_ALIGN, "%s: pointers must be 16-byte aligned and the modulation stride a multiple of 8 elements", what);
    if (rows == 0) return 0;
    const long long ctas = (rows + GLUE_WARPS - 1) / GLUE_WARPS;
    WA_REQUIRE(ctas < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many rows", what);
    ln_modulate_kernel<<<(unsigned)ctas, GLUE_WARPS * 32, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16 *)x, (__nv_bfloat16 *)out, rows, C, eps, (const __nv_bfloat16 *)weight, (const __nv_bfloat16 *)bias,
        (const __nv_bfloat16 *)scale, (const __nv_bfloat16 *)shift, mod_stride, tokens_per_frame);
    return check_launch(what);
}

extern "C" int wa_gated_residual(const void *x, const void *y, void *out, long long rows, int C, const void *gate,
                                 long long mod_stride, int tokens_per_frame, void *stream) {
    const char *what = "wa_gated_residual";
    WA_REQUIRE(x && y && out, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(rows >= 0 && C > 0 && tokens_per_frame > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    WA_REQUIRE(C % 8 == 0, WA_ERR_UNSUPPORTED, "%s: row length must be a multiple of 8, got %d", what, C);
    WA_REQUIRE(aligned16(x) && aligned16(y) && aligned16(out) && aligned16(gate) && mod_stride % 8 == 0, WA_ERR_ALIGN,
               "%s: pointers must be 16-byte aligned and the modulation stride a multiple of 8 elements", what);
    if (rows == 0) return 0;
    const long long vecs = rows * (C / 8);
    long long ctas = (vecs + 255) / 256;
    if (ctas > 148 * 16) ctas = 148 * 16;
    gated_residual_kernel<<<(unsigned)ctas, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, (const __nv_bfloat16 *)y,
                                                                             (__nv_bfloat16 *)out, rows, C, (const __nv_bfloat16 *)gate,
                                                                             mod_stride, tokens_per_frame);
    return check_launch(what);
}
