// Shape-generic SIMT attention kernels: block-sparse branch, compressed ("linear") branch, gate and
// combine, shard-partial merge.
//
// These accept any head_dim <= 256, any block size, float32 or bf16 tensors in either
// `[B, L, H, D]` or `[B, H, N, D]` layout, and compute in float32.  They serve the shapes the
// tcgen05 kernel does not cover and are the in-library cross-check for it.  Stand-ins for
// wan/modules/hsa/block_sparse_torch.py:16-64 and wan/modules/hsa/attention.py:113-118, 246-259.
#include "wa_common.cuh"

namespace wa {

constexpr int GA_THREADS = 256;
constexpr int GA_WARPS = GA_THREADS / 32;
constexpr int GA_ROWS_PER_WARP = 4;
constexpr int GA_QT = GA_WARPS * GA_ROWS_PER_WARP;  // 32 query rows per CTA
constexpr int GA_TK = 32;                           // key tokens per shared-memory chunk
constexpr int GA_MAXD = 256;
constexpr int GA_DC = GA_MAXD / 32;                 // channels per lane

struct GenericAttnParams {
    View4 q, k, v;
    void *out;
    int out_dtype;
    long long osb, osl, osh;
    int H, Lq, Lkv, D;
    int q_block;    // query rows per routing block
    int q_tile;     // query rows per CTA (<= GA_QT, divides the work inside one routing block)
    int tiles_per_block;
    int kv_block;   // key tokens per block
    int n_kv_blocks;
    int dense;      // 1: visit every key block in order (no index / num)
    const int32_t *index;
    const int32_t *num;
    int index_stride;
    const int32_t *block_sizes;
    int round_in, round_out;
    float scale;
    float *lse;
};

__global__ void __launch_bounds__(GA_THREADS)
generic_attention_kernel(GenericAttnParams p) {
    extern __shared__ float ga_smem[];
    const int D = p.D;
    const int ldk = D + 1;
    float *qs = ga_smem;                 // [GA_QT][D]
    float *ks = qs + GA_QT * D;          // [GA_TK][D + 1]
    float *vs = ks + GA_TK * ldk;        // [GA_TK][D]

    const int qb = blockIdx.x / p.tiles_per_block;
    const int tile = blockIdx.x % p.tiles_per_block;
    const int h = blockIdx.y, b = blockIdx.z;
    const int row0 = qb * p.q_block + tile * p.q_tile;
    const int rows_here = max(0, min(min(p.q_tile, p.q_block - tile * p.q_tile), p.Lq - row0));
    if (rows_here <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // stage the query rows
    const long long qbase = (long long)b * p.q.sb + (long long)h * p.q.sh;
    for (int e = threadIdx.x; e < rows_here * D; e += GA_THREADS) {
        const int r = e / D, d = e % D;
        float x = load_elem(p.q.ptr, p.q.dtype, qbase + (long long)(row0 + r) * p.q.sl + d);
        qs[r * D + d] = p.round_in ? bf16_round_f(x) : x;
    }

    float m_i[GA_ROWS_PER_WARP], l_i[GA_ROWS_PER_WARP], acc[GA_ROWS_PER_WARP][GA_DC];
#pragma unroll
    for (int r = 0; r < GA_ROWS_PER_WARP; ++r) {
        m_i[r] = -INFINITY;
        l_i[r] = 0.f;
#pragma unroll
        for (int c = 0; c < GA_DC; ++c) acc[r][c] = 0.f;
    }

    const long long meta = ((long long)b * p.H + h) * (long long)((p.Lq + p.q_block - 1) / p.q_block) + qb;
    const int n_sel = p.dense ? p.n_kv_blocks : max(0, min(p.num[meta], p.index_stride));
    const int32_t *ids = p.dense ? nullptr : p.index + meta * (long long)p.index_stride;
    const long long kbase = (long long)b * p.k.sb + (long long)h * p.k.sh;
    const long long vbase = (long long)b * p.v.sb + (long long)h * p.v.sh;

    for (int s = 0; s < n_sel; ++s) {
        int id = p.dense ? s : ids[s];
        id = max(0, min(id, p.n_kv_blocks - 1));
        int size = p.block_sizes ? p.block_sizes[id] : p.Lkv - id * p.kv_block;
        size = max(0, min(size, min(p.kv_block, p.Lkv - id * p.kv_block)));
        for (int c0 = 0; c0 < size; c0 += GA_TK) {
            const int n_tok = min(GA_TK, size - c0);
            __syncthreads();
            for (int e = threadIdx.x; e < GA_TK * D; e += GA_THREADS) {
                const int t = e / D, d = e % D;
                float kx = 0.f, vx = 0.f;
                if (t < n_tok) {
                    const long long tok = (long long)id * p.kv_block + c0 + t;
                    kx = load_elem(p.k.ptr, p.k.dtype, kbase + tok * p.k.sl + d);
                    vx = load_elem(p.v.ptr, p.v.dtype, vbase + tok * p.v.sl + d);
                    if (p.round_in) {
                        kx = bf16_round_f(kx);
                        vx = bf16_round_f(vx);
                    }
                }
                ks[t * ldk + d] = kx;
                vs[t * D + d] = vx;
            }
            __syncthreads();

            // scores: lane = key token, four query rows per warp share each K element
            float sc[GA_ROWS_PER_WARP] = {0.f, 0.f, 0.f, 0.f};
            const float *krow = ks + lane * ldk;
            const float *q0 = qs + (warp * GA_ROWS_PER_WARP) * D;
            for (int d = 0; d < D; ++d) {
                const float kx = krow[d];
#pragma unroll
                for (int r = 0; r < GA_ROWS_PER_WARP; ++r) sc[r] = fmaf(q0[r * D + d], kx, sc[r]);
            }
#pragma unroll
            for (int r = 0; r < GA_ROWS_PER_WARP; ++r) {
                const float sv = lane < n_tok ? sc[r] * p.scale : -INFINITY;
                const float m_new = fmaxf(m_i[r], warp_max(sv));
                const float pr = lane < n_tok ? expf(sv - m_new) : 0.f;
                const float alpha = m_i[r] == -INFINITY ? 0.f : expf(m_i[r] - m_new);
                l_i[r] = l_i[r] * alpha + warp_sum(pr);
                m_i[r] = m_new;
#pragma unroll
                for (int c = 0; c < GA_DC; ++c) acc[r][c] *= alpha;
                sc[r] = pr;
            }
            for (int t = 0; t < n_tok; ++t) {
                float pt[GA_ROWS_PER_WARP];
#pragma unroll
                for (int r = 0; r < GA_ROWS_PER_WARP; ++r) pt[r] = __shfl_sync(0xffffffffu, sc[r], t);
#pragma unroll
                for (int c = 0; c < GA_DC; ++c) {
                    const int d = lane + 32 * c;
                    if (d < D) {
                        const float vx = vs[t * D + d];
#pragma unroll
                        for (int r = 0; r < GA_ROWS_PER_WARP; ++r) acc[r][c] = fmaf(pt[r], vx, acc[r][c]);
                    }
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < GA_ROWS_PER_WARP; ++r) {
        const int lr = warp * GA_ROWS_PER_WARP + r;
        if (lr >= rows_here) continue;
        const int row = row0 + lr;
        const float inv = l_i[r] > 0.f ? 1.0f / l_i[r] : 0.f;
        const long long obase = (long long)b * p.osb + (long long)row * p.osl + (long long)h * p.osh;
#pragma unroll
        for (int c = 0; c < GA_DC; ++c) {
            const int d = lane + 32 * c;
            if (d < D) {
                float o = acc[r][c] * inv;
                if (p.round_out) o = bf16_round_f(o);
                store_elem(p.out, p.out_dtype, obase + d, o);
            }
        }
        if (p.lse && lane == 0)
            p.lse[((long long)b * p.H + h) * p.Lq + row] = l_i[r] > 0.f ? m_i[r] + logf(l_i[r]) : -INFINITY;
    }
}

int launch_generic_attention(GenericAttnParams &p, int B, int n_q_blocks, cudaStream_t stream,
                             const char *what) {
    WA_REQUIRE(p.D <= GA_MAXD, WA_ERR_UNSUPPORTED, "%s: head_dim %d > %d", what, p.D, GA_MAXD);
    p.q_tile = p.q_block < GA_QT ? p.q_block : GA_QT;
    p.tiles_per_block = ceil_div(p.q_block, p.q_tile);
    const long long gx = (long long)n_q_blocks * p.tiles_per_block;
    WA_REQUIRE(gx < (1ll << 31) && p.H <= 65535 && B <= 65535, WA_ERR_UNSUPPORTED, "%s: grid too large", what);
    const size_t smem = ((size_t)GA_QT * p.D + (size_t)GA_TK * (p.D + 1) + (size_t)GA_TK * p.D) * sizeof(float);
    static PerDeviceOnce attr_set;
    if (smem > 48 * 1024 && !attr_set.done()) {
        cudaError_t e = cudaFuncSetAttribute(generic_attention_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
        attr_set.mark();
    }
    dim3 grid((unsigned)gx, p.H, B);
    generic_attention_kernel<<<grid, GA_THREADS, smem, stream>>>(p);
    return check_launch(what);
}

// ------------------------------------------------------------------------------------------------
// Gate + combine.  One warp per (batch, token, head) vector.
// ------------------------------------------------------------------------------------------------
constexpr int GC_WARPS = 8;

__global__ void __launch_bounds__(GC_WARPS * 32)
gate_combine_kernel(View4 q, View4 sp, View4 li, void *out, int out_dtype, long long osb, long long osl,
                    long long osh, long long n_vec, int L, int H, int D, const void *gw, const void *gb,
                    int gdt, int round_gate) {
    extern __shared__ float gc_smem[];  // [GC_WARPS][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long vec = (long long)blockIdx.x * GC_WARPS + warp;
    if (vec >= n_vec) return;
    const int h = (int)(vec % H);
    const int l = (int)((vec / H) % L);
    const int b = (int)(vec / ((long long)H * L));
    float *qv = gc_smem + warp * D;
    const long long qoff = (long long)b * q.sb + (long long)l * q.sl + (long long)h * q.sh;
    for (int d = lane; d < D; d += 32) qv[d] = load_elem(q.ptr, q.dtype, qoff + d);
    __syncwarp();
    const long long soff = (long long)b * sp.sb + (long long)l * sp.sl + (long long)h * sp.sh;
    const long long loff = (long long)b * li.sb + (long long)l * li.sl + (long long)h * li.sh;
    const long long ooff = (long long)b * osb + (long long)l * osl + (long long)h * osh;
    for (int e = lane; e < D; e += 32) {
        float z;
        if (gw) {
            z = gb ? load_elem(gb, gdt, e) : 0.f;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(qv[d], load_elem(gw, gdt, (long long)e * D + d), dot);
            z += dot;
        } else {
            z = qv[e];
        }
        float g = 1.0f / (1.0f + expf(-z));
        if (round_gate) g = bf16_round_f(g);
        const float s = load_elem(sp.ptr, sp.dtype, soff + e);
        const float x = load_elem(li.ptr, li.dtype, loff + e);
        store_elem(out, out_dtype, ooff + e, fmaf(x, g, s));
    }
}

// Same operation with the gate weight staged in shared memory (head_dim <= 128): a persistent grid, each
// warp walks over (batch, token, head) vectors, a lane produces outputs lane, lane + 32, ...
constexpr int GS_WARPS = 8;

__global__ void __launch_bounds__(GS_WARPS * 32)
gate_combine_smem_kernel(View4 q, View4 sp, View4 li, void *out, int out_dtype, long long osb, long long osl,
                         long long osh, long long n_vec, int L, int H, int D, const void *gw, const void *gb, int gdt,
                         int round_gate) {
    extern __shared__ float gs_smem[];
    const int ldw = D + 1;
    float *ws = gs_smem;                       // [D][D + 1]
    float *bs = ws + D * ldw;                  // [D]
    float *qv = bs + D + (threadIdx.x >> 5) * D;   // [GS_WARPS][D]
    for (int e = threadIdx.x; e < D * D; e += GS_WARPS * 32) ws[(e / D) * ldw + (e % D)] = load_elem(gw, gdt, e);
    for (int e = threadIdx.x; e < D; e += GS_WARPS * 32) bs[e] = gb ? load_elem(gb, gdt, e) : 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const long long stride = (long long)gridDim.x * GS_WARPS;
    for (long long vec = (long long)blockIdx.x * GS_WARPS + (threadIdx.x >> 5); vec < n_vec; vec += stride) {
        const int h = (int)(vec % H);
        const int l = (int)((vec / H) % L);
        const int b = (int)(vec / ((long long)H * L));
        const long long qoff = (long long)b * q.sb + (long long)l * q.sl + (long long)h * q.sh;
        __syncwarp();
        for (int d = lane; d < D; d += 32) qv[d] = load_elem(q.ptr, q.dtype, qoff + d);
        __syncwarp();
        const long long soff = (long long)b * sp.sb + (long long)l * sp.sl + (long long)h * sp.sh;
        const long long loff = (long long)b * li.sb + (long long)l * li.sl + (long long)h * li.sh;
        const long long ooff = (long long)b * osb + (long long)l * osl + (long long)h * osh;
        for (int e = lane; e < D; e += 32) {
            float z = bs[e];
            const float *w = ws + e * ldw;
            for (int d = 0; d < D; ++d) z = fmaf(qv[d], w[d], z);
            float g = 1.0f / (1.0f + expf(-z));
            if (round_gate) g = bf16_round_f(g);
            store_elem(out, out_dtype, ooff + e,
                       fmaf(load_elem(li.ptr, li.dtype, loff + e), g, load_elem(sp.ptr, sp.dtype, soff + e)));
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Merge shard partials of one softmax branch.
// ------------------------------------------------------------------------------------------------
__global__ void merge_partials_kernel(const float *__restrict__ outs, const float *__restrict__ lses, int G,
                                      long long rows, int D, float *__restrict__ out, float *__restrict__ lse) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float m = -INFINITY;
    for (int g = 0; g < G; ++g) m = fmaxf(m, lses[(long long)g * rows + row]);
    const float m_safe = m == -INFINITY ? 0.f : m;
    float total = 0.f;
    for (int g = 0; g < G; ++g) total += expf(lses[(long long)g * rows + row] - m_safe);
    const float inv = total > 0.f ? 1.0f / total : 0.f;
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int g = 0; g < G; ++g) {
            const float w = expf(lses[(long long)g * rows + row] - m_safe) * inv;
            acc = fmaf(w, outs[((long long)g * rows + row) * D + d], acc);
        }
        out[row * D + d] = acc;
    }
    if (lse && lane == 0) lse[row] = total > 0.f ? m_safe + logf(total) : -INFINITY;
}

// Merge of packed shard partials.  A record is [sparse (D) | linear (D) | lse_sparse, lse_linear, pad, pad] floats; `recv`
// holds G x vectors of them (shard-major).  One warp per (token, head) vector: per branch out = sum_g e^(lse_g - LSE) O_g,
// the sparse branch rounded to bf16 (the reference stores it so), the linear one kept in float32.
__global__ void __launch_bounds__(256)
merge_packed_kernel(const float *__restrict__ recv, int G, long long vectors, int D, int record,
                    __nv_bfloat16 *__restrict__ sparse_out, float *__restrict__ linear_out) {
    const long long vec = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (vec >= vectors) return;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int branch = 0; branch < 2; ++branch) {
        float m = -INFINITY;
        for (int g = 0; g < G; ++g) m = fmaxf(m, __ldg(recv + ((long long)g * vectors + vec) * record + 2 * D + branch));
        const float m_safe = m == -INFINITY ? 0.f : m;
        float total = 0.f;
        for (int g = 0; g < G; ++g) total += expf(__ldg(recv + ((long long)g * vectors + vec) * record + 2 * D + branch) - m_safe);
        const float inv = total > 0.f ? 1.0f / total : 0.f;
        for (int d = lane * 4; d < D; d += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int g = 0; g < G; ++g) {
                const float *rec = recv + ((long long)g * vectors + vec) * record;
                const float w = expf(__ldg(rec + 2 * D + branch) - m_safe) * inv;
                const float4 o = __ldg(reinterpret_cast<const float4 *>(rec + branch * D + d));
                acc.x = fmaf(w, o.x, acc.x); acc.y = fmaf(w, o.y, acc.y); acc.z = fmaf(w, o.z, acc.z); acc.w = fmaf(w, o.w, acc.w);
            }
            if (branch == 0) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
                uint2 packed = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
                *reinterpret_cast<uint2 *>(sparse_out + vec * D + d) = packed;
            } else {
                *reinterpret_cast<float4 *>(linear_out + vec * D + d) = acc;
            }
        }
    }
}

static int check_view(const wa_tensor4 *t, const char *what, const char *name) {
    WA_REQUIRE(t && t->ptr, WA_ERR_ARG, "%s: %s is null", what, name);
    WA_REQUIRE(valid_dtype(t->dtype), WA_ERR_ARG, "%s: %s has bad dtype %d", what, name, t->dtype);
    return 0;
}

}  // namespace wa

using namespace wa;

extern "C" int wa_block_sparse_forward(const wa_tensor4 *q, const wa_tensor4 *k, const wa_tensor4 *v,
                                       const wa_tensor4 *out, int B, int H, int Lq, int Lkv, int D,
                                       int block_size, const int32_t *index, const int32_t *num,
                                       int index_stride, const int32_t *block_sizes, int round_inputs_bf16,
                                       int round_output_bf16, float *lse, void *stream) {
    const char *what = "wa_block_sparse_forward";
    int rc;
    if ((rc = check_view(q, what, "q")) || (rc = check_view(k, what, "k")) || (rc = check_view(v, what, "v")) ||
        (rc = check_view(out, what, "out")))
        return rc;
    WA_REQUIRE(index && num, WA_ERR_ARG, "%s: index / num is null", what);
    WA_REQUIRE(B > 0 && H > 0 && Lq > 0 && Lkv > 0 && D > 0 && block_size > 0 && index_stride > 0, WA_ERR_ARG,
               "%s: sizes must be positive", what);
    GenericAttnParams p{};
    p.q = make_view(q); p.k = make_view(k); p.v = make_view(v);
    p.out = out->ptr; p.out_dtype = out->dtype; p.osb = out->stride_b; p.osl = out->stride_l; p.osh = out->stride_h;
    p.H = H; p.Lq = Lq; p.Lkv = Lkv; p.D = D;
    p.q_block = block_size; p.kv_block = block_size; p.n_kv_blocks = ceil_div(Lkv, block_size);
    p.dense = 0; p.index = index; p.num = num; p.index_stride = index_stride; p.block_sizes = block_sizes;
    p.round_in = round_inputs_bf16; p.round_out = round_output_bf16;
    p.scale = (float)(1.0 / sqrt((double)D));
    p.lse = lse;
    return launch_generic_attention(p, B, ceil_div(Lq, block_size), (cudaStream_t)stream, what);
}

extern "C" int wa_linear_branch(const wa_tensor4 *q, const wa_tensor4 *k_coarse, const wa_tensor4 *v_coarse,
                                const wa_tensor4 *out, int B, int H, int Lq, int Lc, int D,
                                int round_output_bf16, float *lse, void *stream) {
    const char *what = "wa_linear_branch";
    int rc;
    if ((rc = check_view(q, what, "q")) || (rc = check_view(k_coarse, what, "k_coarse")) ||
        (rc = check_view(v_coarse, what, "v_coarse")) || (rc = check_view(out, what, "out")))
        return rc;
    WA_REQUIRE(B > 0 && H > 0 && Lq > 0 && Lc > 0 && D > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    GenericAttnParams p{};
    p.q = make_view(q); p.k = make_view(k_coarse); p.v = make_view(v_coarse);
    p.out = out->ptr; p.out_dtype = out->dtype; p.osb = out->stride_b; p.osl = out->stride_l; p.osh = out->stride_h;
    p.H = H; p.Lq = Lq; p.Lkv = Lc; p.D = D;
    p.q_block = GA_QT; p.kv_block = GA_TK; p.n_kv_blocks = ceil_div(Lc, GA_TK);
    p.dense = 1; p.index = nullptr; p.num = nullptr; p.index_stride = 1; p.block_sizes = nullptr;
    p.round_in = 0; p.round_out = round_output_bf16;
    p.scale = (float)pow((double)D, -0.5);
    p.lse = lse;
    return launch_generic_attention(p, B, ceil_div(Lq, GA_QT), (cudaStream_t)stream, what);
}

extern "C" int wa_gate_combine(const wa_tensor4 *q, const wa_tensor4 *sparse, const wa_tensor4 *linear,
                               const wa_tensor4 *out, int B, int L, int H, int D, const void *gate_w,
                               const void *gate_b, int gate_dtype, int round_gate_bf16, void *stream) {
    const char *what = "wa_gate_combine";
    int rc;
    if ((rc = check_view(q, what, "q")) || (rc = check_view(sparse, what, "sparse")) ||
        (rc = check_view(linear, what, "linear")) || (rc = check_view(out, what, "out")))
        return rc;
    WA_REQUIRE(B > 0 && L > 0 && H > 0 && D > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    WA_REQUIRE(!gate_w || valid_dtype(gate_dtype), WA_ERR_ARG, "%s: bad gate dtype", what);
    const long long n_vec = (long long)B * L * H;
    const long long blocks = (n_vec + GC_WARPS - 1) / GC_WARPS;
    WA_REQUIRE(blocks < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many tokens", what);
    if (gate_w && D <= 128) {
        const size_t smem2 = ((size_t)D * (D + 1) + D + (size_t)GS_WARPS * D) * sizeof(float);
        static PerDeviceOnce attr_set;
        if (smem2 > 48 * 1024 && !attr_set.done()) {
            cudaError_t e = cudaFuncSetAttribute(gate_combine_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)(((size_t)128 * 129 + 128 + GS_WARPS * 128) * sizeof(float)));
            if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
            attr_set.mark();
        }
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long want = (n_vec + GS_WARPS - 1) / GS_WARPS;
        const unsigned grid = (unsigned)(want < 2ll * sms ? want : 2ll * sms);
        gate_combine_smem_kernel<<<grid, GS_WARPS * 32, smem2, (cudaStream_t)stream>>>(
            make_view(q), make_view(sparse), make_view(linear), out->ptr, out->dtype, out->stride_b, out->stride_l,
            out->stride_h, n_vec, L, H, D, gate_w, gate_b, gate_dtype, round_gate_bf16);
        return check_launch(what);
    }
    const size_t smem = (size_t)GC_WARPS * D * sizeof(float);
    WA_REQUIRE(smem <= 48 * 1024, WA_ERR_UNSUPPORTED, "%s: head_dim %d too large", what, D);
    gate_combine_kernel<<<(unsigned)blocks, GC_WARPS * 32, smem, (cudaStream_t)stream>>>(
        make_view(q), make_view(sparse), make_view(linear), out->ptr, out->dtype, out->stride_b, out->stride_l,
        out->stride_h, n_vec, L, H, D, gate_w, gate_b, gate_dtype, round_gate_bf16);
    return check_launch(what);
}

extern "C" int wa_merge_partials(const float *outs, const float *lses, int G, int64_t rows, int D, float *out,
                                 float *lse, void *stream) {
    WA_REQUIRE(outs && lses && out, WA_ERR_ARG, "wa_merge_partials: null pointer");
    WA_REQUIRE(G > 0 && rows > 0 && D > 0, WA_ERR_ARG, "wa_merge_partials: sizes must be positive");
    const int warps = 8;
    const long long blocks = (rows + warps - 1) / warps;
    WA_REQUIRE(blocks < (1ll << 31), WA_ERR_UNSUPPORTED, "wa_merge_partials: too many rows");
    merge_partials_kernel<<<(unsigned)blocks, warps * 32, 0, (cudaStream_t)stream>>>(outs, lses, G, rows, D, out,
                                                                                     lse);
    return check_launch("wa_merge_partials");
}

extern "C" int wa_merge_packed(const float *recv, int G, int64_t vectors, int D, int record, void *sparse_out, float *linear_out,
                               void *stream) {
    const char *what = "wa_merge_packed";
    WA_REQUIRE(recv && sparse_out && linear_out, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(G > 0 && vectors > 0 && D > 0, WA_ERR_ARG, "%s: sizes must be positive", what);
    WA_REQUIRE(D % 4 == 0 && record % 4 == 0 && record >= 2 * D + 2, WA_ERR_ARG,
               "%s: D and the record length must be multiples of 4 and a record must hold two vectors and two normalisers", what);
    WA_REQUIRE(((uintptr_t)recv | (uintptr_t)linear_out) % 16 == 0 && (uintptr_t)sparse_out % 8 == 0, WA_ERR_ALIGN,
               "%s: buffers must be 16-byte aligned", what);
    const int warps = 8;
    const long long blocks = (vectors + warps - 1) / warps;
    WA_REQUIRE(blocks < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many vectors", what);
    merge_packed_kernel<<<(unsigned)blocks, warps * 32, 0, (cudaStream_t)stream>>>(recv, G, vectors, D, record,
                                                                                   (__nv_bfloat16 *)sparse_out, linear_out);
    return check_launch(what);
}
