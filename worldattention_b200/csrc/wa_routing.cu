// HSA block routing on the GPU: block-mean pooling, block attention map, Gini-adaptive selection.
//
// Stands in for wan/modules/hsa/routing.py.  The work is bandwidth- and latency-bound (one read
// of Q and K, then a few hundred short rows), so the kernels are plain coalesced / warp-shuffle
// code; every reduction that feeds the discrete selection accumulates in float64 and rounds once,
// which makes the chosen block ids independent of the summation order.
#include "wa_common.cuh"

namespace wa {

// ------------------------------------------------------------------------------------------------
// Pooling.  One CTA per (batch, block, head): block_size token rows of D contiguous elements.
// ------------------------------------------------------------------------------------------------
constexpr int POOL_THREADS = 256;

template <bool VEC_BF16>
__global__ void __launch_bounds__(POOL_THREADS)
pool_blocks_kernel(View4 x, int L, int H, int D, int block_size, int num_blocks, int aligned,
                   float *__restrict__ pooled, View4 x2, int L2, int num_blocks2, int aligned2,
                   float *__restrict__ pooled2) {
    int nb = blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    if (nb >= num_blocks) {   // second tensor (keys) pooled by the same launch
        nb -= num_blocks;
        x = x2; L = L2; num_blocks = num_blocks2; aligned = aligned2; pooled = pooled2;
    }
    const int t0 = nb * block_size;
    const int n_real = min(block_size, L - t0);
    extern __shared__ double pool_smem[];  // [rows_in_flight][D]

    const long long base = (long long)b * x.sb + (long long)h * x.sh;
    float *dst = pooled + (((long long)b * H + h) * num_blocks + nb) * (long long)D;

    if (VEC_BF16) {
        // 8 bf16 per thread per token; lanes_per_row threads cover one token row.
        const int lanes_per_row = D >> 3;
        const int rows = POOL_THREADS / lanes_per_row;
        const int lane = threadIdx.x % lanes_per_row, row = threadIdx.x / lanes_per_row;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (row < rows) {
            const __nv_bfloat16 *p = (const __nv_bfloat16 *)x.ptr + base + lane * 8;
            for (int t = row; t < n_real; t += rows) {
                uint4 raw = *reinterpret_cast<const uint4 *>(p + (long long)(t0 + t) * x.sl);
                const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 f = __bfloat1622float2(h2[i]);
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            }
        }
        float *sm = reinterpret_cast<float *>(pool_smem);  // [rows][D]
        if (row < rows) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sm[row * D + lane * 8 + i] = acc[i];
        }
        __syncthreads();
        for (int d = threadIdx.x; d < D; d += POOL_THREADS) {
            float s = 0.f;
            for (int r = 0; r < rows; ++r) s += sm[r * D + d];  // fixed order
            float out;
            if (aligned) out = bf16_round_f((float)((double)s / (double)block_size));
            else out = __fdiv_rn(bf16_round_f(s), (float)n_real);
            dst[d] = out;
        }
    } else {
        // generic: thread per channel (strided), float64 accumulation.
        const int rows = max(1, POOL_THREADS / D);
        const int per_row = min(D, POOL_THREADS);
        const int row = threadIdx.x / per_row, lane = threadIdx.x % per_row;
        for (int d0 = 0; d0 < D; d0 += per_row) {
            const int d = d0 + lane;
            double acc = 0.0;
            if (row < rows && d < D) {
                for (int t = row; t < n_real; t += rows)
                    acc += (double)load_elem(x.ptr, x.dtype, base + (long long)(t0 + t) * x.sl + d);
                pool_smem[row * per_row + lane] = acc;
            }
            __syncthreads();
            if (row == 0 && d < D) {
                double s = 0.0;
                for (int r = 0; r < rows; ++r) s += pool_smem[r * per_row + lane];
                float out;
                if (aligned) {
                    out = (float)(s / (double)block_size);
                    if (x.dtype == WA_BF16) out = bf16_round_f(out);
                } else {
                    float sum32 = (float)s;
                    if (x.dtype == WA_BF16) sum32 = bf16_round_f(sum32);
                    out = __fdiv_rn(sum32, (float)n_real);
                }
                dst[d] = out;
            }
            __syncthreads();
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Block attention map.  One CTA per (b, h, query block) row; a warp per key block for the dot.
// ------------------------------------------------------------------------------------------------
constexpr int SCORE_THREADS = 256;

__global__ void __launch_bounds__(SCORE_THREADS)
route_scores_kernel(const float *__restrict__ qp, const float *__restrict__ kp, int Nq, int Nkv,
                    int D, float scale, float *__restrict__ attn) {
    const long long row = blockIdx.x;  // (b*H + h)*Nq + i
    const long long bh = row / Nq;
    const float *q = qp + row * D;
    const float *k = kp + bh * (long long)Nkv * D;
    float *out = attn + row * Nkv;
    __shared__ double red[SCORE_THREADS / 32];
    __shared__ float bcast;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = SCORE_THREADS / 32;
    for (int j0 = warp * 4; j0 < Nkv; j0 += nwarps * 4) {   // four independent dot products in flight
        double acc[4] = {0.0, 0.0, 0.0, 0.0};
        for (int d = lane; d < D; d += 32) {
            const double qd = (double)q[d];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (j0 + u < Nkv) acc[u] = fma(qd, (double)k[(long long)(j0 + u) * D + d], acc[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const double t = warp_sum_d(acc[u]);
            if (lane == 0 && j0 + u < Nkv) out[j0 + u] = __fmul_rn((float)t, scale);
        }
    }
    __syncthreads();

    float m = -INFINITY;
    for (int j = threadIdx.x; j < Nkv; j += SCORE_THREADS) m = fmaxf(m, out[j]);
    m = warp_max(m);
    if (lane == 0) red[warp] = (double)m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < nwarps; ++w) mm = fmaxf(mm, (float)red[w]);
        bcast = mm;
    }
    __syncthreads();
    m = bcast;
    __syncthreads();

    double s = 0.0;
    for (int j = threadIdx.x; j < Nkv; j += SCORE_THREADS) {
        float e = (float)exp((double)__fsub_rn(out[j], m));
        out[j] = e;
        s += (double)e;
    }
    s = warp_sum_d(s);
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < nwarps; ++w) t += red[w];
        bcast = (float)t;
    }
    __syncthreads();
    const float denom = bcast;
    for (int j = threadIdx.x; j < Nkv; j += SCORE_THREADS) out[j] = __fdiv_rn(out[j], denom);
}

// ------------------------------------------------------------------------------------------------
// Selection, pass A: per row, sort (probability descending, id ascending) and the row's Gini term.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t descending_key(float p) {
    if (p == 0.0f) p = 0.0f;  // -0 -> +0
    uint32_t u = __float_as_uint(p);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending-orderable
    return ~u;                                        // descending
}

__global__ void route_sort_kernel(const float *__restrict__ attn, int Nkv, int n_pow2,
                                  int32_t *__restrict__ index, float *__restrict__ gini_rows) {
    extern __shared__ unsigned long long keys[];  // n_pow2
    __shared__ double red[32];
    const long long row = blockIdx.x;
    const float *p = attn + row * Nkv;
    const int T = blockDim.x;

    for (int j = threadIdx.x; j < n_pow2; j += T)
        keys[j] = j < Nkv ? (((unsigned long long)descending_key(p[j]) << 32) | (unsigned)j)
                          : 0xFFFFFFFFFFFFFFFFull;
    __syncthreads();
    for (int k = 2; k <= n_pow2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n_pow2; i += T) {
                const int ixj = i ^ j;
                if (ixj > i) {
                    const unsigned long long a = keys[i], b = keys[ixj];
                    const bool up = (i & k) == 0;
                    if ((a > b) == up) {
                        keys[i] = b;
                        keys[ixj] = a;
                    }
                }
            }
            __syncthreads();
        }
    }
    // index + Gini: sum_m fp32((N + 1 - 2m) * p_(m)), m 1-based, accumulated in float64.
    int32_t *idx = index + row * Nkv;
    double acc = 0.0;
    for (int m = threadIdx.x; m < Nkv; m += T) {
        const int id = (int)(keys[m] & 0xFFFFFFFFull);
        idx[m] = id;
        const float w = __fsub_rn((float)(Nkv + 1), __fmul_rn(2.0f, (float)(m + 1)));
        acc += (double)__fmul_rn(w, p[id]);
    }
    acc = warp_sum_d(acc);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < (T + 31) / 32; ++w) t += red[w];
        gini_rows[row] = __fdiv_rn((float)t, (float)Nkv);
    }
}

// ------------------------------------------------------------------------------------------------
// Selection, pass B: per-head threshold, float64 cumulative mass, count (and optional mask).
// ------------------------------------------------------------------------------------------------
constexpr int SELECT_THREADS = 256;

__global__ void __launch_bounds__(SELECT_THREADS)
route_count_kernel(const float *__restrict__ attn, const int32_t *__restrict__ index,
                   const float *__restrict__ gini_rows, int B, int H, int Nq, int Nkv,
                   float tau_min, float tau_span, const int32_t *__restrict__ fixed_num,
                   int32_t *__restrict__ num, uint8_t *__restrict__ mask,
                   float *__restrict__ thresholds) {
    const long long row = blockIdx.x;
    const int i = (int)(row % Nq);
    const int h = (int)((row / Nq) % H);
    const int b = (int)(row / ((long long)Nq * H));
    __shared__ double part[SELECT_THREADS];
    __shared__ float thr_s;
    __shared__ int cnt_s;

    // threshold of this head: mean of the Gini rows over (batch, query block)
    double g = 0.0;
    const int count = B * Nq;
    for (int r = threadIdx.x; r < count; r += SELECT_THREADS) {
        const int bb = r / Nq, ii = r % Nq;
        g += (double)gini_rows[((long long)bb * H + h) * Nq + ii];
    }
    part[threadIdx.x] = g;
    if (threadIdx.x == 0) cnt_s = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < SELECT_THREADS; ++w) t += part[w];
        const float head_gini = (float)(t / (double)count);
        const float thr = __fadd_rn(tau_min, __fmul_rn(head_gini, tau_span));
        thr_s = thr;
        if (b == 0 && i == 0) thresholds[h] = thr;
    }
    __syncthreads();
    const float thr = thr_s;
    const float *p = attn + row * Nkv;
    const int32_t *idx = index + row * Nkv;
    uint8_t *mrow = mask ? mask + row * Nkv : nullptr;

    if (fixed_num) {
        const int n = max(0, min(fixed_num[h], Nkv));
        if (threadIdx.x == 0) num[row] = n;
        if (mrow)
            for (int m = threadIdx.x; m < Nkv; m += SELECT_THREADS) mrow[idx[m]] = m < n;
        return;
    }

    // contiguous chunk per thread, float64 running sums, exclusive scan of the chunk totals
    const int chunk = (Nkv + SELECT_THREADS - 1) / SELECT_THREADS;
    const int m0 = threadIdx.x * chunk, m1 = min(Nkv, m0 + chunk);
    double local = 0.0;
    for (int m = m0; m < m1; ++m) local += (double)p[idx[m]];
    __syncthreads();
    part[threadIdx.x] = local;
    __syncthreads();
    double offset = 0.0;
    for (int w = 0; w < threadIdx.x; ++w) offset += part[w];  // fixed order prefix
    int kept = 0;
    double run = offset;
    for (int m = m0; m < m1; ++m) {
        const float pm = p[idx[m]];
        run += (double)pm;
        const bool keep = __fsub_rn((float)run, pm) < thr;
        kept += keep;
        if (mrow) mrow[idx[m]] = keep;
    }
    if (kept) atomicAdd(&cnt_s, kept);
    __syncthreads();
    if (threadIdx.x == 0) num[row] = cnt_s;
}

// ------------------------------------------------------------------------------------------------
// Mask -> ascending index list.  One warp per row, ballot-ordered compaction.
// ------------------------------------------------------------------------------------------------
__global__ void map_to_index_kernel(const uint8_t *__restrict__ mask, long long rows, int Nkv,
                                    int32_t *__restrict__ index, int32_t *__restrict__ num) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint8_t *m = mask + row * Nkv;
    int32_t *idx = index + row * Nkv;
    int n = 0;
    for (int j0 = 0; j0 < Nkv; j0 += 32) {
        const int j = j0 + lane;
        const bool on = j < Nkv && m[j] != 0;
        const unsigned bal = __ballot_sync(0xffffffffu, on);
        if (on) idx[n + __popc(bal & ((1u << lane) - 1u))] = j;
        n += __popc(bal);
    }
    for (int j = n + lane; j < Nkv; j += 32) idx[j] = -1;
    if (lane == 0) num[row] = n;
}

}  // namespace wa

using namespace wa;

namespace wa {
static bool pool_vec_ok(const wa_tensor4 *x, int D) {
    return x->dtype == WA_BF16 && D % 8 == 0 && D / 8 <= POOL_THREADS && ((uintptr_t)x->ptr % 16 == 0) &&
           x->stride_b % 8 == 0 && x->stride_l % 8 == 0 && x->stride_h % 8 == 0;
}

// Pools `x` (and, when given, `y`, e.g. queries and keys of one forward) in a single launch.
int pool_launch(const wa_tensor4 *x, int Lx, float *px, const wa_tensor4 *y, int Ly, float *py, int B, int H, int D,
                int block_size, cudaStream_t stream) {
    const int nbx = ceil_div(Lx, block_size), nby = y ? ceil_div(Ly, block_size) : 0;
    View4 vx = make_view(x), vy = y ? make_view(y) : vx;
    dim3 grid(nbx + nby, H, B);
    const bool vec = pool_vec_ok(x, D) && (!y || pool_vec_ok(y, D));
    if (vec) {
        const int rows = POOL_THREADS / (D / 8);
        const size_t smem = (size_t)rows * D * sizeof(float);
        WA_REQUIRE(smem <= 48 * 1024, WA_ERR_UNSUPPORTED, "wa_pool_blocks: D=%d too large", D);
        pool_blocks_kernel<true><<<grid, POOL_THREADS, smem, stream>>>(vx, Lx, H, D, block_size, nbx, Lx % block_size == 0,
                                                                       px, vy, Ly, nby, y ? Ly % block_size == 0 : 0, py);
    } else {
        const int rows = D >= POOL_THREADS ? 1 : POOL_THREADS / D;
        const size_t smem = (size_t)rows * (D < POOL_THREADS ? D : POOL_THREADS) * sizeof(double);
        pool_blocks_kernel<false><<<grid, POOL_THREADS, smem, stream>>>(vx, Lx, H, D, block_size, nbx, Lx % block_size == 0,
                                                                        px, vy, Ly, nby, y ? Ly % block_size == 0 : 0, py);
    }
    return check_launch("wa_pool_blocks");
}
}  // namespace wa

extern "C" int wa_pool_blocks(const wa_tensor4 *x, int B, int L, int H, int D, int block_size,
                              float *pooled, void *stream) {
    WA_REQUIRE(x && x->ptr && pooled, WA_ERR_ARG, "wa_pool_blocks: null pointer");
    WA_REQUIRE(valid_dtype(x->dtype), WA_ERR_ARG, "wa_pool_blocks: bad dtype %d", x->dtype);
    WA_REQUIRE(B > 0 && L > 0 && H > 0 && D > 0 && block_size > 0, WA_ERR_ARG,
               "wa_pool_blocks: sizes must be positive (B=%d L=%d H=%d D=%d block=%d)", B, L, H, D,
               block_size);
    WA_REQUIRE(H <= 65535 && B <= 65535, WA_ERR_UNSUPPORTED, "wa_pool_blocks: B, H must be <= 65535");
    return pool_launch(x, L, pooled, nullptr, 0, nullptr, B, H, D, block_size, (cudaStream_t)stream);
}

extern "C" int wa_route_scores(const float *q_pooled, const float *k_pooled, int B, int H, int Nq,
                               int Nkv, int D, float *block_attn, void *stream) {
    WA_REQUIRE(q_pooled && k_pooled && block_attn, WA_ERR_ARG, "wa_route_scores: null pointer");
    WA_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nkv > 0 && D > 0, WA_ERR_ARG,
               "wa_route_scores: sizes must be positive");
    const long long rows = (long long)B * H * Nq;
    WA_REQUIRE(rows < (1ll << 31), WA_ERR_UNSUPPORTED, "wa_route_scores: too many rows");
    const float scale = (float)pow((double)D, -0.5);
    route_scores_kernel<<<(unsigned)rows, SCORE_THREADS, 0, (cudaStream_t)stream>>>(
        q_pooled, k_pooled, Nq, Nkv, D, scale, block_attn);
    return check_launch("wa_route_scores");
}

namespace wa {
int route_select_launch(const float *block_attn, int B, int H, int Nq, int Nkv, double tau_min,
                        double tau_max, const int32_t *fixed_num_per_head, int32_t *index,
                        int32_t *num, uint8_t *mask, float *thresholds, float *gini_scratch,
                        cudaStream_t stream) {
    int n_pow2 = 1;
    while (n_pow2 < Nkv) n_pow2 <<= 1;
    WA_REQUIRE(n_pow2 <= 16384, WA_ERR_UNSUPPORTED,
               "wa_route_select: at most 16384 key blocks per row, got %d", Nkv);
    const long long rows = (long long)B * H * Nq;
    WA_REQUIRE(rows < (1ll << 31), WA_ERR_UNSUPPORTED, "wa_route_select: too many rows");
    const size_t smem = (size_t)n_pow2 * sizeof(unsigned long long);
    int threads = n_pow2 / 2;
    threads = threads < 32 ? 32 : (threads > 1024 ? 1024 : threads);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(route_sort_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "wa_route_select: %s", cudaGetErrorString(e));
    }
    route_sort_kernel<<<(unsigned)rows, threads, smem, stream>>>(block_attn, Nkv, n_pow2, index,
                                                                 gini_scratch);
    int rc = check_launch("wa_route_select(sort)");
    if (rc) return rc;
    route_count_kernel<<<(unsigned)rows, SELECT_THREADS, 0, stream>>>(
        block_attn, index, gini_scratch, B, H, Nq, Nkv, (float)tau_min, (float)(tau_max - tau_min),
        fixed_num_per_head, num, mask, thresholds);
    return check_launch("wa_route_select(count)");
}
}  // namespace wa

extern "C" int wa_route_select(const float *block_attn, int B, int H, int Nq, int Nkv,
                               double tau_min, double tau_max, const int32_t *fixed_num_per_head,
                               int32_t *index, int32_t *num, uint8_t *mask, float *thresholds,
                               float *gini_scratch, void *stream) {
    WA_REQUIRE(block_attn && index && num && thresholds && gini_scratch, WA_ERR_ARG,
               "wa_route_select: null pointer");
    WA_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nkv > 0, WA_ERR_ARG,
               "wa_route_select: sizes must be positive");
    return route_select_launch(block_attn, B, H, Nq, Nkv, tau_min, tau_max, fixed_num_per_head,
                               index, num, mask, thresholds, gini_scratch, (cudaStream_t)stream);
}

extern "C" int wa_map_to_index(const uint8_t *mask, int B, int H, int Nq, int Nkv, int32_t *index,
                               int32_t *num, void *stream) {
    WA_REQUIRE(mask && index && num, WA_ERR_ARG, "wa_map_to_index: null pointer");
    WA_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nkv > 0, WA_ERR_ARG,
               "wa_map_to_index: sizes must be positive");
    const long long rows = (long long)B * H * Nq;
    const int warps = 4;
    map_to_index_kernel<<<(unsigned)((rows + warps - 1) / warps), warps * 32, 0,
                          (cudaStream_t)stream>>>(mask, rows, Nkv, index, num);
    return check_launch("wa_map_to_index");
}

// ------------------------------------------------------------------------------------------------
// wa_route_select_static: the same selection with its per-row scratch inside the library.
//
// For callers that are not allowed to allocate device memory at the point where routing runs: a
// serving process that hands out its whole HBM budget at start-up and forbids later allocation, a
// plugin whose host owns the allocator, or a loop that must not call anything that can synchronise
// the device (cudaMalloc / cudaFree do).  Such a caller has nowhere to get the B*H*Nq floats of
// Gini scratch from, so this entry point keeps them in a file-scope device array of fixed size.
// Every GPU that loads the library carries that array (256 KiB) until the process exits.
// ------------------------------------------------------------------------------------------------
namespace wa {
constexpr int STATIC_SELECT_MAX_ROWS = WA_ROUTE_SELECT_STATIC_MAX_ROWS;
static __device__ __align__(256) float g_select_scratch[STATIC_SELECT_MAX_ROWS];

// The array's name is only a host-side handle; the device address comes from the runtime, once
// per device, with that device current.
static float *select_scratch_address() {
    constexpr int MAX_DEVICES = 64;
    static float *cached[MAX_DEVICES] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        fail(WA_ERR_DEVICE, "wa_route_select_static: no usable current device");
        return nullptr;
    }
    if (!cached[dev]) {
        float *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_select_scratch);
        if (e != cudaSuccess || !ptr) {
            fail((int)e, "wa_route_select_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev] = ptr;
    }
    return cached[dev];
}
}  // namespace wa

extern "C" int wa_route_select_static(const float *block_attn, int B, int H, int Nq, int Nkv, double tau_min,
                                      double tau_max, const int32_t *fixed_num_per_head, int32_t *index,
                                      int32_t *num, uint8_t *mask, float *thresholds, void *stream) {
    WA_REQUIRE(block_attn && index && num && thresholds, WA_ERR_ARG, "wa_route_select_static: null pointer");
    WA_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nkv > 0, WA_ERR_ARG, "wa_route_select_static: sizes must be positive");
    const long long rows = (long long)B * H * Nq;
    WA_REQUIRE(rows <= STATIC_SELECT_MAX_ROWS, WA_ERR_UNSUPPORTED,
               "wa_route_select_static: %lld rows (B*H*Nq) exceed the built-in scratch of %d rows; "
               "use wa_route_select with caller-provided scratch",
               rows, STATIC_SELECT_MAX_ROWS);
    float *scratch = select_scratch_address();
    if (!scratch) return WA_ERR_DEVICE;
    // Nothing in the scratch has to start at zero: pass A writes every row's Gini term before pass B reads it.
    return route_select_launch(block_attn, B, H, Nq, Nkv, tau_min, tau_max, fixed_num_per_head, index, num, mask,
                               thresholds, scratch, (cudaStream_t)stream);
}
