// HSA block routing on the GPU: block-mean pooling, block attention map, Gini-adaptive selection.
//
// Stands in for wan/modules/hsa/routing.py.  The work is bandwidth- and latency-bound (one read
// of Q and K, then a few hundred short rows), so the kernels are plain coalesced / warp-shuffle
// code; every reduction that feeds the discrete selection accumulates in float64 and rounds once,
// which makes the chosen block ids independent of the summation order.
#include "wa_internal.cuh"

namespace wa {

// ------------------------------------------------------------------------------------------------
// Pooling.  One CTA per (batch, block, head): block_size token rows of D contiguous elements.
// ------------------------------------------------------------------------------------------------
constexpr int POOL_THREADS = 256;

template <bool VEC_BF16>
__global__ void __launch_bounds__(POOL_THREADS)
pool_blocks_kernel(View4 x, int L, int H, int D, int block_size, int num_blocks, int aligned,
                   float *__restrict__ pooled, View4 x2, int L2, int num_blocks2, int aligned2,
                   float *__restrict__ pooled2, int out_blocks2, int *__restrict__ zero, int n_zero) {
    int nb = blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    if (n_zero && nb == 0 && h == 0 && b == 0)   // counters of the kernel that follows on the stream
        for (int i = threadIdx.x; i < n_zero; i += POOL_THREADS) zero[i] = 0;
    int out_blocks = num_blocks;   // rows per (batch, head) of the output buffer
    if (nb >= num_blocks) {   // second tensor (keys) pooled by the same launch
        nb -= num_blocks;
        x = x2; L = L2; num_blocks = num_blocks2; aligned = aligned2; pooled = pooled2; out_blocks = out_blocks2;
    }
    const int t0 = nb * block_size;
    const int n_real = min(block_size, L - t0);
    extern __shared__ double pool_smem[];  // [rows_in_flight][D]

    const long long base = (long long)b * x.sb + (long long)h * x.sh;
    float *dst = pooled + (((long long)b * H + h) * out_blocks + nb) * (long long)D;

    if (VEC_BF16) {
        // 8 bf16 per thread per token; lanes_per_row threads cover one token row.
        const int lanes_per_row = D >> 3;
        const int rows = POOL_THREADS / lanes_per_row;
        const int lane = threadIdx.x % lanes_per_row, row = threadIdx.x / lanes_per_row;
        double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};   // float64: exact for a block of bf16 values, so order-free
        if (row < rows) {
            const __nv_bfloat16 *p = (const __nv_bfloat16 *)x.ptr + base + lane * 8;
            // eight row loads in flight per thread; rows past the end contribute zeros
            for (int t = row; t < n_real; t += 8 * rows) {
                uint4 raw[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int tt = t + u * rows;
                    raw[u] = tt < n_real ? *reinterpret_cast<const uint4 *>(p + (long long)(t0 + tt) * x.sl)
                                         : make_uint4(0u, 0u, 0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&raw[u]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float2 f = __bfloat1622float2(h2[i]);
                        acc[2 * i] += (double)f.x;
                        acc[2 * i + 1] += (double)f.y;
                    }
                }
            }
        }
        double *sm = pool_smem;  // [rows][D]
        if (row < rows) {
#pragma unroll
            for (int i = 0; i < 8; ++i) sm[row * D + lane * 8 + i] = acc[i];
        }
        __syncthreads();
        for (int d = threadIdx.x; d < D; d += POOL_THREADS) {
            double s = 0.0;
            for (int r = 0; r < rows; ++r) s += sm[r * D + d];
            float out;
            if (aligned) out = bf16_round_f((float)(s / (double)block_size));
            else out = __fdiv_rn(bf16_round_f((float)s), (float)n_real);
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
// Pooling, streaming form for bf16 rows of 8..256 channels (a power of two): SPLIT warps per (batch,
// block, head), no block-level synchronisation on the load path.  The D/8 lanes that cover one token
// row form a group; the groups of the item's warps take token rows round-robin.  Every lane keeps
// UNROLL 16-byte row loads in flight and issues the next batch before it consumes the current one.
// Sums are float64: a sum of a few hundred bf16 values is exact there, so the result does not depend
// on the order of the additions (the routing decision downstream is discrete).
// ------------------------------------------------------------------------------------------------
#ifndef WA_POOL_SPLIT
#define WA_POOL_SPLIT 2
#endif
#ifndef WA_POOL_UNROLL
#define WA_POOL_UNROLL 4
#endif

#ifndef WA_POOL_MIN_CTAS
#define WA_POOL_MIN_CTAS 3
#endif

template <int UNROLL, int SPLIT>
__global__ void __launch_bounds__(POOL_THREADS, WA_POOL_MIN_CTAS)
pool_warp_kernel(View4 x, int L, int H, int D, int block_size, int num_blocks, int aligned, float *__restrict__ pooled,
                 View4 x2, int L2, int num_blocks2, int aligned2, float *__restrict__ pooled2, int out_blocks2, int B,
                 int *__restrict__ zero, int n_zero) {
    constexpr int ITEMS_PER_CTA = POOL_THREADS / 32 / SPLIT;
    __shared__ double partial[ITEMS_PER_CTA][SPLIT > 1 ? SPLIT - 1 : 1][256];   // [item][warp - 1][channel]
    if (n_zero && blockIdx.x == 0)   // counters of the kernel that follows on the stream
        for (int i = threadIdx.x; i < n_zero; i += POOL_THREADS) zero[i] = 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = warp / SPLIT, part = warp % SPLIT;   // item of this CTA, this warp's share of its rows
    long long item = (long long)blockIdx.x * ITEMS_PER_CTA + slot;   // ((b, block), head), head fastest
    const long long items1 = (long long)B * num_blocks * H;
    int out_blocks = num_blocks;   // rows per (batch, head) of the output buffer
    bool live = true;
    if (item >= items1) {   // second tensor (keys) pooled by the same launch
        item -= items1;
        live = item < (long long)B * num_blocks2 * H;
        x = x2; L = L2; num_blocks = num_blocks2; aligned = aligned2; pooled = pooled2; out_blocks = out_blocks2;
    }
    if (!live) item = 0;   // keeps the CTA's barrier below unconditional; nothing is stored
    const int h = (int)(item % H);
    const int nb = (int)((item / H) % num_blocks);
    const int b = (int)(item / ((long long)H * num_blocks));
    const int t0 = nb * block_size;
    const int n_real = live ? min(block_size, L - t0) : 0;
    const int lanes_per_row = D >> 3, groups = 32 / lanes_per_row;
    const int col = (lane % lanes_per_row) * 8, group = lane / lanes_per_row;
    const int stride = groups * SPLIT;               // token rows between two loads of one lane
    const __nv_bfloat16 *p = (const __nv_bfloat16 *)x.ptr + (long long)b * x.sb + (long long)h * x.sh +
                             (long long)t0 * x.sl + col;
    double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    uint4 cur[UNROLL], nxt[UNROLL];
    auto fetch = [&](uint4 (&dst)[UNROLL], int t) {
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int tt = t + u * stride;
            dst[u] = tt < n_real ? __ldg(reinterpret_cast<const uint4 *>(p + (long long)tt * x.sl)) : make_uint4(0u, 0u, 0u, 0u);
        }
    };
    const int first = part * groups + group;
    fetch(cur, first);
    for (int t = first; t < n_real; t += UNROLL * stride) {
        fetch(nxt, t + UNROLL * stride);   // rows past the end load nothing
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&cur[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(h2[i]);
                acc[2 * i] += (double)f.x;
                acc[2 * i + 1] += (double)f.y;
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) cur[u] = nxt[u];
    }
    // the groups of a warp, then the warps of the item
    for (int step = lanes_per_row; step < 32; step <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], step);
    }
    if (SPLIT > 1) {
        if (part > 0 && group == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) partial[slot][part - 1][col + i] = acc[i];
        }
        __syncthreads();
        if (part == 0 && group == 0) {
#pragma unroll
            for (int w = 0; w < SPLIT - 1; ++w)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += partial[slot][w][col + i];
        }
    }
    if (live && part == 0 && group == 0) {
        float out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            out[i] = aligned ? bf16_round_f((float)(acc[i] / (double)block_size))
                             : __fdiv_rn(bf16_round_f((float)acc[i]), (float)n_real);
        float4 *dst = reinterpret_cast<float4 *>(pooled + (((long long)b * H + h) * out_blocks + nb) * (long long)D + col);
        dst[0] = make_float4(out[0], out[1], out[2], out[3]);
        dst[1] = make_float4(out[4], out[5], out[6], out[7]);
    }
}

// ------------------------------------------------------------------------------------------------
// Block attention map.  One CTA per (b, h, query block) row; a warp per key block for the dot.
// ------------------------------------------------------------------------------------------------
constexpr int SCORE_THREADS = 256;

#ifdef WA_ROUTE_TRACE   // tuning aid: per-CTA phase timestamps (ns) of the fused routing kernel
__device__ long long g_route_trace[4096 * 12];
#define ROUTE_STAMP(i)                                                                         \
    do {                                                                                       \
        if (threadIdx.x == 0 && blockIdx.x < 4096) {                                           \
            long long t_;                                                                      \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                            \
            g_route_trace[blockIdx.x * 12 + (i)] = t_;                                          \
        }                                                                                      \
    } while (0)
#else
#define ROUTE_STAMP(i)
#endif

// One row of logits: out[j] = fl32(q . k_j) * scale, the dot accumulated in float64 and rounded once.  `out` may be
// shared or global memory.  Called by every thread of the CTA; no barrier at the end.
__device__ __forceinline__ void row_logits(const float *__restrict__ q, const float *__restrict__ k, int Nkv, int D, float scale,
                                           float *out) {
    const int T = blockDim.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = T >> 5;
    const bool vec = (D & 3) == 0;
    for (int j0 = warp * 8; j0 < Nkv; j0 += nwarps * 8) {   // eight independent dot products in flight
        double acc[8] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
        if (vec) {
            for (int d = lane * 4; d < D; d += 128) {
                const float4 qv = *reinterpret_cast<const float4 *>(q + d);
                float4 kv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    kv[u] = j0 + u < Nkv ? *reinterpret_cast<const float4 *>(k + (long long)(j0 + u) * D + d)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    acc[u] = fma((double)qv.x, (double)kv[u].x, acc[u]);
                    acc[u] = fma((double)qv.y, (double)kv[u].y, acc[u]);
                    acc[u] = fma((double)qv.z, (double)kv[u].z, acc[u]);
                    acc[u] = fma((double)qv.w, (double)kv[u].w, acc[u]);
                }
            }
        } else {
            for (int d = lane; d < D; d += 32) {
                const double qd = (double)q[d];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (j0 + u < Nkv) acc[u] = fma(qd, (double)k[(long long)(j0 + u) * D + d], acc[u]);
            }
        }
        // transposed reduction: halve the number of live sums at each of the first three exchange steps,
        // so the eight 32-lane sums cost 9 exchanges instead of 40; lane l ends with dot (l >> 2) & 7
        const bool b16 = lane & 16, b8 = lane & 8, b4 = lane & 4;
        double r4[4], r2[2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const double keep = b16 ? acc[u + 4] : acc[u], give = b16 ? acc[u] : acc[u + 4];
            r4[u] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const double keep = b8 ? r4[u + 2] : r4[u], give = b8 ? r4[u] : r4[u + 2];
            r2[u] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
        }
        double t = (b4 ? r2[1] : r2[0]) + __shfl_xor_sync(0xffffffffu, b4 ? r2[0] : r2[1], 4);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        const int u = (lane >> 2) & 7;
        if ((lane & 3) == 0 && j0 + u < Nkv) out[j0 + u] = __fmul_rn((float)t, scale);
    }
}

// Softmax of one row of logits in place: float64 sum, each value rounded once to float32.  `out` may be shared or global
// memory; `red` holds >= 32 doubles.  Called by every thread of the CTA after the logits are complete (and a barrier).
__device__ __forceinline__ void row_softmax(int Nkv, float *out, double *red, float *bcast) {
    const int T = blockDim.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = T >> 5;
    float m = -INFINITY;
    for (int j = threadIdx.x; j < Nkv; j += T) m = fmaxf(m, out[j]);
    m = warp_max(m);
    if (lane == 0) red[warp] = (double)m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float mm = -INFINITY;
        for (int w = 0; w < nwarps; ++w) mm = fmaxf(mm, (float)red[w]);
        *bcast = mm;
    }
    __syncthreads();
    m = *bcast;
    __syncthreads();

    double s = 0.0;
    for (int j = threadIdx.x; j < Nkv; j += T) {
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
        *bcast = (float)t;
    }
    __syncthreads();
    const float denom = *bcast;
    for (int j = threadIdx.x; j < Nkv; j += T) out[j] = __fdiv_rn(out[j], denom);
    __syncthreads();
}

// One row: out[j] = softmax_j(q . k_j * scale) with float64 dots and sums, each rounded once to float32.
__device__ __forceinline__ void row_block_attention(const float *__restrict__ q, const float *__restrict__ k, int Nkv, int D,
                                                    float scale, float *out, double *red, float *bcast) {
    row_logits(q, k, Nkv, D, scale, out);
    __syncthreads();
    ROUTE_STAMP(1);
    row_softmax(Nkv, out, red, bcast);
}

// Logits of R neighbouring rows of one head against ONE pass over the head's pooled keys (D = 128 only): with thousands
// of key blocks a row's CTA otherwise re-reads megabytes of pooled keys that its neighbours read too and converts each to
// float64 again.  A lane owns a key: the keys are staged through `stage` (shared memory, 2 tiles of `tile_keys` rows)
// TRANSPOSED in 16-byte pieces ([piece][key] with an odd pitch, filled one tile ahead through registers: coalesced reads,
// conflict-free writes), so that a warp reads the same piece of 32 keys without bank conflicts, converts it once and uses
// it for all R rows, whose float64 queries come from
// shared memory as broadcasts.  No sum crosses a lane; a dot is accumulated dimension by dimension in float64 and rounded
// once, like every other sum on the routing path.  Measured at 11 700 key blocks (one group = its rows x 11 700 keys):
// see the numbers in the design notes.  Other forms that were built and measured: each key split over all 32 lanes with the queries
// in registers (no transposition, but most instructions go into the transposed float64 reduction: 284 us for four rows);
// a key per 4 lanes with a quarter of the dimensions each, so that all 16 warps compute (the query reads are then four
// different addresses per load instead of one broadcast: 220 us + 56 us per row); the rows spread over four warp groups
// so that all 16 warps compute whole keys (each key converted four times: 25-40 us slower).  What is left of the fixed
// part is the keys' way from L2: every group streams its head's 6 MB, 720 MB for the 120 groups of config 5.  `q` holds the
// rows 128 apart, `out` holds them `Nkv` apart; rows >= nrows repeat row 0's query and are not stored.
template <int R>
__device__ __forceinline__ void row_logits_keys(const float *__restrict__ q, int nrows, const float *__restrict__ k, int Nkv,
                                                float scale, float *out, double *qsh, float4 *stage, int tile_keys) {
    constexpr int D = 128, VPK = D / 4;   // 16-byte pieces per key
    const int T = blockDim.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < R * D; i += T) qsh[i] = (double)q[((i / D) < nrows ? (i / D) : 0) * D + (i % D)];
    const float4 *kvec = reinterpret_cast<const float4 *>(k);
    const int pitch = tile_keys + 1;                  // 16-byte slots per piece row: the odd pitch spreads a key's 32 pieces over the banks
    const int tile_vecs = tile_keys * VPK, tile_slots = pitch * VPK;
    const int n_tiles = (Nkv + tile_keys - 1) / tile_keys;
    // a warp loads one key's 512 bytes per instruction (coalesced) into registers while the previous tile is computed on,
    // and stores them transposed afterwards (16-byte asynchronous copies were measured at about 16 bytes per clock per SM,
    // which made the staging, not the arithmetic, the larger part of this routine)
    constexpr int PER_THREAD = 8;      // 16-byte loads per thread and tile: tile_keys * 32 <= 8 * 512
    float4 pre[PER_THREAD];
    auto fetch = [&](int tile) {
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int v = i * T + threadIdx.x, key = v / VPK, piece = v % VPK;
            const long long gkey = (long long)tile * tile_keys + key;
            pre[i] = (v < tile_vecs && gkey < Nkv) ? __ldg(kvec + gkey * VPK + piece) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto park = [&](int tile) {
        float4 *dst = stage + (tile & 1) * tile_slots;
#pragma unroll
        for (int i = 0; i < PER_THREAD; ++i) {
            const int v = i * T + threadIdx.x, key = v / VPK, piece = v % VPK;
            if (v < tile_vecs) dst[piece * pitch + key] = pre[i];
        }
    };
    fetch(0);
    park(0);
    __syncthreads();
    for (int tile = 0; tile < n_tiles; ++tile) {
        if (tile + 1 < n_tiles) fetch(tile + 1);
        const int key = warp * 32 + lane;      // a lane owns a key of the tile: the first tile_keys / 32 warps compute, all warps fetch
        const long long gkey = (long long)tile * tile_keys + key;
        if (key < tile_keys && (long long)tile * tile_keys + warp * 32 < Nkv) {
            const float4 *kt = stage + (tile & 1) * tile_slots + key;
            double acc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = 0.0;
#pragma unroll 4
            for (int piece = 0; piece < VPK; ++piece) {
                const float4 kv = kt[piece * pitch];
                const double k0 = (double)kv.x, k1 = (double)kv.y, k2 = (double)kv.z, k3 = (double)kv.w;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const double2 qa = *reinterpret_cast<const double2 *>(qsh + r * D + piece * 4);      // broadcast reads
                    const double2 qb = *reinterpret_cast<const double2 *>(qsh + r * D + piece * 4 + 2);
                    double a = fma(qa.x, k0, acc[r]);
                    a = fma(qa.y, k1, a);
                    a = fma(qb.x, k2, a);
                    acc[r] = fma(qb.y, k3, a);
                }
            }
            if (gkey < Nkv) {
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (r < nrows) out[(long long)r * Nkv + gkey] = __fmul_rn((float)acc[r], scale);
            }
        }
        if (tile + 1 < n_tiles) park(tile + 1);      // that buffer was last read while tile - 1 was computed, before the last barrier
        __syncthreads();      // (after the last tile: the logits are complete and visible to the whole CTA, the staging memory is free)
    }
}

__global__ void __launch_bounds__(SCORE_THREADS)
route_scores_kernel(const float *__restrict__ qp, const float *__restrict__ kp, int Nq, int Nkv,
                    int D, float scale, float *__restrict__ attn) {
    const long long row = blockIdx.x;  // (b*H + h)*Nq + i
    const long long bh = row / Nq;
    __shared__ double red[32];
    __shared__ float bcast;
    row_block_attention(qp + row * D, kp + bh * (long long)Nkv * D, Nkv, D, scale, attn + row * Nkv, red, &bcast);
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

// Mean of a head's Gini rows over (batch, query block) -> the head's cumulative-mass threshold.  256 strided
// float64 partials, a shuffle tree inside each warp, the eight warp totals added in order.  Called by every
// thread of a CTA of >= 256 threads; `red` holds >= 8 doubles; the result is valid in every thread.
__device__ __forceinline__ float head_threshold(const float *gini_rows, int B, int H, int Nq, int h, float tau_min,
                                                float tau_span, double *red, float *bcast) {
    const int count = B * Nq, tid = threadIdx.x;
    if (tid < 256) {
        double g = 0.0;
        for (int r = tid; r < count; r += 256) {
            const int bb = r / Nq, ii = r % Nq;
            g += (double)__ldcg(&gini_rows[((long long)bb * H + h) * Nq + ii]);
        }
        g = warp_sum_d(g);
        if ((tid & 31) == 0) red[tid >> 5] = g;
    }
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < 8; ++w) t += red[w];
        const float head_gini = (float)(t / (double)count);
        *bcast = __fadd_rn(tau_min, __fmul_rn(head_gini, tau_span));
    }
    __syncthreads();
    return *bcast;
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

    if (threadIdx.x == 0) cnt_s = 0;
    const float thr = head_threshold(gini_rows, B, H, Nq, h, tau_min, tau_span, part, &thr_s);
    if (threadIdx.x == 0 && b == 0 && i == 0) thresholds[h] = thr;
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
// The forward's routing in ONE launch.  Each CTA owns a (batch, head, query block) row: scores,
// softmax, sort and the row's Gini term, with the probabilities kept in shared memory.  The CTA that
// finishes a head last (a counter per head) turns the head's Gini rows into its threshold and counts
// every row of that head, a warp per row over the sorted probabilities; the CTA that finishes the
// last head prepares the attention kernel's launch (work order, counters).  Same arithmetic as the
// three separate kernels above; no CTA ever waits for another.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void sort_keys_smem(unsigned long long *keys, int n_pow2);

// The k best blocks of a row, in order, WITHOUT sorting the row: for a fixed per-head count over thousands of key blocks
// the full bitonic sort (105 passes over 16384 keys) was two thirds of the routing kernel.  Keys are the sort's own
// 64-bit keys (descending probability, then ascending id; all distinct).  A most-significant-byte-first radix select
// narrows down the k-th smallest key (histogram passes over the row: it stops as soon as one histogram bin holds exactly the
// keys still needed, or the keys at or below the bin are at most 1024), the keys at or below it are collected and only
// they are sorted.  `idx[0..k)` receive the same ids in the same order as the full sort; slots past k are not written.
// `keys` is shared memory for `key_slots` >= max(1024, pow2(k)) entries.  Called by every thread of the CTA (>= 256 threads).
__device__ __forceinline__ void select_top_blocks(const float *probs, int Nkv, int k, unsigned long long *keys, int key_slots,
                                                  int32_t *idx, int id_offset = 0, unsigned long long *keys_out = nullptr) {
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long prefix_s, mask_s;
    __shared__ int need_s, done_s;
    __shared__ unsigned int taken_s;
    const int T = blockDim.x, tid = threadIdx.x;
    if (k <= 0) return;
    auto key_of = [&](int j) { return ((unsigned long long)descending_key(probs[j]) << 32) | (unsigned)(id_offset + j); };
    // the keys of a row usually agree in their leading bytes (probabilities of one softmax share sign and most of the
    // exponent; near-uniform attention agrees much further): find the common prefix with one min/max pass and start the
    // digit passes below it
    __shared__ unsigned long long lo_s[32], hi_s[32];
    unsigned long long lo = 0xFFFFFFFFFFFFFFFFull, hi = 0ull;
    for (int j = tid; j < Nkv; j += T) {
        const unsigned long long key = key_of(j);
        lo = key < lo ? key : lo;
        hi = key > hi ? key : hi;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long l2 = __shfl_xor_sync(0xffffffffu, lo, o), h2 = __shfl_xor_sync(0xffffffffu, hi, o);
        lo = l2 < lo ? l2 : lo;
        hi = h2 > hi ? h2 : hi;
    }
    if ((tid & 31) == 0) {
        lo_s[tid >> 5] = lo;
        hi_s[tid >> 5] = hi;
    }
    __syncthreads();
    int first_byte = 7;
    if (tid == 0) {
        for (int w = 1; w < (T >> 5); ++w) {
            lo = lo_s[w] < lo ? lo_s[w] : lo;
            hi = hi_s[w] > hi ? hi_s[w] : hi;
        }
        const unsigned long long diff = lo ^ hi;
        const int top = diff ? (63 - __clzll((long long)diff)) >> 3 : 0;      // highest byte in which two keys differ
        const unsigned long long mask = top >= 7 ? 0ull : (0xFFFFFFFFFFFFFFFFull << (8 * (top + 1)));
        prefix_s = lo & mask;
        mask_s = mask;
        need_s = k;
        done_s = k >= Nkv;     // every block is kept: nothing to select
        taken_s = 0u;
        lo_s[0] = (unsigned long long)top;
    }
    __syncthreads();
    first_byte = (int)lo_s[0];
    // a histogram per warp (in the keys' memory, idle until the collection below): the probabilities of a row share their
    // leading bits, so in the first passes every warp adds to the same bin, and one shared bin serialised them
    unsigned int *warp_hist = reinterpret_cast<unsigned int *>(keys);
    const int copies = min(T >> 5, key_slots / 128), wid = (tid >> 5) % copies;      // 256 counters of 4 bytes per copy
    for (int byte = first_byte; byte >= 0 && !done_s; --byte) {
        for (int i = tid; i < copies * 256; i += T) warp_hist[i] = 0u;
        __syncthreads();
        const unsigned long long prefix = prefix_s, mask = mask_s;
        for (int j0 = 0; j0 < Nkv; j0 += T) {      // whole warps iterate together: the votes below need every lane
            const int j = j0 + tid;
            const unsigned long long key = j < Nkv ? key_of(j) : 0ull;
            const bool cand = j < Nkv && (key & mask) == prefix;
            const unsigned int voters = __ballot_sync(0xffffffffu, cand);
            if (voters) {
                // the probabilities of a row share their leading bits: the digit of the warp's first candidate is usually
                // the digit of most of them; those are counted with one addition, the others add for themselves
                const unsigned int digit = (unsigned)(key >> (8 * byte)) & 255u;
                const int leader = __ffs(voters) - 1;
                const unsigned int common = __shfl_sync(0xffffffffu, digit, leader);
                const unsigned int same = __ballot_sync(0xffffffffu, cand && digit == common);
                if ((tid & 31) == leader) atomicAdd(&warp_hist[wid * 256 + common], (unsigned)__popc(same));
                else if (cand && digit != common) atomicAdd(&warp_hist[wid * 256 + digit], 1u);
            }
        }
        __syncthreads();
        if (tid < 256) {
            unsigned int total = 0;
            for (int w = 0; w < copies; ++w) total += warp_hist[w * 256 + tid];
            hist[tid] = total;
        }
        __syncthreads();
        if (tid < 32) {      // first digit at which the running count reaches what is still needed
            unsigned int mine[8], sum = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                mine[i] = hist[tid * 8 + i];
                sum += mine[i];
            }
            unsigned int incl = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (tid >= o) incl += v;
            }
            const unsigned int need = (unsigned)need_s, before = incl - sum;
            if (before < need && need <= incl) {      // exactly one lane
                unsigned int run = before, in_bin = 0;
                int d = -1;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (d < 0) {
                        if (need <= run + mine[i]) {
                            d = i;
                            in_bin = mine[i];
                        } else {
                            run += mine[i];
                        }
                    }
                }
                prefix_s = prefix | ((unsigned long long)(tid * 8 + d) << (8 * byte));
                mask_s = mask | (0xFFull << (8 * byte));
                need_s = (int)(need - run);
                // stop refining when the whole bin is wanted, or when the keys at or below this bin are few enough to sort
                // directly (every further digit would cost another pass over the whole row)
                if (in_bin == need - run || (unsigned)k - (need - run) + in_bin <= 1024u) done_s = 1;
            }
        }
        __syncthreads();
    }
    ROUTE_STAMP(11);
    // collect the keys at or below the k-th (with all keys kept when k >= Nkv: mask 0, prefix 0), then sort just those
    const unsigned long long prefix = prefix_s, mask = mask_s;
    for (int j = tid; j < Nkv; j += T) {
        const unsigned long long key = key_of(j);
        if ((key & mask) <= prefix) keys[atomicAdd(&taken_s, 1u)] = key;
    }
    __syncthreads();
    const int kept = (int)taken_s;      // >= min(k, Nkv): the k best and, when the selection stopped early, the rest of the last bin
    int k_pow2 = 1;
    while (k_pow2 < kept) k_pow2 <<= 1;
    for (int j = kept + tid; j < k_pow2; j += T) keys[j] = 0xFFFFFFFFFFFFFFFFull;
    __syncthreads();
    sort_keys_smem(keys, k_pow2);
    for (int m = tid; m < min(k, kept); m += T) {
        if (idx) idx[m] = (int32_t)(keys[m] & 0xFFFFFFFFull);
        if (keys_out) keys_out[m] = keys[m];      // the sortable keys themselves (ids offset by `id_offset`)
    }
    __syncthreads();
}

// One (batch, head, query block) row of the fused routing; called by every thread of the CTA.  With `logits_ready`
// the row's scaled logits already lie in `sorted + row * Nkv` (written by this CTA).
__device__ __forceinline__ void route_row(const long long row, const bool logits_ready, const float *__restrict__ qp,
                                          const float *__restrict__ kp, int B, int H, int Nq, int Nkv, int n_pow2, int D, float scale,
                                          float tau_min, float tau_span, const int32_t *__restrict__ fixed_num, float *sorted,
                                          int32_t *__restrict__ index, int32_t *num, float *__restrict__ thresholds, float *gini_rows,
                                          int *counters, const SchedJob &job, unsigned long long *keys, float *probs, double *red,
                                          float &bcast, int &last_flag, const bool select_only) {
    const int T = blockDim.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = T >> 5;
    const long long bh = row / Nq;
    const int h = (int)(bh % H);

    if (logits_ready) {
        const float *lrow = sorted + row * Nkv;
        for (int j = tid; j < Nkv; j += T) probs[j] = lrow[j];
    } else {
        row_logits(qp + row * D, kp + bh * (long long)Nkv * D, Nkv, D, scale, probs);
    }
    __syncthreads();
    ROUTE_STAMP(1);
    row_softmax(Nkv, probs, red, &bcast);
    ROUTE_STAMP(2);

    if (select_only) {
        // fixed per-head count and nobody asked for the whole order or the thresholds: pick the head's k best blocks
        select_top_blocks(probs, Nkv, max(0, min(fixed_num[h], Nkv)), keys, max(n_pow2, T), index + row * Nkv);
    } else if (n_pow2 <= T) {
        // one key per thread in a register: exchange distances below 32 go through shuffles, the rest through smem
        unsigned long long key = tid < Nkv ? (((unsigned long long)descending_key(probs[tid]) << 32) | (unsigned)tid)
                                           : 0xFFFFFFFFFFFFFFFFull;
        for (int k = 2; k <= n_pow2; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                unsigned long long other;
                if (j >= 32) {
                    keys[tid] = key;
                    __syncthreads();
                    other = keys[tid ^ j];
                    __syncthreads();
                } else {
                    other = __shfl_xor_sync(0xffffffffu, key, j);
                }
                const bool keep_min = ((tid & j) == 0) == ((tid & k) == 0);
                key = (other < key) == keep_min ? other : key;
            }
        }
        keys[tid] = key;
        __syncthreads();
    } else {
        for (int j = tid; j < n_pow2; j += T)
            keys[j] = j < Nkv ? (((unsigned long long)descending_key(probs[j]) << 32) | (unsigned)j)
                              : 0xFFFFFFFFFFFFFFFFull;
        __syncthreads();
        for (int k = 2; k <= n_pow2; k <<= 1) {
            for (int j = k >> 1; j > 0; j >>= 1) {
                for (int i = tid; i < n_pow2; i += T) {
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
    }
    ROUTE_STAMP(3);
    if (!select_only) {
        int32_t *idx = index + row * Nkv;
        double acc = 0.0;
        for (int m = tid; m < Nkv; m += T) {
            const int id = (int)(keys[m] & 0xFFFFFFFFull);
            idx[m] = id;
            const float w = __fsub_rn((float)(Nkv + 1), __fmul_rn(2.0f, (float)(m + 1)));
            acc += (double)__fmul_rn(w, probs[id]);
        }
        acc = warp_sum_d(acc);
        if (lane == 0) red[warp] = acc;
        __syncthreads();
        if (tid == 0) {
            double t = 0.0;
            for (int w = 0; w < nwarps; ++w) t += red[w];
            gini_rows[row] = __fdiv_rn((float)t, (float)Nkv);
        }
        __syncthreads();
    }
    if (!fixed_num) {
        // What the count needs of this row once the head's threshold is known: for every sorted position the
        // cumulative mass before it, fl32(fl64 prefix including m) - p_m.  A contiguous run of positions per thread,
        // float64 run totals scanned over the CTA (lane order inside a warp, warp order across warps).
        float *crow = sorted + row * Nkv;
        const int chunk = (Nkv + T - 1) / T;
        const int m0 = min(Nkv, tid * chunk), m1 = min(Nkv, m0 + chunk);
        double local = 0.0;
        for (int m = m0; m < m1; ++m) local += (double)probs[(int)(keys[m] & 0xFFFFFFFFull)];
        double incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const double v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) red[warp] = incl;
        __syncthreads();
        double run = incl - local;
        for (int w = 0; w < warp; ++w) run += red[w];
        for (int m = m0; m < m1; ++m) {
            const float pm = probs[(int)(keys[m] & 0xFFFFFFFFull)];
            run += (double)pm;
            crow[m] = __fsub_rn((float)run, pm);
        }
    }

    // ---- last CTA of this head? ------------------------------------------------------------------
    const int rows_per_head = B * Nq;
    ROUTE_STAMP(4);
    __threadfence();
    __syncthreads();
    if (tid == 0) last_flag = atomicAdd(&counters[1 + h], 1) == rows_per_head - 1;
    __syncthreads();
    ROUTE_STAMP(5);
    // experiment: let the attention kernel's CTAs become resident while only the heads' last CTAs are still at work
    if (job.release_dependents_after_rows) pdl_release_dependents();
    if (!last_flag) return;
    __threadfence();

    const float thr = select_only ? 0.f : head_threshold(gini_rows, B, H, Nq, h, tau_min, tau_span, red, &bcast);
    if (tid == 0 && !select_only) thresholds[h] = thr;
    ROUTE_STAMP(8);
    if (fixed_num) {
        const int n = max(0, min(fixed_num[h], Nkv));
        for (int r = tid; r < rows_per_head; r += T) num[((long long)(r / Nq) * H + h) * Nq + r % Nq] = n;
    } else {
        // kept blocks of a row = positions whose mass-before is under the threshold.  All rows of the head are
        // counted together, a batch of independent loads per thread at a time: the loop is one CTA's, so it is the
        // memory round trips, not the arithmetic, that it has to keep few.
        constexpr int ROWS_AT_ONCE = 128, LOADS = 8;
        __shared__ int row_count[ROWS_AT_ONCE];
        __shared__ long long row_base[ROWS_AT_ONCE];
        const int step_r = T / Nkv, step_m = T % Nkv;   // element e -> (row e / Nkv, position e % Nkv), advanced without dividing
        for (int r0 = 0; r0 < rows_per_head; r0 += ROWS_AT_ONCE) {
            const int nr = min(ROWS_AT_ONCE, rows_per_head - r0);
            for (int r = tid; r < nr; r += T) {
                const int rg = r0 + r;
                row_count[r] = 0;
                row_base[r] = (((long long)(rg / Nq) * H + h) * Nq + rg % Nq) * Nkv;
            }
            __syncthreads();
            if ((Nkv & 3) == 0) {
                // four positions per load; a thread's loads are all issued before the first is used
                const int quads_per_row = Nkv >> 2, total = nr * quads_per_row;
                constexpr int QLOADS = 8;
                for (int e0 = 0; e0 < total; e0 += QLOADS * T) {
                    float4 c[QLOADS];
                    int rr[QLOADS];
#pragma unroll
                    for (int u = 0; u < QLOADS; ++u) {
                        const int e = e0 + u * T + tid;
                        rr[u] = -1;
                        if (e < total) {
                            const int r = e / quads_per_row;
                            rr[u] = r;
                            c[u] = __ldcg(reinterpret_cast<const float4 *>(sorted + row_base[r]) + (e - r * quads_per_row));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < QLOADS; ++u)
                        if (rr[u] >= 0) {
                            const int n = (c[u].x < thr) + (c[u].y < thr) + (c[u].z < thr) + (c[u].w < thr);
                            if (n) atomicAdd(&row_count[rr[u]], n);
                        }
                }
            } else {
            const int total = nr * Nkv;   // <= 128 * 16384
            int r = tid / Nkv, m = tid % Nkv;
            for (int e0 = 0; e0 < total; e0 += LOADS * T) {
                float c[LOADS];
                int rr[LOADS];
#pragma unroll
                for (int u = 0; u < LOADS; ++u) {
                    const bool in = e0 + u * T + tid < total;
                    rr[u] = in ? r : -1;
                    c[u] = in ? __ldcg(sorted + row_base[r] + m) : 0.f;
                    r += step_r;
                    m += step_m;
                    if (m >= Nkv) {
                        m -= Nkv;
                        ++r;
                    }
                }
#pragma unroll
                for (int u = 0; u < LOADS; ++u) {
                    const bool keep = rr[u] >= 0 && c[u] < thr;
                    const int first = __shfl_sync(0xffffffffu, rr[u], 0);
                    if (__all_sync(0xffffffffu, rr[u] == first)) {   // the warp is inside one row: one atomic for all lanes
                        const int n = __popc(__ballot_sync(0xffffffffu, keep));
                        if (lane == 0 && first >= 0 && n) atomicAdd(&row_count[first], n);
                    } else if (keep) {
                        atomicAdd(&row_count[rr[u]], 1);
                    }
                }
            }
            }
            __syncthreads();
            ROUTE_STAMP(9);
            for (int r2 = tid; r2 < nr; r2 += T) num[row_base[r2] / Nkv] = row_count[r2];
            __syncthreads();
        }
    }

    // ---- last head? ------------------------------------------------------------------------------
    ROUTE_STAMP(6);
    __threadfence();
    __syncthreads();
    if (tid == 0) last_flag = atomicAdd(&counters[0], 1) == H - 1;
    __syncthreads();
    if (!last_flag || !job.order) return;
    __threadfence();
    schedule_items(num, B * H * Nq, Nkv, job.order, job.work_counter, job.error_flag);
    ROUTE_STAMP(7);
}

// ------------------------------------------------------------------------------------------------
// The forward's routing in ONE launch.  Each CTA owns one row, or (thousands of key blocks, head_dim 128) four
// neighbouring rows of a head whose logits it computes in one pass over the pooled keys.
// ------------------------------------------------------------------------------------------------
template <int ROWS>   // rows per CTA: 1, 4 or 8 (several rows: 512 threads)
__global__ void __launch_bounds__(ROWS > 1 ? 512 : 1024)
route_fused_kernel(const float *__restrict__ qp, const float *__restrict__ kp, int B, int H, int Nq, int Nkv, int n_pow2,
                   int D, float scale, float tau_min, float tau_span, const int32_t *__restrict__ fixed_num,
                   float *sorted, int32_t *__restrict__ index, int32_t *num, float *__restrict__ thresholds,
                   float *gini_rows, int *counters, SchedJob job, int gate_per_cta, int sm_count, int slots, int groups_per_bh,
                   int select_only) {
    constexpr int rows_per_cta = ROWS;
    extern __shared__ __align__(16) unsigned char fused_smem[];
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(fused_smem);   // max(n_pow2, threads)
    float *probs = reinterpret_cast<float *>(keys + max(n_pow2, (int)blockDim.x));    // Nkv
    __shared__ double red[256];
    __shared__ __align__(16) double q_rows[ROWS > 1 ? ROWS * 128 : 2];
    __shared__ float bcast;
    __shared__ int last_flag;

    // CTAs are dealt to the SMs round-robin, so CTAs b, b + sm_count, ... tend to share an SM: give them
    // neighbouring rows (same head, same pooled keys) so that their key reads can meet in L1
    const long long group = (long long)(blockIdx.x % sm_count) * slots + blockIdx.x / sm_count;
    // No early release of the attention kernel here: its CTAs, once resident and waiting, slowed the tail of this
    // kernel (the per-head count and the work order are a few CTAs' work) by about 5 us.
    pdl_wait();                 // pooled means and zeroed counters come from the launch before
    if (group >= (long long)B * H * groups_per_bh) return;
    const long long bh = group / groups_per_bh;
    const int i0 = (int)(group % groups_per_bh) * rows_per_cta, nrows = min(rows_per_cta, Nq - i0);
    const long long row0 = bh * Nq + i0;

    ROUTE_STAMP(0);
    if (job.order && job.gate_w) convert_gate_slice(job, (int)group * gate_per_cta, gate_per_cta);

    if constexpr (ROWS > 1) {
        // the sort keys' shared memory is free until the first row is sorted: the pooled keys are staged through it
        // (and through the head of the probabilities' memory behind it, which is not in use yet either)
        const int stage_bytes = max(n_pow2, (int)blockDim.x) * 8 + Nkv * 4;
        int tile_keys = 128;      // two staging buffers of (tile_keys + 1) x 512 bytes; whole warps of keys
        while (tile_keys > 32 && 2 * (tile_keys + 1) * 512 > stage_bytes) tile_keys -= 32;
        row_logits_keys<ROWS>(qp + row0 * D, nrows, kp + bh * (long long)Nkv * D, Nkv, scale, sorted + row0 * Nkv, q_rows,
                              reinterpret_cast<float4 *>(keys), tile_keys);      // ends with a barrier: the rows below read these logits back
        ROUTE_STAMP(10);
    }
    if constexpr (ROWS == 1) {
        route_row(row0, false, qp, kp, B, H, Nq, Nkv, n_pow2, D, scale, tau_min, tau_span, fixed_num, sorted, index, num, thresholds,
                  gini_rows, counters, job, keys, probs, red, bcast, last_flag, select_only != 0);
        return;
    }
    for (int r = 0; r < nrows; ++r) {
        route_row(row0 + r, true, qp, kp, B, H, Nq, Nkv, n_pow2, D, scale, tau_min, tau_span, fixed_num, sorted, index,
                  num, thresholds, gini_rows, counters, job, keys, probs, red, bcast, last_flag, select_only != 0);
        __syncthreads();
    }
}

#ifdef WA_ROUTE_TRACE
}  // namespace wa
extern "C" int wa_route_trace_read(long long *dst, int n_ctas) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(dst, wa::g_route_trace, (size_t)n_ctas * 12 * sizeof(long long));
    return 0;
}
namespace wa {
#endif

// ------------------------------------------------------------------------------------------------
// Fixed top-k routing over a SHARDED key cache (no reference counterpart: the reference is single-device).
// Every rank scores only the key blocks it owns and keeps its best `kcap` per row as sortable 64-bit keys
// (descending logit, then ascending global block id); the ranks exchange those keys; each rank then merges
// the W * kcap candidates of a row, takes the head's k best and keeps the ones it owns.  Work and traffic per
// rank fall with the number of ranks, where gathering every pooled key and repeating the whole routing on
// every rank does not.  Selection is by LOGIT: softmax is monotone, so this is the single-device choice
// except where distinct logits round to one probability at the k-th place (there the single-device rule
// orders by block id, this one by logit).
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void sort_keys_smem(unsigned long long *keys, int n_pow2) {   // ascending bitonic sort, whole CTA
    const int T = blockDim.x;
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
}

__global__ void __launch_bounds__(1024)
route_local_candidates_kernel(const float *__restrict__ qp, const float *__restrict__ kp, int Nq, int Nloc, int n_pow2, int D,
                              float scale, int block_lo, int kcap, unsigned long long *__restrict__ cand) {
    extern __shared__ __align__(16) unsigned char cand_smem[];
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(cand_smem);   // n_pow2
    float *logits = reinterpret_cast<float *>(keys + n_pow2);                       // Nloc
    const long long row = blockIdx.x;   // (b * H + h) * Nq + i
    const long long bh = row / Nq;
    row_logits(qp + row * D, kp + bh * (long long)Nloc * D, Nloc, D, scale, logits);
    __syncthreads();
    if (n_pow2 > (int)blockDim.x && kcap <= 1024) {
        // a long row: pick the kcap best instead of sorting all of them (same keys, same order)
        const int k = min(kcap, Nloc);
        select_top_blocks(logits, Nloc, k, keys, n_pow2, nullptr, block_lo, cand + row * kcap);
        for (int j = k + threadIdx.x; j < kcap; j += blockDim.x) cand[row * kcap + j] = 0xFFFFFFFFFFFFFFFFull;
        return;
    }
    for (int j = threadIdx.x; j < n_pow2; j += blockDim.x)
        keys[j] = j < Nloc ? (((unsigned long long)descending_key(logits[j]) << 32) | (unsigned)(block_lo + j))
                           : 0xFFFFFFFFFFFFFFFFull;
    __syncthreads();
    sort_keys_smem(keys, n_pow2);
    for (int j = threadIdx.x; j < kcap; j += blockDim.x) cand[row * kcap + j] = j < n_pow2 ? keys[j] : 0xFFFFFFFFFFFFFFFFull;
}

__global__ void __launch_bounds__(256)
route_merge_candidates_kernel(const unsigned long long *__restrict__ cand, int W, long long rows, int Nq, int H, int kcap,
                              int n_pow2, const int32_t *__restrict__ topk, int Nkv_total, int block_lo, int block_hi,
                              int index_stride, int32_t *__restrict__ local_index, int32_t *__restrict__ local_num) {
    extern __shared__ __align__(16) unsigned char merge_smem[];
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(merge_smem);   // n_pow2 >= W * kcap
    __shared__ int count;
    const long long row = blockIdx.x;
    const int h = (int)((row / Nq) % H);
    const int n = W * kcap;
    for (int j = threadIdx.x; j < n_pow2; j += blockDim.x)
        keys[j] = j < n ? cand[((long long)(j / kcap) * rows + row) * kcap + (j % kcap)] : 0xFFFFFFFFFFFFFFFFull;
    if (threadIdx.x == 0) count = 0;
    __syncthreads();
    sort_keys_smem(keys, n_pow2);
    const int k = max(0, min(min(topk[h], Nkv_total), n));
    // the head's k best; the ones this rank owns, in ascending block order (candidates of one rank arrive id-distinct,
    // so an id appears once)
    int32_t *out = local_index + row * index_stride;
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const unsigned id = (unsigned)(keys[j] & 0xFFFFFFFFull);
        if (keys[j] != 0xFFFFFFFFFFFFFFFFull && (int)id >= block_lo && (int)id < block_hi) {
            // rank among the owned ones = number of owned selected ids below this one
            int below = 0;
            for (int t = 0; t < k; ++t) {
                const unsigned other = (unsigned)(keys[t] & 0xFFFFFFFFull);
                below += keys[t] != 0xFFFFFFFFFFFFFFFFull && (int)other >= block_lo && (int)other < block_hi && other < id;
            }
            out[below] = (int)id - block_lo;
            atomicAdd(&count, 1);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) local_num[row] = count;
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

// ------------------------------------------------------------------------------------------------
// Selection of one KV shard.  One warp per row: a bitmap of the shard's blocks in shared memory,
// then two ballot-ordered compactions (selected blocks, then the rest).
// ------------------------------------------------------------------------------------------------
constexpr int LOCAL_SEL_WARPS = 8;

__global__ void __launch_bounds__(LOCAL_SEL_WARPS * 32)
local_selection_kernel(const int32_t *__restrict__ index, const int32_t *__restrict__ num, long long rows, int Nkv,
                       int block_lo, int width, int words, int32_t *__restrict__ local_index,
                       int32_t *__restrict__ local_num) {
    extern __shared__ unsigned int sel_bitmap[];   // [warps][words]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * LOCAL_SEL_WARPS + warp;
    if (row >= rows) return;
    unsigned int *bm = sel_bitmap + warp * words;
    for (int w = lane; w < words; w += 32) bm[w] = 0u;
    __syncwarp();
    const int32_t *idx = index + row * Nkv;
    const int n = max(0, min(num[row], Nkv));
    for (int j = lane; j < n; j += 32) {
        const int id = max(0, min(idx[j], Nkv - 1)) - block_lo;
        if (id >= 0 && id < width) atomicOr(&bm[id >> 5], 1u << (id & 31));
    }
    __syncwarp();
    int32_t *out = local_index + row * width;
    int at = 0;
    for (int pass = 0; pass < 2; ++pass) {   // members first, then the rest
        for (int base = 0; base < width; base += 32) {
            const int c = base + lane;
            const bool member = c < width && ((bm[base >> 5] >> lane) & 1u);
            const bool take = c < width && (pass == 0 ? member : !member);
            const unsigned bal = __ballot_sync(0xffffffffu, take);
            if (take) out[at + __popc(bal & ((1u << lane) - 1u))] = c;
            at += __popc(bal);
        }
        if (pass == 0 && lane == 0) local_num[row] = at;
    }
}

}  // namespace wa

using namespace wa;

extern "C" int wa_route_local_selection(const int32_t *index, const int32_t *num, long long rows, int Nkv, int block_lo,
                                        int block_hi, int32_t *local_index, int32_t *local_num, void *stream) {
    WA_REQUIRE(index && num && local_index && local_num, WA_ERR_ARG, "wa_route_local_selection: null pointer");
    WA_REQUIRE(rows > 0 && Nkv > 0 && block_lo >= 0 && block_hi > block_lo, WA_ERR_ARG,
               "wa_route_local_selection: need rows > 0, Nkv > 0 and a non-empty block range");
    const int width = block_hi - block_lo;
    WA_REQUIRE(width <= 16384, WA_ERR_UNSUPPORTED, "wa_route_local_selection: at most 16384 blocks per shard, got %d", width);
    const int words = (width + 31) / 32;
    const long long ctas = (rows + LOCAL_SEL_WARPS - 1) / LOCAL_SEL_WARPS;
    WA_REQUIRE(ctas < (1ll << 31), WA_ERR_UNSUPPORTED, "wa_route_local_selection: too many rows");
    local_selection_kernel<<<(unsigned)ctas, LOCAL_SEL_WARPS * 32, (size_t)LOCAL_SEL_WARPS * words * sizeof(unsigned int),
                             (cudaStream_t)stream>>>(index, num, rows, Nkv, block_lo, width, words, local_index, local_num);
    return check_launch("wa_route_local_selection");
}

namespace wa {
static bool pool_vec_ok(const wa_tensor4 *x, int D) {
    return x->dtype == WA_BF16 && D % 8 == 0 && D / 8 <= POOL_THREADS && ((uintptr_t)x->ptr % 16 == 0) &&
           x->stride_b % 8 == 0 && x->stride_l % 8 == 0 && x->stride_h % 8 == 0;
}

// Pools `x` (and, when given, `y`, e.g. queries and keys of one forward) in a single launch.
int pool_launch(const wa_tensor4 *x, int Lx, float *px, const wa_tensor4 *y, int Ly, float *py, int B, int H, int D,
                int block_size, cudaStream_t stream, int *zero, int n_zero, int y_first_block, int *status_mirror) {
    const int nbx = ceil_div(Lx, block_size);
    const int nby_all = y ? ceil_div(Ly, block_size) : 0;   // rows per (batch, head) of py
    const int y_aligned = y ? Ly % block_size == 0 : 0;
    wa_tensor4 y_tail;
    if (y && y_first_block >= nby_all) y = nullptr;   // every key block is pooled already
    if (y && y_first_block > 0) {   // the first blocks of y are pooled already: start at token y_first_block * block_size
        y_tail = *y;
        y_tail.ptr = (char *)y->ptr + (size_t)y_first_block * block_size * y->stride_l * dtype_size(y->dtype);
        y = &y_tail;
        Ly -= y_first_block * block_size;
        py += (size_t)y_first_block * D;
    }
    const int nby = y ? ceil_div(Ly, block_size) : 0;
    if (pool_sm100_supported(x, y, H, D, block_size) && (uintptr_t)px % 8 == 0 && (!y || (uintptr_t)py % 8 == 0))
        return pool_sm100_launch(x, Lx, px, y, Ly, py, nby_all, B, H, D, block_size, stream, zero, n_zero, status_mirror);
    View4 vx = make_view(x), vy = y ? make_view(y) : vx;
    dim3 grid(nbx + nby, H, B);
    const bool vec = pool_vec_ok(x, D) && (!y || pool_vec_ok(y, D));
    const int lanes = D / 8;
    if (vec && D % 8 == 0 && lanes <= 32 && (lanes & (lanes - 1)) == 0 && ((uintptr_t)px % 16 == 0) &&
        (!y || (uintptr_t)py % 16 == 0)) {
        constexpr int items_per_cta = POOL_THREADS / 32 / WA_POOL_SPLIT;
        const long long items = (long long)B * H * (nbx + nby);
        const long long ctas = (items + items_per_cta - 1) / items_per_cta;
        WA_REQUIRE(ctas < (1ll << 31), WA_ERR_UNSUPPORTED, "wa_pool_blocks: too many blocks");
        pool_warp_kernel<WA_POOL_UNROLL, WA_POOL_SPLIT><<<(unsigned)ctas, POOL_THREADS, 0, stream>>>(
            vx, Lx, H, D, block_size, nbx, Lx % block_size == 0, px, vy, Ly, nby, y_aligned, py, nby_all, B, zero, n_zero);
    } else if (vec) {
        const int rows = POOL_THREADS / (D / 8);
        const size_t smem = (size_t)rows * D * sizeof(double);
        WA_REQUIRE(smem <= 48 * 1024, WA_ERR_UNSUPPORTED, "wa_pool_blocks: D=%d too large", D);
        pool_blocks_kernel<true><<<grid, POOL_THREADS, smem, stream>>>(vx, Lx, H, D, block_size, nbx, Lx % block_size == 0,
                                                                       px, vy, Ly, nby, y_aligned, py, nby_all, zero, n_zero);
    } else {
        const int rows = D >= POOL_THREADS ? 1 : POOL_THREADS / D;
        const size_t smem = (size_t)rows * (D < POOL_THREADS ? D : POOL_THREADS) * sizeof(double);
        pool_blocks_kernel<false><<<grid, POOL_THREADS, smem, stream>>>(vx, Lx, H, D, block_size, nbx, Lx % block_size == 0,
                                                                        px, vy, Ly, nby, y_aligned, py, nby_all, zero, n_zero);
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
    return pool_launch(x, L, pooled, nullptr, 0, nullptr, B, H, D, block_size, (cudaStream_t)stream, nullptr, 0, 0);
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

namespace wa {
int route_fused_launch(const float *q_pooled, const float *k_pooled, int B, int H, int Nq, int Nkv, int D, double tau_min,
                       double tau_max, const int32_t *fixed_num_per_head, float *sorted, int32_t *index, int32_t *num,
                       float *thresholds, float *gini, int *counters, const SchedJob &job_in, cudaStream_t stream, bool whole_order) {
    int n_pow2 = 1;
    while (n_pow2 < Nkv) n_pow2 <<= 1;
    WA_REQUIRE(n_pow2 <= 16384, WA_ERR_UNSUPPORTED, "wa_hsa_forward(routing): at most 16384 key blocks per row, got %d", Nkv);
    const long long rows = (long long)B * H * Nq;
    WA_REQUIRE(rows < (1ll << 31), WA_ERR_UNSUPPORTED, "wa_hsa_forward(routing): too many rows");
    int threads = n_pow2 / 2;
    threads = threads < 256 ? 256 : (threads > 1024 ? 1024 : threads);
    const size_t smem = (size_t)(n_pow2 > threads ? n_pow2 : threads) * sizeof(unsigned long long) + (size_t)Nkv * sizeof(float);
    if (smem > 24 * 1024) {   // static shared memory of the kernel takes ~19 KB of the default 48 KB
        cudaError_t e = cudaFuncSetAttribute(route_fused_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(route_fused_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(route_fused_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "wa_hsa_forward(routing): %s", cudaGetErrorString(e));
    }
    // several rows per CTA where a row's keys are megabytes (see row_logits_keys); one row per CTA where the kernel is latency.
    // More rows per CTA share more key reads and conversions, but the CTAs come in waves of one per SM (their shared memory
    // fills it) and a CTA's rows are softmaxed and selected one after the other: take the count with the lowest estimate.
    int dev = 0, sm_count = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
        sm_count = 148;
    int rows_per_cta = 1;
    if (Nkv > 2048 && D == 128 && ((uintptr_t)q_pooled % 16 == 0) && ((uintptr_t)k_pooled % 16 == 0)) {
        // measured at 11 700 key blocks (microseconds; everything scales with the block count, so the comparison holds):
        // scoring one row per CTA 115, R rows per CTA 190 + 29 R, and 21 per row for softmax and selection
        auto cost = [&](int r) {
            const long long g = (long long)B * H * ((Nq + r - 1) / r);
            return ((g + sm_count - 1) / sm_count) * (r == 1 ? 115 + 21 : 190 + (29 + 21) * r);
        };
        rows_per_cta = cost(4) < cost(8) ? 4 : 8;
        if (cost(1) < cost(rows_per_cta)) rows_per_cta = 1;
        if (const char *e = getenv("WA_B200_ROUTE_ROWS"))      // tuning aid
            if (e[0] == '1' || e[0] == '4' || e[0] == '8') rows_per_cta = e[0] - '0';
    }
    const int groups_per_bh = (Nq + rows_per_cta - 1) / rows_per_cta;
    const long long groups = (long long)B * H * groups_per_bh;
    const int gate_per_cta = (int)((128 * 128 + groups - 1) / groups);
    if (groups < sm_count) sm_count = (int)groups;
    const int slots = (int)((groups + sm_count - 1) / sm_count);
    const dim3 grid((unsigned)((long long)sm_count * slots));
    const float scale = (float)pow((double)D, -0.5), span = (float)(tau_max - tau_min);
    SchedJob job = job_in;
    job.release_dependents_after_rows = pdl_mode() == 2;
    // a fixed count per head over more key blocks than one pass of the register sort covers, and nobody reads the whole
    // order or the thresholds: select the best blocks instead of sorting all of them
    const int select_only = fixed_num_per_head && !whole_order && n_pow2 > threads;
    if (rows_per_cta > 1 && threads > 512) threads = 512;
    auto launch = [&](auto kernel) {
        return launch_dependent(kernel, grid, dim3(threads), smem, stream, q_pooled, k_pooled, B, H, Nq, Nkv, n_pow2, D, scale,
                                (float)tau_min, span, fixed_num_per_head, sorted, index, num, thresholds, gini, counters, job,
                                gate_per_cta, sm_count, slots, groups_per_bh, select_only);
    };
    cudaError_t le = rows_per_cta == 8 ? launch(route_fused_kernel<8>)
                                       : (rows_per_cta == 4 ? launch(route_fused_kernel<4>) : launch(route_fused_kernel<1>));
    if (le != cudaSuccess) return fail((int)le, "wa_hsa_forward(routing): %s", cudaGetErrorString(le));
    return check_launch("wa_hsa_forward(routing)");
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

extern "C" int wa_route_local_candidates(const float *q_pooled, const float *k_pooled_local, int B, int H, int Nq, int Nloc, int D,
                                         int block_lo, int kcap, unsigned long long *candidates, void *stream) {
    const char *what = "wa_route_local_candidates";
    WA_REQUIRE(q_pooled && candidates && (k_pooled_local || Nloc == 0), WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nloc >= 0 && D > 0 && kcap > 0 && block_lo >= 0, WA_ERR_ARG, "%s: bad sizes", what);
    int n_pow2 = 1;
    while (n_pow2 < Nloc) n_pow2 <<= 1;
    WA_REQUIRE(n_pow2 <= 16384, WA_ERR_UNSUPPORTED, "%s: at most 16384 key blocks per shard, got %d", what, Nloc);
    const long long rows = (long long)B * H * Nq;
    WA_REQUIRE(rows < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many rows", what);
    int threads = n_pow2 / 2;
    threads = threads < 256 ? 256 : (threads > 1024 ? 1024 : threads);
    const size_t smem = (size_t)n_pow2 * sizeof(unsigned long long) + (size_t)(Nloc > 0 ? Nloc : 1) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(route_local_candidates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
    }
    route_local_candidates_kernel<<<(unsigned)rows, threads, smem, (cudaStream_t)stream>>>(
        q_pooled, k_pooled_local, Nq, Nloc, n_pow2, D, (float)pow((double)D, -0.5), block_lo, kcap, candidates);
    return check_launch(what);
}

extern "C" int wa_route_merge_candidates(const unsigned long long *candidates, int W, int B, int H, int Nq, int kcap,
                                         const int32_t *topk_per_head, int Nkv_total, int block_lo, int block_hi, int index_stride,
                                         int32_t *local_index, int32_t *local_num, void *stream) {
    const char *what = "wa_route_merge_candidates";
    WA_REQUIRE(candidates && topk_per_head && local_index && local_num, WA_ERR_ARG, "%s: null pointer", what);
    WA_REQUIRE(W > 0 && B > 0 && H > 0 && Nq > 0 && kcap > 0 && Nkv_total > 0 && block_lo >= 0 && block_hi >= block_lo, WA_ERR_ARG,
               "%s: bad sizes", what);
    WA_REQUIRE(index_stride >= kcap || index_stride >= block_hi - block_lo, WA_ERR_ARG,
               "%s: index rows of %d entries cannot hold the selection", what, index_stride);
    int n_pow2 = 1;
    while (n_pow2 < W * kcap) n_pow2 <<= 1;
    WA_REQUIRE(n_pow2 <= 4096, WA_ERR_UNSUPPORTED, "%s: at most 4096 candidates per row, got %d", what, W * kcap);
    const long long rows = (long long)B * H * Nq;
    WA_REQUIRE(rows < (1ll << 31), WA_ERR_UNSUPPORTED, "%s: too many rows", what);
    route_merge_candidates_kernel<<<(unsigned)rows, 256, (size_t)n_pow2 * sizeof(unsigned long long), (cudaStream_t)stream>>>(
        candidates, W, rows, Nq, H, kcap, n_pow2, topk_per_head, Nkv_total, block_lo, block_hi, index_stride, local_index,
        local_num);
    return check_launch(what);
}
