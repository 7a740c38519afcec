// compress_kv -- and the KV-cache append fused with it -- as a TMA-fed tcgen05 stream for sm_100a.
//
// compress_kv (wan/modules/hsa/attention.py:64-110) is, per segment, the product of the [rank x tokens]
// projection with the [tokens x H*D] token rows: 13..25 output rows for 1560 x 1536 inputs, so the
// kernel's job is to read K and V once at HBM speed; the contraction itself rides along on the tensor
// cores.  Work item = (128 columns, segment, K|V, batch).  A persistent CTA of four warps streams the
// item's tokens in 128-token tiles through a three-stage shared-memory ring:
//   warp 1  TMA loads: the token tile [128 tokens x 128 columns] and the matching [128 rows x 128 tokens]
//           tile of the projection (rows past the rank and tokens past the segment come back as zeros);
//   warp 2  tcgen05.mma, D[rank rows x 128 columns] (+)= E_tile . X_tile, float32 in tensor memory,
//           two accumulators so that the next item starts while the last one is read out;
//   warp 3  (append only) TMA store of the same shared-memory tile into the KV cache -- the rows are
//           read from HBM once and leave twice;
//   warp 0  reads the accumulator's first `rank` lanes and writes the bf16 slots.
// Every mbarrier wait is bounded; a wait that runs out raises a flag that wa_compress_status reads.
#include "wa_internal.cuh"
#include "wa_sm100_ptx.cuh"

namespace wa {
namespace sm100 {
namespace compress {

constexpr int THREADS = 128;
constexpr int STAGES = 3;
constexpr int STAGE_BYTES = 2 * TILE_BYTES;                // token tile + projection tile
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
constexpr int TMEM_COLS = 256;                             // two [128 x 128] float32 accumulators

struct Barriers {
    uint64_t full[STAGES], empty[STAGES];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct Job {
    int n_seg, tiles_cols, B;          // items = B * 2 * n_seg * tiles_cols
    int L, segment_len, block_size, proj_rank;
    int slot0, slot_stride;            // first compressed slot of segment 0; slots between consecutive segments
    int copy;                          // also store the token tiles through the destination maps
    __nv_bfloat16 *out_k, *out_v;
    long long osb, osl;
    int *status;
};

__device__ int g_status;               // 0, or the site code of a wait that ran out

__global__ void __launch_bounds__(THREADS, 1)
compress_stream_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const __grid_constant__ CUtensorMap tm_ek, const __grid_constant__ CUtensorMap tm_ev,
                       const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv, const Job job) {
    extern __shared__ __align__(1024) uint8_t smem[];
    Barriers *bar = reinterpret_cast<Barriers *>(smem + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &bar->abort_flag;
    const FailSink sink{job.status, nullptr};

    if (threadIdx.x == 0) {
        bar->abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;
        if (bar->abort_flag) report_failure(sink, 99);
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&bar->full[i], 1);
            mbar_init(&bar->empty[i], job.copy ? 2 : 1);   // the products that read the stage have landed (+ the store warp is done with it)
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar->acc_full[i], 1);
            mbar_init(&bar->acc_empty[i], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bar->tmem_base;
    const int n_items = job.B * 2 * job.n_seg * job.tiles_cols;

    // item -> (column tile fastest, then segment, K|V, batch): neighbouring CTAs read neighbouring columns of the same rows
    auto decode = [&](int item, int &ct, int &seg, int &which, int &b) {
        ct = item % job.tiles_cols;
        seg = (item / job.tiles_cols) % job.n_seg;
        which = (item / (job.tiles_cols * job.n_seg)) & 1;
        b = item / (job.tiles_cols * job.n_seg * 2);
    };
    auto seg_tiles = [&](int seg) {
        const int n_tok = min(job.segment_len, job.L - seg * job.segment_len);
        return (n_tok + TILE - 1) / TILE;
    };

    if (warp == 1) {
        // ================= producer =================
        if (lane == 0) {
            uint32_t count = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int ct, seg, which, b;
                decode(item, ct, seg, which, b);
                const CUtensorMap *tx = which ? &tm_v : &tm_k, *te = which ? &tm_ev : &tm_ek;
                const int tok0 = seg * job.segment_len, n_tiles = seg_tiles(seg);
                for (int t = 0; t < n_tiles && ok; ++t, ++count) {
                    const uint32_t s = count % STAGES;
                    ok = mbar_wait(&bar->empty[s], ((count / STAGES) & 1u) ^ 1u, abort_flag, sink, 1);
                    if (!ok) break;
                    uint8_t *xs = smem + s * STAGE_BYTES, *es = xs + TILE_BYTES;
                    mbar_expect_tx(&bar->full[s], STAGE_BYTES);
                    tma_load_3d(xs, tx, &bar->full[s], ct * TILE, tok0 + t * TILE, b);
                    tma_load_3d(xs + HALF_BYTES, tx, &bar->full[s], ct * TILE + 64, tok0 + t * TILE, b);
                    tma_load_2d(es, te, &bar->full[s], t * TILE, 0);
                    tma_load_2d(es + HALF_BYTES, te, &bar->full[s], t * TILE + 64, 0);
                }
            }
        }
    } else if (warp == 2) {
        // ================= issuer =================
        const bool leader = elect_one();
        constexpr uint32_t IDESC = instr_desc(true, TILE);   // A = projection tile (K-major), B = token tile (columns contiguous)
        uint32_t count = 0, n_done = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_done) {
            int ct, seg, which, b;
            decode(item, ct, seg, which, b);
            const uint32_t buf = n_done & 1u;
            // the accumulator was read out two items ago
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->acc_empty[buf], ((n_done >> 1) & 1u) ^ 1u, abort_flag, sink, 2));
            if (!ok) break;
            const int n_tiles = seg_tiles(seg);
            for (int t = 0; t < n_tiles && ok; ++t, ++count) {
                const uint32_t s = count % STAGES;
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->full[s], (count / STAGES) & 1u, abort_flag, sink, 3));
                if (!ok) break;
                tc_fence_after();
                if (leader) {
                    const uint32_t xs = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t bd = smem_desc(xs, HALF_BYTES, 1024), ad = smem_desc(xs + TILE_BYTES, 16, 1024);
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        mma_ss(tmem + buf * TILE, ad + (uint64_t)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4),
                               bd + (uint64_t)((kk * 2048) >> 4), IDESC, !(t == 0 && kk == 0));
                    tc_commit(&bar->empty[s]);
                    if (t == n_tiles - 1) tc_commit(&bar->acc_full[buf]);
                }
                __syncwarp();
            }
        }
    } else if (warp == 3) {
        // ================= store warp: the token tile also goes to the cache (append), or straight back to the producer ===
        if (lane == 0 && job.copy) {
            uint32_t count = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                int ct, seg, which, b;
                decode(item, ct, seg, which, b);
                const CUtensorMap *td = which ? &tm_dv : &tm_dk;
                const int tok0 = seg * job.segment_len, n_tiles = seg_tiles(seg);
                for (int t = 0; t < n_tiles && ok; ++t, ++count) {
                    const uint32_t s = count % STAGES;
                    ok = mbar_wait(&bar->full[s], (count / STAGES) & 1u, abort_flag, sink, 4);
                    if (!ok) break;
                    uint8_t *xs = smem + s * STAGE_BYTES;
                    // rows past the appended range are clipped by the destination map
                    tma_store_3d(td, xs, ct * TILE, tok0 + t * TILE, b);
                    tma_store_3d(td, xs + HALF_BYTES, ct * TILE + 64, tok0 + t * TILE, b);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    mbar_arrive(&bar->empty[s]);
                }
            }
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
    } else {
        // ================= epilogue: accumulator rows (= ranks) of lanes 0..31, 32 columns at a time =================
        uint32_t n_done = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++n_done) {
            int ct, seg, which, b;
            decode(item, ct, seg, which, b);
            const uint32_t buf = n_done & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->acc_full[buf], (n_done >> 1) & 1u, abort_flag, sink, 5));
            if (!ok) break;
            tc_fence_after();
            const int n_tok = min(job.segment_len, job.L - seg * job.segment_len);
            const int rank = min(job.proj_rank, (n_tok + job.block_size - 1) / job.block_size);
            __nv_bfloat16 *out = (which ? job.out_v : job.out_k) + (long long)b * job.osb +
                                 (long long)(job.slot0 + seg * job.slot_stride + lane) * job.osl + ct * TILE;
            {   // this warp reads tensor-memory lanes 0..31: rank <= 32 is a condition of this path
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    TMEM_LD32(tmem + buf * TILE + c * 32, v);
                    tmem_wait_ld();
                    if (lane < rank) {
                        uint32_t packed[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                            packed[j] = *reinterpret_cast<uint32_t *>(&h);
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            *reinterpret_cast<uint4 *>(out + c * 32 + j * 8) =
                                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// `[B, rows, H*D]` bf16 rows with contiguous heads -> 3-D map (column, row, batch), box 64 x 128 x 1, 128-byte swizzle.
static bool map_rows(CUtensorMap *map, void *base, int cols, int rows, int B, long long stride_row, long long stride_b) {
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)B};
    cuuint64_t strides[2] = {(cuuint64_t)stride_row * 2, (cuuint64_t)(B == 1 ? stride_row * rows : stride_b) * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)TILE, 1}, elem[3] = {1, 1, 1};
    return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// projection `[rank, proj_cols]` bf16 -> 2-D map (token, rank) restricted to the first `tokens` columns, box 64 x 128
static bool map_projection(CUtensorMap *map, const void *base, int tokens, int rank, int proj_cols) {
    cuuint64_t dims[2] = {(cuuint64_t)tokens, (cuuint64_t)rank};
    cuuint64_t strides[1] = {(cuuint64_t)proj_cols * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TILE}, elem[2] = {1, 1};
    return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace compress
}  // namespace sm100

// Whether the tcgen05 stream covers this call (bf16 everything, contiguous heads, 16-byte aligned rows, rank <= 32,
// an sm_100 device); `dst_*` are null for a plain compress_kv.
bool compress_sm100_supported(const wa_tensor4 *k, const wa_tensor4 *v, const wa_tensor4 *ok, const wa_tensor4 *ov,
                              const wa_tensor4 *dst_k, const wa_tensor4 *dst_v, int H, int D, int proj_dtype, int proj_cols,
                              int rank_full, const void *k_proj, const void *v_proj) {
    using namespace sm100::compress;
    const wa_tensor4 *views[6] = {k, v, ok, ov, dst_k, dst_v};
    for (const wa_tensor4 *t : views) {
        if (!t) continue;
        if (t->dtype != WA_BF16 || t->stride_h != D || (uintptr_t)t->ptr % 16 || t->stride_l % 8 || t->stride_b % 8 || t->stride_l < (long long)H * D)
            return false;
    }
    if (proj_dtype != WA_BF16 || (H * D) % sm100::TILE || rank_full > 32 || proj_cols % 8 || (uintptr_t)k_proj % 16 || (uintptr_t)v_proj % 16)
        return false;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        major != 10)
        return false;
    return encode_fn() != nullptr;
}

// Compress the L tokens of `k` / `v` (segments of segment_len from token 0) into slots slot0 + seg * slot_stride + r of
// out_k / out_v; with dst_k / dst_v also copy the rows to rows [dst_row0, dst_row0 + L) of those tensors.
int compress_sm100_launch(const wa_tensor4 *k, const wa_tensor4 *v, const wa_tensor4 *ok, const wa_tensor4 *ov,
                          const wa_tensor4 *dst_k, const wa_tensor4 *dst_v, int dst_row0, int B, int L, int H, int D,
                          int segment_len, int block_size, const void *k_proj, const void *v_proj, int proj_rank, int proj_cols,
                          int slot0, int slot_stride, cudaStream_t stream) {
    using namespace sm100::compress;
    const char *what = "wa_compress_kv(tcgen05)";
    const int cols = H * D;
    CUtensorMap tk, tv, tek, tev, tdk, tdv;
    bool good = map_rows(&tk, k->ptr, cols, L, B, k->stride_l, k->stride_b) && map_rows(&tv, v->ptr, cols, L, B, v->stride_l, v->stride_b);
    const int e_tokens = proj_cols < segment_len ? proj_cols : segment_len;
    good = good && map_projection(&tek, k_proj, e_tokens, proj_rank, proj_cols) && map_projection(&tev, v_proj, e_tokens, proj_rank, proj_cols);
    const bool copy = dst_k != nullptr;
    if (copy) {
        char *bk = (char *)dst_k->ptr + (size_t)dst_row0 * dst_k->stride_l * 2, *bv = (char *)dst_v->ptr + (size_t)dst_row0 * dst_v->stride_l * 2;
        good = good && map_rows(&tdk, bk, cols, L, B, dst_k->stride_l, dst_k->stride_b) &&
               map_rows(&tdv, bv, cols, L, B, dst_v->stride_l, dst_v->stride_b);
    } else {
        tdk = tk;
        tdv = tv;
    }
    WA_REQUIRE(good, WA_ERR_ALIGN, "%s: a tensor map was rejected", what);
    static PerDeviceOnce attr_set;
    if (!attr_set.done()) {
        cudaError_t e = cudaFuncSetAttribute(compress_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
        attr_set.mark();
    }
    // the flag's device address, looked up once per device
    static int *status_of[64] = {nullptr};
    int dev_now = 0;
    if (cudaGetDevice(&dev_now) != cudaSuccess || dev_now < 0 || dev_now >= 64) return fail(WA_ERR_DEVICE, "%s: no usable current device", what);
    if (!status_of[dev_now]) {
        cudaError_t e = cudaGetSymbolAddress((void **)&status_of[dev_now], g_status);
        if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
    }
    int *status = status_of[dev_now];
    Job job{};
    job.n_seg = ceil_div(L, segment_len);
    job.tiles_cols = cols / sm100::TILE;
    job.B = B;
    job.L = L; job.segment_len = segment_len; job.block_size = block_size; job.proj_rank = proj_rank;
    job.slot0 = slot0; job.slot_stride = slot_stride;
    job.copy = copy ? 1 : 0;
    job.out_k = (__nv_bfloat16 *)ok->ptr; job.out_v = (__nv_bfloat16 *)ov->ptr;
    job.osb = ok->stride_b; job.osl = ok->stride_l;
    job.status = status;
    const long long items = (long long)B * 2 * job.n_seg * job.tiles_cols;
    WA_REQUIRE(items < (1ll << 30), WA_ERR_UNSUPPORTED, "%s: too many work items", what);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    const int grid = items < sms ? (int)items : sms;
    compress_stream_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tk, tv, tek, tev, tdk, tdv, job);
    return check_launch(what);
}

}  // namespace wa

extern "C" int wa_compress_status(int *status) {
    using namespace wa;
    WA_REQUIRE(status, WA_ERR_ARG, "wa_compress_status: null pointer");
    cudaError_t e = cudaMemcpyFromSymbol(status, sm100::compress::g_status, sizeof(int));
    if (e != cudaSuccess) return fail((int)e, "wa_compress_status: %s", cudaGetErrorString(e));
    return 0;
}
