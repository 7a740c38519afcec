// Block-mean pooling as a TMA stream for sm_100a (bf16 rows with contiguous heads).
//
// block_mean_pool (wan/modules/hsa/routing.py:45-61) reads Q and K once and writes one float32 row per
// (block, head); at 32K tokens that is 115 MB in and 1.8 MB out, so the kernel is an HBM stream.  A persistent
// CTA keeps a ring of boxes [32 tokens x 256 columns] in flight with TMA (one instruction per 16 KB instead of
// hundreds of per-thread loads).  A work item is one routing block x 256 columns; a group of four warps owns an
// item, each thread two neighbouring columns of it, so no sum crosses a thread.  The rows are added in float64:
// a sum of a few hundred bf16 values is exact there, so the pooled value, and the discrete routing decision that
// is taken on it, do not depend on the order of the additions.  The float64 conversion is what bounds the
// arithmetic (16 per clock per SM); three groups with four boxes in flight each measured fastest (22.5 us for 100 MB, 4.5 TB/s).
#include "wa_internal.cuh"
#include "wa_sm100_ptx.cuh"

namespace wa {
namespace sm100 {
namespace pool {

constexpr int COLS = 256;            // columns of a work item: one 512-byte row piece per token
constexpr int SUB_ROWS = 32;         // token rows of one TMA box: 16 KB
constexpr int STAGE_BYTES = SUB_ROWS * COLS * 2;
#ifndef WA_POOLT_GROUPS
#define WA_POOLT_GROUPS 3
#endif
constexpr int GROUPS = WA_POOLT_GROUPS, GROUP_THREADS = COLS / 2;   // a thread owns two neighbouring columns of its group's item
constexpr int THREADS = 32 + GROUPS * GROUP_THREADS;                // warp 0 issues the loads
// Every group has a ring of its own.  With one ring shared by all groups a group could be asked for a box two laps
// ahead of a slower group's, and a phase-parity wait cannot tell "two laps behind" from "done".
constexpr int STAGES = 12 / GROUPS;                                 // boxes in flight per group
constexpr int SMEM_BYTES = GROUPS * STAGES * STAGE_BYTES + 1024;

struct Barriers {
    uint64_t full[GROUPS][STAGES], empty[GROUPS][STAGES];
    int abort_flag;
};

struct Job {
    // two tensors pooled by one launch: x (queries) then y (keys); items = (tensor, batch, block, column tile), tile fastest
    int B, H, D, block_size, tiles;          // tiles = H * D / 256
    int Lx, nbx, Ly, nby, out_blocks_y;      // out_blocks_y: rows per (batch, head) of the y output buffer
    float *px, *py;
    int *zero;
    int n_zero;
    int *status, *status_mirror;
};

__device__ int g_status;

// The row pieces of a box are 512 bytes wide on purpose: the copy engine issues one request per row piece, and with
// 128-byte pieces (64 columns) that request rate, not HBM, bounded the stream at 2.7 TB/s.
__global__ void __launch_bounds__(THREADS, 1)
pool_stream_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_y, const Job job) {
    extern __shared__ __align__(1024) uint8_t smem[];
    Barriers *bar = reinterpret_cast<Barriers *>(smem + GROUPS * STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &bar->abort_flag;
    const FailSink sink{job.status, job.status_mirror};

    if (threadIdx.x == 0) {
        bar->abort_flag = 0;
        for (int i = 0; i < GROUPS * STAGES; ++i) {
            mbar_init(&bar->full[0][i], 1);
            mbar_init(&bar->empty[0][i], GROUP_THREADS / 32);   // one arrival per warp of the group that read the box
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (job.n_zero && blockIdx.x == 0)   // counters of the kernel that follows on the stream
        for (int i = threadIdx.x; i < job.n_zero; i += THREADS) job.zero[i] = 0;
    __syncthreads();

    const long long items_x = (long long)job.B * job.nbx * job.tiles;
    const long long items = items_x + (long long)job.B * job.nby * job.tiles;
    const int subs = job.block_size / SUB_ROWS;      // boxes per item

    if (warp == 0) {
        if (lane == 0) {
            uint32_t n_item = 0;   // items of this CTA so far: item n goes to group n % GROUPS as its (n / GROUPS)-th
            for (long long item = blockIdx.x; item < items; item += gridDim.x, ++n_item) {
                const bool second = item >= items_x;
                const long long it = second ? item - items_x : item;
                const int nb_all = second ? job.nby : job.nbx;
                const int ct = (int)(it % job.tiles), nb = (int)((it / job.tiles) % nb_all), b = (int)(it / ((long long)job.tiles * nb_all));
                const uint32_t g = n_item % GROUPS;
                for (int sub = 0; sub < subs; ++sub) {
                    const uint32_t count = (n_item / GROUPS) * subs + sub, s = count % STAGES;
                    if (!mbar_wait(&bar->empty[g][s], ((count / STAGES) & 1u) ^ 1u, abort_flag, sink, 201)) return;   // 201, 202: wait sites of this kernel in the status word
                    mbar_expect_tx(&bar->full[g][s], (uint32_t)STAGE_BYTES);
                    // rows past the end of the tensor arrive as zeros
                    tma_load_3d(smem + (g * STAGES + s) * STAGE_BYTES, second ? &tm_y : &tm_x, &bar->full[g][s], ct * COLS,
                                nb * job.block_size + sub * SUB_ROWS, b);
                }
            }
        }
        return;
    }

    // ---- consumers: group g takes the CTA's items g, g + GROUPS, ...; no thread of it shares a column with another ----
    const int gid = (warp - 1) / (GROUP_THREADS / 32), t = threadIdx.x - 32 - gid * GROUP_THREADS;
    uint32_t n_item = 0;
    for (long long item = blockIdx.x; item < items; item += gridDim.x, ++n_item) {
        if ((int)(n_item % GROUPS) != gid) continue;
        const bool second = item >= items_x;
        const long long it = second ? item - items_x : item;
        const int nb_all = second ? job.nby : job.nbx, L = second ? job.Ly : job.Lx;
        const int ct = (int)(it % job.tiles), nb = (int)((it / job.tiles) % nb_all), b = (int)(it / ((long long)job.tiles * nb_all));
        double lo[4] = {0.0, 0.0, 0.0, 0.0}, hi[4] = {0.0, 0.0, 0.0, 0.0};   // four chains per column: additions of one chain wait on each other
        bool ok = true;
        for (int sub = 0; sub < subs; ++sub) {
            const uint32_t count = (n_item / GROUPS) * subs + sub, s = count % STAGES;
            ok = mbar_wait(&bar->full[gid][s], (count / STAGES) & 1u, abort_flag, sink, 202);
            if (!ok) break;
            const uint32_t *box = reinterpret_cast<const uint32_t *>(smem + (gid * STAGES + s) * STAGE_BYTES) + t;
#pragma unroll
            for (int r = 0; r < SUB_ROWS; r += 4) {
                uint32_t w[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) w[c] = box[(r + c) * (COLS / 2)];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    lo[c] += (double)__uint_as_float(w[c] << 16);
                    hi[c] += (double)__uint_as_float(w[c] & 0xffff0000u);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar->empty[gid][s]);
        }
        if (!ok) break;
        const double s0 = (lo[0] + lo[1]) + (lo[2] + lo[3]), s1 = (hi[0] + hi[1]) + (hi[2] + hi[3]);
        const int n_real = min(job.block_size, L - nb * job.block_size);
        float2 out;
        if (L % job.block_size == 0) {
            out.x = bf16_round_f((float)(s0 / (double)job.block_size));
            out.y = bf16_round_f((float)(s1 / (double)job.block_size));
        } else {
            out.x = __fdiv_rn(bf16_round_f((float)s0), (float)n_real);
            out.y = __fdiv_rn(bf16_round_f((float)s1), (float)n_real);
        }
        const int col = ct * COLS + 2 * t, h = col / job.D, d = col % job.D;
        float *dst = second ? job.py : job.px;
        const int out_blocks = second ? job.out_blocks_y : job.nbx;
        *reinterpret_cast<float2 *>(dst + (((long long)b * job.H + h) * out_blocks + nb) * (long long)job.D + d) = out;
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

static bool map_rows(CUtensorMap *map, const wa_tensor4 *x, int cols, int rows, int B) {
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)B};
    cuuint64_t strides[2] = {(cuuint64_t)x->stride_l * 2, (cuuint64_t)(B == 1 ? x->stride_l * (long long)rows : x->stride_b) * 2};
    cuuint32_t box[3] = {(cuuint32_t)COLS, (cuuint32_t)SUB_ROWS, 1}, elem[3] = {1, 1, 1};
    return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, x->ptr, dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace pool
}  // namespace sm100

bool pool_sm100_supported(const wa_tensor4 *x, const wa_tensor4 *y, int H, int D, int block_size) {
    using namespace sm100::pool;
    for (const wa_tensor4 *t : {x, y}) {
        if (!t) continue;
        if (t->dtype != WA_BF16 || t->stride_h != D || (uintptr_t)t->ptr % 16 || t->stride_l % 8 || t->stride_b % 8 ||
            t->stride_l < (long long)H * D)
            return false;
    }
    if ((H * D) % COLS || D % 2 || block_size % SUB_ROWS || block_size > 8 * SUB_ROWS) return false;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        major != 10)
        return false;
    return encode_fn() != nullptr;
}

int pool_sm100_launch(const wa_tensor4 *x, int Lx, float *px, const wa_tensor4 *y, int Ly, float *py, int out_blocks_y, int B, int H,
                      int D, int block_size, cudaStream_t stream, int *zero, int n_zero, int *status_mirror) {
    using namespace sm100::pool;
    const char *what = "wa_pool_blocks(tma)";
    CUtensorMap tx, ty;
    bool good = map_rows(&tx, x, H * D, Lx, B);
    good = good && (y ? map_rows(&ty, y, H * D, Ly, B) : true);
    WA_REQUIRE(good, WA_ERR_ALIGN, "%s: a tensor map was rejected", what);
    if (!y) ty = tx;
    static PerDeviceOnce attr_set;
    if (!attr_set.done()) {
        cudaError_t e = cudaFuncSetAttribute(pool_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
        attr_set.mark();
    }
    static int *status_of[64] = {nullptr};
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(WA_ERR_DEVICE, "%s: no usable current device", what);
    if (!status_of[dev]) {
        cudaError_t e = cudaGetSymbolAddress((void **)&status_of[dev], g_status);
        if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
    }
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    Job job{};
    job.B = B; job.H = H; job.D = D; job.block_size = block_size; job.tiles = H * D / COLS;
    job.Lx = Lx; job.nbx = ceil_div(Lx, block_size);
    job.Ly = y ? Ly : 0; job.nby = y ? ceil_div(Ly, block_size) : 0; job.out_blocks_y = out_blocks_y;
    job.px = px; job.py = py; job.zero = zero; job.n_zero = n_zero; job.status = status_of[dev]; job.status_mirror = status_mirror;
    const long long items = (long long)B * (job.nbx + job.nby) * job.tiles;
    WA_REQUIRE(items < (1ll << 40), WA_ERR_UNSUPPORTED, "%s: too many blocks", what);
    const int grid = items < sms ? (int)items : sms;
    pool_stream_kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(tx, ty, job);
    return check_launch(what);
}

}  // namespace wa
