// Fused HSA forward for sm_100a: block-sparse softmax branch, compressed ("linear") branch, gate
// GEMM and combine in one persistent, warp-specialised kernel.
//
// Replaces the reference's Triton `_fwd_kernel` (wan/modules/hsa/block_sparse_triton.py:67-139)
// plus `_linear_branch` and the gate/addcmul epilogue (wan/modules/hsa/attention.py:113-118,
// 246-259) for bf16, head_dim 128, 128- or 64-token routing blocks.
//
// Work item = (batch, head, query block).  Per item the CTA runs a chain of 128x128 tiles:
//   sparse:  for each selected key block   S = Q K^T -> online softmax -> O += P V
//   linear:  for each 128 compressed slots  S = Q Kc^T -> online softmax -> O += P Vc
//   gate:    S = Q Wg^T ; out = O_sparse/l_s + sigmoid(S + b) * O_linear/l_l
// Data path: TMA (cp.async.bulk.tensor, 128-byte swizzle, one consumer CTA per copy) -> shared memory ->
// tcgen05.mma with the S and O accumulators in tensor memory; P goes back to tensor memory as
// bf16 and is the A operand of the PV product.  One persistent CTA of 12 warps per SM owns all 512
// tensor-memory columns (three S buffers + O) and ~227 KB of shared memory (Q x2, K x3, V x2 tiles):
// warps 0-7 do the softmax and the epilogue (a query row is shared by four lanes of one warp, a tile's
// columns by two warps), warp 8 issues TMA loads, warp 9 the QK products, warp 11 the PV products and
// warp 10 the TMA store of the finished tile.  Items are taken heaviest first from a global counter.
//
// Every mbarrier wait is bounded (about two seconds); on expiry the kernel raises a flag in
// global memory, all roles leave their loops, tensor memory is released and the kernel returns.
#include <climits>
#include <cstdlib>

#include "wa_internal.cuh"
#include "wa_sm100_ptx.cuh"

namespace wa {
namespace sm100 {

constexpr int THREADS = 384;         // warps 0..7 softmax (two threads per query row), warp 8 TMA, warp 9 QK products, warp 10 output store, warp 11 PV products
constexpr int REGS_SOFTMAX = 224;    // register budget per thread after the roles split (two warpgroups of softmax warps)
constexpr int REGS_OTHER = 56;       // ... and of the warpgroup that holds the four single-purpose warps; 256*224 + 128*56 = 384*168
constexpr int TMEM_COLS = 512;       // three S buffers: columns [0,128), [128,256), [256,384); O: [384,512)
constexpr int S_BUFS = 3;            // score products run up to two tiles ahead of the softmax
constexpr int Q_STAGES = 2;          // the staged output of item j leaves from one Q buffer while item j+1 loads the other
constexpr int KV_STAGES = 3;         // shared-memory ring depth for K tiles
constexpr int V_STAGES = 2;          // shared-memory ring depth for V tiles
constexpr int SMEM_BYTES = (Q_STAGES + KV_STAGES + V_STAGES) * TILE_BYTES + 3072 /*barriers, bias*/;

// Optional event trace for kernel tuning (compile with -DWA_SM100_TRACE): CTA 0 appends
// (event id, clock) pairs from one thread per role to a global buffer.
#ifdef WA_SM100_TRACE
constexpr int TRACE_SLOTS = 8192;            // (id, clock) pairs per traced role
__device__ long long g_trace[4][2 * TRACE_SLOTS];
__device__ int g_trace_n[4];
#define WA_TRACE_ROLE ((threadIdx.x >> 5) == 0 ? 2 : (threadIdx.x >> 5) == 8 ? 0 : (threadIdx.x >> 5) == 9 ? 1 : (threadIdx.x >> 5) == 11 ? 3 : 4)
__device__ long long g_cta_stats[1024][6];
__device__ __forceinline__ unsigned long long wa_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned wa_smid() {
    unsigned r;
    asm volatile("mov.u32 %0, %smid;" : "=r"(r));
    return r;
}
#define WA_TRACE_DECL int trace_at = 0; long long st_items = 0, st_tiles = 0; const unsigned long long st_t0 = wa_globaltimer(); const long long st_c0 = clock64()
#define WA_STATS_ITEM(n) do { st_items += 1; st_tiles += (n); } while (0)
#define WA_TRACE(id)                                                                         \
    do {                                                                                     \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && WA_TRACE_ROLE <= 3 &&              \
            trace_at < TRACE_SLOTS) {                                                        \
            g_trace[WA_TRACE_ROLE][2 * trace_at] = (id);                                     \
            g_trace[WA_TRACE_ROLE][2 * trace_at + 1] = clock64();                            \
            ++trace_at;                                                                      \
        }                                                                                    \
    } while (0)
#define WA_TRACE_FLUSH                                                                       \
    do {                                                                                     \
        if (threadIdx.x == 0 && blockIdx.x < 1024) {                                         \
            g_cta_stats[blockIdx.x][0] = wa_smid();                                          \
            g_cta_stats[blockIdx.x][1] = (long long)st_t0;                                   \
            g_cta_stats[blockIdx.x][2] = (long long)wa_globaltimer();                        \
            g_cta_stats[blockIdx.x][3] = st_items;                                           \
            g_cta_stats[blockIdx.x][4] = st_tiles;                                           \
            g_cta_stats[blockIdx.x][5] = clock64() - st_c0;                                  \
        }                                                                                    \
        if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && WA_TRACE_ROLE <= 3)                \
            g_trace_n[WA_TRACE_ROLE] = trace_at;                                             \
    } while (0)
#else
#define WA_TRACE_DECL
#define WA_STATS_ITEM(n) do { } while (0)
#define WA_TRACE(id) do { } while (0)
#define WA_TRACE_FLUSH do { } while (0)
#endif

struct Barriers {
    uint64_t item_full[2], item_empty[2];
    uint64_t q_full[Q_STAGES], q_empty[Q_STAGES], out_ready[Q_STAGES];
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES], v_full[V_STAGES], v_empty[V_STAGES];
    // K-type tile g (global count) lives in S buffer g % S_BUFS; it is that buffer's occupancy number g / S_BUFS, which
    // is the phase of s_full / p_full the tile completes (every tile completes exactly one phase of each).
    uint64_t s_full[S_BUFS], p_full[S_BUFS];
    uint64_t s_free[S_BUFS];   // the PV product that read P from the buffer has landed
    uint64_t o_done, o_free;   // v_empty[s] doubles as "PV product done" for the rescale path
    uint32_t tmem_base;
    int abort_flag;
    ItemDesc items[2];
    int valid[8];            // real token count of the K-type tiles in flight, ring indexed by global tile number
    float bias[TILE];        // gate bias
};

static_assert(sizeof(Barriers) <= 3072, "barrier block exceeds its shared-memory budget");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget exceeded");

// ---- the kernel ----------------------------------------------------------------------------------
// The three roles run their own loops over work items and meet only at mbarriers, so the producer
// prefetches the next item's Q/K/V and the MMA warp starts its first products while the softmax
// warps are still in the previous item's epilogue.
template <int BLK>   // routing block size: 128, or 64 (see Params::blk)
__global__ void __launch_bounds__(THREADS, 1)
hsa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                     const __grid_constant__ CUtensorMap tm_vc, const __grid_constant__ CUtensorMap tm_w,
                     const __grid_constant__ CUtensorMap tm_out, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];   // swizzled TMA tiles need 1024-byte alignment (checked below)
    uint8_t *q_s = smem, *k_s = smem + Q_STAGES * TILE_BYTES, *v_s = smem + (Q_STAGES + KV_STAGES) * TILE_BYTES;
    Barriers *bar = reinterpret_cast<Barriers *>(smem + (Q_STAGES + KV_STAGES + V_STAGES) * TILE_BYTES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &bar->abort_flag;
    const FailSink sink{p.error_flag, p.status_mirror};

    if (threadIdx.x == 0) {
        bar->abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;   // misaligned shared memory: give up before any TMA
        if (bar->abort_flag) report_failure(sink, 99);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar->item_full[i], 1);
            mbar_init(&bar->item_empty[i], 2 + 8 + 1);   // both MMA leaders + every softmax warp + store warp
        }
        for (int i = 0; i < S_BUFS; ++i) {
            mbar_init(&bar->s_full[i], 1);
            mbar_init(&bar->p_full[i], 8);   // one arrival per softmax warp
            mbar_init(&bar->s_free[i], 1);
        }
        for (int i = 0; i < Q_STAGES; ++i) {
            mbar_init(&bar->q_full[i], 1);
            mbar_init(&bar->q_empty[i], 1);
            mbar_init(&bar->out_ready[i], 8);
        }
        for (int i = 0; i < KV_STAGES; ++i) {
            mbar_init(&bar->k_full[i], 1);
            mbar_init(&bar->k_empty[i], 1);
        }
        for (int i = 0; i < V_STAGES; ++i) {
            mbar_init(&bar->v_full[i], 1);
            mbar_init(&bar->v_empty[i], 1);
        }
        mbar_init(&bar->o_done, 1);
        mbar_init(&bar->o_free, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // everything above is private to this CTA; from here on the routing kernel's results (work order, selection,
    // converted gate weights) are read, so the launch before this one has to be complete
    pdl_wait();
    if (threadIdx.x >= 64 && threadIdx.x < 64 + TILE) bar->bias[threadIdx.x - 64] = (p.has_gate && p.gate_bias) ? p.gate_bias[threadIdx.x - 64] : 0.f;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bar->tmem_base;
    const uint32_t tmem_s = tmem, tmem_o = tmem + S_BUFS * TILE;   // S buffer b at tmem_s + b * TILE
    WA_TRACE_DECL;
    WA_TRACE(0);
    const int lin_tiles = (p.Lc + TILE - 1) / TILE;

    // The softmax threads keep 64 scores, the packed probabilities and the parked sparse result in registers; the
    // other four warps need few.  Shift the register file accordingly (whole warpgroups, as the instruction requires).
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHER));
    if (warp == 8) {
        // ================= producer: work queue + TMA =================
        if (lane == 0) {
            uint32_t jcount = 0, kcount = 0, vcount = 0;
            bool ok = true;
            // Work queue: the first item of a CTA is fixed by its index (no round trip to the counter before the first
            // load); later items come from the counter, which is asked for the next position one item ahead.
            int at = blockIdx.x;
            while (ok) {
                const uint32_t slot = jcount & 1u;
                ok = mbar_wait(&bar->item_empty[slot], ((jcount >> 1) & 1u) ^ 1u, abort_flag, sink, 11);
                if (!ok) break;
                int item = -1, n_sel = 0;
                if (at < p.n_items) {
                    item = p.order[at];
                    n_sel = max(0, min(p.num[item], p.Nkv));
                }
                // the other roles count sparse TILES: with 64-token blocks a tile holds two selected blocks
                const int n_st = BLK == TILE ? n_sel : (n_sel + 1) >> 1;
                bar->items[slot].item = item;
                bar->items[slot].n_sel = n_st;
                mbar_arrive(&bar->item_full[slot]);
                if (item < 0) break;
                at = (int)gridDim.x + atomicAdd(p.work_counter, 1);   // consumed at the top of the next round
                const int qb = item % p.Nq, h = (item / p.Nq) % p.H, b = item / (p.Nq * p.H);
                const int32_t *ids = p.index + (long long)item * p.Nkv;
                const int n_kv = n_st + lin_tiles;
                WA_STATS_ITEM(n_kv + 1);

                const uint32_t qs = jcount % Q_STAGES;
                ok = mbar_wait(&bar->q_empty[qs], ((jcount / Q_STAGES) & 1u) ^ 1u, abort_flag, sink, 12);
                if (!ok) break;
                uint8_t *qdst = q_s + qs * TILE_BYTES;
                mbar_expect_tx(&bar->q_full[qs], TILE_BYTES);
                tma_load_4d(qdst, &tm_q, &bar->q_full[qs], 0, h, qb * BLK, b);
                tma_load_4d(qdst + HALF_BYTES, &tm_q, &bar->q_full[qs], 64, h, qb * BLK, b);

                // K tiles and V tiles advance on cursors of their own: the V ring is shallower and its stages come back
                // later (after the PV product), and a K load that queued behind a V wait would reach the QK warp late.
                int tv = 0;   // next V tile of this item
                auto load_v = [&]() {   // V tile tv into the next stage of its ring (the stage is free)
                    const uint32_t vs = vcount % V_STAGES;
                    ++vcount;
                    uint8_t *vdst = v_s + vs * TILE_BYTES;
                    mbar_expect_tx(&bar->v_full[vs], TILE_BYTES);
                    if (tv < n_st) {
                        if (BLK == TILE) {
                            const int id = max(0, min(ids[tv], p.Nkv - 1));
                            tma_load_4d(vdst, &tm_v, &bar->v_full[vs], 0, h, id * TILE, b);
                            tma_load_4d(vdst + HALF_BYTES, &tm_v, &bar->v_full[vs], 64, h, id * TILE, b);
                        } else {
                            const int id = max(0, min(ids[2 * tv], p.Nkv - 1));
                            const int id2 = 2 * tv + 1 < n_sel ? max(0, min(ids[2 * tv + 1], p.Nkv - 1)) : id;
                            tma_load_4d(vdst, &tm_v, &bar->v_full[vs], 0, h, id * HALF, b);
                            tma_load_4d(vdst + HALF_BYTES / 2, &tm_v, &bar->v_full[vs], 0, h, id2 * HALF, b);
                            tma_load_4d(vdst + HALF_BYTES, &tm_v, &bar->v_full[vs], 64, h, id * HALF, b);
                            tma_load_4d(vdst + HALF_BYTES + HALF_BYTES / 2, &tm_v, &bar->v_full[vs], 64, h, id2 * HALF, b);
                        }
                    } else {
                        const int c = (tv - n_st) * TILE;
                        tma_load_4d(vdst, &tm_vc, &bar->v_full[vs], 0, h, c, b);
                        tma_load_4d(vdst + HALF_BYTES, &tm_vc, &bar->v_full[vs], 64, h, c, b);
                    }
                    ++tv;
                };
                auto v_free = [&]() { return mbar_test(&bar->v_empty[vcount % V_STAGES], ((vcount / V_STAGES) & 1u) ^ 1u); };

                for (int t = 0; t <= n_kv && ok; ++t) {
                    const uint32_t ks = kcount % KV_STAGES, kpar = ((kcount / KV_STAGES) & 1u) ^ 1u;
                    // wait for the K stage; V tiles whose K tile is out already go out as their stages come back
                    if (!mbar_test(&bar->k_empty[ks], kpar)) {
                        const long long w0 = clock64();
                        while (ok) {
                            if (tv < t && v_free()) load_v();
                            if (tv >= t) {   // nothing else to feed
                                ok = mbar_wait(&bar->k_empty[ks], kpar, abort_flag, sink, 1);
                                break;
                            }
                            if (mbar_try_wait_ns(&bar->k_empty[ks], kpar, 200u)) break;
                            if (*abort_flag) ok = false;
                            else if (clock64() - w0 > WAIT_CYCLES) {
                                *abort_flag = 1;
                                report_failure(sink, 1);
                                ok = false;
                            }
                        }
                        if (!ok) break;
                    }
                    uint8_t *kdst = k_s + ks * TILE_BYTES;
                    // real tokens of the tile: low byte = of its first 64 keys, next byte = of its last 64
                    int id = 0, id2 = 0, valid = 0;
                    if (t < n_st) {
                        if (BLK == TILE) {
                            id = max(0, min(ids[t], p.Nkv - 1));
                            const int n = min(TILE, p.Lkv - id * TILE);
                            valid = min(n, HALF) | (max(0, n - HALF) << 8);
                        } else {   // two 64-token blocks; a missing second block repeats the first and is masked out
                            id = max(0, min(ids[2 * t], p.Nkv - 1));
                            const bool two = 2 * t + 1 < n_sel;
                            id2 = two ? max(0, min(ids[2 * t + 1], p.Nkv - 1)) : id;
                            valid = min(HALF, p.Lkv - id * HALF) | ((two ? min(HALF, p.Lkv - id2 * HALF) : 0) << 8);
                        }
                    } else {
                        const int n = max(0, min(TILE, p.Lc - (t - n_st) * TILE));
                        valid = min(n, HALF) | (max(0, n - HALF) << 8);
                    }
                    bar->valid[kcount & 7] = valid;
                    ++kcount;
                    mbar_expect_tx(&bar->k_full[ks], TILE_BYTES);
                    if (t < n_st) {
                        if (BLK == TILE) {
                            tma_load_4d(kdst, &tm_k, &bar->k_full[ks], 0, h, id * TILE, b);
                            tma_load_4d(kdst + HALF_BYTES, &tm_k, &bar->k_full[ks], 64, h, id * TILE, b);
                        } else {   // 64-row boxes: rows 0..63 of each half-tile from the first block, 64..127 from the second
                            tma_load_4d(kdst, &tm_k, &bar->k_full[ks], 0, h, id * HALF, b);
                            tma_load_4d(kdst + HALF_BYTES / 2, &tm_k, &bar->k_full[ks], 0, h, id2 * HALF, b);
                            tma_load_4d(kdst + HALF_BYTES, &tm_k, &bar->k_full[ks], 64, h, id * HALF, b);
                            tma_load_4d(kdst + HALF_BYTES + HALF_BYTES / 2, &tm_k, &bar->k_full[ks], 64, h, id2 * HALF, b);
                        }
                    } else if (t < n_kv) {
                        const int c = (t - n_st) * TILE;
                        tma_load_4d(kdst, &tm_kc, &bar->k_full[ks], 0, h, c, b);
                        tma_load_4d(kdst + HALF_BYTES, &tm_kc, &bar->k_full[ks], 64, h, c, b);
                    } else {
                        tma_load_2d(kdst, &tm_w, &bar->k_full[ks], 0, 0);
                        tma_load_2d(kdst + HALF_BYTES, &tm_w, &bar->k_full[ks], 64, 0);
                    }
                    while (tv <= t && tv < n_kv && v_free()) load_v();
                }
                // the item's remaining V tiles, in order
                while (ok && tv < n_kv) {
                    ok = mbar_wait(&bar->v_empty[vcount % V_STAGES], ((vcount / V_STAGES) & 1u) ^ 1u, abort_flag, sink, 2);
                    if (ok) load_v();
                }
                ++jcount;
            }
        }
    } else if (warp == 9) {
        // ================= QK issuer =================
        // Two warps issue tensor-core work: this one the score products Q.K^T (and the gate product), warp 11 the
        // P.V products.  One thread blocks for about as long as its products execute, so a single issuer leaves the
        // pipe idle during its own waits and commits; two issuers cover each other.  Score products run up to two
        // tiles ahead of the softmax (three S buffers).  Products of different warps are ordered by completion
        // barriers only.  The whole warp runs the role so that operands stay warp-uniform; one elected lane issues.
        const bool leader = elect_one();
        constexpr uint32_t IDESC_QK = instr_desc(false, TILE);
        uint32_t jcount = 0, kcount = 0;
        uint32_t occ_pv = 0, occ_gate = 0;   // bit b: S buffer b last held a PV tile / a gate tile
        uint32_t ph_sf = 0;                  // bit b: parity of the next s_free[b] phase to wait for
        bool ok = true;

        auto issue_qk = [&](uint64_t qd, bool is_gate) -> bool {
            const uint32_t buf = kcount % S_BUFS;
            // the K tile first: it is there long before the S buffer comes back, so that nothing but the fence and the
            // products themselves stand between that and the scores
            const uint32_t ks = kcount % KV_STAGES, kpar = (kcount / KV_STAGES) & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(&bar->k_full[ks], kpar, abort_flag, sink, 4))) return false;
            if (occ_gate & (1u << buf)) {
                // the epilogue has read the gate scores of tile kcount - S_BUFS out of this buffer
                if (!__all_sync(0xffffffffu, mbar_wait(&bar->p_full[buf], ((kcount - S_BUFS) / S_BUFS) & 1u, abort_flag, sink, 13)))
                    return false;
            } else if (occ_pv & (1u << buf)) {
                // the PV product that read P from this buffer has landed
                if (!__all_sync(0xffffffffu, mbar_wait(&bar->s_free[buf], (ph_sf >> buf) & 1u, abort_flag, sink, 19)))
                    return false;
                ph_sf ^= 1u << buf;
            }
            occ_gate &= ~(1u << buf);
            occ_pv &= ~(1u << buf);
            ++kcount;
            WA_TRACE(1);
            tc_fence_after();
            if (leader) {
                const uint64_t kd = smem_desc(smem_u32(k_s + ks * TILE_BYTES), 16, 1024);
                const uint32_t d = tmem_s + buf * TILE;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4);
                    mma_ss(d, qd + off, kd + off, IDESC_QK, kk > 0);
                }
                tc_commit(&bar->s_full[buf]);   // the softmax waits for this one
                tc_commit(&bar->k_empty[ks]);
            }
            __syncwarp();
            if (is_gate) occ_gate |= 1u << buf;
            else occ_pv |= 1u << buf;
            WA_TRACE(4);
            return true;
        };

        while (ok) {
            const uint32_t slot = jcount & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->item_full[slot], (jcount >> 1) & 1u, abort_flag, sink, 14));
            if (!ok) break;
            const int item = bar->items[slot].item, n_sel = bar->items[slot].n_sel;
            __syncwarp();
            if (leader) mbar_arrive(&bar->item_empty[slot]);
            if (item < 0) break;
            const int n_kv = n_sel + lin_tiles;   // K-type tiles 0 .. n_kv - 1 feed a PV product, tile n_kv is the gate
            const uint32_t qs = jcount % Q_STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->q_full[qs], (jcount / Q_STAGES) & 1u, abort_flag, sink, 3));
            if (!ok) break;
            const uint64_t qd = smem_desc(smem_u32(q_s + qs * TILE_BYTES), 16, 1024);
            for (int t = 0; t <= n_kv && ok; ++t) ok = issue_qk(qd, t == n_kv);
            ++jcount;
        }
    } else if (warp == 11) {
        // ================= PV issuer =================
        const bool leader = elect_one();
        constexpr uint32_t IDESC_PV = instr_desc(true, TILE);
        uint32_t jcount = 0, g = 0, vcount = 0, ph_of = 1;   // g: global K-type tile count; ph_of = 1: the first wait passes
        bool ok = true;
        while (ok) {
            const uint32_t slot = jcount & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->item_full[slot], (jcount >> 1) & 1u, abort_flag, sink, 20));
            if (!ok) break;
            const int item = bar->items[slot].item, n_sel = bar->items[slot].n_sel;
            __syncwarp();
            if (leader) mbar_arrive(&bar->item_empty[slot]);
            if (item < 0) break;
            const int n_kv = n_sel + lin_tiles;
            for (int t = 0; t < n_kv && ok; ++t, ++g) {
                const uint32_t buf = g % S_BUFS;
                const bool first = (t == 0) || (t == n_sel);
                // the V tile first (it lands long before the probabilities do)
                const uint32_t vs = vcount % V_STAGES, vpar = (vcount / V_STAGES) & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->v_full[vs], vpar, abort_flag, sink, 6));
                if (!ok) break;
                ++vcount;
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->p_full[buf], (g / S_BUFS) & 1u, abort_flag, sink, 5));
                if (!ok) break;
                WA_TRACE(5);
                if (first) {
                    // the accumulator of the previous branch (or item) must have been read out
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->o_free, ph_of, abort_flag, sink, 7));
                    if (!ok) break;
                    ph_of ^= 1u;
                }
                tc_fence_after();
                if (leader) {
                    const uint64_t vd = smem_desc(smem_u32(v_s + vs * TILE_BYTES), HALF_BYTES, 1024);
#pragma unroll
                    for (int kk = 0; kk < 8; ++kk)
                        mma_ts(tmem_o, tmem_s + buf * TILE + kk * 8, vd + (uint64_t)((kk * 2048) >> 4), IDESC_PV,
                               !(first && kk == 0));
                    tc_commit(&bar->s_free[buf]);   // first: the next score product waits for it
                    tc_commit(&bar->v_empty[vs]);   // frees the V stage; the rescale path reads it as "this product has landed"
                    if (t == n_sel - 1 || t == n_kv - 1) tc_commit(&bar->o_done);
                }
                __syncwarp();
                WA_TRACE(7);
            }
            ++g;   // the gate tile
            ++jcount;
        }
    } else if (warp == 10) {
        // ================= store warp: TMA store of the staged output tile, then release of the Q stage =========
        if (lane == 0) {
            uint32_t jcount = 0;
            bool ok = true;
            while (ok) {
                const uint32_t slot = jcount & 1u;
                ok = mbar_wait(&bar->item_full[slot], (jcount >> 1) & 1u, abort_flag, sink, 16);
                if (!ok) break;
                const int item = bar->items[slot].item;
                mbar_arrive(&bar->item_empty[slot]);
                if (item < 0) break;
                const int qb = item % p.Nq, h = (item / p.Nq) % p.H, b = item / (p.Nq * p.H);
                const uint32_t qs = jcount % Q_STAGES;
                ok = mbar_wait(&bar->out_ready[qs], (jcount / Q_STAGES) & 1u, abort_flag, sink, 17);
                if (!ok) break;
                if (!p.part_linear) {
                    // rows beyond q_len are clipped by the tensor map
                    // (with 64-token blocks the map's box is 64 rows: the tile's upper rows belong to the next item)
                    tma_store_4d(&tm_out, q_s + qs * TILE_BYTES, 0, h, qb * BLK, b);
                    tma_store_4d(&tm_out, q_s + qs * TILE_BYTES + HALF_BYTES, 64, h, qb * BLK, b);
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the Q stage is reusable afterwards
                }
                mbar_arrive(&bar->q_empty[qs]);
                ++jcount;
            }
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all stores have landed before the CTA exits
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
        // ================= softmax / epilogue: a quad of threads per query row =================
        // A warp may only touch the 32 tensor-memory lanes (rows) selected by warp % 4; warps w and w + 4 share that
        // row group and take 16 rows each.  Scores are read in the quad-row shape: thread t holds rows t/4 and t/4 + 8
        // of its 16 and, of each, the column pairs 8j + 2(t%4), +1 (32 columns per row).  A row therefore lives in
        // one quad of one warp: the row maximum and the row sum are two shuffles, no shared memory, no rendezvous of
        // warps -- the eight softmax warps run independently and drift apart, so the arithmetic of one covers the
        // tensor-memory round trips and barrier waits of the other on the same scheduler.
        const int rg = warp & 3, hb = warp >> 2;            // row group (32 rows), 16-row half inside it
        const int g = lane >> 2, c2 = lane & 3;
        const int rowA = rg * 32 + hb * 16 + g, rowB = rowA + 8;
        const uint32_t lane_addr = ((uint32_t)(rg * 32 + hb * 16)) << 16;
        uint32_t jcount = 0, sg = 0;       // items and K-type tiles seen so far
        uint32_t ph_od = 0;
        uint32_t pv_count = 0;             // PV products requested so far
        bool ok = true;
        const float2 sc = make_float2(p.scale_log2, p.scale_log2);

        while (ok) {
            const uint32_t slot = jcount & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->item_full[slot], (jcount >> 1) & 1u, abort_flag, sink, 15));
            if (!ok) break;
            const int item = bar->items[slot].item, n_sel = bar->items[slot].n_sel;
            warp_arrive(&bar->item_empty[slot]);
            if (item < 0) break;
            const int qb = item % p.Nq, h = (item / p.Nq) % p.H, b = item / (p.Nq * p.H);
            const int n_kv = n_sel + lin_tiles;
            const uint32_t qs = jcount % Q_STAGES;
            uint8_t *q_stage = q_s + qs * TILE_BYTES;
            const int tokenA = qb * BLK + rowA, tokenB = tokenA + 8;
            const bool okA = rowA < BLK && tokenA < p.Lq, okB = rowB < BLK && tokenB < p.Lq;
            // float32 offsets of the rows' normalisers
            long long lseA = (long long)b * p.lse_sb + (long long)h * p.lse_sh + (long long)tokenA * p.lse_st, lseB = lseA + 8 * p.lse_st;
            if (p.peer_rows > 0) {
                // the rank that merges a query row receives it directly (plain stores into its buffer, over NVLink for
                // another GPU): row t is rank t / peer_rows' row peer_self * peer_rows + t % peer_rows
                const int dA = min(tokenA / p.peer_rows, 7), dB = min(tokenB / p.peer_rows, 7);
                const long long rA = (long long)p.peer_self * p.peer_rows + (tokenA - dA * p.peer_rows);
                const long long rB = (long long)p.peer_self * p.peer_rows + (tokenB - dB * p.peer_rows);
                lseA = (long long)h * p.lse_sh + rA * p.lse_st + p.peer_delta[dA];
                lseB = (long long)h * p.lse_sh + rB * p.lse_st + p.peer_delta[dB];
            }
            const int gbuf = (sg + n_kv) % S_BUFS;
            float inv_linA = 0.f, inv_linB = 0.f, inv_spA = 0.f, inv_spB = 0.f;
            // The sparse branch's result, parked until the item's end.  Combined output: park word 2j = row A, 2j + 1 = row B,
            // bf16 pair of step j (gpk then holds the gate values in the same form).  Partial-output mode: float32, park
            // words 2j, 2j + 1 = row A's column pair of step j, gpk the same of row B.
            uint32_t park[32], gpk[32];
            float ls_spA = 0.f, ls_spB = 0.f;   // the sparse branch's log-sum-exp (packed records write both in one store)

            for (int phase = 0; phase < 2 && ok; ++phase) {
                const int t0 = phase == 0 ? 0 : n_sel, t1 = phase == 0 ? n_sel : n_kv;
                float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;   // l: this thread's columns only
                for (int t = t0; t < t1 && ok; ++t) {
                    const int buf = (sg + t) % S_BUFS;
                    const uint32_t s_addr = tmem_s + buf * TILE + lane_addr;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_full[buf], ((sg + t) / S_BUFS) & 1u, abort_flag, sink, 8));
                    if (!ok) break;
                    WA_TRACE(2);
                    tc_fence_after();
                    // real tokens of the tile's first and last 64 keys (the producer wrote the counts); key column c is real
                    // when c < v0 (c < 64) or c - 64 < v1: per 8-column step j that is c < lim(j)
                    const int vword = bar->valid[(sg + t) & 7];
                    const int v0 = vword & 0xff, v1 = (vword >> 8) & 0xff;
                    const bool full = vword == (HALF | (HALF << 8));
                    const int lim_lo = v0, lim_hi = HALF + v1;
                    uint32_t r[64];
                    TMEM_LDQ64(s_addr, r);
                    tmem_wait_ld();
                    float xa0 = -INFINITY, xa1 = -INFINITY, xb0 = -INFINITY, xb1 = -INFINITY;
                    if (full) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            xa0 = fmaxf(xa0, __uint_as_float(r[4 * j]));
                            xa1 = fmaxf(xa1, __uint_as_float(r[4 * j + 1]));
                            xb0 = fmaxf(xb0, __uint_as_float(r[4 * j + 2]));
                            xb1 = fmaxf(xb1, __uint_as_float(r[4 * j + 3]));
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int col = 8 * j + 2 * c2, lim = j < 8 ? lim_lo : lim_hi;
                            if (col < lim) {
                                xa0 = fmaxf(xa0, __uint_as_float(r[4 * j]));
                                xb0 = fmaxf(xb0, __uint_as_float(r[4 * j + 2]));
                            }
                            if (col + 1 < lim) {
                                xa1 = fmaxf(xa1, __uint_as_float(r[4 * j + 1]));
                                xb1 = fmaxf(xb1, __uint_as_float(r[4 * j + 3]));
                            }
                        }
                    }
                    const float mxA = quad_max(fmaxf(xa0, xa1)) * p.scale_log2, mxB = quad_max(fmaxf(xb0, xb1)) * p.scale_log2;
                    WA_TRACE(8);
                    // lazy rescale: only when a running maximum grows by more than 2^8
                    float mA_new = mA, mB_new = mB;
                    const bool growA = mxA > mA + 8.0f, growB = mxB > mB + 8.0f;
                    if (growA) mA_new = mxA;
                    if (growB) mB_new = mxB;
                    if (__any_sync(0xffffffffu, (growA || growB) && t > t0)) {
                        // every PV requested so far must have landed before the accumulator is touched
                        ok = __all_sync(0xffffffffu, mbar_wait(&bar->v_empty[(pv_count - 1u) % V_STAGES],
                                                               ((pv_count - 1u) / V_STAGES) & 1u, abort_flag, sink, 9));
                        if (!ok) break;
                        tc_fence_after();
                        const float fA = (growA && t > t0) ? ex2(mA - mA_new) : 1.0f, fB = (growB && t > t0) ? ex2(mB - mB_new) : 1.0f;
                        lA *= fA;
                        lB *= fB;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                            uint32_t ro[16];
                            TMEM_LDQ16(tmem_o + lane_addr + c * 32, ro);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                ro[4 * j] = __float_as_uint(__uint_as_float(ro[4 * j]) * fA);
                                ro[4 * j + 1] = __float_as_uint(__uint_as_float(ro[4 * j + 1]) * fA);
                                ro[4 * j + 2] = __float_as_uint(__uint_as_float(ro[4 * j + 2]) * fB);
                                ro[4 * j + 3] = __float_as_uint(__uint_as_float(ro[4 * j + 3]) * fB);
                            }
                            TMEM_STQ16(tmem_o + lane_addr + c * 32, ro);
                        }
                        tmem_wait_st();
                    }
                    mA = mA_new;
                    mB = mB_new;
                    // p = 2^(s*c - m), row sums, pack to bf16, write P over the consumed S columns
                    uint32_t pk[32];
                    const float2 nmA = make_float2(-mA, -mA), nmB = make_float2(-mB, -mB);
                    float2 accA = make_float2(0.f, 0.f), accB = make_float2(0.f, 0.f);
                    if (full) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (j % POLY_EVERY == 0)
                                exp_step<true, false>(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3], sc, nmA, nmB, accA, accB,
                                                      pk[2 * j], pk[2 * j + 1], 0, 0);
                            else
                                exp_step<false, false>(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3], sc, nmA, nmB, accA, accB,
                                                       pk[2 * j], pk[2 * j + 1], 0, 0);
                        }
                    } else {
                        // ragged tile (the last one of a branch): 8-column steps without a real token cost nothing
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int lim = j < 8 ? lim_lo : lim_hi;
                            if (8 * j < lim)
                                exp_step<false, true>(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3], sc, nmA, nmB, accA, accB,
                                                      pk[2 * j], pk[2 * j + 1], 8 * j + 2 * c2, lim);
                            else
                                pk[2 * j] = pk[2 * j + 1] = 0u;
                        }
                    }
                    WA_TRACE(20);
                    TMEM_STP32(s_addr, pk);
                    lA += accA.x + accA.y;
                    lB += accB.x + accB.y;
                    tmem_wait_st();
                    WA_TRACE(21);
                    tc_fence_before();
                    warp_arrive(&bar->p_full[buf]);
                    WA_TRACE(3);
                    ++pv_count;
                    if (phase == 1 && t == t0 && n_sel > 0) {
                        // The sparse branch's accumulator: its last PV product had this whole tile to land.  Normalise,
                        // round to bf16 (the reference stores this branch in bf16) and park it in registers until the
                        // combine; then the linear branch's first PV product may overwrite it.
                        ok = __all_sync(0xffffffffu, mbar_wait(&bar->o_done, ph_od, abort_flag, sink, 9));
                        if (!ok) break;
                        ph_od ^= 1u;
                        tc_fence_after();
                        WA_TRACE(12);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                            uint32_t ro[16];
                            TMEM_LDQ16(tmem_o + lane_addr + c * 32, ro);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float a0 = __uint_as_float(ro[4 * j]) * inv_spA, a1 = __uint_as_float(ro[4 * j + 1]) * inv_spA;
                                const float b0 = __uint_as_float(ro[4 * j + 2]) * inv_spB, b1 = __uint_as_float(ro[4 * j + 3]) * inv_spB;
                                if (p.part_sparse) {
                                    park[2 * (4 * c + j)] = __float_as_uint(a0);
                                    park[2 * (4 * c + j) + 1] = __float_as_uint(a1);
                                    gpk[2 * (4 * c + j)] = __float_as_uint(b0);
                                    gpk[2 * (4 * c + j) + 1] = __float_as_uint(b1);
                                } else {
                                    __nv_bfloat162 ha = __floats2bfloat162_rn(a0, a1), hbv = __floats2bfloat162_rn(b0, b1);
                                    park[2 * (4 * c + j)] = *reinterpret_cast<uint32_t *>(&ha);
                                    park[2 * (4 * c + j) + 1] = *reinterpret_cast<uint32_t *>(&hbv);
                                }
                            }
                        }
                        tc_fence_before();
                        warp_arrive(&bar->o_free);
                    }
                }
                if (!ok) break;
                // ---- end of a branch: total row sums (the four threads of a quad hold the parts of a row).  The
                // accumulator itself is read out later, when the PV products have surely landed: the sparse one after
                // the first tile of the linear branch (above), the linear one in the combine. ----
                lA = quad_sum(lA);
                lB = quad_sum(lB);
                const float invA = lA > 0.f ? 1.0f / lA : 0.f, invB = lB > 0.f ? 1.0f / lB : 0.f;
                const float lsA = lA > 0.f ? (mA + log2f(lA)) * 0.6931471805599453f : -INFINITY;
                const float lsB = lB > 0.f ? (mB + log2f(lB)) * 0.6931471805599453f : -INFINITY;
                if (phase == 0) {
                    inv_spA = invA;
                    inv_spB = invB;
                    ls_spA = lsA;
                    ls_spB = lsB;
                    if (p.lse_sparse && !p.lse_packed && c2 == 0) {
                        if (okA) p.lse_sparse[lseA] = lsA;
                        if (okB) p.lse_sparse[lseB] = lsB;
                    }
                    if (n_sel == 0) {   // no selected block: the sparse term is zero and there is no accumulator to wait for
#pragma unroll
                        for (int j = 0; j < 32; ++j) park[j] = gpk[j] = 0u;   // +0.0f and a bf16 pair of zeros alike
                    }
                } else {
                    inv_linA = invA;
                    inv_linB = invB;
                    if (p.lse_linear && c2 == 0) {
                        if (p.lse_packed) {   // [lse_sparse, lse_linear, 0, 0] behind the two branches of the record: one 16-byte store
                            if (okA) *reinterpret_cast<float4 *>(p.lse_sparse + lseA) = make_float4(ls_spA, lsA, 0.f, 0.f);
                            if (okB) *reinterpret_cast<float4 *>(p.lse_sparse + lseB) = make_float4(ls_spB, lsB, 0.f, 0.f);
                        } else {
                            if (okA) p.lse_linear[lseA] = lsA;
                            if (okB) p.lse_linear[lseB] = lsB;
                        }
                    }
                }
            }
            // ---- gate tile + combine ----
            // gate values of this thread's columns, rounded to bf16 as the reference's gate is (word 2j = row A, 2j + 1 =
            // row B); computed while the last PV product of the linear branch is still in flight
            // byte offset of this thread's 4 bytes inside 16-byte chunk j of a row in the swizzled 128 x 128 bf16 tiles
            auto tile_off = [&](int row, int j) -> int {
                return (j >> 3) * HALF_BYTES + row * 128 + (((j & 7) ^ (row & 7)) << 4) + 4 * c2;
            };
            if (ok) {
                WA_TRACE(18);
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_full[gbuf], ((sg + n_kv) / S_BUFS) & 1u, abort_flag, sink, 10));
            }
            if (ok) {
                tc_fence_after();
                WA_TRACE(13);
                if (!p.part_linear) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                        uint32_t gsc[16];
                        if (p.has_gate) {
                            TMEM_LDQ16(tmem_s + gbuf * TILE + lane_addr + c * 32, gsc);
                            tmem_wait_ld();
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int jj = 4 * c + j;
                            float zA0, zA1, zB0, zB1;
                            if (p.has_gate) {
                                const float2 bias2 = *reinterpret_cast<const float2 *>(&bar->bias[8 * jj + 2 * c2]);
                                zA0 = __uint_as_float(gsc[4 * j]) + bias2.x;
                                zA1 = __uint_as_float(gsc[4 * j + 1]) + bias2.y;
                                zB0 = __uint_as_float(gsc[4 * j + 2]) + bias2.x;
                                zB1 = __uint_as_float(gsc[4 * j + 3]) + bias2.y;
                            } else {
                                // no gate module: gate = sigmoid(q); q sits in the swizzled tile that the output overwrites below
                                const uint32_t qa = *reinterpret_cast<const uint32_t *>(q_stage + tile_off(rowA, jj));
                                const uint32_t qbv = *reinterpret_cast<const uint32_t *>(q_stage + tile_off(rowB, jj));
                                zA0 = __uint_as_float(qa << 16);
                                zA1 = __uint_as_float(qa & 0xffff0000u);
                                zB0 = __uint_as_float(qbv << 16);
                                zB1 = __uint_as_float(qbv & 0xffff0000u);
                            }
                            // sigmoid, one special-function op per element
                            __nv_bfloat162 ga = __floats2bfloat162_rn(fmaf(tanh_approx(0.5f * zA0), 0.5f, 0.5f),
                                                                       fmaf(tanh_approx(0.5f * zA1), 0.5f, 0.5f));
                            __nv_bfloat162 gb = __floats2bfloat162_rn(fmaf(tanh_approx(0.5f * zB0), 0.5f, 0.5f),
                                                                       fmaf(tanh_approx(0.5f * zB1), 0.5f, 0.5f));
                            gpk[2 * jj] = *reinterpret_cast<uint32_t *>(&ga);
                            gpk[2 * jj + 1] = *reinterpret_cast<uint32_t *>(&gb);
                        }
                    }
                }
                // the gate scores are consumed: their S buffer goes back to the QK warp
                tc_fence_before();
                warp_arrive(&bar->p_full[gbuf]);
                if (lin_tiles > 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->o_done, ph_od, abort_flag, sink, 9));
                    ph_od ^= 1u;
                    tc_fence_after();
                    WA_TRACE(12);
                }
            }
            if (ok && p.part_linear) {
                // Partial outputs leave as whole rows: a quad holds 32 bytes of a row per step, and stores of that size are
                // what a peer's buffer takes worst over NVLink.  The Q stage is free by now (every score product of the item
                // has landed), so each warp turns its 16 rows x 64 columns of float32 around in 4 KB of it (32-byte pieces
                // XOR-swizzled by row) and writes 512 contiguous bytes of two rows per instruction.
                uint8_t *scr = q_stage + warp * 4096;
                const int lr = lane & 15, row_l = rg * 32 + hb * 16 + lr;
                const int token_l = qb * BLK + row_l;
                constexpr long long NO_ROW = LLONG_MIN;   // (a peer's buffer may lie below this rank's: offsets can be negative)
                long long rec = NO_ROW;      // float offset of this lane's row (rows 0..15 of the warp) in the records
                if (row_l < BLK && token_l < p.Lq) {
                    if (p.peer_rows > 0) {
                        const int d = min(token_l / p.peer_rows, 7);
                        rec = (((long long)p.peer_self * p.peer_rows + (token_l - d * p.peer_rows)) * p.H + h) * p.part_stride
                              + p.peer_delta[d];
                    } else {
                        rec = (((long long)b * p.Lq + token_l) * p.H + h) * p.part_stride;
                    }
                }
                const int q16 = lane & 15, up = lane >> 4;
                auto put = [&](int jl, float x0, float x1, float y0, float y1) {   // step jl (0..7) of this 64-column half
                    *reinterpret_cast<float2 *>(scr + g * 256 + ((jl ^ g) << 5) + c2 * 8) = make_float2(x0, x1);
                    *reinterpret_cast<float2 *>(scr + (8 + g) * 256 + ((jl ^ g) << 5) + c2 * 8) = make_float2(y0, y1);
                };
                auto flush = [&](float *base, int half) {
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r16 = 2 * i + up;
                        const long long at = __shfl_sync(0xffffffffu, rec, r16);
                        const float4 val = *reinterpret_cast<const float4 *>(scr + r16 * 256 + (((q16 >> 1) ^ (r16 & 7)) << 5) + (q16 & 1) * 16);
                        if (at != NO_ROW) *reinterpret_cast<float4 *>(base + at + 64 * half + 4 * q16) = val;
                    }
                    __syncwarp();
                };
                if (p.part_sparse) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
#pragma unroll
                        for (int jl = 0; jl < 8; ++jl) {
                            const int jj = 8 * half + jl;
                            put(jl, __uint_as_float(park[2 * jj]), __uint_as_float(park[2 * jj + 1]), __uint_as_float(gpk[2 * jj]),
                                __uint_as_float(gpk[2 * jj + 1]));
                        }
                        flush(p.part_sparse, half);
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                    uint32_t o[16];
                    TMEM_LDQ16(tmem_o + lane_addr + c * 32, o);
                    tmem_wait_ld();
                    if (c == 3) {
                        // the linear accumulator is in registers: the next item's PV products may overwrite it
                        tc_fence_before();
                        warp_arrive(&bar->o_free);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        put(4 * (c & 1) + j, __uint_as_float(o[4 * j]) * inv_linA, __uint_as_float(o[4 * j + 1]) * inv_linA,
                            __uint_as_float(o[4 * j + 2]) * inv_linB, __uint_as_float(o[4 * j + 3]) * inv_linB);
                    if (c & 1) flush(p.part_linear, c >> 1);
                }
            } else if (ok) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                    uint32_t o[16];
                    TMEM_LDQ16(tmem_o + lane_addr + c * 32, o);
                    tmem_wait_ld();
                    WA_TRACE(14);
                    if (c == 3) {
                        // the linear accumulator is in registers: the next item's PV products may overwrite it
                        tc_fence_before();
                        warp_arrive(&bar->o_free);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int jj = 4 * c + j;
                        const float a0 = __uint_as_float(o[4 * j]) * inv_linA, a1 = __uint_as_float(o[4 * j + 1]) * inv_linA;
                        const float b0 = __uint_as_float(o[4 * j + 2]) * inv_linB, b1 = __uint_as_float(o[4 * j + 3]) * inv_linB;
                        const uint32_t spA = park[2 * jj], spB = park[2 * jj + 1], gA = gpk[2 * jj], gB = gpk[2 * jj + 1];   // low half = even column
                        __nv_bfloat162 ra = __floats2bfloat162_rn(fmaf(a0, __uint_as_float(gA << 16), __uint_as_float(spA << 16)),
                                                                   fmaf(a1, __uint_as_float(gA & 0xffff0000u), __uint_as_float(spA & 0xffff0000u)));
                        __nv_bfloat162 rb = __floats2bfloat162_rn(fmaf(b0, __uint_as_float(gB << 16), __uint_as_float(spB << 16)),
                                                                   fmaf(b1, __uint_as_float(gB & 0xffff0000u), __uint_as_float(spB & 0xffff0000u)));
                        // the finished tile is staged in the shared-memory stage that held Q (the layout the TMA store expects)
                        *reinterpret_cast<uint32_t *>(q_stage + tile_off(rowA, jj)) = *reinterpret_cast<uint32_t *>(&ra);
                        *reinterpret_cast<uint32_t *>(q_stage + tile_off(rowB, jj)) = *reinterpret_cast<uint32_t *>(&rb);
                    }
                    WA_TRACE(15);
                }
            }
            // Hand the staged tile to the store warp (in partial-output mode nothing was staged, but the Q stage
            // is released the same way).
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            warp_arrive(&bar->out_ready[qs]);
            WA_TRACE(10);
            sg += n_kv + 1;
            ++jcount;
        }
        tc_fence_before();
    }

    WA_TRACE(9);
    WA_TRACE_FLUSH;
    __syncthreads();
    tc_fence_after();
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- launch preparation as a kernel of its own (used when the routing kernel has not done it) --------
__global__ void __launch_bounds__(1024)
schedule_kernel(const int32_t *__restrict__ num, int n_items, int Nkv, SchedJob job) {
    if (blockIdx.x > 0) {
        if (job.gate_w) convert_gate_slice(job, (blockIdx.x - 1) * 1024, 1024);
        return;
    }
    schedule_items(num, n_items, Nkv, job.order, job.work_counter, job.error_flag);
}

// ---- host side -----------------------------------------------------------------------------------
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

// `[B, L, H, 128]` bf16 view -> 4-D map (d, h, token, batch), box 64 x 1 x 128 x 1, 128-byte swizzle.
static int make_map_4d(CUtensorMap *map, const wa_tensor4 *t, int B, int L, int H, const char *name, int box_rows = TILE) {
    EncodeTiledFn fn = encode_fn();
    WA_REQUIRE(fn, WA_ERR_DEVICE, "tcgen05 path: cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[4] = {(cuuint64_t)TILE, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)t->stride_h * 2, (cuuint64_t)t->stride_l * 2, (cuuint64_t)t->stride_b * 2};
    if (B == 1) strides[2] = strides[1] * (cuuint64_t)L;   // unused extent: any legal stride
    if (H == 1) strides[0] = 256;
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
    cuuint32_t elem[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, t->ptr, dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    WA_REQUIRE(r == CUDA_SUCCESS, WA_ERR_ALIGN, "tcgen05 path: tensor map for %s rejected (CUresult %d)", name, (int)r);
    return 0;
}

static int make_map_w(CUtensorMap *map, const void *w) {
    EncodeTiledFn fn = encode_fn();
    WA_REQUIRE(fn, WA_ERR_DEVICE, "tcgen05 path: cuTensorMapEncodeTiled is unavailable");
    cuuint64_t dims[2] = {(cuuint64_t)TILE, (cuuint64_t)TILE};
    cuuint64_t strides[1] = {(cuuint64_t)TILE * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TILE};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(w), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    WA_REQUIRE(r == CUDA_SUCCESS, WA_ERR_ALIGN, "tcgen05 path: tensor map for the gate weight rejected (CUresult %d)",
               (int)r);
    return 0;
}

static bool view_ok(const wa_tensor4 *t) {
    return t->ptr && t->dtype == WA_BF16 && ((uintptr_t)t->ptr % 16 == 0) && t->stride_h % 8 == 0 &&
           t->stride_l % 8 == 0 && t->stride_b % 8 == 0 && t->stride_h > 0 && t->stride_l > 0;
}

static int max_grid() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0)
        sms = 160;
    return sms;
}

struct TunedWs {
    size_t order, counter, w_bf16, bias, zeros, total;
};
static TunedWs tuned_plan(const wa_hsa_params *p) {
    TunedWs w{};
    size_t c = 0;
    const size_t items = (size_t)p->B * p->H * ceil_div(p->Lq, p->block_size < TILE ? p->block_size : TILE);
    w.order = c; c = align_up(c + items * sizeof(int32_t), 256);
    w.counter = c; c = align_up(c + 2 * sizeof(int), 256);
    w.w_bf16 = c; c = align_up(c + (size_t)TILE * TILE * 2, 256);
    w.bias = c; c = align_up(c + TILE * sizeof(float), 256);
    w.zeros = c; c = align_up(c + items * sizeof(int32_t), 256);   // an all-zero `num` for the linear-branch-only launch
    w.total = c;
    return w;
}

}  // namespace sm100

#ifdef WA_SM100_TRACE
extern "C" int wa_stats_read(long long *dst, int n_ctas) {
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(dst, sm100::g_cta_stats, (size_t)n_ctas * 6 * sizeof(long long));
    return 0;
}
extern "C" int wa_trace_read(long long *dst, int max_words) {
    // concatenates the three roles' (id, clock) pairs; returns the number of 64-bit words written
    int n[4] = {0, 0, 0, 0}, out = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(n, sm100::g_trace_n, sizeof(n));
    for (int r = 0; r < 4; ++r) {
        const int words = 2 * n[r];
        if (out + words > max_words) break;
        cudaMemcpyFromSymbol(dst + out, sm100::g_trace, (size_t)words * sizeof(long long),
                             (size_t)r * 2 * sm100::TRACE_SLOTS * sizeof(long long));
        out += words;
    }
    return out;
}
#endif

size_t hsa_sm100_workspace_bytes(const wa_hsa_params *p) { return sm100::tuned_plan(p).total; }
size_t hsa_sm100_status_offset(const wa_hsa_params *p) { return sm100::tuned_plan(p).counter + sizeof(int); }

SchedJob hsa_sm100_sched_job(const wa_hsa_params *p, void *workspace) {
    const sm100::TunedWs w = sm100::tuned_plan(p);
    char *ws = (char *)workspace;
    SchedJob job{};
    job.order = (int32_t *)(ws + w.order);
    job.work_counter = (int *)(ws + w.counter);
    job.error_flag = job.work_counter + 1;
    job.gate_w = p->gate_w; job.gate_b = p->gate_b; job.gate_dt = p->gate_dtype;
    job.w_out = (__nv_bfloat16 *)(ws + w.w_bf16);
    job.b_out = (float *)(ws + w.bias);
    return job;
}

static bool device_is_sm100() {
    static PerDeviceOnce known_sm100;   // the answer belongs to the current device, not to the process
    if (known_sm100.done()) return true;
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
        return false;
    if (major == 10) known_sm100.mark();
    return major == 10;
}

bool hsa_sm100_supported(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc) {
    using namespace sm100;
    if (p->D != TILE || (p->block_size != TILE && p->block_size != HALF) || Lc <= 0) return false;
    if (!view_ok(&p->q) || !view_ok(&p->k) || !view_ok(&p->v) || !view_ok(kc) || !view_ok(vc)) return false;
    if (!p->part_sparse && (p->out.dtype != WA_BF16 || !p->out.ptr || (uintptr_t)p->out.ptr % 16 || p->out.stride_h % 8 ||
                            p->out.stride_l % 8 || p->out.stride_b % 8))
        return false;
    if (p->part_sparse && (((uintptr_t)p->part_sparse | (uintptr_t)p->part_linear) % 16 || p->part_stride % 4 || p->part_stride < 0 ||
                           (p->part_stride > 0 && p->part_stride < TILE)))
        return false;
    if ((long long)p->B * p->H * ceil_div(p->Lq, p->block_size) > (1 << 24)) return false;
    return device_is_sm100() && encode_fn() != nullptr;
}

int hsa_sm100_launch(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc, const int32_t *index,
                     const int32_t *num, int Nq, int Nkv, void *workspace, bool prepared, cudaStream_t stream) {
    using namespace sm100;
    const SchedJob job = hsa_sm100_sched_job(p, workspace);
    int32_t *order = job.order;
    int *counter = job.work_counter;
    __nv_bfloat16 *w_bf16 = job.w_out;
    float *bias = job.b_out;

    CUtensorMap tq, tk, tv, tkc, tvc, tw, tout;
    int rc;
    if ((rc = make_map_4d(&tq, &p->q, p->B, p->Lq, p->H, "q"))) return rc;
    const int blk = p->block_size == HALF ? HALF : TILE;   // the linear-branch-only launch (other sizes) never loads k / v
    if ((rc = make_map_4d(&tk, &p->k, p->B, p->Lkv, p->H, "k", blk))) return rc;
    if ((rc = make_map_4d(&tv, &p->v, p->B, p->Lkv, p->H, "v", blk))) return rc;
    if ((rc = make_map_4d(&tkc, kc, p->B, Lc, p->H, "k_coarse"))) return rc;
    if ((rc = make_map_4d(&tvc, vc, p->B, Lc, p->H, "v_coarse"))) return rc;
    if ((rc = make_map_w(&tw, w_bf16))) return rc;
    if ((rc = make_map_4d(&tout, p->part_sparse ? &p->q : &p->out, p->B, p->Lq, p->H, "out", blk))) return rc;   // unused in partial mode

    const int n_items = p->B * p->H * Nq;
    if (!prepared) {
        schedule_kernel<<<p->gate_w ? 1 + TILE * TILE / 1024 : 1, 1024, 0, stream>>>(num, n_items, Nkv, job);
        if ((rc = check_launch("wa_hsa_forward(schedule)"))) return rc;
    }

    Params kp{};
    kp.B = p->B; kp.H = p->H; kp.Lq = p->Lq; kp.Lkv = p->Lkv; kp.Lc = Lc; kp.Nq = Nq; kp.Nkv = Nkv;
    kp.n_items = n_items;
    kp.blk = blk;
    kp.index = index; kp.num = num; kp.order = order; kp.work_counter = counter; kp.error_flag = counter + 1;
    kp.status_mirror = p->status_mirror;
    kp.out = (__nv_bfloat16 *)p->out.ptr; kp.osb = p->out.stride_b; kp.osl = p->out.stride_l; kp.osh = p->out.stride_h;
    kp.gate_bias = bias; kp.has_gate = p->gate_w != nullptr;
    kp.q = (const __nv_bfloat16 *)p->q.ptr; kp.qsb = p->q.stride_b; kp.qsl = p->q.stride_l; kp.qsh = p->q.stride_h;
    kp.scale_log2 = (float)(pow((double)TILE, -0.5) * 1.4426950408889634);
    kp.part_sparse = p->part_sparse; kp.part_linear = p->part_linear;
    kp.lse_sparse = p->lse_sparse; kp.lse_linear = p->lse_linear;
    kp.peer_rows = p->part_sparse ? p->peer_rows : 0; kp.peer_self = p->peer_self;
    for (int r = 0; r < 8; ++r) kp.peer_delta[r] = p->peer_delta[r];
    // default layouts: contiguous [B, Lq, H, 128] vectors and [B, H, Lq] normalisers; the packed exchange layout of the
    // KV-sharded path puts both branches of a (token, head) into one record
    kp.part_stride = p->part_stride > 0 ? p->part_stride : TILE;
    // packed records [sparse | linear | lse_sparse, lse_linear, 0, 0]: both normalisers leave in one 16-byte store
    kp.lse_packed = p->part_sparse && p->lse_sparse == p->part_sparse + 2 * TILE && p->lse_linear == p->lse_sparse + 1 &&
                    kp.part_stride >= 2 * TILE + 4 && p->lse_stride_token > 0 && p->lse_stride_token % 4 == 0 &&
                    p->lse_stride_head % 4 == 0;
    if (p->lse_stride_token > 0) {
        kp.lse_st = p->lse_stride_token; kp.lse_sh = p->lse_stride_head; kp.lse_sb = (long long)p->Lq * p->lse_stride_token;
    } else {
        kp.lse_st = 1; kp.lse_sh = p->Lq; kp.lse_sb = (long long)p->H * p->Lq;
    }


    static PerDeviceOnce attr_set;
    if (!attr_set.done()) {
        cudaError_t e = cudaFuncSetAttribute(hsa_fwd_sm100_kernel<TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(hsa_fwd_sm100_kernel<HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return fail((int)e, "wa_hsa_forward(tcgen05): %s", cudaGetErrorString(e));
        attr_set.mark();
    }
    int grid = n_items < max_grid() ? n_items : max_grid();
#ifdef WA_SM100_TRACE
    if (getenv("WA_SM100_ONE_CTA") && grid > max_grid() / 2) grid = max_grid() / 2;   // tuning aid: one CTA per SM
#endif
    profile_mark(true, stream);
    cudaError_t le = blk == TILE ? launch_dependent(hsa_fwd_sm100_kernel<TILE>, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, tq, tk,
                                                    tv, tkc, tvc, tw, tout, kp)
                                 : launch_dependent(hsa_fwd_sm100_kernel<HALF>, dim3(grid), dim3(THREADS), SMEM_BYTES, stream, tq, tk,
                                                    tv, tkc, tvc, tw, tout, kp);
    profile_mark(false, stream);
    if (le != cudaSuccess) return fail((int)le, "wa_hsa_forward(tcgen05): %s", cudaGetErrorString(le));
    return check_launch("wa_hsa_forward(tcgen05)");
}

// The linear branch alone on the tcgen05 kernel (any routing block size): every item runs with an empty selection
// and the normalised float32 result goes to `linear_out` [B, Lq, H, 128].
bool hsa_sm100_linear_supported(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc) {
    using namespace sm100;
    if (p->D != TILE || Lc <= 0 || p->part_sparse) return false;
    if (!view_ok(&p->q) || !view_ok(&p->k) || !view_ok(&p->v) || !view_ok(kc) || !view_ok(vc)) return false;
    if (p->out.dtype != WA_BF16 || !p->out.ptr || (uintptr_t)p->out.ptr % 16 || p->out.stride_h % 8 || p->out.stride_l % 8 ||
        p->out.stride_b % 8)
        return false;
    if ((long long)p->B * p->H * ceil_div(p->Lq, TILE) > (1 << 24)) return false;
    return device_is_sm100() && encode_fn() != nullptr;
}

int hsa_sm100_launch_linear(const wa_hsa_params *p, int Lc, const wa_tensor4 *kc, const wa_tensor4 *vc, float *linear_out,
                            void *workspace, cudaStream_t stream) {
    using namespace sm100;
    WA_REQUIRE((uintptr_t)linear_out % 16 == 0, WA_ERR_ALIGN, "wa_hsa_forward(tcgen05 linear): output must be 16-byte aligned");
    const TunedWs w = tuned_plan(p);
    int32_t *zeros = (int32_t *)((char *)workspace + w.zeros);
    const int nq = ceil_div(p->Lq, TILE);
    cudaError_t e = cudaMemsetAsync(zeros, 0, (size_t)p->B * p->H * nq * sizeof(int32_t), stream);
    if (e != cudaSuccess) return fail((int)e, "wa_hsa_forward(tcgen05 linear): %s", cudaGetErrorString(e));
    wa_hsa_params pl = *p;
    pl.part_sparse = nullptr; pl.lse_sparse = nullptr; pl.lse_linear = nullptr;
    pl.part_linear = linear_out;
    profile_pause(true);   // the timing bracket of this forward belongs to the sparse-branch kernel
    const int rc = hsa_sm100_launch(&pl, Lc, kc, vc, zeros /*never read: no item selects a block*/, zeros, nq, 1, workspace, false,
                                    stream);
    profile_pause(false);
    return rc;
}

}  // namespace wa
