// Fused HSA forward for sm_100a, two work items in flight per SM.
//
// Same job as the kernel in wa_hsa_sm100.cu -- block-sparse softmax branch, compressed ("linear")
// branch, gate product and combine, replacing the reference's Triton `_fwd_kernel`
// (wan/modules/hsa/block_sparse_triton.py:67-139), `_linear_branch` and the gate/addcmul epilogue
// (wan/modules/hsa/attention.py:113-118, 246-259) -- laid out differently: TWO CTAs share an SM, each
// with half of the tensor memory (256 columns: one S buffer and one O accumulator) and half of the
// shared memory (one Q, one K and one V tile).  Inside a CTA the tile chain of a work item is strictly
// serial -- S = Q K^T, softmax, O += P V, next S -- and ONE thread issues every tensor-core product in
// program order, so the product that overwrites S follows the product that read P out of it without a
// completion barrier in between.  The hardware interleaves the two CTAs: while one runs its softmax the
// other's products own the tensor pipe, and the epilogue of one item hides behind the tiles of the other.
//
// CTA = 8 warps: warps 0-3 softmax and epilogue (warp w owns tensor-memory lanes 32w..32w+31 = query
// rows, handled as two 16-row slabs in the quad-row shapes: a row lives in four lanes of one warp),
// warp 4 work queue + TMA loads, warp 5 issues the products, warp 6 stores the finished tile with TMA,
// warp 7 idles (it completes the second warpgroup for the register hand-over).
//
// Barrier protocol (every K-type tile -- sparse, linear or gate -- completes exactly one phase of
// s_full and of p_full; every wait is bounded, see mbar_wait):
//   k_full / v_full  : TMA landed            k_empty / v_empty : the product that read the stage is done
//   s_full           : scores are in S       p_full            : the softmax warps have written P (or, for
//                                                                 the gate tile, read the gate scores)
// A completed s_full(t) also says that every earlier product of this CTA has landed, so the softmax
// warps may rescale or read out the O accumulator after it without another barrier; the product that
// starts a branch waits for p_full of that branch's first tile, which the softmax warps signal only
// after they have read the previous accumulator out.
#include "wa_internal.cuh"
#include "wa_sm100_ptx.cuh"

namespace wa {
namespace sm100 {
namespace pair {

constexpr int THREADS = 256;
constexpr int REGS_SOFTMAX = 216;    // per thread after the hand-over: 128 * 216 + 128 * 40 = 256 * 128
constexpr int REGS_OTHER = 40;
constexpr int TMEM_COLS = 256;       // S: columns [0,128); O: [128,256)
constexpr int PARK_SMEM_WORDS = 24;  // of the 64 words a softmax thread parks per item, this many live in shared memory
constexpr int PARK_BYTES = PARK_SMEM_WORDS * 128 * 4;
constexpr int SMEM_BYTES = 3 * TILE_BYTES + 2048 + PARK_BYTES;   // Q, K, V tiles + barriers and bias + parked words

struct Barriers {
    uint64_t item_full[2], item_empty[2];
    uint64_t q_full, q_empty, k_full, k_empty, v_full, v_empty;
    uint64_t s_full, p_full, out_ready;
    uint32_t tmem_base;
    int abort_flag;
    ItemDesc items[2];
    int valid[4];            // real token counts of the K-type tiles in flight, ring indexed by tile number
    float bias[TILE];        // gate bias
};
static_assert(sizeof(Barriers) <= 2048, "barrier block exceeds its shared-memory budget");
static_assert(2 * (SMEM_BYTES + 1024) <= 228 * 1024, "two CTAs must fit one SM");

struct RowState {   // running maximum (scaled, base 2) and this thread's share of the row sum, rows A and B of a slab
    float mA, mB, lA, lB;
};

// One 16-row slab of a score tile: row maximum, lazy rescale of the accumulator, probabilities written
// back over the scores.  `s_addr` / `o_addr`: tensor-memory addresses of S and O with the slab's lane
// offset applied.  Called by whole warps.
__device__ __forceinline__ void softmax_slab(uint32_t s_addr, uint32_t o_addr, RowState &st, bool first_tile, int vword,
                                             float scale_log2, int c2) {
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
    const float mxA = quad_max(fmaxf(xa0, xa1)) * scale_log2, mxB = quad_max(fmaxf(xb0, xb1)) * scale_log2;
    // lazy rescale: only when a running maximum grows by more than 2^8
    float mA_new = st.mA, mB_new = st.mB;
    const bool growA = mxA > st.mA + 8.0f, growB = mxB > st.mB + 8.0f;
    if (growA) mA_new = mxA;
    if (growB) mB_new = mxB;
    if (__any_sync(0xffffffffu, (growA || growB) && !first_tile)) {
        // every product issued so far has landed (the scores of this tile came after them in program order)
        const float fA = (growA && !first_tile) ? ex2(st.mA - mA_new) : 1.0f, fB = (growB && !first_tile) ? ex2(st.mB - mB_new) : 1.0f;
        st.lA *= fA;
        st.lB *= fB;
#pragma unroll
        for (int c = 0; c < 4; ++c) {   // 32 columns at a time
            uint32_t ro[16];
            TMEM_LDQ16(o_addr + c * 32, ro);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                ro[4 * j] = __float_as_uint(__uint_as_float(ro[4 * j]) * fA);
                ro[4 * j + 1] = __float_as_uint(__uint_as_float(ro[4 * j + 1]) * fA);
                ro[4 * j + 2] = __float_as_uint(__uint_as_float(ro[4 * j + 2]) * fB);
                ro[4 * j + 3] = __float_as_uint(__uint_as_float(ro[4 * j + 3]) * fB);
            }
            TMEM_STQ16(o_addr + c * 32, ro);
        }
        tmem_wait_st();
    }
    st.mA = mA_new;
    st.mB = mB_new;
    // p = 2^(s*c - m), row sums, pack to bf16, write P over the consumed S columns
    uint32_t pk[32];
    const float2 sc = make_float2(scale_log2, scale_log2);
    const float2 nmA = make_float2(-st.mA, -st.mA), nmB = make_float2(-st.mB, -st.mB);
    float2 accA = make_float2(0.f, 0.f), accB = make_float2(0.f, 0.f);
    if (full) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j % POLY_EVERY == 0)
                exp_step<true, false>(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3], sc, nmA, nmB, accA, accB, pk[2 * j],
                                      pk[2 * j + 1], 0, 0);
            else
                exp_step<false, false>(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3], sc, nmA, nmB, accA, accB, pk[2 * j],
                                       pk[2 * j + 1], 0, 0);
        }
    } else {
        // ragged tile (the last one of a branch): 8-column steps without a real token cost nothing
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int lim = j < 8 ? lim_lo : lim_hi;
            if (8 * j < lim)
                exp_step<false, true>(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3], sc, nmA, nmB, accA, accB, pk[2 * j],
                                      pk[2 * j + 1], 8 * j + 2 * c2, lim);
            else
                pk[2 * j] = pk[2 * j + 1] = 0u;
        }
    }
    TMEM_STP32(s_addr, pk);
    st.lA += accA.x + accA.y;
    st.lB += accB.x + accB.y;
}

template <int BLK>   // routing block size: 128, or 64 (see Params::blk)
__global__ void __launch_bounds__(THREADS, 2)
hsa_fwd_sm100_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_kc,
                          const __grid_constant__ CUtensorMap tm_vc, const __grid_constant__ CUtensorMap tm_w,
                          const __grid_constant__ CUtensorMap tm_out, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];   // swizzled TMA tiles need 1024-byte alignment (checked below)
    uint8_t *q_s = smem, *k_s = smem + TILE_BYTES, *v_s = smem + 2 * TILE_BYTES;
    Barriers *bar = reinterpret_cast<Barriers *>(smem + 3 * TILE_BYTES);
    uint32_t *park_s = reinterpret_cast<uint32_t *>(smem + 3 * TILE_BYTES + 2048) + (threadIdx.x & 127);   // word w at park_s[w * 128]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int *abort_flag = &bar->abort_flag;
    const FailSink sink{p.error_flag, p.status_mirror};

    if (threadIdx.x == 0) {
        bar->abort_flag = (smem_u32(smem) & 1023u) ? 1 : 0;   // misaligned shared memory: give up before any TMA
        if (bar->abort_flag) report_failure(sink, 99);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar->item_full[i], 1);
            mbar_init(&bar->item_empty[i], 1 + 4 + 1);   // issuer + every softmax warp + store warp
        }
        mbar_init(&bar->q_full, 1);
        mbar_init(&bar->q_empty, 1 + 4);   // the gate product has read Q + every softmax warp is done with it
        mbar_init(&bar->k_full, 1);
        mbar_init(&bar->k_empty, 1);
        mbar_init(&bar->v_full, 1);
        mbar_init(&bar->v_empty, 1);
        mbar_init(&bar->s_full, 1);
        mbar_init(&bar->p_full, 4);
        mbar_init(&bar->out_ready, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x >= 128 && threadIdx.x < 128 + TILE)
        bar->bias[threadIdx.x - 128] = (p.has_gate && p.gate_bias) ? p.gate_bias[threadIdx.x - 128] : 0.f;
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bar->tmem_base)),
                     "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bar->tmem_base;
    const uint32_t tmem_s = tmem, tmem_o = tmem + TILE;
    const int lin_tiles = (p.Lc + TILE - 1) / TILE;

    if (warp >= 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_OTHER));
        if (warp == 4) {
            // ================= producer: work queue + TMA =================
            if (lane == 0) {
                uint32_t jcount = 0, kcount = 0, vcount = 0;
                bool ok = true;
                // The first item of a CTA is fixed by its index (no round trip to the counter before the first load);
                // later items come from the counter, which is asked for the next position one item ahead.
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

                    ok = mbar_wait(&bar->q_empty, (jcount & 1u) ^ 1u, abort_flag, sink, 12);
                    if (!ok) break;
                    mbar_expect_tx(&bar->q_full, TILE_BYTES);
                    tma_load_4d(q_s, &tm_q, &bar->q_full, 0, h, qb * BLK, b);
                    tma_load_4d(q_s + HALF_BYTES, &tm_q, &bar->q_full, 64, h, qb * BLK, b);

                    // Loads follow the order in which the stages come back: K(t) after the score product of tile t-1,
                    // V(t) after the P.V product of tile t-1, which lands between score products t-1 and t.
                    for (int t = 0; t <= n_kv && ok; ++t) {
                        ok = mbar_wait(&bar->k_empty, (kcount & 1u) ^ 1u, abort_flag, sink, 1);
                        if (!ok) break;
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
                        bar->valid[kcount & 3] = valid;
                        ++kcount;
                        mbar_expect_tx(&bar->k_full, TILE_BYTES);
                        if (t < n_st) {
                            if (BLK == TILE) {
                                tma_load_4d(k_s, &tm_k, &bar->k_full, 0, h, id * TILE, b);
                                tma_load_4d(k_s + HALF_BYTES, &tm_k, &bar->k_full, 64, h, id * TILE, b);
                            } else {   // 64-row boxes: rows 0..63 of each half-tile from the first block, 64..127 from the second
                                tma_load_4d(k_s, &tm_k, &bar->k_full, 0, h, id * HALF, b);
                                tma_load_4d(k_s + HALF_BYTES / 2, &tm_k, &bar->k_full, 0, h, id2 * HALF, b);
                                tma_load_4d(k_s + HALF_BYTES, &tm_k, &bar->k_full, 64, h, id * HALF, b);
                                tma_load_4d(k_s + HALF_BYTES + HALF_BYTES / 2, &tm_k, &bar->k_full, 64, h, id2 * HALF, b);
                            }
                        } else if (t < n_kv) {
                            const int c = (t - n_st) * TILE;
                            tma_load_4d(k_s, &tm_kc, &bar->k_full, 0, h, c, b);
                            tma_load_4d(k_s + HALF_BYTES, &tm_kc, &bar->k_full, 64, h, c, b);
                        } else {   // the gate weight takes the K stage of the item's last tile
                            tma_load_2d(k_s, &tm_w, &bar->k_full, 0, 0);
                            tma_load_2d(k_s + HALF_BYTES, &tm_w, &bar->k_full, 64, 0);
                            break;
                        }
                        ok = mbar_wait(&bar->v_empty, (vcount & 1u) ^ 1u, abort_flag, sink, 2);
                        if (!ok) break;
                        ++vcount;
                        mbar_expect_tx(&bar->v_full, TILE_BYTES);
                        if (t < n_st) {
                            if (BLK == TILE) {
                                tma_load_4d(v_s, &tm_v, &bar->v_full, 0, h, id * TILE, b);
                                tma_load_4d(v_s + HALF_BYTES, &tm_v, &bar->v_full, 64, h, id * TILE, b);
                            } else {
                                tma_load_4d(v_s, &tm_v, &bar->v_full, 0, h, id * HALF, b);
                                tma_load_4d(v_s + HALF_BYTES / 2, &tm_v, &bar->v_full, 0, h, id2 * HALF, b);
                                tma_load_4d(v_s + HALF_BYTES, &tm_v, &bar->v_full, 64, h, id * HALF, b);
                                tma_load_4d(v_s + HALF_BYTES + HALF_BYTES / 2, &tm_v, &bar->v_full, 64, h, id2 * HALF, b);
                            }
                        } else {
                            const int c = (t - n_st) * TILE;
                            tma_load_4d(v_s, &tm_vc, &bar->v_full, 0, h, c, b);
                            tma_load_4d(v_s + HALF_BYTES, &tm_vc, &bar->v_full, 64, h, c, b);
                        }
                    }
                    ++jcount;
                }
            }
        } else if (warp == 5) {
            // ================= issuer of every tensor-core product =================
            // The whole warp runs the role so that operands stay warp-uniform; one elected lane issues.
            const bool leader = elect_one();
            constexpr uint32_t IDESC_QK = instr_desc(false, TILE), IDESC_PV = instr_desc(true, TILE);
            uint32_t jcount = 0, kcount = 0, vcount = 0, pcount = 0;
            bool ok = true;
            const uint64_t qd = smem_desc(smem_u32(q_s), 16, 1024);
            const uint64_t kd = smem_desc(smem_u32(k_s), 16, 1024);
            const uint64_t vd = smem_desc(smem_u32(v_s), HALF_BYTES, 1024);
            auto issue_qk = [&]() {   // S = Q . (K stage)^T
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4);
                    mma_ss(tmem_s, qd + off, kd + off, IDESC_QK, kk > 0);
                }
                tc_commit(&bar->s_full);
                tc_commit(&bar->k_empty);
            };
            while (ok) {
                const uint32_t slot = jcount & 1u;
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->item_full[slot], (jcount >> 1) & 1u, abort_flag, sink, 14));
                if (!ok) break;
                const int item = bar->items[slot].item, n_sel = bar->items[slot].n_sel;
                __syncwarp();
                if (leader) mbar_arrive(&bar->item_empty[slot]);
                if (item < 0) break;
                const int n_kv = n_sel + lin_tiles;   // tiles 0 .. n_kv - 1 feed a P.V product, tile n_kv is the gate
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->q_full, jcount & 1u, abort_flag, sink, 3));
                if (!ok) break;
                if (jcount > 0) {   // the gate scores of the previous item have been read out of S
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->p_full, pcount & 1u, abort_flag, sink, 13));
                    if (!ok) break;
                    ++pcount;
                }
                ok = __all_sync(0xffffffffu, mbar_wait(&bar->k_full, kcount & 1u, abort_flag, sink, 4));
                if (!ok) break;
                ++kcount;
                tc_fence_after();
                if (leader) issue_qk();
                __syncwarp();
                for (int t = 0; t < n_kv && ok; ++t) {
                    // operands that are there long before the probabilities first
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->k_full, kcount & 1u, abort_flag, sink, 4));
                    if (!ok) break;
                    ++kcount;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->v_full, vcount & 1u, abort_flag, sink, 6));
                    if (!ok) break;
                    ++vcount;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->p_full, pcount & 1u, abort_flag, sink, 5));
                    if (!ok) break;
                    ++pcount;
                    tc_fence_after();
                    if (leader) {
                        const bool first = (t == 0) || (t == n_sel);   // a branch starts: overwrite the accumulator
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk)
                            mma_ts(tmem_o, tmem_s + kk * 8, vd + (uint64_t)((kk * 2048) >> 4), IDESC_PV, !(first && kk == 0));
                        // the V stage of the item's last tile goes back through the store warp: the finished tile is staged in it
                        if (t != n_kv - 1) tc_commit(&bar->v_empty);
                        issue_qk();   // tile t + 1 (the gate product when t + 1 == n_kv): in order behind the product that read P
                        if (t == n_kv - 1) tc_commit(&bar->q_empty);
                    }
                    __syncwarp();
                }
                ++jcount;
            }
        } else if (warp == 6) {
            // ================= store warp: TMA store of the staged output tile, then release of the V stage =========
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
                    ok = mbar_wait(&bar->out_ready, jcount & 1u, abort_flag, sink, 17);
                    if (!ok) break;
                    if (!p.part_linear) {
                        // rows beyond q_len are clipped by the tensor map
                        // (with 64-token blocks the map's box is 64 rows: the tile's upper rows belong to the next item)
                        tma_store_4d(&tm_out, v_s, 0, h, qb * BLK, b);
                        tma_store_4d(&tm_out, v_s + HALF_BYTES, 64, h, qb * BLK, b);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the V stage is reusable afterwards
                    }
                    mbar_arrive(&bar->v_empty);
                    ++jcount;
                }
                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all stores have landed before the CTA exits
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
        // ================= softmax / epilogue =================
        // Warp w may only touch tensor-memory lanes 32w .. 32w + 31.  A slab is 16 of them, read in the quad-row shape:
        // thread t holds rows t/4 and t/4 + 8 of the slab and, of each, the column pairs 8j + 2(t%4), +1.
        const int g = lane >> 2, c2 = lane & 3;
        uint32_t jcount = 0, sg = 0;       // items and K-type tiles seen so far
        bool ok = true;

        while (ok) {
            const uint32_t slot = jcount & 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(&bar->item_full[slot], (jcount >> 1) & 1u, abort_flag, sink, 15));
            if (!ok) break;
            const int item = bar->items[slot].item, n_sel = bar->items[slot].n_sel;
            warp_arrive(&bar->item_empty[slot]);
            if (item < 0) break;
            const int qb = item % p.Nq, h = (item / p.Nq) % p.H, b = item / (p.Nq * p.H);
            const int n_kv = n_sel + lin_tiles;
            float inv_sp[4], inv_lin[4];   // [2 * slab + (row B)]
            // The sparse branch's result waits for the combine: slab s, step j: word 32s + 2j = row A, + 1 = row B (bf16
            // pairs).  The last PARK_SMEM_WORDS words wait in shared memory (a column of words per thread), the rest in
            // registers: all 64 in registers do not fit beside a slab of scores.
            uint32_t park[64 - PARK_SMEM_WORDS];
            auto put_park = [&](int w, uint32_t x) {
                if (w < 64 - PARK_SMEM_WORDS) park[w] = x;
                else park_s[(w - (64 - PARK_SMEM_WORDS)) * 128] = x;
            };
            auto get_park = [&](int w) -> uint32_t {
                return w < 64 - PARK_SMEM_WORDS ? park[w] : park_s[(w - (64 - PARK_SMEM_WORDS)) * 128];
            };

            for (int phase = 0; phase < 2 && ok; ++phase) {
                const int t0 = phase == 0 ? 0 : n_sel, t1 = phase == 0 ? n_sel : n_kv;
                RowState st[2];
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    st[s].mA = st[s].mB = -INFINITY;
                    st[s].lA = st[s].lB = 0.f;
                }
                for (int t = t0; t < t1 && ok; ++t) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_full, sg & 1u, abort_flag, sink, 8));
                    if (!ok) break;
                    tc_fence_after();
                    const int vword = bar->valid[sg & 3];
                    ++sg;
                    if (phase == 1 && t == t0 && n_sel > 0) {
                        // The sparse branch's accumulator is complete (its last product precedes these scores).  Normalise,
                        // round to bf16 (the reference stores this branch in bf16) and park it in registers until the
                        // combine; the first product of the linear branch overwrites it after this tile's p_full.
#pragma unroll
                        for (int s = 0; s < 2; ++s) {
                            const uint32_t o_addr = tmem_o + ((uint32_t)(warp * 32 + s * 16) << 16);
                            const int rowA = warp * 32 + s * 16 + g, tokenA = qb * BLK + rowA;
                            const bool okA = rowA < BLK && tokenA < p.Lq, okB = rowA + 8 < BLK && tokenA + 8 < p.Lq;
                            const long long partA = (((long long)b * p.Lq + tokenA) * p.H + h) * p.part_stride + 2 * c2;
                            const long long partB = partA + 8ll * p.H * p.part_stride;
#pragma unroll
                            for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                                uint32_t ro[16];
                                TMEM_LDQ16(o_addr + c * 32, ro);
                                tmem_wait_ld();
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    const float a0 = __uint_as_float(ro[4 * j]) * inv_sp[2 * s], a1 = __uint_as_float(ro[4 * j + 1]) * inv_sp[2 * s];
                                    const float b0 = __uint_as_float(ro[4 * j + 2]) * inv_sp[2 * s + 1], b1 = __uint_as_float(ro[4 * j + 3]) * inv_sp[2 * s + 1];
                                    if (p.part_sparse) {
                                        if (okA) *reinterpret_cast<float2 *>(p.part_sparse + partA + 8 * (4 * c + j)) = make_float2(a0, a1);
                                        if (okB) *reinterpret_cast<float2 *>(p.part_sparse + partB + 8 * (4 * c + j)) = make_float2(b0, b1);
                                    } else {
                                        __nv_bfloat162 ha = __floats2bfloat162_rn(a0, a1), hbv = __floats2bfloat162_rn(b0, b1);
                                        put_park(32 * s + 2 * (4 * c + j), *reinterpret_cast<uint32_t *>(&ha));
                                        put_park(32 * s + 2 * (4 * c + j) + 1, *reinterpret_cast<uint32_t *>(&hbv));
                                    }
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        const uint32_t lane_addr = (uint32_t)(warp * 32 + s * 16) << 16;
                        softmax_slab(tmem_s + lane_addr, tmem_o + lane_addr, st[s], t == t0, vword, p.scale_log2, c2);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    warp_arrive(&bar->p_full);
                }
                if (!ok) break;
                // ---- end of a branch: total row sums (the four threads of a quad hold the parts of a row) ----
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const float lA = quad_sum(st[s].lA), lB = quad_sum(st[s].lB);
                    const float invA = lA > 0.f ? 1.0f / lA : 0.f, invB = lB > 0.f ? 1.0f / lB : 0.f;
                    if (phase == 0) {
                        inv_sp[2 * s] = invA;
                        inv_sp[2 * s + 1] = invB;
                    } else {
                        inv_lin[2 * s] = invA;
                        inv_lin[2 * s + 1] = invB;
                    }
                    float *lse = phase == 0 ? p.lse_sparse : p.lse_linear;
                    if (lse && c2 == 0) {
                        const int rowA = warp * 32 + s * 16 + g, tokenA = qb * BLK + rowA;
                        const long long lseA = (long long)b * p.lse_sb + (long long)h * p.lse_sh + (long long)tokenA * p.lse_st;
                        if (rowA < BLK && tokenA < p.Lq)
                            lse[lseA] = lA > 0.f ? (st[s].mA + log2f(lA)) * 0.6931471805599453f : -INFINITY;
                        if (rowA + 8 < BLK && tokenA + 8 < p.Lq)
                            lse[lseA + 8 * p.lse_st] = lB > 0.f ? (st[s].mB + log2f(lB)) * 0.6931471805599453f : -INFINITY;
                    }
                }
                if (phase == 0 && n_sel == 0) {   // no selected block: the sparse term is zero and there is no accumulator to read
                    if (p.part_sparse) {
#pragma unroll
                        for (int s = 0; s < 2; ++s) {
                            const int rowA = warp * 32 + s * 16 + g, tokenA = qb * BLK + rowA;
                            const long long partA = (((long long)b * p.Lq + tokenA) * p.H + h) * p.part_stride + 2 * c2;
                            const long long partB = partA + 8ll * p.H * p.part_stride;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                if (rowA < BLK && tokenA < p.Lq) *reinterpret_cast<float2 *>(p.part_sparse + partA + 8 * j) = make_float2(0.f, 0.f);
                                if (rowA + 8 < BLK && tokenA + 8 < p.Lq) *reinterpret_cast<float2 *>(p.part_sparse + partB + 8 * j) = make_float2(0.f, 0.f);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 64; ++j) put_park(j, 0u);
                    }
                }
            }
            // ---- gate tile + combine ----
            // byte offset of this thread's 4 bytes inside 16-byte chunk j of a row in the swizzled 128 x 128 bf16 tiles
            auto tile_off = [&](int row, int j) -> int {
                return (j >> 3) * HALF_BYTES + row * 128 + (((j & 7) ^ (row & 7)) << 4) + 4 * c2;
            };
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bar->s_full, sg & 1u, abort_flag, sink, 10));
            if (ok) {
                ++sg;
                tc_fence_after();   // every product of the item has landed: the linear accumulator is complete, the V stage is free
                // Per slab: gate values of this thread's columns, rounded to bf16 as the reference's gate is (step j: word
                // 2j = row A, 2j + 1 = row B), then the linear accumulator, the combine and the staging of the result.
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    const uint32_t lane_addr = (uint32_t)(warp * 32 + s * 16) << 16;
                    const int rowA = warp * 32 + s * 16 + g, rowB = rowA + 8, tokenA = qb * BLK + rowA;
                    const bool okA = rowA < BLK && tokenA < p.Lq, okB = rowB < BLK && tokenA + 8 < p.Lq;
                    const long long partA = (((long long)b * p.Lq + tokenA) * p.H + h) * p.part_stride + 2 * c2;
                    const long long partB = partA + 8ll * p.H * p.part_stride;
                    uint32_t gpk[32];
                    if (!p.part_linear) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                            uint32_t gsc[16];
                            if (p.has_gate) {
                                TMEM_LDQ16(tmem_s + lane_addr + c * 32, gsc);
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
                                    // no gate module: gate = sigmoid(q); q is still in its shared-memory stage
                                    const uint32_t qa = *reinterpret_cast<const uint32_t *>(q_s + tile_off(rowA, jj));
                                    const uint32_t qbv = *reinterpret_cast<const uint32_t *>(q_s + tile_off(rowB, jj));
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
                    if (s == 1) {
                        // the gate scores and Q are consumed: S goes back to the issuer (next item's first scores), Q to the producer
                        tc_fence_before();
                        warp_arrive(&bar->p_full);
                        warp_arrive(&bar->q_empty);
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {   // 32 columns at a time
                        uint32_t o[16];
                        TMEM_LDQ16(tmem_o + lane_addr + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int jj = 4 * c + j;
                            const float a0 = __uint_as_float(o[4 * j]) * inv_lin[2 * s], a1 = __uint_as_float(o[4 * j + 1]) * inv_lin[2 * s];
                            const float b0 = __uint_as_float(o[4 * j + 2]) * inv_lin[2 * s + 1], b1 = __uint_as_float(o[4 * j + 3]) * inv_lin[2 * s + 1];
                            if (p.part_linear) {
                                if (okA) *reinterpret_cast<float2 *>(p.part_linear + partA + 8 * jj) = make_float2(a0, a1);
                                if (okB) *reinterpret_cast<float2 *>(p.part_linear + partB + 8 * jj) = make_float2(b0, b1);
                                continue;
                            }
                            const uint32_t spA = get_park(32 * s + 2 * jj), spB = get_park(32 * s + 2 * jj + 1);   // low half = even column
                            const uint32_t gA = gpk[2 * jj], gB = gpk[2 * jj + 1];
                            __nv_bfloat162 ra = __floats2bfloat162_rn(fmaf(a0, __uint_as_float(gA << 16), __uint_as_float(spA << 16)),
                                                                       fmaf(a1, __uint_as_float(gA & 0xffff0000u), __uint_as_float(spA & 0xffff0000u)));
                            __nv_bfloat162 rb = __floats2bfloat162_rn(fmaf(b0, __uint_as_float(gB << 16), __uint_as_float(spB << 16)),
                                                                       fmaf(b1, __uint_as_float(gB & 0xffff0000u), __uint_as_float(spB & 0xffff0000u)));
                            // the finished tile is staged in the V stage (free: every product has landed) in the layout the TMA store expects
                            *reinterpret_cast<uint32_t *>(v_s + tile_off(rowA, jj)) = *reinterpret_cast<uint32_t *>(&ra);
                            *reinterpret_cast<uint32_t *>(v_s + tile_off(rowB, jj)) = *reinterpret_cast<uint32_t *>(&rb);
                        }
                    }
                }
                // The accumulator is in registers / staged: the next item's first P.V product waits for the p_full of its
                // first tile, which this warp signals later in program order.
                tc_fence_before();
            }
            // Hand the staged tile to the store warp (in partial-output mode nothing was staged, but the V stage is
            // released the same way).
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            warp_arrive(&bar->out_ready);
            ++jcount;
        }
        tc_fence_before();
    }

    __syncthreads();
    tc_fence_after();
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace pair

int pair_kernel_prepare() {
    using namespace pair;
    static PerDeviceOnce attr_set;
    if (!attr_set.done()) {
        cudaError_t e = cudaFuncSetAttribute(hsa_fwd_sm100_pair_kernel<TILE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(hsa_fwd_sm100_pair_kernel<HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        // two CTAs need the largest shared-memory carve-out of the SM; ask for it rather than leave it to a heuristic
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(hsa_fwd_sm100_pair_kernel<TILE>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(hsa_fwd_sm100_pair_kernel<HALF>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return fail((int)e, "wa_hsa_forward(tcgen05): %s", cudaGetErrorString(e));
        attr_set.mark();
#ifdef WA_DEBUG_OCCUPANCY   // tuning aid: how many CTAs of this kernel the driver places on an SM
        cudaFuncAttributes fa{};
        cudaFuncGetAttributes(&fa, hsa_fwd_sm100_pair_kernel<TILE>);
        int dev = 0, smem_sm = 0, smem_res = 0, regs_sm = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
        cudaDeviceGetAttribute(&smem_res, cudaDevAttrReservedSharedMemoryPerBlock, dev);
        cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev);
        fprintf(stderr, "pair kernel: regs %d, static smem %zu, max dyn %d, carveout %d; device: smem/SM %d, reserved/block %d, regs/SM %d\n",
                fa.numRegs, fa.sharedSizeBytes, fa.maxDynamicSharedSizeBytes, fa.preferredShmemCarveout, smem_sm, smem_res, regs_sm);
        for (int bytes : {SMEM_BYTES, 110 * 1024, 100 * 1024, 96 * 1024, 64 * 1024, 32 * 1024}) {
            int n = -1;
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, hsa_fwd_sm100_pair_kernel<TILE>, THREADS, bytes);
            fprintf(stderr, "  dynamic smem %d -> %d CTAs per SM\n", bytes, n);
        }
#endif
    }
    return 0;
}

void pair_kernel_launch(int blk, int grid, cudaStream_t stream, const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv,
                        const CUtensorMap &tkc, const CUtensorMap &tvc, const CUtensorMap &tw, const CUtensorMap &tout,
                        const Params &kp) {
    using namespace pair;
    if (blk == TILE) hsa_fwd_sm100_pair_kernel<TILE><<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, tkc, tvc, tw, tout, kp);
    else hsa_fwd_sm100_pair_kernel<HALF><<<grid, THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, tkc, tvc, tw, tout, kp);
}

}  // namespace sm100
}  // namespace wa
