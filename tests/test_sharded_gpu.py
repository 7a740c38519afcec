"""GPU pieces of the KV-sharded path that need no second GPU."""
import numpy as np
import pytest
import torch

from tests.helpers import dev

pytestmark = pytest.mark.gpu


def test_local_selection_kernel_matches_the_tensor_formulation():
    """`wa_route_local_selection` against the same restriction written with tensor operations (CPU)."""
    from worldattention_b200 import sharded
    rng = np.random.default_rng(5)
    for nkv, lo, hi in ((256, 0, 128), (256, 128, 256), (70, 33, 70), (5, 0, 5), (300, 10, 11)):
        rows = (2, 3, 7)
        index = np.stack([rng.permutation(nkv) for _ in range(int(np.prod(rows)))]).reshape(*rows, nkv).astype(np.int32)
        index[0, 0, 0, :3] = index[0, 0, 0, 0]          # duplicates are allowed and collapse
        index[1, 2, 3, 0] = nkv + 7                      # out-of-range ids are clamped
        num = rng.integers(0, nkv + 1, size=rows).astype(np.int32)
        num[0, 1, 2] = 0
        want_idx, want_num = sharded.local_selection(torch.from_numpy(index), torch.from_numpy(num), lo, hi)
        got_idx, got_num = sharded.local_selection(torch.from_numpy(index).to(dev()), torch.from_numpy(num).to(dev()), lo, hi)
        assert torch.equal(got_num.cpu(), want_num)
        assert torch.equal(got_idx.cpu(), want_idx)


def _emulated_kv_shard_forward(wa, hsa, q, k, v, kc, vc, topk, world, routing, seg):
    """The KV-sharded forward with the ranks played one after another on ONE GPU: every collective is replaced by the
    slicing it amounts to (no process group, no kernel waits for another)."""
    from worldattention_b200 import sharded
    from worldattention_b200.hsa import branches
    from worldattention_b200.hsa.routing import block_attention_map, build_block_routing
    bs = hsa.block_size
    _, q_len, heads, d = q.shape
    kv_len = k.shape[1]
    shards = sharded.plan_kv_shards(kv_len, bs, world, seg)
    blocks = [-(-(b - a) // bs) for a, b in shards]
    q_pooled = sharded._pool_blhd(q, bs)
    pooled = [sharded._pool_blhd(k[:, a:b].contiguous(), bs) if b > a else q_pooled.new_zeros((1, heads, 0, d)) for a, b in shards]
    nq = q_pooled.shape[2]
    if routing == "candidates":
        kmax = int(topk.max())
        every = torch.stack([sharded.local_candidates(q_pooled, pooled[r], block_lo=sum(blocks[:r]), topk_max=kmax)
                             for r in range(world)])
        sel = [sharded.merge_candidates(every, (1, heads, nq), topk_per_head=topk, blocks_total=sum(blocks),
                                        block_lo=sum(blocks[:r]), block_hi=sum(blocks[:r + 1])) for r in range(world)]
    else:
        decided = build_block_routing(block_attention_map(q_pooled, torch.cat(pooled, dim=2)), hsa.tau_min, hsa.tau_max,
                                      topk_per_head=topk)
        sel = [sharded.local_selection(decided.index, decided.num, sum(blocks[:r]), sum(blocks[:r + 1])) for r in range(world)]
    rp, row_plan = sharded.exchange_rows(q_len, world)
    rec = branches.record_floats(d)
    r_ = hsa.proj_rank
    sent = []
    for r, (a, b) in enumerate(shards):
        records = torch.full((1, rp * world, heads, rec), float("nan"), device=q.device)
        records[:, q_len:] = 0
        s_lo = -(-a // seg)
        s_hi = -(-b // seg) if r < world - 1 else -(-kv_len // seg)
        sharded.partial_records(q, k[:, a:b].contiguous(), v[:, a:b].contiguous(), kc[:, s_lo * r_: s_hi * r_].contiguous(),
                                vc[:, s_lo * r_: s_hi * r_].contiguous(), sel[r][0], sel[r][1], bs, records)
        assert torch.isfinite(records[:, :, :, :2 * d]).all()
        sent.append(records[0])
    out = torch.empty_like(q)
    for j, (first, count) in enumerate(row_plan):      # what rank j receives: slice j of every rank's records
        recv = torch.stack([s[j * rp:(j + 1) * rp] for s in sent])                       # [W, rp, H, rec]
        sparse, linear = branches.merge_packed(recv.view(world, rp * heads, rec), d)
        if count:
            out[:, first:first + count] = branches.gate_combine(
                q[:, first:first + count], sparse.view(1, rp, heads, d)[:, :count], linear.view(1, rp, heads, d)[:, :count],
                hsa.gate_lin, round_bf16=True)
    return out, sel


@pytest.mark.parametrize("routing,world", [("gather", 3), ("candidates", 3), ("candidates", 8)])
def test_kv_shard_pipeline_emulated_on_one_gpu(routing, world):
    """Packed partial records, their merge and the candidate routing against the single-GPU forward."""
    import worldattention_b200 as wa
    heads, d, q_len, kv_len, seg, bs = 4, 128, 333, 12480, 1560, 128      # 8 segments: every shard of 3 or 8 owns at least one
    g = torch.Generator().manual_seed(2)
    q = (torch.randn(1, q_len, heads, d, generator=g) * 0.6).to(dev(), torch.bfloat16)
    k = (torch.randn(1, kv_len, heads, d, generator=g) * 0.6).to(dev(), torch.bfloat16)
    v = torch.randn(1, kv_len, heads, d, generator=g).to(dev(), torch.bfloat16)
    hsa = wa.hsa.HSAAttention(heads, d, block_size=bs, proj_segment_len=seg).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        hsa.gate_lin.weight.normal_(0, 0.05)
        kc, vc = hsa.compress_kv_cache(k, v)
    topk = torch.tensor([3, 17, 1, 8], dtype=torch.int32, device=dev())
    want, (index, num, _, used) = wa.hsa.hsa_attention(q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=hsa.k_proj_mat,
                                                       v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin, block_size=bs,
                                                       proj_segment_len=seg, topk_per_head=topk, return_routing=True)
    assert used
    got, sel = _emulated_kv_shard_forward(wa, hsa, q, k, v, kc, vc, topk, world, routing, seg)
    # the union of the shards' selections is the single-GPU selection (logits here are far apart: no equal probabilities)
    nkv = index.shape[-1]
    from worldattention_b200 import sharded
    shards = sharded.plan_kv_shards(kv_len, bs, world, seg)
    blocks = [-(-(b - a) // bs) for a, b in shards]
    chosen = torch.zeros((1, heads, index.shape[2], nkv + 1), dtype=torch.bool, device=dev())
    for r in range(world):
        idx, n = sel[r]
        slots = torch.arange(idx.shape[-1], device=dev())[None, None, None, :] < n[..., None]
        # entries past the count are not part of the selection (and may be anything): park them in the spare column
        ids = torch.where(slots, (idx.long() + sum(blocks[:r])).clamp(0, nkv - 1), torch.full_like(idx.long(), nkv))
        chosen.scatter_(-1, ids, torch.ones_like(slots))
    want_sel = torch.zeros_like(chosen)
    slots = torch.arange(nkv, device=dev())[None, None, None, :] < num[..., None]
    want_sel.scatter_(-1, torch.where(slots, index.long(), torch.full_like(index.long(), nkv)), torch.ones_like(slots))
    assert torch.equal(chosen[..., :nkv], want_sel[..., :nkv])
    diff = (got.float() - want.float()).abs()
    assert float(diff.max()) < 2e-2 and float(diff.mean() / want.float().abs().mean()) < 1e-2


def test_local_candidates_of_a_long_shard_are_the_best_blocks_in_order():
    """Thousands of local key blocks: the candidate kernel selects instead of sorting; the candidates must still be the
    `topk_max` highest logits of the row, best first, as (descending logit, ascending global id) keys."""
    from worldattention_b200 import sharded
    rng = np.random.default_rng(21)
    heads, nq, d, block_lo, kcap = 2, 3, 128, 5000, 32
    for nloc in (3000, 700):                                    # radix selection; full sort
        q = rng.standard_normal((1, heads, nq, d)).astype(np.float32)
        k = rng.standard_normal((1, heads, nloc, d)).astype(np.float32)
        cand = sharded.local_candidates(torch.from_numpy(q).to(dev()), torch.from_numpy(k).to(dev()), block_lo=block_lo,
                                        topk_max=kcap).cpu().numpy().view(np.uint64).reshape(heads, nq, kcap)
        logits = np.einsum("hqd,hkd->hqk", q[0].astype(np.float64), k[0].astype(np.float64))
        for h in range(heads):
            for i in range(nq):
                keys = cand[h, i]
                assert np.all(keys[:-1] < keys[1:])                                        # ascending keys = best first
                ids = (keys & np.uint64(0xFFFFFFFF)).astype(np.int64) - block_lo
                assert np.array_equal(ids, np.argsort(-logits[h, i], kind="stable")[:kcap])


@pytest.mark.parametrize("world", [3, 8])
def test_partial_records_stored_into_the_merging_ranks_buffers(world):
    """The peer-store form of the exchange with the ranks' receive buffers all on one GPU: every "rank" runs the partial
    kernel with the distances to the other buffers, and each buffer must end up holding exactly what the all-to-all form
    delivers (slice j of every rank's records)."""
    import worldattention_b200 as wa
    from worldattention_b200 import sharded
    from worldattention_b200.hsa import branches
    from worldattention_b200.hsa.routing import block_attention_map, build_block_routing
    heads, d, q_len, kv_len, seg, bs = 4, 128, 333, 24960, 1560, 128      # 16 segments: every shard owns compressed slots
    g = torch.Generator().manual_seed(4)
    q = (torch.randn(1, q_len, heads, d, generator=g) * 0.6).to(dev(), torch.bfloat16)
    k = (torch.randn(1, kv_len, heads, d, generator=g) * 0.6).to(dev(), torch.bfloat16)
    v = torch.randn(1, kv_len, heads, d, generator=g).to(dev(), torch.bfloat16)
    hsa = wa.hsa.HSAAttention(heads, d, block_size=bs, proj_segment_len=seg).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        kc, vc = hsa.compress_kv_cache(k, v)
    topk = torch.tensor([3, 17, 1, 8], dtype=torch.int32, device=dev())
    shards = sharded.plan_kv_shards(kv_len, bs, world, seg)
    blocks = [-(-(b - a) // bs) for a, b in shards]
    q_pooled = sharded._pool_blhd(q, bs)
    pooled = torch.cat([sharded._pool_blhd(k[:, a:b].contiguous(), bs) for a, b in shards], dim=2)
    decided = build_block_routing(block_attention_map(q_pooled, pooled), hsa.tau_min, hsa.tau_max, topk_per_head=topk)
    rp, _ = sharded.exchange_rows(q_len, world)
    rec = branches.record_floats(d)
    receive = [torch.zeros((1, world * rp, heads, rec), device=dev()) for _ in range(world)]      # one buffer per "rank"
    r_ = hsa.proj_rank
    sent = []
    for r, (a, b) in enumerate(shards):
        idx, n = sharded.local_selection(decided.index, decided.num, sum(blocks[:r]), sum(blocks[:r + 1]))
        s_lo, s_hi = -(-a // seg), (-(-b // seg) if r < world - 1 else -(-kv_len // seg))
        args = (q, k[:, a:b].contiguous(), v[:, a:b].contiguous(), kc[:, s_lo * r_: s_hi * r_].contiguous(),
                vc[:, s_lo * r_: s_hi * r_].contiguous(), idx, n, bs)
        plain = torch.zeros((1, rp * world, heads, rec), device=dev())
        assert branches.hsa_partials_packed(*args, plain)
        sent.append(plain[0])
        deltas = [(receive[t].data_ptr() - receive[r].data_ptr()) // 4 for t in range(world)]
        assert branches.hsa_partials_packed(*args, receive[r], peer=(rp, r, deltas))
    torch.cuda.synchronize()
    for j in range(world):
        want = torch.stack([s[j * rp:(j + 1) * rp] for s in sent])                           # [W, rp, H, rec]
        got = receive[j][0].view(world, rp, heads, rec)
        rows = max(0, min(q_len, (j + 1) * rp) - j * rp)
        assert torch.equal(got[:, :rows], want[:, :rows]), j
        assert torch.count_nonzero(got[:, rows:]) == 0
