"""The tcgen05 fused kernel (bf16, head_dim 128, 128-token blocks) against the oracle and the SIMT kernels.

Routing ids/counts are produced by the same routing kernels on both paths and must be identical;
outputs meet max-abs 2e-2 / mean-rel 1e-2 against the oracle (the tolerance the benchmark definition states) and
are much closer to the library's own generic path.
"""
import math

import numpy as np
import pytest
import torch

from oracle import hsa_oracle as O
from tests.helpers import attention_error, dev, to_gpu, to_np

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_REL = 2e-2, 1e-2
D = 128


@pytest.fixture(scope="module")
def wa():
    import worldattention_b200 as pkg
    return pkg


def _draw(rng, shape, scale):
    return O.bf16_round((rng.standard_normal(shape) * scale).astype(np.float32))


def _proj(rank, seg, bs, rng):
    e = np.zeros((rank, seg), np.float32)
    for r in range(rank):
        lo, hi = r * bs, min((r + 1) * bs, seg)
        if hi > lo:
            e[r, lo:hi] = 1.0 / (hi - lo)
    return O.bf16_round(e + 0.002 * rng.standard_normal(e.shape).astype(np.float32))


def _run_case(wa, *, seed, bsz, heads, q_len, kv_len, seg, topk, scale, gate=True, coarse_len=None, whole_order=False):
    rng = np.random.default_rng(seed)
    q = _draw(rng, (bsz, q_len, heads, D), scale)
    k = _draw(rng, (bsz, kv_len, heads, D), scale)
    v = _draw(rng, (bsz, kv_len, heads, D), 1.0)
    ek = _proj(math.ceil(seg / 128), seg, 128, rng)
    gw = (rng.standard_normal((D, D)) * 0.05).astype(np.float32)
    gb = (rng.standard_normal((D,)) * 0.3).astype(np.float32)
    kc = vc = None
    if coarse_len:
        kc = _draw(rng, (bsz, coarse_len, heads, D), scale)
        vc = _draw(rng, (bsz, coarse_len, heads, D), 1.0)
    lin = None
    if gate:
        lin = torch.nn.Linear(D, D).to(dev())
        with torch.no_grad():
            lin.weight.copy_(to_gpu(gw)); lin.bias.copy_(to_gpu(gb))
    tk = None if topk is None else torch.tensor(topk, dtype=torch.int32)
    kwargs = dict(k_proj_mat=to_gpu(ek, "bf16"), v_proj_mat=to_gpu(ek, "bf16"), gate_lin=lin, block_size=128,
                  proj_segment_len=seg, topk_per_head=tk, return_routing=True)
    if coarse_len:
        kwargs.update(k_coarse=to_gpu(kc, "bf16"), v_coarse=to_gpu(vc, "bf16"))
    args = [to_gpu(x, "bf16") for x in (q, k, v)]
    out, (index, num, thr, used) = wa.hsa.hsa_attention(*args, check_status=True, **kwargs)
    assert used, "the tcgen05 kernel did not run"
    ref, (index_g, num_g, thr_g, used_g) = wa.hsa.hsa_attention(*args, force_generic=True, **kwargs)
    assert not used_g
    assert torch.equal(index, index_g) and torch.equal(num, num_g) and torch.equal(thr, thr_g)
    # bf16 rounding of the gate weights is the only arithmetic the generic path does not share
    gw_used = O.bf16_round(gw) if gate else None
    want, parts = O.hsa_attention(q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=ek, v_proj_mat=ek,
                                  gate_weight=gw_used, gate_bias=gb if gate else None, block_size=128,
                                  proj_segment_len=seg, dtype="bf16", topk_per_head=topk, return_parts=True)
    assert np.array_equal(to_np(num), parts["num"])
    if whole_order:      # the complete descending order of every row, not only the counts
        assert np.array_equal(to_np(index), parts["index"])
        assert np.array_equal(to_np(thr), parts["thresholds"])
    max_abs, mean_rel = attention_error(to_np(out), want)
    assert max_abs < MAX_ABS and mean_rel < MEAN_REL, ("vs oracle", max_abs, mean_rel)
    max_abs_g, mean_rel_g = attention_error(to_np(out), to_np(ref))
    assert max_abs_g < MAX_ABS and mean_rel_g < MEAN_REL, ("vs generic", max_abs_g, mean_rel_g)
    return to_np(out), parts


def test_small_ragged_shapes_fixed_topk(wa):
    _run_case(wa, seed=1, bsz=1, heads=2, q_len=300, kv_len=1170, seg=390, topk=[3, 10], scale=1.0 / math.sqrt(D))


def test_cumulative_mass_routing_batch_two(wa):
    _run_case(wa, seed=2, bsz=2, heads=3, q_len=520, kv_len=2000, seg=500, topk=None, scale=0.5)


def test_supplied_compressed_cache_spanning_several_tiles(wa):
    _run_case(wa, seed=3, bsz=1, heads=4, q_len=128, kv_len=900, seg=300, topk=[1, 8, 2, 5], scale=0.3, coarse_len=300)


def test_empty_selection_gives_the_linear_term_only(wa):
    out, parts = _run_case(wa, seed=4, bsz=1, heads=2, q_len=200, kv_len=700, seg=350, topk=[0, 4], scale=0.3)
    assert np.count_nonzero(parts["sparse"][:, :, 0]) == 0
    want = O.as_dtype(parts["linear"][:, :, 0] * parts["gate"][:, :, 0], "bf16")
    assert np.max(np.abs(out[:, :, 0] - want)) < MAX_ABS


def test_no_gate_module_uses_sigmoid_of_q(wa):
    _run_case(wa, seed=5, bsz=1, heads=2, q_len=256, kv_len=512, seg=256, topk=[2, 4], scale=0.4, gate=False)


def test_large_logits_exercise_the_running_max_rescale(wa):
    _run_case(wa, seed=6, bsz=1, heads=2, q_len=256, kv_len=2048, seg=512, topk=[16, 9], scale=3.0)


def test_thousands_of_key_blocks_route_several_rows_per_cta(wa):
    # 2063 key blocks: the routing kernel scores four or eight query blocks per CTA in one pass over the pooled keys; 5
    # query blocks = a full group and a ragged one.  Same order, counts and thresholds as the oracle.
    import os
    try:
        for rows in ("8", "4", "1"):      # rows scored per CTA: the launcher's choice depends on the SM count, so pin each
            os.environ["WA_B200_ROUTE_ROWS"] = rows
            _run_case(wa, seed=7, bsz=1, heads=2, q_len=600, kv_len=264000, seg=1320, topk=[3, 10], scale=1.0 / math.sqrt(D),
                      whole_order=True)
        os.environ["WA_B200_ROUTE_ROWS"] = "4"
        _run_case(wa, seed=8, bsz=2, heads=1, q_len=300, kv_len=262200, seg=1311, topk=None, scale=0.5, whole_order=True)
    finally:
        os.environ.pop("WA_B200_ROUTE_ROWS", None)


def test_fixed_counts_over_many_key_blocks_select_instead_of_sorting(wa):
    # without `return_routing` nobody reads the whole order, so the routing kernel picks each head's k best blocks by
    # radix select; the attention output must be the one the full sort gives, bit for bit (same ids, same order)
    rng = np.random.default_rng(12)
    heads, q_len, kv_len, seg = 3, 650, 160000, 1600
    q, k, v = (to_gpu(_draw(rng, (1, n, heads, D), s), "bf16") for n, s in ((q_len, 0.2), (kv_len, 0.2), (kv_len, 1.0)))
    ek = to_gpu(_proj(math.ceil(seg / 64), seg, 64, rng), "bf16")
    lin = torch.nn.Linear(D, D).to(dev())
    import os
    for topk, rows in (([32, 1, 7], "8"), ([0, 2600, 64], "4"), ([5, 9, 2], "1")):        # 2600 > 2500 key blocks: every block kept
        os.environ["WA_B200_ROUTE_ROWS"] = rows
        kw = dict(k_proj_mat=ek, v_proj_mat=ek, gate_lin=lin, block_size=64, proj_segment_len=seg,
                  topk_per_head=torch.tensor(topk, dtype=torch.int32), check_status=True)
        sorted_out, (index, num, _, used) = wa.hsa.hsa_attention(q, k, v, return_routing=True, **kw)
        picked_out = wa.hsa.hsa_attention(q, k, v, **kw)
        assert used and torch.equal(sorted_out, picked_out)
        assert num[0, :, 0].tolist() == [min(t, 2500) for t in topk]
    os.environ.pop("WA_B200_ROUTE_ROWS", None)


def test_config2_shape_head_adaptive_topk(wa):
    """Benchmark config 2 at full size: the property checked is agreement with the SIMT path of this library."""
    heads, q_len, kv_len, seg = 12, 4680, 32760, 1560
    g = torch.Generator().manual_seed(1)
    topk = torch.tensor([4, 8, 16, 32])[torch.randint(0, 4, (heads,), generator=g)].to(torch.int32)
    torch.manual_seed(1)
    q = (torch.randn(1, q_len, heads, D, device=dev()) / math.sqrt(D)).bfloat16()
    k = (torch.randn(1, kv_len, heads, D, device=dev()) / math.sqrt(D)).bfloat16()
    v = (torch.randn(1, kv_len, heads, D, device=dev()) / math.sqrt(D)).bfloat16()
    hsa = wa.hsa.HSAAttention(heads, D, block_size=128, proj_segment_len=seg).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        hsa.gate_lin.weight.normal_(0, 0.02)
        kc, vc = hsa.compress_kv_cache(k, v)
    kwargs = dict(k_coarse=kc, v_coarse=vc, k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin,
                  block_size=128, proj_segment_len=seg, topk_per_head=topk, return_routing=True)
    out, (index, num, _, used) = wa.hsa.hsa_attention(q, k, v, check_status=True, **kwargs)
    ref, (index_g, num_g, _, _) = wa.hsa.hsa_attention(q, k, v, force_generic=True, **kwargs)
    assert used and torch.equal(index, index_g) and torch.equal(num, num_g)
    assert torch.equal(num[0, :, 0].cpu(), topk)
    max_abs, mean_rel = attention_error(to_np(out), to_np(ref))
    assert max_abs < MAX_ABS and mean_rel < MEAN_REL, (max_abs, mean_rel)
    assert torch.isfinite(out).all()


def test_partial_output_mode_merges_to_the_full_result(wa):
    """Two key shards through the partial-output mode (tcgen05 kernel) merge to the single-pass result."""
    from worldattention_b200 import sharded
    from worldattention_b200.hsa import branches
    heads, q_len, kv_len, seg = 4, 300, 3120, 1560
    rng = np.random.default_rng(9)
    q, k, v = (to_gpu(_draw(rng, (1, n, heads, D), s), "bf16") for n, s in ((q_len, 0.3), (kv_len, 0.3), (kv_len, 1.0)))
    hsa = wa.hsa.HSAAttention(heads, D, block_size=128, proj_segment_len=seg).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        hsa.gate_lin.weight.normal_(0, 0.05)
    hsa.topk_per_head = torch.tensor([3, 9, 1, 25], dtype=torch.int32)
    kc, vc = hsa.compress_kv_cache(k, v)
    want, (index, num, _, used) = wa.hsa.hsa_attention(
        q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin,
        block_size=128, proj_segment_len=seg, topk_per_head=hsa.topk_per_head, return_routing=True)
    assert used
    shards = sharded.plan_kv_shards(kv_len, 128, 2, seg)
    outs_s, lses_s, outs_l, lses_l = [], [], [], []
    r, blk = hsa.proj_rank, 0
    for i, (lo, hi) in enumerate(shards):
        nb = -(-(hi - lo) // 128)
        idx_l, num_l = sharded.local_selection(index, num, blk, blk + nb)
        blk += nb
        s_lo, s_hi = -(-lo // seg), (-(-hi // seg) if i == 0 else kv_len // seg)   # segments partitioned by start token
        o_s, l_s, o_l, l_l, tuned = branches.hsa_partials(q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                                                          kc[:, s_lo * r:s_hi * r].contiguous(),
                                                          vc[:, s_lo * r:s_hi * r].contiguous(), idx_l, num_l, 128)
        assert tuned
        rows = lambda o: o.permute(0, 2, 1, 3).reshape(-1, D)
        outs_s.append(rows(o_s)); lses_s.append(l_s.reshape(-1)); outs_l.append(rows(o_l)); lses_l.append(l_l.reshape(-1))
    sp, _ = branches.merge_partials(torch.stack(outs_s), torch.stack(lses_s))
    li, _ = branches.merge_partials(torch.stack(outs_l), torch.stack(lses_l))
    back = lambda x: x.view(1, heads, q_len, D).permute(0, 2, 1, 3).contiguous()
    got = branches.gate_combine(q, back(sp).to(torch.bfloat16), back(li), hsa.gate_lin, round_bf16=True)
    max_abs, mean_rel = attention_error(to_np(got), to_np(want))
    assert max_abs < MAX_ABS and mean_rel < MEAN_REL, (max_abs, mean_rel)


def test_head_slices_of_a_resident_cache_equal_the_full_call(wa):
    """Heads are independent: the layer on a strided head slice of q/k/v/compressed cache gives that slice of the
    full result bit for bit (what the pipelined end-to-end step and the head-split sharding rely on)."""
    heads, q_len, kv_len, seg = 6, 700, 3120, 1560
    rng = np.random.default_rng(11)
    q, k, v = (to_gpu(_draw(rng, (1, n, heads, D), s), "bf16") for n, s in ((q_len, 0.3), (kv_len, 0.3), (kv_len, 1.0)))
    hsa = wa.hsa.HSAAttention(heads, D, block_size=128, proj_segment_len=seg).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        hsa.gate_lin.weight.normal_(0, 0.05)
        kc, vc = hsa.compress_kv_cache(k, v)
    topk = torch.tensor([3, 9, 1, 25, 4, 16], dtype=torch.int32, device=dev())
    common = dict(k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin, block_size=128,
                  proj_segment_len=seg, return_routing=True)
    full, (_, num, _, used) = wa.hsa.hsa_attention(q, k, v, k_coarse=kc, v_coarse=vc, topk_per_head=topk, **common)
    assert used
    for hs in (slice(0, 2), slice(2, 6)):
        part, (_, num_p, _, used_p) = wa.hsa.hsa_attention(q[:, :, hs], k[:, :, hs], v[:, :, hs], k_coarse=kc[:, :, hs],
                                                           v_coarse=vc[:, :, hs], topk_per_head=topk[hs], **common)
        assert used_p and not q[:, :, hs].is_contiguous()
        assert torch.equal(num_p, num[:, hs])
        assert torch.equal(part, full[:, :, hs])


def _run_case_64(wa, *, seed, heads, q_len, kv_len, seg, topk, scale=0.3, bsz=1):
    bs = 64
    rng = np.random.default_rng(seed)
    q = _draw(rng, (bsz, q_len, heads, D), scale)
    k = _draw(rng, (bsz, kv_len, heads, D), scale)
    v = _draw(rng, (bsz, kv_len, heads, D), 1.0)
    ek = _proj(math.ceil(seg / bs), seg, bs, rng)
    gw = (rng.standard_normal((D, D)) * 0.05).astype(np.float32)
    gb = (rng.standard_normal((D,)) * 0.3).astype(np.float32)
    lin = torch.nn.Linear(D, D).to(dev())
    with torch.no_grad():
        lin.weight.copy_(to_gpu(gw)); lin.bias.copy_(to_gpu(gb))
    tk = None if topk is None else torch.tensor(topk, dtype=torch.int32)
    kwargs = dict(k_proj_mat=to_gpu(ek, "bf16"), v_proj_mat=to_gpu(ek, "bf16"), gate_lin=lin, block_size=bs,
                  proj_segment_len=seg, topk_per_head=tk, return_routing=True)
    args = [to_gpu(x, "bf16") for x in (q, k, v)]
    out, (index, num, _, used) = wa.hsa.hsa_attention(*args, check_status=True, **kwargs)
    ref, (index_g, num_g, _, used_g) = wa.hsa.hsa_attention(*args, force_generic=True, **kwargs)
    assert used and not used_g
    assert torch.equal(index, index_g) and torch.equal(num, num_g)
    want = O.hsa_attention(q, k, v, k_proj_mat=ek, v_proj_mat=ek, gate_weight=O.bf16_round(gw), gate_bias=gb, block_size=bs,
                           proj_segment_len=seg, dtype="bf16", topk_per_head=topk)
    max_abs, mean_rel = attention_error(to_np(out), want)
    assert max_abs < MAX_ABS and mean_rel < MEAN_REL, ("vs oracle", max_abs, mean_rel)
    max_abs_g, mean_rel_g = attention_error(to_np(out), to_np(ref))
    assert max_abs_g < MAX_ABS and mean_rel_g < MEAN_REL, ("vs generic", max_abs_g, mean_rel_g)


def test_64_token_blocks_run_on_the_tcgen05_kernel(wa):
    """Routing block size 64 (the reference class's default): a work item is a 64-row query block and a key tile holds
    two selected blocks.  Odd and even counts, an empty head, ragged query and key tails."""
    _run_case_64(wa, seed=21, heads=3, q_len=500, kv_len=2100, seg=700, topk=[5, 12, 0])
    _run_case_64(wa, seed=24, heads=2, q_len=150, kv_len=1400, seg=700, topk=[7, 2], bsz=2)


def test_64_token_blocks_with_the_ragged_last_key_block_anywhere_in_the_list(wa):
    """Every key block selected (33 blocks, the last one 40 tokens): the short block sits wherever the routing order puts
    it, in the first or the second half of a tile; cumulative-mass routing for the second case."""
    _run_case_64(wa, seed=22, heads=2, q_len=200, kv_len=2088, seg=696, topk=[33, 32])
    _run_case_64(wa, seed=23, heads=2, q_len=130, kv_len=1000, seg=500, topk=None, scale=0.5)


def test_pooled_key_cache_gives_the_same_result_and_only_pools_new_blocks(wa):
    """The caller-kept pooled-key buffer: a first call fills it, a later call on the grown cache trusts the rows of
    the blocks that were complete before and pools only the rest; outputs and routing equal the plain call."""
    heads, q_len, kv_old, kv_len, seg = 3, 300, 1560, 3120, 1560
    rng = np.random.default_rng(31)
    q, k, v = (to_gpu(_draw(rng, (1, n, heads, D), s), "bf16") for n, s in ((q_len, 0.3), (kv_len, 0.3), (kv_len, 1.0)))
    hsa = wa.hsa.HSAAttention(heads, D, block_size=128, proj_segment_len=seg).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        hsa.gate_lin.weight.normal_(0, 0.05)
    common = dict(k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin, block_size=128,
                  proj_segment_len=seg, return_routing=True)
    nb_old, nb_new = -(-kv_old // 128), -(-kv_len // 128)
    # call 1 on the old cache fills the buffer
    cache_old = torch.full((1, heads, nb_old, D), float("nan"), device=dev())
    out1, (idx1, num1, _, _) = wa.hsa.hsa_attention(q, k[:, :kv_old], v[:, :kv_old], k_pooled_cache=cache_old, **common)
    plain1, (pidx1, pnum1, _, _) = wa.hsa.hsa_attention(q, k[:, :kv_old], v[:, :kv_old], **common)
    assert torch.equal(out1, plain1) and torch.equal(idx1, pidx1) and torch.equal(num1, pnum1)
    assert torch.isfinite(cache_old).all()
    # call 2 on the grown cache: the blocks that were complete (kv_old // 128) are trusted, the rest recomputed
    valid = kv_old // 128
    cache_new = torch.full((1, heads, nb_new, D), float("nan"), device=dev())
    cache_new[:, :, :valid] = cache_old[:, :, :valid]
    out2, (idx2, num2, _, used) = wa.hsa.hsa_attention(q, k, v, k_pooled_cache=cache_new, k_pooled_valid=valid, **common)
    plain2, (pidx2, pnum2, _, _) = wa.hsa.hsa_attention(q, k, v, **common)
    assert used and torch.equal(out2, plain2) and torch.equal(idx2, pidx2) and torch.equal(num2, pnum2)
    assert torch.isfinite(cache_new).all()
    # the trusted rows are really not recomputed: a poisoned trusted row changes the routing
    cache_bad = cache_new.clone()
    cache_bad[:, :, 0] = 50.0
    _, (idx3, _, _, _) = wa.hsa.hsa_attention(q, k, v, k_pooled_cache=cache_bad, k_pooled_valid=valid, **common)
    assert not torch.equal(idx3, pidx2) and torch.equal(cache_bad[:, :, 0], torch.full_like(cache_bad[:, :, 0], 50.0))
