"""GPU parity of the HSA kernels against the numpy oracle and the reference-generated vectors.

Integer outputs (block ids, counts) must be bit-exact; float outputs meet the stated tolerances:
fp32 paths 1e-4 absolute, attention outputs max-abs 2e-2 and mean-rel 1e-2 (the reference's own
composition tolerance, tests/test_hsa_attention.py:91-99).
"""
import math

import numpy as np
import pytest
import torch

from oracle import hsa_oracle as O
from tests.helpers import attention_error, dev, tie_aware_index_check, to_gpu, to_np

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_REL = 2e-2, 1e-2


@pytest.fixture(scope="module")
def wa():
    import worldattention_b200 as pkg
    return pkg


# ---------------------------------------------------------------- routing
def test_routing_is_bit_exact_against_oracle_and_reference(wa, golden):
    for name in ("routing_small", "routing_wide"):
        g = golden(name)
        tau_min, tau_max = float(g["tau"][0]), float(g["tau"][1])
        r = wa.hsa.build_block_routing(to_gpu(g["block_attn"]), tau_min, tau_max, return_mask=True)
        index, num, mask, thr = O.build_block_routing(g["block_attn"], tau_min, tau_max, return_mask=True)
        assert np.array_equal(to_np(r.index), index)
        assert np.array_equal(to_np(r.num), num)
        assert np.array_equal(to_np(r.mask), mask)
        assert np.array_equal(to_np(r.thresholds), thr)
        # and against what the reference itself produced
        assert np.array_equal(to_np(r.num), g["num"])
        np.testing.assert_allclose(to_np(r.thresholds), g["thresholds"], atol=1e-6)
        tie_aware_index_check(g["block_attn"], to_np(r.index), g["index"])


def test_routing_ties_and_degenerate_rows(wa):
    n = 16
    uniform = np.full((1, 1, 1, n), 1.0 / n, np.float32)
    one_hot = np.zeros((1, 1, 1, n), np.float32)
    one_hot[..., 3] = 1.0
    ru = wa.hsa.build_block_routing(to_gpu(uniform), 0.0, 1.0)
    rh = wa.hsa.build_block_routing(to_gpu(one_hot), 0.0, 1.0)
    assert abs(float(ru.thresholds[0])) < 1e-6
    assert abs(float(rh.thresholds[0]) - (n - 1) / n) < 1e-6
    # equal probabilities come out in ascending id order
    assert to_np(ru.index)[0, 0, 0].tolist() == list(range(n))
    assert to_np(rh.index)[0, 0, 0].tolist() == [3] + [i for i in range(n) if i != 3]
    assert int(ru.num[0, 0, 0]) == 0          # tau_h = 0: nothing is kept
    assert int(rh.num[0, 0, 0]) == 1
    both = np.stack([uniform[0, 0], one_hot[0, 0]], axis=0)[None]
    thr = to_np(wa.hsa.build_block_routing(to_gpu(both), 0.35, 1.0).thresholds)
    assert thr.shape == (2,) and thr[1] > thr[0] + 0.5


def test_routing_large_rows_and_fixed_topk(wa):
    rng = np.random.default_rng(5)
    attn = rng.standard_normal((1, 3, 4, 5850)).astype(np.float32) * 2
    attn = np.exp(attn - attn.max(-1, keepdims=True))
    attn = (attn / attn.sum(-1, keepdims=True)).astype(np.float32)
    attn[0, 0, 0, 100:140] = attn[0, 0, 0, 100]          # a run of exact ties
    r = wa.hsa.build_block_routing(to_gpu(attn), 0.35, 1.0, return_mask=True)
    index, num, mask, thr = O.build_block_routing(attn, 0.35, 1.0, return_mask=True)
    assert np.array_equal(to_np(r.index), index)
    assert np.array_equal(to_np(r.num), num)
    assert np.array_equal(to_np(r.mask), mask)
    assert np.array_equal(to_np(r.thresholds), thr)
    k = torch.tensor([4, 32, 9000], dtype=torch.int32)
    rk = wa.hsa.build_block_routing(to_gpu(attn), 0.35, 1.0, topk_per_head=k, return_mask=True)
    assert np.array_equal(to_np(rk.index), index)
    assert np.array_equal(to_np(rk.num), O.fixed_topk_num([4, 32, 9000], 1, 4, 5850))
    assert np.array_equal(to_np(rk.mask).sum(-1), to_np(rk.num))


def test_block_mean_pool_matches_oracle_and_reference(wa, golden):
    for name in ("pool_ragged_fp32", "pool_aligned_fp32", "pool_ragged_bf16", "pool_aligned_bf16"):
        g = golden(name)
        dtype = "bf16" if name.endswith("bf16") else "fp32"
        bs, length = int(g["block_size"]), int(g["length"])
        nb = g["x"].shape[2] // bs
        got = wa.hsa.block_mean_pool(to_gpu(g["x"], dtype), length, nb, bs)
        want = O.block_mean_pool(g["x"], length, nb, bs, dtype)
        assert np.array_equal(to_np(got), want), name
        np.testing.assert_allclose(to_np(got), g["pooled"], atol=2e-6 if dtype == "fp32" else 0, rtol=0)
        assert got.dtype == (torch.float32 if length % bs else to_gpu(g["x"], dtype).dtype)
    x = np.zeros((1, 1, 12, 2), np.float32)
    x[0, 0, :10] = 1.0
    pooled = wa.hsa.block_mean_pool(to_gpu(x), 10, 3, 4)
    assert torch.allclose(pooled[0, 0, 2], torch.ones(2, device=dev()))


def test_block_mean_pool_token_major_rows_take_the_tma_stream(wa):
    # [B, L, H, D] storage (what the forward hands over) is pooled by the TMA kernel; same bits as the oracle
    rng = np.random.default_rng(11)
    for B, L, H, D, bs in ((2, 700, 3, 64, 128), (1, 768, 2, 128, 128), (2, 333, 4, 32, 64), (1, 4680, 12, 128, 64),
                           (1, 130, 1, 64, 128), (2, 333, 8, 32, 64), (2, 700, 4, 64, 128), (1, 130, 4, 64, 128),
                           (1, 4680, 12, 128, 128), (3, 64, 2, 128, 32)):
        nb = -(-L // bs)
        x = (rng.standard_normal((B, nb * bs, H, D)) * 3).astype(np.float32)
        x[:, L:] = 7.0                                            # padding rows must not reach the means
        xt = to_gpu(x, "bf16")                                    # [B, tokens, H, D]
        got = wa.hsa.block_mean_pool(xt.permute(0, 2, 1, 3), L, nb, bs)
        xh = to_np(xt.float()).transpose(0, 2, 1, 3).copy()
        xh[:, :, L:] = 0.0
        want = O.block_mean_pool(xh, L, nb, bs, "bf16")
        assert np.array_equal(to_np(got.float()), want), (B, L, H, D, bs)


def test_block_attention_map_matches_oracle(wa, golden):
    g = golden("block_map")
    got = to_np(wa.hsa.block_attention_map(to_gpu(g["q_pooled"]), to_gpu(g["k_pooled"])))
    want = O.block_attention_map(g["q_pooled"], g["k_pooled"])
    assert np.max(np.abs(got.view(np.int32) - want.view(np.int32))) <= 1       # <= 1 ulp (exp rounding)
    np.testing.assert_allclose(got, g["block_attn"], rtol=2e-6, atol=1e-8)
    np.testing.assert_allclose(got.sum(-1), 1.0, atol=1e-5)


# ---------------------------------------------------------------- sparse branch
def test_sparse_branch_matches_reference_vectors(wa, golden):
    g = golden("sparse_ref")
    bs = int(g["block_size"])
    args = [to_gpu(g[k], "bf16") for k in ("q", "k", "v")]
    got = wa.hsa.block_sparse_attention_reference(*args, to_gpu(g["index"]), to_gpu(g["num"]), to_gpu(g["sizes"]), bs)
    assert got.dtype == torch.bfloat16
    np.testing.assert_allclose(to_np(got), g["out"], rtol=2 ** -7, atol=1e-6)
    assert torch.count_nonzero(got[0, 1, :bs]) == 0                 # num == 0 -> exact zeros
    # slots past num are ignored, ids are clamped instead of faulting
    scrambled = g["index"].copy()
    for h in range(2):
        for i in range(3):
            n = int(g["num"][0, h, i])
            scrambled[0, h, i, n:] = 10_000 + i
    got2 = wa.hsa.block_sparse_attention_reference(*args, to_gpu(scrambled), to_gpu(g["num"]), to_gpu(g["sizes"]), bs)
    assert torch.equal(got, got2)
    # the Triton-backend signature serves the same result
    from worldattention_b200.hsa.block_sparse_triton import block_sparse_attention, map_to_index
    got3 = block_sparse_attention(*args, block_sizes=to_gpu(g["sizes"]), q2k_index=to_gpu(g["index"]),
                                  q2k_num=to_gpu(g["num"]))
    assert torch.equal(got, got3)
    mask = np.zeros((1, 2, 3, 5), bool)
    for h in range(2):
        for i in range(3):
            mask[0, h, i, g["index"][0, h, i, : g["num"][0, h, i]]] = True
    idx, cnt = map_to_index(torch.from_numpy(mask).to(dev()))
    want_idx, want_cnt = O.map_to_index(mask)
    assert np.array_equal(to_np(idx), want_idx) and np.array_equal(to_np(cnt), want_cnt)


def test_sparse_branch_full_selection_is_dense_attention(wa):
    torch.manual_seed(0)
    b, h, n, d, bs = 1, 2, 128, 16, 64
    q, k, v = (torch.randn(b, h, n, d, device=dev()) for _ in range(3))
    nb = n // bs
    index = torch.arange(nb, dtype=torch.int32, device=dev()).view(1, 1, 1, nb).expand(b, h, nb, nb).contiguous()
    num = torch.full((b, h, nb), nb, dtype=torch.int32, device=dev())
    sizes = torch.full((nb,), bs, dtype=torch.int32, device=dev())
    got, lse = wa.hsa.block_sparse_attention_reference(q, k, v, index, num, sizes, bs, return_lse=True)
    want, want_lse = O.block_sparse_attention(to_np(q), to_np(k), to_np(v), to_np(index), to_np(num), to_np(sizes), bs,
                                              dtype="fp32", return_lse=True)
    np.testing.assert_allclose(to_np(got), want, atol=1e-5)
    np.testing.assert_allclose(to_np(lse), want_lse, atol=1e-5)
    dense = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    assert torch.allclose(got, dense, atol=1e-5)


# ---------------------------------------------------------------- compressed branch
def test_compress_and_linear_branch(wa, golden):
    from worldattention_b200.hsa.attention import _linear_branch
    for name, dtype, tol in (("compress_linear_fp32", "fp32", 1e-5), ("compress_linear_bf16", "bf16", 2 ** -7)):
        g = golden(name)
        kc, vc = wa.hsa.compress_kv(to_gpu(g["k"], dtype), to_gpu(g["v"], dtype), segment_len=int(g["segment_len"]),
                                    k_proj_mat=to_gpu(g["ek"], "bf16"), v_proj_mat=to_gpu(g["ev"], "bf16"),
                                    block_size=int(g["block_size"]))
        assert tuple(kc.shape) == g["kc"].shape
        np.testing.assert_allclose(to_np(kc), g["kc"], rtol=tol, atol=1e-5)
        np.testing.assert_allclose(to_np(vc), g["vc"], rtol=tol, atol=1e-5)
        lin = _linear_branch(to_gpu(g["q"], dtype), to_gpu(g["kc"], dtype), to_gpu(g["vc"], dtype))
        np.testing.assert_allclose(to_np(lin), g["linear"], rtol=2 * tol, atol=1e-5 if dtype == "fp32" else 2e-2)
    with pytest.raises(ValueError):
        wa.hsa.compress_kv(to_gpu(g["k"]), to_gpu(g["v"]), segment_len=60, k_proj_mat=to_gpu(g["ek"], "bf16"),
                           v_proj_mat=to_gpu(g["ev"], "bf16"), block_size=32)


# ---------------------------------------------------------------- whole forward
def _module(wa, g, heads, d, dtype):
    hsa = wa.hsa.HSAAttention(num_heads=heads, head_dim=d, block_size=int(g["block_size"]), tau_min=float(g["tau"][0]),
                              tau_max=float(g["tau"][1]), proj_segment_len=int(g["segment_len"]), backend="torch").to(dev())
    with torch.no_grad():
        hsa.k_proj_mat.copy_(to_gpu(g["ek"], "bf16"))
        hsa.v_proj_mat.copy_(to_gpu(g["ev"], "bf16"))
        hsa.gate_lin.weight.copy_(to_gpu(g["gw"]))
        hsa.gate_lin.bias.copy_(to_gpu(g["gb"]))
    return hsa


def test_forward_matches_reference_vectors(wa, golden):
    for name, dtype in (("hsa_fp32", "fp32"), ("hsa_bf16", "bf16")):
        g = golden(name)
        _, q_len, heads, d = g["q"].shape
        hsa = _module(wa, g, heads, d, dtype)
        q, k, v = (to_gpu(g[x], dtype) for x in ("q", "k", "v"))
        with torch.no_grad():
            out = hsa(q, k, v)
            cached = hsa(q, k, v, k_coarse=to_gpu(g["kc"], dtype), v_coarse=to_gpu(g["vc"], dtype))
            kc, vc = hsa.compress_kv_cache(k, v)
        assert out.shape == q.shape and out.dtype == q.dtype
        for got, want in ((out, g["out"]), (cached, g["out_cached"])):
            max_abs, mean_rel = attention_error(to_np(got), want)
            assert max_abs < (1e-3 if dtype == "fp32" else MAX_ABS), (name, max_abs)   # one bf16 ulp of the sparse branch
            assert mean_rel < (1e-5 if dtype == "fp32" else MEAN_REL), (name, mean_rel)
        np.testing.assert_allclose(to_np(kc), g["kc"], rtol=2 ** -7 if dtype == "bf16" else 1e-5, atol=1e-5)
        assert torch.allclose(out.float(), hsa(q, k, v, k_coarse=kc, v_coarse=vc).float(), atol=1e-5)


def test_output_is_the_gated_sum_of_the_two_branches(wa, golden):
    g = golden("hsa_fp32")
    q, k, v = (to_gpu(g[x]) for x in ("q", "k", "v"))
    for gate_bias in (-12.0, 0.0, 8.0):
        hsa = _module(wa, g, 3, 16, "fp32")
        with torch.no_grad():
            hsa.gate_lin.weight.zero_()
            hsa.gate_lin.bias.fill_(gate_bias)
            out = hsa(q, k, v)
        want, parts = O.hsa_attention(g["q"], g["k"], g["v"], k_proj_mat=g["ek"], v_proj_mat=g["ev"],
                                      gate_weight=np.zeros_like(g["gw"]), gate_bias=np.full_like(g["gb"], gate_bias),
                                      block_size=64, proj_segment_len=int(g["segment_len"]), return_parts=True)
        np.testing.assert_allclose(to_np(out), parts["sparse"] + parts["linear"] * parts["gate"], atol=2e-2)
        np.testing.assert_allclose(to_np(out), want, atol=1e-3)       # one bf16 ulp of the sparse branch


def _seeded_case(seed, q_len, kv_len, heads, d, dtype, scale=1.0):
    rng = np.random.default_rng(seed)
    def draw(n):
        x = (rng.standard_normal((1, n, heads, d)) * scale).astype(np.float32)
        return O.bf16_round(x) if dtype == "bf16" else x
    return draw(q_len), draw(kv_len), draw(kv_len)


def _block_average_proj(rank, seg, bs):
    e = np.zeros((rank, seg), np.float32)
    for r in range(rank):
        lo, hi = r * bs, min((r + 1) * bs, seg)
        if hi > lo:
            e[r, lo:hi] = 1.0 / (hi - lo)
    return O.bf16_round(e)


@pytest.mark.parametrize("dtype,bs,topk", [("fp32", 64, None), ("bf16", 64, [8, 3, 5, 1]), ("bf16", 128, None),
                                           ("fp32", 128, [2, 2, 7, 1])])
def test_forward_generic_path_against_oracle(wa, dtype, bs, topk):
    """Medium shapes through routing + both branches + gate, raw q/k/v in, ids and output out."""
    heads, d, q_len, kv_len, seg = 4, 64, 500, 1900, 390
    q, k, v = _seeded_case(11, q_len, kv_len, heads, d, dtype)
    rank = math.ceil(seg / bs)
    ek = _block_average_proj(rank, seg, bs)
    rng = np.random.default_rng(3)
    gw = (rng.standard_normal((d, d)) * 0.1).astype(np.float32)
    gb = (rng.standard_normal((d,)) * 0.3).astype(np.float32)
    lin = torch.nn.Linear(d, d).to(dev())
    with torch.no_grad():
        lin.weight.copy_(to_gpu(gw)); lin.bias.copy_(to_gpu(gb))
    tk = None if topk is None else torch.tensor(topk, dtype=torch.int32)
    out, (index, num, thr, used_tuned) = wa.hsa.hsa_attention(
        to_gpu(q, dtype), to_gpu(k, dtype), to_gpu(v, dtype), k_proj_mat=to_gpu(ek, "bf16"), v_proj_mat=to_gpu(ek, "bf16"),
        gate_lin=lin, block_size=bs, proj_segment_len=seg, topk_per_head=tk, return_routing=True, force_generic=True)
    want, parts = O.hsa_attention(q, k, v, k_proj_mat=ek, v_proj_mat=ek, gate_weight=gw, gate_bias=gb, block_size=bs,
                                  proj_segment_len=seg, dtype=dtype, topk_per_head=topk, return_parts=True)
    assert not used_tuned
    assert np.array_equal(to_np(num), parts["num"])
    assert np.array_equal(to_np(thr), parts["thresholds"])
    mismatch = float((to_np(index) != parts["index"]).mean())
    assert mismatch < 1e-3, f"routing order differs from the oracle on {mismatch:.2%} of slots"
    max_abs, mean_rel = attention_error(to_np(out), want)
    assert max_abs < MAX_ABS and mean_rel < MEAN_REL, (max_abs, mean_rel)


def test_config1_shape_fp32(wa):
    """Benchmark config 1: q = 1 frame (1560 tokens), KV = 3 frames, 12 heads x 128, block 64, top-8, seed 0."""
    heads, d, q_len, kv_len, bs, seg = 12, 128, 1560, 4680, 64, 1560
    q, k, v = _seeded_case(0, q_len, kv_len, heads, d, "fp32")
    ek = _block_average_proj(math.ceil(seg / bs), seg, bs)
    lin = torch.nn.Linear(d, d).to(dev())
    with torch.no_grad():
        lin.weight.zero_(); lin.bias.zero_()
    for topk in (None, [8] * heads):
        tk = None if topk is None else torch.tensor(topk, dtype=torch.int32)
        out, (index, num, thr, _) = wa.hsa.hsa_attention(
            to_gpu(q), to_gpu(k), to_gpu(v), k_proj_mat=to_gpu(ek, "bf16"), v_proj_mat=to_gpu(ek, "bf16"), gate_lin=lin,
            block_size=bs, proj_segment_len=seg, topk_per_head=tk, return_routing=True)
        want, parts = O.hsa_attention(q, k, v, k_proj_mat=ek, v_proj_mat=ek, gate_weight=np.zeros((d, d), np.float32),
                                      gate_bias=np.zeros((d,), np.float32), block_size=bs, proj_segment_len=seg,
                                      topk_per_head=topk, return_parts=True)
        assert np.array_equal(to_np(num), parts["num"])
        assert np.array_equal(to_np(index), parts["index"])
        max_abs, mean_rel = attention_error(to_np(out), want)
        assert max_abs < MAX_ABS and mean_rel < MEAN_REL, (max_abs, mean_rel)


# ---------------------------------------------------------------- API behaviour
def test_argument_errors(wa):
    hsa = wa.hsa.HSAAttention(2, 16, proj_segment_len=50).to(dev())
    wa.hsa_stage.init_hsa_parameters(hsa)
    q = torch.randn(1, 10, 2, 16, device=dev())
    k = torch.randn(1, 100, 2, 16, device=dev())
    with pytest.raises(ValueError):
        hsa(q, k, k, k_coarse=k)
    with pytest.raises(ValueError):
        hsa(q, k, k, k_coarse=torch.zeros(1, 4, 3, 16, device=dev()), v_coarse=torch.zeros(1, 4, 3, 16, device=dev()))
    with pytest.raises(ValueError):
        wa.hsa.hsa_attention(q, k[:, :0], k[:, :0], k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat)
    with pytest.raises(ValueError):
        hsa.compress_kv_cache(k, k[:, :50])
    with pytest.raises(RuntimeError):
        hsa(q.cpu(), k.cpu(), k.cpu())          # no CPU path: fails loudly
    out = wa.hsa.hsa_attention(q, k, k, k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat, gate_lin=None,
                               proj_segment_len=50)
    assert out.shape == q.shape and torch.isfinite(out).all()


def test_merge_partials_matches_single_pass(wa):
    torch.manual_seed(2)
    b, h, n, d, bs = 1, 2, 64, 32, 16
    q, k, v = (torch.randn(b, h, n, d, device=dev()) for _ in range(3))
    nb = n // bs
    sizes = torch.full((nb,), bs, dtype=torch.int32, device=dev())
    full_index = torch.arange(nb, dtype=torch.int32, device=dev()).view(1, 1, 1, nb).expand(b, h, nb, nb).contiguous()
    full_num = torch.full((b, h, nb), nb, dtype=torch.int32, device=dev())
    want = wa.hsa.block_sparse_attention_reference(q, k, v, full_index, full_num, sizes, bs)
    outs, lses = [], []
    for shard in ((0, 1), (2,), ()):                      # the empty shard contributes -inf
        idx = torch.zeros_like(full_index)
        idx[..., : len(shard)] = torch.tensor(shard, dtype=torch.int32, device=dev()) if shard else 0
        num = torch.full((b, h, nb), len(shard), dtype=torch.int32, device=dev())
        o, l = wa.hsa.block_sparse_attention_reference(q, k, v, idx, num, sizes, bs, return_lse=True)
        outs.append(o.reshape(-1, d)); lses.append(l.reshape(-1))
    shard3 = torch.full_like(full_index, 3)
    o, l = wa.hsa.block_sparse_attention_reference(q, k, v, shard3, torch.ones_like(full_num), sizes, bs, return_lse=True)
    outs.append(o.reshape(-1, d)); lses.append(l.reshape(-1))
    from worldattention_b200.sharded import merge_partials
    merged, lse = merge_partials(torch.stack(outs), torch.stack(lses))
    assert torch.allclose(merged.view_as(want), want, atol=1e-5)
    want_o, want_l = O.merge_partials([to_np(x) for x in outs], [to_np(x) for x in lses])
    np.testing.assert_allclose(to_np(merged), want_o, atol=1e-5)
    np.testing.assert_allclose(to_np(lse), want_l, atol=1e-5)
