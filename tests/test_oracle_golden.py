"""Pin the numpy oracle against vectors produced by the reference's own PyTorch functions."""
import numpy as np

from oracle import hkv_oracle as hkv
from oracle import hsa_oracle as hsa


def _tie_aware_index_equal(probs, got_index, want_index):
    """Indices must agree wherever the probability is unique in its row; tied runs may permute."""
    got_p = np.take_along_axis(probs, got_index.astype(np.int64), axis=-1)
    want_p = np.take_along_axis(probs, want_index.astype(np.int64), axis=-1)
    assert np.array_equal(got_p, want_p), "sorted probability sequences differ"
    differs = got_index != want_index
    if differs.any():
        left = np.concatenate([got_p[..., :1] * 0 - 1, got_p[..., :-1]], axis=-1)
        right = np.concatenate([got_p[..., 1:], got_p[..., -1:] * 0 - 1], axis=-1)
        tied = (got_p == left) | (got_p == right)
        assert tied[differs].all(), "index differs outside a run of equal probabilities"


def test_routing_matches_reference(golden):
    for name in ("routing_small", "routing_wide"):
        g = golden(name)
        index, num, mask, thr = hsa.build_block_routing(g["block_attn"], float(g["tau"][0]),
                                                        float(g["tau"][1]), return_mask=True)
        np.testing.assert_allclose(thr, g["thresholds"], atol=1e-6)
        assert np.array_equal(num, g["num"]), name
        _tie_aware_index_equal(g["block_attn"], index, g["index"])
        assert np.array_equal(mask.sum(-1), g["mask"].sum(-1))


def test_pooling_matches_reference(golden):
    for name in ("pool_ragged_fp32", "pool_aligned_fp32", "pool_ragged_bf16", "pool_aligned_bf16"):
        g = golden(name)
        bs, length = int(g["block_size"]), int(g["length"])
        dtype = "bf16" if name.endswith("bf16") else "fp32"
        pooled = hsa.block_mean_pool(g["x"], length, g["x"].shape[2] // bs, bs, dtype)
        # fp32 sums differ from torch's blocked order by an ulp; bf16 results are rounded and agree.
        np.testing.assert_allclose(pooled, g["pooled"], rtol=0, atol=2e-6 if dtype == "fp32" else 0)


def test_block_map_matches_reference(golden):
    g = golden("block_map")
    np.testing.assert_allclose(hsa.block_attention_map(g["q_pooled"], g["k_pooled"]), g["block_attn"],
                               rtol=2e-6, atol=1e-8)


def test_sparse_branch_matches_reference(golden):
    g = golden("sparse_ref")
    got = hsa.block_sparse_attention(g["q"], g["k"], g["v"], g["index"], g["num"], g["sizes"],
                                     int(g["block_size"]), dtype="bf16")
    # one bf16 ulp where the fp32 results straddle a rounding boundary
    np.testing.assert_allclose(got, g["out"], rtol=2 ** -7, atol=1e-6)
    assert np.count_nonzero(got[0, 1, :16]) == 0          # num == 0 row block is exactly zero


def test_compress_and_linear_match_reference(golden):
    for name, dtype, tol in (("compress_linear_fp32", "fp32", 2e-6), ("compress_linear_bf16", "bf16", 2 ** -7)):
        g = golden(name)
        kc, vc = hsa.compress_kv(g["k"], g["v"], segment_len=int(g["segment_len"]), k_proj_mat=g["ek"],
                                 v_proj_mat=g["ev"], block_size=int(g["block_size"]), dtype=dtype)
        assert kc.shape == g["kc"].shape
        np.testing.assert_allclose(kc, g["kc"], rtol=tol, atol=1e-5)
        np.testing.assert_allclose(vc, g["vc"], rtol=tol, atol=1e-5)
        lin = hsa.linear_branch(g["q"], g["kc"], g["vc"], dtype=dtype)
        np.testing.assert_allclose(lin, g["linear"], rtol=2 * tol, atol=1e-5 if dtype == "fp32" else 4e-3)


def test_hsa_forward_matches_reference(golden):
    for name, dtype in (("hsa_fp32", "fp32"), ("hsa_bf16", "bf16")):
        g = golden(name)
        kwargs = dict(k_proj_mat=g["ek"], v_proj_mat=g["ev"], gate_weight=g["gw"], gate_bias=g["gb"],
                      block_size=int(g["block_size"]), tau_min=float(g["tau"][0]), tau_max=float(g["tau"][1]),
                      proj_segment_len=int(g["segment_len"]), dtype=dtype)
        out = hsa.hsa_attention(g["q"], g["k"], g["v"], **kwargs)
        cached = hsa.hsa_attention(g["q"], g["k"], g["v"], k_coarse=g["kc"], v_coarse=g["vc"], **kwargs)
        atol = 1e-4 if dtype == "fp32" else 2e-2
        assert np.max(np.abs(out - g["out"])) < atol, name
        assert np.max(np.abs(cached - g["out_cached"])) < atol, name
        rel = np.mean(np.abs(out - g["out"])) / np.mean(np.abs(g["out"]))
        assert rel < 1e-2


def test_hkv_rope_and_index_match_reference(golden):
    g = golden("hkv_rope")
    freqs = g["freqs"]
    np.testing.assert_allclose(hkv.shift_temporal_rope(g["keys"], freqs, 9, 3), g["shifted"], atol=1e-6)
    np.testing.assert_allclose(hkv.derope_temporal(g["keys"], freqs, g["frame_ids"]), g["deroped"], atol=1e-6)
    spans = [tuple(int(x) for x in s) for s in g["spans"]]
    pidx = hkv.page_key_index(g["keys"], spans, frame_seq_length=4, start_frame=5, temporal_freqs=freqs)
    np.testing.assert_allclose(pidx, g["page_index"], atol=1e-6)
    pidx16 = hkv.page_key_index(g["keys16"], spans, frame_seq_length=4, start_frame=5,
                                temporal_freqs=freqs, dtype="bf16")
    np.testing.assert_allclose(pidx16, g["page_index16"], atol=2e-3)
    got16 = hkv.shift_temporal_rope(g["keys16"], freqs, 200, 3, dtype="bf16")
    np.testing.assert_allclose(got16, g["shifted16"], rtol=2 ** -7, atol=1e-6)
    np.testing.assert_allclose(hkv.score_pages(g["qvec"], g["page_index"]), g["scores"], atol=1e-6)


def test_hkv_retrieval_matches_reference(golden):
    g = golden("hkv_retrieval")
    np.testing.assert_allclose(hkv.prompt_index(g["prompt"]), g["prompt_index"], atol=1e-6)
    assert hkv.select_top_chunks(g["prompt_index"], g["bank"], 2) == [int(x) for x in g["top_chunks"]]
    cands = [(int(c), int(p), vec) for (c, p), vec in zip(g["cand_ids"], g["cand_vecs"])]
    sel = hkv.select_topk_pages(g["qvec"], cands, 5)
    assert [(c, p) for c, p, _ in sel] == [tuple(int(x) for x in row) for row in g["sel_ids"]]
    np.testing.assert_allclose([s for _, _, s in sel], g["sel_scores"], atol=1e-6)


def _replay_hkv(g, dtype):
    """Re-run store -> retrieve -> apply with oracle functions on the recorded chunk contents."""
    ft, pf, cap, layers, heads, hd, cur = (int(x) for x in g["dims"])
    freqs = g["freqs"]
    page_tokens = ft * pf
    n_chunks = len(g["valid"])
    spans = [hkv.page_spans(int(g["valid"][c]), page_tokens) for c in range(n_chunks)]
    start_frames = [int(g["starts"][c]) - int(g["valid"][c]) // ft for c in range(n_chunks)]
    for c in range(n_chunks):
        assert start_frames[c] == int(g[f"c{c}_start_frame"])
        pidx = hkv.page_key_index(g[f"c{c}_l0_k"], spans[c], frame_seq_length=ft,
                                  start_frame=start_frames[c], temporal_freqs=freqs, dtype=dtype)
        np.testing.assert_allclose(pidx, g[f"c{c}_page_index"], atol=1e-6 if dtype == "fp32" else 2e-3)
    pairs = [tuple(int(x) for x in row) for row in g["pairs"]]
    entries = [(c, *spans[c][p]) for c, p in pairs]
    installed = hkv.plan_install(entries, cap)
    moves = hkv.plan_rerope(installed, start_frames, ft, cur)
    return layers, cap, installed, moves, freqs, n_chunks


def test_hkv_install_matches_reference(golden):
    for name, dtype in (("hkv_cache_fp32", "fp32"), ("hkv_cache_bf16", "bf16")):
        g = golden(name)
        layers, cap, installed, moves, freqs, n_chunks = _replay_hkv(g, dtype)
        total = sum(e - s for _, s, e in installed)
        assert total == int(g["installed"])
        for layer in range(layers):
            ck = {c: g[f"c{c}_l{layer}_k"] for c in range(n_chunks)}
            cv = {c: g[f"c{c}_l{layer}_v"] for c in range(n_chunks)}
            out_k, out_v, n = hkv.install_pages(cap, ck, cv, installed, moves, freqs, dtype)
            assert n == total
            np.testing.assert_allclose(out_k, g[f"out_l{layer}_k"], rtol=2 ** -7 if dtype == "bf16" else 0, atol=2e-6)
            assert np.array_equal(out_v, g[f"out_l{layer}_v"])
            assert tuple(g[f"out_l{layer}_ends"]) == (int(g["dims"][6]) * int(g["dims"][0]), total)
            # compressed tier rebuilt from the installed pages with this layer's projection
            seg = int(g["dims"][0])
            kc, vc = hsa.compress_kv(out_k[:, :total].transpose(0, 2, 1, 3), out_v[:, :total].transpose(0, 2, 1, 3),
                                     segment_len=seg, k_proj_mat=g["ek"][layer], v_proj_mat=g["ev"][layer],
                                     block_size=64, dtype=dtype)
            slots = kc.shape[2]
            np.testing.assert_allclose(kc.transpose(0, 2, 1, 3), g[f"out_l{layer}_kc"][:, :slots],
                                       rtol=2 ** -6 if dtype == "bf16" else 1e-5, atol=1e-5)
            np.testing.assert_allclose(vc.transpose(0, 2, 1, 3), g[f"out_l{layer}_vc"][:, :slots],
                                       rtol=2 ** -6 if dtype == "bf16" else 1e-5, atol=1e-5)
            assert np.count_nonzero(g[f"out_l{layer}_kc"][:, slots:]) == 0


def test_qk_norm_and_causal_rope_match_reference(golden):
    from oracle import rope_oracle as R
    g = golden("qk_norm_rope")
    grid, start = tuple(int(v) for v in g["grid"]), int(g["start_frame"])
    for tag, tol in (("fp32", 2e-6), ("bf16", 0.0)):
        normed = R.rms_norm(g[f"x_{tag}"], g[f"weight_{tag}"], float(g["eps"]), tag)
        if tag == "bf16":      # torch's float32 mean has its own summation order: a value may land one bf16 step away
            assert np.mean(normed != g[f"normed_{tag}"]) < 2e-3
            np.testing.assert_allclose(normed, g[f"normed_{tag}"], rtol=2 ** -7, atol=0)
        else:
            np.testing.assert_allclose(normed, g[f"normed_{tag}"], rtol=tol, atol=tol)
        heads = 2
        rope_only = R.causal_rope_apply(g[f"x_{tag}"].reshape(1, -1, heads, 128), grid, g["freqs"], start, tag)
        np.testing.assert_allclose(rope_only, g[f"rope_only_{tag}"], rtol=0, atol=tol)       # float64 product: exact after the store
        roped = R.causal_rope_apply(g[f"normed_{tag}"].reshape(1, -1, heads, 128), grid, g["freqs"], start, tag)
        np.testing.assert_allclose(roped, g[f"roped_{tag}"], rtol=0, atol=tol)
