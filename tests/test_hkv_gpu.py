"""GPU parity of the HKV kernels and cache logic against the numpy oracle and reference vectors.

Page ids are bit-exact; re-rotated keys and centroids meet the reference's own tolerances
(1e-4 fp32, one bf16 ulp for bf16 tensors).
"""
import shutil
import tempfile

import numpy as np
import pytest
import torch

from oracle import hkv_oracle as K
from tests.helpers import dev, to_gpu, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def wa():
    import worldattention_b200 as pkg
    return pkg


def test_temporal_rope_shift_and_derope(wa, golden):
    g = golden("hkv_rope")
    freqs = torch.from_numpy(g["freqs"])
    keys = to_gpu(g["keys"])
    shifted = wa.hkv.shift_temporal_rope(keys, freqs, 9, 3)
    assert np.array_equal(to_np(shifted), K.shift_temporal_rope(g["keys"], g["freqs"], 9, 3))
    np.testing.assert_allclose(to_np(shifted), g["shifted"], atol=1e-6)
    back = wa.hkv.shift_temporal_rope(shifted, freqs, 3, 9)
    np.testing.assert_allclose(to_np(back), g["keys"], atol=1e-5)                 # invertible
    nt = wa.hkv.temporal_complex_dims(24)
    assert torch.equal(shifted[..., 2 * nt:], keys[..., 2 * nt:])                # spatial bands untouched
    deroped = wa.hkv.derope_temporal(keys, freqs, torch.from_numpy(g["frame_ids"]))
    assert np.array_equal(to_np(deroped), K.derope_temporal(g["keys"], g["freqs"], g["frame_ids"]))
    np.testing.assert_allclose(to_np(deroped), g["deroped"], atol=1e-6)
    got16 = wa.hkv.shift_temporal_rope(to_gpu(g["keys16"], "bf16"), freqs, 200, 3)   # clamps to the table
    assert np.array_equal(to_np(got16), K.shift_temporal_rope(g["keys16"], g["freqs"], 200, 3, dtype="bf16"))
    np.testing.assert_allclose(to_np(got16), g["shifted16"], rtol=2 ** -7, atol=1e-6)


def test_page_index_and_scores(wa, golden):
    g = golden("hkv_rope")
    freqs = torch.from_numpy(g["freqs"])
    spans = [tuple(int(x) for x in s) for s in g["spans"]]
    for key, dtype, tol in (("keys", "fp32", 1e-6), ("keys16", "bf16", 2e-3)):
        pidx = wa.hkv.page_key_index(to_gpu(g[key], dtype), spans, frame_seq_length=4, start_frame=5, temporal_freqs=freqs)
        want = K.page_key_index(g[key], spans, frame_seq_length=4, start_frame=5, temporal_freqs=g["freqs"], dtype=dtype)
        assert np.array_equal(to_np(pidx), want)
        np.testing.assert_allclose(to_np(pidx), g["page_index" if dtype == "fp32" else "page_index16"], atol=tol)
    assert wa.hkv.page_key_index(to_gpu(g["keys"]), [], frame_seq_length=4, start_frame=0, temporal_freqs=freqs) is None
    scores = wa.hkv.score_pages(to_gpu(g["qvec"]), to_gpu(g["page_index"]))
    assert np.array_equal(to_np(scores), K.score_pages(g["qvec"], g["page_index"]))
    np.testing.assert_allclose(to_np(scores), g["scores"], atol=1e-6)
    assert wa.hkv.score_pages(to_gpu(g["qvec"]), torch.zeros(0, 48, device=dev())).numel() == 0


def test_two_stage_selection(wa, golden):
    g = golden("hkv_retrieval")
    np.testing.assert_allclose(to_np(wa.hkv.prompt_index(to_gpu(g["prompt"]))), g["prompt_index"], atol=1e-6)
    assert wa.hkv.select_top_chunks(to_gpu(g["prompt_index"]), to_gpu(g["bank"]), 2) == [int(x) for x in g["top_chunks"]]
    cands = [(int(c), int(p), to_gpu(vec)) for (c, p), vec in zip(g["cand_ids"], g["cand_vecs"])]
    sel = wa.hkv.select_topk_pages(to_gpu(g["qvec"]), cands, 5)
    assert [(c, p) for c, p, _ in sel] == [tuple(int(x) for x in row) for row in g["sel_ids"]]
    np.testing.assert_allclose([s for _, _, s in sel], g["sel_scores"], atol=1e-6)
    assert wa.hkv.select_topk_pages(to_gpu(g["qvec"]), cands, 0) == []
    assert wa.hkv.select_top_chunks(to_gpu(g["prompt_index"]), torch.zeros(0, 8, device=dev()), 2) == []
    assert len(wa.hkv.select_topk_pages(to_gpu(g["qvec"]), cands[:3], 5)) == 3        # fewer pages than the budget


def test_topk_ties_prefer_lower_page_id_and_per_head_mode(wa):
    from worldattention_b200.hkv.retrieval import score_and_topk
    rng = np.random.default_rng(0)
    pages, heads, d = 480, 12, 128
    index = rng.standard_normal((pages, heads * d)).astype(np.float32)
    index[17] = index[400]                      # identical pages -> identical scores
    index[3] = index[400]
    q = rng.standard_normal((heads * d,)).astype(np.float32)
    scores, ids, vals = score_and_topk(to_gpu(q), to_gpu(index), pages)
    want_scores = K.score_pages(q, index)
    assert np.array_equal(to_np(scores)[0], want_scores)
    want_ids, want_vals = K.topk_lower_index_first(want_scores, pages)
    assert np.array_equal(to_np(ids)[0], want_ids)
    pos = {int(p): i for i, p in enumerate(to_np(ids)[0])}
    assert pos[3] < pos[17] < pos[400]
    # per-head scoring and selection: [H, P] scores, top-16 per head
    scores_h, ids_h, vals_h = score_and_topk(to_gpu(q), to_gpu(index), 16, groups=heads)
    for h in range(heads):
        want = K.score_pages(q[h * d:(h + 1) * d], index[:, h * d:(h + 1) * d])
        assert np.array_equal(to_np(scores_h)[h], want)
        wi, wv = K.topk_lower_index_first(want, 16)
        assert np.array_equal(to_np(ids_h)[h], wi)
        assert np.array_equal(to_np(vals_h)[h], wv)


def _cache(g, dtype, fill=0.0):
    ft, pf, cap, layers, heads, hd, cur = (int(x) for x in g["dims"])
    return [dict(k=torch.full((1, cap, heads, hd), fill, dtype=dtype, device=dev()),
                 v=torch.full((1, cap, heads, hd), fill, dtype=dtype, device=dev()),
                 k_coarse=torch.full((1, 5, heads, hd), -9.0, dtype=dtype, device=dev()),
                 v_coarse=torch.full((1, 5, heads, hd), -9.0, dtype=dtype, device=dev()),
                 global_end_index=torch.zeros([], dtype=torch.long, device=dev()),
                 local_end_index=torch.zeros([], dtype=torch.long, device=dev())) for _ in range(layers)]


def _hsa_modules(wa, g):
    ft, pf, cap, layers, heads, hd, cur = (int(x) for x in g["dims"])
    mods = []
    for layer in range(layers):
        m = wa.hsa.HSAAttention(num_heads=heads, head_dim=hd, block_size=64, proj_segment_len=ft).to(dev())
        with torch.no_grad():
            m.k_proj_mat.copy_(to_gpu(g["ek"][layer], "bf16"))
            m.v_proj_mat.copy_(to_gpu(g["ev"][layer], "bf16"))
        mods.append(m)
    return mods


@pytest.mark.parametrize("name,dtype,tier", [("hkv_cache_fp32", "fp32", "cpu"), ("hkv_cache_bf16", "bf16", "cpu"),
                                             ("hkv_cache_bf16", "bf16", "hbm"), ("hkv_cache_fp32", "fp32", "nvme")])
def test_store_retrieve_apply_matches_reference(wa, golden, name, dtype, tier):
    g = golden(name)
    ft, pf, cap, layers, heads, hd, cur = (int(x) for x in g["dims"])
    tdtype = torch.bfloat16 if dtype == "bf16" else torch.float32
    freqs = torch.from_numpy(g["freqs"])
    nvme_dir = tempfile.mkdtemp() if tier == "nvme" else None
    try:
        bank = wa.hkv.HKVCache(frame_seq_length=ft, page_size_frames=pf, topk_pages=3, stage1_topk_chunks=2,
                               cpu_max_chunks=1 if tier == "nvme" else 8, nvme_enabled=tier == "nvme", nvme_dir=nvme_dir,
                               hbm_max_chunks=8 if tier == "hbm" else 0)
        for c in range(3):
            cache = _cache(g, tdtype)
            valid = int(g["valid"][c])
            for layer, blk in enumerate(cache):
                blk["k"][:, :valid] = to_gpu(g[f"c{c}_l{layer}_k"], dtype)
                blk["v"][:, :valid] = to_gpu(g[f"c{c}_l{layer}_v"], dtype)
                blk["local_end_index"].fill_(valid)
            cid = bank.store(cache, prompt_embeds=to_gpu(g["prompts"][c]), current_start_frame=int(g["starts"][c]),
                             temporal_freqs=freqs)
            assert cid == c
            assert bank.chunks[c]["start_frame"] == int(g[f"c{c}_start_frame"])
            np.testing.assert_allclose(to_np(bank.chunks[c]["page_index"]), g[f"c{c}_page_index"],
                                       atol=1e-6 if dtype == "fp32" else 2e-3)
        assert len(bank) == 3
        expect = {"cpu": "cpu", "hbm": "hbm", "nvme": "nvme"}[tier]
        assert bank.tier.location(0) == expect
        empty = _cache(g, tdtype)
        assert bank.store(empty, prompt_embeds=to_gpu(g["prompts"][0]), current_start_frame=0, temporal_freqs=freqs) == -1

        pairs = [tuple(int(x) for x in row) for row in g["pairs"]]
        target = _cache(g, tdtype, fill=7.0)
        with pytest.raises(ValueError):
            bank.apply(target, pairs, current_start_frame=cur, temporal_freqs=freqs)      # coarse tier needs modules
        mods = _hsa_modules(wa, g)
        junk = [(99, 0), (0, 99)]
        assert bank.apply(target, junk, current_start_frame=cur, temporal_freqs=freqs, hsa_modules=mods) == 0
        assert float(target[0]["k"][0, 0, 0, 0]) == 7.0                                   # untouched
        installed = bank.apply(target, junk + pairs, current_start_frame=cur, temporal_freqs=freqs, hsa_modules=mods)
        assert installed == int(g["installed"])
        for layer, blk in enumerate(target):
            np.testing.assert_allclose(to_np(blk["k"]), g[f"out_l{layer}_k"], rtol=2 ** -7 if dtype == "bf16" else 0, atol=2e-6)
            assert np.array_equal(to_np(blk["v"]), g[f"out_l{layer}_v"])
            np.testing.assert_allclose(to_np(blk["k_coarse"]), g[f"out_l{layer}_kc"], rtol=2 ** -6, atol=1e-5)
            np.testing.assert_allclose(to_np(blk["v_coarse"]), g[f"out_l{layer}_vc"], rtol=2 ** -6, atol=1e-5)
            assert (int(blk["global_end_index"]), int(blk["local_end_index"])) == tuple(int(x) for x in g[f"out_l{layer}_ends"])
        if tier == "nvme":
            assert bank.tier.stats()["n_loads"] >= 1
    finally:
        if nvme_dir:
            shutil.rmtree(nvme_dir, ignore_errors=True)


def test_retrieve_is_chronological_and_validates_query(wa, golden):
    g = golden("hkv_cache_fp32")
    ft, pf, cap, layers, heads, hd, cur = (int(x) for x in g["dims"])
    freqs = torch.from_numpy(g["freqs"])
    bank = wa.hkv.HKVCache(frame_seq_length=ft, page_size_frames=pf, topk_pages=3, stage1_topk_chunks=3)
    assert bank.retrieve(prompt_embeds=to_gpu(g["prompts"][0]), query_vec=to_gpu(g["qvec"])) == []
    for c in range(3):
        cache = _cache(g, torch.float32)
        valid = int(g["valid"][c])
        for layer, blk in enumerate(cache):
            blk["k"][:, :valid] = to_gpu(g[f"c{c}_l{layer}_k"])
            blk["v"][:, :valid] = to_gpu(g[f"c{c}_l{layer}_v"])
            blk["local_end_index"].fill_(valid)
        bank.store(cache, prompt_embeds=to_gpu(g["prompts"][c]), current_start_frame=int(g["starts"][c]), temporal_freqs=freqs)
    got = bank.retrieve(prompt_embeds=to_gpu(g["prompts"][1]), query_vec=to_gpu(g["qvec"]))
    keys = [(bank.chunks[c]["start_frame"], bank.chunks[c]["page_spans"][p][0]) for c, p in got]
    assert keys == sorted(keys) and len(got) == 3
    # oracle replay of the same two-stage selection
    pool = [(c, p, g[f"c{c}_page_index"][p]) for c in K.select_top_chunks(K.prompt_index(g["prompts"][1]), g["prompt_bank"], 3)
            for p in range(g[f"c{c}_page_index"].shape[0])]
    want = sorted([(c, p) for c, p, _ in K.select_topk_pages(g["qvec"], pool, 3)],
                  key=lambda cp: (int(g[f"c{cp[0]}_start_frame"]), cp[1] * ft * pf))
    assert got == want
    with pytest.raises(ValueError):
        bank.retrieve(prompt_embeds=to_gpu(g["prompts"][1]), query_vec=to_gpu(g["qvec"][:-1]))
    per_head = bank.retrieve(prompt_embeds=to_gpu(g["prompts"][1]), query_vec=to_gpu(g["qvec"]), per_head=True)
    assert len(per_head) == heads and all(len(x) == 3 for x in per_head)


def test_apply_truncates_to_capacity_and_skips_rerope_when_disabled(wa, golden):
    g = golden("hkv_cache_fp32")
    ft, pf, cap, layers, heads, hd, cur = (int(x) for x in g["dims"])
    freqs = torch.from_numpy(g["freqs"])
    bank = wa.hkv.HKVCache(frame_seq_length=ft, page_size_frames=pf, topk_pages=8, rerope=False)
    cache = _cache(g, torch.float32)
    for blk in cache:
        blk.pop("k_coarse"); blk.pop("v_coarse")
        blk["k"][:, :20] = to_gpu(g["c1_l0_k"])
        blk["v"][:, :20] = to_gpu(g["c1_l0_v"])
        blk["local_end_index"].fill_(20)
    bank.store(cache, prompt_embeds=to_gpu(g["prompts"][0]), current_start_frame=9, temporal_freqs=freqs)
    small = [dict(k=torch.ones(1, 12, heads, hd, device=dev()), v=torch.ones(1, 12, heads, hd, device=dev()),
                  global_end_index=torch.zeros([], dtype=torch.long, device=dev()),
                  local_end_index=torch.zeros([], dtype=torch.long, device=dev())) for _ in range(layers)]
    n = bank.apply(small, [(0, 0), (0, 2)], current_start_frame=40, temporal_freqs=freqs)
    assert n == 12                                       # second page only partly fits (8 + 4 of 4)
    want = np.concatenate([g["c1_l0_k"][:, 0:8], g["c1_l0_k"][:, 16:20]], axis=1)
    assert np.array_equal(to_np(small[0]["k"]), want)    # verbatim: re-rotation disabled
    assert int(small[0]["local_end_index"]) == 12 and int(small[0]["global_end_index"]) == 40 * ft


def test_device_resident_retrieval_matches_the_host_formulation(wa):
    """Scoring of all layers in one launch and copy records built on the device give the same installed cache as
    the per-layer scoring + host-built records."""
    from worldattention_b200.hkv.install import (build_records_device, gather_pages, gather_records_device,
                                                  per_head_records)
    from worldattention_b200.hkv.retrieval import score_and_topk, score_and_topk_layers
    layers, heads, d, pages, hot, tok, topk = 3, 4, 16, 20, 6, 5, 4
    g = torch.Generator().manual_seed(7)
    row = heads * d
    centroids = torch.randn((layers, pages, row), generator=g).to(dev())
    query = torch.randn((row,), generator=g).to(dev())
    pool = torch.randn((2, layers, hot, tok, heads, d), generator=g).to(dev()).bfloat16()
    nt = 3
    rot = torch.randn((topk, nt, 2), generator=g)
    rot = (rot / rot.norm(dim=-1, keepdim=True)).to(dev()).contiguous()
    # host formulation
    ids = torch.stack([score_and_topk(query, centroids[l], topk, groups=heads)[1] for l in range(layers)])
    scores_l, ids_l, vals_l = score_and_topk_layers(query, centroids, topk, groups=heads)
    assert torch.equal(ids, ids_l)
    chron = np.sort(ids.cpu().numpy(), axis=-1)
    slots = chron % hot
    esz = 2
    common = dict(src_page_stride=tok * row * esz, src_layer_stride=hot * tok * row * esz, dst_layer_stride=topk * tok * row * esz,
                  page_tokens=tok, heads=heads, head_dim=d, elem_size=esz)
    want = torch.zeros((2, layers, topk * tok, heads, d), dtype=torch.bfloat16, device=dev())
    rot_ids = np.broadcast_to(np.arange(topk, dtype=np.int32), slots.shape)
    rec = np.concatenate([
        per_head_records(slots, src_base=pool[0].data_ptr(), dst_base=want[0].data_ptr(), rot=rot_ids, **common),
        per_head_records(slots, src_base=pool[1].data_ptr(), dst_base=want[1].data_ptr(), rot=None, **common)])
    gather_pages(rec, max_tokens=tok, row_elems=d, head_dim=d, dtype=torch.bfloat16, device=dev(), rotations=rot, n_temporal=nt)
    # device formulation; page 3 is declared absent in a second run
    got = torch.zeros_like(want)
    slot_of = torch.arange(pages, dtype=torch.int64, device=dev()) % hot
    page_stride = tok * row * esz
    lc = dict(src_layer_stride=hot * page_stride, src_token_stride=row, dst_layer_stride=topk * page_stride, dst_token_stride=row,
              page_tokens=tok, head_dim=d)
    rk = build_records_device(ids_l, pool[0].data_ptr() + slot_of * page_stride, dst=got[0], rotate=True, **lc)
    rv = build_records_device(ids_l, pool[1].data_ptr() + slot_of * page_stride, dst=got[1], rotate=False, **lc)
    gather_records_device(torch.cat([rk, rv]), max_tokens=tok, row_elems=d, head_dim=d, dtype=torch.bfloat16, rotations=rot,
                          n_temporal=nt)
    assert torch.equal(got, want)
    missing = torch.zeros((1,), dtype=torch.int32, device=dev())
    src = pool[1].data_ptr() + slot_of * page_stride
    absent_id = int(ids_l[0, 0, 0])
    src[absent_id] = 0
    build_records_device(ids_l, src, dst=got[1], rotate=False, missing=missing, **lc)
    assert int(missing.item()) == int((ids_l == absent_id).sum().item())
