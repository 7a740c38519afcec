"""Host-side logic that needs no GPU: shape helpers, parameter contract, tier manager, sharding plans."""
import math
import shutil
import tempfile

import numpy as np
import pytest
import torch

import worldattention_b200 as wa
from worldattention_b200 import sharded
from worldattention_b200.hsa.routing import block_counts, pad_to_len, variable_block_sizes


def test_block_helpers():
    assert block_counts(1560, 4680, 64) == (1600, 4736, 25, 74)
    assert block_counts(4680, 32760, 128) == (4736, 32768, 37, 256)
    sizes = variable_block_sizes(4680, 4736, 64, "cpu")
    assert sizes.dtype == torch.int32 and sizes[-1] == 8 and (sizes[:-1] == 64).all()
    x = torch.ones(1, 10, 2, 4)
    assert pad_to_len(x, 16).shape == (1, 16, 2, 4) and pad_to_len(x, 16)[:, 10:].abs().sum() == 0
    assert pad_to_len(x, 8) is x


def test_module_contract():
    hsa = wa.hsa.HSAAttention(num_heads=12, head_dim=128)
    assert hsa.proj_rank == 25 and hsa.k_proj_mat.shape == (25, 1560) and hsa.k_proj_mat.dtype == torch.bfloat16
    assert sorted(wa.hsa.hsa_parameter_names(hsa)) == ["gate_lin.bias", "gate_lin.weight", "k_proj_mat", "v_proj_mat"]
    assert all(torch.count_nonzero(p) == 0 for p in hsa.parameters())
    assert wa.hsa_stage.init_hsa_parameters(hsa) == 1
    row = hsa.k_proj_mat[0]
    assert int((row != 0).sum()) == 64 and abs(row[0].item() - 1 / 64) < 1e-3
    last = hsa.k_proj_mat[24]
    assert int((last != 0).sum()) == 1560 - 24 * 64
    hsa.reset_parameters()
    assert torch.count_nonzero(hsa.k_proj_mat) == 0
    assert hsa.coarse_cache_size(0) == 0 and hsa.coarse_cache_size(32760) == 21 * 25
    assert hsa.token_range_to_coarse(1560, 4680) == (25, 75)
    with pytest.raises(ValueError):
        hsa.token_range_to_coarse(0, 1561)
    with pytest.raises(ValueError):
        wa.hsa.HSAAttention(num_heads=1, head_dim=8, block_size=32)
    with pytest.raises(ValueError):
        wa.hsa.HSAAttention(num_heads=1, head_dim=8, proj_segment_len=0)
    assert wa.hsa.HSAAttention(num_heads=1, head_dim=8, block_size=128).proj_rank == 13
    wa.hsa.require_trained_hsa([], "ckpt.pt")
    wa.hsa.require_trained_hsa(["blocks.0.self_attn.q.weight"])
    with pytest.raises(RuntimeError, match="HSA training") as err:
        wa.hsa.require_trained_hsa(["blocks.0.self_attn.hsa_attention.k_proj_mat"], "ckpt.pt")
    assert "ckpt.pt" in str(err.value)
    assert wa.hsa.resolve_backend("torch") == "torch" and wa.hsa.resolve_backend("triton") == "triton"
    assert wa.hsa.resolve_backend("auto") in ("torch", "triton")
    with pytest.raises(ValueError):
        wa.hsa.resolve_backend("nope")


def test_cpu_tensors_are_rejected_loudly():
    hsa = wa.hsa.HSAAttention(num_heads=2, head_dim=16, proj_segment_len=50)
    q = torch.randn(1, 8, 2, 16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        hsa(q, q, q)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        wa.hsa.build_block_routing(torch.rand(1, 1, 2, 4), 0.35, 1.0)


def test_reference_import_paths_resolve():
    wa.install_reference_aliases()
    from wan.modules.hsa import HSAAttention                      # noqa: F401
    from wan.modules.hsa.attention import _linear_branch          # noqa: F401
    from wan.modules.hsa.routing import block_counts as bc        # noqa: F401
    from pipeline.hkv import HKVCache, HKVTierManager             # noqa: F401
    from pipeline.hkv.rope import temporal_band                   # noqa: F401
    from trainer.hsa_stage import init_hsa_parameters             # noqa: F401
    assert HSAAttention is wa.hsa.HSAAttention and HKVCache is wa.hkv.HKVCache


def _blob(tag):
    return {"k": [torch.full((1, 4, 1, 2), float(tag))], "v": [torch.full((1, 4, 1, 2), -float(tag))]}


def test_tier_manager_lru_spill_and_reload():
    tmp = tempfile.mkdtemp()
    try:
        tier = wa.hkv.HKVTierManager(cpu_max_chunks=2, nvme_enabled=True, nvme_dir=tmp)
        for c in range(3):
            tier.put(c, _blob(c))
        assert [tier.location(c) for c in range(3)] == ["nvme", "cpu", "cpu"]
        assert tier.stats()["n_spills"] == 1 and tier.stats()["backups"] == 1
        blob = tier.get(0)                                  # reload evicts the least recently used (1)
        assert blob["k"][0][0, 0, 0, 0] == 0.0 and tier.stats()["n_loads"] == 1
        assert [tier.location(c) for c in range(3)] == ["cpu", "nvme", "cpu"]
        tier.get(2); tier.put(3, _blob(3))                   # 0 is now the oldest -> re-spilled without rewriting
        assert tier.location(0) == "nvme" and tier.stats()["backups"] == 2 and tier.stats()["n_spills"] == 3
        assert tier.get(42) is None and tier.location(42) == "absent"
        tier.cleanup()
        assert tier.stats()["cpu_resident"] == 0 and tier.location(0) == "absent"
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    drop = wa.hkv.HKVTierManager(cpu_max_chunks=0)           # capacity floors at 1
    drop.put(0, _blob(0)); drop.put(1, _blob(1))
    assert drop.location(0) == "absent" and drop.stats()["n_drops"] == 1 and drop.get(0) is None
    with pytest.raises(ValueError):
        wa.hkv.HKVTierManager(cpu_max_chunks=1, nvme_enabled=True)


def test_temporal_band_sizes():
    assert wa.hkv.temporal_complex_dims(128) == 22
    assert wa.hkv.temporal_complex_dims(24) == 4
    assert wa.hkv.temporal_band(torch.zeros(1024, 64), 128).shape == (1024, 22)


def test_head_split_plans():
    assert sharded.plan_head_split(12, 2) == [list(range(6)), list(range(6, 12))]
    assert [len(x) for x in sharded.plan_head_split(12, 8)] == [2, 2, 2, 2, 1, 1, 1, 1]
    k = [8, 32, 4, 4, 32, 8, 32, 8, 32, 4, 4, 8]
    for world in (2, 4):
        plan = sharded.plan_head_split(12, world, k)
        assert sorted(h for p in plan for h in p) == list(range(12))
        assert all(len(p) == 12 // world for p in plan)
        loads = [sum(k[h] for h in p) for p in plan]
        assert max(loads) - min(loads) <= 8, loads
    with pytest.raises(ValueError):
        sharded.plan_head_split(4, 8)


def test_kv_shard_plans_cut_at_block_boundaries():
    for kv_len, bs, world, page in ((748_800, 64, 8, 1560), (32_760, 128, 8, 1560), (1000, 64, 4, 0), (100, 64, 8, 0),
                                    (120, 64, 8, 0), (120, 64, 8, 50), (160, 64, 8, 100), (4681, 128, 3, 1560)):
        shards = sharded.plan_kv_shards(kv_len, bs, world, page)
        assert len(shards) == world and shards[0][0] == 0 and shards[-1][1] == kv_len
        for (a, b), (c, d) in zip(shards, shards[1:]):
            # a cut is a block boundary, or the end of the cache when the ragged last block has been given away already
            assert b == c and a <= b <= kv_len and (b % bs == 0 or b == kv_len)
        assert sum(b - a for a, b in shards) == kv_len                     # a partition of [0, kv_len): no token twice
        assert sum(math.ceil((b - a) / bs) for a, b in shards) == math.ceil(kv_len / bs)
    # the ragged case that used to claim tokens past the end: 120 tokens, 64-token blocks, 8 ranks
    assert sharded.plan_kv_shards(120, 64, 8)[-2:] == [(64, 120), (120, 120)]


def test_local_selection_partitions_the_global_selection():
    torch.manual_seed(0)
    nkv = 37
    index = torch.stack([torch.randperm(nkv) for _ in range(6)]).view(1, 2, 3, nkv).int()
    num = torch.randint(0, nkv + 1, (1, 2, 3)).int()
    bounds = [0, 5, 5, 20, 37]
    seen = torch.zeros(1, 2, 3, nkv, dtype=torch.int32)
    for lo, hi in zip(bounds, bounds[1:]):
        li, ln = sharded.local_selection(index, num, lo, hi)
        for h in range(2):
            for i in range(3):
                ids = li[0, h, i, : int(ln[0, h, i])].tolist()
                assert ids == sorted(ids) and all(0 <= x < hi - lo for x in ids)
                seen[0, h, i, [x + lo for x in ids]] += 1
    want = torch.zeros_like(seen)
    for h in range(2):
        for i in range(3):
            want[0, h, i, index[0, h, i, : int(num[0, h, i])].long()] = 1
    assert torch.equal(seen, want)


def test_install_plan_matches_the_oracle_plan():
    """The array-form install plan of `HKVCache.apply` against the oracle's restatement of the reference loops:
    unknown chunks/pages and chunks no tier holds are skipped, the page that crosses the capacity is cut, frames
    count back from the current start frame."""
    import numpy as np
    from oracle import hkv_oracle as K
    rng = np.random.default_rng(5)
    frame_len, page_frames = 6, 2
    bank = wa.hkv.HKVCache(frame_seq_length=frame_len, page_size_frames=page_frames)
    valid = [40, 31, 24, 12]
    for c, n in enumerate(valid):
        bank.chunks.append({"chunk_id": c, "valid_tokens": n, "page_spans": K.page_spans(n, frame_len * page_frames),
                            "start_frame": 3 + 7 * c, "page_index": None, "heads": 1})

    class Tier:                      # chunk 2 has been dropped by every tier; nothing is on disk
        def get(self, chunk_id):
            return None if chunk_id == 2 else {"k": [], "v": []}

        def page_reader(self, chunk_id):
            return None
    bank.tier = Tier()
    for trial in range(60):
        pairs = [(int(rng.integers(-1, 5)), int(rng.integers(-1, 5))) for _ in range(int(rng.integers(0, 7)))]
        capacity = int(rng.integers(0, 70))
        current = int(rng.integers(20, 40))
        entries = [(c, *bank.chunks[c]["page_spans"][p]) for c, p in pairs
                   if 0 <= c < len(valid) and c != 2 and 0 <= p < len(bank.chunks[c]["page_spans"])]
        plan, blobs = bank._install_plan(pairs, capacity=capacity, current_start_frame=current)
        if not entries:
            assert plan is None and blobs == {}
            continue
        installed = K.plan_install(entries, capacity)
        moves = K.plan_rerope(installed, [ch["start_frame"] for ch in bank.chunks], frame_len, current)
        rows = [r for r in plan if int(r["count"]) > 0 or installed]
        assert int(plan["count"].sum()) == sum(e - s for _, s, e in installed)
        if not installed:
            continue
        assert [(int(r["chunk"]), int(r["src"]), int(r["src"] + r["count"])) for r in rows] == installed
        assert [(int(r["frame_from"]), int(r["frame_to"])) for r in rows] == moves
        assert [int(r["dst"]) for r in rows] == list(np.cumsum([0] + [e - s for _, s, e in installed])[:-1])


def test_chunk_loop_window_bookkeeping_on_the_host():
    """The chunk loop's cache plan (causal_model.py:331-343, 395-399) as properties: rows are written at the tail, the
    window never overflows, a chunk that runs again rewrites the same rows, and once the window is full every chunk
    evicts exactly one chunk; `reset(keep_buffers=True)` clears the caches without moving them."""
    from worldattention_b200.causal_dit import CausalDiT, ChunkPipeline, DiTConfig
    cfg = DiTConfig(dim=256, heads=2, ffn_dim=512, layers=2, latent_hw=(16, 32), text_dim=64, text_len=16, window_frames=7,
                    hsa_block=64, denoising_steps=(1000, 500))
    torch.manual_seed(0)
    pipe = ChunkPipeline(CausalDiT(cfg), device="cpu", dtype=torch.float32)
    s, size = cfg.frames_per_chunk * cfg.frame_tokens, cfg.window_frames * cfg.frame_tokens
    seen_roll = 0
    for chunk in range(6):
        frame = chunk * cfg.frames_per_chunk
        plan = pipe._plan(frame)
        assert 0 <= plan["write"] and plan["write"] + s <= size                 # the chunk's rows fit behind what is kept
        assert plan["local_end"] == plan["write"] + s and plan["local_end"] <= size
        assert plan["global_end"] == (frame + cfg.frames_per_chunk) * cfg.frame_tokens
        if plan["roll"]:
            seen_roll += 1
            assert plan["keep"] + plan["evict"] == pipe.local_end and plan["keep"] == plan["write"]
            assert plan["local_end"] == size                                    # a rolled window is exactly full
        else:
            assert plan["write"] == pipe.local_end                              # appended right behind the valid rows
        again = pipe._plan(frame)                                               # planning is pure
        assert again == plan
        pipe._commit(plan)
        # the later forwards of the same chunk (and its clean-context forward) see the committed state: same rows again
        repeat = pipe._plan(frame)
        assert not repeat["roll"] and repeat["write"] == plan["write"] and repeat["local_end"] == plan["local_end"]
        assert int(pipe.kv_cache[0]["local_end_index"]) == pipe.local_end
        assert int(pipe.kv_cache[1]["global_end_index"]) == pipe.global_end
    assert seen_roll == 4 and pipe.local_end == size      # 7-frame window, 3-frame chunks: two chunks fit, the third rolls
    addresses = [t.data_ptr() for c in pipe.kv_cache for t in c.values()]
    pipe.kv_cache[0]["k"].fill_(1.0)
    pipe.reset(keep_buffers=True)
    assert [t.data_ptr() for c in pipe.kv_cache for t in c.values()] == addresses
    assert pipe.local_end == 0 and pipe.global_end == 0 and not pipe.kv_cache[0]["k"].any()
    pipe.reset()
    assert pipe._plan(0)["write"] == 0


def test_peer_store_addressing_delivers_what_the_all_to_all_delivers():
    """The address rule of the peer-store exchange (`wa_hsa_params.peer_rows / peer_self / peer_delta`), restated on the
    host: storing query row t of rank s as row `s * rows + t % rows` of rank `t // rows`'s buffer fills every receive
    buffer exactly as `all_to_all_single` of the ranks' records does, ragged last slice included."""
    from worldattention_b200 import sharded
    rng = np.random.default_rng(5)
    for q_len, world in ((333, 3), (10, 4), (4680, 8), (5, 8)):
        rows, plan = sharded.exchange_rows(q_len, world)
        assert rows * world >= q_len and sum(c for _, c in plan) == q_len
        assert all(first == r * rows for r, (first, _) in enumerate(plan))
        sent = rng.integers(1, 1 << 30, size=(world, rows * world))            # one word per record; rows >= q_len are padding
        sent[:, q_len:] = 0
        # the collective: rank r's slice j lands in slot r of rank j
        want = np.stack([np.concatenate([sent[r, j * rows:(j + 1) * rows] for r in range(world)]) for j in range(world)])
        got = np.zeros_like(want)
        for s in range(world):
            for t in range(q_len):
                got[min(t // rows, 7), s * rows + t % rows] = sent[s, t]
        assert np.array_equal(got, want)


def test_sharded_forward_rejects_unknown_options_before_touching_tensors():
    hsa = wa.hsa.HSAAttention(2, 128, block_size=64, proj_segment_len=128)
    q = torch.zeros(1, 64, 2, 128)
    for bad in (dict(exchange="ring"), dict(routing="everything"), dict(routing="candidates")):   # the last: no fixed top-k given
        with pytest.raises(ValueError):
            sharded.hsa_attention_kv_sharded(hsa, q, q, q, q, q, kv_len=64, shards=[(0, 64)], **bad)
