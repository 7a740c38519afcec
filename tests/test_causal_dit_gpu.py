"""The end-to-end chunk loop around the HSA layer: cache bookkeeping, tier consistency, prompt switches through the bank."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _small(**kw):
    from worldattention_b200.causal_dit import DiTConfig
    base = dict(dim=256, heads=2, ffn_dim=512, layers=2, latent_hw=(16, 32), text_dim=64, text_len=16, window_frames=6,
                hsa_block=64, denoising_steps=(1000, 500))
    base.update(kw)
    return DiTConfig(**base)


def _build(cfg, hkv=None):
    from worldattention_b200.causal_dit import CausalDiT, ChunkPipeline
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    model = CausalDiT(cfg).to(dev, torch.bfloat16).eval()
    model.init_hsa(0)
    return model, ChunkPipeline(model, hkv=hkv, device=dev)


def test_rolling_cache_keeps_both_tiers_consistent():
    cfg = _small()
    assert cfg.frame_tokens == 128
    model, pipe = _build(cfg)
    frames = 12                                   # 4 chunks: the 6-frame window fills after 2 and rolls twice
    noise = torch.randn((1, frames, 16, 16, 32), device="cuda:0", dtype=torch.bfloat16)
    prompts = [torch.randn(16, 64)]
    out = pipe.generate(noise, prompts)
    assert out.shape == noise.shape and torch.isfinite(out.float()).all()
    assert pipe.local_end == 6 * 128 and pipe.global_end == 12 * 128
    assert pipe.stats.forwards == 4 * 3
    for blk, cache in zip(model.blocks, pipe.kv_cache):
        hsa = blk.self_attn.hsa_attention
        kc, vc = hsa.compress_kv_cache(cache["k"], cache["v"])      # the compressed tier rebuilt from the token tier
        assert torch.equal(kc, cache["k_coarse"]) and torch.equal(vc, cache["v_coarse"])
        assert int(cache["local_end_index"]) == 6 * 128
        assert torch.count_nonzero(cache["k"]) > 0.9 * cache["k"].numel()


def test_last_chunk_of_the_window_is_the_last_append():
    cfg = _small(layers=1)
    model, pipe = _build(cfg)
    frames = 9
    noise = torch.randn((1, frames, 16, 16, 32), device="cuda:0", dtype=torch.bfloat16)
    attn = model.blocks[0].self_attn
    orig = attn.hsa_attention.append_kv

    def spy(k_new, v_new, *rest, position):
        spy.last = (k_new.clone(), v_new.clone())
        return orig(k_new, v_new, *rest, position=position)
    attn.hsa_attention.append_kv = spy
    g = torch.Generator(device="cuda:0").manual_seed(3)
    pipe.reset()
    out = pipe.generate(noise, [torch.randn(16, 64)], generator=g)
    assert torch.isfinite(out.float()).all()
    # after three chunks of a 6-frame window: the cache holds frames 3..8; its last chunk is the last recorded append
    k_last, v_last = spy.last
    cache = pipe.kv_cache[0]
    assert torch.equal(cache["k"][:, 3 * 128:], k_last) and torch.equal(cache["v"][:, 3 * 128:], v_last)


def test_prompt_switch_installs_pages_from_the_bank():
    from worldattention_b200.hkv.cache import HKVCache
    cfg = _small()
    hkv = HKVCache(frame_seq_length=cfg.frame_tokens, page_size_frames=2, topk_pages=2)
    model, pipe = _build(cfg, hkv=hkv)
    frames = 12
    noise = torch.randn((1, frames, 16, 16, 32), device="cuda:0", dtype=torch.bfloat16)
    prompts = [torch.randn(16, 64), torch.randn(16, 64)]
    out = pipe.generate(noise, prompts, switch_frames=[6])
    assert torch.isfinite(out.float()).all()
    assert pipe.stats.switches == 1 and pipe.stats.pages_installed == 2 and len(hkv) == 1
    # 2 pages of 2 frames were installed at the switch, then two more chunks were generated into the 6-frame window
    assert pipe.local_end == 6 * 128
    for blk, cache in zip(model.blocks, pipe.kv_cache):
        kc, vc = blk.self_attn.hsa_attention.compress_kv_cache(cache["k"], cache["v"])
        assert torch.equal(kc, cache["k_coarse"]) and torch.equal(vc, cache["v_coarse"])


def test_fused_block_wrappers_match_the_tensor_expressions():
    from worldattention_b200.causal_dit import _LayerNorm, gated_residual, ln_modulate
    dev = torch.device("cuda:0")
    torch.manual_seed(5)
    for b, frames, tokens, c in ((1, 3, 40, 1536), (2, 2, 7, 256), (1, 1, 33, 4096)):
        x = (torch.randn(b, frames * tokens, c, device=dev) * 2 + 0.3).bfloat16()
        y = torch.randn(b, frames * tokens, c, device=dev).bfloat16()
        e = (torch.randn(b, frames, 6, c, device=dev) * 0.5).bfloat16().chunk(6, dim=2)
        norm = _LayerNorm(c, 1e-6).to(dev)
        want = (norm(x).unflatten(1, (frames, tokens)) * (1 + e[1]) + e[0]).flatten(1, 2)
        got = ln_modulate(x, 1e-6, scale=e[1], shift=e[0], tokens_per_frame=tokens)
        # identical rounding points; the float32 statistics are summed in another order: allow one bf16 ulp on a few values
        diff = (got.float() - want.float()).abs()
        assert float((diff > 0).float().mean()) < 0.02 and float(diff.max()) <= 2 ** -6 * float(want.detach().float().abs().max())
        affine = _LayerNorm(c, 1e-6, elementwise_affine=True).to(dev, torch.bfloat16)
        with torch.no_grad():
            affine.weight.normal_(1, 0.2)
            affine.bias.normal_(0, 0.2)
        want = affine(x)
        got = ln_modulate(x, 1e-6, weight=affine.weight, bias=affine.bias)
        diff = (got.float() - want.float()).abs()
        assert float(diff.max()) <= 2 ** -6 * float(want.detach().float().abs().max())
        want = x + (y.unflatten(1, (frames, tokens)) * e[2]).flatten(1, 2)
        assert torch.equal(gated_residual(x, y, e[2], tokens_per_frame=tokens), want)
        assert torch.equal(gated_residual(x, y), x + y)


def test_fused_and_unfused_models_agree():
    cfg = _small()
    model, pipe = _build(cfg)
    noise = torch.randn((1, 6, 16, 16, 32), device="cuda:0", dtype=torch.bfloat16)
    prompts = [torch.randn(16, 64)]
    g = torch.Generator(device="cuda:0").manual_seed(9)
    fused = pipe.generate(noise, prompts, generator=g)
    for blk in model.blocks:
        blk.fused = False
    pipe.reset()
    g = torch.Generator(device="cuda:0").manual_seed(9)
    plain = pipe.generate(noise, prompts, generator=g)
    err = (fused.float() - plain.float()).abs()
    assert float(err.mean()) < 2e-2 * float(plain.float().abs().mean()) + 1e-3


def test_graph_replay_of_steady_chunks_equals_launch_by_launch():
    from worldattention_b200.causal_dit import ChunkPipeline
    cfg = _small()
    model, pipe = _build(cfg)
    noise = torch.randn((1, 18, 16, 16, 32), device="cuda:0", dtype=torch.bfloat16)     # 6 chunks: 4 of them roll the window
    prompts = [torch.randn(16, 64)]
    g = torch.Generator(device="cuda:0").manual_seed(2)
    plain = pipe.generate(noise, prompts, generator=g)
    caches = [{k: v.clone() for k, v in c.items()} for c in pipe.kv_cache]
    pipe2 = ChunkPipeline(model, device="cuda:0", cuda_graph=True)
    g = torch.Generator(device="cuda:0").manual_seed(2)
    replayed = pipe2.generate(noise, prompts, generator=g)
    assert pipe2.stats.graph_error is None and pipe2.stats.graph_replays == 4
    assert torch.equal(plain, replayed)
    for a, b in zip(caches, pipe2.kv_cache):
        assert torch.equal(a["k"], b["k"]) and torch.equal(a["k_coarse"], b["k_coarse"])
