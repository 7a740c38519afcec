"""Chunk-by-chunk autoregressive generation around the HSA layer and the HKV bank, for end-to-end timing.

A plain-torch restatement of the parts of the reference pipeline that surround the hot path, so that frames/s can be
measured with the hot path in its real place and with random-init weights of the Wan2.1-T2V-1.3B architecture:

* `CausalDiT` -- the 30-block diffusion transformer in KV-cache mode (wan/modules/causal_model.py:544-700 for a block
  and the head, :1121-1280 for the forward): patch embedding, time and text embeddings, per block a modulated
  self-attention over the rolling KV cache, a cross-attention over the cached text keys/values, a modulated FFN.
  GEMMs, layer norms and the cross-attention are library calls (cuBLAS, `scaled_dot_product_attention`): they are
  not the path this package accelerates.
* the self-attention of a block (causal_model.py:143-543) uses this package's kernels: q/k RMSNorm + causal RoPE in
  one launch each (`rope.qk_norm_rope`), the new rows and their compressed slots written into the layer's caches in
  place by one fused launch (`HSAAttention.append_kv`; the reference clones both caches every forward, :294-299), and
  `HSAAttention` over the window.
* `ChunkPipeline` -- the chunk loop (pipeline/causal_inference.py:200-259): per chunk of 3 latent frames 4 denoising
  forwards and one clean-context forward; with prompt switches served from the HKV bank
  (pipeline/interactive_causal_inference.py:93-130, 249-262): store the window, retrieve pages, install them.

The text encoder and the VAE are outside: the prompt embeddings are synthetic `[512, 4096]` tensors and the output is
the latent video.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, rope
from .hkv.cache import HKVCache
from .hkv.retrieval import query_index
from .hkv.rope import temporal_band
from .hsa.attention import HSAAttention

__all__ = ["DiTConfig", "CausalDiT", "ChunkPipeline", "rope_table"]


@dataclass
class DiTConfig:
    """Wan2.1-T2V-1.3B sizes (causal_model.py:704-730) and the cache policy of the inference config."""
    dim: int = 1536
    heads: int = 12
    ffn_dim: int = 8960
    layers: int = 30
    in_channels: int = 16
    out_channels: int = 16
    patch: tuple = (1, 2, 2)
    text_dim: int = 4096
    text_len: int = 512
    freq_dim: int = 256
    eps: float = 1e-6
    latent_hw: tuple = (60, 104)          # 480 x 832 video
    frames_per_chunk: int = 3
    window_frames: int = 21               # local attention window held in the KV cache
    hsa_block: int = 128
    hsa_topk: Optional[Sequence[int]] = None   # fixed per-head block counts; None = cumulative-mass routing
    denoising_steps: tuple = (1000, 750, 500, 250)
    context_noise: int = 0

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads

    @property
    def grid_hw(self) -> tuple:
        return (self.latent_hw[0] // self.patch[1], self.latent_hw[1] // self.patch[2])

    @property
    def frame_tokens(self) -> int:
        return self.grid_hw[0] * self.grid_hw[1]


def rope_table(head_dim: int, rows: int = 1024) -> torch.Tensor:
    """Complex rotary table `[rows, head_dim / 2]`: temporal, height and width bands side by side (model.py:32-44, 790-797)."""
    def band(dim):
        inv = 1.0 / torch.pow(10000.0, torch.arange(0, dim, 2, dtype=torch.float64) / dim)
        ang = torch.outer(torch.arange(rows, dtype=torch.float64), inv)
        return torch.polar(torch.ones_like(ang), ang)
    d = head_dim
    return torch.cat([band(d - 4 * (d // 6)), band(2 * (d // 6)), band(2 * (d // 6))], dim=1)


def _frame_vectors(e: Optional[torch.Tensor], dim: int):
    """`[B, F, 1, C]` modulation view -> (pointer, elements between consecutive frames); it must step uniformly over (b, f)."""
    if e is None:
        return None, 0
    b, f = e.shape[:2]
    if e.stride(-1) != 1 or e.shape[-1] != dim or (b > 1 and e.stride(0) != f * e.stride(1)):
        e = e.contiguous()
    return e.data_ptr(), e.stride(1)


def ln_modulate(x: torch.Tensor, eps: float, *, weight=None, bias=None, scale=None, shift=None, tokens_per_frame: int = 1):
    """`LayerNorm(x) [* weight + bias]`, then `* (1 + scale) + shift` per frame, in one pass over bf16 `[B, L, C]`
    (causal_model.py:616-619, 642-646; model.py:89-103)."""
    dev = _lib.require_cuda(x)
    if x.dtype != torch.bfloat16:
        raise NotImplementedError("the fused block glue is bf16 only")
    x = x.contiguous()
    out = torch.empty_like(x)
    c = x.shape[-1]
    sp, s_stride = _frame_vectors(scale, c)
    hp, h_stride = _frame_vectors(shift, c)
    if sp is not None and hp is not None and s_stride != h_stride:
        raise ValueError("scale and shift must share a layout")
    _lib.check(_lib.lib().wa_ln_modulate(x.data_ptr(), out.data_ptr(), x.numel() // c, c, float(eps), _lib.ptr(weight), _lib.ptr(bias),
                                         sp, hp, s_stride or h_stride, int(tokens_per_frame), _lib.stream_ptr(dev)))
    return out


def gated_residual(x: torch.Tensor, y: torch.Tensor, gate=None, *, tokens_per_frame: int = 1):
    """`x + y * gate` per frame (gate None: `x + y`) in one pass (causal_model.py:633, 637-638, 647-648)."""
    dev = _lib.require_cuda(x)
    if x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16:
        raise NotImplementedError("the fused block glue is bf16 only")
    x, y = x.contiguous(), y.contiguous()
    out = torch.empty_like(x)
    c = x.shape[-1]
    gp, g_stride = _frame_vectors(gate, c)
    _lib.check(_lib.lib().wa_gated_residual(x.data_ptr(), y.data_ptr(), out.data_ptr(), x.numel() // c, c, gp, g_stride,
                                            int(tokens_per_frame), _lib.stream_ptr(dev)))
    return out


class _RMSNorm(nn.Module):   # model.py:70-86
    def __init__(self, dim, eps):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        y = x.float()
        return (y * torch.rsqrt(y.pow(2).mean(dim=-1, keepdim=True) + self.eps)).type_as(x) * self.weight


class _LayerNorm(nn.LayerNorm):   # model.py:89-103: float32 statistics, no affine unless asked
    def __init__(self, dim, eps, elementwise_affine=False):
        super().__init__(dim, elementwise_affine=elementwise_affine, eps=eps)

    def forward(self, x):
        w = None if self.weight is None else self.weight.float()
        b = None if self.bias is None else self.bias.float()
        return F.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).type_as(x)


class _SelfAttention(nn.Module):
    """causal_model.py:65-111, 143-543, KV-cache branch, HSA backend, no sink tokens."""

    def __init__(self, cfg: DiTConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        self.q, self.k, self.v, self.o = (nn.Linear(d, d) for _ in range(4))
        self.norm_q, self.norm_k = _RMSNorm(d, cfg.eps), _RMSNorm(d, cfg.eps)
        self.hsa_attention = HSAAttention(cfg.heads, cfg.head_dim, block_size=cfg.hsa_block, proj_segment_len=cfg.frame_tokens)

    def forward(self, x, cache: dict, plan: dict, table: torch.Tensor):
        cfg = self.cfg
        b, s, _ = x.shape
        grid = (s // cfg.frame_tokens,) + cfg.grid_hw
        q = rope.qk_norm_rope(self.q(x), self.norm_q.weight, cfg.eps, grid, None, plan["start_frame"], heads=cfg.heads, table=table)
        k = rope.qk_norm_rope(self.k(x), self.norm_k.weight, cfg.eps, grid, None, plan["start_frame"], heads=cfg.heads, table=table)
        v = self.v(x).view(b, s, cfg.heads, cfg.head_dim)
        hsa = self.hsa_attention
        if plan["roll"]:
            # the window is full: drop the oldest frames (causal_model.py:331-360).  Source and destination overlap,
            # so each tensor goes through one scratch copy of the kept rows.
            ev, keep = plan["evict"], plan["keep"]
            c0, c1 = hsa.token_range_to_coarse(ev, ev + keep)
            for name, a, n in (("k", ev, keep), ("v", ev, keep), ("k_coarse", c0, c1 - c0), ("v_coarse", c0, c1 - c0)):
                cache[name][:, :n] = cache[name][:, a:a + n].clone()
        hsa.append_kv(k, v, cache["k"], cache["v"], cache["k_coarse"], cache["v_coarse"], position=plan["write"])
        end = plan["write"] + s
        c_end = hsa.token_range_to_coarse(0, end)[1]
        y = hsa(q, cache["k"][:, :end], cache["v"][:, :end], k_coarse=cache["k_coarse"][:, :c_end],
                v_coarse=cache["v_coarse"][:, :c_end])
        return self.o(y.flatten(2))


class _CrossAttention(nn.Module):   # model.py:165-200 (text-to-video), keys/values of the text cached per prompt
    def __init__(self, cfg: DiTConfig):
        super().__init__()
        d = cfg.dim
        self.heads = cfg.heads
        self.q, self.k, self.v, self.o = (nn.Linear(d, d) for _ in range(4))
        self.norm_q, self.norm_k = _RMSNorm(d, cfg.eps), _RMSNorm(d, cfg.eps)

    def forward(self, x, context, cache: dict):
        b, s, d = x.shape
        h = self.heads
        if x.is_cuda and x.dtype == torch.bfloat16:
            q = rope.qk_norm_rope(self.q(x), self.norm_q.weight, self.norm_q.eps, None, None, heads=h).transpose(1, 2)
        else:
            q = self.norm_q(self.q(x)).view(b, s, h, d // h).transpose(1, 2)
        if not cache.get("is_init", False):
            k_new = self.norm_k(self.k(context)).view(b, -1, h, d // h).transpose(1, 2).contiguous()
            v_new = self.v(context).view(b, -1, h, d // h).transpose(1, 2).contiguous()
            if "k" in cache and cache["k"].shape == k_new.shape:      # keep the addresses: a captured graph may hold them
                cache["k"].copy_(k_new)
                cache["v"].copy_(v_new)
            else:
                cache["k"], cache["v"] = k_new, v_new
            cache["is_init"] = True
        y = F.scaled_dot_product_attention(q, cache["k"], cache["v"])
        return self.o(y.transpose(1, 2).reshape(b, s, d))


class _Block(nn.Module):   # causal_model.py:544-659
    def __init__(self, cfg: DiTConfig):
        super().__init__()
        d = cfg.dim
        self.norm1, self.norm2 = _LayerNorm(d, cfg.eps), _LayerNorm(d, cfg.eps)
        self.norm3 = _LayerNorm(d, cfg.eps, elementwise_affine=True)
        self.self_attn = _SelfAttention(cfg)
        self.cross_attn = _CrossAttention(cfg)
        self.ffn = nn.Sequential(nn.Linear(d, cfg.ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(cfg.ffn_dim, d))
        self.modulation = nn.Parameter(torch.randn(1, 6, d) / d ** 0.5)
        self.fused = True     # False: the wrappers as the reference's tensor expressions (kept for the comparison test)

    def forward(self, x, e, context, cache, cross_cache, plan, table):
        frames = e.shape[1]
        tokens = x.shape[1] // frames
        e = (self.modulation.unsqueeze(1) + e).contiguous().chunk(6, dim=2)          # six [B, F, 1, C] views of one tensor
        eps = self.norm1.eps
        if not self.fused:
            def per_frame(t, scale, shift=None):
                t = t.unflatten(1, (frames, tokens)) * scale
                return (t + shift if shift is not None else t).flatten(1, 2)
            y = self.self_attn(per_frame(self.norm1(x), 1 + e[1], e[0]), cache, plan, table)
            x = x + per_frame(y, e[2])
            x = x + self.cross_attn(self.norm3(x), context, cross_cache)
            y = self.ffn(per_frame(self.norm2(x), 1 + e[4], e[3]))
            return x + per_frame(y, e[5])
        # the same sub-layers with each wrapper as one launch
        y = self.self_attn(ln_modulate(x, eps, scale=e[1], shift=e[0], tokens_per_frame=tokens), cache, plan, table)
        x = gated_residual(x, y, e[2], tokens_per_frame=tokens)
        y = self.cross_attn(ln_modulate(x, eps, weight=self.norm3.weight, bias=self.norm3.bias), context, cross_cache)
        x = gated_residual(x, y)
        y = self.ffn(ln_modulate(x, eps, scale=e[4], shift=e[3], tokens_per_frame=tokens))
        return gated_residual(x, y, e[5], tokens_per_frame=tokens)


class CausalDiT(nn.Module):
    """The diffusion transformer in KV-cache mode: one call denoises one chunk against the layer caches."""

    def __init__(self, cfg: DiTConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        self.patch_embedding = nn.Conv3d(cfg.in_channels, d, kernel_size=cfg.patch, stride=cfg.patch)
        self.text_embedding = nn.Sequential(nn.Linear(cfg.text_dim, d), nn.GELU(approximate="tanh"), nn.Linear(d, d))
        self.time_embedding = nn.Sequential(nn.Linear(cfg.freq_dim, d), nn.SiLU(), nn.Linear(d, d))
        self.time_projection = nn.Sequential(nn.SiLU(), nn.Linear(d, 6 * d))
        self.blocks = nn.ModuleList(_Block(cfg) for _ in range(cfg.layers))
        self.head_norm = _LayerNorm(d, cfg.eps)
        self.head = nn.Linear(d, math.prod(cfg.patch) * cfg.out_channels)
        self.head_modulation = nn.Parameter(torch.randn(1, 2, d) / d ** 0.5)
        self.freqs = rope_table(cfg.head_dim)
        self._table = None

    def init_hsa(self, seed: int = 0) -> None:
        """Random stand-ins for the trained HSA parameters (the constructor leaves them at zero, as the reference does)."""
        g = torch.Generator(device="cpu").manual_seed(seed)
        for blk in self.blocks:
            hsa = blk.self_attn.hsa_attention
            with torch.no_grad():
                for p in (hsa.k_proj_mat, hsa.v_proj_mat):
                    p.copy_((torch.randn(p.shape, generator=g) / math.sqrt(self.cfg.hsa_block)).to(p.dtype))
                hsa.gate_lin.weight.copy_(torch.randn(hsa.gate_lin.weight.shape, generator=g) * 0.05)
                hsa.gate_lin.bias.copy_(torch.randn(hsa.gate_lin.bias.shape, generator=g) * 0.2)
                if self.cfg.hsa_topk is not None:
                    hsa.topk_per_head = torch.tensor(list(self.cfg.hsa_topk), dtype=torch.int32, device=p.device)

    def table(self, dev) -> torch.Tensor:
        if self._table is None or self._table.device != dev:
            self._table = torch.view_as_real(self.freqs.to(torch.complex128)).to(device=dev, dtype=torch.float64).contiguous()
        return self._table

    def embed_text(self, prompt_embeds: torch.Tensor) -> torch.Tensor:
        return self.text_embedding(prompt_embeds)

    def forward(self, latents, timestep, context, kv_cache: List[dict], cross_cache: List[dict], plan: dict):
        """`latents` [B, F, C, H, W], `timestep` [B, F] -> flow prediction of the same shape (causal_model.py:1121-1280)."""
        cfg = self.cfg
        b, f = latents.shape[:2]
        x = self.patch_embedding(latents.permute(0, 2, 1, 3, 4)).flatten(2).transpose(1, 2)        # [B, F*tokens, C]
        half = cfg.freq_dim // 2
        pos = timestep.flatten().to(torch.float64)
        ang = torch.outer(pos, torch.pow(10000.0, -torch.arange(half, dtype=torch.float64, device=pos.device) / half))
        sin = torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(x.dtype)                       # model.py:19-29
        e = self.time_embedding(sin)
        e0 = self.time_projection(e).unflatten(1, (6, cfg.dim)).unflatten(0, (b, f))               # [B, F, 6, C]
        table = self.table(x.device)
        for blk, cache, cross in zip(self.blocks, kv_cache, cross_cache):
            x = blk(x, e0, context, cache, cross, plan, table)
        m = (self.head_modulation.unsqueeze(1) + e.unflatten(0, (b, f)).unsqueeze(2)).chunk(2, dim=2)
        tokens = cfg.frame_tokens
        x = self.head(self.head_norm(x).unflatten(1, (f, tokens)) * (1 + m[1]) + m[0])              # [B, F, tokens, p*C]
        gh, gw = cfg.grid_hw
        x = x.view(b, f, gh, gw, cfg.patch[1], cfg.patch[2], cfg.out_channels)
        return x.permute(0, 1, 6, 2, 4, 3, 5).reshape(b, f, cfg.out_channels, gh * cfg.patch[1], gw * cfg.patch[2])


@dataclass
class _Stats:
    chunks: int = 0
    forwards: int = 0
    switches: int = 0
    pages_installed: int = 0
    chunk_ms: List[float] = field(default_factory=list)
    switch_ms: List[float] = field(default_factory=list)
    switch_parts_ms: List[List[float]] = field(default_factory=list)      # [store, retrieve, apply] per switch
    graph_replays: int = 0
    graph_error: Optional[str] = None


class ChunkPipeline:
    """The chunk loop with the rolling per-layer caches and an optional HKV bank for prompt switches."""

    def __init__(self, model: CausalDiT, *, hkv: Optional[HKVCache] = None, device=None, dtype=torch.bfloat16,
                 cuda_graph: bool = False):
        self.model = model
        self.cfg = model.cfg
        self.hkv = hkv
        # once the window is full every chunk runs the same launches on the same addresses (roll, write at the tail);
        # with `cuda_graph` those five forwards are captured once and replayed, the frame index being read from device memory
        self.cuda_graph = bool(cuda_graph)
        self._graph = None
        self.dev = torch.device(device) if device is not None else next(model.parameters()).device
        self.dtype = dtype
        self.stats = _Stats()
        self.reset()

    def reset(self, keep_buffers: bool = False) -> None:
        """Empty caches for a new video.  `keep_buffers`: clear the existing cache tensors instead of allocating new
        ones, so that a graph captured over their addresses stays valid (a serving process captures once)."""
        cfg, dev = self.cfg, self.dev
        if keep_buffers and getattr(self, "kv_cache", None):
            for cache in self.kv_cache:
                for t in cache.values():
                    t.zero_()
            for c in self.cross_cache:
                c["is_init"] = False
            self.local_end = self.global_end = 0
            if self.hkv is not None:
                self.hkv.reset()
            return
        size = cfg.window_frames * cfg.frame_tokens
        self.kv_cache = []
        for blk in self.model.blocks:
            hsa = blk.self_attn.hsa_attention
            coarse = hsa.coarse_cache_size(size)
            shape, cshape = (1, size, cfg.heads, cfg.head_dim), (1, coarse, cfg.heads, cfg.head_dim)
            self.kv_cache.append({
                "k": torch.zeros(shape, dtype=self.dtype, device=dev), "v": torch.zeros(shape, dtype=self.dtype, device=dev),
                "k_coarse": torch.zeros(cshape, dtype=self.dtype, device=dev),
                "v_coarse": torch.zeros(cshape, dtype=self.dtype, device=dev),
                "global_end_index": torch.zeros(1, dtype=torch.long, device=dev),
                "local_end_index": torch.zeros(1, dtype=torch.long, device=dev),
            })
        self.cross_cache = [{"is_init": False} for _ in self.model.blocks]
        self.local_end = 0          # host copies of the two indices: the loop never reads them back from the device
        self.global_end = 0
        self._graph = None
        if self.hkv is not None:
            self.hkv.reset()

    # ---- cache bookkeeping (causal_model.py:331-343, 395-399), on the host
    def _plan(self, start_frame: int) -> dict:
        cfg = self.cfg
        s = cfg.frames_per_chunk * cfg.frame_tokens
        current_start, current_end = start_frame * cfg.frame_tokens, start_frame * cfg.frame_tokens + s
        size = cfg.window_frames * cfg.frame_tokens
        plan = {"start_frame": start_frame, "roll": False}
        if current_end > self.global_end and s + self.local_end > size:
            evict = s + self.local_end - size
            plan.update(roll=True, evict=evict, keep=self.local_end - evict)
            local_end = self.local_end + current_end - self.global_end - evict
        else:
            local_end = self.local_end + current_end - self.global_end
        plan["write"] = local_end - s
        plan["local_end"], plan["global_end"] = local_end, max(self.global_end, current_end)
        return plan

    def _commit(self, plan: dict) -> None:
        self.local_end, self.global_end = plan["local_end"], plan["global_end"]
        for cache in self.kv_cache:      # kept for consumers that read the device copies (the HKV bank does)
            cache["local_end_index"].fill_(self.local_end)
            cache["global_end_index"].fill_(self.global_end)

    # ---- prompt switch through the bank (interactive_causal_inference.py:93-130)
    def _switch(self, prev_prompt, next_prompt, noisy_chunk, start_frame: int) -> int:
        model, cfg = self.model, self.cfg
        marks = [time.perf_counter()]

        def mark():      # a switch is rare: synchronising here only makes its three parts separately visible
            torch.cuda.synchronize(self.dev)
            marks.append(time.perf_counter())

        band = temporal_band(model.freqs, cfg.head_dim).to(self.dev)
        self.hkv.store(self.kv_cache, prompt_embeds=prev_prompt, current_start_frame=start_frame, temporal_freqs=band)
        mark()
        for c in self.cross_cache:
            c["is_init"] = False
        attn = model.blocks[0].self_attn
        tokens = model.patch_embedding(noisy_chunk.permute(0, 2, 1, 3, 4)).flatten(2).transpose(1, 2)
        qvec = query_index(attn.norm_q(attn.q(tokens)))
        pages = self.hkv.retrieve(prompt_embeds=next_prompt, query_vec=qvec)
        mark()
        installed = 0
        if pages:
            installed = self.hkv.apply(self.kv_cache, pages, current_start_frame=start_frame, temporal_freqs=band,
                                       hsa_modules=[b.self_attn.hsa_attention for b in model.blocks])
            if installed > 0:
                self.local_end, self.global_end = installed, start_frame * cfg.frame_tokens
            self.stats.pages_installed += len(pages)
        mark()
        self.stats.switch_parts_ms.append([round((b - a) * 1e3, 2) for a, b in zip(marks, marks[1:])])
        return installed

    def _chunk_body(self, x_t, eps, context, plan: dict, start_frame):
        """The chunk's denoising forwards and the clean-context forward (causal_inference.py:222-259) -> the clean latent."""
        cfg, model = self.cfg, self.model
        plan = dict(plan, start_frame=start_frame)
        later = dict(plan, roll=False)          # the window is rolled once; later forwards rewrite the same rows
        x0 = None
        for i, t in enumerate(cfg.denoising_steps):
            flow = model(x_t, self._timestep(t), context, self.kv_cache, self.cross_cache, plan if i == 0 else later)
            x0 = x_t - (t / 1000.0) * flow                                  # flow prediction -> clean latent
            if i + 1 < len(cfg.denoising_steps):
                nxt = cfg.denoising_steps[i + 1] / 1000.0
                x_t = (1 - nxt) * x0 + nxt * eps[i]                         # re-noise for the next step (utils/scheduler.py add_noise)
        model(x0, self._timestep(cfg.context_noise), context, self.kv_cache, self.cross_cache, later)   # clean keys and values
        return x0

    def _timestep(self, t) -> torch.Tensor:
        cache = self.__dict__.setdefault("_ts", {})
        if t not in cache:
            cache[t] = torch.full((1, self.cfg.frames_per_chunk), float(t), device=self.dev)
        return cache[t]

    def _replay(self, x_t, eps, context, plan, frame):
        """A steady-state chunk through the captured graph (captured on first use; any failure turns graphs off)."""
        if self._graph is None:
            try:
                static = {"x": x_t.clone(), "eps": eps.clone(), "ctx": context.clone(),
                          "frame": torch.tensor([frame], dtype=torch.int32, device=self.dev)}
                for t in list(self.cfg.denoising_steps) + [self.cfg.context_noise]:
                    self._timestep(t)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    static["out"] = self._chunk_body(static["x"], static["eps"], static["ctx"], plan, static["frame"])
                self._graph = (graph, static, (plan["evict"], plan["keep"], plan["write"]))
            except Exception as exc:      # reported by the caller's stats; the chunk then runs launch by launch
                self.stats.graph_error = f"{type(exc).__name__}: {exc}"
                torch.cuda.synchronize(self.dev)
                return self._chunk_body(x_t, eps, context, plan, frame)
        graph, static, key = self._graph
        assert key == (plan["evict"], plan["keep"], plan["write"])
        static["x"].copy_(x_t)
        static["eps"].copy_(eps)
        static["ctx"].copy_(context)
        static["frame"].fill_(frame)
        graph.replay()
        self.stats.graph_replays += 1
        return static["out"]

    @torch.no_grad()
    def generate(self, noise: torch.Tensor, prompts: Sequence[torch.Tensor], switch_frames: Sequence[int] = (),
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """`noise` [1, T, C, H, W]; `prompts` synthetic text embeddings `[512, 4096]`, one more than `switch_frames`."""
        cfg, model = self.cfg, self.model
        assert noise.shape[1] % cfg.frames_per_chunk == 0 and len(prompts) == len(switch_frames) + 1
        contexts = [model.embed_text(p.to(self.dev, self.dtype).unsqueeze(0)) for p in prompts]
        out = torch.empty_like(noise)
        segment, frame = 0, 0
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        while frame < noise.shape[1]:
            ev[0].record()
            if segment < len(switch_frames) and frame >= switch_frames[segment]:
                segment += 1
                if self.hkv is not None:
                    self._switch(prompts[segment - 1].to(self.dev, self.dtype).unsqueeze(0),      # [B, tokens, dim], as the bank expects
                                 prompts[segment].to(self.dev, self.dtype).unsqueeze(0),
                                 noise[:, frame:frame + cfg.frames_per_chunk], frame)
                    self.stats.switches += 1
                else:
                    for c in self.cross_cache:
                        c["is_init"] = False
            ev[1].record()
            context = contexts[segment]
            x_t = noise[:, frame:frame + cfg.frames_per_chunk]
            plan = self._plan(frame)
            steps = len(cfg.denoising_steps)
            eps = torch.randn((steps - 1,) + tuple(x_t.shape), device=self.dev, dtype=x_t.dtype, generator=generator)
            steady = plan["roll"] and plan["write"] + x_t.shape[1] * cfg.frame_tokens == cfg.window_frames * cfg.frame_tokens
            if (self.cuda_graph and steady and self.stats.graph_error is None
                    and all(c.get("is_init", False) for c in self.cross_cache)):
                x0 = self._replay(x_t, eps, context, plan, frame)
            else:
                x0 = self._chunk_body(x_t, eps, context, plan, frame)
            self.stats.forwards += steps + 1
            out[:, frame:frame + cfg.frames_per_chunk] = x0
            self._commit(plan)
            ev[2].record()
            ev[2].synchronize()
            self.stats.switch_ms.append(ev[0].elapsed_time(ev[1]))
            self.stats.chunk_ms.append(ev[0].elapsed_time(ev[2]))
            self.stats.chunks += 1
            frame += cfg.frames_per_chunk
        return out


def time_generation(cfg: DiTConfig, *, chunks: int, switch_every_chunks: int = 0, hkv_kwargs: Optional[dict] = None,
                    seed: int = 0, device="cuda:0", cuda_graph: bool = False) -> dict:
    """Build a random-init model, generate `chunks` chunks, and return frames/s with the per-chunk times."""
    dev = torch.device(device)
    torch.manual_seed(seed)
    model = CausalDiT(cfg).to(dev, torch.bfloat16).eval()
    model.init_hsa(seed)
    hkv = None
    if switch_every_chunks > 0:
        hkv = HKVCache(frame_seq_length=cfg.frame_tokens, **(hkv_kwargs or {}))
    pipe = ChunkPipeline(model, hkv=hkv, device=dev, cuda_graph=cuda_graph)
    frames = chunks * cfg.frames_per_chunk
    g = torch.Generator(device=dev).manual_seed(seed)
    noise = torch.randn((1, frames, cfg.in_channels) + tuple(cfg.latent_hw), device=dev, dtype=torch.bfloat16, generator=g)
    switches = [c * cfg.frames_per_chunk for c in range(switch_every_chunks, chunks, switch_every_chunks)] if switch_every_chunks else []
    gp = torch.Generator(device="cpu").manual_seed(seed + 1)
    prompts = [torch.randn((cfg.text_len, cfg.text_dim), generator=gp) for _ in range(len(switches) + 1)]
    # untimed: enough chunks to fill the window and run one steady-state chunk (with `cuda_graph` that is where the
    # graph is captured: once per process, as a serving process would), then with a bank one prompt switch (store,
    # retrieve, install), so that library initialisation and first-call set-up are not counted as generation time
    fpc = cfg.frames_per_chunk
    fill = -(-cfg.window_frames // fpc) + 1
    warm = min(fill + (1 if hkv is not None else 0), chunks)
    if hkv is not None and warm > 1:
        pipe.generate(noise[:, :warm * fpc], [prompts[0], prompts[0]], [(warm - 1) * fpc], generator=g)
    else:
        pipe.generate(noise[:, :warm * fpc], prompts[:1], generator=g)
    reserved = 0
    if hkv is not None:
        # the bank's HBM: one allocation handed to the caching allocator, which the stored windows then come out of
        # (growing the pool by one stored window at a time costs a driver allocation of several GB inside a switch);
        # after the warm-up, because entering a graph capture returns cached blocks to the driver
        window_bytes = 2 * cfg.layers * cfg.window_frames * cfg.frame_tokens * cfg.heads * cfg.head_dim * 2
        banked = min(len(switches), int((hkv_kwargs or {}).get("hbm_max_chunks", 0)) + 1)
        free_bytes, _ = torch.cuda.mem_get_info(dev)
        reserved = min(banked * window_bytes, max(0, free_bytes - (32 << 30)))
        if reserved > 0:
            del_me = torch.empty(reserved, dtype=torch.uint8, device=dev)
            del del_me
    pipe.reset(keep_buffers=True)
    pipe.stats = _Stats()
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    out = pipe.generate(noise, prompts, switches, generator=g)
    torch.cuda.synchronize(dev)
    wall = time.perf_counter() - t0
    _lib.raise_if_failed(dev)         # replayed launches are not checked one by one
    st = pipe.stats
    steady = sorted(st.chunk_ms[len(st.chunk_ms) // 2:]) or [float("nan")]
    return {
        "frames": frames, "chunks": chunks, "forwards": st.forwards, "wall_s": wall, "frames_per_s": frames / wall,
        "frames_per_s_steady": cfg.frames_per_chunk / (steady[len(steady) // 2] * 1e-3),
        "chunk_ms_median_second_half": steady[len(steady) // 2], "chunk_ms_first": st.chunk_ms[0] if st.chunk_ms else None,
        "switches": st.switches, "pages_installed": st.pages_installed,
        "switch_ms": [round(v, 3) for v in st.switch_ms if v > 0.05],
        "switch_store_retrieve_apply_ms": st.switch_parts_ms,
        "finite": bool(torch.isfinite(out.float()).all()),
        "cuda_graph": {"asked": bool(cuda_graph), "replayed_chunks": st.graph_replays, "error": st.graph_error,
                       "captured": "in the untimed warm-up (once per process)"},
        "warmup_chunks": warm, "bank_hbm_reserved_gb": round(reserved / 2 ** 30, 1),
        "window_frames": cfg.window_frames, "hsa_block": cfg.hsa_block,
        "hsa_topk": "cumulative-mass" if cfg.hsa_topk is None else list(cfg.hsa_topk),
    }
