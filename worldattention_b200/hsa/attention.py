"""Hybrid Sparse Attention (HSA) forward on B200.

Drop-in for the reference's `wan/modules/hsa/attention.py`: the same module class, parameter
names, functional entry point and helper signatures.  One call of `hsa_attention` becomes one
call of `wa_hsa_forward` in libwa_b200.so, which reads the `[B, L, H, D]` tensors in place (no
transpose / pad / cast copies) and runs routing, the block-sparse branch, the compressed
("linear") branch and the gated combine on the current CUDA stream.

Inference only: the CUDA forward builds no autograd graph.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.nn as nn

from .. import _lib
from . import distill

__all__ = [
    "HSAAttention", "hsa_attention", "compress_kv", "append_kv", "resolve_backend", "hsa_parameter_names",
    "require_trained_hsa",
]

_BACKENDS = ("auto", "triton", "torch")
_HSA_ATTR = "hsa_attention"
SUPPORTED_BLOCK_SIZES = (64, 128)


def resolve_backend(backend: str) -> str:
    """Validate a backend name (reference: attention.py:47-61).

    The names are kept for configuration compatibility; every one of them runs the CUDA library.
    `"auto"` reports `"triton"` on a GPU box, as the reference does off sm_90, and `"torch"` where
    no CUDA device is visible.
    """
    backend = str(backend or "auto").lower()
    if backend not in _BACKENDS:
        raise ValueError(f"unknown HSA backend {backend!r}; expected one of {_BACKENDS}")
    if backend != "auto":
        return backend
    return "triton" if torch.cuda.is_available() else "torch"


def _coarse_len(kv_len: int, segment_len: int, rank: int, block_size: int) -> int:
    if segment_len <= 0:
        segment_len = kv_len
    total = 0
    for start in range(0, kv_len, segment_len):
        total += min(rank, math.ceil(min(segment_len, kv_len - start) / block_size))
    return total


def _compress_blhd(k, v, *, segment_len, k_proj_mat, v_proj_mat, block_size):
    """compress on `[B, L, H, D]` views -> contiguous `[B, Lc, H, D]`."""
    if k_proj_mat.shape != v_proj_mat.shape:
        raise ValueError(
            "k_proj_mat and v_proj_mat must have the same shape, got "
            f"{tuple(k_proj_mat.shape)} and {tuple(v_proj_mat.shape)}"
        )
    dev = _lib.require_cuda(k, v)
    bsz, kv_len, heads, head_dim = k.shape
    seg = segment_len if segment_len > 0 else kv_len
    longest = min(seg, kv_len)
    if longest > k_proj_mat.shape[1]:
        raise ValueError(
            f"segment length {longest} exceeds projection length {k_proj_mat.shape[1]}; "
            "increase proj_segment_len"
        )
    v = v.to(k.dtype)
    lc = _coarse_len(kv_len, seg, k_proj_mat.shape[0], block_size)
    out_k = torch.empty((bsz, lc, heads, head_dim), device=dev, dtype=k.dtype)
    out_v = torch.empty_like(out_k)
    pk = k_proj_mat.detach().to(device=dev).contiguous()
    pv = v_proj_mat.detach().to(device=dev, dtype=pk.dtype).contiguous()
    _lib.check(_lib.lib().wa_compress_kv(
        _lib.t4_blhd(k), _lib.t4_blhd(v), _lib.t4_blhd(out_k), _lib.t4_blhd(out_v), bsz, kv_len, heads, head_dim,
        seg, block_size, pk.data_ptr(), pv.data_ptr(), _lib.dtype_code(pk.dtype), pk.shape[0], pk.shape[1],
        _lib.stream_ptr(dev)))
    return out_k, out_v


_append_workspaces: dict = {}


def append_kv(k_new, v_new, k_cache, v_cache, k_coarse, v_coarse, *, position: int, segment_len: int, k_proj_mat, v_proj_mat,
              block_size: int) -> None:
    """Write `n_new` token rows into the K/V cache at `position` and compress the segments they complete, in ONE kernel.

    Stands in for the cache update of the reference's `CausalWanSelfAttention.forward` (causal_model.py:294-327,
    395-413: clone the layer cache, write the rows, `compress_kv_cache` of the new segments into the coarse cache).
    All tensors `[B, *, H, D]` bf16; `position` is a multiple of `segment_len`.  `k_new` / `v_new` may be views of the
    cache rows themselves (rows already in place): then the call only compresses.  Shapes the fused kernel does not cover
    go through a copy and `compress_kv`.
    """
    dev = _lib.require_cuda(k_new, v_new, k_cache, v_cache, k_coarse, v_coarse)
    bsz, n_new, heads, head_dim = k_new.shape
    if position % segment_len:
        raise ValueError(f"rows are appended at segment boundaries, got position={position}, segment_len={segment_len}")
    if position + n_new > k_cache.shape[1]:
        raise ValueError("the rows do not fit the cache")
    pk = k_proj_mat.detach().to(device=dev).contiguous()
    pv = v_proj_mat.detach().to(device=dev, dtype=pk.dtype).contiguous()
    lib = _lib.lib()
    need = lib.wa_kv_append_workspace_bytes(bsz, n_new, heads, head_dim, segment_len, block_size, pk.shape[0])
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    ws = _append_workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 16), device=dev, dtype=torch.uint8)      # zeroed once; every call leaves it zeroed
        _append_workspaces[key] = ws
    with _lib.device_guard(dev):
        rc = lib.wa_kv_append_compress(
            _lib.t4_blhd(k_new), _lib.t4_blhd(v_new), _lib.t4_blhd(k_cache), _lib.t4_blhd(v_cache), _lib.t4_blhd(k_coarse),
            _lib.t4_blhd(v_coarse), bsz, n_new, int(position), heads, head_dim, int(segment_len), int(block_size), pk.data_ptr(),
            pv.data_ptr(), _lib.dtype_code(pk.dtype), pk.shape[0], pk.shape[1], ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev))
    if rc == _lib.WA_ERR_UNSUPPORTED:
        rows_k, rows_v = k_cache[:, position:position + n_new], v_cache[:, position:position + n_new]
        if rows_k.data_ptr() != k_new.data_ptr():
            rows_k.copy_(k_new)
            rows_v.copy_(v_new)
        per_segment = min(pk.shape[0], math.ceil(segment_len / block_size))      # slots of a whole segment in the cache
        for s0 in range(0, n_new, segment_len):                                 # the last segment may be short (fewer slots)
            s1 = min(n_new, s0 + segment_len)
            kn, vn = _compress_blhd(rows_k[:, s0:s1], rows_v[:, s0:s1], segment_len=segment_len, k_proj_mat=pk, v_proj_mat=pv,
                                    block_size=block_size)
            first = (position + s0) // segment_len * per_segment
            k_coarse[:, first:first + kn.shape[1]].copy_(kn)
            v_coarse[:, first:first + vn.shape[1]].copy_(vn)
        return
    _lib.check(rc)


def compress_kv(k, v, *, segment_len: int, k_proj_mat, v_proj_mat, block_size: int):
    """Project `[B, H, L, D]` keys and values onto the low-rank sequence basis (attention.py:64-110)."""
    out_k, out_v = _compress_blhd(k.transpose(1, 2), v.transpose(1, 2), segment_len=segment_len,
                                  k_proj_mat=k_proj_mat, v_proj_mat=v_proj_mat, block_size=block_size)
    return out_k.transpose(1, 2).contiguous(), out_v.transpose(1, 2).contiguous()


def _linear_branch(q: torch.Tensor, k_coarse: torch.Tensor, v_coarse: torch.Tensor) -> torch.Tensor:
    """Attention of `[B, H, Lq, D]` queries over the compressed keys/values (attention.py:113-118)."""
    dev = _lib.require_cuda(q, k_coarse, v_coarse)
    bsz, heads, q_len, head_dim = q.shape
    lc = k_coarse.shape[2]
    k_coarse = k_coarse.to(v_coarse.dtype)
    out = torch.empty((bsz, heads, q_len, head_dim), device=dev, dtype=v_coarse.dtype)
    _lib.check(_lib.lib().wa_linear_branch(
        _lib.t4_bhnd(q), _lib.t4_bhnd(k_coarse), _lib.t4_bhnd(v_coarse), _lib.t4_bhnd(out), bsz, heads, q_len, lc,
        head_dim, int(v_coarse.dtype == torch.bfloat16), None, _lib.stream_ptr(dev)))
    return out


def hsa_parameter_names(model: nn.Module) -> list[str]:
    """State-dict keys of every HSA parameter in `model`, found by module type (attention.py:121-132)."""
    names = []
    for module_name, module in model.named_modules():
        if isinstance(module, HSAAttention):
            prefix = f"{module_name}." if module_name else ""
            names.extend(prefix + name for name, _ in module.named_parameters())
    return names


def require_trained_hsa(missing_keys, checkpoint_path: str = "") -> None:
    """Raise if a checkpoint load left any HSA parameter unfilled (attention.py:135-150)."""
    missing_hsa = [key for key in missing_keys if _HSA_ATTR in key]
    if not missing_hsa:
        return
    where = f" in {checkpoint_path}" if checkpoint_path else ""
    raise RuntimeError(
        f"{len(missing_hsa)} HSA parameters are absent{where}: the checkpoint predates HSA training. "
        f"Load a checkpoint produced by the HSA stage (or run the dense attn_backend=flash baseline). "
        f"First missing keys: {missing_hsa[:6]}"
    )


def _unit_last(t: torch.Tensor) -> torch.Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


_workspaces: dict = {}


def _workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
    """One growing scratch buffer per (device, stream); kernels of one stream are ordered."""
    key = (dev, torch.cuda.current_stream(dev).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), device=dev, dtype=torch.uint8)
        _workspaces[key] = buf
    return buf


def hsa_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    k_coarse: torch.Tensor | None = None,
    v_coarse: torch.Tensor | None = None,
    k_proj_mat: torch.Tensor,
    v_proj_mat: torch.Tensor,
    gate_lin: nn.Module | None = None,
    block_size: int = 64,
    tau_min: float = 0.35,
    tau_max: float = 1.0,
    proj_segment_len: int = 1560,
    backend: str = "auto",
    topk_per_head: torch.Tensor | None = None,
    force_generic: bool = False,
    return_routing: bool = False,
    check_status: bool = False,
    k_pooled_cache: torch.Tensor | None = None,
    k_pooled_valid: int = 0,
):
    """Run HSA over `[B, L, H, D]` queries, keys and values (attention.py:153-259).

    Beyond the reference signature: `topk_per_head` (int32 `[H]`) selects a fixed number of blocks
    per head instead of the cumulative-mass count; `force_generic` skips the tcgen05 kernel;
    `return_routing` also returns `(index, num, thresholds, used_tuned)`; `check_status` waits for
    the launch and raises if a bounded wait inside the tcgen05 kernel ran out (without it, such a
    failure raises at the next call on the device, or when the caller runs `_lib.raise_if_failed`
    after its own synchronisation).

    `k_pooled_cache` (float32 `[B, H, ceil(Lkv / block_size), D]`, contiguous) is state the caller
    keeps next to a growing key cache: its first `k_pooled_valid` rows already hold the block means of
    `k` (blocks that were complete at an earlier call and have not changed).  Only the later blocks
    are pooled, into the buffer; the result is the same as without it.  The reference pools the
    whole cache on every call (routing.py:45-61); at a 748 800-token cache that is 2.3 GB per call.
    """
    if (k_coarse is None) != (v_coarse is None):
        raise ValueError("k_coarse and v_coarse must be provided together")
    resolve_backend(backend)

    bsz, q_len, heads, head_dim = q.shape
    kv_len = k.shape[1]
    if q_len <= 0 or kv_len <= 0:
        raise ValueError("q_len and kv_len must be positive")
    dev = _lib.require_cuda(q, k, v, k_coarse, v_coarse)
    _lib.raise_if_failed(dev)

    p = _lib.HsaParams()
    p.B, p.H, p.D, p.Lq, p.Lkv = bsz, heads, head_dim, q_len, kv_len
    p.block_size = int(block_size)
    p.tau_min, p.tau_max = float(tau_min), float(tau_max)
    p.flags = _lib.WA_HSA_FORCE_GENERIC if force_generic else 0
    p.status_mirror = _lib.status_word(dev).data_ptr()
    q, k, v = _unit_last(q), _unit_last(k), _unit_last(v.to(k.dtype))
    keep = [q, k, v]
    p.q, p.k, p.v = _lib.t4_blhd(q), _lib.t4_blhd(k), _lib.t4_blhd(v)
    if k_pooled_cache is not None:
        n_blocks = -(-kv_len // int(block_size))
        if (k_pooled_cache.dtype != torch.float32 or tuple(k_pooled_cache.shape) != (bsz, heads, n_blocks, head_dim)
                or not k_pooled_cache.is_contiguous() or k_pooled_cache.device != dev):
            raise ValueError(f"expected k_pooled_cache: contiguous float32 [{bsz}, {heads}, {n_blocks}, {head_dim}] on {dev}")
        if not 0 <= int(k_pooled_valid) <= n_blocks:
            raise ValueError(f"k_pooled_valid must be in [0, {n_blocks}], got {k_pooled_valid}")
        p.k_pooled, p.k_pooled_valid = k_pooled_cache.data_ptr(), int(k_pooled_valid)
        keep.append(k_pooled_cache)

    if k_coarse is not None:
        if k_coarse.shape[0] != bsz or tuple(k_coarse.shape[2:]) != (heads, head_dim):
            raise ValueError(
                f"expected k_coarse shaped [B, Lc, {heads}, {head_dim}], got {tuple(k_coarse.shape)}"
            )
        if v_coarse.shape != k_coarse.shape:
            raise ValueError("v_coarse must have the same shape as k_coarse")
        k_coarse, v_coarse = _unit_last(k_coarse.to(v_coarse.dtype)), _unit_last(v_coarse)
        p.Lc = k_coarse.shape[1]
        p.k_coarse, p.v_coarse = _lib.t4_blhd(k_coarse), _lib.t4_blhd(v_coarse)
        keep += [k_coarse, v_coarse]
    else:
        if k_proj_mat.shape != v_proj_mat.shape:
            raise ValueError(
                "k_proj_mat and v_proj_mat must have the same shape, got "
                f"{tuple(k_proj_mat.shape)} and {tuple(v_proj_mat.shape)}"
            )
        seg = proj_segment_len if proj_segment_len > 0 else kv_len
        if min(seg, kv_len) > k_proj_mat.shape[1]:
            raise ValueError(
                f"segment length {min(seg, kv_len)} exceeds projection length {k_proj_mat.shape[1]}; "
                "increase proj_segment_len"
            )
        pk = k_proj_mat.detach().to(device=dev).contiguous()
        pv = v_proj_mat.detach().to(device=dev, dtype=pk.dtype).contiguous()
        keep += [pk, pv]
        p.Lc = 0
        p.proj_segment_len, p.proj_rank, p.proj_cols = int(seg), pk.shape[0], pk.shape[1]
        p.proj_dtype = _lib.dtype_code(pk.dtype)
        p.k_proj, p.v_proj = pk.data_ptr(), pv.data_ptr()

    if gate_lin is not None:
        gw = gate_lin.weight.detach().to(device=dev).contiguous()
        gb = gate_lin.bias.detach().to(device=dev, dtype=gw.dtype).contiguous() if gate_lin.bias is not None else None
        keep += [gw, gb]
        p.gate_dtype = _lib.dtype_code(gw.dtype)
        p.gate_w, p.gate_b = gw.data_ptr(), _lib.ptr(gb)

    if topk_per_head is not None:
        topk = topk_per_head.to(device=dev, dtype=torch.int32).contiguous()
        if topk.numel() != heads:
            raise ValueError(f"topk_per_head must have {heads} entries")
        keep.append(topk)
        p.topk_per_head = topk.data_ptr()

    out = torch.empty((bsz, q_len, heads, head_dim), device=dev, dtype=q.dtype)
    p.out = _lib.t4_blhd(out)

    routing = None
    if return_routing:
        nq, nkv = math.ceil(q_len / block_size), math.ceil(kv_len / block_size)
        index = torch.empty((bsz, heads, nq, nkv), device=dev, dtype=torch.int32)
        num = torch.empty((bsz, heads, nq), device=dev, dtype=torch.int32)
        thresholds = torch.empty((heads,), device=dev, dtype=torch.float32)
        p.index_out, p.num_out, p.thresholds_out = index.data_ptr(), num.data_ptr(), thresholds.data_ptr()
        routing = (index, num, thresholds)

    lib = _lib.lib()
    need = lib.wa_hsa_workspace_bytes(ctypes.byref(p))
    ws = _workspace(dev, need)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    used = ctypes.c_int(0)
    with _lib.device_guard(dev):
        _lib.check(lib.wa_hsa_forward(ctypes.byref(p), ctypes.byref(used), _lib.stream_ptr(dev)))
    if check_status and used.value:
        status = ctypes.c_int(0)
        _lib.check(lib.wa_hsa_status(ctypes.byref(p), ctypes.byref(status), _lib.stream_ptr(dev)))
        if status.value:
            _lib.status_word(dev).zero_()
            raise RuntimeError(f"tcgen05 HSA kernel gave up at wait site {status.value}; its output is invalid")

    if distill.distill_enabled() and torch.is_grad_enabled():
        distill.record_against_dense(out, q, k, v)
    if return_routing:
        return out, (*routing, bool(used.value))
    return out


class HSAAttention(nn.Module):
    """Hybrid Sparse Attention over a KV window (reference: attention.py:262-380).

    Owns the trained parameters under the reference's names: `k_proj_mat`, `v_proj_mat` (bf16
    `[ceil(seg / block), seg]`) and `gate_lin` (`Linear(head_dim, head_dim)`), all allocated as
    zeros.  `block_size` may be 64 (the reference's only value) or 128.
    """

    def __init__(self, num_heads: int, head_dim: int, block_size: int = 64, tau_min: float = 0.35,
                 tau_max: float = 1.0, proj_segment_len: int = 1560, backend: str = "auto"):
        super().__init__()
        if block_size not in SUPPORTED_BLOCK_SIZES:
            raise ValueError(f"the sparse-branch kernels are specialized for block_size in {SUPPORTED_BLOCK_SIZES}")
        if proj_segment_len <= 0:
            raise ValueError(f"proj_segment_len must be positive, got {proj_segment_len}")
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.block_size = block_size
        self.tau_min = tau_min
        self.tau_max = tau_max
        self.proj_segment_len = proj_segment_len
        self.proj_rank = math.ceil(proj_segment_len / block_size)
        self.backend = backend
        self.topk_per_head = None   # optional int32 [H]: fixed per-head block count

        self.k_proj_mat = nn.Parameter(torch.zeros((self.proj_rank, proj_segment_len), dtype=torch.bfloat16))
        self.v_proj_mat = nn.Parameter(torch.zeros((self.proj_rank, proj_segment_len), dtype=torch.bfloat16))
        self.gate_lin = nn.Linear(head_dim, head_dim, bias=True)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Return every HSA parameter to its zero placeholder (attention.py:318-329)."""
        with torch.no_grad():
            self.k_proj_mat.zero_()
            self.v_proj_mat.zero_()
            self.gate_lin.weight.zero_()
            self.gate_lin.bias.zero_()

    def coarse_cache_size(self, kv_cache_size: int) -> int:
        """Compressed slots needed to mirror a token cache of `kv_cache_size` (attention.py:331-335)."""
        if kv_cache_size <= 0:
            return 0
        return math.ceil(kv_cache_size / self.proj_segment_len) * self.proj_rank

    def token_range_to_coarse(self, start_index: int, end_index: int) -> tuple[int, int]:
        """Map a segment-aligned token range onto compressed-cache slots (attention.py:337-347)."""
        if start_index % self.proj_segment_len != 0 or end_index % self.proj_segment_len != 0:
            raise ValueError(
                "coarse-cache access requires segment-aligned token indices, got "
                f"start={start_index}, end={end_index}, proj_segment_len={self.proj_segment_len}"
            )
        return ((start_index // self.proj_segment_len) * self.proj_rank,
                (end_index // self.proj_segment_len) * self.proj_rank)

    def compress_kv_cache(self, k: torch.Tensor, v: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Compress `[B, L, H, D]` keys and values for the compressed cache (attention.py:349-361)."""
        if k.shape != v.shape:
            raise ValueError(f"k and v must match, got {tuple(k.shape)} and {tuple(v.shape)}")
        if k.ndim != 4:
            raise ValueError(f"expected [B, L, H, D] tensors, got ndim={k.ndim}")
        return _compress_blhd(k, v, segment_len=self.proj_segment_len, k_proj_mat=self.k_proj_mat,
                              v_proj_mat=self.v_proj_mat, block_size=self.block_size)

    def append_kv(self, k_new, v_new, k_cache, v_cache, k_coarse, v_coarse, *, position: int) -> None:
        """Write new token rows into the layer's K/V cache and their compressed slots into the coarse cache, fused
        (see `append_kv`; the reference does this in three steps, causal_model.py:294-327, 395-413)."""
        append_kv(k_new, v_new, k_cache, v_cache, k_coarse, v_coarse, position=position, segment_len=self.proj_segment_len,
                  k_proj_mat=self.k_proj_mat, v_proj_mat=self.v_proj_mat, block_size=self.block_size)

    def forward(self, q, k, v, k_coarse=None, v_coarse=None):
        return hsa_attention(
            q, k, v, k_coarse=k_coarse, v_coarse=v_coarse,
            k_proj_mat=self.k_proj_mat, v_proj_mat=self.v_proj_mat, gate_lin=self.gate_lin,
            block_size=self.block_size, tau_min=self.tau_min, tau_max=self.tau_max,
            proj_segment_len=self.proj_segment_len, backend=self.backend,
            topk_per_head=self.topk_per_head,
        )
