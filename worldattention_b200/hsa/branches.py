"""Branch-level entry points on `[B, L, H, D]` tensors, used by the sharded (multi-GPU) path.

Each function is one C-ABI call; outputs that feed a log-sum-exp merge come with their natural-log
row normalisers.
"""
from __future__ import annotations

import torch

from .. import _lib

__all__ = ["sparse_branch", "linear_branch", "gate_combine", "merge_partials"]


def sparse_branch(q, k, v, index, num, block_size: int, *, kv_len: int | None = None, lse: bool = True,
                  round_output_bf16: bool = False):
    """Block-sparse softmax branch (reference: block_sparse_torch.py:16-64) with bf16-rounded inputs.

    Returns `(out float32 [B, Lq, H, D], lse float32 [B, H, Lq] or None)`.
    """
    dev = _lib.require_cuda(q, k, v, index, num)
    bsz, q_len, heads, head_dim = q.shape
    kv_len = k.shape[1] if kv_len is None else kv_len
    out = torch.empty((bsz, q_len, heads, head_dim), device=dev, dtype=torch.float32)
    row_lse = torch.empty((bsz, heads, q_len), device=dev, dtype=torch.float32) if lse else None
    index = index.to(torch.int32).contiguous()
    num = num.to(torch.int32).contiguous()
    _lib.check(_lib.lib().wa_block_sparse_forward(
        _lib.t4_blhd(q), _lib.t4_blhd(k), _lib.t4_blhd(v), _lib.t4_blhd(out), bsz, heads, q_len, kv_len, head_dim,
        block_size, index.data_ptr(), num.data_ptr(), index.shape[-1], None, 1, int(round_output_bf16), _lib.ptr(row_lse),
        _lib.stream_ptr(dev)))
    return out, row_lse


def linear_branch(q, k_coarse, v_coarse, *, lse: bool = True):
    """Compressed-slot softmax branch (reference: attention.py:113-118) on `[B, L, H, D]` tensors."""
    dev = _lib.require_cuda(q, k_coarse, v_coarse)
    bsz, q_len, heads, head_dim = q.shape
    out = torch.empty((bsz, q_len, heads, head_dim), device=dev, dtype=torch.float32)
    row_lse = torch.empty((bsz, heads, q_len), device=dev, dtype=torch.float32) if lse else None
    _lib.check(_lib.lib().wa_linear_branch(
        _lib.t4_blhd(q), _lib.t4_blhd(k_coarse), _lib.t4_blhd(v_coarse), _lib.t4_blhd(out), bsz, heads, q_len,
        k_coarse.shape[1], head_dim, 0, _lib.ptr(row_lse), _lib.stream_ptr(dev)))
    return out, row_lse


def gate_combine(q, sparse, linear, gate_lin, *, round_bf16: bool):
    """`sparse + linear * sigmoid(gate_lin(q))` in q's dtype (reference: attention.py:246-259)."""
    dev = _lib.require_cuda(q, sparse, linear)
    bsz, q_len, heads, head_dim = q.shape
    out = torch.empty((bsz, q_len, heads, head_dim), device=dev, dtype=q.dtype)
    gw = gb = None
    gdt = 0
    if gate_lin is not None:
        gw = gate_lin.weight.detach().to(device=dev).contiguous()
        gb = gate_lin.bias.detach().to(device=dev, dtype=gw.dtype).contiguous() if gate_lin.bias is not None else None
        gdt = _lib.dtype_code(gw.dtype)
    _lib.check(_lib.lib().wa_gate_combine(
        _lib.t4_blhd(q), _lib.t4_blhd(sparse), _lib.t4_blhd(linear), _lib.t4_blhd(out), bsz, q_len, heads, head_dim,
        _lib.ptr(gw), _lib.ptr(gb), gdt, int(round_bf16), _lib.stream_ptr(dev)))
    return out


def merge_partials(outs: torch.Tensor, lses: torch.Tensor):
    """Combine `G` shard partials of one branch: `outs [G, rows, D]`, `lses [G, rows]` (natural log)."""
    dev = _lib.require_cuda(outs, lses)
    g, rows, d = outs.shape
    outs = outs.float().contiguous()
    lses = lses.float().contiguous()
    out = torch.empty((rows, d), device=dev, dtype=torch.float32)
    lse = torch.empty((rows,), device=dev, dtype=torch.float32)
    _lib.check(_lib.lib().wa_merge_partials(outs.data_ptr(), lses.data_ptr(), g, rows, d, out.data_ptr(),
                                            lse.data_ptr(), _lib.stream_ptr(dev)))
    return out, lse
