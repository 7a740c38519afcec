"""Branch-level entry points on `[B, L, H, D]` tensors, used by the sharded (multi-GPU) path.

Each function is one C-ABI call; outputs that feed a log-sum-exp merge come with their natural-log
row normalisers.
"""
from __future__ import annotations

import torch

from .. import _lib

__all__ = ["sparse_branch", "linear_branch", "gate_combine", "merge_partials", "hsa_partials", "hsa_partials_packed",
           "merge_packed", "record_floats"]


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


def gate_combine(q, sparse, linear, gate_lin, *, round_bf16: bool, out: torch.Tensor | None = None):
    """`sparse + linear * sigmoid(gate_lin(q))` in q's dtype (reference: attention.py:246-259); `out` may be supplied."""
    dev = _lib.require_cuda(q, sparse, linear)
    bsz, q_len, heads, head_dim = q.shape
    if out is None:
        out = torch.empty((bsz, q_len, heads, head_dim), device=dev, dtype=q.dtype)
    elif tuple(out.shape) != (bsz, q_len, heads, head_dim) or out.dtype != q.dtype or out.stride(3) != 1:
        raise ValueError("out must be [B, L, H, D] in q's dtype with a contiguous last axis")
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


def hsa_partials(q, k, v, k_coarse, v_coarse, index, num, block_size: int, *, force_generic: bool = False):
    """Both branches over one key shard, in one `wa_hsa_forward` call with the routing supplied.

    `index` / `num` are the routing restricted to this shard (`sharded.local_selection`).  Returns
    `(sparse, lse_sparse, linear, lse_linear, used_tuned)`: float32 `[B, Lq, H, D]` normalised branch
    outputs and `[B, H, Lq]` natural-log normalisers, ready for `merge_partials`.  The tcgen05 kernel
    runs when the shape qualifies (bf16, head_dim 128, 128-token blocks), the SIMT kernels otherwise.
    """
    import ctypes
    from .attention import _unit_last, _workspace
    dev = _lib.require_cuda(q, k, v, k_coarse, v_coarse, index, num)
    _lib.raise_if_failed(dev)
    bsz, q_len, heads, head_dim = q.shape
    p = _lib.HsaParams()
    p.B, p.H, p.D, p.Lq, p.Lkv, p.Lc = bsz, heads, head_dim, q_len, k.shape[1], k_coarse.shape[1]
    p.block_size = int(block_size)
    p.flags = _lib.WA_HSA_FORCE_GENERIC if force_generic else 0
    p.status_mirror = _lib.status_word(dev).data_ptr()
    q, k, v = _unit_last(q), _unit_last(k), _unit_last(v.to(k.dtype))
    k_coarse, v_coarse = _unit_last(k_coarse.to(v_coarse.dtype)), _unit_last(v_coarse)
    p.q, p.k, p.v = _lib.t4_blhd(q), _lib.t4_blhd(k), _lib.t4_blhd(v)
    p.k_coarse, p.v_coarse = _lib.t4_blhd(k_coarse), _lib.t4_blhd(v_coarse)
    index = index.to(torch.int32).contiguous()
    num = num.to(torch.int32).contiguous()
    if index.shape[-1] != -(-k.shape[1] // block_size):
        raise ValueError("index rows must span exactly this shard's key blocks")
    p.index_in, p.num_in = index.data_ptr(), num.data_ptr()
    sparse = torch.empty((bsz, q_len, heads, head_dim), device=dev, dtype=torch.float32)
    linear = torch.empty_like(sparse)
    lse_s = torch.empty((bsz, heads, q_len), device=dev, dtype=torch.float32)
    lse_l = torch.empty_like(lse_s)
    p.part_sparse, p.part_linear = sparse.data_ptr(), linear.data_ptr()
    p.lse_sparse, p.lse_linear = lse_s.data_ptr(), lse_l.data_ptr()
    lib = _lib.lib()
    ws = _workspace(dev, lib.wa_hsa_workspace_bytes(ctypes.byref(p)))
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    used = ctypes.c_int(0)
    with _lib.device_guard(dev):
        _lib.check(lib.wa_hsa_forward(ctypes.byref(p), ctypes.byref(used), _lib.stream_ptr(dev)))
    return sparse, lse_s, linear, lse_l, bool(used.value)


def record_floats(head_dim: int) -> int:
    """Floats in one packed partial record of a (token, head): [sparse (D) | linear (D) | lse_sparse, lse_linear, 0, 0]."""
    return 2 * head_dim + 4


def hsa_partials_packed(q, k, v, k_coarse, v_coarse, index, num, block_size: int, records: torch.Tensor, *,
                        peer=None) -> bool:
    """`hsa_partials` writing straight into packed records (`records`: float32 `[B, rows >= Lq, H, 2 D + 4]`, contiguous).

    Both branch outputs and both normalisers of a (token, head) land in one record, so the rows of a query range are
    one contiguous block -- the unit the KV-sharded path sends to the rank that merges those rows.  Only the tcgen05
    kernel writes this layout; returns False (nothing launched) where it does not cover the shape, and the caller packs
    the output of `hsa_partials` itself.

    `peer = (rows_per_rank, this_rank, deltas)`: the records go straight into the buffers of the ranks that merge them
    (`records` is then this rank's receive buffer `[1, ranks * rows_per_rank, H, 2 D + 4]`, `deltas[r]` the distance in
    floats from it to rank r's buffer as mapped into this process): query row t becomes row
    `this_rank * rows_per_rank + t % rows_per_rank` of rank `t // rows_per_rank`.
    """
    import ctypes
    from .attention import _unit_last, _workspace
    dev = _lib.require_cuda(q, k, v, k_coarse, v_coarse, index, num, records)
    _lib.raise_if_failed(dev)
    bsz, q_len, heads, head_dim = q.shape
    rec = record_floats(head_dim)
    if records.dtype != torch.float32 or not records.is_contiguous() or records.dim() != 4 or records.shape[0] != bsz \
            or records.shape[1] < q_len or tuple(records.shape[2:]) != (heads, rec) or (bsz > 1 and records.shape[1] != q_len):
        raise ValueError(f"records must be contiguous float32 [{bsz}, >= {q_len}, {heads}, {rec}]")
    p = _lib.HsaParams()
    p.B, p.H, p.D, p.Lq, p.Lkv, p.Lc = bsz, heads, head_dim, q_len, k.shape[1], k_coarse.shape[1]
    p.block_size = int(block_size)
    p.flags = _lib.WA_HSA_REQUIRE_TUNED
    p.status_mirror = _lib.status_word(dev).data_ptr()
    q, k, v = _unit_last(q), _unit_last(k), _unit_last(v.to(k.dtype))
    k_coarse, v_coarse = _unit_last(k_coarse.to(v_coarse.dtype)), _unit_last(v_coarse)
    p.q, p.k, p.v = _lib.t4_blhd(q), _lib.t4_blhd(k), _lib.t4_blhd(v)
    p.k_coarse, p.v_coarse = _lib.t4_blhd(k_coarse), _lib.t4_blhd(v_coarse)
    index = index.to(torch.int32).contiguous()
    num = num.to(torch.int32).contiguous()
    if index.shape[-1] != -(-k.shape[1] // block_size):
        raise ValueError("index rows must span exactly this shard's key blocks")
    p.index_in, p.num_in = index.data_ptr(), num.data_ptr()
    base = records.data_ptr()
    p.part_sparse, p.part_linear = base, base + 4 * head_dim
    p.lse_sparse, p.lse_linear = base + 8 * head_dim, base + 8 * head_dim + 4
    p.part_stride, p.lse_stride_token, p.lse_stride_head = rec, heads * rec, rec
    if peer is not None:
        rows_per_rank, this_rank, deltas = peer
        if bsz != 1 or len(deltas) > 8 or rows_per_rank * len(deltas) < q_len or records.shape[1] < rows_per_rank * len(deltas):
            raise ValueError("peer stores need B = 1, at most 8 ranks whose rows cover Lq, and a receive buffer of ranks * rows")
        p.peer_rows, p.peer_self = int(rows_per_rank), int(this_rank)
        for r, delta in enumerate(deltas):
            p.peer_delta[r] = int(delta)
    lib = _lib.lib()
    ws = _workspace(dev, lib.wa_hsa_workspace_bytes(ctypes.byref(p)))
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    used = ctypes.c_int(0)
    with _lib.device_guard(dev):
        rc = lib.wa_hsa_forward(ctypes.byref(p), ctypes.byref(used), _lib.stream_ptr(dev))
    if rc == _lib.WA_ERR_UNSUPPORTED:
        return False
    _lib.check(rc)
    return True


def merge_packed(recv: torch.Tensor, head_dim: int):
    """Merge packed shard partials `recv` (float32 `[G, vectors, 2 D + 4]`): returns the sparse branch rounded to bf16
    (as the reference stores it) and the linear branch in float32, both `[vectors, D]`."""
    dev = _lib.require_cuda(recv)
    g, vectors, rec = recv.shape
    recv = recv.float().contiguous()
    sparse = torch.empty((vectors, head_dim), device=dev, dtype=torch.bfloat16)
    linear = torch.empty((vectors, head_dim), device=dev, dtype=torch.float32)
    _lib.check(_lib.lib().wa_merge_packed(recv.data_ptr(), g, vectors, head_dim, rec, sparse.data_ptr(), linear.data_ptr(),
                                          _lib.stream_ptr(dev)))
    return sparse, linear
