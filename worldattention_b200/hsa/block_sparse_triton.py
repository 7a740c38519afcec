"""Inference entry points of the reference's Triton backend, served by the CUDA library.

`block_sparse_attention(q, k, v, *, block_sizes, q2k_index, q2k_num, block_map)` and
`map_to_index(block_map)` keep the signatures of wan/modules/hsa/block_sparse_triton.py:44-57,
371-382.  No Triton is involved: the module name is kept only so that code importing the
reference's backend module keeps working.  Forward only (the backward kernels are training code).
"""
from __future__ import annotations

import torch

from .. import _lib
from .block_sparse_torch import block_sparse_attention_reference

__all__ = ["block_sparse_attention", "map_to_index"]


def map_to_index(block_map: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Boolean `[B, H, Nq, Nkv]` selection mask -> (ascending index padded with -1, count)."""
    dev = _lib.require_cuda(block_map)
    bsz, heads, nq, nkv = block_map.shape
    mask = block_map.to(torch.bool).contiguous()
    index = torch.empty(mask.shape, dtype=torch.int32, device=dev)
    num = torch.empty((bsz, heads, nq), dtype=torch.int32, device=dev)
    _lib.check(_lib.lib().wa_map_to_index(mask.data_ptr(), bsz, heads, nq, nkv, index.data_ptr(),
                                          num.data_ptr(), _lib.stream_ptr(dev)))
    return index, num


def block_sparse_attention(q, k, v, *, block_sizes, q2k_index=None, q2k_num=None, block_map=None):
    """Block-sparse attention over `[B, H, N, D]` tensors padded to the block size.

    The block size is `N_kv / len(block_sizes)`.  Pass `(q2k_index, q2k_num)`, or a `block_map`
    that is converted with `map_to_index`.
    """
    if block_map is not None:
        q2k_index, q2k_num = map_to_index(block_map)
    if q2k_index is None or q2k_num is None:
        raise ValueError("provide either block_map or both q2k_index and q2k_num")
    block_size = k.shape[2] // block_sizes.shape[0]
    return block_sparse_attention_reference(q, k, v, q2k_index, q2k_num, block_sizes, block_size)
