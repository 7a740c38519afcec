"""Vectorised construction of page-copy records and the one-launch page install.

`HKVCache.apply` builds a handful of records per call; retrieval at scale (per-head top-k over many
layers) builds thousands, so the records are assembled as one numpy structured array whose layout
is `wa_page_copy` (include/worldattention_b200.h) and shipped to the device in a single copy.
Stands in for the copy loop of the reference's `HKVCache.apply` (pipeline/hkv/cache.py:229-246).
"""
from __future__ import annotations

import numpy as np
import torch

from .. import _lib

__all__ = ["RECORD_DTYPE", "per_head_records", "gather_pages"]

RECORD_DTYPE = np.dtype([("src", "<u8"), ("dst", "<u8"), ("src_stride", "<i8"), ("dst_stride", "<i8"),
                         ("n_tokens", "<i4"), ("rot", "<i4")])
assert RECORD_DTYPE.itemsize == 40


def per_head_records(page_ids: np.ndarray, *, src_base: int, src_page_stride: int, src_layer_stride: int,
                     dst_base: int, dst_layer_stride: int, page_tokens: int, heads: int, head_dim: int,
                     elem_size: int, rot: np.ndarray | None) -> np.ndarray:
    """Records that copy, for every (layer, head), its selected pages into consecutive cache slots.

    `page_ids` is `[layers, heads, k]` (slot of each selected page inside the source pool, in
    installation order).  Source pool layout `[layers, pages, page_tokens, heads, head_dim]`,
    destination `[layers, capacity, heads, head_dim]`; all offsets and strides are byte counts
    given by the caller (`*_stride`) and turned into element strides of one head row here.
    `rot` (`[layers, heads, k]` int32 or None) selects the rotation of each copy.
    """
    layers, h, k = page_ids.shape
    assert h == heads
    rec = np.zeros((layers, heads, k), dtype=RECORD_DTYPE)
    layer = np.arange(layers, dtype=np.int64)[:, None, None]
    head = np.arange(heads, dtype=np.int64)[None, :, None]
    slot = np.arange(k, dtype=np.int64)[None, None, :]
    row_bytes = heads * head_dim * elem_size
    rec["src"] = (src_base + layer * src_layer_stride + page_ids.astype(np.int64) * src_page_stride
                  + head * head_dim * elem_size).astype(np.uint64)
    rec["dst"] = (dst_base + layer * dst_layer_stride + slot * page_tokens * row_bytes
                  + head * head_dim * elem_size).astype(np.uint64)
    rec["src_stride"] = heads * head_dim
    rec["dst_stride"] = heads * head_dim
    rec["n_tokens"] = page_tokens
    rec["rot"] = -1 if rot is None else rot.astype(np.int32)
    return rec.reshape(-1)


def build_records_device(top_ids: torch.Tensor, page_src: torch.Tensor, *, src_layer_stride: int, src_token_stride: int,
                         dst: torch.Tensor, dst_layer_stride: int, dst_token_stride: int, page_tokens: int,
                         head_dim: int, rotate: bool, missing: torch.Tensor | None = None) -> torch.Tensor:
    """Copy records for a per-head retrieval, built on the device from the device-resident top-k ids.

    `top_ids` int32 `[layers, heads, k]` (as `score_and_topk_layers` returns them), `page_src` int64 `[P]` device
    addresses of the pages' first tokens (layer 0, head 0; 0 = not resident).  Per (layer, head) the pages are
    installed in ascending id (chronological) order into consecutive `page_tokens`-row slots of `dst`
    (`[layers, capacity, heads, head_dim]`-like, strides given).  Returns the records as a uint8 device tensor
    for `gather_pages(..., records_dev=...)`; nothing crosses to the host.
    """
    dev = _lib.require_cuda(top_ids, page_src, dst)
    layers, heads, k = top_ids.shape
    ids = top_ids.to(torch.int32).contiguous()
    src = page_src.to(torch.int64).contiguous()
    records = torch.empty((layers * heads * k * RECORD_DTYPE.itemsize,), dtype=torch.uint8, device=dev)
    _lib.check(_lib.lib().wa_hkv_build_records(
        ids.data_ptr(), layers, heads, k, src.data_ptr(), src.shape[0], int(src_layer_stride), int(src_token_stride),
        dst.data_ptr(), int(dst_layer_stride), int(dst_token_stride), int(page_tokens), int(head_dim), dst.element_size(),
        1 if rotate else 0, records.data_ptr(), _lib.ptr(missing), _lib.stream_ptr(dev)))
    return records


def gather_records_device(records_dev: torch.Tensor, *, max_tokens: int, row_elems: int, head_dim: int, dtype: torch.dtype,
                          rotations: torch.Tensor | None = None, n_temporal: int = 0) -> None:
    """Run the page-copy kernel over records that already live on the device (`build_records_device`)."""
    n = records_dev.numel() // RECORD_DTYPE.itemsize
    lib = _lib.lib()
    base = records_dev.data_ptr()
    for start in range(0, n, 65535):
        count = min(65535, n - start)
        _lib.check(lib.wa_hkv_gather_pages(base + start * RECORD_DTYPE.itemsize, count, max_tokens, row_elems, head_dim,
                                           _lib.dtype_code(dtype), _lib.ptr(rotations), n_temporal,
                                           _lib.stream_ptr(records_dev.device)))


def gather_pages(records: np.ndarray, *, max_tokens: int, row_elems: int, head_dim: int, dtype: torch.dtype,
                 device: torch.device, rotations: torch.Tensor | None = None, n_temporal: int = 0,
                 records_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Ship `records` to the device (unless `records_dev` is given) and run the page-copy kernel once.

    At most 65535 records per launch; longer lists are split.  Returns the device copy of the records.
    """
    if records_dev is None:
        host = torch.from_numpy(records.view(np.uint8).reshape(-1))
        records_dev = host.to(device, non_blocking=True)
    n = records.shape[0]
    lib = _lib.lib()
    base = records_dev.data_ptr()
    for start in range(0, n, 65535):
        count = min(65535, n - start)
        _lib.check(lib.wa_hkv_gather_pages(base + start * RECORD_DTYPE.itemsize, count, max_tokens, row_elems, head_dim,
                                           _lib.dtype_code(dtype), _lib.ptr(rotations), n_temporal,
                                           _lib.stream_ptr(device)))
    return records_dev
