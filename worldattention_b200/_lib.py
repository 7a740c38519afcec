"""ctypes binding of libwa_b200.so (the C ABI declared in include/worldattention_b200.h).

There is no fallback: if the library is missing or a tensor is not on a CUDA device the call
fails with an explicit error.  Build the library with `python -m worldattention_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("WORLDATTENTION_B200_LIB") or os.path.join(_HERE, "libwa_b200.so")

WA_F32, WA_BF16 = 0, 1
WA_ERR_ARG, WA_ERR_UNSUPPORTED, WA_ERR_WORKSPACE, WA_ERR_ALIGN, WA_ERR_DEVICE = -1, -2, -3, -4, -5
WA_HSA_FORCE_GENERIC, WA_HSA_REQUIRE_TUNED = 1, 2


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("reserved", C.c_int32),
                ("stride_b", C.c_int64), ("stride_l", C.c_int64), ("stride_h", C.c_int64)]


class HsaParams(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("D", C.c_int32), ("Lq", C.c_int32), ("Lkv", C.c_int32),
        ("Lc", C.c_int32), ("block_size", C.c_int32), ("proj_segment_len", C.c_int32),
        ("proj_rank", C.c_int32), ("proj_cols", C.c_int32), ("proj_dtype", C.c_int32),
        ("gate_dtype", C.c_int32), ("flags", C.c_int32), ("reserved", C.c_int32),
        ("tau_min", C.c_double), ("tau_max", C.c_double),
        ("q", Tensor4), ("k", Tensor4), ("v", Tensor4), ("k_coarse", Tensor4), ("v_coarse", Tensor4),
        ("out", Tensor4),
        ("k_proj", C.c_void_p), ("v_proj", C.c_void_p), ("gate_w", C.c_void_p), ("gate_b", C.c_void_p),
        ("topk_per_head", C.c_void_p), ("index_out", C.c_void_p), ("num_out", C.c_void_p),
        ("thresholds_out", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("index_in", C.c_void_p), ("num_in", C.c_void_p), ("part_sparse", C.c_void_p), ("part_linear", C.c_void_p),
        ("lse_sparse", C.c_void_p), ("lse_linear", C.c_void_p),
        ("k_pooled", C.c_void_p), ("k_pooled_valid", C.c_int32), ("reserved2", C.c_int32),
        ("status_mirror", C.c_void_p),
        ("part_stride", C.c_int64), ("lse_stride_token", C.c_int64), ("lse_stride_head", C.c_int64),
        ("peer_rows", C.c_int32), ("peer_self", C.c_int32), ("peer_delta", C.c_int64 * 8),
    ]


class PageCopy(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("src_stride", C.c_int64),
                ("dst_stride", C.c_int64), ("n_tokens", C.c_int32), ("rot", C.c_int32)]


_T4P = C.POINTER(Tensor4)
_vp, _i, _f, _d, _i64 = C.c_void_p, C.c_int, C.c_float, C.c_double, C.c_int64

# name -> argtypes (restype is int unless listed in _RESTYPES)
SIGNATURES = {
    "wa_abi_version": [],
    "wa_last_error": [],
    "wa_hsa_params_size": [],
    "wa_launch_count": [],
    "wa_profile_enable": [_i],
    "wa_profile_attention_ms": [C.POINTER(C.c_float)],
    "wa_pool_blocks": [_T4P, _i, _i, _i, _i, _i, _vp, _vp],
    "wa_route_scores": [_vp, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "wa_route_select": [_vp, _i, _i, _i, _i, _d, _d, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "wa_route_select_static": [_vp, _i, _i, _i, _i, _d, _d, _vp, _vp, _vp, _vp, _vp, _vp],
    "wa_map_to_index": [_vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "wa_route_local_selection": [_vp, _vp, C.c_longlong, _i, _i, _i, _vp, _vp, _vp],
    "wa_route_local_candidates": [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "wa_route_merge_candidates": [_vp, _i, _i, _i, _i, _i, _vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "wa_block_sparse_forward": [_T4P, _T4P, _T4P, _T4P, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i, _i,
                                _vp, _vp],
    "wa_compress_kv": [_T4P, _T4P, _T4P, _T4P, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _vp],
    "wa_kv_append_workspace_bytes": [_i, _i, _i, _i, _i, _i, _i],
    "wa_kv_append_compress": [_T4P, _T4P, _T4P, _T4P, _T4P, _T4P, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _i, _vp,
                              C.c_size_t, _vp],
    "wa_compress_status": [C.POINTER(C.c_int)],
    "wa_linear_branch": [_T4P, _T4P, _T4P, _T4P, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "wa_gate_combine": [_T4P, _T4P, _T4P, _T4P, _i, _i, _i, _i, _vp, _vp, _i, _i, _vp],
    "wa_merge_partials": [_vp, _vp, _i, _i64, _i, _vp, _vp, _vp],
    "wa_merge_packed": [_vp, _i, _i64, _i, _i, _vp, _vp, _vp],
    "wa_hsa_workspace_bytes": [C.POINTER(HsaParams)],
    "wa_hsa_forward": [C.POINTER(HsaParams), C.POINTER(C.c_int), _vp],
    "wa_hsa_status": [C.POINTER(HsaParams), C.POINTER(C.c_int), _vp],
    "wa_ln_modulate": [_vp, _vp, _i64, _i, _f, _vp, _vp, _vp, _vp, _i64, _i, _vp],
    "wa_gated_residual": [_vp, _vp, _vp, _i64, _i, _vp, _i64, _i, _vp],
    "wa_qk_norm_rope": [_T4P, _T4P, _i, _i, _i, _i, _vp, _i, _f, _vp, _i, _i, _i, _i, _vp],
    "wa_qk_norm_rope_at": [_T4P, _T4P, _i, _i, _i, _i, _vp, _i, _f, _vp, _i, _vp, _i, _i, _vp],
    "wa_hkv_page_centroids": [_T4P, _i, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp, _vp],
    "wa_hkv_score_topk": [_vp, _vp, _i, _i, _i, _f, _i, _vp, _vp, _vp, _vp],
    "wa_hkv_score_topk_layers": [_vp, _vp, _i, _i, _i, _i, C.c_longlong, _f, _i, _vp, _vp, _vp, _vp],
    "wa_hkv_build_records": [_vp, _i, _i, _i, _vp, _i, C.c_longlong, C.c_longlong, _vp, C.c_longlong, C.c_longlong,
                             _i, _i, _i, _i, _vp, _vp, _vp],
    "wa_hkv_promote_pages": [_vp, _i, _i, _i, _vp],
    "wa_hkv_gather_pages": [_vp, _i, _i, _i, _i, _i, _vp, _i, _vp],
}
_RESTYPES = {"wa_last_error": C.c_char_p, "wa_hsa_workspace_bytes": C.c_size_t, "wa_hsa_params_size": C.c_size_t, "wa_kv_append_workspace_bytes": C.c_size_t,
             "wa_launch_count": C.c_ulonglong}

_lib: Optional[C.CDLL] = None


def lib() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library has not been built "
                "(run `python -m worldattention_b200.build`). There is no CPU or PyTorch fallback."
            )
        handle = C.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)
        if handle.wa_abi_version() != 3 or handle.wa_hsa_params_size() != C.sizeof(HsaParams):
            raise RuntimeError("libwa_b200.so ABI mismatch (version or wa_hsa_params layout); rebuild the library")
        _lib = handle
    return _lib


def check(rc: int) -> None:
    """Turn a C-ABI status into the exception type the reference raises for that failure."""
    if rc == 0:
        return
    msg = lib().wa_last_error().decode("utf-8", "replace")
    if rc in (WA_ERR_ARG, WA_ERR_ALIGN, WA_ERR_WORKSPACE):
        raise ValueError(msg)
    if rc == WA_ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"CUDA error {rc}: {msg}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return WA_F32
    if dtype == torch.bfloat16:
        return WA_BF16
    raise ValueError(f"worldattention_b200 kernels take float32 or bfloat16 tensors, got {dtype}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "worldattention_b200 runs on CUDA tensors only (there is no CPU path); "
                f"got a tensor on {t.device}"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors live on different devices: {dev} and {t.device}")
    return dev


_status_words: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The page-locked int32 that the tcgen05 kernel writes its failure code to on `device` (one per device)."""
    key = torch.device(device).index or 0
    word = _status_words.get(key)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device="cpu").pin_memory()
        _status_words[key] = word
    return word


def raise_if_failed(device: torch.device) -> None:
    """Raise if an earlier launch of an HSA forward on `device` gave up at a bounded wait (its output is invalid).

    Reads host memory only: no copy, no synchronisation.  A failure of a launch that is still in flight shows
    at the next call or at the caller's next synchronisation point followed by this check.
    """
    word = _status_words.get(torch.device(device).index or 0)
    if word is not None and int(word[0]) != 0:
        code = int(word[0])
        word.zero_()
        kernel = "block-pooling (TMA stream)" if code in (201, 202) else "tcgen05 attention"
        raise RuntimeError(f"an earlier {kernel} launch of an HSA forward on {device} gave up at wait site {code}; "
                           "its output is invalid")


def device_guard(device: torch.device):
    """Make `device` the current CUDA device for the calls inside (function set-up and launches act on the current one)."""
    return torch.cuda.device(device)


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def t4_blhd(t: torch.Tensor) -> Tensor4:
    """View a `[B, L, H, D]` tensor (any strides, unit last stride)."""
    if t.stride(3) != 1:
        t = t.contiguous()
    return _keep(Tensor4(t.data_ptr(), dtype_code(t.dtype), 0, t.stride(0), t.stride(1), t.stride(2)), t)


def t4_bhnd(t: torch.Tensor) -> Tensor4:
    """View a `[B, H, N, D]` tensor as the ABI's `[B, L, H, D]` descriptor."""
    if t.stride(3) != 1:
        t = t.contiguous()
    return _keep(Tensor4(t.data_ptr(), dtype_code(t.dtype), 0, t.stride(0), t.stride(2), t.stride(1)), t)


def _keep(desc: Tensor4, owner: torch.Tensor) -> Tensor4:
    desc._owner = owner          # keep a possibly re-laid-out tensor alive for the call
    return desc


def null_t4() -> Tensor4:
    return Tensor4(None, 0, 0, 0, 0, 0)
