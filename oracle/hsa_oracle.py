"""CPU oracle for Hybrid Sparse Attention (HSA) -- TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference algorithm, used as the checker in the test-suite, in the smoke
test and as the timed CPU baseline of the benchmark.  Nothing in the product package imports it.

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own PyTorch functions on
seeded inputs and stores their outputs; `tests/test_oracle_golden.py` checks every function below
against those vectors.

Each function names the reference code it restates (paths relative to the reference project).

Numerical conventions
---------------------
Arrays are float32 numpy arrays.  A tensor whose reference dtype is bfloat16 is carried as float32
values that are exactly representable in bfloat16; `dtype` arguments ("fp32" | "bf16") say which
rounding the reference would apply when it stores a result in "the input dtype".

Routing is a discrete decision taken on float32 numbers, so the order of floating-point additions
matters.  PyTorch's CPU reductions use an unspecified blocked order; the oracle (and the CUDA
kernels, which use the same rule) define every reduction on the routing path as *accumulate in
float64, round once to float32*, and break equal probabilities by the lower block index (the
reference's `torch.sort` leaves that order unspecified).
"""
from __future__ import annotations

import math

import numpy as np

__all__ = [
    "bf16_round", "as_dtype", "block_counts", "pad_to_len", "variable_block_sizes",
    "block_mean_pool", "block_attention_map", "build_block_routing", "fixed_topk_num",
    "block_sparse_attention", "compress_kv", "linear_branch", "gate_values", "hsa_attention",
    "map_to_index", "merge_partials",
]


# --------------------------------------------------------------------------------------------
# dtype helpers
# --------------------------------------------------------------------------------------------

def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even); result stays float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    with np.errstate(over="ignore"):
        r = (u + (((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF))) & np.uint32(0xFFFF0000)
    return r.view(np.float32)


def as_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """Store `x` in the reference dtype: identity for fp32, bfloat16 rounding for bf16."""
    if dtype == "bf16":
        return bf16_round(x)
    if dtype == "fp32":
        return np.asarray(x, dtype=np.float32)
    raise ValueError(f"unknown dtype tag {dtype!r}")


def _f64sum_to_f32(x: np.ndarray, axis) -> np.ndarray:
    return np.sum(x.astype(np.float64), axis=axis).astype(np.float32)


# --------------------------------------------------------------------------------------------
# wan/modules/hsa/routing.py
# --------------------------------------------------------------------------------------------

def block_counts(q_len: int, kv_len: int, block_size: int):
    """routing.py:138-142 -- padded lengths and block counts."""
    q_pad = math.ceil(q_len / block_size) * block_size
    kv_pad = math.ceil(kv_len / block_size) * block_size
    return q_pad, kv_pad, q_pad // block_size, kv_pad // block_size


def pad_to_len(x: np.ndarray, target_len: int) -> np.ndarray:
    """routing.py:129-135 -- zero-pad `[B, L, H, D]` along the token axis."""
    pad = target_len - x.shape[1]
    if pad <= 0:
        return x
    return np.concatenate([x, np.zeros((x.shape[0], pad) + x.shape[2:], dtype=x.dtype)], axis=1)


def variable_block_sizes(kv_len: int, kv_len_padded: int, block_size: int) -> np.ndarray:
    """routing.py:121-126 -- real token count per key block (only the last can be short)."""
    n = kv_len_padded // block_size
    sizes = np.full((n,), block_size, dtype=np.int32)
    sizes[-1] = kv_len - (n - 1) * block_size
    return sizes


def block_mean_pool(x: np.ndarray, logical_len: int, num_blocks: int, block_size: int,
                    dtype: str = "fp32") -> np.ndarray:
    """routing.py:45-61 -- mean over the real tokens of each block of `[B, H, Nb*BS, D]`.

    Aligned length: the mean is returned in the input dtype (`mean(dim=3)`, routing.py:54), so for
    bf16 inputs it is rounded to bf16.  Ragged length: the masked *sum* is taken in the input dtype
    (rounded to bf16 for bf16 inputs) and divided by the float32 block size, and that quotient is
    not rounded again (routing.py:56-61).
    """
    b, h, _, d = x.shape
    blocks = x.reshape(b, h, num_blocks, block_size, d)
    if logical_len % block_size == 0:
        mean = (np.sum(blocks.astype(np.float64), axis=3) / block_size).astype(np.float32)
        return as_dtype(mean, dtype)
    sizes = np.full((num_blocks,), block_size, dtype=np.float32)
    sizes[-1] = logical_len - (num_blocks - 1) * block_size
    valid = np.arange(block_size)[None, :] < sizes.astype(np.int64)[:, None]          # [Nb, BS]
    masked = blocks.astype(np.float64) * valid[None, None, :, :, None]
    pooled = as_dtype(np.sum(masked, axis=3).astype(np.float32), dtype)
    return (pooled / sizes[None, None, :, None]).astype(np.float32)


def block_attention_map(q_pooled: np.ndarray, k_pooled: np.ndarray) -> np.ndarray:
    """routing.py:64-68 -- softmax over pooled `q.k^T / sqrt(D)`, float32 `[B, H, Nq, Nkv]`.

    Every reduction accumulates in float64 and rounds once to float32 (module docstring).
    """
    d = q_pooled.shape[-1]
    scale = np.float32(d ** -0.5)
    logits = np.matmul(q_pooled.astype(np.float64),
                       np.swapaxes(k_pooled.astype(np.float64), -1, -2)).astype(np.float32)
    logits = (logits * scale).astype(np.float32)
    shifted = (logits - np.max(logits, axis=-1, keepdims=True)).astype(np.float32)
    e = np.exp(shifted.astype(np.float64)).astype(np.float32)
    denom = _f64sum_to_f32(e, axis=-1)[..., None]
    return (e / denom).astype(np.float32)


def _stable_descending(block_attn: np.ndarray):
    """Sort rows descending, equal values ordered by ascending index (routing.py:97 + tie rule)."""
    order = np.argsort(-block_attn.astype(np.float32), axis=-1, kind="stable")
    return np.take_along_axis(block_attn, order, axis=-1), order


def build_block_routing(block_attn: np.ndarray, tau_min: float, tau_max: float,
                        return_mask: bool = False):
    """routing.py:71-118 -- Gini-adaptive cumulative-mass selection.

    Returns `(index int32 [B,H,Nq,Nkv], num int32 [B,H,Nq], mask bool or None, thresholds f32 [H])`.
    """
    block_attn = np.asarray(block_attn, dtype=np.float32)
    _, heads, _, nkv = block_attn.shape
    probs, order = _stable_descending(block_attn)

    ranks = np.arange(1, nkv + 1, dtype=np.float32)
    weights = (np.float32(nkv + 1) - np.float32(2.0) * ranks).astype(np.float32)
    terms = (weights * probs).astype(np.float32)                       # float32 products
    gini = (_f64sum_to_f32(terms, axis=-1) / np.float32(nkv)).astype(np.float32)
    head_gini = np.mean(gini.astype(np.float64), axis=(0, 2)).astype(np.float32)
    span = np.float32(tau_max - tau_min)
    thresholds = (np.float32(tau_min) + (head_gini * span).astype(np.float32)).astype(np.float32)

    cumulative = np.cumsum(probs.astype(np.float64), axis=-1).astype(np.float32)
    keep = (cumulative - probs).astype(np.float32) < thresholds.reshape(1, heads, 1, 1)
    num = np.sum(keep, axis=-1).astype(np.int32)
    index = order.astype(np.int32)

    mask = None
    if return_mask:
        mask = np.zeros(block_attn.shape, dtype=bool)
        np.put_along_axis(mask, order, keep, axis=-1)
    return index, num, mask, thresholds


def fixed_topk_num(k_per_head, bsz: int, num_q_blocks: int, num_kv_blocks: int) -> np.ndarray:
    """Fixed per-head top-k expressed through the reference's own (index, num) interface.

    The reference kernels take `q2k_num` (block_sparse_torch.py:56-57); a top-k policy keeps the
    descending `index` of routing.py:97 and sets `num[b, h, i] = min(k_h, Nkv)`.
    """
    k = np.minimum(np.asarray(k_per_head, dtype=np.int64), num_kv_blocks).astype(np.int32)
    return np.broadcast_to(k.reshape(1, -1, 1), (bsz, k.shape[0], num_q_blocks)).copy()


def map_to_index(block_map: np.ndarray):
    """block_sparse_triton.py:20-57 -- bool mask to ascending index list (-1 filled) and count."""
    b, h, nq, nkv = block_map.shape
    index = np.full(block_map.shape, -1, dtype=np.int32)
    num = np.zeros((b, h, nq), dtype=np.int32)
    for bi in range(b):
        for hi in range(h):
            for qi in range(nq):
                ids = np.nonzero(block_map[bi, hi, qi])[0]
                index[bi, hi, qi, : ids.size] = ids
                num[bi, hi, qi] = ids.size
    return index, num


# --------------------------------------------------------------------------------------------
# wan/modules/hsa/block_sparse_torch.py
# --------------------------------------------------------------------------------------------

def block_sparse_attention(q, k, v, q2k_index, q2k_num, block_sizes, block_size: int,
                           dtype: str = "bf16", return_lse: bool = False):
    """block_sparse_torch.py:16-64 -- exact softmax over the selected key blocks.

    `q, k, v` are `[B, H, N, D]` padded to `block_size`; computation is float32; the result is
    stored in the input dtype.  Ids are clamped to `[0, Nkv-1]` (:37), slots `>= num` and tokens
    `>= block_sizes[id]` are masked (:56-60), an empty selection gives exact zeros (:63).
    With `return_lse` also returns the natural-log sum-exp per query row (-inf for empty rows).
    """
    q = np.asarray(q, np.float32); k = np.asarray(k, np.float32); v = np.asarray(v, np.float32)
    b, h, nq_tok, d = q.shape
    nq = nq_tok // block_size
    nkv = k.shape[2] // block_size
    out = np.zeros_like(q)
    lse = np.full((b, h, nq_tok), -np.inf, dtype=np.float32)
    scale = np.float32(1.0 / math.sqrt(d))
    kb = k.reshape(b, h, nkv, block_size, d)
    vb = v.reshape(b, h, nkv, block_size, d)
    tok = np.arange(block_size)
    for bi in range(b):
        for hi in range(h):
            for qi in range(nq):
                n = int(q2k_num[bi, hi, qi])
                if n <= 0:
                    continue
                ids = np.clip(q2k_index[bi, hi, qi, :n].astype(np.int64), 0, max(nkv - 1, 0))
                ks = kb[bi, hi, ids].reshape(n * block_size, d)
                vs = vb[bi, hi, ids].reshape(n * block_size, d)
                valid = (tok[None, :] < block_sizes[ids].astype(np.int64)[:, None]).reshape(-1)
                qs = q[bi, hi, qi * block_size:(qi + 1) * block_size]
                s = (qs @ ks.T) * scale
                s[:, ~valid] = -np.inf
                m = np.max(s, axis=-1, keepdims=True)
                m_safe = np.where(np.isfinite(m), m, 0.0)
                e = np.exp(s - m_safe)
                l = np.sum(e, axis=-1, keepdims=True)
                with np.errstate(invalid="ignore", divide="ignore"):
                    p = np.where(l > 0, e / l, 0.0).astype(np.float32)
                    row_lse = np.where(l[:, 0] > 0, m_safe[:, 0] + np.log(l[:, 0]), -np.inf)
                out[bi, hi, qi * block_size:(qi + 1) * block_size] = p @ vs
                lse[bi, hi, qi * block_size:(qi + 1) * block_size] = row_lse
    out = as_dtype(out, dtype)
    return (out, lse) if return_lse else out


# --------------------------------------------------------------------------------------------
# wan/modules/hsa/attention.py
# --------------------------------------------------------------------------------------------

def compress_kv(k, v, *, segment_len: int, k_proj_mat, v_proj_mat, block_size: int,
                dtype: str = "fp32"):
    """attention.py:64-110 -- per-segment low-rank sequence projection of `[B, H, L, D]`."""
    k_proj_mat = np.asarray(k_proj_mat, np.float32)
    v_proj_mat = np.asarray(v_proj_mat, np.float32)
    if k_proj_mat.shape != v_proj_mat.shape:
        raise ValueError("k_proj_mat and v_proj_mat must have the same shape")
    kv_len = k.shape[2]
    if segment_len <= 0:
        segment_len = kv_len
    outs_k, outs_v = [], []
    for start in range(0, kv_len, segment_len):
        end = min(start + segment_len, kv_len)
        seg = end - start
        if seg > k_proj_mat.shape[1]:
            raise ValueError(f"segment length {seg} exceeds projection length {k_proj_mat.shape[1]}")
        rank = min(k_proj_mat.shape[0], math.ceil(seg / block_size))
        ek = k_proj_mat[:rank, :seg]
        ev = v_proj_mat[:rank, :seg]
        outs_k.append(as_dtype(np.einsum("rt,bhtd->bhrd", ek, k[:, :, start:end], optimize=True), dtype))
        outs_v.append(as_dtype(np.einsum("rt,bhtd->bhrd", ev, v[:, :, start:end], optimize=True), dtype))
    return np.concatenate(outs_k, axis=2), np.concatenate(outs_v, axis=2)


def linear_branch(q, k_coarse, v_coarse, dtype: str = "fp32", return_lse: bool = False):
    """attention.py:113-118 -- softmax attention of `[B,H,Lq,D]` queries over compressed slots.

    Logits and softmax are float32; the weights are cast to the value dtype before `weights @ v`
    and the product is stored in the value dtype (attention.py:118).
    """
    d = q.shape[-1]
    scale = np.float32(d ** -0.5)
    logits = np.matmul(q.astype(np.float32), np.swapaxes(k_coarse, -1, -2).astype(np.float32)) * scale
    m = np.max(logits, axis=-1, keepdims=True)
    e = np.exp(logits - m)
    l = np.sum(e, axis=-1, keepdims=True)
    w = as_dtype((e / l).astype(np.float32), dtype)
    out = as_dtype(np.matmul(w, v_coarse.astype(np.float32)), dtype)
    if return_lse:
        return out, (m[..., 0] + np.log(l[..., 0])).astype(np.float32)
    return out


def gate_values(q, gate_weight, gate_bias, dtype: str = "fp32"):
    """attention.py:246-251 -- `sigmoid(q W^T + b)` over the last axis, or `sigmoid(q)` with no gate."""
    q = np.asarray(q, np.float32)
    if gate_weight is None:
        return as_dtype(1.0 / (1.0 + np.exp(-q)), dtype)
    z = q @ np.asarray(gate_weight, np.float32).T
    if gate_bias is not None:
        z = z + np.asarray(gate_bias, np.float32)
    return as_dtype((1.0 / (1.0 + np.exp(-z.astype(np.float64)))).astype(np.float32), dtype)


def hsa_attention(q, k, v, *, k_coarse=None, v_coarse=None, k_proj_mat, v_proj_mat,
                  gate_weight=None, gate_bias=None, block_size: int = 64, tau_min: float = 0.35,
                  tau_max: float = 1.0, proj_segment_len: int = 1560, dtype: str = "fp32",
                  topk_per_head=None, return_parts: bool = False):
    """attention.py:153-259 -- the whole HSA forward over `[B, L, H, D]` tensors.

    `dtype` is the dtype of q/k/v in the reference call.  `topk_per_head` (optional, `[H]`)
    replaces the cumulative-mass count by a fixed per-head count over the same descending order.
    """
    if (k_coarse is None) != (v_coarse is None):
        raise ValueError("k_coarse and v_coarse must be provided together")
    q = np.asarray(q, np.float32); k = np.asarray(k, np.float32); v = np.asarray(v, np.float32)
    bsz, q_len, heads, d = q.shape
    kv_len = k.shape[1]
    if q_len <= 0 or kv_len <= 0:
        raise ValueError("q_len and kv_len must be positive")

    q_t = np.ascontiguousarray(q.transpose(0, 2, 1, 3))
    if k_coarse is None:
        kc, vc = compress_kv(np.ascontiguousarray(k.transpose(0, 2, 1, 3)),
                             np.ascontiguousarray(v.transpose(0, 2, 1, 3)),
                             segment_len=proj_segment_len, k_proj_mat=k_proj_mat,
                             v_proj_mat=v_proj_mat, block_size=block_size, dtype=dtype)
    else:
        kc = np.ascontiguousarray(np.asarray(k_coarse, np.float32).transpose(0, 2, 1, 3))
        vc = np.ascontiguousarray(np.asarray(v_coarse, np.float32).transpose(0, 2, 1, 3))
    out_linear = linear_branch(q_t, kc, vc, dtype=dtype)                      # [B,H,Lq,D]

    q_pad, kv_pad, nq, nkv = block_counts(q_len, kv_len, block_size)
    q_tp = np.ascontiguousarray(pad_to_len(q, q_pad).transpose(0, 2, 1, 3))
    k_tp = np.ascontiguousarray(pad_to_len(k, kv_pad).transpose(0, 2, 1, 3))
    v_tp = np.ascontiguousarray(pad_to_len(v, kv_pad).transpose(0, 2, 1, 3))

    block_attn = block_attention_map(block_mean_pool(q_tp, q_len, nq, block_size, dtype),
                                     block_mean_pool(k_tp, kv_len, nkv, block_size, dtype))
    index, num, _, thresholds = build_block_routing(block_attn, tau_min, tau_max)
    if topk_per_head is not None:
        num = fixed_topk_num(topk_per_head, bsz, nq, nkv)
    sizes = variable_block_sizes(kv_len, kv_pad, block_size)

    out_sparse = block_sparse_attention(bf16_round(q_tp), bf16_round(k_tp), bf16_round(v_tp),
                                        index, num, sizes, block_size, dtype="bf16")
    gate = gate_values(q, gate_weight, gate_bias, dtype=dtype)                # [B,Lq,H,D]
    sparse = as_dtype(out_sparse.transpose(0, 2, 1, 3)[:, :q_len], dtype)
    linear = out_linear.transpose(0, 2, 1, 3)
    out = as_dtype(sparse + linear * gate, dtype)
    if return_parts:
        return out, dict(sparse=sparse, linear=linear, gate=gate, index=index, num=num,
                         thresholds=thresholds, block_attn=block_attn)
    return out


def merge_partials(outs, lses):
    """Combine per-shard softmax partials of one branch: `O = sum_g exp(LSE_g - LSE) O_g`.

    `outs[g]` is the shard's normalised output `[..., D]`, `lses[g]` its natural-log sum-exp
    `[...]` (-inf where the shard saw no keys).  The reference has no sharded path; this is the
    standard log-sum-exp identity its single-device softmax (block_sparse_torch.py:62-64,
    attention.py:116-118) satisfies over any partition of the key set.
    """
    lses = np.stack([np.asarray(x, np.float64) for x in lses])
    outs = np.stack([np.asarray(x, np.float64) for x in outs])
    m = np.max(lses, axis=0)
    m_safe = np.where(np.isfinite(m), m, 0.0)
    w = np.exp(lses - m_safe)
    total = np.sum(w, axis=0)
    with np.errstate(invalid="ignore", divide="ignore"):
        coef = np.where(total > 0, w / total, 0.0)
        lse = np.where(total > 0, m_safe + np.log(total), -np.inf)
    return np.sum(coef[..., None] * outs, axis=0).astype(np.float32), lse.astype(np.float32)
