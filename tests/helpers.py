"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch


def dev():
    return torch.device("cuda:0")


def to_gpu(x: np.ndarray, dtype: str = "fp32") -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(x))
    if t.is_floating_point():
        t = t.to(torch.bfloat16 if dtype == "bf16" else torch.float32)
    return t.to(dev())


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def tie_aware_index_check(probs: np.ndarray, got_index: np.ndarray, want_index: np.ndarray) -> float:
    """Sorted probability sequences must be identical; ids may differ only inside runs of equal values.

    Returns the fraction of positions whose id differs.
    """
    got_p = np.take_along_axis(probs, got_index.astype(np.int64), axis=-1)
    want_p = np.take_along_axis(probs, want_index.astype(np.int64), axis=-1)
    assert np.array_equal(got_p, want_p), "sorted probability sequences differ"
    differs = got_index != want_index
    if differs.any():
        left = np.concatenate([np.full_like(got_p[..., :1], -1), got_p[..., :-1]], axis=-1)
        right = np.concatenate([got_p[..., 1:], np.full_like(got_p[..., :1], -1)], axis=-1)
        tied = (got_p == left) | (got_p == right)
        assert tied[differs].all(), "index differs outside a run of equal probabilities"
    return float(differs.mean())


def attention_error(got: np.ndarray, want: np.ndarray):
    """(max-abs, mean-rel) error metrics used for the attention output tolerance."""
    max_abs = float(np.max(np.abs(got - want)))
    mean_rel = float(np.mean(np.abs(got - want)) / max(np.mean(np.abs(want)), 1e-12))
    return max_abs, mean_rel
