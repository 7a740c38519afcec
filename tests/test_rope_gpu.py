"""The fused q/k RMSNorm + causal rotary embedding kernel against the numpy oracle and the reference's own outputs."""
import numpy as np
import pytest
import torch

from oracle import rope_oracle as R
from tests.helpers import dev, to_gpu, to_np

pytestmark = pytest.mark.gpu


def test_norm_and_rope_match_oracle_and_reference(golden):
    from worldattention_b200 import rope
    g = golden("qk_norm_rope")
    grid, start, eps = tuple(int(v) for v in g["grid"]), int(g["start_frame"]), float(g["eps"])
    freqs = torch.from_numpy(g["freqs"])
    for tag, one_step in (("fp32", 0.0), ("bf16", 2 ** -7)):
        x = to_gpu(g[f"x_{tag}"], tag)
        w = to_gpu(g[f"weight_{tag}"], tag)
        got = rope.qk_norm_rope(x, w, eps, [grid], freqs, start, heads=2)
        want = R.qk_norm_rope(g[f"x_{tag}"], g[f"weight_{tag}"], eps, grid, g["freqs"], start, 2, tag)
        assert np.array_equal(to_np(got), want)                               # same arithmetic as the oracle, bit for bit
        ref = g[f"roped_{tag}"]                                              # the reference's own output
        if tag == "fp32":
            np.testing.assert_allclose(to_np(got), ref, rtol=0, atol=5e-6)
        else:       # torch's float32 mean may put a normalised value one bf16 step away; the rotation mixes a pair
            np.testing.assert_allclose(to_np(got), ref, rtol=0, atol=2 * one_step * np.abs(ref).max())
            assert np.mean(to_np(got) != ref) < 5e-3
        # rotation alone, the reference's signature; float64 product stored once: identical to the reference
        only = rope.causal_rope_apply(x.view(1, -1, 2, 128), torch.tensor([grid]), freqs, start_frame=start)
        assert np.array_equal(to_np(only), g[f"rope_only_{tag}"])
    # strided input (a slice of a fused q/k/v projection) and a frame offset beyond the table are handled
    qkv = torch.randn(1, 24, 3 * 256, device=dev()).bfloat16()
    q = qkv[..., :256]
    a = rope.qk_norm_rope(q, to_gpu(g["weight_bf16"], "bf16"), eps, [grid], freqs, start, heads=2)
    b = rope.qk_norm_rope(q.contiguous(), to_gpu(g["weight_bf16"], "bf16"), eps, [grid], freqs, start, heads=2)
    assert torch.equal(a, b)
    with pytest.raises(NotImplementedError):
        rope.causal_rope_apply(x.view(1, -1, 2, 128), torch.tensor([[1, 3, 4]]), freqs)
