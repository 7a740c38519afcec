"""GPU pieces of the KV-sharded path that need no second GPU."""
import numpy as np
import pytest
import torch

from tests.helpers import dev

pytestmark = pytest.mark.gpu


def test_local_selection_kernel_matches_the_tensor_formulation():
    """`wa_route_local_selection` against the same restriction written with tensor operations (CPU)."""
    from worldattention_b200 import sharded
    rng = np.random.default_rng(5)
    for nkv, lo, hi in ((256, 0, 128), (256, 128, 256), (70, 33, 70), (5, 0, 5), (300, 10, 11)):
        rows = (2, 3, 7)
        index = np.stack([rng.permutation(nkv) for _ in range(int(np.prod(rows)))]).reshape(*rows, nkv).astype(np.int32)
        index[0, 0, 0, :3] = index[0, 0, 0, 0]          # duplicates are allowed and collapse
        index[1, 2, 3, 0] = nkv + 7                      # out-of-range ids are clamped
        num = rng.integers(0, nkv + 1, size=rows).astype(np.int32)
        num[0, 1, 2] = 0
        want_idx, want_num = sharded.local_selection(torch.from_numpy(index), torch.from_numpy(num), lo, hi)
        got_idx, got_num = sharded.local_selection(torch.from_numpy(index).to(dev()), torch.from_numpy(num).to(dev()), lo, hi)
        assert torch.equal(got_num.cpu(), want_num)
        assert torch.equal(got_idx.cpu(), want_idx)
