"""The allocation-free routing entry point against the ordinary one.

`wa_route_select_static` exists for callers that may not allocate device memory when routing runs
(an inference server that splits HBM among its models once at start-up, a plugin inside a host that
owns the allocator, a loop that has to avoid the device synchronisation an allocation implies).
Its scratch is a fixed array inside the library, so what has to hold is: same block ids, counts,
mask and thresholds as `wa_route_select` on the same probabilities, also on a second call that
finds the previous call's data still in that array, and a clear refusal beyond the built-in size.
Collected last on purpose (file name), so an `-x` run has already exercised everything else.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_static, attn, tau_min, tau_max, fixed=None):
    from worldattention_b200 import _lib
    b, h, nq, nkv = attn.shape
    dev = attn.device
    outs = []
    for static in (False, True):
        index = torch.empty((b, h, nq, nkv), device=dev, dtype=torch.int32)
        num = torch.empty((b, h, nq), device=dev, dtype=torch.int32)
        mask = torch.empty((b, h, nq, nkv), device=dev, dtype=torch.bool)
        thr = torch.empty((h,), device=dev, dtype=torch.float32)
        stream = _lib.stream_ptr(dev)
        if static:
            rc = lib.wa_route_select_static(attn.data_ptr(), b, h, nq, nkv, tau_min, tau_max, _lib.ptr(fixed),
                                            index.data_ptr(), num.data_ptr(), mask.data_ptr(), thr.data_ptr(), stream)
        else:
            gini = torch.empty((b * h * nq,), device=dev, dtype=torch.float32)
            rc = lib.wa_route_select(attn.data_ptr(), b, h, nq, nkv, tau_min, tau_max, _lib.ptr(fixed),
                                     index.data_ptr(), num.data_ptr(), mask.data_ptr(), thr.data_ptr(),
                                     gini.data_ptr(), stream)
        _lib.check(rc)
        torch.cuda.synchronize()
        outs.append((index, num, mask, thr))
    return outs


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from worldattention_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    first = torch.softmax(torch.randn(2, 4, 37, 256, device=dev) * 2.0, dim=-1).contiguous()
    second = torch.softmax(torch.randn(1, 12, 5, 1000, device=dev) * 3.0, dim=-1).contiguous()   # other shape, stale scratch
    fixed = torch.tensor([4, 8, 16, 32, 4, 8, 16, 32, 1, 0, 2000, 7], dtype=torch.int32, device=dev)
    for attn, tau, fx in ((first, (0.35, 1.0), None), (second, (0.2, 0.9), None), (second, (0.35, 1.0), fixed)):
        (i0, n0, m0, t0), (i1, n1, m1, t1) = _call(lib, True, attn, tau[0], tau[1], fx)
        assert torch.equal(i0, i1) and torch.equal(n0, n1) and torch.equal(m0, m1)
        assert torch.equal(t0, t1)          # bit-identical: same kernels, same arithmetic
    # and it agrees with the oracle like the ordinary entry point does
    from oracle import hsa_oracle as O
    index, num, mask, thr = O.build_block_routing(first.cpu().numpy(), 0.35, 1.0, return_mask=True)
    _, (i1, n1, m1, t1) = _call(lib, True, first, 0.35, 1.0)
    assert np.array_equal(i1.cpu().numpy(), index) and np.array_equal(n1.cpu().numpy(), num)
    assert np.array_equal(t1.cpu().numpy(), thr)


def test_static_scratch_entry_point_rejects_oversized_problems():
    from worldattention_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    dummy = torch.zeros(16, device=dev)
    rc = lib.wa_route_select_static(dummy.data_ptr(), 1, 16, 65536 // 16 + 1, 4, 0.35, 1.0, None, dummy.data_ptr(),
                                    dummy.data_ptr(), None, dummy.data_ptr(), _lib.stream_ptr(dev))
    assert rc == _lib.WA_ERR_UNSUPPORTED
    assert b"exceed the built-in scratch" in lib.wa_last_error()
