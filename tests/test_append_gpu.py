"""The fused KV-cache append + compress (`HSAAttention.append_kv`) against the numpy oracle's `compress_kv` and a plain
copy: rows land where they belong and nowhere else, the new segments' compressed slots match the oracle within one bf16
ulp of the float32 sums, rows that are in place already are only compressed, and shapes outside the fused kernel take
the copy + compress path with the same result.
"""
import math

import numpy as np
import pytest
import torch

from oracle import hsa_oracle as O
from tests.helpers import dev, to_gpu, to_np

pytestmark = pytest.mark.gpu


def _setup(wa, heads, d, seg, bs, frames_cached, frames_cap, dtype=torch.bfloat16, seed=0):
    rng = np.random.default_rng(seed)
    cap, slots_per = frames_cap * seg, math.ceil(seg / bs)
    hsa = wa.hsa.HSAAttention(heads, d, block_size=bs, proj_segment_len=seg).to(dev())
    ek = O.bf16_round((rng.standard_normal((slots_per, seg)) * 0.05).astype(np.float32))
    ev = O.bf16_round((rng.standard_normal((slots_per, seg)) * 0.05).astype(np.float32))
    with torch.no_grad():
        hsa.k_proj_mat.copy_(to_gpu(ek, "bf16")); hsa.v_proj_mat.copy_(to_gpu(ev, "bf16"))
    mk = lambda n: O.bf16_round(rng.standard_normal((1, n, heads, d)).astype(np.float32))
    old_k, old_v = mk(cap), mk(cap)
    k_cache, v_cache = to_gpu(old_k).to(dtype), to_gpu(old_v).to(dtype)
    kc = torch.full((1, frames_cap * slots_per, heads, d), 7.0, dtype=dtype, device=dev())
    vc = torch.full_like(kc, -7.0)
    return hsa, rng, mk, ek, ev, old_k, old_v, k_cache, v_cache, kc, vc, frames_cached * seg, slots_per


@pytest.mark.parametrize("heads,seg,bs,n_new", [(4, 390, 128, 2 * 390), (12, 1560, 128, 3 * 1560), (4, 390, 64, 390 + 100), (2, 200, 64, 150)])
def test_append_writes_rows_and_compressed_slots(heads, seg, bs, n_new):
    import worldattention_b200 as wa
    d = 128
    hsa, rng, mk, ek, ev, old_k, old_v, k_cache, v_cache, kc, vc, position, slots_per = _setup(wa, heads, d, seg, bs, 2, 6)
    new_k, new_v = mk(n_new), mk(n_new)
    hsa.append_kv(to_gpu(new_k, "bf16"), to_gpu(new_v, "bf16"), k_cache, v_cache, kc, vc, position=position)
    torch.cuda.synchronize()
    # rows: exactly the new ones, exactly there
    want_k, want_v = old_k.copy(), old_v.copy()
    want_k[:, position:position + n_new], want_v[:, position:position + n_new] = new_k, new_v
    assert np.array_equal(to_np(k_cache), want_k) and np.array_equal(to_np(v_cache), want_v)
    # compressed slots of the new segments against the oracle (float32 sums rounded to bf16: one ulp of slack)
    okc, ovc = O.compress_kv(np.ascontiguousarray(new_k.transpose(0, 2, 1, 3)), np.ascontiguousarray(new_v.transpose(0, 2, 1, 3)),
                             segment_len=seg, k_proj_mat=ek, v_proj_mat=ev, block_size=bs, dtype="bf16")
    okc, ovc = okc.transpose(0, 2, 1, 3), ovc.transpose(0, 2, 1, 3)
    n_seg = math.ceil(n_new / seg)
    first = position // seg * slots_per       # the compressed cache is laid out for whole segments
    got_kc, got_vc = to_np(kc), to_np(vc)
    at = 0
    for s_ in range(n_seg):
        r = min(slots_per, math.ceil(min(seg, n_new - s_ * seg) / bs))
        lo = first + s_ * slots_per
        np.testing.assert_allclose(got_kc[:, lo:lo + r], okc[:, at:at + r], rtol=2 ** -7, atol=1e-5)
        np.testing.assert_allclose(got_vc[:, lo:lo + r], ovc[:, at:at + r], rtol=2 ** -7, atol=1e-5)
        at += r
    # slots of other segments are untouched
    assert (got_kc[:, :first] == 7.0).all() and (got_vc[:, first + n_seg * slots_per:] == -7.0).all()
    # a second call on the same workspace (its counters were left ready) gives the same bits
    kc2, vc2 = torch.full_like(kc, 7.0), torch.full_like(vc, -7.0)
    hsa.append_kv(to_gpu(new_k, "bf16"), to_gpu(new_v, "bf16"), k_cache, v_cache, kc2, vc2, position=position)
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)
    # rows that are in place already: the call only compresses, with the same bits
    kc3, vc3 = torch.full_like(kc, 7.0), torch.full_like(vc, -7.0)
    hsa.append_kv(k_cache[:, position:position + n_new], v_cache[:, position:position + n_new], k_cache, v_cache, kc3, vc3,
                  position=position)
    assert torch.equal(kc3, kc) and torch.equal(vc3, vc)
    assert np.array_equal(to_np(k_cache), want_k)


def test_append_rejects_unaligned_positions_and_falls_back_for_other_dtypes():
    import worldattention_b200 as wa
    heads, d, seg, bs = 2, 128, 200, 64
    hsa, rng, mk, ek, ev, old_k, old_v, k_cache, v_cache, kc, vc, position, slots_per = _setup(wa, heads, d, seg, bs, 1, 4,
                                                                                              dtype=torch.float32)
    new_k, new_v = mk(seg), mk(seg)
    with pytest.raises(ValueError):
        hsa.append_kv(to_gpu(new_k), to_gpu(new_v), k_cache, v_cache, kc, vc, position=position + 1)
    with pytest.raises(ValueError):
        hsa.append_kv(to_gpu(new_k), to_gpu(new_v), k_cache, v_cache, kc, vc, position=3 * seg + seg)
    hsa.append_kv(to_gpu(new_k), to_gpu(new_v), k_cache, v_cache, kc, vc, position=position)       # float32: copy + compress path
    assert np.array_equal(to_np(k_cache[:, position:position + seg]), new_k)
    okc, _ = O.compress_kv(np.ascontiguousarray(new_k.transpose(0, 2, 1, 3)), np.ascontiguousarray(new_v.transpose(0, 2, 1, 3)),
                           segment_len=seg, k_proj_mat=ek, v_proj_mat=ev, block_size=bs, dtype="fp32")
    first = position // seg * slots_per
    np.testing.assert_allclose(to_np(kc)[:, first:first + slots_per], okc.transpose(0, 2, 1, 3), rtol=1e-5, atol=1e-5)
