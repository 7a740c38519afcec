"""HKV retrieval at benchmark config 3's shape -- 480 pages of 1560 tokens, 12 heads x 128, bf16, top-16 pages per
head -- for two layers, held against the numpy oracle: the per-head page ids (exact, equal scores by lower id) and
the installed cache (keys re-rotated page by page, values verbatim) of the device-resident path, where ids never
leave the GPU.
"""
import numpy as np
import pytest
import torch

from oracle import hkv_oracle as K
from tests.helpers import dev, to_np

pytestmark = pytest.mark.gpu


def test_config3_shape_ids_and_installed_pages_against_the_oracle():
    import worldattention_b200 as wa
    from worldattention_b200.hkv.install import build_records_device, gather_records_device
    from worldattention_b200.hkv.retrieval import score_and_topk_layers
    layers, pages, heads, d, page_tokens, topk = 2, 480, 12, 128, 1560, 16
    row = heads * d
    g = torch.Generator().manual_seed(3)
    centroids = torch.randn((layers, pages, row), generator=g) * 0.5      # per-page offsets: the separating part of a mean key
    centroids[0, 77] = centroids[0, 300]                                  # identical pages: the lower id must win
    query = torch.randn((row,), generator=g)
    nt = wa.hkv.temporal_complex_dims(d)
    rot = torch.randn((topk, nt, 2), generator=g)
    rot = (rot / rot.norm(dim=-1, keepdim=True)).contiguous()
    # every page resident in HBM: [K|V, layers, pages, tokens, H, D] bf16, filled on the device
    pool = torch.empty((2, layers, pages, page_tokens, heads, d), dtype=torch.bfloat16, device=dev())
    gen = torch.Generator(device=dev()).manual_seed(33)
    for i in range(2):
        for l in range(layers):
            pool[i, l].normal_(0, 1, generator=gen)

    scores, ids, vals = score_and_topk_layers(query.to(dev()), centroids.to(dev()), topk, groups=heads)
    ids_np = to_np(ids)
    for l in range(layers):
        for h in range(heads):
            want_scores = K.score_pages(query[h * d:(h + 1) * d].numpy(), centroids[l, :, h * d:(h + 1) * d].numpy())
            want_ids, want_vals = K.topk_lower_index_first(want_scores, topk)
            assert np.array_equal(to_np(scores)[l, h], want_scores)
            assert np.array_equal(ids_np[l, h], want_ids), (l, h)
            assert np.array_equal(to_np(vals)[l, h], want_vals)
    # the tie: both copies are selected or neither, and the lower id always comes first
    for h in range(heads):
        got = list(ids_np[0, h])
        if 300 in got:
            assert 77 in got and got.index(77) < got.index(300)

    cache = torch.zeros((2, layers, topk * page_tokens, heads, d), dtype=torch.bfloat16, device=dev())
    esz = 2
    page_stride = page_tokens * row * esz
    addr = torch.arange(pages, dtype=torch.int64, device=dev()) * page_stride
    common = dict(src_layer_stride=pages * page_stride, src_token_stride=row, dst_layer_stride=topk * page_stride,
                  dst_token_stride=row, page_tokens=page_tokens, head_dim=d)
    rec_k = build_records_device(ids, pool[0].data_ptr() + addr, dst=cache[0], rotate=True, **common)
    rec_v = build_records_device(ids, pool[1].data_ptr() + addr, dst=cache[1], rotate=False, **common)
    gather_records_device(torch.cat([rec_k, rec_v]), max_tokens=page_tokens, row_elems=d, head_dim=d, dtype=torch.bfloat16,
                          rotations=rot.to(dev()), n_temporal=nt)
    torch.cuda.synchronize()

    factors = (rot[..., 0].numpy() + 1j * rot[..., 1].numpy()).astype(np.complex64)      # [topk, nt]
    for l in range(layers):
        for h in range(heads):
            order = np.sort(ids_np[l, h])                  # installed in chronological (page id) order
            for r, page in enumerate(order):
                src_k = pool[0, l, int(page), :, h].float().cpu().numpy()           # [tokens, D]
                src_v = pool[1, l, int(page), :, h].float().cpu().numpy()
                want_k = K.apply_factor(src_k, factors[r][None, :], nt, "bf16")
                got_k = cache[0, l, r * page_tokens:(r + 1) * page_tokens, h].float().cpu().numpy()
                got_v = cache[1, l, r * page_tokens:(r + 1) * page_tokens, h].float().cpu().numpy()
                assert np.array_equal(got_k, want_k), (l, h, r)
                assert np.array_equal(got_v, src_v), (l, h, r)
