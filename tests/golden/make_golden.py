"""Generate the golden vectors under tests/golden/ from the reference's own PyTorch functions.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/WorldAttention

The reference's hot-path files depend only on torch, but their parent packages import heavy
optional dependencies; empty namespace packages are registered for the parents so that only
`wan.modules.hsa`, `pipeline.hkv` and `trainer.hsa_stage` load.  Inputs come from
`torch.manual_seed`; both inputs and reference outputs are stored (bf16 tensors as the float32
values they represent), so the fixtures need neither the reference nor torch's RNG to be replayed.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch


def _stub_reference(ref: str) -> None:
    for name, sub in [("wan", "wan"), ("wan.modules", "wan/modules"), ("pipeline", "pipeline"),
                      ("trainer", "trainer")]:
        mod = types.ModuleType(name)
        mod.__path__ = [os.path.join(ref, sub)]
        sys.modules[name] = mod


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    if torch.is_complex(t):
        return t.numpy()
    return t.detach().numpy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("WORLDATTENTION_REFERENCE"), required="WORLDATTENTION_REFERENCE" not in os.environ,
                    help="checkout of alibaba-damo-academy/WorldAttention (or set WORLDATTENTION_REFERENCE)")
    ap.add_argument("--out", default=os.path.dirname(os.path.abspath(__file__)))
    args = ap.parse_args()
    _stub_reference(args.reference)

    from wan.modules.hsa import (HSAAttention, block_sparse_attention_reference,
                                 build_block_routing, compress_kv)
    from wan.modules.hsa.attention import _linear_branch
    from wan.modules.hsa.routing import (block_attention_map, block_mean_pool,
                                         variable_block_sizes)
    from trainer.hsa_stage import init_hsa_parameters
    from pipeline.hkv import HKVCache
    from pipeline.hkv.retrieval import (page_key_index, prompt_index, query_index, score_pages,
                                        select_top_chunks, select_topk_pages)
    from pipeline.hkv.rope import derope_temporal, shift_temporal_rope, temporal_band

    torch.set_grad_enabled(False)
    out = {}

    # ---- routing: probabilities -> (index, num, mask, thresholds) -------------------------------
    torch.manual_seed(0)
    attn = torch.softmax(torch.randn(2, 4, 5, 16) * 2.0, dim=-1)
    r = build_block_routing(attn, 0.35, 1.0, return_mask=True)
    out["routing_small"] = dict(block_attn=_np(attn), index=_np(r.index), num=_np(r.num),
                                mask=_np(r.mask), thresholds=_np(r.thresholds),
                                tau=np.array([0.35, 1.0]))
    torch.manual_seed(10)
    attn = torch.softmax(torch.randn(1, 3, 7, 203) * 3.0, dim=-1)
    r = build_block_routing(attn, 0.2, 0.9, return_mask=True)
    out["routing_wide"] = dict(block_attn=_np(attn), index=_np(r.index), num=_np(r.num),
                               mask=_np(r.mask), thresholds=_np(r.thresholds),
                               tau=np.array([0.2, 0.9]))

    # ---- pooling + map --------------------------------------------------------------------------
    for name, dtype, length, bs in [("pool_ragged_fp32", torch.float32, 200, 64),
                                    ("pool_aligned_fp32", torch.float32, 192, 64),
                                    ("pool_ragged_bf16", torch.bfloat16, 200, 64),
                                    ("pool_aligned_bf16", torch.bfloat16, 256, 128)]:
        torch.manual_seed(2)
        nb = -(-length // bs)
        x = torch.randn(1, 2, length, 16).to(dtype)
        xp = torch.cat([x, torch.zeros(1, 2, nb * bs - length, 16, dtype=dtype)], dim=2)
        pooled = block_mean_pool(xp, length, nb, bs)
        out[name] = dict(x=_np(xp), pooled=_np(pooled.float()), length=np.array(length),
                         block_size=np.array(bs))
    torch.manual_seed(3)
    qp, kp = torch.randn(1, 2, 3, 16), torch.randn(1, 2, 9, 16)
    out["block_map"] = dict(q_pooled=_np(qp), k_pooled=_np(kp), block_attn=_np(block_attention_map(qp, kp)))

    # ---- sparse branch reference ---------------------------------------------------------------
    torch.manual_seed(4)
    bs, nq, nkv, d = 16, 3, 5, 24
    kv_len = nkv * bs - 5
    q = torch.randn(1, 2, nq * bs, d).bfloat16()
    k = torch.randn(1, 2, nkv * bs, d).bfloat16()
    v = torch.randn(1, 2, nkv * bs, d).bfloat16()
    k[:, :, kv_len:] = 0
    v[:, :, kv_len:] = 0
    index = torch.stack([torch.stack([torch.randperm(nkv) for _ in range(nq)]) for _ in range(2)])[None].int()
    num = torch.tensor([[[1, 3, 5], [0, 2, 4]]], dtype=torch.int32)
    sizes = variable_block_sizes(kv_len, nkv * bs, bs, "cpu")
    got = block_sparse_attention_reference(q, k, v, index, num, sizes, bs)
    out["sparse_ref"] = dict(q=_np(q), k=_np(k), v=_np(v), index=_np(index), num=_np(num),
                             sizes=_np(sizes), block_size=np.array(bs), out=_np(got))

    # ---- compress + linear ---------------------------------------------------------------------
    torch.manual_seed(5)
    kk, vv = torch.randn(1, 3, 130, 16), torch.randn(1, 3, 130, 16)
    ek, ev = torch.randn(2, 50).bfloat16(), torch.randn(2, 50).bfloat16()
    kc, vc = compress_kv(kk, vv, segment_len=50, k_proj_mat=ek, v_proj_mat=ev, block_size=32)
    qq = torch.randn(1, 3, 70, 16)
    lin = _linear_branch(qq, kc, vc)
    out["compress_linear_fp32"] = dict(k=_np(kk), v=_np(vv), ek=_np(ek), ev=_np(ev), kc=_np(kc),
                                       vc=_np(vc), q=_np(qq), linear=_np(lin),
                                       segment_len=np.array(50), block_size=np.array(32))
    kc16, vc16 = compress_kv(kk.bfloat16(), vv.bfloat16(), segment_len=50, k_proj_mat=ek,
                             v_proj_mat=ev, block_size=32)
    lin16 = _linear_branch(qq.bfloat16(), kc16, vc16)
    out["compress_linear_bf16"] = dict(k=_np(kk.bfloat16()), v=_np(vv.bfloat16()), ek=_np(ek),
                                       ev=_np(ev), kc=_np(kc16), vc=_np(vc16),
                                       q=_np(qq.bfloat16()), linear=_np(lin16),
                                       segment_len=np.array(50), block_size=np.array(32))

    # ---- whole module forward ------------------------------------------------------------------
    for name, dtype, heads, d, q_len, kv_len, seg in [("hsa_fp32", torch.float32, 3, 16, 100, 200, 50),
                                                      ("hsa_bf16", torch.bfloat16, 2, 32, 150, 500, 100)]:
        torch.manual_seed(0)
        hsa = HSAAttention(num_heads=heads, head_dim=d, block_size=64, tau_min=0.35, tau_max=1.0,
                           proj_segment_len=seg, backend="torch")
        init_hsa_parameters(hsa)
        torch.manual_seed(6)
        hsa.gate_lin.weight.copy_(torch.randn(d, d) * 0.2)
        hsa.gate_lin.bias.copy_(torch.randn(d) * 0.5)
        hsa.k_proj_mat.add_((torch.randn_like(hsa.k_proj_mat.float()) * 0.01).bfloat16())
        hsa.v_proj_mat.add_((torch.randn_like(hsa.v_proj_mat.float()) * 0.01).bfloat16())
        torch.manual_seed(1)
        q = torch.randn(1, q_len, heads, d).to(dtype)
        k = torch.randn(1, kv_len, heads, d).to(dtype)
        v = torch.randn(1, kv_len, heads, d).to(dtype)
        y = hsa(q, k, v)
        kc, vc = hsa.compress_kv_cache(k, v)
        y2 = hsa(q, k, v, k_coarse=kc, v_coarse=vc)
        out[name] = dict(q=_np(q), k=_np(k), v=_np(v), out=_np(y), out_cached=_np(y2),
                         kc=_np(kc), vc=_np(vc), ek=_np(hsa.k_proj_mat), ev=_np(hsa.v_proj_mat),
                         gw=_np(hsa.gate_lin.weight), gb=_np(hsa.gate_lin.bias),
                         segment_len=np.array(seg), block_size=np.array(64),
                         tau=np.array([0.35, 1.0]))

    # ---- HKV rope / retrieval ------------------------------------------------------------------
    head_dim, heads = 24, 2
    pairs = head_dim // 2
    inv = 1.0 / (10000.0 ** (torch.arange(0, pairs, dtype=torch.float64) / pairs))
    table = torch.polar(torch.ones(128, pairs, dtype=torch.float64),
                        torch.outer(torch.arange(128, dtype=torch.float64), inv))
    freqs = temporal_band(table, head_dim)
    torch.manual_seed(7)
    keys = torch.randn(2, 24, heads, head_dim)
    shifted = shift_temporal_rope(keys, freqs, 9, 3)
    frame_ids = 5 + torch.arange(24) // 4
    deroped = derope_temporal(keys, freqs, frame_ids)
    spans = [(0, 8), (8, 16), (16, 24)]
    pidx = page_key_index(keys, spans, frame_seq_length=4, start_frame=5, temporal_freqs=freqs)
    keys16 = keys.bfloat16()
    pidx16 = page_key_index(keys16, spans, frame_seq_length=4, start_frame=5, temporal_freqs=freqs)
    shifted16 = shift_temporal_rope(keys16, freqs, 200, 3)     # clamps to the 128-row table
    qvec = query_index(torch.randn(2, 10, heads * head_dim))
    scores = score_pages(qvec, pidx)
    out["hkv_rope"] = dict(freqs=_np(freqs), keys=_np(keys), shifted=_np(shifted),
                           frame_ids=_np(frame_ids), deroped=_np(deroped), page_index=_np(pidx),
                           keys16=_np(keys16), page_index16=_np(pidx16), shifted16=_np(shifted16),
                           qvec=_np(qvec), scores=_np(scores), spans=np.array(spans))
    torch.manual_seed(8)
    pe = torch.randn(2, 6, 8)
    pi = prompt_index(pe)
    bank = torch.nn.functional.normalize(torch.randn(5, 8), dim=1)
    chunks = select_top_chunks(pi, bank, 2)
    cands = [(c, p, torch.randn(heads * head_dim)) for c in range(3) for p in range(4)]
    sel = select_topk_pages(qvec, cands, 5)
    out["hkv_retrieval"] = dict(prompt=_np(pe), prompt_index=_np(pi), bank=_np(bank),
                                top_chunks=np.array(chunks), qvec=_np(qvec),
                                cand_ids=np.array([(c, p) for c, p, _ in cands]),
                                cand_vecs=np.stack([_np(x) for _, _, x in cands]),
                                sel_ids=np.array([(c, p) for c, p, _ in sel]),
                                sel_scores=np.array([s for _, _, s in sel], dtype=np.float32))

    # ---- HKV store / retrieve / apply end to end ------------------------------------------------
    frame_tokens, page_frames, capacity, layers = 4, 2, 20, 2
    hsa_mods = []
    for layer in range(layers):
        m = HSAAttention(num_heads=heads, head_dim=head_dim, block_size=64,
                         proj_segment_len=frame_tokens, backend="torch")
        m.k_proj_mat[0, :] = (layer + 1) / frame_tokens
        m.v_proj_mat[0, :] = (layer + 2) / frame_tokens
        hsa_mods.append(m)
    coarse_slots = hsa_mods[0].coarse_cache_size(capacity)

    def make_cache(dtype):
        return [dict(k=torch.zeros(1, capacity, heads, head_dim, dtype=dtype),
                     v=torch.zeros(1, capacity, heads, head_dim, dtype=dtype),
                     k_coarse=torch.full((1, coarse_slots, heads, head_dim), -9.0, dtype=dtype),
                     v_coarse=torch.full((1, coarse_slots, heads, head_dim), -9.0, dtype=dtype),
                     global_end_index=torch.zeros([], dtype=torch.long),
                     local_end_index=torch.zeros([], dtype=torch.long)) for _ in range(layers)]

    for name, dtype in [("hkv_cache_fp32", torch.float32), ("hkv_cache_bf16", torch.bfloat16)]:
        torch.manual_seed(9)
        bank_cache = HKVCache(frame_seq_length=frame_tokens, page_size_frames=page_frames,
                              topk_pages=3, stage1_topk_chunks=2, cpu_max_chunks=8)
        rec = {}
        prompts = [torch.randn(1, 6, 8) for _ in range(3)]
        valid = [16, 20, 12]
        starts = [4, 9, 12]
        for c in range(3):
            cache = make_cache(dtype)
            for layer, blk in enumerate(cache):
                blk["k"][:, : valid[c]] = torch.randn(1, valid[c], heads, head_dim).to(dtype)
                blk["v"][:, : valid[c]] = torch.randn(1, valid[c], heads, head_dim).to(dtype)
                blk["local_end_index"].fill_(valid[c])
                rec[f"c{c}_l{layer}_k"] = _np(blk["k"][:, : valid[c]])
                rec[f"c{c}_l{layer}_v"] = _np(blk["v"][:, : valid[c]])
            bank_cache.store(cache, prompt_embeds=prompts[c], current_start_frame=starts[c],
                             temporal_freqs=freqs)
            rec[f"c{c}_page_index"] = _np(bank_cache.chunks[c]["page_index"])
            rec[f"c{c}_start_frame"] = np.array(bank_cache.chunks[c]["start_frame"])
        qv = torch.randn(heads * head_dim)
        pairs_sel = bank_cache.retrieve(prompt_embeds=prompts[1] + 0.05 * torch.randn(1, 6, 8), query_vec=qv)
        target = make_cache(dtype)
        for blk in target:
            blk["k"].fill_(7.0)
            blk["v"].fill_(7.0)
        installed = bank_cache.apply(target, pairs_sel, current_start_frame=30, temporal_freqs=freqs,
                                     hsa_modules=hsa_mods)
        rec.update(qvec=_np(qv), pairs=np.array(pairs_sel), installed=np.array(installed),
                   valid=np.array(valid), starts=np.array(starts), freqs=_np(freqs),
                   prompts=np.stack([_np(p) for p in prompts]),
                   prompt_bank=np.stack([_np(p) for p in bank_cache.prompt_bank]),
                   ek=np.stack([_np(m.k_proj_mat) for m in hsa_mods]),
                   ev=np.stack([_np(m.v_proj_mat) for m in hsa_mods]),
                   dims=np.array([frame_tokens, page_frames, capacity, layers, heads, head_dim, 30]))
        for layer, blk in enumerate(target):
            rec[f"out_l{layer}_k"] = _np(blk["k"])
            rec[f"out_l{layer}_v"] = _np(blk["v"])
            rec[f"out_l{layer}_kc"] = _np(blk["k_coarse"])
            rec[f"out_l{layer}_vc"] = _np(blk["v_coarse"])
            rec[f"out_l{layer}_ends"] = np.array([int(blk["global_end_index"]), int(blk["local_end_index"])])
        out[name] = rec

    # ---- q/k RMSNorm + causal RoPE (wan/modules/model.py:29-36, 70-86; wan/modules/causal_model.py:34-62) -------------
    # The modules that hold these functions import the whole model zoo, so the three definitions are taken out of the
    # reference's source text and executed on their own: the code that runs is still the reference's.
    import ast
    import torch.nn as nn

    def reference_definitions(path, names):
        text = open(path).read()
        chunks = [ast.get_source_segment(text, node) for node in ast.parse(text).body
                  if isinstance(node, (ast.FunctionDef, ast.ClassDef)) and node.name in names]
        scope = {"torch": torch, "nn": nn, "math": __import__("math")}
        exec("\n\n".join(chunks), scope)
        return [scope[n] for n in names]

    rope_params, WanRMSNorm = reference_definitions(os.path.join(args.reference, "wan", "modules", "model.py"),
                                                    ["rope_params", "WanRMSNorm"])
    (causal_rope_apply,) = reference_definitions(os.path.join(args.reference, "wan", "modules", "causal_model.py"),
                                                 ["causal_rope_apply"])
    torch.manual_seed(77)
    heads, head_dim, grid, start_frame = 2, 128, (2, 3, 4), 5
    dim, tokens = heads * head_dim, grid[0] * grid[1] * grid[2]
    freqs = torch.cat([rope_params(1024, head_dim - 4 * (head_dim // 6)), rope_params(1024, 2 * (head_dim // 6)),
                       rope_params(1024, 2 * (head_dim // 6))], dim=1)
    rec = dict(freqs=_np(freqs[:16]), grid=np.array(grid), start_frame=np.array(start_frame), eps=np.array(1e-6))
    weight = 1.0 + 0.1 * torch.randn(dim)
    x = torch.randn(1, tokens, dim)
    for tag, dtype in (("fp32", torch.float32), ("bf16", torch.bfloat16)):
        norm = WanRMSNorm(dim, eps=1e-6).to(dtype)
        norm.weight.copy_(weight.to(dtype))
        xin = x.to(dtype)
        normed = norm(xin)
        roped = causal_rope_apply(normed.view(1, tokens, heads, head_dim), torch.tensor([grid]), freqs, start_frame=start_frame)
        rope_only = causal_rope_apply(xin.view(1, tokens, heads, head_dim), torch.tensor([grid]), freqs, start_frame=start_frame)
        rec.update({f"x_{tag}": _np(xin), f"weight_{tag}": _np(norm.weight), f"normed_{tag}": _np(normed),
                    f"roped_{tag}": _np(roped), f"rope_only_{tag}": _np(rope_only)})
    out["qk_norm_rope"] = rec

    for name, arrays in out.items():
        path = os.path.join(args.out, f"{name}.npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
