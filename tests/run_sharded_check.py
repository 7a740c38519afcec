"""Multi-GPU parity check of the sharded HSA forward (not collected by pytest; run under torchrun):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29511 \
        tests/run_sharded_check.py

Every rank computes the single-GPU forward on the full tensors and compares it with the head-split and the
KV-sharded results (max-abs 2e-2 / mean-rel 1e-2; the head-split output is bit-identical by construction).
"""
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import worldattention_b200 as wa  # noqa: E402
from worldattention_b200 import sharded  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    heads, d, q_len, kv_len, seg, bs = 12, 128, 700, 6240, 1560, 128
    torch.manual_seed(0)                              # same tensors on every rank
    q = (torch.randn(1, q_len, heads, d, device=dev) * 0.3).bfloat16()
    k = (torch.randn(1, kv_len, heads, d, device=dev) * 0.3).bfloat16()
    v = torch.randn(1, kv_len, heads, d, device=dev).bfloat16()
    hsa = wa.hsa.HSAAttention(heads, d, block_size=bs, proj_segment_len=seg).to(dev)
    wa.hsa_stage.init_hsa_parameters(hsa)
    with torch.no_grad():
        hsa.gate_lin.weight.normal_(0, 0.05)
        hsa.gate_lin.bias.normal_(0, 0.2)
    for p in hsa.parameters():
        dist.broadcast(p.data, 0)
    topk = torch.tensor([4, 8, 16, 32, 2, 1, 9, 5, 12, 3, 7, 6], dtype=torch.int32, device=dev)
    for tk in (None, topk):
        hsa.topk_per_head = tk
        kc, vc = hsa.compress_kv_cache(k, v)
        want = hsa(q, k, v, k_coarse=kc, v_coarse=vc)

        plan = sharded.plan_head_split(heads, world, None if tk is None else tk.tolist())
        mine = plan[rank]
        got = sharded.hsa_attention_head_split(hsa, q[:, :, mine].contiguous(), k[:, :, mine].contiguous(),
                                               v[:, :, mine].contiguous(), k_coarse=kc[:, :, mine].contiguous(),
                                               v_coarse=vc[:, :, mine].contiguous(),
                                               topk_local=None if tk is None else tk[mine].contiguous(), head_plan=plan)
        assert torch.equal(got, want), "head-split output differs from the single-GPU output"

        shards = sharded.plan_kv_shards(kv_len, bs, world, seg)
        lo, hi = shards[rank]
        r = hsa.proj_rank
        seg_lo = math.ceil(lo / seg)
        seg_hi = math.ceil(hi / seg) if rank < world - 1 else math.ceil(kv_len / seg)
        got_kv = sharded.hsa_attention_kv_sharded(hsa, q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                                                  kc[:, seg_lo * r: seg_hi * r].contiguous(),
                                                  vc[:, seg_lo * r: seg_hi * r].contiguous(), kv_len=kv_len, shards=shards,
                                                  topk_per_head=tk)
        err = (got_kv.float() - want.float()).abs()
        max_abs = float(err.max())
        mean_rel = float(err.mean() / want.float().abs().mean())
        assert max_abs < 2e-2 and mean_rel < 1e-2, (max_abs, mean_rel)
        info = dict(sharded.last_call_info)
        assert info.get("collectives") == 3 or world == 1, info
        # the same forward with the all-to-all instead of peer stores (or the other way round): identical records, so
        # identical output
        other = "nccl" if info.get("exchange") == "peer stores" else "peer"
        try:
            got_other = sharded.hsa_attention_kv_sharded(hsa, q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                                                         kc[:, seg_lo * r: seg_hi * r].contiguous(),
                                                         vc[:, seg_lo * r: seg_hi * r].contiguous(), kv_len=kv_len, shards=shards,
                                                         topk_per_head=tk, exchange=other)
            assert torch.equal(got_other, got_kv), f"exchange={other} differs from exchange={info.get('exchange')}"
            info["other_exchange_equal"] = other
        except (ValueError, RuntimeError) as exc:      # e.g. a shard without compressed slots: peer stores do not apply
            info["other_exchange_skipped"] = str(exc)[:80]
        if rank == 0:
            print(f"topk={'fixed' if tk is not None else 'cum-mass'}: head-split exact, kv-shard max_abs={max_abs:.2e} "
                  f"mean_rel={mean_rel:.2e} {info}", flush=True)
        if tk is not None:
            # fixed top-k again, routed by exchanging each rank's best candidates instead of gathering the pooled keys
            got_c = sharded.hsa_attention_kv_sharded(hsa, q, k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous(),
                                                     kc[:, seg_lo * r: seg_hi * r].contiguous(),
                                                     vc[:, seg_lo * r: seg_hi * r].contiguous(), kv_len=kv_len, shards=shards,
                                                     topk_per_head=tk, routing="candidates", topk_max=32)
            err = (got_c.float() - want.float()).abs()
            max_abs = float(err.max())
            mean_rel = float(err.mean() / want.float().abs().mean())
            assert max_abs < 2e-2 and mean_rel < 1e-2, ("candidates", max_abs, mean_rel)
            if rank == 0:
                print(f"topk=fixed routing=candidates: max_abs={max_abs:.2e} mean_rel={mean_rel:.2e} "
                      f"{dict(sharded.last_call_info)}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
