"""Benchmark config 2 at FULL size (4680-token chunk over a 32760-token cache, 12 heads x 128, bf16, seed 1,
per-head top-k as drawn) through the tcgen05 path, held against the numpy oracle -- not against another
path of this library.  Routing is compared exactly: the whole descending order of every row, the counts
and the per-head thresholds.  Outputs meet the benchmark definition's tolerance.  Both routing block
sizes: 128 (the benchmark's) and 64 (the reference class's).
"""
import json
import math
import os

import numpy as np
import pytest
import torch

import bench
from oracle import hsa_oracle as O
from tests.helpers import attention_error, dev, to_np

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_REL = 2e-2, 1e-2


@pytest.mark.parametrize("workload", ["c2", "c2-64"])
def test_full_size_config2_routing_and_output_against_the_oracle(workload):
    import worldattention_b200 as wa
    spec = bench.WORKLOADS[workload]
    block = spec["block"]
    q_h, k_h, v_h = bench.host_inputs(spec, pin=False)
    topk = bench.draw_topk(spec)
    gw, gb = bench.gate_params()
    proj = bench.block_average_projection(block)
    q, k, v = (x.float().numpy() for x in (q_h, k_h, v_h))
    ek = proj.float().numpy()
    # one compressed cache for both sides, so that the comparison is of the forward alone
    kc, vc = O.compress_kv(np.ascontiguousarray(k.transpose(0, 2, 1, 3)), np.ascontiguousarray(v.transpose(0, 2, 1, 3)),
                           segment_len=bench.FRAME_TOKENS, k_proj_mat=ek, v_proj_mat=ek, block_size=block, dtype="bf16")
    kc, vc = np.ascontiguousarray(kc.transpose(0, 2, 1, 3)), np.ascontiguousarray(vc.transpose(0, 2, 1, 3))
    gw_bf16 = O.bf16_round(gw.numpy())            # the gate weight is a bf16 tensor-core operand in the fused kernel
    want, parts = O.hsa_attention(q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=ek, v_proj_mat=ek, gate_weight=gw_bf16,
                                  gate_bias=gb.numpy(), block_size=block, proj_segment_len=bench.FRAME_TOKENS, dtype="bf16",
                                  topk_per_head=topk.numpy(), return_parts=True)

    lin = torch.nn.Linear(bench.HEAD_DIM, bench.HEAD_DIM).to(dev())
    with torch.no_grad():
        lin.weight.copy_(gw); lin.bias.copy_(gb)
    bf = lambda x: torch.from_numpy(x).to(dev(), torch.bfloat16)
    out, (index, num, thresholds, used) = wa.hsa.hsa_attention(
        q_h.to(dev()), k_h.to(dev()), v_h.to(dev()), k_coarse=bf(kc), v_coarse=bf(vc), k_proj_mat=proj.to(dev()),
        v_proj_mat=proj.to(dev()), gate_lin=lin, block_size=block, proj_segment_len=bench.FRAME_TOKENS,
        topk_per_head=topk, return_routing=True, check_status=True)
    assert used, "the tcgen05 kernel did not run"

    got_index, got_num = to_np(index), to_np(num)
    assert np.array_equal(got_num, parts["num"])
    assert np.array_equal(to_np(thresholds), parts["thresholds"]), "per-head thresholds differ from the oracle's"
    differs = got_index != parts["index"]
    rate = float(differs.mean())
    selected = np.arange(got_index.shape[-1])[None, None, None, :] < got_num[..., None]
    rate_selected = float((differs & selected).sum() / max(int(selected.sum()), 1))
    log_dir = os.environ.get("WA_TEST_LOG_DIR")
    if log_dir:
        os.makedirs(log_dir, exist_ok=True)
        with open(os.path.join(log_dir, f"routing_parity_{workload}.json"), "w") as f:
            json.dump({"workload": workload, "rows": int(np.prod(got_index.shape[:-1])), "blocks_per_row": int(got_index.shape[-1]),
                       "id_mismatch_rate_all_positions": rate, "id_mismatch_rate_selected_positions": rate_selected}, f)
    if rate > 0:
        # say how far apart the two probabilities of every disagreeing position are before failing
        p = parts["block_attn"]
        a = np.take_along_axis(p, got_index.astype(np.int64), -1)[differs]
        b = np.take_along_axis(p, parts["index"].astype(np.int64), -1)[differs]
        ulps = np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))
        raise AssertionError(f"{workload}: {rate:.3e} of routing ids differ from the oracle ({rate_selected:.3e} of the selected "
                             f"ones); the probabilities at those positions are up to {int(ulps.max())} ulp apart")

    max_abs, mean_rel = attention_error(to_np(out), want)
    assert max_abs < MAX_ABS and mean_rel < MEAN_REL, (max_abs, mean_rel)
    assert math.isfinite(max_abs)
