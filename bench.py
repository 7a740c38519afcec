"""Benchmark of the HSA forward (and HKV retrieval) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c2-64|c5|c5-128]

Workload "c2" (default, benchmark config 2): one HSA layer forward, bf16, B=1, 12 heads x 128, a 4680-token
query chunk over a 32760-token KV cache, 128x128 blocks, per-head top-k drawn from {4, 8, 16, 32} (seed 1),
q/k/v ~ N(0,1)/sqrt(128) (seed 1).  One "step" is one chunk through `hsa_attention` with the compressed
cache supplied, as the causal pipeline calls it.  Metric: chunks per second (`ms_per_step` is ms/chunk).
Prints ONE JSON line on rank 0.  Beside the headline the line carries, at one GPU: the same chunk with
64-token blocks (`block64`), the long-horizon workload (`long_horizon`, config 5), the HKV retrieval of
config 3 (`hkv`: hot gather, cold-tier promotion, page centroids), `compress_kv`, the reference's Triton
kernel on this GPU (`triton_incumbent`) and the CPU baseline.

N > 1 shards the same chunk (strong scaling): heads are split over 2 / 4 GPUs, the KV range is sharded over
8 (or any N that does not divide the heads) with a log-sum-exp merge over NCCL; the sharded result is
checked (untimed) against the single-GPU call, and `long_horizon` reports config 5 sharded the same way.

`--impl reference` times the reference's own PyTorch CPU path (staged by `oracle/stage_reference.py`) on the
host cores, or, where that staging is absent, the numpy restatement of the same algorithm.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

HEADS, HEAD_DIM = 12, 128
FRAME_TOKENS = 1560
WORKLOADS = {
    # name: (q frames, kv frames, block, top-k policy)
    "c2": dict(q_frames=3, kv_frames=21, block=128, topk="adaptive", seed=1, scale=1.0 / math.sqrt(HEAD_DIM)),
    # config 2 with the reference class's default 64-token blocks and twice the block counts (the same selected tokens)
    "c2-64": dict(q_frames=3, kv_frames=21, block=64, topk="adaptive-x2", seed=1, scale=1.0 / math.sqrt(HEAD_DIM)),
    "c5": dict(q_frames=3, kv_frames=480, block=64, topk=32, seed=4, scale=1.0),
    # the long-horizon cache with 128-token blocks; top-16 blocks = the same 2048 selected tokens per query row as top-32 at 64
    "c5-128": dict(q_frames=3, kv_frames=480, block=128, topk=16, seed=4, scale=1.0),
}
L2_FLUSH_BYTES = 256 << 20
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused kernel on workload c2 (ncu capture summarised
# in profiles/hsa_fwd_sm100_config2.md)
NCU_TRAFFIC_BYTES = 167.3e6   # dram__bytes_read.sum + dram__bytes_write.sum of one launch of the attention kernel (profiles/hsa_fwd_sm100_config2.md)


# ------------------------------------------------------------------------------------------------
# workload construction (seeded)
# ------------------------------------------------------------------------------------------------
def draw_topk(spec, heads=HEADS):
    if spec["topk"] in ("adaptive", "adaptive-x2"):
        g = torch.Generator().manual_seed(spec["seed"])
        k = torch.tensor([4, 8, 16, 32])[torch.randint(0, 4, (heads,), generator=g)].to(torch.int32)
        return k * 2 if spec["topk"] == "adaptive-x2" else k
    return torch.full((heads,), int(spec["topk"]), dtype=torch.int32)


def host_inputs(spec, pin: bool):
    """q, k, v as bf16 host tensors `[1, L, H, D]` from the workload's seed."""
    g = torch.Generator().manual_seed(spec["seed"])
    q_len, kv_len = spec["q_frames"] * FRAME_TOKENS, spec["kv_frames"] * FRAME_TOKENS

    def draw(n):
        out = torch.empty((1, n, HEADS, HEAD_DIM), dtype=torch.bfloat16, pin_memory=pin)
        step = 65536
        for s in range(0, n, step):
            e = min(n, s + step)
            out[:, s:e] = (torch.randn((1, e - s, HEADS, HEAD_DIM), generator=g) * spec["scale"]).to(torch.bfloat16)
        return out
    return draw(q_len), draw(kv_len), draw(kv_len)


def device_inputs(spec, dev):
    """The same shapes drawn on the device (seeded device generator): for the long-horizon cache, whose 4.6 GB of
    keys and values would take minutes to draw on the host of every rank."""
    g = torch.Generator(device=dev).manual_seed(spec["seed"])
    q_len, kv_len = spec["q_frames"] * FRAME_TOKENS, spec["kv_frames"] * FRAME_TOKENS

    def draw(n):
        out = torch.empty((1, n, HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
        step = 131072
        for s in range(0, n, step):
            e = min(n, s + step)
            out[:, s:e] = (torch.randn((1, e - s, HEADS, HEAD_DIM), generator=g, device=dev) * spec["scale"]).to(torch.bfloat16)
        return out
    return draw(q_len), draw(kv_len), draw(kv_len)


def gate_params(seed=7):
    g = torch.Generator().manual_seed(seed)
    return torch.randn((HEAD_DIM, HEAD_DIM), generator=g) * 0.02, torch.zeros(HEAD_DIM)


def block_average_projection(block):
    rank = math.ceil(FRAME_TOKENS / block)
    e = torch.zeros((rank, FRAME_TOKENS))
    for r in range(rank):
        lo, hi = r * block, min((r + 1) * block, FRAME_TOKENS)
        e[r, lo:hi] = 1.0 / (hi - lo)
    return e.to(torch.bfloat16)


def algorithmic_flops(num: np.ndarray, index: np.ndarray, q_len, kv_len, block, lc, head_dim=HEAD_DIM):
    """Sparse 4*D*sum(rows_i * selected tokens), linear 4*D*H*Lq*Lc, gate 2*Lq*H*D^2."""
    nq, nkv = math.ceil(q_len / block), math.ceil(kv_len / block)
    rows = np.full((nq,), block, np.int64)
    rows[-1] = q_len - (nq - 1) * block
    sizes = np.full((nkv,), block, np.int64)
    sizes[-1] = kv_len - (nkv - 1) * block
    slots = np.arange(index.shape[-1])[None, None, None, :] < num[..., None]
    tokens = (sizes[np.clip(index, 0, nkv - 1)] * slots).sum(-1)           # [B, H, Nq]
    sparse = 4.0 * head_dim * float((tokens * rows[None, None, :]).sum())
    heads = num.shape[1]
    linear = 4.0 * head_dim * heads * q_len * lc
    gate = 2.0 * q_len * heads * head_dim * head_dim
    return sparse, linear, gate


def fixed_topk_flops(topk, q_len, kv_len, block, lc, heads):
    """The same count for a fixed per-head top-k without the routing tensors (an upper bound by less than one ragged
    block per row: the last key block is shorter)."""
    nkv = math.ceil(kv_len / block)
    sparse = 4.0 * HEAD_DIM * q_len * block * float(np.minimum(np.asarray(topk, np.float64), nkv).sum())
    return sparse, 4.0 * HEAD_DIM * heads * q_len * lc, 2.0 * q_len * heads * HEAD_DIM * HEAD_DIM


# ------------------------------------------------------------------------------------------------
# clocks sampler
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU during the timed region (NVML reads only)."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int, period_s: float = 0.002):
        self.gpu_index, self.period_s = gpu_index, period_s
        self.sm, self.mask, self.max_mhz = [], 0, None
        self.thread, self.stop_flag, self.error = None, threading.Event(), None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.gpu_index]) if visible and visible.split(",")[self.gpu_index].isdigit() else self.gpu_index
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception as err:  # noqa: BLE001
            self.error = f"NVML unavailable: {err}"
            return

        def loop():
            while not self.stop_flag.is_set():
                try:
                    self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
                    self.mask |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(self.period_s)
        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def mark(self):
        """Forget what was sampled so far: the timed region starts here (the thread itself was started earlier, so that
        NVML's start-up cost and the thread's first samples fall into the warm-up)."""
        self.sm, self.mask = [], 0

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error or "not sampled"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        reasons = [name for name, bit in self.REASONS.items() if self.mask & bit]
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own PyTorch path when its files are staged, else the numpy restatement
# ------------------------------------------------------------------------------------------------
def staged_reference():
    """The reference's hsa / hkv modules from the staged copy (`oracle/stage_reference.py`), or None."""
    try:
        from oracle import stage_reference
        if not stage_reference.staged():
            return None
        return stage_reference.import_staged()
    except Exception:  # noqa: BLE001
        return None


def reference_fixed_topk(topk):
    """Make the staged reference's `hsa_attention` select a fixed number of blocks per head.

    The reference has no top-k switch: its kernels read `(index, num)` (block_sparse_torch.py:56-57), so a top-k
    policy is its own descending `index` with `num := min(k_h, Nkv)`.  Its forward is left as it is; only the routing
    function it calls is wrapped to overwrite the count."""
    att = sys.modules["wan.modules.hsa.attention"]
    original = getattr(att, "_bench_original_routing", None) or att.build_block_routing
    att._bench_original_routing = original

    def routing(block_attn, tau_min, tau_max, *, return_mask=False):
        r = original(block_attn, tau_min=tau_min, tau_max=tau_max, return_mask=return_mask)
        if topk is not None:
            k = torch.clamp(topk.to(device=r.num.device, dtype=torch.int64), max=r.index.shape[-1])
            r.num = k.view(1, -1, 1).expand_as(r.num).to(torch.int32).contiguous()
        return r
    att.build_block_routing = routing
    return att.hsa_attention


def cpu_step_setup(spec):
    """One whole chunk of the workload on the host cores.  Returns `(step, kind, what)`."""
    q, k, v = host_inputs(spec, pin=False)
    block = spec["block"]
    topk = draw_topk(spec)
    gw, gb = gate_params()
    proj = block_average_projection(block)
    q_len, kv_len = q.shape[1], k.shape[1]
    size = f"whole chunk, all {HEADS} heads ({q_len} q x {kv_len} kv tokens)"
    ref = staged_reference()
    if ref is not None:
        hsa_mod, _ = ref
        forward = reference_fixed_topk(topk)
        lin = torch.nn.Linear(HEAD_DIM, HEAD_DIM).to(torch.bfloat16)
        with torch.no_grad():
            lin.weight.copy_(gw); lin.bias.copy_(gb)
            kc, vc = hsa_mod.compress_kv(k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous(),
                                         segment_len=FRAME_TOKENS, k_proj_mat=proj, v_proj_mat=proj, block_size=block)
            kc, vc = kc.transpose(1, 2).contiguous(), vc.transpose(1, 2).contiguous()

        def step():
            with torch.no_grad():
                return forward(q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=proj, v_proj_mat=proj, gate_lin=lin,
                               block_size=block, proj_segment_len=FRAME_TOKENS, backend="torch")
        return step, "reference", f"{size}; the reference's own hsa_attention (backend='torch', bf16 tensors) from its staged sources, " \
                                  "count of selected blocks overridden per head"
    from oracle import hsa_oracle as O
    qs, ks, vs = (x.float().numpy() for x in (q, k, v))
    ek = proj.float().numpy()
    kc, vc = O.compress_kv(np.ascontiguousarray(ks.transpose(0, 2, 1, 3)), np.ascontiguousarray(vs.transpose(0, 2, 1, 3)),
                           segment_len=FRAME_TOKENS, k_proj_mat=ek, v_proj_mat=ek, block_size=block, dtype="bf16")
    kc, vc = kc.transpose(0, 2, 1, 3), vc.transpose(0, 2, 1, 3)

    def step():
        return O.hsa_attention(qs, ks, vs, k_coarse=kc, v_coarse=vc, k_proj_mat=ek, v_proj_mat=ek, gate_weight=gw.numpy(),
                               gate_bias=gb.numpy(), block_size=block, proj_segment_len=FRAME_TOKENS, dtype="bf16",
                               topk_per_head=topk.numpy())
    return step, "port", f"{size}; numpy restatement of the reference algorithm (oracle/), the reference sources are not staged here"


def run_cpu(spec, steps, warmup):
    step, kind, what = cpu_step_setup(spec)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return 1.0 / dt, dt * 1e3, kind, what


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # a step is one whole chunk (seconds on the host): a handful of them bounds the run
    steps, warmup = max(1, min(args.steps, 3)), max(0, min(args.warmup, 1))
    value, ms, kind, what = run_cpu(spec, steps, warmup)
    line = {
        "impl": "reference", "metric": "hsa_fwd_chunks_per_s", "value": value, "unit": "chunks/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args.workload, 1),
        "cpu_baseline": {"value": value, "unit": "chunks/s", "cores": cores, "kind": kind, "sample": what},
        "e2e": {"value": value, "unit": "chunks/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, n_gpus, mode=None):
    spec = WORKLOADS[name]
    if mode is None:
        mode = "single" if n_gpus == 1 else ("heads" if HEADS % n_gpus == 0 and n_gpus <= 4 else "kv")
    sharding = {"single": "none", "heads": "head-split, no data-path collective (outputs stay head-sharded)",
                "kv": "kv-shard: pooled keys all-gathered; per-branch partial outputs + log-sum-exp go to the rank that merges "
                      "their query rows (stored by the attention kernel into that rank's buffer over NVLink, or ONE NCCL "
                      "all-to-all: see 'exchange'); merge + gate fused; finished rows all-gathered"}[mode]
    note = "" if spec["block"] == 64 else " (128-token blocks are the benchmark's; the reference's HSAAttention class accepts 64 only, " \
                                          "its functional hsa_attention any size)"
    return {
        "workload": f"{name}: HSA layer forward, B=1 H={HEADS} D={HEAD_DIM}, q={spec['q_frames'] * FRAME_TOKENS} "
                    f"kv={spec['kv_frames'] * FRAME_TOKENS} tokens, block {spec['block']}{note}, top-k {spec['topk']}, seed {spec['seed']}",
        "compressed_cache": "precomputed (maintained incrementally, as the causal pipeline does)",
        "sharding": sharding,
        "l2": f"{L2_FLUSH_BYTES >> 20} MiB buffer written, then {L2_FLUSH_BYTES >> 20} MiB read (so its write-back is over), "
              "between timed steps",
    }


# ------------------------------------------------------------------------------------------------
# a workload on this rank: tensors, the (possibly sharded) forward, the single-GPU forward for checks
# ------------------------------------------------------------------------------------------------
class Work:
    def __init__(self, name, dev, world, rank, *, shard="auto", force_generic=False, gather_heads=False,
                 on_device=False, exchange="auto"):
        import worldattention_b200 as wa
        from worldattention_b200 import sharded
        from worldattention_b200.hsa.attention import _compress_blhd
        self.wa, self.sharded = wa, sharded
        self.name, self.dev, self.world, self.rank = name, dev, world, rank
        self.force_generic, self.gather = force_generic, gather_heads
        self.exchange, self.exchange_used = exchange, None
        spec = self.spec = WORKLOADS[name]
        self.block = block = spec["block"]
        self.topk_all = draw_topk(spec)
        if on_device:
            self.q_h = self.k_h = self.v_h = None
            q, k, v = device_inputs(spec, dev)
        else:
            self.q_h, self.k_h, self.v_h = host_inputs(spec, pin=True)
            q, k, v = (x.to(dev, non_blocking=True) for x in (self.q_h, self.k_h, self.v_h))
        self.q_len, self.kv_len = q.shape[1], k.shape[1]
        hsa = self.hsa = wa.hsa.HSAAttention(HEADS, HEAD_DIM, block_size=block, proj_segment_len=FRAME_TOKENS).to(dev)
        gw, gb = gate_params()
        with torch.no_grad():
            proj = block_average_projection(block)
            hsa.k_proj_mat.copy_(proj); hsa.v_proj_mat.copy_(proj)
            hsa.gate_lin.weight.copy_(gw); hsa.gate_lin.bias.copy_(gb)
        mode = "single"
        if world > 1:
            mode = "heads" if (HEADS % world == 0 and world <= 4) else "kv"
            if shard != "auto":
                mode = shard
        self.mode = mode
        self.full = None            # (q, k, v, kc, vc) of the unsharded problem, kept on rank 0 for the untimed check
        with torch.no_grad():
            if mode == "heads":
                self.plan = sharded.plan_head_split(HEADS, world, self.topk_all.tolist())
                mine = self.plan[rank]
                if rank == 0:
                    kc_f, vc_f = hsa.compress_kv_cache(k, v)
                    self.full = (q, k, v, kc_f, vc_f)
                if self.q_h is not None:
                    self.q_h, self.k_h, self.v_h = (x[:, :, mine].contiguous().pin_memory() for x in (self.q_h, self.k_h, self.v_h))
                q, k, v = (x[:, :, mine].contiguous() for x in (q, k, v))
                self.topk = self.topk_all[mine].contiguous().to(dev)
                self.kc, self.vc = hsa.compress_kv_cache(k, v)
            elif mode == "kv":
                self.shards = sharded.plan_kv_shards(self.kv_len, block, world, FRAME_TOKENS)
                lo, hi = self.shards[rank]
                self.k_loc, self.v_loc = k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous()
                # compressed segments are owned by the rank that owns their first token
                seg_lo = math.ceil(lo / FRAME_TOKENS)
                seg_hi = math.ceil(hi / FRAME_TOKENS) if rank < world - 1 else spec["kv_frames"]
                kc_all, vc_all = _compress_blhd(k, v, segment_len=FRAME_TOKENS, k_proj_mat=hsa.k_proj_mat,
                                                v_proj_mat=hsa.v_proj_mat, block_size=block)
                r = hsa.proj_rank
                self.kc, self.vc = kc_all[:, seg_lo * r: seg_hi * r].contiguous(), vc_all[:, seg_lo * r: seg_hi * r].contiguous()
                self.topk = self.topk_all.to(dev)
                if rank == 0:
                    self.full = (q, k, v, kc_all, vc_all)
                else:
                    del kc_all, vc_all
            else:
                self.topk = self.topk_all.to(dev)
                self.kc, self.vc = hsa.compress_kv_cache(k, v)
        self.q, self.k, self.v = q, k, v
        self.used_tuned = False
        torch.cuda.synchronize()

    def _single(self, q, k, v, kc, vc, topk, **extra):
        hsa = self.hsa
        return self.wa.hsa.hsa_attention(q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat,
                                         gate_lin=hsa.gate_lin, block_size=self.block, proj_segment_len=FRAME_TOKENS,
                                         topk_per_head=topk, force_generic=self.force_generic, **extra)

    def forward(self, gather=None):
        gather = self.gather if gather is None else gather
        with torch.no_grad():
            if self.mode == "single":
                return self._single(self.q, self.k, self.v, self.kc, self.vc, self.topk)
            if self.mode == "heads":
                out = self._single(self.q, self.k, self.v, self.kc, self.vc, self.topk)
                return self.sharded.gather_heads(out, self.plan) if gather else out
            out = self.sharded.hsa_attention_kv_sharded(self.hsa, self.q, self.k_loc, self.v_loc, self.kc, self.vc,
                                                        kv_len=self.kv_len, shards=self.shards, topk_per_head=self.topk,
                                                        topk_max=int(self.topk_all.max()), exchange=self.exchange)
            self.used_tuned = bool(self.sharded.last_call_info.get("used_tuned"))
            self.exchange_used = self.sharded.last_call_info.get("exchange")
            return out

    def flops(self):
        """(sparse, linear, gate) algorithmic FLOPs of what THIS rank's attention kernel computes; sets `used_tuned`."""
        lc = self.kc.shape[1]
        if self.mode in ("single", "heads"):
            with torch.no_grad():
                _, (index, num, _, used) = self._single(self.q, self.k, self.v, self.kc, self.vc, self.topk, return_routing=True)
            self.used_tuned = bool(used)
            return algorithmic_flops(num.cpu().numpy(), index.cpu().numpy(), self.q_len, self.kv_len, self.block, lc)
        self.forward()
        sparse, _, _ = fixed_topk_flops(self.topk_all.numpy(), self.q_len, self.kv_len, self.block, lc, HEADS)
        # every rank sees 1/world of the selected blocks on average, its own compressed slots, and no gate product
        return sparse / self.world, 4.0 * HEAD_DIM * HEADS * self.q_len * lc, 0.0

    def check_against_single_gpu(self):
        """Untimed: the sharded result against the single-GPU call on the full tensors (rank 0 holds them)."""
        import torch.distributed as dist
        if self.world == 1:
            return None
        got = self.forward(gather=True)
        res = None
        if self.rank == 0:
            q, k, v, kc, vc = self.full
            with torch.no_grad():
                want = self._single(q, k, v, kc, vc, self.topk_all.to(self.dev))
            diff = (got.float() - want.float()).abs()
            res = {"max_abs": float(diff.max()), "mean_rel": float(diff.mean() / want.float().abs().mean()),
                   "bit_equal": bool(torch.equal(got, want)), "ranks": self.world, "sharding": self.mode}
        dist.barrier()
        return res


class Flusher:
    def __init__(self, dev):
        self.flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        self.drain = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)

    def __call__(self):
        # evict everything, then read another buffer larger than L2: the timed step starts with a cold L2 that holds
        # no dirty lines, so it does not pay for the write-back of the flush itself
        self.flush.zero_()
        self.drain.sum()


def timed_steps(fn, steps, warmup, flush, lib=None, barrier=None):
    """Per-step milliseconds (CUDA events around each step, L2 flushed before) and, when `lib` profiles, the attention
    kernel's milliseconds per step."""
    for _ in range(warmup):
        flush()
        fn()
    if barrier:
        barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    step_ms, kern_ms = [], []
    for _ in range(steps):
        flush()
        ev0.record()
        fn()
        ev1.record()
        ev1.synchronize()
        step_ms.append(ev0.elapsed_time(ev1))
        if lib is not None:
            ms = ctypes.c_float(0.0)
            if lib.wa_profile_attention_ms(ctypes.byref(ms)) == 0:
                kern_ms.append(ms.value)
    return step_ms, kern_ms


def max_over_ranks(x: float, dev, world) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def side_workload(name, dev, world, rank, lib, flush, *, steps, shard="auto", on_device=False, check=True, exchange="auto"):
    """A second workload measured the same way as the headline (fewer steps): ms/chunk, kernel time, fractions."""
    import torch.distributed as dist
    work = Work(name, dev, world, rank, shard=shard, on_device=on_device, exchange=exchange)
    sparse_f, linear_f, gate_f = work.flops()
    barrier = (lambda: (dist.barrier(), torch.cuda.synchronize())) if world > 1 else None
    lib.wa_profile_enable(1)
    step_ms, kern_ms = timed_steps(work.forward, steps, 3, flush, lib, barrier)
    lib.wa_profile_enable(0)
    total = max_over_ranks(sum(step_ms), dev, world)
    peak_tf, _, _ = measured_peaks()
    kernel_ms = float(np.mean(kern_ms)) if kern_ms else None
    counted = sparse_f + (linear_f + gate_f if work.used_tuned else 0.0)
    out = {"workload": workload_config(name, world, work.mode)["workload"], "sharding": work.mode, "exchange": work.exchange_used,
           "ms_per_step": total / steps, "steps": steps, "kernel_ms_rank0": kernel_ms, "tcgen05_kernel": work.used_tuned,
           "flops_rank0": {"sparse": sparse_f, "linear": linear_f, "gate": gate_f},
           "frac_of_bf16_peak": (counted / (kernel_ms * 1e-3) / 1e12 / peak_tf) if kernel_ms else None,
           "sparse_only_frac": (sparse_f / (kernel_ms * 1e-3) / 1e12 / peak_tf) if kernel_ms else None}
    if check and world > 1:
        out["equals_single_gpu"] = work.check_against_single_gpu()
    del work
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# the reference's Triton kernel on this GPU (runs in a child process: a JIT failure must not take the bench down)
# ------------------------------------------------------------------------------------------------
def triton_incumbent_child():
    """Config 2 with 64-token blocks (the only size the reference's Triton launch supports): its `block_sparse_attention`
    on the `(index, num)` lists this library's routing produced, timed beside this library's fused kernel; and the
    reference's whole `hsa_attention(backend='triton')`."""
    import worldattention_b200 as wa
    ref = staged_reference()
    if ref is None:
        print(json.dumps({"unavailable": "reference sources are not staged (oracle/stage_reference.py)"}))
        return
    from wan.modules.hsa.block_sparse_triton import block_sparse_attention
    from wan.modules.hsa.routing import variable_block_sizes
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = wa._lib.lib()
    flush = Flusher(dev)
    work = Work("c2-64", dev, 1, 0)
    block, q_len, kv_len = work.block, work.q_len, work.kv_len
    with torch.no_grad():
        ours, (index, num, _, used) = work._single(work.q, work.k, work.v, work.kc, work.vc, work.topk, return_routing=True)
    q_pad, kv_pad = math.ceil(q_len / block) * block, math.ceil(kv_len / block) * block

    def padded(x, n):   # [1, L, H, D] -> [1, H, n, D], zero rows behind the real ones, as the reference prepares them
        out = torch.zeros((1, HEADS, n, HEAD_DIM), dtype=torch.bfloat16, device=dev)
        out[:, :, : x.shape[1]] = x.transpose(1, 2)
        return out
    q_t, k_t, v_t = padded(work.q, q_pad), padded(work.k, kv_pad), padded(work.v, kv_pad)
    sizes = variable_block_sizes(kv_len, kv_pad, block, dev)

    def triton_kernel():
        return block_sparse_attention(q_t, k_t, v_t, block_sizes=sizes, q2k_index=index, q2k_num=num)
    t_ms, _ = timed_steps(triton_kernel, 30, 5, flush)
    # this library's sparse branch alone (SIMT kernel, bf16-rounded output) is the like-for-like output check
    from worldattention_b200.hsa import branches
    want, _ = branches.sparse_branch(work.q, work.k, work.v, index, num, block, lse=False, round_output_bf16=True)
    got = triton_kernel().transpose(1, 2)[:, :q_len].float()
    diff = (got - want).abs()
    lib.wa_profile_enable(1)
    _, k_ms = timed_steps(work.forward, 30, 5, flush, lib)
    lib.wa_profile_enable(0)
    sparse_f, linear_f, gate_f = algorithmic_flops(num.cpu().numpy(), index.cpu().numpy(), q_len, kv_len, block, work.kc.shape[1])
    # the reference's whole forward on the GPU, Triton backend, same per-head counts
    forward_ref = reference_fixed_topk(work.topk)
    hsa = work.hsa
    gate_bf16 = torch.nn.Linear(HEAD_DIM, HEAD_DIM).to(dev, torch.bfloat16)
    with torch.no_grad():
        gate_bf16.weight.copy_(hsa.gate_lin.weight); gate_bf16.bias.copy_(hsa.gate_lin.bias)

    def reference_forward():
        with torch.no_grad():
            return forward_ref(work.q, work.k, work.v, k_coarse=work.kc, v_coarse=work.vc, k_proj_mat=hsa.k_proj_mat,
                               v_proj_mat=hsa.v_proj_mat, gate_lin=gate_bf16, block_size=block,
                               proj_segment_len=FRAME_TOKENS, backend="triton")
    try:
        ref_out = reference_forward()
        f_ms, _ = timed_steps(reference_forward, 10, 2, flush)
        o_ms, _ = timed_steps(work.forward, 30, 5, flush)
        d2 = (ref_out.float() - ours.float()).abs()
        whole = {"reference_forward_ms": float(np.mean(f_ms)), "this_library_forward_ms": float(np.mean(o_ms)),
                 "max_abs_between_outputs": float(d2.max()), "mean_rel": float(d2.mean() / ours.float().abs().mean())}
    except Exception as err:  # noqa: BLE001
        whole = {"unavailable": f"{type(err).__name__}: {err}"[:300]}
    peak_tf, _, _ = measured_peaks()
    tms, kms = float(np.mean(t_ms)), float(np.mean(k_ms))
    print(json.dumps({
        "workload": workload_config("c2-64", 1)["workload"],
        "triton_fwd_kernel_ms": tms, "triton_sparse_frac_of_bf16_peak": sparse_f / (tms * 1e-3) / 1e12 / peak_tf,
        "fused_tcgen05_kernel_ms": kms, "fused_kernel_does": "sparse + linear + gate + combine", "triton_kernel_does": "sparse branch only",
        "sparse_flops": sparse_f, "fused_sparse_only_frac": sparse_f / (kms * 1e-3) / 1e12 / peak_tf,
        "triton_vs_this_library_sparse_branch": {"max_abs": float(diff.max()), "mean_rel": float(diff.mean() / want.abs().mean())},
        "whole_forward": whole, "tcgen05_kernel_ran": bool(used)}))


def bench_triton_incumbent(timeout_s=420):
    try:
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--triton-incumbent-child"], capture_output=True, text=True,
                             timeout=timeout_s, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the child process did not finish in {timeout_s} s"}
    for line in reversed(res.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": ("child failed: " + (res.stderr.strip().splitlines() or ["no output"])[-1])[:400]}


# ------------------------------------------------------------------------------------------------
# compress_kv: the whole 21-frame cache, and the 3 new frames of one chunk (what the causal pipeline does per forward)
# ------------------------------------------------------------------------------------------------
def bench_compress(dev, flush, block=128, steps=20):
    from worldattention_b200.hsa.attention import _compress_blhd
    _, peak_gbs, _ = measured_peaks()
    proj = block_average_projection(block).to(dev)
    out = {}
    for label, frames in (("cache_21_segments", 21), ("chunk_3_segments", 3)):
        n = frames * FRAME_TOKENS
        k = torch.randn((1, n, HEADS, HEAD_DIM), device=dev).bfloat16()
        v = torch.randn((1, n, HEADS, HEAD_DIM), device=dev).bfloat16()

        def step():
            return _compress_blhd(k, v, segment_len=FRAME_TOKENS, k_proj_mat=proj, v_proj_mat=proj, block_size=block)
        ms, _ = timed_steps(step, steps, 3, flush)
        kc, _ = step()
        moved = 2.0 * (k.numel() + kc.numel()) * 2          # K and V: read the tokens, write the slots
        flops = 2 * 2.0 * proj.shape[0] * FRAME_TOKENS * frames * HEADS * HEAD_DIM
        t = float(np.mean(ms)) * 1e-3
        out[label] = {"tokens": n, "slots": int(kc.shape[1]), "ms": t * 1e3, "bytes": moved, "gbs": moved / t / 1e9,
                      "frac_of_hbm": moved / t / 1e9 / peak_gbs, "gflop": flops / 1e9, "tflops": flops / t / 1e12}
        if frames == 3:
            # the same three segments through the fused append entry point (rows in place: compress only), whose token split
            # fills the GPU where one CTA per (column tile, segment) leaves half of it idle
            import worldattention_b200 as wa
            hsa = wa.hsa.HSAAttention(HEADS, HEAD_DIM, block_size=block, proj_segment_len=FRAME_TOKENS).to(dev)
            with torch.no_grad():
                hsa.k_proj_mat.copy_(proj); hsa.v_proj_mat.copy_(proj)
            kc2, vc2 = torch.empty_like(kc), torch.empty_like(kc)
            ms2, _ = timed_steps(lambda: hsa.append_kv(k, v, k, v, kc2, vc2, position=0), steps, 3, flush)
            t2 = float(np.mean(ms2)) * 1e-3
            close = float((kc2.float() - kc.float()).abs().max())
            out["chunk_3_segments_fused_append"] = {"ms": t2 * 1e3, "gbs": moved / t2 / 1e9, "frac_of_hbm": moved / t2 / 1e9 / peak_gbs,
                                                    "max_abs_vs_compress_kv": close}
        del k, v
    out["hbm_peak_gbs"] = peak_gbs
    return out


# ------------------------------------------------------------------------------------------------
# HKV retrieval (benchmark config 3): per-head page scoring, top-16, gather; hot tier, cold tier, page centroids
# ------------------------------------------------------------------------------------------------
def bench_hkv(dev, steps=5, layers=30, pages_total=480, pages_hot=64, topk=16):
    """Score 480 page centroids per (layer, head), take the top-16 per head, gather those pages.

    The hot pool holds `pages_hot` pages per layer in HBM (`[layers, pages, 1560, H, D]` bf16, K and V);
    a selected page id maps to hot slot `id % pages_hot` (a synthetic residency map: the timing is that of
    a retrieval whose pages are all resident; `bench_hkv_cold` measures the other case).  Keys are re-rotated
    in flight, values copied verbatim.  Returns GB/s of the gather kernel against the algorithmic bytes
    (read + write of every selected page).
    """
    import worldattention_b200 as wa
    from worldattention_b200.hkv.install import gather_pages, per_head_records
    from worldattention_b200.hkv.retrieval import score_and_topk
    g = torch.Generator(device="cpu").manual_seed(3)
    page_tokens, row = FRAME_TOKENS, HEADS * HEAD_DIM
    pool = torch.empty((2, layers, pages_hot, page_tokens, HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    for i in range(2):
        for l in range(layers):                      # seeded on the device side in slices to bound host time
            pool[i, l].normal_(0, 1)
    offsets = torch.randn((layers, pages_total, row), generator=g) * 0.5
    centroids = offsets.to(dev)                      # page index: per-page mean key = per-page offset
    query = torch.randn((row,), generator=g).to(dev)
    cache = torch.zeros((2, layers, topk * page_tokens, HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    nt = wa.hkv.temporal_complex_dims(HEAD_DIM)
    rot = torch.randn((topk, nt, 2), generator=g)
    rot = (rot / rot.norm(dim=-1, keepdim=True)).to(dev).contiguous()
    esz = 2
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gather_ms, total_ms = [], []
    for it in range(steps + 2):
        torch.cuda.synchronize()
        ev0.record()
        ids = torch.empty((layers, HEADS, topk), dtype=torch.int32, device=dev)
        for l in range(layers):
            _, top, _ = score_and_topk(query, centroids[l], topk, groups=HEADS)
            ids[l] = top
        ids_h = ids.cpu().numpy()
        chron = np.sort(ids_h, axis=-1)              # install in chronological (page id) order
        slots = chron % pages_hot
        rot_ids = np.broadcast_to(np.arange(topk, dtype=np.int32), slots.shape)
        common = dict(src_page_stride=page_tokens * row * esz, src_layer_stride=pages_hot * page_tokens * row * esz,
                      dst_layer_stride=topk * page_tokens * row * esz, page_tokens=page_tokens, heads=HEADS,
                      head_dim=HEAD_DIM, elem_size=esz)
        rec = np.concatenate([
            per_head_records(slots, src_base=pool[0].data_ptr(), dst_base=cache[0].data_ptr(), rot=rot_ids, **common),
            per_head_records(slots, src_base=pool[1].data_ptr(), dst_base=cache[1].data_ptr(), rot=None, **common)])
        rec_dev = torch.from_numpy(rec.view(np.uint8).reshape(-1)).to(dev)
        ev2.record()
        gather_pages(rec, max_tokens=page_tokens, row_elems=HEAD_DIM, head_dim=HEAD_DIM, dtype=torch.bfloat16,
                     device=dev, rotations=rot, n_temporal=nt, records_dev=rec_dev)
        ev3.record()
        ev1.record()
        ev1.synchronize()
        if it >= 2:
            gather_ms.append(ev2.elapsed_time(ev3))
            total_ms.append(ev0.elapsed_time(ev1))
    # ---- the same retrieval without the host in the loop: one scoring launch for all layers, records built on the
    # device from the device-resident ids (a table of page addresses stands for the residency map), one gather ----
    from worldattention_b200.hkv.install import build_records_device, gather_records_device
    from worldattention_b200.hkv.retrieval import score_and_topk_layers
    want_k, want_v = cache[0].clone(), cache[1].clone()
    page_stride = page_tokens * row * esz
    slot_of = torch.arange(pages_total, dtype=torch.int64, device=dev) % pages_hot
    src_k = pool[0].data_ptr() + slot_of * page_stride
    src_v = pool[1].data_ptr() + slot_of * page_stride
    layer_common = dict(src_layer_stride=pages_hot * page_stride, src_token_stride=row, dst_layer_stride=topk * page_stride,
                        dst_token_stride=row, page_tokens=page_tokens, head_dim=HEAD_DIM)
    dev_ms = []
    for it in range(steps + 2):
        cache.zero_()
        torch.cuda.synchronize()
        ev0.record()
        _, ids_dev, _ = score_and_topk_layers(query, centroids, topk, groups=HEADS)
        rec_k = build_records_device(ids_dev, src_k, dst=cache[0], rotate=True, **layer_common)
        rec_v = build_records_device(ids_dev, src_v, dst=cache[1], rotate=False, **layer_common)
        recs = torch.cat([rec_k, rec_v])
        gather_records_device(recs, max_tokens=page_tokens, row_elems=HEAD_DIM, head_dim=HEAD_DIM, dtype=torch.bfloat16,
                              rotations=rot, n_temporal=nt)
        ev1.record()
        ev1.synchronize()
        if it >= 2:
            dev_ms.append(ev0.elapsed_time(ev1))
    same_as_host_path = bool(torch.equal(cache[0], want_k) and torch.equal(cache[1], want_v))
    moved = 2.0 * 2 * layers * HEADS * topk * page_tokens * HEAD_DIM * esz     # K and V, read + write
    # spot check: first selected page of layer 0 / head 0, values are copied verbatim
    src0 = pool[1, 0, int(slots[0, 0, 0]), :, 0]
    ok = bool(torch.equal(cache[1, 0, :page_tokens, 0], src0))
    _, peak_gbs, _ = measured_peaks()
    gbs = moved / (float(np.mean(gather_ms)) * 1e-3) / 1e9
    return {"workload": f"c3: {layers} layers x {HEADS} heads, {pages_total} page centroids scored per head, top-{topk} pages "
                        f"of {page_tokens} tokens gathered from a {pages_hot}-page HBM-hot pool (every selected page resident), keys re-rotated",
            "gather_ms": float(np.mean(gather_ms)), "gather_gbs": gbs, "hbm_peak_gbs": peak_gbs,
            "gather_frac_of_hbm": gbs / peak_gbs, "bytes_moved": moved, "retrieval_ms_end_to_end": float(np.mean(total_ms)),
            "retrieval_ms_device_resident": float(np.mean(dev_ms)), "device_resident_equals_host_path": same_as_host_path,
            "retrieval_gbs_device_resident": moved / (float(np.mean(dev_ms)) * 1e-3) / 1e9,
            "records": int(rec.shape[0]), "verbatim_value_check": ok}


def bench_hkv_centroids(dev, flush, pages=480, steps=5):
    """The page index of one layer built from real keys: 480 pages x 1560 tokens, keys ~ N(0,1) + a per-page offset
    ~ N(0, 0.5) so that page scores separate; the temporal rotation is removed on the fly.  Reads the layer's keys once."""
    import worldattention_b200 as wa
    from worldattention_b200.hkv.retrieval import page_key_index, score_and_topk
    _, peak_gbs, _ = measured_peaks()
    tokens = pages * FRAME_TOKENS
    g = torch.Generator(device=dev).manual_seed(3)
    keys = torch.empty((1, tokens, HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    offsets = torch.randn((pages, HEADS, HEAD_DIM), generator=g, device=dev) * 0.5
    for p0 in range(0, pages, 40):
        p1 = min(pages, p0 + 40)
        block = torch.randn((p1 - p0, FRAME_TOKENS, HEADS, HEAD_DIM), generator=g, device=dev) + offsets[p0:p1, None]
        keys[0, p0 * FRAME_TOKENS: p1 * FRAME_TOKENS] = block.reshape(-1, HEADS, HEAD_DIM).to(torch.bfloat16)
    nt = wa.hkv.temporal_complex_dims(HEAD_DIM)
    pairs = HEAD_DIM // 2
    inv = 1.0 / (10000.0 ** (torch.arange(nt, dtype=torch.float64) / pairs))
    freqs = torch.polar(torch.ones(1024, nt, dtype=torch.float64), torch.outer(torch.arange(1024, dtype=torch.float64), inv))
    spans = [(p * FRAME_TOKENS, (p + 1) * FRAME_TOKENS) for p in range(pages)]

    # the kernel alone: the rotation table and the page spans are built and uploaded once, outside the timed region (the
    # Python entry point rebuilds them per call, on the host, which is not what this number is about)
    from worldattention_b200 import _lib
    from worldattention_b200.hkv.rope import rotation_table
    frames = np.arange(pages)
    rot = torch.from_numpy(rotation_table(freqs, np.zeros_like(frames), frames, nt)).to(dev)
    spans_dev = torch.tensor(spans, dtype=torch.int32).to(dev)
    out = torch.empty((pages, HEADS * HEAD_DIM), device=dev, dtype=torch.float32)

    def step():
        _lib.check(_lib.lib().wa_hkv_page_centroids(_lib.t4_blhd(keys), 1, tokens, HEADS, HEAD_DIM, spans_dev.data_ptr(), pages,
                                                    rot.data_ptr(), pages, nt, FRAME_TOKENS, out.data_ptr(), _lib.stream_ptr(dev)))
    ms, _ = timed_steps(step, steps, 2, flush)
    index = page_key_index(keys, spans, frame_seq_length=FRAME_TOKENS, start_frame=0, temporal_freqs=freqs)
    same = bool(torch.equal(index, out))
    # a query made of page 100's own offset must rank page 100 first in every head
    query = offsets[100].reshape(-1)
    _, ids, _ = score_and_topk(query, index, 16, groups=HEADS)
    own = bool((ids[:, 0] == 100).all().item())
    t = float(np.mean(ms)) * 1e-3
    moved = float(keys.numel() * 2)
    return {"pages": pages, "tokens": tokens, "ms": t * 1e3, "bytes_read": moved, "gbs": moved / t / 1e9, "frac_of_hbm": moved / t / 1e9 / peak_gbs,
            "hbm_peak_gbs": peak_gbs, "a_page_s_offset_retrieves_that_page": own, "equals_the_python_entry_point": same}


def bench_config4(dev, chunks):
    """Benchmark config 4: autoregressive generation with a random-init Wan2.1-T2V-1.3B-architecture DiT (30 blocks, dim
    1536, 12 heads, FFN 8960, bf16), 480 x 832 latents, chunks of 3 latent frames, 4 denoising forwards + 1 clean-context
    forward per chunk, HSA over a rolling 21-frame window (128-token blocks, per-head block counts drawn from
    {4, 8, 16, 32} as in config 2), synthetic 512 x 4096 prompt embeddings, and a prompt switch served from the HKV bank
    every 8 chunks (pages of 3 frames, top-4 pages, up to twelve banked windows (6 GB each) kept in HBM, older ones in pinned host memory).  Text encoder and VAE are outside the timed region; frames are
    latent frames.  Everything around the attention layer is plain torch (cuBLAS GEMMs, library cross-attention)."""
    from worldattention_b200.causal_dit import DiTConfig, time_generation
    rng = np.random.default_rng(1)
    cfg = DiTConfig(hsa_topk=[int(v) for v in rng.choice([4, 8, 16, 32], size=12)])
    kwargs = dict(chunks=chunks, switch_every_chunks=8, device=dev,
                  hkv_kwargs=dict(page_size_frames=3, topk_pages=4, cpu_max_chunks=64, hbm_max_chunks=12))
    try:
        res = time_generation(cfg, cuda_graph=True, **kwargs)      # steady-state chunks replayed from one captured graph
        torch.cuda.empty_cache()
        eager = time_generation(cfg, cuda_graph=False, **kwargs)
        res["launch_by_launch"] = {k: eager[k] for k in ("frames_per_s", "frames_per_s_steady", "chunk_ms_median_second_half", "wall_s")}
    except torch.OutOfMemoryError as exc:      # reported, not hidden: the harness needs about 12 GB
        return {"error": f"out of memory: {exc}"}
    res["workload"] = ("c4: 30-block DiT (dim 1536, 12 heads, FFN 8960), 1560 tokens/frame, 3-frame chunks, 4+1 forwards per chunk, "
                       f"{chunks} chunks (80 in the benchmark definition), HSA window 21 frames, HKV switch every 8 chunks")
    res["unit"] = "latent frames/s"
    return res


def bench_hkv_cold(dev, layers=2, pages_total=480, pages_hot=64, topk=16, steps=4):
    """Config 3 with its residency: pages 0..63 of every layer in HBM, the other 416 in page-locked host memory.

    Per retrieval: all layers scored in one launch, the ids read back (the host drives the DMA engine, so it has to
    know them), every selected cold page-of-one-head queued as one host-to-device copy on a side stream
    (`wa_hkv_promote_pages`; cold pages are stored head-major so that such a slice is one contiguous block) into a
    staging buffer, an event, and ONE gather launch that installs hot pages from the pool and promoted pages from
    the staging buffer.  The promotion is bound by the host link, not by HBM: its rate is reported against a plain
    page-locked copy measured here.  Fewer layers than the 30 of config 3 bound the page-locked allocation
    (416 cold pages x 30 layers would pin 120 GB); the rate does not depend on the layer count.
    """
    import worldattention_b200 as wa
    from worldattention_b200 import _lib
    from worldattention_b200.hkv.install import RECORD_DTYPE, gather_pages
    from worldattention_b200.hkv.retrieval import score_and_topk_layers
    lib = _lib.lib()
    page_tokens, row, esz = FRAME_TOKENS, HEADS * HEAD_DIM, 2
    pages_cold = pages_total - pages_hot
    g = torch.Generator().manual_seed(3)
    hot = torch.empty((2, layers, pages_hot, page_tokens, HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    hot.normal_(0, 1)
    t0 = time.perf_counter()
    cold = torch.empty((2, layers, pages_cold, HEADS, page_tokens, HEAD_DIM), dtype=torch.bfloat16, pin_memory=True)   # head-major
    pin_s = time.perf_counter() - t0
    seed_page = torch.randn((HEADS, page_tokens, HEAD_DIM), generator=g).to(torch.bfloat16)
    for i in range(2):
        for l in range(layers):
            for p in range(pages_cold):   # cheap to fill, and every page distinct: a page's first element names it
                cold[i, l, p] = seed_page
                cold[i, l, p, :, 0, 0] = float(p % 256)
    centroids = (torch.randn((layers, pages_total, row), generator=g) * 0.5).to(dev)
    query = torch.randn((row,), generator=g).to(dev)
    cache = torch.zeros((2, layers, topk * page_tokens, HEADS, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    staging = torch.empty((2, layers, HEADS, topk, page_tokens, HEAD_DIM), dtype=torch.bfloat16, device=dev)
    nt = wa.hkv.temporal_complex_dims(HEAD_DIM)
    rot = torch.randn((topk, nt, 2), generator=g)
    rot = (rot / rot.norm(dim=-1, keepdim=True)).to(dev).contiguous()
    side = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    # the denominator: a plain page-locked host-to-device copy of 256 MiB
    probe_h = torch.empty(256 << 20, dtype=torch.uint8, pin_memory=True)
    probe_d = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    link = []
    for it in range(4):
        e0.record(); probe_d.copy_(probe_h, non_blocking=True); e1.record(); e1.synchronize()
        if it:
            link.append(probe_h.numel() / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    link_gbs = float(np.median(link))
    del probe_h, probe_d

    page_bytes_head = page_tokens * HEAD_DIM * esz
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    total_ms, promote_ms, n_cold_pages = [], [], 0
    for it in range(steps + 1):
        cache.zero_()
        torch.cuda.synchronize()
        ev[0].record()
        _, ids_dev, _ = score_and_topk_layers(query, centroids, topk, groups=HEADS)
        ids = np.sort(ids_dev.cpu().numpy(), axis=-1)                      # [layers, heads, topk], chronological
        is_cold = ids >= pages_hot
        # records as arrays: [K|V, layer, head, rank]
        kv, ll, hh, rr = np.meshgrid(np.arange(2), np.arange(layers), np.arange(HEADS), np.arange(topk), indexing="ij")
        page = np.broadcast_to(ids[None], kv.shape)
        coldm = page >= pages_hot
        dst = np.where(kv == 0, cache[0].data_ptr(), cache[1].data_ptr()) + ((ll * topk * page_tokens + rr * page_tokens) * row + hh * HEAD_DIM) * esz
        stage = staging.data_ptr() + ((((kv * layers + ll) * HEADS + hh) * topk + rr) * page_bytes_head)
        src_host = cold.data_ptr() + ((((kv * layers + ll) * pages_cold + (page - pages_hot)) * HEADS + hh) * page_bytes_head)
        src_hot = hot.data_ptr() + (((kv * layers + ll) * pages_hot + page) * page_tokens * row + hh * HEAD_DIM) * esz
        records = np.zeros(kv.size, dtype=RECORD_DTYPE)
        records["src"] = np.where(coldm, stage, src_hot).reshape(-1).astype(np.uint64)
        records["dst"] = dst.reshape(-1).astype(np.uint64)
        records["src_stride"] = np.where(coldm, HEAD_DIM, row).reshape(-1)
        records["dst_stride"] = row
        records["n_tokens"] = page_tokens
        records["rot"] = np.where(kv == 0, rr, -1).reshape(-1)
        promote = np.zeros(int(coldm.sum()), dtype=RECORD_DTYPE)
        promote["src"] = src_host[coldm].astype(np.uint64)
        promote["dst"] = stage[coldm].astype(np.uint64)
        promote["src_stride"] = promote["dst_stride"] = HEAD_DIM
        promote["n_tokens"] = page_tokens
        promote["rot"] = -1
        side.wait_stream(main)
        ev[1].record(side)
        _lib.check(lib.wa_hkv_promote_pages(promote.ctypes.data, len(promote), HEAD_DIM, esz, side.cuda_stream))
        ev[2].record(side)
        main.wait_stream(side)
        gather_pages(records, max_tokens=page_tokens, row_elems=HEAD_DIM, head_dim=HEAD_DIM, dtype=torch.bfloat16, device=dev,
                     rotations=rot, n_temporal=nt)
        ev[3].record()
        ev[3].synchronize()
        if it >= 1:
            total_ms.append(ev[0].elapsed_time(ev[3]))
            promote_ms.append(ev[1].elapsed_time(ev[2]))
            n_cold_pages = len(promote)
    # verbatim check of the values (layer 0, head 0): every installed page, hot or promoted, equals its source rows
    ok = True
    for r in range(topk):
        page_id = int(ids[0, 0, r])
        got = cache[1, 0, r * page_tokens:(r + 1) * page_tokens, 0]
        want = cold[1, 0, page_id - pages_hot, 0].to(dev) if page_id >= pages_hot else hot[1, 0, page_id, :, 0]
        ok = ok and bool(torch.equal(got, want))
    promoted_bytes = float(n_cold_pages) * page_bytes_head
    pm = float(np.mean(promote_ms)) * 1e-3
    installed = 2.0 * layers * HEADS * topk * page_bytes_head
    return {"workload": f"c3 residency: {layers} layers (of 30) x {HEADS} heads, pages 0..{pages_hot - 1} in HBM, {pages_cold} in page-locked "
                        f"host memory ({cold.numel() * 2 / 1e9:.1f} GB pinned in {pin_s:.1f} s), top-{topk} per head",
            "selected_pages": int(ids.size), "cold_fraction": float(is_cold.mean()),
            "promoted_bytes": promoted_bytes, "promotion_ms": pm * 1e3, "promotion_gbs": promoted_bytes / pm / 1e9,
            "host_link_gbs_plain_copy": link_gbs, "promotion_frac_of_host_link": promoted_bytes / pm / 1e9 / link_gbs,
            "retrieval_ms": float(np.mean(total_ms)), "installed_bytes": installed,
            "retrieval_gbs_installed": installed / (float(np.mean(total_ms)) * 1e-3) / 1e9,
            "copies_per_retrieval": n_cold_pages, "verbatim_value_check": ok,
            "note": "bound by the host link, not HBM; ids are read back because the host queues the copies"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--force-generic", action="store_true")
    ap.add_argument("--no-hkv", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip block64 / long_horizon / compress / triton_incumbent")
    ap.add_argument("--c4-chunks", type=int, default=80,
                    help="chunks generated by the end-to-end harness (80 = benchmark config 4; 0 skips it)")
    ap.add_argument("--hkv-only", action="store_true", help="run only the HKV retrieval measurements (one GPU)")
    ap.add_argument("--hkv-layers", type=int, default=30, help="layers in the hot HKV measurement (30 = benchmark config 3)")
    ap.add_argument("--hkv-cold-layers", type=int, default=2, help="layers in the cold-tier HKV measurement")
    ap.add_argument("--shard", default="auto", choices=["auto", "heads", "kv"], help="sharding for --gpus > 1")
    ap.add_argument("--exchange", default="auto", choices=["auto", "nccl", "peer"],
                    help="kv sharding: how the partial records reach the merging rank (peer = stored by the attention kernel "
                         "into the peers' buffers over NVLink; nccl = one all-to-all; auto = peer where it applies)")
    ap.add_argument("--gather-heads", action="store_true",
                    help="head split: also all-gather the outputs (off: they stay head-sharded for a head-parallel consumer)")
    ap.add_argument("--triton-incumbent-child", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.triton_incumbent_child:
        triton_incumbent_child()
        return
    if args.impl == "reference":
        reference_arm(args)
        return
    if args.hkv_only:
        torch.cuda.set_device(0)
        dev0 = torch.device("cuda", 0)
        print(json.dumps({"metric": "hkv_gather_gbs", "hkv": bench_hkv(dev0, layers=args.hkv_layers),
                          "hkv_cold": bench_hkv_cold(dev0, layers=args.hkv_cold_layers),
                          "hkv_centroids": bench_hkv_centroids(dev0, Flusher(dev0))}), flush=True)
        return
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist

    import worldattention_b200 as wa
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = wa._lib.lib()
    spec = WORKLOADS[args.workload]
    block = spec["block"]

    work = Work(args.workload, dev, world, rank, shard=args.shard, force_generic=args.force_generic,
                gather_heads=args.gather_heads, exchange=args.exchange)
    mode, hsa = work.mode, work.hsa
    q, k, v, kc, vc = work.q, work.k, work.v, work.kc, work.vc
    q_h, k_h, v_h = work.q_h, work.k_h, work.v_h
    q_len, kv_len = work.q_len, work.kv_len
    flush_l2 = Flusher(dev)
    forward = work.forward

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- routing statistics for the FLOP count (untimed) ---------------------------------------
    sparse_f, linear_f, gate_f = work.flops()
    used_tuned = work.used_tuned

    # ---- device-resident timing ------------------------------------------------------------------
    # warm-up steps are what the timed steps are: L2 flushed, the kernel's event bracket on, the clock sampler running
    lib.wa_profile_enable(1)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        flush_l2()
        forward()
    barrier()
    sampler.mark()
    launches0 = lib.wa_launch_count()
    barrier()
    wall0 = time.perf_counter()
    step_ms, kern_ms = timed_steps(forward, args.steps, 0, flush_l2, lib)
    barrier()
    wall = time.perf_counter() - wall0
    launches = lib.wa_launch_count() - launches0
    lib.wa_profile_enable(0)
    total_ms = max_over_ranks(sum(step_ms), dev, world)
    ms_per_step = total_ms / args.steps
    step_stats = {"median_ms_rank0": float(np.median(step_ms)), "min_ms_rank0": float(np.min(step_ms)),
                  "max_ms_rank0": float(np.max(step_ms)), "slowest_step": int(np.argmax(step_ms))}     # spread of the timed steps (the headline is their mean)
    wa._lib.raise_if_failed(dev)          # a bounded wait that ran out inside the kernel would have left its code here

    # ---- N > 1: the sharded result against the single-GPU call (untimed) ------------------------------
    equals_single = work.check_against_single_gpu() if world > 1 else None

    # ---- KV-sharded runs: the head split on the same ranks, for comparison (extra, not the headline) ------------------
    head_split_alt = None
    if mode == "kv" and HEADS >= world:
        plan_a = work.sharded.plan_head_split(HEADS, world, work.topk_all.tolist())
        mine_a = plan_a[rank]
        # every rank drew the same host tensors, so the head slice is cut from a local device copy of the full keys
        k_all, v_all = k_h.to(dev), v_h.to(dev)
        qa, ka, va = (x[:, :, mine_a].contiguous() for x in (q, k_all, v_all))
        del k_all, v_all
        with torch.no_grad():
            kca, vca = hsa.compress_kv_cache(ka, va)
        topk_a = work.topk_all[mine_a].to(dev)

        def forward_alt():
            with torch.no_grad():
                return wa.hsa.hsa_attention(qa, ka, va, k_coarse=kca, v_coarse=vca, k_proj_mat=hsa.k_proj_mat,
                                            v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin, block_size=block,
                                            proj_segment_len=FRAME_TOKENS, topk_per_head=topk_a)
        barrier()
        alt_ms, _ = timed_steps(forward_alt, min(args.steps, 30), 3, flush_l2)
        head_split_alt = {"sharding": "head-split, uneven (longest-processing-time on the per-head top-k), no collective",
                          "heads_per_rank": [len(x) for x in plan_a],
                          "ms_per_step": max_over_ranks(float(np.mean(alt_ms)), dev, world)}
        del qa, ka, va, kca, vca

    # ---- the same step with the pooled keys of the cached frames kept by the caller (extra, not the headline) -------
    # In the causal pipeline only the chunk's own rows of the key cache change between forwards; the block means of
    # the older frames can stay resident next to the compressed cache, and the call then pools the new blocks only.
    pooled_cache = None
    if mode == "single" and not args.force_generic:
        n_blocks = -(-kv_len // block)
        valid = (kv_len - q_len) // block
        k_pool = torch.empty((1, HEADS, n_blocks, HEAD_DIM), dtype=torch.float32, device=dev)

        def forward_cached(valid_blocks):
            with torch.no_grad():
                return wa.hsa.hsa_attention(q, k, v, k_coarse=kc, v_coarse=vc, k_proj_mat=hsa.k_proj_mat,
                                            v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin, block_size=block,
                                            proj_segment_len=FRAME_TOKENS, topk_per_head=work.topk,
                                            k_pooled_cache=k_pool, k_pooled_valid=valid_blocks)
        same = bool(torch.equal(forward_cached(0), forward()))   # fills the buffer; the result does not change
        pc_ms, _ = timed_steps(lambda: forward_cached(valid), min(args.steps, 50), 3, flush_l2)
        same = same and bool(torch.equal(forward_cached(valid), forward()))
        pooled_cache = {"ms_per_step": float(np.mean(pc_ms)), "trusted_blocks": int(valid), "pooled_blocks": int(n_blocks - valid),
                        "equals_plain_call": same}

    # ---- end to end through the public API with host buffers ------------------------------------
    # Per step: the chunk's q and its new K/V rows arrive from page-locked host memory, the rows are written at the tail
    # of the resident cache and compressed into the tail of the compressed cache, the layer runs, and the output returns
    # to page-locked host memory.
    new = q_len
    out_shape = tuple(forward().shape)
    out_rows = slice(0, out_shape[1])
    if mode == "kv":
        # every rank ends up with the whole output; the rows a rank merged are the ones it hands back, so that the output
        # reaches the host once (the head split returns each rank's heads in the same way)
        first_row, n_rows = work.sharded.exchange_rows(q_len, world)[1][rank]
        out_rows = slice(first_row, first_row + n_rows)
        out_shape = (out_shape[0], n_rows) + out_shape[2:]
    out_h = torch.empty(out_shape, dtype=torch.bfloat16, pin_memory=True)
    q_new_h, k_new_h, v_new_h = q_h, k_h[:, kv_len - new:].contiguous().pin_memory(), v_h[:, kv_len - new:].contiguous().pin_memory()
    h2d = (q_new_h.numel() + (k_new_h.numel() + v_new_h.numel() if mode != "kv" else 0)) * 2
    d2h = out_h.numel() * 2

    def append_chunk(k_cache, v_cache, kc_cache, vc_cache, k_rows, v_rows):
        """The chunk's rows go from page-locked host memory to the cache tail; their compressed slots follow."""
        k_cache[:, kv_len - new:].copy_(k_rows, non_blocking=True)
        v_cache[:, kv_len - new:].copy_(v_rows, non_blocking=True)
        # the rows are in place: one launch compresses the three new segments into the tail of the compressed cache
        hsa.append_kv(k_cache[:, kv_len - new:], v_cache[:, kv_len - new:], k_cache, v_cache, kc_cache, vc_cache,
                      position=kv_len - new)

    # One GPU: the heads are independent, so the step is pipelined over head groups on separate streams -- group g+1's
    # rows cross PCIe while group g computes and group g-1's output returns (the copies are most of the step).
    # (four groups of three heads measured 1.16 ms on a box where three groups took 1.22-1.25 and six 1.23)
    E2E_GROUPS = int(os.environ.get("WA_E2E_GROUPS", "4")) if mode == "single" else 1
    # outputs leave as soon as they exist (0: only after the last group's rows have arrived; with four groups that
    # measured 1.12-1.14 ms against 1.10-1.12 ms, pairwise on one box)
    E2E_EARLY_OUT = os.environ.get("WA_E2E_EARLY_OUT", "1") == "1"
    e2e_note = "one stream: copy in, compress the new segments (one fused launch), layer, copy out"
    if mode == "kv":
        e2e_note = ("one stream per rank: q copied in on every rank (the shards' K/V rows are resident), the sharded layer, each "
                    "rank copies out the rows it merged; bytes are rank 0's")
    if E2E_GROUPS > 1:
        hg = HEADS // E2E_GROUPS
        e2e_note = (f"{E2E_GROUPS} head groups of {hg} heads, each with its own resident cache tensors and stream: copy in, "
                    f"compress the new segments (one fused launch), layer (`hsa_attention` on the group's heads), copy out; groups overlap")
        streams = [torch.cuda.Stream(device=dev) for _ in range(E2E_GROUPS)]
        done = [torch.cuda.Event() for _ in range(E2E_GROUPS)]
        arrived = [torch.cuda.Event() for _ in range(E2E_GROUPS)]
        grp = []
        for g in range(E2E_GROUPS):
            hs = slice(g * hg, (g + 1) * hg)
            # the group's resident state lives in tensors of its own ([B, L, H/G, D], heads of the group only), so the
            # rows that arrive land with plain contiguous copies
            grp.append(dict(
                q_h=q_new_h[:, :, hs].contiguous().pin_memory(), k_h=k_new_h[:, :, hs].contiguous().pin_memory(),
                v_h=v_new_h[:, :, hs].contiguous().pin_memory(),
                out_h=torch.empty((1, q_len, hg, HEAD_DIM), dtype=torch.bfloat16, pin_memory=True),
                q=q[:, :, hs].contiguous(), k=k[:, :, hs].contiguous(), v=v[:, :, hs].contiguous(),
                kc=kc[:, :, hs].contiguous(), vc=vc[:, :, hs].contiguous(),
                topk=work.topk[hs].contiguous()))

    def e2e_step_grouped():
        start = torch.cuda.Event()
        start.record()
        for g, st in enumerate(streams):
            d = grp[g]
            with torch.cuda.stream(st), torch.no_grad():
                st.wait_event(start if g == 0 else arrived[g - 1])   # one group's rows at a time on the link
                d["q"].copy_(d["q_h"], non_blocking=True)
                d["k"][:, kv_len - new:].copy_(d["k_h"], non_blocking=True)
                d["v"][:, kv_len - new:].copy_(d["v_h"], non_blocking=True)
                arrived[g].record(st)
                hsa.append_kv(d["k"][:, kv_len - new:], d["v"][:, kv_len - new:], d["k"], d["v"], d["kc"], d["vc"],
                              position=kv_len - new)
                out = wa.hsa.hsa_attention(d["q"], d["k"], d["v"], k_coarse=d["kc"], v_coarse=d["vc"],
                                           k_proj_mat=hsa.k_proj_mat, v_proj_mat=hsa.v_proj_mat, gate_lin=hsa.gate_lin,
                                           block_size=block, proj_segment_len=FRAME_TOKENS, topk_per_head=d["topk"],
                                           force_generic=args.force_generic)
                d["out"] = out
        # the copies out: large copies in both directions overlap on this link
        for g, st in enumerate(streams):
            d = grp[g]
            with torch.cuda.stream(st):
                if not E2E_EARLY_OUT:
                    st.wait_event(arrived[E2E_GROUPS - 1])
                d["out_h"].copy_(d["out"], non_blocking=True)
                done[g].record(st)
        for ev in done:
            torch.cuda.current_stream().wait_event(ev)

    def e2e_step():
        if E2E_GROUPS > 1:
            return e2e_step_grouped()
        q.copy_(q_new_h, non_blocking=True)
        if mode != "kv":
            with torch.no_grad():
                append_chunk(k, v, kc, vc, k_new_h, v_new_h)
        out = forward()
        out_h.copy_(out[:, out_rows], non_blocking=True)

    e2e_ms, _ = timed_steps(e2e_step, args.steps, 2, flush_l2)
    e2e_same = None
    if E2E_GROUPS > 1:   # untimed: the pipelined step produces what the single call produces
        torch.cuda.synchronize()
        whole = forward().cpu()
        e2e_same = bool(torch.equal(torch.cat([d["out_h"] for d in grp], dim=2), whole))
        del grp
    e2e_total = max_over_ranks(sum(e2e_ms), dev, world)
    e2e_value = args.steps / (e2e_total * 1e-3)
    clocks = sampler.stop() if rank == 0 else None
    wa._lib.raise_if_failed(dev)

    # ---- the long-horizon cache (config 5) sharded the way the headline is: the configuration the sharding is for -----
    extras = {}
    exchange_used = work.exchange_used
    if not args.no_extras and not args.force_generic:
        del work, q, k, v, kc, vc, forward
        torch.cuda.empty_cache()
        if args.workload != "c5":
            extras["long_horizon"] = side_workload("c5", dev, world, rank, lib, flush_l2, steps=10,
                                                   shard=args.shard, on_device=True, exchange=args.exchange)
        if world == 1 and args.workload != "c2-64":
            extras["block64"] = side_workload("c2-64", dev, 1, 0, lib, flush_l2, steps=30)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak_tf, peak_gbs, peak_src = measured_peaks()
    flops = sparse_f + (linear_f + gate_f if used_tuned else 0.0)
    kernel_ms = float(np.mean(kern_ms)) if kern_ms else None
    achieved = flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms else None
    line = {
        "metric": "hsa_fwd_chunks_per_s", "value": args.steps / (total_ms * 1e-3), "unit": "chunks/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(args.workload, world, mode),
        "roofline": {
            "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
            "frac": (achieved / peak_tf) if achieved else None,
            "traffic": NCU_TRAFFIC_BYTES if (used_tuned and world == 1 and args.workload == "c2") else None,
            "peak_source": peak_src,
            "kernel": (f"hsa_fwd_sm100 (tcgen05: sparse + linear + gate{'; partial-output mode, rank 0' if mode == 'kv' else ''})"
                       if used_tuned else "generic_attention_kernel (SIMT sparse branch)"),
            "kernel_ms": kernel_ms,
            "flops": {"sparse": sparse_f, "linear": linear_f, "gate": gate_f, "counted": flops},
            "sparse_only_frac": (sparse_f / (kernel_ms * 1e-3) / 1e12 / peak_tf) if kernel_ms else None,
        },
        "e2e": {"value": e2e_value, "unit": "chunks/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_total / args.steps, "how": e2e_note, "equals_single_call": e2e_same},
        "gpu_launches": int(launches),
        "pooled_key_cache": pooled_cache,
        "head_split_on_the_same_ranks": head_split_alt,
        "equals_single_gpu": equals_single,
        "exchange": exchange_used,
        "step_spread": step_stats,
        "clocks": clocks,
        "wall_s": wall,
    }
    line.update(extras)
    if world == 1 and not args.no_extras and not args.force_generic:
        line["compress_kv"] = bench_compress(dev, flush_l2, block)
        line["triton_incumbent"] = bench_triton_incumbent()
    if world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        value, ms, kind, what = run_cpu(spec, steps=1, warmup=0)
        line["cpu_baseline"] = {"value": value, "unit": "chunks/s", "cores": cores, "kind": kind, "sample": what + "; one step, no warm-up",
                                "ms_per_chunk": ms}
    if world == 1 and not args.no_hkv:
        del flush_l2
        torch.cuda.empty_cache()
        line["hkv"] = bench_hkv(dev, layers=args.hkv_layers)
        torch.cuda.empty_cache()
        line["hkv"]["cold_tier"] = bench_hkv_cold(dev, layers=args.hkv_cold_layers)
        torch.cuda.empty_cache()
        line["hkv"]["page_centroids"] = bench_hkv_centroids(dev, Flusher(dev))
    if world == 1 and not args.no_extras and not args.force_generic and args.c4_chunks > 0:
        torch.cuda.empty_cache()
        line["config4"] = bench_config4(dev, args.c4_chunks)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
