"""Multi-tier residency for KV chunk blobs: HBM (hot) -> pinned host DRAM -> NVMe.

Keeps the interface of the reference's `HKVTierManager` (pipeline/hkv/tiering.py): `put`, `get`,
`location`, `stats`, `cleanup`, LRU migration, a full NVMe backup of anything ever spilled.  Two
additions: an optional HBM tier in front (`hbm_max_chunks`, off by default so that behaviour
matches the reference: a fresh chunk is host-resident), and host copies live in page-locked memory
so that demotion and promotion are asynchronous DMA transfers on a side stream.

A blob is a dict of tensor lists, e.g. `{"k": [per-layer tensors], "v": [...]}`.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from typing import Dict, Optional

import torch

__all__ = ["HKVTierManager"]


def _map_blob(blob: dict, fn) -> dict:
    return {key: [fn(t) for t in tensors] for key, tensors in blob.items()}


class HKVTierManager:
    """Track per-chunk KV blobs across HBM, host DRAM and NVMe with LRU migration.

    Args:
        cpu_max_chunks: host-resident chunk capacity (floored at 1).
        nvme_enabled: spill over-capacity host chunks to disk instead of dropping them.
        nvme_dir: directory for spilled chunks; required when `nvme_enabled`.
        hbm_max_chunks: chunks kept resident on the GPU in front of the host tier (0 disables).
        pin_host: allocate host copies in page-locked memory when a CUDA device is present.
    """

    def __init__(self, cpu_max_chunks: int, nvme_enabled: bool = False, nvme_dir: Optional[str] = None,
                 hbm_max_chunks: int = 0, pin_host: bool = True):
        self.cpu_max_chunks = max(int(cpu_max_chunks), 1)
        self.hbm_max_chunks = max(int(hbm_max_chunks), 0)
        self.nvme_enabled = bool(nvme_enabled)
        self.nvme_dir = nvme_dir
        self.pin_host = bool(pin_host)
        if self.nvme_enabled:
            if not nvme_dir:
                raise ValueError("nvme_dir is required when nvme_enabled=True")
            os.makedirs(nvme_dir, exist_ok=True)
        self._hbm: "OrderedDict[int, dict]" = OrderedDict()
        self._cpu: "OrderedDict[int, dict]" = OrderedDict()
        self._nvme: Dict[int, str] = {}
        self._backup: Dict[int, str] = {}
        self._side_stream = None
        self.n_spills = 0
        self.n_loads = 0
        self.n_drops = 0
        self.n_demotions = 0
        self.n_hbm_hits = 0
        self.n_host_hits = 0

    # ------------------------------------------------------------------ helpers
    def _path(self, chunk_id: int) -> str:
        return os.path.join(self.nvme_dir, f"hkv_chunk_{chunk_id}.pt")

    def side_stream(self, device: torch.device):
        """The stream demotions and promotions run on, created on first use."""
        if self._side_stream is None or self._side_stream.device != device:
            self._side_stream = torch.cuda.Stream(device=device)
        return self._side_stream

    def _to_host(self, blob: dict) -> dict:
        """Device blob -> host blob; page-locked and asynchronous when possible."""
        first = next(iter(blob.values()))[0]
        if not first.is_cuda:
            return blob
        device = first.device
        side = self.side_stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            def copy(t):
                host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.pin_host)
                host.copy_(t, non_blocking=True)
                t.record_stream(side)
                return host
            host_blob = _map_blob(blob, copy)
        side.synchronize()   # the host copy must be complete before anyone reads or spills it
        return host_blob

    # ------------------------------------------------------------------ reference interface
    def put(self, chunk_id: int, blob: dict) -> None:
        """Register a freshly produced chunk in the hottest enabled tier."""
        self._nvme.pop(chunk_id, None)
        self._hbm.pop(chunk_id, None)
        self._cpu.pop(chunk_id, None)
        first = next(iter(blob.values()))[0]
        if self.hbm_max_chunks > 0 and first.is_cuda:
            self._hbm[chunk_id] = blob
        else:
            self._cpu[chunk_id] = self._to_host(blob)
        self._evict_if_needed()

    def get(self, chunk_id: int) -> Optional[dict]:
        """Return a chunk blob (device tensors when hot, host tensors otherwise), reloading from NVMe."""
        if chunk_id in self._hbm:
            self._hbm.move_to_end(chunk_id)
            self.n_hbm_hits += 1
            return self._hbm[chunk_id]
        if chunk_id in self._cpu:
            self._cpu.move_to_end(chunk_id)
            self.n_host_hits += 1
            return self._cpu[chunk_id]
        if chunk_id in self._nvme:
            blob = torch.load(self._nvme[chunk_id], map_location="cpu", weights_only=False)
            if self.pin_host and torch.cuda.is_available():
                blob = _map_blob(blob, lambda t: t.pin_memory())
            self.n_loads += 1
            self._cpu[chunk_id] = blob
            self._nvme.pop(chunk_id, None)
            self._evict_if_needed()
            return blob
        return None

    def location(self, chunk_id: int) -> str:
        """Current tier of a chunk: `"hbm"`, `"cpu"`, `"nvme"` or `"absent"`."""
        if chunk_id in self._hbm:
            return "hbm"
        if chunk_id in self._cpu:
            return "cpu"
        if chunk_id in self._nvme:
            return "nvme"
        return "absent"

    def _evict_if_needed(self) -> None:
        while len(self._hbm) > self.hbm_max_chunks:
            victim, blob = self._hbm.popitem(last=False)
            self._cpu[victim] = self._to_host(blob)
            self.n_demotions += 1
        while len(self._cpu) > self.cpu_max_chunks:
            victim, blob = self._cpu.popitem(last=False)
            if self.nvme_enabled:
                path = self._backup.get(victim) or self._path(victim)
                if victim not in self._backup:
                    torch.save(blob, path)
                    self._backup[victim] = path
                self._nvme[victim] = path
                self.n_spills += 1
            else:
                self.n_drops += 1

    def stats(self) -> dict:
        return {
            "cpu_resident": len(self._cpu),
            "nvme_resident": len(self._nvme),
            "backups": len(self._backup),
            "n_spills": self.n_spills,
            "n_loads": self.n_loads,
            "n_drops": self.n_drops,
            "hbm_resident": len(self._hbm),
            "n_demotions": self.n_demotions,
            "n_hbm_hits": self.n_hbm_hits,
            "n_host_hits": self.n_host_hits,
        }

    def cleanup(self) -> None:
        """Delete spilled files and clear all bookkeeping."""
        for path in set(list(self._backup.values()) + list(self._nvme.values())):
            try:
                os.remove(path)
            except OSError:
                pass
        self._hbm.clear()
        self._cpu.clear()
        self._nvme.clear()
        self._backup.clear()
