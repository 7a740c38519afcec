"""Residency of KV chunk blobs across three tiers: HBM (hot) -> page-locked host DRAM -> files on NVMe.

Same interface as the reference's `HKVTierManager` (pipeline/hkv/tiering.py:18-127) -- `put`, `get`,
`location`, `stats`, `cleanup`; least-recently-used chunks move down a tier when the one above is full; a
chunk that has been written to disk once keeps that file as its backup, so spilling it again costs nothing
-- with three changes in how the bytes move:

* an optional HBM tier in front (`hbm_max_chunks`; 0 keeps the reference behaviour: a fresh chunk is
  host-resident);
* host copies live in page-locked memory and a demotion is an asynchronous DMA on a side stream: `put`
  returns while the copy runs, and whoever needs the host bytes first (`get`, a spill) waits for that
  chunk's copy only;
* the disk format is not a pickled blob but a raw, page-addressable file (`ChunkFile`): a small JSON
  header and every tensor's bytes at a 4 KiB-aligned offset, so `read_rows` brings one page of one
  layer straight into a page-locked buffer without loading the rest of the chunk
  (reference: whole-chunk `torch.save` / `torch.load`, tiering.py:56-57, 72, 98).

A blob is a dict of tensor lists, e.g. `{"k": [per-layer [B, T, H, D] tensors], "v": [...]}`.
"""
from __future__ import annotations

import json
import os
import struct
from collections import OrderedDict
from typing import Dict, Optional

import torch

__all__ = ["HKVTierManager", "ChunkFile"]

_ALIGN = 4096
_MAGIC = b"HKVCHNK1"
_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16, "float64": torch.float64,
           "int32": torch.int32, "int64": torch.int64, "uint8": torch.uint8, "int8": torch.int8, "int16": torch.int16}


def _host_buffer(shape, dtype, pinned: bool) -> torch.Tensor:
    return torch.empty(tuple(shape), dtype=dtype, device="cpu", pin_memory=bool(pinned and torch.cuda.is_available()))


def _bytes_of(t: torch.Tensor):
    """A writable byte view of a contiguous host tensor (numpy has no bfloat16, so go through uint8)."""
    return t.view(torch.uint8).numpy().reshape(-1)


class ChunkFile:
    """One chunk on disk.  Layout: magic (8 bytes), header length (uint64, little endian), a JSON header
    `{"tensors": [{"key", "layer", "dtype", "shape", "offset"}, ...]}`, then, from the next 4 KiB boundary on, each
    tensor's raw bytes (contiguous `[B, T, H, D]`, native little-endian) at its 4 KiB-aligned `offset` into that region."""

    def __init__(self, path: str, entries: list, data_start: int):
        self.path = path
        self.entries = entries               # offsets are relative to data_start
        self.data_start = data_start
        self._by_name = {(e["key"], e["layer"]): e for e in entries}

    # ---------------------------------------------------------------- writing
    @classmethod
    def write(cls, path: str, blob: dict) -> "ChunkFile":
        entries, cursor = [], 0
        for key, tensors in blob.items():
            for layer, t in enumerate(tensors):
                name = str(t.dtype).replace("torch.", "")
                if name not in _DTYPES:
                    raise ValueError(f"cannot spill a tensor of dtype {t.dtype}")
                entries.append({"key": key, "layer": layer, "dtype": name, "shape": list(t.shape), "offset": cursor})
                cursor += -(-t.numel() * t.element_size() // _ALIGN) * _ALIGN
        header = json.dumps({"tensors": entries}).encode("utf-8")
        data_start = -(-(16 + len(header)) // _ALIGN) * _ALIGN          # the data region starts at the next 4 KiB boundary
        tmp = path + ".part"
        with open(tmp, "wb") as f:
            f.write(_MAGIC + struct.pack("<Q", len(header)) + header)
            for e in entries:
                t = blob[e["key"]][e["layer"]].detach()
                if t.is_cuda:
                    t = t.cpu()
                f.seek(data_start + e["offset"])
                f.write(memoryview(_bytes_of(t.contiguous())))
        os.replace(tmp, path)            # a reader never sees a half-written chunk
        return cls(path, entries, data_start)

    @classmethod
    def open(cls, path: str) -> "ChunkFile":
        with open(path, "rb") as f:
            head = f.read(16)
            if head[:8] != _MAGIC:
                raise ValueError(f"{path} is not a chunk file")
            (n,) = struct.unpack("<Q", head[8:])
            return cls(path, json.loads(f.read(n).decode("utf-8"))["tensors"], -(-(16 + n) // _ALIGN) * _ALIGN)

    # ---------------------------------------------------------------- reading
    def read_rows(self, key: str, layer: int, start: int, end: int, *, pinned: bool = True) -> torch.Tensor:
        """Token rows `[start, end)` of one tensor as a host tensor `[B, end - start, H, D]`; only those bytes are read."""
        e = self._by_name[(key, layer)]
        bsz, tokens, *rest = e["shape"]
        start, end = max(0, int(start)), min(int(end), tokens)
        dtype = _DTYPES[e["dtype"]]
        out = _host_buffer([bsz, max(end - start, 0), *rest], dtype, pinned)
        if end <= start:
            return out
        row_bytes = out.element_size()
        for extent in rest:
            row_bytes *= extent
        flat = _bytes_of(out)
        span = (end - start) * row_bytes
        fd = os.open(self.path, os.O_RDONLY)
        try:
            for b in range(bsz):
                got = os.preadv(fd, [memoryview(flat[b * span:(b + 1) * span])],
                                self.data_start + e["offset"] + (b * tokens + start) * row_bytes)
                if got != span:
                    raise IOError(f"short read from {self.path}: {got} of {span} bytes")
        finally:
            os.close(fd)
        return out

    def read_all(self, *, pinned: bool = True) -> dict:
        blob: dict = {}
        for e in self.entries:
            blob.setdefault(e["key"], []).append(self.read_rows(e["key"], e["layer"], 0, e["shape"][1], pinned=pinned))
        return blob


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
        # recency order inside a tier = insertion order of its dict (oldest first)
        self._hbm: "OrderedDict[int, dict]" = OrderedDict()
        self._cpu: "OrderedDict[int, dict]" = OrderedDict()
        self._on_disk: Dict[int, ChunkFile] = {}     # chunks whose only live copy is the file
        self._files: Dict[int, ChunkFile] = {}       # every file ever written (the backups)
        self._landing: Dict[int, "torch.cuda.Event"] = {}   # host copies still in flight, by chunk
        self._side_stream = None
        self.counters = dict(n_spills=0, n_loads=0, n_drops=0, n_demotions=0, n_hbm_hits=0, n_host_hits=0, n_page_reads=0)

    # counters stay readable as attributes, as in the reference (`tier.n_spills`, ...)
    def __getattr__(self, name):
        counters = self.__dict__.get("counters")
        if counters is not None and name in counters:
            return counters[name]
        raise AttributeError(name)

    # ------------------------------------------------------------------ streams and demotion
    def side_stream(self, device: torch.device):
        """The stream demotions and promotions run on, created on first use."""
        if self._side_stream is None or self._side_stream.device != device:
            self._side_stream = torch.cuda.Stream(device=device)
        return self._side_stream

    def _demote(self, chunk_id: int, blob: dict) -> dict:
        """Device blob -> host blob.  The copies are queued on the side stream and an event marks their end; nobody
        waits here."""
        first = next(iter(blob.values()))[0]
        if not first.is_cuda:
            return blob
        device = first.device
        side = self.side_stream(device)
        side.wait_stream(torch.cuda.current_stream(device))     # the blob's producer has finished writing it
        host_blob: dict = {}
        with torch.cuda.stream(side):
            for key, tensors in blob.items():
                host_blob[key] = []
                for t in tensors:
                    host = _host_buffer(t.shape, t.dtype, self.pin_host)
                    host.copy_(t, non_blocking=True)
                    t.record_stream(side)                        # the device memory outlives the caller's reference
                    host_blob[key].append(host)
            done = torch.cuda.Event()
            done.record(side)
        self._landing[chunk_id] = done
        return host_blob

    def _landed(self, chunk_id: int) -> None:
        """Block until `chunk_id`'s host copy (if one is in flight) is complete."""
        event = self._landing.pop(chunk_id, None)
        if event is not None:
            event.synchronize()

    # ------------------------------------------------------------------ reference interface
    def put(self, chunk_id: int, blob: dict) -> None:
        """Register a freshly produced chunk in the hottest enabled tier."""
        for tier in (self._hbm, self._cpu, self._on_disk):
            tier.pop(chunk_id, None)
        first = next(iter(blob.values()))[0]
        if self.hbm_max_chunks > 0 and first.is_cuda:
            self._hbm[chunk_id] = blob
        else:
            self._cpu[chunk_id] = self._demote(chunk_id, blob)
        self._rebalance()

    def get(self, chunk_id: int) -> Optional[dict]:
        """The chunk's blob -- device tensors from the hot tier, host tensors otherwise; a spilled chunk is read back
        into host memory first.  `None` for a chunk no tier holds."""
        if chunk_id in self._hbm:
            self._hbm.move_to_end(chunk_id)
            self.counters["n_hbm_hits"] += 1
            return self._hbm[chunk_id]
        if chunk_id in self._cpu:
            self._cpu.move_to_end(chunk_id)
            self.counters["n_host_hits"] += 1
            self._landed(chunk_id)
            return self._cpu[chunk_id]
        spilled = self._on_disk.pop(chunk_id, None)
        if spilled is None:
            return None
        blob = spilled.read_all(pinned=self.pin_host)
        self.counters["n_loads"] += 1
        self._cpu[chunk_id] = blob
        self._rebalance()
        return blob

    def page_reader(self, chunk_id: int):
        """For a SPILLED chunk: a function `rows(key, layer, start, end)` that reads those token rows of one tensor
        straight from the chunk's file into a page-locked buffer.  The chunk stays on disk and keeps its place in no
        recency order; opening the reader counts as one load.  `None` when the chunk is not disk-resident (use `get`)."""
        spilled = self._on_disk.get(chunk_id)
        if spilled is None:
            return None
        self.counters["n_loads"] += 1

        def rows(key: str, layer: int, start: int, end: int) -> torch.Tensor:
            self.counters["n_page_reads"] += 1
            return spilled.read_rows(key, layer, start, end, pinned=self.pin_host)
        return rows

    def location(self, chunk_id: int) -> str:
        """Current tier of a chunk: `"hbm"`, `"cpu"`, `"nvme"` or `"absent"`."""
        for name, tier in (("hbm", self._hbm), ("cpu", self._cpu), ("nvme", self._on_disk)):
            if chunk_id in tier:
                return name
        return "absent"

    def _rebalance(self) -> None:
        """Push the least recently used chunks of an over-full tier one tier down."""
        while len(self._hbm) > self.hbm_max_chunks:
            victim, blob = self._hbm.popitem(last=False)
            self._cpu[victim] = self._demote(victim, blob)
            self.counters["n_demotions"] += 1
        while len(self._cpu) > self.cpu_max_chunks:
            victim, blob = self._cpu.popitem(last=False)
            if not self.nvme_enabled:
                self._landing.pop(victim, None)
                self.counters["n_drops"] += 1
                continue
            if victim not in self._files:                      # first spill of this chunk writes its backup
                self._landed(victim)
                self._files[victim] = ChunkFile.write(os.path.join(self.nvme_dir, f"hkv_chunk_{victim}.bin"), blob)
            self._landing.pop(victim, None)
            self._on_disk[victim] = self._files[victim]
            self.counters["n_spills"] += 1

    def stats(self) -> dict:
        return {"cpu_resident": len(self._cpu), "nvme_resident": len(self._on_disk), "backups": len(self._files),
                "hbm_resident": len(self._hbm), **self.counters}

    def cleanup(self) -> None:
        """Delete spilled files and clear all bookkeeping."""
        for chunk_file in self._files.values():
            try:
                os.remove(chunk_file.path)
            except OSError:
                pass
        for event in self._landing.values():
            event.synchronize()
        for table in (self._hbm, self._cpu, self._on_disk, self._files, self._landing):
            table.clear()
