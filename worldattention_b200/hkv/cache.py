"""Hierarchical KV Cache (HKV) on B200 (reference: pipeline/hkv/cache.py).

The history of an autoregressive rollout is kept outside the online cache as *chunks* split into
fixed-size *pages*; a prompt switch retrieves the most relevant pages and installs exactly those
into the online cache.  Interface, page/span arithmetic, re-rotation plan and soft-failure
behaviour follow the reference.  What changes is where the bytes move:

* `store` copies the populated cache device-to-device (hot tier) or into page-locked host memory
  on a side stream, and builds the page index from layer 0's keys with one pooling kernel that
  removes the temporal rotation on the fly;
* `retrieve` scores and selects pages in one kernel launch and reads back only the chosen ids;
* `apply` installs all pages of all layers with one page-copy kernel launch (keys re-rotated in
  flight, values verbatim), promoting host-resident pages through page-locked async copies on a
  side stream, clears only the tail of the cache beyond the installed span, and rebuilds the
  compressed tier with the compress kernel writing straight into the cache slots.

Online cache contract: a list with one dict per transformer block holding `k`, `v`
(`[B, capacity, H, D]`), scalar tensors `global_end_index`, `local_end_index`, and optionally
`k_coarse`, `v_coarse`.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _lib
from .retrieval import page_key_index, prompt_index, score_and_topk, select_top_chunks
from .rope import rotation_table, temporal_complex_dims
from .tiering import HKVTierManager

__all__ = ["HKVCache"]


class HKVCache:
    """KV bank with two-stage page retrieval and multi-tier residency.

    Args (reference: cache.py:39-71):
        frame_seq_length: tokens per latent frame.
        page_size_frames: frames per page.
        topk_pages: page budget installed per retrieval.
        stage1_topk_chunks: how many prompt-similar chunks feed stage 2.
        cpu_max_chunks: host-resident chunk capacity.
        nvme_enabled, nvme_dir: enable and locate the NVMe tier.
        rerope: re-rotate retrieved keys to the cache slots they are replayed at.
        hbm_max_chunks: (addition) chunks kept on the GPU in front of the host tier.
    """

    def __init__(self, *, frame_seq_length: int, page_size_frames: int = 8, topk_pages: int = 4,
                 stage1_topk_chunks: int = 1, cpu_max_chunks: int = 64, nvme_enabled: bool = False,
                 nvme_dir: Optional[str] = None, rerope: bool = True, hbm_max_chunks: int = 0):
        self.frame_seq_length = int(frame_seq_length)
        self.page_size_frames = int(page_size_frames)
        self.topk_pages = int(topk_pages)
        self.stage1_topk_chunks = int(stage1_topk_chunks)
        self.rerope = bool(rerope)
        self._tier_kwargs = dict(cpu_max_chunks=cpu_max_chunks, nvme_enabled=nvme_enabled, nvme_dir=nvme_dir,
                                 hbm_max_chunks=hbm_max_chunks)
        self.reset()

    def reset(self) -> None:
        """Drop the bank and start a fresh rollout."""
        self.chunks: List[dict] = []
        self.prompt_bank: List[torch.Tensor] = []
        self.tier = HKVTierManager(**self._tier_kwargs)

    def __len__(self) -> int:
        return len(self.chunks)

    @property
    def page_tokens(self) -> int:
        return self.page_size_frames * self.frame_seq_length

    # ------------------------------------------------------------------ store
    def store(self, kv_cache: Sequence[dict], *, prompt_embeds: torch.Tensor, current_start_frame: int,
              temporal_freqs: torch.Tensor) -> int:
        """Write the populated part of the online cache into the bank as a new chunk (cache.py:87-133).

        Returns the new chunk id, or -1 when the cache holds nothing to store.
        """
        valid_tokens = int(kv_cache[0]["local_end_index"].item())
        if valid_tokens <= 0:
            return -1
        _lib.require_cuda(kv_cache[0]["k"])

        chunk_id = len(self.chunks)
        # one allocation for the whole chunk (views per layer) instead of one per layer and tensor: growing the
        # allocator's pool costs a driver call per allocation, which at 60 calls per stored window showed as stalls of
        # up to a second at a prompt switch
        first = kv_cache[0]["k"]
        uniform = all(block[name].shape == first.shape and block[name].dtype == first.dtype and block[name].device == first.device
                      for block in kv_cache for name in ("k", "v"))
        blob = {"k": [], "v": []}
        if uniform:
            slab = torch.empty((2, len(kv_cache), first.shape[0], valid_tokens) + tuple(first.shape[2:]), dtype=first.dtype,
                               device=first.device)
            for layer, block in enumerate(kv_cache):
                for which, name in enumerate(("k", "v")):
                    slab[which, layer].copy_(block[name][:, :valid_tokens].detach())
                    blob[name].append(slab[which, layer])
        else:
            for block in kv_cache:
                blob["k"].append(block["k"][:, :valid_tokens].detach().clone())
                blob["v"].append(block["v"][:, :valid_tokens].detach().clone())

        page_spans = [(start, min(start + self.page_tokens, valid_tokens))
                      for start in range(0, valid_tokens, self.page_tokens)]
        start_frame = int(current_start_frame - valid_tokens // self.frame_seq_length)
        page_index = page_key_index(blob["k"][0], page_spans, frame_seq_length=self.frame_seq_length,
                                    start_frame=start_frame, temporal_freqs=temporal_freqs)
        self.chunks.append({
            "chunk_id": chunk_id,
            "valid_tokens": valid_tokens,
            "page_spans": page_spans,
            "start_frame": start_frame,
            "page_index": page_index,
            "heads": int(kv_cache[0]["k"].shape[2]),
        })
        self.prompt_bank.append(prompt_index(prompt_embeds).detach().to(page_index.device))
        self.tier.put(chunk_id, blob)
        return chunk_id

    # ------------------------------------------------------------------ retrieve
    def retrieve(self, *, prompt_embeds: torch.Tensor, query_vec: torch.Tensor,
                 per_head: bool = False):
        """Select the pages to install for the incoming prompt (cache.py:135-178).

        Returns `(chunk_id, page_id)` pairs in chronological order.  With `per_head=True` (an
        addition) the page vectors are scored per head and a list of such lists, one per head,
        is returned.
        """
        if not self.chunks:
            return []
        bank = torch.stack(self.prompt_bank, dim=0)
        candidates = select_top_chunks(prompt_index(prompt_embeds).detach(), bank, self.stage1_topk_chunks)

        owners: List[Tuple[int, int]] = []
        vectors = []
        for chunk_id in candidates:
            page_index = self.chunks[chunk_id].get("page_index")
            if page_index is None or page_index.numel() == 0:
                continue
            vectors.append(page_index)
            owners.extend((chunk_id, page_id) for page_id in range(page_index.shape[0]))
        if not owners:
            return []
        pool = vectors[0] if len(vectors) == 1 else torch.cat(vectors, dim=0)

        query = query_vec.reshape(-1)
        if query.shape[0] != pool.shape[1]:
            raise ValueError(f"query dim {query.shape[0]} does not match page index dim {pool.shape[1]}")

        def chronological(pairs):
            return sorted(pairs, key=lambda pair: (self.chunks[pair[0]]["start_frame"],
                                                   self.chunks[pair[0]]["page_spans"][pair[1]][0]))

        if per_head:
            heads = self.chunks[owners[0][0]].get("heads", 1)
            _, ids, _ = score_and_topk(query, pool, self.topk_pages, groups=heads)
            return [chronological([owners[i] for i in row]) for row in ids.tolist()]
        if self.topk_pages <= 0:
            return []
        _, ids, _ = score_and_topk(query, pool, self.topk_pages)
        return chronological([owners[i] for i in ids[0].tolist()])

    # ------------------------------------------------------------------ apply
    def apply(self, kv_cache: Sequence[dict], selected_pairs: Sequence[Tuple[int, int]], *,
              current_start_frame: int, temporal_freqs: torch.Tensor,
              hsa_modules: Optional[Sequence] = None) -> int:
        """Install the selected pages into the online cache, replacing its contents (cache.py:180-254).

        Returns the number of tokens installed; 0 (cache untouched) when nothing resolves.
        """
        k0 = kv_cache[0]["k"]
        plan, blobs = self._install_plan(selected_pairs, capacity=int(k0.shape[1]),
                                         current_start_frame=int(current_start_frame))
        if plan is None:
            return 0
        dev = _lib.require_cuda(k0)
        tokens = int(plan["count"].sum())

        compressed = all(name in kv_cache[0] for name in ("k_coarse", "v_coarse"))
        if compressed and hsa_modules is None:
            raise ValueError(
                "the online cache carries a compressed tier, so hsa_modules must be supplied so it "
                "can be rebuilt for the installed pages"
            )

        if tokens > 0:
            self._install(kv_cache, plan, blobs, temporal_freqs, dev, k0.dtype)

        end_token = current_start_frame * self.frame_seq_length
        for layer, block in enumerate(kv_cache):
            # only the tail beyond the installed span needs clearing: the copy kernel wrote everything before it
            for name in ("k", "v"):
                block[name][:, tokens:].zero_()
            if compressed:
                filled = self._write_coarse(block, hsa_modules[layer], tokens) if tokens > 0 else 0
                for name in ("k_coarse", "v_coarse"):
                    block[name][:, filled:].zero_()
            block["global_end_index"].fill_(end_token)
            block["local_end_index"].fill_(tokens)
        return tokens

    _PLAN_DTYPE = np.dtype([("chunk", "<i8"), ("src", "<i8"), ("count", "<i8"), ("dst", "<i8"),
                            ("frame_from", "<i8"), ("frame_to", "<i8")])

    def _install_plan(self, selected_pairs, *, capacity: int, current_start_frame: int):
        """The install as a table, one row per page that resolves and (at least partly) fits.

        Columns: owning chunk, first source token and token count inside the chunk, first destination token in
        the cache, and the frame the page was written at / is replayed at.  Pairs that name an unknown chunk or
        page, or a chunk no tier holds any more, are left out (cache.py:256-271); pages fill the cache front to
        back and the one that crosses the capacity is cut (cache.py:203-211); the installed span ends at
        `current_start_frame`, so a page's new frame is that minus the frames still to come (cache.py:273-287).
        Returns `(None, {})` when no row remains.
        """
        blobs: dict = {}
        rows = []
        for chunk_id, page_id in selected_pairs:
            meta = self.chunks[chunk_id] if 0 <= chunk_id < len(self.chunks) else None
            if meta is None or not 0 <= page_id < len(meta["page_spans"]):
                continue
            if chunk_id not in blobs:
                # a spilled chunk is read page by page from its file; anything else comes as a whole blob
                held = self.tier.page_reader(chunk_id) or self.tier.get(chunk_id)
                if held is None:
                    continue
                blobs[chunk_id] = held
            first, last = meta["page_spans"][page_id]
            rows.append((chunk_id, first, last - first))
        if not rows:
            return None, {}
        plan = np.zeros(len(rows), dtype=self._PLAN_DTYPE)
        plan["chunk"], plan["src"], plan["count"] = (np.asarray(col, dtype=np.int64) for col in zip(*rows))
        before = np.cumsum(plan["count"]) - plan["count"]               # tokens installed ahead of each page
        plan["count"] = np.clip(capacity - before, 0, plan["count"])    # the page that crosses the capacity is cut
        plan = plan[: int(np.searchsorted(before, capacity, side="left"))] if capacity > 0 else plan[:0]
        if plan.size == 0:
            plan = np.zeros(1, dtype=self._PLAN_DTYPE)   # everything resolved but nothing fits: an empty install
            plan["chunk"] = rows[0][0]
        plan["dst"] = np.cumsum(plan["count"]) - plan["count"]
        frame_len = self.frame_seq_length
        chunk_frame = np.asarray([self.chunks[int(c)]["start_frame"] for c in plan["chunk"]], dtype=np.int64)
        plan["frame_from"] = chunk_frame + plan["src"] // frame_len
        plan["frame_to"] = current_start_frame - int(plan["count"].sum()) // frame_len + plan["dst"] // frame_len
        return plan, blobs

    def _install(self, kv_cache, plan, blobs, temporal_freqs, dev, dtype) -> None:
        """One page-copy launch for every (layer, page, K|V, batch item) of the plan."""
        k0 = kv_cache[0]["k"]
        bsz, _, heads, head_dim = k0.shape
        row_elems = heads * head_dim
        esize = k0.element_size()
        nt = temporal_complex_dims(head_dim)
        rot = None
        if self.rerope:
            rot = rotation_table(temporal_freqs, plan["frame_to"].tolist(), plan["frame_from"].tolist(), nt)

        main = torch.cuda.current_stream(dev)
        side = self.tier.side_stream(dev)
        # pass 1: where every page comes from
        sources = []         # (layer, name, plan row index, tensor or host page, staging offset in elements or None)
        staged_elems = 0
        for layer, block in enumerate(kv_cache):
            for name in ("k", "v"):
                dst = block[name]
                if dst.stride(3) != 1 or dst.stride(2) != head_dim or dst.stride(1) != row_elems:
                    raise ValueError("online cache tensors must be contiguous [B, capacity, H, D]")
                for i, row in enumerate(plan):
                    n = int(row["count"])
                    if n == 0:
                        continue
                    held, first = blobs[int(row["chunk"])], int(row["src"])
                    page = held(name, layer, first, first + n) if callable(held) else held[name][layer][:, first: first + n]
                    slot = None
                    if not page.is_cuda and page.dtype == dtype and page.stride(3) == 1 and page.stride(2) == head_dim \
                            and page.stride(1) == row_elems:
                        slot = staged_elems                      # cold page in the cache's own layout: one block copy per item
                        staged_elems += bsz * n * row_elems
                    sources.append((layer, name, i, page, slot))

        # pass 2: cold pages cross on the side stream into ONE staging buffer; whatever conversion a page needs runs on
        # that stream too, behind its copy, so that nothing reads a landing buffer early
        staging = torch.empty((max(staged_elems, 1),), dtype=dtype, device=dev) if staged_elems else None
        keep_alive = [staging]
        promote, records = [], []
        promoted = False
        for layer, name, i, page, slot in sources:
            row = plan[i]
            n = int(row["count"])
            dst = kv_cache[layer][name]
            if slot is not None:
                src_ptr, src_batch, src_stride = staging.data_ptr() + slot * esize, n * row_elems, row_elems
                for b in range(bsz):
                    promote.append(_lib.PageCopy(page.data_ptr() + b * page.stride(0) * esize,
                                                 src_ptr + b * src_batch * esize, row_elems, row_elems, n, -1))
                keep_alive.append(page)
            else:
                if not page.is_cuda:
                    with torch.cuda.stream(side):
                        landed = torch.empty(page.shape, dtype=page.dtype, device=dev)
                        landed.copy_(page, non_blocking=True)
                        page = self._as_cache_rows(landed, dtype, head_dim)
                    promoted = True
                else:
                    page = self._as_cache_rows(page, dtype, head_dim)
                keep_alive.append(page)
                src_ptr, src_batch, src_stride = page.data_ptr(), page.stride(0), page.stride(1)
            for b in range(bsz):
                records.append(_lib.PageCopy(
                    src_ptr + b * src_batch * esize,
                    dst.data_ptr() + (b * dst.stride(0) + int(row["dst"]) * row_elems) * esize,
                    src_stride, row_elems, n,
                    i if (name == "k" and rot is not None) else -1))
        if promote:
            arr = (_lib.PageCopy * len(promote))(*promote)
            side.wait_stream(main)            # the staging block may be recycled memory that the main stream still uses
            staging.record_stream(side)
            with _lib.device_guard(dev):
                _lib.check(_lib.lib().wa_hkv_promote_pages(arr, len(promote), row_elems, esize, side.cuda_stream))
            promoted = True
        if promoted:
            main.wait_stream(side)
        arr = (_lib.PageCopy * len(records))(*records)
        dev_records = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(dev)
        rot_dev = torch.from_numpy(np.ascontiguousarray(rot)).to(dev) if rot is not None else None
        _lib.check(_lib.lib().wa_hkv_gather_pages(
            dev_records.data_ptr(), len(records), int(plan["count"].max()), row_elems, head_dim, _lib.dtype_code(dtype),
            _lib.ptr(rot_dev), nt, main.cuda_stream))
        for t in keep_alive:
            if t is not None and t.is_cuda:
                t.record_stream(main)

    @staticmethod
    def _as_cache_rows(page: torch.Tensor, dtype: torch.dtype, head_dim: int) -> torch.Tensor:
        """`page` in the cache's dtype with head rows contiguous (a no-op for pages stored the way the cache is)."""
        if page.dtype != dtype:
            page = page.to(dtype)
        if page.stride(3) != 1 or page.stride(2) != head_dim:
            page = page.contiguous()
        return page

    @staticmethod
    def _write_coarse(block: dict, hsa, total_tokens: int) -> int:
        """Rebuild the compressed tier from the tokens installed at cache offset 0 (cache.py:289-299).

        The compress kernel writes directly into the cache's compressed slots.
        """
        k, v = block["k"][:, :total_tokens], block["v"][:, :total_tokens]
        dev = k.device
        bsz, _, heads, head_dim = k.shape
        coarse_start, coarse_end = hsa.token_range_to_coarse(0, int(total_tokens))
        kc, vc = block["k_coarse"], block["v_coarse"]
        if kc.dtype != k.dtype or vc.dtype != k.dtype or kc.stride() != vc.stride() or kc.stride(3) != 1:
            k_new, v_new = hsa.compress_kv_cache(k, v)
            kc[:, coarse_start:coarse_end] = k_new.to(kc.dtype)
            vc[:, coarse_start:coarse_end] = v_new.to(vc.dtype)
            return coarse_end
        if coarse_end > kc.shape[1]:
            raise ValueError("compressed cache is too small for the installed pages")
        pk = hsa.k_proj_mat.detach().to(device=dev).contiguous()
        pv = hsa.v_proj_mat.detach().to(device=dev, dtype=pk.dtype).contiguous()
        _lib.check(_lib.lib().wa_compress_kv(
            _lib.t4_blhd(k), _lib.t4_blhd(v), _lib.t4_blhd(kc), _lib.t4_blhd(vc), bsz, int(total_tokens), heads,
            head_dim, hsa.proj_segment_len, hsa.block_size, pk.data_ptr(), pv.data_ptr(), _lib.dtype_code(pk.dtype),
            pk.shape[0], pk.shape[1], _lib.stream_ptr(dev)))
        return coarse_end
