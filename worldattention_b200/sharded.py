"""Multi-GPU execution of the HSA forward on one NVSwitch box.

The reference runs HSA on a single device.  Two shardings are provided, both one process per GPU
over `torch.distributed` (NCCL on GPUs; the planning and exchange logic also runs under gloo):

* **head split** (2 / 4 GPUs): every quantity in HSA is per head (pooling, block map, the Gini
  mean over (batch, query block), both softmaxes; the projections and the gate are shared and
  replicated), so a rank runs the ordinary forward on its heads.  No data-path collective is
  needed; `gather_heads` all-gathers the outputs for a consumer that wants every head.
* **KV shard** (8 GPUs; 12 heads do not divide by 8): the key range is cut at attention-block
  boundaries.  Ranks all-gather their pooled keys, take the identical global routing decision,
  attend to the selected blocks and compressed slots they own, and all-gather per-branch partial
  outputs with log-sum-exp normalisers that `merge_partials` combines before the gate.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .hsa import branches
from .hsa.routing import block_attention_map, block_mean_pool, build_block_routing  # noqa: F401

__all__ = ["plan_head_split", "plan_kv_shards", "local_selection", "gather_heads", "all_gather_cat", "exchange_rows",
           "partial_records", "route_candidates", "local_candidates", "merge_candidates", "merge_partials", "hsa_attention_head_split", "hsa_attention_kv_sharded"]

merge_partials = branches.merge_partials


# --------------------------------------------------------------------------- planning (pure host logic)
def plan_head_split(num_heads: int, world: int, cost_per_head: Optional[Sequence[float]] = None) -> List[List[int]]:
    """Assign heads to ranks: longest-processing-time greedy on `cost_per_head` (e.g. k_h), sorted ids per rank.

    With no costs the split is contiguous and even.  Every rank receives `num_heads // world` or
    one more head.
    """
    if world <= 0 or num_heads < world:
        raise ValueError(f"cannot split {num_heads} heads over {world} ranks")
    if cost_per_head is None:
        base, extra = divmod(num_heads, world)
        out, h = [], 0
        for r in range(world):
            n = base + (1 if r < extra else 0)
            out.append(list(range(h, h + n)))
            h += n
        return out
    if len(cost_per_head) != num_heads:
        raise ValueError("cost_per_head must have one entry per head")
    cap = math.ceil(num_heads / world)
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for h in sorted(range(num_heads), key=lambda i: (-float(cost_per_head[i]), i)):
        r = min((r for r in range(world) if len(out[r]) < cap), key=lambda r: (loads[r], r))
        out[r].append(h)
        loads[r] += float(cost_per_head[h])
    return [sorted(x) for x in out]


def plan_kv_shards(kv_len: int, block_size: int, world: int, page_tokens: int = 0) -> List[Tuple[int, int]]:
    """Contiguous token ranges `[lo, hi)` per rank, cut at attention-block boundaries.

    With `page_tokens > 0` each cut is the block boundary nearest to a page boundary, so a shard
    holds (almost) whole pages even though pages and blocks do not align.
    """
    if world <= 0:
        raise ValueError("world must be positive")
    n_blocks = math.ceil(kv_len / block_size)
    cuts = [0]
    for r in range(1, world):
        target = kv_len * r / world
        if page_tokens > 0:
            target = round(target / page_tokens) * page_tokens
        blk = min(max(int(round(target / block_size)), -(-cuts[-1] // block_size)), n_blocks)
        cuts.append(min(blk * block_size, kv_len))   # the last block may be ragged: never cut past the end
    cuts.append(kv_len)
    shards = [(cuts[r], cuts[r + 1]) for r in range(world)]
    assert shards[0][0] == 0 and shards[-1][1] == kv_len and all(lo <= hi for lo, hi in shards)
    assert all(shards[r][1] == shards[r + 1][0] for r in range(world - 1))
    assert all(lo % block_size == 0 or lo == kv_len for lo, _ in shards)
    return shards


def local_selection(index: torch.Tensor, num: torch.Tensor, block_lo: int, block_hi: int):
    """Restrict a global routing `(index, num)` to the key blocks `[block_lo, block_hi)`.

    Returns `(local_index int32 [..., Nkv_local], local_num int32 [...])`, ids rebased to the
    shard and listed in ascending order.  The union over a partition of the block range is the
    global selection.
    """
    nkv = index.shape[-1]
    if index.is_cuda:   # one launch instead of a dozen tensor operations
        from . import _lib
        width = max(block_hi - block_lo, 1)
        index_c, num_c = index.to(torch.int32).contiguous(), num.to(torch.int32).contiguous()
        rows = num_c.numel()
        local_index = torch.empty(index.shape[:-1] + (width,), dtype=torch.int32, device=index.device)
        local_num = torch.empty(num.shape, dtype=torch.int32, device=index.device)
        _lib.check(_lib.lib().wa_route_local_selection(index_c.data_ptr(), num_c.data_ptr(), rows, nkv, block_lo,
                                                       block_lo + width, local_index.data_ptr(), local_num.data_ptr(),
                                                       _lib.stream_ptr(index.device)))
        return local_index, local_num
    slots = torch.arange(nkv, device=index.device).view(*([1] * (index.dim() - 1)), nkv)
    selected = slots < num.unsqueeze(-1).long()
    ids = index.long().clamp(0, nkv - 1)
    owned = selected & (ids >= block_lo) & (ids < block_hi)
    width = max(block_hi - block_lo, 1)
    hits = torch.zeros(index.shape[:-1] + (width,), dtype=torch.int32, device=index.device)
    hits.scatter_add_(-1, (ids - block_lo).clamp(0, width - 1), owned.to(torch.int32))
    member = hits > 0
    # duplicates in the global list (allowed by the reference) collapse to one visit here
    local_num = member.sum(-1).to(torch.int32)
    order = torch.argsort((~member).to(torch.int8), dim=-1, stable=True)
    return order.to(torch.int32).contiguous(), local_num.contiguous()


# --------------------------------------------------------------------------- exchange
def all_gather_cat(t: torch.Tensor, dim: int, group=None, sizes: Optional[Sequence[int]] = None) -> torch.Tensor:
    """All-gather tensors that may differ in `dim` (sizes per rank given) and concatenate along it."""
    world = dist.get_world_size(group)
    if world == 1:
        return t
    t = t.contiguous()
    if sizes is None:
        flat = torch.empty(world * t.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(flat, t.view(-1), group=group)
        return torch.cat(list(flat.view([world] + list(t.shape)).unbind(0)), dim=dim)
    longest = max(sizes)
    pad_shape = list(t.shape)
    pad_shape[dim] = longest
    padded = torch.zeros(pad_shape, dtype=t.dtype, device=t.device)
    padded.narrow(dim, 0, t.shape[dim]).copy_(t)
    flat = torch.empty(world * padded.numel(), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(flat, padded.view(-1), group=group)      # one collective on one buffer (the list form copies per rank)
    every = flat.view([world] + pad_shape)
    if all(n == longest for n in sizes):
        return torch.cat(list(every.unbind(0)), dim=dim)
    return torch.cat([every[r].narrow(dim, 0, n) for r, n in enumerate(sizes)], dim=dim)


def gather_heads(out_local: torch.Tensor, head_plan: List[List[int]], group=None) -> torch.Tensor:
    """All-gather `[B, L, H_local, D]` head-split outputs into `[B, L, H, D]` in head order."""
    sizes = [len(h) for h in head_plan]
    cat = all_gather_cat(out_local, 2, group=group, sizes=sizes)
    order = [h for heads in head_plan for h in heads]
    inverse = torch.empty(len(order), dtype=torch.long)
    inverse[torch.tensor(order)] = torch.arange(len(order))
    return cat.index_select(2, inverse.to(cat.device))


# --------------------------------------------------------------------------- forwards
def hsa_attention_head_split(hsa_module, q_local, k_local, v_local, *, k_coarse=None, v_coarse=None,
                             topk_local=None, head_plan=None, group=None, gather: bool = True):
    """Head-split forward: each rank holds its heads of q/k/v (and of the compressed cache)."""
    from .hsa.attention import hsa_attention
    out = hsa_attention(
        q_local, k_local, v_local, k_coarse=k_coarse, v_coarse=v_coarse,
        k_proj_mat=hsa_module.k_proj_mat, v_proj_mat=hsa_module.v_proj_mat, gate_lin=hsa_module.gate_lin,
        block_size=hsa_module.block_size, tau_min=hsa_module.tau_min, tau_max=hsa_module.tau_max,
        proj_segment_len=hsa_module.proj_segment_len, topk_per_head=topk_local)
    if gather and head_plan is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        return gather_heads(out, head_plan, group=group)
    return out


last_call_info: dict = {}     # what the most recent `hsa_attention_kv_sharded` on this process ran (for reporting)


def exchange_rows(q_len: int, world: int) -> Tuple[int, List[Tuple[int, int]]]:
    """Query rows per rank in the exchange of partials: `(rows_per_rank, [(first, count) per rank])`.

    Rank j merges rows `[j * rp, (j + 1) * rp)`; the last slices may be short or empty when `q_len` is not a multiple
    of the rank count."""
    rp = -(-q_len // world)
    return rp, [(r * rp, max(0, min(q_len, (r + 1) * rp) - r * rp)) for r in range(world)]


def local_candidates(q_pooled, k_pooled_local, *, block_lo: int, topk_max: int) -> torch.Tensor:
    """This rank's best `topk_max` key blocks per row as sortable keys: int64 `[B * H * Nq, topk_max]`."""
    from . import _lib
    dev = _lib.require_cuda(q_pooled, k_pooled_local)
    bsz, heads, nq, head_dim = q_pooled.shape
    nloc = k_pooled_local.shape[2]
    cand = torch.empty((bsz * heads * nq, topk_max), dtype=torch.int64, device=dev)
    _lib.check(_lib.lib().wa_route_local_candidates(
        q_pooled.contiguous().data_ptr(), k_pooled_local.contiguous().data_ptr() if nloc else None, bsz, heads, nq, nloc,
        head_dim, block_lo, topk_max, cand.data_ptr(), _lib.stream_ptr(dev)))
    return cand


def merge_candidates(every: torch.Tensor, shape, *, topk_per_head, blocks_total: int, block_lo: int, block_hi: int):
    """From the candidates of all ranks (`[W, rows, topk_max]` int64) the selection restricted to `[block_lo, block_hi)`:
    `(local_index int32 [B, H, Nq, max(block_hi - block_lo, 1)], local_num int32 [B, H, Nq])`."""
    from . import _lib
    dev = _lib.require_cuda(every)
    bsz, heads, nq = shape
    world, _, topk_max = every.shape
    width = max(block_hi - block_lo, 1)
    local_index = torch.empty((bsz, heads, nq, width), dtype=torch.int32, device=dev)
    local_num = torch.empty((bsz, heads, nq), dtype=torch.int32, device=dev)
    topk = topk_per_head.to(device=dev, dtype=torch.int32).contiguous()
    _lib.check(_lib.lib().wa_route_merge_candidates(
        every.contiguous().data_ptr(), world, bsz, heads, nq, topk_max, topk.data_ptr(), blocks_total, block_lo, block_hi, width,
        local_index.data_ptr(), local_num.data_ptr(), _lib.stream_ptr(dev)))
    return local_index, local_num


def route_candidates(q_pooled, k_pooled_local, *, block_lo: int, blocks_total: int, topk_per_head, topk_max: int, group=None):
    """Fixed top-k routing without gathering the pooled keys: every rank scores its own key blocks, the ranks exchange
    their `topk_max` best candidates per row (ONE all-gather of 8 bytes per candidate), and each rank keeps, of the
    global top-k of a row, the blocks it owns.  Returns `(local_index int32 [B, H, Nq, Nloc], local_num int32 [B, H, Nq])`.
    """
    bsz, heads, nq, _ = q_pooled.shape
    nloc = k_pooled_local.shape[2]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    cand = local_candidates(q_pooled, k_pooled_local, block_lo=block_lo, topk_max=topk_max)
    if world > 1:
        every = torch.empty((world,) + tuple(cand.shape), dtype=torch.int64, device=cand.device)
        dist.all_gather_into_tensor(every, cand, group=group)
    else:
        every = cand.unsqueeze(0)
    return merge_candidates(every, (bsz, heads, nq), topk_per_head=topk_per_head, blocks_total=blocks_total, block_lo=block_lo,
                            block_hi=block_lo + nloc)


def _partials_unpacked(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs):
    """Per-branch partial outputs of one rank through the contiguous interface (any shape; SIMT kernels where the
    tcgen05 kernel does not apply; empty branches where the rank owns no keys or no compressed slots)."""
    bsz, q_len, heads, head_dim = q.shape
    has_kv = k_local is not None and k_local.shape[1] > 0
    has_coarse = kc_local is not None and kc_local.shape[1] > 0
    if has_kv and has_coarse:
        return branches.hsa_partials(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs)
    if has_kv:
        o_s, l_s = branches.sparse_branch(q, k_local, v_local, index_l, num_l, bs, kv_len=k_local.shape[1])
    else:
        o_s = q.new_zeros((bsz, q_len, heads, head_dim), dtype=torch.float32)
        l_s = q.new_full((bsz, heads, q_len), float("-inf"), dtype=torch.float32)
    if has_coarse:
        o_l, l_l = branches.linear_branch(q, kc_local, vc_local)
    else:
        o_l = torch.zeros_like(o_s)
        l_l = torch.full_like(l_s, float("-inf"))
    return o_s, l_s, o_l, l_l, False


_peer_exchange_failed = False      # set when the IPC set-up did not work on this machine: "auto" then stays on NCCL


def _peer_exchange(world, rank, rows, heads, rec, dev, group, *, required: bool):
    """The cached `PeerExchange` for these sizes, or None when it cannot be set up (every rank then agrees to use NCCL)."""
    global _peer_exchange_failed
    key = (world, rank, rows, heads, rec, dev.index, id(group))
    if key in PeerExchange._cache:
        return PeerExchange._cache[key]
    xchg, error = None, None
    try:
        xchg = PeerExchange(world, rank, rows, heads, rec, dev, group)
    except Exception as exc:      # reported below; the decision has to be common to all ranks
        error = f"{type(exc).__name__}: {exc}"
    flags = [None] * world
    dist.all_gather_object(flags, error, group=group)
    if any(f is not None for f in flags):
        _peer_exchange_failed = True
        if required:
            raise RuntimeError(f"peer exchange set-up failed: {[f for f in flags if f is not None][0]}")
        return None
    PeerExchange._cache[key] = xchg
    return xchg


class PeerExchange:
    """This rank's receive buffer for the partial records, mapped into every rank of the group.

    The partial-output kernel of rank s then stores the record of query row t directly into the buffer of the rank that
    merges t (`branches.hsa_partials_packed(peer=...)`): the all-to-all of the exchange disappears into the kernel's own
    stores, which travel over NVLink while the kernel computes.  The buffer is one `cudaMalloc` allocation shared through
    a CUDA IPC handle (peer access is enabled when a handle is opened); it lives as long as the process.

    Ordering: a receiver may read after every sender's kernel has completed -- the forward puts a one-element all-reduce
    on the stream behind the kernel -- and a sender may overwrite after the receivers have merged, which the all-gather of
    the finished rows at the end of the forward implies.
    """

    _cache: dict = {}

    def __init__(self, world: int, rank: int, rows: int, heads: int, rec: int, dev: torch.device, group=None):
        from cuda.bindings import runtime as rt
        self.world, self.rank, self.rows, self.heads, self.rec = world, rank, rows, heads, rec
        nbytes = world * rows * heads * rec * 4

        def ok(result):
            err = result[0] if isinstance(result, tuple) else result
            if int(err) != 0:
                raise RuntimeError(f"CUDA runtime error {int(err)} while setting up the peer exchange")
            return result[1] if isinstance(result, tuple) and len(result) > 1 else None

        with torch.cuda.device(dev):
            self.ptr = int(ok(rt.cudaMalloc(nbytes)))
            ok(rt.cudaMemset(self.ptr, 0, nbytes))          # rows past the query length are never written: keep them finite
            handle = ok(rt.cudaIpcGetMemHandle(self.ptr))
            mine = bytes(handle.reserved)
            every = [None] * world
            if world > 1:
                dist.all_gather_object(every, mine, group=group)
            else:
                every = [mine]
            self.ptrs = []
            for r in range(world):
                if r == rank:
                    self.ptrs.append(self.ptr)
                else:
                    h = rt.cudaIpcMemHandle_t()
                    h.reserved = every[r]
                    self.ptrs.append(int(ok(rt.cudaIpcOpenMemHandle(h, rt.cudaIpcMemLazyEnablePeerAccess))))
        if any((p - self.ptr) % 4 for p in self.ptrs):
            raise RuntimeError("peer buffers are not float-aligned relative to each other")
        self.deltas = [(p - self.ptr) // 4 for p in self.ptrs]
        self.local = _raw_tensor(self.ptr, (1, world * rows, heads, rec), dev)      # [1, W * rows, H, rec] float32

    @classmethod
    def get(cls, world, rank, rows, heads, rec, dev, group=None):
        key = (world, rank, rows, heads, rec, dev.index, id(group))
        if key not in cls._cache:
            cls._cache[key] = cls(world, rank, rows, heads, rec, dev, group)
        return cls._cache[key]


class _RawBuffer:
    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False), "version": 3,
                                         "strides": None}


def _raw_tensor(ptr: int, shape, dev: torch.device) -> torch.Tensor:
    """A float32 tensor over device memory that torch did not allocate."""
    return torch.as_tensor(_RawBuffer(ptr, shape), device=dev)


def partial_records(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs, records) -> bool:
    """One rank's partials as packed records (`records`: float32 `[1, rows >= Lq, H, 2 D + 4]`, see
    `branches.hsa_partials_packed`): written by the tcgen05 kernel where it applies, packed here otherwise.  Rows from
    Lq on are zeroed so that whoever merges the last slice sees finite numbers.  Returns whether the tcgen05 kernel ran."""
    _, q_len, heads, head_dim = q.shape
    if records.shape[1] > q_len:
        records[:, q_len:].zero_()
    has_kv = k_local is not None and k_local.shape[1] > 0
    has_coarse = kc_local is not None and kc_local.shape[1] > 0
    if has_kv and has_coarse and branches.hsa_partials_packed(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs, records):
        return True
    o_s, l_s, o_l, l_l, used = _partials_unpacked(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs)
    records[:, :q_len, :, :head_dim] = o_s
    records[:, :q_len, :, head_dim:2 * head_dim] = o_l
    records[:, :q_len, :, 2 * head_dim] = l_s.transpose(1, 2)
    records[:, :q_len, :, 2 * head_dim + 1] = l_l.transpose(1, 2)
    records[:, :q_len, :, 2 * head_dim + 2:] = 0
    return bool(used)


def hsa_attention_kv_sharded(hsa_module, q, k_local, v_local, kc_local, vc_local, *, kv_len: int,
                             shards: List[Tuple[int, int]], topk_per_head=None, group=None, routing: str = "auto",
                             topk_max: Optional[int] = None, exchange: str = "auto"):
    """KV-sharded forward.  `q` is replicated; `k_local`/`v_local` hold this rank's token range.

    `kc_local`/`vc_local` are the compressed slots of the segments this rank owns.  Returns the
    full `[B, Lq, H, D]` output on every rank.

    Routing: `"gather"` all-gathers the pooled keys and repeats the whole decision on every rank (identical to the
    single-device decision); `"candidates"` (fixed top-k only) lets every rank score its own blocks and exchanges the
    best `topk_max` per row instead (see `route_candidates`); `"auto"` takes the second for fixed top-k over caches of
    4096 key blocks or more, where gathering and re-sorting everything would not shrink with the rank count.

    Exchange (B = 1, more than one rank): the tcgen05 kernel writes both branch outputs and both normalisers of a
    (token, head) into one packed record; ONE all-to-all hands rank j the records of query rows
    `[j * rp, (j + 1) * rp)` of every shard; rank j merges them, gate-combines its rows, and one all-gather
    distributes the finished bf16 rows.  Three collectives per forward.

    `exchange="peer"` (and `"auto"` where it applies: at most 8 ranks, every shard with keys and compressed slots, the
    tcgen05 kernel's shapes) removes the all-to-all: the kernel stores every record directly into the receive buffer of
    the rank that merges its row (`PeerExchange`: CUDA IPC, plain stores over NVLink during the kernel), and a one-element
    all-reduce behind the kernel tells every rank that its rows have arrived.  `exchange="nccl"` keeps the all-to-all.
    """
    if exchange not in ("auto", "nccl", "peer"):
        raise ValueError("exchange must be 'auto', 'nccl' or 'peer'")
    if routing not in ("auto", "gather", "candidates") or (routing == "candidates" and topk_per_head is None):
        raise ValueError("routing must be 'auto', 'gather' or (with a fixed top-k) 'candidates'")
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    bs = hsa_module.block_size
    bsz, q_len, heads, head_dim = q.shape
    lo, hi = shards[rank]
    n_local = hi - lo

    nq = math.ceil(q_len / bs)
    q_pooled = _pool_blhd(q, bs)
    k_pooled_local = _pool_blhd(k_local, bs) if n_local > 0 else q_pooled.new_zeros((bsz, heads, 0, head_dim))
    blocks_per_rank = [math.ceil((b - a) / bs) for a, b in shards]
    blocks_total = sum(blocks_per_rank)
    block_lo = sum(blocks_per_rank[:rank])
    by_candidates = topk_per_head is not None and (routing == "candidates" or (routing == "auto" and blocks_total >= 4096))
    if by_candidates:
        if topk_max is None:
            topk_max = int(topk_per_head.max().item())       # a host read: pass topk_max to avoid it
        index_l, num_l = route_candidates(q_pooled, k_pooled_local, block_lo=block_lo, blocks_total=blocks_total,
                                          topk_per_head=topk_per_head, topk_max=max(1, min(int(topk_max), blocks_total)),
                                          group=group)
    else:
        # pooled keys are exchanged, the decision is taken identically everywhere
        k_pooled = all_gather_cat(k_pooled_local, 2, group=group, sizes=blocks_per_rank) if world > 1 else k_pooled_local
        decided = build_block_routing(block_attention_map(q_pooled, k_pooled), hsa_module.tau_min, hsa_module.tau_max,
                                      topk_per_head=topk_per_head)
        index_l, num_l = local_selection(decided.index, decided.num, block_lo, block_lo + blocks_per_rank[rank])

    rec = branches.record_floats(head_dim)
    records = None
    recv = None
    o_s = l_s = o_l = l_l = None
    if world > 1 and bsz == 1:
        rp, row_plan = exchange_rows(q_len, world)
        # every rank takes the same decision from what every rank knows: the shard plan and the shapes
        seg = hsa_module.proj_segment_len
        owns_segments = all((-(-(b if r < world - 1 else kv_len) // seg)) > -(-a // seg) for r, (a, b) in enumerate(shards))
        peer_ok = (world <= 8 and head_dim == 128 and q.dtype == torch.bfloat16 and bs in (64, 128)
                   and all(b > a for a, b in shards) and owns_segments)
        if exchange == "peer" and not peer_ok:
            raise ValueError("the peer exchange needs <= 8 ranks, bf16, head_dim 128, 64- or 128-token blocks and no empty shard")
        use_peer = peer_ok and exchange != "nccl" and not _peer_exchange_failed
        xchg = None
        if use_peer:
            xchg = _peer_exchange(world, rank, rp, heads, rec, q.device, group, required=exchange == "peer")
        if xchg is not None:
            used_tuned = branches.hsa_partials_packed(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs, xchg.local,
                                                      peer=(rp, rank, xchg.deltas))
            if not used_tuned:      # the kernel declined: deliver the records with plain peer copies instead
                records = torch.empty((1, rp * world, heads, rec), dtype=torch.float32, device=q.device)
                used_tuned = partial_records(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs, records)
                for r in range(world):
                    dst = _raw_tensor(xchg.ptrs[r], (world, rp, heads, rec), q.device)[rank]
                    dst.copy_(records[0, r * rp:(r + 1) * rp])
                records = None
            arrived = torch.zeros(1, dtype=torch.int32, device=q.device)
            dist.all_reduce(arrived, group=group)      # every rank's kernel is behind its contribution: the rows are here
            recv = xchg.local[0]
        else:
            records = torch.empty((1, rp * world, heads, rec), dtype=torch.float32, device=q.device)
            used_tuned = partial_records(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs, records)
    else:
        o_s, l_s, o_l, l_l, used_tuned = _partials_unpacked(q, k_local, v_local, kc_local, vc_local, index_l, num_l, bs)
    last_call_info.update(used_tuned=bool(used_tuned), routing="candidates" if by_candidates else "gather", ranks=world,
                          # routing exchange + (packed: one all-to-all, or a one-element all-reduce behind peer stores, and
                          # one all-gather | unpacked: two all-gathers)
                          collectives=0 if world == 1 else 3, packed_exchange=records is not None or recv is not None,
                          exchange="peer stores" if recv is not None else ("all-to-all" if records is not None else "all-gather"))

    if records is not None:
        recv = torch.empty_like(records[0])                                  # [W * rp, H, rec]: slice j of every rank
        dist.all_to_all_single(recv, records[0], group=group)
    if recv is not None:
        sparse, linear = branches.merge_packed(recv.view(world, rp * heads, rec), head_dim)
        first, count = row_plan[rank]
        out_rows = q.new_zeros((rp, heads, head_dim)) if count < rp else q.new_empty((rp, heads, head_dim))
        if count > 0:
            done = branches.gate_combine(q[:, first:first + count], sparse.view(1, rp, heads, head_dim)[:, :count],
                                         linear.view(1, rp, heads, head_dim)[:, :count], hsa_module.gate_lin,
                                         round_bf16=q.dtype == torch.bfloat16, out=out_rows[:count].unsqueeze(0))
            assert done.data_ptr() == out_rows.data_ptr()
        full = q.new_empty((world * rp, heads, head_dim))
        dist.all_gather_into_tensor(full, out_rows, group=group)
        return full[:q_len].unsqueeze(0)

    # single rank or batched input: merge everything everywhere (rows ordered [B, H, Lq] to match the normalisers)
    def rows(o):
        return o.permute(0, 2, 1, 3).reshape(1, bsz * heads * q_len, head_dim)

    packed_o = torch.cat([rows(o_s), rows(o_l)], dim=1)                    # [1, 2R, D]
    packed_l = torch.cat([l_s.reshape(1, -1), l_l.reshape(1, -1)], dim=1)  # [1, 2R]
    if world > 1:
        packed_o = all_gather_cat(packed_o, 0, group=group)
        packed_l = all_gather_cat(packed_l, 0, group=group)
    merged, _ = merge_partials(packed_o, packed_l)
    r = bsz * heads * q_len
    sparse = merged[:r].view(bsz, heads, q_len, head_dim).permute(0, 2, 1, 3)
    linear = merged[r:].view(bsz, heads, q_len, head_dim).permute(0, 2, 1, 3)
    sparse = sparse.to(torch.bfloat16).contiguous()       # the reference stores the sparse branch in bf16
    return branches.gate_combine(q, sparse, linear.contiguous(), hsa_module.gate_lin,
                                 round_bf16=q.dtype == torch.bfloat16)


def _pool_blhd(x: torch.Tensor, block_size: int) -> torch.Tensor:
    """Pool an unpadded `[B, L, H, D]` tensor -> float32 `[B, H, Nb, D]` (one C-ABI call)."""
    from . import _lib
    dev = _lib.require_cuda(x)
    bsz, length, heads, head_dim = x.shape
    nb = math.ceil(length / block_size)
    pooled = torch.empty((bsz, heads, nb, head_dim), device=dev, dtype=torch.float32)
    x = x if x.stride(-1) == 1 else x.contiguous()
    _lib.check(_lib.lib().wa_pool_blocks(_lib.t4_blhd(x), bsz, length, heads, head_dim, block_size,
                                         pooled.data_ptr(), _lib.stream_ptr(dev)))
    return pooled
