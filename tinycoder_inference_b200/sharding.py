"""Partitioning of the attention hot path over the GPUs of one box.

The reference engine is single-device (no collectives, no device selection), so
everything here is new capability.  Three independent axes:

* KV-head groups -- each rank holds the K/V rows of a contiguous block of kv heads
  and the q heads that read them.  Outputs are disjoint [nHeads_local][hd] slices;
  no data-path collective (an all-gather only if one rank wants the full vector).
* sequences -- whole sequences are assigned to ranks so that the TOKEN counts are
  balanced (longest-processing-time greedy on the context lengths).  No collective.
* the context axis -- one sequence's rows are cut into contiguous ranges; each rank
  computes split-KV partials (m, l, acc) over its range and the partials are
  exchanged (all-gather over NCCL, a few tens of KB) and merged with the same
  log-sum-exp rule that merges chunks inside one GPU.

The planning functions are pure Python (tested on CPU); `gather_partials` works on
any torch.distributed backend (gloo on CPU tensors in the tests, NCCL on device
tensors in the bench).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class HeadShard:
    kv_lo: int   # first kv head of this rank
    kv_hi: int   # one past the last
    q_lo: int    # first q head (kv_lo * group)
    q_hi: int


def plan_kv_head_shards(nHeads: int, nKV: int, parts: int) -> List[HeadShard]:
    """Contiguous kv-head blocks for `parts` ranks (parts must divide nKV)."""
    if nKV % parts != 0:
        raise ValueError(f"{parts} head shards do not divide {nKV} kv heads")
    group = nHeads // nKV
    per = nKV // parts
    return [HeadShard(r * per, (r + 1) * per, r * per * group, (r + 1) * per * group) for r in range(parts)]


def plan_sequence_shards(lens: Sequence[int], parts: int) -> List[List[int]]:
    """Sequence indices per rank, balanced by tokens: longest first, always onto
    the rank with the fewest tokens so far (ties to the lower rank)."""
    order = sorted(range(len(lens)), key=lambda i: (-int(lens[i]), i))
    load = [0] * parts
    out: List[List[int]] = [[] for _ in range(parts)]
    for i in order:
        r = min(range(parts), key=lambda x: (load[x], x))
        out[r].append(i)
        load[r] += int(lens[i])
    return [sorted(x) for x in out]


def plan_context_ranges(length: int, parts: int, quantum: int = 256) -> List[Tuple[int, int]]:
    """Contiguous row ranges [lo, hi) of one sequence for `parts` ranks, cut at
    multiples of `quantum` rows (the decode kernel's stage size) so that no rank
    carries a ragged first tile; empty ranges are allowed for short sequences."""
    blocks = (length + quantum - 1) // quantum
    out = []
    lo = 0
    for r in range(parts):
        nb = blocks // parts + (1 if r < blocks % parts else 0)
        hi = min(length, lo + nb * quantum)
        out.append((lo, hi))
        lo = hi
    return out


@dataclass(frozen=True)
class GridPlan:
    head_parts: int   # ranks along the kv-head axis
    seq_parts: int    # ranks along the sequence axis
    ctx_parts: int    # ranks along the context axis

    def coords(self, rank: int) -> Tuple[int, int, int]:
        """(head index, sequence index, context index) of a rank; the head axis is
        the fastest so that the ranks that exchange partials (same head and
        sequence group, different context index) are `head_parts * seq_parts` apart."""
        return rank % self.head_parts, (rank // self.head_parts) % self.seq_parts, rank // (
            self.head_parts * self.seq_parts)


def plan_grid(world: int, nKV: int, n_sequences: int, prefer_context: bool = False) -> GridPlan:
    """Fill `world` ranks: kv-head groups first (no collective at all), then whole
    sequences, and only what is left over goes to the context axis."""
    head = 1
    while head * 2 <= min(world, nKV) and nKV % (head * 2) == 0 and world % (head * 2) == 0:
        head *= 2
    if prefer_context:
        head = 1
    rest = world // head
    seq = 1
    while seq * 2 <= min(rest, max(1, n_sequences)) and rest % (seq * 2) == 0:
        seq *= 2
    return GridPlan(head, seq, rest // seq)


def gather_partials(acc, m, l, group=None):
    """All-gather split-KV partials over the ranks of `group`.

    acc [nH][C][hd], m, l [nH][C] on every rank -> ([nH][W*C][hd], [nH][W*C], [nH][W*C])
    laid out as the merge expects (chunk slots of rank 0, then rank 1, ...).  Slots a
    rank did not write must hold l == 0; the merge skips them."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    outs = []
    for t in (acc, m, l):
        t = t.contiguous()
        buf = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(buf, t, group=group)
        outs.append(torch.cat(buf, dim=1).contiguous())
    return tuple(outs)


class ContextSplitDecoder:
    """One decode token attended over a context that is split by rows across the ranks of
    `group`.  Every rank holds rows [0, local_len) of ITS range in its own pool and runs the
    split-KV kernel in partials-only form; then

    * exchange="p2p" (default when symmetric memory can be set up): one launch of the
      exchange-merge kernel per rank -- it merges the rank's chunks, stores the result into
      every peer's buffer over NVLink and merges what the peers stored here;
    * exchange="nccl": the rank's [acc | m | l] block is all-gathered and merged by
      tc_attn_merge_gathered.

    Buffers are allocated once; a step is two or three enqueues and can be captured in a
    CUDA graph."""

    def __init__(self, nHeads, nKV, hd, max_local_len, group=None, chunk_slots=64, exchange="p2p"):
        import torch
        import torch.distributed as dist

        from . import ops

        self.nH, self.nKV, self.hd, self.group = nHeads, nKV, hd, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.C = chunk_slots
        ml = nHeads * self.C
        self.block = torch.zeros(ml * hd + 2 * ml, dtype=torch.float32, device="cuda")
        self.acc = self.block[:ml * hd]
        self.m = self.block[ml * hd:ml * hd + ml]
        self.l = self.block[ml * hd + ml:]
        self.max_local_len = max_local_len
        self.exchange = exchange
        if exchange == "p2p":
            words = ops.exchange_bytes(nHeads, hd, self.world) // 4
            if self.world > 1:
                import torch.distributed._symmetric_memory as symm

                self.xbuf = symm.empty(words, dtype=torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
                self.xbuf.zero_()
                self.handle = symm.rendezvous(self.xbuf, group if group is not None else dist.group.WORLD)
                self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
                torch.cuda.synchronize()
                dist.barrier(group)
            else:
                self.xbuf = torch.zeros(words, dtype=torch.float32, device="cuda")
                self.ptrs = [self.xbuf.data_ptr()]
        else:
            self.gathered = torch.zeros(self.world * self.block.numel(), dtype=torch.float32, device="cuda")

    def __call__(self, q, k8, v8, ks, vs, out, local_len, invSqrt=None, pdl=False):
        import torch.distributed as dist

        from . import ops

        used = 0
        if self.exchange != "p2p":
            self.l.zero_()   # chunk slots this rank does not write must read as empty
        if local_len > 0:
            used = ops.decode_i8_batch(q, k8, v8, ks, vs, out, (self.acc, self.m, self.l), None, 1, self.nH,
                                       self.nKV, self.hd, local_len, self.C, invSqrt=invSqrt, partials_only=True,
                                       pdl=pdl, prefetch_rows=local_len - 1 if pdl else 0)
        if self.exchange == "p2p":
            ops.merge_exchange((self.acc, self.m, self.l), out, self.nH, self.C, used, self.hd, self.ptrs, self.rank,
                               pdl=pdl)
            return
        if self.world > 1:
            dist.all_gather_into_tensor(self.gathered, self.block, group=self.group)
            src = self.gathered
        else:
            src = self.block
        ops.merge_gathered(src, out, self.nH, self.world, self.C, self.hd)


def decode_i8_context_split(q, k8, v8, ks, vs, out, nHeads, nKV, hd, local_len, numChunks, invSqrt=None,
                            group=None):
    """One decode token attended over a context that is split by rows across the
    ranks of `group`: every rank holds rows [0, local_len) of ITS range in its own
    pool, runs the split-KV kernel in partials-only form, the (m, l, acc) partials
    are all-gathered and merged on every rank.  Returns nothing; `out` [1][nH][hd]."""
    import torch

    from . import ops

    acc, m, l = ops.workspace(1, nHeads, hd, numChunks)
    l.zero_()   # chunk slots this rank does not write must read as empty
    m.fill_(-1e30)
    acc.zero_()
    if local_len > 0:
        ops.decode_i8_batch(q, k8, v8, ks, vs, out, (acc, m, l), None, 1, nHeads, nKV, hd, local_len, numChunks,
                            invSqrt=invSqrt, partials_only=True)
    gacc, gm, gl = gather_partials(acc.view(nHeads, numChunks, hd), m.view(nHeads, numChunks),
                                   l.view(nHeads, numChunks), group)
    ops.merge_partials(gacc, gm, gl, out, 1, nHeads, gm.shape[1], hd)
