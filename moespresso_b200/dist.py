"""Multi-GPU drivers for the sparse decode path: one process per GPU, torch.distributed.

The reference is single-device; this partitioning is new.  Two cases:

* sequence sharding — independent sequences are dealt to ranks, balanced by context
  length; the step needs no collective (``assign_sequences``);
* KV-range sharding of ONE long sequence — rank g owns latent rows
  [g*R/G, (g+1)*R/G).  Per step: local indexer scores -> local exact top-k with global
  row ids -> all_gather of (score, id) candidates (k * 8 bytes per rank) -> every rank
  runs the same exact global selection (ties to the lower global id) and keeps the ids
  it owns -> local sparse attention producing un-normalised (o, m, l) partials ->
  all_gather of the partials -> log-sum-exp merge in rank order, the sink joining once.
  The result equals the single-GPU result: the selected id set bit-for-bit (scores do
  not depend on the partition), the output up to fp32 summation order.

The device operators are injected through ``ops`` so that the host-side logic
(candidate exchange, ownership, merge order) can be exercised on CPU ranks with the
gloo backend.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


def assign_sequences(lens, world: int) -> list[list[int]]:
    """Deal sequences to ranks: longest first onto the least-loaded rank (ties to the
    lower rank); each rank's list is returned in ascending sequence order."""
    lens = [int(x) for x in lens]
    order = sorted(range(len(lens)), key=lambda i: (-lens[i], i))
    load = [0] * world
    out: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += lens[i]
    return [sorted(x) for x in out]


def row_range(n_rows: int, world: int, rank: int, align: int = 128) -> tuple[int, int]:
    """Rows [lo, hi) of rank `rank`; boundaries are multiples of `align` (the score
    kernel's tile height) except the last one."""
    per = -(-n_rows // world)
    per = -(-per // align) * align
    lo = min(rank * per, n_rows)
    return lo, min(lo + per, n_rows)


@dataclass
class RangeShard:
    """This rank's slice of one sequence's tables (device tensors)."""
    kv: torch.Tensor                 # [rows_local, Dqk]
    kv_scales: torch.Tensor | None   # [rows_local] fp16 (int8 KV)
    idx_keys: torch.Tensor           # [rows_local, Di]
    row_lo: int                      # first global row owned


class CudaOps:
    """The CUDA operators behind the driver."""

    def scores(self, idx_q, idx_w, keys):
        from .deepseek_v4.indexed_attention_kernel import indexer_scores
        return indexer_scores(idx_q[None, :, None, :], idx_w[None, None, :].contiguous(), keys,
                              n_rows=int(keys.shape[0]))[0, 0]

    def topk(self, scores, k):
        from .deepseek_v4.attention import topk_select
        return topk_select(scores[None], k)[0]

    def attend_partial(self, q, kv, kv_scales, ids, scale, d_v):
        from .deepseek_v4.indexed_attention_kernel import sparse_attention
        o, ml = sparse_attention(q[None, :, None, :], kv, ids[None, None, :], None, pos0=0, window=0, ratio=0,
                                 scale=scale, d_v=d_v, kv_scales=kv_scales, n_comp=int(kv.shape[0]), partial=True,
                                 out_layout="bthd")
        return o[0, 0], ml[0, 0]          # [H, Dv], [H, 2]

    def merge(self, o_parts, ml_parts, sinks):
        from .deepseek_v4.indexed_attention_kernel import merge_partials
        return merge_partials(o_parts[:, None, None], ml_parts[:, None, None], sinks)[0, 0]

    # The index arithmetic between the kernels and the collectives, one launch each (the generic drivers below do
    # the same with a chain of element-wise torch operations, which is what the NumPy stand-ins of the CPU tests get).
    def candidates(self, scores, local_ids, row_lo, out_scores, out_ids):
        """out_scores / out_ids [k] (float32 / int32): the local top-k as (score, global id) candidates."""
        from . import _abi, _torchabi as _t
        a = _abi.RangeCandidatesArgs()
        a.scores, a.ids, a.out_scores, a.out_ids = _t.ptr(scores), _t.ptr(local_ids), _t.ptr(out_scores), _t.ptr(out_ids)
        a.k, a.row_lo = int(local_ids.numel()), int(row_lo)
        _abi.check(_t.launch("range_candidates", _abi.load().mxb_range_candidates, a))

    def local_ids(self, pos, cand_ids, rank_stride, row_lo, rows_local, out):
        """out [k] int32: the globally selected rows this rank owns, as local ids (-1 elsewhere)."""
        from . import _abi, _torchabi as _t
        a = _abi.RangeLocalIdsArgs()
        a.pos, a.cand_ids, a.cand_rank_stride, a.out = _t.ptr(pos), _t.ptr(cand_ids), int(rank_stride), _t.ptr(out)
        a.k, a.row_lo, a.rows_local = int(pos.numel()), int(row_lo), int(rows_local)
        _abi.check(_t.launch("range_local_ids", _abi.load().mxb_range_local_ids, a))


def _all_gather(t: torch.Tensor, group=None) -> torch.Tensor:
    world = dist.get_world_size(group)
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t.contiguous(), group=group)
    return torch.stack(out)


def range_step_candidates(idx_q, idx_w, shard: RangeShard, *, k: int, ops):
    """Steps 1-2 of the range-sharded decode step on one rank: local scores and the local exact top-k as
    (score, global id) candidates, ascending by id, padded with (-inf, -1)."""
    rows_local = int(shard.idx_keys.shape[0])
    dev = idx_q.device
    if rows_local > 0:
        scores = ops.scores(idx_q, idx_w, shard.idx_keys)
        local_ids = ops.topk(scores, k).long()
        cand_scores = torch.where(local_ids >= 0, scores[local_ids.clamp(min=0)],
                                  torch.full((k,), float("-inf"), device=dev))
        cand_ids = torch.where(local_ids >= 0, local_ids + shard.row_lo, torch.full_like(local_ids, -1))
    else:
        cand_scores = torch.full((k,), float("-inf"), device=dev)
        cand_ids = torch.full((k,), -1, dtype=torch.int64, device=dev)
    return cand_scores.float(), cand_ids


def range_step_partial(q, shard: RangeShard, all_scores, all_ids, *, k: int, scale: float, d_v: int, ops,
                       want_ids: bool = True):
    """Steps 4-5 on one rank, given every rank's candidates concatenated in rank order: the same exact global
    selection on every rank (ties go to the lower position == lower global id, because ranks own ascending row
    ranges and each list is ascending), then partial attention over the rows this rank owns.
    Returns (o [H,d_v], ml [H,2], global ids attended here)."""
    rows_local = int(shard.idx_keys.shape[0])
    dev = q.device
    pos = ops.topk(all_scores.reshape(-1), k).long()
    chosen = torch.where(pos >= 0, all_ids.reshape(-1)[pos.clamp(min=0)], torch.full_like(pos, -1))
    hi = shard.row_lo + rows_local
    mine = (chosen >= shard.row_lo) & (chosen < hi)
    my_ids = torch.where(mine, chosen - shard.row_lo, torch.full_like(chosen, -1)).to(torch.int32)
    if rows_local > 0:
        o, ml = ops.attend_partial(q, shard.kv, shard.kv_scales, my_ids, scale, d_v)
    else:   # no rows here: m = -inf, l = 0
        H = int(q.shape[0])
        o = torch.zeros((H, d_v), dtype=torch.float32, device=dev)
        ml = torch.stack([torch.full((H,), float("-inf"), device=dev), torch.zeros(H, device=dev)], dim=1)
    # the list of attended ids has a data-dependent length (a device-to-host round trip): only on request
    return o.float(), ml.float(), (chosen[mine] if want_ids else None)


def range_sharded_decode_step(q, idx_q, idx_w, shard: RangeShard, *, k: int, scale: float, d_v: int, sinks=None,
                              ops=None, group=None, return_ids: bool = False):
    """One decode step of ONE sequence whose rows are range-sharded over the ranks of
    `group`.  q [H,Dqk], idx_q [Hi,Di], idx_w [Hi] are replicated.  Every rank returns the
    full output [H,d_v] (and, on request, the global ids this rank attended)."""
    ops = ops or CudaOps()
    # 1-2: local scores and local exact top-k
    cand_scores, cand_ids = range_step_candidates(idx_q, idx_w, shard, k=k, ops=ops)
    # 3: exchange candidates (k (score, id) pairs per rank)
    all_scores = _all_gather(cand_scores, group)
    all_ids = _all_gather(cand_ids, group)
    # 4-5: identical global selection, local partial attention
    o, ml, attended = range_step_partial(q, shard, all_scores, all_ids, k=k, scale=scale, d_v=d_v, ops=ops)
    # 6-7: exchange partials, merge in rank order, sink joins once
    out = ops.merge(_all_gather(o, group), _all_gather(ml, group), sinks)
    if return_ids:
        return out, attended
    return out


class RangeDecodePlan:
    """The range-sharded decode step of one sequence with everything between the collectives captured as CUDA
    graphs: per step three graph launches and two ``all_gather`` calls (candidates: 8 bytes x k per rank; partials:
    (d_v + 2) floats per head per rank), no allocation and no device-to-host round trip.  Results are those of
    ``range_sharded_decode_step`` bit for bit.  The shard's tensors are captured by address."""

    def __init__(self, shard: RangeShard, *, heads: int, d_qk: int, idx_heads: int, idx_dim: int, k: int,
                 scale: float, d_v: int, q_dtype=torch.bfloat16, sinks=None, group=None, ops=None,
                 graph: bool = True):
        dev = shard.kv.device
        self.shard, self.k, self.scale, self.d_v, self.sinks = shard, int(k), float(scale), int(d_v), sinks
        self.group, self.ops = group, ops or CudaOps()
        world = dist.get_world_size(group)
        self.q = torch.zeros((heads, d_qk), dtype=q_dtype, device=dev)
        self.idx_q = torch.zeros((idx_heads, idx_dim), dtype=q_dtype, device=dev)
        self.idx_w = torch.zeros((idx_heads,), dtype=torch.float32, device=dev)
        # candidates travel as one tensor: row 0 = the float32 scores' bits, row 1 = global row ids (< 2^31)
        self.cand = torch.empty((2, self.k), dtype=torch.int32, device=dev)
        self.all_cand = torch.empty((world, 2, self.k), dtype=torch.int32, device=dev)
        # partials travel as one tensor: [H, d_v] un-normalised output, then (m, l)
        self.part = torch.empty((heads, self.d_v + 2), dtype=torch.float32, device=dev)
        self.all_part = torch.empty((world, heads, self.d_v + 2), dtype=torch.float32, device=dev)
        self.mine = torch.empty((self.k,), dtype=torch.int32, device=dev)   # the selected rows this rank owns
        self.out = None
        self._graphs = None
        if graph:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._candidates()
                    self.all_cand.copy_(self.cand[None].expand_as(self.all_cand))
                    self._partial()
                    self.all_part.copy_(self.part[None].expand_as(self.all_part))
                    self._merge()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            graphs = []
            for phase in (self._candidates, self._partial, self._merge):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    phase()
                graphs.append(g)
            self._graphs = graphs

    def _fused(self) -> bool:
        return hasattr(self.ops, "candidates") and int(self.shard.idx_keys.shape[0]) > 0

    def _candidates(self):
        if self._fused():    # scores -> local top-k -> candidates written straight into the send buffer
            scores = self.ops.scores(self.idx_q, self.idx_w, self.shard.idx_keys)
            self.ops.candidates(scores, self.ops.topk(scores, self.k), self.shard.row_lo,
                                self.cand[0].view(torch.float32), self.cand[1])
            return
        cs, ci = range_step_candidates(self.idx_q, self.idx_w, self.shard, k=self.k, ops=self.ops)
        self.cand[0].copy_(cs.contiguous().view(torch.int32))
        self.cand[1].copy_(ci)

    def _partial(self):
        if self._fused():    # global selection over every rank's candidates -> the rows this rank owns -> attention
            pos = self.ops.topk(self.all_cand[:, 0].contiguous().view(torch.float32).reshape(-1), self.k)
            self.ops.local_ids(pos, self.all_cand[:, 1], self.all_cand.stride(0), self.shard.row_lo,
                               int(self.shard.idx_keys.shape[0]), self.mine)
            o, ml = self.ops.attend_partial(self.q, self.shard.kv, self.shard.kv_scales, self.mine, self.scale, self.d_v)
        else:
            o, ml, _ = range_step_partial(self.q, self.shard, self.all_cand[:, 0].contiguous().view(torch.float32),
                                          self.all_cand[:, 1].long(), k=self.k, scale=self.scale, d_v=self.d_v,
                                          ops=self.ops, want_ids=False)
        self.part[:, :self.d_v].copy_(o)
        self.part[:, self.d_v:].copy_(ml)

    def _merge(self):
        self.out = self.ops.merge(self.all_part[:, :, :self.d_v].contiguous(),
                                  self.all_part[:, :, self.d_v:].contiguous(), self.sinks)

    def step(self, q, idx_q, idx_w):
        """One decode step; q [H,Dqk], idx_q [Hi,Di], idx_w [Hi] replicated on every rank.  Returns out [H,d_v]
        (the plan's own buffer when graphs are in use: consume it before the next step)."""
        self.q.copy_(q, non_blocking=True)
        self.idx_q.copy_(idx_q, non_blocking=True)
        self.idx_w.copy_(idx_w, non_blocking=True)
        phases = self._graphs and [g.replay for g in self._graphs] or [self._candidates, self._partial, self._merge]
        phases[0]()
        dist.all_gather_into_tensor(self.all_cand, self.cand, group=self.group)
        phases[1]()
        dist.all_gather_into_tensor(self.all_part, self.part, group=self.group)
        phases[2]()
        return self.out

    def timed_step(self, q, idx_q, idx_w, reps: int = 20) -> list[float]:
        """Device time of the five parts of a step, in microseconds, averaged over ``reps`` steps: local candidates,
        all-gather of the candidates, local partial attention, all-gather of the partials, merge.  CUDA events on
        the current stream (the collectives run on NCCL's stream; the events bracket the waits for them)."""
        phases = self._graphs and [g.replay for g in self._graphs] or [self._candidates, self._partial, self._merge]
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(reps)]
        for e in evs:
            self.q.copy_(q, non_blocking=True)
            self.idx_q.copy_(idx_q, non_blocking=True)
            self.idx_w.copy_(idx_w, non_blocking=True)
            e[0].record()
            phases[0]()
            e[1].record()
            dist.all_gather_into_tensor(self.all_cand, self.cand, group=self.group)
            e[2].record()
            phases[1]()
            e[3].record()
            dist.all_gather_into_tensor(self.all_part, self.part, group=self.group)
            e[4].record()
            phases[2]()
            e[5].record()
        torch.cuda.synchronize(self.q.device)
        return [sum(e[i].elapsed_time(e[i + 1]) for e in evs) / reps * 1e3 for i in range(5)]


def numpy_lens_to_tables(c: dict, seqs: list[int]) -> dict:
    """Slice a synthetic batch (moespresso_b200.synth.config3 layout) down to `seqs`,
    re-basing row_start; used by the sequence-sharded drivers and the benchmark."""
    lens = np.asarray([c["lens"][i] for i in seqs], dtype=np.int64)
    parts = [slice(int(c["row_start"][i]), int(c["row_start"][i] + c["lens"][i])) for i in seqs]
    cat = lambda a: np.concatenate([a[p] for p in parts], axis=0) if parts else a[:0]
    out = dict(c)
    out.update(lens=lens, row_start=np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int64) if len(seqs) else
               np.zeros(0, np.int64), kv=cat(c["kv"]), kv_scales=cat(c["kv_scales"]),
               idx_key_bits=cat(c["idx_key_bits"]), q=c["q"][seqs], idx_q=c["idx_q"][seqs], idx_w=c["idx_w"][seqs])
    return out
