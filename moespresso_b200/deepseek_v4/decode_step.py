"""Batched sparse decode step: indexer score -> top-k -> indexed sparse attention.

The reference runs this chain once per layer for batch 1
(``_IndexerDS4ScoreContract.__call__`` then gather + SDPA,
``src/moespresso/runtime/deepseek_v4/model.py:867-1065,1604-1650``; fused island
``fused_decode_prep`` / ``fused_decode_sdpa``,
``src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:669-786``).  Here a
ragged batch of sequences shares one flat latent-KV table and one flat index-key
table; every row of every sequence is visible (decode applies no causal mask,
model.py:1047-1055).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .attention import topk_select
from .indexed_attention_kernel import DIGIT_BINS, indexer_scores, scan_counts_digits, sparse_attention


@dataclass
class LatentCache:
    """Device-resident tables of a batch of sequences.

    kv         [rows_total, Dqk]  int8 / bf16 / fp16 / fp32 latent rows (K = row, V = row[:d_v])
    kv_scales  [rows_total]       fp16 per-row scale (int8 only, else None)
    idx_keys   [rows_total, Di]   indexer keys (fp8-e4m3 / bf16 / fp16 / fp32)
    row_start  [B] int64, row_count [B] int32; max_rows = longest sequence (host int)
    """
    kv: torch.Tensor
    kv_scales: torch.Tensor | None
    idx_keys: torch.Tensor
    row_start: torch.Tensor
    row_count: torch.Tensor
    max_rows: int

    @property
    def batch(self) -> int:
        return int(self.row_start.numel())


def quantize_kv_int8(rows):
    """Per-token int8 quantisation of latent KV rows ``[n, width]`` (float32 / float16 / bfloat16): returns
    ``(q int8 [n, width], scales float16 [n])`` with ``rows ~= q * scales[:, None]`` — the cache format the sparse
    decode operators read through ``kv_scales``."""
    from .. import _abi
    from .. import _torchabi as _t
    if rows.ndim != 2 or rows.shape[0] == 0 or rows.shape[1] == 0:
        raise ValueError("rows must be a non-empty [n, width] matrix")
    if rows.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("rows must be float32, float16, or bfloat16")
    dev = _t.require_cuda(rows)
    rows = rows.contiguous()
    q = torch.empty(rows.shape, dtype=torch.int8, device=dev)
    scales = torch.empty((rows.shape[0],), dtype=torch.float16, device=dev)
    a = _abi.QuantizeKvInt8Args()
    a.x, a.x_dtype, a.q, a.scales = _t.ptr(rows), _t.dtype_code(rows), _t.ptr(q), _t.ptr(scales)
    a.n_rows, a.width = int(rows.shape[0]), int(rows.shape[1])
    _abi.check(_t.launch("quantize_kv_int8", _abi.load().mxb_quantize_kv_int8, a))
    return q, scales


def sparse_decode_step(q, idx_q, idx_w, cache: LatentCache, *, k: int, scale: float, d_v: int,
                       sinks=None, out_dtype=torch.float32, exact_fp32: bool = False, partial: bool = False,
                       return_ids: bool = False, return_scores: bool = False, digit_hist=None):
    """q [B,H,Dqk]; idx_q [B,Hi,Di]; idx_w [B,Hi] float32.  Returns out [B,H,d_v]
    (plus ids [B,k] int32 ascending / scores flat [rows_total] on request).  ``digit_hist``: a zeroed int32
    ``[B, 2048]`` scratch that lets the scan count the selection's first radix digit while it writes the scores
    (used when the scan kernel takes the call, see ``scan_counts_digits``; it is zero again afterwards)."""
    B = cache.batch
    q4 = idx_q[:, :, None, :]
    if digit_hist is not None and not scan_counts_digits(q4, cache.idx_keys, n_tokens=1, ratio=0, exact_fp32=exact_fp32):
        digit_hist = None
    scores = indexer_scores(q4, idx_w[:, None, :].contiguous(), cache.idx_keys,
                            n_rows=cache.max_rows, row_start=cache.row_start, row_count=cache.row_count,
                            exact_fp32=exact_fp32, digit_hist=digit_hist)
    ids = topk_select(scores, k, valid=cache.row_count, row_start=cache.row_start, n=cache.max_rows,
                      digit_hist=digit_hist)
    res = sparse_attention(q[:, :, None, :], cache.kv, ids[:, None, :], sinks, pos0=0, window=0, ratio=0,
                           scale=scale, d_v=d_v, kv_scales=cache.kv_scales, comp_row_start=cache.row_start,
                           comp_row_count=cache.row_count, n_comp=cache.max_rows, out_dtype=out_dtype,
                           partial=partial)
    if partial:
        out, ml = res
        out = (out[:, :, 0, :], ml[:, 0])
    else:
        out = res[:, :, 0, :]
    extra = []
    if return_ids:
        extra.append(ids)
    if return_scores:
        extra.append(scores)
    return (out, *extra) if extra else out


class SparseDecodePlan:
    """A decode step with fixed shapes, pre-allocated buffers and (by default) one CUDA
    graph holding its launches, so that a step costs one graph launch on the host.

    The cache tensors are captured by address: the plan stays valid while ``cache`` keeps
    its storage (rows appended in place within ``max_rows`` and updated ``row_count`` are
    picked up, because the kernels read the counts from device memory).
    """

    def __init__(self, cache: LatentCache, *, heads: int, d_qk: int, idx_heads: int, idx_dim: int, k: int,
                 scale: float, d_v: int, q_dtype=torch.bfloat16, out_dtype=torch.float32, sinks=None,
                 graph: bool = True, count_digits_in_scan: bool = False):
        dev = cache.kv.device
        B = cache.batch
        self.cache, self.k, self.scale, self.d_v, self.sinks, self.out_dtype = cache, int(k), float(scale), int(d_v), sinks, out_dtype
        # one device buffer behind the three inputs, so that a caller who keeps its step inputs in one pinned
        # host buffer of the same layout (``host_views``) pays for a single host->device copy per step
        esz = torch.empty((), dtype=q_dtype).element_size()
        nq, niq, nw = B * heads * d_qk * esz, B * idx_heads * idx_dim * esz, B * idx_heads * 4
        self._offs = (0, (nq + 255) // 256 * 256, ((nq + 255) // 256 * 256) + (niq + 255) // 256 * 256)
        self._sizes = (nq, niq, nw)
        self._shapes = ((B, heads, d_qk), (B, idx_heads, idx_dim), (B, idx_heads))
        self._dtypes = (q_dtype, q_dtype, torch.float32)
        self.packed = torch.zeros(self._offs[2] + (nw + 255) // 256 * 256, dtype=torch.uint8, device=dev)
        self.q, self.idx_q, self.idx_w = self._views(self.packed)
        # Optional: the scan counts the selection's first radix digit (scratch, zero between steps).  Off by
        # default: on a B200 the scan is co-limited by instruction issue, and the extra key + shared-memory atomic
        # per score cost it more (37.8 -> 42.2 us at batch 32 x 82 K rows) than the selection saved (20.5 -> 19.3 us).
        self.digit_hist = None
        if count_digits_in_scan and scan_counts_digits(self.idx_q[:, :, None, :], cache.idx_keys, n_tokens=1, ratio=0):
            self.digit_hist = torch.zeros((B, DIGIT_BINS), dtype=torch.int32, device=dev)
        self.graph = None
        self.out = None
        self.ids = None
        if graph:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.out, self.ids = self._step()
            self.graph = g
            # the same step as two graphs (select, attend): a host-fed step copies q on a second stream while the
            # selection runs, because only the attention reads q
            g1, g2 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g1):
                self._ids2 = self._select()
            with torch.cuda.graph(g2):
                self._out2 = self._attend(self._ids2)
            self._graph_select, self._graph_attend = g1, g2
        self._copy_stream = torch.cuda.Stream(device=dev)
        self._q_copied = torch.cuda.Event()
        self._attend_done = torch.cuda.Event()
        self._attend_done.record(torch.cuda.current_stream(dev))

    def _views(self, buf):
        return tuple(buf[o:o + n].view(dt).view(sh)
                     for o, n, sh, dt in zip(self._offs, self._sizes, self._shapes, self._dtypes))

    def host_buffer(self):
        """A pinned host buffer with the plan's input layout and its (q, idx_q, idx_w) views.  Fill the views,
        then ``run_packed(buffer)``: one host->device copy instead of three."""
        buf = torch.zeros(self.packed.numel(), dtype=torch.uint8).pin_memory()
        return buf, self._views(buf)

    def run_packed(self, host_buf):
        """One step fed from a pinned host buffer laid out like ``host_buffer()``.  The small selection inputs are
        copied first; q (97 % of the bytes) travels on a second stream while the scores and the top-k run, and the
        attention waits for it.  Returns out [B,H,d_v] (asynchronously, on the current stream)."""
        main = torch.cuda.current_stream(self.packed.device)
        nq = self._offs[1]
        if self.graph is None:
            self.packed.copy_(host_buf, non_blocking=True)
            return self.launch()
        from .. import _abi
        self.packed[nq:].copy_(host_buf[nq:], non_blocking=True)       # selection inputs first: the device starts at once
        self._graph_select.replay()
        self._copy_stream.wait_event(self._attend_done)                # the previous step's attention has read q
        _abi.check(_abi.load().mxb_copy_h2d_async(self.packed.data_ptr(), host_buf.data_ptr(), nq,
                                                  self._copy_stream.cuda_stream))
        self._q_copied.record(self._copy_stream)
        main.wait_event(self._q_copied)
        self._graph_attend.replay()
        self._attend_done.record(main)
        return self._out2

    def _select(self):
        scores = indexer_scores(self.idx_q[:, :, None, :], self.idx_w[:, None, :].contiguous(), self.cache.idx_keys,
                                n_rows=self.cache.max_rows, row_start=self.cache.row_start,
                                row_count=self.cache.row_count, digit_hist=self.digit_hist)
        return topk_select(scores, self.k, valid=self.cache.row_count, row_start=self.cache.row_start,
                           n=self.cache.max_rows, digit_hist=self.digit_hist)

    def _attend(self, ids):
        return sparse_attention(self.q[:, :, None, :], self.cache.kv, ids[:, None, :], self.sinks, pos0=0, window=0,
                                ratio=0, scale=self.scale, d_v=self.d_v, kv_scales=self.cache.kv_scales,
                                comp_row_start=self.cache.row_start, comp_row_count=self.cache.row_count,
                                n_comp=self.cache.max_rows, out_dtype=self.out_dtype)[:, :, 0, :]

    def _step(self):
        return sparse_decode_step(self.q, self.idx_q, self.idx_w, self.cache, k=self.k, scale=self.scale,
                                  d_v=self.d_v, sinks=self.sinks, out_dtype=self.out_dtype, return_ids=True,
                                  digit_hist=self.digit_hist)

    def load_inputs(self, q, idx_q, idx_w) -> None:
        """Copy one step's inputs (device or pinned-host tensors) into the plan's buffers."""
        self.q.copy_(q, non_blocking=True)
        self.idx_q.copy_(idx_q, non_blocking=True)
        self.idx_w.copy_(idx_w, non_blocking=True)

    def launch(self):
        """Run the step on the inputs currently in the plan's buffers; returns out [B,H,d_v]."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self.out, self.ids = self._step()
        return self.out

    def run(self, q, idx_q, idx_w):
        self.load_inputs(q, idx_q, idx_w)
        return self.launch()
