"""Ratio-4 compressed-KV sparse prefill of one chunk: indexer scores -> per-token top-k ->
indexed sparse attention.

Operator-calling part of the reference's ``_Ratio4PrefillFastAttention.__call__``
(``src/moespresso/runtime/deepseek_v4/model.py:1320-1480``): scores by the tiled score
kernel with the causal compressed-row mask (:1434-1441), ``argpartition`` + ascending sort
(:1442-1451), then the indexed prefill consumer (:1453-1472); when the pool holds no more
than ``k`` rows every row is selected (:1393-1395).  Projections, RoPE and the QAT pre-op
are outside this operator.

The [tokens x rows] fp32 score matrix is never materialised: tokens are processed in
chunks whose scores (``token_chunk`` x rows x 4 bytes) are written to one reused buffer that
stays in the 126 MB L2 between the score kernel and the selection kernel.  The default chunk
is four tokens per SM (592 on a B200: 78 MB of scores at 32768 rows), which fills whole waves
of both kernels; measured per 4096-token chunk: 128 -> 7.5 ms, 256 -> 5.5, 592 -> 5.0,
1024 -> 5.0, 4096 (537 MB of scores) -> 4.9.
"""
from __future__ import annotations

import torch

from .attention import topk_select
from .indexed_attention_kernel import indexer_scores_tiled_live, sparse_attention


def sparse_prefill_step(q, comp_kv, idx_q, idx_keys, idx_w, *, pos0: int, ratio: int = 4, k: int = 512,
                        scale=None, d_v=None, sinks=None, raw_kv=None, window: int = 128, raw_start: int = 0,
                        token_chunk: int | None = None, return_ids: bool = False):
    """q [T,H,Dqk]; comp_kv [R,Dqk]; idx_q [T,Hi,Di]; idx_keys [R,Di]; idx_w [T,Hi] float32
    (all scale factors folded in); raw_kv [raw_cap,Dqk] or None.  Token t sits at ``pos0 + t``.
    Returns float32 [T,H,d_v] (and the int32 ids [T,k], ascending, -1 padded)."""
    T, H, Dqk = (int(x) for x in q.shape)
    R = int(comp_kv.shape[0])
    dev = q.device
    kk = min(int(k), R)
    if R <= int(k):
        # every pooled row is a candidate; visibility is still applied by the attention kernel's walk
        ids = torch.arange(R, dtype=torch.int32, device=dev).expand(T, R).contiguous()
    else:
        ids = torch.empty((T, kk), dtype=torch.int32, device=dev)
        if token_chunk is None:
            token_chunk = 4 * torch.cuda.get_device_properties(dev).multi_processor_count
        chunk = max(1, min(int(token_chunk), T))
        buf = torch.empty((1, chunk, R), dtype=torch.float32, device=dev)
        iq = idx_q.permute(1, 0, 2)[None]            # [1,Hi,T,Di]
        for t0 in range(0, T, chunk):
            n = min(chunk, T - t0)
            scores = indexer_scores_tiled_live(iq[:, :, t0:t0 + n], idx_w[None, t0:t0 + n].contiguous(),
                                               idx_keys[None], pos0=pos0 + t0, ratio=ratio, out=buf[:, :n])
            ids[t0:t0 + n] = topk_select(scores[0, :n], kk)
    out = sparse_attention(q.permute(1, 0, 2)[None], comp_kv, ids[None], sinks, pos0=pos0, window=window,
                           ratio=ratio, raw_kv=None if raw_kv is None else raw_kv[None], raw_start=raw_start,
                           scale=scale, d_v=d_v, n_comp=R, out_layout="bthd")[0]
    return (out, ids) if return_ids else out
