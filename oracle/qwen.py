"""CPU oracle for the Qwen/Ornith causal GQA prefill attention (NumPy).

TEST INFRASTRUCTURE ONLY (same rule as ``oracle/ds4.py``).

PARITY UNPINNED: the reference computes this operator inside the third-party
package ``mlx-kquant`` 0.3.0 (git e165cafafa149493d298871c610e29e95ffa8f10,
``sdpa_fa_prefill_q8``), whose source is not part of the reference tree, and
its own tests for the call site (tests/test_qwen_flash_prefill_attention.py)
need MLX and are skipped on Linux.  This file restates the published
definition the reference's wrapper relies on
(src/moespresso/runtime/qwen/full_attention.py:279-397): softmax(Q K^T * scale
+ causal) V with each KV head shared by Hq/Hkv query heads (q head h uses kv
head h // (Hq/Hkv)), every past key visible, then ``out * sigmoid(gate)``
(:396-397).
"""
from __future__ import annotations

import numpy as np


def causal_gqa_prefill(q, k, v, gate=None, *, scale, past_len: int = 0, dtype=np.float64,
                       q_rows=None) -> np.ndarray:
    """q [S, Hq, D]; k, v [P+S, Hkv, D] (first ``past_len`` keys are the past,
    all visible); gate [S, Hq, D] or None.  Key j is visible to query row i iff
    j <= i + past_len.  Returns [S, Hq, D] (``q_rows``: only those query rows,
    used to bound the timed CPU baseline)."""
    f = dtype
    q = np.asarray(q, dtype=f)
    k = np.asarray(k, dtype=f)
    v = np.asarray(v, dtype=f)
    S, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    rows = np.arange(S) if q_rows is None else np.asarray(q_rows)
    out = np.zeros((rows.size, Hq, D), dtype=f)
    kpos = np.arange(k.shape[0])
    for h in range(Hq):
        kh = k[:, h // group, :]
        vh = v[:, h // group, :]
        s = (q[rows, h, :] @ kh.T) * f(scale)
        s = np.where(kpos[None, :] <= (rows[:, None] + past_len), s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        p = np.exp(s - m)
        out[:, h, :] = (p @ vh) / p.sum(axis=1, keepdims=True)
    if gate is not None:
        g = np.asarray(gate, dtype=f)[rows]
        out = out * (1.0 / (1.0 + np.exp(-g)))
    return out
