"""Fixed-capacity decode state for the DS4 indexer chain
(reference: src/moespresso/runtime/deepseek_v4/fixed_decode_state.py and its call site
runtime/deepseek_v4/model.py:905-944).

A decode loop appends one pooled row every ``ratio`` tokens.  The derived caches of that pool (the indexer's
QAT'd rows, the FP8-rounded KV rows) are kept in buffers of the pool's full capacity and appended IN PLACE, so
that their addresses never change (a captured CUDA graph stays valid) and only the new rows are transformed;
consumers read the valid-row count from a small device array and mask the rest.

``decode_step_params``      the per-token (position, valid rows) array (:186-193)
``pad_scores_to_capacity``  scores at and past the valid-row count become -inf, the valid prefix passes bitwise (:196-208)
``CapacityCache`` / ``FixedBranch`` / ``aux_fixed_update``   append-transform of new pool rows into a capacity buffer, with adoption of
                            the legacy ``state[name]`` / ``state[rows_key]`` keys, shrink recompute and the
                            fall-back-to-stock ``None`` results (:215-280)
``pooled_qat_update``       the call of model.py:911-918: ``name="pooled_qat"``, transform = the indexer QAT
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch


def decode_step_params(*, offset: int, pool_rows: int, device="cuda"):
    """int32 ``[position, valid rows]`` on ``device``: per-token scalars travel as data, so a captured graph reads
    them instead of baking them in."""
    return torch.tensor([int(offset), int(pool_rows)], dtype=torch.int32, device=device)


def pad_scores_to_capacity(scores, params):
    """``scores`` ``[..., capacity]``; ``params[1]`` = valid-row count (read on the device).  Columns at and past
    it become -inf; valid columns pass through bitwise."""
    capacity = int(scores.shape[-1])
    valid = torch.arange(capacity, dtype=torch.int32, device=scores.device) < params.reshape(-1)[1]
    return torch.where(valid.reshape((1,) * (scores.ndim - 1) + (capacity,)), scores,
                       torch.full((), float("-inf"), dtype=scores.dtype, device=scores.device))


class CapacityCache:
    """One derived cache held in a ``[B, capacity, D]`` buffer whose address never changes; ``rows`` of it are valid."""

    def __init__(self, capacity: int):
        self.capacity = int(capacity)
        self.buf = None
        self.rows = 0
        self.view = None     # buf[:, :rows]: the very object published under state[name]

    def _ensure(self, like, batch: int, width: int):
        if self.buf is None:
            self.buf = torch.zeros((batch, self.capacity, width), dtype=like.dtype, device=like.device)

    def holds(self, published, published_rows: int) -> bool:
        """Is what the caller's dict publishes still this cache's own last view?"""
        return self.view is not None and published is self.view and published_rows == self.rows

    def adopt(self, legacy, legacy_rows: int, pool_rows: int) -> bool:
        """Start over from a legacy (concatenated) cache; False when it is malformed or does not fit."""
        self.buf, self.rows, self.view = None, 0, None
        if legacy is None or legacy_rows <= 0:
            return True
        if legacy_rows > self.capacity or legacy_rows > pool_rows or int(legacy.shape[1]) != legacy_rows:
            return False
        self._ensure(legacy, int(legacy.shape[0]), int(legacy.shape[-1]))
        self.buf[:, :legacy_rows] = legacy
        self.rows = legacy_rows
        return True

    def extend(self, pooled, transform):
        """Bring the cache to ``pooled``'s row count by transforming only the rows it does not hold yet (all of
        them after a shrink).  Returns the rows held before, or None when the transform's dtype no longer matches."""
        rows = int(pooled.shape[1])
        if rows < self.rows:
            self.rows = 0
        prior = self.rows
        if rows > prior:
            fresh = transform(pooled[:, prior:, :])
            self._ensure(fresh, int(fresh.shape[0]), int(fresh.shape[-1]))
            if fresh.dtype != self.buf.dtype:
                return None
            self.buf[:, prior:rows] = fresh
            self.rows = rows
        self._ensure(pooled, int(pooled.shape[0]), int(pooled.shape[-1]))
        self.view = self.buf[:, :rows]
        return prior


@dataclass
class FixedBranch:
    """The fixed layout of one cache branch: the pool's row capacity and its derived caches by name."""
    pool_capacity: int
    aux: dict = field(default_factory=dict)


def aux_fixed_update(branch: FixedBranch, state: dict, *, name: str, rows_key: str, pooled, transform):
    """Append ``transform(new rows)`` of ``pooled`` ``[B, rows, D]`` (the valid-row view of the pool) into the
    capacity buffer ``name`` of ``branch`` and publish ``state[name]`` (the valid view) and ``state[rows_key]``.

    Returns ``(valid_view, prior_rows)``, or ``None`` when the fixed path cannot proceed (pool beyond capacity, a
    malformed legacy cache, a transform whose dtype changed) — the caller then takes the stock concat path, which
    trusts the legacy keys as they stand.  The dict is authoritative: if somebody replaced ``state[name]`` behind
    this cache's back, the replacement is adopted.  ``transform`` must act row by row (QAT, FP8 round trip)."""
    if int(pooled.shape[1]) > branch.pool_capacity:
        return None
    published, published_rows = state.get(name), int(state.get(rows_key, 0) or 0)
    cache = branch.aux.get(name)
    if cache is None or not cache.holds(published, published_rows):
        cache = CapacityCache(branch.pool_capacity)
        if not cache.adopt(published, published_rows, int(pooled.shape[1])):
            return None
        branch.aux[name] = cache
    prior = cache.extend(pooled, transform)
    if prior is None:
        branch.aux.pop(name, None)
        return None
    state[name] = cache.view
    state[rows_key] = cache.rows
    return cache.view, prior


def aux_capacity_buffer(branch: FixedBranch, name: str):
    """The full capacity buffer of a derived cache (stable address), or None before the first update."""
    cache = branch.aux.get(name)
    return None if cache is None else cache.buf


def pooled_qat_update(branch: FixedBranch, state: dict, pooled):
    """The indexer's derived cache: new pool rows go through the indexer QAT (Hadamard-128, FP4 lattice) and are
    appended behind the rows already held (model.py:911-918)."""
    from .indexer_score_kernel import indexer_qat_rows
    return aux_fixed_update(branch, state, name="pooled_qat", rows_key="pooled_qat_rows", pooled=pooled,
                            transform=indexer_qat_rows)
