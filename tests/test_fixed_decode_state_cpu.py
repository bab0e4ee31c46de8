"""Host logic of the fixed-capacity derived caches (CPU tensors, a row-wise stand-in transform).  Mirrors the
properties the reference tests for this layer (tests/test_deepseek_v4_fixed_decode_state.py): parity with the
concat path while decoding, fail-closed on capacity, adoption of a replaced legacy cache, shrink recompute."""
import torch

from moespresso_b200.deepseek_v4 import fixed_decode_state as fds


def _transform(rows):
    return torch.round(rows * 4.0) / 4.0 + 1.0      # acts row by row, like the QAT and the FP8 round trip


def test_append_matches_the_concat_path_and_transforms_only_new_rows():
    torch.manual_seed(0)
    pool = torch.randn(1, 40, 8)
    branch, state, calls = fds.FixedBranch(pool_capacity=64), {}, []

    def tr(rows):
        calls.append(int(rows.shape[1]))
        return _transform(rows)

    buf_addr = None
    for rows in (1, 2, 2, 5, 17, 40):
        view, prior = fds.aux_fixed_update(branch, state, name="pooled_qat", rows_key="pooled_qat_rows",
                                           pooled=pool[:, :rows], transform=tr)
        assert torch.equal(view, _transform(pool[:, :rows])) and tuple(view.shape) == (1, rows, 8)
        assert state["pooled_qat"] is view and state["pooled_qat_rows"] == rows
        cap = fds.aux_capacity_buffer(branch, "pooled_qat")
        assert tuple(cap.shape) == (1, 64, 8) and torch.all(cap[:, rows:] == 0)
        buf_addr = buf_addr or cap.data_ptr()
        assert cap.data_ptr() == buf_addr                      # appended in place: the address never changes
    assert calls == [1, 1, 3, 12, 23]                          # (the repeated row count transformed nothing)
    assert prior == 17


def test_capacity_exhaustion_fails_closed():
    branch, state = fds.FixedBranch(pool_capacity=4), {}
    pool = torch.ones(1, 6, 8)
    assert fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool[:, :4], transform=_transform)
    before = dict(state)
    assert fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool, transform=_transform) is None
    assert state == before                                     # the legacy keys are left as they stand


def test_replaced_legacy_cache_is_adopted_and_malformed_one_refused():
    pool = torch.randn(1, 10, 8)
    branch, state = fds.FixedBranch(pool_capacity=16), {}
    fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool[:, :3], transform=_transform)
    # somebody replaces the published cache (e.g. the stock concat path ran for a while)
    legacy = _transform(pool[:, :6]) + 100.0
    state["a"], state["a_rows"] = legacy, 6
    view, prior = fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool[:, :8], transform=_transform)
    assert prior == 6 and torch.equal(view[:, :6], legacy) and torch.equal(view[:, 6:], _transform(pool[:, 6:8]))
    # a legacy cache whose width disagrees with its row count stays on the stock path
    state["a"], state["a_rows"] = legacy, 5
    assert fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool[:, :8], transform=_transform) is None
    # and one that holds more rows than the pool
    state["a"], state["a_rows"] = legacy, 6
    assert fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool[:, :4], transform=_transform) is None


def test_shrunk_pool_is_recomputed_and_dtype_change_falls_back():
    pool = torch.randn(1, 10, 8)
    branch, state = fds.FixedBranch(pool_capacity=16), {}
    fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=pool[:, :9], transform=_transform)
    other = torch.randn(1, 10, 8)
    view, prior = fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=other[:, :4], transform=_transform)
    assert prior == 0 and torch.equal(view, _transform(other[:, :4]))
    assert fds.aux_fixed_update(branch, state, name="a", rows_key="a_rows", pooled=other[:, :6],
                                transform=lambda r: _transform(r).half()) is None
    assert "a" not in branch.aux


def test_padded_scores_keep_the_valid_prefix_bitwise():
    torch.manual_seed(1)
    scores = torch.randn(1, 1, 1024)
    params = fds.decode_step_params(offset=3844, pool_rows=961, device="cpu")
    assert params.dtype == torch.int32 and params.tolist() == [3844, 961]
    padded = fds.pad_scores_to_capacity(scores, params)
    assert torch.equal(padded[..., :961], scores[..., :961]) and torch.all(torch.isneginf(padded[..., 961:]))
    k = 512
    assert torch.equal(torch.topk(padded, k).indices, torch.topk(scores[..., :961], k).indices)
