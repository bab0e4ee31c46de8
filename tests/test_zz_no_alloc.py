"""The allocation-free top-k entry point (`mxb_topk_select_static`), through the C ABI.

Who needs it: hosts that may not allocate device memory when the call is made — a serving
process that froze its pool after start-up, or code inside another framework's allocator
callback.  The entry point keeps its scratch in an array built into the library, so this
test hands it nothing but inputs and an output buffer, calls it twice in a row (the second
call finds the first call's leftovers in the scratch) and compares both results with the
regular entry point, bit for bit.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.gpu_util import need_gpu

pytestmark = pytest.mark.gpu


def _call(lib, fn, scores, out, k, workspace=None):
    from moespresso_b200 import _abi
    a = _abi.TopkArgs()
    rows, n = scores.shape
    a.scores = scores.data_ptr(); a.row_stride = n; a.out_ids = out.data_ptr()
    a.rows, a.n, a.k = rows, n, k
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    rc = fn(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.mxb_last_error()
    return out


def test_static_scratch_topk_matches_regular_entry_point_twice():
    need_gpu()
    from moespresso_b200 import _abi
    lib = _abi.load()
    rng = np.random.default_rng(42)
    rows, n, k = 3, 150000, 2048
    # heavy ties: ~38 % of every row shares each rounded value, so the threshold bin holds far more
    # candidates than fit in shared memory and the kernel has to use its global scratch
    tied = torch.from_numpy(np.round(rng.standard_normal((rows, n))).astype(np.float32)).cuda()
    rand = torch.from_numpy(rng.standard_normal((rows, n)).astype(np.float32)).cuda()
    ws = torch.empty(int(lib.mxb_topk_workspace_bytes(rows, n, k)), dtype=torch.uint8, device="cuda")
    for scores in (tied, rand, tied):
        want = _call(lib, lib.mxb_topk_select, scores, torch.empty((rows, k), dtype=torch.int32, device="cuda"), k, ws)
        out = torch.full((rows, k), -7, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        got = _call(lib, lib.mxb_topk_select_static, scores, out, k)
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == before   # no torch allocation either
        assert torch.equal(got, want)
    # and against the CPU oracle for one row
    from oracle import ds4
    np.testing.assert_array_equal(got[0].cpu().numpy(), ds4.topk_ids(tied[0].cpu().numpy(), k)[0])


def test_static_scratch_rejects_oversize():
    need_gpu()
    from moespresso_b200 import _abi
    lib = _abi.load()
    a = _abi.TopkArgs()
    s = torch.zeros(8, device="cuda"); o = torch.zeros(8, dtype=torch.int32, device="cuda")
    a.scores, a.out_ids, a.rows, a.n, a.k, a.row_stride = s.data_ptr(), o.data_ptr(), 9, 131072, 8, 131072
    assert lib.mxb_topk_select_static(C.byref(a), None) == -1
    assert b"exceeds the built-in scratch" in lib.mxb_last_error()
