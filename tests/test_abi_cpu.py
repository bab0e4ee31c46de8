"""CPU-side checks of the boundary: the shared library builds, loads, exports every
symbol the header declares, and the ctypes structures match the C layout."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "moespresso_b200.h")


def test_library_loads_and_exports_every_declared_symbol():
    from moespresso_b200 import _abi
    lib = _abi.load()
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(mxb_[a-z_0-9]+)\s*\(", text))
    assert declared, "no declarations found in the header"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_abi.EXPORTS), "the ctypes binding and the header disagree"
    assert lib.mxb_abi_version() == 1


def test_struct_layouts_match_c(tmp_path):
    from moespresso_b200 import _abi
    pairs = [("mxb_indexer_scores_args", _abi.IndexerScoresArgs), ("mxb_topk_args", _abi.TopkArgs),
             ("mxb_sparse_attn_args", _abi.SparseAttnArgs), ("mxb_merge_args", _abi.MergeArgs),
             ("mxb_flash_prefill_args", _abi.FlashPrefillArgs)]
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', 'int main(void){']
    for cname, cls in pairs:
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines.append('return 0;}')
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", str(src), "-o", str(exe)], check=True)
    got = dict(l.split() for l in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, cls in pairs:
        assert int(got[cname]) == C.sizeof(cls)
        for fname, _ in cls._fields_:
            assert int(got[f"{cname}.{fname}"]) == getattr(cls, fname).offset, f"{cname}.{fname}"


def test_host_side_validation_needs_no_gpu():
    """Contract violations are reported by the C entry points before any CUDA call."""
    from moespresso_b200 import _abi
    lib = _abi.load()
    a = _abi.TopkArgs()
    a.rows, a.n, a.k = 1, 10, 0
    assert lib.mxb_topk_select(C.byref(a), None) == -1
    assert b"between 1 and 8192" in lib.mxb_last_error()
    s = _abi.IndexerScoresArgs()
    s.B, s.T, s.H, s.D, s.n_rows = 1, 1, 16, 48, 10
    assert lib.mxb_indexer_scores(C.byref(s), None) == -1
    assert b"head_dim" in lib.mxb_last_error()
    f = _abi.FlashPrefillArgs()
    f.D, f.dtype = 128, 2
    assert lib.mxb_flash_prefill(C.byref(f), None) == -1
    assert b"head_dim=256" in lib.mxb_last_error()
    assert lib.mxb_topk_workspace_bytes(2, 131072, 2048) == 0            # one cluster per row, keys in shared memory
    assert lib.mxb_topk_workspace_bytes(2, 1 << 20, 2048) >= 2 * (1 << 20) * 8
    assert lib.mxb_topk_workspace_bytes(4096, 32768, 2048) == 0


def test_operators_refuse_cpu_tensors():
    import torch
    from moespresso_b200.deepseek_v4 import indexed_attention_kernel as iak
    from moespresso_b200.deepseek_v4.attention import topk_select
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        topk_select(torch.zeros(2, 8), 2)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        iak.indexer_scores_tiled_live(torch.zeros(1, 16, 1, 64), torch.zeros(1, 1, 16), torch.zeros(1, 4, 64), pos0=0)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "moespresso_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text.replace("oracle_free", ""), f"{f} mentions the oracle package"


def test_synth_rounding_helpers():
    import torch
    from moespresso_b200 import synth
    x = np.random.default_rng(0).standard_normal(5000).astype(np.float32) * 3
    np.testing.assert_array_equal(synth.to_bf16_f32(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())
    bits = synth.to_e4m3_bits(x)
    np.testing.assert_array_equal(bits, torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    np.testing.assert_array_equal(synth.e4m3_bits_to_f32(bits),
                                  torch.from_numpy(bits).view(torch.float8_e4m3fn).float().numpy())
    c = synth.config3(seed=1, lens=[10, 20])
    assert c["kv"].shape == (30, 576) and c["kv"].dtype == np.int8 and c["kv_scales"].dtype == np.float16
    assert float(c["kv_scales"].min()) >= 9e-4 and float(c["kv_scales"].max()) <= 1.01e-1
