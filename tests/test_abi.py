"""CPU-side checks of the C-ABI boundary: the library loads, exports every function the
header declares, and the ctypes mirrors have the C structs' sizes.  No kernel is launched."""

from __future__ import annotations

import ctypes
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "ssm_b200.h"


def _declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(ssm_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from ssm_b200 import _lib

    lib = _lib.load()
    names = _declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.ENTRY_POINTS, f"{name} has no ctypes prototype"
    assert lib.ssm_b200_abi_version() == 3
    assert lib.ssm_scan_checkpoint_interval() == 32


def test_ctypes_structs_match_c_layout(tmp_path):
    from ssm_b200 import _lib

    pairs = {
        "ssm_scan_fwd_args": _lib.ScanFwdArgs, "ssm_scan_bwd_args": _lib.ScanBwdArgs,
        "ssm_step_args": _lib.StepArgs, "ssm_step_bwd_args": _lib.StepBwdArgs,
        "ssm_bcast4": _lib.Bcast4, "ssm_chunk_args": _lib.ChunkArgs, "ssm_chunk_bwd_args": _lib.ChunkBwdArgs,
        "ssm_conv_args": _lib.ConvArgs, "ssm_conv_bwd_args": _lib.ConvBwdArgs, "ssm_conv_update_args": _lib.ConvUpdateArgs,
        "ssm_norm_args": _lib.NormArgs, "ssm_norm_bwd_args": _lib.NormBwdArgs, "ssm_ssd_args": _lib.SsdArgs,
    }
    src = tmp_path / "sizes.c"
    body = "".join(f'  printf("{n} %zu\\n", sizeof({n}));\n' for n in pairs)
    src.write_text(f'#include <stdio.h>\n#include "{HEADER}"\nint main(void) {{\n{body}  return 0;\n}}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    for line in out.splitlines():
        name, size = line.split()
        assert ctypes.sizeof(pairs[name]) == int(size), name


def test_null_and_bad_arguments_are_rejected_without_a_gpu():
    from ssm_b200 import _lib

    lib = _lib.load()
    assert lib.ssm_selective_scan_fwd(None, None) == -1
    assert b"NULL" in lib.ssm_b200_last_error()
    a = _lib.ConvArgs()
    a.batch, a.channels, a.len, a.width = 1, 1, 1, 9
    assert lib.ssm_dw_causal_conv_fwd(ctypes.byref(a), None) == -5
    n = _lib.NormArgs()
    n.rows, n.hidden, n.io_dtype = 1, 8, 7
    assert lib.ssm_fused_add_norm_fwd(ctypes.byref(n), None) == -3
    assert lib.ssm_norm_bwd_scratch_floats(10, 768) == 2 * 768 * 592
    assert lib.ssm_chunk_scan_scratch_floats(2, 100, 3, 4, 32) == 2 * 2 * 4 * 12


def test_operators_refuse_cpu_tensors():
    import torch

    from ssm_b200 import ops

    x = torch.zeros(1, 2, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ops.dw_causal_conv(x, torch.zeros(2, 4))
    with pytest.raises(ValueError):
        ops.dw_causal_conv(torch.zeros(2, 8), torch.zeros(2, 4))


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    from ssm_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
