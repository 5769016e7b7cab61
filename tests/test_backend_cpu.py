"""The C++ torch extension and the ``install()`` hook, as far as they go without a GPU: the module
imports, exports the ten names of upstream's compiled backend with their keyword arguments, rejects
CPU tensors and malformed shapes with ``RuntimeError`` (which upstream's facade turns into
``ValueError``), and ``install()`` fills upstream's backend slot."""

from __future__ import annotations

import sys
import types
from pathlib import Path

import pytest
import torch

# a checkout of upstream next to this repository (present where the fixtures are built; the test is skipped elsewhere)
REFERENCE_SRC = Path(__file__).resolve().parents[2] / "reference" / "src"


def test_extension_exports_the_ten_upstream_names_with_their_keywords():
    from ssm_b200 import backend

    ext = backend.load_extension()
    assert ext.abi_version() == 3
    for name in backend.NAMES:
        assert callable(getattr(ext, name)), name
    # keyword names and defaults of src/ssm/ops/cuda/bindings.cpp:96-152, as pybind records them
    doc = ext.selective_scan.__doc__
    for kw in ("u:", "delta:", "A:", "B:", "C:", "D:", "z:", "dt_bias:", "softplus: bool = False", "return_last_state: bool = False"):
        assert kw in doc, kw
    assert "softplus: bool = True" in ext.selective_state_step.__doc__
    for kw in ("chunk_size:", "seq_lens:", "cu_seqlens:", "initial_states:"):
        assert kw in ext.ssd_chunk_scan.__doc__, kw
    assert "activation: str = 'silu'" in ext.dw_causal_conv.__doc__
    for kw in ("is_rms: bool = False", "= 1e-05", "prenorm: bool = True", "residual_in_fp32: bool = True"):
        assert kw in ext.fused_layer_norm.__doc__, kw
    assert "grad_last_state:" in ext.selective_scan_backward.__doc__ and "cache:" in ext.selective_scan_backward.__doc__


def test_extension_rejects_cpu_tensors_and_bad_shapes_before_any_launch():
    from ssm_b200 import backend

    ext = backend.load_extension()
    x = torch.zeros(1, 2, 8)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        ext.dw_causal_conv(x, torch.zeros(2, 4))
    with pytest.raises(RuntimeError, match="delta must match"):
        ext.selective_scan(torch.zeros(2, 8, 16), torch.zeros(2, 8, 17), torch.zeros(8, 4), torch.zeros(8, 4), torch.zeros(8, 4))
    with pytest.raises(RuntimeError, match="x and dt must match"):
        ext.selective_state_step(torch.zeros(2, 8, 4), torch.zeros(2, 9), torch.zeros(2, 8), torch.zeros(8, 4), torch.zeros(8, 4), torch.zeros(8, 4))
    with pytest.raises(RuntimeError, match="dt must align"):
        ext.ssd_chunk_scan(torch.zeros(2, 64, 4, 8), torch.zeros(2, 65, 4), torch.zeros(4), torch.zeros(4, 8), torch.zeros(4, 8), 32)
    with pytest.raises(RuntimeError, match="Unsupported activation"):
        ext.dw_causal_conv(x, torch.zeros(2, 4), None, "relu")
    with pytest.raises(RuntimeError, match="weight must match"):
        ext.fused_layer_norm(torch.zeros(1, 2, 8), torch.zeros(7))


def test_install_fills_the_backend_slot_of_a_facade_module():
    import ssm_b200

    fake = types.ModuleType("ssm.ops")
    fake._CUDA_OPS = None
    fake._CUDA_LOAD_ERROR = RuntimeError("CUDA is not available")
    be = ssm_b200.install(fake)
    assert fake._CUDA_OPS is be and fake._CUDA_LOAD_ERROR is None
    from ssm_b200 import backend

    for name in backend.NAMES:
        assert callable(getattr(be, name)), name


@pytest.mark.skipif(not REFERENCE_SRC.exists(), reason="the upstream package is only present in the build container")
def test_install_into_the_real_upstream_facade(monkeypatch):
    import ssm_b200

    monkeypatch.syspath_prepend(str(REFERENCE_SRC))
    for mod in [m for m in sys.modules if m == "ssm" or m.startswith("ssm.")]:
        monkeypatch.delitem(sys.modules, mod)
    import ssm.ops as upstream

    be = ssm_b200.install()
    assert upstream._load_cuda_ops() is be
    assert upstream._cuda_backend_status().available
    assert upstream._should_use_cuda(torch.zeros(1)) is False  # CPU tensors keep taking upstream's own CPU / Python path
    for mod in [m for m in sys.modules if m == "ssm" or m.startswith("ssm.")]:
        monkeypatch.delitem(sys.modules, mod)
