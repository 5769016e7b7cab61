"""Drop-in object for the upstream package's compiled-CUDA-backend slot.

Upstream's façade (src/ssm/ops/__init__.py:85-109) caches its CUDA extension module in the
global ``ssm.ops._CUDA_OPS`` and calls ten functions on it whose names, argument order,
defaults and return tuples are fixed by src/ssm/ops/cuda/bindings.cpp:96-152.  Those ten
functions are provided by the C++ extension ``ssm_b200_ext`` (csrc/torch_ext/ssm_b200_ext.cpp:
ATen tensors in, the C ABI of include/ssm_b200.h underneath).  ``load_extension()`` imports
it, ``install()`` stores a :class:`Backend` around it in upstream's slot, so that
``ssm.ops.selective_scan`` etc. dispatch CUDA tensors to the sm_100a kernels with no change to
upstream code.  The extension reports contract violations as ``RuntimeError``, which upstream
translates to ``ValueError`` (src/ssm/ops/__init__.py:1244-1252).
"""

from __future__ import annotations

import importlib.util
from pathlib import Path

EXT_PATH = Path(__file__).resolve().parent / "lib" / "ssm_b200_ext.so"

NAMES = (
    "selective_scan", "selective_scan_backward", "selective_state_step", "selective_state_step_backward",
    "ssd_chunk_scan", "ssd_chunk_scan_backward", "dw_causal_conv", "dw_causal_conv_backward",
    "fused_layer_norm", "fused_layer_norm_backward",
)

_ext = None


def load_extension():
    """Import the compiled extension module (once).  Raises if it or the C-ABI library has not been built."""
    global _ext
    if _ext is not None:
        return _ext
    import torch  # noqa: F401  (the extension links against libtorch: it must be loaded first)

    from . import _lib

    _lib.load()  # loads libssm_b200.so and checks its ABI version; fails loudly if it is missing
    if not EXT_PATH.exists():
        raise RuntimeError(f"{EXT_PATH} is missing: run `python -m ssm_b200.build`; there is no fallback")
    spec = importlib.util.spec_from_file_location("ssm_b200_ext", EXT_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if mod.abi_version() != _lib.ABI_VERSION:
        raise RuntimeError("ssm_b200_ext was built against another version of the C ABI; rebuild it")
    _ext = mod
    return mod


class Backend:
    """The ten entry points of upstream's ``ssm_cuda_ops`` module, served by ``ssm_b200_ext``.

    Nine are the extension's functions as they are for fp32 / bf16 / fp16 tensors; float64 tensors (upstream's
    ``gradcheck`` matrix) go to the double-precision kernels through ``ops_f64.backend_*``.  ``selective_scan`` adapts the return arity to
    upstream's two call sites: its autograd wrapper unpacks ``(out, last_state, cache)``
    (src/ssm/ops/__init__.py:317), its inference path -- taken when no input requires a gradient
    -- unpacks ``(out, last_state)`` (src/ssm/ops/__init__.py:1304) and would fail on the
    3-tuple that bindings.cpp:11-16 declares.
    """

    def __init__(self) -> None:
        ext = load_extension()
        self.ext = ext
        for name in NAMES:
            if name != "selective_scan":
                setattr(self, name, self._route(name, getattr(ext, name)))

    @staticmethod
    def _is_f64(args) -> bool:
        """float64 calls (upstream's gradient checks) go to the double-precision kernels: ``ops_f64.backend_*``."""
        import torch

        for a in args[:3]:  # the activation tensor is the first argument, or follows one or two gradients
            if isinstance(a, torch.Tensor) and a.is_floating_point():
                return a.dtype == torch.float64
        return False

    def _route(self, name, fn):
        def call(*args, **kw):
            if self._is_f64(args):
                from . import ops_f64

                return getattr(ops_f64, "backend_" + name)(*args, **kw)
            return fn(*args, **kw)

        call.__name__ = name
        call.__doc__ = fn.__doc__
        return call

    def selective_scan(self, u, delta, A, B, C, D=None, z=None, dt_bias=None, softplus=False, return_last_state=False):
        if self._is_f64((u,)):
            from . import ops_f64

            out, last, cache = ops_f64.backend_selective_scan(u, delta, A, B, C, D, z, dt_bias, softplus, return_last_state)
        else:
            out, last, cache = self._scan(u, delta, A, B, C, D, z, dt_bias, softplus, return_last_state)
        if any(t is not None and t.requires_grad for t in (u, delta, A, B, C, D, z, dt_bias)):
            return out, last, cache
        return out, last

    def _scan(self, u, delta, A, B, C, D, z, dt_bias, softplus, return_last_state):
        return self.ext.selective_scan(u, delta, A, B, C, D, z, dt_bias, softplus, return_last_state)


def install(ssm_ops_module=None) -> Backend:
    """Put a :class:`Backend` into upstream's ``ssm.ops._CUDA_OPS`` slot (and clear a cached
    load failure).  Pass the module explicitly or let it be imported as ``ssm.ops``."""
    be = Backend()  # fails now, loudly, if the CUDA library or the extension is not built
    if ssm_ops_module is None:
        import importlib

        ssm_ops_module = importlib.import_module("ssm.ops")
    ssm_ops_module._CUDA_OPS = be
    ssm_ops_module._CUDA_LOAD_ERROR = None
    return be
