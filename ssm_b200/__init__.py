"""ssm_b200: hand-written sm_100a CUDA kernels for the state-space operator hot path of
b-vitamins/ssm (selective scan, state step, chunked scan, depthwise causal conv, fused
add + LayerNorm/RMSNorm), behind a C ABI (``include/ssm_b200.h``) and the upstream operator
signatures (``ssm_b200.ops``).  ``ssm_b200.install()`` plugs the backend into an importable
upstream ``ssm.ops`` so that its CUDA dispatch uses these kernels."""

from __future__ import annotations

__all__ = ["ops", "backend", "install", "mixer", "seqpar"]


def __getattr__(name):
    import importlib

    if name in ("ops", "backend", "mixer", "seqpar"):
        return importlib.import_module(f"{__name__}.{name}")
    if name == "install":
        return importlib.import_module(f"{__name__}.backend").install
    raise AttributeError(name)
