"""Loader for the golden fixture packs in ``tests/golden`` (see make_fixtures.py there)."""

from __future__ import annotations

import json
from functools import lru_cache
from pathlib import Path
from typing import Any

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


class Case:
    """One fixture case: ``ins``/``outs``/``grads`` are dicts of CPU tensors in their
    recorded dtypes, ``opts`` the per-case scalars."""

    def __init__(self, name: str, ins, outs, grads, opts):
        self.name, self.ins, self.outs, self.grads, self.opts = name, ins, outs, grads, opts

    def __repr__(self) -> str:  # shows up in pytest ids
        return self.name


@lru_cache(maxsize=None)
def _load(pack: str) -> dict[str, Case]:
    with np.load(GOLDEN / f"{pack}.npz", allow_pickle=False) as npz:
        meta: dict[str, dict[str, Any]] = json.loads(str(npz["__meta__"]))
        cases: dict[str, Case] = {}
        for case, opts in meta.items():
            cases[case] = Case(case, {}, {}, {}, {k: v for k, v in opts.items() if k != "dtypes"})
        for key in npz.files:
            if key == "__meta__":
                continue
            case, kind, name = key.rsplit("/", 2)
            arr = npz[key]
            dts = meta[case].get("dtypes", {}).get(f"{kind}/{name}")
            t = torch.from_numpy(np.array(arr))
            if dts is not None:
                t = t.to(getattr(torch, dts))
            {"in": cases[case].ins, "out": cases[case].outs, "grad": cases[case].grads}[kind][name] = t
    return cases


def cases(pack: str, family: str) -> list[Case]:
    """All cases of ``family`` (``scan``, ``step``, ``chunk``, ``conv``, ``norm``, ``ssd``)."""
    return [c for n, c in sorted(_load(pack).items()) if n.startswith(family + "/")]


def tol(case: Case, grad: bool = False) -> dict[str, float]:
    """Comparison bar for a case.  fp32: rtol 1e-4 / atol 1e-5.  Half-precision I/O:
    rtol 2e-2 (atol 2e-2) against values computed from the same rounded inputs."""
    o = case.opts
    if grad and "grad_rtol" in o:
        return dict(rtol=o["grad_rtol"], atol=o["grad_atol"])
    if "rtol" in o:
        return dict(rtol=o["rtol"], atol=o["atol"])
    if o.get("half"):
        return dict(rtol=2e-2, atol=2e-2)
    return dict(rtol=1e-4, atol=1e-5)
