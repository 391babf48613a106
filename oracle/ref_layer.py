"""TEST INFRASTRUCTURE ONLY — access to the reference's own torch layer, `verify_step`
(benchmarks/training_reference.py:15-79), when `make -C oracle ref` byte-compiled it into
oracle/_ref/training_reference.bytecode.  Nothing of it is copied or restated here.

Only tests/ and bench.py's CPU legs (`--impl reference`, `cpu_baseline`) may import this module.
`verify_step(runtime, x, routes, gates, w1, w2, dy)` runs the layer expert by expert on the host
(forward, autograd backward), and compares the five results with what `runtime` returned; it needs an
initialised torch.distributed group (gloo, world 1 here)."""
from __future__ import annotations

import importlib.machinery
import importlib.util
from pathlib import Path

COMPILED = Path(__file__).resolve().parent / "_ref" / "training_reference.bytecode"


def load_verify_step():
    """The reference's verify_step, or None when oracle/_ref was not built in this checkout."""
    if not COMPILED.is_file():
        return None
    loader = importlib.machinery.SourcelessFileLoader("weftmoe_ref_training_reference", str(COMPILED))
    spec = importlib.util.spec_from_loader(loader.name, loader)
    module = importlib.util.module_from_spec(spec)
    try:
        loader.exec_module(module)
    except Exception:   # a .pyc of another interpreter version: treat as absent
        return None
    return module.verify_step


class PrecomputedRuntime:
    """The `runtime` argument of verify_step: hands back tensors computed beforehand, so that a timing
    of verify_step covers the reference's own code only."""

    class _Tape:
        def __init__(self, output):
            self.output = output

    def __init__(self, y, dx, dgates, dw1, dw2):
        self._tape = self._Tape(y)
        self._grads = (dx, dgates, dw1, dw2)

    def forward(self, *args):
        return self._tape

    def backward(self, tape, dy):
        return self._grads


def ensure_single_rank_group():
    """A gloo group of one rank over an in-process store (verify_step calls all_gather / all_reduce).
    Returns True when this call created the group (the caller destroys it)."""
    import torch.distributed as dist
    if dist.is_initialized():
        return False
    dist.init_process_group("gloo", store=dist.HashStore(), rank=0, world_size=1)
    return True
