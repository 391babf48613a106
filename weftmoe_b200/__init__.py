"""weftmoe_b200 — B200 (sm_100a) routed-MoE expert operator behind the WeftMoE Tensor API.

Public names follow the reference package (`weftmoe/runtime.py`): `TensorRuntime`, `moe`, `Tape`.
"""
from .runtime import SingleRankGroup, Tape, TensorRuntime, moe

__all__ = ["TensorRuntime", "moe", "Tape", "SingleRankGroup"]
