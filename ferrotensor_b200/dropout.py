"""Seeds for attention dropout (ferrotensor-graph/src/dropout.rs).

A dropout mask is a pure function of its seed, so nothing here keeps state: training derives one
seed per forward pass from the run seed, the rank, the optimizer step and the position in the
accumulation window (`Trainer::attention_dropout_seed`, ferrotensor-trainer/src/lib.rs:185-197),
and each attention layer derives its own from that.  A resumed run that restores its step counter
draws the same masks as an uninterrupted one.
"""

from __future__ import annotations

from typing import Sequence

_M = (1 << 64) - 1


def _mix(z: int) -> int:
    """SplitMix64's finaliser: a bijective mix of all 64 bits."""
    z = (z + 0x9E3779B97F4A7C15) & _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def derive_seed(parts: Sequence[int]) -> int:
    """A well-mixed seed from an ordered list of integers; equal lists give equal seeds and a
    change of any element (or of the length) changes the result."""
    acc = _mix(len(parts))
    for p in parts:
        acc = _mix(acc ^ _mix(int(p) & _M))
    return acc


def layer_seed(step_seed: int, layer: int) -> int:
    """The seed of attention layer `layer` for the forward pass whose seed is `step_seed`."""
    return derive_seed([step_seed, layer])


def attention_dropout_seed(run_seed: int, rank: int, optimizer_step: int, step_in_accum: int) -> int:
    return derive_seed([run_seed, rank, optimizer_step, step_in_accum])
