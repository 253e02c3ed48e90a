"""What every part is: declared parameters, bound tensors, and a registry from specification
class to part class.

A part is built from its specification and a ``Runtime`` (device and compute dtype). It declares
the tensors it wants with ``param_decls`` (names relative to its own prefix in the checkpoint),
receives them through ``bind`` and may fuse or re-lay them there. It never sees the model it is
in: sizes and constants come from the specification only.

Interfaces (duck-typed; see the classes in this package for the working examples):

* norm:            ``add_forward(h, delta, out, rows=None)`` with ``h`` the float32 residual
                   stream, updated in place by ``delta`` (None: nothing to add) unless ``rows``
                   selects rows, which are then normalised into ``out`` without touching ``h``.
                   ``takes_partial = True`` if ``delta`` may be a ``csrc.api.Partial``.
* position:        ``fused_tables = True`` and ``tables(n)``, or ``apply(qkv, ctx, nh, nkv, hd)``;
                   used by the mixer that owns it.
* mixer:           ``cache_requests()`` -> list of ``cache.KVRequest`` / ``cache.StateRequest``;
                   ``forward(ctx, views, a, writes)`` -> [tokens, hidden] in the compute dtype.
                   ``views`` are the cache views answering the requests, ``ctx`` the step's
                   ``engine.StepContext`` (token rows, their sequences and positions, page tables).
* feed-forward:    ``forward(ctx, a)`` -> [tokens, hidden].

Every part may also give ``step_weights()`` (the tensors a step reads once whatever the batch: the
bytes a decode step must stream), ``step_plans()`` (``StepPlan`` objects: index arrays its kernels
need each step, built on the host from the step's sequences and uploaded with the step context)
and ``prepare(max_positions)``; the defaults are empty.
"""
from dataclasses import dataclass
from typing import Tuple

import numpy as np
import torch


@dataclass(frozen=True)
class Runtime:
    device: torch.device
    dtype: torch.dtype          # compute dtype: torch.float32 or torch.bfloat16


@dataclass(frozen=True)
class ParamDecl:
    name: str                   # relative to the part's prefix, e.g. "q_proj.weight"
    shape: Tuple[int, ...]
    init: str = "matrix"        # random-weights mode: "matrix" N(0, 0.02), "norm" 1 + N(0, 0.1)
    keep_float32: bool = False  # small vectors (norm weights) are held in float32 for every dtype


class StepPlan:
    """Index data a part's kernels want for every step, e.g. a list of work tiles. ``key`` names
    it (equal keys are built once a step, whoever asks); ``build(seqs)`` gets the step's sequences
    as numpy arrays ``lens`` (new tokens each), ``pos0`` (tokens cached before) and ``is_decode``,
    and returns an int32 array, which reaches the kernels as ``ctx.plans[key]`` on the device."""
    key = None

    def build(self, lens, pos0, is_decode):
        return np.zeros((0,), np.int32)


class Part:
    def __init__(self, spec, rt):
        self.spec = spec
        self.rt = rt

    def param_decls(self):
        return []

    def bind(self, tensors):
        """``tensors``: name (as declared) -> tensor on the device, already cast."""

    def step_weights(self):
        return []

    def step_plans(self):
        return []

    def prepare(self, max_positions):
        """Called before steps that reach positions up to ``max_positions`` (tables that grow)."""


_PART_CLASSES = {}


def register_part(spec_cls, part_cls):
    """Makes ``build_part`` construct ``part_cls(spec, rt)`` for specifications of ``spec_cls``."""
    _PART_CLASSES[spec_cls] = part_cls


def build_part(spec, rt):
    try:
        cls = _PART_CLASSES[type(spec)]
    except KeyError:
        raise TypeError(f"no part registered for specification {type(spec).__name__}; "
                        f"call parts.register_part({type(spec).__name__}, YourPart)") from None
    return cls(spec, rt)
