"""Rotary position encoding with half-split pairs (i, i + half).

angle = pos / theta^(2i/rotary_dim); src/model/math.rs:52-99.  ``prepare``
fills one cos/sin table per step; every mixer that shares the same
specification reuses it.
"""
from __future__ import annotations

import torch

from ..config.spec import PositionSpec
from ..kernels import ops
from .base import ROTATION, Part, Rotation, register_position_encoding


@register_position_encoding("rotary_half")
class RotaryHalf(Part):
    applies = ROTATION

    def __init__(self, spec: PositionSpec, mctx):
        self.spec = spec
        self.half = spec.rotary_dim // 2
        self.key = ("rotary_half", spec.theta, spec.rotary_dim)

    def rotation(self, ctx) -> Rotation:
        """The rotation of this step's tokens: cos / sin float32 [T, rotary_dim/2], half-split pairs."""
        got = ctx.tables.get(self.key)
        if got is None:
            cos = ctx.workspace.get(f"rope.cos.{self.spec.theta}", ctx.T, self.half, torch.float32)
            sin = ctx.workspace.get(f"rope.sin.{self.spec.theta}", ctx.T, self.half, torch.float32)
            ops.rope_table(ctx.positions, cos, sin, self.spec.theta, self.spec.rotary_dim)
            got = ctx.tables[self.key] = Rotation(cos, sin, self.half, interleaved=False)
        return got
