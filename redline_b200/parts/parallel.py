"""Two mixers side by side: both read the same input, and the layer's mixer output is
left_scale * left(h) + right_scale * right(h).

Each side stops before its output projection and writes its (scaled) heads into its columns of one
buffer; ONE product with the two output weights laid side by side, [W_o,left | W_o,right], then gives the
sum.  A side is any mixer that has ``inner_size()``, ``forward_inner(x, ctx, cache, state, y, scale)`` and
``out_weight()``.  At most one side keeps a cache and at most one keeps a state; the pair hands the
engine that side's ``cache_spec`` / ``state_spec``.  Tensor names of the pair are the sides' own with
``left.`` / ``right.`` in front (``parallel_spec`` builds the ``PartSpec``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch

from ..ops.linear import linear
from .base import Mixer, build_part, op_mark, register
from .spec import PartSpec, TensorSpec

SIDES = ("left", "right")


@dataclass(frozen=True)
class ParallelMixersParams:
    hidden_size: int
    left: PartSpec
    right: PartSpec
    left_scale: float = 1.0
    right_scale: float = 1.0


def parallel_spec(hidden_size: int, left: PartSpec, right: PartSpec, left_scale: float = 1.0,
                  right_scale: float = 1.0) -> PartSpec:
    names = {f"{side}.{k}": v for side, part in zip(SIDES, (left, right)) for k, v in part.names.items()}
    return PartSpec("parallel_mixers", ParallelMixersParams(hidden_size, left, right, left_scale, right_scale), names)


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.params
        self.sides = [build_part("mixer", p.left, rt), build_part("mixer", p.right, rt)]
        self.scales = [p.left_scale, p.right_scale]
        for side, m in zip(SIDES, self.sides):
            if not all(hasattr(m, a) for a in ("inner_size", "forward_inner", "out_weight")):
                raise ValueError(f"the {side} mixer '{m.spec.kind}' cannot run beside another one: it has no "
                                 "forward_inner / inner_size / out_weight")
        if sum(m.cache_spec() is not None for m in self.sides) > 1 or sum(m.state_spec() is not None for m in self.sides) > 1:
            raise ValueError("of two mixers side by side at most one keeps a cache and at most one a state")
        self.widths = [m.inner_size() for m in self.sides]

    # -- what the engine asks of a mixer: answered by the side that has it
    def cache_spec(self):
        return next((m.cache_spec() for m in self.sides if m.cache_spec() is not None), None)

    def state_spec(self):
        return next((m.state_spec() for m in self.sides if m.state_spec() is not None), None)

    def state_in_graphs(self) -> bool:
        return all(m.state_in_graphs() for m in self.sides if m.state_spec() is not None)

    def tiling(self):
        named = {m.tiling() for m in self.sides} - {None}
        if len(named) > 1:
            raise ValueError(f"the two sides want the step's work lists cut in different ways: {sorted(named)}")
        return next(iter(named)) if named else None

    def decode_variant(self, ctx) -> int:
        return self.sides[0].decode_variant(ctx) * 1024 + self.sides[1].decode_variant(ctx)

    # -- tensors
    def tensors(self) -> Dict[str, TensorSpec]:
        return {f"{side}.{k}": v for side, m in zip(SIDES, self.sides) for k, v in m.tensors().items()}

    def fused(self) -> Dict[str, list]:
        return {f"{side}.{k}": [f"{side}.{n}" for n in members]
                for side, m in zip(SIDES, self.sides) for k, members in m.fused().items()}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for side, m in zip(SIDES, self.sides):
            m.load({k[len(side) + 1:]: v for k, v in tensors.items() if k.startswith(side + ".")})
        ws = [m.out_weight() for m in self.sides]
        dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_o = torch.cat([w.to(dt) for w in ws], dim=1).contiguous()

    def nbytes(self) -> int:
        return sum(m.nbytes() for m in self.sides) + self.w_o.numel() * self.w_o.element_size()

    def forward(self, x, ctx, cache, state) -> torch.Tensor:
        p, rt = self.params, self.rt
        T = ctx.T
        y = rt.workspace.get("parallel.y", (rt.max_tokens, sum(self.widths)), rt.dtype)[:T]
        col = 0
        for m, width, scale in zip(self.sides, self.widths, self.scales):
            m.forward_inner(x, ctx, cache if m.cache_spec() is not None else None,
                            state if m.state_spec() is not None else None, y[:, col:col + width], scale)
            col += width
        out = rt.workspace.get("mixer.out", (rt.max_tokens, p.hidden_size), rt.dtype)[:T]
        linear(y, self.w_o, out)
        op_mark(ctx, "o_proj", self.w_o, T)
        return out
