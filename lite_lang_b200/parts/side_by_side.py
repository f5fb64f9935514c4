"""Two mixers side by side: both read the same input, and their outputs are joined.

``left`` and ``right`` are ordinary mixer parts (each given as {"kind": ..., "params": ...}; their tensors live
under ``left.`` and ``right.`` of this part's prefix, and each owns its memory in the cache manager: pages for
one, a state record for the other, whatever they ask for).  The join is

    out = (rms(left(x)) * w_left + rms(right(x)) * w_right) / 2

with RMS norms over the model width (x / sqrt(mean(x^2) + eps), plain weights ``left.out`` and ``right.out``).
A bias on the left mixer's output projection is added inside the join's pass instead of in one of its own.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, TensorDecl, build_part, register_part, whole_output

_SIDES = ("left", "right")


class SideBySide(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.eps = float(p["eps"])
        self.sides: Dict[str, Mixer] = {}
        for side in _SIDES:
            sub = p[side]
            m = build_part("mixer", PartSpec(str(sub["kind"]), dict(sub["params"]), self.prefix + side + "."))
            m.partial_ok = False
            self.sides[side] = m
        self.left, self.right = self.sides["left"], self.sides["right"]
        if hasattr(self.left, "defer_out_bias"):
            self.left.defer_out_bias = True     # added in the join
        self.w_left = self.w_right = None

    def sub_mixers(self) -> List[Tuple[str, Mixer]]:
        return [(side, self.sides[side]) for side in _SIDES]

    def tensors(self) -> Dict[str, TensorDecl]:
        d: Dict[str, TensorDecl] = {}
        for side in _SIDES:
            for rel, decl in self.sides[side].tensors().items():
                d[f"{side}.{rel}"] = decl
            d[f"{side}.out"] = TensorDecl((self.hidden_size,), "norm")
        return d

    def load(self, fetch, dtype, device) -> None:
        for side in _SIDES:
            self.sides[side].load(lambda rel, _s=side: fetch(f"{_s}.{rel}"), dtype, device)
        self.w_left = fetch("left.out").to(torch.float32).to(device).contiguous()
        self.w_right = fetch("right.out").to(torch.float32).to(device).contiguous()

    def prepare(self, device, dtype) -> None:
        for side in _SIDES:
            self.sides[side].prepare(device, dtype)

    def kernel_libraries(self):
        libs = ["core"]
        for side in _SIDES:
            for name in self.sides[side].kernel_libraries():
                if name not in libs:
                    libs.append(name)
        return libs

    def weight_bytes(self) -> int:
        return sum(self.sides[s].weight_bytes() for s in _SIDES) + 8 * self.hidden_size

    def forward(self, x, step, cache):
        a = whole_output(self.left.forward(x, step, cache["left"]), x.dtype)
        b = whole_output(self.right.forward(x, step, cache["right"]), x.dtype)
        out = torch.empty((x.shape[0], self.hidden_size), dtype=x.dtype, device=x.device)
        ops.rms_pair_mean(out, a, getattr(self.left, "deferred_out_bias", None), self.w_left, b, self.w_right, self.eps)
        return out


register_part("mixer", "side_by_side", SideBySide)
