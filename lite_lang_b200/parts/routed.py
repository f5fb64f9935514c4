"""Routed feed-forward (mixture of experts), optionally with an expert that every token uses.

A router scores all ``experts`` in float32 (scores = ``score``(W_router x): "softmax" over all experts, or
"sigmoid"), the ``top`` largest are chosen, and the output is the sum of the chosen experts' outputs weighted
by their scores (divided by their sum first if ``renormalize``).  An expert is down(act(up x)) without biases,
act = ``activation`` ("relu2": the square of relu; "silu"; "gelu_tanh").  ``shared_ff`` > 0 adds an expert of
that width (tensors ``shared.up``, ``shared.down``) that runs for every token with weight 1.

All experts' up matrices are stacked into one (the shared expert's rows first), so the first product is one
product over all hidden units; the activation kernel multiplies each unit by its expert's weight for the
token (an exact zero for experts that were not chosen), and one product with the stacked down matrices gives
the weighted sum.  A token's result does not depend on which other tokens are in the step.
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_part


class RoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.E = int(p["experts"])
        self.top = int(p["top"])
        self.ff = int(p["expert_ff"])
        self.shared_ff = int(p.get("shared_ff") or 0)
        self.activation = str(p.get("activation", "relu2"))
        self.score = str(p.get("score", "softmax"))
        self.renormalize = bool(p.get("renormalize", False))
        if self.activation not in ops.MOE_ACT or self.score not in ops.MOE_SCORE:
            raise ValueError(f"routed_experts: activation {self.activation!r} / score {self.score!r} is not built")
        if not (0 < self.top <= self.E <= 256):
            raise ValueError("routed_experts: 0 < top <= experts <= 256")
        self.w_up = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        d = {"router": TensorDecl((self.E, h), std=0.3)}
        for e in range(self.E):
            d[f"e{e}.up"] = TensorDecl((self.ff, h))
            d[f"e{e}.down"] = TensorDecl((h, self.ff))
        if self.shared_ff:
            d["shared.up"] = TensorDecl((self.shared_ff, h))
            d["shared.down"] = TensorDecl((h, self.shared_ff))
        return d

    def load(self, fetch, dtype, device) -> None:
        ups = ([fetch("shared.up")] if self.shared_ff else []) + [fetch(f"e{e}.up") for e in range(self.E)]
        downs = ([fetch("shared.down")] if self.shared_ff else []) + [fetch(f"e{e}.down") for e in range(self.E)]
        self.w_up = torch.cat([u.to(dtype) for u in ups], dim=0).to(device).contiguous()
        self.w_down = torch.cat([w.to(dtype) for w in downs], dim=1).to(device).contiguous()
        self.w_router = fetch("router").to(torch.float32).to(device).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_up, self.w_down, self.w_router))

    def kernel_libraries(self):
        libs = ["core", "moe"]
        if self.w_up is not None and self.w_up.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
        return libs

    def route(self, x):
        n, dev = x.shape[0], x.device
        gates = torch.empty((n, self.E), dtype=torch.float32, device=dev)
        top_idx = torch.empty((n, self.top), dtype=torch.int32, device=dev)
        top_w = torch.empty((n, self.top), dtype=torch.float32, device=dev)
        ops.moe_router(x, self.w_router, gates, top_idx, top_w, self.top, self.score, self.renormalize)
        return gates, top_idx, top_w

    def forward(self, x, step):
        gates, _idx, _w = self.route(x)
        hidden = ops.linear(x, self.w_up)
        ops.moe_act(hidden, gates, self.shared_ff, self.ff, self.E, self.activation)
        # (few tokens and many hidden units: float32 partial sums of a split inner dimension, added up by the norm)
        return ops.linear(hidden, self.w_down, partial_ok=True)


register_part("feed_forward", "routed_experts", RoutedExperts)
