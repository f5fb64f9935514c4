"""Routed feed-forward (mixture of experts), optionally with an expert that every token uses.

A router scores all ``experts`` in float32 (scores = ``score``(W_router x): "softmax" over all experts, or
"sigmoid"), the ``top`` largest are chosen, and the output is the sum of the chosen experts' outputs weighted
by their scores (divided by their sum first if ``renormalize``).  An expert is down(act(up x)) without biases,
act = ``activation`` ("relu2": the square of relu; "silu"; "gelu_tanh").  ``shared_ff`` > 0 adds an expert of
that width (tensors ``shared.up``, ``shared.down``) that runs for every token with weight 1.

Two ways through the experts, both without the host ever knowing who chose whom:

* few tokens (decode steps, short portions) and the float32 path: all experts' up matrices are stacked into one
  (the shared expert's rows first), so the first product is one product over all hidden units; the activation
  kernel multiplies each unit by its expert's weight for the token (an exact zero for experts that were not
  chosen), and one product with the stacked down matrices gives the weighted sum.  With few tokens a step reads
  every expert's weights anyway, and that is what bounds it.
* many tokens (``GROUPED_MIN_TOKENS``; bfloat16; widths that are multiples of 8): the (token, expert) pairs are
  put in the order of the experts on the device, the chosen tokens' rows gathered, and two grouped library
  products (a group an expert, the groups' ends a device array) do only the chosen experts' arithmetic; the
  pairs' results are added per token in the order of the pairs, onto the shared expert's output.

A token's result does not depend on which other tokens are in the step (beyond which of the two ways it takes).
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
        # views for the grouped way: the experts' up matrices [E, ff, hidden] inside the stacked one; their down
        # matrices [E, hidden, ff] as strided views of the stacked one's columns
        sff, ff, E, h = self.shared_ff, self.ff, self.E, self.hidden_size
        self.w_up_experts = self.w_up[sff:].view(E, ff, h)
        self.w_down_experts = self.w_down[:, sff:].unflatten(1, (E, ff)).permute(1, 0, 2)
        self.grouped = (dtype == torch.bfloat16 and h % 8 == 0 and ff % 8 == 0 and sff % 8 == 0
                        and ops.grouped_product_available())

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

    GROUPED_MIN_TOKENS = 128

    def forward(self, x, step):
        gates, idx, wts = self.route(x)
        if self.grouped and x.shape[0] >= self.GROUPED_MIN_TOKENS and not getattr(step, "captured", False):
            try:
                return self._forward_grouped(x, idx, wts)
            except (RuntimeError, NotImplementedError) as exc:      # a shape the library's grouped product refuses
                import sys
                print(f"[lite_lang_b200] routed_experts {self.prefix}: grouped product refused ({str(exc)[:120]}); "
                      "the stacked way is used instead", file=sys.stderr)
                self.grouped = False
        hidden = ops.linear(x, self.w_up)
        ops.moe_act(hidden, gates, self.shared_ff, self.ff, self.E, self.activation)
        # (few tokens and many hidden units: float32 partial sums of a split inner dimension, added up by the norm)
        return ops.linear(hidden, self.w_down, partial_ok=True)


    def _forward_grouped(self, x, idx, wts):
        sff = self.shared_ff
        base = None
        if sff:
            hs = ops.linear(x, self.w_up[:sff])
            ops.moe_act(hs, wts, sff, self.ff, 0, self.activation)      # (no routed columns: every weight is 1)
            base = ops.linear(hs, self.w_down[:, :sff])
        ends, row_token, row_w, pair_row = ops.moe_sort(idx, wts, self.E)
        rows = ops.moe_gather_rows(x, row_token)
        hidden = ops.grouped_product(rows, self.w_up_experts, ends)
        ops.moe_row_act(hidden, row_w, self.activation)
        y = ops.grouped_product(hidden, self.w_down_experts, ends)
        return ops.moe_combine(base, y, pair_row)


register_part("feed_forward", "routed_experts", RoutedExperts)
