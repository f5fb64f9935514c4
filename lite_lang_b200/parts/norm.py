"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * w, computed in float32.

Formula: ``litelang/kernel/develop_rmsnorm/rms_norm.py:11-17,43-53``; used before
the mixer, before the feed-forward and before the lm_head
(``litelang/models/qwen2/layer/transformer_layer.py:86-92``, ``post_layer.py:43-45``).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .base import Norm, TensorDecl, register_part, whole_output


class RMSNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {"weight": TensorDecl((self.hidden_size,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch("weight").to(torch.float32).to(device).contiguous()

    def split_params(self):
        return self.weight, self.eps

    def forward(self, x, out=None):
        if out is None:
            out = torch.empty_like(x)
        ops.rmsnorm(out, x, self.weight, self.eps)
        return out

    def add_forward(self, residual, delta, rows=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, residual.shape[1]), dtype=residual.dtype, device=residual.device)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, rows)
        return out


class LayerNormF32Residual(Norm):
    """Layer norm with a weight and no bias, y = (x - mean) / sqrt(var + eps) * w, over a residual stream
    that is kept in float32 whatever the engine's dtype is; its output has the engine's dtype.

    ``add_forward`` takes the not yet added outputs of the parts before it as one tensor or as a tuple of
    up to two (a block whose mixer and feed-forward read the same norm hands on both): they are added to
    each other, then to the residual, in float32.  ``tensor`` is the weight's name under the prefix.
    """

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden_size = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.tensor = str(spec.params.get("tensor", "weight"))
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def tensors(self) -> Dict[str, TensorDecl]:
        return {self.tensor: TensorDecl((self.hidden_size,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        self.weight = fetch(self.tensor).to(torch.float32).to(device).contiguous()
        self.out_dtype = dtype

    def forward(self, x, out=None):
        return self.add_forward(x, None)

    def add_forward(self, residual, delta, rows=None):
        if residual.dtype != torch.float32:
            raise TypeError("layer_norm_f32: the residual stream of this norm is float32")
        deltas = [d for d in (delta if isinstance(delta, (tuple, list)) else (delta,)) if d is not None]
        if len(deltas) > 2:
            raise ValueError("layer_norm_f32: at most two pending outputs can be added in the norm")
        # one of them may come as float32 partial sums of a product split over its inner dimension
        partial = next((d for d in deltas if d.dim() == 3), None)
        deltas = [whole_output(d, self.out_dtype) for d in deltas if d is not partial] + [None, None]
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, residual.shape[1]), dtype=self.out_dtype, device=residual.device)
        ops.add_layernorm(out, residual, deltas[0], deltas[1], self.weight, self.eps, rows, partial)
        return out


register_part("norm", "rms_norm", RMSNorm)
register_part("norm", "layer_norm_f32", LayerNormF32Residual)
