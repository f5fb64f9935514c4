"""Linear attention with a decay per head ("lightning attention"): a recurrent mixer with a matrix state.

q = silu(W_q x), k = silu(W_k x) (``heads`` x ``key_dim``) and v = silu(W_v x) (``heads`` x ``value_dim``);
per head, token by token,

    S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t        (nothing else multiplies the scores)

The heads' o side by side are RMS-normed as one vector with the weight ``norm``, multiplied by
sigmoid(W_g x) and projected by W_o.  A request's state is all zeros before its first token; it is float32 and
lives in the request's record of the cache manager's state pool, so a request goes on in a later step, alone or
beside others, from where it stopped.  Everything between the projections and the output projection is float32.
Tensors: ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``; ``decay`` is a parameter (one number a head).
"""

from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, StateNeed, TensorDecl, register_part


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class DecayLinearAttention(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.H = int(p["heads"])
        self.dk = int(p["key_dim"])
        self.dv = int(p["value_dim"])
        self.decay_values = [float(d) for d in p["decay"]]
        self.eps = float(p["eps"])
        if len(self.decay_values) != self.H:
            raise ValueError(f"decay_linear_attention: {len(self.decay_values)} decays for {self.H} heads")
        if not (0 < self.dk <= 256):
            raise ValueError("decay_linear_attention: key heads of 1 to 256 channels are built")
        self.Cq, self.Cv = self.H * self.dk, self.H * self.dv
        self.w_in = None

    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        return {"q": TensorDecl((self.Cq, h)), "k": TensorDecl((self.Cq, h)), "v": TensorDecl((self.Cv, h)),
                "g": TensorDecl((self.Cv, h)), "o": TensorDecl((h, self.Cv)), "norm": TensorDecl((self.Cv,), "norm")}

    def load(self, fetch, dtype, device) -> None:
        # one product for everything that reads the mixer's input; every segment starts at a multiple of 8 rows
        self.off, rows, at = {}, [], 0
        for name in ("q", "k", "v", "g"):
            w = fetch(name).to(dtype)
            self.off[name] = at
            rows.append(w)
            pad = _pad8(w.shape[0]) - w.shape[0]
            if pad:
                rows.append(torch.zeros((pad, self.hidden_size), dtype=dtype))
            at += _pad8(w.shape[0])
        self.w_in = torch.cat(rows, dim=0).to(device).contiguous()
        self.w_o = fetch("o").to(dtype).to(device).contiguous()
        self.norm_w = fetch("norm").to(torch.float32).to(device).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.norm_w))

    def cache_need(self):
        return StateNeed((self.H * self.dv * self.dk,), "float32")

    def kernel_libraries(self):
        libs = ["core", "linear_attn"]
        if self.w_in is not None and self.w_in.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
        return libs

    def forward(self, x, step, cache):
        n, dev = x.shape[0], x.device
        proj = ops.linear(x, self.w_in)
        ops.silu_rows(proj[:, :self.off["g"]])        # q | k | v (and the zero columns that pad them)
        o = torch.empty((n, self.Cv), dtype=torch.float32, device=dev)
        ops.decay_scan(proj, self.off["q"], self.off["k"], self.off["v"], self.decay, cache.state, step, o,
                       self.H, self.dk, self.dv, cache.writable)
        y = torch.empty((n, self.Cv), dtype=x.dtype, device=dev)
        ops.linear_attn_out(y, o, self.norm_w, proj[:, self.off["g"]:self.off["g"] + self.Cv], self.eps)
        return ops.linear(y, self.w_o, partial_ok=self.partial_ok)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
