"""Gated delta rule mixer: a linear recurrence with a matrix state per head.

q, k (``kv_heads`` x ``key_dim``) and v (``heads`` x ``value_dim``) are projections of the input, each
passed through a short causal depthwise convolution over time (``conv_taps`` taps, the last one the current
token's, no bias) and SiLU.  q and k become unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times
key_dim^-1/2; query head h uses q/k head h // (heads / kv_heads).  With beta = sigmoid(B x) and a decay g,
a head's state S [key_dim, value_dim] goes, token by token,

    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

and o / rms(o) * weight * gate is projected back.  What differs between variants is a parameter:

``decay``       "head": g = exp(-exp(A_log_h) softplus(a_h + dt_bias_h)), one per head;
                "channel": the same per head and key channel (a, dt_bias laid out heads x key_dim).
``decay_rank``  0: a = W_a x (tensor ``a``); otherwise a = W_a2 (W_a1 x) through ``decay_rank`` numbers
                (tensors ``a1``, ``a2``); None: low-rank with the width read from the checkpoint.
``gate``        "silu" or "sigmoid": the activation of the output gate.
``gate_rank``   as ``decay_rank`` for the gate (tensors ``g`` or ``g1``, ``g2``).

The state (float32) and the convolutions' last ``conv_taps - 1`` inputs live in the request's record of the
cache manager's state pool, so a request goes on in a later step, alone or beside others, from where it
stopped.  Everything between the projections and the output projection is float32.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import Mixer, StateNeed, TensorDecl, register_part


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class GatedDeltaRule(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.H = int(p["heads"])
        self.Hk = int(p.get("kv_heads", self.H))
        self.dk = int(p["key_dim"])
        self.dv = int(p["value_dim"])
        self.taps = int(p.get("conv_taps", 1))
        self.decay = str(p.get("decay", "head"))
        self.gate = str(p.get("gate", "silu"))
        self.decay_rank = p.get("decay_rank", 0)
        self.gate_rank = p.get("gate_rank", 0)
        self.eps = float(p["eps"])
        if self.H <= 0 or self.Hk <= 0 or self.H % self.Hk:
            raise ValueError("gated_delta_rule: heads must be a multiple of kv_heads")
        if self.decay not in ("head", "channel") or self.gate not in ("silu", "sigmoid"):
            raise ValueError("gated_delta_rule: decay is 'head' or 'channel', gate 'silu' or 'sigmoid'")
        if self.taps < 1 or self.dk > 256:
            raise ValueError("gated_delta_rule: conv_taps >= 1 and key_dim <= 256 are built")
        self.Cq = self.Hk * self.dk
        self.Cv = self.H * self.dv
        self.n_decay = self.H * self.dk if self.decay == "channel" else self.H
        self.state_floats = self.H * self.dk * self.dv
        self.w_in = None

    # ------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorDecl]:
        h = self.hidden_size
        d = {
            "q": TensorDecl((self.Cq, h)), "q.conv": TensorDecl((self.Cq, self.taps), "bias", std=0.4),
            "k": TensorDecl((self.Cq, h)), "k.conv": TensorDecl((self.Cq, self.taps), "bias", std=0.4),
            "v": TensorDecl((self.Cv, h)), "v.conv": TensorDecl((self.Cv, self.taps), "bias", std=0.4),
            "b": TensorDecl((self.H, h)),
            "A_log": TensorDecl((self.H,), "bias", std=0.5, mean=-1.0),
            "dt_bias": TensorDecl((self.n_decay,), "bias", std=0.5),
            "norm": TensorDecl((self.dv,), "norm"),
            "o": TensorDecl((h, self.Cv)),
        }
        if self.decay_rank == 0:
            d["a"] = TensorDecl((self.n_decay, h))
        else:
            d["a1"] = TensorDecl((self.decay_rank, h))
            d["a2"] = TensorDecl((self.n_decay, self.decay_rank))
        if self.gate_rank == 0:
            d["g"] = TensorDecl((self.Cv, h))
        else:
            d["g1"] = TensorDecl((self.gate_rank, h))
            d["g2"] = TensorDecl((self.Cv, self.gate_rank))
        return d

    def load(self, fetch, dtype, device) -> None:
        h = self.hidden_size

        def f32(name):
            return fetch(name).to(torch.float32).to(device).contiguous()

        # one product for everything that reads the mixer's input; every segment starts at a multiple of 8 rows
        segs = [("q", fetch("q")), ("k", fetch("k")), ("v", fetch("v")), ("b", fetch("b"))]
        self.w_a2 = self.w_g2 = None
        if self.decay_rank == 0:
            segs.append(("a", fetch("a")))
        else:
            a1, a2 = fetch("a1"), fetch("a2")
            if a2.shape[1] != a1.shape[0]:
                raise ValueError(f"{self.prefix}a2 takes {a2.shape[1]} numbers but a1 makes {a1.shape[0]}")
            segs.append(("a", a1))
            self.w_a2 = a2.to(dtype).to(device).contiguous()
        if self.gate_rank == 0:
            segs.append(("g", fetch("g")))
        else:
            g1, g2 = fetch("g1"), fetch("g2")
            if g2.shape[1] != g1.shape[0]:
                raise ValueError(f"{self.prefix}g2 takes {g2.shape[1]} numbers but g1 makes {g1.shape[0]}")
            segs.append(("g", g1))
            self.w_g2 = g2.to(dtype).to(device).contiguous()
        self.off, self.width = {}, {}
        rows, at = [], 0
        for name, w in segs:
            self.off[name], self.width[name] = at, w.shape[0]
            rows.append(w.to(dtype))
            pad = _pad8(w.shape[0]) - w.shape[0]
            if pad:
                rows.append(torch.zeros((pad, h), dtype=dtype, device=w.device))
            at += _pad8(w.shape[0])
        self.w_in = torch.cat(rows, dim=0).to(device).contiguous()
        self.conv_q, self.conv_k, self.conv_v = f32("q.conv"), f32("k.conv"), f32("v.conv")
        self.A_log, self.dt_bias, self.norm_w = f32("A_log"), f32("dt_bias"), f32("norm")
        self.w_o = fetch("o").to(dtype).to(device).contiguous()

    def weight_bytes(self) -> int:
        ts = [self.w_in, self.w_o, self.w_a2, self.w_g2, self.conv_q, self.conv_k, self.conv_v]
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def cache_need(self):
        return StateNeed((self.state_floats + (self.taps - 1) * (2 * self.Cq + self.Cv),), "float32")

    def kernel_libraries(self):
        libs = ["core", "delta_rule"]
        if self.w_in is not None and self.w_in.dtype == torch.bfloat16:
            libs.extend(["gemm_smallm", "gemm_stream", "gemm_tc"])
        return libs

    # ------------------------------------------------------------------
    def forward(self, x, step, cache):
        n, dev = x.shape[0], x.device
        proj = ops.linear(x, self.w_in)
        a_in = proj[:, self.off["a"]:self.off["a"] + self.width["a"]]
        if self.w_a2 is not None:
            a_in = ops.linear(a_in, self.w_a2)
        gate = proj[:, self.off["g"]:self.off["g"] + self.width["g"]]
        if self.w_g2 is not None:
            gate = ops.linear(gate, self.w_g2)
        f32 = dict(dtype=torch.float32, device=dev)
        qn = torch.empty((n, self.Cq), **f32)
        kn = torch.empty((n, self.Cq), **f32)
        vc = torch.empty((n, self.Cv), **f32)
        beta = torch.empty((n, self.H), **f32)
        g = torch.empty((n, self.n_decay), **f32)
        o = torch.empty((n, self.Cv), **f32)
        per_channel = self.decay == "channel"
        ops.delta_prepare(proj, self.off["q"], self.off["k"], self.off["v"], self.off["b"], a_in, self.conv_q,
                          self.conv_k, self.conv_v, self.A_log, self.dt_bias, cache.state, self.state_floats, step,
                          qn, kn, vc, beta, g, self.H, self.Hk, self.dk, self.dv, self.taps, per_channel)
        ops.delta_recurrence(qn, kn, vc, beta, g, cache.state, step, o, self.H, self.Hk, self.dk, self.dv,
                             per_channel)
        y = torch.empty((n, self.Cv), dtype=x.dtype, device=dev)
        ops.delta_out(y, o, self.norm_w, gate, self.eps, self.H, self.dv, 0 if self.gate == "silu" else 1)
        return ops.linear(y, self.w_o)


register_part("mixer", "gated_delta_rule", GatedDeltaRule)
