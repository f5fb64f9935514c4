"""Plain, slow Nevurax forward pass: the oracle of the Nevurax tests.

Whole sequences, no cache, no batching, one function for each mechanism, float64
throughout.  It shares no code with ``lite_lang_b200``: it reads ``config.json``
and ``model.safetensors`` itself and works on torch tensors on the CPU.

The design in this file's notation.  A layer is *parallel*: with n = LN(x)
(layer norm with a weight and no bias), x <- x + (mixer(n) + ff(n)).  Mixers:

``delta`` / ``channel_delta``  gated delta rule.  q, k (kv_heads x dk) and v
    (heads x dv) are projections of n, each passed through a causal depthwise
    convolution over time and SiLU; q and k are made unit vectors per head and
    q is scaled by dk^-1/2.  With b = sigmoid(B n) and a decay g in (0, 1) (one
    per head, or one per head and key channel), a head's state S [dk, dv]
    evolves as S <- diag(g) S; u = b (v - S^T k); S <- S + k u^T; o = S^T q.
    o is RMS-normed over dv, times a weight, times a gate, then projected.
``latent_attention``  softmax attention over a sliding window whose keys and
    values are expanded from one normed latent vector per token, plus one
    rotated key part per token shared by all heads.

Feed-forward: a router's softmax picks ``top`` of ``experts`` small
feed-forwards (down(relu(up n)^2)), weighted by their unrenormalised scores,
plus a shared expert of the same form that always runs.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Tuple

import torch
from safetensors import safe_open

F = torch.float64


def read_model_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as fh:
        for name in fh.keys():
            t = fh.get_tensor(name)
            tensors[name] = t.to(F) if t.is_floating_point() else t
    return cfg, tensors


# --------------------------------------------------------------------------
# small pieces
# --------------------------------------------------------------------------

def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_div(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def short_conv(x: torch.Tensor, taps_w: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps_w [C, K]: y[t, c] = sum_j taps_w[c, K-1-j] x[t-j, c], zeros before the start."""
    T, C = x.shape
    K = taps_w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            if t - j >= 0:
                y[t] += taps_w[:, K - 1 - j] * x[t - j]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g, S0=None):
    """One head.  q, k [T, dk]; v [T, dv]; beta [T]; g [T] or [T, dk].  Returns o [T, dv] and the last state."""
    T, dk = q.shape
    dv = v.shape[1]
    S = torch.zeros(dk, dv, dtype=F) if S0 is None else S0.clone()
    out = torch.zeros(T, dv, dtype=F)
    for t in range(T):
        gt = g[t].reshape(-1, 1) if g.dim() == 2 else g[t]
        S = gt * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.t() @ q[t]
    return out, S


# --------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------

def delta_mixer(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, per_channel: bool):
    """``p`` is the tensor prefix of the mixer ('l3.mix.')."""
    T = n.shape[0]
    H, Hk, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(n @ w[p + "q"].t(), w[p + "q.conv"])).view(T, Hk, dk)
    k = silu(short_conv(n @ w[p + "k"].t(), w[p + "k.conv"])).view(T, Hk, dk)
    v = silu(short_conv(n @ w[p + "v"].t(), w[p + "v.conv"])).view(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = sigmoid(n @ w[p + "b"].t())                                     # [T, H]
    rate = torch.exp(w[p + "A_log"])                                       # [H]
    if per_channel:
        a = ((n @ w[p + "a1"].t()) @ w[p + "a2"].t() + w[p + "dt_bias"]).view(T, H, dk)
        g = torch.exp(-rate.view(1, H, 1) * softplus(a))                   # [T, H, dk]
        gate = sigmoid((n @ w[p + "g1"].t()) @ w[p + "g2"].t()).view(T, H, dv)
    else:
        a = n @ w[p + "a"].t() + w[p + "dt_bias"]
        g = torch.exp(-rate.view(1, H) * softplus(a))                      # [T, H]
        gate = silu(n @ w[p + "g"].t()).view(T, H, dv)
    rep = H // Hk
    outs = []
    for h in range(H):
        o, _ = delta_rule(q[:, h // rep], k[:, h // rep], v[:, h], beta[:, h], g[:, h])
        outs.append(rms_div(o, eps) * w[p + "norm"] * gate[:, h])
    return torch.cat(outs, dim=1) @ w[p + "o"].t()


def rotate_pairs(x: torch.Tensor, pos: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., d]: dimension 2i is paired with 2i+1 for 2i < dims; the rest passes unchanged."""
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    a = pos.to(F).view(-1, *([1] * (x.dim() - 2)), 1) * f
    c, s = torch.cos(a), torch.sin(a)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention_mixer(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    T = n.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (n @ w[p + "q"].t()).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], q[..., d:]
    dkv = n @ w[p + "dkv"].t()
    c = rms_div(dkv[:, :R], eps) * w[p + "dkv.norm"]
    k_rot = dkv[:, R:]
    rot = m["rot"]
    q_rot = rotate_pairs(q_rot, pos, float(rot["base"]), int(rot["dims"]))
    k_rot = rotate_pairs(k_rot, pos, float(rot["base"]), int(rot["dims"]))
    k_plain = (c @ w[p + "uk"].t()).view(T, H, d)
    val = (c @ w[p + "uv"].t()).view(T, H, dv)
    window = int(m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        lo = max(0, t - window + 1)
        for h in range(H):
            s = (k_plain[lo:t + 1, h] @ q_plain[t, h] + k_rot[lo:t + 1] @ q_rot[t, h]) * m["scale"]
            pr = torch.softmax(s, dim=0)
            out[t, h] = pr @ val[lo:t + 1, h]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


# --------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------

def expert(n, up, down):
    return (torch.relu(n @ up.t()) ** 2) @ down.t()


def routed_choice(n: torch.Tensor, router: torch.Tensor, top: int):
    """Chosen experts [T, top] and their weights (softmax scores, not renormalised)."""
    s = torch.softmax(n @ router.t(), dim=-1)
    wts, idx = torch.topk(s, top, dim=-1)
    return idx, wts


def moe(n: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, wts = routed_choice(n, w[p + "router"], top)
    out = torch.zeros(n.shape[0], w[p + "e0.down"].shape[0], dtype=F)
    for t in range(n.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wts[t, j] * expert(n[t:t + 1], w[p + f"e{e}.up"], w[p + f"e{e}.down"])[0]
    if mlp.get("shared") is not None:
        out = out + expert(n, w[p + "shared.up"], w[p + "shared.down"])
    return out


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------

def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, keep_layers: bool = False):
    """Logits [T, vocab] (float64); with ``keep_layers`` also the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * float(cfg["embedding"]["scale"])
    kept = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = layer_norm(x, w[p + "norm1"], eps)
        kind = layer["type"]
        if kind == "latent_attention":
            a = latent_attention_mixer(n, w, p + "mix.", layer["mixer"], eps)
        elif kind in ("delta", "channel_delta"):
            a = delta_mixer(n, w, p + "mix.", layer["mixer"], eps, kind == "channel_delta")
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        f = moe(n, w, p + "mlp.", layer["mlp"]) if layer.get("mlp") is not None else 0.0
        x = x + (a + f)
        if keep_layers:
            kept.append(x.clone())
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].t()
    return (logits, torch.stack(kept)) if keep_layers else logits
