"""Plain, slow Redirax forward pass: the oracle of the Redirax tests.

Whole sequences, no cache, no batching, one function for each mechanism, float64
throughout.  It shares no code with ``lite_lang_b200``: it reads ``config.json``
and ``model.safetensors`` itself and works on torch tensors on the CPU.

The design in this file's notation.

*Streams.*  The residual is s copies X[0..s-1] of the embedding row.  A sublayer
f with its norm N, read weights a [s], write weights c [s] and mixing matrix
M [s, s] (from, to) does

    y = f(N(sum_i a_i X_i));    X_j <- sum_i M[i, j] X_i + c_j y    (all j from the old X)

A layer is two sublayers, mixer then feed-forward (the latter may be absent).
The output norm reads sum_i X_i.

*Norm.*  N(u) = tanh(alpha u) * w + b with a scalar alpha: no statistics.

*Mixer.*  Two mixers read the same input h and are joined as
(R_l(left(h)) + R_r(right(h))) / 2, R being an RMS norm over the model width.
left: softmax attention with grouped key/value heads, biases on all four
projections, value heads that may be wider than key heads, rotation of the
first ``dims`` channels of q and k in interleaved pairs (2i, 2i+1) with angle
p * base^(-2i/dims) / factor, score = q.k * scale, causal.
right: linear attention with a decay per head: q, k, v = silu of projections,
S_t = d S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; all heads' o side by side are
RMS-normed as one vector, times sigmoid(G h), projected.

*Feed-forward.*  dense: D(relu(G h) * (U h)).  moe: router logits z = R h + r;
the ``top`` largest are chosen, weights = softmax over the chosen logits; an
expert is D(a * sigmoid(1.702 a) * (c + 1)) with a = min(G h, L), c = clamp(U h,
-L, L); a shared expert of the same form (its own L) is added times
sigmoid(w_sg . h).

*Output.*  logits = cap * tanh(H N(sum_i X_i) / cap).
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional, Tuple

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

def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def tanh_norm(u: torch.Tensor, alpha: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return torch.tanh(alpha * u) * w + b


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i+1), i < dims/2, turned by positions * base^(-2i/dims) / factor."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(F) * (base ** (-2.0 * i / dims) / factor)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        a, b = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


# --------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------

def causal_softmax(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """One head: q, k [T, d], v [T, dv]; row i sees keys 0..i."""
    T = q.shape[0]
    s = (q @ k.T) * scale
    s = s.masked_fill(torch.arange(T)[None, :] > torch.arange(T)[:, None], float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def softmax_attention(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str, m: Mapping) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ t[p + "q"].T + t[p + "q.b"]).view(T, H, d)
    k = (h @ t[p + "k"].T + t[p + "k.b"]).view(T, G, d)
    v = (h @ t[p + "v"].T + t[p + "v.b"]).view(T, G, dv)
    pos = torch.arange(T)
    rot = m["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    q = rotate_pairs(q, pos, int(rot["dims"]), float(rot["base"]), factor)
    k = rotate_pairs(k, pos, int(rot["dims"]), float(rot["base"]), factor)
    out = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        g = head // (H // G)
        out[:, head] = causal_softmax(q[:, head], k[:, g], v[:, g], float(m["scale"]))
    return out.reshape(T, H * dv) @ t[p + "o"].T + t[p + "o.b"]


def decay_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: float,
                     S: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One head: q, k [T, d], v [T, dv] -> o [T, dv] and the state after the last token."""
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F) if S is None else S.clone()
    o = torch.zeros(q.shape[0], v.shape[1], dtype=F)
    for i in range(q.shape[0]):
        S = decay * S + k[i][:, None] * v[i][None, :]
        o[i] = S.T @ q[i]
    return o, S


def decayed_linear_attention(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str, m: Mapping,
                             eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ t[p + "q"].T).view(T, H, d)
    k = silu(h @ t[p + "k"].T).view(T, H, d)
    v = silu(h @ t[p + "v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F)
    for head in range(H):
        o[:, head], _ = decay_recurrence(q[:, head], k[:, head], v[:, head], float(m["decay"][head]))
    o = rms_norm(o.reshape(T, H * dv), t[p + "norm"], eps) * sigmoid(h @ t[p + "g"].T)
    return o @ t[p + "o"].T


def side_by_side(h: torch.Tensor, t: Mapping[str, torch.Tensor], p: str, m: Mapping, eps: float) -> torch.Tensor:
    a = softmax_attention(h, t, p + "left.", m["left"])
    b = decayed_linear_attention(h, t, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(a, t[p + "left.out"], eps) + rms_norm(b, t[p + "right.out"], eps))


# --------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------

def dense_ff(h, t, p):
    return (torch.relu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def clamped_gate(g, u, limit: float):
    a = torch.clamp(g, max=limit)
    c = torch.clamp(u, min=-limit, max=limit)
    return a * sigmoid(1.702 * a) * (c + 1.0)


def clamped_expert(h, t, p, limit: float):
    return clamped_gate(h @ t[p + "gate"].T, h @ t[p + "up"].T, limit) @ t[p + "down"].T


def route(h, t, p, top: int) -> Tuple[torch.Tensor, torch.Tensor]:
    z = h @ t[p + "router"].T + t[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def moe_ff(h, t, p, mlp: Mapping) -> torch.Tensor:
    idx, w = route(h, t, p, int(mlp["router"]["top"]))
    out = torch.zeros(h.shape[0], t[p + "e0.down"].shape[0], dtype=F)
    limit = float(mlp["expert"]["limit"])
    for i in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[i, j])
            out[i] += w[i, j] * clamped_expert(h[i:i + 1], t, f"{p}e{e}.", limit)[0]
    shared = mlp.get("shared")
    if shared is not None:
        out = out + sigmoid(h @ t[p + "shared.sg"].T) * clamped_expert(h, t, p + "shared.", float(shared["limit"]))
    return out


def feed_forward(h, t, p, mlp: Mapping) -> torch.Tensor:
    if mlp["kind"] == "dense":
        return dense_ff(h, t, p)
    if mlp["kind"] == "moe":
        return moe_ff(h, t, p, mlp)
    raise ValueError(mlp["kind"])


# --------------------------------------------------------------------------
# streams, layers, model
# --------------------------------------------------------------------------

def stream_sublayer(X: torch.Tensor, f, t, norm: str, hc: str) -> torch.Tensor:
    """X [s, T, W] -> new X.  f maps the normed read-out [T, W] to the sublayer's output."""
    a, c, M = t[hc + "in"], t[hc + "out"], t[hc + "mix"]
    u = torch.einsum("i,itw->tw", a, X)
    y = f(tanh_norm(u, t[norm + ".alpha"], t[norm], t[norm + ".b"]))
    return torch.einsum("ij,itw->jtw", M, X) + c[:, None, None] * y[None]


def forward(cfg: Mapping, t: Mapping[str, torch.Tensor], tokens: List[int], return_layers: bool = False):
    """float64 logits [T, vocab] (and the sum of the streams after every layer run [runs, T, W])."""
    eps = float(cfg["norm"]["eps"])
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)]
    X = torch.stack([x] * int(cfg["streams"]))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        src = int(layer.get("weights_of", i))
        p = f"l{src}."
        X = stream_sublayer(X, lambda h: side_by_side(h, t, p + "mix.", layer["mixer"], eps), t, p + "norm1", p + "hc1.")
        if layer.get("mlp") is not None:
            X = stream_sublayer(X, lambda h: feed_forward(h, t, p + "mlp.", layer["mlp"]), t, p + "norm2", p + "hc2.")
        after.append(X.sum(0))
    z = tanh_norm(X.sum(0), t["final.norm.alpha"], t["final.norm"], t["final.norm.b"]) @ t["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        z = float(cap) * torch.tanh(z / float(cap))
    if return_layers:
        return z, torch.stack(after)
    return z
