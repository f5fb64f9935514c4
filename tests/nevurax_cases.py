"""Small Nevurax configurations for the tests, and helpers that write them as model folders."""

from __future__ import annotations

import json
import os
import tempfile
from typing import Optional


def _moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, window, base, dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
            "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim if dims is None else dims},
            "scale": 2.0 * (dim + rot_dim) ** -0.5}


def _delta(heads, kv_heads, dim, vdim, conv, ranks=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if ranks is not None:
        m["decay_rank"], m["gate_rank"] = ranks
    return m


CASES = {
    # odd sizes everywhere: no width, head size or rank is a power of two; a layer without a feed-forward; one
    # expert chosen of three; kv heads shared by query heads in both delta kinds; convolutions of 2, 3 and 5 taps
    "P": {
        "config": {"architecture": "Nevurax", "vocab": 211, "width": 88, "embedding": {"scale": 1.7},
                   "norm": {"eps": 3e-6},
                   "layers": [
                       {"type": "latent_attention", "mixer": _latent(3, 24, 8, 20, 40, 19, 10000.0),
                        "mlp": _moe(5, 2, 24, 40)},
                       {"type": "delta", "mixer": _delta(4, 2, 24, 20, 3), "mlp": None},
                       {"type": "channel_delta", "mixer": _delta(2, 1, 16, 24, 2, (10, 6)), "mlp": _moe(3, 1, 32, None)},
                       {"type": "delta", "mixer": _delta(1, 1, 40, 36, 5), "mlp": _moe(4, 4, 16, 8)},
                   ]},
        "seed": 5, "page_size": 4},
    # a window longer than any test sequence beside a short one; rotation on a part of the rotated numbers only;
    # many experts; one tap (no convolution state)
    "Q": {
        "config": {"architecture": "Nevurax", "vocab": 300, "width": 128, "embedding": {"scale": 0.5},
                   "norm": {"eps": 1e-5},
                   "layers": [
                       {"type": "channel_delta", "mixer": _delta(3, 3, 40, 72, 4, (12, 20)), "mlp": _moe(12, 3, 24, 48)},
                       {"type": "latent_attention", "mixer": _latent(5, 32, 16, 32, 64, 33, 500.0, dims=8),
                        "mlp": _moe(6, 2, 40, 16)},
                       {"type": "delta", "mixer": _delta(2, 2, 64, 48, 1), "mlp": _moe(2, 1, 64, 64)},
                       {"type": "latent_attention", "mixer": _latent(2, 16, 32, 48, 24, 4000, 77.0), "mlp": None},
                   ]},
        "seed": 6, "page_size": 16},
    # a width that is no multiple of 8 (rows of bfloat16 that are not 16-byte aligned), cached rows of 43 numbers,
    # a window of one page
    "R": {
        "config": {"architecture": "Nevurax", "vocab": 97, "width": 100, "embedding": {"scale": 4.0},
                   "norm": {"eps": 1e-6},
                   "layers": [
                       {"type": "delta", "mixer": _delta(6, 3, 12, 28, 4), "mlp": _moe(7, 3, 20, 12)},
                       {"type": "latent_attention", "mixer": _latent(9, 20, 6, 12, 37, 8, 1e6, dims=4),
                        "mlp": _moe(3, 2, 44, 20)},
                       {"type": "channel_delta", "mixer": _delta(4, 4, 20, 12, 3, (5, 7)), "mlp": None},
                   ]},
        "seed": 7, "page_size": 8},
}


def write_folder(name: str, folder: Optional[str] = None, strip_ranks: bool = False, sharpen: float = 1.0) -> str:
    """Write the case as a model folder with random weights.  ``strip_ranks`` removes the low-rank widths from
    config.json afterwards, so that they have to be read from the checkpoint; ``sharpen`` multiplies the
    attention queries' and the router's weights, so that a wrong key or expert would show."""
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    case = CASES[name]
    cfg = config_from_dict(case["config"])
    folder = folder or tempfile.mkdtemp(prefix=f"ll_nevurax_{name}_")
    write_random_model(folder, cfg, case["seed"], {"matrix": 0.12, "bias": 0.1, "norm": 0.1})
    if sharpen != 1.0:
        from safetensors.torch import load_file, save_file
        path = os.path.join(folder, "model.safetensors")
        t = load_file(path)
        for k in list(t):
            if k.endswith(".mix.uk") or k.endswith(".mlp.router"):
                t[k] = (t[k].float() * sharpen).to(t[k].dtype)
        save_file(t, path, metadata={"format": "pt"})
    if strip_ranks:
        path = os.path.join(folder, "config.json")
        d = json.load(open(path))
        for layer in d["layers"]:
            layer["mixer"].pop("decay_rank", None)
            layer["mixer"].pop("gate_rank", None)
        for k in ("vocab_size", "initializer_range"):
            d.pop(k, None)
        json.dump(d, open(path, "w"))
    return folder
