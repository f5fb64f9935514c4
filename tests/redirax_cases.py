"""Small Redirax configurations for the tests, and a helper that writes them as model folders."""

from __future__ import annotations

import os
import tempfile
from typing import Optional


def _left(heads, kv_heads, dim, vdim, rot_dims, base, factor, scale):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor}}}


def _right(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def _moe(experts, top, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(left, right, mlp, weights_of=None):
    d = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


_P0 = (_left(3, 3, 24, 40, 10, 10000.0, 3.0, 0.31), _right(3, 20, 12, [0.5, 0.9, 0.995]))
_P1 = (_left(6, 2, 16, 8, 16, 500.0, 1.0, 0.2), _right(1, 40, 36, [0.97]))
_Q0 = (_left(8, 2, 64, 64, 32, 1e6, 4.0, 0.11), _right(2, 128, 64, [0.8, 0.999]))
_Q1 = (_left(4, 4, 128, 128, 128, 10000.0, 2.0, 0.07), _right(5, 16, 16, [0.3, 0.6, 0.9, 0.99, 1.0]))
_R0 = (_left(9, 1, 20, 28, 6, 77.0, 16.0, 0.4), _right(2, 24, 44, [0.9, 0.95]))

CASES = {
    # odd sizes: three streams, no width or head size a power of two, every query head with a key head of its own
    # in one layer and narrow values in another, rotation on a part of the channels, a scale that is not
    # dim^-1/2, a layer without a feed-forward, layers run with another layer's weights (one borrows from a
    # layer that comes after it), all experts chosen, no shared expert, no cap on the logits
    "P": {
        "config": {"architecture": "Redirax", "vocab": 211, "width": 88, "streams": 3, "norm": {"eps": 3e-6},
                   "layers": [
                       _layer(*_P0, _moe(4, 4, 24, 1.5)),
                       _layer(*_P1, None, weights_of=3),
                       _layer(*_P0, _moe(4, 4, 24, 1.5), weights_of=0),
                       _layer(*_P1, None),
                       _layer(*_P0, _dense(50)),
                   ]},
        "seed": 5, "page_size": 4},
    # heads of 64 and 128 with values as wide as keys (the tensor-core attention kernels in bfloat16), one
    # stream, a decay of exactly 1, many experts with one chosen, a shared expert wider than the routed ones
    "Q": {
        "config": {"architecture": "Redirax", "vocab": 300, "width": 128, "streams": 1, "norm": {"eps": 1e-5},
                   "logit_softcap": 12.0,
                   "layers": [
                       _layer(*_Q0, _moe(12, 1, 24, 0.7, (48, 2.5))),
                       _layer(*_Q1, _dense(96)),
                       _layer(*_Q0, _moe(12, 1, 24, 0.7, (48, 2.5)), weights_of=0),
                   ]},
        "seed": 6, "page_size": 16},
    # a width that is no multiple of 4 or 8, four streams, nine query heads on one key head (more than a block of
    # the attention kernel takes at once), values wider than keys, strong position scaling
    "R": {
        "config": {"architecture": "Redirax", "vocab": 97, "width": 90, "streams": 4, "norm": {"eps": 1e-6},
                   "logit_softcap": 50.0,
                   "layers": [
                       _layer(*_R0, _dense(33)),
                       _layer(*_R0, _moe(5, 2, 20, 3.0, (12, 0.5))),
                   ]},
        "seed": 7, "page_size": 8},
}


def write_folder(name: str, folder: Optional[str] = None, sharpen: float = 1.0) -> str:
    """Write the case as a model folder with random weights.  ``sharpen`` multiplies the attention queries' and the
    router's weights, so that a wrong key or expert would show."""
    from lite_lang_b200.config import config_from_dict
    from lite_lang_b200.weights import write_random_model

    case = CASES[name]
    cfg = config_from_dict(case["config"])
    folder = folder or tempfile.mkdtemp(prefix=f"ll_redirax_{name}_")
    write_random_model(folder, cfg, case["seed"], {"matrix": 0.12, "bias": 0.1, "norm": 0.1})
    if sharpen != 1.0:
        from safetensors.torch import load_file, save_file
        path = os.path.join(folder, "model.safetensors")
        t = load_file(path)
        for k in list(t):
            if k.endswith(".left.q") or k.endswith(".mlp.router"):
                t[k] = (t[k].float() * sharpen).to(t[k].dtype)
        save_file(t, path, metadata={"format": "pt"})
    return folder
