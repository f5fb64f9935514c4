"""Nevurax: a decoder-only model of parallel layers whose mixers differ from layer to layer.

config.json (``"architecture": "Nevurax"``) gives ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``
and ``layers``: a list whose entries name the layer's mixer (``type``), the mixer's sizes (``mixer``) and
its feed-forward (``mlp``, or null for none).  Every layer is the parallel arrangement
h += mixer(n) + feed_forward(n) with n = layer norm of h (a weight, no bias); the residual stream is float32.

Mixers, by ``type``:
  ``delta``             gated delta rule, one decay per head (tensor ``a``), SiLU output gate (``g``)
  ``channel_delta``     gated delta rule, a decay per head and key channel through a low-rank pair
                        (``a1``, ``a2``), sigmoid output gate through a low-rank pair (``g1``, ``g2``); the
                        pairs' inner widths are read from the checkpoint unless the configuration names
                        them (``decay_rank``, ``gate_rank``: keys that a written random model carries)
  ``latent_attention``  latent attention with a sliding window (``mask.size``) and interleaved rotary
                        pairs (``rot.base``, ``rot.dims``) on the ``rot_dim`` part
Feed-forward, by ``mlp.kind``: ``moe``: ``router.experts`` experts of width ``expert.ff`` of which each token
uses ``router.top``, weighted by the router's softmax scores (not renormalised), activation relu squared,
plus a shared expert of width ``shared.ff`` where ``shared`` is given.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..config.base import ConfigError, ModelConfig, _require, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

MIXER_TYPES = ("delta", "channel_delta", "latent_attention")
# positions are float32 inside the rotation: every position below 2^24 is exact
MAX_POSITIONS = 1 << 24


def _sub(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"Nevurax: {where} lacks the section {key!r}")
    return v


@dataclass(frozen=True)
class NevuraxConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]      # as in config.json (validated)
    eos_token_id: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    architecture = "Nevurax"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "NevuraxConfig":
        a = cls.architecture
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{a}: config.json lacks the list 'layers'")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cfg = cls(vocab=_require(d, "vocab", int, a), width=_require(d, "width", int, a),
                  embedding_scale=float(_require(_sub(d, "embedding", "config.json"), "scale", float, a)),
                  norm_eps=float(_require(_sub(d, "norm", "config.json"), "eps", float, a)),
                  layers=tuple(copy.deepcopy(dict(l)) for l in layers), eos_token_id=eos_ids,
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        a = self.architecture
        if self.vocab <= 0 or self.width <= 0 or self.norm_eps <= 0:
            raise ConfigError(f"{a}: vocab, width and norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{a}: {where} has the type {kind!r}; built: {', '.join(MIXER_TYPES)}")
            m = _sub(layer, "mixer", where)
            if kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale"):
                    _require(m, key, float, f"{a} {where} mixer")
                _require(_sub(m, "mask", where), "size", int, f"{a} {where} mask")
                rot = _sub(m, "rot", where)
                _require(rot, "base", float, f"{a} {where} rot")
                if int(_require(rot, "dims", int, f"{a} {where} rot")) > int(m["rot_dim"]):
                    raise ConfigError(f"{a}: {where}: rot.dims exceeds rot_dim")
            else:
                for key in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    _require(m, key, int, f"{a} {where} mixer")
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ConfigError(f"{a}: {where}: heads is not a multiple of kv_heads")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "moe":
                    raise ConfigError(f"{a}: {where} has a feed-forward of kind {mlp.get('kind')!r}; built: 'moe'")
                r = _sub(mlp, "router", where)
                _require(r, "experts", int, f"{a} {where} router")
                _require(r, "top", int, f"{a} {where} router")
                _require(_sub(mlp, "expert", where), "ff", int, f"{a} {where} expert")
                if mlp.get("shared") is not None:
                    _require(mlp["shared"], "ff", int, f"{a} {where} shared")

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [copy.deepcopy(dict(l)) for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
            # (read by this package's own tools: the tests' trace helper and the random-weights writer)
            "vocab_size": self.vocab,
            "initializer_range": self.initializer_range,
        }
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def init_scales(self) -> Dict[str, float]:
        s = self.initializer_range
        return {"matrix": s, "bias": s, "norm": s}

    # ------------------------------------------------------------------
    def _mixer_spec(self, i: int, layer: Mapping[str, Any]) -> PartSpec:
        m, kind, prefix = layer["mixer"], layer["type"], f"l{i}.mix."
        if kind == "latent_attention":
            return PartSpec("latent_attention", {
                "hidden_size": self.width, "heads": int(m["heads"]), "dim": int(m["dim"]),
                "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]),
                "window": int(m["mask"]["size"]), "scale": float(m["scale"]), "rot_base": float(m["rot"]["base"]),
                "rot_dims": int(m["rot"]["dims"]), "eps": self.norm_eps}, prefix)
        params = {"hidden_size": self.width, "heads": int(m["heads"]), "kv_heads": int(m["kv_heads"]),
                  "key_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "conv_taps": int(m["conv"]),
                  "eps": self.norm_eps}
        if kind == "channel_delta":
            params.update(decay="channel", gate="sigmoid",
                          decay_rank=None if m.get("decay_rank") is None else int(m["decay_rank"]),
                          gate_rank=None if m.get("gate_rank") is None else int(m["gate_rank"]))
        else:
            params.update(decay="head", gate="silu", decay_rank=0, gate_rank=0)
        return PartSpec("gated_delta_rule", params, prefix)

    def model_spec(self) -> ModelSpec:
        norm = {"hidden_size": self.width, "eps": self.norm_eps, "tensor": ""}
        layers: List[LayerSpec] = []
        for i, layer in enumerate(self.layers):
            parts = {"norm": PartSpec("layer_norm_f32", norm, f"l{i}.norm1"), "mixer": self._mixer_spec(i, layer)}
            mlp = layer.get("mlp")
            if mlp is None:
                layers.append(LayerSpec("parallel_mixer_only", parts))
                continue
            shared = mlp.get("shared")
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden_size": self.width, "experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]),
                "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": 0 if shared is None else int(shared["ff"]),
                "activation": "relu2", "score": "softmax", "renormalize": False}, f"l{i}.mlp.")
            layers.append(LayerSpec("parallel", parts))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "scale": self.embedding_scale, "residual": "float32",
                                                   "tensor": ""}, "embed"),
            layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(layers))),
            final_norm=PartSpec("layer_norm_f32", norm, "final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": None,
                                      "tensor": ""}, "head"),
            eos_token_ids=self.eos_token_id)


register_architecture(NevuraxConfig.architecture, NevuraxConfig)
