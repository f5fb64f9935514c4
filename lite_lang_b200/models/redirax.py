"""Redirax: a decoder-only model whose residual is several streams wide and whose mixer is two mixers side by side.

config.json (``"architecture": "Redirax"``) gives ``vocab``, ``width``, ``streams``, ``norm.eps``,
``logit_softcap`` (optional) and ``layers``: a list whose entries name the layer's ``type`` (``parallel``), the
mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  ``weights_of: j`` in an entry makes it a second run of layer j's
parts (the checkpoint holds nothing under its own index); cache planes and state records are per run.

A layer is pre-norm over ``streams`` residual rows a token (``parts/streams.py``): each sublayer reads a weighted
sum of the streams through a dynamic-tanh norm and is written back through a small mixing matrix.

Mixer ``parallel`` (``parts/side_by_side.py``): ``left`` is softmax attention with grouped key/value heads
(``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``; biases on q, k, v and the output projection; rotary pairs
(2i, 2i+1) on the first ``rot.dims`` channels with ``rot.base``, positions divided by ``rot.scaling.factor``);
``right`` is linear attention with a decay per head (``heads``, ``dim``, ``vdim``, ``decay``); the two outputs
are RMS-normed and averaged.

Feed-forward, by ``mlp.kind``: ``dense``: down(relu(gate x) * up x) of width ``ff``.  ``moe``: ``router.experts``
gated experts of width ``expert.ff`` clamped at ``expert.limit``; a token goes through the ``router.top`` best by
router logit (the router has a bias), weighted by the softmax over just those logits; ``shared`` (optional:
``ff``, ``limit``) adds an always-on expert, times a sigmoid gate.

Tensor names: ``embed``, ``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``), ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.mix.left|right.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from ..config.base import ConfigError, ModelConfig, _require, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunStep

LAYER_TYPES = ("parallel",)
# positions are float32 inside the rotation: every position below 2^24 is exact
MAX_POSITIONS = 1 << 24


def _sub(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"Redirax: {where} lacks the section {key!r}")
    return v


@dataclass(frozen=True)
class RediraxConfig(ModelConfig):
    vocab: int
    width: int
    streams: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]      # as in config.json (validated)
    logit_softcap: Optional[float] = None
    eos_token_id: Tuple[int, ...] = ()
    initializer_range: float = 0.05

    architecture = "Redirax"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RediraxConfig":
        a = cls.architecture
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{a}: config.json lacks the list 'layers'")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        cap = d.get("logit_softcap")
        cfg = cls(vocab=_require(d, "vocab", int, a), width=_require(d, "width", int, a),
                  streams=int(d.get("streams") or 1),
                  norm_eps=float(_require(_sub(d, "norm", "config.json"), "eps", float, a)),
                  layers=tuple(copy.deepcopy(dict(l)) for l in layers),
                  logit_softcap=None if not cap else float(cap), eos_token_id=eos_ids,
                  initializer_range=float(d.get("initializer_range", 0.05)))
        cfg.validate()
        return cfg

    def source(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it says ``weights_of``)."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            if i in seen:
                raise ConfigError(f"{self.architecture}: 'weights_of' goes in a circle at layer {i}")
            seen.add(i)
            i = int(self.layers[i]["weights_of"])
        return i

    def validate(self) -> None:
        a = self.architecture
        if self.vocab <= 0 or self.width <= 0 or self.norm_eps <= 0 or not (1 <= self.streams <= 8):
            raise ConfigError(f"{a}: vocab, width and norm.eps must be positive, streams 1 to 8")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            if layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"{a}: {where} has the type {layer.get('type')!r}; built: {', '.join(LAYER_TYPES)}")
            j = layer.get("weights_of")
            if j is not None and not (0 <= int(j) < len(self.layers)):
                raise ConfigError(f"{a}: {where} uses the weights of layer {j}, which does not exist")
            m = _sub(layer, "mixer", where)
            left, right = _sub(m, "left", where), _sub(m, "right", where)
            for key in ("heads", "kv_heads", "dim", "vdim", "scale"):
                _require(left, key, float, f"{a} {where} left")
            if int(left["heads"]) % int(left["kv_heads"]):
                raise ConfigError(f"{a}: {where}: heads is not a multiple of kv_heads")
            rot = _sub(left, "rot", where)
            _require(rot, "base", float, f"{a} {where} rot")
            dims = int(_require(rot, "dims", int, f"{a} {where} rot"))
            if dims > int(left["dim"]) or dims % 2:
                raise ConfigError(f"{a}: {where}: rot.dims must be even and at most dim")
            for key in ("heads", "dim", "vdim"):
                _require(right, key, int, f"{a} {where} right")
            decay = right.get("decay")
            if not isinstance(decay, (list, tuple)) or len(decay) != int(right["heads"]):
                raise ConfigError(f"{a}: {where}: right.decay must give one number a head")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if mlp.get("kind") == "dense":
                _require(mlp, "ff", int, f"{a} {where} mlp")
            elif mlp.get("kind") == "moe":
                r = _sub(mlp, "router", where)
                _require(r, "experts", int, f"{a} {where} router")
                _require(r, "top", int, f"{a} {where} router")
                e = _sub(mlp, "expert", where)
                _require(e, "ff", int, f"{a} {where} expert")
                _require(e, "limit", float, f"{a} {where} expert")
                if mlp.get("shared") is not None:
                    _require(mlp["shared"], "ff", int, f"{a} {where} shared")
                    _require(mlp["shared"], "limit", float, f"{a} {where} shared")
            else:
                raise ConfigError(f"{a}: {where} has a feed-forward of kind {mlp.get('kind')!r}; built: dense, moe")
        for i in range(len(self.layers)):
            self.source(i)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(dict(l)) for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "streams": self.streams,
            "vocab": self.vocab,
            "width": self.width,
            # (read by this package's own tools: the tests' trace helper and the random-weights writer)
            "vocab_size": self.vocab,
            "initializer_range": self.initializer_range,
        }
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def init_scales(self) -> Dict[str, float]:
        s = self.initializer_range
        return {"matrix": s, "bias": s, "norm": s}

    # ------------------------------------------------------------------
    def _mixer_spec(self, prefix: str, m: Mapping[str, Any]) -> PartSpec:
        left, right = m["left"], m["right"]
        rot = left["rot"]
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        names = {r: (r, r + ".b") for r in ("q", "k", "v", "o")}
        left_params = {
            "hidden_size": self.width, "num_heads": int(left["heads"]), "num_kv_heads": int(left["kv_heads"]),
            "head_dim": int(left["dim"]), "value_head_dim": int(left["vdim"]), "qkv_bias": True, "out_bias": True,
            "scale": float(left["scale"]), "tensor_names": names,
            "position": PartSpec("rope_computed", {"rotary_dim": int(rot["dims"]), "theta": float(rot["base"]),
                                                   "position_scale": factor, "layout": "interleaved"})}
        right_params = {"hidden_size": self.width, "heads": int(right["heads"]), "key_dim": int(right["dim"]),
                        "value_dim": int(right["vdim"]), "decay": [float(x) for x in right["decay"]],
                        "eps": self.norm_eps}
        return PartSpec("side_by_side", {"hidden_size": self.width, "eps": self.norm_eps,
                                         "left": {"kind": "gqa_attention", "params": left_params},
                                         "right": {"kind": "decay_linear_attention", "params": right_params}}, prefix)

    def _mlp_spec(self, prefix: str, mlp: Mapping[str, Any]) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                          "activation": "relu", "tensor_names": ("gate", "up", "down")}, prefix)
        shared = mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "experts": int(mlp["router"]["experts"]), "top": int(mlp["router"]["top"]),
            "expert_ff": int(mlp["expert"]["ff"]), "shared_ff": 0 if shared is None else int(shared["ff"]),
            "gated": True, "limit": float(mlp["expert"]["limit"]),
            "shared_limit": None if shared is None else float(shared["limit"]), "swish_alpha": 1.702,
            "score": "softmax_top", "router_bias": True, "shared_gate": shared is not None}, prefix)

    def model_spec(self) -> ModelSpec:
        layers: List[LayerSpec] = []
        where: Dict[int, int] = {}       # config layer with tensors of its own -> index among the built layers
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            p = f"l{i}."
            norm = {"hidden_size": self.width, "streams": self.streams, "tensor": ""}
            parts = {"mixer_norm": PartSpec("dynamic_tanh", norm, p + "norm1"),
                     "mixer": self._mixer_spec(p + "mix.", layer["mixer"]),
                     "mixer_link": PartSpec("stream_link", {"streams": self.streams}, p + "hc1.")}
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward_norm"] = PartSpec("dynamic_tanh", norm, p + "norm2")
                parts["feed_forward"] = self._mlp_spec(p + "mlp.", mlp)
                parts["feed_forward_link"] = PartSpec("stream_link", {"streams": self.streams}, p + "hc2.")
            where[i] = len(layers)
            layers.append(LayerSpec("hyper_pre_norm" if mlp is not None else "hyper_mixer_only", parts))
        order = tuple(RunStep(where[self.source(i)]) for i in range(len(self.layers)))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": self.width,
                                                   "residual": "float32", "streams": self.streams, "tensor": ""},
                               "embed"),
            layers=tuple(layers), order=order,
            final_norm=PartSpec("dynamic_tanh", {"hidden_size": self.width, "streams": self.streams, "tensor": ""},
                                "final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": self.width, "tied_to": None,
                                      "tensor": "", "softcap": self.logit_softcap}, "head"),
            eos_token_ids=self.eos_token_id)


register_architecture(RediraxConfig.architecture, RediraxConfig)
