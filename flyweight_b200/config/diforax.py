"""Typed configuration of Diforax: a decoder whose layers wrap each sublayer in two weighted RMS norms
(one in front, one on its output) and mix two kinds of token mixers -- attention inside chunks of the
sequence, and a gated delta rule with a matrix state per head -- with dense gated feed-forwards or
routed experts.

``config.json`` keys: ``architecture`` ("Diforax"), ``vocab``, ``width``, ``norm.eps`` and ``layers``, a
list whose entries give ``type`` ("attention" | "delta"), ``mixer`` (its sizes and constants) and ``mlp``
(a feed-forward, or null).

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` (``base``, ``dims``),
  ``mask.size`` (the chunk length; absent: every earlier key is seen) and optionally ``kv_from``, the index
  of an earlier attention layer whose cached keys and values this layer reads with queries of its own.
* ``delta``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps of the short convolution).
* ``mlp``: ``{"kind": "dense", "ff": F}`` (gelu, tanh form, on the gate) or ``{"kind": "moe", "expert":
  {"ff": F}, "router": {"experts": E, "identity": I, "top": k, "groups": {"count": g, "keep": m}}}`` (silu on
  the gate; the router has E + I outputs, the last I of which are identity experts).

Tensor names: ``embed``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``norm1b``, ``norm2``, ``norm2b``;
``l<i>.mix.{q,k,v,o}`` for attention; ``l<i>.mix.{q,k,v,q.conv,k.conv,v.conv,b,a,A_log,dt_bias,g,norm,o}``
for the delta rule; ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router,correction,e<j>.gate,e<j>.up,e<j>.down}``.
The file states no context limit: the engine's page pool is the only one.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Tuple

from .lfm2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

UNBOUNDED_POSITIONS = 1 << 24


def _need(mapping: Any, keys, where: str) -> None:
    if not isinstance(mapping, Mapping):
        raise ConfigError(f"Diforax config.json: {where} must be an object")
    missing = [key for key in keys if mapping.get(key) is None]
    if missing:
        raise ConfigError(f"Diforax config.json: {where} is missing " + ", ".join(missing))


def _positive(mapping: Mapping[str, Any], keys, where: str) -> None:
    for key in keys:
        if int(mapping[key]) <= 0:
            raise ConfigError(f"Diforax config.json: {where}: {key} must be positive")


@dataclass(frozen=True)
class DiforaxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]          # as config.json gives them, checked and completed
    architectures: Tuple[str, ...] = ("Diforax",)
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ reading / writing
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "DiforaxConfig":
        _need(raw, ("vocab", "width", "norm", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("Diforax config.json: 'layers' must be a list with at least one layer")
        layers = []
        for index, layer in enumerate(raw["layers"]):
            where = f"layer {index}"
            _need(layer, ("type", "mixer"), where)
            layer = copy.deepcopy(dict(layer))
            mixer = layer["mixer"]
            if layer["type"] == "attention":
                cls._check_attention(mixer, index, layers, where)
            elif layer["type"] == "delta":
                _need(mixer, ("heads", "kv_heads", "dim", "vdim", "conv"), f"{where}'s mixer")
                _positive(mixer, ("heads", "kv_heads", "dim", "vdim", "conv"), f"{where}'s mixer")
                if int(mixer["heads"]) % int(mixer["kv_heads"]):
                    raise ConfigError(f"Diforax config.json: {where}: heads must be a multiple of kv_heads")
            else:
                raise ConfigError(f"Diforax config.json: {where} has the unknown type {layer['type']!r} "
                                  "(known: attention, delta)")
            cls._check_mlp(layer.get("mlp"), where)
            layers.append(layer)
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   layers=tuple(layers), extra={k: v for k, v in raw.items() if k not in known})

    @staticmethod
    def _check_attention(mixer, index, earlier, where) -> None:
        source = mixer.get("kv_from") if isinstance(mixer, Mapping) else None
        if source is not None:
            source = int(source)
            if (not 0 <= source < index or earlier[source]["type"] != "attention"
                    or earlier[source]["mixer"].get("kv_from") is not None):
                raise ConfigError(f"Diforax config.json: {where} reads the keys of layer {source}, which is no "
                                  "earlier attention layer with keys of its own")
            # what a layer that reads another's keys does not say about them is the source's
            for key in ("kv_heads", "dim", "vdim", "rot"):
                if mixer.get(key) is None and earlier[source]["mixer"].get(key) is not None:
                    mixer[key] = copy.deepcopy(earlier[source]["mixer"][key])
        _need(mixer, ("heads", "kv_heads", "dim", "vdim", "scale"), f"{where}'s mixer")
        _positive(mixer, ("heads", "kv_heads", "dim", "vdim"), f"{where}'s mixer")
        if int(mixer["heads"]) % int(mixer["kv_heads"]):
            raise ConfigError(f"Diforax config.json: {where}: heads must be a multiple of kv_heads")
        rot = mixer.get("rot")
        if rot is not None:
            _need(rot, ("base", "dims"), f"{where}'s mixer.rot")
            if int(rot["dims"]) % 2 or not 0 <= int(rot["dims"]) <= int(mixer["dim"]):
                raise ConfigError(f"Diforax config.json: {where}: rot.dims must be even and at most dim")
        mask = mixer.get("mask")
        if mask is not None:
            _need(mask, ("size",), f"{where}'s mixer.mask")
            _positive(mask, ("size",), f"{where}'s mixer.mask")
        if source is not None:
            theirs = earlier[source]["mixer"]
            if any(theirs.get(key) != mixer.get(key) for key in ("kv_heads", "dim", "vdim", "rot")):
                raise ConfigError(f"Diforax config.json: {where} and layer {source} must agree on kv_heads, "
                                  "dim, vdim and rot")

    @staticmethod
    def _check_mlp(mlp, where) -> None:
        if mlp is None:
            return
        _need(mlp, ("kind",), f"{where}'s mlp")
        if mlp["kind"] == "dense":
            _need(mlp, ("ff",), f"{where}'s mlp")
            _positive(mlp, ("ff",), f"{where}'s mlp")
        elif mlp["kind"] == "moe":
            _need(mlp, ("expert", "router"), f"{where}'s mlp")
            _need(mlp["expert"], ("ff",), f"{where}'s mlp.expert")
            router = mlp["router"]
            _need(router, ("experts", "top"), f"{where}'s mlp.router")
            outputs = int(router["experts"]) + int(router.get("identity") or 0)
            groups = router.get("groups") or {}
            count = int(groups.get("count") or 1)
            keep = int(groups.get("keep") or count)
            if count <= 0 or outputs % count or not 0 < keep <= count:
                raise ConfigError(f"Diforax config.json: {where}: {outputs} router outputs do not form {count} "
                                  f"equal groups of which {keep} are kept")
            if not 0 < int(router["top"]) <= keep * (outputs // count):
                raise ConfigError(f"Diforax config.json: {where}: top does not fit the kept groups")
        else:
            raise ConfigError(f"Diforax config.json: {where} has the unknown feed-forward {mlp['kind']!r} "
                              "(known: dense, moe)")

    def to_dict(self) -> dict:
        out = {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        out.update(self.extra)
        return out

    # ------------------------------------------------------------------ the model in parts
    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps

        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": W, "eps": eps}, {"weight": name})

        layers, unused = [], []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            m = layer["mixer"]
            if layer["type"] == "attention":
                shares = m.get("kv_from") is not None
                rot = m.get("rot")
                if rot is not None and int(rot["dims"]) > 0:
                    position = PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]),
                                                 "pairing": "half_split"})
                else:
                    position = PartSpec("no_position")
                tensors = {"q": prefix + "mix.q", "o": prefix + "mix.o"}
                if shares:
                    unused += [prefix + "mix.k", prefix + "mix.v"]
                else:
                    tensors.update({"k": prefix + "mix.k", "v": prefix + "mix.v"})
                mixer = PartSpec(
                    "gqa_attention",
                    {"hidden_size": W, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                     "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
                     "qk_norm_eps": None, "qk_unit_rms_eps": eps, "shares_cache": shares,
                     "chunk": int((m.get("mask") or {}).get("size") or 0), "position": position},
                    tensors)
            else:
                mixer = PartSpec(
                    "gated_delta_rule",
                    {"hidden_size": W, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
                     "dim": int(m["dim"]), "vdim": int(m["vdim"]), "taps": int(m["conv"]), "eps": eps},
                    {"q": prefix + "mix.q", "k": prefix + "mix.k", "v": prefix + "mix.v",
                     "q_conv": prefix + "mix.q.conv", "k_conv": prefix + "mix.k.conv",
                     "v_conv": prefix + "mix.v.conv", "b": prefix + "mix.b", "a": prefix + "mix.a",
                     "a_log": prefix + "mix.A_log", "dt_bias": prefix + "mix.dt_bias", "gate": prefix + "mix.g",
                     "norm": prefix + "mix.norm", "o": prefix + "mix.o"})
            parts = {"mixer_norm": norm(prefix + "norm1"), "mixer": mixer, "mixer_out_norm": norm(prefix + "norm1b")}
            mlp = layer.get("mlp")
            if mlp is None:
                unused += [prefix + "norm2", prefix + "norm2b"]
            else:
                parts["ffn_norm"] = norm(prefix + "norm2")
                parts["ffn_out_norm"] = norm(prefix + "norm2b")
                if mlp["kind"] == "dense":
                    parts["feed_forward"] = PartSpec(
                        "swiglu", {"hidden_size": W, "ffn_dim": int(mlp["ff"]), "activation": "gelu_tanh"},
                        {"gate": prefix + "mlp.gate", "up": prefix + "mlp.up", "down": prefix + "mlp.down"})
                else:
                    router = mlp["router"]
                    groups = router.get("groups") or {}
                    count = int(groups.get("count") or 1)
                    tensors = {"router": prefix + "mlp.router", "correction": prefix + "mlp.correction"}
                    for j in range(int(router["experts"])):
                        for role in ("gate", "up", "down"):
                            tensors[f"{role}{j}"] = f"{prefix}mlp.e{j}.{role}"
                    parts["feed_forward"] = PartSpec(
                        "routed_experts",
                        {"hidden_size": W, "ffn_dim": int(mlp["expert"]["ff"]), "experts": int(router["experts"]),
                         "identity": int(router.get("identity") or 0), "top": int(router["top"]), "groups": count,
                         "keep_groups": int(groups.get("keep") or count), "activation": "silu"},
                        tensors)
            layers.append(LayerSpec("sandwich_residual", parts=parts))
        spec = ModelSpec(
            architecture=self.architectures[0], hidden_size=W, vocab_size=self.vocab,
            max_positions=UNBOUNDED_POSITIONS, embedding_tensor="embed", final_norm=norm("final.norm"),
            head_tensor="head", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, cache_of=(layer["mixer"].get("kv_from")
                                                      if layer["type"] == "attention" else None))
                           for i, layer in enumerate(self.layers)),
            unused_tensors=tuple(unused))
        spec.validate()
        return spec
