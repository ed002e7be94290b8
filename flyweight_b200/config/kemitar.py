"""Typed configuration of Kemitar: a decoder whose layers put a gain-only RMS norm on each
sublayer's output, shift tokens in front of the mixer, attend over a cached low-rank latent with a
softmax sink, and whose embedding adds a hashed table of token pairs.

``config.json`` keys: ``architecture`` ("Kemitar"), ``vocab``, ``width``, ``norm.eps``,
``embedding.scale``, ``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``) and ``layers``, a
list whose entries give ``type`` (the mixer), ``mixer`` (its sizes and constants) and ``mlp``
(``{"kind": "dense", "ff": F}`` or null).  A mixer of type ``latent_attention`` has ``heads``,
``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``scale``, ``rot`` (``base``, ``dims``) and optionally
``kv_from``: the index of an earlier layer whose cached rows it reads instead of projecting its own.
Every size and constant comes from there; the file states no context limit, so the engine's own
limit (its page pool) is the only one.

Tensor names: ``embed``, ``bigram``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.shift``, ``l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}``, ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# config.json names no longest sequence; positions are bounded by the engine's cache alone
UNBOUNDED_POSITIONS = 1 << 24


def _need(mapping: Mapping[str, Any], keys, where: str) -> None:
    if not isinstance(mapping, Mapping):
        raise ConfigError(f"Kemitar config.json: {where} must be an object")
    missing = [key for key in keys if mapping.get(key) is None]
    if missing:
        raise ConfigError(f"Kemitar config.json: {where} is missing " + ", ".join(missing))


@dataclass(frozen=True)
class KemitarConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    bigram: Optional[Mapping[str, int]]           # buckets, mul_prev, mul_cur (None: no pair table)
    layers: Tuple[Mapping[str, Any], ...]         # as config.json gives them, checked
    architectures: Tuple[str, ...] = ("Kemitar",)
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ reading / writing
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KemitarConfig":
        _need(raw, ("vocab", "width", "norm", "embedding", "layers"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
        _need(raw["embedding"], ("scale",), "'embedding'")
        bigram = raw["embedding"].get("bigram")
        if bigram is not None:
            _need(bigram, ("buckets", "mul_prev", "mul_cur"), "'embedding.bigram'")
            bigram = {key: int(bigram[key]) for key in ("buckets", "mul_prev", "mul_cur")}
            if bigram["buckets"] <= 0:
                raise ConfigError("Kemitar config.json: embedding.bigram.buckets must be positive")
        if not isinstance(raw["layers"], (list, tuple)) or not raw["layers"]:
            raise ConfigError("Kemitar config.json: 'layers' must be a list with at least one layer")
        layers = []
        for index, layer in enumerate(raw["layers"]):
            where = f"layer {index}"
            _need(layer, ("type", "mixer"), where)
            if layer["type"] != "latent_attention":
                raise ConfigError(f"Kemitar config.json: {where} has the unknown type {layer['type']!r} "
                                  "(known: latent_attention)")
            layer = copy.deepcopy(dict(layer))
            mixer = layer["mixer"]
            given = mixer.get("kv_from") if isinstance(mixer, Mapping) else None
            if isinstance(given, int) and 0 <= given < index:
                # what a layer that reads another's rows does not state about them is the source's
                for key in ("kv_rank", "rot_dim", "rot"):
                    if mixer.get(key) is None and layers[given]["mixer"].get(key) is not None:
                        mixer[key] = copy.deepcopy(layers[given]["mixer"][key])
            _need(mixer, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), f"{where}'s mixer")
            _need(mixer["rot"], ("base", "dims"), f"{where}'s mixer.rot")
            if int(mixer["rot"]["dims"]) > int(mixer["rot_dim"]) or int(mixer["rot"]["dims"]) % 2:
                raise ConfigError(f"Kemitar config.json: {where}: rot.dims must be even and at most rot_dim")
            source = mixer.get("kv_from")
            if source is not None:
                source = int(source)
                if not 0 <= source < index or layers[source]["mixer"].get("kv_from") is not None:
                    raise ConfigError(f"Kemitar config.json: {where} reads the cache of layer {source}, which "
                                      "is no earlier layer with a cache of its own")
                theirs = layers[source]["mixer"]
                if any(theirs[key] != mixer[key] for key in ("kv_rank", "rot_dim", "rot")):
                    raise ConfigError(f"Kemitar config.json: {where} and layer {source} must agree on "
                                      "kv_rank, rot_dim and rot")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind", "ff"), f"{where}'s mlp")
                if mlp["kind"] != "dense":
                    raise ConfigError(f"Kemitar config.json: {where} has the unknown feed-forward "
                                      f"{mlp['kind']!r} (known: dense)")
            layers.append(layer)
        known = {"architecture", "architectures", "vocab", "width", "norm", "embedding", "layers"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float(raw["embedding"]["scale"]), bigram=bigram, layers=tuple(layers),
                   extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        embedding: dict = {"scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = dict(self.bigram)
        out = {"architecture": self.architectures[0], "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": embedding,
               "layers": copy.deepcopy(list(self.layers))}
        out.update(self.extra)
        return out

    # ------------------------------------------------------------------ the model in parts
    def model_spec(self) -> ModelSpec:
        W, eps = self.width, self.norm_eps

        def gain_norm(name: str) -> PartSpec:
            return PartSpec("rms_gain", {"size": W, "eps": eps}, {"weight": name})

        layers = []
        unused = [] if self.bigram is not None else ["bigram"]
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}."
            m = layer["mixer"]
            shares = m.get("kv_from") is not None
            # a checkpoint may carry a left-out sublayer's tensors all the same; they are passed over
            if shares:
                unused += [prefix + "mix.dkv", prefix + "mix.dkv.norm"]
            if layer.get("mlp") is None:
                unused += [prefix + name for name in ("norm2", "mlp.gate", "mlp.up", "mlp.down")]
            tensors = {"q": prefix + "mix.q", "uk": prefix + "mix.uk", "uv": prefix + "mix.uv",
                       "o": prefix + "mix.o", "sink": prefix + "mix.sink"}
            if not shares:
                tensors.update({"dkv": prefix + "mix.dkv", "dkv_norm": prefix + "mix.dkv.norm"})
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": W, "num_heads": int(m["heads"]), "dim": int(m["dim"]),
                 "rot_dim": int(m["rot_dim"]), "vdim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]),
                 "scale": float(m["scale"]), "eps": eps, "sink": True, "shares_cache": shares,
                 "position": PartSpec("rope", {"theta": float(m["rot"]["base"]),
                                               "rotary_dim": int(m["rot"]["dims"]),
                                               "pairing": "half_split"})},
                tensors)
            parts = {"shift": PartSpec("token_shift", {"size": W}, {"weight": prefix + "shift"}),
                     "mixer": mixer, "mixer_out_norm": gain_norm(prefix + "norm1")}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = PartSpec(
                    "swiglu", {"hidden_size": W, "ffn_dim": int(layer["mlp"]["ff"])},
                    {"gate": prefix + "mlp.gate", "up": prefix + "mlp.up", "down": prefix + "mlp.down"})
                parts["ffn_out_norm"] = gain_norm(prefix + "norm2")
            layers.append(LayerSpec("outnorm_residual", parts=parts))
        embedding = None
        if self.bigram is not None:
            embedding = PartSpec("hashed_pairs", {"hidden_size": W, "scale": self.embedding_scale,
                                                  **self.bigram}, {"pairs": "bigram"})
        spec = ModelSpec(
            architecture=self.architectures[0], hidden_size=W, vocab_size=self.vocab,
            max_positions=UNBOUNDED_POSITIONS, embedding_tensor="embed", final_norm=gain_norm("final.norm"),
            head_tensor="head", layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i, cache_of=layer["mixer"].get("kv_from"))
                           for i, layer in enumerate(self.layers)),
            embedding_scale=self.embedding_scale, embedding=embedding, unused_tensors=tuple(unused))
        spec.validate()
        return spec
