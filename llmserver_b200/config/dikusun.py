"""Typed configuration of the Dikusun decoder, read from its own config.json keys.

Dikusun describes itself layer by layer; a layer has one of three mixers and, optionally, a dense gated feed-forward.
A layer may name another layer whose tensors it uses (``weights_of``): it then runs with that layer's weights and a
cache or state of its own.  Nothing is assumed equal between layers.

    vocab, width, norm.eps, embedding.scale
    layers[i].type            "attention" | "latent_attention" | "gla"
    layers[i].mixer           attention:         heads, kv_heads, dim, vdim, scale, diff, softcap | null,
                                                 mask: {size} | null, rot: {base, dims} | null
                              latent_attention:  heads, dim, vdim, q_rank, kv_rank, scale
                              gla:               heads, dim, vdim, tau  (a_rank: optional, else the tensor's shape says)
    layers[i].mlp             null | {kind: "dense", ff, limit}
    layers[i].weights_of      absent | index of the layer whose tensors this one uses
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .errors import UnsupportedModelError

MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "diff"),
    "latent_attention": ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale"),
    "gla": ("heads", "dim", "vdim", "tau"),
}
FEED_FORWARD_KINDS = ("dense",)


def _need(where: str, raw, *keys):
    if not isinstance(raw, dict):
        raise UnsupportedModelError(f"Dikusun config: {where} must be an object")
    missing = [key for key in keys if raw.get(key) is None]
    if missing:
        raise UnsupportedModelError(f"Dikusun config: {where} lacks {', '.join(missing)}")


@dataclass(frozen=True)
class DikusunLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class DikusunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[DikusunLayer, ...]
    eos_token_id: Tuple[int, ...] = ()
    architecture: str = "Dikusun"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def owner_of(self, index: int) -> int:
        """The layer whose tensors layer ``index`` uses (itself, unless it names another)."""
        named = self.layers[index].weights_of
        return index if named is None else named

    # ---------------------------------------------------------------- parsing
    @classmethod
    def from_dict(cls, raw: dict) -> "DikusunConfig":
        _need("config.json", raw, "vocab", "width", "layers", "norm")
        _need("norm", raw["norm"], "eps")
        if int(raw["vocab"]) <= 0 or int(raw["width"]) <= 0:
            raise UnsupportedModelError("Dikusun config: vocab and width must be positive")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise UnsupportedModelError("Dikusun config: layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(raw["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, "type", "mixer")
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise UnsupportedModelError(f"Dikusun config: {where} has the unknown mixer type {kind!r} "
                                            f"(known: {', '.join(sorted(MIXER_KEYS))})")
            mixer = entry["mixer"]
            _need(where + ".mixer", mixer, *MIXER_KEYS[kind])
            for key in ("heads", "dim", "vdim"):
                if int(mixer[key]) <= 0:
                    raise UnsupportedModelError(f"Dikusun config: {where}.mixer.{key} must be positive")
            if kind == "attention":
                heads, kv_heads = int(mixer["heads"]), int(mixer["kv_heads"])
                if kv_heads <= 0 or heads % kv_heads:
                    raise UnsupportedModelError(f"Dikusun config: {where}: {heads} heads are no multiple of {kv_heads} kv_heads")
                rot = mixer.get("rot")
                if rot:
                    _need(where + ".mixer.rot", rot, "base", "dims")
                    if int(rot["dims"]) % 2 or not 0 < int(rot["dims"]) <= int(mixer["dim"]):
                        raise UnsupportedModelError(f"Dikusun config: {where}: rot.dims must be even and at most dim")
                mask = mixer.get("mask")
                if mask:
                    _need(where + ".mixer.mask", mask, "size")
                    if int(mask["size"]) <= 0:
                        raise UnsupportedModelError(f"Dikusun config: {where}: mask.size must be positive")
                if not 0.0 <= float(mixer["diff"]) < 1.0:
                    raise UnsupportedModelError(f"Dikusun config: {where}: diff must lie in [0, 1)")
            elif kind == "latent_attention":
                if int(mixer["q_rank"]) <= 0 or int(mixer["kv_rank"]) <= 0:
                    raise UnsupportedModelError(f"Dikusun config: {where}: q_rank and kv_rank must be positive")
            elif float(mixer["tau"]) <= 0:
                raise UnsupportedModelError(f"Dikusun config: {where}: tau must be positive")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind", "dense") not in FEED_FORWARD_KINDS:
                    raise UnsupportedModelError(f"Dikusun config: {where}.mlp has the unknown kind {mlp.get('kind')!r} "
                                                f"(known: {', '.join(FEED_FORWARD_KINDS)})")
                _need(where + ".mlp", mlp, "ff", "limit")
            named = entry.get("weights_of")
            if named is not None:
                named = int(named)
                if not 0 <= named < len(raw["layers"]) or named == index:
                    raise UnsupportedModelError(f"Dikusun config: {where}.weights_of names layer {named}, which is not another layer")
            layers.append(DikusunLayer(kind, copy.deepcopy(mixer), copy.deepcopy(mlp), named))
        for index, layer in enumerate(layers):
            if layer.weights_of is not None:
                owner = layers[layer.weights_of]
                if owner.weights_of is not None:
                    raise UnsupportedModelError(f"Dikusun config: layers[{index}] uses the weights of layer {layer.weights_of}, "
                                                "which has none of its own")
                if owner.type != layer.type:
                    raise UnsupportedModelError(f"Dikusun config: layers[{index}] uses the weights of layer {layer.weights_of}, "
                                                f"a {owner.type} layer, but calls itself {layer.type}")
        embedding = raw.get("embedding") or {}
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "embedding", "eos_token_id"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   embedding_scale=float(embedding.get("scale", 1.0)), layers=tuple(layers), eos_token_id=eos,
                   extra={key: value for key, value in raw.items() if key not in known})

    @classmethod
    def from_json_file(cls, path: str) -> "DikusunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as handle:
            return cls.from_dict(json.load(handle))

    def to_dict(self) -> dict:
        """config.json form (round-trips through ``from_dict``)."""
        layers = []
        for layer in self.layers:
            entry = {"type": layer.type, "mixer": copy.deepcopy(layer.mixer), "mlp": copy.deepcopy(layer.mlp)}
            if layer.weights_of is not None:
                entry["weights_of"] = layer.weights_of
            layers.append(entry)
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
