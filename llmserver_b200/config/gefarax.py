"""Typed configuration of the Gefarax decoder, read from its own config.json keys.

Gefarax describes itself layer by layer: ``layers`` is a list whose entries give the kind of mixer (``type``), the
mixer's sizes and constants (``mixer``) and the feed-forward (``mlp``, or null for a layer without one); ``loop`` names
a run of layers that is executed several times in a row.  Nothing is assumed equal between layers.

    vocab, width, norm.eps
    layers[i].type            "attention"
    layers[i].mixer           heads, kv_heads, dim, vdim, scale,
                              rot: {base, dims, scaling: {factor, original, fast, slow} | null} | null
    layers[i].mlp             null | {kind: "moe", router: {experts, top, scale}, expert: {ff, limit},
                              shared: {ff, limit} | null}
    loop                      null | {start, stop, times}
"""
from __future__ import annotations

import copy
import json
import os
from dataclasses import dataclass, field
from typing import Optional, Tuple

from .errors import UnsupportedModelError

MIXER_TYPES = ("attention",)
FEED_FORWARD_KINDS = ("moe",)


def _need(where: str, raw: dict, *keys):
    if not isinstance(raw, dict):
        raise UnsupportedModelError(f"Gefarax config: {where} must be an object")
    missing = [key for key in keys if raw.get(key) is None]
    if missing:
        raise UnsupportedModelError(f"Gefarax config: {where} lacks {', '.join(missing)}")


@dataclass(frozen=True)
class GefaraxLayer:
    type: str
    mixer: dict
    mlp: Optional[dict]


@dataclass(frozen=True)
class GefaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[GefaraxLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_id: Tuple[int, ...] = ()
    architecture: str = "Gefarax"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def layer_runs(self):
        """(layer index, whether a new pass of the loop begins with this run) in the order the layers run: layers
        ``loop_start`` .. ``loop_stop`` - 1 are executed ``loop_times`` times in a row, every pass but the first
        beginning with the embedded tokens added to the stream."""
        runs = [(index, False) for index in range(self.loop_start)]
        for turn in range(self.loop_times):
            runs += [(index, turn > 0 and index == self.loop_start) for index in range(self.loop_start, self.loop_stop)]
        runs += [(index, False) for index in range(self.loop_stop, len(self.layers))]
        return runs

    # ---------------------------------------------------------------- parsing
    @classmethod
    def from_dict(cls, raw: dict) -> "GefaraxConfig":
        _need("config.json", raw, "vocab", "width", "layers", "norm")
        _need("norm", raw["norm"], "eps")
        if int(raw["vocab"]) <= 0 or int(raw["width"]) <= 0:
            raise UnsupportedModelError("Gefarax config: vocab and width must be positive")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise UnsupportedModelError("Gefarax config: layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(raw["layers"]):
            where = f"layers[{index}]"
            _need(where, entry, "type", "mixer")
            if entry["type"] not in MIXER_TYPES:
                raise UnsupportedModelError(f"Gefarax config: {where} has the unknown mixer type {entry['type']!r} "
                                            f"(known: {', '.join(MIXER_TYPES)})")
            mixer = entry["mixer"]
            _need(where + ".mixer", mixer, "heads", "kv_heads", "dim", "vdim", "scale")
            heads, kv_heads = int(mixer["heads"]), int(mixer["kv_heads"])
            if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
                raise UnsupportedModelError(f"Gefarax config: {where}: {heads} heads are no multiple of {kv_heads} kv_heads")
            rot = mixer.get("rot")
            if rot:
                _need(where + ".mixer.rot", rot, "base", "dims")
                if int(rot["dims"]) % 2 or not 0 < int(rot["dims"]) <= int(mixer["dim"]):
                    raise UnsupportedModelError(f"Gefarax config: {where}: rot.dims must be even and at most dim")
                if rot.get("scaling"):
                    _need(where + ".mixer.rot.scaling", rot["scaling"], "factor", "original", "fast", "slow")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(where + ".mlp", mlp, "router", "expert")
                if mlp.get("kind", "moe") not in FEED_FORWARD_KINDS:
                    raise UnsupportedModelError(f"Gefarax config: {where}.mlp has the unknown kind {mlp.get('kind')!r} "
                                                f"(known: {', '.join(FEED_FORWARD_KINDS)})")
                _need(where + ".mlp.router", mlp["router"], "experts", "top", "scale")
                _need(where + ".mlp.expert", mlp["expert"], "ff", "limit")
                if not 0 < int(mlp["router"]["top"]) <= int(mlp["router"]["experts"]):
                    raise UnsupportedModelError(f"Gefarax config: {where}.mlp.router: top must lie in 1..experts")
                if mlp.get("shared"):
                    _need(where + ".mlp.shared", mlp["shared"], "ff", "limit")
            layers.append(GefaraxLayer(entry["type"], copy.deepcopy(mixer), copy.deepcopy(mlp)))
        loop = raw.get("loop")
        start = stop = 0
        times = 1
        if loop:
            _need("loop", loop, "start", "stop", "times")
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not 0 <= start <= stop <= len(layers) or times < 1:
                raise UnsupportedModelError(f"Gefarax config: loop {loop} does not fit {len(layers)} layers")
        eos = raw.get("eos_token_id")
        eos = () if eos is None else ((int(eos),) if isinstance(eos, int) else tuple(int(e) for e in eos))
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "loop", "eos_token_id"}
        return cls(vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times, eos_token_id=eos,
                   extra={key: value for key, value in raw.items() if key not in known})

    @classmethod
    def from_json_file(cls, path: str) -> "GefaraxConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as handle:
            return cls.from_dict(json.load(handle))

    def to_dict(self) -> dict:
        """config.json form (round-trips through ``from_dict``)."""
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": layer.type, "mixer": copy.deepcopy(layer.mixer), "mlp": copy.deepcopy(layer.mlp)}
                          for layer in self.layers],
               "loop": ({"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
                        if self.loop_stop > self.loop_start and self.loop_times > 1 else None)}
        if self.eos_token_id:
            out["eos_token_id"] = list(self.eos_token_id)
        return out
