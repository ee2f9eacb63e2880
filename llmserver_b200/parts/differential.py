"""Differential attention: every head attends with two score maps over the same values and subtracts one result
from the other."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import KVPagesNeed
from ..weights.declare import NORM, WIDE, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """Per head h (key/value head h // (heads / kv_heads)), with q and k of a head laid out as [map 1 | map 2]:

        q_m, k_m  <- rotate(rmsnorm(q_m) * w_q), rotate(rmsnorm(k_m) * w_k)        m = 1, 2; weights shared by all units
        a_m       = softmax(cap(q_m . k_m * scale)) V          cap(s) = softcap * tanh(s / softcap) when softcap is given
        lambda    = exp(lq1 . lk1) - exp(lq2 . lk2) + diff                          one number per layer
        o         = a_1 - lambda * a_2;  o <- o / sqrt(mean(o^2) + eps) * (1 - diff);  o <- o * sigmoid(W_g x)_h
        y         = W_o concat(o) + b_o

    (The subtraction of two softmax maps is the scheme of Ye et al., "Differential Transformer".)  A query at position
    p sees keys p - window + 1 .. p (``window`` None: every earlier key).  Both maps of a key head live in one cache row
    of 2 * dim elements, so the layer's cache is ``kv_heads`` key heads of 2 * dim and value heads of ``value_dim``.

    Parameters: ``hidden``, ``heads``, ``kv_heads``, ``dim`` (of one map), ``value_dim``, ``scale``, ``diff``, ``eps``;
    optional ``softcap``, ``window``, ``bias`` (q, k, v and o have biases), ``qk_norm`` (default True), ``gate`` (default
    True), ``names`` (pairs (role, tensor name behind the prefix); roles q, k, v, o, g, q_norm, k_norm, lq1, lk1, lq2,
    lk2; a bias is the tensor's name with ".b" added).  Rotation comes from the position encoding the layer names:
    ``inv_freq`` and ``rotary_dim`` (at most dim), paired as halves.

    Kernels: one product for q, k, v and the gate; ``norm_rope_units`` (bias, per-unit norm, rotation, cache write);
    ``attention_diff`` (both maps, the subtraction, the head norm and the gate); the output product, whose bias the
    next kernel on the stream adds (``output_bias``)."""

    KNOWN_PARAMS = ("hidden", "heads", "kv_heads", "dim", "value_dim", "scale", "diff", "eps", "softcap", "window", "bias",
                    "qk_norm", "gate", "names")
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm", "k_norm": "k.norm",
             "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"differential_attention has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def declare_weights(cls, params):
        hidden, heads, kv_heads = int(params["hidden"]), int(params["heads"]), int(params["kv_heads"])
        dim, value_dim = int(params["dim"]), int(params["value_dim"])
        name = cls.names(params)
        wanted = {name["q"]: WeightDecl((heads * 2 * dim, hidden)), name["k"]: WeightDecl((kv_heads * 2 * dim, hidden)),
                  name["v"]: WeightDecl((kv_heads * value_dim, hidden)), name["o"]: WeightDecl((hidden, heads * value_dim))}
        if params.get("bias"):
            for role in ("q", "k", "v", "o"):
                wanted[name[role] + ".b"] = WeightDecl((wanted[name[role]].shape[0],), WIDE)
        if params.get("qk_norm", True):
            wanted[name["q_norm"]] = WeightDecl((dim,), NORM)
            wanted[name["k_norm"]] = WeightDecl((dim,), NORM)
        if params.get("gate", True):
            wanted[name["g"]] = WeightDecl((heads, hidden))
        for role in ("lq1", "lk1", "lq2", "lk2"):
            wanted[name[role]] = WeightDecl((dim,), WIDE)
        return wanted

    @classmethod
    def cache_need(cls, params):
        return KVPagesNeed(int(params["kv_heads"]), 2 * int(params["dim"]), params.get("window"), int(params["value_dim"]))

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.kv_heads = int(params["heads"]), int(params["kv_heads"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads are no multiple of {self.kv_heads} kv heads")
        self.dim, self.value_dim = int(params["dim"]), int(params["value_dim"])
        self.scale, self.diff, self.eps = float(params["scale"]), float(params["diff"]), float(params["eps"])
        self.softcap = float(params.get("softcap") or 0.0)
        self.window = int(params["window"]) if params.get("window") else 0
        name = self.names(params)
        rows = [weights[name["q"]], weights[name["k"]], weights[name["v"]]]
        self.qkv_columns = sum(int(w.shape[0]) for w in rows)
        self.gate_column = None
        if params.get("gate", True):
            self.gate_column = self.qkv_columns
            rows.append(weights[name["g"]])
        total = sum(int(w.shape[0]) for w in rows)
        if total % 8:       # rows of the packed projection keep their 16-byte alignment
            rows.append(torch.zeros((8 - total % 8, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
        self.fused = torch.cat(rows, dim=0).contiguous()
        self.out = weights[name["o"]].contiguous()
        self.bias = self.output_bias = None
        if params.get("bias"):
            self.bias = torch.cat([weights[name[role] + ".b"].to(torch.float32) for role in ("q", "k", "v")]).contiguous()
            self.output_bias = weights[name["o"] + ".b"].to(torch.float32).contiguous()
        self.q_norm = weights[name["q_norm"]].contiguous() if params.get("qk_norm", True) else None
        self.k_norm = weights[name["k_norm"]].contiguous() if params.get("qk_norm", True) else None
        # one number per layer, made once from the stored values: exp(lq1 . lk1) - exp(lq2 . lk2) + diff
        wide = {role: weights[name[role]].to(torch.float64) for role in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = float(torch.exp((wide["lq1"] * wide["lk1"]).sum()) - torch.exp((wide["lq2"] * wide["lk2"]).sum())) + self.diff
        self.inv_freq, self.rotary_dim = None, 0

    def attach(self, position):
        if position is None:
            return
        inv_freq = getattr(position, "inv_freq", None)
        if inv_freq is None:
            raise ValueError(f"differential_attention rotates queries and keys: the position encoding "
                             f"{type(position).__name__} gives no inv_freq")
        rotary_dim = int(getattr(position, "rotary_dim", 2 * inv_freq.numel()))
        if rotary_dim != 2 * inv_freq.numel() or rotary_dim > self.dim or rotary_dim % 2:
            raise ValueError(f"the position encoding rotates {rotary_dim} elements; differential_attention needs an even "
                             f"rotary_dim of at most {self.dim}")
        if getattr(position, "pairing", "halves") != "halves" or float(getattr(position, "attention_factor", 1.0)) != 1.0:
            raise ValueError("differential_attention pairs rotated elements as halves and does not scale them")
        self.inv_freq, self.rotary_dim = inv_freq, rotary_dim

    def forward(self, x, batch, cache):
        tables = batch.block_tables[cache.group]
        qkv = ops.linear(x, self.fused)
        ops.norm_rope_units(qkv, batch.positions, batch.seq_of_token, tables, cache.k_pages, cache.v_pages, self.heads,
                            self.kv_heads, 2, self.dim, self.dim, self.value_dim, batch.error_flag, bias=self.bias,
                            q_weight=self.q_norm, k_weight=self.k_norm, eps=self.eps, inv_freq=self.inv_freq,
                            rotary_dim=self.rotary_dim, write_cache=cache.writes)
        attended = ops.attention_diff(qkv, self.gate_column, batch, tables, cache.k_pages, cache.v_pages, self.heads,
                                      self.kv_heads, self.dim, self.value_dim, self.scale, self.softcap, self.window, self.lam,
                                      self.eps, 1.0 - self.diff)
        return ops.linear(attended, self.out)
