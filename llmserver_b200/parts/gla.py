"""Gated linear attention: a matrix-valued state per head that decays channel by channel."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.declare import NORM, WIDE, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Per head, with S in R^(dim x value_dim) starting at zero for every request (the recurrence of Yang et al.,
    "Gated Linear Attention Transformers with Hardware-Efficient Training"):

        q = W_q x * dim^(-1/2),  k = W_k x,  v = W_v x
        alpha = sigmoid(W_a2 (W_a1 x) + b_a2) ^ (1 / tau)                    one decay per key channel
        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
        y = W_o (concat_h(rmsnorm(o_h) * w) * silu(W_g x))                   w of value_dim, shared by the heads

    The state is float32 [heads, dim, value_dim] in the request's state slot; the decay (from the 32-bit sums of its
    second projection on) and the recurrence are 32-bit in either path; the other projections run in the activation type.  Parameters: ``hidden``,
    ``heads``, ``dim``, ``value_dim``, ``tau``, ``decay_rank`` (rows of W_a1; None: the tensor's shape says), ``eps``; ``names``: pairs (role, tensor
    name behind the prefix) for q, k, v, g, o, norm, a1, a2 (the bias is a2's name with ".b" added)."""

    KNOWN_PARAMS = ("hidden", "heads", "dim", "value_dim", "tau", "decay_rank", "eps", "names")
    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2"}

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"gated_linear_attention has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def check_params(cls, params):
        super().check_params(params)
        if float(params["tau"]) <= 0:
            raise ValueError("gated_linear_attention: tau must be positive")

    @classmethod
    def declare_weights(cls, params):
        hidden, heads, dim, value_dim = int(params["hidden"]), int(params["heads"]), int(params["dim"]), int(params["value_dim"])
        rank = int(params["decay_rank"]) if params.get("decay_rank") else -1      # -1: whatever the checkpoint holds
        name = cls.names(params)
        return {name["q"]: WeightDecl((heads * dim, hidden)), name["k"]: WeightDecl((heads * dim, hidden)),
                name["v"]: WeightDecl((heads * value_dim, hidden)), name["g"]: WeightDecl((heads * value_dim, hidden)),
                name["o"]: WeightDecl((hidden, heads * value_dim)), name["norm"]: WeightDecl((value_dim,), NORM),
                name["a1"]: WeightDecl((rank, hidden)), name["a2"]: WeightDecl((heads * dim, rank)),
                name["a2"] + ".b": WeightDecl((heads * dim,), WIDE)}

    @classmethod
    def cache_need(cls, params):
        return StateNeed((int(params["heads"]), int(params["dim"]), int(params["value_dim"])), "float32")

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.dim, self.value_dim = int(params["heads"]), int(params["dim"]), int(params["value_dim"])
        self.tau, self.eps = float(params["tau"]), float(params["eps"])
        if not ops.gla_supported(self.dim, self.value_dim):
            raise ValueError(f"gated_linear_attention: no kernel for heads of {self.dim} key and {self.value_dim} value channels")
        name = self.names(params)
        self.fused = torch.cat([weights[name[role]] for role in ("q", "k", "v", "g")], dim=0).contiguous()
        keys, values = self.heads * self.dim, self.heads * self.value_dim
        self.columns = (0, keys, 2 * keys, 2 * keys + values)
        self.decay_in, self.decay_out = weights[name["a1"]].contiguous(), weights[name["a2"]].contiguous()
        self.decay_bias = weights[name["a2"] + ".b"].to(torch.float32).contiguous()
        self.norm = weights[name["norm"]].contiguous()
        self.out = weights[name["o"]].contiguous()

    def forward(self, x, batch, cache):
        proj = ops.linear(x, self.fused)
        z = ops.linear_wide(ops.linear(x, self.decay_in), self.decay_out)      # 32-bit sums, never rounded to the activation type
        q_column, k_column, v_column, g_column = self.columns
        mixed = ops.gla_recurrent(proj, q_column, k_column, v_column, g_column, z, self.decay_bias, self.norm, cache.state,
                                  batch, self.heads, self.dim, self.value_dim, self.tau, self.dim ** -0.5, self.eps)
        return ops.linear(mixed, self.out)
