"""Latent attention: keys and values are made from one small latent per token, which is all the cache holds."""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import KVPagesNeed
from ..weights.declare import NORM, WeightDecl
from .base import Mixer
from .registry import MIXERS


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Queries through a latent of ``q_rank``, keys and values from a latent of ``kv_rank`` (the low-rank scheme of
    DeepSeek-AI, "DeepSeek-V2: A Strong, Economical, and Efficient Mixture-of-Experts Language Model", here without a
    rotated part):

        c_q = rmsnorm(W_dq x) * w_dq,   q = W_uq c_q                      [heads, dim]
        c   = rmsnorm(W_dkv x) * w_dkv                                    [kv_rank]      the only thing cached
        k   = W_uk c,  v = W_uv c                                         [heads, dim], [heads, value_dim]
        y   = W_o concat_h(softmax_j(q_h . k_h,j * scale) v_h,j)          causal, every earlier key

    The engine never forms k and v: q_h . (W_uk,h c_j) = (W_uk,h^T q_h) . c_j and sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j,
    so the latents are read as ONE key/value head of ``kv_rank`` that all query heads share, keys and values being the
    same tensor (``KVPagesNeed(keys_only=True)``); queries are carried into the latent space head by head in front of the
    attention kernel and the attended latents out of it behind (``ops.head_linear``).

    Parameters: ``hidden``, ``heads``, ``dim``, ``value_dim``, ``q_rank``, ``kv_rank``, ``scale``, ``eps``; ``names``:
    pairs (role, tensor name behind the prefix) for dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o."""

    KNOWN_PARAMS = ("hidden", "heads", "dim", "value_dim", "q_rank", "kv_rank", "scale", "eps", "names")
    NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv",
             "o": "o"}

    @classmethod
    def names(cls, params) -> dict:
        given = dict(params.get("names") or ())
        unknown = sorted(set(given) - set(cls.NAMES))
        if unknown:
            raise ValueError(f"latent_attention has no tensor in the role(s) {', '.join(unknown)}")
        return {**cls.NAMES, **given}

    @classmethod
    def declare_weights(cls, params):
        hidden, heads, dim, value_dim = int(params["hidden"]), int(params["heads"]), int(params["dim"]), int(params["value_dim"])
        q_rank, kv_rank = int(params["q_rank"]), int(params["kv_rank"])
        name = cls.names(params)
        return {name["dq"]: WeightDecl((q_rank, hidden)), name["dq_norm"]: WeightDecl((q_rank,), NORM),
                name["uq"]: WeightDecl((heads * dim, q_rank)), name["dkv"]: WeightDecl((kv_rank, hidden)),
                name["dkv_norm"]: WeightDecl((kv_rank,), NORM), name["uk"]: WeightDecl((heads * dim, kv_rank)),
                name["uv"]: WeightDecl((heads * value_dim, kv_rank)), name["o"]: WeightDecl((hidden, heads * value_dim))}

    @classmethod
    def cache_need(cls, params):
        return KVPagesNeed(1, int(params["kv_rank"]), None, None, keys_only=True)

    def __init__(self, params, weights, runtime):
        super().__init__(params, weights, runtime)
        self.heads, self.dim, self.value_dim = int(params["heads"]), int(params["dim"]), int(params["value_dim"])
        self.q_rank, self.kv_rank = int(params["q_rank"]), int(params["kv_rank"])
        self.scale, self.eps = float(params["scale"]), float(params["eps"])
        name = self.names(params)
        self.down = torch.cat([weights[name["dq"]], weights[name["dkv"]]], dim=0).contiguous()
        self.q_norm, self.c_norm = weights[name["dq_norm"]].contiguous(), weights[name["dkv_norm"]].contiguous()
        if self.q_norm.dtype != self.c_norm.dtype:
            self.q_norm, self.c_norm = self.q_norm.to(torch.float32), self.c_norm.to(torch.float32)
        self.up_q = weights[name["uq"]].contiguous()
        # per head: the transposed key matrix [kv_rank, dim], which carries a query into the latent space, and the value
        # matrix [value_dim, kv_rank], which carries an attended latent out of it
        self.key_in = weights[name["uk"]].view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.value_out = weights[name["uv"]].view(self.heads, self.value_dim, self.kv_rank).contiguous()
        self.out = weights[name["o"]].contiguous()

    def forward(self, x, batch, cache):
        tables = batch.block_tables[cache.group]
        down = ops.linear(x, self.down)
        c_q = torch.empty((x.shape[0], self.q_rank), dtype=x.dtype, device=x.device)
        ops.norm_rope_units(down, batch.positions, batch.seq_of_token, tables, cache.k_pages, None, 1, 1, 1, self.q_rank,
                            self.kv_rank, 0, batch.error_flag, q_weight=self.q_norm, k_weight=self.c_norm, eps=self.eps,
                            q_out=c_q, write_cache=cache.writes)
        q = ops.head_linear(ops.linear(c_q, self.up_q), self.key_in)
        attended = ops.attention(q, batch, tables, cache.k_pages, cache.v_pages, self.heads, 1, self.kv_rank, self.scale,
                                 precise=True, q_stride=self.heads * self.kv_rank)
        return ops.linear(ops.head_linear(attended, self.value_out), self.out)
