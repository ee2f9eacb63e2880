"""Dikusun: from its typed configuration to the architecture-neutral model specification.

This is the only place that knows how Dikusun arranges its parts and names its tensors.  Every layer normalises the
output of each sub-layer and lets the sub-layers read the stream as it is (``output_norm``); its mixer is differential
attention over a sliding window (``differential_attention``), attention through low-rank latents (``latent_attention``)
or gated linear attention (``gated_linear_attention``); its feed-forward, where it has one, is a dense gated layer with
clamped gate and up values (``clamped_glu``).  The embedded tokens are scaled as they enter the stream.  A layer that
names another layer's weights is a further schedule entry of that layer, with a cache or state of its own.

Tensors: ``embed``, ``head``, ``final.norm``; layer i: ``l<i>.norm1`` (behind the mixer), ``l<i>.norm2`` (behind the
feed-forward), ``l<i>.mix.*``, ``l<i>.mlp.gate`` / ``.up`` / ``.down``.
"""
from __future__ import annotations

from ..config.dikusun import DikusunConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _position_of(mixer: dict, positions: dict):
    """Name of the position encoding this mixer uses (made on first use; equal constants share one)."""
    rot = mixer.get("rot")
    if not rot:
        return None
    part = PartSpec.of("rotary", head_dim=int(mixer["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]))
    for name, known in positions.items():
        if known == part:
            return name
    name = f"rot{len(positions)}"
    positions[name] = part
    return name


def _mixer_of(kind: str, mixer: dict, config: DikusunConfig) -> PartSpec:
    if kind == "attention":
        mask = mixer.get("mask") or {}
        return PartSpec.of("differential_attention", hidden=config.width, heads=int(mixer["heads"]), kv_heads=int(mixer["kv_heads"]),
                           dim=int(mixer["dim"]), value_dim=int(mixer["vdim"]), scale=float(mixer["scale"]),
                           diff=float(mixer["diff"]), eps=config.norm_eps, softcap=float(mixer.get("softcap") or 0.0),
                           window=int(mask["size"]) if mask.get("size") else None, bias=True)
    if kind == "latent_attention":
        return PartSpec.of("latent_attention", hidden=config.width, heads=int(mixer["heads"]), dim=int(mixer["dim"]),
                           value_dim=int(mixer["vdim"]), q_rank=int(mixer["q_rank"]), kv_rank=int(mixer["kv_rank"]),
                           scale=float(mixer["scale"]), eps=config.norm_eps)
    # the rank of the decay's first projection is given by its tensor's shape; a configuration may name it ("a_rank")
    # for models whose weights are made rather than read
    rank = mixer.get("a_rank")
    return PartSpec.of("gated_linear_attention", hidden=config.width, heads=int(mixer["heads"]), dim=int(mixer["dim"]),
                       value_dim=int(mixer["vdim"]), tau=float(mixer["tau"]), decay_rank=int(rank) if rank else None,
                       eps=config.norm_eps)


def dikusun_spec(config: DikusunConfig) -> ModelSpec:
    def norm():
        return PartSpec.of("rmsnorm", width=config.width, eps=config.norm_eps, tensor="")

    positions, layers, spec_index = {}, [], {}
    for index, layer in enumerate(config.layers):
        if layer.weights_of is not None:
            continue
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec.of("clamped_glu", hidden=config.width, intermediate=int(layer.mlp["ff"]),
                                       limit=float(layer.mlp["limit"]))
        block = PartSpec.of("output_norm", feed_forward=feed_forward is not None, mixer_prefix="mix.", feed_forward_prefix="mlp.",
                            mixer_out_norm_prefix="norm1", feed_forward_out_norm_prefix="norm2")
        extra = (("mixer_out_norm", norm()),) + ((("feed_forward_out_norm", norm()),) if feed_forward is not None else ())
        spec_index[index] = len(layers)
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=_mixer_of(layer.type, layer.mixer, config),
                                feed_forward=feed_forward, position=_position_of(layer.mixer, positions) if layer.type == "attention" else None,
                                extra=extra))
    schedule = [ScheduleEntry(spec_index[config.owner_of(index)]) for index in range(len(config.layers))]
    return ModelSpec(architecture=config.architecture, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                     schedule=schedule, positions=positions, final_norm=norm(), embedding_name="embed",
                     final_norm_prefix="final.norm", head_name="head", tie_head=False, embedding_scale=config.embedding_scale,
                     eos_token_ids=config.eos_token_id)


register_architecture("Dikusun", DikusunConfig, dikusun_spec)
