"""Gefarax: from its typed configuration to the architecture-neutral model specification.

This is the only place that knows how Gefarax arranges its parts and names its tensors.  Every layer has a norm in
front of and behind each sub-layer (``sandwich_norm``); its mixer is grouped-query attention whose values may have
another size than its keys, with a learned sink per head in the softmax and rotary positions on the first ``rot.dims``
elements of a head, stretched for long contexts (``stretched_rotary``); its feed-forward, where it has one, is a routed
mixture of clamped gated experts with a shared expert (``routed_experts``).  A run of layers may be executed several
times with the same weights: each execution is a schedule entry with a cache of its own, and every pass but the first
starts by adding the embedded tokens to the stream again.

Tensors: ``embed``, ``head``, ``final.norm``; layer i: ``l<i>.norm1``, ``.norm1b`` (around the mixer), ``.norm2``,
``.norm2b`` (around the feed-forward), ``.mix.q`` / ``.k`` / ``.v`` / ``.o`` / ``.sink``, ``.mlp.*``.
"""
from __future__ import annotations

from ..config.gefarax import GefaraxConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("sinks", "sink"))


def _position_of(mixer: dict, positions: dict):
    """Name of the position encoding this mixer uses (made on first use; equal constants share one)."""
    rot = mixer.get("rot")
    if not rot:
        return None
    scaling = rot.get("scaling")
    if scaling:
        part = PartSpec.of("stretched_rotary", head_dim=int(mixer["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]),
                           factor=float(scaling["factor"]), original=float(scaling["original"]),
                           fast=float(scaling["fast"]), slow=float(scaling["slow"]))
    else:
        part = PartSpec.of("rotary", head_dim=int(mixer["dim"]), theta=float(rot["base"]), rotary_dim=int(rot["dims"]))
    for name, known in positions.items():
        if known == part:
            return name
    name = f"rot{len(positions)}"
    positions[name] = part
    return name


def gefarax_spec(config: GefaraxConfig) -> ModelSpec:
    def norm(prefix_is_name: bool = True):
        return PartSpec.of("rmsnorm", width=config.width, eps=config.norm_eps, tensor="")

    positions, layers = {}, []
    for index, layer in enumerate(config.layers):
        mixer = layer.mixer
        attention = PartSpec.of("gqa_attention", hidden=config.width, heads=int(mixer["heads"]), kv_heads=int(mixer["kv_heads"]),
                                head_dim=int(mixer["dim"]), value_dim=int(mixer["vdim"]), scale=float(mixer["scale"]),
                                sinks=True, precise_weights=True, names=ATTENTION_NAMES)
        feed_forward = None
        if layer.mlp is not None:
            mlp = layer.mlp
            shared = mlp.get("shared") or {}
            extras = {"shared_intermediate": int(shared["ff"]), "shared_limit": float(shared["limit"])} if shared else {}
            feed_forward = PartSpec.of("routed_experts", hidden=config.width, experts=int(mlp["router"]["experts"]),
                                       top=int(mlp["router"]["top"]), route_scale=float(mlp["router"]["scale"]),
                                       intermediate=int(mlp["expert"]["ff"]), limit=float(mlp["expert"]["limit"]), **extras)
        block = PartSpec.of("sandwich_norm", feed_forward=feed_forward is not None, mixer_prefix="mix.", feed_forward_prefix="mlp.",
                            mixer_norm_prefix="norm1", mixer_out_norm_prefix="norm1b", feed_forward_norm_prefix="norm2",
                            feed_forward_out_norm_prefix="norm2b")
        extra = (("mixer_out_norm", norm()),) + ((("feed_forward_out_norm", norm()),) if feed_forward is not None else ())
        layers.append(LayerSpec(prefix=f"l{index}.", block=block, mixer=attention, feed_forward=feed_forward,
                                mixer_norm=norm(), feed_forward_norm=norm() if feed_forward is not None else None,
                                position=_position_of(mixer, positions), extra=extra))
    schedule = [ScheduleEntry(index, add_embedding=again) for index, again in config.layer_runs()]
    return ModelSpec(architecture=config.architecture, vocab_size=config.vocab, hidden_size=config.width, layers=layers,
                     schedule=schedule, positions=positions, final_norm=norm(), embedding_name="embed",
                     final_norm_prefix="final.norm", head_name="head", tie_head=False, eos_token_ids=config.eos_token_id)


register_architecture("Gefarax", GefaraxConfig, gefarax_spec)
