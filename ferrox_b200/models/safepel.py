"""Safepel as a description made of parts.

A decoder whose layers alternate, in whatever order ``config.json`` lists them, between two mixers that keep a
matrix state per head (a gated delta rule, and a decayed linear attention that runs beside a windowed soft-capped
attention whose values are its unrotated keys).  Per layer, with layer norms (weight, no bias) on both sides of
each sublayer:

    h += post1(mixer(norm1(h)));   h += post2(ffn(norm2(h)))        ffn = down(relu(gate x) * (up x)), or none

The embedding rows are normed before the first layer; the logits are the head's product times ``logit_scale``.
Tensor names: ``embed``, ``embed.norm``, ``l<i>.{norm1,norm1b,norm2,norm2b}``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.safepel import ARCHITECTURE, DeltaMixerConfig, ParallelMixerConfig, SafepelConfig
from ..parts.specs import (
    AdjacentRotarySpec,
    AttentionSpec,
    DecayedLinearAttentionSpec,
    DenseMlpSpec,
    GatedDeltaSpec,
    LayerNormSpec,
    MixerSumSpec,
    ModelSpec,
    SandwichBlockSpec,
    ScheduleEntry,
)


def _mixer(cfg: SafepelConfig, m, prefix: str):
    W, eps = cfg.width, cfg.norm_eps
    if isinstance(m, DeltaMixerConfig):
        return GatedDeltaSpec(hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                              conv_taps=m.conv, norm_eps=eps, prefix=prefix)
    assert isinstance(m, ParallelMixerConfig)
    l, r = m.left, m.right
    left = AttentionSpec(
        hidden=W, n_heads=l.heads, n_kv_heads=l.kv_heads, head_dim=l.dim, qkv_bias=False,
        position=AdjacentRotarySpec(rotary_dim=l.rot_dims, theta=l.rot_base) if l.rot_dims > 0 else None,
        window=l.window, prefix=prefix + "left.", softmax_scale=l.scale, softcap=l.softcap, tied_values=True,
        tensor_names=(("q", "q"), ("k", "k"), ("o", "o")),
    )
    right = DecayedLinearAttentionSpec(hidden=W, n_heads=r.heads, head_dim=r.dim, value_dim=r.vdim, decay=r.decay,
                                       norm_eps=eps, prefix=prefix + "right.")
    return MixerSumSpec(mixers=(left, right), scales=(m.left_scale, m.right_scale))


def model_spec(cfg: SafepelConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        has_ff = layer.ff is not None
        layers.append(SandwichBlockSpec(
            norm1=LayerNormSpec(W, eps, p + "norm1"),
            mixer=_mixer(cfg, layer.mixer, p + "mix."),
            post1=LayerNormSpec(W, eps, p + "norm1b"),
            norm2=LayerNormSpec(W, eps, p + "norm2") if has_ff else None,
            ffn=DenseMlpSpec(hidden=W, intermediate=layer.ff, prefix=p + "mlp.", activation="relu",
                             tensor_names=("gate", "up", "down")) if has_ff else None,
            post2=LayerNormSpec(W, eps, p + "norm2b") if has_ff else None,
        ))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden=W,
        max_positions=cfg.max_positions,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=l, cache=l) for l in range(len(layers))),
        final_norm=LayerNormSpec(W, eps, "final.norm"),
        embedding_name="embed",
        head_name="head",
        embedding_norm=LayerNormSpec(W, eps, "embed.norm"),
        logit_scale=cfg.logit_scale,
    )


register_architecture(ARCHITECTURE, SafepelConfig.from_json, model_spec, replace=True)
