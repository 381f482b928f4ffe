"""Bobepel as a description made of parts.

A decoder whose layers, in whatever order ``config.json`` lists them, mix with one of three attentions and run
their feed-forward beside the mixer, both on the output of the layer's one norm:

    x = norm1(h);   h += mixer(x) + ffn(x)                    norm: h / sqrt(mean(h^2) + eps) * (1 + w)

* ``attention``: grouped-query attention without rotation.  Queries and keys are RMS-normed per head; the query at
  position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1); the score of key j for query i is
  scale (q . k) - 2^(-8 (h + 1) / H) (i - j) in head h of H; keys and values may differ in width.
* ``latent_attention``: a position caches one normed latent vector and one rotated key part shared by all heads;
  a sliding window; the heads' outputs are gated by sigmoid(g . x).
* ``latent_attention_2``: the same cache; queries through a normed latent of their own; all earlier positions.
* feed-forward: experts chosen by the largest sigmoid(router logit); the chosen scores, as they are, multiply
  the experts' INPUT; an expert is down(min(g, l) sigmoid(1.702 min(g, l)) (clamp(u, -l, l) + 1)) with g, u its
  gate and up products and l its limit; a shared expert with a limit of its own is added for every token.
* a layer with ``weights_of: j`` runs layer j's tensors against a cache of its own: one block, two schedule entries.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.{router, e<k>.{gate,up,down}, shared.{...}}``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.bobepel import ARCHITECTURE, AttentionConfig, BobepelConfig, LatentAttentionConfig
from ..config.registry import register_architecture
from ..parts.specs import (
    AttentionSpec,
    LatentAttentionSpec,
    ModelSpec,
    MoeSpec,
    NormSpec,
    ParallelBlockSpec,
    ScheduleEntry,
)

GATE_ALPHA = 1.702          # the experts' gate passes through g * sigmoid(GATE_ALPHA * g)
SLOPE_EXPONENT = 8.0        # head h of H lowers a score by 2^(-SLOPE_EXPONENT (h + 1) / H) per position of distance


def distance_slopes(n_heads: int):
    return tuple(2.0 ** (-SLOPE_EXPONENT * (h + 1) / n_heads) for h in range(n_heads))


def _mixer(cfg: BobepelConfig, m, prefix: str):
    W, eps = cfg.width, cfg.norm_eps
    if isinstance(m, AttentionConfig):
        return AttentionSpec(
            hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qkv_bias=False, position=None,
            window=m.window, prefix=prefix, softmax_scale=m.scale, value_dim=m.vdim,
            tensor_names=(("q", "q"), ("k", "k"), ("v", "v"), ("o", "o")),
            qk_norm=("q.norm", "k.norm", eps), query_temperature=m.q_temp, distance_slopes=distance_slopes(m.heads),
        )
    assert isinstance(m, LatentAttentionConfig)
    return LatentAttentionSpec(
        hidden=W, n_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, kv_rank=m.kv_rank,
        q_rank=m.q_rank, rotary_dims=m.rot_dims, rotary_base=m.rot_base, window=m.window, scale=m.scale,
        output_gate=m.output_gate, norm_eps=eps, prefix=prefix,
    )


def _ffn(cfg: BobepelConfig, f, prefix: str):
    if f is None:
        return None
    return MoeSpec(
        hidden=cfg.width, n_experts=f.experts, top_k=f.top, expert_intermediate=f.ff, shared_intermediate=f.shared_ff,
        norm_topk_prob=False, shared_gate=False, prefix=prefix, scores="sigmoid", weight_on_input=True,
        activation=("clamped_swish", f.limit, GATE_ALPHA),
        shared_activation=("clamped_swish", f.shared_limit, GATE_ALPHA) if f.shared_ff else None,
        tensor_names=("router", "e{e}.{part}", "shared.{part}"),
    )


def model_spec(cfg: BobepelConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.norm_eps
    blocks, block_of, schedule = [], {}, []
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is None:
            p = f"l{i}."
            block_of[i] = len(blocks)
            blocks.append(ParallelBlockSpec(
                norm1=NormSpec(W, eps, p, name=p + "norm1", one_plus=True),
                mixer=_mixer(cfg, layer.mixer, p + "mix."),
                ffn=_ffn(cfg, layer.mlp, p + "mlp."),
            ))
    for i, layer in enumerate(cfg.layers):
        src = i if layer.weights_of is None else layer.weights_of
        schedule.append(ScheduleEntry(layer=block_of[src], cache=i))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden=W,
        max_positions=cfg.max_positions,
        layers=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=NormSpec(W, eps, "final.", name="final.norm", one_plus=True),
        embedding_name="embed",
        head_name="head",
    )


register_architecture(ARCHITECTURE, BobepelConfig.from_json, model_spec, replace=True)
