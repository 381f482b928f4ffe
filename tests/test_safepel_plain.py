"""The plain Safepel implementation checked against itself (properties that any correct implementation has), the
configuration reader, the model description's tensors and cache needs.  No GPU."""
import copy

import pytest
import torch

import plain_safepel as ps
from safepel_configs import CONFIGS, SAFEPEL_A, SAFEPEL_B, SAFEPEL_C


def weights_for(cfg, seed=0, std=0.2, dtype=torch.float64):
    from ferrox_b200.config.registry import resolve
    from ferrox_b200.parts.build import build_model
    from ferrox_b200.weights.random_init import random_tensors

    decls = build_model(resolve(cfg)[1]).tensor_decls()
    return {n: t.to(dtype) for n, t in random_tensors(decls, seed, torch.bfloat16, std, "around_one")}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_position_depends_on_earlier_tokens_only(name):
    cfg, seed = CONFIGS[name]
    w = weights_for(cfg, seed)
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, cfg["vocab"], (30,), generator=g).tolist()
    whole = ps.forward(cfg, w, toks)
    assert torch.isfinite(whole).all()
    for n in (1, 2, 9, 29):
        assert torch.allclose(ps.forward(cfg, w, toks[:n]), whole[:n], rtol=0, atol=1e-9)
    other = list(toks)
    other[20] = (other[20] + 1) % cfg["vocab"]
    changed = ps.forward(cfg, w, other)
    assert torch.equal(changed[:20], whole[:20]) and not torch.allclose(changed[20:], whole[20:])


def test_window_of_the_capped_attention_is_its_own_token_and_the_ones_before():
    m = copy.deepcopy(SAFEPEL_A["layers"][1]["mixer"]["left"])
    g = torch.Generator().manual_seed(3)
    w = {"p.q": torch.randn(128, 64, generator=g, dtype=torch.float64), "p.k": torch.randn(64, 64, generator=g, dtype=torch.float64),
         "p.o": torch.randn(64, 128, generator=g, dtype=torch.float64)}
    h = torch.randn(20, 64, generator=g, dtype=torch.float64)
    pos = torch.arange(20)
    base = ps.capped_window_attention(h, w, "p.", m, pos)
    W = m["mask"]["size"]
    moved = h.clone()
    moved[5] += 1.0
    out = ps.capped_window_attention(moved, w, "p.", m, pos)
    same = (out - base).abs().max(dim=1).values < 1e-12
    assert same[:5].all() and not same[5:5 + W].any() and same[5 + W:].all()
    # the cap: scores pushed far beyond it change nothing any more
    big = {k: v * (1e6 if k == "p.q" else 1.0) for k, v in w.items()}
    bigger = {k: v * (1e7 if k == "p.q" else 1.0) for k, v in w.items()}
    a, b = ps.capped_window_attention(h, big, "p.", m, pos), ps.capped_window_attention(h, bigger, "p.", m, pos)
    assert torch.allclose(a, b, atol=1e-6)


def test_delta_rule_replaces_what_a_key_holds():
    """With beta = 1, no decay and orthogonal unit keys, writing v under k and reading with q = k returns v; writing
    under the same key again returns the new v alone (the old one is taken out)."""
    D, V = 4, 3
    S = torch.zeros(D, V, dtype=torch.float64)
    k = torch.eye(D, dtype=torch.float64)
    vs = torch.tensor([[1.0, 2, 3], [4, 5, 6], [7, 8, 9]], dtype=torch.float64)
    for key, v in ((0, vs[0]), (1, vs[1]), (0, vs[2])):
        u = 1.0 * (v - S.T @ k[key])
        S = S + torch.outer(k[key], u)
    assert torch.allclose(S.T @ k[0], vs[2]) and torch.allclose(S.T @ k[1], vs[1])


def test_short_convolution_reads_the_current_token_with_its_last_column():
    x = torch.arange(12, dtype=torch.float64).view(6, 2)
    w = torch.tensor([[0.0, 0, 1], [1, 0, 0]], dtype=torch.float64)     # channel 0: now; channel 1: two tokens ago
    y = ps.short_conv(x, w)
    assert torch.equal(y[:, 0], x[:, 0])
    assert torch.equal(y[:, 1], torch.cat([torch.zeros(2, dtype=torch.float64), x[:-2, 1]]))


def test_rotation_of_neighbours_keeps_relative_positions():
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 8, generator=g, dtype=torch.float64), torch.randn(1, 1, 8, generator=g, dtype=torch.float64)
    def score(pq, pk):
        a = ps.rotate_adjacent(q, torch.tensor([pq]), 100.0, 6)
        b = ps.rotate_adjacent(k, torch.tensor([pk]), 100.0, 6)
        return float((a * b).sum())
    assert abs(score(9, 4) - score(105, 100)) < 1e-9 and abs(score(9, 4) - score(9, 5)) > 1e-6
    r = ps.rotate_adjacent(q, torch.tensor([7]), 100.0, 6)
    assert torch.equal(r[..., 6:], q[..., 6:])       # beyond the rotary width nothing moves


# ------------------------------------------------------------------ configuration and description
def test_config_reads_every_layer_and_refuses_what_is_not_implemented():
    from ferrox_b200 import ConfigError
    from ferrox_b200.config.safepel import SafepelConfig

    c = SafepelConfig.from_json(SAFEPEL_B)
    assert [l.type for l in c.layers] == ["parallel", "parallel", "delta", "delta"]
    assert c.layers[0].ff is None and c.layers[1].ff == 56 and c.layers[3].ff is None
    assert c.layers[1].mixer.left.window == 40 and c.layers[1].mixer.right.decay[-1] == 0.999
    assert c.norm_eps == 3e-6 and c.logit_scale == 2.0 and c.vocab == 97
    for path, value, text in (
        (("layers", 0, "type"), "hyena", "layer type"),
        (("layers", 1, "mlp", "kind"), "experts", "kind"),
        (("layers", 1, "mixer", "right", "decay"), [0.5], "decay"),
        (("layers", 0, "mixer", "left", "rot", "dims"), 25, "rot.dims"),
        (("layers", 2, "mixer", "kv_heads"), 2, "kv_heads"),
    ):
        bad = copy.deepcopy(SAFEPEL_B)
        at = bad
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            SafepelConfig.from_json(bad)
    missing = copy.deepcopy(SAFEPEL_A)
    del missing["layers"][0]["mixer"]["conv"]
    with pytest.raises(ConfigError, match="conv"):
        SafepelConfig.from_json(missing)


def test_description_declares_the_tensors_and_cache_needs_of_each_layer():
    from ferrox_b200.config.registry import resolve
    from ferrox_b200.parts.build import build_model

    _, spec = resolve(SAFEPEL_B)
    model = build_model(spec)
    d = {x.name: tuple(x.shape) for x in model.tensor_decls()}
    assert d["embed"] == (97, 80) and d["head"] == (97, 80) and d["embed.norm"] == (80,) and d["final.norm"] == (80,)
    assert d["l0.mix.left.q"] == (144, 80) and d["l0.mix.left.k"] == (72, 80) and "l0.mix.left.v" not in d
    assert d["l1.mix.right.v"] == (200, 80) and d["l1.mix.right.norm"] == (200,) and d["l1.mlp.gate"] == (56, 80)
    assert d["l2.mix.q"] == (20, 80) and d["l2.mix.v.conv"] == (36, 2) and d["l2.mix.norm"] == (12,)
    assert d["l2.mix.A_log"] == (3,) and d["l3.mix.o"] == (80, 72)
    assert "l0.norm2" not in d and "l0.mlp.up" not in d and "l3.norm2b" not in d and "l2.norm2b" in d
    cs = model.cache_specs()
    assert cs[0].paged.window == 21 and dict(cs[0].state.parts)["1.matrix"] == (2, 12, 20)
    assert cs[1].paged.window == 40 and cs[1].paged.tensors[0].token_shape == (1, 48)
    assert cs[2].paged is None and dict(cs[2].state.parts) == {"matrix": (3, 12, 20), "conv_tail": (1, 76)}
    assert model.graph_safe()


def test_state_slots_hold_named_tensors_and_are_cleared_for_a_new_request():
    from ferrox_b200.cache.manager import CacheManager
    from ferrox_b200.cache.specs import CacheSpec, KvCacheSpec, StateSpec

    specs = [CacheSpec(state=StateSpec(parts=(("matrix", (2, 3, 4)), ("tail", (1, 5))))),
             CacheSpec(paged=KvCacheSpec(1, 8, window=6), state=StateSpec(parts=(("1.matrix", (2, 2)),)))]
    mgr = CacheManager(specs, page_size=4, n_pages=6, max_slots=2, max_positions=64, device="cpu", dtype=torch.float32)
    a = mgr.open_request()
    lc = mgr.layer_cache(0)
    assert lc.state is None and lc.states["matrix"].shape == (2, 2, 3, 4) and lc.states["tail"].shape == (2, 1, 5)
    lc.states["matrix"][a] += 1.0
    mgr.layer_cache(1).states["1.matrix"][a] += 2.0
    mgr.close_request(a)
    b = mgr.open_request()
    assert b == a and float(lc.states["matrix"][b].abs().sum()) == 0.0
    assert float(mgr.layer_cache(1).states["1.matrix"][b].abs().sum()) == 0.0
    assert mgr.layer_cache(1).k.shape == (6, 1, 4, 8)
