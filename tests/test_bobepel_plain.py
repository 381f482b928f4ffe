"""Bobepel without a GPU: the configuration reader, the description made of parts, the work list of the tensor-core
attention, and the plain implementation against restatements of its mechanisms as explicit loops."""
import copy
import math

import pytest
import torch

import plain_bobepel as pb
from bobepel_configs import BOBEPEL_A, BOBEPEL_B, CONFIGS


def resolve(cfg):
    import ferrox_b200  # noqa: F401  (registers the architectures)
    from ferrox_b200.config.registry import resolve as r

    return r(cfg)


def test_configuration_is_read_layer_by_layer():
    cfg, spec = resolve(BOBEPEL_A)
    assert [l.type for l in cfg.layers] == ["attention", "latent_attention", "latent_attention_2", "attention",
                                            "latent_attention"]
    assert cfg.layers[3].weights_of == 0 and cfg.layers[1].mixer.window == 21 and cfg.layers[2].mixer.q_rank == 32
    assert cfg.layers[0].mixer.q_temp == (0.5, 8) and cfg.layers[0].mlp.top == 2 and cfg.layers[2].mlp.shared_ff == 0
    # three blocks own weights; five schedule entries, each with a cache of its own
    assert len(spec.layers) == 3 and [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (0, 3), (1, 4)]
    cfgB, specB = resolve(BOBEPEL_B)
    assert cfgB.layers[1].mlp is None and specB.layers[1].ffn is None
    assert [(e.layer, e.cache) for e in specB.schedule] == [(0, 0), (1, 1), (0, 2), (2, 3), (3, 4)]


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="ring"), "not implemented"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not implemented"),
    (lambda c: c["layers"][3].update(weights_of=9), "names no other layer"),
    (lambda c: c["layers"][4].update(weights_of=3), "no tensors of its own"),
    (lambda c: c["layers"][3]["mixer"].update(dim=16), "differs"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "exceeds"),
    (lambda c: c["layers"][1]["mixer"].update(mask={"size": 0}), "mask.size"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configurations_that_are_refused(change, text):
    from ferrox_b200 import ConfigError

    cfg = copy.deepcopy(BOBEPEL_A)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        resolve(cfg)


def test_description_declares_the_tensors_of_the_layers_that_own_weights():
    from ferrox_b200.parts.build import build_model

    _, spec = resolve(BOBEPEL_A)
    decls = {d.name: d.shape for d in build_model(spec).tensor_decls()}
    assert decls["embed"] == (211, 64) and decls["head"] == (211, 64) and decls["final.norm"] == (64,)
    assert decls["l0.mix.q"] == (4 * 32, 64) and decls["l0.mix.v"] == (2 * 48, 64) and decls["l0.mix.o"] == (64, 4 * 48)
    assert decls["l0.mix.q.norm"] == (32,) and decls["l0.mlp.e5.down"] == (64, 32) and decls["l0.mlp.shared.up"] == (64, 64)
    assert decls["l1.mix.dkv"] == (48 + 32, 64) and decls["l1.mix.uk"] == (4 * 16, 48) and decls["l1.mix.g"] == (4 * 16, 64)
    assert decls["l2.mix.dq"] == (32, 64) and decls["l2.mix.uq"] == (2 * 48, 32) and "l2.mix.g" not in decls
    assert not any(n.startswith(("l3.", "l4.")) for n in decls) and "l2.mlp.shared.gate" not in decls
    caches = build_model(spec).cache_specs()
    assert caches[0].paged.window is None and caches[1].paged.window == 21 and caches[4].paged.window == 21
    assert [t.name for t in caches[0].paged.tensors] == ["k", "v"] and caches[1].paged.tensors[0].token_shape == (80,)


@pytest.mark.parametrize("heads,kv_heads,entries", [(4, 2, [5, 1, 130]), (8, 1, [3]), (96, 1, [2, 7]), (200, 2, [1, 1, 4]),
                                                     (3, 3, [64, 65])])
def test_work_list_of_the_tensor_core_attention_covers_every_row_once(heads, kv_heads, entries):
    from ferrox_b200.kernels import ops

    items = ops.general_attention_items(entries, heads, kv_heads)
    group = heads // kv_heads
    seen = set()
    starts = [sum(entries[:i]) for i in range(len(entries))]
    for tok0, n_tok, entry, head0, n_h in items.tolist():
        assert 1 <= n_tok * n_h <= ops.GENERAL_TILE_ROWS
        assert starts[entry] <= tok0 and tok0 + n_tok <= starts[entry] + entries[entry]      # one request a tile
        assert head0 // group == (head0 + n_h - 1) // group                                  # one kv head a tile
        for t in range(tok0, tok0 + n_tok):
            for h in range(head0, head0 + n_h):
                assert (t, h) not in seen
                seen.add((t, h))
    assert len(seen) == sum(entries) * heads


def _weights(cfg, seed):
    from ferrox_b200.parts.build import build_model
    from ferrox_b200.weights.random_init import random_tensors

    _, spec = resolve(cfg)
    return {n: t.float() for n, t in random_tensors(build_model(spec).tensor_decls(), seed, torch.bfloat16, 0.15, "around_one")}


def test_plain_attention_against_loops():
    """Scores, bias, temperature and visibility written out query by query and key by key."""
    cfg = BOBEPEL_B
    w = _weights(cfg, 3)
    m = cfg["layers"][4]["mixer"]
    g = torch.Generator().manual_seed(1)
    h = torch.randn(70, cfg["width"], generator=g)
    want = pb.mixer_attention(h, m, w, "l4.mix.", 1e-6)
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    out = torch.zeros(70, H * V)
    for i in range(70):
        temp = 1 + m["q_temp"]["coef"] * math.log((i + 1) // m["q_temp"]["every"] + 1)
        for hd in range(H):
            q = w["l4.mix.q"][hd * D:(hd + 1) * D] @ h[i]
            q = q / torch.sqrt((q * q).mean() + 1e-6) * w["l4.mix.q.norm"] * temp
            kv = hd // (H // G)
            scores, vals = [], []
            for j in range(i + 1):
                k = w["l4.mix.k"][kv * D:(kv + 1) * D] @ h[j]
                k = k / torch.sqrt((k * k).mean() + 1e-6) * w["l4.mix.k.norm"]
                scores.append(float(q @ k) * m["scale"] - 2.0 ** (-8 * (hd + 1) / H) * (i - j))
                vals.append(w["l4.mix.v"][kv * V:(kv + 1) * V] @ h[j])
            p = torch.softmax(torch.tensor(scores), 0)
            out[i, hd * V:(hd + 1) * V] = sum(pj * v for pj, v in zip(p, vals))
    assert float((out @ w["l4.mix.o"].T - want).abs().max()) < 1e-4


def test_plain_latent_attention_window_and_rotation_against_loops():
    cfg = BOBEPEL_A
    w = _weights(cfg, 4)
    m = cfg["layers"][1]["mixer"]
    g = torch.Generator().manual_seed(2)
    n = 50
    h = torch.randn(n, cfg["width"], generator=g)
    want = pb.mixer_latent_attention(h, m, w, "l1.mix.", 1e-6, query_latent=False, gated=True)
    H, D, R, V, C, Wn = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["mask"]["size"]
    dims, base = m["rot"]["dims"], m["rot"]["base"]

    def turn(x, p):
        y = x.clone()
        for i in range(dims // 2):
            a = torch.tensor(float(p), dtype=torch.float32) * torch.tensor(base ** (-2.0 * i / dims), dtype=torch.float32)
            c, s = torch.cos(a), torch.sin(a)
            y[2 * i], y[2 * i + 1] = x[2 * i] * c - x[2 * i + 1] * s, x[2 * i + 1] * c + x[2 * i] * s
        return y

    lat, rot = [], []
    for j in range(n):
        d = w["l1.mix.dkv"] @ h[j]
        c = d[:C]
        lat.append(c / torch.sqrt((c * c).mean() + 1e-6) * w["l1.mix.dkv.norm"])
        rot.append(turn(d[C:], j))
    out = torch.zeros(n, H * V)
    for i in range(n):
        q = (w["l1.mix.q"] @ h[i]).view(H, D + R)
        for hd in range(H):
            qr = turn(q[hd, D:], i)
            keys = range(max(0, i - Wn + 1), i + 1)
            sc = torch.tensor([float(q[hd, :D] @ (w["l1.mix.uk"][hd * D:(hd + 1) * D] @ lat[j]) + qr @ rot[j]) * m["scale"]
                               for j in keys])
            p = torch.softmax(sc, 0)
            out[i, hd * V:(hd + 1) * V] = sum(pj * (w["l1.mix.uv"][hd * V:(hd + 1) * V] @ lat[j]) for pj, j in zip(p, keys))
    out = out * torch.sigmoid(h @ w["l1.mix.g"].T)
    assert float((out @ w["l1.mix.o"].T - want).abs().max()) < 1e-4


def test_plain_whole_model_equals_its_prefixes_and_shares_weights():
    """Causal: the logits of a prefix do not change when tokens follow; a layer with weights_of reads the other
    layer's tensors (the model has none of its own for it)."""
    for name, (cfg, seed) in CONFIGS.items():
        w = _weights(cfg, seed)
        toks = [(7 * i + 3) % cfg["vocab"] for i in range(45)]
        full = pb.forward(cfg, w, toks)
        assert float((pb.forward(cfg, w, toks[:20]) - full[:20]).abs().max()) < 1e-4, name
    assert not any(k.startswith("l3.") for k in _weights(BOBEPEL_A, 1))
