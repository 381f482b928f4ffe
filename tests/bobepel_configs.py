"""Tiny Bobepel configurations that differ from each other in every size, constant, in the order of layers and in
which layers share weights, and the helper that writes a folder of random weights for one (into a temporary folder,
never committed)."""
from __future__ import annotations

import copy

ARCH = "Bobepel"


def moe(experts, top, ff, limit, shared_ff=None, shared_limit=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top},
            "shared": None if shared_ff is None else {"ff": shared_ff, "limit": shared_limit}}


def attention(heads, kv_heads, dim, vdim, scale, coef, every, mlp, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
         "q_temp": {"coef": coef, "every": every}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, rot_dims, base, vdim, kv_rank, scale, mlp, window=None, q_rank=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "rot": {"dims": rot_dims, "base": base}, "vdim": vdim,
         "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if q_rank:
        m["q_rank"] = q_rank
    return {"type": "latent_attention_2" if q_rank else "latent_attention", "mixer": m, "mlp": mlp}


def shares(layer, j):
    out = copy.deepcopy(layer)
    out["weights_of"] = j
    return out


# A: sizes in steps of 16 (the tensor-core attention takes them in bfloat16); values wider than keys; two experts of
# six with a shared one; a window that crosses pages; the rotated part wider than what is rotated; a temperature that
# changes every 8 positions; the last two layers run the first two's weights again.
_A0 = attention(4, 2, 32, 48, 0.21, 0.5, 8, moe(6, 2, 32, 1.0, 64, 0.7))
_A1 = latent(4, 16, 32, 16, 10000.0, 16, 48, 0.17, moe(6, 2, 32, 1.0, 64, 0.7), window=21)
BOBEPEL_A = {
    "architecture": ARCH, "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "layers": [_A0, _A1, latent(2, 32, 16, 16, 300000.0, 32, 64, 0.2, moe(4, 1, 48, 2.5), q_rank=32),
               shares(_A0, 0), shares(_A1, 1)],
}

# B: sizes that are no multiple of 16 or 8 (the warp-per-row attention in both engines); as many key heads as query
# heads; a layer without feed-forward; one expert of three without a shared one; three of three; a window of one; a
# latent layer first; sharing that skips a layer.
_B0 = latent(3, 12, 6, 4, 77.0, 20, 40, 0.3, moe(3, 1, 24, 0.8), window=1)
BOBEPEL_B = {
    "architecture": ARCH, "vocab": 97, "width": 72, "norm": {"eps": 3e-6},
    "layers": [_B0, attention(3, 3, 20, 12, 0.35, 0.25, 3, None), shares(_B0, 0),
               latent(2, 24, 8, 8, 1000.0, 28, 36, 0.25, moe(3, 3, 40, 3.0, 24, 1.2), q_rank=20),
               attention(6, 1, 24, 40, 0.15, 1.0, 50, moe(5, 2, 16, 0.5, 8, 0.4))],
}

# C: one layer of each kind with larger heads: keys of 128 and values of 64, all heads on one kv head, a latent of
# 192 with 64 rotated (rows of 256, values of 192: both halves of the value columns), windows beyond a page of 64,
# a windowed plain attention and an unwindowed latent one.
BOBEPEL_C = {
    "architecture": ARCH, "vocab": 131, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        attention(8, 1, 128, 64, 0.09, 0.35, 64, moe(8, 2, 96, 1.25, 160, 1.75), window=70),
        latent(8, 64, 64, 64, 250000.0, 64, 192, 0.1, moe(8, 2, 96, 1.25, 160, 1.75)),
        latent(4, 32, 32, 32, 10000.0, 64, 128, 0.15, None, window=65, q_rank=96),
    ],
}

CONFIGS = {"A": (BOBEPEL_A, 21), "B": (BOBEPEL_B, 22), "C": (BOBEPEL_C, 23)}


def make_folder(tmp_path, name, std=0.15):
    from ferrox_b200 import write_random_model

    cfg, seed = CONFIGS[name]
    folder = str(tmp_path / f"bobepel_{name}")
    write_random_model(folder, cfg, seed, dtype="bfloat16", std=std, norm_init="around_one")
    return folder
