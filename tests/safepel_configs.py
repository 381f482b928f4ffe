"""Tiny Safepel configurations that differ from each other in every size, constant and in the order of layers, and
the helper that writes a folder of random weights for one (into a temporary folder, never committed)."""
from __future__ import annotations

ARCH = "Safepel"


def delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def parallel(heads, kv_heads, dim, window, rot_dims, base, scale, softcap, rheads, rdim, rvdim, decay, ls, rs, ff):
    return {"type": "parallel", "mlp": None if ff is None else {"kind": "dense", "ff": ff}, "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
                 "rot": {"dims": rot_dims, "base": base}, "scale": scale, "softcap": softcap},
        "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "decay": decay},
        "left_scale": ls, "right_scale": rs}}


# A: delta first, alternating; grouped q/k heads; window shorter than a page; rotary on half of the head.
SAFEPEL_A = {
    "architecture": ARCH, "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [
        delta(4, 2, 16, 24, 4, 96),
        parallel(4, 2, 32, 7, 16, 10000.0, 0.25, 8.0, 3, 16, 24, [0.5, 0.9, 0.995], 0.7, 1.3, 96),
        delta(4, 2, 16, 24, 4, 96),
    ],
}

# B: parallel first, two of the same type in a row, a layer without feed-forward, sizes that are no power of two and
# no multiple of 16, one q/k head for all, taps 2, a window that crosses pages, full rotary, scales of 1.
SAFEPEL_B = {
    "architecture": ARCH, "vocab": 97, "width": 80, "norm": {"eps": 3e-6}, "logit_scale": 2.0,
    "layers": [
        parallel(6, 3, 24, 21, 24, 500.0, 0.3, 3.0, 2, 20, 12, [0.8, 0.97], 1.0, 1.0, None),
        parallel(2, 1, 48, 40, 32, 1000000.0, 0.11, 30.0, 5, 8, 40, [0.3, 0.6, 0.9, 0.99, 0.999], 1.5, 0.4, 56),
        delta(3, 1, 20, 12, 2, 120),
        delta(2, 2, 40, 36, 3, None),
    ],
}

# C: one layer of each type with heads == kv_heads, a window of one (a token sees itself only), no rotation, taps 1.
SAFEPEL_C = {
    "architecture": ARCH, "vocab": 50, "width": 32, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
    "layers": [
        parallel(2, 2, 16, 1, 0, 10000.0, 0.5, 5.0, 1, 8, 8, [0.9], 1.0, 2.0, 48),
        delta(2, 2, 8, 8, 1, 48),
    ],
}

# D: delta layers only (no layer keeps pages: the cache manager has no page group at all), q/k heads of 130 rows
# (more than 128: the recurrence kernel's wide form), an odd number of value columns.
SAFEPEL_D = {
    "architecture": ARCH, "vocab": 61, "width": 40, "norm": {"eps": 1e-6}, "logit_scale": 0.3,
    "layers": [delta(2, 1, 130, 9, 4, 64), delta(1, 1, 6, 70, 5, None)],
}

# E: parallel layers only, as many key heads as query heads, a head size that is no multiple of 8, a window longer
# than anything the tests feed, a rotary width of 2, a width and a feed-forward that are no multiple of 8.
SAFEPEL_E = {
    "architecture": ARCH, "vocab": 73, "width": 44, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
    "layers": [
        parallel(3, 3, 20, 500, 2, 77.0, 0.4, 2.5, 4, 12, 5, [0.9, 0.8, 0.7, 0.6], 0.9, 0.2, 70),
        parallel(2, 1, 36, 33, 36, 10000.0, 0.2, 50.0, 1, 24, 48, [0.98], 0.5, 1.0, None),
    ],
}

# F: attention heads of 64 and of 128 (the sizes the kernels that stream pages by TMA and the tcgen05 prompt kernel
# take when scores are not capped), windows that cross the 64-key blocks, state heads of 64 and 128 rows.
SAFEPEL_F = {
    "architecture": ARCH, "vocab": 131, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.7,
    "layers": [
        parallel(4, 1, 64, 70, 64, 10000.0, 0.125, 15.0, 2, 64, 32, [0.9, 0.99], 1.0, 0.5, 192),
        delta(2, 1, 128, 64, 4, 192),
        parallel(2, 2, 128, 65, 32, 500.0, 0.09, 25.0, 1, 128, 128, [0.95], 0.6, 1.2, None),
    ],
}

CONFIGS = {"A": (SAFEPEL_A, 11), "B": (SAFEPEL_B, 12), "C": (SAFEPEL_C, 13), "D": (SAFEPEL_D, 14), "E": (SAFEPEL_E, 15),
           "F": (SAFEPEL_F, 16)}


def make_folder(tmp_path, name, std=0.15):
    from ferrox_b200 import write_random_model

    cfg, seed = CONFIGS[name]
    folder = str(tmp_path / f"safepel_{name}")
    write_random_model(folder, cfg, seed, dtype="bfloat16", std=std, norm_init="around_one")
    return folder
