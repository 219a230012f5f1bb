"""Small Nirotar configurations and random weights for the tests, written with the ``safetensors`` library (not with the
engine's own writer).  Weights are drawn so that every mechanism matters: norm weights spread around one, sinks of order one
on both sides of zero, expert tables whose rows name different experts.  Values are rounded to bfloat16 so that a 32-bit
engine and the plain implementation read the same numbers.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch


def _attn(heads, kv, dim, vdim, scale, mask=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if mask:
        m["mask"] = {"size": mask}
    if rot:
        m["rot"] = rot
    return m


def _latent(heads, dim, rot_dim, vdim, rank, scale, rot=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rot:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(ff, experts, top, shared=None):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


BANDS_A = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}
# Sizes that fit no tensor-core kernel; a latent layer first, read again two layers later by a layer with other head sizes;
# windows of 9 positions and none; rotation of half a head with band-scaled frequencies, of a whole rotated part, and none;
# two, all and one of the experts chosen; with and without a shared expert; a layer without feed-forward.
CONFIG_A = {
    "architecture": "Nirotar", "vocab": 83, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 12, 6, 10, 20, 0.3, rot={"base": 100.0, "dims": 6}), "mlp": _moe(24, 5, 2, shared=40)},
        {"type": "attention", "mixer": _attn(4, 2, 16, 24, 0.3, mask=9, rot={"base": 50.0, "dims": 8, "scaling": BANDS_A}), "mlp": None},
        {"type": "latent_attention", "mixer": _latent(2, 8, 6, 16, 20, 0.4, rot={"base": 100.0, "dims": 6}, kv_from=0), "mlp": _moe(16, 3, 3)},
        {"type": "attention", "mixer": _attn(2, 2, 8, 8, 0.35), "mlp": _moe(32, 4, 1, shared=16)},
    ],
}
# Sizes the tensor-core kernels are made for: heads of 64 with values as wide and pages of 16 (prompt portions on the tcgen05
# kernel), page rows of 80 numbers (a latent of 64, whose prompt portions run on the tcgen05 kernel too, the second 64-column
# panel of a row partly filled) and of 128 in two latent groups of different sizes, a window that is no multiple of anything
# and one of exactly a page, experts in whole steps of 64; sixteen latent heads (a full tile of the single-token kernel).
BANDS_B = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
CONFIG_B = {
    "architecture": "Nirotar", "vocab": 160, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 1, 64, 64, 0.125, mask=70, rot={"base": 10000.0, "dims": 64, "scaling": BANDS_B}), "mlp": _moe(64, 8, 2, shared=128)},
        {"type": "latent_attention", "mixer": _latent(8, 32, 16, 32, 64, 0.15, rot={"base": 1000.0, "dims": 16}), "mlp": _moe(128, 4, 1, shared=64)},
        {"type": "latent_attention", "mixer": _latent(2, 64, 16, 64, 64, 0.11, rot={"base": 1000.0, "dims": 16}, kv_from=1), "mlp": None},
        {"type": "attention", "mixer": _attn(6, 2, 32, 48, 0.2, mask=16, rot={"base": 500.0, "dims": 16}), "mlp": _moe(64, 6, 3)},
        {"type": "latent_attention", "mixer": _latent(16, 16, 16, 16, 112, 0.18, rot={"base": 30000.0, "dims": 16}), "mlp": _moe(64, 8, 2, shared=64)},
    ],
}
# Edges of the parameter space: a window of one position (a token sees itself and the sink), a window longer than any
# sequence, as many kv heads as heads, ten latent heads on one page row (the lower half of the single-token kernel's tile
# partly filled), a rotated part that is not rotated at all, two experts that are both always chosen.
CONFIG_C = {
    "architecture": "Nirotar", "vocab": 70, "width": 64, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _attn(2, 1, 32, 32, 0.2, mask=1, rot={"base": 100.0, "dims": 32}), "mlp": _moe(64, 2, 2, shared=64)},
        {"type": "latent_attention", "mixer": _latent(10, 16, 16, 16, 32, 0.2), "mlp": None},
        {"type": "attention", "mixer": _attn(4, 4, 16, 16, 0.25, mask=300, rot={"base": 20.0, "dims": 4}), "mlp": _moe(64, 3, 1)},
    ],
}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
PAGE = {"A": 4, "B": 16, "C": 8}


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    width, vocab = raw["width"], raw["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(shape, generator=g) * std + mean

    def matrix(rows, cols, gain=1.0):
        return normal(rows, cols, std=gain / math.sqrt(cols))

    w: Dict[str, torch.Tensor] = {"embed": normal(vocab, width), "final.norm": normal(width, std=0.2, mean=1.0),
                                  "head": matrix(vocab, width, 1.5)}
    tables: Dict[str, torch.Tensor] = {}
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}", layer["mixer"]
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        w[p + ".norm1"] = normal(width, std=0.2, mean=1.0)
        if layer["type"] == "attention":
            G = m["kv_heads"]
            w[p + ".mix.q"], w[p + ".mix.k"], w[p + ".mix.v"] = matrix(H * d, width, 2.0), matrix(G * d, width, 2.0), matrix(G * dv, width)
        else:
            r, dr = m["kv_rank"], m["rot_dim"]
            w[p + ".mix.q"] = matrix(H * (d + dr), width, 2.0)
            if m.get("kv_from") is None:
                w[p + ".mix.dkv"] = matrix(r + dr, width, 2.0)
                w[p + ".mix.dkv.norm"] = normal(r, std=0.3, mean=1.2)
            w[p + ".mix.uk"], w[p + ".mix.uv"] = matrix(H * d, r, 1.5), matrix(H * dv, r, 1.5)
        w[p + ".mix.sink"] = normal(H, std=1.5)
        w[p + ".mix.o"] = matrix(width, H * dv, 1.5)
        if layer.get("mlp") is not None:
            mlp = layer["mlp"]
            w[p + ".norm2"] = normal(width, std=0.2, mean=1.0)
            ff, E, top = mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"]
            for e in range(E):
                w[f"{p}.mlp.e{e}.up"], w[f"{p}.mlp.e{e}.down"] = matrix(ff, width, 2.0), matrix(width, ff, 1.5)
            tables[p + ".mlp.table"] = torch.rand(vocab, E, generator=g).argsort(dim=1)[:, :top].to(torch.int32).contiguous()
            if mlp.get("shared"):
                w[p + ".mlp.shared.up"], w[p + ".mlp.shared.down"] = matrix(mlp["shared"]["ff"], width, 2.0), matrix(width, mlp["shared"]["ff"], 1.5)
    out = {k: v.to(torch.bfloat16) for k, v in w.items()}
    out.update(tables)
    return out


def write_model(path: str, raw: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(raw, fh)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def make_model_dir(path: str, name: str, seed: int = 3) -> str:
    return write_model(path, CONFIGS[name], random_weights(CONFIGS[name], seed))
