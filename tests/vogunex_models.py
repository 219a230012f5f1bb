"""Small Vogunex configurations and random weights for the tests, written with the ``safetensors`` library (not with the
engine's own writer).  Weights are drawn so that every mechanism matters: shifts inside (0, 1), mixing matrices of the heads'
weights near the identity with entries of both signs, decay rates from slow to fast, router logits spread over several
units.  Values are rounded to bfloat16 so that a 32-bit engine and the plain implementation read the same numbers.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict

import torch


def _attn(heads, kv, dim, vdim, scale, size=None, pool=None, rot=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        m["mask"] = {"size": size}
        if pool:
            m["mask"]["pool"] = pool
    if rot:
        m["rot"] = rot
    if softcap:
        m["softcap"] = softcap
    return m


def _latent(heads, dim, rot_dim, vdim, rank, q_rank, scale, base, size=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if size:
        m["mask"] = {"size": size}
    return m


def _ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _moe(ff, experts, top, limit, shared=None, shared_limit=None):
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared, "limit": shared_limit or limit}
    return mlp


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _again(layer: dict, source: int) -> dict:
    return dict(layer, weights_of=source)


# Sizes that fit no tensor-core kernel; every mixer twice (the second run with the first one's weights); a pool of three
# positions over pages of four (blocks straddle pages), half a head rotated, a capped score; two of five and all of three
# experts chosen, with and without a shared expert.
_A0 = {"type": "attention", "mixer": _attn(4, 2, 12, 10, 0.3, size=9, pool=3, rot={"base": 100.0, "dims": 6}, softcap=5.0), "mlp": _dense(56)}
_A1 = {"type": "mamba2", "mixer": _ssm(3, 10, 6, 1, 3, 1), "mlp": _moe(24, 5, 2, 0.8, shared=40, shared_limit=1.5)}
_A3 = {"type": "latent_attention", "mixer": _latent(3, 12, 6, 10, 20, 14, 0.3, 100.0, size=7), "mlp": _moe(16, 3, 3, 1.2)}
CONFIG_A = {"architecture": "Vogunex", "vocab": 77, "width": 40, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
            "layers": [_A0, _A1, _again(_A0, 0), _A3, _again(_A1, 1), _again(_A3, 3)]}
# Sizes the tensor-core kernels are made for: heads of 64, page rows of 80 and 128 numbers, experts in whole steps of 64, a
# pool of eight over pages of sixteen, a window that is no multiple of anything; two groups and two norm parts in the state
# space layer; a latent layer without a window and without a feed-forward.
_B0 = {"type": "mamba2", "mixer": _ssm(4, 32, 16, 2, 4, 2), "mlp": _moe(64, 8, 2, 1.0, shared=128)}
_B1 = {"type": "attention", "mixer": _attn(8, 2, 64, 64, 0.125, size=70, pool=8, rot={"base": 10000.0, "dims": 32}, softcap=30.0), "mlp": _dense(256)}
_B2 = {"type": "latent_attention", "mixer": _latent(8, 32, 16, 32, 64, 48, 0.15, 1000.0, size=33), "mlp": _moe(128, 4, 1, 2.0, shared=64, shared_limit=0.5)}
_B4 = {"type": "latent_attention", "mixer": _latent(16, 16, 16, 16, 112, 64, 0.18, 30000.0), "mlp": None}
CONFIG_B = {"architecture": "Vogunex", "vocab": 160, "width": 128, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
            "layers": [_B0, _B1, _B2, _again(_B1, 1), _B4, _again(_B0, 0)]}
# Edges of the parameter space: a layer that uses the weights of a later one; a window shorter than a block (tokens that
# have left it wait, unseen, for their block to end); a window longer than any sequence (no block is ever seen); as many kv
# heads as heads and one for all; a whole head rotated and none; no cap; a state of five rows with one group per head and a
# norm part per head; a convolution of two taps and one of a single tap; one expert of two and both; no embedding scale.
_C2 = {"type": "attention", "mixer": _attn(2, 2, 32, 16, 0.2, size=3, pool=5, rot={"base": 50.0, "dims": 32}), "mlp": _dense(64)}
CONFIG_C = {"architecture": "Vogunex", "vocab": 70, "width": 64, "norm": {"eps": 1e-6},
            "layers": [_again(_C2, 2),
                       {"type": "mamba2", "mixer": _ssm(4, 16, 5, 4, 2, 4), "mlp": None},
                       _C2,
                       {"type": "attention", "mixer": _attn(4, 1, 16, 16, 0.25, size=300, pool=2, softcap=2.0), "mlp": _moe(64, 2, 2, 1.0)},
                       {"type": "latent_attention", "mixer": _latent(2, 16, 8, 24, 32, 16, 0.2, 20.0, size=1), "mlp": _moe(32, 2, 1, 0.7, shared=32)},
                       {"type": "mamba2", "mixer": _ssm(2, 24, 8, 1, 1, 1), "mlp": _dense(32)},
                       {"type": "attention", "mixer": _attn(4, 4, 8, 8, 0.35, size=6, pool=1, rot={"base": 10.0, "dims": 2}), "mlp": None}]}
CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
PAGE = {"A": 4, "B": 16, "C": 8}


def random_weights(raw: dict, seed: int) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    width, vocab = raw["width"], raw["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return torch.randn(shape, generator=g) * std + mean

    def matrix(rows, cols, gain=1.0):
        return normal(rows, cols, std=gain / math.sqrt(cols))

    w: Dict[str, torch.Tensor] = {"embed": normal(vocab, width, std=1.0 / (raw.get("embedding") or {}).get("scale", 1.0)),
                                  "final.norm": normal(width, std=0.2, mean=1.0), "head": matrix(vocab, width, 1.5)}
    for i, layer in enumerate(raw["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m = f"l{i}", layer["mixer"]
        w[p + ".norm1"] = normal(width, std=0.2, mean=1.0)
        w[p + ".shift"] = torch.rand(width, generator=g) * 0.9
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + ".mix.q"], w[p + ".mix.k"], w[p + ".mix.v"] = matrix(H * d, width, 2.0), matrix(G * d, width, 2.0), matrix(G * dv, width)
            w[p + ".mix.q.b"], w[p + ".mix.k.b"], w[p + ".mix.v.b"] = normal(H * d, std=0.5), normal(G * d, std=0.5), normal(G * dv, std=0.3)
            w[p + ".mix.talk"] = torch.eye(H) + normal(H, H, std=0.3)
            w[p + ".mix.o"] = matrix(width, H * dv, 1.5)
        elif layer["type"] == "latent_attention":
            H, d, dv, r, dr, qr = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["rot_dim"], m["q_rank"]
            w[p + ".mix.dq"], w[p + ".mix.dq.norm"] = matrix(qr, width, 2.0), normal(qr, std=0.3, mean=1.2)
            w[p + ".mix.uq"] = matrix(H * (d + dr), qr, 2.0)
            w[p + ".mix.dkv"], w[p + ".mix.dkv.norm"] = matrix(r + dr, width, 2.0), normal(r, std=0.3, mean=1.2)
            w[p + ".mix.uk"], w[p + ".mix.uv"] = matrix(H * d, r, 1.5), matrix(H * dv, r, 1.5)
            w[p + ".mix.g"] = matrix(H, width, 3.0)
            w[p + ".mix.o"] = matrix(width, H * dv, 1.5)
        else:
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, channels = H * P, H * P + 2 * G * N
            w[p + ".mix.in"] = matrix(2 * inner + 2 * G * N + H, width, 1.5)
            w[p + ".mix.conv"], w[p + ".mix.conv.b"] = normal(channels, taps, std=0.6), normal(channels, std=0.2)
            w[p + ".mix.dt_bias"] = normal(H, std=0.7, mean=-0.5)
            w[p + ".mix.A_log"] = torch.rand(H, generator=g) * 4.5 - 4.0           # rates from 0.02 (long memory) to 1.6
            w[p + ".mix.D"] = normal(H, std=0.3, mean=1.0)
            w[p + ".mix.norm"] = normal(inner, std=0.2, mean=1.0)
            w[p + ".mix.o"] = matrix(width, inner, 1.5)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        w[p + ".norm2"] = normal(width, std=0.2, mean=1.0)
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            w[p + ".mlp.up"], w[p + ".mlp.up.b"] = matrix(ff, width, 2.0), normal(ff, std=0.5)
            w[p + ".mlp.down"], w[p + ".mlp.down.b"] = matrix(width, ff, 1.5), normal(width, std=0.3)
            continue
        ff, E = mlp["expert"]["ff"], mlp["router"]["experts"]
        for e in range(E):
            w[f"{p}.mlp.e{e}.gate"], w[f"{p}.mlp.e{e}.up"] = matrix(ff, width, 2.0), matrix(ff, width, 2.0)
            w[f"{p}.mlp.e{e}.down"] = matrix(width, ff, 1.5)
        w[p + ".mlp.router"], w[p + ".mlp.router.b"] = matrix(E, width, 4.0), normal(E, std=0.5)
        if mlp.get("shared"):
            sf = mlp["shared"]["ff"]
            w[p + ".mlp.shared.gate"], w[p + ".mlp.shared.up"] = matrix(sf, width, 2.0), matrix(sf, width, 2.0)
            w[p + ".mlp.shared.down"], w[p + ".mlp.shared.sg"] = matrix(width, sf, 1.5), matrix(1, width, 3.0)
    return {k: v.to(torch.bfloat16) for k, v in w.items()}


def write_model(path: str, raw: dict, weights: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(raw, fh)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(path, "model.safetensors"))
    return path


def make_model_dir(path: str, name: str, seed: int = 3) -> str:
    return write_model(path, CONFIGS[name], random_weights(CONFIGS[name], seed))
