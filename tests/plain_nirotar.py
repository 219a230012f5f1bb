"""A plain, slow Nirotar in float64: one function per mechanism, loops where a loop says it best.

It shares nothing with the package: tensors come as a dict of torch tensors (any dtype; everything is widened to
float64), the configuration as the raw dict of ``config.json``.  A whole sequence is computed at once, with no cache:
what the engine gives for any cut of the prompt, any batch and any page must equal this up to rounding.

Notation: ``x`` the residual stream ``[T, width]``, ``h`` a sublayer's normed input, ``p`` a position, matrices ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def f64(t) -> torch.Tensor:
    return t.to(F64)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Rows over their root mean square (eps under the root), times ``w``."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * f64(w)


def pair_frequencies(rot: dict) -> torch.Tensor:
    """The angle per position of every rotated pair ``i < dims/2``: ``base^(-2i/dims)``; with ``scaling``, pairs whose
    wavelength ``2 pi / f`` is shorter than ``original / high`` keep it, those longer than ``original / low`` turn ``factor``
    times slower, and those between are blended by ``s = (original / wavelength - low) / (high - low)``."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength > orig / low:
                f = f / factor
            elif wavelength >= orig / high:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """``x`` ``[T, heads, dim]``: of every head the first ``dims`` elements turn, element ``2i`` together with ``2i + 1``, by
    the angle ``p f_i``; the rest pass.  Without ``rot`` nothing turns."""
    if not rot or not int(rot["dims"]):
        return x
    dims = int(rot["dims"])
    ang = positions.to(F64)[:, None] * pair_frequencies(rot)[None, :]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(T: int, window: Optional[int]) -> torch.Tensor:
    """``[T, T]`` booleans: position ``i`` (row) looks at ``j`` (column) when ``0 <= i - j`` and, with a window, ``i - j < window``."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    see = j <= i
    if window:
        see = see & (i - j < int(window))
    return see


def sink_softmax_mix(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int], sink: float) -> torch.Tensor:
    """One head.  Weights ``exp(s_j) / (exp(sink) + sum_j exp(s_j))`` over the keys a position sees; the sink has no value."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~visible(q.shape[0], window), -math.inf)
    m = torch.clamp(s.max(dim=-1, keepdim=True).values, min=sink)
    e = torch.exp(s - m)
    return (e @ v) / (torch.exp(sink - m) + e.sum(dim=-1, keepdim=True))


def window_attention(h: torch.Tensor, positions: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict) -> torch.Tensor:
    """Grouped-query attention with rotated pairs, a sliding window and a learned sink per head."""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ f64(W[pre + "q"]).T).view(T, H, d)
    k = (h @ f64(W[pre + "k"]).T).view(T, G, d)
    v = (h @ f64(W[pre + "v"]).T).view(T, G, dv)
    if m.get("rot"):
        q, k = rotate_pairs(q, positions, m["rot"]), rotate_pairs(k, positions, m["rot"])
    window = m["mask"]["size"] if m.get("mask") else None
    sink = f64(W[pre + "sink"])
    heads = [sink_softmax_mix(q[:, a], k[:, a // (H // G)], v[:, a // (H // G)], float(m["scale"]), window, float(sink[a])) for a in range(H)]
    return torch.cat(heads, dim=-1) @ f64(W[pre + "o"]).T


def latent_of(h: torch.Tensor, positions: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict, eps: float):
    """What a latent-attention layer keeps per position: the normed latent ``[T, kv_rank]`` and the rotated key part ``[T, rot_dim]``."""
    r = int(m["kv_rank"])
    both = h @ f64(W[pre + "dkv"]).T
    c = rms_norm(both[:, :r], W[pre + "dkv.norm"], eps)
    k_rot = rotate_pairs(both[:, None, r:], positions, m.get("rot"))[:, 0]
    return c, k_rot


def latent_attention(h: torch.Tensor, positions: torch.Tensor, W: Dict[str, torch.Tensor], pre: str, m: dict, c: torch.Tensor,
                     k_rot: torch.Tensor) -> torch.Tensor:
    """Attention whose keys and values are expanded per head from a shared latent; one rotated key part serves all heads."""
    H, d, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    T = h.shape[0]
    q = (h @ f64(W[pre + "q"]).T).view(T, H, d + dr)
    q_rot = rotate_pairs(q[..., d:], positions, m.get("rot"))
    k_up = (c @ f64(W[pre + "uk"]).T).view(T, H, d)
    v_up = (c @ f64(W[pre + "uv"]).T).view(T, H, dv)
    sink = f64(W[pre + "sink"])
    heads = []
    for a in range(H):
        qa = torch.cat([q[:, a, :d], q_rot[:, a]], dim=-1)
        ka = torch.cat([k_up[:, a], k_rot], dim=-1)
        heads.append(sink_softmax_mix(qa, ka, v_up[:, a], float(m["scale"]), None, float(sink[a])))
    return torch.cat(heads, dim=-1) @ f64(W[pre + "o"]).T


def relu2_expert(x: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    z = torch.relu(f64(up) @ x)
    return f64(down) @ (z * z)


def table_experts(h: torch.Tensor, tokens: List[int], W: Dict[str, torch.Tensor], pre: str, mlp: dict) -> torch.Tensor:
    """A token's id names its experts in a table; each counts ``1 / top``.  A shared expert, where there is one, is added."""
    top = int(mlp["router"]["top"])
    table = W[pre + "table"]
    out = torch.zeros_like(h)
    for t, tok in enumerate(tokens):
        for c in range(top):
            e = int(table[tok, c])
            out[t] += relu2_expert(h[t], W[f"{pre}e{e}.up"], W[f"{pre}e{e}.down"]) / top
        if mlp.get("shared"):
            out[t] += relu2_expert(h[t], W[pre + "shared.up"], W[pre + "shared.down"])
    return out


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    import os

    return load_file(os.path.join(model_dir, "model.safetensors"))


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int]):
    """Logits ``[T, vocab]`` and the residual stream after every layer ``[layers, T, width]``."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = f64(W["embed"])[torch.tensor(tokens)]
    kept: Dict[int, tuple] = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, W[pre + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + window_attention(h, positions, W, pre + "mix.", m)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_of(h, positions, W, pre + "mix.", m, eps)
            c, k_rot = kept[i if m.get("kv_from") is None else int(m["kv_from"])]
            x = x + latent_attention(h, positions, W, pre + "mix.", m, c, k_rot)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + table_experts(rms_norm(x, W[pre + "norm2"], eps), tokens, W, pre + "mlp.", layer["mlp"])
        after.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ f64(W["head"]).T
    return logits, torch.stack(after)
