"""A plain, slow implementation of Vogunex in float64: one function per mechanism, whole sequences only, no cache, no
batch.  It shares nothing with the package; the GPU tests compare the engine with it.

``config`` is the dictionary of a model's ``config.json``; ``tensors`` maps tensor names to float64 tensors.  Matrices are
stored ``[out, in]``.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """A row divided by its root mean square, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def token_shift(h: torch.Tensor, mu: torch.Tensor) -> torch.Tensor:
    """Every row moves towards the row before it (zeros before the first), element by element by ``mu``."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    return h + (before - h) * mu


def rotate(x: torch.Tensor, base: float, dims: int, neighbours: bool) -> torch.Tensor:
    """``x`` ``[T, heads, d]``: the first ``dims`` elements of every head turn by the position times a frequency per pair;
    pairs are ``(i, i + dims / 2)`` or, with ``neighbours``, ``(2i, 2i + 1)``."""
    T = x.shape[0]
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = torch.arange(T, dtype=F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    if neighbours:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def pooled_keys(rows: torch.Tensor, pool: int) -> torch.Tensor:
    """Means of whole blocks of ``pool`` rows: ``[T, ...] -> [T // pool, ...]``."""
    n = rows.shape[0] // pool
    return rows[: n * pool].reshape(n, pool, *rows.shape[1:]).mean(1)


def pooled_window_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], name: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query softmax attention: biases, part of every head rotated in half-split pairs, q and k divided by their
    root mean square per head after the rotation, scores capped by a tanh, a window of single tokens plus one pooled key and
    value for every block that lies wholly before the window, and the heads' weights mixed by a matrix."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ t[f"{name}.q"].T + t[f"{name}.q.b"]).reshape(T, H, d)
    k = (h @ t[f"{name}.k"].T + t[f"{name}.k.b"]).reshape(T, G, d)
    v = (h @ t[f"{name}.v"].T + t[f"{name}.v.b"]).reshape(T, G, dv)
    rot = m.get("rot")
    if rot is not None:
        q, k = rotate(q, rot["base"], rot["dims"], False), rotate(k, rot["base"], rot["dims"], False)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    mask = m.get("mask") or {}
    size, pool = mask.get("size"), mask.get("pool")
    cap = m.get("softcap")
    talk = t.get(f"{name}.talk")
    kb = pooled_keys(k, pool) if pool else None
    vb = pooled_keys(v, pool) if pool else None
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        first = max(0, i - size + 1) if size else 0
        blocks = max(0, (i - size + 1) // pool) if (size and pool) else 0
        weights = []
        for a in range(H):
            c = a // (H // G)
            keys = torch.cat([kb[:blocks, c], k[first:i + 1, c]], dim=0) if blocks else k[first:i + 1, c]
            s = (keys @ q[i, a]) * m["scale"]
            if cap:
                s = cap * torch.tanh(s / cap)
            weights.append(torch.softmax(s, dim=0))
        w = torch.stack(weights)                       # [H, keys]
        if talk is not None:
            w = talk @ w
        for a in range(H):
            c = a // (H // G)
            values = torch.cat([vb[:blocks, c], v[first:i + 1, c]], dim=0) if blocks else v[first:i + 1, c]
            out[i, a] = w[a] @ values
    return out.reshape(T, H * dv) @ t[f"{name}.o"].T


def latent_attention(h: torch.Tensor, t: Dict[str, torch.Tensor], name: str, m: dict, eps: float) -> torch.Tensor:
    """Attention whose keys and values are expanded per head from one latent row, with queries through a latent of their
    own, one rotated key part for all heads (neighbouring pairs), a window and a gate per head."""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ t[f"{name}.dq"].T, t[f"{name}.dq.norm"], eps)
    q = (cq @ t[f"{name}.uq"].T).reshape(T, H, d + dr)
    rows = h @ t[f"{name}.dkv"].T
    c = rms_norm(rows[:, :r], t[f"{name}.dkv.norm"], eps)
    kr = rows[:, r:].reshape(T, 1, dr)
    rot = m["rot"]
    qr = rotate(q[..., d:], rot["base"], rot["dims"], True)
    kr = rotate(kr, rot["base"], rot["dims"], True)[:, 0]
    kn = (c @ t[f"{name}.uk"].T).reshape(T, H, d)
    v = (c @ t[f"{name}.uv"].T).reshape(T, H, dv)
    size = (m.get("mask") or {}).get("size")
    gate = torch.sigmoid(h @ t[f"{name}.g"].T) if f"{name}.g" in t else None
    out = torch.zeros(T, H, dv, dtype=F)
    for i in range(T):
        first = max(0, i - size + 1) if size else 0
        for a in range(H):
            s = (kn[first:i + 1, a] @ q[i, a, :d] + kr[first:i + 1] @ qr[i, a]) * m["scale"]
            out[i, a] = torch.softmax(s, dim=0) @ v[first:i + 1, a]
            if gate is not None:
                out[i, a] = out[i, a] * gate[i, a]
    return out.reshape(T, H * dv) @ t[f"{name}.o"].T


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def mamba2(h: torch.Tensor, t: Dict[str, torch.Tensor], name: str, m: dict, eps: float) -> torch.Tensor:
    """A selective state space layer with one decay per head and token: short causal convolution over x | B | C, a state
    ``N x vdim`` per head walked token by token, gate, norm in equal parts, output projection."""
    T = h.shape[0]
    H, P, N, G, taps, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * P
    rows = h @ t[f"{name}.in"].T
    z, xbc, dt = rows[:, :inner], rows[:, inner:2 * inner + 2 * G * N], rows[:, 2 * inner + 2 * G * N:]
    w, b = t[f"{name}.conv"], t[f"{name}.conv.b"]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=F), xbc], dim=0)
    conv = torch.zeros_like(xbc)
    for i in range(T):
        conv[i] = (padded[i:i + taps].T * w).sum(1) + b          # the last column meets the current token
    conv = silu(conv)
    x = conv[:, :inner].reshape(T, H, P)
    B = conv[:, inner:inner + G * N].reshape(T, G, N)
    C = conv[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + t[f"{name}.dt_bias"], beta=1.0, threshold=1e9)
    rate = torch.exp(t[f"{name}.A_log"])
    D = t[f"{name}.D"]
    y = torch.zeros(T, H, P, dtype=F)
    S = torch.zeros(H, N, P, dtype=F)
    for i in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = torch.exp(-rate[a] * dt[i, a]) * S[a] + dt[i, a] * torch.outer(B[i, g], x[i, a])
            y[i, a] = S[a].T @ C[i, g] + D[a] * x[i, a]
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * t[f"{name}.norm"]
    return y @ t[f"{name}.o"].T


def dense_mlp(h: torch.Tensor, t: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    up = h @ t[f"{name}.up"].T + t[f"{name}.up.b"]
    act = 0.5 * up * (1.0 + torch.erf(up / math.sqrt(2.0)))
    return act @ t[f"{name}.down"].T + t[f"{name}.down.b"]


def capped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def router_margins(h: torch.Tensor, t: Dict[str, torch.Tensor], name: str, mlp: dict) -> torch.Tensor:
    """Per row, how far the last chosen expert's logit lies above the first one not chosen (infinite where all are chosen)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    if top >= E:
        return torch.full((h.shape[0],), float("inf"), dtype=F)
    z = torch.sort(h @ t[f"{name}.router"].T + t[f"{name}.router.b"], dim=1, descending=True).values
    return z[:, top - 1] - z[:, top]


def routed_mlp(h: torch.Tensor, t: Dict[str, torch.Tensor], name: str, mlp: dict) -> torch.Tensor:
    """The ``top`` experts with the largest router logits, weighted by the softmax over those logits alone, plus a shared
    expert times a sigmoid of the token."""
    T = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ t[f"{name}.router"].T + t[f"{name}.router.b"]
    out = torch.zeros(T, h.shape[1], dtype=F)
    for i in range(T):
        chosen = torch.topk(logits[i], top).indices
        weights = torch.softmax(logits[i, chosen], dim=0)
        for e, w in zip(chosen.tolist(), weights):
            out[i] += w * capped_expert(h[i:i + 1], t[f"{name}.e{e}.gate"], t[f"{name}.e{e}.up"], t[f"{name}.e{e}.down"],
                                        mlp["expert"]["limit"])[0]
    shared = mlp.get("shared")
    if shared is not None:
        y = capped_expert(h, t[f"{name}.shared.gate"], t[f"{name}.shared.up"], t[f"{name}.shared.down"], shared["limit"])
        out += y * torch.sigmoid(h @ t[f"{name}.shared.sg"].T)
    return out


MIXERS = {"attention": pooled_window_attention, "latent_attention": latent_attention, "mamba2": mamba2}


def read_weights(path: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    import os

    return {k: v.to(F) for k, v in load_file(os.path.join(path, "model.safetensors")).items()}


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens: List[int], residuals: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence from its first position; ``residuals`` collects the stream after every layer,
    ``margins`` every routed layer's ``router_margins``."""
    eps = config["norm"]["eps"]
    x = tensors["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i) if layer.get('weights_of') is not None else i}"
        h = rms_norm(x, tensors[f"{p}.norm1"], eps)
        if f"{p}.shift" in tensors:
            h = token_shift(h, tensors[f"{p}.shift"])
        x = x + MIXERS[layer["type"]](h, tensors, f"{p}.mix", layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, tensors[f"{p}.norm2"], eps)
            if margins is not None and mlp["kind"] != "dense":
                margins.append(router_margins(h, tensors, f"{p}.mlp", mlp))
            x = x + (dense_mlp(h, tensors, f"{p}.mlp") if mlp["kind"] == "dense" else routed_mlp(h, tensors, f"{p}.mlp", mlp))
        if residuals is not None:
            residuals.append(x.clone())
    return rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
