"""Vogunex as data: pre-norm layers over one residual stream; in front of every mixer a token shift; each layer with one of
three mixers and a dense or routed feed-forward.

* ``attention``: grouped-query softmax attention with biases, part of every head rotated in half-split pairs, q and k divided
  by their root mean square per head, scores capped by a tanh, a window of single positions plus one pooled key and value per
  block of positions that lies wholly before it, the heads' softmax weights mixed by a learned matrix.
* ``latent_attention``: attention over a latent that keys and values share, queries through a latent of their own, one
  rotated key part for all heads, a window, a sigmoid gate per head.
* ``mamba2``: a selective state space layer (a short causal convolution, one decay per head and token, a gated norm in parts).
* feed-forward: dense with biases and the erf gelu, or experts chosen by a learned router (softmax over the chosen logits)
  with capped gate and up projections, plus a shared expert times a sigmoid of the token.

A layer with ``weights_of`` is a second run of that layer's block in the schedule, with a cache or state of its own.
Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2`` / ``shift``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Optional

from ..config.vogunex import VogunexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .registry import register_architecture

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "talk": "talk"}
LATENT_NAMES = {"q_down": "dq", "q_norm": "dq.norm", "q": "uq", "dkv": "dkv", "c_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o", "g": "g"}
SSM_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "rate": "A_log", "skip": "D", "norm": "norm", "o": "o"}
EXPERT_NAMES = {"router": "router", "router_bias": "router.b", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
                "shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down", "shared_scale": "shared.sg"}
#: what the design fixes of the experts' activation ``g sigmoid(alpha g) (u + shift)``
EXPERT_ALPHA, EXPERT_SHIFT = 1.702, 1.0


def _position(rot: Optional[dict], width: int, neighbours: bool) -> PartSpec:
    if rot is None:
        return PartSpec("none", {})
    return PartSpec("rope", {"head_dim": width, "theta": rot["base"], "rotary_dim": rot["dims"], "interleaved": neighbours})


def _mixer(kind: str, m: dict, h: int, eps: float) -> PartSpec:
    mask = m.get("mask")
    if kind == "attention":
        return PartSpec("pooled_attention", {
            "hidden": h, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
            "scale": m["scale"], "bias": True, "qk_norm": True, "norm_eps": eps, "position": _position(m["rot"], m["dim"], False),
            "window": mask["size"] if mask is not None else None, "pool": mask.get("pool") if mask is not None else None,
            "softcap": m["softcap"], "talk": True, "names": ATTENTION_NAMES})
    if kind == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden": h, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"], "norm_eps": eps,
            "position": _position(m["rot"], m["rot_dim"], True), "window": mask["size"] if mask is not None else None,
            "gate": "head", "sink": False, "names": LATENT_NAMES})
    return PartSpec("mamba2", {"hidden": h, "heads": m["heads"], "v_head_dim": m["vdim"], "state": m["state"], "groups": m["groups"],
                               "taps": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": eps, "names": SSM_NAMES})


def _feedforward(mlp: Optional[dict], h: int) -> Optional[PartSpec]:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("act_mlp", {"hidden": h, "intermediate": mlp["ff"], "activation": "gelu", "bias": True,
                                    "names": ("up", "down"), "bias_names": ("up.b", "down.b")})
    shared = mlp["shared"]
    return PartSpec("routed_experts", {
        "hidden": h, "intermediate": mlp["expert"]["ff"], "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
        "score": "softmax", "renormalize": True, "router_bias": True, "weight_on": "output", "activation": "glu_capped",
        "act_limit": mlp["expert"]["limit"], "act_alpha": EXPERT_ALPHA, "act_shift": EXPERT_SHIFT,
        "shared_intermediate": shared["ff"] if shared is not None else None,
        "shared_limit": shared["limit"] if shared is not None else None, "shared_scaled": shared is not None, "names": EXPERT_NAMES})


def build_spec(cfg: VogunexConfig) -> ModelSpec:
    h = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"dim": h, "eps": cfg.norm_eps, "tensor": ""})
    layers, schedule, block_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        block_of[i] = len(layers)
        mixer = PartSpec("token_shifted", {"hidden": h, "tensor": f"l{i}.shift", "inner": _mixer(layer.type, layer.mixer, h, cfg.norm_eps)})
        layers.append(LayerSpec(block="prenorm", norm=norm, mixer=mixer, feedforward=_feedforward(layer.mlp, h), prefix=f"l{i}",
                                names={"norm1": "norm1", "mixer": "mix", "norm2": "norm2", "feedforward": "mlp"}))
    for i, layer in enumerate(cfg.layers):
        schedule.append(ScheduleEntry(block_of[layer.weights_of if layer.weights_of is not None else i]))
    return ModelSpec(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "embed", "tensor": "embed", "scale": cfg.embedding_scale}),
        final_norm=PartSpec("rmsnorm", {"dim": h, "eps": cfg.norm_eps, "name": "final.norm", "tensor": ""}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "head", "tied": False, "tensor": "head"}),
        layers=layers,
        schedule=schedule,
    )


register_architecture(VogunexConfig.ARCHITECTURE, VogunexConfig.MODEL_TYPE, VogunexConfig, build_spec)
