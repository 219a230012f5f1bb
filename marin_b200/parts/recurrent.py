"""Mixers whose memory is a fixed-size state per request instead of a cache that grows: a matrix per head that every
token updates (``StateNeed``), kept in float32 in the request's state slot.

Both walk the tokens a request brings to a step in order, from the state the steps before left (zeros at admission), so
a prompt may be cut anywhere and single decoded tokens take the same path.  Which tokens belong to which request and
which slot they use is read on the device (``ctx.cu_tokens``, ``cache.slots``): single-token steps may be captured.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import ops
from .base import Runtime
from .mixer import Mixer, StateNeed
from .registry import register_mixer
from .spec import TensorSpec


@register_mixer("linear_attention")
class LinearAttention(Mixer):
    """Linear attention with a fixed decay per head and an output gate.

    ``q = silu(W_q x)``, ``k = silu(W_k x)`` (``heads`` x ``dim``), ``v = silu(W_v x)`` (``heads`` x ``vdim``); per head
    ``S_t = decay_h S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t`` (no other scale).  The heads side by side are divided by
    their common root mean square (``norm_eps`` under the root), times the weight ``norm``, times ``sigmoid(W_g x)``, and go
    through ``W_o`` into the residual.  ``decay``: one number per head.
    """

    NAMES = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, decay: Sequence[float], name: str, norm_eps: float = 1e-6,
                 names=None):
        self.hidden, self.heads, self.dim, self.vdim = int(hidden), int(heads), int(dim), int(vdim)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.heads} heads")
        self.name, self.norm_eps = name, float(norm_eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.qk, self.hv = self.heads * self.dim, self.heads * self.vdim
        self.w_in = self.w_o = self.norm_w = self.decay = None

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        return StateNeed((self.heads, self.dim, self.vdim), torch.float32)

    def tensor_specs(self) -> List[TensorSpec]:
        h = self.hidden
        return [TensorSpec(self._n("q"), (self.qk, h)), TensorSpec(self._n("k"), (self.qk, h)), TensorSpec(self._n("v"), (self.hv, h)),
                TensorSpec(self._n("g"), (self.hv, h)), TensorSpec(self._n("o"), (h, self.hv)), TensorSpec(self._n("norm"), (self.hv,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        # one matrix for the four projections of x: q | k | v | g
        self.w_in = rt.matrix(torch.cat([tensors.pop(self._n(p)) for p in "qkvg"], dim=0))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        self.norm_w = rt.f32(tensors.pop(self._n("norm")))
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return super().flops(tokens, pairs) + 4.0 * tokens * self.heads * self.dim * self.vdim

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.linear_attention_jobs(dtype, self.dim, self.vdim)

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        qk, hv = self.qk, self.hv
        ops.stage_name = "q|k|v|g"
        proj = ws.get("lin_proj", (T, 2 * qk + 2 * hv), x.dtype)
        ops.gemm(x, self.w_in, proj)
        ops.stage_name = "recurrence"
        o = ws.get("lin_o", (T, hv), torch.float32)
        # prompt portions 64 tokens at a time on the tensor cores; single tokens (and sizes that kernel is not made for, and
        # the 32-bit path) token by token
        chunked = (ctx.max_query_len > 1 and ops.use_chunked_linear_attention
                   and ops.linear_attention_chunked_supported(x.dtype, self.dim, self.vdim))
        run = ops.linear_attention_chunked if chunked else ops.linear_attention_scan
        run(proj[:, :qk], proj[:, qk:2 * qk], proj[:, 2 * qk:2 * qk + hv], self.decay, cache.state, ctx, cache.slots, o,
            self.heads, self.dim, self.vdim)
        ops.stage_name = "norm, gate"
        gated = ws.get("lin_gated", (T, hv), x.dtype)
        ops.gated_rmsnorm(o, self.norm_w, proj[:, 2 * qk + hv:], "sigmoid", self.norm_eps, gated)
        ops.stage_name = "o"
        ops.gemm(gated, self.w_o, residual, accumulate=True)
        return None


@register_mixer("wkv")
class WKV(Mixer):
    """Time mixing with a decay that depends on the token (RWKV-style).

    With ``x'`` the row before in the sequence (zeros before the first token) each of r, k, v, g, w reads its own mix
    ``x + (x' - x) * mu_s``.  ``r, k, v = W_r, W_k, W_v`` of their mixes (``heads`` x ``dim``), ``gate = silu(W_g mix_g)``,
    ``decay = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0))`` per head and key channel.  Per head
    ``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t`` (the bonus ``u`` for the current token only), then
    ``S_t = diag(decay_t) S_(t-1) + k_t v_t^T``.  Each head's ``o`` is divided by its root mean square (``norm_eps`` under the
    root); heads side by side, times ``norm``, times the gate, through ``W_o`` into the residual.  The state of a request is
    the matrices of all heads and the last row of ``x`` it has seen.
    """

    NAMES = {"r": "r", "k": "k", "v": "v", "g": "g", "o": "o", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u", "norm": "norm",
             "mu": "mu"}
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, hidden: int, heads: int, dim: int, decay_rank: int, name: str, norm_eps: float = 1e-6, names=None):
        self.hidden, self.heads, self.dim, self.rank = int(hidden), int(heads), int(dim), int(decay_rank)
        self.name, self.norm_eps = name, float(norm_eps)
        self.names = dict(self.NAMES, **(names or {}))
        self.n = self.heads * self.dim
        self.matrix_floats = self.heads * self.dim * self.dim

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        return StateNeed((self.matrix_floats + self.hidden,), torch.float32)

    def tensor_specs(self) -> List[TensorSpec]:
        h, n = self.hidden, self.n
        specs = [TensorSpec(f"{self._n('mu')}.{s}", (h,), "bias") for s in self.MIXES]
        specs += [TensorSpec(self._n(p), (n, h)) for p in "rkvg"]
        specs += [TensorSpec(self._n("w1"), (self.rank, h)), TensorSpec(self._n("w2"), (n, self.rank)),
                  TensorSpec(self._n("w0"), (n,), "bias"), TensorSpec(self._n("u"), (self.heads, self.dim), "bias"),
                  TensorSpec(self._n("norm"), (n,), "norm"), TensorSpec(self._n("o"), (h, n))]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.mu = rt.f32(torch.stack([tensors.pop(f"{self._n('mu')}.{s}").to(torch.float32) for s in self.MIXES]))
        self.w_r, self.w_k, self.w_v, self.w_g = (rt.matrix(tensors.pop(self._n(p))) for p in "rkvg")
        self.w_1, self.w_2 = rt.matrix(tensors.pop(self._n("w1"))), rt.matrix(tensors.pop(self._n("w2")))
        self.w0 = rt.f32(tensors.pop(self._n("w0")))
        self.u = rt.f32(tensors.pop(self._n("u"))).reshape(-1)
        self.norm_w = rt.f32(tensors.pop(self._n("norm")))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return super().flops(tokens, pairs) + 6.0 * tokens * self.heads * self.dim * self.dim

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.library_jobs("mb_activations", "mb_recurrent")

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        n = self.n
        state = cache.state[:, : self.matrix_floats]
        carry = cache.state[:, self.matrix_floats:]
        ops.stage_name = "token shift"
        mixes = ws.get("wkv_mixes", (len(self.MIXES), T, self.hidden), x.dtype)
        ops.shift_mix(x, carry, ctx, cache.slots, self.mu, mixes)
        ops.stage_name = "r, k, v, g"
        rkvg = ws.get("wkv_rkvg", (4, T, n), x.dtype)
        for i, w in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            ops.gemm(mixes[i], w, rkvg[i])
        ops.stage_name = "decay"
        low = ws.get("wkv_low", (T, self.rank), x.dtype)
        ops.gemm(mixes[4], self.w_1, low)
        ops.tanh_cap(low, 1.0)
        wraw = ws.get("wkv_wraw", (T, n), torch.float32)
        ops.gemm(low, self.w_2, wraw)
        ops.stage_name = "recurrence"
        o = ws.get("wkv_o", (T, n), torch.float32)
        ops.wkv_scan(rkvg[0], rkvg[1], rkvg[2], wraw, self.w0, self.u, state, carry, x, ctx, cache.slots, o, self.heads, self.dim)
        ops.stage_name = "norm, gate"
        out = ws.get("wkv_out", (T, n), x.dtype)
        ops.head_norm_gate(o, self.norm_w, rkvg[3], self.norm_eps, out, self.heads, self.dim)
        ops.stage_name = "o"
        ops.gemm(out, self.w_o, residual, accumulate=True)
        return None


@register_mixer("mamba2")
class Mamba2(Mixer):
    """A selective state space layer with one decay per head and token (Mamba-2: Dao, Gu, "Transformers are SSMs: Generalized
    Models and Efficient Algorithms Through Structured State Space Duality").

    With ``inner = heads * v_head_dim``, N = ``state`` and G = ``groups``, ``W_in h`` is laid out as ``z [inner] | x [inner] |
    B [G N] | C [G N] | dt [heads]``.  x, B and C together pass a causal convolution per channel of ``taps`` taps (weight
    ``[channels, taps]`` whose last column meets the current token, a bias) and silu.  ``dt <- softplus(dt + dt_bias)``; per
    head (head ``a`` uses group ``a // (heads / G)``): ``S_t = exp(-exp(rate_a) dt) S_(t-1) + dt B_t x_t^T`` (``N x v_head_dim``),
    ``y_t = S_t^T C_t + skip_a x_t``.  ``y`` (heads side by side) times ``silu(z)`` is divided by its root mean square in
    ``norm_groups`` equal parts (each by its own), times a weight, then ``W_o`` into the residual.  A request's state is the
    matrices of all heads (float32, zero at first) and the convolution's last ``taps - 1`` inputs: two slots' worth, kept as
    two needs."""

    NAMES = {"in": "in_proj", "conv": "conv", "conv_bias": "conv.bias", "dt_bias": "dt_bias", "rate": "A_log", "skip": "D", "norm": "norm",
             "o": "out_proj"}

    def __init__(self, hidden: int, heads: int, v_head_dim: int, state: int, groups: int, taps: int, name: str, norm_groups: int = 1,
                 norm_eps: float = 1e-6, names=None):
        self.hidden, self.heads, self.v_head_dim, self.state = int(hidden), int(heads), int(v_head_dim), int(state)
        self.groups, self.taps, self.norm_groups = int(groups), int(taps), int(norm_groups)
        self.name, self.norm_eps = name, float(norm_eps)
        if self.heads % self.groups != 0:
            raise ValueError(f"mamba2: {heads} heads cannot share {groups} groups evenly")
        self.inner = self.heads * self.v_head_dim
        if self.inner % self.norm_groups != 0:
            raise ValueError(f"mamba2: the norm's {norm_groups} parts do not divide {self.inner}")
        if self.state > 256 or self.taps > 64:
            raise ValueError("mamba2: a state above 256 rows or more than 64 taps is not supported")
        self.channels = self.inner + 2 * self.groups * self.state
        self.in_dim = 2 * self.inner + 2 * self.groups * self.state + self.heads
        self.names = dict(self.NAMES, **(names or {}))

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        return (StateNeed((self.heads, self.state, self.v_head_dim), torch.float32),
                StateNeed((max(self.taps - 1, 1), self.channels), torch.float32))

    def tensor_specs(self) -> List[TensorSpec]:
        h = self.hidden
        return [TensorSpec(self._n("in"), (self.in_dim, h)), TensorSpec(self._n("conv"), (self.channels, self.taps), "bias", 1.0 / self.taps),
                TensorSpec(self._n("conv_bias"), (self.channels,), "bias"), TensorSpec(self._n("dt_bias"), (self.heads,), "bias"),
                TensorSpec(self._n("rate"), (self.heads,), "bias"), TensorSpec(self._n("skip"), (self.heads,), "bias", 1.0),
                TensorSpec(self._n("norm"), (self.inner,), "norm"), TensorSpec(self._n("o"), (h, self.inner))]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.w_in = rt.matrix(tensors.pop(self._n("in")))
        self.conv_w, self.conv_b = rt.f32(tensors.pop(self._n("conv"))), rt.f32(tensors.pop(self._n("conv_bias")))
        self.dt_bias, self.rate, self.skip = (rt.f32(tensors.pop(self._n(k))) for k in ("dt_bias", "rate", "skip"))
        self.norm_w = rt.f32(tensors.pop(self._n("norm")))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return super().flops(tokens, pairs) + tokens * (6.0 * self.heads * self.state * self.v_head_dim + 2.0 * self.channels * self.taps)

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.library_jobs("mb_ssm")

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        matrices, kept = cache
        ops.stage_name = "z|x|B|C|dt"
        rows = ws.get("ssm_rows", (T, self.in_dim), x.dtype)
        ops.gemm(x, self.w_in, rows)
        ops.stage_name = "convolution"
        xbc = ws.get("ssm_xbc", (T, self.channels), x.dtype)
        ops.ssm_conv(rows, self.inner, self.conv_w, self.conv_b, kept.state if self.taps > 1 else kept.state[:, :0], ctx, kept.slots, xbc)
        ops.stage_name = "recurrence"
        y = ws.get("ssm_y", (T, self.inner), torch.float32)
        ops.ssm_scan(xbc, rows, self.inner + self.channels, self.dt_bias, self.rate, self.skip, matrices.state, ctx, matrices.slots, y,
                     self.heads, self.v_head_dim, self.state, self.groups)
        ops.stage_name = "gate, norm"
        out = ws.get("ssm_out", (T, self.inner), x.dtype)
        ops.ssm_gate_norm(y, rows, 0, self.norm_w, self.norm_eps, self.norm_groups, out)
        ops.stage_name = "o"
        ops.gemm(out, self.w_o, residual, accumulate=True)
        return None
