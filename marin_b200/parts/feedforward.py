"""Feed-forward parts.

Interface: ``forward(x, ctx, residual)`` reads ``x`` ``[T, hidden]`` (activation dtype) and
**adds** its output into ``residual`` (float32 ``[T, hidden]``).  A routed feed-forward
(experts) has the same interface; what it routes on is its own business.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Part, Runtime, element_size
from .registry import register_feedforward
from .spec import TensorSpec


class FeedForward(Part):
    #: True if ``forward`` takes ``x`` as ``ops.NormedRows`` too, and a keyword ``then_norm`` (an ``ops.NormOut``),
    #: returning ``ops.NormedRows`` if its last product carried that norm and None otherwise (see ``Mixer``).
    couples_norm = False
    #: as ``Mixer.capturable``: single-token steps launch the same kernels whatever the batch holds, without a wait
    #: on the host (a routed feed-forward that reads its routing back to the host says False)
    capturable = True

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        raise NotImplementedError


@register_feedforward("swiglu")
class SwiGLU(FeedForward):
    """``down( g / (1 + exp(-g)) * u )`` with ``g = x W_gate^T`` and ``u = x W_up^T``, no bias
    (crates/model/src/qwen3/mlp.rs:22-37, crates/tensor/src/silu.rs:18)."""

    def __init__(self, hidden: int, intermediate: int, name: str):
        self.hidden, self.intermediate, self.name = int(hidden), int(intermediate), name
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        n, h, i = self.name, self.hidden, self.intermediate
        return [
            TensorSpec(f"{n}.gate_proj.weight", (i, h)),
            TensorSpec(f"{n}.up_proj.weight", (i, h)),
            TensorSpec(f"{n}.down_proj.weight", (h, i)),
        ]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        n = self.name
        gate, up = tensors.pop(f"{n}.gate_proj.weight"), tensors.pop(f"{n}.up_proj.weight")
        # One matrix for both projections.  Where the tensor-core kernel can apply the activation in its epilogue
        # the rows are interleaved in blocks of 16 (gate, up, gate, ...) so that a gate value and its up value
        # meet in one warp; otherwise gate rows come first, then up rows.
        self.fused = ops.can_fuse_swiglu(rt.dtype, self.hidden, self.intermediate)
        if self.fused:
            self.w_gate_up = rt.matrix(ops.interleave_gate_up(gate, up))
        else:
            self.w_gate_up = rt.matrix(torch.cat([gate, up], dim=0))
        self.w_down = rt.matrix(tensors.pop(f"{n}.down_proj.weight"))

    couples_norm = True

    def forward(self, x, ctx, residual: torch.Tensor, then_norm=None):
        T = x.shape[0]
        ws = ctx.workspace
        act = ws.get("ffn_act", (T, self.intermediate), x.dtype)
        ops.stage_name = "gate|up, SwiGLU"
        if self.fused:
            ops.gemm_swiglu(x, self.w_gate_up, act, ws)
        else:
            gate_up = ws.get("gate_up", (T, 2 * self.intermediate), x.dtype)
            ops.gemm(x, self.w_gate_up, gate_up)
            ops.swiglu(gate_up, act)
        ops.stage_name = "down"
        return ops.gemm(act, self.w_down, residual, accumulate=True, then_norm=then_norm)


@register_feedforward("polynorm_mlp")
class PolyNormMLP(FeedForward):
    """``down( act( x W_up^T ) )`` with ``act = a N(z) + b N(z^2) + c N(z^3) + e``: powers element by element, ``N`` a token's
    row divided by its root mean square (``eps`` under the root), the four numbers learned (tensor ``<name>.<act>``).  The
    sums run in float32; in bfloat16 mode the up projection is kept in float32 for them."""

    def __init__(self, hidden: int, intermediate: int, name: str, eps: float, names=("up", "down", "act")):
        self.hidden, self.intermediate, self.name, self.eps = int(hidden), int(intermediate), name, float(eps)
        self.up_name, self.down_name, self.act_name = (f"{name}.{n}" for n in names)
        self.w_up = self.w_down = self.coef = None

    def tensor_specs(self) -> List[TensorSpec]:
        h, i = self.hidden, self.intermediate
        return [TensorSpec(self.up_name, (i, h)), TensorSpec(self.down_name, (h, i)), TensorSpec(self.act_name, (4,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.w_up = rt.matrix(tensors.pop(self.up_name))
        self.w_down = rt.matrix(tensors.pop(self.down_name))
        self.coef = rt.f32(tensors.pop(self.act_name))

    def forward(self, x, ctx, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        ops.stage_name = "up"
        z = ws.get("ffn_up", (T, self.intermediate), torch.float32)
        ops.gemm(x, self.w_up, z)
        ops.stage_name = "polynorm"
        act = ws.get("ffn_act", (T, self.intermediate), x.dtype)
        ops.polynorm(z, self.coef, self.eps, act)
        ops.stage_name = "down"
        ops.gemm(act, self.w_down, residual, accumulate=True)
        return None


@register_feedforward("act_mlp")
class ActMLP(FeedForward):
    """``down( act( x W_up^T (+ b_up) ) ) (+ b_down)`` without a gate; ``activation`` "relu2": the square of relu, "gelu": the
    exact gelu ``z (1 + erf(z / sqrt 2)) / 2``, "gelu_tanh": its tanh form, element by element.  ``bias``: both projections have
    one (``bias_names``)."""

    ACTIVATIONS = ("relu2", "gelu", "gelu_tanh")

    def __init__(self, hidden: int, intermediate: int, name: str, activation: str = "relu2", names=("up", "down"), bias: bool = False,
                 bias_names=("up.bias", "down.bias")):
        self.hidden, self.intermediate, self.name, self.activation = int(hidden), int(intermediate), name, activation
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"act_mlp: unknown activation {activation!r}")
        self.up_name, self.down_name = (f"{name}.{n}" for n in names)
        self.bias = bool(bias)
        self.up_bias_name, self.down_bias_name = (f"{name}.{n}" for n in bias_names)
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        h, i = self.hidden, self.intermediate
        specs = [TensorSpec(self.up_name, (i, h)), TensorSpec(self.down_name, (h, i))]
        if self.bias:
            specs += [TensorSpec(self.up_bias_name, (i,), "bias"), TensorSpec(self.down_bias_name, (h,), "bias")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.w_up = rt.matrix(tensors.pop(self.up_name))
        self.w_down = rt.matrix(tensors.pop(self.down_name))
        if self.bias:
            self.b_up, self.b_down = rt.f32(tensors.pop(self.up_bias_name)), rt.f32(tensors.pop(self.down_bias_name))

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.library_jobs("mb_activations")

    def forward(self, x, ctx, residual: torch.Tensor):
        T = x.shape[0]
        act = ctx.workspace.get("ffn_act", (T, self.intermediate), x.dtype)
        ops.stage_name = "up, activation"
        if self.activation == "relu2" and not self.bias:
            ops.gemm_act(x, self.w_up, act, self.activation)
        else:
            ops.gemm(x, self.w_up, act)
            if self.activation == "relu2":
                ops.bias_act(act, self.b_up, None)
                ops.relu2(act)
            else:
                ops.bias_act(act, self.b_up, self.activation)
        ops.stage_name = "down"
        ops.gemm(act, self.w_down, residual, accumulate=True)
        if self.bias:
            ops.add_row_bias(residual, self.b_down)
        return None


class CappedGLU(FeedForward):
    """``down( g sigmoid(alpha g) (u + shift) )`` with ``g = min(x W_gate^T, limit)`` and ``u = clamp(x W_up^T, -limit, limit)``, no
    biases; ``scaled``: the result times ``sigmoid(x . w_s)``, one number per token (tensor ``[1, hidden]``): its row rides in
    the same product as gate and up, and since the down projection is linear the number multiplies the activation's rows."""

    def __init__(self, hidden: int, intermediate: int, name: str, limit: float, alpha: float, shift: float, scaled: bool, names):
        self.hidden, self.intermediate, self.name = int(hidden), int(intermediate), name
        self.limit, self.alpha, self.shift, self.scaled = float(limit), float(alpha), float(shift), bool(scaled)
        self.gate_name, self.up_name, self.down_name, self.scale_name = (f"{name}.{n}" for n in names)
        self.w_in = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        h, i = self.hidden, self.intermediate
        specs = [TensorSpec(self.gate_name, (i, h)), TensorSpec(self.up_name, (i, h)), TensorSpec(self.down_name, (h, i))]
        if self.scaled:
            specs.append(TensorSpec(self.scale_name, (1, h)))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        parts = [tensors.pop(self.gate_name), tensors.pop(self.up_name)]
        if self.scaled:
            parts.append(tensors.pop(self.scale_name).reshape(1, self.hidden))
            # (rows up to a multiple of 8, so that every product kernel takes the matrix)
            parts.append(torch.zeros((-(2 * self.intermediate + 1)) % 8, self.hidden, dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = rt.matrix(torch.cat(parts, dim=0))
        self.w_down = rt.matrix(tensors.pop(self.down_name))

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.library_jobs("mb_activations")

    def forward(self, x, ctx, residual: torch.Tensor):
        T, ff = x.shape[0], self.intermediate
        ws = ctx.workspace
        ops.stage_name = "shared gate|up"
        rows = ws.get("glu_rows", (T, self.w_in.shape[0]), x.dtype)
        ops.gemm(x, self.w_in, rows)
        act = ws.get("glu_act", (T, ff), x.dtype)
        ops.glu_capped(rows, ff, act, self.limit, self.alpha, self.shift, 2 * ff if self.scaled else -1)
        ops.stage_name = "shared down"
        ops.gemm(act, self.w_down, residual, accumulate=True)
        return None


@register_feedforward("routed_experts")
class RoutedExperts(FeedForward):
    """A mixture of small feed-forwards of which every token uses ``top``: ``out = sum_e expert_e(.)`` over the chosen ones.

    Router (``router="learned"``): ``z = h W_r^T`` in float32 (the matrix is kept in float32), scores ``sigmoid(z)``
    (``score="sigmoid"``) or the softmax of ``z`` over all experts; the ``top`` largest are chosen (the lower expert among
    equals) and their scores are the weights, divided by their sum if ``renormalize``.  ``router="table"``: no scores at all;
    an integer table ``[vocab, top]`` names the experts of every token id, each with the weight ``1 / top`` (the choice
    depends on the token alone, not on the layer's input).  ``weight_on`` "input": the weight multiplies what the expert
    reads, ``expert(w h)``, so it passes through the activation; "output": ``w expert(h)``.  Experts have no biases;
    ``activation`` "swiglu": ``down( silu(gate x) * (up x) )``; "relu2": no gate, ``down( relu(up x)^2 )``.
    ``shared_intermediate``: one more expert of that width (same form, tensors ``shared.*``) that every token uses with
    weight 1.  Nothing is read back to the host: routing, grouping and the experts' products are kernels over device arrays,
    so single-token steps can be captured in graphs.
    ``names``: the router's (or table's) tensor and the pattern of an expert's tensors inside ``name`` (``{e}`` the expert's
    number)."""

    NAMES = {"router": "router.weight", "router_bias": "router.bias", "table": "table", "gate": "experts.{e}.gate_proj.weight",
             "up": "experts.{e}.up_proj.weight", "down": "experts.{e}.down_proj.weight", "shared_gate": "shared.gate", "shared_up": "shared.up",
             "shared_down": "shared.down", "shared_scale": "shared.scale"}

    def __init__(self, hidden: int, intermediate: int, experts: int, top: int, name: str, score: str = "sigmoid",
                 renormalize: bool = False, weight_on: str = "input", names=None, router: str = "learned", vocab: int = 0,
                 activation: str = "swiglu", shared_intermediate: Optional[int] = None, router_bias: bool = False,
                 act_limit: float = 0.0, act_alpha: float = 1.0, act_shift: float = 0.0, shared_limit: Optional[float] = None,
                 shared_scaled: bool = False):
        self.hidden, self.intermediate, self.experts, self.top, self.name = int(hidden), int(intermediate), int(experts), int(top), name
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"routed_experts: top {top} of {experts} experts")
        if score not in ops.SCORE_MODES or weight_on not in ("input", "output"):
            raise ValueError(f"routed_experts: score {score!r} / weight_on {weight_on!r}")
        if router not in ("learned", "table") or activation not in ops.EXPERT_ACTIVATIONS:
            raise ValueError(f"routed_experts: router {router!r} / activation {activation!r}")
        if router == "table" and int(vocab) <= 0:
            raise ValueError("routed_experts: a table over the token ids needs the vocabulary's size")
        self.score, self.renormalize, self.weight_on = score, bool(renormalize), weight_on
        self.routing, self.vocab, self.activation = router, int(vocab), activation
        self.gated = activation != "relu2"
        # "glu_capped": g sigmoid(alpha g) (u + shift) with g <- min(g, limit), u <- clamp(u, -limit, limit); the softmax of the
        # chosen logits alone is score "softmax" with ``renormalize`` (the common denominator cancels)
        self.form = (float(act_limit), float(act_alpha), float(act_shift)) if activation == "glu_capped" else None
        self.router_bias = bool(router_bias)
        self.names = dict(self.NAMES, **(names or {}))
        self.router = self.router_b = self.table = self.w_gate_up = self.w_down = None
        self.shared = None
        if shared_intermediate:
            if activation == "glu_capped":
                self.shared = CappedGLU(hidden, int(shared_intermediate), name, self.form[0] if shared_limit is None else float(shared_limit),
                                        self.form[1], self.form[2], shared_scaled,
                                        tuple(self.names[k] for k in ("shared_gate", "shared_up", "shared_down", "shared_scale")))
            elif self.gated:
                self.shared = SwiGLU(hidden, int(shared_intermediate), f"{name}.shared")
            else:
                self.shared = ActMLP(hidden, int(shared_intermediate), name, activation,
                                     names=(self.names["shared_up"], self.names["shared_down"]))

    def _n(self, key: str, e: int = 0) -> str:
        return f"{self.name}.{self.names[key].format(e=e)}"

    def tensor_specs(self) -> List[TensorSpec]:
        h, i = self.hidden, self.intermediate
        specs = []
        for e in range(self.experts):
            if self.gated:
                specs.append(TensorSpec(self._n("gate", e), (i, h)))
            specs += [TensorSpec(self._n("up", e), (i, h)), TensorSpec(self._n("down", e), (h, i))]
        if self.routing == "table":
            specs.append(TensorSpec(self._n("table"), (self.vocab, self.top), "int_table", limit=self.experts))
        else:
            specs.append(TensorSpec(self._n("router"), (self.experts, h), "bias"))
            if self.router_bias:
                specs.append(TensorSpec(self._n("router_bias"), (self.experts,), "bias"))
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        # one tensor per kind for all experts: an expert's gate and up rows in one matrix, [E, 2 ff, h]; down [E, h, ff].  Where
        # the dense product's SwiGLU epilogue applies, the rows alternate in blocks of 16 as it reads them, so that an expert
        # with many tokens can go to that product as it is; otherwise gate rows come first.  Without a gate: up alone, [E, ff, h].
        if self.gated:
            self.interleaved = self.form is None and ops.can_fuse_swiglu(rt.dtype, self.hidden, self.intermediate)
            join = ops.interleave_gate_up if self.interleaved else (lambda g, u: torch.cat([g, u], dim=0))
            self.w_gate_up = rt.matrix(torch.stack([join(tensors.pop(self._n("gate", e)), tensors.pop(self._n("up", e)))
                                                    for e in range(self.experts)]))
        else:
            self.interleaved = False
            self.w_gate_up = rt.matrix(torch.stack([tensors.pop(self._n("up", e)) for e in range(self.experts)]))
        self.w_down = rt.matrix(torch.stack([tensors.pop(self._n("down", e)) for e in range(self.experts)]))
        if self.routing == "table":
            table = tensors.pop(self._n("table")).to(torch.int32)
            if int(table.min()) < 0 or int(table.max()) >= self.experts:
                raise ValueError(f"{self._n('table')}: names experts outside 0..{self.experts - 1}")
            self.table = table.to(rt.device).contiguous()
        else:
            self.router = rt.f32(tensors.pop(self._n("router")))
            if self.router_bias:
                self.router_b = rt.f32(tensors.pop(self._n("router_bias")))
        if self.shared is not None:
            self.shared.load(tensors, rt)
        self.rt = rt

    def bytes_read(self, tokens: int, dtype) -> int:
        """Only the experts that some token chose are read: at most ``tokens * top`` of them."""
        per_expert = (3 if self.gated else 2) * self.hidden * self.intermediate * element_size(dtype)
        routing = tokens * self.top * 4 if self.routing == "table" else self.experts * self.hidden * 4
        shared = self.shared.bytes_read(tokens, dtype) if self.shared is not None else 0
        return min(self.experts, tokens * self.top) * per_expert + routing + shared

    def flops(self, tokens: int, pairs: int = 0) -> float:
        routing = self.experts if self.routing == "learned" else 0
        shared = self.shared.flops(tokens, pairs) if self.shared is not None else 0.0
        return 2.0 * tokens * self.hidden * (routing + (3 if self.gated else 2) * self.top * self.intermediate) + shared

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        jobs = ops.moe_jobs(dtype, self.hidden, self.intermediate)
        if not self.gated or self.form is not None:
            jobs.update(ops.library_jobs("mb_activations"))
        return jobs

    def forward(self, x, ctx, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        chosen = ws.get("moe_experts", (T, self.top), torch.int32)
        weights = ws.get("moe_weights", (T, self.top), torch.float32)
        ops.stage_name = "router"
        if self.routing == "table":
            ops.moe_table_route(ctx.token_ids, self.table, self.experts, chosen, weights)
        else:
            ops.moe_route(x, self.router, chosen, weights, self.score, self.renormalize, self.router_b)
        ops.stage_name = "experts"
        ops.moe_experts(x, self.w_gate_up, self.w_down, chosen, weights, residual, self.weight_on == "input", ws, self.interleaved,
                        self.activation, self.form)
        if self.shared is not None:
            self.shared.forward(x, ctx, residual)
        return None
