"""Mixers: the parts that let tokens see other tokens.

Interface every mixer has (a test can register its own):

``cache_need()`` → what it keeps between steps: a :class:`PagedKV` (keys and values
in pages, all of them or a window), a :class:`StateNeed` (fixed-size per-request
state), or None.

``forward(x, ctx, cache, residual)`` → reads ``x`` ``[T, hidden]`` (activation dtype),
mixes over each request's tokens and what ``cache`` holds, and **adds** its output
into ``residual`` (float32 ``[T, hidden]``).  ``ctx`` is the step's
:class:`marin_b200.engine.context.StepContext`; ``cache`` is this run's view of the
cache (:class:`marin_b200.cache.manager.PagedView` or ``StateView``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops
from .base import Part, Runtime, element_size
from .registry import lookup, register_mixer
from .spec import PartSpec, TensorSpec


@dataclass(frozen=True)
class PagedKV:
    """Keys and values of ``kv_heads`` heads of ``head_dim`` per position, kept in pages.
    ``window`` = how many of the latest positions are ever read again (None: all).
    ``v_head_dim``: the size of a value head where it differs from a key head's."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    #: True: a position's values are the first ``v_head_dim`` elements of its key row (a latent that keys and values share);
    #: no value pages are kept, and the mixer's view hands the key pages out as values too
    values_in_keys: bool = False
    #: > 0: beside every position's row the cache keeps one key and one value for each whole block of ``pooled`` positions
    #: (their means).  A block's row lies in the page that holds the block's last position, at ``(offset of that position)
    #: // pooled``, so a page has ``ceil(page_size / pooled)`` such rows and the pooled rows need no block table of their own;
    #: the pages of such a group are kept however old (``window`` must be None)
    pooled: int = 0
    #: with ``pooled``: how many of the latest positions a reader looks at one by one (what lies before them, by blocks)
    pooled_window: int = 0

    def __post_init__(self):
        if self.pooled and self.window is not None:
            raise ValueError("a cache that keeps pooled blocks in its pages cannot give pages back behind a window")

    @property
    def value_dim(self) -> int:
        return self.v_head_dim if self.v_head_dim is not None else self.head_dim

    def pooled_rows(self, page_size: int) -> int:
        """Pooled rows a page of ``page_size`` positions holds (0 without pooling)."""
        return -(-page_size // self.pooled) if self.pooled else 0

    def bytes_per_token(self, dtype: torch.dtype, page_size: int = 0) -> int:
        """Bytes one position of one layer holds in the cache (keys and values; with ``page_size`` given, its share of the
        page's pooled rows too)."""
        row = self.kv_heads * (self.head_dim + (0 if self.values_in_keys else self.value_dim)) * element_size(dtype)
        if self.pooled and page_size:
            return row + -(-row * self.pooled_rows(page_size) // page_size)
        return row

    def bytes_read(self, context: int, dtype: torch.dtype) -> int:
        """Bytes one decoded token reads of a sequence of ``context`` positions."""
        kept = context if self.window is None else min(context, self.window)
        if self.pooled and self.pooled_window:
            kept = min(context, self.pooled_window) + max(0, context - self.pooled_window) // self.pooled
        return kept * self.bytes_per_token(dtype)


@dataclass(frozen=True)
class StateNeed:
    """A fixed-size state per request: ``shape`` elements of ``dtype``, zeroed when a request starts."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32

    def bytes(self) -> int:
        count = 1
        for s in self.shape:
            count *= int(s)
        return count * element_size(self.dtype)

    def bytes_read(self, context: int, dtype: torch.dtype) -> int:
        return self.bytes()


class Mixer(Part):
    #: True if ``forward`` takes ``x`` as ``ops.NormedRows`` too, and a keyword ``then_norm`` (an ``ops.NormOut``:
    #: the norm wanted of the updated residual), returning ``ops.NormedRows`` if its last product carried that norm
    #: and None otherwise.  A block couples norms only between parts that both say so.
    couples_norm = False
    #: True if a step in which every request brings one token may be captured in a CUDA graph and replayed for other
    #: requests of the same number: ``forward`` then launches the same kernels whatever the lengths and slots are,
    #: reads them from ``ctx``'s device tensors only (never ``ctx.spans`` or another host value), and waits for
    #: nothing on the host.  The step function captures graphs only for models whose parts all say so.  Rows that
    #: pad a captured batch stand for empty requests: length 0, the spare state slot (see ``CacheManager``).
    capturable = True

    def cache_need(self):
        return None

    def decode_plan_key(self):
        """Mixers that answer the same (hashable) key share one decode plan per captured graph; None: no plan."""
        return None

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        """What this mixer fixes ahead for single-token steps of ``requests`` requests whose sequences are at most
        ``span`` long: how it splits the work and the scratch memory it then needs.  A captured graph owns the plan;
        ``forward`` finds it as ``ctx.decode_plans[self.decode_plan_key()]``."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache, residual: torch.Tensor) -> None:
        raise NotImplementedError


@register_mixer("gqa_attention")
class GQAttention(Mixer):
    """Causal grouped-query attention over the paged cache.

    ``q,k,v = x W^T`` (no bias); optional per-head RMSNorm of q and k over ``head_dim``
    *before* the rotation; keys (normed, rotated) and values (raw) go to the cache; query
    head ``h`` reads kv head ``h // (heads // kv_heads)``; scores scaled by
    ``1/sqrt(head_dim)``; softmax in float32 over positions ``0..=pos`` (or the last
    ``window``); output through ``o_proj`` added to the residual
    (crates/model/src/qwen3/layer.rs:59-88, crates/tensor/src/attention.rs:148-169).
    """

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, name: str,
                 position: PartSpec, qk_norm: bool = True, norm_eps: float = 1e-6,
                 window: Optional[int] = None, scale: Optional[float] = None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"{heads} heads cannot share {kv_heads} kv heads evenly")
        self.name, self.qk_norm, self.norm_eps = name, bool(qk_norm), float(norm_eps)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = lookup("position", position.kind)(**position.params)
        self.q_dim, self.kv_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.w_qkv = self.w_o = self.q_weight = self.k_weight = None

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> List[TensorSpec]:
        n, h, d = self.name, self.hidden, self.head_dim
        specs = [
            TensorSpec(f"{n}.q_proj.weight", (self.q_dim, h)),
            TensorSpec(f"{n}.k_proj.weight", (self.kv_dim, h)),
            TensorSpec(f"{n}.v_proj.weight", (self.kv_dim, h)),
            TensorSpec(f"{n}.o_proj.weight", (h, self.q_dim)),
        ]
        if self.qk_norm:
            specs += [TensorSpec(f"{n}.q_norm.weight", (d,), "norm"), TensorSpec(f"{n}.k_norm.weight", (d,), "norm")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        n = self.name
        q, k, v = (tensors.pop(f"{n}.{p}_proj.weight") for p in "qkv")
        # One matrix for the three projections: one pass over x instead of three.
        self.w_qkv = rt.matrix(torch.cat([q, k, v], dim=0))
        self.w_o = rt.matrix(tensors.pop(f"{n}.o_proj.weight"))
        if self.qk_norm:
            self.q_weight = rt.f32(tensors.pop(f"{n}.q_norm.weight"))
            self.k_weight = rt.f32(tensors.pop(f"{n}.k_norm.weight"))
        self.position.load(tensors, rt)
        self.rt = rt

    couples_norm = True

    def flops(self, tokens: int, pairs: int = 0) -> float:
        """The four projections, and per (query, key) pair a score and a weighted value of ``head_dim`` each."""
        return super().flops(tokens, pairs) + 4.0 * pairs * self.heads * self.head_dim

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.attention_jobs(dtype, self.heads, self.kv_heads, self.head_dim)

    def decode_plan_key(self):
        return ("paged_attention", self.heads, self.kv_heads, self.head_dim)

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        return ops.decode_plan(rt.device, rt.dtype, requests, self.heads, self.kv_heads, self.head_dim, span)

    def forward(self, x, ctx, cache, residual: torch.Tensor, then_norm=None):
        T = x.shape[0]
        ws = ctx.workspace
        writes = cache.owner
        pos = self.position
        q = ws.get("q", (T, self.q_dim), x.dtype)
        # A run that reads another run's cache computes only the queries.
        w = self.w_qkv if writes else self.w_qkv[: self.q_dim]
        ops.stage_name = "q|k|v, heads"
        if not ops.gemm_qkv_heads(x, w, q, self.q_weight, self.k_weight, self.norm_eps, ctx.positions, pos.inv_freq,
                                  pos.rotary_dim, pos.interleaved, cache.slot_mapping, cache.k, cache.v, self.heads,
                                  self.kv_heads, self.head_dim, writes, ctx):
            qkv = ws.get("qkv", (T, w.shape[0]), x.dtype)
            ops.gemm(x, w, qkv)
            ops.qk_norm_rope_write(
                qkv, q, self.q_weight, self.k_weight, self.norm_eps, ctx.positions,
                pos.inv_freq, pos.rotary_dim, pos.interleaved, cache.slot_mapping,
                cache.k, cache.v, self.heads, self.kv_heads, self.head_dim, writes,
            )
        out = ws.get("attn_out", (T, self.q_dim), x.dtype)
        ops.stage_name = "attention"
        plans = ctx.decode_plans
        ops.attention(q, cache.k, cache.v, out, ctx, cache.block_table, self.heads, self.kv_heads,
                      self.head_dim, self.scale, self.window or 0, plans.get(self.decode_plan_key()) if plans else None)
        ops.stage_name = "o"
        return ops.gemm(out, self.w_o, residual, accumulate=True, then_norm=then_norm)


def distance_bucket(n: int, rows: int, farthest: float) -> int:
    """Row of a distance table of ``rows`` rows for the distance ``n >= 0``: the first half of the rows take one distance
    each; the other half are spread evenly over the logarithm of the distance, up to ``farthest``; what lies beyond takes
    the last row."""
    half = rows // 2
    if n < half:
        return n
    if half == 0 or farthest <= half:
        return rows - 1
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(farthest / half) * (rows - half))))


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    """Causal grouped-query attention without a softmax, over the paged cache.

    ``q, k, v = x W^T`` (no bias; value heads ``v_head_dim`` wide); per-head RMS norm of q and k over ``head_dim`` (one
    weight each, shared by the heads); no rotation.  Positions enter in two ways: queries are multiplied by
    ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)`` (``temp_coef = 0``: not at all), and a learned table over the
    distance is added to the score, ``rel[distance_bucket(i - j), head]`` with ``bias_rows`` rows reaching to ``bias_max``
    (``bias_rows = 0``: no table).  The weight of a key ``j <= i`` is ``sigmoid(q . k * scale + rel + pb[head])`` with a
    learned number ``pb`` per head; weights are not normalised over the keys.  Output through ``o`` into the residual.
    At load the table and ``pb`` become one float32 table ``[heads, span]`` over the distance, which the kernels index.
    """

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "rel": "distance_bias", "pb": "head_bias"}

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, name: str, v_head_dim: Optional[int] = None,
                 scale: Optional[float] = None, qk_norm: bool = True, norm_eps: float = 1e-6, temp_coef: float = 0.0,
                 temp_every: int = 1, bias_rows: int = 0, bias_max: float = 0.0, head_bias: bool = True, names=None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"{heads} heads cannot share {kv_heads} kv heads evenly")
        self.v_head_dim = int(v_head_dim) if v_head_dim is not None else self.head_dim
        self.name, self.qk_norm, self.norm_eps = name, bool(qk_norm), float(norm_eps)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every)
        if self.temp_every <= 0:
            raise ValueError("temp_every must be positive")
        self.bias_rows, self.bias_max, self.head_bias = int(bias_rows), float(bias_max), bool(head_bias)
        self.names = dict(self.NAMES, **(names or {}))
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.kv_heads * self.v_head_dim
        self.w_qkv = self.w_o = self.q_weight = self.k_weight = self.bias = None

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        return PagedKV(self.kv_heads, self.head_dim, None, self.v_head_dim)

    def tensor_specs(self) -> List[TensorSpec]:
        h = self.hidden
        specs = [TensorSpec(self._n("q"), (self.q_dim, h)), TensorSpec(self._n("k"), (self.k_dim, h)),
                 TensorSpec(self._n("v"), (self.v_dim, h)), TensorSpec(self._n("o"), (h, self.heads * self.v_head_dim))]
        if self.qk_norm:
            specs += [TensorSpec(self._n("q_norm"), (self.head_dim,), "norm"), TensorSpec(self._n("k_norm"), (self.head_dim,), "norm")]
        if self.bias_rows:
            specs.append(TensorSpec(self._n("rel"), (self.bias_rows, self.heads), "bias"))
        if self.head_bias:
            specs.append(TensorSpec(self._n("pb"), (self.heads,), "bias"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        q, k, v = (tensors.pop(self._n(p)) for p in "qkv")
        self.w_qkv = rt.matrix(torch.cat([q, k, v], dim=0))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        if self.qk_norm:
            self.q_weight = rt.f32(tensors.pop(self._n("q_norm")))
            self.k_weight = rt.f32(tensors.pop(self._n("k_norm")))
        # everything added to a score as a function of head and distance, as one table over the distance: beyond
        # bias_max every distance falls into the last row, so the table ends there
        span = int(math.floor(self.bias_max)) + 2 if self.bias_rows else 1
        table = torch.zeros(self.heads, span, dtype=torch.float32)
        if self.bias_rows:
            rel = tensors.pop(self._n("rel")).to("cpu", torch.float32)
            rows = torch.tensor([distance_bucket(n, self.bias_rows, self.bias_max) for n in range(span)], dtype=torch.long)
            table += rel[rows].t()
        if self.head_bias:
            table += tensors.pop(self._n("pb")).to("cpu", torch.float32)[:, None]
        self.bias = table.to(rt.device).contiguous()
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return super().flops(tokens, pairs) + 2.0 * pairs * self.heads * (self.head_dim + self.v_head_dim)

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.sigmoid_attention_jobs(dtype, self.heads, self.kv_heads, self.head_dim, self.v_head_dim)

    def decode_plan_key(self):
        return ("sigmoid_attention", self.kv_heads)

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        return ops.sigmoid_decode_plan(requests, self.kv_heads, span)

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        writes = cache.owner
        w = self.w_qkv if writes else self.w_qkv[: self.q_dim]
        ops.stage_name = "q|k|v"
        qkv = ws.get("qkv", (T, w.shape[0]), x.dtype)
        ops.gemm(x, w, qkv)
        ops.stage_name = "heads"
        q = ws.get("q", (T, self.q_dim), x.dtype)
        ops.qkv_heads_sigmoid(qkv, q, self.q_weight, self.k_weight, self.norm_eps, ctx.positions, self.temp_coef, self.temp_every,
                              cache.slot_mapping, cache.k, cache.v, self.heads, self.kv_heads, self.head_dim, self.v_head_dim, writes)
        out = ws.get("attn_out", (T, self.heads * self.v_head_dim), x.dtype)
        ops.stage_name = "attention"
        plans = ctx.decode_plans
        ops.attention_sigmoid(q, cache.k, cache.v, out, ctx, cache.block_table, self.bias, self.heads, self.kv_heads,
                              self.head_dim, self.v_head_dim, self.scale, plans.get(self.decode_plan_key()) if plans else None)
        ops.stage_name = "o"
        ops.gemm(out, self.w_o, residual, accumulate=True)
        return None


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    """Causal grouped-query softmax attention over the paged cache, with the variations a design may switch on one by one.

    ``q, k, v = x W^T (+ b)`` (``bias``); value heads ``v_head_dim`` wide.  RMS norm of q and k before the rotation:
    ``qk_norm`` "head" (per head over ``head_dim``, one weight ``[head_dim]`` each), "whole" (over the whole projection at
    once, before it is split into heads, weights ``[heads head_dim]`` and ``[kv_heads head_dim]``) or None.  The rotation
    comes from ``position`` (any registered encoding: partial width, rescaled frequencies and magnitudes are its
    business).  Score ``q . k * scale``.  A position sees the keys before it and itself; ``window`` keeps the last so
    many, ``chunk`` keeps those of its own chunk (``floor(i / chunk) = floor(j / chunk)``, counted from the sequence's
    first position wherever a prompt was cut).  ``sink``: the softmax has one more term in its denominator, a key of
    score 0 without a value: ``p_j = exp(s_j) / (1 + sum_j exp(s_j))``; ``sink="learned"``: the term is ``exp(b_h)`` with a
    learned number ``b_h`` per query head (tensor ``sink`` ``[heads]``, not scaled).

    ``value_mix``: None, or a name that ties layers together: the first layer of that name in the model leaves its values
    (of the step's tokens) where the later ones find them, and those cache ``(1 - lam) v + lam v_first`` with their own
    learned ``lam`` (``first_of_mix`` says which a layer is; the first one's ``lam`` tensor is expected and unused).
    ``gate``: the heads' outputs are multiplied by ``sigmoid(x W_g^T)`` before the output projection.  One fused product
    makes q | k | v | g.
    """

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "g": "g_proj.weight",
             "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
             "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "lam": "value_mix", "sink": "sink"}

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, name: str, position: PartSpec,
                 v_head_dim: Optional[int] = None, scale: Optional[float] = None, bias: bool = False, qk_norm: Optional[str] = "head",
                 norm_eps: float = 1e-6, window: Optional[int] = None, chunk: Optional[int] = None, sink: bool = True,
                 value_mix: Optional[str] = None, first_of_mix: bool = False, gate: bool = False, names=None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"{heads} heads cannot share {kv_heads} kv heads evenly")
        if qk_norm not in (None, "head", "whole"):
            raise ValueError(f"qk_norm {qk_norm!r} is not one of None, 'head', 'whole'")
        self.v_head_dim = int(v_head_dim) if v_head_dim is not None else self.head_dim
        self.name, self.bias, self.qk_norm, self.norm_eps = name, bool(bias), qk_norm, float(norm_eps)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(window) if window else None
        self.chunk = int(chunk) if chunk else None
        self.sink, self.gate = bool(sink), bool(gate)
        self.learned_sink = sink == "learned"
        self.sink_logits = None
        self.value_mix, self.first_of_mix = value_mix, bool(first_of_mix)
        self.position = lookup("position", position.kind)(**position.params)
        self.names = dict(self.NAMES, **(names or {}))
        self.q_dim, self.k_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_dim, self.o_dim = self.kv_heads * self.v_head_dim, self.heads * self.v_head_dim
        self.w_in = self.w_o = self.q_weight = self.k_weight = self.q_b = self.k_b = self.v_b = self.lam = None

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        # (a chunked mask never looks behind its chunk's start, but pages are not given back there: the keys a window
        # has passed are dropped by the cache manager, a chunk's are only skipped)
        return PagedKV(self.kv_heads, self.head_dim, self.window, self.v_head_dim)

    def tensor_specs(self) -> List[TensorSpec]:
        h = self.hidden
        specs = [TensorSpec(self._n("q"), (self.q_dim, h)), TensorSpec(self._n("k"), (self.k_dim, h)),
                 TensorSpec(self._n("v"), (self.v_dim, h)), TensorSpec(self._n("o"), (h, self.o_dim))]
        if self.gate:
            specs.append(TensorSpec(self._n("g"), (self.o_dim, h)))
        if self.bias:
            specs += [TensorSpec(self._n("q_bias"), (self.q_dim,), "bias"), TensorSpec(self._n("k_bias"), (self.k_dim,), "bias"),
                      TensorSpec(self._n("v_bias"), (self.v_dim,), "bias")]
        if self.qk_norm is not None:
            n = 1 if self.qk_norm == "head" else None
            specs += [TensorSpec(self._n("q_norm"), (self.head_dim if n else self.q_dim,), "norm"),
                      TensorSpec(self._n("k_norm"), (self.head_dim if n else self.k_dim,), "norm")]
        if self.value_mix is not None:
            specs.append(TensorSpec(self._n("lam"), (), "bias", 0.5))
        if self.learned_sink:
            specs.append(TensorSpec(self._n("sink"), (self.heads,), "bias"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        parts = [tensors.pop(self._n(p)) for p in "qkv"]
        if self.gate:
            parts.append(tensors.pop(self._n("g")))
        self.w_in = rt.matrix(torch.cat(parts, dim=0))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        if self.bias:
            self.q_b, self.k_b, self.v_b = (rt.f32(tensors.pop(self._n(f"{p}_bias"))) for p in "qkv")
        if self.qk_norm is not None:
            self.q_weight = rt.f32(tensors.pop(self._n("q_norm")))
            self.k_weight = rt.f32(tensors.pop(self._n("k_norm")))
        if self.value_mix is not None:
            self.lam = rt.f32(tensors.pop(self._n("lam"))).reshape(1)
        if self.learned_sink:
            self.sink_logits = rt.f32(tensors.pop(self._n("sink")))
        self.position.load(tensors, rt)
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        w = self.window
        if w and tokens > w and pairs == tokens * (tokens + 1) // 2:
            pairs = w * (w + 1) // 2 + (tokens - w) * w          # one prompt from its first position: the window's pairs
        elif w:
            pairs = min(pairs, tokens * w)
        return super().flops(tokens, pairs) + 2.0 * pairs * self.heads * (self.head_dim + self.v_head_dim)

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.sink_attention_jobs(dtype, self.heads, self.kv_heads, self.head_dim, self.v_head_dim)

    def decode_plan_key(self):
        return ("sink_attention", self.heads, self.kv_heads, self.head_dim, self.v_head_dim, self.chunk, self.window)

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        return ops.sink_decode_plan(rt.dtype, requests, self.heads, self.kv_heads, self.head_dim, self.v_head_dim, span,
                                    self.window or 0, self.chunk or 0)

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        writes = cache.owner
        if not writes and self.gate:
            raise ValueError("sink_attention: a gated layer cannot read another run's cache")   # its columns lie behind k and v
        w = self.w_in if writes else self.w_in[: self.q_dim]
        ops.stage_name = "q|k|v|g"
        rows = ws.get("qkvg", (T, w.shape[0]), x.dtype)
        ops.gemm(x, w, rows)
        ops.stage_name = "heads"
        q = ws.get("q", (T, self.q_dim), x.dtype)
        shared = None
        mode = None
        if self.value_mix is not None and writes:
            # the first layer's values of this step's tokens, for the later layers of the same name
            shared = ws.get(f"values:{self.value_mix}", (T, self.v_dim), x.dtype)
            mode = "leave" if self.first_of_mix else "mix"
        pos = self.position
        ops.qkv_finish(rows, q, self.q_b, self.k_b, self.v_b, self.qk_norm, self.q_weight, self.k_weight, self.norm_eps, ctx.positions,
                       pos.inv_freq, pos.rotary_dim, pos.magnitude, cache.slot_mapping, cache.k, cache.v, mode, shared, self.lam,
                       self.heads, self.kv_heads, self.head_dim, self.v_head_dim, writes, pos.interleaved)
        out = ws.get("attn_out", (T, self.o_dim), x.dtype)
        ops.stage_name = "attention"
        gate = rows[:, self.q_dim + self.k_dim + self.v_dim:] if self.gate else None
        plans = ctx.decode_plans
        ops.attention_sink(q, cache.k, cache.v, out, ctx, cache.block_table, self.heads, self.kv_heads, self.head_dim, self.v_head_dim,
                           self.scale, self.window or 0, self.chunk or 0, self.sink, gate,
                           plans.get(self.decode_plan_key()) if plans else None, self.sink_logits)
        ops.stage_name = "o"
        ops.gemm(out, self.w_o, residual, accumulate=True)
        return None


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """Causal softmax attention whose keys and values are expanded per head from one latent row per position
    (multi-head latent attention: DeepSeek-AI, "DeepSeek-V2: A Strong, Economical, and Efficient Mixture-of-Experts
    Language Model").

    ``q = W_q h``, per head ``head_dim`` unrotated and ``rot_dim`` rotated numbers.  ``W_dkv h`` gives ``kv_rank`` numbers
    that, divided by their root mean square times a weight, are the latent ``c``, and ``rot_dim`` numbers that, rotated, are a
    key part ``k_r`` shared by all heads; the page row of a position is ``[c | k_r]``, nothing else is cached.  Head ``a`` has
    the key ``[W_uk_a c | k_r]`` and the value ``W_uv_a c``; the score is their product with ``[q_a | rotated q_a]`` times
    ``scale``; the softmax may have a sink as in :class:`SinkAttention`.  Computed in the absorbed form: the queries are taken
    into the latent's space, ``q'_a = [W_uk_a^T q_a | rotated q_a]``, every head then reads the same page rows (one kv head
    whose values are the rows' first ``kv_rank`` elements), and the heads' sums of latents are expanded once per token,
    ``W_uv_a (sum_j p_j c_j)``.  A run that reads another run's cache (``cache_of``) has no ``W_dkv`` of its own in use: it
    computes its queries, reads the owner's rows and applies its own ``W_uk``, ``W_uv``, sink and ``W_o``; ``own_latent=False``
    says the layer brings no ``dkv`` tensors at all.

    ``q_rank``: the queries go through a latent of their own, ``q = W_q (W_qd h / rms(W_qd h) * w)`` (tensors ``q_down``,
    ``q_norm``).  ``window``: a position sees the last so many positions only (the cache manager gives older pages back).
    ``gate`` "head": head ``a``'s output is multiplied by ``sigmoid(W_g h)_a`` (tensor ``g`` ``[heads, hidden]``).
    """

    NAMES = {"q": "q", "dkv": "dkv", "c_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o", "sink": "sink", "q_down": "q_down",
             "q_norm": "q_down.norm", "g": "g"}

    def __init__(self, hidden: int, heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int, name: str, position: PartSpec,
                 scale: Optional[float] = None, norm_eps: float = 1e-6, sink=False, own_latent: bool = True, names=None,
                 q_rank: Optional[int] = None, window: Optional[int] = None, gate: Optional[str] = None):
        if gate not in (None, "head"):
            raise ValueError(f"latent_attention: gate {gate!r} is not one of None, 'head'")
        self.q_rank = int(q_rank) if q_rank else None
        self.window = int(window) if window else None
        self.gate = gate
        self.hidden, self.heads, self.head_dim, self.rot_dim = int(hidden), int(heads), int(head_dim), int(rot_dim)
        self.v_head_dim, self.kv_rank = int(v_head_dim), int(kv_rank)
        self.name, self.norm_eps = name, float(norm_eps)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim + self.rot_dim)
        self.sink, self.learned_sink = bool(sink), sink == "learned"
        self.own_latent = bool(own_latent)
        self.position = lookup("position", position.kind)(**position.params)
        if self.position.rotary_dim > self.rot_dim:
            raise ValueError(f"latent_attention: {self.position.rotary_dim} rotated dimensions in a rotated part of {self.rot_dim}")
        self.names = dict(self.NAMES, **(names or {}))
        self.q_head = self.head_dim + self.rot_dim
        self.q_dim, self.row_dim = self.heads * self.q_head, self.kv_rank + self.rot_dim
        self.o_dim = self.heads * self.v_head_dim
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_weight = self.sink_logits = None

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        return PagedKV(1, self.row_dim, self.window, self.kv_rank, values_in_keys=True)

    def tensor_specs(self) -> List[TensorSpec]:
        h, r = self.hidden, self.kv_rank
        if self.q_rank:
            specs = [TensorSpec(self._n("q_down"), (self.q_rank, h)), TensorSpec(self._n("q_norm"), (self.q_rank,), "norm"),
                     TensorSpec(self._n("q"), (self.q_dim, self.q_rank))]
        else:
            specs = [TensorSpec(self._n("q"), (self.q_dim, h))]
        if self.gate:
            specs.append(TensorSpec(self._n("g"), (self.heads, h)))
        if self.own_latent:
            specs += [TensorSpec(self._n("dkv"), (self.row_dim, h)), TensorSpec(self._n("c_norm"), (r,), "norm")]
        specs += [TensorSpec(self._n("uk"), (self.heads * self.head_dim, r)), TensorSpec(self._n("uv"), (self.o_dim, r)),
                  TensorSpec(self._n("o"), (h, self.o_dim))]
        if self.learned_sink:
            specs.append(TensorSpec(self._n("sink"), (self.heads,), "bias"))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        # one product of the layer's input: the queries (or their latent) | the latent and the key part | the heads' gates
        self.w_q = self.q_weight = None
        if self.q_rank:
            parts = [tensors.pop(self._n("q_down"))]
            self.q_weight = rt.f32(tensors.pop(self._n("q_norm")))
            self.w_q = rt.matrix(tensors.pop(self._n("q")))
        else:
            parts = [tensors.pop(self._n("q"))]
        self.first = parts[0].shape[0]                  # columns of the queries (or of their latent) in that product
        if self.own_latent:
            parts.append(tensors.pop(self._n("dkv")))
            self.c_weight = rt.f32(tensors.pop(self._n("c_norm")))
        self.gate_col = sum(p.shape[0] for p in parts)
        if self.gate:
            parts.append(tensors.pop(self._n("g")))
        self.w_in = rt.matrix(torch.cat(parts, dim=0))
        # per head the key expansion transposed, [heads, kv_rank, head_dim]: the queries are multiplied into the latent's space
        uk = tensors.pop(self._n("uk")).reshape(self.heads, self.head_dim, self.kv_rank)
        self.w_uk_t = rt.matrix(uk.transpose(1, 2))
        self.w_uv = rt.matrix(tensors.pop(self._n("uv")).reshape(self.heads, self.v_head_dim, self.kv_rank))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        if self.learned_sink:
            self.sink_logits = rt.f32(tensors.pop(self._n("sink")))
        self.position.load(tensors, rt)
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        w = self.window
        if w and tokens > w and pairs == tokens * (tokens + 1) // 2:
            pairs = w * (w + 1) // 2 + (tokens - w) * w          # one prompt from its first position: the window's pairs
        elif w:
            pairs = min(pairs, tokens * w)
        return super().flops(tokens, pairs) + 2.0 * pairs * self.heads * (self.row_dim + self.kv_rank)

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        jobs = ops.library_jobs("mb_attention_latent", "mb_activations")
        jobs.update(ops.sink_attention_jobs(dtype, self.heads, 1, self.row_dim, self.kv_rank, values_in_keys=True))
        return jobs

    def decode_plan_key(self):
        return ("latent_attention", self.heads, self.row_dim, self.kv_rank, self.window)

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        return ops.sink_decode_plan(rt.dtype, requests, self.heads, 1, self.row_dim, self.kv_rank, span, self.window or 0, 0,
                                    values_in_keys=True)

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        writes = cache.owner
        if writes and not self.own_latent:
            raise ValueError("latent_attention: a layer without a latent of its own must read another run's cache")
        H, dn, dr, r, D = self.heads, self.head_dim, self.rot_dim, self.kv_rank, self.row_dim
        if not writes and self.gate:
            raise ValueError("latent_attention: a gated layer cannot read another run's cache")      # its columns lie behind the latent's
        w = self.w_in if writes else self.w_in[: self.first]
        ops.stage_name = "q|dkv"
        rows = ws.get("q_dkv", (T, w.shape[0]), x.dtype)
        ops.gemm(x, w, rows)
        heads, kv_rows = rows, None
        if self.q_rank:
            # the queries' latent, normed, then the queries themselves; the latent and key part stay where the first product left them
            ops.stage_name = "q from its latent"
            cq = ws.get("q_small", (T, self.q_rank), x.dtype)
            ops.rmsnorm_cols(rows, 0, self.q_weight, self.norm_eps, cq)
            heads = ws.get("q_heads", (T, self.q_dim), x.dtype)
            ops.gemm(cq, self.w_q, heads)
            kv_rows = rows[:, self.first:self.first + D] if writes else None
        ops.stage_name = "heads"
        q = ws.get("q_latent", (T, H * D), x.dtype)
        pos = self.position
        ops.latent_finish(heads, q, self.c_weight, self.norm_eps, ctx.positions, pos.inv_freq, pos.rotary_dim, pos.interleaved,
                          cache.slot_mapping, cache.k, H, dn, dr, r, writes, kv_rows)
        ops.stage_name = "q into the latent"
        ops.heads_product(heads, self.q_head, dn, self.w_uk_t, q, D)
        mixed = ws.get("latent_out", (T, H * r), x.dtype)
        ops.stage_name = "attention, latent"
        plans = ctx.decode_plans
        ops.attention_sink(q, cache.k, cache.k, mixed, ctx, cache.block_table, H, 1, D, r, self.scale, self.window or 0, 0, self.sink, None,
                           plans.get(self.decode_plan_key()) if plans else None, self.sink_logits)
        ops.stage_name = "v from the latent"
        out = ws.get("attn_out", (T, self.o_dim), x.dtype)
        ops.heads_product(mixed, r, r, self.w_uv, out, self.v_head_dim)
        if self.gate:
            ops.stage_name = "gate"
            ops.head_gate(out, rows, self.gate_col, H)
        ops.stage_name = "o"
        ops.gemm(out, self.w_o, residual, accumulate=True)
        return None


@register_mixer("pooled_attention")
class PooledAttention(Mixer):
    """Causal grouped-query softmax attention over a window of single positions and, before it, pooled blocks.

    ``q, k, v = x W^T (+ b)`` (``bias``); value heads ``v_head_dim`` wide; the rotation comes from ``position``; ``qk_norm``: q
    and k are divided by their root mean square per head, without a weight (before or after a rotation in pairs it is the same
    number).  Score ``q . k * scale``, then ``softcap tanh(s / softcap)`` where ``softcap`` is given.  Position ``i`` sees the
    positions ``j`` with ``0 <= i - j < window`` and, with ``pool`` = P, one key and one value for every block ``b`` of P
    positions with ``b P + P - 1 <= i - window``: the means of the block's keys and values as the cache holds them.  Positions
    that have left the window and whose block is not complete behind it are not seen.  One softmax over both kinds.  ``talk``: a
    learned matrix ``[heads, heads]`` mixes the heads' softmax weights, ``w'_h = sum_g talk[h, g] w_g``, and head ``h`` applies
    ``w'_h`` to the values of its own kv head.  Without ``window`` every earlier position is seen and ``pool`` has no effect.
    The cache keeps every position's key and value (the pooled rows live in the pages, see ``PagedKV.pooled``).
    """

    NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight", "q_bias": "q_proj.bias",
             "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "talk": "talk"}

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, name: str, position: PartSpec, v_head_dim: Optional[int] = None,
                 scale: Optional[float] = None, bias: bool = False, qk_norm: bool = False, norm_eps: float = 1e-6, window: Optional[int] = None,
                 pool: Optional[int] = None, softcap: Optional[float] = None, talk: bool = False, names=None):
        self.hidden, self.heads, self.kv_heads, self.head_dim = int(hidden), int(heads), int(kv_heads), int(head_dim)
        if self.heads % self.kv_heads != 0:
            raise ValueError(f"{heads} heads cannot share {kv_heads} kv heads evenly")
        self.v_head_dim = int(v_head_dim) if v_head_dim is not None else self.head_dim
        self.name, self.bias, self.qk_norm, self.norm_eps = name, bool(bias), bool(qk_norm), float(norm_eps)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.window = int(window) if window else None
        self.pool = int(pool) if pool and self.window else None
        self.softcap = float(softcap) if softcap else None
        self.talk = bool(talk)
        self.position = lookup("position", position.kind)(**position.params)
        self.names = dict(self.NAMES, **(names or {}))
        self.q_dim, self.k_dim = self.heads * self.head_dim, self.kv_heads * self.head_dim
        self.v_dim, self.o_dim = self.kv_heads * self.v_head_dim, self.heads * self.v_head_dim
        self.w_in = self.w_o = self.q_b = self.k_b = self.v_b = self.talk_w = self.ones = None

    def _n(self, key: str) -> str:
        return f"{self.name}.{self.names[key]}"

    def cache_need(self):
        if self.pool:
            return PagedKV(self.kv_heads, self.head_dim, None, self.v_head_dim, pooled=self.pool, pooled_window=self.window)
        return PagedKV(self.kv_heads, self.head_dim, self.window, self.v_head_dim)

    def tensor_specs(self) -> List[TensorSpec]:
        h = self.hidden
        specs = [TensorSpec(self._n("q"), (self.q_dim, h)), TensorSpec(self._n("k"), (self.k_dim, h)),
                 TensorSpec(self._n("v"), (self.v_dim, h)), TensorSpec(self._n("o"), (h, self.o_dim))]
        if self.bias:
            specs += [TensorSpec(self._n("q_bias"), (self.q_dim,), "bias"), TensorSpec(self._n("k_bias"), (self.k_dim,), "bias"),
                      TensorSpec(self._n("v_bias"), (self.v_dim,), "bias")]
        if self.talk:
            specs.append(TensorSpec(self._n("talk"), (self.heads, self.heads), "bias", 1.0 / self.heads))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.w_in = rt.matrix(torch.cat([tensors.pop(self._n(p)) for p in "qkv"], dim=0))
        self.w_o = rt.matrix(tensors.pop(self._n("o")))
        if self.bias:
            self.q_b, self.k_b, self.v_b = (rt.f32(tensors.pop(self._n(f"{p}_bias"))) for p in "qkv")
        if self.talk:
            self.talk_w = rt.f32(tensors.pop(self._n("talk")))
        if self.qk_norm:
            self.ones = torch.ones(self.head_dim, device=rt.device, dtype=torch.float32)
        self.position.load(tensors, rt)
        self.rt = rt

    def flops(self, tokens: int, pairs: int = 0) -> float:
        w = self.window
        if w and tokens > 0:
            each = pairs / tokens                               # keys a token would see without the window, on average
            pairs = int(tokens * (min(each, w) + (max(0.0, each - w) / self.pool if self.pool else 0.0)))
        values = (self.kv_heads if self.talk else 1) * self.v_head_dim
        return super().flops(tokens, pairs) + 2.0 * pairs * self.heads * (self.head_dim + values)

    def workspace_per_token(self, dtype) -> int:
        """Bytes a step keeps per token beside the products' rows: with mixed weights, every head's float32 sum over every kv
        head's values."""
        return 4 * self.heads * self.kv_heads * self.v_head_dim if self.talk else 0

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        return ops.pooled_attention_jobs(dtype, self.heads, self.kv_heads, self.head_dim, self.v_head_dim)

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        T = x.shape[0]
        ws = ctx.workspace
        writes = cache.owner
        w = self.w_in if writes else self.w_in[: self.q_dim]
        ops.stage_name = "q|k|v"
        rows = ws.get("qkv", (T, w.shape[0]), x.dtype)
        ops.gemm(x, w, rows)
        ops.stage_name = "heads"
        q = ws.get("q", (T, self.q_dim), x.dtype)
        pos = self.position
        ops.qkv_finish(rows, q, self.q_b, self.k_b, self.v_b, "head" if self.qk_norm else None, self.ones, self.ones, self.norm_eps,
                       ctx.positions, pos.inv_freq, pos.rotary_dim, pos.magnitude, cache.slot_mapping, cache.k, cache.v, None, None, None,
                       self.heads, self.kv_heads, self.head_dim, self.v_head_dim, writes, pos.interleaved)
        if self.pool and writes:
            ops.stage_name = "pooled blocks"
            ops.pool_blocks(cache.k, cache.v, cache.k_pool, cache.v_pool, ctx, cache.block_table, cache.slot_mapping, self.pool)
        out = ws.get("attn_out", (T, self.o_dim), x.dtype)
        ops.stage_name = "attention"
        ops.attention_pooled(q, cache.k, cache.v, cache.k_pool, cache.v_pool, out, ctx, cache.block_table, self.heads, self.kv_heads,
                             self.head_dim, self.v_head_dim, self.scale, self.softcap or 0.0, self.window or 0, self.pool or 0, self.talk_w)
        ops.stage_name = "o"
        ops.gemm(out, self.w_o, residual, accumulate=True)
        return None


@register_mixer("token_shifted")
class ShiftedMixer(Mixer):
    """Any mixer behind a token shift: what the inner mixer reads is ``h + (h' - h) * mu`` element by element, ``h'`` the row the
    token before brought (as it was before its own shift; zeros before a sequence's first token) and ``mu`` a learned vector
    (tensor ``tensor``, a full name).  The last row a request has brought is part of its state, beside whatever the inner mixer
    keeps: ``cache_need`` answers both, the view is the pair of their views."""

    def __init__(self, hidden: int, tensor: str, inner: PartSpec, name: str):
        self.hidden, self.tensor, self.name = int(hidden), tensor, name
        self.inner = lookup("mixer", inner.kind)(name=name, **inner.params)
        self.capturable = getattr(self.inner, "capturable", True)
        self.mu = None

    def cache_need(self):
        return (StateNeed((self.hidden,), torch.float32), self.inner.cache_need())

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.tensor, (self.hidden,), "bias", 0.5)] + self.inner.tensor_specs()

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.mu = rt.f32(tensors.pop(self.tensor)).reshape(1, self.hidden)
        self.inner.load(tensors, rt)
        self.rt = rt

    def bytes_read(self, tokens: int, dtype) -> int:
        return self.hidden * 4 + self.inner.bytes_read(tokens, dtype)

    def flops(self, tokens: int, pairs: int = 0) -> float:
        return self.inner.flops(tokens, pairs)

    def kernel_jobs(self, dtype) -> Dict[str, tuple]:
        jobs = ops.library_jobs("mb_activations")
        jobs.update(self.inner.kernel_jobs(dtype))
        return jobs

    def workspace_per_token(self, dtype) -> int:
        return self.inner.workspace_per_token(dtype) if hasattr(self.inner, "workspace_per_token") else 0

    def decode_plan_key(self):
        return self.inner.decode_plan_key()

    def decode_plan(self, requests: int, span: int, rt: Runtime):
        return self.inner.decode_plan(requests, span, rt)

    def forward(self, x, ctx, cache, residual: torch.Tensor):
        last, inner_cache = cache
        if not last.owner:
            raise ValueError("token_shifted: a run that reads another run's cache would share its last row too")
        ops.stage_name = "token shift"
        shifted = ctx.workspace.get("shifted", (1,) + tuple(x.shape), x.dtype)
        ops.shift_mix(x, last.state, ctx, last.slots, self.mu, shifted)
        ops.keep_last_row(x, last.state, ctx, last.slots)
        return self.inner.forward(shifted[0], ctx, inner_cache, residual)
