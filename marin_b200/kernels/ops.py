"""The kernels as Python functions over torch CUDA tensors.

Every function checks shapes and dtypes on the host, then launches hand-written CUDA on the
current stream through ``ctypes``; results land in the ``out`` argument.  There is no other
implementation behind these names: on a machine without CUDA, or if a library cannot be built,
the call raises.  (The reference funnels its launches through checked wrappers the same way,
crates/cuda/src/ops.rs:53-236.)
"""
from __future__ import annotations

import ctypes
import functools
import os
import weakref
from typing import Optional

import torch

from . import build

_c_int, _c_float, _c_void_p, _c_size_t = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {-2: "unsupported dtype combination", -3: "unsupported size", -4: "a device-side wait gave up"}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    return _c_void_p(t.data_ptr()) if t is not None else _c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle (asked of torch on every launch: streams change under graph capture)."""
    if _raw_stream is not None:
        return _c_void_p(_raw_stream(torch.cuda.current_device()))
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("marin_b200 kernels run on CUDA tensors only; there is no CPU path")
        if t is not None and not t.is_contiguous():
            raise KernelError("marin_b200 kernels need contiguous tensors")


#: how many kernels of this package were launched (a launcher that returned 0 launched one kernel)
launches = 0


def launches_extra(n: int) -> None:
    """A launcher that started more than one kernel says so here."""
    global launches
    launches += n


#: While this is a list, every launch appends what it was and what it had to move and compute (``engine/profile.py``
#: reads it: the stages of a step with their bytes and flops, in launch order).  ``stage_name`` is set by the parts
#: before their calls ("qkv", "attention", "o", ...) and names the launches that follow.
launch_log: Optional[list] = None
stage_name = ""
_pending_cost: Optional[dict] = None


def _cost(nbytes: float = 0, flops: float = 0.0, bytes_per_key: float = 0, flops_per_pair: float = 0.0) -> None:
    """What the next launch has to read and write (bytes) and compute (flops), as the algorithm needs it: every input
    and output once.  Attention's share that grows with the cache is given per cached key read and per (query, key)
    pair, because a captured graph is replayed at other lengths than it was captured at."""
    global _pending_cost
    if launch_log is not None:
        _pending_cost = {"bytes": float(nbytes), "flops": float(flops), "bytes_per_key": float(bytes_per_key),
                         "flops_per_pair": float(flops_per_pair)}


def _size(t) -> int:
    return t.numel() * t.element_size()


def _check(rc: int, what: str) -> None:
    global launches, _pending_cost
    if rc == 0:
        launches += 1
        if launch_log is not None:
            entry = _pending_cost or {"bytes": 0.0, "flops": 0.0, "bytes_per_key": 0.0, "flops_per_pair": 0.0}
            entry["stage"], entry["kernel"] = stage_name, what
            launch_log.append(entry)
            _pending_cost = None
        return
    if rc in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[rc]}")
    raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.cudart().cudaGetErrorString(rc) if hasattr(torch.cuda.cudart(), 'cudaGetErrorString') else ''})")


def _lib(name: str):
    return build.load(name, build.LIBRARIES[name])


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, pos_table: Optional[torch.Tensor] = None,
          positions: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """``out[t] = float32(table[ids[t]]) * scale``, plus ``float32(pos_table[positions[t]])`` where a learned position table is given."""
    _need_cuda(ids, table, out, pos_table, positions)
    T, h = out.shape
    assert ids.dtype == torch.int32 and ids.numel() == T and table.shape[1] == h and out.dtype == torch.float32
    if pos_table is not None:
        assert positions is not None and positions.dtype == torch.int32 and positions.numel() == T
        assert pos_table.dtype == table.dtype and pos_table.shape[1] == h
    _cost(T * h * table.element_size() * (2 if pos_table is not None else 1) + _size(out) + _size(ids))
    _check(_lib("mb_elementwise").mb_embed(_ptr(ids), _ptr(table), _code(table), _ptr(pos_table), _ptr(positions if pos_table is not None else None),
                                          _ptr(out), _c_int(T), _c_int(h), _c_float(scale), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, unit_offset: bool = False) -> None:
    _need_cuda(x, weight, out)
    rows, n = x.shape
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == n and out.shape == x.shape
    _cost(_size(x) + _size(out) + _size(weight), 4.0 * rows * n)
    _check(_lib("mb_elementwise").mb_rmsnorm(_ptr(x), _ptr(weight), _c_float(eps), _c_int(int(unit_offset)), _ptr(out),
                                            _code(out), _c_int(rows), _c_int(n), _stream()), "rmsnorm")


#: bf16 products go to the tcgen05 kernel when their shape allows (False: always the plain kernel)
use_tensor_cores = True
#: with few tokens an RMS norm rides on the products around it instead of running as a kernel of its own
couple_norms = True
#: the same with many tokens, in the persistent kernel.  Off: measured on B200 at 2,048 tokens (Qwen3-4B layers) the
#: per-token factors that every tile's epilogue has to gather cost the gate/up product 39 us where the norm's own
#: kernel costs 7.
couple_norms_in_prefill = False
SM_COUNT = 148


class NonFiniteLogits(KernelError):
    """Logits that are NaN or infinite among the values a token may be chosen from; the sampling kernels give such
    rows the id -1 (the reference refuses them: crates/sampler/src/lib.rs:135-137, crates/model/src/qwen3/model.rs:128)."""


class Scratch:
    """Device memory the kernels use besides their inputs and outputs, for ONE stream of work at a time: an engine
    owns one (``Runner.scratch``) and makes it current around its steps (``using``), so that two engines in one
    process, each on a stream of its own, never share a counter or a flag.  Calls outside any ``using`` block
    take a default per device.

    ``error``        one int: the code a kernel leaves when a bounded wait gives up (zero otherwise);
    ``report``       four ints, of which a sampling kernel fills the first with a copy of ``error`` when that is not
                     zero; the sampled ids of a step lie right behind it (``ids``), so that one copy brings both
                     to the host (``read``) and every step learns of a wait that gave up without a wait of its own;
    ``sumsq``        per-token sums of squares that ride from one product to the next (coupled norms);
    ``parked``, ``parked_flags``  stream-K: the partial tile each CTA may park, and a flag per epilogue warp;
    ``argmax_keys``, ``argmax_count``  arg-max over several blocks per row; zero between launches;
    decode attention's partial results grow on demand (``decode_buffers``) unless a captured graph brings its own.
    """

    ARGMAX_ROWS = 4096
    RESULT_ROWS = 4096

    def __init__(self, device):
        global SM_COUNT
        self.device = torch.device(device)
        SM_COUNT = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.sm_count = SM_COUNT
        i32, f32 = dict(device=self.device, dtype=torch.int32), dict(device=self.device, dtype=torch.float32)
        self.error = torch.zeros(1, **i32)
        self.result = torch.zeros(4 + self.RESULT_ROWS, **i32)      # the report, then the sampled ids: one copy reads both
        self.report = self.result[:4]
        self.sumsq = torch.empty(1 << 22, **f32)
        self.parked = torch.empty(self.sm_count * 256 * 128, **f32)
        self.parked_flags = torch.zeros(self.sm_count * 8, **i32)
        self.argmax_keys = torch.zeros(self.ARGMAX_ROWS, device=self.device, dtype=torch.int64)
        self.argmax_count = torch.zeros(self.ARGMAX_ROWS, **i32)
        self._decode = None
        _all_scratch.add(self)

    def decode_buffers(self, requests: int, H: int, K: int, chunks: int, d: int):
        """Partial accumulators, partial (max, sum) and arrival counters of the split-KV decode kernel, at least as
        large as this call needs; they only ever grow, so layers of different head layouts share them."""
        need = requests * H * chunks
        sizes = (need * d, need * 2, requests * K)
        held = self._decode
        if held is None or any(t.numel() < n for t, n in zip(held, sizes)):
            sizes = tuple(max(n, t.numel()) for t, n in zip(held, sizes)) if held is not None else sizes
            held = (torch.empty(sizes[0], device=self.device, dtype=torch.float32),
                    torch.empty(sizes[1], device=self.device, dtype=torch.float32),
                    torch.zeros(sizes[2], device=self.device, dtype=torch.int32))
            self._decode = held
        return held

    def ids(self, rows: int) -> torch.Tensor:
        """Where a step's sampled ids go (int32 ``[rows]``), right behind the report."""
        if rows > self.RESULT_ROWS:
            raise KernelError(f"{rows} rows are sampled in one step; the result buffer holds {self.RESULT_ROWS}")
        return self.result[4:4 + rows]

    def read(self, rows: int):
        """The ids of ``ids(rows)`` as host ints (-1: that row's logits were not finite), read together with the
        report (one copy, one wait): raises ``KernelError`` if a kernel's wait gave up."""
        both = self.result[:4 + rows].tolist()
        if both[0]:
            self.clear()
            raise KernelError(f"a tensor-core kernel's wait on an mbarrier gave up (code {both[0]})")
        return both[4:]

    def check(self) -> None:
        """Raises if a kernel's bounded wait gave up since the last check (reads one int: synchronises)."""
        code = int(self.error.item())
        if code != 0:
            self.clear()
            raise KernelError(f"a tensor-core kernel's wait on an mbarrier gave up (code {code})")

    def clear(self) -> None:
        """After an error: a kernel that gave up may have left its counters and flags set."""
        self.error.zero_()
        self.report.zero_()
        self.parked_flags.zero_()
        self.argmax_keys.zero_()
        self.argmax_count.zero_()
        if self._decode is not None:
            self._decode[2].zero_()


_default_scratch = {}
_all_scratch = weakref.WeakSet()
_current_scratch: Optional[Scratch] = None


def _scratch_for(device) -> Scratch:
    if _current_scratch is not None and _current_scratch.device == device:
        return _current_scratch
    key = (device.type, device.index)
    s = _default_scratch.get(key)
    if s is None:
        s = _default_scratch[key] = Scratch(device)
    return s


class using:
    """``with ops.using(scratch): ...`` — the kernels launched inside take their scratch memory from ``scratch``."""

    def __init__(self, scratch: Optional[Scratch]):
        self.scratch = scratch

    def __enter__(self):
        global _current_scratch
        self.before, _current_scratch = _current_scratch, self.scratch
        return self.scratch

    def __exit__(self, *exc):
        global _current_scratch
        _current_scratch = self.before
        return False


def check_device_errors(device=None) -> None:
    """Raises if a kernel's bounded wait gave up since the last check, under any scratch of this process (on
    ``device`` if one is given).  Reads one int per scratch: synchronises."""
    for s in list(_all_scratch):
        if device is None or s.device == torch.device(device):
            s.check()


def gemm_plan(T: int, N: int, K: int):
    """Tokens per CTA and the number of K slices (1, 2, 4 or 8: the CTAs of one cluster) for the tensor-core
    kernel.  K is cut when there are fewer tiles than SMs, as far as every slice keeps at least 4 k-blocks."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
    tiles = -(-N // 128) * -(-T // bn)
    nkb = -(-K // 64)
    splits = 1
    if tiles < SM_COUNT:
        for cand in (8, 4, 2):
            per = -(-nkb // cand)
            if tiles * cand <= 2 * SM_COUNT + 32 and per >= 4 and (cand - 1) * per < nkb:
                splits = cand
                break
    return bn, splits


PERSISTENT_TILES = (128, 144, 160, 176, 192, 208, 224, 240, 256)
STREAM_K_TILES = (128, 192, 256)


def persistent_plan(T: int, N: int) -> int:
    """Tokens per tile for the persistent kernel: the tile width whose rounds over the SMs waste the least.
    A tile's time grows with its width plus a fixed part (ramp-up of the ring, the epilogue's tail)."""
    return _tile_by_tile(T, N)[1]


def _tile_by_tile(T: int, N: int):
    best = None
    for bn in PERSISTENT_TILES:
        tiles = -(-N // 128) * -(-T // bn)
        cost = -(-tiles // SM_COUNT) * (bn + 24)
        if best is None or cost < best[0]:
            best = (cost, bn)
    return best


def many_tokens(T: int, N: int, with_heads: bool = False) -> bool:
    """Whether a product of T tokens and N weight rows goes to the persistent kernel (else: one CTA per tile, K cut
    over the CTAs of a cluster where tiles are few).  It needs a round of tiles to be worth it: with fewer tiles than SMs
    the clusters' many CTAs ask for more at once (measured at Qwen3-4B sizes: the down product at 512 tokens 43 us
    against 52, at 768 tokens 45 against 53; o at 768 tokens 23 against 26).  The q|k|v product that finishes its heads
    stays persistent from half a round on: beyond 128 tokens only that kernel can finish them (17.6 us at 256 tokens
    against 18.2 plus the q/k kernel)."""
    tiles = -(-N // 128) * -(-T // 128)
    return T > 128 and tiles >= (SM_COUNT // 2 if with_heads else SM_COUNT)


#: the persistent kernel deals k-blocks instead of tiles over the SMs where whole tiles would leave SMs idle
stream_k = True


#: Stream-K against tile by tile, fitted to timings on B200 (2,048 and 1,024 tokens, layer sizes of 4B to 14B models):
#: a k-block of a 128 x bn tile costs about bn + 138 (the weight tile is fetched whatever the width), and stream-K
#: pays a fixed part worth 7,700 such units (about 8 us: every CTA parks a partial tile at the start and the last
#: epilogue, which nothing overlaps, is longer).  Measured times came out up to 0.1 above the predicted ratio, hence
#: the margin.  Groups walk different k at the same time, so x has to stay in L2 (at 71 MB stream-K lost 6 % where
#: the fit promised 9 %), and with fewer than four token tiles the fit did not hold (0.98 and 1.07 for 0.75 and 0.91).
_KBLOCK_FIXED, _STREAM_K_FIXED, _STREAM_K_MARGIN, _STREAM_K_MAX_X_BYTES = 138, 7700, 0.87, 48 << 20


def stream_k_plan(T: int, N: int, K: int) -> Optional[int]:
    """Tokens per tile if the product should run stream-K, else None.  The CTAs form groups, one CTA per token tile,
    and every group gets the same number of k-blocks of the weight-row tiles laid end to end: the time goes with
    row tiles / groups, without rounding up to whole rounds of tiles.  It needs at least one row tile per group."""
    if not stream_k:
        return None
    best = None
    rows, nkb = -(-N // 128), -(-K // 64)
    for bn in STREAM_K_TILES:
        across = -(-T // bn)
        if across > SM_COUNT or rows < SM_COUNT // across or (_STREAM_K_FIXED > 0 and (across < 4 or T * K * 2 > _STREAM_K_MAX_X_BYTES)):
            continue
        cost = rows / (SM_COUNT // across) * nkb * (bn + _KBLOCK_FIXED) + _STREAM_K_FIXED
        if best is None or cost <= best[0]:
            best = (cost, bn)
    if best is None:
        return None
    bn = persistent_plan(T, N)
    whole = -(-(rows * -(-T // bn)) // SM_COUNT) * nkb * (bn + _KBLOCK_FIXED)
    return best[1] if best[0] < _STREAM_K_MARGIN * whole else None


def _persistent_product(x, w, out, mode: int, T: int, N: int, K: int, s, what: str) -> None:
    lib = _lib("mb_gemm_tc")
    bn = stream_k_plan(T, N, K)
    if bn is not None:
        _check(lib.mb_gemm_tc_persistent_streamk(
            _ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K), _c_int(bn), _c_int(SM_COUNT),
            _ptr(s.parked), ctypes.c_longlong(s.parked.numel()), _ptr(s.parked_flags), _ptr(s.error), _stream()),
            what + ", stream-K")
        return
    _check(lib.mb_gemm_tc_persistent(_ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K),
                                     _c_int(persistent_plan(T, N)), _c_int(SM_COUNT), _ptr(s.error), _stream()), what)


class NormOut:
    """An RMS norm that may ride on a ``+=`` product: ``rows`` (activation dtype ``[T, N]``) is where the normed
    rows are wanted, ``weight`` float32 ``[N]``."""
    __slots__ = ("weight", "unit_offset", "eps", "rows")

    def __init__(self, weight: torch.Tensor, unit_offset: bool, eps: float, rows: torch.Tensor):
        self.weight, self.unit_offset, self.eps, self.rows = weight, bool(unit_offset), float(eps), rows


class NormedRows:
    """The input of a product whose RMS norm is half done: ``rows`` holds ``bf16(h * g)`` (g the norm's weight) and
    ``sumsq[slot, t]`` sums of squares of ``h[t]`` over disjoint groups of columns.  The product that reads it
    multiplies token ``t`` of its result by ``1 / sqrt(sum_slots sumsq[:, t] / dim + eps)``: the same value as
    normalising first, because the factor is one scalar per token.  Only ``gemm`` and ``gemm_swiglu`` read it."""
    __slots__ = ("rows", "sumsq", "slots", "dim", "eps")

    def __init__(self, rows, sumsq, slots, dim, eps):
        self.rows, self.sumsq, self.slots, self.dim, self.eps = rows, sumsq, slots, dim, eps

    shape = property(lambda self: self.rows.shape)
    dtype = property(lambda self: self.rows.dtype)
    device = property(lambda self: self.rows.device)


#: the most tokens for which a norm rides on the product before it.  The kernel takes up to 64; measured on B200
#: (Qwen3-4B layers) a decode step gains 5 % at 1 token and 3 % at 8, and loses 2 % at 64, where the norm's own
#: kernel is small beside the products.
COUPLED_NORM_MAX_TOKENS = 16


def gemm(x, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False, then_norm: Optional[NormOut] = None,
         activation: Optional[str] = None):
    """``out[t, n] (+)= sum_k x[t, k] * w[n, k]``.  bfloat16 inputs run on the tensor cores (tcgen05, float32
    accumulate); float32 inputs run on the CUDA cores in true float32.  ``activation`` "relu2": ``out = max(x w^T, 0)^2`` in
    the activation dtype, applied to the float32 sums in the tensor-core product's epilogue (as a kernel of its own behind
    the plain product).

    ``then_norm`` (with ``accumulate``) asks for the RMS norm of the updated ``out``: if this product can carry it,
    a ``NormedRows`` is returned for the next product to finish; otherwise None, and the caller runs the norm."""
    scaled = x if isinstance(x, NormedRows) else None
    if scaled is not None:
        x = scaled.rows
    _need_cuda(x, w, out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and tuple(out.shape) == (T, N), (x.shape, w.shape, out.shape)
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulate needs a float32 output")
    _cost(_size(w) + _size(x) + _size(out) * (2 if accumulate else 1) + (_size(then_norm.rows) if then_norm is not None else 0), 2.0 * T * N * K)
    if (use_tensor_cores and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and T > 0):
        mode = 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1)
        if activation is not None:
            if activation != "relu2" or accumulate or out.dtype != torch.bfloat16 or then_norm is not None:
                raise KernelError(f"gemm: activation {activation!r} goes with a plain bfloat16 output")
            mode = 4
        if many_tokens(T, N):
            s = _scratch_for(x.device)
            lib = _lib("mb_gemm_tc")
            carried = None
            if (then_norm is not None and accumulate and couple_norms and couple_norms_in_prefill and N % 8 == 0
                    and then_norm.rows.dtype == torch.bfloat16 and then_norm.rows.data_ptr() % 16 == 0):
                slots = int(lib.mb_gemm_tc_norm_slots(_c_int(N), _c_int(1)))
                if slots * T <= s.sumsq.numel():
                    carried = NormedRows(then_norm.rows, s.sumsq, slots, N, then_norm.eps)
            if carried is None and scaled is None:
                _persistent_product(x, w, out, mode, T, N, K, s, "gemm (tensor cores, persistent)")
                return None
            _check(lib.mb_gemm_tc_persistent_coupled(
                _ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K), _c_int(persistent_plan(T, N)), _c_int(SM_COUNT),
                _ptr(then_norm.weight) if carried is not None else None, _c_int(int(then_norm.unit_offset)) if carried is not None else _c_int(0),
                _ptr(carried.rows) if carried is not None else None, _ptr(carried.sumsq) if carried is not None else None,
                _ptr(scaled.sumsq) if scaled is not None else None, _c_int(scaled.slots if scaled is not None else 0),
                _c_int(scaled.dim if scaled is not None else 0), _c_float(scaled.eps if scaled is not None else 0.0),
                _ptr(s.error), _stream()), "gemm (tensor cores, persistent, coupled with a norm)")
            return carried
        bn, splits = gemm_plan(T, N, K)
        s = _scratch_for(x.device)
        lib = _lib("mb_gemm_tc")
        carried = None
        if (then_norm is not None and accumulate and couple_norms and T <= COUPLED_NORM_MAX_TOKENS and N % 8 == 0
                and then_norm.rows.dtype == torch.bfloat16 and then_norm.rows.data_ptr() % 16 == 0):
            slots = int(lib.mb_gemm_tc_norm_slots(_c_int(N), _c_int(splits)))
            if slots * T <= s.sumsq.numel():
                carried = NormedRows(then_norm.rows, s.sumsq, slots, N, then_norm.eps)
        if carried is None and scaled is None:
            _check(lib.mb_gemm_tc_cluster(_ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K),
                                          _c_int(bn), _c_int(splits), _ptr(s.error), _stream()), "gemm (tensor cores)")
            return None
        _check(lib.mb_gemm_tc_coupled(
            _ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K), _c_int(bn), _c_int(splits),
            _ptr(then_norm.weight) if carried is not None else None, _c_int(int(then_norm.unit_offset)) if carried is not None else _c_int(0),
            _ptr(carried.rows) if carried is not None else None, _ptr(carried.sumsq) if carried is not None else None,
            _ptr(scaled.sumsq) if scaled is not None else None, _c_int(scaled.slots if scaled is not None else 0),
            _c_int(scaled.dim if scaled is not None else 0), _c_float(scaled.eps if scaled is not None else 0.0),
            _ptr(s.error), _stream()), "gemm (tensor cores, coupled with a norm)")
        return carried
    assert scaled is None, "rows with a pending norm reach only the tensor-core product"
    _check(_lib("mb_gemm_simple").mb_gemm_simple(_ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), _c_int(T),
                                                _c_int(N), _c_int(K), _c_int(int(accumulate)), _stream()), "gemm")
    if activation is not None:
        if activation != "relu2" or accumulate:
            raise KernelError(f"gemm: activation {activation!r} goes with a plain output")
        relu2(out)
    return None


#: with few tokens the q|k|v product finishes its heads itself (norm, rotation, cache write) where the layout allows
fuse_heads = True
FUSED_HEADS_MAX_TOKENS = 128


#: the same for many tokens, in the persistent kernel's epilogue (tile by tile, no stream-K)
fuse_heads_many_tokens = True


def rope_table(ctx, positions, inv_freq) -> torch.Tensor:
    """cos and sin of ``positions * inv_freq`` for every token of the step, float32 ``[T, 2 * len(inv_freq)]`` (cos
    first), made once per step and position encoding and kept in ``ctx.extras``."""
    key = ("rope_table", inv_freq.data_ptr())
    table = ctx.extras.get(key)
    if table is None:
        T, half = positions.shape[0], inv_freq.shape[0]
        table = ctx.workspace.get(f"rope_table_{len(ctx.extras)}", (T, 2 * half), torch.float32)
        _cost(_size(table), 2.0 * T * half)
        _check(_lib("mb_elementwise").mb_rope_table(_ptr(positions), _ptr(inv_freq), _c_int(half), _ptr(table), _c_int(T), _stream()),
               "rope_table")
        ctx.extras[key] = table
    return table


def gemm_qkv_heads(x, w: torch.Tensor, q_out: torch.Tensor, q_weight, k_weight, eps: float, positions, inv_freq, rotary_dim: int,
                   interleaved: bool, slot_mapping, k_cache, v_cache, H: int, K: int, d: int, write_kv: bool = True, ctx=None) -> bool:
    """The product ``x w^T`` with ``w`` = query, key and value rows (or query rows only), each head normed, rotated
    and stored by the product's own epilogue: queries to ``q_out``, keys and values into the paged caches at
    ``slot_mapping``.  Two kernels do it: the one for up to sixteen tokens computes the angles itself; the persistent
    one for many tokens reads them from the step's table (``rope_table``, which needs ``ctx``).  Returns False,
    having done nothing, where neither applies (heads that are not 128 wide, a partial or interleaved rotation,
    float32, a token count between the two): the caller then runs ``gemm`` and ``qk_norm_rope_write``."""
    scaled = x if isinstance(x, NormedRows) else None
    rows = scaled.rows if scaled is not None else x
    T, Kdim = rows.shape
    N = w.shape[0]
    heads_total = H + 2 * K if write_kv else H
    if not (fuse_heads and use_tensor_cores and rows.is_cuda and rows.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and q_out.dtype == torch.bfloat16 and d == 128 and T > 0 and N == heads_total * d
            and Kdim % 8 == 0 and not interleaved and (inv_freq is None or rotary_dim == d)
            and rows.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (not write_kv or k_cache.dtype == torch.bfloat16)):
        return False
    page_size = k_cache.shape[2] if write_kv else 0
    if T > FUSED_HEADS_MAX_TOKENS:
        if not (fuse_heads_many_tokens and scaled is None and many_tokens(T, N, with_heads=True)
                and (inv_freq is None or ctx is not None)):
            return False
        _need_cuda(rows, w, q_out)
        assert tuple(q_out.shape) == (T, H * d) and w.shape[1] == Kdim
        table = rope_table(ctx, positions, inv_freq) if inv_freq is not None else None
        _cost(_size(w) + _size(rows) + T * N * 2 + (_size(table) if table is not None else 0), 2.0 * T * N * Kdim)
        s = _scratch_for(rows.device)
        _check(_lib("mb_gemm_tc").mb_gemm_tc_persistent_heads(
            _ptr(rows), _ptr(w), _c_int(T), _c_int(N), _c_int(Kdim), _c_int(persistent_plan(T, N)), _c_int(SM_COUNT), _ptr(q_out),
            _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, _ptr(q_weight), _ptr(k_weight), _c_float(eps),
            _ptr(table), _ptr(slot_mapping) if write_kv else None, _c_int(H), _c_int(K), _c_int(page_size), _ptr(s.error), _stream()),
            "gemm (persistent) with heads finished in the epilogue")
        return True
    bn, splits = gemm_plan(T, N, Kdim)
    if T > bn or splits < 2:
        return False
    _need_cuda(rows, w, q_out)
    assert tuple(q_out.shape) == (T, H * d) and w.shape[1] == Kdim
    _cost(_size(w) + _size(rows) + T * N * 2, 2.0 * T * N * Kdim)
    s = _scratch_for(rows.device)
    _check(_lib("mb_gemm_tc").mb_gemm_tc_heads(
        _ptr(rows), _ptr(w), _c_int(T), _c_int(N), _c_int(Kdim), _c_int(bn), _c_int(splits), _ptr(q_out),
        _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, _ptr(q_weight), _ptr(k_weight), _c_float(eps),
        _ptr(positions), _ptr(inv_freq), _ptr(slot_mapping) if write_kv else None, _c_int(H), _c_int(K), _c_int(page_size),
        _ptr(scaled.sumsq) if scaled is not None else None, _c_int(scaled.slots if scaled is not None else 0),
        _c_int(scaled.dim if scaled is not None else 0), _c_float(scaled.eps if scaled is not None else 0.0),
        _ptr(s.error), _stream()), "gemm with heads finished in the epilogue")
    return True


def qk_norm_rope_write(qkv, q_out, q_weight, k_weight, eps, positions, inv_freq, rotary_dim, interleaved,
                       slot_mapping, k_cache, v_cache, H, K, d, write_kv=True) -> None:
    _need_cuda(qkv, q_out, q_weight, k_weight, positions, inv_freq, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    heads_total = H + 2 * K if write_kv else H
    assert qkv.shape[1] == heads_total * d and tuple(q_out.shape) == (T, H * d) and q_out.dtype == qkv.dtype
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert k_cache.shape[1] == K and k_cache.shape[3] == d
    page_size = k_cache.shape[2]
    _cost(2 * _size(qkv), 8.0 * T * heads_total * d)
    _check(_lib("mb_elementwise").mb_qk_norm_rope_write(
        _ptr(qkv), _code(qkv), _ptr(q_out), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(positions),
        _ptr(inv_freq), _c_int(rotary_dim if inv_freq is not None else 0), _c_int(int(interleaved)), _ptr(slot_mapping),
        _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(page_size),
        _c_int(int(write_kv)), _stream()), "qk_norm_rope_write")


#: bf16 attention goes to the tensor-core / split-KV kernels when the head layout allows (False: the plain kernel)
use_fast_attention = True
#: prompt portions go to the tcgen05 attention kernel where it applies (heads of 64 or 128, pages >= 16)
use_tc_attention = True
DECODE_SPLITS = (4096, 2048, 1024, 512, 256, 128, 64)      # keys per CTA the split-KV decode kernel may be given
DECODE_CLUSTER_CHUNKS = 8                                   # most chunks the kernel merges as one cluster (see _attention_lib)
_cluster_asked = set()


def decode_split(requests: int, kv_heads: int, longest: int):
    """Keys per CTA and chunks per sequence for decode attention over sequences of up to ``longest`` keys.

    Up to eight chunks of one (request, kv head), sixteen where the device allows (``DECODE_CLUSTER_CHUNKS``), run as
    one thread-block cluster and merge through distributed shared memory; that is preferred, with chunks as long as still give 256 CTAs (measured on B200 at batch 1, 8 and 64 and
    contexts 1024 and 4096).  A few long sequences would leave most SMs idle that way: they get more chunks, merged
    through scratch memory, as long as still give 128 CTAs."""
    pairs = requests * kv_heads
    best = None
    for split in DECODE_SPLITS:
        chunks = -(-longest // split)
        if chunks > DECODE_CLUSTER_CHUNKS:
            break
        best = (split, chunks)
        if pairs * chunks >= 256:
            break
    if best is not None and (pairs * best[1] >= 128 or best[0] <= 1024):
        # clusters of 3, 5, 6 or 7 CTAs are placed badly (measured: 5 chunks take 36 us where 4 take 26): the grid
        # gets a power of two of chunks, those past the sequences' end have nothing to do and say so to their cluster
        chunks = 1
        while chunks < best[1]:
            chunks *= 2
        return best[0], chunks
    for split in DECODE_SPLITS:
        chunks = -(-longest // split)
        if pairs * chunks >= 128 or split == DECODE_SPLITS[-1]:
            return split, chunks


def _attention_lib(d: int, group: int):
    """The fast attention kernels are compiled for one head size and one group size, at first use.  A library also
    says how many chunks the device lets the decode kernel merge as one cluster (8, or 16 where clusters of a
    non-portable size can be placed): ``decode_split`` plans with the smallest answer so far."""
    global DECODE_CLUSTER_CHUNKS, _cluster_asked
    lib = build.load(f"mb_attention_fast_d{d}_g{group}", *build.attention_job(d, group))
    if (d, group) not in _cluster_asked and torch.cuda.is_available():
        widest = int(lib.mb_attn_decode_max_cluster())
        DECODE_CLUSTER_CHUNKS = widest if not _cluster_asked else min(DECODE_CLUSTER_CHUNKS, widest)
        _cluster_asked.add((d, group))
    return lib


def fast_attention_supported(dtype, H: int, K: int, d: int) -> bool:
    return dtype == torch.bfloat16 and d % 16 == 0 and 16 <= d <= 128 and H % K == 0 and 1 <= H // K <= 8


def decode_scratch(device, requests: int, H: int, K: int, chunks: int, d: int):
    """Scratch of the split-KV decode kernel: partial accumulators, partial (max, sum), and one counter per
    (request, kv head) that is zero between launches."""
    need = requests * H * chunks
    return (torch.empty(need * d, device=device, dtype=torch.float32), torch.empty(need * 2, device=device, dtype=torch.float32),
            torch.zeros(requests * K, device=device, dtype=torch.int32))


class DecodePlan:
    """How single-token attention splits its keys, fixed ahead for a captured graph: keys per CTA, chunks per
    sequence, and scratch memory of the capture's own (partial accumulators, partial (max, sum), counters)."""
    __slots__ = ("split", "chunks", "buffers")

    def __init__(self, split: int, chunks: int, buffers=None):
        self.split, self.chunks, self.buffers = int(split), int(chunks), buffers


def decode_plan(device, dtype, requests: int, H: int, K: int, d: int, span: int) -> Optional[DecodePlan]:
    """The plan for ``requests`` single-token requests over sequences of up to ``span`` keys, with scratch sized for
    exactly this head layout; None where the split-KV kernel does not apply (the plain kernel needs no plan)."""
    if not (use_fast_attention and fast_attention_supported(dtype, H, K, d)):
        return None
    _attention_lib(d, H // K)                        # the library says how wide a cluster may be: plan after asking
    split, chunks = decode_split(requests, K, span)
    return DecodePlan(split, chunks, decode_scratch(device, requests, H, K, chunks, d))


def attention_jobs(dtype, H: int, K: int, d: int) -> dict:
    """``{library: (sources, defines)}`` of the attention kernels a mixer of this head layout runs."""
    if not fast_attention_supported(dtype, H, K, d):
        return {"mb_attention_simple": (build.LIBRARIES["mb_attention_simple"], [])}
    jobs = {f"mb_attention_fast_d{d}_g{H // K}": build.attention_job(d, H // K)}
    if d in (64, 128):
        jobs[f"mb_attention_tc_d{d}_g{H // K}"] = build.attention_tc_job(d, H // K)
    return jobs


def _attention_cost(q, rows: int, H: int, K: int, d: int, which: str) -> None:
    """Queries in, results out; per cached key read, its key and value over all kv heads; per (query, key) pair a
    score and a weighted value for every head.  ``which`` says whose keys and pairs count: the single-token rows'
    ("decode"), the portions' ("prefill") or everyone's ("all")."""
    if launch_log is not None:
        size = q.element_size()
        _cost(2 * rows * H * d * size, 0.0, 2 * K * d * size, 4.0 * H * d)
        _pending_cost["rows"] = which


def attention(q, k_cache, v_cache, out, ctx, block_table, H, K, d, scale, window=0, plan: Optional[DecodePlan] = None) -> None:
    """Causal attention of the step's tokens over the paged cache (their own keys included).  The first
    ``ctx.num_decode`` requests bring one token each (rows 0..num_decode-1); the rest bring portions.  ``plan``
    fixes the split of the single-token rows' keys (a captured graph brings it); without one the split follows the
    longest sequence of the step."""
    _need_cuda(q, k_cache, v_cache, out, block_table)
    T = q.shape[0]
    page_size = k_cache.shape[2]
    assert tuple(q.shape) == (T, H * d) and out.shape == q.shape and k_cache.dtype == q.dtype
    if T == 0:
        return
    if use_fast_attention and fast_attention_supported(q.dtype, H, K, d):
        lib = _attention_lib(d, H // K)
        max_pages = block_table.shape[1]
        nd = ctx.num_decode
        if nd > 0:
            split, chunks = (plan.split, plan.chunks) if plan is not None else decode_split(nd, K, ctx.max_seq_len)
            buffers = plan.buffers if plan is not None and plan.buffers is not None else None
            part_acc, part_ml, counters = buffers or _scratch_for(q.device).decode_buffers(nd, H, K, chunks, d)
            _attention_cost(q, nd, H, K, d, "decode")
            _check(lib.mb_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                      _ptr(ctx.seq_lens), _c_int(nd), _c_int(K), _c_int(page_size),
                                      ctypes.c_longlong(k_cache.shape[0]), _c_float(scale), _c_int(window), _ptr(part_acc),
                                      _ptr(part_ml), _ptr(counters), _c_int(chunks), _c_int(split),
                                      _ptr(_scratch_for(q.device).error), _stream()), "attention (decode)")
        if ctx.num_requests > nd and use_tc_attention and d in (64, 128) and page_size >= 16:
            tc = build.load(f"mb_attention_tc_d{d}_g{H // K}", *build.attention_tc_job(d, H // K))
            _attention_cost(q, T - nd, H, K, d, "prefill")
            _check(tc.mb_attn_prefill_tc(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                         _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                         _c_int(ctx.max_query_len), _c_int(T), _c_int(K), _c_int(page_size),
                                         ctypes.c_longlong(k_cache.shape[0]), _c_float(scale), _c_int(window),
                                         _ptr(_scratch_for(q.device).error), _c_int(0), _c_int(0), _ptr(None), _c_int(0), _ptr(None), _stream()),
                   "attention (prefill, tensor cores)")
        elif ctx.num_requests > nd:
            _attention_cost(q, T - nd, H, K, d, "prefill")
            _check(lib.mb_attn_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                       _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                       _c_int(ctx.max_query_len), _c_int(K), _c_int(page_size), _c_float(scale),
                                       _c_int(window), _stream()), "attention (prefill)")
        return
    _attention_cost(q, T, H, K, d, "all")
    _check(_lib("mb_attention_simple").mb_attention_simple(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _code(q), _ptr(block_table), _c_int(block_table.shape[1]),
        _ptr(ctx.req_index), _ptr(ctx.positions), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(page_size),
        _c_float(scale), _c_int(window), _stream()), "attention")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """``out[t, i] = silu(g) * u``; gate and up are the two halves of a row of ``gate_up``, or (``interleaved``)
    alternate in blocks of 16 columns."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype and (not interleaved or I % 16 == 0)
    _cost(_size(gate_up) + _size(out), 8.0 * T * I)
    _check(_lib("mb_elementwise").mb_swiglu(_ptr(gate_up), _ptr(out), _code(out), _c_int(T), _c_int(I), _c_int(int(interleaved)),
                                           _stream()), "swiglu")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """One matrix whose rows alternate 16 gate rows and the 16 up rows of the same indices: the layout the
    fused SwiGLU epilogue of the matrix product reads (``[I, h]`` twice → ``[2 I, h]``; ``I`` a multiple of 16)."""
    I, h = gate.shape
    assert up.shape == gate.shape and I % 16 == 0
    return torch.stack([gate.view(I // 16, 16, h), up.view(I // 16, 16, h)], dim=1).reshape(2 * I, h)


def can_fuse_swiglu(dtype, hidden: int, intermediate: int) -> bool:
    return dtype == torch.bfloat16 and intermediate % 16 == 0 and hidden % 8 == 0


def gemm_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor, workspace=None) -> None:
    """``out = silu(x Wg^T) * (x Wu^T)`` with ``w_interleaved = interleave_gate_up(Wg, Wu)``: on the tensor cores the
    activation is applied to the float32 accumulators in the epilogue and the ``[T, 2 I]`` intermediate never
    exists; otherwise the product and the activation run as two kernels."""
    scaled = x if isinstance(x, NormedRows) else None
    if scaled is not None:
        x = scaled.rows
    _need_cuda(x, w_interleaved, out)
    T, K = x.shape
    N = w_interleaved.shape[0]
    I = N // 2
    assert tuple(out.shape) == (T, I) and w_interleaved.shape[1] == K and out.dtype == x.dtype
    fused = (use_tensor_cores and x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and K % 8 == 0
             and N % 32 == 0 and x.data_ptr() % 16 == 0 and w_interleaved.data_ptr() % 16 == 0 and T > 0)
    if not fused:
        tmp = workspace.get("gate_up", (T, N), x.dtype) if workspace is not None else torch.empty(T, N, device=x.device, dtype=x.dtype)
        gemm(scaled if scaled is not None else x, w_interleaved, tmp)
        swiglu(tmp, out, interleaved=True)
        return
    s = _scratch_for(x.device)
    _cost(_size(w_interleaved) + _size(x) + _size(out), 2.0 * T * N * K)
    if many_tokens(T, N):
        if scaled is not None:
            _check(_lib("mb_gemm_tc").mb_gemm_tc_persistent_coupled(
                _ptr(x), _ptr(w_interleaved), _ptr(out), _c_int(3), _c_int(T), _c_int(N), _c_int(K), _c_int(persistent_plan(T, N)),
                _c_int(SM_COUNT), None, _c_int(0), None, None, _ptr(scaled.sumsq), _c_int(scaled.slots), _c_int(scaled.dim),
                _c_float(scaled.eps), _ptr(s.error), _stream()), "gemm+swiglu (tensor cores, persistent, coupled with a norm)")
            return
        _persistent_product(x, w_interleaved, out, 3, T, N, K, s, "gemm+swiglu (tensor cores, persistent)")
        return
    bn, _ = gemm_plan(T, N, K)
    if scaled is not None:
        _check(_lib("mb_gemm_tc").mb_gemm_tc_coupled(
            _ptr(x), _ptr(w_interleaved), _ptr(out), _c_int(3), _c_int(T), _c_int(N), _c_int(K), _c_int(bn), _c_int(1),
            None, _c_int(0), None, None, _ptr(scaled.sumsq), _c_int(scaled.slots), _c_int(scaled.dim), _c_float(scaled.eps),
            _ptr(s.error), _stream()), "gemm+swiglu (tensor cores, coupled with a norm)")
        return
    _check(_lib("mb_gemm_tc").mb_gemm_tc_cluster(_ptr(x), _ptr(w_interleaved), _ptr(out), _c_int(3), _c_int(T), _c_int(N), _c_int(K),
                                                _c_int(bn), _c_int(1), _ptr(s.error), _stream()), "gemm+swiglu (tensor cores)")


def gemm_act(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, activation: str = "relu2") -> None:
    """``out = act(x w^T)`` in the activation dtype, for a feed-forward without a gate (``activation`` "relu2": the square of
    relu).  The tensor-core product applies it in its epilogue; behind the plain product it runs in place over the result."""
    if activation != "relu2":
        raise KernelError(f"gemm_act: unknown activation {activation!r}")
    gemm(x, w, out, activation=activation)


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(src, rows, out)
    W, h = out.shape
    assert src.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32 and rows.numel() == W
    _cost(2 * _size(out))
    _check(_lib("mb_elementwise").mb_gather_rows(_ptr(src), _ptr(rows), _ptr(out), _c_int(W), _c_int(h), _stream()), "gather_rows")


def add_into(y: torch.Tensor, x: torch.Tensor) -> None:
    """``y += x`` with ``y`` float32 (the residual stream)."""
    _need_cuda(y, x)
    assert y.dtype == torch.float32 and y.numel() == x.numel()
    _cost(2 * _size(y) + _size(x), float(y.numel()))
    _check(_lib("mb_elementwise").mb_add_into(_ptr(y), _ptr(x), _code(x), _c_size_t(y.numel()), _stream()), "add_into")


def argmax(logits: torch.Tensor, usable: int, out: torch.Tensor, feed: Optional[torch.Tensor] = None,
           mirror: Optional[torch.Tensor] = None, which: Optional[torch.Tensor] = None) -> None:
    """``out[r]`` = id of the largest of the first ``usable`` logits of row ``r`` (lowest id among equals); -1 for a
    row that holds a NaN or an infinity among them.

    ``feed`` (int32 ``[rows]`` on the device) receives the ids too (0 for such a row): the next step's token ids, for a
    step that is launched before the host has seen these.  ``mirror`` (pinned host memory, int32 ``[2, 4 + rows or more]``)
    with ``which`` (a device int, 0 or 1): row ``which`` of it receives the error code of the current scratch, three zeros
    and the ids, written by the kernel itself; the host reads them once an event recorded behind the launch has completed."""
    _need_cuda(logits, out, feed, which)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == rows
    assert feed is None or (feed.dtype == torch.int32 and feed.numel() >= rows)
    if mirror is not None:
        assert (mirror.dtype == torch.int32 and mirror.is_pinned() and mirror.dim() == 2 and mirror.shape[0] == 2 and mirror.is_contiguous()
                and mirror.shape[1] >= 4 + rows and which is not None and which.dtype == torch.int32 and rows <= _scratch_for(logits.device).ARGMAX_ROWS)
    s = _scratch_for(logits.device)
    _cost(rows * usable * 4)
    _check(_lib("mb_sampling").mb_argmax(_ptr(logits), _c_int(rows), _c_int(vocab), _c_int(usable), _ptr(out), _ptr(s.argmax_keys),
                                        _ptr(s.argmax_count), _c_int(s.ARGMAX_ROWS), _c_int(2 * s.sm_count), _ptr(s.report),
                                        _ptr(s.error), _ptr(feed), _ptr(mirror), _c_int(mirror.shape[1] if mirror is not None else 0),
                                        _ptr(which), _stream()), "argmax")


def sample(logits: torch.Tensor, usable: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor) -> None:
    """Draws one token per row from the reference's kept set (temperature, top-k, top-p; temperature 0 = greedy):
    ``uniform[r]`` in [0, 1) selects the token by walking the kept ids in increasing order.  Rows with a logit that is
    not finite get the id -1."""
    _need_cuda(logits, usable, temperature, top_k, top_p, uniform, out)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and usable.dtype == torch.int32 and top_k.dtype == torch.int32
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and uniform.dtype == torch.float32
    assert all(t.numel() == rows for t in (usable, temperature, top_k, top_p, uniform, out))
    s = _scratch_for(logits.device)
    _cost(_size(logits))
    _check(_lib("mb_sampling").mb_sample(_ptr(logits), _c_int(rows), _c_int(vocab), _ptr(usable), _ptr(temperature), _ptr(top_k),
                                        _ptr(top_p), _ptr(uniform), _ptr(out), _ptr(s.report), _ptr(s.error), _stream()), "sample")


# ---- norms and activations beside RMSNorm and SwiGLU (csrc/activations.cu) ---------------------------------------------

def dynamic_tanh(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], alpha: torch.Tensor, out: torch.Tensor) -> None:
    """``out = tanh(alpha * x) * weight + bias`` element by element; ``x`` float32 ``[rows, n]``, ``alpha`` one float32 on the device."""
    _need_cuda(x, weight, bias, alpha, out)
    rows, n = x.shape
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == n and out.shape == x.shape
    assert alpha.dtype == torch.float32 and alpha.numel() == 1 and (bias is None or (bias.dtype == torch.float32 and bias.numel() == n))
    _cost(_size(x) + _size(out) + 2 * _size(weight), 4.0 * rows * n)
    _check(_lib("mb_activations").mb_dyt(_ptr(x), _ptr(weight), _ptr(bias), _ptr(alpha), _ptr(out), _code(out), _c_int(rows), _c_int(n),
                                        _stream()), "dynamic tanh")


def polynorm(z: torch.Tensor, coef: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out = a N(z) + b N(z^2) + c N(z^3) + e`` with ``coef = (a, b, c, e)`` (float32 on the device) and ``N`` a row divided by
    its root mean square (``eps`` under the root); sums in float32."""
    _need_cuda(z, coef, out)
    rows, n = z.shape
    assert coef.dtype == torch.float32 and coef.numel() == 4 and out.shape == z.shape
    _cost(2 * _size(z) + _size(out), 12.0 * rows * n)
    _check(_lib("mb_activations").mb_polynorm(_ptr(z), _code(z), _ptr(coef), _c_float(eps), _ptr(out), _code(out), _c_int(rows), _c_int(n),
                                             _stream()), "polynorm")


GATES = {"sigmoid": 0, "silu": 1, None: 2}


def gated_rmsnorm(o: torch.Tensor, weight: torch.Tensor, gate_rows: Optional[torch.Tensor], gate: Optional[str], eps: float,
                  out: torch.Tensor) -> None:
    """``out = o / sqrt(mean(o^2) + eps) * weight * gate(gate_rows)`` over whole rows; ``o`` float32 ``[rows, n]``, ``gate_rows``
    ``[rows, n]`` in the activation dtype (it may be a column slice of a wider matrix), ``gate`` "sigmoid", "silu" or None."""
    _need_cuda(o, weight, out)
    rows, n = o.shape
    assert o.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == n and tuple(out.shape) == (rows, n)
    stride = 0
    if gate is not None:
        assert gate_rows is not None and gate_rows.is_cuda and gate_rows.dtype == out.dtype and tuple(gate_rows.shape) == (rows, n)
        assert gate_rows.stride(1) == 1
        stride = gate_rows.stride(0)
    _cost(_size(o) + 2 * _size(out), 8.0 * rows * n)
    _check(_lib("mb_activations").mb_gated_rmsnorm(_ptr(o), _ptr(weight), _ptr(gate_rows if gate is not None else None), _c_int(stride),
                                                  _c_int(GATES[gate]), _c_float(eps), _ptr(out), _code(out), _c_int(rows), _c_int(n),
                                                  _stream()), "gated rmsnorm")


def shift_mix(h: torch.Tensor, carry: torch.Tensor, ctx, slots: torch.Tensor, mu: torch.Tensor, out: torch.Tensor) -> None:
    """``out[m, t] = h[t] + (h'[t] - h[t]) * mu[m]`` with ``h'`` the row before in the same sequence; before a request's first
    token of this step it is the row its state keeps: ``carry`` is that part of the state tensor, float32 ``[slots, n]`` (a
    column slice: its row stride is the state's)."""
    _need_cuda(h, mu, out, slots)
    T, n = h.shape
    mixes = mu.shape[0]
    assert carry.is_cuda and carry.dtype == torch.float32 and carry.shape[1] == n and carry.stride(1) == 1
    assert mu.dtype == torch.float32 and tuple(mu.shape) == (mixes, n) and tuple(out.shape) == (mixes, T, n) and out.dtype == h.dtype
    _cost(_size(h) + _size(out), 2.0 * mixes * T * n)
    _check(_lib("mb_activations").mb_shift_mix(_ptr(h), _code(h), _c_void_p(carry.data_ptr()), ctypes.c_longlong(carry.stride(0)),
                                              _ptr(ctx.req_index), _ptr(ctx.cu_tokens), _ptr(slots), _ptr(mu), _c_int(mixes), _ptr(out),
                                              _c_int(T), _c_int(n), _stream()), "token shift")


def tanh_cap(x: torch.Tensor, cap: float) -> None:
    """``x <- cap * tanh(x / cap)`` in place (``cap = 1``: a plain tanh)."""
    _need_cuda(x)
    _cost(2 * _size(x), 2.0 * x.numel())
    _check(_lib("mb_activations").mb_tanh_cap(_ptr(x), _code(x), _c_size_t(x.numel()), _c_float(cap), _stream()), "tanh cap")


def relu2(x: torch.Tensor) -> None:
    """``x <- max(x, 0)^2`` in place: the activation of a feed-forward without a gate."""
    _need_cuda(x)
    _cost(2 * _size(x), 2.0 * x.numel())
    _check(_lib("mb_activations").mb_relu2(_ptr(x), _code(x), _c_size_t(x.numel()), _stream()), "relu squared")


# ---- recurrences with a matrix state per head (csrc/recurrent.cu) ------------------------------------------------------

def linear_attention_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, ctx,
                          slots: torch.Tensor, o: torch.Tensor, heads: int, dim: int, vdim: int) -> None:
    """``S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t`` per head over each request's tokens of the step, from and into
    ``state[slot]`` (float32 ``[slots, heads, dim, vdim]``).  ``q``, ``k``, ``v`` are column slices of one projection (before
    their silu, which the kernel applies); ``o`` float32 ``[T, heads * vdim]``."""
    _need_cuda(decay, state, o, slots)
    T = q.shape[0]
    stride = q.stride(0)
    assert q.is_cuda and q.dtype == k.dtype == v.dtype and k.stride(0) == stride and v.stride(0) == stride
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    assert tuple(q.shape) == (T, heads * dim) and tuple(k.shape) == (T, heads * dim) and tuple(v.shape) == (T, heads * vdim)
    assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dim, vdim) and decay.dtype == torch.float32 and decay.numel() == heads
    assert o.dtype == torch.float32 and tuple(o.shape) == (T, heads * vdim)
    R = ctx.num_requests
    _cost(T * heads * (2 * dim + vdim) * q.element_size() + _size(o) + 2.0 * R * heads * dim * vdim * 4, 4.0 * T * heads * dim * vdim)
    _check(_lib("mb_recurrent").mb_linear_attention_scan(
        _c_void_p(q.data_ptr()), _c_void_p(k.data_ptr()), _c_void_p(v.data_ptr()), _code(q), _c_int(stride), _ptr(decay), _ptr(state),
        _ptr(ctx.cu_tokens), _ptr(slots), _ptr(o), _c_int(R), _c_int(heads), _c_int(dim), _c_int(vdim), _stream()), "linear attention (scan)")


#: prompt portions of a bf16 linear-attention layer run in chunks of 64 tokens on the tensor cores where the head layout allows
use_chunked_linear_attention = True


def linear_attention_chunked_supported(dtype, dim: int, vdim: int) -> bool:
    return dtype == torch.bfloat16 and dim % 16 == 0 and 16 <= dim <= 128 and vdim % 32 == 0


def _chunked_slice(vdim: int) -> int:
    """Value channels a CTA of the chunked kernel takes.  32: twice the CTAs for a head (each repeats the small q k^T product);
    a request's tokens are walked in order by one CTA per head and slice, so more, lighter CTAs fill more of the device."""
    return 32


def _chunked_job(dim: int, vdim: int) -> tuple:
    return (["linear_attention_chunked.cu"], [f"QK_DIM={dim}", f"V_SLICE={_chunked_slice(vdim)}"])


def linear_attention_jobs(dtype, dim: int, vdim: int) -> dict:
    """The kernels a linear-attention mixer of this head layout runs: the scan (any size, both dtypes; single tokens) and,
    where the layout allows, the chunked tensor-core kernel for prompt portions."""
    jobs = library_jobs("mb_activations", "mb_recurrent")
    if use_chunked_linear_attention and linear_attention_chunked_supported(dtype, dim, vdim):
        jobs[f"mb_linear_attention_chunked_d{dim}_v{_chunked_slice(vdim)}"] = _chunked_job(dim, vdim)
    return jobs


def linear_attention_chunked(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, ctx,
                             slots: torch.Tensor, o: torch.Tensor, heads: int, dim: int, vdim: int) -> None:
    """The same recurrence as ``linear_attention_scan``, 64 tokens at a time on the tensor cores (bf16 operands, the state
    and the weights in float32, split into two bf16 numbers where they are operands)."""
    _need_cuda(decay, state, o, slots)
    T = q.shape[0]
    stride = q.stride(0)
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16 and k.stride(0) == stride and v.stride(0) == stride
    assert tuple(q.shape) == (T, heads * dim) and tuple(k.shape) == (T, heads * dim) and tuple(v.shape) == (T, heads * vdim)
    assert state.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dim, vdim) and decay.numel() == heads
    assert o.dtype == torch.float32 and tuple(o.shape) == (T, heads * vdim)
    R = ctx.num_requests
    _cost(T * heads * (2 * dim + vdim) * 2 + _size(o) + 2.0 * R * heads * dim * vdim * 4, 4.0 * T * heads * dim * vdim + 4.0 * T * 64 * heads * (dim + vdim) / 2)
    lib = build.load(f"mb_linear_attention_chunked_d{dim}_v{_chunked_slice(vdim)}", *_chunked_job(dim, vdim))
    _check(lib.mb_linear_attention_chunked(
        _c_void_p(q.data_ptr()), _c_void_p(k.data_ptr()), _c_void_p(v.data_ptr()), _c_int(stride), _ptr(decay), _ptr(state),
        _ptr(ctx.cu_tokens), _ptr(slots), _ptr(o), _c_int(R), _c_int(heads), _c_int(vdim), _stream()), "linear attention (chunked)")


#: bf16 time mixing cuts long prompt portions into blocks of this many tokens that are walked side by side (0: never)
WKV_BLOCK_TOKENS = 128
#: ... when the step's longest portion has at least this many tokens
WKV_BLOCKS_FROM = 256


def wkv_scan(r, k, v, wraw, w0, u, state: torch.Tensor, carry: torch.Tensor, h: torch.Tensor, ctx, slots: torch.Tensor,
             o: torch.Tensor, heads: int, dim: int) -> None:
    """``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t; S_t = diag(w_t) S_(t-1) + k_t v_t^T`` with ``w = exp(-exp(wraw + w0))``; ``o``
    float32 ``[T, heads * dim]`` before its norm (``head_norm_gate``).  ``state`` and ``carry`` are column slices of one float32
    state tensor (``[slots, heads * dim * dim]`` and ``[slots, width]``); the last row of ``h`` of every request goes to ``carry``.

    The recurrence is linear in the state, so a long portion (bfloat16 mode, key sizes 16, 32, 64, 128) is cut into blocks that
    are walked side by side: each from a zero state for its end state and the product of its decays; a short pass turns these
    into the states the blocks start from (``S <- W_b S + S_b``, block after block); each block again from its true start, for
    the outputs.  Twice the arithmetic, on all of the device instead of one CTA per head.  The result differs from the single
    walk by rounding (the sums are associated differently), which is why the 32-bit path never does it."""
    _need_cuda(r, k, v, wraw, w0, u, h, o, slots)
    T, n = r.shape
    assert n == heads * dim and all(tuple(x.shape) == (T, n) and x.dtype == r.dtype for x in (k, v))
    assert wraw.dtype == torch.float32 and tuple(wraw.shape) == (T, n) and all(x.dtype == torch.float32 and x.numel() == n for x in (w0, u))
    assert o.dtype == torch.float32 and tuple(o.shape) == (T, n)
    assert state.dtype == torch.float32 and carry.dtype == torch.float32 and state.stride(0) == carry.stride(0)
    assert state.shape[1] == heads * dim * dim and carry.shape[1] == h.shape[1] and h.dtype == r.dtype and h.shape[0] == T
    R = ctx.num_requests
    nblocks, block_state, block_decay = 1, None, None
    if (WKV_BLOCK_TOKENS and r.dtype == torch.bfloat16 and dim in (16, 32, 64, 128) and ctx.max_query_len >= WKV_BLOCKS_FROM):
        nblocks = -(-ctx.max_query_len // WKV_BLOCK_TOKENS)
        block_state = ctx.workspace.get("wkv_block_state", (R * nblocks, heads, dim, dim), torch.float32)
        block_decay = ctx.workspace.get("wkv_block_decay", (R * nblocks, heads, dim), torch.float32)
    _cost(3 * _size(r) + _size(wraw) + _size(o) + 2.0 * R * heads * dim * dim * 4, 6.0 * T * heads * dim * dim * (2 if nblocks > 1 else 1))
    _check(_lib("mb_recurrent").mb_wkv_scan(
        _ptr(r), _ptr(k), _ptr(v), _code(r), _ptr(wraw), _ptr(w0), _ptr(u), _c_void_p(state.data_ptr()), _c_void_p(carry.data_ptr()),
        ctypes.c_longlong(state.stride(0)), _ptr(h), _c_int(h.shape[1]), _ptr(ctx.cu_tokens), _ptr(slots), _ptr(o), _c_int(R),
        _c_int(heads), _c_int(dim), _ptr(block_state), _ptr(block_decay), _c_int(nblocks), _c_int(WKV_BLOCK_TOKENS or 1), _stream()),
        "wkv (blocks: from zero)" if nblocks > 1 else "wkv (scan)")
    if nblocks > 1:                       # three kernels were launched: the blocks from zero, the combination, the blocks again
        launches_extra(2)
        if launch_log is not None:
            for what in ("wkv (blocks: start states)", "wkv (blocks: outputs)"):
                launch_log.append({"bytes": 0.0, "flops": 0.0, "bytes_per_key": 0.0, "flops_per_pair": 0.0, "stage": stage_name, "kernel": what})


def head_norm_gate(o: torch.Tensor, weight: torch.Tensor, g: torch.Tensor, eps: float, out: torch.Tensor, heads: int, dim: int) -> None:
    """Each head's ``o`` divided by its own root mean square (``eps`` under the root), times ``weight`` (float32 ``[heads * dim]``),
    times ``silu(g)``; ``o`` float32 ``[T, heads * dim]``, ``g`` and ``out`` in the activation dtype."""
    _need_cuda(o, weight, g, out)
    T = o.shape[0]
    assert o.dtype == torch.float32 and tuple(o.shape) == (T, heads * dim) and g.shape == o.shape and out.shape == o.shape
    assert g.dtype == out.dtype and weight.dtype == torch.float32 and weight.numel() == heads * dim
    _cost(_size(o) + _size(g) + _size(out), 8.0 * o.numel())
    _check(_lib("mb_recurrent").mb_head_norm_gate(_ptr(o), _ptr(weight), _ptr(g), _code(g), _c_float(eps), _ptr(out), _c_int(T),
                                                 _c_int(heads), _c_int(dim), _stream()), "head norm, gate")


# ---- attention with sigmoid weights (csrc/attention_sigmoid.cu) ---------------------------------------------------------

def qkv_heads_sigmoid(qkv, q_out, q_weight, k_weight, eps: float, positions, temp_coef: float, temp_every: int, slot_mapping,
                      k_cache, v_cache, H: int, K: int, d: int, dv: int, write_kv: bool = True) -> None:
    """Finishes the heads of a fused q|k|v projection: per-head RMS norm of q and k (weights shared by the heads), queries times
    ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)``, keys (``d`` wide) and values (``dv`` wide) into their pages."""
    _need_cuda(qkv, q_out, positions, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    assert qkv.shape[1] == ((H + K) * d + K * dv if write_kv else H * d) and tuple(q_out.shape) == (T, H * d)
    page_size = k_cache.shape[2]
    _cost(_size(qkv) * 2)
    _check(_lib("mb_attention_sigmoid").mb_qkv_heads_sigmoid(
        _ptr(qkv), _code(qkv), _ptr(q_out), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(positions), _c_float(temp_coef),
        _c_int(temp_every), _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(dv),
        _c_int(page_size), _c_int(int(write_kv)), _stream()), "q|k|v heads (sigmoid attention)")


#: bf16 sigmoid attention goes to the tensor-core kernels where the head layout allows (False: always the plain kernel)
use_fast_sigmoid_attention = True


def fast_sigmoid_attention_supported(dtype, H: int, K: int, d: int, dv: int) -> bool:
    return (dtype == torch.bfloat16 and d % 16 == 0 and dv % 16 == 0 and 16 <= d <= 128 and 16 <= dv <= 128
            and H % K == 0 and 1 <= H // K <= 8)


def _sigmoid_job(d: int, dv: int, group: int) -> tuple:
    return (["attention_sigmoid_fast.cu"], [f"HEAD_DIM={d}", f"V_DIM={dv}", f"GROUP={group}"])


def _sigmoid_lib(d: int, dv: int, group: int):
    return build.load(f"mb_attention_sigmoid_fast_d{d}_v{dv}_g{group}", *_sigmoid_job(d, dv, group))


class SigmoidDecodePlan:
    """How single-token sigmoid attention splits a sequence's keys over CTAs: ``split`` keys (a multiple of 64) per chunk,
    ``chunks`` chunks cover the longest sequence.  The parts add up, so any split gives the same sum up to rounding."""
    __slots__ = ("split", "chunks")

    def __init__(self, split: int, chunks: int):
        self.split, self.chunks = int(split), int(chunks)


def sigmoid_decode_plan(requests: int, K: int, longest: int) -> SigmoidDecodePlan:
    """Enough chunks for about four CTAs per SM over all requests and kv heads, none shorter than 64 keys."""
    want = max(1, -(-4 * SM_COUNT // max(1, requests * K)))
    split = max(64, -(-(-(-max(longest, 1) // want)) // 64) * 64)
    return SigmoidDecodePlan(split, max(1, -(-max(longest, 1) // split)))


def attention_sigmoid(q, k_cache, v_cache, out, ctx, block_table, bias: torch.Tensor, H: int, K: int, d: int, dv: int, scale: float,
                      plan: Optional[SigmoidDecodePlan] = None) -> None:
    """``out_i = sum_{j <= i} sigmoid(q_i . k_j * scale + bias[head, min(i - j, span - 1)]) v_j`` over the paged cache; ``bias``
    float32 ``[H, span]``.  The first ``ctx.num_decode`` requests bring one token each, the rest portions.  ``plan`` fixes the
    split of the single tokens' keys (a captured graph brings it); without one it follows the step's longest sequence."""
    _need_cuda(q, k_cache, v_cache, out, block_table, bias)
    T = q.shape[0]
    page_size = k_cache.shape[2]
    assert tuple(q.shape) == (T, H * d) and tuple(out.shape) == (T, H * dv) and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
    assert bias.dtype == torch.float32 and bias.shape[0] == H and k_cache.shape[3] == d and v_cache.shape[3] == dv
    if T == 0:
        return
    size = q.element_size()
    span = bias.shape[1]
    if use_fast_sigmoid_attention and fast_sigmoid_attention_supported(q.dtype, H, K, d, dv) and page_size & (page_size - 1) == 0:
        lib = _sigmoid_lib(d, dv, H // K)
        max_pages = block_table.shape[1]
        nd = ctx.num_decode
        if nd > 0:
            if plan is None:
                plan = sigmoid_decode_plan(nd, K, ctx.max_seq_len)
            part = ctx.workspace.get("sigmoid_parts", (plan.chunks, nd, H, dv), torch.float32)
            if launch_log is not None:
                _cost(nd * H * (d + dv) * size, 0.0, K * (d + dv) * size, 2.0 * H * (d + dv))
                _pending_cost["rows"] = "decode"
            _check(lib.mb_attn_sigmoid_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(part), _ptr(block_table),
                                              _c_int(max_pages), _ptr(ctx.seq_lens), _c_int(nd), _c_int(K), _c_int(page_size),
                                              _c_float(scale), _ptr(bias), _c_int(span), _c_int(plan.split), _c_int(plan.chunks),
                                              _stream()), "attention (sigmoid, decode)")
            _cost(plan.chunks * nd * H * dv * 4 + nd * H * dv * size)
            _check(lib.mb_attn_sigmoid_merge(_ptr(part), _ptr(out), _ptr(ctx.seq_lens), _c_int(nd), _c_int(K), _c_int(plan.split), _stream()),
                   "attention (sigmoid, parts added)")
        if ctx.num_requests > nd:
            if launch_log is not None:
                _cost((T - nd) * H * (d + dv) * size, 0.0, K * (d + dv) * size, 2.0 * H * (d + dv))
                _pending_cost["rows"] = "prefill"
            _check(lib.mb_attn_sigmoid_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                               _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                               _c_int(ctx.max_query_len), _c_int(K), _c_int(page_size), _c_float(scale), _ptr(bias),
                                               _c_int(span), _stream()), "attention (sigmoid, prefill)")
        return
    if launch_log is not None:
        _cost(T * H * (d + dv) * size, 0.0, K * (d + dv) * size, 2.0 * H * (d + dv))
        _pending_cost["rows"] = "all"
    _check(_lib("mb_attention_sigmoid").mb_attention_sigmoid(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _code(q), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(ctx.req_index),
        _ptr(ctx.positions), _ptr(bias), _c_int(bias.shape[1]), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(dv), _c_int(page_size),
        _c_float(scale), _stream()), "attention (sigmoid)")


def library_jobs(*names: str) -> dict:
    """``{library: (sources, defines)}`` for libraries of the package that a part wants compiled before its model first runs."""
    return {n: (build.LIBRARIES[n], []) for n in names}


def sigmoid_attention_jobs(dtype, H: int, K: int, d: int, dv: int) -> dict:
    """The kernels a sigmoid-attention mixer of this head layout runs: the head preparation and the plain kernel, and the
    tensor-core kernels compiled for the layout where it allows."""
    jobs = library_jobs("mb_attention_sigmoid")
    if use_fast_sigmoid_attention and fast_sigmoid_attention_supported(dtype, H, K, d, dv):
        jobs[f"mb_attention_sigmoid_fast_d{d}_v{dv}_g{H // K}"] = _sigmoid_job(d, dv, H // K)
    return jobs


# ---- hyper-connections: the residual kept as several streams ------------------------------------------------------------------
def hc_step(streams: torch.Tensor, y: Optional[torch.Tensor], write=None, read=None) -> None:
    """One pass over the residual streams (float32 ``[S, T, h]``) between two sublayers.  ``write = (mix [S, S], out [S])``:
    ``x_t <- sum_s mix[s, t] x_s + out[t] y`` for all streams at once, ``y`` (float32 ``[T, h]``) the sublayer's output.
    ``read = (w_in [S], norm_weight [h], eps, unit_offset, rows)``: ``rows <- rmsnorm(sum_s w_in[s] x_s)`` of the streams as
    they are after the write, in ``rows``' dtype.  ``y`` is left zeroed for the next sublayer to add into."""
    _need_cuda(streams, y)
    S, T, h = streams.shape
    assert streams.dtype == torch.float32 and (y is None or (y.dtype == torch.float32 and tuple(y.shape) == (T, h)))
    mix = w_out = w_in = norm_w = rows = None
    eps, unit = 0.0, False
    if write is not None:
        mix, w_out = write
        assert y is not None and mix.dtype == torch.float32 and tuple(mix.shape) == (S, S) and w_out.numel() == S
    if read is not None:
        w_in, norm_w, eps, unit, rows = read
        assert w_in.numel() == S and norm_w.numel() == h and tuple(rows.shape) == (T, h)
    _cost(_size(streams) * (2 if write is not None else 1) + (_size(y) * 2 if y is not None else 0) + (_size(rows) if rows is not None else 0),
          2.0 * T * h * S * (S + 1))
    _check(_lib("mb_hyper").mb_hc_step(_ptr(streams), _c_int(S), _c_int(T), _c_int(h), _ptr(mix), _ptr(w_out), _ptr(y), _ptr(w_in),
                                      _ptr(norm_w), _c_float(eps), _c_int(int(unit)), _ptr(rows),
                                      _c_int(_code(rows) if rows is not None else F32), _stream()), "hyper-connection step")


def hc_spread(streams: torch.Tensor) -> None:
    """Stream 0 copied to all others."""
    _need_cuda(streams)
    S, T, h = streams.shape
    assert streams.dtype == torch.float32
    if S > 1 and T > 0:
        _cost(_size(streams))
        _check(_lib("mb_hyper").mb_hc_spread(_ptr(streams), _c_int(S), _c_int(T), _c_int(h), _stream()), "streams spread")


def hc_sum(streams: torch.Tensor, rows: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out[r] = sum_s streams[s, rows[r]]`` (``rows`` None: every token in order)."""
    _need_cuda(streams, rows, out)
    S, T, h = streams.shape
    count = out.shape[0]
    assert out.dtype == torch.float32 and out.shape[1] == h and (rows is None or (rows.dtype == torch.int32 and rows.numel() == count))
    assert rows is not None or count == T
    _cost(count * h * 4 * (S + 1))
    _check(_lib("mb_hyper").mb_hc_sum(_ptr(streams), _c_int(S), _c_int(T), _c_int(h), _ptr(rows), _ptr(out), _c_int(count), _stream()),
           "streams summed")


# ---- softmax attention with a sink, a chunked mask, values of their own width and an output gate ------------------------------
NORM_MODES = {None: 0, "head": 1, "whole": 2}
VALUE_MODES = {None: 0, "leave": 1, "mix": 2}


def qkv_finish(rows: torch.Tensor, q_out: torch.Tensor, q_b, k_b, v_b, norm: Optional[str], q_w, k_w, eps: float, positions,
               inv_freq, rot_dim: int, rot_mag: float, slot_mapping, k_cache, v_cache, value_mode: Optional[str], v_shared,
               v_lambda, H: int, K: int, d: int, dv: int, write_kv: bool = True, interleaved: bool = False) -> None:
    """Finishes the heads of a fused projection whose rows hold q | k | v (| more columns that are left alone): biases, the
    RMS norm of q and k (``norm`` "head": per head with a weight ``[d]``; "whole": over the whole of q, and of k, with weights
    ``[H d]`` / ``[K d]``), the rotation of the first ``rot_dim`` elements of each head (half-split pairs, or neighbours
    ``(2i, 2i + 1)`` if ``interleaved``; sines and cosines times ``rot_mag``), and the values: as they are, also left in ``v_shared`` ("leave"), or mixed with what ``v_shared`` holds,
    ``(1 - lam) v + lam v_shared`` ("mix").  Queries go to ``q_out``, keys and values into their pages."""
    _need_cuda(rows, q_out, q_b, k_b, v_b, q_w, k_w, positions, inv_freq, slot_mapping, k_cache, v_cache, v_shared, v_lambda)
    T = rows.shape[0]
    assert tuple(q_out.shape) == (T, H * d) and q_out.dtype == rows.dtype and rows.shape[1] >= ((H + K) * d + K * dv if write_kv else H * d)
    assert k_cache.dtype == rows.dtype and v_cache.dtype == rows.dtype and k_cache.shape[3] == d and v_cache.shape[3] == dv
    assert v_shared is None or (v_shared.dtype == rows.dtype and v_shared.numel() >= T * K * dv)
    page_size = k_cache.shape[2]
    _cost(2 * T * ((H + K) * d + K * dv) * rows.element_size(), 10.0 * T * (H + K) * d)
    _check(_lib("mb_attention_sink").mb_qkv_finish(
        _ptr(rows), _c_int(rows.shape[1]), _code(rows), _ptr(q_out), _ptr(q_b), _ptr(k_b), _ptr(v_b), _c_int(NORM_MODES[norm]), _ptr(q_w),
        _ptr(k_w), _c_float(eps), _ptr(positions), _ptr(inv_freq), _c_int(rot_dim if inv_freq is not None else 0), _c_float(rot_mag),
        _ptr(slot_mapping), _ptr(k_cache), _ptr(v_cache), _c_int(VALUE_MODES[value_mode]), _ptr(v_shared), _ptr(v_lambda), _c_int(T),
        _c_int(H), _c_int(K), _c_int(d), _c_int(dv), _c_int(page_size), _c_int(int(write_kv)), _c_int(int(interleaved)), _stream()),
        "q|k|v heads (sink attention)")


def attention_sink(q, k_cache, v_cache, out, ctx, block_table, H: int, K: int, d: int, dv: int, scale: float, window: int = 0,
                   chunk: int = 0, sink: bool = True, gate: Optional[torch.Tensor] = None, plan=None,
                   sink_logits: Optional[torch.Tensor] = None) -> None:
    """Causal softmax attention of the step's tokens over the paged cache.  A position sees the keys before it (its own
    included), of them only the last ``window`` (0: all) and only those of its own chunk of ``chunk`` positions (0: no
    chunks).  ``sink``: ``exp(sink_logits[head])`` is added to the softmax's denominator (float32 ``[H]``, not scaled; None: a
    score of 0, so one is added).  ``gate`` (activation dtype, a view ``[T, H dv]`` whose rows may be strided): the result is
    multiplied by ``sigmoid(gate)``.  ``v_cache`` may be ``k_cache`` itself: the values are then the first ``dv`` elements
    of the key rows (a latent that keys and values share)."""
    _need_cuda(q, k_cache, v_cache, out, block_table, sink_logits)
    T = q.shape[0]
    page_size = k_cache.shape[2]
    values_in_keys = v_cache.data_ptr() == k_cache.data_ptr()
    assert tuple(q.shape) == (T, H * d) and tuple(out.shape) == (T, H * dv) and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
    assert k_cache.shape[3] == d and (v_cache.shape[3] == dv or (values_in_keys and dv <= d))
    assert sink_logits is None or (sink and sink_logits.dtype == torch.float32 and sink_logits.numel() == H)
    v_stride = d if values_in_keys else dv
    gate_stride = 0
    if gate is not None:
        assert gate.is_cuda and gate.dtype == q.dtype and tuple(gate.shape) == (T, H * dv) and gate.stride(1) == 1
        gate_stride = gate.stride(0)
    if T == 0:
        return
    size = q.element_size()
    per_row = H * (d + (3 if gate is not None else 2) * dv) * size
    key_bytes = (d if values_in_keys else K * (d + dv)) * size      # what one cached position holds for this layer
    if use_fast_sink_attention and fast_sink_attention_supported(q.dtype, H, K, d, dv, values_in_keys) and page_size & (page_size - 1) == 0:
        kv_heads = K
        if values_in_keys:
            # one kv head that every query head reads: a CTA takes as many query heads as the kernels group, and `K` counts
            # those groups from here on
            K = H // sink_group(H, 1, True)
        lib = _sink_lib(d, dv, H // K, values_in_keys)
        max_pages = block_table.shape[1]
        nd = ctx.num_decode
        if nd > 0:
            if plan is None:
                plan = sink_decode_plan(q.dtype, nd, H, 1 if values_in_keys else K, d, dv, ctx.max_seq_len, window, chunk, values_in_keys)
            acc = ctx.workspace.get("sink_parts", (plan.chunks, nd, H, dv), torch.float32)
            ml = ctx.workspace.get("sink_part_sums", (plan.chunks, nd, H, 2), torch.float32)
            if launch_log is not None:
                _cost(nd * per_row + 2 * _size(acc), 0.0, key_bytes, 2.0 * H * (d + dv))
                _pending_cost["rows"], _pending_cost["window"] = "decode", window
            _check(lib.mb_attn_sink_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(acc), _ptr(ml), _ptr(block_table),
                                           _c_int(max_pages), _ptr(ctx.seq_lens), _c_int(nd), _c_int(K), _c_int(page_size), _c_float(scale),
                                           _c_int(window), _c_int(chunk), _c_int(plan.split), _c_int(plan.chunks), _stream()),
                   "attention (sink, decode)")
            _cost(_size(acc) + nd * H * dv * size * (2 if gate is not None else 1))
            _check(lib.mb_attn_sink_merge(_ptr(acc), _ptr(ml), _ptr(out), _ptr(ctx.seq_lens), _c_int(nd), _c_int(K), _c_int(window),
                                          _c_int(chunk), _c_int(int(sink)), _ptr(gate), _c_int(gate_stride), _c_int(plan.split), _ptr(sink_logits),
                                          _stream()), "attention (sink, parts merged)")
        if ctx.num_requests > nd and launch_log is not None:
            _cost((T - nd) * per_row, 0.0, key_bytes, 2.0 * H * (d + dv))
            _pending_cost["rows"], _pending_cost["window"] = "prefill", window
        if (ctx.num_requests > nd and use_tc_attention and tc_sink_attention_supported(d, dv, values_in_keys) and page_size >= 16
                and (gate is None or (gate.data_ptr() % 16 == 0 and gate_stride % 8 == 0))):
            # heads of 64 or 128 with values as wide: the tcgen05 kernel that plain causal attention uses takes the chunked
            # mask, the sink and the gate as parameters; over a shared latent one CTA per query head reads the one kv head's rows
            g = H // kv_heads
            tc = build.load(build.attention_tc_name(d, g, dv, values_in_keys), *build.attention_tc_job(d, g, dv, values_in_keys))
            _check(tc.mb_attn_prefill_tc(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                         _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                         _c_int(ctx.max_query_len), _c_int(T), _c_int(kv_heads), _c_int(page_size),
                                         ctypes.c_longlong(k_cache.shape[0]), _c_float(scale), _c_int(window),
                                         _ptr(_scratch_for(q.device).error), _c_int(chunk), _c_int(int(sink)), _ptr(gate),
                                         _c_int(gate_stride), _ptr(sink_logits), _stream()), "attention (sink, prefill, tensor cores)")
        elif ctx.num_requests > nd:
            _check(lib.mb_attn_sink_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                            _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                            _c_int(ctx.max_query_len), _c_int(K), _c_int(page_size), _c_float(scale), _c_int(window),
                                            _c_int(chunk), _c_int(int(sink)), _ptr(gate), _c_int(gate_stride), _ptr(sink_logits), _stream()),
                   "attention (sink, prefill)")
        return
    if launch_log is not None:
        _cost(T * per_row, 0.0, key_bytes, 2.0 * H * (d + dv))
        _pending_cost["rows"], _pending_cost["window"] = "all", window
    _check(_lib("mb_attention_sink").mb_attention_sink(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _code(q), _ptr(block_table), _c_int(block_table.shape[1]), _ptr(ctx.req_index),
        _ptr(ctx.positions), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(dv), _c_int(page_size), _c_float(scale), _c_int(window),
        _c_int(chunk), _c_int(int(sink)), _ptr(sink_logits), _c_int(v_stride), _ptr(gate), _c_int(gate_stride), _stream()), "attention (sink)")


#: bf16 sink attention goes to the tensor-core kernels where the head layout allows (False: always the plain kernel)
use_fast_sink_attention = True


#: query heads a CTA of the single-token kernel can take: the 16 rows of an mma tile
SINK_GROUP_MAX = 16


def sink_group(H: int, K: int, values_in_keys: bool = False) -> int:
    """Query heads a CTA of the tensor-core kernels takes together (the rows of one 16-row tile): those of one kv head; where
    every query head reads the same page rows (a shared latent: one kv head), the largest divisor of the head count up to 16."""
    if not values_in_keys:
        return H // K
    return max(g for g in range(1, SINK_GROUP_MAX + 1) if H % g == 0)


def tc_sink_attention_supported(d: int, dv: int, values_in_keys: bool = False) -> bool:
    """Head layouts the tcgen05 prompt kernel is compiled for: keys and values of 64 or of 128; or values that are the
    first 64 or 128 elements of key rows of 64 to 192 (a multiple of 16)."""
    if values_in_keys:
        return dv in (64, 128) and dv <= d <= 192 and d % 16 == 0
    return d == dv and d in (64, 128)


def fast_sink_attention_supported(dtype, H: int, K: int, d: int, dv: int, values_in_keys: bool = False) -> bool:
    """Head sizes in multiples of 16, values up to 128 wide, keys up to 128 (up to 256 where the values are the start of
    the key rows), at most 16 query heads per kv head (any number of heads over a shared latent)."""
    if values_in_keys and K != 1:
        return False
    return (dtype == torch.bfloat16 and d % 16 == 0 and dv % 16 == 0 and 16 <= d <= (256 if values_in_keys else 128) and 16 <= dv <= 128
            and H % K == 0 and 1 <= sink_group(H, K, values_in_keys) <= SINK_GROUP_MAX and (not values_in_keys or dv <= d))


def _sink_job(d: int, dv: int, group: int, values_in_keys: bool = False) -> tuple:
    return (["attention_sink_fast.cu"], [f"HEAD_DIM={d}", f"V_DIM={dv}", f"GROUP={group}"] + (["V_IN_K"] if values_in_keys else []))


def _sink_name(d: int, dv: int, group: int, values_in_keys: bool = False) -> str:
    return f"mb_attention_sink_fast_d{d}_v{dv}_g{group}" + ("_vk" if values_in_keys else "")


def _sink_lib(d: int, dv: int, group: int, values_in_keys: bool = False):
    return build.load(_sink_name(d, dv, group, values_in_keys), *_sink_job(d, dv, group, values_in_keys))


def sink_attention_jobs(dtype, H: int, K: int, d: int, dv: int, values_in_keys: bool = False) -> dict:
    """The kernels a sink-attention mixer of this head layout runs: the head preparation and the plain kernel, and the
    tensor-core kernels compiled for the layout where it allows."""
    jobs = library_jobs("mb_attention_sink")
    if use_fast_sink_attention and fast_sink_attention_supported(dtype, H, K, d, dv, values_in_keys):
        g = sink_group(H, K, values_in_keys)
        jobs[_sink_name(d, dv, g, values_in_keys)] = _sink_job(d, dv, g, values_in_keys)
        if use_tc_attention and tc_sink_attention_supported(d, dv, values_in_keys):
            jobs[build.attention_tc_name(d, H // K, dv, values_in_keys)] = build.attention_tc_job(d, H // K, dv, values_in_keys)
    return jobs


#: CTAs of the single-token kernel that an SM holds at a time (its launch bounds promise as many; a CTA walks its keys one
#: 64-key block at a time and waits for each: it is the number of CTAs in flight that hides the latency)
SINK_DECODE_CTAS_PER_SM = int(os.environ.get("MARIN_B200_SINK_CTAS", "4"))
SINK_DECODE_LEAST_SPLIT = 128


class SinkDecodePlan:
    """How single-token sink attention splits the keys a token sees over CTAs: ``split`` keys (a multiple of 64) per chunk,
    counted from the first seen key rounded down to a block of 64; ``chunks`` chunks cover the most keys any token sees."""
    __slots__ = ("split", "chunks")

    def __init__(self, split: int, chunks: int):
        self.split, self.chunks = int(split), int(chunks)


def sink_decode_plan(dtype, requests: int, H: int, K: int, d: int, dv: int, span: int, window: int, chunk: int,
                     values_in_keys: bool = False):
    """The number of chunks whose CTAs finish soonest: the CTAs of all requests, kv heads and chunks run in waves of as many as
    the device holds at a time, and a wave lasts as long as one CTA's walk over its chunk, so the cost of ``c`` chunks is
    ``waves(c) * (blocks per chunk + a CTA's start and end)``; among equals, the fewest chunks (the merge reads them all).  A
    chunk is a multiple of 64 keys, two blocks at least where there are that many (with one request the merge of 74
    one-block chunks took twice as long as the attention itself).  A token sees at most its window or its chunk of keys,
    whatever the sequence's length: the split follows that, not the context.  None where the plain kernel runs (it needs no
    plan).  (Filling "about four CTAs per SM" rounded up instead left a second wave of a few CTAs, which doubled the call:
    640 CTAs over 592 places took 70 us at batch 64 over a shared latent, where one CTA's walk takes 35.)"""
    if not (use_fast_sink_attention and fast_sink_attention_supported(dtype, H, K, d, dv, values_in_keys)):
        return None
    K = H // sink_group(H, K, values_in_keys)          # CTAs per request and chunk
    seen = max(int(span), 1)
    if window > 0:
        seen = min(seen, window)
    if chunk > 0:
        seen = min(seen, chunk)
    longest = seen + 63                                # the first chunk starts on a block border at or before the first seen key
    split = _sink_split(max(1, requests * K), longest, max(1, SINK_DECODE_CTAS_PER_SM * SM_COUNT))
    return SinkDecodePlan(split, max(1, -(-longest // split)))


@functools.lru_cache(maxsize=4096)
def _sink_split(per_chunk: int, longest: int, places: int) -> int:
    """Keys per chunk (see :func:`sink_decode_plan`): ``per_chunk`` CTAs a chunk, ``places`` CTAs on the device at a time."""
    blocks = -(-longest // 64)
    least = SINK_DECODE_LEAST_SPLIT // 64 if longest > SINK_DECODE_LEAST_SPLIT else 1
    best = None
    for c in range(1, min(1024, max(1, -(-blocks // least))) + 1):          # (the merge kernel takes up to 1,024 chunks)
        per = -(-blocks // c)
        waves = -(-c * per_chunk // places)
        cost = waves * (per + 1.5)                     # a CTA's start (its queries) and end (its part written) beside its blocks
        if best is None or cost < best[0] - 1e-9:
            best = (cost, per)
    return best[1] * 64


# ---- attention over a latent that keys and values share (csrc/attention_latent.cu) -------------------------------------------
def latent_finish(rows: torch.Tensor, q_out: torch.Tensor, c_weight, eps: float, positions, inv_freq, rot_dims: int, interleaved: bool,
                  slot_mapping, k_cache, H: int, dn: int, dr: int, r: int, write_kv: bool = True,
                  kv_rows: Optional[torch.Tensor] = None) -> None:
    """Finishes a fused projection whose rows hold ``H`` query heads of ``dn`` unrotated and ``dr`` rotated numbers and, for a
    layer that owns its cache, ``r`` latent numbers and ``dr`` key numbers.  The queries' rotated parts go, rotated, to
    ``q_out[:, head, r:]`` (``[T, H, r + dr]``; the first ``r`` of every head are left for ``heads_product``); the latent is
    divided by its root mean square (times ``c_weight``) and written with the rotated key part into the page row ``[r + dr]``."""
    _need_cuda(rows, q_out, c_weight, positions, inv_freq, slot_mapping, k_cache)
    T = rows.shape[0]
    D = r + dr
    assert tuple(q_out.shape) == (T, H * D) and q_out.dtype == rows.dtype
    assert rows.shape[1] >= H * (dn + dr) + (D if write_kv and kv_rows is None else 0)
    # ``kv_rows``: the latent and the key part come from rows of their own (a column slice ``[T, r + dr]`` of a wider matrix)
    assert kv_rows is None or (kv_rows.is_cuda and kv_rows.dtype == rows.dtype and tuple(kv_rows.shape) == (T, D) and kv_rows.stride(1) == 1)
    assert not write_kv or (k_cache.dtype == rows.dtype and k_cache.shape[1] == 1 and k_cache.shape[3] == D and c_weight is not None)
    _cost((rows.shape[1] - H * dn) * T * rows.element_size() + T * (H * dr + D) * rows.element_size(), 6.0 * T * (H * dr + D))
    _check(_lib("mb_attention_latent").mb_latent_finish(
        _ptr(rows), _c_int(rows.shape[1]), _code(rows), _ptr(q_out), _ptr(c_weight), _c_float(eps), _ptr(positions), _ptr(inv_freq),
        _c_int(rot_dims if inv_freq is not None else 0), _c_int(int(interleaved)), _ptr(slot_mapping), _ptr(k_cache), _c_int(T), _c_int(H),
        _c_int(dn), _c_int(dr), _c_int(r), _c_int(k_cache.shape[2] if write_kv else 0), _c_int(int(write_kv)),
        _c_void_p(kv_rows.data_ptr()) if kv_rows is not None else None, _c_int(kv_rows.stride(0) if kv_rows is not None else 0), _stream()),
        "latent heads")


#: bf16 products per head go to the tensor-core kernel where the layout allows (False: always the plain kernel)
use_fast_heads_product = True


def heads_product(x: torch.Tensor, x_head: int, K: int, w: torch.Tensor, out: torch.Tensor, o_head: int) -> None:
    """A product per head over strided rows: ``out[t, a o_head + n] = sum_k w[a, n, k] x[t, a x_head + k]`` for every head ``a``
    of ``w`` ``[H, N, K]``.  ``x`` and ``out`` are ``[T, row]`` tensors of which every head reads / writes a slice."""
    _need_cuda(x, w, out)
    T = x.shape[0]
    H, N = w.shape[0], w.shape[1]
    assert w.shape[2] == K and w.dtype == x.dtype == out.dtype and out.shape[0] == T
    assert (H - 1) * x_head + K <= x.shape[1] and (H - 1) * o_head + N <= out.shape[1]
    size = x.element_size()
    _cost(_size(w) + T * H * (K + N) * size, 2.0 * T * H * N * K)
    _check(_lib("mb_attention_latent").mb_heads_product(
        _ptr(x), _c_int(x.shape[1]), _c_int(x_head), _ptr(w), _ptr(out), _c_int(out.shape[1]), _c_int(o_head), _code(x), _c_int(T), _c_int(H),
        _c_int(N), _c_int(K), _c_int(int(use_fast_heads_product)), _stream()), "product per head")


# ---- routed feed-forward ------------------------------------------------------------------------------------------------------
SCORE_MODES = {"sigmoid": 0, "softmax": 1}


def moe_route(x: torch.Tensor, router: torch.Tensor, experts_out: torch.Tensor, weights_out: torch.Tensor, score: str = "sigmoid",
              renormalize: bool = False, bias: Optional[torch.Tensor] = None) -> None:
    """Router logits ``x router^T (+ bias)`` in float32, scores by ``score``, the ``top`` best experts per token (``top`` = the outputs'
    second size) in order of decreasing score, the lower expert among equals; their scores are the weights."""
    _need_cuda(x, router, experts_out, weights_out)
    T, h = x.shape
    E, top = router.shape[0], experts_out.shape[1]
    assert router.dtype == torch.float32 and router.shape[1] == h and experts_out.dtype == torch.int32 and weights_out.dtype == torch.float32
    assert tuple(experts_out.shape) == (T, top) and tuple(weights_out.shape) == (T, top)
    assert bias is None or (bias.is_cuda and bias.dtype == torch.float32 and bias.numel() == E)
    _cost(_size(x) + _size(router) + _size(experts_out) * 2, 2.0 * T * E * h)
    _check(_lib("mb_moe").mb_moe_route(_ptr(x), _code(x), _ptr(router), _ptr(bias), _ptr(experts_out), _ptr(weights_out), _c_int(T), _c_int(h), _c_int(E),
                                      _c_int(top), _c_int(SCORE_MODES[score]), _c_int(int(renormalize)), _stream()), "router")


def moe_table_route(token_ids: torch.Tensor, table: torch.Tensor, E: int, experts_out: torch.Tensor, weights_out: torch.Tensor) -> None:
    """Experts named by a table over the token ids: ``experts_out[t] = table[token_ids[t]]`` (``[vocab, top]`` int32), every
    weight ``1 / top``."""
    _need_cuda(token_ids, table, experts_out, weights_out)
    T, top = experts_out.shape
    assert table.dtype == torch.int32 and table.shape[1] == top and token_ids.dtype == torch.int32 and token_ids.numel() == T
    assert experts_out.dtype == torch.int32 and weights_out.dtype == torch.float32 and tuple(weights_out.shape) == (T, top)
    _cost(_size(token_ids) + 3 * _size(experts_out))
    _check(_lib("mb_moe").mb_moe_table_route(_ptr(token_ids), _ptr(table), _ptr(experts_out), _ptr(weights_out), _c_int(T), _c_int(top),
                                            _c_int(table.shape[0]), _c_int(E), _stream()), "experts from the table")


def moe_group(experts: torch.Tensor, E: int, offsets: torch.Tensor, order: torch.Tensor) -> None:
    """The (token, choice) pairs grouped by expert: ``order[offsets[e] : offsets[e + 1]]`` are expert ``e``'s pairs."""
    _need_cuda(experts, offsets, order)
    pairs = experts.numel()
    assert offsets.dtype == torch.int32 and offsets.numel() >= E + 1 and order.dtype == torch.int32 and order.numel() >= pairs
    _cost(_size(experts) * 3)
    _check(_lib("mb_moe").mb_moe_group(_ptr(experts), _c_int(pairs), _c_int(E), _ptr(offsets), _ptr(order), _stream()), "pairs grouped")


EXPERT_ACTIVATIONS = {"swiglu": 0, "relu2": 1, "glu_capped": 0}
#: the gated form ``g sigmoid(alpha g) (u + shift)`` with both inputs capped at ``limit`` (0: not capped), as (limit, alpha, shift);
#: "swiglu" is this
SILU_FORM = (0.0, 1.0, 0.0)


def _glu_form(activation: str, form) -> tuple:
    if activation == "glu_capped":
        if form is None:
            raise KernelError("glu_capped: the form (limit, alpha, shift) is needed")
        return tuple(float(v) for v in form)
    return SILU_FORM


def moe_experts_plain(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, experts: torch.Tensor, weights: torch.Tensor,
                      act: torch.Tensor, y: torch.Tensor, weight_on_input: bool, interleaved: bool = False, activation: str = "swiglu",
                      form=None) -> None:
    """``y[t] += sum_c down_e( silu(gate_e x) * (up_e x) )`` over token ``t``'s chosen experts ``e`` in choice order, ``x = w h[t]``
    where the weight goes on the input, else the result times ``w``.  Any sizes, both dtypes.  ``interleaved``: an expert's
    gate and up rows alternate in blocks of 16 (``interleave_gate_up``) instead of gate rows first.  ``activation`` "relu2":
    experts without a gate, ``down_e( relu(up_e x)^2 )``, ``w_gate_up`` then holds the up matrices ``[E, ff, h]`` alone."""
    _need_cuda(x, w_gate_up, w_down, experts, weights, act, y)
    T, h = x.shape
    top = experts.shape[1]
    ff = w_down.shape[2]
    gated = activation != "relu2"
    limit, alpha, shift = _glu_form(activation, form)
    assert tuple(w_gate_up.shape[1:]) == ((2 if gated else 1) * ff, h) and tuple(w_down.shape[1:]) == (h, ff) and w_gate_up.dtype == x.dtype == w_down.dtype
    assert act.dtype == x.dtype and act.numel() >= T * top * ff and y.dtype == torch.float32 and tuple(y.shape) == (T, h)
    pairs = T * top
    touched = min(pairs, w_down.shape[0])
    for which, what in ((0, "experts, gate|up"), (1, "experts, down")):
        if which == 0:
            _cost(touched * (2 if gated else 1) * ff * h * x.element_size() + _size(x) + pairs * ff * x.element_size(), (4.0 if gated else 2.0) * pairs * ff * h)
        else:
            _cost(touched * ff * h * x.element_size() + pairs * ff * x.element_size() + 2 * _size(y), 2.0 * pairs * ff * h)
        _check(_lib("mb_moe").mb_moe_experts_plain(_ptr(x), _code(x), _ptr(w_gate_up), _ptr(w_down), _ptr(experts), _ptr(weights), _ptr(act),
                                                  _ptr(y), _c_int(T), _c_int(h), _c_int(ff), _c_int(top), _c_int(int(weight_on_input)),
                                                  _c_int(int(interleaved)), _c_int(which), _c_int(EXPERT_ACTIVATIONS[activation]), _c_float(limit),
                                                  _c_float(alpha), _c_float(shift), _stream()), what)


#: bf16 experts go to the grouped tensor-core kernels where the sizes allow (False: always the plain kernels)
use_fast_experts = True


def fast_experts_supported(h: int, ff: int) -> bool:
    """Both inner sizes of the experts' products in whole steps of 64 (the grouped kernel's k-step)."""
    return h % 64 == 0 and ff % 64 == 0


def moe_jobs(dtype, h: int, ff: int) -> dict:
    return library_jobs("mb_moe")


#: from this many (token, choice) pairs per expert on, a step that is not being captured in a graph reads the experts'
#: counts back to the host and gives every expert's rows to the dense tcgen05 products (``gemm_swiglu``, ``gemm``) instead
#: of the grouped mma.sync kernel
EXPERTS_DENSE_FROM = 96
#: streams the experts' dense products are dealt over: one expert's products fill the device only partly (a quarter of the
#: step's rows, tiles that do not make whole rounds over the SMs), several at a time fill the gaps.  1: one after the other.
EXPERT_STREAMS = 4
_side_streams = {}


def _expert_streams(device, n: int):
    key = (device.index, n)
    if key not in _side_streams:
        _side_streams[key] = [torch.cuda.Stream(device=device) for _ in range(n)]
    return _side_streams[key]


def moe_experts(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, experts: torch.Tensor, weights: torch.Tensor,
                y: torch.Tensor, weight_on_input: bool, workspace, interleaved: bool = False, activation: str = "swiglu", form=None) -> None:
    """The chosen experts' outputs added into ``y`` (float32 ``[T, h]``); see ``moe_experts_plain``.  bf16 with sizes in steps
    of 64: the pairs are sorted by expert on the device and their inputs gathered in that order; then either two grouped
    products over all experts (few pairs: single-token steps, captured or not: nothing is read back), or, with many pairs
    per expert, the dense tensor-core products expert by expert over the sorted rows (the counts are read back once)."""
    T, top = experts.shape
    E, h, ff = w_down.shape
    pairs = T * top
    act = workspace.get("moe_act", (pairs, ff), x.dtype)
    if not (use_fast_experts and x.dtype == torch.bfloat16 and fast_experts_supported(h, ff)):
        moe_experts_plain(x, w_gate_up, w_down, experts, weights, act, y, weight_on_input, interleaved, activation, form)
        return
    _need_cuda(x, w_gate_up, w_down, experts, weights, y)
    gated = activation != "relu2"
    limit, alpha, shift = _glu_form(activation, form)
    assert tuple(w_gate_up.shape) == (E, (2 if gated else 1) * ff, h) and w_gate_up.dtype == w_down.dtype == x.dtype and tuple(y.shape) == (T, h)
    assert y.dtype == torch.float32 and experts.dtype == torch.int32 and weights.dtype == torch.float32
    ints = workspace.get("moe_ints", (E + 1 + 3 * pairs,), torch.int32)
    offsets, order, inv, token_sorted = ints[:E + 1], ints[E + 1:E + 1 + pairs], ints[E + 1 + pairs:E + 1 + 2 * pairs], ints[E + 1 + 2 * pairs:]
    weight_sorted = workspace.get("moe_weight_sorted", (pairs,), torch.float32)
    xs = workspace.get("moe_xs", (pairs, h), x.dtype)
    size = x.element_size()
    lib = _lib("mb_moe")
    touched = min(pairs, E)
    moe_group(experts, E, offsets, order)
    _cost(2 * pairs * h * size)
    _check(lib.mb_moe_gather(_ptr(x), _ptr(order), _ptr(weights), _ptr(xs), _ptr(token_sorted), _ptr(weight_sorted), _ptr(inv), _c_int(pairs),
                             _c_int(h), _c_int(top), _c_int(int(weight_on_input)), _stream()), "experts' inputs gathered")
    dense = ((interleaved or not gated or activation == "glu_capped") and pairs >= EXPERTS_DENSE_FROM * E and use_tensor_cores and not torch.cuda.is_current_stream_capturing())
    if dense:
        rows = workspace.get("moe_rows", (pairs, h), torch.float32)
        bounds = offsets.tolist()                       # the one wait on the host: how many pairs each expert got
        active = [e for e in range(E) if bounds[e + 1] > bounds[e]]
        # (while the stages of a step are being recorded everything stays on one stream, in launch order)
        lanes = min(EXPERT_STREAMS, len(active)) if launch_log is None else 1
        gate_up = workspace.get("moe_gate_up", (pairs, 2 * ff), x.dtype) if activation == "glu_capped" else None

        def first_product(lo, hi, e):
            if activation == "glu_capped":        # the dense product, then the capped form over its rows (gate rows first)
                gemm(xs[lo:hi], w_gate_up[e], gate_up[lo:hi])
                glu_capped(gate_up[lo:hi], ff, act[lo:hi], limit, alpha, shift)
            elif gated:
                gemm_swiglu(xs[lo:hi], w_gate_up[e], act[lo:hi], workspace)
            else:
                gemm_act(xs[lo:hi], w_gate_up[e], act[lo:hi], "relu2")

        if lanes <= 1:
            for e in active:
                lo, hi = bounds[e], bounds[e + 1]
                first_product(lo, hi, e)
                gemm(act[lo:hi], w_down[e], rows[lo:hi])
        else:
            global stream_k
            current = torch.cuda.current_stream(x.device)
            side = _expert_streams(x.device, lanes)
            ready = torch.cuda.Event()
            ready.record(current)
            keep, stream_k = stream_k, False            # stream-K parks tiles in scratch memory that one stream of work owns
            try:
                for i, e in enumerate(active):
                    lo, hi = bounds[e], bounds[e + 1]
                    if i < lanes:
                        side[i].wait_event(ready)
                    with torch.cuda.stream(side[i % lanes]):
                        first_product(lo, hi, e)
                        gemm(act[lo:hi], w_down[e], rows[lo:hi])
            finally:
                stream_k = keep
            for st in side:
                done = torch.cuda.Event()
                done.record(st)
                current.wait_event(done)
        _cost(_size(rows) + 2 * _size(y))
        _check(lib.mb_moe_combine(_ptr(rows), _ptr(inv), _ptr(None if weight_on_input else weights), _ptr(y), _c_int(T), _c_int(h),
                                  _c_int(top), _stream()), "experts' outputs added")
        return
    _cost(touched * (2 if gated else 1) * ff * h * size + pairs * (h + ff) * size, (4.0 if gated else 2.0) * pairs * ff * h)
    _check(lib.mb_moe_grouped_gate_up(_ptr(xs), _ptr(w_gate_up), _ptr(offsets), _ptr(act), _c_int(pairs), _c_int(h), _c_int(ff), _c_int(E),
                                      _c_int(int(interleaved)), _c_int(EXPERT_ACTIVATIONS[activation]), _c_float(limit), _c_float(alpha),
                                      _c_float(shift), _stream()),
           "experts, gate|up, SwiGLU (grouped, tensor cores)" if gated else "experts, up, relu squared (grouped, tensor cores)")
    scale = None if weight_on_input else weight_sorted
    _cost(touched * ff * h * size + pairs * ff * size + 2 * pairs * h * 4, 2.0 * pairs * ff * h)
    if top == 1:           # every pair has a row of y to itself: the product adds into it
        _check(lib.mb_moe_grouped_down(_ptr(act), _ptr(w_down), _ptr(offsets), _ptr(y), _ptr(token_sorted), _ptr(scale), _c_int(1),
                                       _c_int(pairs), _c_int(h), _c_int(ff), _c_int(E), _stream()), "experts, down (grouped, tensor cores)")
        return
    rows = workspace.get("moe_rows", (pairs, h), torch.float32)
    _check(lib.mb_moe_grouped_down(_ptr(act), _ptr(w_down), _ptr(offsets), _ptr(rows), _ptr(None), _ptr(scale), _c_int(0),
                                   _c_int(pairs), _c_int(h), _c_int(ff), _c_int(E), _stream()), "experts, down (grouped, tensor cores)")
    _cost(_size(rows) + 2 * _size(y))
    _check(lib.mb_moe_combine(_ptr(rows), _ptr(inv), _ptr(None), _ptr(y), _c_int(T), _c_int(h), _c_int(top), _stream()), "experts' outputs added")


# ---- attention over a window and pooled blocks before it (csrc/attention_pooled.cu) ------------------------------------------------
def pool_blocks(k_cache, v_cache, k_pool, v_pool, ctx, block_table, slot_mapping, pool: int) -> None:
    """For every token of the step that ends a block of ``pool`` positions: the means of the block's keys and of its values, as
    the pages hold them, into the pooled rows of the page that holds the token (row ``offset // pool``)."""
    _need_cuda(k_cache, v_cache, k_pool, v_pool, block_table, slot_mapping)
    T = ctx.num_tokens
    K, page_size, d, dv = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    rows = -(-page_size // pool)
    assert tuple(k_pool.shape[1:]) == (K, rows, d) and tuple(v_pool.shape[1:]) == (K, rows, dv) and k_pool.dtype == k_cache.dtype == v_pool.dtype
    _cost(T * K * (d + dv) * k_cache.element_size() * (1 + 1.0 / pool))
    _check(_lib("mb_attention_pooled").mb_pool_blocks(
        _ptr(k_cache), _ptr(v_cache), _ptr(k_pool), _ptr(v_pool), _code(k_cache), _ptr(block_table), _c_int(block_table.shape[1]),
        _ptr(ctx.req_index), _ptr(ctx.positions), _ptr(slot_mapping), _c_int(T), _c_int(K), _c_int(d), _c_int(dv), _c_int(page_size),
        _c_int(pool), _c_int(rows), _stream()), "pooled blocks")


def attention_pooled(q, k_cache, v_cache, k_pool, v_pool, out, ctx, block_table, H: int, K: int, d: int, dv: int, scale: float,
                     softcap: float = 0.0, window: int = 0, pool: int = 0, talk: Optional[torch.Tensor] = None) -> None:
    """Softmax attention of the step's tokens over the last ``window`` positions (0: all) and, with ``pool``, one pooled key and
    value per block of ``pool`` positions that lies wholly before the window; scores capped by ``softcap tanh(s / softcap)``
    where ``softcap`` > 0; ``talk`` (float32 ``[H, H]``): head ``h``'s weights are ``sum_g talk[h, g] w_g``, applied to the values
    of its own kv head."""
    _need_cuda(q, k_cache, v_cache, k_pool, v_pool, out, block_table, talk)
    T = q.shape[0]
    page_size = k_cache.shape[2]
    assert tuple(q.shape) == (T, H * d) and tuple(out.shape) == (T, H * dv) and k_cache.dtype == q.dtype == v_cache.dtype == out.dtype
    assert k_cache.shape[3] == d and v_cache.shape[3] == dv and (not pool or (k_pool is not None and k_pool.dtype == q.dtype))
    assert talk is None or (talk.dtype == torch.float32 and tuple(talk.shape) == (H, H))
    if T == 0:
        return
    size = q.element_size()
    parts = ctx.workspace.get("pooled_parts", (T, H, K, dv), torch.float32) if talk is not None else None
    rows = -(-page_size // pool) if pool else 0
    pair_flops = 2.0 * H * (d + (K if talk is not None else 1) * dv)
    plain_tokens = T
    if use_fast_pooled_attention and fast_pooled_attention_supported(q.dtype, H, K, d, dv) and page_size & (page_size - 1) == 0:
        # the tensor-core kernel takes every request of the step: a prompt portion in tiles of 64 queries, a single token as a
        # tile of one (the plain kernel walks a token's keys in one block of threads, far too slowly for a window of a thousand)
        plain_tokens = 0
        if launch_log is not None:
            _cost(T * H * (d + dv) * size, 0.0, K * (d + dv) * size, pair_flops)
            _pending_cost["rows"], _pending_cost["window"] = "all", window
        lib = _pooled_lib(d, dv, H // K, pooled_value_heads(K, dv))
        _check(lib.mb_attn_pooled_prefill(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(k_pool), _ptr(v_pool), _ptr(parts), _ptr(out), _ptr(block_table),
            _c_int(block_table.shape[1]), _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(0), _c_int(ctx.num_requests),
            _c_int(ctx.max_query_len), _c_int(K), _c_int(page_size), _c_float(scale), _c_float(softcap or 0.0), _c_int(window), _c_int(pool),
            _c_int(rows), _c_int(int(talk is not None)), _c_int(int(ctx.max_query_len == 1 and ctx.num_decode == ctx.num_requests)), _c_int(POOLED_BY_WARP_FROM), _stream()),
            "attention (window and pooled blocks, tensor cores)")
    if plain_tokens > 0:
        if launch_log is not None:
            _cost(plain_tokens * H * (d + dv) * size, 0.0, K * (d + dv) * size, pair_flops)
            _pending_cost["rows"], _pending_cost["window"] = ("all" if plain_tokens == T else "decode"), window
        _check(_lib("mb_attention_pooled").mb_attention_pooled(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(k_pool), _ptr(v_pool), _ptr(parts), _ptr(out), _code(q), _ptr(block_table),
            _c_int(block_table.shape[1]), _ptr(ctx.req_index), _ptr(ctx.positions), _ptr(ctx.seq_lens), _c_int(plain_tokens), _c_int(H), _c_int(K),
            _c_int(d), _c_int(dv), _c_int(page_size), _c_float(scale), _c_float(softcap or 0.0), _c_int(window), _c_int(pool), _c_int(rows),
            _c_int(int(talk is not None)), _stream()), "attention (window and pooled blocks)")
    if talk is not None:
        _cost(_size(parts) + _size(out), 2.0 * T * H * H * dv)
        _check(_lib("mb_attention_pooled").mb_talk_mix(_ptr(parts), _ptr(talk), _ptr(out), _code(out), _c_int(T), _c_int(H), _c_int(K), _c_int(dv),
                                                      _stream()), "heads' weights mixed")


#: bf16 attention over a window and pooled blocks goes to the tensor-core kernel where the head layout allows
use_fast_pooled_attention = True
#: single-token steps with mixed weights: from this many (request, kv head) CTAs on, a CTA takes every pair of value heads, a warp
#: each, over one copy of the keys (fewer, larger CTAs: it pays once they still fill the device twice)
POOLED_BY_WARP_FROM = 2 * SM_COUNT


def fast_pooled_attention_supported(dtype, H: int, K: int, d: int, dv: int) -> bool:
    """Head sizes in multiples of 16 up to 128."""
    return dtype == torch.bfloat16 and d % 16 == 0 and dv % 16 == 0 and 16 <= d <= 128 and 16 <= dv <= 128 and H % K == 0


def pooled_value_heads(K: int, dv: int) -> int:
    """Kv heads whose values a CTA of the tensor-core kernel sums at a time: as many as its registers hold (256 columns),
    a divisor of ``K``."""
    most = max(1, 256 // dv)
    return max(v for v in range(1, min(K, most) + 1) if K % v == 0)


def _pooled_job(d: int, dv: int, group: int, value_heads: int) -> tuple:
    return (["attention_pooled_fast.cu"], [f"HEAD_DIM={d}", f"V_DIM={dv}", f"GROUP={group}", f"VALUE_HEADS={value_heads}"])


def _pooled_name(d: int, dv: int, group: int, value_heads: int) -> str:
    return f"mb_attention_pooled_fast_d{d}_v{dv}_g{group}_c{value_heads}"


def _pooled_lib(d: int, dv: int, group: int, value_heads: int):
    return build.load(_pooled_name(d, dv, group, value_heads), *_pooled_job(d, dv, group, value_heads))


def pooled_attention_jobs(dtype, H: int, K: int, d: int, dv: int) -> dict:
    """The kernels a mixer with this head layout runs: head preparation, the plain kernels, and the tensor-core kernel compiled
    for the layout where it allows."""
    jobs = library_jobs("mb_attention_sink", "mb_attention_pooled")
    if use_fast_pooled_attention and fast_pooled_attention_supported(dtype, H, K, d, dv):
        vh = pooled_value_heads(K, dv)
        jobs[_pooled_name(d, dv, H // K, vh)] = _pooled_job(d, dv, H // K, vh)
    return jobs


# ---- a selective state space layer (csrc/ssm.cu) ---------------------------------------------------------------------------------
def ssm_conv(rows: torch.Tensor, col: int, weight: torch.Tensor, bias: Optional[torch.Tensor], carry: torch.Tensor, ctx, slots: torch.Tensor,
             out: torch.Tensor) -> None:
    """``out = silu(conv(rows[:, col : col + channels]) + bias)``: a causal convolution per channel over each request's tokens,
    ``weight`` float32 ``[channels, taps]`` whose last column meets the current token.  ``carry`` (float32 ``[slots, taps - 1,
    channels]``, oldest first) holds a request's last inputs from earlier steps and is brought up to date."""
    _need_cuda(rows, weight, bias, carry, slots, out)
    T, (channels, taps) = rows.shape[0], weight.shape
    assert tuple(out.shape) == (T, channels) and out.dtype == rows.dtype and weight.dtype == torch.float32 and col + channels <= rows.shape[1]
    assert carry.dtype == torch.float32 and carry.is_contiguous() and tuple(carry.shape[1:]) == (taps - 1, channels) and rows.stride(1) == 1
    _cost(2 * T * channels * rows.element_size() + _size(weight), 2.0 * T * channels * taps)
    _check(_lib("mb_ssm").mb_ssm_conv(_ptr(rows), _c_int(rows.stride(0)), _c_int(col), _code(rows), _ptr(weight), _ptr(bias), _ptr(carry),
                                     _ptr(ctx.req_index), _ptr(ctx.cu_tokens), _ptr(slots), _ptr(out), _c_int(T), _c_int(channels), _c_int(taps),
                                     _stream()), "short convolution")
    if taps > 1:
        _cost(2 * ctx.num_requests * (taps - 1) * channels * 4)
        _check(_lib("mb_ssm").mb_ssm_conv_carry(_ptr(rows), _c_int(rows.stride(0)), _c_int(col), _code(rows), _ptr(carry), _ptr(ctx.cu_tokens),
                                               _ptr(slots), _c_int(ctx.num_requests), _c_int(channels), _c_int(taps), _stream()),
               "convolution's inputs kept")


def ssm_scan(xbc: torch.Tensor, rows: torch.Tensor, dt_col: int, dt_bias: torch.Tensor, rate_log: torch.Tensor, skip: torch.Tensor,
             state: torch.Tensor, ctx, slots: torch.Tensor, y: torch.Tensor, heads: int, P: int, N: int, groups: int) -> None:
    """Per head ``S <- exp(-exp(rate) dt) S + dt B x^T; y = S^T C + skip x`` over each request's tokens, ``dt = softplus(dt' +
    dt_bias)`` with ``dt'`` of head ``h`` at ``rows[:, dt_col + h]``; ``xbc`` ``[T, heads P + 2 groups N]`` holds x | B | C;
    ``state`` float32 ``[slots, heads, N, P]`` is read and written; ``y`` float32 ``[T, heads P]``."""
    _need_cuda(xbc, rows, dt_bias, rate_log, skip, state, slots, y)
    T = xbc.shape[0]
    assert xbc.shape[1] == heads * P + 2 * groups * N and xbc.is_contiguous() and rows.dtype == xbc.dtype and rows.stride(1) == 1
    assert state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, N, P)
    assert y.dtype == torch.float32 and tuple(y.shape) == (T, heads * P) and dt_bias.dtype == rate_log.dtype == skip.dtype == torch.float32
    R = ctx.num_requests
    lib = _lib("mb_ssm")

    def run(mode, segments, seg_len, seg_state, seg_decay, what):
        _check(lib.mb_ssm_scan(_ptr(xbc), _ptr(rows), _c_int(rows.stride(0)), _c_int(dt_col), _code(xbc), _ptr(dt_bias), _ptr(rate_log), _ptr(skip),
                               _ptr(state), _ptr(ctx.cu_tokens), _ptr(slots), _ptr(y), _c_int(R), _c_int(heads), _c_int(P), _c_int(N), _c_int(groups),
                               _c_int(mode), _c_int(segments), _c_int(seg_len), _ptr(seg_state), _ptr(seg_decay), _stream()), what)

    longest = ctx.max_query_len
    if xbc.dtype == torch.bfloat16 and longest >= SSM_SEGMENTS_FROM and not torch.cuda.is_current_stream_capturing():
        # long portions in segments walked side by side: end states and decay products from zero, the start states from those,
        # then the outputs (float32 mode keeps the one walk: its sums must not depend on how a prompt was cut)
        segments = -(-longest // SSM_SEGMENT_TOKENS)
        seg_state = ctx.workspace.get("ssm_segment_states", (R, segments, heads, N, P), torch.float32)
        seg_decay = ctx.workspace.get("ssm_segment_decays", (R, segments, heads), torch.float32)
        _cost(_size(xbc) + 2 * _size(seg_state), 4.0 * T * heads * N * P)
        run(1, segments, SSM_SEGMENT_TOKENS, seg_state, seg_decay, "state space recurrence (segments' end states)")
        _cost(2 * _size(seg_state) + 2 * R * heads * N * P * 4, 2.0 * _size(seg_state) / 4)
        run(3, segments, SSM_SEGMENT_TOKENS, seg_state, seg_decay, "state space recurrence (segments' start states)")
        _cost(_size(xbc) + _size(y) + _size(seg_state), 6.0 * T * heads * N * P)
        run(2, segments, SSM_SEGMENT_TOKENS, seg_state, seg_decay, "state space recurrence (segments' outputs)")
        return
    _cost(_size(xbc) + _size(y) + 2 * R * heads * N * P * 4, 6.0 * T * heads * N * P)
    run(0, 1, 0, None, None, "state space recurrence")


#: portions from this many tokens on are walked in segments side by side (bf16 mode), of so many tokens each
SSM_SEGMENTS_FROM = 256
SSM_SEGMENT_TOKENS = 128


def ssm_gate_norm(y: torch.Tensor, rows: torch.Tensor, z_col: int, weight: torch.Tensor, eps: float, parts: int, out: torch.Tensor) -> None:
    """``out = v / rms(v) * weight`` with ``v = y silu(rows[:, z_col : z_col + n])``, the root mean square taken over each of
    ``parts`` equal parts of the row by itself."""
    _need_cuda(y, rows, weight, out)
    T, n = y.shape
    assert y.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == n and tuple(out.shape) == (T, n) and out.dtype == rows.dtype
    assert rows.stride(1) == 1 and z_col + n <= rows.shape[1] and n % parts == 0
    _cost(_size(y) + 2 * _size(out), 12.0 * T * n)
    _check(_lib("mb_ssm").mb_ssm_gate_norm(_ptr(y), _ptr(rows), _c_int(rows.stride(0)), _c_int(z_col), _code(rows), _ptr(weight), _c_float(eps),
                                          _ptr(out), _c_int(T), _c_int(n), _c_int(parts), _stream()), "gate, norm in parts")


# ---- small element-wise steps (csrc/activations.cu) --------------------------------------------------------------------------------
BIAS_ACTS = {None: 0, "gelu": 1, "gelu_tanh": 2}


def bias_act(x: torch.Tensor, bias: Optional[torch.Tensor], activation: Optional[str]) -> None:
    """``x <- act(x + bias)`` in place; ``activation`` None, "gelu" (erf) or "gelu_tanh"."""
    _need_cuda(x, bias)
    rows, n = x.shape
    assert x.is_contiguous() and (bias is None or (bias.dtype == torch.float32 and bias.numel() == n))
    _cost(2 * _size(x), 10.0 * x.numel())
    _check(_lib("mb_activations").mb_bias_act(_ptr(x), _code(x), _ptr(bias), _c_int(rows), _c_int(n), _c_int(BIAS_ACTS[activation]), _stream()),
           "bias, activation")


def glu_capped(rows: torch.Tensor, ff: int, out: torch.Tensor, limit: float, alpha: float, shift: float, scale_col: int = -1) -> None:
    """``out = g sigmoid(alpha g) (u + shift)`` with ``g = min(rows[:, :ff], limit)``, ``u = clamp(rows[:, ff : 2 ff], -limit, limit)``
    (``limit`` 0: as they are); ``scale_col`` >= 0: each row times ``sigmoid(rows[:, scale_col])``."""
    _need_cuda(rows, out)
    T = rows.shape[0]
    assert rows.stride(1) == 1 and rows.shape[1] >= 2 * ff and tuple(out.shape) == (T, ff) and out.dtype == rows.dtype and out.is_contiguous()
    _cost(T * 3 * ff * rows.element_size(), 12.0 * T * ff)
    _check(_lib("mb_activations").mb_glu_capped(_ptr(rows), _c_int(rows.stride(0)), _code(rows), _ptr(out), _c_int(T), _c_int(ff), _c_float(limit),
                                               _c_float(alpha), _c_float(shift), _c_int(scale_col), _stream()), "capped gate")


def head_gate(x: torch.Tensor, rows: torch.Tensor, col: int, heads: int) -> None:
    """``x[t, a, :] *= sigmoid(rows[t, col + a])`` in place, ``x`` ``[T, heads dim]``."""
    _need_cuda(x, rows)
    T = x.shape[0]
    assert x.is_contiguous() and x.shape[1] % heads == 0 and rows.dtype == x.dtype and rows.stride(1) == 1 and col + heads <= rows.shape[1]
    _cost(2 * _size(x), 2.0 * x.numel())
    _check(_lib("mb_activations").mb_head_gate(_ptr(x), _code(x), _ptr(rows), _c_int(rows.stride(0)), _c_int(col), _c_int(T), _c_int(heads),
                                              _c_int(x.shape[1] // heads), _stream()), "gate per head")


def keep_last_row(h: torch.Tensor, carry: torch.Tensor, ctx, slots: torch.Tensor) -> None:
    """``carry[slot of request] = h[the request's last token of the step]`` (float32; ``carry`` may be a column slice of a state)."""
    _need_cuda(h, slots)
    T, n = h.shape
    assert carry.is_cuda and carry.dtype == torch.float32 and carry.shape[1] == n and carry.stride(1) == 1 and h.is_contiguous()
    _cost(ctx.num_requests * n * (4 + h.element_size()))
    _check(_lib("mb_activations").mb_keep_last_row(_ptr(h), _code(h), _c_void_p(carry.data_ptr()), ctypes.c_longlong(carry.stride(0)),
                                                  _ptr(ctx.cu_tokens), _ptr(slots), _c_int(ctx.num_requests), _c_int(n), _stream()), "last row kept")


def add_row_bias(y: torch.Tensor, bias: torch.Tensor) -> None:
    """``y[t] += bias`` over the float32 residual."""
    _need_cuda(y, bias)
    rows, n = y.shape
    assert y.dtype == torch.float32 and y.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == n
    _cost(2 * _size(y))
    _check(_lib("mb_activations").mb_add_row_bias(_ptr(y), _ptr(bias), _c_int(rows), _c_int(n), _stream()), "bias")


def rmsnorm_cols(rows: torch.Tensor, col: int, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """``out = v / rms(v) * weight`` with ``v = rows[:, col : col + n]`` (activation dtype in and out, sums in float32)."""
    _need_cuda(rows, weight, out)
    T, n = out.shape
    assert rows.shape[0] == T and rows.stride(1) == 1 and col + n <= rows.shape[1] and out.dtype == rows.dtype and out.is_contiguous()
    assert weight.dtype == torch.float32 and weight.numel() == n
    _cost(2 * T * n * rows.element_size(), 4.0 * T * n)
    _check(_lib("mb_activations").mb_rmsnorm_cols(_ptr(rows), _c_int(rows.stride(0)), _c_int(col), _code(rows), _ptr(weight), _c_float(eps), _ptr(out),
                                                 _c_int(T), _c_int(n), _stream()), "rmsnorm of a column block")
