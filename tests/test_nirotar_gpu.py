"""Nirotar on the GPU against the plain implementation (``plain_nirotar``, float64 on the CPU): every mechanism alone, then
whole models under every way of cutting the work: each request alone and whole; most of it in one step and the rest one
token at a time (eagerly and from captured graphs); portions of changing size down to two tokens; mixed batches of unequal
requests with so few pages that they are used again; greedy generation through the engine's entry point and scheduler; and
the trace replay as a user runs it.

Tolerances.  float32: |diff| <= 2e-4 (1 + |ref|), the plain result being float64.  bfloat16: the root mean square of the
difference over a row at most 0.06 of the reference's own root mean square, and at most 0.03 on average; one row in fifty (or
one row) may lie between 0.06 and 0.09: the squared activation doubles a relative error, and the narrowest models have few
columns to average it over.  (The experts are chosen by the token ids, so no choice is ever a close call.)
"""
import json
import math
import os
import random
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_nirotar as plain
from helpers import mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole
from nirotar_models import CONFIGS, PAGE, make_model_dir

pytestmark = pytest.mark.gpu
DEV = torch.device(os.environ.get("MARIN_B200_TEST_DEVICE", "cuda:0"))
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": {"a": 37, "b": 9, "c": 150, "d": 1, "e": 66, "f": 41, "g": 27},
           "B": {"a": 140, "b": 2, "c": 65, "d": 300, "e": 31, "f": 129, "g": 400},
           "C": {"a": 100, "b": 1, "c": 190, "d": 17, "e": 64}}


def close(got, want, dtype, what=""):
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if str(dtype).endswith("float32"):
        bad = (got - want).abs() > 2e-4 * (1 + want.abs())
        if bad.any():
            first = int(torch.nonzero(bad.reshape(bad.shape[0], -1).any(dim=1))[0])
            raise AssertionError(f"{what}: first wrong row {first} of {got.shape[0]}, max err {(got - want).abs().max():.3e}")
    else:
        scale = want.pow(2).mean().sqrt()
        rows = (got - want).reshape(got.shape[0], -1).pow(2).mean(dim=1).sqrt() / scale
        over = rows > 0.06
        if int(over.sum()) > max(1, rows.numel() // 50) or bool((rows > 0.09).any()) or rows.mean() > 0.03:
            raise AssertionError(f"{what}: {int(over.sum())} of {rows.numel()} rows beyond 0.06 (first {int(torch.nonzero(over)[0]) if over.any() else -1}, "
                                 f"max {rows.max():.3e}), mean {rows.mean():.3e}")


def torch_dtype(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def runtime(dtype):
    from marin_b200.parts import Runtime
    return Runtime(DEV, torch_dtype(dtype))


def bf(t):
    return t.to(torch.bfloat16)


def harness(needs, rt, cache_of=None, page=8, pages=80, ctx_len=2048):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner

    cache = CacheManager(list(needs), list(cache_of) if cache_of else [None] * len(needs), page, pages, 4)
    cache.allocate(rt.device, rt.dtype)
    return Runner(SimpleNamespace(spec=SimpleNamespace(vocab_size=1 << 30)), cache, rt, ctx_len)


def feed(mixers, runner, x, cuts, req="r"):
    """Runs ``x`` [T, hidden] through the mixers (one after the other on the same input, each with its view of the cache) in
    portions ``cuts``; returns what each added to a zero residual."""
    from marin_b200.engine import StepEntry

    runner.begin(req)
    got, at = [[] for _ in mixers], 0
    for n in cuts:
        runner.cache.reserve(req, at + n)
        ctx = runner.build_context([StepEntry(req, [0] * n, [])])
        for i, mixer in enumerate(mixers):
            residual = torch.zeros(n, x.shape[1], device=DEV)
            mixer.forward(x[at:at + n].to(DEV).contiguous(), ctx, runner.views.view(i, ctx), residual)
            got[i].append(residual.cpu())
        runner.cache.commit(req, at + n)
        at += n
    runner.end(req)
    assert at == x.shape[0]
    return [torch.cat(g) for g in got]


def mat(g, r, c, gain=1.0):
    return torch.randn(r, c, generator=g) * gain / math.sqrt(c)


# ---- grouped-query attention with a window and a learned sink, alone -------------------------------------------------

def attention_weights(hidden, m, seed, same_qk=False):
    g = torch.Generator().manual_seed(seed)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"m.q": mat(g, H * d, hidden, 2.0), "m.k": mat(g, G * d, hidden, 2.0), "m.v": mat(g, G * dv, hidden), "m.o": mat(g, hidden, H * dv),
         "m.sink": 1.5 * torch.randn(H, generator=g)}
    if same_qk:
        assert H == G
        w["m.k"] = w["m.q"].clone()
    return {k: bf(v) for k, v in w.items()}


def build_attention(hidden, m, name="m"):
    from marin_b200.config.nirotar import NirotarLayer
    from marin_b200.models.nirotar import ATTENTION_NAMES, _position
    from marin_b200.parts import lookup

    parsed = NirotarLayer.parse({"type": "attention", "mixer": m, "mlp": None}, 0).mixer
    return lookup("mixer", "sink_attention")(
        hidden=hidden, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"], scale=m["scale"], bias=False,
        qk_norm=None, position=_position(parsed["rot"], m["dim"]), window=(m.get("mask") or {}).get("size"), sink="learned",
        names=ATTENTION_NAMES, name=name)


def plain_attention(x, w, m):
    return plain.window_attention(x.double(), torch.arange(x.shape[0]), w, "m.", m)


CUTS = [[61], [29, 1, 1, 30], [2, 2, 1, 56], [1] * 61, [16, 17, 15, 13]]
BANDS = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 13}, "rot": {"base": 100.0, "dims": 8, "scaling": BANDS}},
    {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "mask": {"size": 1}, "rot": {"base": 100.0, "dims": 32}},
    {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 20}, "rot": {"base": 500.0, "dims": 32, "scaling": BANDS}},
    {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "mask": {"size": 50}, "rot": {"base": 500.0, "dims": 128}},
    {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 97}, "rot": {"base": 500.0, "dims": 64, "scaling": BANDS}},
    {"heads": 2, "kv_heads": 1, "dim": 80, "vdim": 48, "scale": 0.11, "rot": {"base": 100.0, "dims": 80, "scaling": BANDS}},
    {"heads": 5, "kv_heads": 1, "dim": 24, "vdim": 40, "scale": 0.25, "mask": {"size": 64}, "rot": {"base": 100.0, "dims": 2}},
    {"heads": 2, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125},
    # more than 8 query heads a kv head: both halves of the single-token kernel's 16-row tile, the lower one partly filled
    {"heads": 12, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.18, "mask": {"size": 40}, "rot": {"base": 100.0, "dims": 16}},
    {"heads": 32, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.25, "mask": {"size": 23}, "rot": {"base": 100.0, "dims": 16, "scaling": BANDS}},
], ids=lambda m: f"{m['heads']}x{m['kv_heads']}x{m['dim']}x{m['vdim']}")
def test_window_attention_alone(dtype, m):
    rt = runtime(dtype)
    hidden = 48
    mixer = build_attention(hidden, m)
    w = attention_weights(hidden, m, 1)
    mixer.load(dict(w), rt)
    x = torch.randn(61, hidden, generator=torch.Generator().manual_seed(2)).to(rt.dtype)
    want = plain_attention(x, w, m)
    # heads of 64 or 128 with values as wide and pages of 16: prompt portions go to the kernel plain causal attention uses
    page = 16 if m["dim"] == m["vdim"] and m["dim"] in (64, 128) else 8
    for cuts in CUTS:
        close(feed([mixer], harness([mixer.cache_need()], rt, page=page), x, cuts)[0], want, dtype, f"cuts {cuts[:4]}")
    if m["dim"] % 16 == 0 and m["vdim"] % 16 == 0:   # a longer sequence: several key blocks, the window's edge inside and on block borders
        x = torch.randn(333, hidden, generator=torch.Generator().manual_seed(3)).to(rt.dtype)
        want = plain_attention(x, w, m)
        for cuts in ([333], [130, 1, 1, 201], [64, 64, 64, 141]):
            close(feed([mixer], harness([mixer.cache_need()], rt, page=page), x, cuts)[0], want, dtype, f"long, cuts {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sink", [12.0, 0.0, -12.0])
def test_the_learned_sink_takes_its_share(dtype, sink):
    """A sink far above every score leaves the keys next to nothing (the output vanishes); far below, the keys share the
    whole weight as in a softmax without it; a sink of 0 is one more in the denominator."""
    rt = runtime(dtype)
    hidden = 32
    m = {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.05}
    w = attention_weights(hidden, m, 7)
    w["m.sink"] = bf(torch.tensor([sink, sink]))
    mixer = build_attention(hidden, m)
    mixer.load(dict(w), rt)
    x = torch.randn(9, hidden, generator=torch.Generator().manual_seed(4)).to(rt.dtype)
    want = plain_attention(x, w, m)
    without = dict(w, **{"m.sink": torch.tensor([-1e4, -1e4])})
    free = plain_attention(x, without, m)
    if sink > 5:
        assert want.abs().max() < 1e-3 * free.abs().max()
    elif sink < -5:
        assert (want - free).abs().max() < 1e-3 * free.abs().max()
    else:
        assert (want - free).abs().max() > 0.05 * free.abs().max()
    for cuts in ([9], [1] * 9, [4, 1, 4]):
        got = feed([mixer], harness([mixer.cache_need()], rt), x, cuts)[0]
        if sink > 5:
            assert got.abs().max() < 2e-3 * free.abs().max()
        else:
            close(got, want, dtype, f"cuts {cuts}")


def standout_case(T, at_query, at_key, window, hidden=32, seed=8):
    """A sequence in which the query at ``at_query`` and the key at ``at_key`` come from one strong input row (the key's a
    longer copy, so its value differs) while all other rows are weak: with k = q (the same matrix, no rotation) that score
    stands far above the rest, the query's own key included."""
    m = {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3}
    if window:
        m["mask"] = {"size": window}
    w = attention_weights(hidden, m, seed, same_qk=True)
    g = torch.Generator().manual_seed(seed + 1)
    x = 0.3 * torch.randn(T, hidden, generator=g)
    strong = torch.randn(hidden, generator=g)
    x[at_query] = strong
    x[at_key] = 1.5 * strong
    return m, w, x


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [64, 50, 137])
def test_window_edges_in_prompts_and_in_decoding(dtype, window):
    """The strong key is the oldest position the query still sees (``window - 1`` back) or the one before it (not seen); the
    query lies early (the window not yet full), in the middle, and on page borders (pages of 16)."""
    rt = runtime(dtype)
    T = 2 * window + 40
    for at_query, back, seen in ((T - 1, window - 1, True), (T - 1, window, False), (window - 1, window - 1, True), (window, window, False),
                                 (window + 16, window - 1, True), (window + 15, window, False), (T - 20, 1, True)):
        at_key = at_query - back
        m, w, x = standout_case(T, at_query, at_key, window, seed=20 + at_query % 7)
        x = x.to(rt.dtype)
        mixer = build_attention(32, m)
        mixer.load(dict(w), rt)
        want = plain_attention(x, w, m)
        x_without = x.clone()
        x_without[at_key] = 0.0
        moved = (plain_attention(x_without, w, m)[at_query] - want[at_query]).abs().max() > 0.1 * want[at_query].abs().max()
        assert bool(moved) == seen
        for cuts in ([T], [at_query, 1, T - at_query - 1], [at_key, 1] + [1] * back + [T - at_query - 1],
                     [max(at_query - 9, 1), 2, 2, 2] + [1] * 4 + [T - max(at_query - 9, 1) - 10]):
            cuts = [c for c in cuts if c > 0]
            assert sum(cuts) == T
            got = feed([mixer], harness([mixer.cache_need()], rt, page=16, pages=60), x, cuts)[0]
            close(got[at_query:at_query + 1], want[at_query:at_query + 1], dtype, f"query {at_query} key {at_key} cuts {cuts[:4]}")
            close(got, want, dtype, f"all rows, query {at_query} key {at_key} cuts {cuts[:4]}")


def test_a_window_gives_its_pages_back():
    """Decoding far beyond the window holds no more pages than the window needs, and the results stay right."""
    rt = runtime("float32")
    m = {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.3, "mask": {"size": 20}, "rot": {"base": 100.0, "dims": 16}}
    mixer = build_attention(32, m)
    w = attention_weights(32, m, 5)
    mixer.load(dict(w), rt)
    x = torch.randn(400, 32, generator=torch.Generator().manual_seed(6))
    runner = harness([mixer.cache_need()], rt, page=8, pages=10)         # 80 positions: far fewer than the sequence
    got = feed([mixer], runner, x, [30] + [1] * 300 + [35, 35])[0]
    close(got, plain_attention(x, w, m), "float32", "long decoding in a small pool")
    runner.cache.check()


# ---- attention over a shared latent, alone ---------------------------------------------------------------------------------

def latent_weights(hidden, m, seed, own=True):
    g = torch.Generator().manual_seed(seed)
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    w = {"m.q": mat(g, H * (d + dr), hidden, 2.0), "m.uk": mat(g, H * d, r, 1.5), "m.uv": mat(g, H * dv, r, 1.5), "m.o": mat(g, hidden, H * dv),
         "m.sink": 1.5 * torch.randn(H, generator=g)}
    if own:
        w["m.dkv"], w["m.dkv.norm"] = mat(g, r + dr, hidden, 2.0), 1.2 + 0.3 * torch.randn(r, generator=g)
    return {k: bf(v) for k, v in w.items()}


def build_latent(hidden, m, name="m", own=True, eps=1e-5):
    from marin_b200.config.nirotar import NirotarLayer
    from marin_b200.models.nirotar import _position
    from marin_b200.parts import lookup

    parsed = NirotarLayer.parse({"type": "latent_attention", "mixer": m, "mlp": None}, 0).mixer
    return lookup("mixer", "latent_attention")(
        hidden=hidden, heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"],
        norm_eps=eps, position=_position(parsed["rot"], m["rot_dim"]), sink="learned", own_latent=own, name=name)


def plain_latent(x, w, m, kept=None, eps=1e-5):
    T = x.shape[0]
    pos = torch.arange(T)
    m = dict(m, rot=m.get("rot") or {"base": 1.0, "dims": 0})
    c, k_rot = kept if kept is not None else plain.latent_of(x.double(), pos, w, "m.", m, eps)
    return plain.latent_attention(x.double(), pos, w, "m.", m, c, k_rot), (c, k_rot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 3, "dim": 12, "rot_dim": 6, "vdim": 10, "kv_rank": 20, "scale": 0.3, "rot": {"base": 100.0, "dims": 6}},
    {"heads": 8, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 48, "scale": 0.15, "rot": {"base": 1000.0, "dims": 16}},
    {"heads": 4, "dim": 16, "rot_dim": 16, "vdim": 24, "kv_rank": 112, "scale": 0.18, "rot": {"base": 30000.0, "dims": 16}},
    {"heads": 2, "dim": 64, "rot_dim": 32, "vdim": 128, "kv_rank": 128, "scale": 0.1, "rot": {"base": 1000.0, "dims": 32}},
    {"heads": 10, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 32, "scale": 0.2},
    {"heads": 12, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 64, "scale": 0.12, "rot": {"base": 500.0, "dims": 16}},
    {"heads": 16, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 48, "scale": 0.2, "rot": {"base": 50.0, "dims": 8}},
    {"heads": 2, "dim": 32, "rot_dim": 64, "vdim": 64, "kv_rank": 128, "scale": 0.09, "rot": {"base": 10000.0, "dims": 64}},
    {"heads": 1, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 24, "scale": 0.3, "rot": {"base": 10.0, "dims": 4}},
], ids=lambda m: f"{m['heads']}x{m['dim']}+{m['rot_dim']}x{m['vdim']}r{m['kv_rank']}")
def test_latent_attention_alone_and_read_by_a_second_layer(dtype, m):
    """A layer that keeps the latent, and a second one with other head sizes and weights of its own that reads the first
    one's page rows."""
    rt = runtime(dtype)
    hidden = 48
    m2 = dict(m, heads=max(1, m["heads"] // 2), dim=m["dim"] + 16, vdim=16)
    w1, w2 = latent_weights(hidden, m, 1), latent_weights(hidden, m2, 2, own=False)
    first, second = build_latent(hidden, m), build_latent(hidden, m2, own=False)
    first.load(dict(w1), rt)
    second.load(dict(w2), rt)
    assert first.cache_need() == second.cache_need()
    for T, all_cuts in ((61, CUTS), (333, ([333], [130, 1, 1, 201], [64, 64, 64, 141]))):
        x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(2 + T)).to(rt.dtype)
        want1, kept = plain_latent(x, w1, m)
        want2, _ = plain_latent(x, w2, m2, kept)
        for cuts in all_cuts:
            got = feed([first, second], harness([first.cache_need(), None], rt, cache_of=[None, 0], page=16, pages=40), x, cuts)
            close(got[0], want1, dtype, f"owner, cuts {cuts[:4]}")
            close(got[1], want2, dtype, f"reader, cuts {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank", [32, 64])
def test_one_far_latent_stands_out_among_hundreds(dtype, rank):
    """Every head's rotated query part and the shared key part come from the same matrix, read the first half of the input
    only and are not rotated; the row at position 5 repeats the last row's first half, longer, with a second half of its own
    (so its latent, and with it its value, differs).  Its key then scores far above the rest for the last query, 700
    positions later."""
    rt = runtime(dtype)
    T, hidden = 700, 32
    m = {"heads": 2, "dim": 16, "rot_dim": 16, "vdim": 24, "kv_rank": rank, "scale": 0.3}
    w = latent_weights(hidden, m, 9)
    q = w["m.q"].float().view(2, 32, hidden)
    q[0, 16:, 16:] = 0.0
    q[1, 16:] = q[0, 16:]
    w["m.q"] = bf(q.reshape(64, hidden))
    dkv = w["m.dkv"].float()
    dkv[rank:] = q[0, 16:]
    w["m.dkv"] = bf(dkv)
    w["m.uk"] = bf(0.2 * w["m.uk"].float())                 # the unrotated part stays small beside the shared part
    g = torch.Generator().manual_seed(10)
    x = 0.3 * torch.randn(T, hidden, generator=g)
    strong = 2.0 * torch.randn(hidden, generator=g)
    x[T - 1] = strong
    x[5] = torch.cat([1.5 * strong[:16], torch.randn(16, generator=g)])
    x = x.to(rt.dtype)
    mixer = build_latent(hidden, m)
    mixer.load(dict(w), rt)
    want, _ = plain_latent(x, w, m)
    x_without = x.clone()
    x_without[5] = 0.3 * torch.randn(hidden, generator=torch.Generator().manual_seed(1)).to(rt.dtype)
    assert (plain_latent(x_without, w, m)[0][-1] - want[-1]).abs().max() > 0.1 * want[-1].abs().max()     # the far key matters
    for cuts in ([T], [T - 1, 1], [300, 399, 1], [64] * 10 + [59, 1]):
        got = feed([mixer], harness([mixer.cache_need()], rt, page=16, pages=60), x, cuts)[0]
        close(got[-3:], want[-3:], dtype, f"cuts {cuts[:3]}")
        close(got, want, dtype, f"all rows, cuts {cuts[:3]}")


# ---- experts named by a table, alone ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, ff, E, top, shared, T", [(48, 40, 5, 2, 24, 37), (64, 16, 7, 3, None, 150), (256, 128, 8, 2, 64, 300),
                                                           (96, 48, 4, 1, 48, 64), (32, 24, 3, 3, None, 9), (128, 64, 16, 1, 128, 1),
                                                           (256, 64, 6, 2, 192, 1500)])
def test_table_experts_alone(dtype, hidden, ff, E, top, shared, T):
    from marin_b200.engine.context import Workspace
    from marin_b200.models.nirotar import EXPERT_NAMES
    from marin_b200.parts import lookup

    rt = runtime(dtype)
    vocab = 53
    g = torch.Generator().manual_seed(hidden + E)
    w = {}
    for e in range(E):
        w[f"f.e{e}.up"], w[f"f.e{e}.down"] = bf(mat(g, ff, hidden, 2.0)), bf(mat(g, hidden, ff, 1.5))
    if shared:
        w["f.shared.up"], w["f.shared.down"] = bf(mat(g, shared, hidden, 2.0)), bf(mat(g, hidden, shared, 1.5))
    w["f.table"] = torch.rand(vocab, E, generator=g).argsort(dim=1)[:, :top].to(torch.int32).contiguous()
    part = lookup("feedforward", "routed_experts")(hidden=hidden, intermediate=ff, experts=E, top=top, name="f", names=EXPERT_NAMES,
                                                   router="table", vocab=vocab, activation="relu2", weight_on="output", shared_intermediate=shared)
    assert {s.name for s in part.tensor_specs()} == set(w)
    part.load(dict(w), rt)
    tokens = torch.randint(0, vocab, (T,), generator=g).tolist()
    x = torch.randn(T, hidden, generator=g).to(rt.dtype)
    mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.table_experts(x.double(), tokens, w, "f.", mlp)
    ids = torch.tensor(tokens, dtype=torch.int32, device=DEV)
    ws = Workspace(DEV)
    y = torch.zeros(T, hidden, device=DEV)
    part.forward(x.to(DEV), SimpleNamespace(workspace=ws, token_ids=ids), y)
    close(y, want, dtype, "all rows at once")
    for lo, hi in ((0, 1), (T // 2, min(T, T // 2 + 3))):
        part_y = torch.ones(hi - lo, hidden, device=DEV)            # it adds into what is there
        part.forward(x[lo:hi].contiguous().to(DEV), SimpleNamespace(workspace=ws, token_ids=ids[lo:hi].contiguous()), part_y)
        close(part_y - 1.0, want[lo:hi], dtype, f"rows {lo}:{hi} alone")
        if dtype == "float32":
            again = torch.zeros(hi - lo, hidden, device=DEV)
            part.forward(x[lo:hi].contiguous().to(DEV), SimpleNamespace(workspace=ws, token_ids=ids[lo:hi].contiguous()), again)
            assert torch.equal(again, y[lo:hi])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, N, K", [(1, 3, 20, 12), (37, 4, 112, 16), (200, 8, 48, 32), (70, 2, 40, 96), (16, 5, 33, 24)])
def test_products_per_head_over_strided_rows(dtype, T, H, N, K):
    from marin_b200.kernels import ops

    td = torch_dtype(dtype)
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, H * (K + 8) + 8, generator=g).to(td)
    w = (torch.randn(H, N, K, generator=g) / math.sqrt(K)).to(td)
    out = torch.full((T, H * (N + 2)), 7.0, dtype=td, device=DEV)
    ops.heads_product(x.to(DEV), K + 8, K, w.to(DEV), out, N + 2)
    got = out.cpu().view(T, H, N + 2)
    assert bool((got[:, :, N:] == 7.0).all())                       # what lies between the heads' slices is left alone
    xs = x[:, :H * (K + 8)].view(T, H, K + 8)[:, :, :K].double()
    want = torch.einsum("thk,hnk->thn", xs, w.double())
    torch.testing.assert_close(got[:, :, :N].double(), want, **(dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)))


@pytest.mark.parametrize("T", [1, 8, 40, 200, 2100])
def test_the_product_applies_the_squared_relu(T):
    """bfloat16: the tensor-core product squares the positive part of its float32 sums before it rounds them; float32: the
    same through the plain product and the activation's own kernel."""
    from marin_b200.kernels import ops

    g = torch.Generator().manual_seed(T)
    x, w = torch.randn(T, 192, generator=g), torch.randn(320, 192, generator=g) / math.sqrt(192)
    for td, tol in ((torch.bfloat16, dict(rtol=2e-2, atol=2e-2)), (torch.float32, dict(rtol=1e-5, atol=1e-5))):
        xd, wd = x.to(td), w.to(td)
        want = torch.relu(xd.double() @ wd.double().T) ** 2
        out = torch.empty(T, 320, dtype=td, device=DEV)
        ops.gemm_act(xd.to(DEV), wd.to(DEV), out, "relu2")
        torch.testing.assert_close(out.double().cpu(), want, **tol)
        assert float(out.min()) >= 0.0 and bool((out == 0).any())


# ---- whole models -----------------------------------------------------------------------------------------------------

class Case:
    def __init__(self, tmp, name, dtype):
        from marin_b200.engine import load_model

        self.name, self.dtype = name, dtype
        self.raw = CONFIGS[name]
        self.dir = make_model_dir(str(tmp / f"{name}-{dtype}"), name, seed=11)
        self.w = plain.read_weights(self.dir)
        rng = random.Random(5)
        self.tokens = {rid: random_prompt(rng, self.raw["vocab"], n) for rid, n in LENGTHS[name].items()}
        self.want = {rid: plain.forward(self.raw, self.w, t)[0] for rid, t in self.tokens.items()}
        self.rt = runtime(dtype)
        self.config, self.model = load_model(self.dir, self.rt)
        self.page = PAGE[name]

    def runner(self, num_pages, max_requests=4, graphs=False):
        from marin_b200.cache import CacheManager
        from marin_b200.engine import Runner

        cache = CacheManager(self.model.cache_needs(), [e.cache_of for e in self.model.spec.schedule], self.page, num_pages, max_requests)
        cache.allocate(self.rt.device, self.rt.dtype)
        runner = Runner(self.model, cache, self.rt, 512)
        if graphs:
            runner.enable_graphs((1, 2, 4))
        return runner

    def close(self, got, rid, what):
        close(got, self.want[rid], self.dtype, what)


@pytest.fixture(scope="module", params=[(n, d) for n in CONFIGS for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    return Case(tmp_path_factory.mktemp("nirotar"), *request.param)


def test_the_residual_stream_after_every_layer(case):
    from marin_b200.engine import StepEntry

    rid = "a"
    _, want = plain.forward(case.raw, case.w, case.tokens[rid])
    got = {}
    runner = case.runner(64)
    runner.begin(rid)
    runner.step([StepEntry(rid, case.tokens[rid], [0])], observe=lambda i, h: got.__setitem__(i, h.clone()))
    assert len(got) == want.shape[0] + 1
    for i in range(want.shape[0]):
        close(got[i + 1], want[i], case.dtype, f"after layer {i}")


def test_whole_prompts_and_the_first_tokens(case):
    runner = case.runner(64)
    for rid, tokens in case.tokens.items():
        case.close(run_whole(runner, rid, tokens), rid, f"{rid} whole")
    runner.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
def test_prefill_then_token_by_token(case, graphs):
    """Most of a prompt in one step and the rest one token at a time, eagerly and from captured graphs: a tail long enough
    for a window to pass wholly over decoded tokens; and a request decoded from its very first token."""
    runner = case.runner(64, graphs=graphs)
    for rid, tail in (("c", 90), ("a", 30), ("e", 5)):
        tokens = case.tokens[rid]
        n = max(len(tokens) - tail, 0)
        sizes = ([n] if n > 0 else []) + [1] * (len(tokens) - n)
        case.close(run_portions(runner, rid + "t", tokens, sizes), rid, f"{rid}, last {tail} one by one")
    rid = "e"
    case.close(run_portions(runner, rid + "1", case.tokens[rid], [1] * len(case.tokens[rid])), rid, f"{rid} token by token")
    runner.cache.check()


def test_portions_of_changing_size_down_to_two_tokens(case):
    runner = case.runner(64)
    for rid in ("c", "a"):
        tokens = case.tokens[rid]
        for sizes in ([7, 2, 13, 3, 2, 5], [2], [case.page, case.page + 1, case.page - 1], [64, 1, 2]):
            case.close(run_portions(runner, rid + "p", tokens, portions(len(tokens), sizes)), rid, f"{rid} in {sizes}")


@pytest.mark.parametrize("graphs", [False, True])
def test_mixed_batches_reuse_pages_and_slots(case, graphs):
    """Up to four live requests, portions of some beside single tokens of others, in a pool that holds the four largest
    only: pages and slots of finished requests are handed to the next ones."""
    rng = random.Random(9)
    lengths = {rid: len(t) for rid, t in case.tokens.items()}
    sched = mixed_schedule(rng, lengths, max_live=4, decode_tail=6)
    pool = sum(sorted((-(-n // case.page) for n in lengths.values()), reverse=True)[:4])
    runner = case.runner(pool, max_requests=4, graphs=graphs)
    got = run_mixed(runner, case.tokens, sched)
    for rid in case.tokens:
        case.close(got[rid], rid, f"{rid} mixed")
    runner.cache.check()
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    again = run_mixed(runner, case.tokens, sched)
    for rid in case.tokens:
        case.close(again[rid], rid, f"{rid} mixed, second time")


def test_a_batch_gives_each_request_what_it_gets_alone(case):
    """float32: the logits of a request are the same bits whatever else the step holds and however its prompt was cut."""
    if case.dtype != "float32":
        pytest.skip("bit equality is the 32-bit path's claim")
    from marin_b200.engine import StepEntry

    runner = case.runner(64)
    alone = {rid: run_whole(runner, rid, case.tokens[rid]) for rid in ("a", "b", "e")}
    for rid in alone:
        runner.begin(rid)
    logits = runner.step([StepEntry(rid, case.tokens[rid], list(range(len(case.tokens[rid])))) for rid in ("a", "b", "e")])
    k = 0
    for rid in ("a", "b", "e"):
        n = len(case.tokens[rid])
        assert torch.equal(logits[k:k + n], alone[rid]), rid
        k += n
        runner.end(rid)
    cut = run_portions(runner, "ap", case.tokens["a"], portions(len(case.tokens["a"]), [5, 2, 9, 1]))
    assert torch.equal(cut, alone["a"])


def test_greedy_generation_through_the_engine(case):
    """The entry point, the scheduler and device sampling: the tokens are those the plain implementation's logits rank
    first (a token whose plain logit lies within 1e-3 (32-bit) or 0.15 (16-bit) of the largest counts as first)."""
    from marin_b200.engine import Engine
    from marin_b200.sampling.sampler import SamplingParams

    engine = Engine(case.dir, dtype=case.dtype, ctx=256, page_size=case.page, num_pages=64, max_batch=4, token_budget=32)
    prompts = [case.tokens["a"][:21], case.tokens["e"][:3], case.tokens["c"][:40]]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    slack = 1e-3 if case.dtype == "float32" else 0.15
    for prompt, out in zip(prompts, outs):
        assert len(out.tokens) == 10
        seq = list(prompt)
        for token in out.tokens:
            logits = plain.forward(case.raw, case.w, seq)[0][-1]
            assert logits[token] >= logits.max() - slack, (len(seq), token, int(logits.argmax()))
            seq.append(token)


def test_trace_replay_as_a_user_runs_it(tmp_path):
    """bin/trace_run in a process of its own: steps on standard input, logits read back from files."""
    name, dtype = "B", "bfloat16"
    raw = CONFIGS[name]
    d = make_model_dir(str(tmp_path / "model"), name, seed=12)
    w = plain.read_weights(d)
    rng = random.Random(3)
    lengths = {"a": 70, "b": 130, "c": 41, "d": 64, "e": 100, "f": 2}
    tokens = {rid: random_prompt(rng, raw["vocab"], n) for rid, n in lengths.items()}
    want = {rid: plain.forward(raw, w, t)[0] for rid, t in tokens.items()}
    sched = mixed_schedule(rng, lengths, max_live=4, decode_tail=5)
    pool = sum(sorted((-(-n // 64) * 64 for n in lengths.values()), reverse=True)[:4])
    out = str(tmp_path / "out")
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
                             "--max-tokens", str(pool)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    fed = {rid: 0 for rid in tokens}
    for i, (entries, ends) in enumerate(sched):
        line, rows = [], []
        for rid, n in entries:
            wanted = [n - 1] if n > 2 else list(range(n))
            line.append({"id": rid, "tokens": tokens[rid][fed[rid]:fed[rid] + n], "want": wanted})
            rows.append(want[rid][[fed[rid] + k for k in wanted]])
            fed[rid] += n
        proc.stdin.write(json.dumps({"step": i, "entries": line, "end": ends}) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {i}"
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, raw["vocab"]).copy())
        close(got, torch.cat(rows), dtype, f"step {i}")
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


def test_the_command_line_takes_a_nirotar_folder(tmp_path):
    """Random-weights mode from a config.json of this design, greedy generation, and the bench command with its stage table."""
    run = [sys.executable, os.path.join(ROOT, "bin", "marin-run")]
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["B"]))
    model = str(tmp_path / "model")
    out = subprocess.run(run + ["random", "--config", str(cfg), "--seed", "3", "--out", model], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert sorted(os.listdir(model)) == ["config.json", "model.safetensors"]
    a = subprocess.run(run + [model, "--prompt-ids", "5,6,7,8,9", "--temp", "0", "--max-tokens", "6"], capture_output=True, text=True)
    b = subprocess.run(run + [model, "--prompt-ids", "5 6 7 8 9", "--temp", "0", "--max-tokens", "6"], capture_output=True, text=True)
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    assert a.stdout == b.stdout and len(a.stdout.split()) == 6
    e = subprocess.run(run + ["bench", model, "--prompt-tokens", "16", "--tokens", "8", "--runs", "2", "--warmup", "1", "--profile"],
                       capture_output=True, text=True)
    assert e.returncode == 0, e.stderr
    for stage in ("embedding", "q|k|v|g", "q|dkv", "heads", "q into the latent", "attention", "v from the latent", "router",
                  "experts", "head", "sampling"):
        assert stage in e.stdout, stage
