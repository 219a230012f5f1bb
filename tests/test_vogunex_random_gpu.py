"""Vogunex configurations drawn at random (any order of the three mixers, layers that use another layer's weights, earlier or
later ones; head counts and sizes inside and outside what the tensor-core kernels take; windows from one position to longer
than the sequence, pools of one position to more than a page, larger and smaller than the window; rotation of a whole head,
of a part, of nothing; states of odd sizes, one to many groups and norm parts, one to five taps; dense, routed and no
feed-forwards, two to sixteen experts) through the step function in float32 and in bfloat16, with pages of 16: whole, with a
decoded tail, in changing portions and in a mixed batch with few pages, against the plain implementation.  Every size a
configuration allows must run, through a fused path or a plain one, and give the same result.  ``MARIN_B200_RANDOM_SEEDS``
widens the sweep."""
import math
import os
import random

import pytest
import torch

import plain_vogunex as plain
from helpers import mixed_schedule, random_prompt, run_mixed, run_portions, run_whole
from test_vogunex_gpu import close, runtime
from vogunex_models import _attn, _dense, _latent, _moe, _ssm, random_weights, write_model

pytestmark = pytest.mark.gpu
SEEDS = int(os.environ.get("MARIN_B200_RANDOM_SEEDS", "8"))
PAGE = 16


def draw_layer(rng: random.Random) -> dict:
    kind = rng.choice(["attention", "latent_attention", "mamba2"])
    experts = rng.choice([2, 3, 4, 8, 16])
    mlp = rng.choice([None, _dense(rng.choice([48, 64, 200])),
                      _moe(rng.choice([32, 64, 96, 128]), experts, min(experts, rng.choice([1, 2, 4])), rng.choice([0.5, 1.0, 3.0]),
                           shared=rng.choice([None, 64, 96]), shared_limit=rng.choice([None, 2.0]))])
    if kind == "attention":
        kv = rng.choice([1, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 3, 4])
        dim = rng.choice([16, 24, 32, 48, 64, 96, 128])
        vdim = rng.choice([dim, 16, 32, 40, 64])
        dims = rng.choice([dim, dim // 2 - (dim // 2) % 2, 2, 0])
        size = rng.choice([None, 1, 5, 16, 33, 64, 100, 300])
        m = _attn(heads, kv, dim, vdim, rng.choice([1.0, 0.8]) / math.sqrt(dim) * 3.0, size=size, pool=rng.choice([None, 1, 2, 7, 8, 16, 24]),
                  rot={"base": rng.choice([50.0, 10000.0, 500000.0]), "dims": dims} if dims >= 2 else None, softcap=rng.choice([None, 3.0, 50.0]))
    elif kind == "latent_attention":
        heads, dim, vdim = rng.choice([1, 2, 4, 5, 8, 16]), rng.choice([16, 24, 32, 64]), rng.choice([16, 32, 40, 64])
        rot_dim = rng.choice([8, 16, 32])
        m = _latent(heads, dim, rot_dim, vdim, rng.choice([24, 32, 48, 64, 112, 128]), rng.choice([16, 40, 64]), 1.0 / math.sqrt(dim + rot_dim),
                    rng.choice([50.0, 10000.0, 250000.0]), size=rng.choice([None, 1, 9, 40, 64, 300]))
    else:
        groups = rng.choice([1, 1, 2, 4])
        heads = groups * rng.choice([1, 2, 3])
        vdim = rng.choice([8, 16, 24, 32, 48, 64])
        inner = heads * vdim
        m = _ssm(heads, vdim, rng.choice([4, 6, 16, 32, 33, 64]), groups, rng.choice([1, 2, 3, 4, 5]),
                 rng.choice([p for p in (1, 2, heads, 4) if inner % p == 0]))
    return {"type": kind, "mixer": m, "mlp": mlp}


def draw(rng: random.Random) -> dict:
    own = [draw_layer(rng) for _ in range(rng.randint(2, 4))]
    layers = [dict(layer) for layer in own]
    for _ in range(rng.randint(0, 3)):              # runs with another layer's weights, anywhere in the order
        src = rng.randrange(len(own))
        at = rng.randint(0, len(layers))
        layers.insert(at, dict(own[src], weights_of=None, _src=src))
    # (indices of the layers that have weights of their own, after the insertions)
    where = [i for i, layer in enumerate(layers) if "_src" not in layer]
    out = []
    for layer in layers:
        if "_src" in layer:
            layer = {k: v for k, v in layer.items() if k != "_src"} | {"weights_of": where[layer["_src"]]}
        out.append(layer)
    raw = {"architecture": "Vogunex", "vocab": rng.choice([97, 300, 512]), "width": rng.choice([64, 96, 128, 200, 256]),
           "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": out}
    if rng.random() < 0.7:
        raw["embedding"] = {"scale": rng.choice([2.0, 12.0])}
    return raw


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(SEEDS))
def test_a_random_vogunex_configuration(tmp_path, seed, dtype):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model

    rng = random.Random(2000 + seed)
    raw = draw(rng)
    d = write_model(str(tmp_path / "m"), raw, random_weights(raw, 70 + seed))
    w = plain.read_weights(d)
    lengths = {"a": rng.choice([150, 190, 230]), "b": rng.choice([1, 2, 17]), "c": rng.choice([64, 65, 129]), "d": 40, "e": 90}
    tokens = {rid: random_prompt(rng, raw["vocab"], n) for rid, n in lengths.items()}
    want, safe = {}, {}
    for rid, t in tokens.items():
        margins = []
        want[rid] = plain.forward(raw, w, t, None, margins)
        tight = torch.stack(margins).min(dim=0).values < 0.2 if margins else torch.zeros(len(t), dtype=torch.bool)
        safe[rid] = int(torch.nonzero(tight)[0]) if bool(tight.any()) else len(t)
    rt = runtime(dtype)
    _, model = load_model(d, rt)

    def runner(num_pages, graphs=False):
        cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], PAGE, num_pages, 4)
        cache.allocate(rt.device, rt.dtype)
        r = Runner(model, cache, rt, 512)
        if graphs:
            r.enable_graphs((1, 2, 4))
        return r

    def same(got, rid, how):
        what = f"seed {seed}: {[(l['type'][0], l['mixer']['heads'], l.get('weights_of')) for l in raw['layers']]}"
        # (float32: 5e-4, not 2e-4: an angle of 200 radians is good to 1e-5 in 32 bits, and the sharpest of these attentions
        # multiply that by scores of 20)
        close(got, want[rid], dtype, f"{what}, {rid} {how}", 0.03 if dtype == "bfloat16" else 0.0, safe[rid], 0.12, 0.05, 5e-4)

    r = runner(64, graphs=True)
    for rid in ("a", "c"):
        same(run_whole(r, rid, tokens[rid]), rid, "whole")
    n = lengths["a"]
    same(run_portions(r, "at", tokens["a"], [n - 40] + [1] * 40), "a", "with a decoded tail")
    same(run_portions(r, "ap", tokens["a"], [63, 2, 1, 30, n - 96]), "a", "in portions")
    pool = sum(sorted((-(-k // PAGE) for k in lengths.values()), reverse=True)[:4])
    r = runner(pool)
    got = run_mixed(r, tokens, mixed_schedule(random.Random(seed), lengths, max_live=4, decode_tail=8))
    for rid in tokens:
        same(got[rid], rid, "in a mixed batch")
    r.cache.check()


# Sizes nearer a real model's: wide heads, many experts, a latent wider than any tensor-core kernel takes (its attention runs the
# plain kernels), a state of 128 rows, sixteen heads on four kv heads, a pool larger than a page.
LARGER = {
    "architecture": "Vogunex", "vocab": 1000, "width": 512, "embedding": {"scale": 20.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba2", "mixer": _ssm(16, 64, 128, 2, 4, 4), "mlp": _moe(256, 32, 8, 2.0, shared=512, shared_limit=4.0)},
        {"type": "attention", "mixer": _attn(16, 4, 128, 128, 3.0 / math.sqrt(128), size=90, pool=24, rot={"base": 1000000.0, "dims": 128}, softcap=20.0),
         "mlp": _dense(1024)},
        {"type": "latent_attention", "mixer": _latent(16, 128, 64, 128, 512, 384, 1.0 / math.sqrt(192), 10000.0, size=50), "mlp": _moe(128, 6, 2, 1.0)},
        {"type": "attention", "mixer": _attn(16, 4, 128, 128, 3.0 / math.sqrt(128), size=90, pool=24, rot={"base": 1000000.0, "dims": 128}, softcap=20.0),
         "mlp": _dense(1024), "weights_of": 1},
        {"type": "latent_attention", "mixer": _latent(8, 64, 32, 64, 128, 256, 1.0 / math.sqrt(96), 10000.0), "mlp": None},
    ],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_larger_vogunex_configuration(tmp_path, dtype):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model

    raw = LARGER
    d = write_model(str(tmp_path / "m"), raw, random_weights(raw, 5))
    w = plain.read_weights(d)
    rng = random.Random(77)
    lengths = {"a": 170, "b": 3, "c": 65}
    tokens = {rid: random_prompt(rng, raw["vocab"], n) for rid, n in lengths.items()}
    want, safe = {}, {}
    for rid, t in tokens.items():
        margins = []
        want[rid] = plain.forward(raw, w, t, None, margins)
        tight = torch.stack(margins).min(dim=0).values < 0.2
        safe[rid] = int(torch.nonzero(tight)[0]) if bool(tight.any()) else len(t)
    rt = runtime(dtype)
    _, model = load_model(d, rt)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], PAGE, 40, 4)
    cache.allocate(rt.device, rt.dtype)
    r = Runner(model, cache, rt, 512)
    r.enable_graphs((1, 2, 4))

    def same(got, rid, how):
        close(got, want[rid], dtype, f"larger, {rid} {how}", 0.03 if dtype == "bfloat16" else 0.0, safe[rid], 0.12, 0.05, 5e-4)

    same(run_whole(r, "a", tokens["a"]), "a", "whole")
    same(run_portions(r, "at", tokens["a"], [120] + [1] * 50), "a", "with a decoded tail")
    got = run_mixed(r, tokens, mixed_schedule(random.Random(1), lengths, max_live=3, decode_tail=8))
    for rid in tokens:
        same(got[rid], rid, "in a mixed batch")
    r.cache.check()
