"""Nirotar configurations drawn at random (any order of the two mixers, readers of earlier latents, head counts and sizes
inside and outside what the tensor-core kernels take, windows from one position to longer than the sequence, rotation of a
whole head, of a part, of nothing, with and without bands, two to sixteen experts, layers without feed-forward) through the
step function in float32 and in bfloat16, with pages of 16: whole, with a decoded tail, in changing portions and in a mixed
batch with few pages, against the plain implementation.  Every size a configuration allows must run, through a fused path
or a plain one, and give the same result.  ``MARIN_B200_RANDOM_SEEDS`` widens the sweep."""
import math
import os
import random

import pytest
import torch

import plain_nirotar as plain
from helpers import mixed_schedule, random_prompt, run_mixed, run_portions, run_whole
from nirotar_models import _attn, _latent, _moe, random_weights, write_model
from test_nirotar_gpu import close, runtime

pytestmark = pytest.mark.gpu
SEEDS = int(os.environ.get("MARIN_B200_RANDOM_SEEDS", "8"))
PAGE = 16


def draw_rot(rng: random.Random, width: int, bands: bool):
    dims = rng.choice([width, width, width // 2 - (width // 2) % 2, 2, 0])
    if dims < 2:
        return None
    rot = {"base": rng.choice([50.0, 1000.0, 10000.0, 500000.0]), "dims": dims}
    if bands and rng.random() < 0.6:
        rot["scaling"] = {"factor": rng.choice([2.0, 8.0, 32.0]), "low": 1.0, "high": rng.choice([2.0, 4.0]),
                          "original": rng.choice([16, 64, 1024])}
    return rot


def draw(rng: random.Random) -> dict:
    layers, owners = [], []
    for i in range(rng.randint(2, 5)):
        experts = rng.choice([2, 3, 4, 8, 16])
        mlp = None if rng.random() < 0.15 else _moe(rng.choice([32, 64, 96, 128, 192]), experts, min(experts, rng.choice([1, 1, 2, 3])),
                                                    shared=rng.choice([None, 64, 96, 128]))
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3, 4])
            heads = kv * rng.choice([1, 2, 3, 4, 6, 12, 16] if kv == 1 else [1, 2, 3, 4, 6])
            dim = rng.choice([16, 24, 32, 48, 64, 64, 80, 128])
            vdim = rng.choice([dim, dim, 16, 32, 40, 64, 128])
            m = _attn(heads, kv, dim, vdim, rng.choice([1.0, 0.8]) / math.sqrt(dim), mask=rng.choice([None, 1, 7, 16, 33, 64, 100, 150]),
                      rot=draw_rot(rng, dim, True))
            layers.append({"type": "attention", "mixer": m, "mlp": mlp})
            continue
        heads, dim, vdim = rng.choice([1, 2, 4, 5, 8, 12, 16, 20]), rng.choice([16, 24, 32, 64]), rng.choice([16, 32, 40, 64, 128])
        if owners and rng.random() < 0.4:
            src = rng.choice(owners)
            o = layers[src]["mixer"]
            m = _latent(heads, dim, o["rot_dim"], vdim, o["kv_rank"], 1.0 / math.sqrt(dim + o["rot_dim"]), rot=o.get("rot"), kv_from=src)
        else:
            rot_dim = rng.choice([8, 16, 32, 64])
            m = _latent(heads, dim, rot_dim, vdim, rng.choice([24, 32, 48, 64, 64, 112, 128, 128]), 1.0 / math.sqrt(dim + rot_dim),
                        rot=draw_rot(rng, rot_dim, False))
            owners.append(i)
        layers.append({"type": "latent_attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Nirotar", "vocab": rng.choice([97, 300, 512, 777]), "width": rng.choice([64, 96, 128, 192, 200, 256, 320]),
            "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(SEEDS))
def test_a_random_nirotar_configuration(tmp_path, seed, dtype):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model

    rng = random.Random(1000 + seed)
    raw = draw(rng)
    d = write_model(str(tmp_path / "m"), raw, random_weights(raw, 50 + seed))
    w = plain.read_weights(d)
    lengths = {"a": rng.choice([150, 190, 230]), "b": rng.choice([1, 2, 17]), "c": rng.choice([64, 65, 129]), "d": 40, "e": 90}
    tokens = {rid: random_prompt(rng, raw["vocab"], n) for rid, n in lengths.items()}
    want = {rid: plain.forward(raw, w, t)[0] for rid, t in tokens.items()}
    rt = runtime(dtype)
    _, model = load_model(d, rt)

    def runner(num_pages, graphs=False):
        cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], PAGE, num_pages, 4)
        cache.allocate(rt.device, rt.dtype)
        r = Runner(model, cache, rt, 512)
        if graphs:
            r.enable_graphs((1, 2, 4))
        return r

    what = f"seed {seed}: {[(l['type'][0], l['mixer']['heads']) for l in raw['layers']]}"
    r = runner(64, graphs=True)
    for rid in ("a", "c"):
        close(run_whole(r, rid, tokens[rid]), want[rid], dtype, f"{what}, {rid} whole")
    n = lengths["a"]
    close(run_portions(r, "at", tokens["a"], [n - 40] + [1] * 40), want["a"], dtype, f"{what}, a with a decoded tail")
    close(run_portions(r, "ap", tokens["a"], [63, 2, 1, 30, n - 96]), want["a"], dtype, f"{what}, a in portions")
    pool = sum(sorted((-(-k // PAGE) for k in lengths.values()), reverse=True)[:4])
    r = runner(pool)
    got = run_mixed(r, tokens, mixed_schedule(random.Random(seed), lengths, max_live=4, decode_tail=8))
    for rid in tokens:
        close(got[rid], want[rid], dtype, f"{what}, {rid} in a mixed batch")
    r.cache.check()
