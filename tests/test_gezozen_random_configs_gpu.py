"""Gezozen configurations drawn from a seed: one to six layers of any kind in any order, 1 to 12 heads, head sizes
that are and are not multiples of 8, rotations of 2 coordinates up to the whole head, windows of 1 to 300, 1 to 16
experts with and without a shared expert, 1 to 7 norm groups, pages of 4 to 64.  Every configuration runs whole,
in portions and token by token, in 32-bit and in bfloat16, against the plain implementation."""
import random

import pytest
import torch

import helpers
import plain_gezozen as plain
from gezozen_configs import every_expert
from test_gezozen_engine_gpu import TOL, Tally, check, make_runner, write_folder

pytestmark = pytest.mark.gpu


def draw(seed):
    r = random.Random(seed)
    groups = r.choice([1, 1, 2, 3, 4, 7])
    width = groups * r.choice([8, 8, 16, 24, 10, 14, 32])
    eps = r.choice([1e-5, 1e-6, 3e-6])

    def rot(dim, stretched):
        dims = r.choice([2, dim - dim % 2, max(2, (dim // 2) - (dim // 2) % 2)])
        out = {"base": r.choice([50.0, 10000.0, 250000.0]), "dims": dims}
        if stretched:
            out["scaling"] = {"factor": r.choice([2.0, 8.0]), "original": r.choice([16, 64, 512]),
                              "fast": r.choice([4.0, 32.0]), "slow": r.choice([0.5, 1.0])}
        return out

    def mlp():
        if r.random() < 0.15:
            return None
        experts = r.randint(1, 16)
        m = {"kind": "moe", "expert": {"ff": r.choice([8, 12, 24, 40])},
             "router": {"experts": experts, "top": r.randint(1, min(experts, 6))}}
        if r.random() < 0.7:
            m["shared"] = {"ff": r.choice([8, 20, 48])}
        return m
    layers = []
    for _ in range(r.randint(1, 6)):
        kind = r.choice(["delta", "parallel", "parallel_2"])
        if kind == "delta":
            g = r.choice([1, 2, 3])
            mixer = {"heads": g * r.choice([1, 2, 4]), "kv_heads": g, "dim": r.choice([4, 12, 16, 32, 128]),
                     "vdim": r.choice([6, 8, 32, 72]), "conv": r.randint(1, 5)}
        else:
            g = r.choice([1, 2, 3])
            dim = r.choice([8, 12, 20, 32, 64, 128])
            left = {"heads": g * r.choice([1, 2, 4]), "kv_heads": g, "dim": dim, "vdim": r.choice([8, 12, 40, 64, 128]),
                    "scale": r.choice([0.1, 0.25, dim ** -0.5]), "rot": rot(dim, kind == "parallel_2" or r.random() < 0.3)}
            if kind == "parallel" or r.random() < 0.3:
                left["softcap"] = r.choice([2.0, 10.0, 50.0])
            if kind == "parallel_2" or r.random() < 0.3:
                left["mask"] = {"size": r.choice([1, 2, 7, 16, 40, 300])}
            rd, rh = r.choice([6, 8, 16, 48, 64]), r.randint(1, 6)
            right = {"heads": rh, "dim": rd, "vdim": r.choice([4, 10, 32, 64])}
            if kind == "parallel":
                right.update(tau=r.choice([1.0, 4.0, 16.0]), rank=r.choice([1, 3, 8, 16]))
            else:
                right.update(decay=[1.0 - 2.0 ** -r.randint(1, 11) for _ in range(rh)], rot=rot(rd, False))
            mixer = {"left": left, "right": right, "left_scale": r.choice([0.5, 1.0, 1.2]),
                     "right_scale": r.choice([0.5, 0.9, 2.0])}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp()})
    return {"architecture": "Gezozen", "vocab": r.choice([53, 128, 300]), "width": width,
            "norm": {"eps": eps, "groups": groups}, "postln_alpha": r.choice([1.0, 1.5, 2.5]), "layers": layers}


@pytest.mark.parametrize("seed", range(10))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_drawn_configuration(tmp_path, seed, dtype):
    from allpaca_b200.engine.batch import BatchEntry
    config = draw(1000 + seed)
    if dtype == "bfloat16":
        config = every_expert(config)
    weights = write_folder(tmp_path, config, seed=seed, dtype=dtype)
    r = random.Random(seed)
    page = r.choice([4, 8, 16, 64])
    seqs = {k: helpers.random_tokens(n, config["vocab"], 10 * seed + k) for k, n in enumerate([r.randint(40, 90), 1, 19])}
    want = {k: plain.forward(weights, config, t) for k, t in seqs.items()}
    runner = make_runner(tmp_path, dtype, 256, page_size=page, max_seqs=3)
    tally = Tally()
    # whole; then two requests side by side in portions of any size and single rows
    for k, toks in seqs.items():
        check(runner.step([BatchEntry(("w", k), toks, list(range(len(toks))))]), want[k], TOL[dtype], (seed, "whole", k), tally)
        runner.finish(("w", k))
    at = {0: 0, 2: 0}
    while any(at[k] < len(seqs[k]) for k in at):
        entries, rows = [], []
        for k in at:
            if at[k] < len(seqs[k]):
                n = min(r.choice([1, 1, 2, 5, 17]), len(seqs[k]) - at[k])
                entries.append(BatchEntry(k, seqs[k][at[k]:at[k] + n], list(range(n))))
                rows.append((k, at[k], n))
                at[k] += n
        logits = runner.step(entries)
        row = 0
        for k, a, n in rows:
            check(logits[row:row + n], want[k][a:a + n], TOL[dtype], (seed, "portion", k, a, n), tally)
            row += n
    tally.finish((seed, dtype))
    runner.finish(0)
    runner.finish(2)
    runner.cache.check()
