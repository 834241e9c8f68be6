"""Lazolix configurations drawn at random (number and order of layers, head counts and sizes, latents that
are and are not multiples of 8 and are shared by several layers, windows from one token to longer than the
prompt, dense, routed and absent feed-forwards, numbers of real and identity experts, page sizes) through the
engine in 32-bit and in bfloat16 against the plain implementation: the whole prompt in one step, then portions
beside another request's decoding, then the last tokens one by one."""
import random

import numpy as np
import pytest
import torch

import helpers
import plain_lazolix
from test_lazolix_engine_gpu import write_folder

pytestmark = pytest.mark.gpu
# 32-bit: three times what rounding alone does to the drawn stack (the plain implementation in 32-bit against
# itself in 64-bit), at least 2e-5 of the largest logit; this run pins every branch.  bfloat16: the root mean square
# of a row's deviations against that of the logits; the median row within the tolerance and no row beyond five
# times it (a router whose two candidates lie within rounding of one another or a sharp softmax shows a few times the usual error in single
# rows; a wrong key, window, latent, state or page moves most rows by tens of per cent).
FLOOR32 = 2e-5
TOL16 = 3e-2


def draw(seed):
    rnd = random.Random(seed)
    width = rnd.choice([8 * rnd.randrange(6, 40), 8 * rnd.randrange(6, 40), rnd.randrange(40, 200)])
    layers, latents = [], []
    for i in range(rnd.choice([1, 2, 3, 4, 5, 7])):
        roll = rnd.random()
        if roll < 0.4:
            mlp = {"kind": "dense", "ff": rnd.choice([8 * rnd.randrange(6, 50), rnd.randrange(30, 200)])}
        elif roll < 0.85:
            experts, identity = rnd.choice([1, 2, 3, 5, 8, 11, 20]), rnd.choice([0, 0, 1, 2, 4])
            router = {"experts": experts, "top": rnd.randrange(1, min(experts + identity, 6) + 1)}
            if identity or rnd.random() < 0.5:
                router["identity"] = identity
            mlp = {"kind": "moe", "expert": {"ff": rnd.choice([8 * rnd.randrange(2, 20), rnd.randrange(10, 90)])},
                   "router": router}
        else:
            mlp = None
        src = rnd.choice(latents) if latents and rnd.random() < 0.5 else None
        if src is None:
            kv_rank = rnd.choice([8 * rnd.randrange(2, 12), 8 * rnd.randrange(12, 40), rnd.randrange(10, 150)])
            latents.append(i)
        else:
            kv_rank = layers[src]["mixer"]["kv_rank"]
        dim = rnd.choice([8, 16, 24, 32, 64, 20, 128, 96])
        mixer = {"heads": rnd.choice([1, 2, 3, 4, 6, 8, 12, 17]), "dim": dim,
                 "vdim": rnd.choice([8, 16, 40, 64, 80, 128, 12]), "kv_rank": kv_rank,
                 "scale": round(dim ** -0.5 * rnd.choice([1.0, 2.0]), 4),
                 "mask": {"size": rnd.choice([1, 2, 3, 16, 31, 64, 65, 100, 1000])}}
        if src is not None:
            mixer["kv_from"] = src
        layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
    config = {"architecture": "Lazolix", "vocab": rnd.choice([130, 257, 300, 511]), "width": width,
              "norm": {"eps": rnd.choice([1e-5, 1e-6, 1e-3])}, "layers": layers}
    return config, rnd.choice([4, 8, 16, 32, 64]), rnd.choice([70, 150, 333])


@pytest.mark.parametrize("seed", [2, 13, 27, 40, 59, 66, 73, 88, 105, 117, 121, 134])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration(tmp_path, seed, dtype):
    from allpaca_b200 import ops
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.batch import BatchEntry
    from allpaca_b200.engine.runner import ModelRunner
    config, page, n = draw(seed)
    weights = write_folder(tmp_path / "m", config, seed, dtype)
    toks = helpers.random_tokens(n, config["vocab"], seed)
    plain = plain_lazolix.forward(config, weights, toks).numpy()
    rounding = np.abs(plain_lazolix.forward(config, weights, toks, dtype=torch.float32).numpy() - plain).max()
    rounding /= np.abs(plain).max()
    tol = max(FLOOR32, 3.0 * rounding)
    runner = ModelRunner(str(tmp_path / "m"), EngineConfig(dtype=dtype, page_size=page, max_cache_tokens=2048,
                                                           max_num_seqs=4, max_num_batched_tokens=512))
    errors = []

    def compare(got, rows, what):
        want = plain[rows]
        assert np.isfinite(got).all(), (config, what)
        if dtype == "float32":
            e = np.abs(got - want).max() / np.abs(plain).max()
            assert e < tol, (config, what, float(e), tol)
        else:
            errors.extend((np.sqrt(((got - want) ** 2).mean(axis=-1)) / np.sqrt((plain ** 2).mean())).tolist())
    want = sorted({0, 1, n // 2, n - 2, n - 1})
    compare(runner.step([BatchEntry("w", toks, want)]).double().cpu().numpy(), want, "whole")
    runner.finish("w")
    at = 0
    runner.step([BatchEntry("o", toks[:9], [])])
    for k, c in enumerate([n // 3, 2, n - 20 - n // 3 - 2]):
        out = runner.step([BatchEntry("o", toks[9 + k:10 + k], [0]), BatchEntry("p", toks[at:at + c], [c - 1])])
        out = out.double().cpu().numpy()
        compare(out[:1], [9 + k], ("the decoding request", k))
        compare(out[1:], [at + c - 1], ("portion", at, c))
        at += c
    while at < n:
        compare(runner.step([BatchEntry("p", toks[at:at + 1], [0])]).double().cpu().numpy(), [at], ("decoded", at))
        at += 1
    ops.check_kernel_status()
    if dtype == "bfloat16":
        assert float(np.median(errors)) <= TOL16, (config, page, n, float(np.median(errors)))
        assert max(errors) <= 5 * TOL16, (config, page, n, max(errors))
