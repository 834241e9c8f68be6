"""The Gezozen decoder without a GPU: configuration, tensor names and shapes against the plain list, what each
layer asks of the cache and of the state slots, refused configurations, the size that the tensors' shapes give,
and each mechanism of the plain implementation by hand."""
import copy
import math

import pytest
import torch

import plain_gezozen as plain
from gezozen_configs import CONFIGS


def build(config, dtype=torch.float32):
    from allpaca_b200.models import DecoderModel, resolve
    from allpaca_b200.parts import BuildEnv, Workspace
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    dev = torch.device("cpu")
    return cfg, DecoderModel(arch.spec_builder(cfg), BuildEnv(dtype, dev, Workspace(dev), page_size=8, max_seqs=2))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_names_and_shapes(name):
    _, model = build(CONFIGS[name])
    got = {n: tuple(ws.shape) for n, (ws, _, _) in model.weight_targets().items()}
    assert got == plain.tensor_shapes(CONFIGS[name])


def test_cache_plan_and_state():
    _, model = build(CONFIGS["A"])
    plan = model.cache_plan()
    # layer 0: 3 key/value heads of 24 + 40 behind a window of 21; layer 2: 2 heads of 32 + 16, no window
    assert [(g.need.outer, g.need.inner, g.need.window, g.runs) for g in plan] == \
        [((3,), (64,), 21, [0]), ((2,), (48,), None, [2])]
    # retention 3 x 16 x 8; delta 3 x 16 x 24 and two inputs of 16 + 16 + 72 channels; linear attention 5 x 8 x 12
    assert model.state_bytes() == [4 * 3 * 16 * 8, 4 * (3 * 16 * 24 + 2 * (16 + 16 + 72)), 4 * 5 * 8 * 12]
    assert not model.host_control()
    _, model = build(CONFIGS["B"])
    assert model.state_bytes()[0] == 4 * 2 * 32 * 16            # a convolution of one tap keeps no inputs
    assert [g.need.window for g in model.cache_plan()] == [None, 1]


def test_refused_configurations():
    from allpaca_b200.config import ConfigError, GezozenConfig
    base = CONFIGS["A"]

    def broken(change):
        c = copy.deepcopy(base)
        change(c)
        with pytest.raises(ConfigError):
            GezozenConfig.from_dict(c)
    broken(lambda c: c["layers"][0].update(type="parallel_3"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4))              # 6 heads on 4
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7))            # odd
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=26))           # more than the head has
    broken(lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.9, 0.9]))        # three heads
    broken(lambda c: c["layers"][2]["mixer"]["right"].pop("rank"))                     # and no tensors to read it off
    broken(lambda c: c["layers"][2]["mixer"]["right"].update(tau=0.0))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))                    # of four
    broken(lambda c: c["layers"][1]["mlp"].update(kind="dense"))
    broken(lambda c: c["norm"].update(groups=5))                                       # 64 columns
    broken(lambda c: c.pop("width"))
    c = copy.deepcopy(base)
    c["layers"][2]["mixer"]["left"].pop("kv_heads")
    assert GezozenConfig.from_dict(c).layers[2].mixer.left.kv_heads == 2              # left out: one per query head


def test_the_rank_comes_from_the_tensors(tmp_path):
    """config.json need not name the inner width of the decay's pair of products: the checkpoint's shapes do."""
    from allpaca_b200.models import load_config
    from allpaca_b200.weights import write_model_folder
    config = copy.deepcopy(CONFIGS["A"])
    tensors = {k: v.to(torch.bfloat16) for k, v in plain.random_tensors(config, 3).items()}
    del config["layers"][2]["mixer"]["right"]["rank"]
    write_model_folder(str(tmp_path), config, tensors)
    _, cfg = load_config(str(tmp_path))
    assert cfg.layers[2].mixer.right.rank == 6


def test_stretched_frequencies_by_hand():
    # 8 coordinates, base 5000, trained length 64, factor 4: index(t) = 8 ln(64 / (2 pi t)) / (2 ln 5000)
    f, mag = plain.rotary_frequencies({"base": 5000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64,
                                                                              "fast": 8.0, "slow": 1.0}})
    lo = max(math.floor(8 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(5000.0))), 0)
    hi = min(math.ceil(8 * math.log(64 / (2 * math.pi * 1.0)) / (2 * math.log(5000.0))), 7)
    assert (lo, hi) == (0, 2)
    plainf = [5000.0 ** (-2 * i / 8) for i in range(4)]
    assert f[0] == pytest.approx(plainf[0]) and f[1] == pytest.approx(plainf[1] * (0.5 / 4 + 0.5))
    assert f[2] == pytest.approx(plainf[2] / 4) and f[3] == pytest.approx(plainf[3] / 4)
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    from allpaca_b200.parts.rope import inverse_frequencies, magnitude
    sc = {"rope_type": "yarn", "factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    assert torch.allclose(inverse_frequencies(8, 5000.0, sc), f, rtol=1e-12)
    assert magnitude(sc) == pytest.approx(mag)


def test_mechanisms_by_hand():
    # norm in groups: every run has unit mean square before the weight
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    y = plain.group_norm(x, torch.tensor([1.0, 1.0, 2.0, 2.0], dtype=torch.float64), 2, 0.0)
    assert torch.allclose(y, torch.tensor([[3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0.0, 2 * 2 / math.sqrt(2.0)]],
                                          dtype=torch.float64))
    # the convolution's last tap is the row's own; nothing before the start
    c = plain.short_conv(torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64),
                         torch.tensor([[0.5, 0.0, 2.0]], dtype=torch.float64))
    silu = lambda z: z / (1 + math.exp(-z))
    assert torch.allclose(c[:, 0], torch.tensor([silu(2.0), silu(4.0), silu(6.5)], dtype=torch.float64))
    # a window of 2 shows the row and the one before it
    q = torch.ones(3, 1, 1, dtype=torch.float64)
    v = torch.tensor([[[1.0]], [[2.0]], [[4.0]]], dtype=torch.float64)
    out = plain.attend(q, torch.zeros(3, 1, 1, dtype=torch.float64), v, 1.0, None, 2)
    assert torch.allclose(out[:, 0, 0], torch.tensor([1.0, 1.5, 3.0], dtype=torch.float64))
    # the share multiplies what the expert reads
    W = {"r": torch.tensor([[0.0], [1.0]], dtype=torch.float64)}
    for e in (0, 1):
        W.update({f"m.e{e}.gate": torch.tensor([[1.0 + e]], dtype=torch.float64),
                  f"m.e{e}.up": torch.tensor([[1.0]], dtype=torch.float64),
                  f"m.e{e}.down": torch.tensor([[1.0]], dtype=torch.float64)})
    W["m.router"] = W["r"]
    h = torch.tensor([[2.0]], dtype=torch.float64)
    s = 1 / (1 + math.exp(-2.0))
    got = plain.routed_feed_forward(W, "m.", {"router": {"experts": 2, "top": 1}, "expert": {"ff": 1}}, h)
    assert float(got) == pytest.approx(silu(2.0 * s * 2.0) * (s * 2.0))
