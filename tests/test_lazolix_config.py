"""The Lazolix configuration and model description without a GPU: tensor names and shapes against the
plain list, the cache plan (latents shared between layers, pages kept for the widest reader), the
state a request carries, refused configurations, and the plain implementation's mechanisms on cases
small enough to work out by hand."""
import copy

import pytest
import torch

import plain_lazolix
from lazolix_configs import CONFIGS, ONE_LAYER

from allpaca_b200.config import ConfigError
from allpaca_b200.models import DecoderModel, known_architectures, resolve
from allpaca_b200.parts import BuildEnv, PartError, PartSpec, Workspace, build as build_part, registered


def build(config, dtype=torch.float32):
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    env = BuildEnv(dtype=dtype, device=torch.device("cpu"), workspace=Workspace(torch.device("cpu")), page_size=8)
    return cfg, DecoderModel(arch.spec_builder(cfg), env)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    _, model = build(CONFIGS[name])
    got = {n: tuple(ws.shape) for n, (ws, _, _) in model.weight_targets().items() if n != "head"}
    assert got == plain_lazolix.tensor_shapes(CONFIGS[name])
    assert model.weight_targets()["head"][0].optional and model.spec.tie_word_embeddings


def test_the_design_is_registered_beside_the_others():
    assert "Lazolix" in known_architectures()
    assert {"token_shift", "depth_average"} <= set(registered("stream"))
    assert "dynamic_tanh" in registered("norm") and "dense_act" in registered("feed_forward")


def test_cache_plan_keeps_pages_for_the_widest_reader():
    cfg, model = build(CONFIGS["A"])
    needs = [(g.need.outer, g.need.inner, g.need.window, g.runs) for g in model.cache_plan()]
    # layer 0 (window 21) is read by layer 1 (window 33); layer 2 and its reader both have 5
    assert needs == [((), (48,), 33, [0]), ((), (40,), 5, [2])]
    assert [(r.layer, r.cache_from) for r in model.spec.order] == [(0, None), (1, 0), (2, None), (3, 2)]
    assert [cfg.cache_window(i) for i in (0, 2)] == [33, 5]
    # a layer without a window, or read by one: nothing goes back
    cfg_b, model_b = build(CONFIGS["B"])
    assert [g.need.window for g in model_b.cache_plan()] == [None, 12]
    assert not model.host_control()


def test_every_layer_carries_the_previous_normed_row():
    _, model = build(CONFIGS["C"])
    assert model.state_bytes() == [4 * 42] * 3
    _, one = build(ONE_LAYER)
    assert one.state_bytes() == [4 * 32]


def test_refused_configurations():
    arch = resolve(CONFIGS["A"])

    def broken(change):
        c = copy.deepcopy(CONFIGS["A"])
        change(c)
        with pytest.raises(ConfigError):
            arch.config_class.from_dict(c)
    broken(lambda c: c["layers"][1]["mixer"].update(kv_from=1))            # itself
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=1))            # a layer that reads another's
    broken(lambda c: c["layers"][1]["mixer"].update(kv_rank=40))           # another latent width than its source
    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="gated"))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=9))        # more than there are
    broken(lambda c: c["norm"].update(eps=0))
    broken(lambda c: c.update(layers=[]))
    broken(lambda c: c["layers"][0]["mixer"].pop("scale"))
    env = BuildEnv(dtype=torch.float32, device=torch.device("cpu"), workspace=Workspace(torch.device("cpu")))
    with pytest.raises(PartError):                                          # pages given back before the window ends
        build_part("mixer", PartSpec("latent_attention", {
            "hidden_size": 8, "num_heads": 1, "head_dim": 4, "rot_dim": 0, "value_dim": 4, "kv_rank": 4, "scale": 1.0,
            "norm_eps": 1e-5, "window": 9, "cache_window": 5}), env)
    with pytest.raises(PartError):
        build_part("stream", PartSpec("depth_average", {"hidden_size": 8, "index": 3, "count": 3}), env)


def test_token_shift_by_hand():
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 0.0]], dtype=torch.float64)
    out = plain_lazolix.token_shift(h, torch.tensor([0.5, 1.0], dtype=torch.float64))
    # column 0 moves half way to the row before, column 1 all the way; the row before row 0 is zero
    assert out.tolist() == [[0.5, 0.0], [2.0, 2.0], [4.0, 6.0]]


def test_sink_and_window_by_hand():
    """One head, keys and values equal to the latent: with all scores zero a row's weights are
    1 / (keys in its window + exp(sink))."""
    T = 5
    latent = torch.eye(T, dtype=torch.float64)
    q = torch.zeros(T, 1, T, dtype=torch.float64)
    ident = torch.eye(T, dtype=torch.float64)
    sink = torch.tensor([0.0], dtype=torch.float64)                         # counts as one more key
    out = plain_lazolix.windowed_sink_attention(q, latent, ident, ident, sink, 1.0, window=2)[:, 0]
    assert torch.allclose(out[0], torch.tensor([0.5, 0, 0, 0, 0], dtype=torch.float64))
    assert torch.allclose(out[3], torch.tensor([0, 0, 1 / 3, 1 / 3, 0], dtype=torch.float64))
    none = plain_lazolix.windowed_sink_attention(q, latent, ident, ident, sink, 1.0, window=None)[:, 0]
    assert torch.allclose(none[3], torch.tensor([0.2, 0.2, 0.2, 0.2, 0], dtype=torch.float64))


def test_routing_by_hand():
    """The correction steers the choice, not the shares; identity experts pass the row on."""
    h = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    router = torch.tensor([[0.0, 0.0], [1.0, 0.0], [2.0, 0.0]], dtype=torch.float64)
    s = torch.softmax(torch.tensor([0.0, 1.0, 2.0], dtype=torch.float64), 0)
    chosen, share = plain_lazolix.route(h, router, torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64), 2)
    assert sorted(chosen[0].tolist()) == [0, 2]                             # 0 is lifted over 1 by its correction
    got = dict(zip(chosen[0].tolist(), share[0].tolist()))
    assert abs(got[0] - float(s[0] / (s[0] + s[2]))) < 1e-12 and abs(got[2] - float(s[2] / (s[0] + s[2]))) < 1e-12
    w = {"m.router": router[:2], "m.correction": torch.zeros(2, dtype=torch.float64)}
    out = plain_lazolix.routed_feed_forward(h, w, "m.", experts=0, top=2)  # two identity experts, shares sum to one
    assert torch.allclose(out, h)


def test_depth_average_by_hand():
    a, b = torch.ones(1, 2, dtype=torch.float64), 2 * torch.ones(1, 2, dtype=torch.float64)
    out = plain_lazolix.depth_average([a, b], torch.tensor([0.5, -1.0], dtype=torch.float64))
    assert out.tolist() == [[-1.5, -1.5]]


def test_random_model_folder_from_the_command_line(tmp_path):
    """``allpaca init-random --config`` writes a Lazolix folder the engine's reader accepts: every tensor the
    description names and no other (a layer that reads another's latents has no down-projection to them, identity
    experts have no tensors, a layer without a feed-forward has no second norm)."""
    import json
    from allpaca_b200 import cli
    from allpaca_b200.models import load_config
    from allpaca_b200.weights.safetensors_io import Checkpoint
    src = tmp_path / "config.json"
    src.write_text(json.dumps(CONFIGS["A"]))
    assert cli.main(["init-random", "--config", str(src), "--seed", "3", "--out", str(tmp_path / "m"),
                     "--dtype", "bfloat16"]) == 0
    arch, cfg = load_config(str(tmp_path / "m"))
    assert arch.name == "Lazolix" and cfg.torch_dtype == "bfloat16" and len(cfg.layers) == 4
    ckpt = Checkpoint(str(tmp_path / "m"))
    shapes = plain_lazolix.tensor_shapes(CONFIGS["A"])
    assert set(ckpt.names()) == set(shapes)
    assert "l1.mix.dkv" not in shapes and "l2.norm2" not in shapes and "l1.mlp.e6.gate" not in shapes
    assert tuple(ckpt.tensor("l0.mix.dkv").shape) == (48, 64) and tuple(ckpt.tensor("l1.mlp.router").shape) == (8, 64)
    assert tuple(ckpt.tensor("l3.dwa").shape) == (5,) and tuple(ckpt.tensor("final.norm.alpha").shape) == ()
