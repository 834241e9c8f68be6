"""The Gezozen decoder through the engine against the plain implementation: the stream after every layer,
whole prompts, prefill against token-by-token decoding, portions down to two tokens, batches of unequal requests
against each alone, pages and state slots that are given back and used again, long decoding across several
windows, the first tokens of a sequence, the trace runner as a user starts it, and greedy generation through
the entry point and its scheduler."""
import random

import numpy as np
import pytest
import torch

import helpers
import plain_gezozen as plain
from gezozen_configs import CONFIGS, every_expert

pytestmark = pytest.mark.gpu

TOL = {"float32": 2e-5, "bfloat16": 3e-2}
LENGTHS = {"A": [1, 2, 23, 61, 150], "B": [1, 3, 40, 97], "C": [1, 5, 50, 33]}


def write_folder(path, config, seed, dtype):
    from allpaca_b200.weights import write_model_folder
    tensors = plain.random_tensors(config, seed)
    stored = {k: v.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in tensors.items()}
    write_model_folder(str(path), config, stored)
    return tensors


def make_runner(path, dtype, max_tokens, page_size=8, graphs=True, max_seqs=4):
    from allpaca_b200.config import EngineConfig
    from allpaca_b200.engine.runner import ModelRunner
    return ModelRunner(str(path), EngineConfig(
        dtype=dtype, page_size=page_size, num_pages=-(-max_tokens // page_size), max_num_seqs=max_seqs,
        max_num_batched_tokens=max(max_tokens, max_seqs), prefill_chunk=max_tokens, use_cuda_graphs=graphs))


class Tally:
    """Row errors of one bfloat16 test.  Rounding noise has a long tail, so a test passes if no row is over three
    times the tolerance and at most one row in fifty is over it; a wrong key, window, state or page moves whole
    runs of rows by tens of per cent and fails both."""

    def __init__(self):
        self.rows = self.over = 0

    def finish(self, what):
        assert self.over <= max(1, self.rows // 50), (what, f"{self.over} of {self.rows} rows over the tolerance")


def check(got, want, tol, what, tally=None):
    """32-bit (a tolerance below 1e-3): the largest deviation of any logit against the largest plain logit.
    bfloat16: the root mean square of a row's deviations against that of the plain logits, judged by the tally."""
    got, want = got.double().cpu().numpy(), want.numpy()
    assert np.isfinite(got).all(), (what, "non-finite logits")
    if tol < 1e-3:
        err = np.abs(got - want).max(axis=-1) / np.abs(want).max()
        assert err.max() <= tol, (what, "first wrong row", int(np.argmax(err > tol)), float(err.max()))
        return
    err = np.sqrt(((got - want) ** 2).mean(axis=-1)) / np.sqrt((want ** 2).mean())
    assert err.max() <= 3 * tol, (what, "first wrong row", int(np.argmax(err > 3 * tol)), float(err.max()))
    assert tally is not None or err.max() <= tol, (what, float(err.max()))
    if tally is not None:
        tally.rows += len(err)
        tally.over += int((err > tol).sum())


@pytest.fixture(scope="module", params=[("A", "float32"), ("B", "float32"), ("C", "float32"),
                                        ("A", "bfloat16"), ("B", "bfloat16"), ("C", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    name, dtype = request.param
    config = CONFIGS[name] if dtype == "float32" else every_expert(CONFIGS[name])
    path = tmp_path_factory.mktemp(f"gezozen_{name}_{dtype}")
    weights = write_folder(path, config, seed=23 + len(name), dtype=dtype)
    seqs = {f"s{i}": helpers.random_tokens(n, config["vocab"], 250 + i) for i, n in enumerate(LENGTHS[name])}
    want = {r: plain.forward(weights, config, t) for r, t in seqs.items()}
    return name, dtype, config, path, weights, seqs, want


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_stream_after_every_layer(tmp_path, name):
    """In 32-bit, a prompt in two portions: what leaves each layer against the plain implementation's, so that a
    fault names its layer."""
    from allpaca_b200.engine.batch import BatchEntry
    config = CONFIGS[name]
    weights = write_folder(tmp_path, config, seed=5, dtype="float32")
    toks = helpers.random_tokens(45, config["vocab"], 77)
    want = []
    plain.forward(weights, config, toks, streams=want)
    runner = make_runner(tmp_path, "float32", 64, graphs=False)
    seen = []
    for block in runner.model.blocks:
        def forward(x, delta, step, cache, inner=block.forward):
            out = inner(x, delta, step, cache)
            seen.append(x.clone())
            return out
        block.forward = forward
    runner.step([BatchEntry("r", toks[:31], [])])
    runner.step([BatchEntry("r", toks[31:], [])])
    layers = len(config["layers"])
    for i in range(layers):
        got = torch.cat([seen[i], seen[layers + i]]).double().cpu()
        err = float((got - want[i]).abs().max() / want[i].abs().max())
        assert err <= 1e-5, (name, "first wrong layer", i, err)


def test_whole_prompts_and_decoding_one_by_one(case):
    from allpaca_b200.engine.batch import BatchEntry
    name, dtype, config, path, _, seqs, want = case
    runner = make_runner(path, dtype, 192)
    tally = Tally()
    for r, toks in seqs.items():
        logits = runner.step([BatchEntry(("w", r), toks, list(range(len(toks))))])
        check(logits, want[r], TOL[dtype], (name, "whole", r), tally)
        runner.finish(("w", r))
    # the longest: a short prompt, then every token alone (the window passes over decoded tokens, the state is
    # carried a hundred steps; steps are replayed as CUDA graphs from the third on)
    r, toks = max(seqs.items(), key=lambda kv: len(kv[1]))
    logits = runner.step([BatchEntry("d", toks[:3], [0, 1, 2])])
    check(logits, want[r][:3], TOL[dtype], (name, "decode head"), tally)
    for i in range(3, len(toks)):
        logits = runner.step([BatchEntry("d", toks[i:i + 1], [0])])
        check(logits, want[r][i:i + 1], TOL[dtype], (name, "decoded token", i), tally)
    runner.finish("d")
    tally.finish((name, dtype))
    assert runner.graph_replays > 0
    runner.cache.check()
    assert runner.cache.num_running() == 0


@pytest.mark.parametrize("portions", [[2], [3, 2, 7, 2, 16, 5, 2, 33, 9], [1, 1, 2, 1, 31], [64, 2, 1]])
def test_portions_cut_anywhere(case, portions):
    from allpaca_b200.engine.batch import BatchEntry
    name, dtype, config, path, _, seqs, want = case
    runner = make_runner(path, dtype, 192, page_size=16)
    tally = Tally()
    for r, toks in seqs.items():
        at = k = 0
        while at < len(toks):
            n = min(portions[k % len(portions)], len(toks) - at)
            k += 1
            logits = runner.step([BatchEntry(r, toks[at:at + n], list(range(n)))])
            check(logits, want[r][at:at + n], TOL[dtype], (name, "portion", r, at, n), tally)
            at += n
        runner.finish(r)
    tally.finish((name, dtype, portions))


def test_mixed_batches_on_a_small_pool(case):
    """Up to three live requests, portions beside single tokens, each request run twice: the pool holds what
    three hold at most, so pages and state slots change hands."""
    from allpaca_b200.engine.batch import BatchEntry
    name, dtype, config, path, _, seqs, want = case
    rng = random.Random(11)
    order = [(k, r) for k in "xy" for r in seqs]
    rng.shuffle(order)
    longest = sorted(2 * [len(t) for t in seqs.values()])[-3:]
    runner = make_runner(path, dtype, sum(-(-n // 8) * 8 for n in longest), page_size=8, max_seqs=3)
    live, at = [], {}
    tally = Tally()
    while order or live:
        while order and len(live) < 3:
            live.append(order.pop(0))
            at[live[-1]] = 0
        entries, rows, ending = [], [], []
        for key in list(live):
            toks = seqs[key[1]]
            if entries and rng.random() < 0.25:
                continue                                    # left out of this step, goes on later
            a = at[key]
            n = min(rng.choice([1, 1, 2, 3, 9, 20]), len(toks) - a) if a < len(toks) // 2 else 1
            entries.append(BatchEntry(key, toks[a:a + n], list(range(n))))
            rows.append((key, a, n))
            at[key] = a + n
            if a + n == len(toks):
                ending.append(key)
                live.remove(key)
        logits = runner.step(entries)
        row = 0
        for key, a, n in rows:
            check(logits[row:row + n], want[key[1]][a:a + n], TOL[dtype], (name, "mixed", key, a, n), tally)
            row += n
        for key in ending:
            runner.finish(key)
    tally.finish((name, dtype))
    runner.cache.check()
    assert runner.cache.num_running() == 0


def test_pages_behind_the_window_go_back(tmp_path):
    """The windowed side of a pair keeps its pages only as far back as the window; older pages go back to the pool
    while the request runs.  Free pages are poisoned, so a read of a page that was given back would show."""
    from allpaca_b200.engine.batch import BatchEntry
    config = CONFIGS["A"]                       # layer 0: window 21; layer 2: no window
    weights = write_folder(tmp_path, config, seed=3, dtype="float32")
    toks = helpers.random_tokens(120, config["vocab"], 9)
    want = plain.forward(weights, config, toks)
    runner = make_runner(tmp_path, "float32", 128, page_size=4, graphs=False, max_seqs=1)
    groups = {g.need.window: i for i, g in enumerate(runner.cache_plan)}
    assert set(groups) == {21, None}
    at = 0
    for n in [50, 3, 1, 1, 30, 2, 1, 1, 1, 30]:
        logits = runner.step([BatchEntry("r", toks[at:at + n], list(range(n)))])
        check(logits, want[at:at + n], TOL["float32"], ("window release", at, n))
        at += n
        table = runner.cache.block_table("r", groups[21])
        dead = max(0, at - 21 + 1) // 4
        assert all(p == -1 for p in table[:dead]) and all(p >= 0 for p in table[dead:]), table
        free = sorted(set(range(runner.num_pages)) - {p for p in table if p >= 0})
        runner.storages[groups[21]].pages[:, free] = float("nan")
    runner.finish("r")
    runner.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_state_slot_that_is_used_again_starts_from_zero(tmp_path, name):
    """The recurrent state and the convolution's last inputs live in a request's state slot.  With ONE slot, every
    request takes over the slot of the one before: it must start from zeros, not from what was left there."""
    from allpaca_b200.engine.batch import BatchEntry
    config = CONFIGS[name]
    weights = write_folder(tmp_path, config, seed=6, dtype="float32")
    runner = make_runner(tmp_path, "float32", 64, max_seqs=1, graphs=False)
    for k, n in enumerate([9, 1, 17, 2]):
        toks = helpers.random_tokens(n, config["vocab"], 40 + k)
        want = plain.forward(weights, config, toks)
        cut = n // 2
        rows = []
        if cut:
            rows.append(runner.step([BatchEntry(k, toks[:cut], list(range(cut)))]).clone())
        rows.append(runner.step([BatchEntry(k, toks[cut:], list(range(n - cut)))]).clone())
        check(torch.cat(rows), want, TOL["float32"], ("slot used again", k))
        runner.finish(k)


def test_batch_and_cut_change_32_bit_rows_by_rounding_only(tmp_path):
    """In 32-bit a row alone, in a batch and in a portion cut elsewhere differs by the order of a few sums at most."""
    from allpaca_b200.engine.batch import BatchEntry
    config = CONFIGS["A"]
    write_folder(tmp_path, config, seed=4, dtype="float32")
    a, b = helpers.random_tokens(70, config["vocab"], 1), helpers.random_tokens(33, config["vocab"], 2)
    runner = make_runner(tmp_path, "float32", 256, graphs=False)
    alone = runner.step([BatchEntry("a", a, list(range(70)))]).clone()
    runner.finish("a")
    first = runner.step([BatchEntry("b", b[:20], []), BatchEntry("a", a[:41], list(range(41)))]).clone()
    second = runner.step([BatchEntry("a", a[41:], list(range(29))), BatchEntry("b", b[20:], [])]).clone()
    both = torch.cat([first, second])
    assert float((both - alone).abs().max() / alone.abs().max()) <= 2e-6


def test_trace_runner_as_a_user_starts_it(tmp_path):
    config = CONFIGS["A"]
    weights = write_folder(tmp_path / "model", config, seed=21, dtype="float32")
    toks = {r: helpers.random_tokens(n, config["vocab"], 30 + n) for r, n in (("p", 45), ("q", 18), ("r", 1))}
    want = {r: plain.forward(weights, config, t).numpy() for r, t in toks.items()}
    tb = helpers.TraceBuilder()
    tb.step([("p", toks["p"][:30], [0, 29]), ("r", toks["r"], [0])], end=["r"])
    tb.step([("p", toks["p"][30:32], [0, 1]), ("q", toks["q"][:17], list(range(17)))])
    for i in range(32, 45):
        entries = [("p", toks["p"][i:i + 1], [0])]
        if i == 32:
            entries.append(("q", toks["q"][17:], [0]))
        tb.step(entries, end=(["q"] if i == 32 else []) + (["p"] if i == 44 else []))
    out = helpers.run_trace(str(tmp_path / "model"), "float32", str(tmp_path / "out"), tb.steps, 128)
    helpers.compare(out, tb, want, TOL["float32"], "trace runner")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(tmp_path, dtype):
    """LLM.generate with its scheduler: prompts cut into portions of 16, three requests on two slots, against
    greedy decoding with the plain implementation."""
    from allpaca_b200 import LLM, SamplingParams
    config = CONFIGS["B"] if dtype == "float32" else every_expert(CONFIGS["B"])
    weights = write_folder(tmp_path, config, seed=8, dtype=dtype)
    prompts = [helpers.random_tokens(n, config["vocab"], 70 + n) for n in (5, 37, 22)]
    llm = LLM(model=str(tmp_path), dtype=dtype, page_size=16, max_cache_tokens=256, max_num_seqs=2,
              max_num_batched_tokens=48, prefill_chunk=16)
    outs = llm.generate(prompts, SamplingParams.greedy_params(max_tokens=12))
    for p, o in zip(prompts, outs):
        if dtype == "float32":
            assert o.token_ids == plain.greedy(weights, config, p, 12), (p[:3], o.token_ids)
        else:
            # bfloat16: every chosen token is within the tolerance of the plain maximum
            logits = plain.forward(weights, config, p + o.token_ids)
            for i, t in enumerate(o.token_ids):
                row = logits[len(p) + i - 1]
                assert float(row.max() - row[t]) <= 2 * TOL[dtype] * float(logits.abs().max()), (i, t)


def test_generation_from_the_command_line(tmp_path):
    """``bin/allpaca generate`` on a Gezozen folder, greedy, in 32-bit: the tokens of the plain implementation."""
    import json
    import os
    import subprocess
    import sys
    config = CONFIGS["C"]
    weights = write_folder(tmp_path, config, seed=4, dtype="float32")
    prompts = [helpers.random_tokens(n, config["vocab"], 30 + n) for n in (3, 19)]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bin", "allpaca"), "generate", "--model", str(tmp_path), "--dtype", "float32",
           "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids", " ".join(map(str, prompts[1])),
           "--max-tokens", "7", "--temperature", "0", "--json"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [json.loads(line) for line in p.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 2
    for pr, out in zip(prompts, lines):
        assert out["token_ids"] == plain.greedy(weights, config, pr, 7), out
        assert out["finish_reason"] == "length" and out["prompt_tokens"] == len(pr)


def test_preempted_requests_are_computed_again(tmp_path):
    """A pool too small for three requests: the scheduler preempts one (its pages and state slot given back) and
    computes it again from position 0 later; the tokens equal the plain implementation's."""
    from allpaca_b200 import LLM, SamplingParams
    config = CONFIGS["B"]
    weights = write_folder(tmp_path, config, seed=15, dtype="float32")
    prompts = [helpers.random_tokens(n, config["vocab"], 90 + n) for n in (30, 28, 26)]
    llm = LLM(model=str(tmp_path), dtype="float32", page_size=16, max_cache_tokens=96, max_num_seqs=3,
              max_num_batched_tokens=64, prefill_chunk=32)
    outs = llm.generate(prompts, SamplingParams.greedy_params(max_tokens=10))
    assert sum(o.num_preemptions for o in outs) > 0, "the pool was meant to run out"
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.greedy(weights, config, p, 10), (p[:3], o.token_ids)
