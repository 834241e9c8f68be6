"""Prefill and decode throughput of one design beside the dense Llama decoder of equal size,
with the time of every kind of kernel in a step:

    python bench.py --design viresun|bivatar|lazolix|gezozen [--design-size small|base|wide]

Gezozen runs beside the Viresun decoder (the closest existing model: windowed attention, a recurrent mixer
with fixed-size state, routed experts) and the Llama decoder.  Lazolix runs beside two models: the Bivatar decoder reduced to its latent layers (the closest existing
mixer) and the Llama decoder.  All models have random bfloat16 weights drawn on the device, the same width, heads, head size,
feed-forward size, number of layers and vocabulary.  Timed on the device with CUDA events after
warm-up; the per-kernel table comes from a separate pass that brackets every kernel call with
events (so it includes each launch's own start and end, and is not what the step time is made of).
Prints one JSON line.
"""
from __future__ import annotations

import contextlib
import json
import statistics
import sys
import time
from typing import Dict

import torch

# name: (width, heads, kv_heads, head size, dense ff, experts, top, expert ff, window, mamba heads, mamba vdim, state)
SIZES = {
    "small": (1024, 8, 2, 128, 4096, 8, 2, 1024, 256, 16, 64, 64),
    "base": (2048, 16, 4, 128, 8192, 16, 4, 1024, 512, 32, 64, 128),
    "wide": (4096, 32, 8, 128, 14336, 32, 4, 2048, 1024, 64, 64, 128),
}
VOCAB = 32000


def viresun_config(size: str) -> dict:
    W, H, G, D, ff, E, top, eff, window, mh, mv, N = SIZES[size]
    attn = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": window},
            "q_temp": {"coef": 0.3, "every": 256}}
    mamba = {"heads": mh, "vdim": mv, "state": N, "groups": 1, "conv": 4, "norm_groups": 1}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": eff, "limit": 1.5}, "router": {"experts": E, "top": top}}
    return {"architecture": "Viresun", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": attn, "mlp": dense}, {"type": "attention", "mixer": attn, "mlp": moe},
                       {"type": "mamba2", "mixer": mamba, "mlp": dense}, {"type": "attention", "mixer": attn, "mlp": moe}]}


# name: (latent rank of keys and values, of queries, unrotated and rotated dimensions per head, value size,
#        kept first tokens of the windowed layers); widths, heads, feed-forward and window as above
LATENT_SIZES = {"small": (256, 512, 64, 32, 64, 16), "base": (512, 768, 128, 64, 128, 64),
                "wide": (512, 1536, 128, 64, 128, 64)}


def bivatar_config(size: str) -> dict:
    """Four layers: attention through a latent, windowed attention that keeps first tokens, a latent layer of its
    own, and one that reads the third layer's latent; all with the dense feed-forward."""
    W, H, G, D, ff = SIZES[size][:5]
    window = SIZES[size][8]
    R, Q, nope, rot, E, keep = LATENT_SIZES[size]
    rotation = {"dims": rot, "base": 10000.0, "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    latent = {"heads": H, "dim": nope, "rot_dim": rot, "vdim": E, "kv_rank": R, "q_rank": Q,
              "scale": (nope + rot) ** -0.5, "rot": rotation}
    attn = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
            "mask": {"size": window, "keep_first": keep}}
    dense = {"kind": "dense", "ff": ff}
    return {"architecture": "Bivatar", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
            "embedding": {"scale": 1.0},
            "layers": [{"type": "latent_attention", "mixer": latent, "mlp": dense},
                       {"type": "attention", "mixer": attn, "mlp": dense},
                       {"type": "latent_attention", "mixer": latent, "mlp": dense},
                       {"type": "latent_attention", "mixer": dict(latent, kv_from=2), "mlp": dense}]}


def lazolix_config(size: str) -> dict:
    """Four layers of latent attention without positions behind a window, with a sink: a latent of its own and the
    dense squared-ReLU feed-forward; a latent of its own and routed experts (two identity experts behind the real
    ones); two layers that read the second layer's latents, one dense and one routed."""
    W, H, G, D, ff, E, top, eff, window = SIZES[size][:9]
    R = LATENT_SIZES[size][0]
    nope, vd = LATENT_SIZES[size][2], LATENT_SIZES[size][4]
    mixer = {"heads": H, "dim": nope, "vdim": vd, "kv_rank": R, "scale": nope ** -0.5, "mask": {"size": window}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "identity": 2, "top": top}}
    return {"architecture": "Lazolix", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6},
            "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": dense},
                       {"type": "latent_attention", "mixer": mixer, "mlp": moe},
                       {"type": "latent_attention", "mixer": dict(mixer, kv_from=1), "mlp": dense},
                       {"type": "latent_attention", "mixer": dict(mixer, kv_from=1), "mlp": moe}]}


def gezozen_config(size: str) -> dict:
    """Four layers, all with routed experts (sigmoid scores on the experts' inputs) and a gated shared expert: a
    gated delta rule; softmax attention (soft cap) beside gated linear attention; softmax attention behind a window
    with stretched rotation beside retention; a gated delta rule."""
    W, H, G, D, ff, E, top, eff, window = SIZES[size][:9]
    delta = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "conv": 4}
    half = max(H // 2, 1)
    pair = {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "softcap": 50.0,
                     "rot": {"base": 250000.0, "dims": D // 2}},
            "right": {"heads": half, "dim": D, "vdim": D, "tau": 16.0, "rank": 64}, "left_scale": 1.0, "right_scale": 0.5}
    pair2 = {"left": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": window},
                      "rot": {"base": 10000.0, "dims": D // 2,
                              "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
             "right": {"heads": half, "dim": D, "vdim": D, "decay": [1.0 - 2.0 ** (-5 - (i % 6)) for i in range(half)],
                       "rot": {"base": 10000.0, "dims": D}}, "left_scale": 1.0, "right_scale": 0.5}
    moe = {"kind": "moe", "expert": {"ff": eff}, "router": {"experts": E, "top": top}, "shared": {"ff": eff}}
    return {"architecture": "Gezozen", "vocab": VOCAB, "width": W, "norm": {"eps": 1e-6, "groups": 4},
            "postln_alpha": 2.0,
            "layers": [{"type": "delta", "mixer": delta, "mlp": moe}, {"type": "parallel", "mixer": pair, "mlp": moe},
                       {"type": "parallel_2", "mixer": pair2, "mlp": moe}, {"type": "delta", "mixer": delta, "mlp": moe}]}


def bivatar_latent_config(size: str) -> dict:
    """The Bivatar decoder with latent layers only (the windowed layer left out): what Lazolix runs beside."""
    raw = bivatar_config(size)
    L = raw["layers"]
    raw["layers"] = [L[0], L[2], L[3], dict(L[3])]
    raw["layers"][2] = dict(L[3], mixer=dict(L[3]["mixer"], kv_from=1))
    raw["layers"][3] = dict(L[3], mixer=dict(L[3]["mixer"], kv_from=1))
    return raw


DESIGNS = {
    "gezozen": (gezozen_config, "norm after the gated sum; gated delta rule, softmax attention beside gated linear "
                                "attention, windowed softmax attention beside retention, gated delta rule; routed "
                                "experts with a gated shared expert in every layer"),
    "lazolix": (lazolix_config, "latent attention without positions behind a window with a sink, token shift, Dynamic "
                                "Tanh norms, depth-weighted average: own latent + squared-ReLU, own latent + routed "
                                "(2 identity experts), second layer's latent + squared-ReLU, second layer's latent + "
                                "routed"),
    "viresun": (viresun_config, "attention+dense, attention+routed, mamba2+dense, attention+routed"),
    "bivatar": (bivatar_config, "latent attention, windowed attention with kept first tokens, latent attention, "
                                "latent attention on the third layer's latent; dense feed-forwards"),
}


def llama_config(size: str) -> dict:
    W, H, G, D, ff = SIZES[size][:5]
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 4, "hidden_size": W,
            "num_attention_heads": H, "num_key_value_heads": G, "head_dim": D, "intermediate_size": ff,
            "vocab_size": VOCAB, "rope_theta": 500000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 8192}


@contextlib.contextmanager
def kernel_times(table: Dict[str, float]):
    """Every kernel call bracketed by events and a synchronisation; milliseconds summed by name."""
    from allpaca_b200 import ops
    from allpaca_b200.ops import library, mixers, recurrent, routed, stream
    plain = library.call

    def timed(lib, name, *args):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        plain(lib, name, *args)
        b.record()
        b.synchronize()
        table[name] = table.get(name, 0.0) + a.elapsed_time(b)
    mods = (ops, mixers, recurrent, routed, stream, library)
    for m in mods:
        m.call = timed
    try:
        yield
    finally:
        for m in mods:
            m.call = plain


class DesignBench:
    def __init__(self, raw: dict, context: int, prefill: int, batch: int, seed: int = 2):
        from allpaca_b200.config import EngineConfig
        from allpaca_b200.engine.runner import ModelRunner
        from allpaca_b200.parts import BuildEnv, Workspace
        from allpaca_b200.weights.random_model import random_model_on_device
        self.device = torch.device("cuda:0")
        torch.cuda.set_device(self.device)
        self.context, self.prefill, self.batch = context, prefill, batch
        engine = EngineConfig(dtype="bfloat16", page_size=16, max_cache_tokens=batch * (context + 16) + prefill + 64,
                              max_num_seqs=batch, max_num_batched_tokens=max(prefill, batch), prefill_chunk=prefill,
                              max_model_len=max(context, prefill) + 16, seed=seed)
        engine.validate()
        env = BuildEnv(dtype=engine.dtype, device=self.device, workspace=Workspace(self.device), page_size=16,
                       max_seqs=batch)
        self.cfg, model = random_model_on_device(raw, seed, env)
        for block in model.blocks:                       # a distance bias a trained model could have
            if getattr(block.mixer, "r1", None) is not None and getattr(block.mixer, "r2", None) is not None:
                block.mixer.r1.fill_(1.0)
                block.mixer.r2.fill_(0.25)
        self.runner = ModelRunner(None, engine, model=model, model_config=self.cfg)
        self.runner.workspace = env.workspace
        self.gen = torch.Generator().manual_seed(seed)
        self.vocab = model.spec.vocab_size

    def tokens(self, n):
        return torch.randint(0, self.vocab, (n,), generator=self.gen).tolist()

    def prefill_ms(self, table=None):
        from allpaca_b200.engine.batch import BatchEntry
        times = []
        for i in range(2 if table is not None else 6):
            prompt = self.tokens(self.prefill)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            if table is not None and i == 1:
                with kernel_times(table):
                    self.runner.step([BatchEntry(("p", i), prompt, [self.prefill - 1])])
            else:
                self.runner.step([BatchEntry(("p", i), prompt, [self.prefill - 1])])
            b.record()
            torch.cuda.synchronize()
            self.runner.finish(("p", i))
            times.append(a.elapsed_time(b))
        return min(times[1:]), statistics.median(times[1:])

    def decode_ms(self, steps: int, warmup: int, table=None):
        """Requests that hold ``context - steps - warmup - 1`` tokens of synthetic (zero) cache and state,
        then one row each per step, next tokens chosen on the GPU."""
        from allpaca_b200 import ops
        from allpaca_b200.engine.batch import BatchEntry
        runner = self.runner
        held = self.context - steps - warmup - 4
        ids = [("d", i) for i in range(self.batch)]
        for rid in ids:
            runner.cache.begin(rid)
            runner.cache.append(rid, held)
            if runner.cache.has_windows():
                runner.cache.release_passed(rid)
        out = torch.randint(0, self.vocab, (self.batch,), generator=self.gen).to(torch.int32).to(self.device)
        entries = [BatchEntry(rid, [0], [0]) for rid in ids]

        def one():
            ops.argmax(runner.step(entries, device_tokens=out), out)
        for _ in range(warmup):
            one()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            one()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        if table is not None:
            graphs, runner.engine.use_cuda_graphs = runner.engine.use_cuda_graphs, False
            with kernel_times(table):
                one()
            runner.engine.use_cuda_graphs = graphs
        for rid in ids:
            runner.finish(rid)
        return ms

    def close(self):
        self.runner = None
        import gc
        gc.collect()
        torch.cuda.empty_cache()


def run(design: str, size: str, steps: int, warmup: int, batch: int, context: int, prefill: int, peaks: dict,
        sampler) -> dict:
    if design not in DESIGNS:
        raise SystemExit(f"bench.py: no design named {design!r} (known: {', '.join(sorted(DESIGNS))})")
    from allpaca_b200 import ops
    from allpaca_b200.ops import library
    make_config, layers = DESIGNS[design]
    sizes = dict(zip(("width", "heads", "kv_heads", "head_dim", "ff", "experts", "top", "expert_ff", "window",
                      "mamba_heads", "mamba_vdim", "state"), SIZES[size]))
    others = [("llama", llama_config(size))]
    if design == "lazolix":
        sizes = {k: v for k, v in sizes.items() if k in ("width", "heads", "ff", "experts", "top", "expert_ff", "window")}
        R, _, nope, _, vd, _ = LATENT_SIZES[size]
        sizes.update({"kv_rank": R, "dim": nope, "vdim": vd, "identity": 2})
        others.insert(0, ("bivatar_latent", bivatar_latent_config(size)))
    if design == "gezozen":
        sizes = {k: v for k, v in sizes.items() if k in ("width", "heads", "kv_heads", "head_dim", "experts", "top",
                                                         "expert_ff", "window")}
        sizes.update({"linear_heads": max(sizes["heads"] // 2, 1), "shared_ff": sizes["expert_ff"], "conv": 4,
                      "decay_rank": 64, "norm_groups": 4})
        others.insert(0, ("viresun", viresun_config(size)))
    if design == "bivatar":
        sizes = {k: v for k, v in sizes.items() if k in ("width", "heads", "kv_heads", "head_dim", "ff", "window")}
        sizes.update(zip(("kv_rank", "q_rank", "dim", "rot_dim", "vdim", "keep_first"), LATENT_SIZES[size]))
    out = {"metric": f"decode tok/s ({design} {size}, bf16)", "unit": "tok/s", "n_gpus": 1, "steps": steps,
           "warmup": warmup, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
           "config": {"design": design, "size": size, "global_batch": batch, "seq_len": context,
                      "prefill_tokens": prefill, "sizes": sizes,
                      "layers": layers + "; beside " + " and ".join(f"4 {n} layers" for n, _ in others),
                      "weights": "random N(0,0.02)", "peaks": peaks["source"]}}
    sampler.start()
    for name, raw in [(design, make_config(size))] + others:
        t0 = time.time()
        wb = DesignBench(raw, context, prefill, batch)
        print(f"[bench] {name} {size} ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        launches0 = library.launch_count()
        dms = wb.decode_ms(steps, warmup)
        launches = library.launch_count() - launches0
        best, median = wb.prefill_ms()
        ptab, dtab = {}, {}
        wb.prefill_ms(ptab)
        wb.decode_ms(8, 3, dtab)
        out[name] = {"decode_tok_s": round(batch / (dms / 1e3), 1), "decode_ms_per_step": round(dms, 4),
                     "prefill_tok_s": round(prefill / (best / 1e3), 1), "prefill_ms": round(best, 3),
                     "prefill_median_ms": round(median, 3),
                     "prefill_kernels_ms": {k: round(v, 4) for k, v in sorted(ptab.items(), key=lambda kv: -kv[1])},
                     "decode_kernels_ms": {k: round(v, 4) for k, v in sorted(dtab.items(), key=lambda kv: -kv[1])}}
        if name == design:
            out["value"], out["ms_per_step"], out["gpu_launches"] = out[name]["decode_tok_s"], round(dms, 4), launches
        ops.check_kernel_status()
        wb.close()
    out["clocks"] = sampler.stop()
    return out
