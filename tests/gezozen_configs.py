"""Small Gezozen configurations for the tests.  Between them every size differs, sizes that are often equal are
not (key and value size, heads of the two sides of a pair, query/key heads and value heads of the delta rule), and
what a configuration may leave out is left out once (the window, the soft cap, the stretched rotation, the shared
expert, the feed-forward, norm groups)."""


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def left(heads, kv_heads, dim, vdim, scale, rotation, softcap=None, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation}
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window}
    return m


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def retention(heads, dim, vdim, decay, rotation):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rotation}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def pair(kind, l, r, ls, rs, mlp):
    return {"type": kind, "mixer": {"left": l, "right": r, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


# a pair first (the first layer reads the embedding itself), key 24 against value 40, 6 query heads on 3, a window of
# 21 that is no multiple of a page, rotation of 8 of 24 coordinates, three fixed decays; a delta rule with 3 value
# heads on one query/key head and a convolution of 3; a pair with soft cap whose feed-forward has no shared expert
GEZOZEN_A = {
    "architecture": "Gezozen", "vocab": 211, "width": 64, "norm": {"eps": 1e-5, "groups": 2}, "postln_alpha": 1.5,
    "layers": [
        pair("parallel_2", left(6, 3, 24, 40, 0.2, rot(5000.0, 8, (4.0, 64, 8.0, 1.0)), window=21),
             retention(3, 16, 8, [0.9, 0.97, 0.995], rot(300.0, 16)), 0.7, 1.1, moe(5, 2, 24, shared=40)),
        {"type": "delta", "mixer": delta(3, 1, 16, 24, 3), "mlp": moe(4, 1, 32, shared=16)},
        pair("parallel", left(2, 2, 32, 16, 0.18, rot(90000.0, 32), softcap=3.0), gla(5, 8, 12, 4.0, 6), 1.3, 0.4,
             moe(7, 3, 16)),
    ],
}
# a delta rule first with equal head counts and a convolution of ONE tap (no inputs kept), one norm group, a layer
# without a feed-forward, a window of one (a row sees itself), a soft cap on the windowed side too, a rotation
# without stretching behind a window, every expert chosen
GEZOZEN_B = {
    "architecture": "Gezozen", "vocab": 320, "width": 96, "norm": {"eps": 1e-6, "groups": 1}, "postln_alpha": 1.0,
    "layers": [
        {"type": "delta", "mixer": delta(2, 2, 32, 16, 1), "mlp": moe(3, 3, 40, shared=24)},
        pair("parallel", left(4, 1, 16, 24, 0.3, rot(10000.0, 4, (8.0, 32, 4.0, 0.5))), gla(2, 40, 24, 16.0, 3), 1.0, 1.0,
             None),
        pair("parallel_2", left(3, 3, 8, 8, 0.4, rot(1000.0, 8), softcap=5.0, window=1),
             retention(1, 64, 32, [0.99], rot(10000.0, 2)), 0.5, 2.0, moe(2, 1, 48, shared=8)),
        {"type": "delta", "mixer": delta(4, 2, 8, 40, 5), "mlp": None},
    ],
}
# a width that is no multiple of 8 (no tensor-core product) in three norm groups, head sizes 20 and 12, an odd
# vocabulary, a window wider than any test sequence, a rank of one, one expert of one
GEZOZEN_C = {
    "architecture": "Gezozen", "vocab": 97, "width": 42, "norm": {"eps": 3e-6, "groups": 3}, "postln_alpha": 3.0,
    "layers": [
        pair("parallel", left(3, 1, 20, 12, 0.25, rot(777.0, 6), softcap=20.0), gla(1, 12, 20, 2.0, 1), 0.9, 0.8,
             moe(1, 1, 20, shared=12)),
        pair("parallel_2", left(2, 1, 12, 20, 0.3, rot(50.0, 12, (2.0, 16, 2.0, 1.0)), window=400),
             retention(2, 6, 10, [0.5, 0.999], rot(20.0, 4)), 1.0, 1.0, moe(6, 2, 8)),
        {"type": "delta", "mixer": delta(2, 1, 12, 6, 2), "mlp": moe(3, 2, 12, shared=20)},
    ],
}
CONFIGS = {"A": GEZOZEN_A, "B": GEZOZEN_B, "C": GEZOZEN_C}


def every_expert(config):
    """The same configuration with every expert chosen: in bfloat16 a row's rounding can swap two experts with
    close scores, which is no fault and moves the row by far more than rounding does."""
    import copy
    c = copy.deepcopy(config)
    for L in c["layers"]:
        if L["mlp"]:
            L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
    return c
