"""Small Lazolix configurations for the tests.  Between them every size differs, sizes that are often
equal are not (key and value size, latent and width, the windows of a layer and of the layer that reads its
latents, heads of layers that share latents), and the branches a configuration may leave out are left out
once (the window, identity experts, the feed-forward)."""


def mixer(heads, dim, vdim, kv_rank, scale, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def layer(m, mlp):
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


# 3 heads of 24 with values of 40 on a latent of 48 behind a window of 21 (no multiple of a page); layer 1 reads
# layer 0's latents with 5 heads of other sizes through a LARGER window (the pages must stay for it); layer 2
# keeps a latent of another width behind a window of 5 and has no feed-forward; layer 3 reads it with one
# expert chosen of five and no identity experts
LAZOLIX_A = {
    "architecture": "Lazolix", "vocab": 211, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer(mixer(3, 24, 40, 48, 0.17, window=21), dense(88)),
        layer(mixer(5, 8, 16, 48, 0.3, window=33, kv_from=0), moe(6, 2, 3, 24)),
        layer(mixer(2, 32, 24, 40, 0.15, window=5), None),
        layer(mixer(4, 16, 8, 40, 0.25, window=5, kv_from=2), moe(5, 0, 1, 40)),
    ],
}
# 9 heads (more than 8 share the one latent), a layer without a window whose latents a windowed layer reads (no
# page may go back), a window that never cuts, every router output chosen (3 experts and one identity expert,
# top 4), routed layers first and dense last
LAZOLIX_B = {
    "architecture": "Lazolix", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        layer(mixer(9, 16, 24, 80, 0.2), moe(3, 1, 4, 48)),
        layer(mixer(2, 64, 32, 80, 0.125, window=400, kv_from=0), moe(7, 3, 2, 16)),
        layer(mixer(4, 32, 32, 64, 0.2, window=12), dense(192)),
    ],
}
# a width that is no multiple of 4 (no vector loads, no tensor-core product), head sizes 20 and 12, a window of
# ONE (a row sees itself and the sink), a latent of 20, a single head, an odd vocabulary, more identity experts
# than real ones
LAZOLIX_C = {
    "architecture": "Lazolix", "vocab": 97, "width": 42, "norm": {"eps": 3e-6},
    "layers": [
        layer(mixer(1, 12, 20, 20, 0.4, window=1), dense(52)),
        layer(mixer(3, 20, 12, 28, 0.4, window=7), moe(2, 3, 2, 36)),
        layer(mixer(2, 10, 14, 28, 0.35, window=4, kv_from=1), None),
    ],
}
# a latent wider than the tensor-core attention kernel takes in the latent space (136): prompt portions in bfloat16
# run on keys and values formed per head, single rows in the latent space; a second layer reads the same latents
# through another window with head sizes the per-head kernel does not take (no multiple of 8)
LAZOLIX_D = {
    "architecture": "Lazolix", "vocab": 128, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer(mixer(3, 24, 40, 136, 0.17, window=30), moe(4, 1, 2, 32)),
        layer(mixer(5, 40, 8, 136, 0.14, window=19, kv_from=0), dense(40)),
        layer(mixer(2, 20, 12, 136, 0.2, window=64, kv_from=0), None),
    ],
}
ONE_LAYER = {
    "architecture": "Lazolix", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
    "layers": [layer(mixer(2, 8, 8, 16, 0.3, window=9), dense(40))],
}
CONFIGS = {"A": LAZOLIX_A, "B": LAZOLIX_B, "C": LAZOLIX_C, "D": LAZOLIX_D}
