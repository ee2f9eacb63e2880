"""Small Dikusun configurations of the tests.  Between them they vary what a configuration may vary: the order of the
three kinds of layers, layers with and without a feed-forward, layers that run with another layer's weights (an earlier
one, a later one, twice), grouped and ungrouped key/value heads, windows of one token, of a few and longer than any
prompt, no window, capped and uncapped scores, the whole unit rotating, a part of it or nothing, value heads smaller
and larger than key units, latents smaller and larger than the heads they feed, decay ranks, and an embedding scale of
one, below and above it."""


def _attention(heads, kv_heads, dim, vdim, scale, diff, window, dims, base=10000.0, softcap=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff, "softcap": softcap,
            "mask": {"size": window} if window else None, "rot": {"base": base, "dims": dims} if dims else None}


def _latent(heads, dim, vdim, q_rank, kv_rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}


def _gla(heads, dim, vdim, tau, a_rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "a_rank": a_rank}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


ATTENTION_ONLY = {
    "architecture": "Dikusun", "vocab": 211, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
    "layers": [
        {"type": "attention", "mixer": _attention(3, 3, 16, 24, 0.25, 0.2, 5, 8, softcap=20.0), "mlp": None},
        {"type": "attention", "mixer": _attention(6, 2, 8, 8, 0.35, 0.5, None, 8, base=500.0), "mlp": _dense(40, 1.0)},
        {"type": "attention", "mixer": _attention(2, 1, 24, 40, 0.2, 0.0, 1, None, softcap=5.0), "mlp": None},
    ],
}

LATENT_ONLY = {
    "architecture": "Dikusun", "vocab": 190, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 16, 8, 24, 40, 0.25), "mlp": _dense(56, 2.5)},
        {"type": "latent_attention", "mixer": _latent(5, 8, 24, 72, 16, 0.35), "mlp": None},
    ],
}

GLA_ONLY = {
    "architecture": "Dikusun", "vocab": 150, "width": 40, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.25},
    "layers": [
        {"type": "gla", "mixer": _gla(2, 24, 40, 8.0, 8), "mlp": None},
        {"type": "gla", "mixer": _gla(5, 8, 16, 1.0, 24), "mlp": _dense(72, 0.8)},
        {"type": "gla", "mixer": _gla(1, 72, 33, 32.0, 4), "mlp": None},
    ],
}

# every kind of layer; layer 0 runs with the weights of layer 3 (a later one), layers 4 and 5 with those of layer 1
ALL_KINDS = {
    "architecture": "Dikusun", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.7},
    "layers": [
        {"type": "gla", "mixer": _gla(3, 16, 32, 4.0, 12), "mlp": _dense(64, 1.2), "weights_of": 3},
        {"type": "attention", "mixer": _attention(4, 2, 16, 16, 0.25, 0.4, 23, 16, base=1e6, softcap=30.0), "mlp": _dense(80, 3.0)},
        {"type": "latent_attention", "mixer": _latent(2, 32, 48, 40, 56, 0.18), "mlp": None},
        {"type": "gla", "mixer": _gla(3, 16, 32, 4.0, 12), "mlp": _dense(64, 1.2)},
        {"type": "attention", "mixer": _attention(4, 2, 16, 16, 0.25, 0.4, 23, 16, base=1e6, softcap=30.0), "mlp": _dense(80, 3.0),
         "weights_of": 1},
        {"type": "attention", "mixer": _attention(4, 2, 16, 16, 0.25, 0.4, 23, 16, base=1e6, softcap=30.0), "mlp": _dense(80, 3.0),
         "weights_of": 1},
    ],
}

# sizes at which the bfloat16 path takes its tensor-core kernels (units and latents of 64 and 128, widths in 64s)
TENSOR_CORE_SIZES = {
    "architecture": "Dikusun", "vocab": 384, "width": 192, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 32, 64, 64, 128, 0.18), "mlp": _dense(256, 2.0)},
        {"type": "attention", "mixer": _attention(4, 2, 64, 64, 0.125, 0.3, 70, 32, base=1e5, softcap=40.0), "mlp": None},
        {"type": "gla", "mixer": _gla(2, 64, 128, 12.0, 16), "mlp": _dense(128, 2.5)},
        {"type": "latent_attention", "mixer": _latent(8, 64, 32, 128, 64, 0.125), "mlp": None},
        {"type": "attention", "mixer": _attention(2, 1, 128, 128, 0.09, 0.1, 150, 128, base=1e4), "mlp": _dense(128, 0.9)},
    ],
}

# name -> (config.json contents, seed of the random weights)
DIKUSUN = {"attention_only": (ATTENTION_ONLY, 3), "latent_only": (LATENT_ONLY, 4), "gla_only": (GLA_ONLY, 5),
           "all_kinds": (ALL_KINDS, 6), "tensor_core_sizes": (TENSOR_CORE_SIZES, 7)}
