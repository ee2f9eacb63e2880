"""Small Gefarax configurations of the tests.  Between them they vary what a configuration may vary: layers with and
without a feed-forward, value heads smaller than, equal to and larger than key heads, one kv head, as many kv heads as
heads, the whole head rotating or a part of it or nothing, stretched and plain frequencies, a router that takes one
expert, some, or all of them, with and without a shared expert, a loop that starts at the first layer, one in the
middle, and no loop."""


def _rot(base, dims, scaling=None):
    return {"base": base, "dims": dims, "scaling": scaling}


def _mlp(experts, top, scale, ff, limit, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff, "limit": limit},
            "shared": shared}


LOOP_FROM_START = {
    "architecture": "Gefarax", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 16, "scale": 0.2,
                   "rot": _rot(10000.0, 16, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0})},
         "mlp": _mlp(4, 2, 1.5, 48, 1.0, {"ff": 32, "limit": 2.5})},
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.25, "rot": _rot(500.0, 16)},
         "mlp": None},
        {"type": "attention",
         "mixer": {"heads": 6, "kv_heads": 1, "dim": 24, "vdim": 40, "scale": 0.3, "rot": None},
         "mlp": _mlp(5, 1, 0.7, 24, 0.8)},
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

NO_LOOP = {
    "architecture": "Gefarax", "vocab": 257, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 64, "vdim": 64, "scale": 0.125,
                   "rot": _rot(100000.0, 32, {"factor": 16.0, "original": 128, "fast": 16.0, "slow": 1.0})},
         "mlp": _mlp(3, 3, 1.0, 40, 3.0, {"ff": 56, "limit": 1.2})},
        {"type": "attention",
         "mixer": {"heads": 8, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.4,
                   "rot": _rot(3000.0, 8, {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 0.5})},
         "mlp": _mlp(6, 2, 2.0, 32, 1.5)},
    ],
    "loop": None,
}

LOOP_IN_THE_MIDDLE = {
    "architecture": "Gefarax", "vocab": 190, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.3, "rot": _rot(20000.0, 16, None)},
         "mlp": _mlp(4, 1, 1.2, 16, 2.0, {"ff": 16, "limit": 2.0})},
        {"type": "attention",
         "mixer": {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.18,
                   "rot": _rot(8000.0, 8, {"factor": 6.0, "original": 48, "fast": 6.0, "slow": 1.5})},
         "mlp": _mlp(5, 2, 0.9, 24, 1.1, {"ff": 8, "limit": 0.9})},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 4, "dim": 8, "vdim": 8, "scale": 0.35, "rot": _rot(100.0, 4)},
         "mlp": None},
    ],
    "loop": {"start": 1, "stop": 2, "times": 3},
}

# sizes at which the bfloat16 path leaves the kernels for every size: key and value heads of 64 and 128 (tensor-core
# attention), widths and expert sizes that are multiples of 64 (the tiled expert product for steps of 16 tokens or more)
TENSOR_CORE_SIZES = {
    "architecture": "Gefarax", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention",
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 128, "scale": 0.125,
                   "rot": _rot(40000.0, 32, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0})},
         "mlp": _mlp(4, 2, 1.1, 64, 1.4, {"ff": 64, "limit": 1.8})},
        {"type": "attention",
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09,
                   "rot": _rot(10000.0, 128, {"factor": 8.0, "original": 32, "fast": 8.0, "slow": 2.0})},
         "mlp": _mlp(3, 1, 1.6, 128, 0.7)},
    ],
    "loop": {"start": 1, "stop": 2, "times": 2},
}

# name -> (config.json dict, weight seed)
GEFARAX = {"loop_from_start": (LOOP_FROM_START, 11), "no_loop": (NO_LOOP, 12), "loop_in_the_middle": (LOOP_IN_THE_MIDDLE, 13),
           "tensor_core_sizes": (TENSOR_CORE_SIZES, 14)}
