"""A plain, slow implementation of the Gefarax design: one function per mechanism, float64 on the CPU.

It shares no code with the engine.  ``weights`` is a dict name -> torch tensor (any float type), ``config`` the
dict form of config.json.  Everything is computed per sequence, whole prompt at once.

    norm(x)      = x / sqrt(mean(x^2) + eps) * w
    layer        x += norm_1b(mixer(norm_1(x)));  x += norm_2b(ff(norm_2(x)))
    attention    softmax over the visible keys and one sink per head that has neither key nor value
    rotation     pairs (i, i + dims/2) of the first dims elements; frequencies stretched for long contexts
    experts      the top choices by sigmoid(router) + correction, weighted by sigmoid(router) * scale, plus a shared one
    loop         a run of layers repeated with the same weights; each later pass adds the embedded tokens first
"""
import math

import torch

F = torch.float64


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F)


def rotary_frequencies(rot):
    """Per pair i < dims/2: the angular frequency and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = [base ** (-2.0 * i / dims) for i in range(half)]
    scaling = rot.get("scaling")
    if not scaling:
        return torch.tensor(freq, dtype=F), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(freq[i] / factor * ramp + freq[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x: [T, heads, dim]; the first rot.dims elements of each head turn, paired (i, i + dims/2)."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    freq, magnitude = rotary_frequencies(rot)
    angle = positions.to(F)[:, None] * freq[None, :]           # [T, half]
    cos, sin = (torch.cos(angle) * magnitude)[:, None, :], (torch.sin(angle) * magnitude)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def attention_mixer(h, positions, mixer, weights, prefix):
    """h: [T, width] of ONE sequence, positions 0..T-1 in order."""
    heads, groups, dim, vdim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    T = h.shape[0]
    q = (h @ weights[prefix + "q"].to(F).T).view(T, heads, dim)
    k = (h @ weights[prefix + "k"].to(F).T).view(T, groups, dim)
    v = (h @ weights[prefix + "v"].to(F).T).view(T, groups, vdim)
    q, k = rotate(q, positions, mixer.get("rot")), rotate(k, positions, mixer.get("rot"))
    sink = weights[prefix + "sink"].to(F)
    out = torch.zeros(T, heads, vdim, dtype=F)
    per_group = heads // groups
    for head in range(heads):
        g = head // per_group
        scores = (q[:, head, :] @ k[:, g, :].T) * float(mixer["scale"])        # [T, T]
        visible = positions[None, :] <= positions[:, None]
        scores = scores.masked_fill(~visible, -math.inf)
        top = torch.maximum(scores.max(-1).values, sink[head])
        e = torch.exp(scores - top[:, None])
        denominator = e.sum(-1) + torch.exp(sink[head] - top)
        out[:, head, :] = (e / denominator[:, None]) @ v[:, g, :]
    return out.reshape(T, heads * vdim) @ weights[prefix + "o"].to(F).T


def clamped_expert(h, weights, prefix, limit):
    g = torch.clamp(h @ weights[prefix + "gate"].to(F).T, max=limit)
    u = torch.clamp(h @ weights[prefix + "up"].to(F).T, min=-limit, max=limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return y @ weights[prefix + "down"].to(F).T


def route(h, weights, prefix, router):
    """(chosen experts [T, top], their weights [T, top], margin [T]: by how much the last chosen expert's choice
    score beats the best one left out; infinite when every expert is chosen)."""
    z = h @ weights[prefix + "router"].to(F).T
    s = torch.sigmoid(z)
    choice = s + weights[prefix + "correction"].to(F) if prefix + "correction" in weights else s
    top = int(router["top"])
    ordered = torch.sort(choice, dim=-1, descending=True, stable=True)
    chosen = ordered.indices[:, :top]
    if top < choice.shape[1]:
        margin = ordered.values[:, top - 1] - ordered.values[:, top]
    else:
        margin = torch.full((h.shape[0],), math.inf, dtype=F)
    return chosen, torch.gather(s, 1, chosen) * float(router["scale"]), margin


def moe(h, mlp, weights, prefix, margins=None):
    chosen, weight, margin = route(h, weights, prefix, mlp["router"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], weights[prefix + "e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for slot in range(chosen.shape[1]):
            e = int(chosen[t, slot])
            out[t] += weight[t, slot] * clamped_expert(h[t:t + 1], weights, f"{prefix}e{e}.", float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared"):
        out = out + clamped_expert(h, weights, prefix + "shared.", float(mlp["shared"]["limit"]))
    return out


def layer_order(config):
    """Indices of the layers in the order they run, and for each run whether a new pass of the loop starts there
    (so that the embedding output is added first)."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, False) for i in range(count)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, False) for i in range(start)]
    for p in range(times):
        for i in range(start, stop):
            order.append((i, p > 0 and i == start))
    order += [(i, False) for i in range(stop, count)]
    return order


def forward(config, weights, tokens, keep_layers=False, margins=None):
    """Logits [T, vocab] (float64) of one sequence; with keep_layers also the stream after every layer run.
    ``margins``: a list that receives one [T] tensor of routing margins per routed layer run."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    embedded = weights["embed"].to(F)[tokens]
    x = embedded.clone()
    kept = []
    for index, new_pass in layer_order(config):
        layer = config["layers"][index]
        name = f"l{index}."
        if new_pass:
            x = x + embedded
        h = rms_norm(x, weights[name + "norm1"], eps)
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        mixed = attention_mixer(h, positions, layer["mixer"], weights, name + "mix.")
        x = x + rms_norm(mixed, weights[name + "norm1b"], eps)
        if layer.get("mlp"):
            h = rms_norm(x, weights[name + "norm2"], eps)
            x = x + rms_norm(moe(h, layer["mlp"], weights, name + "mlp.", margins), weights[name + "norm2b"], eps)
        kept.append(x.clone())
    logits = rms_norm(x, weights["final.norm"], eps) @ weights["head"].to(F).T
    return (logits, torch.stack(kept)) if keep_layers else logits
