"""A plain, slow implementation of the Dikusun design: one function per mechanism, float64 on the CPU.

It shares no code with the engine.  ``weights`` is a dict name -> torch tensor (any float type), ``config`` the
dict form of config.json.  Everything is computed per sequence, whole prompt at once, except where a function
says that it walks the tokens one by one.

    rms(x)            = x / sqrt(mean(x^2) + eps)
    layer             x += rms(mixer(x)) * w1;  x += rms(ff(x)) * w2      (sub-layers read the stream as it is)
    attention         two score maps per head over the same values, a1 - lambda * a2, per-head rms, a gate per head
    latent_attention  queries and keys/values through low-rank latents; the key/value latent is all a token leaves
    gla               S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t
    feed-forward      g * sigmoid(1.702 g) * (u + 1) with g and u clamped
"""
import math

import torch

F = torch.float64
GATE_SLOPE = 1.702


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight.to(F)


def linear(x, weights, name):
    """W x for W stored [out, in], plus the bias ``name.b`` where the checkpoint has one."""
    y = x @ weights[name].to(F).T
    if name + ".b" in weights:
        y = y + weights[name + ".b"].to(F)
    return y


def rotate(x, positions, rot):
    """x: [T, ..., dim]; the first rot.dims elements of the last axis turn, element i paired with i + dims/2."""
    if not rot:
        return x
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def visible(positions, window=None):
    """[T, T] bool: query i (rows) sees key j (columns)."""
    distance = positions[:, None] - positions[None, :]
    seen = distance >= 0
    if window:
        seen = seen & (distance < int(window))
    return seen


def softmax_rows(scores, seen):
    scores = scores.masked_fill(~seen, -math.inf)
    e = torch.exp(scores - scores.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def differential_lambda(weights, prefix, diff):
    def dot(a, b):
        return (weights[prefix + a].to(F) * weights[prefix + b].to(F)).sum()
    return torch.exp(dot("lq1", "lk1")) - torch.exp(dot("lq2", "lk2")) + diff


def attention_mixer(h, positions, mixer, weights, prefix, eps):
    """Differential attention with grouped key/value heads, a sliding window and capped scores."""
    heads, groups, dim, vdim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer["vdim"])
    T = h.shape[0]
    q = linear(h, weights, prefix + "q").view(T, heads, 2, dim)
    k = linear(h, weights, prefix + "k").view(T, groups, 2, dim)
    v = linear(h, weights, prefix + "v").view(T, groups, vdim)
    q = rotate(rms_norm(q, weights[prefix + "q.norm"], eps), positions, mixer.get("rot"))
    k = rotate(rms_norm(k, weights[prefix + "k.norm"], eps), positions, mixer.get("rot"))
    window = (mixer.get("mask") or {}).get("size")
    seen = visible(positions, window)
    cap = mixer.get("softcap")
    diff = float(mixer["diff"])
    lam = differential_lambda(weights, prefix, diff)
    gate = torch.sigmoid(h @ weights[prefix + "g"].to(F).T)       # [T, heads]
    out = torch.zeros(T, heads, vdim, dtype=F)
    for head in range(heads):
        g = head // (heads // groups)
        maps = []
        for m in range(2):
            scores = (q[:, head, m, :] @ k[:, g, m, :].T) * float(mixer["scale"])
            if cap:
                scores = float(cap) * torch.tanh(scores / float(cap))
            maps.append(softmax_rows(scores, seen) @ v[:, g, :])
        o = rms(maps[0] - lam * maps[1], eps) * (1.0 - diff)
        out[:, head, :] = o * gate[:, head:head + 1]
    return linear(out.reshape(T, heads * vdim), weights, prefix + "o")


def latent_of(h, weights, prefix, eps):
    """What a token leaves in the cache of a latent-attention layer: [T, kv_rank]."""
    return rms_norm(linear(h, weights, prefix + "dkv"), weights[prefix + "dkv.norm"], eps)


def latent_attention_mixer(h, positions, mixer, weights, prefix, eps):
    heads, dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    T = h.shape[0]
    c_q = rms_norm(linear(h, weights, prefix + "dq"), weights[prefix + "dq.norm"], eps)
    q = linear(c_q, weights, prefix + "uq").view(T, heads, dim)
    c = latent_of(h, weights, prefix, eps)
    k = linear(c, weights, prefix + "uk").view(T, heads, dim)
    v = linear(c, weights, prefix + "uv").view(T, heads, vdim)
    seen = visible(positions)
    out = torch.zeros(T, heads, vdim, dtype=F)
    for head in range(heads):
        scores = (q[:, head, :] @ k[:, head, :].T) * float(mixer["scale"])
        out[:, head, :] = softmax_rows(scores, seen) @ v[:, head, :]
    return linear(out.reshape(T, heads * vdim), weights, prefix + "o")


def gla_decay(h, mixer, weights, prefix):
    """alpha = sigmoid(z)^(1/tau) per key channel, z = W_a2 (W_a1 h) + b: [T, heads, dim]."""
    heads, dim = int(mixer["heads"]), int(mixer["dim"])
    z = linear(linear(h, weights, prefix + "a1"), weights, prefix + "a2")
    return (torch.sigmoid(z) ** (1.0 / float(mixer["tau"]))).view(-1, heads, dim)


def gla_mixer(h, mixer, weights, prefix, eps, state=None):
    """Walks the tokens one by one.  ``state``: [heads, dim, vdim] to start from (zeros when None); returns
    (output, last state)."""
    heads, dim, vdim = int(mixer["heads"]), int(mixer["dim"]), int(mixer["vdim"])
    T = h.shape[0]
    q = linear(h, weights, prefix + "q").view(T, heads, dim) * dim ** -0.5
    k = linear(h, weights, prefix + "k").view(T, heads, dim)
    v = linear(h, weights, prefix + "v").view(T, heads, vdim)
    alpha = gla_decay(h, mixer, weights, prefix)
    S = torch.zeros(heads, dim, vdim, dtype=F) if state is None else state.to(F).clone()
    out = torch.zeros(T, heads, vdim, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms_norm(out, weights[prefix + "norm"], eps).reshape(T, heads * vdim)
    gate = linear(h, weights, prefix + "g")
    out = out * (gate * torch.sigmoid(gate))
    return linear(out, weights, prefix + "o"), S


def dense_feed_forward(h, mlp, weights, prefix):
    limit = float(mlp["limit"])
    g = torch.clamp(linear(h, weights, prefix + "gate"), max=limit)
    u = torch.clamp(linear(h, weights, prefix + "up"), min=-limit, max=limit)
    return linear(g * torch.sigmoid(GATE_SLOPE * g) * (u + 1.0), weights, prefix + "down")


def layer_prefix(config, index):
    """Layers that name another layer's weights read that layer's tensors."""
    entry = config["layers"][index]
    return f"l{entry['weights_of']}." if entry.get("weights_of") is not None else f"l{index}."


def mixer_output(h, positions, entry, weights, prefix, eps):
    kind = entry["type"]
    if kind == "attention":
        return attention_mixer(h, positions, entry["mixer"], weights, prefix, eps)
    if kind == "latent_attention":
        return latent_attention_mixer(h, positions, entry["mixer"], weights, prefix, eps)
    if kind == "gla":
        return gla_mixer(h, entry["mixer"], weights, prefix, eps)[0]
    raise ValueError(f"unknown mixer type {kind!r}")


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the stream after every layer."""
    eps = float(config["norm"]["eps"])
    positions = torch.arange(len(tokens))
    x = weights["embed"].to(F)[torch.tensor(tokens)] * float(config["embedding"]["scale"])
    streams = []
    for index, entry in enumerate(config["layers"]):
        prefix = layer_prefix(config, index)
        x = x + rms_norm(mixer_output(x, positions, entry, weights, prefix + "mix.", eps), weights[prefix + "norm1"], eps)
        if entry.get("mlp") is not None:
            x = x + rms_norm(dense_feed_forward(x, entry["mlp"], weights, prefix + "mlp."), weights[prefix + "norm2"], eps)
        streams.append(x.clone())
    logits = rms_norm(x, weights["final.norm"], eps) @ weights["head"].to(F).T
    return (logits, torch.stack(streams)) if return_layers else logits
