"""Gefarax on the GPU against the plain implementation in plain_gefarax.py: each mechanism alone, then whole models
through the step function, the cache and the scheduler, cut and batched in different ways, in 32-bit and bfloat16."""
import copy
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_gefarax as plain
import traces
from gefarax_configs import GEFARAX
from helpers import tokens_for

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(GEFARAX)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
# bfloat16 rounds activations, so a token whose router all but ties may go to another expert than in the plain
# implementation; rows are compared only where every routing decision of the token has at least this margin
SAFE_MARGIN = 0.03
# Largest allowed |engine - plain| as a fraction of the row's largest |plain logit|.  bfloat16: a layer rounds its
# activations at twice as many places as a layer with two norms does (four norms, the routed and the shared expert), and
# a token's expert weights scale whole expert outputs, so the allowance is wider than for the dense models' tests.
ALLOWED = {"float32": 2e-5, "bfloat16": 5e-2}


def _every_expert(raw):
    """The same model with routers that choose all of their experts: no routing decision is left that bfloat16
    rounding could turn, so every row can be compared."""
    changed = copy.deepcopy(raw)
    for layer in changed["layers"]:
        if layer["mlp"]:
            layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return changed


EVERY_EXPERT = {name + "/every_expert": (_every_expert(raw), seed + 100) for name, (raw, seed) in GEFARAX.items()}


# ------------------------------------------------------------------------------------------------ model folders
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Model folders with random weights.  Routers, corrections and sinks are redrawn wider than the generic random
    mode draws them, so that experts are chosen by the token and a sink that is left out shows."""
    from safetensors.torch import load_file, save_file

    import llmserver_b200.models  # noqa: F401
    from llmserver_b200.config import GefaraxConfig
    from llmserver_b200.weights import write_model_folder

    root = tmp_path_factory.mktemp("gefarax")
    made = {}
    for name, (raw, seed) in list(GEFARAX.items()) + list(EVERY_EXPERT.items()):
        folder = write_model_folder(GefaraxConfig.from_dict(raw), str(root / name.replace("/", "_")), seed, torch.bfloat16)
        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        generator = torch.Generator().manual_seed(seed)
        for key in sorted(tensors):
            if key.endswith(".router"):
                tensors[key] = (torch.randn(tensors[key].shape, generator=generator) * 0.3).to(torch.bfloat16)
            elif key.endswith(".correction"):
                tensors[key] = (torch.randn(tensors[key].shape, generator=generator) * 0.2).to(torch.bfloat16)
            elif key.endswith(".sink"):
                tensors[key] = (torch.randn(tensors[key].shape, generator=generator) * 1.5).to(torch.bfloat16)
        save_file(tensors, path)
        made[name] = folder
    return made


_PLAIN = {}


def plain_model_of(folder):
    if folder not in _PLAIN:
        from safetensors.torch import load_file
        with open(os.path.join(folder, "config.json")) as handle:
            config = json.load(handle)
        _PLAIN[folder] = (config, {key: value.to(F64) for key, value in load_file(os.path.join(folder, "model.safetensors")).items()})
    return _PLAIN[folder]


_LOGITS = {}


def plain_logits(folder, tokens):
    """(float64 logits [T, V], smallest routing margin of each token [T]) of the whole sequence."""
    key = (folder, tuple(tokens))
    if key not in _LOGITS:
        config, weights = plain_model_of(folder)
        margins = []
        logits = plain.forward(config, weights, list(tokens), margins=margins)
        margin = torch.stack(margins).min(dim=0).values if margins else torch.full((len(tokens),), math.inf)
        _LOGITS[key] = (logits.numpy(), margin.numpy())
    return _LOGITS[key]


def run_in_process(folder, dtype, records, max_tokens, page_size=16):
    from llmserver_b200.engine.replay import TraceReplayer

    replayer = TraceReplayer(folder, dtype, max_tokens, page_size)
    out = {}
    for record in records:
        logits = replayer.run_step(record)
        if logits is not None:
            out[record["step"]] = logits
    replayer.cache.check_invariants()
    assert not replayer.cache.requests, "requests left in the cache after the trace ended"
    for group in replayer.cache.groups:
        assert group.pool.num_available == group.pool.num_pages, "pages were lost"
    return out, replayer


def compare(got, records, requests, folder, dtype, what):
    want = traces.expected_rows(records, requests, lambda name: plain_logits(folder, requests[name])[0])
    safe = traces.expected_rows(records, requests, lambda name: plain_logits(folder, requests[name])[1][:, None])
    assert set(got) == set(want), f"{what}: steps with logits differ"
    compared = total = 0
    for step in sorted(want):
        assert got[step].shape == want[step].shape and np.isfinite(got[step]).all(), f"{what} step {step}"
        rows = np.arange(len(want[step])) if dtype == "float32" else np.nonzero(safe[step][:, 0] >= SAFE_MARGIN)[0]
        total += len(want[step])
        compared += len(rows)
        if len(rows):
            scale = np.abs(want[step][rows]).max(axis=-1)
            error = np.abs(got[step][rows] - want[step][rows]).max(axis=-1) / scale
            assert error.max() <= ALLOWED[dtype], (f"{what} step {step}: row {int(rows[error.argmax()])} differs by "
                                                   f"{error.max():.3e} of its largest logit, allowed {ALLOWED[dtype]:.1e}")
    assert total < 20 or compared >= 0.3 * total, f"{what}: only {compared} of {total} rows had a safe routing margin"


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_stretched_frequencies_and_magnitude():
    from llmserver_b200.parts import POSITION_ENCODINGS, Runtime
    for rot in ({"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}},
                {"base": 50000.0, "dims": 64, "scaling": {"factor": 32.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                {"base": 300.0, "dims": 6, "scaling": {"factor": 1.5, "original": 16, "fast": 2.0, "slow": 0.25}}):
        scaling = rot["scaling"]
        part = POSITION_ENCODINGS.get("stretched_rotary")(
            dict(head_dim=rot["dims"] + 8, theta=rot["base"], rotary_dim=rot["dims"], factor=scaling["factor"],
                 original=scaling["original"], fast=scaling["fast"], slow=scaling["slow"]), {}, Runtime(torch.float32, torch.device(DEVICE)))
        want, magnitude = plain.rotary_frequencies(rot)
        assert torch.allclose(part.inv_freq.cpu().double(), want, rtol=1e-6, atol=0)
        assert abs(part.attention_factor - magnitude) < 1e-12
        assert part.rotary_dim == rot["dims"]
        # the ramp really has both ends in these cases: some pair keeps its frequency, some pair is fully stretched
        plain_freq = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=F64)
        ratio = want / plain_freq
        assert ratio.max() > 0.999 and ratio.min() < 1.0 / scaling["factor"] + 1e-9


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,dims", [(4, 2, 32, 16, 16), (3, 1, 24, 40, 24), (2, 2, 16, 16, 0), (5, 5, 64, 8, 6)])
def test_rotation_and_cache_write(dtype, heads, kv_heads, dim, vdim, dims):
    from llmserver_b200 import ops
    generator = torch.Generator().manual_seed(dim + vdim)
    page_size, pages = 4, 12
    # two sequences: positions 5..10 of one (it crosses a page border) and position 0..2 of another
    positions = torch.tensor([5, 6, 7, 8, 9, 10, 0, 1, 2], dtype=torch.int32)
    seq = torch.tensor([0] * 6 + [1] * 3, dtype=torch.int32)
    tables = torch.tensor([[7, 3, 9], [2, 0, 0]], dtype=torch.int32)
    width = (heads + kv_heads) * dim + kv_heads * vdim
    packed = torch.randn((len(positions), width), generator=generator).to(dtype)
    rot = {"base": 1000.0, "dims": dims, "scaling": {"factor": 4.0, "original": 8, "fast": 2.0, "slow": 0.5}} if dims else None
    inv_freq, magnitude = (None, 1.0)
    if rot:
        freq, magnitude = plain.rotary_frequencies(rot)
        inv_freq = freq.to(torch.float32).to(DEVICE)
    k_pages = torch.zeros((pages, kv_heads, page_size, dim), dtype=dtype, device=DEVICE)
    v_pages = torch.zeros((pages, kv_heads, page_size, vdim), dtype=dtype, device=DEVICE)
    flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    on_device = packed.to(DEVICE)
    ops.rope_kv_write_split(on_device, inv_freq, magnitude, positions.to(DEVICE), seq.to(DEVICE), tables.to(DEVICE), k_pages,
                            v_pages, heads, kv_heads, dim, vdim, True, flag, dims)
    assert int(flag.item()) == 0
    source = packed.double()
    q = plain.rotate(source[:, :heads * dim].view(-1, heads, dim), positions, rot)
    k = plain.rotate(source[:, heads * dim:(heads + kv_heads) * dim].view(-1, kv_heads, dim), positions, rot)
    v = source[:, (heads + kv_heads) * dim:].view(-1, kv_heads, vdim)
    tolerance = 1e-5 if dtype == torch.float32 else 2e-2
    got = on_device.cpu().double()
    assert torch.allclose(got[:, :heads * dim].view(-1, heads, dim), q, atol=tolerance, rtol=tolerance)
    written = torch.zeros_like(k_pages, dtype=F64, device="cpu"), torch.zeros_like(v_pages, dtype=F64, device="cpu")
    for token in range(len(positions)):
        page = int(tables[seq[token], positions[token] // page_size])
        written[0][page, :, positions[token] % page_size] = k[token]
        written[1][page, :, positions[token] % page_size] = v[token]
    assert torch.allclose(k_pages.cpu().double(), written[0], atol=tolerance, rtol=tolerance)   # untouched slots stay zero
    assert torch.allclose(v_pages.cpu().double(), written[1], atol=tolerance, rtol=tolerance)


def _paged_attention_case(dtype, heads, kv_heads, dim, vdim, lengths, queries, page_size, seed, sinks, spike=None):
    """Random keys and values of sequences of ``lengths`` tokens in shuffled pages; ``queries``: (sequence, position)
    pairs.  ``spike`` = (query index, key position): that query and that key are scaled so that their score stands out.
    Returns what the kernel needs and the plain result [queries, heads * vdim]."""
    generator = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-length // page_size) for length in lengths) + 3
    order = torch.randperm(n_pages, generator=generator).tolist()
    width = max(-(-length // page_size) for length in lengths)
    tables = torch.zeros((len(lengths), width), dtype=torch.int32)
    keys = [torch.randn((length, kv_heads, dim), generator=generator).to(dtype) for length in lengths]
    values = [torch.randn((length, kv_heads, vdim), generator=generator).to(dtype) for length in lengths]
    q = torch.randn((len(queries), heads, dim), generator=generator).to(dtype)
    if spike is not None:
        index, position = spike
        sequence = queries[index][0]
        direction = torch.randn((dim,), generator=generator)
        direction = direction / direction.norm()
        length = math.sqrt(14.0 * math.sqrt(dim))       # a score of 14 after the scale
        q[index] = (direction * length).to(dtype)
        keys[sequence][position] = (direction * length).to(dtype)
    k_pages = torch.zeros((n_pages, kv_heads, page_size, dim), dtype=dtype)
    v_pages = torch.zeros((n_pages, kv_heads, page_size, vdim), dtype=dtype)
    for sequence, length in enumerate(lengths):
        for block in range(-(-length // page_size)):
            page = order.pop()
            tables[sequence, block] = page
            rows = slice(block * page_size, min(length, (block + 1) * page_size))
            count = rows.stop - rows.start
            k_pages[page, :, :count] = keys[sequence][rows].transpose(0, 1)
            v_pages[page, :, :count] = values[sequence][rows].transpose(0, 1)
    want = torch.zeros((len(queries), heads, vdim), dtype=F64)
    spike_weight = 1.0
    scale = 1.0 / math.sqrt(dim)
    for index, (sequence, position) in enumerate(queries):
        for head in range(heads):
            group = head // (heads // kv_heads)
            scores = (keys[sequence][:position + 1, group].double() @ q[index, head].double()) * scale
            terms = torch.cat([scores, sinks[head:head + 1].double()]) if sinks is not None else scores
            weights = torch.softmax(terms, dim=0)[:position + 1]
            want[index, head] = weights @ values[sequence][:position + 1, group].double()
            if spike is not None and index == spike[0]:
                spike_weight = min(spike_weight, float(weights[spike[1]]))
    return q, k_pages, v_pages, tables, scale, want.reshape(len(queries), heads * vdim), spike_weight


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 32, 16), (6, 1, 24, 40), (2, 2, 64, 64), (8, 2, 128, 128), (4, 1, 64, 80)])
def test_attention_with_sinks_and_value_size(dtype, heads, kv_heads, dim, vdim):
    """Prompt rows and single decoded rows side by side, sequences of unequal length, keys found through shuffled
    pages; one query's score for a key far back, the last slot of a page, towers over the rest; sinks from -2 to 3."""
    from llmserver_b200 import ops
    page_size = 8
    lengths = [300, 41, 1, 130]
    queries = [(0, 299), (1, 40), (2, 0), (3, 100), (3, 101), (3, 102), (3, 129), (0, 7), (0, 8)]
    sinks = torch.linspace(-2.0, 3.0, heads)
    for spike in ((0, 7), (0, 8), (3, 0), None):
        q, k_pages, v_pages, tables, scale, want, spike_weight = _paged_attention_case(
            dtype, heads, kv_heads, dim, vdim, lengths, queries, page_size, 17, sinks, spike)
        packed = q.reshape(len(queries), heads * dim).contiguous()
        out = ops.attention_generic(packed.to(DEVICE), heads * dim, k_pages.to(DEVICE), v_pages.to(DEVICE), tables.to(DEVICE),
                                    torch.tensor([s for s, _ in queries], dtype=torch.int32, device=DEVICE),
                                    torch.tensor([p for _, p in queries], dtype=torch.int32, device=DEVICE),
                                    heads, kv_heads, dim, scale, value_dim=vdim, sinks=sinks.to(DEVICE))
        tolerance = 2e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(out.cpu().double(), want, atol=tolerance, rtol=tolerance), f"spike {spike}"
        if spike is not None:
            assert spike_weight > 0.9       # the far key really carries the row: a kernel that missed it would be far off
    # a sink that is left out shows: the same case without sinks gives other numbers
    without = ops.attention_generic(packed.to(DEVICE), heads * dim, k_pages.to(DEVICE), v_pages.to(DEVICE), tables.to(DEVICE),
                                    torch.tensor([s for s, _ in queries], dtype=torch.int32, device=DEVICE),
                                    torch.tensor([p for _, p in queries], dtype=torch.int32, device=DEVICE),
                                    heads, kv_heads, dim, scale, value_dim=vdim)
    assert (without.cpu().double() - want).abs().max() > 0.05


@pytest.mark.parametrize("prefill", ["tcgen05", "mma"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(4, 2, 64, 64), (8, 1, 128, 128), (10, 2, 128, 128), (6, 2, 64, 128), (16, 1, 128, 64), (5, 5, 64, 64)])
def test_tensor_core_attention_with_sinks(heads, kv_heads, dim, vdim, prefill):
    """The bfloat16 kernels a step uses for these head sizes: a whole prompt, a portion behind cached tokens, single
    decoded tokens of short contexts and of one long enough to be split, all in one batch; sinks from -2 to 3; one
    decoded query's score for a key far back towers over the rest, so weights rounded to 8 bits would not pass either
    (the row is compared to 3e-3 of its size)."""
    from llmserver_b200 import ops
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    from llmserver_b200.ops import attention_bf16
    from llmserver_b200.ops.library import check_wait_errors
    if prefill == "mma" and not (dim == vdim == 128):
        pytest.skip("only heads of 128 have two prompt kernels to choose from")
    page_size = 16
    lengths = [300, 41, 1, 130, 2500]
    new_tokens = [1, 41, 1, 30, 1]
    queries = [(s, p) for s, (length, count) in enumerate(zip(lengths, new_tokens)) for p in range(length - count, length)]
    sinks = torch.linspace(-2.0, 3.0, heads)
    for spike in ((len(queries) - 1, 15), (0, 16), (60, 15), None):      # query 60: a prompt row at position 117
        q, k_pages, v_pages, tables, scale, want, spike_weight = _paged_attention_case(
            torch.bfloat16, heads, kv_heads, dim, vdim, lengths, queries, page_size, 23, sinks, spike)
        slices = [SequenceSlice(f"r{s}", [0] * count, length - count, [], [tables[s, :-(-length // page_size)].tolist()], 0)
                  for s, (length, count) in enumerate(zip(lengths, new_tokens))]
        batch = build_batch(slices, 1, DEVICE)
        width = (heads + kv_heads) * dim + kv_heads * vdim
        packed = torch.zeros((len(queries), width), dtype=torch.bfloat16)
        packed[:, :heads * dim] = q.reshape(len(queries), heads * dim)
        before, attention_bf16.PRECISE_PREFILL_KERNEL = attention_bf16.PRECISE_PREFILL_KERNEL, prefill
        try:
            out = ops.attention(packed.to(DEVICE), batch, batch.block_tables[0], k_pages.to(DEVICE), v_pages.to(DEVICE), heads,
                                kv_heads, dim, scale, value_dim=vdim, sinks=sinks.to(DEVICE), precise=True)
        finally:
            attention_bf16.PRECISE_PREFILL_KERNEL = before
        torch.cuda.synchronize()
        check_wait_errors()
        error = (out.cpu().double() - want).abs().max(dim=-1).values / want.abs().max(dim=-1).values.clamp_min(0.05)
        assert error.max() < 6e-3, f"spike {spike}: row {int(error.argmax())} of {len(queries)} differs by {float(error.max()):.2e}"
        if spike is not None:
            assert spike_weight > 0.9


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,width", [(4, 2, 64), (5, 1, 48), (3, 3, 96), (40, 6, 160)])
def test_router(dtype, experts, top, width):
    from llmserver_b200 import ops
    generator = torch.Generator().manual_seed(experts * 7 + top)
    tokens = 50
    x = torch.randn((tokens, width), generator=generator).to(dtype)
    weights = {"r.router": (torch.randn((experts, width), generator=generator) * 0.2).to(torch.bfloat16).double(),
               "r.correction": (torch.randn((experts,), generator=generator) * 0.3).to(torch.bfloat16).double()}
    chosen, weight, margin = plain.route(x.double(), weights, "r.", {"top": top, "scale": 1.7})
    got_chosen, got_weight = ops.moe_route(x.to(DEVICE), weights["r.router"].float().to(DEVICE),
                                           weights["r.correction"].float().to(DEVICE), top, 1.7)
    clear = margin > 1e-4
    assert clear.sum() >= tokens * 0.9
    # the chosen set, in order of their choice scores, wherever the plain implementation's choice is not a near tie
    assert torch.equal(got_chosen.cpu().long()[clear], chosen[clear])
    assert torch.allclose(got_weight.cpu().double()[clear], weight[clear], atol=1e-5, rtol=1e-5)
    # equal choice scores go to the lower index
    tied, _ = ops.moe_route(torch.zeros((2, width), dtype=dtype, device=DEVICE), torch.zeros((experts, width), device=DEVICE),
                            None, top, 1.0)
    assert tied.cpu().tolist() == [list(range(top))] * 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,width,inter,shared,tokens", [
    (4, 2, 64, 48, 32, 37), (5, 1, 48, 24, None, 37), (3, 3, 96, 40, 56, 37),
    # sizes the tiled product over sorted pairs takes (bfloat16, 16 tokens or more): experts with several row tiles, with
    # a handful of rows and with none, feature counts that fill a column tile and that do not; and the same sizes with
    # so few tokens that each pair multiplies alone
    (3, 2, 128, 64, 64, 400), (5, 2, 128, 192, 64, 300), (7, 3, 320, 448, None, 260), (9, 3, 192, 136, None, 150),
    (6, 2, 128, 64, 64, 5), (40, 4, 64, 72, 8, 33)])
@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
def test_routed_experts_part(dtype, experts, top, width, inter, shared, tokens, kernel):
    from llmserver_b200 import ops
    from llmserver_b200.ops.library import check_wait_errors
    from llmserver_b200.parts import FEED_FORWARDS, Runtime
    if kernel == "mma" and (dtype == "float32" or tokens < 16 or width % 64 or inter % 64):
        pytest.skip("the choice of tiled kernel only matters where one runs")
    generator = torch.Generator().manual_seed(experts + width)
    params = dict(hidden=width, experts=experts, top=top, intermediate=inter, limit=0.9, route_scale=1.3)
    mlp = {"router": {"experts": experts, "top": top, "scale": 1.3}, "expert": {"ff": inter, "limit": 0.9}, "shared": None}
    if shared:
        params.update(shared_intermediate=shared, shared_limit=0.6)
        mlp["shared"] = {"ff": shared, "limit": 0.6}
    cls = FEED_FORWARDS.get("routed_experts")
    raw = {}
    for name, declaration in cls.declare_weights(params).items():
        spread = 0.3 if name in ("router", "correction") else 0.25     # wide enough for the clamps to bite
        raw[name] = (torch.randn(declaration.shape, generator=generator) * spread).to(torch.bfloat16)
    torch_dtype = getattr(torch, dtype)
    part = cls(params, {name: (value.float() if name in ("router", "correction") else value.to(torch_dtype)).to(DEVICE)
                        for name, value in raw.items()}, Runtime(torch_dtype, torch.device(DEVICE)))
    x = torch.randn((tokens, width), generator=generator).to(torch_dtype)
    want_weights = {"m." + name: value.double() for name, value in raw.items()}
    margins = []
    want = plain.moe(x.double(), mlp, want_weights, "m.", margins)
    before, ops.MOE_GROUPED_KERNEL = ops.MOE_GROUPED_KERNEL, kernel
    try:
        got = part.forward(x.to(DEVICE)).cpu().double()
    finally:
        ops.MOE_GROUPED_KERNEL = before
    check_wait_errors()
    rows = margins[0] > (1e-4 if dtype == "float32" else 1e-2)
    tolerance = 2e-5 if dtype == "float32" else 2e-2
    assert rows.sum() > tokens // 2
    assert torch.allclose(got[rows], want[rows], atol=tolerance * float(want.abs().max()), rtol=tolerance)
    # the clamps were exercised: some gate or up value lay beyond the limit
    gate = x.double() @ want_weights["m.e0.gate"].T
    assert (gate > 0.9).any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [48, 50, 64, 1000, 4100])
def test_normed_delta_joins_the_stream(dtype, width):
    from llmserver_b200 import ops
    generator = torch.Generator().manual_seed(width)
    rows = 9
    stream = torch.randn((rows, width), generator=generator)
    delta = (torch.randn((rows, width), generator=generator) * 3.0).to(dtype)
    extra = torch.randn((rows, width), generator=generator)
    post = (1.0 + 0.1 * torch.randn((width,), generator=generator)).to(dtype)
    after = (1.0 + 0.1 * torch.randn((width,), generator=generator)).to(dtype)
    for use_extra in (False, True):
        updated = stream.double() + plain.rms_norm(delta.double(), post.double(), 1e-5) + (extra.double() if use_extra else 0.0)
        want = plain.rms_norm(updated, after.double(), 1e-6)
        on_device = stream.to(DEVICE)
        got = ops.normed_add_rmsnorm(on_device, delta.to(DEVICE), post.to(DEVICE), 1e-5, after.to(DEVICE), 1e-6,
                                     extra=extra.to(DEVICE) if use_extra else None, act_dtype=dtype)
        tolerance = 1e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(on_device.cpu().double(), updated, atol=1e-5, rtol=1e-5)          # the stream is 32-bit in either path
        assert torch.allclose(got.cpu().double(), want, atol=tolerance, rtol=tolerance)
        if use_extra:
            # a second stream alone, nothing to normalise: what the model does when the block in front left a plain delta
            on_device = stream.to(DEVICE)
            assert ops.normed_add_rmsnorm(on_device, None, None, 0.0, None, 0.0, extra=extra.to(DEVICE), want_output=False,
                                          act_dtype=dtype) is None
            assert torch.allclose(on_device.cpu().double(), stream.double() + extra.double(), atol=1e-6, rtol=1e-6)
        # selected rows: the stream stays as it was
        on_device = stream.to(DEVICE)
        picked = torch.tensor([4, 0, 8], dtype=torch.int32, device=DEVICE)
        got = ops.normed_add_rmsnorm(on_device, delta.to(DEVICE), post.to(DEVICE), 1e-5, after.to(DEVICE), 1e-6,
                                     extra=extra.to(DEVICE) if use_extra else None, rows=picked, act_dtype=dtype)
        assert torch.equal(on_device.cpu(), stream)
        assert torch.allclose(got.cpu().double(), want[[4, 0, 8]], atol=tolerance, rtol=tolerance)


# ------------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests_and_first_tokens(folders, name, dtype):
    vocab = GEFARAX[name][0]["vocab"]
    for length, page_size in ((1, 16), (2, 16), (5, 4), (67, 8), (210, 16)):
        tokens = tokens_for(vocab, length, 100 + length)
        records = traces.whole("r", tokens)
        got, _ = run_in_process(folders[name], dtype, records, traces.rounded(length), page_size)
        compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} whole {length}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_against_decoding_one_by_one(folders, name, dtype):
    vocab = GEFARAX[name][0]["vocab"]
    tokens = tokens_for(vocab, 150, 7)
    records = traces.tail_decoded("r", tokens, 40)
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)))
    compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} tail decoded")
    # and from the very first token on, one by one
    short = tokens[:24]
    records = traces.tail_decoded("r", short, 23)
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(short)), page_size=4)
    compare(got, records, {"r": short}, folders[name], dtype, f"{name} decoded from the start")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(folders, name, dtype):
    vocab = GEFARAX[name][0]["vocab"]
    tokens = tokens_for(vocab, 141, 11)
    records = traces.portions("r", tokens, [7, 2, 5, 3, 2, 16, 33, 2, 64, 1, 17])
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
    compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    vocab = GEFARAX[name][0]["vocab"]
    lengths = {"r0": 110, "r1": 67, "r2": 40, "r3": 131, "r4": 64, "r5": 18, "r6": 99}
    requests = {key: tokens_for(vocab, length, 31 + index) for index, (key, length) in enumerate(lengths.items())}
    records, peak = traces.mixed(requests, seed=5)
    got, replayer = run_in_process(folders[name], dtype, records, peak)
    compare(got, records, requests, folders[name], dtype, f"{name} mixed")
    for group in replayer.cache.groups:
        assert group.pool.allocations > group.pool.num_pages, "the trace was meant to reuse pages"
    # every layer run has a cache of its own: a looped layer holds one per pass
    runs = len(replayer.model.spec.schedule)
    assert sum(len(group.entries) for group in replayer.cache.groups) == runs


@pytest.mark.parametrize("name", NAMES)
def test_bfloat16_every_row_when_every_expert_is_chosen(folders, name):
    """With nothing for rounding to turn, every bfloat16 row of a mixed trace and of a decoded tail must agree."""
    folder = folders[name + "/every_expert"]
    vocab = GEFARAX[name][0]["vocab"]
    lengths = {"r0": 90, "r1": 47, "r2": 30, "r3": 101, "r4": 64}
    requests = {key: tokens_for(vocab, length, 61 + index) for index, (key, length) in enumerate(lengths.items())}
    records, peak = traces.mixed(requests, seed=8)
    got, _ = run_in_process(folder, "bfloat16", records, peak)
    want = traces.expected_rows(records, requests, lambda key: plain_logits(folder, requests[key])[0])
    tokens = requests["r3"]
    tail = traces.tail_decoded("r3", tokens, 40)
    got_tail, _ = run_in_process(folder, "bfloat16", tail, traces.rounded(len(tokens)))
    want_tail = traces.expected_rows(tail, {"r3": tokens}, lambda key: plain_logits(folder, tokens)[0])
    for produced, expected in ((got, want), (got_tail, want_tail)):
        assert set(produced) == set(expected)
        for step in expected:
            error = np.abs(produced[step] - expected[step]).max(axis=-1) / np.abs(expected[step]).max(axis=-1)
            assert error.max() <= ALLOWED["bfloat16"], f"{name} step {step}: {error.max():.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    name = "loop_in_the_middle"
    vocab = GEFARAX[name][0]["vocab"]
    tokens = tokens_for(vocab, 300, 3)
    records = traces.tail_decoded("r", tokens, tail=292)
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)))
    compare(got, records, {"r": tokens}, folders[name], dtype, "long decoding")


def test_float32_logits_do_not_depend_on_the_cut(folders):
    name = "loop_from_start"
    vocab = GEFARAX[name][0]["vocab"]
    tokens = tokens_for(vocab, 120, 19)
    other = tokens_for(vocab, 75, 20)
    whole, _ = run_in_process(folders[name], "float32", traces.whole("r", tokens), 128)
    pieces, _ = run_in_process(folders[name], "float32", traces.portions("r", tokens, [3, 2, 40, 1, 1, 9]), 128, page_size=4)
    assert np.array_equal(np.concatenate([pieces[step] for step in sorted(pieces)]), whole[0])
    records, peak = traces.mixed({"r": tokens, "o": other}, seed=2)
    mixed, _ = run_in_process(folders[name], "float32", records, peak)
    fed = 0
    for record in records:
        row = 0
        for entry in record["entries"]:
            for place in entry["want"]:
                if entry["id"] == "r":
                    assert np.array_equal(mixed[record["step"]][row], whole[0][fed + place])
                row += 1
            if entry["id"] == "r":
                fed += len(entry["tokens"])


def test_bfloat16_rows_do_not_depend_on_their_batch(folders):
    """The same request alone and among others: the routed feed-forward, the norms and the products give a row the same
    result whatever shares its step, so the logits agree far more closely than bfloat16 rounding."""
    name = "no_loop"
    vocab = GEFARAX[name][0]["vocab"]
    requests = {"r": tokens_for(vocab, 70, 19), "o": tokens_for(vocab, 45, 20), "p": tokens_for(vocab, 90, 21)}
    alone, _ = run_in_process(folders[name], "bfloat16", traces.whole("r", requests["r"]), 128)
    records, peak = traces.mixed(requests, seed=4)
    mixed, _ = run_in_process(folders[name], "bfloat16", records, peak)
    fed, seen = 0, 0
    for record in records:
        row = 0
        for entry in record["entries"]:
            for place in entry["want"]:
                if entry["id"] == "r":
                    want = alone[0][fed + place]
                    assert np.abs(mixed[record["step"]][row] - want).max() <= 2e-2 * np.abs(want).max()
                    seen += 1
                row += 1
            if entry["id"] == "r":
                fed += len(entry["tokens"])
    assert seen > 20


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """Requests of unequal length through the engine's own scheduler (portions, continuous batching, a pool so small
    that pages come back and are used again): every generated token maximises the plain logits of its own prefix."""
    from llmserver_b200 import Engine
    vocab = GEFARAX[name][0]["vocab"]
    prompts = [tokens_for(vocab, length, 50 + length) for length in (5, 23, 41, 9, 30)]
    engine = Engine(folders[name], max_new_tokens=10, max_batch_size=3, max_num_batched_tokens=32, prefill_chunk_size=12,
                    kv_cache_num_blocks=40, kv_cache_block_size=4, ignore_eos=True, dtype=dtype)
    if name == "tensor_core_sizes":
        engine.warmup()      # products tuned and decode graphs captured ahead of the first request
    generated = engine.generate(prompts)
    assert all(len(tokens) == 10 for tokens in generated)
    for prompt, tokens in zip(prompts, generated):
        logits, margin = plain_logits(folders[name], list(prompt) + list(tokens))
        for index, token in enumerate(tokens):
            at = len(prompt) - 1 + index
            if dtype == "bfloat16" and margin[at] < SAFE_MARGIN:
                break       # from here on the plain implementation may have routed otherwise
            row = logits[at]
            assert row[token] >= row.max() - 2 * ALLOWED[dtype] * np.abs(row).max(), f"token {index} of a prompt of {len(prompt)}"
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()


def test_running_out_of_pages_preempts_and_changes_no_token(folders):
    """A pool too small for all requests: the youngest is put out, its pages (of every pass of the looped layer) come
    back, its cache is rebuilt later; in 32-bit no token changes, and temperature sampling gives the same draws."""
    from llmserver_b200 import Engine
    name = "loop_from_start"
    vocab = GEFARAX[name][0]["vocab"]
    prompts = [tokens_for(vocab, length, 70 + length) for length in (30, 21, 44, 9)]
    roomy = Engine(folders[name], max_new_tokens=40, max_batch_size=4, max_num_batched_tokens=32, kv_cache_num_blocks=128,
                   kv_cache_block_size=4, ignore_eos=True, dtype="float32")
    expected = roomy.generate(prompts, temperature=0.7, seed=3)
    assert roomy.stats["preemptions"] == 0
    tight = Engine(roomy.model, max_new_tokens=40, max_batch_size=4, max_num_batched_tokens=32, kv_cache_num_blocks=48,
                   kv_cache_block_size=4, ignore_eos=True)
    assert tight.generate(prompts, temperature=0.7, seed=3) == expected
    assert tight.stats["preemptions"] > 0
    tight.cache.check_invariants()
    assert tight.cache.available() == tight.cache.capacity()


def test_shared_prefix_pages_serve_every_pass_of_a_loop(folders):
    """Two prompts that begin alike: the second takes the first one's complete pages over in every cache group (each
    pass of a looped layer has pages of its own), computes only its own tail, and still generates the plain
    implementation's tokens."""
    from llmserver_b200 import Engine
    name = "loop_in_the_middle"
    vocab = GEFARAX[name][0]["vocab"]
    shared = tokens_for(vocab, 24, 5)
    prompts = [shared + tokens_for(vocab, 3, 6), shared + tokens_for(vocab, 9, 7)]
    engine = Engine(folders[name], max_new_tokens=5, max_batch_size=2, max_num_batched_tokens=64, kv_cache_num_blocks=32,
                    kv_cache_block_size=8, ignore_eos=True, dtype="float32")
    first = engine.add_request(prompt_token_ids=prompts[0])
    while first.status.value != "Decoding":
        engine.step()
    second = engine.add_request(prompt_token_ids=prompts[1])
    while engine.step():
        pass
    assert engine.stats["prefill_tokens"] == len(prompts[0]) + len(prompts[1]) - 24
    for prompt, request in zip(prompts, (first, second)):
        logits, _ = plain_logits(folders[name], list(prompt) + list(request.generated_token_ids))
        assert request.generated_token_ids == [int(logits[len(prompt) - 1 + index].argmax()) for index in range(5)]
    engine.cache.check_invariants()


def test_trace_run_program(folders, tmp_path):
    name, dtype = "loop_in_the_middle", "float32"
    vocab = GEFARAX[name][0]["vocab"]
    requests = {"x": tokens_for(vocab, 90, 1), "y": tokens_for(vocab, 33, 2), "z": tokens_for(vocab, 130, 3)}
    records, peak = traces.mixed(requests, seed=9, max_live=2)
    out_dir = tmp_path / "out"
    process = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name],
                              "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(peak)],
                             input="\n".join(json.dumps(record) for record in records) + "\n",
                             capture_output=True, text=True, timeout=600)
    assert process.returncode == 0, process.stderr[-2000:]
    assert [line for line in process.stdout.splitlines() if line.startswith("done ")] == [f"done {r['step']}" for r in records]
    got = {}
    for record in records:
        wanted = sum(len(entry["want"]) for entry in record["entries"])
        if wanted:
            got[record["step"]] = np.fromfile(out_dir / f"{record['step']}.f32", dtype="<f4").reshape(wanted, vocab)
    compare(got, records, requests, folders[name], dtype, f"trace_run {name}")


def test_generate_command(folders):
    """The command line a user generates with: ids in, ids out, the model chosen by its config.json."""
    name = "no_loop"
    vocab = GEFARAX[name][0]["vocab"]
    prompts = [tokens_for(vocab, 19, 71), tokens_for(vocab, 3, 72)]
    command = [sys.executable, "-m", "llmserver_b200.cli.generate", "--model", folders[name], "--dtype", "float32",
               "--max-new-tokens", "6", "--ignore-eos", "--block-size", "8", "--json"]
    for prompt in prompts:
        command += ["--prompt-ids", ",".join(str(token) for token in prompt)]
    process = subprocess.run(command, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert process.returncode == 0, process.stderr[-2000:]
    generated = json.loads(process.stdout.strip().splitlines()[-1])["generated"]
    for prompt, tokens in zip(prompts, generated):
        assert len(tokens) == 6
        logits, _ = plain_logits(folders[name], list(prompt) + list(tokens))
        assert tokens == [int(logits[len(prompt) - 1 + index].argmax()) for index in range(6)]
