"""Dikusun on the GPU against the plain implementation in plain_dikusun.py: each mechanism alone, then whole models
through the step function, the cache and the scheduler, cut and batched in different ways, in 32-bit and bfloat16."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_dikusun as plain
import traces
from dikusun_configs import DIKUSUN
from helpers import tokens_for

pytestmark = pytest.mark.gpu

DEVICE = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = sorted(DIKUSUN)
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F64 = torch.float64
# Largest allowed |engine - plain| as a fraction of the row's largest |plain logit|.  bfloat16: besides the activations
# between kernels, every sub-layer reads the 32-bit stream itself rounded to 8 significant bits (there is no norm in
# front that would bring it to unit size first), and the weights here are drawn for peaked attention and long memories.
ALLOWED = {"float32": 2e-5, "bfloat16": 6e-2}


# ------------------------------------------------------------------------------------------------ model folders
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Model folders with random weights, redrawn where the generic random mode would hide a fault: query and key
    projections large enough for peaked attention, decays that keep state for hundreds of tokens in some channels and
    lose it at once in others, biases and lambda vectors far from zero."""
    from safetensors.torch import load_file, save_file

    import llmserver_b200.models  # noqa: F401
    from llmserver_b200.config import DikusunConfig
    from llmserver_b200.weights import write_model_folder

    root = tmp_path_factory.mktemp("dikusun")
    made = {}
    for name, (raw, seed) in DIKUSUN.items():
        folder = write_model_folder(DikusunConfig.from_dict(raw), str(root / name), seed, torch.bfloat16)
        path = os.path.join(folder, "model.safetensors")
        tensors = load_file(path)
        generator = torch.Generator().manual_seed(seed)
        width = raw["width"]
        for key in sorted(tensors):
            shape = tensors[key].shape

            def draw(deviation):
                return (torch.randn(shape, generator=generator) * deviation).to(torch.bfloat16)
            if key.endswith((".mix.q", ".mix.k", ".mix.dq", ".mix.dkv")):
                tensors[key] = draw(2.0 / math.sqrt(shape[1]))
            elif key.endswith((".mix.uq", ".mix.uk")):       # scores a few units apart: peaked, yet not an argmax
                tensors[key] = draw(1.5 / math.sqrt(shape[1]))
            elif key.endswith((".mix.v", ".mix.uv", ".mix.g", ".mix.o", ".mix.a1", ".mix.a2", ".mlp.gate", ".mlp.up", ".mlp.down", "head")):
                tensors[key] = draw(1.0 / math.sqrt(shape[1]))
            elif key.endswith(".b") and ".a2" not in key:
                tensors[key] = draw(0.5)
            elif key.endswith(".a2.b"):
                tensors[key] = (torch.linspace(-2.0, 7.0, shape[0]) + torch.randn(shape, generator=generator) * 0.3).to(torch.bfloat16)
            elif key.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
                tensors[key] = draw(0.3)
            elif key == "embed":
                tensors[key] = draw(1.0)
        save_file(tensors, path)
        made[name] = folder
    return made


_PLAIN, _LOGITS = {}, {}


def plain_model_of(folder):
    if folder not in _PLAIN:
        from safetensors.torch import load_file
        with open(os.path.join(folder, "config.json")) as handle:
            config = json.load(handle)
        _PLAIN[folder] = (config, {key: value.to(F64) for key, value in load_file(os.path.join(folder, "model.safetensors")).items()})
    return _PLAIN[folder]


def plain_logits(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _LOGITS:
        config, weights = plain_model_of(folder)
        _LOGITS[key] = plain.forward(config, weights, list(tokens)).numpy()
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
    """32-bit: every row within the allowance.  bfloat16: a row whose head outputs nearly cancel before they are
    normalised (the first tokens of a linear-attention layer, whose state holds one or two keys) amplifies rounding, so
    up to one row in fifty may exceed the allowance, none by more than twice."""
    want = traces.expected_rows(records, requests, lambda name: plain_logits(folder, requests[name]))
    assert set(got) == set(want), f"{what}: steps with logits differ"
    errors = []
    for step in sorted(want):
        assert got[step].shape == want[step].shape and np.isfinite(got[step]).all(), f"{what} step {step}"
        scale = np.abs(want[step]).max(axis=-1)
        errors += [(float(e), step, row) for row, e in enumerate(np.abs(got[step] - want[step]).max(axis=-1) / scale)]
    worst, step, row = max(errors)
    over = sum(1 for error, _, _ in errors if error > ALLOWED[dtype])
    hard = ALLOWED[dtype] if dtype == "float32" else 2 * ALLOWED[dtype]
    assert worst <= hard, f"{what} step {step}: row {row} differs by {worst:.3e} of its largest logit, allowed {hard:.1e}"
    assert dtype != "float32" or over == 0
    assert over <= max(1, len(errors) // 50), f"{what}: {over} of {len(errors)} rows differ by more than {ALLOWED[dtype]:.1e}"


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_scaled_embedding():
    from llmserver_b200 import ops
    table = torch.randn((50, 24), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    for scale in (1.0, 0.3, 11.0):
        got = ops.embedding(table.to(DEVICE), ids.to(DEVICE), scale=scale)
        assert torch.equal(got.cpu(), table.float()[ids.long()] * torch.tensor(scale, dtype=torch.float32))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 96, 1000])
def test_output_norm_add_and_stream_read(dtype, width):
    """What stands between two sub-layers of an output-norm block: the pending output (plus its projection's bias) is
    normalised, weighted and added to the 32-bit stream, and the updated stream itself comes back as the next input."""
    from llmserver_b200 import ops
    generator = torch.Generator().manual_seed(width)
    stream = torch.randn((7, width), generator=generator)
    delta = (torch.randn((7, width), generator=generator) * 3).to(dtype)
    bias = torch.randn((width,), generator=generator)
    weight = (1 + 0.1 * torch.randn((width,), generator=generator)).to(dtype)
    for use_bias in (False, True):
        d = delta.double() + (bias.double() if use_bias else 0)
        want = stream.double() + plain.rms_norm(d, weight.double(), 1e-5)
        on_device = stream.clone().to(DEVICE)
        out = ops.normed_add_rmsnorm(on_device, delta.to(DEVICE), weight.to(DEVICE), 1e-5, None, 0.0, act_dtype=dtype,
                                     delta_bias=bias.to(DEVICE) if use_bias else None)
        assert torch.allclose(on_device.cpu().double(), want, atol=2e-6, rtol=2e-6)      # the stream stays 32-bit
        assert torch.equal(out.cpu(), on_device.cpu().to(dtype))                         # and is read as it is
    untouched = stream.clone().to(DEVICE)
    out = ops.normed_add_rmsnorm(untouched, None, None, 0.0, None, 0.0, act_dtype=dtype)
    assert torch.equal(untouched.cpu(), stream) and torch.equal(out.cpu(), stream.to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,maps,q_dim,k_dim,vdim,dims,extra", [
    (4, 2, 2, 16, 16, 24, 8, 4), (3, 1, 2, 24, 24, 40, 24, 3), (2, 2, 2, 8, 8, 8, 0, 0), (1, 1, 1, 72, 40, 0, 0, 0),
    (5, 5, 1, 64, 64, 16, 6, 0), (2, 1, 2, 128, 128, 64, 64, 2)])
def test_bias_unit_norms_rotation_and_cache_write(dtype, heads, kv_heads, maps, q_dim, k_dim, vdim, dims, extra):
    from llmserver_b200 import ops
    generator = torch.Generator().manual_seed(q_dim + vdim)
    page_size, pages = 4, 12
    # two sequences: positions 5..10 of one (it crosses a page border) and positions 0..2 of another
    positions = torch.tensor([5, 6, 7, 8, 9, 10, 0, 1, 2], dtype=torch.int32)
    seq = torch.tensor([0] * 6 + [1] * 3, dtype=torch.int32)
    tables = torch.tensor([[7, 3, 9], [2, 0, 0]], dtype=torch.int32)
    q_cols, k_cols, v_cols = heads * maps * q_dim, kv_heads * maps * k_dim, kv_heads * vdim
    packed = torch.randn((len(positions), q_cols + k_cols + v_cols + extra), generator=generator).to(dtype)
    bias = torch.randn((q_cols + k_cols + v_cols,), generator=generator)
    q_weight = (1 + 0.2 * torch.randn((q_dim,), generator=generator)).to(dtype)
    k_weight = (1 + 0.2 * torch.randn((k_dim,), generator=generator)).to(dtype)
    rot = {"base": 1000.0, "dims": dims} if dims else None
    inv_freq = torch.tensor([1000.0 ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32).to(DEVICE) if dims else None
    for use_bias, use_norm, packed_out in ((True, True, False), (False, True, True), (True, False, False), (False, False, True)):
        k_pages = torch.zeros((pages, kv_heads, page_size, maps * k_dim), dtype=dtype, device=DEVICE)
        v_pages = torch.zeros((pages, kv_heads, page_size, vdim), dtype=dtype, device=DEVICE) if vdim else None
        flag = torch.zeros(1, dtype=torch.int32, device=DEVICE)
        on_device = packed.to(DEVICE)
        q_out = torch.zeros((len(positions), q_cols), dtype=dtype, device=DEVICE) if packed_out else None
        ops.norm_rope_units(on_device, positions.to(DEVICE), seq.to(DEVICE), tables.to(DEVICE), k_pages, v_pages, heads, kv_heads,
                            maps, q_dim, k_dim, vdim, flag, bias=bias.to(DEVICE) if use_bias else None,
                            q_weight=q_weight.to(DEVICE) if use_norm else None, k_weight=k_weight.to(DEVICE) if use_norm else None,
                            eps=1e-5, inv_freq=inv_freq, rotary_dim=dims, q_out=q_out)
        assert int(flag.item()) == 0
        source = packed.double()[:, :q_cols + k_cols + v_cols] + (bias.double() if use_bias else 0)
        q = source[:, :q_cols].view(-1, heads * maps, q_dim)
        k = source[:, q_cols:q_cols + k_cols].view(-1, kv_heads * maps, k_dim)
        if use_norm:
            q, k = plain.rms_norm(q, q_weight.double(), 1e-5), plain.rms_norm(k, k_weight.double(), 1e-5)
        q, k = plain.rotate(q, positions, rot), plain.rotate(k, positions, rot)
        v = source[:, q_cols + k_cols:].reshape(len(positions), kv_heads, vdim)
        tolerance = 2e-5 if dtype == torch.float32 else 3e-2
        got_q = (q_out if packed_out else on_device[:, :q_cols]).cpu().double()
        assert torch.allclose(got_q.view(-1, heads * maps, q_dim), q, atol=tolerance, rtol=tolerance)
        if extra:      # columns behind the values are nobody's business
            assert torch.equal(on_device[:, -extra:].cpu(), packed[:, -extra:])
        want_k = torch.zeros(k_pages.shape, dtype=F64)
        want_v = torch.zeros((pages, kv_heads, page_size, vdim), dtype=F64)
        for token in range(len(positions)):
            page = int(tables[seq[token], positions[token] // page_size])
            want_k[page, :, positions[token] % page_size] = k[token].reshape(kv_heads, maps * k_dim)
            want_v[page, :, positions[token] % page_size] = v[token]
        assert torch.allclose(k_pages.cpu().double(), want_k, atol=tolerance, rtol=tolerance)   # untouched slots stay zero
        if vdim:
            assert torch.allclose(v_pages.cpu().double(), want_v, atol=tolerance, rtol=tolerance)


def _differential_case(dtype, heads, kv_heads, dim, vdim, lengths, queries, page_size, seed, spike=None):
    """Random two-map keys and values of sequences of ``lengths`` tokens in shuffled pages; ``queries``: (sequence,
    position) pairs.  ``spike`` = (query index, key position, map): that query's and that key's units of the map are
    scaled so that their score stands out."""
    generator = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-length // page_size) for length in lengths) + 3
    order = torch.randperm(n_pages, generator=generator).tolist()
    width = max(-(-length // page_size) for length in lengths)
    tables = torch.zeros((len(lengths), width), dtype=torch.int32)
    keys = [torch.randn((length, kv_heads, 2, dim), generator=generator).to(dtype) for length in lengths]
    values = [torch.randn((length, kv_heads, vdim), generator=generator).to(dtype) for length in lengths]
    q = torch.randn((len(queries), heads, 2, dim), generator=generator).to(dtype)
    gate = torch.randn((len(queries), heads), generator=generator).to(dtype)
    if spike is not None:
        index, position, which = spike
        direction = torch.randn((dim,), generator=generator)
        direction = direction / direction.norm()
        length = math.sqrt(14.0 * math.sqrt(dim))       # a score of 14 after the scale
        q[index, :, which] = (direction * length).to(dtype)
        keys[queries[index][0]][position, :, which] = (direction * length).to(dtype)
    k_pages = torch.zeros((n_pages, kv_heads, page_size, 2 * dim), dtype=dtype)
    v_pages = torch.zeros((n_pages, kv_heads, page_size, vdim), dtype=dtype)
    for sequence, length in enumerate(lengths):
        for block in range(-(-length // page_size)):
            page = order.pop()
            tables[sequence, block] = page
            rows = slice(block * page_size, min(length, (block + 1) * page_size))
            count = rows.stop - rows.start
            k_pages[page, :, :count] = keys[sequence][rows].reshape(count, kv_heads, 2 * dim).transpose(0, 1)
            v_pages[page, :, :count] = values[sequence][rows].transpose(0, 1)
    return q, gate, keys, values, k_pages, v_pages, tables


def _differential_plain(q, gate, keys, values, queries, heads, kv_heads, scale, cap, window, lam, eps, out_scale, use_gate):
    out = torch.zeros((len(queries), heads, values[0].shape[-1]), dtype=F64)
    weights_of_maps = []
    for index, (sequence, position) in enumerate(queries):
        first = max(0, position - window + 1) if window else 0
        row = []
        for head in range(heads):
            group = head // (heads // kv_heads)
            maps = []
            for m in range(2):
                scores = (keys[sequence][first:position + 1, group, m].double() @ q[index, head, m].double()) * scale
                if cap:
                    scores = cap * torch.tanh(scores / cap)
                p = torch.softmax(scores, dim=0)
                maps.append(p @ values[sequence][first:position + 1, group].double())
                row.append((first, p))
            o = plain.rms(maps[0] - lam * maps[1], eps) * out_scale
            out[index, head] = o * (torch.sigmoid(gate[index, head].double()) if use_gate else 1.0)
        weights_of_maps.append(row)
    return out.reshape(len(queries), -1), weights_of_maps


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,cap", [(4, 2, 16, 24, 9, 20.0), (6, 1, 24, 40, 0, 0.0), (2, 2, 64, 64, 33, 50.0),
                                                                (8, 2, 128, 128, 0, 30.0), (3, 3, 8, 80, 1, 0.0), (4, 1, 64, 128, 100, 0.0)])
def test_differential_attention_kernel(dtype, heads, kv_heads, dim, vdim, window, cap):
    """Prompt rows and single decoded rows side by side, sequences of unequal length, keys found through shuffled pages.
    One query's score for one key towers over the rest in one of the maps: a key far back where there is no window,
    the first key inside the window (it must carry the row) and the key just outside it (it must not be seen)."""
    from llmserver_b200 import ops
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    page_size = 8
    lengths = [300, 41, 1, 130]
    new_tokens = [1, 41, 1, 30]
    queries = [(s, p) for s, (length, count) in enumerate(zip(lengths, new_tokens)) for p in range(length - count, length)]
    last = 299
    inside = last - window + 1 if window else 7        # without a window: a far key in the last slot of a page
    spikes = [(0, inside, 0), (0, inside, 1), None]
    if window > 1:
        spikes.append((0, inside - 1, 0))              # just outside
    lam, eps, out_scale, scale = 0.37, 1e-5, 0.7, 1.0 / math.sqrt(dim)
    for spike in spikes:
        q, gate, keys, values, k_pages, v_pages, tables = _differential_case(dtype, heads, kv_heads, dim, vdim, lengths, queries,
                                                                             page_size, 29, spike)
        slices = [SequenceSlice(f"r{s}", [0] * count, length - count, [], [tables[s, :-(-length // page_size)].tolist()], 0)
                  for s, (length, count) in enumerate(zip(lengths, new_tokens))]
        batch = build_batch(slices, 1, DEVICE)
        q_cols = heads * 2 * dim
        for use_gate in (True, False):
            packed = torch.zeros((len(queries), -(-(q_cols + 24 + heads) // 8) * 8), dtype=dtype)
            packed[:, :q_cols] = q.reshape(len(queries), q_cols)
            packed[:, q_cols + 24:q_cols + 24 + heads] = gate
            want, maps = _differential_plain(q, gate, keys, values, queries, heads, kv_heads, scale, cap, window, lam, eps, out_scale, use_gate)
            out = ops.attention_diff(packed.to(DEVICE), q_cols + 24 if use_gate else None, batch, batch.block_tables[0],
                                     k_pages.to(DEVICE), v_pages.to(DEVICE), heads, kv_heads, dim, vdim, scale, cap, window, lam,
                                     eps, out_scale)
            tolerance = 3e-5 if dtype == torch.float32 else 2e-2
            assert torch.allclose(out.cpu().double(), want, atol=tolerance, rtol=tolerance), f"spike {spike}, gate {use_gate}"
        if spike is not None and window != 1:
            first, p = maps[0][spike[2]]
            if spike[1] >= first:
                assert float(p[spike[1] - first]) > 0.9      # the spiked key really carries the row of its map
            else:
                assert float(p.max()) < 0.9                  # outside the window it is not there at all


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,cap", [(4, 2, 64, 64, 70, 40.0), (8, 1, 64, 128, 0, 0.0), (6, 2, 128, 128, 300, 50.0),
                                                                (3, 3, 128, 64, 1000, 0.0), (32, 2, 64, 64, 17, 0.0)])
def test_tiled_differential_attention_kernel(heads, kv_heads, dim, vdim, window, cap):
    """The bfloat16 kernel on the tensor cores against the plain implementation and against the kernel that takes every
    size: a whole prompt, a portion behind cached tokens, single decoded tokens of short contexts and of a long one, all
    in one batch, and a batch of single tokens alone (the launch shape of a decode step); keys through shuffled pages
    that do not align with the kernel's tiles.  One decoded query's score for the first key inside its window (or, with
    no window, for a key far back) towers over the rest, so weights rounded to 8 bits would not pass either."""
    from llmserver_b200 import ops
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    from llmserver_b200.ops import attention_bf16
    from llmserver_b200.ops.library import check_wait_errors, launch_count
    page_size = 16 if dim == 64 else 24
    lengths = [300, 41, 1, 130, 2500]
    lam, eps, out_scale, scale = 0.41, 1e-6, 0.8, 1.0 / math.sqrt(dim)
    for new_tokens in ([1, 41, 1, 30, 1], [1, 1, 1, 1, 1]):
        queries = [(s, p) for s, (length, count) in enumerate(zip(lengths, new_tokens)) for p in range(length - count, length)]
        last_query = len(queries) - 1
        inside = 2499 - window + 1 if window else 15
        for spike in ((last_query, inside, 0), (last_query, inside, 1), (last_query, inside - 1, 1) if window else None, None):
            q, gate, keys, values, k_pages, v_pages, tables = _differential_case(torch.bfloat16, heads, kv_heads, dim, vdim, lengths,
                                                                                 queries, page_size, 31, spike)
            slices = [SequenceSlice(f"r{s}", [0] * count, length - count, [], [tables[s, :-(-length // page_size)].tolist()], 0)
                      for s, (length, count) in enumerate(zip(lengths, new_tokens))]
            batch = build_batch(slices, 1, DEVICE)
            q_cols = heads * 2 * dim
            packed = torch.zeros((len(queries), -(-(q_cols + 8 + heads) // 8) * 8), dtype=torch.bfloat16)
            packed[:, :q_cols] = q.reshape(len(queries), q_cols)
            packed[:, q_cols + 8:q_cols + 8 + heads] = gate
            want, maps = _differential_plain(q, gate, keys, values, queries, heads, kv_heads, scale, cap, window, lam, eps, out_scale, True)
            got = {}
            for kernel in ("mma", "generic"):
                before, attention_bf16.DIFF_KERNEL = attention_bf16.DIFF_KERNEL, kernel
                try:
                    got[kernel] = ops.attention_diff(packed.to(DEVICE), q_cols + 8, batch, batch.block_tables[0], k_pages.to(DEVICE),
                                                     v_pages.to(DEVICE), heads, kv_heads, dim, vdim, scale, cap, window, lam, eps,
                                                     out_scale).cpu().double()
                finally:
                    attention_bf16.DIFF_KERNEL = before
            torch.cuda.synchronize()
            check_wait_errors()
            for kernel, out in got.items():
                error = (out - want).abs().max(dim=-1).values / want.abs().max(dim=-1).values.clamp_min(0.05)
                assert error.max() < 1e-2, f"{kernel}, spike {spike}: row {int(error.argmax())} of {len(queries)} differs by {float(error.max()):.2e}"
            if spike is not None and window != 1:
                first, p = maps[last_query][spike[2]]
                assert (float(p[spike[1] - first]) > 0.9) if spike[1] >= first else (float(p.max()) < 0.9)
    # the tiled kernel really took these sizes (rows of the packed projection are 16-byte aligned here)
    from llmserver_b200.ops.library import library
    assert library().llm_attention_diff_mma_supports(dim, vdim, heads, kv_heads) and packed.shape[1] % 8 == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,rows,inner,tokens", [(3, 40, 16, 5), (5, 16, 72, 1), (4, 128, 32, 70), (8, 64, 128, 33), (2, 7, 9, 12)])
def test_per_head_products(dtype, heads, rows, inner, tokens):
    from llmserver_b200 import ops
    generator = torch.Generator().manual_seed(rows + inner)
    x = torch.randn((tokens, heads * inner), generator=generator).to(dtype)
    weight = (torch.randn((heads, rows, inner), generator=generator) / math.sqrt(inner)).to(dtype)
    want = torch.einsum("thk,hrk->thr", x.double().view(tokens, heads, inner), weight.double()).reshape(tokens, heads * rows)
    got = ops.head_linear(x.to(DEVICE), weight.to(DEVICE))
    tolerance = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got.cpu().double(), want, atol=tolerance, rtol=tolerance)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim,tau", [(2, 24, 40, 8.0), (5, 8, 16, 1.0), (1, 72, 33, 32.0), (2, 64, 128, 16.0), (3, 128, 64, 4.0),
                                                (1, 200, 96, 16.0), (2, 16, 256, 2.0), (1, 256, 256, 8.0), (2, 200, 160, 3.0)])
def test_gated_linear_attention_kernel(dtype, heads, dim, vdim, tau):
    """Three sequences in one step: one continues from a state that an earlier step left (in another slot order), one
    starts from zero, one is a single token.  Decays run from 'forgets at once' to 'keeps for hundreds of tokens'; the
    state behind the step is compared too."""
    from llmserver_b200 import ops
    from llmserver_b200.engine.batch import SequenceSlice, build_batch
    generator = torch.Generator().manual_seed(dim * 7 + vdim)
    keys, values = heads * dim, heads * vdim
    lengths = [(0, 37), (19, 11), (45, 1)]            # (tokens before this step, tokens of this step)
    total = [before + now for before, now in lengths]
    proj = [torch.randn((count, 2 * keys + 2 * values + 5), generator=generator).to(dtype) for count in total]
    z = [torch.randn((count, keys), generator=generator) * 2 for count in total]
    z_bias = torch.linspace(-2.0, 7.0, keys)
    weight = (1 + 0.2 * torch.randn((vdim,), generator=generator)).to(dtype)
    q_scale, eps = dim ** -0.5, 1e-5
    columns = (5, 5 + keys, 5 + 2 * keys, 5 + 2 * keys + values)

    def plain_run(sequence, count):
        p, zz = proj[sequence].double(), z[sequence].double() + z_bias.double()
        alpha = (torch.sigmoid(zz) ** (1.0 / tau)).view(-1, heads, dim)
        q = p[:, columns[0]:columns[0] + keys].view(-1, heads, dim) * q_scale
        k = p[:, columns[1]:columns[1] + keys].view(-1, heads, dim)
        v = p[:, columns[2]:columns[2] + values].view(-1, heads, vdim)
        g = p[:, columns[3]:columns[3] + values]
        S = torch.zeros((heads, dim, vdim), dtype=F64)
        out = torch.zeros((count, heads, vdim), dtype=F64)
        for t in range(count):
            S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, q[t])
        out = plain.rms_norm(out, weight.double(), eps).reshape(count, values) * (g[:count] * torch.sigmoid(g[:count]))
        return out, S

    slots = [2, 0, 3]
    tolerance = 2e-5 if dtype == torch.float32 else 2e-2
    # segment 0: one pass over a sequence's tokens; 8 and 16: the form that walks segments in parallel (here 5, 2 and 1
    # segments, or 3, 1 and 1), which must agree to rounding
    for segment in (0, 8, 16):
        state = torch.zeros((4, heads, dim, vdim), dtype=torch.float32, device=DEVICE)
        state[1] = 7.0          # nobody's slot: must stay as it is
        # the step before: sequences 1 and 2 run their earlier tokens (sequence 2 first, to change the slot order)
        earlier = [(2, lengths[2][0]), (1, lengths[1][0])]
        batch = build_batch([SequenceSlice(f"r{s}", [0] * count, 0, [], [[0]], slots[s]) for s, count in earlier], 1, DEVICE)
        rows = torch.cat([proj[s][:count] for s, count in earlier]).to(DEVICE)
        ops.gla_recurrent(rows, *columns, torch.cat([z[s][:count] for s, count in earlier]).to(DEVICE), z_bias.to(DEVICE),
                          weight.to(DEVICE), state, batch, heads, dim, vdim, tau, q_scale, eps, segment=segment)
        # this step
        batch = build_batch([SequenceSlice(f"r{s}", [0] * now, before, [], [[0]], slots[s]) for s, (before, now) in enumerate(lengths)], 1, DEVICE)
        rows = torch.cat([proj[s][before:] for s, (before, _) in enumerate(lengths)]).to(DEVICE)
        got = ops.gla_recurrent(rows, *columns, torch.cat([z[s][before:] for s, (before, _) in enumerate(lengths)]).to(DEVICE),
                                z_bias.to(DEVICE), weight.to(DEVICE), state, batch, heads, dim, vdim, tau, q_scale, eps,
                                segment=segment).cpu().double()
        at = 0
        for s, (before, now) in enumerate(lengths):
            want, last = plain_run(s, before + now)
            assert torch.allclose(got[at:at + now], want[before:], atol=tolerance, rtol=tolerance), f"sequence {s}, segment {segment}"
            assert torch.allclose(state[slots[s]].cpu().double(), last, atol=2e-4, rtol=2e-4), f"state of sequence {s}, segment {segment}"
            at += now
        assert bool((state[1] == 7.0).all())


# ------------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt_and_token_by_token(folders, name, dtype):
    vocab = DIKUSUN[name][0]["vocab"]
    tokens = tokens_for(vocab, 203, 7)
    records = traces.whole("r", tokens)
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)))
    compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} whole")
    records = traces.tail_decoded("r", tokens, 60)      # the windows of these models pass over decoded tokens
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
    compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} tail decoded")
    short = tokens[:30]                                 # and from the very first token on, one by one
    records = traces.tail_decoded("r", short, 29)
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(short)), page_size=4)
    compare(got, records, {"r": short}, folders[name], dtype, f"{name} decoded from the start")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(folders, name, dtype):
    vocab = DIKUSUN[name][0]["vocab"]
    tokens = tokens_for(vocab, 181, 11)
    records = traces.portions("r", tokens, [7, 2, 5, 3, 2, 16, 33, 2, 64, 1, 17])
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)), page_size=8)
    compare(got, records, {"r": tokens}, folders[name], dtype, f"{name} portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    vocab = DIKUSUN[name][0]["vocab"]
    lengths = {"r0": 110, "r1": 67, "r2": 40, "r3": 131, "r4": 64, "r5": 18, "r6": 99}
    requests = {key: tokens_for(vocab, length, 31 + index) for index, (key, length) in enumerate(lengths.items())}
    records, peak = traces.mixed(requests, seed=5)
    got, replayer = run_in_process(folders[name], dtype, records, peak)
    compare(got, records, requests, folders[name], dtype, f"{name} mixed")
    for group in replayer.cache.groups:
        if group.window is None:
            assert group.pool.allocations > group.pool.num_pages, "the trace was meant to reuse pages"
    # seven requests went through four state slots
    assert replayer.cache.slots.num_slots == 4 and len(replayer.cache.slots.free) == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    name = "all_kinds"
    vocab = DIKUSUN[name][0]["vocab"]
    tokens = tokens_for(vocab, 330, 3)
    records = traces.tail_decoded("r", tokens, tail=322)
    got, _ = run_in_process(folders[name], dtype, records, traces.rounded(len(tokens)))
    compare(got, records, {"r": tokens}, folders[name], dtype, "long decoding")


def test_a_lost_state_or_a_window_one_token_off_would_show(folders):
    """The plain implementation with the recurrent state dropped at a portion's start, or with windows one token longer,
    gives logits far outside the allowance: the models of these tests do not hide such faults."""
    import copy
    for name in ("gla_only", "all_kinds", "attention_only"):
        config, weights = plain_model_of(folders[name])
        tokens = tokens_for(config["vocab"], 90, 13)
        want = plain_logits(folders[name], tokens)
        scale = np.abs(want).max(axis=-1)
        if name != "attention_only":
            lost = plain.forward(config, weights, tokens[60:]).numpy()       # the state of the first 60 tokens is gone
            assert (np.abs(lost - want[60:]).max(axis=-1) / scale[60:]).max() > 10 * ALLOWED["bfloat16"]
        if name != "gla_only":
            longer = copy.deepcopy(config)
            for layer in longer["layers"]:
                if layer["type"] == "attention" and layer["mixer"].get("mask"):
                    layer["mixer"]["mask"]["size"] += 1
            off = plain.forward(longer, weights, tokens).numpy()
            assert (np.abs(off - want).max(axis=-1) / scale).max() > 2 * ALLOWED["bfloat16"]


def test_float32_logits_do_not_depend_on_the_cut(folders):
    name = "all_kinds"
    vocab = DIKUSUN[name][0]["vocab"]
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
    name = "tensor_core_sizes"
    vocab = DIKUSUN[name][0]["vocab"]
    requests = {"r": tokens_for(vocab, 170, 19), "o": tokens_for(vocab, 45, 20), "p": tokens_for(vocab, 90, 21)}
    alone, _ = run_in_process(folders[name], "bfloat16", traces.whole("r", requests["r"]), 192)
    records, peak = traces.mixed(requests, seed=4)
    mixed, _ = run_in_process(folders[name], "bfloat16", records, peak)
    fed, seen = 0, 0
    for record in records:
        row = 0
        for entry in record["entries"]:
            for place in entry["want"]:
                if entry["id"] == "r":
                    want = alone[0][fed + place]
                    assert np.abs(mixed[record["step"]][row] - want).max() <= 3e-2 * np.abs(want).max()
                    seen += 1
                row += 1
            if entry["id"] == "r":
                fed += len(entry["tokens"])
    assert seen > 20


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_engine(folders, name, dtype):
    """Requests of unequal length through the engine's own scheduler (portions, continuous batching, a pool so small
    that pages come back and are used again, fewer state slots than requests): every generated token maximises the
    plain logits of its own prefix."""
    from llmserver_b200 import Engine
    vocab = DIKUSUN[name][0]["vocab"]
    prompts = [tokens_for(vocab, length, 50 + length) for length in (5, 23, 41, 9, 30)]
    engine = Engine(folders[name], max_new_tokens=10, max_batch_size=3, max_num_batched_tokens=32, prefill_chunk_size=12,
                    kv_cache_num_blocks=40, kv_cache_block_size=4, ignore_eos=True, dtype=dtype)
    if name == "tensor_core_sizes":
        engine.warmup()      # products tuned and decode graphs captured ahead of the first request
    generated = engine.generate(prompts)
    assert all(len(tokens) == 10 for tokens in generated)
    for prompt, tokens in zip(prompts, generated):
        logits = plain_logits(folders[name], list(prompt) + list(tokens))
        for index, token in enumerate(tokens):
            row = logits[len(prompt) - 1 + index]
            assert row[token] >= row.max() - 2 * ALLOWED[dtype] * np.abs(row).max(), f"token {index} of a prompt of {len(prompt)}"
    engine.cache.check_invariants()
    assert engine.cache.available() == engine.cache.capacity()


def test_trace_run_program(folders, tmp_path):
    name, dtype = "all_kinds", "float32"
    vocab = DIKUSUN[name][0]["vocab"]
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
    name = "all_kinds"
    vocab = DIKUSUN[name][0]["vocab"]
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
        logits = plain_logits(folders[name], list(prompt) + list(tokens))
        assert tokens == [int(logits[len(prompt) - 1 + index].argmax()) for index in range(6)]
