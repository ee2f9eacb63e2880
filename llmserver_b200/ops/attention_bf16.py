"""bfloat16 tensor-core attention kernels over the paged cache (prompt portions and split-KV decode).

``try_attention`` returns None when the tensor-core kernels do not take the sizes; the caller then
uses the generic 32-bit-arithmetic kernel, which takes every size."""
from __future__ import annotations

import os

import torch

from .library import call, check, library, stream_handle, wait_error_flag

TILE = 64          # rows per block of the portions kernel, keys per tile of both kernels
MIN_SPLIT = 192    # fewest keys one decode block walks
DECODE_BLOCKS_PER_SM = 2    # blocks of the decode kernel an SM holds at a time (shared memory)
# Up to this many splits of a sequence form a thread-block cluster and merge their results in shared memory; more go
# through scratch memory and a merge kernel (as do all, with LLMSERVER_B200_DECODE_MERGE=kernel).
CLUSTER_MERGE = os.environ.get("LLMSERVER_B200_DECODE_MERGE", "cluster") != "kernel"
MAX_CLUSTER_SPLITS = 8
# With so few (sequence, kv head) pairs that 16 blocks each still leave every block an SM of its own (batch 1 of the
# 8B shape), clusters of 16 (beyond the portable size, which the hardware allows on request) get each block's keys in
# flight at once: 3.21 against 3.25 ms per batch-1 step.  With more pairs they are slower (batch 2: 3.49 against 3.30).
WIDE_CLUSTER_SPLITS = 16


# "tcgen05": the 256-row kernel for long portions and the 128-row kernel otherwise; "tcgen05-128" / "tcgen05-256":
# always that kernel; "mma": the mma.sync kernel
PREFILL_KERNEL = os.environ.get("LLMSERVER_B200_PREFILL_ATTENTION", "tcgen05")
PREFILL_TILE = 128   # rows per block of the tcgen05 portions kernel
WIDE_TILE = 256      # rows per block of the 256-row kernel
# the 256-row kernel is used when the longest portion has this many rows (tokens x heads of a group), its request
# holds this many tokens and the group divides 128: measured on the 8B, 14B and 32B head shapes, it wins from about
# there (long key loops, enough row tiles; 8 % at 16384 tokens, 25 % at 32768), and not with groups of 5
WIDE_MIN_ROWS = int(os.environ.get("LLMSERVER_B200_PREFILL_WIDE_ROWS", "8192"))
WIDE_MIN_CONTEXT = int(os.environ.get("LLMSERVER_B200_PREFILL_WIDE_CONTEXT", "16384"))


def prefill_tcgen05_supported(head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int) -> bool:
    return PREFILL_KERNEL.startswith("tcgen05") and bool(
        library().llm_attention_prefill_tcgen05_supports(head_dim, n_q_heads, n_kv_heads, page_size))


FORCE_PAIRING = None     # True / False: tests set it to run both ways of handing out row tiles
_SM_COUNT = {}


def _sm_count(device) -> int:
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SM_COUNT[index]


def _block_slots(device, wide: bool) -> int:
    """Blocks of a prompt kernel the GPU holds at a time (one per SM for the 256-row kernel, two for the 128-row one)."""
    return _sm_count(device) * (1 if wide else 2)


def prefill_wide_wanted(batch, group: int, head_dim: int, n_q_heads: int, n_kv_heads: int, page_size: int) -> bool:
    """Whether the prompt portions of this batch go to the 256-row kernel: when the longest of them has enough
    rows and keys, or when asked for."""
    if PREFILL_KERNEL == "tcgen05-128":
        return False
    if not library().llm_attention_prefill_wide_supports(head_dim, n_q_heads, n_kv_heads, page_size):
        return False
    if PREFILL_KERNEL == "tcgen05-256":
        return True
    length, context = max(zip(batch.q_lens, batch.context_lens))
    return length * group >= WIDE_MIN_ROWS and context >= WIDE_MIN_CONTEXT and PREFILL_TILE % group == 0


def supported(head_dim: int, n_q_heads: int, n_kv_heads: int) -> bool:
    return bool(library().llm_attention_mma_supports(head_dim, n_q_heads, n_kv_heads))


def plan(batch, group: int, n_kv_heads: int, device=None, blocks_per_sm: int = DECODE_BLOCKS_PER_SM, cluster: bool = None):
    """Launch shape of a batch, derived once per step from its host-side lengths (and the number of SMs: the split
    count fixes the order of the partial sums, so it is a function of the batch and the GPU model only).
    ``blocks_per_sm``: decode blocks an SM holds at a time; ``cluster``: whether splits merge inside a cluster (which
    bounds their number) or through the merge kernel."""
    cluster = CLUSTER_MERGE if cluster is None else cluster
    key = ("attention_mma", group, n_kv_heads, blocks_per_sm, cluster)
    cached = batch.scratch.get(key)
    if cached is not None:
        return cached
    wave_blocks = blocks_per_sm * _sm_count(device if device is not None else batch.context_len.device)
    singles = sum(1 for length in batch.q_lens if length == 1)
    run_decode = singles > 0
    run_portions = singles < batch.n_seqs
    tiles = sum(-(-length * group // TILE) for length in batch.q_lens if length > 1)
    split_len, max_splits = MIN_SPLIT, 1
    if run_decode:
        longest = max(context for context, length in zip(batch.context_lens, batch.q_lens) if length == 1)
        # As many equal splits of the longest context as give about one wave of blocks (two per SM); with a
        # wave's worth of (sequence, kv head) pairs already, no split at all.  Measured on the 8B head shape:
        # equal splits beat ragged ones, and one wave beats one and a half.
        pairs = singles * n_kv_heads
        splits = max(1, min(wave_blocks // pairs, -(-longest // MIN_SPLIT)))
        if cluster:
            lone_blocks = pairs * WIDE_CLUSTER_SPLITS <= wave_blocks // blocks_per_sm
            # a cluster has up to 8 blocks, or exactly 16
            splits = WIDE_CLUSTER_SPLITS if lone_blocks and splits > 12 else min(splits, MAX_CLUSTER_SPLITS)
        if pairs > wave_blocks:
            # More than a wave of whole contexts: when the last wave would leave most SMs idle (40 sequences x 8 kv
            # heads = 1.08 waves take as long as 2), the contexts are split after all.  Measured on the 8B head shape at
            # context 3072: unsplit wins while the waves are three quarters full, else the fewest splits that fill
            # them to 0.85 (batch 40: 119 -> 100 us, batch 48: 123 -> 105, batch 80: 182 -> 170).
            def filled(count):
                blocks = pairs * count
                return blocks / (-(-blocks // wave_blocks) * wave_blocks)
            if filled(1) < 0.75:
                candidates = [count for count in (2, 3, 4) if longest // count >= 4 * TILE]
                good = [count for count in candidates if filled(count) >= 0.85]
                if good:
                    splits = good[0]
                elif candidates:
                    splits = max(candidates, key=filled)
        # every sequence is divided into this many equal parts (a negative split length says so to the kernel): the
        # longest gets the planned splits, shorter ones the same number of shorter blocks
        split_len, max_splits = -splits, splits
        forced = os.environ.get("LLMSERVER_B200_DECODE_SPLIT")
        if forced:
            split_len = int(forced)
            max_splits = -(-longest // split_len) + 1     # + 1: a window may start inside a tile
    cached = (run_portions, tiles, run_decode, split_len, max_splits)
    batch.scratch[key] = cached
    return cached


# A decode row's older keys were cached by earlier steps, which lie behind the step's batch copy; the decode kernel may
# start copying them before the kernel in front of it (which writes the newest key) has ended.  Only batches that say
# so (``keys_settled``, set where the engine packs a step) get this.
EARLY_KEYS = os.environ.get("LLMSERVER_B200_DECODE_EARLY_KEYS", "1") != "0"


def try_attention(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, scale, window):
    if not supported(head_dim, n_q_heads, n_kv_heads):
        return None
    check(qkv, "qkv", torch.bfloat16)
    check(k_pages, "k pages", torch.bfloat16, head_dim)
    check(v_pages, "v pages", torch.bfloat16, head_dim)
    check(block_tables, "block_tables", torch.int32)
    run_portions, tiles, run_decode, split_len, max_splits = plan(batch, n_q_heads // n_kv_heads, n_kv_heads, qkv.device)
    out = torch.empty((batch.n_tokens, n_q_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    partial_out = partial_ml = None
    if run_decode and max_splits > 1:
        # scratch of the split-KV decode, shared by every layer of the step
        key = ("attention_mma_scratch", n_q_heads, head_dim, max_splits)
        scratch = batch.scratch.get(key)
        if scratch is None:
            scratch = (torch.empty((batch.n_tokens, n_q_heads, max_splits, head_dim), dtype=torch.float32, device=qkv.device),
                       torch.empty((batch.n_tokens, n_q_heads, max_splits, 2), dtype=torch.float32, device=qkv.device))
            batch.scratch[key] = scratch
        partial_out, partial_ml = scratch
    page_size = k_pages.shape[2]
    flag = wait_error_flag(qkv.device).data_ptr()
    if run_portions and prefill_tcgen05_supported(head_dim, n_q_heads, n_kv_heads, page_size):
        # prompt portions on the tcgen05 kernel (128-row tiles); single tokens, if any, on the decode kernel
        group = n_q_heads // n_kv_heads
        wide = prefill_wide_wanted(batch, group, head_dim, n_q_heads, n_kv_heads, page_size)
        # a tile holds whole tokens: floor(128 / group) of them per 128 rows (the 256-row kernel has two such halves)
        tokens_per_tile = (PREFILL_TILE // group) * (2 if wide else 1)
        tile_counts = [-(-length // tokens_per_tile) for length in batch.q_lens if length > 1 or not run_decode]
        # A block takes a row tile and its mirror image (the light one with the heavy one), which gives every block of a
        # causal prompt the same work, or tiles go out one by one, heaviest first.  Pairs cost whole waves of double
        # blocks; single tiles fill the GPU more finely but end raggedly (about 1.3 x their mean, measured).
        paired = sum((count + 1) // 2 for count in tile_counts)
        slots = _block_slots(qkv.device, wide)
        cost_paired = 2.0 * -(-paired * n_kv_heads // slots)
        cost_single = 1.3 * max(sum(tile_counts) * n_kv_heads / slots, 1.0)
        pairing = cost_paired < cost_single if FORCE_PAIRING is None else FORCE_PAIRING
        call("llm_attention_prefill_wide" if wide else "llm_attention_prefill_tcgen05", qkv.data_ptr(), q_stride, batch.n_tokens,
             k_pages.data_ptr(), v_pages.data_ptr(),
             block_tables.data_ptr(), block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(),
             out.data_ptr(), batch.n_seqs, n_q_heads, n_kv_heads, head_dim, page_size, k_pages.shape[0], float(scale), int(window),
             int(run_decode), int(pairing), paired if pairing else sum(tile_counts), flag, stream_handle())
        run_portions = False
        if not run_decode:
            return out
    call("llm_attention_mma", qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(), batch.n_seqs,
         n_q_heads, n_kv_heads, head_dim, page_size, k_pages.shape[0], float(scale), int(window), int(run_portions), tiles,
         int(run_decode), split_len, max_splits, 0 if partial_out is None else partial_out.data_ptr(),
         0 if partial_ml is None else partial_ml.data_ptr(), int(EARLY_KEYS and getattr(batch, "keys_settled", False)), flag,
         stream_handle())
    return out


# "tcgen05" (default): prompts of heads of 128 run the tcgen05 kernel's two-part-weights form; "mma": the mma.sync kernel
PRECISE_PREFILL_KERNEL = os.environ.get("LLMSERVER_B200_PRECISE_PREFILL", "tcgen05")
PRECISE_DECODE_BLOCKS_PER_SM = int(os.environ.get("LLMSERVER_B200_PRECISE_DECODE_BLOCKS", "3"))


def try_attention_precise(qkv, q_stride, batch, block_tables, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, value_dim,
                          scale, window, sinks):
    """The tensor-core kernels in the form that keeps attention weights at 16 significant bits through the P V product,
    takes value heads of another size than key heads and adds exp(sinks[h]) to each softmax denominator; None when the
    sizes are not ones it takes (64 or 128 each)."""
    if not library().llm_attention_mma_sinks_supports(head_dim, value_dim, n_q_heads, n_kv_heads):
        return None
    check(qkv, "qkv", torch.bfloat16)
    check(k_pages, "k pages", torch.bfloat16, head_dim)
    check(v_pages, "v pages", torch.bfloat16, value_dim)
    check(block_tables, "block_tables", torch.int32)
    if sinks is not None:
        check(sinks, "sinks", torch.float32, n_q_heads)
    # the cp.async decode kernel keeps two tiles in flight per block: three blocks an SM (its shared memory allows them)
    # and splits without the cluster's bound keep more bytes in flight
    run_portions, tiles, run_decode, split_len, max_splits = plan(batch, n_q_heads // n_kv_heads, n_kv_heads, qkv.device,
                                                                  blocks_per_sm=PRECISE_DECODE_BLOCKS_PER_SM, cluster=False)
    out = torch.empty((batch.n_tokens, n_q_heads * value_dim), dtype=torch.bfloat16, device=qkv.device)
    partial_out = partial_ml = None
    if run_decode and max_splits > 1:
        key = ("attention_mma_scratch", n_q_heads, value_dim, max_splits)
        scratch = batch.scratch.get(key)
        if scratch is None:
            scratch = (torch.empty((batch.n_tokens, n_q_heads, max_splits, value_dim), dtype=torch.float32, device=qkv.device),
                       torch.empty((batch.n_tokens, n_q_heads, max_splits, 2), dtype=torch.float32, device=qkv.device))
            batch.scratch[key] = scratch
        partial_out, partial_ml = scratch
    page_size = k_pages.shape[2]
    if run_portions and value_dim == head_dim and PRECISE_PREFILL_KERNEL == "tcgen05" and \
            prefill_tcgen05_supported(head_dim, n_q_heads, n_kv_heads, page_size):
        # prompt portions on the 128-row tcgen05 kernel in its form with two-part weights; single tokens, if any, below
        group = n_q_heads // n_kv_heads
        tokens_per_tile = PREFILL_TILE // group
        tile_counts = [-(-length // tokens_per_tile) for length in batch.q_lens if length > 1 or not run_decode]
        paired = sum((count + 1) // 2 for count in tile_counts)
        slots = _block_slots(qkv.device, False)
        cost_paired = 2.0 * -(-paired * n_kv_heads // slots)
        cost_single = 1.3 * max(sum(tile_counts) * n_kv_heads / slots, 1.0)
        pairing = cost_paired < cost_single if FORCE_PAIRING is None else FORCE_PAIRING
        call("llm_attention_prefill_tcgen05_precise", qkv.data_ptr(), q_stride, batch.n_tokens, k_pages.data_ptr(), v_pages.data_ptr(),
             block_tables.data_ptr(), block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(),
             out.data_ptr(), batch.n_seqs, n_q_heads, n_kv_heads, head_dim, page_size, k_pages.shape[0], float(scale), int(window),
             int(run_decode), int(pairing), paired if pairing else sum(tile_counts), wait_error_flag(qkv.device).data_ptr(),
             0 if sinks is None else sinks.data_ptr(), stream_handle())
        run_portions = False
        if not run_decode:
            return out
    call("llm_attention_mma_sinks", qkv.data_ptr(), q_stride, k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(), batch.n_seqs,
         n_q_heads, n_kv_heads, head_dim, value_dim, k_pages.shape[2], k_pages.shape[0], float(scale), int(window),
         0 if sinks is None else sinks.data_ptr(), int(run_portions), tiles, int(run_decode), split_len, max_splits,
         0 if partial_out is None else partial_out.data_ptr(), 0 if partial_ml is None else partial_ml.data_ptr(),
         wait_error_flag(qkv.device).data_ptr(), stream_handle())
    return out


DIFF_KERNEL = os.environ.get("LLMSERVER_B200_DIFF_ATTENTION", "mma")      # "generic": always the kernel that takes every size
# row tiles per block of the tiled kernel: 0 = by the step (2, and 2 key splits, with prompt portions; 1 and 4 key splits
# for single tokens); 1, 2 or 4 force an arrangement
DIFF_ROW_TILES = int(os.environ.get("LLMSERVER_B200_DIFF_ROW_TILES", "0"))


def try_attention_diff(qkv, gate_column, batch, block_tables, k_pages, v_pages, n_q_heads, n_kv_heads, dim, value_dim, scale,
                       cap, window, lam, eps, out_scale, out) -> bool:
    """Differential attention on the tensor cores where the tiled kernel takes the sizes (units and values of 64 or 128,
    rows of the packed projection 16-byte aligned); False when it does not (the caller then runs the kernel that takes
    every size).  Prompt portions and single tokens go in one launch."""
    row_width = qkv.shape[1]
    if DIFF_KERNEL != "mma" or row_width % 8 or not library().llm_attention_diff_mma_supports(dim, value_dim, n_q_heads, n_kv_heads):
        return False
    check(qkv, "qkv", torch.bfloat16)
    gate = 0 if gate_column is None else qkv.data_ptr() + gate_column * qkv.element_size()
    # A step of single tokens has few (sequence, key/value head) pairs: several blocks then share a pair's keys, four
    # warp splits each, and leave partial results that a merge kernel adds up.  The count is a function of the batch's
    # host-side shape (so a captured graph keeps it): about four key tiles of 16 per warp, at most 16 blocks a pair,
    # and no more blocks than fill the GPU twice.
    block_splits, partials, group = 1, None, n_q_heads // n_kv_heads
    if batch.max_q_len == 1 and group <= 16 and DIFF_ROW_TILES in (0, 1):
        span = min(int(window), batch.max_context) if window else batch.max_context
        wanted = -(-span // (16 * 4 * 4))
        room = max(1, 2 * _sm_count(qkv.device) // max(1, batch.n_seqs * n_kv_heads))
        block_splits = max(1, min(wanted, room, 16))
        if block_splits > 1:
            key = ("attention_diff_partials", batch.n_seqs, n_kv_heads, block_splits, group, value_dim)
            partials = batch.scratch.get(key)
            if partials is None:
                partials = torch.empty((batch.n_seqs, n_kv_heads, block_splits * 4, 2, group, value_dim + 2), dtype=torch.float32,
                                       device=qkv.device)
                batch.scratch[key] = partials
    call("llm_attention_diff_mma", qkv.data_ptr(), row_width, gate, row_width, k_pages.data_ptr(), v_pages.data_ptr(),
         block_tables.data_ptr(), block_tables.shape[-1], batch.q_start.data_ptr(), batch.context_len.data_ptr(), out.data_ptr(),
         batch.n_seqs, int(batch.max_q_len), n_q_heads, n_kv_heads, int(dim), int(value_dim), k_pages.shape[2], k_pages.shape[0],
         float(scale), float(cap or 0.0), int(window or 0), float(lam), float(eps), float(out_scale),
         wait_error_flag(qkv.device).data_ptr(), DIFF_ROW_TILES, block_splits, 0 if partials is None else partials.data_ptr(),
         stream_handle())
    return True
