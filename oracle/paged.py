"""CPU restatement of PagedAttentionExtension over a block-table KV cache — test infrastructure only.

The reference has no paged attention (its KV cache is ``ReadValue``/``Assign`` around a
contiguous ``CudaVariableState``, ``modules/nvidia_plugin/src/ops/read_value.cpp:31-72``,
``ops/assign.cpp:29-56``, grown with ``kernels/concat.cu:16-32``).  The operand contract
restated here is OpenVINO's public ``PagedAttentionExtension``:

    query [tokens, Hq*D], key [tokens, Hkv*D], value [tokens, Hkv*Dv],
    key_cache, value_cache  (block pools, see ``oracle.quant``),
    past_lens [seqs] i32, subsequence_begins [seqs+1] i32,
    block_indices [sum blocks] i32, block_indices_begins [seqs+1] i32,
    scale, sliding_window.

Step semantics: first the new K/V rows of every sequence ``s`` are appended at
positions ``past_lens[s] .. past_lens[s]+q_len-1`` through the block table
(``kv_store_ref``); then query token ``i`` of sequence ``s`` attends to cache
positions ``0 .. past_lens[s]+i`` (``paged_attention_ref``), restricted to the last
``sliding_window`` of them when that is positive.  The attention arithmetic is the
same softmax(QK^T·scale)·V as ``oracle.sdpa`` (pinned against the reference's dense
attention); scores and sums are float32.
"""
from __future__ import annotations

import numpy as np

from .quant import chunk_views, dequantize_rows, quantize_rows
from .sdpa import _as_f32


def physical_slot(pos, seq, block_indices, block_indices_begins, block_size):
    """(physical block, slot in block) of logical position ``pos`` of sequence ``seq``."""
    lb = pos // block_size
    return int(block_indices[int(block_indices_begins[seq]) + lb]), pos % block_size


def kv_store_ref(new_rows, cache, past_lens, subsequence_begins, block_indices,
                 block_indices_begins, hkv, d, block_size):
    """Quantise and append ``new_rows`` [tokens, Hkv*D] into the u8 ``cache`` in place.

    Returns the list of (physical block, slot) written per token, for index checks.
    """
    x = _as_f32(new_rows).reshape(-1, hkv, d)
    data, sc, zp = chunk_views(cache, block_size, d)
    written = []
    for s in range(len(past_lens)):
        b, e = int(subsequence_begins[s]), int(subsequence_begins[s + 1])
        for t in range(b, e):
            pos = int(past_lens[s]) + (t - b)
            pb, slot = physical_slot(pos, s, block_indices, block_indices_begins, block_size)
            q, s16, z16 = quantize_rows(x[t])  # [Hkv, D], [Hkv], [Hkv]
            data[pb, :, slot, :] = q
            sc[pb, :, slot] = s16
            zp[pb, :, slot] = z16
            written.append((pb, slot))
    return written


def gather_sequence(cache, seq, n_tokens, block_indices, block_indices_begins, d, block_size):
    """De-quantised contiguous [Hkv, n_tokens, D] float32 view of one sequence's cache."""
    data, sc, zp = chunk_views(cache, block_size, d)
    nblk = (n_tokens + block_size - 1) // block_size
    b0 = int(block_indices_begins[seq])
    phys = np.asarray(block_indices[b0 : b0 + nblk], dtype=np.int64)
    x = dequantize_rows(data[phys], sc[phys], zp[phys])  # [nblk, Hkv, bs, D]
    x = np.transpose(x, (1, 0, 2, 3)).reshape(x.shape[1], nblk * block_size, d)
    return x[:, :n_tokens]


def paged_attention_ref(query, k_cache, v_cache, past_lens, subsequence_begins, block_indices,
                        block_indices_begins, hq, hkv, d, block_size, scale=None, sliding_window=0):
    """Attention of every query token over its sequence's cache.  Returns f32 [tokens, Hq*D]."""
    q = _as_f32(query).reshape(-1, hq, d)
    g = hq // hkv
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(d))
    out = np.zeros_like(q)
    for s in range(len(past_lens)):
        b, e = int(subsequence_begins[s]), int(subsequence_begins[s + 1])
        qlen = e - b
        if qlen == 0:
            continue
        past = int(past_lens[s])
        ctx = past + qlen
        kk = gather_sequence(k_cache, s, ctx, block_indices, block_indices_begins, d, block_size)
        vv = gather_sequence(v_cache, s, ctx, block_indices, block_indices_begins, d, block_size)
        # the g query heads of a KV head share its keys and values (grouped-query attention): they are stacked
        # along the row axis instead of repeating K and V g times
        qs = np.transpose(q[b:e], (1, 0, 2)).reshape(hkv, g * qlen, d)  # [Hkv, g*qlen, D], row = head-in-group * qlen + i
        sc = np.matmul(qs, np.swapaxes(kk, -1, -2)) * np.float32(scale)  # [Hkv, g*qlen, ctx]
        pos_q = np.tile(past + np.arange(qlen), g)[:, None]
        pos_k = np.arange(ctx)[None, :]
        keep = pos_k <= pos_q
        if sliding_window and sliding_window > 0:
            keep &= (pos_q - pos_k) < sliding_window
        sc = np.where(keep[None], sc, np.float32(-np.inf))
        mx = sc.max(axis=-1, keepdims=True)
        p = np.exp(sc - mx)
        o = np.matmul(p / p.sum(axis=-1, keepdims=True), vv).reshape(hq, qlen, d)  # [Hq, qlen, D]
        out[b:e] = np.transpose(o, (1, 0, 2))
    return out.reshape(-1, hq * d)


def last_token_scores_ref(query, k_cache, past_lens, subsequence_begins, block_indices, block_indices_begins,
                          hq, hkv, d, block_size, scale=None, sliding_window=0):
    """Score output: per sequence, the softmax row of its LAST query token over the sequence's keys, summed over the
    query heads (what an eviction policy accumulates, modules/genai_optimizations/genai_opt/token_eviction.py:154-183:
    attention weights summed over query rows and heads per key).  Returns (scores f32 flat, begins i32 [seqs+1]);
    a sequence without a query token has no entries; keys a sliding window leaves out score 0.
    PARITY UNPINNED: the reference has no paged attention; the arithmetic is the pinned softmax of this file."""
    q = _as_f32(query).reshape(-1, hq, d)
    g = hq // hkv
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(d))
    parts, begins = [], [0]
    for s in range(len(past_lens)):
        b, e = int(subsequence_begins[s]), int(subsequence_begins[s + 1])
        if e - b < 1:
            begins.append(begins[-1])
            continue
        ctx = int(past_lens[s]) + (e - b)
        kk = gather_sequence(k_cache, s, ctx, block_indices, block_indices_begins, d, block_size)  # [Hkv, ctx, D]
        qs = q[e - 1].reshape(hkv, g, d)
        sc = np.matmul(qs, np.swapaxes(kk, -1, -2)) * np.float32(scale)  # [Hkv, g, ctx]
        if sliding_window and sliding_window > 0:
            keep = (ctx - 1 - np.arange(ctx)) < sliding_window
            sc = np.where(keep[None, None], sc, np.float32(-np.inf))
        p = np.exp(sc - sc.max(axis=-1, keepdims=True))
        p = p / p.sum(axis=-1, keepdims=True)
        parts.append(p.sum(axis=(0, 1)).astype(np.float32))
        begins.append(begins[-1] + ctx)
    flat = np.concatenate(parts) if parts else np.zeros(0, np.float32)
    return flat, np.asarray(begins, np.int32)


# ---------------------------------------------------------------------------------------
# Seeded workload builders shared by tests and bench (shapes follow the benchmark configs).
# ---------------------------------------------------------------------------------------

def build_block_tables(context_lens, block_size, seed, spare_blocks=1):
    """Random block assignment: the pool holds sum(ceil(len/bs)) + spare blocks, and the
    sequences' logical blocks are a seeded permutation of the non-spare ones.

    Returns (block_indices i32 [sum blocks], block_indices_begins i32 [seqs+1], num_blocks).
    """
    nblk = [(int(c) + block_size - 1) // block_size for c in context_lens]
    total = int(sum(nblk))
    rng = np.random.default_rng(seed)
    perm = rng.permutation(total + spare_blocks)[:total].astype(np.int32)
    begins = np.zeros(len(nblk) + 1, dtype=np.int32)
    begins[1:] = np.cumsum(nblk)
    return perm, begins, total + spare_blocks


def fill_cache_from_rows(rows, context_lens, block_indices, block_indices_begins, num_blocks,
                         hkv, d, block_size, poison=0xFF):
    """Quantise per-sequence rows (list of [len, Hkv, D] f32) into a fresh u8 pool (vectorised).

    Unused slots and spare blocks are filled with ``poison`` bytes so that a stray read shows.
    """
    from .quant import chunk_bytes
    cache = np.full((num_blocks, hkv, chunk_bytes(block_size, d)), poison, dtype=np.uint8)
    data, sc, zp = chunk_views(cache, block_size, d)
    for s, x in enumerate(rows):
        n = int(context_lens[s])
        if n == 0:
            continue
        q, s16, z16 = quantize_rows(x[:n])  # [n, Hkv, D]
        pos = np.arange(n)
        b0 = int(block_indices_begins[s])
        pb = np.asarray(block_indices, dtype=np.int64)[b0 + pos // block_size]
        slot = pos % block_size
        data[pb, :, slot, :] = q
        sc[pb, :, slot] = s16
        zp[pb, :, slot] = z16
    return cache
