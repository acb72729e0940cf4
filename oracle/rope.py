"""CPU restatement of rotary position embedding for the key rows of a KV store - test infrastructure only.

PARITY UNPINNED: the reference holds no rotary-embedding code (its models reach the plugin with the rotation
decomposed into Multiply / Concat / Add nodes like any other arithmetic).  What is restated here is the published
"rotate-half" form used by the Llama family:

    inv_freq[i] = base ** (-2 i / r)                   i < r/2,  r = rotary_dim
    angle[p][i] = p * inv_freq[i]
    x'[i]       = x[i]       * cos(angle[p][i]) - x[i + r/2] * sin(angle[p][i])
    x'[i + r/2] = x[i + r/2] * cos(angle[p][i]) + x[i]       * sin(angle[p][i])

with values beyond ``rotary_dim`` passed through.  The tables are float32; each product and each sum is one float32
operation rounded to nearest (numpy float32 arithmetic, no fused multiply-add), which is the order the CUDA kernel
follows with ``__fmul_rn`` / ``__fsub_rn`` / ``__fadd_rn`` - so the rotated rows, and the u8 codes quantised from
them, agree bit for bit.
"""
from __future__ import annotations

import numpy as np


def rope_tables(positions: int, rotary_dim: int, base: float = 10000.0):
    """(cos, sin) float32 tables of shape [positions, rotary_dim // 2]."""
    half = rotary_dim // 2
    inv_freq = (1.0 / (np.float64(base) ** (np.arange(half, dtype=np.float64) * 2.0 / rotary_dim)))
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def rope_rows(x, positions, cos, sin, rotary_dim: int):
    """x [tokens, H, D] (any float) at cache positions ``positions`` [tokens] -> rotated float32 [tokens, H, D]."""
    x = np.asarray(x, dtype=np.float32)
    pos = np.asarray(positions, dtype=np.int64)
    half = rotary_dim // 2
    c = cos[pos][:, None, :].astype(np.float32)   # [tokens, 1, half]
    s = sin[pos][:, None, :].astype(np.float32)
    lo, hi = x[..., :half], x[..., half:rotary_dim]
    out = x.copy()
    out[..., :half] = (lo * c).astype(np.float32) - (hi * s).astype(np.float32)
    out[..., half:rotary_dim] = (hi * c).astype(np.float32) + (lo * s).astype(np.float32)
    return out


def token_positions(past_lens, subsequence_begins):
    """Cache position of every token of a step: past_lens[s] + offset inside sequence s."""
    sb = np.asarray(subsequence_begins, dtype=np.int64)
    pos = np.zeros(int(sb[-1]), dtype=np.int64)
    for s in range(len(past_lens)):
        pos[sb[s]:sb[s + 1]] = int(past_lens[s]) + np.arange(sb[s + 1] - sb[s])
    return pos
