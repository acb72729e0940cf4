"""u8 per-token KV-cache quantiser and block layout — test infrastructure only.

PARITY UNPINNED: the reference holds no paged KV cache (its cache is the
contiguous ``CudaVariableState``, ``modules/nvidia_plugin/src/cuda_variable_state.hpp:31-183``).
The formulae restate OpenVINO's published by-token asymmetric u8 quantisation,
with the scale and zero-point stored as float16:

    mn, mx = min(x), max(x)                      over the D values of one (token, head)
    s      = f16( (mx - mn) / 255 )              f32 division, then round-to-nearest-even to f16
    s      = 1.0  if s == 0 or not finite
    zp     = f16( -mn / f32(s) )                 f32 division by the *rounded* scale
    q[d]   = clamp( rint( x[d] / f32(s) + f32(zp) ), 0, 255 )     f32 divide, f32 add, ties-to-even
    x^[d]  = ( f32(q[d]) - f32(zp) ) * f32(s)    de-quantisation, f32

Every step is a single IEEE-754 binary32 operation rounded to nearest-even, so a
CUDA kernel using ``__fdiv_rn`` / ``__fadd_rn`` / ``rintf`` reproduces it bit for bit.

Block layout (one *chunk* per (physical block, KV head), chunks contiguous as
``[num_blocks, Hkv, chunk_bytes]``):

    bytes [0, bs*D)            u8 values, token-major: token t at t*D
    bytes [bs*D, bs*D+2*bs)    f16 scale of token 0..bs-1
    bytes [bs*D+2*bs, +2*bs)   f16 zero-point of token 0..bs-1

For bs=16, D=128 a chunk is 2112 bytes = 16 * 132: every chunk starts on a 16-byte
boundary, every token row on a 128-byte boundary inside it.
"""
from __future__ import annotations

import numpy as np


def chunk_bytes(block_size: int, d: int) -> int:
    return block_size * d + 4 * block_size


def quantize_rows(x):
    """x [..., D] float -> (q u8 [..., D], scale f16 [...], zp f16 [...])."""
    x = np.asarray(x, dtype=np.float32)
    mn = x.min(axis=-1)
    mx = x.max(axis=-1)
    with np.errstate(over="ignore", invalid="ignore", divide="ignore"):
        s16 = ((mx - mn) / np.float32(255.0)).astype(np.float32).astype(np.float16)
        bad = (s16 == 0) | ~np.isfinite(s16)
        s16 = np.where(bad, np.float16(1.0), s16).astype(np.float16)
        sf = s16.astype(np.float32)
        zp16 = ((-mn) / sf).astype(np.float32).astype(np.float16)
        zf = zp16.astype(np.float32)
        t = (x / sf[..., None]).astype(np.float32) + zf[..., None]
        q = np.clip(np.rint(t.astype(np.float32)), 0.0, 255.0).astype(np.uint8)
    return q, s16, zp16


def dequantize_rows(q, s16, zp16):
    """(q u8 [..., D], scale f16 [...], zp f16 [...]) -> f32 [..., D]."""
    sf = np.asarray(s16, dtype=np.float16).astype(np.float32)[..., None]
    zf = np.asarray(zp16, dtype=np.float16).astype(np.float32)[..., None]
    return ((q.astype(np.float32) - zf) * sf).astype(np.float32)


def chunk_views(cache, block_size: int, d: int):
    """Split a C-contiguous u8 cache [num_blocks, Hkv, chunk_bytes] into aliasing views.

    Returns (data u8 [num_blocks, Hkv, bs, D], scale f16 [num_blocks, Hkv, bs], zp f16 [same]).
    Writes through the views land in ``cache``.
    """
    nb, hkv, cb = cache.shape
    assert cache.dtype == np.uint8 and cache.flags["C_CONTIGUOUS"]
    assert cb == chunk_bytes(block_size, d), (cb, block_size, d)
    assert (block_size * d) % 2 == 0
    data = np.lib.stride_tricks.as_strided(
        cache, shape=(nb, hkv, block_size, d), strides=(hkv * cb, cb, d, 1), writeable=True)
    h = cache.view(np.float16)  # [nb, hkv, cb/2]
    o = block_size * d // 2
    return data, h[:, :, o : o + block_size], h[:, :, o + block_size : o + 2 * block_size]
