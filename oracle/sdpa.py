"""CPU restatement of ScaledDotProductAttention — test infrastructure only.

Follows the op semantics the reference plugin obtains by decomposing
``ov::op::v13::ScaledDotProductAttention``
(``modules/nvidia_plugin/src/transformer/cuda_graph_transformer.cpp:151-156``):
``softmax(Q·K^T·scale + mask)·V`` with

  * ``scale`` defaulting to ``1/sqrt(E)``;
  * ``causal=True`` meaning the top-left aligned lower triangle (query ``i`` sees
    keys ``0..i``) and the mask operand being ignored;
  * a boolean mask keeping the positions that are true, a float mask being added;
  * grouped-query attention by repeating each K/V head ``Hq/Hkv`` times, the way
    the reference's ``repeat_kv`` does
    (``modules/genai_optimizations/genai_opt/sparse_attention.py:87-93``);
  * softmax evaluated in float32 on max-subtracted scores
    (``sparse_attention.py:118``; ``modules/nvidia_plugin/src/ops/softmax.cpp:184-192``
    uses CUDNN_SOFTMAX_ACCURATE, i.e. max-subtracted).

Accumulation is float32 (float64 on request); the result is rounded once to the
requested output type by the caller.
"""
from __future__ import annotations

import numpy as np


def _as_f32(x):
    """float32 view of a numpy array or a torch tensor (bf16 included)."""
    if hasattr(x, "detach"):
        x = x.detach().cpu().float().numpy()
    return np.asarray(x, dtype=np.float32)


def causal_keep(sq: int, skv: int) -> np.ndarray:
    """Boolean [sq, skv] matrix of kept positions: key j kept for query i iff j <= i."""
    return np.tril(np.ones((sq, skv), dtype=bool), k=0)


def sdpa_ref(q, k, v, mask=None, scale=None, causal=False, acc=np.float32):
    """q [..., Hq, Sq, E], k [..., Hkv, Skv, E], v [..., Hkv, Skv, Ev]  ->  [..., Hq, Sq, Ev] (``acc`` dtype).

    3-D inputs are [N, S, E] (leading dimension = batch, one head).
    """
    q, k, v = _as_f32(q), _as_f32(k), _as_f32(v)
    squeeze = q.ndim == 3
    if squeeze:
        q, k, v = q[:, None], k[:, None], v[:, None]
    hq, hkv = q.shape[-3], k.shape[-3]
    if hq != hkv:
        assert hq % hkv == 0, "query heads must be a multiple of KV heads"
        g = hq // hkv
        k = np.repeat(k, g, axis=-3)
        v = np.repeat(v, g, axis=-3)
    sq, skv, e = q.shape[-2], k.shape[-2], q.shape[-1]
    if scale is None:
        scale = 1.0 / np.sqrt(np.float32(e))
    s = np.matmul(q.astype(acc), np.swapaxes(k, -1, -2).astype(acc)) * acc(scale)
    neg_inf = acc(-np.inf)
    if causal:
        s = np.where(causal_keep(sq, skv), s, neg_inf)
    elif mask is not None:
        m = mask.detach().cpu().numpy() if hasattr(mask, "detach") and str(mask.dtype) == "torch.bool" else mask
        if hasattr(m, "detach"):
            m = _as_f32(m)
        m = np.asarray(m)
        if m.dtype == np.bool_:
            s = np.where(m, s, neg_inf)
        else:
            s = s + m.astype(acc)
    mx = np.max(s, axis=-1, keepdims=True)
    mx = np.where(np.isfinite(mx), mx, acc(0))  # fully masked row -> zeros, not NaN
    p = np.exp(s - mx)
    den = np.sum(p, axis=-1, keepdims=True)
    den = np.where(den == 0, acc(1), den)
    out = np.matmul(p / den, v.astype(acc))
    return out[:, 0] if squeeze else out


def sdpa_flops(b, hq, sq, skv, e, ev, causal):
    """Algorithmic FLOPs: 2·E and 2·Ev per kept (query, key) pair."""
    if causal:
        pairs = sum(min(i + 1, skv) for i in range(sq)) if sq != skv else sq * (sq + 1) // 2
    else:
        pairs = sq * skv
    return 2 * b * hq * pairs * (e + ev)
