"""Multi-threaded CPU form of the oracle's dense attention, for timing — test/bench infrastructure only.

Same arithmetic as ``oracle.sdpa.sdpa_ref`` and as the reference's PyTorch dense attention
(``modules/genai_optimizations/genai_opt/sparse_attention.py:95-121``): repeat K/V heads for grouped queries,
``QK^T * scale``, additive causal mask, float32 softmax, ``P V``.  It exists because numpy's matmul is what the
parity tests want (deterministic, simple) while a CPU *baseline* should use every host core.
"""
from __future__ import annotations

import torch


def dense_attention_cpu(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                        scale: float | None = None) -> torch.Tensor:
    """q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] on the CPU -> [B,Hq,Sq,D] float32."""
    q, k, v = q.float(), k.float(), v.float()
    g = q.shape[1] // k.shape[1]
    if g > 1:
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    w = torch.matmul(q, k.transpose(-2, -1)) * scale
    if causal:
        sq, skv = q.shape[-2], k.shape[-2]
        w = w.masked_fill(~torch.ones(sq, skv, dtype=torch.bool).tril(0), float("-inf"))
    w = torch.softmax(w, dim=-1, dtype=torch.float32)
    return torch.matmul(w, v)
