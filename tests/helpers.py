"""Shared builders for the parity tests: seeded workloads in the oracle's formats, moved to the device."""
from __future__ import annotations

import numpy as np
import torch

from oracle import paged as opaged

TOL = {torch.float32: dict(atol=2e-5, rtol=1e-4),
       # the bar stated for half-precision outputs: 2e-3 max-abs / 1e-2 relative
       torch.float16: dict(atol=2e-3, rtol=1e-2),
       torch.bfloat16: dict(atol=2e-3, rtol=1e-2)}


def assert_close(actual: torch.Tensor, expected: np.ndarray, dtype, what=""):
    a = actual.detach().float().cpu().numpy()
    tol = dict(TOL[dtype])
    if dtype == torch.bfloat16:
        # the output itself is rounded to bf16 (8 significant bits): half an ulp of the result is not an error
        tol["atol"] = max(tol["atol"], 0.0) + 0.0
        tol["rtol"] = max(tol["rtol"], 2 ** -8)
    np.testing.assert_allclose(a, expected.reshape(a.shape), err_msg=what, **tol)


class PagedWorkload:
    """A seeded paged-attention problem: pools filled by the ORACLE's quantiser, tables, queries."""

    def __init__(self, context_lens, q_lens, hq, hkv, d, block_size=16, seed=0, table_seed=3, spare_blocks=2,
                 q_scale=1.0, value_fn=None, key_fn=None):
        self.hq, self.hkv, self.d, self.bs = hq, hkv, d, block_size
        self.ctx = np.asarray(context_lens, dtype=np.int64)      # context INCLUDING this step's tokens
        self.qlen = np.asarray(q_lens, dtype=np.int32)
        self.past = (self.ctx - self.qlen).astype(np.int32)
        assert (self.past >= 0).all()
        rng = np.random.default_rng(seed)
        self.bi, self.bb, self.nb = opaged.build_block_tables(self.ctx, block_size, table_seed, spare_blocks)
        self.rows_k = [(key_fn(s, int(c)) if key_fn else rng.standard_normal((int(c), hkv, d), dtype=np.float32))
                       for s, c in enumerate(self.ctx)]
        self.rows_v = [(value_fn(s, int(c)) if value_fn else rng.standard_normal((int(c), hkv, d), dtype=np.float32))
                       for s, c in enumerate(self.ctx)]
        self.sb = np.zeros(len(self.ctx) + 1, dtype=np.int32)
        self.sb[1:] = np.cumsum(self.qlen)
        self.query = (rng.standard_normal((int(self.sb[-1]), hq * d), dtype=np.float32) * q_scale)
        self.k_cache = opaged.fill_cache_from_rows(self.rows_k, self.ctx, self.bi, self.bb, self.nb, hkv, d, block_size)
        self.v_cache = opaged.fill_cache_from_rows(self.rows_v, self.ctx, self.bi, self.bb, self.nb, hkv, d, block_size)

    def reference(self, query_rounded: np.ndarray, scale=None, sliding_window=0):
        return opaged.paged_attention_ref(query_rounded, self.k_cache, self.v_cache, self.past, self.sb, self.bi,
                                          self.bb, self.hq, self.hkv, self.d, self.bs, scale, sliding_window)

    def device_tables(self, device="cuda"):
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(device)
        return t(self.past), t(self.sb), t(self.bi), t(self.bb)

    def device_cache(self, device="cuda"):
        from openvino_contrib_b200 import PagedKvCache
        return PagedKvCache(torch.from_numpy(self.k_cache).to(device), torch.from_numpy(self.v_cache).to(device),
                            self.hkv, self.d, self.d, self.bs, torch.uint8)
