"""b2a_paged_attention_noalloc: decode attention for callers that cannot hand over a workspace.

Some users of the library sit where no device memory can be obtained at call time: an operator body that runs
while its stream is being captured into a CUDA graph, an extension op that is only ever given its input and
output buffers, a server that gave all device memory to the KV pool at start-up.  For them the split-K partials
live in a 16 MiB array inside the library.  This file is collected last on purpose (see its name): it checks
that the variant gives the same bytes as the workspace-taking entry point, on two calls in a row — the second
call finds the array full of the first call's partials — and that an over-sized step is refused.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.helpers import PagedWorkload

pytestmark = pytest.mark.gpu


def _desc(lib_mod, w, num_seqs, max_ctx):
    d = lib_mod.PagedDesc()
    d.q_dtype, d.kv_dtype = lib_mod.F16, lib_mod.U8
    d.Hq, d.Hkv, d.D, d.Dv, d.block_size = w.hq, w.hkv, w.d, w.d, w.bs
    d.num_seqs = d.num_tokens = num_seqs
    d.num_blocks_total = w.nb
    d.max_context_len, d.max_q_len = max_ctx, 1
    d.scale, d.sliding_window = 0.0, 0
    return d


def test_noalloc_matches_workspace_entry_point_twice():
    from openvino_contrib_b200 import _lib
    lib = _lib.load()
    assert torch.cuda.is_available()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (ctx, seed) in enumerate([([1, 17, 333, 5000], 21), ([4096, 64, 2047, 9], 22)]):
        w = PagedWorkload(ctx, [1] * len(ctx), 32, 8, 128, seed=seed)
        cache = w.device_cache()
        past, sb, bi, bb = w.device_tables()
        q = torch.from_numpy(w.query).to(torch.float16).cuda()
        d = _desc(_lib, w, len(ctx), max(ctx))
        ws_bytes = C.c_size_t(0)
        assert lib.b2a_paged_workspace_bytes(C.byref(d), 0, C.byref(ws_bytes)) == 0
        assert 0 < ws_bytes.value <= _lib.BUILTIN_SCRATCH_BYTES
        ws = torch.empty(ws_bytes.value, dtype=torch.uint8, device="cuda")
        ref = torch.zeros_like(q)
        out = torch.zeros_like(q)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        args = (q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), past.data_ptr(), sb.data_ptr(),
                bi.data_ptr(), bb.data_ptr())
        assert lib.b2a_paged_attention(C.byref(d), *args, ref.data_ptr(), ws.data_ptr(), ws_bytes.value,
                                       status.data_ptr(), stream) == 0
        assert lib.b2a_paged_attention_noalloc(C.byref(d), *args, out.data_ptr(), status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        # same kernels, same split plan, same order of operations: the outputs are identical, not merely close
        assert torch.equal(out, ref), f"call {call}"
        # and right: against the CPU oracle within the half-precision bar
        np.testing.assert_allclose(out.float().cpu().numpy(), w.reference(q.float().cpu().numpy()),
                                   atol=2e-3, rtol=1e-2)


def test_noalloc_refuses_what_does_not_fit():
    from openvino_contrib_b200 import _lib
    lib = _lib.load()
    w = PagedWorkload([40], [1], 32, 8, 128, seed=23)
    # a descriptor sized for 256 sequences of 32768 tokens needs more partial storage than the built-in array
    d = _desc(_lib, w, 256, 32768)
    need = C.c_size_t(0)
    assert lib.b2a_paged_workspace_bytes(C.byref(d), 0, C.byref(need)) == 0
    assert need.value > _lib.BUILTIN_SCRATCH_BYTES
    x = torch.zeros(256, 32 * 128, dtype=torch.float16, device="cuda")
    t = torch.zeros(300, dtype=torch.int32, device="cuda")
    cache = w.device_cache()
    rc = lib.b2a_paged_attention_noalloc(C.byref(d), x.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                         t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), x.data_ptr(),
                                         None, torch.cuda.current_stream().cuda_stream)
    assert rc == 10 and b"16 MiB" in lib.b2a_status_string(rc)
    # shapes the decode kernel does not take are refused as unsupported, not routed elsewhere
    d2 = _desc(_lib, w, 1, 40)
    d2.D = d2.Dv = 64
    rc = lib.b2a_paged_attention_noalloc(C.byref(d2), x.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                         t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), x.data_ptr(),
                                         None, torch.cuda.current_stream().cuda_stream)
    assert rc == 7
