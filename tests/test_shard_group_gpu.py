"""The head-shard exchange on ONE GPU, through the C ABI: what can be checked without a second device.

* a group of world size 1 runs the very kernels of the multi-GPU step (decode with the merge in its last CTA per
  (sequence, KV head), low-latency words, receiving kernel; the in-place form; the prefill epilogue stores) and
  must give the bits of the plain entry points;
* failure detection: two ranks of a world-2 group live in this process, connected by pointer, and only rank 0 ever
  runs a step.  Its waits on rank 1 are given a bound of a few milliseconds; they must run out, the kernels must
  return, and the status word must carry DEV_TIMEOUT.  Nothing here faults or hangs the GPU: the wait is on a
  flag that nothing sets, and it is bounded.
"""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from tests.helpers import PagedWorkload, assert_close

pytestmark = pytest.mark.gpu

HQ, HKV, D = 32, 4, 128   # G = 8: the eight-columns-per-thread merge


@pytest.fixture(scope="module")
def b2a():
    import openvino_contrib_b200 as m
    assert torch.cuda.is_available()
    return m


def _decode_problem(seed=41, ctx=(37, 1000, 2049, 16, 513, 4096)):
    w = PagedWorkload(list(ctx), [1] * len(ctx), HQ, HKV, D, seed=seed)
    return w, w.device_cache(), w.device_tables()


def test_world1_low_latency_and_in_place_match_plain_decode(b2a):
    from openvino_contrib_b200.sharding import HeadShard, ShardGroup
    w, cache, tables = _decode_problem()
    n, maxc = len(w.ctx), int(w.ctx.max())
    shard = HeadShard(0, 1, HQ, HKV)
    ws = torch.empty(max(16, b2a.ops.paged_workspace_bytes(torch.float16, cache, HQ, n, n, maxc, 1)),
                     dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = ShardGroup(shard, staging_bytes=2 * n * HQ * D * 2)
    for step in range(3):  # odd and even steps use different staging halves
        q = torch.from_numpy(w.query * (1.0 + 0.25 * step)).to(torch.float16).cuda()
        plain = b2a.paged_attention(q, cache, *tables, hq=HQ, max_context_len=maxc, max_q_len=1, workspace=ws)
        out = torch.zeros(n, HQ * D, dtype=torch.float16, device="cuda")
        group.paged_attention(q, cache, *tables, max_context_len=maxc, out_full=out, workspace=ws, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert_close(out, w.reference(q.float().cpu().numpy()), torch.float16, f"step {step}")
        assert torch.equal(out, plain)  # the in-kernel merge performs the merge kernel's arithmetic exactly
    group.close()
    # staging of just the output size cannot carry the 8-byte words of a step into a caller's buffer
    small = ShardGroup(shard, staging_bytes=n * HQ * D * 2)
    with pytest.raises(b2a.B2AError) as e:
        small.paged_attention(q, cache, *tables, max_context_len=maxc, out_full=out, workspace=ws)
    assert e.value.code == 8
    # ... but it serves the in-place form
    for step in range(2):
        q = torch.from_numpy(w.query * (0.5 + step)).to(torch.float16).cuda()
        view = small.paged_attention(q, cache, *tables, max_context_len=maxc, out_full=None, workspace=ws, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert_close(view, w.reference(q.float().cpu().numpy()), torch.float16, f"in-place step {step}")
        assert torch.equal(view, b2a.paged_attention(q, cache, *tables, hq=HQ, max_context_len=maxc, max_q_len=1))
    small.close()


def test_world1_low_latency_reports_bad_rows_and_still_delivers(b2a):
    # a sequence with inconsistent tables: its row arrives as zeros, the others are right, nothing waits for ever
    from openvino_contrib_b200.sharding import HeadShard, ShardGroup
    w, cache, (past, sb, bi, bb) = _decode_problem(seed=42)
    n, maxc = len(w.ctx), int(w.ctx.max())
    ws = torch.empty(max(16, b2a.ops.paged_workspace_bytes(torch.float16, cache, HQ, n, n, maxc, 1)),
                     dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    group = ShardGroup(HeadShard(0, 1, HQ, HKV), staging_bytes=2 * n * HQ * D * 2)
    group.set_wait_ms(50)
    bad = past.clone()
    bad[2] = -5
    q = torch.from_numpy(w.query).to(torch.float16).cuda()
    out = torch.full((n, HQ * D), 7.0, dtype=torch.float16, device="cuda")
    group.paged_attention(q, cache, bad, sb, bi, bb, max_context_len=maxc, out_full=out, workspace=ws, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == b2a._lib.DEV_BAD_LEN
    ref = w.reference(q.float().cpu().numpy())
    assert float(out[2].float().abs().max()) == 0.0
    keep = [i for i in range(n) if i != 2]
    assert_close(out[keep], ref[keep], torch.float16)
    group.close()


def _ranks_in_one_process(lib, staging_bytes, world=2):
    """Groups of all ranks of a world, every one on the current device, connected by pointer."""
    gs = []
    for r in range(world):
        h = C.c_void_p()
        assert lib.b2a_shard_group_create(r, world, staging_bytes, C.byref(h)) == 0
        gs.append(h)
    bases = (C.c_void_p * world)()
    for r in range(world):
        p = C.c_void_p()
        assert lib.b2a_shard_group_output(gs[r], C.byref(p)) == 0
        bases[r] = p.value
    for r in range(world):
        assert lib.b2a_shard_group_connect_pointers(gs[r], bases) == 0
    return gs


def _two_ranks_in_one_process(lib, staging_bytes):
    return _ranks_in_one_process(lib, staging_bytes, 2)


def _local_desc(_lib, w, n, maxc, hq_local, hkv_local):
    d = _lib.PagedDesc()
    d.q_dtype, d.kv_dtype = _lib.F16, _lib.U8
    d.Hq, d.Hkv, d.D, d.Dv, d.block_size = hq_local, hkv_local, D, D, 16
    d.num_seqs = d.num_tokens = n
    d.num_blocks_total = w.nb
    d.max_context_len, d.max_q_len = maxc, 1
    return d


@pytest.mark.parametrize("in_place", [False, True])
def test_absent_rank_times_out_decode(b2a, in_place):
    from openvino_contrib_b200 import _lib
    lib = _lib.load()
    w, cache, (past, sb, bi, bb) = _decode_problem(seed=43)
    n, maxc = len(w.ctx), int(w.ctx.max())
    g0, g1 = _two_ranks_in_one_process(lib, 2 * n * 2 * HQ * D * 2)
    assert lib.b2a_shard_group_set_wait_ms(g0, 20) == 0
    d = _local_desc(_lib, w, n, maxc, HQ, HKV)   # this rank's heads: the pool is taken as its shard
    need = C.c_size_t(0)
    assert lib.b2a_paged_workspace_bytes(C.byref(d), 0, C.byref(need)) == 0
    ws = torch.empty(max(16, need.value), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = torch.from_numpy(w.query).to(torch.float16).cuda()
    if in_place:
        p = C.c_void_p()
        assert lib.b2a_shard_group_output(g0, C.byref(p)) == 0
        out_ptr = p.value
    else:
        out = torch.zeros(n, 2 * HQ * D, dtype=torch.float16, device="cuda")
        out_ptr = out.data_ptr()
    for attempt in range(2):  # after a reset the group serves again - and times out again, rank 1 is still absent
        status.zero_()
        t0 = time.time()
        rc = lib.b2a_paged_attention_sharded(g0, C.byref(d), q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                             past.data_ptr(), sb.data_ptr(), bi.data_ptr(), bb.data_ptr(), out_ptr,
                                             ws.data_ptr(), ws.numel(), status.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()   # returns: the waits are bounded
        assert time.time() - t0 < 5.0
        assert int(status.item()) & _lib.DEV_TIMEOUT
        if not in_place:
            # rank 0's own columns did arrive and are right; rank 1's never came
            ref = w.reference(q.float().cpu().numpy())
            assert_close(out[:, : HQ * D], ref, torch.float16, "own columns")
        assert lib.b2a_shard_group_reset(g0) == 0 and lib.b2a_shard_group_reset(g1) == 0
    lib.b2a_shard_group_destroy(g0)
    lib.b2a_shard_group_destroy(g1)


@pytest.mark.parametrize("world", [2, 4])
def test_absent_ranks_time_out_prefill_and_own_tiles_reach_every_rank(b2a, world):
    # Only rank 0 of the world runs the step (all ranks' buffers live on this one GPU).  Its wait for the others must
    # run out; its own heads must nevertheless sit, bit-identical to the plain kernel, in the buffer of EVERY rank -
    # the epilogue's tensor stores to the peers (with four ranks the CTAs also walk their items lightest first).
    from openvino_contrib_b200 import _lib
    from openvino_contrib_b200.sharding import _device_view
    lib = _lib.load()
    B, hq, hkv, S = 2, 4, 1, 200   # S not a multiple of a row piece: the ragged last rows are clipped
    gen = torch.Generator().manual_seed(3)
    q = (torch.randn(B, hq, S, D, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    k = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    v = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16).cuda()
    groups = _ranks_in_one_process(lib, B * world * hq * S * D * 2, world)
    assert lib.b2a_shard_group_set_wait_ms(groups[0], 20) == 0
    d = _lib.SdpaDesc()
    d.dtype = _lib.BF16
    d.B, d.Hq, d.Hkv, d.Sq, d.Skv, d.D, d.Dv = B, hq, hkv, S, S, D, D
    d.causal = 1
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = C.c_void_p()
    rc = lib.b2a_sdpa_forward_sharded(groups[0], C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), C.byref(out),
                                      status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.DEV_TIMEOUT
    plain = b2a.sdpa(q, k, v, causal=True)
    offset = out.value - _base_of(lib, groups[0])   # which half of the staging area this step used
    for r in range(world):
        full = _device_view(_base_of(lib, groups[r]) + offset, (B, world * hq, S, D), torch.bfloat16, q.device)
        assert torch.equal(full[:, :hq], plain), f"rank {r}'s copy of rank 0's heads"
    for g in groups:
        lib.b2a_shard_group_destroy(g)


def _base_of(lib, group) -> int:
    p = C.c_void_p()
    assert lib.b2a_shard_group_output(group, C.byref(p)) == 0
    return p.value
