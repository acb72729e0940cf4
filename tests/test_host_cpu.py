"""Host-side logic and the C ABI surface, without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from openvino_contrib_b200 import _lib
from openvino_contrib_b200.build import build_library

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "b2a.h")).read()
    declared = set(re.findall(r"\b(b2a_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found in include/b2a.h"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.b2a_version() >= 100
    assert lib.b2a_status_string(0) == b"ok"


def test_descriptor_validation_happens_before_any_launch(lib):
    d = _lib.SdpaDesc()
    ws = C.c_size_t(7)
    assert lib.b2a_sdpa_workspace_bytes(None, 148, C.byref(ws)) == 1           # NULL
    assert lib.b2a_sdpa_workspace_bytes(C.byref(d), 148, C.byref(ws)) == 2     # dtype 0 = f32 is fine, dims are 0
    d.dtype = 9
    assert lib.b2a_sdpa_workspace_bytes(C.byref(d), 148, C.byref(ws)) == 3     # DTYPE
    d.dtype = _lib.BF16
    d.B, d.Hq, d.Hkv, d.Sq, d.Skv, d.D, d.Dv = 1, 6, 4, 8, 8, 64, 64
    assert lib.b2a_sdpa_workspace_bytes(C.byref(d), 148, C.byref(ws)) == 2     # Hq % Hkv
    d.Hkv = 2
    assert lib.b2a_sdpa_workspace_bytes(C.byref(d), 148, C.byref(ws)) == 0 and ws.value == 0
    assert lib.b2a_sdpa_forward(C.byref(d), None, None, None, None, None, None, 0, None, None) == 1
    d.q_strides[:] = (1, 1, 1, 2)  # innermost stride must be 1
    assert lib.b2a_sdpa_forward(C.byref(d), 16, 16, 16, None, 16, None, 0, None, None) == 4

    p = _lib.PagedDesc()
    p.q_dtype, p.kv_dtype = _lib.F16, _lib.U8
    p.Hq, p.Hkv, p.D, p.Dv, p.block_size = 32, 8, 128, 128, 16
    p.num_seqs, p.num_tokens, p.num_blocks_total, p.max_context_len, p.max_q_len = 64, 64, 100, 8192, 1
    assert lib.b2a_paged_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 0 and ws.value > 0
    splits = ws.value // (64 * 32 * 130 * 4)
    assert ws.value == splits * 64 * 32 * 130 * 4 and 1 <= splits <= 512
    p.kv_dtype = _lib.F32
    assert lib.b2a_paged_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 3
    p.kv_dtype = _lib.U8
    # decode launch without a workspace is refused on the host (needs a device only to read the SM count)
    assert lib.b2a_paged_chunk_bytes(_lib.U8, 16, 128) == 2112
    assert lib.b2a_paged_chunk_bytes(_lib.BF16, 16, 128) == 4096
    assert lib.b2a_paged_chunk_bytes(_lib.F32, 16, 128) == 0


def test_decode_chunk_plan(lib):
    """The split-K plan as it shows in the workspace size (seqs * Hq * splits * 130 floats), for 148 SMs."""
    ws = C.c_size_t(0)

    def splits(hq, hkv, seqs, max_ctx):
        p = _lib.PagedDesc()
        p.q_dtype, p.kv_dtype = _lib.F16, _lib.U8
        p.Hq, p.Hkv, p.D, p.Dv, p.block_size = hq, hkv, 128, 128, 16
        p.num_seqs, p.num_tokens, p.num_blocks_total, p.max_context_len, p.max_q_len = seqs, seqs, 1 << 20, max_ctx, 1
        assert lib.b2a_paged_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 0
        per_split = seqs * hq * 130 * 4
        assert ws.value % per_split == 0
        return ws.value // per_split

    assert splits(32, 8, 64, 8192) == 4      # 64 ragged sequences: 128-block chunks, the longest sequence in 4
    assert splits(64, 8, 16, 32768) == 16    # 16 x 32768: 128-block chunks
    assert splits(8, 1, 16, 32768) == 16     # its one-head shard: still long chunks, at most 16 per sequence
    assert splits(4, 1, 64, 8192) == 10      # the ragged batch's one-head shard: 56-block chunks fill the slots
    assert splits(32, 8, 4, 64) == 1         # tiny step: one chunk per sequence
    assert splits(16, 2, 16, 32768) == 19    # two-head shard: 112-block chunks, one wave of 4 CTAs per SM


def test_score_entry_points_validate_on_the_host(lib):
    """b2a_paged_scores_workspace_bytes / b2a_paged_last_token_scores refuse on the host what the score kernels do not
    take (no GPU needed: every check comes before the first launch)."""
    ws = C.c_size_t(0)
    p = _lib.PagedDesc()
    p.q_dtype, p.kv_dtype = _lib.F16, _lib.U8
    p.Hq, p.Hkv, p.D, p.Dv, p.block_size = 32, 8, 128, 128, 16
    p.num_seqs, p.num_tokens, p.num_blocks_total, p.max_context_len, p.max_q_len = 64, 64, 100, 8192, 1
    assert lib.b2a_paged_scores_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 0 and ws.value > 0
    small = ws.value
    p.max_context_len = 32768
    assert lib.b2a_paged_scores_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 0 and ws.value >= small
    assert lib.b2a_paged_scores_workspace_bytes(C.byref(p), 148, None) == 1                     # NULL
    p.D = p.Dv = 64
    assert lib.b2a_paged_scores_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 7              # head size
    p.D = p.Dv = 128
    p.Hq = 128                                                                                  # 16 query heads per KV head
    assert lib.b2a_paged_scores_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 7
    p.Hq = 32
    p.kv_dtype = _lib.F16
    assert lib.b2a_paged_scores_workspace_bytes(C.byref(p), 148, C.byref(ws)) == 7              # only u8 caches
    p.kv_dtype = _lib.U8
    assert lib.b2a_paged_last_token_scores(C.byref(p), None, None, None, None, None, None, None, 0, None, None, 0,
                                           None, None) == 1                                      # NULL operands
    assert lib.b2a_paged_last_token_scores(C.byref(p), 16, 16, 16, 16, 16, 16, 16, -1, 16, 16, 1 << 30, None, None) == 2


def test_kv_block_manager_tables():
    from openvino_contrib_b200 import KvBlockManager
    from openvino_contrib_b200._lib import B2AError
    m = KvBlockManager(num_blocks=10, block_size=16)
    for s in (7, 8, 9):
        m.add_sequence(s)
    with pytest.raises(B2AError):
        m.add_sequence(7)
    past, sb, bi, bb, mctx = m.schedule_step([7, 8, 9], [33, 16, 1])  # prefill: 3 + 1 + 1 blocks
    assert past.tolist() == [0, 0, 0] and sb.tolist() == [0, 33, 49, 50]
    assert bb.tolist() == [0, 3, 4, 5] and sorted(bi.tolist()) == [0, 1, 2, 3, 4] and mctx == 33
    assert m.free_blocks == 5 and m.sequence_len(7) == 33
    # the two hints a step descriptor can carry: 128-row blocks and 128-rounded contexts of the multi-token sequences
    assert m.last_prefill_row_blocks == 2 and m.last_prefill_kv_tokens == 256
    past, sb, bi2, bb, mctx = m.schedule_step([8, 7], [1, 15])  # decode-like: seq 8 crosses into a new block
    assert past.tolist() == [16, 33] and bb.tolist() == [0, 2, 5] and mctx == 48
    assert m.last_prefill_row_blocks == 1 and m.last_prefill_kv_tokens == 128  # only the 15-token continuation
    assert bi2[0] == bi[3] and bi2[2:5].tolist() == bi[0:3].tolist() and m.free_blocks == 4
    # all-or-nothing on exhaustion: nothing changes
    with pytest.raises(B2AError) as e:
        m.schedule_step([9], [16 * 5])
    assert e.value.code == 8 and m.sequence_len(9) == 1 and m.free_blocks == 4
    with pytest.raises(B2AError) as e:
        m.schedule_step([42], [1])
    assert e.value.code == 9
    m.free_sequence(7)
    assert m.free_blocks == 7 and m.sequence_len(7) == -1
    # freed blocks are reused
    m.add_sequence(10)
    _, _, bi3, _, _ = m.schedule_step([10], [48])
    assert set(bi3.tolist()) <= set(range(10)) and m.free_blocks == 4


def test_kv_block_manager_shuffle_is_a_permutation():
    from openvino_contrib_b200 import KvBlockManager
    m = KvBlockManager(num_blocks=257, block_size=16, shuffle_seed=12345)
    m.add_sequence(1)
    _, _, bi, _, _ = m.schedule_step([1], [257 * 16])
    assert sorted(bi.tolist()) == list(range(257)) and bi.tolist() != list(range(257))
    m2 = KvBlockManager(num_blocks=257, block_size=16, shuffle_seed=12345)
    m2.add_sequence(1)
    assert m2.schedule_step([1], [257 * 16])[2].tolist() == bi.tolist()  # reproducible


def test_no_cpu_fallback():
    import torch
    from openvino_contrib_b200 import sdpa
    x = torch.zeros(1, 1, 4, 8)
    with pytest.raises(ValueError):
        sdpa(x, x, x)


def test_python_operator_work_buffer_covers_every_step_of_its_capacity(lib):
    """The Python twin of the C++ capacity test: the operator's work-buffer request is at least what the library
    asks for any step the capacity admits, with and without a scratch reserve, whatever the hints."""
    import torch
    from openvino_contrib_b200 import B2AError, PagedAttentionOp
    from openvino_contrib_b200.ops import paged_workspace_bytes
    for reserve in (0, 2048):
        op = PagedAttentionOp(32, 8, 128, 16, torch.uint8, max_seqs=24, max_context_len=4096,
                              max_prefill_kv_tokens=reserve, q_dtype=torch.bfloat16)
        have = op.GetWorkBufferRequest()["mutable_sizes"][0]
        cache, worst = op._geometry(), 0
        for n in range(1, op.max_seqs + 1):
            for tokens in (n, n + 1, n + 500, op.max_step_tokens):
                for hints in ((0, 0), (3, 384), (1 << 20, 1 << 20)):
                    rb, kvt = op.step_hints(tokens, n, *hints)
                    assert kvt <= reserve and rb <= tokens // 128 + n
                    need = paged_workspace_bytes(torch.bfloat16, cache, 32, n, tokens, op.max_context_len,
                                                 tokens - n + 1, rb, kvt)
                    assert need <= have, (reserve, n, tokens, hints)
                    worst = max(worst, need)
        assert 2 * worst > have
    # constants arriving as device tensors would make Execute wait for the device: refused
    from openvino_contrib_b200.ops import _host_scalar
    assert _host_scalar(0.5, "x") == 0.5 and _host_scalar(torch.tensor(3), "x") == 3 and _host_scalar(None, "x") is None
