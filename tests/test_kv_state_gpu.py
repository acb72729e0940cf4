"""KvPoolState through the C ABI: the KV variables of a stateful model ([B, Hkv, T, D] tensors with reset / set_state /
get_state, as the reference's CudaVariableState has them) served from the paged pool.

Checks: set_state -> get_state returns the oracle's de-quantised quantisation of the tensor (bit for bit: same
quantiser, same float32 de-quantisation); append grows the state without touching the past; the attention operator
reads the pool through the step tables and matches the oracle; reset empties; export / import reproduce the pool image
exactly, through a different physical block assignment.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import quant as oquant
from oracle import sdpa as osdpa

pytestmark = pytest.mark.gpu

B, HKV, HQ, D, BS = 3, 2, 8, 128, 16


class Step(C.Structure):
    _fields_ = [("k_cache", C.c_void_p), ("v_cache", C.c_void_p), ("past_lens", C.c_void_p),
                ("subsequence_begins", C.c_void_p), ("block_indices", C.c_void_p), ("block_indices_begins", C.c_void_p),
                ("num_seqs", C.c_int32), ("num_tokens", C.c_int32), ("num_blocks_total", C.c_int32),
                ("max_context_len", C.c_int32), ("max_q_len", C.c_int32), ("prefill_row_blocks", C.c_int32),
                ("prefill_kv_tokens", C.c_int32)]


@pytest.fixture(scope="module")
def lib():
    from openvino_contrib_b200 import _lib
    assert torch.cuda.is_available()
    return _lib.load()


def _create(lib, kv_dtype, x_dtype, num_blocks=64, max_step=40):
    h = C.c_void_p()
    assert lib.b2a_kvstate_create(kv_dtype, x_dtype, B, HKV, D, BS, num_blocks, max_step, C.byref(h)) == 0
    return h


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _roundtrip_expected(x: np.ndarray) -> np.ndarray:
    q, s, z = oquant.quantize_rows(x)
    return oquant.dequantize_rows(q, s, z)


def test_set_get_reset_u8(lib):
    from openvino_contrib_b200 import _lib
    st = _create(lib, _lib.U8, _lib.F32)
    rng = np.random.default_rng(0)
    T = 53                                   # not a multiple of the block size, more than one set_state slice
    k = rng.standard_normal((B, HKV, T, D), dtype=np.float32)
    v = (rng.standard_normal((B, HKV, T, D), dtype=np.float32) * 3 + 1).astype(np.float32)
    assert lib.b2a_kvstate_length(st) == 0
    assert lib.b2a_kvstate_set_state(st, k.ctypes.data, v.ctypes.data, T, _stream()) == 0
    assert lib.b2a_kvstate_length(st) == T
    ko, vo = np.empty_like(k), np.empty_like(v)
    assert lib.b2a_kvstate_get_state(st, ko.ctypes.data, vo.ctypes.data, T, _stream()) == 0
    assert np.array_equal(ko, _roundtrip_expected(k)) and np.array_equal(vo, _roundtrip_expected(v))
    assert lib.b2a_kvstate_get_state(st, ko.ctypes.data, vo.ctypes.data, T - 1, _stream()) == 2   # wrong length
    assert lib.b2a_kvstate_reset(st) == 0 and lib.b2a_kvstate_length(st) == 0
    # a state larger than the pool is refused and leaves the (empty) state as it was
    big = np.zeros((B, HKV, 64 * BS, D), np.float32)
    assert lib.b2a_kvstate_set_state(st, big.ctypes.data, big.ctypes.data, 64 * BS, _stream()) == 8
    assert lib.b2a_kvstate_length(st) == 0
    lib.b2a_kvstate_destroy(st)


def test_append_then_attention_matches_oracle(lib):
    import openvino_contrib_b200 as b2a
    from openvino_contrib_b200 import _lib
    st = _create(lib, _lib.U8, _lib.F16)
    g = torch.Generator().manual_seed(1)
    steps = [37, 1, 1, 20]                    # a prefill, two decode steps, a chunk of 20
    k_all = torch.randn(B, HKV, sum(steps), D, generator=g).to(torch.float16)
    v_all = torch.randn(B, HKV, sum(steps), D, generator=g).to(torch.float16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = 0
    for q_len in steps:
        kn = k_all[:, :, t0:t0 + q_len].contiguous().cuda()
        vn = v_all[:, :, t0:t0 + q_len].contiguous().cuda()
        assert lib.b2a_kvstate_append(st, kn.data_ptr(), vn.data_ptr(), q_len, status.data_ptr(), _stream()) == 0
        t0 += q_len
        assert lib.b2a_kvstate_length(st) == t0
        step = Step()
        assert lib.b2a_kvstate_last_step(st, C.byref(step)) == 0
        assert (step.num_seqs, step.num_tokens, step.max_context_len, step.max_q_len) == (B, B * q_len, t0, q_len)
        # the attention operator over the state: queries of this step's tokens, [B*q, Hq*D] token-major
        q = torch.randn(B * q_len, HQ * D, generator=g).to(torch.float16)
        d = _lib.PagedDesc()
        d.q_dtype, d.kv_dtype = _lib.F16, _lib.U8
        d.Hq, d.Hkv, d.D, d.Dv, d.block_size = HQ, HKV, D, D, BS
        d.num_seqs, d.num_tokens, d.num_blocks_total = step.num_seqs, step.num_tokens, step.num_blocks_total
        d.max_context_len, d.max_q_len = step.max_context_len, step.max_q_len
        need = C.c_size_t(0)
        assert lib.b2a_paged_workspace_bytes(C.byref(d), 0, C.byref(need)) == 0
        ws = torch.empty(max(16, need.value), dtype=torch.uint8, device="cuda")
        out = torch.empty(B * q_len, HQ * D, dtype=torch.float16, device="cuda")
        qd = q.cuda()
        assert lib.b2a_paged_attention(C.byref(d), qd.data_ptr(), step.k_cache, step.v_cache, step.past_lens,
                                       step.subsequence_begins, step.block_indices, step.block_indices_begins,
                                       out.data_ptr(), ws.data_ptr(), ws.numel(), status.data_ptr(), _stream()) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        # oracle: dense attention of the step's queries over the de-quantised state, causal inside the step
        kd = _roundtrip_expected(k_all[:, :, :t0].float().numpy())
        vd = _roundtrip_expected(v_all[:, :, :t0].float().numpy())
        qs = q.float().numpy().reshape(B, q_len, HQ, D).transpose(0, 2, 1, 3)          # [B, Hq, q, D]
        keep = (np.arange(t0)[None, :] <= (t0 - q_len + np.arange(q_len))[:, None])
        ref = osdpa.sdpa_ref(qs, kd, vd, mask=keep[None, None])                          # [B, Hq, q, D]
        got = out.float().cpu().numpy().reshape(B, q_len, HQ, D).transpose(0, 2, 1, 3)
        np.testing.assert_allclose(got, ref, atol=2e-3, rtol=1e-2)
    # the dense view an operation would read (ReadValue): the whole state, the past untouched by the appends
    kd_dev = torch.empty(B, HKV, t0, D, dtype=torch.float16, device="cuda")
    vd_dev = torch.empty_like(kd_dev)
    assert lib.b2a_kvstate_read_dense(st, kd_dev.data_ptr(), vd_dev.data_ptr(), t0, status.data_ptr(), _stream()) == 0
    torch.cuda.synchronize()
    expect = torch.from_numpy(_roundtrip_expected(k_all.float().numpy())).to(torch.float16)
    assert torch.equal(kd_dev.cpu(), expect)
    lib.b2a_kvstate_destroy(st)


@pytest.mark.parametrize("kv", ["u8", "f16"])
def test_export_import_is_exact(lib, kv):
    from openvino_contrib_b200 import _lib
    kv_dtype = _lib.U8 if kv == "u8" else _lib.F16
    a = _create(lib, kv_dtype, _lib.F16)
    g = torch.Generator().manual_seed(2)
    T = 45
    k = torch.randn(B, HKV, T, D, generator=g).to(torch.float16)
    v = torch.randn(B, HKV, T, D, generator=g).to(torch.float16)
    assert lib.b2a_kvstate_set_state(a, k.data_ptr(), v.data_ptr(), T, _stream()) == 0
    n = lib.b2a_kvstate_export_bytes(a)
    blob = np.empty(n, np.uint8)
    assert lib.b2a_kvstate_export(a, blob.ctypes.data, n, _stream()) == 0
    # into a second state whose free list has been stirred (different physical blocks), through the exact image
    b = _create(lib, kv_dtype, _lib.F16)
    junk = torch.zeros(B, HKV, 20, D, dtype=torch.float16)
    assert lib.b2a_kvstate_set_state(b, junk.data_ptr(), junk.data_ptr(), 20, _stream()) == 0
    assert lib.b2a_kvstate_import(b, blob.ctypes.data, n, _stream()) == 0
    assert lib.b2a_kvstate_length(b) == T
    blob2 = np.empty(n, np.uint8)
    assert lib.b2a_kvstate_export(b, blob2.ctypes.data, n, _stream()) == 0
    assert np.array_equal(blob, blob2)
    ka, kb = torch.empty_like(k), torch.empty_like(k)
    va, vb = torch.empty_like(v), torch.empty_like(v)
    assert lib.b2a_kvstate_get_state(a, ka.data_ptr(), va.data_ptr(), T, _stream()) == 0
    assert lib.b2a_kvstate_get_state(b, kb.data_ptr(), vb.data_ptr(), T, _stream()) == 0
    assert torch.equal(ka, kb) and torch.equal(va, vb)
    if kv == "f16":
        assert torch.equal(ka, k)            # an f16 pool holds the values themselves
    # an image of another geometry is refused
    c = C.c_void_p()
    assert lib.b2a_kvstate_create(kv_dtype, _lib.F16, B + 1, HKV, D, BS, 64, 40, C.byref(c)) == 0
    assert lib.b2a_kvstate_import(c, blob.ctypes.data, n, _stream()) == 2
    for h in (a, b, c):
        lib.b2a_kvstate_destroy(h)
