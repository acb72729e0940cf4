"""Score output of the paged attention (b2a_paged_last_token_scores) against the oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from oracle import paged as opaged
from tests.helpers import PagedWorkload

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b2a():
    import openvino_contrib_b200 as m
    assert torch.cuda.is_available()
    return m


def _round(a, dtype):
    return torch.from_numpy(a).to(dtype)


def _check(b2a, w, dtype, window=0, scale=None):
    q = _round(w.query, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scores, begins = b2a.paged_last_token_scores(q.cuda(), w.device_cache(), *w.device_tables(), hq=w.hq,
                                                 max_context_len=int(w.ctx.max()), scale=scale, sliding_window=window,
                                                 status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref, ref_begins = opaged.last_token_scores_ref(q.float().numpy(), w.k_cache, w.past, w.sb, w.bi, w.bb, w.hq, w.hkv,
                                                   w.d, w.bs, scale, window)
    assert np.array_equal(begins.cpu().numpy(), ref_begins)
    got = scores.cpu().numpy()[: ref_begins[-1]]
    # probabilities: f32 accumulation of exact f16 products, ex2.approx (2 ulp) - the floating-point bar of f32 outputs
    np.testing.assert_allclose(got, ref, atol=2e-5 * w.hq, rtol=2e-3)
    for s in range(len(w.ctx)):
        seg = got[ref_begins[s]:ref_begins[s + 1]]
        if len(seg):
            assert abs(float(seg.sum()) - w.hq) < 1e-2 * w.hq   # every head's probabilities sum to one


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ctx,hq,hkv", [
    ([1, 16, 17, 300], 32, 8),          # one key; exactly one block; one key into the second block
    ([5, 64, 129, 2048, 4099], 64, 8),  # GQA 8, several chunks per sequence
    ([7, 300], 8, 8),                   # no grouping
    ([40, 9000], 12, 4),                # GQA 3: unused columns of the score tile
    ([33], 2, 1),                       # one KV head
])
def test_decode_rows(b2a, dtype, ctx, hq, hkv):
    _check(b2a, PagedWorkload(ctx, [1] * len(ctx), hq, hkv, 128, seed=3 * hq + len(ctx)), dtype)


def test_last_row_of_prefill_and_idle_sequences(b2a):
    # the last of several new tokens is the row that is scored; a sequence without a new token has no entries
    past = np.array([0, 40, 99, 16, 0], np.int64)
    qlen = np.array([70, 25, 1, 0, 130], np.int32)
    _check(b2a, PagedWorkload(past + qlen, qlen, 16, 4, 128, seed=5), torch.float16)


@pytest.mark.parametrize("window", [1, 16, 100, 4096])
def test_sliding_window_and_scale(b2a, window):
    _check(b2a, PagedWorkload([9, 250, 1500], [1, 1, 1], 32, 8, 128, seed=8), torch.float16, window=window, scale=0.05)


def test_buffer_too_small_is_reported_and_respected(b2a):
    w = PagedWorkload([100, 200], [1, 1], 16, 2, 128, seed=9)
    q = _round(w.query, torch.float16).cuda()
    scores = torch.full((250,), -7.0, dtype=torch.float32, device="cuda")   # room for the first sequence only
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    from openvino_contrib_b200 import _lib
    out, begins = b2a.paged_last_token_scores(q, w.device_cache(), *w.device_tables(), hq=16, max_context_len=200,
                                              scores=scores, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & _lib.DEV_BAD_LEN
    assert begins.cpu().tolist() == [0, 100, 300]
    ref, _ = opaged.last_token_scores_ref(q.float().cpu().numpy(), w.k_cache, w.past, w.sb, w.bi, w.bb, 16, 2, 128, 16)
    np.testing.assert_allclose(out[:100].cpu().numpy(), ref[:100], atol=4e-4, rtol=2e-3)
    assert bool((out[100:] == -7.0).all())   # the sequence that does not fit is left alone


def test_config3_shape(b2a):
    ctx = np.random.default_rng(2).integers(512, 8193, size=64)
    _check(b2a, PagedWorkload(ctx, [1] * 64, 32, 8, 128, seed=31), torch.float16)


def test_graph_replay_with_new_lengths(b2a):
    w = PagedWorkload([700, 90, 4000], [1, 1, 1], 32, 8, 128, seed=12)
    q = _round(w.query, torch.float16).cuda()
    cache = w.device_cache()
    past, sb, bi, bb = w.device_tables()
    scores = torch.zeros(3 * 4096, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ws = torch.empty(1 << 22, dtype=torch.uint8, device="cuda")
    begins = []

    def run():
        begins.append(b2a.paged_last_token_scores(q, cache, past, sb, bi, bb, hq=32, max_context_len=4096,
                                                  scores=scores, workspace=ws, status=status)[1])
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            run()
    torch.cuda.current_stream().wait_stream(side)
    new_past = np.array([500, 10, 2000], np.int32)    # shorter contexts: same tables, other lengths
    past.copy_(torch.from_numpy(new_past))
    g.replay()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref, rb = opaged.last_token_scores_ref(q.float().cpu().numpy(), w.k_cache, new_past, w.sb, w.bi, w.bb, 32, 8, 128, 16)
    assert np.array_equal(begins[-1].cpu().numpy(), rb)
    np.testing.assert_allclose(scores.cpu().numpy()[: rb[-1]], ref, atol=2e-5 * 32, rtol=2e-3)


def test_second_output_of_the_operator(b2a):
    # a mixed step through the operator: its second output carries the scores of every sequence's last new token
    hq, hkv, d, bs = 16, 4, 128, 16
    past = np.array([0, 40, 99], np.int32)
    qlen = np.array([70, 25, 1], np.int32)
    w = PagedWorkload(past + qlen, qlen, hq, hkv, d, seed=14)
    rng = np.random.default_rng(6)
    nk = _round(rng.standard_normal((int(w.sb[-1]), hkv * d), dtype=np.float32), torch.float16)
    nv = _round(rng.standard_normal((int(w.sb[-1]), hkv * d), dtype=np.float32), torch.float16)
    ref_k = w.k_cache.copy()
    opaged.kv_store_ref(nk, ref_k, w.past, w.sb, w.bi, w.bb, hkv, d, bs)
    q = _round(w.query, torch.float16)
    ref, ref_begins = opaged.last_token_scores_ref(q.float().numpy(), ref_k, w.past, w.sb, w.bi, w.bb, hq, hkv, d, bs)
    op = b2a.PagedAttentionOp(hq, hkv, d, bs, torch.uint8, max_seqs=4, max_context_len=256, q_dtype=torch.float16)
    wb = {"mutable": [torch.empty(n, dtype=torch.uint8, device="cuda") for n in op.GetWorkBufferRequest()["mutable_sizes"]]}
    cache = w.device_cache()
    out = torch.empty(int(w.sb[-1]), hq * d, dtype=torch.float16, device="cuda")
    scores = torch.zeros(4 * 256, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    begins = op.Execute([q.cuda(), nk.cuda(), nv.cuda(), cache.k, cache.v, *w.device_tables(), None, 0, None, 256],
                        [out, scores], workbuffers=wb, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(begins.cpu().numpy(), ref_begins)
    np.testing.assert_allclose(scores.cpu().numpy()[: ref_begins[-1]], ref, atol=2e-5 * hq, rtol=2e-3)
