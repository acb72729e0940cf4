"""PagedAttentionExtension on the GPU, through the C ABI, against the oracle: the u8 bytes and the indices
bit for bit, the attention outputs within the half-precision bar."""
import os

import numpy as np
import pytest
import torch

from oracle import paged as opaged
from oracle import quant as oquant
from tests.helpers import PagedWorkload, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b2a():
    import openvino_contrib_b200 as m
    assert torch.cuda.is_available()
    return m


def _round(x: np.ndarray, dtype) -> torch.Tensor:
    return torch.from_numpy(x).to(dtype)


# ---------------------------------------------------------------- KV store: bit-exact

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d", [128, 64, 80])
def test_kv_store_bit_exact(b2a, dtype, d):
    hkv, bs = 4, 16
    ctx = np.array([1, 15, 16, 17, 33, 250])
    past = np.array([0, 3, 15, 16, 0, 200], dtype=np.int32)
    qlen = (ctx - past).astype(np.int32)
    bi, bb, nb = opaged.build_block_tables(ctx, bs, seed=5, spare_blocks=3)
    sb = np.zeros(len(ctx) + 1, np.int32)
    sb[1:] = np.cumsum(qlen)
    g = torch.Generator().manual_seed(1)
    key = (torch.randn(int(sb[-1]), hkv * d, generator=g) * 1.7).to(dtype)
    val = (torch.randn(int(sb[-1]), hkv * d, generator=g) + 0.3).to(dtype)
    val[0] = 0.75                      # constant rows: the scale guard
    key[1, :d] = 0.0
    cache = b2a.PagedKvCache.allocate(nb, hkv, d, bs, torch.uint8)
    t = [torch.from_numpy(a).cuda() for a in (past, sb, bi, bb)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    b2a.paged_kv_store(key.cuda(), val.cuda(), cache, *t, status=status)
    ref_k = np.full((nb, hkv, bs * (d + 4)), 0xFF, np.uint8)
    ref_v = ref_k.copy()
    wk = opaged.kv_store_ref(key, ref_k, past, sb, bi, bb, hkv, d, bs)
    opaged.kv_store_ref(val, ref_v, past, sb, bi, bb, hkv, d, bs)
    assert int(status.item()) == 0
    assert np.array_equal(cache.k.cpu().numpy(), ref_k)   # codes, f16 scales, f16 zero-points, untouched poison
    assert np.array_equal(cache.v.cpu().numpy(), ref_v)
    assert len(wk) == int(sb[-1])


def test_kv_store_into_f16_cache(b2a):
    hkv, d, bs = 2, 64, 16
    ctx = np.array([20, 5])
    bi, bb, nb = opaged.build_block_tables(ctx, bs, seed=1)
    past = np.zeros(2, np.int32)
    sb = np.array([0, 20, 25], np.int32)
    key = torch.randn(25, hkv * d, generator=torch.Generator().manual_seed(2)).to(torch.float16)
    cache = b2a.PagedKvCache.allocate(nb, hkv, d, bs, torch.float16, poison=0)
    t = [torch.from_numpy(a).cuda() for a in (past, sb, bi, bb)]
    b2a.paged_kv_store(key.cuda(), key.cuda(), cache, *t)
    kc = cache.k.cpu().view(torch.float16).reshape(nb, hkv, bs, d)
    for s in range(2):
        for i in range(int(ctx[s])):
            blk = int(bi[bb[s] + i // bs])
            assert torch.equal(kc[blk, :, i % bs], key[sb[s] + i].reshape(hkv, d))


# ---------------------------------------------------------------- decode

DECODE_CASES = [
    # (context lens, Hq, Hkv)
    ([1, 15, 16, 17, 33, 100, 1000, 4097], 32, 8),   # GQA 4
    ([5, 64, 129, 2048], 64, 8),                     # GQA 8
    ([7, 300], 8, 8),                                # no grouping
    ([31, 32, 513], 32, 2),                          # GQA 16
    ([40, 9000], 12, 4),                             # GQA 3
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("ctx,hq,hkv", DECODE_CASES)
def test_decode_parity(b2a, dtype, ctx, hq, hkv):
    w = PagedWorkload(ctx, [1] * len(ctx), hq, hkv, 128, seed=hq + len(ctx))
    q = _round(w.query, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=hq, max_context_len=max(ctx),
                              max_q_len=1, status=status)
    assert int(status.item()) == 0
    assert_close(out, w.reference(q.float().numpy()), dtype)


def test_decode_grid_sized_for_longer_contexts(b2a):
    # a launch sized for max_context_len 8192 serves shorter contexts (graph replay with changing lengths)
    ctx = [3, 700]
    w = PagedWorkload(ctx, [1, 1], 32, 8, 128, seed=3)
    q = _round(w.query, torch.float16)
    out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=32, max_context_len=8192, max_q_len=1)
    assert_close(out, w.reference(q.float().numpy()), torch.float16)


def test_decode_sliding_window_and_scale(b2a):
    ctx = [10, 100, 1000]
    w = PagedWorkload(ctx, [1] * 3, 32, 8, 128, seed=4)
    q = _round(w.query, torch.float16)
    for win in (1, 16, 50, 4096):
        out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=32, max_context_len=1000,
                                  max_q_len=1, scale=0.05, sliding_window=win)
        assert_close(out, w.reference(q.float().numpy(), scale=0.05, sliding_window=win), torch.float16, f"win={win}")


def test_decode_constant_values_and_table_permutation(b2a):
    # V rows constant per sequence -> the output is that constant whatever the scores are (up to the u8 step);
    # re-shuffling the physical placement leaves the result bit-identical.
    ctx = [4000, 777]
    consts = [0.5, -1.25]
    vf = lambda s, n: np.full((n, 8, 128), consts[s], np.float32)
    w1 = PagedWorkload(ctx, [1, 1], 32, 8, 128, seed=6, table_seed=1, value_fn=vf)
    w2 = PagedWorkload(ctx, [1, 1], 32, 8, 128, seed=6, table_seed=2, value_fn=vf)
    assert not np.array_equal(w1.bi, w2.bi)
    q = _round(w1.query, torch.float16).cuda()
    o1 = b2a.paged_attention(q, w1.device_cache(), *w1.device_tables(), hq=32, max_context_len=4000, max_q_len=1)
    o2 = b2a.paged_attention(q, w2.device_cache(), *w2.device_tables(), hq=32, max_context_len=4000, max_q_len=1)
    assert torch.equal(o1, o2)
    for s in range(2):
        np.testing.assert_allclose(o1[s].float().cpu().numpy(), consts[s], atol=2e-3)


def test_bad_block_index_is_reported_not_followed(b2a):
    w = PagedWorkload([100, 50], [1, 1], 32, 8, 128, seed=8)
    past, sb, bi, bb = w.device_tables()
    bi = bi.clone()
    bi[2] = w.nb + 1000  # far outside the pool
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = _round(w.query, torch.float16).cuda()
    out = b2a.paged_attention(q, w.device_cache(), past, sb, bi, bb, hq=32, max_context_len=100, max_q_len=1,
                              status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & 2
    assert torch.isfinite(out.float()).all()
    # the untouched sequence is still right
    ref = w.reference(q.float().cpu().numpy())
    assert_close(out[1], ref[1], torch.float16)


def test_decode_graph_replay_with_new_lengths(b2a):
    ctx = [900, 1500, 64]
    w = PagedWorkload(ctx, [1] * 3, 32, 8, 128, seed=9)
    cache = w.device_cache()
    past, sb, bi, bb = w.device_tables()
    q = _round(w.query, torch.float16).cuda()
    out = torch.empty_like(q)
    ws = torch.empty(b2a.ops.paged_workspace_bytes(torch.float16, cache, 32, 3, 3, 2048, 1), dtype=torch.uint8,
                     device="cuda")
    run = lambda stream=None: b2a.paged_attention(q, cache, past, sb, bi, bb, hq=32, max_context_len=2048,
                                                  max_q_len=1, out=out, workspace=ws, stream=stream)
    run()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            run(s)
    # same pool, shorter histories: only past_lens changes on the device
    new_past = np.array([500, 1499, 10], np.int32)
    past.copy_(torch.from_numpy(new_past))
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    ref = opaged.paged_attention_ref(q.float().cpu().numpy(), w.k_cache, w.v_cache, new_past, w.sb, w.bi, w.bb,
                                     32, 8, 128, 16)
    assert_close(out, ref, torch.float16)


# ---------------------------------------------------------------- multi-token rows (general kernel)

def test_reference_golden_paged_vectors(b2a, golden_dir):
    g = np.load(os.path.join(golden_dir, "paged_reference.npz"))
    hq, hkv, d, bs = (int(x) for x in g["geom"])
    cache = b2a.PagedKvCache(torch.from_numpy(g["k_cache"]).cuda(), torch.from_numpy(g["v_cache"]).cuda(),
                             hkv, d, d, bs, torch.uint8)
    t = [torch.from_numpy(g[n]).cuda() for n in ("past_lens", "subsequence_begins", "block_indices",
                                                 "block_indices_begins")]
    qlen = np.diff(g["subsequence_begins"])
    ctx = int((g["past_lens"] + qlen).max())
    out = b2a.paged_attention(torch.from_numpy(g["query"]).cuda(), cache, *t, hq=hq, max_context_len=ctx,
                              max_q_len=int(qlen.max()))
    assert_close(out, g["out"], torch.float32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_mixed_step_through_the_operator(b2a, dtype):
    # two prefill sequences, one chunked-prefill continuation, three decode sequences, one idle sequence
    hq, hkv, d, bs = 16, 4, 128, 16
    past = np.array([0, 0, 40, 99, 16, 511, 30], np.int32)
    qlen = np.array([70, 33, 25, 1, 1, 1, 0], np.int32)
    ctx = past + qlen
    w = PagedWorkload(ctx, qlen, hq, hkv, d, seed=12)
    # pools holding only the past; this step's rows go in through the operator
    rng = np.random.default_rng(5)
    new_k = rng.standard_normal((int(w.sb[-1]), hkv * d), dtype=np.float32)
    new_v = rng.standard_normal((int(w.sb[-1]), hkv * d), dtype=np.float32)
    nk, nv = _round(new_k, dtype), _round(new_v, dtype)
    ref_k, ref_v = w.k_cache.copy(), w.v_cache.copy()
    opaged.kv_store_ref(nk, ref_k, w.past, w.sb, w.bi, w.bb, hkv, d, bs)
    opaged.kv_store_ref(nv, ref_v, w.past, w.sb, w.bi, w.bb, hkv, d, bs)
    q = _round(w.query, dtype)
    ref = opaged.paged_attention_ref(q.float().numpy(), ref_k, ref_v, w.past, w.sb, w.bi, w.bb, hq, hkv, d, bs)

    op = b2a.PagedAttentionOp(hq, hkv, d, bs, torch.uint8, max_seqs=8, max_context_len=1024, q_dtype=dtype)
    wb = {"mutable": [torch.empty(n, dtype=torch.uint8, device="cuda") for n in op.GetWorkBufferRequest()["mutable_sizes"]]}
    cache = w.device_cache()
    out = torch.empty(int(w.sb[-1]), hq * d, dtype=dtype, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    op.Execute([q.cuda(), nk.cuda(), nv.cuda(), cache.k, cache.v, *w.device_tables(), None, 0, None, int(ctx.max())],
               [out], workbuffers=wb, status=status)
    assert int(status.item()) == 0
    assert np.array_equal(cache.k.cpu().numpy(), ref_k) and np.array_equal(cache.v.cpu().numpy(), ref_v)
    assert_close(out, ref, dtype)


def test_decode_steps_through_the_operator_see_their_new_tokens(b2a):
    # Pure decode steps through the operator: its attention call promises that only the new tokens' rows changed
    # (cache_rows_settled), so the decode kernel copies earlier blocks while the store kernel before it still runs.
    # Three consecutive steps in one captured graph (store, attention, store, attention, ...: every attention kernel
    # is launched while a store kernel drains); every step's new row - first row of a fresh block, last row of a
    # block, somewhere inside - must be seen, and nothing else may differ from the oracle.
    hq, hkv, d, bs = 32, 4, 128, 16
    past0 = np.array([15, 16, 31, 700, 4095, 2050], np.int32)
    steps = 3
    n = len(past0)
    w = PagedWorkload(past0 + steps, [1] * n, hq, hkv, d, seed=77)   # tables sized for the last step's contexts
    rng = np.random.default_rng(78)
    new_k = [_round(rng.standard_normal((n, hkv * d), dtype=np.float32), torch.float16) for _ in range(steps)]
    new_v = [_round(rng.standard_normal((n, hkv * d), dtype=np.float32), torch.float16) for _ in range(steps)]
    qs = [_round(rng.standard_normal((n, hq * d), dtype=np.float32), torch.float16) for _ in range(steps)]
    sb = np.arange(n + 1, dtype=np.int32)
    ref_k, ref_v = w.k_cache.copy(), w.v_cache.copy()
    refs = []
    for i in range(steps):
        past = (past0 + i).astype(np.int32)
        opaged.kv_store_ref(new_k[i], ref_k, past, sb, w.bi, w.bb, hkv, d, bs)
        opaged.kv_store_ref(new_v[i], ref_v, past, sb, w.bi, w.bb, hkv, d, bs)
        refs.append(opaged.paged_attention_ref(qs[i].float().numpy(), ref_k, ref_v, past, sb, w.bi, w.bb, hq, hkv, d, bs))

    op = b2a.PagedAttentionOp(hq, hkv, d, bs, torch.uint8, max_seqs=8, max_context_len=8192, q_dtype=torch.float16)
    wb = {"mutable": [torch.empty(m, dtype=torch.uint8, device="cuda") for m in op.GetWorkBufferRequest()["mutable_sizes"]]}
    cache = w.device_cache()
    _, sb_d, bi_d, bb_d = w.device_tables()
    pasts = [torch.from_numpy((past0 + i).astype(np.int32)).cuda() for i in range(steps)]
    dk, dv, dq = [t.cuda() for t in new_k], [t.cuda() for t in new_v], [t.cuda() for t in qs]
    outs = [torch.empty(n, hq * d, dtype=torch.float16, device="cuda") for _ in range(steps)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run():
        for i in range(steps):
            op.Execute([dq[i], dk[i], dv[i], cache.k, cache.v, pasts[i], sb_d, bi_d, bb_d, None, 0, None, 8192],
                       [outs[i]], workbuffers=wb, status=status)

    pool_k, pool_v = cache.k.clone(), cache.v.clone()
    run()                                   # eager
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for i in range(steps):
        assert_close(outs[i], refs[i], torch.float16)
    assert np.array_equal(cache.k.cpu().numpy(), ref_k) and np.array_equal(cache.v.cpu().numpy(), ref_v)
    eager = [o.clone() for o in outs]
    cache.k.copy_(pool_k)                   # the same three steps again, captured and replayed
    cache.v.copy_(pool_v)
    for o in outs:
        o.zero_()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            run()
    torch.cuda.current_stream().wait_stream(side)
    cache.k.copy_(pool_k)
    cache.v.copy_(pool_v)
    g.replay()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for i in range(steps):
        assert torch.equal(outs[i], eager[i]), f"step {i}"


# ---------------------------------------------------------------- benchmark-sized cases

def test_config3_shape_against_oracle(b2a):
    # 64 sequences, contexts uniform in [512, 8192] from seed 2, block table from seed 3, Hq 32 / Hkv 8 / D 128
    rng = np.random.default_rng(2)
    ctx = rng.integers(512, 8193, size=64)
    w = PagedWorkload(ctx, [1] * 64, 32, 8, 128, seed=2, table_seed=3)
    q = _round(w.query, torch.float16)
    out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=32, max_context_len=8192, max_q_len=1)
    assert_close(out, w.reference(q.float().numpy()), torch.float16)


def _config5_problem(b2a, value_fn):
    """Batch 16 x context 32768, Hq 64 / Hkv 8, pools filled through the library's own store path in slices
    (exercises kv_store at scale); keys N(0,1), values from ``value_fn(first position, positions per sequence)``."""
    hq, hkv, d, bs, n, ctxlen = 64, 8, 128, 16, 16, 32768
    nblk = ctxlen // bs
    gen = torch.Generator(device="cuda").manual_seed(5)
    cache = b2a.PagedKvCache.allocate(n * nblk + 1, hkv, d, bs, torch.uint8, poison=0xFF)
    perm = torch.randperm(n * nblk + 1, generator=torch.Generator().manual_seed(6))[: n * nblk].to(torch.int32)
    bi = perm.cuda()
    bb = (torch.arange(n + 1, dtype=torch.int32) * nblk).cuda()
    sb = torch.arange(n + 1, dtype=torch.int32).cuda()
    step = 4096
    for p0 in range(0, ctxlen, step):
        key = torch.randn(n * step, hkv * d, generator=gen, device="cuda", dtype=torch.float16)
        val = value_fn(gen, n, step, hkv, d)
        past = torch.full((n,), p0, dtype=torch.int32, device="cuda")
        sbs = (torch.arange(n + 1, dtype=torch.int32) * step).cuda()
        b2a.paged_kv_store(key, val, cache, past, sbs, bi, bb)
    past = torch.full((n,), ctxlen - 1, dtype=torch.int32, device="cuda")
    q = torch.randn(n, hq * d, generator=gen, device="cuda", dtype=torch.float16)
    return cache, q, past, sb, bi, bb


def test_config5_shape_against_oracle(b2a):
    # The long-context batch at full size with random keys AND values.  Two complete sequences (32768 tokens x 64
    # heads each) are checked against the oracle: their blocks are copied out of the pool into a compact one-sequence
    # pool with an identity block table, which the oracle then walks exactly as it would the large one.
    hq, hkv, d, bs, n, ctxlen = 64, 8, 128, 16, 16, 32768
    nblk = ctxlen // bs
    rand_v = lambda gen, n_, step, hkv_, d_: torch.randn(n_ * step, hkv_ * d_, generator=gen, device="cuda",
                                                          dtype=torch.float16)
    cache, q, past, sb, bi, bb = _config5_problem(b2a, rand_v)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = b2a.paged_attention(q, cache, past, sb, bi, bb, hq=hq, max_context_len=ctxlen, max_q_len=1, status=status)
    assert int(status.item()) == 0
    one = lambda a: np.asarray(a, dtype=np.int32)
    for s in (0, 11):
        phys = bi[s * nblk:(s + 1) * nblk].long()
        k_small, v_small = cache.k[phys].cpu().numpy(), cache.v[phys].cpu().numpy()
        ref = opaged.paged_attention_ref(q[s:s + 1].float().cpu().numpy(), k_small, v_small, one([ctxlen - 1]),
                                         one([0, 1]), np.arange(nblk, dtype=np.int32), one([0, nblk]), hq, hkv, d, bs)
        assert_close(out[s:s + 1], ref, torch.float16, f"sequence {s}")
    # a sliding window equal to the context changes nothing
    out_w = b2a.paged_attention(q, cache, past, sb, bi, bb, hq=hq, max_context_len=ctxlen, max_q_len=1,
                                sliding_window=ctxlen)
    assert torch.equal(out, out_w)


def test_config5_shape_constant_values(b2a):
    # the same shape with V constant per (sequence, head): every output row must reproduce its constant, whatever
    # the scores are - a check of all 16 x 64 rows that needs no oracle
    hq, hkv, d, n, ctxlen = 64, 8, 128, 16, 32768

    def const_v(gen, n_, step, hkv_, d_):
        hv = torch.arange(hkv_, device="cuda", dtype=torch.float16).repeat_interleave(d_)[None] * 0.125
        sv = torch.arange(n_, device="cuda", dtype=torch.float16).repeat_interleave(step)[:, None] * 0.0625
        return (hv + sv - 0.5).contiguous()
    cache, q, past, sb, bi, bb = _config5_problem(b2a, const_v)
    out = b2a.paged_attention(q, cache, past, sb, bi, bb, hq=hq, max_context_len=ctxlen, max_q_len=1)
    o = out.float().reshape(n, hkv, hq // hkv, d)
    expect = (torch.arange(hkv, device="cuda").float()[None, :, None, None] * 0.125
              + torch.arange(n, device="cuda").float()[:, None, None, None] * 0.0625 - 0.5)
    assert torch.allclose(o, expect.expand_as(o), atol=2e-3)


# ---------------------------------------------------------------- multi-token rows on the tensor-core kernel

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_prefill_parity(b2a, dtype):
    # (past, new tokens): fresh prefills, chunked-prefill continuations, ragged tails, decode rows in between
    past = np.array([0, 100, 1000, 37, 0, 5, 255], np.int32)
    qlen = np.array([300, 129, 2, 1, 1024, 128, 1], np.int32)
    hq, hkv, d = 32, 8, 128
    w = PagedWorkload(past + qlen, qlen, hq, hkv, d, seed=31)
    q = _round(w.query, dtype)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=hq,
                              max_context_len=int((past + qlen).max()), max_q_len=int(qlen.max()), status=status)
    assert int(status.item()) == 0
    assert_close(out, w.reference(q.float().numpy()), dtype)
    # with the scheduler's hints the prefill contexts are de-quantised once into a scratch and staged by TMA
    ctx = past + qlen
    hint_rb = int(sum((int(x) + 127) // 128 for x in qlen if x >= 2))
    hint_kv = int(sum((int(c) + 127) // 128 * 128 for c, x in zip(ctx, qlen) if x >= 2))
    out2 = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=hq, max_context_len=int(ctx.max()),
                               max_q_len=int(qlen.max()), status=status, prefill_row_blocks=hint_rb,
                               prefill_kv_tokens=hint_kv)
    assert int(status.item()) == 0
    assert_close(out2, w.reference(q.float().numpy()), dtype)
    assert torch.equal(out2, out)  # same de-quantised values, same kernel body
    # a hint that is too small is reported, not followed
    b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), hq=hq, max_context_len=int(ctx.max()),
                        max_q_len=int(qlen.max()), status=status, prefill_row_blocks=hint_rb,
                        prefill_kv_tokens=hint_kv - 128)
    assert int(status.item()) & 4  # B2A_DEV_BAD_LEN


def test_mixed_step_graph_replay_with_new_lengths(b2a):
    # a captured mixed step replays correctly after the device tables changed: other histories, and the step's 500
    # tokens split differently over the sequences (work list and scratch layout are rebuilt on the device)
    hq, hkv, d = 32, 8, 128
    w = PagedWorkload([600, 300, 400, 90], [300, 129, 1, 70], hq, hkv, d, seed=41)
    cache = w.device_cache()
    past, sb, bi, bb = w.device_tables()
    q = _round(w.query, torch.bfloat16).cuda()
    out = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    hints = dict(prefill_row_blocks=6, prefill_kv_tokens=1280)
    ws = torch.empty(b2a.ops.paged_workspace_bytes(torch.bfloat16, cache, hq, 4, 500, 640, 300, 6, 1280),
                     dtype=torch.uint8, device="cuda")
    run = lambda stream=None: b2a.paged_attention(q, cache, past, sb, bi, bb, hq=hq, max_context_len=640, max_q_len=300,
                                                  out=out, workspace=ws, stream=stream, status=status, **hints)
    run()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_close(out, w.reference(q.float().cpu().numpy()), torch.bfloat16)
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            run(s)
    new_past = np.array([400, 0, 100, 20], np.int32)
    new_qlen = np.array([129, 300, 70, 1], np.int32)
    new_sb = np.zeros(5, np.int32)
    new_sb[1:] = np.cumsum(new_qlen)
    past.copy_(torch.from_numpy(new_past))
    sb.copy_(torch.from_numpy(new_sb))
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = opaged.paged_attention_ref(q.float().cpu().numpy(), w.k_cache, w.v_cache, new_past, new_sb, w.bi, w.bb,
                                     hq, hkv, d, 16)
    assert_close(out, ref, torch.bfloat16)


@pytest.mark.parametrize("window", [16, 100, 128, 300, 5000])
@pytest.mark.parametrize("hq", [32, 24])
def test_paged_prefill_sliding_window(b2a, window, hq):
    # multi-token sequences with a sliding window run on the tensor-core kernel too (both prefill variants): a query at
    # position p sees keys p - window + 1 .. p.  hq = 24 gives groups of three query heads, where the two tiles of a
    # work item are different row blocks with different first key tiles.
    past = np.array([0, 100, 700, 37, 0, 255], np.int32)
    qlen = np.array([300, 129, 2, 1, 640, 1], np.int32)
    hkv, d = 8, 128
    w = PagedWorkload(past + qlen, qlen, hq, hkv, d, seed=51)
    q = _round(w.query, torch.bfloat16)
    ref = w.reference(q.float().numpy(), sliding_window=window)
    ctx = past + qlen
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kw = dict(hq=hq, max_context_len=int(ctx.max()), max_q_len=int(qlen.max()), status=status, sliding_window=window)
    out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), **kw)
    hint_rb = int(sum((int(x) + 127) // 128 for x in qlen if x >= 2))
    hint_kv = int(sum((int(c) + 127) // 128 * 128 for c, x in zip(ctx, qlen) if x >= 2))
    out2 = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), prefill_row_blocks=hint_rb,
                               prefill_kv_tokens=hint_kv, **kw)
    assert int(status.item()) == 0
    assert_close(out, ref, torch.bfloat16, "contexts de-quantised in the kernel")
    assert_close(out2, ref, torch.bfloat16, "contexts de-quantised once")
    assert torch.equal(out, out2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_rows_far_from_zero(b2a, dtype):
    # Rows that sit far from zero have zero-points of thousands (mean 8, deviation 0.1: zp around -2500; the
    # mirrored rows: +2700), where a de-quantiser that subtracts in f16 would be off by whole code steps.  A mixed
    # step (two prefills, a continuation, decode rows) through both prefill variants and the decode kernel.
    past = np.array([0, 300, 1000, 5, 0], np.int32)
    qlen = np.array([260, 130, 1, 1, 128], np.int32)
    hq, hkv, d = 32, 8, 128
    rows = lambda sign: (lambda s, c: (sign * 8.0 + 0.1 * np.random.default_rng(1000 + s).standard_normal(
        (c, hkv, d))).astype(np.float32))
    w = PagedWorkload(past + qlen, qlen, hq, hkv, d, seed=33, key_fn=rows(1.0), value_fn=rows(-1.0), q_scale=0.25)
    zp = oquant.chunk_views(w.k_cache, 16, d)[2]
    assert np.abs(zp[w.bi[0]].astype(np.float32)).max() > 2048  # the case is what it claims to be
    q = _round(w.query, dtype)
    ref = w.reference(q.float().numpy())
    ctx = past + qlen
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kw = dict(hq=hq, max_context_len=int(ctx.max()), max_q_len=int(qlen.max()), status=status)
    out = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), **kw)
    hint_rb = int(sum((int(x) + 127) // 128 for x in qlen if x >= 2))
    hint_kv = int(sum((int(c) + 127) // 128 * 128 for c, x in zip(ctx, qlen) if x >= 2))
    out2 = b2a.paged_attention(q.cuda(), w.device_cache(), *w.device_tables(), prefill_row_blocks=hint_rb,
                               prefill_kv_tokens=hint_kv, **kw)
    assert int(status.item()) == 0
    assert_close(out, ref, dtype, "prefill contexts de-quantised in the kernel")
    assert_close(out2, ref, dtype, "prefill contexts de-quantised once")
    assert torch.equal(out, out2)


def test_config4_mixed_step(b2a):
    # 8 prefill sequences of 1024 tokens plus 120 decode sequences with contexts uniform in [256, 4096] (seed 4),
    # bf16 queries, u8 cache, through the operator (store, then attend)
    rng = np.random.default_rng(4)
    dec_ctx = rng.integers(256, 4097, size=120)
    past = np.concatenate([np.zeros(8, np.int64), dec_ctx - 1]).astype(np.int32)
    qlen = np.concatenate([np.full(8, 1024), np.ones(120, np.int64)]).astype(np.int32)
    hq, hkv, d, bs = 32, 8, 128, 16
    w = PagedWorkload(past + qlen, qlen, hq, hkv, d, seed=4, table_seed=4)
    new_k = _round(rng.standard_normal((int(w.sb[-1]), hkv * d), dtype=np.float32), torch.bfloat16)
    new_v = _round(rng.standard_normal((int(w.sb[-1]), hkv * d), dtype=np.float32), torch.bfloat16)
    ref_k, ref_v = w.k_cache.copy(), w.v_cache.copy()
    opaged.kv_store_ref(new_k, ref_k, w.past, w.sb, w.bi, w.bb, hkv, d, bs)
    opaged.kv_store_ref(new_v, ref_v, w.past, w.sb, w.bi, w.bb, hkv, d, bs)
    q = _round(w.query, torch.bfloat16)
    ref = opaged.paged_attention_ref(q.float().numpy(), ref_k, ref_v, w.past, w.sb, w.bi, w.bb, hq, hkv, d, bs)
    # no scratch reserve: the prefill contexts are de-quantised inside the prefill kernel
    op = b2a.PagedAttentionOp(hq, hkv, d, bs, torch.uint8, max_seqs=128, max_context_len=4096, q_dtype=torch.bfloat16,
                              max_step_tokens=8 * 1024 + 120)
    wb = {"mutable": [torch.empty(n, dtype=torch.uint8, device="cuda") for n in op.GetWorkBufferRequest()["mutable_sizes"]]}
    cache = w.device_cache()
    out = torch.empty(int(w.sb[-1]), hq * d, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    op.Execute([q.cuda(), new_k.cuda(), new_v.cuda(), cache.k, cache.v, *w.device_tables(), None, 0, None, 4096],
               [out], workbuffers=wb, status=status)
    assert int(status.item()) == 0
    assert np.array_equal(cache.k.cpu().numpy(), ref_k) and np.array_equal(cache.v.cpu().numpy(), ref_v)
    assert_close(out, ref, torch.bfloat16)
    # An operator with a scratch reserve de-quantises the contexts once: with the scheduler's hints for this step,
    # and with none (the reserve is then laid out on the device).  Storing the same rows again leaves the pools as
    # they are, and the output is the same to the bit.  A work buffer that is too small is refused, not replaced.
    op2 = b2a.PagedAttentionOp(hq, hkv, d, bs, torch.uint8, max_seqs=128, max_context_len=4096,
                               max_prefill_kv_tokens=12 * 1024, q_dtype=torch.bfloat16, max_step_tokens=8 * 1024 + 120)
    with pytest.raises(b2a.B2AError):
        op2.Execute([q.cuda(), new_k.cuda(), new_v.cuda(), cache.k, cache.v, *w.device_tables(), None, 0, None, 4096],
                    [out], workbuffers=wb, status=status)
    wb2 = {"mutable": [torch.empty(n, dtype=torch.uint8, device="cuda") for n in op2.GetWorkBufferRequest()["mutable_sizes"]]}
    for hints in (dict(prefill_row_blocks=8 * 8, prefill_kv_tokens=8 * 1024), dict()):
        out2 = torch.empty_like(out)
        op2.Execute([q.cuda(), new_k.cuda(), new_v.cuda(), cache.k, cache.v, *w.device_tables(), None, 0, None, 4096],
                    [out2], workbuffers=wb2, status=status, **hints)
        assert int(status.item()) == 0
        assert np.array_equal(cache.k.cpu().numpy(), ref_k) and torch.equal(out2, out)
