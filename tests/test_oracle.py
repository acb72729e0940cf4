"""The CPU oracle against the reference's golden vectors (no GPU)."""
import os

import numpy as np
import pytest

from oracle import paged, quant, sdpa


def _cases(npz):
    return sorted({k.split("/")[0] for k in npz.files})


@pytest.fixture(scope="module")
def sdpa_golden(golden_dir):
    return np.load(os.path.join(golden_dir, "sdpa_reference.npz"))


def test_sdpa_oracle_matches_reference_vectors(sdpa_golden):
    g = sdpa_golden
    names = _cases(g)
    assert len(names) == 14
    for n in names:
        mask = g[f"{n}/mask"] if f"{n}/mask" in g.files else None
        scale = float(g[f"{n}/scale"]) or None
        o = sdpa.sdpa_ref(g[f"{n}/q"], g[f"{n}/k"], g[f"{n}/v"], mask=mask, scale=scale,
                          causal=bool(g[f"{n}/causal"]))
        np.testing.assert_allclose(o, g[f"{n}/o"], rtol=1e-5, atol=2e-6, err_msg=n)


def test_sdpa_oracle_3d_layout(sdpa_golden):
    g = sdpa_golden
    n = "t3d_4x2x8_c1"
    q, k, v = (g[f"{n}/{x}"][:, 0] for x in "qkv")  # [4, 2, 8]: batch 4, L=2, E=8
    o = sdpa.sdpa_ref(q, k, v, causal=True)
    np.testing.assert_allclose(o, g[f"{n}/o"][:, 0], rtol=1e-5, atol=2e-6)


def test_paged_oracle_matches_reference_vectors(golden_dir):
    g = np.load(os.path.join(golden_dir, "paged_reference.npz"))
    hq, hkv, d, bs = (int(x) for x in g["geom"])
    o = paged.paged_attention_ref(g["query"], g["k_cache"], g["v_cache"], g["past_lens"],
                                  g["subsequence_begins"], g["block_indices"],
                                  g["block_indices_begins"], hq, hkv, d, bs)
    np.testing.assert_allclose(o, g["out"], rtol=1e-5, atol=3e-6)


def test_quantiser_properties():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, 8, 128)).astype(np.float32)
    q, s, z = quant.quantize_rows(x)
    assert q.dtype == np.uint8 and s.dtype == np.float16 and z.dtype == np.float16
    xh = quant.dequantize_rows(q, s, z)
    step = s.astype(np.float32)[..., None]
    # error bounded by one quantisation step (half a step plus the f16 rounding of zp)
    assert np.all(np.abs(xh - x) <= step * 1.01)
    # re-quantising the de-quantised row reproduces the same bytes where the range is kept
    q2, s2, z2 = quant.quantize_rows(np.stack([xh[0, 0], xh[0, 0]]))
    assert np.array_equal(q2[0], q2[1])
    # constant row: scale guard
    qc, sc, zc = quant.quantize_rows(np.full((1, 128), 0.75, np.float32))
    assert float(sc[0]) == 1.0
    np.testing.assert_allclose(quant.dequantize_rows(qc, sc, zc), 0.75, atol=1e-3)
    # all-zero row
    q0, s0, z0 = quant.quantize_rows(np.zeros((1, 16), np.float32))
    assert np.all(quant.dequantize_rows(q0, s0, z0) == 0)


def test_store_then_gather_roundtrip():
    rng = np.random.default_rng(1)
    hkv, d, bs = 2, 64, 16
    ctx = [1, 15, 16, 17, 33]
    bi, bb, nb = paged.build_block_tables(ctx, bs, seed=5, spare_blocks=2)
    rows = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    filled = paged.fill_cache_from_rows(rows, ctx, bi, bb, nb, hkv, d, bs)
    # the same pool built by two store steps (a prefill of all but the last token, then a decode step)
    cache = np.full_like(filled, 0xFF)
    first = [c - 1 for c in ctx]
    sb = np.zeros(len(ctx) + 1, np.int32)
    sb[1:] = np.cumsum(first)
    new = np.concatenate([r[:-1].reshape(len(r) - 1, hkv * d) for r in rows])
    paged.kv_store_ref(new, cache, np.zeros(len(ctx), np.int32), sb, bi, bb, hkv, d, bs)
    last = np.stack([r[-1].reshape(-1) for r in rows])
    w = paged.kv_store_ref(last, cache, np.array(first, np.int32), np.arange(len(ctx) + 1, dtype=np.int32),
                           bi, bb, hkv, d, bs)
    assert np.array_equal(cache, filled)
    # physical indices: last token of sequence s sits in its last logical block
    for s, (pb, slot) in enumerate(w):
        assert pb == bi[bb[s] + (ctx[s] - 1) // bs] and slot == (ctx[s] - 1) % bs
    # spare blocks keep their poison
    used = set(int(b) for b in bi)
    for b in range(nb):
        if b not in used:
            assert np.all(cache[b] == 0xFF)
    # gather is the de-quantised rows
    for s, c in enumerate(ctx):
        x = paged.gather_sequence(cache, s, c, bi, bb, d, bs)
        q, s16, z16 = quant.quantize_rows(rows[s])
        np.testing.assert_array_equal(x, np.transpose(quant.dequantize_rows(q, s16, z16), (1, 0, 2)))


def test_sliding_window_and_empty_sequence():
    rng = np.random.default_rng(2)
    hq, hkv, d, bs = 4, 2, 32, 16
    ctx = [40, 0, 9]
    bi, bb, nb = paged.build_block_tables(ctx, bs, seed=9)
    rows_k = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    rows_v = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    kc = paged.fill_cache_from_rows(rows_k, ctx, bi, bb, nb, hkv, d, bs)
    vc = paged.fill_cache_from_rows(rows_v, ctx, bi, bb, nb, hkv, d, bs)
    past = np.array([39, 0, 8], np.int32)
    sb = np.array([0, 1, 1, 2], np.int32)  # the middle sequence has no token this step
    q = rng.standard_normal((2, hq * d)).astype(np.float32)
    full = paged.paged_attention_ref(q, kc, vc, past, sb, bi, bb, hq, hkv, d, bs)
    win = paged.paged_attention_ref(q, kc, vc, past, sb, bi, bb, hq, hkv, d, bs, sliding_window=8)
    assert not np.allclose(full[0], win[0])
    # window 8 on the 40-token sequence == attention over its last 8 tokens only
    kk = paged.gather_sequence(kc, 0, 40, bi, bb, d, bs)[:, -8:]
    vv = paged.gather_sequence(vc, 0, 40, bi, bb, d, bs)[:, -8:]
    ref = sdpa.sdpa_ref(q[0].reshape(1, hq, 1, d), kk[None], vv[None]).reshape(-1)
    np.testing.assert_allclose(win[0], ref, rtol=1e-5, atol=1e-6)


def test_division_by_scale_identity(tmp_path):
    """The store kernel's reciprocal-plus-fused-correction form of x / scale equals the IEEE division for every
    f16-valued scale visited and every f16 / bf16 x (every 16th scale here; the exhaustive run is stride 1)."""
    import os
    import shutil
    import subprocess
    src = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "div_by_scale_check.c")
    if shutil.which("gcc") is None or "fma" not in open("/proc/cpuinfo").read():
        pytest.skip("needs gcc and a host CPU with FMA")
    exe = str(tmp_path / "div_by_scale_check")
    subprocess.run(["gcc", "-O2", "-mfma", "-o", exe, src, "-lm"], check=True)
    r = subprocess.run([exe, "16"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and " 0 mismatches" in r.stdout, r.stdout


def test_rope_oracle_properties():
    """The rotary-embedding restatement: position 0 is the identity, values beyond rotary_dim pass through, every
    (i, i + r/2) pair keeps its norm, and a rotation by p then by q - the tables being angles p*f and q*f - equals the
    rotation by p + q up to float32 rounding."""
    from oracle import rope
    r, d = 32, 48
    cos, sin = rope.rope_tables(128, r)
    assert cos.dtype == np.float32 and cos.shape == (128, r // 2)
    x = np.random.default_rng(0).standard_normal((6, 3, d)).astype(np.float32)
    pos = np.array([0, 1, 5, 17, 64, 127])
    y = rope.rope_rows(x, pos, cos, sin, r)
    assert np.array_equal(y[0], x[0]) and np.array_equal(y[..., r:], x[..., r:])
    n0 = x[..., : r // 2] ** 2 + x[..., r // 2: r] ** 2
    n1 = y[..., : r // 2] ** 2 + y[..., r // 2: r] ** 2
    np.testing.assert_allclose(n1, n0, rtol=1e-5, atol=1e-6)
    twice = rope.rope_rows(rope.rope_rows(x, [3] * 6, cos, sin, r), [9] * 6, cos, sin, r)
    np.testing.assert_allclose(twice, rope.rope_rows(x, [12] * 6, cos, sin, r), rtol=1e-4, atol=1e-5)
    assert rope.token_positions([4, 0], [0, 2, 5]).tolist() == [4, 5, 0, 1, 2]


def test_score_oracle_is_the_softmax_of_the_attention_oracle():
    """last_token_scores_ref restates the probabilities inside paged_attention_ref: with V = one-hot of the key
    position (one sequence, D >= context), the attention output of the last row IS its probability vector."""
    from oracle import paged as opaged
    hq, hkv, d, bs = 4, 2, 32, 16
    ctx = np.array([20], np.int64)
    rng = np.random.default_rng(0)
    bi, bb, nb = opaged.build_block_tables(ctx, bs, 1)
    rows_k = [rng.standard_normal((20, hkv, d), dtype=np.float32)]
    onehot = np.zeros((20, hkv, d), np.float32)
    for t in range(20):
        onehot[t, :, t] = 1.0
    k_cache = opaged.fill_cache_from_rows(rows_k, ctx, bi, bb, nb, hkv, d, bs)
    v_cache = opaged.fill_cache_from_rows([onehot], ctx, bi, bb, nb, hkv, d, bs)
    q = rng.standard_normal((1, hq * d), dtype=np.float32)
    past, sb = np.array([19], np.int32), np.array([0, 1], np.int32)
    out = opaged.paged_attention_ref(q, k_cache, v_cache, past, sb, bi, bb, hq, hkv, d, bs).reshape(hq, d)
    scores, begins = opaged.last_token_scores_ref(q, k_cache, past, sb, bi, bb, hq, hkv, d, bs)
    assert begins.tolist() == [0, 20]
    # (one-hot values go through the u8 quantiser: exact 0 and 1 up to its rounding of the scale)
    np.testing.assert_allclose(scores, out[:, :20].sum(axis=0), atol=5e-3)
    assert abs(scores.sum() - hq) < 1e-4
