"""ScaledDotProductAttention on the GPU, through the C ABI, against the oracle and the reference's vectors."""
import os

import numpy as np
import pytest
import torch

from oracle import sdpa as osdpa
from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def b2a():
    import openvino_contrib_b200 as m
    assert torch.cuda.is_available()
    return m


def _rand(shape, seed, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def test_reference_golden_vectors(b2a, golden_dir):
    g = np.load(os.path.join(golden_dir, "sdpa_reference.npz"))
    for n in sorted({k.split("/")[0] for k in g.files}):
        q, k, v = (torch.from_numpy(g[f"{n}/{x}"]).cuda() for x in "qkv")
        mask = torch.from_numpy(g[f"{n}/mask"]).cuda() if f"{n}/mask" in g.files else None
        scale = float(g[f"{n}/scale"]) or None
        o = b2a.sdpa(q, k, v, mask, scale, bool(g[f"{n}/causal"]))
        assert_close(o, g[f"{n}/o"], torch.float32, n)


# the shapes of the reference's functional test (scaled_dot_product_attention.cpp:76-104)
REF_SHAPES = [(1, 1, 4, 8), (1, 4, 16, 32), (1, 8, 32, 64), (4, 2, 8)]


@pytest.mark.parametrize("shape", REF_SHAPES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_reference_test_grid(b2a, shape, causal, dtype):
    q, k, v = (_rand(shape, 10 + i, dtype) for i in range(3))
    o = b2a.SdpaOp(causal=causal)
    out = torch.empty(shape, dtype=dtype, device="cuda")
    o.Execute([q.cuda(), k.cuda(), v.cuda()], [out])
    assert_close(out, osdpa.sdpa_ref(q, k, v, causal=causal), dtype)


def test_config1_f32_causal(b2a):
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 8, 256, 64, generator=g) for _ in range(3))
    o = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), scale=0.125, causal=True)
    assert_close(o, osdpa.sdpa_ref(q, k, v, scale=0.125, causal=True), torch.float32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [
    # (B, Hq, Hkv, Sq, Skv, D)
    (1, 8, 2, 512, 512, 128),     # Llama-shaped GQA, several key tiles
    (2, 4, 4, 128, 128, 128),     # one tile, no GQA
    (1, 8, 2, 384, 384, 128),     # ragged against 256-row query tiles
    (1, 4, 1, 200, 333, 128),     # nothing a multiple of the tile sizes, Sq != Skv
    (1, 2, 2, 1, 129, 128),       # a single query row
    (1, 4, 2, 77, 77, 64),        # head size 64
])
def test_half_precision_shapes(b2a, dtype, causal, shape):
    B, Hq, Hkv, Sq, Skv, D = shape
    q = _rand((B, Hq, Sq, D), 1, dtype, 0.5)
    k = _rand((B, Hkv, Skv, D), 2, dtype, 0.5)
    v = _rand((B, Hkv, Skv, D), 3, dtype, 0.5)
    o = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    assert_close(o, osdpa.sdpa_ref(q, k, v, causal=causal), dtype, str(shape))


def test_strided_views_and_out_argument(b2a):
    # [B, S, H, D] storage viewed as [B, H, S, D]: the layout LLM runtimes hand over
    B, S, Hq, Hkv, D = 2, 160, 8, 2, 128
    dtype = torch.bfloat16
    qs = _rand((B, S, Hq, D), 4, dtype, 0.5).cuda()
    ks = _rand((B, S, Hkv, D), 5, dtype, 0.5).cuda()
    vs = _rand((B, S, Hkv, D), 6, dtype, 0.5).cuda()
    q, k, v = qs.transpose(1, 2), ks.transpose(1, 2), vs.transpose(1, 2)
    out_store = torch.zeros(B, S, Hq, D, dtype=dtype, device="cuda")
    b2a.sdpa(q, k, v, causal=True, out=out_store.transpose(1, 2))
    ref = osdpa.sdpa_ref(q.cpu(), k.cpu(), v.cpu(), causal=True)
    assert_close(out_store.transpose(1, 2), ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_masks_broadcast_and_uneven_head_sizes(b2a, dtype):
    B, H, Sq, Skv, D, Dv = 2, 3, 19, 45, 80, 48
    q = _rand((B, H, Sq, D), 7, dtype)
    k = _rand((B, H, Skv, D), 8, dtype)
    v = _rand((B, H, Skv, Dv), 9, dtype)
    g = torch.Generator().manual_seed(11)
    bmask = torch.rand(B, 1, Sq, Skv, generator=g) > 0.4
    bmask[..., 0] = True
    o = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), bmask.cuda())
    assert_close(o, osdpa.sdpa_ref(q, k, v, mask=bmask.numpy()), dtype)
    amask = torch.randn(1, H, 1, Skv, generator=g).to(dtype)
    o = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), amask.cuda(), scale=0.2)
    assert_close(o, osdpa.sdpa_ref(q, k, v, mask=amask.float().numpy(), scale=0.2), dtype)
    # a fully masked row yields zeros, not NaN
    bmask[0, 0, 3, :] = False
    o = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), bmask.cuda())
    assert torch.isfinite(o.float()).all() and float(o[0, :, 3].abs().max()) == 0.0


def test_causal_ignores_mask_and_is_deterministic(b2a):
    q, k, v = (_rand((1, 4, 64, 64), 20 + i, torch.float16).cuda() for i in range(3))
    m = torch.zeros(64, 64, dtype=torch.bool, device="cuda")
    a = b2a.sdpa(q, k, v, m, causal=True)
    b = b2a.sdpa(q, k, v, None, causal=True)
    assert torch.equal(a, b)


def test_bad_arguments_raise(b2a):
    from openvino_contrib_b200._lib import B2AError
    q = torch.zeros(1, 6, 8, 64, device="cuda")
    k = torch.zeros(1, 4, 8, 64, device="cuda")
    with pytest.raises(B2AError) as e:
        b2a.sdpa(q, k, k)
    assert e.value.code == 2
    with pytest.raises(TypeError):
        b2a.sdpa(q.double(), q.double(), q.double())
    big = torch.zeros(1, 1, 4, 512, device="cuda")
    with pytest.raises(B2AError) as e:
        b2a.sdpa(big, big, big)
    assert e.value.code == 7


def test_graph_capture_and_replay(b2a):
    q, k, v = (_rand((1, 8, 96, 128), 30 + i, torch.bfloat16, 0.5).cuda() for i in range(3))
    out = torch.empty_like(q)
    b2a.sdpa(q, k, v, causal=True, out=out)  # warm-up outside capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            b2a.sdpa(q, k, v, causal=True, out=out, stream=s)
    q2 = _rand((1, 8, 96, 128), 99, torch.bfloat16, 0.5).cuda()
    q.copy_(q2)
    out.zero_()
    g.replay()
    torch.cuda.synchronize()
    assert_close(out, osdpa.sdpa_ref(q2.cpu(), k.cpu(), v.cpu(), causal=True), torch.bfloat16)


def test_config2_full_size_properties(b2a):
    # Llama-3-8B-shaped causal bf16 prefill at full size (B=4, Hq=32, Hkv=8, S=4096, D=128), checked through
    # properties that do not need the whole oracle: causality (the first rows only see the first keys, so they
    # equal the oracle on the truncated problem), a late row block against the oracle, V = 1 gives 1,
    # and run-to-run determinism of the persistent kernel.
    B, hq, hkv, S, D = 4, 32, 8, 4096, 128
    gen = torch.Generator().manual_seed(1)
    q = (torch.randn(B, hq, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    k = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    v = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out = b2a.sdpa(qd, kd, vd, causal=True)
    assert torch.equal(out, b2a.sdpa(qd, kd, vd, causal=True))
    for b, h in ((0, 0), (3, 31), (1, 14)):
        hk = h // (hq // hkv)
        ref = osdpa.sdpa_ref(q[b:b + 1, h:h + 1, :384].float().numpy(), k[b:b + 1, hk:hk + 1, :384].float().numpy(),
                             v[b:b + 1, hk:hk + 1, :384].float().numpy(), causal=True)
        assert_close(out[b:b + 1, h:h + 1, :384], ref, torch.bfloat16, f"first rows of ({b},{h})")
    # rows 3968..4095 of one head against the oracle with an explicit mask (they see all 4096 keys up to their own)
    b, h, r0 = 2, 9, 3968
    hk = h // (hq // hkv)
    keep = (np.arange(S)[None, :] <= (r0 + np.arange(128))[:, None])
    ref = osdpa.sdpa_ref(q[b:b + 1, h:h + 1, r0:].float().numpy(), k[b:b + 1, hk:hk + 1].float().numpy(),
                         v[b:b + 1, hk:hk + 1].float().numpy(), mask=keep[None, None])
    assert_close(out[b:b + 1, h:h + 1, r0:], ref, torch.bfloat16, "last row block")
    ones = b2a.sdpa(qd, kd, torch.ones_like(vd), causal=True)
    assert float((ones.float() - 1.0).abs().max()) <= 2.0 ** -8  # P is rounded to bf16 before the PV product


def test_config2_full_size_planes_against_oracle(b2a):
    # the same full-size problem: four complete (batch, head) planes - all 4096 rows over all their keys, one per
    # batch entry, over four different KV heads and positions in the group - against the oracle
    B, hq, hkv, S, D = 4, 32, 8, 4096, 128
    gen = torch.Generator().manual_seed(1)
    q = (torch.randn(B, hq, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    k = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    v = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), causal=True, status=status).cpu()
    assert int(status.item()) == 0
    for b, h in ((0, 0), (1, 13), (2, 22), (3, 31)):
        hk = h // (hq // hkv)
        ref = osdpa.sdpa_ref(q[b:b + 1, h:h + 1], k[b:b + 1, hk:hk + 1], v[b:b + 1, hk:hk + 1], causal=True)
        assert_close(out[b:b + 1, h:h + 1], ref, torch.bfloat16, f"plane ({b},{h})")


def test_host_pipeline_matches_device_call(b2a):
    # host tensors in, host tensor out, one piece per (batch entry, KV head) pipelined on three streams through the
    # C++ operator: same bits as the plain call
    B, hq, hkv, S, D = 3, 8, 2, 384, 128
    gen = torch.Generator().manual_seed(9)
    q = (torch.randn(B, hq, S, D, generator=gen) * 0.5).to(torch.bfloat16).pin_memory()
    k = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16).pin_memory()
    v = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(torch.bfloat16).pin_memory()
    out = torch.empty(B, hq, S, D, dtype=torch.bfloat16).pin_memory()
    pipe = b2a.HostSdpaPipeline(B, hq, hkv, S, S, D, torch.bfloat16, causal=True, kv_heads_per_piece=1)
    assert pipe.pieces == B * hkv
    for _ in range(3):  # the second call captures the step into a graph, the third replays it
        pipe(q, k, v, out)
        torch.cuda.synchronize()
        ref = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), causal=True)
        assert torch.equal(out.cuda(), ref)
    with pytest.raises(ValueError):
        pipe(q.cuda(), k, v, out)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kind", ["bool", "add"])
def test_masks_on_the_tensor_core_shape(b2a, dtype, kind):
    # D = 128 half-precision with an explicit mask (the tensor-core kernel reads the mask rows in 16-byte pieces):
    # per-batch, per-head and fully broadcast masks, a key count that ends inside a key tile, a query count that ends
    # inside a row tile, one fully masked row (zeros, not NaN) and, for additive masks, -inf entries.
    B, hq, hkv, sq, skv, D = 2, 8, 2, 200, 272, 128
    g = torch.Generator().manual_seed(21)
    q = (torch.randn(B, hq, sq, D, generator=g) * 0.5).to(dtype)
    k = (torch.randn(B, hkv, skv, D, generator=g) * 0.5).to(dtype)
    v = (torch.randn(B, hkv, skv, D, generator=g) * 0.5).to(dtype)
    for shape in ((B, 1, sq, skv), (1, hq, sq, skv), (sq, skv)):
        keep = torch.rand(shape, generator=g) > 0.3
        keep[..., 7, :] = False                       # a fully masked query row
        keep[..., 0, 0] = True
        if kind == "bool":
            mask = keep
        else:
            mask = (torch.randn(shape, generator=g) * 2.0).to(dtype)
            mask = torch.where(keep, mask, torch.tensor(float("-inf"), dtype=dtype))
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), attn_mask=mask.cuda(), status=status)
        ref = osdpa.sdpa_ref(q, k, v, mask=mask if kind == "bool" else mask.float())
        assert int(status.item()) == 0
        assert not torch.isnan(out).any()
        assert_close(out, ref, dtype, f"{kind} mask of shape {shape}")
