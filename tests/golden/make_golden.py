"""Generate the golden vectors of ``tests/golden/sdpa_reference.npz``.

Runs the REFERENCE's own dense attention
(``modules/genai_optimizations/genai_opt/sparse_attention.py:95-121``,
``SparseAttention('dense')._dense_attention``) on seeded inputs and stores inputs and
outputs.  The reference is only present in the development container, so the vectors are
committed; run this script again only there:

    python tests/golden/make_golden.py /path/to/reference

Cases: the shapes of the reference's functional test
(``modules/nvidia_plugin/tests/functional/shared_tests_instances/single_layer_tests/scaled_dot_product_attention.cpp:76-104``:
[1,1,4,8], [1,4,16,32], [1,8,32,64], and the 3-D [4,2,8]) x {causal, non-causal}, plus
grouped-query, boolean-mask, additive-mask, explicit-scale and Sq != Skv cases, plus paged cases:
a de-quantised u8 block pool gathered into contiguous K/V and run through the same function.
"""
import sys
import types

import numpy as np
import torch


def load_reference(root):
    sys.path.insert(0, f"{root}/modules/genai_optimizations")
    from genai_opt.sparse_attention import SparseAttention  # noqa: E402
    return SparseAttention(algorithm="dense")


def ref_dense(att, q, k, v, mask=None, scale=None, causal=False):
    """q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] float32 torch -> [B,Hq,Sq,D] numpy."""
    hq, hkv = q.shape[1], k.shape[1]
    module = types.SimpleNamespace(num_key_value_groups=hq // hkv, head_dim=q.shape[-1])
    m = mask
    if causal:
        sq, skv = q.shape[2], k.shape[2]
        m = torch.ones(sq, skv, dtype=torch.bool).tril(0)[None, None]
    out, _ = att._dense_attention(module, q, k, v, m, scaling=scale)
    return out.transpose(1, 2).contiguous().numpy()  # the reference returns [B,Sq,H,D]


def main(root):
    att = load_reference(root)
    out = {}
    cases = []
    for shp in [(1, 1, 4, 8), (1, 4, 16, 32), (1, 8, 32, 64)]:
        for causal in (False, True):
            cases.append(dict(name=f"t4d_{'x'.join(map(str, shp))}_c{int(causal)}", q=shp, kv=shp, causal=causal))
    for causal in (False, True):
        cases.append(dict(name=f"t3d_4x2x8_c{int(causal)}", q=(4, 1, 2, 8), kv=(4, 1, 2, 8), causal=causal, three_d=True))
    cases += [
        dict(name="gqa_causal", q=(2, 8, 48, 64), kv=(2, 2, 48, 64), causal=True),
        dict(name="gqa_d128", q=(1, 8, 40, 128), kv=(1, 2, 40, 128), causal=True),
        dict(name="cross_len", q=(1, 4, 7, 32), kv=(1, 4, 29, 32), causal=False),
        dict(name="bool_mask", q=(1, 4, 17, 32), kv=(1, 4, 33, 32), causal=False, mask="bool"),
        dict(name="add_mask", q=(2, 4, 17, 32), kv=(2, 4, 33, 32), causal=False, mask="float"),
        dict(name="scale", q=(1, 2, 16, 64), kv=(1, 2, 16, 64), causal=True, scale=0.3),
    ]
    g = torch.Generator().manual_seed(1234)
    for c in cases:
        q = torch.randn(c["q"], generator=g)
        k = torch.randn(c["kv"], generator=g)
        v = torch.randn(c["kv"], generator=g)
        mask = None
        if c.get("mask") == "bool":
            mask = torch.rand(1, 1, c["q"][2], c["kv"][2], generator=g) > 0.3
            mask[..., 0] = True  # no fully masked row
        elif c.get("mask") == "float":
            mask = torch.randn(c["q"][0], 1, c["q"][2], c["kv"][2], generator=g)
        o = ref_dense(att, q, k, v, mask, c.get("scale"), c["causal"])
        n = c["name"]
        out[f"{n}/q"], out[f"{n}/k"], out[f"{n}/v"], out[f"{n}/o"] = q.numpy(), k.numpy(), v.numpy(), o
        out[f"{n}/causal"] = np.array(c["causal"])
        out[f"{n}/scale"] = np.array(c.get("scale") or 0.0, dtype=np.float32)
        out[f"{n}/three_d"] = np.array(bool(c.get("three_d")))
        if mask is not None:
            out[f"{n}/mask"] = mask.numpy()
    np.savez_compressed("tests/golden/sdpa_reference.npz", **out)

    # Paged cases: pool built with the oracle's quantiser, de-quantised contiguous K/V fed
    # to the reference's dense attention with a causal mask offset by past_len.
    sys.path.insert(0, ".")
    from oracle import paged
    pout = {}
    rng = np.random.default_rng(4321)
    hq, hkv, d, bs = 8, 2, 128, 16
    past = np.array([0, 31, 16, 77], dtype=np.int32)
    qlen = np.array([5, 1, 1, 3], dtype=np.int32)
    ctx = past + qlen
    bi, bb, nb = paged.build_block_tables(ctx, bs, seed=7, spare_blocks=2)
    rows_k = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    rows_v = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    kc = paged.fill_cache_from_rows(rows_k, ctx, bi, bb, nb, hkv, d, bs)
    vc = paged.fill_cache_from_rows(rows_v, ctx, bi, bb, nb, hkv, d, bs)
    sb = np.zeros(len(ctx) + 1, dtype=np.int32)
    sb[1:] = np.cumsum(qlen)
    query = rng.standard_normal((int(sb[-1]), hq * d)).astype(np.float32)
    outs = np.zeros_like(query)
    for s in range(len(ctx)):
        kk = torch.from_numpy(paged.gather_sequence(kc, s, int(ctx[s]), bi, bb, d, bs))[None]
        vv = torch.from_numpy(paged.gather_sequence(vc, s, int(ctx[s]), bi, bb, d, bs))[None]
        qs = torch.from_numpy(query[sb[s]:sb[s + 1]].reshape(-1, hq, d)).transpose(0, 1)[None].contiguous()
        pos_q = int(past[s]) + torch.arange(int(qlen[s]))[:, None]
        m = (torch.arange(int(ctx[s]))[None, :] <= pos_q)[None, None]
        module = types.SimpleNamespace(num_key_value_groups=hq // hkv, head_dim=d)
        o, _ = att._dense_attention(module, qs, kk, vv, m)  # [1, qlen, Hq, D]
        outs[sb[s]:sb[s + 1]] = o[0].reshape(int(qlen[s]), hq * d).numpy()
    pout.update(query=query, k_cache=kc, v_cache=vc, past_lens=past, subsequence_begins=sb,
                block_indices=bi, block_indices_begins=bb, out=outs,
                geom=np.array([hq, hkv, d, bs], dtype=np.int32))
    np.savez_compressed("tests/golden/paged_reference.npz", **pout)
    print("wrote", len(cases), "sdpa cases and 1 paged case")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to an openvino_contrib checkout>")
    main(sys.argv[1])
