"""b2a_paged_kv_store_rope: the key rows are rotated on their way into the cache.  The pool bytes (u8 codes, f16 scale
and zero-point, untouched poison) must equal, bit for bit, the oracle's store of the oracle's rotated rows."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import paged as opaged
from oracle import rope as orope

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("d,rotary_dim", [(128, 128), (128, 64), (64, 64), (80, 32)])
def test_rope_store_bit_exact(dtype, d, rotary_dim):
    import openvino_contrib_b200 as b2a
    from openvino_contrib_b200 import _lib
    from openvino_contrib_b200.ops import _paged_desc
    lib = _lib.load()
    hkv, bs = 4, 16
    ctx = np.array([1, 17, 33, 250, 40])
    past = np.array([0, 3, 16, 200, 39], dtype=np.int32)
    qlen = (ctx - past).astype(np.int32)
    bi, bb, nb = opaged.build_block_tables(ctx, bs, seed=7, spare_blocks=2)
    sb = np.zeros(len(ctx) + 1, np.int32)
    sb[1:] = np.cumsum(qlen)
    ntok = int(sb[-1])
    g = torch.Generator().manual_seed(3)
    key = (torch.randn(ntok, hkv * d, generator=g) * 1.3).to(dtype)
    val = (torch.randn(ntok, hkv * d, generator=g) - 0.2).to(dtype)
    cos, sin = orope.rope_tables(256, rotary_dim)
    # oracle: rotate the key rows, then the ordinary store
    pos = orope.token_positions(past, sb)
    k_rot = orope.rope_rows(key.float().numpy().reshape(ntok, hkv, d), pos, cos, sin, rotary_dim).reshape(ntok, hkv * d)
    ref_k = np.full((nb, hkv, bs * (d + 4)), 0xFF, np.uint8)
    ref_v = ref_k.copy()
    opaged.kv_store_ref(k_rot, ref_k, past, sb, bi, bb, hkv, d, bs)
    opaged.kv_store_ref(val, ref_v, past, sb, bi, bb, hkv, d, bs)
    cache = b2a.PagedKvCache.allocate(nb, hkv, d, bs, torch.uint8)
    t = [torch.from_numpy(a).cuda() for a in (past, sb, bi, bb)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    desc = _paged_desc(dtype, cache, hkv, len(ctx), ntok, 0, 0, None, 0)
    kd, vd, cd, sd = key.cuda(), val.cuda(), torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda()
    rc = lib.b2a_paged_kv_store_rope(C.byref(desc), kd.data_ptr(), vd.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                     t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), cd.data_ptr(),
                                     sd.data_ptr(), rotary_dim, 256, status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(cache.k.cpu().numpy(), ref_k)
    assert np.array_equal(cache.v.cpu().numpy(), ref_v)   # values are not rotated
    # a table that ends before the last position: reported, that row is left alone
    status.zero_()
    rc = lib.b2a_paged_kv_store_rope(C.byref(desc), kd.data_ptr(), vd.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                     t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), cd.data_ptr(),
                                     sd.data_ptr(), rotary_dim, 249, status.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == _lib.DEV_BAD_LEN
    # descriptors that make no sense are refused on the host
    assert lib.b2a_paged_kv_store_rope(C.byref(desc), kd.data_ptr(), vd.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                       t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), cd.data_ptr(),
                                       sd.data_ptr(), d + 2, 256, status.data_ptr(), None) == 2
