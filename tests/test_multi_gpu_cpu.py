"""Head sharding + output all-gather with two gloo ranks on CPU: the N > 1 host logic without a GPU."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from openvino_contrib_b200.sharding import HeadShard, gather_heads_rows, sharded_sdpa
        from oracle import sdpa as osdpa
        B, Hq, Hkv, S, D = 2, 8, 4, 40, 16
        g = torch.Generator().manual_seed(0)  # every rank draws the same full problem
        q = torch.randn(B, Hq, S, D, generator=g)
        k = torch.randn(B, Hkv, S, D, generator=g)
        v = torch.randn(B, Hkv, S, D, generator=g)
        shard = HeadShard(rank, world, Hq, Hkv)
        attend = lambda ql, kl, vl, causal: torch.from_numpy(osdpa.sdpa_ref(ql, kl, vl, causal=causal))
        full = sharded_sdpa(q, k, v, shard, attend, causal=True)
        ref = osdpa.sdpa_ref(q, k, v, causal=True)
        np.testing.assert_allclose(full.numpy(), ref, rtol=1e-6, atol=1e-6)
        # paged row layout [tokens, Hq*D]: rank r's columns are heads [r*Hq/N, (r+1)*Hq/N)
        rows = torch.arange(3 * Hq * D, dtype=torch.float32).reshape(3, Hq * D)
        mine = shard.take_q_rows(rows, D)
        assert mine.shape == (3, Hq // world * D)
        back = gather_heads_rows(mine, shard, D)
        assert torch.equal(back, rows)
        kvrows = torch.arange(3 * Hkv * D, dtype=torch.float32).reshape(3, Hkv * D)
        assert torch.equal(shard.take_kv_rows(kvrows, D), kvrows.view(3, Hkv, D)[:, shard.kv_heads].reshape(3, -1))
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_two_rank_head_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _absent_worker(rank, world, port, out_dir):
    """Rank 1 never posts its shard: rank 0's all-gather must end with an error inside the process-group timeout
    instead of waiting for ever - the host-side half of failure detection (the device-side half is the bounded
    wait of the peer-store exchange)."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from openvino_contrib_b200.sharding import HeadShard, gather_heads_rows
    shard = HeadShard(rank, world, 8, 4)
    mine = torch.full((3, shard.hq_local * 16), float(rank))
    if rank == 0:
        t0 = time.time()
        try:
            gather_heads_rows(mine, shard, 16)
            outcome = "completed"          # must not happen: the other rank never joined
        except Exception as e:             # gloo reports the timeout as a RuntimeError / DistBackendError
            outcome = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
        open(os.path.join(out_dir, "outcome"), "w").write(outcome)
    else:
        time.sleep(6.0)                    # stays alive, between steps, and simply never calls the collective
    # no destroy_process_group: its own barrier would wait for the rank that left the protocol


def test_absent_rank_ends_the_gather_with_an_error(tmp_path):
    world = 2
    ctx = mp.spawn(_absent_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=False)
    ctx.join(timeout=60)
    for p in ctx.processes:
        if p.is_alive():
            p.terminate()
    outcome = (tmp_path / "outcome").read_text()
    assert outcome.startswith("error after"), outcome
    assert float(outcome.split()[2][:-2]) < 30.0


def test_shard_rejects_uneven_split():
    import pytest
    from openvino_contrib_b200.sharding import HeadShard
    with pytest.raises(ValueError):
        HeadShard(0, 3, 32, 8)
    s = HeadShard(1, 4, 32, 8)
    assert s.kv_heads == slice(2, 4) and s.q_heads == slice(8, 16)
