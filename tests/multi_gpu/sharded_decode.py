"""Head-sharded decode on N GPUs (one process per GPU): the peer-store exchange against the oracle and against
the NCCL all-gather of the same shards.  Launch:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/multi_gpu/sharded_decode.py

Every rank builds the same full problem from one seed, keeps its KV heads, runs three steps (the exchange
alternates two staging buffers, so odd and even steps are both exercised) and checks the full-width output
against the oracle, against the NCCL gather of the plain kernel and between the ranks.
NVLS is not needed and left off.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import openvino_contrib_b200 as b2a
    from openvino_contrib_b200.sharding import HeadShard, ShardGroup, gather_heads_rows
    from tests.helpers import PagedWorkload, assert_close

    hq, hkv, d = 64, 8, 128
    ctx = [37, 1000, 2049, 16, 513, 4096]
    w = PagedWorkload(ctx, [1] * len(ctx), hq, hkv, d, seed=77)
    shard = HeadShard(rank, world, hq, hkv)
    n = len(ctx)
    # this rank's slice of the pools: [blocks, Hkv, chunk] -> local KV heads
    kc = torch.from_numpy(w.k_cache[:, shard.kv_heads].copy()).cuda()
    vc = torch.from_numpy(w.v_cache[:, shard.kv_heads].copy()).cuda()
    cache = b2a.PagedKvCache(kc, vc, shard.hkv_local, d, d, 16, torch.uint8)
    tables = w.device_tables()
    ws = torch.empty(max(16, b2a.ops.paged_workspace_bytes(torch.float16, cache, shard.hq_local, n, n, max(ctx), 1)),
                     dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # a caller's output buffer: the decode kernel's last CTA per (sequence, KV head) merges and sends the value pairs
    # with the step number, the receiving kernel polls the words (staging of twice the output size)
    group = ShardGroup(shard, staging_bytes=2 * n * hq * d * 2)
    for step in range(3):
        q_full = torch.from_numpy(w.query * (1.0 + 0.25 * step)).to(torch.float16)
        ref = w.reference(q_full.float().numpy())
        q_local = shard.take_q_rows(q_full, d).contiguous().cuda()
        out = torch.zeros(n, hq * d, dtype=torch.float16, device="cuda")
        group.paged_attention(q_local, cache, *tables, max_context_len=max(ctx), out_full=out, workspace=ws,
                              status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"rank {rank} step {step}: status {int(status.item())}"
        assert_close(out, ref, torch.float16, f"rank {rank} step {step}")
        # and bit-identical to the NCCL all-gather of the plain kernel's shards (the in-kernel merge performs the
        # merge kernel's arithmetic operation for operation)
        o_local = b2a.paged_attention(q_local, cache, *tables, hq=shard.hq_local, max_context_len=max(ctx),
                                      max_q_len=1, workspace=ws)
        o_nccl = gather_heads_rows(o_local, shard, d)
        assert torch.equal(o_nccl, out), f"rank {rank} step {step}: differs from the NCCL gather"
        # every rank holds the same bits
        mine = out.clone()
        dist.broadcast(mine, src=0)
        assert torch.equal(mine, out), f"rank {rank} step {step}: ranks disagree"
    # a sequence with inconsistent tables arrives as zeros on every rank and is reported; no rank waits for ever
    bad = tables[0].clone()
    bad[1] = -3
    out = torch.full((n, hq * d), 3.0, dtype=torch.float16, device="cuda")
    group.paged_attention(q_local, cache, bad, *tables[1:], max_context_len=max(ctx), out_full=out, workspace=ws,
                          status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 4 and float(out[1].float().abs().max()) == 0.0, f"rank {rank}: bad row"
    assert_close(out[2:], ref[2:], torch.float16, f"rank {rank}: rows next to the bad one")
    status.zero_()
    dist.barrier()
    group.close()
    # the one-kernel step: results produced in place in the group's own buffer on every rank
    group2 = ShardGroup(shard, staging_bytes=n * hq * d * 2)
    for step in range(3):
        q_full = torch.from_numpy(w.query * (1.0 - 0.125 * step)).to(torch.float16)
        q_local = shard.take_q_rows(q_full, d).contiguous().cuda()
        out = group2.paged_attention(q_local, cache, *tables, max_context_len=max(ctx), out_full=None, workspace=ws,
                                     status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"rank {rank} in-place step {step}: status {int(status.item())}"
        o_local = b2a.paged_attention(q_local, cache, *tables, hq=shard.hq_local, max_context_len=max(ctx),
                                      max_q_len=1, workspace=ws)
        o_nccl = gather_heads_rows(o_local, shard, d)
        assert torch.equal(o_nccl, out), f"rank {rank} in-place step {step}: differs from the NCCL gather"
        assert_close(out, w.reference(q_full.float().numpy()), torch.float16, f"rank {rank} in-place step {step}")
    # the same captured once and replayed: the step counter lives on the device
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            out_g = group2.paged_attention(q_local, cache, *tables, max_context_len=max(ctx), out_full=None,
                                           workspace=ws, status=status, stream=side)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.equal(o_nccl, out_g), f"rank {rank}: graph replay of the in-place step"
    dist.barrier()
    group2.close()
    if rank == 0:
        print(f"sharded decode ok on {world} GPUs")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
