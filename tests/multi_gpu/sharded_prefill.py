"""Head-sharded prefill SDPA on N GPUs (one process per GPU): the tensor-core kernel storing its output tiles into
every rank's buffer, checked against the single-GPU kernel over all heads and against the numpy oracle.  Launch:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/multi_gpu/sharded_prefill.py

Every rank builds the same full problem from one seed, keeps its heads and runs three steps (the result alternates
between two buffers, so odd and even steps are both exercised; the second step also checks that the first step's
view was not overwritten).
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
    from openvino_contrib_b200.sharding import HeadShard, ShardGroup
    from oracle.sdpa import sdpa_ref
    from tests.helpers import assert_close

    B, hq, hkv, S, D = 2, 16, 8, 640, 128  # S not a multiple of the 256-row CTA: ragged last tile pair
    shard = HeadShard(rank, world, hq, hkv)
    group = ShardGroup(shard, staging_bytes=B * hq * S * D * 2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    prev = None
    for step, (dtype, causal) in enumerate([(torch.bfloat16, True), (torch.float16, False), (torch.bfloat16, True)]):
        gen = torch.Generator().manual_seed(100 + step)
        q = (torch.randn(B, hq, S, D, generator=gen) * 0.5).to(dtype)
        k = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(dtype)
        v = (torch.randn(B, hkv, S, D, generator=gen) * 0.5).to(dtype)
        ql = q[:, shard.q_heads].contiguous().cuda()
        kl = k[:, shard.kv_heads].contiguous().cuda()
        vl = v[:, shard.kv_heads].contiguous().cuda()
        full = group.sdpa(ql, kl, vl, causal=causal, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0, f"rank {rank} step {step}: status {int(status.item())}"
        single = b2a.sdpa(q.cuda(), k.cuda(), v.cuda(), causal=causal)  # all heads on this GPU, same kernel
        assert torch.equal(full, single), f"rank {rank} step {step}: differs from the single-GPU kernel"
        if step == 0:
            ref = sdpa_ref(q.float().numpy(), k.float().numpy(), v.float().numpy(), causal=causal)
            assert_close(full, ref, dtype, f"rank {rank} step {step}")
        if prev is not None:
            assert torch.equal(prev[0], prev[1]), f"rank {rank}: step {step} overwrote the previous step's result"
        prev = (full, single.clone())
        dist.barrier()
    group.close()
    if rank == 0:
        print(f"sharded prefill ok on {world} GPUs")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
