"""KV-head sharding of the attention path over the GPUs of one node.

Heads are independent, so rank r of N owns KV heads [r*Hkv/N, (r+1)*Hkv/N) and the Hq/Hkv query heads that read
each of them; its K/V tensors and KV pools hold only those heads and nothing of K or V ever crosses NVLink.  The
single exchange is the all-gather of the per-head outputs (NCCL over NVLink in production; any
``torch.distributed`` backend works, which is how the host logic is tested on CPU with gloo).

The reference plugin has no counterpart: it never spans devices (one independent plugin configuration per device
id, ``modules/nvidia_plugin/src/cuda_plugin.cpp:25-32``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    hq: int
    hkv: int

    def __post_init__(self):
        if self.hkv % self.world != 0 or self.hq % self.hkv != 0:
            raise ValueError(f"cannot shard Hq={self.hq}, Hkv={self.hkv} over {self.world} ranks by KV head")

    @property
    def hkv_local(self) -> int:
        return self.hkv // self.world

    @property
    def hq_local(self) -> int:
        return self.hq // self.world

    @property
    def kv_heads(self) -> slice:
        return slice(self.rank * self.hkv_local, (self.rank + 1) * self.hkv_local)

    @property
    def q_heads(self) -> slice:
        return slice(self.rank * self.hq_local, (self.rank + 1) * self.hq_local)

    # ---- SDPA layout [B, H, S, D]
    def take_q(self, q: torch.Tensor) -> torch.Tensor:
        return q[:, self.q_heads]

    def take_kv(self, kv: torch.Tensor) -> torch.Tensor:
        return kv[:, self.kv_heads]

    # ---- paged layout [tokens, H*D]
    def take_q_rows(self, q: torch.Tensor, d: int) -> torch.Tensor:
        return q.view(q.shape[0], self.hq, d)[:, self.q_heads].reshape(q.shape[0], self.hq_local * d)

    def take_kv_rows(self, kv: torch.Tensor, d: int) -> torch.Tensor:
        return kv.view(kv.shape[0], self.hkv, d)[:, self.kv_heads].reshape(kv.shape[0], self.hkv_local * d)


def gather_heads_bhsd(local_out: torch.Tensor, shard: HeadShard, group=None,
                      buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather [B, Hq/N, S, D] shards into [B, Hq, S, D].

    One collective per batch entry, each landing directly in its [Hq, S, D] slab of the result (heads are the
    outermost axis there, so rank-major concatenation is already the final layout): no re-layout copy afterwards.
    ``buffer`` is the [B, Hq, S, D] result to fill.
    """
    if shard.world == 1:
        return local_out
    b, hl, s, d = local_out.shape
    if buffer is None:
        buffer = torch.empty((b, shard.world * hl, s, d), dtype=local_out.dtype, device=local_out.device)
    local_out = local_out.contiguous()
    for i in range(b):
        dist.all_gather_into_tensor(buffer[i], local_out[i], group=group)
    return buffer


def gather_heads_rows(local_out: torch.Tensor, shard: HeadShard, d: int, group=None,
                      buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather [tokens, Hq/N*D] shards into [tokens, Hq*D]."""
    if shard.world == 1:
        return local_out
    t = local_out.shape[0]
    if buffer is None:
        buffer = torch.empty((shard.world * t, shard.hq_local * d), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(buffer, local_out.contiguous(), group=group)
    return buffer.view(shard.world, t, shard.hq_local * d).permute(1, 0, 2).reshape(t, shard.hq * d)


def sharded_sdpa(q, k, v, shard: HeadShard, attend: Callable, group=None, **kw) -> torch.Tensor:
    """Run ``attend(q_local, k_local, v_local, **kw)`` on this rank's heads and gather the full output.

    ``attend`` is the device attention (``openvino_contrib_b200.sdpa`` on a GPU); the tests pass a CPU function to
    check the slicing and the gather order.
    """
    o = attend(shard.take_q(q).contiguous(), shard.take_kv(k).contiguous(), shard.take_kv(v).contiguous(), **kw)
    return gather_heads_bhsd(o, shard, group)


class ShardGroup:
    """Python face of ``b2a_shard_group``: staging buffers on every rank, mapped into every process with CUDA IPC.

    The 64-byte handles travel through ``torch.distributed`` (any backend) at set-up; after that a decode step
    involves no collective call: ``paged_attention`` enqueues the split-K decode of the local heads - whose last CTA
    per (sequence, KV head) merges the splits and stores this rank's output columns on every rank - and a small
    kernel that polls the arriving words and fills ``out_full``.
    """

    def __init__(self, shard: HeadShard, staging_bytes: int, group=None):
        import ctypes as C

        from . import _lib
        self._C, self._lib, self.shard = C, _lib.load(), shard
        self._h = C.c_void_p()
        _lib.check(self._lib.b2a_shard_group_create(shard.rank, shard.world, staging_bytes, C.byref(self._h)),
                   "b2a_shard_group_create")
        buf = C.create_string_buffer(64)
        _lib.check(self._lib.b2a_shard_group_handle(self._h, buf), "b2a_shard_group_handle")
        handles = [None] * shard.world
        if shard.world > 1:
            dist.all_gather_object(handles, bytes(buf.raw), group=group)
        else:
            handles[0] = bytes(buf.raw)
        _lib.check(self._lib.b2a_shard_group_connect(self._h, b"".join(handles)), "b2a_shard_group_connect")
        if shard.world > 1:
            dist.barrier(group=group)  # every rank has mapped every peer before anyone pushes

    def close(self):
        if getattr(self, "_h", None):
            self._lib.b2a_shard_group_destroy(self._h)
            self._h = None

    def set_wait_ms(self, milliseconds: int) -> None:
        """Bound of every device-side wait on another rank (default one second); when it runs out the step's kernels
        return and the status word carries ``DEV_TIMEOUT``."""
        from . import _lib
        _lib.check(self._lib.b2a_shard_group_set_wait_ms(self._h, int(milliseconds)), "b2a_shard_group_set_wait_ms")

    def reset(self, group=None) -> None:
        """Back to the state of a fresh group, on all ranks together (after a timeout the ranks' step counters no
        longer agree).  Call it on every rank, between steps."""
        from . import _lib
        torch.cuda.synchronize()
        if self.shard.world > 1:
            dist.barrier(group=group)   # every rank's device is idle: nobody stores into a peer any more
        _lib.check(self._lib.b2a_shard_group_reset(self._h), "b2a_shard_group_reset")
        if self.shard.world > 1:
            dist.barrier(group=group)

    def __del__(self):
        self.close()

    def paged_attention(self, query_local, cache_local, past_lens, subsequence_begins, block_indices,
                        block_indices_begins, max_context_len: int, out_full: Optional[torch.Tensor],
                        workspace: torch.Tensor, scale: Optional[float] = None,
                        status: Optional[torch.Tensor] = None, stream=None, cache_rows_settled: bool = False):
        """One decode step on this rank's heads; the [tokens, Hq*D] result is complete on every rank afterwards.

        With ``out_full=None`` the step is a single kernel that produces the rows in the group's own buffer on every
        rank; the returned tensor is a view of that buffer (valid until the next step on this group).  With a
        caller's ``out_full`` the rows travel as 8-byte {two values, step number} words through staging buffers of
        twice the output size and the decode kernel's own CTAs (a second kernel when there are more rows than SMs)
        copy them there.  ``cache_rows_settled``: see ``ops.paged_attention``.
        """
        from . import _lib
        from .ops import _paged_desc, _ptr, _stream_ptr
        C = self._C
        n = query_local.shape[0]
        if out_full is None:
            ptr = C.c_void_p()
            _lib.check(self._lib.b2a_shard_group_output(self._h, C.byref(ptr)), "b2a_shard_group_output")
            out_full = _device_view(ptr.value, (n, self.shard.hq * cache_local.dv), query_local.dtype,
                                    query_local.device)
        d = _paged_desc(query_local.dtype, cache_local, self.shard.hq_local, past_lens.shape[0], n, max_context_len,
                        1, scale, 0, cache_rows_settled=cache_rows_settled)
        _lib.check(self._lib.b2a_paged_attention_sharded(
            self._h, C.byref(d), query_local.data_ptr(), cache_local.k.data_ptr(), cache_local.v.data_ptr(),
            past_lens.data_ptr(), subsequence_begins.data_ptr(), block_indices.data_ptr(),
            block_indices_begins.data_ptr(), out_full.data_ptr(), workspace.data_ptr(),
            workspace.numel() * workspace.element_size(), _ptr(status), _stream_ptr(stream)),
            "b2a_paged_attention_sharded")
        return out_full

    def sdpa(self, q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor, causal: bool = False,
             scale: Optional[float] = None, status: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """Prefill SDPA on this rank's heads (q [B, Hq_local, S, 128], k/v [B, Hkv_local, S, 128], f16/bf16).

        Returns the complete [B, Hq, S, 128] result of all ranks as a view of the group's own memory: every rank's
        kernel stores its output tiles into every rank's buffer while it computes.  The view alternates between
        two buffers from call to call: use it (on the same stream) before the next call on this group.
        """
        from . import _lib
        from .ops import _dtype_code, _ptr, _stream_ptr
        C = self._C
        fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
        q4, k4, v4 = fix(q_local), fix(k_local), fix(v_local)
        B, Hq, Sq, D = q4.shape
        d = _lib.SdpaDesc()
        d.dtype = _dtype_code(q4.dtype)
        d.B, d.Hq, d.Hkv, d.Sq, d.Skv, d.D, d.Dv = B, Hq, k4.shape[1], Sq, k4.shape[2], D, v4.shape[-1]
        d.causal = int(bool(causal))
        d.scale = 0.0 if scale is None else float(scale)
        d.q_strides[:] = q4.stride()
        d.k_strides[:] = k4.stride()
        d.v_strides[:] = v4.stride()
        d.mask_kind = _lib.MASK_NONE
        out = C.c_void_p()
        _lib.check(self._lib.b2a_sdpa_forward_sharded(self._h, C.byref(d), q4.data_ptr(), k4.data_ptr(),
                                                      v4.data_ptr(), C.byref(out), _ptr(status), _stream_ptr(stream)),
                   "b2a_sdpa_forward_sharded")
        shape = (B, Hq * self.shard.world, Sq, v4.shape[-1])
        return _device_view(out.value, shape, q4.dtype, q4.device)


class _RawDeviceMemory:
    """Device memory owned by the library, described through ``__cuda_array_interface__`` (as 16-bit words)."""

    def __init__(self, ptr: int, n16: int):
        self.__cuda_array_interface__ = {"shape": (n16,), "typestr": "<i2", "data": (ptr, False), "version": 2}


def _device_view(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    words = torch.as_tensor(_RawDeviceMemory(ptr, n), device=device)
    return words.view(dtype).view(*shape)
