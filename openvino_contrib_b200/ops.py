"""Host-side callers of the C ABI for Python users and for the parity tests.

The operator classes mirror the interface every nvidia_plugin operation implements
(``modules/nvidia_plugin/src/cuda_operation_base.hpp:33-60``): construct once from the node's static
attributes, ask ``GetWorkBufferRequest()`` for scratch sizes, then ``Execute(inputs, outputs, workbuffers)``
on device buffers, any number of times, on any stream.  ``torch`` is used for device memory and streams only;
all arithmetic happens in libb2a.so.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import B2AError, PagedDesc, SdpaDesc, check

_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.uint8: _lib.U8}


def _dtype_code(t: torch.dtype) -> int:
    if t not in _DTYPES:
        raise TypeError(f"unsupported element type {t}")
    return _DTYPES[t]


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("libb2a works on device memory only: pass CUDA tensors (there is no CPU path)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


# ------------------------------------------------------------------------------------------------------------
# ScaledDotProductAttention
# ------------------------------------------------------------------------------------------------------------

def _as_bhsd(x: torch.Tensor) -> torch.Tensor:
    """[..., S, E] -> a 4-D [B, H, S, E] view (rank 3 is [N, S, E]: batch N, one head)."""
    if x.dim() < 3:
        raise ValueError("SDPA operands need rank >= 3")
    if x.dim() == 3:
        return x.unsqueeze(1)
    if x.dim() == 4:
        return x
    return x.reshape(-1, *x.shape[-3:])


def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attn_mask: Optional[torch.Tensor] = None,
         scale: Optional[float] = None, causal: bool = False, out: Optional[torch.Tensor] = None,
         stream: Optional[torch.cuda.Stream] = None, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``ov::op::v13::ScaledDotProductAttention`` on device tensors: softmax(q k^T * scale + mask) v.

    q [..., Hq, Sq, E], k [..., Hkv, Skv, E], v [..., Hkv, Skv, Ev]; Hq a multiple of Hkv.  ``causal`` ignores
    ``attn_mask``.  A boolean mask keeps where true, a floating mask is added.  Strided views are passed
    through as they are, provided the innermost stride is 1.
    """
    _require_cuda(q, k, v, attn_mask, out)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k and v must share one element type")
    q4, k4, v4 = _as_bhsd(q), _as_bhsd(k), _as_bhsd(v)
    fix = lambda t: t if t.stride(-1) == 1 else t.contiguous()
    q4, k4, v4 = fix(q4), fix(k4), fix(v4)
    B, Hq, Sq, D = q4.shape
    Bk, Hkv, Skv, Dk = k4.shape
    Dv = v4.shape[-1]
    if Bk != B or v4.shape[:3] != k4.shape[:3] or Dk != D:
        raise ValueError(f"inconsistent SDPA shapes q{tuple(q.shape)} k{tuple(k.shape)} v{tuple(v.shape)}")
    out_shape = (*q.shape[:-1], Dv)
    if out is None:
        out = torch.empty(out_shape, dtype=q.dtype, device=q.device)
    o4 = _as_bhsd(out)
    if o4.stride(-1) != 1:
        raise ValueError("the output needs a unit innermost stride")

    d = SdpaDesc()
    d.dtype = _dtype_code(q.dtype)
    d.B, d.Hq, d.Hkv, d.Sq, d.Skv, d.D, d.Dv = B, Hq, Hkv, Sq, Skv, D, Dv
    d.causal = int(bool(causal))
    d.scale = 0.0 if scale is None else float(scale)
    d.q_strides[:] = q4.stride()
    d.k_strides[:] = k4.stride()
    d.v_strides[:] = v4.stride()
    d.o_strides[:] = o4.stride()
    mask_t = None
    d.mask_kind = _lib.MASK_NONE
    if attn_mask is not None and not causal:
        m = attn_mask
        if m.dtype == torch.bool:
            d.mask_kind = _lib.MASK_BOOL
            m = m.view(torch.uint8) if m.is_contiguous() else m.to(torch.uint8)
        else:
            d.mask_kind = _lib.MASK_ADD
            m = m.to(q.dtype)
        while m.dim() < 4:
            m = m.unsqueeze(0)
        if m.dim() > 4:
            m = m.reshape(-1, *m.shape[-3:])
        m = m.expand(B, Hq, Sq, Skv)  # broadcast dimensions get stride 0
        d.mask_strides[:] = m.stride()
        mask_t = m
    lib = _lib.load()
    ws = C.c_size_t(0)
    check(lib.b2a_sdpa_workspace_bytes(C.byref(d), sm_count(), C.byref(ws)), "b2a_sdpa_workspace_bytes")
    wbuf = torch.empty(ws.value, dtype=torch.uint8, device=q.device) if ws.value else None
    check(lib.b2a_sdpa_forward(C.byref(d), q4.data_ptr(), k4.data_ptr(), v4.data_ptr(), _ptr(mask_t),
                               o4.data_ptr(), _ptr(wbuf), ws.value, _ptr(status), _stream_ptr(stream)),
          "b2a_sdpa_forward")
    return out


class HostSdpaPipeline:
    """SDPA on HOST tensors (pinned memory) through the C++ ``HostSdpaRunner``.

    What a plugin does for a model whose inputs and outputs live in host memory (``ParameterOp`` uploads,
    ``ResultOp`` downloads, modules/nvidia_plugin/src/ops/parameter.cpp:24-33 and result.cpp:28-43) - except that
    the problem is cut into pieces of a few KV heads of one batch entry and the upload of piece i+1, ``SdpaOp::Execute`` on
    piece i and the download of piece i-1 run on three streams at the same time, so a step costs about the longer
    of the two copy directions instead of their sum plus the kernel.  The C++ operator is created once, through the
    operation registry; device tensors are allocated once, for the shapes given at construction.
    """

    def __init__(self, b: int, hq: int, hkv: int, sq: int, skv: int, d: int, dtype: torch.dtype, causal: bool = False,
                 kv_heads_per_piece: int = 0):
        self._lib = _lib.load()
        self._h = C.c_void_p()
        self.shape_q, self.shape_kv, self.dtype = (b, hq, sq, d), (b, hkv, skv, d), dtype
        check(self._lib.b2a_host_sdpa_create(_dtype_code(dtype), b, hq, hkv, sq, skv, d, int(bool(causal)),
                                             int(kv_heads_per_piece), C.byref(self._h)), "b2a_host_sdpa_create")
        self.pieces = self._lib.b2a_host_sdpa_pieces(self._h)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.b2a_host_sdpa_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def __call__(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                 out_host: torch.Tensor) -> torch.Tensor:
        """Enqueues the whole step behind the current stream's work; ``out_host`` is complete when the current stream
        has been synchronised."""
        for t, shape in ((q_host, self.shape_q), (k_host, self.shape_kv), (v_host, self.shape_kv), (out_host, self.shape_q)):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("HostSdpaPipeline takes pinned host tensors")
            if tuple(t.shape) != shape or t.dtype != self.dtype or not t.is_contiguous():
                raise ValueError(f"HostSdpaPipeline was built for dense {self.dtype} tensors of shape {shape}")
        check(self._lib.b2a_host_sdpa_run(self._h, q_host.data_ptr(), k_host.data_ptr(), v_host.data_ptr(),
                                          out_host.data_ptr(), _stream_ptr(None)), "b2a_host_sdpa_run")
        return out_host


def _host_scalar(x, what: str):
    """A constant operand: a Python number or a host tensor.  A device tensor is refused - reading it would make
    ``Execute`` wait for the device, which an operation that reports full CUDA-graph compatibility must not do."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        if x.is_cuda:
            raise B2AError(7, f"{what} must be a constant (host value), not a device tensor")
        return x.item()
    return x


class SdpaOp:
    """Operator-shaped wrapper: static attributes at construction, device buffers at ``Execute``.

    Mirrors what a nvidia_plugin operation for ``ScaledDotProductAttention`` looks like
    (``cuda_operation_base.hpp:80-149``); inputs are (q, k, v[, attention_mask[, scale]]).
    """

    type_name = "ScaledDotProductAttention"

    def __init__(self, causal: bool = False):
        self.causal = bool(causal)

    def GetCudaGraphCompatibility(self) -> str:
        return "FULL"  # launches only; no allocation, no synchronisation

    def GetWorkBufferRequest(self):
        return {"immutable_sizes": [], "mutable_sizes": []}

    def Execute(self, inputs: Sequence[torch.Tensor], outputs: Sequence[torch.Tensor], workbuffers=None,
                stream: Optional[torch.cuda.Stream] = None) -> None:
        if not 3 <= len(inputs) <= 5 or len(outputs) != 1:
            raise ValueError("ScaledDotProductAttention takes 3 to 5 inputs and 1 output")
        mask = inputs[3] if len(inputs) > 3 else None
        scale = _host_scalar(inputs[4], "ScaledDotProductAttention: scale") if len(inputs) > 4 else None
        sdpa(inputs[0], inputs[1], inputs[2], mask, scale, self.causal, out=outputs[0], stream=stream)


# ------------------------------------------------------------------------------------------------------------
# PagedAttentionExtension
# ------------------------------------------------------------------------------------------------------------

@dataclass
class PagedKvCache:
    """Device-resident block pools [num_blocks, Hkv, chunk_bytes] (u8) or [num_blocks, Hkv, bs, D] (f16/bf16)."""
    k: torch.Tensor
    v: torch.Tensor
    hkv: int
    d: int
    dv: int
    block_size: int
    kv_dtype: torch.dtype

    @staticmethod
    def allocate(num_blocks: int, hkv: int, d: int, block_size: int = 16, kv_dtype: torch.dtype = torch.uint8,
                 device="cuda", dv: Optional[int] = None, poison: Optional[int] = 0xFF) -> "PagedKvCache":
        dv = d if dv is None else dv
        lib = _lib.load()
        code = _dtype_code(kv_dtype)
        ck, cv = lib.b2a_paged_chunk_bytes(code, block_size, d), lib.b2a_paged_chunk_bytes(code, block_size, dv)
        if ck == 0 or cv == 0:
            raise ValueError("unsupported cache geometry")
        mk = lambda cb: (torch.full((num_blocks, hkv, cb), poison, dtype=torch.uint8, device=device)
                         if poison is not None else torch.empty((num_blocks, hkv, cb), dtype=torch.uint8, device=device))
        return PagedKvCache(mk(ck), mk(cv), hkv, d, dv, block_size, kv_dtype)

    @property
    def num_blocks(self) -> int:
        return self.k.shape[0]


def _paged_desc(q_dtype, cache: PagedKvCache, hq: int, num_seqs: int, num_tokens: int, max_context_len: int,
                max_q_len: int, scale: Optional[float], sliding_window: int, prefill_row_blocks: int = 0,
                prefill_kv_tokens: int = 0, cache_rows_settled: bool = False) -> PagedDesc:
    d = PagedDesc()
    d.q_dtype = _dtype_code(q_dtype)
    d.kv_dtype = _dtype_code(cache.kv_dtype)
    d.Hq, d.Hkv, d.D, d.Dv, d.block_size = hq, cache.hkv, cache.d, cache.dv, cache.block_size
    d.num_seqs, d.num_tokens, d.num_blocks_total = num_seqs, num_tokens, cache.num_blocks
    d.max_context_len, d.max_q_len = max_context_len, max_q_len
    d.scale = 0.0 if scale is None else float(scale)
    d.sliding_window = int(sliding_window)
    d.prefill_row_blocks = int(prefill_row_blocks)
    d.prefill_kv_tokens = int(prefill_kv_tokens)
    d.cache_rows_settled = 1 if cache_rows_settled else 0
    return d


def _i32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise TypeError("step tables must be contiguous int32 device tensors")
    return t


def paged_kv_store(key: torch.Tensor, value: torch.Tensor, cache: PagedKvCache, past_lens, subsequence_begins,
                   block_indices, block_indices_begins, stream=None, status: Optional[torch.Tensor] = None) -> None:
    """Append key [tokens, Hkv*D] / value [tokens, Hkv*Dv] to the pools through the block table."""
    _require_cuda(key, value, cache.k, cache.v, past_lens, subsequence_begins, block_indices, block_indices_begins)
    if key.dtype != value.dtype or not key.is_contiguous() or not value.is_contiguous():
        raise ValueError("key and value must be dense and share one element type")
    num_tokens, num_seqs = key.shape[0], past_lens.shape[0]
    if key.shape[1] != cache.hkv * cache.d or value.shape[1] != cache.hkv * cache.dv or value.shape[0] != num_tokens:
        raise ValueError("key/value row width does not match the cache geometry")
    d = _paged_desc(key.dtype, cache, cache.hkv, num_seqs, num_tokens, 0, 0, None, 0)
    check(_lib.load().b2a_paged_kv_store(C.byref(d), key.data_ptr(), value.data_ptr(), cache.k.data_ptr(),
                                         cache.v.data_ptr(), _i32(past_lens).data_ptr(),
                                         _i32(subsequence_begins).data_ptr(), _i32(block_indices).data_ptr(),
                                         _i32(block_indices_begins).data_ptr(), _ptr(status), _stream_ptr(stream)),
          "b2a_paged_kv_store")


def paged_workspace_bytes(q_dtype, cache: PagedKvCache, hq: int, num_seqs: int, num_tokens: int,
                          max_context_len: int, max_q_len: int, prefill_row_blocks: int = 0,
                          prefill_kv_tokens: int = 0) -> int:
    d = _paged_desc(q_dtype, cache, hq, num_seqs, num_tokens, max_context_len, max_q_len, None, 0,
                    prefill_row_blocks, prefill_kv_tokens)
    ws = C.c_size_t(0)
    check(_lib.load().b2a_paged_workspace_bytes(C.byref(d), 0, C.byref(ws)), "b2a_paged_workspace_bytes")
    return ws.value


def paged_attention(query: torch.Tensor, cache: PagedKvCache, past_lens, subsequence_begins, block_indices,
                    block_indices_begins, hq: int, max_context_len: int, max_q_len: int,
                    scale: Optional[float] = None, sliding_window: int = 0, out: Optional[torch.Tensor] = None,
                    workspace: Optional[torch.Tensor] = None, stream=None,
                    status: Optional[torch.Tensor] = None, prefill_row_blocks: int = 0,
                    prefill_kv_tokens: int = 0, cache_rows_settled: bool = False) -> torch.Tensor:
    """Attention of query [tokens, Hq*D] over the cache; returns [tokens, Hq*Dv].

    ``prefill_row_blocks`` and ``prefill_kv_tokens`` are the optional scheduler hints of ``b2a_paged_desc``
    (``KvBlockManager`` reports both); the second lets a mixed step de-quantise its prefill contexts once.
    ``cache_rows_settled``: the caller's promise that the kernel directly before this call on the stream writes no
    cache row other than this step's new tokens (see ``b2a_paged_desc``)."""
    _require_cuda(query, cache.k, cache.v, past_lens, subsequence_begins, block_indices, block_indices_begins, out)
    if not query.is_contiguous() or query.shape[1] != hq * cache.d:
        raise ValueError("query must be dense [tokens, Hq*D]")
    num_tokens, num_seqs = query.shape[0], past_lens.shape[0]
    if out is None:
        out = torch.empty((num_tokens, hq * cache.dv), dtype=query.dtype, device=query.device)
    d = _paged_desc(query.dtype, cache, hq, num_seqs, num_tokens, max_context_len, max_q_len, scale, sliding_window,
                    prefill_row_blocks, prefill_kv_tokens, cache_rows_settled)
    lib = _lib.load()
    ws = C.c_size_t(0)
    check(lib.b2a_paged_workspace_bytes(C.byref(d), 0, C.byref(ws)), "b2a_paged_workspace_bytes")
    if ws.value and (workspace is None or workspace.numel() * workspace.element_size() < ws.value):
        workspace = torch.empty(ws.value, dtype=torch.uint8, device=query.device)
    wbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(lib.b2a_paged_attention(C.byref(d), query.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(),
                                  _i32(past_lens).data_ptr(), _i32(subsequence_begins).data_ptr(),
                                  _i32(block_indices).data_ptr(), _i32(block_indices_begins).data_ptr(),
                                  out.data_ptr(), _ptr(workspace), wbytes, _ptr(status), _stream_ptr(stream)),
          "b2a_paged_attention")
    return out


def paged_last_token_scores(query: torch.Tensor, cache: PagedKvCache, past_lens, subsequence_begins, block_indices,
                            block_indices_begins, hq: int, max_context_len: int, scale: Optional[float] = None,
                            sliding_window: int = 0, scores: Optional[torch.Tensor] = None,
                            workspace: Optional[torch.Tensor] = None, stream=None,
                            status: Optional[torch.Tensor] = None):
    """Score output of the paged attention: per sequence, the attention probabilities of its last query token over
    its cached keys, summed over the query heads.  Returns ``(scores, score_begins)``: flat float32 scores and the
    int32 [num_seqs + 1] offsets of the sequences in it (``b2a_paged_last_token_scores``).  ``scores`` defaults to a
    buffer of ``num_seqs * max_context_len`` floats."""
    _require_cuda(query, cache.k, past_lens, subsequence_begins, block_indices, block_indices_begins, scores)
    if not query.is_contiguous() or query.shape[1] != hq * cache.d:
        raise ValueError("query must be dense [tokens, Hq*D]")
    num_tokens, num_seqs = query.shape[0], past_lens.shape[0]
    if scores is None:
        scores = torch.empty(num_seqs * max_context_len, dtype=torch.float32, device=query.device)
    if scores.dtype != torch.float32 or not scores.is_contiguous():
        raise TypeError("scores must be a contiguous float32 tensor")
    begins = torch.empty(num_seqs + 1, dtype=torch.int32, device=query.device)
    d = _paged_desc(query.dtype, cache, hq, num_seqs, num_tokens, max_context_len, max(1, num_tokens - num_seqs + 1),
                    scale, sliding_window)
    lib = _lib.load()
    ws = C.c_size_t(0)
    check(lib.b2a_paged_scores_workspace_bytes(C.byref(d), 0, C.byref(ws)), "b2a_paged_scores_workspace_bytes")
    if workspace is None or workspace.numel() * workspace.element_size() < ws.value:
        workspace = torch.empty(max(16, ws.value), dtype=torch.uint8, device=query.device)
    check(lib.b2a_paged_last_token_scores(C.byref(d), query.data_ptr(), cache.k.data_ptr(), _i32(past_lens).data_ptr(),
                                          _i32(subsequence_begins).data_ptr(), _i32(block_indices).data_ptr(),
                                          _i32(block_indices_begins).data_ptr(), scores.data_ptr(), scores.numel(),
                                          begins.data_ptr(), workspace.data_ptr(),
                                          workspace.numel() * workspace.element_size(), _ptr(status),
                                          _stream_ptr(stream)),
          "b2a_paged_last_token_scores")
    return scores, begins


class PagedAttentionOp:
    """Operator-shaped wrapper for ``PagedAttentionExtension`` (the Python twin of the C++ ``PagedAttentionOp``).

    ``Execute`` takes the operands in the op's order: query, key, value, key_cache, value_cache, past_lens,
    subsequence_begins, block_indices, block_indices_begins, scale, sliding_window[, alibi_slopes,
    max_context_len].  It first appends key/value to the caches, then attends.  The constructor fixes what is
    static for a compiled model - head counts, head size, block size, the capacity maxima, and the scale and
    sliding window (Constants in an exported model) - so one instance serves every step of a continuous-batching
    loop whatever its token and sequence counts, and nothing about it changes afterwards: what a scheduler knows
    about one step is passed to that ``Execute`` call.  ``Execute`` only enqueues: it allocates nothing (the work
    buffer must be the one ``GetWorkBufferRequest`` asked for) and never waits for the device.
    """

    type_name = "PagedAttentionExtension"

    def __init__(self, hq: int, hkv: int, d: int, block_size: int = 16, kv_dtype: torch.dtype = torch.uint8,
                 max_seqs: int = 256, max_context_len: int = 32768, max_prefill_kv_tokens: int = 0,
                 scale: Optional[float] = None, sliding_window: int = 0, q_dtype: torch.dtype = torch.float16,
                 max_step_tokens: Optional[int] = None):
        self.hq, self.hkv, self.d, self.block_size, self.kv_dtype = hq, hkv, d, block_size, kv_dtype
        self.max_seqs, self.max_context_len = int(max_seqs), int(max_context_len)
        # tokens of one step: by default one full context plus a token for every other sequence
        self.max_step_tokens = int(max_step_tokens) if max_step_tokens else self.max_context_len + self.max_seqs
        self.max_prefill_kv_tokens = (int(max_prefill_kv_tokens) + 127) // 128 * 128
        self.scale, self.sliding_window, self.q_dtype = scale, int(sliding_window), q_dtype
        self._workspace_bytes = self._workspace_bound()

    def GetCudaGraphCompatibility(self) -> str:
        return "FULL"

    def _geometry(self) -> "PagedKvCache":
        return PagedKvCache(torch.empty((0, self.hkv, 1), dtype=torch.uint8), torch.empty(0), self.hkv, self.d, self.d,
                            self.block_size, self.kv_dtype)

    def _workspace_bound(self) -> int:
        """Largest request over every step the capacity admits (the split plan depends on the sequence count)."""
        cache, tokens = self._geometry(), self.max_step_tokens
        return max(16, max(paged_workspace_bytes(self.q_dtype, cache, self.hq, n, tokens, self.max_context_len, 2, 0,
                                                 self.max_prefill_kv_tokens) for n in range(1, self.max_seqs + 1)))

    def GetWorkBufferRequest(self):
        return {"immutable_sizes": [], "mutable_sizes": [self._workspace_bytes]}

    def step_hints(self, num_tokens: int, num_seqs: int, prefill_row_blocks: int = 0, prefill_kv_tokens: int = 0):
        """The (prefill_row_blocks, prefill_kv_tokens) a step is launched with: a row-block hint can only tighten
        the reserved bound, a context hint beyond the scratch reserve switches to de-quantising inside the prefill
        kernel, and no context hint means the whole reserve."""
        if num_tokens == num_seqs:
            return 0, 0
        rb = prefill_row_blocks if 0 < prefill_row_blocks <= num_tokens // 128 + num_seqs else 0
        if prefill_kv_tokens > 0:
            kvt = prefill_kv_tokens if prefill_kv_tokens <= self.max_prefill_kv_tokens else 0
        else:
            kvt = self.max_prefill_kv_tokens
        return rb, kvt

    def Execute(self, inputs: Sequence, outputs: Sequence[torch.Tensor], workbuffers: Optional[dict] = None,
                stream=None, status: Optional[torch.Tensor] = None, prefill_row_blocks: int = 0,
                prefill_kv_tokens: int = 0):
        """Store this step's K/V rows, then attention into ``outputs[0]``.  A second output tensor (float32, flat)
        receives the node's score output - per sequence, the last query token's attention probabilities summed over
        the heads - and the int32 offsets of the sequences in it are returned (else None)."""
        if len(inputs) < 11 or len(outputs) < 1:
            raise ValueError("PagedAttentionExtension takes at least 11 inputs and 1 output")
        (query, key, value, k_cache, v_cache, past_lens, subsequence_begins, block_indices,
         block_indices_begins, scale, sliding_window) = inputs[:11]
        if len(inputs) > 11 and inputs[11] is not None and getattr(inputs[11], "numel", lambda: 0)() > 0:
            raise B2AError(7, "PagedAttentionOp: alibi slopes")
        # operands 9 and 10 are Constants of the model: they must agree with what the operator was built with
        sc, sw = _host_scalar(scale, "PagedAttentionExtension: scale"), _host_scalar(sliding_window, "sliding_window")
        if sc is not None and self.scale is not None and abs(float(sc) - self.scale) > 1e-6 * abs(self.scale):
            raise ValueError("PagedAttentionOp: the scale operand differs from the constant the operator was built with")
        if sw and int(sw) != self.sliding_window:
            raise ValueError("PagedAttentionOp: the sliding_window operand differs from the operator's constant")
        num_tokens, num_seqs = query.shape[0], past_lens.shape[0]
        if num_seqs > self.max_seqs or num_tokens > self.max_step_tokens or num_tokens < num_seqs:
            raise B2AError(8, "PagedAttentionOp: the step exceeds the capacity the operator was built for")
        cache = PagedKvCache(k_cache, v_cache, self.hkv, self.d, self.d, self.block_size, self.kv_dtype)
        max_q_len = num_tokens - num_seqs + 1  # every scheduled sequence has at least one token
        ws = workbuffers["mutable"][0] if workbuffers and workbuffers.get("mutable") else None
        if ws is None or ws.numel() * ws.element_size() < self._workspace_bytes:
            raise B2AError(5, "PagedAttentionOp: pass the work buffer GetWorkBufferRequest() asked for")
        rb, kvt = self.step_hints(num_tokens, num_seqs, prefill_row_blocks, prefill_kv_tokens)
        paged_kv_store(key, value, cache, past_lens, subsequence_begins, block_indices, block_indices_begins,
                       stream=stream, status=status)
        paged_attention(query, cache, past_lens, subsequence_begins, block_indices, block_indices_begins,
                        self.hq, self.max_context_len, max_q_len, self.scale if sc is None else float(sc),
                        self.sliding_window, out=outputs[0], workspace=ws, stream=stream,
                        status=status, prefill_row_blocks=rb, prefill_kv_tokens=kvt,
                        cache_rows_settled=True)  # the kernel before it is this step's store
        if len(outputs) > 1 and outputs[1] is not None:
            _, begins = paged_last_token_scores(query, cache, past_lens, subsequence_begins, block_indices,
                                                block_indices_begins, self.hq, self.max_context_len,
                                                self.scale if sc is None else float(sc), self.sliding_window,
                                                scores=outputs[1], stream=stream, status=status)
            return begins
        return None


# ------------------------------------------------------------------------------------------------------------
# KV block manager (host)
# ------------------------------------------------------------------------------------------------------------

class KvBlockManager:
    """Python face of the C++ ``b2a::KvBlockManager`` (free list + per-sequence block lists + step tables)."""

    def __init__(self, num_blocks: int, block_size: int = 16, shuffle_seed: int = 0):
        self._lib = _lib.load()
        self._h = C.c_void_p()
        check(self._lib.b2a_kvmgr_create(num_blocks, block_size, shuffle_seed, C.byref(self._h)), "b2a_kvmgr_create")
        self.num_blocks, self.block_size = num_blocks, block_size

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.b2a_kvmgr_destroy(self._h)
            self._h = None

    def add_sequence(self, seq_id: int) -> None:
        check(self._lib.b2a_kvmgr_add_sequence(self._h, seq_id), "b2a_kvmgr_add_sequence")

    def free_sequence(self, seq_id: int) -> None:
        check(self._lib.b2a_kvmgr_free_sequence(self._h, seq_id), "b2a_kvmgr_free_sequence")

    @property
    def free_blocks(self) -> int:
        return self._lib.b2a_kvmgr_free_blocks(self._h)

    def sequence_len(self, seq_id: int) -> int:
        return self._lib.b2a_kvmgr_sequence_len(self._h, seq_id)

    @property
    def last_prefill_kv_tokens(self) -> int:
        """``prefill_kv_tokens`` hint of the step scheduled last."""
        return self._lib.b2a_kvmgr_last_prefill_kv_tokens(self._h)

    @property
    def last_prefill_row_blocks(self) -> int:
        """``prefill_row_blocks`` hint of the step scheduled last."""
        return self._lib.b2a_kvmgr_last_prefill_row_blocks(self._h)

    def schedule_step(self, seq_ids: Sequence[int], q_lens: Sequence[int]):
        """Reserve blocks for the new tokens and return the step tables as numpy int32 arrays:
        (past_lens, subsequence_begins, block_indices, block_indices_begins, max_context_len)."""
        n = len(seq_ids)
        ids = (C.c_int64 * n)(*seq_ids)
        ql = (C.c_int32 * n)(*q_lens)
        cap = sum((max(self.sequence_len(s), 0) + q + self.block_size - 1) // self.block_size
                  for s, q in zip(seq_ids, q_lens)) + 1
        past = np.zeros(n, np.int32)
        sb = np.zeros(n + 1, np.int32)
        bi = np.zeros(cap, np.int32)
        bb = np.zeros(n + 1, np.int32)
        nbi, mctx = C.c_int32(0), C.c_int32(0)
        p = lambda a: a.ctypes.data_as(C.POINTER(C.c_int32))
        check(self._lib.b2a_kvmgr_schedule_step(self._h, ids, ql, n, p(past), p(sb), p(bi), cap, p(bb),
                                                C.byref(nbi), C.byref(mctx)), "b2a_kvmgr_schedule_step")
        return past, sb, bi[: nbi.value].copy(), bb, mctx.value
