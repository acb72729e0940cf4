"""B200-native attention path for OpenVINO's nvidia_plugin: ScaledDotProductAttention and
PagedAttentionExtension as hand-written sm_100a CUDA behind a C ABI (include/b2a.h), with the host-side
mirror of the plugin's operator interface in ``openvino_contrib_b200/host`` (C++) and ``ops`` (Python)."""
from . import _lib
from ._lib import B2AError
from .ops import (HostSdpaPipeline, KvBlockManager, PagedAttentionOp, PagedKvCache, SdpaOp, paged_attention,
                  paged_kv_store, paged_last_token_scores, sdpa)

__all__ = ["_lib", "B2AError", "sdpa", "HostSdpaPipeline", "paged_kv_store", "paged_attention", "paged_last_token_scores", "SdpaOp", "PagedAttentionOp", "PagedKvCache",
           "KvBlockManager"]
