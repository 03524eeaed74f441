"""Gated DeltaNet-2 forward and serving kernels for NVIDIA B200 (sm_100a).

Drop-in for the forward / serving API of the reference ``gdn2`` package:

    from gdn2_tilelang_b200 import GatedDeltaNet2, GatedDeltaNet2Config, gdn2_attention

    config.py           GDN2Config, GatedDeltaNet2Config (same fields as the reference)
    attention.py        gdn2_attention(), GatedDeltaNet2, GDN2Cache, GraphedStep, resolve_backend
    forward.py          chunk_gdn2_fwd (chunk-local stage + fused scan/output, optional chunk states)
    inference.py        gdn2_prefill, gdn2_prefill_from_host, gdn2_decode, gdn2_decode_step
    tensor_parallel.py  head-parallel layer with one all-reduce after o_proj
    _cabi.py            ctypes binding of libgdn2_b200.so (include/gdn2_b200.h)
    csrc/               the CUDA kernels and the C ABI
"""

from .attention import GDN2Cache, GatedDeltaNet2, GraphedStep, gdn2_attention, resolve_backend
from .config import GDN2Config, GatedDeltaNet2Config
from .forward import chunk_gdn2_fwd, chunk_gdn2_output
from .inference import gdn2_decode, gdn2_decode_step, gdn2_prefill, gdn2_prefill_from_host
from .tensor_parallel import TensorParallelGatedDeltaNet2, shard_config, shard_state_dict

__all__ = [
    "GatedDeltaNet2", "GatedDeltaNet2Config", "GDN2Cache",
    "GraphedStep", "gdn2_attention", "gdn2_prefill", "gdn2_prefill_from_host", "gdn2_decode", "gdn2_decode_step", "GDN2Config",
    "chunk_gdn2_fwd", "chunk_gdn2_output", "resolve_backend",
    "TensorParallelGatedDeltaNet2", "shard_config", "shard_state_dict",
]
