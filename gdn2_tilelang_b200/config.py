"""Configuration objects, field-for-field those of the reference project
(gdn2/config.py:22-89) so existing call sites and config files keep working.

``GDN2Config`` describes how the kernels are run. The tile-shape knobs of the
reference's TileLang kernels (``sub_chunk_size``, ``block_DK``, ``block_DV``,
``threads``, ``num_stages``) are accepted and ignored: the CUDA kernels here fix
their own tiling. ``chunk_size`` must be 64 and ``state_dtype`` float32.
``GatedDeltaNet2Config`` describes the layer.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

__all__ = ["GDN2Config", "GatedDeltaNet2Config", "DEFAULT_KERNEL_CONFIG"]


@dataclass(frozen=True)
class GDN2Config:
    chunk_size: int = 64
    sub_chunk_size: int = 16
    block_DK: int = 64
    block_DV: int = 64
    threads: int = 128
    num_stages: int = 2
    state_dtype: torch.dtype = torch.float32
    backend: str = "auto"
    backward: str = "tilelang"

    def validate(self) -> None:
        """Raise for settings the CUDA kernels do not implement."""
        if self.chunk_size != 64:
            raise ValueError(f"chunk_size must be 64 for the sm_100a kernels, got {self.chunk_size}")
        if self.state_dtype != torch.float32:
            raise ValueError(f"state_dtype must be torch.float32, got {self.state_dtype}")


DEFAULT_KERNEL_CONFIG = GDN2Config()


@dataclass
class GatedDeltaNet2Config:
    """Layer hyper-parameters (same names, defaults and meaning as the reference).

    ``num_heads`` counts value heads, ``num_kv_heads`` key heads (must divide
    ``num_heads``); ``erase_gate_scale`` bounds the erase gate ``b``;
    ``a_init_range`` / ``dt_init_range`` initialise the decay parameterisation
    ``g = -exp(A_log) * softplus(f_proj(x) + dt_bias)``.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int | None = None
    head_dim_k: int = 128
    head_dim_v: int | None = None
    conv_size: int = 4
    norm_eps: float = 1e-5
    erase_gate_scale: float = 1.0
    a_init_range: tuple[float, float] = (1.0, 16.0)
    dt_init_range: tuple[float, float] = (0.001, 0.1)
    kernel: GDN2Config = field(default_factory=GDN2Config)
