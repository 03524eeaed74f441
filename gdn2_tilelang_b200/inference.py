"""Serving entry points: ``gdn2_prefill``, ``gdn2_decode``, ``gdn2_decode_step``.

Same signatures, shapes, dtype rules and state-ownership rules as the reference
(gdn2/inference.py:156-196, 306-353, 482-555 of the reference project):

* ``gdn2_decode`` / ``gdn2_decode_step`` update ``state`` in place and return ``o`` in ``v.dtype``;
* ``gdn2_prefill`` sends whole 64-token chunks through the chunkwise kernels (the fused scan never
  stores per-chunk states) and the ragged tail through the decode kernel, and returns the state as
  a new tensor -- except when the prompt is shorter than one chunk, where, as in the reference, the
  float32 contiguous ``state`` passed in is itself updated and returned.

All arithmetic runs in the CUDA kernels behind :mod:`gdn2_tilelang_b200._cabi`.
"""

from __future__ import annotations

import torch

from . import _cabi
from .config import DEFAULT_KERNEL_CONFIG, GDN2Config

__all__ = ["gdn2_prefill", "gdn2_decode", "gdn2_decode_step"]


def _check_inputs(q, k, v, g, b, w):
    if q.dim() != 4:
        raise ValueError(f"expected [B, S, H, D] tensors, got shape {tuple(q.shape)}")
    B, S, H, DK = q.shape
    DV = v.shape[-1]
    if k.shape != q.shape or b.shape != q.shape or g.shape != q.shape:
        raise ValueError("q, k, b and g must share the shape [B, S, H, DK]")
    if v.shape != (B, S, H, DV) or w.shape != v.shape:
        raise ValueError("v and w must share the shape [B, S, H, DV]")
    _cabi.dtype_code(q.dtype)
    if not (k.dtype == v.dtype == b.dtype == w.dtype == q.dtype):
        raise TypeError("q, k, v, b and w must share one dtype")
    return B, S, H, DK, DV


def gdn2_decode(q, k, v, g, b, w, state, scale=None):
    """Decode ``n`` tokens (``[B, n, H, D]``), updating ``state [B, H, DK, DV]`` in place.

    Returns ``o [B, n, H, DV]`` in ``v.dtype``. ``g`` is coerced to float32.
    """
    B, n, H, DK, DV = _check_inputs(q, k, v, g, b, w)
    scale = DK**-0.5 if scale is None else scale
    if state.shape != (B, H, DK, DV):
        raise ValueError(f"state must have shape {(B, H, DK, DV)}, got {tuple(state.shape)}")
    return _cabi.kernels().decode(q, k, v, g.float(), b, w, state, scale)


def gdn2_decode_step(q, k, v, g, b, w, state, scale=None):
    """One token with ``[B, H, D]``-shaped inputs; ``state`` is updated in place. Returns ``[B, H, DV]``."""
    if q.dim() != 3:
        raise ValueError(f"expected [B, H, D] tensors, got shape {tuple(q.shape)}")
    o = gdn2_decode(*(t.unsqueeze(1) for t in (q, k, v, g, b, w)), state, scale)
    return o[:, 0]


@torch.no_grad()
def gdn2_prefill(q, k, v, g, b, w, state=None, scale=None, config: GDN2Config = DEFAULT_KERNEL_CONFIG):
    """Prefill a prompt. Returns ``(o [B, S, H, DV] in v.dtype, state [B, H, DK, DV] float32)``.

    Pass the returned state back in to prefill a long prompt in segments.
    """
    config.validate()
    B, S, H, DK, DV = _check_inputs(q, k, v, g, b, w)
    BS = config.chunk_size
    scale = DK**-0.5 if scale is None else scale
    n_full = (S // BS) * BS
    K = _cabi.kernels()
    g = g.float()
    if state is None:
        state = torch.zeros(B, H, DK, DV, dtype=config.state_dtype, device=q.device)
    else:
        if state.shape != (B, H, DK, DV):
            raise ValueError(f"state must have shape {(B, H, DK, DV)}, got {tuple(state.shape)}")
        state = state.to(config.state_dtype).contiguous()

    o = torch.empty(B, S, H, DV, dtype=v.dtype, device=q.device)
    if n_full:
        _, state, _ = K.chunk_forward(*(t[:, :n_full] for t in (q, k, v, g, b, w)), scale, state,
                                      out=o, out_batch_stride=S)
    if S > n_full:
        K.decode(*(t[:, n_full:] for t in (q, k, v, g, b, w)), state, scale, out=o[:, n_full:])
    return o, state
