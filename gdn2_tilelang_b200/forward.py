"""Training-style chunkwise forward driver: ``chunk_gdn2_fwd``.

Mirrors the reference driver (gdn2/forward.py:832-899 of the reference project): the chunk-local
stage, then the state scan, then the output. Here the scan and the output are one fused kernel
that can also store the state entering every chunk (``return_chunk_states=True``), which is what
the reference's ``state_kernel`` materialises as ``h [B, NC, H, DK, DV]``; they are kept in
float32. A sequence length that is not a multiple of 64 is not padded: the ragged tail runs
through the recurrent decode kernel, which is arithmetically the same recurrence.
"""

from __future__ import annotations

import torch

from . import _cabi
from .config import DEFAULT_KERNEL_CONFIG, GDN2Config
from .inference import _check_inputs

__all__ = ["chunk_gdn2_fwd", "chunk_gdn2_output"]


@torch.no_grad()
def chunk_gdn2_fwd(q, k, v, g, b, w, scale, initial_state=None, output_final_state=False,
                   config: GDN2Config = DEFAULT_KERNEL_CONFIG, return_chunk_states=False, out=None):
    """Returns ``(o, final_state | None)`` or, with ``return_chunk_states``, ``(o, final_state | None, h)``.

    ``o`` is ``[B, S, H, DV]`` in the input dtype, ``final_state`` ``[B, H, DK, DV]`` float32,
    ``h`` ``[B, S // 64, H, DK, DV]`` float32 (whole chunks only). ``out`` (optional) is a ``[B, S, H, DV]``
    tensor or view with dense ``[S, H, DV]`` blocks that receives ``o`` (a slice of a packed batch, for instance).
    """
    config.validate()
    B, S, H, DK, DV = _check_inputs(q, k, v, g, b, w)
    BS = config.chunk_size
    n_full = (S // BS) * BS
    K = _cabi.kernels()
    g = g.float()
    if out is None:
        o = torch.empty(B, S, H, DV, dtype=v.dtype, device=q.device)
    else:
        if tuple(out.shape) != (B, S, H, DV) or out.dtype != v.dtype or out.stride(3) != 1 or out.stride(2) != DV \
                or out.stride(1) != H * DV or (B > 1 and out.stride(0) % (H * DV)):
            raise ValueError("`out` must be [B, S, H, DV] in v's dtype with dense [S, H, DV] blocks")
        o = out
    o_bs = S if (out is None or B == 1) else out.stride(0) // (H * DV)
    state, hs = initial_state, None
    if state is not None and state.shape != (B, H, DK, DV):
        raise ValueError(f"initial_state must have shape {(B, H, DK, DV)}, got {tuple(state.shape)}")
    def tail(st):                                     # the ragged tail through the decode kernel, state in place
        K.decode(*(t[:, n_full:] for t in (q, k, v, g, b, w)), st, scale, out=o[:, n_full:])

    if n_full:
        # the tail needs the final state only: a cut scan lets it run beside its correction pass
        _, state, hs = K.chunk_forward(*(t[:, :n_full] for t in (q, k, v, g, b, w)), scale, state,
                                       want_chunk_states=return_chunk_states, out=o, out_batch_stride=o_bs,
                                       then_with_state=tail if S > n_full else None)
    elif S > n_full:
        if state is None:
            state = torch.zeros(B, H, DK, DV, dtype=torch.float32, device=q.device)
        else:
            state = state.to(torch.float32).clone()   # never write into the caller's initial state
        tail(state)
    K.maybe_check_device_status(q.device)
    final = state if output_final_state else None
    return (o, final, hs) if return_chunk_states else (o, final)


@torch.no_grad()
def chunk_gdn2_output(q, k, v, g, b, w, scale, chunk_states, config: GDN2Config = DEFAULT_KERNEL_CONFIG):
    """Chunk-parallel output from stored chunk states ``h`` (the reference's ``output_kernel`` stage,
    gdn2/forward.py:644-727). ``S`` must be a multiple of 64. Returns ``o [B, S, H, DV]``."""
    config.validate()
    _check_inputs(q, k, v, g, b, w)
    return _cabi.kernels().chunk_output(q, k, v, g.float(), b, w, scale, chunk_states)
