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

__all__ = ["gdn2_prefill", "gdn2_prefill_from_host", "gdn2_decode", "gdn2_decode_step"]


def _check_inputs(q, k, v, g, b, w):
    """Shapes and dtypes. ``q, k, b, g`` may carry fewer heads than ``v, w`` (``HK`` key heads, ``H`` a multiple
    of it): value head ``h`` then reads key head ``h // (H // HK)``, which is what the reference's layer gets by
    ``repeat_interleave`` (gdn2/attention.py:295-297) before calling the op; here nothing is repeated."""
    if q.dim() != 4 or v.dim() != 4:
        raise ValueError(f"expected [B, S, H, D] tensors, got shapes {tuple(q.shape)} and {tuple(v.shape)}")
    B, S, HK, DK = q.shape
    H, DV = v.shape[2], v.shape[-1]
    if k.shape != q.shape or b.shape != q.shape or g.shape != q.shape:
        raise ValueError("q, k, b and g must share the shape [B, S, HK, DK]")
    if v.shape != (B, S, H, DV) or w.shape != v.shape:
        raise ValueError("v and w must share the shape [B, S, H, DV]")
    if HK < 1 or H % HK:
        raise ValueError(f"the {H} value heads must be a multiple of the {HK} key heads")
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
    K = _cabi.kernels()
    o = K.decode(q, k, v, g.float(), b, w, state, scale)
    K.maybe_check_device_status(q.device)
    return o


def gdn2_decode_step(q, k, v, g, b, w, state, scale=None):
    """One token with ``[B, H, D]``-shaped inputs; ``state`` is updated in place. Returns ``[B, H, DV]``."""
    if q.dim() != 3:
        raise ValueError(f"expected [B, H, D] tensors, got shape {tuple(q.shape)}")
    o = gdn2_decode(*(t.unsqueeze(1) for t in (q, k, v, g, b, w)), state, scale)
    return o[:, 0]


@torch.no_grad()
def gdn2_prefill(q, k, v, g, b, w, state=None, scale=None, config: GDN2Config = DEFAULT_KERNEL_CONFIG,
                 gated_norm=None):
    """Prefill a prompt. Returns ``(o [B, S, H, DV] in v.dtype, state [B, H, DK, DV] float32)``.

    Pass the returned state back in to prefill a long prompt in segments.

    ``gated_norm = (gate, gate_column, weight, eps)`` (no counterpart in the reference's signature; used by the
    layer): the rows of the WHOLE chunks come out as ``rmsnorm(o) * weight * silu(gate)`` (see
    ``NativeKernels.chunk_forward``); the rows of a ragged tail are left plain for the caller to finish.
    """
    config.validate()
    B, S, H, DK, DV = _check_inputs(q, k, v, g, b, w)
    BS = config.chunk_size
    scale = DK**-0.5 if scale is None else scale
    n_full = (S // BS) * BS
    K = _cabi.kernels()
    g = g.float()
    if state is None:
        if n_full == 0:                                    # the chunkwise kernels take "no state" as zeros themselves
            state = torch.zeros(B, H, DK, DV, dtype=config.state_dtype, device=q.device)
    else:
        if state.shape != (B, H, DK, DV):
            raise ValueError(f"state must have shape {(B, H, DK, DV)}, got {tuple(state.shape)}")
        state = state.to(config.state_dtype).contiguous()

    if gated_norm is None and n_full:
        res = K.prefill_ragged(q, k, v, g, b, w, scale, state)      # the whole call in the library, where it applies
        if res is not None:
            K.maybe_check_device_status(q.device)
            return res

    o = torch.empty(B, S, H, DV, dtype=v.dtype, device=q.device)

    def tail(st):                                          # the ragged tail through the decode kernel, state in place
        K.decode(*(t[:, n_full:] for t in (q, k, v, g, b, w)), st, scale, out=o[:, n_full:])

    if n_full:
        # the tail needs the final state only: a cut scan lets it run beside its correction pass
        _, state, _ = K.chunk_forward(*(t[:, :n_full] for t in (q, k, v, g, b, w)), scale, state,
                                      out=o, out_batch_stride=S, gated_norm=gated_norm,
                                      then_with_state=tail if S > n_full else None)
    elif S > n_full:
        tail(state)
    K.maybe_check_device_status(q.device)
    return o, state


@torch.no_grad()
def gdn2_prefill_from_host(q, k, v, g, b, w, state=None, scale=None, config: GDN2Config = DEFAULT_KERNEL_CONFIG,
                           device=None, out=None):
    """``gdn2_prefill`` for prompts whose tensors live in host memory (pinned, for the copies to be
    asynchronous). No counterpart in the reference, whose callers upload first and call ``gdn2_prefill``.

    The batch is streamed one sequence (long sequences: a quarter of one) at a time through double-buffered
    device inputs: the upload of unit i + 1 and the download of the outputs of unit i - 1 run on their own
    CUDA streams while unit i is computed, so the call costs about as much as its host-to-device traffic alone instead
    of upload + kernels + download one after the other. Sequences are independent, so the results are
    those of one ``gdn2_prefill`` over the whole batch.

    Returns ``(o, state)``: ``o`` [B, S, H, DV] in host memory (``out`` if given, else a new pinned
    tensor), complete when the current stream reaches the end of this call; ``state`` [B, H, DK, DV]
    float32 on the device. ``state`` (initial, optional) may live on either side.
    """
    config.validate()
    B, S, H, DK, DV = _check_inputs(q, k, v, g, b, w)
    dev = torch.device(device if device is not None else "cuda")
    if dev.type != "cuda":                                 # host-logic tests: nothing to overlap
        o, st = gdn2_prefill(q, k, v, g, b, w, state, scale, config)
        if out is not None:
            out.copy_(o)
            o = out
        return o, st
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    ins = (q, k, v, g, b, w)
    if out is None:
        out = torch.empty(B, S, H, DV, dtype=v.dtype).pin_memory()
    elif out.shape != (B, S, H, DV) or out.dtype != v.dtype or out.device.type != "cpu":
        raise ValueError("out must be a host tensor of shape [B, S, H, DV] in v.dtype")
    if state is not None and state.shape != (B, H, DK, DV):
        raise ValueError(f"state must have shape {(B, H, DK, DV)}, got {tuple(state.shape)}")

    with torch.cuda.device(dev):
        main = torch.cuda.current_stream(dev)
        up, down = _transfer_streams(dev)
        # pipeline units: (sequence, token range), ranges cut at multiples of the chunk size so that the
        # state chains from one unit of a sequence to the next; long sequences are cut so that the last
        # unit's compute and download, which nothing overlaps, are short
        BS = config.chunk_size
        pieces = max(1, min(4, S // (64 * BS)))
        step = -(-S // pieces)
        step = -(-step // BS) * BS
        bounds = [(lo, min(S, lo + step)) for lo in range(0, S, step)]
        units = [(i, lo, hi) for i in range(B) for lo, hi in bounds]
        U = len(units)
        slots = [[torch.empty((1, step) + tuple(t.shape[2:]), dtype=t.dtype, device=dev) for t in ins] for _ in range(2)]
        state_out = torch.empty(B, H, DK, DV, dtype=config.state_dtype, device=dev)
        if state is not None:
            state_out.copy_(state, non_blocking=True)
        uploaded = [torch.cuda.Event() for _ in range(U)]
        consumed = [torch.cuda.Event() for _ in range(U)]      # unit u's input slot may be overwritten
        outputs = []                                            # device outputs stay alive until the call ends
        up.wait_stream(main)                                    # the buffers above exist before anything lands in them
        down.wait_stream(main)

        def upload(u):
            i, lo, hi = units[u]
            with torch.cuda.stream(up):
                if u >= 2:
                    up.wait_event(consumed[u - 2])
                for d, h in zip(slots[u & 1], ins):
                    d[:, :hi - lo].copy_(h[i:i + 1, lo:hi], non_blocking=True)
                uploaded[u].record(up)

        upload(0)
        for u, (i, lo, hi) in enumerate(units):
            if u + 1 < U:
                upload(u + 1)
            main.wait_event(uploaded[u])
            st_in = state_out[i:i + 1] if (state is not None or lo > 0) else None
            o_u, st_u = gdn2_prefill(*(t[:, :hi - lo] for t in slots[u & 1]), st_in, scale, config)
            outputs.append(o_u)
            state_out[i:i + 1].copy_(st_u)
            consumed[u].record(main)
            with torch.cuda.stream(down):
                down.wait_event(consumed[u])
                out[i:i + 1, lo:hi].copy_(o_u, non_blocking=True)
        main.wait_stream(down)
        main.wait_stream(up)
    return out, state_out


_TRANSFER_STREAMS: dict = {}


def _transfer_streams(dev):
    key = (dev.type, dev.index)
    if key not in _TRANSFER_STREAMS:
        _TRANSFER_STREAMS[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _TRANSFER_STREAMS[key]
