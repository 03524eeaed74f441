"""ctypes binding of ``libgdn2_b200.so`` (declared in ``include/gdn2_b200.h``).

The library is the product: there is no other implementation behind these
functions. If it is missing, cannot be built, or no CUDA device is present, the
calls raise -- nothing falls back to the host.

``NativeKernels`` is the one object the host-side API talks to; it turns torch
tensors into raw pointers, sizes and the current CUDA stream.
"""

from __future__ import annotations

import ctypes
import os
import pathlib
import threading

import torch

_PKG = pathlib.Path(__file__).resolve().parent
_LIB_PATH = _PKG / "libgdn2_b200.so"

GDN2_F32, GDN2_BF16, GDN2_F16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TCGEN05, PATH_TCGEN05_SERIAL = 0, 1, 2, 3
_PATHS = {"auto": PATH_AUTO, "simt": PATH_SIMT, "tcgen05": PATH_TCGEN05, "tcgen05_serial": PATH_TCGEN05_SERIAL}
CHUNK = 64

_DTYPES = {torch.float32: GDN2_F32, torch.bfloat16: GDN2_BF16, torch.float16: GDN2_F16}

_vp, _i64, _f32, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_int, ctypes.c_size_t

# name -> (restype, argtypes); every symbol include/gdn2_b200.h declares
SIGNATURES = {
    "gdn2_abi_version": (_int, []),
    "gdn2_status_string": (ctypes.c_char_p, [_int]),
    "gdn2_last_cuda_error": (_int, []),
    "gdn2_decode": (_int, [_vp] * 8 + [_i64] * 8 + [_f32, _int, _vp]),
    "gdn2_prefill_workspace_bytes": (_sz, [_i64] * 6 + [_int, _int]),
    "gdn2_prefill_scan_segments": (_int, [_i64] * 5 + [_int, _int]),
    "gdn2_prefill_scan_launches": (_int, [_i64] * 5 + [_int, _int]),
    "gdn2_prefill_scan_part": (_int, [_vp, _sz, _vp, _vp, _vp] + [_i64] * 7 + [_int, _int, _int, _vp]),
    "gdn2_prefill_ragged": (_int, [_vp] * 10 + [_sz] + [_i64] * 8 + [_f32, _int, _int, _vp, _vp]),
    "gdn2_prefill_workspace_layout": (_int, [_i64] * 6 + [_int, _int, ctypes.POINTER(ctypes.c_int64)]),
    "gdn2_chunk_prep": (_int, [_vp] * 7 + [_sz] + [_i64] * 7 + [_f32, _int, _int, _vp]),
    "gdn2_prefill_scan": (_int, [_vp, _sz, _vp, _vp, _vp, _vp] + [_i64] * 7 + [_int, _int, _vp]),
    "gdn2_chunk_output": (_int, [_vp, _sz, _vp, _vp] + [_i64] * 7 + [_int, _int, _vp]),
    "gdn2_prefill_scan_gated_norm": (_int, [_vp, _sz, _vp, _vp, _vp] + [_i64] * 7 + [_int, _int, _vp, _vp]),
    "gdn2_check_device_status": (_int, [_vp, ctypes.POINTER(ctypes.c_uint32)]),
    "gdn2_selftest_mma": (_int, [_vp, _vp, _vp, _vp]),
    "gdn2_selftest_wait": (_int, [_i64, _vp, _vp]),
    "gdn2_prefill_static": (_int, [_vp] * 9 + [_i64] * 7 + [_f32, _int, _vp]),
    "gdn2_layer_front": (_int, [_vp, _int, _vp]),
    "gdn2_oproj_reduce_buffer_bytes": (_sz, [_i64, _i64, ctypes.POINTER(_sz)]),
    "gdn2_oproj_reduce": (_int, [_vp, _int, _vp]),
    "gdn2_layer_back": (_int, [_vp] * 4 + [_i64] * 5 + [_f32, _int, _vp]),
}


class LayerFrontArgs(ctypes.Structure):
    """``gdn2_layer_front_args`` of include/gdn2_b200.h."""

    _fields_ = ([(n, _vp) for n in ("proj", "conv_state", "conv_weight", "conv_bias", "A_log", "dt_bias",
                                    "q", "k", "v", "g", "b", "w", "new_conv_state")]
                + [(n, _i64) for n in ("B", "S", "H", "HK", "DK", "DV", "K", "NP",
                                       "off_q", "off_k", "off_v", "off_b", "off_w", "off_f")]
                + [("erase_scale", _f32)])

class GatedNormArgs(ctypes.Structure):
    """``gdn2_gated_norm`` of include/gdn2_b200.h."""

    _fields_ = [("gate", _vp), ("weight", _vp), ("gate_row_stride", _i64), ("gate_batch_stride", _i64), ("eps", _f32)]


class OProjReduceArgs(ctypes.Structure):
    """``gdn2_oproj_reduce_args`` of include/gdn2_b200.h."""

    _fields_ = ([(n, _vp) for n in ("x", "weight", "out", "peer_slots", "peer_flags", "epochs")]
                + [(n, _i64) for n in ("rows", "K", "hidden")] + [("rank", _int), ("world", _int), ("wait_cycles", _i64)])


_lock = threading.Lock()
_lib = None


class GDN2KernelError(RuntimeError):
    """A C-ABI call returned a negative status."""


def library_path() -> pathlib.Path:
    return _LIB_PATH


def load_library(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load (building in-tree first if needed) the shared library and bind every symbol."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            if not build_if_missing:
                raise GDN2KernelError(f"{_LIB_PATH} is missing; run `python -m gdn2_tilelang_b200.build`")
            from . import build as _build

            _build.build()
        lib = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = lib
        return lib


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; use float16, bfloat16 or float32") from None


def _check(lib, status: int, what: str):
    if status != 0:
        msg = lib.gdn2_status_string(status).decode()
        extra = f" (cudaError {lib.gdn2_last_cuda_error()})" if status == -6 else ""
        raise GDN2KernelError(f"{what}: {msg}{extra} [status {status}]")


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and t.device.type != "cuda":
            raise ValueError(
                "gdn2_tilelang_b200 runs on CUDA devices only (no host implementation is shipped); "
                f"got a tensor on {t.device}"
            )


class _on_device:
    """``with _on_device(dev):`` makes ``dev`` the current CUDA device for the C calls inside, like
    ``torch.cuda.device`` but without touching the driver when it already is (the usual case, and these calls sit
    on paths where a microsecond of host time counts)."""

    __slots__ = ("idx", "prev")

    def __init__(self, dev):
        dev = torch.device(dev) if not isinstance(dev, torch.device) else dev
        self.idx, self.prev = dev.index, -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and cur != self.idx:
            torch.cuda.set_device(self.idx)
            self.prev = cur

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _seq_view(t: torch.Tensor):
    """(tensor, batch stride in tokens) for a ``[B,S,H,D]`` tensor whose ``[S,H,D]`` block is dense.

    A slice ``x[:, a:b]`` of a contiguous tensor qualifies and is passed through without a copy.
    """
    B, S, H, D = t.shape
    if t.stride(3) == 1 and t.stride(2) == D and t.stride(1) == H * D and (B == 1 or t.stride(0) % (H * D) == 0):
        if t.data_ptr() % 16 == 0:
            return t, (t.stride(0) // (H * D) if B > 1 else S)
    t = t.contiguous()
    return t, S


class NativeKernels:
    """Launches the CUDA kernels through the C ABI on the current stream of the tensors' device."""

    def __init__(self):
        self.lib = load_library()
        self.prefill_path = _PATHS[os.environ.get("GDN2_B200_PREFILL_PATH", "auto")]
        self.launches = 0   # kernels launched through this object (for the benchmark's accounting)
        self._side_streams = {}

    # -- helpers ---------------------------------------------------------------------------
    @staticmethod
    def _stream(t: torch.Tensor) -> int:
        return torch.cuda.current_stream(t.device).cuda_stream

    def resolved_path(self, DK: int, DV: int, dtype: torch.dtype, path=None) -> int:
        p = self.prefill_path if path is None else _PATHS[path] if isinstance(path, str) else path
        if p == PATH_AUTO:
            p = PATH_TCGEN05 if (DK == 128 and DV == 128 and dtype == torch.bfloat16) else PATH_SIMT
        return p

    def scan_segments(self, B, S, H, DK, DV, dtype, path) -> int:
        """Sequence segments the scan kernel itself cuts this problem into (1 = one block per (batch, head))."""
        return self.lib.gdn2_prefill_scan_segments(B, S, H, DK, DV, dtype_code(dtype), path)

    def _segments(self, B, S, H, DK, DV, dtype, path: int) -> int:
        """How many sequence segments the host cuts the chunkwise prefill into so that the chunk-local stage
        of one segment overlaps the scan of the previous one (1 = no cut). Only worth it while the scan runs
        one block per (batch, head) and leaves SMs idle; a scan that cuts the sequence itself fills the GPU."""
        if path not in (PATH_TCGEN05, PATH_TCGEN05_SERIAL):
            return 1
        if self.scan_segments(B, S, H, DK, DV, dtype, path) > 1:
            return 1
        want = int(os.environ.get("GDN2_B200_PREFILL_SEGMENTS", "2"))
        return max(1, min(want, (S // CHUNK) // 16))

    def _side_stream(self, dev):
        key = (dev.type, dev.index)
        st = self._side_streams.get(key)
        if st is None:
            st = self._side_streams[key] = torch.cuda.Stream(device=dev, priority=-1)
        return st

    # -- decode ----------------------------------------------------------------------------
    def decode(self, q, k, v, g, b, w, state, scale: float, out=None) -> torch.Tensor:
        """``[B,n,H,D]`` tokens, ``state [B,H,DK,DV]`` fp32 contiguous, updated in place. Returns ``o``.

        ``out`` may be a ``[B,n,H,DV]`` view into a longer preallocated sequence tensor.
        """
        _require_cuda(q, k, v, g, b, w, state)
        B, n, HK, DK = q.shape
        H, DV = v.shape[2], v.shape[-1]
        code = dtype_code(q.dtype)
        if state.dtype != torch.float32 or not state.is_contiguous():
            raise ValueError("the recurrent state must be a contiguous float32 tensor")
        views = [_seq_view(t) for t in (q, k, v, g, b, w)]
        strides = {s for _, s in views}
        if len(strides) != 1:
            views = [(t.contiguous(), n) for t, _ in views]
        in_bs = views[0][1]
        q, k, v, g, b, w = (t for t, _ in views)
        if out is None:
            o, o_bs = torch.empty(B, n, H, DV, dtype=v.dtype, device=v.device), n
        else:
            o, o_bs = _seq_view(out)
            if o is not out or out.dtype != v.dtype or tuple(out.shape) != (B, n, H, DV):
                raise ValueError("`out` must be a [B,n,H,DV] view with dense [n,H,DV] blocks in v's dtype")
        with _on_device(q.device):
            rc = self.lib.gdn2_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                      w.data_ptr(), state.data_ptr(), o.data_ptr(), B, n, H, HK, DK, DV, in_bs, o_bs,
                                      float(scale), code, self._stream(q))
        _check(self.lib, rc, "gdn2_decode")
        self.launches += 1
        return o

    # -- prefill in one call ---------------------------------------------------------------
    def prefill_ragged(self, q, k, v, g, b, w, scale: float, initial_state=None):
        """``gdn2_prefill`` as ONE library call (``gdn2_prefill_ragged``): chunk-local stage and scan on the whole
        chunks, decode on the ragged tail, the tail beside the scan's correction pass when the scan is cut.
        Returns ``(o, final_state)`` or ``None`` when this form does not apply (fewer than 64 tokens; a problem
        whose two stages the host overlaps segment by segment) and the caller composes the stages itself."""
        _require_cuda(q, k, v, g, b, w, initial_state)
        B, S, HK, DK = q.shape
        H, DV = v.shape[2], v.shape[-1]
        n_full = S // CHUNK * CHUNK
        if n_full == 0:
            return None
        code = dtype_code(q.dtype)
        p = self.resolved_path(DK, DV, q.dtype, None)
        if self._segments(B, n_full, H, DK, DV, q.dtype, p) > 1:
            return None
        views = [_seq_view(t) for t in (q, k, v, g, b, w)]
        if len({s_ for _, s_ in views}) != 1:
            views = [(t.contiguous(), S) for t, _ in views]
        in_bs = views[0][1]
        q, k, v, g, b, w = (t for t, _ in views)
        dev = q.device
        nbytes = self.lib.gdn2_prefill_workspace_bytes(B, n_full, H, HK, DK, DV, code, p)
        if nbytes == 0:
            raise GDN2KernelError(
                f"no kernel for DK={DK}, DV={DV}, dtype={q.dtype} (SIMT family: DK<=128, DK%8==0, DV%4==0)")
        if initial_state is not None and (initial_state.dtype != torch.float32 or not initial_state.is_contiguous()):
            initial_state = initial_state.to(torch.float32).contiguous()
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        o = torch.empty(B, S, H, DV, dtype=v.dtype, device=dev)
        final_state = torch.empty(B, H, DK, DV, dtype=torch.float32, device=dev)
        with _on_device(dev):
            main = torch.cuda.current_stream(dev)
            side = self._side_stream(dev) if S > n_full else None
            rc = self.lib.gdn2_prefill_ragged(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(), w.data_ptr(),
                None if initial_state is None else initial_state.data_ptr(), o.data_ptr(), final_state.data_ptr(),
                ws.data_ptr(), nbytes, B, S, H, HK, DK, DV, in_bs, S, float(scale), code, p,
                None if side is None else side.cuda_stream, main.cuda_stream)
        _check(self.lib, rc, "gdn2_prefill_ragged")
        self.launches += (2 if p != PATH_SIMT else 1) + self.lib.gdn2_prefill_scan_launches(B, n_full, H, DK, DV, code, p) \
            + (1 if S > n_full else 0)
        return o, final_state

    # -- chunkwise forward -----------------------------------------------------------------
    def fuses_gated_norm(self, DK: int, DV: int, dtype: torch.dtype) -> bool:
        """Whether ``chunk_forward`` can apply the layer's gated RMSNorm as the scan's epilogue for this shape."""
        return self.resolved_path(DK, DV, dtype) in (PATH_TCGEN05, PATH_TCGEN05_SERIAL)

    def chunk_forward(self, q, k, v, g, b, w, scale: float, initial_state=None, want_chunk_states=False,
                      path=None, out=None, out_batch_stride=None, gated_norm=None, then_with_state=None):
        """Whole chunks only (``S % 64 == 0``). Returns ``(o, final_state, chunk_states | None)``.

        ``then_with_state``: a callable ``f(final_state)`` for work that needs only the final state (the decode
        of a ragged tail, which updates it in place and writes other rows of ``out``). It is always called, after
        the scan; when the scan runs as a cut scan it is called on a side stream between the scan's two parts
        (``gdn2_prefill_scan_part``), so that it runs beside the correction pass, and the caller's stream waits
        for it before this method returns.

        ``out`` may be a preallocated ``[B, S_total >= S, H, DV]`` tensor whose first ``S`` tokens
        per batch entry receive the result (``out_batch_stride`` = its token stride).
        ``gated_norm = (gate, gate_column, weight, eps)`` (tensor-core family only): the rows written are
        ``rmsnorm(o) * weight * silu(gate)`` with the gate of ``o[b, t, h, c]`` read from
        ``gate[b, t, gate_column + h*DV + c]`` (``gate``: a contiguous ``[B, >= S, NP]`` buffer, e.g. the
        layer's projection buffer); the plain ``o`` is then never written.
        """
        _require_cuda(q, k, v, g, b, w, initial_state)
        B, S, HK, DK = q.shape
        H, DV = v.shape[2], v.shape[-1]
        if S % CHUNK:
            raise ValueError(f"sequence length {S} must be a multiple of {CHUNK}")
        code = dtype_code(q.dtype)
        p = self.resolved_path(DK, DV, q.dtype, path)
        views = [_seq_view(t) for t in (q, k, v, g, b, w)]
        if len({s for _, s in views}) != 1:
            views = [(t.contiguous(), S) for t, _ in views]
        in_bs = views[0][1]
        q, k, v, g, b, w = (t for t, _ in views)
        dev = q.device
        nbytes = self.lib.gdn2_prefill_workspace_bytes(B, S, H, HK, DK, DV, code, p)
        if nbytes == 0:
            raise GDN2KernelError(
                f"no kernel for DK={DK}, DV={DV}, dtype={q.dtype} (SIMT family: DK<=128, DK%8==0, DV%4==0)")
        if out is None:
            out = torch.empty(B, S, H, DV, dtype=v.dtype, device=dev)
            out_batch_stride = S
        final_state = torch.empty(B, H, DK, DV, dtype=torch.float32, device=dev)
        hs = torch.empty(B, S // CHUNK, H, DK, DV, dtype=torch.float32, device=dev) if want_chunk_states else None
        if initial_state is not None:
            if initial_state.dtype != torch.float32 or not initial_state.is_contiguous():
                initial_state = initial_state.to(torch.float32).contiguous()
        NC = S // CHUNK
        nseg = 1 if want_chunk_states else self._segments(B, S, H, DK, DV, q.dtype, p)
        esz = out.element_size()
        with _on_device(dev):
            main = torch.cuda.current_stream(dev)
            # The scan runs on only B*H thread blocks and is bound by its chunk-to-chunk chain, while the
            # chunk-local stage is chunk-parallel. With several segments, the chunk-local stage of segment i+1
            # runs on the caller's stream while the scan of segment i runs on a high-priority side stream.
            bounds = [NC * i // nseg for i in range(nseg + 1)]
            states = [torch.empty_like(final_state) for _ in range(nseg - 1)] + [final_state]
            side = None
            if nseg > 1:
                side = self._side_stream(dev)
                side.wait_stream(main)
            state_ptr = None if initial_state is None else initial_state.data_ptr()
            scratch = []   # every segment's workspace stays alive until the side stream has been joined
            launched = 0
            for i in range(nseg):
                c0, c1 = bounds[i], bounds[i + 1]
                t0, S_i = c0 * CHUNK, (c1 - c0) * CHUNK
                nb_i = nbytes if nseg == 1 else self.lib.gdn2_prefill_workspace_bytes(B, S_i, H, HK, DK, DV, code, p)
                ws_i = torch.empty(nb_i, dtype=torch.uint8, device=dev)
                scratch.append(ws_i)
                ptrs = [x.data_ptr() + t0 * x.shape[2] * x.shape[-1] * x.element_size() for x in (q, k, v, g, b, w)]
                rc = self.lib.gdn2_chunk_prep(*ptrs, ws_i.data_ptr(), nb_i, B, S_i, H, HK, DK, DV, in_bs, float(scale),
                                              code, p, main.cuda_stream)
                _check(self.lib, rc, "gdn2_chunk_prep")
                scan_stream = main
                if side is not None:
                    ev = torch.cuda.Event()
                    ev.record(main)
                    side.wait_event(ev)
                    scan_stream = side
                two_parts = (then_with_state is not None and gated_norm is None and hs is None and nseg == 1
                             and self.lib.gdn2_prefill_scan_launches(B, S_i, H, DK, DV, code, p) > 1)
                if two_parts:
                    part = lambda which: self.lib.gdn2_prefill_scan_part(       # noqa: E731
                        ws_i.data_ptr(), nb_i, state_ptr, out.data_ptr(), final_state.data_ptr(), B, S_i, H, HK, DK, DV,
                        out_batch_stride, code, p, which, main.cuda_stream)
                    rc = part(1)
                    _check(self.lib, rc, "gdn2_prefill_scan_part")
                    tail_stream = self._side_stream(dev)
                    ready = torch.cuda.Event()
                    ready.record(main)
                    tail_stream.wait_event(ready)
                    with torch.cuda.stream(tail_stream):
                        then_with_state(final_state)
                    then_with_state = None
                    rc = part(2)
                    main.wait_stream(tail_stream)
                elif gated_norm is None:
                    rc = self.lib.gdn2_prefill_scan(ws_i.data_ptr(), nb_i, state_ptr, out.data_ptr() + t0 * H * DV * esz,
                                                    states[i].data_ptr(), None if hs is None else hs.data_ptr(),
                                                    B, S_i, H, HK, DK, DV, out_batch_stride, code, p, scan_stream.cuda_stream)
                else:
                    gate, gcol, gweight, geps = gated_norm
                    if hs is not None or gate.dim() != 3 or not gate.is_contiguous() or gate.dtype != v.dtype:
                        raise ValueError("gated_norm needs a contiguous [B, S, NP] gate buffer in the input dtype "
                                         "and cannot be combined with chunk states")
                    NP = gate.shape[-1]
                    na = GatedNormArgs(gate.data_ptr() + (t0 * NP + gcol) * gate.element_size(), gweight.data_ptr(),
                                       NP, gate.shape[1], float(geps))
                    rc = self.lib.gdn2_prefill_scan_gated_norm(
                        ws_i.data_ptr(), nb_i, state_ptr, out.data_ptr() + t0 * H * DV * esz, states[i].data_ptr(),
                        B, S_i, H, HK, DK, DV, out_batch_stride, code, p, ctypes.byref(na), scan_stream.cuda_stream)
                _check(self.lib, rc, "gdn2_prefill_scan")
                state_ptr = states[i].data_ptr()
                launched += (2 if p != PATH_SIMT else 1) + (
                    1 if want_chunk_states else self.lib.gdn2_prefill_scan_launches(B, S_i, H, DK, DV, code, p))
            if side is not None:
                main.wait_stream(side)             # from here on the caller's stream is ordered after every scan
            del scratch                            # ... so only now may the allocator hand these blocks out again
        self.launches += launched
        if then_with_state is not None:
            then_with_state(final_state)
        return out, final_state, hs

    def chunk_output(self, q, k, v, g, b, w, scale: float, chunk_states, path=None):
        """Chunk-parallel output from stored chunk states (re-runs the chunk-local stage)."""
        _require_cuda(q, chunk_states)
        B, S, HK, DK = q.shape
        H, DV = v.shape[2], v.shape[-1]
        code = dtype_code(q.dtype)
        p = self.resolved_path(DK, DV, q.dtype, path)
        q, k, v, g, b, w = (t.contiguous() for t in (q, k, v, g, b, w))
        nbytes = self.lib.gdn2_prefill_workspace_bytes(B, S, H, HK, DK, DV, code, p)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        out = torch.empty(B, S, H, DV, dtype=v.dtype, device=q.device)
        st = self._stream(q)
        with _on_device(q.device):
            rc = self.lib.gdn2_chunk_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                          w.data_ptr(), ws.data_ptr(), nbytes, B, S, H, HK, DK, DV, S, float(scale),
                                          code, p, st)
            _check(self.lib, rc, "gdn2_chunk_prep")
            rc = self.lib.gdn2_chunk_output(ws.data_ptr(), nbytes, chunk_states.data_ptr(), out.data_ptr(),
                                            B, S, H, HK, DK, DV, S, code, p, st)
            _check(self.lib, rc, "gdn2_chunk_output")
        self.launches += 3 if p != PATH_SIMT else 2
        return out

    # -- diagnostics -------------------------------------------------------------------------
    def check_device_status(self, device=None):
        """Raise if any kernel on ``device`` gave up on a bounded wait since the last check."""
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        detail = ctypes.c_uint32(0)
        with _on_device(device):
            rc = self.lib.gdn2_check_device_status(torch.cuda.current_stream(device).cuda_stream,
                                                   ctypes.byref(detail))
        if rc != 0:
            raise GDN2KernelError(f"device status word = {detail.value:#x}: "
                                  f"{self.lib.gdn2_status_string(rc).decode()}")

    @staticmethod
    def layer_front_updates_cache_itself(proj, offsets, DK, DV, K) -> bool:
        """True when ``gdn2_layer_front`` writes the new convolution cache from the kernel that reads the old one
        (its one-token form: 16-bit storage, DK = DV = 128, four taps, fewer than 8 tokens), so that for ONE token
        the new cache may be the old cache's own memory."""
        return (proj.dtype in (torch.bfloat16, torch.float16) and DK == 128 and DV == 128 and K == 4
                and proj.shape[1] < 8 and proj.shape[2] % 4 == 0 and all(o % 4 == 0 for o in offsets))

    def layer_front(self, proj, offsets, conv_state, conv_weight, conv_bias, A_log, dt_bias, H, HK, DK, DV, K,
                    erase_scale, want_conv_state, conv_out=None):
        """Fused pre-processing of the layer: ``proj [B, S, NP]`` -> ``(q, k, v, g, b, w, new_conv_state)``.
        ``offsets`` = columns of the q, k, v, b, w, f projections inside ``proj``. ``conv_out``: where the new
        convolution cache goes instead of a fresh tensor; it may be ``conv_state`` itself only for a single token
        and only when ``layer_front_updates_cache_itself`` holds."""
        _require_cuda(proj)
        B, S, NP = proj.shape
        dt, dev = proj.dtype, proj.device
        q = torch.empty(B, S, HK, DK, dtype=dt, device=dev)        # one copy per key head: the kernels index them
        k, b = torch.empty_like(q), torch.empty_like(q)
        g = torch.empty(B, S, HK, DK, dtype=torch.float32, device=dev)
        v = torch.empty(B, S, H, DV, dtype=dt, device=dev)
        w = torch.empty_like(v)
        new_conv = None
        fused_tail = self.layer_front_updates_cache_itself(proj, offsets, DK, DV, K)
        if K > 1 and want_conv_state:
            if conv_out is not None:
                if conv_out.shape != (B, 2 * HK * DK + H * DV, K - 1) or conv_out.dtype != dt or not conv_out.is_contiguous():
                    raise ValueError("conv_out must be a contiguous [B, 2*HK*DK + H*DV, K-1] tensor of the input dtype")
                if conv_state is not None and conv_out.data_ptr() == conv_state.data_ptr() and not (fused_tail and S == 1):
                    raise ValueError("the convolution cache can be updated in place only for one token on the fused path")
                new_conv = conv_out
            else:
                new_conv = torch.empty(B, 2 * HK * DK + H * DV, K - 1, dtype=dt, device=dev)
        ptr = lambda t: None if t is None else t.data_ptr()
        a = LayerFrontArgs(ptr(proj), ptr(conv_state), ptr(conv_weight), ptr(conv_bias), ptr(A_log), ptr(dt_bias),
                           ptr(q), ptr(k), ptr(v), ptr(g), ptr(b), ptr(w), ptr(new_conv),
                           B, S, H, HK, DK, DV, K, NP, *offsets, erase_scale)
        with _on_device(dev):
            rc = self.lib.gdn2_layer_front(ctypes.byref(a), dtype_code(dt), self._stream(proj))
        _check(self.lib, rc, "gdn2_layer_front")
        self.launches += 2 if (new_conv is not None and not fused_tail) else 1
        return q, k, v, g, b, w, new_conv

    def layer_back(self, o, proj, norm_weight, off_gate, eps):
        """Fused gated RMSNorm: ``o [B, S, H, DV]`` and the o_gate columns of ``proj`` -> ``[B, S, H*DV]``."""
        _require_cuda(o, proj)
        B, S, H, DV = o.shape
        out = torch.empty(B, S, H * DV, dtype=o.dtype, device=o.device)
        with _on_device(o.device):
            rc = self.lib.gdn2_layer_back(o.data_ptr(), proj.data_ptr(), norm_weight.data_ptr(), out.data_ptr(),
                                          B * S, H, DV, proj.shape[-1], off_gate, eps, dtype_code(o.dtype),
                                          self._stream(o))
        _check(self.lib, rc, "gdn2_layer_back")
        self.launches += 1
        return out

    def maybe_check_device_status(self, device):
        """With ``GDN2_B200_CHECK_STATUS=1`` every public call ends with a synchronising status check, so a
        kernel that gave up on a bounded wait raises at the call that launched it (debugging aid; off by default
        because it serialises the host with the device)."""
        if os.environ.get("GDN2_B200_CHECK_STATUS", "0") not in ("", "0"):
            if torch.cuda.is_current_stream_capturing():
                return                   # a captured stream cannot be synchronised; the replaying caller checks
            self.check_device_status(device)

    def workspace_layout(self, B, S, H, DK, DV, dtype, path=None, HK=None) -> dict:
        """Byte offsets of the record arrays inside the prefill workspace (``gdn2_prefill_workspace_layout``)."""
        p = self.resolved_path(DK, DV, dtype, path)
        out = (ctypes.c_int64 * 8)()
        _check(self.lib, self.lib.gdn2_prefill_workspace_layout(B, S, H, HK or H, DK, DV, dtype_code(dtype), p, out),
               "gdn2_prefill_workspace_layout")
        return dict(zip(("wq", "aqk", "kgt", "ut", "gl", "flags", "seg", "total"), list(out)))

    def chunk_prep(self, q, k, v, g, b, w, scale: float, path=None):
        """The chunk-local stage alone. Returns ``(workspace uint8 tensor, resolved path)``."""
        _require_cuda(q)
        B, S, HK, DK = q.shape
        H, DV = v.shape[2], v.shape[-1]
        code = dtype_code(q.dtype)
        p = self.resolved_path(DK, DV, q.dtype, path)
        q, k, v, g, b, w = (t.contiguous() for t in (q, k, v, g, b, w))
        nbytes = self.lib.gdn2_prefill_workspace_bytes(B, S, H, HK, DK, DV, code, p)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        with _on_device(q.device):
            rc = self.lib.gdn2_chunk_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                          w.data_ptr(), ws.data_ptr(), nbytes, B, S, H, HK, DK, DV, S, float(scale),
                                          code, p, self._stream(q))
        _check(self.lib, rc, "gdn2_chunk_prep")
        self.launches += 2 if p != PATH_SIMT else 1
        return ws, p

    def oproj_reduce(self, x, weight, out, peer_slots, peer_flags, epochs, rank, world, wait_cycles=0):
        """``gdn2_oproj_reduce``: ``x [rows, K]``, ``weight [hidden, K]`` -> ``out [rows, hidden]`` summed over ranks.
        ``peer_slots`` / ``peer_flags``: int64 device tensors holding the peer-mapped buffer addresses."""
        _require_cuda(x, weight, out)
        rows, K = x.shape
        a = OProjReduceArgs(x.data_ptr(), weight.data_ptr(), out.data_ptr(),
                            None if peer_slots is None else peer_slots.data_ptr(),
                            None if peer_flags is None else peer_flags.data_ptr(), epochs.data_ptr(),
                            rows, K, weight.shape[0], rank, world, wait_cycles)
        with _on_device(x.device):
            rc = self.lib.gdn2_oproj_reduce(ctypes.byref(a), dtype_code(x.dtype), self._stream(x))
        _check(self.lib, rc, "gdn2_oproj_reduce")
        self.launches += 1
        return out

    def selftest_wait(self, limit_cycles: int, device=None) -> int:
        """Launch the block whose bounded wait nothing satisfies; returns how many threads gave up."""
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        counter = torch.zeros(1, dtype=torch.int32, device=device)
        with _on_device(device):
            rc = self.lib.gdn2_selftest_wait(limit_cycles, counter.data_ptr(),
                                             torch.cuda.current_stream(device).cuda_stream)
        _check(self.lib, rc, "gdn2_selftest_wait")
        return int(counter.item())

    def selftest_mma(self, a: torch.Tensor, bt: torch.Tensor) -> torch.Tensor:
        _require_cuda(a, bt)
        out = torch.zeros(4, 128, 128, dtype=torch.float32, device=a.device)
        with _on_device(a.device):
            rc = self.lib.gdn2_selftest_mma(a.data_ptr(), bt.data_ptr(), out.data_ptr(), self._stream(a))
        _check(self.lib, rc, "gdn2_selftest_mma")
        return out


_kernels = None


def kernels() -> NativeKernels:
    """The process-wide kernel launcher (created on first use)."""
    global _kernels
    if _kernels is None:
        _kernels = NativeKernels()
    return _kernels
