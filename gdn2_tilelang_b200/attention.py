"""``gdn2_attention`` and the ``GatedDeltaNet2`` token mixer, API-compatible with the reference
(gdn2/attention.py of the reference project: ``resolve_backend`` 44-61, ``gdn2_attention``
102-164, ``GDN2Cache`` 172-183, ``_ShortConv`` 186-215, ``_GatedRMSNorm`` 218-229,
``GatedDeltaNet2`` 232-491).

Differences a user of the reference should know about:

* inference only -- the functional op runs under ``no_grad`` and has no backward;
* the only backend is the CUDA kernel library. ``"auto"`` and ``"tilelang"`` (kept as an alias so
  existing configs load) resolve to ``"cuda"``; ``"torch"`` and non-CUDA tensors raise, because no
  host implementation is shipped;
* ``init_cache`` allocates ``conv_state`` in the layer's parameter dtype (the reference allocates
  it in float32 and then fails on a bf16 layer); ``recurrent_state`` stays float32;
* the module's parameter names and shapes are unchanged, so ``state_dict``s are interchangeable.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

from . import _cabi
from .config import DEFAULT_KERNEL_CONFIG, GDN2Config, GatedDeltaNet2Config
from .forward import chunk_gdn2_fwd
from .inference import gdn2_decode, gdn2_prefill

__all__ = ["gdn2_attention", "GatedDeltaNet2", "GDN2Cache", "GraphedStep", "resolve_backend"]

_BACKENDS = ("auto", "cuda", "tilelang", "torch")


def resolve_backend(backend: str, on_cuda: bool, needs_grad: bool = False) -> str:
    """Validate ``backend`` and return the concrete one, which can only be ``"cuda"``.

    Raises ``ValueError`` for an unknown name, for the host-only ``"torch"`` backend, when the
    tensors are not on a CUDA device, and when gradients are requested.
    """
    if backend not in _BACKENDS:
        raise ValueError(f"unknown backend {backend!r}; expected one of {_BACKENDS}")
    if backend == "torch":
        raise ValueError("backend 'torch' (the host reference path) is not part of this package; "
                         "use the reference project's gdn2.reference for a host evaluation")
    if not on_cuda:
        raise ValueError(f"backend {backend!r} requires a CUDA device")
    if needs_grad:
        raise ValueError("the sm_100a kernels implement the forward / serving path only; "
                         "call under torch.no_grad() or detach the inputs")
    return "cuda"


def gdn2_attention(q, k, v, g, b, w, scale=None, initial_state=None, output_final_state=False,
                   config: GDN2Config = DEFAULT_KERNEL_CONFIG, cu_seqlens=None):
    """Gated DeltaNet-2 attention over a full sequence.

    ``q, k, b, g``: ``[B, S, H, DK]``; ``v, w``: ``[B, S, H, DV]``; ``g`` is the natural-log decay
    (``<= 0``). Returns ``(o [B, S, H, DV] in the input dtype, final_state float32 | None)``.

    ``cu_seqlens`` (``[N + 1]`` increasing token offsets starting at 0, the packing convention of the reference's
    signature, gdn2/attention.py:142-145, where it still raises): the tensors hold ``N`` sequences packed along
    the token axis of ONE batch entry (``B == 1``); sequence ``i`` is tokens ``cu_seqlens[i]:cu_seqlens[i+1]``
    and starts from ``initial_state[i]`` (``[N, H, DK, DV]``) or zero. ``final_state`` is then ``[N, H, DK, DV]``.
    Every sequence runs through the same kernels as an unpacked call on its slice: no padding, no copies.
    """
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (q, k, v, g, b, w, initial_state))
    resolve_backend(config.backend, q.device.type == "cuda", needs_grad)
    if cu_seqlens is not None:
        return _packed_attention(q, k, v, g, b, w, scale, initial_state, output_final_state, config, cu_seqlens)
    return chunk_gdn2_fwd(q, k, v, g, b, w, scale, initial_state, output_final_state, config)


@torch.no_grad()
def _packed_attention(q, k, v, g, b, w, scale, initial_state, output_final_state, config, cu_seqlens):
    """Variable-length batch packed into one row: one chunkwise (+ tail) evaluation per sequence, all queued on
    the current stream, results written straight into the packed output."""
    offs = [int(x) for x in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]
    B, T, _, DK = q.shape
    H, DV = v.shape[2], v.shape[-1]
    N = len(offs) - 1
    if B != 1:
        raise ValueError("with cu_seqlens the sequences are packed into one batch entry: expected B == 1")
    if N < 1 or offs[0] != 0 or offs[-1] != T or any(hi < lo for lo, hi in zip(offs, offs[1:])):
        raise ValueError(f"cu_seqlens must rise from 0 to the packed length {T}, got {offs}")
    if initial_state is not None and tuple(initial_state.shape) != (N, H, DK, DV):
        raise ValueError(f"initial_state must have shape {(N, H, DK, DV)} for {N} packed sequences")
    o = torch.empty(1, T, H, DV, dtype=v.dtype, device=q.device)
    finals = torch.zeros(N, H, DK, DV, dtype=torch.float32, device=q.device) if output_final_state else None
    g = g.float()
    for i, (lo, hi) in enumerate(zip(offs, offs[1:])):
        if hi == lo:
            if finals is not None and initial_state is not None:
                finals[i].copy_(initial_state[i])
            continue
        s0 = None if initial_state is None else initial_state[i:i + 1]
        _, s_i = chunk_gdn2_fwd(*(t[:, lo:hi] for t in (q, k, v, g, b, w)), scale, s0, output_final_state, config,
                                out=o[:, lo:hi])
        if finals is not None:
            finals[i:i + 1].copy_(s_i)
    return o, finals


@dataclass
class GDN2Cache:
    """Per-layer decoding cache: ``recurrent_state [B, H_v, DK, DV]`` float32 and ``conv_state
    [B, 2*HK*DK + H*DV, conv_size-1]`` (the last pre-convolution q | k | v projections) or ``None``."""

    recurrent_state: torch.Tensor
    conv_state: torch.Tensor | None = None


class _ShortConv(nn.Module):
    """Parameter holder of the causal depthwise conv1d (+ SiLU) over ``[B, S, C]``: ``conv.weight [C, 1, K]``,
    ``conv.bias [C]``, the names and shapes of the reference module. The convolution itself runs inside
    ``gdn2_layer_front`` together with everything else element-wise."""

    def __init__(self, channels: int, kernel_size: int = 4, activation: bool = True):
        super().__init__()
        if not activation:
            raise ValueError("the fused kernel always applies SiLU after the convolution, as the layer does")
        self.channels, self.kernel_size, self.activation = channels, kernel_size, activation
        self.conv = nn.Conv1d(channels, channels, kernel_size, groups=channels, padding=kernel_size - 1)


class _GatedRMSNorm(nn.Module):
    """Parameter holder of the per-head RMSNorm multiplied by a SiLU gate (``weight [DV]``, ``eps``); evaluated
    in float32 by ``gdn2_layer_back``."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))


class GatedDeltaNet2(nn.Module):
    """Gated DeltaNet-2 token mixer: projections, short convolution, L2-normalised q/k, the decay /
    erase / write gates, the recurrent attention kernels, gated RMSNorm and the output projection."""

    def __init__(self, config: GatedDeltaNet2Config):
        super().__init__()
        self.cfg = config
        H = config.num_heads
        HK = config.num_kv_heads or H
        if H % HK != 0:
            raise ValueError(f"num_heads {H} must be a multiple of num_kv_heads {HK}")
        DK = config.head_dim_k
        DV = config.head_dim_v or config.head_dim_k
        self.num_heads, self.num_kv_heads = H, HK
        self.head_dim_k, self.head_dim_v = DK, DV
        self.head_repeat = H // HK
        d_qk, d_v = HK * DK, H * DV
        hid = config.hidden_size
        self.q_proj = nn.Linear(hid, d_qk, bias=False)
        self.k_proj = nn.Linear(hid, d_qk, bias=False)
        self.v_proj = nn.Linear(hid, d_v, bias=False)
        self.b_proj = nn.Linear(hid, d_qk, bias=False)
        self.w_proj = nn.Linear(hid, d_v, bias=False)
        self.f_proj = nn.Linear(hid, d_qk, bias=False)
        self.o_gate_proj = nn.Linear(hid, d_v, bias=False)
        self.o_proj = nn.Linear(d_v, hid, bias=False)
        if config.conv_size > 0:
            self.q_conv = _ShortConv(d_qk, config.conv_size)
            self.k_conv = _ShortConv(d_qk, config.conv_size)
            self.v_conv = _ShortConv(d_v, config.conv_size)
        else:
            self.q_conv = self.k_conv = self.v_conv = None
        lo, hi = config.a_init_range
        self.A_log = nn.Parameter(torch.empty(HK).uniform_(lo, hi).log_())
        dt_lo, dt_hi = config.dt_init_range
        dt = torch.empty(HK, DK).uniform_(dt_lo, dt_hi)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))   # inverse softplus of dt
        self.o_norm = _GatedRMSNorm(DV, config.norm_eps)
        self.scale = DK**-0.5
        self.erase_scale = config.erase_gate_scale

    # ------------------------------------------------------------------ pieces
    def _fused_tables(self):
        """Concatenated projection weight ``[NP, hidden]`` (q | k | v | b | w | f | o_gate), its column
        offsets, and the convolution weight ``[CC, K]`` / bias ``[CC]`` (q | k | v); rebuilt when a
        parameter changes."""
        lin = (self.q_proj, self.k_proj, self.v_proj, self.b_proj, self.w_proj, self.f_proj, self.o_gate_proj)
        convs = () if self.q_conv is None else (self.q_conv.conv, self.k_conv.conv, self.v_conv.conv)
        params = [m.weight for m in lin] + [c.weight for c in convs] + [c.bias for c in convs if c.bias is not None]
        key = tuple((p.data_ptr(), p._version, p.dtype) for p in params)
        if getattr(self, "_fused_key", None) != key:
            w_cat = torch.cat([m.weight for m in lin], 0).contiguous()
            sizes = [m.weight.shape[0] for m in lin]
            offs = [sum(sizes[:i]) for i in range(len(sizes))]
            cw = cb = None
            if convs:
                cw = torch.cat([c.weight.reshape(c.weight.shape[0], -1) for c in convs], 0).contiguous()
                if all(c.bias is not None for c in convs):
                    cb = torch.cat([c.bias for c in convs], 0).contiguous()
            self._fused_key, self._fused = key, (w_cat, offs, cw, cb)
        return self._fused

    def _check_supported(self, x):
        """The element-wise stages run in the fused kernels only; configurations they do not cover raise."""
        if self.head_dim_k > 256 or self.head_dim_v > 256:
            raise ValueError("the fused layer kernels support head dimensions up to 256")
        if self.q_proj.weight.dtype != x.dtype:
            raise TypeError(f"input dtype {x.dtype} differs from the layer's parameter dtype {self.q_proj.weight.dtype}")
        if any(m.bias is not None for m in (self.q_proj, self.k_proj, self.v_proj, self.b_proj, self.w_proj,
                                            self.f_proj, self.o_gate_proj)):
            raise ValueError("projection biases are not supported (the reference layer has none)")

    def _front(self, x, conv_state, cached: bool, update_cache_in_place: bool = False):
        """Everything before the attention kernels: ONE GEMM for the seven input projections, then one kernel
        for everything element-wise. Returns ``(q, k, v, g, b, w, new_conv_state, proj)``; the o_gate columns
        of the projection buffer ``proj`` feed ``_back``. ``update_cache_in_place``: for a single token, let the
        kernel write the new convolution cache into ``conv_state`` itself where it can (the returned
        ``new_conv_state`` is then ``conv_state``)."""
        self._check_supported(x)
        H, HK, DK, DV = self.num_heads, self.num_kv_heads, self.head_dim_k, self.head_dim_v
        w_cat, offs, cw, cb = self._fused_tables()
        proj = F.linear(x, w_cat)
        K = self.cfg.conv_size if self.q_conv is not None else 0
        state = None
        if cached and conv_state is not None:
            state = conv_state if conv_state.dtype == x.dtype else conv_state.to(x.dtype)
            state = state.contiguous()
        K_ = _cabi.kernels()
        conv_out = None
        if (update_cache_in_place and state is not None and state is conv_state and x.shape[1] == 1
                and K_.layer_front_updates_cache_itself(proj, offs[:6], DK, DV, K)):
            conv_out = state
        q, k, v, g, b, w, new_conv = K_.layer_front(
            proj, offs[:6], state, cw, cb, self.A_log.detach().to(x.dtype), self.dt_bias.detach().to(x.dtype).contiguous(),
            H, HK, DK, DV, K, float(self.erase_scale), want_conv_state=True, conv_out=conv_out)
        return q, k, v, g, b, w, new_conv, proj

    def _back(self, x, o, proj, normed_rows: int = 0):
        """Gated RMSNorm and output projection. The first ``normed_rows`` tokens of ``o`` have already been
        normalised by the scan's epilogue; the rest (a ragged tail, or everything) goes through ``gdn2_layer_back``."""
        B, S, H, DV = o.shape
        off_gate = self._fused_tables()[1][6]
        K = _cabi.kernels()
        weight = self.o_norm.weight.detach().to(o.dtype)
        if normed_rows == 0:
            normed = K.layer_back(o.contiguous(), proj, weight, off_gate, float(self.o_norm.eps))
        else:
            normed = o.view(B, S, H * DV)
            if normed_rows < S:
                tail = K.layer_back(o[:, normed_rows:].contiguous(), proj[:, normed_rows:].contiguous(), weight, off_gate,
                                    float(self.o_norm.eps))
                normed[:, normed_rows:] = tail
        return self._project_out(normed)

    def _gated_norm_args(self, x, proj):
        """Arguments that make the scan apply the gated RMSNorm itself (``cfg.kernel`` unchanged; switched on with
        ``layer.fuse_output_norm = True``), or ``None``. Off by default: the scan is bound by its chunk-to-chunk
        chain and its four output warps have little slack, so the epilogue (64 SiLUs and a norm per thread and
        chunk) stretches a chunk from 1.5 to 2.8 us, which costs more than the separate kernel's 0.06 ms at the
        benchmark's layer size."""
        if not getattr(self, "fuse_output_norm", False):
            return None
        if not _cabi.kernels().fuses_gated_norm(self.head_dim_k, self.head_dim_v, x.dtype):
            return None
        return (proj, self._fused_tables()[1][6], self.o_norm.weight.detach().to(x.dtype), float(self.o_norm.eps))

    def _project_out(self, normed):
        """``o_proj``; the head-parallel variant overrides it to add the sum over ranks."""
        return self.o_proj(normed)

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def forward(self, hidden_states, cache: GDN2Cache | None = None, use_cache: bool = False, cu_seqlens=None):
        """Full-sequence forward. Returns ``(output [B, S, hidden], GDN2Cache | None)``.

        ``cu_seqlens`` raises here, as in the reference (gdn2/attention.py:299-357): the short convolution
        would have to restart at every packed boundary, which the fused pre-processing kernel does not do;
        the functional op ``gdn2_attention`` does take packed batches."""
        if cu_seqlens is not None:
            raise NotImplementedError("packed variable-length batches through the layer need a convolution that "
                                      "restarts at sequence boundaries; call gdn2_attention with cu_seqlens on "
                                      "pre-processed tensors, or pad the batch")
        q, k, v, g, b, w, conv, proj = self._front(hidden_states, None, cached=False)
        o, final_state = gdn2_attention(
            q, k, v, g, b, w, scale=self.scale,
            initial_state=cache.recurrent_state if cache is not None else None,
            output_final_state=use_cache, config=self.cfg.kernel, cu_seqlens=cu_seqlens)
        out = self._back(hidden_states, o, proj)
        return out, (GDN2Cache(final_state, conv if use_cache else None) if use_cache else None)

    @torch.no_grad()
    def prefill(self, hidden_states, cache: GDN2Cache | None = None):
        """Prefill a prompt (or a segment of one) and return ``(output, cache)`` to decode from."""
        if cache is None:
            cache = self.init_cache(hidden_states.shape[0], device=hidden_states.device)
        q, k, v, g, b, w, conv, proj = self._front(hidden_states, cache.conv_state, cached=self.q_conv is not None)
        if conv is not None:
            cache.conv_state = conv
        norm = self._gated_norm_args(hidden_states, proj)
        o, state = gdn2_prefill(q, k, v, g, b, w, cache.recurrent_state, scale=self.scale, config=self.cfg.kernel,
                                gated_norm=norm)
        cache.recurrent_state = state
        S = hidden_states.shape[1]
        return self._back(hidden_states, o, proj, normed_rows=0 if norm is None else S // 64 * 64), cache

    @torch.no_grad()
    def decode(self, hidden_states, cache: GDN2Cache):
        """Decode ``n`` tokens ``[B, n, hidden]``; ``cache.recurrent_state`` is updated in place."""
        q, k, v, g, b, w, conv, proj = self._front(hidden_states, cache.conv_state, cached=self.q_conv is not None)
        if conv is not None:
            cache.conv_state = conv
        o = gdn2_decode(q, k, v, g, b, w, cache.recurrent_state, scale=self.scale)
        return self._back(hidden_states, o, proj), cache

    @torch.no_grad()
    def step(self, hidden_states, cache: GDN2Cache):
        """Decode one token ``[B, hidden]``."""
        out, cache = self.decode(hidden_states.unsqueeze(1), cache)
        return out[:, 0], cache

    def init_cache(self, batch_size: int, device=None, dtype=torch.float32) -> GDN2Cache:
        """Empty cache: float32 recurrent state, conv tail in the layer's parameter dtype."""
        if dtype != torch.float32:
            raise ValueError("the recurrent state is kept in float32")
        device = self.o_proj.weight.device if device is None else device
        state = torch.zeros(batch_size, self.num_heads, self.head_dim_k, self.head_dim_v, device=device, dtype=dtype)
        conv_state = None
        if self.q_conv is not None:
            channels = 2 * self.num_kv_heads * self.head_dim_k + self.num_heads * self.head_dim_v
            conv_state = torch.zeros(batch_size, channels, self.cfg.conv_size - 1, device=device,
                                     dtype=self.o_proj.weight.dtype)
        return GDN2Cache(state, conv_state)


class GraphedStep:
    """One-token ``GatedDeltaNet2.step`` captured in a CUDA graph (no counterpart in the reference).

    ``step`` is some forty small launches (projections, convolutions, gates, the decode kernel, the gated
    norm); at batch sizes where each of them takes microseconds the host's launch cost sets the latency.
    Capturing them once and replaying the graph makes a step one launch. The cache is updated in place
    (``recurrent_state`` by the decode kernel, ``conv_state`` by a copy), so the ``GDN2Cache`` given here
    is THE cache of the sequence from then on; its tensors must not be replaced, only written into.

    >>> cache = layer.prefill(prompt)[1]
    >>> step = GraphedStep(layer, cache)
    >>> y = step(x_t)            # [B, hidden] -> [B, hidden]; a view of a static buffer, valid until the next call
    """

    def __init__(self, layer: "GatedDeltaNet2", cache: GDN2Cache, warmup: int = 2):
        state = cache.recurrent_state
        if not state.is_cuda:
            raise ValueError("GraphedStep needs a cache on a CUDA device")
        self.layer, self.cache = layer, cache
        B = state.shape[0]
        weight = layer.o_proj.weight
        self.x = torch.zeros(B, layer.cfg.hidden_size, device=state.device, dtype=weight.dtype)
        keep_state = state.clone()
        keep_conv = None if cache.conv_state is None else cache.conv_state.clone()
        side = torch.cuda.Stream(state.device)
        side.wait_stream(torch.cuda.current_stream(state.device))
        with torch.cuda.stream(side):                     # library handles and workspaces come to life here
            for _ in range(max(1, warmup)):
                self._step_in_place()
        torch.cuda.current_stream(state.device).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = self._step_in_place()
        state.copy_(keep_state)                           # the warm-up and the capture advanced the cache
        if keep_conv is not None:
            cache.conv_state.copy_(keep_conv)

    @torch.no_grad()
    def _step_in_place(self):
        layer, cache = self.layer, self.cache
        x = self.x.unsqueeze(1)
        q, k, v, g, b, w, conv, proj = layer._front(x, cache.conv_state, cached=layer.q_conv is not None,
                                                     update_cache_in_place=True)
        if conv is not None and conv is not cache.conv_state:
            cache.conv_state.copy_(conv)
        o = gdn2_decode(q, k, v, g, b, w, cache.recurrent_state, scale=layer.scale)
        return layer._back(x, o, proj)[:, 0]

    def __call__(self, hidden_states):
        self.x.copy_(hidden_states)
        self.graph.replay()
        return self.out
