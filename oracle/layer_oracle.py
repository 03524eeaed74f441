"""CPU oracle for the GatedDeltaNet2 token-mixer layer around the hot path.

TEST INFRASTRUCTURE, NOT PRODUCT (see ``gdn2_oracle.py``). A functional
restatement of the reference layer, driven by a plain ``state_dict`` whose keys
are the reference module's parameter names, so weights are interchangeable:

    q_proj.weight k_proj.weight v_proj.weight b_proj.weight w_proj.weight
    f_proj.weight o_gate_proj.weight o_proj.weight
    q_conv.conv.{weight,bias} k_conv.conv.{weight,bias} v_conv.conv.{weight,bias}
    A_log dt_bias o_norm.weight

Follows gdn2/attention.py: ``_ShortConv`` 186-215, ``_GatedRMSNorm`` 218-229,
``_gates`` 290-293, ``_expand`` 295-297, ``forward`` 299-357, ``prefill``
359-414, ``decode`` 416-465, ``init_cache`` 481-491.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import gdn2_oracle as core

__all__ = ["LayerDims", "random_state_dict", "init_cache", "forward", "prefill", "decode"]


@dataclass
class LayerDims:
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim_k: int = 128
    head_dim_v: int = 128
    conv_size: int = 4
    norm_eps: float = 1e-5
    erase_gate_scale: float = 1.0
    chunk_size: int = 64
    sub_chunk_size: int = 16

    @property
    def d_qk(self):
        return self.num_kv_heads * self.head_dim_k

    @property
    def d_v(self):
        return self.num_heads * self.head_dim_v


def random_state_dict(dims: LayerDims, seed=0, std=0.02, dtype=torch.float32):
    """Every parameter ``N(0, std^2)`` from one seeded host generator (benchmark init)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    d = dims

    def r(*shape):
        return (torch.randn(*shape, generator=gen, dtype=torch.float32) * std).to(dtype)

    sd = {}
    for name, out in (("q_proj", d.d_qk), ("k_proj", d.d_qk), ("v_proj", d.d_v), ("b_proj", d.d_qk),
                      ("w_proj", d.d_v), ("f_proj", d.d_qk), ("o_gate_proj", d.d_v)):
        sd[f"{name}.weight"] = r(out, d.hidden_size)
    sd["o_proj.weight"] = r(d.hidden_size, d.d_v)
    if d.conv_size > 0:
        for name, ch in (("q_conv", d.d_qk), ("k_conv", d.d_qk), ("v_conv", d.d_v)):
            sd[f"{name}.conv.weight"] = r(ch, 1, d.conv_size)
            sd[f"{name}.conv.bias"] = r(ch)
    sd["A_log"] = r(d.num_kv_heads)
    sd["dt_bias"] = r(d.num_kv_heads, d.head_dim_k)
    sd["o_norm.weight"] = r(d.head_dim_v)
    return sd


def init_cache(dims: LayerDims, batch, conv_dtype=torch.float32):
    """``(recurrent_state fp32 [B,H,DK,DV], conv_state [B, 2*d_qk+d_v, conv_size-1] | None)``."""
    state = torch.zeros(batch, dims.num_heads, dims.head_dim_k, dims.head_dim_v)
    conv = None
    if dims.conv_size > 0:
        conv = torch.zeros(batch, 2 * dims.d_qk + dims.d_v, dims.conv_size - 1, dtype=conv_dtype)
    return state, conv


def _conv_full(x, weight, bias, width):
    y = F.conv1d(x.transpose(1, 2), weight, bias, groups=x.shape[-1], padding=width - 1)
    return F.silu(y[..., : x.shape[1]].transpose(1, 2))


def _conv_cached(x, tail, weight, bias, width):
    buf = torch.cat([tail, x.transpose(1, 2)], dim=-1)
    y = F.conv1d(buf, weight, bias, groups=x.shape[-1]).transpose(1, 2)
    return F.silu(y), buf[..., -(width - 1):]


def _front(sd, dims, x, conv_state, cached):
    """Projections, short conv, L2 norm, gates, head expansion. ``x``: ``[B,S,hidden]``."""
    B, S, _ = x.shape
    H, HK, DK, DV = dims.num_heads, dims.num_kv_heads, dims.head_dim_k, dims.head_dim_v
    lin = lambda name: F.linear(x, sd[f"{name}.weight"])  # noqa: E731
    q, k, v = lin("q_proj"), lin("k_proj"), lin("v_proj")
    new_conv = None
    if dims.conv_size > 0:
        d = dims.d_qk
        cw = lambda n: (sd[f"{n}.conv.weight"], sd[f"{n}.conv.bias"], dims.conv_size)  # noqa: E731
        if cached:
            q, cq = _conv_cached(q, conv_state[:, :d], *cw("q_conv"))
            k, ck = _conv_cached(k, conv_state[:, d:2 * d], *cw("k_conv"))
            v, cv = _conv_cached(v, conv_state[:, 2 * d:], *cw("v_conv"))
            new_conv = torch.cat([cq, ck, cv], dim=1)
        else:
            width = dims.conv_size - 1
            tail = torch.cat([q, k, v], dim=-1).transpose(1, 2)
            new_conv = F.pad(tail, (max(0, width - S), 0))[..., -width:]
            q, k, v = _conv_full(q, *cw("q_conv")), _conv_full(k, *cw("k_conv")), _conv_full(v, *cw("v_conv"))
    q = F.normalize(q.view(B, S, HK, DK), p=2, dim=-1)
    k = F.normalize(k.view(B, S, HK, DK), p=2, dim=-1)
    v = v.view(B, S, H, DV)
    f = lin("f_proj").view(B, S, HK, DK)
    g = -sd["A_log"].float().exp().unsqueeze(-1) * F.softplus(f.float() + sd["dt_bias"].float())
    b = torch.sigmoid(lin("b_proj").view(B, S, HK, DK)) * dims.erase_gate_scale
    w = torch.sigmoid(lin("w_proj").view(B, S, H, DV))
    rep = H // HK
    if rep > 1:
        q, k, b, g = (t.repeat_interleave(rep, dim=-2) for t in (q, k, b, g))
    return q, k, v, g, b, w, new_conv


def _back(sd, dims, x, o):
    B, S, _ = x.shape
    gate = F.linear(x, sd["o_gate_proj.weight"]).view(B, S, dims.num_heads, dims.head_dim_v)
    of = o.float()
    of = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + dims.norm_eps)
    y = (of * sd["o_norm.weight"].float() * F.silu(gate.float())).to(gate.dtype)
    return F.linear(y.reshape(B, S, dims.d_v), sd["o_proj.weight"])


def forward(sd, dims, x, state=None):
    """Full-sequence forward (zero-history conv). Returns ``(out, final_state, conv_state)``."""
    q, k, v, g, b, w, conv = _front(sd, dims, x, None, cached=False)
    o, s = core.attention(q, k, v, g, b, w, dims.head_dim_k**-0.5, state, dims.chunk_size, dims.sub_chunk_size)
    return _back(sd, dims, x, o), s, conv


def prefill(sd, dims, x, state, conv_state):
    """Serving prefill from a cache. Returns ``(out, state, conv_state)``."""
    q, k, v, g, b, w, conv = _front(sd, dims, x, conv_state, cached=dims.conv_size > 0)
    o, s = core.prefill(q, k, v, g, b, w, state, dims.head_dim_k**-0.5, dims.chunk_size, dims.sub_chunk_size)
    return _back(sd, dims, x, o), s, conv


def decode(sd, dims, x, state, conv_state):
    """``n``-token decode; ``state`` is updated in place. Returns ``(out, state, conv_state)``."""
    q, k, v, g, b, w, conv = _front(sd, dims, x, conv_state, cached=dims.conv_size > 0)
    o = core.decode(q, k, v, g, b, w, state, dims.head_dim_k**-0.5)
    return _back(sd, dims, x, o), state, conv
