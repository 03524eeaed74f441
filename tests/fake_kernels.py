"""Test double for ``gdn2_tilelang_b200._cabi.NativeKernels`` backed by the CPU oracle.

Used ONLY by the CPU tests of the host-side logic (tail routing, state ownership, caches, head
sharding): it lets that logic run without a GPU. The product never uses it."""

from __future__ import annotations

import torch

from oracle import gdn2_oracle as orc


def _expanded(q, k, v, g, b, w):
    """Key heads repeated to the value heads (the oracle, like the reference op, takes equal head counts)."""
    rep = v.shape[2] // q.shape[2]
    if rep > 1:
        q, k, g, b = (t.repeat_interleave(rep, dim=2) for t in (q, k, g, b))
    return q, k, v, g, b, w


class OracleKernels:
    def __init__(self):
        self.calls = []
        self.launches = 0

    def decode(self, q, k, v, g, b, w, state, scale, out=None):
        self.calls.append(("decode", q.shape[1]))
        q, k, v, g, b, w = _expanded(q, k, v, g, b, w)
        o = orc.decode(q, k, v, g, b, w, state, scale)
        if out is not None:
            out.copy_(o)
            return out
        return o

    def prefill_ragged(self, q, k, v, g, b, w, scale, initial_state=None):
        return None                      # the double composes the stages, which is what the host-logic tests watch

    def fuses_gated_norm(self, DK, DV, dtype):
        return False                     # the double keeps the norm a separate stage (layer_back)

    def chunk_forward(self, q, k, v, g, b, w, scale, initial_state=None, want_chunk_states=False,
                      path=None, out=None, out_batch_stride=None, gated_norm=None, then_with_state=None):
        self.calls.append(("chunk_forward", q.shape[1]))
        assert q.shape[1] % 64 == 0 and gated_norm is None
        q, k, v, g, b, w = _expanded(q, k, v, g, b, w)
        res = orc.chunkwise(q, k, v, g, b, w, scale, initial_state, return_chunk_states=want_chunk_states)
        o, s = res[0].to(v.dtype), res[1]
        if out is not None:
            out[:, : q.shape[1]].copy_(o)
            o = out
        if then_with_state is not None:
            then_with_state(s)
        return o, s, (res[2] if want_chunk_states else None)

    def chunk_output(self, q, k, v, g, b, w, scale, chunk_states, path=None):
        q, k, v, g, b, w = _expanded(q, k, v, g, b, w)
        f = orc.chunk_factors(q, k, v, g, b, w, scale)
        B, S, H, DK = q.shape
        h = chunk_states.permute(0, 2, 1, 3, 4).float()
        un = f["U"] - f["W"] @ h
        o = f["Qg"] @ h + f["Aqk"] @ un
        return o.permute(0, 2, 3, 1, 4).reshape(B, S, H, -1).to(v.dtype)

    # -- the layer's element-wise stages, restated with torch operators (gdn2/attention.py:186-229, 290-297 of
    #    the reference project): what gdn2_layer_front / gdn2_layer_back compute on the device
    @staticmethod
    def layer_front_updates_cache_itself(proj, offsets, DK, DV, K):
        return False

    def layer_front(self, proj, offsets, conv_state, conv_weight, conv_bias, A_log, dt_bias, H, HK, DK, DV, K,
                    erase_scale, want_conv_state, conv_out=None):
        return layer_front_chain(proj, offsets, conv_state, conv_weight, conv_bias, A_log, dt_bias, H, HK, DK, DV, K,
                                 erase_scale)

    def layer_back(self, o, proj, norm_weight, off_gate, eps):
        return layer_back_chain(o, proj, norm_weight, off_gate, eps)

    def maybe_check_device_status(self, device):
        pass


def layer_front_chain(proj, offsets, conv_state, conv_weight, conv_bias, A_log, dt_bias, H, HK, DK, DV, K, erase_scale):
    """Torch-operator form of ``gdn2_layer_front`` on the fused projection buffer ``proj [B, S, NP]``."""
    import torch.nn.functional as F

    B, S, _ = proj.shape
    oq, ok, ov, ob, ow, of = offsets
    dqk, dv = HK * DK, H * DV
    qkv = torch.cat([proj[..., oq:oq + dqk], proj[..., ok:ok + dqk], proj[..., ov:ov + dv]], -1)
    new_conv = None
    if K > 0:
        tail = conv_state if conv_state is not None else torch.zeros(B, qkv.shape[-1], K - 1, dtype=proj.dtype)
        buf = torch.cat([tail.to(proj.dtype), qkv.transpose(1, 2)], -1)
        new_conv = buf[..., -(K - 1):].contiguous()
        y = F.conv1d(buf, conv_weight.reshape(-1, 1, K), conv_bias, groups=buf.shape[1]).transpose(1, 2)
        qkv = F.silu(y)
    q = F.normalize(qkv[..., :dqk].reshape(B, S, HK, DK), p=2, dim=-1)
    k = F.normalize(qkv[..., dqk:2 * dqk].reshape(B, S, HK, DK), p=2, dim=-1)
    v = qkv[..., 2 * dqk:].reshape(B, S, H, DV)
    f = proj[..., of:of + dqk].reshape(B, S, HK, DK)
    g = -A_log.float().exp().unsqueeze(-1) * F.softplus(f.float() + dt_bias.float())
    b = torch.sigmoid(proj[..., ob:ob + dqk].reshape(B, S, HK, DK)) * erase_scale
    w = torch.sigmoid(proj[..., ow:ow + dv].reshape(B, S, H, DV))
    return q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), b.contiguous(), w.contiguous(), new_conv


def layer_back_chain(o, proj, norm_weight, off_gate, eps):
    """Torch-operator form of ``gdn2_layer_back``: per-head RMSNorm times SiLU(o_gate)."""
    import torch.nn.functional as F

    B, S, H, DV = o.shape
    gate = proj[..., off_gate:off_gate + H * DV].reshape(B, S, H, DV)
    x = o.float()
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return (x * norm_weight.float() * F.silu(gate.float())).to(gate.dtype).reshape(B, S, H * DV)
