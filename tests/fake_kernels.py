"""Test double for ``gdn2_tilelang_b200._cabi.NativeKernels`` backed by the CPU oracle.

Used ONLY by the CPU tests of the host-side logic (tail routing, state ownership, caches, head
sharding): it lets that logic run without a GPU. The product never uses it."""

from __future__ import annotations

import torch

from oracle import gdn2_oracle as orc


class OracleKernels:
    def __init__(self):
        self.calls = []
        self.launches = 0

    def decode(self, q, k, v, g, b, w, state, scale, out=None):
        self.calls.append(("decode", q.shape[1]))
        o = orc.decode(q, k, v, g, b, w, state, scale)
        if out is not None:
            out.copy_(o)
            return out
        return o

    def chunk_forward(self, q, k, v, g, b, w, scale, initial_state=None, want_chunk_states=False,
                      path=None, out=None, out_batch_stride=None):
        self.calls.append(("chunk_forward", q.shape[1]))
        assert q.shape[1] % 64 == 0
        res = orc.chunkwise(q, k, v, g, b, w, scale, initial_state, return_chunk_states=want_chunk_states)
        o, s = res[0].to(v.dtype), res[1]
        if out is not None:
            out[:, : q.shape[1]].copy_(o)
            o = out
        return o, s, (res[2] if want_chunk_states else None)

    def chunk_output(self, q, k, v, g, b, w, scale, chunk_states, path=None):
        f = orc.chunk_factors(q, k, v, g, b, w, scale)
        B, S, H, DK = q.shape
        h = chunk_states.permute(0, 2, 1, 3, 4).float()
        un = f["U"] - f["W"] @ h
        o = f["Qg"] @ h + f["Aqk"] @ un
        return o.permute(0, 2, 3, 1, 4).reshape(B, S, H, -1).to(v.dtype)
