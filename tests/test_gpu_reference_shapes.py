"""The GPU test shapes of the reference's own test-suite, carried over (tests/test_gdn2.py:226-266 and
tests/test_inference.py:181-230 of the reference project): bf16 / fp16 chunkwise forward against the token
recurrence at (2,512,4,64,64), (1,1024,8,128,128) and (2,320,2,64,128) (DK != DV), the single-step decode
loop, prefill with and without a ragged tail, and the peak-memory property of the fused prefill (no
[B, NC, H, DK, DV] array). Tolerances are the reference's own: 3e-2 (bf16) / 1e-2 (fp16) of the largest value.
"""

from __future__ import annotations

import pytest
import torch

import gdn2_tilelang_b200 as gdn2
from gdn2_tilelang_b200 import _cabi
from oracle import gdn2_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def inputs(B, S, H, DK, DV, seed=0):
    return orc.make_inputs(B, S, H, DK, DV, seed=seed, gate="softplus")


def state0(B, H, DK, DV):
    return torch.randn(B, H, DK, DV, generator=torch.Generator().manual_seed(99)) * 0.2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,DK,DV", [(2, 512, 4, 64, 64), (1, 1024, 8, 128, 128), (2, 320, 2, 64, 128)])
def test_kernel_matches_reference(dtype, B, S, H, DK, DV):
    q, k, v, g, b, w = inputs(B, S, H, DK, DV)
    s0 = state0(B, H, DK, DV)
    o_ref, s_ref = orc.recurrence(q, k, v, g, b, w, None, s0)
    o, s = gdn2.chunk_gdn2_fwd(*(t.to(dtype).to(DEV) for t in (q, k, v)), g.to(DEV), b.to(dtype).to(DEV), w.to(dtype).to(DEV),
                               scale=DK**-0.5, initial_state=s0.to(DEV), output_final_state=True)
    _cabi.kernels().check_device_status()
    tol = 3e-2 if dtype is torch.bfloat16 else 1e-2
    assert o.dtype == dtype
    assert orc.rel_max_err(o.float().cpu(), o_ref) < tol
    assert orc.rel_max_err(s.cpu(), s_ref) < tol


def test_kernel_decode_step_matches_reference():
    q, k, v, g, b, w = inputs(2, 8, 4, 64, 64)
    s0 = state0(2, 4, 64, 64)
    o_ref, _ = orc.recurrence(q, k, v, g, b, w, None, s0)
    state = s0.to(DEV)
    outs = [gdn2.gdn2_decode_step(q[:, t].bfloat16().to(DEV), k[:, t].bfloat16().to(DEV), v[:, t].bfloat16().to(DEV),
                                  g[:, t].to(DEV), b[:, t].bfloat16().to(DEV), w[:, t].bfloat16().to(DEV), state).float()
            for t in range(8)]
    assert orc.rel_max_err(torch.stack(outs, 1).cpu(), o_ref) < 3e-2


@pytest.mark.parametrize("S", [512, 1000])
def test_prefill_kernel_matches_reference(S):
    q, k, v, g, b, w = inputs(2, S, 4, 64, 64)
    s0 = state0(2, 4, 64, 64)
    o_ref, s_ref = orc.recurrence(q, k, v, g, b, w, 64**-0.5, s0)
    o, state = gdn2.gdn2_prefill(*(t.bfloat16().to(DEV) for t in (q, k, v)), g.to(DEV), b.bfloat16().to(DEV),
                                 w.bfloat16().to(DEV), s0.to(DEV), 64**-0.5)
    assert orc.rel_max_err(o.float().cpu(), o_ref) < 3e-2
    assert orc.rel_max_err(state.cpu(), s_ref) < 3e-2


def test_prefill_does_not_allocate_chunk_states():
    """The fused scan keeps the state on chip: the serving prefill's peak memory stays below that of the
    training-style forward with stored chunk states by at least half the size of that array, and above its
    own inputs it holds only the workspace, the output and two states."""
    B, S, H, DK, DV = 2, 2048, 8, 128, 128
    q, k, v, g, b, w = inputs(B, S, H, DK, DV)
    args = [t.bfloat16().to(DEV) for t in (q, k, v)] + [g.to(DEV)] + [t.bfloat16().to(DEV) for t in (b, w)]
    scale = DK**-0.5
    gdn2.gdn2_prefill(*args, scale=scale)                     # library handles, side stream
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    gdn2.chunk_gdn2_fwd(*args, scale=scale, return_chunk_states=True)
    torch.cuda.synchronize()
    peak_train = torch.cuda.max_memory_allocated() - base
    torch.cuda.reset_peak_memory_stats()
    gdn2.gdn2_prefill(*args, scale=scale)
    torch.cuda.synchronize()
    peak_prefill = torch.cuda.max_memory_allocated() - base
    h_bytes = B * (S // 64) * H * DK * DV * 4                 # fp32 per-chunk states
    assert peak_prefill < peak_train - h_bytes * 0.5
    ws = _cabi.kernels().lib.gdn2_prefill_workspace_bytes(B, S, H, H, DK, DV, _cabi.GDN2_BF16, _cabi.PATH_AUTO)
    assert peak_prefill < ws + B * S * H * DV * 2 + 4 * B * H * DK * DV * 4 + (8 << 20)
