"""``gdn2_prefill_static`` -- the prefill entry point for callers that may not allocate device
memory (a plugin inside an engine that owns all of HBM, a latency-critical loop that cannot take
cudaMalloc's device-wide synchronisation) -- must give exactly what the two-call form
``gdn2_chunk_prep`` + ``gdn2_prefill_scan`` gives with a caller-provided workspace.

Both forms run the same kernels in the same order, so the comparison is bit-exact. Two calls in a
row on different inputs check that whatever one call leaves in the shared static scratch does not
leak into the next. The file name sorts last so that a run stopping at the first failure has
already executed every other test; the test has no dependence on what ran before it.
"""

from __future__ import annotations

import pytest
import torch

from gdn2_tilelang_b200 import _cabi
from oracle import gdn2_oracle as orc

pytestmark = pytest.mark.gpu


def _two_call_form(lib, dev_in, s0, B, S, H, D, code, stream):
    q, k, v, g, b, w = dev_in
    nbytes = lib.gdn2_prefill_workspace_bytes(B, S, H, H, D, D, code, _cabi.PATH_AUTO)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    o = torch.empty(B, S, H, D, dtype=v.dtype, device=q.device)
    fin = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
    rc = lib.gdn2_chunk_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(), w.data_ptr(),
                             ws.data_ptr(), nbytes, B, S, H, H, D, D, S, D**-0.5, code, _cabi.PATH_AUTO, stream)
    assert rc == 0
    rc = lib.gdn2_prefill_scan(ws.data_ptr(), nbytes, s0.data_ptr(), o.data_ptr(), fin.data_ptr(), None,
                               B, S, H, H, D, D, S, code, _cabi.PATH_AUTO, stream)
    assert rc == 0
    return o, fin


def _static_form(lib, dev_in, s0, B, S, H, D, code, stream):
    q, k, v, g, b, w = dev_in
    o = torch.empty(B, S, H, D, dtype=v.dtype, device=q.device)
    fin = torch.empty(B, H, D, D, dtype=torch.float32, device=q.device)
    rc = lib.gdn2_prefill_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                 w.data_ptr(), s0.data_ptr(), o.data_ptr(), fin.data_ptr(), B, S, H, D, D, S, S,
                                 D**-0.5, code, stream)
    assert rc == 0, lib.gdn2_status_string(rc)
    return o, fin


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_prefill_equals_two_call_form(dtype):
    lib = _cabi.load_library()
    dev = torch.device("cuda", 0)
    B, S, H, D = 2, 256, 4, 128            # 32 chunk-heads: well inside the static scratch
    code = _cabi.dtype_code(dtype)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        for seed in (31, 32):              # two calls in a row, different data
            q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=seed)
            dev_in = tuple(t.to(dtype).to(dev) for t in (q, k, v)) + (g.to(dev), b.to(dtype).to(dev), w.to(dtype).to(dev))
            s0 = (torch.randn(B, H, D, D, generator=torch.Generator().manual_seed(seed)) * 0.1).to(dev)
            o_ref, fin_ref = _two_call_form(lib, dev_in, s0, B, S, H, D, code, stream)
            o, fin = _static_form(lib, dev_in, s0, B, S, H, D, code, stream)
            torch.cuda.synchronize(dev)
            assert torch.equal(o, o_ref)
            assert torch.equal(fin, fin_ref)
            # and the result is right, not merely equal: compare with the oracle as the other tests do
            host = tuple(t.float().cpu() for t in dev_in)
            o_orc, s_orc = orc.chunkwise(*host, None, s0.cpu())
            assert orc.max_abs_err(o.float().cpu(), o_orc) < 2e-2
            assert orc.rel_fro_err(fin.cpu(), s_orc) < 1e-3


def test_static_scratch_rejects_oversized_problems():
    lib = _cabi.load_library()
    dev = torch.device("cuda", 0)
    one = torch.zeros(64, device=dev)
    p = one.data_ptr()
    # 4 * 16 * 250 chunk-heads needs ~1.7 GB of scratch: refused before anything is launched
    rc = lib.gdn2_prefill_static(p, p, p, p, p, p, None, p, None, 4, 16000, 16, 128, 128, 16000, 16000,
                                 1.0, _cabi.GDN2_BF16, None)
    assert rc == -9 and b"static" in lib.gdn2_status_string(rc)
    rc = lib.gdn2_prefill_static(p, p, p, p, p, p, None, p, None, 1, 100, 1, 128, 128, 100, 100,
                                 1.0, _cabi.GDN2_BF16, None)
    assert rc == -2                        # S not a multiple of 64 is a shape error, not a size error


def test_static_scratch_limit_is_exact():
    """The largest problem that fits the built-in scratch runs (and equals the two-call form); one chunk more is
    refused with GDN2_ERR_STATIC_LIMIT. One (batch, head) pair, so the scan of the fitting problem is also the
    form that cuts the sequence into segments, whose records live in the same scratch."""
    lib = _cabi.load_library()
    dev = torch.device("cuda", 0)
    code, D = _cabi.GDN2_BF16, 128
    limit = 32 * 1024 * 1024
    nc = max(n for n in range(1, 600) if lib.gdn2_prefill_workspace_bytes(1, 64 * n, 1, 1, D, D, code, _cabi.PATH_AUTO) <= limit)
    assert lib.gdn2_prefill_workspace_bytes(1, 64 * (nc + 1), 1, 1, D, D, code, _cabi.PATH_AUTO) > limit
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        q, k, v, g, b, w = orc.make_inputs(1, 64 * (nc + 1), 1, D, D, seed=33)
        full = tuple(t.bfloat16().to(dev) for t in (q, k, v)) + (g.to(dev), b.bfloat16().to(dev), w.bfloat16().to(dev))
        s0 = torch.zeros(1, 1, D, D, device=dev)
        S = 64 * nc
        fits = tuple(t[:, :S].contiguous() for t in full)
        o_ref, fin_ref = _two_call_form(lib, fits, s0, 1, S, 1, D, code, stream)
        o, fin = _static_form(lib, fits, s0, 1, S, 1, D, code, stream)
        torch.cuda.synchronize(dev)
        assert torch.equal(o, o_ref) and torch.equal(fin, fin_ref)
        o_big = torch.empty(1, S + 64, 1, D, dtype=torch.bfloat16, device=dev)
        rc = lib.gdn2_prefill_static(*(t.data_ptr() for t in full), None, o_big.data_ptr(), None, 1, S + 64, 1, D, D,
                                     S + 64, S + 64, D**-0.5, code, stream)
        assert rc == -9
