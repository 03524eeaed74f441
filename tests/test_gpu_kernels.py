"""Parity of the CUDA kernels (through the C ABI) with the oracle and the golden fixtures.

Tolerances: float32 inputs -> the reference tests' own bounds (rel-max 2e-5 chunkwise, 1e-5 decode);
bf16 inputs -> output max-abs <= 2e-2 and final-state relative Frobenius error <= 1e-3 against the
oracle fed the same bf16-rounded inputs (the acceptance bounds of the benchmark definition)."""

from __future__ import annotations

import pytest
import torch

import gdn2_tilelang_b200 as gdn2
from gdn2_tilelang_b200 import _cabi
from oracle import gdn2_oracle as orc
from tests.conftest import golden_state, load_golden, note
from tests.golden.make_golden import CORE_CASES, DECODE_CASES, PREFILL_CASES

pytestmark = pytest.mark.gpu
DEV = "cuda"
O_ABS_BF16, STATE_FRO = 2e-2, 1e-3


def cuda(*ts):
    return tuple(t.to(DEV) for t in ts)


def bf16_inputs(B, S, H, DK, DV, **kw):
    """bf16-rounded inputs: returns (device bf16 tensors + fp32 g, host fp32 copies of the rounded values)."""
    q, k, v, g, b, w = orc.make_inputs(B, S, H, DK, DV, **kw)
    qh, kh, vh, bh, wh = (t.bfloat16() for t in (q, k, v, b, w))
    dev = (qh.to(DEV), kh.to(DEV), vh.to(DEV), g.to(DEV), bh.to(DEV), wh.to(DEV))
    host = (qh.float(), kh.float(), vh.float(), g, bh.float(), wh.float())
    return dev, host


@pytest.fixture(scope="module")
def K():
    k = _cabi.kernels()
    yield k
    k.check_device_status()


# ---- tensor-core building blocks -------------------------------------------------------------------


def test_tcgen05_selftest(K):
    gen = torch.Generator().manual_seed(0)
    a = torch.randn(128, 64, generator=gen)
    bt = torch.randn(128, 64, generator=gen)
    out = K.selftest_mma(a.to(DEV), bt.to(DEV)).cpu()
    K.check_device_status()
    ref16 = a.bfloat16().float() @ bt.bfloat16().float().T
    ref32 = a.double() @ bt.double().T
    assert orc.rel_max_err(out[0], ref16) < 1e-5          # exact products, fp32 accumulation
    assert orc.rel_max_err(out[1], ref32) < 3e-3          # tf32 operands: 10-bit mantissa
    assert torch.equal(out[2], 2 * out[1] + 1)            # TMEM store/load round trip
    assert torch.equal(out[3], out[0])                    # A operand from tensor memory == from shared memory


# ---- decode ------------------------------------------------------------------------------------------


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_decode_fp32_matches_golden(K, name):
    B, n, H, DK, DV = DECODE_CASES[name]
    gold = load_golden(name)
    ins = orc.make_inputs(B, n, H, DK, DV, seed=1, gate="softplus")
    state = golden_state(B, H, DK, DV, 1, 0.3).to(DEV)
    o = gdn2.gdn2_decode(*cuda(*ins), state)
    assert orc.rel_max_err(o.cpu(), gold["o"]) < 1e-5
    assert orc.rel_max_err(state.cpu(), gold["state"]) < 1e-5


@pytest.mark.parametrize("DK,DV", [(128, 128), (64, 64), (32, 24), (256, 40), (72, 100)])
@pytest.mark.parametrize("n", [1, 8, 37])
def test_decode_bf16_vs_oracle(K, DK, DV, n):
    B, H = 3, 5
    dev, host = bf16_inputs(B, n, H, DK, DV, seed=n, gate="softplus", decay_scale=1.0)
    s0 = golden_state(B, H, DK, DV, n, 0.3)
    state = s0.to(DEV)
    o = gdn2.gdn2_decode(*dev, state)
    s_ref = s0.clone()
    o_ref = orc.decode(*host, s_ref)
    assert o.dtype == torch.bfloat16
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16
    assert orc.rel_fro_err(state.cpu(), s_ref) < 1e-5


def test_decode_multi_equals_repeated_single(K):
    dev, _ = bf16_inputs(4, 12, 16, 128, 128, seed=3)
    s0 = (torch.randn(4, 16, 128, 128, generator=torch.Generator().manual_seed(1)) * 0.02).to(DEV)
    sm = s0.clone()
    om = gdn2.gdn2_decode(*dev, sm)
    s1 = s0.clone()
    o1 = torch.cat([gdn2.gdn2_decode(*(t[:, i:i + 1] for t in dev), s1) for i in range(12)], 1)
    # n >= 4 takes the blocked kernel (sums regrouped), single tokens the sweep kernel: equal up to fp32
    # reassociation, and up to one bf16 step in the rounded outputs
    assert orc.rel_max_err(sm.cpu(), s1.cpu()) < 1e-5
    assert orc.rel_max_err(om.float().cpu(), o1.float().cpu()) < 8e-3
    s3, s4 = s0.clone(), s0.clone()
    o3 = gdn2.gdn2_decode(*(t[:, :3] for t in dev), s3)      # n = 3: the sweep kernel, bit-exact with single steps
    o4 = torch.cat([gdn2.gdn2_decode(*(t[:, i:i + 1] for t in dev), s4) for i in range(3)], 1)
    assert torch.equal(o3, o4) and torch.equal(s3, s4)
    st = s0.clone()
    os_ = gdn2.gdn2_decode_step(*(t[:, 0] for t in dev), st)
    assert torch.equal(os_, o1[:, 0])


@pytest.mark.parametrize("n", [4, 5, 9, 16, 23])
@pytest.mark.parametrize("decay_scale", [1.0, 40.0])
def test_decode_blocked_lengths_and_fast_decay_fp32(K, n, decay_scale):
    """n >= 4 at DK = DV = 128 takes the blocked kernel: every block length, padded last blocks, and gates
    strong enough that a factorised decay would overflow (here every ratio stays <= 1)."""
    B, H, D = 2, 3, 128
    ins = orc.make_inputs(B, n, H, D, D, seed=40 + n, gate="softplus", decay_scale=decay_scale)
    s0 = golden_state(B, H, D, D, n, 0.3)
    state = s0.to(DEV)
    o = gdn2.gdn2_decode(*cuda(*ins), state)
    s_ref = s0.clone()
    o_ref = orc.decode(*ins, s_ref)
    assert torch.isfinite(o).all() and torch.isfinite(state).all()
    assert orc.rel_max_err(o.cpu(), o_ref) < 2e-5
    assert orc.rel_max_err(state.cpu(), s_ref) < 2e-5


def test_decode_zero_gates_only_decay(K):
    dev, host = bf16_inputs(2, 9, 4, 128, 128, seed=5)
    q, k, v, g, b, w = dev
    s0 = golden_state(2, 4, 128, 128, 9, 1.0)
    st = s0.to(DEV)
    gdn2.gdn2_decode(q, k, v, g, torch.zeros_like(b), torch.zeros_like(w), st)
    want = s0 * host[3].sum(dim=1).exp().unsqueeze(-1)
    assert orc.rel_max_err(st.cpu(), want) < 1e-5


# ---- chunkwise forward, SIMT family (float32 inputs) ---------------------------------------------------


@pytest.mark.parametrize("name", sorted(CORE_CASES))
def test_chunk_forward_fp32_matches_golden(K, name):
    B, S, H, DK, DV, gate, ds, with_s0 = CORE_CASES[name]
    gold = load_golden(name)
    ins = orc.make_inputs(B, S, H, DK, DV, seed=0, gate=gate, decay_scale=ds)
    s0 = golden_state(B, H, DK, DV, 0, 0.5).to(DEV) if with_s0 else None
    o, s, h = gdn2.chunk_gdn2_fwd(*cuda(*ins), DK**-0.5, s0, True, return_chunk_states=True)
    tol = 1e-4 if ds >= 8 else 2e-5
    assert o.dtype == torch.float32
    assert orc.rel_max_err(o.cpu(), gold["o_recurrent"]) < tol
    assert orc.rel_max_err(s.cpu(), gold["s_recurrent"]) < tol
    assert torch.isfinite(o).all()
    if "f_h" in gold:
        assert orc.rel_max_err(h.cpu().permute(0, 2, 1, 3, 4), gold["f_h"]) < tol
    o2 = gdn2.chunk_gdn2_output(*cuda(*ins), DK**-0.5, h)
    assert orc.rel_max_err(o2.cpu(), o.cpu()) < 1e-5


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_fp32_matches_golden(K, name):
    B, S, H, DK, DV = PREFILL_CASES[name]
    gold = load_golden(name)
    ins = orc.make_inputs(B, S, H, DK, DV, seed=2, gate="softplus")
    s0 = golden_state(B, H, DK, DV, 2, 0.3).to(DEV)
    o, state = gdn2.gdn2_prefill(*cuda(*ins), s0.clone())
    assert o.shape == (B, S, H, DV)
    assert orc.rel_max_err(o.cpu(), gold["o"]) < 2e-5
    assert orc.rel_max_err(state.cpu(), gold["state"]) < 2e-5


@pytest.mark.parametrize("decay_scale", [0.0, 1.0, 8.0, 30.0])
def test_fast_decay_stays_finite(K, decay_scale):
    ins = orc.make_inputs(1, 128, 2, 32, 32, gate="softplus", decay_scale=decay_scale)
    o_ref, _ = orc.recurrence(*ins)
    o, _ = gdn2.gdn2_attention(*cuda(*ins))
    assert torch.isfinite(o).all()
    assert orc.rel_max_err(o.cpu(), o_ref) < 1e-4


def test_attention_cfg0_matches_reference_torch_backend(K):
    gold = load_golden("cfg0_b1_s256_h4_d64")
    ins = orc.make_inputs(1, 256, 4, 64, 64, seed=0)
    o, s = gdn2.gdn2_attention(*cuda(*ins), output_final_state=True)
    assert orc.rel_max_err(o.cpu(), gold["o_attention"]) < 2e-5
    assert orc.rel_max_err(s.cpu(), gold["s_attention"]) < 2e-5


# ---- chunkwise forward, D = 128 bf16: both kernel families --------------------------------------------


def _run_paths(K, dev, s0, paths=("simt", "tcgen05")):
    out = {}
    for p in paths:
        o, s, h = K.chunk_forward(*dev, 128**-0.5, s0, want_chunk_states=True, path=p)
        K.check_device_status()
        out[p] = (o.float().cpu(), s.cpu(), h.cpu())
    return out


@pytest.mark.parametrize("variant", ["gdn2", "kda", "gdn"])
def test_d128_bf16_both_families_vs_oracle(K, variant):
    B, S, H, D = 2, 512, 4, 128
    q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=11)
    if variant in ("kda", "gdn"):
        w = b.clone()                                    # tied erase / write gates
    if variant == "gdn":
        g = g[..., :1].expand(-1, -1, -1, D).contiguous()  # one decay per head
    host = tuple(t.bfloat16().float() for t in (q, k, v)) + (g, b.bfloat16().float(), w.bfloat16().float())
    dev = tuple(t.bfloat16().to(DEV) for t in (q, k, v)) + (g.to(DEV), b.bfloat16().to(DEV), w.bfloat16().to(DEV))
    s0 = golden_state(B, H, D, D, 11, 0.1)
    o_ref, s_ref, h_ref = orc.chunkwise(*host, None, s0, return_chunk_states=True)
    res = _run_paths(K, dev, s0.to(DEV))
    for p, (o, s, h) in res.items():
        assert orc.max_abs_err(o, o_ref) < O_ABS_BF16, p
        assert orc.rel_fro_err(s, s_ref) < STATE_FRO, p
        assert orc.rel_fro_err(h, h_ref) < STATE_FRO, p
    assert orc.max_abs_err(res["simt"][0], res["tcgen05"][0]) < O_ABS_BF16


def test_d128_golden_case_tcgen05(K):
    gold = load_golden("d128_s128_h2")
    q, k, v, g, b, w = orc.make_inputs(1, 128, 2, 128, 128, seed=0)
    dev = tuple(t.bfloat16().to(DEV) for t in (q, k, v)) + (g.to(DEV), b.bfloat16().to(DEV), w.bfloat16().to(DEV))
    s0 = golden_state(1, 2, 128, 128, 0, 0.5).to(DEV)
    o, s, _ = K.chunk_forward(*dev, 128**-0.5, s0, path="tcgen05")
    K.check_device_status()
    # golden outputs come from unrounded fp32 inputs, so allow the bf16 input rounding on top
    assert orc.max_abs_err(o.float().cpu(), gold["o_recurrent"]) < 3e-2
    assert orc.rel_fro_err(s.cpu(), gold["s_recurrent"]) < 1e-2


def test_prefill_ragged_d128_bf16(K):
    B, S, H, D = 2, 64 * 5 + 37, 3, 128
    dev, host = bf16_inputs(B, S, H, D, D, seed=13)
    o, state = gdn2.gdn2_prefill(*dev)
    o_ref, s_ref = orc.prefill(*host)
    assert o.shape == (B, S, H, D) and o.dtype == torch.bfloat16
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16
    assert orc.rel_fro_err(state.cpu(), s_ref) < STATE_FRO


def test_prefill_from_host_streams_sequences(K):
    B, S, H, D = 3, 64 * 6 + 21, 4, 128
    dev, host = bf16_inputs(B, S, H, D, D, seed=15)
    s0 = torch.randn(B, H, D, D, device="cuda") * 0.1
    o_ref, s_ref = gdn2.gdn2_prefill(*dev, s0)
    pinned = [t.cpu().pin_memory() for t in dev]
    o, s = gdn2.gdn2_prefill_from_host(*pinned, s0.cpu())
    torch.cuda.synchronize()
    assert o.device.type == "cpu" and o.is_pinned() and s.is_cuda
    assert torch.equal(o, o_ref.cpu())                       # same kernels on the same values
    assert torch.equal(s, s_ref)
    o2, s2 = gdn2.gdn2_prefill_from_host(*pinned)            # no initial state
    o_ref2, s_ref2 = gdn2.gdn2_prefill(*dev)
    torch.cuda.synchronize()
    assert torch.equal(o2, o_ref2.cpu()) and torch.equal(s2, s_ref2)
    K.check_device_status()


def test_prefill_on_a_side_stream_matches_default_stream(K):
    """The calls launch on the caller's current stream (and, for long prompts, hand the scan of one sequence
    segment to an internal stream): results on a user stream equal those on the default stream, and work
    queued behind the call on that stream sees the finished outputs."""
    B, S, H, D = 2, 64 * 40 + 9, 4, 128
    dev, _ = bf16_inputs(B, S, H, D, D, seed=23)
    o_ref, s_ref = gdn2.gdn2_prefill(*dev)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        o, st = gdn2.gdn2_prefill(*dev)
        total = o.float().sum() + st.sum()                 # consumer queued right behind the call
    side.synchronize()
    assert torch.equal(o, o_ref) and torch.equal(st, s_ref)
    assert torch.equal(total, o_ref.float().sum() + s_ref.sum())
    K.check_device_status()


def test_prefill_from_host_cuts_long_sequences(K):
    """Sequences of 8192+ tokens travel in several units with the state chained between them."""
    B, S, H, D = 2, 64 * 64 * 2 + 21, 2, 128
    dev, _ = bf16_inputs(B, S, H, D, D, seed=16)
    o_ref, s_ref = gdn2.gdn2_prefill(*dev)
    o, s = gdn2.gdn2_prefill_from_host(*[t.cpu().pin_memory() for t in dev])
    torch.cuda.synchronize()
    # with so few (batch, head) pairs the scan cuts a sequence into segments, differently for a unit than for the
    # whole: equal up to the rounding of the state hand-over between segments, not bit for bit
    assert orc.max_abs_err(o.float(), o_ref.float().cpu()) < 8e-3 and float((o.float() - o_ref.float().cpu()).abs().mean()) < 1e-5
    assert orc.rel_fro_err(s, s_ref) < 1e-4
    K.check_device_status()


@pytest.mark.parametrize("D", [64, 128])
def test_fp16_inputs_prefill_and_decode(K, D):
    """fp16 tensors (the third dtype the reference accepts) go through the SIMT family with fp32 records."""
    B, S, H = 2, 64 * 3 + 11, 3
    q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=31, gate="softplus")
    host = tuple(t.half().float() for t in (q, k, v)) + (g, b.half().float(), w.half().float())
    dev = tuple(t.half().to(DEV) for t in (q, k, v)) + (g.to(DEV), b.half().to(DEV), w.half().to(DEV))
    o, state = gdn2.gdn2_prefill(*dev)
    o_ref, s_ref = orc.prefill(*host)
    assert o.dtype == torch.float16
    assert orc.max_abs_err(o.float().cpu(), o_ref) < 5e-3          # fp16 output rounding only
    assert orc.rel_fro_err(state.cpu(), s_ref) < 1e-4
    st = state.clone()
    o2 = gdn2.gdn2_decode(*(t[:, :9] for t in dev), st)
    s2 = s_ref.clone()
    o2_ref = orc.decode(*(t[:, :9] for t in host), s2)
    assert o2.dtype == torch.float16
    assert orc.max_abs_err(o2.float().cpu(), o2_ref) < 5e-3
    assert orc.rel_fro_err(st.cpu(), s2) < 1e-4


@pytest.mark.parametrize("decay_scale", [1.5, 2.5, 3.5, 5.0, 6.5, 9.0])
def test_decay_spans_around_the_tensor_core_limit(K, decay_scale):
    """Sub-block decay from well inside the factorised range through its limit (2^96 per half sub-block) to chunks
    that are flagged and redone exactly: all within the bf16 bounds against the recurrence."""
    dev, host = bf16_inputs(2, 64 * 6, 3, 128, 128, seed=19, gate="softplus", decay_scale=decay_scale)
    o_ref, s_ref = orc.recurrence(*host)
    o, s = gdn2.gdn2_attention(*dev, output_final_state=True)
    assert torch.isfinite(o).all() and torch.isfinite(s).all()
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16
    assert orc.rel_fro_err(s.cpu(), s_ref) < 2e-3          # states this decayed are a few tokens of history only
    K.check_device_status()


def test_fast_decay_d128_bf16_takes_exact_path(K):
    dev, host = bf16_inputs(1, 128, 2, 128, 128, seed=17, gate="softplus", decay_scale=30.0)
    o_ref, s_ref = orc.recurrence(*host)
    o, s = gdn2.gdn2_attention(*dev, output_final_state=True)
    assert torch.isfinite(o).all()
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16


# ---- size-independent properties at benchmark-like sizes ---------------------------------------------


def test_large_segmented_prefill_and_linearity(K):
    B, S, H, D = 2, 64 * 40 + 37, 16, 128
    dev, _ = bf16_inputs(B, S, H, D, D, seed=21)
    q, k, v, g, b, w = dev
    o_all, s_all = gdn2.gdn2_prefill(*dev)
    outs, state = [], None
    for lo, hi in ((0, 64 * 10), (64 * 10, 64 * 25 + 5), (64 * 25 + 5, S)):
        o, state = gdn2.gdn2_prefill(*(t[:, lo:hi] for t in dev), state)
        outs.append(o)
    assert orc.max_abs_err(torch.cat(outs, 1).float(), o_all.float()) < O_ABS_BF16
    assert orc.rel_fro_err(state, s_all) < STATE_FRO
    # with a zero initial state the output is linear in v
    o2, s2 = gdn2.gdn2_prefill(q, k, (2 * v.float()).bfloat16(), g, b, w)
    assert orc.max_abs_err(o2.float(), 2 * o_all.float()) < 2 * O_ABS_BF16
    assert orc.rel_fro_err(s2, 2 * s_all) < STATE_FRO
    K.check_device_status()


def test_zero_gates_only_decay_large(K):
    B, S, H, D = 1, 64 * 8, 16, 128
    dev, host = bf16_inputs(B, S, H, D, D, seed=23)
    q, k, v, g, b, w = dev
    s0 = golden_state(B, H, D, D, 23, 1.0)
    _, s = gdn2.gdn2_attention(q, k, v, g, torch.zeros_like(b), torch.zeros_like(w),
                               initial_state=s0.to(DEV), output_final_state=True)
    want = s0 * host[3].sum(dim=1).exp().unsqueeze(-1)
    assert orc.rel_fro_err(s.cpu(), want) < STATE_FRO


# ---- chunk-local intermediates against the stored intermediates of the reference ------------------------


def test_workspace_records_match_reference_intermediates(K):
    """The records the chunk-local stage hands to the scan, de-scaled, against (a) the oracle's factors on the
    same bf16-rounded inputs and (b) the reference's own forward_intermediates stored in the golden file (those
    come from unrounded fp32 inputs, so the bf16 input rounding is allowed on top)."""
    from tests.ws_records import decode_tc_workspace

    B, S, H, D = 1, 128, 2, 128
    gold = load_golden("d128_s128_h2")
    q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=0)
    host = tuple(t.bfloat16().float() for t in (q, k, v)) + (g, b.bfloat16().float(), w.bfloat16().float())
    dev = tuple(t.bfloat16().to(DEV) for t in (q, k, v)) + (g.to(DEV), b.bfloat16().to(DEV), w.bfloat16().to(DEV))
    ws, p = K.chunk_prep(*dev, D**-0.5, path="tcgen05")
    K.check_device_status()
    rec = decode_tc_workspace(ws, K.workspace_layout(B, S, H, D, D, torch.bfloat16, p), B, S, H)
    assert int(rec["flags"].sum()) == 0
    f = orc.chunk_factors(*host)
    # relative to the largest entry of each matrix: bf16 records carry 8 bits, fp16 ones 11
    tight = {"Aqk": 5e-3, "W": 8e-3, "Qg": 6e-3, "U": 4e-3, "KG": 2e-3, "gamma_last": 1e-5}   # Aqk, W: bf16 operands
    for name, tol in tight.items():
        assert orc.rel_max_err(rec[name], f[name]) < tol, name
    for mine, theirs in (("Aqk", "Aqk"), ("W", "W"), ("U", "U"), ("KG", "Ktail")):
        assert orc.rel_max_err(rec[mine], gold[f"f_{theirs}"]) < 2e-2, mine


def test_burst_decay_across_sub_block_references(K):
    """Two decay steps of about 2^-90 placed right after the reference row of one 16-token sub-block and right
    before the reference row of the next, no decay elsewhere: every half sub-block stays inside the factorised
    range, but consecutive reference rows are about 2^-180 apart. Keys between the two steps still pair with
    the rows before the second step through factors that are normal numbers; they must not vanish."""
    B, S, H, D = 1, 128, 2, 128
    q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=29)
    big = -90.0 * 0.6931471805599453
    for per_head in (False, True):
        g2 = torch.zeros_like(g)
        g2[:, 16 + 9] = big              # sub-block 1: rows 0..8 at G = 0, rows 9..15 at -90 (log2)
        g2[:, 32 + 8] = big              # sub-block 2: rows 0..7 at -90, rows 8.. at -180
        g2[:, 64 + 32 + 9] = big         # the same pattern in the second chunk, one sub-block later
        g2[:, 64 + 48 + 8] = big
        if not per_head:                 # per-channel variant: only half of the channels burst
            g2[..., ::2] = 0.0
        host = tuple(t.bfloat16().float() for t in (q, k, v)) + (g2, b.bfloat16().float(), w.bfloat16().float())
        dev = tuple(t.bfloat16().to(DEV) for t in (q, k, v)) + (g2.to(DEV), b.bfloat16().to(DEV), w.bfloat16().to(DEV))
        o_ref, s_ref = orc.recurrence(*host)
        res = _run_paths(K, dev, None)
        for p, (o, s, _) in res.items():
            assert torch.isfinite(o).all(), p
            assert orc.max_abs_err(o, o_ref) < O_ABS_BF16, (p, per_head)
            assert orc.rel_fro_err(s, s_ref) < STATE_FRO, (p, per_head)
        from tests.ws_records import decode_tc_workspace
        ws, p = K.chunk_prep(*dev, D**-0.5, path="tcgen05")
        rec = decode_tc_workspace(ws, K.workspace_layout(B, S, H, D, D, torch.bfloat16, p), B, S, H)
        assert int(rec["flags"].sum()) == 0          # the tensor-core path itself handled these chunks
        f = orc.chunk_factors(*host)
        assert orc.rel_max_err(rec["Aqk"], f["Aqk"]) < 5e-3, per_head


# ---- chunk-parallel output on the tensor-core family -------------------------------------------------------


def test_chunk_output_tcgen05_vs_oracle(K):
    """gdn2_chunk_output on the 16-bit workspace (tcgen05 products) from stored chunk states: against the
    oracle's outputs, and from the ORACLE's chunk states, so the check does not lean on this library's scan."""
    B, S, H, D = 2, 64 * 24, 3, 128
    dev, host = bf16_inputs(B, S, H, D, D, seed=37)
    s0 = golden_state(B, H, D, D, 37, 0.1)
    o_ref, _, h_ref = orc.chunkwise(*host, None, s0, return_chunk_states=True)
    o = K.chunk_output(*dev, D**-0.5, h_ref.to(DEV), path="tcgen05")
    K.check_device_status()
    assert o.dtype == torch.bfloat16
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16
    o_simt = K.chunk_output(*dev, D**-0.5, h_ref.to(DEV), path="simt")
    assert orc.max_abs_err(o_simt.float().cpu(), o_ref) < O_ABS_BF16


# ---- the scan cut into sequence segments ------------------------------------------------------------------


@pytest.mark.parametrize("B,H,NC,decay", [(1, 2, 40, "bench"), (2, 4, 72, "bench"), (1, 1, 130, "bench"),
                                          (1, 2, 40, "slow"), (2, 2, 64, "none"), (4, 2, 250, "bench"),
                                          (4, 16, 100, "bench"), (4, 16, 100, "slow"), (2, 16, 120, "bench"),
                                          (2, 16, 120, "none")])
def test_scan_cut_into_segments_matches_one_block_walk_and_oracle(K, B, H, NC, decay):
    """Few (batch, head) pairs: the scan cuts the sequence (transition matrices + correction pass). Against the
    one-block-per-head walk of the same workspace and against the oracle, for gates that let the carried state
    vanish within a few chunks ("bench"), that keep it alive across whole segments ("slow": the correction pass
    redoes everything) and for no decay at all."""
    S, D = 64 * NC, 128
    q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=41 + NC)
    if decay == "slow":
        g = g / 64.0
    elif decay == "none":
        g = torch.zeros_like(g)
    host = tuple(t.bfloat16().float() for t in (q, k, v)) + (g, b.bfloat16().float(), w.bfloat16().float())
    dev = tuple(t.bfloat16().to(DEV) for t in (q, k, v)) + (g.to(DEV), b.bfloat16().to(DEV), w.bfloat16().to(DEV))
    s0 = golden_state(B, H, D, D, 41, 0.1)
    assert K.scan_segments(B, S, H, D, D, torch.bfloat16, _cabi.PATH_TCGEN05) > 1
    assert K.scan_segments(B, S, H, D, D, torch.bfloat16, _cabi.PATH_TCGEN05_SERIAL) == 1
    o_cut, s_cut, _ = K.chunk_forward(*dev, D**-0.5, s0.to(DEV), path="tcgen05")
    o_one, s_one, _ = K.chunk_forward(*dev, D**-0.5, s0.to(DEV), path="tcgen05_serial")
    K.check_device_status()
    o_ref, s_ref = orc.chunkwise(*host, None, s0)
    e = dict(o_cut=orc.max_abs_err(o_cut.float().cpu(), o_ref), s_cut=orc.rel_fro_err(s_cut.cpu(), s_ref),
             o_one=orc.max_abs_err(o_one.float().cpu(), o_ref), s_one=orc.rel_fro_err(s_one.cpu(), s_ref),
             o_cut_vs_one=orc.max_abs_err(o_cut.float(), o_one.float()),
             o_cut_vs_one_mean=float((o_cut.float() - o_one.float()).abs().mean()),
             s_cut_vs_one=orc.rel_fro_err(s_cut, s_one))
    note("scan_cut", B=B, H=H, NC=NC, decay=decay, **e)
    # without decay nothing forgets the bf16 rounding of the state operand: both forms drift alike
    s_tol = STATE_FRO if decay == "bench" else 4e-3
    assert e["o_cut"] < O_ABS_BF16 and e["o_one"] < O_ABS_BF16
    assert e["s_cut"] < s_tol and e["s_one"] < s_tol
    # the two forms differ only by the rounding of the state hand-over between segments: at most one bf16
    # step on single outputs, nothing on average
    assert e["o_cut_vs_one"] < O_ABS_BF16 and e["o_cut_vs_one_mean"] < 5e-4
    assert e["s_cut_vs_one"] < s_tol


def test_host_cut_prefill_three_segments_equals_one(K, monkeypatch):
    """The host-side cut (chunk-local stage of one segment overlapping the scan of the previous one on a side
    stream) with three segments: bit-equal to the uncut evaluation, repeatedly, with allocations in between."""
    B, S, H, D = 5, 64 * 64, 16, 128          # 80 (batch, head) pairs: the scan itself stays one block per pair
    dev, _ = bf16_inputs(B, S, H, D, D, seed=43)
    assert K.scan_segments(B, S, H, D, D, torch.bfloat16, _cabi.PATH_TCGEN05) == 1
    monkeypatch.setenv("GDN2_B200_PREFILL_SEGMENTS", "1")
    o1, s1 = gdn2.gdn2_prefill(*dev)
    monkeypatch.setenv("GDN2_B200_PREFILL_SEGMENTS", "3")
    for _ in range(3):
        o3, s3 = gdn2.gdn2_prefill(*dev)
        junk = torch.full((1 << 22,), 7.0, device=DEV)      # reuses freed blocks of the caching allocator
        assert torch.equal(o3, o1) and torch.equal(s3, s1)
        del junk
    K.check_device_status()


# ---- failure path and out-of-bounds guards ---------------------------------------------------------------


def test_bounded_wait_runs_out_and_reports(K):
    """A wait that nothing satisfies gives up after its limit, the kernel returns, the status word says so once,
    and the device keeps working."""
    K.check_device_status()                                   # clean before
    gave_up = K.selftest_wait(200_000)                        # about 0.1 ms
    assert gave_up == 64
    with pytest.raises(_cabi.GDN2KernelError, match="bounded wait"):
        K.check_device_status()
    K.check_device_status()                                   # the word was cleared by the failed check
    dev, host = bf16_inputs(1, 128, 2, 128, 128, seed=47)
    o, _ = gdn2.gdn2_prefill(*dev)
    o_ref, _ = orc.prefill(*host)
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16
    K.check_device_status()


def _guarded(shape, dtype, guard=4096):
    """A tensor of `shape` carved out of a larger buffer with `guard` bytes of 0xA5 on both sides."""
    n = 1
    for x in shape:
        n *= x
    esz = torch.empty((), dtype=dtype).element_size()
    buf = torch.full((2 * guard + n * esz,), 0xA5, dtype=torch.uint8, device=DEV)
    view = buf[guard: guard + n * esz].view(dtype).reshape(shape)
    return buf, view, guard


def _guards_intact(buf, guard):
    return bool((buf[:guard] == 0xA5).all()) and bool((buf[-guard:] == 0xA5).all())


@pytest.mark.parametrize("H,NC", [(3, 5), (2, 40)])
def test_kernels_stay_inside_their_buffers(K, H, NC):
    """Guard bytes around the workspace, the outputs and the states of every kernel family stay untouched
    (stand-in for a memory checker): chunk-local stage, scan (one block per head and cut), chunk output, decode."""
    B, D = 2, 128
    S = 64 * NC
    dev, _ = bf16_inputs(B, S, H, D, D, seed=53)
    code = _cabi.GDN2_BF16
    st = torch.cuda.current_stream().cuda_stream
    for path in (_cabi.PATH_TCGEN05, _cabi.PATH_TCGEN05_SERIAL, _cabi.PATH_SIMT):
        nbytes = K.lib.gdn2_prefill_workspace_bytes(B, S, H, H, D, D, code, path)
        wbuf, ws, gd = _guarded((nbytes,), torch.uint8)
        obuf, o, _ = _guarded((B, S, H, D), torch.bfloat16)
        sbuf, sT, _ = _guarded((B, H, D, D), torch.float32)
        hbuf, hs, _ = _guarded((B, NC, H, D, D), torch.float32)
        ptrs = [t.data_ptr() for t in dev]
        assert K.lib.gdn2_chunk_prep(*ptrs, ws.data_ptr(), nbytes, B, S, H, H, D, D, S, D**-0.5, code, path, st) == 0
        assert K.lib.gdn2_prefill_scan(ws.data_ptr(), nbytes, None, o.data_ptr(), sT.data_ptr(), None,
                                       B, S, H, H, D, D, S, code, path, st) == 0
        assert K.lib.gdn2_prefill_scan(ws.data_ptr(), nbytes, None, o.data_ptr(), sT.data_ptr(), hs.data_ptr(),
                                       B, S, H, H, D, D, S, code, path, st) == 0
        assert K.lib.gdn2_chunk_output(ws.data_ptr(), nbytes, hs.data_ptr(), o.data_ptr(), B, S, H, H, D, D, S,
                                       code, path, st) == 0
        torch.cuda.synchronize()
        for name, buf in (("workspace", wbuf), ("o", obuf), ("state", sbuf), ("chunk states", hbuf)):
            assert _guards_intact(buf, gd), (path, name)
    for n in (1, 8, 13):
        sbuf, state, gd = _guarded((B, H, D, D), torch.float32)
        state.zero_()
        obuf, o, _ = _guarded((B, n, H, D), torch.bfloat16)
        ptrs = [t[:, :n].contiguous() for t in dev]
        assert K.lib.gdn2_decode(*(t.data_ptr() for t in ptrs), state.data_ptr(), o.data_ptr(), B, n, H, H, D, D, n, n,
                                 D**-0.5, code, st) == 0
        torch.cuda.synchronize()
        assert _guards_intact(sbuf, gd) and _guards_intact(obuf, gd), n
    K.check_device_status()


def test_packed_variable_length_batch_on_device(K):
    """cu_seqlens on the device kernels (D = 128 bf16, the tensor-core family): every packed sequence against the
    oracle on its slice, and the packed call against the same sequences evaluated one call each."""
    offs = [0, 64 * 9 + 5, 64 * 9 + 5, 64 * 30, 64 * 30 + 17, 64 * 41 + 3]
    H, D = 3, 128
    dev, host = bf16_inputs(1, offs[-1], H, D, D, seed=61)
    s0 = golden_state(5, H, D, D, 61, 0.1)
    o, s = gdn2.gdn2_attention(*dev, initial_state=s0.to(DEV), output_final_state=True, cu_seqlens=offs)
    K.check_device_status()
    for i, (lo, hi) in enumerate(zip(offs, offs[1:])):
        if hi == lo:
            assert torch.equal(s[i].cpu(), s0[i])
            continue
        # (a copy: for a prompt shorter than a chunk the oracle, like the reference, updates the state it is given)
        o_ref, s_ref = orc.prefill(*(t[:, lo:hi] for t in host), s0[i:i + 1].clone())
        assert orc.max_abs_err(o[:, lo:hi].float().cpu(), o_ref) < O_ABS_BF16, i
        assert orc.rel_fro_err(s[i:i + 1].cpu(), s_ref) < STATE_FRO, i
        o_one, s_one = gdn2.gdn2_attention(*(t[:, lo:hi].contiguous() for t in dev), initial_state=s0[i:i + 1].to(DEV),
                                           output_final_state=True)
        assert torch.equal(o[:, lo:hi], o_one) and torch.equal(s[i:i + 1], s_one)


# ---- grouped-query heads: key heads indexed by the kernels, nothing repeated in memory ------------------------


def _gqa_inputs(B, S, H, HK, D, seed, dtype=torch.bfloat16):
    """q, k, b, g with HK heads, v, w with H heads; returns (device tensors, the same with key heads repeated,
    host fp32 copies of the repeated form for the oracle)."""
    q, k, _, g, b, _ = orc.make_inputs(B, S, HK, D, D, seed=seed)
    _, _, v, _, _, w = orc.make_inputs(B, S, H, D, D, seed=seed + 1)
    lo = [t.to(dtype) for t in (q, k, v, b, w)]
    dev = (lo[0].to(DEV), lo[1].to(DEV), lo[2].to(DEV), g.to(DEV), lo[3].to(DEV), lo[4].to(DEV))
    rep = H // HK
    ex = lambda t: t.repeat_interleave(rep, dim=2)     # noqa: E731
    dev_rep = (ex(dev[0]), ex(dev[1]), dev[2], ex(dev[3]), ex(dev[4]), dev[5])
    host = (ex(lo[0]).float(), ex(lo[1]).float(), lo[2].float(), ex(g), ex(lo[3]).float(), lo[4].float())
    return dev, dev_rep, host


@pytest.mark.parametrize("H,HK,D,path", [(4, 2, 128, "tcgen05"), (6, 2, 128, "tcgen05"), (4, 1, 128, "tcgen05"),
                                         (2, 1, 128, "tcgen05"), (16, 8, 128, "tcgen05"),
                                         (4, 2, 128, "simt"), (6, 3, 64, "simt")])
def test_grouped_query_heads_chunkwise(K, H, HK, D, path):
    """Fewer key heads than value heads through the chunkwise kernels: bit-equal to the same call on repeated key
    heads (the arithmetic per value head is the same, only done once per key head), right against the oracle,
    chunk states and the chunk-parallel output included."""
    B, S = 2, 64 * 24
    dev, dev_rep, host = _gqa_inputs(B, S, H, HK, D, seed=67)
    s0 = golden_state(B, H, D, D, 67, 0.1)
    o, s, h = K.chunk_forward(*dev, D**-0.5, s0.to(DEV), want_chunk_states=True, path=path)
    o_r, s_r, h_r = K.chunk_forward(*dev_rep, D**-0.5, s0.to(DEV), want_chunk_states=True, path=path)
    K.check_device_status()
    assert torch.equal(o, o_r) and torch.equal(s, s_r) and torch.equal(h, h_r)
    o_ref, s_ref, h_ref = orc.chunkwise(*host, None, s0, return_chunk_states=True)
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16
    assert orc.rel_fro_err(s.cpu(), s_ref) < STATE_FRO and orc.rel_fro_err(h.cpu(), h_ref) < STATE_FRO
    o2 = K.chunk_output(*dev, D**-0.5, h, path=path)
    assert orc.max_abs_err(o2.float().cpu(), o_ref) < O_ABS_BF16
    if path == "tcgen05":                                   # the scan cut into segments reads the shared records too
        o3, s3, _ = K.chunk_forward(*dev, D**-0.5, s0.to(DEV), path=path)
        assert orc.max_abs_err(o3.float().cpu(), o_ref) < O_ABS_BF16 and orc.rel_fro_err(s3.cpu(), s_ref) < STATE_FRO


@pytest.mark.parametrize("n", [1, 3, 8, 21])
@pytest.mark.parametrize("H,HK,D", [(4, 2, 128), (6, 3, 64), (8, 1, 128)])
def test_grouped_query_heads_decode_and_prefill(K, n, H, HK, D):
    B = 3
    dev, dev_rep, host = _gqa_inputs(B, n, H, HK, D, seed=69 + n)
    s0 = golden_state(B, H, D, D, 69, 0.3)
    st, st_r = s0.to(DEV), s0.to(DEV)
    o = gdn2.gdn2_decode(*dev, st)
    o_r = gdn2.gdn2_decode(*dev_rep, st_r)
    assert torch.equal(o, o_r) and torch.equal(st, st_r)
    s_ref = s0.clone()
    o_ref = orc.decode(*host, s_ref)
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16 and orc.rel_fro_err(st.cpu(), s_ref) < 1e-5
    # ragged prefill through the public op: whole chunks + tail
    S = 64 * 3 + n
    dev, dev_rep, host = _gqa_inputs(B, S, H, HK, D, seed=71 + n)
    o, s = gdn2.gdn2_prefill(*dev, s0.to(DEV))
    o_ref, s_ref = orc.prefill(*host, s0.clone())
    assert o.shape == (B, S, H, D)
    assert orc.max_abs_err(o.float().cpu(), o_ref) < O_ABS_BF16 and orc.rel_fro_err(s.cpu(), s_ref) < STATE_FRO


def test_grouped_query_heads_reject_uneven_groups(K):
    dev, _, _ = _gqa_inputs(1, 4, 4, 2, 128, seed=3)
    q3 = dev[0][:, :, :1].repeat(1, 1, 3, 1)
    with pytest.raises(ValueError, match="multiple"):
        gdn2.gdn2_decode(q3, q3, dev[2], q3.float(), q3, dev[5], torch.zeros(1, 4, 128, 128, device=DEV))
