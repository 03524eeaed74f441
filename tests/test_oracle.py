"""Pin the CPU oracle: against outputs of the reference's own functions (the
golden fixtures) and against the self-consistency properties the reference's
test-suite states (tests/test_gdn2.py:47-121, tests/test_inference.py:21-150,
tests/test_pipeline_simulation.py:103-130 of the reference project)."""

from __future__ import annotations

import pytest
import torch

from oracle import gdn2_oracle as orc
from oracle import layer_oracle as lorc
from tests.conftest import golden_checksum, golden_state, load_golden
from tests.golden.make_golden import CORE_CASES, DECODE_CASES, LAYER, PREFILL_CASES


def _close(a, ref, tol):
    assert a.shape == ref.shape
    assert orc.rel_max_err(a, ref) < tol


@pytest.mark.parametrize("name", sorted(CORE_CASES))
def test_core_cases_match_reference_outputs(name):
    B, S, H, DK, DV, gate, ds, with_s0 = CORE_CASES[name]
    gold = load_golden(name)
    q, k, v, g, b, w = orc.make_inputs(B, S, H, DK, DV, seed=0, gate=gate, decay_scale=ds)
    assert golden_checksum(q, k, v, g, b, w) == pytest.approx(gold["inputs_checksum"], rel=1e-12)
    s0 = golden_state(B, H, DK, DV, 0, 0.5) if with_s0 else None
    o, s = orc.recurrence(q, k, v, g, b, w, None, s0)
    _close(o, gold["o_recurrent"], 1e-6)
    _close(s, gold["s_recurrent"], 1e-6)
    o, s, h = orc.chunkwise(q, k, v, g, b, w, None, s0, return_chunk_states=True)
    _close(o, gold["o_chunk"], 2e-6)
    _close(s, gold["s_chunk"], 2e-6)
    if "o_attention" in gold:
        o, s = orc.attention(q, k, v, g, b, w)
        _close(o, gold["o_attention"], 2e-6)
        _close(s, gold["s_attention"], 2e-6)
    if "f_Aqk" in gold:
        f = orc.chunk_factors(q, k, v, g, b, w)
        for mine, theirs in (("Aqk", "Aqk"), ("Ai", "Ai"), ("W", "W"), ("U", "U"), ("KG", "Ktail")):
            _close(f[mine], gold[f"f_{theirs}"], 5e-6)
        _close(h.permute(0, 2, 1, 3, 4), gold["f_h"], 2e-6)


@pytest.mark.parametrize("name", sorted(DECODE_CASES))
def test_decode_matches_reference_outputs(name):
    B, n, H, DK, DV = DECODE_CASES[name]
    gold = load_golden(name)
    q, k, v, g, b, w = orc.make_inputs(B, n, H, DK, DV, seed=1, gate="softplus")
    s0 = golden_state(B, H, DK, DV, 1, 0.3)
    assert golden_checksum(q, k, v, g, b, w, s0) == pytest.approx(gold["inputs_checksum"], rel=1e-12)
    state = s0.clone()
    o = orc.decode(q, k, v, g, b, w, state)
    _close(o, gold["o"], 1e-6)
    _close(state, gold["state"], 1e-6)


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_matches_reference_outputs(name):
    B, S, H, DK, DV = PREFILL_CASES[name]
    gold = load_golden(name)
    q, k, v, g, b, w = orc.make_inputs(B, S, H, DK, DV, seed=2, gate="softplus")
    s0 = golden_state(B, H, DK, DV, 2, 0.3)
    o, state = orc.prefill(q, k, v, g, b, w, s0.clone())
    _close(o, gold["o"], 2e-6)
    _close(state, gold["state"], 2e-6)


def test_layer_matches_reference_module():
    gold = load_golden("layer_h64")
    dims = lorc.LayerDims(**LAYER)
    sd = lorc.random_state_dict(dims, seed=3, std=0.2)
    gen = torch.Generator(device="cpu").manual_seed(4)
    x = torch.randn(2, 90, LAYER["hidden_size"], generator=gen)
    assert golden_checksum(x, *sd.values()) == pytest.approx(gold["inputs_checksum"], rel=1e-12)
    full, s_full, conv_full = lorc.forward(sd, dims, x)
    _close(full, gold["full"], 1e-5)
    _close(s_full, gold["full_state"], 1e-5)
    _close(conv_full, gold["full_conv"], 1e-6)
    state, conv = lorc.init_cache(dims, 2)
    pre, state, conv = lorc.prefill(sd, dims, x[:, :70], state, conv)
    dec, state, conv = lorc.decode(sd, dims, x[:, 70:75], state, conv)
    steps = []
    for t in range(75, 90):
        y, state, conv = lorc.decode(sd, dims, x[:, t:t + 1], state, conv)
        steps.append(y[:, 0])
    _close(pre, gold["prefill"], 1e-5)
    _close(dec, gold["decode"], 1e-5)
    _close(torch.stack(steps, 1), gold["steps"], 1e-5)
    _close(state, gold["final_state"], 1e-5)
    _close(conv, gold["final_conv"], 1e-6)
    # the serving path reproduces the one-shot forward (reference tests/test_inference.py:166-178)
    _close(torch.cat([pre, dec, torch.stack(steps, 1)], 1), gold["full"], 1e-4)


# ---- properties the reference's own tests pin -------------------------------------------


@pytest.mark.parametrize("S,BS,BC", [(128, 64, 16), (256, 64, 32), (192, 32, 16), (64, 64, 8)])
def test_chunkwise_equals_recurrence(S, BS, BC):
    q, k, v, g, b, w = orc.make_inputs(2, S, 3, 32, 48, gate="softplus")
    o_ref, s_ref = orc.recurrence(q, k, v, g, b, w)
    o, s = orc.chunkwise(q, k, v, g, b, w, chunk_size=BS, sub_chunk_size=BC)
    assert orc.rel_max_err(o, o_ref) < 2e-5
    assert orc.rel_max_err(s, s_ref) < 2e-5


@pytest.mark.parametrize("decay_scale", [0.0, 1.0, 8.0, 30.0])
def test_fast_decay_stays_finite(decay_scale):
    q, k, v, g, b, w = orc.make_inputs(1, 128, 2, 32, 32, gate="softplus", decay_scale=decay_scale)
    o_ref, _ = orc.recurrence(q, k, v, g, b, w)
    o, _ = orc.chunkwise(q, k, v, g, b, w)
    assert torch.isfinite(o).all()
    assert orc.rel_max_err(o, o_ref) < 1e-4


def test_tied_gates_reduce_to_kda():
    q, k, v, g, _, _ = orc.make_inputs(2, 128, 3, 32, 32, gate="softplus")
    beta = torch.rand(2, 128, 3, 1, generator=torch.Generator().manual_seed(5))
    bw = beta.expand(-1, -1, -1, 32).contiguous()
    o, _ = orc.chunkwise(q, k, v, g, bw, bw)
    S = torch.zeros(2, 3, 32, 32)
    o_kda = torch.empty_like(o)
    for t in range(128):
        S = S * g[:, t].exp().unsqueeze(-1)
        kt, bt = k[:, t], beta[:, t, :, 0][..., None, None]
        S = S - bt * kt.unsqueeze(-1) * torch.einsum("bhkd,bhk->bhd", S, kt).unsqueeze(-2)
        S = S + bt * kt.unsqueeze(-1) * v[:, t].unsqueeze(-2)
        o_kda[:, t] = torch.einsum("bhkd,bhk->bhd", S, q[:, t] * 32**-0.5)
    assert orc.rel_max_err(o, o_kda) < 2e-5


def test_scalar_gate_reduces_to_gated_deltanet():
    """g broadcast over channels and b=w=beta is Gated DeltaNet: S = a (I - beta k k^T) S + beta k v^T."""
    q, k, v, g, _, _ = orc.make_inputs(1, 128, 2, 32, 32, gate="softplus")
    g = g[..., :1].expand(-1, -1, -1, 32).contiguous()
    beta = torch.rand(1, 128, 2, 1, generator=torch.Generator().manual_seed(6))
    bw = beta.expand(-1, -1, -1, 32).contiguous()
    o, _ = orc.chunkwise(q, k, v, g, bw, bw)
    S = torch.zeros(1, 2, 32, 32)
    o_gdn = torch.empty_like(o)
    for t in range(128):
        a = g[:, t, :, 0].exp()[..., None, None]
        kt, bt = k[:, t], beta[:, t, :, 0][..., None, None]
        S = a * S
        S = S - bt * kt.unsqueeze(-1) * torch.einsum("bhkd,bhk->bhd", S, kt).unsqueeze(-2) \
            + bt * kt.unsqueeze(-1) * v[:, t].unsqueeze(-2)
        o_gdn[:, t] = torch.einsum("bhkd,bhk->bhd", S, q[:, t] * 32**-0.5)
    assert orc.rel_max_err(o, o_gdn) < 2e-5


def test_zero_gates_only_decay_the_state():
    q, k, v, g, _, _ = orc.make_inputs(1, 128, 2, 32, 32, gate="softplus")
    z = torch.zeros(1, 128, 2, 32)
    s0 = golden_state(1, 2, 32, 32, 7, 1.0)
    _, s = orc.chunkwise(q, k, v, g, z, z, initial_state=s0)
    assert orc.rel_max_err(s, s0 * g.sum(dim=1).exp().unsqueeze(-1)) < 2e-5


def test_multi_token_decode_equals_single_steps():
    q, k, v, g, b, w = orc.make_inputs(2, 12, 3, 32, 24, gate="softplus")
    s0 = golden_state(2, 3, 32, 24, 8, 0.3)
    sm = s0.clone()
    om = orc.decode(q, k, v, g, b, w, sm)
    s1 = s0.clone()
    o1 = torch.cat([orc.decode(*(t[:, i:i + 1] for t in (q, k, v, g, b, w)), s1) for i in range(12)], 1)
    assert orc.rel_max_err(om, o1) < 1e-5
    assert orc.rel_max_err(sm, s1) < 1e-5


def test_segmented_prefill_equals_one_pass():
    q, k, v, g, b, w = orc.make_inputs(2, 192, 3, 32, 24, gate="softplus")
    o_all, s_all = orc.prefill(q, k, v, g, b, w)
    outs, state = [], None
    for lo, hi in ((0, 64), (64, 160), (160, 192)):
        o, state = orc.prefill(*(t[:, lo:hi] for t in (q, k, v, g, b, w)), state)
        outs.append(o)
    assert orc.rel_max_err(torch.cat(outs, 1), o_all) < 2e-5
    assert orc.rel_max_err(state, s_all) < 2e-5


def test_oracle_matches_the_vendored_reference_when_built():
    """``oracle/_ref`` (the reference's own gdn2/reference.py, placed there by oracle/build_ref.py) against the
    restatement, on a ragged prefill: whole chunks through the chunkwise form, the tail through the recurrence."""
    from oracle.build_ref import load_ref

    ref = load_ref()
    if ref is None:
        pytest.skip("oracle/_ref has not been built (no reference checkout on this machine)")
    q, k, v, g, b, w = orc.make_inputs(2, 64 * 3 + 11, 3, 32, 24, seed=7)
    s0 = golden_state(2, 3, 32, 24, 7, 0.3)
    o, s = orc.prefill(q, k, v, g, b, w, s0.clone())
    n_full, scale = 64 * 3, 32**-0.5
    o1, st = ref.chunk_gdn2_torch(*(t[:, :n_full] for t in (q, k, v, g, b, w)), scale, s0.clone(), True)
    o2, st = ref.recurrent_gdn2(*(t[:, n_full:] for t in (q, k, v, g, b, w)), scale, st, True)
    _close(o, torch.cat([o1, o2], 1), 5e-6)
    _close(s, st, 5e-6)
