"""Parity with the oracle at the sizes the benchmark definition names (configs 1-4), through the public API.

The oracle runs one sequence at a time on the host (a few seconds each); the GPU side runs the whole
configuration in one call. Tolerances are the acceptance bounds of the benchmark definition: output max-abs
error <= 2e-2 with bf16 I/O, final / per-chunk state relative Frobenius error <= 1e-3 with fp32 state.
"""

from __future__ import annotations

import pytest
import torch

import gdn2_tilelang_b200 as gdn2
from gdn2_tilelang_b200 import _cabi
from oracle import gdn2_oracle as orc
from oracle import layer_oracle as lorc
from tests.conftest import note

pytestmark = pytest.mark.gpu
DEV = "cuda"
O_ABS_BF16, STATE_FRO = 2e-2, 1e-3


def rounded(ins):
    """(device bf16 tensors + fp32 g, host fp32 copies of the bf16-rounded values)."""
    q, k, v, g, b, w = ins
    lo = [t.bfloat16() for t in (q, k, v, b, w)]
    dev = (lo[0].to(DEV), lo[1].to(DEV), lo[2].to(DEV), g.to(DEV), lo[3].to(DEV), lo[4].to(DEV))
    host = (lo[0].float(), lo[1].float(), lo[2].float(), g, lo[3].float(), lo[4].float())
    return dev, host


@pytest.fixture(scope="module")
def K():
    k = _cabi.kernels()
    yield k
    k.check_device_status()


@pytest.fixture(scope="module")
def cfg2():
    """Config 2: B=4, S=16037 (250 chunks + 37-token tail), H=16, D=128; sequence i drawn with seed i."""
    B, S, H, D = 4, 16037, 16, 128
    devs, o_refs, s_refs = [], [], []
    for i in range(B):
        dev, host = rounded(orc.make_inputs(1, S, H, D, D, seed=i))
        o_ref, s_ref = orc.prefill(*host)
        devs.append(dev)
        o_refs.append(o_ref)
        s_refs.append(s_ref)
        del host
    dev = tuple(torch.cat([d[j] for d in devs], 0) for j in range(6))
    return dev, torch.cat(o_refs, 0), torch.cat(s_refs, 0)


def test_config2_serving_prefill_whole_workload(K, cfg2):
    dev, o_ref, s_ref = cfg2
    o, state = gdn2.gdn2_prefill(*dev)
    K.check_device_status()
    assert o.shape == o_ref.shape and o.dtype == torch.bfloat16
    e_o, e_s = orc.max_abs_err(o.float().cpu(), o_ref), orc.rel_fro_err(state.cpu(), s_ref)
    note("config2", heads=16, o_max_abs=e_o, state_rel_fro=e_s)
    assert e_o < O_ABS_BF16 and e_s < STATE_FRO


@pytest.mark.parametrize("world", [2, 4, 8])
def test_config2_head_sharded_rank_problem(K, cfg2, world):
    """What one rank of a head-sharded run computes (16 / world heads): same oracle values. With 4 and 2 heads
    the scan cuts the sequence into segments."""
    dev, o_ref, s_ref = cfg2
    hl = 16 // world
    r = world - 1                                            # the last rank's slice
    sl = slice(r * hl, (r + 1) * hl)
    part = tuple(t[:, :, sl].contiguous() for t in dev)
    o, state = gdn2.gdn2_prefill(*part)
    K.check_device_status()
    e_o = orc.max_abs_err(o.float().cpu(), o_ref[:, :, sl])
    e_s = orc.rel_fro_err(state.cpu(), s_ref[:, sl])
    note("config2_sharded", heads=hl, segments=K.scan_segments(4, 16000, hl, 128, 128, torch.bfloat16, _cabi.PATH_AUTO),
         o_max_abs=e_o, state_rel_fro=e_s)
    assert e_o < O_ABS_BF16 and e_s < STATE_FRO


@pytest.mark.parametrize("variant", ["gdn2", "kda", "gdn"])
def test_config1_chunkwise_forward_with_fp32_chunk_states(K, variant):
    """Config 1: B=2, S=4096, H=16, D=128, bf16 inputs, fp32 per-chunk states h [B, NC, H, DK, DV]; plus the
    tied-gate (KDA, b = w) and per-head scalar decay (GDN) degeneracies."""
    B, S, H, D = 2, 4096, 16, 128
    q, k, v, g, b, w = orc.make_inputs(B, S, H, D, D, seed=0)
    if variant in ("kda", "gdn"):
        w = b.clone()
    if variant == "gdn":
        g = g[..., :1].expand(-1, -1, -1, D).contiguous()
    dev, host = rounded((q, k, v, g, b, w))
    o_ref, s_ref, h_ref = orc.chunkwise(*host, return_chunk_states=True)
    o, s, h = gdn2.chunk_gdn2_fwd(*dev, D**-0.5, None, True, return_chunk_states=True)
    K.check_device_status()
    assert h.shape == (B, S // 64, H, D, D) and h.dtype == torch.float32
    e = dict(o_max_abs=orc.max_abs_err(o.float().cpu(), o_ref), state_rel_fro=orc.rel_fro_err(s.cpu(), s_ref),
             h_rel_fro=orc.rel_fro_err(h.cpu(), h_ref))
    note("config1", variant=variant, **e)
    assert e["o_max_abs"] < O_ABS_BF16 and e["state_rel_fro"] < STATE_FRO and e["h_rel_fro"] < STATE_FRO
    # the chunk-parallel output from those states (tensor-core products on the 16-bit workspace)
    o2 = gdn2.chunk_gdn2_output(*dev, D**-0.5, h)
    assert orc.max_abs_err(o2.float().cpu(), o_ref) < O_ABS_BF16
    # the functional op on the same inputs
    o3, s3 = gdn2.gdn2_attention(*dev, output_final_state=True)
    assert orc.max_abs_err(o3.float().cpu(), o_ref) < O_ABS_BF16 and orc.rel_fro_err(s3.cpu(), s_ref) < STATE_FRO


def test_config3_decode_b256(K):
    """Config 3: B=256, H=16, D=128, state ~ N(0, 0.02): one token through decode_step, then 8 draft tokens."""
    B, H, D = 256, 16, 128
    gen = torch.Generator().manual_seed(0)
    dev1, host1 = rounded(orc.make_inputs(B, 1, H, D, D, seed=0))
    dev8, host8 = rounded(orc.make_inputs(B, 8, H, D, D, seed=1))
    s0 = torch.randn(B, H, D, D, generator=gen) * 0.02
    state = s0.to(DEV)
    s_ref = s0.clone()
    o1 = gdn2.gdn2_decode_step(*(t[:, 0] for t in dev1), state)
    o1_ref = orc.decode(*host1, s_ref)[:, 0]
    e1 = dict(o_max_abs=orc.max_abs_err(o1.float().cpu(), o1_ref), state_rel_fro=orc.rel_fro_err(state.cpu(), s_ref))
    o8 = gdn2.gdn2_decode(*dev8, state)
    o8_ref = orc.decode(*host8, s_ref)
    e8 = dict(o_max_abs=orc.max_abs_err(o8.float().cpu(), o8_ref), state_rel_fro=orc.rel_fro_err(state.cpu(), s_ref))
    K.check_device_status()
    note("config3", n1=e1, n8=e8)
    for e in (e1, e8):
        assert e["o_max_abs"] < O_ABS_BF16 and e["state_rel_fro"] < 1e-5


def test_config4_layer_hidden2048(K):
    """Config 4: the full layer, hidden 2048, 16 heads, 8 kv heads, D=128, bf16 weights ~ N(0, 0.02):
    prefill of x [2, 4096, 2048], then single-token steps (8 of the 128 are checked against the oracle; the
    oracle evaluates in fp32 on the same bf16 weights and inputs)."""
    dims = lorc.LayerDims(hidden_size=2048, num_heads=16, num_kv_heads=8)
    sd = lorc.random_state_dict(dims, seed=0, std=0.02, dtype=torch.bfloat16)
    cfg = gdn2.GatedDeltaNet2Config(hidden_size=2048, num_heads=16, num_kv_heads=8)
    layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval()
    layer.load_state_dict(sd)
    layer.to(DEV)
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(2, 4096 + 8, 2048, generator=gen).bfloat16()
    pre, cache = layer.prefill(x[:, :4096].to(DEV))
    steps = torch.stack([layer.step(x[:, t].to(DEV), cache)[0] for t in range(4096, 4104)], 1)
    got = torch.cat([pre, steps], 1).float().cpu()
    K.check_device_status()
    sd32 = {k_: v_.float() for k_, v_ in sd.items()}
    state, conv = lorc.init_cache(dims, 2)
    ref, state, conv = lorc.prefill(sd32, dims, x.float(), state, conv)
    e = dict(out_rel_max=orc.rel_max_err(got, ref), out_rel_fro=orc.rel_fro_err(got, ref),
             steps_rel_max=orc.rel_max_err(got[:, 4096:], ref[:, 4096:]),
             state_rel_fro=orc.rel_fro_err(cache.recurrent_state.cpu(), state))
    note("config4", **e)
    # bf16 GEMMs feed the kernels bf16-rounded q, k, v, gates where the oracle keeps fp32: the layer's bound is
    # the bf16 one, a few 1e-2 of the largest output
    assert e["out_rel_max"] < 5e-2 and e["out_rel_fro"] < 2e-2
    assert e["state_rel_fro"] < 2e-2
