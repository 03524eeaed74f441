"""Host-side logic of the public API on CPU: routing of whole chunks vs the ragged tail, state
ownership, error behaviour, the layer's cache handling and the head-parallel sharding.

The CUDA kernels are replaced by ``tests.fake_kernels.OracleKernels`` (the CPU oracle behind the
launcher's interface), so only the Python around the kernels is under test here; the kernels
themselves are covered by the ``gpu``-marked tests."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import gdn2_tilelang_b200 as gdn2
from gdn2_tilelang_b200 import _cabi
from oracle import gdn2_oracle as orc
from oracle import layer_oracle as lorc
from tests.conftest import golden_state, load_golden
from tests.fake_kernels import OracleKernels
from tests.golden.make_golden import LAYER, PREFILL_CASES


@pytest.fixture()
def fake(monkeypatch):
    k = OracleKernels()
    monkeypatch.setattr(_cabi, "_kernels", k)
    return k


# ---- functional ops ---------------------------------------------------------------------------


@pytest.mark.parametrize("name", sorted(PREFILL_CASES))
def test_prefill_routes_chunks_and_tail(fake, name):
    B, S, H, DK, DV = PREFILL_CASES[name]
    gold = load_golden(name)
    q, k, v, g, b, w = orc.make_inputs(B, S, H, DK, DV, seed=2, gate="softplus")
    s0 = golden_state(B, H, DK, DV, 2, 0.3)
    o, state = gdn2.gdn2_prefill(q, k, v, g, b, w, s0.clone())
    want = ([("chunk_forward", S // 64 * 64)] if S >= 64 else []) + ([("decode", S % 64)] if S % 64 else [])
    assert fake.calls == want
    assert o.shape == (B, S, H, DV) and o.dtype == v.dtype
    assert orc.rel_max_err(o, gold["o"]) < 2e-5
    assert orc.rel_max_err(state, gold["state"]) < 2e-5


def test_prefill_state_ownership(fake):
    q, k, v, g, b, w = orc.make_inputs(1, 70, 2, 32, 24, gate="softplus")
    s0 = golden_state(1, 2, 32, 24, 3, 0.3)
    keep = s0.clone()
    _, s1 = gdn2.gdn2_prefill(q, k, v, g, b, w, s0)
    assert torch.equal(s0, keep) and s1.data_ptr() != s0.data_ptr()      # whole chunks: a new tensor
    short = tuple(t[:, :7] for t in (q, k, v, g, b, w))
    _, s2 = gdn2.gdn2_prefill(*short, s0)
    assert s2.data_ptr() == s0.data_ptr() and not torch.equal(s0, keep)   # shorter than a chunk: in place
    o3, s3 = gdn2.gdn2_prefill(*short, None)
    assert s3.dtype == torch.float32 and s3.shape == (1, 2, 32, 24)


def test_segmented_prefill_equals_one_pass(fake):
    q, k, v, g, b, w = orc.make_inputs(2, 192, 3, 32, 24, gate="softplus")
    o_all, s_all = gdn2.gdn2_prefill(q, k, v, g, b, w)
    outs, state = [], None
    for lo, hi in ((0, 64), (64, 160), (160, 192)):
        o, state = gdn2.gdn2_prefill(*(t[:, lo:hi] for t in (q, k, v, g, b, w)), state)
        outs.append(o)
    assert orc.rel_max_err(torch.cat(outs, 1), o_all) < 2e-5
    assert orc.rel_max_err(state, s_all) < 2e-5


def test_prefill_from_host_without_a_gpu_equals_prefill(fake):
    ins = orc.make_inputs(2, 100, 3, 32, 24, gate="softplus")
    s0 = torch.randn(2, 3, 32, 24)
    o_ref, s_ref = gdn2.gdn2_prefill(*ins, s0)
    out = torch.empty_like(o_ref)
    o, s = gdn2.gdn2_prefill_from_host(*ins, s0, device="cpu", out=out)
    assert o is out and torch.equal(o, o_ref) and torch.equal(s, s_ref)
    with pytest.raises(ValueError):
        gdn2.gdn2_prefill_from_host(*ins, torch.zeros(1, 3, 32, 24), device="cpu")


def test_decode_step_shapes_and_in_place_state(fake):
    q, k, v, g, b, w = orc.make_inputs(2, 1, 3, 32, 24, gate="softplus")
    s0 = golden_state(2, 3, 32, 24, 4, 0.3)
    st = s0.clone()
    o = gdn2.gdn2_decode_step(*(t[:, 0] for t in (q, k, v, g, b, w)), st)
    o_ref, s_ref = orc.recurrence(q, k, v, g, b, w, None, s0)
    assert o.shape == (2, 3, 24)
    assert orc.rel_max_err(o, o_ref[:, 0]) < 1e-5 and orc.rel_max_err(st, s_ref) < 1e-5
    with pytest.raises(ValueError):
        gdn2.gdn2_decode(q, k, v, g, b, w, st[:, :2])


def test_attention_handles_ragged_length_and_initial_state(fake):
    q, k, v, g, b, w = orc.make_inputs(2, 100, 2, 32, 32, gate="softplus")
    s0 = golden_state(2, 2, 32, 32, 5, 0.5)
    keep = s0.clone()
    cfg = gdn2.GDN2Config()
    # the fake runs on CPU, so bypass the device check of resolve_backend only
    import gdn2_tilelang_b200.attention as att
    o, s = att.chunk_gdn2_fwd(q, k, v, g, b, w, 32**-0.5, s0, True, cfg)
    o_ref, s_ref = orc.recurrence(q, k, v, g, b, w, None, keep)
    assert orc.rel_max_err(o, o_ref) < 2e-5 and orc.rel_max_err(s, s_ref) < 2e-5
    assert torch.equal(s0, keep)
    o2, none = att.chunk_gdn2_fwd(*(t[:, :7] for t in (q, k, v, g, b, w)), 32**-0.5, s0, False, cfg)
    assert none is None and torch.equal(s0, keep) and o2.shape == (2, 7, 2, 32)
    o3, s3, h = att.chunk_gdn2_fwd(*(t[:, :64] for t in (q, k, v, g, b, w)), 32**-0.5, s0, True, cfg,
                                   return_chunk_states=True)
    assert h.shape == (2, 1, 2, 32, 32) and torch.equal(h[:, 0], s0)


def test_error_behaviour():
    q, k, v, g, b, w = orc.make_inputs(1, 64, 1, 32, 32)
    with pytest.raises(ValueError, match="requires a CUDA device"):
        gdn2.gdn2_attention(q, k, v, g, b, w)
    with pytest.raises(ValueError, match="unknown backend"):
        gdn2.resolve_backend("fla", True, False)
    with pytest.raises(ValueError, match="host reference path"):
        gdn2.resolve_backend("torch", False, False)
    with pytest.raises(ValueError, match="forward / serving path only"):
        gdn2.resolve_backend("auto", True, True)
    assert gdn2.resolve_backend("auto", True, False) == "cuda"
    assert gdn2.resolve_backend("tilelang", True, False) == "cuda"
    with pytest.raises(ValueError, match="chunk_size must be 64"):
        gdn2.gdn2_prefill(q, k, v, g, b, w, config=gdn2.GDN2Config(chunk_size=32))
    with pytest.raises(ValueError, match="state_dtype"):
        gdn2.gdn2_prefill(q, k, v, g, b, w, config=gdn2.GDN2Config(state_dtype=torch.bfloat16))
    with pytest.raises(TypeError):
        gdn2.gdn2_prefill(*(t.double() for t in (q, k, v)), g, b.double(), w.double())
    with pytest.raises(TypeError, match="share one dtype"):
        gdn2.gdn2_prefill(q, k.bfloat16(), v, g, b, w)
    with pytest.raises(ValueError, match="CUDA devices only"):   # the real launcher refuses host tensors
        _cabi.NativeKernels().decode(q, k, v, g, b, w, torch.zeros(1, 1, 32, 32), 1.0)


def test_packed_variable_length_batch(fake, monkeypatch):
    """cu_seqlens: sequences packed along the token axis of one batch entry, each evaluated on its own slice
    (whole chunks, ragged tail, a sequence shorter than a chunk, an empty one), states per sequence."""
    import gdn2_tilelang_b200.attention as att
    monkeypatch.setattr(att, "resolve_backend", lambda *a, **kw: "cuda")
    offs = [0, 130, 130, 194, 201, 330]
    q, k, v, g, b, w = orc.make_inputs(1, offs[-1], 2, 32, 24, seed=9)
    s0 = golden_state(5, 2, 32, 24, 9, 0.3)
    o, s = gdn2.gdn2_attention(q, k, v, g, b, w, initial_state=s0, output_final_state=True,
                               cu_seqlens=torch.tensor(offs))
    assert o.shape == (1, offs[-1], 2, 24) and s.shape == (5, 2, 32, 24)
    for i, (lo, hi) in enumerate(zip(offs, offs[1:])):
        if hi == lo:
            assert torch.equal(s[i], s0[i])
            continue
        o_ref, s_ref = orc.recurrence(*(t[:, lo:hi] for t in (q, k, v, g, b, w)), None, s0[i:i + 1])
        assert orc.rel_max_err(o[:, lo:hi], o_ref) < 2e-5
        assert orc.rel_max_err(s[i:i + 1], s_ref) < 2e-5
    o2, s2 = gdn2.gdn2_attention(q, k, v, g, b, w, cu_seqlens=offs)          # a plain list, no states
    assert s2 is None and o2.shape == o.shape
    with pytest.raises(ValueError, match="B == 1"):
        gdn2.gdn2_attention(*(t.repeat(2, 1, 1, 1) for t in (q, k, v, g, b, w)), cu_seqlens=offs)
    with pytest.raises(ValueError, match="rise from 0"):
        gdn2.gdn2_attention(q, k, v, g, b, w, cu_seqlens=[0, 100])
    layer = gdn2.GatedDeltaNet2(gdn2.GatedDeltaNet2Config(**LAYER)).eval()
    with pytest.raises(NotImplementedError, match="convolution"):
        layer(torch.zeros(1, 8, LAYER["hidden_size"]), cu_seqlens=[0, 8])


# ---- the layer --------------------------------------------------------------------------------


def _layer_and_input(monkeypatch):
    import gdn2_tilelang_b200.attention as att
    monkeypatch.setattr(att, "resolve_backend", lambda *a, **kw: "cuda")
    dims = lorc.LayerDims(**LAYER)
    sd = lorc.random_state_dict(dims, seed=3, std=0.2)
    layer = gdn2.GatedDeltaNet2(gdn2.GatedDeltaNet2Config(**LAYER)).eval()
    layer.load_state_dict(sd, strict=True)
    x = torch.randn(2, 90, LAYER["hidden_size"], generator=torch.Generator().manual_seed(4))
    return layer, sd, x


def test_layer_matches_reference_module_outputs(fake, monkeypatch):
    layer, sd, x = _layer_and_input(monkeypatch)
    gold = load_golden("layer_h64")
    full, cache_f = layer(x, use_cache=True)
    assert orc.rel_max_err(full, gold["full"]) < 1e-5
    assert orc.rel_max_err(cache_f.recurrent_state, gold["full_state"]) < 1e-5
    assert orc.rel_max_err(cache_f.conv_state, gold["full_conv"]) < 1e-6
    pre, cache = layer.prefill(x[:, :70])
    dec, cache = layer.decode(x[:, 70:75], cache)
    steps = torch.stack([layer.step(x[:, t], cache)[0] for t in range(75, 90)], 1)
    for mine, key in ((pre, "prefill"), (dec, "decode"), (steps, "steps"),
                      (cache.recurrent_state, "final_state"), (cache.conv_state, "final_conv")):
        assert orc.rel_max_err(mine, gold[key]) < 1e-5
    assert set(layer.state_dict()) == set(sd)


def test_init_cache_layout_and_dtypes():
    cfg = gdn2.GatedDeltaNet2Config(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim_k=16, head_dim_v=32)
    layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16)
    c = layer.init_cache(3)
    assert c.recurrent_state.shape == (3, 4, 16, 32) and c.recurrent_state.dtype == torch.float32
    assert c.conv_state.shape == (3, 2 * 2 * 16 + 4 * 32, 3) and c.conv_state.dtype == torch.bfloat16
    with pytest.raises(ValueError):
        layer.init_cache(1, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        gdn2.GatedDeltaNet2(gdn2.GatedDeltaNet2Config(hidden_size=64, num_heads=3, num_kv_heads=2))


# ---- head-parallel layer, 2 gloo ranks -----------------------------------------------------------


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import gdn2_tilelang_b200.attention as att
        att.resolve_backend = lambda *a, **kw: "cuda"
        _cabi._kernels = OracleKernels()
        torch.set_num_threads(1)
        dims = lorc.LayerDims(**LAYER)
        sd = lorc.random_state_dict(dims, seed=3, std=0.2)
        cfg = gdn2.GatedDeltaNet2Config(**LAYER)
        layer = gdn2.TensorParallelGatedDeltaNet2(cfg).eval()
        layer.load_full_state_dict(sd)
        x = torch.randn(2, 90, LAYER["hidden_size"], generator=torch.Generator().manual_seed(4))
        pre, cache = layer.prefill(x[:, :70])
        dec, cache = layer.decode(x[:, 70:75], cache)
        steps = torch.stack([layer.step(x[:, t], cache)[0] for t in range(75, 90)], 1)
        gold = load_golden("layer_h64")
        errs = [orc.rel_max_err(pre, gold["prefill"]), orc.rel_max_err(dec, gold["decode"]),
                orc.rel_max_err(steps, gold["steps"])]
        hl = LAYER["num_heads"] // world
        errs.append(orc.rel_max_err(cache.recurrent_state, gold["final_state"][:, rank * hl:(rank + 1) * hl]))
        ret[rank] = (max(errs), tuple(cache.recurrent_state.shape))
    finally:
        dist.destroy_process_group()


def test_head_parallel_layer_two_ranks():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err, shape = ret[rank]
        assert err < 1e-5, (rank, err)
        assert shape == (2, LAYER["num_heads"] // world, LAYER["head_dim_k"], LAYER["head_dim_v"])


def test_shard_state_dict_partitions_every_parameter():
    cfg = gdn2.GatedDeltaNet2Config(**LAYER)
    sd = lorc.random_state_dict(lorc.LayerDims(**LAYER), seed=1)
    parts = [gdn2.shard_state_dict(sd, cfg, r, 2) for r in range(2)]
    for name, full in sd.items():
        if name == "o_norm.weight":
            assert all(torch.equal(p[name], full) for p in parts)
        elif name == "o_proj.weight":
            assert torch.equal(torch.cat([p[name] for p in parts], 1), full)
        else:
            assert torch.equal(torch.cat([p[name] for p in parts], 0), full)
    with pytest.raises(ValueError):
        gdn2.shard_config(cfg, 3)
