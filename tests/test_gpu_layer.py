"""The GatedDeltaNet2 layer on the GPU: golden parity (float32, small heads), a bf16 D=128 layer
against the layer oracle, and serving-path self-consistency."""

from __future__ import annotations

import pytest
import torch

import gdn2_tilelang_b200 as gdn2
from oracle import gdn2_oracle as orc
from oracle import layer_oracle as lorc
from tests.conftest import load_golden
from tests.golden.make_golden import LAYER

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_layer_fp32_matches_reference_module_outputs():
    gold = load_golden("layer_h64")
    sd = lorc.random_state_dict(lorc.LayerDims(**LAYER), seed=3, std=0.2)
    layer = gdn2.GatedDeltaNet2(gdn2.GatedDeltaNet2Config(**LAYER)).eval()
    layer.load_state_dict(sd)
    layer.to(DEV)
    x = torch.randn(2, 90, LAYER["hidden_size"], generator=torch.Generator().manual_seed(4)).to(DEV)
    full, cache_f = layer(x, use_cache=True)
    pre, cache = layer.prefill(x[:, :70])
    dec, cache = layer.decode(x[:, 70:75], cache)
    steps = torch.stack([layer.step(x[:, t], cache)[0] for t in range(75, 90)], 1)
    for mine, key in ((full, "full"), (cache_f.recurrent_state, "full_state"), (pre, "prefill"), (dec, "decode"),
                      (steps, "steps"), (cache.recurrent_state, "final_state"), (cache.conv_state, "final_conv")):
        assert orc.rel_max_err(mine.float().cpu(), gold[key]) < 1e-4, key


def test_layer_bf16_d128_vs_oracle():
    dims = lorc.LayerDims(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim_k=128, head_dim_v=128)
    sd = lorc.random_state_dict(dims, seed=5, std=0.05, dtype=torch.bfloat16)
    cfg = gdn2.GatedDeltaNet2Config(hidden_size=256, num_heads=4, num_kv_heads=2)
    layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval()
    layer.load_state_dict(sd)
    layer.to(DEV)
    x = torch.randn(2, 200, 256, generator=torch.Generator().manual_seed(6)).bfloat16()
    pre, cache = layer.prefill(x[:, :150].to(DEV))
    dec, cache = layer.decode(x[:, 150:158].to(DEV), cache)
    steps = torch.stack([layer.step(x[:, t].to(DEV), cache)[0] for t in range(158, 200)], 1)
    got = torch.cat([pre, dec, steps], 1).float().cpu()
    # oracle in float32 on the same bf16 weights and inputs
    sd32 = {k: v.float() for k, v in sd.items()}
    state, conv = lorc.init_cache(dims, 2)
    ref, state, conv = lorc.prefill(sd32, dims, x.float(), state, conv)
    assert orc.rel_max_err(got, ref) < 5e-2
    assert orc.rel_fro_err(cache.recurrent_state.cpu(), state) < 2e-2
    assert cache.conv_state.dtype == torch.bfloat16 and cache.recurrent_state.dtype == torch.float32


def test_graphed_step_equals_eager_steps():
    """The captured one-token step replays the same kernels: identical outputs and cache, token after token."""
    cfg = gdn2.GatedDeltaNet2Config(hidden_size=256, num_heads=4, num_kv_heads=2)
    layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval().to(DEV)
    x = (torch.randn(3, 40, 256, generator=torch.Generator().manual_seed(8)) * 0.5).bfloat16().to(DEV)
    _, cache_a = layer.prefill(x[:, :24])
    _, cache_b = layer.prefill(x[:, :24])
    step = gdn2.GraphedStep(layer, cache_b)
    assert torch.equal(cache_a.recurrent_state, cache_b.recurrent_state)      # the capture left the cache as it was
    assert torch.equal(cache_a.conv_state, cache_b.conv_state)
    for t in range(24, 40):
        want, cache_a = layer.step(x[:, t], cache_a)
        got = step(x[:, t]).clone()
        assert torch.equal(got, want), t
    assert torch.equal(cache_a.recurrent_state, cache_b.recurrent_state)
    assert torch.equal(cache_a.conv_state, cache_b.conv_state)


@pytest.mark.parametrize("cached", [False, True])
@pytest.mark.parametrize("S", [1, 2, 9])
def test_fused_front_and_back_match_the_operator_chain(cached, S):
    """gdn2_layer_front / gdn2_layer_back against the torch operator chain of the reference layer, evaluated on
    the host on the same projection buffer (float32, so the only differences are fast-math exponentials): every
    output, the new convolution cache, the gated norm."""
    from tests.fake_kernels import layer_back_chain, layer_front_chain

    cfg = gdn2.GatedDeltaNet2Config(hidden_size=96, num_heads=6, num_kv_heads=2, head_dim_k=32, head_dim_v=48)
    layer = gdn2.GatedDeltaNet2(cfg).eval().to(DEV)
    gen = torch.Generator().manual_seed(11)
    with torch.no_grad():
        for prm in layer.parameters():
            prm.copy_(torch.randn(prm.shape, generator=gen).to(DEV) * 0.3)
    x = torch.randn(2, S, 96, generator=gen).to(DEV)
    state = torch.randn(2, 2 * 2 * 32 + 6 * 48, 3, generator=gen).to(DEV) if cached else None
    fused = layer._front(x, state, cached=cached)
    proj = fused[7].cpu()
    _, offs, cw, cb = layer._fused_tables()
    chain = layer_front_chain(proj, offs[:6], None if state is None else state.cpu(), cw.cpu(), cb.cpu(),
                              layer.A_log.detach().cpu(), layer.dt_bias.detach().cpu(), 6, 2, 32, 48, cfg.conv_size,
                              float(layer.erase_scale))
    for name, a, b in zip("q k v g b w conv".split(), fused[:7], chain):
        assert a.shape == b.shape and a.dtype == b.dtype, name
        assert orc.rel_max_err(a.float().cpu(), b.float()) < 2e-5, name
    o = torch.randn(2, S, 6, 48, generator=gen)
    want = layer_back_chain(o, proj, layer.o_norm.weight.detach().cpu(), offs[6], layer.o_norm.eps)
    got = gdn2._cabi.kernels().layer_back(o.to(DEV), fused[7], layer.o_norm.weight.detach(), offs[6],
                                           float(layer.o_norm.eps))
    assert orc.rel_max_err(got.cpu(), want) < 2e-5


def _exchange_buffers(K, world, hidden):
    import ctypes

    off = ctypes.c_size_t(0)
    nbytes = K.lib.gdn2_oproj_reduce_buffer_bytes(world, hidden, ctypes.byref(off))
    bufs = [torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV) for _ in range(world)]
    slots = torch.tensor([b_.data_ptr() for b_ in bufs], dtype=torch.int64, device=DEV)
    flags = torch.tensor([b_.data_ptr() + off.value for b_ in bufs], dtype=torch.int64, device=DEV)
    epochs = [torch.zeros(hidden // 32, dtype=torch.int32, device=DEV) for _ in range(world)]
    return bufs, slots, flags, epochs


@pytest.mark.parametrize("dtype,rows,Kdim", [(torch.bfloat16, 2, 256), (torch.bfloat16, 8, 1024), (torch.float32, 3, 96),
                                             (torch.float16, 1, 2048)])
def test_fused_output_projection_single_rank(dtype, rows, Kdim):
    """gdn2_oproj_reduce with one rank is the plain product x W^T (fp32 accumulation, one rounding)."""
    K = gdn2._cabi.kernels()
    hidden = 2048
    gen = torch.Generator().manual_seed(71)
    x = torch.randn(rows, Kdim, generator=gen).to(dtype).to(DEV)
    wt = (torch.randn(hidden, Kdim, generator=gen) * 0.05).to(dtype).to(DEV)
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    epochs = torch.zeros(hidden // 32, dtype=torch.int32, device=DEV)
    for call in (1, 2):
        K.oproj_reduce(x, wt, out, None, None, epochs, 0, 1)
        want = (x.double() @ wt.double().T).float()
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert orc.rel_max_err(out.float().cpu(), want.cpu()) < tol
        assert int(epochs[0]) == call and int(epochs[-1]) == call
    K.check_device_status()


def test_fused_output_projection_two_ranks_emulated_on_one_gpu():
    """Two ranks' exchange buffers on ONE GPU, the ranks' kernels launched one after the other: rank 1 goes first,
    writes its partial sums and flags into both buffers, waits (200 k cycles) for rank 0's flags that nothing has
    set yet, gives up and reports it; rank 0 then finds rank 1's partials in place and produces the sum. Twice,
    so both parities of the double-buffered slots and the epoch counters are exercised. (Kernels that wait on
    one another must not share a GPU, so the concurrent form runs only in the multi-GPU test.)"""
    K = gdn2._cabi.kernels()
    K.check_device_status()
    hidden, rows, Kdim, world = 512, 2, 256, 2
    bufs, slots, flags, epochs = _exchange_buffers(K, world, hidden)
    gen = torch.Generator().manual_seed(73)
    w = [(torch.randn(hidden, Kdim, generator=gen) * 0.05).bfloat16().to(DEV) for _ in range(world)]
    for step in range(4):
        x = [torch.randn(rows, Kdim, generator=gen).bfloat16().to(DEV) for _ in range(world)]
        out1 = torch.empty(rows, hidden, dtype=torch.bfloat16, device=DEV)
        K.oproj_reduce(x[1], w[1], out1, slots, flags, epochs[1], 1, world, wait_cycles=200_000)
        with pytest.raises(gdn2._cabi.GDN2KernelError, match="bounded wait"):
            K.check_device_status()
        out0 = torch.empty(rows, hidden, dtype=torch.bfloat16, device=DEV)
        K.oproj_reduce(x[0], w[0], out0, slots, flags, epochs[0], 0, world, wait_cycles=200_000)
        K.check_device_status()                               # rank 0 found everything in place
        want = (x[0].double() @ w[0].double().T + x[1].double() @ w[1].double().T).float()
        assert orc.rel_max_err(out0.float().cpu(), want.cpu()) < 1e-2, step
        assert int(epochs[0][0]) == step + 1 and int(epochs[1][3]) == step + 1


@pytest.mark.parametrize("B,S,H,HK", [(2, 64 * 5, 4, 2), (4, 64 * 30, 2, 2), (1, 64 * 40, 16, 8)])
def test_gated_norm_as_scan_epilogue_equals_separate_kernel(B, S, H, HK):
    """gdn2_prefill_scan_gated_norm (the norm applied to the rows as they leave the scan; one block per head and
    the scan cut into segments) against gdn2_prefill_scan followed by gdn2_layer_back on the same bf16 rows: the
    same arithmetic on the same rounded values, the sum of squares added in another order."""
    K = gdn2._cabi.kernels()
    D = 128
    gen = torch.Generator().manual_seed(81)
    q, k, _, g, b, _ = orc.make_inputs(B, S, HK, D, D, seed=81)
    _, _, v, _, _, w = orc.make_inputs(B, S, H, D, D, seed=82)
    dev = tuple(t.bfloat16().to(DEV) for t in (q, k, v)) + (g.to(DEV), b.bfloat16().to(DEV), w.bfloat16().to(DEV))
    NP, off = H * D + 3 * 64, 2 * 64                       # gate columns inside a wider projection buffer
    proj = torch.randn(B, S, NP, generator=gen).bfloat16().to(DEV)
    weight = (1.0 + 0.1 * torch.randn(D, generator=gen)).bfloat16().to(DEV)
    eps = 1e-5
    o_plain, s_plain, _ = K.chunk_forward(*dev, D**-0.5)
    want = K.layer_back(o_plain, proj, weight, off, eps).view(B, S, H, D)
    got, s_got, _ = K.chunk_forward(*dev, D**-0.5, gated_norm=(proj, off, weight, eps))
    K.check_device_status()
    assert torch.equal(s_got, s_plain)
    diff = (got.float() - want.float()).abs()
    # the epilogue evaluates SiLU through tanh.approx (relative error 2^-11): a last-place step of bf16 at most,
    # on a minority of the entries
    assert float(diff.max()) <= 2.0**-7 * float(want.float().abs().max())
    assert float((diff > 0).float().mean()) < 0.25


def test_layer_prefill_with_the_norm_fused_into_the_scan():
    """`layer.fuse_output_norm = True` routes the gated RMSNorm through the scan's epilogue (whole chunks) and the
    separate kernel (ragged tail): same outputs as the default up to a last-place step of bf16 before o_proj."""
    cfg = gdn2.GatedDeltaNet2Config(hidden_size=256, num_heads=4, num_kv_heads=2)
    layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval().to(DEV)
    x = (torch.randn(2, 64 * 5 + 19, 256, generator=torch.Generator().manual_seed(9)) * 0.5).bfloat16().to(DEV)
    want, cache_a = layer.prefill(x)
    layer.fuse_output_norm = True
    got, cache_b = layer.prefill(x)
    assert torch.equal(cache_a.recurrent_state, cache_b.recurrent_state)
    assert orc.rel_max_err(got.float().cpu(), want.float().cpu()) < 2e-2
    assert float((got.float() - want.float()).abs().mean()) < 2e-3 * float(want.float().abs().max())


@pytest.mark.parametrize("cached", [False, True])
@pytest.mark.parametrize("S", [1, 3, 7, 8, 9, 13, 64])
def test_fused_front_d128_bf16_matches_the_operator_chain(cached, S):
    """The D = 128 16-bit forms of gdn2_layer_front (one token per warp for S < 8, four tokens per warp for
    prompts, ragged last group included) against the operator chain evaluated in float32 on the same bf16
    projection buffer: every output within bf16 rounding, the convolution cache exactly."""
    from tests.fake_kernels import layer_front_chain

    cfg = gdn2.GatedDeltaNet2Config(hidden_size=128, num_heads=4, num_kv_heads=2)
    layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval().to(DEV)
    gen = torch.Generator().manual_seed(12)
    with torch.no_grad():
        for prm in layer.parameters():
            prm.copy_((torch.randn(prm.shape, generator=gen) * 0.3).to(DEV))
    x = torch.randn(3, S, 128, generator=gen).bfloat16().to(DEV)
    state = torch.randn(3, 2 * 2 * 128 + 4 * 128, 3, generator=gen).bfloat16().to(DEV) if cached else None
    fused = layer._front(x, state, cached=cached)
    proj = fused[7].float().cpu()
    _, offs, cw, cb = layer._fused_tables()
    chain = layer_front_chain(proj, offs[:6], None if state is None else state.float().cpu(), cw.float().cpu(),
                              cb.float().cpu(), layer.A_log.detach().float().cpu(), layer.dt_bias.detach().float().cpu(),
                              4, 2, 128, 128, cfg.conv_size, float(layer.erase_scale))
    for name, a, b in zip("q k v g b w".split(), fused[:6], chain[:6]):
        assert a.shape == b.shape, name
        assert orc.rel_max_err(a.float().cpu(), b.float()) < 1e-2, name
    assert torch.equal(fused[6].float().cpu(), chain[6])          # the cache holds copies of bf16 values
    # the D = 128 form of gdn2_layer_back (four rows per warp), a row count that is not a multiple of four included
    from tests.fake_kernels import layer_back_chain

    for rows, heads in ((3, 4), (1, 3)):
        o = torch.randn(rows, S, heads, 128, generator=gen).bfloat16()
        want = layer_back_chain(o.float(), proj[:rows], layer.o_norm.weight.detach().float().cpu(), offs[6], layer.o_norm.eps)
        got = gdn2._cabi.kernels().layer_back(o.to(DEV), fused[7][:rows].contiguous(), layer.o_norm.weight.detach(), offs[6],
                                               float(layer.o_norm.eps))
        assert got.dtype == torch.bfloat16
        assert orc.rel_max_err(got.float().cpu(), want) < 1e-2
