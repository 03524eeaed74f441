"""Generate the golden fixtures in this directory from the reference project itself.

Run once, in a container where the reference checkout is importable (torch on
CPU and an importable ``tilelang`` are enough; no GPU):

    python tests/golden/make_golden.py --reference /path/to/GDT2_TileLang

Each ``*.npz`` holds the outputs of the REFERENCE's own functions
(``gdn2.reference.recurrent_gdn2`` / ``chunk_gdn2_torch`` /
``forward_intermediates``, the host branches of ``gdn2.inference.gdn2_decode`` /
``gdn2_prefill``, ``gdn2.attention.gdn2_attention`` with the torch backend and
the ``GatedDeltaNet2`` module) on seeded inputs drawn by
``oracle.gdn2_oracle.make_inputs``. The inputs themselves are not stored, only a
checksum of them, so a change in the host random generator is detected rather
than silently compared against stale outputs.

The committed fixtures are what the CPU tests pin the oracle against and what
the GPU tests compare the CUDA kernels with; nothing reads the reference at
test time.
"""

from __future__ import annotations

import argparse
import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from oracle import gdn2_oracle as orc  # noqa: E402
from oracle import layer_oracle as lorc  # noqa: E402

# name -> (B, S, H, DK, DV, gate, decay_scale, with_initial_state)
CORE_CASES = {
    "cfg0_b1_s256_h4_d64": (1, 256, 4, 64, 64, "logsigmoid16", 0.0, False),
    "small_s128_dk32_dv48": (2, 128, 3, 32, 48, "softplus", 4.0, False),
    "small_s128_dk32_dv48_s0": (2, 128, 3, 32, 48, "softplus", 4.0, True),
    "fastdecay30_s128_d32": (1, 128, 2, 32, 32, "softplus", 30.0, False),
    "d128_s128_h2": (1, 128, 2, 128, 128, "logsigmoid16", 0.0, True),
}
DECODE_CASES = {f"decode_n{n}": (2, n, 3, 32, 24) for n in (1, 3, 8, 16)}
DECODE_CASES["decode_n8_d128"] = (2, 8, 2, 128, 128)
PREFILL_CASES = {f"prefill_s{S}": (2, S, 3, 32, 24) for S in (64, 128, 100, 7)}
PREFILL_CASES["prefill_s165_d128"] = (1, 165, 2, 128, 128)

LAYER = dict(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim_k=16, head_dim_v=16)


def checksum(*tensors):
    """Order-sensitive fp64 fingerprint of the inputs."""
    acc = 0.0
    for i, t in enumerate(tensors):
        t = t.double().flatten()
        ramp = torch.arange(1, t.numel() + 1, dtype=torch.float64) / t.numel()
        acc += (i + 1) * float((t * ramp).sum())
    return np.float64(acc)


def initial_state(B, H, DK, DV, seed, std):
    gen = torch.Generator(device="cpu").manual_seed(1000 + seed)
    return torch.randn(B, H, DK, DV, generator=gen) * std


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    import gdn2  # the reference package
    from gdn2 import reference as ref

    save = lambda name, **kw: np.savez(HERE / f"{name}.npz", **{k: np.asarray(v) for k, v in kw.items()})  # noqa: E731

    for name, (B, S, H, DK, DV, gate, ds, with_s0) in CORE_CASES.items():
        q, k, v, g, b, w = orc.make_inputs(B, S, H, DK, DV, seed=0, gate=gate, decay_scale=ds)
        s0 = initial_state(B, H, DK, DV, 0, 0.5) if with_s0 else None
        scale = DK**-0.5
        o_rec, s_rec = ref.recurrent_gdn2(q, k, v, g, b, w, scale, s0, True)
        o_chk, s_chk = ref.chunk_gdn2_torch(q, k, v, g, b, w, scale, s0, True)
        out = dict(inputs_checksum=checksum(q, k, v, g, b, w), o_recurrent=o_rec, s_recurrent=s_rec,
                   o_chunk=o_chk, s_chunk=s_chk)
        if name == "cfg0_b1_s256_h4_d64":
            o_att, s_att = gdn2.gdn2_attention(q, k, v, g, b, w, output_final_state=True,
                                               config=gdn2.GDN2Config(backend="torch"))
            out.update(o_attention=o_att, s_attention=s_att)
        if name in ("small_s128_dk32_dv48_s0", "d128_s128_h2"):
            f = ref.forward_intermediates(q, k, v, g, b, w, scale, s0, 64, 16)
            out.update({f"f_{key}": f[key] for key in ("Aqk", "Ai", "W", "U", "Ktail", "h", "Un")})
        save(name, **out)

    for name, (B, n, H, DK, DV) in DECODE_CASES.items():
        q, k, v, g, b, w = orc.make_inputs(B, n, H, DK, DV, seed=1, gate="softplus", decay_scale=4.0)
        s0 = initial_state(B, H, DK, DV, 1, 0.3)
        state = s0.clone()
        o = gdn2.gdn2_decode(q, k, v, g, b, w, state, DK**-0.5)
        save(name, inputs_checksum=checksum(q, k, v, g, b, w, s0), o=o, state=state)

    for name, (B, S, H, DK, DV) in PREFILL_CASES.items():
        q, k, v, g, b, w = orc.make_inputs(B, S, H, DK, DV, seed=2, gate="softplus", decay_scale=4.0)
        s0 = initial_state(B, H, DK, DV, 2, 0.3)
        o, state = gdn2.gdn2_prefill(q, k, v, g, b, w, s0.clone(), DK**-0.5)
        save(name, inputs_checksum=checksum(q, k, v, g, b, w, s0), o=o, state=state)

    # the layer: parameters from the oracle's seeded init, loaded into the reference module
    dims = lorc.LayerDims(**LAYER)
    sd = lorc.random_state_dict(dims, seed=3, std=0.2)
    layer = gdn2.GatedDeltaNet2(gdn2.GatedDeltaNet2Config(**LAYER)).eval()
    layer.load_state_dict(sd, strict=True)
    gen = torch.Generator(device="cpu").manual_seed(4)
    x = torch.randn(2, 90, LAYER["hidden_size"], generator=gen)
    with torch.no_grad():
        full, cache_f = layer(x, use_cache=True)
        pre, cache = layer.prefill(x[:, :70])
        dec, cache = layer.decode(x[:, 70:75], cache)
        steps = torch.stack([layer.step(x[:, t], cache)[0] for t in range(75, 90)], dim=1)
    save("layer_h64", inputs_checksum=checksum(x, *sd.values()), full=full, full_state=cache_f.recurrent_state,
         full_conv=cache_f.conv_state, prefill=pre, decode=dec, steps=steps,
         final_state=cache.recurrent_state, final_conv=cache.conv_state)
    print("wrote", len(list(HERE.glob("*.npz"))), "fixtures to", HERE)


if __name__ == "__main__":
    main()
