"""Benchmark of the GDN-2 serving hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the serving prefill of the benchmark definition -- B=4, S=16037 (250 chunks of 64 plus a
37-token ragged tail), H=16, DK=DV=128, bf16 q/k/v/b/w, fp32 g, fp32 state, zero initial state --
one step = one `gdn2_prefill` over the whole batch. With N > 1 ranks (torchrun, one per GPU) every
rank runs the whole workload on its own sequences ("weak" scaling, no collective: sequences and heads
are independent); the `head_sharded` object adds the fixed global problem with its 16 heads split
over the ranks, the way a tensor-parallel layer calls the op.
Inputs are seeded synthetic tensors of the stated shapes and distributions.

One JSON line on rank 0:
  value       prefill tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e         the same metric through the public API with pinned-host inputs: per step the H2D copy
              of all six inputs and the D2H read of o are inside the timed region
  roofline    the dominant kernel's algorithmic HBM bytes per launch / its event-timed duration,
              against the measured copy bandwidth in MEASURED_PEAKS.json
  decode      state HBM GB/s of decode (n=1) and decode_multi (n=8) at B=256, H=16 (rank 0, N=1)
  cpu_baseline  the CPU oracle timed on the host cores on a bounded sample of the same workload

`--impl reference` times the reference algorithm's CPU restatement (oracle/) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import pathlib
import statistics
import subprocess
import sys
import time

import torch

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(B=4, S=16037, H=16, DK=128, DV=128)
WORKLOAD = "serving prefill B=4 S=16037 (250x64 + 37 tail) H=16 DK=DV=128 bf16 io / fp32 g,state"
FALLBACK_HBM_GBS = 6650.0


# dram__bytes_read.sum + dram__bytes_write.sum per chunk-head (64 tokens of one head), from the ncu captures
# in the committed ncu summaries (1024 chunk-heads per launch): traffic grows in proportion to the chunk-heads
NCU_DRAM_BYTES_PER_CHUNK_HEAD = {"chunk_prep": (117.602560e6 + 39.747328e6) / 1024,
                                 "prefill_scan": (77.114112e6 + 5.137408e6) / 1024}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock and throttle-reason samples while the timed region runs: NVML from a thread (a sample
    every 2 ms), or nvidia-smi in a child process when the NVML binding is missing. Read-only."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    MASKS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def _nvml_loop(self, nv, h):
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                self._sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = int(get_reasons(h))
                for name, bit in self.MASKS.items():
                    if mask & bit:
                        self._reasons.add(name)
            except Exception:
                break
            self._stop.wait(0.002)

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc = gpu_index, None

    def __enter__(self):
        self._thread = None
        try:
            import threading
            nv, h = self._nvml_handle()
            self._max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            self._sm, self._reasons, self._stop = [], set(), threading.Event()
            self._thread = threading.Thread(target=self._nvml_loop, args=(nv, h), daemon=True)
            self._thread.start()
            return self
        except Exception:
            self._thread = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            if self._sm:
                self.result = {"sm_mhz": statistics.median(self._sm), "sm_max_mhz": self._max,
                               "reasons": sorted(self._reasons), "samples": len(self._sm), "source": "nvml"}
            return
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            busy = [x for x in sm if x > 0]
            self.result = {"sm_mhz": statistics.median(busy or sm), "sm_max_mhz": max(mx),
                           "reasons": sorted(reasons), "samples": len(sm)}


def device_inputs(B, S, H, DK, DV, device, seed):
    """Seeded synthetic inputs generated on the device (same distributions as the oracle's make_inputs)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    kw = dict(generator=gen, dtype=torch.float32, device=device)
    norm = torch.nn.functional.normalize
    q = norm(torch.randn(B, S, H, DK, **kw), dim=-1).bfloat16()
    k = norm(torch.randn(B, S, H, DK, **kw), dim=-1).bfloat16()
    v = torch.randn(B, S, H, DV, **kw).bfloat16()
    g = torch.nn.functional.logsigmoid(torch.randn(B, S, H, DK, **kw)) / 16.0
    b = torch.sigmoid(torch.randn(B, S, H, DK, **kw)).bfloat16()
    w = torch.sigmoid(torch.randn(B, S, H, DV, **kw)).bfloat16()
    return q, k, v, g, b, w


def time_events(fn, steps, warmup, stream_sync):
    for _ in range(warmup):
        fn()
    stream_sync()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / steps   # ms per step


def cpu_baseline(threads):
    """The oracle's prefill over the whole benchmark workload, one sequence (B = 1) at a time so that the
    fp32 intermediates stay within a few GB: 4 x 16037 tokens, H=16, D=128, fp32 (about 10 s of CPU work)."""
    from oracle import gdn2_oracle as orc

    torch.set_num_threads(threads)
    B, S = CFG["B"], CFG["S"]
    warm = orc.make_inputs(1, 128, CFG["H"], CFG["DK"], CFG["DV"], seed=0)
    orc.prefill(*warm)
    dt = 0.0
    for i in range(B):
        ins = orc.make_inputs(1, S, CFG["H"], CFG["DK"], CFG["DV"], seed=i)
        t = time.perf_counter()
        orc.prefill(*ins)
        dt += time.perf_counter() - t
        del ins
    return B * S / dt, f"the whole workload, {B} passes of B=1 S={S} H=16 DK=DV=128 fp32 ({dt:.1f} s)"


def run_reference(args, rank, world):
    """CPU arm: the reference algorithm (oracle restatement of gdn2/reference.py) on the host cores."""
    if rank != 0:
        return
    from oracle import gdn2_oracle as orc

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    S = 63 * 64 + 5
    ins = orc.make_inputs(1, S, CFG["H"], CFG["DK"], CFG["DV"], seed=0)
    for _ in range(args.warmup):
        orc.prefill(*ins)
    t = time.perf_counter()
    for _ in range(args.steps):
        orc.prefill(*ins)
    dt = (time.perf_counter() - t) / args.steps
    val = S / dt
    sample = f"each step: oracle prefill of B=1 S={S} H=16 DK=DV=128 fp32 (a bounded sample of the workload)"
    print(json.dumps({
        "impl": "reference", "metric": "gdn2_prefill_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg")
    ap.add_argument("--skip-decode", action="store_true", help="omit the decode leg")
    ap.add_argument("--skip-layer", action="store_true", help="omit the layer leg (launch-list captures)")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the end-to-end leg (launch-list captures)")
    ap.add_argument("--profile-case", choices=["prefill", "decode"],
                    help="run a small case a profiler can capture (3 iterations, no JSON line) and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return run_reference(args, rank, world)

    import torch.distributed as dist

    import gdn2_tilelang_b200 as gdn2
    from gdn2_tilelang_b200 import _cabi

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no host path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")      # keeps NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=dev)
    B, S, H, DK, DV = (CFG[x] for x in ("B", "S", "H", "DK", "DV"))
    if args.profile_case:
        # small enough for a multi-pass capture, larger than L2: prefill B=1 S=4096+37 (workspace 107 MB),
        # decode B=128 (state 134 MB)
        if args.profile_case == "prefill":
            ins = device_inputs(1, 4096 + 37, H, DK, DV, dev, seed=0)
            for _ in range(3):
                gdn2.gdn2_prefill(*ins)
        else:
            state = torch.randn(128, H, DK, DV, device=dev) * 0.02
            for n in (1, 8):
                dq = device_inputs(128, n, H, DK, DV, dev, seed=n)
                for _ in range(3):
                    gdn2.gdn2_decode(*dq, state)
        torch.cuda.synchronize()
        _cabi.kernels().check_device_status(dev)
        print(f"profile case {args.profile_case} done")
        return
    # N > 1: data parallel. Every rank runs the whole workload on its own sequences (seeded by rank);
    # the op has no cross-sequence or cross-head term, so there is no collective on the data path.
    Hl = H
    K = _cabi.kernels()
    q, k, v, g, b, w = device_inputs(B, S, Hl, DK, DV, dev, seed=rank)
    ins = (q, k, v, g, b, w)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def step():
        return gdn2.gdn2_prefill(*ins)

    # ---- headline: inputs resident in HBM
    barrier()
    launches0 = K.launches
    with ClockSampler(local) as clk:
        ms = time_events(step, args.steps, args.warmup, barrier)
    launches = (K.launches - launches0) // (args.steps + args.warmup) * args.steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    tokens = B * S * world
    value = tokens / (ms * 1e-3)
    K.check_device_status(dev)

    # ---- the other way to use N GPUs: ONE copy of the workload with its heads split over the ranks
    # (how a tensor-parallel layer calls the op); fixed global problem, still no collective
    head_sharded = None
    if world > 1 and H % world == 0:
        hs_ins = device_inputs(B, S, H // world, DK, DV, dev, seed=1000 + rank)
        barrier()
        ms_hs = time_events(lambda: gdn2.gdn2_prefill(*hs_ins), args.steps, args.warmup, barrier)
        t = torch.tensor([ms_hs], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_hs = float(t.item())
        head_sharded = {"heads_per_gpu": H // world, "ms_per_step": ms_hs, "value": B * S / (ms_hs * 1e-3),
                        "unit": "tokens/s", "scaling": "strong"}
        del hs_ins

    # ---- end to end: pinned host inputs, H2D + kernels + D2H of o per step
    host = [x.cpu().pin_memory() for x in ins]
    o_host = torch.empty(B, S, Hl, DV, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        gdn2.gdn2_prefill_from_host(*host, device=dev, out=o_host)

    barrier()
    e2e_steps = max(2, min(args.steps, 5))
    ms_e2e = float("nan") if args.skip_e2e else time_events(e2e_step, e2e_steps, 1, barrier)
    t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())
    h2d = sum(x.numel() * x.element_size() for x in host) * world
    d2h = o_host.numel() * o_host.element_size() * world
    del host, o_host

    # ---- per-kernel timing of the two chunkwise stages (same stream, CUDA events)
    n_full = S // 64 * 64
    code = _cabi.dtype_code(q.dtype)
    path = K.resolved_path(DK, DV, q.dtype)
    nbytes = K.lib.gdn2_prefill_workspace_bytes(B, n_full, Hl, DK, DV, code, path)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    o = torch.empty(B, S, Hl, DV, dtype=torch.bfloat16, device=dev)
    fin = torch.empty(B, Hl, DK, DV, dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream

    def prep():
        rc = K.lib.gdn2_chunk_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                   w.data_ptr(), ws.data_ptr(), nbytes, B, n_full, Hl, DK, DV, S, DK**-0.5,
                                   code, path, st)
        assert rc == 0, rc

    def scan():
        rc = K.lib.gdn2_prefill_scan(ws.data_ptr(), nbytes, None, o.data_ptr(), fin.data_ptr(), None,
                                     B, n_full, Hl, DK, DV, S, code, path, st)
        assert rc == 0, rc

    ms_prep = time_events(prep, args.steps, 3, barrier)
    ms_scan = time_events(scan, args.steps, 3, barrier)
    th = B * n_full * Hl                                   # token-heads per launch on this rank
    ws_per_th = (2 * DK * 2 + 64 * 2 + DK * 2 + DV * 2) + DK * 4 / 64.0   # WQ + AQK + KG^T + U^T (fp16) + gamma_last
    in_per_th = 3 * DK * 2 + 2 * DV * 2 + DK * 4                          # q,k,b + v,w (bf16) + g (fp32)
    stages = {
        "chunk_prep": (ms_prep, th * (in_per_th + ws_per_th)),
        "prefill_scan": (ms_scan, th * (ws_per_th + DV * 2) + B * Hl * DK * DV * 4),
    }
    dom = max(stages, key=lambda s: stages[s][0])
    peak, peak_kind = measured_peaks()
    dom_ms, dom_bytes = stages[dom]
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
    whole_op_bytes = B * S * Hl * 2048.0                  # per GPU
    roofline = {
        "bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak, "peak_source": f"{peak_kind} copy bandwidth",
        "traffic": NCU_DRAM_BYTES_PER_CHUNK_HEAD[dom] * (th / 64) / 1e9, "traffic_unit": "GB per launch",
        "traffic_source": "dram__bytes_read+write of one ncu capture of a 1024-chunk-head launch "
                          "(the committed ncu summary of the prefill kernels), scaled by chunk-heads; writes still in L2 "
                          "when the small launch ends are not in it",
        "stages_ms": {s: stages[s][0] for s in stages},
        "stages_frac": {s: stages[s][1] / (stages[s][0] * 1e-3) / 1e9 / peak for s in stages},
        "whole_op_frac": whole_op_bytes / (ms * 1e-3) / 1e9 / peak,       # per GPU, of its own HBM
    }
    del ws, o, fin

    # ---- decode leg (benchmark definition: B=256, H=16, state ~ N(0, 0.02))
    decode = None
    if rank == 0 and world == 1 and not args.skip_decode:
        Bd = 256
        state = torch.randn(Bd, H, DK, DV, device=dev) * 0.02
        decode = {"unit": "GB/s (state read + write only)", "B": Bd, "H": H}
        for n in (1, 8):
            dq = device_inputs(Bd, n, H, DK, DV, dev, seed=100 + n)
            ms_d = time_events(lambda: gdn2.gdn2_decode(*dq, state), 20, 5, torch.cuda.synchronize)
            gbs = 2 * Bd * H * DK * DV * 4 / (ms_d * 1e-3) / 1e9
            decode[f"n{n}"] = {"ms": ms_d, "state_gbs": gbs, "frac_of_peak": gbs / peak,
                               "total_gbs": (2 * Bd * H * DK * DV * 4 + Bd * n * H * 2048) / (ms_d * 1e-3) / 1e9}
        del state

    # ---- the layer around the op (hidden 2048, 16 heads, 8 kv heads, D = 128, bf16): prefill of
    # [2, 4096, hidden], then 128 one-token steps, eager and replayed from a CUDA graph
    layer_leg = None
    if rank == 0 and world == 1 and not args.skip_layer:
        cfg = gdn2.GatedDeltaNet2Config(hidden_size=2048, num_heads=16, num_kv_heads=8)
        gen = torch.Generator(device=dev).manual_seed(0)
        layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval().to(dev)
        with torch.no_grad():
            for name, prm in layer.named_parameters():      # projections ~ N(0, 0.02); gate parameters keep their init
                if name.endswith("proj.weight"):
                    prm.copy_(torch.randn(prm.shape, device=dev, generator=gen) * 0.02)
        x = torch.randn(2, 4096, 2048, device=dev, generator=gen).bfloat16()
        ms_pre = time_events(lambda: layer.prefill(x), 5, 3, torch.cuda.synchronize)
        _, cache = layer.prefill(x)
        xt = torch.randn(2, 2048, device=dev, generator=gen).bfloat16()

        def eager_steps():
            for _ in range(128):
                layer.step(xt, cache)

        ms_eager = time_events(eager_steps, 3, 1, torch.cuda.synchronize)
        step = gdn2.GraphedStep(layer, cache)

        def graphed_steps():
            for _ in range(128):
                step(xt)

        ms_graph = time_events(graphed_steps, 3, 1, torch.cuda.synchronize)
        layer_leg = {"config": "hidden 2048, H=16, HK=8, DK=DV=128, bf16, x [2,4096,2048]",
                     "prefill_ms": ms_pre, "prefill_tokens_per_s": 2 * 4096 / (ms_pre * 1e-3),
                     "step_us_eager": ms_eager * 1e3 / 128, "step_us_cuda_graph": ms_graph * 1e3 / 128}
        del layer, x, cache, step

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        threads = os.cpu_count() or 1
        val, sample = cpu_baseline(threads)
        cpu = {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        print(json.dumps({
            "metric": "gdn2_prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "heads_per_gpu": Hl,
                       "parallelism": f"data-parallel x{world}: the whole workload per GPU on its own sequences, no collective",
                       "l2": "inputs (2.1 GB) exceed L2, no flush needed", "prefill_path":
                       {1: "simt", 2: "tcgen05"}[path]},
            "clocks": clk.result,
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches * world,
            "roofline": roofline, "decode": decode, "layer": layer_leg, "cpu_baseline": cpu,
            "head_sharded": head_sharded,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
