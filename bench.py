"""Benchmark of the GDN-2 serving hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: the serving prefill of the benchmark definition -- B=4, S=16037 (250 chunks of 64 plus a
37-token ragged tail), H=16, DK=DV=128, bf16 q/k/v/b/w, fp32 g, fp32 state, zero initial state --
one step = one `gdn2_prefill` over the whole batch. With N > 1 ranks (torchrun, one per GPU) the SAME
global problem is split by heads, 16 / N per rank ("strong" scaling; sequences and heads are independent,
so there is no collective on the data path) and `value` = global tokens / max-over-ranks time; the
`replicas` object adds the other way to use N GPUs, every rank running the whole workload on its own
sequences. Inputs are seeded synthetic tensors of the stated shapes and distributions.

One JSON line on rank 0:
  value       prefill tokens/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e         the same metric through the public API with pinned-host inputs: per step the H2D copy
              of all six inputs and the D2H read of o are inside the timed region
  parity      the outputs of the timed GPU step (N > 1: of rank 0's head shard) against the CPU path's outputs on the same
              bf16-rounded inputs: output max-abs error and final-state relative Frobenius error
  roofline    the dominant kernel's algorithmic HBM bytes per launch / its event-timed duration,
              against the measured copy bandwidth in MEASURED_PEAKS.json
  decode      state HBM GB/s of decode (n=1) and decode_multi (n=8) at B=256, H=16 (rank 0, N=1)
  layer       the full layer (hidden 2048, 16 heads, 8 kv heads): prefill of [2,4096,2048] and 128 one-token
              steps; with N > 1 the head-parallel layer with its all-reduce after o_proj inside the timed
              region, the all-reduce's own time for both message sizes, and a parity check against the
              unsharded layer
  cpu_baseline  the reference's CPU path (oracle/_ref when built, else the oracle port) timed on the host
              cores on the whole workload, one sequence at a time

`--impl reference` times that CPU path alone, the whole workload per step.
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
NCU_DRAM_BYTES_PER_CHUNK_HEAD = {"chunk_prep": (117.523456e6 + 38.075648e6) / 1024,
                                 "prefill_scan": (77.139968e6 + 4.598784e6 + 37.224704e6 + 0.046848e6) / 1024}   # first + redo pass


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


def config_dict(world):
    """The workload description both arms print: identical for `--impl ours` and `--impl reference`."""
    H = CFG["H"]
    par = ("one GPU" if world == 1 else
           f"heads split over {world} GPUs ({H // world} per GPU), one global problem, no collective")
    return {"workload": WORKLOAD, "parallelism": par, "l2": "inputs (2.1 GB) exceed L2, no flush needed"}


# ---- the CPU arm: the reference's own host path, or its restatement ---------------------------------------


def cpu_prefill_fn():
    """(prefill(q,k,v,g,b,w) -> (o, state), kind): the reference's own gdn2/reference.py when the build step
    placed a copy under oracle/_ref (chunk_gdn2_torch on the whole chunks, the token recurrence on the ragged
    tail: the host branch of the reference's gdn2_prefill), else the oracle restatement."""
    from oracle.build_ref import load_ref

    ref = load_ref()
    if ref is not None:

        def prefill(q, k, v, g, b, w):
            S, DK = q.shape[1], q.shape[-1]
            scale, n_full = DK**-0.5, S // 64 * 64
            o1, state = ref.chunk_gdn2_torch(*(t[:, :n_full] for t in (q, k, v, g, b, w)), scale, None, True)
            o2, state = ref.recurrent_gdn2(*(t[:, n_full:] for t in (q, k, v, g, b, w)), scale, state, True)
            return torch.cat([o1, o2], 1), state

        return prefill, "reference"
    from oracle import gdn2_oracle as orc

    return (lambda *ins: orc.prefill(*ins)), "port"


def host_sequences(B, S, H, DK, DV):
    """Per sequence i (seed i): bf16-rounded host inputs as fp32, the values both arms compute on."""
    from oracle import gdn2_oracle as orc

    seqs = []
    for i in range(B):
        q, k, v, g, b, w = orc.make_inputs(1, S, H, DK, DV, seed=i)
        seqs.append(tuple(t.bfloat16().float() for t in (q, k, v)) + (g, b.bfloat16().float(), w.bfloat16().float()))
    return seqs


def cpu_workload_pass(prefill, seqs):
    """One pass of the CPU path over the whole workload, one sequence (B = 1) at a time so that the fp32
    intermediates stay within a few GB. Returns (seconds, [o_i], [state_i])."""
    outs, states, dt = [], [], 0.0
    for ins in seqs:
        t = time.perf_counter()
        o, s = prefill(*ins)
        dt += time.perf_counter() - t
        outs.append(o)
        states.append(s)
    return dt, outs, states


def run_reference(args, rank, world):
    """CPU arm: the reference's host path on the box's cores, the whole workload per step."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    B, S, H, DK, DV = (CFG[x] for x in ("B", "S", "H", "DK", "DV"))
    prefill, kind = cpu_prefill_fn()
    seqs = host_sequences(B, S, H, DK, DV)
    for _ in range(args.warmup):
        cpu_workload_pass(prefill, seqs[:1])                 # warm-up: one sequence is enough to page everything in
    total = 0.0
    for _ in range(args.steps):
        total += cpu_workload_pass(prefill, seqs)[0]
    dt = total / args.steps
    val = B * S / dt
    sample = (f"each step: the whole workload, {B} passes of B=1 S={S} H={H} DK=DV={DK} fp32 on bf16-rounded inputs; "
              f"warm-up steps run one sequence")
    print(json.dumps({
        "impl": "reference", "metric": "gdn2_prefill_tokens_per_s", "value": val, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(world),
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (and with it the parity object)")
    ap.add_argument("--skip-decode", action="store_true", help="omit the decode leg")
    ap.add_argument("--skip-layer", action="store_true", help="omit the layer leg (launch-list captures)")
    ap.add_argument("--skip-e2e", action="store_true", help="omit the end-to-end leg (launch-list captures)")
    ap.add_argument("--heads", type=int, default=None,
                    help="single GPU only: run the problem of ONE rank of a head-sharded job (this many of the 16 heads)")
    ap.add_argument("--profile-case", choices=["prefill", "prefill-sharded", "decode", "output", "layer", "simt"],
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
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # exchange buffers use plain peer stores only
        import datetime
        # NCCL writes its version banner to the C-level stdout when the first communicator comes up; this process's
        # stdout is for the one JSON line, so file descriptor 1 points at stderr until the communicator exists
        sys.stdout.flush()
        saved_fd = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_fd, 1)
            os.close(saved_fd)
    B, S, H, DK, DV = (CFG[x] for x in ("B", "S", "H", "DK", "DV"))
    K = _cabi.kernels()
    if args.profile_case:
        # small enough for a multi-pass capture, larger than L2: prefill B=1 S=4096+37 (workspace 107 MB),
        # the same with 2 heads and the full length (the scan cut into segments), decode B=128 (state 134 MB),
        # chunk-parallel output B=1 S=4096 H=16 (chunk states 67 MB + workspace 76 MB), the layer's prefill at the
        # benchmark's layer size
        if args.profile_case == "prefill":
            ins = device_inputs(1, 4096 + 37, H, DK, DV, dev, seed=0)
            for _ in range(3):
                gdn2.gdn2_prefill(*ins)
        elif args.profile_case == "prefill-sharded":
            ins = device_inputs(4, 16037, 2, DK, DV, dev, seed=0)
            for _ in range(3):
                gdn2.gdn2_prefill(*ins)
        elif args.profile_case == "layer":
            cfg = gdn2.GatedDeltaNet2Config(hidden_size=2048, num_heads=16, num_kv_heads=8)
            torch.manual_seed(0)
            layer = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval().to(dev)
            x = torch.randn(2, 4096, 2048, device=dev).bfloat16()      # projection buffer 201 MB, larger than L2
            for _ in range(3):
                layer.prefill(x)
        elif args.profile_case == "simt":
            # the exact CUDA-core family (what fp32 / fp16 inputs and head sizes other than 128 take): fp32, D = 128
            ins = tuple(t.float() for t in device_inputs(1, 2048, H, DK, DV, dev, seed=0))
            for _ in range(3):
                gdn2.gdn2_prefill(*ins)
        elif args.profile_case == "output":
            ins = device_inputs(1, 4096, H, DK, DV, dev, seed=0)
            _, _, hs = gdn2.chunk_gdn2_fwd(*ins, DK**-0.5, None, False, return_chunk_states=True)
            for _ in range(3):
                gdn2.chunk_gdn2_output(*ins, DK**-0.5, hs)
        else:
            state = torch.randn(128, H, DK, DV, device=dev) * 0.02
            for n in (1, 8):
                dq = device_inputs(128, n, H, DK, DV, dev, seed=n)
                for _ in range(3):
                    gdn2.gdn2_decode(*dq, state)
        torch.cuda.synchronize()
        K.check_device_status(dev)
        print(f"profile case {args.profile_case} done")
        return

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- inputs. One GPU: host-generated, bf16-rounded, the very values the CPU baseline computes on (its
    # outputs are kept for the parity object). N GPUs: the global problem generated identically on every
    # device, this rank keeping its 16 / N heads.
    cpu, cpu_ref = None, None
    run_cpu = rank == 0 and world == 1 and not args.skip_cpu and args.heads is None
    if world > 1 and H % world:
        raise SystemExit(f"{H} heads do not split over {world} GPUs")
    Hl = H // world if world > 1 else (args.heads or H)
    if run_cpu:
        threads = os.cpu_count() or 1
        torch.set_num_threads(threads)
        prefill_cpu, kind = cpu_prefill_fn()
        seqs = host_sequences(B, S, H, DK, DV)
        cpu_workload_pass(prefill_cpu, [tuple(t[:, :128] for t in seqs[0])])       # warm-up
        dt, o_ref, s_ref = cpu_workload_pass(prefill_cpu, seqs)
        cpu = {"value": B * S / dt, "unit": "tokens/s", "cores": threads, "kind": kind,
               "sample": f"the whole workload, {B} passes of B=1 S={S} H={H} DK=DV={DK} fp32 on the bf16-rounded "
                         f"inputs of the GPU arm ({dt:.1f} s)"}
        cpu_ref = (torch.cat(o_ref, 0), torch.cat(s_ref, 0))
        ins = tuple(torch.cat([sq[j] for sq in seqs], 0).to(torch.float32 if j == 3 else torch.bfloat16).to(dev)
                    for j in range(6))
        del seqs, o_ref, s_ref
    else:
        full = device_inputs(B, S, H, DK, DV, dev, seed=0)
        h0 = rank * Hl if world > 1 else 0
        ins = tuple(t[:, :, h0:h0 + Hl].contiguous() for t in full)
        del full
    q, k, v, g, b, w = ins

    def step():
        return gdn2.gdn2_prefill(*ins)

    # ---- headline: inputs resident in HBM
    barrier()
    launches0 = K.launches
    with ClockSampler(local) as clk:
        ms = max_over_ranks(time_events(step, args.steps, args.warmup, barrier))
    launches = (K.launches - launches0) // (args.steps + args.warmup) * args.steps
    launches_all = max_over_ranks(float(launches)) * world
    tokens = B * S                                         # the global problem, whatever N
    value = tokens / (ms * 1e-3) * (Hl * world / H)        # --heads: scaled to the share of the problem that ran
    K.check_device_status(dev)

    parity, parity_job = None, None
    if cpu_ref is not None:
        o_gpu, s_gpu = step()
        torch.cuda.synchronize()
        o_cpu, s_cpu = cpu_ref
        parity = {"o_max_abs": float((o_gpu.float().cpu() - o_cpu).abs().max()),
                  "state_rel_fro": float((s_gpu.cpu() - s_cpu).norm() / s_cpu.norm()),
                  "against": cpu["kind"], "bounds": {"o_max_abs": 2e-2, "state_rel_fro": 1e-3}}
        parity["ok"] = bool(parity["o_max_abs"] <= 2e-2 and parity["state_rel_fro"] <= 1e-3)
        del o_gpu, s_gpu, cpu_ref
    elif world > 1 and rank == 0 and not args.skip_cpu:
        # N GPUs: rank 0 checks its own head shard (heads are independent) against the CPU path on the same values.
        # The outputs of sequence 0 are kept here; the CPU pass itself runs after every timed leg (its worker
        # threads would otherwise compete with the end-to-end leg's copies).
        o_gpu, s_gpu = step()
        torch.cuda.synchronize()
        parity_job = (tuple(t[0:1].float().cpu() for t in ins), o_gpu[0:1].float().cpu(), s_gpu[0:1].cpu())
        del o_gpu, s_gpu

    # ---- end to end: pinned host inputs, H2D + kernels + D2H of o per step
    host = [x.cpu().pin_memory() for x in ins]
    o_host = torch.empty(B, S, Hl, DV, dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        gdn2.gdn2_prefill_from_host(*host, device=dev, out=o_host)

    barrier()
    e2e_steps = max(2, min(args.steps, 5))
    ms_e2e = float("nan") if args.skip_e2e else time_events(e2e_step, e2e_steps, 1, barrier)
    ms_e2e = max_over_ranks(ms_e2e)
    h2d = sum(x.numel() * x.element_size() for x in host) * world
    d2h = o_host.numel() * o_host.element_size() * world
    del host, o_host

    # ---- per-kernel timing of the two chunkwise stages (same stream, CUDA events) on this rank's problem
    n_full = S // 64 * 64
    code = _cabi.dtype_code(q.dtype)
    path = K.resolved_path(DK, DV, q.dtype)
    nbytes = K.lib.gdn2_prefill_workspace_bytes(B, n_full, Hl, Hl, DK, DV, code, path)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    o = torch.empty(B, S, Hl, DV, dtype=torch.bfloat16, device=dev)
    fin = torch.empty(B, Hl, DK, DV, dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream

    def prep():
        rc = K.lib.gdn2_chunk_prep(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), b.data_ptr(),
                                   w.data_ptr(), ws.data_ptr(), nbytes, B, n_full, Hl, Hl, DK, DV, S, DK**-0.5,
                                   code, path, st)
        assert rc == 0, rc

    def scan():
        rc = K.lib.gdn2_prefill_scan(ws.data_ptr(), nbytes, None, o.data_ptr(), fin.data_ptr(), None,
                                     B, n_full, Hl, Hl, DK, DV, S, code, path, st)
        assert rc == 0, rc

    ms_prep = time_events(prep, args.steps, 3, barrier)
    ms_scan = time_events(scan, args.steps, 3, barrier)
    scan_segments = K.scan_segments(B, n_full, Hl, DK, DV, q.dtype, path)
    th = B * n_full * Hl                                   # token-heads per launch on this rank
    ws_per_th = (2 * DK * 2 + 64 * 2 + DK * 2 + DV * 2) + DK * 4 / 64.0   # WQ + AQK + KG^T + U^T (fp16) + gamma_last
    in_per_th = 3 * DK * 2 + 2 * DV * 2 + DK * 4                          # q,k,b + v,w (bf16) + g (fp32)
    stages = {
        "chunk_prep": (ms_prep, th * (in_per_th + ws_per_th)),
        "prefill_scan": (ms_scan, th * (ws_per_th + DV * 2) + B * Hl * DK * DV * 4),
    }
    dom = max(stages, key=lambda s_: stages[s_][0])
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
        "stages_ms": {s_: stages[s_][0] for s_ in stages},
        "stages_frac": {s_: stages[s_][1] / (stages[s_][0] * 1e-3) / 1e9 / peak for s_ in stages},
        "stage_sum_frac": sum(stages[s_][1] for s_ in stages) / 1e9 / peak / (sum(stages[s_][0] for s_ in stages) * 1e-3),
        "whole_op_frac": whole_op_bytes / (ms * 1e-3) / 1e9 / peak,       # per GPU, of its own HBM
        "scan_segments": scan_segments,
    }
    del ws, o, fin

    # ---- the other way to use N GPUs: every rank runs the whole workload on its own sequences
    replicas = None
    if world > 1:
        rep_ins = device_inputs(B, S, H, DK, DV, dev, seed=1000 + rank)
        barrier()
        ms_rep = max_over_ranks(time_events(lambda: gdn2.gdn2_prefill(*rep_ins), max(3, args.steps // 2), 3, barrier))
        replicas = {"ms_per_step": ms_rep, "value": B * S * world / (ms_rep * 1e-3), "unit": "tokens/s", "scaling": "weak"}
        del rep_ins

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

    layer_leg = None if args.skip_layer else layer_bench(gdn2, dist, dev, rank, world, barrier, max_over_ranks)

    if world > 1:
        barrier()
        dist.destroy_process_group()                       # every rank is done with the GPUs; what follows is host work of rank 0
    if parity_job is not None:
        torch.set_num_threads(max(1, min(16, (os.cpu_count() or 1) // world)))
        prefill_cpu, kind = cpu_prefill_fn()
        p_in, o_g, s_g = parity_job
        o_c, s_c = prefill_cpu(*p_in)
        parity = {"o_max_abs": float((o_g - o_c).abs().max()), "state_rel_fro": float((s_g - s_c).norm() / s_c.norm()),
                  "against": kind, "scope": f"rank 0's shard: heads 0..{Hl - 1} of {H}, sequence 0 of {B}",
                  "bounds": {"o_max_abs": 2e-2, "state_rel_fro": 1e-3}}
        parity["ok"] = bool(parity["o_max_abs"] <= 2e-2 and parity["state_rel_fro"] <= 1e-3)
    if rank == 0:
        cfg = config_dict(world)
        if args.heads is not None:
            cfg["parallelism"] = f"ONE rank's share of a head-sharded job: {Hl} of {H} heads on one GPU"
        print(json.dumps({
            "metric": "gdn2_prefill_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": cfg, "heads_per_gpu": Hl, "prefill_path": {1: "simt", 2: "tcgen05", 3: "tcgen05"}[path],
            "clocks": clk.result,
            "e2e": {"value": tokens * (Hl * world / H) / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches_all), "parity": parity,
            "roofline": roofline, "decode": decode, "layer": layer_leg, "cpu_baseline": cpu,
            "replicas": replicas,
        }))


def layer_bench(gdn2, dist, dev, rank, world, barrier, max_over_ranks):
    """The layer around the op (hidden 2048, 16 heads, 8 kv heads, D = 128, bf16 weights ~ N(0, 0.02)): prefill of
    x [2, 4096, 2048], then 128 one-token steps. One GPU: eager and replayed from a CUDA graph. N GPUs: the
    head-parallel layer, its one all-reduce after o_proj inside the timed region; the all-reduce alone is timed
    for both message sizes, and every rank's output is compared with the unsharded layer run on the same GPU."""
    cfg = gdn2.GatedDeltaNet2Config(hidden_size=2048, num_heads=16, num_kv_heads=8)
    gen = torch.Generator(device=dev).manual_seed(0)
    torch.manual_seed(0)                                   # the constructor's own draws (conv, gates): the same layer on every rank
    full = gdn2.GatedDeltaNet2(cfg).to(torch.bfloat16).eval().to(dev)
    with torch.no_grad():
        for name, prm in full.named_parameters():      # projections ~ N(0, 0.02); gate parameters keep their init
            if name.endswith("proj.weight"):
                prm.copy_(torch.randn(prm.shape, device=dev, generator=gen) * 0.02)
    x = torch.randn(2, 4096, 2048, device=dev, generator=gen).bfloat16()
    xt = torch.randn(2, 2048, device=dev, generator=gen).bfloat16()
    sync = barrier
    leg = {"config": "hidden 2048, H=16, HK=8, DK=DV=128, bf16, x [2,4096,2048], then 128 one-token steps"}
    if world == 1:
        layer = full
    else:
        if cfg.num_kv_heads % world:
            return {"skipped": f"{cfg.num_kv_heads} kv heads do not split over {world} GPUs"}
        layer = gdn2.TensorParallelGatedDeltaNet2(cfg).to(torch.bfloat16).eval()
        layer.load_full_state_dict({k_: v_.cpu() for k_, v_ in full.state_dict().items()})   # same seed on every rank
        layer.to(dev)
        # parity of the sharded layer with the unsharded one (prefill + 4 steps), on every rank
        ref_out, ref_cache = full.prefill(x)
        got_out, got_cache = layer.prefill(x)
        errs = [float((got_out.float() - ref_out.float()).abs().max() / ref_out.float().abs().max())]
        for _ in range(4):
            r_, ref_cache = full.step(xt, ref_cache)
            g_, got_cache = layer.step(xt, got_cache)
            errs.append(float((g_.float() - r_.float()).abs().max() / r_.float().abs().max()))
        hl = cfg.num_heads // world
        s_ref = ref_cache.recurrent_state[:, rank * hl:(rank + 1) * hl]
        s_err = float((got_cache.recurrent_state - s_ref).norm() / s_ref.norm())
        leg["tp_parity"] = {"out_rel_max": max_over_ranks(max(errs)), "state_rel_fro": max_over_ranks(s_err),
                            "bounds": {"out_rel_max": 2e-2, "state_rel_fro": 1e-3}}
        leg["tp_parity"]["ok"] = bool(leg["tp_parity"]["out_rel_max"] <= 2e-2 and leg["tp_parity"]["state_rel_fro"] <= 1e-3)
        del ref_out, got_out, ref_cache, got_cache
    ms_pre = max_over_ranks(time_events(lambda: layer.prefill(x), 5, 3, sync))
    _, cache = layer.prefill(x)

    def eager_steps():
        for _ in range(128):
            layer.step(xt, cache)

    ms_eager = max_over_ranks(time_events(eager_steps, 3, 1, sync))
    leg.update(prefill_ms=ms_pre, prefill_tokens_per_s=2 * 4096 / (ms_pre * 1e-3), step_us_eager=ms_eager * 1e3 / 128)
    if world == 1:
        step = gdn2.GraphedStep(layer, cache)

        def graphed_steps():
            for _ in range(128):
                step(xt)

        leg["step_us_cuda_graph"] = time_events(graphed_steps, 3, 1, sync) * 1e3 / 128
    else:
        big = torch.zeros(2, 4096, 2048, device=dev, dtype=torch.bfloat16)       # 32 MiB: the prefill message
        small = torch.zeros(2, 2048, device=dev, dtype=torch.bfloat16)           # 8 KiB: the step message
        ms_big = max_over_ranks(time_events(lambda: dist.all_reduce(big), 10, 3, sync))
        ms_small = max_over_ranks(time_events(lambda: dist.all_reduce(small), 200, 20, sync))
        leg["all_reduce"] = {"prefill_32MiB_ms": ms_big, "prefill_share": ms_big / ms_pre,
                             "step_8KiB_us": ms_small * 1e3, "step_share": ms_small * 1e3 / (ms_eager * 1e3 / 128),
                             "backend": "nccl", "n_ranks": world}
        # o_proj + sum over ranks as ONE kernel (peer stores over NVLink), eager and replayed from a CUDA graph.
        # The set-up is collective; whether it worked is agreed on by all ranks before anyone goes on.
        ok, msg = 1.0, ""
        try:
            layer.enable_fused_reduce()
        except Exception as e:
            ok, msg = 0.0, f"{type(e).__name__}: {e}"[:300]
        if -max_over_ranks(-ok) < 1.0:
            layer.fused_reduce = None
            leg["fused_reduce"] = {"error": msg or "the set-up failed on another rank"}
            return leg
        keep, layer.fused_reduce = layer.fused_reduce, None
        _, cache_n = layer.prefill(x)
        y_nccl, _ = layer.step(xt, cache_n)
        layer.fused_reduce = keep
        _, cache_f = layer.prefill(x)
        y_fused, _ = layer.step(xt, cache_f)
        err = float((y_fused.float() - y_nccl.float()).abs().max() / y_nccl.float().abs().max())
        ms_fused = max_over_ranks(time_events(eager_steps, 3, 1, sync))
        step = gdn2.GraphedStep(layer, cache)

        def graphed_steps():
            for _ in range(128):
                step(xt)

        ms_graph = max_over_ranks(time_events(graphed_steps, 3, 1, sync))
        leg["fused_reduce"] = {"step_us_eager": ms_fused * 1e3 / 128, "step_us_cuda_graph": ms_graph * 1e3 / 128,
                               "vs_nccl_rel_max": max_over_ranks(err)}
    return leg


if __name__ == "__main__":
    main()
