"""MoE-layer throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--config c2] [--tokens T] [--experts E] [--path auto] [--eager] [--no-prefill]

One step = one pass of the MoE block over one batch of synthetic tokens.  Prints
ONE JSON line (rank 0).

Headline (`value`): the Qwen3.5-MoE-shaped decode step (c2: 64 tokens, hidden 2048,
256 experts, top-8, intermediate 512, shared expert, affine 4-bit g64, seed 0); at
N > 1 every rank brings 64 tokens (weak scaling) and the experts are split over the
ranks (all-gather + reduce-scatter schedule).

  value     tokens/s with the tokens already resident in HBM (CUDA events around
            the K timed steps, max over ranks)
  e2e       tokens/s with pinned host activations in and a pinned host result out,
            copies inside the timed region
  roofline  the first expert product (gate/up + SwiGLU), the kernel that moves the
            most bytes: algorithmic bytes per launch / its average duration from
            CUDA events recorded around it on its stream
  parity    the timed configuration's output against the CPU checker (N = 1) or
            against the single-GPU block on the same tokens (N > 1)
  prefill   the same layer on the prefill workload (c3: 8192 tokens, seed 1).
            N = 1: one GPU, tensor-bound roofline of the tcgen05 gate/up kernel.
            N > 1: the 8192 tokens sharded evenly, E/N experts per rank, dispatch and
            combine as NCCL all-to-all; ms/step of the slowest rank, bytes exchanged
            per rank and the share of the step spent in the two exchanges
  cpu_baseline  the CPU restatement of the reference's algorithm timed on this host's
            cores on a bounded sample, before CUDA is initialised (rank 0, N = 1)

--impl reference times that CPU restatement alone, with every host thread, the same
K and W, and the same global token count (the reference's own MLX backend cannot be
built here: MLX is not in its tree).  --tokens/--experts/--path/--eager select a
reduced case and plain launches for profiler captures.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "moe_layer_tokens_per_sec"
UNIT = "tokens/s"
# DRAM read + write of one launch of the decode gate/up kernel per expert it touches, from the ncu capture of a
# 97-expert case (113.9 MB read + 4.2 MB written, profiles/decode_kernels_c2.md); each touched expert's bytes are
# read exactly once
DECODE_GU_TRAFFIC_PER_EXPERT = 118.1e6 / 97


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2")
    ap.add_argument("--tokens", type=int, default=0, help="override the configuration's token count")
    ap.add_argument("--experts", type=int, default=0, help="keep only this many experts")
    ap.add_argument("--path", default="auto", help="expert-kernel path (auto, decode, prefill, generic)")
    ap.add_argument("--eager", action="store_true", help="plain launches instead of a CUDA-graph replay")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill block")
    ap.add_argument("--prefill-steps", type=int, default=0, help="timed steps of the prefill block (default: min(steps, 50))")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def config_from(args, name=None):
    from ironmlx_b200.workloads import CONFIGS
    cfg = CONFIGS[name or args.config]
    if name is None:
        if args.experts:
            cfg = cfg.with_(num_experts=args.experts)
        if args.tokens:
            cfg = cfg.with_(tokens=args.tokens)
    return cfg


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the
    timed region runs (read-only queries)."""

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = get(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def peaks():
    """(HBM GB/s, dense bf16 TFLOP/s burst, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def workload_desc(cfg, extra=None):
    d = {"workload": f"{cfg.name}: {cfg.tokens} tokens, hidden {cfg.hidden}, {cfg.num_experts} experts top-{cfg.top_k}, "
                     f"intermediate {cfg.intermediate}, shared {cfg.shared_intermediate}, "
                     f"{cfg.mode} {cfg.bits}-bit g{cfg.group_size}, seed {cfg.seed}",
         "l2": "inputs larger than L2: the packed weights streamed every step (453 MB at 256 experts) exceed the 126 MB L2; no flush"}
    if extra:
        d.update(extra)
    return d


# ── the CPU restatement of the reference's algorithm (checker, baseline, reference arm) ──────────────────
def set_host_threads():
    """Every host core for the C/OpenMP restatement, whatever the launcher exported (torch.distributed.run
    sets OMP_NUM_THREADS=1): must run before the library is loaded."""
    n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(n)
    os.environ.pop("OMP_THREAD_LIMIT", None)
    return n


def host_case(cfg, blocks=1):
    """Checker-side parameters and activations of a configuration (numpy generation and quantization);
    `blocks` batches of cfg.tokens tokens (one per rank of the repo arm)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from util import make_params
    from ironmlx_b200.workloads import Workload
    x, p = make_params(cfg)
    if blocks > 1:
        wl = Workload(cfg)
        x = np.concatenate([wl.activations(block=b) for b in range(blocks)], 0)
    return x, p


def cpu_sample(cfg, x, p, seconds):
    """Times the restatement on as many whole steps of the workload as fit the budget (at least two, the first
    untimed); returns (baseline dict, output of the last step)."""
    from oracle import cref
    run, _ = cref.prepare(x, p)
    out = run()                                      # untimed first pass (page-in)
    t0 = time.perf_counter()
    steps = 0
    while True:
        out = run()
        steps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or steps >= 200:
            break
    return ({"value": x.shape[0] * steps / dt, "unit": UNIT, "cores": cref.threads(), "kind": "port",
             "sample": f"{steps} full step(s) of {cfg.name} in {dt:.1f} s with the C/OpenMP restatement "
                       f"(per-expert loop, dequantize + fp32 dot products), before CUDA is initialised"},
            {k: v.copy() for k, v in out.items()})


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's algorithm on all of this host's cores, rank 0
    only, same K and W as the repo arm, same global token count.  The reference's own MLX backend cannot be
    built: MLX/mlx-c are not in its tree and there is no Rust toolchain."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    set_host_threads()
    from oracle import cref
    cfg = config_from(args)
    world = max(1, args.gpus)
    x, p = host_case(cfg, blocks=world)              # untimed
    run, _ = cref.prepare(x, p)
    # a step is the whole batch unless K + W full steps would run for more than a few minutes; then every step is
    # a bounded sample of the batch's tokens
    t0 = time.perf_counter()
    run()
    t_full = time.perf_counter() - t0
    budget = 150.0
    n_tok = x.shape[0]
    total = (args.steps + args.warmup) * t_full
    sample = n_tok if total <= budget else max(1, int(n_tok * budget / total))
    if sample < n_tok:
        run, _ = cref.prepare(x[:sample], p)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t0
    val = sample * args.steps / dt
    what = (f"{args.steps} full step(s) of {n_tok} tokens" if sample == n_tok else
            f"{args.steps} step(s) on the first {sample} of {n_tok} tokens (bounded sample)")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_desc(cfg, {"parallelism": f"ep{world}" if world > 1 else "single",
                                      "launch": "the step's kernels replayed as one CUDA graph"}),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cref.threads(), "kind": "port",
                         "sample": what + f" of {cfg.name} with the C/OpenMP restatement"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's MLX backend is not buildable here (MLX absent from its tree, no Rust toolchain); "
                "this is the C/OpenMP restatement of its algorithm (oracle/moe_ref.c)",
    }
    print(json.dumps(line))


# ── GPU side ─────────────────────────────────────────────────────────────────────────────────────────────
def timed_steps(step, steps, warmup, barrier, dev, world, sampler_index):
    """W untimed + K timed calls of `step` between barriers; CUDA events; max over ranks -> (ms/step, clocks)."""
    import torch
    import torch.distributed as dist
    for _ in range(max(warmup, 3)):
        step()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(sampler_index) as clocks:
        barrier()
        start.record()
        for _ in range(steps):
            step()
        end.record()
        barrier()
    t = torch.tensor([start.elapsed_time(end) / steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), clocks.summary()


def wall_steps(step, steps, barrier, dev, world):
    """Host-clock time per call of a `step` that synchronises itself (end-to-end numbers), max over ranks."""
    import torch
    import torch.distributed as dist
    for _ in range(3):
        step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    t = torch.tensor([(time.perf_counter() - t0) / steps * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def rel_l2(a, b):
    import numpy as np
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def single_gpu(args, dev, barrier):
    import numpy as np
    import torch
    from ironmlx_b200 import synthetic, _lib
    from ironmlx_b200.workloads import Workload, algorithmic_bytes_decode, algorithmic_flops

    cfg = config_from(args)
    hbm_peak, tf_peak, which = peaks()
    lib = _lib.lib()

    def measure(cfg, steps, path):
        """Device-resident and end-to-end timing of one configuration on this GPU, stage times, launches."""
        moe = synthetic.build_moe(cfg, dev, path=path)
        x = torch.from_numpy(Workload(cfg).activations()).to(dev).to(torch.bfloat16)
        torch.cuda.synchronize()
        out = {}
        if args.eager:
            y_box = [None]

            def step():
                y_box[0] = moe.forward_with_stream(x)
            c0 = lib.imx_launch_count()
            step()
            out["launches_per_step"] = int(lib.imx_launch_count() - c0)
            get_y = lambda: y_box[0]
        else:
            c0 = lib.imx_launch_count()
            captured = moe.capture(x)                # the step's kernels as one CUDA graph on static buffers
            out["launches_per_step"] = int(lib.imx_launch_count() - c0) // 3     # two warm-up passes + the capture
            step = lambda: captured()
            get_y = lambda: captured.y
        ms, clocks = timed_steps(step, steps, args.warmup, barrier, dev, 1, dev.index or 0)
        out.update(ms=ms, clocks=clocks)
        # end to end: pinned host activations in, pinned host result out, copies inside the timed region
        xh = x.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        if args.eager:
            e2e_step = lambda: moe.forward_host(xh, yh)
        else:
            e2e_step = moe.capture(x, xh, yh).run_host      # copy in, block, copy out as one graph; sync per step
        out["e2e_ms"] = wall_steps(e2e_step, max(10, steps // 10), barrier, dev, 1)
        stage = np.zeros(5)
        reps = 30
        for _ in range(reps):
            # the device is kept busy for ~0.1 ms while the call's launches and event records queue up behind it,
            # so that the events bracket what the kernels take on the device, not the host's launch pace
            # (the timed step is a graph replay: its kernels never wait for the host either)
            try:
                torch.cuda._sleep(200000)
            except Exception:
                pass
            _, st = moe.forward_timed(x)
            stage += np.array(st)
        out["stage"] = stage / reps
        y, tr = moe.forward_with_stream(x, trace=True)
        torch.cuda.synchronize()
        moe.check_status()                            # a bounded wait that ran out would leave its mark here
        out.update(y=y.float().cpu().numpy(), counts=tr["counts"].cpu().numpy(), step_y=get_y().float().cpu().numpy())
        return out

    m = measure(cfg, args.steps, args.path)
    stage = m["stage"]
    stage_ms = {"router": float(stage[0]), "sort": float(stage[1]), "gate_up": float(stage[2]),
                "down": float(stage[3]), "combine": float(stage[4])}
    io_bytes = cfg.tokens * cfg.hidden * 2
    line = {
        "metric": METRIC, "value": cfg.tokens / (m["ms"] * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": m["ms"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": workload_desc(cfg, {"parallelism": "single",
                                      "launch": "plain launches" if args.eager else "the step's kernels replayed as one CUDA graph"}),
        "e2e": {"value": cfg.tokens / (m["e2e_ms"] * 1e-3), "unit": UNIT, "h2d_bytes_per_step": io_bytes,
                "d2h_bytes_per_step": io_bytes, "ms_per_step": m["e2e_ms"]},
        "clocks": m["clocks"],
        "gpu_launches": m["launches_per_step"] * args.steps,
        "gpu_launches_note": f"{m['launches_per_step']} kernels of this library per step, counted by the library "
                             "(imx_launch_count) while the step was recorded",
    }
    touched = int((m["counts"] > 0).sum())
    per_w = {"affine": cfg.bits / 8 + 4 / cfg.group_size, "mxfp8": 1 + 1 / 32, "nvfp4": 0.5 + 1 / 16}[cfg.mode]
    prefill_like = cfg.tokens * cfg.top_k >= 32 * cfg.num_experts
    if not prefill_like:
        gu_bytes = (touched * 2 * cfg.intermediate + 2 * cfg.shared_intermediate) * cfg.hidden * per_w
        achieved = gu_bytes / (stage[2] * 1e-3) / 1e9
        total_bytes = algorithmic_bytes_decode(cfg, touched)
        tmap = cfg.mode == "affine" and cfg.bits == 4 and cfg.group_size == 64
        line["roofline"] = {
            "bound": "hbm", "kernel": "decode_first_kernel (gate/up + SwiGLU)" if tmap else "decode kernel, first product",
            "achieved": achieved, "peak": hbm_peak, "peak_source": f"of {which}", "unit": "GB/s", "frac": achieved / hbm_peak,
            "traffic": DECODE_GU_TRAFFIC_PER_EXPERT * (touched + 1) if tmap and cfg.name == "c2" else None,
            "traffic_note": "dram read + write per touched expert from the ncu capture of a 97-expert case "
                            "(profiles/decode_kernels_c2.md), times the experts this launch touches: each expert's "
                            "bytes are read once, so traffic grows in proportion",
            "algorithmic_bytes_per_launch": gu_bytes, "launch_ms": float(stage[2]), "stage_ms": stage_ms,
            "launch_ms_note": "mean of 30 plain launches, CUDA events on the launching stream, launches queued ahead of the device",
            "layer": {"algorithmic_bytes": total_bytes, "touched_experts": touched,
                      "achieved_gbs": total_bytes / (m["ms"] * 1e-3) / 1e9,
                      "frac": total_bytes / (m["ms"] * 1e-3) / 1e9 / hbm_peak},
        }
    else:
        line["roofline"] = tensor_roofline(cfg, stage, stage_ms, m["ms"], tf_peak, which)
    line["_y"] = m["step_y"]
    line["_cfg"] = cfg

    if not args.no_prefill and not prefill_like and args.config == "c2" and not (args.tokens or args.experts):
        torch.cuda.empty_cache()
        pcfg = config_from(args, "c3")
        psteps = args.prefill_steps or min(args.steps, 50)
        pm = measure(pcfg, psteps, "auto")
        pst = pm["stage"]
        pstage_ms = {"router": float(pst[0]), "sort": float(pst[1]), "gate_up": float(pst[2]),
                     "down": float(pst[3]), "combine": float(pst[4])}
        pio = pcfg.tokens * pcfg.hidden * 2
        line["prefill"] = {
            "config": workload_desc(pcfg, {"parallelism": "single"}), "steps": psteps,
            "ms_per_step": pm["ms"], "value": pcfg.tokens / (pm["ms"] * 1e-3), "unit": UNIT,
            "e2e": {"value": pcfg.tokens / (pm["e2e_ms"] * 1e-3), "unit": UNIT, "h2d_bytes_per_step": pio,
                    "d2h_bytes_per_step": pio, "ms_per_step": pm["e2e_ms"]},
            "roofline": tensor_roofline(pcfg, pst, pstage_ms, pm["ms"], tf_peak, which),
            "clocks": pm["clocks"], "gpu_launches": pm["launches_per_step"] * psteps,
        }
    return line


def tensor_roofline(cfg, stage, stage_ms, ms, tf_peak, which):
    from ironmlx_b200.workloads import algorithmic_flops
    gu_flops = 4 * cfg.tokens * cfg.hidden * (cfg.top_k * cfg.intermediate + cfg.shared_intermediate)
    achieved = gu_flops / (stage[2] * 1e-3) / 1e12
    total_flops = algorithmic_flops(cfg)
    return {
        "bound": "tensor", "kernel": "prefill_tc_kernel<SwiGLU> (gate/up + SwiGLU, tcgen05, A operand in tensor memory)",
        "achieved": achieved, "peak": tf_peak, "peak_source": f"of {which} (bf16 burst)", "unit": "TFLOP/s",
        "frac": achieved / tf_peak, "traffic": None, "algorithmic_flops_per_launch": gu_flops,
        "launch_ms": float(stage[2]), "stage_ms": stage_ms,
        "launch_ms_note": "mean of 30 plain launches, CUDA events on the launching stream, launches queued ahead of the device; "
                          "the stage includes the slot-order gather that precedes the first product",
        "layer": {"algorithmic_flops": total_flops, "achieved_tflops": total_flops / (ms * 1e-3) / 1e12,
                  "frac": total_flops / (ms * 1e-3) / 1e12 / tf_peak},
    }


def multi_gpu(args, dev, rank, world, barrier):
    """N > 1: the experts split over the ranks (C-ABI expert-parallel layer, NCCL)."""
    import numpy as np
    import torch
    from ironmlx_b200 import _lib, ep, synthetic
    from ironmlx_b200.workloads import Workload

    cfg = config_from(args)
    lib = _lib.lib()
    _, tf_peak, which = peaks()

    def note(msg):                                   # progress on stderr: a collective that never returns shows where
        if rank == 0:
            print(f"[bench] {msg}", file=sys.stderr, flush=True)

    def build(cfg, comm_of=None):
        return ep.ExpertParallel(ep.build_local(cfg, dev, rank, world), cfg.num_experts, cfg.top_k, cfg.norm_topk_prob,
                                 cfg.hidden, cfg.intermediate, cfg.shared_intermediate, comm_of=comm_of)

    # ---- headline: decode step, cfg.tokens tokens per rank, gathered schedule replayed as one CUDA graph ----
    moe = build(cfg)
    note("context and communicator up")
    x = torch.from_numpy(Workload(cfg).activations(block=rank)).to(dev).to(torch.bfloat16)
    xd, y = x.clone(), torch.empty_like(x)
    for _ in range(3):
        moe.forward(xd, "gathered", y)
    torch.cuda.synchronize()
    graph = None
    launches = None
    if not args.eager:
        try:
            g = torch.cuda.CUDAGraph()
            c0 = lib.imx_launch_count()
            with torch.cuda.graph(g):
                moe.forward(xd, "gathered", y)
            launches = int(lib.imx_launch_count() - c0)
            graph = g
        except Exception as e:                       # capture not possible on this stack: plain launches
            graph = None
            torch.cuda.synchronize()
    if launches is None:
        c0 = lib.imx_launch_count()
        moe.forward(xd, "gathered", y)
        launches = int(lib.imx_launch_count() - c0)
    step = (lambda: graph.replay()) if graph is not None else (lambda: moe.forward(xd, "gathered", y))
    note(f"decode step recorded ({'graph' if graph is not None else 'plain launches'}, {launches} kernels)")
    ms, clocks = timed_steps(step, args.steps, args.warmup, barrier, dev, world, dev.index or 0)
    xh, yh = x.cpu().pin_memory(), torch.empty_like(x).cpu().pin_memory()

    def e2e_step():
        xd.copy_(xh, non_blocking=True)
        step()
        yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    note(f"decode step timed: {ms:.4f} ms")
    e2e_ms = wall_steps(e2e_step, max(10, args.steps // 10), barrier, dev, world)
    torch.cuda.synchronize()
    moe.check_status()
    note("end-to-end timed")
    y_timed = y.clone()
    info = {"schedule": int(moe.info.schedule), "bytes_sent": int(moe.info.bytes_sent)}

    # ---- parity of what was timed: rank 0 against the single-GPU block on its own tokens (untimed) ----
    parity = None
    y_a2a, tr_a2a = None, None
    a2a_ok = True
    try:
        y_a2a, tr_a2a = moe.forward(xd, "a2a", trace=True)   # the other schedule on the same tokens
        torch.cuda.synchronize()
    except _lib.IronMLXError:
        a2a_ok = False
    if rank == 0:
        full = synthetic.build_moe(cfg, dev)
        y1, tr1 = full.forward_with_stream(x, trace=True)
        torch.cuda.synchronize()
        parity = {"rel_l2_vs_single_gpu": rel_l2(y_timed.float().cpu().numpy(), y1.float().cpu().numpy()),
                  "schedule": "gathered"}
        if a2a_ok:
            parity["perm_bit_exact"] = bool(torch.equal(tr_a2a["perm"], tr1["perm"]) and
                                            torch.equal(tr_a2a["topk_idx"], tr1["topk_idx"]))
            parity["all_to_all_rel_l2_vs_single_gpu"] = rel_l2(y_a2a.float().cpu().numpy(), y1.float().cpu().numpy())
        del full
    # (the context and its communicator stay alive to the end: NCCL can block in its destructor while a captured
    # graph still holds its collectives; the prefill block below borrows the same communicator)
    first = moe
    first.w = None                                   # this block's weights are no longer needed
    torch.cuda.empty_cache()

    tokens_per_step = cfg.tokens * world
    io_bytes = cfg.tokens * cfg.hidden * 2
    line = {
        "metric": METRIC, "value": tokens_per_step / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": workload_desc(cfg, {"parallelism": f"ep{world}",
                                      "launch": "the step's kernels replayed as one CUDA graph" if graph is not None else "plain launches"}),
        "e2e": {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": io_bytes,
                "d2h_bytes_per_step": io_bytes, "ms_per_step": e2e_ms},
        "clocks": clocks,
        "gpu_launches": launches * args.steps,
        "gpu_launches_note": f"{launches} kernels of this library per step and rank (imx_launch_count), plus NCCL's two collectives",
        "parity": parity,
        "ep": {"experts_per_rank": cfg.num_experts // world, "tokens_per_rank": cfg.tokens,
               "schedule": "gathered: NCCL all-gather of the tokens + reduce-scatter of fp32 partial rows, issued by the library",
               "bytes_per_rank_per_step": info["bytes_sent"], "cuda_graph": graph is not None},
    }

    # ---- prefill block: c3's 8192 tokens sharded evenly; both schedules are timed, the faster one is the block's value ----
    if not args.no_prefill and args.config == "c2" and not (args.tokens or args.experts):
        pcfg = config_from(args, "c3")
        n_loc = pcfg.tokens // world
        note("parity of the decode step checked; prefill block")
        pmoe = build(pcfg, comm_of=first)
        px = torch.from_numpy(Workload(pcfg).activations()[rank * n_loc:(rank + 1) * n_loc]).to(dev).to(torch.bfloat16)
        py = torch.empty_like(px)
        psteps = args.prefill_steps or min(args.steps, 50)
        pms, pclocks = timed_steps(lambda: pmoe.forward(px, "a2a", py), psteps, args.warmup, barrier, dev, world, dev.index or 0)
        note(f"prefill step timed (all-to-all): {pms:.4f} ms")
        pyg = torch.empty_like(px)
        gms, gclocks = timed_steps(lambda: pmoe.forward(px, "gathered", pyg), psteps, args.warmup, barrier, dev, world, dev.index or 0)
        note(f"prefill step timed (gathered): {gms:.4f} ms")
        gathered_bytes = int(pmoe.info.bytes_sent)
        phases = np.zeros(5)
        reps = 10
        for _ in range(reps):
            pmoe.forward(px, "a2a", py, timed=True)
            phases += np.array(list(pmoe.info.phase_ms))
        phases /= reps
        torch.cuda.synchronize()
        pmoe.check_status()
        t = torch.tensor(list(phases) + [float(pmoe.info.bytes_sent), float(pmoe.info.rows_received)], device=dev, dtype=torch.float64)
        import torch.distributed as dist
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ph = tmax[:5].tolist()
        # parity: rank 0's rows against the single-GPU block on the same tokens
        pparity = None
        if rank == 0:
            full = synthetic.build_moe(pcfg, dev)
            y1 = full.forward_with_stream(px)
            torch.cuda.synchronize()
            pparity = {"rel_l2_vs_single_gpu": rel_l2(py.float().cpu().numpy(), y1.float().cpu().numpy()),
                       "bit_identical": bool(torch.equal(py, y1)),
                       "gathered_rel_l2_vs_single_gpu": rel_l2(pyg.float().cpu().numpy(), y1.float().cpu().numpy())}
            if pparity["gathered_rel_l2_vs_single_gpu"] > 5e-4 or pparity["rel_l2_vs_single_gpu"] > 5e-4:
                raise SystemExit(f"bench: the expert-parallel prefill step differs from one GPU: {pparity}")
            del full
        from ironmlx_b200.workloads import algorithmic_flops
        flops = algorithmic_flops(pcfg)
        best_ms, best = (gms, "gathered") if gms < pms else (pms, "all_to_all")
        line["prefill"] = {
            "config": workload_desc(pcfg, {"parallelism": f"ep{world}: {n_loc} tokens and {pcfg.num_experts // world} experts per rank"}),
            "steps": psteps, "ms_per_step": best_ms, "value": pcfg.tokens / (best_ms * 1e-3), "unit": UNIT, "scaling": "strong",
            "schedule": best,
            "schedules": {
                "all_to_all": {
                    "ms_per_step": pms,
                    "phase_ms_slowest_rank": {"route_sort_pack": ph[0], "dispatch": ph[1], "experts": ph[2], "return": ph[3], "combine": ph[4]},
                    "exchange_share_of_step": (ph[1] + ph[3]) / max(sum(ph), 1e-9),
                    "bytes_exchanged_per_rank_per_step": int(tmax[5].item()), "rows_on_busiest_rank": int(tmax[6].item()),
                    "exchange": "NCCL grouped ncclSend/ncclRecv of fp16 rows each way + an all-gather of the [E] counts (one host "
                                "synchronisation); bit-identical to one GPU"},
                "gathered": {
                    "ms_per_step": gms, "bytes_exchanged_per_rank_per_step": gathered_bytes,
                    "exchange": "NCCL all-gather of the bf16 tokens, every rank routes all of them and runs its own experts on the "
                                "tensor-core kernels, reduce-scatter of fp32 partial rows; no host synchronisation"}},
            "achieved_tflops": flops / (best_ms * 1e-3) / 1e12, "frac_of_n_gpu_peak": flops / (best_ms * 1e-3) / 1e12 / (tf_peak * world),
            "peak_source": f"of {which} (bf16 burst, x{world})", "clocks": gclocks if best == "gathered" else pclocks, "parity": pparity,
        }
    return line


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    # the CPU baseline first: nothing of CUDA, NVML or the sampler thread is alive yet
    baseline, checker_y = None, None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        set_host_threads()
        cfg = config_from(args)
        xh, ph = host_case(cfg)
        baseline, out = cpu_sample(cfg, xh, ph, args.cpu_seconds)
        checker_y = out["y"]

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # A collective that never returns (a rank that died, a fabric problem) must not hold the ranks for ever:
        # after ten minutes the process says where it was and leaves.
        import threading

        def give_up():
            print(f"[bench] rank {rank}: no result after 600 s, leaving", file=sys.stderr, flush=True)
            os._exit(4)

        watchdog = threading.Timer(600.0, give_up)
        watchdog.daemon = True
        watchdog.start()
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    line = single_gpu(args, dev, barrier) if world == 1 else multi_gpu(args, dev, rank, world, barrier)
    y_step = line.pop("_y", None)
    line.pop("_cfg", None)
    if baseline is not None:
        line["cpu_baseline"] = baseline
        # the timed step's own output against the checker (same seeded inputs, same packed weights)
        err = rel_l2(y_step, checker_y)
        line["parity"] = {"rel_l2_vs_checker": err, "tolerance": 2e-3, "ok": bool(err <= 2e-3)}
        if err > 2e-3:
            print(json.dumps(line), flush=True)
            raise SystemExit(f"bench: the timed step's output is {err:.3e} from the checker (tolerance 2e-3)")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicators down: destroying NCCL while captured CUDA graphs
        # that contain its collectives are still alive can block.  Every rank is past its last
        # collective here (barrier), nothing is in flight (synchronize).
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
