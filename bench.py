"""MoE-layer throughput benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2]

One step = one pass of the MoE block over one batch of synthetic tokens.
At N=1 the workload is the Qwen3.5-MoE-shaped decode step (64 tokens, hidden
2048, 256 experts, top-8, intermediate 512, shared expert, affine 4-bit g64,
seed 0).  Prints ONE JSON line (rank 0).

  value     tokens/s with the tokens already resident in HBM (CUDA events
            around the K timed steps, max over ranks)
  e2e       tokens/s through the host-buffer entry point: pinned host
            activations in, pinned host result out, copies inside the timed
            region
  roofline  the first expert product (gate/up + SwiGLU), the kernel that moves
            the most bytes: algorithmic bytes per launch / its average
            duration from CUDA events recorded around it on its stream
  cpu_baseline  the CPU restatement of the reference's algorithm timed on this
            host's cores on a bounded sample (rank 0, N=1 only)

--impl reference times that CPU restatement alone (the reference's own MLX
backend cannot be built here: MLX is not in its tree).
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


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2")
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


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
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload_desc(cfg, extra=None):
    d = {"workload": f"{cfg.name}: {cfg.tokens} tokens, hidden {cfg.hidden}, {cfg.num_experts} experts top-{cfg.top_k}, "
                     f"intermediate {cfg.intermediate}, shared {cfg.shared_intermediate}, "
                     f"{cfg.mode} {cfg.bits}-bit g{cfg.group_size}, seed {cfg.seed}",
         "l2": "inputs larger than L2: the packed weights streamed every step (453 MB at 256 experts) exceed the 126 MB L2; no flush"}
    if extra:
        d.update(extra)
    return d


# ── CPU baseline: the checker's restatement of the reference algorithm ───────
def cpu_baseline(cfg, moe_host_params, x, seconds):
    """Times the C/OpenMP restatement of the reference's algorithm
    (oracle/moe_ref.c) on this host's cores on a bounded sample: as many whole
    steps of the same workload as fit the budget (at least two, first untimed)."""
    from oracle import cref
    run, _ = cref.prepare(x, moe_host_params)
    run()                                            # untimed first pass (page-in)
    t0 = time.perf_counter()
    steps = 0
    while True:
        run()
        steps += 1
        dt = time.perf_counter() - t0
        if dt >= seconds or steps >= 200:
            break
    return {"value": cfg.tokens * steps / dt, "unit": UNIT, "cores": cref.threads(), "kind": "port",
            "sample": f"{steps} full step(s) of {cfg.name} in {dt:.1f} s with the C/OpenMP restatement "
                      f"(per-expert loop, dequantize + fp32 dot products), same packed weights as the GPU"}


def host_params_from_device(moe, cfg):
    """Checker-side parameters holding the very bytes the GPU uses."""
    import numpy as np
    from oracle import formats as F
    from oracle import moe as O

    def q(ql):
        w = ql.weight.cpu().numpy().view(np.uint32)
        if ql.mode == "affine":
            s = ql.scales.view(__import__("torch").int16).cpu().numpy().view(F.bf16)
            b = ql.biases.view(__import__("torch").int16).cpu().numpy().view(F.bf16)
        else:
            s, b = ql.scales.cpu().numpy(), None
        return O.QLinear(w, s, b, ql.group_size, ql.bits, ql.mode, ql.global_scale)

    import torch
    p = O.MoEParams(router_w=moe.gate.weight.float().cpu().numpy().astype(F.bf16),
                    gate_up=q(moe._fused.gate_up), down=q(moe._fused.down),
                    num_experts_per_tok=cfg.top_k, norm_topk_prob=cfg.norm_topk_prob)
    if moe.shared_expert is not None:
        p.shared_gate_proj = q(moe.shared_expert.gate_proj)
        p.shared_up_proj = q(moe.shared_expert.up_proj)
        p.shared_down_proj = q(moe.shared_expert.down_proj)
        p.shared_expert_gate_w = moe.shared_expert_gate.weight.float().cpu().numpy().astype(F.bf16)
    if moe.router_logit_bias is not None:
        p.router_logit_bias = moe.router_logit_bias.cpu().numpy()
    return p


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's algorithm on this
    host's cores (rank 0 only).  The reference's own MLX backend cannot be built:
    MLX/mlx-c are not in its tree and there is no Rust toolchain."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from ironmlx_b200.workloads import CONFIGS
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from util import make_params
    from oracle import cref
    cfg = CONFIGS[args.config]
    x, p = make_params(cfg)                          # numpy generation + quantization, untimed
    run, _ = cref.prepare(x, p)
    warm = max(1, min(args.warmup, 2))
    for _ in range(warm):
        run()
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = time.perf_counter() - t0
    val = cfg.tokens * steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_desc(cfg),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cref.threads(), "kind": "port",
                         "sample": f"{steps} full step(s) of {cfg.name} with the C/OpenMP restatement"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's MLX backend is not buildable here (MLX absent from its tree, no Rust toolchain); "
                "this is the C/OpenMP restatement of its algorithm (oracle/moe_ref.c)",
    }
    print(json.dumps(line))


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import numpy as np
    import torch
    import torch.distributed as dist

    from ironmlx_b200 import synthetic
    from ironmlx_b200.workloads import CONFIGS, Workload, algorithmic_bytes_decode

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = CONFIGS[args.config]
    wl = Workload(cfg)

    if world > 1:
        from ironmlx_b200 import ep
        runner = ep.build_bench_runner(cfg, dev, rank, world)
    else:
        moe = synthetic.build_moe(cfg, dev)
        x = torch.from_numpy(wl.activations()).to(dev).to(torch.bfloat16)
        runner = None
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput ----
    if runner is None:
        captured = moe.capture(x)                # the step's kernels as one CUDA graph on static buffers
        step = lambda: captured()
    else:
        step = runner.step
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            step()
        end.record()
        barrier()
    ms = start.elapsed_time(end) / args.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    tokens_per_step = cfg.tokens * world
    value = tokens_per_step / (ms * 1e-3)

    # ---- end to end through the host-buffer entry point ----
    if runner is None:
        xh = x.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()
        captured_host = moe.capture(x, xh, yh)   # copy in, block, copy out as one graph; sync per step
        e2e_step = captured_host.run_host
    else:
        e2e_step = runner.step_host
    for _ in range(3):
        e2e_step()
    barrier()
    e2e_steps = max(10, args.steps // 10)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    t = torch.tensor([e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    io_bytes = cfg.tokens * cfg.hidden * 2

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 operands, f32 accumulate", "data": "synthetic",
        "config": workload_desc(cfg, {"parallelism": f"ep{world}" if world > 1 else "single",
                                      "launch": "the step's kernels replayed as one CUDA graph"}),
        "e2e": {"value": tokens_per_step / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": io_bytes,
                "d2h_bytes_per_step": io_bytes, "ms_per_step": e2e_ms},
        "clocks": clocks.summary(),
    }

    if runner is None:
        # ---- roofline of the dominant kernel, timed live with CUDA events ----
        stage = np.zeros(5)
        reps = 50
        for _ in range(reps):
            _, st = moe.forward_timed(x)
            stage += np.array(st)
        stage /= reps
        _, tr = moe.forward_with_stream(x, trace=True)
        touched = int((tr["counts"] > 0).sum().item())
        per_w = cfg.bits / 8 + 4 / cfg.group_size if cfg.mode == "affine" else (1 + 1 / 32 if cfg.mode == "mxfp8" else 0.5 + 1 / 16)
        gu_bytes = (touched * 2 * cfg.intermediate + 2 * cfg.shared_intermediate) * cfg.hidden * per_w
        peak, which = peaks()
        stage_ms = {"router": float(stage[0]), "sort": float(stage[1]), "gate_up": float(stage[2]),
                    "down": float(stage[3]), "combine": float(stage[4])}
        prefill = cfg.tokens * cfg.top_k >= 32 * cfg.num_experts and cfg.mode == "affine" and cfg.bits == 4
        if not prefill:
            achieved = gu_bytes / (stage[2] * 1e-3) / 1e9
            total_bytes = algorithmic_bytes_decode(cfg, touched)
            line["roofline"] = {
                "bound": "hbm", "kernel": "decode_tmap_kernel<true> (gate/up + SwiGLU)", "achieved": achieved,
                "peak": peak, "peak_source": f"of {which}", "unit": "GB/s", "frac": achieved / peak,
                "traffic": 265.1e6 if cfg.name == "c2" else None,
                "traffic_note": "dram read+write per launch from the ncu capture of a 97-expert case, scaled by touched experts "
                                "(profiles/decode_tmap_kernel_c2.md): the algorithmic bytes plus the SwiGLU rows written",
                "algorithmic_bytes_per_launch": gu_bytes, "launch_ms": float(stage[2]), "stage_ms": stage_ms,
                "layer": {"algorithmic_bytes": total_bytes, "touched_experts": touched,
                          "achieved_gbs": total_bytes / (ms * 1e-3) / 1e9, "frac": total_bytes / (ms * 1e-3) / 1e9 / peak},
            }
        else:
            # tensor-core bound: dense-equivalent flops of the first expert product / its duration
            tf_peak = 1590.0
            pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
            if os.path.exists(pk):
                tf_peak = float(json.load(open(pk))["bf16_tflops"])
            from ironmlx_b200.workloads import algorithmic_flops
            gu_flops = 4 * cfg.tokens * cfg.hidden * (cfg.top_k * cfg.intermediate + cfg.shared_intermediate)
            achieved = gu_flops / (stage[2] * 1e-3) / 1e12
            total_flops = algorithmic_flops(cfg)
            line["roofline"] = {
                "bound": "tensor", "kernel": "prefill_umma_kernel<true> (gate/up + SwiGLU, tcgen05)", "achieved": achieved,
                "peak": tf_peak, "peak_source": f"of {which} (bf16 burst)", "unit": "TFLOP/s", "frac": achieved / tf_peak,
                "traffic": None, "algorithmic_flops_per_launch": gu_flops, "launch_ms": float(stage[2]),
                "stage_ms": stage_ms,
                "layer": {"algorithmic_flops": total_flops, "achieved_tflops": total_flops / (ms * 1e-3) / 1e12,
                          "frac": total_flops / (ms * 1e-3) / 1e12 / tf_peak},
            }
        line["gpu_launches"] = (8 if prefill else 6) * args.steps      # decode: router x2, sort, 2 products, combine
        if rank == 0 and not args.no_cpu_baseline:
            p = host_params_from_device(moe, cfg)
            xs = wl.activations()
            line["cpu_baseline"] = cpu_baseline(cfg, p, xs, args.cpu_seconds)
    else:
        line["gpu_launches"] = runner.launches_per_step * args.steps
        line.update(runner.extra())
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing the communicator down: destroying NCCL while captured CUDA graphs
        # that contain its collectives are still alive can block.  Every rank is past its last
        # collective here (barrier), nothing is in flight (synchronize).
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
