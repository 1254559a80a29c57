"""Benchmark of the neural-net forward pass: NN evals/s for b18c384nbt, fp16, batch 256, 19x19.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One process per GPU (under torchrun for N > 1); every rank owns a full weight replica and evaluates its own
batch of 256 positions per step (replicas only: nothing is exchanged between GPUs).  A step is one forward
pass over one batch.  Rank 0 prints one JSON line.

  value     evals/s with the inputs resident in device memory, timed on the device (CUDA events on the
            library's stream, max over ranks), each step preceded by an L2 flush
  e2e       evals/s through kb_forward_host (the call NeuralNet::getOutput makes): page-locked host buffers in,
            host buffers out, host<->device copies inside the timed region
  roofline  the dominant kernel (3x3 convolution 192->192 on tcgen05): algorithmic FLOPs per launch over its mean
            launch time measured with CUDA events around every launch of a second pass over the same K steps
  sustained back-to-back steps for at least 3 s with their own clock samples (a short run prints a higher figure than a
            settled one: the 1000 W power cap takes a second to pull the SM clock down)
  cpu_baseline  the CPU oracle (port of the reference's Eigen backend) on a bounded sample, rank 0 only: all cores
            on batches of 8, and the reference's own CPU operating point (batches of 2, one single-threaded worker per
            core: cpp/program/setup.cpp:279-287, 330-339)

--through-katago (secondary figure, (N = --gpus) GPUs in ONE process): runs the reference program's own `benchmark`
subcommand linked with this backend (oracle/_ref/katago_b200: search threads -> NNEvaluator queue -> getOutput) with
--server-threads-per-gpu server threads per GPU, cudaDeviceToUseThread<i> = i mod N, on a random-weight b18c384nbt model
file, and prints its nnEvals/s.  --c-abi-threads T (also in-process) runs T host threads per GPU, each with its own
handle, calling kb_forward_host in a loop: the same multi-GPU process model without NNEvaluator's queue.

--impl reference times that CPU port alone (the reference's own CPU backend needs Eigen3, which is not
installed on this image), on the same config and metric.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

BATCH = 256
FLOPS_PER_EVAL = 18.87e9  # direct-convolution FLOPs of b18c384nbt on the 19x19 grid
METRIC = "NN evals/sec, b18c384nbt fp16 batch 256 19x19"
WORKLOAD = "b18c384nbt nested-bottleneck net (18 blocks, 384/192 channels, Mish), fp16 storage fp32 accumulate, 19x19, batch 256 per GPU"

# The headline workload is "b18" (the configuration the metric is quoted on).  The others are the remaining
# configurations of the parity suite, selectable for measurement only; the default line never changes.
WORKLOADS = {
    "b18": dict(builder="make_b18c384nbt", precision="fp16", batch=256, sizes=None, metric=METRIC, text=WORKLOAD,
                dominant="conv3x3 192->192"),
    "b28": dict(builder="make_b28c512nbt", precision="bf16", batch=512, sizes=None,
                metric="NN evals/sec, b28c512nbt bf16 batch 512 19x19",
                text="b28c512nbt nested-bottleneck net (28 blocks, 512/256 channels, Mish), bf16 storage fp32 accumulate, 19x19, batch 512 per GPU",
                dominant="conv3x3 256->256"),
    "transformer": dict(builder="make_transformer", precision="fp16", batch=128, sizes=None,
                        metric="NN evals/sec, transformer trunk 12x(6x64, SwiGLU 1024) fp16 batch 128 19x19",
                        text="3x3 stem to d=384, 12 pre-norm layers (6 heads x 64, learnable RoPE, SwiGLU 1024), fp16, 19x19, batch 128 per GPU",
                        dominant="attention"),
    "transformer_relbias": dict(builder="make_transformer_relbias", precision="fp16", batch=128, sizes=None,
                                metric="NN evals/sec, transformer trunk 12x(6x64, relative-position bias, SwiGLU 1024) fp16 batch 128 19x19",
                                text="3x3 stem to d=384, 12 pre-norm layers (6 heads x 64, learned per-head 19x19 relative-position bias, SwiGLU 1024), fp16, 19x19, batch 128 per GPU",
                                dominant="attention"),
    "mixed": dict(builder="make_b18c384nbt", precision="fp16", batch=128, sizes=[9, 13, 19, 19],
                  metric="NN evals/sec, b18c384nbt fp16 mixed 9/13/19 boards padded to 19x19, batch 128 per GPU",
                  text="b18c384nbt, fp16, boards 9x9/13x13/19x19 in ratio 1:1:2 zero-padded to 19x19 with the on-board mask, batch 128 per GPU (1024 over 8)",
                  dominant="conv3x3 192->192"),
}


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops_sustained"]), burst=float(p["bf16_tflops"]), hbm=float(p["hbm_gbs"]), src="measured")
    except Exception:
        return dict(tflops=1400.0, burst=1590.0, hbm=6650.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        # nvidia-smi numbers GPUs without regard to CUDA_VISIBLE_DEVICES: address the device by its UUID
        self.gpu, self.lines, self.proc = str(gpu_index), [], None
        try:
            import torch
            self.gpu = "GPU-" + str(torch.cuda.get_device_properties(gpu_index).uuid)
        except Exception:
            pass

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons), samples=len(sm))


def _dist():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    pg = None
    if world > 1:
        import torch.distributed as dist
        # control plane only (barrier, max over ranks); the data path has no collective
        dist.init_process_group(backend="gloo", init_method="env://")
        pg = dist
    return rank, world, local, pg


def _barrier_sync(pg):
    import torch
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if pg is not None:
        pg.barrier()
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def _max_over_ranks(pg, x):
    if pg is None:
        return x
    import torch
    t = torch.tensor([x], dtype=torch.float64)
    pg.all_reduce(t, op=pg.ReduceOp.MAX)
    return float(t.item())


def _use_all_host_cores():
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core this process may run
    on, so the variable is reset before the oracle's OpenMP runtime is loaded."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    os.environ["OMP_NUM_THREADS"] = str(max(1, n))


def _host_cores():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_reference_operating_point(budget_s, wl=None):
    """evals/s of the CPU port run the way the reference runs its CPU backend: batches of at most 2 positions, one
    single-threaded server thread per core (cpp/program/setup.cpp:279-287, 330-339)."""
    from concurrent.futures import ThreadPoolExecutor
    from katago_b200 import modelfile as mf
    from oracle import pyoracle as po
    wl = wl or WORKLOADS["b18"]
    om = po.OracleModel(mf.to_blob(getattr(mf, wl["builder"])()))
    cores = _host_cores()
    sp, gl = mf.random_positions(2, seed=2000)
    deadline = time.perf_counter() + budget_s

    def worker(_):
        po.set_num_threads(1)
        done = 0
        while True:
            om.forward(sp, gl)
            done += 2
            if time.perf_counter() > deadline:
                return done
    t0 = time.perf_counter()
    with ThreadPoolExecutor(cores) as ex:
        done = sum(ex.map(worker, range(cores)))
    return dict(value=done / (time.perf_counter() - t0), workers=cores, evals=done)


def cpu_oracle_rate(budget_s, positions_per_call, max_calls, wl=None):
    """evals/s of the CPU port of the reference's Eigen backend on the same net and position scheme."""
    _use_all_host_cores()
    from katago_b200 import modelfile as mf
    from oracle import pyoracle as po
    po.set_num_threads(_host_cores())  # an OpenMP runtime loaded earlier (torch under torchrun) may have fixed it at 1
    wl = wl or WORKLOADS["b18"]
    om = po.OracleModel(mf.to_blob(getattr(mf, wl["builder"])()))
    sizes = (wl["sizes"] * positions_per_call)[:positions_per_call] if wl["sizes"] else None
    sp, gl = mf.random_positions(positions_per_call, seed=2000, board_sizes=sizes)
    om.forward(sp[:1], gl[:1])  # touch the weights once
    done, t0 = 0, time.perf_counter()
    per_call = []
    while done < max_calls:
        t = time.perf_counter()
        om.forward(sp, gl)
        per_call.append(time.perf_counter() - t)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    total = time.perf_counter() - t0
    return dict(value=done * positions_per_call / total, cores=po.num_threads(), calls=done, per_call_s=per_call)


def run_reference(args, rank, world, pg):
    if rank != 0:
        return
    _use_all_host_cores()
    from oracle import pyoracle as po
    per_step = 8
    from katago_b200 import modelfile as mf
    # torchrun exports OMP_NUM_THREADS=1 and torch.distributed loads the OpenMP runtime before this point, which fixes
    # the thread count at 1 whatever the environment says later: set it through the runtime itself
    po.set_num_threads(_host_cores())
    om = po.OracleModel(mf.to_blob(mf.make_b18c384nbt()))
    sp, gl = mf.random_positions(per_step, seed=2000)
    for _ in range(max(args.warmup, 1)):
        om.forward(sp[:2], gl[:2])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        om.forward(sp, gl)
    dt = time.perf_counter() - t0
    v = args.steps * per_step / dt
    unit = "evals/s"
    sample = f"{per_step} of the 256 positions of a batch per step ({args.steps} steps), CPU port of the reference's Eigen backend (oracle/kata_oracle.cpp, OpenMP)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "note": "reference arm = CPU port on host cores; Eigen3 is not installed, so the reference's own eigenbackend.cpp cannot be compiled"},
        "cpu_baseline": {"value": v, "unit": unit, "cores": po.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def run_b200(args, rank, world, local, pg):
    import katago_b200 as kb
    from katago_b200 import capi, modelfile as mf
    ndev = kb.device_count()
    device = local % max(ndev, 1)
    os.environ.setdefault("CUDA_DEVICE_ORDER", "PCI_BUS_ID")
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.set_device(device)
    except Exception:
        pass

    wl = WORKLOADS[args.workload]
    BATCH = wl["batch"]
    precision = dict(fp16=kb.PRECISION_FP16, bf16=kb.PRECISION_BF16)[wl["precision"]]
    model = kb.Model(mf.to_blob(getattr(mf, wl["builder"])()))
    h = kb.Handle(model, BATCH, precision=precision, device=device)
    sizes = (wl["sizes"] * BATCH)[:BATCH] if wl["sizes"] else None
    sp, gl = mf.random_positions(BATCH, seed=2000 + rank, board_sizes=sizes)
    S = 19 * 19
    # page-locked staging, as the backend's InputBuffers hold it
    pin_sp = capi.PinnedArray((BATCH, 19, 19, model.in_c)); pin_sp.array[...] = sp
    pin_gl = capi.PinnedArray((BATCH, model.in_global_c)); pin_gl.array[...] = gl
    pin_sym = capi.PinnedArray((BATCH,), np.int32); pin_sym.array[...] = 0
    outs = {k: capi.PinnedArray(shape) for k, shape in dict(policy=(BATCH, S, model.policy_c), policyPass=(BATCH, model.policy_c),
                                                              value=(BATCH, model.value_c), scoreValue=(BATCH, model.score_c), ownership=(BATCH, S)).items()}
    out_arrays = {k: v.array for k, v in outs.items()}
    flush = 256 << 20

    # ---- device-resident throughput ----
    h.upload(pin_sp.array, pin_gl.array)
    sampler = ClockSampler(device)
    sampler.start()  # started before the warm-up: nvidia-smi needs ~0.1 s to deliver its first sample
    h.time_forward_steps(BATCH, max(args.warmup, 3), flush)
    _barrier_sync(pg)
    ms_each = h.time_forward_steps(BATCH, args.steps, flush)
    _barrier_sync(pg)
    ms_total = _max_over_ranks(pg, sum(ms_each))
    value = world * BATCH * args.steps / (ms_total * 1e-3)

    # ---- sustained: back-to-back steps for at least 3 s, with their own clock samples ----
    sust_steps = max(args.steps, int(3000.0 / max(ms_total / args.steps, 1e-3)) + 1)
    sust_sampler = ClockSampler(device)
    sust_sampler.start()
    _barrier_sync(pg)
    sust_ms = h.time_forward_steps(BATCH, sust_steps, flush)
    _barrier_sync(pg)
    sust_clocks = sust_sampler.stop()
    sust_total = _max_over_ranks(pg, sum(sust_ms))
    sustained = world * BATCH * sust_steps / (sust_total * 1e-3)

    # ---- end to end through the host-buffer call ----
    for _ in range(max(args.warmup, 3)):
        h.forward(pin_sp.array, pin_gl.array, pin_sym.array, out=out_arrays)
    _barrier_sync(pg)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        h.forward(pin_sp.array, pin_gl.array, pin_sym.array, out=out_arrays)
    _barrier_sync(pg)
    e2e_s = _max_over_ranks(pg, time.perf_counter() - t0)
    clocks = sampler.stop()
    e2e = world * BATCH * args.steps / e2e_s
    h2d = pin_sp.nbytes + pin_gl.nbytes + pin_sym.nbytes
    d2h = sum(v.nbytes for v in outs.values())

    # ---- per-kernel timing of the same K steps (second pass, events around every launch) ----
    h.upload(pin_sp.array, pin_gl.array)
    h.profile_enable(True); h.profile_reset()
    for _ in range(args.steps):
        h.forward_resident(BATCH)
    prof = h.profile_read()
    h.profile_enable(False)
    launches = h.launches_per_forward()
    h.close()

    if rank != 0:
        return
    peaks = _peaks()
    total_ms = sum(p["ms"] for p in prof) or 1.0
    dom = [p for p in prof if p["name"].startswith(wl["dominant"]) and "tcgen05" in p["name"] and "reg|gpool" not in p["name"]]
    dom_ms = sum(p["ms"] for p in dom); dom_launches = sum(p["launches"] for p in dom); dom_flops = sum(p["flops"] for p in dom)
    achieved = (dom_flops / (dom_ms * 1e-3) / 1e12) if dom_ms > 0 else 0.0
    traffic = None
    if args.workload == "b18":
        try:
            with open(os.path.join(ROOT, "profiles", "conv3x3_192_b18_n256_traffic.json")) as f:
                per = json.load(f)["dram_bytes_per_launch"]
            # DRAM bytes per launch of the dominant class (ncu, small case of the same shapes and batch), averaged over its launches
            num = sum(per[k] * p["launches"] for p in dom for k in per if p["name"].endswith(k))
            traffic = num / dom_launches if dom_launches and num > 0 else None
        except Exception:
            pass
    all_conv_flops = sum(p["flops"] for p in prof)
    flops_per_eval = FLOPS_PER_EVAL if args.workload == "b18" else all_conv_flops / (args.steps * BATCH)
    # the CPU baseline is taken at N=1 only (at N>1 the other ranks' processes share the host cores)
    cpu = cpu_oracle_rate(budget_s=12.0, positions_per_call=8, max_calls=8, wl=wl) if world == 1 else None
    cpu_op = cpu_reference_operating_point(budget_s=8.0, wl=wl) if world == 1 else None
    # The timed region of the default run is a fraction of a second, which the power cap has not settled yet: the
    # burst figure of the measured cuBLAS peak is its denominator; a timed region of a second or more takes the
    # sustained one.  Both ratios are printed.
    timed_s = ms_total * 1e-3
    peak_used = peaks["burst"] if timed_s < 1.0 else peaks["tflops"]
    peak_name = "bf16_tflops (burst: timed region %.2f s)" % timed_s if timed_s < 1.0 else "bf16_tflops_sustained (timed region %.1f s)" % timed_s
    line = {
        "metric": wl["metric"], "value": value, "unit": "evals/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_total / args.steps, "p50_batch_latency_ms": statistics.median(ms_each), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": {"fp16": "f16", "bf16": "bf16"}[wl["precision"]], "data": "synthetic",
        "config": {"workload": wl["text"], "batch_per_gpu": BATCH, "parallelism": f"replicas x{world}, no collective",
                   "l2": "256 MiB memset between timed steps (L2 flush); per-step activations (~0.4 GB) also exceed the 126 MB L2",
                   "weights": "random init N(0,1/fan_in), BN scale U(0.5,1.5) bias N(0,0.1), seed 1001", "positions": "seeded synthetic, empty/black/white 0.6/0.2/0.2"},
        "clocks": clocks,
        "sustained": {"value": sustained, "unit": "evals/s", "steps": sust_steps, "seconds": sust_total * 1e-3,
                      "ms_per_step": sust_total / sust_steps, "clocks": sust_clocks},
        "e2e": {"value": e2e, "unit": "evals/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s / args.steps * 1e3},
        "gpu_launches": launches * args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak_used, "unit": "TFLOP/s", "frac": achieved / peak_used,
                     "frac_of_sustained_peak": achieved / peaks["tflops"], "frac_of_burst_peak": achieved / peaks["burst"],
                     "traffic": traffic, "kernel": ("convChainKernel<half>: runs of 3-4 consecutive 3x3 192->192 convolutions per launch" if args.workload in ("b18", "mixed") else wl["dominant"] + " (tcgen05)"), "launches": dom_launches,
                     "avg_launch_ms": dom_ms / dom_launches if dom_launches else None, "share_of_step": dom_ms / total_ms,
                     "peak_source": f"MEASURED_PEAKS.json {peak_name} ({peaks['src']}); burst {peaks['burst']}, sustained {peaks['tflops']}",
                     "whole_step_tflops": all_conv_flops / (total_ms * 1e-3) / 1e12,
                     "whole_step_frac_of_peak": flops_per_eval * value / world / 1e12 / peak_used,
                     "sustained_step_frac_of_sustained_peak": flops_per_eval * sustained / world / 1e12 / peaks["tflops"]},
        "cpu_baseline": None if cpu is None else {
            "value": cpu["value"], "unit": "evals/s", "cores": cpu["cores"], "kind": "port",
            "sample": f"{cpu['calls']} calls of 8 positions of the same net and position scheme (oracle/kata_oracle.cpp, OpenMP, fp32)",
            "reference_operating_point": {"value": cpu_op["value"], "unit": "evals/s", "workers": cpu_op["workers"], "batch": 2,
                                          "sample": f"{cpu_op['evals']} evaluations in batches of 2 by {cpu_op['workers']} single-threaded workers, as the reference configures its CPU backend"}},
        "kernels": [{"name": p["name"], "launches": p["launches"], "ms": round(p["ms"], 4), "share": round(p["ms"] / total_ms, 4)}
                    for p in sorted(prof, key=lambda p: -p["ms"])[:8] if p["launches"]],
        # bandwidth-bound classes: algorithmic bytes (each tensor read or written once) over the measured time, against
        # the measured copy bandwidth
        "hbm_kernels": [{"name": p["name"], "launches": p["launches"], "gb_per_s": round(p["bytes"] / (p["ms"] * 1e-3) / 1e9, 1),
                         "frac_of_copy_peak": round(p["bytes"] / (p["ms"] * 1e-3) / 1e9 / peaks["hbm"], 3), "us_per_launch": round(p["ms"] / p["launches"] * 1e3, 2)}
                        for p in sorted(prof, key=lambda p: -p["ms"]) if p["launches"] and p["ms"] > 0 and p["bytes"] > 0 and "conv" not in p["name"] and "attention" not in p["name"]],
    }
    print(json.dumps(line), flush=True)


KATAGO_CFG = """logFile = /dev/null
logToStderr = false
logAllGTPCommunication = false
logSearchInfo = false
rules = tromp-taylor
numSearchThreads = 256
nnMaxBatchSize = 256
nnCacheSizePowerOfTwo = 20
nnMutexPoolSizePowerOfTwo = 14
numNNServerThreadsPerModel = {server_threads}
cudaUseFP16 = true
maxVisits = {visits}
"""


def run_through_katago(args):
    """The reference's `benchmark` subcommand on this backend, N GPUs in one process (setup.cpp:183-220 device map)."""
    import re
    import tempfile
    from katago_b200 import modelfile as mf
    binary = os.path.join(ROOT, "oracle", "_ref", "katago_b200")
    if not os.path.exists(binary):
        print(json.dumps({"impl": "b200-through-katago", "unavailable": "oracle/_ref/katago_b200 is not built (make -C oracle ref_b200 needs the reference sources)"}))
        return
    G, per = max(1, args.gpus), max(1, args.server_threads_per_gpu)
    with tempfile.TemporaryDirectory() as d:
        model = os.path.join(d, "b18c384nbt-random.bin.gz")
        cfg = os.path.join(d, "benchmark.cfg")
        mf.save_model_file(mf.make_b18c384nbt(), model)
        text = KATAGO_CFG.format(visits=args.visits, server_threads=G * per)
        for i in range(G * per):
            text += f"cudaDeviceToUseThread{i} = {i % G}\n"
        with open(cfg, "w") as f:
            f.write(text)
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = os.path.join(ROOT, "katago_b200") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
        env["KATAB200_TIMING"] = "1"  # the backend prints, per server thread, where getOutput's wall time went
        cmd = [binary, "benchmark", "-model", model, "-config", cfg, "-v", str(args.visits), "-t", args.search_threads, "-n", str(args.positions)]
        t0 = time.perf_counter()
        r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=1800)
        wall = time.perf_counter() - t0
    text = (r.stdout + r.stderr).replace("\r", "\n")
    rows = []
    for line in text.splitlines():
        m = re.search(r"numSearchThreads\s*=\s*(\d+):.*?nnEvals/s\s*=\s*([0-9.]+)", line)
        if m:
            rows.append({"search_threads": int(m.group(1)), "nn_evals_per_s": float(m.group(2)), "line": line.strip()[:200]})
    best = max((x["nn_evals_per_s"] for x in rows), default=None)
    # host profile of the server threads: seconds spent staging rows, inside kb_forward_host, unpacking, and waiting for
    # the NNEvaluator queue to hand over the next batch (summed over the threads)
    prof = {"server_threads": 0, "calls": 0, "rows": 0, "staging_s": 0.0, "kb_forward_host_s": 0.0, "unpacking_s": 0.0, "waiting_s": 0.0}
    for m in re.finditer(r"B200 backend timing: .*?: (\d+) getOutput calls, (\d+) rows .*?staging rows ([0-9.]+) s, kb_forward_host ([0-9.]+) s, "
                         r"unpacking ([0-9.]+) s, waiting for the next batch ([0-9.]+) s", text):
        prof["server_threads"] += 1
        prof["calls"] += int(m.group(1)); prof["rows"] += int(m.group(2))
        prof["staging_s"] += float(m.group(3)); prof["kb_forward_host_s"] += float(m.group(4))
        prof["unpacking_s"] += float(m.group(5)); prof["waiting_s"] += float(m.group(6))
    busy = prof["staging_s"] + prof["kb_forward_host_s"] + prof["unpacking_s"]
    prof["busy_fraction"] = busy / (busy + prof["waiting_s"]) if busy + prof["waiting_s"] > 0 else None
    prof["host_cores"] = _host_cores()
    print(json.dumps({"impl": "b200-through-katago", "host_profile": prof, "metric": "nnEvals/s of the reference's benchmark subcommand on this backend", "value": best,
                      "unit": "evals/s", "n_gpus": G, "server_threads_per_gpu": per, "visits": args.visits, "rows": rows, "rc": r.returncode,
                      "wall_s": wall, "tail": None if rows else text[-1500:]}), flush=True)


def run_c_abi_threads(args):
    """N GPUs in one process without NNEvaluator: T host threads per GPU, one handle each (as createComputeHandle is called
    once per server thread), each calling kb_forward_host on its own page-locked buffers in a loop for a fixed time."""
    import katago_b200 as kb
    from katago_b200 import capi, modelfile as mf
    G, T = max(1, args.gpus), max(1, args.c_abi_threads)
    wl = WORKLOADS["b18"]
    batch = wl["batch"]
    blob = mf.to_blob(mf.make_b18c384nbt())
    S = 19 * 19
    seconds = 4.0
    counts = [0] * (G * T)
    handles = []
    ready = threading.Barrier(G * T + 1)

    def worker(i):
        dev = i % G
        model = kb.Model(blob)
        h = kb.Handle(model, batch, precision=kb.PRECISION_FP16, device=dev)
        sp, gl = mf.random_positions(batch, seed=2000 + i)
        pin_sp = capi.PinnedArray((batch, 19, 19, model.in_c)); pin_sp.array[...] = sp
        pin_gl = capi.PinnedArray((batch, model.in_global_c)); pin_gl.array[...] = gl
        pin_sym = capi.PinnedArray((batch,), np.int32); pin_sym.array[...] = 0
        outs = {k: capi.PinnedArray(shape) for k, shape in dict(policy=(batch, S, model.policy_c), policyPass=(batch, model.policy_c), value=(batch, model.value_c),
                                                                  scoreValue=(batch, model.score_c), ownership=(batch, S)).items()}
        arrays = {k: v.array for k, v in outs.items()}
        for _ in range(3):
            h.forward(pin_sp.array, pin_gl.array, pin_sym.array, out=arrays)
        handles.append((h, pin_sp, pin_gl, pin_sym, outs))
        ready.wait()
        ready.wait()
        end = time.perf_counter() + seconds
        while time.perf_counter() < end:
            h.forward(pin_sp.array, pin_gl.array, pin_sym.array, out=arrays)
            counts[i] += 1
    threads = [threading.Thread(target=worker, args=(i,)) for i in range(G * T)]
    for t in threads:
        t.start()
    ready.wait()
    t0 = time.perf_counter()
    ready.wait()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    value = sum(counts) * batch / wall
    print(json.dumps({"impl": "b200-c-abi-threads", "metric": METRIC + ", kb_forward_host from host threads of one process", "value": value, "unit": "evals/s",
                      "n_gpus": G, "threads_per_gpu": T, "seconds": wall, "batches_per_thread": counts}), flush=True)
    for h, *_ in handles:
        h.close()


def run_forward_only(args):
    """Two forward passes of a workload at reduced depth, nothing timed: the small case that profiler captures run on
    (same kernels and shapes as the full net, a fraction of its launches and memory)."""
    import katago_b200 as kb
    from katago_b200 import modelfile as mf
    wl = WORKLOADS[args.workload]
    kwargs = {"layers": args.blocks} if "transformer" in args.workload else {"num_blocks": args.blocks}
    model = kb.Model(mf.to_blob(getattr(mf, wl["builder"])(**kwargs)))
    batch = wl["batch"]
    h = kb.Handle(model, batch, precision=dict(fp16=kb.PRECISION_FP16, bf16=kb.PRECISION_BF16)[wl["precision"]], device=0)
    sizes = (wl["sizes"] * batch)[:batch] if wl["sizes"] else None
    sp, gl = mf.random_positions(batch, seed=2000, board_sizes=sizes)
    h.upload(sp, gl)
    for _ in range(2):
        h.forward_resident(batch)
    h.download(batch)
    print(json.dumps({"forward_only": args.workload, "blocks": args.blocks, "batch": batch, "launches_per_forward": h.launches_per_forward()}))
    h.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="b18", choices=sorted(WORKLOADS), help="b18 is the headline configuration; the others are for measurement of the remaining configurations")
    ap.add_argument("--through-katago", action="store_true", help="run the reference's benchmark subcommand on this backend, --gpus GPUs in one process")
    ap.add_argument("--server-threads-per-gpu", type=int, default=2)
    ap.add_argument("--visits", type=int, default=30000)
    ap.add_argument("--search-threads", default="512,1024")
    ap.add_argument("--positions", type=int, default=4)
    ap.add_argument("--c-abi-threads", type=int, default=0, help="T > 0: T host threads per GPU in one process, each calling kb_forward_host in a loop")
    ap.add_argument("--forward-only", action="store_true", help="two untimed forward passes of --workload at --blocks blocks (for profiler captures)")
    ap.add_argument("--blocks", type=int, default=6)
    args = ap.parse_args()
    if args.forward_only:
        return run_forward_only(args)
    if args.through_katago:
        return run_through_katago(args)
    if args.c_abi_threads > 0:
        return run_c_abi_threads(args)
    rank, world, local, pg = _dist()
    if args.impl == "reference":
        run_reference(args, rank, world, pg)
    else:
        run_b200(args, rank, world, local, pg)
    if pg is not None:
        pg.barrier()
        pg.destroy_process_group()


if __name__ == "__main__":
    main()
