#!/usr/bin/env python
"""Benchmark of the quantized decode matvec path (BASELINE.json configs[1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("ffn_decode_q4k_q6k"): the FFN-shaped decode matvecs at batch 1 over
LAYERS distinct sets of weights (so the working set is far larger than L2):
    x(4096) f32 -> Q8_1 -> gate  Q4_K 4096->14336
                        -> up    Q4_K 4096->14336
    h(14336) f32 -> Q8_1 -> down Q4_K 14336->4096
                         -> down Q6_K 14336->4096
One pass = all LAYERS sets: 2*LAYERS activation-quantize launches and ONE job-list launch
(launch_qmatvec_batch) that walks the 4*LAYERS projections with persistent CTAs, captured as
one CUDA graph.  One step = PASSES graph replays (so that the timed region is long enough to
be insensitive to scheduler noise).  value = packed weight bytes streamed per second, whole job.
With N > 1 every rank owns the same amount of work (weak scaling): the FFN is N times wider,
gate/up are split by output rows, down by input columns, and the N partial down outputs of a
pass are summed across the ranks.

Further sections of the JSON line: the same shapes as single launches and at the decode batch
sizes, the Q8_0 matvec of configs[0], the Q4_K prefill GEMM of configs[2], decode tok/s of the
two stacks of configs[3] and [4], and (N > 1) a tensor-parallel parity check of the engine.

`--impl reference` times the CPU restatement of the same path (oracle/, the only
CPU implementation there is: the upstream has none) on the host cores.

`--case ...` runs one small case and exits (for profiler captures; see profiles/):
    --case matvec:<q8_0|q4_k|q6_k>:<n>:<k>:<m>[:launches]    single-matrix launches over rotating weights
    --case jobs:<q4k|ffn>[:launches]                          one job-list launch (24 Q4_K / 32 FFN jobs)
    --case gemm:<n>:<k>:<m>[:launches]                        Q4_K x bf16 prefill GEMM
    --case decode:<8b|70b>:<batch>[:steps[:layers]]           eager decode steps of a (cut) stack
    --case prefill:<8b|70b>:<tokens>[:layers]                 a prompt through a (cut) stack at once, twice
    --case seqattn:<t>:<q heads>:<kv heads>:<head dim>[:f32]  causal attention over a sequence (k, v f16 rows of a cache,
                                                              or f32), a few launches, device-timed
    --case shard:<8b|70b>:<tp>:<batch>                        step time of a decoder with the per-rank shapes of a
                                                              tensor-parallel layout, on one GPU (no exchange)
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HID, FFN = 4096, 14336
LAYERS = 8
SEED = 0x5EED
METRIC = "ffn_decode_matvec_weight_bandwidth"
UNIT = "GB/s"
WORKLOAD = "ffn_decode_q4k_q6k"


def layer_weight_bytes():
    from nates_recipe_rs_b200._lib import BLOCK_BYTES, Q4_K, Q6_K
    q4 = HID * FFN // 256 * BLOCK_BYTES[Q4_K]
    q6 = HID * FFN // 256 * BLOCK_BYTES[Q6_K]
    return 3 * q4 + q6, q4, q6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json)"
    return 6650.0, 1590.0, "fallback (6.65 TB/s, 1.59 PFLOP/s)"


def profile_traffic(name):
    """DRAM bytes per launch of the dominant kernel, from the committed ncu summary (profiles/<name>.json)."""
    path = os.path.join(ROOT, "profiles", name)
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["dram_bytes_read"]) + float(d["dram_bytes_write"]), f"profiles/{name}"
    except (OSError, KeyError, ValueError):
        return None, "no ncu summary committed for this launch"


class ClockSampler:
    """nvidia-smi in the background during the timed region."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.path = f"/tmp/qmm_bench_clocks_{os.getpid()}.csv"
        self.proc = None
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.kill()
        self.proc.wait()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            p = [s.strip() for s in line.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
            except ValueError:
                continue
            for nm, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.path)
        busy = [s for s in sm if s > 0.5 * max(mx or [1])] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def note(msg):
    """Progress line on stderr (QMM_BENCH_VERBOSE=1): where a multi-rank run is, should it stall."""
    if os.environ.get("QMM_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


# ------------------------------------------------------------------------- CPU arm
def cpu_time_sample(budget_s=12.0):
    """Times the oracle on one layer set (gate, up, down Q4_K, down Q6_K; activation
    quantization included) repeatedly for about budget_s seconds, on every host core."""
    import oracle
    oracle.set_num_threads(os.cpu_count() or 1)  # a launcher may have exported OMP_NUM_THREADS=1
    total, q4, q6 = layer_weight_bytes()
    gate = oracle.quantize(oracle.Q4_K, oracle.fill_normal(FFN * HID, SEED, 0.02).reshape(FFN, HID))
    down4 = oracle.quantize(oracle.Q4_K, oracle.fill_normal(FFN * HID, SEED + 2, 0.02).reshape(HID, FFN))
    down6 = oracle.quantize(oracle.Q6_K, oracle.fill_normal(FFN * HID, SEED + 3, 0.02).reshape(HID, FFN))
    x = oracle.fill_normal(HID, SEED + 10, 1.0)
    h = oracle.fill_normal(FFN, SEED + 11, 1.0)

    def one():
        xq = oracle.quantize(oracle.Q8_1, x)
        oracle.matvec(oracle.Q4_K, gate, xq, HID)
        oracle.matvec(oracle.Q4_K, gate, xq, HID)   # "up" has the same shape; the sample reuses the bytes
        hq = oracle.quantize(oracle.Q8_1, h)
        oracle.matvec(oracle.Q4_K, down4, hq, FFN)
        oracle.matvec(oracle.Q6_K, down6, hq, FFN)

    one()
    reps, t0 = 0, time.perf_counter()
    while True:
        one()
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 5000:
            break
    return {"value": total * reps / dt / 1e9, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{reps} passes over one layer set (gate, up, down Q4_K, down Q6_K = {total} B) in {dt:.1f} s, "
                      f"OpenMP over output rows"}, dt / reps


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    total, _, _ = layer_weight_bytes()
    per_step = []
    base = None
    for i in range(args.warmup + args.steps):
        base, t_layer = cpu_time_sample(budget_s=2.0)
        if i >= args.warmup:
            per_step.append(t_layer)
    t = statistics.mean(per_step)
    value = total / t / 1e9
    base["value"] = value
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 dot / f32 accumulate", "data": "synthetic (seeded closed-form normal, quantized on the host)",
        "config": {"workload": WORKLOAD, "hidden": HID, "ffn": FFN, "batch": 1,
                   "note": "CPU restatement of the path (oracle/): the upstream has no implementation of these block "
                           "formats; each step is a ~2 s sample of one layer set on all host cores"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------- GPU arm
class Timer:
    """CUDA-event timing of graph replays on one stream."""

    def __init__(self, torch, stream):
        self.torch, self.stream = torch, stream

    def graph(self, body):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            body()
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream):
                body()
        return g

    def us(self, body, reps=10, warm=3):
        """Mean microseconds of one replay of `body` captured as a graph."""
        torch = self.torch
        g = self.graph(body)
        with torch.cuda.stream(self.stream):
            for _ in range(warm):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(reps):
                g.replay()
            e1.record(self.stream)
            self.stream.synchronize()
        del g
        return e0.elapsed_time(e1) * 1e3 / reps


def gen_weights(torch, ops, dev, rows, cols, seed, qtype):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return ops.gpu_quantize_weights(qtype, torch.randn(rows, cols, device=dev, generator=g) * 0.02)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nates_recipe_rs_b200 import quant_ops as ops
    from nates_recipe_rs_b200._lib import Q4_K, Q6_K, Q8_0, Q8_1, lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib()
    total_layer, q4_bytes, q6_bytes = layer_weight_bytes()
    hbm_peak, tensor_peak, peak_src = measured_peaks()
    passes = max(1, args.passes)

    # ---- tensor-parallel parity first: a run that computes the wrong thing is not timed
    tp_par = None
    if world > 1:
        from nates_recipe_rs_b200.tp_parity import tp_parity
        note("tensor-parallel parity")
        checks = []
        for wide in (False, True):
            try:
                checks.append(tp_parity(wide=wide))
            except ValueError as e:   # the check model does not divide by this world size
                checks.append({"n": world, "wide": wide, "skipped": str(e), "ok": True})
        tp_par = {"n": world, "max_logit_diff": max(c.get("max_logit_diff", 0.0) for c in checks),
                  "tokens_agree": all(c.get("tokens_agree", True) for c in checks), "ok": all(c["ok"] for c in checks),
                  "checks": checks}
        if not tp_par["ok"]:
            if rank == 0:
                print(json.dumps({"metric": METRIC, "error": "tensor-parallel parity failed", "tp_parity": tp_par}), flush=True)
            dist.barrier()
            os._exit(3)

    # ---- synthetic model: LAYERS sets of FFN weights, generated and quantized on the device
    layers = []
    for li in range(LAYERS):
        s = SEED + 100 * li + 7919 * rank
        layers.append({"gate": gen_weights(torch, ops, dev, FFN, HID, s, Q4_K), "up": gen_weights(torch, ops, dev, FFN, HID, s + 1, Q4_K),
                       "down4": gen_weights(torch, ops, dev, HID, FFN, s + 2, Q4_K),
                       "down6": gen_weights(torch, ops, dev, HID, FFN, s + 3, Q6_K)})
    g = torch.Generator(device=dev)
    g.manual_seed(SEED + 5)
    x = torch.randn(1, HID, device=dev, generator=g)
    h = torch.randn(1, FFN, device=dev, generator=g)
    xq = [torch.empty(ops.row_bytes(Q8_1, HID), dtype=torch.uint8, device=dev) for _ in range(LAYERS)]
    hq = [torch.empty(ops.row_bytes(Q8_1, FFN), dtype=torch.uint8, device=dev) for _ in range(LAYERS)]
    y_gate = torch.empty(LAYERS, FFN, device=dev)
    y_up = torch.empty(LAYERS, FFN, device=dev)
    y_down = torch.empty(LAYERS, 2, HID, device=dev)   # [layer][Q4_K, Q6_K]: the partial sums of this rank when N > 1

    ffn_jobs = ops.MatvecJobs()    # the pass; N > 1: the down projections are summed over the ranks inside the launch
    nccl_jobs = ops.MatvecJobs()   # N > 1, second number: the same pass with the sum done by one NCCL allreduce
    q4_jobs = ops.MatvecJobs()
    for li, lw in enumerate(layers):
        for jobs in (ffn_jobs, nccl_jobs, q4_jobs):
            summed = world > 1 and jobs is ffn_jobs
            jobs.add(Q4_K, lw["gate"], xq[li], y_gate[li], FFN, HID)
            jobs.add(Q4_K, lw["up"], xq[li], y_up[li], FFN, HID)
            jobs.add(Q4_K, lw["down4"], hq[li], y_down[li, 0], HID, FFN, tp_sum=summed)
        ffn_jobs.add(Q6_K, lw["down6"], hq[li], y_down[li, 1], HID, FFN, tp_sum=world > 1)
        nccl_jobs.add(Q6_K, lw["down6"], hq[li], y_down[li, 1], HID, FFN)
    comm = ops.TpComm(2 * LAYERS * HID) if world > 1 else None
    launches_per_pass = 2 * LAYERS + (2 if world > 1 else 1)

    def quantize_all():
        for li in range(LAYERS):
            ops.gpu_quantize_q8_1_into(x, xq[li], 1, HID)
            ops.gpu_quantize_q8_1_into(h, hq[li], 1, FFN)

    def pass_body():
        quantize_all()
        if world > 1:   # partial down outputs pushed into every rank's exchange area by the matvec kernel, then summed
            ops.gpu_qmatvec_batch_tp_into(comm, ffn_jobs, 1)
        else:
            ops.gpu_qmatvec_batch_into(ffn_jobs, 1)

    def nccl_pass_body():
        quantize_all()
        ops.gpu_qmatvec_batch_into(nccl_jobs, 1)
        dist.all_reduce(y_down)   # the 2*LAYERS partial down outputs of the pass in one allreduce

    stream = torch.cuda.Stream(device=dev)
    timer = Timer(torch, stream)
    note("model built; capturing the pass graph")
    use_graph = True
    try:
        graph = timer.graph(pass_body)
    except Exception as e:  # NCCL capture refused: fall back to eager launches of the same kernels
        use_graph = False
        graph = None
        if rank == 0:
            print(f"# graph capture unavailable ({type(e).__name__}); timing eager launches", file=sys.stderr)

    def run_pass():
        if use_graph:
            graph.replay()
        else:
            pass_body()

    def run_step():
        for _ in range(passes):
            run_pass()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    note(f"graph={use_graph}; warm-up")
    with torch.cuda.stream(stream):
        sampler = ClockSampler(local) if rank == 0 else None  # spans warm-up, the timed steps and the legs below
        for _ in range(max(args.warmup, 3)):
            run_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            run_step()
        e1.record(stream)
        barrier()
        elapsed_ms = e0.elapsed_time(e1)
        # keep the same load running for ~1 s more so the clock sampler (20 ms period, slow to start) sees it
        t_soak = time.perf_counter()
        while time.perf_counter() - t_soak < 1.0:
            run_step()
            stream.synchronize()

        # ---- dominant kernel alone: one job-list launch over the 3*LAYERS Q4_K projections of the pass
        note("timed steps done; Q4_K job list alone")
        q4_list_us = timer.us(lambda: ops.gpu_qmatvec_batch_into(q4_jobs, 1), reps=max(args.steps, 20))
        ffn_list_us = timer.us(lambda: ops.gpu_qmatvec_batch_into(nccl_jobs, 1), reps=max(args.steps, 20))
        nccl_pass_us = None
        if world > 1:
            # check the fused sum against NCCL on the same partial outputs, then time the NCCL form of the pass
            pass_body()
            fused = y_down.clone()
            nccl_pass_body()
            stream.synchronize()
            sum_diff = float((fused - y_down).abs().max() / y_down.abs().max())
            try:
                barrier()
                nccl_pass_us = timer.us(nccl_pass_body, reps=50)
            except Exception:
                nccl_pass_us = None

        # ---- end to end through the C ABI with host buffers: activations come from pinned host
        # memory and the projections go back to it every pass; the weights stay resident in HBM
        note("end-to-end leg")
        hx = torch.randn(1, HID).pin_memory()
        hh = torch.randn(1, FFN).pin_memory()
        hy = torch.empty(2, HID).pin_memory()

        def e2e_pass():
            x.copy_(hx, non_blocking=True)
            h.copy_(hh, non_blocking=True)
            run_pass()
            hy.copy_(y_down[LAYERS - 1], non_blocking=True)
            stream.synchronize()
        for _ in range(3):
            e2e_pass()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps * passes):
            e2e_pass()
        barrier()
        e2e_s = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None

    t = torch.tensor([elapsed_ms, e2e_s * 1e3, q4_list_us, ffn_list_us, nccl_pass_us or 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, q4_list_us, ffn_list_us, nccl_pass_us = [float(v) for v in t.tolist()]
    ops.check_launch()  # raises if any kernel abandoned a bounded wait

    pass_bytes = total_layer * LAYERS * world
    n_pass = args.steps * passes
    value = pass_bytes * n_pass / (elapsed_ms * 1e-3) / 1e9
    e2e_value = pass_bytes * n_pass / (e2e_ms * 1e-3) / 1e9
    # algorithmic bytes of the Q4_K job-list launch: packed weights + Q8_1 activations + f32 outputs of its 3*LAYERS jobs
    q4_algo = LAYERS * (3 * q4_bytes + (2 * HID + FFN) // 32 * 36 + (2 * FFN + HID) * 4)
    achieved = q4_algo / (q4_list_us * 1e-6) / 1e9
    ffn_algo = q4_algo + LAYERS * (q6_bytes + FFN // 32 * 36 + HID * 4)
    traffic, traffic_src = profile_traffic("qmatvec_jobs_q4k_ffn.json")

    note("FFN legs done")
    sections = {}
    if world == 1:
        with torch.cuda.stream(stream):
            sections["matvec_shapes"] = shapes_section(torch, ops, timer, dev, layers, hbm_peak)
            sections["q8_0_matvec"] = q8_0_section(torch, ops, timer, dev, hbm_peak)
            sections["batched_matvec"] = batched_section(torch, ops, timer, dev, layers, q4_bytes, q6_bytes)
            sections["prefill_gemm"] = gemm_section(torch, ops, timer, dev, layers, tensor_peak)
        ops.check_launch()
    decode = None if args.no_decode else run_decode(world, rank, dev, args.quick_decode)
    if rank == 0:
        cpu, _ = cpu_time_sample() if world == 1 else (None, None)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 dot (dp4a) / f32 accumulate", "data": "synthetic (seeded normal weights sigma 0.02, quantized on the device)",
            "config": {"workload": WORKLOAD, "hidden": HID, "ffn": FFN, "batch": 1, "layers_per_pass": LAYERS,
                       "passes_per_step": passes, "bytes_per_pass": pass_bytes, "ms_per_pass": elapsed_ms / n_pass,
                       "l2": "inputs larger than L2: each pass streams %d MB of distinct weights per GPU" % (pass_bytes // world // 10**6),
                       "launch": ("cuda graph replay" if use_graph else "eager") +
                                 f": per pass {2 * LAYERS} activation-quantize launches + 1 job-list launch of {4 * LAYERS} projections",
                       "parallelism": "single GPU" if world == 1 else
                                      f"tp{world}: gate/up split by rows, down by columns; the matvec kernel stores the partial down outputs "
                                      f"into every rank's exchange area (NVLink peer stores) and one small kernel per pass adds them"},
            "roofline": {"bound": "hbm", "kernel": f"qmatvec_jobs_kernel<1>: one launch = the {3 * LAYERS} Q4_K projections (gate, up, down) of a pass",
                         "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src,
                         "us_per_launch": q4_list_us, "us_per_projection": q4_list_us / (3 * LAYERS),
                         "algorithmic_bytes_per_launch": q4_algo, "traffic": traffic, "traffic_source": traffic_src,
                         "whole_pass_list": {"jobs": 4 * LAYERS, "us_per_launch": ffn_list_us, "GBps": ffn_algo / ffn_list_us / 1e3,
                                             "frac": ffn_algo / ffn_list_us / 1e3 / hbm_peak}},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (HID + FFN) * 4 * passes, "d2h_bytes_per_step": 2 * HID * 4 * passes,
                    "note": "every pass: activations from pinned host memory, the pass, the last layer's projections back to the host, "
                            "stream synchronize; weights resident in HBM"},
            "gpu_launches": launches_per_pass * n_pass,
            "clocks": clocks,
        }
        if cpu:
            out["cpu_baseline"] = cpu
        out.update(sections)
        if decode is not None:
            out["decode"] = decode
            if PREFILL:
                out["prefill"] = PREFILL
        if tp_par is not None:
            out["tp_parity"] = tp_par
            out["tp_exchange"] = {"fused_vs_nccl_max_rel_diff": sum_diff, "fused_pass_us": elapsed_ms * 1e3 / n_pass,
                                  "nccl_allreduce_pass_us": nccl_pass_us or None,
                                  "note": "the same pass with the sum of the partial down outputs done by one NCCL allreduce"}
        print(json.dumps(out), flush=True)
    if world > 1:
        # The NCCL communicator is referenced by the captured graphs: release them first, and do not let
        # a slow teardown outlive the measurement (the line above is already printed).
        import threading
        graph = None
        torch.cuda.synchronize()
        dist.barrier()
        comm.close()
        threading.Timer(20.0, lambda: os._exit(0)).start()
        dist.destroy_process_group()
        os._exit(0)


def shapes_section(torch, ops, timer, dev, layers, hbm_peak):
    """The three FFN shapes one at a time over the same rotation of weights: as single launches of the
    one-matrix kernel and as one job list of LAYERS jobs (time per projection)."""
    from nates_recipe_rs_b200._lib import Q4_K, Q6_K
    _, q4, q6 = layer_weight_bytes()
    xq = ops.gpu_quantize_q8_1(torch.randn(1, HID, device=dev))
    hq = ops.gpu_quantize_q8_1(torch.randn(1, FFN, device=dev))
    yg, yd = torch.empty(1, FFN, device=dev), torch.empty(1, HID, device=dev)
    out = []
    for label, qt, key, xin, y, n, k, nbytes in (("gate_q4_k", Q4_K, "gate", xq, yg, FFN, HID, q4), ("down_q4_k", Q4_K, "down4", hq, yd, HID, FFN, q4),
                                                  ("down_q6_k", Q6_K, "down6", hq, yd, HID, FFN, q6)):
        def single():
            for lw in layers:
                ops.gpu_qmatvec_into(qt, lw[key], xin, y, 1, n, k)
        jobs = ops.MatvecJobs()
        for lw in layers:
            jobs.add(qt, lw[key], xin, y, n, k)
        us_single = timer.us(single) / LAYERS
        us_list = timer.us(lambda: ops.gpu_qmatvec_batch_into(jobs, 1)) / LAYERS
        algo = nbytes + k // 32 * 36 + n * 4
        out.append({"shape": label, "n": n, "k": k, "algorithmic_bytes": algo,
                    "single_launch_us": us_single, "single_launch_frac": algo / us_single / 1e3 / hbm_peak,
                    "job_list_us_per_projection": us_list, "job_list_frac": algo / us_list / 1e3 / hbm_peak,
                    "note": f"job list of {LAYERS} such projections; its launch overhead is shared by only {LAYERS} jobs"})
    return out


def q8_0_section(torch, ops, timer, dev, hbm_peak):
    """BASELINE configs[0]: Q8_0 4096 x 4096 at batch 1, over 16 distinct matrices (285 MB > L2)."""
    from nates_recipe_rs_b200._lib import Q8_0
    n = k = 4096
    copies = 16
    ws = [gen_weights(torch, ops, dev, n, k, SEED + 900 + i, Q8_0) for i in range(copies)]
    xq = ops.gpu_quantize_q8_1(torch.randn(1, k, device=dev))
    y = torch.empty(copies, n, device=dev)
    nbytes = n * k // 32 * 34
    algo = nbytes + k // 32 * 36 + n * 4

    def single():
        for i, w in enumerate(ws):
            ops.gpu_qmatvec_into(Q8_0, w, xq, y[i], 1, n, k)
    jobs = ops.MatvecJobs()
    for i, w in enumerate(ws):
        jobs.add(Q8_0, w, xq, y[i], n, k)
    us_single = timer.us(single) / copies
    us_list = timer.us(lambda: ops.gpu_qmatvec_batch_into(jobs, 1)) / copies
    return {"shape": "q8_0 4096x4096 batch 1", "weight_bytes": nbytes, "algorithmic_bytes": algo, "copies": copies, "bound": "hbm", "peak": hbm_peak,
            "single_launch_us": us_single, "single_launch_GBps": algo / us_single / 1e3, "single_launch_frac": algo / us_single / 1e3 / hbm_peak,
            "job_list_us_per_projection": us_list, "job_list_GBps": algo / us_list / 1e3, "job_list_frac": algo / us_list / 1e3 / hbm_peak}


def batched_section(torch, ops, timer, dev, layers, q4_bytes, q6_bytes):
    """The three FFN shapes at the decode batch sizes of the configs: time per launch over the rotation of
    weights (1-2 rows: dp4a kernel; 3 and more: tensor-core kernel)."""
    from nates_recipe_rs_b200._lib import Q4_K, Q6_K
    out = []
    for m in (1, 8, 16, 32):
        xm = ops.gpu_quantize_q8_1(torch.randn(m, HID, device=dev))
        hm = ops.gpu_quantize_q8_1(torch.randn(m, FFN, device=dev))
        yg, yd = torch.empty(m, FFN, device=dev), torch.empty(m, HID, device=dev)
        for label, qt, key, xin, yout, n_, k_, nbytes in (("gate_q4_k", Q4_K, "gate", xm, yg, FFN, HID, q4_bytes),
                                                          ("down_q4_k", Q4_K, "down4", hm, yd, HID, FFN, q4_bytes),
                                                          ("down_q6_k", Q6_K, "down6", hm, yd, HID, FFN, q6_bytes)):
            def body():
                for lw in layers:
                    ops.gpu_qmatvec_into(qt, lw[key], xin, yout, m, n_, k_)
            us = timer.us(body) / LAYERS
            out.append({"shape": label, "rows": m, "us_per_launch": us, "weight_GBps": nbytes / us / 1e3})
    return out


def gemm_section(torch, ops, timer, dev, layers, tensor_peak):
    """BASELINE configs[2]: Q4_K dequant-GEMM, X bf16 (M, 4096), M = 512 and 2048, N = 4096 and 14336."""
    out = []
    k = HID
    for m in (512, 2048):
        xb = torch.randn(m, k, device=dev).to(torch.bfloat16)
        for n in (4096, 14336):
            y = torch.empty(m, n, device=dev, dtype=torch.bfloat16)

            def body():
                for lw in layers:   # rotating weights (the first n rows of each gate matrix)
                    ops.gpu_qgemm_q4_k_bf16_into(lw["gate"], xb, y, m, n, k)
            us = timer.us(body, reps=5) / LAYERS
            flops = 2.0 * m * n * k
            out.append({"m": m, "n": n, "k": k, "us_per_launch": us, "flops": flops, "TFLOPs": flops / us / 1e6,
                        "bound": "tensor", "peak": tensor_peak, "frac": flops / us / 1e6 / tensor_peak})
    return out


PREFILL = []   # filled by run_decode on one GPU: time to run a whole prompt through the stack


def run_decode(world, rank, dev, quick):
    """Greedy decode tok/s of the random-init 8B- and 70B-class stacks (BASELINE configs[3], [4]):
    whole steps (embedding .. argmax) captured as a CUDA graph, KV cache filled with seeded values,
    positions at the end of the context.  Tensor parallel over all ranks when world > 1."""
    import torch
    import torch.distributed as dist
    from nates_recipe_rs_b200 import decoder as dec, quant_ops as ops
    cases = [("8b", (1, 16)), ("70b", (1, 8, 32))]
    if quick:
        cases = [("8b", (1,))]
    out = []
    for name, batches in cases:
        make = dec.config_8b if name == "8b" else dec.config_70b
        cfg = make(max_batch=max(batches), tp_rank=rank, tp_size=world)
        if cfg.n_kv_heads % world != 0:
            continue
        note(f"decode {name}: building (cache for batch {max(batches)})")
        try:
            d = dec.Decoder(cfg)
        except Exception as e:  # e.g. not enough memory for the 70B stack on this GPU
            out.append({"stack": name, "batch": max(batches), "error": f"{type(e).__name__}: {e}"[:120]})
            continue
        d.fill_cache(3)
        steps_per_graph = 8
        pos0 = cfg.ctx_len - steps_per_graph - 1
        wb = d.weight_bytes * world
        for batch in batches:
            stream = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(stream):
                d.tokens.fill_(11)

                def body():
                    for i in range(steps_per_graph):
                        d.step(batch, pos0 + i)
                        d.tokens.copy_(d.next_tokens)
                note(f"decode {name} batch {batch}: eager steps")
                body()
                stream.synchronize()
                if world > 1:
                    dist.barrier()
                note("decode: capture")
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    body()
                note("decode: first replay")
                graph.replay()
                stream.synchronize()
                if world > 1:
                    dist.barrier()
                note("decode: timed replays")
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 4 if batch < 32 else 2
                e0.record(stream)
                for _ in range(reps):
                    graph.replay()
                e1.record(stream)
                stream.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) * 1e-3 / (reps * steps_per_graph)], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
            ops.check_launch()
            out.append({"stack": name, "batch": batch, "context": cfg.ctx_len, "ms_per_step": sec * 1e3, "tok_s": batch / sec,
                        "weight_GB_per_token": wb / 1e9, "weight_GBps": wb / sec / 1e9, "tp": world})
            del graph
        if world == 1:
            # the prompt path: all positions of a prompt at once (GEMM projections, sequence attention); eager launches
            for t in (512, 2048):
                if t > cfg.ctx_len:
                    continue
                note(f"prefill {name}: {t} tokens")
                prompt = torch.randint(0, cfg.vocab, (t,), dtype=torch.int32, device=dev)
                try:
                    d.prefill(prompt, 0)   # allocates the prompt path's buffers
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(2):
                        d.prefill(prompt, 0)
                    e1.record()
                    torch.cuda.synchronize()
                    ops.check_launch()
                    sec = e0.elapsed_time(e1) * 1e-3 / 2
                    PREFILL.append({"stack": name, "tokens": t, "ms": sec * 1e3, "tok_s": t / sec,
                                    "weight_flops": 2.0 * t * (d.weight_bytes / 0.62), "note": "flops ~ 2 x tokens x weights (0.62 B per weight on average)"})
                except Exception as e:
                    PREFILL.append({"stack": name, "tokens": t, "error": f"{type(e).__name__}: {e}"[:120]})
        d.close()
        del d
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------- profiler cases
def run_case(spec):
    """One small case for a profiler capture (see the module docstring); weights rotate over about 300 MB."""
    import torch
    from nates_recipe_rs_b200 import _lib, quant_ops as ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    for kv in os.environ.get("QMM_TUNE", "").split(","):   # tuning overrides, e.g. QMM_TUNE=jobs_warps=12
        if kv:
            key, val = kv.split("=")
            _lib.check(L.qmm_tune(key.encode(), int(val)), f"qmm_tune({key})")
    parts = spec.split(":")
    kind = parts[0]
    names = {"q8_0": _lib.Q8_0, "q4_k": _lib.Q4_K, "q6_k": _lib.Q6_K}
    if kind in ("matvec", "gemm"):
        if kind == "matvec":
            qt, n, k, m = names[parts[1]], int(parts[2]), int(parts[3]), int(parts[4])
            reps = int(parts[5]) if len(parts) > 5 else 4
        else:
            qt, n, k, m = _lib.Q4_K, int(parts[1]), int(parts[2]), int(parts[3])
            reps = int(parts[4]) if len(parts) > 4 else 4
        rb = ops.row_bytes(qt, k)
        ncopy = max(2, int(300e6 // (n * rb)) + 1)
        ws = [gen_weights(torch, ops, dev, n, k, i, qt) for i in range(ncopy)]
        if kind == "gemm":
            xb = torch.randn(m, k, device=dev).to(torch.bfloat16)
            y = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            torch.cuda.synchronize()
            for i in range(reps):
                ops.gpu_qgemm_q4_k_bf16_into(ws[i % ncopy], xb, y, m, n, k)
        else:
            xq = ops.gpu_quantize_q8_1(torch.randn(m, k, device=dev))
            y = torch.empty(m, n, device=dev)
            torch.cuda.synchronize()
            for i in range(reps):
                ops.gpu_qmatvec_into(qt, ws[i % ncopy], xq, y, m, n, k)
    elif kind == "jobs":
        which = parts[1] if len(parts) > 1 else "q4k"
        reps = int(parts[2]) if len(parts) > 2 else 3
        xq = ops.gpu_quantize_q8_1(torch.randn(1, HID, device=dev))
        hq = ops.gpu_quantize_q8_1(torch.randn(1, FFN, device=dev))
        yg, yd = torch.empty(2, LAYERS, FFN, device=dev), torch.empty(2, LAYERS, HID, device=dev)
        jobs = ops.MatvecJobs()
        for li in range(LAYERS):
            jobs.add(_lib.Q4_K, gen_weights(torch, ops, dev, FFN, HID, 4 * li, _lib.Q4_K), xq, yg[0, li], FFN, HID)
            jobs.add(_lib.Q4_K, gen_weights(torch, ops, dev, FFN, HID, 4 * li + 1, _lib.Q4_K), xq, yg[1, li], FFN, HID)
            jobs.add(_lib.Q4_K, gen_weights(torch, ops, dev, HID, FFN, 4 * li + 2, _lib.Q4_K), hq, yd[0, li], HID, FFN)
            if which == "ffn":
                jobs.add(_lib.Q6_K, gen_weights(torch, ops, dev, HID, FFN, 4 * li + 3, _lib.Q6_K), hq, yd[1, li], HID, FFN)
        torch.cuda.synchronize()
        for _ in range(reps):
            ops.gpu_qmatvec_batch_into(jobs, 1)
    elif kind == "decode":
        from nates_recipe_rs_b200 import decoder as dec
        name, batch = parts[1], int(parts[2])
        steps = int(parts[3]) if len(parts) > 3 else 3
        cfg = (dec.config_8b if name == "8b" else dec.config_70b)(max_batch=batch)
        if len(parts) > 4:
            cfg.n_layers = int(parts[4])
        d = dec.Decoder(cfg)
        d.fill_cache(3)
        d.tokens.fill_(11)
        pos0 = cfg.ctx_len - steps - 1
        for i in range(steps):   # eager launches, so that a launch list attributes the step to its kernels
            d.step(batch, pos0 + i)
            d.tokens.copy_(d.next_tokens)
    elif kind == "seqattn":
        t, nqh, nkv, hd = (int(v) for v in parts[1:5])
        kv_dtype = torch.float32 if len(parts) > 5 and parts[5] == "f32" else torch.float16
        q = torch.randn(t, nqh * hd, device=dev)
        k = torch.randn(t, nkv * hd, device=dev).to(kv_dtype)
        v = torch.randn(t, nkv * hd, device=dev).to(kv_dtype)
        out = torch.empty(t, nqh * hd, device=dev)
        for _ in range(2):
            ops.gpu_gqa_attn_into(q, k, v, out, t, nqh, nkv, hd, t, hd ** -0.5)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            ops.gpu_gqa_attn_into(q, k, v, out, t, nqh, nkv, hd, t, hd ** -0.5)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 3
        flops = 4.0 * hd * nqh * (t * (t + 1) / 2)
        print(json.dumps({"case": spec, "us_per_launch": us, "useful_TFLOPs": flops / us / 1e6}))
    elif kind == "prefill":
        # prefill:<8b|70b>:<tokens>[:layers]: one prompt through a (cut) stack, eager launches (for a launch list)
        from nates_recipe_rs_b200 import decoder as dec
        name, t = parts[1], int(parts[2])
        cfg = (dec.config_8b if name == "8b" else dec.config_70b)(max_batch=1)
        if len(parts) > 3:
            cfg.n_layers = int(parts[3])
        d = dec.Decoder(cfg)
        prompt = torch.randint(0, cfg.vocab, (t,), dtype=torch.int32, device=dev)
        d.prefill(prompt, 0)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        d.prefill(prompt, 0)
        e1.record()
        torch.cuda.synchronize()
        print(json.dumps({"case": spec, "layers": cfg.n_layers, "ms": e0.elapsed_time(e1)}))
    elif kind == "shard":
        # shard:<8b|70b>:<tp>:<batch>: a decoder with the per-rank shapes of a tensor-parallel layout on ONE GPU,
        # i.e. the step without any exchange (what an N-GPU step is compared with); graph replays, device-timed
        from nates_recipe_rs_b200 import decoder as dec
        name, tp, batch = parts[1], int(parts[2]), int(parts[3])
        cfg = (dec.config_8b if name == "8b" else dec.config_70b)(max_batch=batch)
        cfg.n_q_heads //= tp
        cfg.n_kv_heads = max(1, cfg.n_kv_heads // tp)
        cfg.ffn //= tp
        cfg.vocab //= tp
        d = dec.Decoder(cfg)
        d.fill_cache(3)
        steps, reps = 8, 4
        pos0 = cfg.ctx_len - steps - 1
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            d.tokens.fill_(11)

            def body():
                for i in range(steps):
                    d.step(batch, pos0 + i)
                    d.tokens.copy_(d.next_tokens)
            body()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                body()
            g.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1) / (reps * steps)
        print(json.dumps({"case": spec, "ms_per_step": ms, "us_per_layer": ms * 1e3 / cfg.n_layers, "weight_bytes": d.weight_bytes}))
    else:
        raise SystemExit(f"unknown --case {spec!r}")
    torch.cuda.synchronize()
    ops.check_launch()
    print("case done:", spec)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--passes", type=int, default=50, help="graph replays (passes over all layer sets) per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the decode tok/s section")
    ap.add_argument("--quick-decode", action="store_true", help="decode section: 8B batch 1 only")
    ap.add_argument("--case", default=None, help="run one small case for a profiler capture and exit")
    args = ap.parse_args()
    if args.case:
        run_case(args.case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
