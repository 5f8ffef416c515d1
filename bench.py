#!/usr/bin/env python
"""Benchmark of the quantized decode matvec path (BASELINE.json configs[1]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("ffn_decode_q4k_q6k"): the FFN-shaped decode matvecs at batch 1 over
LAYERS distinct sets of weights (so the working set is far larger than L2):
    x(4096) f32 -> Q8_1 -> gate  Q4_K 4096->14336
                        -> up    Q4_K 4096->14336
    h(14336) f32 -> Q8_1 -> down Q4_K 14336->4096
                         -> down Q6_K 14336->4096
One step = one pass over all LAYERS sets (LAYERS * 6 kernel launches), replayed
as one CUDA graph.  value = packed weight bytes streamed per second, whole job.
With N > 1 every rank owns the same amount of work (weak scaling): the FFN is N
times wider, gate/up are split by output rows, down by input columns, and the
N partial down outputs are summed with one NCCL allreduce per down projection.

`--impl reference` times the CPU restatement of the same path (oracle/, the only
CPU implementation there is: the upstream has none) on the host cores.
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


def layer_weight_bytes():
    from nates_recipe_rs_b200._lib import BLOCK_BYTES, Q4_K, Q6_K
    q4 = HID * FFN // 256 * BLOCK_BYTES[Q4_K]
    q6 = HID * FFN // 256 * BLOCK_BYTES[Q6_K]
    return 3 * q4 + q6, q4, q6


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


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


# ------------------------------------------------------------------------- CPU arm
def cpu_time_sample(budget_s=12.0):
    """Times the oracle on one layer set (gate, up, down Q4_K, down Q6_K; activation
    quantization included) repeatedly for about budget_s seconds."""
    import numpy as np
    import oracle
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
        "config": {"workload": "ffn_decode_q4k_q6k", "hidden": HID, "ffn": FFN, "batch": 1,
                   "note": "CPU restatement of the path (oracle/): the upstream has no implementation of these block "
                           "formats; each step is a ~2 s sample of one layer set"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch
    import torch.distributed as dist
    from nates_recipe_rs_b200 import quant_ops as ops
    from nates_recipe_rs_b200._lib import Q4_K, Q6_K, Q8_1, lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = lib()
    total_layer, q4_bytes, q6_bytes = layer_weight_bytes()

    # ---- synthetic model: LAYERS sets of FFN weights, generated and quantized on the device
    def gen(rows, cols, seed, qtype):
        g = torch.Generator(device=dev)
        g.manual_seed(seed)
        w = torch.randn(rows, cols, device=dev, generator=g) * 0.02
        return ops.gpu_quantize_weights(qtype, w)

    layers = []
    for li in range(LAYERS):
        s = SEED + 100 * li + 7919 * rank
        layers.append({"gate": gen(FFN, HID, s, Q4_K), "up": gen(FFN, HID, s + 1, Q4_K),
                       "down4": gen(HID, FFN, s + 2, Q4_K), "down6": gen(HID, FFN, s + 3, Q6_K)})
    g = torch.Generator(device=dev)
    g.manual_seed(SEED + 5)
    x = torch.randn(1, HID, device=dev, generator=g)
    h = torch.randn(1, FFN, device=dev, generator=g)
    xq = torch.empty(ops.row_bytes(Q8_1, HID), dtype=torch.uint8, device=dev)
    hq = torch.empty(ops.row_bytes(Q8_1, FFN), dtype=torch.uint8, device=dev)
    y_gate = torch.empty(1, FFN, device=dev)
    y_up = torch.empty(1, FFN, device=dev)
    y_d4 = torch.empty(1, HID, device=dev)
    y_d6 = torch.empty(1, HID, device=dev)
    launches_per_step = [0]

    def step_body(count=False):
        n = 0
        for lw in layers:
            ops.gpu_quantize_q8_1_into(x, xq, 1, HID)
            ops.gpu_qmatvec_into(Q4_K, lw["gate"], xq, y_gate, 1, FFN, HID)
            ops.gpu_qmatvec_into(Q4_K, lw["up"], xq, y_up, 1, FFN, HID)
            ops.gpu_quantize_q8_1_into(h, hq, 1, FFN)
            ops.gpu_qmatvec_into(Q4_K, lw["down4"], hq, y_d4, 1, HID, FFN)
            if world > 1:
                dist.all_reduce(y_d4)
            ops.gpu_qmatvec_into(Q6_K, lw["down6"], hq, y_d6, 1, HID, FFN)
            if world > 1:
                dist.all_reduce(y_d6)
            n += 6
        if count:
            launches_per_step[0] = n

    stream = torch.cuda.Stream(device=dev)

    def make_graph(body):
        with torch.cuda.stream(stream):
            body()
            stream.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                body()
        return gr

    note("model built; first eager step")
    step_body(count=True)
    torch.cuda.synchronize()
    note("capturing the step graph")
    use_graph = True
    try:
        graph = make_graph(step_body)
    except Exception as e:  # NCCL capture refused: fall back to eager launches of the same kernels
        use_graph = False
        graph = None
        if rank == 0:
            print(f"# graph capture unavailable ({type(e).__name__}); timing eager launches", file=sys.stderr)

    def run_step():
        if use_graph:
            graph.replay()
        else:
            step_body()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    note(f"graph={use_graph}; warm-up")
    with torch.cuda.stream(stream):
        sampler = ClockSampler(local) if rank == 0 else None  # spans warm-up, the timed steps and the two legs below
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
        # keep the same load running for ~1.5 s so the clock sampler (20 ms period, slow to start) sees it
        t_soak = time.perf_counter()
        while time.perf_counter() - t_soak < 1.5:
            for _ in range(20):
                run_step()
            stream.synchronize()
        note("timed steps done; Q4_K-only graph")

        # ---- dominant kernel alone: the Q4_K matvec launches of the same step, same rotation of weights
        def q4_body():
            for lw in layers:
                ops.gpu_qmatvec_into(Q4_K, lw["gate"], xq, y_gate, 1, FFN, HID)
                ops.gpu_qmatvec_into(Q4_K, lw["up"], xq, y_up, 1, FFN, HID)
                ops.gpu_qmatvec_into(Q4_K, lw["down4"], hq, y_d4, 1, HID, FFN)
        q4_graph = make_graph(q4_body)
        for _ in range(3):
            q4_graph.replay()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(args.steps, 10)
        k0.record(stream)
        for _ in range(reps):
            q4_graph.replay()
        k1.record(stream)
        torch.cuda.synchronize()
        q4_launch_s = k0.elapsed_time(k1) * 1e-3 / (reps * 3 * LAYERS)

        # ---- end to end through the C ABI with host buffers: activations come from pinned host
        # memory and the projections go back to it every step; the weights stay resident in HBM
        note("end-to-end leg")
        hx = torch.randn(1, HID).pin_memory()
        hh = torch.randn(1, FFN).pin_memory()
        hy = torch.empty(2, HID).pin_memory()

        def e2e_step():
            x.copy_(hx, non_blocking=True)
            h.copy_(hh, non_blocking=True)
            run_step()
            hy[0].copy_(y_d4[0], non_blocking=True)
            hy[1].copy_(y_d6[0], non_blocking=True)
            stream.synchronize()
        for _ in range(3):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        e2e_s = time.perf_counter() - t0
        clocks = sampler.stop() if sampler else None

    t = torch.tensor([elapsed_ms, e2e_s * 1e3, q4_launch_s * 1e6], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, q4_us = [float(v) for v in t.tolist()]
    check_status = ops.check_launch  # raises if any kernel abandoned a bounded wait
    check_status()

    step_bytes = total_layer * LAYERS * world
    value = step_bytes * args.steps / (elapsed_ms * 1e-3) / 1e9
    e2e_value = step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9
    peak, peak_src = measured_peak()
    # algorithmic bytes of one Q4_K launch: packed weights + Q8_1 activations + f32 outputs
    q4_algo = q4_bytes + (HID // 32 * 36 * 2 + FFN // 32 * 36) / 3 + (FFN * 4 * 2 + HID * 4) / 3
    achieved = q4_algo / (q4_us * 1e-6) / 1e9

    note("FFN legs done")
    batched = None
    if world == 1:
        # ---- the same three FFN shapes at the decode batch sizes of the configs: time per launch over the
        # same rotation of weights (1-2 rows: dp4a kernel; 3 and more: tensor-core kernel, 16 rows per pass)
        batched = []
        with torch.cuda.stream(stream):
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
                    g = make_graph(body)
                    for _ in range(3):
                        g.replay()
                    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    b0.record(stream)
                    for _ in range(10):
                        g.replay()
                    b1.record(stream)
                    stream.synchronize()
                    us = b0.elapsed_time(b1) * 1e3 / (10 * LAYERS)
                    batched.append({"shape": label, "rows": m, "us_per_launch": us, "weight_GBps": nbytes / us / 1e3})
                    del g
        check_status()
    decode = None if args.no_decode else run_decode(world, rank, dev, args.quick_decode)
    if rank == 0:
        cpu, _ = cpu_time_sample() if world == 1 else (None, None)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 dot (dp4a) / f32 accumulate", "data": "synthetic (seeded normal weights sigma 0.02, quantized on the device)",
            "config": {"workload": "ffn_decode_q4k_q6k", "hidden": HID, "ffn": FFN, "batch": 1, "layers_per_step": LAYERS,
                       "bytes_per_step": step_bytes, "l2": "inputs larger than L2: each step streams %d MB of distinct weights" % (step_bytes // world // 10**6),
                       "launch": "cuda graph replay" if use_graph else "eager",
                       "parallelism": "single GPU" if world == 1 else f"tp{world}: gate/up split by rows, down by columns + NCCL allreduce"},
            "roofline": {"bound": "hbm", "kernel": "qmatvec_kernel<Q4_K> (gate, up, down at batch 1)", "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_src, "us_per_launch": q4_us,
                         "algorithmic_bytes_per_launch": q4_algo,
                         "traffic": 33059584.0, "traffic_note": "dram read+write per launch from ncu (profiles/)"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": (HID + FFN) * 4, "d2h_bytes_per_step": 2 * HID * 4,
                    "note": "activations from pinned host memory and projections back to it every step; weights resident in HBM"},
            "gpu_launches": launches_per_step[0] * args.steps,
            "clocks": clocks,
        }
        if cpu:
            out["cpu_baseline"] = cpu
        if batched is not None:
            out["batched_matvec"] = batched
        if decode is not None:
            out["decode"] = decode
        print(json.dumps(out), flush=True)
    if world > 1:
        # The NCCL communicator is referenced by the captured graphs: release them first, and do not let
        # a slow teardown outlive the measurement (the line above is already printed).
        import threading
        graph = q4_graph = None
        torch.cuda.synchronize()
        dist.barrier()
        threading.Timer(20.0, lambda: os._exit(0)).start()
        dist.destroy_process_group()
        os._exit(0)


def note(msg):
    """Progress line on stderr (QMM_BENCH_VERBOSE=1): where a multi-rank run is, should it stall."""
    if os.environ.get("QMM_BENCH_VERBOSE"):
        print(f"[bench rank {os.environ.get('RANK', '0')}] {msg}", file=sys.stderr, flush=True)


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
        d.close()
        del d
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the decode tok/s section")
    ap.add_argument("--quick-decode", action="store_true", help="decode section: 8B batch 1 only")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
