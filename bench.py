#!/usr/bin/env python
"""Benchmark of the contextual-sparsity MLP decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C2] [--impl reference]

A *step* is one decode token through every layer of the workload's sparse-MLP stack:
predictor -> mask -> differential weight-cache update -> sparse gate/up/down projection,
layer after layer, strictly serialised on one stream.  Metric: decode tokens/s = B / t_step.

Default workload (N = 1): "C2", the Llama-3.2-3B-shaped 28-layer stack, fp16, batch 1,
random-init weights N(0, 0.02), AR(1) hidden states, ~20 % active neurons per token.
For N > 1 the intermediate dimension is sharded over the ranks (one process per GPU,
launched by torch.distributed.run); the partial sums of a layer are added over peer memory
inside the step's own kernels (--allreduce nccl selects torch.distributed.all_reduce instead).
Other workloads: --workload C3 | C5 (batched decode stacks), C4 (prefill, tensor roofline),
C2-e2e (the LlamaSkip host end to end: TTFT and output tokens/s).

One JSON line is printed by rank 0:
  value      device-timed (CUDA events), inputs resident in HBM, CUDA-graph replay
  e2e        the same steps through the host-buffer C-ABI call (pinned host x in, result out)
  roofline   dominant kernel (the sparse MLP): algorithmic bytes / measured launch time
  cpu_baseline  the reference's own CPU implementation on this box's host cores, bounded sample
`--impl reference` times only that CPU implementation on the same workload definition.
"""
from __future__ import annotations

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

METRIC = "sparse_mlp_decode_tokens_per_s"
UNIT = "tokens/s"
DTYPE_NAME = {"torch.float32": "f32", "torch.float16": "f16", "torch.bfloat16": "bf16"}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="C2")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = workload default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="N>1: sum of the shards' outputs inside the library's kernels over peer memory, or NCCL")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU baseline sample")
    return ap.parse_args()


# ------------------------------------------------------------------------------ helpers

class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index
        self.t = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.t = threading.Thread(target=self._read, daemon=True)
        self.t.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json copy bandwidth)"
    except Exception:
        return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def traffic_ratio(kernel: str):
    """DRAM bytes / algorithmic bytes of the MLP kernel from the committed ncu capture."""
    try:
        with open(os.path.join(ROOT, "profiles", f"{kernel}_traffic.json")) as f:
            return float(json.load(f)["dram_over_algorithmic"])
    except Exception:
        return None


def mlp_algorithmic_bytes(w, K: float) -> float:
    """Sparse-MLP launch: active gate/up/down rows read once + x, a and the output."""
    s = w.dtype.itemsize if hasattr(w.dtype, "itemsize") else 2
    nmat = 3 if w.has_gate else 2
    return s * nmat * K * w.H + s * w.B * 2 * w.H + 4 * w.B * K


def layer_step_algorithmic_bytes(w, K: float, dK: float) -> float:
    """Whole layer step: predictor weights + active MLP weights + cache rows (pool read +
    packed write) + activations, scores and masks."""
    s = w.dtype.itemsize
    nmat = 3 if w.has_gate else 2
    return (s * (w.r * w.H + w.I * w.r) + s * nmat * K * w.H + 2 * s * nmat * dK * w.H
            + s * w.B * (2 * w.H + w.r + 2 * K) + w.B * w.I * s + 2 * w.I / 8)


# ------------------------------------------------------------------------------ CPU arm

def cpu_reference_run(w, n_layers: int, steps: int, warmup: int, seed: int = 0):
    """Times the reference's CPU path (compiled unmodified, oracle/_ref; else the C oracle) on
    `n_layers` layers of the workload in fp32 (the reference cache is fp32-only).
    Returns dict(value tokens/s for the full stack, kind, cores, sample, split)."""
    import torch

    from sparse_transformers_b200.synth import HiddenStream, layer_weights

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(seed)
    w32 = w.scaled(dtype=torch.float32)
    weights = [layer_weights(w32, gen) for _ in range(n_layers)]
    xs = HiddenStream(w32, gen).take(warmup + steps)
    kind = "reference"
    try:
        from oracle import ref_python as rp

        if not rp.have_reference():
            raise RuntimeError("no compiled reference")
        layers = [rp.RefLayer(*lw, act=w.act, method="threshold", tau=w.tau, has_gate=w.has_gate) for lw in weights]

        def step(x):
            for l in layers:
                l.step(x, op=True)
    except Exception:
        kind = "port"
        import numpy as np

        from oracle import oracle as orc

        f = lambda t: t.float().numpy()
        st = []
        for (g, u, d, A, Bm) in weights:
            c = orc.OracleCache(w.I)
            c.update(np.ones(w.I, bool))
            st.append((c, f(g), f(u), np.ascontiguousarray(f(d).T), f(A), f(Bm)))
        cores = 1

        def step(x):
            xn = f(x)
            for (c, g, u, dT, A, Bm) in st:
                _, s = orc.predictor(xn, A, Bm, orc.F32)
                _, m = orc.mask_threshold(s, orc.F32, w.tau)
                c.update(m)
                wcat = np.concatenate([c.gather(g), c.gather(u)]) if w.has_gate else c.gather(u)
                orc.sparse_mlp(xn, wcat, c.gather(dT), "relu", w.has_gate)

    for i in range(warmup):
        step(xs[i])
    times = []
    for i in range(warmup, warmup + steps):
        t0 = time.perf_counter()
        step(xs[i])
        times.append(time.perf_counter() - t0)
    total = sum(times)
    t_layer = total / (steps * n_layers)
    t_token = t_layer * w.layers
    sample = (f"{n_layers} of {w.layers} layers x {steps} decode steps of {w.name} in fp32 "
              f"(predictor + WeightCache.update_active_weights + sparse_mlp forward), scaled to {w.layers} layers")
    return {"value": w.B / t_token, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
            "ms_per_layer_step": t_layer * 1e3, "ms_per_step": total / steps * 1e3 * w.layers / n_layers}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS[args.workload]
    if args.layers:
        w = w.scaled(layers=args.layers)
    r = cpu_reference_run(w, min(args.cpu_layers, w.layers), args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args.gpus),
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(w, n_gpus, allreduce="peer"):
    return {"workload": w.name, "hidden": w.H, "intermediate": w.I, "predictor_rank": w.r, "layers": w.layers,
            "batch": w.B, "density_per_row": w.density, "activation": w.act, "threshold": round(w.tau, 6),
            "parallelism": "single GPU" if n_gpus == 1 else
            f"intermediate dim sharded over {n_gpus} GPUs + all-reduce per layer ("
            + ("peer-memory stores inside the step's kernels" if allreduce == "peer" else "NCCL") + ")",
            "cache_rows": "copied every step (eager), on a side branch of the step's graph",
            "l2": "distinct weights per layer: one step touches more bytes than the 126 MB L2"}


# ------------------------------------------------------------------------------ GPU arm

def run_native(args):
    import torch
    import torch.distributed as dist

    import sparse_transformers_b200 as stb
    from sparse_transformers_b200 import _capi as C
    from sparse_transformers_b200.sharded import PeerExchange, ShardedLayer, ShardedStack, shard_range
    from sparse_transformers_b200.synth import HiddenStream, WORKLOADS, layer_weights

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)

    w = WORKLOADS[args.workload]
    if args.layers:
        w = w.scaled(layers=args.layers)
    K_steps, W_steps = args.steps, max(args.warmup, 0)

    # ---- weights: generated on the device (identical on every rank), sliced per rank
    gen = torch.Generator(device=dev).manual_seed(0)
    layers = []
    peer = PeerExchange(w.B * w.H) if world > 1 and args.allreduce == "peer" else None
    cpu_weights = []  # first layers kept on the host for the CPU baseline sample (fp32)
    for li in range(w.layers):
        gate, up, down, A, Bm = layer_weights(w, gen, device=dev)
        if world == 1:
            layers.append(stb.SparseLayer(gate, up, down, A, Bm, act=w.act, method="threshold", param=w.tau,
                                          max_batch=w.B, has_gate=w.has_gate, alias_gate_up=True))
        else:
            lo, hi = shard_range(w.I, rank, world)
            layers.append(ShardedLayer(gate[lo:hi].contiguous(), up[lo:hi].contiguous(), down[:, lo:hi].contiguous(), A,
                                       Bm[lo:hi].contiguous(), act=w.act, method="threshold", param=w.tau,
                                       max_batch=w.B, has_gate=w.has_gate, peer=peer))
        del gate, up, down
    torch.cuda.synchronize()

    n_inst = 8  # steps of the stage-timing pass
    xs_cpu = HiddenStream(w, torch.Generator().manual_seed(1)).take(3 * (W_steps + K_steps) + n_inst + 16)
    xs_dev = xs_cpu.to(dev)
    cursor = 0

    if world == 1:
        stack = stb.SparseStack(layers, w.B)
    else:
        stack = ShardedStack(layers, w.B, xs_dev[0])
        cursor = 1

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out_dev = torch.empty(w.layers, w.B, w.H, dtype=w.dtype, device=dev)

    # ---- device-timed region (inputs resident in HBM)
    for _ in range(W_steps):
        stack.step(xs_dev[cursor], out_dev)
        cursor += 1
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(K_steps):
        stack.step(xs_dev[cursor], out_dev)
        cursor += 1
    ev1.record()
    barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the host-buffer call (pinned host in, result back to host)
    x_pin = torch.empty(w.B, w.H, dtype=w.dtype).pin_memory()
    o_pin = torch.empty(w.layers, w.B, w.H, dtype=w.dtype).pin_memory()
    for _ in range(W_steps):
        x_pin.copy_(xs_cpu[cursor])
        stack.step_host(x_pin, o_pin)
        cursor += 1
    barrier()
    t0 = time.perf_counter()
    for _ in range(K_steps):
        x_pin.copy_(xs_cpu[cursor])
        stack.step_host(x_pin, o_pin)
        cursor += 1
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device=dev)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_total = float(e2e_s.item())

    # ---- the same steps with lazy packed-row copies (index plan every step, rows on demand)
    lazy_value = None
    if world == 1:
        for l in layers:
            l.set_lazy_cache(True)
        lazy_stack = stb.SparseStack(layers, w.B)
        for _ in range(W_steps):
            lazy_stack.step(xs_dev[cursor % len(xs_dev)], out_dev)
            cursor += 1
        torch.cuda.synchronize()
        n_lazy = max(8, K_steps // 4)
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for _ in range(n_lazy):
            lazy_stack.step(xs_dev[cursor % len(xs_dev)], out_dev)
            cursor += 1
        l1.record()
        torch.cuda.synchronize()
        lazy_value = w.B / (l0.elapsed_time(l1) / n_lazy * 1e-3)
        lazy_stack.close()
        for l in layers:
            l.set_lazy_cache(False)

    # ---- stage timing pass (single GPU): the dominant kernel's launches timed alone with
    #      CUDA events on the launching stream, all layers back to back in one graph
    roofline, stages_us, k_mean, dk_mean = None, None, None, None
    if world == 1:
        # one row under the threshold rule: [t = A x] [scores + mask + gather + MLP] [sum of partials];
        # otherwise: [predictor] [gate/up] [down]
        fused = layers[0].single_row_fused(w.B)
        if fused:
            names = ("predict_t", "plan", "copy", "mlp_b1", "reduce")
            bits = (C.STAGE_PREDICT_T, C.STAGE_PLAN, C.STAGE_COPY, C.STAGE_PREDICT_MASK | C.STAGE_MLP_GATEUP,
                    C.STAGE_PREDICT_MASK | C.STAGE_MLP_DOWN)
        else:
            names = ("predict", "plan", "copy", "gateup", "down")
            bits = (C.STAGE_PREDICT, C.STAGE_PLAN, C.STAGE_COPY, C.STAGE_MLP_GATEUP, C.STAGE_MLP_DOWN)
        st = {n: stb.SparseStack(layers, w.B, stages=b) for n, b in zip(names, bits)}
        nbytes = w.B * w.H * w.dtype.itemsize
        xin = [torch.as_tensor(_DevBytes(st[n].buffers()[0], nbytes), device=dev) for n in (names[0], names[3])]
        acc = dict.fromkeys(names, 0.0)
        ks, dks = [], []
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        n_warm = 2
        for i in range(n_inst + n_warm):
            x = xs_dev[cursor % len(xs_dev)]
            cursor += 1
            for v in xin:  # stage the input in the stacks' own buffers, outside the timed brackets
                v.copy_(x.contiguous().view(torch.uint8).reshape(-1))
            torch.cuda.synchronize()
            for k, n in enumerate(names):  # one decode step, stage by stage over all layers
                evs[k].record()
                st[n].step(None, None)
            evs[len(names)].record()
            torch.cuda.synchronize()
            if i < n_warm:
                continue
            for n, a, b in zip(names, evs[:-1], evs[1:]):
                acc[n] += a.elapsed_time(b) * 1e3 / w.layers  # microseconds per layer
            for l in layers:
                ks.append(l.num_active())
                dks.append(l.update_stats()[2])
        stages_us = {k: v / n_inst for k, v in acc.items()}
        k_mean, dk_mean = statistics.mean(ks), statistics.mean(dks)
        peak, peak_src = measured_peak_gbs()
        es = w.dtype.itemsize
        if fused:
            # k_mlp_b1: active gate/up/down rows + the predictor's up matrix + x + t + mask bytes.  The
            # per-CTA partial vectors it writes are an artefact of the implementation, not counted.
            top, second, k1, k2 = "mlp_b1", "reduce", ("k_mlp_b1" if w.B == 1 else "k_mlp_bn"), "k_partial_reduce"
            alg = (es * (3 if w.has_gate else 2) * k_mean * w.H + es * w.I * w.r + es * w.B * w.H + 4 * w.B * w.r + w.I / 8)
            alg2 = (4 * (torch.cuda.get_device_properties(dev).multi_processor_count - 1) + es) * w.B * w.H
        else:
            top, second, k1, k2 = "gateup", "down", ("k_gateup_mma" if w.B >= 4 else "k_gateup_tma"), "k_down_rows"
            alg = es * (2 if w.has_gate else 1) * k_mean * w.H + es * w.B * w.H + 4 * w.B * k_mean  # gate/up rows + x + a
            alg2 = es * k_mean * w.H + 4 * w.B * k_mean + es * w.B * w.H                            # down rows + a + out
        achieved = alg / (stages_us[top] * 1e-6) / 1e9
        ratio = traffic_ratio(k1)
        roofline = {"kernel": k1, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "peak_source": peak_src, "frac_of_nominal_8000_gbs": achieved / 8000.0,
                    "traffic": (ratio * alg if ratio else None),
                    "algorithmic_bytes_per_launch": alg, "us_per_launch": stages_us[top],
                    "launches_timed": n_inst * w.layers,
                    "second_kernel": {"kernel": k2, "algorithmic_bytes_per_launch": alg2,
                                      "us_per_launch": stages_us[second],
                                      "achieved": alg2 / (stages_us[second] * 1e-6) / 1e9,
                                      "frac": alg2 / (stages_us[second] * 1e-6) / 1e9 / peak}}
        for s_ in st.values():
            s_.close()

    if world > 1:
        stack.close()
    if peer is not None:
        if peer.timed_out():
            print(f"rank {rank}: a wait for a peer's partial sums timed out; the numbers of this run are invalid",
                  file=sys.stderr)
        peer.close()
    if rank != 0:
        _finish_distributed(dist, world)
        return

    ms_step = ms_total / K_steps
    value = w.B / (ms_step * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K_steps, "warmup": W_steps,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
        "vs_baseline": None, "dtype": DTYPE_NAME[str(w.dtype)], "data": "synthetic",
        "config": workload_config(w, world, args.allreduce),
        "e2e": {"value": w.B / (e2e_total / K_steps), "unit": UNIT, "ms_per_step": e2e_total / K_steps * 1e3,
                "h2d_bytes_per_step": w.B * w.H * w.dtype.itemsize, "d2h_bytes_per_step": w.layers * w.B * w.H * w.dtype.itemsize},
        "gpu_launches": int(stack.launches_per_step * K_steps),
        "clocks": clocks,
    }
    if lazy_value is not None:
        line["value_lazy_cache_rows"] = lazy_value
    if roofline:
        line["roofline"] = roofline
        line["stages_us_per_layer"] = stages_us
        line["active_neurons_mean"] = k_mean
        line["rows_rewritten_mean"] = dk_mean
        step_alg = layer_step_algorithmic_bytes(w, k_mean, dk_mean) * w.layers
        line["step_algorithmic_gbs"] = step_alg / (ms_step * 1e-3) / 1e9
        line["step_frac_of_peak"] = line["step_algorithmic_gbs"] / roofline["peak"]
    if world == 1 and not args.no_cpu_baseline:
        # free the device side first? not needed: the CPU sample uses its own host copies
        try:
            cb = cpu_reference_run(w, min(args.cpu_layers, w.layers), steps=24, warmup=2)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:  # the baseline is a reported extra, never a reason to lose the line
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                    "sample": f"failed: {type(e).__name__}: {e}"}
    print(json.dumps(line), flush=True)
    _finish_distributed(dist, world)


def _finish_distributed(dist, world):
    """Leave a multi-rank run: barrier, then exit without destroy_process_group(), which was
    seen to block after NCCL collectives had been captured in CUDA graphs."""
    if world > 1:
        import torch

        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


class _DevBytes:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def run_prefill(args):
    """C4: the op-level prefill path (rows x packed active weights -> tcgen05 GEMMs) over a sweep
    of active fractions; prints one JSON line with the tensor roofline at K = I."""
    import ctypes

    import torch

    from sparse_transformers_b200 import _capi as C
    from sparse_transformers_b200.synth import WORKLOADS

    w = WORKLOADS["C4"]
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    T, H, I = w.B, w.H, w.I
    x = torch.randn(T, H, generator=gen, device=dev).to(w.dtype)
    cw_full = (torch.randn(2 * I, H, generator=gen, device=dev) * w.wstd).to(w.dtype)
    dp_full = (torch.randn(I, H, generator=gen, device=dev) * w.wstd).to(w.dtype)
    out = torch.empty(T, H, dtype=w.dtype, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
        peak_src = "measured (MEASURED_PEAKS.json cuBLAS bf16 burst)"
    except Exception:
        peak, peak_src = 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"
    sweep = {}
    for frac in (0.10, 0.25, 0.50, 1.00):
        K = int(I * frac)
        cw = torch.cat([cw_full[:K], cw_full[I:I + K]]).contiguous()
        dp = dp_full[:K].contiguous()
        comb = torch.empty(T, 2 * K, dtype=w.dtype, device=dev)
        n = ctypes.c_size_t()
        C.check(C.lib.stx_mlp_scratch_bytes(T, H, K, ctypes.byref(n)))
        scratch = torch.zeros(n.value, dtype=torch.uint8, device=dev)

        def call():
            C.check(C.lib.stx_sparse_mlp_forward(x.data_ptr(), T, H, cw.data_ptr(), dp.data_ptr(), K, out.data_ptr(),
                                                 comb.data_ptr(), C.ACT_RELU, 1, C.F16, scratch.data_ptr(), stream))
        for _ in range(max(3, args.warmup)):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = max(4, min(args.steps, 32))
        e0.record()
        for _ in range(steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        sweep[f"{frac:.2f}"] = {"K": K, "ms": ms, "tflops": 6.0 * T * H * K / (ms * 1e-3) / 1e12,
                                "rows_per_s": T / (ms * 1e-3)}
        del cw, dp, comb, scratch
    top = sweep["1.00"]
    line = {"metric": "sparse_mlp_prefill_tflops", "value": top["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
            "steps": max(4, min(args.steps, 32)), "warmup": max(3, args.warmup), "ms_per_step": top["ms"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": w.name, "rows": T, "hidden": H, "intermediate": I, "activation": "relu",
                       "l2": "x (64 MB) + packed weights (270 MB at K = I) exceed the 126 MB L2"},
            "roofline": {"kernel": "k_umma_gemm", "bound": "tensor", "achieved": top["tflops"], "peak": peak,
                         "unit": "TFLOP/s", "frac": top["tflops"] / peak, "peak_source": peak_src, "traffic": None,
                         "flops_per_step": 6.0 * T * H * I},
            "k_sweep": sweep, "gpu_launches": 3 * max(4, min(args.steps, 32))}
    print(json.dumps(line), flush=True)


def run_llama_skip(args):
    """`--workload C2-e2e`: the Llama-3.2-3B-shaped LlamaSkip host end to end (random-init weights,
    512 random prompt ids, 128 greedy tokens): TTFT and output tokens/s as the reference's benchmark
    defines them.  Prefill, the q/k/v projection and lm_head are torch ops; the decode-time MLP, norms,
    attention and output projection are this library."""
    import torch

    from sparse_transformers_b200.llama_skip import LlamaSkipConfig, LlamaSkipModel

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    dev = torch.device("cuda", 0)
    cfg = LlamaSkipConfig(layers=args.layers or 28)
    prompt = torch.randint(0, cfg.vocab, (512,), generator=torch.Generator().manual_seed(0)).to(dev)
    n_new = 128
    out = {}
    for lazy in (False, True):
        cfg.lazy_cache = lazy
        m = LlamaSkipModel(cfg, dev, seed=0)
        m.generate(prompt, 16)  # warm-up: cuBLAS handles, graph capture
        runs = [m.generate(prompt, n_new) for _ in range(3)]
        best = max(runs, key=lambda r: r["output_tokens_per_s"])
        dens = [float(L["sparse"].num_active()) / cfg.intermediate for L in m.layers]
        out["lazy" if lazy else "eager"] = dict(ttft_s=min(r["ttft_s"] for r in runs), output_tokens_per_s=best["output_tokens_per_s"],
                                                total_tokens_per_s=best["total_tokens_per_s"], active_fraction=sum(dens) / len(dens))
        m.close()
        del m
        torch.cuda.empty_cache()
    e = out["eager"]
    print(json.dumps({
        "metric": "llamaskip_output_tokens_per_s", "value": e["output_tokens_per_s"], "unit": UNIT, "n_gpus": 1,
        "higher_is_better": True, "dtype": "f16", "data": "synthetic", "ttft_s": e["ttft_s"],
        "total_tokens_per_s": e["total_tokens_per_s"], "active_fraction_last_token": e["active_fraction"],
        "value_lazy_cache_rows": out["lazy"]["output_tokens_per_s"], "vs_baseline": None,
        "config": {"workload": "C2-llamaskip-3b-e2e-fp16", "layers": cfg.layers, "hidden": cfg.hidden, "intermediate": cfg.intermediate,
                   "heads": cfg.heads, "kv_heads": cfg.kv_heads, "vocab": cfg.vocab, "rope_theta": cfg.rope_theta,
                   "predictor_rank": cfg.predictor_rank, "density_target": cfg.density, "prompt_tokens": 512, "new_tokens": n_new,
                   "decode": "one CUDA graph per token; sparse MLP, add+RMSNorm, RoPE+KV append+attention and the output projection are this library's kernels; q/k/v projection and lm_head are torch matmuls",
                   "prefill": "dense (torch GEMMs), as the reference does for sequences longer than one token"}}), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "C2-e2e":
        run_llama_skip(args)
    elif args.workload == "C4":
        run_prefill(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
