#!/usr/bin/env python
"""Benchmark of the contextual-sparsity MLP decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C2] [--impl reference]

A *step* is one decode token through every layer of the workload's sparse-MLP stack:
predictor -> mask -> differential weight-cache update -> sparse gate/up/down projection,
layer after layer.  Metric: decode tokens/s = B / t_step.

Default workload (headline at every N): "C2", the Llama-3.2-3B-shaped 28-layer stack, fp16,
batch 1, random-init weights N(0, 0.02), AR(1) hidden states, ~20 % active neurons per token.
Weights and hidden states are generated ONCE ON THE CPU from fixed seeds and uploaded, so the
GPU arm, the CPU reference arm and the parity check all see identical bits.
For N > 1 the intermediate dimension is sharded over the ranks (one process per GPU, launched
by torch.distributed.run); the partial sums of a layer are added over peer memory inside the
step's own kernels (--allreduce nccl selects torch.distributed.all_reduce instead).

One JSON line is printed by rank 0:
  value        device-timed (CUDA events) median over `blocks` timed blocks of exactly K steps
               each, inputs resident in HBM, CUDA-graph replay; value_spread = min / max block
  e2e          the same steps through the host-buffer C-ABI call (pinned host x in, result out)
  roofline     dominant kernel: algorithmic bytes per launch / measured launch time
  parity       2 sampled layers x 4 steps against the reference's own compiled CPU code on
               the same bits, outside the timed region (also at N > 1: summed output, per-shard
               cache orders)
  cpu_baseline the reference's own CPU implementation on this box's host cores, bounded sample
  extra keys   (N = 1) c1, c3, c4, c5, c2_e2e, dropin: the other configurations, bounded;
               (N > 1) c5: the sharded 64-row stack
`--impl reference` times only the reference CPU implementation on the same workload definition.
Other single-workload runs: --workload C3 | C5 (batched decode stacks), C4 (prefill, tensor
roofline), C2-e2e (the LlamaSkip host end to end: TTFT and output tokens/s).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
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
PARITY_STEPS = 4


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--workload", default="C2")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="override the number of layers (0 = workload default)")
    ap.add_argument("--blocks", type=int, default=0, help="timed blocks of --steps steps (0 = 25, bounded by 8192 steps in total)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no c1/c3/c4/c5/c2_e2e/dropin keys)")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-variants", action="store_true",
                    help="skip the variant stacks (lazy rows, strict order, per-layer kernels) and the stage timing pass: few launches, for profiler captures")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="N>1: sum of the shards' outputs inside the library's kernels over peer memory, or NCCL")
    ap.add_argument("--cpu-layers", type=int, default=4, help="layers in the CPU baseline sample")
    return ap.parse_args()


def load_synth():
    """sparse_transformers_b200/synth.py loaded by path: the workload definitions need torch only,
    and the reference arm must not load the native libraries."""
    spec = importlib.util.spec_from_file_location("stx_synth", os.path.join(ROOT, "sparse_transformers_b200", "synth.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["stx_synth"] = mod
    spec.loader.exec_module(mod)
    return mod


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


def measured_peak(key: str, fallback: float, what: str):
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)[key]), f"measured (MEASURED_PEAKS.json {what})"
    except Exception:
        return fallback, f"fallback ({fallback:g}, an earlier measurement of the same GPU type)"


def traffic_ratio(kernel: str):
    """(DRAM bytes / algorithmic bytes, source) of a kernel from the committed ncu capture."""
    path = os.path.join("profiles", f"{kernel}_traffic.json")
    try:
        with open(os.path.join(ROOT, path)) as f:
            d = json.load(f)
        return float(d["dram_over_algorithmic"]), f"{path} ({d.get('source', 'ncu capture of a smaller case, scaled by units')})"
    except Exception:
        return None, None


def layer_step_algorithmic_bytes(w, K: float, dK: float) -> float:
    """Whole layer step: predictor weights + active MLP weights + cache rows (pool read +
    packed write) + activations, scores and masks."""
    s = w.dtype.itemsize
    nmat = 3 if w.has_gate else 2
    return (s * (w.r * w.H + w.I * w.r) + s * nmat * K * w.H + 2 * s * nmat * dK * w.H
            + s * w.B * (2 * w.H + w.r + 2 * K) + w.B * w.I * s + 2 * w.I / 8)


def gen_layers(synth, w, n_layers: int, seed: int = 0):
    """Yields (gate, up, down, A, Bm) CPU tensors in the workload dtype, layer after layer, all
    drawn from ONE CPU generator: both arms and the parity check use this function."""
    import torch

    gen = torch.Generator().manual_seed(seed)
    for _ in range(n_layers):
        yield synth.layer_weights(w, gen)


def hidden_states(synth, w, n: int, seed: int = 1):
    import torch

    return synth.HiddenStream(w, torch.Generator().manual_seed(seed)).take(n)  # [n,B,H] CPU, workload dtype


# ------------------------------------------------------------------------------ CPU arm

def cpu_reference_run(synth, w, n_layers: int, steps: int, warmup: int):
    """Times the reference's CPU path (compiled unmodified, oracle/_ref; else the C oracle) on the
    first `n_layers` layers of the workload, fp32 arithmetic on the SAME bits the GPU arm holds
    (the workload-dtype weights and hidden states, upcast: the reference cache is fp32-only).
    Returns dict(value tokens/s for the full stack, kind, cores, sample, split)."""
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = [tuple(t.float() for t in lw) for lw in gen_layers(synth, w, n_layers)]
    xs = hidden_states(synth, w, warmup + steps).float()
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
    sample = (f"{n_layers} of {w.layers} layers x {steps} decode steps of {w.name} in fp32 on the GPU arm's bits "
              f"(predictor + WeightCache.update_active_weights + sparse_mlp forward), scaled to {w.layers} layers")
    return {"value": w.B / t_token, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
            "ms_per_layer_step": t_layer * 1e3, "ms_per_step": total / steps * 1e3 * w.layers / n_layers}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    synth = load_synth()
    w = synth.WORKLOADS[args.workload]
    if args.layers:
        w = w.scaled(layers=args.layers)
    steps = max(1, min(args.steps, 512))  # a step is a bounded sample (cpu-layers of the stack): the run ends within minutes
    r = cpu_reference_run(synth, w, min(args.cpu_layers, w.layers), steps, min(args.warmup, 4))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 4), "ms_per_step": r["ms_per_step"], "higher_is_better": True,
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
            "inputs": "weights (seed 0) and AR(1) hidden states (seed 1) generated on the CPU and uploaded",
            "cache_rows": "copied every step (eager): inside the step's kernel for single-row stacks, else on side branches "
                          "of the step's graph",
            "layer_order": "every layer reads the same x (the stack's contract), so the layers are independent: one kernel "
                           "forms the masks of all layers, then streams the active rows of layer after layer without a "
                           "grid barrier in between (value_layer_by_layer: the same layers one after the other with two "
                           "grid barriers each; value_strict_layer_order: nothing of layer l+1 starts before out[l] is "
                           "complete, the order a model needs that feeds out[l] into layer l+1)"
                           if w.B == 1 else "layer after layer on one stream",
            "l2": "distinct weights per layer: one step touches more bytes than the 126 MB L2"}


# ------------------------------------------------------------------------------ GPU arm

class _DevBytes:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class Built:
    """Layers + stack of one workload on this rank."""

    def __init__(self, layers, stack, peer, kept):
        self.layers, self.stack, self.peer, self.kept = layers, stack, peer, kept

    def close(self):
        import torch

        torch.cuda.synchronize()
        self.stack.close()
        for l in self.layers:
            l.close()
        self.layers = []


def build_workload(synth, w, dev, rank, world, allreduce, peer, warm_x, keep=()):
    """Uploads the CPU-generated weights (sliced per rank) and builds the step object.  `keep`:
    layer indices whose CPU weights are returned (for the parity check)."""
    import sparse_transformers_b200 as stb
    from sparse_transformers_b200.sharded import ShardedLayer, ShardedStack, shard_range

    layers, kept = [], {}
    for li, (gate, up, down, A, Bm) in enumerate(gen_layers(synth, w, w.layers)):
        if li in keep:
            kept[li] = (gate, up, down, A, Bm)
        if world == 1:
            layers.append(stb.SparseLayer(gate.to(dev), up.to(dev), down.to(dev), A.to(dev), Bm.to(dev), act=w.act,
                                          method="threshold", param=w.tau, max_batch=w.B, has_gate=w.has_gate, alias_gate_up=True))
        else:
            lo, hi = shard_range(w.I, rank, world)
            layers.append(ShardedLayer(gate[lo:hi].contiguous().to(dev), up[lo:hi].contiguous().to(dev),
                                       down[:, lo:hi].contiguous().to(dev), A.to(dev), Bm[lo:hi].contiguous().to(dev), act=w.act,
                                       method="threshold", param=w.tau, max_batch=w.B, has_gate=w.has_gate,
                                       peer=peer if allreduce == "peer" else None))
        del gate, up, down
    stack = stb.SparseStack(layers, w.B) if world == 1 else ShardedStack(layers, w.B, warm_x)
    return Built(layers, stack, peer, kept)


def time_blocks(stack, xs_dev, cursor, K, blocks, out_dev, barrier, dist, world, dev):
    """`blocks` timed blocks of exactly K steps each (CUDA events on the launching stream, max over
    ranks per block).  Returns (list of ms per block, cursor)."""
    import torch

    ms = []
    for _ in range(blocks):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            stack.step(xs_dev[cursor % len(xs_dev)], out_dev)
            cursor += 1
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms.append(float(t.item()))
    return ms, cursor


def parity_check(synth, w, kept, dev, rank, world, allreduce, peer, dist):
    """2 sampled layers x PARITY_STEPS steps on fresh caches, outside any timed region: the GPU step
    (all-reduced output at N > 1) against the reference's compiled CPU code (oracle/_ref; the C
    restatement if that is absent) in fp32 on the same bits.
      mask_flips        GPU mask bits that differ from the reference's own fp32 nn.Linear pair + threshold
                        (the GPU rounds t and the scores to the model dtype like the reference would in that
                        dtype, the fp32 reference arm does not: flips can only sit within rounding distance of tau)
      max_flip_margin   largest |score - tau| among flipped neurons (fp32 reference score)
      mask_equal_fixed_order   GPU mask == the CPU restatement with the kernels' documented summation order
      cache_order_equal every shard's cache order == the reference index plan fed the same masks
      cache_rows_equal  (N = 1) packed gate/up rows == the compiled reference cache's concat weight
      out_rel_err       max |out - ref| / max |ref| over layers and steps"""
    import numpy as np
    import torch

    import sparse_transformers_b200 as stb
    from sparse_transformers_b200.sharded import ShardedLayer, ShardedStack, shard_range

    ids = sorted(kept)
    wp = w.scaled(layers=len(ids))
    xs = hidden_states(synth, w, PARITY_STEPS + 1, seed=7)
    lo, hi = shard_range(w.I, rank, world)
    layers = []
    for li in ids:
        gate, up, down, A, Bm = kept[li]
        if world == 1:
            layers.append(stb.SparseLayer(gate.to(dev), up.to(dev), down.to(dev), A.to(dev), Bm.to(dev), act=w.act,
                                          method="threshold", param=w.tau, max_batch=w.B, has_gate=w.has_gate))
        else:
            layers.append(ShardedLayer(gate[lo:hi].contiguous().to(dev), up[lo:hi].contiguous().to(dev),
                                       down[:, lo:hi].contiguous().to(dev), A.to(dev), Bm[lo:hi].contiguous().to(dev), act=w.act,
                                       method="threshold", param=w.tau, max_batch=w.B, has_gate=w.has_gate,
                                       peer=peer if allreduce == "peer" else None))
    # ShardedStack warms up with two eager steps of its warm-up input: the reference side replays them
    stack = stb.SparseStack(layers, w.B) if world == 1 else ShardedStack(layers, w.B, xs[0].to(dev))
    warm = [xs[0]] * getattr(stack, "warmup_steps", 0)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()  # start the first step together (bounded waits for the peers)
    local = [l if world == 1 else l.local for l in layers]

    ref = None
    if rank == 0:
        from oracle import oracle as orc
        from oracle import ref_python as rp

        kind = "reference" if rp.have_reference() else "port"
        ref = []
        for li in ids:
            g32, u32, d32, A32, B32 = (t.float() for t in kept[li])
            rl = rp.RefLayer(g32, u32, d32, A32, B32, act=w.act, tau=w.tau, has_gate=w.has_gate) if kind == "reference" else None
            ocs = []
            for q in range(world):
                oc = orc.OracleCache(shard_range(w.I, q, world)[1] - shard_range(w.I, q, world)[0])
                oc.update(np.ones(oc.I, bool))
                ocs.append(oc)
            ref.append((rl, ocs, (g32, u32, d32, A32, B32)))
    stats = {"mask_flips": 0, "mask_bits_compared": 0, "max_flip_margin": 0.0, "mask_equal_fixed_order": True,
             "cache_order_equal": True, "cache_rows_equal": True if world == 1 else None, "out_rel_err": 0.0}
    odt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[w.dtype]
    out = torch.empty(len(ids), w.B, w.H, dtype=w.dtype, device=dev)

    def gather(obj):
        if world == 1:
            return [obj]
        got = [None] * world if rank == 0 else None
        dist.gather_object(obj, got, dst=0)
        return got

    def reference_step(k, x, masks, orders, got, check):
        rl, ocs, (g32, u32, d32, A32, B32) = ref[k]
        m_gpu = torch.cat(masks)
        x32 = x.float()
        if check:
            s_ref = torch.nn.functional.linear(torch.nn.functional.linear(x32, A32), B32)  # modeling_skip.py:52-53
            m_ref = (s_ref >= w.tau).any(dim=0)
            flip = m_gpu != m_ref
            stats["mask_flips"] += int(flip.sum())
            stats["mask_bits_compared"] += int(m_gpu.numel())
            if flip.any():
                stats["max_flip_margin"] = max(stats["max_flip_margin"], float((s_ref - w.tau).abs().min(dim=0).values[flip].max()))
            _, s_fix = orc.predictor(x32.numpy(), A32.numpy(), B32.numpy(), odt)
            _, m_fix = orc.mask_threshold(s_fix, odt, w.tau)
            stats["mask_equal_fixed_order"] &= bool(np.array_equal(m_fix, m_gpu.numpy()))
        for q in range(world):
            qlo, qhi = shard_range(w.I, q, world)
            ocs[q].update(m_gpu[qlo:qhi].numpy())
            if check:
                stats["cache_order_equal"] &= (ocs[q].active + qlo).tolist() == orders[q]
        if rl is not None:
            rl.wc.update_active_weights(m_gpu)
            if check:
                cw, dw = rl.wc.get_concat_weight(), rl.wc.get_active_down_weight()
                want = rp.skip_mlp_sparse(x32, cw, dw, w.act, w.has_gate)
                err = float((got.float() - want).abs().max() / want.abs().max())
                stats["out_rel_err"] = max(stats["out_rel_err"], err)
                if world == 1:
                    stats["cache_rows_equal"] &= bool(torch.equal(local[k].concat_weight().float().cpu(), cw))
        elif check:
            act = torch.cat([torch.from_numpy(ocs[q].active.astype(np.int64)) + shard_range(w.I, q, world)[0] for q in range(world)])
            gg, uu, dd = g32[act], u32[act], d32[:, act]
            want = rp.skip_mlp_sparse(x32, torch.cat([gg, uu]) if w.has_gate else uu, dd, w.act, w.has_gate)
            stats["out_rel_err"] = max(stats["out_rel_err"], float((got.float() - want).abs().max() / want.abs().max()))

    # the sharded stack's warm-up steps advanced the shard caches with xs[0]: bring the reference side along
    if warm:
        for k in range(len(ids)):
            masks = gather(local[k].mask().cpu())
            if rank == 0:
                reference_step(k, xs[0], masks, None, None, check=False)
    for t in range(1, PARITY_STEPS + 1):
        x = xs[t]
        if world > 1:
            dist.barrier()  # rank 0 checks against the CPU reference between steps: enter each collective step together
        stack.step(x.to(dev), out)
        torch.cuda.synchronize()
        got = out.cpu()
        for k in range(len(ids)):
            masks = gather(local[k].mask().cpu())
            orders = gather((local[k].active_indices() + lo).tolist())
            if rank == 0:
                reference_step(k, x, masks, orders, got[k], check=True)
    if peer is not None and allreduce == "peer":
        stats["peer_wait_timed_out"] = bool(peer.timed_out())
    stack.close()
    for l in layers:
        l.close()
    if rank != 0:
        return None
    stats.update({"layers": ids, "steps": PARITY_STEPS, "reference": kind, "rows": w.B,
                  "score_rounding_step_at_tau": (0.0 if w.dtype == torch.float32 else
                                                 2.0 ** (math.floor(math.log2(abs(w.tau))) - (10 if w.dtype == torch.float16 else 7))),
                  "tolerance_out_rel_err": 1e-5 if w.dtype == torch.float32 else 2e-2})
    return stats


def stack_measure(synth, w, args, dev, rank, world, dist, peer, extras_mode=False):
    """Builds the workload on this rank, times it, checks parity.  Returns the result dict (rank 0)
    or None.  extras_mode: bounded run for an extra key (fewer blocks, no CPU baseline, no stage pass)."""
    import torch

    import sparse_transformers_b200 as stb
    from sparse_transformers_b200 import _capi as C

    K_steps = args.steps if not extras_mode else min(args.steps, 16)
    W_steps = max(args.warmup, 3)
    blocks = args.blocks or 25
    blocks = max(1, min(blocks, 8192 // max(K_steps, 1)))
    if extras_mode:
        blocks = 3
    n_e2e_blocks = 1 if extras_mode else 3
    n_x = min(4096, W_steps * 4 + K_steps * (blocks + n_e2e_blocks + 3) + 64)
    xs_cpu = hidden_states(synth, w, n_x)
    xs_dev = xs_cpu.to(dev)
    keep = (0, w.layers - 1) if not args.no_parity else ()
    built = build_workload(synth, w, dev, rank, world, args.allreduce, peer, xs_dev[0], keep=keep)
    layers, stack = built.layers, built.stack
    local = [l if world == 1 else l.local for l in layers]
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out_dev = torch.empty(w.layers, w.B, w.H, dtype=w.dtype, device=dev)
    cursor = 1
    barrier()  # the ranks built their shards at different speeds; a step's waits for the peers are bounded (seconds)
    for _ in range(W_steps):
        stack.step(xs_dev[cursor % n_x], out_dev)
        cursor += 1
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    ms_blocks, cursor = time_blocks(stack, xs_dev, cursor, K_steps, blocks, out_dev, barrier, dist, world, dev)
    clocks = sampler.stop() if rank == 0 else None
    ms_med = statistics.median(ms_blocks)

    # ---- end to end through the host-buffer call (pinned host in, result back to host)
    x_pin = torch.empty(w.B, w.H, dtype=w.dtype).pin_memory()
    o_pin = torch.empty(w.layers, w.B, w.H, dtype=w.dtype).pin_memory()
    for _ in range(W_steps):
        x_pin.copy_(xs_cpu[cursor % n_x])
        stack.step_host(x_pin, o_pin)
        cursor += 1
    e2e_blocks = []
    for _ in range(n_e2e_blocks):
        barrier()
        t0 = time.perf_counter()
        for _ in range(K_steps):
            x_pin.copy_(xs_cpu[cursor % n_x])
            stack.step_host(x_pin, o_pin)
            cursor += 1
        barrier()
        t = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_blocks.append(float(t.item()))
    e2e_s = statistics.median(e2e_blocks)

    res = {"ms_blocks": ms_blocks, "ms_per_step": ms_med / K_steps, "value": w.B / (ms_med / K_steps * 1e-3),
           "e2e_value": w.B / (e2e_s / K_steps), "e2e_ms_per_step": e2e_s / K_steps * 1e3,
           "launches_per_step": int(stack.launches_per_step), "steps": K_steps, "warmup": W_steps, "blocks": blocks,
           "clocks": clocks}
    ks = [l.num_active() for l in local]
    dks = [l.update_stats()[2] for l in local]
    res["active_neurons_mean"] = float(sum(ks)) * (world if world > 1 else 1) / len(ks)
    res["rows_rewritten_mean"] = float(sum(dks)) * (world if world > 1 else 1) / len(dks)

    # ---- variants of the same steps (single GPU): other layer order / kernels / lazy cache rows
    def variant(env=None, lazy=False):
        old = {}
        for k, v in (env or {}).items():
            old[k] = os.environ.get(k)
            os.environ[k] = v
        for l in layers:
            l.set_lazy_cache(lazy)
        st = stb.SparseStack(layers, w.B)
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        c = cursor
        for _ in range(W_steps):
            st.step(xs_dev[c % n_x], out_dev)
            c += 1
        ms, _ = time_blocks(st, xs_dev, c, min(K_steps, 64), 3, out_dev, barrier, dist, world, dev)
        st.close()
        for l in layers:
            l.set_lazy_cache(False)
        return w.B / (statistics.median(ms) / min(K_steps, 64) * 1e-3)

    if world == 1 and not extras_mode and not args.no_variants:
        res["value_lazy_cache_rows"] = variant(lazy=True)
        if w.B == 1:
            res["value_layer_by_layer"] = variant({"STX_STACK_ORDER": "layerwise"})
            res["value_strict_layer_order"] = variant({"STX_STACK_STRICT": "1"})
            res["value_per_layer_kernels"] = variant({"STX_STACK_KERNEL": "layers"})

    # ---- stage timing pass (single GPU): the dominant kernel's launches timed alone with CUDA
    #      events on the launching stream
    if world == 1 and not extras_mode and not args.no_variants:
        persistent = w.B == 1 and stack.launches_per_step <= 2 + 2 * w.layers
        fused = layers[0].single_row_fused(w.B)
        if persistent:
            names = ("stack_kernel", "plan", "copy")
            bits = (C.STAGE_PREDICT | C.STAGE_MLP, C.STAGE_PLAN, C.STAGE_COPY)
        elif fused:
            names = ("predict_t", "plan", "copy", "mlp_b1", "reduce")
            bits = (C.STAGE_PREDICT_T, C.STAGE_PLAN, C.STAGE_COPY, C.STAGE_PREDICT_MASK | C.STAGE_MLP_GATEUP,
                    C.STAGE_PREDICT_MASK | C.STAGE_MLP_DOWN)
        else:
            names = ("predict", "plan", "copy", "gateup", "down")
            bits = (C.STAGE_PREDICT, C.STAGE_PLAN, C.STAGE_COPY, C.STAGE_MLP_GATEUP, C.STAGE_MLP_DOWN)
        st = {n: stb.SparseStack(layers, w.B, stages=b) for n, b in zip(names, bits)}
        nbytes = w.B * w.H * w.dtype.itemsize
        xin = [torch.as_tensor(_DevBytes(s_.buffers()[0], nbytes), device=dev) for s_ in st.values()]
        acc = dict.fromkeys(names, 0.0)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)]
        n_inst, n_warm = 16, 3
        for i in range(n_inst + n_warm):
            x = xs_dev[cursor % n_x]
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
        stages_us = {k: v / n_inst for k, v in acc.items()}
        k_mean = statistics.mean(l.num_active() for l in layers)
        dk_mean = statistics.mean(l.update_stats()[2] for l in layers)
        peak, peak_src = measured_peak("hbm_gbs", 6650.0, "copy bandwidth")
        es = w.dtype.itemsize
        nmat = 3 if w.has_gate else 2
        if persistent:
            # one launch = all layers: per layer the active gate/up/down rows + both predictor matrices + x + t + mask
            # bytes (read and written).  The per-CTA partial vectors are an artefact of the implementation, not counted.
            top, k1, launches = "stack_kernel", "k_stack_flow", 1
            alg_layer = es * nmat * k_mean * w.H + es * (w.I * w.r + w.r * w.H) + 2 * es * w.H + 8 * w.r + 2 * w.I / 8
            alg = alg_layer * w.layers
            us = stages_us[top] * w.layers
            second = ("k_cache_copy_rows", "copy", 2 * nmat * dk_mean * w.H * es)
        elif fused:
            top, k1, launches = "mlp_b1", ("k_mlp_b1" if w.B == 1 else "k_mlp_bn"), w.layers
            alg = es * nmat * k_mean * w.H + es * w.I * w.r + es * w.B * w.H + 4 * w.B * w.r + w.I / 8
            us = stages_us[top]
            second = ("k_partial_reduce", "reduce", (4 * (torch.cuda.get_device_properties(dev).multi_processor_count - 1) + es) * w.B * w.H)
        else:
            top, k1, launches = "gateup", ("k_gateup_mma" if w.B >= 4 else "k_gateup_tma"), w.layers
            alg = es * (2 if w.has_gate else 1) * k_mean * w.H + es * w.B * w.H + 4 * w.B * k_mean
            us = stages_us[top]
            second = ("k_down_rows", "down", es * k_mean * w.H + 4 * w.B * k_mean + es * w.B * w.H)
        achieved = alg / (us * 1e-6) / 1e9
        ratio, tsrc = traffic_ratio(k1)
        res["roofline"] = {"kernel": k1, "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                           "frac": achieved / peak, "peak_source": peak_src, "frac_of_nominal_8000_gbs": achieved / 8000.0,
                           "traffic": (ratio * alg if ratio else None), "traffic_source": tsrc,
                           "algorithmic_bytes_per_launch": alg, "us_per_launch": us,
                           "launches_timed": n_inst * launches, "layers_per_launch": w.layers if persistent else 1,
                           "second_kernel": {"kernel": second[0], "algorithmic_bytes_per_launch": second[2],
                                             "us_per_launch": stages_us[second[1]],
                                             "achieved": second[2] / (stages_us[second[1]] * 1e-6) / 1e9,
                                             "frac": second[2] / (stages_us[second[1]] * 1e-6) / 1e9 / peak}}
        res["stages_us_per_layer"] = stages_us
        res["active_neurons_mean"], res["rows_rewritten_mean"] = k_mean, dk_mean
        step_alg = layer_step_algorithmic_bytes(w, k_mean, dk_mean) * w.layers
        res["step_algorithmic_gbs"] = step_alg / (res["ms_per_step"] * 1e-3) / 1e9
        res["step_frac_of_peak"] = res["step_algorithmic_gbs"] / peak
        for s_ in st.values():
            s_.close()

    built.close()
    if world > 1 and peer is not None and args.allreduce == "peer" and peer.timed_out():
        print(f"rank {rank}: a wait for a peer's partial sums timed out; the numbers of this run are invalid", file=sys.stderr)
        res["peer_wait_timed_out"] = True
    torch.cuda.empty_cache()
    if not args.no_parity:
        res["parity"] = parity_check(synth, w, built.kept, dev, rank, world, args.allreduce, peer, dist)
    built.kept = {}
    return res if rank == 0 else None


def run_native(args):
    import torch
    import torch.distributed as dist

    from sparse_transformers_b200.sharded import PeerExchange

    synth = load_synth()
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

    w = synth.WORKLOADS[args.workload]
    if args.layers:
        w = w.scaled(layers=args.layers)
    wc5 = synth.WORKLOADS["C5"]
    peer = None
    if world > 1 and args.allreduce == "peer":
        peer = PeerExchange(max(w.B * w.H, wc5.B * wc5.H))

    r = stack_measure(synth, w, args, dev, rank, world, dist, peer)
    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": world, "steps": r["steps"], "warmup": r["warmup"],
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak" if world == 1 else "strong",
            "vs_baseline": None, "dtype": DTYPE_NAME[str(w.dtype)], "data": "synthetic",
            "config": workload_config(w, world, args.allreduce),
            "blocks": r["blocks"],
            "value_spread": {"min": w.B / (max(r["ms_blocks"]) / r["steps"] * 1e-3), "max": w.B / (min(r["ms_blocks"]) / r["steps"] * 1e-3),
                             "what": f"tokens/s of the slowest and fastest of {r['blocks']} timed blocks of {r['steps']} steps; value is the median block"},
            "e2e": {"value": r["e2e_value"], "unit": UNIT, "ms_per_step": r["e2e_ms_per_step"],
                    "h2d_bytes_per_step": w.B * w.H * w.dtype.itemsize, "d2h_bytes_per_step": w.layers * w.B * w.H * w.dtype.itemsize},
            "gpu_launches": r["launches_per_step"] * r["steps"],
            "gpu_launches_per_step": r["launches_per_step"],
            "clocks": r["clocks"],
        }
        for k in ("value_lazy_cache_rows", "value_layer_by_layer", "value_strict_layer_order", "value_per_layer_kernels", "roofline", "stages_us_per_layer",
                  "active_neurons_mean", "rows_rewritten_mean", "step_algorithmic_gbs", "step_frac_of_peak", "parity", "peer_wait_timed_out"):
            if k in r:
                line[k] = r[k]

    # ---- extra keys: the other configurations, bounded
    if not args.no_extras and args.workload == "C2":
        ex = argparse.Namespace(**vars(args))
        ex.steps, ex.warmup, ex.blocks = 16, 3, 3
        try:
            c5 = stack_measure(synth, wc5, ex, dev, rank, world, dist, peer, extras_mode=True)
            if rank == 0:
                line["c5"] = extra_summary(wc5, c5, world, args.allreduce)
        except Exception as e:  # an extra key never costs the headline
            if rank == 0:
                line["c5"] = {"error": f"{type(e).__name__}: {e}"}
        if world == 1:
            for key, fn in (("c3", lambda: extra_summary(synth.WORKLOADS["C3"],
                                                         stack_measure(synth, synth.WORKLOADS["C3"], ex, dev, 0, 1, dist, None, extras_mode=True), 1, "peer")),
                            ("c1", lambda: extra_summary(synth.WORKLOADS["C1"],
                                                         stack_measure(synth, synth.WORKLOADS["C1"], ex, dev, 0, 1, dist, None, extras_mode=True), 1, "peer")),
                            ("c4", lambda: prefill_measure(args, dev)),
                            ("dropin", lambda: dropin_measure(synth, w, dev)),
                            ("c2_e2e", lambda: llama_skip_measure(args, dev, runs=2))):
                try:
                    line[key] = fn()
                except Exception as e:
                    line[key] = {"error": f"{type(e).__name__}: {e}"}
                torch.cuda.empty_cache()

    if peer is not None:
        peer.close()
    if rank != 0:
        _finish_distributed(dist, world)
        return
    if world == 1 and not args.no_cpu_baseline:
        try:
            cb = cpu_reference_run(synth, w, min(args.cpu_layers, w.layers), steps=24, warmup=2)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:  # the baseline is a reported extra, never a reason to lose the line
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "reference",
                                    "sample": f"failed: {type(e).__name__}: {e}"}
    print(json.dumps(line), flush=True)
    _finish_distributed(dist, world)


def extra_summary(w, r, world, allreduce):
    if r is None:
        return None
    out = {"workload": w.name, "tokens_per_s": r["value"], "ms_per_step": r["ms_per_step"], "e2e_tokens_per_s": r["e2e_value"],
           "steps": r["steps"], "blocks": r["blocks"], "n_gpus": world, "rows": w.B, "layers": w.layers,
           "active_neurons_mean": r["active_neurons_mean"], "rows_rewritten_mean": r["rows_rewritten_mean"],
           "gpu_launches_per_step": r["launches_per_step"]}
    peak, _ = measured_peak("hbm_gbs", 6650.0, "copy bandwidth")
    alg = layer_step_algorithmic_bytes(w, r["active_neurons_mean"], r["rows_rewritten_mean"]) * w.layers
    out["step_algorithmic_gbs"] = alg / (r["ms_per_step"] * 1e-3) / 1e9
    out["step_frac_of_hbm_peak"] = out["step_algorithmic_gbs"] / peak / world
    if "parity" in r:
        out["parity"] = r["parity"]
    return out


def _finish_distributed(dist, world):
    """Leave a multi-rank run: the peer objects are closed and every captured graph is released before this
    point.  The ranks meet once more and tear the process group down; a watchdog ends the process if the
    teardown has not returned after 20 s (it blocked at the end of earlier runs of this benchmark) and says so
    on stderr, so that the run can never hang on its way out."""
    if world > 1:
        import torch

        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()

        def bail():
            sys.stderr.write("bench.py: destroy_process_group() did not return within 20 s; leaving without it\n")
            sys.stderr.flush()
            os._exit(0)

        t = threading.Timer(20.0, bail)
        t.daemon = True
        t.start()
        dist.destroy_process_group()
        t.cancel()


# ------------------------------------------------------------------------------ other workloads

def prefill_measure(args, dev):
    """C4: the op-level prefill path (rows x packed active weights -> tcgen05 GEMMs) over a sweep of
    active fractions."""
    import ctypes

    import torch

    from sparse_transformers_b200 import _capi as C

    synth = load_synth()
    w = synth.WORKLOADS["C4"]
    gen = torch.Generator().manual_seed(0)
    T, H, I = w.B, w.H, w.I
    x = torch.randn(T, H, generator=gen).to(w.dtype).to(dev)
    cw_full = (torch.randn(2 * I, H, generator=gen) * w.wstd).to(w.dtype).to(dev)
    dp_full = (torch.randn(I, H, generator=gen) * w.wstd).to(w.dtype).to(dev)
    out = torch.empty(T, H, dtype=w.dtype, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    peak, peak_src = measured_peak("bf16_tflops", 1590.0, "cuBLAS bf16 burst")
    sweep = {}
    steps = max(4, min(args.steps, 16))
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
    return {"workload": w.name, "tflops": top["tflops"], "ms_per_step": top["ms"], "rows": T, "steps": steps,
            "roofline": {"kernel": "k_umma_gemm", "bound": "tensor", "achieved": top["tflops"], "peak": peak,
                         "unit": "TFLOP/s", "frac": top["tflops"] / peak, "peak_source": peak_src, "traffic": None,
                         "flops_per_step": 6.0 * T * H * I},
            "k_sweep": sweep, "gpu_launches": 3 * steps,
            "l2": "x (64 MB) + packed weights (270 MB at K = I) exceed the 126 MB L2"}


def run_prefill(args):
    import torch

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    r = prefill_measure(args, dev)
    line = {"metric": "sparse_mlp_prefill_tflops", "value": r["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
            "steps": r["steps"], "warmup": max(3, args.warmup), "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": r["workload"], "rows": r["rows"], "activation": "relu", "l2": r["l2"]},
            "roofline": r["roofline"], "k_sweep": r["k_sweep"], "gpu_launches": r["gpu_launches"]}
    print(json.dumps(line), flush=True)


def dropin_measure(synth, w, dev, steps: int = 24):
    """C2 through the reference-named API only, as src/modeling_skip.py:204-217,114-117 calls it:
    predict_mask -> WeightCache.update_active_weights -> get_concat_weight / get_active_down_weight ->
    sparse_mlp.forward, layer after layer from Python (each getter reads K back from the device)."""
    import torch

    import sparse_transformers_b200 as stb

    n_layers = w.layers
    caches, preds = [], []
    for (gate, up, down, A, Bm) in gen_layers(synth, w, n_layers):
        caches.append(stb.WeightCache(torch.ones(w.I, dtype=torch.bool, device=dev), w.H, gate.to(dev), up.to(dev), down.to(dev), True))
        preds.append((A.to(dev), Bm.to(dev)))
    xs = hidden_states(synth, w, steps + 4).to(dev)
    down_buf = torch.zeros(1, w.H, dtype=w.dtype, device=dev)
    comb_buf = torch.zeros(1, 2, dtype=w.dtype, device=dev)

    def token(x):
        for wc, (A, Bm) in zip(caches, preds):
            mask = torch.ops.sparse_mlp.predict_mask(x, A, Bm, "threshold", w.tau)
            wc.update_active_weights(mask)
            stb.sparse_mlp_forward(x, wc.get_concat_weight(), wc.get_active_down_weight(), down_buf, comb_buf, w.act)
    for i in range(4):
        token(xs[i])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(4, 4 + steps):
        token(xs[i])
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps

    # the same calls without the two getters (WeightCache.sparse_forward keeps K on the device): nothing
    # synchronises, so a whole token is captured in one CUDA graph and replayed
    x_static = xs[0].clone()
    bufs = [torch.zeros(1, w.H, dtype=w.dtype, device=dev) for _ in range(n_layers)]

    def token_nosync():
        for wc, (A, Bm), b in zip(caches, preds, bufs):
            wc.update_active_weights(torch.ops.sparse_mlp.predict_mask(x_static, A, Bm, "threshold", w.tau))
            wc.sparse_forward(x_static, b, w.act)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            token_nosync()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        token_nosync()
    for i in range(4):
        x_static.copy_(xs[i])
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(4, 4 + steps):
        x_static.copy_(xs[i])
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    dt_graph = e0.elapsed_time(e1) * 1e-3 / steps
    del graph, caches, preds
    return {"tokens_per_s": w.B / dt, "ms_per_step": dt * 1e3, "steps": steps,
            "path": "torch.ops.sparse_mlp.predict_mask -> WeightCache.update_active_weights -> get_concat_weight -> "
                    "get_active_down_weight -> torch.ops.sparse_mlp.forward per layer, called from Python (wall clock)",
            "host_syncs_per_layer": 2,
            "no_sync": {"tokens_per_s": w.B / dt_graph, "ms_per_step": dt_graph * 1e3,
                        "path": "predict_mask -> update_active_weights -> WeightCache.sparse_forward per layer (K stays on the "
                                "device, no host synchronisation), one CUDA graph per token, device-timed"}}


def llama_skip_measure(args, dev, runs: int = 3):
    import torch

    from sparse_transformers_b200.llama_skip import LlamaSkipConfig, LlamaSkipModel

    cfg = LlamaSkipConfig(layers=args.layers or 28)
    prompt = torch.randint(0, cfg.vocab, (512,), generator=torch.Generator().manual_seed(0)).to(dev)
    n_new = 128
    out = {}
    for lazy in (False, True):
        cfg.lazy_cache = lazy
        m = LlamaSkipModel(cfg, dev, seed=0)
        m.generate(prompt, 16)  # warm-up: cuBLAS handles, graph capture
        rs = [m.generate(prompt, n_new) for _ in range(runs)]
        best = max(rs, key=lambda r: r["output_tokens_per_s"])
        dens = [float(L["sparse"].num_active()) / cfg.intermediate for L in m.layers]
        out["lazy" if lazy else "eager"] = dict(ttft_s=min(r["ttft_s"] for r in rs), output_tokens_per_s=best["output_tokens_per_s"],
                                                total_tokens_per_s=best["total_tokens_per_s"], active_fraction=sum(dens) / len(dens))
        m.close()
        del m
        torch.cuda.empty_cache()
    e = out["eager"]
    return {"output_tokens_per_s": e["output_tokens_per_s"], "ttft_s": e["ttft_s"], "total_tokens_per_s": e["total_tokens_per_s"],
            "active_fraction_last_token": e["active_fraction"], "output_tokens_per_s_lazy_cache_rows": out["lazy"]["output_tokens_per_s"],
            "config": {"workload": "C2-llamaskip-3b-e2e-fp16", "layers": cfg.layers, "hidden": cfg.hidden, "intermediate": cfg.intermediate,
                       "heads": cfg.heads, "kv_heads": cfg.kv_heads, "vocab": cfg.vocab, "rope_theta": cfg.rope_theta,
                       "predictor_rank": cfg.predictor_rank, "density_target": cfg.density, "prompt_tokens": 512, "new_tokens": n_new,
                       "decode": "one CUDA graph per token; sparse MLP, add+RMSNorm, RoPE+KV append+attention and the output projection are this library's kernels; q/k/v projection and lm_head are torch matmuls",
                       "prefill": "dense (torch GEMMs), as the reference does for sequences longer than one token"}}


def run_llama_skip(args):
    """`--workload C2-e2e`: the Llama-3.2-3B-shaped LlamaSkip host end to end (random-init weights,
    512 random prompt ids, 128 greedy tokens): TTFT and output tokens/s as the reference's benchmark
    defines them."""
    import torch

    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    r = llama_skip_measure(args, torch.device("cuda", 0))
    print(json.dumps({
        "metric": "llamaskip_output_tokens_per_s", "value": r["output_tokens_per_s"], "unit": UNIT, "n_gpus": 1,
        "higher_is_better": True, "dtype": "f16", "data": "synthetic", "ttft_s": r["ttft_s"],
        "total_tokens_per_s": r["total_tokens_per_s"], "active_fraction_last_token": r["active_fraction_last_token"],
        "value_lazy_cache_rows": r["output_tokens_per_s_lazy_cache_rows"], "vs_baseline": None, "config": r["config"]}), flush=True)


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
