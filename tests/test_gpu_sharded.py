"""Intermediate-dimension sharding on real GPUs (NCCL): sharded layers + all-reduce equal the
single-GPU layer; per-shard masks and cache orders equal the single-GPU ones restricted to
the shard.  Needs at least two GPUs (skipped otherwise)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.sharded import ShardedLayer, ShardedStack, shard_range, shard_weights
    from sparse_transformers_b200.synth import HiddenStream, Workload, layer_weights

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    w = Workload("shard", H=1024, I=4096, r=32, B=4, dtype=torch.bfloat16, density=0.2, alpha=0.5, layers=2)
    gen = torch.Generator().manual_seed(0)
    ws = [layer_weights(w, gen) for _ in range(w.layers)]
    xs = HiddenStream(w, gen).take(6)
    lo, hi = shard_range(w.I, rank, world)
    sharded = [ShardedLayer(*[t.contiguous().to(dev) for t in shard_weights(*lw, rank, world)], act=w.act, param=w.tau,
                            max_batch=w.B) for lw in ws]
    full = [SparseLayer(*[t.to(dev) for t in lw], act=w.act, param=w.tau, max_batch=w.B) for lw in ws] if rank == 0 else None
    stack = ShardedStack(sharded, w.B, xs[0].to(dev))
    ok = True
    out = torch.empty(w.layers, w.B, w.H, dtype=w.dtype, device=dev)
    # the stack's warm-up advanced the shard caches with xs[0] twice; do the same on the full layers
    if rank == 0:
        for l in full:
            l.step(xs[0].to(dev)); l.step(xs[0].to(dev))
    for t in range(1, 6):
        x = xs[t].to(dev)
        stack.step(x, out)
        torch.cuda.synchronize()
        masks = [l.local.mask().cpu() for l in sharded]
        orders = [l.local.active_indices() + lo for l in sharded]
        if rank == 0:
            for li, l in enumerate(full):
                ref = l.step(x)
                torch.cuda.synchronize()
                err = (out[li].float() - ref.float()).abs().max() / ref.float().abs().max()
                ok &= bool(err <= 2e-2)
                ok &= torch.equal(masks[li], l.mask().cpu()[lo:hi])
                mine = set(orders[li].tolist())
                ok &= mine == {i for i in l.active_indices().tolist() if lo <= i < hi}
    if rank == 0:
        with open(os.path.join(out_dir, "ok.txt"), "w") as fh:
            fh.write("1" if ok else "0")
    stack.close()
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)  # not destroy_process_group(): it blocked after collectives were captured in a graph


def test_two_gpu_sharded_stack_matches_single_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok.txt").read() == "1"
