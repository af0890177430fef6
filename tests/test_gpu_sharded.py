"""Intermediate-dimension sharding on real GPUs: sharded layers + all-reduce (through peer
memory inside the library's own kernels, or NCCL) equal the single-GPU layer; per-shard masks
and cache orders equal the single-GPU ones restricted to the shard.  The multi-GPU cases need
at least two GPUs (skipped otherwise); the bounded-wait case runs on one."""
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


def _rank_main(rank, world, port, out_dir, mode, batch):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from sparse_transformers_b200 import SparseLayer
    from sparse_transformers_b200.sharded import PeerExchange, ShardedLayer, ShardedStack, shard_range, shard_weights
    from sparse_transformers_b200.synth import HiddenStream, Workload, layer_weights

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    w = Workload("shard", H=1024, I=4096, r=32, B=batch, dtype=torch.bfloat16, density=0.2, alpha=0.5, layers=2)
    # "peer": room for every layer's sums side by side (single-row stacks then run the flow kernel, all layers
    # exchanged at once); "peer1": room for one layer (the layer-by-layer kernel exchanges layer after layer)
    peer = PeerExchange(w.B * w.H * (w.layers if mode == "peer" else 1)) if mode.startswith("peer") else None
    ok = True
    if peer is not None:  # the stand-alone collective first: every rank contributes rank + 1
        for dt in (torch.float32, torch.float16, torch.bfloat16):
            for n in (1, 777, w.B * w.H):
                v = (torch.arange(n, device=dev, dtype=torch.float32) % 13 + rank + 1).to(dt)
                want = sum((torch.arange(n, dtype=torch.float32) % 13 + q + 1) for q in range(world)).to(dt)
                peer.all_reduce(v)
                torch.cuda.synchronize()
                ok &= torch.equal(v.cpu(), want)
    gen = torch.Generator().manual_seed(0)
    ws = [layer_weights(w, gen) for _ in range(w.layers)]
    xs = HiddenStream(w, gen).take(6)
    lo, hi = shard_range(w.I, rank, world)
    sharded = [ShardedLayer(*[t.contiguous().to(dev) for t in shard_weights(*lw, rank, world)], act=w.act, param=w.tau,
                            max_batch=w.B, peer=peer) for lw in ws]
    assert sharded[0].local.single_row_fused(w.B)  # 1 row: k_mlp_b1, 2..8 rows: k_mlp_bn
    full = [SparseLayer(*[t.to(dev) for t in lw], act=w.act, param=w.tau, max_batch=w.B) for lw in ws] if rank == 0 else None
    stack = ShardedStack(sharded, w.B, xs[0].to(dev))
    why = []
    out = torch.empty(w.layers, w.B, w.H, dtype=w.dtype, device=dev)
    # the stack's warm-up steps (if it took any) advanced the shard caches with xs[0]; do the same on the full layers
    if rank == 0:
        for l in full:
            for _ in range(stack.warmup_steps):
                l.step(xs[0].to(dev))
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
                checks = {"output": bool(err <= 2e-2), "mask": torch.equal(masks[li], l.mask().cpu()[lo:hi]),
                          "cache order": set(orders[li].tolist()) == {i for i in l.active_indices().tolist() if lo <= i < hi}}
                for name, good in checks.items():
                    if not good:
                        why.append(f"step {t} layer {li}: {name} differs (rel err {float(err):.3g})")
                ok &= all(checks.values())
    if peer is not None:
        ok &= not peer.timed_out()
        # all ranks hold the same bits
        mine = out.float().cpu()
        both = [None] * world
        dist.all_gather_object(both, mine)
        ok &= all(torch.equal(both[0], b) for b in both)
    oks = [None] * world
    dist.all_gather_object(oks, ok)
    if rank == 0:
        with open(os.path.join(out_dir, "ok.txt"), "w") as fh:
            fh.write("1" if all(oks) else "0 " + "; ".join(why[:6]))
    stack.close()
    torch.cuda.synchronize()
    dist.barrier()
    if peer is not None:
        peer.close()
    os._exit(0)  # not destroy_process_group(): it blocked after collectives were captured in a graph


@pytest.mark.parametrize("mode,batch", [("nccl", 4), ("peer", 4), ("peer", 1), ("peer1", 1), ("nccl", 1)])
def test_two_gpu_sharded_stack_matches_single_gpu(tmp_path, mode, batch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, str(tmp_path), mode, batch), nprocs=2, join=True)
    assert open(tmp_path / "ok.txt").read() == "1"


def test_four_gpu_peer_allreduce(tmp_path):
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    port = _free_port()
    mp.spawn(_rank_main, args=(4, port, str(tmp_path), "peer", 1), nprocs=4, join=True)
    assert open(tmp_path / "ok.txt").read() == "1"


def test_peer_wait_is_bounded(monkeypatch):
    """A peer that never sends: the kernel gives up after its poll limit, reports the timeout
    through the status word and the context stays usable.  World of two with the other rank's
    buffer played by a second buffer on this GPU that nobody writes."""
    import ctypes

    from sparse_transformers_b200 import _capi as C

    monkeypatch.setenv("STX_PEER_WAIT_ITERS", "2000")
    a, b = ctypes.c_void_p(), ctypes.c_void_p()
    C.check(C.lib.stx_peer_create(ctypes.byref(a), 0, 2, 4096))
    C.check(C.lib.stx_peer_create(ctypes.byref(b), 1, 2, 4096))  # only its buffer is used
    try:
        pa, pb = ctypes.c_void_p(), ctypes.c_void_p()
        C.check(C.lib.stx_peer_local_buffer(a, ctypes.byref(pa)))
        C.check(C.lib.stx_peer_local_buffer(b, ctypes.byref(pb)))
        bufs = (ctypes.c_void_p * 2)(pa.value, pb.value)
        C.check(C.lib.stx_peer_connect_ptrs(a, bufs))
        v = torch.ones(1000, device="cuda")
        st = ctypes.c_int()
        s = torch.cuda.current_stream().cuda_stream
        C.check(C.lib.stx_peer_status(a, ctypes.byref(st), s))
        assert st.value == C.OK
        C.check(C.lib.stx_peer_allreduce(a, v.data_ptr(), v.numel(), C.F32, s))
        C.check(C.lib.stx_peer_status(a, ctypes.byref(st), s))
        assert st.value == C.ERR_TIMEOUT
        assert torch.equal(v.cpu(), torch.ones(1000))  # the own term only
        assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0  # context alive
    finally:
        C.lib.stx_peer_destroy(a)
        C.lib.stx_peer_destroy(b)
