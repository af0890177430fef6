"""Intermediate-dimension sharding on CPU ranks (gloo, world size 2 and 3): the host-side
logic of the multi-GPU path — shard ranges, per-shard predictor slice / mask / cache, and the
sum of the partial outputs — checked against the unsharded oracle.  The device kernels are
not involved; every rank evaluates its shard with the CPU oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, steps, out_dir):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle import oracle as orc
    from sparse_transformers_b200.sharded import shard_range, shard_weights
    from sparse_transformers_b200.synth import HiddenStream, Workload, layer_weights

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    w = Workload("dist", H=96, I=301, r=12, B=3, dtype=torch.float32, density=0.3, alpha=0.5)
    gen = torch.Generator().manual_seed(0)          # identical on every rank
    gate, up, down, A, Bm = layer_weights(w, gen)
    xs = HiddenStream(w, gen).take(steps)
    f = lambda t: t.float().numpy()

    g_s, u_s, d_s, A_s, Bm_s = shard_weights(gate, up, down, A, Bm, rank, world)
    lo, hi = shard_range(w.I, rank, world)
    I_s = hi - lo
    cache = orc.OracleCache(I_s)
    cache.update(np.ones(I_s, bool))
    full = orc.OracleCache(w.I) if rank == 0 else None
    if full is not None:
        full.update(np.ones(w.I, bool))
    worst = 0.0
    for t in range(steps):
        x = xs[t]
        _, s = orc.predictor(f(x), f(A_s), f(Bm_s), orc.F32)   # the shard's slice of the scores
        _, mask = orc.mask_threshold(s, orc.F32, w.tau)
        cache.update(mask)
        wcat = np.concatenate([cache.gather(f(g_s)), cache.gather(f(u_s))])
        part, _ = orc.sparse_mlp(f(x), wcat, cache.gather(np.ascontiguousarray(f(d_s).T)), w.act, True)
        total = torch.from_numpy(part.copy())
        dist.all_reduce(total, op=dist.ReduceOp.SUM)           # the one exchange step of the path
        masks = [torch.zeros(0, dtype=torch.bool)] * world
        gathered = [None] * world
        dist.all_gather_object(gathered, (lo, mask.tolist(), (cache.active + lo).tolist()))
        if rank == 0:
            _, s_full = orc.predictor(f(x), f(A), f(Bm), orc.F32)
            _, m_full = orc.mask_threshold(s_full, orc.F32, w.tau)
            full.update(m_full)
            cat_mask = np.concatenate([np.array(g[1], bool) for g in sorted(gathered)])
            assert np.array_equal(cat_mask, m_full), "shard masks must tile the full mask"
            assert sorted(sum((g[2] for g in gathered), [])) == sorted(full.active.tolist())
            wc = np.concatenate([full.gather(f(gate)), full.gather(f(up))])
            ref, _ = orc.sparse_mlp(f(x), wc, full.gather(np.ascontiguousarray(f(down).T)), w.act, True)
            worst = max(worst, float(np.abs(total.numpy() - ref).max() / np.abs(ref).max()))
    if rank == 0:
        with open(os.path.join(out_dir, "result.txt"), "w") as fh:
            fh.write(f"{worst}\n")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_path_on_gloo_ranks(world, tmp_path):
    port = _free_port()
    mp.spawn(_rank_main, args=(world, port, 6, str(tmp_path)), nprocs=world, join=True)
    worst = float(open(tmp_path / "result.txt").read())
    assert worst <= 1e-5, worst


def test_shard_ranges_tile_the_index_space():
    from sparse_transformers_b200.sharded import shard_range

    for I in (1, 7, 8192, 14336, 14337):
        for world in (1, 2, 3, 4, 8):
            edges = [shard_range(I, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == I
            assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1
