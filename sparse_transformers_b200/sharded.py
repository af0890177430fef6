"""Intermediate-dimension sharding of the sparse MLP over the GPUs of one node.

Neurons are independent until the down projection sums over them, so rank g owns the
contiguous neuron range shard_range(I, g, G): the matching rows of gate / up / the
predictor's up matrix and the matching columns of down.  The predictor's down matrix A and
the hidden states are replicated.  Every rank runs its own predictor slice, mask and
differential weight cache (identical to a single-GPU cache built on the sliced weights) and
produces a partial [B,H]; one all-reduce(sum) per layer per step combines them.  Two ways:

  peer  (PeerExchange) the step's own last kernel pushes its fp32 sums into the other GPUs'
        memory over NVLink and adds what they pushed, in rank order: no extra launch for a
        single row, one small kernel otherwise; results are bit-identical on all ranks
  nccl  torch.distributed.all_reduce on the layer's output (model dtype)

The per-row rules that need whole-row statistics (topk, statistical_topk) are not
shard-local; sharded layers use the explicit-threshold rule.
"""
from __future__ import annotations

from typing import Sequence

import ctypes

import torch
import torch.distributed as dist

from . import _capi as C
from .layer import SparseLayer


def shard_range(I: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced split; the first I % world shards get one extra neuron."""
    base, rem = divmod(I, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_weights(gate, up, down, A, Bm, rank: int, world: int):
    """Slices of full-size weights owned by `rank` (views; call .contiguous() before upload)."""
    lo, hi = shard_range(up.shape[0], rank, world)
    return (gate[lo:hi] if gate is not None else None), up[lo:hi], down[:, lo:hi], A, Bm[lo:hi]


_DTYPE = {torch.float32: C.F32, torch.float16: C.F16, torch.bfloat16: C.BF16}


class PeerExchange:
    """This rank's exchange buffer for sums over the process group's GPUs (one node, one process
    per GPU, current CUDA device).  Construction is collective: the ranks swap the buffers'
    interprocess handles through torch.distributed and map each other's memory.

    max_elems: the largest sum that will go through the buffer, in elements ([B, H] of a layer: B * H).  A stack
    of L layers stepped with one row exchanges the sums of all its layers side by side, once per token, when the
    buffer has room for them (L * H elements); with less it exchanges layer after layer."""

    def __init__(self, max_elems: int, group=None):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        p = ctypes.c_void_p()
        C.check(C.lib.stx_peer_create(ctypes.byref(p), self.rank, self.world, int(max_elems)))
        self.handle = p
        if self.world > 1:
            h = ctypes.create_string_buffer(C.PEER_HANDLE_BYTES)
            C.check(C.lib.stx_peer_ipc_handle(p, h))
            handles: list = [None] * self.world
            dist.all_gather_object(handles, bytes(h.raw), group=group)
            blob = ctypes.create_string_buffer(b"".join(handles), C.PEER_HANDLE_BYTES * self.world)
            C.check(C.lib.stx_peer_connect_ipc(p, blob))
            dist.barrier(group)  # nobody pushes before everybody has mapped

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """In-place sum of `t` (contiguous CUDA tensor) over the ranks, on the current stream."""
        C.check(C.lib.stx_peer_allreduce(self.handle, t.data_ptr(), t.numel(), _DTYPE[t.dtype],
                                         torch.cuda.current_stream().cuda_stream))
        return t

    def timed_out(self) -> bool:
        """True when some wait for a peer gave up since creation (synchronises the stream)."""
        st = ctypes.c_int()
        C.check(C.lib.stx_peer_status(self.handle, ctypes.byref(st), torch.cuda.current_stream().cuda_stream))
        return st.value != C.OK

    def close(self) -> None:
        """Collective: every rank must be done stepping before anybody unmaps."""
        if self.handle is not None:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(self.group)
            C.lib.stx_peer_destroy(self.handle)
            self.handle = None


class ShardedLayer:
    """SparseLayer on this rank's shard plus the all-reduce of the partial sums (peer: a
    PeerExchange shared by the layers of this rank; None: NCCL)."""

    def __init__(self, gate, up, down, lora_down, lora_up, *, group=None, peer: PeerExchange | None = None, **kw):
        if kw.get("method", "threshold") not in ("threshold", "naive"):
            raise ValueError("sharded layers support the explicit-threshold rule only")
        self.group = group
        self.peer = peer
        self.local = SparseLayer(gate, up, down, lora_down, lora_up, **kw)
        if peer is not None:
            self.local.set_peer(peer)

    def step(self, x_pred, x_mlp=None, out=None):
        out = self.local.step(x_pred, x_mlp, out)
        if self.peer is None:
            dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def close(self):
        self.local.close()


class ShardedStack:
    """L sharded layers fed the same x [B,H]; the whole step (kernels + L all-reduces) is
    captured once in a CUDA graph on this rank and replayed.  out: [L,B,H].
    ``warmup_steps``: eager steps with ``warmup_x`` taken at construction (they advance the caches)."""

    def __init__(self, layers: Sequence[ShardedLayer], batch: int, warmup_x: torch.Tensor):
        self.layers = list(layers)
        l0 = self.layers[0].local
        self.B, self.L, self.H, self.dtype, self.device = int(batch), len(layers), l0.H, l0.dtype, l0.device
        # A single row with the sum over peer memory: the library's own stack object runs the shard as ONE
        # persistent kernel per step, the all-reduce of a layer inside it (stx_stack_create).  No warm-up
        # steps are taken then.
        self._native = None
        self.warmup_steps = 0
        if self.B == 1 and all(l.peer is not None and l.peer is self.layers[0].peer for l in self.layers):
            from .layer import SparseStack

            st = SparseStack([l.local for l in self.layers], 1)
            if st.launches_per_step <= 2 + 2 * self.L:  # one persistent kernel + plan and copy per layer + status collector
                self._native = st
                self.launches_per_step = st.launches_per_step
                return
            st.close()
        self.warmup_steps = 2
        self.x_in = torch.zeros(self.B, self.H, dtype=self.dtype, device=self.device)
        self.out = torch.zeros(self.L, self.B, self.H, dtype=self.dtype, device=self.device)
        # kernels of this library per layer (single row: t, fused MLP, partial sum, plan, copy;
        # else: t, scores, gate/up, down, plan, copy) + 1 NCCL kernel
        # (with a PeerExchange the sum rides in the partial-sum kernel of the single-row path)
        fused, peer = l0.single_row_fused(self.B), self.layers[0].peer is not None
        self.launches_per_step = ((5 if fused else 6) + (0 if fused and peer else 1)) * self.L
        self._side = torch.cuda.Stream(device=self.device)    # index plans
        self._side2 = torch.cuda.Stream(device=self.device)   # row copies (so the next layer's plan does not queue behind them)
        # Construction is collective: the ranks meet here, because the steps below wait (bounded, seconds)
        # for the peers' partial sums and the ranks may have built their shards at very different speeds.
        if dist.is_initialized() and dist.get_world_size(self.layers[0].group) > 1:
            torch.cuda.synchronize()
            dist.barrier(self.layers[0].group)
        # eager warm-up on a side stream (NCCL communicators, function attributes), then capture
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.x_in.copy_(warmup_x)
            for _ in range(2):
                self._eager()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._eager()

    def close(self) -> None:
        """Release the captured graph (it holds NCCL work).  Call before tearing down the process
        group: destroying a process group whose collectives live in a CUDA graph blocked here."""
        if getattr(self, "_native", None) is not None:
            torch.cuda.synchronize()
            self._native.close()
            self._native = None
        if getattr(self, "graph", None) is not None:
            torch.cuda.synchronize()
            self.graph.reset()
            self.graph = None

    def _eager(self):
        # critical path on the current stream: predictor -> sparse MLP -> all-reduce, layer after
        # layer; each layer's cache maintenance (index plan + row copies) forks onto a side stream
        # after its predictor and joins at the end of the step
        main = torch.cuda.current_stream()
        side = self._side
        for i, l in enumerate(self.layers):
            if l.local.single_row_fused(self.B):
                # the mask is made inside the MLP kernel: one call, the side work follows it
                l.local.step_stages(C.STAGE_PREDICT | C.STAGE_MLP, self.x_in, self.x_in, self.out[i], batch=self.B)
                side.wait_stream(main)
            else:
                l.local.step_stages(C.STAGE_PREDICT, self.x_in, batch=self.B)
                side.wait_stream(main)  # the side work needs the mask, nothing later
                l.local.step_stages(C.STAGE_MLP, None, self.x_in, self.out[i], batch=self.B)
            # (row blocks of 9 and more keep their cache upkeep inside STAGE_MLP on the main stream;
            # for them the two calls below enqueue nothing)
            with torch.cuda.stream(side):
                l.local.step_stages(C.STAGE_PLAN, batch=self.B)
            self._side2.wait_stream(side)
            with torch.cuda.stream(self._side2):
                l.local.step_stages(C.STAGE_COPY, batch=self.B)
            if l.peer is None:
                dist.all_reduce(self.out[i], op=dist.ReduceOp.SUM, group=l.group)
        main.wait_stream(side)
        main.wait_stream(self._side2)

    def step(self, x: torch.Tensor | None = None, out: torch.Tensor | None = None) -> None:
        if self._native is not None:
            return self._native.step(x, out)
        if x is not None:
            self.x_in.copy_(x, non_blocking=True)
        self.graph.replay()
        if out is not None:
            out.copy_(self.out, non_blocking=True)

    def step_host(self, x_host: torch.Tensor, out_host: torch.Tensor) -> None:
        if self._native is not None:
            return self._native.step_host(x_host, out_host)
        self.x_in.copy_(x_host, non_blocking=True)
        self.graph.replay()
        out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
