"""KV-sequence sharded paged decode across GPUs: local split-KV decode, one all-gather of
(O, LSE), local merge.

The reference has no multi-GPU attention; it scales the KV length only inside one GPU with
split-KV plus a combine grid (``src/tileops/kernels/attention/gqa_decode_paged.py:176-395``).
This lifts the same algebra one level: rank ``r`` owns a range of every sequence's LOGICAL
pages in a local pool with a local block table and local lengths, runs the ordinary decode
kernel to a normalised fp32 partial ``O_r`` and a log2-domain ``LSE_r``, and the ranks
exchange ``B*H*(D+1)`` floats each (132 KB at B=8, H=32, D=128).  The merge
``O = sum_r 2^(LSE_r - LSE) O_r`` is associative, so intra-GPU and inter-GPU merges compose.

The decode kernel writes its partial straight into the send half of one communication
buffer; the all-gather lands every rank's partial in local memory and the merge kernel reads
only local memory (no kernel here ever loads from a peer).

``decode_fn`` / ``merge_fn`` default to the CUDA kernels; they are injectable so that the
protocol (packing, gather layout, empty shards) can be exercised by CPU ranks over gloo.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import functional as F


def shard_page_range(num_pages: int, rank: int, world: int) -> "tuple[int, int]":
    """Logical pages ``[begin, end)`` of a sequence with ``num_pages`` pages owned by ``rank``
    (contiguous, remainder spread over the first ranks)."""
    base, rem = divmod(num_pages, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class KVSequenceShardedPagedDecode:
    """Paged GQA decode whose KV cache is split by sequence position across a process group.

    ``forward(q, k_local, v_local, local_seqlen_kv, local_block_table)``: ``q`` is replicated;
    the other arguments describe only this rank's slice.  Every rank returns the full result.
    """

    def __init__(self, batch: int, heads: int, heads_kv: int, dim: int, page_size: int,
                 sm_scale: Optional[float] = None, softcap: Optional[float] = None,
                 group: Optional[dist.ProcessGroup] = None,
                 decode_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None) -> None:
        if heads % heads_kv != 0:
            raise ValueError("heads must be divisible by heads_kv")
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.page_size = page_size
        self.sm_scale = dim ** -0.5 if sm_scale is None else sm_scale
        self.softcap = 0.0 if softcap is None else softcap
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._decode = decode_fn or self._cuda_decode
        self._merge = merge_fn or self._cuda_merge
        self._buffers: dict = {}
        self._peer = None
        #: limit of the merge kernel's wait for the other ranks' flags, in GPU clock ticks (0: about 0.5 s)
        self.peer_wait_cycles = 0

    # default compute: the CUDA kernels
    def _cuda_decode(self, q, k, v, lens, bt, out, lse_out):
        F.gqa_decode(q, k, v, real_seqlen_kv=lens, block_table=bt, page_size=self.page_size,
                     sm_scale=self.sm_scale, softcap=self.softcap, out=out, lse_out=lse_out)

    @staticmethod
    def _cuda_merge(o_parts, lse_parts, out_dtype):
        return F.gqa_lse_merge(o_parts, lse_parts, out_dtype)

    def _comm_buffers(self, device: torch.device):
        bufs = self._buffers.get(device)
        if bufs is None:
            n = self.batch * self.heads * (self.dim + 1)
            send = torch.empty(n, dtype=torch.float32, device=device)
            recv = torch.empty(self.world * n, dtype=torch.float32, device=device)
            bufs = (send, recv)
            self._buffers[device] = bufs
        return bufs

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                local_seqlen_kv: torch.Tensor, local_block_table: torch.Tensor) -> torch.Tensor:
        B, H, D = self.batch, self.heads, self.dim
        if tuple(q.shape) != (B, H, D):
            raise ValueError(f"q must have shape {(B, H, D)}, got {tuple(q.shape)}")
        if getattr(self, "_peer", None) is not None:
            return self._forward_peer(q, k, v, local_seqlen_kv, local_block_table)
        send, recv = self._comm_buffers(q.device)
        n_o = B * H * D
        o_part = send[:n_o].view(B, H, D)
        lse_part = send[n_o:].view(B, H)
        self._decode(q, k, v, local_seqlen_kv, local_block_table, o_part, lse_part)
        if self.world == 1:
            return self._merge(o_part.unsqueeze(0), lse_part.unsqueeze(0), q.dtype)
        dist.all_gather_into_tensor(recv, send, group=self.group)
        parts = recv.view(self.world, B * H * (D + 1))
        o_parts = parts[:, :n_o].unflatten(1, (B, H, D))      # strided over ranks, each part contiguous
        lse_parts = parts[:, n_o:].unflatten(1, (B, H))
        return self._merge(o_parts, lse_parts, q.dtype)

    __call__ = forward

    # ---- fused exchange over peer memory ---------------------------------------------------
    def enable_peer_exchange(self, device: torch.device) -> None:
        """Switch the exchange from the NCCL all-gather to stores over NVLink issued by the decode kernel
        itself (``tb200_gqa_decode_sharded`` / ``tb200_gqa_lse_merge_wait``).  The exchange buffer is
        symmetric memory (``torch.distributed._symmetric_memory``): every rank maps every rank's buffer.
        Collective: all ranks call it.  Raises if symmetric memory is not available; the NCCL path is
        untouched in that case."""
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem
        if self.world < 2 or self.world > 8:
            raise RuntimeError("peer exchange serves 2..8 ranks")
        n = self.batch * self.heads * (self.dim + 1)
        flag_words = 64
        buf = symm_mem.empty(2 * self.world * n + flag_words, dtype=torch.float32, device=device)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        if len(ptrs) != self.world or ptrs[self.rank] != buf.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned unexpected buffer pointers")
        flags_off = 2 * self.world * n * 4
        self._peer = {
            "buf": buf, "hdl": hdl, "slot": n,
            "buffers": (ctypes.c_void_p * self.world)(*ptrs),
            "flags": (ctypes.c_void_p * self.world)(*[p + flags_off + self.rank * 4 for p in ptrs]),
            "own_flags": buf.data_ptr() + flags_off,
            "step": torch.zeros(1, dtype=torch.int32, device=device),
            "status": torch.zeros(1, dtype=torch.int32, device=device),
        }
        torch.cuda.synchronize(device)
        dist.barrier(group=group)      # every buffer is zeroed before any rank stores into it

    def peer_status(self, reset: bool = False) -> int:
        """0, or 501 if a merge gave up waiting for another rank's flag (synchronises).  The rows such a
        merge could not produce are NaN.  The word is sticky: every later merge gives up at once until it
        is cleared (``reset=True``), so a failed exchange cannot pass unnoticed."""
        if not getattr(self, "_peer", None):
            return 0
        code = int(self._peer["status"].item())
        if reset and code:
            self._peer["status"].zero_()
        return code

    def _forward_peer(self, q, k, v, lens, bt) -> torch.Tensor:
        import ctypes

        from . import _native as N
        B, H, D, P = self.batch, self.heads, self.dim, self._peer
        Hkv = k.shape[1]
        fp8 = k.dtype == getattr(torch, "float8_e4m3fn", None)
        if fp8:
            raise ValueError("the peer exchange path serves 16-bit caches")
        q, k, v, lens, bt = q.contiguous(), k.contiguous(), v.contiguous(), lens.contiguous(), bt.contiguous()
        ws = F._decode_workspace(q.device, B, H, Hkv, D)
        out = torch.empty((B, H, D), dtype=q.dtype, device=q.device)
        lib, stream = N.lib(), N.current_stream(q.device)
        with torch.cuda.device(q.device):
            st = lib.tb200_gqa_decode_sharded(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), lens.data_ptr(), 0, bt.data_ptr(), bt.shape[1], None, None,
                N.dtype_code(q.dtype), N.dtype_code(k.dtype), B, H, Hkv, D, self.page_size, k.stride(0), k.stride(1), 0,
                float(self.sm_scale), float(self.softcap), k.shape[0], 0, ctypes.addressof(P["buffers"]),
                ctypes.addressof(P["flags"]),
                P["step"].data_ptr(), self.world, self.rank, ws.data_ptr(), ws.numel(), stream)
            N.check(st, "tb200_gqa_decode_sharded")
            base = P["buf"].data_ptr()
            st = lib.tb200_gqa_lse_merge_wait(
                base, base + B * H * D * 4, out.data_ptr(), None, self.world, B * H, D, P["slot"], P["slot"],
                self.world * P["slot"], N.dtype_code(q.dtype), P["own_flags"], P["step"].data_ptr(),
                P["status"].data_ptr(), int(self.peer_wait_cycles), stream)
            N.check(st, "tb200_gqa_lse_merge_wait")
        return out

    def graphed(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, local_seqlen_kv: torch.Tensor,
                local_block_table: torch.Tensor, warmup: int = 3) -> Callable[[], torch.Tensor]:
        """Capture one ``forward`` on these tensors (decode launch, all-gather, merge launch) in a CUDA
        graph and return a callable that replays it and returns the (static) output tensor.  At 4+
        GPUs a long-context step is ~0.1 ms of GPU work, less than the host spends issuing the three
        calls from Python; the replay is one launch.  The tensors are read in place at every replay
        (update them in place between replays); every rank must capture and replay in step.  Drop the
        returned callable before the process group is destroyed: tearing down a communicator that a live
        graph still references blocks.
        """
        args = (q, k, v, local_seqlen_kv, local_block_table)
        side = torch.cuda.Stream(device=q.device)
        side.wait_stream(torch.cuda.current_stream(q.device))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                self.forward(*args)
        torch.cuda.current_stream(q.device).wait_stream(side)
        torch.cuda.synchronize(q.device)
        graph = torch.cuda.CUDAGraph()
        # captured on the stream of the warm-up: the decode workspace is kept per stream, and one that were
        # first asked for during the capture would put its zero fill into the graph (4 us at every replay)
        with torch.cuda.graph(graph, stream=side):
            out = self.forward(*args)

        def replay() -> torch.Tensor:
            graph.replay()
            return out
        replay.graph = graph          # keeps the graph (and its memory pool) alive with the callable
        return replay
