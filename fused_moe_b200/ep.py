"""Expert parallelism: 256 experts sharded over 1/2/4/8 GPUs, one process per GPU.

The reference runs one rank's experts only (it consumes ``local_expert_offset``,
solution/python/kernel.py:591) and has no communication; this module adds the two
exchanges around it.  Per call, on every rank:

  1. route the rank's own tokens (all 256 experts), C ABI ``b200moe_route``;
  2. ``b200moe_ep_pack``: one send row per (token, destination rank that owns one of its
     experts) - e4m3 payload, 1x128 scales, the 8 (id, weight) pairs - stable by token;
  3. exchange the per-destination row counts (tiny all-to-all, one host read);
  4. dispatch: NCCL all-to-all (uneven splits) of the rows into this GPU's own memory;
  5. the local expert pipeline over the received rows (``b200moe_count`` +
     ``b200moe_experts``), which reads payload/scales/ids in place through strides;
  6. combine: NCCL all-to-all of the bf16 partial rows back to their sources;
  7. ``b200moe_ep_combine``: fp32 sum of a token's <= min(4, world) partial rows -> bf16.

No kernel reads another GPU's memory; NVLink traffic is NCCL's.  The exchange logic is
independent of the device: tests drive it over ``gloo`` with CPU stand-ins for the five
device operations (``ops``), the product always uses ``CudaOps``.
"""
from __future__ import annotations

from typing import List, Optional

import os

import torch
import torch.distributed as dist

from . import _capi
from . import kernel as _k

E_GLOBAL = 256
TOP_K = 8
BLOCK = 128


def send_row_bytes(hidden: int) -> int:
    return hidden + 4 * (hidden // BLOCK) + 64


class CudaOps:
    """The five device operations of an EP step, on the C ABI."""

    def route(self, logits, bias, rsf, local_off, e_local, hidden, inter):
        return _k.route(logits, bias, rsf, local_off, e_local, hidden, inter)

    def pack(self, ids, w, hidden_states, hidden_scale, world):
        dev = ids.device
        T, hidden = hidden_states.shape
        hs = _k._as_bytes(hidden_states, "hidden_states")
        if hs.stride(1) != 1 or hs.stride(0) % 16 != 0:
            hs = hs.contiguous()
        st_t, st_kb = _k._scale_strides(hidden_scale, T, hidden // BLOCK)
        rb = send_row_bytes(hidden)
        send_rows = torch.empty((min(4, world) * max(T, 1), rb), dtype=torch.uint8, device=dev)
        dest_counts = torch.empty((world,), dtype=torch.int32, device=dev)
        send_slot = torch.empty((max(T, 1), world), dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            rc = _capi.lib().b200moe_ep_pack(
                ids.data_ptr(), w.data_ptr(), hs.data_ptr(), hs.stride(0), hidden_scale.data_ptr(),
                st_t, st_kb, T, hidden, world, send_rows.data_ptr(), dest_counts.data_ptr(),
                send_slot.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        _capi.check(rc, "b200moe_ep_pack")
        return send_rows, dest_counts, send_slot

    def experts(self, recv_rows, n_rows, w1, s1, w2, s2, local_off, hidden, inter):
        """Local expert pipeline over received send rows -> bf16 [n_rows, hidden]."""
        dev = recv_rows.device
        e_local = w1.shape[0]
        out = torch.empty((max(n_rows, 1), hidden), dtype=torch.bfloat16, device=dev)
        if n_rows == 0:
            return out[:0]
        rb = recv_rows.shape[1]
        base = recv_rows.data_ptr()
        kb = hidden // BLOCK
        w1b, w2b = _k._as_bytes(w1, "gemm1_weights"), _k._as_bytes(w2, "gemm2_weights")
        with torch.cuda.device(dev):
            ws = _k.get_workspace(dev, n_rows, e_local, hidden, inter)
            ws.last_T = n_rows
            stream = torch.cuda.current_stream(dev).cuda_stream
            ids_ptr = base + hidden + 4 * kb
            rc = _capi.lib().b200moe_count(ids_ptr, rb // 4, n_rows, local_off, e_local, hidden, inter,
                                           ws.ptr, ws.nbytes, stream)
            _capi.check(rc, "b200moe_count")
            rc = _capi.lib().b200moe_experts(
                ids_ptr, rb // 4, ids_ptr + 32, rb // 4, base, rb, base + hidden, rb // 4, 1,
                w1b.data_ptr(), s1.data_ptr(), w2b.data_ptr(), s2.data_ptr(),
                n_rows, e_local, local_off, hidden, inter, ws.ptr, ws.nbytes,
                out.data_ptr(), out.stride(0), stream)
            _capi.check(rc, "b200moe_experts")
        return out[:n_rows]

    def combine(self, returned, send_slot, dest_counts, T, hidden, world):
        dev = returned.device
        out = torch.empty((max(T, 1), hidden), dtype=torch.bfloat16, device=dev)
        with torch.cuda.device(dev):
            rc = _capi.lib().b200moe_ep_combine(returned.data_ptr(), send_slot.data_ptr(), dest_counts.data_ptr(),
                                                T, hidden, world, out.data_ptr(),
                                                torch.cuda.current_stream(dev).cuda_stream)
        _capi.check(rc, "b200moe_ep_combine")
        return out[:T]

    def empty(self, shape, dtype, device):
        return torch.empty(shape, dtype=dtype, device=device)


class ExpertParallelMoE:
    """One MoE layer whose experts are sharded over the ranks of ``group``.

    Rank r owns experts [r*256/world, (r+1)*256/world); ``w1, s1, w2, s2`` passed to
    ``forward`` are that slice.  Every rank brings its own tokens and gets back the full
    layer output for them.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, ops=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world not in (1, 2, 4, 8):
            raise ValueError("expert parallelism supports 1, 2, 4 or 8 ranks")
        self.e_local = E_GLOBAL // self.world
        self.local_off = self.rank * self.e_local
        self.ops = ops if ops is not None else CudaOps()
        self.last_recv_rows = 0
        self.last_send_counts: List[int] = []
        # B200MOE_EP_TRACE=1: CUDA events at the phase boundaries of every forward; phase_ms() reads them
        self._trace = bool(os.environ.get("B200MOE_EP_TRACE")) and isinstance(self.ops, CudaOps)
        self._marks: list = []

    def _mark(self, name: str):
        if self._trace:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def phase_ms(self) -> dict:
        """Milliseconds between the phase marks of the last forward (synchronises the device)."""
        if not self._marks:
            return {}
        torch.cuda.synchronize()
        return {b[0]: a[1].elapsed_time(b[1]) for a, b in zip(self._marks[:-1], self._marks[1:])}

    def forward(self, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                w1, s1, w2, s2, routed_scaling_factor: float) -> torch.Tensor:
        world, ops = self.world, self.ops
        T, hidden = hidden_states.shape
        inter = w2.shape[2]
        if w1.shape[0] != self.e_local:
            raise ValueError(f"rank holds {w1.shape[0]} experts, expected {self.e_local}")
        if world == 1:
            self.last_recv_rows = T
            return _k.custom_kernel(routing_logits, routing_bias, hidden_states, hidden_states_scale,
                                    w1, s1, w2, s2, 0, routed_scaling_factor) \
                if isinstance(ops, CudaOps) else self._single(routing_logits, routing_bias, hidden_states,
                                                              hidden_states_scale, w1, s1, w2, s2,
                                                              routed_scaling_factor)
        dev = hidden_states.device
        self._marks = []
        self._mark("start")
        ids, w = ops.route(routing_logits, routing_bias, routed_scaling_factor, self.local_off,
                           self.e_local, hidden, inter)
        send_rows, dest_counts, send_slot = ops.pack(ids, w, hidden_states, hidden_states_scale, world)

        # counts: what I send to d  <->  what d will receive from me
        self._mark("route_pack")
        recv_counts = torch.empty_like(dest_counts)
        dist.all_to_all_single(recv_counts, dest_counts, group=self.group)
        both = torch.stack([dest_counts, recv_counts]).cpu().tolist()    # one host read for both
        self._mark("counts_exchange_and_host_read")
        send_n = [int(x) for x in both[0]]
        recv_n = [int(x) for x in both[1]]
        self.last_send_counts = send_n
        n_recv, n_send = sum(recv_n), sum(send_n)
        self.last_recv_rows = n_recv
        rb = send_rows.shape[1]

        # dispatch: compact per-destination segments out, per-source segments in
        recv_rows = ops.empty((max(n_recv, 1), rb), torch.uint8, dev)
        dist.all_to_all_single(recv_rows[:n_recv], send_rows[:n_send], output_split_sizes=recv_n,
                               input_split_sizes=send_n, group=self.group)

        self._mark("dispatch_all_to_all")
        # local experts over everything that arrived
        partial = ops.experts(recv_rows, n_recv, w1, s1, w2, s2, self.local_off, hidden, inter)

        self._mark("local_experts")
        # combine: the same exchange backwards, bf16 rows
        returned = ops.empty((max(n_send, 1), hidden), torch.bfloat16, dev)
        dist.all_to_all_single(returned[:n_send], partial[:n_recv], output_split_sizes=send_n,
                               input_split_sizes=recv_n, group=self.group)
        self._mark("return_all_to_all")
        out = ops.combine(returned, send_slot, dest_counts, T, hidden, world)
        self._mark("combine")
        return out

    def _single(self, logits, bias, hs, hsc, w1, s1, w2, s2, rsf):
        ids, w = self.ops.route(logits, bias, rsf, 0, self.e_local, hs.shape[1], w2.shape[2])
        send_rows, counts, slot = self.ops.pack(ids, w, hs, hsc, 1)
        n = int(counts.cpu()[0])
        partial = self.ops.experts(send_rows, n, w1, s1, w2, s2, 0, hs.shape[1], w2.shape[2])
        returned = self.ops.empty((max(hs.shape[0], 1), hs.shape[1]), torch.bfloat16, hs.device)
        returned[:n] = partial
        return self.ops.combine(returned, slot, counts, hs.shape[0], hs.shape[1], 1)
