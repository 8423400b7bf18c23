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

With NCCL ranks on one node the two bulk exchanges are folded into the kernels instead
(``PeerExchange``): the send buffer and the partial-output buffer of every rank are
symmetric-memory allocations mapped into every process, steps 3-5 become "exchange (count,
offset) pairs, build the segment table ON THE DEVICE, pull the ids and let the gather read
payload and scales from the senders' buffers" (``b200moe_ep_local_experts``: the host never
reads a count, the workspace is sized for the exchange's capacity) and steps 6-7 become one
kernel that sums the partial rows where they were produced (``b200moe_ep_combine_peers``):
plain loads over NVLink, no multicast.  The two small NCCL all-to-alls that remain (row counts
and offsets before, segment starts after the experts) are also what orders the ranks' kernels.
``B200MOE_EP_P2P=0``, a ``gloo`` group or a failed mapping fall back to the NCCL path above.  Both forms sum the same partial rows in the
same order (tests/test_gpu_ep.py, 2, 4 and 8 GPUs).

The exchange logic is independent of the device: tests drive it over ``gloo`` with CPU
stand-ins for the five device operations (``ops``), the product always uses ``CudaOps``.
"""
from __future__ import annotations

from typing import List, Optional

import os

import torch
import torch.distributed as dist

from . import _capi
from . import kernel as _k

# The mapped exchange buffers are only ever read with plain loads; keep torch from binding them to
# an NVLink multicast object as well.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

E_GLOBAL = 256
TOP_K = 8
BLOCK = 128


def send_row_bytes(hidden: int) -> int:
    return hidden + 4 * (hidden // BLOCK) + 64


class CudaOps:
    """The five device operations of an EP step, on the C ABI."""

    def route(self, logits, bias, rsf, local_off, e_local, hidden, inter):
        return _k.route(logits, bias, rsf, local_off, e_local, hidden, inter)

    def pack(self, ids, w, hidden_states, hidden_scale, world, send_buffer=None):
        dev = ids.device
        T, hidden = hidden_states.shape
        hs = _k._as_bytes(hidden_states, "hidden_states")
        if hs.stride(1) != 1 or hs.stride(0) % 16 != 0:
            hs = hs.contiguous()
        st_t, st_kb = _k._scale_strides(hidden_scale, T, hidden // BLOCK)
        rb = send_row_bytes(hidden)
        cap = min(4, world) * max(T, 1)
        if send_buffer is not None and send_buffer.shape[0] >= cap and send_buffer.shape[1] == rb:
            send_rows = send_buffer          # a symmetric-memory buffer that the peers read in place
        else:
            send_rows = torch.empty((cap, rb), dtype=torch.uint8, device=dev)
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


def exchange_counts(dest_counts: torch.Tensor, fits: bool, group=None):
    """The small all-to-all that opens an exchange through mapped buffers: rank r tells every destination
    d how many rows it has for it, where they start in r's send buffer, and whether r's batch fitted its
    buffers at all.  Returns (rows sent per destination, rows received per source, start of each source's
    segment, ranks whose batch did not fit).  Every rank gets the same list of misfits from the same
    exchange, so they all raise (or all carry on) together and no rank is left waiting in a collective.
    Works on any backend (device tensors on NCCL, CPU tensors on gloo)."""
    world = dist.get_world_size(group)
    seg_off = torch.cumsum(dest_counts, 0, dtype=torch.int32) - dest_counts
    flag = torch.full_like(dest_counts, 0 if fits else 1)
    mine = torch.stack([dest_counts, seg_off, flag], dim=1).contiguous()    # [world, 3]
    theirs = torch.empty_like(mine)
    dist.all_to_all_single(theirs, mine, group=group)
    host = torch.cat([mine, theirs]).cpu().tolist()                         # one host read
    send_n = [int(r[0]) for r in host[:world]]
    recv_n = [int(r[0]) for r in host[world:]]
    recv_off = [int(r[1]) for r in host[world:]]
    misfits = [s for s in range(world) if int(host[world + s][2]) != 0]
    return send_n, recv_n, recv_off, misfits


class PeerExchange:
    """Symmetric-memory buffers of one rank and their addresses in every rank (NCCL, one node)."""

    def __init__(self, group, cap_tokens: int, hidden: int, world: int, dev):
        """``cap_tokens``: the largest token count of any rank (the same number on every rank:
        symmetric allocations have one size)."""
        import torch.distributed._symmetric_memory as symm
        rb = send_row_bytes(hidden)
        self.cap_tokens, self.hidden = cap_tokens, hidden
        self.send = symm.empty((min(4, world) * max(cap_tokens, 1), rb), dtype=torch.uint8, device=dev)
        # every rank may send all of its tokens here
        self.partial = symm.empty((world * max(cap_tokens, 1), hidden), dtype=torch.bfloat16, device=dev)
        grp = group if group is not None else dist.group.WORLD
        self.send_ptrs = [int(x) for x in symm.rendezvous(self.send, grp).buffer_ptrs]
        self.partial_ptrs = [int(x) for x in symm.rendezvous(self.partial, grp).buffer_ptrs]
        self.row_bytes = rb


class ExpertParallelMoE:
    """One MoE layer whose experts are sharded over the ranks of ``group``.

    Rank r owns experts [r*256/world, (r+1)*256/world); ``w1, s1, w2, s2`` passed to
    ``forward`` are that slice.  Every rank brings its own tokens and gets back the full
    layer output for them.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, ops=None, max_tokens: Optional[int] = None):
        """``max_tokens``: capacity (tokens per rank) of the mapped exchange buffers; by default the
        largest token count of any rank at the first call.  A later call with more tokens raises."""
        self.max_tokens = max_tokens
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world not in (1, 2, 4, 8):
            raise ValueError("expert parallelism supports 1, 2, 4 or 8 ranks")
        self.e_local = E_GLOBAL // self.world
        self.local_off = self.rank * self.e_local
        self.ops = ops if ops is not None else CudaOps()
        self._last_recv_rows = 0
        self.last_ws_rows = 0          # the token count the workspace of the last local expert pipeline was laid out for
        self.last_send_counts: List[int] = []
        self._exch_host = None         # pinned copy of what the last peer-memory step exchanged
        self._exch_event = None
        self._exch_pending = False
        self._misfit_dev = None
        # B200MOE_EP_TRACE=1: CUDA events at the phase boundaries of every forward; phase_ms() reads them
        self._trace = bool(os.environ.get("B200MOE_EP_TRACE")) and isinstance(self.ops, CudaOps)
        self._marks: list = []
        self._peer: Optional[PeerExchange] = None
        self._peer_failed = os.environ.get("B200MOE_EP_P2P", "1") == "0"
        self.last_mode = "single" if self.world == 1 else "nccl"

    def _peer_exchange(self, T: int, hidden: int, dev) -> Optional[PeerExchange]:
        """The mapped buffers for this problem size, or None when the NCCL path has to be used."""
        if self._peer_failed or not isinstance(self.ops, CudaOps) or dev.type != "cuda":
            return None
        if dist.get_backend(self.group) != "nccl":
            return None
        if self._peer is None:           # first call: every rank gets here together
            cap = self.max_tokens
            if cap is None:
                t_max = torch.tensor([T], dtype=torch.int32, device=dev)
                dist.all_reduce(t_max, op=dist.ReduceOp.MAX, group=self.group)
                cap = int(t_max.item())
            ok = torch.ones(1, dtype=torch.int32, device=dev)
            try:
                self._peer = PeerExchange(self.group, cap, hidden, self.world, dev)
            except Exception:            # no symmetric memory on this system: every rank must agree
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if int(ok.item()) == 0:
                self._peer, self._peer_failed = None, True
                return None
        # A batch that does not fit this rank's mapped buffers is NOT refused here: the other ranks could not
        # know and would block in the next collective.  _forward_peer sends a "fits" flag along with the row
        # counts; the rank itself sends nothing and raises after the step, the others at their next call.
        if hidden != self._peer.hidden:     # the same on every rank (the model's width): nobody enters a collective
            raise ValueError(f"hidden size {hidden} differs from the mapped exchange buffers' {self._peer.hidden}")
        return self._peer

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
            self.last_ws_rows = T
            return _k.custom_kernel(routing_logits, routing_bias, hidden_states, hidden_states_scale,
                                    w1, s1, w2, s2, 0, routed_scaling_factor) \
                if isinstance(ops, CudaOps) else self._single(routing_logits, routing_bias, hidden_states,
                                                              hidden_states_scale, w1, s1, w2, s2,
                                                              routed_scaling_factor)
        dev = hidden_states.device
        peer = self._peer_exchange(T, hidden, dev)
        if peer is not None:
            return self._forward_peer(peer, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                                      w1, s1, w2, s2, routed_scaling_factor)
        self.last_mode = "nccl"
        self._marks = []
        self._mark("start")
        ids, w = ops.route(routing_logits, routing_bias, routed_scaling_factor, self.local_off,
                           self.e_local, hidden, inter)
        send_rows, dest_counts, send_slot = ops.pack(ids, w, hidden_states, hidden_states_scale, world)

        # counts: what I send to d  <->  what d will receive from me
        self._mark("route_pack")
        send_n, recv_n, _, _ = exchange_counts(dest_counts, True, self.group)   # one host read (NCCL needs split sizes)
        self._mark("counts_exchange_and_host_read")
        self.last_send_counts = send_n
        n_recv, n_send = sum(recv_n), sum(send_n)
        self.last_recv_rows = n_recv
        self.last_ws_rows = n_recv
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

    def _forward_peer(self, peer: PeerExchange, routing_logits, routing_bias, hidden_states, hidden_states_scale,
                      w1, s1, w2, s2, rsf) -> torch.Tensor:
        """The step with both bulk exchanges folded into the kernels (see the module docstring).  Nothing
        is read back by the host inside the step: what the small all-to-all delivered is copied to pinned
        memory behind the step and looked at by ``check_exchange`` (start of the next call, or on demand)."""
        import ctypes as C
        world, ops = self.world, self.ops
        T, hidden = hidden_states.shape
        inter = w2.shape[2]
        dev = hidden_states.device
        lib = _capi.lib()
        self.last_mode = "peer"
        self._marks = []
        self._mark("start")
        fits = T <= peer.cap_tokens
        if fits:
            ids, w = ops.route(routing_logits, routing_bias, rsf, self.local_off, self.e_local, hidden, inter)
            send_rows, dest_counts, send_slot = ops.pack(ids, w, hidden_states, hidden_states_scale, world,
                                                         send_buffer=peer.send)
        else:   # nothing of this batch may touch the mapped buffers: this rank sends nothing and raises below,
            #     the others learn of it from the flag (they still get a complete, collective step)
            dest_counts = torch.zeros((world,), dtype=torch.int32, device=dev)
            send_slot = torch.full((max(T, 1), world), -1, dtype=torch.int32, device=dev)
        self._mark("route_pack")
        # Before the first collective of this step: did some rank overrun its buffers in the previous one (then
        # that rank has raised and may never come here)?  Every other rank raises at this point.  The wait is for
        # the previous step's small copy; this step's routing and packing are already queued behind it.
        self.check_exchange()
        # to every destination: how many rows it gets from me, where they start in my send buffer, and whether
        # my batch fitted.  This exchange completes only after every rank's pack kernel: it is also what makes
        # the send buffers safe to read.
        seg_off = torch.cumsum(dest_counts, 0, dtype=torch.int32) - dest_counts
        flag = torch.full_like(dest_counts, 0 if fits else 1)
        mine = torch.stack([dest_counts, seg_off, flag], dim=1).contiguous()    # [world, 3]
        theirs = torch.empty_like(mine)
        dist.all_to_all_single(theirs, mine, group=self.group)
        self._mark("counts_exchange")

        rb = peer.row_bytes
        cap_rows = world * peer.cap_tokens
        bases = (C.c_void_p * world)(*peer.send_ptrs)
        stream = torch.cuda.current_stream(dev).cuda_stream
        w1b, w2b = _k._as_bytes(w1, "gemm1_weights"), _k._as_bytes(w2, "gemm2_weights")
        with torch.cuda.device(dev):
            ws = _k.get_workspace(dev, cap_rows, self.e_local, hidden, inter)
            ws.last_T = cap_rows
            _capi.check(lib.b200moe_ep_local_experts(
                bases, theirs.data_ptr(), world, cap_rows, rb, w1b.data_ptr(), s1.data_ptr(), w2b.data_ptr(),
                s2.data_ptr(), self.e_local, self.local_off, hidden, inter, ws.ptr, ws.nbytes,
                peer.partial.data_ptr(), hidden, stream), "b200moe_ep_local_experts")
        self.last_ws_rows = cap_rows
        self._mark("local_experts_reading_peers")

        # to every source: where its segment starts in my partial buffer.  Enqueued after the expert
        # kernels, so its completion on a rank means that every rank's partial rows are written.
        recv = theirs[:, 0].contiguous()
        seg_start = (torch.cumsum(recv, 0, dtype=torch.int32) - recv).contiguous()
        row_start = torch.empty_like(seg_start)
        dist.all_to_all_single(row_start, seg_start, group=self.group)
        self._mark("segment_starts_exchange")
        out = torch.empty((max(T, 1), hidden), dtype=torch.bfloat16, device=dev)
        parts = (C.c_void_p * world)(*peer.partial_ptrs)
        with torch.cuda.device(dev):
            _capi.check(lib.b200moe_ep_combine_peers(parts, row_start.data_ptr(), send_slot.data_ptr(), T, hidden,
                                                     world, out.data_ptr(), stream), "b200moe_ep_combine_peers")
        self._mark("combine_reading_peers")
        # what was exchanged, for the host to look at AFTER the step (no wait here); the "did not fit" flags
        # accumulate on the device, so a step the host never looked at cannot hide one
        if self._exch_host is None or self._exch_host.shape[1] != world:
            self._exch_host = torch.zeros((3, world, 3), dtype=torch.int32).pin_memory()
            self._exch_event = torch.cuda.Event()
            self._misfit_dev = torch.zeros((world, 3), dtype=torch.int32, device=dev)
        self._misfit_dev[:, 0].bitwise_or_(theirs[:, 2])
        self._exch_host[0].copy_(mine, non_blocking=True)
        self._exch_host[1].copy_(theirs, non_blocking=True)
        self._exch_host[2].copy_(self._misfit_dev, non_blocking=True)
        self._exch_event.record(torch.cuda.current_stream(dev))
        self._exch_pending = True
        if not fits:
            raise ValueError(f"this rank's batch ({T} x {hidden}) exceeds the mapped exchange buffers "
                             f"({peer.cap_tokens} tokens of width {peer.hidden}); it sent nothing, the other ranks "
                             f"raise at their next call; pass max_tokens to ExpertParallelMoE")
        return out[:T]

    def check_exchange(self, block: bool = True):
        """Looks at what the last peer-memory step exchanged: updates ``last_send_counts`` /
        ``last_recv_rows`` and raises when some rank's batch had not fitted its mapped buffers in any step
        since the last look (every rank sees the same flags, one or more calls later).  ``block=False``
        looks only if that step's small copy has already landed, so the host keeps running ahead."""
        if not self._exch_pending:
            return
        if not block and not self._exch_event.query():
            return
        self._exch_event.synchronize()
        self._exch_pending = False
        mine, theirs, flags = (self._exch_host[i].tolist() for i in range(3))
        self.last_send_counts = [int(r[0]) for r in mine]
        self._last_recv_rows = sum(int(r[0]) for r in theirs)
        misfits = [s for s in range(self.world) if int(flags[s][0]) != 0]
        if misfits:
            self._misfit_dev.zero_()
            raise ValueError(f"rank(s) {misfits} held a batch that exceeds the mapped exchange buffers in an "
                             f"earlier step and sent nothing; pass max_tokens to ExpertParallelMoE")

    @property
    def last_recv_rows(self) -> int:
        self.check_exchange()
        return self._last_recv_rows

    @last_recv_rows.setter
    def last_recv_rows(self, v: int):
        self._last_recv_rows = int(v)

    def _single(self, logits, bias, hs, hsc, w1, s1, w2, s2, rsf):
        ids, w = self.ops.route(logits, bias, rsf, 0, self.e_local, hs.shape[1], w2.shape[2])
        send_rows, counts, slot = self.ops.pack(ids, w, hs, hsc, 1)
        n = int(counts.cpu()[0])
        partial = self.ops.experts(send_rows, n, w1, s1, w2, s2, 0, hs.shape[1], w2.shape[2])
        returned = self.ops.empty((max(hs.shape[0], 1), hs.shape[1]), torch.bfloat16, hs.device)
        returned[:n] = partial
        return self.ops.combine(returned, slot, counts, hs.shape[0], hs.shape[1], 1)
