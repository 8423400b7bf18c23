"""Expert parallelism on the GPU: the pack/combine kernels and the strided expert pipeline
(one GPU, ranks emulated by slicing on the host), and the real NCCL exchange on 2 GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

from fused_moe_b200 import kernel as K
from fused_moe_b200 import synth
from fused_moe_b200.ep import CudaOps, ExpertParallelMoE, send_row_bytes
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

HIDDEN, INTER, SEED = 1024, 256, 4


def _oracle_full(tokens, bias, all_w):
    logits, hq, hsc = tokens
    return O.moe_layer_torch(logits, bias, hq, hsc, *all_w, 0, 2.5)


@pytest.mark.parametrize("world,T", [(2, (70, 33)), (4, (40, 0, 129, 5)), (8, (9,) * 8)])
def test_pack_experts_combine_with_emulated_ranks(world, T):
    """All ranks' kernels run on cuda:0; the all-to-all is replaced by host-side slicing."""
    dev = torch.device("cuda", 0)
    ops = CudaOps()
    per = 256 // world
    all_w = synth.make_weights(256, 0, SEED, HIDDEN, INTER)
    bias = synth.make_bias(SEED)
    toks = [synth.make_tokens(T[r], r, SEED, HIDDEN) for r in range(world)]
    packed = []
    for r in range(world):
        lg, hq, hsc = (t.to(dev) for t in toks[r])
        ids, w = ops.route(lg, bias.to(dev), 2.5, r * per, per, HIDDEN, INTER)
        rows, counts, slot = ops.pack(ids, w, hq, hsc, world)
        torch.cuda.synchronize()
        packed.append((rows, counts.cpu().numpy(), slot, counts))
        ref_ids = O.route(toks[r][0].numpy(), bias.float().numpy(), 2.5)[0]
        need = np.zeros(world, dtype=np.int64)
        for row in ref_ids:
            for d in set(int(i) // per for i in row):
                need[d] += 1
        assert np.array_equal(packed[-1][1], need), "per-destination counts"
    rb = send_row_bytes(HIDDEN)
    returned = [torch.zeros((max(int(p[1].sum()), 1), HIDDEN), dtype=torch.bfloat16, device=dev) for p in packed]
    for d in range(world):
        segs, owners = [], []
        for s in range(world):
            base = int(packed[s][1][:d].sum())
            n = int(packed[s][1][d])
            segs.append(packed[s][0][base:base + n])
            owners.append((s, base, n))
        recv = torch.cat(segs) if sum(o[2] for o in owners) else torch.zeros((1, rb), dtype=torch.uint8, device=dev)
        n_recv = sum(o[2] for o in owners)
        wd = tuple(t[d * per:(d + 1) * per].to(dev) for t in all_w)
        partial = ops.experts(recv.contiguous(), n_recv, *wd, d * per, HIDDEN, INTER)
        torch.cuda.synchronize()
        off = 0
        for s, base, n in owners:
            returned[s][base:base + n] = partial[off:off + n]
            off += n
    for r in range(world):
        out = ops.combine(returned[r], packed[r][2], packed[r][3], T[r], HIDDEN, world)
        torch.cuda.synchronize()
        if T[r] == 0:
            assert out.shape == (0, HIDDEN)
            continue
        ref = _oracle_full(toks[r], bias, all_w)
        frac_all, frac_nz, max_abs = synth.check_close(out, ref["out"])
        assert frac_all >= 0.999, (world, r, frac_all, max_abs)


@pytest.mark.parametrize("world,T", [(2, (70, 33)), (4, (40, 0, 129, 5)), (8, (9,) * 8)])
def test_exchange_read_in_place_with_emulated_ranks(world, T):
    """The peer-memory entry points with every rank's buffers on cuda:0: ids pulled from the senders'
    buffers, the gather reading payload and scales there, and the combine reading the partial rows where
    each expert rank wrote them - no copy between the "ranks" at all."""
    import ctypes as C
    from fused_moe_b200 import _capi
    dev = torch.device("cuda", 0)
    ops, lib = CudaOps(), _capi.lib()
    per = 256 // world
    rb = send_row_bytes(HIDDEN)
    stream = torch.cuda.current_stream(dev).cuda_stream
    all_w = synth.make_weights(256, 0, SEED, HIDDEN, INTER)
    bias = synth.make_bias(SEED)
    toks = [synth.make_tokens(T[r], r, SEED, HIDDEN) for r in range(world)]
    packed = []
    for r in range(world):
        lg, hq, hsc = (t.to(dev) for t in toks[r])
        ids, w = ops.route(lg, bias.to(dev), 2.5, r * per, per, HIDDEN, INTER)
        rows, counts, slot = ops.pack(ids, w, hq, hsc, world)
        torch.cuda.synchronize()
        packed.append((rows, counts.cpu().numpy(), slot))
    partials, starts = [], []          # per expert rank d: its output rows; start of each source's segment in it
    cap_rows = world * max(max(T), 1)  # what the exchange's buffers could deliver to one rank
    for d in range(world):
        recv_n = [int(packed[s][1][d]) for s in range(world)]
        offs = [int(packed[s][1][:d].sum()) for s in range(world)]
        n_recv = sum(recv_n)
        starts.append([sum(recv_n[:s]) for s in range(world)])
        # the whole send buffers and, ON THE DEVICE, (count, first row) per source: what the ranks' small
        # all-to-all delivers; the library builds the segment table from it without a host read
        bases = (C.c_void_p * world)(*[packed[s][0].data_ptr() for s in range(world)])
        from_peers = torch.tensor([[recv_n[s], offs[s], 0] for s in range(world)], dtype=torch.int32, device=dev)
        partial = torch.zeros((cap_rows, HIDDEN), dtype=torch.bfloat16, device=dev)
        wd = tuple(t[d * per:(d + 1) * per].to(dev) for t in all_w)
        w1b, w2b = K._as_bytes(wd[0], "gemm1_weights"), K._as_bytes(wd[2], "gemm2_weights")
        ws = K.get_workspace(dev, cap_rows, per, HIDDEN, INTER)
        ws.last_T = cap_rows
        _capi.check(lib.b200moe_ep_local_experts(
            bases, from_peers.data_ptr(), world, cap_rows, rb, w1b.data_ptr(), wd[1].data_ptr(), w2b.data_ptr(),
            wd[3].data_ptr(), per, d * per, HIDDEN, INTER, ws.ptr, ws.nbytes, partial.data_ptr(), HIDDEN, stream),
            "ep_local_experts")
        torch.cuda.synchronize()
        assert ws.read_status(stream)[0] == 0
        if n_recv:
            # the pulled ids are the senders' routing results, row for row
            r_ids = ws.view("topk_ids", torch.int32, (cap_rows, 8))[:n_recv]
            sent = torch.cat([packed[s][0][offs[s]:offs[s] + recv_n[s]] for s in range(world) if recv_n[s]])
            trailer = HIDDEN + 4 * (HIDDEN // 128)
            assert torch.equal(r_ids.cpu(), sent[:, trailer:trailer + 32].contiguous().view(torch.int32).cpu())
        partials.append(partial)
    for r in range(world):
        if T[r] == 0:
            continue
        parts = (C.c_void_p * world)(*[p.data_ptr() for p in partials])
        row_start = torch.tensor([starts[d][r] for d in range(world)], dtype=torch.int32, device=dev)
        out = torch.empty((T[r], HIDDEN), dtype=torch.bfloat16, device=dev)
        _capi.check(lib.b200moe_ep_combine_peers(parts, row_start.data_ptr(), packed[r][2].data_ptr(), T[r], HIDDEN,
                                                 world, out.data_ptr(), stream), "combine_peers")
        torch.cuda.synchronize()
        ref = _oracle_full(toks[r], bias, all_w)
        frac_all, frac_nz, max_abs = synth.check_close(out, ref["out"])
        assert frac_all >= 0.999, (world, r, frac_all, max_abs)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _nccl_worker(rank, world, port, tokens, ret, p2p):
    import torch.distributed as dist
    os.environ["B200MOE_EP_P2P"] = p2p
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        per = 256 // world
        w = synth.make_weights(per, rank * per, SEED, HIDDEN, INTER, device=dev)
        lg, hq, hsc = (t.to(dev) for t in synth.make_tokens(tokens[rank], rank, SEED, HIDDEN))
        ep = ExpertParallelMoE()
        out = None
        for _ in range(2):          # twice: buffers and workspaces are reused
            out = ep.forward(lg, synth.make_bias(SEED).to(dev), hq, hsc, *w, 2.5)
        torch.cuda.synchronize()
        ret["mode%d" % rank] = ep.last_mode
        ret[rank] = out.cpu().view(torch.int16).numpy().copy()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _both_forms_worker(rank, world, port, tokens, ret):
    """Both exchange forms in one process group: the same partial rows summed in the same order.  A partial
    row itself is the sum of a token's bf16 expert rows in the order GEMM2's tiles finish, so two runs agree
    up to a few bf16 steps, not bit for bit."""
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        per = 256 // world
        w = synth.make_weights(per, rank * per, SEED, HIDDEN, INTER, device=dev)
        lg, hq, hsc = (t.to(dev) for t in synth.make_tokens(tokens[rank], rank, SEED, HIDDEN))
        bias = synth.make_bias(SEED).to(dev)
        outs, modes = [], []
        for p2p in ("1", "0"):
            os.environ["B200MOE_EP_P2P"] = p2p
            ep = ExpertParallelMoE()
            for _ in range(2):
                out = ep.forward(lg, bias, hq, hsc, *w, 2.5)
            torch.cuda.synchronize()
            outs.append(out.clone())
            modes.append(ep.last_mode)
            dist.barrier()
        a32, b32 = outs[0].float(), outs[1].float()
        if a32.numel():
            bound = 8 * 2.0 ** -8 * torch.clamp(torch.maximum(a32.abs().amax(dim=1, keepdim=True),
                                                             b32.abs().amax(dim=1, keepdim=True)), min=1.0)
            same = bool(((a32 - b32).abs() <= bound).all())
        else:
            same = True
        ret[rank] = (modes, same, outs[0].cpu().view(torch.int16).numpy().copy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_both_exchange_forms_agree_and_match_the_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    tokens = tuple([300, 77, 129, 0, 64, 5, 200, 31][:world])
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_both_forms_worker, args=(world, _free_port(), tokens, ret), nprocs=world, join=True)
    all_w = synth.make_weights(256, 0, SEED, HIDDEN, INTER)
    bias = synth.make_bias(SEED)
    for r in range(world):
        modes, same, bits = ret[r]
        assert modes[1] == "nccl" and modes[0] in ("peer", "nccl"), modes
        assert same, f"rank {r}: the two exchange forms differ"
        if tokens[r] == 0:
            continue
        ref = _oracle_full(synth.make_tokens(tokens[r], r, SEED, HIDDEN), bias, all_w)
        got = torch.from_numpy(bits).view(torch.bfloat16)
        frac_all, frac_nz, max_abs = synth.check_close(got, ref["out"])
        assert frac_all >= 0.999, (r, frac_all, max_abs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("p2p", ["1", "0"])
def test_nccl_exchange_on_two_gpus_matches_single_rank_oracle(p2p):
    """p2p=1: the bulk exchanges are loads from mapped peer memory inside the gather and combine kernels
    (falls back to NCCL where symmetric memory is unavailable); p2p=0: NCCL all-to-all."""
    import torch.multiprocessing as mp
    world, tokens = 2, (300, 77)
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_nccl_worker, args=(world, _free_port(), tokens, ret, p2p), nprocs=world, join=True)
    assert ret["mode0"] == ret["mode1"] and (p2p == "1" or ret["mode0"] == "nccl"), dict(ret).get("mode0")
    all_w = synth.make_weights(256, 0, SEED, HIDDEN, INTER)
    bias = synth.make_bias(SEED)
    for r in range(world):
        ref = _oracle_full(synth.make_tokens(tokens[r], r, SEED, HIDDEN), bias, all_w)
        got = torch.from_numpy(ret[r]).view(torch.bfloat16)
        frac_all, frac_nz, max_abs = synth.check_close(got, ref["out"])
        assert frac_all >= 0.999, (r, frac_all, max_abs)


def _overflow_worker(rank, world, port, ret):
    """Step 0 fits on both ranks; in step 1 rank 1 brings more tokens than the mapped buffers hold.  Rank 1 takes
    part in that step's collectives with nothing to send and raises after them; rank 0 completes the step (its
    own tokens only went to experts of both ranks as usual) and raises before the first collective of step 2.
    Nobody is left waiting in a collective, and no device wait is involved."""
    import torch.distributed as dist
    os.environ["B200MOE_EP_P2P"] = "1"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        per = 256 // world
        w = synth.make_weights(per, rank * per, SEED, HIDDEN, INTER, device=dev)
        bias = synth.make_bias(SEED).to(dev)
        small = tuple(t.to(dev) for t in synth.make_tokens(64, rank, SEED, HIDDEN))
        big = tuple(t.to(dev) for t in synth.make_tokens(200, rank, SEED, HIDDEN))
        ep = ExpertParallelMoE(max_tokens=128)
        events = []
        ep.forward(small[0], bias, small[1], small[2], *w, 2.5)
        events.append("step0 ok")
        if ep.last_mode != "peer":
            ret[rank] = ["no peer memory"]
            return
        try:
            batch = big if rank == 1 else small
            ep.forward(batch[0], bias, batch[1], batch[2], *w, 2.5)
            events.append("step1 ok")
        except ValueError as exc:
            events.append("step1 raised: " + str(exc)[:40])
        try:
            ep.forward(small[0], bias, small[1], small[2], *w, 2.5)
            events.append("step2 ok")
        except ValueError as exc:
            events.append("step2 raised: " + str(exc)[:40])
        torch.cuda.synchronize()
        ret[rank] = events
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_batch_over_the_mapped_buffers_raises_on_every_rank_without_a_hang():
    import torch.multiprocessing as mp
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_overflow_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    if ret[0] == ["no peer memory"]:
        pytest.skip("symmetric memory unavailable: the NCCL form has no capacity")
    assert ret[1][1].startswith("step1 raised") and ret[1][2].startswith("step2 raised"), ret[1]
    assert ret[0][1] == "step1 ok" and ret[0][2].startswith("step2 raised"), ret[0]
