"""Expert-parallel exchange logic over gloo (2 CPU ranks): the dispatch/combine index math
of ExpertParallelMoE with numpy stand-ins for the device operations must reproduce the
single-rank oracle on each rank's tokens."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fused_moe_b200 import synth
from fused_moe_b200.ep import ExpertParallelMoE, send_row_bytes
from oracle import moe_oracle as O


class OracleOps:
    """CPU restatement of b200moe_route / ep_pack / experts / ep_combine (test double)."""

    def route(self, logits, bias, rsf, local_off, e_local, hidden, inter):
        ids, w, _, _ = O.route(logits.float().numpy(), bias.float().numpy(), rsf)
        return torch.from_numpy(ids), torch.from_numpy(w)

    def pack(self, ids, w, hidden_states, hidden_scale, world):
        T, hidden = hidden_states.shape
        kb = hidden // 128
        rb = send_row_bytes(hidden)
        cap = max(T, 1)
        slot = -np.ones((cap, world), dtype=np.int32)
        counts = np.zeros(world, dtype=np.int32)
        hs = hidden_states.view(torch.uint8).numpy()
        sc = O.hidden_scale_rows(hidden_scale.numpy(), T, kb)
        idn, wn = ids.numpy(), w.numpy()
        per = 256 // world
        segs = [[] for _ in range(world)]
        for t in range(T):
            for d in sorted(set(int(i) // per for i in idn[t])):
                row = np.zeros(rb, dtype=np.uint8)
                row[:hidden] = hs[t]
                row[hidden:hidden + 4 * kb] = np.ascontiguousarray(sc[t]).view(np.uint8)
                row[hidden + 4 * kb:hidden + 4 * kb + 32] = idn[t].astype(np.int32).view(np.uint8)
                row[hidden + 4 * kb + 32:] = wn[t].astype(np.float32).view(np.uint8)
                slot[t, d] = counts[d]
                counts[d] += 1
                segs[d].append(row)
        flat = [r for seg in segs for r in seg]
        rows = np.stack(flat) if flat else np.zeros((1, rb), dtype=np.uint8)
        return torch.from_numpy(rows), torch.from_numpy(counts), torch.from_numpy(slot)

    def experts(self, recv_rows, n_rows, w1, s1, w2, s2, local_off, hidden, inter):
        kb = hidden // 128
        r = recv_rows.numpy()[:n_rows]
        hs = np.ascontiguousarray(r[:, :hidden])
        sc = np.ascontiguousarray(r[:, hidden:hidden + 4 * kb]).view(np.float32)
        ids = np.ascontiguousarray(r[:, hidden + 4 * kb:hidden + 4 * kb + 32]).view(np.int32)
        w = np.ascontiguousarray(r[:, hidden + 4 * kb + 32:]).view(np.float32)
        u8 = lambda t: t.contiguous().view(torch.uint8).numpy()
        bits = O.experts_and_combine(ids, w, hs, sc.reshape(n_rows, kb), u8(w1), s1.numpy(), u8(w2), s2.numpy(),
                                     local_off)
        return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)

    def combine(self, returned, send_slot, dest_counts, T, hidden, world):
        ret = returned.float().numpy()
        slot = send_slot.numpy()
        base = np.concatenate([[0], np.cumsum(dest_counts.numpy())])
        out = np.zeros((T, hidden), dtype=np.float32)
        for t in range(T):
            for d in range(world):
                if slot[t, d] >= 0:
                    out[t] += ret[base[d] + slot[t, d]]
        return torch.from_numpy(O.to_bf16_bits(out).view(np.int16).copy()).view(torch.bfloat16)

    def empty(self, shape, dtype, device):
        return torch.zeros(shape, dtype=dtype, device=device)


HIDDEN, INTER, SEED = 512, 128, 4


def _worker(rank, world, port, tokens, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(2)
        per = 256 // world
        w1, s1, w2, s2 = synth.make_weights(per, rank * per, SEED, HIDDEN, INTER)
        logits, hq, hsc = synth.make_tokens(tokens[rank], rank, SEED, HIDDEN)
        bias = synth.make_bias(SEED)
        ep = ExpertParallelMoE(ops=OracleOps())
        out = ep.forward(logits, bias, hq, hsc, w1, s1, w2, s2, 2.5)
        ret[rank] = (out.view(torch.int16).numpy().copy(), ep.last_recv_rows, list(ep.last_send_counts))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("tokens", [(37, 21), (5, 0)])
def test_two_rank_exchange_matches_single_rank_oracle(tokens):
    world = 2
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), tokens, ret), nprocs=world, join=True)
    all_w = synth.make_weights(256, 0, SEED, HIDDEN, INTER)
    bias = synth.make_bias(SEED)
    total_sent = 0
    for r in range(world):
        out_bits, n_recv, sent = ret[r]
        total_sent += sum(sent)
        T = tokens[r]
        logits, hq, hsc = synth.make_tokens(T, r, SEED, HIDDEN)
        ref = O.moe_layer_torch(logits, bias, hq, hsc, *all_w, 0, 2.5)
        got = torch.from_numpy(out_bits).view(torch.bfloat16)
        assert got.shape == (T, HIDDEN)
        if T == 0:
            continue
        # each token goes to at most min(4, world) ranks, and to every rank that owns one of its experts
        ranks_needed = sum(len(set(int(i) // 128 for i in row)) for row in ref["ids"])
        assert sum(sent) == ranks_needed
        # partial sums are rounded to bf16 per rank before the final fp32 sum: tolerance of the layer
        frac_all, frac_nz, max_abs = synth.check_close(got, ref["out"])
        assert frac_all >= 0.999, (frac_all, max_abs)
        assert max_abs < 0.13
    assert sum(ret[r][1] for r in range(world)) == total_sent


def _misfit_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fused_moe_b200.ep import exchange_counts
        # rank 1's batch does not fit its buffers: it sends zero rows and the flag
        counts = torch.tensor([3, 4], dtype=torch.int32) if rank == 0 else torch.zeros(2, dtype=torch.int32)
        send_n, recv_n, recv_off, misfits = exchange_counts(counts, fits=(rank == 0))
        # a second exchange right behind it shows that no collective was left half-done
        again = exchange_counts(torch.tensor([1, 2], dtype=torch.int32), fits=True)
        ret[rank] = (send_n, recv_n, recv_off, misfits, again[3])
    finally:
        dist.destroy_process_group()


def test_batch_that_exceeds_one_ranks_buffers_is_seen_by_every_rank():
    world = 2
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_misfit_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        send_n, recv_n, recv_off, misfits, misfits_again = ret[r]
        assert misfits == [1], "every rank learns which rank is over its buffers, from the same exchange"
        assert misfits_again == []
    assert ret[0][0] == [3, 4] and ret[0][1] == [3, 0] and ret[1][1] == [4, 0] and ret[0][2] == [0, 0]


def _silent_rank_worker(rank, world, port, ret):
    """Rank 1 fails on the host before it posts its counts; rank 0 must not wait for ever."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    try:
        from fused_moe_b200.ep import exchange_counts
        if rank == 1:
            ret[rank] = "left before the exchange"
            return                      # a rank that raised or exited between steps: it never joins
        try:
            exchange_counts(torch.tensor([1, 1], dtype=torch.int32), fits=True)
            ret[rank] = "returned"
        except Exception as exc:        # gloo ends the collective with an error once the peer is gone / the limit ran out
            ret[rank] = "error: " + type(exc).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_that_never_posts_its_counts_ends_the_others_collective_with_an_error():
    world = 2
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_silent_rank_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert ret[1] == "left before the exchange"
    assert ret[0].startswith("error"), ret[0]
