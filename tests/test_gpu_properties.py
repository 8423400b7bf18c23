"""Size-independent properties of the layer at the benchmark's full sizes (32 local experts,
hidden 7168, intermediate 2048; up to 16384 tokens), where running the oracle on every token
would take minutes: repeatability, per-token independence, scaling, and a spot check of sampled
tokens against the oracle.

A token's output row is the sum of its (at most eight) expert rows, each rounded to bf16 and added
by GEMM2's epilogue with a bf16 `red.global.add` in whatever order the tiles finish - the reference's
`out[t] += bf16(G2 * w)` on a bf16 tensor, in a free order.  Everything before that sum is
order-deterministic, so two runs differ by the rounding of at most eight bf16 additions:
a few bf16 steps of the largest partial sum.  `_same_up_to_sum_order` asserts exactly that."""
import numpy as np
import pytest
import torch

from fused_moe_b200 import kernel as K
from fused_moe_b200 import synth
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

RSF = 2.5


def _tokens(T, tseed, dev):
    lg, hq, hsc = synth.make_tokens(T, 0, tseed)
    return lg.to(dev), hq.to(dev), hsc.to(dev)


def _run(lg, bias, hq, hsc, w, rsf=RSF):
    return K.custom_kernel(lg, bias, hq, hsc, *w, 0, rsf, check_status=True).clone()


def _bits(t):
    return t.contiguous().view(torch.int16)


def _same_up_to_sum_order(a, b):
    a32, b32 = a.float(), b.float()
    diff = (a32 - b32).abs()
    row_max = torch.maximum(a32.abs().amax(dim=1, keepdim=True), b32.abs().amax(dim=1, keepdim=True))
    bound = 8 * 2.0 ** -8 * torch.clamp(row_max, min=1.0)     # eight roundings at the row's largest magnitude
    assert (diff <= bound).all(), f"max difference {diff.max().item():.4f}"
    frac_all, frac_nz, _ = synth.check_close(a, b)
    assert frac_all >= 0.9999 and frac_nz >= 0.9999


def test_repeat_differs_by_fp32_sum_order_only_at_4096_tokens(full_weights_gpu):
    dev = torch.device("cuda", 0)
    bias = synth.make_bias(0).to(dev)
    lg, hq, hsc = _tokens(4096, 0, dev)
    a = _run(lg, bias, hq, hsc, full_weights_gpu)
    b = _run(lg, bias, hq, hsc, full_weights_gpu)
    _same_up_to_sum_order(a, b)


def test_token_permutation_permutes_the_output_rows(full_weights_gpu):
    """A token's result depends on no other token: same K order and same promotion order whatever
    packed row it lands in; only the order of the final fp32 additions is free."""
    dev = torch.device("cuda", 0)
    bias = synth.make_bias(0).to(dev)
    lg, hq, hsc = _tokens(4096, 0, dev)
    base = _run(lg, bias, hq, hsc, full_weights_gpu)
    perm = torch.randperm(4096, generator=torch.Generator().manual_seed(7)).to(dev)
    out = _run(lg[perm].contiguous(), bias, hq[perm].contiguous(), hsc[:, perm].contiguous(), full_weights_gpu)
    _same_up_to_sum_order(out, base[perm])


def test_subset_of_tokens_gives_the_same_rows(full_weights_gpu):
    dev = torch.device("cuda", 0)
    bias = synth.make_bias(0).to(dev)
    lg, hq, hsc = _tokens(4096, 0, dev)
    base = _run(lg, bias, hq, hsc, full_weights_gpu)
    # 64 tokens: same kernels (128-row tiles), so the same values up to the order of the final sums
    sub = _run(lg[:64].contiguous(), bias, hq[:64].contiguous(), hsc[:, :64].contiguous(), full_weights_gpu)
    _same_up_to_sum_order(sub, base[:64])
    # 16 tokens: the swapped-operand decode kernels; same arithmetic order, compared at the layer's tolerance
    sub = _run(lg[:16].contiguous(), bias, hq[:16].contiguous(), hsc[:, :16].contiguous(), full_weights_gpu)
    frac_all, frac_nz, max_abs = synth.check_close(sub, base[:16].cpu())
    assert frac_all >= 0.999 and frac_nz >= 0.999, (frac_all, frac_nz, max_abs)


def test_doubling_the_routed_scaling_factor_doubles_the_output(full_weights_gpu):
    """weights = s * (rsf / sum): a factor of two is exact in every product and in every bf16 rounding,
    so only the order of the final additions can show."""
    dev = torch.device("cuda", 0)
    bias = synth.make_bias(0).to(dev)
    lg, hq, hsc = _tokens(1024, 0, dev)
    a = _run(lg, bias, hq, hsc, full_weights_gpu, rsf=RSF)
    b = _run(lg, bias, hq, hsc, full_weights_gpu, rsf=2 * RSF)
    assert torch.isfinite(b.float()).all()
    _same_up_to_sum_order(b, (a.float() * 2).to(torch.bfloat16))


def test_largest_batch_sampled_tokens_against_oracle(full_weights_cpu, full_weights_gpu):
    """16384 tokens (the largest benchmark size): tokens without a local expert are exactly zero,
    everything is finite, and 24 sampled tokens match the oracle run on those tokens alone."""
    dev = torch.device("cuda", 0)
    T = 16384
    bias_cpu = synth.make_bias(0)
    lg, hq, hsc = synth.make_tokens(T, 0, 0)
    out = _run(lg.to(dev), bias_cpu.to(dev), hq.to(dev), hsc.to(dev), full_weights_gpu)
    assert torch.isfinite(out.float()).all()
    ws = K.get_workspace(dev, T, 32, synth.HIDDEN, synth.INTER)
    ids = ws.view("topk_ids", torch.int32, (T, 8)).cpu().numpy()
    local = ((ids >= 0) & (ids < 32)).any(axis=1)
    out_cpu = out.cpu()
    assert (out_cpu[torch.from_numpy(~local)] == 0).all()
    counts = ws.view("expert_count", torch.int32, (32,)).cpu().numpy()
    assert np.array_equal(counts, O.local_counts(ids, 0, 32))
    rng = np.random.default_rng(3)
    pick = np.sort(rng.choice(np.nonzero(local)[0], size=24, replace=False))
    sel = torch.from_numpy(pick)
    ora = O.moe_layer_torch(lg[sel], bias_cpu, hq[sel], hsc[:, sel].contiguous(), *full_weights_cpu, 0, RSF)
    assert np.array_equal(ids[pick], ora["ids"]), "expert ids must be bit-exact"
    frac_all, frac_nz, max_abs = synth.check_close(out_cpu[sel], ora["out"])
    assert frac_all >= 0.999 and frac_nz >= 0.999, (frac_all, frac_nz, max_abs)
