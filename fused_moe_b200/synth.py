"""Seeded synthetic inputs for the DeepSeek-V3-shape FP8 block-scale MoE layer.

The contest dataset the reference was measured on is not redistributable, so
tests and the bench use inputs with the same shapes, dtypes and layouts drawn
from fixed CPU generators (identical bytes on every machine):

* routing_logits  fp32 [T, 256]            ~ N(0, 1)
* routing_bias    bf16 [256]               ~ N(0, 0.1)   (or the Zipf stress bias)
* hidden_states   e4m3 [T, H] + fp32 [H/128, T] scales (amax/448 per 1x128 block)
* gemm1_weights   e4m3 [E, 2I, H] + fp32 [E, 2I/128, H/128] scales (per 128x128)
* gemm2_weights   e4m3 [E, H, I]  + fp32 [E, H/128, I/128] scales

Argument order and layouts follow the reference entry point
(solution/python/kernel.py:642-648).  An expert's bytes depend only on its
global id and the base seed, never on the expert-parallel world size, so an
EP run over R ranks sees the same 256 experts as a single-GPU run.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

E_GLOBAL = 256
N_GROUP = 8
GROUP_SIZE = 32
TOPK_GROUP = 4
TOP_K = 8
HIDDEN = 7168
INTER = 2048
BLOCK = 128
FP8_MAX = 448.0


@dataclass
class MoEInputs:
    routing_logits: torch.Tensor
    routing_bias: torch.Tensor
    hidden_states: torch.Tensor
    hidden_states_scale: torch.Tensor
    gemm1_weights: torch.Tensor
    gemm1_weights_scale: torch.Tensor
    gemm2_weights: torch.Tensor
    gemm2_weights_scale: torch.Tensor
    local_expert_offset: int
    routed_scaling_factor: float

    def args(self):
        """The ten positional arguments of ``run``."""
        return (self.routing_logits, self.routing_bias, self.hidden_states,
                self.hidden_states_scale, self.gemm1_weights, self.gemm1_weights_scale,
                self.gemm2_weights, self.gemm2_weights_scale,
                self.local_expert_offset, self.routed_scaling_factor)

    def to(self, device):
        mv = lambda t: t.to(device, non_blocking=False)
        return MoEInputs(mv(self.routing_logits), mv(self.routing_bias), mv(self.hidden_states),
                         mv(self.hidden_states_scale), mv(self.gemm1_weights),
                         mv(self.gemm1_weights_scale), mv(self.gemm2_weights),
                         mv(self.gemm2_weights_scale), self.local_expert_offset,
                         self.routed_scaling_factor)


def quant_rows_1x128(x: torch.Tensor):
    """fp32 [T, K] -> (e4m3 [T, K], fp32 scales [K/128, T]); scale = amax/448 per 1x128."""
    T, K = x.shape
    xb = x.view(T, K // BLOCK, BLOCK)
    s = (xb.abs().amax(-1).clamp_min(1e-12) / FP8_MAX)
    q = (xb / s.unsqueeze(-1)).to(torch.float8_e4m3fn).view(T, K)
    return q, s.t().contiguous()


def quant_blocks_128x128(w: torch.Tensor):
    """fp32 [N, K] -> (e4m3 [N, K], fp32 scales [N/128, K/128]); scale = amax/448 per block."""
    N, K = w.shape
    wb = w.view(N // BLOCK, BLOCK, K // BLOCK, BLOCK)
    s = (wb.abs().amax(dim=(1, 3)).clamp_min(1e-12) / FP8_MAX)
    q = (wb / s[:, None, :, None]).to(torch.float8_e4m3fn).view(N, K)
    return q, s


def make_bias(seed: int = 0, zipf: bool = False) -> torch.Tensor:
    if zipf:
        # 3*ln of a Zipf(s=1.2) weight over the 256 experts: a handful of experts take
        # most tokens, many take none (empty segments, ragged tails).
        i = torch.arange(1, E_GLOBAL + 1, dtype=torch.float64)
        w = i.pow(-1.2)
        w = w / w.sum()
        return (3.0 * w.log()).to(torch.float32).to(torch.bfloat16)
    g = torch.Generator(device="cpu").manual_seed(100 * seed + 1)
    return (0.1 * torch.randn(E_GLOBAL, generator=g)).to(torch.bfloat16)


def _w1_std(hidden: int) -> float:
    """N(0, 0.02) at the benchmark shape; widened at reduced test shapes so that the layer
    output keeps the same O(1) magnitude (and the parity tolerance keeps its meaning)."""
    return 0.02 * math.sqrt(HIDDEN / hidden)


def _w2_std(inter: int) -> float:
    return 0.02 * math.sqrt(INTER / inter)


def make_expert(e_global: int, seed: int = 0, hidden: int = HIDDEN, inter: int = INTER,
                device: str = "cpu"):
    """One expert's quantised weights: (w1 [2I,H], s1, w2 [H,I], s2)."""
    g = torch.Generator(device="cpu").manual_seed(100000 * seed + 10 + e_global)
    w1 = _w1_std(hidden) * torch.randn(2 * inter, hidden, generator=g)
    w2 = _w2_std(inter) * torch.randn(hidden, inter, generator=g)
    if device != "cpu":
        w1, w2 = w1.to(device), w2.to(device)
    q1, s1 = quant_blocks_128x128(w1)
    q2, s2 = quant_blocks_128x128(w2)
    return q1, s1, q2, s2


def make_weights(e_local: int, local_expert_offset: int = 0, seed: int = 0,
                 hidden: int = HIDDEN, inter: int = INTER, device: str = "cpu",
                 fast_device_rng: bool = False):
    """Weights of experts [offset, offset+e_local).

    ``fast_device_rng`` draws directly on ``device`` (different bytes from the
    CPU generator, same distribution); the bench uses it for the 256-expert
    layer where the CPU generator would take minutes.
    """
    w1 = torch.empty(e_local, 2 * inter, hidden, dtype=torch.float8_e4m3fn, device=device)
    s1 = torch.empty(e_local, 2 * inter // BLOCK, hidden // BLOCK, dtype=torch.float32, device=device)
    w2 = torch.empty(e_local, hidden, inter, dtype=torch.float8_e4m3fn, device=device)
    s2 = torch.empty(e_local, hidden // BLOCK, inter // BLOCK, dtype=torch.float32, device=device)
    for e in range(e_local):
        if fast_device_rng:
            g = torch.Generator(device=device).manual_seed(100000 * seed + 10 + local_expert_offset + e)
            a = _w1_std(hidden) * torch.randn(2 * inter, hidden, generator=g, device=device)
            b = _w2_std(inter) * torch.randn(hidden, inter, generator=g, device=device)
            q1, t1 = quant_blocks_128x128(a)
            q2, t2 = quant_blocks_128x128(b)
        else:
            q1, t1, q2, t2 = make_expert(local_expert_offset + e, seed, hidden, inter, device)
        w1[e], s1[e], w2[e], s2[e] = q1, t1, q2, t2
    return w1, s1, w2, s2


def make_tokens(T: int, rank: int = 0, seed: int = 0, hidden: int = HIDDEN):
    """(routing_logits fp32 [T,256], hidden e4m3 [T,H], scales fp32 [H/128,T]) of one rank."""
    g = torch.Generator(device="cpu").manual_seed(100 * seed + 50 + rank)
    logits = torch.randn(T, E_GLOBAL, generator=g)
    hs = torch.randn(T, hidden, generator=g)
    q, s = quant_rows_1x128(hs)
    return logits, q, s


def make_inputs(T: int, e_local: int = 32, local_expert_offset: int = 0, seed: int = 0,
                rank: int = 0, zipf: bool = False, hidden: int = HIDDEN, inter: int = INTER,
                rsf: float = 2.5, weights=None, token_seed=None) -> MoEInputs:
    """``token_seed`` (default: ``seed``) draws other tokens for the same weights and bias."""
    logits, hq, hsc = make_tokens(T, rank, seed if token_seed is None else token_seed, hidden)
    bias = make_bias(seed, zipf)
    if weights is None:
        weights = make_weights(e_local, local_expert_offset, seed, hidden, inter)
    w1, s1, w2, s2 = weights
    return MoEInputs(logits, bias, hq, hsc, w1, s1, w2, s2, int(local_expert_offset), float(rsf))


# --------------------------------------------------------------------------
# Algorithmic work of one layer call (what the roofline fractions are taken of)
# --------------------------------------------------------------------------

def algorithmic_bytes(T: int, n_active: int, hidden: int = HIDDEN, inter: int = INTER) -> int:
    """Compulsory HBM bytes: active experts' weights+scales, token I/O, bias."""
    per_expert = 2 * inter * hidden + hidden * inter \
        + 4 * ((2 * inter // BLOCK) * (hidden // BLOCK) + (hidden // BLOCK) * (inter // BLOCK))
    per_token = hidden + 4 * (hidden // BLOCK) + 4 * E_GLOBAL + 2 * hidden
    return n_active * per_expert + T * per_token + 2 * E_GLOBAL


def algorithmic_flops(m_local: int, hidden: int = HIDDEN, inter: int = INTER) -> int:
    """2*M*(N1*K1 + N2*K2) over the rows that have a local expert."""
    return 2 * m_local * (2 * inter * hidden + hidden * inter)


def gemm1_bytes(m_local: int, n_active: int, hidden: int = HIDDEN, inter: int = INTER) -> int:
    """Compulsory bytes of the GEMM1 launch alone: W1 + scales of active experts,
    the gathered e4m3 rows + their scales in, the e4m3 activation rows out."""
    return n_active * (2 * inter * hidden + 4 * (2 * inter // BLOCK) * (hidden // BLOCK)) \
        + m_local * (hidden + 4 * (hidden // BLOCK)) + m_local * (inter + 4)


def gemm1_flops(m_local: int, hidden: int = HIDDEN, inter: int = INTER) -> int:
    return 2 * m_local * 2 * inter * hidden


def check_close(out: torch.Tensor, ref: torch.Tensor, atol: float = 0.05, rtol: float = 0.05):
    """Fraction of elements with |out-ref| <= atol + rtol*|ref| (all rows, rows with work)."""
    o = out.float().cpu()
    r = ref.float().cpu()
    ok = (o - r).abs() <= atol + rtol * r.abs()
    nz = (r != 0).any(dim=1) | (o != 0).any(dim=1)
    frac_all = ok.float().mean().item() if ok.numel() else 1.0
    frac_nz = ok[nz].float().mean().item() if nz.any() else 1.0
    return frac_all, frac_nz, (o - r).abs().max().item() if ok.numel() else 0.0


def contest_match(out: torch.Tensor, ref: torch.Tensor, atol: float = 1.0, rtol: float = 0.3) -> float:
    """Fraction of elements inside the contest harness's own band, |out-ref| <= 1 + 0.3*|ref|
    (scripts/run_local.py:59-62 of the reference asks for >= 90 %); reported beside the far
    tighter parity tolerance of check_close for comparability with the reference's logs."""
    o = out.float().cpu()
    r = ref.float().cpu()
    ok = (o - r).abs() <= atol + rtol * r.abs()
    return ok.float().mean().item() if ok.numel() else 1.0
