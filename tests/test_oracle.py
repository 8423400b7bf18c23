"""The numpy oracle against the golden vectors made by the reference's own torch function."""
import glob
import os
import zlib

import numpy as np
import pytest
import torch

from conftest import GOLDEN, golden_inputs, load_golden
from fused_moe_b200 import synth
from oracle import moe_oracle as O

SMALL = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "layer_small_*.npz")))


def _crc(inp):
    return np.asarray([zlib.crc32(t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes())
                       for t in inp.args()[:8]], dtype=np.uint64)


def bf16_ulp_distance(a_bits, b_bits):
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, 0x8000 - (b & 0x7FFF), 0x8000 + b)   # monotone in value
    return np.abs(key(a_bits) - key(b_bits))


def test_e4m3_roundtrip_all_codes():
    codes = np.arange(256, dtype=np.uint8)
    vals = O.e4m3_decode(codes)
    finite = ~np.isnan(vals)
    back = O.e4m3_encode(vals[finite])
    # -0 and +0 keep their sign bit; every finite code is a fixed point of decode->encode
    assert np.array_equal(back, codes[finite])


def test_e4m3_encode_matches_torch_cast():
    g = torch.Generator().manual_seed(7)
    x = torch.cat([torch.randn(50000, generator=g) * s for s in (1e-3, 0.05, 1.0, 30.0, 150.0)])
    x = x.clamp(-463.0, 463.0)
    ref = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x.numpy()), ref)
    ties = torch.tensor([0.0, -0.0, 448.0, 463.9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9,
                         17.0, 19.0, 0.0009765625 * 3])
    assert np.array_equal(O.e4m3_encode(ties.numpy()), ties.to(torch.float8_e4m3fn).view(torch.uint8).numpy())


@pytest.mark.parametrize("name", SMALL)
def test_layer_small_matches_reference(name):
    g, inp = golden_inputs(name)
    assert np.array_equal(_crc(inp), g["input_crc"]), "synthetic input generator drifted from the golden run"
    res = O.moe_layer_torch(*inp.args())
    assert np.array_equal(res["ids"].astype(np.uint8), g["ids"]), "expert ids differ from the reference"
    np.testing.assert_allclose(res["weights"], g["weights"], rtol=1e-6, atol=0)
    d = bf16_ulp_distance(res["out_bits"], g["out_bits"])
    # Bit-identical almost everywhere.  numpy and torch sum the fp32 matmuls in different
    # orders; where that moves an activation across an e4m3 rounding boundary one product
    # term changes by one e4m3 step, which is the only source of the few differing elements.
    assert (d == 0).mean() > 0.995, (d == 0).mean()
    ref = torch.from_numpy(g["out_bits"].view(np.int16).copy()).view(torch.bfloat16)
    frac_all, _, max_abs = synth.check_close(res["out"], ref, atol=0.01, rtol=0.01)
    assert frac_all >= 0.9995 and max_abs <= 0.0625, (frac_all, max_abs)


def test_layer_full_T8_and_T1_match_reference(full_weights_cpu):
    for name in ("layer_full_T8_ts0", "layer_full_T8_ts1", "layer_full_T8_ts2", "layer_full_T1_ts1"):
        g, inp = golden_inputs(name, weights=full_weights_cpu)
        assert np.array_equal(_crc(inp), g["input_crc"])
        res = O.moe_layer_torch(*inp.args())
        assert np.array_equal(res["ids"].astype(np.uint8), g["ids"])
        np.testing.assert_allclose(res["weights"], g["weights"], rtol=1e-6, atol=0)
        d = bf16_ulp_distance(res["out_bits"], g["out_bits"])
        assert (d == 0).mean() > 0.995, (name, (d == 0).mean())
        frac_all, frac_nz, max_abs = synth.check_close(
            res["out"], torch.from_numpy(g["out_bits"].view(np.int16).copy()).view(torch.bfloat16))
        assert frac_all == 1.0 and frac_nz == 1.0


def test_routing_ids_match_reference_on_every_benchmark_token_count():
    g = load_golden("routing_ids")
    keys = sorted(k[:-4] for k in g.files if k.endswith("_ids"))
    assert len(keys) >= 19
    for key in keys:
        parts = key.split("_")
        T = int(parts[0][1:])
        zipf = "zipf" in key
        seed = 1 if key.endswith("_s1") else 0
        rank = int(parts[1][4:]) if parts[1].startswith("rank") else 0
        logits, _, _ = synth.make_tokens(T, rank, seed, hidden=128)
        bias = synth.make_bias(seed, zipf)
        crc = np.asarray([zlib.crc32(logits.numpy().tobytes()),
                          zlib.crc32(bias.view(torch.int16).numpy().tobytes())], dtype=np.uint64)
        assert np.array_equal(crc, g[key + "_crc"]), key
        ids, w, _, _ = O.route(logits.numpy(), bias.float().numpy(), 2.5)
        assert np.array_equal(ids.astype(np.uint8), g[key + "_ids"]), f"{key}: ids differ"
        if key + "_w" in g.files:
            np.testing.assert_allclose(w, g[key + "_w"], rtol=1e-6, atol=0)
        assert abs(w.astype(np.float64).sum() - float(g[key + "_wsum"][0])) <= 1e-6 * T * 8


def test_routing_tie_rules():
    # all logits equal, zero bias: every score ties; lowest ids win at every level
    logits = np.zeros((3, 256), dtype=np.float32)
    bias = np.zeros(256, dtype=np.float32)
    ids, w, _, _ = O.route(logits, bias, 2.5)
    assert np.array_equal(ids[0], np.arange(8))
    np.testing.assert_allclose(w.sum(axis=1), 2.5, rtol=1e-6)
    # group score counts the maximum twice when it occurs twice
    logits = np.full((1, 256), -4.0, dtype=np.float32)
    logits[0, 32 * 5 + 3] = 3.0
    logits[0, 32 * 5 + 9] = 3.0
    logits[0, 32 * 2 + 1] = 3.5
    ids, _, s, s_wb = O.route(logits, bias, 1.0)
    assert set(ids[0, :3]) == {32 * 2 + 1, 32 * 5 + 3, 32 * 5 + 9}
    assert ids[0, 0] == 32 * 2 + 1 and ids[0, 1] == 32 * 5 + 3


def test_scale_layout_rule():
    sc = np.arange(12, dtype=np.float32).reshape(4, 3)      # [K/128=4, T=3]
    assert np.array_equal(O.hidden_scale_rows(sc, 3, 4), sc.T)
    assert np.array_equal(O.hidden_scale_rows(sc.T.copy(), 3, 4), sc.T)
    sq = np.arange(16, dtype=np.float32).reshape(4, 4)      # square: read as [K/128, T]
    assert np.array_equal(O.hidden_scale_rows(sq, 4, 4), sq.T)
    with pytest.raises(ValueError):
        O.hidden_scale_rows(sc, 5, 4)


def test_empty_batch_and_no_local_expert():
    inp = synth.make_inputs(T=0, e_local=32, hidden=256, inter=128, seed=1)
    res = O.moe_layer_torch(*inp.args())
    assert res["out"].shape == (0, 256)
    inp = synth.make_inputs(T=5, e_local=1, local_expert_offset=255, hidden=256, inter=128, seed=1)
    res = O.moe_layer_torch(*inp.args())
    untouched = ~(res["ids"] == 255).any(axis=1)
    assert (res["out"][torch.from_numpy(untouched)] == 0).all()
