"""Stage-by-stage comparison of one GPU layer call with the oracle (helper for the GPU tests).

Reads the intermediates out of the workspace (layout from ``b200moe_workspace_layout``) and
checks each against the oracle's value for that stage, so a failure names the first kernel
that went wrong instead of only the final output.
"""
import os

import numpy as np
import torch

from fused_moe_b200 import kernel as K
from fused_moe_b200 import synth
from oracle import moe_oracle as O


def run_gpu(inp_cpu, out=None):
    dev = torch.device("cuda", 0)
    g = inp_cpu.to(dev)
    res = K.custom_kernel(*g.args(), out=out, check_status=True)
    torch.cuda.synchronize()
    T = inp_cpu.routing_logits.shape[0]
    e_local, n1, hidden = inp_cpu.gemm1_weights.shape
    ws = K.get_workspace(dev, T, e_local, hidden, n1 // 2)
    return res, ws


def check_stages(inp_cpu, res, ws, act_rtol=2e-3, verbose=False):
    """Returns a dict of measurements; raises AssertionError naming the failing stage."""
    T = inp_cpu.routing_logits.shape[0]
    e_local, n1, hidden = inp_cpu.gemm1_weights.shape
    inter = n1 // 2
    off = inp_cpu.local_expert_offset
    L = ws.layout_of_last_call()
    ora = O.moe_layer_torch(*inp_cpu.args(), want_stages=True)
    info = {}

    # --- routing
    ids = ws.view("topk_ids", torch.int32, (T, 8)).cpu().numpy()
    w = ws.view("topk_w", torch.float32, (T, 8)).cpu().numpy()
    assert np.array_equal(ids, ora["ids"]), f"routing: {(ids != ora['ids']).any(axis=1).sum()} rows differ"
    np.testing.assert_allclose(w, ora["weights"], rtol=1e-6, atol=0, err_msg="routing weights")

    # --- permutation
    counts = ws.view("expert_count", torch.int32, (e_local,)).cpu().numpy()
    want_counts = O.local_counts(ora["ids"], off, e_local)
    assert np.array_equal(counts, want_counts), "permute: per-expert counts"
    row0 = ws.view("expert_row0", torch.int32, (e_local + 1,)).cpu().numpy()
    meta = ws.view("meta", torch.int32, (8,)).cpu().numpy()
    pad = int(meta[3])                      # rows per M tile
    assert pad == 128
    padded = (want_counts + pad - 1) // pad * pad
    assert np.array_equal(row0, np.concatenate([[0], np.cumsum(padded)])), "permute: padded segment starts"
    m_pad = int(row0[-1])
    assert meta[0] == m_pad // 128 and meta[1] == m_pad and meta[2] == want_counts.sum(), "permute: meta"
    info.update(m_local=int(want_counts.sum()), n_active=int((want_counts > 0).sum()), m_pad=m_pad)
    if m_pad == 0:
        assert (res.float() == 0).all(), "no local work but the output is not zero"
        return info
    row_token = ws.view("row_token", torch.int32, (L.m_cap,))[:m_pad].cpu().numpy()
    row_weight = ws.view("row_weight", torch.float32, (L.m_cap,))[:m_pad].cpu().numpy()
    tile_expert = ws.view("tile_expert", torch.int32, (L.max_tiles,))[:m_pad // 128].cpu().numpy()
    a_packed = ws.view("a_packed", torch.uint8, (L.m_cap, hidden))[:m_pad].cpu().numpy()
    a_scale = ws.view("a_scale", torch.float32, (hidden // 128, L.m_cap))[:, :m_pad].cpu().numpy()
    act = ws.view("act", torch.float16, (L.m_cap, inter))[:m_pad].float().cpu().numpy()
    amax_bits = ws.view("row_amax", torch.int32, (L.m_cap,))[:m_pad].cpu().numpy()
    act_q = ws.view("act_q", torch.uint8, (L.m_cap, inter))[:m_pad].cpu().numpy()
    row_scale = ws.view("row_scale", torch.float32, (L.m_cap,))[:m_pad].cpu().numpy()
    # a call of at most 8 tokens through the fused front kernel runs no gather pass (its GEMM1 reads the caller's rows in place;
    # the activations checked below prove that it read the right rows and scales)
    gathered = not (T <= 8 and os.environ.get("B200MOE_FRONT", "1") != "0"
                    and os.environ.get("B200MOE_DECODE", "1") != "0")
    hs = inp_cpu.hidden_states.view(torch.uint8).numpy()
    hsc = O.hidden_scale_rows(inp_cpu.hidden_states_scale.numpy(), T, hidden // 128)
    worst_act = 0.0
    for e in range(e_local):
        n = int(want_counts[e])
        r0 = int(row0[e])
        assert (tile_expert[r0 // 128:int(row0[e + 1]) // 128] == e).all(), f"permute: tile table of expert {e}"
        assert (row_token[r0 + n:int(row0[e + 1])] == -1).all(), f"permute: padding rows of expert {e}"
        if n == 0:
            continue
        st = ora["stages"][e]
        assert np.array_equal(row_token[r0:r0 + n], st["rows"]), f"permute: token order of expert {e}"
        np.testing.assert_array_equal(row_weight[r0:r0 + n], st["w"], err_msg=f"permute: weights of expert {e}")
        if gathered:
            assert np.array_equal(a_packed[r0:r0 + n], hs[st["rows"]]), f"gather: payload of expert {e}"
            assert np.array_equal(a_scale[:, r0:r0 + n].T, hsc[st["rows"]]), f"gather: scales of expert {e}"
        # --- GEMM1 + SwiGLU
        ref_act = st["act"]
        scale_ref = np.abs(ref_act).max() + 1e-6
        err = np.abs(act[r0:r0 + n] - ref_act).max() / scale_ref
        worst_act = max(worst_act, float(err))
        if err > act_rtol and verbose:
            bad = np.abs(act[r0:r0 + n] - ref_act) / scale_ref > act_rtol
            print(f"expert {e}: act mismatch, rows {np.nonzero(bad.any(1))[0][:8]}, cols {np.nonzero(bad.any(0))[0][:16]}")
            print(" gpu", act[r0:r0 + n][bad][:8], " ref", ref_act[bad][:8])
        assert err <= act_rtol, f"GEMM1+SwiGLU: expert {e} max error {err:.3e} of the expert's max |act|"
        # --- row maxima and requantisation are consistent with the GPU's own activations
        got_amax = amax_bits[r0:r0 + n].view(np.float32)
        assert np.array_equal(got_amax, np.abs(act[r0:r0 + n]).max(axis=1)), f"row amax of expert {e}"
        q_ref, s_ref = O.requant_rows(act[r0:r0 + n])
        np.testing.assert_array_equal(row_scale[r0:r0 + n], s_ref, err_msg=f"requant scale of expert {e}")
        assert np.array_equal(act_q[r0:r0 + n], q_ref), \
            f"requant: expert {e}: {(act_q[r0:r0 + n] != q_ref).sum()} codes differ from RNE(act/scale)"
    info["act_rel_err"] = worst_act
    # --- output
    frac_all, frac_nz, max_abs = synth.check_close(res, ora["out"])
    info.update(frac_all=frac_all, frac_rows_with_work=frac_nz, max_abs=max_abs)
    assert frac_all >= 0.999 and frac_nz >= 0.999, f"output: {frac_all:.5f} / {frac_nz:.5f} within tolerance"
    no_work = ~np.isin(ora["ids"], np.arange(off, off + e_local)).any(axis=1)
    assert (res.float().cpu().numpy()[no_work] == 0).all(), "tokens without a local expert must stay exactly 0"
    return info
