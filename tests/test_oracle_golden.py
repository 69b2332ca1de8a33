"""Pins the CPU oracle to the reference: its own dense test oracles (imported unmodified when the
vectors were generated) and the global results of its four ring functions on gloo ranks."""
import os

import numpy as np
import pytest
import torch

from oracle.dense_attn import attn_flops, dense_attn, dense_attn_fwd_bwd, in_window_pairs, merge_partials
from ring_cases import GOLDEN, case_params, load_pins, make_inputs


def test_oracle_matches_reference_dense_oracles():
    z = np.load(os.path.join(GOLDEN, "ref_dense_oracles.npz"))
    n = 0
    while f"swa{n}_params" in z.files:
        W, hq, hkv, seed = (int(x) for x in z[f"swa{n}_params"])
        torch.manual_seed(seed)
        q = torch.randn(1, 256, hq, 16)
        k = torch.randn(1, 256, hkv, 16)
        v = torch.randn(1, 256, hkv, 16)
        o, _ = dense_attn(q, k, v, W, None, 0)
        assert np.abs(o.numpy() - z[f"swa{n}_out"]).max() < 2e-6
        o, _ = dense_attn(q, k, v, W, None, 1)
        assert np.abs(o.numpy() - z[f"slm{n}_out"]).max() < 2e-6
        n += 1
    assert n == 4


PINS = load_pins() if os.path.exists(os.path.join(GOLDEN, "ref_ring_pins.npz")) else []


@pytest.mark.parametrize("idx", range(len(PINS)))
def test_oracle_matches_reference_ring_outputs(idx):
    c = PINS[idx]
    p = case_params(c)
    fn = str(c["fn"])
    varlen = "varlen" in fn
    n_sink = 1 if "streaming" in fn else 0
    q, k, v, do = make_inputs(p["seed"], p["T"], p["hq"], p["hkv"], p["d"], p["bf16_grid"],
                              None if varlen else p["B"], p["sink_rows"])
    if varlen:
        q, k, v, do = (x.unsqueeze(0) for x in (q, k, v, do))
    o, _lse, dq, dk, dv = dense_attn_fwd_bwd(q, k, v, do, p["W"], None, n_sink, p["cu"], compute_dtype=torch.float64)
    for name, got in (("out", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        got = got.squeeze(0) if varlen else got
        err = np.abs(got.float().numpy() - c[name]).max()
        assert err < 2e-5, f"{fn} W={p['W']} cu={p['cu']} {name}: {err}"


def test_pins_cover_all_four_functions():
    assert len(PINS) >= 100
    assert {str(c["fn"]) for c in PINS} == {
        "ring_sliding_window_attn", "ring_sliding_window_attn_varlen",
        "ring_streaming_llm_attn", "ring_streaming_llm_attn_varlen"}


def test_merge_matches_reference_formula():
    # ring_swa/ops/merge.py:16-50 restated with softplus, as the reference writes it
    g = torch.Generator().manual_seed(3)
    oa, ob = torch.randn(2, 9, 3, 8, generator=g), torch.randn(2, 9, 3, 8, generator=g)
    la, lb = torch.randn(2, 3, 9, generator=g) * 4, torch.randn(2, 3, 9, generator=g) * 4
    diff = lb - la
    sa = torch.exp(-torch.nn.functional.softplus(diff)).movedim(1, 2).unsqueeze(-1)
    sb = torch.exp(-torch.nn.functional.softplus(-diff)).movedim(1, 2).unsqueeze(-1)
    ref_o = oa * sa + ob * sb
    ref_l = torch.maximum(la, lb) + torch.log1p(torch.exp(-diff.abs()))
    o, l = merge_partials(oa, la, ob, lb)
    assert (o - ref_o).abs().max() < 1e-6 and (l - ref_l).abs().max() < 1e-6
    ninf = torch.full_like(la, float("-inf"))
    o, l = merge_partials(torch.zeros_like(oa), ninf, torch.zeros_like(oa), ninf)
    assert (o == 0).all() and torch.isinf(l).all()


def test_partials_merge_to_the_whole():
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 40, 2, 8, generator=g) for _ in range(3))
    o, l = dense_attn(q[:, 20:], k, v, 15, None, 1, None, q_pos0=20)
    o1, l1 = dense_attn(q[:, 20:], k[:, :12], v[:, :12], 15, None, 1, None, q_pos0=20, k_pos0=0)
    o2, l2 = dense_attn(q[:, 20:], k[:, 12:], v[:, 12:], 15, None, 1, None, q_pos0=20, k_pos0=12)
    om, lm = merge_partials(o1, l1, o2, l2)
    assert (om - o).abs().max() < 1e-5 and (lm - l).abs().max() < 1e-5


def test_flop_counts_match_the_baseline_table():
    # pairs of the five benchmark configurations (in-window only)
    assert in_window_pairs([1024], 128) == 123840
    assert in_window_pairs([32768], 1000) == 32300268
    assert in_window_pairs([7204, 3978, 14070, 10318, 13142, 12634, 4190], 4096) == 209773421
    assert in_window_pairs([131072], 8192, 1) == 1040437247
    assert in_window_pairs([262144], 65536) == 15032614912
    fwd, bwd = attn_flops([32768], 1000, 32, 128, batch=2)
    assert abs((fwd + bwd) / 1e9 - 3704.5) < 0.1
    # brute force agreement for the sink formula
    for L, W, ns in ((50, 7, 1), (50, 7, 4), (5, 7, 4), (30, 0, 2)):
        brute = sum(len(set(range(max(0, i - W), i + 1)) | set(range(min(ns, i + 1)))) for i in range(L))
        assert in_window_pairs([L], W, ns) == brute
