"""Pins the attention and scale oracles (oracle/attention_oracle.py, oracle/scales_oracle.py) to fixtures that
tests/golden/make_golden_attention.py produced by running the reference's own definitions on CPU:
benchmarks/benchmark_lowprec_attn.py `reference` / `accuracy`, benchmarks/benchmark_packed_docs.py `reference_docs`,
tests/cute/test_lowprec_api.py `_ref_bottom_right`, flash_attn/cute/device_scales.py `_dq_tile_table` (Triton CPU
interpreter) and `_bwd1_fp8_host`. No GPU, no reference checkout needed."""
import json
import math
import os

import numpy as np
import pytest
import torch

from inputs import attention_inputs, br_inputs, scale_stats
from oracle import attention_oracle as A
from oracle import scales_oracle as S

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = np.load(os.path.join(HERE, "golden", "attention_small.npz"))
SCAL = json.load(open(os.path.join(HERE, "golden", "scales_small.json")))

# fp32 matmuls in a different blocking: a few ulps of the largest term
TOL = dict(rtol=2e-5, atol=2e-5)

ATTN_CASES = {   # as in the generator: (b, s, h, hk, d, causal, window, chunk)
    "causal_gqa": (1, 160, 4, 2, 32, True, None, 64),
    "dense_window": (1, 128, 2, 2, 32, False, (40, 24), 1024),
    "causal_window": (1, 128, 2, 1, 16, True, (48, None), 32),
    "dense": (1, 64, 2, 2, 64, False, None, 1024),
}
BR_CASES = {
    "sq_lt_sk_causal": (1, 64, 128, 4, 2, 32, True),
    "sq_gt_sk_causal": (1, 128, 64, 2, 2, 32, True),
    "sq_lt_sk_dense": (2, 32, 96, 2, 1, 16, False),
}


def _close(got, want, what):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin), what
    np.testing.assert_allclose(got[fin], want[fin], err_msg=what, **TOL)


@pytest.mark.parametrize("name", sorted(ATTN_CASES))
def test_attention_fp32_matches_reference_function(name):
    b, s, h, hk, d, causal, window, chunk = ATTN_CASES[name]
    q, k, v, g = attention_inputs(b, s, h, hk, d, seed=21)
    # a different chunking than the generator's on purpose: the result must not depend on it
    o, lse, dq, dk, dv = A.attention_fp32(q, k, v, g, causal=causal, window=window, chunk=48)
    for key, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        _close(t.numpy(), GOLD[f"ref.{name}.{key}"], f"{name}.{key}")


@pytest.mark.parametrize("name", sorted(BR_CASES))
def test_attention_fp32_bottom_right_and_rectangular(name):
    b, sq, sk, h, hk, d, causal = BR_CASES[name]
    q, k, v, do = br_inputs(b, sq, sk, h, hk, d, seed=33)
    o, lse, dq, dk, dv = A.attention_fp32(q, k, v, do, causal=causal)
    for key, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        want = GOLD[f"br.{name}.{key}"]
        if key == "lse":          # rows that see no key: -inf in both
            assert np.array_equal(np.isneginf(t.numpy()), np.isneginf(want)), name
        _close(np.nan_to_num(t.numpy(), neginf=0.0), np.nan_to_num(want, neginf=0.0), f"{name}.{key}")


def test_attention_fp32_batched_seqused_k():
    q, k, v, do = br_inputs(2, 64, 128, 2, 1, 32, seed=34)
    o, lse, dq, dk, dv = A.attention_fp32(q, k, v, do, causal=True, seqused_k=[100, 37])
    for key, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        want = GOLD[f"seqused.{key}"]
        if key == "lse":
            assert np.array_equal(np.isneginf(t.numpy()), np.isneginf(want))
        _close(np.nan_to_num(t.numpy(), neginf=0.0), np.nan_to_num(want, neginf=0.0), f"seqused.{key}")


def test_attention_fp32_softcap_and_window():
    q, k, v, g = attention_inputs(1, 96, 2, 2, 32, seed=52)
    q = (q.float() * 3.0).to(torch.bfloat16)
    o, _lse, dq, dk, dv = A.attention_fp32(q, k, v, g, causal=True, window=(40, 0), softcap=2.0)
    for key, t in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        _close(t.numpy(), GOLD[f"softcap.{key}"], f"softcap.{key}")


def test_attention_docs_fp32_matches_reference_docs():
    lens, h, hk, d = [37, 128, 91], 2, 1, 32
    q, k, v, g = (t[0] for t in attention_inputs(1, sum(lens), h, hk, d, seed=45))
    o, _lse, dq, dk, dv = A.attention_docs_fp32(q, k, v, g, lens, causal=True)
    for key, t in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
        _close(t.numpy(), GOLD[f"docs.{key}"], f"docs.{key}")


def test_accuracy_matches_reference_accuracy():
    got = A.accuracy(torch.from_numpy(GOLD["acc.x"]), torch.from_numpy(GOLD["acc.ref"]))
    for key, want in SCAL["accuracy"].items():
        assert math.isclose(got[key], want, rel_tol=1e-5, abs_tol=1e-7), (key, got[key], want)


def test_kernel_scalars_match_reference_host_values():
    for row in SCAL["bwd1_fp8_host"]:
        got = S.bwd1_fp8_scalars(*row["args"])
        assert [float(x) for x in got] == row["out"], row["args"]


@pytest.mark.parametrize("i", range(len(SCAL["dq_tables"])))
def test_dq_prescale_tables_bitwise(i):
    row = SCAL["dq_tables"][i]
    b, hq, hk, tq, tk = row["shape"]
    kw = dict(unit=row["unit"], base=1.0, num=row["num"])
    if row["mode"] == "causal_row":
        dn, vn, km = scale_stats(1, 1, 1, tq, tk, row["kind"], seed=row["seed"])
        kern, post = S.dq_prescale_causal_rows(dn.numpy(), vn.numpy(), km.numpy(), **kw)
    else:
        dn, vn, km = scale_stats(b, hq, hk, tq, tk, row["kind"], seed=row["seed"])
        fn = S.dq_prescale_rows if row["mode"] == "row" else S.dq_prescale_causal_tiles
        kern, post = fn(dn.numpy(), vn.numpy(), km.numpy(), b, hq, hk, tq, tk, **kw)
    want_k, want_p = np.asarray(row["kernel"], np.float32), np.asarray(row["post"], np.float32)
    assert np.array_equal(kern.view(np.uint32), want_k.view(np.uint32)), (row["mode"], row["kind"], row["shape"])
    assert np.array_equal(post.view(np.uint32), want_p.view(np.uint32)), (row["mode"], row["kind"], row["shape"])


def test_library_constants_are_the_reference_scalars():
    """The backward folds the reference's kernel scalars (unit operand descales, block-scaled dS-hat) into constants:
    P' = 2^8 P, D'' = -2^-8 D, dV x 2^-8, dK x softmax_scale, dQ postprocess x softmax_scale / B."""
    from flamia_blackwell_attention_b200 import _routes
    for d in (64, 128):
        sm = 1.0 / math.sqrt(d)
        want = S.bwd1_fp8_scalars(sm, 2.0 ** _routes.P_SHIFT_LOG2, 4.0)
        got = _routes.backward_scalars(sm, dq_boost=4.0)
        assert [float(x) for x in got] == [float(x) for x in want]
