"""Generates tests/golden/attention_small.npz and scales_small.json by RUNNING the reference's own plain-Python / Triton
definitions on CPU. Run once where the reference is mounted:

    TRITON_INTERPRET=1 python tests/golden/make_golden_attention.py /path/to/reference

What is executed, unmodified, from the reference checkout:
  * benchmarks/benchmark_lowprec_attn.py   `reference` (chunked fp32 attention fwd + bwd), `accuracy`
  * benchmarks/benchmark_packed_docs.py    `reference_docs` (fp32 attention per packed document)
  * tests/cute/test_lowprec_api.py         `_ref_bottom_right` (s_q != s_k, bottom-right causal, seqused_k, autograd) and
                                           `_ref_attn` (softcap and window; gradients by autograd through it)
  * flash_attn/cute/device_scales.py       `_bwd1_fp8_host`, `_bwd1_fp4_host`, `_bwd2_host` (numpy float32 kernel scalars) and
                                           the Triton kernel `_dq_tile_table` (per-row / per-tile / per-query-row f16 dQ
                                           pre-scale) under Triton's CPU interpreter
The benchmark and test modules import GPU-only packages at module level, so the named functions are taken out of the
parsed file (ast) and executed as they stand with torch / math in scope; device_scales.py imports as a module.
Inputs come from tests/inputs.py (seeded); the reference checkout is not needed to RUN the tests.
"""
import ast
import importlib.util
import json
import math
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from inputs import attention_inputs, br_inputs, scale_stats  # noqa: E402


def functions_of(path, names):
    """The named top-level functions of a Python file, compiled from its own source text."""
    tree = ast.parse(open(path).read(), path)
    ns = {"torch": torch, "math": math, "np": np}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    missing = [n for n in names if n not in ns]
    if missing:
        raise SystemExit(f"{path}: no function {missing}")
    return [ns[n] for n in names]


ATTN_CASES = {   # name -> (b, s, h, hk, d, causal, window, chunk)
    "causal_gqa": (1, 160, 4, 2, 32, True, None, 64),
    "dense_window": (1, 128, 2, 2, 32, False, (40, 24), 1024),
    "causal_window": (1, 128, 2, 1, 16, True, (48, None), 32),
    "dense": (1, 64, 2, 2, 64, False, None, 1024),
}
BR_CASES = {     # name -> (b, s_q, s_k, h, hk, d, causal)
    "sq_lt_sk_causal": (1, 64, 128, 4, 2, 32, True),
    "sq_gt_sk_causal": (1, 128, 64, 2, 2, 32, True),
    "sq_lt_sk_dense": (2, 32, 96, 2, 1, 16, False),
}
SEQUSED_CASE = dict(shape=(2, 64, 128, 2, 1, 32), causal=True, seqused=[100, 37])   # (b, s_q, s_k, h, hk, d)
DOC_CASE = dict(lens=[37, 128, 91], h=2, hk=1, d=32)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden_attention.py <reference checkout>")
    root = sys.argv[1]
    reference, accuracy = functions_of(os.path.join(root, "benchmarks", "benchmark_lowprec_attn.py"),
                                       ["reference", "accuracy"])
    (reference_docs,) = functions_of(os.path.join(root, "benchmarks", "benchmark_packed_docs.py"), ["reference_docs"])
    ref_bottom_right, ref_attn = functions_of(os.path.join(root, "tests", "cute", "test_lowprec_api.py"),
                                              ["_ref_bottom_right", "_ref_attn"])
    out = {}
    for name, (b, s, h, hk, d, causal, window, chunk) in ATTN_CASES.items():
        q, k, v, g = (t.float() for t in attention_inputs(b, s, h, hk, d, seed=21))
        o, lse, dq, dk, dv = reference(q, k, v, g, causal, True, chunk=chunk, window=window)
        for key, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[f"ref.{name}.{key}"] = t.contiguous().numpy()
    for name, (b, sq, sk, h, hk, d, causal) in BR_CASES.items():
        q, k, v, do = br_inputs(b, sq, sk, h, hk, d, seed=33)
        o, lse, dq, dk, dv = ref_bottom_right(q, k, v, do, causal)
        for key, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
            out[f"br.{name}.{key}"] = t.contiguous().numpy()
    q, k, v, do = br_inputs(*SEQUSED_CASE["shape"], seed=34)
    o, lse, dq, dk, dv = ref_bottom_right(q, k, v, do, SEQUSED_CASE["causal"], seqused=torch.tensor(SEQUSED_CASE["seqused"]))
    for key, t in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv)):
        out[f"seqused.{key}"] = t.contiguous().numpy()
    # softcap (with a causal window): _ref_attn is MHA only
    q, k, v, g = attention_inputs(1, 96, 2, 2, 32, seed=52)
    q = (q.float() * 3.0).to(torch.bfloat16)           # scores large enough for the cap to bite
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    oc = ref_attn(qf, kf, vf, True, window=(40, 0), softcap=2.0)
    oc.backward(g.float())
    for key, t in (("o", oc.detach()), ("dq", qf.grad), ("dk", kf.grad), ("dv", vf.grad)):
        out[f"softcap.{key}"] = t.contiguous().numpy()
    lens, h, hk, d = DOC_CASE["lens"], DOC_CASE["h"], DOC_CASE["hk"], DOC_CASE["d"]
    tot = sum(lens)
    q, k, v, g = (t[0] for t in attention_inputs(1, tot, h, hk, d, seed=45))
    r = reference_docs(q, k, v, g, lens, True, True, chunk=64)
    for key in ("o", "dq", "dk", "dv"):
        out[f"docs.{key}"] = r[key].contiguous().numpy()
    # accuracy(): a seeded pair with a planted outlier and a near-zero reference entry
    gen = torch.Generator().manual_seed(5)
    ref_t = torch.randn(4, 33, generator=gen)
    ref_t[0, 0] = 1e-9
    x_t = ref_t + 0.01 * torch.randn(4, 33, generator=gen)
    x_t[1, 2] += 0.7
    acc = accuracy(x_t, ref_t)
    out["acc.x"], out["acc.ref"] = x_t.numpy(), ref_t.numpy()
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), **out)

    # ---- kernel scalars and the f16 dQ pre-scale tables (device_scales.py, imported as a module)
    spec = importlib.util.spec_from_file_location("ref_device_scales", os.path.join(root, "flash_attn", "cute", "device_scales.py"))
    ds = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ds)
    scal = {"accuracy": acc, "bwd1_fp8_host": [], "bwd1_fp4_host": [], "bwd2_host": [], "dq_tables": []}
    for d_head in (64, 128, 96):
        for boost in (1.0, 4.0, 2.0 ** -7):
            a = (1.0 / math.sqrt(d_head), 256.0, boost)
            scal["bwd1_fp8_host"].append({"args": a, "out": ds._bwd1_fp8_host(*a)})
    for a in ((1.0 / math.sqrt(128), 16.0, True, True, True, True, 3), (0.125, 16.0, True, True, True, False, 3)):
        scal["bwd1_fp4_host"].append({"args": a, "out": ds._bwd1_fp4_host(*a)})
    for a in ((1.0 / math.sqrt(128), 256.0, True, True, 3), (0.125, 256.0, False, True, 3)):
        scal["bwd2_host"].append({"args": a, "out": ds._bwd2_host(*a)})
    tab = torch.zeros(8, dtype=torch.int32)
    for kind in ("plain", "zeros", "huge", "tiny"):
        for (b, hq, hk, tq, tk) in ((2, 4, 2, 3, 3), (1, 2, 2, 5, 5), (3, 8, 1, 2, 4)):
            for unit, num in ((1.0, 1.0), (256.0, 0.08838834764831845)):
                dn, vn, km = scale_stats(b, hq, hk, tq, tk, kind, seed=b * 100 + tq)
                n_ent = b * tq
                for mode in ("row", "causal_tile"):
                    if mode == "causal_tile" and tq != tk:
                        continue
                    o = torch.zeros(8 + 2 * n_ent + b)
                    grid = (b,) if mode == "row" else (b * tq,)
                    ds._dq_tile_table[grid](dn, vn, km, tab, o, 1, hq, hk, tq, tk, n_ent, 1.0, num, unit, DOCS=0,
                                            CAUSAL=0 if mode == "row" else 1)
                    scal["dq_tables"].append(dict(mode=mode, kind=kind, shape=[b, hq, hk, tq, tk], unit=unit, num=num,
                                                  seed=b * 100 + tq, kernel=o[8:8 + n_ent].tolist(),
                                                  post=o[8 + n_ent:8 + 2 * n_ent].tolist()))
    # CAUSAL 2: per query row, from per-row statistics (n_ent = rows)
    for kind in ("plain", "tiny"):
        n = 300
        dn, vn, km = scale_stats(1, 1, 1, n, n, kind, seed=7)
        o = torch.zeros(8 + 2 * n + 1)
        ds._dq_tile_table[(1,)](dn, vn, km, tab, o, 1, 1, 1, n, n, n, 1.0, 0.125, 256.0, DOCS=0, CAUSAL=2)
        scal["dq_tables"].append(dict(mode="causal_row", kind=kind, shape=[1, 1, 1, n, n], unit=256.0, num=0.125, seed=7,
                                      kernel=o[8:8 + n].tolist(), post=o[8 + n:8 + 2 * n].tolist()))
    with open(os.path.join(HERE, "scales_small.json"), "w") as f:
        json.dump(scal, f, indent=0, sort_keys=True)
    print("wrote", len(out), "arrays and", len(scal["dq_tables"]), "pre-scale tables")


if __name__ == "__main__":
    main()
