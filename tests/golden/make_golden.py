"""Generates the golden fixtures of tests/golden/ by IMPORTING the reference's own eager quantiser definitions
(tests/cute/quant_reference.py of the reference checkout) on CPU. Run once where the reference is mounted:

    python tests/golden/make_golden.py /path/to/reference

Outputs (committed): quant_small.npz (full arrays, shape (1,128,2,128) and (1,128,2,64)) and quant_digests.json (sha256
of every output for the ten input families at (2,256,3,128); inputs are regenerated from the seed by tests/inputs.py and
their own digest is stored so a generator mismatch is detected). The reference checkout is not needed to RUN the tests.
"""
import hashlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from inputs import DISTS, make  # noqa: E402


def load_reference(root):
    # quant_reference imports flash_attn.cute.quant._rotations / .fp4 lazily; stub the parent packages so that only
    # the two plain-Python modules it needs are found (the CuTe-DSL kernels are never imported).
    for name in ("flash_attn", "flash_attn.cute", "flash_attn.cute.quant"):
        m = types.ModuleType(name)
        m.__path__ = [os.path.join(root, *name.split("."))]
        sys.modules[name] = m
    rot = types.ModuleType("flash_attn.cute.quant._rotations")

    def hadamard_signs(seed=4321, d=128):
        g = torch.Generator(device="cpu").manual_seed(int(seed) & 0x7FFFFFFF)
        return tuple(int(v) for v in (torch.randint(0, 2, (d,), generator=g) * 2 - 1).tolist())
    rot.hadamard_signs = hadamard_signs
    sys.modules["flash_attn.cute.quant._rotations"] = rot
    fp4 = types.ModuleType("flash_attn.cute.quant.fp4")
    fp4.D_SUM_ORDER = (1, 2, 4, 8, 16, 32, 64)
    sys.modules["flash_attn.cute.quant.fp4"] = fp4
    sys.path.insert(0, os.path.join(root, "tests", "cute"))
    import quant_reference as R
    return R


def old_order_row_dot(a, o):
    """The reference test's statement of the D summation order (tests/cute/test_quant_fp8.py:77-92), float64 fma."""
    a, o = a.float(), o.float()
    idx = torch.arange(128)
    lo = idx[(idx >> 1) & 1 == 0]
    v = (a[..., lo].double() * o[..., lo].double() + (a[..., lo + 2] * o[..., lo + 2]).double()).float()
    cols = lo
    for bit in (2, 3, 0, 6, 5, 4):
        keep = ((cols >> bit) & 1) == 0
        partner = cols[keep] | (1 << bit)
        pos = torch.empty(128, dtype=torch.long)
        pos[cols] = torch.arange(cols.numel())
        v = v[..., keep] + v[..., pos[partner]]
        cols = cols[keep]
    return v[..., 0]


def run_case(R, x, o=None, lse=None):
    """every output the oracle restates, from the reference's definitions, as numpy arrays"""
    out = {}
    d = x.shape[-1]
    for tag, kw in (("plain", {}), ("rot", dict(apply_hadamard_rotation=True)), ("tl", dict(token_local_exponents=True))):
        if tag == "rot" and d != 128:
            continue
        r = R.fp8_blocks_reference(x, **kw)
        for k in ("codes", "codes_t", "e", "fac", "sf_tok_raw", "sf_dim_raw"):
            out[f"{tag}.{k}"] = r[k].contiguous().view(torch.uint8).numpy() if r[k].dtype != torch.float32 \
                else r[k].numpy()
        if tag == "tl":
            out["tl.token_factors"] = r["token_factors"].numpy()
    if d == 128:
        for tag, rot in (("nv", False), ("nvrot", True)):
            r = R.fp4_rows_reference(x, apply_hadamard_rotation=rot)
            out[f"{tag}.codes"] = r["codes"].numpy()
            out[f"{tag}.sf"] = r["scale_factors"].permute(6, 5, 2, 4, 0, 1, 3).contiguous().numpy()  # (b,h,Rt,ka,32,4,4)
    if o is not None:
        r = R.fp8_blocks_reference(x, compute_d_with_output=o, shifted_log2_lse_from=lse, log2_lse_shift=8.0)
        sc = torch.where(r["e"][..., 0] == 0, torch.zeros(()), torch.exp2(r["e"][..., 0].float() - 127.0))
        sc = sc.repeat_interleave(32, 2)[..., None]
        a = (r["codes"].float().permute(0, 2, 1, 3).double() * sc.double()).float()
        op = o.float().permute(0, 2, 1, 3)
        if d < 128:
            a, op = (torch.nn.functional.pad(t, (0, 128 - d)) for t in (a, op))
        out["pro.D_tree"] = old_order_row_dot(a, op).numpy()
        out["pro.D_f64"] = r["D"].numpy()
        out["pro.lse_log2"] = r["lse_log2"].numpy()
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of the reference repository>")
    root = sys.argv[1]
    R = load_reference(root)
    small = {}
    for dist in ("n01", "zeros", "mixed"):
        for d in (128, 64):
            x = make((1, 128, 2, d), dist, seed=3)
            o = make((1, 128, 2, d), "n01", seed=5)
            lse = torch.randn(1, 2, 128, generator=torch.Generator().manual_seed(9))
            lse[0, 1, 3:9] = -float("inf")
            small[f"{dist}.{d}.x"] = x.view(torch.int16).numpy()
            small[f"{dist}.{d}.o"] = o.view(torch.int16).numpy()
            small[f"{dist}.{d}.lse"] = lse.numpy()
            for k, v in run_case(R, x, o, lse).items():
                if k.endswith("codes_t") or k.endswith("sf_dim_raw"):
                    continue            # transposes / row-uniform tables: pinned by the digests below
                small[f"{dist}.{d}.{k}"] = v
    np.savez_compressed(os.path.join(HERE, "quant_small.npz"), **small)
    digests = {}
    for dist in DISTS:
        x = make((2, 256, 3, 128), dist, seed=0)
        entry = {"x": hashlib.sha256(x.view(torch.int16).numpy().tobytes()).hexdigest()}
        for k, v in run_case(R, x).items():
            entry[k] = hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest()
        digests[dist] = entry
    with open(os.path.join(HERE, "quant_digests.json"), "w") as f:
        json.dump(digests, f, indent=1, sort_keys=True)
    print("wrote", len(small), "arrays and", len(digests), "digest families")


if __name__ == "__main__":
    main()
