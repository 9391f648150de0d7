"""GPU parity of the fused quantiser against the CPU oracle and the golden fixtures: every byte output bit-exact."""
import json
import hashlib
import os

import numpy as np
import pytest
import torch

from inputs import DISTS, make, attention_inputs
from oracle import quant_oracle as Q

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def same(got, want, what):
    g = got.detach().contiguous().cpu().view(torch.uint8).numpy() if isinstance(got, torch.Tensor) else got
    w = np.ascontiguousarray(want).view(np.uint8)
    assert g.size == w.size, (what, g.shape, w.shape)
    n = int((g.reshape(-1) != w.reshape(-1)).sum())
    assert n == 0, f"{what}: {n} of {w.size} bytes differ"


def run(x, **kw):
    from flamia_blackwell_attention_b200.kernels import quantize_fp8_blocks
    return quantize_fp8_blocks(x.cuda(), **kw)


@pytest.mark.parametrize("dist", DISTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_blocks_ten_families(dist, dtype):
    x = make((2, 256, 3, 128), dist, dtype)
    got = run(x, make_channel_major_copy=True, output_sf_atoms=True)
    ref = Q.fp8_token_blocks(x.float().numpy())
    for k in ("codes", "codes_t", "e", "fac", "sf_tok_raw", "sf_dim_raw"):
        same(got[k], ref[k], f"{dist} {dtype} {k}")


@pytest.mark.parametrize("dist", [d for d in DISTS if d != "huge"])   # rotated "huge" rows overflow to inf / NaN
def test_blocks_rotated(dist):
    x = make((2, 256, 3, 128), dist)
    got = run(x, apply_hadamard_rotation=True, also_make_nvfp4_copy=True, output_sf_atoms=True)
    ref = Q.fp8_token_blocks(x.float().numpy(), rotate=True, nvfp4_copy=True)
    for k in ("codes", "e", "fac", "sf_tok_raw", "sf_dim_raw", "x4"):
        same(got[k], ref[k], f"{dist} rot {k}")
    same(got["sf4_raw"], ref["sf4"], f"{dist} rot sf4")


@pytest.mark.parametrize("dist", DISTS)
def test_nvfp4_copy_and_scope(dist):
    x = make((2, 256, 3, 128), dist)
    got = run(x, also_make_nvfp4_copy=True)
    r4 = Q.nvfp4_rows(x.float().numpy())
    same(got["x4"], r4["codes"], f"{dist} x4")
    same(got["sf4_raw"], r4["sf"], f"{dist} sf4")
    if dist != "huge":
        got = run(x, also_make_nvfp4_copy=True, apply_hadamard_rotation=True, hadamard_rotation_scope="nvfp4_copy")
        r4 = Q.nvfp4_rows(x.float().numpy(), rotate=True)
        same(got["x4"], r4["codes"], f"{dist} rotated x4")
        same(got["sf4_raw"], r4["sf"], f"{dist} rotated sf4")
        same(got["codes"], Q.fp8_token_blocks(x.float().numpy())["codes"], f"{dist} unrotated codes")


@pytest.mark.parametrize("dist", ["n01", "outlier", "zeros", "mixed", "subnorm_sf"])
@pytest.mark.parametrize("d", [128, 64])
def test_token_local_and_d64(dist, d):
    x = make((1, 384, 2, d), dist)
    got = run(x, token_local_exponents=True, output_sf_atoms=True)
    ref = Q.fp8_token_blocks(x.float().numpy(), token_local=True)
    for k in ("codes", "e", "fac", "sf_tok_raw", "sf_dim_raw", "token_factors"):
        same(got[k], ref[k], f"{dist} tl {k}")
    got = run(x, make_channel_major_copy=True, output_sf_atoms=True)
    ref = Q.fp8_token_blocks(x.float().numpy())
    for k in ("codes", "codes_t", "e", "fac", "sf_tok_raw", "sf_dim_raw"):
        same(got[k], ref[k], f"{dist} d{d} {k}")


@pytest.mark.parametrize("dist", ["n01", "outlier", "zeros", "mixed"])
@pytest.mark.parametrize("d", [128, 64])
def test_prologue_d_lse_and_zeroed_accumulator(dist, d):
    x = make((1, 384, 2, d), dist)
    o = make((1, 384, 2, d), "n01", seed=5)
    lse = torch.randn(1, 2, 384, generator=torch.Generator().manual_seed(9))
    lse[0, 1, 3:9] = -float("inf")
    acc = torch.full((1, 2, 384, d), 7.0, dtype=torch.float16, device="cuda")
    got = run(x, compute_d_with_output=o.cuda(), shifted_log2_lse_from=lse.cuda(), log2_lse_shift=8.0,
              d_multiplier=-2.0 ** -8, zero_accumulator=acc)
    ref = Q.fp8_token_blocks(x.float().numpy(), d_with_output=o.float().numpy(), lse=lse.numpy(), lse_shift=8.0,
                             d_multiplier=-2.0 ** -8)
    same(got["codes"], ref["codes"], "codes")
    same(got["D"], ref["D"], "D (tree order, bitwise)")
    same(got["lse_log2"], ref["lse_log2"], "lse_log2")
    assert float(acc.abs().max()) == 0.0


@pytest.mark.parametrize("dist", DISTS)
@pytest.mark.parametrize("rotate", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_one_thread_per_row_kernel(dist, rotate, dtype):
    """The plain head_dim 128 launches (what the 8-bit route issues for Q, K, V) run on the one-thread-per-row kernel:
    codes, exponents and factors against the oracle, and every output, statistics included, bit for bit against the
    four-lanes-per-row kernel."""
    if rotate and dist == "huge":
        pytest.skip("rotated huge rows overflow to inf / NaN")
    x = make((2, 384, 3, 128), dist, dtype)
    b, s = x.shape[:2]
    kind = "norm2" if rotate else "sumsq"
    rs_new, rs_old = (torch.zeros(b, s, dtype=torch.float32, device="cuda") for _ in range(2))
    new = run(x, apply_hadamard_rotation=rotate, output_tile_stats=True, row_stat=(kind, rs_new))
    old = run(x, apply_hadamard_rotation=rotate, output_tile_stats=True, row_stat=(kind, rs_old), legacy_kernel=True)
    ref = Q.fp8_token_blocks(x.float().numpy(), rotate=rotate)
    for k in ("codes", "e", "fac"):
        same(new[k], ref[k], f"{dist} {dtype} rot={rotate} {k}")
        same(new[k], old[k].cpu().view(torch.uint8).numpy(), f"{dist} old/new {k}")
    same(new["tile_stats"], old["tile_stats"].cpu().view(torch.uint8).numpy(), f"{dist} tile_stats")
    same(rs_new, rs_old.cpu().view(torch.uint8).numpy(), f"{dist} row_stat")
    # the NVFP4 copy modes (the mixed route's Q / K launches): rotated codes + copy, and the copy alone rotated
    for scope in ("all", "nvfp4_copy"):
        if not rotate:
            continue
        kw = dict(apply_hadamard_rotation=True, hadamard_rotation_scope=scope, also_make_nvfp4_copy=True,
                  output_tile_stats=True)
        new, old = run(x, **kw), run(x, legacy_kernel=True, **kw)
        for k in ("codes", "e", "fac", "x4", "sf4_raw", "tile_stats"):
            same(new[k], old[k].cpu().view(torch.uint8).numpy(), f"{dist} {scope} old/new {k}")


@pytest.mark.parametrize("dist", DISTS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_one_thread_per_row_kernel_at_head_dim_64(dist, dtype):
    """Head dim 64 (no rotation there) on the one-thread-per-row kernel: against the oracle and bit for bit, statistics
    included, against the four-lanes-per-row kernel."""
    x = make((2, 384, 3, 64), dist, dtype)
    b, s = x.shape[:2]
    rs_new, rs_old = (torch.zeros(b, s, dtype=torch.float32, device="cuda") for _ in range(2))
    new = run(x, output_tile_stats=True, row_stat=("sumsq", rs_new))
    old = run(x, output_tile_stats=True, row_stat=("sumsq", rs_old), legacy_kernel=True)
    ref = Q.fp8_token_blocks(x.float().numpy())
    for k in ("codes", "e", "fac"):
        same(new[k], ref[k], f"{dist} {dtype} d64 {k}")
        same(new[k], old[k].cpu().view(torch.uint8).numpy(), f"{dist} d64 old/new {k}")
    same(new["tile_stats"], old["tile_stats"].cpu().view(torch.uint8).numpy(), f"{dist} d64 tile_stats")
    same(rs_new, rs_old.cpu().view(torch.uint8).numpy(), f"{dist} d64 row_stat")
    for kind in ("amax", "norm2"):
        t_new, t_old = (torch.zeros(b, s, dtype=torch.float32, device="cuda") for _ in range(2))
        run(x, row_stat=(kind, t_new)); run(x, row_stat=(kind, t_old), legacy_kernel=True)
        same(t_new, t_old.cpu().view(torch.uint8).numpy(), f"{dist} d64 row_stat {kind}")


def test_golden_small_fixture_on_gpu():
    small = np.load(os.path.join(HERE, "golden", "quant_small.npz"))
    for dist in ("n01", "zeros", "mixed"):
        for d in (128, 64):
            key = f"{dist}.{d}."
            x = torch.from_numpy(small[key + "x"]).view(torch.bfloat16)
            got = run(x, output_sf_atoms=True)
            same(got["codes"], small[key + "plain.codes"], key + "codes")
            same(got["e"], small[key + "plain.e"], key + "e")
            same(got["fac"], small[key + "plain.fac"], key + "fac")
            same(got["sf_tok_raw"], small[key + "plain.sf_tok_raw"], key + "sf_tok")
            if d == 128:
                got = run(x, apply_hadamard_rotation=True, also_make_nvfp4_copy=True)
                same(got["codes"], small[key + "rot.codes"], key + "rot codes")
                same(got["x4"], small[key + "nvrot.codes"], key + "nvrot codes")
                same(got["sf4_raw"], small[key + "nvrot.sf"], key + "nvrot sf")


def test_config_shapes_digest_property():
    # full-size property at the headline shape: dequantised codes reproduce x within half an E4M3 step of the block scale
    q, _, _, _ = attention_inputs(1, 4096, 16, 16, 128, seed=0)
    got = run(q)
    codes = got["codes"].float()
    fac = got["fac"].repeat_interleave(32, 2).permute(0, 2, 1)[..., None]
    deq = codes * fac
    err = (deq - q.cuda().float()).abs()
    assert float((err / fac).max()) <= 16.0 + 1e-6      # half of the largest E4M3 step (32) in units of the block scale
    assert float(codes.abs().max()) <= 448.0


def test_token_aux_tables_are_exact():
    """fl_token_aux: log2 f and 1 / f of power-of-two token factors (the per-token rows the reference keeps in its
    (6, b, h, s) table, flash_attn/cute/lowprec/_routes.py:749-755), exact for every exponent a token factor can take."""
    from flamia_blackwell_attention_b200 import kernels as K
    e = torch.arange(-126, 127, dtype=torch.float32)
    f = torch.exp2(e).repeat(5).cuda()
    lg, rcp = K.token_aux(f)
    assert torch.equal(lg.cpu(), e.repeat(5)) and torch.equal(rcp.cpu(), torch.exp2(-e).repeat(5))
    x = torch.randn(1, 256, 2, 128).bfloat16().cuda()
    x[0, 7] = 0                                       # an all-zero token: factor 1
    r = K.quantize_fp8_blocks(x, token_local_exponents=True)
    lg, rcp = K.token_aux(r["token_factors"])
    assert torch.equal(lg, torch.log2(r["token_factors"])) and torch.equal(rcp, 1.0 / r["token_factors"])
    assert float(lg[0, :, 7].abs().max()) == 0.0
