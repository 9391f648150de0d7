"""Seeded synthetic inputs shared by the tests, the golden generator and bench.py.

The ten quantiser input families are those the reference's quantiser tests use (tests/cute/test_quant_fp8.py:23-57 of the
reference: same constants), drawn here from torch's CPU generator so that they are reproducible without a GPU.
attention_inputs follows the reference benchmark's make_inputs (benchmarks/benchmark_lowprec_attn.py:880-886): q, k, v
drawn in that order from manual_seed(seed) as fp32 then cast to bf16, dO from manual_seed(seed + 7).
"""
import math

import torch

DISTS = ("n01", "logit3", "outlier", "zeros", "tiny", "denorm", "near_min_normal", "huge", "mixed", "subnorm_sf")


def make(shape, dist, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g, dtype=torch.float32)
    fmax = torch.finfo(dtype).max
    if dist == "logit3":
        x = x * 3.0
    elif dist == "outlier":
        m = torch.rand(*shape, generator=g) < 1e-3
        x = torch.where(m, x * 1000.0, x)
    elif dist == "zeros":
        x = x * (torch.rand(*shape[:-1], 1, generator=g) < 0.5)
        x[..., :32] = 0.0
    elif dist == "tiny":
        x = x * 1e-30
    elif dist == "denorm":
        x = x * 1e-39
    elif dist == "near_min_normal":
        x = x * 1e-37
    elif dist == "huge":
        x = (x.clamp(-4, 4) / 4.0) * (min(fmax, 3e38) * 0.99)
    elif dist == "mixed":
        e = torch.randint(-60, 60, (*shape[:-1], shape[-1] // 16), generator=g).float()
        x = x * torch.exp2(e).repeat_interleave(16, dim=-1)
    elif dist == "subnorm_sf":
        x = x * 1e-3 * (2.0 ** -torch.randint(0, 14, (*shape[:-1], 1), generator=g).float())
    x = x.clamp(-fmax, fmax).to(dtype)
    assert torch.isfinite(x).all()
    return x


def attention_inputs(b, s, h, hk, d, seed=0, outlier_channels=False):
    """(q, k, v, dO) bf16 CPU tensors, (b, s, heads, d). outlier_channels: a seeded 1 % of the (head, channel) pairs of
    Q and of K multiplied by 20 in fp32 before the bf16 cast (config 4 of the benchmark set)."""
    gen = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(b, s, n, d, generator=gen, dtype=torch.float32) for n in (h, hk, hk))
    if outlier_channels:
        for t, n in ((q, h), (k, hk)):
            cnt = max(1, round(0.01 * n * d))
            sel = torch.randperm(n * d, generator=torch.Generator().manual_seed(seed + 11))[:cnt]
            flat = t.view(b, s, n * d)
            flat[..., sel] *= 20.0
    g = torch.randn(b, s, h, d, generator=torch.Generator().manual_seed(seed + 7), dtype=torch.float32)
    return tuple(t.to(torch.bfloat16) for t in (q, k, v, g))


def packed_doc_lengths(spec_total=16384, lo=128, hi=8192, seed=0):
    """Document lengths of the packed benchmark set 'logu<lo>-<hi>-t<total>-s<seed>': exp of a uniform draw in
    [ln lo, ln hi] from random.Random(seed), the last document cut so that the lengths sum to the total (the rule of the
    reference's benchmarks/benchmark_packed_docs.py:55-66)."""
    import random
    rng = random.Random(seed)
    out, tot = [], 0
    while tot < spec_total:
        n = int(round(math.exp(rng.uniform(math.log(lo), math.log(hi)))))
        n = min(n, spec_total - tot)
        out.append(n)
        tot += n
    if len(out) > 1 and out[-1] < 16:
        out[-2] += out.pop()
    return out


def br_inputs(b, sq, sk, h, hk, d, seed):
    """(q, k, v, dO) bf16 with s_q != s_k, drawn in that order from one generator (the reference test's order,
    tests/cute/test_lowprec_api.py:1390-1394)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, sq, h, d, generator=g).to(torch.bfloat16)
    k, v = (torch.randn(b, sk, hk, d, generator=g).to(torch.bfloat16) for _ in range(2))
    do = torch.randn(b, sq, h, d, generator=g).to(torch.bfloat16)
    return q, k, v, do


def scale_stats(b, hq, hk, tq, tk, kind, seed):
    """Per-tile statistics for the f16 dQ pre-scale tables: (max ||dO_q||^2 (b hq tq), max ||V_k||^2, max|K| (b hk tk)) with
    the edge cases of the bound: zeros (the cap), overflow (the floor), tiny values."""
    g = torch.Generator().manual_seed(seed)
    dn = torch.rand(b * hq * tq, generator=g) * 300.0
    vn = torch.rand(b * hk * tk, generator=g) * 200.0
    km = torch.rand(b * hk * tk, generator=g) * 9.0
    if kind == "zeros":
        dn[: hq * tq] = 0.0          # first batch row: zero bound -> the cap 2^40
    if kind == "huge":
        dn *= 1e30
        vn *= 1e30                  # an intermediate overflows -> the floor 2^-40
    if kind == "tiny":
        dn *= 1e-20
        km *= 1e-12
    return dn, vn, km
