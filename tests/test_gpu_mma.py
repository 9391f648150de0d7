"""GPU: the tensor-core building blocks (descriptor encodings, TMEM operand packing, scale-factor placement) against a
CPU product, one 128 x 128 x 128 tile per operand path. Integer-valued operands make the products exact in fp32."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as Q

pytestmark = pytest.mark.gpu


def codes(seed, shape=(128, 128)):
    g = np.random.default_rng(seed)
    vals = g.integers(-4, 5, size=shape).astype(np.float32)         # small integers: exact in E4M3 and in the fp32 sum
    return Q.e4m3_encode(vals), vals


def run(which, a, b, sfa=None, sfb=None):
    from flamia_blackwell_attention_b200.kernels import selftest_mma
    t = lambda z: None if z is None else torch.from_numpy(np.ascontiguousarray(z)).cuda()
    d, st = selftest_mma(which, t(a), t(b), t(sfa), t(sfb))
    assert st == 0
    return d.cpu().numpy()


def test_kmajor():
    a, av = codes(1); b, bv = codes(2)
    np.testing.assert_array_equal(run(0, a, b), av @ bv.T)


def test_b_mn_major():
    a, av = codes(3); b, bv = codes(4)          # b stored (k, n)
    np.testing.assert_array_equal(run(1, a, b), av @ bv)


def test_a_from_tmem():
    a, av = codes(5); b, bv = codes(6)
    np.testing.assert_array_equal(run(2, a, b), av @ bv)


def test_a_mn_major():
    a, av = codes(7); b, bv = codes(8)          # a stored (k, m), b stored (n, k)
    np.testing.assert_array_equal(run(6, a, b), av.T @ bv.T)


def _mx8_expected(av, bv, sfa, sfb):
    out = np.zeros((128, 128), dtype=np.float64)
    for kb in range(4):
        sl = slice(32 * kb, 32 * kb + 32)
        part = av[:, sl].astype(np.float64) @ bv[sl, :].astype(np.float64)
        out += part * np.exp2(sfa[:, kb].astype(np.float64) - 127)[:, None] * np.exp2(sfb[:, kb].astype(np.float64) - 127)[None, :]
    return out.astype(np.float32)


@pytest.mark.parametrize("which", [3, 4])
def test_block_scaled_mxfp8(which):
    a, av = codes(9); b, bv = codes(10)         # a (m, k), b (k, n)
    g = np.random.default_rng(11)
    sfa = g.integers(120, 134, size=(128, 4)).astype(np.uint8)
    sfb = g.integers(120, 134, size=(128, 4)).astype(np.uint8)
    # the four K blocks carry different scales, so the fp32 accumulation rounds: relative 1e-5, not bitwise
    np.testing.assert_allclose(run(which, a, b, sfa, sfb), _mx8_expected(av, bv, sfa, sfb), rtol=1e-5, atol=1e-4)


def test_block_scaled_nvfp4():
    g = np.random.default_rng(12)
    grid = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32)
    ca = g.integers(0, 16, size=(128, 128)).astype(np.uint8)
    cb = g.integers(0, 16, size=(128, 128)).astype(np.uint8)
    av, bv = Q.e2m1_decode(ca), Q.e2m1_decode(cb)
    sfa_v = 2.0 ** g.integers(-2, 3, size=(128, 8)).astype(np.float32)      # powers of two: exact products
    sfb_v = 2.0 ** g.integers(-2, 3, size=(128, 8)).astype(np.float32)
    sfa_b, sfb_b = Q.e4m3_encode(sfa_v), Q.e4m3_encode(sfb_v)
    atoms = lambda t: Q.sf_atoms(t.reshape(1, 1, 128, 8)).reshape(-1)       # two 512-byte atoms
    got = run(5, Q.pack_nibbles(ca), Q.pack_nibbles(cb), atoms(sfa_b), atoms(sfb_b))
    want = (av * np.repeat(sfa_v, 16, 1)).astype(np.float64) @ (bv * np.repeat(sfb_v, 16, 1)).astype(np.float64).T
    np.testing.assert_array_equal(got, want.astype(np.float32))


def test_block_scaled_nvfp4_upper_half_of_b():
    # the operand path of the backward's NVFP4 S^T recompute for the second 64-query half tile
    g = np.random.default_rng(16)
    ca = g.integers(0, 16, size=(128, 128)).astype(np.uint8)
    cb = g.integers(0, 16, size=(128, 128)).astype(np.uint8)
    av, bv = Q.e2m1_decode(ca), Q.e2m1_decode(cb)
    sfa_v = 2.0 ** g.integers(-2, 3, size=(128, 8)).astype(np.float32)
    sfb_v = 2.0 ** g.integers(-2, 3, size=(128, 8)).astype(np.float32)
    atoms = lambda t: Q.sf_atoms(t.reshape(1, 1, 128, 8)).reshape(-1)
    got = run(9, Q.pack_nibbles(ca), Q.pack_nibbles(cb), atoms(Q.e4m3_encode(sfa_v)), atoms(Q.e4m3_encode(sfb_v)))[:, :64]
    want = (av * np.repeat(sfa_v, 16, 1)).astype(np.float64) @ (bv * np.repeat(sfb_v, 16, 1)).astype(np.float64)[64:].T
    np.testing.assert_array_equal(got, want.astype(np.float32))


def test_wait_that_nothing_completes_returns_a_status():
    from flamia_blackwell_attention_b200.kernels import selftest_mma
    d, st = selftest_mma(7, None, None, wait_cycles=200000)
    assert st == (0x100 | 1)
    # the context is still usable afterwards
    a, av = codes(1); b, bv = codes(2)
    np.testing.assert_array_equal(run(0, a, b), av @ bv.T)


def test_block_scaled_mn_major_a_and_64_wide_mn_major_b():
    # the operand layout of the backward's transposed dQ product: A (k, m) 128 B rows, B (k, n = 64) 64 B rows
    a, av = codes(13)
    b, bv = codes(14, (128, 64))
    g = np.random.default_rng(15)
    sfa = g.integers(120, 134, size=(128, 4)).astype(np.uint8)
    sfb = g.integers(120, 134, size=(128, 4)).astype(np.uint8)
    got = run(8, a, b, sfa, sfb)[:, :64]
    want = _mx8_expected(np.ascontiguousarray(av.T), np.pad(bv, ((0, 0), (0, 64))), sfa, sfb)[:, :64]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-4)


def test_block_scaled_a_as_two_64_wide_mn_major_blocks():
    # the operand layout of the d = 64 backward's dQ product: A (k, m) held as two (k, 64) blocks of 64-byte rows
    a, av = codes(17)
    b, bv = codes(18, (128, 64))
    g = np.random.default_rng(19)
    sfa = g.integers(120, 134, size=(128, 4)).astype(np.uint8)
    sfb = g.integers(120, 134, size=(128, 4)).astype(np.uint8)
    got = run(10, a, b, sfa, sfb)[:, :64]
    want = _mx8_expected(np.ascontiguousarray(av.T), np.pad(bv, ((0, 0), (0, 64))), sfa, sfb)[:, :64]
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-4)
