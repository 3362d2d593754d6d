"""The double-precision exp/log kernels of the CUDA backward scan, built for the host, against
libm and against the CPU oracle's backward scan (bit for bit)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _build(name, flags):
    src = os.path.join(HERE, "host_model", "exact_math_host.cpp")
    so = os.path.join(HERE, "host_model", name)
    subprocess.run(["g++", "-O2", "-fPIC", "-shared", "-ffp-contract=off"] + flags + ["-o", so, src], check=True)
    lib = C.CDLL(so)
    fp = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    u8 = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
    lib.host_backward_scan.argtypes = [fp, fp, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.host_fold2.restype = C.c_float
    lib.host_fold2.argtypes = [C.c_float, C.c_float]
    lib.host_lse5_many.argtypes = [fp, fp, C.c_int, fp, u8, u8]
    for f in ("host_exp_neg", "host_log_1to8", "host_round_to_f32", "host_exp_of", "host_exp_of_t2",
              "host_log_1to8_t2"):
        getattr(lib, f).restype = C.c_double
        getattr(lib, f).argtypes = [C.c_double]
    return lib


@pytest.fixture(scope="module")
def host():
    """The arithmetic as the library is built (first tier alone)."""
    return _build("libexact_math_host.so", [])


@pytest.fixture(scope="module")
def host_rigorous():
    """The same with the checks of every rounding and the second tier behind them."""
    return _build("libexact_math_host_rigorous.so", ["-DOFX_RIGOROUS=1"])


def test_exp_log_accuracy(host):
    rng = np.random.default_rng(0)
    a = np.concatenate([rng.uniform(0, 20, 5000), rng.uniform(0, 80, 1000), [0.0, 17.0, 80.0]])
    err = max(abs(host.host_exp_neg(x) - np.exp(-x)) for x in a)
    assert err < 2.0 ** -44
    assert host.host_exp_neg(0.0) == 1.0
    y = np.concatenate([rng.uniform(1, 8, 6000), [1.0, 2.0, 4.0, 5.0, np.nextafter(8.0, 0)]])
    err = max(abs(host.host_log_1to8(v) - np.log(v)) for v in y)
    assert err < 2.0 ** -43


def test_round_to_f32_matches_conversion(host):
    rng = np.random.default_rng(1)
    v = np.concatenate([rng.uniform(0.5, 8, 4000), np.exp(rng.uniform(-80, 2, 4000)),
                        # exact ties between neighbouring floats
                        (np.float32(1.0) + np.arange(1, 200, 2) * 2.0 ** -24).astype(np.float64)])
    for x in v:
        assert host.host_round_to_f32(float(x)) == float(np.float32(x))


def test_fold_matches_oracle(host, oracle_mod):
    rng = np.random.default_rng(2)
    x = rng.uniform(-3000, 3000, 4000).astype(np.float32)
    y = (x + rng.uniform(-20, 20, 4000)).astype(np.float32)
    for a, b in zip(x, y):
        assert host.host_fold2(a, b) == oracle_mod.fold_scores(a, b)
    big = np.float32(-3.4028234663852886e38)
    for a, b in ((big, 1.0), (big, big), (5.0, 5.0), (0.0, 17.0), (0.0, 16.999)):
        assert host.host_fold2(a, b) == oracle_mod.fold_scores(a, b)


@pytest.mark.parametrize("sl,T,N,seed,p_step", [(3, 800, 6, 11, 1.0), (4, 500, 3, 12, 0.5), (5, 120, 1, 13, 1.0)])
def test_backward_scan_bit_exact(host, oracle_mod, sl, T, N, seed, p_step):
    from openfish_b200 import synth
    sc = synth.make_scores(T, N, sl, seed, p_step=p_step).astype(np.float32)
    ref = oracle_mod.backward_scan(sc, sl)
    out = np.zeros_like(ref)
    for c in range(N):
        host.host_backward_scan(sc, out, c, T, N, 4 ** sl)
    assert np.array_equal(out, ref)


@pytest.mark.parametrize("sl,scale,shift,seed", [(4, 8.0, 0.0, 94), (3, 30.0, 0.0, 93), (3, 64.0, 0.0, 8),
                                                 (4, 1.0, -40.0, 94), (3, 0.25, 3.0, 95)])
def test_backward_scan_bit_exact_on_wide_score_ranges(host, oracle_mod, sl, scale, shift, seed):
    # one dominant term makes the sum 1 + k*2^-23; with a round maximum (first timestep: the stay
    # score itself) max + log(sum) then sits within k^2 * 2^-47 of a rounding tie, which only a log
    # with a relative error near 1 decides correctly
    from openfish_b200 import synth
    T, N = 300, 4
    sc = (synth.make_scores(T, N, sl, seed).astype(np.float32) * scale + shift).astype(np.float16).astype(np.float32)
    ref = oracle_mod.backward_scan(sc, sl)
    out = np.zeros_like(ref)
    for c in range(N):
        host.host_backward_scan(sc, out, c, T, N, 4 ** sl)
    assert np.array_equal(out, ref)


def test_log_is_relative_near_one(host):
    for k in (0, 1, 2, 3, 7, 100, 12345):
        y = 1.0 + k * 2.0 ** -23
        want = float(np.log1p(np.float64(k) * 2.0 ** -23))
        assert abs(host.host_log_1to8(y) - want) <= 2.0 ** -52 * max(want, 2.0 ** -30)


def test_backward_scan_bit_exact_on_reference_golden(host, oracle_mod):
    from conftest import load_golden
    sc = load_golden("ref_fast_chunk")["scores"].astype(np.float32)
    ref = oracle_mod.backward_scan(sc, 3)
    out = np.zeros_like(ref)
    host.host_backward_scan(sc, out, 0, 1666, 1, 64)
    assert np.array_equal(out, ref)


def test_second_tier_accuracy(host):
    from decimal import Decimal, getcontext
    getcontext().prec = 50
    rng = np.random.default_rng(3)
    worst1 = worst2 = worst_log = Decimal(0)
    for x in np.concatenate([rng.uniform(-80, 3, 1500), rng.uniform(-5, 2, 1500)]):
        exact = Decimal(float(x)).exp()
        worst1 = max(worst1, abs((Decimal(host.host_exp_of(float(x))) - exact) / exact))
        worst2 = max(worst2, abs((Decimal(host.host_exp_of_t2(float(x))) - exact) / exact))
    for y in rng.uniform(1, 8, 2000):
        worst_log = max(worst_log, abs(Decimal(host.host_log_1to8_t2(float(y))) - Decimal(float(y)).ln()))
    assert worst1 < Decimal(2) ** -43 and worst2 < Decimal(2) ** -51 and worst_log < Decimal(2) ** -50


def _random_terms(rng, n, lo, hi, spread, quantum=None):
    base = rng.uniform(lo, hi, n).astype(np.float32)
    gaps = np.abs(rng.normal(0, spread, (n, 5))).astype(np.float32)
    if quantum:
        gaps = (np.round(gaps / quantum) * quantum).astype(np.float32)
    gaps[np.arange(n), rng.integers(0, 5, n)] = 0
    return np.ascontiguousarray((base[:, None] - gaps).astype(np.float32))


@pytest.mark.parametrize("lo,hi,spread,quantum", [(2000, 6000, 4.0, None), (-50, 50, 3.0, None), (0, 2, 1.0, None),
                                                  (-6000, -2000, 6.0, None), (100, 1000, 2.0, 0.25),
                                                  (2000, 6000, 30.0, None)])
def test_two_tiers_and_confirmation_against_the_oracle(host, oracle_mod, lo, hi, spread, quantum):
    # first tier with its checks, second tier where they ask for it: every value equals the
    # oracle's; the checks do fire now and then (so the second tier is exercised) but rarely; and
    # the shortcut that confirms a guess never confirms a wrong one
    import ctypes
    rng = np.random.default_rng(int(abs(lo) + hi))
    n = 1_500_000
    v = _random_terms(rng, n, lo, hi, spread, quantum)
    orc = ctypes.CDLL(os.path.join(os.path.dirname(HERE), "oracle", "liboracle.so"))
    fp = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
    orc.oracle_lse5_many.argtypes = [fp, C.c_int, fp]
    ref = np.zeros(n, np.float32)
    orc.oracle_lse5_many(v.reshape(-1), n, ref)
    guess = ref.copy()
    pick = rng.random(n)
    guess[pick < 0.1] = np.nextafter(ref[pick < 0.1], np.float32(np.inf))
    guess[pick > 0.9] = np.nextafter(ref[pick > 0.9], np.float32(-np.inf))
    out, flagged, confirmed = np.zeros(n, np.float32), np.zeros(n, np.uint8), np.zeros(n, np.uint8)
    host.host_lse5_many(v.reshape(-1), guess, n, out, flagged, confirmed)
    assert np.array_equal(out, ref)
    right = guess == ref
    assert not (confirmed.astype(bool) & ~right).any()
    assert (confirmed.astype(bool) & right).sum() >= 0.99 * right.sum()
    if lo >= 100 or hi <= -100:   # (results next to zero always ask for the second tier)
        assert flagged.mean() < 1e-3


def test_rigorous_build_scans_bit_exact(host_rigorous, oracle_mod):
    from openfish_b200 import synth
    for sl, T, N, seed in ((3, 500, 4, 31), (4, 300, 2, 32)):
        sc = synth.make_scores(T, N, sl, seed).astype(np.float32)
        ref = oracle_mod.backward_scan(sc, sl)
        out = np.zeros_like(ref)
        for c in range(N):
            host_rigorous.host_backward_scan(sc, out, c, T, N, 4 ** sl)
        assert np.array_equal(out, ref)
