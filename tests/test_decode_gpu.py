"""Parity of the CUDA decode path, called through the C ABI, with the CPU oracle.

Gates (stated in gpu_util.compare / assert_parity): backward scores bit-identical; posterior
within 1e-3 absolutely and within 1e-3 relatively where it is at least 0.01; moves and sequence
byte-identical on at least 99.9 % of chunks (mismatching chunks are listed with their edit
distance in the failure message); qstring within +-1 Phred on sequence-identical chunks."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import SYNTH_CASES, load_golden
from gpu_util import assert_parity, compare, gpu_decode, sequences

pytestmark = pytest.mark.gpu

# gpubuf fields holding the per-timestep outputs, under the oracle's names for them
PER_TIMESTEP = (("qual", "qual_data"), ("states", "states"), ("base_probs", "base_probs"),
                ("total_probs", "total_probs"))


def check(of, oracle, sc16, sl, okw=None, threads=16, **gates):
    okw = okw or {}
    # the library hands options->blank_score to its scans (as the reference's CUDA launcher does)
    # and options->temperature to the beam search as its score_scale; the oracle has a switch for
    # each, both of which are no-ops at the defaults 2.0 and 1.0
    flags = oracle.SCAN_STAY_FROM_OPTIONS | oracle.TEMPERATURE_SCALES_SCORES
    ref = oracle.decode(sc16.astype(np.float32), sl, oracle.decoder_init(**okw), nthreads=threads, tensors=True,
                        flags=flags)
    out = gpu_decode(of, sc16, sl, of.decoder_init(**okw))
    rep = compare(out, ref)
    assert_parity(rep, **gates)
    return out, ref, rep


def test_reference_golden_vector(native_lib, oracle_mod):
    g = load_golden("ref_fast_chunk")
    out = gpu_decode(native_lib, g["scores"], 3, native_lib.decoder_init(q_scale=0.97, q_shift=-1.8), tensors=False)
    assert np.array_equal(out["moves"], g["moves"]) and np.array_equal(out["sequence"], g["sequence"])
    assert np.abs(out["qstring"].astype(int) - g["qstring"].astype(int)).max() <= 1


@pytest.mark.parametrize("name", SYNTH_CASES)
def test_fixtures_from_reference(native_lib, name):
    g = load_golden("synth_" + name)
    out = gpu_decode(native_lib, g["scores"], g["state_len"], native_lib.decoder_init(**g["options"]))
    rep = compare(out, g)
    assert_parity(rep, min_identical=1.0)


def test_config_fast_T1000_N16(native_lib, oracle_mod):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(1000, 16, 3, 0x0F15), 3, min_identical=1.0)


def test_hac_T1666(native_lib, oracle_mod):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(1666, 48, 4, 0x0F16), 4, min_identical=1.0)


def test_sup_T1666(native_lib, oracle_mod):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(1666, 6, 5, 0x0F17), 5, min_identical=1.0)


@pytest.mark.parametrize("sl,T,N", [(3, 1, 1), (3, 2, 3), (3, 7, 5), (4, 9, 1), (3, 257, 7), (4, 513, 3),
                                    (5, 3, 2), (3, 300, 9), (4, 1, 1), (4, 2, 2), (5, 1, 1), (5, 2, 1),
                                    (4, 33, 2), (5, 65, 1)])
def test_ragged_shapes(native_lib, oracle_mod, sl, T, N):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(T, N, sl, 40 + T + N), sl, min_identical=1.0)


@pytest.mark.parametrize("sl,C", [(3, 320), (4, 1280), (3, 264)])
def test_wide_rows_keep_the_reference_two_stride_addressing(native_lib, oracle_mod, sl, C):
    # C > 4*ns: scans stride by N*4ns, beam search by N*C, exactly like the CPU decoder
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(120, 5, sl, 60 + C, C=C), sl, min_identical=1.0)


@pytest.mark.parametrize("p_step", [0.15, 0.5])
def test_stay_heavy_paths_merge_duplicates(native_lib, oracle_mod, p_step):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(600, 12, 3, 71, p_step=p_step), 3, min_identical=1.0)
    check(native_lib, oracle_mod, synth.make_scores(400, 6, 4, 72, p_step=p_step), 4, min_identical=1.0)


def test_degenerate_scores(native_lib, oracle_mod):
    # all candidates tie (bisection guess limit, 32-way clamp), and golden-like mostly -5 scores
    z = np.zeros((50, 3, 256), np.float16)
    check(native_lib, oracle_mod, z, 3, min_identical=1.0)
    rng = np.random.default_rng(5)
    s = np.full((400, 4, 256), -5.0, np.float16)
    s[rng.random(s.shape) < 0.3] = 2.0
    check(native_lib, oracle_mod, s, 3, min_identical=1.0)


@pytest.mark.parametrize("sl,scale,shift", [(4, 8.0, 0.0), (4, 1.0, -40.0), (3, 30.0, 0.0), (5, 0.25, 3.0)])
def test_score_ranges_far_from_the_usual(native_lib, oracle_mod, sl, scale, shift):
    # large scores (coarse float grid, everything certified), strongly negative ones (the running
    # scores fall instead of rising), tiny ones (fine grid, the exact routine everywhere)
    from openfish_b200 import synth
    T, N = (500, 4) if sl < 5 else (200, 2)
    s = (synth.make_scores(T, N, sl, 90 + sl).astype(np.float32) * scale + shift).astype(np.float16)
    check(native_lib, oracle_mod, s, sl, min_identical=1.0)


def test_random_shapes_ranges_and_options(native_lib, oracle_mod):
    # seeded differential runs over shapes, score scale/offset, stay-heavy paths, sparse scores
    # and options; every case must meet the full gates with all chunks identical
    from openfish_b200 import synth
    rng = np.random.default_rng(20261)
    for _ in range(60):
        sl = int(rng.choice([3, 3, 4, 4, 4, 5]))
        T = int(rng.integers(1, 900)) if sl < 5 else int(rng.integers(1, 200))
        N = int(rng.integers(1, 7)) if sl < 5 else int(rng.integers(1, 3))
        scale = float(rng.choice([0.05, 0.3, 1, 1, 2, 4, 8, 16, 40]))
        shift = float(rng.choice([-12, -3, 0, 0, 0, 2, 6]))
        okw = dict(beam_cut=float(rng.choice([100.0, 100.0, 3.0, 1e4, 1.01])), q_scale=float(rng.choice([1.0, 0.95])),
                   q_shift=float(rng.choice([0.0, -0.2])))
        s = synth.make_scores(T, N, sl, int(rng.integers(1, 1 << 30)), p_step=float(rng.choice([0.1, 0.5, 0.8, 1.0])))
        s = (s.astype(np.float32) * scale + shift).astype(np.float16)
        if rng.random() < 0.2:
            s[rng.random(s.shape) < 0.35] = np.float16(-5.0 * min(scale, 4))
        check(native_lib, oracle_mod, s, sl, okw, threads=8, min_identical=1.0)


def test_long_chunks(native_lib, oracle_mod):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(5000, 3, 4, 97), 4, min_identical=1.0)
    check(native_lib, oracle_mod, synth.make_scores(6000, 5, 3, 98), 3, min_identical=1.0)


@pytest.mark.parametrize("okw", [dict(beam_cut=0.0), dict(beam_cut=1.5), dict(beam_cut=1e6),
                                 dict(q_scale=0.95, q_shift=-0.2), dict(q_scale=3.0, q_shift=10.0)])
def test_options(native_lib, oracle_mod, okw):
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(300, 6, 4, 81, p_step=0.7), 4, okw, min_identical=1.0)


@pytest.mark.parametrize("okw", [dict(temperature=0.7), dict(temperature=1.6, beam_cut=20.0),
                                 dict(blank_score=1.0), dict(blank_score=3.5, temperature=0.9)])
def test_temperature_and_blank_score(native_lib, oracle_mod, okw):
    # temperature is the reference beam search's score_scale argument (src/beam_search.c:129,233;
    # pinned by the *_temp* fixtures, which the reference itself produced); blank_score also sets
    # the scans' stay score, as in the reference's CUDA launcher (src/decode_cuda.cu:115)
    from openfish_b200 import synth
    check(native_lib, oracle_mod, synth.make_scores(350, 5, 3, 83, p_step=0.7), 3, okw, min_identical=1.0)
    check(native_lib, oracle_mod, synth.make_scores(200, 3, 4, 84, p_step=0.9), 4, okw, min_identical=1.0)


def test_into_and_submit_wait_match_decode_gpu(native_lib):
    import torch
    from openfish_b200 import synth
    of = native_lib
    sc = torch.from_numpy(synth.make_scores(200, 10, 3, 91)).cuda()
    gb = of.gpubuf_init(200, 10, 3)
    base = of.decode_gpu(sc, 3, gpubuf=gb)
    pinned = [torch.zeros((10, 200), dtype=torch.uint8).pin_memory() for _ in range(3)]
    of.decode_into(sc, 3, gb, *pinned)
    pageable = [torch.zeros((10, 200), dtype=torch.uint8) for _ in range(3)]
    of.decode_into(sc, 3, gb, *pageable, wait=False)
    of.decode_wait(gb)
    for k, a, b in zip(("moves", "sequence", "qstring"), pinned, pageable):
        assert np.array_equal(a.numpy(), base[k]) and np.array_equal(b.numpy(), base[k])
    ms = gb.last_decode_ms()
    assert min(ms["bwd_scan"], ms["fwd_scan"], ms["beam_search"], ms["posterior_seq"]) > 0
    assert ms["total"] >= ms["bwd_scan"] + ms["rest"] - 1e-3 and ms["rest"] >= ms["beam_search"]
    # the blocking call timed by itself (the benchmark's figure) covers at least the device time
    assert of.decode_gpu_wall_ms(sc, 3, gb) >= gb.last_decode_ms()["total"]
    gb.free()


def test_decodes_from_several_host_threads_and_in_flight(native_lib):
    # a gpubuf per host thread, as the reference's driver does it (src/main.c:23,207): decodes of
    # different batches running at the same time must not disturb each other; nor must two
    # decodes submitted back to back on two gpubufs from one thread
    import threading
    import torch
    from openfish_b200 import synth
    of = native_lib
    shapes = [(3, 700, 9), (4, 500, 6), (5, 120, 2), (4, 333, 5)]
    sc = [torch.from_numpy(synth.make_scores(T, N, sl, 130 + i)).cuda() for i, (sl, T, N) in enumerate(shapes)]
    alone = [of.decode_gpu(x, sl) for x, (sl, T, N) in zip(sc, shapes)]
    got, errs = [None] * len(shapes), []

    def work(i):
        try:
            torch.cuda.set_device(0)
            sl, T, N = shapes[i]
            gb = of.gpubuf_init(T, N, sl)
            for _ in range(5):
                got[i] = of.decode_gpu(sc[i], sl, gpubuf=gb)
            gb.free()
        except Exception as exc:
            errs.append(exc)

    th = [threading.Thread(target=work, args=(i,)) for i in range(len(shapes))]
    for t in th:
        t.start()
    for t in th:
        t.join()
    assert not errs, errs
    for a, b in zip(alone, got):
        for k in ("moves", "sequence", "qstring"):
            assert np.array_equal(a[k], b[k]), k

    gbs = [of.gpubuf_init(T, N, sl) for sl, T, N in shapes]
    outs = [[torch.zeros((N, T), dtype=torch.uint8).pin_memory() for _ in range(3)] for sl, T, N in shapes]
    for _ in range(3):
        for i, (sl, T, N) in enumerate(shapes):
            of.decode_into(sc[i], sl, gbs[i], *outs[i], wait=False)
        for g in gbs:
            of.decode_wait(g)
    for a, o in zip(alone, outs):
        for k, t in zip(("moves", "sequence", "qstring"), o):
            assert np.array_equal(a[k], t.numpy()), k
    for g in gbs:
        g.free()


def test_submit_on_a_caller_stream_without_a_host_sync(native_lib):
    # scores produced on a non-blocking side stream immediately before the submit, no host
    # synchronisation in between: the decode must still see them (it waits for that stream on the
    # device), and work queued behind stream_wait_decode must not overtake the decode
    import torch
    from openfish_b200 import synth
    of = native_lib
    sl, T, N = 4, 400, 24
    base = torch.from_numpy(synth.make_scores(T, N, sl, 141)).cuda()
    want = of.decode_gpu(base, sl)
    gb = of.gpubuf_init(T, N, sl)
    side = torch.cuda.Stream()  # non-blocking with respect to the legacy default stream
    out = [torch.zeros((N, T), dtype=torch.uint8).pin_memory() for _ in range(3)]
    big = torch.empty((64, 1024, 1024), device="cuda")
    torch.cuda.synchronize()
    for _ in range(3):
        sc = torch.zeros_like(base)
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            for _ in range(20):          # a few milliseconds of work ahead of the producer
                big.normal_()
            sc.copy_(base)               # the scores appear late, on the side stream
            of.decode_into(sc, sl, gb, *out, wait=False, stream=side)
            of.stream_wait_decode(side, gb)
            sc.zero_()                   # queued behind the decode: must not reach it
        of.decode_wait(gb)
        for k, o in zip(("moves", "sequence", "qstring"), out):
            assert np.array_equal(o.numpy(), want[k]), k
    side.synchronize()
    assert float(sc.abs().max()) == 0.0
    gb.free()


def test_a_wait_that_runs_out_reaches_the_host_as_an_error(native_lib):
    # one block waits 1 ms for a barrier nothing completes; the kernel returns, the host reports
    # ERR_DEVICE_WAIT through the same code as a decode's completion, and the gpubuf is fine after
    import torch
    from openfish_b200 import synth
    of = native_lib
    sc = torch.from_numpy(synth.make_scores(150, 4, 3, 151)).cuda()
    gb = of.gpubuf_init(150, 4, 3)
    before = of.decode_gpu(sc, 3, gpubuf=gb)
    assert of.selfcheck_wait(gb, 1000) == 7      # OPENFISH_B200_ERR_DEVICE_WAIT
    assert of.selfcheck_wait(gb, 200) == 7       # and again: the status word was cleared in between
    after = of.decode_gpu(sc, 3, gpubuf=gb)
    for k in before:
        assert np.array_equal(before[k], after[k])
    gb.free()


def test_argument_errors(native_lib):
    import torch
    of = native_lib
    lib = of.lib()
    lib.set_openfish_log_level(0)
    try:
        sc = torch.zeros((20, 4, 256), dtype=torch.float16, device="cuda")
        gb = of.gpubuf_init(20, 4, 3)
        with pytest.raises(of.OpenfishError) as e:
            of.decode_gpu(torch.zeros((21, 4, 256), dtype=torch.float16, device="cuda"), 3, gpubuf=gb)
        assert e.value.status == 3  # shape differs from the gpubuf's
        with pytest.raises(of.OpenfishError) as e:
            of.decode_gpu(sc, 3, options=of.decoder_init(beam_width=16), gpubuf=gb)
        assert e.value.status == 4
        small = of.gpubuf_init(20, 4, 4)
        with pytest.raises(of.OpenfishError) as e:
            of.decode_gpu(sc, 4, gpubuf=small)  # C=256 < 4*256
        assert e.value.status == 2
        small.free()
        # misaligned scores pointer
        flat = torch.zeros(20 * 4 * 256 + 8, dtype=torch.float16, device="cuda")
        out = [C.c_void_p() for _ in range(3)]
        opt = of.decoder_init()
        lib.openfish_decode_gpu(20, 4, 256, flat.data_ptr() + 2, 3, C.byref(opt), gb.ptr, *[C.byref(o) for o in out])
        assert lib.openfish_b200_last_status() == 2 and out[0].value is None
        # a good call still works afterwards
        assert of.decode_gpu(sc, 3, gpubuf=gb)["moves"].shape == (4, 20)
        gb.free()
    finally:
        lib.set_openfish_log_level(4)


def test_full_size_hac_properties_and_parity(native_lib, oracle_mod):
    """BASELINE-sized batch (hac, T=1666, N=512): size-independent properties and oracle parity on
    every chunk (the oracle takes a few seconds for this on a dozen host cores)."""
    import torch
    from openfish_b200 import synth
    of = native_lib
    T, N, sl = 1666, 512, 4
    d = synth.make_scores_device(T, N, sl, 0x0F16, "cuda")
    gb = of.gpubuf_init(T, N, sl)
    a = of.decode_gpu(d, sl, gpubuf=gb)
    bwd_last = gb.tensor("bwd_NTC")[:, T, :]
    assert float(bwd_last.abs().max()) == 0.0
    rows = gb.tensor("post_NTC")[::37].sum(-1)
    assert float((rows - 1).abs().max()) < 1e-4
    b = of.decode_gpu(d, sl, gpubuf=gb)  # same input, same buffers: identical output
    for k in a:
        assert np.array_equal(a[k], b[k])
    lens = a["moves"].sum(1)
    assert (a["moves"][:, 0] == 1).all()
    for n in range(0, N, 17):
        s, q = a["sequence"][n], a["qstring"][n]
        assert set(bytes(s[: lens[n]])) <= set(b"ACGT") and not s[lens[n]:].any() and not q[lens[n]:].any()
        assert q[: lens[n]].min() >= 34 and q[: lens[n]].max() <= 83
    # the oracle on the whole batch, tensors included (backward scores must be bit-identical)
    full = dict(a, bwd=gb.tensor("bwd_NTC").cpu().numpy(), post=gb.tensor("post_NTC").cpu().numpy(),
                **{k: gb.tensor(name).cpu().numpy() for k, name in PER_TIMESTEP})
    gb.free()
    ref = oracle_mod.decode(d.float().cpu().numpy(), sl, nthreads=os.cpu_count() or 8, tensors=True)
    rep = compare(full, ref)
    assert_parity(rep, min_identical=0.999)  # the gate; every chunk has been identical so far
    assert rep["moves_equal"] == N and rep["seq_equal"] == N, rep["mismatches"]
    del full, ref
    # a chunk's result does not depend on its batch: decode a subset alone
    idx = np.arange(3, N, 41)
    sub16 = d[:, torch.from_numpy(idx).cuda(), :].contiguous().cpu().numpy()
    alone = gpu_decode(of, sub16, sl, tensors=False)
    for k in a:
        assert np.array_equal(alone[k], a[k][idx])


@pytest.mark.parametrize("sl,N,seed,piece", [(5, 256, 0x0F17, 64), (3, 1024, 0x0F15, 512)])
def test_full_size_sup_and_fast_parity(native_lib, oracle_mod, sl, N, seed, piece):
    """The other two BASELINE-sized batches at T = 1666 (sup N = 256, fast N = 1024): one decode of
    the whole batch on the GPU, every chunk against the oracle (which takes the batch in pieces to
    bound host memory), same gates as the hac batch."""
    import torch
    from openfish_b200 import synth
    of = native_lib
    T = 1666
    d = synth.make_scores_device(T, N, sl, seed, "cuda")
    gb = of.gpubuf_init(T, N, sl)
    a = of.decode_gpu(d, sl, gpubuf=gb)
    names = (("bwd", "bwd_NTC"), ("post", "post_NTC")) + PER_TIMESTEP
    identical = 0
    for lo in range(0, N, piece):
        hi = min(N, lo + piece)
        got = {k: v[lo:hi] for k, v in a.items()}
        got.update({k: gb.tensor(name)[lo:hi].cpu().numpy() for k, name in names})
        ref = oracle_mod.decode(d[:, lo:hi, :].float().cpu().numpy(), sl, nthreads=os.cpu_count() or 8, tensors=True)
        rep = compare(got, ref)
        assert_parity(rep, min_identical=0.999)
        identical += min(rep["moves_equal"], rep["seq_equal"])
        del got, ref
    gb.free()
    assert identical == N  # every chunk has been identical so far; the gate itself is 99.9 %


@pytest.mark.parametrize("sl,T,N,clamp", [(3, 300, 5, 0.0), (4, 200, 3, 5.0), (5, 60, 1, 0.0), (3, 1, 1, 5.0),
                                          (4, 33, 7, 4.0)])
def test_scores_with_the_blank_column_inside(native_lib, oracle_mod, sl, T, N, clamp):
    """The 5-wide entry point.  ADAPTOR PARITY UNPINNED: the reference has no implementation of this
    layout; the expectation is this library's own definition of it (drop every state's first entry,
    clamp the other four) written in numpy, followed by the pinned oracle decode."""
    import torch
    from openfish_b200 import synth
    of = native_lib
    ns = 4 ** sl
    s4 = synth.make_scores(T, N, sl, 170 + T)           # what the decode should end up seeing (before the clamp)
    rng = np.random.default_rng(T + N)
    s5 = np.empty((T, N, ns, 5), np.float16)
    s5[..., 0] = rng.standard_normal((T, N, ns)).astype(np.float16) * 3   # blank column: must be ignored
    s5[..., 1:] = s4.reshape(T, N, ns, 4)
    want4 = np.clip(s4.astype(np.float32), -clamp, clamp) if clamp > 0 else s4.astype(np.float32)
    ref = oracle_mod.decode(want4, sl, nthreads=4, tensors=True)
    gb = of.gpubuf_init(T, N, sl)
    out = [torch.zeros((N, T), dtype=torch.uint8).pin_memory() for _ in range(3)]
    d5 = torch.from_numpy(s5.reshape(T, N, 5 * ns)).cuda()
    of.decode_5wide_into(d5, sl, gb, *out, clamp=clamp)
    got = {k: o.numpy() for k, o in zip(("moves", "sequence", "qstring"), out)}
    got.update(bwd=gb.tensor("bwd_NTC").cpu().numpy(), post=gb.tensor("post_NTC").cpu().numpy())
    assert_parity(compare(got, ref), min_identical=1.0)
    # and once more on a side stream, the scores written there just before the call
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        late = torch.zeros_like(d5)
        late.copy_(d5)
        of.decode_5wide_into(late, sl, gb, *out, clamp=clamp, stream=side)
    for k, o in zip(("moves", "sequence", "qstring"), out):
        assert np.array_equal(o.numpy(), got[k]), k
    # the strip's device time is reported beside the decode's, and only for a 5-wide call
    assert gb.last_decode_ms()["strip_blank"] > 0.0
    four = torch.from_numpy(np.ascontiguousarray(want4.astype(np.float16))).cuda()
    of.decode_into(four, sl, gb, *out)
    assert gb.last_decode_ms()["strip_blank"] == 0.0
    for k, o in zip(("moves", "sequence", "qstring"), out):
        assert np.array_equal(o.numpy(), got[k]), k
    gb.free()


def test_a_shard_decoded_alone_equals_the_same_chunks_inside_a_larger_batch(native_lib):
    # chunks 8..11 of a job, generated and decoded on their own (what one GPU of several does),
    # against the same chunks decoded as part of the whole 16-chunk batch
    import torch
    from openfish_b200 import synth
    of = native_lib
    sl, T = 4, 700
    whole = synth.make_scores_device(T, 16, sl, 0x0F16, "cuda")
    part = synth.make_scores_device(T, 4, sl, 0x0F16, "cuda", first_chunk=8)
    assert torch.equal(part, whole[:, 8:12])
    a = gpu_decode(of, whole.cpu().numpy(), sl)
    b = gpu_decode(of, part.cpu().numpy(), sl)
    for k in b:
        assert np.array_equal(a[k][8:12], b[k]), k


def test_hardware_approximations_are_within_the_certificates_bounds(native_lib):
    # the certified fp32 log-sum-exp assumes error bounds of ex2.approx and lg2.approx; the library
    # measures both over their whole domains on this GPU
    st, ex2_rel, lg2_abs = native_lib.selfcheck_arith()
    assert st == 0, (st, ex2_rel, lg2_abs)
    assert 0 < ex2_rel <= 2.0 ** -22 and 0 < lg2_abs <= 2.828e-7
