"""The CPU oracle against the reference: its golden vector, fixtures made by the unmodified
reference decoder, and (when the compiled reference is present) the reference itself live."""
import numpy as np
import pytest

from conftest import FIXTURE_OUTPUTS, SYNTH_CASES, load_golden


def test_reference_golden_vector(oracle_mod):
    # the case the reference's own test/test.sh:26-40 checks, byte for byte
    g = load_golden("ref_fast_chunk")
    opt = oracle_mod.decoder_init(q_scale=0.97, q_shift=-1.8)  # src/main.c:256-258
    out = oracle_mod.decode(g["scores"].astype(np.float32), 3, opt)
    for k in ("moves", "sequence", "qstring"):
        assert np.array_equal(out[k], g[k]), k
    assert out["moves"].sum() == 32 and bytes(out["sequence"][0, :32]) == b"G" * 32


@pytest.mark.parametrize("name", SYNTH_CASES)
def test_fixtures_from_reference(oracle_mod, name):
    g = load_golden("synth_" + name)
    # fixtures whose options carry a temperature were made with it as the reference beam search's
    # score_scale argument
    flags = oracle_mod.TEMPERATURE_SCALES_SCORES if g["options"].get("temperature", 1.0) != 1.0 else 0
    out = oracle_mod.decode(g["scores"].astype(np.float32), g["state_len"],
                            oracle_mod.decoder_init(**g["options"]), tensors=True, nthreads=2, flags=flags)
    for k in FIXTURE_OUTPUTS:
        assert np.array_equal(out[k], g[k], equal_nan=True), (name, k)


def test_crc32c_known_answers(oracle_mod):
    # values probed from the reference's crc32c (src/beam_search.c:103-115)
    assert oracle_mod.crc32c(0x12345678, 0, 32) == 0xFA745634
    assert oracle_mod.crc32c(0xFA745634, 1, 2) == 0x7FE60831


@pytest.mark.parametrize("sl,T,N,seed,p_step", [(3, 1, 1, 1, 1.0), (3, 2, 3, 2, 1.0), (3, 300, 5, 3, 0.4),
                                                 (4, 150, 3, 4, 1.0), (5, 40, 2, 5, 0.7)])
def test_live_against_compiled_reference(oracle_mod, sl, T, N, seed, p_step):
    if not oracle_mod.have_ref():
        pytest.skip("compiled reference (oracle/_ref) not present")
    from openfish_b200 import synth
    sc = synth.make_scores(T, N, sl, seed, p_step=p_step).astype(np.float32)
    a = oracle_mod.decode(sc, sl, tensors=True, nthreads=3)
    b = oracle_mod.ref_decode(sc, sl, nthreads=2)
    t = oracle_mod.ref_scan_tensors(sc, sl)
    for k in b:
        assert np.array_equal(a[k], b[k]), k
    for k in t:
        assert np.array_equal(a[k], t[k]), k


@pytest.mark.parametrize("sl,T,N,seed,scale", [(3, 250, 3, 21, 1.0), (3, 250, 3, 22, 0.6), (4, 120, 2, 23, 1.5),
                                                (5, 30, 1, 24, 0.8)])
def test_per_timestep_outputs_and_score_scale_live(oracle_mod, sl, T, N, seed, scale):
    # states, qual, base_probs, total_probs, and the beam search's score_scale argument, against the
    # reference's own beam_search_cpu / generate_sequence_cpu called piecewise
    if not oracle_mod.have_ref():
        pytest.skip("compiled reference (oracle/_ref) not present")
    from openfish_b200 import synth
    sc = synth.make_scores(T, N, sl, seed, p_step=0.8).astype(np.float32)
    opt = oracle_mod.decoder_init(temperature=scale, q_scale=0.95, q_shift=-0.2)
    a = oracle_mod.decode(sc, sl, opt, tensors=True, nthreads=2, flags=oracle_mod.TEMPERATURE_SCALES_SCORES)
    b = oracle_mod.ref_decode_tensors(sc, sl, opt, score_scale=scale)
    for k in b:
        assert np.array_equal(a[k], b[k], equal_nan=True), k
    # without the flag the temperature is ignored, as the reference's decoder ignores it
    c = oracle_mod.decode(sc, sl, opt, nthreads=2)
    d = oracle_mod.ref_decode(sc, sl, opt, nthreads=2)
    for k in d:
        assert np.array_equal(c[k], d[k]), k


def test_scan_stay_switch(oracle_mod):
    # flags = 0: the scans use the literal 2.0f whatever blank_score says (src/decode_cpu.c:14,56);
    # SCAN_STAY_FROM_OPTIONS: they use blank_score, the reference CUDA launcher's choice
    # (src/decode_cuda.cu:115); at blank_score = 2.0 the two are the same thing
    from openfish_b200 import synth
    sc = synth.make_scores(60, 2, 3, 31).astype(np.float32)
    base = oracle_mod.decode(sc, 3, tensors=True)
    same = oracle_mod.decode(sc, 3, tensors=True, flags=oracle_mod.SCAN_STAY_FROM_OPTIONS)
    assert np.array_equal(base["bwd"], same["bwd"]) and np.array_equal(base["post"], same["post"])
    opt = oracle_mod.decoder_init(blank_score=1.0)
    cpu_like = oracle_mod.decode(sc, 3, opt, tensors=True)
    cuda_like = oracle_mod.decode(sc, 3, opt, tensors=True, flags=oracle_mod.SCAN_STAY_FROM_OPTIONS)
    assert np.array_equal(cpu_like["bwd"], base["bwd"])
    assert not np.array_equal(cuda_like["bwd"], base["bwd"])
    if oracle_mod.have_ref():
        d = oracle_mod.ref_decode(sc, 3, opt)
        for k in d:
            assert np.array_equal(cpu_like[k], d[k]), k


def test_all_equal_scores_ties(oracle_mod):
    # every candidate ties: exercises the guess-limit branch of the threshold bisection
    if not oracle_mod.have_ref():
        pytest.skip("compiled reference (oracle/_ref) not present")
    sc = np.zeros((40, 2, 256), np.float32)
    a = oracle_mod.decode(sc, 3)
    b = oracle_mod.ref_decode(sc, 3)
    for k in b:
        assert np.array_equal(a[k], b[k]), k


def test_threads_do_not_change_results(oracle_mod):
    from openfish_b200 import synth
    sc = synth.make_scores(120, 7, 3, 9).astype(np.float32)
    a = oracle_mod.decode(sc, 3, nthreads=1)
    b = oracle_mod.decode(sc, 3, nthreads=5)
    for k in a:
        assert np.array_equal(a[k], b[k])


def test_rotary_fixture(oracle_mod):
    g = load_golden("rotary_small")
    B, S, _, H, D = g["x"].shape
    y = g["x"].astype(np.float32).copy()
    oracle_mod.rotary(y.reshape(-1), g["sin"], g["cos"], D // 2, S * 3 * H * D, 3 * H * D, D, B, S, 2 * H)
    assert np.array_equal(y, g["out"])
    assert np.array_equal(y[:, :, 2], g["x"].astype(np.float32)[:, :, 2])  # V untouched
