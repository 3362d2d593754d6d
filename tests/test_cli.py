"""The `openfish` command-line driver: the reference's own smoke test (test/test.sh:26-40: run the
tool on the golden score blob, diff moves/sequence/qstring against the stored blobs) and its
debug-build tensor dump, replayed against this library."""
import os
import subprocess

import numpy as np
import pytest

from conftest import load_golden


@pytest.fixture(scope="module")
def cli(native_lib):
    from openfish_b200 import build
    assert os.path.exists(build.CLI), "the driver is built together with the library"
    return build.CLI


def test_usage_and_size_check_need_no_gpu(cli, tmp_path):
    r = subprocess.run([cli], capture_output=True, text=True)
    assert r.returncode == 1 and "Usage:" in r.stderr and "<scores.blob> <BATCH_SIZE> <STATE_LEN>" in r.stderr
    blob = tmp_path / "short.blob"
    blob.write_bytes(b"\0" * 1000)
    r = subprocess.run([cli, str(blob), "1", "3"], capture_output=True, text=True, cwd=tmp_path)
    assert r.returncode == 1 and "needs" in r.stderr
    r = subprocess.run([cli, str(blob), "1", "7"], capture_output=True, text=True, cwd=tmp_path)
    assert r.returncode == 1 and "STATE_LEN" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("elem", ["fp32", "fp16"])
def test_reference_smoke_test(cli, tmp_path, elem):
    g = load_golden("ref_fast_chunk")
    sc = g["scores"] if elem == "fp16" else g["scores"].astype(np.float32)
    sc.tofile(tmp_path / "scores.blob")
    r = subprocess.run([cli, "scores.blob", "1", "3"], capture_output=True, text=True, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert "decode completed in" in r.stderr
    for name in ("moves", "sequence", "qstring"):
        got = np.fromfile(tmp_path / (name + ".blob"), dtype=np.uint8)
        assert np.array_equal(got, g[name].reshape(-1)), name


@pytest.mark.gpu
def test_tensor_dump_matches_the_fixture(cli, tmp_path, oracle_mod):
    g = load_golden("synth_hac")
    T, N, _ = g["scores"].shape
    g["scores"].tofile(tmp_path / "s.blob")
    r = subprocess.run([cli, "s.blob", str(N), "4", "--timesteps", str(T), "--dump", "--batches", "2"],
                       capture_output=True, text=True, cwd=tmp_path)
    assert r.returncode == 0, r.stderr
    assert np.array_equal(np.fromfile(tmp_path / "moves.blob", dtype=np.uint8), g["moves"].reshape(-1))
    assert np.array_equal(np.fromfile(tmp_path / "sequence.blob", dtype=np.uint8), g["sequence"].reshape(-1))
    bwd = np.fromfile(tmp_path / "bwd_NTC.blob", dtype=np.float32).reshape(g["bwd"].shape)
    assert np.array_equal(bwd.view(np.uint32), g["bwd"].view(np.uint32))
    post = np.fromfile(tmp_path / "post_NTC.blob", dtype=np.float32).reshape(g["post"].shape)
    assert np.abs(post - g["post"]).max() <= 1e-3
    # the driver applies the hac quality calibration (q_scale 0.95, q_shift -0.2)
    ref = oracle_mod.decode(g["scores"].astype(np.float32), 4, oracle_mod.decoder_init(q_scale=0.95, q_shift=-0.2))
    q = np.fromfile(tmp_path / "qstring.blob", dtype=np.uint8).reshape(N, T).astype(int)
    assert np.abs(q - ref["qstring"].astype(int)).max() <= 1
    for name, per in (("qual_data", 4), ("base_probs", 1), ("total_probs", 1)):
        assert os.path.getsize(tmp_path / (name + ".blob")) == N * T * per * 4
    # the reference's way of looking at such dumps (test/compare_blob.cpp:49-73): largest and mean
    # absolute difference and number of differing elements against stored tensors
    cmp_bin = os.path.join(os.path.dirname(cli), "compare_blob")
    for name, key, worst in (("bwd_NTC", "bwd", 0.0), ("post_NTC", "post", 1e-3), ("qual_data", "qual", 1e-3),
                             ("total_probs", "total_probs", 1e-3)):
        # (the fixture was decoded with DECODER_INIT; none of these tensors depends on q_scale/q_shift)
        g[key].astype(np.float32).tofile(tmp_path / "want.blob")
        r = subprocess.run([cmp_bin, name + ".blob", "want.blob"], capture_output=True, text=True, cwd=tmp_path)
        assert r.returncode == 0, r.stderr
        max_diff, avg_diff, tens_len, n_diffs = r.stdout.split()
        assert int(tens_len) == g[key].size and "tensor max elem diff by" in r.stderr
        assert float(max_diff) <= worst and float(avg_diff) <= worst, (name, r.stdout)
        if name == "bwd_NTC":
            assert int(n_diffs) == 0
