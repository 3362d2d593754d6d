"""Helpers of the GPU parity tests: run a decode through the C ABI, compare with the CPU oracle."""
import numpy as np


def edit_distance(a, b):
    """Levenshtein distance of two byte strings (numpy row DP)."""
    a, b = np.frombuffer(a, np.uint8), np.frombuffer(b, np.uint8)
    prev = np.arange(len(b) + 1)
    for i, ca in enumerate(a, 1):
        cur = np.empty_like(prev)
        cur[0] = i
        sub = prev[:-1] + (b != ca)
        cur[1:] = np.minimum(sub, prev[1:] + 1)
        # insertions need a running minimum
        for j in range(1, len(cur)):
            if cur[j - 1] + 1 < cur[j]:
                cur[j] = cur[j - 1] + 1
        prev = cur
    return int(prev[-1])


def gpu_decode(of, scores16, state_len, options=None, tensors=True):
    """scores16: numpy float16 [T][N][C].  Returns results (+ gpubuf tensors as numpy)."""
    import torch
    T, N, _ = scores16.shape
    d = torch.from_numpy(np.ascontiguousarray(scores16)).cuda()
    gb = of.gpubuf_init(T, N, state_len)
    try:
        out = of.decode_gpu(d, state_len, options=options, gpubuf=gb)
        if tensors:
            for k, name in (("bwd", "bwd_NTC"), ("post", "post_NTC"), ("qual", "qual_data"),
                            ("states", "states"), ("base_probs", "base_probs"),
                            ("total_probs", "total_probs")):
                out[k] = gb.tensor(name).cpu().numpy()
    finally:
        gb.free()
    return out


def sequences(res):
    return [bytes(r[: int(m.sum())]) for r, m in zip(res["sequence"], res["moves"])]


def _close(a, b, rtol, atol):
    """|a - b| <= atol + rtol * |b|, with equal infinities (and paired NaNs) counting as equal."""
    with np.errstate(invalid="ignore"):
        ok = np.abs(a - b) <= atol + rtol * np.abs(b)
    return ok | (a == b) | (np.isnan(a) & np.isnan(b))


def compare(gpu, ref, post_atol=1e-3, post_rtol=1e-3, post_floor=1e-2):
    """Parity report.  Gates: bwd bit-exact; post within post_atol absolutely and within
    post_rtol relatively wherever the reference posterior is at least post_floor; moves and
    sequence identical; qstring within +-1 on chunks whose sequence matches.  On chunks whose
    moves and sequence match, also the per-timestep outputs (src/beam_search.c:441-496, 49-99):
    states (the base at every timestep) identical; qual_data within 1e-3 absolutely;
    total_probs within 1e-3 relatively; base_probs (-10 log10 of e = 1 - base/total, before
    scale and shift) within 1e-3 relatively, or with e itself within 5e-6: where a base is
    nearly certain the subtraction cancels, and what is left of e is the difference between the
    two posteriors (which agree to a few 1e-6, the gate on them being 1e-3) times the exponent
    0.4, so that a Phred value beyond about 40 cannot agree more closely than that."""
    rep = {}
    if "bwd" in gpu and "bwd" in ref:
        rep["bwd_mismatch"] = int((gpu["bwd"] != ref["bwd"]).sum())
        rep["bwd_max_rel"] = float((np.abs(gpu["bwd"] - ref["bwd"]) / np.maximum(np.abs(ref["bwd"]), 1.0)).max())
        d = np.abs(gpu["post"] - ref["post"])
        rep["post_max_abs"] = float(d.max())
        big = ref["post"] >= post_floor
        rep["post_max_rel"] = float((d[big] / ref["post"][big]).max()) if big.any() else 0.0
        rep["post_ok"] = bool(rep["post_max_abs"] <= post_atol and rep["post_max_rel"] <= post_rtol)
    same_moves = (gpu["moves"] == ref["moves"]).all(1)
    same_seq = (gpu["sequence"] == ref["sequence"]).all(1)
    rep["chunks"] = int(len(same_moves))
    rep["moves_equal"] = int(same_moves.sum())
    rep["seq_equal"] = int(same_seq.sum())
    gs, rs = sequences(gpu), sequences(ref)
    rep["mismatches"] = [dict(chunk=int(i), edit_distance=edit_distance(gs[i], rs[i]))
                         for i in np.nonzero(~(same_moves & same_seq))[0]]
    same = same_moves & same_seq
    if "qual" in gpu and "qual" in ref and same.any():
        rep["states_mismatch"] = int((gpu["states"][same] != ref["states"][same]).sum())
        rep["qual_max_abs"] = float(np.abs(gpu["qual"][same] - ref["qual"][same]).max())
        rep["total_probs_bad"] = int((~_close(gpu["total_probs"][same], ref["total_probs"][same], 1e-3, 0.0)).sum())
        gb, rb = gpu["base_probs"][same], ref["base_probs"][same]
        with np.errstate(over="ignore", invalid="ignore"):
            err_close = np.abs(np.power(10.0, -gb.astype(np.float64) / 10) - np.power(10.0, -rb.astype(np.float64) / 10)) <= 5e-6
        rep["base_probs_bad"] = int((~(_close(gb, rb, 1e-3, 0.0) | err_close)).sum())
    if same_seq.any():
        dq = np.abs(gpu["qstring"][same_seq].astype(np.int32) - ref["qstring"][same_seq].astype(np.int32))
        rep["q_max_diff"] = int(dq.max())
        rep["q_frac_diff"] = float((dq > 0).mean())
    else:
        rep["q_max_diff"], rep["q_frac_diff"] = 0, 0.0
    return rep


def assert_parity(rep, min_identical=0.999, exact_bwd=True):
    if "bwd_mismatch" in rep:
        if exact_bwd:
            assert rep["bwd_mismatch"] == 0, rep
        assert rep["bwd_max_rel"] <= 1e-3, rep
        assert rep["post_ok"], rep
    need = int(np.ceil(min_identical * rep["chunks"]))
    assert rep["moves_equal"] >= need and rep["seq_equal"] >= need, rep
    assert rep["q_max_diff"] <= 1, rep
    if "qual_max_abs" in rep:
        assert rep["states_mismatch"] == 0 and rep["qual_max_abs"] <= 1e-3, rep
        assert rep["total_probs_bad"] == 0 and rep["base_probs_bad"] == 0, rep
