"""openfish_b200_decode_static, the decode for callers that cannot allocate once they run (a
server whose own arena owns all device memory, a steady-state pipeline that must not meet
cudaMalloc's device-wide synchronisation): called through the C ABI and compared with the
regular entry point.  Collected last on purpose (file name), so a run that stops at the first
failure has already been through every other test; it passes alone in a fresh process as well
as after the others, because the entry point sets its static scratch up itself on first use and
clears what must start from zero on every call."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def both_ways(of, sc16, sl, okw):
    import torch
    T, N, _ = sc16.shape
    d = torch.from_numpy(sc16).cuda()
    opt = of.decoder_init(**okw)
    want = of.decode_gpu(d, sl, options=opt)
    out = [torch.full((N, T), 7, dtype=torch.uint8, device="cuda") for _ in range(3)]
    rc = of.decode_static(d, sl, *out, options=opt)
    assert rc == 0
    return want, {k: o.cpu().numpy() for k, o in zip(("moves", "sequence", "qstring"), out)}


def test_static_scratch_decode_matches_regular_decode_twice_in_a_row(native_lib):
    from openfish_b200 import synth
    of = native_lib
    # two calls in a row on different inputs and shapes: the second must not see the first's leftovers
    for sl, T, N, seed, okw in ((3, 400, 6, 11, {}), (4, 150, 3, 12, dict(q_scale=0.95, q_shift=-0.2)),
                                (3, 400, 6, 13, dict(beam_cut=10.0))):
        want, got = both_ways(of, synth.make_scores(T, N, sl, seed, p_step=0.7), sl, okw)
        for k in want:  # same kernels, same arithmetic: byte-identical, the tightest of our tolerances
            assert np.array_equal(want[k], got[k]), (sl, T, N, k)


def test_static_scratch_limit_and_bad_arguments_are_refused(native_lib):
    import torch
    of = native_lib
    lib = of.lib()
    lib.set_openfish_log_level(0)
    try:
        T, N, sl = 1666, 64, 4   # needs ~220 MB of intermediates: far beyond the 48 MiB array
        need = 3 * N * (T + 1) * 4 ** sl * 4
        assert need > of.STATIC_SCRATCH_BYTES
        sc = torch.zeros((T, N, 1024), dtype=torch.float16, device="cuda")
        out = [torch.zeros((N, T), dtype=torch.uint8, device="cuda") for _ in range(3)]
        assert of.decode_static(sc, sl, *out) == 10       # ERR_SCRATCH_LIMIT
        small = torch.zeros((10, 2, 256), dtype=torch.float16, device="cuda")
        o2 = [torch.zeros((2, 10), dtype=torch.uint8, device="cuda") for _ in range(3)]
        assert of.decode_static(small, 3, *o2, options=of.decoder_init(beam_width=8)) == 4
        assert of.decode_static(small, 4, *o2) == 2        # C too small for 256 states
        assert of.decode_static(small, 3, *o2) == 0
    finally:
        lib.set_openfish_log_level(4)
