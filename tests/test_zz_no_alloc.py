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
                                (3, 400, 6, 13, dict(beam_cut=10.0)), (5, 150, 1, 14, {}), (3, 1, 1, 15, {}),
                                (3, 2, 3, 16, {}), (3, 77, 5, 17, {}), (4, 2, 1, 18, {})):
        want, got = both_ways(of, synth.make_scores(T, N, sl, seed, p_step=0.7), sl, okw)
        for k in want:  # same kernels, same arithmetic: byte-identical, the tightest of our tolerances
            assert np.array_equal(want[k], got[k]), (sl, T, N, k)


def test_static_scratch_decode_against_the_oracle_and_without_allocating(native_lib, oracle_mod):
    import torch
    from openfish_b200 import synth
    of = native_lib
    sl, T, N = 4, 300, 4
    sc = synth.make_scores(T, N, sl, 19)
    d = torch.from_numpy(sc).cuda()
    out = [torch.zeros((N, T), dtype=torch.uint8, device="cuda") for _ in range(3)]
    assert of.decode_static(d, sl, *out) == 0          # first call: sets the scratch up
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]          # cudaMemGetInfo: free bytes on the device
    assert of.decode_static(d, sl, *out) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before  # nothing was allocated (or released)
    ref = oracle_mod.decode(sc.astype(np.float32), sl, nthreads=4)
    for k, o in zip(("moves", "sequence"), out):
        assert np.array_equal(o.cpu().numpy(), ref[k]), k
    assert np.abs(out[2].cpu().numpy().astype(int) - ref["qstring"].astype(int)).max() <= 1


@pytest.mark.parametrize("sl,n_fits", [(3, 36), (4, 14)])
def test_static_scratch_documented_limits(native_lib, sl, n_fits):
    # T = 1666: the largest batch the header documents is accepted, one chunk more is refused
    import torch
    of = native_lib
    lib = of.lib()
    T = 1666
    d = torch.zeros((T, n_fits + 1, 4 * 4 ** sl), dtype=torch.float16, device="cuda")
    d.normal_(generator=torch.Generator(device="cuda").manual_seed(5))
    out = [torch.zeros((n_fits + 1, T), dtype=torch.uint8, device="cuda") for _ in range(3)]
    lib.set_openfish_log_level(0)
    try:
        assert of.decode_static(d, sl, *out) == 10     # ERR_SCRATCH_LIMIT
    finally:
        lib.set_openfish_log_level(4)
    fits = d[:, :n_fits, :].contiguous()
    assert of.decode_static(fits, sl, *[o[:n_fits] for o in out]) == 0
    want = of.decode_gpu(fits, sl)
    for k, o in zip(("moves", "sequence", "qstring"), out):
        assert np.array_equal(o[:n_fits].cpu().numpy(), want[k]), k


def test_static_scratch_limit_and_bad_arguments_are_refused(native_lib):
    import torch
    of = native_lib
    lib = of.lib()
    lib.set_openfish_log_level(0)
    try:
        T, N, sl = 1666, 64, 4   # needs ~220 MB of intermediates: far beyond the 48 MiB array
        need = 2 * N * (T + 1) * 4 ** sl * 4
        assert need > of.STATIC_SCRATCH_BYTES
        sc = torch.zeros((T, N, 1024), dtype=torch.float16, device="cuda")
        out = [torch.zeros((N, T), dtype=torch.uint8, device="cuda") for _ in range(3)]
        assert of.decode_static(sc, sl, *out) == 10       # ERR_SCRATCH_LIMIT
        small = torch.zeros((10, 2, 256), dtype=torch.float16, device="cuda")
        o2 = [torch.zeros((2, 10), dtype=torch.uint8, device="cuda") for _ in range(3)]
        assert of.decode_static(small, 3, *o2, options=of.decoder_init(beam_width=8)) == 4
        assert of.decode_static(small, 4, *o2) == 2        # C too small for 256 states
        # a negative C is refused on the host like any other bad layout (nothing is launched)
        opt = of.decoder_init()
        import ctypes
        assert lib.openfish_b200_decode_static(10, 2, -8, small.data_ptr(), 3, ctypes.byref(opt),
                                               o2[0].data_ptr(), o2[1].data_ptr(), o2[2].data_ptr()) == 2
        assert of.decode_static(small, 3, *o2) == 0
    finally:
        lib.set_openfish_log_level(4)
