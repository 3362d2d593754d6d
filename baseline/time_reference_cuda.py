#!/usr/bin/env python
"""Times the reference's own CUDA path (its generic kernels compiled for sm_100a by
baseline/Makefile into baseline/_ref/libopenfish_refcuda.so) on the GPU at hand: the secondary
comparator beside the CPU decoder.  NOT PART OF THE PRODUCT; bench.py runs this file as a child
process, so that whatever happens in the reference's code stays out of the benchmark's own
process, and copies the JSON line it prints into its `reference_cuda` key.

    python baseline/time_reference_cuda.py [--skip-decode]

Order: rotary embedding on the encoder's packed QKV tensor (a streaming kernel; its output is
compared with this library's on the same input), then the decode on one chunk (the shape of the
reference's own test vector), then the hac batch of 512 chunks, timing only -- the reference's
CUDA beam search prunes differently from its CPU decoder (no bisection of the threshold,
src/beam_search_cuda.cu:441-460), so its decode output is not a parity target.  Every stage runs
once more only after the stage before it has finished cleanly.
"""
import ctypes as C
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF_SO = os.path.join(ROOT, "baseline", "_ref", "libopenfish_refcuda.so")


class Opt(C.Structure):
    _fields_ = [("beam_width", C.c_size_t), ("beam_cut", C.c_float), ("blank_score", C.c_float),
                ("q_shift", C.c_float), ("q_scale", C.c_float), ("temperature", C.c_float),
                ("move_pad", C.c_bool)]


def main():
    out = {}
    if not os.path.exists(REF_SO):
        print(json.dumps({"unavailable": "baseline/_ref/libopenfish_refcuda.so has not been built (make -C baseline)"}))
        return
    import numpy as np
    import torch
    import openfish_b200 as of
    from openfish_b200 import synth
    ref = C.CDLL(REF_SO)
    ref.set_openfish_log_level(1)
    vp, i = C.c_void_p, C.c_int
    ref.openfish_rotary_emb_gpu.restype = None
    ref.openfish_rotary_emb_gpu.argtypes = [vp, vp, vp] + [i] * 8
    ref.openfish_gpubuf_init.restype = vp
    ref.openfish_gpubuf_init.argtypes = [i, i, i]
    ref.openfish_gpubuf_free.restype = None
    ref.openfish_gpubuf_free.argtypes = [vp]
    ref.openfish_decode_gpu.restype = None
    ref.openfish_decode_gpu.argtypes = [i, i, i, vp, i, C.POINTER(Opt), vp] + [C.POINTER(vp)] * 3
    libc = C.CDLL(None)
    libc.free.argtypes = [vp]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)

    # ---- rotary, BASELINE configuration 4: fp16 [32][1666][3][8][64], Q and K heads in one call
    B, S, H, D = 32, 1666, 8, 64
    half = D // 2
    pos = np.arange(S)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    sin = torch.from_numpy(np.sin(pos).astype(np.float32)).to(dev)
    cos = torch.from_numpy(np.cos(pos).astype(np.float32)).to(dev)
    g = torch.Generator(device=dev).manual_seed(4)
    x0 = torch.randn((B, S, 3, H, D), generator=g, device=dev, dtype=torch.float32).half()
    args = (B, S, 2 * H, D, half, S * 3 * H * D, 3 * H * D, D)
    ours = x0.clone()
    of.rotary_emb_gpu(ours, sin, cos, *args)
    theirs = x0.clone()
    ref.openfish_rotary_emb_gpu(theirs.data_ptr(), sin.data_ptr(), cos.data_ptr(), *args)
    torch.cuda.synchronize()
    diff = (ours.float() - theirs.float()).abs()
    tol = 1e-3 + 1e-3 * theirs.float().abs()
    xs = [x0.clone() for _ in range(4)]  # 655 MB in rotation: no call finds its input in L2
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    times = []
    for r in range(12):
        x = xs[r % 4]
        torch.cuda.synchronize()
        ev[0].record()  # the reference launches on the legacy default stream, torch's current one here
        ref.openfish_rotary_emb_gpu(x.data_ptr(), sin.data_ptr(), cos.data_ptr(), *args)
        ev[1].record()
        torch.cuda.synchronize()
        if r >= 2:
            times.append(ev[0].elapsed_time(ev[1]))
    out["rotary"] = {"shape": "fp16 [32][1666][3][8][64], nheads=16", "ms": float(np.median(times)),
                     "max_abs_diff_vs_this_library": float(diff.max()),
                     "within_1e-3": bool((diff <= tol).all()),
                     "v_untouched": bool(torch.equal(theirs[:, :, 2], x0[:, :, 2]))}
    del xs, ours, theirs, x0, diff, tol
    print(json.dumps(out), file=sys.stderr, flush=True)
    if "--skip-decode" in sys.argv:
        print(json.dumps(out))
        return

    # ---- decode: one chunk first (the shape of the reference's test vector), then the batch
    opt = Opt(32, 100.0, 2.0, 0.0, 1.0, 1.0, False)

    def decode(scores, state_len, reps):
        T, N, Cc = scores.shape
        gb = ref.openfish_gpubuf_init(T, N, state_len)
        wall, bases = [], 0
        for _ in range(reps):
            m, s, q = vp(), vp(), vp()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ref.openfish_decode_gpu(T, N, Cc, scores.data_ptr(), state_len, C.byref(opt), gb, C.byref(m),
                                    C.byref(s), C.byref(q))
            wall.append(1e3 * (time.perf_counter() - t0))
            mv = np.ctypeslib.as_array(C.cast(m, C.POINTER(C.c_uint8)), shape=(N, T))
            bases = int(mv.sum())
            for p in (m, s, q):
                libc.free(p)
        ref.openfish_gpubuf_free(gb)
        return wall, bases

    one = synth.make_scores_device(1666, 1, 3, 0x0F15, dev)
    wall, bases = decode(one, 3, 2)
    out["decode_one_chunk_fast"] = {"T": 1666, "N": 1, "state_len": 3, "wall_ms": min(wall), "bases": bases}
    print(json.dumps(out), file=sys.stderr, flush=True)
    del one
    batch = synth.make_scores_device(1666, 512, 4, 0x0F16, dev)
    wall, bases = decode(batch, 4, 4)
    best = min(wall[1:])
    out["decode_hac_N512"] = {"T": 1666, "N": 512, "state_len": 4, "wall_ms": best,
                              "chunks_per_sec": 512 / (best * 1e-3), "bases": bases,
                              "timing": "wall clock around openfish_decode_gpu (scores resident; it synchronises the "
                                        "device after every kernel and copies the results back), best of 3 after a warm-up",
                              "note": "timing only: its beam search is not the CPU decoder's"}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
