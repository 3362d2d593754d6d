"""ctypes front end of the parity checkers.  TEST INFRASTRUCTURE ONLY.

Two checkers live here, neither is part of the product and the product never imports this
package:

* ``liboracle.so``  -- the CPU restatement ``crf_oracle.c`` (always buildable: plain C).
* ``_ref/libopenfish_ref.so`` -- the unmodified reference CPU decoder compiled from its own
  sources by ``make -C oracle ref`` (present only where the reference checkout was available
  at build time; the built library travels with the repository snapshot).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libopenfish_ref.so")


class Opt(C.Structure):
    """Byte-compatible with openfish_opt_t (include/openfish/openfish.h:29-37)."""
    _fields_ = [("beam_width", C.c_size_t), ("beam_cut", C.c_float), ("blank_score", C.c_float),
                ("q_shift", C.c_float), ("q_scale", C.c_float), ("temperature", C.c_float),
                ("move_pad", C.c_bool)]


def decoder_init(**kw):
    """DECODER_INIT (include/openfish/openfish.h:14) with optional overrides."""
    o = Opt(32, 100.0, 2.0, 0.0, 1.0, 1.0, False)
    for k, v in kw.items():
        setattr(o, k, v)
    return o


def build(ref=True):
    """Compile the checkers (the restatement always; the reference when its checkout exists)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    if ref:
        subprocess.run(["make", "-s", "-C", _HERE, "ref"], check=True)


_fp = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_u8 = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
_i32 = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_libs = {}


def _oracle():
    if "o" not in _libs:
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        lib = C.CDLL(ORACLE_SO)
        lib.oracle_decode.restype = C.c_int
        lib.oracle_decode.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _fp, C.c_int,
                                      C.POINTER(Opt), _u8, _u8, _u8, _fp, _fp, _fp, _fp, _fp, _fp]
        lib.oracle_decode_ex.restype = C.c_int
        lib.oracle_decode_ex.argtypes = lib.oracle_decode.argtypes + [_i32, C.c_int]
        lib.oracle_rotary_emb.restype = None
        lib.oracle_rotary_emb.argtypes = [_fp, _fp, _fp, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_long, C.c_long, C.c_long]
        lib.oracle_fold_scores.restype = C.c_float
        lib.oracle_fold_scores.argtypes = [C.c_float, C.c_float]
        lib.oracle_backward_scan.restype = None
        lib.oracle_backward_scan.argtypes = [_fp, _fp, C.c_int, C.c_int, C.c_int, C.c_int]
        lib.oracle_crc32c.restype = C.c_uint32
        lib.oracle_crc32c.argtypes = [C.c_uint32, C.c_uint32, C.c_int]
        _libs["o"] = lib
    return _libs["o"]


def have_ref():
    return os.path.exists(REF_SO)


def _ref():
    if "r" not in _libs:
        lib = C.CDLL(REF_SO)
        lib.set_openfish_log_level(1)
        lib.openfish_decode_cpu.restype = None
        lib.openfish_decode_cpu.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                            C.POINTER(Opt), C.POINTER(C.POINTER(C.c_uint8)),
                                            C.POINTER(C.POINTER(C.c_char)),
                                            C.POINTER(C.POINTER(C.c_char))]
        lib.ref_scan_tensors.restype = None
        lib.ref_scan_tensors.argtypes = [_fp, C.c_int, C.c_int, C.c_int, _fp, _fp, _fp]
        lib.ref_beam_search.restype = None
        lib.ref_beam_search.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int,
                                        C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                        C.c_void_p, C.c_void_p]
        lib.ref_beam_search_scaled.restype = None
        lib.ref_beam_search_scaled.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int,
                                               C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.c_float, C.c_float, C.c_void_p]
        lib.ref_generate_sequence.restype = None
        lib.ref_generate_sequence.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float,
                                              C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p]
        lib.openfish_rotary_emb_cpu.restype = None
        lib.openfish_rotary_emb_cpu.argtypes = [C.c_void_p] * 3 + [C.c_int] * 9
        _libs["r"] = lib
        _libs["libc"] = C.CDLL(None)
        _libs["libc"].free.argtypes = [C.c_void_p]
    return _libs["r"]


def crc32c(crc, bits, nbits):
    return int(_oracle().oracle_crc32c(crc, bits, nbits))


def fold_scores(x, y):
    """The reference's two-term log-sum-exp used when beam elements merge."""
    return float(_oracle().oracle_fold_scores(x, y))


def backward_scan(scores, state_len):
    """bwd [N][T+1][ns] from the restatement's backward scan alone."""
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    T, N, _ = scores.shape
    ns = 4 ** state_len
    out = np.zeros((N, T + 1, ns), np.float32)
    for c in range(N):
        _oracle().oracle_backward_scan(scores, out, c, T, N, ns)
    return out


SCAN_STAY_FROM_OPTIONS = 1      # scans use opt.blank_score, as the reference's CUDA launcher does
TEMPERATURE_SCALES_SCORES = 2   # the beam search's score_scale = opt.temperature


def decode(scores, state_len, opt=None, nthreads=1, tensors=False, flags=0):
    """Restatement decode.  scores: float32 [T][N][C] (fp16 values widened).

    Returns dict(moves, sequence, qstring: uint8 [N][T]) plus, with tensors=True, bwd, fwdbwd,
    post [N][T+1][ns], qual [N][T][4], base_probs, total_probs [N][T] and states int32 [N][T]
    (the base of the path at every timestep).  flags = 0 is the reference CPU decoder's
    behaviour; SCAN_STAY_FROM_OPTIONS and TEMPERATURE_SCALES_SCORES switch on the two places
    where the options reach further than in that decoder."""
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    T, N, Cc = scores.shape
    ns = 4 ** state_len
    opt = opt or decoder_init()
    out = {k: np.zeros((N, T), np.uint8) for k in ("moves", "sequence", "qstring")}
    lib = _oracle()
    if tensors:
        for k in ("bwd", "fwdbwd", "post"):
            out[k] = np.zeros((N, T + 1, ns), np.float32)
        out["qual"] = np.zeros((N, T, 4), np.float32)
        out["base_probs"] = np.zeros((N, T), np.float32)
        out["total_probs"] = np.zeros((N, T), np.float32)
        out["states"] = np.zeros((N, T), np.int32)
        extra = [out[k] for k in ("bwd", "fwdbwd", "post", "qual", "base_probs", "total_probs", "states")]
        rc = lib.oracle_decode_ex(T, N, Cc, nthreads, scores, state_len, C.byref(opt),
                                  out["moves"], out["sequence"], out["qstring"], *extra, flags)
    else:
        fn = lib.oracle_decode_ex
        saved = fn.argtypes
        fn.argtypes = saved[:10] + [C.c_void_p] * 7 + [C.c_int]
        try:
            rc = fn(T, N, Cc, nthreads, scores, state_len, C.byref(opt), out["moves"],
                    out["sequence"], out["qstring"], None, None, None, None, None, None, None, flags)
        finally:
            fn.argtypes = saved
    if rc != 0:
        raise MemoryError("oracle_decode could not allocate")
    return out


def ref_decode(scores, state_len, opt=None, nthreads=1):
    """The unmodified reference's openfish_decode_cpu (src/decode_cpu.c:231)."""
    lib = _ref()
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    T, N, Cc = scores.shape
    opt = opt or decoder_init()
    m, s, q = C.POINTER(C.c_uint8)(), C.POINTER(C.c_char)(), C.POINTER(C.c_char)()
    lib.openfish_decode_cpu(T, N, Cc, nthreads, scores.ctypes.data, state_len, C.byref(opt),
                            C.byref(m), C.byref(s), C.byref(q))
    out = {}
    for k, p in (("moves", m), ("sequence", s), ("qstring", q)):
        out[k] = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(N, T)).copy()
        _libs["libc"].free(C.cast(p, C.c_void_p))
    return out


def ref_decode_tensors(scores, state_len, opt=None, score_scale=1.0, posts_scale=1.0):
    """The reference's decode put together from its own routines one chunk at a time, the way
    src/decode_cpu.c:188-229 does, but keeping every intermediate and with beam_search_cpu's two
    scale arguments open (the reference's decoder passes 1.0f for both): backward_scan,
    forward_scan, softmax, beam_search_cpu, generate_sequence_cpu.  Returns the same keys as
    decode(tensors=True)."""
    lib = _ref()
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    T, N, Cc = scores.shape
    ns = 4 ** state_len
    opt = opt or decoder_init()
    out = ref_scan_tensors(scores, state_len)
    out.update({k: np.zeros((N, T), np.uint8) for k in ("moves", "sequence", "qstring")})
    out["states"] = np.zeros((N, T), np.int32)
    out["qual"] = np.zeros((N, T, 4), np.float32)
    out["base_probs"] = np.zeros((N, T), np.float32)
    out["total_probs"] = np.zeros((N, T), np.float32)
    beam_vector = np.zeros(32 * (T + 1) * 8, np.uint8)
    flat = scores.reshape(-1)
    for c in range(N):
        chunk_scores = flat[c * ns * 4:]
        lib.ref_beam_search_scaled(chunk_scores.ctypes.data, N * Cc, out["bwd"][c].ctypes.data,
                                   out["post"][c].ctypes.data, 2 * state_len, T, opt.beam_cut,
                                   opt.blank_score, out["states"][c].ctypes.data,
                                   out["moves"][c].ctypes.data, out["qual"][c].ctypes.data,
                                   score_scale, posts_scale, beam_vector.ctypes.data)
        lib.ref_generate_sequence(out["moves"][c].ctypes.data, out["states"][c].ctypes.data,
                                  out["qual"][c].ctypes.data, opt.q_shift, opt.q_scale, T,
                                  int(out["moves"][c].sum()), out["base_probs"][c].ctypes.data,
                                  out["total_probs"][c].ctypes.data, out["sequence"][c].ctypes.data,
                                  out["qstring"][c].ctypes.data)
    return out


def ref_scan_tensors(scores, state_len):
    """bwd, fwdbwd, post from the reference's static scan routines (src/decode_cpu.c:13-147)."""
    lib = _ref()
    scores = np.ascontiguousarray(scores, dtype=np.float32)
    T, N, _ = scores.shape
    ns = 4 ** state_len
    t = [np.zeros((N, T + 1, ns), np.float32) for _ in range(3)]
    lib.ref_scan_tensors(scores, T, N, state_len, *t)
    return dict(bwd=t[0], fwdbwd=t[1], post=t[2])


def rotary(x, sin, cos, rotary_half, stride_batch, stride_seq, stride_head, batch, seqlen, nheads):
    """Restatement rotary embedding, in place on float32 x (flat)."""
    _oracle().oracle_rotary_emb(x, np.ascontiguousarray(sin, np.float32),
                                np.ascontiguousarray(cos, np.float32), batch, seqlen, nheads,
                                rotary_half, stride_batch, stride_seq, stride_head)
    return x


def ref_rotary(x, sin, cos, rotary_half, stride_batch, stride_seq, stride_head, batch, seqlen,
               nheads, nthreads=1):
    """The reference's openfish_rotary_emb_cpu (src/nn_cpu.c:80), in place on float32 x."""
    sin = np.ascontiguousarray(sin, np.float32)
    cos = np.ascontiguousarray(cos, np.float32)
    _ref().openfish_rotary_emb_cpu(x.ctypes.data, sin.ctypes.data, cos.ctypes.data, batch, seqlen,
                                   nheads, 2 * rotary_half, rotary_half, stride_batch, stride_seq,
                                   stride_head, nthreads)
    return x
