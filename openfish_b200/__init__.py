"""openfish_b200 -- Python mirror of the openfish C API, backed by ``lib/libopenfish.so``.

The functions carry the reference's names and argument meaning (include/openfish/openfish.h):
``gpubuf_init`` / ``gpubuf_free`` / ``decode_gpu`` / ``rotary_emb_gpu``.  Everything goes
through the C ABI with plain device pointers; torch is used only to own device memory.  There
is no CPU fallback: if the shared library is missing or cannot be loaded the import of this
module's native half raises.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("OPENFISH_B200_LIB") or os.path.join(_HERE, "lib", "libopenfish.so")

STATUS_NAMES = ["OK", "ERR_ARGUMENT", "ERR_LAYOUT", "ERR_SHAPE", "ERR_OPTION", "ERR_ALLOC",
                "ERR_CUDA", "ERR_DEVICE_WAIT", "ERR_NO_CPU_PATH", "ERR_TOO_LONG", "ERR_SCRATCH_LIMIT",
                "ERR_ARITH"]
STATIC_SCRATCH_BYTES = 48 << 20


class OpenfishError(RuntimeError):
    def __init__(self, status, text):
        super().__init__("%s: %s" % (STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else status, text))
        self.status = status


class Opt(C.Structure):
    """openfish_opt_t (include/openfish/openfish.h)."""
    _fields_ = [("beam_width", C.c_size_t), ("beam_cut", C.c_float), ("blank_score", C.c_float),
                ("q_shift", C.c_float), ("q_scale", C.c_float), ("temperature", C.c_float),
                ("move_pad", C.c_bool)]


class GpuBufStruct(C.Structure):
    """openfish_gpubuf_t (include/openfish/openfish.h): ten device pointers."""
    _fields_ = [(n, C.c_void_p) for n in ("bwd_NTC", "post_NTC", "moves", "sequence", "qstring",
                                          "beam_vector", "states", "qual_data", "base_probs",
                                          "total_probs")]


def decoder_init(**overrides):
    """DECODER_INIT with optional field overrides."""
    o = Opt(32, 100.0, 2.0, 0.0, 1.0, 1.0, False)
    for k, v in overrides.items():
        setattr(o, k, v)
    return o


# q_scale / q_shift the reference's driver applies per model (src/main.c:256-265)
MODEL_QSCORE = {3: dict(q_scale=0.97, q_shift=-1.8), 4: dict(q_scale=0.95, q_shift=-0.2),
                5: dict(q_scale=0.95, q_shift=0.5)}

_lib = None


def lib():
    """The loaded shared library (raises if it is absent: there is no other implementation)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s not found: build it with `python -m openfish_b200.build` "
                              "(needs nvcc); openfish_b200 has no fallback path" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        vp, i = C.c_void_p, C.c_int
        L.openfish_gpubuf_init.restype = C.POINTER(GpuBufStruct)
        L.openfish_gpubuf_init.argtypes = [i, i, i]
        L.openfish_gpubuf_free.restype = None
        L.openfish_gpubuf_free.argtypes = [C.POINTER(GpuBufStruct)]
        dec = [i, i, i, vp, i, C.POINTER(Opt), C.POINTER(GpuBufStruct)]
        L.openfish_decode_gpu.restype = None
        L.openfish_decode_gpu.argtypes = dec + [C.POINTER(vp)] * 3
        for name in ("openfish_b200_decode_into", "openfish_b200_decode_submit"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = dec + [vp] * 3
        L.openfish_b200_decode_submit_on.restype = None
        L.openfish_b200_decode_submit_on.argtypes = [vp] + dec + [vp] * 3
        L.openfish_b200_decode_submit_5wide.restype = None
        L.openfish_b200_decode_submit_5wide.argtypes = [vp, i, i, vp, i, C.POINTER(Opt), C.c_float,
                                                        C.POINTER(GpuBufStruct)] + [vp] * 3
        L.openfish_b200_stream_wait_decode.restype = None
        L.openfish_b200_stream_wait_decode.argtypes = [vp, C.POINTER(GpuBufStruct)]
        L.openfish_b200_selfcheck_wait.restype = i
        L.openfish_b200_selfcheck_wait.argtypes = [C.POINTER(GpuBufStruct), C.c_uint]
        L.openfish_b200_decode_wait.restype = None
        L.openfish_b200_decode_wait.argtypes = [C.POINTER(GpuBufStruct)]
        L.openfish_rotary_emb_gpu.restype = None
        L.openfish_rotary_emb_gpu.argtypes = [vp, vp, vp] + [i] * 8
        L.openfish_decode_cpu.restype = None
        L.openfish_decode_cpu.argtypes = [i, i, i, i, vp, i, C.POINTER(Opt)] + [C.POINTER(vp)] * 3
        for name in ("openfish_b200_last_decode_ms", "openfish_b200_last_decode_detail_ms"):
            getattr(L, name).restype = None
            getattr(L, name).argtypes = [C.POINTER(GpuBufStruct), C.POINTER(C.c_float)]
        L.openfish_b200_last_status.restype = i
        L.openfish_b200_error_text.restype = C.c_char_p
        L.openfish_b200_set_error_mode.argtypes = [i]
        L.openfish_b200_kernels_per_decode.restype = i
        L.openfish_b200_last_rotary_ms.restype = C.c_float
        L.openfish_b200_selfcheck_arith.restype = i
        L.openfish_b200_selfcheck_arith.argtypes = [C.POINTER(C.c_double)]
        L.openfish_b200_decode_static.restype = i
        L.openfish_b200_decode_static.argtypes = [i, i, i, vp, i, C.POINTER(Opt), vp, vp, vp]
        L.get_openfish_log_level.restype = i
        L.set_openfish_log_level.argtypes = [i]
        # Python callers get exceptions instead of the reference's exit(1)
        L.openfish_b200_set_error_mode(1)
        L.libc_free = C.CDLL(None).free
        L.libc_free.argtypes = [vp]
        _lib = L
    return _lib


def _check():
    st = lib().openfish_b200_last_status()
    if st != 0:
        raise OpenfishError(st, lib().openfish_b200_error_text().decode())


class _DevView:
    """Zero-copy window on device memory for torch.as_tensor (CUDA array interface)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape),
                                         "typestr": typestr, "version": 2}


class GpuBuf:
    """Device buffers for decodes of one shape; mirrors openfish_gpubuf_t's fields as torch
    tensors (views, not copies)."""

    def __init__(self, T, N, state_len):
        self.T, self.N, self.state_len = T, N, state_len
        self.ptr = lib().openfish_gpubuf_init(T, N, state_len)
        _check()

    def free(self):
        if self.ptr:
            lib().openfish_gpubuf_free(self.ptr)
            self.ptr = None
            _check()

    def tensor(self, name):
        import torch
        T, N, ns = self.T, self.N, 4 ** self.state_len
        spec = {"bwd_NTC": ((N, T + 1, ns), "<f4"), "post_NTC": ((N, T + 1, ns), "<f4"),
                "moves": ((N, T), "|u1"), "sequence": ((N, T), "|u1"), "qstring": ((N, T), "|u1"),
                "beam_vector": ((N, T + 1, 32), "|u1"), "states": ((N, T), "<i4"),
                "qual_data": ((N, T, 4), "<f4"), "base_probs": ((N, T), "<f4"),
                "total_probs": ((N, T), "<f4")}[name]
        return torch.as_tensor(_DevView(getattr(self.ptr.contents, name), *spec), device="cuda")

    def last_decode_ms(self):
        ms = (C.c_float * 8)()
        lib().openfish_b200_last_decode_detail_ms(self.ptr, ms)
        return dict(bwd_scan=ms[0], rest=ms[1], d2h=ms[2], total=ms[3], beam_search=ms[4],
                    fwd_scan=ms[5], posterior_seq=ms[6], strip_blank=ms[7])


def gpubuf_init(T, N, state_len):
    return GpuBuf(T, N, state_len)


def gpubuf_free(gpubuf):
    gpubuf.free()


def _scores_args(scores_TNC, state_len, options, gpubuf):
    import torch
    if not (isinstance(scores_TNC, torch.Tensor) and scores_TNC.is_cuda
            and scores_TNC.dtype == torch.float16 and scores_TNC.is_contiguous()
            and scores_TNC.dim() == 3):
        raise TypeError("scores_TNC must be a contiguous CUDA float16 tensor [T][N][C]")
    T, N, Cc = scores_TNC.shape
    return (T, N, Cc, scores_TNC.data_ptr(), state_len, C.byref(options or decoder_init()), gpubuf.ptr)


def decode_gpu(scores_TNC, state_len, options=None, gpubuf=None):
    """openfish_decode_gpu: returns dict(moves, sequence, qstring) of uint8 arrays [N][T]
    (copies of the library's malloc'ed results, which are freed here)."""
    own = gpubuf is None
    if own:
        gpubuf = GpuBuf(scores_TNC.shape[0], scores_TNC.shape[1], state_len)
    try:
        args = _scores_args(scores_TNC, state_len, options, gpubuf)
        out = [C.c_void_p() for _ in range(3)]
        lib().openfish_decode_gpu(*args, *[C.byref(o) for o in out])
        _check()
        T, N = args[0], args[1]
        res = {}
        for k, p in zip(("moves", "sequence", "qstring"), out):
            res[k] = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(N, T)).copy()
            lib().libc_free(p)
        return res
    finally:
        if own:
            gpubuf.free()


def decode_gpu_wall_ms(scores_TNC, state_len, gpubuf, options=None):
    """Wall-clock milliseconds of one openfish_decode_gpu call by itself (what the reference's driver
    times, src/main.c:271-303): the clock runs around the C call only; the malloc'ed results are
    freed afterwards without being copied into Python objects."""
    import time
    args = _scores_args(scores_TNC, state_len, options, gpubuf)
    out = [C.c_void_p() for _ in range(3)]
    refs = [C.byref(o) for o in out]
    fn = lib().openfish_decode_gpu
    t0 = time.perf_counter()
    fn(*args, *refs)
    ms = 1e3 * (time.perf_counter() - t0)
    _check()
    for p in out:
        lib().libc_free(p)
    return ms


def decode_into(scores_TNC, state_len, gpubuf, moves, sequence, qstring, options=None, wait=True, stream=None):
    """openfish_b200_decode_into / _submit / _submit_on: results into caller-owned uint8 host
    tensors [N][T] (torch, ideally pinned).  With wait=False call decode_wait(gpubuf) afterwards.
    stream (a torch.cuda.Stream, implies wait=False): the stream the scores were produced on; the
    decode is ordered after the work queued on it."""
    args = _scores_args(scores_TNC, state_len, options, gpubuf)
    out = (moves.data_ptr(), sequence.data_ptr(), qstring.data_ptr())
    if stream is not None:
        lib().openfish_b200_decode_submit_on(stream.cuda_stream, *args, *out)
    else:
        fn = lib().openfish_b200_decode_into if wait else lib().openfish_b200_decode_submit
        fn(*args, *out)
    _check()


def decode_5wide_into(scores_TN5, state_len, gpubuf, moves, sequence, qstring, options=None, clamp=0.0,
                      stream=None):
    """openfish_b200_decode_submit_5wide + _wait: scores [T][N][5*4^state_len] (stay score first in
    every state's five entries), results into caller-owned uint8 host tensors [N][T]."""
    import torch
    if not (isinstance(scores_TN5, torch.Tensor) and scores_TN5.is_cuda and scores_TN5.dtype == torch.float16
            and scores_TN5.is_contiguous() and scores_TN5.dim() == 3
            and scores_TN5.shape[2] == 5 * 4 ** state_len):
        raise TypeError("scores_TN5 must be a contiguous CUDA float16 tensor [T][N][5*4^state_len]")
    T, N, _ = scores_TN5.shape
    lib().openfish_b200_decode_submit_5wide(stream.cuda_stream if stream is not None else None, T, N,
                                            scores_TN5.data_ptr(), state_len, C.byref(options or decoder_init()),
                                            clamp, gpubuf.ptr, moves.data_ptr(), sequence.data_ptr(),
                                            qstring.data_ptr())
    _check()
    decode_wait(gpubuf)


def stream_wait_decode(stream, gpubuf):
    """openfish_b200_stream_wait_decode: work queued on `stream` from now on runs after the
    gpubuf's decode in flight."""
    lib().openfish_b200_stream_wait_decode(stream.cuda_stream, gpubuf.ptr)
    _check()


def selfcheck_wait(gpubuf, limit_us=1000):
    """openfish_b200_selfcheck_wait: the status code (ERR_DEVICE_WAIT = 7 when the path from a
    kernel's wait that ran out to the host's error works)."""
    return int(lib().openfish_b200_selfcheck_wait(gpubuf.ptr, limit_us))


def decode_static(scores_TNC, state_len, moves_gpu, sequence_gpu, qstring_gpu, options=None):
    """openfish_b200_decode_static: the decode that allocates nothing.  Results go to three
    caller-owned CUDA uint8 tensors [N][T]; intermediates live in the library's fixed device
    array, so the shape must fit OPENFISH_B200_STATIC_SCRATCH_BYTES.  Returns the status code
    (0 = OK) instead of raising, like the C entry point."""
    T, N, Cc = scores_TNC.shape
    return lib().openfish_b200_decode_static(T, N, Cc, scores_TNC.data_ptr(), state_len,
                                             C.byref(options or decoder_init()),
                                             moves_gpu.data_ptr(), sequence_gpu.data_ptr(),
                                             qstring_gpu.data_ptr())


def decode_wait(gpubuf):
    lib().openfish_b200_decode_wait(gpubuf.ptr)
    _check()


def rotary_emb_gpu(x_gpu, sin_gpu, cos_gpu, batch_size, seqlen, nheads, head_dim, rotary_half,
                   stride_batch, stride_seq, stride_head):
    """openfish_rotary_emb_gpu on torch CUDA tensors (x float16 in place, sin/cos float32)."""
    lib().openfish_rotary_emb_gpu(x_gpu.data_ptr(), sin_gpu.data_ptr(), cos_gpu.data_ptr(),
                                  batch_size, seqlen, nheads, head_dim, rotary_half, stride_batch,
                                  stride_seq, stride_head)
    _check()


def selfcheck_arith():
    """openfish_b200_selfcheck_arith: (status, ex2 relative error, lg2 absolute error) measured on
    the current GPU."""
    err = (C.c_double * 2)()
    st = lib().openfish_b200_selfcheck_arith(err)
    return st, err[0], err[1]


def last_rotary_ms():
    """Device time of this thread's last rotary_emb_gpu call."""
    return float(lib().openfish_b200_last_rotary_ms())


from .sharding import shard_range  # noqa: E402,F401
