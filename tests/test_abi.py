"""The C-ABI boundary without a GPU: the library loads, exports every function the public
headers declare, lays its structs out like the reference's header, and follows the reference's
error convention (print and exit) unless told to keep running."""
import ctypes as C
import os
import re
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")
HEADERS = ["openfish/openfish.h", "openfish/openfish_error.h", "openfish_b200.h"]


def declared_functions():
    names = set()
    for h in HEADERS:
        text = open(os.path.join(INC, h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
        for m in re.finditer(r"\b([A-Za-z_]\w*)\s*\(", text):
            if m.group(1) not in ("defined",):
                names.add(m.group(1))
    return sorted(names)


def test_headers_declare_the_reference_entry_points():
    names = declared_functions()
    for f in ("openfish_decode_gpu", "openfish_gpubuf_init", "openfish_gpubuf_free",
              "openfish_rotary_emb_gpu", "openfish_decode_cpu", "openfish_rotary_emb_cpu",
              "get_openfish_log_level", "set_openfish_log_level"):
        assert f in names


def test_library_exports_every_declared_symbol(native_lib):
    lib = native_lib.lib()
    missing = [f for f in declared_functions() if not hasattr(lib, f)]
    assert not missing, missing


def test_struct_layouts_match_the_header(native_lib, tmp_path):
    src = tmp_path / "layout.c"
    src.write_text(textwrap.dedent("""
        #include <stddef.h>
        #include <stdio.h>
        #include "openfish/openfish.h"
        int main(void) {
            openfish_opt_t o = DECODER_INIT;
            printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(openfish_opt_t),
                   offsetof(openfish_opt_t, beam_cut), offsetof(openfish_opt_t, blank_score),
                   offsetof(openfish_opt_t, q_shift), offsetof(openfish_opt_t, q_scale),
                   offsetof(openfish_opt_t, temperature), offsetof(openfish_opt_t, move_pad),
                   sizeof(openfish_gpubuf_t));
            printf("%zu %g %g %g %g %g %d\\n", o.beam_width, o.beam_cut, o.blank_score, o.q_shift,
                   o.q_scale, o.temperature, (int)o.move_pad);
            printf("%d %d\\n", (int)OPENFISH_LOG_OFF, (int)OPENFISH_LOG_TRAC);
            return 0;
        }"""))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", INC, str(src), "-o", str(exe)], check=True)
    text = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout
    l1, l2, l3 = text.splitlines()
    # where a checkout of the reference is at hand, the same probe compiled against ITS header
    # must print the same thing: layouts, DECODER_INIT and the log-level enum are the contract
    ref_inc = os.path.join(os.environ.get("OPENFISH_REF", "/root/reference"), "include")
    if os.path.exists(os.path.join(ref_inc, "openfish", "openfish.h")):
        ref_exe = tmp_path / "layout_ref"
        subprocess.run(["gcc", "-I", ref_inc, str(src), "-o", str(ref_exe)], check=True)
        assert subprocess.run([str(ref_exe)], capture_output=True, text=True, check=True).stdout == text
    O = native_lib.Opt
    assert [int(x) for x in l1.split()] == [C.sizeof(O), O.beam_cut.offset, O.blank_score.offset,
                                            O.q_shift.offset, O.q_scale.offset, O.temperature.offset,
                                            O.move_pad.offset, C.sizeof(native_lib.GpuBufStruct)]
    assert l2.split() == ["32", "100", "2", "0", "1", "1", "0"]
    assert l3.split() == ["0", "6"]
    d = native_lib.decoder_init()
    assert (d.beam_width, d.beam_cut, d.blank_score, d.q_shift, d.q_scale, d.temperature, d.move_pad) == \
        (32, 100.0, 2.0, 0.0, 1.0, 1.0, False)


def test_log_level_roundtrip(native_lib):
    lib = native_lib.lib()
    assert lib.get_openfish_log_level() == 4  # OPENFISH_LOG_VERB, the reference's default
    lib.set_openfish_log_level(1)
    assert lib.get_openfish_log_level() == 1
    lib.set_openfish_log_level(4)


def test_argument_errors_are_reported_not_fatal_in_keep_running_mode(native_lib):
    lib = native_lib.lib()
    assert lib.openfish_b200_get_error_mode() == 1  # the Python mirror switches it on
    lib.set_openfish_log_level(0)
    try:
        assert not lib.openfish_gpubuf_init(0, 4, 3)
        assert lib.openfish_b200_last_status() == 1
        assert not lib.openfish_gpubuf_init(10, 4, 6)
        assert lib.openfish_b200_last_status() == 1
        out = [C.c_void_p(1) for _ in range(3)]
        opt = native_lib.decoder_init()
        lib.openfish_decode_gpu(10, 1, 256, None, 3, C.byref(opt), None, *[C.byref(o) for o in out])
        assert lib.openfish_b200_last_status() == 1 and all(o.value is None for o in out)
        lib.openfish_decode_cpu(10, 1, 256, 1, None, 3, C.byref(opt), *[C.byref(o) for o in out])
        assert lib.openfish_b200_last_status() == 8
        assert b"no CPU decode path" in lib.openfish_b200_error_text()
    finally:
        lib.set_openfish_log_level(4)


def test_default_error_mode_exits_like_the_reference(native_lib):
    code = textwrap.dedent("""
        import ctypes as C
        lib = C.CDLL(%r)
        lib.openfish_gpubuf_init.restype = C.c_void_p
        lib.openfish_gpubuf_init(0, 0, 3)
        print("still alive")
    """ % native_lib.LIB_PATH)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert r.returncode == 1 and "still alive" not in r.stdout
    assert "OPENFISH_ERROR" in r.stderr


def test_no_fallback_without_a_device(native_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    lib = native_lib.lib()
    lib.set_openfish_log_level(0)
    try:
        assert not lib.openfish_gpubuf_init(16, 2, 3)
        assert lib.openfish_b200_last_status() in (5, 6)  # ERR_ALLOC / ERR_CUDA, never a CPU path
    finally:
        lib.set_openfish_log_level(4)


def test_missing_library_fails_loudly(tmp_path):
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        import openfish_b200
        openfish_b200.LIB_PATH = %r
        try:
            openfish_b200.lib()
        except ImportError as e:
            print("ImportError", e)
    """ % (ROOT, str(tmp_path / "nope.so")))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert "ImportError" in r.stdout and "no fallback" in r.stdout
