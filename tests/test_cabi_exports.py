"""The C-ABI library: it builds, loads, exports every symbol the header declares, its argument
struct has the layout the Python binding assumes, and it rejects bad arguments without a GPU."""
import ctypes
import os
import re
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_mla.h")


def _declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_mla_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported(built_lib):
    lib = ctypes.CDLL(built_lib)
    names = _declared_functions()
    assert "b200_mla_decode" in names and "b200_mla_combine" in names
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b200_mla.h but not exported"
    from amd_optimization_challenge_b200 import _cabi
    assert sorted(_cabi.EXPORTS) == sorted(n for n in names)
    assert _cabi.lib.b200_mla_version() >= 1000


def test_struct_layout_matches_header(built_lib, tmp_path):
    from amd_optimization_challenge_b200._cabi import DecodeArgs
    fields = [f[0] for f in DecodeArgs._fields_]
    body = "\n".join('    printf("%s %%zu\\n", offsetof(b200_mla_decode_args, %s));' % (f, f) for f in fields)
    prog = ('#include <stdio.h>\n#include <stddef.h>\n#include "b200_mla.h"\n'
            'int main(void) {\n    printf("%zu\\n", sizeof(b200_mla_decode_args));\n' + body + '\n    return 0;\n}\n')
    c = tmp_path / "layout.c"
    c.write_text(prog)
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(c), "-o", str(exe)], check=True)
    lines = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    assert int(lines[0]) == ctypes.sizeof(DecodeArgs)
    for ln in lines[1:]:
        if ln.strip():
            name, off = ln.split()
            assert getattr(DecodeArgs, name).offset == int(off), name


def test_argument_validation_without_gpu(built_lib):
    from amd_optimization_challenge_b200._cabi import DecodeArgs, lib
    assert lib.b200_mla_decode(None, None) == -1
    a = DecodeArgs()
    assert lib.b200_mla_decode(ctypes.byref(a), None) == -1
    assert b"positive" in lib.b200_mla_last_error()
    a.batch, a.heads, a.q_len = 1, 12, 1
    assert lib.b200_mla_decode(ctypes.byref(a), None) == -2          # heads not a multiple of 16
    a.heads = 16
    a.batch = 100000
    assert lib.b200_mla_decode(ctypes.byref(a), None) == -5
    a.batch = 1
    assert lib.b200_mla_decode(ctypes.byref(a), None) == -1          # null pointers
    assert lib.b200_mla_combine(None, None, 1, 1, 0, 0, None, None, None) == -1
    assert lib.b200_mla_quantize_fp8(None, 8, None, None, None, None) == -1
    assert lib.b200_mla_workspace_bytes(0, 16, 1) == 0
    assert lib.b200_mla_workspace_bytes(32, 16, 1) > 32 * 16 * 512 * 4


def test_package_fails_loudly_without_library(tmp_path):
    """No CPU fallback: with the library absent, touching a library-backed name raises."""
    code = textwrap.dedent(f"""
        import sys, os, shutil
        sys.path.insert(0, {ROOT!r})
        import amd_optimization_challenge_b200._cabi as c
    """)
    pkg = os.path.join(ROOT, "amd_optimization_challenge_b200")
    shadow = tmp_path / "amd_optimization_challenge_b200"
    shadow.mkdir()
    for f in os.listdir(pkg):
        if f.endswith(".py"):
            (shadow / f).write_text(open(os.path.join(pkg, f)).read())
    r = subprocess.run([sys.executable, "-c", "import sys; sys.path.insert(0, %r); import amd_optimization_challenge_b200 as p; p.custom_kernel" % str(tmp_path)],
                       capture_output=True, text=True)
    assert r.returncode != 0 and "libb200mla.so is missing" in r.stderr
    # and a decode call on CPU tensors raises rather than computing anything
    r = subprocess.run([sys.executable, "-c", textwrap.dedent(f"""
        import sys; sys.path.insert(0, {ROOT!r})
        import torch
        from amd_optimization_challenge_b200 import generate_input, custom_kernel
        data = generate_input(1, 1, 8, 0, device="cpu")
        try:
            custom_kernel(data)
        except (RuntimeError, ValueError) as e:
            print("RAISED", e)
    """)], capture_output=True, text=True)
    assert "RAISED" in r.stdout, r.stdout + r.stderr
