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
    """Size and every field offset of the three argument structs: the C header against the ctypes mirror."""
    from amd_optimization_challenge_b200._cabi import DecodeArgs, KvAppendArgs, PeerMergeArgs
    pairs = (("b200_mla_decode_args", DecodeArgs), ("b200_mla_kv_append_args", KvAppendArgs),
             ("b200_mla_peer_merge_args", PeerMergeArgs))
    body = ""
    for cname, cls in pairs:
        body += '    printf("%s %%zu\\n", sizeof(%s));\n' % (cname, cname)
        for f in cls._fields_:
            body += '    printf("%s.%s %%zu\\n", offsetof(%s, %s));\n' % (cname, f[0], cname, f[0])
    prog = ('#include <stdio.h>\n#include <stddef.h>\n#include "b200_mla.h"\nint main(void) {\n' + body + '    return 0;\n}\n')
    c = tmp_path / "layout.c"
    c.write_text(prog)
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(c), "-o", str(exe)], check=True)
    got = dict(ln.split() for ln in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n") if ln.strip())
    for cname, cls in pairs:
        assert int(got[cname]) == ctypes.sizeof(cls), cname
        for f in cls._fields_:
            assert getattr(cls, f[0]).offset == int(got[f"{cname}.{f[0]}"]), f"{cname}.{f[0]}"


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
    # peer-memory entry points: layout arithmetic and the checks that run before any CUDA call
    from amd_optimization_challenge_b200._cabi import PeerMergeArgs
    part = (256 * 513 * 4 + 255) // 256 * 256
    assert lib.b200_mla_peer_exchange_bytes(256) == 256 + 2 * part and lib.b200_mla_peer_exchange_bytes(0) == 0
    assert lib.b200_mla_peer_partial_offset(256, 2) == 256 and lib.b200_mla_peer_partial_offset(256, 3) == 256 + part
    assert lib.b200_mla_peer_merge(None, None) == -1
    m = PeerMergeArgs(world=3, rank=0, epoch=1, rows=16)
    assert lib.b200_mla_peer_merge(ctypes.byref(m), None) == -2 and b"world" in lib.b200_mla_last_error()
    m.world, m.rank = 2, 2
    assert lib.b200_mla_peer_merge(ctypes.byref(m), None) == -1
    m.rank, m.epoch = 1, 0
    assert lib.b200_mla_peer_merge(ctypes.byref(m), None) == -1 and b"epoch" in lib.b200_mla_last_error()
    m.epoch = 1
    assert lib.b200_mla_peer_merge(ctypes.byref(m), None) == -1          # bases and out are NULL
    assert lib.b200_mla_peer_alloc(0, None, None) == -1 and lib.b200_mla_peer_open(None, None) == -1
    assert lib.b200_mla_peer_close(None) == 0 and lib.b200_mla_peer_free(None) == 0


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
