"""b200_mla_decode_static: the decode entry point for callers that cannot allocate device memory
when they call (a serving loop with a frozen memory pool, a host without an allocator of its own).
Its scratch is a fixed array inside the library image, so the caller passes inputs and outputs only.

Checked here through the C ABI: same results as b200_mla_decode with a caller-provided workspace,
twice in a row (the array keeps the previous call's contents), and refusal of a problem whose
scratch would not fit.  Collected last on purpose, and valid both alone and after the other tests.
"""
import ctypes

import pytest
import torch

from helpers import assert_close

pytestmark = pytest.mark.gpu


def _args_fp8(pkg, q8, q_scale, kv, kv_indptr, kv_indices, sm_scale, out, total_kv):
    from amd_optimization_challenge_b200._cabi import DecodeArgs, Q_E4M3, KV_E4M3
    codes, scale = kv
    codes = codes.view(torch.uint8).reshape(-1, 576)
    a = DecodeArgs()
    a.batch, a.heads, a.q_len = kv_indptr.numel() - 1, q8.shape[1], 1
    a.q_format, a.kv_format, a.causal, a.page_size, a.impl = Q_E4M3, KV_E4M3, 1, 1, 0
    a.sm_scale = sm_scale
    a.q, a.q_row_stride, a.q_head_stride, a.q_scale = q8.data_ptr(), q8.stride(0), q8.stride(1), q_scale.data_ptr()
    a.kv_codes, a.kv_codes_stride, a.kv_scale, a.num_slots = codes.data_ptr(), codes.stride(0), scale.data_ptr(), codes.shape[0]
    a.kv_indptr, a.kv_indices, a.total_kv_hint = kv_indptr.data_ptr(), kv_indices.data_ptr(), total_kv
    a.out = out.data_ptr()
    return a, (codes,)          # keep the views alive


def test_static_scratch_matches_workspace_entry_point():
    assert torch.cuda.is_available()
    import amd_optimization_challenge_b200 as pkg
    from amd_optimization_challenge_b200._cabi import lib
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for seed, lens in ((41, [4096] * 8), (42, [900, 0, 77, 3000])):       # the second run reuses the dirty scratch
        data = pkg.generate_input(len(lens), 1, max(lens), seed=seed, kv_lens=lens, shuffle_pages=True, formats=("fp8",))
        q, kvd, _, kvp, cfg = data
        q8, qs = pkg.quantize_q_fp8(q)
        want = pkg.mla_decode(q8, qs, "fp8", kvd["fp8"], kvp, sm_scale=cfg["sm_scale"], kv_indices=cfg["kv_indices"],
                              total_kv_hint=sum(lens))
        for _ in range(2):
            got = torch.full_like(want, float("nan"))
            a, keep = _args_fp8(pkg, q8, qs, kvd["fp8"], kvp, cfg["kv_indices"], cfg["sm_scale"], got, sum(lens))
            rc = lib.b200_mla_decode_static(ctypes.byref(a), stream)
            assert rc == 0, lib.b200_mla_last_error().decode()
            torch.cuda.synchronize()
            assert_close(got, want, rtol=2e-2, atol=2e-2, tight=1.5e-2)
            assert torch.equal(got, want)                                  # same kernels, same schedule


def test_static_scratch_refuses_what_does_not_fit():
    from amd_optimization_challenge_b200._cabi import DecodeArgs, lib
    a = DecodeArgs()
    a.batch, a.heads, a.q_len = 128, 128, 1                               # needs ~100 MB of partials
    assert lib.b200_mla_workspace_bytes(128, 128, 1) > (16 << 20)
    assert lib.b200_mla_decode_static(ctypes.byref(a), None) == -5
    msg = lib.b200_mla_last_error().decode()
    assert "built-in scratch" in msg and "b200_mla_decode" in msg
