"""The fused signal + wait + merge kernel of the cross-GPU split-KV mode (csrc/peer_merge.cu) on ONE GPU.

Kernels that wait on one another must not share a GPU, so no second rank runs here: the test plays the peers on
the host.  It owns all `world` exchange allocations (plain allocations of the same process instead of mapped
ones), writes the peers' partials and their "ready" flags itself BEFORE the launch, and runs the merge as rank 0:
the wait finds every flag set.  Checked: the merged rows against b200_mla_combine and the oracle's merge, that the
signal of rank 0 landed in every allocation, both partial buffers (odd and even steps), and the bounded wait - a
flag nobody sets makes the kernel return in time with the TIMEOUT bit and the missing peer merged with weight 0.
"""
import ctypes
import time

import pytest
import torch

from oracle import mla_oracle as mo

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from amd_optimization_challenge_b200 import _cabi, distributed, submission
    return _cabi, distributed, submission


def _alloc(backend, world, n_rows):
    return [backend.alloc(n_rows)[0] for _ in range(world)]


def _fill(backend, base, n_rows, epoch, o, lse):
    ptr = base + backend.partial_offset(n_rows, epoch)
    buf = backend.floats(ptr, n_rows * 513)
    buf[: n_rows * 512].copy_(o.reshape(-1))
    buf[n_rows * 512:].copy_(lse.reshape(-1))


def _flags(backend, base):
    return backend.floats(base, 64).view(torch.int32)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_merge_reads_every_allocation_and_signals_every_peer(env, world):
    _cabi, D, sub = env
    be = D.CudaPeerBackend("cuda")
    n_rows = 3 * 16
    bases = _alloc(be, world, n_rows)
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    try:
        g = torch.Generator().manual_seed(world)
        for epoch in (1, 2, 3):
            o = torch.randn(world, n_rows, 512, generator=g).cuda()
            lse = (torch.randn(world, n_rows, generator=g) * 3).cuda()
            if world > 1:
                lse[1, 0] = float("-inf")                            # an empty part
                lse[:, 1] = float("-inf")                            # a row empty everywhere: zeros
            for r in range(world):
                _fill(be, bases[r], n_rows, epoch, o[r], lse[r])
                _flags(be, bases[0])[r] = epoch                      # the peers' signals, set by the host
            out = be.merge(bases, 0, epoch, n_rows, 200, workspace=ws)
            torch.cuda.synchronize()
            ref = sub.combine_partials(o.view(world, n_rows, 1, 512), lse.view(world, n_rows, 1)).view(n_rows, 512)
            assert torch.equal(out, ref)
            cpu, _ = mo.merge_partials(o.cpu().view(world, n_rows, 1, 512), lse.cpu().view(world, n_rows, 1))
            assert torch.allclose(out.float().cpu(), cpu.view(n_rows, 512).to(torch.bfloat16).float(), atol=1e-2)
            for r in range(world):
                assert int(_flags(be, bases[r])[0]) == epoch         # rank 0's signal reached allocation r
            assert int(ws[:4].view(torch.int32)[0]) == 0             # no wait ran out
    finally:
        torch.cuda.synchronize()
        for b in bases:
            be.free(b)


def test_missing_peer_times_out_and_is_reported(env):
    _cabi, D, sub = env
    be = D.CudaPeerBackend("cuda")
    n_rows, world = 32, 2
    bases = _alloc(be, world, n_rows)
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    try:
        o = torch.randn(world, n_rows, 512).cuda()
        lse = torch.randn(world, n_rows).cuda()
        for r in range(world):
            _fill(be, bases[r], n_rows, 1, o[r], lse[r])
        t0 = time.time()
        out = be.merge(bases, 0, 1, n_rows, 50, workspace=ws)        # rank 1 never signals
        torch.cuda.synchronize()
        assert time.time() - t0 < 5.0
        word = torch.zeros(1, dtype=torch.int32).pin_memory()
        _cabi.check(_cabi.lib.b200_mla_read_status(ws.data_ptr(), word.data_ptr(), torch.cuda.current_stream().cuda_stream), "status")
        torch.cuda.synchronize()
        assert int(word[0]) == _cabi.STATUS_TIMEOUT
        assert torch.equal(out, o[0].to(torch.bfloat16))              # the absent peer has weight 0
        # the context is intact: the same merge with the flag set completes and is correct
        _flags(be, bases[0])[1] = 1
        out2 = be.merge(bases, 0, 1, n_rows, 50, workspace=ws)
        torch.cuda.synchronize()
        ref = sub.combine_partials(o.view(world, n_rows, 1, 512), lse.view(world, n_rows, 1)).view(n_rows, 512)
        assert torch.equal(out2, ref)
    finally:
        torch.cuda.synchronize()
        for b in bases:
            be.free(b)


def test_argument_checks(env):
    _cabi, D, sub = env
    lib = _cabi.lib
    out = torch.empty(16, 512, dtype=torch.bfloat16, device="cuda")
    be = D.CudaPeerBackend("cuda")
    base = be.alloc(16)[0]
    try:
        arr = (ctypes.c_void_p * 3)(base, base, base)
        stream = torch.cuda.current_stream().cuda_stream

        def call(**kw):
            f = dict(world=1, rank=0, epoch=1, wait_limit_ms=10, bases=arr, rows=16, out=out.data_ptr(), workspace=None)
            f.update(kw)
            return lib.b200_mla_peer_merge(ctypes.byref(_cabi.PeerMergeArgs(**f)), stream)

        assert call() == 0
        assert call(world=3) != 0 and b"world" in lib.b200_mla_last_error()
        assert call(rank=1) != 0
        assert call(epoch=0) != 0 and b"epoch" in lib.b200_mla_last_error()
        assert call(rows=0) != 0
        assert call(out=None) != 0
        assert lib.b200_mla_peer_exchange_bytes(16) == 256 + 2 * ((16 * 513 * 4 + 255) // 256 * 256)
        assert lib.b200_mla_peer_partial_offset(16, 1) - lib.b200_mla_peer_partial_offset(16, 2) == (16 * 513 * 4 + 255) // 256 * 256
        torch.cuda.synchronize()
    finally:
        be.free(base)
