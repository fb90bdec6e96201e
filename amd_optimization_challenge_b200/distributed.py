"""Multi-GPU decode: one process per GPU, `torch.distributed` for the plumbing.

The reference is single-GPU only (no collective call exists anywhere in it); the two modes below
are the ones the decode path shards into naturally.

* Batch sharding (no collective).  Sequences are independent - each touches only its own
  kv_indptr range (mixed-mla/submission.py:154-160) - so ragged batches are split over the ranks
  by a token-balanced partition and every rank runs the ordinary `custom_kernel` on its shard.
* Split-KV across GPUs (one all-gather).  Rank r holds the keys [r*S/n, (r+1)*S/n) of every
  sequence, decodes them into a normalised fp32 partial O and its log-sum-exp, all ranks exchange
  the fused (O || LSE) buffer with ONE all-gather over NVLink, and the LSE-combine kernel merges
  the n partials (the merge of mixed-mla/submission.py:257-294, across GPUs instead of splits).

The compute callables are injectable so that the sharding / gather / merge logic is covered by
CPU tests with the `gloo` backend; the defaults are the CUDA kernels.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

V_DIM = 512


# --------------------------------------------------------------------------------------------
# partitions (host logic, no device work)
# --------------------------------------------------------------------------------------------

def token_balanced_partition(kv_lens: Sequence[int], world: int) -> list[list[int]]:
    """Assign sequences to `world` ranks so that the token counts are balanced: longest first,
    each to the currently lightest rank (LPT).  Returns, per rank, the sequence ids in ascending
    order.  Deterministic; every rank computes the same answer."""
    if world < 1:
        raise ValueError("world must be >= 1")
    order = sorted(range(len(kv_lens)), key=lambda i: (-int(kv_lens[i]), i))
    load = [0] * world
    out: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(kv_lens[i])
    return [sorted(s) for s in out]


def split_kv_shard(kv_indices: torch.Tensor, batch: int, seq_len: int, rank: int, world: int, granule: int = 128):
    """This rank's part of a uniform-length batch in the cross-GPU split-KV mode: the page-table
    entries of keys [a, b) of every sequence, back to back, with the matching local kv_indptr,
    position offsets and total lengths (int32, on kv_indices' device).  `kv_indices` is the
    global page-size-1 table [batch * seq_len]."""
    a, b = kv_range_partition(seq_len, world, granule)[rank]
    n = b - a
    dev = kv_indices.device
    local = kv_indices.view(batch, seq_len)[:, a:b].contiguous().view(-1)
    if n == 0:
        local = torch.zeros(1, dtype=torch.int32, device=dev)      # never read: every local sequence is empty
    indptr = (torch.arange(batch + 1, dtype=torch.int32, device=dev) * n).contiguous()
    off = torch.full((batch,), a, dtype=torch.int32, device=dev)
    tot = torch.full((batch,), seq_len, dtype=torch.int32, device=dev)
    return local, indptr, off, tot, n


def kv_range_partition(seq_len: int, world: int, granule: int = 128) -> list[tuple[int, int]]:
    """Contiguous key ranges [begin, end) per rank for the cross-GPU split-KV mode, boundaries
    rounded to `granule` tokens (the kernels' tile) so that no tile straddles two GPUs."""
    if world < 1:
        raise ValueError("world must be >= 1")
    per = -(-seq_len // world)
    per = -(-per // granule) * granule
    return [(min(r * per, seq_len), min((r + 1) * per, seq_len)) for r in range(world)]


def shard_batch(data, seq_ids: Sequence[int]):
    """The sub-problem made of the sequences `seq_ids` of a (q, kv_data, qo_indptr, kv_indptr,
    config) tuple: q rows, indptrs and the page table are re-based; the cache planes are shared
    (a rank of a real deployment would hold only its own pages).  Host-side helper used by the
    tests and by callers that start from a global batch; needs `config["kv_indices"]`."""
    q, kv_data, qo_indptr, kv_indptr, config = data
    ql = int(config.get("q_seq_len", 1))
    ip = kv_indptr.cpu().tolist()
    idx = config["kv_indices"]
    rows = torch.cat([torch.arange(b * ql, (b + 1) * ql) for b in seq_ids]) if seq_ids else torch.zeros(0, dtype=torch.long)
    lens = [ip[b + 1] - ip[b] for b in seq_ids]
    new_idx = torch.cat([idx[ip[b]:ip[b + 1]] for b in seq_ids]) if seq_ids else idx[:0]
    new_ip = torch.zeros(len(seq_ids) + 1, dtype=torch.int32)
    if lens:
        new_ip[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int64), 0).to(torch.int32)
    cfg = dict(config)
    cfg.update(batch_size=len(seq_ids), kv_indices=new_idx.contiguous(), total_kv=int(sum(lens)), kv_lens=lens)
    new_qo = (torch.arange(len(seq_ids) + 1, dtype=torch.int32) * ql).to(qo_indptr.device)
    return (q[rows.to(q.device)].contiguous(), kv_data, new_qo, new_ip.to(kv_indptr.device), cfg)


# --------------------------------------------------------------------------------------------
# batch sharding: no data-path collective
# --------------------------------------------------------------------------------------------

def decode_batch_sharded(local_data, decode_fn: Callable | None = None):
    """Decode this rank's shard of a batch.  There is nothing to exchange: the result rows belong
    to this rank's sequences only.  Exists so that both multi-GPU modes have the same shape of
    call; `decode_fn` defaults to `custom_kernel`."""
    if decode_fn is None:
        from .submission import custom_kernel as decode_fn
    return decode_fn(local_data)


# --------------------------------------------------------------------------------------------
# split-KV across GPUs: local partial -> one all-gather -> LSE combine
# --------------------------------------------------------------------------------------------

class SplitKVDecoder:
    """Holds the persistent exchange buffers of the cross-GPU split-KV mode for one problem shape.

    rows = batch * q_len query rows, `heads` heads.  The local partial lives in `send`
    (rows*heads*512 floats of O followed by rows*heads floats of LSE) and is written in place by
    the stage-1 / combine kernels; `recv` holds the world's partials after the all-gather and is
    read in place by the merge.  Nothing is copied between the kernels and the collective.
    """

    def __init__(self, rows: int, heads: int, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows, self.heads = rows, heads
        self.n_o = rows * heads * V_DIM
        self.n = self.n_o + rows * heads
        self.send = torch.empty(self.n, dtype=torch.float32, device=device)
        self.recv = torch.empty(self.world * self.n, dtype=torch.float32, device=device)

    # views into the fused buffers ---------------------------------------------------------
    def local_o(self) -> torch.Tensor:
        return self.send[: self.n_o].view(self.rows, self.heads, V_DIM)

    def local_lse(self) -> torch.Tensor:
        return self.send[self.n_o:].view(self.rows, self.heads)

    def gathered(self):
        g = self.recv.view(self.world, self.n)
        return (g[:, : self.n_o].unflatten(1, (self.rows, self.heads, V_DIM)),
                g[:, self.n_o:].unflatten(1, (self.rows, self.heads)))

    # one decode step ------------------------------------------------------------------------
    def step(self, partial_fn: Callable, merge_fn: Callable | None = None, events=None):
        """partial_fn(out_o, out_lse) must fill this rank's normalised partial O and LSE (views
        of the send buffer); returns the merged bf16 O [rows, heads, 512] on every rank.
        `events`, if given, are three CUDA events recorded on the current stream before the
        all-gather, after it and after the merge (for timing the three phases separately)."""
        partial_fn(self.local_o(), self.local_lse())
        if events is not None:
            events[0].record()
        if self.world > 1:
            dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        else:
            self.recv.copy_(self.send)
        if events is not None:
            events[1].record()
        if merge_fn is None:
            from .submission import combine_partials_strided
            out = combine_partials_strided(self.recv, self.world, self.n, self.n_o, self.rows, self.heads)
        else:
            o_parts, lse_parts = self.gathered()
            out = merge_fn(o_parts, lse_parts)
        if events is not None:
            events[2].record()
        return out


def cuda_partial_fn(q, q_scale, kv_format: str, kv_local, kv_indptr_local, *, sm_scale: float, q_len: int,
                    kv_indices=None, kv_pos_offset=None, kv_total_len=None, total_kv_hint: int = 0, impl: str = "auto"):
    """The default producer of a rank's partial for SplitKVDecoder.step: the CUDA decode writing
    its normalised fp32 O and LSE straight into the send buffer."""
    from .submission import mla_decode

    def fn(out_o, out_lse):
        mla_decode(q, q_scale, kv_format, kv_local, kv_indptr_local, sm_scale=sm_scale, q_len=q_len,
                   kv_indices=kv_indices, kv_pos_offset=kv_pos_offset, kv_total_len=kv_total_len,
                   total_kv_hint=total_kv_hint, return_partial=True, partial_out=(out_o, out_lse), impl=impl)
    return fn


# --------------------------------------------------------------------------------------------
# split-KV across GPUs over peer memory: local partial -> fused signal + wait + merge kernel
# --------------------------------------------------------------------------------------------

class _DeviceSpan:
    """A raw device range as something torch.as_tensor can wrap without a copy."""

    def __init__(self, ptr: int, n_floats: int):
        self.__cuda_array_interface__ = {"shape": (n_floats,), "typestr": "<f4", "data": (ptr, False), "version": 2}


class CudaPeerBackend:
    """The exchange allocation and the merge kernel behind the C-ABI (b200_mla_peer_*)."""

    def __init__(self, device):
        from . import _cabi
        self._c = _cabi
        self.device = torch.device(device)

    def exchange_bytes(self, rows: int) -> int:
        return int(self._c.lib.b200_mla_peer_exchange_bytes(rows))

    def partial_offset(self, rows: int, epoch: int) -> int:
        return int(self._c.lib.b200_mla_peer_partial_offset(rows, epoch))

    def alloc(self, rows: int):
        import ctypes
        base = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(self._c.PEER_HANDLE_BYTES)
        with torch.cuda.device(self.device):
            self._c.check(self._c.lib.b200_mla_peer_alloc(rows, ctypes.byref(base), handle), "b200_mla_peer_alloc")
        return int(base.value), bytes(handle.raw)

    def open(self, handle: bytes) -> int:
        import ctypes
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            self._c.check(self._c.lib.b200_mla_peer_open(handle, ctypes.byref(base)), "b200_mla_peer_open")
        return int(base.value)

    def close(self, base: int) -> None:
        self._c.check(self._c.lib.b200_mla_peer_close(base), "b200_mla_peer_close")

    def free(self, base: int) -> None:
        self._c.check(self._c.lib.b200_mla_peer_free(base), "b200_mla_peer_free")

    def floats(self, ptr: int, n: int) -> torch.Tensor:
        return torch.as_tensor(_DeviceSpan(ptr, n), device=self.device)

    def merge(self, bases, rank: int, epoch: int, rows: int, wait_limit_ms: int, workspace=None) -> torch.Tensor:
        import ctypes
        out = torch.empty(rows, V_DIM, dtype=torch.bfloat16, device=self.device)
        arr = (ctypes.c_void_p * len(bases))(*bases)
        a = self._c.PeerMergeArgs(world=len(bases), rank=rank, epoch=epoch, wait_limit_ms=wait_limit_ms, bases=arr, rows=rows,
                                  out=out.data_ptr(), workspace=workspace.data_ptr() if workspace is not None else None)
        with torch.cuda.device(self.device):
            self._c.check(self._c.lib.b200_mla_peer_merge(ctypes.byref(a), torch.cuda.current_stream(self.device).cuda_stream),
                          "b200_mla_peer_merge")
        return out


class PeerSplitKVDecoder:
    """Cross-GPU split-KV without a collective call: every rank's partial (O || LSE) lives in an
    exchange allocation the other ranks have mapped, and one kernel per rank signals, waits and
    merges by reading the peers' memory (csrc/peer_merge.cu).  Same call shape as SplitKVDecoder.

    The handles travel once, at construction, through `dist.all_gather_object`.  All ranks must
    call `step` the same number of times (the step number is the kernels' rendezvous epoch).
    `backend` is injectable so that the protocol (handle exchange, epochs, buffer parity) runs
    under `gloo` on CPU with a shared-memory stand-in."""

    def __init__(self, rows: int, heads: int, device, group=None, backend=None, wait_limit_ms: int = 0):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows, self.heads = rows, heads
        self.n_rows = rows * heads
        self.n_o = self.n_rows * V_DIM
        self.backend = backend if backend is not None else CudaPeerBackend(device)
        self.wait_limit_ms = wait_limit_ms
        self.epoch = 0
        # every rank learns whether every other rank got its allocation and its mappings: either all ranks
        # hold a working decoder afterwards or all of them raise (nobody is left waiting for a peer that gave up)
        self.bases = None
        own, handle, err = None, None, None
        try:
            own, handle = self.backend.alloc(self.n_rows)
        except Exception as e:                                   # noqa: BLE001 - reported to every rank below
            err = f"rank {self.rank}: {e}"
        opened = []
        try:
            handles = self._agree(handle, err)
            err = None
            try:
                for r in range(self.world):
                    opened.append(own if r == self.rank else self.backend.open(handles[r]))
            except Exception as e:                               # noqa: BLE001
                err = f"rank {self.rank}: {e}"
            self._agree(True, err)                               # also: every mapping exists before the first signal
        except Exception:
            for r, b in enumerate(opened):
                if r != self.rank:
                    self.backend.close(b)
            if own is not None:
                self.backend.free(own)
            raise
        self.bases = opened

    def _agree(self, payload, err):
        """All-gather (payload, error string); raises on every rank if any rank reported an error, else returns
        the list of all ranks' payloads."""
        everyone = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(everyone, (payload, err), group=self.group)
        else:
            everyone[0] = (payload, err)
        errors = [e for _, e in everyone if e]
        if errors:
            raise RuntimeError("peer-memory exchange is not available: " + "; ".join(errors))
        return [p for p, _ in everyone]

    def _views(self, epoch: int):
        ptr = self.bases[self.rank] + self.backend.partial_offset(self.n_rows, epoch)
        buf = self.backend.floats(ptr, self.n_o + self.n_rows)
        return buf[: self.n_o].view(self.rows, self.heads, V_DIM), buf[self.n_o:].view(self.rows, self.heads)

    def step(self, partial_fn: Callable, events=None, workspace=None):
        """partial_fn(out_o, out_lse) fills this rank's normalised partial of this step; returns
        the merged bf16 O [rows, heads, 512] on every rank.  `events`: two CUDA events recorded
        before and after the merge kernel."""
        self.epoch += 1
        o, lse = self._views(self.epoch)
        partial_fn(o, lse)
        if events is not None:
            events[0].record()
        out = self.backend.merge(self.bases, self.rank, self.epoch, self.n_rows, self.wait_limit_ms, workspace)
        if events is not None:
            events[1].record()
        return out.view(self.rows, self.heads, V_DIM)

    def close(self):
        """Unmap the peers and free the own allocation; collective (nobody may still be reading)."""
        if self.bases is None:
            return
        if torch.cuda.is_available() and isinstance(self.backend, CudaPeerBackend):
            torch.cuda.synchronize(self.backend.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        for r, b in enumerate(self.bases):
            if r != self.rank:
                self.backend.close(b)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.backend.free(self.bases[self.rank])
        self.bases = None
