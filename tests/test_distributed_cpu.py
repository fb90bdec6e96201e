"""Host-side logic of the two multi-GPU modes, on CPU: partitions, shard construction and - with
two `gloo` ranks - the all-gather + merge plumbing of the cross-GPU split-KV mode and the
collective-free batch-sharded mode, with the CPU oracle standing in for the CUDA kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import mla_oracle as mo
from amd_optimization_challenge_b200 import distributed as D
from amd_optimization_challenge_b200 import inputs


def test_token_balanced_partition_properties():
    g = torch.Generator().manual_seed(0)
    lens = torch.randint(1024, 16385, (128,), generator=g).tolist()
    for world in (1, 2, 4, 8):
        parts = D.token_balanced_partition(lens, world)
        assert sorted(i for p in parts for i in p) == list(range(128))            # a partition
        loads = [sum(lens[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(lens)                                  # LPT bound
        assert max(loads) <= 1.02 * sum(lens) / world + 1                            # near-even for this distribution
        assert parts == D.token_balanced_partition(lens, world)                      # deterministic
    assert D.token_balanced_partition([5, 0, 7], 4) == [[2], [0], [1], []]
    with pytest.raises(ValueError):
        D.token_balanced_partition([1], 0)


def test_kv_range_partition():
    for S, world in ((131072, 8), (131072, 2), (1000, 4), (100, 8), (0, 2)):
        r = D.kv_range_partition(S, world)
        assert r[0][0] == 0 and r[-1][1] == S and all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(a % 128 == 0 for a, _ in r if a < S)
    assert D.kv_range_partition(131072, 8)[3] == (49152, 65536)


def test_shard_batch_matches_whole():
    lens = [40, 0, 33, 70, 5]
    data = inputs.generate_input(5, 2, 70, seed=3, kv_lens=lens, shuffle_pages=True, device="cpu", formats=("fp8",))
    q, kvd, qo, kvp, cfg = data
    whole = mo.decode_from_data(q, None, "fp8", kvd["fp8"], kvp.numpy(), cfg["kv_indices"].numpy(), cfg["sm_scale"], q_len=2)
    parts = D.token_balanced_partition(lens, 2)
    for ids in parts:
        sq, skv, sqo, skp, scfg = D.shard_batch(data, ids)
        assert sqo.tolist() == [2 * i for i in range(len(ids) + 1)] and scfg["batch_size"] == len(ids)
        o = mo.decode_from_data(sq, None, "fp8", skv["fp8"], skp.numpy(), scfg["kv_indices"].numpy(), scfg["sm_scale"], q_len=2)
        rows = torch.cat([torch.arange(2 * b, 2 * b + 2) for b in ids])
        assert torch.equal(o, whole[rows])


def test_split_kv_shard_covers_every_key_once():
    """The per-rank page-table slices of the cross-GPU split-KV mode: every key of every sequence lands on exactly
    one rank, with the position offset and total length the causal mask needs; merged partials equal the whole."""
    B, QL, S, world = 3, 2, 700, 4
    data = inputs.generate_input(B, QL, S, seed=11, shuffle_pages=True, device="cpu", formats=("fp8",))
    q, kvd, _, kvp, cfg = data
    idx = cfg["kv_indices"]
    seen = []
    parts_o, parts_l = [], []
    kf = mo.dequant_kv("fp8", kvd["fp8"])
    for r in range(world):
        local, ip, off, tot, n = D.split_kv_shard(idx, B, S, r, world)
        a, b = D.kv_range_partition(S, world)[r]
        assert n == b - a and ip.tolist() == [i * n for i in range(B + 1)]
        assert off.tolist() == [a] * B and tot.tolist() == [S] * B and local.dtype == torch.int32
        if n:
            seen.append(local.view(B, n))
        o, l = mo.mla_decode(q.float(), kf, ip.numpy(), local.numpy(), cfg["sm_scale"], q_len=QL,
                             kv_pos_offset=off.tolist(), kv_total_len=tot.tolist())
        parts_o.append(o); parts_l.append(l)
    assert torch.equal(torch.cat(seen, dim=1).reshape(-1), idx)
    merged, _ = mo.merge_partials(torch.stack(parts_o), torch.stack(parts_l))
    whole, _ = mo.mla_decode(q.float(), kf, kvp.numpy(), idx.numpy(), cfg["sm_scale"], q_len=QL)
    assert torch.allclose(merged, whole, atol=1e-5)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    return port


def _split_kv_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, QL, H, S = 2, 2, 16, 300
        data = inputs.generate_input(B, QL, S, seed=11, device="cpu", formats=("mxfp4",))   # same on every rank
        q, kvd, _, kvp, cfg = data
        kf = mo.dequant_kv("mxfp4", kvd["mxfp4"])
        a, b = D.kv_range_partition(S, world)[rank]
        n = b - a
        idx = np.concatenate([np.arange(s * S + a, s * S + b) for s in range(B)]).astype(np.int32)
        ip = np.arange(B + 1) * n

        def partial_fn(out_o, out_lse):
            o, l = mo.mla_decode(q.float(), kf, ip, idx, cfg["sm_scale"], q_len=QL, causal=True,
                                 kv_pos_offset=[a] * B, kv_total_len=[S] * B)
            out_o.copy_(o); out_lse.copy_(l)

        dec = D.SplitKVDecoder(B * QL, H, "cpu")
        merged = dec.step(partial_fn, merge_fn=lambda o, l: mo.merge_partials(o, l)[0])
        whole, _ = mo.mla_decode(q.float(), kf, kvp.numpy(), None, cfg["sm_scale"], q_len=QL, causal=True)
        ok = torch.allclose(merged, whole, atol=1e-5)
        # the fused buffer really carries (O || LSE) of every rank
        o_parts, lse_parts = dec.gathered()
        ok = ok and o_parts.shape == (world, B * QL, H, 512) and lse_parts.shape == (world, B * QL, H)
        ok = ok and torch.equal(o_parts[rank], dec.local_o()) and torch.equal(lse_parts[rank], dec.local_lse())
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def _batch_shard_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lens = [90, 10, 64, 33, 0, 128]
        data = inputs.generate_input(len(lens), 1, 128, seed=5, kv_lens=lens, shuffle_pages=True, device="cpu",
                                     formats=("hybrid",))
        ids = D.token_balanced_partition(lens, world)[rank]
        shard = D.shard_batch(data, ids)
        oracle = lambda d: mo.decode_from_data(d[0], None, "hybrid", d[1]["hybrid"], d[3].numpy(),
                                               d[4]["kv_indices"].numpy(), d[4]["sm_scale"])
        mine = D.decode_batch_sharded(shard, decode_fn=oracle)
        whole = oracle(data)
        ok = torch.equal(mine, whole[torch.tensor(ids, dtype=torch.long)]) if ids else mine.shape[0] == 0
        # only bookkeeping crosses ranks: every sequence is owned exactly once
        owned = [None] * world
        dist.all_gather_object(owned, ids)
        ok = ok and sorted(i for p in owned for i in p) == list(range(len(lens)))
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


class ShmPeerBackend:
    """Host stand-in for the exchange allocations of the peer-memory mode: POSIX shared memory with the layout of
    csrc/peer_merge.cu (64 flag words, then the partial of even steps, then the partial of odd steps), a "pointer"
    being (mapping index << 40) + byte offset.  merge() follows the kernel's three steps: signal, bounded wait,
    read the peers' partials and merge."""
    FLAGS = 256

    def __init__(self):
        from multiprocessing import shared_memory
        self._sm = shared_memory
        self.maps = []

    @staticmethod
    def _part_bytes(rows):
        return (rows * 513 * 4 + 255) // 256 * 256

    def exchange_bytes(self, rows):
        return self.FLAGS + 2 * self._part_bytes(rows)

    def partial_offset(self, rows, epoch):
        return self.FLAGS + (epoch & 1) * self._part_bytes(rows)

    def _add(self, shm):
        self.maps.append(shm)
        return len(self.maps) << 40

    def alloc(self, rows):
        shm = self._sm.SharedMemory(create=True, size=self.exchange_bytes(rows))
        shm.buf[:] = bytes(len(shm.buf))
        return self._add(shm), shm.name.encode()

    def open(self, handle):
        return self._add(self._sm.SharedMemory(name=handle.decode()))

    def _array(self, ptr, dtype, n):
        return np.frombuffer(self.maps[(ptr >> 40) - 1].buf, dtype=dtype, count=n, offset=ptr & ((1 << 40) - 1))

    def floats(self, ptr, n):
        return torch.from_numpy(self._array(ptr, np.float32, n))

    def close(self, base):
        self.maps[(base >> 40) - 1].close()

    def free(self, base):
        shm = self.maps[(base >> 40) - 1]
        shm.close(); shm.unlink()

    def merge(self, bases, rank, epoch, rows, wait_limit_ms, workspace=None):
        import time
        for b in bases:
            self._array(b, np.uint32, 64)[rank] = epoch
        mine = self._array(bases[rank], np.uint32, 64)
        t0 = time.time()
        while any(int(mine[i]) < epoch for i in range(len(bases))):
            if time.time() - t0 > (wait_limit_ms or 20000) / 1000:
                raise TimeoutError("peer signal missing")
            time.sleep(0.001)
        off = self.partial_offset(rows, epoch)
        o = torch.stack([self.floats(b + off, rows * 512).view(rows, 512) for b in bases])
        l = torch.stack([self.floats(b + off + rows * 2048, rows) for b in bases])
        return mo.merge_partials(o, l)[0].clone()


def _peer_split_kv_worker(rank, world, port, ret):
    """PeerSplitKVDecoder's protocol (handle exchange, epochs, the two partial buffers) with shared memory
    standing in for mapped device memory; three steps with different queries, so both buffers are reused."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, QL, H, S = 2, 1, 16, 300
        a, b = D.kv_range_partition(S, world)[rank]
        n = b - a
        idx = np.concatenate([np.arange(s * S + a, s * S + b) for s in range(B)]).astype(np.int32)
        ip = np.arange(B + 1) * n
        dec = D.PeerSplitKVDecoder(B * QL, H, "cpu", backend=ShmPeerBackend())
        ok = len(dec.bases) == world and len(set(dec.bases)) == world
        for step in range(3):
            data = inputs.generate_input(B, QL, S, seed=20 + step, device="cpu", formats=("fp8",))
            q, kvd, _, kvp, cfg = data
            kf = mo.dequant_kv("fp8", kvd["fp8"])

            def partial_fn(out_o, out_lse):
                o, l = mo.mla_decode(q.float(), kf, ip, idx, cfg["sm_scale"], q_len=QL, kv_pos_offset=[a] * B,
                                     kv_total_len=[S] * B)
                out_o.copy_(o); out_lse.copy_(l)

            merged = dec.step(partial_fn)
            whole, _ = mo.mla_decode(q.float(), kf, kvp.numpy(), None, cfg["sm_scale"], q_len=QL)
            ok = ok and merged.shape == (B * QL, H, 512) and torch.allclose(merged, whole, atol=1e-5)
            ok = ok and dec.epoch == step + 1
        dec.close()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("worker", [_split_kv_worker, _batch_shard_worker, _peer_split_kv_worker])
def test_two_ranks_gloo(worker):
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
