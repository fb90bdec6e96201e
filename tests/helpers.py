"""Shared helpers for the tests: fixture decoding and oracle-side evaluation of a `data` tuple."""
import numpy as np
import torch

from oracle import mla_oracle as mo


def bf16_from_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def oracle_for_data(data, kv_format, q_format, return_lse=False):
    """Evaluate the CPU oracle on a (q, kv_data, qo_indptr, kv_indptr, config) tuple whose tensors
    may live on the GPU: FP8 Q is re-quantised with the oracle's own per-tensor quantiser."""
    q, kv_data, _, kv_indptr, config = data
    q = q.cpu()
    q_scale = None
    if q_format == "fp8":
        q, q_scale = mo.quantize_fp8_per_tensor(q)
    kv = kv_data[kv_format]
    kv = tuple(t.cpu() for t in kv) if isinstance(kv, tuple) else kv.cpu()
    idx = config.get("kv_indices")
    idx = None if idx is None else idx.cpu().numpy()
    return mo.decode_from_data(q, q_scale, kv_format, kv, kv_indptr.cpu().numpy(), idx, config["sm_scale"],
                               q_len=config["q_seq_len"], causal=True, return_lse=return_lse)


def assert_close(got: torch.Tensor, want: torch.Tensor, rtol=2e-2, atol=2e-2, tight=None):
    """The tolerance of record is rtol = atol = 2e-2 on the bf16 output.  `tight` additionally
    bounds the error relative to the output's own scale: max|diff| <= tight * max|want|."""
    got = got.float().cpu()
    want = want.float().cpu()
    assert got.shape == want.shape
    assert torch.isfinite(got).all()
    diff = (got - want).abs()
    bad = diff > atol + rtol * want.abs()
    assert not bad.any(), f"{int(bad.sum())} elements out of tolerance, max diff {diff.max().item():.4g}"
    if tight is not None:
        scale = want.abs().max().item()
        assert diff.max().item() <= tight * max(scale, 1e-6), \
            f"max diff {diff.max().item():.4g} vs output scale {scale:.4g} (limit {tight})"
