"""CPU oracle for absorbed-MLA decode over a quantised latent KV cache.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is the
checker that the parity tests, the smoke check and the CPU-baseline leg of the benchmark call.

It restates, in plain numpy / torch-CPU fp32, the semantics of the reference workspace's decode
path (paths are relative to the reference project root):

* tensor contract and constants ............ competitor_submissions/mi355x_reference/task.py:4-23,
                                             reference.py:40-49, 288-346
* per-tensor FP8 quantiser .................. reference.py:65-80
* MXFP4 layout (e2m1 x2 per byte, E8M0/32) .. reference.py:88-154, mi355x_reference/README.md:73-81
* e2m1 / E8M0 decode ........................ mixed-mla/triton_mla_mxfp4.py:20-31, :59
* MXFP4 quantiser rounding rule ............. mxfp4-mm/submission_v3_self_contained.py:19-72
  (the in-tree copy of the third-party ROCm/aiter `_mxfp4_quant_op`, aiter itself is un-vendored
  and unpinned: setup.sh:56-61)
* attention semantics (scores over 576 dims, V = first 512 dims of the same row, softmax over
  the sequence's KV range, scalar scales folded) mixed-mla/versions/hip_phase1/submission.py:85-159,
  mixed-mla/triton_fp8_decode.py:44-156
* split / log-sum-exp merge ................. mixed-mla/submission.py:257-294,
                                             competitor_submissions/dgavriloff_v114_hybrid_mxfp4k_fp8v.py:124-160

Parity pin: the functions below are checked against golden vectors produced by executing the
reference's own Python (its FP8 quantiser, its MXFP4 quantiser and its two AITER-free Triton
decode kernels, the latter under Triton's CPU interpreter); see tests/golden/make_golden.py.
The q_len > 1 causal convention (bottom-right aligned) and the paged `kv_indices` / hybrid-format
extensions are never exercised by the reference and are therefore parity-unpinned: they are
defined here.
"""
from __future__ import annotations

import numpy as np
import torch

QK_DIM = 576
V_DIM = 512
ROPE_DIM = 64
MX_BLOCK = 32
E4M3_MAX = 448.0

# --------------------------------------------------------------------------------------------
# byte-level formats
# --------------------------------------------------------------------------------------------

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def e2m1_table() -> np.ndarray:
    """16-entry decode table: code bit3 = sign, bits2..1 = exponent, bit0 = mantissa
    (mixed-mla/triton_mla_mxfp4.py:20-31)."""
    return np.concatenate([E2M1_VALUES, -E2M1_VALUES]).astype(np.float32)


def e4m3fn_table() -> np.ndarray:
    """256-entry decode table for OCP e4m3fn: 1-4-3, bias 7, no inf, 0x7f/0xff = NaN."""
    t = np.empty(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


_E4M3_LUT = e4m3fn_table()
_E2M1_LUT = e2m1_table()


def e8m0_decode(b: np.ndarray) -> np.ndarray:
    """E8M0: value = 2^(byte-127) (mixed-mla/triton_mla_mxfp4.py:59); 255 = NaN."""
    b = np.asarray(b, dtype=np.uint8)
    out = np.ldexp(np.float32(1.0), b.astype(np.int32) - 127).astype(np.float32)
    out[b == 255] = np.nan
    return out


def fp8_e4m3_decode(b: np.ndarray) -> np.ndarray:
    return _E4M3_LUT[np.asarray(b, dtype=np.uint8)]


def fp8_e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> e4m3fn byte, saturating at +-448 (the reference clamps
    before its cast, reference.py:79)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x), np.float32(E4M3_MAX))
    sign = (np.signbit(x)).astype(np.uint8) << 7
    # candidates: the 127 non-negative finite codes, pick nearest, ties to even mantissa
    pos = _E4M3_LUT[:127].astype(np.float64)  # codes 0..126 are monotone, 0x7f is NaN
    idx = np.searchsorted(pos, a.astype(np.float64), side="left")
    idx = np.clip(idx, 1, 126)
    lo = pos[idx - 1]
    hi = pos[idx]
    a64 = a.astype(np.float64)
    pick_hi = (a64 - lo > hi - a64) | ((a64 - lo == hi - a64) & ((idx & 1) == 0))
    code = np.where(pick_hi, idx, idx - 1).astype(np.uint8)
    code = np.where(a == 0, np.uint8(0), code)
    return (code | sign).astype(np.uint8)


# --------------------------------------------------------------------------------------------
# quantisers (input construction)
# --------------------------------------------------------------------------------------------

def quantize_fp8_per_tensor(x_bf16: torch.Tensor):
    """Dynamic per-tensor e4m3fn quantiser with the reference's arithmetic order
    (reference.py:65-80): amax, scale = amax/448 and x/scale are all evaluated in the input
    dtype (bf16), then clamped and cast.  Returns (uint8 codes, fp32 scale[1])."""
    assert x_bf16.dtype == torch.bfloat16
    amax = x_bf16.abs().amax().clamp(min=1e-12)
    scale = amax / E4M3_MAX
    y = (x_bf16 / scale).clamp(min=-E4M3_MAX, max=E4M3_MAX).to(torch.float32)
    codes = fp8_e4m3_encode(y.numpy())
    return torch.from_numpy(codes).reshape(x_bf16.shape), scale.to(torch.float32).reshape(1)


def quantize_mxfp4(x: np.ndarray):
    """MXFP4 quantiser over the last axis in blocks of 32
    (rule of mxfp4-mm/submission_v3_self_contained.py:19-72).

    block amax -> rounded up to the next power of two when its mantissa is >= 1.75
    (integer add of 0x200000, mask 0xFF800000) -> exponent = floor(log2) - 2 clamped to
    [-127, 127], stored biased by 127 -> elements scaled by 2^-exponent and rounded to e2m1
    with round-to-nearest-even, saturating at 6, 0.5 as the only subnormal -> two codes per
    byte, even element in the low nibble.
    Returns (codes uint8 [..., N/2], scales uint8 [..., N/32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[-1]
    assert n % MX_BLOCK == 0
    xb = x.reshape(*x.shape[:-1], n // MX_BLOCK, MX_BLOCK)
    amax = np.abs(xb).max(axis=-1)
    bits = amax.view(np.uint32).astype(np.uint64)
    bits = ((bits + 0x200000) & 0xFF800000).astype(np.uint32)
    e_field = (bits >> 23).astype(np.int32)              # biased exponent of the power of two
    # floor(log2(p)) for a power of two p = e_field-127; p == 0 (e_field 0) -> -inf -> clamps low
    exp = np.where(e_field == 0, -127, e_field - 127 - 2)
    exp = np.clip(exp, -127, 127).astype(np.int32)
    scale_byte = (exp + 127).astype(np.uint8)
    q = xb * np.ldexp(np.float32(1.0), -exp)[..., None].astype(np.float32)
    q = q.astype(np.float32)
    qbits = q.view(np.uint32)
    sign = ((qbits >> 28) & 0x8).astype(np.uint8)
    mag_bits = (qbits & 0x7FFFFFFF).astype(np.uint32)
    mag = mag_bits.view(np.float32)
    sat = mag >= 6.0
    den = (~sat) & (mag < 1.0)
    # subnormal range: round to a multiple of 0.5 (ties to even) by the 2^22 magic add
    magic = np.float32(2.0 ** 22)
    den_code = ((np.where(den, mag, 0).astype(np.float32) + magic).view(np.uint32)
                - magic.view(np.uint32)).astype(np.uint8)
    # normal range: re-bias exponent 127 -> 1, keep one mantissa bit, nearest-even
    odd = (mag_bits >> 22) & 1
    nb = mag_bits.astype(np.int64) + ((-126) << 23) + (1 << 21) - 1 + odd.astype(np.int64)
    nor_code = ((nb >> 22) & 0xFF).astype(np.uint8)
    code = np.where(sat, np.uint8(7), np.where(den, den_code, nor_code)).astype(np.uint8)
    code = code | sign
    code = code.reshape(*x.shape[:-1], n)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).astype(np.uint8)
    return packed, scale_byte


def dequantize_mxfp4(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """(codes [..., N/2], E8M0 [..., >= N/32]) -> fp32 [..., N] (reference.py:116-154)."""
    packed = np.asarray(packed, dtype=np.uint8)
    n = packed.shape[-1] * 2
    vals = np.empty(packed.shape[:-1] + (n,), dtype=np.float32)
    vals[..., 0::2] = _E2M1_LUT[packed & 0xF]
    vals[..., 1::2] = _E2M1_LUT[packed >> 4]
    nb = n // MX_BLOCK
    sc = e8m0_decode(np.asarray(scales)[..., :nb])
    return (vals.reshape(*vals.shape[:-1], nb, MX_BLOCK) * sc[..., None]).reshape(vals.shape)


# --------------------------------------------------------------------------------------------
# KV / Q dequantisation per cache format
# --------------------------------------------------------------------------------------------

def dequant_kv(kv_format: str, kv) -> torch.Tensor:
    """-> fp32 [slots, 576].  kv is
    "fp8":    (codes u8 [T,576], scale f32[1])
    "mxfp4":  (codes u8 [T,288], e8m0 u8 [>=T, >=18])
    "hybrid": (latent codes u8 [T,256], latent e8m0 u8 [T,16], rope codes u8 [T,64], rope scale f32[1])
    "bf16":   bf16 [T,576]
    """
    if kv_format == "fp8":
        codes, scale = kv
        k = fp8_e4m3_decode(_u8(codes).reshape(-1, QK_DIM)) * np.float32(float(scale.reshape(-1)[0]))
    elif kv_format == "mxfp4":
        codes, sc = kv
        codes = _u8(codes).reshape(-1, QK_DIM // 2)
        k = dequantize_mxfp4(codes, _u8(sc)[: codes.shape[0]])
    elif kv_format == "hybrid":
        lat, lsc, rope, rscale = kv
        lat = _u8(lat).reshape(-1, V_DIM // 2)
        kl = dequantize_mxfp4(lat, _u8(lsc)[: lat.shape[0]])
        kr = fp8_e4m3_decode(_u8(rope).reshape(-1, ROPE_DIM)) * np.float32(float(rscale.reshape(-1)[0]))
        k = np.concatenate([kl, kr], axis=1)
    elif kv_format == "bf16":
        return kv.reshape(-1, QK_DIM).to(torch.float32)
    else:
        raise ValueError(kv_format)
    return torch.from_numpy(np.ascontiguousarray(k, dtype=np.float32))


def dequant_q(q, q_scale=None) -> torch.Tensor:
    """bf16 Q, or (e4m3 codes, fp32 scale) -> fp32 [rows, H, 576]."""
    if q_scale is None:
        return q.to(torch.float32)
    v = fp8_e4m3_decode(_u8(q)) * np.float32(float(q_scale.reshape(-1)[0]))
    return torch.from_numpy(v.astype(np.float32)).reshape(q.shape)


def _u8(t) -> np.ndarray:
    if isinstance(t, np.ndarray):
        return t.view(np.uint8) if t.dtype != np.uint8 else t
    if t.dtype != torch.uint8:
        t = t.view(torch.uint8)
    return t.cpu().numpy()


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------

def mla_decode(qf: torch.Tensor, kf: torch.Tensor, kv_indptr, kv_indices, sm_scale: float,
               q_len: int = 1, causal: bool = True, kv_pos_offset=None, kv_total_len=None):
    """Dequantise-then-attend in fp32.

    qf [B*q_len, H, 576] fp32, kf [slots, 576] fp32; sequence b attends to the rows
    kf[kv_indices[kv_indptr[b]:kv_indptr[b+1]]]; V is the first 512 columns of the same rows.
    Query j of a sequence (j = 0..q_len-1) sees key position p (0-based within the *whole*
    sequence) iff p <= S_total - q_len + j when `causal` (bottom-right aligned).  For a KV shard
    of a longer sequence pass kv_pos_offset[b] (position of the shard's first key) and
    kv_total_len[b] (S_total).
    Returns (O fp32 [B*q_len, H, 512], LSE fp32 [B*q_len, H]); an empty key set gives O = 0,
    LSE = -inf.
    """
    kv_indptr = np.asarray(kv_indptr, dtype=np.int64)
    B = len(kv_indptr) - 1
    H = qf.shape[1]
    O = torch.zeros(B * q_len, H, V_DIM, dtype=torch.float32)
    LSE = torch.full((B * q_len, H), float("-inf"), dtype=torch.float32)
    idx_all = None if kv_indices is None else torch.as_tensor(np.asarray(kv_indices), dtype=torch.int64)
    for b in range(B):
        s0, s1 = int(kv_indptr[b]), int(kv_indptr[b + 1])
        n = s1 - s0
        if n <= 0:
            continue
        rows = torch.arange(s0, s1) if idx_all is None else idx_all[s0:s1]
        k = kf[rows]                                           # [n, 576]
        q = qf[b * q_len:(b + 1) * q_len].reshape(q_len * H, QK_DIM)
        s = (q @ k.t()) * sm_scale                              # [q_len*H, n]
        if causal and q_len > 1:
            off = 0 if kv_pos_offset is None else int(kv_pos_offset[b])
            tot = n if kv_total_len is None else int(kv_total_len[b])
            pos = off + torch.arange(n)
            for j in range(q_len):
                limit = tot - q_len + j
                s[j * H:(j + 1) * H, pos > limit] = float("-inf")
        m = s.max(dim=1, keepdim=True).values
        dead = torch.isinf(m) & (m < 0)
        m = torch.where(dead, torch.zeros_like(m), m)
        p = torch.exp(s - m)
        l = p.sum(dim=1, keepdim=True)
        o = (p @ k[:, :V_DIM]) / torch.where(l > 0, l, torch.ones_like(l))
        lse = torch.where(l > 0, m + torch.log(l), torch.full_like(l, float("-inf")))
        O[b * q_len:(b + 1) * q_len] = o.reshape(q_len, H, V_DIM)
        LSE[b * q_len:(b + 1) * q_len] = lse.reshape(q_len, H)
    return O, LSE


def merge_partials(O_parts: torch.Tensor, LSE_parts: torch.Tensor):
    """Log-sum-exp merge of normalised partials (mixed-mla/submission.py:257-294 in (O, LSE)
    form, competitor_submissions/dgavriloff_v114_hybrid_mxfp4k_fp8v.py:131-160).
    O_parts [P, rows, H, 512], LSE_parts [P, rows, H] -> (O, LSE)."""
    M = LSE_parts.max(dim=0).values
    Msafe = torch.where(torch.isinf(M), torch.zeros_like(M), M)
    w = torch.exp(LSE_parts - Msafe)                           # exp(-inf) = 0 for empty shards
    den = w.sum(dim=0)
    O = (w.unsqueeze(-1) * O_parts).sum(dim=0) / torch.where(den > 0, den, torch.ones_like(den)).unsqueeze(-1)
    LSE = torch.where(den > 0, Msafe + torch.log(den), torch.full_like(den, float("-inf")))
    return O, LSE


def decode_from_data(q, q_scale, kv_format, kv, kv_indptr, kv_indices, sm_scale, q_len=1,
                     causal=True, return_lse=False):
    """Convenience: dequantise Q and KV of the given format and attend.  Returns bf16 O."""
    qf = dequant_q(q, q_scale)
    kf = dequant_kv(kv_format, kv)
    O, LSE = mla_decode(qf, kf, kv_indptr, kv_indices, sm_scale, q_len=q_len, causal=causal)
    if return_lse:
        return O, LSE
    return O.to(torch.bfloat16)
