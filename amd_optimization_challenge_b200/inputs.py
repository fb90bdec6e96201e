"""Host-side mirror of the reference problem definition: constants, quantisers and the seeded
input generator (competitor_submissions/mi355x_reference/reference.py:40-154, 288-346).

Everything here is plain torch and runs on whatever device its inputs live on; it constructs
inputs, it is not the decode path.  Differences from the reference, all opt-in through keyword
arguments: random numbers are drawn on the CPU unless generator_device="cuda" is asked for (the
reference draws on a CUDA generator, whose bit stream cannot be reproduced without a GPU), the
MXFP4 quantiser is implemented here (the
reference calls the AMD-only aiter op; the rounding rule is that of
mxfp4-mm/submission_v3_self_contained.py:19-72), and the generator can also emit a page table,
ragged lengths, more heads and the hybrid cache format.
"""
from __future__ import annotations

import math

import torch

NUM_HEADS = 16
NUM_KV_HEADS = 1
KV_LORA_RANK = 512
QK_ROPE_HEAD_DIM = 64
QK_HEAD_DIM = KV_LORA_RANK + QK_ROPE_HEAD_DIM      # 576
V_HEAD_DIM = KV_LORA_RANK                          # 512
SM_SCALE = 1.0 / math.sqrt(QK_HEAD_DIM)
FP8_DTYPE = torch.float8_e4m3fn
FP8_MAX = 448.0
MX_BLOCK = 32


# --------------------------------------------------------------------------------------------
# quantisers
# --------------------------------------------------------------------------------------------

def quantize_fp8(tensor: torch.Tensor):
    """Dynamic per-tensor e4m3fn quantisation; arithmetic order of reference.py:65-80 (amax,
    scale and the quotient are evaluated in the tensor's own dtype).  Returns
    (float8_e4m3fn tensor, fp32 scale of shape [1])."""
    amax = tensor.abs().amax().clamp(min=1e-12)
    scale = amax / FP8_MAX
    q = (tensor / scale).clamp(min=-FP8_MAX, max=FP8_MAX).to(FP8_DTYPE)
    return q, scale.to(torch.float32).reshape(1)


def _mxfp4_rows(x: torch.Tensor):
    """x fp32 [R, N] -> (uint8 [R, N/2], uint8 [R, N/32])."""
    R, N = x.shape
    xb = x.reshape(R, N // MX_BLOCK, MX_BLOCK)
    amax = xb.abs().amax(dim=-1)
    bits = amax.view(torch.int32).to(torch.int64)
    bits = (bits + 0x200000) & 0xFF800000                 # next power of two when mantissa >= 1.75
    e_field = bits >> 23
    exp = torch.where(e_field == 0, torch.full_like(e_field, -127), e_field - 127 - 2).clamp(-127, 127)
    scale_byte = (exp + 127).to(torch.uint8)
    q = xb * torch.exp2(-exp.to(torch.float32)).unsqueeze(-1)
    qbits = q.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    sign = ((qbits >> 28) & 0x8).to(torch.uint8)
    mbits = qbits & 0x7FFFFFFF
    mag = mbits.to(torch.int32).view(torch.float32)
    sat = mag >= 6.0
    den = (~sat) & (mag < 1.0)
    # below 1.0 the only codes are 0, 0.5 and 1.0: round to a multiple of 0.5, ties to even
    den_code = (torch.where(den, mag, torch.zeros_like(mag)) * 2.0).round().to(torch.uint8)
    # [1, 6): re-bias the exponent 127 -> 1, keep one mantissa bit, round to nearest even
    odd = (mbits >> 22) & 1
    nor_code = (((mbits - (126 << 23) + (1 << 21) - 1 + odd) >> 22) & 0xFF).to(torch.uint8)
    code = torch.where(sat, torch.full_like(nor_code, 7), torch.where(den, den_code, nor_code)) | sign
    code = code.reshape(R, N)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), scale_byte.contiguous()


def quantize_mxfp4(tensor: torch.Tensor, rows_per_chunk: int = 1 << 16):
    """MXFP4 block-32 quantisation along the last dim of a [B, M, N] (or [R, N]) tensor.
    Returns (uint8 [..., N/2] e2m1 pairs, even element in the low nibble;
             uint8 [rows, N/32] E8M0 exponents) - the layout of reference.py:88-113 without the
    row/column padding aiter may add to the scale plane."""
    shape = tensor.shape
    N = shape[-1]
    assert N % MX_BLOCK == 0
    x2 = tensor.reshape(-1, N)
    codes = torch.empty(x2.shape[0], N // 2, dtype=torch.uint8, device=tensor.device)
    scales = torch.empty(x2.shape[0], N // MX_BLOCK, dtype=torch.uint8, device=tensor.device)
    for r0 in range(0, x2.shape[0], rows_per_chunk):
        c, s = _mxfp4_rows(x2[r0:r0 + rows_per_chunk].to(torch.float32))
        codes[r0:r0 + rows_per_chunk] = c
        scales[r0:r0 + rows_per_chunk] = s
    return codes.reshape(*shape[:-1], N // 2), scales


_E2M1 = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def dequantize_mxfp4(fp4_data: torch.Tensor, scale_e8m0: torch.Tensor, orig_shape, dtype=torch.bfloat16):
    """Inverse of quantize_mxfp4 (reference.py:116-154): trims a padded scale plane to
    [:rows, :N/32]."""
    N = orig_shape[-1]
    rows = 1
    for d in orig_shape[:-1]:
        rows *= d
    lut = torch.tensor(_E2M1 + [-v for v in _E2M1], dtype=torch.float32, device=fp4_data.device)
    b = fp4_data.reshape(rows, N // 2).view(torch.uint8).to(torch.int64)
    vals = torch.empty(rows, N, dtype=torch.float32, device=fp4_data.device)
    vals[:, 0::2] = lut[b & 0xF]
    vals[:, 1::2] = lut[b >> 4]
    sc = scale_e8m0.view(torch.uint8)[:rows, : N // MX_BLOCK].to(torch.float32)
    sc = torch.exp2(sc - 127.0)
    out = vals.reshape(rows, N // MX_BLOCK, MX_BLOCK) * sc.unsqueeze(-1)
    return out.reshape(orig_shape).to(dtype)


def quantize_hybrid(kv_bf16: torch.Tensor):
    """[T, 1, 576] bf16 -> hybrid cache: the 512 latent dims as MXFP4 (E8M0 per 32), the 64 rope
    dims as e4m3fn with one per-tensor scale.  Returns
    (latent codes u8 [T,1,256], latent E8M0 u8 [T,16], rope e4m3fn [T,1,64], rope scale f32[1])."""
    lat_codes, lat_scales = quantize_mxfp4(kv_bf16[..., :KV_LORA_RANK])
    rope, rope_scale = quantize_fp8(kv_bf16[..., KV_LORA_RANK:].contiguous())
    return lat_codes, lat_scales, rope, rope_scale


# --------------------------------------------------------------------------------------------
# generator
# --------------------------------------------------------------------------------------------

def generate_input(batchsize: int, qseqlen: int, kvseqlen: int, seed: int, *, num_heads: int = NUM_HEADS,
                   kv_lens=None, shuffle_pages: bool = False, sm_scale: float | None = None,
                   formats=("bf16", "fp8", "mxfp4"), device="cuda", generator_device="cpu"):
    """Same contract as reference.generate_input (reference.py:288-346):
    returns (q, kv_data, qo_indptr, kv_indptr, config) with
      q          [batch*q_len, heads, 576] bf16 ~ N(0,1)
      kv_data    {"bf16": [T,1,576], "fp8": (e4m3fn [T,1,576], f32[1]),
                  "mxfp4": (u8 [T,1,288], u8 [T,18]), "hybrid": (see quantize_hybrid)}
      indptrs    int32 [batch+1]
    q is drawn before kv from one seeded generator, the reference's order.  With the default
    generator_device="cpu" the draw and the quantisers run on the host (the same bytes with or without a
    GPU, which is what the oracle comparisons need) and therefore differ from the reference's tensors for
    equal seeds; generator_device="cuda" draws from torch.Generator(device="cuda") exactly as the
    reference does (reference.py:299-315) and quantises on the GPU.

    Extensions: `kv_lens` (ragged lengths; kvseqlen is then only recorded in config),
    `shuffle_pages` (page_size-1 page table: config["kv_indices"] is a seeded permutation of the
    slot pool and the cache rows are stored in slot order), `num_heads`, `formats`.
    """
    gen = torch.Generator(device=generator_device)
    gen.manual_seed(seed)
    gdev = torch.device(generator_device)
    lens = [kvseqlen] * batchsize if kv_lens is None else [int(v) for v in kv_lens]
    assert len(lens) == batchsize
    total_q = batchsize * qseqlen
    total_kv = sum(lens)

    q = torch.randn((total_q, num_heads, QK_HEAD_DIM), dtype=torch.bfloat16, generator=gen, device=gdev)
    kv_logical = torch.randn((total_kv, NUM_KV_HEADS, QK_HEAD_DIM), dtype=torch.bfloat16, generator=gen, device=gdev)

    config = {
        "batch_size": batchsize, "num_heads": num_heads, "num_kv_heads": NUM_KV_HEADS,
        "qk_head_dim": QK_HEAD_DIM, "kv_lora_rank": KV_LORA_RANK, "qk_rope_head_dim": QK_ROPE_HEAD_DIM,
        "v_head_dim": V_HEAD_DIM, "q_seq_len": qseqlen, "kv_seq_len": kvseqlen,
        "sm_scale": SM_SCALE if sm_scale is None else sm_scale,
        "total_kv": total_kv,
    }
    if shuffle_pages:
        perm = torch.randperm(total_kv, generator=gen, device=gdev)   # logical token i lives in slot perm[i]
        kv_store = torch.empty_like(kv_logical)
        kv_store[perm] = kv_logical
        config["kv_indices"] = perm.to(torch.int32).to(device)
        config["page_size"] = 1
    else:
        kv_store = kv_logical

    kv_data = {}
    if "bf16" in formats:
        kv_data["bf16"] = kv_store.to(device)
    if "fp8" in formats:
        c, s = quantize_fp8(kv_store)
        kv_data["fp8"] = (c.to(device), s.to(device))
    if "mxfp4" in formats:
        c, s = quantize_mxfp4(kv_store)
        kv_data["mxfp4"] = (c.to(device), s.to(device))
    if "hybrid" in formats:
        kv_data["hybrid"] = tuple(t.to(device) for t in quantize_hybrid(kv_store))

    qo_indptr = (torch.arange(0, batchsize + 1, dtype=torch.int32) * qseqlen).to(device)
    kv_indptr = torch.zeros(batchsize + 1, dtype=torch.int32)
    kv_indptr[1:] = torch.cumsum(torch.tensor(lens, dtype=torch.int64), 0).to(torch.int32)
    if kv_lens is not None:
        config["kv_lens"] = lens
    return (q.to(device), kv_data, qo_indptr, kv_indptr.to(device), config)
