"""Host-side mirror of the reference problem definition (package `inputs`): quantisers bit-exact
against the independently written oracle, generator contract, round trips."""
import numpy as np
import torch

from helpers import bf16_from_bits
from oracle import mla_oracle as mo
from amd_optimization_challenge_b200 import inputs


def test_package_quantisers_match_oracle_bitwise(golden):
    x = bf16_from_bits(golden["fp8q_in_bf16bits"])
    c, s = inputs.quantize_fp8(x)
    assert np.array_equal(c.view(torch.uint8).numpy(), golden["fp8q_codes"])
    assert float(s) == float(golden["fp8q_scale"][0])
    c4, s4 = inputs.quantize_mxfp4(torch.from_numpy(golden["mxq_in"]))
    assert np.array_equal(c4.numpy(), golden["mxq_codes"])
    assert np.array_equal(s4.numpy(), golden["mxq_scales"])
    g = torch.Generator().manual_seed(11)
    big = (torch.randn(257, 576, generator=g) * torch.logspace(-6, 6, 257).reshape(-1, 1)).bfloat16()
    c5, s5 = inputs.quantize_mxfp4(big, rows_per_chunk=100)
    oc, os_ = mo.quantize_mxfp4(big.float().numpy())
    assert np.array_equal(c5.numpy(), oc) and np.array_equal(s5.numpy(), os_)


def test_mxfp4_round_trip_and_idempotence():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 1, 576, generator=g).bfloat16()
    c, s = inputs.quantize_mxfp4(x)
    d = inputs.dequantize_mxfp4(c, s, x.shape, dtype=torch.float32)
    assert np.array_equal(d.reshape(-1, 576).numpy(), mo.dequantize_mxfp4(c.reshape(-1, 288).numpy(), s.numpy()))
    # a padded scale plane (the reference's aiter op pads rows and columns) is trimmed
    sp = torch.zeros(96, 32, dtype=torch.uint8); sp[:64, :18] = s
    assert torch.equal(inputs.dequantize_mxfp4(c, sp, x.shape, dtype=torch.float32), d)
    # quantising the dequantised values again reproduces the codes
    c2, s2 = inputs.quantize_mxfp4(d)
    d2 = inputs.dequantize_mxfp4(c2, s2, x.shape, dtype=torch.float32)
    assert torch.equal(d2, d)
    # block error bound: |x - deq| <= amax-scaled half-step
    err = (d - x.float()).abs().reshape(-1, 18, 32)
    step = torch.exp2(s.float() - 127).reshape(-1, 18, 1)
    assert (err <= step + 1e-6).all()


def test_generate_input_contract():
    data = inputs.generate_input(3, 1, 40, seed=9, device="cpu", formats=("bf16", "fp8", "mxfp4", "hybrid"))
    q, kv, qo, kvp, cfg = data
    assert q.shape == (3, 16, 576) and q.dtype == torch.bfloat16
    assert kv["bf16"].shape == (120, 1, 576)
    assert kv["fp8"][0].dtype == torch.float8_e4m3fn and kv["fp8"][1].shape == (1,)
    assert kv["mxfp4"][0].shape == (120, 1, 288) and kv["mxfp4"][1].shape == (120, 18)
    lat, ls, rope, rs = kv["hybrid"]
    assert lat.shape == (120, 1, 256) and ls.shape == (120, 16) and rope.shape == (120, 1, 64) and rs.shape == (1,)
    assert qo.tolist() == [0, 1, 2, 3] and kvp.tolist() == [0, 40, 80, 120]
    for k in ("batch_size", "num_heads", "num_kv_heads", "qk_head_dim", "kv_lora_rank", "qk_rope_head_dim",
              "v_head_dim", "q_seq_len", "kv_seq_len", "sm_scale"):
        assert k in cfg
    assert abs(cfg["sm_scale"] - 576 ** -0.5) < 1e-12
    # the latent part of the hybrid cache is the MXFP4 cache restricted to its first 16 blocks
    assert torch.equal(lat.reshape(120, 256), kv["mxfp4"][0].reshape(120, 288)[:, :256])
    assert torch.equal(ls, kv["mxfp4"][1][:, :16])
    # determinism and the q-then-kv draw order
    again = inputs.generate_input(3, 1, 40, seed=9, device="cpu")
    assert torch.equal(again[0], q) and torch.equal(again[1]["bf16"], kv["bf16"])


def test_generate_input_paged_and_ragged():
    lens = [7, 0, 33, 64]
    q, kv, qo, kvp, cfg = inputs.generate_input(4, 2, 64, seed=1, kv_lens=lens, shuffle_pages=True, device="cpu",
                                                num_heads=32, sm_scale=192 ** -0.5)
    assert q.shape == (8, 32, 576) and qo.tolist() == [0, 2, 4, 6, 8]
    assert kvp.tolist() == [0, 7, 7, 40, 104]
    idx = cfg["kv_indices"]
    assert sorted(idx.tolist()) == list(range(104))
    plain = inputs.generate_input(4, 2, 64, seed=1, kv_lens=lens, device="cpu", num_heads=32)
    # token i of the logical order lives in slot idx[i]
    assert torch.equal(kv["bf16"][idx.long()], plain[1]["bf16"])
    assert cfg["sm_scale"] == 192 ** -0.5
