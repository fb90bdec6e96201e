"""GPU: the cache-append kernel writes the bytes the reference's quantisers produce.

Pinned twice: against the golden vectors that the reference's own quantize_fp8 / _mxfp4_quant produced for
201 cache rows (tests/golden/make_golden.py), and against the host mirror of those quantisers
(amd_optimization_challenge_b200.inputs, itself pinned by the same vectors) on larger seeded inputs with
shuffled destination slots; finally a cache filled on the device is decoded and compared with the oracle."""
import numpy as np
import pytest
import torch

from helpers import assert_close, bf16_from_bits, oracle_for_data

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    import amd_optimization_challenge_b200 as pkg
    return pkg


def test_append_reproduces_reference_quantiser_bytes(pkg, golden):
    kv = bf16_from_bits(golden["dec_kv_bf16bits"]).cuda()                      # [201, 1, 576]
    T = kv.shape[0]
    codes8 = torch.zeros(T, 576, dtype=torch.uint8, device="cuda")
    scale8 = torch.from_numpy(golden["dec_fp8_scale"]).cuda()
    st = pkg.kv_append(kv, "fp8", (codes8, scale8))
    codes4 = torch.zeros(T, 288, dtype=torch.uint8, device="cuda")
    scales4 = torch.zeros(T, 18, dtype=torch.uint8, device="cuda")
    st4 = pkg.kv_append(kv, "mxfp4", (codes4, scales4))
    torch.cuda.synchronize()
    assert int(st) == 0 and int(st4) == 0
    assert np.array_equal(codes8.cpu().numpy(), golden["dec_fp8_codes"].reshape(T, 576))
    assert np.array_equal(codes4.cpu().numpy(), golden["dec_mx_codes"])
    assert np.array_equal(scales4.cpu().numpy(), golden["dec_mx_scales"])


def test_append_matches_host_quantisers_at_shuffled_slots(pkg):
    from amd_optimization_challenge_b200 import inputs
    g = torch.Generator().manual_seed(9)
    T, pool = 5000, 6000
    gain = torch.exp2(torch.randint(-12, 9, (T, 1, 1), generator=g).float())          # rows over twenty binades
    kv = (torch.randn(T, 1, 576, generator=g) * gain).bfloat16()
    kv[3] = 0
    kv[4, 0, :32] = torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5, 4.0, 5.0, 6.0, -0.25,
                                  -0.75, -1.25, -2.5, -3.5, -5.0, -6.0, 0.125, 0.375, 0.625, 0.875, 1.125, 1.375, 2.25,
                                  2.75, 4.5, 5.5]).bfloat16()
    slots = torch.randperm(pool, generator=g)[:T].to(torch.int32)
    d_kv, d_slots = kv.cuda(), slots.cuda()
    # fp8
    h_codes, h_scale = inputs.quantize_fp8(kv)
    codes = torch.full((pool, 576), 0xEE, dtype=torch.uint8, device="cuda")
    st = pkg.kv_append(d_kv, "fp8", (codes, h_scale.cuda()), slots=d_slots)
    assert int(st) == 0
    assert torch.equal(codes[d_slots.long()].cpu(), h_codes.view(torch.uint8).reshape(T, 576))
    untouched = torch.ones(pool, dtype=torch.bool); untouched[slots.long()] = False
    assert bool((codes.cpu()[untouched] == 0xEE).all())
    # mxfp4, padded scale plane
    h_c4, h_s4 = inputs.quantize_mxfp4(kv)
    c4 = torch.zeros(pool, 288, dtype=torch.uint8, device="cuda")
    s4 = torch.zeros(pool, 32, dtype=torch.uint8, device="cuda")
    pkg.kv_append(d_kv, "mxfp4", (c4, s4), slots=d_slots)
    assert torch.equal(c4[d_slots.long()].cpu(), h_c4.reshape(T, 288))
    assert torch.equal(s4[d_slots.long()][:, :18].cpu(), h_s4)
    # hybrid
    hl, hs, hr, hrs = inputs.quantize_hybrid(kv)
    lat = torch.zeros(pool, 256, dtype=torch.uint8, device="cuda")
    ls = torch.zeros(pool, 16, dtype=torch.uint8, device="cuda")
    rope = torch.zeros(pool, 64, dtype=torch.uint8, device="cuda")
    pkg.kv_append(d_kv, "hybrid", (lat, ls, rope, hrs.cuda()), slots=d_slots)
    torch.cuda.synchronize()
    assert torch.equal(lat[d_slots.long()].cpu(), hl.reshape(T, 256))
    assert torch.equal(ls[d_slots.long()].cpu(), hs)
    assert torch.equal(rope[d_slots.long()].cpu(), hr.view(torch.uint8).reshape(T, 64))
    # a slot outside the cache is not written and is reported
    bad = d_slots.clone(); bad[7] = pool + 5
    st = pkg.kv_append(d_kv, "mxfp4", (c4, s4), slots=bad)
    assert int(st) == 1


@pytest.mark.parametrize("kv_format,q_format", [("fp8", "fp8"), ("mxfp4", "bf16"), ("hybrid", "fp8")])
def test_decode_of_a_device_filled_cache(pkg, kv_format, q_format):
    """Append in two batches (as prefill + decode steps would), then decode through custom_kernel."""
    lens = [700, 33, 260]
    data = pkg.generate_input(len(lens), 1, max(lens), seed=66, kv_lens=lens, shuffle_pages=True, formats=("bf16", kv_format))
    q, kvd, qo, kvp, cfg = data
    T = sum(lens)
    host = kvd[kv_format]
    planes = tuple(torch.zeros_like(t) if t.dim() > 1 else t for t in host)        # per-tensor scales are kept
    rows = kvd["bf16"]                                                              # stored in slot order
    all_slots = torch.arange(T, dtype=torch.int32, device="cuda")
    pkg.kv_append(rows[:500], kv_format, planes, slots=all_slots[:500])
    pkg.kv_append(rows[500:], kv_format, planes, base_slot=500)
    torch.cuda.synchronize()
    for a, b in zip(planes, host):
        assert torch.equal(a.view(torch.uint8) if a.dim() > 1 else a, b.view(torch.uint8) if b.dim() > 1 else b)
    cfg2 = dict(cfg, kv_format=kv_format, q_format=q_format)
    out = pkg.custom_kernel((q, {kv_format: planes}, qo, kvp, cfg2))
    torch.cuda.synchronize()
    assert_close(out, oracle_for_data(data, kv_format, q_format), tight=1.5e-2)
