"""The CPU oracle against vectors produced by executing the reference's own Python
(tests/golden/make_golden.py): this is what pins the oracle."""
import numpy as np
import torch

from helpers import bf16_from_bits
from oracle import c_oracle as co
from oracle import mla_oracle as mo

SM = 1.0 / 576 ** 0.5


def test_fp8_quantiser_matches_reference(golden):
    x = bf16_from_bits(golden["fp8q_in_bf16bits"])
    codes, scale = mo.quantize_fp8_per_tensor(x)
    assert np.array_equal(codes.numpy(), golden["fp8q_codes"])
    assert float(scale) == float(golden["fp8q_scale"][0])


def test_fp8_tables_agree_with_torch():
    b = torch.arange(256, dtype=torch.uint8)
    ref = b.view(torch.float8_e4m3fn).to(torch.float32).numpy()
    mine = mo.e4m3fn_table()
    assert np.array_equal(np.isnan(ref), np.isnan(mine))
    assert np.array_equal(ref[~np.isnan(ref)], mine[~np.isnan(mine)])
    lib = co.lib()
    c = np.array([lib.mo_e4m3fn_to_float(int(i)) for i in range(256)], dtype=np.float32)
    assert np.array_equal(c[~np.isnan(c)], mine[~np.isnan(mine)])
    x = torch.randn(4096) * 50
    enc = mo.fp8_e4m3_encode(x.numpy())
    assert np.array_equal(enc, x.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy())


def test_mxfp4_quantiser_matches_reference(golden):
    c, s = mo.quantize_mxfp4(golden["mxq_in"])
    assert np.array_equal(s, golden["mxq_scales"])
    assert np.array_equal(c, golden["mxq_codes"])
    cc, sc = co.quantize_mxfp4(golden["mxq_in"])
    assert np.array_equal(sc, golden["mxq_scales"])
    assert np.array_equal(cc, golden["mxq_codes"])


def test_mxfp4_quantiser_matches_reference_on_kv_rows(golden):
    kv = bf16_from_bits(golden["dec_kv_bf16bits"]).float().reshape(-1, 576).numpy()
    c, s = mo.quantize_mxfp4(kv)
    assert np.array_equal(c, golden["dec_mx_codes"])
    assert np.array_equal(s, golden["dec_mx_scales"])


def test_e2m1_and_e8m0_decode(golden):
    assert np.array_equal(mo.e2m1_table(), golden["e2m1_decode"])
    lib = co.lib()
    assert [lib.mo_e2m1_to_float(i) for i in range(16)] == list(golden["e2m1_decode"])
    b = np.array([0, 1, 126, 127, 128, 254], dtype=np.uint8)
    assert np.array_equal(mo.e8m0_decode(b), np.array([2.0 ** -127, 2.0 ** -126, 0.5, 1.0, 2.0, 2.0 ** 127], np.float32))
    assert np.isnan(mo.e8m0_decode(np.array([255], np.uint8))[0])
    e8 = torch.tensor([1, 126, 127, 128, 254], dtype=torch.uint8).view(torch.float8_e8m0fnu).float().numpy()
    assert np.array_equal(mo.e8m0_decode(np.array([1, 126, 127, 128, 254], np.uint8)), e8)


def _bf16_ulp_close(a: torch.Tensor, b: torch.Tensor):
    a, b = a.float(), b.float()
    tol = torch.maximum(a.abs(), b.abs()) * 2.0 ** -7 + 1e-6      # one bf16 ulp
    assert ((a - b).abs() <= tol).all(), (a - b).abs().max()


def test_decode_matches_reference_fp8_kernel(golden):
    q = bf16_from_bits(golden["dec_q_bf16bits"])
    kv = (torch.from_numpy(golden["dec_fp8_codes"]).reshape(-1, 576), torch.from_numpy(golden["dec_fp8_scale"]))
    o = mo.decode_from_data(q, None, "fp8", kv, golden["dec_kv_indptr"], None, SM)
    _bf16_ulp_close(o, bf16_from_bits(golden["dec_fp8_out_bf16bits"]))


def test_fp8_q_decode_matches_reference_chain(golden):
    """Quantiser + decode in one fixture: the reference's quantize_fp8 on Q, then its Triton FP8 kernel on
    the e4m3 values with the Q scale folded into the softmax scale."""
    q = bf16_from_bits(golden["dec_q_bf16bits"])
    codes, scale = mo.quantize_fp8_per_tensor(q)
    assert np.array_equal(codes.numpy(), golden["dec_q8_codes"])
    assert float(scale) == float(golden["dec_q8_scale"][0])
    kv = (torch.from_numpy(golden["dec_fp8_codes"]).reshape(-1, 576), torch.from_numpy(golden["dec_fp8_scale"]))
    o = mo.decode_from_data(codes, scale, "fp8", kv, golden["dec_kv_indptr"], None, SM)
    _bf16_ulp_close(o, bf16_from_bits(golden["dec_fp8q_out_bf16bits"]))


def test_decode_matches_reference_mxfp4_kernel(golden):
    q = bf16_from_bits(golden["dec_q_bf16bits"])
    kv = (torch.from_numpy(golden["dec_mx_codes"]), torch.from_numpy(golden["dec_mx_scales"]))
    o = mo.decode_from_data(q, None, "mxfp4", kv, golden["dec_kv_indptr"], None, SM)
    _bf16_ulp_close(o, bf16_from_bits(golden["dec_mx_out_bf16bits"]))


def test_c_restatement_agrees_with_python_oracle(golden):
    q = bf16_from_bits(golden["dec_q_bf16bits"]).float()
    ip = golden["dec_kv_indptr"]
    for fmt, planes, scales, kv in (
        ("fp8", [golden["dec_fp8_codes"].reshape(-1, 576)], (float(golden["dec_fp8_scale"][0]), 1.0),
         (torch.from_numpy(golden["dec_fp8_codes"]).reshape(-1, 576), torch.from_numpy(golden["dec_fp8_scale"]))),
        ("mxfp4", [golden["dec_mx_codes"], golden["dec_mx_scales"]], (1.0, 1.0),
         (torch.from_numpy(golden["dec_mx_codes"]), torch.from_numpy(golden["dec_mx_scales"]))),
    ):
        oc, lc = co.mla_decode(q.numpy(), fmt, planes, scales, ip, None, 16, 1, True, SM)
        op, lp = mo.mla_decode(q, mo.dequant_kv(fmt, kv), ip, None, SM)
        assert np.abs(oc - op.numpy()).max() < 2e-5
        assert np.abs(lc - lp.numpy()).max() < 2e-5


def test_paged_hybrid_causal_c_vs_python():
    g = torch.Generator().manual_seed(7)
    B, H, QL = 3, 16, 2
    lens = [5, 0, 37]
    T = sum(lens)
    kvf = torch.randn(T + 9, 576, generator=g)
    lat_c, lat_s = mo.quantize_mxfp4(kvf[:, :512].numpy())
    rope_c, rope_s = mo.quantize_fp8_per_tensor(kvf[:, 512:].bfloat16())
    perm = torch.randperm(T + 9, generator=g)[:T].numpy().astype(np.int32)
    ip = np.array([0, 5, 5, 42], np.int32)
    q = torch.randn(B * QL, H, 576, generator=g)
    kv = (torch.from_numpy(lat_c), torch.from_numpy(lat_s), rope_c, rope_s)
    kf = mo.dequant_kv("hybrid", kv)
    op, lp = mo.mla_decode(q, kf, ip, perm, 0.07, q_len=QL, causal=True)
    oc, lc = co.mla_decode(q.numpy(), "hybrid", [lat_c, lat_s, rope_c.numpy()], (1.0, float(rope_s)), ip, perm,
                           H, QL, True, 0.07)
    assert np.abs(oc - op.numpy()).max() < 2e-5
    assert np.array_equal(np.isinf(lc), np.isinf(lp.numpy()))
    fin = ~np.isinf(lc)
    assert np.abs(lc[fin] - lp.numpy()[fin]).max() < 2e-5
    # the empty sequence gives zeros and -inf; the first query of a pair sees one key fewer
    assert (op[2:4] == 0).all() and torch.isinf(lp[2:4]).all()
    o1, _ = mo.mla_decode(q[0:1], kf, np.array([0, 4], np.int32), perm, 0.07, q_len=1)
    assert torch.allclose(o1[0], op[0], atol=1e-6)


def test_merge_of_shards_equals_whole():
    g = torch.Generator().manual_seed(3)
    S, H = 300, 16
    kf = torch.randn(S, 576, generator=g)
    q = torch.randn(2, H, 576, generator=g)            # one sequence, q_len = 2
    whole, lse = mo.mla_decode(q, kf, np.array([0, S]), None, 0.05, q_len=2)
    cuts = [0, 128, 128, 290, 300]                      # includes an empty shard
    parts_o, parts_l = [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        o, l = mo.mla_decode(q, kf[a:b], np.array([0, b - a]), None, 0.05, q_len=2,
                             kv_pos_offset=[a], kv_total_len=[S])
        parts_o.append(o); parts_l.append(l)
    mo_, ml_ = mo.merge_partials(torch.stack(parts_o), torch.stack(parts_l))
    assert torch.allclose(mo_, whole, atol=1e-5)
    assert torch.allclose(ml_, lse, atol=1e-5)
