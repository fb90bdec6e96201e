"""Generate the golden fixtures in this folder by EXECUTING THE REFERENCE'S OWN PYTHON on CPU.

Run once, by hand, in a container that has the reference checkout mounted:

    python tests/golden/make_golden.py /path/to/reference      (the path is required)

What runs (paths relative to the reference project root):

* `quantize_fp8` from competitor_submissions/mi355x_reference/reference.py:65-80.  The module
  imports the AMD-only `aiter` package at import time; a stub module stands in for it whose only
  live attribute is `dtypes.fp8 = torch.float8_e4m3fn` (the flavour gfx950 / NVIDIA use).
* `_mxfp4_quant` from mxfp4-mm/submission_v3_self_contained.py:19-72 (the in-tree copy of
  aiter's MXFP4 quantiser op), called from a three-line wrapper kernel under
  TRITON_INTERPRET=1 (Triton's numpy interpreter; no GPU involved).
* `_e2m1_decode` from mixed-mla/triton_mla_mxfp4.py:20-31, same way.
* `triton_mla_decode_fp8` (mixed-mla/triton_fp8_decode.py:233-280; bf16 Q x FP8 KV, split-KV
  stage 1 + LSE reduce) and `triton_mla_decode_mxfp4` (mixed-mla/triton_mla_mxfp4.py:234-290;
  bf16 Q x MXFP4 KV) under the interpreter, on small ragged seeded inputs.
* One FP8-Q x FP8-KV decode in a single fixture: the same Q through the reference's `quantize_fp8`,
  then `triton_mla_decode_fp8` on the e4m3 values of Q (exact in bf16) with the per-tensor Q scale
  folded into the module's softmax-scale constant for that one call - i.e. quantiser + decode as
  `ref_kernel` chains them (reference.py:349-369), evaluated by the reference's own Triton kernels.

The fixtures store the exact input bytes and the reference's outputs; nothing else in the
repository reads the reference checkout.  The tests that consume them are
tests/test_oracle_golden.py (CPU) and tests/test_gpu_parity.py (GPU).
"""
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import triton
import triton.language as tl

# Triton 3.6's CPU interpreter patches the module-level tl.* functions but not the tensor
# *method* `.floor()`, which the reference quantiser uses; route the method to the function.
tl.tensor.floor = lambda self: tl.floor(self)

# The reference quantiser adds a negative Python int to a uint32 tensor, relying on the
# two's-complement wrap of the Triton release it was written for; Triton 3.6 rejects that mix.
# Restore the older behaviour (wrap the scalar modulo 2^bits) for this script only.
import numbers
from triton.language import semantic as _sem

_orig_check = _sem.TritonSemantic.binary_op_type_checking_impl


def _wrapping_check(self, lhs, rhs, *a, **k):
    def wrap(s, t):
        if (isinstance(s, numbers.Integral) and s < 0 and not isinstance(t, numbers.Number)
                and t.type.scalar.is_int_unsigned()):
            return s % (1 << t.type.scalar.int_bitwidth)
        return s
    return _orig_check(self, wrap(lhs, rhs), wrap(rhs, lhs), *a, **k)


_sem.TritonSemantic.binary_op_type_checking_impl = _wrapping_check



def _with_elementwise_not(jit_fn):
    """Triton's compiler lowers Python `not t` on a tensor to an elementwise logical not; its CPU
    interpreter evaluates it as Python truthiness instead.  Return the reference function
    re-compiled from its own source with `not x` rewritten to `~x` (same meaning for the
    boolean tensors it is applied to), so that it can be called from an interpreted kernel."""
    import ast
    import inspect
    import textwrap

    fn = jit_fn.fn
    tree = ast.parse(textwrap.dedent(inspect.getsource(fn)))
    fdef = tree.body[0]
    fdef.decorator_list = []

    class _Rewrite(ast.NodeTransformer):
        def visit_UnaryOp(self, node):
            self.generic_visit(node)
            if isinstance(node.op, ast.Not):
                return ast.copy_location(ast.UnaryOp(op=ast.Invert(), operand=node.operand), node)
            return node

    tree = ast.fix_missing_locations(_Rewrite().visit(tree))
    ns = dict(fn.__globals__)
    exec(compile(tree, inspect.getsourcefile(fn), "exec"), ns)
    return ns[fdef.name]


mxfp4_quant_ref = None   # the reference quantiser, callable from interpreted kernels (set in main)
mm = None      # reference module mxfp4-mm/submission_v3_self_contained.py (set in main)
ref4 = None    # reference module mixed-mla/triton_mla_mxfp4.py (set in main)


@triton.jit
def _quant_rows(x_ptr, c_ptr, s_ptr, K: tl.constexpr, M: tl.constexpr):
    offs = tl.arange(0, M)[:, None] * K + tl.arange(0, K)[None, :]
    xv = tl.load(x_ptr + offs)
    c, s = mxfp4_quant_ref(xv, K, M, 32)
    tl.store(c_ptr + tl.arange(0, M)[:, None] * (K // 2) + tl.arange(0, K // 2)[None, :], c)
    tl.store(s_ptr + tl.arange(0, M)[:, None] * (K // 32) + tl.arange(0, K // 32)[None, :], s)


@triton.jit
def _dec(c_ptr, o_ptr):
    i = tl.arange(0, 16)
    tl.store(o_ptr + i, ref4._e2m1_decode(tl.load(c_ptr + i)))


@triton.jit
def _quant_kv(x_ptr, c_ptr, s_ptr, row0, K: tl.constexpr, KP: tl.constexpr, M: tl.constexpr):
    r = row0 + tl.arange(0, M)
    kk = tl.arange(0, KP)
    xv = tl.load(x_ptr + r[:, None] * K + kk[None, :], mask=kk[None, :] < K, other=0.0)
    c, s = mxfp4_quant_ref(xv, KP, M, 32)
    k2 = tl.arange(0, KP // 2)
    tl.store(c_ptr + r[:, None] * (K // 2) + k2[None, :], c, mask=k2[None, :] < K // 2)
    k32 = tl.arange(0, KP // 32)
    tl.store(s_ptr + r[:, None] * (K // 32) + k32[None, :], s, mask=k32[None, :] < K // 32)


HERE = os.path.dirname(os.path.abspath(__file__))


class _StubModule(types.ModuleType):
    """Stand-in for the AMD-only aiter package: every attribute and submodule resolves to a
    placeholder; only `dtypes.fp8` carries a real value."""
    __path__ = []

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return None


class _StubFinder:
    @staticmethod
    def find_spec(name, path=None, target=None):
        import importlib.machinery
        if name == "aiter" or name.startswith("aiter."):
            return importlib.machinery.ModuleSpec(name, _StubLoader(), is_package=True)
        return None


class _StubLoader:
    @staticmethod
    def create_module(spec):
        m = _StubModule(spec.name)
        if spec.name == "aiter":
            m.dtypes = types.SimpleNamespace(fp8=torch.float8_e4m3fn)
        return m

    @staticmethod
    def exec_module(module):
        pass


def _stub_aiter():
    sys.meta_path.insert(0, _StubFinder)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str):
    _stub_aiter()
    probdir = os.path.join(ref_root, "competitor_submissions", "mi355x_reference")
    sys.path.insert(0, ref_root)                                   # utils.py
    sys.path.insert(0, probdir)                                    # task.py, reference.py
    sys.path.insert(0, os.path.join(ref_root, "mixed-mla"))
    sys.path.insert(0, os.path.join(ref_root, "mxfp4-mm"))
    global mm, ref4, mxfp4_quant_ref
    import reference as ref                                        # noqa: E402
    import submission_v3_self_contained as mm                      # noqa: E402
    import triton_mla_mxfp4 as ref4                                # noqa: E402
    import triton_fp8_decode as ref8                               # noqa: E402

    mxfp4_quant_ref = _with_elementwise_not(mm._mxfp4_quant)
    out = {}

    # ---- 1. per-tensor FP8 quantiser -------------------------------------------------------
    g = torch.Generator().manual_seed(20240611)
    x = torch.randn(64, 1, 576, generator=g, dtype=torch.float32).to(torch.bfloat16)
    x[0, 0, :8] = torch.tensor([0.0, -0.0, 1e-4, -1e-4, 3.0, -3.0, 5.5, -7.25]).to(torch.bfloat16)
    codes, scale = ref.quantize_fp8(x)
    out["fp8q_in_bf16bits"] = bf16_bits(x)
    out["fp8q_codes"] = codes.view(torch.uint8).numpy()
    out["fp8q_scale"] = scale.numpy()

    # ---- 2. MXFP4 quantiser ----------------------------------------------------------------
    M, K = 32, 64
    xq = torch.randn(M, K, generator=g) * torch.logspace(-3, 3, M).reshape(M, 1)
    xq = xq.to(torch.bfloat16).to(torch.float32)
    # crafted rows: exact ties, saturation, subnormal boundary, zeros, mantissa-1.75 boundary
    xq[0, :32] = torch.tensor([0.0, 0.25, 0.5, 0.75, 1.0, 1.25, 1.5, 1.75, 2.0, 2.5, 3.0, 3.5,
                               4.0, 5.0, 6.0, -0.25, -0.75, -1.25, -2.5, -3.5, -5.0, -6.0,
                               0.125, 0.375, 0.625, 0.875, 1.125, 1.375, 2.25, 2.75, 4.5, 5.5])
    xq[1, :32] = 0.0
    xq[2, :32] = torch.linspace(-7.0, 7.0, 32)           # amax 7 = 1.75 * 4 -> rounds up
    xq[3, :32] = torch.linspace(-6.9375, 6.9375, 32)     # just below the 1.75 boundary
    xq[4, :32] = torch.linspace(-1e-30, 1e-30, 32)
    cq = torch.zeros(M, K // 2, dtype=torch.uint8)
    sq = torch.zeros(M, K // 32, dtype=torch.uint8)
    _quant_rows[(1,)](xq, cq, sq, K=K, M=M)
    out["mxq_in"] = xq.numpy()
    out["mxq_codes"] = cq.numpy()
    out["mxq_scales"] = sq.numpy()

    # ---- 3. e2m1 decode of all 16 codes ----------------------------------------------------
    c16 = torch.arange(16, dtype=torch.int32)
    o16 = torch.zeros(16, dtype=torch.float32)
    _dec[(1,)](c16, o16)
    out["e2m1_decode"] = o16.numpy()

    # ---- 4/5. the two AITER-free decode kernels on a small ragged case ----------------------
    B = 2
    lens = [70, 131]
    T = sum(lens)
    q = torch.randn(B, 16, 576, generator=g).to(torch.bfloat16)
    kv = torch.randn(T, 1, 576, generator=g).to(torch.bfloat16)
    kv_indptr = torch.tensor([0, lens[0], T], dtype=torch.int32)
    cfg = {"batch_size": B, "kv_seq_len": max(lens)}
    kv8, s8 = ref.quantize_fp8(kv)
    o8 = ref8.triton_mla_decode_fp8(q, kv8, s8, kv_indptr, cfg).clone()
    out["dec_q_bf16bits"] = bf16_bits(q)
    out["dec_kv_bf16bits"] = bf16_bits(kv)
    out["dec_kv_indptr"] = kv_indptr.numpy()
    out["dec_fp8_codes"] = kv8.view(torch.uint8).numpy()
    out["dec_fp8_scale"] = s8.numpy()
    out["dec_fp8_out_bf16bits"] = bf16_bits(o8)

    # FP8 Q: quantiser + decode in one fixture.  The e4m3 codes of Q are exact in bf16; their per-tensor
    # scale multiplies every score, so it rides on the softmax scale the kernel reads from its module.
    q8, qs8 = ref.quantize_fp8(q)
    sm_saved = ref8.SM_SCALE
    ref8.SM_SCALE = sm_saved * float(qs8)
    try:
        o88 = ref8.triton_mla_decode_fp8(q8.to(torch.float32).to(torch.bfloat16), kv8, s8, kv_indptr, cfg).clone()
    finally:
        ref8.SM_SCALE = sm_saved
    out["dec_q8_codes"] = q8.view(torch.uint8).numpy()
    out["dec_q8_scale"] = qs8.numpy()
    out["dec_fp8q_out_bf16bits"] = bf16_bits(o88)

    # MXFP4 bytes for the same rows, produced by the reference quantiser (row blocks of 16)
    kv2 = kv.reshape(T, 576).to(torch.float32)
    c4 = torch.zeros(T, 288, dtype=torch.uint8)
    s4 = torch.zeros(T, 18, dtype=torch.uint8)

    Tp = (T + 15) // 16 * 16
    kvp = torch.zeros(Tp, 576); kvp[:T] = kv2
    c4p = torch.zeros(Tp, 288, dtype=torch.uint8); s4p = torch.zeros(Tp, 18, dtype=torch.uint8)
    for r0 in range(0, Tp, 16):
        _quant_kv[(1,)](kvp, c4p, s4p, r0, K=576, KP=1024, M=16)
    c4, s4 = c4p[:T].clone(), s4p[:T].clone()
    o4 = ref4.triton_mla_decode_mxfp4(q, c4.reshape(T, 1, 288), s4, kv_indptr, cfg).clone()
    out["dec_mx_codes"] = c4.numpy()
    out["dec_mx_scales"] = s4.numpy()
    out["dec_mx_out_bf16bits"] = bf16_bits(o4)

    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors.npz"),
          {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
