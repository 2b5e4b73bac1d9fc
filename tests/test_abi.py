"""CPU tests of the boundary: the shared library loads, exports exactly what the header declares, the
ctypes table covers it, and the host-side helpers behave like the reference's. No compute call is made."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def header_functions():
    text = (ROOT / "include" / "webllm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"WB_API\s+(?:const\s+char\s*\*|int)\s*(wb_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = header_functions()
    assert "wb_linear" in names and "wb_gptq_register" in names and len(names) >= 30


def test_library_exports_every_declared_symbol(built_lib):
    out = subprocess.run(["nm", "-D", "--defined-only", str(built_lib)], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r"\sT\s+(wb_\w+)", out))
    declared = set(header_functions())
    assert declared - exported == set(), f"declared but not exported: {sorted(declared - exported)}"
    assert exported - declared == set(), f"exported but not declared: {sorted(exported - declared)}"


def test_ctypes_table_matches_header(built_lib):
    from webllm_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_functions()
    lib = _lib.load()
    assert lib.wb_version() >= 100
    assert isinstance(lib.wb_last_error(), bytes)


def test_library_does_not_depend_on_torch_or_the_oracle(built_lib):
    out = subprocess.run(["ldd", str(built_lib)], capture_output=True, text=True, check=True).stdout
    assert "torch" not in out and "oracle" not in out


def test_null_context_is_an_error_not_a_crash(built_lib):
    from webllm_b200 import _lib
    lib = _lib.load()
    assert lib.wb_synchronize(None) == _lib.WB_ERR_BAD_ARG
    assert b"NULL" in lib.wb_last_error()


def test_product_never_imports_the_oracle():
    for py in (ROOT / "webllm_b200").rglob("*.py"):
        assert not re.search(r"^\s*(from|import)\s+oracle|oracle/|_build", py.read_text(), flags=re.M), py
    for cu in (ROOT / "webllm_b200" / "csrc").iterdir():
        assert "oracle" not in cu.read_text(), cu


def test_align_and_tensor():
    from webllm_b200 import ALIGN, Tensor, align_to
    assert ALIGN == 256 and align_to(1) == 256 and align_to(256) == 256 and align_to(257) == 512 and align_to(0) == 0
    t = Tensor(512, 10, [2, 5])
    assert t.nbytes == 40 and Tensor(0, 3, [3], "f16").nbytes == 6


def test_plan_gemv_split_matches_reference_table():
    """The schedule listed in src/model/qwen.ts:54-59 for Qwen2.5-0.5B."""
    from webllm_b200.plan import plan_gemv_split
    wg = lambda n: -(-n // 256)
    assert plan_gemv_split(wg(128), 896) == 64      # k/v_proj
    assert plan_gemv_split(wg(896), 896) == 64      # q/o_proj
    assert plan_gemv_split(wg(896), 4864) == 64     # down_proj
    assert plan_gemv_split(wg(4864), 896) == 16     # gate/up
    assert plan_gemv_split(wg(151936), 896) == 1    # lm_head
    assert plan_gemv_split(1, 42) == 1              # no legal split


def test_synthetic_packing_round_trip(oracle):
    """The synthetic generators emit the checkpoint packing the oracle (and so the reference) reads."""
    import numpy as np
    from webllm_b200 import synthetic
    t = synthetic.random_gptq(136, 24, group=8, seed=5, zeros="any")
    a = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, t.scales.astype(np.float32), 136, 24, 8)
    b = synthetic.dequant_numpy(t)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    W = np.random.default_rng(1).normal(0, 0.02, size=(24, 256)).astype(np.float32)
    r = synthetic.rtn_quantize(W, 128)
    back = oracle.dequantize_gptq_int4(r.qweight, r.qzeros, r.scales.astype(np.float32), 256, 24, 128)
    assert np.max(np.abs(back - W)) <= 0.51 * float(r.scales.astype(np.float32).max()) + 1e-6
