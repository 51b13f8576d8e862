"""The C-ABI library loads without a GPU and exports exactly what include/latentq.h declares."""
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "latentq.h")).read()
    return set(re.findall(r"LQ_API\s+[\w\s\*]+?\b(lq_\w+)\s*\(", text))


def test_library_builds_and_exports_header_symbols():
    from latentq_llm_b200 import build
    so = build.build()
    out = subprocess.check_output(["nm", "-D", "--defined-only", so], text=True)
    exported = set(re.findall(r" T (lq_\w+)", out))
    declared = _declared()
    assert len(declared) >= 28
    assert declared == exported, (declared - exported, exported - declared)


def test_binding_covers_every_declared_symbol():
    from latentq_llm_b200 import _lib
    assert set(_lib.SIGNATURES) == _declared()
    assert _lib.lib.lq_version() >= 100
    assert _lib.lib.lq_status_string(-2).decode().startswith("unsupported")


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected on the host before any launch."""
    import ctypes as C
    from latentq_llm_b200 import _lib
    null = C.c_void_p(0)
    assert _lib.lib.lq_pack_nibbles(null, null, 16, null) == _lib.LQ_EINVAL
    assert _lib.lib.lq_res3_quant(null, 0, null, 8, 2, 0.125, 2, 0.25, 4, 0.0, null) == _lib.LQ_EINVAL
    fake = C.c_void_p(4096)
    # K not a multiple of 128 -> unsupported, reported before touching the device
    assert _lib.lib.lq_gemm_a8w8(fake, fake, null, null, 1.0, null, fake, null, 8, 64, 100, null, 0, null) == _lib.LQ_EUNSUPPORTED
    assert _lib.lib.lq_gemm_a16w4_fwd(fake, fake, fake, fake, null, fake, 8, 64, 256, 48, null, 0, null) == _lib.LQ_EUNSUPPORTED
    # the split-K plan needs a workspace for a decode-sized problem
    assert _lib.lib.lq_gemm_workspace_bytes(_lib.GEMM_A16W4_FWD, 1, 4096, 4096) > 0
    assert _lib.lib.lq_gemm_workspace_bytes(_lib.GEMM_A16W4_FWD, 4096, 4096, 4096) == 0


def test_ops_refuse_cpu_tensors():
    import pytest
    import torch
    from latentq_llm_b200 import ops
    with pytest.raises(ValueError):
        ops.pack_nibbles(torch.zeros(16, dtype=torch.uint8))
