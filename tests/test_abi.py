"""CPU: the C-ABI library builds, loads, and exports exactly what include/dadattn.h declares."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "dadattn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dadattn_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry
    entry.build()
    from dadgpt_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/dadattn.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "python binding and header disagree"


def test_no_compute_without_device_but_arguments_are_checked(lib):
    # Argument validation happens on the host before any CUDA call.
    assert lib.dadattn_flash_supported(64) == 1 and lib.dadattn_flash_supported(48) == 0
    rc = lib.dadattn_flash_fwd_f32(None, None, None, None, None, 1, 8, 64, 0.125, None)
    assert rc == -1 and b"null" in lib.dadattn_last_error()
    rc = lib.dadattn_flash_fwd_f32(1, 1, 1, 1, 1, 1, 8, 48, 0.125, None)
    assert rc == -2 and b"unsupported d_head 48" in lib.dadattn_last_error()
    rc = lib.dadattn_decode_f32(16, 16, 16, 16, 16, 16, 4, 32, 64, 32, 0.125, None)
    assert rc == -1 and b"outside context length" in lib.dadattn_last_error()
    # tickets (B*H + B uint32, padded to 256) + records [B*H][splits][D+2] fp32; 768 pairs fill
    # the GPU, so a CTA walks a whole sequence (1 split); 8 pairs get their rows split
    assert lib.dadattn_decode_workspace_bytes(64, 12, 64, 1280) == 3328 + 64 * 12 * 1 * 66 * 4
    assert lib.dadattn_decode_workspace_bytes(2, 4, 64, 1280) == 256 + 10752  # 8*5*66*4 padded to 256


def test_gpuops_shim_defines_the_reference_symbols():
    # Itanium-mangled names of the three functions declared in the reference's
    # cuda/gpu_ops.cuh:115-122; model.cpp links against exactly these.
    from dadgpt_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.SHIM_PATH], capture_output=True,
                         text=True, check=True).stdout
    for sym in ("_Z29gpu_flash_attention_supportedi",
                "_Z27gpu_flash_attention_forwardPfS_PKfS1_S1_iiif",
                "_Z28gpu_flash_attention_backwardPfS_S_S_PKfS1_S1_S1_S1_S1_iiif"):
        assert sym in out, sym
    ref_obj = os.path.join(ROOT, "oracle", "_ref", "libdadref_gpu.so")
    if os.path.exists(ref_obj):  # same names as the reference's own object code
        ref = subprocess.run(["nm", "-D", "--defined-only", ref_obj], capture_output=True,
                             text=True, check=True).stdout
        for line in out.splitlines():
            if "gpu_flash_attention" in line:
                assert line.split()[-1] in ref


def test_python_mirror_rejects_cpu_tensors():
    import torch
    import dadgpt_b200 as dad
    t = torch.zeros(1, 8, 64)
    with pytest.raises(ValueError, match="CUDA tensor"):
        dad.gpu_flash_attention_forward(t, torch.zeros(1, 8), t, t, t, 1, 8, 64, 0.125)
    assert dad.gpu_flash_attention_supported(32) and not dad.gpu_flash_attention_supported(128)
