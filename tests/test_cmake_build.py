"""CPU: the CMake build (CMakeLists.txt at the repository root) configures and builds the two
libraries for sm_100a and nothing else, from the same sources as dadgpt_b200/build.py, and what
it builds exports every symbol include/dadattn.h declares. nvcc cross-compiles, so no GPU is
needed. Where the reference tree is present, the integration target (the reference's own
model.cpp, train.cpp and generate.cpp linked against the libraries) is built as well."""
import ctypes
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(cmd, **kw):
    r = subprocess.run(cmd, capture_output=True, text=True, **kw)
    assert r.returncode == 0, f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}"
    return r.stdout + r.stderr


@pytest.mark.timeout(1200)
def test_cmake_configures_and_builds_for_sm100a_only(tmp_path):
    if not shutil.which("cmake") or not shutil.which("nvcc"):
        pytest.skip("cmake or nvcc not installed")
    gen = ["-G", "Ninja"] if shutil.which("ninja") else []
    build = str(tmp_path / "build")
    args = ["cmake", "-S", ROOT, "-B", build, *gen]
    from oracle.oracle import reference_dir
    ref = reference_dir()
    json_inc = None
    if ref:
        import sysconfig
        cand = os.path.join(sysconfig.get_paths()["purelib"], "include", "cudnn_frontend", "thirdparty")
        if os.path.exists(os.path.join(cand, "nlohmann", "json.hpp")):
            json_inc = cand
            args += [f"-DDADGPT_REFERENCE_DIR={ref}", f"-DDADGPT_JSON_INCLUDE_DIR={cand}"]
    _run(args)
    _run(["cmake", "--build", build, "--parallel", str(os.cpu_count() or 4)])
    lib = os.path.join(build, "libdadattn.so")
    shim = os.path.join(build, "libdadattn_gpuops.so")
    assert os.path.exists(lib) and os.path.exists(shim)
    # one architecture in every CUDA compile command
    cmds = open(os.path.join(build, "compile_commands.json")).read() if os.path.exists(
        os.path.join(build, "compile_commands.json")) else ""
    ninja = os.path.join(build, "build.ninja")
    text = cmds + (open(ninja).read() if os.path.exists(ninja) else "")
    archs = set(re.findall(r"arch=compute_(\w+)", text))
    assert archs == {"100a"}, archs
    # same exported C ABI as the header declares
    header = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "dadattn.h")).read(), flags=re.S)
    handle = ctypes.CDLL(lib)
    for name in sorted(set(re.findall(r"\b(dadattn_[a-z0-9_]+)\s*\(", header))):
        assert hasattr(handle, name), name
    syms = _run(["nm", "-D", "--defined-only", shim])
    assert "_Z27gpu_flash_attention_forwardPfS_PKfS1_S1_iiif" in syms
    if json_inc:
        assert os.path.exists(os.path.join(build, "dadgpt_link_check"))


def test_cmake_refuses_other_architectures(tmp_path):
    if not shutil.which("cmake"):
        pytest.skip("cmake not installed")
    r = subprocess.run(["cmake", "-S", ROOT, "-B", str(tmp_path / "b"), "-DCMAKE_CUDA_ARCHITECTURES=90"],
                       capture_output=True, text=True)
    assert r.returncode != 0 and "sm_100a only" in (r.stdout + r.stderr)
