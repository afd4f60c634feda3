"""GPU: the reference's own model, training and generation code (src/model.cpp, src/train.cpp,
src/generate.cpp, cuda/gpu_ops.cu, compiled unmodified; only the PCRE2 tokenizer is a link stub)
linked against libdadattn_gpuops.so in place of its cuda/attention.cu (oracle/Makefile target
_ref/ref_model_link_check). Reproduces, at the model level, the relations the reference's tests
pin for this path: fused == materialized (tests/test_backward.cpp:432-480) and prefill + cached
decode == full forward (tests/test_model.cpp:375-414), both at 1e-4; and fused == materialized
once more with the drop-in switched to bf16 tensor-core arithmetic, at the bf16 tolerances. Then
the reference's generate_tokens (src/generate.cpp:94-139; greedy tokens after a fused prefill equal
those of the materialized model) and its run_training (src/train.cpp:96-285; three optimizer steps
on a synthetic token file, fused against materialized validation loss)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
BIN = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                   "ref_model_link_check")


def test_reference_model_runs_on_our_kernels(cuda):
    if not os.path.exists(BIN):
        pytest.skip("oracle/_ref/ref_model_link_check not built (reference tree absent at build time)")
    r = subprocess.run([BIN], capture_output=True, text=True, timeout=600)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL OK" in r.stdout
    assert r.stdout.count(" OK") >= 7
    assert "(bf16 tensor cores)" in r.stdout
    lines = r.stdout.splitlines()
    assert any(l.startswith("generate_tokens") and l.endswith(" OK") for l in lines)
    assert any(l.startswith("run_training") and l.endswith(" OK") for l in lines)


PATCHED = os.path.join(os.path.dirname(BIN), "ref_patched_check")


def test_patched_reference_model_reaches_fused_dropout_and_one_launch_decode(cuda):
    """The reference's model with the call-site edits of oracle/patch_reference.py (a patched copy
    under oracle/_ref/patched; the reference tree is untouched): attention dropout runs on the
    fused path with the seeds the materialized path would have used (same masks, same results,
    no [B*H, ctx, ctx] buffers), and model_forward_cached's attention is one launch."""
    if not os.path.exists(PATCHED):
        pytest.skip("oracle/_ref/ref_patched_check not built (reference tree absent at build time)")
    r = subprocess.run([PATCHED], capture_output=True, text=True, timeout=600)
    print(r.stdout, r.stderr)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL OK" in r.stdout
    lines = r.stdout.splitlines()
    assert sum(l.startswith("fused_dropout_vs_materialized") and l.endswith(" OK") for l in lines) == 2
    assert sum(l.startswith("prefill_then_one_launch_decode") and l.endswith(" OK") for l in lines) == 2
    assert any(l.startswith("cached_decode") and "ms/token" in l for l in lines)
    assert any(l.startswith("batched_generation 4 sequences") and l.endswith(" OK") for l in lines)
    assert any(l.startswith("batched_generation gpt2-124m") and "ms/token" in l for l in lines)
