"""TEST INFRASTRUCTURE — writes a PATCHED COPY of three reference files into oracle/_ref/patched/
(git-ignored; nothing of the reference is kept in this repository) to exercise the call-site
changes a DadGPT maintainer would make to use what lies beyond the reference's three
fused-attention signatures. The reference tree itself is never modified.

    python oracle/patch_reference.py /path/to/DadGPT [out_dir]

Edits (each anchored on a short, unique piece of reference text; the script stops if an anchor
is missing, i.e. if the reference has changed):

  src/model.cpp
    * use_fused_attention (src/model.cpp:185-197) no longer declines when attention dropout is
      on: the fused kernels take the dropout themselves;
    * the fused branch of model_forward (src/model.cpp:390-394) calls
      gpu_flash_attention_forward_dropout when dropout is on, with the seed the materialized
      branch's gpu_dropout_forward would have consumed (taken from, and advancing, the same
      counter), and remembers it per layer;
    * the fused branch of model_backward (src/model.cpp:568-574) passes that seed to
      gpu_flash_attention_backward_dropout;
    * the attention part of model_forward_cached (src/model.cpp:745-790, 61 launches per layer
      at 12 heads) becomes one gpu_decode_attention call.
  cuda/gpu_ops.cu, cuda/gpu_ops.cuh
    * gpu_dropout_take_seed(): returns the dropout seed counter (cuda/gpu_ops.cu:704) and
      advances it, exactly as gpu_dropout_forward does (cuda/gpu_ops.cu:732).
"""
from __future__ import annotations

import os
import re
import sys


def sub_once(text: str, pattern: str, repl, what: str, flags=re.S) -> str:
    new, n = re.subn(pattern, repl, text, count=1, flags=flags)
    if n != 1:
        raise SystemExit(f"patch_reference: anchor not found: {what}")
    return new


def patch_model(src: str) -> str:
    # includes + per-layer seed store
    src = sub_once(src, r'(#include "model.hpp"\n)',
                   r'\1#include "dadattn_gpu_ops.hpp"\n', "model.hpp include", 0)
    src = sub_once(src, r'(\nbool use_fused_attention\()',
                   "\n// seed of each layer's attention dropout, from forward to backward\n"
                   "static unsigned long long g_fused_attn_seed[256];\n\\1", "use_fused_attention")
    # 1. dropout no longer rules out the fused path
    src = sub_once(src, r'if \(attn_dropout \|\| !gpu_flash_attention_supported\(',
                   'if (!gpu_flash_attention_supported(', "dropout condition", 0)
    # 2. forward
    def fwd(m):
        args = m.group(1)
        return ("if (attn_dropout) {\n"
                "        g_fused_attn_seed[l] = gpu_dropout_take_seed();\n"
                f"        gpu_flash_attention_forward_dropout({args}, model.dropout_rate,\n"
                "                                            g_fused_attn_seed[l]);\n"
                "      } else {\n"
                f"        gpu_flash_attention_forward({args});\n"
                "      }")
    src = sub_once(src, r'gpu_flash_attention_forward\((.*?)\);', fwd, "forward call")
    # 3. backward
    def bwd(m):
        args = m.group(1)
        return ("if (attn_dropout) {\n"
                f"        gpu_flash_attention_backward_dropout({args}, model.dropout_rate,\n"
                "                                             g_fused_attn_seed[l]);\n"
                "      } else {\n"
                f"        gpu_flash_attention_backward({args});\n"
                "      }")
    src = sub_once(src, r'gpu_flash_attention_backward\(\s*(.*?)\);', bwd, "backward call")
    # 4. cached decode: from the cache append to just before the output projection
    start = src.index("// Store K, V into cache at position pos")
    start = src.rindex("\n", 0, start) + 1
    end = src.index("// Output projection", start)
    end = src.rindex("\n", 0, end) + 1
    call = ("    // append k, v at `pos` and attend over rows 0..pos of every head: one launch\n"
            "    gpu_decode_attention(attn_out_buf, q_buf, k_buf, v_buf, cache.k_cache[l], cache.v_cache[l],\n"
            "                         c.n_heads, cache.max_len, dh, pos,\n"
            "                         1.0f / std::sqrt(static_cast<float>(dh)));\n\n")
    return src[:start] + call + src[end:]


def patch_gpu_ops_cu(src: str) -> str:
    return sub_once(src, r'(void gpu_dropout_init\(unsigned long long seed, int[^\n]*\n)',
                    r'\1unsigned long long gpu_dropout_take_seed() { return d_dropout_seed++; }\n',
                    "gpu_dropout_init definition", 0)


def patch_gpu_ops_cuh(src: str) -> str:
    return sub_once(src, r'(void gpu_dropout_free\(\);\n)',
                    r'\1// the seed the next gpu_dropout_forward would use; advances the counter like it\n'
                    r'unsigned long long gpu_dropout_take_seed();\n', "gpu_dropout_free declaration", 0)


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = sys.argv[1]
    out = sys.argv[2] if len(sys.argv) > 2 else os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                                             "_ref", "patched")
    os.makedirs(out, exist_ok=True)
    jobs = (("src/model.cpp", "model.cpp", patch_model),
            ("cuda/gpu_ops.cu", "gpu_ops.cu", patch_gpu_ops_cu),
            ("cuda/gpu_ops.cuh", "gpu_ops.cuh", patch_gpu_ops_cuh))
    for rel, name, fn in jobs:
        with open(os.path.join(ref, rel)) as f:
            text = f.read()
        with open(os.path.join(out, name), "w") as f:
            f.write(fn(text))
    print(out)


if __name__ == "__main__":
    main()
