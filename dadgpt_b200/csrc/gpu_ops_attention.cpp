// Drop-in translation unit for DadGPT: defines the three C++ functions that the reference
// declares in cuda/gpu_ops.cuh:115-122 and implements in cuda/attention.cu:232-252, on top of the
// dadattn C ABI. Link this (and libdadattn) in place of cuda/attention.cu and the reference's
// src/model.cpp, src/train.cpp and src/generate.cpp build and run unchanged.
//
// Precision: with dadattn_set_f32_precision(1) (or DADATTN_PRECISION=bf16 in the environment)
// head size 64 runs on the bf16 tensor-core kernels, operands rounded on the fly as the
// reference's own GEMMs do under gpu_set_matmul_precision(BF16); the workspace that needs comes
// from the library's grow-only scratch buffer, since these signatures cannot carry one.
//
// Behaviour kept from the reference: work is enqueued on the legacy default stream without
// synchronising; a head size outside {32, 64} and any CUDA error surface as std::runtime_error
// (cuda/attention.cu:238,251; CUDA_CHECK in cuda/gpu_ops.cuh:10-17).
#include <stdexcept>
#include <string>

#include "dadattn.h"
#include "dadattn_gpu_ops.hpp"

bool gpu_flash_attention_supported(int d_head) { return d_head == 32 || d_head == 64; }

namespace {
// the bf16 kernels want 16-byte aligned tensors; the reference's arena offsets are multiples of
// B * ctx * d_model floats, which at head size 64 always are
bool use_tensor_cores(int d_head) { return d_head == 64 && dadattn_get_f32_precision() == 1; }
}  // namespace

void gpu_flash_attention_forward(float* out, float* lse, const float* q, const float* k,
                                 const float* v, int BH, int S, int d_head, float scale) {
  if (!gpu_flash_attention_supported(d_head))
    throw std::runtime_error("flash attention: unsupported d_head " + std::to_string(d_head));
  if (use_tensor_cores(d_head)) {
    const size_t bytes = dadattn_flash_f32_via_bf16_workspace_bytes(BH, S, d_head);
    void* ws = nullptr;
    if (dadattn_library_scratch(bytes, &ws) != DADATTN_OK ||
        dadattn_flash_fwd_f32_via_bf16(out, lse, q, k, v, BH, S, d_head, scale, ws, bytes, nullptr) !=
            DADATTN_OK)
      throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
    return;
  }
  if (dadattn_flash_fwd_f32(out, lse, q, k, v, BH, S, d_head, scale, nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

void gpu_flash_attention_backward(float* dq, float* dk, float* dv, float* delta, const float* dout,
                                  const float* out, const float* lse, const float* q,
                                  const float* k, const float* v, int BH, int S, int d_head,
                                  float scale) {
  if (!gpu_flash_attention_supported(d_head))
    throw std::runtime_error("flash attention: unsupported d_head " + std::to_string(d_head));
  if (use_tensor_cores(d_head)) {
    const size_t bytes = dadattn_flash_f32_via_bf16_workspace_bytes(BH, S, d_head);
    void* ws = nullptr;
    if (dadattn_library_scratch(bytes, &ws) != DADATTN_OK ||
        dadattn_flash_bwd_f32_via_bf16(dq, dk, dv, dout, out, lse, q, k, v, BH, S, d_head, scale, ws,
                                       bytes, nullptr) != DADATTN_OK)
      throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
    return;
  }
  if (dadattn_flash_bwd_f32(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, d_head, scale,
                            nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

// ---- additions beyond the reference's three signatures (include/dadattn_gpu_ops.hpp) ----------

void gpu_flash_attention_forward_dropout(float* out, float* lse, const float* q, const float* k,
                                         const float* v, int BH, int S, int d_head, float scale,
                                         float rate, unsigned long long seed) {
  if (!gpu_flash_attention_supported(d_head))
    throw std::runtime_error("flash attention: unsupported d_head " + std::to_string(d_head));
  if (dadattn_flash_fwd_f32_dropout(out, lse, q, k, v, BH, S, d_head, scale, rate, seed, 0, 0, nullptr) !=
      DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

void gpu_flash_attention_backward_dropout(float* dq, float* dk, float* dv, float* delta,
                                          const float* dout, const float* out, const float* lse,
                                          const float* q, const float* k, const float* v, int BH,
                                          int S, int d_head, float scale, float rate,
                                          unsigned long long seed) {
  if (!gpu_flash_attention_supported(d_head))
    throw std::runtime_error("flash attention: unsupported d_head " + std::to_string(d_head));
  if (dadattn_flash_bwd_f32_dropout(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, d_head, scale, rate,
                                    seed, 0, 0, nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

void gpu_decode_attention(float* out, const float* q, const float* k_new, const float* v_new,
                          float* k_cache, float* v_cache, int n_heads, int max_len, int d_head,
                          int pos, float scale) {
  if (pos < 0 || pos >= max_len)
    throw std::out_of_range("gpu_decode_attention: pos " + std::to_string(pos) + " outside cache length " +
                            std::to_string(max_len));
  if (dadattn_decode_f32(out, q, k_new, v_new, k_cache, v_cache, n_heads, max_len, d_head, pos, scale,
                         nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

void gpu_decode_attention_batched(float* out, const float* q, const float* k_new, const float* v_new,
                                  float* k_cache, float* v_cache, int* lengths, int batch, int n_heads,
                                  int max_len, int d_head, float scale, void* workspace,
                                  size_t workspace_bytes) {
  if (dadattn_decode_f32_batched(out, q, k_new, v_new, k_cache, v_cache, lengths, batch, n_heads, d_head,
                                 max_len, scale, workspace, workspace_bytes, nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

void gpu_kv_cache_fill(float* k_cache, float* v_cache, int* lengths, const float* k_heads,
                       const float* v_heads, int b, int batch, int n_heads, int n, int max_len,
                       int d_head) {
  if (n < 1 || n > max_len) throw std::out_of_range("gpu_kv_cache_fill: bad prompt length");
  if (dadattn_kv_cache_fill(k_cache, v_cache, lengths, k_heads, v_heads, b, batch, n_heads, n, max_len,
                            d_head, 0, nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}
