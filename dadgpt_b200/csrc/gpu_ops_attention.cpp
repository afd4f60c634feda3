// Drop-in translation unit for DadGPT: defines the three C++ functions that the reference
// declares in cuda/gpu_ops.cuh:115-122 and implements in cuda/attention.cu:232-252, on top of the
// dadattn C ABI. Link this (and libdadattn) in place of cuda/attention.cu and the reference's
// src/model.cpp, src/train.cpp and src/generate.cpp build and run unchanged.
//
// Behaviour kept from the reference: work is enqueued on the legacy default stream without
// synchronising; a head size outside {32, 64} and any CUDA error surface as std::runtime_error
// (cuda/attention.cu:238,251; CUDA_CHECK in cuda/gpu_ops.cuh:10-17).
#include <stdexcept>
#include <string>

#include "dadattn.h"

bool gpu_flash_attention_supported(int d_head) { return d_head == 32 || d_head == 64; }

void gpu_flash_attention_forward(float* out, float* lse, const float* q, const float* k,
                                 const float* v, int BH, int S, int d_head, float scale) {
  if (!gpu_flash_attention_supported(d_head))
    throw std::runtime_error("flash attention: unsupported d_head " + std::to_string(d_head));
  if (dadattn_flash_fwd_f32(out, lse, q, k, v, BH, S, d_head, scale, nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}

void gpu_flash_attention_backward(float* dq, float* dk, float* dv, float* delta, const float* dout,
                                  const float* out, const float* lse, const float* q,
                                  const float* k, const float* v, int BH, int S, int d_head,
                                  float scale) {
  if (!gpu_flash_attention_supported(d_head))
    throw std::runtime_error("flash attention: unsupported d_head " + std::to_string(d_head));
  if (dadattn_flash_bwd_f32(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, d_head, scale,
                            nullptr) != DADATTN_OK)
    throw std::runtime_error(std::string("CUDA error: ") + dadattn_last_error());
}
