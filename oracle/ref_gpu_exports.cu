// TEST INFRASTRUCTURE — extern "C" doors onto the REFERENCE's own CUDA code.
//
// Compiled together with the reference's cuda/attention.cu and cuda/gpu_ops.cu (unmodified, by
// path) into oracle/_ref/libdadref_gpu.so. It lets the GPU parity tests run the reference's
// fused kernels, its materialized attention sequence and its dropout kernel on the same device
// and inputs as the new kernels, and lets the benchmark time them. No arithmetic lives here:
// each function is the reference's call sequence (cited) with C++ exceptions turned into codes.
#include <cstdio>
#include <cstring>

#include "gpu_ops.cuh"

namespace {
char g_err[512] = "";
cublasHandle_t g_handle = nullptr;

template <class F>
int guarded(F f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    std::snprintf(g_err, sizeof g_err, "%s", e.what());
    return -1;
  }
}

cublasHandle_t handle() {
  if (!g_handle) CUBLAS_CHECK(cublasCreate(&g_handle));
  return g_handle;
}
}  // namespace

extern "C" {

const char* refgpu_last_error() { return g_err; }

int refgpu_flash_supported(int d_head) { return gpu_flash_attention_supported(d_head) ? 1 : 0; }

// cuda/gpu_ops.cuh:115-117
int refgpu_flash_forward(float* out, float* lse, const float* q, const float* k, const float* v,
                         int BH, int S, int d_head, float scale) {
  return guarded([&] { gpu_flash_attention_forward(out, lse, q, k, v, BH, S, d_head, scale); });
}

// cuda/gpu_ops.cuh:118-122
int refgpu_flash_backward(float* dq, float* dk, float* dv, float* delta, const float* dout,
                          const float* out, const float* lse, const float* q, const float* k,
                          const float* v, int BH, int S, int d_head, float scale) {
  return guarded([&] {
    gpu_flash_attention_backward(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, d_head, scale);
  });
}

// cuda/gpu_ops.cu:707,729-734: mask of `size` elements for dropout seed `seed`
int refgpu_dropout_forward(float* out, const float* in, uint8_t* mask, int size, float rate,
                           unsigned long long seed) {
  return guarded([&] {
    gpu_dropout_init(seed, size);
    gpu_dropout_forward(out, in, mask, size, rate);
  });
}

// Materialized forward, src/model.cpp:396-419. P, dropped: [BH,S,S] scratch kept for backward;
// mask: [BH,S,S] u8. rate = 0 skips dropout (dropped/mask unused).
int refgpu_materialized_forward(float* out, float* P, float* dropped, uint8_t* mask,
                                const float* q, const float* k, const float* v, int BH, int S,
                                int dh, float scale, float rate, unsigned long long seed) {
  return guarded([&] {
    long long sq = static_cast<long long>(S) * dh, ss = static_cast<long long>(S) * S;
    gpu_set_matmul_precision(MatmulPrecision::FP32);
    gpu_matmul_strided_batched_bt(handle(), P, q, k, S, dh, S, sq, sq, ss, BH);
    gpu_scale(P, BH * S * S, scale);
    gpu_causal_mask(P, BH, S);
    gpu_softmax(P, P, BH * S, S);
    const float* probs = P;
    if (rate > 0.0f) {
      gpu_dropout_init(seed, BH * S * S);
      gpu_dropout_forward(dropped, P, mask, BH * S * S, rate);
      probs = dropped;
    }
    gpu_matmul_strided_batched(handle(), out, probs, v, S, S, dh, ss, sq, sq, BH);
  });
}

// Materialized backward, src/model.cpp:576-615. dq/dk/dv are zeroed first because the
// reference accumulates dK/dV into gradient buffers that model_backward cleared earlier.
int refgpu_materialized_backward(float* dq, float* dk, float* dv, float* dP, float* dS,
                                 const float* dout, const float* P, const float* dropped,
                                 const uint8_t* mask, const float* q, const float* k,
                                 const float* v, int BH, int S, int dh, float scale, float rate) {
  return guarded([&] {
    long long sq = static_cast<long long>(S) * dh, ss = static_cast<long long>(S) * S;
    size_t n = static_cast<size_t>(BH) * S * dh, scores = static_cast<size_t>(BH) * S * S;
    gpu_set_matmul_precision(MatmulPrecision::FP32);
    gpu_zero(dq, n);
    gpu_zero(dk, n);
    gpu_zero(dv, n);
    const float* probs = rate > 0.0f ? dropped : P;
    gpu_matmul_strided_batched_bt(handle(), dP, dout, v, S, dh, S, sq, sq, ss, BH);
    gpu_matmul_strided_batched_at(handle(), dv, probs, dout, S, S, dh, ss, sq, sq, BH);
    if (rate > 0.0f) gpu_dropout_backward(dP, mask, static_cast<int>(scores), rate);
    gpu_zero(dS, scores);
    gpu_softmax_backward(dS, dP, P, BH * S, S);
    gpu_causal_mask_zero(dS, BH, S);
    gpu_scale(dS, static_cast<int>(scores), scale);
    gpu_matmul_strided_batched(handle(), dq, dS, k, S, S, dh, ss, sq, sq, BH);
    gpu_matmul_strided_batched_at(handle(), dk, dS, q, S, S, dh, ss, sq, sq, BH);
  });
}

// Decode attention of model_forward_cached, src/model.cpp:745-790: append k,v at pos, per-head
// M=1 products, one softmax over H rows. Caches [H,max_len,dh]; scores scratch [H*(pos+1)].
int refgpu_decode_attention(float* out, float* scores, const float* q, const float* k_new,
                            const float* v_new, float* k_cache, float* v_cache, int H,
                            int max_len, int dh, int pos, float scale) {
  return guarded([&] {
    gpu_set_matmul_precision(MatmulPrecision::FP32);
    for (int head = 0; head < H; ++head) {
      size_t at = static_cast<size_t>(head) * max_len * dh + static_cast<size_t>(pos) * dh;
      CUDA_CHECK(cudaMemcpy(k_cache + at, k_new + head * dh, dh * sizeof(float),
                            cudaMemcpyDeviceToDevice));
      CUDA_CHECK(cudaMemcpy(v_cache + at, v_new + head * dh, dh * sizeof(float),
                            cudaMemcpyDeviceToDevice));
    }
    int cache_len = pos + 1;
    for (int head = 0; head < H; ++head) {
      float* s_h = scores + head * cache_len;
      gpu_matmul_transposed_b(handle(), s_h, q + head * dh,
                              k_cache + static_cast<size_t>(head) * max_len * dh, 1, dh,
                              cache_len);
      gpu_scale(s_h, cache_len, scale);
    }
    gpu_softmax(scores, scores, H, cache_len);
    for (int head = 0; head < H; ++head)
      gpu_matmul(handle(), out + head * dh, scores + head * cache_len,
                 v_cache + static_cast<size_t>(head) * max_len * dh, 1, cache_len, dh);
  });
}

}  // extern "C"
