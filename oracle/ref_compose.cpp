// TEST INFRASTRUCTURE — glue that drives the REFERENCE's own host ops as an attention pipeline.
//
// This file holds no arithmetic of its own beyond the two trivial loops the reference runs as
// GPU kernels (scale, cuda/gpu_ops.cu:514-518; causal mask, cuda/gpu_ops.cu:477-485 and
// :495-503). Everything else is a call into the reference's src/tensor_ops.cpp and
// src/backward.cpp, which the Makefile compiles from the reference tree where it lies. The
// resulting library (oracle/_ref/libdadref_host.so) is used to pin oracle/attn_oracle.c and,
// when present, as the "reference" CPU baseline of the benchmark.
//
// Call order = the materialized attention branch of the reference model:
// forward src/model.cpp:396-419, backward src/model.cpp:576-615, decode src/model.cpp:758-790.
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "backward.hpp"
#include "tensor_ops.hpp"

namespace {

void scale_inplace(float* x, size_t n, float s) {
  for (size_t i = 0; i < n; ++i) x[i] *= s;
}

void unit_forward(float* out, float* P, float* Pd, const uint8_t* mask, const float* q,
                  const float* k, const float* v, int S, int D, float scale, float rate) {
  size_t ss = static_cast<size_t>(S) * S;
  matmul_transposed_b(P, q, k, S, D, S);
  scale_inplace(P, ss, scale);
  for (int i = 0; i < S; ++i)
    for (int j = i + 1; j < S; ++j) P[static_cast<size_t>(i) * S + j] = -1e9f;
  softmax(P, P, S, S);
  const float* probs = P;
  if (rate > 0.0f) {
    float keep = 1.0f / (1.0f - rate);
    for (size_t i = 0; i < ss; ++i) Pd[i] = mask[i] ? P[i] * keep : 0.0f;
    probs = Pd;
  }
  matmul(out, probs, v, S, S, D);
}

void unit_backward(float* dq, float* dk, float* dv, const float* dout, const float* P,
                   const float* Pd, const uint8_t* mask, float* dP, float* dS, const float* q,
                   const float* k, const float* v, int S, int D, float scale, float rate) {
  size_t ss = static_cast<size_t>(S) * S;
  matmul_transposed_b(dP, dout, v, S, D, S);
  matmul_transposed_a(dv, rate > 0.0f ? Pd : P, dout, S, S, D);
  if (rate > 0.0f) {
    float keep = 1.0f / (1.0f - rate);
    for (size_t i = 0; i < ss; ++i) dP[i] *= mask[i] * keep;
  }
  std::memset(dS, 0, sizeof(float) * ss);
  softmax_backward(dP, P, dS, S, S);
  for (int i = 0; i < S; ++i)
    for (int j = i + 1; j < S; ++j) dS[static_cast<size_t>(i) * S + j] = 0.0f;
  scale_inplace(dS, ss, scale);
  matmul(dq, dS, k, S, S, D);
  matmul_transposed_a(dk, dS, q, S, S, D);
}

template <class F>
void fan_out(int units, int threads, F f) {
  if (threads < 1) threads = 1;
  if (threads > units) threads = units > 0 ? units : 1;
  if (threads == 1) {
    f(0, 1);
    return;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) pool.emplace_back(f, t, threads);
  for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// mask: [BH,S,S] u8 (1 keep / 0 drop) when rate > 0, else ignored. out: [BH,S,D] or null.
int ref_attention_forward(float* out, const float* q, const float* k, const float* v,
                          const uint8_t* mask, int BH, int S, int D, float scale, float rate,
                          int threads) {
  size_t ss = static_cast<size_t>(S) * S, sd = static_cast<size_t>(S) * D;
  fan_out(BH, threads, [&](int tid, int nt) {
    std::vector<float> P(ss), Pd(rate > 0.0f ? ss : 0), tmp(out ? 0 : sd);
    for (int u = tid; u < BH; u += nt)
      unit_forward(out ? out + u * sd : tmp.data(), P.data(), Pd.data(),
                   mask ? mask + u * ss : nullptr, q + u * sd, k + u * sd, v + u * sd, S, D,
                   scale, rate);
  });
  return 0;
}

int ref_attention_backward(float* dq, float* dk, float* dv, const float* dout, const float* q,
                           const float* k, const float* v, const uint8_t* mask, int BH, int S,
                           int D, float scale, float rate, int threads) {
  size_t ss = static_cast<size_t>(S) * S, sd = static_cast<size_t>(S) * D;
  fan_out(BH, threads, [&](int tid, int nt) {
    std::vector<float> P(ss), Pd(rate > 0.0f ? ss : 0), dP(ss), dS(ss), o(sd);
    for (int u = tid; u < BH; u += nt) {
      const uint8_t* m = mask ? mask + u * ss : nullptr;
      unit_forward(o.data(), P.data(), Pd.data(), m, q + u * sd, k + u * sd, v + u * sd, S, D,
                   scale, rate);
      unit_backward(dq + u * sd, dk + u * sd, dv + u * sd, dout + u * sd, P.data(), Pd.data(), m,
                    dP.data(), dS.data(), q + u * sd, k + u * sd, v + u * sd, S, D, scale, rate);
    }
  });
  return 0;
}

// One sequence, reference KVCache layout [H,max_len,D]; len = pos + 1 keys visible.
int ref_decode_attention(float* out, const float* q, const float* k_cache, const float* v_cache,
                         int H, int max_len, int D, int len, float scale) {
  std::vector<float> s(len);
  for (int h = 0; h < H; ++h) {
    const float* kc = k_cache + static_cast<size_t>(h) * max_len * D;
    const float* vc = v_cache + static_cast<size_t>(h) * max_len * D;
    matmul_transposed_b(s.data(), q + h * D, kc, 1, D, len);
    scale_inplace(s.data(), len, scale);
    softmax(s.data(), s.data(), 1, len);
    matmul(out + h * D, s.data(), vc, 1, len, D);
  }
  return 0;
}

// Direct exports of the reference host ops (for known-answer replays).
void ref_matmul(float* o, const float* a, const float* b, int M, int K, int N) {
  matmul(o, a, b, M, K, N);
}
void ref_matmul_transposed_a(float* o, const float* a, const float* b, int M, int K, int N) {
  matmul_transposed_a(o, a, b, M, K, N);
}
void ref_matmul_transposed_b(float* o, const float* a, const float* b, int M, int K, int N) {
  matmul_transposed_b(o, a, b, M, K, N);
}
void ref_softmax(float* o, const float* in, int rows, int cols) { softmax(o, in, rows, cols); }
void ref_softmax_backward(const float* dout, const float* out, float* din, int rows, int cols) {
  softmax_backward(dout, out, din, rows, cols);
}

}  // extern "C"
