// TEST INFRASTRUCTURE — the reference's model with the call-site edits of
// oracle/patch_reference.py (a patched COPY of src/model.cpp, cuda/gpu_ops.cu and
// cuda/gpu_ops.cuh under oracle/_ref/patched; everything else compiled unmodified from the
// reference tree), linked against libdadattn_gpuops.so. It checks the two call paths that the
// reference's own three fused-attention signatures cannot reach:
//   1. attention dropout on the fused path (training, dropout 0.1): a forward + backward with
//      AttentionImpl::Fused against the same with AttentionImpl::Materialized, both started from
//      gpu_dropout_init(42). The fused calls take their seeds from the same counter, so every
//      dropout mask of the two runs is identical and the results must agree like the
//      reference's FusedAttentionMatchesMaterialized (tests/test_backward.cpp:432-480): logits
//      1e-4, gradients 1e-4 relative L2. The fused run must not have allocated the
//      [B*H, ctx, ctx] probability buffers (src/model.cpp:201-213).
//   2. model_forward_cached with its attention as one gpu_decode_attention launch: prefill +
//      cached decode against a full forward (tests/test_model.cpp:375-414, 1e-4), and the time
//      per generated token on a GPT-2-124M-shaped model (printed; oracle/ref_model_link_check
//      prints the same figure for the unpatched 61-launches-per-layer code).
//   3. batched generation, which the reference does not have (generate_tokens decodes one
//      sequence, src/generate.cpp:94-139): B prompts are prefilled with the reference's
//      model_forward, their K / V heads go into batched caches with gpu_kv_cache_fill, and every
//      step runs ONE cached forward for all B rows, built here from the reference's own ops with
//      rows = B plus gpu_decode_attention_batched. The greedy tokens must equal those of B
//      separate prefill + model_forward_cached loops; the time per token of both is printed.
// Exit code 0 = all within tolerance; every figure is printed.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <vector>

#include "dadattn.h"
#include "dadattn_gpu_ops.hpp"
#include "gpu_ops.cuh"
#include "model.hpp"

namespace {

ModelConfig make_config(int batch, int d_model, int heads, int ctx, int layers = 2, int vocab = 20) {
  ModelConfig c;
  c.d_model = d_model;
  c.n_layers = layers;
  c.n_heads = heads;
  c.d_ff = 2 * d_model;
  c.ctx_len = ctx;
  c.vocab_size = vocab;
  c.batch_size = batch;
  return c;
}

struct RunResult {
  std::vector<float> logits, grads;
  bool probs_allocated;
};

RunResult train_step_with_dropout(const ModelConfig& config, AttentionImpl impl,
                                  const std::vector<uint16_t>& tokens, const uint16_t* d_targets, int batch,
                                  int seq_len) {
  Model model{};
  model_alloc(model, config);
  model.training = true;
  model.dropout_rate = 0.1f;
  model.attention = impl;
  gpu_dropout_init(42, 0);   // both runs draw the same sequence of masks
  model_zero_grad(model);
  gpu_zero(model.activations, model.act_offsets.total);
  gpu_zero(model.grad_activations, model.act_offsets.total);
  model_forward(model, tokens.data(), batch, seq_len);
  gpu_cross_entropy_loss(model.grad_act(model.act_offsets.logits), model.act(model.act_offsets.logits),
                         d_targets, batch * seq_len, config.vocab_size);
  RunResult r;
  r.logits.resize(static_cast<size_t>(batch) * seq_len * config.vocab_size);
  gpu_copy_to_host(r.logits.data(), model.act(model.act_offsets.logits), r.logits.size());
  model_backward(model, tokens.data(), batch, seq_len);
  r.grads.resize(model.param_offsets.total);
  gpu_copy_to_host(r.grads.data(), model.gradients, r.grads.size());
  r.probs_allocated = model.attn_probs != nullptr;
  model_free(model);
  return r;
}

bool fused_dropout_vs_materialized(int d_model, int heads) {
  ModelConfig config = make_config(2, d_model, heads, 80);
  const int batch = 2, seq_len = 70, rows = batch * seq_len;
  std::vector<uint16_t> tokens(rows), targets(rows);
  for (int i = 0; i < rows; ++i) {
    tokens[i] = static_cast<uint16_t>((i * 7 + 3) % config.vocab_size);
    targets[i] = static_cast<uint16_t>((i * 11 + 5) % config.vocab_size);
  }
  uint16_t* d_targets = gpu_alloc_u16(rows);
  gpu_copy_u16_to_device(d_targets, targets.data(), rows);
  RunResult m = train_step_with_dropout(config, AttentionImpl::Materialized, tokens, d_targets, batch, seq_len);
  RunResult f = train_step_with_dropout(config, AttentionImpl::Fused, tokens, d_targets, batch, seq_len);
  gpu_free(d_targets);
  double max_logit = 0.0, diff_sq = 0.0, ref_sq = 0.0;
  for (size_t i = 0; i < m.logits.size(); ++i)
    max_logit = std::max(max_logit, static_cast<double>(std::fabs(f.logits[i] - m.logits[i])));
  for (size_t i = 0; i < m.grads.size(); ++i) {
    diff_sq += static_cast<double>(f.grads[i] - m.grads[i]) * (f.grads[i] - m.grads[i]);
    ref_sq += static_cast<double>(m.grads[i]) * m.grads[i];
  }
  const double rel = std::sqrt(diff_sq / std::max(ref_sq, 1e-20));
  const bool ok = max_logit <= 1e-4 && rel <= 1e-4 && m.probs_allocated && !f.probs_allocated;
  std::printf("fused_dropout_vs_materialized d_head=%d: max|dlogit|=%.3g grad_rel_l2=%.3g "
              "probability buffers: materialized=%d fused=%d %s\n",
              d_model / heads, max_logit, rel, m.probs_allocated ? 1 : 0, f.probs_allocated ? 1 : 0,
              ok ? "OK" : "FAIL");
  return ok;
}

bool prefill_then_one_launch_decode(int d_model, int heads) {
  ModelConfig config = make_config(1, d_model, heads, 48);
  Model model{};
  model_alloc(model, config);
  model.training = false;
  model.attention = AttentionImpl::Fused;
  const int n = 48, prompt = 33;   // decode up to the last slot of the context
  std::vector<uint16_t> tokens(n);
  for (int i = 0; i < n; ++i) tokens[i] = static_cast<uint16_t>((i * 5 + 1) % config.vocab_size);
  model_forward(model, tokens.data(), 1, n);
  std::vector<float> full(static_cast<size_t>(n) * config.vocab_size);
  gpu_copy_to_host(full.data(), model.act(model.act_offsets.logits), full.size());
  KVCache cache;
  kv_cache_alloc(cache, config);
  model_prefill(model, cache, tokens.data(), prompt);
  std::vector<float> row(config.vocab_size);
  double worst = 0.0;
  auto compare = [&](int pos) {
    gpu_copy_to_host(row.data(), model.act(model.act_offsets.logits), row.size());
    for (int v = 0; v < config.vocab_size; ++v)
      worst = std::max(worst, static_cast<double>(
                                  std::fabs(row[v] - full[static_cast<size_t>(pos) * config.vocab_size + v])));
  };
  compare(prompt - 1);
  for (int pos = prompt; pos < n; ++pos) {
    model_forward_cached(model, cache, tokens[pos], pos);
    compare(pos);
  }
  bool threw = false;
  try {
    model_forward_cached(model, cache, tokens[0], n);   // one past the context: must still throw
  } catch (const std::out_of_range&) {
    threw = true;
  }
  kv_cache_free(cache);
  model_free(model);
  const bool ok = worst <= 1e-4 && threw;
  std::printf("prefill_then_one_launch_decode d_head=%d: max|dlogit|=%.3g out_of_range=%d %s\n",
              d_model / heads, worst, threw ? 1 : 0, ok ? "OK" : "FAIL");
  return ok;
}

// ms per decoded token on a GPT-2-124M-shaped model (12 layers, 12 heads of 64, context 1024)
double decode_ms_per_token() {
  ModelConfig config = make_config(1, 768, 12, 1024, 12, 512);
  config.d_ff = 3072;
  Model model{};
  model_alloc(model, config);
  model.training = false;
  KVCache cache;
  kv_cache_alloc(cache, config);
  const int prompt = 512, steps = 64;
  std::vector<uint16_t> tokens(prompt);
  for (int i = 0; i < prompt; ++i) tokens[i] = static_cast<uint16_t>((i * 31 + 7) % config.vocab_size);
  model_prefill(model, cache, tokens.data(), prompt);
  for (int i = 0; i < 4; ++i) model_forward_cached(model, cache, tokens[i], prompt + i);
  cudaDeviceSynchronize();
  auto t0 = std::chrono::steady_clock::now();
  for (int i = 0; i < steps; ++i) model_forward_cached(model, cache, tokens[i], prompt + 4 + i);
  cudaDeviceSynchronize();
  const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
  kv_cache_free(cache);
  model_free(model);
  return ms / steps;
}


// ---- batched generation -------------------------------------------------------------------------
struct BatchedCache {
  int B = 0, max_len = 0;
  std::vector<float*> k, v;      // per layer [B, H, max_len, dh]
  std::vector<int*> lengths;     // per layer [B] (every layer's decode call advances its own)
  std::vector<void*> ws;         // per layer split-K workspace
  size_t ws_bytes = 0;
};

void batched_cache_alloc(BatchedCache& bc, const ModelConfig& c, int B) {
  bc.B = B;
  bc.max_len = c.ctx_len;
  const size_t n = static_cast<size_t>(B) * c.n_heads * c.ctx_len * c.d_head();
  bc.ws_bytes = dadattn_decode_workspace_bytes(B, c.n_heads, c.d_head(), c.ctx_len);
  for (int l = 0; l < c.n_layers; ++l) {
    bc.k.push_back(gpu_alloc(n));
    bc.v.push_back(gpu_alloc(n));
    gpu_zero(bc.k.back(), n);
    gpu_zero(bc.v.back(), n);
    int* len = nullptr;
    cudaMalloc(&len, B * sizeof(int));
    cudaMemset(len, 0, B * sizeof(int));
    bc.lengths.push_back(len);
    void* w = nullptr;
    cudaMalloc(&w, bc.ws_bytes);
    cudaMemset(w, 0, bc.ws_bytes);
    bc.ws.push_back(w);
  }
}
void batched_cache_free(BatchedCache& bc) {
  for (auto p : bc.k) gpu_free(p);
  for (auto p : bc.v) gpu_free(p);
  for (auto p : bc.lengths) cudaFree(p);
  for (auto p : bc.ws) cudaFree(p);
}

// prompt of sequence b: the reference's batch-1 forward, then its K / V heads into the batched caches
void prefill_into(Model& model, BatchedCache& bc, int b, const uint16_t* tokens, int n, float* logits_row) {
  const auto& c = model.config;
  model_forward(model, tokens, 1, n);
  for (int l = 0; l < c.n_layers; ++l) {
    const auto& la = model.act_offsets.layers[l];
    gpu_kv_cache_fill(bc.k[l], bc.v[l], bc.lengths[l], model.act(la.k_heads), model.act(la.v_heads), b, bc.B,
                      c.n_heads, n, bc.max_len, c.d_head());
  }
  cudaMemcpy(logits_row, model.act(model.act_offsets.logits) + static_cast<size_t>(n - 1) * c.vocab_size,
             c.vocab_size * sizeof(float), cudaMemcpyDeviceToDevice);
}

// One decode step for all B sequences: the operations of model_forward_cached (src/model.cpp:687-825)
// with B rows instead of one. `buf` is scratch of B * (12 d + 2 d_ff) floats; logits [B, vocab].
void forward_cached_batched(Model& model, BatchedCache& bc, const uint16_t* tokens, const int* pos, float* buf,
                            float* logits) {
  const auto& c = model.config;
  const auto& po = model.param_offsets;
  auto h = model.cublas_handle;
  const int d = c.d_model, dh = c.d_head(), B = bc.B;
  gpu_copy_u16_to_device(model.d_tokens, tokens, B);
  float* emb = buf;
  float* ln_out = emb + B * d;
  float* q_buf = ln_out + B * d;
  float* k_buf = q_buf + B * d;
  float* v_buf = k_buf + B * d;
  float* attn_out_buf = v_buf + B * d;
  float* proj_buf = attn_out_buf + B * d;
  float* res1_buf = proj_buf + B * d;
  float* ln2_buf = res1_buf + B * d;
  float* fc1_buf = ln2_buf + B * d;
  float* gelu_buf = fc1_buf + B * c.d_ff;
  float* fc2_buf = gelu_buf + B * c.d_ff;
  float* res2_buf = fc2_buf + B * d;
  float* lnf_buf = res2_buf + B * d;
  gpu_embedding_lookup(emb, model.d_tokens, model.param(po.tok_emb), B, d);
  for (int b = 0; b < B; ++b) gpu_add_vectors(emb + b * d, emb + b * d, model.param(po.pos_emb) + pos[b] * d, d);
  float* residual = emb;
  const float scale = 1.0f / std::sqrt(static_cast<float>(dh));
  for (int l = 0; l < c.n_layers; ++l) {
    const auto& lp = po.layers[l];
    gpu_layernorm(ln_out, residual, model.param(lp.ln1_w), model.param(lp.ln1_b), B, d);
    gpu_matmul(h, q_buf, ln_out, model.param(lp.Wq), B, d, d);
    gpu_matmul(h, k_buf, ln_out, model.param(lp.Wk), B, d, d);
    gpu_matmul(h, v_buf, ln_out, model.param(lp.Wv), B, d, d);
    gpu_add_bias(q_buf, model.param(lp.bq), B, d);
    gpu_add_bias(k_buf, model.param(lp.bk), B, d);
    gpu_add_bias(v_buf, model.param(lp.bv), B, d);
    gpu_decode_attention_batched(attn_out_buf, q_buf, k_buf, v_buf, bc.k[l], bc.v[l], bc.lengths[l], B, c.n_heads,
                                 bc.max_len, dh, scale, bc.ws[l], bc.ws_bytes);
    gpu_matmul(h, proj_buf, attn_out_buf, model.param(lp.Wo), B, d, d);
    gpu_add_bias(proj_buf, model.param(lp.bo), B, d);
    gpu_add_vectors(res1_buf, residual, proj_buf, B * d);
    gpu_layernorm(ln2_buf, res1_buf, model.param(lp.ln2_w), model.param(lp.ln2_b), B, d);
    gpu_matmul(h, fc1_buf, ln2_buf, model.param(lp.fc1_w), B, d, c.d_ff);
    gpu_add_bias(fc1_buf, model.param(lp.fc1_b), B, c.d_ff);
    gpu_gelu(gelu_buf, fc1_buf, B * c.d_ff);
    gpu_matmul(h, fc2_buf, gelu_buf, model.param(lp.fc2_w), B, c.d_ff, d);
    gpu_add_bias(fc2_buf, model.param(lp.fc2_b), B, d);
    gpu_add_vectors(res2_buf, res1_buf, fc2_buf, B * d);
    residual = res2_buf;
  }
  gpu_layernorm(lnf_buf, residual, model.param(po.lnf_w), model.param(po.lnf_b), B, d);
  gpu_matmul_transposed_b(h, logits, lnf_buf, model.param(po.tok_emb), B, d, c.vocab_size);
}

int argmax(const float* x, int n) { return static_cast<int>(std::max_element(x, x + n) - x); }

bool batched_generation_matches_single(double* ms_batched, double* ms_single, bool big) {
  ModelConfig config = big ? make_config(1, 768, 12, 1024, 12, 512) : make_config(1, 128, 2, 64);
  if (big) config.d_ff = 3072;
  const int B = big ? 8 : 4, steps = big ? 32 : 12;
  std::vector<int> plen = big ? std::vector<int>{300, 512, 40, 700, 128, 64, 900, 257} : std::vector<int>{5, 9, 17, 30};
  Model model{};
  model_alloc(model, config);
  model.training = false;
  std::vector<std::vector<uint16_t>> prompts(B);
  for (int b = 0; b < B; ++b)
    for (int i = 0; i < plen[b]; ++i)
      prompts[b].push_back(static_cast<uint16_t>((i * (7 + 2 * b) + 3 * b + 1) % config.vocab_size));

  // (a) one sequence at a time: the reference's prefill + cached loop, greedy
  std::vector<std::vector<int>> single(B);
  std::vector<float> row(config.vocab_size);
  auto t0 = std::chrono::steady_clock::now();
  for (int b = 0; b < B; ++b) {
    KVCache cache;
    kv_cache_alloc(cache, config);
    model_prefill(model, cache, prompts[b].data(), plen[b]);
    int pos = plen[b];
    for (int s = 0; s < steps; ++s) {
      gpu_copy_to_host(row.data(), model.act(model.act_offsets.logits), row.size());
      const int tok = argmax(row.data(), config.vocab_size);
      single[b].push_back(tok);
      if (s + 1 < steps) model_forward_cached(model, cache, static_cast<uint16_t>(tok), pos++);
    }
    kv_cache_free(cache);
  }
  cudaDeviceSynchronize();
  *ms_single = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() /
               (static_cast<double>(B) * steps);

  // (b) all B together
  BatchedCache bc;
  batched_cache_alloc(bc, config, B);
  float* buf = gpu_alloc(static_cast<size_t>(B) * (12 * config.d_model + 2 * config.d_ff));
  float* logits = gpu_alloc(static_cast<size_t>(B) * config.vocab_size);
  std::vector<std::vector<int>> batched(B);
  std::vector<float> all(static_cast<size_t>(B) * config.vocab_size);
  std::vector<uint16_t> toks(B);
  std::vector<int> pos(B);
  t0 = std::chrono::steady_clock::now();
  for (int b = 0; b < B; ++b) {
    prefill_into(model, bc, b, prompts[b].data(), plen[b], logits + static_cast<size_t>(b) * config.vocab_size);
    pos[b] = plen[b];
  }
  for (int s = 0; s < steps; ++s) {
    gpu_copy_to_host(all.data(), logits, all.size());
    for (int b = 0; b < B; ++b) {
      toks[b] = static_cast<uint16_t>(argmax(all.data() + static_cast<size_t>(b) * config.vocab_size, config.vocab_size));
      batched[b].push_back(toks[b]);
    }
    if (s + 1 < steps) {
      forward_cached_batched(model, bc, toks.data(), pos.data(), buf, logits);
      for (int b = 0; b < B; ++b) ++pos[b];
    }
  }
  cudaDeviceSynchronize();
  *ms_batched = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() /
                (static_cast<double>(B) * steps);
  gpu_free(buf);
  gpu_free(logits);
  batched_cache_free(bc);
  model_free(model);
  int same = 0;
  for (int b = 0; b < B; ++b) same += (single[b] == batched[b]) ? 1 : 0;
  return same == B;
}

}  // namespace

int main() {
  bool ok = true;
  try {
    ok &= fused_dropout_vs_materialized(128, 2);  // d_head 64
    ok &= fused_dropout_vs_materialized(64, 2);   // d_head 32
    ok &= prefill_then_one_launch_decode(128, 2);
    ok &= prefill_then_one_launch_decode(64, 2);
    std::printf("cached_decode gpt2-124m shape, one attention launch per layer: %.3f ms/token\n",
                decode_ms_per_token());
    double msb = 0, mss = 0;
    const bool same = batched_generation_matches_single(&msb, &mss, false);
    std::printf("batched_generation 4 sequences x 12 greedy tokens vs one at a time: %s\n", same ? "OK" : "FAIL");
    ok &= same;
    const bool same_big = batched_generation_matches_single(&msb, &mss, true);
    std::printf("batched_generation gpt2-124m shape, 8 sequences x 32 tokens (prefill included): %.3f ms/token "
                "batched, %.3f ms/token one at a time, tokens %s\n", msb, mss, same_big ? "equal" : "differ");
  } catch (const std::exception& e) {
    std::printf("exception: %s\n", e.what());
    return 2;
  }
  std::printf("%s\n", ok ? "ALL OK" : "FAILED");
  return ok ? 0 : 1;
}
