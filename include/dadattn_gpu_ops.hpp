/*
 * C++ declarations a DadGPT maintainer adds next to cuda/gpu_ops.cuh to use what the reference's
 * own three fused-attention signatures (cuda/gpu_ops.cuh:115-122) cannot express. All are
 * defined in libdadattn_gpuops.so on top of the C ABI (include/dadattn.h), enqueue on the
 * legacy default stream like the rest of gpu_ops, and throw std::runtime_error on failure
 * (the reference's CUDA_CHECK convention, cuda/gpu_ops.cuh:10-17).
 */
#pragma once

#include <cstddef>

/* Fused causal attention WITH attention-probability dropout: what the reference computes in its
 * materialized branch (src/model.cpp:406-415 forward, :595-602 backward) when
 * use_fused_attention (src/model.cpp:185-197) has to decline because dropout is on. `seed` is
 * the value gpu_dropout_forward (cuda/gpu_ops.cu:729-734) would have consumed for this layer's
 * probabilities: the caller takes it from the same counter (d_dropout_seed, cuda/gpu_ops.cu:704),
 * advances the counter by one, and passes the SAME seed to the backward of that layer. The mask
 * is the reference's, bit for bit (element (bh, r, c) of the [BH,S,S] probabilities is element
 * (bh S + r) S + c of the Philox stream); lse is that of the undropped softmax. rate = 0 is
 * gpu_flash_attention_forward / _backward. */
void gpu_flash_attention_forward_dropout(float* out, float* lse, const float* q, const float* k,
                                         const float* v, int BH, int S, int d_head, float scale,
                                         float rate, unsigned long long seed);
void gpu_flash_attention_backward_dropout(float* dq, float* dk, float* dv, float* delta,
                                          const float* dout, const float* out, const float* lse,
                                          const float* q, const float* k, const float* v, int BH,
                                          int S, int d_head, float scale, float rate,
                                          unsigned long long seed);

/* The attention part of model_forward_cached (src/model.cpp:745-790: 2 H cache-row copies, H
 * score products, H scalings, one softmax, H value products; 61 launches per layer at H = 12) as
 * ONE launch on the reference's own cache layout (struct KVCache, src/model.hpp:140-152): writes
 * k_new, v_new [n_heads * d_head] into row `pos` of k_cache, v_cache [n_heads, max_len, d_head],
 * then out[h] = softmax(q_h K_h[0..pos]^T * scale) V_h[0..pos]. Throws std::out_of_range when pos
 * is outside [0, max_len), as model_forward_cached does (src/model.cpp:693-696). */
void gpu_decode_attention(float* out, const float* q, const float* k_new, const float* v_new,
                          float* k_cache, float* v_cache, int n_heads, int max_len, int d_head,
                          int pos, float scale);

/* The same for `batch` sequences at once: caches [batch, n_heads, max_len, d_head] fp32, device
 * array lengths[batch] (each sequence's current length; advanced by one), q / k_new / v_new / out
 * [batch, n_heads * d_head]. `workspace` as dadattn_decode_workspace_bytes says, zero-filled once.
 * For a generation loop that decodes several sequences per step. */
void gpu_decode_attention_batched(float* out, const float* q, const float* k_new, const float* v_new,
                                  float* k_cache, float* v_cache, int* lengths, int batch, int n_heads,
                                  int max_len, int d_head, float scale, void* workspace,
                                  size_t workspace_bytes);

/* Rows 0..n-1 of sequence b of a batched fp32 cache from the k_heads / v_heads [n_heads, n, d_head]
 * a batch-1 model_forward leaves behind (what model_prefill copies with cudaMemcpy2D,
 * src/model.cpp:835-843); lengths[b] = n. */
void gpu_kv_cache_fill(float* k_cache, float* v_cache, int* lengths, const float* k_heads,
                       const float* v_heads, int b, int batch, int n_heads, int n, int max_len,
                       int d_head);
