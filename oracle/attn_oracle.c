/*
 * TEST INFRASTRUCTURE — CPU oracle for DadGPT's causal-attention path.
 *
 * This file restates, in plain C and fp32, what the reference computes for causal attention.
 * It exists only to check the CUDA kernels (tests, the smoke check, and the CPU-baseline leg of
 * the benchmark). Nothing in the shipped library links or calls it.
 *
 * The reference has no host attention function; its attention is a fixed sequence of primitive
 * ops (materialized branch of src/model.cpp). Each step below cites the reference code it
 * follows, including the order of the fp32 additions, so results agree with the reference's
 * own host functions bit for bit (checked by tests/test_oracle.py when the reference
 * sources are available, and by the committed fixtures under tests/golden/ otherwise).
 *
 * Parity pin: the restatement is pinned against the reference's host functions
 * (src/tensor_ops.cpp, src/backward.cpp) compiled from the reference tree, and against the
 * known-answer vectors in the reference's tests/test_tensor_ops.cpp. The Philox dropout mask has
 * no golden vector in the reference; it is pinned on a GPU against the reference's own
 * dropout_forward_kernel (cuda/gpu_ops.cu:712-727).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------------------------
 * Primitive ops, same loop nests and summation order as the reference host ops.
 * ---------------------------------------------------------------------------------------- */

/* out[M,N] = a[M,K] * b[N,K]^T ; follows src/tensor_ops.cpp:111-123 (k innermost, fp32 sum) */
static void mm_bt(float* out, const float* a, const float* b, int M, int K, int N) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float sum = 0.0f;
      for (int k = 0; k < K; ++k) sum += a[i * K + k] * b[j * K + k];
      out[i * N + j] = sum;
    }
}

/* out[M,N] = a[M,K] * b[K,N] ; follows src/tensor_ops.cpp:6-16 */
static void mm(float* out, const float* a, const float* b, int M, int K, int N) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float sum = 0.0f;
      for (int k = 0; k < K; ++k) sum += a[i * K + k] * b[k * N + j];
      out[i * N + j] = sum;
    }
}

/* out[M,N] = a[K,M]^T * b[K,N] ; follows src/tensor_ops.cpp:18-30 */
static void mm_at(float* out, const float* a, const float* b, int M, int K, int N) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float sum = 0.0f;
      for (int k = 0; k < K; ++k) sum += a[k * M + i] * b[k * N + j];
      out[i * N + j] = sum;
    }
}

/* Row softmax, follows src/tensor_ops.cpp:32-55. Also reports max + log(sum) per row, which is
 * the value the fused kernel saves as lse (cuda/attention.cu:71). */
static void softmax_rows(float* out, const float* in, float* lse, int rows, int cols) {
  for (int r = 0; r < rows; ++r) {
    const float* x = in + (size_t)r * cols;
    float* y = out + (size_t)r * cols;
    float mx = x[0];
    for (int c = 1; c < cols; ++c)
      if (x[c] > mx) mx = x[c];
    float sum = 0.0f;
    for (int c = 0; c < cols; ++c) {
      y[c] = expf(x[c] - mx);
      sum += y[c];
    }
    for (int c = 0; c < cols; ++c) y[c] /= sum;
    if (lse) lse[r] = mx + logf(sum);
  }
}

/* din += out * (dout - sum(dout*out)) per row; follows src/backward.cpp:33-50 */
static void softmax_rows_backward(const float* dout, const float* out, float* din, int rows,
                                  int cols) {
  for (int r = 0; r < rows; ++r) {
    const float* g = dout + (size_t)r * cols;
    const float* y = out + (size_t)r * cols;
    float* d = din + (size_t)r * cols;
    float dot = 0.0f;
    for (int c = 0; c < cols; ++c) dot += g[c] * y[c];
    for (int c = 0; c < cols; ++c) d[c] += y[c] * (g[c] - dot);
  }
}

/* ------------------------------------------------------------------------------------------
 * Philox4x32-10 (Salmon et al., SC'11) with the counter/key set-up of cuRAND's
 * curand_init(seed, subsequence, offset) for curandStatePhilox4_32_10_t (CUDA 12.9 headers
 * curand_kernel.h / curand_philox4x32_x.h — a toolkit dependency, not part of the reference):
 *   key = (seed lo, seed hi); counter = 128-bit { offset/4 , subsequence } (low 64, high 64);
 *   the draw is word (offset mod 4) of the 10-round output;
 *   uniform = word * 2^-32 + 2^-33 in fp32.
 * The reference draws exactly one uniform per element, subsequence = flat element index,
 * offset 0, and drops the element iff uniform < rate (cuda/gpu_ops.cu:712-727).
 * ---------------------------------------------------------------------------------------- */
static inline void philox_round(uint32_t c[4], uint32_t k0, uint32_t k1) {
  uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
  uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
  uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
  uint32_t n1 = (uint32_t)p1;
  uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
  uint32_t n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void oracle_philox4x32_10(uint32_t out[4], uint64_t seed, uint64_t subsequence,
                          uint64_t block_index) {
  uint32_t c[4] = {(uint32_t)block_index, (uint32_t)(block_index >> 32), (uint32_t)subsequence,
                   (uint32_t)(subsequence >> 32)};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  memcpy(out, c, sizeof(uint32_t) * 4);
}

float oracle_philox_uniform(uint64_t seed, uint64_t subsequence, uint64_t offset) {
  uint32_t w[4];
  oracle_philox4x32_10(w, seed, subsequence, offset >> 2);
  return fmaf((float)w[offset & 3], 2.3283064e-10f, 2.3283064e-10f / 2.0f);
}

/* mask[i] = 0 (dropped) / 1 (kept) for flat elements first..first+n-1 */
void oracle_dropout_mask(uint8_t* mask, int64_t n, float rate, uint64_t seed, uint64_t offset,
                         int64_t first) {
  for (int64_t i = 0; i < n; ++i)
    mask[i] = oracle_philox_uniform(seed, (uint64_t)(first + i), offset) < rate ? 0 : 1;
}

/* ------------------------------------------------------------------------------------------
 * Causal attention for ONE (batch, head) unit. q,k,v,out: [S,D]; lse: [S] or NULL.
 * Sequence of src/model.cpp:396-419:
 *   scores = q k^T            (gpu_matmul_strided_batched_bt  -> host matmul_transposed_b)
 *   scores *= scale           (cuda/gpu_ops.cu:514-518)
 *   scores[i][j>i] = -1e9     (cuda/gpu_ops.cu:477-485)
 *   P = softmax(scores)       (src/tensor_ops.cpp:32-55)
 *   Pd = mask ? P/(1-rate) : 0   when rate > 0 (cuda/gpu_ops.cu:712-727)
 *   out = Pd v                (src/tensor_ops.cpp:6-16)
 * P (and Pd, mask when rate > 0) stay in the caller's scratch for the backward pass.
 * unit = index of this (b,h) in the whole [BH] batch: it fixes the dropout element index
 * (unit*S + r)*S + c.
 * ---------------------------------------------------------------------------------------- */
static void unit_forward(float* out, float* lse, float* P, float* Pd, uint8_t* mask,
                         const float* q, const float* k, const float* v, int S, int D,
                         float scale, float rate, uint64_t seed, uint64_t offset, int64_t unit) {
  mm_bt(P, q, k, S, D, S);
  for (int64_t i = 0; i < (int64_t)S * S; ++i) P[i] *= scale;
  for (int i = 0; i < S; ++i)
    for (int j = i + 1; j < S; ++j) P[(size_t)i * S + j] = -1e9f;
  softmax_rows(P, P, lse, S, S);
  const float* probs = P;
  if (rate > 0.0f) {
    float keep = 1.0f / (1.0f - rate);
    oracle_dropout_mask(mask, (int64_t)S * S, rate, seed, offset, unit * (int64_t)S * S);
    for (int64_t i = 0; i < (int64_t)S * S; ++i) Pd[i] = mask[i] ? P[i] * keep : 0.0f;
    probs = Pd;
  }
  mm(out, probs, v, S, S, D);
}

/* Backward for one unit, sequence of src/model.cpp:576-615:
 *   dPd = dO v^T ; dV = Pd^T dO ; dP = mask*keep*dPd ; dS = softmax_backward(dP, P) into zeros ;
 *   dS[j>i] = 0 ; dS *= scale ; dQ = dS k ; dK = dS^T q.
 * (The reference accumulates dV/dK into zeroed buffers; writing is the same thing.) */
static void unit_backward(float* dq, float* dk, float* dv, const float* dout, const float* P,
                          const float* Pd, const uint8_t* mask, float* dP, float* dS,
                          const float* q, const float* k, const float* v, int S, int D,
                          float scale, float rate) {
  mm_bt(dP, dout, v, S, D, S);
  mm_at(dv, rate > 0.0f ? Pd : P, dout, S, S, D);
  if (rate > 0.0f) {
    float keep = 1.0f / (1.0f - rate);
    for (int64_t i = 0; i < (int64_t)S * S; ++i) dP[i] *= mask[i] * keep;
  }
  memset(dS, 0, sizeof(float) * (size_t)S * S);
  softmax_rows_backward(dP, P, dS, S, S);
  for (int i = 0; i < S; ++i)
    for (int j = i + 1; j < S; ++j) dS[(size_t)i * S + j] = 0.0f;
  for (int64_t i = 0; i < (int64_t)S * S; ++i) dS[i] *= scale;
  mm(dq, dS, k, S, S, D);
  mm_at(dk, dS, q, S, S, D);
}

/* ------------------------------------------------------------------------------------------
 * Batch drivers: independent (b,h) units fanned out over pthreads (the reference's host ops
 * are single-threaded; units never interact, so threading does not change any result).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
  float *out, *lse, *dq, *dk, *dv;
  const float *dout, *q, *k, *v;
  int BH, S, D, threads, tid, backward;
  int64_t unit0;
  float scale, rate;
  uint64_t seed, offset;
  int status;
} job_t;

static void* worker(void* arg) {
  job_t* j = (job_t*)arg;
  size_t ss = (size_t)j->S * j->S, sd = (size_t)j->S * j->D;
  int drop = j->rate > 0.0f;
  float* P = (float*)malloc(sizeof(float) * ss);
  float* Pd = drop ? (float*)malloc(sizeof(float) * ss) : NULL;
  uint8_t* mask = drop ? (uint8_t*)malloc(ss) : NULL;
  float* dP = j->backward ? (float*)malloc(sizeof(float) * ss) : NULL;
  float* dS = j->backward ? (float*)malloc(sizeof(float) * ss) : NULL;
  float* tmp_out = (float*)malloc(sizeof(float) * sd);
  if (!P || !tmp_out || (drop && (!Pd || !mask)) || (j->backward && (!dP || !dS))) {
    j->status = -1;
  } else {
    for (int u = j->tid; u < j->BH; u += j->threads) {
      const float* q = j->q + u * sd;
      const float* k = j->k + u * sd;
      const float* v = j->v + u * sd;
      float* out = j->out ? j->out + u * sd : tmp_out;
      float* lse = j->lse ? j->lse + (size_t)u * j->S : NULL;
      unit_forward(out, lse, P, Pd, mask, q, k, v, j->S, j->D, j->scale, j->rate, j->seed,
                   j->offset, j->unit0 + u);
      if (j->backward)
        unit_backward(j->dq + u * sd, j->dk + u * sd, j->dv + u * sd, j->dout + u * sd, P, Pd,
                      mask, dP, dS, q, k, v, j->S, j->D, j->scale, j->rate);
    }
  }
  free(P); free(Pd); free(mask); free(dP); free(dS); free(tmp_out);
  return NULL;
}

static int run_jobs(job_t proto, int threads) {
  if (threads < 1) threads = 1;
  if (threads > proto.BH) threads = proto.BH > 0 ? proto.BH : 1;
  if (threads > 256) threads = 256;
  job_t jobs[256];
  pthread_t th[256];
  for (int t = 0; t < threads; ++t) {
    jobs[t] = proto;
    jobs[t].threads = threads;
    jobs[t].tid = t;
    jobs[t].status = 0;
  }
  if (threads == 1) {
    worker(&jobs[0]);
    return jobs[0].status;
  }
  for (int t = 0; t < threads; ++t) pthread_create(&th[t], NULL, worker, &jobs[t]);
  int status = 0;
  for (int t = 0; t < threads; ++t) {
    pthread_join(th[t], NULL);
    if (jobs[t].status) status = jobs[t].status;
  }
  return status;
}

/* q,k,v,out: [BH,S,D] fp32; lse: [BH,S] or NULL. rate = 0 disables dropout.
 * unit0 = global index of the first (b,h) unit (for sharded runs: dropout indices are global). */
int oracle_attention_forward(float* out, float* lse, const float* q, const float* k,
                             const float* v, int BH, int S, int D, float scale, float rate,
                             uint64_t seed, uint64_t offset, int64_t unit0, int threads) {
  job_t p;
  memset(&p, 0, sizeof p);
  p.out = out; p.lse = lse; p.q = q; p.k = k; p.v = v;
  p.BH = BH; p.S = S; p.D = D; p.scale = scale; p.rate = rate;
  p.seed = seed; p.offset = offset; p.unit0 = unit0; p.backward = 0;
  return run_jobs(p, threads);
}

/* Writes dq,dk,dv [BH,S,D]; out/lse optional (NULL to skip). */
int oracle_attention_backward(float* dq, float* dk, float* dv, float* out, float* lse,
                              const float* dout, const float* q, const float* k, const float* v,
                              int BH, int S, int D, float scale, float rate, uint64_t seed,
                              uint64_t offset, int64_t unit0, int threads) {
  job_t p;
  memset(&p, 0, sizeof p);
  p.out = out; p.lse = lse; p.dq = dq; p.dk = dk; p.dv = dv; p.dout = dout;
  p.q = q; p.k = k; p.v = v;
  p.BH = BH; p.S = S; p.D = D; p.scale = scale; p.rate = rate;
  p.seed = seed; p.offset = offset; p.unit0 = unit0; p.backward = 1;
  return run_jobs(p, threads);
}

/* ------------------------------------------------------------------------------------------
 * KV-cache decode attention for one sequence and one new token, after the token's k,v have
 * been appended at position len-1. Follows src/model.cpp:758-790 with M = 1:
 *   scores_h = q_h K_h[0..len)^T (matmul_transposed_b) ; *= scale ; softmax over len ;
 *   out_h = scores_h V_h[0..len) (matmul).
 * q,out: [H,D]; k_cache,v_cache: [H,max_len,D] (the reference's KVCache layout,
 * src/model.hpp:140-152). scores: scratch [len].
 * ---------------------------------------------------------------------------------------- */
void oracle_decode_attention(float* out, const float* q, const float* k_cache,
                             const float* v_cache, int H, int max_len, int D, int len,
                             float scale) {
  float* s = (float*)malloc(sizeof(float) * (size_t)len);
  for (int h = 0; h < H; ++h) {
    const float* kc = k_cache + (size_t)h * max_len * D;
    const float* vc = v_cache + (size_t)h * max_len * D;
    mm_bt(s, q + h * D, kc, 1, D, len);
    for (int i = 0; i < len; ++i) s[i] *= scale;
    softmax_rows(s, s, NULL, 1, len);
    mm(out + h * D, s, vc, 1, len, D);
  }
  free(s);
}

/* Batched form used by the multi-sequence decode tests: caches [B,H,max_len,D], lens[B]. */
typedef struct {
  float* out; const float *q, *kc, *vc; const int* lens;
  int B, H, max_len, D, threads, tid; float scale;
} djob_t;

static void* dworker(void* arg) {
  djob_t* j = (djob_t*)arg;
  size_t per = (size_t)j->H * j->max_len * j->D;
  for (int b = j->tid; b < j->B; b += j->threads)
    oracle_decode_attention(j->out + (size_t)b * j->H * j->D, j->q + (size_t)b * j->H * j->D,
                            j->kc + b * per, j->vc + b * per, j->H, j->max_len, j->D,
                            j->lens[b], j->scale);
  return NULL;
}

void oracle_decode_attention_batched(float* out, const float* q, const float* k_cache,
                                     const float* v_cache, const int* lens, int B, int H,
                                     int max_len, int D, float scale, int threads) {
  if (threads < 1) threads = 1;
  if (threads > B) threads = B;
  if (threads > 256) threads = 256;
  djob_t jobs[256];
  pthread_t th[256];
  for (int t = 0; t < threads; ++t) {
    djob_t j = {out, q, k_cache, v_cache, lens, B, H, max_len, D, threads, t, scale};
    jobs[t] = j;
  }
  for (int t = 0; t < threads; ++t) pthread_create(&th[t], NULL, dworker, &jobs[t]);
  for (int t = 0; t < threads; ++t) pthread_join(th[t], NULL);
}

/* Known-answer hook: exposes the primitive ops so tests can replay the reference's
 * tests/test_tensor_ops.cpp vectors (MatmulBasic etc.) through this file's loops. */
void oracle_matmul(float* out, const float* a, const float* b, int M, int K, int N) {
  mm(out, a, b, M, K, N);
}
void oracle_matmul_transposed_a(float* out, const float* a, const float* b, int M, int K, int N) {
  mm_at(out, a, b, M, K, N);
}
void oracle_matmul_transposed_b(float* out, const float* a, const float* b, int M, int K, int N) {
  mm_bt(out, a, b, M, K, N);
}
void oracle_softmax(float* out, const float* in, int rows, int cols) {
  softmax_rows(out, in, NULL, rows, cols);
}
void oracle_softmax_backward(const float* dout, const float* out, float* din, int rows,
                             int cols) {
  softmax_rows_backward(dout, out, din, rows, cols);
}
