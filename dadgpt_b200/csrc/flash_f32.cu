// fp32 fused causal attention, forward and backward: the drop-in for DadGPT's
// gpu_flash_attention_forward / gpu_flash_attention_backward (reference cuda/attention.cu).
//
// Exact fp32 FFMA arithmetic (no tensor cores: the 1e-5 parity bar against the fp32 reference
// rules out tf32/bf16 products). Where the reference gives one thread a whole query row and a
// 32-thread block, these kernels tile 64 queries x 64 keys per 256-thread block with 4x4
// register micro-tiles, so a tile of K/V is read from shared memory once per 64 rows instead of
// once per row. Semantics kept from the reference: lse = rowmax + ln(rowsum) of the scaled
// scores (cuda/attention.cu:71), key c visible to query r iff c <= r (:50), rows >= S never
// written (:68), dq/dk/dv written not accumulated, no atomics (deterministic).
// Optional attention-probability dropout follows the reference's materialized branch
// (src/model.cpp:406-415, 595-602).
#include <cfloat>

#include "common.cuh"

namespace dadattn {
namespace {

constexpr int kTile = 64;      // queries per block and keys per shared-memory tile
constexpr int kThreads = 256;  // 16 x 16 threads
constexpr int kPStride = kTile + 4;

template <int N>
__device__ __forceinline__ void load_vec(float (&dst)[N], const float* src) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      float4 t = *reinterpret_cast<const float4*>(src + i);
      dst[i] = t.x; dst[i + 1] = t.y; dst[i + 2] = t.z; dst[i + 3] = t.w;
    }
  } else if constexpr (N == 2) {
    float2 t = *reinterpret_cast<const float2*>(src);
    dst[0] = t.x; dst[1] = t.y;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) dst[i] = src[i];
  }
}

template <int N>
__device__ __forceinline__ void store_vec(float* dst, const float (&src)[N]) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 4)
      *reinterpret_cast<float4*>(dst + i) = make_float4(src[i], src[i + 1], src[i + 2], src[i + 3]);
  } else if constexpr (N == 2) {
    *reinterpret_cast<float2*>(dst) = make_float2(src[0], src[1]);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) dst[i] = src[i];
  }
}

// Copies rows [row0, row0+64) of a [S, D] matrix into shared memory (row stride D+4), zero
// filling rows >= S. Global reads are float4 when the base pointer allows it.
template <int D>
__device__ __forceinline__ void load_tile(float* dst, const float* __restrict__ src, int row0,
                                          int S, bool vec_ok) {
  constexpr int LD = D + 4;
  if (vec_ok) {
    constexpr int V = D / 4;
    for (int i = threadIdx.x; i < kTile * V; i += kThreads) {
      int r = i / V, c = (i % V) * 4;
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < S) t = *reinterpret_cast<const float4*>(src + static_cast<size_t>(row0 + r) * D + c);
      *reinterpret_cast<float4*>(dst + r * LD + c) = t;
    }
  } else {
    for (int i = threadIdx.x; i < kTile * D; i += kThreads) {
      int r = i / D, c = i % D;
      dst[r * LD + c] = row0 + r < S ? src[static_cast<size_t>(row0 + r) * D + c] : 0.f;
    }
  }
}

// acc[i][j] += sum_d A[(a0 + i) * LD + d] * B[(b0 + 16 j) * LD + d]
// A rows are shared by the 16 threads of a half-warp (broadcast); B rows differ per thread and
// the D+4 stride spreads their float4 reads over all banks.
template <int D>
__device__ __forceinline__ void tile_dot(float (&acc)[4][4], const float* A, int a0,
                                         const float* B, int b0) {
  constexpr int LD = D + 4;
#pragma unroll 4
  for (int d = 0; d < D; d += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = *reinterpret_cast<const float4*>(A + (a0 + i) * LD + d);
#pragma unroll
    for (int j = 0; j < 4; ++j) b[j] = *reinterpret_cast<const float4*>(B + (b0 + 16 * j) * LD + d);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] = fmaf(a[i].x, b[j].x, acc[i][j]);
        acc[i][j] = fmaf(a[i].y, b[j].y, acc[i][j]);
        acc[i][j] = fmaf(a[i].z, b[j].z, acc[i][j]);
        acc[i][j] = fmaf(a[i].w, b[j].w, acc[i][j]);
      }
  }
}

// acc[i][x] += sum_{c<64} W[(w0 + i) * kPStride + c] * M[c * LD + m0 + x]
template <int D, int DC>
__device__ __forceinline__ void tile_axpy(float (&acc)[4][DC], const float* W, int w0,
                                          const float* M, int m0) {
  constexpr int LD = D + 4;
#pragma unroll 2
  for (int c = 0; c < kTile; c += 4) {
    float w[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) load_vec<4>(w[i], W + (w0 + i) * kPStride + c);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      float m[DC];
      load_vec<DC>(m, M + (c + cc) * LD + m0);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int x = 0; x < DC; ++x) acc[i][x] = fmaf(w[i][cc], m[x], acc[i][x]);
    }
  }
}

__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float group16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int D>
constexpr size_t fwd_smem_bytes() {
  return sizeof(float) * (3 * kTile * (D + 4) + kTile * kPStride);
}

// ---------------------------------------------------------------------------------------------
// Forward. grid = (ceil(S/64), BH); heaviest (last) query tiles are scheduled first.
// ---------------------------------------------------------------------------------------------
template <int D, bool DROP>
__global__ void __launch_bounds__(kThreads)
flash_fwd_f32_kernel(float* __restrict__ out, float* __restrict__ lse, const float* __restrict__ q,
                     const float* __restrict__ k, const float* __restrict__ v, int S, float scale,
                     float rate, PhiloxKey rng, int64_t unit0, bool vec_ok) {
  constexpr int LD = D + 4;
  constexpr int DC = D / 16;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* Ks = Qs + kTile * LD;
  float* Vs = Ks + kTile * LD;
  float* Ps = Vs + kTile * LD;

  const int qt = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y;
  const size_t base = static_cast<size_t>(bh) * S * D;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int q0 = qt * kTile;

  load_tile<D>(Qs, q + base, q0, S, vec_ok);

  float m[4], l[4], o[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -FLT_MAX;
    l[i] = 0.f;
#pragma unroll
    for (int x = 0; x < DC; ++x) o[i][x] = 0.f;
  }
  const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;

  for (int kt = 0; kt <= qt; ++kt) {
    const int k0 = kt * kTile;
    __syncthreads();  // previous tile's K/V/P fully consumed
    load_tile<D>(Ks, k + base, k0, S, vec_ok);
    load_tile<D>(Vs, v + base, k0, S, vec_ok);
    __syncthreads();

    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
    tile_dot<D>(s, Qs, ty * 4, Ks, tx);

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = q0 + ty * 4 + i;
      float tmax = -FLT_MAX;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = k0 + tx + 16 * j;
        s[i][j] = c <= r ? s[i][j] * scale : -FLT_MAX;
        tmax = fmaxf(tmax, s[i][j]);
      }
      tmax = group16_max(tmax);
      // Every valid row sees key 0 in tile 0, so m_new is finite from the first tile on.
      const float m_new = fmaxf(m[i], tmax);
      const float corr = expf(m[i] - m_new);
      float psum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = k0 + tx + 16 * j;
        float p = c <= r ? expf(s[i][j] - m_new) : 0.f;
        psum += p;
        if (DROP) {
          const uint64_t idx = (static_cast<uint64_t>(unit0 + bh) * S + r) * S + c;
          p = (c <= r && r < S && philox_keep(rng, idx, rate)) ? p * keep_scale : 0.f;
        }
        Ps[(ty * 4 + i) * kPStride + tx + 16 * j] = p;
      }
      psum = group16_sum(psum);
      l[i] = l[i] * corr + psum;
      m[i] = m_new;
#pragma unroll
      for (int x = 0; x < DC; ++x) o[i][x] *= corr;
    }
    __syncthreads();
    tile_axpy<D, DC>(o, Ps, ty * 4, Vs, tx * DC);
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = q0 + ty * 4 + i;
    if (r >= S) continue;
    const float inv = 1.0f / l[i];
    float res[DC];
#pragma unroll
    for (int x = 0; x < DC; ++x) res[x] = o[i][x] * inv;
    float* dst = out + base + static_cast<size_t>(r) * D + tx * DC;
    if (vec_ok) {
      store_vec<DC>(dst, res);
    } else {
#pragma unroll
      for (int x = 0; x < DC; ++x) dst[x] = res[x];
    }
    if (tx == 0) lse[static_cast<size_t>(bh) * S + r] = m[i] + logf(l[i]);
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, three launches as in the reference (cuda/attention.cu:215-228), tiled the same way
// as the forward.
// ---------------------------------------------------------------------------------------------

// delta[r] = sum_d dout[r,d] * out[r,d]; D/4 lanes per row, float4 each.
template <int D>
__global__ void flash_delta_f32_kernel(float* __restrict__ delta, const float* __restrict__ dout,
                                       const float* __restrict__ out, int64_t rows, bool vec_ok) {
  constexpr int L = D / 4;  // lanes per row: 4, 8, 16, 32
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = t / L;
  const int c = static_cast<int>(t % L) * 4;
  float sum = 0.f;
  if (r < rows) {
    const float* a = dout + r * D + c;
    const float* b = out + r * D + c;
    if (vec_ok) {
      float4 x = *reinterpret_cast<const float4*>(a), y = *reinterpret_cast<const float4*>(b);
      sum = x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
    } else {
      sum = a[0] * b[0] + a[1] * b[1] + a[2] * b[2] + a[3] * b[3];
    }
  }
#pragma unroll
  for (int o = L / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (r < rows && c == 0) delta[r] = sum;
}

template <int D>
constexpr size_t bwd_smem_bytes() {
  return sizeof(float) * (4 * kTile * (D + 4) + 2 * kTile * kPStride + 2 * kTile);
}

// One block per 64 keys: dV_j = sum_{r>=j} Pd_rj dO_r ; dK_j = sum_{r>=j} dS_rj Q_r.
template <int D, bool DROP>
__global__ void __launch_bounds__(kThreads)
flash_bwd_dkdv_f32_kernel(float* __restrict__ dk, float* __restrict__ dv,
                          const float* __restrict__ q, const float* __restrict__ k,
                          const float* __restrict__ v, const float* __restrict__ dout,
                          const float* __restrict__ lse, const float* __restrict__ delta, int S,
                          float scale, float rate, PhiloxKey rng, int64_t unit0, bool vec_ok) {
  constexpr int LD = D + 4;
  constexpr int DC = D / 16;
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem;
  float* Vs = Ks + kTile * LD;
  float* Qs = Vs + kTile * LD;
  float* dOs = Qs + kTile * LD;
  float* Pt = dOs + kTile * LD;        // [key][query], dropped probabilities
  float* dSt = Pt + kTile * kPStride;  // [key][query]
  float* lse_s = dSt + kTile * kPStride;
  float* delta_s = lse_s + kTile;

  const int kt = blockIdx.x;  // low key tiles see the most queries and come first
  const int bh = blockIdx.y;
  const size_t base = static_cast<size_t>(bh) * S * D;
  const size_t row_base = static_cast<size_t>(bh) * S;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int k0 = kt * kTile;
  const int n_qt = (S + kTile - 1) / kTile;
  const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;

  load_tile<D>(Ks, k + base, k0, S, vec_ok);
  load_tile<D>(Vs, v + base, k0, S, vec_ok);

  float dk_acc[4][DC], dv_acc[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int x = 0; x < DC; ++x) dk_acc[i][x] = dv_acc[i][x] = 0.f;

  for (int qt = kt; qt < n_qt; ++qt) {
    const int q0 = qt * kTile;
    __syncthreads();
    load_tile<D>(Qs, q + base, q0, S, vec_ok);
    load_tile<D>(dOs, dout + base, q0, S, vec_ok);
    if (threadIdx.x < kTile) {
      const int r = q0 + threadIdx.x;
      lse_s[threadIdx.x] = r < S ? lse[row_base + r] : 0.f;
      delta_s[threadIdx.x] = r < S ? delta[row_base + r] : 0.f;
    }
    __syncthreads();

    // Here the thread owns keys ty*4+i (broadcast operand) and queries tx+16j.
    float s[4][4], dp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
    tile_dot<D>(s, Ks, ty * 4, Qs, tx);
    tile_dot<D>(dp, Vs, ty * 4, dOs, tx);

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = k0 + ty * 4 + i;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int rl = tx + 16 * j, r = q0 + rl;
        float pd = 0.f, ds = 0.f;
        if (c <= r && r < S) {
          const float p = expf(s[i][j] * scale - lse_s[rl]);
          float g = dp[i][j];
          pd = p;
          if (DROP) {
            const uint64_t idx = (static_cast<uint64_t>(unit0 + bh) * S + r) * S + c;
            const float mk = philox_keep(rng, idx, rate) ? keep_scale : 0.f;
            pd = p * mk;
            g *= mk;
          }
          ds = p * (g - delta_s[rl]) * scale;
        }
        Pt[(ty * 4 + i) * kPStride + rl] = pd;
        dSt[(ty * 4 + i) * kPStride + rl] = ds;
      }
    }
    __syncthreads();
    tile_axpy<D, DC>(dv_acc, Pt, ty * 4, dOs, tx * DC);
    tile_axpy<D, DC>(dk_acc, dSt, ty * 4, Qs, tx * DC);
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = k0 + ty * 4 + i;
    if (c >= S) continue;
    float* pk = dk + base + static_cast<size_t>(c) * D + tx * DC;
    float* pv = dv + base + static_cast<size_t>(c) * D + tx * DC;
    if (vec_ok) {
      store_vec<DC>(pk, dk_acc[i]);
      store_vec<DC>(pv, dv_acc[i]);
    } else {
#pragma unroll
      for (int x = 0; x < DC; ++x) {
        pk[x] = dk_acc[i][x];
        pv[x] = dv_acc[i][x];
      }
    }
  }
}

// One block per 64 queries: dQ_r = sum_{c<=r} dS_rc K_c.
template <int D, bool DROP>
__global__ void __launch_bounds__(kThreads)
flash_bwd_dq_f32_kernel(float* __restrict__ dq, const float* __restrict__ q,
                        const float* __restrict__ k, const float* __restrict__ v,
                        const float* __restrict__ dout, const float* __restrict__ lse,
                        const float* __restrict__ delta, int S, float scale, float rate,
                        PhiloxKey rng, int64_t unit0, bool vec_ok) {
  constexpr int LD = D + 4;
  constexpr int DC = D / 16;
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;
  float* dOs = Qs + kTile * LD;
  float* Ks = dOs + kTile * LD;
  float* Vs = Ks + kTile * LD;
  float* dSs = Vs + kTile * LD;  // [query][key]

  const int qt = gridDim.x - 1 - blockIdx.x;
  const int bh = blockIdx.y;
  const size_t base = static_cast<size_t>(bh) * S * D;
  const size_t row_base = static_cast<size_t>(bh) * S;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  const int q0 = qt * kTile;
  const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;

  load_tile<D>(Qs, q + base, q0, S, vec_ok);
  load_tile<D>(dOs, dout + base, q0, S, vec_ok);
  float row_lse[4], row_delta[4], acc[4][DC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = q0 + ty * 4 + i;
    row_lse[i] = r < S ? lse[row_base + r] : 0.f;
    row_delta[i] = r < S ? delta[row_base + r] : 0.f;
#pragma unroll
    for (int x = 0; x < DC; ++x) acc[i][x] = 0.f;
  }

  for (int kt = 0; kt <= qt; ++kt) {
    const int k0 = kt * kTile;
    __syncthreads();
    load_tile<D>(Ks, k + base, k0, S, vec_ok);
    load_tile<D>(Vs, v + base, k0, S, vec_ok);
    __syncthreads();

    float s[4][4], dp[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.f;
    tile_dot<D>(s, Qs, ty * 4, Ks, tx);
    tile_dot<D>(dp, dOs, ty * 4, Vs, tx);

#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = q0 + ty * 4 + i;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int cl = tx + 16 * j, c = k0 + cl;
        float ds = 0.f;
        if (c <= r && r < S) {
          const float p = expf(s[i][j] * scale - row_lse[i]);
          float g = dp[i][j];
          if (DROP) {
            const uint64_t idx = (static_cast<uint64_t>(unit0 + bh) * S + r) * S + c;
            g *= philox_keep(rng, idx, rate) ? keep_scale : 0.f;
          }
          ds = p * (g - row_delta[i]) * scale;
        }
        dSs[(ty * 4 + i) * kPStride + cl] = ds;
      }
    }
    __syncthreads();
    tile_axpy<D, DC>(acc, dSs, ty * 4, Ks, tx * DC);
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = q0 + ty * 4 + i;
    if (r >= S) continue;
    float* dst = dq + base + static_cast<size_t>(r) * D + tx * DC;
    if (vec_ok) {
      store_vec<DC>(dst, acc[i]);
    } else {
#pragma unroll
      for (int x = 0; x < DC; ++x) dst[x] = acc[i][x];
    }
  }
}

template <int D, bool DROP>
int launch_fwd(float* out, float* lse, const float* q, const float* k, const float* v, int BH,
               int S, float scale, float rate, uint64_t seed, uint64_t offset, int64_t unit0,
               cudaStream_t st) {
  const bool vec_ok = aligned(out, 16) && aligned(q, 16) && aligned(k, 16) && aligned(v, 16);
  auto kern = flash_fwd_f32_kernel<D, DROP>;
  DAD_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(fwd_smem_bytes<D>())));
  dim3 grid((S + kTile - 1) / kTile, BH);
  kern<<<grid, kThreads, fwd_smem_bytes<D>(), st>>>(out, lse, q, k, v, S, scale, rate,
                                                   make_philox(seed, offset), unit0, vec_ok);
  DAD_LAUNCH_CHECK("flash_fwd_f32_kernel");
  return DADATTN_OK;
}

template <int D, bool DROP>
int launch_bwd(float* dq, float* dk, float* dv, float* delta, const float* dout, const float* out,
               const float* lse, const float* q, const float* k, const float* v, int BH, int S,
               float scale, float rate, uint64_t seed, uint64_t offset, int64_t unit0,
               cudaStream_t st) {
  const bool vec_ok = aligned(dq, 16) && aligned(dk, 16) && aligned(dv, 16) &&
                      aligned(dout, 16) && aligned(out, 16) && aligned(q, 16) &&
                      aligned(k, 16) && aligned(v, 16);
  const int64_t rows = static_cast<int64_t>(BH) * S;
  const int64_t delta_threads = rows * (D / 4);
  flash_delta_f32_kernel<D><<<static_cast<unsigned>((delta_threads + 255) / 256), 256, 0, st>>>(
      delta, dout, out, rows, vec_ok);
  DAD_LAUNCH_CHECK("flash_delta_f32_kernel");

  const PhiloxKey rng = make_philox(seed, offset);
  dim3 grid((S + kTile - 1) / kTile, BH);
  auto kkv = flash_bwd_dkdv_f32_kernel<D, DROP>;
  DAD_CUDA(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(bwd_smem_bytes<D>())));
  kkv<<<grid, kThreads, bwd_smem_bytes<D>(), st>>>(dk, dv, q, k, v, dout, lse, delta, S, scale,
                                                  rate, rng, unit0, vec_ok);
  DAD_LAUNCH_CHECK("flash_bwd_dkdv_f32_kernel");

  auto kq = flash_bwd_dq_f32_kernel<D, DROP>;
  constexpr size_t dq_smem = sizeof(float) * (4 * kTile * (D + 4) + kTile * kPStride);
  DAD_CUDA(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                static_cast<int>(dq_smem)));
  kq<<<grid, kThreads, dq_smem, st>>>(dq, q, k, v, dout, lse, delta, S, scale, rate, rng, unit0,
                                     vec_ok);
  DAD_LAUNCH_CHECK("flash_bwd_dq_f32_kernel");
  return DADATTN_OK;
}

int check_common(int BH, int S, int d_head, float rate) {
  if (BH <= 0 || S <= 0) return fail(DADATTN_E_ARG, "BH=%d and S=%d must be positive", BH, S);
  if (BH > 65535) return fail(DADATTN_E_UNSUPPORTED, "BH=%d exceeds 65535 per call", BH);
  if (!dadattn_flash_supported(d_head))
    return fail(DADATTN_E_UNSUPPORTED, "flash attention: unsupported d_head %d", d_head);
  if (!(rate >= 0.0f && rate < 1.0f))
    return fail(DADATTN_E_ARG, "dropout rate %f outside [0,1)", static_cast<double>(rate));
  return DADATTN_OK;
}

}  // namespace
}  // namespace dadattn

using namespace dadattn;

extern "C" int dadattn_flash_supported(int d_head) {
  return d_head == 16 || d_head == 32 || d_head == 64 || d_head == 128;
}

extern "C" int dadattn_flash_fwd_f32_dropout(float* out, float* lse, const float* q,
                                             const float* k, const float* v, int BH, int S,
                                             int d_head, float scale, float rate, uint64_t seed,
                                             uint64_t offset, int64_t unit0,
                                             dadattn_stream_t stream) {
  if (int rc = check_common(BH, S, d_head, rate)) return rc;
  if (!out || !lse || !q || !k || !v) return fail(DADATTN_E_ARG, "null tensor pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define DAD_FWD(DH)                                                                             \
  case DH:                                                                                      \
    return rate > 0.f ? launch_fwd<DH, true>(out, lse, q, k, v, BH, S, scale, rate, seed,       \
                                             offset, unit0, st)                                 \
                      : launch_fwd<DH, false>(out, lse, q, k, v, BH, S, scale, 0.f, 0, 0, 0, st);
  switch (d_head) {
    DAD_FWD(16) DAD_FWD(32) DAD_FWD(64) DAD_FWD(128)
  }
#undef DAD_FWD
  return fail(DADATTN_E_UNSUPPORTED, "flash attention: unsupported d_head %d", d_head);
}

extern "C" int dadattn_flash_fwd_f32(float* out, float* lse, const float* q, const float* k,
                                     const float* v, int BH, int S, int d_head, float scale,
                                     dadattn_stream_t stream) {
  return dadattn_flash_fwd_f32_dropout(out, lse, q, k, v, BH, S, d_head, scale, 0.f, 0, 0, 0,
                                       stream);
}

extern "C" int dadattn_flash_bwd_f32_dropout(float* dq, float* dk, float* dv, float* delta,
                                             const float* dout, const float* out,
                                             const float* lse, const float* q, const float* k,
                                             const float* v, int BH, int S, int d_head,
                                             float scale, float rate, uint64_t seed,
                                             uint64_t offset, int64_t unit0,
                                             dadattn_stream_t stream) {
  if (int rc = check_common(BH, S, d_head, rate)) return rc;
  if (!dq || !dk || !dv || !delta || !dout || !out || !lse || !q || !k || !v)
    return fail(DADATTN_E_ARG, "null tensor pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define DAD_BWD(DH)                                                                             \
  case DH:                                                                                      \
    return rate > 0.f ? launch_bwd<DH, true>(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, \
                                             scale, rate, seed, offset, unit0, st)              \
                      : launch_bwd<DH, false>(dq, dk, dv, delta, dout, out, lse, q, k, v, BH,   \
                                              S, scale, 0.f, 0, 0, 0, st);
  switch (d_head) {
    DAD_BWD(16) DAD_BWD(32) DAD_BWD(64) DAD_BWD(128)
  }
#undef DAD_BWD
  return fail(DADATTN_E_UNSUPPORTED, "flash attention: unsupported d_head %d", d_head);
}

extern "C" int dadattn_flash_bwd_f32(float* dq, float* dk, float* dv, float* delta,
                                     const float* dout, const float* out, const float* lse,
                                     const float* q, const float* k, const float* v, int BH,
                                     int S, int d_head, float scale, dadattn_stream_t stream) {
  return dadattn_flash_bwd_f32_dropout(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S, d_head,
                                       scale, 0.f, 0, 0, 0, stream);
}
