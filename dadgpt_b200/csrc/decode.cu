// KV-cache decode attention: one new query token per sequence against that sequence's cache.
//
// The reference runs this as 61 tiny launches per layer (per-head M=1 cuBLAS products, 256-byte
// device-to-device appends, one softmax; src/model.cpp:745-790). Here it is one split-K kernel
// plus a small combine kernel per layer call, for any number of concurrent sequences:
//   * grid = (splits, heads, sequences); a CTA owns `chunk` consecutive cache rows of one
//     (sequence, head) and exits at once when the chunk lies beyond the sequence's length;
//   * a cache row (D elements) is read by D*sizeof(T)/16 adjacent lanes with one 128-bit load
//     each, so a warp instruction covers 512 contiguous bytes of the cache; K and V rows of
//     several iterations are issued before any is consumed (memory-level parallelism is what a
//     bandwidth-bound kernel lives on);
//   * q.k partial sums are reduced over those lanes with warp shuffles; each lane keeps an
//     online-softmax state (max, sum, D/lanes accumulators) for the rows it has seen;
//   * the append is fused: the lanes that own row `len` take k_new/v_new from the token's
//     vectors, use them, and store them into the cache;
//   * per-CTA results go to the split-K workspace as (unnormalised out[D], max, sum) and the
//     combine kernel merges the splits, writes out, and bumps the sequence length.
// In direct mode (one split; the fp32 single-sequence path) the CTA normalises and writes the
// output itself and no workspace is used.
#include <cfloat>
#include <cuda_bf16.h>

#include "common.cuh"

namespace dadattn {
namespace {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeUnroll = 4;

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerLane = 4;
  __device__ static void unpack(float (&f)[4], const uint4& raw) {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
    f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
  }
  __device__ static float to_float(float x) { return x; }
  __device__ static float from_float(float x) { return x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerLane = 8;
  __device__ static void unpack(float (&f)[8], const uint4& raw) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Workspace record per (sequence, head, split): D floats of unnormalised output, then max, sum.
__host__ __device__ inline size_t partial_stride(int D) { return static_cast<size_t>(D) + 2; }

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_splitk_kernel(T* __restrict__ out, float* __restrict__ partial, const T* __restrict__ q,
                     const T* __restrict__ k_new, const T* __restrict__ v_new,
                     T* __restrict__ k_cache, T* __restrict__ v_cache,
                     const int32_t* __restrict__ lengths, int fixed_len, int H, int max_len,
                     int chunk, float scale, int direct, int* __restrict__ status) {
  constexpr int EPL = Elem<T>::kPerLane;  // elements per lane (one 16-byte load)
  constexpr int LPK = D / EPL;            // lanes per cache row
  constexpr int KPI = 32 / LPK;           // cache rows per warp instruction
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "row must split over a warp");

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int splits = gridDim.x;
  const int len = lengths ? lengths[b] : fixed_len;  // rows already in the cache
  if (len < 0 || len >= max_len) {
    if (split == 0 && h == 0 && threadIdx.x == 0) atomicExch(status, DADATTN_E_ARG);
    return;
  }
  const int total = len + 1;  // rows visible to the new token, itself included
  const int row_begin = split * chunk;
  if (row_begin >= total) return;
  const int row_end = min(row_begin + chunk, total);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int slot = lane / LPK, part = lane % LPK;
  const size_t vec_off = (static_cast<size_t>(b) * H + h) * D + part * EPL;
  const size_t cache_base = (static_cast<size_t>(b) * H + h) * max_len * D + part * EPL;

  float qf[EPL];
  Elem<T>::unpack(qf, *reinterpret_cast<const uint4*>(q + vec_off));

  float m = -FLT_MAX, l = 0.f, acc[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) acc[e] = 0.f;

  for (int base = row_begin + warp * KPI; base < row_end; base += kDecodeWarps * KPI * kDecodeUnroll) {
    uint4 kr[kDecodeUnroll], vr[kDecodeUnroll];
    bool ok[kDecodeUnroll];
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      const int row = base + u * kDecodeWarps * KPI + slot;
      ok[u] = row < row_end;
      kr[u] = make_uint4(0, 0, 0, 0);
      vr[u] = make_uint4(0, 0, 0, 0);
      if (ok[u]) {
        if (row == len) {  // the token being appended: use its vectors and store them
          kr[u] = *reinterpret_cast<const uint4*>(k_new + vec_off);
          vr[u] = *reinterpret_cast<const uint4*>(v_new + vec_off);
          *reinterpret_cast<uint4*>(k_cache + cache_base + static_cast<size_t>(row) * D) = kr[u];
          *reinterpret_cast<uint4*>(v_cache + cache_base + static_cast<size_t>(row) * D) = vr[u];
        } else {
          kr[u] = ld_stream(k_cache + cache_base + static_cast<size_t>(row) * D);
          vr[u] = ld_stream(v_cache + cache_base + static_cast<size_t>(row) * D);
        }
      }
    }
    float s[kDecodeUnroll];
    float m_new = m;
#pragma unroll
    for (int u = 0; u < kDecodeUnroll; ++u) {
      float kf[EPL];
      Elem<T>::unpack(kf, kr[u]);
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) dot = fmaf(qf[e], kf[e], dot);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      s[u] = ok[u] ? dot * scale : -FLT_MAX;
      m_new = fmaxf(m_new, s[u]);
    }
    if (m_new > -FLT_MAX) {  // at least one row seen by this lane group so far
      const float corr = expf(m - m_new);
      l *= corr;
#pragma unroll
      for (int e = 0; e < EPL; ++e) acc[e] *= corr;
#pragma unroll
      for (int u = 0; u < kDecodeUnroll; ++u) {
        if (!ok[u]) continue;
        const float p = expf(s[u] - m_new);
        l += p;
        float vf[EPL];
        Elem<T>::unpack(vf, vr[u]);
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] = fmaf(p, vf[e], acc[e]);
      }
      m = m_new;
    }
  }

  // Merge the KPI row-slots of the warp (lanes with equal `part`), then the warps.
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
    const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
    const float m_new = fmaxf(m, m_o);
    const float ca = m > -FLT_MAX ? expf(m - m_new) : 0.f;
    const float cb = m_o > -FLT_MAX ? expf(m_o - m_new) : 0.f;
    l = l * ca + l_o * cb;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float a_o = __shfl_xor_sync(0xffffffffu, acc[e], o);
      acc[e] = acc[e] * ca + a_o * cb;
    }
    m = m_new;
  }

  __shared__ float sh_acc[kDecodeWarps][D];
  __shared__ float sh_m[kDecodeWarps], sh_l[kDecodeWarps];
  if (slot == 0) {
#pragma unroll
    for (int e = 0; e < EPL; ++e) sh_acc[warp][part * EPL + e] = acc[e];
    if (part == 0) {
      sh_m[warp] = m;
      sh_l[warp] = l;
    }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += kDecodeWarps * 32) {
    float mm = -FLT_MAX;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) mm = fmaxf(mm, sh_m[w]);
    float ll = 0.f, aa = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float c = sh_m[w] > -FLT_MAX ? expf(sh_m[w] - mm) : 0.f;
      ll += sh_l[w] * c;
      aa += sh_acc[w][d] * c;
    }
    if (direct) {
      out[(static_cast<size_t>(b) * H + h) * D + d] = Elem<T>::from_float(aa / ll);
    } else {
      float* rec = partial + ((static_cast<size_t>(b) * H + h) * splits + split) * partial_stride(D);
      rec[d] = aa;
      if (d == 0) {
        rec[D] = mm;
        rec[D + 1] = ll;
      }
    }
  }
}

// Merges the split-K records of one (sequence, head), writes out, and (head 0) stores len + 1.
template <typename T, int D>
__global__ void decode_combine_kernel(T* __restrict__ out, const float* __restrict__ partial,
                                      int32_t* __restrict__ lengths, int H, int max_len,
                                      int chunk, int splits) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int len = lengths[b];
  if (len < 0 || len >= max_len) return;
  const int used = min(splits, (len + 1 + chunk - 1) / chunk);
  const float* rec = partial + (static_cast<size_t>(b) * H + h) * splits * partial_stride(D);
  float mm = -FLT_MAX;
  for (int s = 0; s < used; ++s) mm = fmaxf(mm, rec[s * partial_stride(D) + D]);
  float ll = 0.f, aa = 0.f;
  for (int s = 0; s < used; ++s) {
    const float* r = rec + s * partial_stride(D);
    const float c = expf(r[D] - mm);
    ll += r[D + 1] * c;
    aa += r[d] * c;
  }
  out[(static_cast<size_t>(b) * H + h) * D + d] = Elem<T>::from_float(aa / ll);
  __syncthreads();
  // Safe to bump here: every split-K CTA of this call finished before this kernel started.
  if (h == 0 && d == 0) lengths[b] = len + 1;
}

// Rows of the cache per CTA. 128 rows = 32 per warp = 8 K + 8 V 16-byte loads in flight per lane.
constexpr int kChunk = 128;

}  // namespace
}  // namespace dadattn

using namespace dadattn;

extern "C" size_t dadattn_decode_workspace_bytes(int B, int H, int D, int max_len) {
  if (B <= 0 || H <= 0 || D <= 0 || max_len <= 0) return 0;
  const size_t splits = (static_cast<size_t>(max_len) + kChunk - 1) / kChunk;
  return static_cast<size_t>(B) * H * splits * partial_stride(D) * sizeof(float);
}

extern "C" int dadattn_decode_bf16(uint16_t* out, const uint16_t* q, const uint16_t* k_new,
                                   const uint16_t* v_new, uint16_t* k_cache, uint16_t* v_cache,
                                   int32_t* lengths, int B, int H, int D, int max_len,
                                   float scale, void* workspace, size_t workspace_bytes,
                                   dadattn_stream_t stream) {
  if (!out || !q || !k_new || !v_new || !k_cache || !v_cache || !lengths || !workspace)
    return fail(DADATTN_E_ARG, "decode: null pointer");
  if (B <= 0 || H <= 0 || max_len <= 0 || B > 65535 || H > 65535)
    return fail(DADATTN_E_ARG, "decode: bad sizes B=%d H=%d max_len=%d", B, H, max_len);
  if (D != 64 && D != 128) return fail(DADATTN_E_UNSUPPORTED, "decode bf16: unsupported D %d", D);
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16) ||
      !aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(workspace, 16))
    return fail(DADATTN_E_ARG, "decode: pointers must be 16-byte aligned");
  if (workspace_bytes < dadattn_decode_workspace_bytes(B, H, D, max_len))
    return fail(DADATTN_E_WORKSPACE, "decode: workspace %zu < %zu bytes", workspace_bytes,
                dadattn_decode_workspace_bytes(B, H, D, max_len));
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int splits = (max_len + kChunk - 1) / kChunk;
  using T = __nv_bfloat16;
  dim3 grid(splits, H, B), cgrid(H, B);
  float* partial = static_cast<float*>(workspace);
#define DAD_DECODE(DH)                                                                          \
  decode_splitk_kernel<T, DH><<<grid, kDecodeWarps * 32, 0, st>>>(                              \
      reinterpret_cast<T*>(out), partial, reinterpret_cast<const T*>(q),                        \
      reinterpret_cast<const T*>(k_new), reinterpret_cast<const T*>(v_new),                     \
      reinterpret_cast<T*>(k_cache), reinterpret_cast<T*>(v_cache), lengths, 0, H, max_len,     \
      kChunk, scale, 0, status);                                           \
  DAD_LAUNCH_CHECK("decode_splitk_kernel");                                                     \
  decode_combine_kernel<T, DH><<<cgrid, DH, 0, st>>>(reinterpret_cast<T*>(out), partial,        \
                                                     lengths, H, max_len, kChunk, splits);      \
  DAD_LAUNCH_CHECK("decode_combine_kernel");
  if (D == 64) {
    DAD_DECODE(64)
  } else {
    DAD_DECODE(128)
  }
#undef DAD_DECODE
  return DADATTN_OK;
}

extern "C" int dadattn_decode_f32(float* out, const float* q, const float* k_new,
                                  const float* v_new, float* k_cache, float* v_cache, int H,
                                  int max_len, int D, int pos, float scale,
                                  dadattn_stream_t stream) {
  if (!out || !q || !k_new || !v_new || !k_cache || !v_cache)
    return fail(DADATTN_E_ARG, "decode: null pointer");
  if (H <= 0 || max_len <= 0 || H > 65535) return fail(DADATTN_E_ARG, "decode: bad sizes");
  if (pos < 0 || pos >= max_len)
    return fail(DADATTN_E_ARG, "decode: pos %d outside context length %d", pos, max_len);
  if (D != 16 && D != 32 && D != 64 && D != 128)
    return fail(DADATTN_E_UNSUPPORTED, "decode f32: unsupported D %d", D);
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16) ||
      !aligned(k_cache, 16) || !aligned(v_cache, 16))
    return fail(DADATTN_E_ARG, "decode: pointers must be 16-byte aligned");
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(1, H, 1);
#define DAD_DECODE32(DH)                                                                        \
  case DH:                                                                                      \
    decode_splitk_kernel<float, DH><<<grid, kDecodeWarps * 32, 0, st>>>(                        \
        out, nullptr, q, k_new, v_new, k_cache, v_cache, nullptr, pos, H, max_len, max_len,     \
        scale, 1, status);                                                                      \
    break;
  switch (D) {
    DAD_DECODE32(16) DAD_DECODE32(32) DAD_DECODE32(64) DAD_DECODE32(128)
  }
#undef DAD_DECODE32
  DAD_LAUNCH_CHECK("decode_splitk_kernel<float>");
  return DADATTN_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode without any allocation.
//
// Some hosts of this library must not allocate device memory once they are running: a serving
// process that hands every free byte of HBM to its own cache pool at start-up has nothing left
// for a later cudaMalloc; a latency-critical decode loop cannot afford the device-wide
// synchronisation an allocation implies; and DadGPT itself sizes all of its buffers once, in
// model_alloc / kv_cache_alloc, and never allocates inside generate_tokens. For such callers the
// split-K partials live in the fixed array below instead of a caller-provided workspace, and
// the bad-length report goes to a fixed word instead of the lazily allocated status word.
//
// The array is part of the library image: every GPU that loads libdadattn.so holds these
// 8 MiB until the process exits, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------------------------
namespace dadattn {
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_decode_scratch[kNoAllocScratchBytes];
static __device__ int g_decode_noalloc_status;

constexpr int kNoAllocMaxDevices = 64;
float* g_scratch_ptr[kNoAllocMaxDevices] = {};
int* g_noalloc_status_ptr[kNoAllocMaxDevices] = {};

// In host code the names g_decode_scratch / g_decode_noalloc_status are only handles; the
// device addresses a kernel can use come from cudaGetSymbolAddress, per device, with that
// device current. Looked up on the first call on each device and cached.
int noalloc_setup(float** scratch, int** status) {
  int dev = 0;
  DAD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices)
    return fail(DADATTN_E_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (!g_scratch_ptr[dev] || !g_noalloc_status_ptr[dev]) {
    float* s = nullptr;
    int* w = nullptr;
    DAD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&s), g_decode_scratch));
    DAD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&w), g_decode_noalloc_status));
    g_noalloc_status_ptr[dev] = w;
    g_scratch_ptr[dev] = s;
  }
  *scratch = g_scratch_ptr[dev];
  *status = g_noalloc_status_ptr[dev];
  return DADATTN_OK;
}

template <int DH>
int launch_decode_noalloc(uint16_t* out, const uint16_t* q, const uint16_t* k_new,
                          const uint16_t* v_new, uint16_t* k_cache, uint16_t* v_cache,
                          int32_t* lengths, int B, int H, int max_len, float scale,
                          float* partial, int* status, cudaStream_t st) {
  using T = __nv_bfloat16;
  const int splits = (max_len + kChunk - 1) / kChunk;
  dim3 grid(splits, H, B), cgrid(H, B);
  decode_splitk_kernel<T, DH><<<grid, kDecodeWarps * 32, 0, st>>>(
      reinterpret_cast<T*>(out), partial, reinterpret_cast<const T*>(q),
      reinterpret_cast<const T*>(k_new), reinterpret_cast<const T*>(v_new),
      reinterpret_cast<T*>(k_cache), reinterpret_cast<T*>(v_cache), lengths, 0, H, max_len, kChunk,
      scale, 0, status);
  DAD_LAUNCH_CHECK("decode_splitk_kernel (no-alloc)");
  decode_combine_kernel<T, DH><<<cgrid, DH, 0, st>>>(reinterpret_cast<T*>(out), partial, lengths,
                                                     H, max_len, kChunk, splits);
  DAD_LAUNCH_CHECK("decode_combine_kernel (no-alloc)");
  return DADATTN_OK;
}

}  // namespace
}  // namespace dadattn

extern "C" int dadattn_decode_bf16_noalloc(uint16_t* out, const uint16_t* q,
                                           const uint16_t* k_new, const uint16_t* v_new,
                                           uint16_t* k_cache, uint16_t* v_cache, int32_t* lengths,
                                           int B, int H, int D, int max_len, float scale,
                                           dadattn_stream_t stream) {
  if (!out || !q || !k_new || !v_new || !k_cache || !v_cache || !lengths)
    return fail(DADATTN_E_ARG, "decode: null pointer");
  if (B <= 0 || H <= 0 || max_len <= 0 || B > 65535 || H > 65535)
    return fail(DADATTN_E_ARG, "decode: bad sizes B=%d H=%d max_len=%d", B, H, max_len);
  if (D != 64 && D != 128) return fail(DADATTN_E_UNSUPPORTED, "decode bf16: unsupported D %d", D);
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16) ||
      !aligned(k_cache, 16) || !aligned(v_cache, 16))
    return fail(DADATTN_E_ARG, "decode: pointers must be 16-byte aligned");
  const size_t need = dadattn_decode_workspace_bytes(B, H, D, max_len);
  if (need > kNoAllocScratchBytes)
    return fail(DADATTN_E_WORKSPACE,
                "decode (no-alloc): B=%d H=%d D=%d max_len=%d needs %zu bytes of split-K scratch, "
                "the built-in array holds %zu; use dadattn_decode_bf16 with your own workspace",
                B, H, D, max_len, need, static_cast<size_t>(kNoAllocScratchBytes));
  float* partial = nullptr;
  int* status = nullptr;
  if (int rc = noalloc_setup(&partial, &status)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return D == 64 ? launch_decode_noalloc<64>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H,
                                             max_len, scale, partial, status, st)
                 : launch_decode_noalloc<128>(out, q, k_new, v_new, k_cache, v_cache, lengths, B,
                                              H, max_len, scale, partial, status, st);
}
