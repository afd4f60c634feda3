// fp32 tensors in, fp32 tensors out, tensor-core arithmetic in between.
//
// DadGPT keeps every activation in fp32 and selects reduced precision per operation: its
// gpu_set_matmul_precision(BF16) (reference cuda/gpu_ops.cuh:43-44, the training default in
// src/train.hpp:29) makes cuBLAS round the GEMM operands to bf16 and accumulate in fp32. The
// entry points here give the fused attention the same contract: q, k, v (and dO, O) are rounded
// to bf16 on the fly into a workspace, the tcgen05 kernels of flash_bf16_sm100.cu /
// flash_bwd_*_sm100.cu run on them with fp32 softmax and accumulation, and the results are
// widened back to the caller's fp32 tensors. lse is written in fp32 directly. The drop-in shim
// (gpu_ops_attention.cpp) routes the reference's fp32 signatures here when the precision mode
// says so; the exact-fp32 kernels of flash_f32.cu remain the default.
#include <cuda_bf16.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace dadattn {
namespace {

constexpr int kMaxCast = 5;
struct CastList {
  const void* src[kMaxCast];
  void* dst[kMaxCast];
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// blockIdx.y selects the tensor; eight elements per thread
__global__ void cast_f32_to_bf16_kernel(CastList list, int64_t n8) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= n8) return;
  const float4* s = reinterpret_cast<const float4*>(list.src[blockIdx.y]) + 2 * t;
  const float4 a = s[0], b = s[1];
  reinterpret_cast<uint4*>(list.dst[blockIdx.y])[t] =
      make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
}

__global__ void cast_bf16_to_f32_kernel(CastList list, int64_t n8) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= n8) return;
  const uint4 w = reinterpret_cast<const uint4*>(list.src[blockIdx.y])[t];
  float4* d = reinterpret_cast<float4*>(list.dst[blockIdx.y]) + 2 * t;
  d[0] = make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u),
                     __uint_as_float(w.y << 16), __uint_as_float(w.y & 0xffff0000u));
  d[1] = make_float4(__uint_as_float(w.z << 16), __uint_as_float(w.z & 0xffff0000u),
                     __uint_as_float(w.w << 16), __uint_as_float(w.w & 0xffff0000u));
}

int launch_cast(bool to_bf16, const CastList& list, int count, int64_t elems, cudaStream_t st) {
  const int64_t n8 = elems / 8;
  dim3 grid(static_cast<unsigned>((n8 + 255) / 256), count);
  if (to_bf16)
    DAD_CUDA(launch_pdl(cast_f32_to_bf16_kernel, grid, dim3(256), 0, st, list, n8));
  else
    DAD_CUDA(launch_pdl(cast_bf16_to_f32_kernel, grid, dim3(256), 0, st, list, n8));
  return DADATTN_OK;
}

size_t tensor_bytes(int BH, int S, int D) {
  return (static_cast<size_t>(BH) * S * D * sizeof(uint16_t) + 255) / 256 * 256;
}

int check_common(int BH, int S, int D, float scale, const void* workspace, size_t given) {
  if (BH <= 0 || S <= 0) return fail(DADATTN_E_ARG, "via bf16: bad sizes BH=%d S=%d", BH, S);
  if (D != 64 && D != 128) return fail(DADATTN_E_UNSUPPORTED, "via bf16: unsupported d_head %d", D);
  if (!(scale > 0.f)) return fail(DADATTN_E_ARG, "via bf16: scale must be positive");
  if (!workspace || !aligned(workspace, 256))
    return fail(DADATTN_E_ARG, "via bf16: workspace must be a 256-byte aligned device pointer");
  const size_t need = dadattn_flash_f32_via_bf16_workspace_bytes(BH, S, D);
  if (given < need) return fail(DADATTN_E_WORKSPACE, "via bf16: workspace %zu < %zu bytes", given, need);
  return DADATTN_OK;
}

std::atomic<int> g_precision{-1};  // -1: not decided yet (environment consulted on first read)

constexpr int kMaxDevices = 64;
void* g_scratch[kMaxDevices] = {};
size_t g_scratch_bytes[kMaxDevices] = {};
std::mutex g_scratch_mutex;

}  // namespace
}  // namespace dadattn

using namespace dadattn;

extern "C" size_t dadattn_flash_f32_via_bf16_workspace_bytes(int BH, int S, int D) {
  if (BH <= 0 || S <= 0 || D <= 0) return 0;
  // bf16 copies of q, k, v, out, dout and dq, dk, dv, then the bf16 backward's own workspace
  const size_t bwd = (dadattn_flash_bwd_bf16_workspace_bytes(BH, S, D) + 255) / 256 * 256;
  return 8 * tensor_bytes(BH, S, D) + bwd;
}

extern "C" int dadattn_flash_fwd_f32_via_bf16(float* out, float* lse, const float* q, const float* k,
                                              const float* v, int BH, int S, int D, float scale,
                                              void* workspace, size_t workspace_bytes,
                                              dadattn_stream_t stream) {
  if (!out || !lse || !q || !k || !v) return fail(DADATTN_E_ARG, "via bf16: null pointer");
  if (int rc = check_common(BH, S, D, scale, workspace, workspace_bytes)) return rc;
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16))
    return fail(DADATTN_E_ARG, "via bf16: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t tb = tensor_bytes(BH, S, D);
  char* w = static_cast<char*>(workspace);
  uint16_t *bq = reinterpret_cast<uint16_t*>(w), *bk = reinterpret_cast<uint16_t*>(w + tb),
           *bv = reinterpret_cast<uint16_t*>(w + 2 * tb), *bo = reinterpret_cast<uint16_t*>(w + 3 * tb);
  const int64_t elems = static_cast<int64_t>(BH) * S * D;
  CastList in = {{q, k, v}, {bq, bk, bv}};
  if (int rc = launch_cast(true, in, 3, elems, st)) return rc;
  if (int rc = dadattn_flash_fwd_bf16(bo, lse, bq, bk, bv, BH, S, D, scale, 0.f, 0, 0, 0, stream)) return rc;
  CastList back = {{bo}, {out}};
  return launch_cast(false, back, 1, elems, st);
}

extern "C" int dadattn_flash_bwd_f32_via_bf16(float* dq, float* dk, float* dv, const float* dout,
                                              const float* out, const float* lse, const float* q,
                                              const float* k, const float* v, int BH, int S, int D,
                                              float scale, void* workspace, size_t workspace_bytes,
                                              dadattn_stream_t stream) {
  if (!dq || !dk || !dv || !dout || !out || !lse || !q || !k || !v)
    return fail(DADATTN_E_ARG, "via bf16: null pointer");
  if (int rc = check_common(BH, S, D, scale, workspace, workspace_bytes)) return rc;
  if (!aligned(dq, 16) || !aligned(dk, 16) || !aligned(dv, 16) || !aligned(dout, 16) ||
      !aligned(out, 16) || !aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16))
    return fail(DADATTN_E_ARG, "via bf16: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t tb = tensor_bytes(BH, S, D);
  char* w = static_cast<char*>(workspace);
  uint16_t* b[8];
  for (int i = 0; i < 8; ++i) b[i] = reinterpret_cast<uint16_t*>(w + i * tb);
  void* bwd_ws = w + 8 * tb;
  const size_t bwd_bytes = dadattn_flash_bwd_bf16_workspace_bytes(BH, S, D);
  const int64_t elems = static_cast<int64_t>(BH) * S * D;
  CastList in = {{q, k, v, out, dout}, {b[0], b[1], b[2], b[3], b[4]}};
  if (int rc = launch_cast(true, in, 5, elems, st)) return rc;
  if (int rc = dadattn_flash_bwd_bf16(b[5], b[6], b[7], bwd_ws, bwd_bytes, b[4], b[3], lse, b[0], b[1],
                                      b[2], BH, S, D, scale, 0.f, 0, 0, 0, stream))
    return rc;
  CastList back = {{b[5], b[6], b[7]}, {dq, dk, dv}};
  return launch_cast(false, back, 3, elems, st);
}

extern "C" int dadattn_set_f32_precision(int mode) {
  if (mode != 0 && mode != 1) return fail(DADATTN_E_ARG, "precision mode %d (0 = fp32, 1 = bf16)", mode);
  g_precision.store(mode);
  return DADATTN_OK;
}

extern "C" int dadattn_get_f32_precision(void) {
  int mode = g_precision.load();
  if (mode < 0) {
    const char* env = std::getenv("DADATTN_PRECISION");
    mode = (env && (!std::strcmp(env, "bf16") || !std::strcmp(env, "BF16"))) ? 1 : 0;
    g_precision.store(mode);
  }
  return mode;
}

extern "C" int dadattn_library_scratch(size_t bytes, void** ptr) {
  if (!ptr) return fail(DADATTN_E_ARG, "scratch: null pointer");
  int dev = 0;
  DAD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(DADATTN_E_UNSUPPORTED, "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_bytes[dev] < bytes) {
    // Work already enqueued on the old buffer must finish before it is released.
    if (g_scratch[dev]) {
      DAD_CUDA(cudaDeviceSynchronize());
      DAD_CUDA(cudaFree(g_scratch[dev]));
      g_scratch[dev] = nullptr;
      g_scratch_bytes[dev] = 0;
    }
    void* p = nullptr;
    DAD_CUDA(cudaMalloc(&p, bytes));
    g_scratch[dev] = p;
    g_scratch_bytes[dev] = bytes;
  }
  *ptr = g_scratch[dev];
  return DADATTN_OK;
}
