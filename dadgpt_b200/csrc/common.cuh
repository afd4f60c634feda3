// Shared host/device helpers for the dadattn kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "dadattn.h"

namespace dadattn {

// Thread-local error text behind dadattn_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define DAD_CUDA(call)                                                                  \
  do {                                                                                  \
    cudaError_t e_ = (call);                                                            \
    if (e_ != cudaSuccess)                                                              \
      return ::dadattn::fail(DADATTN_E_CUDA, "%s failed: %s (%s:%d)", #call,            \
                             cudaGetErrorString(e_), __FILE__, __LINE__);               \
  } while (0)

#define DAD_LAUNCH_CHECK(name)                                                          \
  do {                                                                                  \
    cudaError_t e_ = cudaGetLastError();                                                \
    if (e_ != cudaSuccess)                                                              \
      return ::dadattn::fail(DADATTN_E_CUDA, "launch of %s failed: %s", name,           \
                             cudaGetErrorString(e_));                                   \
  } while (0)

// Device-side sticky status word (one per device that loads the library). Kernels record a
// DADATTN_E_* code here instead of trapping; dadattn_device_status() reads and clears it.
int* device_status_word();  // device pointer for the current device, nullptr on failure

// ---- Philox4x32-10 with cuRAND's curand_init(seed, subsequence, offset) counter set-up -------
// The reference draws one uniform per attention probability with subsequence = flat element
// index (cuda/gpu_ops.cu:712-727). key = seed; counter = {offset/4 (64 bit), subsequence}.
struct PhiloxKey {
  uint32_t k0, k1;       // seed
  uint32_t c0, c1;       // offset / 4
  uint32_t word;         // offset % 4
};

__host__ __device__ inline PhiloxKey make_philox(uint64_t seed, uint64_t offset) {
  PhiloxKey p;
  p.k0 = static_cast<uint32_t>(seed);
  p.k1 = static_cast<uint32_t>(seed >> 32);
  p.c0 = static_cast<uint32_t>(offset >> 2);
  p.c1 = static_cast<uint32_t>(offset >> 34);
  p.word = static_cast<uint32_t>(offset & 3);
  return p;
}

__device__ __forceinline__ uint32_t philox_draw(const PhiloxKey& p, uint64_t subsequence) {
  uint32_t c0 = p.c0, c1 = p.c1, c2 = static_cast<uint32_t>(subsequence),
           c3 = static_cast<uint32_t>(subsequence >> 32);
  uint32_t k0 = p.k0, k1 = p.k1;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return p.word == 0 ? c0 : p.word == 1 ? c1 : p.word == 2 ? c2 : c3;
}

// The same draw when the wanted word is the first of the block (offset a multiple of 4, as in
// every call the reference makes): both halves of each 32 x 32 product come from one widening
// multiply, the round keys are compile-time offsets of the seed, and the last round computes
// only the word that is used.
__device__ __forceinline__ uint32_t philox_draw_word0(const PhiloxKey& p, uint64_t subsequence) {
  uint32_t c0 = p.c0, c1 = p.c1, c2 = static_cast<uint32_t>(subsequence),
           c3 = static_cast<uint32_t>(subsequence >> 32);
#pragma unroll
  for (int r = 0; r < 9; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t k0 = p.k0 + static_cast<uint32_t>(r) * 0x9E3779B9u;
    const uint32_t k1 = p.k1 + static_cast<uint32_t>(r) * 0xBB67AE85u;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
    c1 = static_cast<uint32_t>(p1);
    c3 = static_cast<uint32_t>(p0);
    c0 = n0;
    c2 = n2;
  }
  return __umulhi(0xCD9E8D57u, c2) ^ c1 ^ (p.k0 + 9u * 0x9E3779B9u);
}

// true = keep. Same float arithmetic as curand_uniform followed by the reference's `r < rate`.
__device__ __forceinline__ bool philox_keep(const PhiloxKey& p, uint64_t subsequence,
                                            float rate) {
  float u = fmaf(static_cast<float>(philox_draw(p, subsequence)), 2.3283064e-10f,
                 2.3283064e-10f / 2.0f);
  return !(u < rate);
}

// ---- bit-packed dropout mask (dadattn_dropout_mask_bits) ----------------------------------------
// One 16-byte record per (batch x head, 128-query tile qt, 128-key tile kt <= qt, query row of
// the tile): bit i of 32-bit word w says whether the probability of key 32 w + i of the key tile
// is kept (1) or dropped (0). Records of a tile are contiguous (2 KB), tiles of a (batch, head)
// are numbered qt (qt + 1) / 2 + kt: only the causal lower triangle exists.
constexpr int kMaskTile = 128;
__host__ __device__ inline size_t mask_bits_record(int bh, int qt, int kt, int row, int n_tiles) {
  const size_t n_tri = static_cast<size_t>(n_tiles) * (n_tiles + 1) / 2;
  return (static_cast<size_t>(bh) * n_tri + static_cast<size_t>(qt) * (qt + 1) / 2 + kt) * kMaskTile + row;
}
inline size_t dropout_mask_bits_bytes(int BH, int S) {
  const size_t n_tiles = (static_cast<size_t>(S) + kMaskTile - 1) / kMaskTile;
  return static_cast<size_t>(BH) * (n_tiles * (n_tiles + 1) / 2) * kMaskTile * 16;
}

// Forward at head size 64 (flash_fwd64_sm100.cu). mask_bits != nullptr with rate > 0: keep bits
// from dadattn_dropout_mask_bits; mask_bits == nullptr with rate > 0: the Philox mask is drawn
// inside the kernel. heads > 0: tensors are the interleaved [B*S, heads*64] activations.
int launch_fwd_bf16_d64(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k,
                        const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                        uint64_t offset, int64_t unit0, const uint32_t* mask_bits, int heads,
                        cudaStream_t st);

// Launch with programmatic stream serialization: the grid may become resident while its
// predecessor in the stream drains, runs its set-up (barriers, TMEM, descriptor prefetch), and
// parks in pdl_wait() until the predecessor has completed and flushed its memory. Kernels
// launched this way call pdl_wait() before their first access to global memory.
template <typename Kernel, typename... Args>
cudaError_t launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                       Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

// Optional timing hooks of the bf16 backward (dadattn_set_stage_events): event i is recorded on
// the call's stream before its i-th kernel, and one more after the last kernel.
extern thread_local cudaEvent_t* g_stage_events;
extern thread_local int g_stage_event_count;
inline void stage_event(int i, cudaStream_t st) {
  if (g_stage_events && i < g_stage_event_count) cudaEventRecord(g_stage_events[i], st);
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace dadattn
