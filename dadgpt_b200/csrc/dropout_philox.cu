// Dropout keep/drop mask, bit-for-bit the mask the reference's dropout_forward_kernel writes
// (reference cuda/gpu_ops.cu:712-727): element i is dropped iff the first Philox4x32-10 uniform
// of curand_init(seed, subsequence = i, offset) is < rate. The reference launches one thread
// per byte; here a thread produces 16 consecutive bytes and stores them with one 128-bit write.
#include "common.cuh"

namespace dadattn {
namespace {

__global__ void dropout_mask_kernel(uint8_t* __restrict__ mask, int64_t n, float rate,
                                    PhiloxKey rng, int64_t first, int head) {
  // Bytes [0, head) bring the pointer to 16-byte alignment and are written singly, like the tail.
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t body = (n - head) / 16;
  if (t < body) {
    const int64_t i0 = head + t * 16;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t x = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b)
        x |= (philox_keep(rng, static_cast<uint64_t>(first + i0 + j * 4 + b), rate) ? 1u : 0u)
             << (8 * b);
      w[j] = x;
    }
    *reinterpret_cast<uint4*>(mask + i0) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
    // Ragged ends: at most 15 + 15 bytes, one per thread.
    const int64_t e = t - body;
    const int64_t tail0 = head + body * 16;
    int64_t i = -1;
    if (e < head) i = e;
    else if (e - head < n - tail0) i = tail0 + (e - head);
    if (i >= 0 && i < n)
      mask[i] = philox_keep(rng, static_cast<uint64_t>(first + i), rate) ? 1 : 0;
  }
}

}  // namespace
}  // namespace dadattn

using namespace dadattn;

extern "C" int dadattn_dropout_mask(uint8_t* mask, int64_t n, float rate, uint64_t seed,
                                    uint64_t offset, int64_t first, dadattn_stream_t stream) {
  if (n == 0) return DADATTN_OK;
  if (!mask || n < 0 || first < 0) return fail(DADATTN_E_ARG, "dropout mask: bad pointer or size");
  if (!(rate >= 0.0f && rate <= 1.0f))
    return fail(DADATTN_E_ARG, "dropout rate %f outside [0,1]", static_cast<double>(rate));
  int head = static_cast<int>((16 - reinterpret_cast<uintptr_t>(mask) % 16) % 16);
  if (head > n) head = static_cast<int>(n);
  const int64_t body = (n - head) / 16;
  const int64_t threads = body + 32;  // 30 ragged bytes at most
  const int64_t blocks = (threads + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(DADATTN_E_UNSUPPORTED, "dropout mask: n too large");
  dropout_mask_kernel<<<static_cast<unsigned>(blocks), 256, 0,
                        static_cast<cudaStream_t>(stream)>>>(mask, n, rate,
                                                             make_philox(seed, offset), first,
                                                             head);
  DAD_LAUNCH_CHECK("dropout_mask_kernel");
  return DADATTN_OK;
}
