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

// The same mask bit-packed for the fused kernels: one thread per 32-bit word = 32 consecutive
// keys of one query row of one 128 x 128 tile of the causal lower triangle (layout: common.cuh,
// mask_bits_record). Entries above the diagonal and rows beyond the sequence stay 0 and cost no
// draw. grid = (lower-triangle tiles, batch x head), 512 threads = 128 rows x 4 words, so a
// CTA's stores are one contiguous 2 KB record block.
template <bool WORD0>
__global__ void __launch_bounds__(512)
dropout_mask_bits_kernel(uint32_t* __restrict__ bits, int S, int n_tiles, float rate, PhiloxKey rng,
                         int64_t unit0) {
  // tile index -> (qt, kt) with qt (qt + 1) / 2 + kt = index
  const int idx = static_cast<int>(blockIdx.x);
  int qt = static_cast<int>((sqrtf(8.0f * static_cast<float>(idx) + 1.0f) - 1.0f) * 0.5f);
  while (qt * (qt + 1) / 2 > idx) --qt;
  while ((qt + 1) * (qt + 2) / 2 <= idx) ++qt;
  const int kt = idx - qt * (qt + 1) / 2;
  const int bh = static_cast<int>(blockIdx.y);
  const int row = threadIdx.x >> 2, w = threadIdx.x & 3;
  const int q = qt * kMaskTile + row;
  const int key0 = kt * kMaskTile + w * 32;
  uint32_t word = 0;
  if (q < S) {
    const uint64_t base = (static_cast<uint64_t>(unit0 + bh) * S + q) * S + key0;
    const int n = min(32, q - key0 + 1);   // keys key0 .. key0 + n - 1 are visible to query q
#pragma unroll 4
    for (int i = 0; i < n; ++i) {
      const uint32_t draw = WORD0 ? philox_draw_word0(rng, base + i) : philox_draw(rng, base + i);
      const float u = fmaf(static_cast<float>(draw), 2.3283064e-10f, 2.3283064e-10f / 2.0f);
      word |= (u < rate ? 0u : 1u) << i;
    }
  }
  bits[mask_bits_record(bh, qt, kt, row, n_tiles) * 4 + w] = word;
}

}  // namespace
}  // namespace dadattn

using namespace dadattn;

extern "C" size_t dadattn_dropout_mask_bits_bytes(int BH, int S) {
  if (BH <= 0 || S <= 0) return 0;
  return dropout_mask_bits_bytes(BH, S);
}

extern "C" int dadattn_dropout_mask_bits(uint32_t* bits, size_t bits_bytes, int BH, int S, float rate,
                                         uint64_t seed, uint64_t offset, int64_t unit0,
                                         dadattn_stream_t stream) {
  if (!bits || !aligned(bits, 16)) return fail(DADATTN_E_ARG, "dropout mask bits: need a 16-byte aligned buffer");
  if (BH <= 0 || S <= 0 || BH > 65535 || unit0 < 0)
    return fail(DADATTN_E_ARG, "dropout mask bits: bad sizes BH=%d S=%d", BH, S);
  if (!(rate >= 0.0f && rate < 1.0f))
    return fail(DADATTN_E_ARG, "dropout rate %f outside [0,1)", static_cast<double>(rate));
  if (bits_bytes < dropout_mask_bits_bytes(BH, S))
    return fail(DADATTN_E_WORKSPACE, "dropout mask bits: buffer %zu < %zu bytes", bits_bytes,
                dropout_mask_bits_bytes(BH, S));
  const int n_tiles = (S + kMaskTile - 1) / kMaskTile;
  const long long n_tri = static_cast<long long>(n_tiles) * (n_tiles + 1) / 2;
  if (n_tri > 0x7fffffffLL) return fail(DADATTN_E_UNSUPPORTED, "dropout mask bits: S too large");
  const PhiloxKey rng = make_philox(seed, offset);
  dim3 grid(static_cast<unsigned>(n_tri), static_cast<unsigned>(BH));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rng.word == 0)
    dropout_mask_bits_kernel<true><<<grid, 512, 0, st>>>(bits, S, n_tiles, rate, rng, unit0);
  else
    dropout_mask_bits_kernel<false><<<grid, 512, 0, st>>>(bits, S, n_tiles, rate, rng, unit0);
  DAD_LAUNCH_CHECK("dropout_mask_bits_kernel");
  return DADATTN_OK;
}

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
