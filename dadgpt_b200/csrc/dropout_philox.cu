// Dropout keep/drop mask, bit-for-bit the mask the reference's dropout_forward_kernel writes
// (reference cuda/gpu_ops.cu:712-727): element i is dropped iff the first Philox4x32-10 uniform
// of curand_init(seed, subsequence = i, offset) is < rate. The reference launches one thread
// per byte; here a thread produces 16 consecutive bytes and stores them with one 128-bit write.
#include <cmath>

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
//
// The kernel is bound by instruction issue (ten Philox rounds per probability), so the draw is
// stripped to what the reference's mask needs: the round keys come precomputed from the host
// (kernel parameters, i.e. constant-bank operands: no per-draw additions, no registers), both
// halves of each 32 x 32 product come from one widening multiply, the last round computes only
// the word that is used, and "uniform < rate" is decided on the integer draw: the uniform is a
// non-decreasing function of the draw (cvt.rn then one fma), so the dropped draws are exactly
// those below a threshold that the host finds with the same float arithmetic.
struct PhiloxRounds {
  uint32_t k0[10], k1[9];   // key words of rounds 0..9 (the last round needs only k0)
  uint32_t c0, c1;          // low counter words: offset / 4
  uint32_t word;            // offset % 4: which word of the block is the draw
  uint32_t drop_below;      // draws below this are dropped (uniform < rate)
};

__device__ __forceinline__ bool keep_word0(const PhiloxRounds& p, uint32_t s_lo, uint32_t s_hi) {
  uint32_t c0 = p.c0, c1 = p.c1, c2 = s_lo, c3 = s_hi;
#pragma unroll
  for (int r = 0; r < 9; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ p.k0[r];
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ p.k1[r];
    c1 = static_cast<uint32_t>(p1);
    c3 = static_cast<uint32_t>(p0);
    c0 = n0;
    c2 = n2;
  }
  const uint32_t draw = __umulhi(0xCD9E8D57u, c2) ^ c1 ^ p.k0[9];
  return draw >= p.drop_below;
}

template <bool WORD0>
__global__ void __launch_bounds__(512)
dropout_mask_bits_kernel(uint32_t* __restrict__ bits, int S, int n_tiles, float rate,
                         const __grid_constant__ PhiloxRounds rounds, PhiloxKey rng, int64_t unit0) {
  // tile index -> (qt, kt) with qt (qt + 1) / 2 + kt = index
  const int idx = static_cast<int>(blockIdx.x);
  int qt = static_cast<int>((sqrtf(8.0f * static_cast<float>(idx) + 1.0f) - 1.0f) * 0.5f);
  while (qt * (qt + 1) / 2 > idx) --qt;
  while ((qt + 1) * (qt + 2) / 2 <= idx) ++qt;
  const int kt = idx - qt * (qt + 1) / 2;
  const int bh = static_cast<int>(blockIdx.y);
  // A warp takes one 32-key word of 32 consecutive rows: on a diagonal tile the 32 x 32 blocks
  // above the diagonal then cost nothing (a warp whose lanes mix words always has a lane with a
  // full word to draw).
  const int row = ((threadIdx.x >> 5) & 3) * 32 + (threadIdx.x & 31), w = threadIdx.x >> 7;
  const int q = qt * kMaskTile + row;
  const int key0 = kt * kMaskTile + w * 32;
  uint32_t word = 0;
  if (q < S) {
    const uint64_t base = (static_cast<uint64_t>(unit0 + bh) * S + q) * S + key0;
    const int n = min(32, q - key0 + 1);   // keys key0 .. key0 + n - 1 are visible to query q
    if (WORD0) {
      const uint32_t lo = static_cast<uint32_t>(base), hi = static_cast<uint32_t>(base >> 32);
      if (n == 32) {
#pragma unroll 8
        for (int i = 0; i < 32; ++i)
          word |= (keep_word0(rounds, lo + i, hi + (lo + i < lo ? 1u : 0u)) ? 1u : 0u) << i;
      } else {
#pragma unroll 4
        for (int i = 0; i < n; ++i)
          word |= (keep_word0(rounds, lo + i, hi + (lo + i < lo ? 1u : 0u)) ? 1u : 0u) << i;
      }
    } else {
#pragma unroll 4
      for (int i = 0; i < n; ++i) word |= (philox_keep(rng, base + i, rate) ? 1u : 0u) << i;
    }
  }
  bits[mask_bits_record(bh, qt, kt, row, n_tiles) * 4 + w] = word;
}

// Smallest draw that is NOT dropped: the uniform fmaf(float(draw), 2^-32, 2^-33) of
// curand_uniform is non-decreasing in the draw, so a binary search with the very same float
// operations finds the threshold exactly. rate < 1 keeps the largest draw (its uniform is 1).
uint32_t drop_threshold(float rate) {
  auto dropped = [rate](uint32_t d) {
    const float u = fmaf(static_cast<float>(d), 2.3283064e-10f, 2.3283064e-10f / 2.0f);
    return u < rate;
  };
  if (!dropped(0)) return 0;
  uint32_t lo = 0, hi = 0xFFFFFFFFu;   // dropped(lo), !dropped(hi)
  while (hi - lo > 1) {
    const uint32_t mid = lo + (hi - lo) / 2;
    if (dropped(mid)) lo = mid; else hi = mid;
  }
  return hi;
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
  PhiloxRounds rounds;
  for (int r = 0; r < 10; ++r) {
    rounds.k0[r] = rng.k0 + static_cast<uint32_t>(r) * 0x9E3779B9u;
    if (r < 9) rounds.k1[r] = rng.k1 + static_cast<uint32_t>(r) * 0xBB67AE85u;
  }
  rounds.c0 = rng.c0;
  rounds.c1 = rng.c1;
  rounds.word = rng.word;
  rounds.drop_below = drop_threshold(rate);
  dim3 grid(static_cast<unsigned>(n_tri), static_cast<unsigned>(BH));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rng.word == 0)
    dropout_mask_bits_kernel<true><<<grid, 512, 0, st>>>(bits, S, n_tiles, rate, rounds, rng, unit0);
  else
    dropout_mask_bits_kernel<false><<<grid, 512, 0, st>>>(bits, S, n_tiles, rate, rounds, rng, unit0);
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
