// bf16 fused causal attention backward for sm_100a (tcgen05 / TMEM / TMA).
//
// Same decomposition as the reference's backward (cuda/attention.cu:215-228): one kernel that
// owns query tiles and produces dQ (and, on the way, the reference's delta pre-pass), one that
// owns key tiles and produces dK/dV.
// Nothing is accumulated across CTAs, so there are no atomics and results are deterministic,
// as in the reference. Both tensor-core kernels are one template:
//
//   resident tiles R1,R2 (128 rows)   streamed tiles C1,C2 (64 rows per step)
//   dK/dV kernel:  K, V               Q, dO      rows of the score tile = keys
//   dQ    kernel:  Q, dO              K, V       rows of the score tile = queries
//
//   X1 = R1 C1^T  (S or S^T)          X2 = R2 C2^T  (dP or dP^T)    128 x 64 each, fp32 in TMEM
//   p  = exp2(X1 * scale * log2e - lse[query] * log2e)
//   ds = p * (X2 * dropmask/(1-rate) - delta[query]) * scale
//   dK/dV kernel:  dV += (p*dropmask/(1-rate))^T-tile . C2,  dK += ds-tile . C1
//   dQ    kernel:  dQ += ds-tile . C1
//
// p and ds are written by the compute warps as bf16 into shared memory in the 128-byte
// swizzled K-major layout and consumed as the A operand; the streamed tiles serve as the
// MN-major B operand of the accumulating MMAs, straight from where TMA put them.
//   warp 0      TMA producer          warp 1      MMA issuer + TMEM owner
//   warps 2-9   compute: two warps per TMEM lane quadrant, each taking 32 of the 64 columns
//
// Streaming 64 rows at a time keeps a CTA at 256 TMEM columns and ~100 KB of shared memory at
// D = 64, so two CTAs share an SM and one CTA's MMAs run under the other's exponentials. At
// D = 128 (one CTA per SM) the score tiles are double-buffered in TMEM instead and the streamed
// tiles get a third stage, so the score GEMMs of step i+2 are issued while step i is computed.
#include <cuda_bf16.h>

#include <cfloat>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace dadattn {
namespace {

using namespace ptx;

constexpr int kTileRows = 128;            // rows owned by a CTA (keys or queries)
constexpr int kSubRows = 64;              // rows of a streamed tile
constexpr int kPanelBytes = 128 * 128;    // [128 rows][64 bf16] swizzled panel
constexpr int kSubPanelBytes = 64 * 128;  // [64 rows][64 bf16] swizzled panel
constexpr int kBwdThreads = 320;
constexpr int kComputeThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

template <int D, bool KV>
struct BwdSmem {
  static constexpr int kPanels = D / 64;
  static constexpr int kXBufs = D == 64 ? 1 : 2;           // score-tile buffers in TMEM
  static constexpr int kStages = 3;                        // streamed-tile ring depth
  static constexpr int kTile = kPanels * kPanelBytes;      // resident [128, D] tile
  static constexpr int kSub = kPanels * kSubPanelBytes;    // streamed [64, D] tile
  static constexpr int kR1 = 0;
  static constexpr int kR2 = kR1 + kTile;
  static constexpr int kC1 = kR2 + kTile;
  static constexpr int kC2 = kC1 + kStages * kSub;
  static constexpr int kDS = kC2 + kStages * kSub;         // [128][64] bf16, one panel
  static constexpr int kP = kDS + kPanelBytes;             // only the dK/dV kernel has a p tile
  static constexpr int kVec = kP + (KV ? kPanelBytes : 0); // lse*log2e, delta: [2][64] fp32
  static constexpr int kBars = kVec + 2 * 64 * 4;
  // At D = 64 two CTAs must fit one SM: 2 x (kBytes + 1 KB reserved) <= 228 KB.
  static constexpr int kBytes = kBars + 192;
  static_assert(D != 64 || 2 * (kBytes + 1024) <= 233472, "two CTAs per SM no longer fit");
};

struct BwdBars {
  uint64_t r_full, c1_full[3], c2_full[3], c_empty[3];
  uint64_t x_full[2], x_free[2], w_full, acc_done, vec_full;
  uint32_t tmem_base;
  int abort_flag;
};

// KV = true: dK/dV kernel (grid.x = key tile). KV = false: dQ kernel (grid.x = query tile).
template <int D, bool KV, bool DROP>
__global__ void __launch_bounds__(kBwdThreads, D == 64 ? 2 : 1)
flash_bwd_bf16_kernel(const __grid_constant__ CUtensorMap map_r1,
                      const __grid_constant__ CUtensorMap map_r2,
                      const __grid_constant__ CUtensorMap map_c1,
                      const __grid_constant__ CUtensorMap map_c2,
                      __nv_bfloat16* __restrict__ out1, __nv_bfloat16* __restrict__ out2,
                      const float* __restrict__ lse, float* __restrict__ delta,
                      const __nv_bfloat16* __restrict__ g_out, const __nv_bfloat16* __restrict__ g_dout,
                      int S, float scale, float rate, PhiloxKey rng, int64_t unit0,
                      int* __restrict__ status) {
  using L = BwdSmem<D, KV>;
  constexpr int kPanels = L::kPanels;
  constexpr int kStages = L::kStages;
  constexpr int kXBufs = L::kXBufs;
  // TMEM: per score buffer X1 [0,64) X2 [64,128); accumulators after the score buffers.
  constexpr uint32_t kTmemCols = D == 64 ? 256 : 512;
  constexpr uint32_t kColA1 = 128 * kXBufs, kColA2 = kColA1 + D;

  extern __shared__ __align__(1024) uint8_t smem[];
  BwdBars* bars = reinterpret_cast<BwdBars*>(smem + L::kBars);
  volatile int* abort_flag = &bars->abort_flag;
  float* vec = reinterpret_cast<float*>(smem + L::kVec);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n_tiles = (S + kTileRows - 1) / kTileRows;
  const int n_sub = (S + kSubRows - 1) / kSubRows;
  const int bh = blockIdx.y;
  // dK/dV: key tile `own` streams the query sub-tiles 2*own .. n_sub-1 (low `own` = most work =
  // scheduled first). dQ: query tile `own` streams the key sub-tiles 0 .. min(2*own+1, n_sub-1).
  const int own = KV ? static_cast<int>(blockIdx.x) : n_tiles - 1 - static_cast<int>(blockIdx.x);
  const int first = KV ? 2 * own : 0;
  const int n_it = KV ? n_sub - 2 * own : min(2 * own + 2, n_sub);
  const int row0 = own * kTileRows;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(status, DADATTN_E_CUDA);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->r_full, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(&bars->c1_full[s], 1);
      mbar_init(&bars->c2_full[s], 1);
      mbar_init(&bars->c_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->x_full[b], 1);
      mbar_init(&bars->x_free[b], kComputeThreads);
    }
    mbar_init(&bars->w_full, kComputeThreads);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->vec_full, kComputeThreads);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  // Set-up is done; from here on global memory is read, which the previous grid in the stream
  // may have produced. Once every CTA of this grid is here the next grid may start its set-up.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      prefetch_tensormap(&map_r1);
      prefetch_tensormap(&map_r2);
      prefetch_tensormap(&map_c1);
      prefetch_tensormap(&map_c2);
      mbar_arrive_expect_tx(&bars->r_full, 2 * L::kTile);
      for (int p = 0; p < kPanels; ++p) {
        tma_load_3d(smem + L::kR1 + p * kPanelBytes, &map_r1, &bars->r_full, p * 64, row0, bh);
        tma_load_3d(smem + L::kR2 + p * kPanelBytes, &map_r2, &bars->r_full, p * 64, row0, bh);
      }
      for (int i = 0; i < n_it; ++i) {
        const int s = i % kStages, use = i / kStages;
        if (use > 0 && !mbar_wait(&bars->c_empty[s], (use - 1) & 1, abort_flag)) break;
        const int c_row0 = (first + i) * kSubRows;
        mbar_arrive_expect_tx(&bars->c1_full[s], L::kSub);
        for (int p = 0; p < kPanels; ++p)
          tma_load_3d(smem + L::kC1 + s * L::kSub + p * kSubPanelBytes, &map_c1,
                      &bars->c1_full[s], p * 64, c_row0, bh);
        mbar_arrive_expect_tx(&bars->c2_full[s], L::kSub);
        for (int p = 0; p < kPanels; ++p)
          tma_load_3d(smem + L::kC2 + s * L::kSub + p * kSubPanelBytes, &map_c2,
                      &bars->c2_full[s], p * 64, c_row0, bh);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_x = make_idesc_bf16(128, 64, 0, 0);  // both operands K-major
      constexpr uint32_t idesc_a = make_idesc_bf16(128, D, 0, 1);   // B = streamed tile, MN-major
      const SmemDescBase r1 = make_desc_base_sw128(smem_u32(smem + L::kR1), 0);
      const SmemDescBase r2 = make_desc_base_sw128(smem_u32(smem + L::kR2), 0);
      const SmemDescBase p_desc = make_desc_base_sw128(smem_u32(smem + L::kP), 0);
      const SmemDescBase ds_desc = make_desc_base_sw128(smem_u32(smem + L::kDS), 0);
      const SmemDescBase c1_desc0 = make_desc_base_sw128(smem_u32(smem + L::kC1), kSubPanelBytes);
      const SmemDescBase c2_desc0 = make_desc_base_sw128(smem_u32(smem + L::kC2), kSubPanelBytes);
      bool ok = mbar_wait(&bars->r_full, 0, abort_flag);

      // X1 = R1 C1^T, X2 = R2 C2^T for step i into score buffer i % kXBufs (the caller has made
      // sure that buffer is free)
      auto issue_x = [&](int i) -> bool {
        const int s = i % kStages, xb = i % kXBufs;
        const uint32_t par = (i / kStages) & 1;
        const SmemDescBase c1{c1_desc0.lo + s * (L::kSub >> 4), c1_desc0.hi};
        const SmemDescBase c2{c2_desc0.lo + s * (L::kSub >> 4), c2_desc0.hi};
        if (!mbar_wait(&bars->c1_full[s], par, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          mma_ss(tmem + xb * 128, desc_at(r1, (kk / 4) * kPanelBytes + (kk % 4) * 32),
                 desc_at(c1, (kk / 4) * kSubPanelBytes + (kk % 4) * 32), idesc_x,
                 kk > 0 ? 1u : 0u);
        }
        if (!mbar_wait(&bars->c2_full[s], par, abort_flag)) return false;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          mma_ss(tmem + xb * 128 + 64, desc_at(r2, (kk / 4) * kPanelBytes + (kk % 4) * 32),
                 desc_at(c2, (kk / 4) * kSubPanelBytes + (kk % 4) * 32), idesc_x,
                 kk > 0 ? 1u : 0u);
        }
        mma_commit(&bars->x_full[xb]);
        return true;
      };
      // accumulators += (p | ds tiles of step i) . streamed tiles of step i (K = 64 rows)
      auto issue_acc = [&](int i) -> bool {
        const int s = i % kStages;
        const SmemDescBase c1{c1_desc0.lo + s * (L::kSub >> 4), c1_desc0.hi};
        const SmemDescBase c2{c2_desc0.lo + s * (L::kSub >> 4), c2_desc0.hi};
        if (!mbar_wait(&bars->w_full, i & 1, abort_flag)) return false;
        tc_fence_after_sync();
        // One MMA per 16 streamed rows covers all D output columns: the streamed tile is
        // MN-major and its 64-column panels are kSubPanelBytes apart (the descriptor's LBO).
#pragma unroll
        for (int kk = 0; kk < kSubRows / 16; ++kk) {
          const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
          if (KV) mma_ss(tmem + kColA1, desc_at(p_desc, kk * 32), desc_at(c2, kk * 2048), idesc_a, acc);
          mma_ss(tmem + (KV ? kColA2 : kColA1), desc_at(ds_desc, kk * 32), desc_at(c1, kk * 2048),
                 idesc_a, acc);
        }
        mma_commit(&bars->c_empty[s]);
        mma_commit(&bars->acc_done);
        return true;
      };

      // Score GEMMs run kXBufs steps ahead of the accumulating GEMMs: step i + kXBufs is issued
      // as soon as the compute warps have pulled step i's scores out of its buffer.
      for (int i = 0; ok && i < kXBufs && i < n_it; ++i) ok = issue_x(i);
      for (int i = 0; ok && i < n_it; ++i) {
        if (i + kXBufs < n_it)
          ok = mbar_wait(&bars->x_free[i % kXBufs], (i / kXBufs) & 1, abort_flag) &&
               issue_x(i + kXBufs);
        ok = ok && issue_acc(i);
      }
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    const int cw = warp - 2;              // 0..7
    const int quad = warp % 4;            // TMEM lane quadrant of this warp
    const int half = cw / 4;              // which 32 columns of the 64
    const int ct = cw * 32 + lane;        // 0..255 among the compute threads
    const int row = quad * 32 + lane;     // row of the score tile = TMEM lane
    const int grow = row0 + row;          // key (KV) or query (dQ) index of this row
    const uint32_t tlane = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float scale_log2 = scale * kLog2e;
    const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;
    const size_t vec_base = static_cast<size_t>(bh) * S;
    uint8_t* p_row = smem + L::kP + row * 128;
    uint8_t* ds_row = smem + L::kDS + row * 128;
    float row_lse2 = 0.f, row_delta = 0.f;
    if (!KV) {  // per-row scalars; rows beyond S contribute nothing (p = exp2(-inf) = 0)
      row_lse2 = grow < S ? lse[vec_base + grow] * kLog2e : INFINITY;
      // delta[r] = sum_d dO[r,d] * O[r,d] (the reference's flash_delta_kernel,
      // cuda/attention.cu:76-85) is formed here, by the threads that own row r, and left in
      // `delta` for the dK/dV kernel, which is launched after this one.
      if (grow < S) {
        const uint4* po = reinterpret_cast<const uint4*>(g_out + (vec_base + grow) * D);
        const uint4* pd = reinterpret_cast<const uint4*>(g_dout + (vec_base + grow) * D);
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
          const uint4 a = po[c], b2 = pd[c];
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b2.x, b2.y, b2.z, b2.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            s4[i] = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), s4[i]);
            s4[i] = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), s4[i]);
          }
        }
        row_delta = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        if (half == 0) delta[vec_base + grow] = row_delta;
      }
    }
    bool ok = true;

    for (int i = 0; i < n_it; ++i) {
      const int col0 = (first + i) * kSubRows;  // first query (KV) / key (dQ) of the streamed tile
      // sub-tiles that straddle the diagonal need the causal comparison
      const bool diagonal = KV ? (i < 2) : (first + i >= 2 * own);
      const int xb = i % kXBufs;
      float* v_lse = vec;
      float* v_delta = vec + 64;
      if (KV) {  // per-column vectors of this query sub-tile (one buffer)
        // w_full(i-1) complete = every compute thread is done with step i-1, reads of the
        // vectors included, so they may be overwritten
        if (i > 0 && !(ok = mbar_wait(&bars->w_full, (i - 1) & 1, abort_flag))) break;
        if (ct < 128) {
          const int q = col0 + (ct & 63);
          if (ct < 64) v_lse[ct] = q < S ? lse[vec_base + q] * kLog2e : INFINITY;
          else v_delta[ct - 64] = q < S ? delta[vec_base + q] : 0.f;
        }
        // an mbarrier rather than a named barrier: its wait is bounded like every other one
        mbar_arrive(&bars->vec_full);
        if (!(ok = mbar_wait(&bars->vec_full, i & 1, abort_flag))) break;
      }
      if (!(ok = mbar_wait(&bars->x_full[xb], (i / kXBufs) & 1, abort_flag))) break;
      tc_fence_after_sync();

      const int cbase = half * 32;  // this thread's columns within the 64
      uint32_t x1[32], x2[32];
      tmem_ld32(tlane + xb * 128 + cbase, x1);
      tmem_ld32(tlane + xb * 128 + 64 + cbase, x2);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&bars->x_free[xb]);  // scores are in registers: the buffer may be overwritten

      uint32_t pw[16], dw[16];
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        float l2[4], dl[4];
        if (KV) {  // 128-bit broadcast reads: all lanes of a warp want the same four columns
          const float4 a = *reinterpret_cast<const float4*>(v_lse + cbase + c);
          const float4 b = *reinterpret_cast<const float4*>(v_delta + cbase + c);
          l2[0] = a.x; l2[1] = a.y; l2[2] = a.z; l2[3] = a.w;
          dl[0] = b.x; dl[1] = b.y; dl[2] = b.z; dl[3] = b.w;
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            l2[e] = row_lse2;
            dl[e] = row_delta;
          }
        }
        float pv[4], dv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int gcol = col0 + cbase + c + e;
          const int key = KV ? grow : gcol, query = KV ? gcol : grow;
          float p = ex2(fmaf(__uint_as_float(x1[c + e]), scale_log2, -l2[e]));
          if (diagonal && key > query) p = 0.f;
          float g = __uint_as_float(x2[c + e]);
          float pd = p;
          if (DROP) {
            const uint64_t idx = (static_cast<uint64_t>(unit0 + bh) * S + query) * S + key;
            const float mk = (p != 0.f && philox_keep(rng, idx, rate)) ? keep_scale : 0.f;
            pd = p * mk;
            g *= mk;
          }
          pv[e] = pd;
          dv[e] = p * (g - dl[e]) * scale;
        }
        pw[c / 2] = pack_bf16(pv[0], pv[1]);
        pw[c / 2 + 1] = pack_bf16(pv[2], pv[3]);
        dw[c / 2] = pack_bf16(dv[0], dv[1]);
        dw[c / 2 + 1] = pack_bf16(dv[2], dv[3]);
      }
      // the previous step's p / ds tiles must have been consumed before they are overwritten
      if (i > 0 && !(ok = mbar_wait(&bars->acc_done, (i - 1) & 1, abort_flag))) break;
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        const int chunk = half * 4 + v4;  // 16-byte chunk within the 128-byte row
        const int off = (chunk ^ (row & 7)) << 4;
        if (KV)
          *reinterpret_cast<uint4*>(p_row + off) =
              make_uint4(pw[4 * v4], pw[4 * v4 + 1], pw[4 * v4 + 2], pw[4 * v4 + 3]);
        *reinterpret_cast<uint4*>(ds_row + off) =
            make_uint4(dw[4 * v4], dw[4 * v4 + 1], dw[4 * v4 + 2], dw[4 * v4 + 3]);
      }
      fence_proxy_async_smem();
      mbar_arrive(&bars->w_full);
    }

    // Epilogue. dK/dV kernel: half 0 stores dV, half 1 stores dK. dQ kernel: halves split D.
    if (ok && (ok = mbar_wait(&bars->acc_done, (n_it - 1) & 1, abort_flag))) {
      tc_fence_after_sync();
      constexpr int kCols = KV ? D : D / 2;
      const uint32_t col_base = KV ? (half == 0 ? kColA1 : kColA2) : kColA1 + half * (D / 2);
      __nv_bfloat16* dst = (KV ? (half == 0 ? out1 : out2) : out1) +
                           (static_cast<size_t>(bh) * S + grow) * D + (KV ? 0 : half * (D / 2));
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tlane + col_base + c * 32, o);
        tmem_wait_ld();
        if (grow < S) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(
                pack_bf16(__uint_as_float(o[8 * i + 0]), __uint_as_float(o[8 * i + 1])),
                pack_bf16(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3])),
                pack_bf16(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5])),
                pack_bf16(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7])));
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) report_timeout(status, bars->abort_flag);
}

template <int D, bool DROP>
int launch_bwd_bf16(uint16_t* dq, uint16_t* dk, uint16_t* dv, float* delta, const uint16_t* dout,
                    const uint16_t* out, const float* lse, const uint16_t* q, const uint16_t* k,
                    const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                    uint64_t offset, int64_t unit0, cudaStream_t st) {
  // resident tiles are loaded with 128-row boxes, streamed tiles with 64-row boxes
  CUtensorMap mq, mk, mv, mdo, mq_s, mk_s, mv_s, mdo_s;
  if (int rc = make_tensor_map_bf16(&mq, q, BH, S, D, kTileRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mk, k, BH, S, D, kTileRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mv, v, BH, S, D, kTileRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mdo, dout, BH, S, D, kTileRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mq_s, q, BH, S, D, kSubRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mk_s, k, BH, S, D, kSubRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mv_s, v, BH, S, D, kSubRows)) return rc;
  if (int rc = make_tensor_map_bf16(&mdo_s, dout, BH, S, D, kSubRows)) return rc;
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  using BF = __nv_bfloat16;

  const PhiloxKey rng = make_philox(seed, offset);
  dim3 grid((S + kTileRows - 1) / kTileRows, BH);

  // dQ first: it also produces delta [BH,S], which the dK/dV kernel then reads.
  stage_event(0, st);
  auto kq = flash_bwd_bf16_kernel<D, false, DROP>;
  DAD_CUDA(cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                BwdSmem<D, false>::kBytes));
  DAD_CUDA(launch_pdl(kq, grid, dim3(kBwdThreads), BwdSmem<D, false>::kBytes, st, mq, mdo, mk_s, mv_s,
                      reinterpret_cast<BF*>(dq), static_cast<BF*>(nullptr), lse, delta,
                      reinterpret_cast<const BF*>(out), reinterpret_cast<const BF*>(dout), S, scale,
                      rate, rng, unit0, status));
  stage_event(1, st);

  auto kkv = flash_bwd_bf16_kernel<D, true, DROP>;
  DAD_CUDA(cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                BwdSmem<D, true>::kBytes));
  DAD_CUDA(launch_pdl(kkv, grid, dim3(kBwdThreads), BwdSmem<D, true>::kBytes, st, mk, mv, mq_s, mdo_s,
                      reinterpret_cast<BF*>(dv), reinterpret_cast<BF*>(dk), lse, delta,
                      static_cast<const BF*>(nullptr), static_cast<const BF*>(nullptr), S, scale,
                      rate, rng, unit0, status));
  stage_event(2, st);
  return DADATTN_OK;
}

}  // namespace

// flash_bwd_fused_sm100.cu
size_t fused_bwd_workspace_bytes(int BH, int S);
int launch_bwd_fused_d64(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace, const uint16_t* dout,
                         const uint16_t* out, const float* lse, const uint16_t* q, const uint16_t* k,
                         const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                         uint64_t offset, int64_t unit0, const uint32_t* mask_bits, int heads, cudaStream_t st);

thread_local cudaEvent_t* g_stage_events = nullptr;
thread_local int g_stage_event_count = 0;

// flash_bwd_fused128_sm100.cu
size_t fused128_bwd_workspace_bytes(int BH, int S);
int launch_bwd_fused_d128(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace, const uint16_t* dout,
                          const uint16_t* out, const float* lse, const uint16_t* q, const uint16_t* k,
                          const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                          uint64_t offset, int64_t unit0, cudaStream_t st);

namespace {
thread_local int g_deterministic = 0;
}
}  // namespace dadattn

using namespace dadattn;


extern "C" int dadattn_set_bwd_deterministic(int on) {
  g_deterministic = on ? 1 : 0;
  return DADATTN_OK;
}

extern "C" int dadattn_set_stage_events(void** events, int count) {
  g_stage_events = reinterpret_cast<cudaEvent_t*>(events);
  g_stage_event_count = events ? count : 0;
  return DADATTN_OK;
}

extern "C" size_t dadattn_flash_bwd_bf16_workspace_bytes(int BH, int S, int D) {
  if (BH <= 0 || S <= 0 || D <= 0) return 0;
  // delta [BH,S]; at D = 64 also the fp32 dQ accumulator of the single-pass kernel
  if (D == 64) return fused_bwd_workspace_bytes(BH, S);
  if (D == 128) return fused128_bwd_workspace_bytes(BH, S);
  return static_cast<size_t>(BH) * S * sizeof(float);
}

static int flash_bwd_bf16_checked(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                                  size_t workspace_bytes, const uint16_t* dout, const uint16_t* out,
                                  const float* lse, const uint16_t* q, const uint16_t* k,
                                  const uint16_t* v, int BH, int S, int D, float scale, float rate,
                                  uint64_t seed, uint64_t offset, int64_t unit0,
                                  const uint32_t* mask_bits, int heads, dadattn_stream_t stream) {
  if (!dq || !dk || !dv || !workspace || !dout || !out || !lse || !q || !k || !v)
    return fail(DADATTN_E_ARG, "null tensor pointer");
  if (BH <= 0 || S <= 0) return fail(DADATTN_E_ARG, "BH=%d and S=%d must be positive", BH, S);
  if (BH > 65535) return fail(DADATTN_E_UNSUPPORTED, "BH=%d exceeds 65535 per call", BH);
  if (!dadattn_flash_bf16_supported(D))
    return fail(DADATTN_E_UNSUPPORTED, "flash attention bf16: unsupported d_head %d", D);
  if (!(rate >= 0.0f && rate < 1.0f))
    return fail(DADATTN_E_ARG, "dropout rate %f outside [0,1)", static_cast<double>(rate));
  for (const void* p : {static_cast<const void*>(dq), static_cast<const void*>(dk),
                        static_cast<const void*>(dv), static_cast<const void*>(dout),
                        static_cast<const void*>(out), static_cast<const void*>(q),
                        static_cast<const void*>(k), static_cast<const void*>(v),
                        static_cast<const void*>(workspace)})
    if (!aligned(p, 16)) return fail(DADATTN_E_ARG, "bf16 tensors and workspace must be 16-byte aligned");
  if (workspace_bytes < dadattn_flash_bwd_bf16_workspace_bytes(BH, S, D))
    return fail(DADATTN_E_WORKSPACE, "backward workspace %zu < %zu bytes", workspace_bytes,
                dadattn_flash_bwd_bf16_workspace_bytes(BH, S, D));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* delta = static_cast<float*>(workspace);
  const bool drop = rate > 0.f;
  if (D == 64 && !g_deterministic) {
    if (!aligned(workspace, 256)) return fail(DADATTN_E_ARG, "backward workspace must be 256-byte aligned");
    return launch_bwd_fused_d64(dq, dk, dv, workspace, dout, out, lse, q, k, v, BH, S, scale, rate,
                                seed, offset, unit0, mask_bits, heads, st);
  }
  if (mask_bits)
    return fail(DADATTN_E_UNSUPPORTED,
                "a bit-packed dropout mask is taken by the single-pass head-size-64 backward only");
  if (heads > 0)
    return fail(DADATTN_E_UNSUPPORTED,
                "interleaved [B*S, H*D] activations are taken by the single-pass head-size-64 backward only");
  if (D == 128 && !g_deterministic) {
    if (!aligned(workspace, 256)) return fail(DADATTN_E_ARG, "backward workspace must be 256-byte aligned");
    return launch_bwd_fused_d128(dq, dk, dv, workspace, dout, out, lse, q, k, v, BH, S, scale, rate,
                                 seed, offset, unit0, st);
  }
#define DAD_BWD16(DH)                                                                            \
  return drop ? launch_bwd_bf16<DH, true>(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S,     \
                                          scale, rate, seed, offset, unit0, st)                  \
              : launch_bwd_bf16<DH, false>(dq, dk, dv, delta, dout, out, lse, q, k, v, BH, S,    \
                                           scale, 0.f, 0, 0, 0, st);
  if (D == 64) {
    DAD_BWD16(64)
  }
  DAD_BWD16(128)
#undef DAD_BWD16
}

extern "C" int dadattn_flash_bwd_bf16(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                                      size_t workspace_bytes, const uint16_t* dout,
                                      const uint16_t* out, const float* lse, const uint16_t* q,
                                      const uint16_t* k, const uint16_t* v, int BH, int S, int D,
                                      float scale, float rate, uint64_t seed, uint64_t offset,
                                      int64_t unit0, dadattn_stream_t stream) {
  return flash_bwd_bf16_checked(dq, dk, dv, workspace, workspace_bytes, dout, out, lse, q, k, v, BH, S, D,
                                scale, rate, seed, offset, unit0, nullptr, 0, stream);
}

extern "C" int dadattn_flash_bwd_bf16_masked(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                                             size_t workspace_bytes, const uint16_t* dout,
                                             const uint16_t* out, const float* lse, const uint16_t* q,
                                             const uint16_t* k, const uint16_t* v, int BH, int S, int D,
                                             float scale, float rate, const uint32_t* mask_bits,
                                             dadattn_stream_t stream) {
  if (!mask_bits || !aligned(mask_bits, 16))
    return fail(DADATTN_E_ARG, "mask_bits must be a 16-byte aligned device pointer");
  if (!(rate > 0.0f)) return fail(DADATTN_E_ARG, "the masked backward needs the rate the mask was drawn with (> 0)");
  return flash_bwd_bf16_checked(dq, dk, dv, workspace, workspace_bytes, dout, out, lse, q, k, v, BH, S, D,
                                scale, rate, 0, 0, 0, mask_bits, 0, stream);
}

extern "C" int dadattn_flash_bwd_bf16_strided(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                                              size_t workspace_bytes, const uint16_t* dout,
                                              const uint16_t* out, const float* lse, const uint16_t* q,
                                              const uint16_t* k, const uint16_t* v, int B, int H, int S, int D,
                                              float scale, float rate, uint64_t seed, uint64_t offset,
                                              int64_t unit0, dadattn_stream_t stream) {
  if (B <= 0 || H <= 0) return fail(DADATTN_E_ARG, "B=%d and H=%d must be positive", B, H);
  if (static_cast<long long>(B) * H > 65535)
    return fail(DADATTN_E_UNSUPPORTED, "B*H=%lld exceeds 65535 per call", static_cast<long long>(B) * H);
  if (D != 64)
    return fail(DADATTN_E_UNSUPPORTED, "interleaved [B*S, H*D] activations are taken at head size 64 only (got %d)", D);
  return flash_bwd_bf16_checked(dq, dk, dv, workspace, workspace_bytes, dout, out, lse, q, k, v, B * H, S, D,
                                scale, rate, seed, offset, unit0, nullptr, H, stream);
}
