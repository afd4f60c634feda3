// bf16 fused causal attention forward for sm_100a, head size 64: a persistent kernel, one CTA
// per SM, that works on TWO 128-row query tiles of one (batch, head) at a time.
//
// The arithmetic is that of the reference's flash_fwd_kernel (cuda/attention.cu:17-73: online
// softmax over key tiles, lse = max + ln(sum) of the scaled scores) with bf16 operands and fp32
// accumulation. What differs is the shape of the work. At head size 64 a 128x128 score tile
// costs 640 clocks of tensor pipe but 1024 clocks of the exp2 unit and, written naively, more
// than 1200 issue slots per scheduler: the softmax, not the MMAs, is what has to be fed. So:
//   * a work item is a PAIR of adjacent query tiles (A = tile 2p, B = tile 2p + 1) of one
//     (batch, head); both use the same K/V tiles from one shared-memory ring and each has its
//     own softmax group. While group A computes exponentials the tensor pipe runs B's products
//     and vice versa;
//   * a K/V tile is worked through in two sub-steps of 64 keys, and every group has TWO score
//     buffers of 64 columns in tensor memory: while the group's threads work on the scores of
//     one sub-step, the product for the next one is already running into the other buffer, so in
//     steady state nobody waits for the tensor pipe and the tensor pipe waits for nobody;
//   * a group is 256 threads, TWO per query row: one takes key columns 0-31 of every sub-step,
//     the other columns 32-63. Each keeps its OWN running max / sum and its OWN output
//     accumulator in tensor memory (split-K inside the CTA), so the two threads of a row never
//     talk inside the loop; they are merged once per item, in the epilogue. Sixteen softmax
//     warps, four per scheduler, are what hides the tensor-memory and exp2 latencies;
//   * the probabilities never touch shared memory: a thread reads its 32 scores from tensor
//     memory once, keeps them in registers for the max and the exponentials, and writes P back
//     as packed bf16 over the first half of the same columns, from where the P V product takes
//     it as its A operand;
//   * scale-and-subtract and the row sums run as packed two-float instructions (fma.rn.f32x2,
//     add.rn.f32x2), the row max as three-input max, and one pair of exponentials in four as a
//     cubic on the FMA pipe (a bf16x2 exp2 on the special-function unit was tried: no faster, and
//     it cost a digit of lse): the softmax is bound by instruction issue, not by any one unit;
//   * CTAs are persistent: barriers, tensor memory and descriptors are set up once, items are
//     dealt out heaviest first in a fixed serpentine order (no global counter to reset), the
//     next item's Q tiles and first K/V tiles are in flight while the current one finishes, and
//     its first score products are issued before the current item's epilogue.
//
//   warp 0        TMA producer (Q pair double-buffered, K/V through a 4-stage ring)
//   warp 1        MMA issuer of group A, owner of the tensor-memory allocation
//   warp 18       MMA issuer of group B (one issuing thread per group: a group's products are
//                 issued the moment its probabilities are ready, whatever the other group does)
//   warps 2-9     softmax group A (2-5: key columns 0-31 of a sub-step, 6-9: 32-63)
//   warps 10-17   softmax group B likewise
// Tensor memory: score buffer b of group X at 128 X + 64 b; O of (group X, half h) at
// 256 + 64 (2 X + h); P of half h aliases the first 16 columns of its 32 columns of the buffer.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh); on expiry the CTA raises its abort flag, all
// roles fall through to the common exit, tensor memory is freed and DADATTN_E_TIMEOUT is left in
// the device status word. No cluster launch, no multicast: each CTA loads its own tiles.
#include <cuda_bf16.h>

#include <cfloat>
#include <vector>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace dadattn {
namespace {

using namespace ptx;

constexpr int kT = 128;               // tile edge: query rows per group, keys per K/V tile
constexpr int kHD = 64;               // head size
constexpr int kPanel = 128 * 128;     // [128 rows][64 bf16]: 16 KB, 128-byte rows, swizzled
constexpr int kKvStages = 4;
constexpr int kFwd64Threads = 19 * 32;
constexpr int kHalfThreads = 128;     // threads of one half of a softmax group
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleAt = 8.0f;    // log2 units: O is rescaled only when the max grew by 2^8

struct F64Smem {
  static constexpr int kQ = 0;                                // [2 items][A, B] panels
  static constexpr int kK = kQ + 4 * kPanel;
  static constexpr int kV = kK + kKvStages * kPanel;
  static constexpr int kStat = kV + kKvStages * kPanel;      // float2 [group][half][128]: (max, sum)
  static constexpr int kBars = kStat + 2 * 2 * 128 * 8;
  static constexpr int kBytes = kBars + 512;
};

struct F64Bars {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[kKvStages], v_full[kKvStages], kv_empty[kKvStages];
  uint64_t s_full[2][2], p_full[2][2], o_done[2][2], o_free[2], stat_full[2];   // [group][buffer]
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(F64Bars) <= 512, "barrier block");

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(taddr)
      : "memory");
}

// ---- work items --------------------------------------------------------------------------------
// Item e (0 = heaviest): query-tile pair p = n_pairs - 1 - e / BH of (batch, head) e % BH.
// Which items a CTA takes, in order, is fixed before the launch; every role computes the same
// list, nothing is shared or reset. For small launches the host deals the weight-sorted list out
// greedily (each item to the CTA with the least work so far) and passes the result as a kernel
// parameter: entry k * G + c is the k-th item of CTA c. With only a handful of items per CTA the
// closed-form deal below can leave some CTAs two K/V steps (of about 26) behind the others.
// Larger launches use the closed form: CTA c of G takes the items k * G + (k even ? c : G-1-c), a
// serpentine deal, so that a CTA that got an early (heavy) item in one row gets a late (light)
// one in the next.
constexpr int kDealEntries = 1536;
constexpr uint16_t kDealNone = 0xffffu;
struct F64Deal {
  int rows;                      // 0: closed-form deal
  uint16_t item[kDealEntries];
};
struct F64Item {
  int bh, qa, n_a, n_b, n_kv;   // n_b = 0 when the pair's second tile lies beyond the sequence
  bool valid;
};
__device__ __forceinline__ F64Item f64_item(const F64Deal& deal, int k, int BH, int n_tiles, int n_items) {
  const int G = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  int e;
  if (deal.rows > 0) {
    const uint16_t t = k < deal.rows ? deal.item[k * G + c] : kDealNone;
    e = t == kDealNone ? n_items : t;
  } else {
    e = k * G + ((k & 1) ? (G - 1 - c) : c);
  }
  F64Item it;
  it.valid = e < n_items;
  const int row = e / BH;
  const int n_pairs = (n_tiles + 1) / 2;
  it.bh = e - row * BH;
  it.qa = 2 * (n_pairs - 1 - row);
  it.n_a = it.qa + 1;
  it.n_b = (it.qa + 1 < n_tiles) ? it.qa + 2 : 0;
  it.n_kv = it.n_b ? it.n_b : it.n_a;
  return it;
}

// DROP: 0 = no dropout, 1 = Philox drawn in the kernel, 2 = keep bits read from `mask_bits`.
template <int DROP>
__global__ void __launch_bounds__(kFwd64Threads, 1)
flash_fwd64_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ lse, int BH, int S, UnitLayout lay, float scale, float rate,
                   PhiloxKey rng, int64_t unit0, const uint4* __restrict__ mask_bits,
                   int* __restrict__ status, const __grid_constant__ F64Deal deal) {
  using L = F64Smem;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColO = 256;   // score buffer (X,b) at 128 X + 64 b, O_(X,h) at kColO + 64 (2 X + h)

  extern __shared__ __align__(1024) uint8_t smem[];
  F64Bars* bars = reinterpret_cast<F64Bars*>(smem + L::kBars);
  volatile int* abort_flag = &bars->abort_flag;

  // the warp index through a shuffle, so that the compiler knows it is uniform across the warp
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x / 32), 0);
  const int lane = threadIdx.x % 32;
  const int n_tiles = (S + kT - 1) / kT;
  const int n_items = BH * ((n_tiles + 1) / 2);

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled layouts need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(status, DADATTN_E_CUDA);
    return;
  }
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->q_full[b], 1);
      mbar_init(&bars->q_empty[b], 2);              // one arrival per issuer
      for (int i = 0; i < 2; ++i) {
        mbar_init(&bars->s_full[b][i], 1);
        mbar_init(&bars->p_full[b][i], 2 * kHalfThreads);
      }
      mbar_init(&bars->o_done[b][0], 1);
      mbar_init(&bars->o_done[b][1], 1);
      mbar_init(&bars->o_free[b], 2 * kHalfThreads);
      mbar_init(&bars->stat_full[b], 2 * kHalfThreads);
    }
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->kv_empty[s], 2);             // one arrival per issuer
    }
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
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      int g = 0;  // K/V tiles loaded so far, over all items
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const F64Item it = f64_item(deal, k, BH, n_tiles, n_items);
        if (!it.valid) break;
        const int qb = k & 1;
        // the Q buffer frees when the last score product of the item before last has completed
        if (k >= 2 && !mbar_wait(&bars->q_empty[qb], ((k >> 1) - 1) & 1, abort_flag)) break;
        const int ub = it.bh / lay.heads, uh = it.bh - ub * lay.heads;   // (batch, head) of the unit
        mbar_arrive_expect_tx(&bars->q_full[qb], it.n_b ? 2 * kPanel : kPanel);
        tma_load_4d(smem + L::kQ + (qb * 2 + 0) * kPanel, &map_q, &bars->q_full[qb], 0, it.qa * kT, uh, ub);
        if (it.n_b)
          tma_load_4d(smem + L::kQ + (qb * 2 + 1) * kPanel, &map_q, &bars->q_full[qb], 0,
                      (it.qa + 1) * kT, uh, ub);
        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const int s = g % kKvStages, use = g / kKvStages;
          if (use > 0 && !(ok = mbar_wait(&bars->kv_empty[s], (use - 1) & 1, abort_flag))) break;
          mbar_arrive_expect_tx(&bars->k_full[s], kPanel);
          tma_load_4d(smem + L::kK + s * kPanel, &map_k, &bars->k_full[s], 0, j * kT, uh, ub);
          mbar_arrive_expect_tx(&bars->v_full[s], kPanel);
          tma_load_4d(smem + L::kV + s * kPanel, &map_v, &bars->v_full[s], 0, j * kT, uh, ub);
        }
      }
    }
  } else if (warp == 1 || warp == 18) {
    // ------------------------------ MMA issuers ------------------------------
    // One issuing thread per group. Issuer X walks the K/V ring tiles of all items in order, each
    // tile as two sub-steps of 64 keys. For sub-step (g, c) it issues O_X += P_X V(g, c) and then
    // S_X = Q_X K(g+1, c)^T, the scores two sub-steps ahead, into the buffer that P_X(g, c) has
    // just left (also across an item boundary). A ring stage and a Q buffer are released by both
    // issuers: each commits (or, where its group has nothing to do with the tile, arrives) once.
    if (elect_one()) {
      const int X = (warp == 1) ? 0 : 1;
      constexpr uint32_t idesc_s = make_idesc_bf16(kT, 64, 0, 0);    // Q, K: K-major; 64 keys
      constexpr uint32_t idesc_o = make_idesc_bf16(kT, kHD, 0, 1);   // P from TMEM, V MN-major
      const SmemDescBase q_desc0 = make_desc_base_sw128(smem_u32(smem + L::kQ), 0);
      const SmemDescBase k_desc0 = make_desc_base_sw128(smem_u32(smem + L::kK), 0);
      const SmemDescBase v_desc0 = make_desc_base_sw128(smem_u32(smem + L::kV), 0);
      const uint32_t tSx = tmem + kColS + X * 128, tOx = tmem + kColO + X * 2 * kHD;
      int n_pv = 0;      // sub-steps of this group whose P V products have been issued
      int n_done = 0;    // items finished so far in which the group took part
      bool ok = true;

      // S_X = Q_X K^T for the 64 keys of sub-step c of K/V ring tile g, item in Q buffer qb; the
      // group's sub-steps alternate between its two score buffers, and c is the buffer
      auto issue_s = [&](int qb, int g, int c) {
        const SmemDescBase qd{q_desc0.lo + (qb * 2 + X) * (kPanel >> 4), q_desc0.hi};
        const SmemDescBase kd{k_desc0.lo + (g % kKvStages) * (kPanel >> 4), k_desc0.hi};
#pragma unroll
        for (int kk = 0; kk < kHD / 16; ++kk)
          mma_ss(tSx + c * 64, desc_at(qd, kk * 32), desc_at(kd, c * 8192 + kk * 32), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(&bars->s_full[X][c]);
      };
      // O_(X,h) (+)= P_(X,h) V[keys 64 c + 32 h .. + 31] of ring tile g, both halves. P of half h
      // sits in the first 16 columns of its 32 columns of buffer c, 16 keys (8 columns of packed
      // bf16 pairs) per MMA; V is MN-major, 16 keys = 2048 bytes further down.
      auto issue_pv = [&](int g, int c, bool first_of_item) -> bool {
        // the epilogue of the group's previous item must have read O_X before it is overwritten
        if (first_of_item && n_done > 0 && !mbar_wait(&bars->o_free[X], (n_done - 1) & 1, abort_flag))
          return false;
        if (!mbar_wait(&bars->p_full[X][c], (n_pv >> 1) & 1, abort_flag)) return false;
        tc_fence_after_sync();
        const SmemDescBase vd{v_desc0.lo + (g % kKvStages) * (kPanel >> 4), v_desc0.hi};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
            mma_ts(tOx + h * kHD, tSx + c * 64 + h * 32 + kk * 8, desc_at(vd, (c * 4 + h * 2 + kk) * 2048),
                   idesc_o, (!first_of_item || kk > 0) ? 1u : 0u);
        }
        mma_commit(&bars->o_done[X][n_pv & 1]);
        ++n_pv;
        return true;
      };
      auto n_of = [&](const F64Item& it) { return X ? it.n_b : it.n_a; };

      F64Item cur = f64_item(deal, 0, BH, n_tiles, n_items);
      F64Item nxt = f64_item(deal, 1, BH, n_tiles, n_items);
      int g = 0;
      if (cur.valid) {
        ok = mbar_wait(&bars->q_full[0], 0, abort_flag) && mbar_wait(&bars->k_full[0], 0, abort_flag);
        if (ok) {
          tc_fence_after_sync();
          if (n_of(cur) > 0) {
            issue_s(0, 0, 0);
            issue_s(0, 0, 1);
          }
          if (n_of(cur) <= 1) {   // the item's only (or no) score products of this group
            if (n_of(cur) == 1) mma_commit(&bars->q_empty[0]); else mbar_arrive(&bars->q_empty[0]);
          }
        }
      }
      for (int k = 0; ok && cur.valid; ++k) {
        const int qb = k & 1;
        const int n_x = n_of(cur);
        for (int j = 0; ok && j < cur.n_kv; ++j, ++g) {
          const int s = g % kKvStages;
          // The tile after this one in the ring: the item's next tile, or the next item's first.
          const bool last = (j + 1 == cur.n_kv);
          const bool have_next = !last || nxt.valid;
          const F64Item& ni = last ? nxt : cur;
          const int nj = last ? 0 : j + 1, nqb = last ? (qb ^ 1) : qb;
          // Every release below follows a wait on the matching "full" barrier of the same use,
          // also where this group has nothing to do with the tile: an idle issuer must not run
          // ahead and arrive twice within one phase of a release barrier.
          bool issued = false;
          ok = mbar_wait(&bars->v_full[s], (g / kKvStages) & 1, abort_flag);
          const int n_next = have_next ? n_of(ni) : 0;
          const bool s_next = have_next && nj < n_next;   // the group has scores to form in the next tile
          bool next_ready = false;
#pragma unroll
          for (int c = 0; c < 2 && ok; ++c) {
            if (j < n_x) {
              ok = issue_pv(g, c, j == 0 && c == 0);
              issued = ok;
            }
            if (ok && s_next) {
              if (!next_ready) {
                if (last) ok = mbar_wait(&bars->q_full[nqb], ((k + 1) >> 1) & 1, abort_flag);
                ok = ok && mbar_wait(&bars->k_full[(g + 1) % kKvStages], ((g + 1) / kKvStages) & 1, abort_flag);
                if (ok) tc_fence_after_sync();
                next_ready = true;
              }
              if (ok) {
                issue_s(nqb, g + 1, c);
                issued = true;
                // the item's last scores of this group
                if (c == 1 && nj + 1 == n_next) mma_commit(&bars->q_empty[nqb]);
              }
            }
          }
          if (ok && have_next && !s_next && nj == 0) {
            // the next item has no tile for this group: hand its Q buffer back (once it is loaded)
            if (last) ok = mbar_wait(&bars->q_full[nqb], ((k + 1) >> 1) & 1, abort_flag);
            if (ok) mbar_arrive(&bars->q_empty[nqb]);
          }
          // this issuer's share of the stage's release: after every product of its that reads it
          if (ok) {
            if (issued) mma_commit(&bars->kv_empty[s]); else mbar_arrive(&bars->kv_empty[s]);
          }
        }
        if (n_x > 0) ++n_done;
        cur = nxt;
        nxt = f64_item(deal, k + 2, BH, n_tiles, n_items);
      }
    }
  } else {
    // ------------------------------ softmax groups ------------------------------
    const int X = (warp - 2) / 8;         // 0: group A (first tile of the pair), 1: group B (warps 2-17)
    const int half = ((warp - 2) / 4) & 1;  // which 32 key columns of every 64-key sub-step
    const int quad = warp % 4;            // TMEM lane quadrant this warp may touch
    const int row = quad * 32 + lane;     // row within the tile = TMEM lane
    const uint32_t tlane = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t tS0 = tlane + kColS + X * 128 + half * 32;   // this thread's columns of buffer 0
    const float scale_log2 = scale * kLog2e;
    const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;
    int t = 0;        // 64-key sub-steps this group has processed so far, over all items
    int n_item = 0;   // items this group has taken part in
    bool ok = true;

    for (int k = 0; ok; ++k) {
      const F64Item it = f64_item(deal, k, BH, n_tiles, n_items);
      if (!it.valid) break;
      const int n_x = X ? it.n_b : it.n_a;
      if (n_x == 0) continue;               // the pair's second tile lies beyond the sequence
      const int qt = it.qa + X;
      float m = -INFINITY;                  // running max of the scaled scores, log2 units
      float2 l2 = make_float2(0.f, 0.f);    // running sum, two interleaved partial sums
      const uint32_t* bits1 = reinterpret_cast<const uint32_t*>(mask_bits);
      uint32_t keep = ~0u, keep_next = ~0u;
      if (DROP == 2) keep_next = __ldg(bits1 + mask_bits_record(it.bh, qt, 0, row, n_tiles) * 4 + half);

      for (int v = 0; v < 2 * n_x; ++v, ++t) {
        const int j = v >> 1, c = v & 1;    // K/V tile and its sub-step; c is also the score buffer
        if (DROP == 2) {
          keep = keep_next;   // fetched a sub-step ahead: its latency hides behind this one's work
          if (v + 1 < 2 * n_x)
            keep_next = __ldg(bits1 + mask_bits_record(it.bh, qt, (v + 1) >> 1, row, n_tiles) * 4 +
                              ((v + 1) & 1) * 2 + half);
        }
        if (!(ok = mbar_wait(&bars->s_full[X][c], (t >> 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
        const uint32_t tS = tS0 + c * 64;
        const bool diagonal = (j == n_x - 1);
        const int limit = row - c * 64 - half * 32;   // diagonal tile: column i visible iff i <= limit

        // ---- the thread's 32 scores: read once, kept in registers for the max and the
        // exponentials ----
        uint32_t xa[32];
        auto load_scores = [&]() {
          tmem_ld32(tS, xa);
          tmem_wait_ld();
          if (diagonal) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i > limit) xa[i] = 0xff800000u;  // -inf
          }
        };
        load_scores();
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          mx0 = fmax3(mx0, __uint_as_float(xa[i]), __uint_as_float(xa[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(xa[i + 2]), __uint_as_float(xa[i + 3]));
        }
        const float mx = fmaxf(mx0, mx1) * scale_log2;   // scale > 0 commutes with max

        // ---- lazy rescale: O and the sum move to a new max only when it grew by 2^8 ----
        if (v == 0) {
          m = mx;  // O is first written by an MMA that does not accumulate: nothing to rescale
        } else if (__any_sync(0xffffffffu, mx > m + kRescaleAt)) {
          // P V of this group's previous sub-step must have completed before O is touched
          if (!(ok = mbar_wait(&bars->o_done[X][(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
          const float m_new = fmaxf(m, mx);
          // m = -inf: nothing but zeros has been accumulated so far (every earlier column masked)
          const float corr = (m == -INFINITY) ? 0.f : ex2(m - m_new);
#pragma unroll 1
          for (int cc = 0; cc < kHD / 32; ++cc) {
            uint32_t o[32];
            tmem_ld32(tlane + kColO + (X * 2 + half) * kHD + cc * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st32(tlane + kColO + (X * 2 + half) * kHD + cc * 32, o);
          }
          tmem_wait_st();
          l2 = fmul2(l2, make_float2(corr, corr));
          m = m_new;
          // read the scores again rather than keep them alive across this rare path
          load_scores();
        }

        // ---- p = exp2(s * scale * log2e - m); P goes back to tensor memory as packed bf16
        // pairs over the first 16 of this thread's columns. A half-row with no visible key yet has
        // m = -inf: its scores are all -inf and must give p = 0, not exp2(nan). ----
        const float neg_m = (m == -INFINITY) ? 0.f : -m;
        const float2 sl = make_float2(scale_log2, scale_log2), nm = make_float2(neg_m, neg_m);
        float2 la = make_float2(0.f, 0.f), lb = la;   // this sub-step's sums, two independent chains
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 e = ffma2(make_float2(__uint_as_float(xa[i]), __uint_as_float(xa[i + 1])), sl, nm);
          float2 p;
          if ((i & 7) == 6) {   // one pair in four on the FMA pipe
            p = ex2_poly2(e);
          } else {
            p.x = ex2(e.x);
            p.y = ex2(e.y);
          }
          if (i & 2) lb = fadd2(lb, p); else la = fadd2(la, p);
          if (DROP == 1) {
            const uint64_t idx = (static_cast<uint64_t>(unit0 + it.bh) * S + qt * kT + row) * S + j * kT +
                                 c * 64 + half * 32 + i;
            p.x = (p.x != 0.f && philox_keep(rng, idx, rate)) ? p.x * keep_scale : 0.f;
            p.y = (p.y != 0.f && philox_keep(rng, idx + 1, rate)) ? p.y * keep_scale : 0.f;
          } else if (DROP == 2) {
            p.x = ((keep >> i) & 1u) ? p.x * keep_scale : 0.f;
            p.y = ((keep >> (i + 1)) & 1u) ? p.y * keep_scale : 0.f;
          }
          pk[i / 2] = pack_bf16(p.x, p.y);
        }
        tmem_st16(tS, pk);          // P of this thread's 32 keys -> its first 16 columns
        l2 = fadd2(l2, fadd2(la, lb));
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(&bars->p_full[X][c]);
      }
      if (!ok) break;

      // ---- epilogue: merge the two halves of each row. out = (O_0 w_0 + O_1 w_1) / (l_0 w_0 +
      // l_1 w_1) with w_h = exp2(m_h - max(m_0, m_1)); lse in natural-log units of the scaled
      // scores. Each thread of the pair writes 32 of the row's 64 outputs. ----
      float2* stat = reinterpret_cast<float2*>(smem + L::kStat) + X * 256;   // [half][128]
      const int r = qt * kT + row;          // query index
      stat[half * 128 + row] = make_float2(m, l2.x + l2.y);
      mbar_arrive(&bars->stat_full[X]);
      if (!(ok = mbar_wait(&bars->stat_full[X], n_item & 1, abort_flag))) break;
      // the group's last P V products (both halves)
      if (!(ok = mbar_wait(&bars->o_done[X][(t - 1) & 1], ((t - 1) >> 1) & 1, abort_flag))) break;
      tc_fence_after_sync();
      const float2 s0 = stat[row], s1 = stat[128 + row];
      const float m_tot = fmaxf(s0.x, s1.x);   // half 0 always sees key 0: finite
      const float w0 = ex2(s0.x - m_tot);
      const float w1 = (s1.x == -INFINITY) ? 0.f : ex2(s1.x - m_tot);
      const float l_tot = s0.y * w0 + s1.y * w1;
      const float f0 = w0 / l_tot, f1 = w1 / l_tot;
      const int ub = it.bh / lay.heads, uh = it.bh - ub * lay.heads;
      __nv_bfloat16* dst = out + ub * lay.batch + uh * lay.head + r * lay.row + half * 32;
#pragma unroll
      for (int c = 0; c < 2; ++c) {   // 16 output columns at a time
        uint32_t oa[16], ob[16];
        tmem_ld16(tlane + kColO + (X * 2 + 0) * kHD + half * 32 + c * 16, oa);
        tmem_ld16(tlane + kColO + (X * 2 + 1) * kHD + half * 32 + c * 16, ob);
        tmem_wait_ld();
        if (c == 1) {
          tc_fence_before_sync();
          mbar_arrive(&bars->o_free[X]);   // O and the statistics have been read: the next item may start
        }
        if (r < S) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              y[e] = __uint_as_float(oa[8 * i + e]) * f0 + __uint_as_float(ob[8 * i + e]) * f1;
            *reinterpret_cast<uint4*>(dst + c * 16 + i * 8) = make_uint4(
                pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]), pack_bf16(y[6], y[7]));
          }
        }
      }
      ++n_item;
      if (r < S) {
        if (half == 0) lse[static_cast<size_t>(it.bh) * S + r] = (m_tot + log2f(l_tot)) * kLn2;
      }
    }
  }

  // ------------------------------ common exit ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) report_timeout(status, bars->abort_flag);
}

// The greedy deal for a launch of G CTAs, or rows = 0 when the closed form serves (too many
// items for the table). An item's weight is its K/V steps plus a half for its prologue and
// epilogue. The last deal is kept: a training loop asks for the same one again and again.
const F64Deal& fwd64_deal(int BH, int n_tiles, int G) {
  struct Cached {
    int BH = -1, n_tiles = -1, G = -1;
    F64Deal deal;
  };
  static thread_local Cached cache;
  if (cache.BH == BH && cache.n_tiles == n_tiles && cache.G == G) return cache.deal;
  cache.BH = BH, cache.n_tiles = n_tiles, cache.G = G;
  F64Deal& d = cache.deal;
  d.rows = 0;
  const int n_pairs = (n_tiles + 1) / 2;
  const long long n_items = static_cast<long long>(BH) * n_pairs;
  if (n_items > kDealEntries || G <= 0) return d;   // (every item takes an entry: no table could hold them)
  std::vector<int> load(G, 0), count(G, 0);
  std::vector<std::vector<uint16_t>> list(G);
  // G is at most a few hundred and the table small: a linear scan for the least loaded CTA
  for (int e = 0; e < static_cast<int>(n_items); ++e) {
    const int qa = 2 * (n_pairs - 1 - e / BH);
    const int n_kv = (qa + 1 < n_tiles) ? qa + 2 : qa + 1;
    int best = 0;
    for (int c = 1; c < G; ++c)
      if (load[c] < load[best]) best = c;
    load[best] += 2 * n_kv + 1;
    list[best].push_back(static_cast<uint16_t>(e));
  }
  size_t rows = 0;
  for (int c = 0; c < G; ++c) rows = list[c].size() > rows ? list[c].size() : rows;
  if (rows * G > kDealEntries) return d;
  for (size_t k = 0; k < rows; ++k)
    for (int c = 0; c < G; ++c) d.item[k * G + c] = k < list[c].size() ? list[c][k] : kDealNone;
  d.rows = static_cast<int>(rows);
  return d;
}

template <int DROP>
int launch_fwd64(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                 int BH, int S, const UnitLayout& lay, float scale, float rate, uint64_t seed,
                 uint64_t offset, int64_t unit0, const uint32_t* mask_bits, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  if (int rc = make_tensor_map_bf16_units(&mq, q, BH, S, kHD, kT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mk, k, BH, S, kHD, kT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mv, v, BH, S, kHD, kT, lay)) return rc;
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  int dev = 0, sms = 0;
  DAD_CUDA(cudaGetDevice(&dev));
  DAD_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int n_tiles = (S + kT - 1) / kT;
  const long long n_items = static_cast<long long>(BH) * ((n_tiles + 1) / 2);
  if (n_items > INT32_MAX / 2) return fail(DADATTN_E_UNSUPPORTED, "too many (query tile pair, batch x head) items");
  auto kern = flash_fwd64_kernel<DROP>;
  DAD_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, F64Smem::kBytes));
  dim3 grid(static_cast<unsigned>(n_items < sms ? n_items : sms));
  DAD_CUDA(launch_pdl(kern, grid, dim3(kFwd64Threads), F64Smem::kBytes, st, mq, mk, mv,
                      reinterpret_cast<__nv_bfloat16*>(out), lse, BH, S, lay, scale, rate,
                      make_philox(seed, offset), unit0, reinterpret_cast<const uint4*>(mask_bits), status,
                      fwd64_deal(BH, n_tiles, static_cast<int>(grid.x))));
  return DADATTN_OK;
}

}  // namespace

// Forward at head size 64. mask_bits != nullptr: keep bits from dadattn_dropout_mask_bits;
// otherwise rate > 0 draws the Philox mask inside the kernel. heads > 0: q, k, v, out are the
// interleaved [B*S, heads*64] activations (BH = B * heads units); heads = 0: heads-split [BH,S,64].
int launch_fwd_bf16_d64(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                        int BH, int S, float scale, float rate, uint64_t seed, uint64_t offset,
                        int64_t unit0, const uint32_t* mask_bits, int heads, cudaStream_t st) {
  const UnitLayout lay = heads > 0 ? unit_layout(BH / heads, heads, S, kHD, true) : unit_layout(BH, 1, S, kHD, false);
  if (rate > 0.f && mask_bits)
    return launch_fwd64<2>(out, lse, q, k, v, BH, S, lay, scale, rate, 0, 0, 0, mask_bits, st);
  if (rate > 0.f)
    return launch_fwd64<1>(out, lse, q, k, v, BH, S, lay, scale, rate, seed, offset, unit0, nullptr, st);
  return launch_fwd64<0>(out, lse, q, k, v, BH, S, lay, scale, 0.f, 0, 0, 0, nullptr, st);
}

}  // namespace dadattn
