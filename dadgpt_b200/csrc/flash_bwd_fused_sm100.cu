// bf16 fused causal attention backward for sm_100a, head size 64: dQ, dK and dV in ONE pass.
//
// The reference computes the probabilities twice, once in its dK/dV kernel and once in its dQ
// kernel (cuda/attention.cu:88-205): 7 GEMM-sized products for 5 gradients' worth. Here a CTA
// owns 128 keys of one (batch, head), streams the 128-query tiles that can see them, and per
// tile forms S = Q K^T and dP = dO V^T once, then
//     dV += P^T dO        dK += dS^T Q        dQ_tile = dS K
// with p = exp2(S scale log2e - lse log2e), ds = p (dP - delta) scale as in the reference.
// dK/dV accumulate in tensor memory over the whole loop; each tile's dQ contribution is added
// into an fp32 workspace with a TMA reduce-add (several CTAs, one per key tile, contribute to
// the same queries), and a last pass rounds the workspace to bf16. The sums into the workspace
// happen in whatever order the CTAs reach them, so dQ may differ in its last bits from run to
// run; dadattn_set_bwd_deterministic(1) selects the two-kernel path of
// flash_bwd_bf16_sm100.cu, which has no such sums.
//
// Rows of the score tile are queries (one TMEM lane each), so lse and delta are per-thread
// scalars. P and dS are written once, bf16, row-major [query][key] in the 128-byte swizzled
// layout: dS is the K-major A operand of dQ = dS K, and the same bytes read as an MN-major A
// operand are dS^T (resp. P^T) for dK (resp. dV). The Q / dO tiles are K-major A operands of the
// score GEMMs and MN-major B operands of dK / dV; K is the K-major B operand of S and the
// MN-major B operand of dQ.
//   warps 0-15   compute: four warps per TMEM lane quadrant, 32 of the 128 key columns each
//   warp 16      TMA producer           warp 17      MMA issuer + TMEM owner
//   warp 18      dQ reducer: issues the TMA reduce-adds and the dK / dV stores   (warp 19 idle)
//   warps 20-23  accumulator drain: one thread per TMEM lane takes each tile's dQ, and each
//                item's dK / dV, out of tensor memory into the shared-memory staging buffers,
//                while the compute warps are already on the next tile's arithmetic
// The roles are whole warpgroups so that registers can move between them (setmaxnreg): the
// compute warps hold two packed tiles' worth of values and get 96 registers, the others 56 / 40.
#include <cuda_bf16.h>

#include <cfloat>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace dadattn {
namespace {

using namespace ptx;

constexpr int kFT = 128;                  // tile edge: queries per step, keys per CTA
constexpr int kFD = 64;                   // head size
constexpr int kFPanel = 128 * 128;        // [128 rows][64 bf16] swizzled panel
constexpr int kFThreads = 24 * 32;
constexpr int kFCompute = 16 * 32;
constexpr int kFDrain = 4 * 32;           // one thread per TMEM lane
constexpr int kWarpProducer = 16, kWarpIssuer = 17, kWarpReducer = 18, kWarpDrain0 = 20;
// Registers per thread after the warpgroups have rebalanced. The pool is what the CTA was launched
// with (kRegsLaunch per thread, the most that 768 threads can have): an increase beyond it would
// wait for ever.
constexpr int kRegsLaunch = 80, kRegsCompute = 96, kRegsHelper = 56, kRegsDrain = 40;
static_assert(kFCompute * kRegsCompute + 128 * kRegsHelper + kFDrain * kRegsDrain <= kFThreads * kRegsLaunch,
              "the warpgroups ask for more registers than the CTA owns");
static_assert(kFThreads * kRegsLaunch <= 65536 && (kRegsLaunch + 8) * kFThreads > 65536,
              "kRegsLaunch is not what the compiler gives a CTA of this size");
constexpr int kFStages = 2;
constexpr int kFRing = 4;                 // entries of the work-item ring (a power of two)
constexpr float kFLog2e = 1.4426950408889634f;
constexpr int kVecBox = 132;   // fp32 words one row-scalar load brings in

struct FusedSmem {
  static constexpr int kK = 0;                          // two buffers: items alternate
  static constexpr int kV = kK + 2 * kFPanel;
  static constexpr int kQ = kV + 2 * kFPanel;
  static constexpr int kDO = kQ + kFStages * kFPanel;
  static constexpr int kP = kDO + kFStages * kFPanel;   // [128 q][128 keys] bf16, two panels
  static constexpr int kDS = kP + 2 * kFPanel;
  static constexpr int kDQ = kDS + 2 * kFPanel;         // [128 q][64] fp32, two 128-byte panels
  static constexpr int kBars = kDQ + 2 * kFPanel;
  // Per-row scalars of a query tile, one buffer per Q / dO stage: lse and delta of kVecBox rows
  // each (the tile's 128 and up to three before them: a TMA load starts on a 16-byte boundary),
  // every vector on its own 128-byte boundary.
  static constexpr int kBarsBytes = 384;
  static constexpr int kVec = kBars + kBarsBytes;
  static constexpr int kVecDelta = 640, kVecStride = 1280;
  static constexpr int kBytes = kVec + kFStages * kVecStride;
  static_assert(kVec % 128 == 0 && kVecBox * 4 <= kVecDelta, "row-scalar buffers misplaced");
  static_assert(kBytes <= 232448, "shared memory budget of one CTA exceeded");
};

struct FusedBars {
  uint64_t kv_full[2], dkv_sent[2], q_full[kFStages], do_full[kFStages], qdo_empty[kFStages];
  uint64_t item_ready[kFRing], item_free[kFRing];
  uint64_t x_full, x_free, w_full, acc_done, dq_drained, dq_staged, dq_sent, dkv_staged[2], vec_full[kFStages];
  uint64_t dkv_drained;
  int ring[kFRing];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(FusedBars) <= FusedSmem::kBarsBytes, "barriers overflow their shared-memory slot");

// TMA reduce-add of one [128 rows][32 fp32] panel from shared memory into the dQ workspace.
// `policy`: an L2 eviction policy (l2_policy_evict_last): the workspace is summed into up to
// T / 128 times and read once more by the rounding pass, so its lines should outlive the streamed
// Q / dO / K / V tiles in L2.
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, const void* smem_src, int x,
                                                  int y, int z, uint64_t policy) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group.L2::cache_hint "
      "[%0, {%2, %3, %4}], [%1], %5;"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// TMA store of one [128 rows][64 bf16] swizzled panel from shared memory to (x, row, head, batch)
// of a tensor in either memory layout (UnitLayout); rows beyond the sequence are dropped.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int x, int y,
                                             int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

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

// One item of work = (key tile kt, batch x head bh): the CTA that takes it streams the n_it query
// tiles that can see those keys. Items are numbered so that batch x head units come in groups of
// `group_bh` (their Q, dO and dQ rows stay in L2 while the group is worked on) and, inside a
// group, key tile by key tile: the key tiles with the most queries first.
struct Item {
  int kt, bh, n_it;
};
__device__ __forceinline__ Item decode_item(int item, int BH, int n_tiles, int group_bh) {
  const int per_group = group_bh * n_tiles;
  const int grp = item / per_group;
  const int r = item - grp * per_group;
  const int bh0 = grp * group_bh;
  const int gb = min(group_bh, BH - bh0);
  Item t;
  t.kt = r / gb;
  t.bh = bh0 + r - t.kt * gb;
  t.n_it = n_tiles - t.kt;
  return t;
}

// Items are handed out by a global counter; the producer thread takes them and publishes each
// through a four-entry ring in shared memory, which the other roles read in the same order.
struct ItemFeed {
  FusedBars* bars;
  volatile int* abort_flag;
  int n_read;
  // the next item of this CTA, or n_items when there is none (or the kernel is aborting)
  __device__ __forceinline__ int fetch(int n_items) {
    const int slot = n_read & (kFRing - 1);
    if (!mbar_wait(&bars->item_ready[slot], (n_read / kFRing) & 1, abort_flag)) return n_items;
    const int v = *reinterpret_cast<volatile int*>(&bars->ring[slot]);
    mbar_arrive(&bars->item_free[slot]);
    ++n_read;
    return v;
  }
};

// DROP: 0 = no dropout, 1 = Philox drawn in the kernel, 2 = keep bits read from `mask_bits`
// (dadattn_dropout_mask_bits; layout in common.cuh).
template <int DROP>
__global__ void __launch_bounds__(kFThreads, 1)
flash_bwd_fused_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                       const __grid_constant__ CUtensorMap map_dqw, const __grid_constant__ CUtensorMap map_dk,
                       const __grid_constant__ CUtensorMap map_dv, const __grid_constant__ CUtensorMap map_lse,
                       const __grid_constant__ CUtensorMap map_delta, int lse_shift,
                       int* __restrict__ item_counter, int BH, int S,
                       int heads, int group_bh, float scale, float rate, PhiloxKey rng, int64_t unit0,
                       const uint32_t* __restrict__ mask_bits, int* __restrict__ status) {
  using L = FusedSmem;
  constexpr int D = kFD;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 320, kColDQ = 384;

  extern __shared__ __align__(1024) uint8_t smem[];
  FusedBars* bars = reinterpret_cast<FusedBars*>(smem + L::kBars);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n_tiles = (S + kFT - 1) / kFT;
  const int n_items = n_tiles * BH;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(status, DADATTN_E_CUDA);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->dkv_sent[s], 1);
    }
    for (int s = 0; s < kFStages; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->do_full[s], 1);
      mbar_init(&bars->qdo_empty[s], 1);
    }
    for (int s = 0; s < kFRing; ++s) {
      mbar_init(&bars->item_ready[s], 1);
      mbar_init(&bars->item_free[s], kFCompute + kFDrain + 2);   // compute, drain, MMA issuer, reducer
    }
    mbar_init(&bars->x_full, 1);
    mbar_init(&bars->x_free, kFCompute);
    mbar_init(&bars->w_full, kFCompute);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->dq_drained, kFDrain);
    mbar_init(&bars->dq_staged, kFDrain);
    mbar_init(&bars->dkv_drained, kFDrain);
    mbar_init(&bars->dq_sent, 1);
    mbar_init(&bars->dkv_staged[0], kFDrain);
    mbar_init(&bars->dkv_staged[1], kFDrain);
    for (int s = 0; s < kFStages; ++s) mbar_init(&bars->vec_full[s], 1);
    bars->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == kWarpIssuer) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  pdl_wait();
  pdl_launch_dependents();

  // Registers move from the helper warpgroups to the compute warpgroups; each branch below sets
  // its own budget first.
  if (warp >= kWarpProducer && warp < kWarpDrain0) {
  setmaxnreg_dec<kRegsHelper>();
  if (warp == kWarpProducer) {
    // ------------------------------ scheduler + TMA producer ------------------------------
    if (elect_one()) {
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      prefetch_tensormap(&map_do);
      prefetch_tensormap(&map_lse);
      prefetch_tensormap(&map_delta);
      int n_pub = 0;
      auto publish = [&](int item) -> bool {
        const int slot = n_pub & (kFRing - 1);
        if (n_pub >= kFRing &&
            !mbar_wait(&bars->item_free[slot], (n_pub / kFRing - 1) & 1, abort_flag))
          return false;
        *reinterpret_cast<volatile int*>(&bars->ring[slot]) = item;
        mbar_arrive(&bars->item_ready[slot]);
        ++n_pub;
        return true;
      };
      // the first item is the CTA's own index; the counter hands out the rest
      int cur = static_cast<int>(blockIdx.x);
      bool ok = publish(cur);
      int g = 0;
      for (int j = 0; ok && cur < n_items; ++j) {
        const Item t = decode_item(cur, BH, n_tiles, group_bh);
        // K / V go to the buffer of the item before last, once its dK / dV have left that buffer
        const int kb = j & 1;
        if (ok && j >= 2) ok = mbar_wait(&bars->dkv_sent[kb], ((j >> 1) - 1) & 1, abort_flag);
        if (!ok) break;
        const int ub = t.bh / heads, uh = t.bh - ub * heads;   // (batch, head) of the unit
        mbar_arrive_expect_tx(&bars->kv_full[kb], 2 * kFPanel);
        tma_load_4d(smem + L::kK + kb * kFPanel, &map_k, &bars->kv_full[kb], 0, t.kt * kFT, uh, ub);
        tma_load_4d(smem + L::kV + kb * kFPanel, &map_v, &bars->kv_full[kb], 0, t.kt * kFT, uh, ub);
        // The following item (or the end mark) is claimed only now, and published at once: the
        // other roles look one item ahead. Every item a CTA holds in advance is work that no idle
        // CTA can take near the end of the kernel, so it holds as few as it can.
        const int nxt = static_cast<int>(gridDim.x) + atomicAdd(item_counter, 1);
        ok = publish(nxt);
        for (int i = 0; ok && i < t.n_it; ++i, ++g) {
          const int s = g % kFStages, use = g / kFStages;
          if (use > 0 && !(ok = mbar_wait(&bars->qdo_empty[s], (use - 1) & 1, abort_flag))) break;
          const int q0 = (t.kt + i) * kFT;
          mbar_arrive_expect_tx(&bars->q_full[s], kFPanel);
          tma_load_4d(smem + L::kQ + s * kFPanel, &map_q, &bars->q_full[s], 0, q0, uh, ub);
          mbar_arrive_expect_tx(&bars->do_full[s], kFPanel);
          tma_load_4d(smem + L::kDO + s * kFPanel, &map_do, &bars->do_full[s], 0, q0, uh, ub);
          // The tile's row scalars ride the same ring: the stage is free once the GEMMs of the
          // tile that used it have completed, and those followed the arithmetic that read the
          // scalars. The load starts at the 16-byte boundary at or below the tile's first row.
          const int at = t.bh * S + q0;
          mbar_arrive_expect_tx(&bars->vec_full[s], 2 * kVecBox * 4);
          tma_load_1d(smem + L::kVec + s * L::kVecStride, &map_lse, &bars->vec_full[s], (at + lse_shift) & ~3);
          tma_load_1d(smem + L::kVec + s * L::kVecStride + L::kVecDelta, &map_delta, &bars->vec_full[s], at & ~3);
        }
        cur = nxt;
      }
    }
  } else if (warp == kWarpIssuer) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_x = make_idesc_bf16(128, 128, 0, 0);   // S, dP: both K-major
      constexpr uint32_t idesc_t = make_idesc_bf16(128, 64, 1, 1);    // dV, dK: A and B MN-major
      constexpr uint32_t idesc_q = make_idesc_bf16(128, 64, 0, 1);    // dQ: A K-major, B MN-major
      const SmemDescBase k0_desc = make_desc_base_sw128(smem_u32(smem + L::kK), 0);
      const SmemDescBase v0_desc = make_desc_base_sw128(smem_u32(smem + L::kV), 0);
      const SmemDescBase q0_desc = make_desc_base_sw128(smem_u32(smem + L::kQ), 0);
      const SmemDescBase do0_desc = make_desc_base_sw128(smem_u32(smem + L::kDO), 0);
      // P / dS read as MN-major A: the two 64-key panels are kFPanel apart (leading byte offset)
      const SmemDescBase p_t = make_desc_base_sw128(smem_u32(smem + L::kP), kFPanel);
      const SmemDescBase ds_t = make_desc_base_sw128(smem_u32(smem + L::kDS), kFPanel);
      const SmemDescBase ds_k = make_desc_base_sw128(smem_u32(smem + L::kDS), 0);

      // S = Q K^T and dP = dO V^T of tile g (counted over all items of this CTA), K / V buffer kb
      auto issue_x = [&](int g, int kb) -> bool {
        const int s = g % kFStages;
        const uint32_t par = (g / kFStages) & 1;
        const SmemDescBase qd{q0_desc.lo + s * (kFPanel >> 4), q0_desc.hi};
        const SmemDescBase dd{do0_desc.lo + s * (kFPanel >> 4), do0_desc.hi};
        const SmemDescBase kd{k0_desc.lo + kb * (kFPanel >> 4), k0_desc.hi};
        const SmemDescBase vd{v0_desc.lo + kb * (kFPanel >> 4), v0_desc.hi};
        if (!mbar_wait(&bars->q_full[s], par, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem + kColS, desc_at(qd, kk * 32), desc_at(kd, kk * 32), idesc_x, kk > 0 ? 1u : 0u);
        if (!mbar_wait(&bars->do_full[s], par, abort_flag)) return false;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem + kColDP, desc_at(dd, kk * 32), desc_at(vd, kk * 32), idesc_x, kk > 0 ? 1u : 0u);
        mma_commit(&bars->x_full);
        return true;
      };
      // dV += P^T dO, dK += dS^T Q (fresh accumulators on an item's first tile), dQ_tile = dS K
      auto issue_acc = [&](int g, int item, bool first_of_item) -> bool {
        const int kb = item & 1;
        const int s = g % kFStages;
        const SmemDescBase qd{q0_desc.lo + s * (kFPanel >> 4), q0_desc.hi};
        const SmemDescBase dd{do0_desc.lo + s * (kFPanel >> 4), do0_desc.hi};
        const SmemDescBase kd{k0_desc.lo + kb * (kFPanel >> 4), k0_desc.hi};
        if (!mbar_wait(&bars->w_full, g & 1, abort_flag)) return false;
        // a new item's first products overwrite dV / dK: the drain warps must have taken the
        // previous item's out of tensor memory
        if (first_of_item && item > 0 && !mbar_wait(&bars->dkv_drained, (item - 1) & 1, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kFT / 16; ++kk) {   // K dimension = 128 queries, 16 per MMA
          const uint32_t acc = (!first_of_item || kk > 0) ? 1u : 0u;
          // A = P^T / dS^T: 16 query rows (2048 bytes) further down per step; B = dO / Q rows
          mma_ss(tmem + kColDV, desc_at(p_t, kk * 2048), desc_at(dd, kk * 2048), idesc_t, acc);
          mma_ss(tmem + kColDK, desc_at(ds_t, kk * 2048), desc_at(qd, kk * 2048), idesc_t, acc);
        }
        // Q and dO of this stage are last read by the products above: the stage goes back to the
        // producer now, not after dQ, which only needs dS and K.
        mma_commit(&bars->qdo_empty[s]);
        // the previous tile's dQ must have left tensor memory before this one overwrites it; the
        // compute warps read it right after they publish P / dS, while dV / dK are running
        if (g > 0 && !mbar_wait(&bars->dq_drained, (g - 1) & 1, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kFT / 16; ++kk) {   // K dimension = 128 keys
          mma_ss(tmem + kColDQ, desc_at(ds_k, (kk / 4) * kFPanel + (kk % 4) * 32),
                 desc_at(kd, kk * 2048), idesc_q, kk > 0 ? 1u : 0u);
        }
        mma_commit(&bars->acc_done);
        return true;
      };

      ItemFeed feed{bars, abort_flag, 0};
      int cur = feed.fetch(n_items);
      int nxt = cur < n_items ? feed.fetch(n_items) : n_items;
      bool ok = cur < n_items && mbar_wait(&bars->kv_full[0], 0, abort_flag) && issue_x(0, 0);
      int g = 0;
      for (int j = 0; ok && cur < n_items; ++j) {
        const int n_it = decode_item(cur, BH, n_tiles, group_bh).n_it;
        for (int i = 0; ok && i < n_it; ++i, ++g) {
          // The next tile's score GEMMs go first, so the arithmetic on them overlaps this tile's
          // accumulating GEMMs; across an item boundary they use the other K / V buffer.
          if (i + 1 < n_it) {
            ok = mbar_wait(&bars->x_free, g & 1, abort_flag) && issue_x(g + 1, j & 1);
          } else if (nxt < n_items) {
            const int kbn = (j + 1) & 1;
            ok = mbar_wait(&bars->x_free, g & 1, abort_flag) &&
                 mbar_wait(&bars->kv_full[kbn], ((j + 1) >> 1) & 1, abort_flag) && issue_x(g + 1, kbn);
          }
          ok = ok && issue_acc(g, j, i == 0);
        }
        cur = nxt;
        nxt = cur < n_items ? feed.fetch(n_items) : n_items;
      }
    }
  } else if (warp == kWarpReducer) {
    // ------------------------------ dQ reducer / dK, dV writer ------------------------------
    if (elect_one()) {
      prefetch_tensormap(&map_dqw);
      const uint64_t keep = l2_policy_evict_last();
      prefetch_tensormap(&map_dk);
      prefetch_tensormap(&map_dv);
      ItemFeed feed{bars, abort_flag, 0};
      int cur = feed.fetch(n_items);
      int nxt = cur < n_items ? feed.fetch(n_items) : n_items;
      int g = 0;
      bool ok = true;
      for (int j = 0; ok && cur < n_items; ++j) {
        const Item t = decode_item(cur, BH, n_tiles, group_bh);
        for (int i = 0; ok && i < t.n_it; ++i, ++g) {
          if (!(ok = mbar_wait(&bars->dq_staged, g & 1, abort_flag))) break;
          const int q0 = (t.kt + i) * kFT;
          tma_reduce_add_3d(&map_dqw, smem + L::kDQ, 0, q0, t.bh, keep);
          tma_reduce_add_3d(&map_dqw, smem + L::kDQ + kFPanel, 32, q0, t.bh, keep);
          bulk_commit();
          if (i + 1 < t.n_it) {
            bulk_wait_read0();
            mbar_arrive(&bars->dq_sent);
          } else {
            // The item's dK / dV were staged (in its K / V buffers) before the dQ of its last
            // tile. Their stores go behind the reduce, so that the dQ staging buffer is handed
            // back as soon as the reduce has read it; the K / V buffers follow.
            // One barrier per K / V buffer, not one for all items: after a single-tile item the
            // compute warps stage the next item's dK / dV without needing this warp, so a single
            // barrier could run two phases ahead of a late reducer, whose parity wait would then
            // never be satisfied (and the compute warps in turn wait for this warp's dq_sent).
            // The next phase of dkv_staged[j & 1] belongs to item j + 2 and cannot complete
            // before this warp has handed back the staging buffer of item j's last tile.
            if (!(ok = mbar_wait(&bars->dkv_staged[j & 1], (j >> 1) & 1, abort_flag))) break;
            const int ub = t.bh / heads, uh = t.bh - ub * heads;
            tma_store_4d(&map_dk, smem + L::kK + (j & 1) * kFPanel, 0, t.kt * kFT, uh, ub);
            tma_store_4d(&map_dv, smem + L::kV + (j & 1) * kFPanel, 0, t.kt * kFT, uh, ub);
            bulk_commit();
            bulk_wait_read1();
            mbar_arrive(&bars->dq_sent);
            bulk_wait_read0();
            mbar_arrive(&bars->dkv_sent[j & 1]);
          }
        }
        cur = nxt;
        nxt = cur < n_items ? feed.fetch(n_items) : n_items;
      }
      bulk_wait0();   // every sum and store has landed before the CTA retires
    }
  }
  } else if (warp >= kWarpDrain0) {
    // ------------------------------ accumulator drain warps ------------------------------
    setmaxnreg_dec<kRegsDrain>();
    const int quad = warp % 4;
    const int row = quad * 32 + lane;     // TMEM lane = query row (dQ) or key row (dK / dV)
    const uint32_t tlane = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    ItemFeed feed{bars, abort_flag, 0};
    int cur = feed.fetch(n_items);
    int nxt = cur < n_items ? feed.fetch(n_items) : n_items;
    bool ok = true;
    int g = 0;
    for (int j = 0; ok && cur < n_items; ++j) {
      const int n_it = decode_item(cur, BH, n_tiles, group_bh).n_it;
      for (int i = 0; i < n_it; ++i, ++g) {
        // the staging buffer back from the previous tile's reduce, then this tile's GEMMs
        if (g > 0 && !(ok = mbar_wait(&bars->dq_sent, (g - 1) & 1, abort_flag))) break;
        if (!(ok = mbar_wait(&bars->acc_done, g & 1, abort_flag))) break;
        tc_fence_after_sync();
        if (i + 1 == n_it) {
          // The item is complete: dK / dV, tensor memory -> bf16 rows in the item's own K / V
          // buffers (every GEMM that read them has completed), from where the reducer warp
          // stores them. Sixteen columns at a time; dV is columns [0, 64), dK [64, 128).
          const int kb = j & 1;
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t o[16];
            tmem_ld16(tlane + kColDV + c * 16, o);   // kColDK = kColDV + 64
            tmem_wait_ld();
            uint8_t* dst = smem + (c < 4 ? L::kV : L::kK) + kb * kFPanel + row * 128;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int chunk = (c & 3) * 2 + h;
              *reinterpret_cast<uint4*>(dst + ((chunk ^ (row & 7)) << 4)) = make_uint4(
                  pack_bf16(__uint_as_float(o[8 * h + 0]), __uint_as_float(o[8 * h + 1])),
                  pack_bf16(__uint_as_float(o[8 * h + 2]), __uint_as_float(o[8 * h + 3])),
                  pack_bf16(__uint_as_float(o[8 * h + 4]), __uint_as_float(o[8 * h + 5])),
                  pack_bf16(__uint_as_float(o[8 * h + 6]), __uint_as_float(o[8 * h + 7])));
            }
          }
          tc_fence_before_sync();
          mbar_arrive(&bars->dkv_drained);          // the next item's products may overwrite dV / dK
          fence_proxy_async_smem();
          mbar_arrive(&bars->dkv_staged[kb]);
        }
        // dQ of the tile: tensor memory -> swizzled fp32 staging ([2 panels][128 rows][32 fp32]),
        // which the reducer warp sends on
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[16];
          tmem_ld16(tlane + kColDQ + c * 16, o);
          tmem_wait_ld();
          if (c == 3) {
            tc_fence_before_sync();
            mbar_arrive(&bars->dq_drained);          // the next tile's dQ may overwrite this one
          }
          uint8_t* dq_row = smem + L::kDQ + (c / 2) * kFPanel + row * 128;
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int chunk = (c & 1) * 4 + c4;
            *reinterpret_cast<uint4*>(dq_row + ((chunk ^ (row & 7)) << 4)) =
                make_uint4(o[4 * c4], o[4 * c4 + 1], o[4 * c4 + 2], o[4 * c4 + 3]);
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars->dq_staged);
      }
      cur = nxt;
      nxt = (ok && cur < n_items) ? feed.fetch(n_items) : n_items;
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    setmaxnreg_inc<kRegsCompute>();
    const int quad = warp % 4;            // TMEM lane quadrant of this warp
    const int cg = warp / 4;              // which 32 key columns of the 128
    const int row = quad * 32 + lane;     // query row within the tile = TMEM lane
    const uint32_t tlane = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float scale_log2 = scale * kFLog2e;
    const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;
    uint8_t* p_row = smem + L::kP + (cg / 2) * kFPanel + row * 128;
    uint8_t* ds_row = smem + L::kDS + (cg / 2) * kFPanel + row * 128;
    bool ok = true;

    // Per-row scalars (lse and delta of the tile's 128 queries) come from the producer's loads:
    // global loads of the compute warps would queue behind the dQ reduce traffic on the SM's
    // path to L2, for thousands of clocks. Queries beyond S contribute nothing (p = exp2(-inf)).
    // Keep bits of this thread's 32 key columns for one tile: word cg of the row's record,
    // fetched a tile ahead like the row scalars.
    auto load_keep = [&](bool valid, int q_tile, int k_tile, int bh) -> uint32_t {
      if (DROP != 2 || !valid) return 0u;
      return __ldg(mask_bits + mask_bits_record(bh, q_tile, k_tile, row, n_tiles) * 4 + cg);
    };

    ItemFeed feed{bars, abort_flag, 0};
    int cur = feed.fetch(n_items);
    int nxt = cur < n_items ? feed.fetch(n_items) : n_items;
    uint32_t keep_word = 0u, next_keep = 0u;
    if (DROP == 2 && cur < n_items) {
      const Item t0 = decode_item(cur, BH, n_tiles, group_bh);
      next_keep = load_keep(true, t0.kt, t0.kt, t0.bh);
    }
    int g = 0, j = 0;

    for (; ok && cur < n_items; ++j) {
      const Item t = decode_item(cur, BH, n_tiles, group_bh);
      const int k0 = t.kt * kFT;
      for (int i = 0; i < t.n_it; ++i, ++g) {
        const int q = (t.kt + i) * kFT + row;
        const bool diagonal = (i == 0);
        const int vs = g % kFStages;
        const float* vbuf = reinterpret_cast<const float*>(smem + L::kVec + vs * L::kVecStride);
        if (DROP == 2) {
          // the next tile's keep bits: requested here, first used in that tile
          keep_word = next_keep;
          if (i + 1 < t.n_it) {
            next_keep = load_keep(true, t.kt + i + 1, t.kt, t.bh);
          } else {
            const Item tn = decode_item(nxt < n_items ? nxt : 0, BH, n_tiles, group_bh);
            next_keep = load_keep(nxt < n_items, tn.kt, tn.kt, tn.bh);
          }
        }
        // (one barrier per stage: its next completion needs the stage back from the GEMMs of tile
        // g, hence this thread's own P / dS, so the phase cannot run away from a slow waiter)
        if (!(ok = mbar_wait(&bars->vec_full[vs], (g / kFStages) & 1, abort_flag))) break;
        const int at = t.bh * S + (t.kt + i) * kFT;     // the tile's first row in the [BH, S] vectors
        const bool in = q < S;
        const float row_lse2 = in ? vbuf[((at + lse_shift) & 3) + row] * kFLog2e : INFINITY;
        const float row_delta_s = in ? vbuf[L::kVecDelta / 4 + (at & 3) + row] * scale : 0.f;
        if (!(ok = mbar_wait(&bars->x_full, g & 1, abort_flag))) break;
        tc_fence_after_sync();
        // Sixteen columns at a time: the packed results have to wait in registers for the P / dS
        // buffers, and nothing here may spill (local memory shares the path the reduce-adds load).
        uint32_t pw[16], dw[16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t x1[16], x2[16];
          tmem_ld16(tlane + kColS + cg * 32 + h * 16, x1);
          tmem_ld16(tlane + kColDP + cg * 32 + h * 16, x2);
          tmem_wait_ld();
          if (h == 1) {
            tc_fence_before_sync();
            mbar_arrive(&bars->x_free);  // scores are in registers: the next tile's GEMMs may overwrite
          }
          // ds = p (dP - delta) scale as p * fma(dP, scale, -delta scale), two columns at a time
          // with packed two-float instructions; the causal compare only exists on an item's first
          // (diagonal) tile
          auto pair = [&](int cc, bool masked, uint32_t& pw_, uint32_t& dw_) {
            const int key = k0 + cg * 32 + h * 16 + cc;
            const float2 e = ffma2(make_float2(__uint_as_float(x1[cc]), __uint_as_float(x1[cc + 1])),
                                   make_float2(scale_log2, scale_log2), make_float2(-row_lse2, -row_lse2));
            float2 p = make_float2(ex2(e.x), ex2(e.y));
            if (masked) {
              if (key > q) p.x = 0.f;
              if (key + 1 > q) p.y = 0.f;
            }
            float2 gr = make_float2(__uint_as_float(x2[cc]), __uint_as_float(x2[cc + 1]));
            float2 pd = p;
            if (DROP == 1) {
              const uint64_t idx = (static_cast<uint64_t>(unit0 + t.bh) * S + q) * S + key;
              const float m0 = (p.x != 0.f && philox_keep(rng, idx, rate)) ? keep_scale : 0.f;
              const float m1 = (p.y != 0.f && philox_keep(rng, idx + 1, rate)) ? keep_scale : 0.f;
              pd = fmul2(p, make_float2(m0, m1));
              gr = fmul2(gr, make_float2(m0, m1));
            } else if (DROP == 2) {
              const float m0 = ((keep_word >> (h * 16 + cc)) & 1u) ? keep_scale : 0.f;
              const float m1 = ((keep_word >> (h * 16 + cc + 1)) & 1u) ? keep_scale : 0.f;
              pd = fmul2(p, make_float2(m0, m1));
              gr = fmul2(gr, make_float2(m0, m1));
            }
            const float2 ds = fmul2(p, ffma2(gr, make_float2(scale, scale), make_float2(-row_delta_s, -row_delta_s)));
            pw_ = pack_bf16(pd.x, pd.y);
            dw_ = pack_bf16(ds.x, ds.y);
          };
          if (diagonal) {
#pragma unroll
            for (int cc = 0; cc < 16; cc += 2) pair(cc, true, pw[h * 8 + cc / 2], dw[h * 8 + cc / 2]);
          } else {
#pragma unroll
            for (int cc = 0; cc < 16; cc += 2) pair(cc, false, pw[h * 8 + cc / 2], dw[h * 8 + cc / 2]);
          }
        }
        // P / dS of tile g-1 consumed and its dQ complete in tensor memory
        if (g > 0) {
          if (!(ok = mbar_wait(&bars->acc_done, (g - 1) & 1, abort_flag))) break;
          tc_fence_after_sync();
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const int chunk = (cg & 1) * 4 + v4;  // 16-byte chunk within the 128-byte row of the panel
          const int off = (chunk ^ (row & 7)) << 4;
          *reinterpret_cast<uint4*>(p_row + off) =
              make_uint4(pw[4 * v4], pw[4 * v4 + 1], pw[4 * v4 + 2], pw[4 * v4 + 3]);
          *reinterpret_cast<uint4*>(ds_row + off) =
              make_uint4(dw[4 * v4], dw[4 * v4 + 1], dw[4 * v4 + 2], dw[4 * v4 + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(&bars->w_full);
      }
      cur = nxt;
      nxt = (ok && cur < n_items) ? feed.fetch(n_items) : n_items;
    }

  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == kWarpIssuer) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (threadIdx.x == 0 && bars->abort_flag) report_timeout(status, bars->abort_flag);
}

// delta[r] = sum_d dO[r,d] O[r,d] (reference flash_delta_kernel, cuda/attention.cu:76-85) and the
// zero fill of the fp32 dQ workspace, in one pass over the rows. The zero fill does not depend on
// the kernel before this one in the stream (normally the forward pass), so it runs ahead of the
// dependency wait and overlaps that kernel's tail. The only kernel that reads the workspace,
// fused_convert_kernel, releases its dependents after its reads.
template <bool INTERLEAVED>
__global__ void fused_prepare_kernel(float* __restrict__ delta, float* __restrict__ dq_ws,
                                     int* __restrict__ item_counter,
                                     const __nv_bfloat16* __restrict__ dout,
                                     const __nv_bfloat16* __restrict__ out, int64_t rows, int S,
                                     UnitLayout lay) {
  constexpr int D = kFD, Lr = D / 8;  // 8 lanes per row
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = t / Lr;   // row of the [BH, S] index space: delta and the workspace are heads-split
  const int c = static_cast<int>(t % Lr) * 8;
  if (r < rows) {
    float4* z = reinterpret_cast<float4*>(dq_ws + r * D + c);
    z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (t == 0) *item_counter = 0;
  pdl_wait();
  pdl_launch_dependents();
  float sum = 0.f;
  if (r < rows) {
    // where row r = (unit, s) lies in dO and O: heads-split rows are simply consecutive
    int64_t at = r * D + c;
    if (INTERLEAVED) {
      const int unit = static_cast<int>(r / S), srow = static_cast<int>(r - static_cast<int64_t>(unit) * S);
      const int ub = unit / lay.heads, uh = unit - ub * lay.heads;
      at = ub * lay.batch + uh * lay.head + srow * lay.row + c;
    }
    const uint4 a = *reinterpret_cast<const uint4*>(dout + at);
    const uint4 b = *reinterpret_cast<const uint4*>(out + at);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sum = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(bw[i] << 16), sum);
      sum = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(bw[i] & 0xffff0000u), sum);
    }
  }
#pragma unroll
  for (int o = Lr / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (r < rows && c == 0) delta[r] = sum;
}

// dQ workspace (fp32) -> dq (bf16). Dependents are released only after the workspace has been
// read: the next backward call's prepare kernel clears it ahead of its own dependency wait.
template <bool INTERLEAVED>
__global__ void fused_convert_kernel(__nv_bfloat16* __restrict__ dq, const float* __restrict__ dq_ws,
                                     int64_t n8, int S, UnitLayout lay) {
  pdl_wait();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
  if (t < n8) {
    a = *reinterpret_cast<const float4*>(dq_ws + t * 8);
    b = *reinterpret_cast<const float4*>(dq_ws + t * 8 + 4);
  }
  // the loads have returned once their values are used; keep the trigger behind that use
  const uint4 w = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
  if (t < n8) {
    // workspace row r = (unit, s), 8 elements at column c; heads-split dq has the same order
    int64_t at = t * 8;
    if (INTERLEAVED) {
      const int64_t r = t / (kFD / 8);
      const int c = static_cast<int>(t - r * (kFD / 8)) * 8;
      const int unit = static_cast<int>(r / S), srow = static_cast<int>(r - static_cast<int64_t>(unit) * S);
      const int ub = unit / lay.heads, uh = unit - ub * lay.heads;
      at = ub * lay.batch + uh * lay.head + srow * lay.row + c;
    }
    *reinterpret_cast<uint4*>(dq + at) = w;
  }
  pdl_launch_dependents();
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 3-D map over the fp32 workspace [BH, S, 64] with a 32 x 128 x 1 box and 128-byte swizzle
int make_dq_workspace_map(CUtensorMap* map, float* ws, int BH, int S) {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  if (!fn) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[3] = {kFD, static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(BH)};
  const cuuint64_t strides[2] = {kFD * 4, static_cast<cuuint64_t>(S) * kFD * 4};
  const cuuint32_t box[3] = {32, kFT, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, ws, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return DADATTN_OK;
}

// A [n] fp32 vector of per-row scalars as a 1-D map with boxes of kVecBox words. `base` need not
// be 16-byte aligned: the map starts at the boundary below it and *shift is the number of words
// in between, which the kernel adds to its row index.
int make_row_scalar_map(CUtensorMap* map, const float* base, int64_t n, int* shift) {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  if (!fn) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const uintptr_t addr = reinterpret_cast<uintptr_t>(base);
  if (addr % 4) return fail(DADATTN_E_ARG, "a float vector is not 4-byte aligned");
  *shift = static_cast<int>((addr % 16) / 4);
  const cuuint64_t dims[1] = {static_cast<cuuint64_t>(n + *shift)};
  const cuuint64_t strides[1] = {0};   // unused with one dimension
  const cuuint32_t box[1] = {kVecBox};
  const cuuint32_t estr[1] = {1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 1, reinterpret_cast<void*>(addr - addr % 16), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return DADATTN_OK;
}

}  // namespace
}  // namespace dadattn
namespace dadattn {

// Workspace: delta [BH,S] fp32, then the dQ accumulator [BH,S,64] fp32 (256-byte aligned), then
// 256 bytes that hold the work-item counter.
size_t fused_bwd_workspace_bytes(int BH, int S) {
  const size_t delta_bytes = (static_cast<size_t>(BH) * S * sizeof(float) + 255) / 256 * 256;
  const size_t dq_bytes = (static_cast<size_t>(BH) * S * kFD * sizeof(float) + 255) / 256 * 256;
  return delta_bytes + dq_bytes + 256;
}

int launch_bwd_fused_d64(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace, const uint16_t* dout,
                         const uint16_t* out, const float* lse, const uint16_t* q, const uint16_t* k,
                         const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                         uint64_t offset, int64_t unit0, const uint32_t* mask_bits, int heads,
                         cudaStream_t st) {
  using BF = __nv_bfloat16;
  // heads > 0: every bf16 tensor is the interleaved [B*S, heads*64] activation (BH = B * heads)
  const UnitLayout lay = heads > 0 ? unit_layout(BH / heads, heads, S, kFD, true) : unit_layout(BH, 1, S, kFD, false);
  const size_t delta_bytes = (static_cast<size_t>(BH) * S * sizeof(float) + 255) / 256 * 256;
  const size_t dq_bytes = (static_cast<size_t>(BH) * S * kFD * sizeof(float) + 255) / 256 * 256;
  float* delta = static_cast<float*>(workspace);
  float* dq_ws = reinterpret_cast<float*>(static_cast<char*>(workspace) + delta_bytes);
  int* item_counter = reinterpret_cast<int*>(static_cast<char*>(workspace) + delta_bytes + dq_bytes);
  CUtensorMap mq, mk, mv, mdo, mws, mdk, mdv, mlse, mdelta;
  int lse_shift = 0, delta_shift = 0;   // the workspace is 256-byte aligned: delta needs none
  if (int rc = make_tensor_map_bf16_units(&mq, q, BH, S, kFD, kFT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mk, k, BH, S, kFD, kFT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mv, v, BH, S, kFD, kFT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mdo, dout, BH, S, kFD, kFT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mdk, dk, BH, S, kFD, kFT, lay)) return rc;
  if (int rc = make_tensor_map_bf16_units(&mdv, dv, BH, S, kFD, kFT, lay)) return rc;
  if (int rc = make_dq_workspace_map(&mws, dq_ws, BH, S)) return rc;
  // (the kernel indexes the [BH, S] vectors with 32-bit TMA coordinates)
  if (static_cast<int64_t>(BH) * S > INT32_MAX - 1024)
    return fail(DADATTN_E_UNSUPPORTED, "BH * S = %lld rows exceed what the fused backward addresses",
                static_cast<long long>(BH) * S);
  if (int rc = make_row_scalar_map(&mlse, lse, static_cast<int64_t>(BH) * S, &lse_shift)) return rc;
  if (int rc = make_row_scalar_map(&mdelta, delta, static_cast<int64_t>(BH) * S, &delta_shift)) return rc;
  if (delta_shift != 0) return fail(DADATTN_E_ARG, "the backward workspace is not 16-byte aligned");
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;

  const int64_t rows = static_cast<int64_t>(BH) * S;
  const int64_t prep_threads = rows * (kFD / 8);
  stage_event(0, st);
  DAD_CUDA(launch_pdl(heads > 0 ? fused_prepare_kernel<true> : fused_prepare_kernel<false>,
                      dim3(static_cast<unsigned>((prep_threads + 255) / 256)),
                      dim3(256), 0, st, delta, dq_ws, item_counter, reinterpret_cast<const BF*>(dout),
                      reinterpret_cast<const BF*>(out), rows, S, lay));
  stage_event(1, st);
  const PhiloxKey rng = make_philox(seed, offset);
  // One persistent CTA per SM; the CTAs draw (key tile, batch x head) items from a counter.
  // Batch x head units are worked on in groups whose Q, dO and dQ rows (1 KiB per query) stay
  // well inside L2.
  const int64_t n_items = static_cast<int64_t>((S + kFT - 1) / kFT) * BH;
  if (n_items > INT32_MAX / 2) return fail(DADATTN_E_UNSUPPORTED, "too many (key tile, batch x head) items");
  int dev = 0, sms = 0;
  DAD_CUDA(cudaGetDevice(&dev));
  DAD_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  dim3 grid(static_cast<unsigned>(n_items < sms ? n_items : sms));
  int group_bh = 65536 / S;
  group_bh = group_bh < 1 ? 1 : (group_bh > 64 ? 64 : group_bh);
  auto kern = rate > 0.f ? (mask_bits ? flash_bwd_fused_kernel<2> : flash_bwd_fused_kernel<1>)
                         : flash_bwd_fused_kernel<0>;
  DAD_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FusedSmem::kBytes));
  // The warpgroups' register budgets add up to what a CTA is launched with only if the compiler
  // gave the kernel kRegsLaunch registers per thread; with fewer, the compute warps' increase
  // would wait for registers that nobody can give back. Refuse rather than hang.
  static int regs_seen[3] = {0, 0, 0};   // per kernel variant; the same value for every device
  int& regs = regs_seen[rate > 0.f ? (mask_bits ? 2 : 1) : 0];
  if (regs == 0) {
    cudaFuncAttributes fattr;
    DAD_CUDA(cudaFuncGetAttributes(&fattr, kern));
    regs = fattr.numRegs;
  }
  if (regs != kRegsLaunch)
    return fail(DADATTN_E_UNSUPPORTED, "the single-pass backward was compiled with %d registers per thread, "
                "its register budgets assume %d", regs, kRegsLaunch);
  DAD_CUDA(launch_pdl(kern, grid, dim3(kFThreads), FusedSmem::kBytes, st, mq, mk, mv, mdo, mws, mdk, mdv,
                      mlse, mdelta, lse_shift, item_counter, BH, S, lay.heads, group_bh, scale, rate,
                      rng, unit0, mask_bits, status));
  stage_event(2, st);
  const int64_t n8 = rows * kFD / 8;
  DAD_CUDA(launch_pdl(heads > 0 ? fused_convert_kernel<true> : fused_convert_kernel<false>,
                      dim3(static_cast<unsigned>((n8 + 255) / 256)), dim3(256), 0,
                      st, reinterpret_cast<BF*>(dq), static_cast<const float*>(dq_ws), n8, S, lay));
  stage_event(3, st);
  return DADATTN_OK;
}

}  // namespace dadattn
