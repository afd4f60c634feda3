// bf16 fused causal attention backward for sm_100a, head size 128: dQ, dK and dV in ONE pass.
//
// The two-kernel backward of flash_bwd_bf16_sm100.cu follows the reference (cuda/attention.cu:
// 88-205) in computing the probabilities twice: 7 GEMM-sized products for 5 gradients' worth.
// Here a CTA owns 128 keys of one (batch, head) and streams the 64-query sub-tiles that can see
// them. Rows of the score tile are keys (one TMEM lane each):
//     S^T = K Q^T,  dP^T = V dO^T                       128 keys x 64 queries, fp32 in TMEM
//     p = exp2(S^T scale log2e - lse[q] log2e),  ds = p (dP^T - delta[q]) scale
//     dV += P^T-tile dO      dK += dS^T-tile Q          accumulate in TMEM over the whole loop
//     dQ^T-tile = K^T dS^T                              128 head dims x 64 queries, per step
// P^T and dS^T go back into tensor memory as packed bf16 and are the A operands of dV / dK from
// there (tcgen05.mma with A in TMEM): an MMA with both operands in shared memory reads them at
// 128 B/clk, and with the TMA loads, the stores and the dQ staging the shared-memory traffic of
// a step (336 KB when P^T / dS^T lived there), not the tensor core, set the step time. dS^T is
// also written, bf16, [key][query] in the 128-byte swizzled layout, as the MN-major B operand
// of dQ^T, whose A operand is the resident K tile read MN-major. Computing dQ transposed keeps
// all 128 TMEM lanes busy (M = 128 head dims) although a step has only 64 queries.
// Each step's dQ^T tile (32 KB fp32) goes TMEM -> staging in shared memory -> bulk reduce-add
// into an fp32 workspace laid out tile by tile ([BH][64-query block][128 dims][64 queries], rows
// swizzled as staged), which a last pass transposes and rounds to bf16. The sums into the
// workspace happen in whatever order the CTAs reach them, so dQ may differ in its last bits from
// run to run; dadattn_set_bwd_deterministic(1) selects the two-kernel path.
//   warp 0      TMA producer          warp 1      MMA issuer + TMEM owner
//   warps 2-17  compute: four warps per TMEM lane quadrant, each taking 16 of the 64 query columns
//   warp 18     dQ reducer
#include <cuda_bf16.h>

#include <cfloat>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace dadattn {
namespace {

using namespace ptx;

constexpr int kGD = 128;                   // head size
constexpr int kGKeys = 128;                // keys owned by a CTA
constexpr int kGSub = 64;                  // queries per step
constexpr int kGPanel = 128 * 128;         // [128 rows][64 bf16] swizzled panel
constexpr int kGSubPanel = 64 * 128;       // [64 rows][64 bf16] swizzled panel
constexpr int kGStages = 3;                // streamed-tile ring depth
constexpr int kGThreads = 19 * 32;
constexpr int kGCompute = 16 * 32;
constexpr int kGDqTileBytes = kGD * kGSub * 4;   // one dQ^T tile, fp32
constexpr float kGLog2e = 1.4426950408889634f;

struct G128Smem {
  static constexpr int kTile = 2 * kGPanel;        // resident [128, 128] tile
  static constexpr int kSubTile = 2 * kGSubPanel;  // streamed [64, 128] tile
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;
  static constexpr int kDO = kQ + kGStages * kSubTile;
  static constexpr int kDS = kDO + kGStages * kSubTile;  // [128 keys][64 q] bf16, one panel
  static constexpr int kDQ = kDS + kGPanel;              // [128 dims][64 q] fp32 staging
  static constexpr int kVec = kDQ + kGDqTileBytes;       // lse*log2e, delta: 2 x [2][64] fp32
  static constexpr int kBars = kVec + 2 * 2 * 64 * 4;
  static constexpr int kBytes = kBars + 256;
  static_assert(kBytes <= 232448, "shared memory budget of one CTA exceeded");
};

struct G128Bars {
  uint64_t kv_full, q_full[kGStages], do_full[kGStages], qdo_empty[kGStages];
  uint64_t x_full, x_free, w_full, acc_done, vec_full, dq_drained, dq_staged, dq_sent;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit_g() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0_g() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait0_g() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};"
               ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(taddr)
               : "memory");
}
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

// 16-byte chunk `c` (0..15) of staging / workspace row `row` (256 bytes = 64 fp32) sits at chunk
// c ^ (row & 15): a warp writing one chunk of 32 consecutive rows then spreads over all banks.
__host__ __device__ __forceinline__ int dq_chunk(int c, int row) { return c ^ (row & 15); }

template <bool DROP>
__global__ void __launch_bounds__(kGThreads, 1)
flash_bwd_fused128_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                          __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                          float* __restrict__ dq_ws, const float* __restrict__ lse,
                          const float* __restrict__ delta, int S, float scale, float rate,
                          PhiloxKey rng, int64_t unit0, int* __restrict__ status) {
  using L = G128Smem;
  constexpr int D = kGD;
  constexpr uint32_t kTmemCols = 512;
  // S^T, dP^T (fp32, 64 columns each), dV, dK (128 each), dQ^T (64), then P^T and dS^T as packed
  // bf16 (two queries per column: 32 columns each)
  constexpr uint32_t kColS = 0, kColDP = 64, kColDV = 128, kColDK = 256, kColDQ = 384;
  constexpr uint32_t kColP = 448, kColDSt = 480;

  extern __shared__ __align__(1024) uint8_t smem[];
  G128Bars* bars = reinterpret_cast<G128Bars*>(smem + L::kBars);
  volatile int* abort_flag = &bars->abort_flag;
  float* vec = reinterpret_cast<float*>(smem + L::kVec);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n_sub = (S + kGSub - 1) / kGSub;
  const int bh = blockIdx.y;
  // key tile `own` streams the query sub-tiles 2*own .. n_sub-1 (low `own` = most work = first)
  const int own = static_cast<int>(blockIdx.x);
  const int first = 2 * own;
  const int n_it = n_sub - first;
  const int k0 = own * kGKeys;

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicExch(status, DADATTN_E_CUDA);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < kGStages; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->do_full[s], 1);
      mbar_init(&bars->qdo_empty[s], 1);
    }
    mbar_init(&bars->x_full, 1);
    mbar_init(&bars->x_free, kGCompute);
    mbar_init(&bars->w_full, kGCompute);
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->vec_full, kGCompute);
    mbar_init(&bars->dq_drained, kGCompute);
    mbar_init(&bars->dq_staged, kGCompute);
    mbar_init(&bars->dq_sent, 1);
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
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      prefetch_tensormap(&map_k);
      prefetch_tensormap(&map_v);
      prefetch_tensormap(&map_q);
      prefetch_tensormap(&map_do);
      mbar_arrive_expect_tx(&bars->kv_full, 2 * L::kTile);
      for (int p = 0; p < 2; ++p) {
        tma_load_3d(smem + L::kK + p * kGPanel, &map_k, &bars->kv_full, p * 64, k0, bh);
        tma_load_3d(smem + L::kV + p * kGPanel, &map_v, &bars->kv_full, p * 64, k0, bh);
      }
      for (int i = 0; i < n_it; ++i) {
        const int s = i % kGStages, use = i / kGStages;
        if (use > 0 && !mbar_wait(&bars->qdo_empty[s], (use - 1) & 1, abort_flag)) break;
        const int q0 = (first + i) * kGSub;
        mbar_arrive_expect_tx(&bars->q_full[s], L::kSubTile);
        for (int p = 0; p < 2; ++p)
          tma_load_3d(smem + L::kQ + s * L::kSubTile + p * kGSubPanel, &map_q, &bars->q_full[s],
                      p * 64, q0, bh);
        mbar_arrive_expect_tx(&bars->do_full[s], L::kSubTile);
        for (int p = 0; p < 2; ++p)
          tma_load_3d(smem + L::kDO + s * L::kSubTile + p * kGSubPanel, &map_do, &bars->do_full[s],
                      p * 64, q0, bh);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_x = make_idesc_bf16(128, 64, 0, 0);    // S^T, dP^T: both K-major
      constexpr uint32_t idesc_a = make_idesc_bf16(128, D, 0, 1);     // dV, dK: B MN-major
      constexpr uint32_t idesc_q = make_idesc_bf16(128, 64, 1, 1);    // dQ^T: A and B MN-major
      const SmemDescBase k_kmaj = make_desc_base_sw128(smem_u32(smem + L::kK), 0);
      const SmemDescBase v_kmaj = make_desc_base_sw128(smem_u32(smem + L::kV), 0);
      // K read as MN-major A (M = head dims): the two 64-dim panels are kGPanel apart
      const SmemDescBase k_mn = make_desc_base_sw128(smem_u32(smem + L::kK), kGPanel);
      const SmemDescBase ds_desc = make_desc_base_sw128(smem_u32(smem + L::kDS), 0);
      // streamed tiles: K-major B of the score GEMMs, MN-major B (panels kGSubPanel apart) of dV / dK
      const SmemDescBase q_desc0 = make_desc_base_sw128(smem_u32(smem + L::kQ), kGSubPanel);
      const SmemDescBase do_desc0 = make_desc_base_sw128(smem_u32(smem + L::kDO), kGSubPanel);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_flag);

      auto issue_x = [&](int i) -> bool {
        const int s = i % kGStages;
        const uint32_t par = (i / kGStages) & 1;
        const SmemDescBase qd{q_desc0.lo + s * (L::kSubTile >> 4), q_desc0.hi};
        const SmemDescBase dd{do_desc0.lo + s * (L::kSubTile >> 4), do_desc0.hi};
        if (!mbar_wait(&bars->q_full[s], par, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem + kColS, desc_at(k_kmaj, (kk / 4) * kGPanel + (kk % 4) * 32),
                 desc_at(qd, (kk / 4) * kGSubPanel + (kk % 4) * 32), idesc_x, kk > 0 ? 1u : 0u);
        if (!mbar_wait(&bars->do_full[s], par, abort_flag)) return false;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          mma_ss(tmem + kColDP, desc_at(v_kmaj, (kk / 4) * kGPanel + (kk % 4) * 32),
                 desc_at(dd, (kk / 4) * kGSubPanel + (kk % 4) * 32), idesc_x, kk > 0 ? 1u : 0u);
        mma_commit(&bars->x_full);
        return true;
      };
      auto issue_acc = [&](int i) -> bool {
        const int s = i % kGStages;
        const SmemDescBase qd{q_desc0.lo + s * (L::kSubTile >> 4), q_desc0.hi};
        const SmemDescBase dd{do_desc0.lo + s * (L::kSubTile >> 4), do_desc0.hi};
        if (!mbar_wait(&bars->w_full, i & 1, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kGSub / 16; ++kk) {   // K dimension = 64 queries, 16 per MMA
          const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
          mma_ts(tmem + kColDV, tmem + kColP + kk * 8, desc_at(dd, kk * 2048), idesc_a, acc);
          mma_ts(tmem + kColDK, tmem + kColDSt + kk * 8, desc_at(qd, kk * 2048), idesc_a, acc);
        }
        // the previous step's dQ^T must have left tensor memory before this one overwrites it;
        // the compute warps read it right after they publish P^T / dS^T, while dV / dK are running
        if (i > 0 && !mbar_wait(&bars->dq_drained, (i - 1) & 1, abort_flag)) return false;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < kGKeys / 16; ++kk)    // K dimension = 128 keys
          mma_ss(tmem + kColDQ, desc_at(k_mn, kk * 2048), desc_at(ds_desc, kk * 2048), idesc_q,
                 kk > 0 ? 1u : 0u);
        mma_commit(&bars->qdo_empty[s]);
        mma_commit(&bars->acc_done);
        return true;
      };

      ok = ok && issue_x(0);
      for (int i = 0; ok && i < n_it; ++i) {
        // the next step's score GEMMs go first: the arithmetic on them overlaps this step's
        // accumulating GEMMs
        if (i + 1 < n_it) ok = mbar_wait(&bars->x_free, i & 1, abort_flag) && issue_x(i + 1);
        ok = ok && issue_acc(i);
      }
    }
  } else if (warp == 18) {
    // ------------------------------ dQ reducer ------------------------------
    if (elect_one()) {
      for (int i = 0; i < n_it; ++i) {
        if (!mbar_wait(&bars->dq_staged, i & 1, abort_flag)) break;
        float* dst = dq_ws + (static_cast<size_t>(bh) * n_sub + first + i) * (kGD * kGSub);
        bulk_reduce_add_f32(dst, smem + L::kDQ, kGDqTileBytes);
        bulk_commit_g();
        bulk_wait_read0_g();
        mbar_arrive(&bars->dq_sent);
      }
      bulk_wait0_g();   // every sum has landed before the CTA retires
    }
  } else {
    // ------------------------------ compute warps ------------------------------
    const int cw = warp - 2;              // 0..15
    const int quad = warp % 4;            // TMEM lane quadrant of this warp
    const int cg = cw / 4;                // which 16 query columns of the 64
    const int ct = cw * 32 + lane;        // 0..511 among the compute threads
    const int row = quad * 32 + lane;     // key within the tile (and head dim of dQ^T) = TMEM lane
    const int key = k0 + row;
    const uint32_t tlane = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const float scale_log2 = scale * kGLog2e;
    const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;
    const size_t vec_base = static_cast<size_t>(bh) * S;
    uint8_t* ds_row = smem + L::kDS + row * 128;
    uint8_t* dq_row = smem + L::kDQ + row * 256;
    bool ok = true;
    // Per-column vectors (lse log2e and delta of the step's 64 queries): threads 0-127 fetch
    // them one step ahead into a register and publish them through one of two shared-memory
    // buffers, so that neither the global load nor a buffer hand-over sits in the step's chain.
    auto fetch_vec = [&](int i) -> float {
      const int qv = (first + i) * kGSub + (ct & 63);
      if (ct >= 128 || i >= n_it || qv >= S) return ct < 64 ? INFINITY : 0.f;
      return ct < 64 ? lse[vec_base + qv] * kGLog2e : delta[vec_base + qv];
    };
    float next_vec = fetch_vec(0);

    // dQ^T of step t: TMEM [128 dims][64 q] -> staging (rows swizzled), which the reducer sends
    // on. The caller has seen acc_done of step t.
    auto drain_dq = [&](int t) -> bool {
      uint32_t o[16];
      tmem_ld16(tlane + kColDQ + cg * 16, o);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&bars->dq_drained);
      // the reduce of the previous step must have finished reading the staging buffer
      if (t > 0 && !mbar_wait(&bars->dq_sent, (t - 1) & 1, abort_flag)) return false;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        *reinterpret_cast<uint4*>(dq_row + (dq_chunk(cg * 4 + c, row) << 4)) =
            make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
      fence_proxy_async_smem();
      mbar_arrive(&bars->dq_staged);
      return true;
    };

    for (int i = 0; i < n_it; ++i) {
      const int q0 = (first + i) * kGSub;
      const bool diagonal = i < 2;   // sub-tiles that straddle the diagonal need the comparison
      // Buffer i % 2 was last read in step i-2, and every thread finished that step before it
      // arrived at vec_full(i-1), which this thread has already seen complete.
      float* v_lse = vec + (i & 1) * 128;
      float* v_delta = v_lse + 64;
      if (ct < 128) v_lse[ct] = next_vec;   // threads 64-127 land in v_delta
      next_vec = fetch_vec(i + 1);
      mbar_arrive(&bars->vec_full);
      if (!(ok = mbar_wait(&bars->vec_full, i & 1, abort_flag))) break;
      if (!(ok = mbar_wait(&bars->x_full, i & 1, abort_flag))) break;
      tc_fence_after_sync();

      const int cbase = cg * 16;
      uint32_t x1[16], x2[16];
      tmem_ld16(tlane + kColS + cbase, x1);
      tmem_ld16(tlane + kColDP + cbase, x2);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(&bars->x_free);  // scores are in registers: the next step's GEMMs may overwrite

      uint32_t pw[8], dw[8];
#pragma unroll
      for (int c = 0; c < 16; c += 4) {
        // 128-bit broadcast reads: all lanes of a warp want the same four columns
        const float4 a = *reinterpret_cast<const float4*>(v_lse + cbase + c);
        const float4 b = *reinterpret_cast<const float4*>(v_delta + cbase + c);
        const float l2[4] = {a.x, a.y, a.z, a.w}, dl[4] = {b.x, b.y, b.z, b.w};
        float pv[4], dv4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int query = q0 + cbase + c + e;
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
          dv4[e] = p * (g - dl[e]) * scale;
        }
        pw[c / 2] = pack_bf16(pv[0], pv[1]);
        pw[c / 2 + 1] = pack_bf16(pv[2], pv[3]);
        dw[c / 2] = pack_bf16(dv4[0], dv4[1]);
        dw[c / 2 + 1] = pack_bf16(dv4[2], dv4[3]);
      }
      // P^T / dS^T of step i-1 consumed and its dQ^T complete in tensor memory
      if (i > 0) {
        if (!(ok = mbar_wait(&bars->acc_done, (i - 1) & 1, abort_flag))) break;
        tc_fence_after_sync();
      }
      // sixteen queries = eight packed columns = one K step of the dV / dK MMAs
      tmem_st8(tlane + kColP + cg * 8, pw);
      tmem_st8(tlane + kColDSt + cg * 8, dw);
#pragma unroll
      for (int v4 = 0; v4 < 2; ++v4) {
        const int chunk = cg * 2 + v4;    // 16-byte chunk within the 128-byte row
        const int off = (chunk ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(ds_row + off) =
            make_uint4(dw[4 * v4], dw[4 * v4 + 1], dw[4 * v4 + 2], dw[4 * v4 + 3]);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive(&bars->w_full);
      if (i > 0 && !(ok = drain_dq(i - 1))) break;
    }

    // the last step's dQ^T, then dV (column groups 0, 1) and dK (2, 3), 64 head dims each
    if (ok && (ok = mbar_wait(&bars->acc_done, (n_it - 1) & 1, abort_flag))) {
      tc_fence_after_sync();
      ok = drain_dq(n_it - 1);
    }
    if (ok) {
      __nv_bfloat16* dst = (cg < 2 ? dv : dk) + (vec_base + key) * D + (cg & 1) * 64;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld32(tlane + (cg < 2 ? kColDV : kColDK) + (cg & 1) * 64 + c * 32, o);
        tmem_wait_ld();
        if (key < S) {
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

// delta[r] = sum_d dO[r,d] O[r,d] (reference flash_delta_kernel, cuda/attention.cu:76-85): 16
// lanes per row of 128.
__global__ void fused128_delta_kernel(float* __restrict__ delta, const __nv_bfloat16* __restrict__ dout,
                                      const __nv_bfloat16* __restrict__ out, int64_t rows) {
  constexpr int D = kGD, Lr = D / 8;
  pdl_wait();
  pdl_launch_dependents();
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t r = t / Lr;
  const int c = static_cast<int>(t % Lr) * 8;
  float sum = 0.f;
  if (r < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(dout + r * D + c);
    const uint4 b = *reinterpret_cast<const uint4*>(out + r * D + c);
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

// Workspace tile [128 dims][64 queries] fp32 (rows swizzled as staged) -> dq[q][128] bf16.
// One CTA of 256 threads per tile: thread t takes query t % 64 and 32 head dims.
__global__ void fused128_convert_kernel(__nv_bfloat16* __restrict__ dq, const float* __restrict__ dq_ws,
                                        int S, int n_sub) {
  pdl_wait();
  const int bh = blockIdx.y, blk = blockIdx.x;
  const float* tile = dq_ws + (static_cast<size_t>(bh) * n_sub + blk) * (kGD * kGSub);
  const int qi = threadIdx.x % 64, dg = threadIdx.x / 64;
  const int q = blk * kGSub + qi;
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const int d0 = dg * 32 + j, d1 = d0 + 1;
    const float a = tile[d0 * 64 + (dq_chunk(qi / 4, d0) << 2) + (qi & 3)];
    const float b = tile[d1 * 64 + (dq_chunk(qi / 4, d1) << 2) + (qi & 3)];
    w[j / 2] = pack_bf16(a, b);
  }
  if (q < S) {
    uint4* dst = reinterpret_cast<uint4*>(dq + (static_cast<size_t>(bh) * S + q) * kGD + dg * 32);
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
  }
  pdl_launch_dependents();
}

}  // namespace

// Workspace: delta [BH,S] fp32 (padded to 256 bytes), then the dQ^T accumulator
// [BH][ceil(S/64)][128][64] fp32.
size_t fused128_bwd_workspace_bytes(int BH, int S) {
  const size_t delta_bytes = (static_cast<size_t>(BH) * S * sizeof(float) + 255) / 256 * 256;
  const size_t n_sub = (static_cast<size_t>(S) + kGSub - 1) / kGSub;
  return delta_bytes + static_cast<size_t>(BH) * n_sub * kGDqTileBytes;
}

int launch_bwd_fused_d128(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace, const uint16_t* dout,
                          const uint16_t* out, const float* lse, const uint16_t* q, const uint16_t* k,
                          const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                          uint64_t offset, int64_t unit0, cudaStream_t st) {
  using BF = __nv_bfloat16;
  const size_t delta_bytes = (static_cast<size_t>(BH) * S * sizeof(float) + 255) / 256 * 256;
  const int n_sub = (S + kGSub - 1) / kGSub;
  float* delta = static_cast<float*>(workspace);
  float* dq_ws = reinterpret_cast<float*>(static_cast<char*>(workspace) + delta_bytes);
  CUtensorMap mk, mv, mq, mdo;
  if (int rc = make_tensor_map_bf16(&mk, k, BH, S, kGD, kGKeys)) return rc;
  if (int rc = make_tensor_map_bf16(&mv, v, BH, S, kGD, kGKeys)) return rc;
  if (int rc = make_tensor_map_bf16(&mq, q, BH, S, kGD, kGSub)) return rc;
  if (int rc = make_tensor_map_bf16(&mdo, dout, BH, S, kGD, kGSub)) return rc;
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;

  stage_event(0, st);
  DAD_CUDA(cudaMemsetAsync(dq_ws, 0, static_cast<size_t>(BH) * n_sub * kGDqTileBytes, st));
  const int64_t rows = static_cast<int64_t>(BH) * S;
  const int64_t threads = rows * (kGD / 8);
  DAD_CUDA(launch_pdl(fused128_delta_kernel, dim3(static_cast<unsigned>((threads + 255) / 256)), dim3(256),
                      0, st, delta, reinterpret_cast<const BF*>(dout), reinterpret_cast<const BF*>(out),
                      rows));
  stage_event(1, st);
  const PhiloxKey rng = make_philox(seed, offset);
  dim3 grid((S + kGKeys - 1) / kGKeys, BH);
  const bool drop = rate > 0.f;
  auto kern = drop ? flash_bwd_fused128_kernel<true> : flash_bwd_fused128_kernel<false>;
  DAD_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, G128Smem::kBytes));
  DAD_CUDA(launch_pdl(kern, grid, dim3(kGThreads), G128Smem::kBytes, st, mk, mv, mq, mdo,
                      reinterpret_cast<BF*>(dk), reinterpret_cast<BF*>(dv), dq_ws, lse,
                      static_cast<const float*>(delta), S, scale, rate, rng, unit0, status));
  stage_event(2, st);
  DAD_CUDA(launch_pdl(fused128_convert_kernel, dim3(n_sub, BH), dim3(256), 0, st,
                      reinterpret_cast<BF*>(dq), static_cast<const float*>(dq_ws), S, n_sub));
  stage_event(3, st);
  return DADATTN_OK;
}

}  // namespace dadattn
