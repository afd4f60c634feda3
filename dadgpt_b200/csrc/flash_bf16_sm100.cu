// bf16 fused causal attention for sm_100a: TMA-staged tiles, tcgen05 MMAs accumulating in tensor
// memory, a warp-specialised online-softmax pipeline. The arithmetic is that of the reference's
// fused kernels (cuda/attention.cu) with bf16 operands and fp32 accumulation; the interface is
// its gpu_flash_attention_forward / _backward with bf16 pointers (include/dadattn.h).
//
// Forward, one CTA per 128 query rows of one (batch, head):
//   warp 0      TMA producer: Q once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 1      MMA issuer (one elected lane) and owner of the TMEM allocation:
//               S = Q K^T (128x128, fp32 in TMEM), O_h += P_h V_h per 64-key half h
//   warps 2-9   softmax, two threads per query row: warps 2-5 own key columns 0-63 of every
//               tile, warps 6-9 columns 64-127 (a warp may only touch the TMEM lane quadrant
//               warp_id % 4). Each half keeps its OWN running max / sum and its OWN output
//               accumulator in TMEM, so the two threads of a row never synchronise inside the
//               loop; the halves are merged once, in the epilogue (split-K inside the CTA).
//               Eight softmax warps give every scheduler two (four with two CTAs per SM) warps
//               to hide the FFMA -> MUFU -> FADD latencies behind each other.
//               A thread reads its 64 scores with tcgen05.ld, writes P as bf16 into shared
//               memory in the 128-byte-swizzled layout the MMA reads, and rescales its O half
//               in TMEM only when its max grew by more than 2^8 (lazy rescale; exact result).
// S_{j+1} is issued before P_j V_j, so the tensor core works on the next tile while the
// exponentials of the current one are computed; at D = 64 two CTAs share an SM, at D = 128 the
// scores are double-buffered in TMEM instead.
//
// The kernel template takes head sizes 64 and 128; the library instantiates it for 128 only: head
// size 64 is served by the persistent two-tile kernel of flash_fwd64_sm100.cu.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh). If one runs out, the CTA raises its abort
// flag, everybody falls through to the common exit, TMEM is freed, and DADATTN_E_TIMEOUT is
// left in the device status word.
#include <cuda_bf16.h>

#include <cfloat>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace dadattn {

// ---------------------------------------------------------------------------------------------
// Tensor maps (host)
// ---------------------------------------------------------------------------------------------
namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
}  // namespace

int make_tensor_map_bf16(CUtensorMap* map, const void* base, int BH, int S, int D, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S),
                              static_cast<cuuint64_t>(BH)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * 2,
                                 static_cast<cuuint64_t>(S) * D * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return DADATTN_OK;
}

int make_tensor_map_bf16_units(CUtensorMap* map, const void* base, int units, int S, int D, int box_rows,
                               const UnitLayout& lay) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int heads = lay.heads, batch = units / lay.heads;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S),
                              static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // a dimension of extent 1 still needs a legal stride (a multiple of 16 bytes)
  const cuuint64_t head_stride = heads > 1 ? static_cast<cuuint64_t>(lay.head) * 2 : static_cast<cuuint64_t>(D) * 2;
  const cuuint64_t strides[3] = {static_cast<cuuint64_t>(lay.row) * 2, head_stride,
                                 static_cast<cuuint64_t>(lay.batch) * 2};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(DADATTN_E_CUDA, "cuTensorMapEncodeTiled (4-D) failed (%d)", (int)r);
  return DADATTN_OK;
}

namespace {

using namespace ptx;

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 128;          // keys per tile
constexpr int kStages = 2;        // K/V ring depth
constexpr int kPanelBytes = 128 * 128;  // [128 rows][64 bf16], 128-byte rows, swizzled
constexpr int kFwdThreads = 320;         // producer warp, MMA warp, 8 softmax warps
constexpr int kSoftmaxThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // log2 units: P stays below 2^8

template <int D>
struct FwdSmem {
  static constexpr int kPanels = D / 64;
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kPanels * kPanelBytes;
  static constexpr int kV = kK + kStages * kPanels * kPanelBytes;
  static constexpr int kP = kV + kStages * kPanels * kPanelBytes;
  // Where the probabilities P live between the softmax warps and the P V MMA. D = 128: in
  // tensor memory, written over the scores they were computed from and read by the MMA as its
  // A operand (an MMA with both operands in shared memory reads 8 KB per 64 clocks, all of an
  // SM's shared-memory bandwidth, so every byte of P kept out of shared memory counts).
  // D = 64: one bf16 tile in shared memory.
  static constexpr bool kPTmem = D == 128;
  static constexpr int kBars = kP + (kPTmem ? 0 : 2 * kPanelBytes);
  static constexpr int kBytes = kBars + 256;
};

struct FwdBars {
  uint64_t q_full, k_full[kStages], v_full[kStages], k_empty[kStages], v_empty[kStages];
  uint64_t s_full[2], s_free[2], p_full, o_done[2], stat_full;  // P_j V_j commits to o_done[j & 1]
  uint32_t tmem_base;
  int abort_flag;
};

// 2^x on the FMA pipe: integer part through the float-rounding trick, fractional part in
// [-0.5, 0.5] through a cubic (relative error 6e-4, below bf16's half ulp of 2e-3). Arguments
// below -125 (masked scores are -inf) give exactly 0, as ex2.approx.ftz does.
__device__ __forceinline__ float ex2_poly(float x0) {
  const float x = fmaxf(x0, -125.f);
  const float t = x + 12582912.f;   // 1.5 * 2^23: the integer part lands in the low mantissa bits
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.0555041087f, 0.2402265070f);
  p = fmaf(p, f, 0.6931471806f);
  p = fmaf(p, f, 1.0f);
  const float r = __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
  return x0 < -125.f ? 0.f : r;
}

template <int D, bool DROP>
__global__ void __launch_bounds__(kFwdThreads, D == 64 ? 2 : 1)
flash_fwd_bf16_kernel(const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                      float* __restrict__ lse, int S, float scale, float rate, PhiloxKey rng,
                      int64_t unit0, int* __restrict__ status) {
  using L = FwdSmem<D>;
  constexpr int kPanels = L::kPanels;
  // TMEM columns. D = 64: S [0,128), O_0 [128,192), O_1 [192,256): 256 columns, two CTAs per SM.
  // D = 128 (one CTA per SM): two S buffers [0,256) so that Q K^T of the next tile runs while
  // this tile's softmax still reads its scores, O_0 [256,384), O_1 [384,512).
  constexpr int kSBufs = D == 128 ? 2 : 1;
  constexpr uint32_t kTmemCols = D == 128 ? 512 : 256;
  constexpr uint32_t kColS = 0, kColO = 128 * kSBufs;

  extern __shared__ __align__(1024) uint8_t smem[];
  FwdBars* bars = reinterpret_cast<FwdBars*>(smem + L::kBars);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heaviest tiles first
  const int bh = blockIdx.y;
  const int q0 = qt * kBM;
  const int n_kv = qt + 1;  // causal: key tiles 0..qt

  if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled layouts need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicExch(status, DADATTN_E_CUDA);
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->s_free[b], kSoftmaxThreads);
    }
    mbar_init(&bars->p_full, kSoftmaxThreads);
    mbar_init(&bars->o_done[0], 1);
    mbar_init(&bars->o_done[1], 1);
    mbar_init(&bars->stat_full, kSoftmaxThreads);
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
      mbar_arrive_expect_tx(&bars->q_full, kPanels * kPanelBytes);
      for (int p = 0; p < kPanels; ++p)
        tma_load_3d(smem + L::kQ + p * kPanelBytes, &map_q, &bars->q_full, p * 64, q0, bh);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % kStages, use = j / kStages;
        uint8_t* kdst = smem + L::kK + s * kPanels * kPanelBytes;
        uint8_t* vdst = smem + L::kV + s * kPanels * kPanelBytes;
        // K's slot frees when Q K^T of its previous tenant is done, V's when P V is done
        if (use > 0 && !mbar_wait(&bars->k_empty[s], (use - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(&bars->k_full[s], kPanels * kPanelBytes);
        for (int p = 0; p < kPanels; ++p)
          tma_load_3d(kdst + p * kPanelBytes, &map_k, &bars->k_full[s], p * 64, j * kBN, bh);
        if (use > 0 && !mbar_wait(&bars->v_empty[s], (use - 1) & 1, abort_flag)) break;
        mbar_arrive_expect_tx(&bars->v_full[s], kPanels * kPanelBytes);
        for (int p = 0; p < kPanels; ++p)
          tma_load_3d(vdst + p * kPanelBytes, &map_v, &bars->v_full[s], p * 64, j * kBN, bh);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kBM, kBN, 0, 0);  // Q, K: K-major
      constexpr uint32_t idesc_o = make_idesc_bf16(kBM, D, 0, 1);    // P K-major, V MN-major
      const SmemDescBase q_desc = make_desc_base_sw128(smem_u32(smem + L::kQ), 0);
      const SmemDescBase p_desc = make_desc_base_sw128(smem_u32(smem + L::kP), 0);
      const SmemDescBase k_desc0 = make_desc_base_sw128(smem_u32(smem + L::kK), 0);
      const SmemDescBase v_desc0 = make_desc_base_sw128(smem_u32(smem + L::kV), kPanelBytes);
      constexpr uint32_t kStageBytes = kPanels * kPanelBytes;
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag);

      // O_h[:, 64 pn .. 64 pn + 63] (+)= P_i[:, 64 h .. 64 h + 63] V_i[64 h .. 64 h + 63, :]
      auto issue_pv = [&](int i) -> bool {
        const int s = i % kStages;
        if (!mbar_wait(&bars->v_full[s], (i / kStages) & 1, abort_flag)) return false;
        if (!mbar_wait(&bars->p_full, i & 1, abort_flag)) return false;
        tc_fence_after_sync();
        const SmemDescBase v_desc{v_desc0.lo + s * (kStageBytes >> 4), v_desc0.hi};
        // One MMA per 16 keys covers all D output columns: the V tile is MN-major, its 64-column
        // panels are kPanelBytes apart, which is what the descriptor's leading byte offset says.
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if (L::kPTmem)  // P_i sits in the first 32 columns of each half of score buffer i % 2
              mma_ts(tmem + kColO + h * D, tmem + kColS + (i % kSBufs) * 128 + h * 64 + kk * 8,
                     desc_at(v_desc, (h * 4 + kk) * 2048), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
            else
              mma_ss(tmem + kColO + h * D, desc_at(p_desc, h * kPanelBytes + kk * 32),
                     desc_at(v_desc, (h * 4 + kk) * 2048), idesc_o, (i > 0 || kk > 0) ? 1u : 0u);
          }
        }
        mma_commit(&bars->v_empty[s]);
        mma_commit(&bars->o_done[i & 1]);
        return true;
      };

      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j % kStages;
        // With P in the only score buffer, P_{j-1} V_{j-1} must be issued before S_j replaces it
        if (L::kPTmem && kSBufs == 1 && j > 0) ok = issue_pv(j - 1);
        ok = ok && mbar_wait(&bars->k_full[s], (j / kStages) & 1, abort_flag);
        const int sb = j % kSBufs;
        // With P in TMEM, score buffer sb is next overwritten by S_j only after P_{j-2} V_{j-2},
        // which was issued earlier by this same thread: the tensor pipe keeps them in order.
        if (!L::kPTmem && ok && j >= kSBufs)
          ok = mbar_wait(&bars->s_free[sb], (j / kSBufs - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const SmemDescBase k_desc{k_desc0.lo + s * (kStageBytes >> 4), k_desc0.hi};
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * kPanelBytes + (kk % 4) * 32;
          mma_ss(tmem + kColS + sb * 128, desc_at(q_desc, off), desc_at(k_desc, off), idesc_s,
                 kk > 0 ? 1u : 0u);
        }
        mma_commit(&bars->k_empty[s]);
        mma_commit(&bars->s_full[sb]);
        if (!(L::kPTmem && kSBufs == 1) && j > 0) ok = issue_pv(j - 1);
      }
      if (ok) issue_pv(n_kv - 1);
    }
  } else {
    // ------------------------------ softmax ------------------------------
    const int quad = warp % 4;            // TMEM lane quadrant this warp may touch
    const int half = (warp - 2) / 4;      // which 64 key columns of every tile
    const int row = quad * 32 + lane;     // row within the tile = TMEM lane
    const int r = q0 + row;               // query index
    const uint32_t tlane = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t tO = tlane + kColO + half * D;  // this half's output accumulator
    const float scale_log2 = scale * kLog2e;
    const float keep_scale = DROP ? 1.0f / (1.0f - rate) : 1.0f;
    uint8_t* p_row0 = smem + L::kP + half * kPanelBytes + row * 128;
    // waits for P_i V_i (tile i) to have completed
    auto wait_pv = [&](int i) { return mbar_wait(&bars->o_done[i & 1], (i >> 1) & 1, abort_flag); };
    float m = -INFINITY, l = 0.f;  // running max (log2 units, scaled) and sum of this half-row
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int sb = j % kSBufs;
      const uint32_t tS = tlane + kColS + sb * 128 + half * 64;
      if (!(ok = mbar_wait(&bars->s_full[sb], (j / kSBufs) & 1, abort_flag))) break;
      tc_fence_after_sync();
      const int c0 = j * kBN + half * 64;  // first key of this thread's 64 columns
      // Only the diagonal tile needs the causal mask: columns beyond `limit` are dropped.
      const bool diagonal = (j == n_kv - 1);
      const int limit = r - c0;

      // The thread's 64 scores are read from TMEM (both 32-column loads in flight together).
      // At D = 128 (registers to spare) they stay in registers for the max and for the
      // exponentials and S is handed back to the MMA warp at once; at D = 64 (two CTAs per SM,
      // 96 registers) they are read a second time after the max instead of being kept.
      constexpr bool kKeepScores = (D == 128);
      uint32_t xa[32], xb[32];
      auto load_scores = [&]() {
        tmem_ld32(tS, xa);
        tmem_ld32(tS + 32, xb);
        tmem_wait_ld();
        if (diagonal) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i > limit) xa[i] = 0xff800000u;  // -inf
            if (32 + i > limit) xb[i] = 0xff800000u;
          }
        }
      };
      auto release_scores = [&]() {  // S is in registers: the next QK^T may overwrite it
        if (!L::kPTmem) {
          tc_fence_before_sync();
          mbar_arrive(&bars->s_free[sb]);
        }
      };
      load_scores();
      if (kKeepScores) release_scores();
      // max of the raw scores (scale > 0 commutes with max)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < 32; ++i)
        mx4[i & 3] = fmaxf(mx4[i & 3], fmaxf(__uint_as_float(xa[i]), __uint_as_float(xb[i])));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;

      bool waited_o = false;
      if (j == 0) {
        m = mx;  // O is first written by an MMA with accumulate = 0: nothing to rescale
      } else if (__any_sync(0xffffffffu, mx > m + kRescaleThreshold)) {
        if (!(ok = wait_pv(j - 1))) break;
        waited_o = true;
        tc_fence_after_sync();
        const float m_new = fmaxf(m, mx);
        // m = -inf: nothing but zeros has been accumulated so far (every earlier column masked)
        const float corr = (m == -INFINITY) ? 0.f : ex2(m - m_new);
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st32(tO + c * 32, o);
        }
        tmem_wait_st();
        l *= corr;
        m = m_new;
      }
      // P in shared memory: the MMA that read the buffer last (tile j - 1) must have completed
      if (!L::kPTmem && j > 0 && !waited_o && !(ok = wait_pv(j - 1))) break;
      uint8_t* p_row = p_row0;

      // ---- p = exp2(s * scale * log2e - m), one FFMA + one MUFU per score; bf16 P goes
      // to shared memory in the swizzled K-major layout. A half-row with no visible key yet has
      // m = -inf: its scores are all -inf and must give p = 0, not exp2(nan). ----
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      const float neg_m = (m == -INFINITY) ? 0.f : -m;
      uint32_t pk[L::kPTmem ? 32 : 1];  // packed P of this thread when it goes to TMEM
      auto process = [&](uint32_t (&x)[32], int ch) {
        float pv[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float e = fmaf(__uint_as_float(x[i]), scale_log2, neg_m);
          // at D = 64 (MUFU- and shared-memory-bound) part of the exponentials go to the FMA pipe
          pv[i] = (D == 64 && (i & 3) == 3) ? ex2_poly(e) : ex2(e);
          sum4[i & 3] += pv[i];
        }
        if (DROP) {
          const uint64_t idx0 = (static_cast<uint64_t>(unit0 + bh) * S + r) * S + c0 + ch * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            pv[i] = (pv[i] != 0.f && philox_keep(rng, idx0 + i, rate)) ? pv[i] * keep_scale : 0.f;
        }
        if (L::kPTmem) {
          // bf16 pairs (k, k+1) per 32-bit TMEM column: 16 columns for these 32 probabilities
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[ch * 16 + i] = pack_bf16(pv[2 * i], pv[2 * i + 1]);
        } else {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 w;
            w.x = pack_bf16(pv[v4 * 8 + 0], pv[v4 * 8 + 1]);
            w.y = pack_bf16(pv[v4 * 8 + 2], pv[v4 * 8 + 3]);
            w.z = pack_bf16(pv[v4 * 8 + 4], pv[v4 * 8 + 5]);
            w.w = pack_bf16(pv[v4 * 8 + 6], pv[v4 * 8 + 7]);
            const int chunk = ch * 4 + v4;  // 16-byte chunk within the 128-byte row
            *reinterpret_cast<uint4*>(p_row + ((chunk ^ (row & 7)) << 4)) = w;
          }
        }
      };
      if (!kKeepScores) {
        load_scores();
        release_scores();
      }
      process(xa, 0);
      process(xb, 1);
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      if (L::kPTmem) {
        tmem_st32(tS, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_wait_st();
      } else {
        fence_proxy_async_smem();
      }
      tc_fence_before_sync();
      mbar_arrive(&bars->p_full);
    }

    // Epilogue: merge the two halves of each row. out = (O_0 w_0 + O_1 w_1) / (l_0 w_0 + l_1 w_1)
    // with w_h = exp2(m_h - max(m_0, m_1)); lse in natural-log units of the scaled scores.
    // Each thread of the pair writes half of the row's D outputs.
    // The (max, sum) pairs are exchanged through the Q tile's shared memory, which nobody reads
    // any more: every Q K^T has completed before the last s_full was observed.
    float2* stat = reinterpret_cast<float2*>(smem + L::kQ);  // [2][128]
    if (ok) {
      stat[half * 128 + row] = make_float2(m, l);
      mbar_arrive(&bars->stat_full);
      ok = mbar_wait(&bars->stat_full, 0, abort_flag) &&
           wait_pv(n_kv - 1);
    }
    if (ok) {
      tc_fence_after_sync();
      const float2 s0 = stat[row], s1 = stat[128 + row];
      const float m_tot = fmaxf(s0.x, s1.x);  // half 0 always sees key 0: finite
      const float w0 = ex2(s0.x - m_tot);
      const float w1 = (s1.x == -INFINITY) ? 0.f : ex2(s1.x - m_tot);
      const float l_tot = s0.y * w0 + s1.y * w1;
      const float f0 = w0 / l_tot, f1 = w1 / l_tot;
      constexpr int kCols = D / 2;  // output columns per thread
      __nv_bfloat16* dst = out + (static_cast<size_t>(bh) * S + r) * D + half * kCols;
#pragma unroll
      for (int c = 0; c < kCols / 32; ++c) {
        uint32_t oa[32], ob[32];
        tmem_ld32(tlane + kColO + half * kCols + c * 32, oa);
        tmem_ld32(tlane + kColO + D + half * kCols + c * 32, ob);
        tmem_wait_ld();
        if (r < S) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float y[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              y[e] = __uint_as_float(oa[8 * i + e]) * f0 + __uint_as_float(ob[8 * i + e]) * f1;
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) =
                make_uint4(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]), pack_bf16(y[4], y[5]),
                           pack_bf16(y[6], y[7]));
          }
        }
      }
      if (half == 0 && r < S) lse[static_cast<size_t>(bh) * S + r] = (m_tot + log2f(l_tot)) * kLn2;
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

template <int D, bool DROP>
int launch_fwd_bf16(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k,
                    const uint16_t* v, int BH, int S, float scale, float rate, uint64_t seed,
                    uint64_t offset, int64_t unit0, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  if (int rc = make_tensor_map_bf16(&mq, q, BH, S, D, kBM)) return rc;
  if (int rc = make_tensor_map_bf16(&mk, k, BH, S, D, kBN)) return rc;
  if (int rc = make_tensor_map_bf16(&mv, v, BH, S, D, kBN)) return rc;
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  auto kern = flash_fwd_bf16_kernel<D, DROP>;
  DAD_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                FwdSmem<D>::kBytes));
  dim3 grid((S + kBM - 1) / kBM, BH);
  DAD_CUDA(launch_pdl(kern, grid, dim3(kFwdThreads), FwdSmem<D>::kBytes, st, mq, mk, mv,
                      reinterpret_cast<__nv_bfloat16*>(out), lse, S, scale, rate,
                      make_philox(seed, offset), unit0, status));
  return DADATTN_OK;
}

}  // namespace
}  // namespace dadattn

using namespace dadattn;


extern "C" int dadattn_flash_bf16_supported(int d_head) { return d_head == 64 || d_head == 128; }

extern "C" int dadattn_flash_fwd_bf16(uint16_t* out, float* lse, const uint16_t* q,
                                      const uint16_t* k, const uint16_t* v, int BH, int S, int D,
                                      float scale, float rate, uint64_t seed, uint64_t offset,
                                      int64_t unit0, dadattn_stream_t stream) {
  if (!out || !lse || !q || !k || !v) return fail(DADATTN_E_ARG, "null tensor pointer");
  if (BH <= 0 || S <= 0) return fail(DADATTN_E_ARG, "BH=%d and S=%d must be positive", BH, S);
  if (BH > 65535) return fail(DADATTN_E_UNSUPPORTED, "BH=%d exceeds 65535 per call", BH);
  if (!dadattn_flash_bf16_supported(D))
    return fail(DADATTN_E_UNSUPPORTED, "flash attention bf16: unsupported d_head %d", D);
  if (!(rate >= 0.0f && rate < 1.0f))
    return fail(DADATTN_E_ARG, "dropout rate %f outside [0,1)", static_cast<double>(rate));
  if (!(scale > 0.0f)) return fail(DADATTN_E_ARG, "bf16 forward needs scale > 0");
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) ||
      !aligned(lse, 4))
    return fail(DADATTN_E_ARG, "bf16 tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool drop = rate > 0.f;
  if (D == 64)   // head size 64 has a kernel of its own (flash_fwd64_sm100.cu)
    return launch_fwd_bf16_d64(out, lse, q, k, v, BH, S, scale, rate, seed, offset, unit0, nullptr, 0, st);
  return drop ? launch_fwd_bf16<128, true>(out, lse, q, k, v, BH, S, scale, rate, seed, offset, unit0, st)
              : launch_fwd_bf16<128, false>(out, lse, q, k, v, BH, S, scale, 0.f, 0, 0, 0, st);
}

extern "C" int dadattn_flash_fwd_bf16_masked(uint16_t* out, float* lse, const uint16_t* q,
                                             const uint16_t* k, const uint16_t* v, int BH, int S, int D,
                                             float scale, float rate, const uint32_t* mask_bits,
                                             dadattn_stream_t stream) {
  if (!out || !lse || !q || !k || !v) return fail(DADATTN_E_ARG, "null tensor pointer");
  if (!mask_bits || !aligned(mask_bits, 16))
    return fail(DADATTN_E_ARG, "mask_bits must be a 16-byte aligned device pointer");
  if (BH <= 0 || S <= 0) return fail(DADATTN_E_ARG, "BH=%d and S=%d must be positive", BH, S);
  if (BH > 65535) return fail(DADATTN_E_UNSUPPORTED, "BH=%d exceeds 65535 per call", BH);
  if (D != 64)
    return fail(DADATTN_E_UNSUPPORTED, "a bit-packed dropout mask is taken at head size 64 only (got %d)", D);
  if (!(rate > 0.0f && rate < 1.0f))
    return fail(DADATTN_E_ARG, "the masked forward needs the rate the mask was drawn with, in (0,1)");
  if (!(scale > 0.0f)) return fail(DADATTN_E_ARG, "bf16 forward needs scale > 0");
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(lse, 4))
    return fail(DADATTN_E_ARG, "bf16 tensors must be 16-byte aligned");
  return launch_fwd_bf16_d64(out, lse, q, k, v, BH, S, scale, rate, 0, 0, 0, mask_bits, 0,
                             static_cast<cudaStream_t>(stream));
}

extern "C" int dadattn_flash_fwd_bf16_strided(uint16_t* out, float* lse, const uint16_t* q,
                                              const uint16_t* k, const uint16_t* v, int B, int H, int S,
                                              int D, float scale, float rate, uint64_t seed,
                                              uint64_t offset, int64_t unit0, dadattn_stream_t stream) {
  if (!out || !lse || !q || !k || !v) return fail(DADATTN_E_ARG, "null tensor pointer");
  if (B <= 0 || H <= 0 || S <= 0) return fail(DADATTN_E_ARG, "B=%d, H=%d and S=%d must be positive", B, H, S);
  if (static_cast<long long>(B) * H > 65535)
    return fail(DADATTN_E_UNSUPPORTED, "B*H=%lld exceeds 65535 per call", static_cast<long long>(B) * H);
  if (D != 64)
    return fail(DADATTN_E_UNSUPPORTED, "interleaved [B*S, H*D] activations are taken at head size 64 only (got %d)", D);
  if (!(rate >= 0.0f && rate < 1.0f))
    return fail(DADATTN_E_ARG, "dropout rate %f outside [0,1)", static_cast<double>(rate));
  if (!(scale > 0.0f)) return fail(DADATTN_E_ARG, "bf16 forward needs scale > 0");
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k, 16) || !aligned(v, 16) || !aligned(lse, 4))
    return fail(DADATTN_E_ARG, "bf16 tensors must be 16-byte aligned");
  return launch_fwd_bf16_d64(out, lse, q, k, v, B * H, S, scale, rate, seed, offset, unit0, nullptr, H,
                             static_cast<cudaStream_t>(stream));
}
