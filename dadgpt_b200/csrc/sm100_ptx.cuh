// Inline-PTX wrappers for the Blackwell (sm_100a) features the bf16 kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, never multicast), tcgen05 MMA / TMEM / commit, and the
// shared-memory and instruction descriptors tcgen05.mma consumes.
//
// Every wait here is bounded: it returns false after kSpinLimit polls (or as soon as the CTA's
// abort flag is raised) instead of spinning forever, so a protocol bug surfaces as an error
// code, not as a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace dadattn {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

constexpr uint32_t kSpinLimit = 1u << 24;  // with the back-off below: a few seconds
// Non-blocking polls before the suspending wait takes over. More than a few hundred cost time:
// the polling of waiting warps competes for issue slots with the warps that still work.
constexpr uint32_t kHotPolls = 128;

// Waits for the phase with the given parity to complete. `abort_flag` (shared memory) is
// polled too: once any thread of the CTA has given up, everybody leaves quickly. The thread
// whose own wait runs out leaves `site` (the source line of the wait, through DAD_MBAR_WAIT)
// in the flag, from where the kernel's exit path copies it next to the device status word.
template <uint32_t HOT = kHotPolls>
__device__ __forceinline__ bool mbar_wait_at(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                             int site) {
  // Most waits in these kernels are short (a few hundred clocks: the next link of a pipeline). A
  // suspending try_wait that has to be woken costs more than that, so the wait starts as a plain
  // poll and only then turns into the suspending form with back-off.
  for (uint32_t i = 0; i < HOT; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 32) {
      if (*abort_flag) return false;
      __nanosleep(i > 4096 ? 256 : 32);
    }
  }
  atomicCAS(const_cast<int*>(abort_flag), 0, site);
  return false;
}
#define mbar_wait(bar, parity, abort_flag) mbar_wait_at(bar, parity, abort_flag, __LINE__)

// Common exit of a kernel whose CTA raised its abort flag: the flag holds the line of the wait
// that ran out; it goes to the word behind the status word, the status becomes E_TIMEOUT.
__device__ __forceinline__ void report_timeout(int* status, int site) {
  status[1] = site;
  atomicExch(status, DADATTN_E_TIMEOUT);
}

// ---- register rebalancing between warpgroups -------------------------------------------------
// Every warp of a warpgroup (four consecutive warps, the first a multiple of four) executes the
// same one. N is a multiple of 8; an increase waits until other warpgroups have given enough back.
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- proxies / fences -----------------------------------------------------------------------
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA (tiled, 3-D, no multicast) ------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// x = innermost coordinate in elements; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x),
      "r"(y), "r"(z)
      : "memory");
}

// 1-D form, for vectors of per-row scalars. x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_1d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x) {
  asm volatile(
      "cp.async.bulk.tensor.1d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x)
      : "memory");
}

// 4-D form: (x, row, head, batch). The bf16 kernels address a (batch, head) unit this way so
// that one code path serves both memory layouts (see UnitLayout below).
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x),
      "r"(y), "r"(z), "r"(w)
      : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------------
// Whole-warp calls. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// ---- tcgen05.mma ------------------------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues for the CTA.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulation.
// a_mn_major / b_mn_major: 0 = K-major (K contiguous in shared memory), 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn_major,
                                                       int b_mn_major) {
  return (1u << 4)                                  // accumulator format: fp32
         | (1u << 7)                                // A format: bf16
         | (1u << 10)                               // B format: bf16
         | (static_cast<uint32_t>(a_mn_major) << 15)
         | (static_cast<uint32_t>(b_mn_major) << 16)
         | (static_cast<uint32_t>(N >> 3) << 17)
         | (static_cast<uint32_t>(M >> 4) << 24);
}

// Shared-memory matrix descriptor for a 128-byte-swizzled tile whose rows are 128 bytes
// (64 bf16) and whose 8-row groups are 1024 bytes apart — what a TMA box of inner extent 64
// bf16 with CU_TENSOR_MAP_SWIZZLE_128B writes. The same encoding serves K-major operands
// (rows = M/N index, 128 B = 64 K elements) and MN-major operands (rows = K index, 128 B = 64
// M/N elements); `lbo_bytes` is only read for MN-major operands wider than 64 elements.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);        // start address
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset (8 rows)
  d |= static_cast<uint64_t>(1) << 46;                           // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                           // layout: SWIZZLE_128B
  return d;
}

// The same descriptor split in halves so that the issuing thread spends one 32-bit add per MMA:
// `hi` is constant for a tile, `lo` carries the start address (in 16-byte units) and the LBO.
struct SmemDescBase {
  uint32_t lo, hi;
};
__device__ __forceinline__ SmemDescBase make_desc_base_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  const uint64_t d = make_smem_desc_sw128(smem_addr, lbo_bytes);
  return SmemDescBase{static_cast<uint32_t>(d), static_cast<uint32_t>(d >> 32)};
}
// Descriptor of the same tile advanced by `byte_offset` (a multiple of 16 that stays inside the
// tile, so the 14-bit address field cannot carry into its neighbours).
__device__ __forceinline__ uint64_t desc_at(SmemDescBase b, uint32_t byte_offset) {
  return (static_cast<uint64_t>(b.hi) << 32) | static_cast<uint64_t>(b.lo + (byte_offset >> 4));
}

// ---- tcgen05.ld / st: 32 lanes x 32-bit, N consecutive columns per thread ---------------------
// A warp may only touch the TMEM lane quadrant (warp_id % 4) * 32 .. + 31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// ---- packed two-float arithmetic and three-input max (sm_100) --------------------------------
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for two values on the FMA pipe: integer part through the float-rounding trick, fraction
// in [-0.5, 0.5] through a cubic (relative error 6e-4, below bf16's half ulp of 2e-3).
// Arguments below -125 (masked scores are -inf) give exactly 0, as ex2.approx.ftz does.
__device__ __forceinline__ float2 ex2_poly2(float2 x0) {
  const float2 x = make_float2(fmaxf(x0.x, -125.f), fmaxf(x0.y, -125.f));
  const float2 big = make_float2(12582912.f, 12582912.f);  // 1.5 * 2^23
  const float2 t = fadd2(x, big);
  const float2 f = fadd2(x, make_float2(big.x - t.x, big.y - t.y));
  float2 p = ffma2(f, make_float2(0.0555041087f, 0.0555041087f), make_float2(0.2402265070f, 0.2402265070f));
  p = ffma2(p, f, make_float2(0.6931471806f, 0.6931471806f));
  p = ffma2(p, f, make_float2(1.0f, 1.0f));
  float2 r;
  r.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23));
  if (x0.x < -125.f) r.x = 0.f;
  if (x0.y < -125.f) r.y = 0.f;
  return r;
}


// Two floats -> packed bf16x2 (lo in the low half), round to nearest even.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace ptx

// ---- host side: tensor maps -------------------------------------------------------------------
// 3-D map over a contiguous bf16 [BH, S, D] tensor with a box of 64 x `box_rows` x 1 elements
// and 128-byte swizzle; out-of-range rows read as zero. Returns 0 or a DADATTN_E_* code.
int make_tensor_map_bf16(CUtensorMap* map, const void* base, int BH, int S, int D, int box_rows);

// Where the rows of a (batch, head) unit lie. Heads-split (the reference's q_heads / k_heads /
// v_heads after gpu_split_heads, cuda/gpu_ops.cu:428-474): [B*H, S, D] contiguous. Interleaved
// (the reference's activations BEFORE the split, [B*S, H*D], src/model.cpp:372-387): row s of
// unit (b, h) starts at ((b S + s) H + h) D. Both are a 4-D tensor (d, s, h, b) with different
// strides, so one tensor map and one (x, row, h, b) coordinate serve both; the heads-split form is
// used with heads = 1, batch = B*H.
struct UnitLayout {
  int heads;            // H of the (h, b) split of a unit index: b = unit / heads, h = unit % heads
  int64_t row, head, batch;   // element strides of a query / key row, a head, a batch entry
};
inline UnitLayout unit_layout(int B, int H, int S, int D, bool interleaved) {
  if (!interleaved) return UnitLayout{1, D, 0, static_cast<int64_t>(S) * D};  // unit = b H + h, heads folded
  return UnitLayout{H, static_cast<int64_t>(H) * D, D, static_cast<int64_t>(S) * H * D};
}
// 4-D map (d, s, h, b) over a bf16 tensor in either layout; box 64 x box_rows x 1 x 1, 128-byte
// swizzle; rows beyond S read as zero and are dropped on stores. For the heads-split layout
// pass units = B*H: the map is then (D, S, 1, B*H).
int make_tensor_map_bf16_units(CUtensorMap* map, const void* base, int units, int S, int D, int box_rows,
                               const UnitLayout& lay);

}  // namespace dadattn
