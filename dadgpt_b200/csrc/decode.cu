// KV-cache decode attention: one new query token per sequence against that sequence's cache.
//
// The reference runs this as 61 tiny launches per layer (per-head M=1 cuBLAS products, 256-byte
// device-to-device appends, one softmax; src/model.cpp:745-790). Here it is ONE split-K kernel
// per layer call, for any number of concurrent sequences:
//   * grid = (sequences x heads, splits); a CTA of 8 warps owns `chunk` consecutive cache rows
//     of one (sequence, head): the whole sequence when there are enough pairs to fill the GPU,
//     a slice otherwise. Splits are the slow grid dimension, so CTAs whose chunk lies
//     beyond the sequence's length (they exit at once) are scheduled last, not in between;
//   * a cache row (D elements) is read by D*sizeof(T)/16 adjacent lanes with one 128-bit load
//     each, so a warp instruction covers 512 contiguous bytes of the cache; a lane issues the K
//     and V loads of 4 row groups (128 bytes) before it consumes any, and 16-24 such warps per
//     SM keep ~100 KB in flight: memory-level parallelism is what a bandwidth-bound kernel
//     lives on;
//   * q.k partial sums are reduced over those lanes with warp shuffles; each lane keeps an
//     online-softmax state (max, sum, D/lanes accumulators) for the rows it has seen;
//   * the append is fused: the lanes that own row `len` take k_new/v_new from the token's
//     vectors, use them, and store them into the cache;
//   * split-K merge without a second kernel and without waiting: a CTA writes (unnormalised
//     out[D], max, sum) to the workspace, fences, and takes a ticket; whoever draws the last
//     ticket of its (sequence, head) merges the records and writes `out`. A second ticket per
//     sequence, taken by every CTA after it has read the length, lets the very last CTA of a
//     sequence store length + 1. Tickets are returned to zero by their last holder, so a
//     workspace zeroed once stays usable forever;
//   * launched with programmatic stream serialization: the next decode call's CTAs are already
//     resident (parked in griddepcontrol.wait) when this grid drains.
// In direct mode (one split; the fp32 single-sequence path) the CTA normalises and writes the
// output itself and no workspace is used.
#include <cfloat>
#include <climits>
#include <cuda_bf16.h>

#include "common.cuh"

namespace dadattn {
namespace {

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kDecodeBatch = 4;   // row groups whose loads a lane keeps in flight
constexpr unsigned kTicketGroups = 32;  // first-level counters of the "all lengths read" tickets
constexpr int kMinChunk = 256;    // smallest number of cache rows a CTA is given
constexpr int kTargetCtas = 592;  // 4 per SM: below that the cache is split across CTAs

// Rows per CTA. With enough (sequence, head) pairs to fill the GPU a CTA walks a whole
// sequence (measured fastest: no records, no tickets); with few pairs the rows are split so
// that about kTargetCtas CTAs exist. Depends only on (B, H, max_len), so the workspace size and
// the kernel agree.
inline int chunk_rows(int B, int H, int max_len) {
  const long long pairs = static_cast<long long>(B) * H;
  long long want_splits = (kTargetCtas + pairs - 1) / pairs;
  if (want_splits < 1) want_splits = 1;
  long long rows = (max_len + want_splits - 1) / want_splits;
  if (rows < kMinChunk) rows = kMinChunk;
  rows = (rows + 127) / 128 * 128;
  return static_cast<int>(rows);
}
inline int split_count(int B, int H, int max_len) {
  const int c = chunk_rows(B, H, max_len);
  return (max_len + c - 1) / c;
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerLane = 4;
  __device__ static void unpack(float (&f)[4], const uint4& raw) {
    f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
    f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
  }
  __device__ static float from_float(float x) { return x; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerLane = 8;
  __device__ static void unpack(float (&f)[8], const uint4& raw) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// Workspace: one ticket per (sequence, head), then the 1 + kTicketGroups counters of the "all
// lengths read" tickets (uint32, zero between calls), padded to 256 bytes, then the records [B*H][splits][D + 2] fp32 (unnormalised output, max, sum).
__host__ __device__ inline size_t partial_stride(int D) { return static_cast<size_t>(D) + 2; }
inline size_t record_bytes(int B, int H, int D, int max_len) {
  const int splits = split_count(B, H, max_len);
  if (splits == 1) return 0;  // every CTA finishes its (sequence, head) itself: no records
  return static_cast<size_t>(B) * H * splits * partial_stride(D) * sizeof(float);
}
inline size_t ticket_bytes(int B, int H) {
  return (sizeof(uint32_t) * (static_cast<size_t>(B) * H + 1 + kTicketGroups) + 255) / 256 * 256;
}
inline size_t workspace_bytes(int B, int H, int D, int max_len) {
  return ticket_bytes(B, H) + (record_bytes(B, H, D, max_len) + 255) / 256 * 256;
}

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeThreads, 3)
decode_splitk_kernel(T* __restrict__ out, float* __restrict__ partial,
                     unsigned* __restrict__ tickets, unsigned* __restrict__ seq_tickets,
                     const T* __restrict__ q, const T* __restrict__ k_new,
                     const T* __restrict__ v_new, T* __restrict__ k_cache, T* __restrict__ v_cache,
                     int32_t* __restrict__ lengths, int fixed_len, int H, int max_len, int chunk,
                     int reorder, int early, float scale, int* __restrict__ status) {
  constexpr int EPL = Elem<T>::kPerLane;  // elements per lane (one 16-byte load)
  constexpr int LPK = D / EPL;            // lanes per cache row
  constexpr int KPI = 32 / LPK;           // cache rows per warp instruction
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "row must split over a warp");

  // Everything this grid reads may have been written by the grid before it — unless the caller
  // has promised (dadattn_set_decode_early_start) that the grid before it does not write this
  // call's caches, lengths and workspace: then the lengths, the ranking and each warp's first
  // cache rows are fetched while that grid drains, and only the token vectors wait for it.
  if (!early) pdl_wait();
  pdl_launch_dependents();

  const int split = blockIdx.y, splits = gridDim.y;
  __shared__ int sh_len, sh_b, sh_last, sh_adv;
  __shared__ __align__(16) int sh_lens[kDecodeThreads];
  __shared__ int sh_rank[kDecodeThreads];
  __shared__ float sh_acc[kDecodeWarps][D];
  __shared__ float sh_m[kDecodeWarps], sh_l[kDecodeWarps];
  // Which sequence this CTA works on. CTAs are handed to the SMs in blockIdx order, and a CTA
  // lasts as long as its sequence is long: with the sequences taken longest first, the short
  // ones fill the gaps at the end instead of a long one starting last (measured: 13 % less time
  // per call on lengths uniform in 1..1024). The order is recomputed by every CTA from the
  // lengths themselves (rank by counting), for up to one sequence per thread.
  const int n_seq = static_cast<int>(gridDim.x) / H;
  const int slot_seq = static_cast<int>(blockIdx.x) / H;
  if (reorder) {
    // rank(s) = number of sequences that come before s (longer, or as long with a smaller
    // index). All threads take part: with the sequence count padded to a power of two n_pad
    // (32..256; padding entries are INT_MIN and come last), sequence s = t % n_pad is compared
    // with a slice of n_pad^2 / 256 others by thread t, four at a time, and the partial counts
    // are summed in shared memory. Shifts only: no integer division on this path.
    const int t = threadIdx.x;
    sh_lens[t] = t < n_seq ? lengths[t] : INT_MIN;
    sh_rank[t] = 0;
    __syncthreads();
    const int lg = 32 - __clz(n_seq - 1);          // n_pad = 1 << lg, 5 <= lg <= 8
    const int s_idx = t & ((1 << lg) - 1), g = t >> lg;
    const int per4 = 1 << (2 * lg - 10);           // int4 loads per thread
    const int mine = sh_lens[s_idx];
    const int4* slice = reinterpret_cast<const int4*>(sh_lens) + g * per4;
    int count = 0;
#pragma unroll 4
    for (int j = 0; j < per4; ++j) {
      const int4 o = slice[j];  // one address per warp: a broadcast read
      const int j0 = (g * per4 + j) * 4;
      count += static_cast<int>(o.x > mine) | (static_cast<int>(o.x == mine) & static_cast<int>(j0 + 0 < s_idx));
      count += static_cast<int>(o.y > mine) | (static_cast<int>(o.y == mine) & static_cast<int>(j0 + 1 < s_idx));
      count += static_cast<int>(o.z > mine) | (static_cast<int>(o.z == mine) & static_cast<int>(j0 + 2 < s_idx));
      count += static_cast<int>(o.w > mine) | (static_cast<int>(o.w == mine) & static_cast<int>(j0 + 3 < s_idx));
    }
    if (count) atomicAdd(&sh_rank[s_idx], count);
    __syncthreads();
    if (t < n_seq && sh_rank[t] == slot_seq) {
      sh_b = t;
      sh_len = sh_lens[t];
    }
  } else if (threadIdx.x == 0) {
    sh_b = slot_seq;
    sh_len = lengths ? lengths[slot_seq] : fixed_len;  // rows already in the cache
  }
  __syncthreads();  // the CTA's ticket below is taken strictly after these reads
  // Every CTA of the call draws a ticket once it has read the lengths (all of them, when it
  // ranks the sequences); whoever holds the last one knows that nobody will read them again and
  // advances them. Two levels keep the atomics off one address: the CTAs are dealt into
  // kTicketGroups groups, a CTA draws its group's ticket here, at the start, and looks at it
  // only at the very end (the round trip through L2 costs it nothing); the last of each group
  // then draws from a second counter, and the last of those advances the lengths.
  unsigned my_ticket = 0;
  if (lengths != nullptr && threadIdx.x == 0)
    my_ticket = atomicAdd(&seq_tickets[1 + (blockIdx.y * gridDim.x + blockIdx.x) % kTicketGroups], 1u);
  auto advance_lengths = [&]() {
    if (lengths == nullptr) return;
    if (threadIdx.x == 0) {
      // recomputed here rather than kept in registers across the main loop: the kernel lives on
      // three CTAs per SM
      const unsigned all_ctas = gridDim.x * gridDim.y;
      const unsigned group = (blockIdx.y * gridDim.x + blockIdx.x) % kTicketGroups;
      const unsigned group_size = (all_ctas - group + kTicketGroups - 1) / kTicketGroups;
      int last = 0;
      if (my_ticket == group_size - 1) {
        seq_tickets[1 + group] = 0;   // ready for the next call
        const unsigned groups = all_ctas < kTicketGroups ? all_ctas : kTicketGroups;
        last = atomicAdd(&seq_tickets[0], 1u) == groups - 1;
        if (last) seq_tickets[0] = 0;
      }
      sh_adv = last;
    }
    __syncthreads();
    if (!sh_adv) return;
    for (int s = threadIdx.x; s < n_seq; s += kDecodeThreads) {
      const int l = lengths[s];
      if (l >= 0 && l < max_len) lengths[s] = l + 1;   // a full or invalid sequence is left alone
    }
  };
  const int b = sh_b;
  const int bh = b * H + static_cast<int>(blockIdx.x) % H;
  const int len = sh_len;
  if (len < 0 || len >= max_len) {
    if (split == 0 && bh % H == 0 && threadIdx.x == 0) atomicExch(status, DADATTN_E_ARG);
    advance_lengths();
    return;
  }
  const int total = len + 1;  // rows visible to the new token, itself included
  const int n_active = (total + chunk - 1) / chunk;

  if (split < n_active) {
    const int row_begin = split * chunk;
    const int row_end = min(row_begin + chunk, total);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int slot = lane / LPK, part = lane % LPK;
    const size_t vec_off = static_cast<size_t>(bh) * D + part * EPL;
    const size_t cache_base = static_cast<size_t>(bh) * max_len * D + part * EPL;

    uint4 kr[kDecodeBatch], vr[kDecodeBatch];
    int base = row_begin + warp * KPI * kDecodeBatch;
    // early start: the warp's first batch, if it lies wholly among the rows already in the cache
    // (the row being appended needs k_new / v_new, which must wait)
    const bool prefetched = early && base + KPI * kDecodeBatch <= len;
    if (prefetched) {
#pragma unroll
      for (int u = 0; u < kDecodeBatch; ++u) {
        const int row = base + u * KPI + slot;
        kr[u] = ld_stream(k_cache + cache_base + static_cast<size_t>(row) * D);
        vr[u] = ld_stream(v_cache + cache_base + static_cast<size_t>(row) * D);
      }
    }
    if (early) pdl_wait();

    float qf[EPL];
    Elem<T>::unpack(qf, *reinterpret_cast<const uint4*>(q + vec_off));
    float m = -FLT_MAX, l = 0.f, acc[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[e] = 0.f;

    bool fetched = prefetched;   // the batch at `base` is already in registers
    for (; base < row_end; base += kDecodeWarps * KPI * kDecodeBatch, fetched = false) {
      if (!fetched) {
#pragma unroll
      for (int u = 0; u < kDecodeBatch; ++u) {
        const int row = base + u * KPI + slot;
        kr[u] = make_uint4(0, 0, 0, 0);
        vr[u] = make_uint4(0, 0, 0, 0);
        if (row < row_end) {
          if (row == len) {  // the token being appended: use its vectors and store them
            kr[u] = *reinterpret_cast<const uint4*>(k_new + vec_off);
            vr[u] = *reinterpret_cast<const uint4*>(v_new + vec_off);
            *reinterpret_cast<uint4*>(k_cache + cache_base + static_cast<size_t>(row) * D) = kr[u];
            *reinterpret_cast<uint4*>(v_cache + cache_base + static_cast<size_t>(row) * D) = vr[u];
          } else {
            kr[u] = ld_stream(k_cache + cache_base + static_cast<size_t>(row) * D);
            vr[u] = ld_stream(v_cache + cache_base + static_cast<size_t>(row) * D);
          }
        }
      }
      }
      float s[kDecodeBatch];
      float m_new = m;
#pragma unroll
      for (int u = 0; u < kDecodeBatch; ++u) {
        float kf[EPL];
        Elem<T>::unpack(kf, kr[u]);
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) dot = fmaf(qf[e], kf[e], dot);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        s[u] = (base + u * KPI + slot < row_end) ? dot * scale : -FLT_MAX;
        m_new = fmaxf(m_new, s[u]);
      }
      if (m_new > -FLT_MAX) {  // at least one row seen by this lane group so far
        const float corr = expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[e] *= corr;
#pragma unroll
        for (int u = 0; u < kDecodeBatch; ++u) {
          if (!(base + u * KPI + slot < row_end)) continue;
          const float p = expf(s[u] - m_new);
          l += p;
          float vf[EPL];
          Elem<T>::unpack(vf, vr[u]);
#pragma unroll
          for (int e = 0; e < EPL; ++e) acc[e] = fmaf(p, vf[e], acc[e]);
        }
        m = m_new;
      }
    }

    // Merge the KPI row slots of the warp (lanes with equal `part`), then the warps.
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m, o);
      const float l_o = __shfl_xor_sync(0xffffffffu, l, o);
      const float m_new = fmaxf(m, m_o);
      const float ca = m > -FLT_MAX ? expf(m - m_new) : 0.f;
      const float cb = m_o > -FLT_MAX ? expf(m_o - m_new) : 0.f;
      l = l * ca + l_o * cb;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float a_o = __shfl_xor_sync(0xffffffffu, acc[e], o);
        acc[e] = acc[e] * ca + a_o * cb;
      }
      m = m_new;
    }
    if (slot == 0) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) sh_acc[warp][part * EPL + e] = acc[e];
      if (part == 0) {
        sh_m[warp] = m;
        sh_l[warp] = l;
      }
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += kDecodeThreads) {
      float mm = -FLT_MAX;
#pragma unroll
      for (int w = 0; w < kDecodeWarps; ++w) mm = fmaxf(mm, sh_m[w]);
      float ll = 0.f, aa = 0.f;
#pragma unroll
      for (int w = 0; w < kDecodeWarps; ++w) {
        const float c = sh_m[w] > -FLT_MAX ? expf(sh_m[w] - mm) : 0.f;
        ll += sh_l[w] * c;
        aa += sh_acc[w][d] * c;
      }
      if (n_active == 1) {  // the only split of this (sequence, head): finish here
        out[static_cast<size_t>(bh) * D + d] = Elem<T>::from_float(aa / ll);
      } else {
        float* rec = partial + (static_cast<size_t>(bh) * splits + split) * partial_stride(D);
        rec[d] = aa;
        if (d == 0) {
          rec[D] = mm;
          rec[D + 1] = ll;
        }
      }
    }

    if (n_active > 1) {
      // Publish the record, then draw a ticket; the holder of the last one merges.
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) sh_last = (atomicAdd(&tickets[bh], 1u) == static_cast<unsigned>(n_active - 1));
      __syncthreads();
      if (sh_last) {
        __threadfence();
        const float* rec = partial + static_cast<size_t>(bh) * splits * partial_stride(D);
        for (int d = threadIdx.x; d < D; d += kDecodeThreads) {
          float mm = -FLT_MAX;
          for (int s2 = 0; s2 < n_active; ++s2) mm = fmaxf(mm, __ldcg(rec + s2 * partial_stride(D) + D));
          float ll = 0.f, aa = 0.f;
          for (int s2 = 0; s2 < n_active; ++s2) {
            const float* r = rec + s2 * partial_stride(D);
            const float c = expf(__ldcg(r + D) - mm);
            ll += __ldcg(r + D + 1) * c;
            aa += __ldcg(r + d) * c;
          }
          out[static_cast<size_t>(bh) * D + d] = Elem<T>::from_float(aa / ll);
        }
        if (threadIdx.x == 0) tickets[bh] = 0;  // ready for the next call
      }
    }
  }

  advance_lengths();
}

template <typename T, typename Raw, int DH>
int launch_decode_batched(Raw* out, const Raw* q, const Raw* k_new, const Raw* v_new, Raw* k_cache,
                          Raw* v_cache, int32_t* lengths, int B, int H, int max_len, float scale,
                          unsigned* tickets, float* partial, int* status, int early, cudaStream_t st) {
  const int chunk = chunk_rows(B, H, max_len);
  const int splits = split_count(B, H, max_len);
  unsigned* seq_tickets = tickets + static_cast<size_t>(B) * H;
  dim3 grid(static_cast<unsigned>(B) * H, splits);
  // Longest-first order pays once the CTAs no longer all fit on the GPU at the same time (about
  // three of them per SM); the in-kernel ranking handles 32..256 sequences.
  int dev = 0, sms = 0;
  DAD_CUDA(cudaGetDevice(&dev));
  DAD_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int reorder = (B >= 32 && B <= kDecodeThreads &&
                       static_cast<long long>(B) * H * splits > 3LL * sms) ? 1 : 0;
  DAD_CUDA(launch_pdl(decode_splitk_kernel<T, DH>, grid, dim3(kDecodeThreads), 0, st,
                             reinterpret_cast<T*>(out), partial, tickets, seq_tickets,
                             reinterpret_cast<const T*>(q), reinterpret_cast<const T*>(k_new),
                             reinterpret_cast<const T*>(v_new), reinterpret_cast<T*>(k_cache),
                             reinterpret_cast<T*>(v_cache), lengths, 0, H, max_len, chunk, reorder,
                             early, scale, status));
  return DADATTN_OK;
}

template <int DH>
int launch_decode_bf16(uint16_t* out, const uint16_t* q, const uint16_t* k_new,
                       const uint16_t* v_new, uint16_t* k_cache, uint16_t* v_cache,
                       int32_t* lengths, int B, int H, int max_len, float scale,
                       unsigned* tickets, float* partial, int* status, int early, cudaStream_t st) {
  return launch_decode_batched<__nv_bfloat16, uint16_t, DH>(out, q, k_new, v_new, k_cache, v_cache, lengths, B,
                                                            H, max_len, scale, tickets, partial, status,
                                                            early, st);
}

// Rows 0..n-1 of sequence b's cache from the K / V heads a prefill leaves behind: k_heads,
// v_heads [H, n, D] fp32 (the reference's q_heads / k_heads / v_heads layout for batch 1,
// src/model.cpp:385-387) -> k_cache, v_cache [B, H, max_len, D] in T; sets lengths[b] = n. One
// launch for both tensors; the reference does two cudaMemcpy2D per layer (src/model.cpp:835-843).
template <typename T>
__global__ void kv_cache_fill_kernel(T* __restrict__ k_cache, T* __restrict__ v_cache,
                                     int32_t* __restrict__ lengths, const float* __restrict__ k_heads,
                                     const float* __restrict__ v_heads, int b, int H, int n, int max_len,
                                     int D) {
  const int64_t per = static_cast<int64_t>(H) * n * D / 4;   // float4 groups per tensor
  const int64_t t = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t == 0 && lengths) lengths[b] = n;
  if (t >= 2 * per) return;
  const bool is_v = t >= per;
  const int64_t i = (is_v ? t - per : t) * 4;         // element index in [H, n, D]
  const int64_t h = i / (static_cast<int64_t>(n) * D), rem = i - h * n * D;
  const float4 x = *reinterpret_cast<const float4*>((is_v ? v_heads : k_heads) + i);
  T* dst = (is_v ? v_cache : k_cache) + ((static_cast<int64_t>(b) * H + h) * max_len) * D + rem;
  dst[0] = Elem<T>::from_float(x.x);
  dst[1] = Elem<T>::from_float(x.y);
  dst[2] = Elem<T>::from_float(x.z);
  dst[3] = Elem<T>::from_float(x.w);
}

int check_decode_bf16(const void* out, const void* q, const void* k_new, const void* v_new,
                      const void* k_cache, const void* v_cache, const void* lengths, int B, int H,
                      int D, int max_len) {
  if (!out || !q || !k_new || !v_new || !k_cache || !v_cache || !lengths)
    return fail(DADATTN_E_ARG, "decode: null pointer");
  if (B <= 0 || H <= 0 || max_len <= 0 || H > 65535 ||
      static_cast<long long>(B) * H > 0x7fffffffLL)
    return fail(DADATTN_E_ARG, "decode: bad sizes B=%d H=%d max_len=%d", B, H, max_len);
  if (D != 64 && D != 128) return fail(DADATTN_E_UNSUPPORTED, "decode bf16: unsupported D %d", D);
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16) ||
      !aligned(k_cache, 16) || !aligned(v_cache, 16))
    return fail(DADATTN_E_ARG, "decode: pointers must be 16-byte aligned");
  return DADATTN_OK;
}

thread_local int g_decode_early = 0;

}  // namespace
}  // namespace dadattn

using namespace dadattn;

extern "C" size_t dadattn_decode_workspace_bytes(int B, int H, int D, int max_len) {
  if (B <= 0 || H <= 0 || D <= 0 || max_len <= 0) return 0;
  return workspace_bytes(B, H, D, max_len);
}

extern "C" int dadattn_decode_bf16(uint16_t* out, const uint16_t* q, const uint16_t* k_new,
                                   const uint16_t* v_new, uint16_t* k_cache, uint16_t* v_cache,
                                   int32_t* lengths, int B, int H, int D, int max_len,
                                   float scale, void* workspace, size_t workspace_bytes_given,
                                   dadattn_stream_t stream) {
  if (int rc = check_decode_bf16(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H, D, max_len))
    return rc;
  if (!workspace || !aligned(workspace, 16))
    return fail(DADATTN_E_ARG, "decode: workspace must be a 16-byte aligned device pointer");
  if (workspace_bytes_given < workspace_bytes(B, H, D, max_len))
    return fail(DADATTN_E_WORKSPACE, "decode: workspace %zu < %zu bytes", workspace_bytes_given,
                workspace_bytes(B, H, D, max_len));
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned* tickets = static_cast<unsigned*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + ticket_bytes(B, H));
  return D == 64 ? launch_decode_bf16<64>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H,
                                          max_len, scale, tickets, partial, status, g_decode_early, st)
                 : launch_decode_bf16<128>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H,
                                           max_len, scale, tickets, partial, status, g_decode_early, st);
}

extern "C" int dadattn_set_decode_early_start(int on) {
  g_decode_early = on ? 1 : 0;
  return DADATTN_OK;
}

extern "C" int dadattn_decode_f32(float* out, const float* q, const float* k_new,
                                  const float* v_new, float* k_cache, float* v_cache, int H,
                                  int max_len, int D, int pos, float scale,
                                  dadattn_stream_t stream) {
  if (!out || !q || !k_new || !v_new || !k_cache || !v_cache)
    return fail(DADATTN_E_ARG, "decode: null pointer");
  if (H <= 0 || max_len <= 0 || H > 65535) return fail(DADATTN_E_ARG, "decode: bad sizes");
  if (pos < 0 || pos >= max_len)
    return fail(DADATTN_E_ARG, "decode: pos %d outside context length %d", pos, max_len);
  if (D != 16 && D != 32 && D != 64 && D != 128)
    return fail(DADATTN_E_UNSUPPORTED, "decode f32: unsupported D %d", D);
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16) ||
      !aligned(k_cache, 16) || !aligned(v_cache, 16))
    return fail(DADATTN_E_ARG, "decode: pointers must be 16-byte aligned");
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(H, 1);  // one CTA per head walks the whole cache: direct mode, no workspace
#define DAD_DECODE32(DH)                                                                        \
  case DH:                                                                                      \
    DAD_CUDA(launch_pdl(decode_splitk_kernel<float, DH>, grid, dim3(kDecodeThreads), 0, st, out, \
                               static_cast<float*>(nullptr), static_cast<unsigned*>(nullptr),   \
                               static_cast<unsigned*>(nullptr), q, k_new, v_new, k_cache,       \
                               v_cache, static_cast<int32_t*>(nullptr), pos, H, max_len,        \
                               max_len, 0, 0, scale, status));                                  \
    break;
  switch (D) {
    DAD_DECODE32(16) DAD_DECODE32(32) DAD_DECODE32(64) DAD_DECODE32(128)
  }
#undef DAD_DECODE32
  return DADATTN_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode without any allocation.
//
// Some hosts of this library must not allocate device memory once they are running: a serving
// process that hands every free byte of HBM to its own cache pool at start-up has nothing left
// for a later cudaMalloc; a latency-critical decode loop cannot afford the device-wide
// synchronisation an allocation implies; and DadGPT itself sizes all of its buffers once, in
// model_alloc / kv_cache_alloc, and never allocates inside generate_tokens. For such callers the
// split-K tickets and records live in the fixed array below instead of a caller-provided
// workspace, and the bad-length report goes to a fixed word instead of the lazily allocated
// status word.
//
// The array is part of the library image: every GPU that loads libdadattn.so holds these
// 8 MiB until the process exits, whether or not this entry point is ever called. Its first
// 64 KiB are the tickets, at a fixed place whatever the shape of a call: they are zero when the
// module is loaded and every call returns them to zero, which is the only state a call needs
// from its predecessors. The records behind them are written before they are read.
// A sequence that is already at max_len is skipped and noted in g_decode_noalloc_status, which
// dadattn_decode_noalloc_status() reads and clears (a symbol copy: no allocation either).
// ---------------------------------------------------------------------------------------------
namespace dadattn {
namespace {

constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;
constexpr size_t kNoAllocTicketBytes = size_t(64) << 10;
static __device__ __align__(256) unsigned char g_decode_scratch[kNoAllocScratchBytes];
static __device__ int g_decode_noalloc_status;

constexpr int kNoAllocMaxDevices = 64;
float* g_scratch_ptr[kNoAllocMaxDevices] = {};
int* g_noalloc_status_ptr[kNoAllocMaxDevices] = {};

// In host code the names g_decode_scratch / g_decode_noalloc_status are only handles; the
// device addresses a kernel can use come from cudaGetSymbolAddress, per device, with that
// device current. Looked up on the first call on each device and cached.
int noalloc_setup(float** scratch, int** status) {
  int dev = 0;
  DAD_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices)
    return fail(DADATTN_E_UNSUPPORTED, "device ordinal %d not supported", dev);
  if (!g_scratch_ptr[dev] || !g_noalloc_status_ptr[dev]) {
    float* s = nullptr;
    int* w = nullptr;
    DAD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&s), g_decode_scratch));
    DAD_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&w), g_decode_noalloc_status));
    g_noalloc_status_ptr[dev] = w;
    g_scratch_ptr[dev] = s;
  }
  *scratch = g_scratch_ptr[dev];
  *status = g_noalloc_status_ptr[dev];
  return DADATTN_OK;
}

}  // namespace
}  // namespace dadattn

extern "C" int dadattn_decode_bf16_noalloc(uint16_t* out, const uint16_t* q,
                                           const uint16_t* k_new, const uint16_t* v_new,
                                           uint16_t* k_cache, uint16_t* v_cache, int32_t* lengths,
                                           int B, int H, int D, int max_len, float scale,
                                           dadattn_stream_t stream) {
  if (int rc = check_decode_bf16(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H, D, max_len))
    return rc;
  const size_t need_tickets = ticket_bytes(B, H), need_records = record_bytes(B, H, D, max_len);
  if (need_tickets > kNoAllocTicketBytes || need_records > kNoAllocScratchBytes - kNoAllocTicketBytes)
    return fail(DADATTN_E_WORKSPACE,
                "decode (no-alloc): B=%d H=%d D=%d max_len=%d needs %zu bytes of tickets and %zu "
                "bytes of split-K records; the built-in array of %zu bytes holds %zu and %zu; use "
                "dadattn_decode_bf16 with your own workspace",
                B, H, D, max_len, need_tickets, need_records,
                static_cast<size_t>(kNoAllocScratchBytes), static_cast<size_t>(kNoAllocTicketBytes),
                static_cast<size_t>(kNoAllocScratchBytes - kNoAllocTicketBytes));
  float* scratch = nullptr;
  int* status = nullptr;
  if (int rc = noalloc_setup(&scratch, &status)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned* tickets = reinterpret_cast<unsigned*>(scratch);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kNoAllocTicketBytes);
  // never with early start: every call shares the one scratch array with the call before it
  return D == 64 ? launch_decode_bf16<64>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H,
                                          max_len, scale, tickets, partial, status, 0, st)
                 : launch_decode_bf16<128>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H,
                                           max_len, scale, tickets, partial, status, 0, st);
}

extern "C" int dadattn_decode_noalloc_status(dadattn_stream_t stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int host = 0;
  const int zero = 0;
  DAD_CUDA(cudaMemcpyFromSymbolAsync(&host, g_decode_noalloc_status, sizeof(int), 0,
                                     cudaMemcpyDeviceToHost, st));
  DAD_CUDA(cudaMemcpyToSymbolAsync(g_decode_noalloc_status, &zero, sizeof(int), 0,
                                   cudaMemcpyHostToDevice, st));
  DAD_CUDA(cudaStreamSynchronize(st));
  if (host == DADATTN_E_ARG)
    fail(host, "decode (no-alloc): a sequence was skipped, its length is outside [0, max_len)");
  else if (host != 0)
    fail(host, "decode (no-alloc): device status %d", host);
  return host;
}

// Batched decode on fp32 caches: the arithmetic of dadattn_decode_f32 for many sequences at once.
extern "C" int dadattn_decode_f32_batched(float* out, const float* q, const float* k_new, const float* v_new,
                                          float* k_cache, float* v_cache, int32_t* lengths, int B, int H,
                                          int D, int max_len, float scale, void* workspace,
                                          size_t workspace_bytes_given, dadattn_stream_t stream) {
  if (!out || !q || !k_new || !v_new || !k_cache || !v_cache || !lengths)
    return fail(DADATTN_E_ARG, "decode: null pointer");
  if (B <= 0 || H <= 0 || max_len <= 0 || H > 65535 || static_cast<long long>(B) * H > 0x7fffffffLL)
    return fail(DADATTN_E_ARG, "decode: bad sizes B=%d H=%d max_len=%d", B, H, max_len);
  if (D != 16 && D != 32 && D != 64 && D != 128)
    return fail(DADATTN_E_UNSUPPORTED, "decode f32: unsupported D %d", D);
  if (!aligned(out, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16) ||
      !aligned(k_cache, 16) || !aligned(v_cache, 16))
    return fail(DADATTN_E_ARG, "decode: pointers must be 16-byte aligned");
  if (!workspace || !aligned(workspace, 16))
    return fail(DADATTN_E_ARG, "decode: workspace must be a 16-byte aligned device pointer");
  if (workspace_bytes_given < workspace_bytes(B, H, D, max_len))
    return fail(DADATTN_E_WORKSPACE, "decode: workspace %zu < %zu bytes", workspace_bytes_given,
                workspace_bytes(B, H, D, max_len));
  int* status = device_status_word();
  if (!status) return DADATTN_E_CUDA;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned* tickets = static_cast<unsigned*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + ticket_bytes(B, H));
  switch (D) {
    case 16: return launch_decode_batched<float, float, 16>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H, max_len, scale, tickets, partial, status, 0, st);
    case 32: return launch_decode_batched<float, float, 32>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H, max_len, scale, tickets, partial, status, 0, st);
    case 64: return launch_decode_batched<float, float, 64>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H, max_len, scale, tickets, partial, status, 0, st);
    default: return launch_decode_batched<float, float, 128>(out, q, k_new, v_new, k_cache, v_cache, lengths, B, H, max_len, scale, tickets, partial, status, 0, st);
  }
}

extern "C" int dadattn_kv_cache_fill(void* k_cache, void* v_cache, int32_t* lengths, const float* k_heads,
                                     const float* v_heads, int b, int B, int H, int n, int max_len, int D,
                                     int cache_is_bf16, dadattn_stream_t stream) {
  if (!k_cache || !v_cache || !k_heads || !v_heads) return fail(DADATTN_E_ARG, "cache fill: null pointer");
  if (B <= 0 || H <= 0 || D <= 0 || D % 4 != 0 || b < 0 || b >= B || n < 1 || n > max_len)
    return fail(DADATTN_E_ARG, "cache fill: bad sizes b=%d B=%d H=%d n=%d max_len=%d D=%d", b, B, H, n, max_len, D);
  if (!aligned(k_heads, 16) || !aligned(v_heads, 16))
    return fail(DADATTN_E_ARG, "cache fill: k_heads / v_heads must be 16-byte aligned");
  const int64_t groups = 2 * (static_cast<int64_t>(H) * n * D / 4);
  const unsigned blocks = static_cast<unsigned>((groups + 255) / 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cache_is_bf16)
    kv_cache_fill_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<__nv_bfloat16*>(k_cache),
                                                                static_cast<__nv_bfloat16*>(v_cache), lengths,
                                                                k_heads, v_heads, b, H, n, max_len, D);
  else
    kv_cache_fill_kernel<float><<<blocks, 256, 0, st>>>(static_cast<float*>(k_cache), static_cast<float*>(v_cache),
                                                        lengths, k_heads, v_heads, b, H, n, max_len, D);
  DAD_LAUNCH_CHECK("kv_cache_fill_kernel");
  return DADATTN_OK;
}
