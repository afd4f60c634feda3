/*
 * dadattn — C ABI of the B200 (sm_100a) causal-attention library for DadGPT.
 *
 * Every entry point takes plain device pointers and sizes, enqueues work on the given CUDA
 * stream (pass NULL for the legacy default stream, which is what DadGPT itself uses) and
 * returns without synchronising. Return value: 0 on success, a negative DADATTN_E_* code
 * otherwise; dadattn_last_error() then describes the failure (thread-local string).
 * All tensors and workspaces belong to the caller. What the library itself holds on a device:
 *  - two 4-byte status words (see dadattn_device_status), allocated with cudaMalloc by the first
 *    bf16, decode or fp32-decode call on that device and kept until exit. Because of that
 *    allocation the FIRST such call on a device must come before any stream capture; later
 *    calls allocate nothing;
 *  - the grow-only buffer behind dadattn_library_scratch, only if that function is called;
 *  - an 8 MiB array in the library image for dadattn_decode_bf16_noalloc (no allocation call).
 * There is no CPU fallback: without a CUDA device every compute call fails.
 *
 * Device-side waits are bounded. If one runs out, the kernel records DADATTN_E_TIMEOUT and
 * exits; copies and tensor-core operations it had in flight may still land afterwards, so every
 * result enqueued on that device up to the next dadattn_device_status() call is void.
 *
 * Tensor layouts follow DadGPT: heads already split, [BH, S, D] contiguous, row-major;
 * lse / delta are [BH, S] fp32. "bf16" pointers are raw 16-bit bfloat16 (uint16_t here so the
 * header needs no CUDA include).
 */
#ifndef DADATTN_H_
#define DADATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DADATTN_OK 0
#define DADATTN_E_ARG (-1)         /* null pointer, non-positive size, misaligned pointer */
#define DADATTN_E_UNSUPPORTED (-2) /* head dimension or size outside what the kernels cover */
#define DADATTN_E_CUDA (-3)        /* a CUDA runtime/driver call failed */
#define DADATTN_E_TIMEOUT (-4)     /* a bounded device-side wait ran out (see dadattn_device_status) */
#define DADATTN_E_WORKSPACE (-5)   /* workspace too small */

typedef void* dadattn_stream_t; /* cudaStream_t */

const char* dadattn_last_error(void);
/* Library/kernels version string, e.g. "dadattn 0.1 sm_100a". */
const char* dadattn_version(void);

/* ---- fp32 drop-in path ---------------------------------------------------------------- */

/* Replaces gpu_flash_attention_supported (reference cuda/gpu_ops.cuh:115, cuda/attention.cu:232).
 * Returns 1 for the head sizes the fp32 kernels cover: 16, 32, 64, 128. */
int dadattn_flash_supported(int d_head);

/* Replaces gpu_flash_attention_forward (reference cuda/gpu_ops.cuh:116-117,
 * cuda/attention.cu:234-239): out = softmax(causal(q k^T * scale)) v, lse = rowmax + ln(rowsum)
 * of the scaled scores. q,k,v,out: [BH,S,d_head] fp32; lse: [BH,S] fp32. */
int dadattn_flash_fwd_f32(float* out, float* lse, const float* q, const float* k, const float* v,
                          int BH, int S, int d_head, float scale, dadattn_stream_t stream);

/* Replaces gpu_flash_attention_backward (reference cuda/gpu_ops.cuh:118-122,
 * cuda/attention.cu:241-252). Writes (does not accumulate) dq, dk, dv; delta: [BH,S] scratch
 * owned by the caller, overwritten. */
int dadattn_flash_bwd_f32(float* dq, float* dk, float* dv, float* delta, const float* dout,
                          const float* out, const float* lse, const float* q, const float* k,
                          const float* v, int BH, int S, int d_head, float scale,
                          dadattn_stream_t stream);

/* The same two calls with attention-probability dropout fused in, reproducing the reference's
 * materialized branch (src/model.cpp:406-415 forward, :595-602 backward; mask from
 * dropout_forward_kernel, cuda/gpu_ops.cu:712-727): score element (bh,r,c) is dropped iff the
 * Philox4x32-10 uniform of subsequence ((unit0+bh)*S + r)*S + c, offset `offset`, seed `seed`
 * is < rate; kept probabilities are scaled by 1/(1-rate) after normalisation; lse is that of the
 * undropped softmax. rate = 0 gives exactly the calls above. unit0 is the global index of the
 * first (batch,head) unit of this call (0 unless the BH axis is sharded). */
int dadattn_flash_fwd_f32_dropout(float* out, float* lse, const float* q, const float* k,
                                  const float* v, int BH, int S, int d_head, float scale,
                                  float rate, uint64_t seed, uint64_t offset, int64_t unit0,
                                  dadattn_stream_t stream);
int dadattn_flash_bwd_f32_dropout(float* dq, float* dk, float* dv, float* delta,
                                  const float* dout, const float* out, const float* lse,
                                  const float* q, const float* k, const float* v, int BH, int S,
                                  int d_head, float scale, float rate, uint64_t seed,
                                  uint64_t offset, int64_t unit0, dadattn_stream_t stream);

/* ---- dropout mask ---------------------------------------------------------------------- */

/* Replaces the mask output of gpu_dropout_forward (reference cuda/gpu_ops.cuh:126-127,
 * cuda/gpu_ops.cu:712-734) for flat elements first .. first+n-1: mask[i] = 0 if dropped, 1 if
 * kept. The reference's seed is a process counter (cuda/gpu_ops.cu:704,732); here it is an
 * argument. */
int dadattn_dropout_mask(uint8_t* mask, int64_t n, float rate, uint64_t seed, uint64_t offset,
                         int64_t first, dadattn_stream_t stream);

/* The same mask, bit-packed for the fused bf16 kernels, lower triangle only. The reference
 * materialises its mask as one byte per probability, [BH,S,S], and reads it back in the backward
 * (src/model.cpp:406-415,595-602); drawing it costs ten Philox rounds per probability, far more
 * than the attention arithmetic itself. This call draws it ONCE per (seed, offset, shape) into
 * `bits`; dadattn_flash_fwd_bf16_masked and dadattn_flash_bwd_bf16_masked then read 2 KB per
 * 128 x 128 tile instead of each repeating the draw. Layout: for every (batch x head bh, query
 * tile qt, key tile kt <= qt) in the order bh, qt (qt + 1) / 2 + kt, 128 records of 16 bytes, one
 * per query row of the tile; bit i of 32-bit word w of a record = key 128 kt + 32 w + i, 1 = kept.
 * Bits above the diagonal and rows beyond S are 0. unit0 as in dadattn_flash_fwd_f32_dropout.
 * `bits`: 16-byte aligned device buffer of at least dadattn_dropout_mask_bits_bytes(BH, S)
 * bytes. No counterpart signature in the reference (its mask is gpu_dropout_forward's output,
 * cuda/gpu_ops.cu:729-734). */
size_t dadattn_dropout_mask_bits_bytes(int BH, int S);
int dadattn_dropout_mask_bits(uint32_t* bits, size_t bits_bytes, int BH, int S, float rate,
                              uint64_t seed, uint64_t offset, int64_t unit0,
                              dadattn_stream_t stream);

/* ---- bf16 tensor-core path (tcgen05 / TMEM / TMA) ---------------------------------------- */

/* Head sizes the bf16 kernels cover (64, 128). */
int dadattn_flash_bf16_supported(int d_head);

/* bf16 form of gpu_flash_attention_forward (reference cuda/attention.cu:234-239 is the fp32
 * original): q,k,v,out bf16 [BH,S,D], fp32 softmax and accumulation, lse fp32 [BH,S] in the
 * reference's convention (natural log, scaled scores). Dropout arguments as above. All tensor
 * pointers must be 16-byte aligned. */
int dadattn_flash_fwd_bf16(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k,
                           const uint16_t* v, int BH, int S, int D, float scale, float rate,
                           uint64_t seed, uint64_t offset, int64_t unit0,
                           dadattn_stream_t stream);

/* bf16 form of gpu_flash_attention_backward (reference cuda/attention.cu:241-252). dq,dk,dv bf16,
 * written not accumulated. workspace: caller-owned scratch of at least
 * dadattn_flash_bwd_bf16_workspace_bytes(BH,S,D) bytes, 256-byte aligned (it takes the place of
 * the fp32 call's `delta` scratch and also holds the fp32 dQ accumulator of the single-pass
 * kernels, 4*BH*S*D bytes; contents are overwritten). */
size_t dadattn_flash_bwd_bf16_workspace_bytes(int BH, int S, int D);
int dadattn_flash_bwd_bf16(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                           size_t workspace_bytes, const uint16_t* dout, const uint16_t* out,
                           const float* lse, const uint16_t* q, const uint16_t* k,
                           const uint16_t* v, int BH, int S, int D, float scale, float rate,
                           uint64_t seed, uint64_t offset, int64_t unit0,
                           dadattn_stream_t stream);

/* dadattn_flash_fwd_bf16 / dadattn_flash_bwd_bf16 with the dropout mask taken from `mask_bits`
 * (dadattn_dropout_mask_bits, drawn with the same BH, S, rate and the caller's seed, offset and
 * unit0) instead of being drawn inside the kernels: same results bit for bit, a fraction of the
 * time. Head size 64 only; the backward must be the single-pass one (the default). */
int dadattn_flash_fwd_bf16_masked(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k,
                                  const uint16_t* v, int BH, int S, int D, float scale, float rate,
                                  const uint32_t* mask_bits, dadattn_stream_t stream);
int dadattn_flash_bwd_bf16_masked(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                                  size_t workspace_bytes, const uint16_t* dout, const uint16_t* out,
                                  const float* lse, const uint16_t* q, const uint16_t* k,
                                  const uint16_t* v, int BH, int S, int D, float scale, float rate,
                                  const uint32_t* mask_bits, dadattn_stream_t stream);

/* The same two calls on the activations BEFORE the reference's head split: q, k, v, out, dout,
 * dq, dk, dv are [B*S, H*D] row-major (row = b S + s, column = h D + d), exactly what the
 * projections write and read (reference src/model.cpp:372-387,423,564,619-624), so the three
 * gpu_split_heads copies before and the gpu_merge_heads copy after the forward, and the one split
 * and three merges around the backward (cuda/gpu_ops.cu:428-474), are not needed: the kernels
 * address the rows of a (batch, head) unit through strided tensor maps. lse stays [B*H, S];
 * results equal split -> dadattn_flash_*_bf16 -> merge. Head size 64; the backward must be the
 * single-pass one (the default). workspace as for dadattn_flash_bwd_bf16 with BH = B*H. No
 * counterpart signature in the reference. */
int dadattn_flash_fwd_bf16_strided(uint16_t* out, float* lse, const uint16_t* q, const uint16_t* k,
                                   const uint16_t* v, int B, int H, int S, int D, float scale,
                                   float rate, uint64_t seed, uint64_t offset, int64_t unit0,
                                   dadattn_stream_t stream);
int dadattn_flash_bwd_bf16_strided(uint16_t* dq, uint16_t* dk, uint16_t* dv, void* workspace,
                                   size_t workspace_bytes, const uint16_t* dout, const uint16_t* out,
                                   const float* lse, const uint16_t* q, const uint16_t* k,
                                   const uint16_t* v, int B, int H, int S, int D, float scale,
                                   float rate, uint64_t seed, uint64_t offset, int64_t unit0,
                                   dadattn_stream_t stream);

/* By default the backward is a single-pass kernel (one per head size) that forms the
 * probabilities once and adds each key tile's dQ contribution into an fp32 accumulator in the
 * workspace (TMA / bulk reduce-add): about 1.4-2x as fast as recomputing them, but the order of
 * those additions is not fixed, so dQ may differ in its last bits between runs (dK and dV do
 * not). dadattn_set_bwd_deterministic(1) makes the calling thread use the two-kernel backward,
 * which like the reference (cuda/attention.cu:4-6) accumulates nothing across thread blocks;
 * 0 (the default) restores the single-pass kernels. No counterpart in the reference. */
int dadattn_set_bwd_deterministic(int on);

/* Measurement aid (no counterpart in the reference): when `events` (an array of `count`
 * cudaEvent_t) is set for the calling thread, dadattn_flash_bwd_bf16 records events[i] on the
 * call's stream before its i-th kernel and one more event after its last kernel. The single-pass
 * backward launches three kernels (delta and workspace clear, the fused gradient kernel,
 * fp32 -> bf16 of dQ: four events); the two-kernel backward launches dQ, then dK/dV
 * (three events). Events beyond `count` are not recorded. Pass NULL to switch it off. */
int dadattn_set_stage_events(void** events, int count);

/* ---- fp32 tensors, tensor-core arithmetic ---------------------------------------------------- */

/* The reference keeps activations in fp32 and lowers precision per operation:
 * gpu_set_matmul_precision(BF16) (reference cuda/gpu_ops.cuh:43-44; the training default,
 * src/train.hpp:29) makes its GEMMs round operands to bf16 and accumulate in fp32. These calls
 * give the fused attention the same contract on the reference's own fp32 tensors: operands are
 * rounded to bf16 into `workspace`, the bf16 tensor-core kernels run (fp32 softmax and
 * accumulation), results are widened back to fp32; lse is written in fp32 directly. Argument
 * meaning as dadattn_flash_fwd_f32 / dadattn_flash_bwd_f32 (no `delta`: the workspace holds it).
 * D must be 64 or 128, scale > 0, tensors 16-byte aligned, workspace 256-byte aligned and at
 * least dadattn_flash_f32_via_bf16_workspace_bytes(BH,S,D) bytes (its contents need not
 * survive between calls). No counterpart in the reference, whose fused kernels are fp32 only. */
size_t dadattn_flash_f32_via_bf16_workspace_bytes(int BH, int S, int D);
int dadattn_flash_fwd_f32_via_bf16(float* out, float* lse, const float* q, const float* k,
                                   const float* v, int BH, int S, int D, float scale,
                                   void* workspace, size_t workspace_bytes,
                                   dadattn_stream_t stream);
int dadattn_flash_bwd_f32_via_bf16(float* dq, float* dk, float* dv, const float* dout,
                                   const float* out, const float* lse, const float* q,
                                   const float* k, const float* v, int BH, int S, int D,
                                   float scale, void* workspace, size_t workspace_bytes,
                                   dadattn_stream_t stream);

/* Process-wide precision of the drop-in symbols gpu_flash_attention_forward / _backward
 * (libdadattn_gpuops.so): 0 = the exact fp32 kernels (default), 1 = the calls above at head size
 * 64 (other head sizes stay fp32). A host that calls the reference's
 * gpu_set_matmul_precision(MatmulPrecision::BF16) calls dadattn_set_f32_precision(1) next to it;
 * without any call the environment variable DADATTN_PRECISION=bf16 selects 1. */
int dadattn_set_f32_precision(int mode);
int dadattn_get_f32_precision(void);

/* A grow-only device buffer owned by the library, one per device, for hosts that have no way to
 * pass a workspace (the drop-in symbols above: the reference's signatures carry none). Allocates
 * (cudaMalloc) on first use and when `bytes` exceeds what it holds, after waiting for the
 * device to finish work on the old buffer; every other library entry point allocates nothing.
 * The buffer is shared: calls that use it must not overlap on the GPU. */
int dadattn_library_scratch(size_t bytes, void** ptr);

/* ---- KV-cache decode --------------------------------------------------------------------- */

/* Decode attention of model_forward_cached for ONE sequence on the reference's own cache
 * (reference src/model.cpp:745-790; struct KVCache src/model.hpp:140-152): appends k_new,v_new
 * [H*D] at row `pos` of k_cache,v_cache [H,max_len,D] fp32, then out[h] =
 * softmax(q_h K_h[0..pos]^T * scale) V_h[0..pos]. Returns DADATTN_E_ARG when pos is outside
 * [0, max_len) (the reference throws std::out_of_range, src/model.cpp:693-696). */
int dadattn_decode_f32(float* out, const float* q, const float* k_new, const float* v_new,
                       float* k_cache, float* v_cache, int H, int max_len, int D, int pos,
                       float scale, dadattn_stream_t stream);

/* Batched bf16 decode for many concurrent sequences (no counterpart signature in the reference,
 * which decodes one fp32 sequence at a time; the arithmetic is that of src/model.cpp:758-790).
 * Caches: [B,H,max_len,D] bf16. lengths[B] (int32, device) holds each sequence's current length
 * L_b; the call writes k_new,v_new [B,H,D] at row L_b, attends over rows 0..L_b, and stores
 * L_b + 1 back. Sequences with L_b >= max_len are left untouched and reported through
 * DADATTN_E_ARG at the next dadattn_device_status(). workspace: split-K tickets and records, at
 * least dadattn_decode_workspace_bytes() bytes, 16-byte aligned. It must be zero-filled
 * (cudaMemset) before its first use and again whenever B, H or max_len change; between calls of
 * one shape the library leaves it in a reusable state. Two calls that share a workspace must not
 * overlap on the GPU. */
size_t dadattn_decode_workspace_bytes(int B, int H, int D, int max_len);
int dadattn_decode_bf16(uint16_t* out, const uint16_t* q, const uint16_t* k_new,
                        const uint16_t* v_new, uint16_t* k_cache, uint16_t* v_cache,
                        int32_t* lengths, int B, int H, int D, int max_len, float scale,
                        void* workspace, size_t workspace_bytes, dadattn_stream_t stream);

/* dadattn_decode_f32 for B sequences at once, on fp32 caches [B,H,max_len,D] with lengths[B] as in
 * dadattn_decode_bf16 (same workspace rules, dadattn_decode_workspace_bytes). Head sizes 16, 32,
 * 64, 128. This is what a batched generation loop over the reference's fp32 model calls once per
 * layer; results equal B separate dadattn_decode_f32 calls. No counterpart in the reference, which
 * decodes one sequence at a time (src/generate.cpp:94-139). */
int dadattn_decode_f32_batched(float* out, const float* q, const float* k_new, const float* v_new,
                               float* k_cache, float* v_cache, int32_t* lengths, int B, int H, int D,
                               int max_len, float scale, void* workspace, size_t workspace_bytes,
                               dadattn_stream_t stream);

/* Fills sequence b of a batched cache from a prefill: k_heads, v_heads [H, n, D] fp32 (what the
 * reference's model_forward leaves in k_heads / v_heads for batch 1) go to rows 0..n-1 of
 * k_cache, v_cache [B,H,max_len,D] — bf16 (rounded to nearest even) when cache_is_bf16, else fp32
 * — and lengths[b] becomes n (lengths may be NULL). One launch for both tensors; replaces the two
 * cudaMemcpy2D per layer of model_prefill (reference src/model.cpp:835-843), which can neither
 * convert nor address a batch entry. */
int dadattn_kv_cache_fill(void* k_cache, void* v_cache, int32_t* lengths, const float* k_heads,
                          const float* v_heads, int b, int B, int H, int n, int max_len, int D,
                          int cache_is_bf16, dadattn_stream_t stream);

/* Lets dadattn_decode_bf16 calls of the calling thread start early: the kernel reads `lengths`
 * and each warp's first cache rows while the kernel ahead of it in the stream is still draining,
 * and waits for that kernel only before it touches q, k_new and v_new. The caller thereby
 * promises that the kernel ahead does not write THIS call's k_cache, v_cache, lengths or
 * workspace. That holds for the layers of a model with two or more layers, each with its own
 * cache and workspace (the call ahead of layer l's attention is layer l's projection, and the
 * previous write to this cache was a whole step ago); it does not hold for back-to-back calls
 * on one cache, which would see a stale length. 0 (the default) restores the fully ordered
 * behaviour. dadattn_decode_bf16_noalloc and dadattn_decode_f32 never start early. No counterpart
 * in the reference. */
int dadattn_set_decode_early_start(int on);

/* dadattn_decode_bf16 for callers that cannot allocate device memory or hand over a workspace
 * (no counterpart in the reference). Typical cases: a server that gave all remaining HBM to its
 * own KV-cache pool at start-up, a decode loop that must not hit the device-wide stall of an
 * allocation, or DadGPT's own generation loop, which sizes every buffer once in kv_cache_alloc
 * and never allocates afterwards. Same arguments and results as dadattn_decode_bf16 minus the
 * workspace: the split-K partials go to a fixed 8 MiB array inside the library image (held by
 * every GPU that loads the library, until exit). The call performs no cudaMalloc/cudaFree and
 * uses no allocating routine.
 *  - Limit: the array is 8 MiB (8388608 bytes). Its first 64 KiB hold the tickets, which need
 *    B*H + 33 <= 16384, i.e. B*H <= 16351: that is the binding limit for any shape with
 *    B*H >= 592, where each CTA walks a whole sequence and there are no records at all. With
 *    fewer (sequence, head) pairs the cache rows are split across CTAs and the records
 *    (B*H*splits*(D+2)*4 bytes, at most ~5 splits) must fit in the remaining 8 MiB - 64 KiB,
 *    which they do for every max_len up to about 100 000 rows at D = 64.
 *    dadattn_decode_workspace_bytes(B,H,D,max_len) tells what a shape needs; shapes beyond the
 *    array return DADATTN_E_WORKSPACE.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call before starting any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents. Only the tickets
 *    have to be zero when a call starts: they are zero when the library is loaded and every call
 *    hands them back zeroed (records are written before they are read within a call). Two calls
 *    that overlap on the GPU (different streams, or threads) race on the array: serialise them.
 *  - A sequence already at max_len is skipped as in dadattn_decode_bf16 and noted in a word
 *    beside the array; dadattn_decode_noalloc_status reads it (dadattn_device_status belongs to
 *    the allocating calls and does not see it). */
int dadattn_decode_bf16_noalloc(uint16_t* out, const uint16_t* q, const uint16_t* k_new,
                                const uint16_t* v_new, uint16_t* k_cache, uint16_t* v_cache,
                                int32_t* lengths, int B, int H, int D, int max_len, float scale,
                                dadattn_stream_t stream);
/* Waits for `stream`, then returns and clears the status word of dadattn_decode_bf16_noalloc on
 * the current device: 0, or DADATTN_E_ARG when a call since the last read skipped a sequence
 * whose length was outside [0, max_len). Copies from and to a symbol of the library image, so it
 * allocates nothing either. No counterpart in the reference. */
int dadattn_decode_noalloc_status(dadattn_stream_t stream);

/* Synchronises the stream and returns the sticky device-side status word of this device
 * (0, or a DADATTN_E_* code recorded by a kernel: a bounded wait that ran out, a sequence at
 * max_len). Clears the word. For a wait that ran out dadattn_last_error() names the source line
 * of that wait inside its kernel. */
int dadattn_device_status(dadattn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* DADATTN_H_ */
