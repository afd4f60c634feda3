// placeholder until the tcgen05 kernels land (replaced in the next commit)
#include "common.cuh"
using namespace dadattn;
extern "C" int dadattn_flash_bf16_supported(int d) { return d == 64 || d == 128; }
extern "C" int dadattn_flash_fwd_bf16(uint16_t*, float*, const uint16_t*, const uint16_t*, const uint16_t*, int, int, int, float, float, uint64_t, uint64_t, int64_t, dadattn_stream_t) { return fail(DADATTN_E_UNSUPPORTED, "bf16 forward not built"); }
extern "C" size_t dadattn_flash_bwd_bf16_workspace_bytes(int BH, int S, int D) { return (size_t)BH * S * (D + 1) * 4; }
extern "C" int dadattn_flash_bwd_bf16(uint16_t*, uint16_t*, uint16_t*, void*, size_t, const uint16_t*, const uint16_t*, const float*, const uint16_t*, const uint16_t*, const uint16_t*, int, int, int, float, float, uint64_t, uint64_t, int64_t, dadattn_stream_t) { return fail(DADATTN_E_UNSUPPORTED, "bf16 backward not built"); }
