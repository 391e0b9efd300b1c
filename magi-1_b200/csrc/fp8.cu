// FP8 e4m3 path: block quantiser, FP8 cache pages, FP8 attention forward.
#include "common.cuh"

namespace magi {

int launch_attn_fp8(magi_ctx* ctx, const magi_attn_params*, int, cudaStream_t) {
  return set_err(ctx, MAGI_E_BADARG, "fp8 attention is not built in this version");
}
int launch_cache_quant_append(magi_kv_cache* c, int, const void*, int64_t, int64_t, const void*, int64_t, int64_t, int,
                              int, cudaStream_t) {
  return set_err(c->ctx, MAGI_E_BADARG, "fp8 cache is not built in this version");
}
int launch_cache_dequant_read(magi_kv_cache* c, int, void*, void*, int, int, cudaStream_t) {
  return set_err(c->ctx, MAGI_E_BADARG, "fp8 cache is not built in this version");
}

}  // namespace magi

extern "C" int magi_quantize_e4m3_block128(magi_ctx* ctx, const void*, int64_t, int64_t, int, int, int, void*, float*,
                                           void*) {
  return magi::set_err(ctx, MAGI_E_BADARG, "fp8 quantiser is not built in this version");
}
