// C ABI of libmagi_attn.so: contexts, the chunk-paged KV cache and the attention entry points.
#include <math.h>
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace magi {

int launch_attn_bf16(magi_ctx* ctx, const magi_attn_params* p, int max_items, cudaStream_t stream);
int launch_attn_fp8(magi_ctx* ctx, const magi_attn_params* p, int max_items, cudaStream_t stream);
int launch_attn_simt(magi_ctx* ctx, const magi_attn_params* p, int max_items, cudaStream_t stream);
int attn_init_device(magi_ctx* ctx);
int launch_cache_quant_append(magi_kv_cache* c, int slot, const void* k, int64_t kst, int64_t ksh, const void* v,
                              int64_t vst, int64_t vsh, int n_tokens, int token_offset, cudaStream_t stream);
int launch_cache_dequant_read(magi_kv_cache* c, int slot, void* k_out, void* v_out, int n_tokens, int token_offset,
                              cudaStream_t stream);

int set_err(magi_ctx* ctx, int code, const char* fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

int cache_slot(const magi_kv_cache* c, int layer, int chunk_id) {
  if (!c || layer < 0 || layer >= c->d.n_layers || chunk_id < 0 || chunk_id >= c->slot_cap) return -1;
  const int s = c->slot_of_chunk[chunk_id];
  return s < 0 ? -1 : layer * c->d.max_chunks + s;
}

}  // namespace magi

using namespace magi;

extern "C" int magi_version(void) { return 100; }

extern "C" const char* magi_strerror(int code) {
  switch (code) {
    case MAGI_OK: return "ok";
    case MAGI_E_BADARG: return "bad argument";
    case MAGI_E_ALIGN: return "pointer or stride not aligned";
    case MAGI_E_ARCH: return "device is not sm_100";
    case MAGI_E_RANGE: return "inconsistent range or page bookkeeping";
    case MAGI_E_NOMEM: return "out of device memory or fixed capacity exceeded";
    case MAGI_E_NCCL: return "NCCL failure";
    case MAGI_E_TIMEOUT: return "bounded device-side wait gave up";
    case MAGI_E_CUDA: return "CUDA call failed";
    default: return "unknown error";
  }
}

extern "C" int magi_ctx_create(int device, magi_ctx** out) {
  if (!out) return MAGI_E_BADARG;
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return MAGI_E_CUDA;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return MAGI_E_CUDA;
  if (prop.major != 10) return MAGI_E_ARCH;
  int prev = 0;
  cudaGetDevice(&prev);
  if (cudaSetDevice(device) != cudaSuccess) return MAGI_E_CUDA;
  magi_ctx* ctx = static_cast<magi_ctx*>(calloc(1, sizeof(magi_ctx)));
  if (!ctx) return MAGI_E_NOMEM;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  int rc = MAGI_OK;
  if (cudaMalloc(&ctx->workspace, kPlanBytes) != cudaSuccess) rc = MAGI_E_NOMEM;
  if (!rc && cudaMemset(ctx->workspace, 0, kPlanBytes) != cudaSuccess) rc = MAGI_E_CUDA;
  if (!rc) rc = attn_init_device(ctx);
  cudaSetDevice(prev);
  if (rc) {
    if (ctx->workspace) cudaFree(ctx->workspace);
    free(ctx);
    return rc;
  }
  *out = ctx;
  return MAGI_OK;
}

extern "C" int magi_ctx_destroy(magi_ctx* ctx) {
  if (!ctx) return MAGI_E_BADARG;
  if (ctx->workspace) cudaFree(ctx->workspace);
  free(ctx);
  return MAGI_OK;
}

extern "C" const char* magi_last_error(const magi_ctx* ctx) { return ctx ? ctx->err : "null context"; }

extern "C" int magi_ctx_status(magi_ctx* ctx, void* stream, int* device_status) {
  if (!ctx || !device_status) return MAGI_E_BADARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  PlanHeader h;
  MAGI_CUDA_OK(ctx, cudaMemcpyAsync(&h, ctx->workspace, sizeof(h), cudaMemcpyDeviceToHost, st));
  MAGI_CUDA_OK(ctx, cudaStreamSynchronize(st));
  *device_status = h.status;
  if (h.status != 0) {
    h.status = 0;
    MAGI_CUDA_OK(ctx, cudaMemcpyAsync(reinterpret_cast<char*>(ctx->workspace) + offsetof(PlanHeader, status), &h.status,
                                      sizeof(int), cudaMemcpyHostToDevice, st));
    MAGI_CUDA_OK(ctx, cudaStreamSynchronize(st));
  }
  return MAGI_OK;
}

// ------------------------------------------------------------------------------------------- KV cache
extern "C" int magi_kv_cache_create(magi_ctx* ctx, const magi_kv_cache_desc* d, magi_kv_cache** out) {
  if (!ctx || !out) return MAGI_E_BADARG;
  *out = nullptr;
  if (!d || d->struct_size != sizeof(magi_kv_cache_desc)) return set_err(ctx, MAGI_E_BADARG, "kv cache: bad struct_size");
  if (d->n_layers <= 0 || d->max_chunks <= 0 || d->chunk_tokens <= 0 || d->n_kv_heads <= 0)
    return set_err(ctx, MAGI_E_BADARG, "kv cache: sizes must be positive");
  if (d->dtype != MAGI_DTYPE_BF16 && d->dtype != MAGI_DTYPE_FP8_E4M3)
    return set_err(ctx, MAGI_E_BADARG, "kv cache: unknown dtype %d", d->dtype);
  magi_kv_cache* c = static_cast<magi_kv_cache*>(calloc(1, sizeof(magi_kv_cache)));
  if (!c) return MAGI_E_NOMEM;
  c->ctx = ctx;
  c->d = *d;
  c->page_cap = (d->chunk_tokens + kTileN - 1) / kTileN * kTileN;
  c->blocks_per_page = c->page_cap / kTileN;
  c->n_slots = d->n_layers * d->max_chunks;
  const int64_t rows = (int64_t)c->n_slots * c->page_cap;
  if (rows >= (1ll << 31)) {
    free(c);
    return set_err(ctx, MAGI_E_NOMEM, "kv cache: %lld pool rows exceed the 2^31 row addressing of a tensor map", (long long)rows);
  }
  const int esz = d->dtype == MAGI_DTYPE_BF16 ? 2 : 1;
  const size_t pool_bytes = (size_t)rows * d->n_kv_heads * kHeadDim * esz;
  const size_t scale_bytes = d->dtype == MAGI_DTYPE_FP8_E4M3 ? (size_t)c->n_slots * c->blocks_per_page * d->n_kv_heads * 4 : 0;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(ctx->device);
  bool ok = cudaMalloc(&c->k_pool, pool_bytes) == cudaSuccess && cudaMalloc(&c->v_pool, pool_bytes) == cudaSuccess;
  if (ok && scale_bytes)
    ok = cudaMalloc(reinterpret_cast<void**>(&c->k_scale), scale_bytes) == cudaSuccess &&
         cudaMalloc(reinterpret_cast<void**>(&c->v_scale), scale_bytes) == cudaSuccess;
  // Pages are zero-filled once: the rows between chunk_tokens and the 128-aligned page capacity are read
  // (and masked) by the last tile of a page, so they must hold finite values.
  if (ok) ok = cudaMemset(c->k_pool, 0, pool_bytes) == cudaSuccess && cudaMemset(c->v_pool, 0, pool_bytes) == cudaSuccess;
  if (ok && scale_bytes)
    ok = cudaMemset(c->k_scale, 0, scale_bytes) == cudaSuccess && cudaMemset(c->v_scale, 0, scale_bytes) == cudaSuccess;
  cudaSetDevice(prev);
  c->slot_cap = 64;
  c->slot_of_chunk = static_cast<int*>(malloc(sizeof(int) * c->slot_cap));
  c->chunk_of_slot = static_cast<int*>(malloc(sizeof(int) * d->max_chunks));
  if (!ok || !c->slot_of_chunk || !c->chunk_of_slot) {
    cudaGetLastError();
    magi_kv_cache_destroy(c);
    return set_err(ctx, MAGI_E_NOMEM, "kv cache: allocation of %zu bytes failed", 2 * pool_bytes + 2 * scale_bytes);
  }
  for (int i = 0; i < c->slot_cap; ++i) c->slot_of_chunk[i] = -1;
  for (int i = 0; i < d->max_chunks; ++i) c->chunk_of_slot[i] = -1;
  c->bytes = (int64_t)(2 * pool_bytes + 2 * scale_bytes);
  *out = c;
  return MAGI_OK;
}

extern "C" int magi_kv_cache_destroy(magi_kv_cache* c) {
  if (!c) return MAGI_E_BADARG;
  if (c->k_pool) cudaFree(c->k_pool);
  if (c->v_pool) cudaFree(c->v_pool);
  if (c->k_scale) cudaFree(c->k_scale);
  if (c->v_scale) cudaFree(c->v_scale);
  free(c->slot_of_chunk);
  free(c->chunk_of_slot);
  free(c);
  return MAGI_OK;
}

extern "C" int64_t magi_kv_cache_bytes(const magi_kv_cache* c) { return c ? c->bytes : 0; }

static int cache_get_or_assign_slot(magi_kv_cache* c, int chunk_id) {
  if (chunk_id >= c->slot_cap) {
    int ncap = c->slot_cap;
    while (ncap <= chunk_id) ncap *= 2;
    int* n = static_cast<int*>(realloc(c->slot_of_chunk, sizeof(int) * ncap));
    if (!n) return -1;
    for (int i = c->slot_cap; i < ncap; ++i) n[i] = -1;
    c->slot_of_chunk = n;
    c->slot_cap = ncap;
  }
  if (c->slot_of_chunk[chunk_id] >= 0) return c->slot_of_chunk[chunk_id];
  for (int s = 0; s < c->d.max_chunks; ++s)
    if (c->chunk_of_slot[s] < 0) {
      c->chunk_of_slot[s] = chunk_id;
      c->slot_of_chunk[chunk_id] = s;
      return s;
    }
  return -1;
}

extern "C" int magi_kv_cache_append(magi_kv_cache* c, int layer, int chunk_id, const void* k, int64_t k_stride_t,
                                    int64_t k_stride_h, const void* v, int64_t v_stride_t, int64_t v_stride_h,
                                    int n_tokens, int token_offset, void* stream) {
  if (!c) return MAGI_E_BADARG;
  magi_ctx* ctx = c->ctx;
  if (!k || !v || n_tokens < 0 || token_offset < 0 || chunk_id < 0 || chunk_id >= (1 << 20) || layer < 0 ||
      layer >= c->d.n_layers)
    return set_err(ctx, MAGI_E_BADARG, "kv cache append: bad argument");
  if (token_offset + n_tokens > c->d.chunk_tokens)
    return set_err(ctx, MAGI_E_RANGE, "kv cache append: tokens [%d,%d) exceed the chunk size %d", token_offset,
                   token_offset + n_tokens, c->d.chunk_tokens);
  const int s = cache_get_or_assign_slot(c, chunk_id);
  if (s < 0) return set_err(ctx, MAGI_E_NOMEM, "kv cache append: no free page for chunk %d (max_chunks %d)", chunk_id, c->d.max_chunks);
  if (n_tokens == 0) return MAGI_OK;
  const int slot = layer * c->d.max_chunks + s;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (c->d.dtype == MAGI_DTYPE_FP8_E4M3) {
    if (token_offset % kTileN) return set_err(ctx, MAGI_E_ALIGN, "kv cache append (fp8): token_offset must be a multiple of 128");
    return launch_cache_quant_append(c, slot, k, k_stride_t, k_stride_h, v, v_stride_t, v_stride_h, n_tokens, token_offset, st);
  }
  const int64_t row_elems = (int64_t)c->d.n_kv_heads * kHeadDim;
  const int64_t row0 = (int64_t)slot * c->page_cap + token_offset;
  magi_prologue_params pp;
  memset(&pp, 0, sizeof(pp));
  pp.struct_size = sizeof(pp);
  pp.T = n_tokens;
  pp.H = c->d.n_kv_heads;
  pp.out_stride_t = row_elems;
  pp.out_stride_h = kHeadDim;
  pp.x = k;
  pp.x_stride_t = k_stride_t;
  pp.x_stride_h = k_stride_h;
  pp.out = static_cast<uint16_t*>(c->k_pool) + row0 * row_elems;
  int rc = magi_head_block_copy(ctx, &pp, stream);
  if (rc) return rc;
  pp.x = v;
  pp.x_stride_t = v_stride_t;
  pp.x_stride_h = v_stride_h;
  pp.out = static_cast<uint16_t*>(c->v_pool) + row0 * row_elems;
  return magi_head_block_copy(ctx, &pp, stream);
}

extern "C" int magi_kv_cache_evict(magi_kv_cache* c, int chunk_id) {
  if (!c) return MAGI_E_BADARG;
  if (chunk_id < 0 || chunk_id >= c->slot_cap || c->slot_of_chunk[chunk_id] < 0)
    return set_err(c->ctx, MAGI_E_RANGE, "kv cache evict: chunk %d is not cached", chunk_id);
  c->chunk_of_slot[c->slot_of_chunk[chunk_id]] = -1;
  c->slot_of_chunk[chunk_id] = -1;
  return MAGI_OK;
}

extern "C" int magi_kv_cache_read(magi_kv_cache* c, int layer, int chunk_id, void* k_out, void* v_out, int n_tokens,
                                  int token_offset, void* stream) {
  if (!c) return MAGI_E_BADARG;
  magi_ctx* ctx = c->ctx;
  const int slot = cache_slot(c, layer, chunk_id);
  if (slot < 0) return set_err(ctx, MAGI_E_RANGE, "kv cache read: chunk %d not cached in layer %d", chunk_id, layer);
  if (!k_out || !v_out || n_tokens < 0 || token_offset < 0 || token_offset + n_tokens > c->d.chunk_tokens)
    return set_err(ctx, MAGI_E_BADARG, "kv cache read: bad argument");
  if (n_tokens == 0) return MAGI_OK;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (c->d.dtype == MAGI_DTYPE_FP8_E4M3) {
    if (token_offset % kTileN) return set_err(ctx, MAGI_E_ALIGN, "kv cache read (fp8): token_offset must be a multiple of 128");
    return launch_cache_dequant_read(c, slot, k_out, v_out, n_tokens, token_offset, st);
  }
  const int64_t row_elems = (int64_t)c->d.n_kv_heads * kHeadDim;
  const int64_t row0 = (int64_t)slot * c->page_cap + token_offset;
  const size_t bytes = (size_t)n_tokens * row_elems * 2;
  // cudaMemcpyDefault: the destinations may be device memory or pinned host memory (the spill tier)
  MAGI_CUDA_OK(ctx, cudaMemcpyAsync(k_out, static_cast<uint16_t*>(c->k_pool) + row0 * row_elems, bytes, cudaMemcpyDefault, st));
  MAGI_CUDA_OK(ctx, cudaMemcpyAsync(v_out, static_cast<uint16_t*>(c->v_pool) + row0 * row_elems, bytes, cudaMemcpyDefault, st));
  return MAGI_OK;
}

// ------------------------------------------------------------------------------------------- peer buffers (CUDA IPC)
extern "C" int magi_peer_alloc(magi_ctx* ctx, uint64_t bytes, void** dev_ptr, unsigned char handle_out[64]) {
  if (!ctx || !dev_ptr || !handle_out || bytes == 0) return set_err(ctx, MAGI_E_BADARG, "peer alloc: bad argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(ctx->device);
  void* ptr = nullptr;
  cudaError_t e = cudaMalloc(&ptr, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    if (ptr) cudaFree(ptr);
    cudaGetLastError();
    return set_err(ctx, e == cudaErrorMemoryAllocation ? MAGI_E_NOMEM : MAGI_E_CUDA, "peer alloc of %llu bytes: %s",
                   (unsigned long long)bytes, cudaGetErrorString(e));
  }
  memcpy(handle_out, &h, 64);
  *dev_ptr = ptr;
  return MAGI_OK;
}

extern "C" int magi_peer_open(magi_ctx* ctx, const unsigned char handle[64], void** dev_ptr) {
  if (!ctx || !handle || !dev_ptr) return set_err(ctx, MAGI_E_BADARG, "peer open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(ctx->device);
  cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  cudaSetDevice(prev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return set_err(ctx, MAGI_E_CUDA, "peer open: %s", cudaGetErrorString(e));
  }
  return MAGI_OK;
}

extern "C" int magi_peer_close(magi_ctx* ctx, void* dev_ptr) {
  if (!ctx || !dev_ptr) return set_err(ctx, MAGI_E_BADARG, "peer close: bad argument");
  MAGI_CUDA_OK(ctx, cudaIpcCloseMemHandle(dev_ptr));
  return MAGI_OK;
}

extern "C" int magi_peer_free(magi_ctx* ctx, void* dev_ptr) {
  if (!ctx || !dev_ptr) return set_err(ctx, MAGI_E_BADARG, "peer free: bad argument");
  MAGI_CUDA_OK(ctx, cudaFree(dev_ptr));
  return MAGI_OK;
}

// ------------------------------------------------------------------------------------------- attention
static int attn_common(magi_ctx* ctx, const magi_attn_params* p, void* stream, int impl) {
  if (!ctx) return MAGI_E_BADARG;
  if (!p || p->struct_size != sizeof(magi_attn_params)) return set_err(ctx, MAGI_E_BADARG, "attn: bad struct_size");
  if (!p->q || (!p->out && p->n_o_peers == 0) || !p->q_ranges || !p->k_ranges) return set_err(ctx, MAGI_E_BADARG, "attn: null q/out/ranges");
  if (p->total_q <= 0 || p->total_k < 0 || p->n_q_heads <= 0 || p->n_kv_heads <= 0 || p->n_ranges <= 0 ||
      p->n_k_ranges <= 0 || p->max_seqlen_q <= 0)
    return set_err(ctx, MAGI_E_BADARG, "attn: sizes must be positive");
  if (p->n_q_heads % p->n_kv_heads) return set_err(ctx, MAGI_E_BADARG, "attn: n_q_heads must be a multiple of n_kv_heads");
  if (p->total_k > 0 && (!p->k || !p->v)) return set_err(ctx, MAGI_E_BADARG, "attn: null k/v with total_k > 0");
  if (!p->k_range_offsets && p->n_k_ranges != p->n_ranges)
    return set_err(ctx, MAGI_E_BADARG, "attn: n_k_ranges must equal n_ranges without k_range_offsets");
  if (p->n_ranges > kMaxRanges) return set_err(ctx, MAGI_E_NOMEM, "attn: more than %d ranges", kMaxRanges);
  if (p->n_q_heads > 65535) return set_err(ctx, MAGI_E_BADARG, "attn: too many heads");
  if ((reinterpret_cast<uintptr_t>(p->out) & 15) || (p->o_stride_t & 7) || (p->o_stride_h & 7))
    return set_err(ctx, MAGI_E_ALIGN, "attn: out must be 16-byte aligned with strides multiple of 8 elements");
  if (p->o_heads_per_block < 0 || (p->o_heads_per_block > 0 && (p->o_stride_block & 7)))
    return set_err(ctx, MAGI_E_ALIGN, "attn: o_heads_per_block must be >= 0 and o_stride_block a multiple of 8 elements");
  if (p->n_o_peers != 0) {
    if (p->n_o_peers < 0 || p->n_o_peers > 16 || !p->o_peer_ptrs || !p->o_peer_offsets || impl == 2 || p->lse)
      return set_err(ctx, MAGI_E_BADARG, "attn: fused output exchange needs 1..16 peers, pointer and offset tables, no lse, tensor-core kernel");
    if (p->o_peer_offsets[0] != 0 || p->o_peer_offsets[p->n_o_peers] != p->total_q)
      return set_err(ctx, MAGI_E_RANGE, "attn: o_peer_offsets must run from 0 to total_q");
    for (int i = 0; i < p->n_o_peers; ++i)
      if (!p->o_peer_ptrs[i] || (reinterpret_cast<uintptr_t>(p->o_peer_ptrs[i]) & 15) || p->o_peer_offsets[i + 1] < p->o_peer_offsets[i])
        return set_err(ctx, MAGI_E_BADARG, "attn: bad o_peer table entry %d", i);
  }
  if (p->dtype != MAGI_DTYPE_BF16 && p->dtype != MAGI_DTYPE_FP8_E4M3) return set_err(ctx, MAGI_E_BADARG, "attn: unknown dtype");
  const bool fp8 = p->dtype == MAGI_DTYPE_FP8_E4M3;
  if (fp8 && impl == 2) return set_err(ctx, MAGI_E_BADARG, "attn: the diagnostic kernel is bf16 only");
  if (fp8 && (!p->q_scale || (p->total_k > 0 && (!p->k_scale || !p->v_scale)) || p->scale_chunk_tokens <= 0))
    return set_err(ctx, MAGI_E_BADARG, "attn (fp8): scales and scale_chunk_tokens are required");

  PrefixTable pt;
  memset(&pt, 0, sizeof(pt));
  pt.chunk_tokens = 1;
  if (p->n_prefix_chunks > 0) {
    const magi_kv_cache* c = p->cache;
    if (!c || !p->prefix_chunk_ids) return set_err(ctx, MAGI_E_BADARG, "attn: prefix chunks need a cache and ids");
    if (p->n_prefix_chunks > kMaxPrefix) return set_err(ctx, MAGI_E_NOMEM, "attn: more than %d prefix chunks", kMaxPrefix);
    if (c->d.n_kv_heads != p->n_kv_heads) return set_err(ctx, MAGI_E_BADARG, "attn: cache has %d kv heads, call has %d", c->d.n_kv_heads, p->n_kv_heads);
    if ((c->d.dtype == MAGI_DTYPE_FP8_E4M3) != fp8) return set_err(ctx, MAGI_E_BADARG, "attn: cache dtype does not match call dtype");
    pt.n_prefix = p->n_prefix_chunks;
    pt.chunk_tokens = c->d.chunk_tokens;
    for (int i = 0; i < p->n_prefix_chunks; ++i) {
      const int slot = cache_slot(c, p->layer, p->prefix_chunk_ids[i]);
      if (slot < 0) return set_err(ctx, MAGI_E_RANGE, "attn: prefix chunk %d is not cached in layer %d", p->prefix_chunk_ids[i], p->layer);
      pt.row0[i] = slot * c->page_cap;
      pt.blk0[i] = slot * c->blocks_per_page;
    }
  }
  PlanArgs pa;
  pa.q_ranges = p->q_ranges;
  pa.k_ranges = p->k_ranges;
  pa.k_range_offsets = p->k_range_offsets;
  pa.n_ranges = p->n_ranges;
  pa.n_k_ranges = p->n_k_ranges;
  pa.total_q = p->total_q;
  pa.total_k = p->total_k;
  pa.max_seqlen_q = p->max_seqlen_q;
  pa.split_new_at = fp8 ? p->scale_chunk_tokens : 0;
  const int rows_per_item = kTileM * kTilesPerCta;
  const int64_t max_items = (int64_t)p->n_ranges * ((p->max_seqlen_q + rows_per_item - 1) / rows_per_item);
  if (max_items > kMaxItems) return set_err(ctx, MAGI_E_NOMEM, "attn: %lld work items exceed the plan capacity %d", (long long)max_items, kMaxItems);

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  launch_plan(ctx->workspace, pa, pt, st);
  int rc;
  if (impl == 2) rc = launch_attn_simt(ctx, p, (int)max_items, st);
  else if (fp8) rc = launch_attn_fp8(ctx, p, (int)max_items, st);
  else rc = launch_attn_bf16(ctx, p, (int)max_items, st);
  if (prev != ctx->device) cudaSetDevice(prev);
  return rc;
}

extern "C" int magi_chunk_attn_fwd(magi_ctx* ctx, const magi_attn_params* p, void* stream) {
  return attn_common(ctx, p, stream, 0);
}

extern "C" int magi_chunk_attn_fwd_simt(magi_ctx* ctx, const magi_attn_params* p, void* stream) {
  return attn_common(ctx, p, stream, 2);
}

// ------------------------------------------------------------------------------------------- no-allocation entry
// Plan scratch for callers that must not allocate: lives in the library image, one copy per GPU that loads the
// library, held until the process exits.  Same layout and capacity as a context's workspace (kPlanBytes = 640 KiB:
// at most 16384 work items, 8192 K/V segments, 1024 ranges).
static __device__ __align__(256) unsigned char g_noalloc_plan_scratch[magi::kPlanBytes];

namespace {
constexpr int kNoAllocMaxDevices = 64;
magi_ctx g_noalloc_ctx[kNoAllocMaxDevices];   // host-side bookkeeping only (device index, SM count, scratch address)
bool g_noalloc_ready[kNoAllocMaxDevices];

void copy_err(char* dst, int dst_len, const char* src) {
  if (!dst || dst_len <= 0) return;
  strncpy(dst, src, (size_t)dst_len - 1);
  dst[dst_len - 1] = 0;
}
}  // namespace

extern "C" int magi_chunk_attn_fwd_noalloc(const magi_attn_params* p, void* stream, int32_t* status_dev, char* err,
                                           int err_len) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    copy_err(err, err_len, "no-alloc attention: no usable current CUDA device");
    return MAGI_E_CUDA;
  }
  magi_ctx* ctx = &g_noalloc_ctx[dev];
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!g_noalloc_ready[dev]) {
    // One-time set-up for this device, done with it current.  g_noalloc_plan_scratch named from host code is only a
    // stand-in for the symbol, not a device address: the address a kernel may use has to be asked for.
    int major = 0, sms = 0;
    void* scratch = nullptr;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess && major != 10) {
      copy_err(err, err_len, "no-alloc attention: device is not sm_100");
      return MAGI_E_ARCH;
    }
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&scratch, g_noalloc_plan_scratch);
    if (e != cudaSuccess || !scratch) {
      copy_err(err, err_len, cudaGetErrorString(e));
      return MAGI_E_CUDA;
    }
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = dev;
    ctx->sm_count = sms;
    ctx->workspace = scratch;
    int rc = attn_init_device(ctx);  // raises the kernels' dynamic shared memory limit; allocates nothing
    if (rc) {
      copy_err(err, err_len, ctx->err);
      return rc;
    }
    g_noalloc_ready[dev] = true;
  }
  if (!p || p->struct_size != sizeof(magi_attn_params)) {
    copy_err(err, err_len, "no-alloc attention: bad struct_size");
    return MAGI_E_BADARG;
  }
  if (p->dtype != MAGI_DTYPE_BF16) {
    copy_err(err, err_len, "no-alloc attention: bf16 only");
    return MAGI_E_BADARG;
  }
  const int rows_per_item = kTileM * kTilesPerCta;
  const long long items = (long long)p->n_ranges * ((p->max_seqlen_q + rows_per_item - 1) / rows_per_item);
  if (p->n_ranges > kMaxRanges || items > kMaxItems || (long long)p->n_k_ranges + p->n_prefix_chunks > kMaxSegs / 2) {
    if (err && err_len > 0)
      snprintf(err, (size_t)err_len,
               "no-alloc attention: problem exceeds the fixed scratch (%d ranges <= %d, %lld work items <= %d, "
               "%d k intervals + %d prefix chunks <= %d)",
               p->n_ranges, kMaxRanges, items, kMaxItems, p->n_k_ranges, p->n_prefix_chunks, kMaxSegs / 2);
    return MAGI_E_NOMEM;
  }
  // The scratch keeps what the previous call left: the header (item count, status word) must start from zero.
  cudaError_t e = cudaMemsetAsync(ctx->workspace, 0, sizeof(PlanHeader), st);
  if (e != cudaSuccess) {
    copy_err(err, err_len, cudaGetErrorString(e));
    return MAGI_E_CUDA;
  }
  int rc = attn_common(ctx, p, stream, 0);
  if (rc) {
    copy_err(err, err_len, ctx->err);
    return rc;
  }
  if (status_dev) {
    e = cudaMemcpyAsync(status_dev, reinterpret_cast<char*>(ctx->workspace) + offsetof(PlanHeader, status), sizeof(int32_t),
                        cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) {
      copy_err(err, err_len, cudaGetErrorString(e));
      return MAGI_E_CUDA;
    }
  }
  return MAGI_OK;
}
