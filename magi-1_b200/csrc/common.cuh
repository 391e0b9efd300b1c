// Internal declarations shared by the translation units of libmagi_attn.so.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/magi_attn.h"

namespace magi {

constexpr int kHeadDim = 128;
constexpr int kTileM = 128;      // rows of one Q tile (one UMMA M)
constexpr int kTilesPerCta = 2;  // Q tiles per CTA: the two softmax warpgroups ping-pong on the tensor pipe
constexpr int kTileN = 128;      // K/V tokens per step
constexpr int kMaxPrefix = 64;

// ---- plan workspace (device) ---------------------------------------------------------------
// A K/V segment: `len` consecutive rows starting at `row0` of source `src` (0 = current K/V, 1 = cache pool).
// `blk0` = index of the first 128-token scale block (FP8), unused for bf16.
struct Segment {
  int32_t src;
  int32_t row0;
  int32_t len;
  int32_t blk0;
};
// One CTA's work: up to 256 q rows of one range, all K/V segments of that range.
struct WorkItem {
  int32_t q_row0;     // first q row
  int32_t q_rows;     // valid rows (1..256)
  int32_t seg_begin;  // [seg_begin, seg_end) into segs
  int32_t seg_end;
  int32_t n_tiles;    // total K/V tiles over the segments
  int32_t q_blk0;     // first q scale block (FP8)
  int32_t pad0, pad1;
};
struct PlanHeader {
  int32_t n_items;
  int32_t n_segs;
  int32_t status;  // 0 or a MAGI_E_* code written by a kernel
  int32_t pad;
};
constexpr int kMaxItems = 16384;
constexpr int kMaxSegs = 8192;
constexpr int kMaxRanges = 1024;
constexpr size_t kPlanBytes = sizeof(PlanHeader) + sizeof(WorkItem) * kMaxItems + sizeof(Segment) * kMaxSegs;

struct PlanView {
  PlanHeader* hdr;
  WorkItem* items;
  Segment* segs;
};
__host__ __device__ inline PlanView plan_view(void* base) {
  PlanView v;
  v.hdr = reinterpret_cast<PlanHeader*>(base);
  v.items = reinterpret_cast<WorkItem*>(reinterpret_cast<char*>(base) + sizeof(PlanHeader));
  v.segs = reinterpret_cast<Segment*>(reinterpret_cast<char*>(base) + sizeof(PlanHeader) + sizeof(WorkItem) * kMaxItems);
  return v;
}

// By-value argument of the plan kernel: where each prefix chunk lives in the cache pool.
struct PrefixTable {
  int32_t n_prefix;
  int32_t chunk_tokens;          // virtual tokens per prefix chunk
  int32_t row0[kMaxPrefix];      // pool row of token 0 of the page
  int32_t blk0[kMaxPrefix];      // pool scale-block index of block 0 of the page
};

struct PlanArgs {
  const int32_t* q_ranges;
  const int32_t* k_ranges;
  const int32_t* k_range_offsets;
  int32_t n_ranges, n_k_ranges;
  int32_t total_q, total_k;
  int32_t max_seqlen_q;
  int32_t split_new_at;  // >0: split current-K/V segments at multiples of this (FP8 scale blocks), also q block base
};

void launch_plan(void* workspace, const PlanArgs& a, const PrefixTable& pt, cudaStream_t stream);

// Element offset of head h's 128 output columns inside a token row: h * o_stride_h, or with the head-block layout
// (o_hpb heads per block, blocks o_stride_block apart) (h / o_hpb) * o_stride_block + (h % o_hpb) * o_stride_h.
template <class P>
__device__ __forceinline__ int64_t head_col(const P& p, int h) {
  return p.o_hpb > 0 ? (int64_t)(h / p.o_hpb) * p.o_stride_block + (int64_t)(h % p.o_hpb) * p.o_stride_h
                     : (int64_t)h * p.o_stride_h;
}

// Where the 128 output columns of q row `t`, (local) head `h` go.  Plain output: out + t * o_stride_t + head_col(h).
// Fused output exchange (n_peers > 0): the row belongs to the rank d with peer_off[d] <= t < peer_off[d+1] and lands in
// that rank's result buffer at this rank's global head position.  P carries out, o_stride_*, o_hpb, n_peers, head_offset,
// peer_off[17], peer_out[16].
template <class P>
__device__ __forceinline__ __nv_bfloat16* out_row(const P& p, int t, int h) {
  if (p.n_peers > 0) {
    int d = 0;
    while (d + 1 < p.n_peers && t >= p.peer_off[d + 1]) ++d;
    return p.peer_out[d] + (int64_t)(t - p.peer_off[d]) * p.o_stride_t + head_col(p, p.head_offset + h);
  }
  return p.out + (int64_t)t * p.o_stride_t + head_col(p, h);
}

// A q-range without keys: the output rows are defined as zeros (lse = -inf), wherever they live.
template <class P>
__device__ __forceinline__ void zero_fill_item(const P& p, const WorkItem& it, int head) {
  for (int idx = threadIdx.x; idx < it.q_rows * (kHeadDim / 8); idx += blockDim.x) {
    const int r = idx / (kHeadDim / 8), c = idx % (kHeadDim / 8);
    *reinterpret_cast<uint4*>(out_row(p, it.q_row0 + r, head) + c * 8) = make_uint4(0, 0, 0, 0);
  }
  if (p.lse)
    for (int r = threadIdx.x; r < it.q_rows; r += blockDim.x)
      p.lse[(int64_t)(it.q_row0 + r) * p.n_q_heads + head] = -INFINITY;
}

// Host: copies the peer table of the call into the by-value kernel parameters.
template <class P>
inline void fill_peer_table(P& kp, const magi_attn_params* p) {
  kp.n_peers = p->n_o_peers;
  kp.head_offset = p->o_head_offset;
  for (int i = 0; i < 17; ++i) kp.peer_off[i] = (p->n_o_peers > 0 && i <= p->n_o_peers) ? p->o_peer_offsets[i] : 0;
  for (int i = 0; i < 16; ++i)
    kp.peer_out[i] = i < p->n_o_peers ? reinterpret_cast<__nv_bfloat16*>(p->o_peer_ptrs[i]) : nullptr;
}

}  // namespace magi

// ---- host-side objects -------------------------------------------------------------------------
struct magi_ctx {
  int device;
  int sm_count;
  void* workspace;  // kPlanBytes
  char err[512];
};

struct magi_kv_cache {
  magi_ctx* ctx;
  magi_kv_cache_desc d;
  int page_cap;        // chunk_tokens rounded up to a multiple of 128
  int blocks_per_page; // page_cap / 128
  int n_slots;         // n_layers * max_chunks
  void* k_pool;        // [n_slots * page_cap, Hkv, 128] bf16 or e4m3
  void* v_pool;
  float* k_scale;      // fp8: [n_slots * blocks_per_page, Hkv]
  float* v_scale;
  int* slot_of_chunk;  // host: chunk id -> slot within a layer (-1 = none); grows on demand
  int slot_cap;
  int* chunk_of_slot;  // host: [max_chunks]
  int64_t bytes;
};

namespace magi {
int set_err(magi_ctx* ctx, int code, const char* fmt, ...);
int cache_slot(const magi_kv_cache* c, int layer, int chunk_id);  // global slot index or -1
}  // namespace magi

#define MAGI_CUDA_OK(ctx, call)                                                                      \
  do {                                                                                               \
    cudaError_t e__ = (call);                                                                        \
    if (e__ != cudaSuccess)                                                                          \
      return magi::set_err((ctx), MAGI_E_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));     \
  } while (0)
