// Output epilogue shared by the bf16 and the e4m3 attention kernels: O (fp32, TMEM) -> normalised bf16 rows in global
// memory, local or on the context-parallel rank that owns the token (inference/infra/parallelism/context_parallel.py:404-423
// and :596 fused into the store address, see out_row()).
#pragma once
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace magi {

// One softmax warp owns 32 rows (TMEM lanes 32*quarter ..) of Q tile x.  Its 32 rows x 256 B are staged through
// `stage` (8 KB of shared memory that nothing else touches any more), so that the global stores are whole 256-byte
// rows per half-warp instead of 16-byte pieces of 32 different rows; this matters when the destination is a peer GPU
// (NVLink packets) and costs nothing locally.  16-byte chunks are XOR-swizzled by the row index: conflict-free in both
// directions.  Rows beyond it.q_rows are not stored.
template <class P>
__device__ __forceinline__ void store_o_rows_staged(const P& p, const WorkItem& it, int head, int x, int quarter, int lane,
                                                    uint32_t tO, float inv, uint8_t* stage) {
  using namespace ptx;
#pragma unroll 1
  for (int c4 = 0; c4 < 4; ++c4) {
    uint32_t o[32];
    tmem_ld32(tO + c4 * 32, o);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 v;
      v.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
      v.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
      v.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
      v.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
      *reinterpret_cast<uint4*>(stage + lane * 256 + (((c4 * 4 + c) ^ (lane & 15)) << 4)) = v;
    }
  }
  __syncwarp();
  const int l16 = lane & 15, hsel = lane >> 4;
#pragma unroll 4
  for (int i = 0; i < 16; ++i) {
    const int rr = 2 * i + hsel;                        // row inside this warp's 32
    const int r_item = x * kTileM + quarter * 32 + rr;  // row inside the work item
    if (r_item < it.q_rows) {
      const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * 256 + (l16 << 4));
      __nv_bfloat16* dst_row = out_row(p, it.q_row0 + r_item, head);
      *reinterpret_cast<uint4*>(dst_row + ((l16 ^ (rr & 15)) << 3)) = v;
    }
  }
}

}  // namespace magi
