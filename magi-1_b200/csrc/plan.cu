// Device-side planner: turns (q_ranges, k_ranges, prefix page table) - all resident on the device, as the
// reference passes them (inference/model/dit/dit_module.py:1036-1037) - into the work list the attention
// kernels walk, without a host round trip.  Ranges are ordered longest-K first so the heavy CTAs start first.
#include "common.cuh"

namespace magi {

__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

__global__ void plan_kernel(void* workspace, PlanArgs a, PrefixTable pt) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  PlanView pv = plan_view(workspace);
  __shared__ int s_seg_begin[kMaxRanges];
  __shared__ int s_seg_end[kMaxRanges];
  __shared__ int s_tiles[kMaxRanges];
  __shared__ short s_order[kMaxRanges];

  int status = 0;
  int n_segs = 0;
  const int C = pt.chunk_tokens;
  const int prefix_tokens = pt.n_prefix * C;
  const int kv_total = prefix_tokens + a.total_k;
  const int S = a.split_new_at;
  const int nbS = S > 0 ? ceil_div(S, kTileN) : 0;

  if (a.n_ranges > kMaxRanges) status = MAGI_E_NOMEM;

  for (int i = 0; i < a.n_ranges && status == 0; ++i) {
    const int qs = a.q_ranges[2 * i], qe = a.q_ranges[2 * i + 1];
    if (qs < 0 || qe < qs || qe > a.total_q) { status = MAGI_E_RANGE; break; }
    if (qe - qs > a.max_seqlen_q) { status = MAGI_E_RANGE; break; }
    if (S > 0 && (qs % S) % kTileM != 0) { status = MAGI_E_RANGE; break; }
    int kb = i, ke_ = i + 1;
    if (a.k_range_offsets) { kb = a.k_range_offsets[i]; ke_ = a.k_range_offsets[i + 1]; }
    if (kb < 0 || ke_ < kb || ke_ > a.n_k_ranges) { status = MAGI_E_RANGE; break; }
    s_seg_begin[i] = n_segs;
    int tiles = 0;
    for (int r = kb; r < ke_ && status == 0; ++r) {
      int ks = a.k_ranges[2 * r], ke = a.k_ranges[2 * r + 1];
      if (ks < 0 || ke < ks || ke > kv_total) { status = MAGI_E_RANGE; break; }
      int t = ks;
      while (t < ke) {
        Segment sg;
        int end;
        if (t < prefix_tokens) {
          const int p = t / C;
          const int in_page = t - p * C;
          end = min(ke, (p + 1) * C);
          sg.src = 1;
          sg.row0 = pt.row0[p] + in_page;
          sg.blk0 = pt.blk0[p] + in_page / kTileN;
          if (S > 0 && in_page % kTileN != 0) { status = MAGI_E_RANGE; break; }
        } else {
          const int tn = t - prefix_tokens;
          end = ke;
          sg.src = 0;
          sg.row0 = tn;
          sg.blk0 = 0;
          if (S > 0) {
            const int c = tn / S, in_c = tn - c * S;
            end = min(ke, prefix_tokens + (c + 1) * S);
            sg.blk0 = c * nbS + in_c / kTileN;
            if (in_c % kTileN != 0) { status = MAGI_E_RANGE; break; }
          }
        }
        sg.len = end - t;
        if (n_segs >= kMaxSegs) { status = MAGI_E_NOMEM; break; }
        pv.segs[n_segs++] = sg;
        tiles += ceil_div(sg.len, kTileN);
        t = end;
      }
    }
    s_seg_end[i] = n_segs;
    s_tiles[i] = tiles;
  }

  int n_items = 0;
  if (status == 0) {
    // insertion sort of range indices by K tiles, descending (stable)
    for (int i = 0; i < a.n_ranges; ++i) {
      int j = i;
      while (j > 0 && s_tiles[s_order[j - 1]] < s_tiles[i]) { s_order[j] = s_order[j - 1]; --j; }
      s_order[j] = (short)i;
    }
    const int rows_per_item = kTileM * kTilesPerCta;
    for (int o = 0; o < a.n_ranges && status == 0; ++o) {
      const int i = s_order[o];
      const int qs = a.q_ranges[2 * i], qe = a.q_ranges[2 * i + 1];
      for (int q0 = qs; q0 < qe; q0 += rows_per_item) {
        if (n_items >= kMaxItems) { status = MAGI_E_NOMEM; break; }
        WorkItem it;
        it.q_row0 = q0;
        it.q_rows = min(rows_per_item, qe - q0);
        it.seg_begin = s_seg_begin[i];
        it.seg_end = s_seg_end[i];
        it.n_tiles = s_tiles[i];
        it.q_blk0 = S > 0 ? (q0 / S) * nbS + (q0 % S) / kTileM : 0;
        it.pad0 = it.pad1 = 0;
        pv.items[n_items++] = it;
      }
    }
  }
  if (status != 0) {
    n_items = 0;
    pv.hdr->status = status;
  }
  pv.hdr->n_items = n_items;
  pv.hdr->n_segs = n_segs;
}

void launch_plan(void* workspace, const PlanArgs& a, const PrefixTable& pt, cudaStream_t stream) {
  plan_kernel<<<1, 32, 0, stream>>>(workspace, a, pt);
}

}  // namespace magi
