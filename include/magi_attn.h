/*
 * libmagi_attn.so - C ABI of the B200 (sm_100a) chunk-wise block-causal GQA attention core.
 *
 * Every entry point replaces a piece of MAGI-1's DiT self-attention (paths below are relative to the
 * MAGI-1 project root).  Rules shared by all functions:
 *   - plain pointers and sizes only; device pointers are raw CUDA device addresses, `stream` is a cudaStream_t
 *     passed as void* (NULL = legacy default stream); all work is stream-ordered, nothing synchronises unless
 *     the function says so;
 *   - return value: 0 (MAGI_OK) or a negative MAGI_E_* code; never throws, never aborts, never computes on the
 *     CPU.  magi_last_error() gives the text of the last failure recorded on a context;
 *   - head_dim is fixed at 128 (the only value MAGI-1 ships: kv_channels = 128);
 *   - one context per (device, stream in flight): contexts own a small device workspace that calls share.
 */
#ifndef MAGI_ATTN_H_
#define MAGI_ATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAGI_HEAD_DIM 128
#if defined(__GNUC__)
#define MAGI_API __attribute__((visibility("default")))
#else
#define MAGI_API
#endif

enum {
  MAGI_OK = 0,
  MAGI_E_BADARG = -1,   /* null pointer, non-positive size, unsupported combination            */
  MAGI_E_ALIGN = -2,    /* pointer not 16-byte aligned or stride not a multiple of 8 elements  */
  MAGI_E_ARCH = -3,     /* device is not compute capability 10.x                               */
  MAGI_E_RANGE = -4,    /* range / page bookkeeping inconsistent (caught on host or on device) */
  MAGI_E_NOMEM = -5,    /* cudaMalloc failed or a fixed capacity was exceeded                  */
  MAGI_E_NCCL = -6,     /* NCCL call failed                                                    */
  MAGI_E_TIMEOUT = -7,  /* a bounded device-side wait gave up (reported by magi_ctx_status)    */
  MAGI_E_CUDA = -8      /* a CUDA runtime / driver call failed                                 */
};

enum { MAGI_DTYPE_BF16 = 0, MAGI_DTYPE_FP8_E4M3 = 1, MAGI_DTYPE_F32 = 2 };
enum { MAGI_NORM_LAYERNORM_1P = 0, MAGI_NORM_RMSNORM_1P = 1, MAGI_NORM_NONE = 2 /* magi_linear_qk_norm_rope_fwd only */ };

typedef struct magi_ctx magi_ctx;
typedef struct magi_kv_cache magi_kv_cache;
typedef struct magi_ulysses magi_ulysses;

/* Library version (major*10000 + minor*100 + patch).  No counterpart in the reference. */
MAGI_API int magi_version(void);
/* Text for a MAGI_E_* code.  Replaces the Python asserts / exceptions the reference raises on this path. */
MAGI_API const char* magi_strerror(int code);

/* One context per GPU worker; mirrors "one Python process per GPU" of the reference launcher
 * (example/24B/run.sh:27-38).  Allocates the plan workspace (640 KiB) on `device`.  Fails with MAGI_E_ARCH on
 * anything but sm_100. */
MAGI_API int magi_ctx_create(int device, magi_ctx** out);
MAGI_API int magi_ctx_destroy(magi_ctx* ctx);
MAGI_API const char* magi_last_error(const magi_ctx* ctx);
/* Synchronises `stream`, then reads the device status word: 0, MAGI_E_RANGE (plan kernel met an
 * inconsistent range) or MAGI_E_TIMEOUT (a bounded mbarrier wait in a kernel gave up).  Clears the word. */
MAGI_API int magi_ctx_status(magi_ctx* ctx, void* stream, int* device_status);
/* Self-test of the device-side failure detection (no reference counterpart).  Every wait inside the attention kernels
 * is bounded: after a cycle limit the waiting role gives up, the other roles of the CTA follow, the kernel frees what it
 * holds, returns, and magi_ctx_status reads MAGI_E_TIMEOUT.  This entry runs that same wait on a barrier that nothing
 * completes, with `limit_cycles` (1e3 .. 2e8 SM cycles) as the limit: the launch returns normally and the status word
 * reads MAGI_E_TIMEOUT afterwards.  Nothing faults, traps or hangs; the context stays usable. */
MAGI_API int magi_selftest_bounded_wait(magi_ctx* ctx, long long limit_cycles, void* stream);

/* ------------------------------------------------------------------------------------------------------
 * Prologue: per-head norm + 3D RoPE, fused.  Replaces FullyParallelAttention.get_q / get_k
 * (inference/model/dit/dit_module.py:953-963, :970-980) after the linear projection:
 * fp32 upcast, FusedLayerNorm with weight gamma+1 (:355-357), non-interleaved rotary on the first
 * 2*rot_pairs channels (:961), cast to bf16, and the "(sq b) hn hd" re-layout - one pass over HBM.
 * The destination is generic enough to be (a) the packed tensor, (b) the Ulysses send buffer
 * "seq (cp hn) hd -> (cp seq) hn hd" (inference/infra/parallelism/context_parallel.py:396) or (c) a KV-cache
 * page: head h goes to block h / heads_per_block, head slot h % heads_per_block.
 */
typedef struct {
  uint32_t struct_size;      /* sizeof(magi_prologue_params) */
  int32_t norm_mode;         /* MAGI_NORM_*                                                        */
  const void* x;             /* bf16 [T, H, 128] view: element (t,h,d) at x + t*x_stride_t + h*x_stride_h + d */
  int64_t x_stride_t, x_stride_h;
  int32_t T, H;
  const float* gamma;        /* fp32 [128]; applied as gamma + 1                                   */
  const float* beta;         /* fp32 [128] or NULL; ignored for RMSNORM                            */
  float eps;
  int32_t rot_pairs;         /* <= 64, multiple of 4; the reference uses 48.  0 = no rotary        */
  const float* cos;          /* fp32 [T, rot_pairs]                                                */
  const float* sin;
  void* out;                 /* bf16; element (t,h,d) at out + (h / heads_per_block)*out_stride_block
                                + t*out_stride_t + (h % heads_per_block)*out_stride_h + d         */
  int64_t out_stride_t, out_stride_h, out_stride_block;
  int32_t heads_per_block;   /* 0 or >= H: no blocking */
  /* Optional: one destination base per block instead of out + block*out_stride_block (HOST array of
     H / heads_per_block device pointers, at most 16).  With peer-mapped pointers (magi_peer_open) the prologue
     writes each context-parallel rank's share of the heads straight into that rank's receive buffer over NVLink:
     the "scatter heads" all-to-all of context_parallel.py:381-401 fused into its producer. */
  void* const* out_block_ptrs;
  int32_t x_heads_per_block; /* source blocking (the inverse re-layout "(cp sq) hn hd -> sq (cp hn) hd" after the
                                output all-to-all, context_parallel.py:596): element (t,h,d) is read at
                                x + (h / x_heads_per_block)*x_stride_block + t*x_stride_t + (h % x_heads_per_block)*x_stride_h + d.
                                0 or >= H: no blocking */
  int64_t x_stride_block;
} magi_prologue_params;
MAGI_API int magi_qk_norm_rope_fwd(magi_ctx* ctx, const magi_prologue_params* p, void* stream);

/* Strided copy with the same destination addressing as the prologue (used for V, which has no norm/rope:
 * FullyParallelAttention.get_v, inference/model/dit/dit_module.py:987-989, and the torch.cat of K and V at
 * :996).  x, out: bf16. */
MAGI_API int magi_head_block_copy(magi_ctx* ctx, const magi_prologue_params* p, void* stream);

/* ------------------------------------------------------------------------------------------------------
 * Projection + prologue in one kernel: out = prologue( bf16( x @ w^T ) ), the prologue running in the GEMM's
 * epilogue.  Replaces FullyParallelAttention.get_q / get_k / get_v including the linear they start with
 * (inference/model/dit/dit_module.py:953-963 with linear_qkv.forward_q :415-416; :970-980 with forward_k
 * :421-422; :987-989 with forward_v :424-425), for the bf16 torch.nn.Linear case of CustomLayerNormLinear
 * (:406-408), and - with dtype MAGI_DTYPE_FP8_E4M3 - for its PerTensorQuantizedFp8Linear members (:409-410, forward
 * :445-456): x is then the e4m3 output of magi_div_clamp_to_e4m3, w the e4m3 weight [out_features, in_features], and
 * x_scale / w_scale what the reference hands to bmm_fp8 (input_scale, weight_scale; applied as scalars, as bmm_fp8 does).
 * norm_mode MAGI_NORM_NONE = plain linear (get_v): gamma, beta, cos, sin ignored.
 * The linear's result is rounded to bf16 before the norm, as the reference's Linear output is, and never
 * reaches HBM.  in_features must be a multiple of 128; rot_pairs one of 0, 32, 48, 64.  Destination
 * addressing (blocks of heads, optional per-block base pointers, peer-mapped or not) as magi_prologue_params.
 */
typedef struct {
  uint32_t struct_size;      /* sizeof(magi_linear_prologue_params) */
  int32_t norm_mode;         /* MAGI_NORM_*                                                        */
  const void* x;             /* bf16 [T, in_features], row stride x_stride elements (multiple of 8), 16-byte aligned */
  int64_t x_stride;
  const void* w;             /* bf16 [H * 128, in_features] = torch.nn.Linear.weight, row stride w_stride */
  int64_t w_stride;
  int32_t T, H, in_features;
  float eps;
  const float* gamma;        /* fp32 [128]; applied as gamma + 1                                   */
  const float* beta;         /* fp32 [128] or NULL; ignored for RMSNORM                            */
  int32_t rot_pairs;
  int32_t heads_per_block;   /* 0 or >= H: no blocking */
  const float* cos;          /* fp32 [T, rot_pairs], 16-byte aligned                               */
  const float* sin;
  void* out;                 /* bf16; element (t,h,d) at out + (h / heads_per_block)*out_stride_block
                                + t*out_stride_t + (h % heads_per_block)*out_stride_h + d         */
  int64_t out_stride_t, out_stride_h, out_stride_block;
  void* const* out_block_ptrs; /* optional HOST array of H / heads_per_block device pointers (at most 16) */
  int32_t dtype;             /* operands: MAGI_DTYPE_BF16, or MAGI_DTYPE_FP8_E4M3 (x and w both e4m3, strides in elements) */
  int32_t plain_odd_heads;   /* 1: heads 1, 3, 5, ... are plain (no norm, no rotary): the weight of linear_kv_xattn, whose rows are
                                (k of head 0, v of head 0, k of head 1, ...) so that out [T, 2*Hkv, 128] IS the K|V buffer [T, Hkv, 256]
                                of get_xqkv (inference/model/dit/dit_module.py:1010-1020) */
  const float* x_scale;      /* e4m3 only: DEVICE pointers to one fp32 each; the fp32 accumulator is multiplied by          */
  const float* w_scale;      /* x_scale[0] * w_scale[0] before the bf16 rounding (NULL = 1)                                 */
} magi_linear_prologue_params;
MAGI_API int magi_linear_qk_norm_rope_fwd(magi_ctx* ctx, const magi_linear_prologue_params* p, void* stream);
/* Up to four projections of the same x in ONE launch - q, qx, k, v, the members of the reference's CustomLayerNormLinear
 * (inference/model/dit/dit_module.py:404): FullyParallelAttention.get_qkv / get_kv (:991-1003) and the query half of
 * get_xqkv (:1005-1008: forward_qx, then q_layernorm_xattn, no rotary).  `projections` is an array of n (1..4) structs,
 * each with its own w, H, norm_mode, gamma, beta, rot_pairs (0 = normed but not rotated), w_scale and destination; x,
 * x_stride, T, in_features, dtype, x_scale and eps must be the same in all of them, and the projections that are rotated
 * share rot_pairs, cos and sin.  Every row block of x is then fetched from HBM once for all of them. */
MAGI_API int magi_linear_qkv_norm_rope_fwd(magi_ctx* ctx, const magi_linear_prologue_params* projections, int n, void* stream);

/* ------------------------------------------------------------------------------------------------------
 * Chunk-paged KV cache.  Replaces Attention._allocate_key_and_value_memory
 * (inference/model/dit/dit_module.py:800-819) and _full_adjust_key_and_value (:891-931): instead of one flat
 * [max_seq, Hkv, 2*128] buffer per layer that is sliced, written and torch.cat'ed with the current K|V on
 * every call, clean chunks live in fixed pages (one page = one chunk of one layer, K and V separate) that
 * the attention kernel reads in place through a page list.  The cache is head-sharded under context
 * parallelism exactly like the reference's (num_query_groups_per_partition, :794-798): create it with the
 * local number of KV heads.
 */
typedef struct {
  uint32_t struct_size;
  int32_t dtype;            /* MAGI_DTYPE_BF16 or MAGI_DTYPE_FP8_E4M3 (per-(head,128-token block) fp32 scales) */
  int32_t n_layers;
  int32_t max_chunks;       /* pages per layer                                                   */
  int32_t chunk_tokens;     /* tokens of a full chunk (e.g. 9360, 21600)                         */
  int32_t n_kv_heads;       /* local KV heads                                                    */
} magi_kv_cache_desc;
MAGI_API int magi_kv_cache_create(magi_ctx* ctx, const magi_kv_cache_desc* d, magi_kv_cache** out);
MAGI_API int magi_kv_cache_destroy(magi_kv_cache* c);
/* Writes tokens [token_offset, token_offset + n_tokens) of chunk `chunk_id` in `layer` from bf16 K and V
 * views [n_tokens, Hkv, 128] (strides in elements).  The page is allocated on first use of a chunk id.
 * FP8 caches quantise here; token_offset must then be a multiple of 128.  Counterpart of the cache write
 * at inference/model/dit/dit_module.py:918-929. */
MAGI_API int magi_kv_cache_append(magi_kv_cache* c, int layer, int chunk_id, const void* k, int64_t k_stride_t,
                         int64_t k_stride_h, const void* v, int64_t v_stride_t, int64_t v_stride_h, int n_tokens,
                         int token_offset, void* stream);
/* Frees the pages of a chunk in every layer (the reference never frees; its windows
 * - inference/pipeline/video_generate.py:467-508 - make old chunks dead). */
MAGI_API int magi_kv_cache_evict(magi_kv_cache* c, int chunk_id);
/* Copies a page back out as bf16 [n_tokens, Hkv, 128] (dequantising an FP8 page); for tests, for callers that want the
 * reference's materialised prefix (inference/model/dit/dit_module.py:914-915), and - bf16 pages, k_out / v_out in pinned
 * host memory - for spilling a page to the host tier (the reference's kv_offload, :803-811).  magi_kv_cache_append
 * accepts pinned host sources the same way (the copy kernel reads them over PCIe), which brings a page back. */
MAGI_API int magi_kv_cache_read(magi_kv_cache* c, int layer, int chunk_id, void* k_out, void* v_out, int n_tokens,
                       int token_offset, void* stream);
/* Bytes of device memory the cache holds. */
MAGI_API int64_t magi_kv_cache_bytes(const magi_kv_cache* c);

/* ------------------------------------------------------------------------------------------------------
 * Core attention.  Replaces the module-level `flex_attention` call in FullyParallelAttention.core_attention
 * (inference/model/dit/dit_module.py:1032-1043; same packed varlen surface: q_ranges / k_ranges int32 [n,2] on
 * the device, max_seqlen_q / max_seqlen_k, softmax_scale) and the per-range flash_attn_func loop (:1049-1065):
 * for every q-range i, out[q_i] = softmax(Q[q_i] K[k_i]^T * scale) V[k_i], non-causal inside the rectangle,
 * GQA head h -> h / (Hq/Hkv).  Rows of q covered by no range are not written.
 *
 * Key/value address space ("virtual" tokens) that k_ranges index, as in the reference's
 * torch.cat([cache[:slice_point*C], current]) (:931):
 *     [ prefix chunk 0 | prefix chunk 1 | ... | prefix chunk P-1 | current k/v tokens ]
 * each prefix chunk being exactly cache->chunk_tokens tokens read in place from its page.
 * Extension over the reference: with k_range_offsets a q-range may own several k intervals (their union is
 * attended), which expresses "own cached prefix + own chunk" for concurrently denoising chunks.
 */
typedef struct {
  uint32_t struct_size;
  int32_t dtype;                 /* MAGI_DTYPE_BF16; MAGI_DTYPE_FP8_E4M3 with the *_scale fields        */
  const void* q;                 /* [total_q, Hq, 128]; strides in elements                              */
  int64_t q_stride_t, q_stride_h;
  const void* k;                 /* current K [total_k, Hkv, 128] (may be NULL if total_k == 0)          */
  int64_t k_stride_t, k_stride_h;
  const void* v;                 /* current V [total_k, Hkv, 128]                                        */
  int64_t v_stride_t, v_stride_h;
  void* out;                     /* bf16 [total_q, Hq, 128]                                              */
  int64_t o_stride_t, o_stride_h;
  float* lse;                    /* fp32 [total_q, Hq] natural-log-sum-exp, or NULL                      */
  int32_t total_q, total_k;
  int32_t n_q_heads, n_kv_heads;
  const int32_t* q_ranges;       /* device int32 [n_ranges, 2]                                           */
  const int32_t* k_ranges;       /* device int32 [n_k_ranges, 2], virtual token coordinates              */
  const int32_t* k_range_offsets;/* device int32 [n_ranges+1] or NULL (then n_k_ranges == n_ranges, 1:1) */
  int32_t n_ranges, n_k_ranges;
  int32_t max_seqlen_q;          /* upper bound of q-range lengths (sizes the grid; no host sync needed)  */
  int32_t max_seqlen_k;          /* accepted for surface parity; unused                                  */
  float softmax_scale;           /* <= 0: 1/sqrt(128), the reference's softmax_scale=None                */
  const magi_kv_cache* cache;    /* NULL: no prefix                                                      */
  int32_t layer;
  int32_t n_prefix_chunks;       /* P <= 64                                                              */
  const int32_t* prefix_chunk_ids; /* HOST int32 [P]                                                     */
  /* FP8 only: fp32 scales [n_blocks, heads]; 128-token blocks counted from each multiple of scale_chunk_tokens, so
   * q_scale has ceil(total_q / scale_chunk_tokens) * ceil(scale_chunk_tokens / 128) rows of n_q_heads entries, k_scale
   * and v_scale the same with total_k and n_kv_heads (what magi_quantize_e4m3_block128 writes); prefix pages carry
   * their own scales inside the cache.  A block without tokens is never read. */
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  int32_t scale_chunk_tokens;
  int32_t reserved;
  /* FP8 only, optional: second e4m3 term of Q (rounding residual of the first, same scales, same strides as q).
   * When given, the kernel runs its two-term mode: S = (Q8 + Q8_lo) K8^T and O += (P8 + P8_lo) V8, which removes the
   * quantisation noise of Q and of P (K and V stay single e4m3) at the price of twice the UMMA work. */
  const void* q_lo;
  /* Optional fused output exchange (the "gather heads" all-to-all of context_parallel.py:404-423 and the final
   * "(cp sq) hn hd -> sq (cp hn) hd" re-layout at :596, fused into the attention epilogue): q row t belongs to the
   * context-parallel rank d with o_peer_offsets[d] <= t < o_peer_offsets[d+1] and is stored at
   * o_peer_ptrs[d] + (t - o_peer_offsets[d]) * o_stride_t + (o_head_offset + head) * o_stride_h, with plain stores
   * (peer-mapped pointers from magi_peer_open for d != own rank).  `out` is then ignored.  HOST arrays, n_o_peers <= 16.
   * Both the bf16 and the FP8 kernel support it; lse must be NULL; rows of a q-range without keys are stored as zeros at
   * the same destinations. */
  void* const* o_peer_ptrs;
  const int32_t* o_peer_offsets;   /* [n_o_peers + 1] */
  int32_t n_o_peers;
  int32_t o_head_offset;
  /* Optional head-block output layout: with o_heads_per_block > 0 the 128 columns of (global) head h start at
   * (h / o_heads_per_block) * o_stride_block + (h % o_heads_per_block) * o_stride_h instead of h * o_stride_h.  This
   * writes core_attn_out (and, with `out` advanced by one block width, cross_attn_out) straight into the operand of the
   * output projection, i.e. the concat + rearrange "sq b (n hn hd) -> sq b (hn n hd)", n=2, hn=8 of attn_linear_proj
   * (inference/model/dit/dit_module.py:1332-1346): o_heads_per_block = Hq/8, o_stride_block = 2 * (Hq/8) * 128. */
  int32_t o_heads_per_block;
  int32_t reserved2;
  int64_t o_stride_block;
} magi_attn_params;
MAGI_API int magi_chunk_attn_fwd(magi_ctx* ctx, const magi_attn_params* p, void* stream);
/* DIAGNOSTIC ONLY - not a fallback and never dispatched to by the library or its Python shim: same plan, same arguments
 * (bf16 only, no fused output exchange), plain CUDA-core arithmetic in fp32, one to two orders of magnitude slower.  It
 * exists so that a numerical failure can be attributed to the plan or to the tensor-core kernel.  No reference
 * counterpart. */
MAGI_API int magi_chunk_attn_fwd_simt(magi_ctx* ctx, const magi_attn_params* p, void* stream);

/* Attention forward for callers that are not allowed to allocate device memory.  It has no counterpart in the
 * reference.  Who needs it: a serving process that has already handed (nearly) all of HBM to its own arenas - KV pools
 * sized to fill the GPU, a framework allocator that owns the rest - where a late cudaMalloc, even of the 640 KiB a
 * context needs, can fail or stall the device; and plug-in hosts that forbid raw CUDA allocations in their workers.
 * Same arithmetic and same kernel as magi_chunk_attn_fwd (bf16), but no context: the planner's scratch is a fixed
 * 640 KiB array inside the library image (one per GPU that loads the library, kept until exit).  The caller passes
 * inputs and outputs as usual; nothing here calls cudaMalloc/cudaFree or any allocating routine.
 *   - Limits: n_ranges <= 1024, n_ranges * ceil(max_seqlen_q / 256) <= 16384, n_k_ranges + n_prefix_chunks <= 4096;
 *     anything larger is rejected with MAGI_E_NOMEM and a message, nothing is launched.
 *   - Works on the CURRENT device.  The first call on each device also does a one-time set-up (symbol address
 *     lookup, shared-memory opt-in); make that first call outside any stream capture, from one thread.
 *   - Every call on a device shares the one scratch array, which keeps the previous call's contents; the entry point
 *     clears the part that must start at zero.  Two calls whose GPU work can overlap (different streams, or several
 *     threads) race on it: keep the calls of one device stream-ordered.
 *   - status_dev (device int32*, may be NULL) receives, stream-ordered, the planner/kernel status word
 *     (0, MAGI_E_RANGE or MAGI_E_TIMEOUT) of THIS call.  Clearing the scratch header at the start of every call also
 *     clears that word, so a failure of an earlier call (a sticky MAGI_E_TIMEOUT included) is visible only to the
 *     caller that passed status_dev on that earlier call; without status_dev a device-side failure goes unreported.
 *     err/err_len (host buffer, may be NULL/0) receives the failure text. */
MAGI_API int magi_chunk_attn_fwd_noalloc(const magi_attn_params* p, void* stream, int32_t* status_dev, char* err,
                                         int err_len);

/* ------------------------------------------------------------------------------------------------------
 * Gated post-norm residual around the attention (and MLP) block.  Replaces bias_modulate_add
 * (inference/model/dit/dit_module.py:288-307) and the Triton range_mod kernel inside it (:201-285), as called by
 * TransformerLayer.gating_and_mlp (:1348-1367) on the output of the attention projection:
 *     out[row] = post_norm( x[row] * gate[condition_map[row]] ) + residual[row]        (fp32 arithmetic, bf16 result)
 * with post_norm = FusedLayerNorm over `hidden` (weight gamma, +1 when gamma_plus_one; :355-357).  One pass over HBM
 * instead of the reference's x.float() / gating / layer_norm / add / cast passes.
 * Rows are the flattened (batch, sequence) rows the reference forms with x.transpose(0, 1).flatten(0, 1); condition_map
 * holds, per row, the row of `gate` (gatings.flatten(0, 1)) to use.  gamma == NULL skips the norm (plain range_mod),
 * residual == NULL skips the add.  A map entry outside [0, n_gates) leaves that row unwritten and sets the context's
 * device status word to MAGI_E_RANGE (read it with magi_ctx_status).
 */
typedef struct {
  uint32_t struct_size;
  int32_t x_dtype;              /* MAGI_DTYPE_BF16 or MAGI_DTYPE_F32 (the projection runs in fp32 when not quantised) */
  const void* x;                /* [rows, hidden], row stride in elements                              */
  int64_t x_stride;
  const void* residual;         /* [rows, hidden] or NULL                                              */
  int64_t residual_stride;
  int32_t residual_dtype;       /* MAGI_DTYPE_BF16 or MAGI_DTYPE_F32                                   */
  int32_t gate_dtype;           /* MAGI_DTYPE_BF16 or MAGI_DTYPE_F32                                   */
  const void* gate;             /* [n_gates, hidden]; gate_stride lets it be one half of the fused (msa | mlp) gates */
  int64_t gate_stride;
  const void* condition_map;    /* device int32 or int64 [rows], or NULL (every row uses gate row 0)   */
  int32_t map_is_int64;
  int32_t n_gates;
  const float* gamma;           /* fp32 [hidden] or NULL                                               */
  const float* beta;            /* fp32 [hidden] or NULL                                               */
  float eps;
  int32_t gamma_plus_one;       /* the reference's apply_layernorm_1p                                  */
  void* out;                    /* bf16 [rows, hidden]                                                 */
  int64_t out_stride;
  int32_t rows, hidden;         /* hidden: multiple of 8, at most 8192                                 */
} magi_modulate_params;
MAGI_API int magi_bias_modulate_add(magi_ctx* ctx, const magi_modulate_params* p, void* stream);

/* Activation quantiser of the FP8 linear layers.  Replaces div_clamp_to (inference/model/dit/dit_module.py:364-384) as
 * called by PerTensorQuantizedFp8Linear.forward (:449-461) and PerChannelQuantizedFp8Linear.forward (:484-495):
 *     out = e4m3( bf16( clamp( float(x) / scale, -448, 448 ) ) )       x bf16 [rows, cols], out e4m3 [rows, cols]
 * with `scale` fp32 [cols] (one per input channel) or, with scale_is_scalar, a single fp32.  Both roundings of the
 * reference (to bf16, then to e4m3) are reproduced, so the bytes equal the reference's.  Strides in elements; cols a
 * multiple of 8.  The GEMM that follows in the reference (bmm_fp8) is a library GEMM and is not part of this library. */
MAGI_API int magi_div_clamp_to_e4m3(magi_ctx* ctx, const void* x, int64_t x_stride, int rows, int cols, const float* scale,
                                    int scale_is_scalar, void* out, int64_t out_stride, void* stream);

/* Peer-visible device buffers for the fused Ulysses exchange: cudaMalloc + CUDA IPC (plain peer loads / stores over
 * NVLink; no multicast object is created).  magi_peer_alloc returns the local pointer and a 64-byte handle to hand to
 * the other ranks of the box (e.g. through torch.distributed all_gather_object); magi_peer_open maps a peer's handle.
 * No reference counterpart (the reference moves the data with NCCL all_to_all_single, context_parallel.py:398,420). */
MAGI_API int magi_peer_alloc(magi_ctx* ctx, uint64_t bytes, void** dev_ptr, unsigned char handle_out[64]);
MAGI_API int magi_peer_open(magi_ctx* ctx, const unsigned char handle[64], void** dev_ptr);
MAGI_API int magi_peer_close(magi_ctx* ctx, void* dev_ptr);
MAGI_API int magi_peer_free(magi_ctx* ctx, void* dev_ptr);

/* bf16 [T,H,128] -> e4m3 [T,H,128] + fp32 scales [n_blocks,H] (scale = absmax/448 per (128-token block, head),
 * blocks counted from each multiple of chunk_tokens).  x8_lo (optional, same shape) receives the e4m3 rounding
 * residual e4m3(x/scale - x8).  No reference counterpart: the reference's attention is never FP8 (its fp8 path is
 * the linear layers, inference/model/dit/dit_module.py:431-487). */
MAGI_API int magi_quantize_e4m3_block128(magi_ctx* ctx, const void* x, int64_t stride_t, int64_t stride_h, int T, int H,
                                int chunk_tokens, void* x8, void* x8_lo, float* scales, void* stream);

/* ------------------------------------------------------------------------------------------------------
 * Ulysses head-split exchange on a communicator the library owns, for hosts that do not route their collectives through
 * torch.distributed.  Replaces all_to_all_input_split / all_to_all_output_split
 * (inference/infra/parallelism/context_parallel.py:381-401, :404-423): grouped ncclSend / ncclRecv with the uneven
 * contiguous sequence split of cp_ulysses_process (:227-254).  NCCL is resolved at run time from the libnccl.so.2 already
 * in the process; without it these entry points return MAGI_E_NCCL.  All calls are stream-ordered on `stream`.
 *   magi_ulysses_unique_id: on one rank; the caller distributes the 128 bytes (as the reference's launcher does with
 *                           its rendezvous) and every rank passes them to magi_ulysses_create (collective).
 *   split_sizes:            HOST int32 [cp], tokens per rank; rank r owns rows [sum(split[:r]), +split[r]).
 *   a2a_in  ("scatter heads"): send [cp, s_local, row_bytes] (block r = the heads of rank r, as the prologue writes it
 *                           with heads_per_block) -> recv [s_total, row_bytes] (all tokens, own heads).
 *   a2a_out ("gather heads"):  full [s_total, row_bytes] -> recv [cp, s_local, row_bytes]; magi_head_block_copy then
 *                           gives "(cp sq) hn hd -> sq (cp hn) hd" (:596).
 */
typedef struct magi_ulysses magi_ulysses;
MAGI_API int magi_ulysses_unique_id(magi_ctx* ctx, void* id128);
MAGI_API int magi_ulysses_create(magi_ctx* ctx, const void* id128, int rank, int cp, const int32_t* split_sizes,
                                 magi_ulysses** out);
MAGI_API int magi_ulysses_destroy(magi_ulysses* u);
MAGI_API int magi_ulysses_a2a_in(magi_ulysses* u, const void* send, void* recv, int64_t row_bytes, void* stream);
MAGI_API int magi_ulysses_a2a_out(magi_ulysses* u, const void* full, void* recv, int64_t row_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MAGI_ATTN_H_ */
