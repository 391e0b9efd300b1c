// Ulysses head-split exchange at the C level for hosts without torch.distributed: the two all-to-alls of
// inference/infra/parallelism/context_parallel.py:381-423 (all_to_all_input_split / all_to_all_output_split) as grouped
// ncclSend / ncclRecv with uneven sequence splits, on a communicator this library owns.  NCCL is looked up at run time
// (dlopen of libnccl.so.2, i.e. the copy the process already has when PyTorch is loaded), so the library neither links
// against it nor fails to load without it; every entry point returns MAGI_E_NCCL in that case.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

struct magi_ulysses {
  magi_ctx* ctx;
  ncclComm_t comm;
  int rank, cp;
  int64_t s_local, s_total;
  int64_t* offsets;  // [cp + 1] token offsets of the ranks' sequence slices
};

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) {
      *reinterpret_cast<void**>(&api.GetUniqueId) = dlsym(api.handle, "ncclGetUniqueId");
      *reinterpret_cast<void**>(&api.CommInitRank) = dlsym(api.handle, "ncclCommInitRank");
      *reinterpret_cast<void**>(&api.CommDestroy) = dlsym(api.handle, "ncclCommDestroy");
      *reinterpret_cast<void**>(&api.GroupStart) = dlsym(api.handle, "ncclGroupStart");
      *reinterpret_cast<void**>(&api.GroupEnd) = dlsym(api.handle, "ncclGroupEnd");
      *reinterpret_cast<void**>(&api.Send) = dlsym(api.handle, "ncclSend");
      *reinterpret_cast<void**>(&api.Recv) = dlsym(api.handle, "ncclRecv");
      *reinterpret_cast<void**>(&api.GetErrorString) = dlsym(api.handle, "ncclGetErrorString");
      api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd && api.Send &&
               api.Recv && api.GetErrorString;
    }
  }
  return &api;
}

int nccl_err(magi_ctx* ctx, const char* what, ncclResult_t r) {
  return magi::set_err(ctx, MAGI_E_NCCL, "%s: %s", what, nccl_api()->GetErrorString(r));
}

#define MAGI_NCCL_OK(ctx, call)                          \
  do {                                                   \
    ncclResult_t r__ = (call);                           \
    if (r__ != ncclSuccess) return nccl_err((ctx), #call, r__); \
  } while (0)

// One grouped exchange: block r of `send` (send_count[r] bytes at send_off[r]) goes to rank r, and rank r's block lands
// at recv_off[r].
int exchange(magi_ulysses* u, const char* send, const int64_t* send_off, const int64_t* send_cnt, char* recv,
             const int64_t* recv_off, const int64_t* recv_cnt, cudaStream_t st) {
  NcclApi* n = nccl_api();
  MAGI_NCCL_OK(u->ctx, n->GroupStart());
  for (int r = 0; r < u->cp; ++r) {
    if (send_cnt[r] > 0) MAGI_NCCL_OK(u->ctx, n->Send(send + send_off[r], (size_t)send_cnt[r], ncclUint8, r, u->comm, st));
    if (recv_cnt[r] > 0) MAGI_NCCL_OK(u->ctx, n->Recv(recv + recv_off[r], (size_t)recv_cnt[r], ncclUint8, r, u->comm, st));
  }
  MAGI_NCCL_OK(u->ctx, n->GroupEnd());
  return MAGI_OK;
}

}  // namespace

extern "C" int magi_ulysses_unique_id(magi_ctx* ctx, void* id128) {
  if (!ctx || !id128) return MAGI_E_BADARG;
  NcclApi* n = nccl_api();
  if (!n->ok) return magi::set_err(ctx, MAGI_E_NCCL, "NCCL (libnccl.so.2) is not available in this process");
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  ncclUniqueId id;
  MAGI_NCCL_OK(ctx, n->GetUniqueId(&id));
  memcpy(id128, &id, sizeof(id));
  return MAGI_OK;
}

extern "C" int magi_ulysses_create(magi_ctx* ctx, const void* id128, int rank, int cp, const int32_t* split_sizes,
                                   magi_ulysses** out) {
  if (!ctx || !out) return MAGI_E_BADARG;
  *out = nullptr;
  if (!id128 || !split_sizes || cp < 1 || cp > 64 || rank < 0 || rank >= cp)
    return magi::set_err(ctx, MAGI_E_BADARG, "ulysses: need a unique id, split sizes and 0 <= rank < cp <= 64");
  NcclApi* n = nccl_api();
  if (!n->ok) return magi::set_err(ctx, MAGI_E_NCCL, "NCCL (libnccl.so.2) is not available in this process");
  magi_ulysses* u = static_cast<magi_ulysses*>(calloc(1, sizeof(magi_ulysses)));
  if (!u) return magi::set_err(ctx, MAGI_E_NOMEM, "ulysses: out of host memory");
  u->ctx = ctx;
  u->rank = rank;
  u->cp = cp;
  u->offsets = static_cast<int64_t*>(calloc(cp + 1, sizeof(int64_t)));
  for (int r = 0; r < cp; ++r) {
    if (split_sizes[r] < 0) {
      free(u->offsets);
      free(u);
      return magi::set_err(ctx, MAGI_E_BADARG, "ulysses: negative split size");
    }
    u->offsets[r + 1] = u->offsets[r] + split_sizes[r];
  }
  u->s_local = split_sizes[rank];
  u->s_total = u->offsets[cp];
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != ctx->device) cudaSetDevice(ctx->device);
  ncclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  ncclResult_t r = n->CommInitRank(&u->comm, cp, id, rank);
  if (prev != ctx->device) cudaSetDevice(prev);
  if (r != ncclSuccess) {
    free(u->offsets);
    free(u);
    return nccl_err(ctx, "ncclCommInitRank", r);
  }
  *out = u;
  return MAGI_OK;
}

extern "C" int magi_ulysses_destroy(magi_ulysses* u) {
  if (!u) return MAGI_OK;
  if (u->comm) nccl_api()->CommDestroy(u->comm);
  free(u->offsets);
  free(u);
  return MAGI_OK;
}

// "scatter heads": send [cp, s_local, row_bytes] -> recv [s_total, row_bytes]
extern "C" int magi_ulysses_a2a_in(magi_ulysses* u, const void* send, void* recv, int64_t row_bytes, void* stream) {
  if (!u) return MAGI_E_BADARG;
  if (!send || !recv || row_bytes <= 0) return magi::set_err(u->ctx, MAGI_E_BADARG, "ulysses a2a_in: bad argument");
  int64_t so[64], sc[64], ro[64], rc[64];
  for (int r = 0; r < u->cp; ++r) {
    so[r] = (int64_t)r * u->s_local * row_bytes;
    sc[r] = u->s_local * row_bytes;
    ro[r] = u->offsets[r] * row_bytes;
    rc[r] = (u->offsets[r + 1] - u->offsets[r]) * row_bytes;
  }
  return exchange(u, static_cast<const char*>(send), so, sc, static_cast<char*>(recv), ro, rc, reinterpret_cast<cudaStream_t>(stream));
}

// "gather heads": full [s_total, row_bytes] -> recv [cp, s_local, row_bytes]
extern "C" int magi_ulysses_a2a_out(magi_ulysses* u, const void* full, void* recv, int64_t row_bytes, void* stream) {
  if (!u) return MAGI_E_BADARG;
  if (!full || !recv || row_bytes <= 0) return magi::set_err(u->ctx, MAGI_E_BADARG, "ulysses a2a_out: bad argument");
  int64_t so[64], sc[64], ro[64], rc[64];
  for (int r = 0; r < u->cp; ++r) {
    so[r] = u->offsets[r] * row_bytes;
    sc[r] = (u->offsets[r + 1] - u->offsets[r]) * row_bytes;
    ro[r] = (int64_t)r * u->s_local * row_bytes;
    rc[r] = u->s_local * row_bytes;
  }
  return exchange(u, static_cast<const char*>(full), so, sc, static_cast<char*>(recv), ro, rc, reinterpret_cast<cudaStream_t>(stream));
}
