// The optional exchange of the sharded operators: an in-place all-gather of a row-sharded output
// through NCCL, for host code that holds an ncclComm_t (the C++ front end's sharded run()).
//
// The reference has no multi-GPU code; the partition is the one kcg_shard_range() defines.  NCCL
// is not linked: its entry points are looked up at run time in the libnccl.so.2 the process has
// already loaded (the communicator a caller passes in was created by that same library), or, for
// callers that do not link NCCL themselves, in the first one the loader finds.
#include "common.cuh"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace kcg {
namespace {

struct NcclUniqueId { char internal[128]; };   // layout of ncclUniqueId (NCCL_UNIQUE_ID_BYTES = 128)
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(void**, int, NcclUniqueId, int);
typedef int (*CommDestroyFn)(void*);
typedef int (*CommCountFn)(void*, int*);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*BroadcastFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*GroupFn)();
typedef const char* (*ErrStrFn)(int);
constexpr int kNcclInt8 = 0;   // ncclInt8 / ncclChar

struct Nccl {
  void* handle = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  CommCountFn comm_count = nullptr, comm_user_rank = nullptr;
  AllGatherFn all_gather = nullptr;
  BroadcastFn broadcast = nullptr;
  GroupFn group_start = nullptr, group_end = nullptr;
  ErrStrFn error_string = nullptr;
  bool ok = false;
};

const Nccl& nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* nm : names) {
      n.handle = dlopen(nm, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);   // the copy the process already uses
      if (n.handle) break;
    }
    for (int i = 0; i < 2 && !n.handle; ++i) n.handle = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!n.handle) return;
    n.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(n.handle, "ncclGetUniqueId"));
    n.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(n.handle, "ncclCommInitRank"));
    n.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(n.handle, "ncclCommDestroy"));
    n.comm_count = reinterpret_cast<CommCountFn>(dlsym(n.handle, "ncclCommCount"));
    n.comm_user_rank = reinterpret_cast<CommCountFn>(dlsym(n.handle, "ncclCommUserRank"));
    n.all_gather = reinterpret_cast<AllGatherFn>(dlsym(n.handle, "ncclAllGather"));
    n.broadcast = reinterpret_cast<BroadcastFn>(dlsym(n.handle, "ncclBroadcast"));
    n.group_start = reinterpret_cast<GroupFn>(dlsym(n.handle, "ncclGroupStart"));
    n.group_end = reinterpret_cast<GroupFn>(dlsym(n.handle, "ncclGroupEnd"));
    n.error_string = reinterpret_cast<ErrStrFn>(dlsym(n.handle, "ncclGetErrorString"));
    n.ok = n.get_unique_id && n.comm_init_rank && n.comm_destroy && n.comm_count && n.comm_user_rank && n.all_gather &&
           n.broadcast && n.group_start && n.group_end;
  });
  return n;
}

int nccl_fail(const char* what, int rc) {
  const Nccl& n = nccl();
  return fail(KCG_ERR_CUDA, "%s failed: %s", what, n.error_string ? n.error_string(rc) : "NCCL error");
}

int need_nccl() {
  if (!nccl().ok) return fail(KCG_ERR_UNSUPPORTED, "NCCL (libnccl.so.2) could not be loaded in this process");
  return KCG_OK;
}

}  // namespace
}  // namespace kcg

extern "C" int kcg_nccl_unique_id(unsigned char id[128]) {
  using namespace kcg;
  clear_error();
  if (!id) return fail(KCG_ERR_INVALID_ARG, "nccl_unique_id: null pointer");
  if (int rc = need_nccl()) return rc;
  NcclUniqueId u;
  if (int rc = nccl().get_unique_id(&u)) return nccl_fail("ncclGetUniqueId", rc);
  std::memcpy(id, &u, 128);
  return KCG_OK;
}

extern "C" int kcg_nccl_comm_create(int world, int rank, const unsigned char id[128], void** comm) {
  using namespace kcg;
  clear_error();
  if (!id || !comm || world < 1 || rank < 0 || rank >= world)
    return fail(KCG_ERR_INVALID_ARG, "nccl_comm_create: world %d, rank %d", world, rank);
  if (int rc = need_nccl()) return rc;
  NcclUniqueId u;
  std::memcpy(&u, id, 128);
  void* c = nullptr;
  if (int rc = nccl().comm_init_rank(&c, world, u, rank)) return nccl_fail("ncclCommInitRank", rc);
  *comm = c;
  return KCG_OK;
}

extern "C" int kcg_nccl_comm_destroy(void* comm) {
  using namespace kcg;
  clear_error();
  if (!comm) return KCG_OK;
  if (int rc = need_nccl()) return rc;
  if (int rc = nccl().comm_destroy(comm)) return nccl_fail("ncclCommDestroy", rc);
  return KCG_OK;
}

extern "C" int kcg_shard_allgather(void* buffer, int64_t total_units, int64_t unit_bytes, int64_t granule, int world,
                                   int rank, void* nccl_comm, void* stream) {
  using namespace kcg;
  clear_error();
  if (total_units < 0 || unit_bytes <= 0 || granule <= 0 || world < 1 || rank < 0 || rank >= world)
    return fail(KCG_ERR_INVALID_ARG, "shard_allgather: total=%lld unit_bytes=%lld granule=%lld world=%d rank=%d",
                static_cast<long long>(total_units), static_cast<long long>(unit_bytes), static_cast<long long>(granule),
                world, rank);
  if (total_units == 0 || world == 1) return KCG_OK;
  if (!buffer) return fail(KCG_ERR_INVALID_ARG, "shard_allgather: null buffer");
  if (!nccl_comm) return fail(KCG_ERR_INVALID_ARG, "shard_allgather: null communicator");
  if (int rc = need_nccl()) return rc;
  const Nccl& n = nccl();
  int cw = 0, cr = -1;
  if (int rc = n.comm_count(nccl_comm, &cw)) return nccl_fail("ncclCommCount", rc);
  if (int rc = n.comm_user_rank(nccl_comm, &cr)) return nccl_fail("ncclCommUserRank", rc);
  if (cw != world || cr != rank)
    return fail(KCG_ERR_INVALID_ARG, "shard_allgather: the communicator has %d ranks and this is its rank %d, the call says %d / %d",
                cw, cr, world, rank);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(buffer);
  int64_t begin[64], count[64];
  if (world > 64) return fail(KCG_ERR_UNSUPPORTED, "shard_allgather: more than 64 ranks");
  bool even = true;
  for (int r = 0; r < world; ++r) {
    if (int rc = kcg_shard_range(total_units, world, r, granule, &begin[r], &count[r])) return rc;
    even = even && count[r] == count[0] && begin[r] == r * count[0];
  }
  if (even) {
    // in-place form: this rank's block already sits at its place in the receive buffer
    const size_t bytes = static_cast<size_t>(count[0]) * unit_bytes;
    if (int rc = n.all_gather(base + begin[rank] * unit_bytes, base, bytes, kNcclInt8, nccl_comm, s))
      return nccl_fail("ncclAllGather", rc);
    return KCG_OK;
  }
  // ragged blocks: one broadcast per owner, fused into one group
  if (int rc = n.group_start()) return nccl_fail("ncclGroupStart", rc);
  int first_err = 0;
  for (int r = 0; r < world; ++r) {
    if (count[r] == 0) continue;
    char* blk = base + begin[r] * unit_bytes;
    const int rc = n.broadcast(blk, blk, static_cast<size_t>(count[r]) * unit_bytes, kNcclInt8, r, nccl_comm, s);
    if (rc && !first_err) first_err = rc;
  }
  const int rc_end = n.group_end();
  if (first_err) return nccl_fail("ncclBroadcast", first_err);
  if (rc_end) return nccl_fail("ncclGroupEnd", rc_end);
  return KCG_OK;
}
