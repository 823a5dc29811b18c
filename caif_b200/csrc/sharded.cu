// Multi-GPU forms of the frozen-linear path behind the C ABI: the same kernels plus the NCCL
// collective that a sharded layer needs, enqueued on the caller's stream with the caller's
// communicator.  The reference is single-device (no collective anywhere in it); these entry points
// exist so that a C++ host reaches the column-parallel and expert-parallel paths without Python.
//
// NCCL is not linked: the communicator comes from the host process, so the calls must go to the
// very NCCL library the host created it with.  The functions are looked up at first use among the
// libraries already loaded into the process, then in libnccl.so.2.
#include <dlfcn.h>

#include <mutex>

#include "common.cuh"

namespace caifq
{
namespace
{

// the few NCCL declarations used here (nccl.h: ncclDataType_t, ncclRedOp_t, ncclResult_t)
typedef void *nccl_comm_t;
constexpr int kNcclFloat16 = 6;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclBfloat16 = 9;
constexpr int kNcclUint8 = 1;
constexpr int kNcclSum = 0;

struct NcclFns
{
  int (*all_gather)(const void *, void *, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*reduce_scatter)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*all_reduce)(const void *, void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*send)(const void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*recv)(void *, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*group_start)() = nullptr;
  int (*group_end)() = nullptr;
  int (*comm_count)(nccl_comm_t, int *) = nullptr;
  int (*comm_user_rank)(nccl_comm_t, int *) = nullptr;
  const char *(*error_string)(int) = nullptr;
  bool ok = false;
};

NcclFns g_nccl;
std::once_flag g_nccl_once;

void *lookup(void *lib, const char *name)
{
  void *p = dlsym(RTLD_DEFAULT, name);
  if (p == nullptr && lib != nullptr)
  {
    p = dlsym(lib, name);
  }
  return p;
}

const NcclFns &nccl()
{
  std::call_once(g_nccl_once, []() {
    void *lib = nullptr;
    if (dlsym(RTLD_DEFAULT, "ncclAllGather") == nullptr)
    {
      lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    }
    NcclFns f;
    f.all_gather = reinterpret_cast<decltype(f.all_gather)>(lookup(lib, "ncclAllGather"));
    f.reduce_scatter = reinterpret_cast<decltype(f.reduce_scatter)>(lookup(lib, "ncclReduceScatter"));
    f.all_reduce = reinterpret_cast<decltype(f.all_reduce)>(lookup(lib, "ncclAllReduce"));
    f.send = reinterpret_cast<decltype(f.send)>(lookup(lib, "ncclSend"));
    f.recv = reinterpret_cast<decltype(f.recv)>(lookup(lib, "ncclRecv"));
    f.group_start = reinterpret_cast<decltype(f.group_start)>(lookup(lib, "ncclGroupStart"));
    f.group_end = reinterpret_cast<decltype(f.group_end)>(lookup(lib, "ncclGroupEnd"));
    f.comm_count = reinterpret_cast<decltype(f.comm_count)>(lookup(lib, "ncclCommCount"));
    f.comm_user_rank = reinterpret_cast<decltype(f.comm_user_rank)>(lookup(lib, "ncclCommUserRank"));
    f.error_string = reinterpret_cast<decltype(f.error_string)>(lookup(lib, "ncclGetErrorString"));
    f.ok = f.all_gather && f.reduce_scatter && f.all_reduce && f.send && f.recv && f.group_start && f.group_end &&
           f.comm_count && f.comm_user_rank && f.error_string;
    g_nccl = f;
  });
  return g_nccl;
}

int nccl_dtype(int dtype)
{
  switch (dtype)
  {
    case CAIFQ_F32:
      return kNcclFloat32;
    case CAIFQ_F16:
      return kNcclFloat16;
    case CAIFQ_BF16:
      return kNcclBfloat16;
    default:
      return -1;
  }
}

#define CAIFQ_CHECK_NCCL(expr, who)                                                  \
  do                                                                                 \
  {                                                                                  \
    const int rc__ = (expr);                                                         \
    if (rc__ != 0)                                                                   \
    {                                                                                \
      set_error("%s: %s failed: %s", who, #expr, nccl().error_string(rc__));        \
      return CAIFQ_ERR_CUDA;                                                         \
    }                                                                                \
  } while (0)

int need_nccl(const char *who, void *comm)
{
  if (!nccl().ok)
  {
    set_error("%s: NCCL is not loaded in this process and libnccl.so.2 was not found", who);
    return CAIFQ_ERR_UNSUPPORTED;
  }
  if (comm == nullptr)
  {
    set_error("%s: null communicator", who);
    return CAIFQ_ERR_INVALID;
  }
  return CAIFQ_OK;
}

}  // namespace
}  // namespace caifq

using namespace caifq;

extern "C" {

int caifq_linear_fwd_sharded(const caifq_weight *w_shard, const void *x, int32_t x_dtype, int64_t m, void *y_local,
                             void *y_gathered, int32_t y_dtype, int32_t compute_dtype, void *nccl_comm, void *stream)
{
  const char *who = "caifq_linear_fwd_sharded";
  int rc = need_nccl(who, nccl_comm);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(w_shard != nullptr && y_local != nullptr && y_gathered != nullptr, "%s: null pointer", who);
  CAIFQ_CHECK_ARG(nccl_dtype(y_dtype) >= 0, "%s: y dtype must be F32, F16 or BF16", who);
  rc = caifq_linear_fwd(w_shard, x, x_dtype, m, y_local, y_dtype, compute_dtype, stream);
  if (rc != CAIFQ_OK || m == 0)
  {
    return rc;
  }
  const size_t count = static_cast<size_t>(m) * static_cast<size_t>(w_shard->out_dim);
  CAIFQ_CHECK_NCCL(nccl().all_gather(y_local, y_gathered, count, nccl_dtype(y_dtype), nccl_comm,
                                     static_cast<cudaStream_t>(stream)),
                   who);
  return CAIFQ_OK;
}

int caifq_linear_dx_sharded(const caifq_weight *w_shard, const void *dy_local, int32_t dy_dtype, int64_t m,
                            void *dx_partial, void *dx_out, int32_t reduce_scatter, int32_t dx_dtype,
                            int32_t compute_dtype, void *nccl_comm, void *stream)
{
  const char *who = "caifq_linear_dx_sharded";
  int rc = need_nccl(who, nccl_comm);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(w_shard != nullptr && dx_partial != nullptr && dx_out != nullptr, "%s: null pointer", who);
  CAIFQ_CHECK_ARG(nccl_dtype(dx_dtype) >= 0, "%s: dx dtype must be F32, F16 or BF16", who);
  rc = caifq_linear_dx(w_shard, dy_local, dy_dtype, m, dx_partial, dx_dtype, compute_dtype, stream);
  if (rc != CAIFQ_OK || m == 0)
  {
    return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t total = static_cast<size_t>(m) * static_cast<size_t>(w_shard->in_dim);
  if (reduce_scatter)
  {
    int ranks = 0;
    CAIFQ_CHECK_NCCL(nccl().comm_count(nccl_comm, &ranks), who);
    CAIFQ_CHECK_ARG(ranks > 0 && (m % ranks) == 0, "%s: %lld rows do not split over %d ranks", who,
                    static_cast<long long>(m), ranks);
    CAIFQ_CHECK_NCCL(nccl().reduce_scatter(dx_partial, dx_out, total / static_cast<size_t>(ranks),
                                           nccl_dtype(dx_dtype), kNcclSum, nccl_comm, s),
                     who);
  }
  else
  {
    CAIFQ_CHECK_NCCL(nccl().all_reduce(dx_partial, dx_out, total, nccl_dtype(dx_dtype), kNcclSum, nccl_comm, s), who);
  }
  return CAIFQ_OK;
}

int caifq_rows_all_to_all(const void *send, const int64_t *send_rows_host, void *recv, const int64_t *recv_rows_host,
                          int64_t row_bytes, void *nccl_comm, void *stream)
{
  const char *who = "caifq_rows_all_to_all";
  int rc = need_nccl(who, nccl_comm);
  if (rc != CAIFQ_OK)
  {
    return rc;
  }
  CAIFQ_CHECK_ARG(send_rows_host != nullptr && recv_rows_host != nullptr && row_bytes > 0, "%s: bad arguments", who);
  int ranks = 0;
  int me = 0;
  CAIFQ_CHECK_NCCL(nccl().comm_count(nccl_comm, &ranks), who);
  CAIFQ_CHECK_NCCL(nccl().comm_user_rank(nccl_comm, &me), who);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char *src = static_cast<const char *>(send);
  char *dst = static_cast<char *>(recv);
  int64_t send_off = 0;
  int64_t recv_off = 0;
  for (int r = 0; r < ranks; ++r)
  {
    CAIFQ_CHECK_ARG(send_rows_host[r] >= 0 && recv_rows_host[r] >= 0, "%s: negative row count", who);
  }
  CAIFQ_CHECK_ARG(send_rows_host[me] == recv_rows_host[me], "%s: a rank must keep as many rows as it takes from itself",
                  who);
  CAIFQ_CHECK_ARG(send_rows_host[me] == 0 || (send != nullptr && recv != nullptr), "%s: null buffer", who);
  CAIFQ_CHECK_NCCL(nccl().group_start(), who);
  for (int r = 0; r < ranks; ++r)
  {
    const int64_t ns = send_rows_host[r];
    const int64_t nr = recv_rows_host[r];
    if (r == me)
    {
      // a rank's own rows never touch the network
      if (ns > 0)
      {
        CAIFQ_CHECK_CUDA(cudaMemcpyAsync(dst + recv_off * row_bytes, src + send_off * row_bytes,
                                         static_cast<size_t>(ns * row_bytes), cudaMemcpyDeviceToDevice, s));
      }
    }
    else
    {
      if (ns > 0)
      {
        CAIFQ_CHECK_NCCL(nccl().send(src + send_off * row_bytes, static_cast<size_t>(ns * row_bytes), kNcclUint8, r,
                                     nccl_comm, s),
                         who);
      }
      if (nr > 0)
      {
        CAIFQ_CHECK_NCCL(nccl().recv(dst + recv_off * row_bytes, static_cast<size_t>(nr * row_bytes), kNcclUint8, r,
                                     nccl_comm, s),
                         who);
      }
    }
    send_off += ns;
    recv_off += nr;
  }
  CAIFQ_CHECK_NCCL(nccl().group_end(), who);
  return CAIFQ_OK;
}

}  // extern "C"
