// Library-wide runtime state: error text, device properties, the per-device scratch
// buffer, and the small entry points that launch nothing.
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace kcg {

namespace {
thread_local char g_error[512] = {0};

constexpr int kScratchSlots = 2;   // 0: LayerNorm split-row statistics, 1: fp32 GEMM operand splits
struct DeviceState {
  int sms = 0;
  void* scratch[kScratchSlots] = {nullptr, nullptr};
  size_t scratch_bytes[kScratchSlots] = {0, 0};
  // buffers a larger request has replaced: launches already queued, and CUDA graphs captured
  // earlier, may still name them, so they stay allocated until the process exits
  std::vector<void*> retired;
};
constexpr int kMaxDevices = 64;
DeviceState g_dev[kMaxDevices];
std::mutex g_mutex;

int current_device() {
  int d = -1;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return -1;
  return d;
}
}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_error[0] = 0; }

bool overlap_launch_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("KCG_OVERLAP_LAUNCH");
    return !(e && e[0] == '0');
  }();
  return on;
}

int sm_count() {
  const int d = current_device();
  if (d < 0) return 1;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_dev[d].sms == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
    g_dev[d].sms = n;
  }
  return g_dev[d].sms;
}

// Returns a device buffer of at least `bytes` bytes for `slot`, or nullptr with *why set to a
// kcg_status.  A buffer that has been handed out is never freed: when a larger request replaces
// it, the old one is parked until the process exits, because launches in flight and CUDA graphs
// captured earlier still hold its address.  Growth allocates (cudaMalloc), which is not allowed
// while `stream` is being captured: that request is refused with KCG_ERR_UNSUPPORTED and the
// capture stays valid.
void* device_scratch(size_t bytes, int slot, cudaStream_t stream, int* why) {
  auto refuse = [&](int code, const char* fmt, size_t n) -> void* {
    if (why) *why = fail(code, fmt, n);
    return nullptr;
  };
  const int d = current_device();
  if (d < 0 || slot < 0 || slot >= kScratchSlots) return refuse(KCG_ERR_CUDA, "scratch: no current device (%zu bytes)", bytes);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState& st = g_dev[d];
  if (st.scratch_bytes[slot] >= bytes && st.scratch[slot]) return st.scratch[slot];
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
  if (cap != cudaStreamCaptureStatusNone)
    return refuse(KCG_ERR_UNSUPPORTED,
                  "the library's scratch buffer would have to grow to %zu bytes while the stream is being captured; "
                  "make one call of this size before starting the capture", bytes);
  size_t want = bytes < (1u << 20) ? (1u << 20) : bytes;
  void* p = nullptr;
  if (cudaMalloc(&p, want) != cudaSuccess) {
    cudaGetLastError();
    return refuse(KCG_ERR_CUDA, "could not allocate %zu bytes of scratch memory", want);
  }
  if (st.scratch[slot]) st.retired.push_back(st.scratch[slot]);
  st.scratch[slot] = p;
  st.scratch_bytes[slot] = want;
  return p;
}

// One host-mapped word per process that kernels write a kcg_status into when a bounded
// device-side wait gives up.  Host memory, so reading it needs no device synchronisation
// beyond the caller's own wait for the stream.
int* device_status_word() {
  static int* word = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    if (cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped) == cudaSuccess) {
      word = static_cast<int*>(p);
      *word = 0;
    } else {
      cudaGetLastError();
    }
  });
  return word;
}

}  // namespace kcg

extern "C" int kcg_device_status(void) {
  int* w = kcg::device_status_word();
  if (!w) return KCG_OK;
  const int v = *reinterpret_cast<volatile int*>(w);
  *reinterpret_cast<volatile int*>(w) = 0;
  return v;
}

extern "C" const char* kcg_status_string(int status) {
  switch (status) {
    case KCG_OK: return "ok";
    case KCG_ERR_INVALID_ARG: return "invalid argument";
    case KCG_ERR_UNSUPPORTED: return "unsupported configuration";
    case KCG_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
    case KCG_ERR_CUDA: return "CUDA call failed";
    case KCG_ERR_TIMEOUT: return "device-side wait timed out";
    case KCG_ERR_NO_DEVICE: return "no sm_100 device";
    default: return "unknown status";
  }
}

extern "C" const char* kcg_last_error(void) { return kcg::g_error; }

extern "C" int kcg_version(void) { return 100; }

extern "C" size_t kcg_dtype_size(int dtype) {
  switch (dtype) {
    case KCG_F32: case KCG_I32: return 4;
    case KCG_F16: case KCG_BF16: case KCG_I16: return 2;
    case KCG_F8E4M3: case KCG_BOOL: return 1;
    case KCG_F64: case KCG_I64: return 8;
    default: return 0;
  }
}

extern "C" int kcg_shard_range(int64_t total, int world, int rank, int64_t granule,
                               int64_t* begin, int64_t* count) {
  using namespace kcg;
  clear_error();
  if (total < 0 || world <= 0 || rank < 0 || rank >= world || granule <= 0 || !begin || !count)
    return fail(KCG_ERR_INVALID_ARG, "shard_range: total=%lld world=%d rank=%d granule=%lld",
                static_cast<long long>(total), world, rank, static_cast<long long>(granule));
  // Split the granules as evenly as possible; earlier ranks take the remainder.
  const int64_t granules = (total + granule - 1) / granule;
  const int64_t base = granules / world, extra = granules % world;
  const int64_t g0 = base * rank + (rank < extra ? rank : extra);
  const int64_t gn = base + (rank < extra ? 1 : 0);
  int64_t b = g0 * granule, e = (g0 + gn) * granule;
  if (b > total) b = total;
  if (e > total) e = total;
  *begin = b;
  *count = e - b;
  return KCG_OK;
}

// ---- device memory that other processes on the node can map ---------------------------------
// Plain cudaMalloc allocations shared through CUDA IPC handles: the owner exports a 64-byte
// handle, each peer process opens it and gets a pointer it can hand to kernels on its own GPU
// (loads and stores then travel over NVLink).
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI passes IPC handles as 64 bytes");

extern "C" int kcg_peer_alloc(size_t bytes, void** ptr) {
  using namespace kcg;
  clear_error();
  if (!ptr || bytes == 0) return fail(KCG_ERR_INVALID_ARG, "peer_alloc: null pointer or zero size");
  KCG_CUDA_OK(cudaMalloc(ptr, bytes));
  return KCG_OK;
}

extern "C" int kcg_peer_free(void* ptr) {
  using namespace kcg;
  clear_error();
  if (ptr) KCG_CUDA_OK(cudaFree(ptr));
  return KCG_OK;
}

extern "C" int kcg_peer_export(void* ptr, unsigned char handle[64]) {
  using namespace kcg;
  clear_error();
  if (!ptr || !handle) return fail(KCG_ERR_INVALID_ARG, "peer_export: null pointer");
  cudaIpcMemHandle_t h;
  KCG_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  std::memcpy(handle, &h, 64);
  return KCG_OK;
}

extern "C" int kcg_peer_open(const unsigned char handle[64], void** ptr) {
  using namespace kcg;
  clear_error();
  if (!ptr || !handle) return fail(KCG_ERR_INVALID_ARG, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  KCG_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return KCG_OK;
}

extern "C" int kcg_peer_close(void* ptr) {
  using namespace kcg;
  clear_error();
  if (ptr) KCG_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return KCG_OK;
}

// ---- small device utilities for host code that does not link the CUDA runtime itself ---------
extern "C" int kcg_device_count(int* count) {
  using namespace kcg;
  clear_error();
  if (!count) return fail(KCG_ERR_INVALID_ARG, "device_count: null pointer");
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
  *count = n;
  return KCG_OK;
}

extern "C" int kcg_device_memset(void* ptr, int byte_value, size_t bytes, void* stream) {
  using namespace kcg;
  clear_error();
  if (!ptr && bytes) return fail(KCG_ERR_INVALID_ARG, "device_memset: null pointer");
  if (bytes) KCG_CUDA_OK(cudaMemsetAsync(ptr, byte_value, bytes, static_cast<cudaStream_t>(stream)));
  return KCG_OK;
}

namespace {
struct KcgTimer { cudaEvent_t begin, end; };
}

extern "C" int kcg_timer_begin(void* stream, void** timer) {
  using namespace kcg;
  clear_error();
  if (!timer) return fail(KCG_ERR_INVALID_ARG, "timer_begin: null pointer");
  KcgTimer* t = new KcgTimer;
  if (cudaEventCreate(&t->begin) != cudaSuccess || cudaEventCreate(&t->end) != cudaSuccess) {
    delete t;
    return fail(KCG_ERR_CUDA, "timer_begin: cudaEventCreate failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  cudaEventRecord(t->begin, static_cast<cudaStream_t>(stream));
  *timer = t;
  return KCG_OK;
}

extern "C" int kcg_timer_end(void* stream, void* timer, float* milliseconds) {
  using namespace kcg;
  clear_error();
  if (!timer || !milliseconds) return fail(KCG_ERR_INVALID_ARG, "timer_end: null pointer");
  KcgTimer* t = static_cast<KcgTimer*>(timer);
  cudaEventRecord(t->end, static_cast<cudaStream_t>(stream));
  cudaError_t e = cudaEventSynchronize(t->end);
  if (e == cudaSuccess) e = cudaEventElapsedTime(milliseconds, t->begin, t->end);
  cudaEventDestroy(t->begin);
  cudaEventDestroy(t->end);
  delete t;
  if (e != cudaSuccess) return fail(KCG_ERR_CUDA, "timer_end: %s", cudaGetErrorString(e));
  return KCG_OK;
}
