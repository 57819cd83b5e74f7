// splitd_bwd_static_scratch: the whole backward for callers that cannot allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- a real-time or interrupt-like host
// thread that must not take the allocator's locks, a plugin whose host framework owns all device memory and
// hands out only the tensors of the op's signature, or a process that was given a fixed memory budget up
// front. splitd_bwd needs three scratch buffers besides its
// inputs and outputs (dpsum, lse_log2 and the P/dS tile workspace); here they live in one file-scope
// __device__ array of fixed size, so the entry point calls no cudaMalloc / cudaFree / allocating library
// routine at all. The price is a hard upper bound on the problem size and 17 MiB of device memory held by
// every GPU that loads the library, until the process exits.
//
// Host code must not use the array's name as a pointer: on the host that name is only a stand-in symbol, and
// a kernel handed it would fault (or quietly scribble on host-mapped memory). The device address is
// obtained once per device with cudaGetSymbolAddress while that device is current. That lookup happens in the
// first call on a device, so make that first call before any stream capture starts.
// All calls share the array and it keeps the last call's contents; calls that overlap on the GPU race on it.
#include <mutex>

#include "launch.cuh"

namespace sd {

constexpr size_t kStaticStatElems = 64 * 1024;              // floats per row-statistics buffer
constexpr size_t kStaticWorkspaceBytes = 16u << 20;         // bf16 P / dS tiles
constexpr size_t kStaticBytes = 2 * kStaticStatElems * sizeof(float) + kStaticWorkspaceBytes;

static __device__ __align__(256) unsigned char g_bwd_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static unsigned char* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device (resolved on first use per device).
static int scratch_base(unsigned char** out) {
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(ce));
  if (dev < 0 || dev >= kMaxDevices) return fail(SPLITD_ERR_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    ce = cudaGetSymbolAddress(&ptr, g_bwd_scratch);  // `dev` is current here
    if (ce != cudaSuccess || ptr == nullptr)
      return fail(SPLITD_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(ce));
    g_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace sd

using namespace sd;

extern "C" {

size_t splitd_bwd_static_scratch_limit_workspace(void) { return kStaticWorkspaceBytes; }
size_t splitd_bwd_static_scratch_limit_rowstat(void) { return kStaticStatElems; }

int splitd_bwd_static_scratch(const splitd_params* p, void* stream) {
  clear_error();
  if (!p) return fail(SPLITD_ERR_INVALID_ARGUMENT, "params is NULL");
  splitd_params q = *p;
  // placeholders so the shared argument checks see non-NULL scratch pointers
  q.dpsum = reinterpret_cast<float*>(1);
  q.lse_log2 = reinterpret_cast<float*>(1);
  if (int e = check_common(&q, true)) return e;
  if (int e = check_device()) return e;
  const size_t need_stat = bwd_rowstat_elems(&q);
  const size_t need_ws = bwd_workspace_bytes_full(&q);  // everything in one piece: no chunking here
  if (need_stat > kStaticStatElems)
    return fail(SPLITD_ERR_WORKSPACE,
                "problem too large for the static scratch: %zu row statistics needed, limit %zu "
                "(batch*heads_q*seqlen_q or heads_q*total_q); use splitd_bwd with caller buffers",
                need_stat, kStaticStatElems);
  if (need_ws > kStaticWorkspaceBytes)
    return fail(SPLITD_ERR_WORKSPACE,
                "problem too large for the static scratch: %zu workspace bytes needed, limit %zu; "
                "use splitd_bwd with caller buffers",
                need_ws, kStaticWorkspaceBytes);
  unsigned char* base = nullptr;
  if (int e = scratch_base(&base)) return e;
  q.dpsum = reinterpret_cast<float*>(base);
  q.lse_log2 = reinterpret_cast<float*>(base) + kStaticStatElems;
  q.workspace = base + 2 * kStaticStatElems * sizeof(float);
  q.workspace_bytes = kStaticWorkspaceBytes;
  // The array keeps the previous call's contents. What must start at zero is the head of the workspace (the
  // work counters of the persistent kernels and the running maxima the preprocess step collects); the
  // preprocess launch clears it with a memset on `stream` first. Every row statistic and every P / dS tile
  // that a later kernel reads is written by an earlier kernel of the same call.
  BwdPlan pl;
  if (int e = plan_bwd(&q, pl)) return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int e = launch_bwd_preprocess(&q, s)) return e;
  for (int i = 0; i < pl.n_chunks; ++i)
    if (int e = launch_bwd_chunk(&q, pl, i, 7, s)) return e;
  return 0;
}

}  // extern "C"
