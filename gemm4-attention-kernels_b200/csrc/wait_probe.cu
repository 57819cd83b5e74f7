// splitd_wait_probe: runs the bounded wait of ptx.cuh to its limit, on purpose and harmlessly.
//
// Every mbarrier wait in the attention kernels gives up after a time limit, records a code in the caller's
// status word and lets the kernel end. This export exercises exactly that path in isolation: one CTA of one
// warp waits on an mbarrier that nobody will ever arrive on, with a limit chosen by the caller (milliseconds
// are enough), then returns through the status word like the real kernels do. No tensor memory, no cluster,
// no copy in flight, nothing to clean up; the context stays usable. It is not on any product path.
#include "launch.cuh"
#include "ptx.cuh"

namespace sd {

__global__ void splitd_wait_probe_kernel(int* status, unsigned long long limit_ns, unsigned long long* waited_ns) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
  }
  __syncthreads();
  const uint64_t t0 = globaltimer_ns();
  const bool ok = mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, status, ST_TIMEOUT_PEER, limit_ns);
  if (threadIdx.x == 0 && waited_ns) *waited_ns = ok ? 0ull : globaltimer_ns() - t0;
}

}  // namespace sd

extern "C" int splitd_wait_probe(int* status_flag, unsigned int limit_us, unsigned long long* waited_ns, void* stream) {
  using namespace sd;
  clear_error();
  if (!status_flag) return fail(SPLITD_ERR_INVALID_ARGUMENT, "status_flag is NULL");
  if (limit_us == 0 || limit_us > 100000) return fail(SPLITD_ERR_INVALID_ARGUMENT, "limit_us must be in [1, 100000]");
  splitd_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status_flag, 1000ull * limit_us, waited_ns);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "wait probe launch failed: %s", cudaGetErrorString(ce));
  return 0;
}
