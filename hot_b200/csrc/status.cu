// The status word of the kernels' bounded waits: how a caller reads it, the knob that sets the time
// limit, and a probe that makes a wait run out on purpose (a barrier nothing arrives on) so that the
// give-up path can be tested without hanging or faulting anything.
#include "tma.cuh"

namespace hot {

void set_wait_limit_ns(uint64_t ns);
void set_sm_margin(int sms);

namespace {

// One warp waits, with the same routine the kernels use, on an mbarrier that no thread and no copy
// ever arrives on.  The wait runs out after `limit_ns`; the kernel then does what the real kernels do:
// sets the CTA's abort flag, ORs its bit into the caller's status word and returns normally.
__global__ void wait_probe_kernel(uint32_t* status, uint64_t limit_ns) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool ok = threadIdx.x < 16 ? mbar_wait(&bar, 0u, &abort_flag, limit_ns) : mbar_wait_parked(&bar, 0u, &abort_flag, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0 && (!ok || abort_flag) && status) atomicOr(status, HOT_STATUS_PROBE);
}

}  // namespace
}  // namespace hot

extern "C" void hot_set_wait_limit_ns(uint64_t limit_ns) { hot::set_wait_limit_ns(limit_ns ? limit_ns : 1500ull * 1000ull * 1000ull); }

extern "C" void hot_set_sm_margin(int sms) { hot::set_sm_margin(sms); }

extern "C" uint64_t hot_get_wait_limit_ns(void) { return hot::wait_limit_ns(); }

extern "C" int hot_wait_probe(uint32_t* status_word, hot_stream_t stream) {
  using namespace hot;
  if (!status_word) HOT_FAIL(HOT_ERR_ARG, "hot_wait_probe: null status word");
  const uint64_t limit = wait_limit_ns();
  if (limit > 100ull * 1000ull * 1000ull)
    HOT_FAIL(HOT_ERR_ARG, "hot_wait_probe: set a wait limit of at most 100 ms first (hot_set_wait_limit_ns); it is %llu ns",
             (unsigned long long)limit);
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status_word, limit);
  HOT_CUDA(cudaGetLastError());
  return HOT_OK;
}

extern "C" int hot_check_status(uint32_t status_value) {
  using namespace hot;
  if (status_value == 0) return HOT_OK;
  HOT_FAIL(HOT_ERR_TIMEOUT, "a bounded device-side wait ran out in:%s%s%s%s (status word 0x%x); the results of that launch are incomplete",
           (status_value & HOT_STATUS_GEMM) ? " the integer GEMM" : "", (status_value & HOT_STATUS_GO_DUAL) ? " the fused grad_out kernels" : "",
           (status_value & HOT_STATUS_GO_DUAL_TC) ? " the tensor-core grad_out kernels" : "",
           (status_value & HOT_STATUS_PROBE) ? " the wait probe" : "", status_value);
}
