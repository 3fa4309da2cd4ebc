// Bounded-wait primitive and its probe. `wait_flag_bounded` is the device-side wait used wherever
// a kernel must see a flag that another agent sets: it polls with acquire loads and gives up after
// a time limit, returning false so that the caller can record a status and leave. The probe kernel
// runs exactly that wait on one flag; tests use it with a flag that nothing sets to check that a
// missing peer ends in a TIMEOUT status, with the context still usable, never in a hang or a trap.
#include "../common/ptx.cuh"

namespace lb {
namespace {

__device__ __forceinline__ bool wait_flag_bounded(const unsigned* flag, unsigned expected,
                                                  unsigned long long limit_ns) {
  const unsigned long long t0 = globaltimer_ns();
  for (unsigned it = 0;; ++it) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == expected) return true;
    if ((it & 15u) == 15u) {
      if (globaltimer_ns() - t0 > limit_ns) return false;
      __nanosleep(200);
    }
  }
}

__global__ void bounded_wait_probe_kernel(const unsigned* flag, unsigned expected,
                                          unsigned long long limit_ns, int* status,
                                          unsigned long long* waited_ns) {
  const unsigned long long t0 = globaltimer_ns();
  const bool ok = wait_flag_bounded(flag, expected, limit_ns);
  if (!ok) report_status(status, kStatusTimeoutPeer);
  if (waited_ns != nullptr) *waited_ns = globaltimer_ns() - t0;
}

}  // namespace
}  // namespace lb

// Waits until *flag == expected or limit_ns elapsed; on expiry writes kStatusTimeoutPeer (4) into
// *status (if it was 0). waited_ns (nullable) receives the time spent waiting.
extern "C" int lb_bounded_wait_probe(const unsigned* flag, unsigned expected,
                                     unsigned long long limit_ns, int* status,
                                     unsigned long long* waited_ns, void* stream) {
  if (limit_ns > 5000000000ull) return -3;  // the probe never waits longer than 5 s
  lb::bounded_wait_probe_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      flag, expected, limit_ns, status, waited_ns);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
