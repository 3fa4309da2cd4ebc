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

// ------------------------------------------------------------------------------------------------
// Device barrier over symmetric memory: orders the ranks of a group on the stream without a
// collective-library call. Every rank owns a signal pad of `world` words; rank r announces epoch e
// by storing e into word [r] of every peer's pad (release, system scope) and then waits until every
// word of its own pad has reached e. One warp; lane p handles peer p. The wait is bounded: after
// limit_ns the kernel records kStatusTimeoutPeer and returns, so a missing peer costs a status
// word, never a hang. Epochs only grow, which makes a peer that is one barrier ahead harmless.
namespace lb {
namespace {

struct BarrierArgs {
  unsigned* pads[8];
  int world, rank;
  unsigned epoch;
  unsigned long long limit_ns;
  int* status;
};

__global__ void __launch_bounds__(32) device_barrier_kernel(BarrierArgs a) {
  const int lane = threadIdx.x;
  __threadfence_system();  // everything this rank's earlier kernels wrote is ordered before the flag
  if (lane < a.world) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.pads[lane] + a.rank), "r"(a.epoch)
                 : "memory");
    const unsigned* mine = a.pads[a.rank] + lane;
    const unsigned long long t0 = globaltimer_ns();
    for (unsigned it = 0;; ++it) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (static_cast<int>(v - a.epoch) >= 0) break;
      if ((it & 15u) == 15u) {
        if (globaltimer_ns() - t0 > a.limit_ns) {
          report_status(a.status, kStatusTimeoutPeer);
          break;
        }
        __nanosleep(100);
      }
    }
  }
  __syncwarp();
  __threadfence_system();
}

}  // namespace
}  // namespace lb

// pads[r]: rank r's signal pad (>= world u32 words, zero-initialised once) as mapped into this
// process. epoch: 1, 2, 3, … on successive barriers of this pad set (the same on every rank).
extern "C" int lb_device_barrier(const void* const* pads, int world, int rank, unsigned epoch,
                                 unsigned long long limit_ns, int* status, void* stream) {
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return -3;
  if (limit_ns > 5000000000ull) return -3;
  lb::BarrierArgs a{};
  for (int i = 0; i < world; ++i)
    a.pads[i] = static_cast<unsigned*>(const_cast<void*>(pads[i]));
  a.world = world;
  a.rank = rank;
  a.epoch = epoch;
  a.limit_ns = limit_ns;
  a.status = status;
  lb::device_barrier_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
