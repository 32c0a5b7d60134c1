// Diagnostic: one thread samples (globaltimer, clock64) on its SM at a fixed period while other
// kernels run, so the SM clock under load can be read at tens of microseconds resolution
// (nvidia-smi samples every few hundred milliseconds and misses what happens inside a burst).
// The kernel runs for n * period_ns and ends by itself; it waits on a timer only, never on
// another kernel.  While it is resident one SM has less room: a persistent cluster kernel
// beside it may run one CTA pair short, so throughput measured with the spy running is not a
// benchmark figure; the clock trace is what it is for.
#include <cuda_runtime.h>

extern "C" __global__ void clock_spy_kernel(unsigned long long* out, int n, unsigned long long period_ns) {
  if (threadIdx.x != 0) return;
  unsigned long long t_next;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_next));
  for (int i = 0; i < n; i++) {
    unsigned long long t;
    do {
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t < t_next) __nanosleep(2000);
    } while (t < t_next);
    out[2 * i] = t;                                              // nanoseconds
    out[2 * i + 1] = static_cast<unsigned long long>(clock64()); // SM clocks
    t_next += period_ns;
  }
}

// out: 2*n 64-bit words in device memory.  Returns the CUDA error code of the launch.
extern "C" int clock_spy_launch(unsigned long long* out, int n, unsigned long long period_ns, void* stream) {
  if (n <= 0 || n > (1 << 20) || period_ns < 1000 || static_cast<double>(n) * period_ns > 5e9) return -1;  // at most 5 s
  clock_spy_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(out, n, period_ns);
  return static_cast<int>(cudaGetLastError());
}
