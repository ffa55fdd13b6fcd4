// wait_probe.cu -- test-only kernels that make the library's bounded device waits run out.
//
// Every wait in the library's kernels (on an mbarrier, on a counter another CTA increments) is
// bounded: when its cycle budget is spent it records FLUKE_SM100_STATUS_TIMEOUT | (site << 8) in
// the device status word, raises the CTA's abort flag and returns, so the kernel drains and
// exits instead of hanging the GPU. The kernels below call those same wait routines
// (fluke_b200/csrc/sm100_ptx.cuh) on a barrier nobody arrives at and on a counter nobody
// increments, with a budget of about a millisecond, and return what the routines reported.
// Nothing here faults, traps or spins without a limit. Built into lib/libfluke_waitprobe.so
// (`make waitprobe cuda=1`), which is not part of libfluke; the status word it reads is its own
// copy of the same variable.
#include "../../fluke_b200/csrc/sm100_ptx.cuh"

namespace {

using namespace fluke_sm100;

// out[0]: what mbar_wait returned, out[1]: the abort flag afterwards, out[2]: cycles waited.
__global__ void probe_mbar_kernel(int arrive_first, long long limit, unsigned int site, long long *out) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
        if (arrive_first) mbar_arrive(&bar);
        const long long t0 = clock64();
        const bool ok = mbar_wait(&bar, 0, &abort_flag, site, limit);
        out[0] = ok ? 1 : 0;
        out[1] = abort_flag;
        out[2] = clock64() - t0;
    }
}

// Thread 0 waits for counter[0] >= target; words[1] is the launch's global abort word.
__global__ void probe_counter_kernel(unsigned int *words, unsigned int target, long long limit, unsigned int site,
                                     long long *out) {
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        const long long t0 = clock64();
        const bool ok = wait_counter(words, target, words + 1, &abort_flag, site, limit);
        out[0] = ok ? 1 : 0;
        out[1] = abort_flag;
        out[2] = clock64() - t0;
    }
}

}  // namespace

extern "C" int fluke_probe_wait_mbar(int arrive_first, long long limit_cycles, unsigned int site, void *out_dev,
                                     void *stream) {
    probe_mbar_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(arrive_first, limit_cycles, site,
                                                                      static_cast<long long *>(out_dev));
    return (int)cudaGetLastError();
}

extern "C" int fluke_probe_wait_counter(void *words_dev, unsigned int target, long long limit_cycles, unsigned int site,
                                        void *out_dev, void *stream) {
    probe_counter_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned int *>(words_dev), target,
                                                                         limit_cycles, site,
                                                                         static_cast<long long *>(out_dev));
    return (int)cudaGetLastError();
}

// Same contract as fluke_sm100_read_status, on this library's copy of the status word.
extern "C" int fluke_probe_read_status(unsigned int *status_out, int reset) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, fluke_sm100::g_status, sizeof(v));
    if (e != cudaSuccess) return (int)e;
    if (status_out) *status_out = v;
    if (reset && v != 0) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(fluke_sm100::g_status, &zero, sizeof(zero));
    }
    return (int)e;
}
