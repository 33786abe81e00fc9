// Host plumbing shared by every library built from this directory: the thread-local error text behind wf_last_error(),
// CUDA status mapping, the launch counter and the cached SM count.
#include "common.cuh"
#include <stdarg.h>
#include <stdio.h>

namespace wf {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

int cuda_check(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return WF_OK;
    set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
    return WF_ERR_CUDA;
}

static thread_local long long g_launches = 0;
int launch_check(cudaError_t e, const char* what) {
    ++g_launches;
    return cuda_check(e, what);
}
long long launch_count() { return g_launches; }

int sm_count() {
    static int per_dev[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev > 63) dev = 0;
    int& n = per_dev[dev];
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

}  // namespace wf

extern "C" const char* wf_last_error(void) { return wf::g_err; }
