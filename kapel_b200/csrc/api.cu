// Error reporting shared by all launchers, and a few queries the Python side needs.
#include "common.cuh"

namespace kb {

static thread_local char g_error[1024] = "";

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return 1;
}

static unsigned long long g_launches = 0;
static bool g_pdl = false;
bool pdl_enabled() { return g_pdl; }

int check_launch(const char* what) {
    ++g_launches;                         // every kernel launch of this library passes here once
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: launch failed: %s", what, cudaGetErrorString(e));
    return 0;
}

}  // namespace kb

extern "C" const char* kb_last_error() { return kb::g_error; }

// Kernels this library has launched (or recorded into a graph under capture) so far.
extern "C" unsigned long long kb_launch_count() { return kb::g_launches; }

// 1: the kernels of a decode step are launched as programmatic dependents of one another.
extern "C" void kb_set_pdl(int on) { kb::g_pdl = on != 0; }

// The compute capability this library was built for, as major * 10 + minor.
extern "C" int kb_built_for() { return 100; }

extern "C" int kb_device_info(int* sms, int* cc_major, int* cc_minor) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return kb::fail("device_info: no current CUDA device");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return kb::fail("device_info: cannot read device properties");
    *sms = prop.multiProcessorCount;
    *cc_major = prop.major;
    *cc_minor = prop.minor;
    return 0;
}
