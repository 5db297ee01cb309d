// Host-side plumbing shared by every entry point: error text, status mapping, device properties,
// and the device-visible error word that bounded waits report into.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace ucmx {

static thread_local char g_err[256] = "";

void set_last_error(const char* what, cudaError_t e)
{
    snprintf(g_err, sizeof(g_err), "%s: %s (%d)", what, cudaGetErrorString(e), (int)e);
}

void set_last_text(const char* text)
{
    snprintf(g_err, sizeof(g_err), "%s", text);
}

int32_t cuda_status(const char* what, cudaError_t e)
{
    set_last_error(what, e);
    cudaGetLastError();  // clear the sticky-less error so that later calls start clean
    if (e == cudaErrorMemoryAllocation) return UCMX_EOOM;
    if (e == cudaErrorInvalidValue) return UCMX_EPARAM;
    return UCMX_EOSERROR;
}

int sm_count()
{
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kSmCountHint;
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = kSmCountHint;
        cached[dev] = n;
    }
    return cached[dev];
}

// One page-locked, device-mapped int per process.  Kernels write a non-zero code into it when a
// bounded wait gives up; the host reads it without a CUDA call.
static int32_t* g_error_word = nullptr;
static std::mutex g_error_mu;

int32_t* error_word()
{
    std::lock_guard<std::mutex> lk(g_error_mu);
    if (!g_error_word) {
        void* p = nullptr;
        if (cudaHostAlloc(&p, 64, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        memset(p, 0, 64);
        g_error_word = (int32_t*)p;
    }
    return g_error_word;
}

static thread_local int32_t g_early_start = 0;

bool early_start() { return g_early_start != 0; }

}  // namespace ucmx

extern "C" {

int32_t ucmx_version(void) { return 100; }

int32_t ucmx_set_early_start(int32_t on)
{
    const int32_t was = ucmx::g_early_start;
    ucmx::g_early_start = on ? 1 : 0;
    return was;
}

int32_t ucmx_compiled_arch(void) { return 100; }

const char* ucmx_last_error(void) { return ucmx::g_err; }

int32_t ucmx_device_error(int32_t* code, int32_t clear)
{
    if (!code) return UCMX_EPARAM;
    int32_t* w = ucmx::error_word();
    if (!w) return UCMX_EOOM;
    *code = *(volatile int32_t*)w;
    if (clear) *(volatile int32_t*)w = 0;
    return UCMX_OK;
}

}  // extern "C"
