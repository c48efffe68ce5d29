// Library-wide entry points: version, error strings.
#include <string.h>

#include "common.cuh"

namespace mbema {
static thread_local char g_last_cuda_error[256] = "no CUDA error recorded";
void set_last_cuda_error(cudaError_t e) {
    const char* s = cudaGetErrorString(e);
    strncpy(g_last_cuda_error, s ? s : "unknown", sizeof(g_last_cuda_error) - 1);
    g_last_cuda_error[sizeof(g_last_cuda_error) - 1] = 0;
}
}  // namespace mbema

extern "C" int mbema_version(void) { return MBEMA_VERSION; }

extern "C" const char* mbema_last_cuda_error(void) { return mbema::g_last_cuda_error; }

extern "C" const char* mbema_strerror(int code) {
    switch (code) {
        case MBEMA_OK: return "ok";
        case MBEMA_ERR_NULL: return "a required pointer is NULL";
        case MBEMA_ERR_SHAPE: return "invalid shape";
        case MBEMA_ERR_UNSUPPORTED: return "shape or option not supported by this build";
        case MBEMA_ERR_WORKSPACE: return "workspace too small";
        case MBEMA_ERR_CUDA: return "CUDA runtime error (see mbema_last_cuda_error)";
        case MBEMA_ERR_DTYPE: return "unknown dtype code";
        case MBEMA_ERR_ALIGN: return "pointer not 16-byte aligned";
        case MBEMA_ERR_STATIC_LIMIT: return "problem larger than the fixed scratch of the allocation-free entry point (B*T <= 32768, B <= 1024)";
        default: return "unknown error code";
    }
}
