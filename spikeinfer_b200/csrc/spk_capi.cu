// Version, error strings and per-thread launch-error bookkeeping of the C ABI.
#include "spk_common.cuh"

#include <atomic>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

namespace {
thread_local int g_last_cuda_error = 0;
std::atomic<long long> g_launches{0};
}

namespace {
bool nvtx_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("SPK_NVTX");
        return v != nullptr && std::strcmp(v, "0") != 0 && v[0] != '\0';
    }();
    return on;
}
}  // namespace

SpkRange::SpkRange(const char* name) : on(nvtx_enabled()) {
    if (on) nvtxRangePushA(name);
}

SpkRange::~SpkRange() {
    if (on) nvtxRangePop();
}

extern "C" int spk_nvtx_enabled(void) { return nvtx_enabled() ? 1 : 0; }

void spk_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

extern "C" int64_t spk_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int spk_set_cuda_error(cudaError_t err) {
    g_last_cuda_error = static_cast<int>(err);
    return SPK_ERR_CUDA;
}

extern "C" int spk_version(void) { return (0 << 16) | (1 << 8) | 0; }

extern "C" int spk_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" const char* spk_error_string(int code) {
    switch (code) {
        case SPK_OK: return "ok";
        case SPK_ERR_BAD_DTYPE: return "unsupported element type";
        case SPK_ERR_BAD_SHAPE: return "invalid shape or size argument";
        case SPK_ERR_BAD_STRIDE: return "invalid stride argument";
        case SPK_ERR_NULL_POINTER: return "required pointer is null";
        case SPK_ERR_WORKSPACE_TOO_SMALL: return "workspace missing or too small";
        case SPK_ERR_UNSUPPORTED: return "configuration not supported";
        case SPK_ERR_TOO_LARGE: return "problem exceeds a launch or capacity limit";
        case SPK_ERR_STATIC_SCRATCH_TOO_SMALL:
            return "problem needs more scratch than the library's built-in array holds (use spk_attn_decode with a workspace)";
        case SPK_ERR_CUDA: return "CUDA launch failed (see spk_last_cuda_error)";
        default: return "unknown error code";
    }
}
