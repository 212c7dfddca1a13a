// Small C-ABI entry points that are not tied to one kernel file.
#include "common.cuh"

namespace spgt {
thread_local int g_last_cuda_error = 0;
}

extern "C" const char* spgt_error_string(int code) {
    switch (code) {
        case SPGT_OK: return "ok";
        case SPGT_ERR_NULL: return "a required pointer is NULL";
        case SPGT_ERR_SHAPE: return "a size is out of range or the combination of sizes is not supported";
        case SPGT_ERR_ALIGN: return "a base pointer is not 16-byte aligned";
        case SPGT_ERR_WORKSPACE: return "workspace missing or too small";
        case SPGT_ERR_LAUNCH: return "the CUDA runtime refused the launch";
        case SPGT_ERR_TOO_LARGE: return "the problem needs more scratch than the fixed array of the no-allocation entry point holds";
        case SPGT_ERR_NOT_CONVERGED: return "the iterative solver reached its iteration limit before the requested tolerance";
        default: return "unknown spgt error code";
    }
}
extern "C" int spgt_last_cuda_error(void) { return spgt::g_last_cuda_error; }
extern "C" int spgt_abi_version(void) { return 1; }
