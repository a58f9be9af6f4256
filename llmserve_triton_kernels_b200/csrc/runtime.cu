// Small helpers of the library itself: error names, and what it was built for.
#include "common.cuh"

LLM_EXPORT const char* llm_error_string(int code) {
    if (code == LLM_ERR_BAD_ARGUMENT) return "bad argument";
    if (code == LLM_ERR_UNSUPPORTED) return "size not supported by this kernel";
    return cudaGetErrorString((cudaError_t)code);
}

LLM_EXPORT const char* llm_built_for() { return "sm_100a"; }

namespace {
int* error_flag_of_library = nullptr;
}
int* library_error_flag() { return error_flag_of_library; }
// A word of pinned host memory (or null) that kernels whose entry points take no error flag set to 1 when one of their
// bounded waits gives up.
LLM_EXPORT int llm_set_error_flag(int* flag) {
    error_flag_of_library = flag;
    return 0;
}
