// Small helpers of the library itself: error names, and what it was built for.
#include "common.cuh"

LLM_EXPORT const char* llm_error_string(int code) {
    if (code == LLM_ERR_BAD_ARGUMENT) return "bad argument";
    if (code == LLM_ERR_UNSUPPORTED) return "size not supported by this kernel";
    return cudaGetErrorString((cudaError_t)code);
}

LLM_EXPORT const char* llm_built_for() { return "sm_100a"; }
