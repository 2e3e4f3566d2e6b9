// Error handling and device selection of the CUV surface (tools/cuv_general.hpp:16-57,
// tools/cuv_general.cu:45-80 in CUV): precondition failures and CUDA / cuvdia errors become
// std::runtime_error, exactly as cuvAssert and cuvSafeCall do there.
#pragma once
#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

#include "cuvdia.h"

namespace cuv {

inline void cuvAssertFailed(const char* msg) { throw std::runtime_error(std::string(msg)); }

inline void checkCudaError(const char* msg) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) throw std::runtime_error(std::string(msg) + ": " + cudaGetErrorString(err));
}

inline void cuvdia_check(int rc) {
    if (rc != CUVDIA_OK)
        throw std::runtime_error(std::string(cuvdia_error_string(rc)) + ": " + cuvdia_last_error_message());
}

// After a blocking operation: a kernel of this plan that ran out of polls while waiting for an asynchronous copy
// left its output incomplete and a code in the plan's health word.  CUV reports a failed operation by throwing
// (checkCudaError, tools/cuv_general.cu:51-61); so does this.  The word is cleared first, so the next call starts clean.
inline void cuvdia_check_plan(cuvdia_plan* plan) {
    int status = 0;
    cuvdia_check(cuvdia_plan_status(plan, &status));
    if (status != 0) {
        cuvdia_plan_status_clear(plan, 0);
        throw std::runtime_error("a kernel gave up a bounded wait on an asynchronous copy (status " +
                                 std::to_string(status) + "): the output is incomplete");
    }
}

inline void initCUDA(int dev = 0) {
    if (cudaSetDevice(dev) != cudaSuccess) throw std::runtime_error("initCUDA: cannot select device");
}
inline void exitCUDA() { cudaDeviceSynchronize(); }
inline void safeThreadSync() {
    if (cudaDeviceSynchronize() != cudaSuccess) checkCudaError("safeThreadSync");
}

}  // namespace cuv

#define cuvAssert(X) \
    if (!(X)) { cuv::cuvAssertFailed(#X); }
#define cuvSafeCall(X) \
    if (1) { if ((X) != cudaSuccess) cuv::checkCudaError(#X); }
