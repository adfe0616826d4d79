// Status strings, last-error bookkeeping and ABI version of the C interface.
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace xl {

static thread_local char g_last_cuda_error[512] = "";

void set_last_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_cuda_error, sizeof(g_last_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}

int check_launch(const char* where) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    set_last_cuda_error(e, where);
    (void)cudaGetLastError();  // clear the non-sticky launch error so that later calls are not blamed for it
    return XL_ERR_CUDA;
  }
  return XL_OK;
}

}  // namespace xl

extern "C" const char* xl_strerror(int status) {
  switch (status) {
    case XL_OK: return "ok";
    case XL_ERR_NULL_POINTER: return "a required pointer is NULL (or only part of an optional group was given)";
    case XL_ERR_BAD_SHAPE: return "a dimension is non-positive or outside what the kernel supports";
    case XL_ERR_BAD_STRIDE: return "a stride is not compatible with 16-byte vector / TMA access";
    case XL_ERR_BAD_ALIGNMENT: return "a base pointer is not sufficiently aligned";
    case XL_ERR_BAD_DTYPE: return "unsupported element type for this entry point";
    case XL_ERR_UNSUPPORTED: return "shape/dtype combination not handled by this entry point";
    case XL_ERR_CUDA: return "a CUDA call failed (see xl_last_cuda_error)";
    case XL_ERR_TOO_LARGE: return "request exceeds a fixed capacity of this entry point";
    case XL_ERR_ALIASING: return "an output overlaps an input that other thread blocks still read";
    default: return "unknown status";
  }
}

extern "C" const char* xl_last_cuda_error(void) { return xl::g_last_cuda_error; }

extern "C" int xl_abi_version(void) { return 3; }
