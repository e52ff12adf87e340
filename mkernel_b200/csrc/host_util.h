// Host helpers shared by the translation units of the library: thread-local error text, CUDA
// error mapping, and lazy lookup of driver entry points (the library never links libcuda, so it
// loads on machines without a driver and fails only when a GPU call is made).
#pragma once
#include <cuda_runtime_api.h>

namespace mkb {

// Records a printf-style message for mk_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// Looks up a driver API symbol through the runtime.  Returns MK_OK or MK_ERR_CUDA.
int driver_entry(const char* symbol, void** fn);

}  // namespace mkb

#define MKB_CUDA(expr)                                                                      \
  do {                                                                                      \
    cudaError_t mkb_e_ = (expr);                                                            \
    if (mkb_e_ != cudaSuccess)                                                              \
      return ::mkb::set_error(-2, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(mkb_e_), \
                              __FILE__, __LINE__);                                          \
  } while (0)
