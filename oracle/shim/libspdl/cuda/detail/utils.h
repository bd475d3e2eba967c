// Stand-in for the reference's libspdl/cuda/detail/utils.h, used only when the
// reference kernel source is compiled on its own as a parity oracle.  The real
// header pulls in glog and fmt, which are not needed by the kernel file; the
// only thing that file uses from it is CHECK_CUDA.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>
#define CHECK_CUDA(expr, msg)                                                        \
  do {                                                                               \
    auto _status = (expr);                                                           \
    if (_status != cudaSuccess)                                                      \
      throw std::runtime_error(std::string(msg) + " (" + cudaGetErrorName(_status) + \
                               ")");                                                 \
  } while (0)
