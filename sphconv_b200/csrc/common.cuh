// Shared helpers of the sphconv_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>

#include "sphconv_b200.h"

namespace sph {

void set_error(const char* fmt, ...);
void note_launch();  // counts kernels launched by this library (sph_kernel_launches)

#define SPH_CHECK_ARG(cond, msg)                         \
  do {                                                   \
    if (!(cond)) {                                       \
      ::sph::set_error("%s: %s", __func__, msg);         \
      return SPH_ERR_INVALID;                            \
    }                                                    \
  } while (0)

#define SPH_CUDA(call)                                                                   \
  do {                                                                                   \
    cudaError_t e__ = (call);                                                            \
    if (e__ != cudaSuccess) {                                                            \
      ::sph::set_error("%s: %s failed: %s", __func__, #call, cudaGetErrorString(e__));   \
      return SPH_ERR_CUDA;                                                               \
    }                                                                                    \
  } while (0)

#define SPH_LAUNCH_CHECK()                                                               \
  do {                                                                                   \
    cudaError_t e__ = cudaGetLastError();                                                \
    if (e__ != cudaSuccess) {                                                            \
      ::sph::set_error("%s: kernel launch failed: %s", __func__, cudaGetErrorString(e__)); \
      return SPH_ERR_CUDA;                                                               \
    }                                                                                    \
    ::sph::note_launch();                                                                \
  } while (0)

__host__ __device__ inline int div_up(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t div_up64(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline int dtype_bytes(int dtype) {
  switch (dtype) {
    case SPH_F32: return 4;
    case SPH_F16: return 2;
    case SPH_BF16: return 2;
    case SPH_I8: return 1;
    default: return 0;
  }
}

// Multiprocessor count of the CURRENT device (cached per device ordinal, thread-safe); 0 with the error set on failure.
int current_sm_count();

// Geometry in the form the kernels take by value.
struct Geom {
  int B, H, W, D, oH, oW, oD;
  int KH, KW, KD, KV;
  int sH, sW, sD, pH, pW, pD;
  int dH, dW, dD;   // dilation: kernel offset k reads input o*s - p + k*d
  int tH, tW, tgH, tgW, nTile;
};

// Validates and converts; returns SPH_OK or an error code (message set).
int make_geom(const sph_geom* g, Geom* out);

// rules.cu: inclusive prefix over columns of the popcounts of per-column bit masks.
int column_prefix_from_masks(const uint32_t* mask, int words, int64_t ncols, const int* zero_flag, int* prefix,
                             int* blocksum, int* total_dev, cudaStream_t st);

}  // namespace sph
