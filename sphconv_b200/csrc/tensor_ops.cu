// COO <-> range-voxel <-> dense: the tensor operations on either side of the convolution path.
//
// The reference (src/sphconv/tensor.cu) builds a dense int32 grid [B,H,W,D] to count the voxels of every column
// (fillGridKernel + torch::sum + cumsum, tensor.cu:96-109), places the rows with one atomic per voxel (order inside a
// column = arrival order, tensor.cu:55-76) and hard-codes float.  Here the grid is one BIT per voxel (a depth bitmask
// per column), a voxel's row is "column start + set bits below its depth" - no atomics on positions, rows of a column
// come out in ascending depth (what the rule kernels' column index wants) - and rows are copied as bytes, so every
// dtype goes through the same kernels.
#include "common.cuh"

namespace sph {

namespace {

constexpr int kOpsThreads = 256;

__device__ __forceinline__ int col_begin(const int* __restrict__ zp, int64_t c) { return c == 0 ? 0 : __ldg(zp + c - 1); }

// indices [nnz][4] = (b, s0, s1, s2).  Sets the voxel's bit; out-of-range coordinates raise the status bit.
__global__ void __launch_bounds__(kOpsThreads)
mark_voxels_kernel(const int* __restrict__ idx, int64_t nnz, int B, int H, int W, int D, int words,
                   uint32_t* __restrict__ mask, int* __restrict__ status) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= nnz) return;
  const int4 v = __ldg((const int4*)idx + n);
  if ((unsigned)v.x >= (unsigned)B || (unsigned)v.y >= (unsigned)H || (unsigned)v.z >= (unsigned)W ||
      (unsigned)v.w >= (unsigned)D) {
    if (status) atomicOr(status, SPH_STATUS_BAD_INDEX);
    return;
  }
  const int64_t col = ((int64_t)v.x * H + v.y) * W + v.z;
  atomicOr(mask + col * words + (v.w >> 5), 1u << (v.w & 31));
}

// Row of every COO entry: column start + number of set bits below its depth.
__global__ void __launch_bounds__(kOpsThreads)
place_voxels_kernel(const int* __restrict__ idx, int64_t nnz, int B, int H, int W, int D, int words,
                    const uint32_t* __restrict__ mask, const int* __restrict__ z_ptr, int* __restrict__ z_idx,
                    int* __restrict__ permutation) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= nnz) return;
  const int4 v = __ldg((const int4*)idx + n);
  if ((unsigned)v.x >= (unsigned)B || (unsigned)v.y >= (unsigned)H || (unsigned)v.z >= (unsigned)W ||
      (unsigned)v.w >= (unsigned)D) {
    permutation[n] = -1;
    return;
  }
  const int64_t col = ((int64_t)v.x * H + v.y) * W + v.z;
  const uint32_t* m = mask + col * words;
  int below = 0;
  const int w_hit = v.w >> 5;
  for (int w = 0; w < w_hit; ++w) below += __popc(__ldg(m + w));
  below += __popc(__ldg(m + w_hit) & ((1u << (v.w & 31)) - 1u));
  const int pos = col_begin(z_ptr, col) + below;
  permutation[n] = pos;
  z_idx[pos] = v.w;
}

// dst[perm[n]] = src[n] (scatter) or dst[n] = src[perm[n]] (gather); rows of `row_bytes` bytes copied in pieces of
// `piece` bytes (16, 4, 2 or 1, whatever divides the row and the base addresses).
template <typename V>
__global__ void __launch_bounds__(kOpsThreads)
permute_rows_kernel(const V* __restrict__ src, V* __restrict__ dst, const int* __restrict__ perm, int64_t n_rows,
                    int pieces, int gather) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t n = t / pieces;
  const int c = (int)(t % pieces);
  if (n >= n_rows) return;
  const int p = __ldg(perm + n);
  if (p < 0) return;
  if (gather) dst[n * pieces + c] = src[(int64_t)p * pieces + c];
  else dst[(int64_t)p * pieces + c] = src[n * pieces + c];
}

// Range-voxel rows <-> dense [B,H,W,D,C]: the row's column is found by a search in z_ptr.
template <typename V>
__global__ void __launch_bounds__(kOpsThreads)
dense_rows_kernel(V* __restrict__ rows, const int* __restrict__ z_idx, const int* __restrict__ z_ptr, int64_t nnz,
                  int64_t ncols, int D, int pieces, V* __restrict__ dense, int backward, int* __restrict__ status) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t n = t / pieces;
  const int c = (int)(t % pieces);
  if (n >= nnz) return;
  int64_t lo = 0, hi = ncols - 1;          // first column whose inclusive prefix exceeds n
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (__ldg(z_ptr + mid) > n) hi = mid; else lo = mid + 1;
  }
  const int z = __ldg(z_idx + n);
  if ((unsigned)z >= (unsigned)D) {
    if (status) atomicOr(status, SPH_STATUS_BAD_INDEX);
    return;
  }
  const int64_t off = ((lo * D + z) * pieces) + c;
  if (backward) rows[n * pieces + c] = dense[off];
  else dense[off] = rows[n * pieces + c];
}

int piece_bytes(int row_bytes, const void* a, const void* b) {
  const uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)row_bytes;
  if ((bits & 15) == 0) return 16;
  if ((bits & 3) == 0) return 4;
  if ((bits & 1) == 0) return 2;
  return 1;
}

struct InitScratch {
  int words;
  int64_t ncols;
  size_t mask_bytes, blocksum_bytes;
};
InitScratch init_layout(int B, const int32_t shape[3]) {
  InitScratch l;
  l.words = div_up(shape[2], 32);
  l.ncols = (int64_t)B * shape[0] * shape[1];
  l.mask_bytes = ((size_t)l.ncols * l.words * sizeof(uint32_t) + 255) & ~(size_t)255;
  l.blocksum_bytes = ((size_t)div_up64(l.ncols, 256) * sizeof(int) + 255) & ~(size_t)255;
  return l;
}

}  // namespace

}  // namespace sph

using namespace sph;

extern "C" int64_t sph_init_tensor_scratch_bytes(int32_t B, const int32_t shape[3]) {
  if (B <= 0 || !shape || shape[0] <= 0 || shape[1] <= 0 || shape[2] <= 0) return SPH_ERR_INVALID;
  const InitScratch l = init_layout(B, shape);
  return (int64_t)(256 + l.mask_bytes + l.blocksum_bytes);
}

extern "C" int sph_init_tensor(const void* d_feature, int32_t row_bytes, int64_t nnz, const int32_t* d_indices,
                               int32_t B, const int32_t shape[3], void* d_scratch, void* d_out_feature,
                               int32_t* d_z_idx, int32_t* d_z_ptr, int32_t* d_permutation, int32_t* d_status,
                               void* stream) {
  SPH_CHECK_ARG(B > 0 && shape && shape[0] > 0 && shape[1] > 0 && shape[2] > 0, "batch and shape must be positive");
  SPH_CHECK_ARG(nnz >= 0 && row_bytes >= 0 && nnz < 0x7fffffffLL, "bad sizes");
  SPH_CHECK_ARG(d_scratch && d_z_ptr, "null pointer");
  SPH_CHECK_ARG(nnz == 0 || (d_indices && d_z_idx && d_permutation && (row_bytes == 0 || (d_feature && d_out_feature))),
                "null pointer");
  SPH_CHECK_ARG(((uintptr_t)d_indices & 15) == 0, "indices must be 16-byte aligned");
  const InitScratch l = init_layout(B, shape);
  SPH_CHECK_ARG(l.ncols <= 0x7fffffffLL, "more than 2^31 columns");
  cudaStream_t st = (cudaStream_t)stream;
  int* header = (int*)d_scratch;                           // [0] = 0 (flag for the scan), [1] = total
  uint32_t* mask = (uint32_t*)((char*)d_scratch + 256);
  int* blocksum = (int*)((char*)d_scratch + 256 + l.mask_bytes);
  SPH_CUDA(cudaMemsetAsync(d_scratch, 0, 256 + l.mask_bytes, st));
  const int H = shape[0], W = shape[1], D = shape[2];
  if (nnz > 0) {
    mark_voxels_kernel<<<(unsigned)div_up64(nnz, kOpsThreads), kOpsThreads, 0, st>>>(d_indices, nnz, B, H, W, D, l.words,
                                                                                      mask, d_status);
    SPH_LAUNCH_CHECK();
  }
  int rc = column_prefix_from_masks(mask, l.words, l.ncols, header, d_z_ptr, blocksum, header + 1, st);
  if (rc != SPH_OK) return rc;
  if (nnz > 0) {
    place_voxels_kernel<<<(unsigned)div_up64(nnz, kOpsThreads), kOpsThreads, 0, st>>>(d_indices, nnz, B, H, W, D, l.words,
                                                                                       mask, d_z_ptr, d_z_idx,
                                                                                       d_permutation);
    SPH_LAUNCH_CHECK();
    if (row_bytes > 0) {
      rc = sph_permute_rows(d_feature, row_bytes, nnz, d_permutation, 0, d_out_feature, stream);
      if (rc != SPH_OK) return rc;
    }
  }
  return SPH_OK;
}

extern "C" int sph_permute_rows(const void* d_src, int32_t row_bytes, int64_t n_rows, const int32_t* d_permutation,
                                int gather, void* d_dst, void* stream) {
  SPH_CHECK_ARG(n_rows >= 0 && row_bytes >= 0, "bad sizes");
  if (n_rows == 0 || row_bytes == 0) return SPH_OK;
  SPH_CHECK_ARG(d_src && d_dst && d_permutation, "null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int pb = piece_bytes(row_bytes, d_src, d_dst);
  const int pieces = row_bytes / pb;
  const unsigned blocks = (unsigned)div_up64(n_rows * pieces, kOpsThreads);
  switch (pb) {
    case 16: permute_rows_kernel<uint4><<<blocks, kOpsThreads, 0, st>>>((const uint4*)d_src, (uint4*)d_dst, d_permutation, n_rows, pieces, gather); break;
    case 4: permute_rows_kernel<uint32_t><<<blocks, kOpsThreads, 0, st>>>((const uint32_t*)d_src, (uint32_t*)d_dst, d_permutation, n_rows, pieces, gather); break;
    case 2: permute_rows_kernel<uint16_t><<<blocks, kOpsThreads, 0, st>>>((const uint16_t*)d_src, (uint16_t*)d_dst, d_permutation, n_rows, pieces, gather); break;
    default: permute_rows_kernel<uint8_t><<<blocks, kOpsThreads, 0, st>>>((const uint8_t*)d_src, (uint8_t*)d_dst, d_permutation, n_rows, pieces, gather); break;
  }
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

extern "C" int sph_to_dense(void* d_rows, int32_t row_bytes, int64_t nnz, const int32_t* d_z_idx,
                            const int32_t* d_z_ptr, int32_t B, const int32_t shape[3], void* d_dense, int backward,
                            int32_t* d_status, void* stream) {
  SPH_CHECK_ARG(B > 0 && shape && shape[0] > 0 && shape[1] > 0 && shape[2] > 0, "batch and shape must be positive");
  SPH_CHECK_ARG(nnz >= 0 && row_bytes >= 0, "bad sizes");
  if (nnz == 0 || row_bytes == 0) return SPH_OK;
  SPH_CHECK_ARG(d_rows && d_z_idx && d_z_ptr && d_dense, "null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t ncols = (int64_t)B * shape[0] * shape[1];
  const int pb = piece_bytes(row_bytes, d_rows, d_dense);
  const int pieces = row_bytes / pb;
  const unsigned blocks = (unsigned)div_up64(nnz * pieces, kOpsThreads);
  switch (pb) {
    case 16: dense_rows_kernel<uint4><<<blocks, kOpsThreads, 0, st>>>((uint4*)d_rows, d_z_idx, d_z_ptr, nnz, ncols, shape[2], pieces, (uint4*)d_dense, backward, d_status); break;
    case 4: dense_rows_kernel<uint32_t><<<blocks, kOpsThreads, 0, st>>>((uint32_t*)d_rows, d_z_idx, d_z_ptr, nnz, ncols, shape[2], pieces, (uint32_t*)d_dense, backward, d_status); break;
    case 2: dense_rows_kernel<uint16_t><<<blocks, kOpsThreads, 0, st>>>((uint16_t*)d_rows, d_z_idx, d_z_ptr, nnz, ncols, shape[2], pieces, (uint16_t*)d_dense, backward, d_status); break;
    default: dense_rows_kernel<uint8_t><<<blocks, kOpsThreads, 0, st>>>((uint8_t*)d_rows, d_z_idx, d_z_ptr, nnz, ncols, shape[2], pieces, (uint8_t*)d_dense, backward, d_status); break;
  }
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

// ---- backward of the fused epilogue relu(acc + bias): gradient mask and bias gradient in one pass ---------------
namespace sph {
namespace {

__device__ __forceinline__ float ld_f(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld_f(const __half* p, int64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ float ld_f(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_f(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void st_f(__half* p, int64_t i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void st_f(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

constexpr int kEpiThreads = 256;

// d_pre[r][c] = out[r][c] > 0 ? d_out[r][c] : 0 (relu) or d_out (no relu); d_bias[c] += sum_r d_pre[r][c].
// A thread stays on one channel (the first floor(256 / C) * C threads of a block work, the rest only join the
// barrier), walks rows with a grid stride and keeps its sum in a register; sums of equal channels meet in shared
// memory, one atomic per channel and block.
template <typename T>
__global__ void __launch_bounds__(kEpiThreads)
epilogue_backward_kernel(const T* __restrict__ d_out, const T* __restrict__ out, int64_t n, int C, int relu,
                         T* __restrict__ d_pre, float* __restrict__ d_bias) {
  __shared__ float s_sum[kEpiThreads];
  const int c = threadIdx.x % C;
  const int rows_per_block = kEpiThreads / C;
  const int active = rows_per_block * C;
  float sum = 0.f;
  for (int64_t r = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / C; r < n && (int)threadIdx.x < active;
       r += (int64_t)gridDim.x * rows_per_block) {
    const int64_t i = r * C + c;
    float g = ld_f(d_out, i);
    if (relu && !(ld_f(out, i) > 0.f)) g = 0.f;
    if (d_pre) st_f(d_pre, i, g);
    sum += g;
  }
  if (d_bias) {
    s_sum[threadIdx.x] = sum;
    __syncthreads();
    if (threadIdx.x < C) {
      float t = 0.f;
      for (int j = threadIdx.x; j < active; j += C) t += s_sum[j];
      atomicAdd(d_bias + threadIdx.x, t);
    }
  }
}

}  // namespace
}  // namespace sph

extern "C" int sph_epilogue_backward(const void* d_dout, const void* d_out, int dtype, int64_t n, int32_t channels,
                                     int relu, void* d_dpre, float* d_dbias, void* stream) {
  SPH_CHECK_ARG(n >= 0 && channels > 0, "bad sizes");
  SPH_CHECK_ARG(dtype == SPH_F32 || dtype == SPH_F16 || dtype == SPH_BF16, "unsupported dtype");
  SPH_CHECK_ARG(channels <= kEpiThreads, "at most 256 channels");
  cudaStream_t st = (cudaStream_t)stream;
  if (d_dbias) SPH_CUDA(cudaMemsetAsync(d_dbias, 0, (size_t)channels * sizeof(float), st));
  if (n == 0) return SPH_OK;
  SPH_CHECK_ARG(d_dout && (!relu || d_out) && (d_dpre || d_dbias), "null pointer");
  const int rows_per_block = kEpiThreads / channels;
  int64_t blocks = div_up64(n, (int64_t)rows_per_block * 8);      // ~8 rows per thread
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  switch (dtype) {
    case SPH_F32: epilogue_backward_kernel<float><<<(unsigned)blocks, kEpiThreads, 0, st>>>((const float*)d_dout, (const float*)d_out, n, channels, relu, (float*)d_dpre, d_dbias); break;
    case SPH_F16: epilogue_backward_kernel<__half><<<(unsigned)blocks, kEpiThreads, 0, st>>>((const __half*)d_dout, (const __half*)d_out, n, channels, relu, (__half*)d_dpre, d_dbias); break;
    default: epilogue_backward_kernel<__nv_bfloat16><<<(unsigned)blocks, kEpiThreads, 0, st>>>((const __nv_bfloat16*)d_dout, (const __nv_bfloat16*)d_out, n, channels, relu, (__nv_bfloat16*)d_dpre, d_dbias); break;
  }
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}
