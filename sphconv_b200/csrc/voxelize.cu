// Points -> range-voxel tensor on the device: the step in front of the convolution path.
//
// The reference does this on the host, one point after the other (include/point2voxel.h:411-511, driven by
// sphconv/utils/voxelize.py:122-219): transform xyz to the grid's coordinate system
// (sphconv/utils/coord_transform.py), floor the three coordinates to a cell, number voxels in the order their first
// point appears with a dense lookup grid, keep the first max_points points of a voxel, stop the walk when voxel
// number max_voxels would be opened; then a mean over the kept points (sphconv/vfe.py:223-228), a copy to the device
// and init_tensor (src/sphconv/tensor.cu:78-127).
//
// Here nothing depends on a walk.  The order-dependent parts are restated as order statistics of the point index:
//   * a voxel keeps the max_points SMALLEST point indices that fall into it      (rounds of atomicMin),
//   * the walk stops at the point that is the (max_voxels+1)-th "first point of its voxel" in index order
//     (a block scan over first-point flags, run only for a scan with more voxels than max_voxels); every point from
//     there on is dropped and the passes are repeated once.
// Rows come out directly in range-voxel order: a bit per voxel in per-column depth masks, z_ptr = prefix of the
// popcounts, row = column start + set bits below the depth (the same scheme as init_tensor's, without COO rows in
// between and without a lookup grid).
//
// Cell arithmetic follows the reference's float32 operations one by one (subtract, divide, floor), each rounded to
// nearest, so cells are identical for identical system coordinates; the transforms use CUDA's asinf/acosf/logf,
// whose last-bit rounding may differ from the host library's.
#include "common.cuh"

#include <cfloat>
#include <climits>

namespace sph {

namespace {

constexpr int kVoxThreads = 256;
constexpr int kCutThreads = 1024;
constexpr int kNone = 0x7f7f7f7f;        // what a byte-wise fill with 0x7f leaves: "no point"

struct VoxGrid {
  int B;
  int g0, g1, g2;          // cells along the first, second, third system coordinate
  float lo[3], hi[3];
  int max_points, max_voxels, append_mode;
  int words;               // 32-bit mask words per column (depth = first coordinate, g0 cells)
  int64_t ncols;           // B * g2 * g1
};

struct VoxScratch {
  size_t header, cut, mask, blocksum, cell, row, sel, total;
};

VoxScratch vox_layout(const VoxGrid& g, int64_t n) {
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  VoxScratch l;
  l.header = 0;
  l.cut = 256;
  l.mask = l.cut + up((size_t)g.B * sizeof(int));
  l.blocksum = l.mask + up((size_t)g.ncols * g.words * sizeof(uint32_t));
  l.cell = l.blocksum + up((size_t)div_up64(g.ncols, 256) * sizeof(int));
  l.row = l.cell + up((size_t)n * sizeof(int2));
  l.sel = l.row + up((size_t)n * sizeof(int));
  l.total = l.sel + up((size_t)n * sizeof(int) * (size_t)g.max_points);
  return l;
}

int make_vox_grid(const sph_voxel_grid* s, VoxGrid* o) {
  SPH_CHECK_ARG(s != nullptr, "grid is null");
  VoxGrid g;
  g.B = s->B;
  g.g0 = s->cells[0]; g.g1 = s->cells[1]; g.g2 = s->cells[2];
  for (int i = 0; i < 3; ++i) { g.lo[i] = s->range[i]; g.hi[i] = s->range[3 + i]; }
  g.max_points = s->max_points; g.max_voxels = s->max_voxels; g.append_mode = s->append_mode;
  SPH_CHECK_ARG(g.B > 0 && g.g0 > 0 && g.g1 > 0 && g.g2 > 0, "batch and cells must be positive");
  SPH_CHECK_ARG(g.max_points > 0 && g.max_points <= 64, "max_points must be in 1..64");
  SPH_CHECK_ARG(g.max_voxels > 0, "max_voxels must be positive");
  SPH_CHECK_ARG(g.append_mode >= 0 && g.append_mode <= 2, "append_mode must be 0, 1 or 2");
  g.words = div_up(g.g0, 32);
  g.ncols = (int64_t)g.B * g.g2 * g.g1;
  SPH_CHECK_ARG(g.ncols <= 0x7fffffffLL, "more than 2^31 columns");
  *o = g;
  return SPH_OK;
}

// Largest b with scan_ptr[b] <= i (scan_ptr ascending, scan_ptr[0] = 0, i < scan_ptr[B]).
__device__ __forceinline__ int scan_of(const int* __restrict__ scan_ptr, int B, int64_t i) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((int64_t)__ldg(scan_ptr + mid) <= i) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// floor((v - lo) / ((hi - lo) / cells)) in float32, one rounding per operation; -1 when outside [0, cells) or not a
// number (the reference converts the float to int, which sends those to INT_MIN, and skips the point).
__device__ __forceinline__ int cell_of(float v, float lo, float hi, int cells) {
  const float size = __fdiv_rn(__fsub_rn(hi, lo), (float)cells);
  const float f = floorf(__fdiv_rn(__fsub_rn(v, lo), size));
  return (f >= 0.0f && f < (float)cells) ? (int)f : -1;
}

// sys [n][4] = (first, second, third coordinate, intensity) of every point.
__global__ void __launch_bounds__(kVoxThreads)
voxel_transform_kernel(const float* __restrict__ pts, int stride, int64_t n, int system, float4* __restrict__ sys) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float* p = pts + i * stride;
  const float x = __ldg(p), y = __ldg(p + 1), z = __ldg(p + 2), w = __ldg(p + 3);
  const float x2y2 = __fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y));
  const float planar = __fsqrt_rn(x2y2);
  const float radial = __fsqrt_rn(__fadd_rn(x2y2, __fmul_rn(z, z)));
  const int base = system >> 1;                    // 0 spherical, 1 cylinder, 2 hybrid; bit 0: logarithmic range
  float first = base == 0 ? radial : planar;
  if (system & 1) first = logf(first);
  const float phi = asinf(__fdiv_rn(y, planar));
  const float third = base == 1 ? z : acosf(__fdiv_rn(z, radial));
  sys[i] = make_float4(first, phi, third, w);
}

// Cell of every point ({column, depth} or {-1, -1}) and the voxel's bit in the column mask.
__global__ void __launch_bounds__(kVoxThreads)
voxel_bin_kernel(const float4* __restrict__ sys, int64_t n, const int* __restrict__ scan_ptr, VoxGrid g,
                 const int* __restrict__ cut, uint32_t* __restrict__ mask, int2* __restrict__ cell) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int b = scan_of(scan_ptr, g.B, i);
  int2 out = make_int2(-1, -1);
  if (i < (int64_t)__ldg(cut + b)) {
    const float4 s = __ldg(sys + i);
    const int c0 = cell_of(s.z, g.lo[2], g.hi[2], g.g2);
    const int c1 = cell_of(s.y, g.lo[1], g.hi[1], g.g1);
    const int c2 = cell_of(s.x, g.lo[0], g.hi[0], g.g0);
    if (c0 >= 0 && c1 >= 0 && c2 >= 0) {
      const int64_t col = ((int64_t)b * g.g2 + c0) * g.g1 + c1;
      out = make_int2((int)col, c2);
      atomicOr(mask + col * g.words + (c2 >> 5), 1u << (c2 & 31));
    }
  }
  cell[i] = out;
}

// Row of every point's voxel, and the smallest point index of every row.
__global__ void __launch_bounds__(kVoxThreads)
voxel_rows_kernel(const int2* __restrict__ cell, int64_t n, int words, const uint32_t* __restrict__ mask,
                  const int* __restrict__ z_ptr, int* __restrict__ row, int* __restrict__ sel0) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int2 c = cell[i];
  int r = -1;
  if (c.x >= 0) {
    const uint32_t* m = mask + (int64_t)c.x * words;
    int below = 0;
    const int w_hit = c.y >> 5;
    for (int w = 0; w < w_hit; ++w) below += __popc(__ldg(m + w));
    below += __popc(__ldg(m + w_hit) & ((1u << (c.y & 31)) - 1u));
    r = (c.x == 0 ? 0 : __ldg(z_ptr + c.x - 1)) + below;
    atomicMin(sel0 + r, (int)i);
  }
  row[i] = r;
}

// Next smallest point index of every row: the smallest one above the previous round's.
__global__ void __launch_bounds__(kVoxThreads)
voxel_next_kernel(const int* __restrict__ row, int64_t n, const int* __restrict__ sel_prev, int* __restrict__ sel_cur) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = __ldg(row + i);
  if (r >= 0 && (int)i > __ldg(sel_prev + r)) atomicMin(sel_cur + r, (int)i);
}

// One block per scan.  A scan with more than max_voxels voxels: find the point that opens voxel number
// max_voxels + 1 in index order and record it as the scan's cut.
__global__ void __launch_bounds__(kCutThreads)
voxel_cut_kernel(const int* __restrict__ scan_ptr, VoxGrid g, const int* __restrict__ z_ptr,
                 const int* __restrict__ row, const int* __restrict__ sel0, int64_t n, int* __restrict__ cut,
                 int* __restrict__ any_cut) {
  __shared__ int s_warp[kCutThreads / 32];
  __shared__ int s_running;
  const int b = blockIdx.x;
  const int64_t cols_per_scan = (int64_t)g.g2 * g.g1;
  const int end_rows = __ldg(z_ptr + (b + 1) * cols_per_scan - 1);
  const int begin_rows = b == 0 ? 0 : __ldg(z_ptr + b * cols_per_scan - 1);
  if (end_rows - begin_rows <= g.max_voxels) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_running = 0;
  __syncthreads();
  const int begin = max(__ldg(scan_ptr + b), 0), end = (int)min((int64_t)__ldg(scan_ptr + b + 1), n);
  for (int base = begin; base < end; base += kCutThreads) {
    const int i = base + tid;
    int flag = 0;
    if (i < end) {
      const int r = __ldg(row + i);
      flag = r >= 0 && __ldg(sel0 + r) == i;
    }
    const unsigned bal = __ballot_sync(0xffffffffu, flag);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int before = s_running;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    const int ordinal = before + __popc(bal & ((2u << lane) - 1u));      // 1-based number of this first point
    if (flag && ordinal == g.max_voxels + 1) {
      cut[b] = i;
      *any_cut = 1;
    }
    int total = 0;
    for (int w = 0; w < kCutThreads / 32; ++w) total += s_warp[w];
    __syncthreads();
    if (tid == 0) s_running += total;
    __syncthreads();
    if (s_running > g.max_voxels) break;
  }
}

// One thread per (row, feature): mean of the kept points in index order; the feature-0 thread also writes the row's
// depth, coordinates and point count.
__global__ void __launch_bounds__(kVoxThreads)
voxel_mean_kernel(const float* __restrict__ pts, int stride, const float4* __restrict__ sys,
                  const int* __restrict__ scan_ptr, VoxGrid g, const int2* __restrict__ cell,
                  const int* __restrict__ sel, int64_t sel_stride, int64_t nnz, int C, float* __restrict__ feature,
                  int* __restrict__ z_idx, int4* __restrict__ coords, int* __restrict__ num_points) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r = t / C;
  const int c = (int)(t % C);
  if (r >= nnz) return;
  float sum = 0.0f;
  int count = 0;
  int first = -1;
  for (int j = 0; j < g.max_points; ++j) {
    const int i = __ldg(sel + j * sel_stride + r);
    if (i == kNone) break;
    if (j == 0) first = i;
    float v;
    if (g.append_mode == 0) v = __ldg(pts + (int64_t)i * stride + c);
    else if (g.append_mode == 1) v = c < stride ? __ldg(pts + (int64_t)i * stride + c)
                                                : __ldg((const float*)(sys + i) + (c - stride));
    else v = c < 3 ? __ldg((const float*)(sys + i) + c) : __ldg(pts + (int64_t)i * stride + 3);
    sum = __fadd_rn(sum, v);
    ++count;
  }
  feature[t] = __fdiv_rn(sum, (float)count);
  if (c == 0 && first >= 0) {
    const int2 cl = cell[first];
    if (z_idx) z_idx[r] = cl.y;
    if (num_points) num_points[r] = count;
    if (coords) {
      const int c1 = cl.x % g.g1;
      const int rest = cl.x / g.g1;
      coords[r] = make_int4(rest / g.g2, rest % g.g2, c1, cl.y);
    }
  }
}

int run_passes(const float4* sys, const int* scan_ptr, int64_t n, const VoxGrid& g, const VoxScratch& l, char* scratch,
               int* z_ptr, bool with_cut_search, cudaStream_t st) {
  int* header = (int*)(scratch + l.header);            // [0] = 0 (flag for the scan), [1] = rows, [2] = a scan was cut
  int* cut = (int*)(scratch + l.cut);
  uint32_t* mask = (uint32_t*)(scratch + l.mask);
  int* blocksum = (int*)(scratch + l.blocksum);
  int2* cell = (int2*)(scratch + l.cell);
  int* row = (int*)(scratch + l.row);
  int* sel = (int*)(scratch + l.sel);
  SPH_CUDA(cudaMemsetAsync(header, 0, 256, st));
  SPH_CUDA(cudaMemsetAsync(mask, 0, l.blocksum - l.mask, st));
  const unsigned blocks = (unsigned)div_up64(n, kVoxThreads);
  if (n > 0) {
    SPH_CUDA(cudaMemsetAsync(sel, 0x7f, (size_t)n * sizeof(int) * g.max_points, st));
    voxel_bin_kernel<<<blocks, kVoxThreads, 0, st>>>(sys, n, scan_ptr, g, cut, mask, cell);
    SPH_LAUNCH_CHECK();
  }
  int rc = column_prefix_from_masks(mask, g.words, g.ncols, header, z_ptr, blocksum, header + 1, st);
  if (rc != SPH_OK) return rc;
  if (n > 0) {
    voxel_rows_kernel<<<blocks, kVoxThreads, 0, st>>>(cell, n, g.words, mask, z_ptr, row, sel);
    SPH_LAUNCH_CHECK();
    for (int j = 1; j < g.max_points; ++j) {
      voxel_next_kernel<<<blocks, kVoxThreads, 0, st>>>(row, n, sel + (int64_t)(j - 1) * n, sel + (int64_t)j * n);
      SPH_LAUNCH_CHECK();
    }
    if (with_cut_search) {
      voxel_cut_kernel<<<g.B, kCutThreads, 0, st>>>(scan_ptr, g, z_ptr, row, sel, n, cut, header + 2);
      SPH_LAUNCH_CHECK();
    }
  }
  return SPH_OK;
}

}  // namespace

}  // namespace sph

using namespace sph;

extern "C" int sph_voxel_transform(const float* d_points, int32_t point_stride, int64_t n_points, int system,
                                   float* d_sys_points, void* stream) {
  SPH_CHECK_ARG(n_points >= 0 && n_points < 0x7fffffffLL, "bad point count");
  SPH_CHECK_ARG(point_stride >= 4, "a point has at least x, y, z and an intensity");
  SPH_CHECK_ARG(system >= 0 && system <= 5, "unknown coordinate system");
  if (n_points == 0) return SPH_OK;
  SPH_CHECK_ARG(d_points && d_sys_points, "null pointer");
  SPH_CHECK_ARG(((uintptr_t)d_sys_points & 15) == 0, "system points must be 16-byte aligned");
  voxel_transform_kernel<<<(unsigned)div_up64(n_points, kVoxThreads), kVoxThreads, 0, (cudaStream_t)stream>>>(
      d_points, point_stride, n_points, system, (float4*)d_sys_points);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

extern "C" int64_t sph_voxelize_scratch_bytes(const sph_voxel_grid* grid, int64_t n_points) {
  VoxGrid g;
  int rc = make_vox_grid(grid, &g);
  if (rc != SPH_OK) return rc;
  if (n_points < 0 || n_points >= 0x7fffffffLL) return SPH_ERR_INVALID;
  return (int64_t)vox_layout(g, n_points).total;
}

extern "C" int sph_voxelize_count(const float* d_sys_points, const int32_t* d_scan_ptr, int64_t n_points,
                                  const sph_voxel_grid* grid, void* d_scratch, int32_t* d_z_ptr, int32_t* h_nnz,
                                  void* stream) {
  VoxGrid g;
  int rc = make_vox_grid(grid, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(n_points >= 0 && n_points < 0x7fffffffLL, "bad point count");
  SPH_CHECK_ARG(d_scan_ptr && d_scratch && d_z_ptr && h_nnz, "null pointer");
  SPH_CHECK_ARG(n_points == 0 || d_sys_points, "null pointer");
  SPH_CHECK_ARG(((uintptr_t)d_sys_points & 15) == 0 && ((uintptr_t)d_scratch & 255) == 0, "misaligned pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const VoxScratch l = vox_layout(g, n_points);
  char* scratch = (char*)d_scratch;
  SPH_CUDA(cudaMemsetAsync(scratch + l.cut, 0x7f, (size_t)g.B * sizeof(int), st));     // no scan is cut
  rc = run_passes((const float4*)d_sys_points, d_scan_ptr, n_points, g, l, scratch, d_z_ptr, true, st);
  if (rc != SPH_OK) return rc;
  int32_t host[2] = {0, 0};                            // rows, a scan was cut
  SPH_CUDA(cudaMemcpyAsync(host, scratch + l.header + 4, 8, cudaMemcpyDeviceToHost, st));
  SPH_CUDA(cudaStreamSynchronize(st));
  if (host[1]) {                                       // rare: repeat without the points behind the cuts
    rc = run_passes((const float4*)d_sys_points, d_scan_ptr, n_points, g, l, scratch, d_z_ptr, false, st);
    if (rc != SPH_OK) return rc;
    SPH_CUDA(cudaMemcpyAsync(host, scratch + l.header + 4, 8, cudaMemcpyDeviceToHost, st));
    SPH_CUDA(cudaStreamSynchronize(st));
  }
  *h_nnz = host[0];
  return SPH_OK;
}

extern "C" int sph_voxelize_fill(const float* d_points, int32_t point_stride, const float* d_sys_points,
                                 const int32_t* d_scan_ptr, int64_t n_points, const sph_voxel_grid* grid,
                                 const void* d_scratch, int64_t nnz, float* d_feature, int32_t* d_z_idx,
                                 int32_t* d_coordinates, int32_t* d_num_points, void* stream) {
  VoxGrid g;
  int rc = make_vox_grid(grid, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(n_points >= 0 && n_points < 0x7fffffffLL && nnz >= 0 && nnz <= n_points, "bad sizes");
  SPH_CHECK_ARG(point_stride >= 4, "a point has at least x, y, z and an intensity");
  if (nnz == 0) return SPH_OK;
  SPH_CHECK_ARG(d_points && d_sys_points && d_scan_ptr && d_scratch && d_feature, "null pointer");
  SPH_CHECK_ARG(((uintptr_t)d_coordinates & 15) == 0, "coordinates must be 16-byte aligned");
  const VoxScratch l = vox_layout(g, n_points);
  const char* scratch = (const char*)d_scratch;
  const int C = sph_voxel_feature_count(point_stride, g.append_mode);
  voxel_mean_kernel<<<(unsigned)div_up64(nnz * C, kVoxThreads), kVoxThreads, 0, (cudaStream_t)stream>>>(
      d_points, point_stride, (const float4*)d_sys_points, d_scan_ptr, g, (const int2*)(scratch + l.cell),
      (const int*)(scratch + l.sel), n_points, nnz, C, d_feature, d_z_idx, (int4*)d_coordinates, d_num_points);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

extern "C" int sph_voxel_feature_count(int32_t point_stride, int append_mode) {
  if (point_stride < 4 || append_mode < 0 || append_mode > 2) return SPH_ERR_INVALID;
  return append_mode == 0 ? point_stride : append_mode == 1 ? point_stride + 3 : 4;
}
