// CUDA-core (FFMA / IMAD) kernels of the rule-driven convolution.
//
// These cover what the tensor-core kernels do not: fp32 (the 1e-4 tolerance rules out single-pass
// TF32), channel counts that are not multiples of 16, and the weight gradient of every dtype.
// Output-stationary: a thread group owns one output row, walks its KV neighbour-table entries and
// accumulates in registers, so there is no scatter and no atomic in forward / dgrad
// (the reference scatters with read-modify-write per 8 pairs, include/sphconv/iterator.cu.h:1467-1625).
#include "common.cuh"

namespace sph {

namespace {

template <typename T> struct Acc { using type = float; };
template <> struct Acc<int8_t> { using type = int; };

__device__ __forceinline__ float to_acc(float v) { return v; }
__device__ __forceinline__ float to_acc(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_acc(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ int to_acc(int8_t v) { return (int)v; }

__device__ __forceinline__ void store_out(void* out, int out_dtype, int64_t idx, float v) {
  switch (out_dtype) {
    case SPH_F32: ((float*)out)[idx] = v; break;
    case SPH_F16: ((__half*)out)[idx] = __float2half_rn(v); break;
    case SPH_BF16: ((__nv_bfloat16*)out)[idx] = __float2bfloat16_rn(v); break;
    default: {
      float r = rintf(v);
      r = fminf(fmaxf(r, -127.f), 127.f);
      ((int8_t*)out)[idx] = (int8_t)(int)r;
    }
  }
}

constexpr int kGenThreads = 128;

// TPR threads per output row, each owning 4 consecutive output channels.
template <typename T>
__global__ void __launch_bounds__(kGenThreads)
conv_gather_generic_kernel(const T* __restrict__ rows, int64_t n_rows, const T* __restrict__ weight,
                           const int* __restrict__ nbr, int64_t n_out, int kv, int K, int N, int tpr, int flip_k,
                           const float* __restrict__ scale, const float* __restrict__ bias, int relu,
                           void* __restrict__ out, int out_dtype, int* __restrict__ status) {
  using A = typename Acc<T>::type;
  const int rows_per_block = kGenThreads / tpr;
  const int sub = threadIdx.x % tpr;
  const int64_t r = (int64_t)blockIdx.x * rows_per_block + threadIdx.x / tpr;
  if (r >= n_out) return;
  const int oc0 = sub * 4;
  if (oc0 >= N) return;
  const int noc = min(4, N - oc0);
  A acc[4] = {0, 0, 0, 0};
  for (int k = 0; k < kv; ++k) {
    const int tk = flip_k ? kv - 1 - k : k;
    const int i = __ldg(nbr + (int64_t)tk * n_out + r);
    if (i < 0) continue;
    if (i >= n_rows) {
      if (status) atomicOr(status, SPH_STATUS_BAD_INDEX);
      continue;
    }
    const T* x = rows + (int64_t)i * K;
    const T* w = weight + (int64_t)k * K * N + oc0;
    for (int ic = 0; ic < K; ++ic) {
      A xv = to_acc(x[ic]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < noc) acc[j] += xv * to_acc(w[(int64_t)ic * N + j]);
      }
    }
  }
  for (int j = 0; j < noc; ++j) {
    float v = (float)acc[j];
    if (scale) v *= scale[oc0 + j];
    if (bias) v += bias[oc0 + j];
    if (relu) v = fmaxf(v, 0.f);
    store_out(out, out_dtype, r * N + oc0 + j, v);
  }
}

// ---- weight gradient ---------------------------------------------------------------------------
// grid (row chunks, KV).  A block compacts the rows of its chunk that have a neighbour at offset k,
// stages 16 (x, dy) row pairs at a time in shared memory as floats and accumulates a K x N partial
// in registers (up to kWgElems per thread), then adds it to the fp32 gradient with atomics.
constexpr int kWgThreads = 256;
constexpr int kWgChunk = 2048;
constexpr int kWgTile = 16;
constexpr int kWgElems = 16;   // K*N <= 256*16 = 4096
constexpr int kWgMaxCh = 64;

template <typename T>
__global__ void __launch_bounds__(kWgThreads)
conv_wgrad_generic_kernel(const T* __restrict__ rows, const T* __restrict__ dout, int64_t n_rows,
                          const int* __restrict__ nbr, int64_t n_out, int K, int N, float* __restrict__ dw,
                          int* __restrict__ status) {
  __shared__ int s_in[kWgChunk];
  __shared__ int s_out[kWgChunk];
  __shared__ int s_n;
  __shared__ float s_x[kWgTile][kWgMaxCh];
  __shared__ float s_d[kWgTile][kWgMaxCh];
  const int k = blockIdx.y;
  const int64_t r0 = (int64_t)blockIdx.x * kWgChunk;
  const int nr = (int)min((int64_t)kWgChunk, n_out - r0);
  const int tid = threadIdx.x, lane = tid & 31;
  // deterministic compaction (ascending rows) by all warps: each counts the hits of its slice of the chunk, a prefix
  // over the eight counts places the slices, then each warp writes its hits
  __shared__ int s_wcnt[kWgThreads / 32];
  constexpr int kSlice = kWgChunk / (kWgThreads / 32);
  const int warp = tid >> 5;
  const int c_begin = warp * kSlice, c_end = min(nr, c_begin + kSlice);
  int cnt = 0;
  for (int c = c_begin; c < c_end; c += 32) {
    const int v = c + lane;
    const int i = v < c_end ? __ldg(nbr + (int64_t)k * n_out + r0 + v) : -1;
    cnt += __popc(__ballot_sync(0xffffffffu, i >= 0 && i < n_rows));
  }
  if (lane == 0) s_wcnt[warp] = cnt;
  __syncthreads();
  int n0 = 0;
  for (int w = 0; w < warp; ++w) n0 += s_wcnt[w];
  if (tid == 0) {
    int t = 0;
    for (int w = 0; w < kWgThreads / 32; ++w) t += s_wcnt[w];
    s_n = t;
  }
  for (int c = c_begin; c < c_end; c += 32) {
    const int v = c + lane;
    int i = v < c_end ? __ldg(nbr + (int64_t)k * n_out + r0 + v) : -1;
    if (i >= n_rows) {
      if (status) atomicOr(status, SPH_STATUS_BAD_INDEX);
      i = -1;
    }
    const unsigned m = __ballot_sync(0xffffffffu, i >= 0);
    if (i >= 0) {
      const int slot = n0 + __popc(m & ((1u << lane) - 1u));
      s_in[slot] = i;
      s_out[slot] = v;
    }
    n0 += __popc(m);
  }
  __syncthreads();
  const int n = s_n;
  if (n == 0) return;
  const int KN = K * N;
  float acc[kWgElems];
#pragma unroll
  for (int j = 0; j < kWgElems; ++j) acc[j] = 0.f;
  for (int p0 = 0; p0 < n; p0 += kWgTile) {
    const int np = min(kWgTile, n - p0);
    for (int e = tid; e < kWgTile * K; e += kWgThreads) {
      int rr = e / K, c = e % K;
      s_x[rr][c] = rr < np ? (float)to_acc(rows[(int64_t)s_in[p0 + rr] * K + c]) : 0.f;
    }
    for (int e = tid; e < kWgTile * N; e += kWgThreads) {
      int rr = e / N, c = e % N;
      s_d[rr][c] = rr < np ? (float)to_acc(dout[(r0 + s_out[p0 + rr]) * N + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kWgElems; ++j) {
      int e = tid + j * kWgThreads;
      if (e < KN) {
        int ic = e / N, oc = e % N;
        float a = acc[j];
#pragma unroll
        for (int rr = 0; rr < kWgTile; ++rr) a += s_x[rr][ic] * s_d[rr][oc];
        acc[j] = a;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < kWgElems; ++j) {
    int e = tid + j * kWgThreads;
    if (e < KN) atomicAdd(dw + (int64_t)k * KN + e, acc[j]);
  }
}

template <typename T>
int launch_generic(const void* rows, int64_t n_rows, const void* weight, const int* nbr, int64_t n_out, int kv,
                   int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                   int out_dtype, int* status, cudaStream_t st) {
  int tpr = 1;
  while (tpr * 4 < N) tpr <<= 1;
  if (tpr > kGenThreads) {
    set_error("n_ch %d too large for the CUDA-core kernel", N);
    return SPH_ERR_LIMIT;
  }
  int rows_per_block = kGenThreads / tpr;
  int64_t blocks = div_up64(n_out, rows_per_block);
  conv_gather_generic_kernel<T><<<(unsigned)blocks, kGenThreads, 0, st>>>(
      (const T*)rows, n_rows, (const T*)weight, nbr, n_out, kv, K, N, tpr, flip_k, scale, bias, relu, out,
      out_dtype, status);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

template <typename T>
int launch_wgrad(const void* rows, const void* dout, int64_t n_rows, const int* nbr, int64_t n_out, int kv, int K,
                 int N, float* dw, int* status, cudaStream_t st) {
  dim3 grid((unsigned)div_up64(n_out, kWgChunk), (unsigned)kv);
  conv_wgrad_generic_kernel<T><<<grid, kWgThreads, 0, st>>>((const T*)rows, (const T*)dout, n_rows, nbr, n_out, K,
                                                            N, dw, status);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

}  // namespace

int conv_gather_generic(const void* rows, int dtype, int64_t n_rows, const void* weight, const int* nbr,
                        int64_t n_out, int kv, int K, int N, int flip_k, const float* scale, const float* bias,
                        int relu, void* out, int out_dtype, int* status, cudaStream_t st) {
  switch (dtype) {
    case SPH_F32:
      return launch_generic<float>(rows, n_rows, weight, nbr, n_out, kv, K, N, flip_k, scale, bias, relu, out,
                                   out_dtype, status, st);
    case SPH_F16:
      return launch_generic<__half>(rows, n_rows, weight, nbr, n_out, kv, K, N, flip_k, scale, bias, relu, out,
                                    out_dtype, status, st);
    case SPH_BF16:
      return launch_generic<__nv_bfloat16>(rows, n_rows, weight, nbr, n_out, kv, K, N, flip_k, scale, bias, relu,
                                           out, out_dtype, status, st);
    case SPH_I8:
      return launch_generic<int8_t>(rows, n_rows, weight, nbr, n_out, kv, K, N, flip_k, scale, bias, relu, out,
                                    out_dtype, status, st);
  }
  set_error("unknown dtype %d", dtype);
  return SPH_ERR_INVALID;
}

int conv_wgrad_generic(const void* rows, const void* dout, int dtype, int64_t n_rows, const int* nbr,
                       int64_t n_out, int kv, int K, int N, float* dw, int* status, cudaStream_t st) {
  if (K > kWgMaxCh || N > kWgMaxCh) {
    set_error("weight gradient supports up to %d channels (got %d x %d)", kWgMaxCh, K, N);
    return SPH_ERR_LIMIT;
  }
  switch (dtype) {
    case SPH_F32: return launch_wgrad<float>(rows, dout, n_rows, nbr, n_out, kv, K, N, dw, status, st);
    case SPH_F16: return launch_wgrad<__half>(rows, dout, n_rows, nbr, n_out, kv, K, N, dw, status, st);
    case SPH_BF16: return launch_wgrad<__nv_bfloat16>(rows, dout, n_rows, nbr, n_out, kv, K, N, dw, status, st);
  }
  set_error("weight gradient is not defined for dtype %d", dtype);
  return SPH_ERR_UNSUPPORTED;
}

}  // namespace sph
