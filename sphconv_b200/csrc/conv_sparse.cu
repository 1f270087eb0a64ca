// CUDA-core kernel of the rule-driven convolution for the SPARSE levels of an encoder (few neighbours per output row,
// few channels): the first layers of a LiDAR scan have ~1.5 of 27 neighbours present per row, so a kernel that walks
// every (row, offset) slot of the table - as the tensor-core kernels do, 256 rows x all offsets per tile - spends its
// time on slots that hold nothing.  Here the work is the PRESENT pairs:
//
//   * a CTA copies the filter [KV, iC, oC] into shared memory once (as fp32, or as 16-bit values when it is large); its
//     warps then take chunks of 32 consecutive output rows.  A lane reads its row's table entries eight offsets at a
//     time (one coalesced 128-byte load per offset), the next eight requested before the current ones are looked at;
//   * the warp walks the offsets and compacts the present entries into a list of (input row, output row in the chunk,
//     weight index) with a ballot + prefix popcount;
//   * whenever 32 items are listed, each lane fetches ONE item's input row (32 independent loads in flight per warp
//     instruction), widens it to fp32 and stages it in shared memory;
//   * the items are then multiplied oC/4 lanes per item (four output channels per lane) and added to the warp's fp32
//     accumulator tile [32 rows x oC] in shared memory.  Two items of one pass can name the same output row
//     (consecutive offsets); `match.any` finds them and those few passes add in turns;
//   * after the last offset the lane that owns a row applies relu(acc*scale + bias), converts and stores it with
//     16-byte stores, and clears its accumulator row.
//
// No scatter and no atomic: the output is written once, like in the other forward kernels (the reference scatters with a
// read-modify-write per 8 pairs, include/sphconv/iterator.cu.h:1467-1625).
#include "common.cuh"

#include <type_traits>

namespace sph {

namespace {

constexpr int kSpWarps = 8;
constexpr int kSpThreads = kSpWarps * 32;
constexpr int kSpList = 64;          // an offset adds at most 32 items to fewer than 32 waiting ones

struct SparseParams {
  const void* rows;
  const void* weight;                // [KV, IC, OC] in the rows' dtype
  const int* nbr;                    // [KV, n_out]
  int64_t n_rows, n_out, n_chunks;
  int kv, flip_k, relu, out_dtype;
  const float* scale;
  const float* bias;
  void* out;
  int* status;
};

template <typename T> __device__ __forceinline__ float2 pair_to_float2(const T* p);
template <> __device__ __forceinline__ float2 pair_to_float2<__half>(const __half* p) {
  return __half22float2(*(const __half2*)p);
}
template <> __device__ __forceinline__ float2 pair_to_float2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*(const __nv_bfloat162*)p);
}
template <> __device__ __forceinline__ float2 pair_to_float2<float>(const float* p) { return *(const float2*)p; }
template <> __device__ __forceinline__ float2 pair_to_float2<int8_t>(const int8_t* p) {
  const char2 v = *(const char2*)p;
  return make_float2((float)v.x, (float)v.y);
}

// Four consecutive filter weights as floats (the filter sits in shared memory as fp32, or as 16-bit values when it is large).
template <typename W> __device__ __forceinline__ float4 quad_to_float4(const W* p);
template <> __device__ __forceinline__ float4 quad_to_float4<float>(const float* p) { return *(const float4*)p; }
template <> __device__ __forceinline__ float4 quad_to_float4<__half>(const __half* p) {
  const uint2 raw = *(const uint2*)p;
  const float2 a = __half22float2(*(const __half2*)&raw.x), b = __half22float2(*(const __half2*)&raw.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <> __device__ __forceinline__ float4 quad_to_float4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *(const uint2*)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162*)&raw.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename W> __device__ __forceinline__ void store_pair(W* p, float2 v);
template <> __device__ __forceinline__ void store_pair<float>(float* p, float2 v) { *(float2*)p = v; }
template <> __device__ __forceinline__ void store_pair<__half>(__half* p, float2 v) { *(__half2*)p = __floats2half2_rn(v.x, v.y); }
template <> __device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float2 v) {
  *(__nv_bfloat162*)p = __floats2bfloat162_rn(v.x, v.y);
}

// One input row (IC elements of T) -> IC floats in shared memory.
template <typename T, int IC>
__device__ __forceinline__ void stage_row(const T* __restrict__ src, float* __restrict__ dst) {
  constexpr int BYTES = IC * (int)sizeof(T);
  if constexpr (sizeof(T) == 1) {
    uint32_t raw[BYTES / 4];
    if constexpr (BYTES == 4) {
      raw[0] = __ldg((const uint32_t*)src);
    } else if constexpr (BYTES == 8) {
      const uint2 v = __ldg((const uint2*)src);
      raw[0] = v.x; raw[1] = v.y;
    } else {
#pragma unroll
      for (int q = 0; q < BYTES / 16; ++q) {
        const uint4 v = __ldg((const uint4*)src + q);
        raw[4 * q] = v.x; raw[4 * q + 1] = v.y; raw[4 * q + 2] = v.z; raw[4 * q + 3] = v.w;
      }
    }
#pragma unroll
    for (int q = 0; q < BYTES / 4; ++q) {
      const uint32_t w = raw[q];
      *(float4*)(dst + 4 * q) = make_float4((float)(int8_t)(w & 0xffu), (float)(int8_t)((w >> 8) & 0xffu),
                                            (float)(int8_t)((w >> 16) & 0xffu), (float)(int8_t)(w >> 24));
    }
  } else if constexpr (BYTES == 8) {
    const uint2 raw = __ldg((const uint2*)src);
    const T* e = (const T*)&raw;
    const float2 a = pair_to_float2<T>(e), b = pair_to_float2<T>(e + 2);
    *(float4*)dst = make_float4(a.x, a.y, b.x, b.y);
  } else {
    constexpr int PER = 16 / (int)sizeof(T);     // elements per 16-byte load
    uint4 raw[BYTES / 16];
#pragma unroll
    for (int q = 0; q < BYTES / 16; ++q) raw[q] = __ldg((const uint4*)src + q);
#pragma unroll
    for (int q = 0; q < BYTES / 16; ++q) {
      const T* e = (const T*)&raw[q];
#pragma unroll
      for (int j = 0; j < PER; j += 4) {
        const float2 a = pair_to_float2<T>(e + j), b = pair_to_float2<T>(e + j + 2);
        *(float4*)(dst + q * PER + j) = make_float4(a.x, a.y, b.x, b.y);
      }
    }
  }
}

// G consecutive channels of one output row, converted and stored with one or two vector stores.
template <int G>
__device__ __forceinline__ void store_group(void* out, int out_dtype, int64_t elem, const float* v) {
  if (out_dtype == SPH_F32) {
#pragma unroll
    for (int j = 0; j < G; j += 4) *(float4*)((float*)out + elem + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
  } else if (out_dtype == SPH_I8) {   // round to nearest, saturate at +-127
    uint32_t w[G / 4];
#pragma unroll
    for (int j = 0; j < G; j += 4) {
      uint32_t acc = 0;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int q = (int)fminf(fmaxf(rintf(v[j + t]), -127.f), 127.f);
        acc |= ((uint32_t)q & 0xffu) << (8 * t);
      }
      w[j / 4] = acc;
    }
    uint8_t* dst = (uint8_t*)out + elem;
    if constexpr (G == 8) *(uint2*)dst = make_uint2(w[0], w[1]);
    else *(uint32_t*)dst = w[0];
  } else {
    uint32_t w[G / 2];
#pragma unroll
    for (int j = 0; j < G; j += 2) {
      if (out_dtype == SPH_F16) {
        const __half2 h = __floats2half2_rn(v[j], v[j + 1]);
        w[j / 2] = *(const uint32_t*)&h;
      } else {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[j], v[j + 1]);
        w[j / 2] = *(const uint32_t*)&h;
      }
    }
    uint16_t* dst = (uint16_t*)out + elem;
    if constexpr (G == 8) *(uint4*)dst = make_uint4(w[0], w[1], w[2], w[3]);
    else *(uint2*)dst = make_uint2(w[0], w[1]);
  }
}

constexpr int kSpGroup = 8;          // table offsets a lane looks at per step; the next step's are in flight meanwhile
constexpr int kSpWPad = 16;          // floats between the filters of two offsets: neighbouring offsets on other banks

// The filter in shared memory: fp32 when an offset has at most 256 weights (no conversions in the inner loop), else 16-bit
// (the rows' own type; int8 weights as fp16, which holds them exactly) so that two CTAs still share a multiprocessor.
template <typename T, bool Large> struct FilterType { using type = float; };
template <> struct FilterType<__half, true> { using type = __half; };
template <> struct FilterType<__nv_bfloat16, true> { using type = __nv_bfloat16; };
template <> struct FilterType<int8_t, true> { using type = __half; };

template <typename T, int IC, int OC> struct SparseShape {
  using W = typename FilterType<T, (IC * OC > 256)>::type;
  static constexpr int XS = IC + 4;            // staged row stride in floats: 16-byte stores of 8 lanes hit 8 bank groups
  static constexpr int AS = OC + 4;            // accumulator row stride in floats
  static constexpr int WS = IC * OC + kSpWPad; // filter stride of an offset in elements
  static constexpr int WARP_BYTES = 32 * XS * 4 + 32 * AS * 4 + kSpList * 8;
  static int smem_bytes(int kv) { return kv * WS * (int)sizeof(W) + 2 * OC * 4 + kSpWarps * WARP_BYTES; }
};

// Multiplies the first n listed items (n <= 32) of the warp into its accumulator tile.  `wb` is the warp's region of
// shared memory: stage [32][XS] floats, acc [32][AS] floats, list_i [kSpList], list_rk [kSpList].
// OC/4 lanes work on one item, four output channels each: a step of four input channels is one 16-byte read of the
// staged row, four 16-byte reads of the filter and 16 FMAs.
template <typename T, int IC, int OC>
__device__ __noinline__ void sparse_flush(const T* __restrict__ rows, const typename SparseShape<T, IC, OC>::W* sW,
                                          unsigned char* wb, int n) {
  using S = SparseShape<T, IC, OC>;
  using W = typename S::W;
  constexpr int LPI = OC / 4;                  // lanes per item
  constexpr int IPP = 32 / LPI;                // items per pass
  constexpr int XS = S::XS, AS = S::AS;
  const int lane = threadIdx.x & 31;
  float* stage = (float*)wb;
  float* acc = stage + 32 * XS;
  const int* list_i = (const int*)(acc + 32 * AS);
  const int* list_rk = list_i + kSpList;
  const int grp = lane / LPI, cl = lane % LPI;
  const unsigned grp_mask = (LPI == 32 ? 0xffffffffu : ((1u << LPI) - 1u)) << (grp * LPI);
  const unsigned below_grp = (1u << (grp * LPI)) - 1u;

  if (lane < n) stage_row<T, IC>(rows + (int64_t)list_i[lane] * IC, stage + lane * XS);
  __syncwarp();
  for (int p0 = 0; p0 < n; p0 += IPP) {
    const int it = p0 + grp;
    const bool valid = it < n;
    const int rk = valid ? list_rk[it] : 0;
    const int r = rk & 31;
    const float* x = stage + (valid ? it : 0) * XS;
    const W* w = sW + (rk >> 5) * S::WS + 4 * cl;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < IC; j += 4) {
      const float4 xv = *(const float4*)(x + j);
      const float4 w0 = quad_to_float4<W>(w + (j + 0) * OC), w1 = quad_to_float4<W>(w + (j + 1) * OC);
      const float4 w2 = quad_to_float4<W>(w + (j + 2) * OC), w3 = quad_to_float4<W>(w + (j + 3) * OC);
      s.x = fmaf(xv.x, w0.x, s.x); s.y = fmaf(xv.x, w0.y, s.y); s.z = fmaf(xv.x, w0.z, s.z); s.w = fmaf(xv.x, w0.w, s.w);
      s.x = fmaf(xv.y, w1.x, s.x); s.y = fmaf(xv.y, w1.y, s.y); s.z = fmaf(xv.y, w1.z, s.z); s.w = fmaf(xv.y, w1.w, s.w);
      s.x = fmaf(xv.z, w2.x, s.x); s.y = fmaf(xv.z, w2.y, s.y); s.z = fmaf(xv.z, w2.z, s.z); s.w = fmaf(xv.z, w2.w, s.w);
      s.x = fmaf(xv.w, w3.x, s.x); s.y = fmaf(xv.w, w3.y, s.y); s.z = fmaf(xv.w, w3.z, s.z); s.w = fmaf(xv.w, w3.w, s.w);
    }
    float4* a = (float4*)(acc + r * AS + 4 * cl);
    // items of one pass that name the same output row add in turns (ascending item), the others at once
    const unsigned others = __match_any_sync(0xffffffffu, valid ? r : 32 + grp) & ~grp_mask;
    if (__any_sync(0xffffffffu, others != 0u)) {
      const int turn = __popc(others & below_grp) / LPI;
      const int turns = __reduce_max_sync(0xffffffffu, valid ? turn : 0) + 1;
      for (int t = 0; t < turns; ++t) {
        if (valid && turn == t) { float4 v = *a; v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w; *a = v; }
        __syncwarp();
      }
    } else if (valid) {
      float4 v = *a; v.x += s.x; v.y += s.y; v.z += s.z; v.w += s.w; *a = v;
    }
  }
  __syncwarp();
}

template <typename T, int IC, int OC>
__global__ void __launch_bounds__(kSpThreads, 4) conv_sparse_rows_kernel(SparseParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  using S = SparseShape<T, IC, OC>;
  constexpr int AS = S::AS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  using W = typename S::W;
  W* sW = (W*)smem;                                              // [kv][WS]: the filter
  float* s_epi = (float*)(sW + p.kv * S::WS);                    // scale[OC], bias[OC]
  unsigned char* wb = (unsigned char*)(s_epi + 2 * OC) + warp * S::WARP_BYTES;
  float* acc = (float*)wb + 32 * S::XS;                          // [32][AS]
  int* list_i = (int*)(acc + 32 * AS);                           // [kSpList] input row
  int* list_rk = list_i + kSpList;                               // [kSpList] row in the chunk | weight index << 5

  {
    const T* gw = (const T*)p.weight;
    const int w_elems = p.kv * IC * OC;
    for (int e = threadIdx.x * 2; e < w_elems; e += kSpThreads * 2) {
      const int k = e / (IC * OC);
      store_pair<W>(sW + k * S::WS + (e - k * (IC * OC)), pair_to_float2<T>(gw + e));
    }
  }
  for (int c = threadIdx.x; c < OC; c += kSpThreads) {
    s_epi[c] = p.scale ? __ldg(p.scale + c) : 1.f;
    s_epi[OC + c] = p.bias ? __ldg(p.bias + c) : 0.f;
  }
  for (int e = lane; e < 32 * AS; e += 32) acc[e] = 0.f;
  __syncthreads();

  const T* rows = (const T*)p.rows;
  const unsigned lane_lt = (1u << lane) - 1u;
  const int64_t warps_total = (int64_t)gridDim.x * kSpWarps;
  for (int64_t ch = (int64_t)blockIdx.x * kSpWarps + warp; ch < p.n_chunks; ch += warps_total) {
    const int64_t o = ch * 32 + lane;
    const bool row_ok = o < p.n_out;
    const int* col = p.nbr + o;
    int cnt = 0;
    // the row's entries, kSpGroup offsets at a time, the next group requested before this one is looked at
    int ahead[kSpGroup];
#pragma unroll
    for (int u = 0; u < kSpGroup; ++u) ahead[u] = (row_ok && u < p.kv) ? __ldg(col + (int64_t)u * p.n_out) : -1;
#pragma unroll 1
    for (int k0 = 0; k0 < p.kv; k0 += kSpGroup) {
      int v[kSpGroup];
#pragma unroll
      for (int u = 0; u < kSpGroup; ++u) {
        v[u] = ahead[u];
        const int kk = k0 + kSpGroup + u;
        ahead[u] = (row_ok && kk < p.kv) ? __ldg(col + (int64_t)kk * p.n_out) : -1;
      }
#pragma unroll
      for (int u = 0; u < kSpGroup; ++u) {
        int i = v[u];
        if (i >= p.n_rows) {
          if (p.status) atomicOr(p.status, SPH_STATUS_BAD_INDEX);
          i = -1;
        }
        const unsigned m = __ballot_sync(0xffffffffu, i >= 0);
        if (m == 0u) continue;
        const int tk = k0 + u;
        if (i >= 0) {
          const int pos = cnt + __popc(m & lane_lt);
          list_i[pos] = i;
          list_rk[pos] = lane | ((p.flip_k ? p.kv - 1 - tk : tk) << 5);
        }
        cnt += __popc(m);
        if (cnt >= 32) {
          __syncwarp();
          sparse_flush<T, IC, OC>(rows, sW, wb, 32);
          // the items behind the first 32 move to the front
          const int rem = cnt - 32;
          int ti = 0, trk = 0;
          if (lane < rem) { ti = list_i[32 + lane]; trk = list_rk[32 + lane]; }
          __syncwarp();
          if (lane < rem) { list_i[lane] = ti; list_rk[lane] = trk; }
          cnt = rem;
        }
      }
    }
    if (cnt) {
      __syncwarp();
      sparse_flush<T, IC, OC>(rows, sW, wb, cnt);
    }
    __syncwarp();
    // epilogue: the lane owns row `lane` of the tile, and clears it for the next chunk
    float* a = acc + lane * AS;
    constexpr int G = OC >= 8 ? 8 : 4;
#pragma unroll
    for (int c0 = 0; c0 < OC; c0 += G) {
      float vals[G];
#pragma unroll
      for (int j = 0; j < G; j += 4) {
        const float4 t = *(const float4*)(a + c0 + j);
        vals[j] = t.x; vals[j + 1] = t.y; vals[j + 2] = t.z; vals[j + 3] = t.w;
        *(float4*)(a + c0 + j) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < G; ++j) {
        const float t = fmaf(vals[j], s_epi[c0 + j], s_epi[OC + c0 + j]);
        vals[j] = p.relu ? fmaxf(t, 0.f) : t;
      }
      if (row_ok) store_group<G>(p.out, p.out_dtype, o * OC + c0, vals);
    }
    __syncwarp();
  }
}

template <typename T, int IC, int OC>
int launch_sparse(const SparseParams& p, cudaStream_t st) {
  using S = SparseShape<T, IC, OC>;
  const int smem = S::smem_bytes(p.kv);
  auto kern = conv_sparse_rows_kernel<T, IC, OC>;
  if (smem > 48 * 1024) SPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 0;
  SPH_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kSpThreads, smem));
  const int sms = current_sm_count();
  if (sms <= 0 || per_sm <= 0) {
    set_error("conv_gather_sparse: the kernel does not fit on a multiprocessor");
    return SPH_ERR_CUDA;
  }
  const int64_t want = div_up64(p.n_chunks, kSpWarps);
  const int64_t grid = want < (int64_t)sms * per_sm ? want : (int64_t)sms * per_sm;
  kern<<<(unsigned)grid, kSpThreads, smem, st>>>(p);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

template <typename T, int IC>
int launch_sparse_oc(const SparseParams& p, int N, cudaStream_t st) {
  switch (N) {
    case 4: return launch_sparse<T, IC, 4>(p, st);
    case 8: return launch_sparse<T, IC, 8>(p, st);
    case 16: return launch_sparse<T, IC, 16>(p, st);
    case 32: return launch_sparse<T, IC, 32>(p, st);
  }
  return SPH_ERR_UNSUPPORTED;
}

template <typename T>
int launch_sparse_ic(const SparseParams& p, int K, int N, cudaStream_t st) {
  switch (K) {
    case 4: return launch_sparse_oc<T, 4>(p, N, st);
    case 8: return launch_sparse_oc<T, 8>(p, N, st);
    case 16: return launch_sparse_oc<T, 16>(p, N, st);
    case 32: return launch_sparse_oc<T, 32>(p, N, st);
  }
  return SPH_ERR_UNSUPPORTED;
}

bool channels_ok(int c) { return c == 4 || c == 8 || c == 16 || c == 32; }

// ---- weight gradient of the same narrow, sparse layers --------------------------------------------------------------
//   dW[k] += x[i,:]^T dY[o,:]   over the present pairs (i, o) of offset k
// Same walk as the forward kernel: a warp takes 32 consecutive output rows, stages their dY rows once, lists the present
// (input row, row in the chunk, offset) items offset by offset, fetches 32 input rows at a time and then goes through the
// items one after the other with the lanes spread over the iC x oC elements of the product.  The list is offset-major,
// so a lane's running sums belong to one offset at a time and are added to the CTA's copy of dW (shared memory) when the
// offset changes; the CTA adds its copy to the fp32 gradient in global memory once, at the end.
struct WgradParams {
  const void* rows;                  // [n_rows, IC]
  const void* dout;                  // [n_out, OC]
  const int* nbr;                    // [KV, n_out]
  int64_t n_rows, n_out, n_chunks;
  int kv;
  float* dw;                         // [KV, IC, OC], accumulated into
  int* status;
};

template <int IC, int OC> struct WgradShape {
  static constexpr int E = IC * OC;                      // elements of one offset's gradient
  static constexpr int EPL = (E + 31) / 32;              // elements per lane
  static constexpr int XS = IC + 4, DS = OC + 4;         // staged row strides in floats
  static constexpr int WARP_BYTES = 32 * XS * 4 + 32 * DS * 4 + kSpList * 8;
  static int smem_bytes(int kv) { return kv * E * 4 + kSpWarps * WARP_BYTES; }
};

template <typename T, int IC, int OC>
__global__ void __launch_bounds__(kSpThreads, 3) conv_wgrad_pairs_kernel(WgradParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  using S = WgradShape<IC, OC>;
  constexpr int E = S::E, EPL = S::EPL, XS = S::XS, DS = S::DS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* s_dw = (float*)smem;                                    // [kv][E]
  unsigned char* wb = (unsigned char*)(s_dw + p.kv * E) + warp * S::WARP_BYTES;
  float* stage = (float*)wb;                                     // [32][XS]: input rows of the listed items
  float* dys = stage + 32 * XS;                                  // [32][DS]: dY rows of the chunk
  int* list_i = (int*)(dys + 32 * DS);
  int* list_rk = list_i + kSpList;

  for (int e = threadIdx.x; e < p.kv * E; e += kSpThreads) s_dw[e] = 0.f;
  __syncthreads();

  const T* rows = (const T*)p.rows;
  const T* dout = (const T*)p.dout;
  const unsigned lane_lt = (1u << lane) - 1u;
  int ic_of[EPL], oc_of[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const int e = lane + 32 * j;
    ic_of[j] = (e / OC) % IC;                                    // lanes beyond E (E < 32) repeat an element and skip the add
    oc_of[j] = e % OC;
  }
  float acc[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) acc[j] = 0.f;
  int cur_k = 0;

  // Adds the running sums to the CTA's gradient of offset cur_k.
  auto spill = [&]() {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = lane + 32 * j;
      if (e < E && acc[j] != 0.f) atomicAdd(s_dw + cur_k * E + e, acc[j]);
      acc[j] = 0.f;
    }
  };
  // The first n listed items: fetch their input rows, then one item after the other.
  auto flush = [&](int n) {
    if (lane < n) stage_row<T, IC>(rows + (int64_t)list_i[lane] * IC, stage + lane * XS);
    __syncwarp();
    for (int it = 0; it < n; ++it) {
      const int rk = list_rk[it];
      const int k = rk >> 5;
      if (k != cur_k) {                                          // uniform: the list is offset-major
        spill();
        cur_k = k;
      }
      const float* x = stage + it * XS;
      const float* d = dys + (rk & 31) * DS;
#pragma unroll
      for (int j = 0; j < EPL; ++j) acc[j] = fmaf(x[ic_of[j]], d[oc_of[j]], acc[j]);
    }
    __syncwarp();
  };

  const int64_t warps_total = (int64_t)gridDim.x * kSpWarps;
  for (int64_t ch = (int64_t)blockIdx.x * kSpWarps + warp; ch < p.n_chunks; ch += warps_total) {
    const int64_t o = ch * 32 + lane;
    const bool row_ok = o < p.n_out;
    const int* col = p.nbr + o;
    __syncwarp();                                                // the previous chunk's items are done with dys
    if (row_ok) stage_row<T, OC>(dout + o * OC, dys + lane * DS);
    int cnt = 0;
    int ahead[kSpGroup];
#pragma unroll
    for (int u = 0; u < kSpGroup; ++u) ahead[u] = (row_ok && u < p.kv) ? __ldg(col + (int64_t)u * p.n_out) : -1;
    __syncwarp();
#pragma unroll 1
    for (int k0 = 0; k0 < p.kv; k0 += kSpGroup) {
      int v[kSpGroup];
#pragma unroll
      for (int u = 0; u < kSpGroup; ++u) {
        v[u] = ahead[u];
        const int kk = k0 + kSpGroup + u;
        ahead[u] = (row_ok && kk < p.kv) ? __ldg(col + (int64_t)kk * p.n_out) : -1;
      }
#pragma unroll
      for (int u = 0; u < kSpGroup; ++u) {
        int i = v[u];
        if (i >= p.n_rows) {
          if (p.status) atomicOr(p.status, SPH_STATUS_BAD_INDEX);
          i = -1;
        }
        const unsigned m = __ballot_sync(0xffffffffu, i >= 0);
        if (m == 0u) continue;
        if (i >= 0) {
          const int pos = cnt + __popc(m & lane_lt);
          list_i[pos] = i;
          list_rk[pos] = lane | ((k0 + u) << 5);
        }
        cnt += __popc(m);
        if (cnt >= 32) {
          __syncwarp();
          flush(32);
          const int rem = cnt - 32;
          int ti = 0, trk = 0;
          if (lane < rem) { ti = list_i[32 + lane]; trk = list_rk[32 + lane]; }
          __syncwarp();
          if (lane < rem) { list_i[lane] = ti; list_rk[lane] = trk; }
          cnt = rem;
        }
      }
    }
    if (cnt) {
      __syncwarp();
      flush(cnt);
    }
  }
  spill();
  __syncthreads();
  for (int e = threadIdx.x; e < p.kv * E; e += kSpThreads) {
    const float v = s_dw[e];
    if (v != 0.f) atomicAdd(p.dw + e, v);
  }
}

template <typename T, int IC, int OC>
int launch_wgrad_pairs(const WgradParams& p, cudaStream_t st) {
  using S = WgradShape<IC, OC>;
  const int smem = S::smem_bytes(p.kv);
  auto kern = conv_wgrad_pairs_kernel<T, IC, OC>;
  if (smem > 48 * 1024) SPH_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 0;
  SPH_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kSpThreads, smem));
  const int sms = current_sm_count();
  if (sms <= 0 || per_sm <= 0) {
    set_error("conv_wgrad_pairs: the kernel does not fit on a multiprocessor");
    return SPH_ERR_CUDA;
  }
  const int64_t want = div_up64(p.n_chunks, kSpWarps);
  const int64_t grid = want < (int64_t)sms * per_sm ? want : (int64_t)sms * per_sm;
  kern<<<(unsigned)grid, kSpThreads, smem, st>>>(p);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

template <typename T, int IC>
int launch_wgrad_pairs_oc(const WgradParams& p, int N, cudaStream_t st) {
  switch (N) {
    case 4: return launch_wgrad_pairs<T, IC, 4>(p, st);
    case 8: return launch_wgrad_pairs<T, IC, 8>(p, st);
    case 16: return launch_wgrad_pairs<T, IC, 16>(p, st);
    case 32: return launch_wgrad_pairs<T, IC, 32>(p, st);
  }
  return SPH_ERR_UNSUPPORTED;
}

template <typename T>
int launch_wgrad_pairs_ic(const WgradParams& p, int K, int N, cudaStream_t st) {
  switch (K) {
    case 4: return launch_wgrad_pairs_oc<T, 4>(p, N, st);
    case 8: return launch_wgrad_pairs_oc<T, 8>(p, N, st);
    case 16: return launch_wgrad_pairs_oc<T, 16>(p, N, st);
    case 32: return launch_wgrad_pairs_oc<T, 32>(p, N, st);
  }
  return SPH_ERR_UNSUPPORTED;
}


}  // namespace

// Shapes the kernel takes: fp32 / fp16 / bf16 / int8 rows of 4, 8, 16 or 32 channels in and out, the whole filter (plus
// the warps' tiles) within 112 KB of shared memory so that at least two CTAs share a multiprocessor.  int8 products are
// summed in fp32, which is exact while every partial sum stays below 2^24: KV * K * 127^2 must.
bool conv_sparse_supported(int dtype, int kv, int K, int N) {
  if (dtype != SPH_F32 && dtype != SPH_F16 && dtype != SPH_BF16 && dtype != SPH_I8) return false;
  if (!channels_ok(K) || !channels_ok(N)) return false;
  if (dtype == SPH_I8 && (int64_t)kv * K * 16129 >= (1 << 24)) return false;
  const int w_size = (K * N > 256 && dtype != SPH_F32) ? 2 : 4;
  const int64_t smem = (int64_t)kv * (K * N + kSpWPad) * w_size + 2 * N * 4 +
                       (int64_t)kSpWarps * (32 * (K + 4) * 4 + 32 * (N + 4) * 4 + kSpList * 8);
  return kv < (1 << 20) && smem <= 112 * 1024;
}

int conv_gather_sparse(const void* rows, int dtype, int64_t n_rows, const void* weight, const int* nbr, int64_t n_out,
                       int kv, int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                       int out_dtype, int* status, cudaStream_t st) {
  if (!conv_sparse_supported(dtype, kv, K, N) || (out_dtype == SPH_I8 && dtype != SPH_I8)) {
    set_error("conv_gather_sparse: unsupported dtype/shape");
    return SPH_ERR_UNSUPPORTED;
  }
  if (((uintptr_t)rows | (uintptr_t)weight | (uintptr_t)out) & 15u) {
    set_error("conv_gather_sparse: rows, weight and out must be 16-byte aligned");
    return SPH_ERR_INVALID;
  }
  SparseParams p;
  p.rows = rows; p.weight = weight; p.nbr = nbr;
  p.n_rows = n_rows; p.n_out = n_out; p.n_chunks = div_up64(n_out, 32);
  p.kv = kv; p.flip_k = flip_k; p.relu = relu; p.out_dtype = out_dtype;
  p.scale = scale; p.bias = bias; p.out = out; p.status = status;
  switch (dtype) {
    case SPH_F32: return launch_sparse_ic<float>(p, K, N, st);
    case SPH_F16: return launch_sparse_ic<__half>(p, K, N, st);
    case SPH_BF16: return launch_sparse_ic<__nv_bfloat16>(p, K, N, st);
    case SPH_I8: return launch_sparse_ic<int8_t>(p, K, N, st);
  }
  return SPH_ERR_UNSUPPORTED;
}

// Weight gradient by the pair-compacting walk: fp32 / fp16 / bf16 rows of 4, 8, 16 or 32 channels on both sides, at
// most 512 elements per offset, the CTA's copy of the gradient plus the warps' tiles within 120 KB of shared memory.
bool conv_wgrad_pairs_supported(int dtype, int kv, int K, int N) {
  if (dtype != SPH_F32 && dtype != SPH_F16 && dtype != SPH_BF16) return false;
  if (!channels_ok(K) || !channels_ok(N) || K * N > 512) return false;
  const int64_t smem = (int64_t)kv * K * N * 4 + (int64_t)kSpWarps * (32 * (K + 4) * 4 + 32 * (N + 4) * 4 + kSpList * 8);
  return kv < (1 << 20) && smem <= 120 * 1024;
}

int conv_wgrad_pairs(const void* rows, const void* dout, int dtype, int64_t n_rows, const int* nbr, int64_t n_out,
                     int kv, int K, int N, float* dw, int* status, cudaStream_t st) {
  if (!conv_wgrad_pairs_supported(dtype, kv, K, N)) {
    set_error("conv_wgrad_pairs: unsupported dtype/shape");
    return SPH_ERR_UNSUPPORTED;
  }
  if (((uintptr_t)rows | (uintptr_t)dout) & 15u) {
    set_error("conv_wgrad_pairs: rows and dout must be 16-byte aligned");
    return SPH_ERR_INVALID;
  }
  WgradParams p;
  p.rows = rows; p.dout = dout; p.nbr = nbr;
  p.n_rows = n_rows; p.n_out = n_out; p.n_chunks = div_up64(n_out, 32);
  p.kv = kv; p.dw = dw; p.status = status;
  switch (dtype) {
    case SPH_F32: return launch_wgrad_pairs_ic<float>(p, K, N, st);
    case SPH_F16: return launch_wgrad_pairs_ic<__half>(p, K, N, st);
    case SPH_BF16: return launch_wgrad_pairs_ic<__nv_bfloat16>(p, K, N, st);
  }
  return SPH_ERR_UNSUPPORTED;
}

}  // namespace sph
