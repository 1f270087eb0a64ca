// Output-stationary gather-GEMM on the Blackwell tensor cores (tcgen05 + TMEM).
//
//   out[r,:] = epilogue( sum_k rows[nbr[k][r], :] @ W[k] )          r in [0, n_out)
//
// A CTA owns 128 consecutive output rows at a time (UMMA M = 128) and is persistent over row blocks.
// For every kernel offset k it builds the A operand [128 x K_ch] by gathering the neighbour rows with
// 16-byte cp.async copies straight into the UMMA core-matrix layout (absent neighbours are zero-filled
// without touching memory), multiplies by W[k] ([N_ch x K_ch], K-major, pre-packed) and accumulates in
// TMEM; after the last offset four epilogue warps read the accumulator back, apply scale/bias/ReLU and
// store whole rows.  There is no scatter, no atomic and the output is written exactly once
// (the reference does a read-modify-write of the output per 8 pairs, include/sphconv/iterator.cu.h:1467-1625,
// driven by the per-tile loop of include/sphconv/rule_conv_kernel.cu.h:91-153).
//
// Warp roles (288 threads): warps 0-3 gather, warp 4 issues the MMAs (one thread) and owns TMEM,
// warps 5-8 run the epilogue.  Stages are handed over with mbarriers; the accumulator is double
// buffered in TMEM so the epilogue of block i overlaps the MMAs of block i+1.
//
// Shared-memory operand layout (no swizzle): 8-row x 16-byte core matrices of 128 contiguous bytes;
// A: core (row group g, chunk c) at c*2048 + g*128; B: core (channel group gn, chunk c) at c*(N/8)*128 + gn*128.
#include <stdlib.h>

#include "common.cuh"
#include "tc_common.cuh"

namespace sph {

namespace {

using namespace tc;

constexpr int kTcMaxKV = 32;       // kernel volume the tensor-core kernel handles (3x3x3 = 27)
constexpr int kTcThreads = 288;
constexpr int kProducerThreads = 128;
constexpr int kBlockRows = 128;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 227 * 1024 - 2048 - 4 * kTcMaxKV * 32 * 4;   // minus barriers and the table buffer

struct TcParams {
  const void* rows;
  const void* packed;   // [KV][N_ch x K_ch] UMMA images
  const int* nbr;       // [KV][n_out]
  int64_t n_rows, n_out;
  int kv, K, N;         // channels gathered / produced
  int row_bytes;        // K * elem bytes
  int kc;               // 16-byte chunks per gathered row
  int stages;
  int w_resident;       // all KV weight images live in shared memory
  int a_bytes, b_bytes; // per-offset operand bytes
  int flip_k;
  int is_i8, is_bf16;
  const float* scale;
  const float* bias;
  int relu;
  void* out;
  int out_dtype;
  int* status;
  int tmem_cols;
  int num_blocks;
  int gk;               // kernel offsets gathered per pipeline stage
};

__device__ __forceinline__ void store16(void* out, int out_dtype, int64_t elem_idx, const float (&v)[16]) {
  switch (out_dtype) {
    case SPH_F32: {
      float4* p = (float4*)((float*)out + elem_idx);
#pragma unroll
      for (int j = 0; j < 4; ++j) p[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      break;
    }
    case SPH_F16: {
      uint4* p = (uint4*)((__half*)out + elem_idx);
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *(uint32_t*)&h;
      }
      p[0] = make_uint4(w[0], w[1], w[2], w[3]);
      p[1] = make_uint4(w[4], w[5], w[6], w[7]);
      break;
    }
    case SPH_BF16: {
      uint4* p = (uint4*)((__nv_bfloat16*)out + elem_idx);
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        w[j] = *(uint32_t*)&h;
      }
      p[0] = make_uint4(w[0], w[1], w[2], w[3]);
      p[1] = make_uint4(w[4], w[5], w[6], w[7]);
      break;
    }
    default: {
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t acc = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          float r = fminf(fmaxf(rintf(v[4 * j + b]), -127.f), 127.f);
          acc |= ((uint32_t)(int)r & 0xffu) << (8 * b);
        }
        w[j] = acc;
      }
      *(uint4*)((int8_t*)out + elem_idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

__global__ void __launch_bounds__(kTcThreads, 1) conv_gather_tc_kernel(TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ __align__(8) uint64_t s_w_full;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_tbl[4][kTcMaxKV][32];   // per producer warp: neighbour-table entries of the current row block

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int S = p.stages;
  const int GK = p.gk;                                             // kernel offsets per pipeline stage
  const int stage_bytes = GK * (p.a_bytes + (p.w_resident ? 0 : p.b_bytes));
  uint8_t* w_smem = smem;                                          // resident weights (if any)
  uint8_t* stage0 = smem + (p.w_resident ? p.kv * p.b_bytes : 0);  // multiple of 128 bytes either way
  const int groups = (p.kv + GK - 1) / GK;                         // stages per row block

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&s_full[s]), kProducerThreads + (p.w_resident ? 0 : 1));
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_acc_full[b]), 1);
      mbar_init(smem_u32(&s_acc_empty[b]), 4);
    }
    mbar_init(smem_u32(&s_w_full), 1);
    mbar_init_fence();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&s_tmem_base), (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  // blocks handled by this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const int my_blocks = (p.num_blocks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (warp < 4) {
    // ======================= gather producers =======================
    // Lane <-> output row (32*warp + lane of the block).  The per-stage instruction stream of a producer
    // warp is the pipeline's critical path, so it is kept to: one barrier poll, one shared-memory read
    // of the neighbour row id, kc 16-byte cp.async per offset, one arrive.  The neighbour-table entries
    // of the NEXT block are loaded into registers while the current block is gathered and parked in
    // shared memory at the block boundary, so no global-load latency sits on that path.
    if (p.w_resident && tid == 0) {
      const uint32_t bytes = (uint32_t)(p.kv * p.b_bytes);
      mbar_arrive_expect_tx(smem_u32(&s_w_full), bytes);
      // one bulk copy per offset keeps each transfer well under the mbarrier tx-count limit
      for (int k = 0; k < p.kv; ++k)
        bulk_g2s(smem_u32(w_smem + (size_t)k * p.b_bytes), (const uint8_t*)p.packed + (size_t)k * p.b_bytes,
                 (uint32_t)p.b_bytes, smem_u32(&s_w_full));
    }
    const uint8_t* rows = (const uint8_t*)p.rows;
    int* tbl = &s_tbl[warp][0][lane];   // entry of offset k at tbl[k * 32]
    int tmp[kTcMaxKV];
    auto load_table = [&](int blk) {
      const int64_t r = (int64_t)blk * kBlockRows + warp * 32 + lane;
#pragma unroll
      for (int k = 0; k < kTcMaxKV; ++k) {
        if (k < p.kv) {
          const int tk = p.flip_k ? p.kv - 1 - k : k;
          tmp[k] = r < p.n_out ? __ldg(p.nbr + (int64_t)tk * p.n_out + r) : -1;
        }
      }
    };
    auto park_table = [&]() {
#pragma unroll
      for (int k = 0; k < kTcMaxKV; ++k)
        if (k < p.kv) tbl[k * 32] = tmp[k];
    };
    load_table((int)blockIdx.x);
    park_table();

    int s = 0;
    uint32_t use = 0;
    bool bad = false, dead = false;
    const uint32_t row_off = (uint32_t)((warp * 32 + lane) * 16);
    for (int bi = 0; bi < my_blocks && !dead; ++bi) {
      const bool has_next = bi + 1 < my_blocks;
      if (has_next) load_table((int)blockIdx.x + (bi + 1) * (int)gridDim.x);
      for (int grp = 0; grp < groups; ++grp) {
        if (!mbar_wait(smem_u32(&s_empty[s]), (use & 1u) ^ 1u, abort_flag)) { dead = true; break; }
        uint8_t* stage = stage0 + (size_t)s * stage_bytes;
        const int k0 = grp * GK;
        const int nk = min(GK, p.kv - k0);
        if (!p.w_resident && tid == 0) {
          const uint32_t bytes = (uint32_t)(nk * p.b_bytes);
          mbar_arrive_expect_tx(smem_u32(&s_full[s]), bytes);
          bulk_g2s(smem_u32(stage + GK * p.a_bytes), (const uint8_t*)p.packed + (size_t)k0 * p.b_bytes, bytes,
                   smem_u32(&s_full[s]));
        }
        for (int g = 0; g < nk; ++g) {
          int in_row = tbl[(k0 + g) * 32];
          if (in_row >= p.n_rows) { bad = true; in_row = -1; }
          const uint32_t ok = in_row >= 0 ? 16u : 0u;
          const uint8_t* src = rows + (size_t)(in_row >= 0 ? in_row : 0) * p.row_bytes;
          const uint32_t dst = smem_u32(stage) + (uint32_t)(g * p.a_bytes) + row_off;
          for (int c = 0; c < p.kc; ++c) cp_async_16(dst + (uint32_t)c * 2048u, src + c * 16, ok);
        }
        cp_async_arrive_noinc(smem_u32(&s_full[s]));
        if (++s == S) { s = 0; ++use; }
      }
      if (has_next) park_table();
    }
    cp_async_wait_all();
    if (bad && p.status) atomicOr(p.status, SPH_STATUS_BAD_INDEX);
  } else if (warp == 4) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      const uint32_t idesc = p.is_i8 ? make_idesc(2u, 1u, 0u, 0u, kBlockRows, (uint32_t)p.N)
                                     : make_idesc(1u, p.is_bf16 ? 1u : 0u, 0u, 0u, kBlockRows, (uint32_t)p.N);
      const uint32_t lbo_a = 2048u, sbo_a = 128u;
      const uint32_t lbo_b = (uint32_t)(p.N / 8) * 128u, sbo_b = 128u;
      const int n_mma = p.kc / 2;  // 32 bytes of K per instruction (16 x 16-bit or 32 x 8-bit)
      bool dead = false;
      if (p.w_resident) dead = !mbar_wait(smem_u32(&s_w_full), 0u, abort_flag);
      int s = 0;
      uint32_t use = 0;
      for (int bi = 0; bi < my_blocks && !dead; ++bi) {
        const int buf = bi & 1;
        if (!mbar_wait(smem_u32(&s_acc_empty[buf]), (((uint32_t)bi >> 1) & 1u) ^ 1u, abort_flag)) break;
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * p.N);
        for (int grp = 0; grp < groups; ++grp) {
          if (!mbar_wait(smem_u32(&s_full[s]), use & 1u, abort_flag)) { dead = true; break; }
          fence_proxy_async();
          tc_fence_after();
          const int k0 = grp * GK;
          const int nk = min(GK, p.kv - k0);
          const uint32_t stage = smem_u32(stage0 + (size_t)s * stage_bytes);
          for (int g = 0; g < nk; ++g) {
            const uint32_t a_addr = stage + (uint32_t)(g * p.a_bytes);
            const uint32_t b_addr = p.w_resident ? smem_u32(w_smem + (size_t)(k0 + g) * p.b_bytes)
                                                 : stage + (uint32_t)(GK * p.a_bytes + g * p.b_bytes);
            for (int j = 0; j < n_mma; ++j) {
              const uint64_t a_desc = make_smem_desc(a_addr + (uint32_t)j * 2u * lbo_a, lbo_a, sbo_a);
              const uint64_t b_desc = make_smem_desc(b_addr + (uint32_t)j * 2u * lbo_b, lbo_b, sbo_b);
              const uint32_t accumulate = (k0 + g != 0 || j != 0) ? 1u : 0u;
              if (p.is_i8) umma_i8(d_tmem, a_desc, b_desc, idesc, accumulate);
              else umma_f16(d_tmem, a_desc, b_desc, idesc, accumulate);
            }
          }
          umma_commit(smem_u32(&s_empty[s]));   // the slot is free once these MMAs have read it
          if (++s == S) { s = 0; ++use; }
        }
        if (!dead) umma_commit(smem_u32(&s_acc_full[buf]));
      }
    }
    __syncwarp();
  } else {
    // ======================= epilogue =======================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    for (int blk_i = 0; blk_i < my_blocks; ++blk_i) {
      const int buf = blk_i & 1;
      const int64_t blk = (int64_t)blockIdx.x + (int64_t)blk_i * gridDim.x;
      const bool ok = mbar_wait(smem_u32(&s_acc_full[buf]), ((uint32_t)blk_i >> 1) & 1u, abort_flag);
      if (__any_sync(0xffffffffu, !ok)) break;  // warp-uniform: tcgen05.ld is warp-wide
      tc_fence_after();
      const int64_t r = blk * kBlockRows + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * p.N);
      for (int c0 = 0; c0 < p.N; c0 += 16) {
        uint32_t raw[16];
        tmem_ld16(taddr + (uint32_t)c0, raw);
        tmem_ld_wait();
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float x = p.is_i8 ? (float)(int)raw[j] : __uint_as_float(raw[j]);
          if (p.scale) x *= __ldg(p.scale + c0 + j);
          if (p.bias) x += __ldg(p.bias + c0 + j);
          if (p.relu) x = fmaxf(x, 0.f);
          v[j] = x;
        }
        if (r < p.n_out) store16(p.out, p.out_dtype, r * p.N + c0, v);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_acc_empty[buf]));
    }
  }

  // ---- wind down: every thread arrives here, also after an abort
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    // let copies still in flight land before the CTA's shared memory is released
    if (warp < 4) cp_async_wait_all();
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000ll) { }
    if (tid == 0 && p.status) atomicOr(p.status, SPH_STATUS_TIMEOUT);
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// [KV][K][N] row-major weights -> per-offset UMMA image of B = W[k]^T ([N x K], K-major, no swizzle).
template <typename T>
__global__ void pack_weight_kernel(const T* __restrict__ w, int kv, int K, int N, T* __restrict__ packed) {
  const int64_t total = (int64_t)kv * K * N;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int oc = (int)(e % N);
  const int ic = (int)((e / N) % K);
  const int k = (int)(e / ((int64_t)N * K));
  const int cpe = 16 / (int)sizeof(T);  // elements per 16-byte chunk
  const int64_t img = (int64_t)k * K * N;
  const int64_t off_bytes = (int64_t)(ic / cpe) * (N / 8) * 128 + (oc / 8) * 128 + (oc % 8) * 16 + (ic % cpe) * (int)sizeof(T);
  packed[img + off_bytes / (int64_t)sizeof(T)] = w[e];
}

bool tc_shape_ok(int dtype, int kv, int K, int N) {
  if (dtype != SPH_F16 && dtype != SPH_BF16 && dtype != SPH_I8) return false;
  const int e = dtype_bytes(dtype);
  const int row_bytes = K * e;
  if (row_bytes % 32 != 0 || row_bytes < 32 || row_bytes > 512) return false;
  if (N % 16 != 0 || N < 16 || N > 256) return false;
  if (kv < 1 || kv > kTcMaxKV) return false;
  return true;
}

}  // namespace

int conv_gather_tc(const void* rows, int dtype, int64_t n_rows, const void* packed, const int* nbr, int64_t n_out,
                   int kv, int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                   int out_dtype, int* status, cudaStream_t st) {
  if (!tc_shape_ok(dtype, kv, K, N)) {
    set_error("conv_gather_tc: unsupported dtype/shape");
    return SPH_ERR_UNSUPPORTED;
  }
  TcParams p;
  p.rows = rows; p.packed = packed; p.nbr = nbr;
  p.n_rows = n_rows; p.n_out = n_out;
  p.kv = kv; p.K = K; p.N = N;
  p.row_bytes = K * dtype_bytes(dtype);
  p.kc = p.row_bytes / 16;
  p.a_bytes = kBlockRows * p.row_bytes;
  p.b_bytes = N * p.row_bytes;
  p.flip_k = flip_k;
  p.is_i8 = dtype == SPH_I8;
  p.is_bf16 = dtype == SPH_BF16;
  p.scale = scale; p.bias = bias; p.relu = relu;
  p.out = out; p.out_dtype = out_dtype; p.status = status;
  int cols = 32;
  while (cols < 2 * N) cols <<= 1;
  p.tmem_cols = cols;
  p.num_blocks = (int)div_up64(n_out, kBlockRows);
  // offsets per stage: aim at ~16 KB of gathered rows per stage so barrier traffic is amortised
  int gk = 16384 / p.a_bytes;
  if (gk < 1) gk = 1;
  if (gk > 4) gk = 4;
  p.gk = gk;
  // weights resident when they leave room for at least 4 stages of gathered rows
  const int w_all = kv * p.b_bytes;
  p.w_resident = (w_all + 4 * gk * p.a_bytes <= kSmemBudget) ? 1 : 0;
  const int stage_bytes = gk * (p.a_bytes + (p.w_resident ? 0 : p.b_bytes));
  int avail = kSmemBudget - (p.w_resident ? w_all : 0);
  int stages = avail / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) {
    set_error("conv_gather_tc: operands do not fit in shared memory");
    return SPH_ERR_UNSUPPORTED;
  }
  p.stages = stages;
  const int smem_bytes = (p.w_resident ? w_all : 0) + stages * stage_bytes;

  static int s_sms = 0;
  if (s_sms == 0) {
    int dev = 0;
    SPH_CUDA(cudaGetDevice(&dev));
    SPH_CUDA(cudaDeviceGetAttribute(&s_sms, cudaDevAttrMultiProcessorCount, dev));
  }
  SPH_CUDA(cudaFuncSetAttribute(conv_gather_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  int occ = 1;
  SPH_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, conv_gather_tc_kernel, kTcThreads, smem_bytes));
  if (occ < 1) occ = 1;
  if (occ > 512 / cols) occ = 512 / cols;  // every resident CTA holds `cols` TMEM columns
  if (occ > 2) occ = 2;
  int grid = s_sms * occ;
  if (grid > p.num_blocks) grid = p.num_blocks;
  if (grid < 1) return SPH_OK;
  conv_gather_tc_kernel<<<grid, kTcThreads, smem_bytes, st>>>(p);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

bool conv_tc_supported(int dtype, int kv, int K, int N) { return tc_shape_ok(dtype, kv, K, N); }

int64_t packed_weight_bytes(int dtype, int kv, int K, int N) {
  return (int64_t)kv * K * N * dtype_bytes(dtype);
}

int pack_weight(const void* w, int dtype, int kv, int K, int N, void* packed, cudaStream_t st) {
  if (!tc_shape_ok(dtype, kv, K, N)) {
    set_error("pack_weight: unsupported dtype/shape");
    return SPH_ERR_UNSUPPORTED;
  }
  const int64_t total = (int64_t)kv * K * N;
  const int threads = 256;
  const unsigned blocks = (unsigned)div_up64(total, threads);
  if (dtype == SPH_I8) pack_weight_kernel<int8_t><<<blocks, threads, 0, st>>>((const int8_t*)w, kv, K, N, (int8_t*)packed);
  else pack_weight_kernel<uint16_t><<<blocks, threads, 0, st>>>((const uint16_t*)w, kv, K, N, (uint16_t*)packed);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

}  // namespace sph
