// Output-stationary gather-GEMM on the Blackwell tensor cores (tcgen05 + TMEM).
//
//   out[r,:] = epilogue( sum_k rows[nbr[k][r], :] @ W[k] )          r in [0, n_out)
//
// A tcgen05.mma takes 55-128 SM cycles whatever its shape below M = 128, N = 256 (measured on B200), so the
// instruction has to be as large as the problem allows.  The channel counts here are small (<= 128) and
// the row count is huge, so the product is computed
// transposed:  D^T[oC x 256 rows] += W[k]^T[oC x iC] * X_k^T[iC x 256 rows]
//   A operand = W[k]^T, M = oC padded to 64 or 128, K-major, pre-packed once per weight;
//   B operand = the 256 gathered neighbour rows of offset k, N = 256, K-major: each row is copied with
//               16-byte cp.async straight into the UMMA core-matrix layout (absent neighbours are
//               zero-filled without touching memory);
//   D         = fp32 / int32 accumulator in TMEM, lane = output channel, column = output row.
// A CTA owns 256 consecutive output rows at a time and is persistent over such tiles.  After the last
// offset four epilogue warps read the accumulator back, apply scale/bias/ReLU and store from registers (the lanes
// of a warp hold consecutive channels of one row: each store instruction writes whole sectors of that row).
// No scatter, no atomics, every output row is written exactly once
// (the reference does a read-modify-write of the output per 8 pairs, include/sphconv/iterator.cu.h:1467-1625,
// driven by the per-tile loop of include/sphconv/rule_conv_kernel.cu.h:91-153).
//
// Warp roles (416 threads): warps 0-7 gather, as two teams of four that fill alternate pipeline stages (a
// warp gathers 64 rows of its team's stage), warp 8 issues the MMAs (one thread) and owns TMEM, warps 9-12 run
// the epilogue.  Stages are handed over with mbarriers; the accumulator is double buffered in TMEM
// (2 x 256 columns) so the epilogue of tile i overlaps the MMAs of tile i+1.
//
// Shared-memory operand layout (no swizzle): 8-row x 16-byte core matrices of 128 contiguous bytes;
// rows: core (row group g, chunk c) at c*4112 + g*128; weights: core (channel group gn, chunk c) at
// c*(N/8)*128 + gn*128 (images hold the N real channels only: the rows up to M = 64/128 that the instruction also
// reads are whatever follows in shared memory and only feed accumulator rows nobody reads).
#include "conv_tc_gather.cuh"

namespace sph {

namespace {

using namespace tc;
using namespace tcgather;

constexpr int kMmaWarp = kProducerWarps;
constexpr int kTcThreads = (kProducerWarps + 1 + 4) * 32;
constexpr int kSubRows = 64;        // accumulator columns (output rows) an epilogue thread reads back at a time

struct TcParams {
  const void* rows;
  const void* packed;   // [KV] images of W[k]^T, each N x K_ch, K-major
  const int* nbr;       // [KV][n_out]
  int64_t n_rows, n_out;
  int kv, K, N;         // channels gathered / produced
  int MP;               // N padded to the UMMA M (64 or 128)
  int row_bytes;        // K * elem bytes
  int kc;               // 16-byte chunks per gathered row
  int stages;
  int groups;           // gather-warp teams (2); team q fills stages q, q + 2, ...
  int w_resident;       // all KV weight images live in shared memory
  int x_bytes, w_bytes; // per-offset operand bytes: gathered rows, weight image
  int flip_k;
  int is_i8, is_bf16;
  const float* scale;
  const float* bias;
  int relu;
  void* out;
  int out_dtype, out_esize;
  int* status;
  int num_tiles;
  int tbl_off, w_off, stage_off;   // dynamic shared memory layout (byte offsets)
#ifdef SPH_TEST_HOOKS
  int test_withhold;               // test build only: one thread never reports its copies of stage 1
#endif
};

// 64 accumulator values of one output channel (64 consecutive output rows) -> the output, one element per row.
// The lanes of a warp hold consecutive channels, so every store instruction writes one contiguous piece of a row
// (16 or 32 channels: whole 32-byte sectors for the 16- and 32-bit types).  `dst` points at (row 0 of the 64, this
// channel); rows >= n_valid do not exist.  The dtype switch sits outside the element loop.
template <bool I8, typename OutT, typename Cvt>
__device__ __forceinline__ void store_rows64(uint8_t* dst, int row_pitch, const uint32_t (&raw)[64], float sc, float bi,
                                             int relu, int n_valid, Cvt cvt) {
  if (n_valid >= 64) {
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      float x = I8 ? (float)(int)raw[j] : __uint_as_float(raw[j]);
      x = fmaf(x, sc, bi);
      *(OutT*)(dst + (size_t)j * row_pitch) = cvt(relu ? fmaxf(x, 0.f) : x);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      float x = I8 ? (float)(int)raw[j] : __uint_as_float(raw[j]);
      x = fmaf(x, sc, bi);
      if (j < n_valid) *(OutT*)(dst + (size_t)j * row_pitch) = cvt(relu ? fmaxf(x, 0.f) : x);
    }
  }
}

template <bool I8>
__device__ __forceinline__ void store_rows64_any(uint8_t* dst, int row_pitch, int out_dtype, const uint32_t (&raw)[64],
                                                 float sc, float bi, int relu, int n_valid) {
  switch (out_dtype) {
    case SPH_F32:
      store_rows64<I8, float>(dst, row_pitch, raw, sc, bi, relu, n_valid, [](float v) { return v; });
      break;
    case SPH_F16:
      store_rows64<I8, __half>(dst, row_pitch, raw, sc, bi, relu, n_valid, [](float v) { return __float2half_rn(v); });
      break;
    case SPH_BF16:
      store_rows64<I8, __nv_bfloat16>(dst, row_pitch, raw, sc, bi, relu, n_valid,
                                      [](float v) { return __float2bfloat16_rn(v); });
      break;
    default:
      store_rows64<I8, int8_t>(dst, row_pitch, raw, sc, bi, relu, n_valid,
                               [](float v) { return (int8_t)(int)fminf(fmaxf(rintf(v), -127.f), 127.f); });
  }
}

// KC = 16-byte chunks per gathered row (2, 4, 8, 16), I8 = int8 operands.  Both are compile-time so that the
// per-stage instruction streams of the gather warps and of the MMA thread have no loops or branches to
// resolve: with two or three warps per scheduler nothing hides a lone warp's instruction latency, and those
// streams, not the tensor pipe or the memory system, set the pace once the data path is asynchronous.
template <int KC, bool I8>
__global__ void __maxnreg__(112) conv_gather_tc_kernel(TcParams p) {
  constexpr int GK = RowShape<KC>::GK, NMMA = RowShape<KC>::NMMA;
  constexpr uint32_t X_BYTES = RowShape<KC>::X_BYTES;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ __align__(8) uint64_t s_w_full;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int S = p.stages;
  const int stage_bytes = GK * ((int)X_BYTES + (p.w_resident ? 0 : p.w_bytes));
  int* s_tbl = (int*)(smem + p.tbl_off);          // per producer warp: neighbour rows of its share of one stage
  uint8_t* w_smem = smem + p.w_off;               // resident weight images (if any)
  uint8_t* stage0 = smem + p.stage_off;
  const int groups = (p.kv + GK - 1) / GK;        // stages per tile

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&s_full[s]), 32 * (kProducerWarps / p.groups) + (p.w_resident ? 0 : 1));
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_acc_full[b]), 1);
      mbar_init(smem_u32(&s_acc_empty[b]), 4);
    }
    mbar_init(smem_u32(&s_w_full), 1);
    mbar_init_fence();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&s_tmem_base), 512u);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  // tiles handled by this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const int my_tiles = (p.num_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (warp < kProducerWarps) {
    // ======================= gather warps (conv_tc_gather.cuh), zero-filling form =======================
#ifdef SPH_TEST_HOOKS
    const int withhold = p.test_withhold;
#else
    const int withhold = 0;
#endif
    GatherCtx c;
    c.rows = p.rows; c.packed = p.packed; c.nbr = p.nbr;
    c.n_rows = p.n_rows; c.n_out = p.n_out;
    c.kv = p.kv; c.flip_k = p.flip_k;
    c.w_resident = p.w_resident; c.w_bytes = p.w_bytes;
    c.stages = S; c.stage_bytes = stage_bytes; c.my_tiles = my_tiles;
    c.status = p.status;
    c.tbl = s_tbl; c.msk = nullptr; c.w_smem = w_smem;
    c.stage0 = smem_u32(stage0);
    c.full0 = smem_u32(&s_full[0]); c.empty0 = smem_u32(&s_empty[0]); c.w_full = smem_u32(&s_w_full);
    c.abort_flag = abort_flag;
    c.test_withhold = withhold;
    run_gather_warps<KC, false>(c);
  } else if (warp == kMmaWarp) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      const uint32_t idesc = I8 ? make_idesc(2u, 1u, 0u, 0u, (uint32_t)p.MP, kTileRows)
                                : make_idesc(1u, p.is_bf16 ? 1u : 0u, 0u, 0u, (uint32_t)p.MP, kTileRows);
      // Descriptors are a constant high word plus a low word that only needs adds (start address and LBO
      // live in the low 32 bits, in 16-byte units).
      const uint32_t lbo_w = (uint32_t)(p.N / 8) * 128u;
      const uint64_t w_desc0 = make_smem_desc(0u, lbo_w, 128u);
      const uint64_t x_desc0 = make_smem_desc(0u, kRowsLbo, 128u);
      const uint64_t w_hi = w_desc0 & 0xffffffff00000000ull, x_hi = x_desc0 & 0xffffffff00000000ull;
      const uint32_t w_step = (2u * lbo_w) >> 4;                 // two K chunks per instruction
      constexpr uint32_t x_step = (2u * kRowsLbo) >> 4;
      const uint32_t w_units = (uint32_t)p.w_bytes >> 4;
      const uint32_t stage_units = (uint32_t)stage_bytes >> 4;
      const uint32_t x_lo_first = (uint32_t)x_desc0 + (smem_u32(stage0) >> 4);
      const uint32_t w_lo_res = (uint32_t)w_desc0 + (smem_u32(w_smem) >> 4);          // resident images
      const uint32_t w_in_stage = (uint32_t)w_desc0 - (uint32_t)x_desc0 + ((GK * X_BYTES) >> 4);   // streamed: behind the rows
      const uint32_t full0 = smem_u32(&s_full[0]), empty0 = smem_u32(&s_empty[0]);
      bool dead = false;
      if (p.w_resident) dead = !mbar_wait(smem_u32(&s_w_full), 0u, abort_flag);
      int s = 0;
      uint32_t par = 0u;                                          // parity to wait for on the full barriers
      uint32_t x_lo = x_lo_first;
      for (int ti = 0; ti < my_tiles && !dead; ++ti) {
        const int buf = ti & 1;
        if (!mbar_wait(smem_u32(&s_acc_empty[buf]), (((uint32_t)ti >> 1) & 1u) ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kTileRows);
        uint32_t accumulate = 0u;
        uint32_t w_lo = w_lo_res;
        for (int k0 = 0; k0 < p.kv; k0 += GK) {
          if (!mbar_wait(full0 + 8u * s, par, abort_flag)) { dead = true; break; }
          // the gather warps wrote the stage with cp.async (generic proxy); the MMA reads it through the async proxy
          fence_proxy_async();
          tc_fence_after();
          const uint32_t wl0 = p.w_resident ? w_lo : x_lo + w_in_stage;
#pragma unroll
          for (int g = 0; g < GK; ++g) {
            if (GK == 1 || k0 + g < p.kv) {
#pragma unroll
              for (int j = 0; j < NMMA; ++j) {
                const uint64_t wd = w_hi | (uint64_t)(wl0 + (uint32_t)g * w_units + (uint32_t)j * w_step);
                const uint64_t xd = x_hi | (uint64_t)(x_lo + (uint32_t)g * (X_BYTES >> 4) + (uint32_t)j * x_step);
                if (I8) umma_i8(d_tmem, wd, xd, idesc, accumulate);
                else umma_f16(d_tmem, wd, xd, idesc, accumulate);
                accumulate = 1u;
              }
            }
          }
          umma_commit(empty0 + 8u * s);          // the slot is free once these MMAs have read it
          w_lo += GK * w_units;
          x_lo += stage_units;
          if (++s == S) { s = 0; par ^= 1u; x_lo = x_lo_first; }
        }
        if (!dead) umma_commit(smem_u32(&s_acc_full[buf]));
      }
    }
    __syncwarp();
  } else {
    // ======================= epilogue =======================
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    // accumulator row (= output channel) held by this thread's TMEM lane
    const int oc = p.MP == 64 ? (lane < 16 ? 16 * q + lane : -1) : 32 * q + lane;
    const bool has_oc = oc >= 0 && oc < p.N;
    const float sc = (has_oc && p.scale) ? __ldg(p.scale + oc) : 1.f;
    const float bi = (has_oc && p.bias) ? __ldg(p.bias + oc) : 0.f;
    const int row_pitch = p.N * p.out_esize;      // bytes of one output row
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int buf = ti & 1;
      const int64_t tile = (int64_t)blockIdx.x + (int64_t)ti * gridDim.x;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(smem_u32(&s_acc_full[buf]), ((uint32_t)ti >> 1) & 1u, abort_flag, 128u);
      if (__any_sync(0xffffffffu, !ok)) break;    // warp-uniform: tcgen05.ld is warp-wide
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kTileRows);
      for (int sub = 0; sub < kTileRows / kSubRows; ++sub) {
        const int64_t row0 = tile * kTileRows + sub * kSubRows;
        if (row0 >= p.n_out) break;               // warp-uniform
        uint32_t raw[kSubRows];
        tmem_ld64(taddr + (uint32_t)(sub * kSubRows), raw);
        tmem_ld_wait();
        // straight from registers to the output: no staging buffer, no barrier between the four warps (each
        // writes its own channels of the 64 rows)
        if (has_oc)
          store_rows64_any<I8>((uint8_t*)p.out + row0 * row_pitch + oc * p.out_esize, row_pitch, p.out_dtype, raw, sc,
                               bi, p.relu, (int)min((int64_t)kSubRows, p.n_out - row0));
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
    if (warp < kProducerWarps) cp_async_wait_all();
    const long long t0 = clock64();
    while (clock64() - t0 < 4000000ll) { }
    if (tid == 0 && p.status) atomicOr(p.status, SPH_STATUS_TIMEOUT);
    __syncthreads();
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512u);
  }
}

// [KV][K][N] row-major weights -> per-offset UMMA image of W[k]^T ([N x K], K-major, no swizzle).
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

int padded_m(int N) { return N <= 64 ? 64 : 128; }

// Dynamic shared-memory layout: neighbour table, (resident weights), stages.
// Fills the layout fields of p; false when two stages do not fit.
bool plan_smem(TcParams* p, int kv, int* smem_bytes) {
  int off = 0;
  p->tbl_off = off; off += kProducerWarps * 32 * 32 * (int)sizeof(int);   // 32 entries per lane and tile
  off = (off + 1023) & ~1023;
  p->w_off = off;
  const int gk = offsets_per_stage(p->kc);
  const int w_all = kv * p->w_bytes;
  const int avail = kSmemTotal - 1024 - off;            // 1 KB slack: the M = 64/128 instruction reads past a short image
  // resident weights or one image per stage: whichever keeps more gathered offsets in flight (memory latency is
  // hidden by the depth of the ring); resident wins ties because it saves the re-streaming
  int st_res = avail >= w_all ? (avail - w_all) / (gk * p->x_bytes) : 0;
  int st_str = avail / (gk * (p->x_bytes + p->w_bytes));
  // Four slots are enough run-ahead for the two teams; a deeper ring measured no faster, and the shared memory it
  // does not take stays with L1, which the gathers hit (the depth offsets of one (kh,kw) share rows).
  if (st_res > kRingStages) st_res = kRingStages;
  if (st_str > kRingStages) st_str = kRingStages;
  p->w_resident = (st_res >= 2 && st_res >= st_str) ? 1 : 0;
  int stages = p->w_resident ? st_res : st_str;
  if (p->w_resident) off += w_all;
  p->stage_off = off;
  const int stage_bytes = gk * (p->x_bytes + (p->w_resident ? 0 : p->w_bytes));
  if (stages < 2) return false;
  p->stages = stages;
  const int gpt = (kv + gk - 1) / gk;               // stages per tile
  if (((gpt + 1) / 2) * gk * 64 > 32 * 32) return false;   // 32 table entries per lane and tile
  p->groups = 2;
  *smem_bytes = off + stages * stage_bytes + 1024;
  return true;
}

void fill_shape(TcParams* p, int dtype, int K, int N, int out_esize) {
  p->K = K; p->N = N;
  p->MP = padded_m(N);
  p->row_bytes = K * dtype_bytes(dtype);
  p->kc = p->row_bytes / 16;
  p->x_bytes = p->kc * (int)kRowsLbo;   // kc chunk planes of 256 rows x 16 bytes (+ the bank skew)
  p->w_bytes = N * p->row_bytes;       // image of the N real channels
  p->out_esize = out_esize;
}

bool tc_shape_ok(int dtype, int kv, int K, int N) {
  if (dtype != SPH_F16 && dtype != SPH_BF16 && dtype != SPH_I8) return false;
  const int row_bytes = K * dtype_bytes(dtype);
  if (row_bytes != 32 && row_bytes != 64 && row_bytes != 128 && row_bytes != 256) return false;
  if (N % 8 != 0 || N < 8 || N > 128) return false;
  if (kv < 1 || kv > kTcMaxKV) return false;
  TcParams p;
  fill_shape(&p, dtype, K, N, 4);   // widest output element
  int bytes = 0;
  return plan_smem(&p, kv, &bytes);
}

#ifdef SPH_TEST_HOOKS
int g_test_withhold = 0;
#endif

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
  p.kv = kv;
  fill_shape(&p, dtype, K, N, dtype_bytes(out_dtype));
  p.flip_k = flip_k;
  p.is_i8 = dtype == SPH_I8;
  p.is_bf16 = dtype == SPH_BF16;
  p.scale = scale; p.bias = bias; p.relu = relu;
  p.out = out; p.out_dtype = out_dtype; p.status = status;
  p.num_tiles = (int)div_up64(n_out, kTileRows);
#ifdef SPH_TEST_HOOKS
  p.test_withhold = g_test_withhold;
#endif
  int smem_bytes = 0;
  if (!plan_smem(&p, kv, &smem_bytes)) {
    set_error("conv_gather_tc: operands do not fit in shared memory");
    return SPH_ERR_UNSUPPORTED;
  }
  const int s_sms = current_sm_count();
  if (s_sms <= 0) return SPH_ERR_CUDA;
  // every CTA takes all 512 TMEM columns, so exactly one is resident per SM
  int grid = s_sms < p.num_tiles ? s_sms : p.num_tiles;
  if (grid < 1) return SPH_OK;
#define SPH_TC_LAUNCH(KC_, I8_)                                                                                  \
  do {                                                                                                         \
    SPH_CUDA(cudaFuncSetAttribute(conv_gather_tc_kernel<KC_, I8_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  smem_bytes));                                                                \
    conv_gather_tc_kernel<KC_, I8_><<<grid, kTcThreads, smem_bytes, st>>>(p);                                  \
  } while (0)
  if (p.is_i8) {
    switch (p.kc) {
      case 2: SPH_TC_LAUNCH(2, true); break;
      case 4: SPH_TC_LAUNCH(4, true); break;
      case 8: SPH_TC_LAUNCH(8, true); break;
      default: SPH_TC_LAUNCH(16, true); break;
    }
  } else {
    switch (p.kc) {
      case 2: SPH_TC_LAUNCH(2, false); break;
      case 4: SPH_TC_LAUNCH(4, false); break;
      case 8: SPH_TC_LAUNCH(8, false); break;
      default: SPH_TC_LAUNCH(16, false); break;
    }
  }
#undef SPH_TC_LAUNCH
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
  if (dtype == SPH_I8)
    pack_weight_kernel<int8_t><<<blocks, threads, 0, st>>>((const int8_t*)w, kv, K, N, (int8_t*)packed);
  else
    pack_weight_kernel<uint16_t><<<blocks, threads, 0, st>>>((const uint16_t*)w, kv, K, N, (uint16_t*)packed);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

}  // namespace sph

#ifdef SPH_TEST_HOOKS
// Test build only (a second library beside the shipped one, see sphconv_b200/build.py): makes the next tensor-core
// convolution launches withhold one arrival, so that a test can watch a bounded wait run out.
extern "C" void sph_test_withhold_arrival(int on) { sph::g_test_withhold = on; }
#endif
