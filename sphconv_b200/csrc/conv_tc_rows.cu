// Output-stationary gather-GEMM on the Blackwell tensor cores (tcgen05 + TMEM), rows as the MMA's M dimension.
//
//   out[r,:] = epilogue( sum_k rows[nbr[k][r], :] @ W[k] )          r in [0, n_out)
//
//   D[128 rows x oC] += X_k[128 rows x iC] * W[k][iC x oC]
//   A operand = 128 gathered neighbour rows of offset k (M = 128, K-major): each row is copied with 16-byte cp.async
//               straight into the UMMA core-matrix layout;
//   B operand = W[k]^T, N = oC, K-major, pre-packed once per weight (the image conv_tc.cu uses as its A operand);
//   D         = fp32 / int32 accumulator in TMEM, lane = output row, column = output channel.
// Two things follow from having the output row on the TMEM lane:
//  * the instruction's disable-output-lane mask switches off the rows that have no neighbour at offset k, so such
//    rows are neither copied nor zero-filled: what sits in their shared-memory slot is multiplied but never
//    accumulated.  Only the first offset of a tile, which starts the accumulator (it overwrites), zero-fills.  A layer
//    with 12 of 27 neighbours present copies 12 rows per output row instead of 27, one with 1.5 copies 2.5;
//  * an epilogue thread owns a whole output row and stores it with 16-byte stores.
// A CTA owns 256 consecutive output rows at a time (two M = 128 halves) and is persistent over such tiles.
// (The reference walks its pair lists and read-modify-writes the output per 8 pairs,
// include/sphconv/iterator.cu.h:1467-1625 driven by include/sphconv/rule_conv_kernel.cu.h:91-153.)
//
// Warp roles (416 threads): warps 0-7 gather, as two teams of four that fill alternate pipeline stages (a warp
// gathers 64 rows of its team's stage), warp 8 issues the MMAs (one thread) and owns TMEM, warps 9-12 run the
// epilogue.  Stages are handed over with mbarriers; the accumulator is double buffered in TMEM so the epilogue of
// tile i overlaps the MMAs of tile i+1.
//
// Shared-memory operand layout (no swizzle): 8-row x 16-byte core matrices of 128 contiguous bytes;
// rows: core (row group g, chunk c) at c*4112 + g*128; weights: core (channel group gn, chunk c) at
// c*(N/8)*128 + gn*128.
#include "conv_tc_gather.cuh"

namespace sph {

namespace {
namespace rowsform {

using namespace tc;
using namespace tcgather;

constexpr int kMmaWarp = kProducerWarps;
constexpr int kMmaWarp2 = kProducerWarps + 5;       // second MMA issuer (rows 128..255 of a tile), after the epilogue warps
constexpr int kTcThreads = (kProducerWarps + 1 + 4 + 1) * 32;
constexpr int kHalfRows = 128;      // rows per MMA (M)

struct RowsParams {
  const void* rows;
  const void* packed;   // [KV] images of W[k]^T, each N x K_ch, K-major
  const int* nbr;       // [KV][n_out]
  int64_t n_rows, n_out;
  int kv, K, N;         // channels gathered / produced
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
  int tbl_off, msk_off, epi_off, w_off, stage_off;   // dynamic shared memory layout (byte offsets)
};

// 16 accumulator values of one output row (channels c0 .. c0+15) -> the output row, with 16-byte stores.
template <bool I8>
__device__ __forceinline__ void store_row16(uint8_t* dst, int out_dtype, const uint32_t (&raw)[16], const float* sc,
                                            const float* bi, int relu) {
  float x[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float v = I8 ? (float)(int)raw[j] : __uint_as_float(raw[j]);
    v = fmaf(v, sc[j], bi[j]);
    x[j] = relu ? fmaxf(v, 0.f) : v;
  }
  if (out_dtype == SPH_F32) {
#pragma unroll
    for (int j = 0; j < 16; j += 4) *(float4*)(dst + j * 4) = make_float4(x[j], x[j + 1], x[j + 2], x[j + 3]);
  } else if (out_dtype == SPH_F16) {
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __half2 v = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
      h[j] = *(const uint32_t*)&v;
    }
    *(uint4*)dst = make_uint4(h[0], h[1], h[2], h[3]);
    *(uint4*)(dst + 16) = make_uint4(h[4], h[5], h[6], h[7]);
  } else if (out_dtype == SPH_BF16) {
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
      h[j] = *(const uint32_t*)&v;
    }
    *(uint4*)dst = make_uint4(h[0], h[1], h[2], h[3]);
    *(uint4*)(dst + 16) = make_uint4(h[4], h[5], h[6], h[7]);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t acc = 0;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int q = (int)fminf(fmaxf(rintf(x[4 * j + t]), -127.f), 127.f);
        acc |= ((uint32_t)q & 0xffu) << (8 * t);
      }
      w[j] = acc;
    }
    *(uint4*)dst = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// KC = 16-byte chunks per gathered row (2, 4, 8, 16), I8 = int8 operands.  Both are compile-time so that the
// per-stage instruction streams of the gather warps and of the MMA thread have no loops or branches to
// resolve: with two or three warps per scheduler nothing hides a lone warp's instruction latency, and those
// streams, not the tensor pipe or the memory system, set the pace once the data path is asynchronous.
template <int KC, bool I8>
__global__ void __maxnreg__(112) conv_gather_rows_kernel(RowsParams p) {
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
  uint32_t* s_msk = (uint32_t*)(smem + p.msk_off);   // [kMaskTiles][kTcMaxKV][8]: rows WITHOUT a neighbour, 32 per word
  float* s_epi = (float*)(smem + p.epi_off);      // [2][128]: scale, bias of the epilogue
  uint8_t* w_smem = smem + p.w_off;               // resident weight images (if any)
  uint8_t* stage0 = smem + p.stage_off;
  const int groups = (p.kv + GK - 1) / GK;        // stages per tile

  for (int c = tid; c < 128; c += kTcThreads) {
    s_epi[c] = (c < p.N && p.scale) ? __ldg(p.scale + c) : 1.f;
    s_epi[128 + c] = (c < p.N && p.bias) ? __ldg(p.bias + c) : 0.f;
  }
  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&s_full[s]), 32 * (kProducerWarps / p.groups) + (p.w_resident ? 0 : 1));
      mbar_init(smem_u32(&s_empty[s]), 2);          // both MMA issuers are done with the slot
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_acc_full[b]), 2);
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
    // ======================= gather warps (conv_tc_gather.cuh), masked form =======================
    GatherCtx c;
    c.rows = p.rows; c.packed = p.packed; c.nbr = p.nbr;
    c.n_rows = p.n_rows; c.n_out = p.n_out;
    c.kv = p.kv; c.flip_k = p.flip_k;
    c.w_resident = p.w_resident; c.w_bytes = p.w_bytes;
    c.stages = S; c.stage_bytes = stage_bytes; c.my_tiles = my_tiles;
    c.status = p.status;
    c.tbl = s_tbl; c.msk = s_msk; c.w_smem = w_smem;
    c.stage0 = smem_u32(stage0);
    c.full0 = smem_u32(&s_full[0]); c.empty0 = smem_u32(&s_empty[0]); c.w_full = smem_u32(&s_w_full);
    c.abort_flag = abort_flag;
    c.test_withhold = 0;
    run_gather_warps<KC, true>(c);
  } else if (warp == kMmaWarp || warp == kMmaWarp2) {
    // ======================= MMA issuers =======================
    // One thread per half of the tile (rows 0..127 / 128..255): the two accumulators are disjoint TMEM columns, so the
    // two instruction streams need no ordering between them, and the per-stage cost of an issuing thread (barrier
    // wait, fences, ~80 cycles per instruction issued, commit) is paid by two threads side by side.
    const int h = warp == kMmaWarp ? 0 : 1;
    if (lane == 0) {
      const uint32_t idesc = I8 ? make_idesc(2u, 1u, 0u, 0u, kHalfRows, (uint32_t)p.N)
                                : make_idesc(1u, p.is_bf16 ? 1u : 0u, 0u, 0u, kHalfRows, (uint32_t)p.N);
      // Descriptors are a constant high word plus a low word that only needs adds (start address and LBO
      // live in the low 32 bits, in 16-byte units).  A = gathered rows, B = weight image.
      const uint32_t lbo_w = (uint32_t)(p.N / 8) * 128u;
      const uint64_t w_desc0 = make_smem_desc(0u, lbo_w, 128u);
      const uint64_t x_desc0 = make_smem_desc(0u, kRowsLbo, 128u);
      const uint64_t w_hi = w_desc0 & 0xffffffff00000000ull, x_hi = x_desc0 & 0xffffffff00000000ull;
      const uint32_t w_step = (2u * lbo_w) >> 4;                 // two K chunks per instruction
      constexpr uint32_t x_step = (2u * kRowsLbo) >> 4;
      constexpr uint32_t x_half = (kHalfRows * 16u) >> 4;        // rows 128..255 of a chunk plane
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
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kTileRows);   // half h at column + h * 128
        const uint32_t* msk = s_msk + (ti % kMaskTiles) * (kTcMaxKV * 8);
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
              const int k = k0 + g;
              // rows without a neighbour at this offset are switched off in the instruction; the tile's first offset
              // was zero-filled instead and runs unmasked (its first instruction overwrites the accumulator)
              const uint4 mk = k ? *(const uint4*)(msk + k * 8 + h * 4) : make_uint4(0u, 0u, 0u, 0u);
              {
#pragma unroll
                for (int j = 0; j < NMMA; ++j) {
                  const uint64_t wd = w_hi | (uint64_t)(wl0 + (uint32_t)g * w_units + (uint32_t)j * w_step);
                  const uint64_t xd = x_hi | (uint64_t)(x_lo + (uint32_t)g * (X_BYTES >> 4) + (uint32_t)h * x_half +
                                                        (uint32_t)j * x_step);
                  const uint32_t acc = (k | j) ? 1u : 0u;
                  if (I8) umma_i8_masked(d_tmem + (uint32_t)(h * kHalfRows), xd, wd, idesc, acc, mk);
                  else umma_f16_masked(d_tmem + (uint32_t)(h * kHalfRows), xd, wd, idesc, acc, mk);
                }
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
    const int q = warp & 3;                       // TMEM lane quarter this warp may read: rows 32q .. 32q+31 of a half
    const int row_pitch = p.N * p.out_esize;      // bytes of one output row
    const int chunk_bytes = 16 * p.out_esize;
    for (int ti = 0; ti < my_tiles; ++ti) {
      const int buf = ti & 1;
      const int64_t tile = (int64_t)blockIdx.x + (int64_t)ti * gridDim.x;
      bool ok = true;
      if (lane == 0) ok = mbar_wait(smem_u32(&s_acc_full[buf]), ((uint32_t)ti >> 1) & 1u, abort_flag, 128u);
      if (__any_sync(0xffffffffu, !ok)) break;    // warp-uniform: tcgen05.ld is warp-wide
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        const int64_t row0 = tile * kTileRows + h * kHalfRows + q * 32;
        if (row0 >= p.n_out) break;               // warp-uniform
        const int64_t row = row0 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kTileRows + h * kHalfRows);
        uint8_t* dst = (uint8_t*)p.out + row * row_pitch;
#pragma unroll 1
        for (int c0 = 0; c0 < p.N; c0 += 16) {
          uint32_t raw[16];
          tmem_ld16(taddr + (uint32_t)c0, raw);   // this thread's row, channels c0 .. c0+15
          tmem_ld_wait();
          if (row < p.n_out) store_row16<I8>(dst, p.out_dtype, raw, s_epi + c0, s_epi + 128 + c0, p.relu);
          dst += chunk_bytes;
        }
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

// Dynamic shared-memory layout: neighbour table, row masks, epilogue constants, (resident weights), stages.
// Fills the layout fields of p; false when two stages do not fit.
bool plan_smem(RowsParams* p, int kv, int* smem_bytes) {
  int off = 0;
  p->tbl_off = off; off += kProducerWarps * 32 * 32 * (int)sizeof(int);   // 32 entries per lane and tile
  p->msk_off = off; off += kMaskTiles * kTcMaxKV * 8 * (int)sizeof(uint32_t);
  p->epi_off = off; off += 2 * 128 * (int)sizeof(float);
  off = (off + 1023) & ~1023;
  p->w_off = off;
  const int gk = offsets_per_stage(p->kc);
  const int w_all = kv * p->w_bytes;
  const int avail = kSmemTotal - 1024 - off;
  // resident weights or one image per stage: whichever keeps more gathered offsets in flight; resident wins ties
  int st_res = avail >= w_all ? (avail - w_all) / (gk * p->x_bytes) : 0;
  int st_str = avail / (gk * (p->x_bytes + p->w_bytes));
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
  // the gather runs at most `stages` pipeline stages ahead of the MMAs: the tiles it can have entered beyond the one
  // being multiplied must all fit in the ring of row masks
  if ((stages + gpt - 1) / gpt + 1 >= kMaskTiles) return false;
  p->groups = 2;
  *smem_bytes = off + stages * stage_bytes + 1024;
  return true;
}

void fill_shape(RowsParams* p, int dtype, int K, int N, int out_esize) {
  p->K = K; p->N = N;
  p->row_bytes = K * dtype_bytes(dtype);
  p->kc = p->row_bytes / 16;
  p->x_bytes = p->kc * (int)kRowsLbo;   // kc chunk planes of 256 rows x 16 bytes (+ the bank skew)
  p->w_bytes = N * p->row_bytes;       // image of the N channels
  p->out_esize = out_esize;
}

bool shape_ok(int dtype, int kv, int K, int N) {
  if (dtype != SPH_F16 && dtype != SPH_BF16 && dtype != SPH_I8) return false;
  const int row_bytes = K * dtype_bytes(dtype);
  if (row_bytes != 32 && row_bytes != 64 && row_bytes != 128 && row_bytes != 256) return false;
  if (N % 16 != 0 || N < 16 || N > 128) return false;     // M = 128 takes N in steps of 16
  if (kv < 1 || kv > kTcMaxKV) return false;
  RowsParams p;
  fill_shape(&p, dtype, K, N, 4);   // widest output element
  int bytes = 0;
  return plan_smem(&p, kv, &bytes);
}

}  // namespace rowsform
}  // namespace

bool conv_tc_rows_supported(int dtype, int kv, int K, int N) { return rowsform::shape_ok(dtype, kv, K, N); }

int conv_gather_tc_rows(const void* rows, int dtype, int64_t n_rows, const void* packed, const int* nbr, int64_t n_out,
                        int kv, int K, int N, int flip_k, const float* scale, const float* bias, int relu, void* out,
                        int out_dtype, int* status, cudaStream_t st) {
  using namespace rowsform;
  if (!shape_ok(dtype, kv, K, N)) {
    set_error("conv_gather_tc_rows: unsupported dtype/shape");
    return SPH_ERR_UNSUPPORTED;
  }
  RowsParams p;
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
  int smem_bytes = 0;
  if (!plan_smem(&p, kv, &smem_bytes)) {
    set_error("conv_gather_tc_rows: operands do not fit in shared memory");
    return SPH_ERR_UNSUPPORTED;
  }
  const int s_sms = current_sm_count();
  if (s_sms <= 0) return SPH_ERR_CUDA;
  // every CTA takes all 512 TMEM columns, so exactly one is resident per SM
  int grid = s_sms < p.num_tiles ? s_sms : p.num_tiles;
  if (grid < 1) return SPH_OK;
#define SPH_TC_LAUNCH(KC_, I8_)                                                                                    \
  do {                                                                                                           \
    SPH_CUDA(cudaFuncSetAttribute(conv_gather_rows_kernel<KC_, I8_>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                  smem_bytes));                                                                  \
    conv_gather_rows_kernel<KC_, I8_><<<grid, kTcThreads, smem_bytes, st>>>(p);                                  \
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

}  // namespace sph
