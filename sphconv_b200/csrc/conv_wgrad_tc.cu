// Weight gradient on the tensor cores (fp16 / bf16):  dW[k] (iC x oC) = sum_r X[nbr[k][r], :]^T  dY[r, :].
//
// The sum over output rows is the MMA's K dimension.  Both operands are "MN-major" views of row tiles that sit
// in shared memory in the same 8-row x 16-byte core-matrix layout the forward kernel gathers into:
//   A = [X_k0 | X_k1 | ...]^T : M = 128 = 128/iC kernel offsets side by side (the gathered tiles of a batch of
//       offsets are adjacent in shared memory, and a tile is iC/8 chunk planes at a constant stride, so the batch is
//       one operand of 16 planes), K = 256 output rows
//   B = dY     : N = oC, K = the same 256 output rows (a plain contiguous copy, not a gather)
//   D          : fp32 in TMEM, rows o*iC .. o*iC+iC-1 of a batch's accumulator are dW of its o-th offset.
// An instruction costs the same ~60 cycles whether M is 32 or 128, and a tile needs 16 of them (K = 16 rows each)
// per operand pair, so batching the offsets divides the instruction count by 128/iC.
// TMEM holds 512 columns, i.e. floor(512/oC) batch accumulators; if the offsets need more they are split into groups
// and the grid into (row-tile slice) x (offset group): a CTA keeps its accumulators in TMEM across ALL of its tiles
// and adds them to the fp32 gradient once at the end with red.global.add.f32 (the reference writes a partial per
// tile, [NTile,KV,iC,oC], and torch::sum's them, src/sphconv/rule_conv.cu:483-484,517).
//
// Warps 0-7 copy (dY tile once per tile, one batch of X tiles per stage), warp 8 issues the MMAs; the final flush is
// done by warps 0-3.  Same bounded waits and abort path as the forward kernel.
#include "common.cuh"
#include "tc_common.cuh"

namespace sph {

namespace {

using namespace tc;

constexpr int kTileRows = 256;
constexpr int kCopyWarps = 8;
constexpr int kCopyThreads = kCopyWarps * 32;
constexpr int kMmaWarp = kCopyWarps;
constexpr int kThreads = (kCopyWarps + 1) * 32;
constexpr int kRowsPerWarp = kTileRows / kCopyWarps;
constexpr uint32_t kPlane = kTileRows * 16 + 16;   // bytes of one chunk plane (256 rows x 16 B + bank skew)
constexpr int kMaxStages = 6;
constexpr int kSmemTotal = 227 * 1024 - 12288;   // dynamic shared memory next to the ~10 KB static part

struct WgParams {
  const void* rows;     // X [n_rows, K]
  const void* dout;     // dY [n_out, N]
  const int* nbr;       // [KV][n_out]
  float* dw;            // [KV][K][N] fp32, accumulated into
  int64_t n_rows, n_out;
  int kv, K, N;
  int kc_x, kc_y;       // 16-byte chunks per X row / dY row
  int ob;               // offsets per batch = 128 / K: one stage, one accumulator, one MMA operand
  int is_bf16;
  int groups;           // offset groups
  int per_group;        // offsets per group (a multiple of ob)
  int slices;           // row-tile slices = gridDim.x / groups
  int num_tiles;
  int stages;
  int x_bytes, y_bytes; // bytes of one X tile / one dY tile in shared memory
  int y_off, x_off;     // dynamic shared memory offsets
  int* status;
};

// KCX = 16-byte chunks per gathered X row (2, 4, 8, 16); compile-time so that the gather of a batch is straight-line code.
template <int KCX>
__global__ void __launch_bounds__(kThreads, 1) conv_wgrad_tc_kernel(WgParams p) {
  constexpr int OB = 16 / KCX;                   // offsets per batch (= p.ob)
  constexpr int LPR = KCX < 8 ? KCX : 8;         // lanes per row = consecutive rows per lane
  constexpr int PASSES = KCX / LPR;              // 2 only for 256-byte rows
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_yfull[2];
  __shared__ __align__(8) uint64_t s_yempty[2];
  __shared__ __align__(8) uint64_t s_done;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.stages;
  const int grp = (int)blockIdx.x % p.groups;       // which offsets
  const int slice = (int)blockIdx.x / p.groups;     // which tiles: slice, slice + slices, ...
  const int k_begin = grp * p.per_group;
  const int k_end = min(p.kv, k_begin + p.per_group);
  const int nk = k_end - k_begin;
  const int my_tiles = slice < p.num_tiles ? (p.num_tiles - slice + p.slices - 1) / p.slices : 0;
  uint8_t* y_smem = smem + p.y_off;
  uint8_t* x_smem = smem + p.x_off;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&s_full[s]), kCopyThreads);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_yfull[b]), kCopyThreads);
      mbar_init(smem_u32(&s_yempty[b]), 1);
    }
    mbar_init(smem_u32(&s_done), 1);
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

  if (warp < kCopyWarps) {
    // ======================= copy warps =======================
    __shared__ __align__(16) int s_ids[kCopyWarps][1 + 8][kRowsPerWarp];   // per warp: [1+o] neighbour ids of the batch's o-th offset
    int s = 0;
    uint32_t par = 1u;
    bool dead = false;
    // neighbour ids of one batch of offsets for this lane's row of tile ti (the table streams from HBM: the ids
    // of the next batch are requested before the current batch is copied)
    auto load_ids = [&](int ti, int kb, int (&nb)[8]) {
      const int64_t rr = (int64_t)(slice + ti * p.slices) * kTileRows + warp * kRowsPerWarp + lane;
#pragma unroll
      for (int o = 0; o < 8; ++o)
        nb[o] = (ti < my_tiles && o < p.ob && kb + o < k_end && rr < p.n_out) ? __ldg(p.nbr + (int64_t)(kb + o) * p.n_out + rr) : -1;
    };
    int nb[8], nb_next[8];
    load_ids(0, k_begin, nb_next);
    for (int ti = 0; ti < my_tiles && !dead; ++ti) {
      const int tile = slice + ti * p.slices;
      const int64_t r = (int64_t)tile * kTileRows + warp * kRowsPerWarp + lane;
      const int yb = ti & 1;
      // ---- dY tile (contiguous rows)
      bool ok = true;
      if (lane == 0) ok = mbar_wait(smem_u32(&s_yempty[yb]), (((uint32_t)ti >> 1) & 1u) ^ 1u, abort_flag);
      if (__any_sync(0xffffffffu, !ok)) { dead = true; break; }
      {
        // the warp's 32 dY rows are one contiguous piece of memory: lanes walk it in 16-byte steps (coalesced) and
        // drop each piece into its chunk plane
        const int64_t row0 = (int64_t)tile * kTileRows + warp * kRowsPerWarp;
        const uint8_t* src0 = (const uint8_t*)p.dout + row0 * (int64_t)(p.kc_y * 16);
        const uint32_t ydst = smem_u32(y_smem + (size_t)yb * p.y_bytes) + (uint32_t)(warp * kRowsPerWarp) * 16u;
        const int sh = 31 - __clz(p.kc_y);
        for (int t = 0; t < p.kc_y; ++t) {
          const int idx = t * 32 + lane;
          const int rl = idx >> sh, ch = idx & (p.kc_y - 1);
          const bool present = row0 + rl < p.n_out;
          cp_async_16(ydst + (uint32_t)ch * kPlane + (uint32_t)rl * 16u, present ? src0 + (size_t)idx * 16 : (const uint8_t*)p.dout,
                      present ? 16u : 0u);
        }
      }
      cp_async_arrive_noinc(smem_u32(&s_yfull[yb]));
      // ---- one batch of gathered X tiles per stage (offsets past the group's end keep stale planes: they only
      //      feed accumulator rows that are never flushed)
      for (int kb = k_begin; kb < k_end; kb += p.ob) {
#pragma unroll
        for (int o = 0; o < 8; ++o) nb[o] = nb_next[o];
        if (kb + p.ob < k_end) load_ids(ti, kb + p.ob, nb_next);
        else load_ids(ti + 1, k_begin, nb_next);
        if (lane == 0) ok = mbar_wait(smem_u32(&s_empty[s]), par, abort_flag);
        if (__any_sync(0xffffffffu, !ok)) { dead = true; break; }
        const uint32_t stage = smem_u32(x_smem + (size_t)s * p.x_bytes);
        __syncwarp();   // every lane has finished reading the previous batch's ids
#pragma unroll
        for (int o = 0; o < OB; ++o) s_ids[warp][1 + o][lane] = nb[o];
        __syncwarp();
        {
          const int l_chunk = lane % LPR;
          const int l_row0 = (lane / LPR) * LPR;
          const uint8_t* rows_c = (const uint8_t*)p.rows + l_chunk * 16;
          const unsigned n_rows_u = (unsigned)p.n_rows;
          const uint32_t dst_lane = stage + (uint32_t)l_chunk * kPlane + (uint32_t)(warp * kRowsPerWarp + l_row0) * 16u;
#pragma unroll
          for (int o = 0; o < OB; ++o) {
            if (kb + o < k_end) {      // uniform
              const int* ids = &s_ids[warp][1 + o][l_row0];
              int r[LPR];
              if (LPR == 8) {
                const int4 a = *(const int4*)ids, b = *(const int4*)(ids + 4);
                r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w;
                r[4 % LPR] = b.x; r[5 % LPR] = b.y; r[6 % LPR] = b.z; r[7 % LPR] = b.w;
              } else if (LPR == 4) {
                const int4 a = *(const int4*)ids;
                r[0] = a.x; r[1] = a.y; r[2 % LPR] = a.z; r[3 % LPR] = a.w;
              } else {
                const int2 a = *(const int2*)ids;
                r[0] = a.x; r[1] = a.y;
              }
              const uint32_t dst0 = dst_lane + (uint32_t)(o * KCX) * kPlane;
#pragma unroll
              for (int j = 0; j < LPR; ++j) {
                const bool present = (unsigned)r[j] < n_rows_u;
                const uint8_t* src = rows_c + (size_t)(present ? (uint32_t)r[j] : 0u) * (uint32_t)(KCX * 16);
                const uint32_t sz = present ? 16u : 0u;
                cp_async_16_ca(dst0 + (uint32_t)j * 16u, src, sz);
                if (PASSES == 2) cp_async_16_ca(dst0 + (uint32_t)j * 16u + 8u * kPlane, src + 128, sz);
              }
            }
          }
        }
        cp_async_arrive_noinc(smem_u32(&s_full[s]));
        __syncwarp();
        if (++s == S) { s = 0; par ^= 1u; }
      }
    }
    cp_async_wait_all();
  } else if (lane == 0) {
    // ======================= MMA issuer =======================
    // both operands MN-major: SBO = stride between 8-element blocks along M/N (= chunk planes),
    // LBO = stride between 8-row groups along K (= 128 bytes); one instruction consumes 16 rows = 2 groups
    const uint32_t idesc = make_idesc(1u, p.is_bf16 ? 1u : 0u, 1u, 1u, 128u, (uint32_t)p.N);
    const int nbatch = (nk + p.ob - 1) / p.ob;
    const uint64_t d0 = make_smem_desc(0u, 128u, kPlane);
    const uint64_t hi = d0 & 0xffffffff00000000ull;
    const uint32_t lo0 = (uint32_t)d0;
    int s = 0;
    uint32_t par = 0u;
    bool dead = false;
    for (int ti = 0; ti < my_tiles && !dead; ++ti) {
      const int yb = ti & 1;
      if (!mbar_wait(smem_u32(&s_yfull[yb]), ((uint32_t)ti >> 1) & 1u, abort_flag)) break;
      const uint32_t y_lo = lo0 + (smem_u32(y_smem + (size_t)yb * p.y_bytes) >> 4);
      for (int k = 0; k < nbatch; ++k) {
        if (!mbar_wait(smem_u32(&s_full[s]), par, abort_flag)) { dead = true; break; }
        fence_proxy_async();
        tc_fence_after();
        const uint32_t x_lo = lo0 + (smem_u32(x_smem + (size_t)s * p.x_bytes) >> 4);
        const uint32_t d_tmem = tmem_base + (uint32_t)(k * p.N);
#pragma unroll 4
        for (int j = 0; j < kTileRows / 16; ++j) {
          const uint32_t step = (uint32_t)j * ((2u * 128u) >> 4);
          umma_f16(d_tmem, hi | (uint64_t)(x_lo + step), hi | (uint64_t)(y_lo + step), idesc, (ti | j) ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_empty[s]));
        if (++s == S) { s = 0; par ^= 1u; }
      }
      if (!dead) umma_commit(smem_u32(&s_yempty[yb]));
    }
    umma_commit(smem_u32(&s_done));
    mbar_wait(smem_u32(&s_done), 0u, abort_flag);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // ======================= flush: warps 0-3 add the accumulators to the fp32 gradient =======================
  if (!s_abort && warp < 4 && my_tiles > 0) {
    const int q = warp;
    const int m = 32 * q + lane;                    // accumulator row = TMEM lane (M = 128)
    const int o = m / p.K, ic = m % p.K;            // offset inside the batch, input channel
    const int nbatch = (nk + p.ob - 1) / p.ob;
    for (int b = 0; b < nbatch; ++b) {
      const int k = k_begin + b * p.ob + o;
      for (int c0 = 0; c0 < p.N; c0 += 16) {
        uint32_t raw[16];
        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * p.N + c0), raw);
        tmem_ld_wait();
        if (o < p.ob && k < k_end) {
          float* dst = p.dw + ((int64_t)k * p.K + ic) * p.N + c0;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < p.N) atomicAdd(dst + j, __uint_as_float(raw[j]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (s_abort) {
    if (warp < kCopyWarps) cp_async_wait_all();
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

bool wgrad_plan(WgParams* p, int dtype, int kv, int K, int N) {
  if (dtype != SPH_F16 && dtype != SPH_BF16) return false;
  const int xb = K * 2, yb = N * 2;
  if (xb != 32 && xb != 64 && xb != 128 && xb != 256) return false;   // same row widths as the forward kernel
  if (yb != 32 && yb != 64 && yb != 128 && yb != 256) return false;
  if (kv < 1 || kv > 64) return false;
  p->kv = kv; p->K = K; p->N = N;
  p->kc_x = xb / 16; p->kc_y = yb / 16;
  if (N % 16 != 0) return false;                      // M = 128 needs N in steps of 16
  p->ob = 128 / K;                                   // K is 16, 32, 64 or 128
  p->x_bytes = 16 * (int)kPlane;                     // ob tiles of K/8 planes = 16 planes
  p->y_bytes = p->kc_y * (int)kPlane;
  const int nbatch = (kv + p->ob - 1) / p->ob;
  const int acc_max = 512 / N;                       // batch accumulators that fit in TMEM
  p->groups = (nbatch + acc_max - 1) / acc_max;
  p->per_group = ((nbatch + p->groups - 1) / p->groups) * p->ob;
  p->y_off = 0;
  p->x_off = 2 * p->y_bytes;
  int stages = (kSmemTotal - p->x_off) / p->x_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return false;
  p->stages = stages;
  return true;
}

}  // namespace

bool conv_wgrad_tc_supported(int dtype, int kv, int K, int N) {
  WgParams p;
  return wgrad_plan(&p, dtype, kv, K, N);
}

int conv_wgrad_tc(const void* rows, const void* dout, int dtype, int64_t n_rows, const int* nbr, int64_t n_out, int kv,
                  int K, int N, float* dw, int* status, cudaStream_t st) {
  WgParams p;
  if (!wgrad_plan(&p, dtype, kv, K, N)) {
    set_error("conv_wgrad_tc: unsupported dtype/shape");
    return SPH_ERR_UNSUPPORTED;
  }
  p.rows = rows; p.dout = dout; p.nbr = nbr; p.dw = dw;
  p.n_rows = n_rows; p.n_out = n_out;
  p.is_bf16 = dtype == SPH_BF16;
  p.status = status;
  p.num_tiles = (int)div_up64(n_out, kTileRows);
  const int s_sms = current_sm_count();
  if (s_sms <= 0) return SPH_ERR_CUDA;
  int slices = s_sms / p.groups;
  if (slices > p.num_tiles) slices = p.num_tiles;
  if (slices < 1) slices = 1;
  p.slices = slices;
  const int grid = slices * p.groups;
  const int smem_bytes = p.x_off + p.stages * p.x_bytes;
#define SPH_WG_LAUNCH(KCX_)                                                                                        \
  do {                                                                                                           \
    SPH_CUDA(cudaFuncSetAttribute(conv_wgrad_tc_kernel<KCX_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes)); \
    conv_wgrad_tc_kernel<KCX_><<<grid, kThreads, smem_bytes, st>>>(p);                                           \
  } while (0)
  switch (p.kc_x) {
    case 2: SPH_WG_LAUNCH(2); break;
    case 4: SPH_WG_LAUNCH(4); break;
    case 8: SPH_WG_LAUNCH(8); break;
    default: SPH_WG_LAUNCH(16); break;
  }
#undef SPH_WG_LAUNCH
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

}  // namespace sph

