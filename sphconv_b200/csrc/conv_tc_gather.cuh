// The gather side of the tensor-core convolution kernels (conv_tc.cu, conv_tc_rows.cu): constants of the tile and of the
// pipeline, and the code of the eight gather warps.  Both kernels stage 256 gathered neighbour rows per kernel offset in
// the same no-swizzle UMMA core-matrix layout and hand stages to their MMA threads through the same mbarriers; they
// differ in what happens to a row WITHOUT a neighbour (zero-filled there, masked out of the instruction here).
#pragma once

#include "common.cuh"
#include "tc_common.cuh"

namespace sph {
namespace tcgather {

using namespace tc;

constexpr int kTcMaxKV = 32;        // kernel volume the tensor-core kernels handle (3x3x3 = 27)
constexpr int kTileRows = 256;      // output rows per tile
constexpr int kProducerWarps = 8;   // gather warps
// Kernel offsets per pipeline stage by row width (16-byte chunks per row).  A stage costs ~600 cycles of barrier
// hand-over whatever it holds, so narrow rows take as many offsets per stage as the table registers (32 entries per lane
// and tile) and three ring slots allow: 7 for 32-byte rows (4 stages per 27-offset tile; measured 0.087 ms against
// 0.103 ms with 4 on a 16->16 layer), 3 for 64-byte rows (9 stages; 0.343 against 0.366 ms with 2 on a 32->32 layer), 1
// for wider rows (two offsets of 128-byte rows leave only two slots: no faster).
__host__ __device__ constexpr int offsets_per_stage(int kc) { return kc == 2 ? 7 : kc == 4 ? 3 : 1; }
constexpr int kMaxStages = 8;
constexpr int kRingStages = 4;      // pipeline slots used (see plan_smem of either kernel)
constexpr int kMaskTiles = 8;       // ring of tiles whose row masks are kept (masked form)
constexpr int kSmemTotal = 227 * 1024 - 2048;   // dynamic shared memory available next to the static part
// Byte distance between K-adjacent core matrices of the gathered-row tile.  The extra 16 bytes skew the
// chunks of one row across the shared-memory banks.
constexpr uint32_t kRowsLbo = kTileRows * 16 + 16;

// KC = 16-byte chunks per gathered row (2, 4, 8, 16).
template <int KC> struct RowShape {
  static constexpr int GK = offsets_per_stage(KC);               // kernel offsets per pipeline stage
  static constexpr int LPR = KC < 8 ? KC : 8;                    // lanes per row = rows per lane
  static constexpr int PASSES = KC / LPR;                        // 2 only for 256-byte rows
  static constexpr int NMMA = KC / 2;                            // 32 bytes of K per instruction
  static constexpr uint32_t X_BYTES = (uint32_t)KC * kRowsLbo;   // gathered rows of one offset
};

// What the gather warps need from their kernel.
struct GatherCtx {
  const void* rows;
  const void* packed;          // [KV] weight images
  const int* nbr;              // [KV][n_out]
  int64_t n_rows, n_out;
  int kv, flip_k;
  int w_resident, w_bytes;     // all weight images live in shared memory / bytes of one image
  int stages, stage_bytes;     // pipeline slots, bytes per slot
  int my_tiles;                // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  int* status;
  int* tbl;                    // shared: per gather warp 32 x 32 parked table entries
  uint32_t* msk;               // shared: [kMaskTiles][kTcMaxKV][8] rows WITHOUT a neighbour, 32 per word (masked form)
  uint8_t* w_smem;             // shared: resident weight images
  uint32_t stage0;             // shared-space address of slot 0
  uint32_t full0, empty0, w_full;   // shared-space addresses of the barriers (8 bytes apart per slot)
  volatile int* abort_flag;
  int test_withhold;           // test build only: one thread never reports its copies of stage 1
};

// Runs on warps 0 .. kProducerWarps-1 of the CTA.  MASKED: publish, per tile, offset and 32 rows, the rows that have no
// neighbour (the MMA threads pass the words to the instruction as its disable-output-lane mask) and copy nothing for
// them, except at a tile's first offset, which starts the accumulator and is zero-filled.  Otherwise absent neighbours
// are zero-filled (a 16-byte cp.async with source size 0).
//
template <int KC, bool MASKED>
__device__ __forceinline__ void run_gather_warps(const GatherCtx& c) {
  using RS = RowShape<KC>;
  constexpr int GK = RS::GK, LPR = RS::LPR, PASSES = RS::PASSES;
  constexpr uint32_t X_BYTES = RS::X_BYTES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = c.stages;
  const int stage_bytes = c.stage_bytes;
  // Stage ownership: the gather warps form two teams; team q fills pipeline stages q, q + 2, ... (all 256 rows
  // of the stage, 64 per warp).  The arrive that ties a stage's barrier to the completion of a thread's copies
  // (cp.async.mbarrier.arrive.noinc) holds back the later memory instructions of that warp until the copies
  // have landed; with every warp working on every stage, the copies of stage f+1 could not be issued while
  // those of stage f were landing.  With ownership one team issues while the other team's copies land.
  // Everything below is compile-time (team count, rows per warp and lane), so a stage is straight-line code.
  constexpr int G = 2;                           // two teams of warps take alternate stages
  constexpr int wpg = kProducerWarps / G;        // warps per team
  const int grp = warp / wpg, wig = warp % wpg;
  constexpr int RPW = kTileRows / wpg;           // rows of each stage this warp gathers
  constexpr int RPL = RPW * LPR / 32;            // rows per lane and offset (LPR lanes share a row)
  if (c.w_resident && tid == 0) {
    mbar_arrive_expect_tx(c.w_full, (uint32_t)(c.kv * c.w_bytes));
    for (int k = 0; k < c.kv; ++k)   // one bulk copy per offset keeps each transfer small
      bulk_g2s(smem_u32(c.w_smem + (size_t)k * c.w_bytes), (const uint8_t*)c.packed + (size_t)k * c.w_bytes,
               (uint32_t)c.w_bytes, c.w_full);
  }
  const uint8_t* rows = (const uint8_t*)c.rows;
  // Neighbour-table entries this warp needs for ONE TILE: the offsets of the stages it owns in that tile
  // times its RPW rows, [owned stage][GK][RPW], private to the warp (at most 1024 entries: the launcher
  // checks).  They are loaded a whole tile ahead into registers (coalesced; the table streams from HBM, and
  // a load issued only a stage ahead sits behind the stage's copies) and parked at the tile boundary.
  constexpr int kMaxEnt = 32;                    // registers per lane
  constexpr int eps = GK * RPW;                  // entries per owned stage
  int* tbl = c.tbl + warp * (kMaxEnt * 32);
  int ent[kMaxEnt];
  const unsigned n_rows_u = (unsigned)c.n_rows;
  uint32_t bad = 0u;
  const int groups = (c.kv + GK - 1) / GK;        // stages per tile
  const int total = c.my_tiles * groups;           // flat stage count of this CTA
  auto first_owned = [&](int ti) {               // first flat stage >= ti * groups that this group owns
    const int base = ti * groups;
    int d = (grp - base) % G;
    if (d < 0) d += G;
    return base + d;
  };
  // Entry e of a lane is compile-time (owned stage os, offset g of the stage, 32-row chunk h); lane = row inside the
  // chunk, so a tile's loads are coalesced and cost a few instructions each.
  constexpr int CH = RPW / 32;                   // 32-row chunks of the warp's rows
  auto load_tile = [&](int ti) {
    const int sj0 = first_owned(ti) - ti * groups;           // first owned stage inside the tile
    const int64_t r0 = ((int64_t)blockIdx.x + (int64_t)ti * gridDim.x) * kTileRows + wig * RPW + lane;
    bool row_ok[CH];
#pragma unroll
    for (int h = 0; h < CH; ++h) row_ok[h] = ti < c.my_tiles && r0 + h * 32 < c.n_out;
#pragma unroll
    for (int e = 0; e < kMaxEnt; ++e) {
      constexpr int per_stage = GK * CH;
      const int os = e / per_stage, g = (e / CH) % GK, h = e % CH;   // compile-time after unrolling
      const int k = (sj0 + os * G) * GK + g;
      const int* plane = c.nbr + (int64_t)(c.flip_k ? c.kv - 1 - k : k) * c.n_out + r0;
      // plain loads with no dependent work here: all 32 stay in flight; they are checked when parked
      ent[e] = (row_ok[h] && k < c.kv) ? __ldg(plane + h * 32) : -1;
    }
  };
  // Parks the entries of tile ti (held in registers) and publishes, per offset and 32 rows, which rows have NO
  // neighbour: the MMA thread passes those words to the instruction as its disable-output-lane mask.
  auto park_tile = [&](int ti) {
    __syncwarp();   // every lane has finished reading the previous tile's entries
    const int sj0 = first_owned(ti) - ti * groups;
    uint32_t* msk = MASKED ? c.msk + (ti % kMaskTiles) * (kTcMaxKV * 8) : nullptr;
#pragma unroll
    for (int e = 0; e < kMaxEnt; ++e) {
      constexpr int per_stage = GK * CH;
      const int os = e / per_stage, g = (e / CH) % GK, h = e % CH;
      int v = ent[e];
      if ((unsigned)v >= n_rows_u) {             // -1 (absent) or an id out of range
        bad |= (uint32_t)(v + 1);                // non-zero only for an id that is neither -1 nor valid
        v = -1;
      }
      tbl[e * 32 + lane] = v;
      if constexpr (MASKED) {
        const uint32_t absent = __ballot_sync(0xffffffffu, v < 0);
        const int k = (sj0 + os * G) * GK + g;
        if (lane == 0 && k < c.kv) msk[k * 8 + wig * CH + h] = absent;
      }
    }
    if constexpr (MASKED) __threadfence_block();   // the masks are read by the MMA threads after this team's next full-barrier arrival
    __syncwarp();
  };
  const int l_chunk = lane % LPR;
  const int l_row0 = (lane / LPR) * RPL;         // first of this lane's RPL consecutive rows inside the warp's RPW
  const uint32_t lane_dst = (uint32_t)l_chunk * kRowsLbo + (uint32_t)(wig * RPW + l_row0) * 16u;
  const uint8_t* rows_c = rows + l_chunk * 16;
  const uint32_t row_bytes = (uint32_t)KC * 16u;
  const uint32_t stage0_u = c.stage0;
  const uint32_t full0 = c.full0, empty0 = c.empty0;
  int s = grp % S;                                // slot of flat stage f is f % S
  uint32_t par = ((uint32_t)(grp / S) & 1u) ^ 1u; // parity to wait for on the slot's empty barrier
  int ti = 0;                                     // tile of the current stage
  int tile_end = groups;                          // first flat stage of the next tile
  int own_j = 0;                                  // index of the current stage among this tile's owned stages
  const int batch = S >= 5 ? 2 : 1;               // owned stages acquired per poll (costs two slots of run-ahead)
  int credits = 0;
  load_tile(0);
  park_tile(0);
  load_tile(1);
  for (int f = grp; f < total; f += G) {
    while (f >= tile_end) {                       // entered the next tile: its entries are in registers
      ++ti;
      park_tile(ti);
      tile_end += groups;
      own_j = 0;
      load_tile(ti + 1);
    }
    // One lane polls (hundreds of threads polling one mbarrier serialise on it), and only every `batch` owned
    // stages: an mbarrier operation costs ~200 cycles of the polling thread, and the MMA thread releases the
    // slots in order, so "the slot of my stage after next is free" implies the slot of this one is too.
    if (credits == 0) {
      bool ok_w = true;
      if (lane == 0) {
        int sa = s + (batch - 1) * G;
        uint32_t pa = par;
        if (sa >= S) { sa -= S; pa ^= 1u; }
        ok_w = mbar_wait(empty0 + 8u * sa, pa, c.abort_flag);
      }
      if (__any_sync(0xffffffffu, !ok_w)) break;   // also orders the other lanes behind the poll
      credits = batch;
    }
    --credits;
    const uint32_t stage = stage0_u + (uint32_t)(s * stage_bytes);
    const int k0 = (f - (tile_end - groups)) * GK;
    if (!c.w_resident && wig == 0 && lane == 0) {
      const uint32_t bytes = (uint32_t)(min(GK, c.kv - k0) * c.w_bytes);
      mbar_arrive_expect_tx(full0 + 8u * s, bytes);
      bulk_g2s(stage + GK * X_BYTES, (const uint8_t*)c.packed + (size_t)k0 * c.w_bytes, bytes, full0 + 8u * s);
    }
#pragma unroll
    for (int g = 0; g < GK; ++g) {
      if (GK == 1 || k0 + g < c.kv) {
        const int* trow = tbl + own_j * eps + g * RPW + l_row0;
        // the first offset of a tile starts the accumulator: rows without a neighbour must contribute zeros there;
        // for every other offset they are masked out of the MMA and their slots are left as they are
        const bool fill = k0 + g == 0;
        const uint32_t dst0 = stage + (uint32_t)g * X_BYTES + lane_dst;
#pragma unroll
        for (int j0 = 0; j0 < RPL; j0 += LPR) {
          int r[LPR];
          if (LPR == 8) {
            const int4 a = *(const int4*)(trow + j0), b = *(const int4*)(trow + j0 + 4);
            r[0] = a.x; r[1] = a.y; r[2] = a.z; r[3] = a.w;
            r[4 % LPR] = b.x; r[5 % LPR] = b.y; r[6 % LPR] = b.z; r[7 % LPR] = b.w;
          } else if (LPR == 4) {
            const int4 a = *(const int4*)(trow + j0);
            r[0] = a.x; r[1] = a.y; r[2 % LPR] = a.z; r[3 % LPR] = a.w;
          } else {
            const int2 a = *(const int2*)(trow + j0);
            r[0] = a.x; r[1] = a.y;
          }
#pragma unroll
          for (int j = 0; j < LPR; ++j) {
            const bool present = r[j] >= 0;
            const uint8_t* src = rows_c + (size_t)(present ? (uint32_t)r[j] : 0u) * row_bytes;
            const uint32_t sz = present ? 16u : 0u;
            // .ca: the three depth offsets of one (kh,kw) read nearly the same input rows a stage or two
            // apart, and the slice of L1 that the shared-memory carve-out leaves catches most of the repeats
            if (!MASKED || present || fill) {
              cp_async_16_ca(dst0 + (uint32_t)(j0 + j) * 16u, src, sz);
              if (PASSES == 2) cp_async_16_ca(dst0 + (uint32_t)(j0 + j) * 16u + 8u * kRowsLbo, src + 128, sz);
            }
          }
        }
      }
    }
#ifdef SPH_TEST_HOOKS
    // Test build only: the bounded waits and the wind-down are exercised by a stage that never becomes full.
    if (!(c.test_withhold && f == 1 && wig == 0 && lane == 0))
#endif
    cp_async_arrive_noinc(full0 + 8u * s);
    ++own_j;
    s += G;
    if (s >= S) { s -= S; par ^= 1u; }
  }
  cp_async_wait_all();
  if (bad && c.status) atomicOr(c.status, SPH_STATUS_BAD_INDEX);
}

}  // namespace tcgather
}  // namespace sph
