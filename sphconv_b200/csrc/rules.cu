// Rule generation over the range-voxel format without a dense voxel grid.
//
// What the reference does with a dense int32 grid [B,H,W,D] plus one global atomic per pair
// (src/sphconv/rules.cu:55-82,98-150,156-228,234-311) is done here with per-column searches:
// an output voxel o and kernel offset k name exactly one candidate input voxel i = o*s - pad + k,
// and "is i active, and which row is it" is a scan of the (short) input column that holds it.
//
//  * one CTA per output tile, one warp per kernel offset (round-robin when KV > warps);
//  * the CTA stages the tile's output voxels (row id + coordinates) in shared memory once;
//  * each warp walks that list 32 voxels at a time for its offset, ballots the hits and writes the
//    (in,out) pairs to consecutive slots of its own list, so list order is deterministic
//    (ascending output row inside a batch, batches in order) and no global atomics are used;
//  * the same pass fills the neighbour tables nbr[k][out] / nbr_t[k][in] the convolution kernels read.
#include <atomic>
#include <mutex>

#include "common.cuh"

namespace sph {

namespace {

constexpr int kEmitWarps = 9;
constexpr int kEmitThreads = kEmitWarps * 32;
constexpr int kEmitCap = 1024;      // output voxels staged per pass
constexpr int kEmitMaxRanges = 128; // (batch, tile row) ranges handled per group
constexpr int kMaxKV = 343;         // 7x7x7
constexpr int kMaxKD = 7;           // kernel extent along depth

__device__ __forceinline__ int col_start(const int* __restrict__ zp, int64_t c) {
  return c == 0 ? 0 : __ldg(zp + c - 1);
}

// Per-column depth bitmask of the INPUT tensor, used when columns are long: word w of column c holds
// {bits of depths [32w, 32w+32), number of set bits in the words before w}.  "Is depth iz active, and which
// row is it" is then one 8-byte load plus the column start - valid only when every column is stored in
// ascending depth order, which the table's builder checks (flag != 0 means some column is not).
struct ColMask {
  const uint2* table;  // null: not built (short columns), scan the column instead
  int words;
  const int* unsorted;  // device flag written by the builder
};

// Row id of input voxel (b,ix,iy,iz) or -1.
__device__ __forceinline__ int find_row(const int* __restrict__ zi, const int* __restrict__ zp, const Geom& g,
                                        const ColMask& cm, bool use_mask, int b, int ix, int iy, int iz) {
  int64_t c = ((int64_t)b * g.H + ix) * g.W + iy;
  if (use_mask) {
    uint2 e = __ldg(cm.table + c * cm.words + (iz >> 5));
    uint32_t bit = 1u << (iz & 31);
    if (!(e.x & bit)) return -1;
    return col_start(zp, c) + (int)e.y + __popc(e.x & (bit - 1u));
  }
  int s = col_start(zp, c);
  int e = __ldg(zp + c);
  for (int r = s; r < e; ++r) {
    if (__ldg(zi + r) == iz) return r;
  }
  return -1;
}

// One thread per (input column, 32-bin word): the thread walks the column's rows (a handful; the threads of one
// column read the same addresses, one transaction per warp), keeps the bits of its word and the number of rows below
// its word, and writes its {bits, prefix} entry: every entry of the table is written exactly once, coalesced, so the
// table needs no clearing beforehand.  The thread of word 0 also checks the depth order and parks the column id of
// every row in row_col (optional).
__global__ void __launch_bounds__(256)
build_colmask_kernel(const int* __restrict__ zi, const int* __restrict__ zp, int64_t ncols, int words, int D,
                     uint2* __restrict__ table, int* __restrict__ unsorted, int* __restrict__ row_col) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= ncols * words) return;
  const int64_t c = t / words;
  const int w = (int)(t - c * words);
  const int s = col_start(zp, c), e = __ldg(zp + c);
  uint32_t bits = 0u;
  int below = 0, prev = -1;
  bool bad = false;
  for (int r = s; r < e; ++r) {
    const int z = __ldg(zi + r);
    if (w == 0) {
      if (z <= prev || z >= D) bad = true;
      prev = z;
      if (row_col) row_col[r] = (int)c;
    }
    if (z >= 0 && z < D) {
      const int zw = z >> 5;
      if (zw == w) bits |= 1u << (z & 31);
      else if (zw < w) ++below;
    }
  }
  if (bad) *unsorted = 1;
  table[t] = make_uint2(bits, (uint32_t)below);
}

// The same index with one thread per COLUMN for columns of up to 8 words (depth <= 256): the column's rows are read
// once, the words are built in registers and written with 16-byte stores (one thread per column and word reads the rows
// of the column WORDS times).
template <int WORDS>
__global__ void __launch_bounds__(256)
build_colmask_cols_kernel(const int* __restrict__ zi, const int* __restrict__ zp, int64_t ncols, int D,
                          uint2* __restrict__ table, int* __restrict__ unsorted, int* __restrict__ row_col) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ncols) return;
  const int s = col_start(zp, c), e = __ldg(zp + c);
  uint32_t bits[WORDS];
#pragma unroll
  for (int w = 0; w < WORDS; ++w) bits[w] = 0u;
  int prev = -1;
  bool bad = false;
  for (int r = s; r < e; ++r) {
    const int z = __ldg(zi + r);
    if (z <= prev || z >= D) bad = true;
    prev = z;
    if (row_col) row_col[r] = (int)c;
    if (z >= 0 && z < D) {
      const int zw = z >> 5;
      const uint32_t bit = 1u << (z & 31);
#pragma unroll
      for (int w = 0; w < WORDS; ++w)
        if (zw == w) bits[w] |= bit;
    }
  }
  if (bad) *unsorted = 1;
  uint32_t below = 0u;
  uint2* dst = table + c * WORDS;
  if constexpr (WORDS == 1) {
    dst[0] = make_uint2(bits[0], 0u);
  } else {
#pragma unroll
    for (int w = 0; w < WORDS; w += 2) {
      const uint32_t b1 = below + (uint32_t)__popc(bits[w]);
      *(uint4*)(dst + w) = make_uint4(bits[w], below, bits[w + 1], b1);
      below = b1 + (uint32_t)__popc(bits[w + 1]);
    }
  }
}

// One CTA per output tile.  in_* describe the input tensor, out_* the output tensor (the same
// arrays for a submanifold layer).
__global__ void __launch_bounds__(kEmitThreads)
emit_rules_kernel(const int* __restrict__ in_zi, const int* __restrict__ in_zp, const int* __restrict__ out_zi,
                  const int* __restrict__ out_zp, Geom g, int64_t in_nnz, int64_t out_nnz, int tile_n_max,
                  int* __restrict__ rules, int* __restrict__ rule_size, int* __restrict__ nbr,
                  int* __restrict__ nbr_t, ColMask cm, int* __restrict__ status, int fast_done) {
  // fast_done: the row-parallel kernels below were launched for this call; they did the work unless
  // they found a column stored out of depth order
  if (fast_done && *cm.unsorted == 0) return;
  __shared__ int s_cnt[kMaxKV];
  __shared__ int s_rstart[kEmitMaxRanges];
  __shared__ int s_roff[kEmitMaxRanges + 1];
  __shared__ int s_vrow[kEmitCap];
  __shared__ int s_vb[kEmitCap];
  __shared__ unsigned s_vxy[kEmitCap];
  __shared__ int s_voz[kEmitCap];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int t = blockIdx.x;
  const int th = t / g.tgW, tw = t % g.tgW;
  const int ox0 = th * g.tH, oy0 = tw * g.tW;
  const int tHe = min(g.tH, g.oH - ox0);
  const int tWe = min(g.tW, g.oW - oy0);
  const int R = g.B * tHe;  // (batch, tile row) ranges; each is one contiguous run of output rows
  const bool use_mask = cm.table != nullptr && *cm.unsorted == 0;

  for (int k = tid; k < g.KV; k += kEmitThreads) s_cnt[k] = 0;
  __syncthreads();

  for (int rg = 0; rg < R; rg += kEmitMaxRanges) {
    const int nr = min(kEmitMaxRanges, R - rg);
    if (tid < nr) {
      int r = rg + tid;
      int b = r / tHe, dx = r % tHe;
      int64_t c0 = ((int64_t)b * g.oH + (ox0 + dx)) * g.oW + oy0;
      int s = col_start(out_zp, c0);
      int e = __ldg(out_zp + c0 + tWe - 1);
      s_rstart[tid] = s;
      s_roff[tid + 1] = e - s;
    }
    __syncthreads();
    if (tid == 0) {
      s_roff[0] = 0;
      for (int i = 0; i < nr; ++i) s_roff[i + 1] += s_roff[i];
    }
    __syncthreads();
    const int T = s_roff[nr];

    for (int p0 = 0; p0 < T; p0 += kEmitCap) {
      const int np = min(kEmitCap, T - p0);
      // ---- stage the output voxels [p0, p0+np) of this range group
      for (int v = tid; v < np; v += kEmitThreads) {
        int gv = p0 + v;
        int lo = 0, hi = nr;  // largest j with s_roff[j] <= gv
        while (hi - lo > 1) {
          int mid = (lo + hi) >> 1;
          if (s_roff[mid] <= gv) lo = mid; else hi = mid;
        }
        int row = s_rstart[lo] + (gv - s_roff[lo]);
        int r = rg + lo;
        int b = r / tHe, dx = r % tHe;
        int64_t c0 = ((int64_t)b * g.oH + (ox0 + dx)) * g.oW + oy0;
        int dy = 0;
        while (dy < tWe - 1 && __ldg(out_zp + c0 + dy) <= row) ++dy;
        s_vrow[v] = row;
        s_vb[v] = b;
        s_vxy[v] = ((unsigned)(ox0 + dx) << 16) | (unsigned)(oy0 + dy);
        s_voz[v] = __ldg(out_zi + row);
      }
      __syncthreads();

      // ---- one warp per (kh,kw): the KD offsets along depth read the same input column, so one look at
      //      that column serves all of them
      for (int kk = warp; kk < g.KH * g.KW; kk += kEmitWarps) {
        const int kh = kk / g.KW, kw = kk % g.KW;
        const int k0 = kk * g.KD;
        int base[kMaxKD];
#pragma unroll
        for (int j = 0; j < kMaxKD; ++j) base[j] = j < g.KD ? s_cnt[k0 + j] : 0;
        for (int c = 0; c < np; c += 32) {
          const int v = c + lane;
          int found[kMaxKD];
#pragma unroll
          for (int j = 0; j < kMaxKD; ++j) found[j] = -1;
          int out_row = -1;
          if (v < np) {
            out_row = s_vrow[v];
            const int b = s_vb[v];
            const unsigned xy = s_vxy[v];
            const int ix = (int)(xy >> 16) * g.sH - g.pH + kh * g.dH;
            const int iy = (int)(xy & 0xffffu) * g.sW - g.pW + kw * g.dW;
            const int iz0 = s_voz[v] * g.sD - g.pD;   // input depth for kd = 0; kd = j reads iz0 + j * dD
            if (ix >= 0 && ix < g.H && iy >= 0 && iy < g.W) {
              const int64_t ci = ((int64_t)b * g.H + ix) * g.W + iy;
              if (use_mask) {
                int cur_w = -1;
                uint2 e = make_uint2(0u, 0u);
                int cstart = -1;
#pragma unroll
                for (int j = 0; j < kMaxKD; ++j) {
                  const int iz = iz0 + j * g.dD;
                  if (j < g.KD && iz >= 0 && iz < g.D) {
                    if ((iz >> 5) != cur_w) {
                      cur_w = iz >> 5;
                      e = __ldg(cm.table + ci * cm.words + cur_w);
                    }
                    const uint32_t bit = 1u << (iz & 31);
                    if (e.x & bit) {
                      if (cstart < 0) cstart = col_start(in_zp, ci);
                      found[j] = cstart + (int)e.y + __popc(e.x & (bit - 1u));
                    }
                  }
                }
              } else {
                const int cs = col_start(in_zp, ci), ce = __ldg(in_zp + ci);
                for (int r = cs; r < ce; ++r) {
                  const int d = __ldg(in_zi + r) - iz0;
#pragma unroll
                  for (int j = 0; j < kMaxKD; ++j)
                    if (d == j * g.dD && j < g.KD && found[j] < 0) found[j] = r;
                }
              }
            }
          }
#pragma unroll
          for (int j = 0; j < kMaxKD; ++j) {
            if (j < g.KD) {   // uniform across the warp
              const int k = k0 + j;
              const int in_row = found[j];
              if (v < np && nbr) nbr[(int64_t)k * out_nnz + out_row] = in_row;
              const unsigned m = __ballot_sync(0xffffffffu, in_row >= 0);
              if (in_row >= 0) {
                const int slot = base[j] + __popc(m & ((1u << lane) - 1u));
                if (rules) {
                  int* lst_in = rules + ((int64_t)t * g.KV + k) * 2 * tile_n_max;
                  if (slot < tile_n_max) {
                    lst_in[slot] = in_row;
                    lst_in[tile_n_max + slot] = out_row;
                  } else if (status) {
                    atomicOr(status, SPH_STATUS_RULE_OVERFLOW);
                  }
                }
                if (nbr_t) nbr_t[(int64_t)k * in_nnz + in_row] = out_row;
              }
              base[j] += __popc(m);
            }
          }
        }
        if (lane == 0) {
#pragma unroll
          for (int j = 0; j < kMaxKD; ++j)
            if (j < g.KD) s_cnt[k0 + j] = base[j];
        }
      }
      __syncthreads();
    }
  }
  if (rule_size) {
    for (int k = tid; k < g.KV; k += kEmitThreads) rule_size[(int64_t)t * g.KV + k] = s_cnt[k];
  }
}


// ---------------------------------------------------------------------------------------------
// Row-parallel path (needs the input column masks and the neighbour table as an output).
//  1. nbr_rows_kernel: one thread per OUTPUT row looks its KH*KW input columns up in the mask table and
//     writes the KV entries nbr[k][row] (coalesced over rows) and, if asked, nbr_t[k][in] = row.
//     The row's column id was parked in the last plane of nbr by the kernel that enumerated the rows
//     (build_colmask_kernel for a submanifold layer, write_oz_idx_kernel for a strided one); the thread reads
//     it first and overwrites it last.
//  2. rule_lists_kernel: one warp per (tile, group of offsets) walks the tile's row ranges in list order
//     (batch, tile row, row), reads nbr[k][row] and ballot-compacts the hits into rules[tile][k].
// Both do nothing when a column was found out of depth order; emit_rules_kernel then does the work.
// ---------------------------------------------------------------------------------------------
// KD_CT = 3: the filter is 3 wide and 3 deep (those two loops are unrolled), 0 = extents read from the geometry.
template <int KD_CT, bool HAS_T>
__global__ void __launch_bounds__(256)
nbr_rows_kernel(const int* __restrict__ in_zp, const int* __restrict__ out_zi, Geom g, int64_t in_nnz,
                int64_t out_nnz, int* nbr, int* __restrict__ nbr_t, ColMask cm, int* __restrict__ status) {
  if (*cm.unsorted) return;
  const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= out_nnz) return;
  const int c = nbr[(int64_t)(g.KV - 1) * out_nnz + r];
  // A row nobody parked a column id for (the caller's row count exceeds the prefix total) holds whatever the buffer
  // held: it gets no neighbours and the status bit, instead of reads outside the index.
  if ((unsigned)c >= (unsigned)(g.B * g.oH * g.oW)) {
    for (int k = 0; k < g.KV; ++k) nbr[(int64_t)k * out_nnz + r] = -1;
    if (status) atomicOr(status, SPH_STATUS_BAD_INDEX);
    return;
  }
  const int oy = c % g.oW;
  const int t2 = c / g.oW;
  const int ox = t2 % g.oH;
  const int b = t2 / g.oH;
  const int iz0 = __ldg(out_zi + r) * g.sD - g.pD;
  int* dst = nbr + r;
  int* dst_t = nbr_t;
  for (int kh = 0; kh < g.KH; ++kh) {
    const int ix = ox * g.sH - g.pH + kh * g.dH;
    const int KW = KD_CT ? KD_CT : g.KW;   // the unrolled form is the cubic 3 x 3 x 3 filter
#pragma unroll
    for (int kw = 0; kw < KW; ++kw) {
      const int iy = oy * g.sW - g.pW + kw * g.dW;
      const bool col_ok = ix >= 0 && ix < g.H && iy >= 0 && iy < g.W;
      int cstart = 0;
      const uint2* row = cm.table;
      if (col_ok) {
        const int64_t ci = ((int64_t)b * g.H + ix) * g.W + iy;
        cstart = col_start(in_zp, ci);
        row = cm.table + ci * cm.words;
      }
      int cur_w = -1;
      uint2 e = make_uint2(0u, 0u);
      const int KD = KD_CT ? KD_CT : g.KD;
#pragma unroll
      for (int kd = 0; kd < KD; ++kd) {
        const int iz = iz0 + kd * g.dD;
        int found = -1;
        if (col_ok && iz >= 0 && iz < g.D) {
          if ((iz >> 5) != cur_w) {
            cur_w = iz >> 5;
            e = __ldg(row + cur_w);
          }
          const uint32_t bit = 1u << (iz & 31);
          if (e.x & bit) found = cstart + (int)e.y + __popc(e.x & (bit - 1u));
        }
        *dst = found;
        dst += out_nnz;
        if (HAS_T) {
          if (found >= 0) dst_t[found] = (int)r;
          dst_t += in_nnz;
        }
      }
    }
  }
}

constexpr int kListWarps = 8;
constexpr int kListRanges = 128;   // (batch, tile row) ranges staged per pass

// Stages runs [rg, rg + nr) of a tile - each (batch, tile row) is one contiguous run of output rows - for one warp:
// rs[i] = first row of run i, off[i] = list position of its first row (exclusive prefix of the run lengths, off[nr] =
// the number of rows).  Returns that number.  Ends with a __syncwarp().
__device__ __forceinline__ int stage_tile_runs(const int* __restrict__ out_zp, const Geom& g, int ox0, int oy0, int tHe,
                                               int tWe, int rg, int nr, int* rs, int* off, int lane) {
  int carry = 0;
  for (int base = 0; base < nr; base += 32) {
    const int i = base + lane;
    int s = 0, len = 0;
    if (i < nr) {
      const int rr = rg + i;
      const int b = rr / tHe, dx = rr % tHe;
      const int64_t c0 = ((int64_t)b * g.oH + (ox0 + dx)) * g.oW + oy0;
      s = col_start(out_zp, c0);
      len = __ldg(out_zp + c0 + tWe - 1) - s;
    }
    int incl = len;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (i < nr) {
      rs[i] = s;
      off[i + 1] = carry + incl;
    }
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) off[0] = 0;
  __syncwarp();
  return carry;
}


// The same lists for a kernel volume that is a multiple of NK, with NK offsets per warp held in registers: a warp takes
// CH x 32 list positions at a time, reads their NK table entries (CH x NK independent coalesced loads, the next
// positions' requested before these are compacted) and appends offset by offset with a ballot and a prefix popcount.
// The running count of every offset is a register of its own (the offset loop is unrolled), and the position -> row
// mapping of the tile is walked once for all NK offsets.  About a fifth of the instructions of rule_lists_kernel per
// table entry.
constexpr int kFixWarps = 4;

template <int NK, int CH>
__global__ void __launch_bounds__(kFixWarps * 32)
rule_lists_fixed_kernel(const int* __restrict__ out_zp, Geom g, int64_t out_nnz, int tile_n_max, int n_kg,
                        const int* __restrict__ nbr, int* __restrict__ rules, int* __restrict__ rule_size,
                        const int* __restrict__ unsorted, int* __restrict__ status) {
  __shared__ int s_rs[kFixWarps][kListRanges];
  __shared__ int s_off[kFixWarps][kListRanges + 1];
  if (unsorted && *unsorted) return;
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t item = (int64_t)blockIdx.x * kFixWarps + wib;
  if (item >= (int64_t)g.nTile * n_kg) return;
  const int t = (int)(item / n_kg);
  const int k_lo = (int)(item % n_kg) * NK;
  const int th = t / g.tgW, tw = t % g.tgW;
  const int ox0 = th * g.tH, oy0 = tw * g.tW;
  const int tHe = min(g.tH, g.oH - ox0);
  const int tWe = min(g.tW, g.oW - oy0);
  const int R = g.B * tHe;
  const unsigned lt = (1u << lane) - 1u;
  int* rs = s_rs[wib];
  int* off = s_off[wib];
  const int* plane0 = nbr + (int64_t)k_lo * out_nnz;
  int* lst0 = rules ? rules + ((int64_t)t * g.KV + k_lo) * 2 * tile_n_max : nullptr;
  const int64_t lst_stride = 2 * (int64_t)tile_n_max;
  int base[NK];
#pragma unroll
  for (int j = 0; j < NK; ++j) base[j] = 0;
  bool overflow = false;
  for (int rg = 0; rg < R; rg += kListRanges) {
    const int nr = min(kListRanges, R - rg);
    const int T = stage_tile_runs(out_zp, g, ox0, oy0, tHe, tWe, rg, nr, rs, off, lane);
    // positions only grow, so each lane walks the runs forward, keeping the bounds of its current run in registers
    int cur = 0, cur_lo = 0, cur_hi = off[1], cur_rs = rs[0];
    auto fetch = [&](int p0, int (&row)[CH], int (&v)[CH][NK]) {
#pragma unroll
      for (int u = 0; u < CH; ++u) {
        const int p = p0 + u * 32 + lane;
        row[u] = -1;
        if (p < T) {
          while (p >= cur_hi) {
            ++cur;
            cur_lo = cur_hi;
            cur_hi = off[cur + 1];
            cur_rs = rs[cur];
          }
          row[u] = cur_rs + (p - cur_lo);
        }
        const int* src = plane0 + (row[u] >= 0 ? row[u] : 0);
#pragma unroll
        for (int j = 0; j < NK; ++j) v[u][j] = row[u] >= 0 ? __ldg(src + (int64_t)j * out_nnz) : -1;
      }
    };
    int row[CH], v[CH][NK];
    if (T > 0) fetch(0, row, v);
    for (int p0 = 0; p0 < T; p0 += 32 * CH) {
      int nrow[CH], nv[CH][NK];
      const bool more = p0 + 32 * CH < T;
      if (more) fetch(p0 + 32 * CH, nrow, nv);
#pragma unroll
      for (int j = 0; j < NK; ++j) {
        int* lst = lst0 + j * lst_stride;
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          const unsigned m = __ballot_sync(0xffffffffu, v[u][j] >= 0);
          if (m == 0u) continue;
          if (v[u][j] >= 0 && lst0) {
            const int slot = base[j] + __popc(m & lt);
            if (slot < tile_n_max) {
              lst[slot] = v[u][j];
              lst[tile_n_max + slot] = row[u];
            } else {
              overflow = true;
            }
          }
          base[j] += __popc(m);
        }
      }
      if (more) {
#pragma unroll
        for (int u = 0; u < CH; ++u) {
          row[u] = nrow[u];
#pragma unroll
          for (int j = 0; j < NK; ++j) v[u][j] = nv[u][j];
        }
      }
    }
    __syncwarp();   // the next group overwrites the staged runs
  }
  if (rule_size) {
    int mine = 0;
#pragma unroll
    for (int j = 0; j < NK; ++j)
      if (lane == j) mine = base[j];
    if (lane < NK) rule_size[(int64_t)t * g.KV + k_lo + lane] = mine;
  }
  if (overflow && status) atomicOr(status, SPH_STATUS_RULE_OVERFLOW);
}

// kListChunks: 32-row chunks whose table reads are in flight together (8 for tiles of hundreds of rows; 1 or 2 for
// tiles of a few dozen, where the chunks beyond the tile's rows would only cost instructions)
template <int kListChunks>
__global__ void __launch_bounds__(kListWarps * 32)
rule_lists_kernel(const int* __restrict__ out_zp, Geom g, int64_t out_nnz, int tile_n_max, int kg, int n_kg,
                  const int* __restrict__ nbr, int* __restrict__ rules, int* __restrict__ rule_size,
                  const int* __restrict__ unsorted, int* __restrict__ status) {
  __shared__ int s_rs[kListWarps][kListRanges];
  __shared__ int s_off[kListWarps][kListRanges + 1];
  if (unsorted && *unsorted) return;
  const int lane = threadIdx.x & 31;
  const int wib = threadIdx.x >> 5;
  const int64_t item = (int64_t)blockIdx.x * kListWarps + wib;
  if (item >= (int64_t)g.nTile * n_kg) return;
  const int t = (int)(item / n_kg);
  const int k_lo = (int)(item % n_kg) * kg;
  const int nk = min(kg, g.KV - k_lo);          // <= 32: lane j keeps the running count of offset k_lo + j
  const int th = t / g.tgW, tw = t % g.tgW;
  const int ox0 = th * g.tH, oy0 = tw * g.tW;
  const int tHe = min(g.tH, g.oH - ox0);
  const int tWe = min(g.tW, g.oW - oy0);
  const int R = g.B * tHe;                       // each (batch, tile row) is one contiguous run of output rows
  const unsigned lt = (1u << lane) - 1u;
  int* rs = s_rs[wib];
  int* off = s_off[wib];
  int cnt = 0;
  bool overflow = false;
  for (int rg = 0; rg < R; rg += kListRanges) {
    const int nr = min(kListRanges, R - rg);
    // ---- the runs of this group and the exclusive prefix of their lengths (list position -> row)
    const int T = stage_tile_runs(out_zp, g, ox0, oy0, tHe, tWe, rg, nr, rs, off, lane);
    // list position -> row: positions only grow, so each lane walks the runs forward, keeping the bounds of
    // its current run in registers
    int cur = 0, cur_lo = 0, cur_hi = off[1], cur_rs = rs[0];
    auto rows_for = [&](int p0, int* row) {
#pragma unroll
      for (int u = 0; u < kListChunks; ++u) {
        const int p = p0 + u * 32 + lane;
        row[u] = -1;
        if (p < T) {
          while (p >= cur_hi) {
            ++cur;
            cur_lo = cur_hi;
            cur_hi = off[cur + 1];
            cur_rs = rs[cur];
          }
          row[u] = cur_rs + (p - cur_lo);
        }
      }
    };
    auto load = [&](int j, const int* row, int* val) {
      const int* plane = nbr + (int64_t)(k_lo + j) * out_nnz;
#pragma unroll
      for (int u = 0; u < kListChunks; ++u) val[u] = row[u] >= 0 ? __ldg(plane + row[u]) : -1;
    };
    // The table reads of the next step (next offset of this group of rows, or first offset of the next
    // group) are issued before the current step is compacted, so their latency overlaps the stores.
    int row[kListChunks], val[kListChunks];
    if (T > 0) {
      rows_for(0, row);
      load(0, row, val);
    }
    for (int p0 = 0; p0 < T; p0 += 32 * kListChunks) {
      int nrow[kListChunks];
      const bool more = p0 + 32 * kListChunks < T;
      for (int j = 0; j < nk; ++j) {
        int nval[kListChunks];
        if (j + 1 < nk) {
          load(j + 1, row, nval);
        } else if (more) {
          rows_for(p0 + 32 * kListChunks, nrow);
          load(0, nrow, nval);
        }
        int base = __shfl_sync(0xffffffffu, cnt, j);
        int* lst = rules ? rules + ((int64_t)t * g.KV + (k_lo + j)) * 2 * tile_n_max : nullptr;
#pragma unroll
        for (int u = 0; u < kListChunks; ++u) {
          const unsigned m = __ballot_sync(0xffffffffu, val[u] >= 0);
          if (val[u] >= 0 && lst) {
            const int slot = base + __popc(m & lt);
            if (slot < tile_n_max) {
              lst[slot] = val[u];
              lst[tile_n_max + slot] = row[u];
            } else {
              overflow = true;
            }
          }
          base += __popc(m);
        }
        if (lane == j) cnt = base;
#pragma unroll
        for (int u = 0; u < kListChunks; ++u) val[u] = nval[u];
      }
      if (more) {
#pragma unroll
        for (int u = 0; u < kListChunks; ++u) row[u] = nrow[u];
      }
    }
    __syncwarp();   // the next group overwrites the staged runs
  }
  if (rule_size && lane < nk) rule_size[(int64_t)t * g.KV + k_lo + lane] = cnt;
  if (overflow && status) atomicOr(status, SPH_STATUS_RULE_OVERFLOW);
}

// ---------------------------------------------------------------------------------------------
// Strided conv: output sparsity pattern.
// Per output column a depth bitmask (ceil(oD/32) words) = OR over the KH*KW input columns that reach it
// of the shifted/strided depth bits; popcount = column count; a three-kernel scan gives oz_ptr.
// ---------------------------------------------------------------------------------------------
constexpr int kScanThreads = 256;

__device__ __forceinline__ int block_inclusive_scan(int v, int* s_warp /*[8]*/, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  if (lane == 31) s_warp[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (kScanThreads / 32) ? s_warp[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    if (lane < (kScanThreads / 32)) s_warp[lane] = w;
  }
  __syncthreads();
  if (warp > 0) v += s_warp[warp - 1];
  if (total) *total = s_warp[kScanThreads / 32 - 1];
  __syncthreads();
  return v;
}

__global__ void __launch_bounds__(kScanThreads)
strided_mask_kernel(const int* __restrict__ zi, const int* __restrict__ zp, Geom g, int words, int64_t ncols,
                    ColMask cm, uint32_t* __restrict__ mask, int* __restrict__ counts, int* __restrict__ blocksum,
                    int fast_done) {
  if (fast_done && *cm.unsorted == 0) return;   // strided_bits_kernel + count_columns_kernel do the work
  __shared__ int s_warp[kScanThreads / 32];
  const int64_t c = (int64_t)blockIdx.x * kScanThreads + threadIdx.x;
  const bool use_mask = cm.table != nullptr && *cm.unsorted == 0;
  int count = 0;
  if (c < ncols) {
    const int oy = (int)(c % g.oW);
    const int ox = (int)((c / g.oW) % g.oH);
    const int b = (int)(c / ((int64_t)g.oW * g.oH));
    for (int w0 = 0; w0 < words; w0 += 8) {   // 8 output words (256 depth bins) per pass
      uint32_t m[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) m[j] = 0;
      auto add_depth = [&](int z) {
        for (int kd = 0; kd < g.KD; ++kd) {
          int num = z + g.pD - kd * g.dD;
          if (num < 0) break;
          if (num % g.sD) continue;
          int oz = num / g.sD;
          int wi = (oz >> 5) - w0;
          if (oz < g.oD && wi >= 0 && wi < 8) {
            uint32_t bit = 1u << (oz & 31);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (wi == j) m[j] |= bit;
          }
        }
      };
      for (int kh = 0; kh < g.KH; ++kh) {
        int ix = ox * g.sH - g.pH + kh * g.dH;
        if (ix < 0 || ix >= g.H) continue;
        for (int kw = 0; kw < g.KW; ++kw) {
          int iy = oy * g.sW - g.pW + kw * g.dW;
          if (iy < 0 || iy >= g.W) continue;
          int64_t ci = ((int64_t)b * g.H + ix) * g.W + iy;
          if (use_mask) {
            for (int w = 0; w < cm.words; ++w) {
              uint32_t bits = __ldg(cm.table + ci * cm.words + w).x;
              while (bits) {
                int z = w * 32 + __ffs(bits) - 1;
                bits &= bits - 1;
                add_depth(z);
              }
            }
          } else {
            int s = col_start(zp, ci), e = __ldg(zp + ci);
            for (int r = s; r < e; ++r) add_depth(__ldg(zi + r));
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (w0 + j < words) {
          mask[c * words + w0 + j] = m[j];
          count += __popc(m[j]);
        }
      }
    }
    counts[c] = count;
  }
  int total;
  block_inclusive_scan(count, s_warp, &total);
  if (threadIdx.x == 0) blocksum[blockIdx.x] = total;
}

// Bit-parallel form of the output pattern: one thread per (output column, 32-bin output word).  The input
// words that can reach the output word are OR-ed over the KH*KW input columns first, then every output bin
// tests its KD input bins in that union.  kBitsWords bounds the input words one output word can depend on.
constexpr int kBitsWords = 8;

__host__ __device__ inline bool strided_bits_ok(const Geom& g) {
  return (31 * g.sD + (g.KD - 1) * g.dD) / 32 + 2 <= kBitsWords;
}

__global__ void __launch_bounds__(256)
strided_bits_kernel(Geom g, int words_out, int64_t ncols_out, ColMask cm, uint32_t* __restrict__ mask) {
  if (*cm.unsorted) return;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= ncols_out * words_out) return;
  const int w = (int)(t % words_out);
  const int64_t c = t / words_out;
  const int oy = (int)(c % g.oW);
  const int ox = (int)((c / g.oW) % g.oH);
  const int b = (int)(c / ((int64_t)g.oW * g.oH));
  const int oz_lo = w * 32;
  const int n_bits = min(g.oD - oz_lo, 32);
  const int iz_lo = max(0, oz_lo * g.sD - g.pD);
  const int iz_hi = min(g.D - 1, (oz_lo + n_bits - 1) * g.sD - g.pD + (g.KD - 1) * g.dD);
  uint32_t out = 0;
  if (iz_lo <= iz_hi) {
    const int w_lo = iz_lo >> 5;
    const int nw = (iz_hi >> 5) - w_lo + 1;
    uint32_t u[kBitsWords];
#pragma unroll
    for (int j = 0; j < kBitsWords; ++j) u[j] = 0u;
    for (int kh = 0; kh < g.KH; ++kh) {
      const int ix = ox * g.sH - g.pH + kh * g.dH;
      if (ix < 0 || ix >= g.H) continue;
      for (int kw = 0; kw < g.KW; ++kw) {
        const int iy = oy * g.sW - g.pW + kw * g.dW;
        if (iy < 0 || iy >= g.W) continue;
        const uint2* row = cm.table + (((int64_t)b * g.H + ix) * g.W + iy) * cm.words + w_lo;
#pragma unroll
        for (int j = 0; j < kBitsWords; ++j)
          if (j < nw) u[j] |= __ldg(row + j).x;
      }
    }
    if (g.sD == 2 && g.pD == 1 && g.KD == 3 && g.dD == 1) {
      // The usual stride-2, 3-deep, padding-1 layer: output bin o looks at input bins 2o-1, 2o, 2o+1, i.e. at the even
      // bits of x | x << 1 | x >> 1 over the 64 input bins [64w, 64w + 64) plus the last bin of the word before.
      // w_lo is 2w - 1 (that word) for w > 0 and 0 for w = 0.
      const int first = 2 * w - w_lo;                      // index of input word 2w in u[]
      const uint32_t prev = first ? u[0] : 0u;
      const uint32_t a = first ? u[1] : u[0], bw = first ? u[2] : u[1];
      const uint32_t xa = a | (a << 1) | (a >> 1) | (prev >> 31);
      const uint32_t xb = bw | (bw << 1) | (bw >> 1) | (a >> 31);
      auto even_bits = [](uint32_t x) {                    // bits 0, 2, ..., 30 of x packed into bits 0 .. 15
        x &= 0x55555555u;
        x = (x | (x >> 1)) & 0x33333333u;
        x = (x | (x >> 2)) & 0x0f0f0f0fu;
        x = (x | (x >> 4)) & 0x00ff00ffu;
        x = (x | (x >> 8)) & 0x0000ffffu;
        return x;
      };
      out = even_bits(xa) | (even_bits(xb) << 16);
      if (n_bits < 32) out &= (1u << n_bits) - 1u;
    } else
    for (int bit = 0; bit < n_bits; ++bit) {
      const int base = (oz_lo + bit) * g.sD - g.pD;
      uint32_t hit = 0u;
      for (int kd = 0; kd < g.KD; ++kd) {
        const int iz = base + kd * g.dD;
        if (iz >= 0 && iz < g.D) {
          const int wi = (iz >> 5) - w_lo;
          uint32_t word = 0u;
#pragma unroll
          for (int j = 0; j < kBitsWords; ++j)
            if (wi == j) word = u[j];
          hit |= (word >> (iz & 31)) & 1u;
        }
      }
      out |= hit << bit;
    }
  }
  mask[t] = out;
}

// One thread per output column: bin count of the column, block-level sums for the scan.
__global__ void __launch_bounds__(kScanThreads)
count_columns_kernel(const uint32_t* __restrict__ mask, int words, int64_t ncols, const int* __restrict__ unsorted,
                     int* __restrict__ counts, int* __restrict__ blocksum) {
  if (*unsorted) return;
  __shared__ int s_warp[kScanThreads / 32];
  const int64_t c = (int64_t)blockIdx.x * kScanThreads + threadIdx.x;
  int count = 0;
  if (c < ncols) {
    for (int w = 0; w < words; ++w) count += __popc(mask[c * words + w]);
    counts[c] = count;
  }
  int total;
  block_inclusive_scan(count, s_warp, &total);
  if (threadIdx.x == 0) blocksum[blockIdx.x] = total;
}

// Single CTA: exclusive scan of the block sums in place, grand total to *out_total.
__global__ void __launch_bounds__(kScanThreads)
scan_blocksums_kernel(int* __restrict__ blocksum, int n, int* __restrict__ out_total, int* out_total_host) {
  __shared__ int s_warp[kScanThreads / 32];
  int carry = 0;
  for (int base = 0; base < n; base += kScanThreads) {
    int i = base + threadIdx.x;
    int v = i < n ? blocksum[i] : 0;
    int total;
    int inc = block_inclusive_scan(v, s_warp, &total);
    if (i < n) blocksum[i] = carry + inc - v;
    carry += total;
  }
  if (threadIdx.x == 0) {
    *out_total = carry;
    if (out_total_host) {          // mapped pinned host word: the host reads it after synchronising the stream
      *(volatile int*)out_total_host = carry;
      __threadfence_system();
    }
  }
}

// counts -> inclusive prefix (in place) using the scanned block sums.
__global__ void __launch_bounds__(kScanThreads)
scan_columns_kernel(int* __restrict__ counts, int64_t ncols, const int* __restrict__ blocksum) {
  __shared__ int s_warp[kScanThreads / 32];
  const int64_t c = (int64_t)blockIdx.x * kScanThreads + threadIdx.x;
  int v = c < ncols ? counts[c] : 0;
  int inc = block_inclusive_scan(v, s_warp, nullptr);
  if (c < ncols) counts[c] = inc + blocksum[blockIdx.x];
}

__global__ void __launch_bounds__(kScanThreads)
write_oz_idx_kernel(const uint32_t* __restrict__ mask, const int* __restrict__ oz_ptr, int words, int64_t ncols,
                    int* __restrict__ oz_idx, int* __restrict__ row_col) {
  // one thread per (column, 32-bin word): its first row is the column's start plus the bins of the words before it
  const int64_t t = (int64_t)blockIdx.x * kScanThreads + threadIdx.x;
  if (t >= ncols * words) return;
  const int64_t c = t / words;
  const int w = (int)(t - c * words);
  uint32_t m = mask[t];
  if (m == 0u) return;
  int pos = c == 0 ? 0 : oz_ptr[c - 1];
  for (int j = 0; j < w; ++j) pos += __popc(mask[c * words + j]);
  while (m) {
    const int bit = __ffs(m) - 1;
    if (row_col) row_col[pos] = (int)c;   // column id of the row, for nbr_rows_kernel
    oz_idx[pos++] = w * 32 + bit;
    m &= m - 1;
  }
}

// rules [NTile,KV,2,tnm] -> neighbour tables; one warp per (tile,k) list.
__global__ void rules_to_nbr_kernel(const int* __restrict__ rules, const int* __restrict__ rule_size, int n_lists,
                                    int kv, int tnm, int64_t in_rows, int64_t out_rows, int* __restrict__ nbr,
                                    int* __restrict__ nbr_t, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int64_t lst = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (lst >= n_lists) return;
  const int k = (int)(lst % kv);
  int n = rule_size[lst];
  if (n > tnm) {
    n = tnm;
    if (status && lane == 0) atomicOr(status, SPH_STATUS_RULE_OVERFLOW);
  }
  const int* in = rules + lst * 2 * tnm;
  const int* out = in + tnm;
  for (int v = lane; v < n; v += 32) {
    int i = in[v], o = out[v];
    if (i < 0 || i >= in_rows || o < 0 || o >= out_rows) {
      if (status) atomicOr(status, SPH_STATUS_BAD_INDEX);
      continue;
    }
    if (nbr) nbr[(int64_t)k * out_rows + o] = i;
    if (nbr_t) nbr_t[(int64_t)k * in_rows + i] = o;
  }
}

// The input column masks cost 8 bytes per (column, 32 depth bins); they are built unless the grid is so
// empty that the table would dwarf the voxel list (then the per-column scans of emit_rules_kernel are used).
bool want_colmask(const Geom& g, int64_t in_nnz) {
  return (int64_t)g.B * g.H * g.W * div_up(g.D, 32) <= 8 * in_nnz;
}

size_t colmask_bytes(const Geom& g, int64_t in_nnz) {
  if (!want_colmask(g, in_nnz)) return 0;
  size_t b = 256 + (size_t)g.B * g.H * g.W * div_up(g.D, 32) * sizeof(uint2);
  return (b + 255) & ~(size_t)255;
}

// Builds the table at `scratch` (layout: 256-byte header holding the unsorted flag, then the table).
int build_colmask(const int* zi, const int* zp, const Geom& g, int64_t in_nnz, void* scratch, ColMask* cm,
                  cudaStream_t st, int* row_col = nullptr) {
  cm->table = nullptr;
  cm->words = 0;
  cm->unsorted = nullptr;
  if (!want_colmask(g, in_nnz) || scratch == nullptr) return SPH_OK;
  const int64_t ncols = (int64_t)g.B * g.H * g.W;
  const int words = div_up(g.D, 32);
  SPH_CUDA(cudaMemsetAsync(scratch, 0, 256, st));      // the header (flag); the kernel writes every table entry
  cm->unsorted = (const int*)scratch;
  cm->words = words;
  cm->table = (const uint2*)((char*)scratch + 256);
  uint2* table = (uint2*)((char*)scratch + 256);
  const unsigned col_grid = (unsigned)div_up64(ncols, 256);
  // one thread per column pays off on large grids; a small grid (a few hundred CTAs of the other form) is launch-bound
  // either way and has more threads in flight with one thread per column and word
  switch (ncols >= 100000 ? words : 0) {
    case 1: build_colmask_cols_kernel<1><<<col_grid, 256, 0, st>>>(zi, zp, ncols, g.D, table, (int*)scratch, row_col); break;
    case 2: build_colmask_cols_kernel<2><<<col_grid, 256, 0, st>>>(zi, zp, ncols, g.D, table, (int*)scratch, row_col); break;
    case 4: build_colmask_cols_kernel<4><<<col_grid, 256, 0, st>>>(zi, zp, ncols, g.D, table, (int*)scratch, row_col); break;
    case 8: build_colmask_cols_kernel<8><<<col_grid, 256, 0, st>>>(zi, zp, ncols, g.D, table, (int*)scratch, row_col); break;
    default:
      build_colmask_kernel<<<(unsigned)div_up64(ncols * words, 256), 256, 0, st>>>(zi, zp, ncols, words, g.D, table,
                                                                            (int*)scratch, row_col);
  }
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

// Last plane of the neighbour table: where the row-enumerating kernel parks each output row's column id.
int* parked_columns(const Geom& g, int* nbr, int64_t out_nnz) {
  return nbr ? nbr + (int64_t)(g.KV - 1) * out_nnz : nullptr;
}

// Pair lists of every (tile, offset) from a finished neighbour table.
int launch_rule_lists(const int* out_zp, const Geom& g, int64_t out_nnz, int tnm, const int* nbr, int* rules,
                      int* rule_size, const int* unsorted, int* status, cudaStream_t st) {
  if (g.KV == 27) {
    // the usual 3 x 3 x 3 filter: the kernel with the offsets' running counts in registers
    // nine offsets per warp where that gives the machine enough warps, else three (small tile grids have long tiles:
    // more warps per tile also evens out their lengths).  Measured beside the convolution kernels: one chunk of 32
    // positions per step beats 2, 4 or 8 (more registers per thread = fewer list warps resident beside the persistent
    // convolution CTA), and 27 offsets per warp leaves too few warps.
#define SPH_LISTS_FIXED(NK)                                                                                           \
  rule_lists_fixed_kernel<NK, 1><<<(unsigned)div_up64((int64_t)g.nTile * (27 / NK), kFixWarps), kFixWarps * 32, 0,     \
                                   st>>>(out_zp, g, out_nnz, tnm, 27 / NK, nbr, rules, rule_size, unsorted, status)
    if ((int64_t)g.nTile * 3 >= 6000) SPH_LISTS_FIXED(9);
    else SPH_LISTS_FIXED(3);
#undef SPH_LISTS_FIXED
    SPH_LAUNCH_CHECK();
    return SPH_OK;
  }
  // enough warps to fill the machine, at most 32 offsets per warp (one running count per lane)
  const int64_t lists = (int64_t)g.nTile * g.KV;
  int kg = (int)(lists / 20000);
  kg = kg < 3 ? 3 : kg > 32 ? 32 : kg;
  if (kg > g.KV) kg = g.KV;
  const int n_kg = div_up(g.KV, kg);
  const int64_t items = (int64_t)g.nTile * n_kg;
  const unsigned grid = (unsigned)div_up64(items, kListWarps);
  // chunks per step: the smallest that holds 1.25 x the average tile (larger tiles take more steps)
  const int64_t want = (out_nnz / (g.nTile > 0 ? g.nTile : 1)) * 5 / 4;
#define SPH_LISTS(CH)                                                                                             \
  rule_lists_kernel<CH><<<grid, kListWarps * 32, 0, st>>>(out_zp, g, out_nnz, tnm, kg, n_kg, nbr, rules, rule_size, \
                                                          unsorted, status)
  if (want <= 32) SPH_LISTS(1);
  else if (want <= 64) SPH_LISTS(2);
  else if (want <= 128) SPH_LISTS(4);
  else SPH_LISTS(8);
#undef SPH_LISTS
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

// rows_parked: the column ids of the output rows are in parked_columns() (row-parallel path possible).
int launch_emit(const int* in_zi, const int* in_zp, const int* out_zi, const int* out_zp, const Geom& g,
                int64_t in_nnz, int64_t out_nnz, int tnm, int* rules, int* rule_size, int* nbr, int* nbr_t,
                const ColMask& cm, bool rows_parked, int fill_unused, int* status, cudaStream_t st) {
  if (rules && fill_unused) {
    SPH_CUDA(cudaMemsetAsync(rules, 0xFF, (size_t)g.nTile * g.KV * 2 * (size_t)tnm * sizeof(int), st));
  }
  if (nbr_t && in_nnz > 0) {
    SPH_CUDA(cudaMemsetAsync(nbr_t, 0xFF, (size_t)g.KV * (size_t)in_nnz * sizeof(int), st));
  }
  const bool fast = rows_parked && cm.table != nullptr && nbr != nullptr;
  if (fast) {
    if (out_nnz > 0) {
      const unsigned grid = (unsigned)div_up64(out_nnz, 256);
#define SPH_NBR_ROWS(KD, T) nbr_rows_kernel<KD, T><<<grid, 256, 0, st>>>(in_zp, out_zi, g, in_nnz, out_nnz, nbr, nbr_t, cm, status)
      if (g.KD == 3 && g.KW == 3) {
        if (nbr_t) SPH_NBR_ROWS(3, true); else SPH_NBR_ROWS(3, false);
      } else {
        if (nbr_t) SPH_NBR_ROWS(0, true); else SPH_NBR_ROWS(0, false);
      }
#undef SPH_NBR_ROWS
      SPH_LAUNCH_CHECK();
    }
    if (rule_size) {
      const int rc = launch_rule_lists(out_zp, g, out_nnz, tnm, nbr, rules, rule_size, cm.unsorted, status, st);
      if (rc != SPH_OK) return rc;
    }
  }
  emit_rules_kernel<<<g.nTile, kEmitThreads, 0, st>>>(in_zi, in_zp, out_zi, out_zp, g, in_nnz, out_nnz, tnm, rules,
                                                      rule_size, nbr, nbr_t, cm, status, fast ? 1 : 0);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

}  // namespace

// Inclusive prefix over columns of the popcounts of per-column bit masks (shared with the tensor ops):
// prefix[c] = number of set bits in columns 0..c; *total_dev = the grand total.  `zero_flag` points to a device int
// that holds 0; `blocksum` needs ceil(ncols / 256) ints.
int column_prefix_from_masks(const uint32_t* mask, int words, int64_t ncols, const int* zero_flag, int* prefix,
                             int* blocksum, int* total_dev, cudaStream_t st) {
  const int nblk = (int)div_up64(ncols, kScanThreads);
  count_columns_kernel<<<nblk, kScanThreads, 0, st>>>(mask, words, ncols, zero_flag, prefix, blocksum);
  SPH_LAUNCH_CHECK();
  scan_blocksums_kernel<<<1, kScanThreads, 0, st>>>(blocksum, nblk, total_dev, nullptr);
  SPH_LAUNCH_CHECK();
  scan_columns_kernel<<<nblk, kScanThreads, 0, st>>>(prefix, ncols, blocksum);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}

int make_geom(const sph_geom* s, Geom* o) {
  SPH_CHECK_ARG(s != nullptr, "geometry is null");
  Geom g;
  g.B = s->B;
  g.H = s->in_shape[0]; g.W = s->in_shape[1]; g.D = s->in_shape[2];
  g.oH = s->out_shape[0]; g.oW = s->out_shape[1]; g.oD = s->out_shape[2];
  g.KH = s->ksize[0]; g.KW = s->ksize[1]; g.KD = s->ksize[2];
  g.sH = s->stride[0]; g.sW = s->stride[1]; g.sD = s->stride[2];
  g.pH = s->padding[0]; g.pW = s->padding[1]; g.pD = s->padding[2];
  g.tH = s->tile[0]; g.tW = s->tile[1];
  g.dH = s->dilation[0] ? s->dilation[0] : 1;
  g.dW = s->dilation[1] ? s->dilation[1] : 1;
  g.dD = s->dilation[2] ? s->dilation[2] : 1;
  SPH_CHECK_ARG(g.B > 0 && g.H > 0 && g.W > 0 && g.D > 0, "batch and input shape must be positive");
  SPH_CHECK_ARG(g.oH > 0 && g.oW > 0 && g.oD > 0, "output shape must be positive");
  SPH_CHECK_ARG(g.KH > 0 && g.KW > 0 && g.KD > 0, "kernel size must be positive");
  SPH_CHECK_ARG(g.sH > 0 && g.sW > 0 && g.sD > 0, "stride must be positive");
  SPH_CHECK_ARG(g.pH >= 0 && g.pW >= 0 && g.pD >= 0, "padding must be non-negative");
  SPH_CHECK_ARG(g.tH > 0 && g.tW > 0, "tile size must be positive");
  SPH_CHECK_ARG(g.dH > 0 && g.dW > 0 && g.dD > 0, "dilation must be positive");
  g.KV = g.KH * g.KW * g.KD;
  if (g.KV > kMaxKV) {
    set_error("kernel volume %d exceeds the maximum %d", g.KV, kMaxKV);
    return SPH_ERR_LIMIT;
  }
  if (g.KD > kMaxKD) {
    set_error("kernel depth %d exceeds the maximum %d", g.KD, kMaxKD);
    return SPH_ERR_LIMIT;
  }
  if (g.oH > 65535 || g.oW > 65535) {
    set_error("output H/W beyond 65535 are not supported");
    return SPH_ERR_LIMIT;
  }
  if ((int64_t)g.B * g.H * g.W > 0x7fffffffLL || (int64_t)g.B * g.oH * g.oW > 0x7fffffffLL) {
    set_error("more than 2^31 columns");
    return SPH_ERR_LIMIT;
  }
  g.tgH = div_up(g.oH, g.tH);
  g.tgW = div_up(g.oW, g.tW);
  g.nTile = g.tgH * g.tgW;
  *o = g;
  return SPH_OK;
}

}  // namespace sph

using namespace sph;

extern "C" int sph_out_spatial(const int32_t in_shape[3], const int32_t ksize[3], const int32_t stride[3],
                               const int32_t padding[3], const int32_t dilation[3], int32_t out_shape[3]) {
  SPH_CHECK_ARG(in_shape && ksize && stride && padding && out_shape, "null argument");
  for (int d = 0; d < 3; ++d) {
    const int dil = dilation && dilation[d] ? dilation[d] : 1;
    SPH_CHECK_ARG(stride[d] > 0 && ksize[d] > 0 && dil > 0, "stride, kernel size and dilation must be positive");
    // floor((i + 2p - d(k-1) - 1)/s + 1) as the reference computes it in floating point
    int num = in_shape[d] + 2 * padding[d] - dil * (ksize[d] - 1) - 1;
    int q = num >= 0 ? num / stride[d] : -((-num + stride[d] - 1) / stride[d]);
    out_shape[d] = q + 1;
  }
  return SPH_OK;
}

extern "C" int sph_num_tiles(const sph_geom* s) {
  Geom g;
  int rc = make_geom(s, &g);
  return rc != SPH_OK ? rc : g.nTile;
}

extern "C" int sph_tile_n_max(const sph_geom* s, int64_t nnz) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(g.sH <= g.KH && g.sW <= g.KW, "stride larger than the kernel");
  int in_th = g.sH * (g.tH - 1) + g.dH * (g.KH - 1) + 1;   // = s(t-1) + K of the reference when the dilation is 1
  int in_tw = g.sW * (g.tW - 1) + g.dW * (g.KW - 1) + 1;
  // same expression, evaluation order and types as the reference: the int product is formed first,
  // then multiplied by the double sparsity, then by 2
  double sparsity = (double)nnz / (double)((int64_t)g.B * g.H * g.W * g.D);
  double size = g.B * in_th * in_tw * g.D * sparsity * 2;
  return (int)(size + 64) & (-1 << 4);
}

extern "C" int64_t sph_rules_subm_scratch_bytes(const sph_geom* s, int64_t nnz) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  return (int64_t)colmask_bytes(g, nnz);
}

extern "C" int sph_rules_subm(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* s,
                              void* d_scratch, int32_t tile_n_max, int32_t* d_rules, int32_t* d_rule_size,
                              int32_t* d_nbr, int fill_unused, int32_t* d_status, void* stream) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(d_z_ptr != nullptr && nnz >= 0 && (nnz == 0 || d_z_idx != nullptr), "null input");
  SPH_CHECK_ARG(g.H == g.oH && g.W == g.oW && g.D == g.oD, "submanifold rules need out_shape == in_shape");
  SPH_CHECK_ARG((d_rules == nullptr) == (d_rule_size == nullptr), "rules and rule_size go together");
  SPH_CHECK_ARG(d_rules == nullptr || tile_n_max > 0, "tile_n_max must be positive");
  ColMask cm;
  rc = build_colmask(d_z_idx, d_z_ptr, g, nnz, d_scratch, &cm, (cudaStream_t)stream, parked_columns(g, d_nbr, nnz));
  if (rc != SPH_OK) return rc;
  return launch_emit(d_z_idx, d_z_ptr, d_z_idx, d_z_ptr, g, nnz, nnz, tile_n_max, d_rules, d_rule_size, d_nbr,
                     nullptr, cm, /*rows_parked=*/d_nbr != nullptr, fill_unused, d_status, (cudaStream_t)stream);
}

extern "C" int sph_rule_lists(const int32_t* d_oz_ptr, const sph_geom* s, int64_t out_nnz, const int32_t* d_nbr,
                              int32_t tile_n_max, int32_t* d_rules, int32_t* d_rule_size, int fill_unused,
                              int32_t* d_status, void* stream) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(d_oz_ptr && d_rule_size && (out_nnz == 0 || d_nbr), "null argument");
  SPH_CHECK_ARG((d_rules == nullptr || tile_n_max > 0) && out_nnz >= 0, "bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  if (d_rules && fill_unused)
    SPH_CUDA(cudaMemsetAsync(d_rules, 0xFF, (size_t)g.nTile * g.KV * 2 * (size_t)tile_n_max * sizeof(int), st));
  // without d_rules the kernel only counts: d_rule_size gets the exact list lengths
  return launch_rule_lists(d_oz_ptr, g, out_nnz, tile_n_max, d_nbr, d_rules, d_rule_size, nullptr, d_status, st);
}

// ---- allocation-free variant of sph_rules_subm ---------------------------------------------------
// The scratch of the submanifold rule kernel (the per-column depth-bitmask index) lives in a fixed
// device array instead of caller memory.  The array's name is only a host-side handle: the kernels need
// its device address, looked up once per device with cudaGetSymbolAddress while that device is current.
static __device__ __align__(256) unsigned char g_subm_static_scratch[SPH_RULES_SUBM_STATIC_SCRATCH_BYTES];

extern "C" int sph_rules_subm_static(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz,
                                     const sph_geom* s, int32_t tile_n_max, int32_t* d_rules,
                                     int32_t* d_rule_size, int32_t* d_nbr, int fill_unused, int32_t* d_status,
                                     void* stream) {
  constexpr int kMaxDevices = 64;
  static std::atomic<void*> s_addr[kMaxDevices];   // zero-initialised; two threads racing on the first call store the same address
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  const size_t need = colmask_bytes(g, nnz);
  if (need > (size_t)SPH_RULES_SUBM_STATIC_SCRATCH_BYTES) {
    set_error("sph_rules_subm_static: this input needs %zu bytes of scratch, the built-in buffer holds %d; "
              "use sph_rules_subm with caller-provided scratch", need, (int)SPH_RULES_SUBM_STATIC_SCRATCH_BYTES);
    return SPH_ERR_LIMIT;
  }
  int dev = 0;
  SPH_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("sph_rules_subm_static: device ordinal %d not supported", dev);
    return SPH_ERR_LIMIT;
  }
  void* scratch = s_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    SPH_CUDA(cudaGetSymbolAddress(&scratch, g_subm_static_scratch));
    if (scratch == nullptr) {
      set_error("sph_rules_subm_static: the built-in buffer has no device address");
      return SPH_ERR_CUDA;
    }
    s_addr[dev].store(scratch, std::memory_order_release);
  }
  // the index is rebuilt (cleared first) by every call; nothing is carried over from the previous one
  return sph_rules_subm(d_z_idx, d_z_ptr, nnz, s, scratch, tile_n_max, d_rules, d_rule_size, d_nbr, fill_unused,
                        d_status, stream);
}

namespace {
struct StridedScratch {
  int words;
  int64_t ncols;
  int nblk;
  size_t mask_bytes, blocksum_bytes, colmask_bytes;
};
StridedScratch strided_layout(const Geom& g, int64_t nnz) {
  StridedScratch s;
  s.words = div_up(g.oD, 32);
  s.ncols = (int64_t)g.B * g.oH * g.oW;
  s.nblk = (int)div_up64(s.ncols, kScanThreads);
  s.mask_bytes = ((size_t)s.ncols * s.words * sizeof(uint32_t) + 255) & ~(size_t)255;
  s.blocksum_bytes = ((size_t)s.nblk * sizeof(int) + 255) & ~(size_t)255;
  s.colmask_bytes = colmask_bytes(g, nnz);
  return s;
}
// The input column-mask table sits behind the output masks and block sums; step 1 builds it, step 2 reuses it.
ColMask strided_colmask(const Geom& g, int64_t nnz, const StridedScratch& l, const void* scratch) {
  ColMask cm;
  cm.table = nullptr;
  cm.words = 0;
  cm.unsorted = nullptr;
  if (l.colmask_bytes) {
    const char* base = (const char*)scratch + l.mask_bytes + l.blocksum_bytes;
    cm.unsorted = (const int*)base;
    cm.words = div_up(g.D, 32);
    cm.table = (const uint2*)(base + 256);
  }
  return cm;
}
}  // namespace

// The host needs the output row count before it can size the outputs.  A cudaMemcpyAsync of those 4 bytes
// would queue on the device-to-host copy engine behind whatever bulk copy another stream has in flight there
// (measured: a result read-back of 90 MB on a side stream delayed it by milliseconds); instead the scan kernel
// writes the count to a word of mapped pinned host memory.  A small ring of words per device, allocated on first
// use, keeps concurrent calls apart.
namespace {
constexpr int kCountSlots = 256;
struct CountRing {
  int32_t* host = nullptr;
  int32_t* dev = nullptr;
  unsigned next = 0;          // per device: a word is reused only after kCountSlots - 1 further calls on ITS device
};
int count_slot(int32_t** host_word, int32_t** dev_word) {
  constexpr int kMaxDevices = 64;
  static CountRing rings[kMaxDevices];
  static std::mutex mu;
  int dev = 0;
  SPH_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("device ordinal %d not supported", dev);
    return SPH_ERR_LIMIT;
  }
  std::lock_guard<std::mutex> lock(mu);
  CountRing& r = rings[dev];
  if (r.host == nullptr) {
    void* h = nullptr;
    SPH_CUDA(cudaHostAlloc(&h, kCountSlots * sizeof(int32_t), cudaHostAllocMapped | cudaHostAllocPortable));
    void* d = nullptr;
    SPH_CUDA(cudaHostGetDevicePointer(&d, h, 0));
    r.host = (int32_t*)h;
    r.dev = (int32_t*)d;
  }
  const unsigned slot = r.next++ % kCountSlots;
  *host_word = r.host + slot;
  *dev_word = r.dev + slot;
  return SPH_OK;
}
}  // namespace

extern "C" int64_t sph_rules_strided_scratch_bytes(const sph_geom* s, int64_t nnz) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  StridedScratch l = strided_layout(g, nnz);
  return (int64_t)(l.mask_bytes + l.blocksum_bytes + l.colmask_bytes);
}

namespace {

// Launches the kernels of step 1.  With want_host_word the scan also writes the count to a word of mapped pinned
// host memory whose address is returned (readable once the work enqueued so far has completed).
int strided_count_impl(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* s, void* d_scratch,
                       int32_t* d_oz_ptr, int32_t* d_out_nnz, bool want_host_word, int32_t** host_word_out,
                       cudaStream_t st) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(d_z_ptr && d_scratch && d_oz_ptr && d_out_nnz && (nnz == 0 || d_z_idx), "null argument");
  StridedScratch l = strided_layout(g, nnz);
  uint32_t* mask = (uint32_t*)d_scratch;
  int* blocksum = (int*)((char*)d_scratch + l.mask_bytes);
  ColMask cm;
  rc = build_colmask(d_z_idx, d_z_ptr, g, nnz, l.colmask_bytes ? (char*)d_scratch + l.mask_bytes + l.blocksum_bytes : nullptr,
                     &cm, st);
  if (rc != SPH_OK) return rc;
  const bool fast = cm.table != nullptr && strided_bits_ok(g);
  if (fast) {
    strided_bits_kernel<<<(unsigned)div_up64(l.ncols * l.words, 256), 256, 0, st>>>(g, l.words, l.ncols, cm, mask);
    SPH_LAUNCH_CHECK();
  }
  strided_mask_kernel<<<l.nblk, kScanThreads, 0, st>>>(d_z_idx, d_z_ptr, g, l.words, l.ncols, cm, mask, d_oz_ptr,
                                                       blocksum, fast ? 1 : 0);
  SPH_LAUNCH_CHECK();
  if (fast) {
    count_columns_kernel<<<l.nblk, kScanThreads, 0, st>>>(mask, l.words, l.ncols, cm.unsorted, d_oz_ptr, blocksum);
    SPH_LAUNCH_CHECK();
  }
  int32_t* host_word = nullptr;
  int32_t* dev_word = nullptr;
  if (want_host_word) {
    rc = count_slot(&host_word, &dev_word);
    if (rc != SPH_OK) return rc;
  }
  scan_blocksums_kernel<<<1, kScanThreads, 0, st>>>(blocksum, l.nblk, d_out_nnz, dev_word);
  SPH_LAUNCH_CHECK();
  scan_columns_kernel<<<l.nblk, kScanThreads, 0, st>>>(d_oz_ptr, l.ncols, blocksum);
  SPH_LAUNCH_CHECK();
  if (host_word_out) *host_word_out = host_word;
  return SPH_OK;
}

}  // namespace

extern "C" int sph_rules_strided_count(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz,
                                       const sph_geom* s, void* d_scratch, int32_t* d_oz_ptr, int32_t* d_out_nnz,
                                       int32_t* h_out_nnz, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* host_word = nullptr;
  int rc = strided_count_impl(d_z_idx, d_z_ptr, nnz, s, d_scratch, d_oz_ptr, d_out_nnz, h_out_nnz != nullptr,
                              &host_word, st);
  if (rc != SPH_OK) return rc;
  if (h_out_nnz) {
    SPH_CUDA(cudaStreamSynchronize(st));
    *h_out_nnz = *(volatile int32_t*)host_word;
  }
  return SPH_OK;
}

extern "C" int sph_rules_strided_count_async(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz,
                                             const sph_geom* s, void* d_scratch, int32_t* d_oz_ptr,
                                             int32_t* d_out_nnz, const int32_t** h_count_word, void* stream) {
  SPH_CHECK_ARG(h_count_word != nullptr, "null argument");
  int32_t* host_word = nullptr;
  int rc = strided_count_impl(d_z_idx, d_z_ptr, nnz, s, d_scratch, d_oz_ptr, d_out_nnz, true, &host_word,
                              (cudaStream_t)stream);
  if (rc != SPH_OK) return rc;
  *h_count_word = host_word;
  return SPH_OK;
}

extern "C" int sph_rules_strided_fill(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz,
                                      const sph_geom* s, const void* d_scratch, const int32_t* d_oz_ptr,
                                      int64_t out_nnz, int32_t tile_n_max, int32_t* d_oz_idx, int32_t* d_rules,
                                      int32_t* d_rule_size, int32_t* d_nbr, int32_t* d_nbr_t, int fill_unused,
                                      int32_t* d_status, void* stream) {
  Geom g;
  int rc = make_geom(s, &g);
  if (rc != SPH_OK) return rc;
  SPH_CHECK_ARG(d_z_ptr && d_scratch && d_oz_ptr && (nnz == 0 || d_z_idx), "null argument");
  SPH_CHECK_ARG(out_nnz >= 0 && (out_nnz == 0 || d_oz_idx), "oz_idx is null");
  SPH_CHECK_ARG((d_rules == nullptr) == (d_rule_size == nullptr), "rules and rule_size go together");
  SPH_CHECK_ARG(d_rules == nullptr || tile_n_max > 0, "tile_n_max must be positive");
  cudaStream_t st = (cudaStream_t)stream;
  StridedScratch l = strided_layout(g, nnz);
  const uint32_t* mask = (const uint32_t*)d_scratch;
  if (out_nnz > 0) {
    write_oz_idx_kernel<<<(unsigned)div_up64(l.ncols * l.words, kScanThreads), kScanThreads, 0, st>>>(
        mask, d_oz_ptr, l.words, l.ncols, d_oz_idx, parked_columns(g, d_nbr, out_nnz));
    SPH_LAUNCH_CHECK();
  }
  return launch_emit(d_z_idx, d_z_ptr, d_oz_idx, d_oz_ptr, g, nnz, out_nnz, tile_n_max, d_rules, d_rule_size,
                     d_nbr, d_nbr_t, strided_colmask(g, nnz, l, d_scratch), /*rows_parked=*/d_nbr != nullptr,
                     fill_unused, d_status, st);
}

extern "C" int sph_rules_to_nbr(const int32_t* d_rules, const int32_t* d_rule_size, int32_t n_tile, int32_t kv,
                                int32_t tile_n_max, int64_t in_rows, int64_t out_rows, int32_t* d_nbr,
                                int32_t* d_nbr_t, int32_t* d_status, void* stream) {
  SPH_CHECK_ARG(d_rules && d_rule_size, "null rules");
  SPH_CHECK_ARG(n_tile > 0 && kv > 0 && tile_n_max > 0 && in_rows >= 0 && out_rows >= 0, "bad sizes");
  cudaStream_t st = (cudaStream_t)stream;
  if (d_nbr && out_rows > 0) SPH_CUDA(cudaMemsetAsync(d_nbr, 0xFF, (size_t)kv * out_rows * sizeof(int), st));
  if (d_nbr_t && in_rows > 0) SPH_CUDA(cudaMemsetAsync(d_nbr_t, 0xFF, (size_t)kv * in_rows * sizeof(int), st));
  int64_t n_lists = (int64_t)n_tile * kv;
  int threads = 256;
  int64_t blocks = div_up64(n_lists * 32, threads);
  rules_to_nbr_kernel<<<(unsigned)blocks, threads, 0, st>>>(d_rules, d_rule_size, (int)n_lists, kv, tile_n_max,
                                                            in_rows, out_rows, d_nbr, d_nbr_t, d_status);
  SPH_LAUNCH_CHECK();
  return SPH_OK;
}
