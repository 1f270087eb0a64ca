/*
 * sphconv_b200 - C ABI of the B200 (sm_100a) implementation of the sphconv hot path:
 * rule (input/output index pair) generation over the range-voxel format and the
 * rule-driven sparse convolution (forward, dgrad, wgrad).
 *
 * Conventions
 *  - Every pointer named d_* or documented "device" is a CUDA device pointer on the current device.
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises
 *    unless stated.
 *  - Every function returns SPH_OK (0) or a negative SPH_ERR_* code and never exits the process.
 *    sph_last_error() returns a human readable message for the calling thread.
 *  - No function allocates device memory; scratch is caller-provided and sized by the
 *    *_scratch_bytes helpers.
 *  - Range-voxel format (reference: sphconv/tensor.py:33-125, src/sphconv/tensor.cu:107-109):
 *    z_ptr int32 [B,H,W] is an INCLUSIVE prefix sum over (b,h,w) row-major, global over the batch;
 *    column c (flat index) owns feature rows [c ? z_ptr[c-1] : 0, z_ptr[c]); z_idx int32 [NNZ] holds the
 *    depth index of every row.  in_shape/out_shape are {H, W, D} with D the compressed axis.
 *
 * Citations "ref:" give the file:line of reveriel/sphconv that the entry point replaces.
 */
#ifndef SPHCONV_B200_H_
#define SPHCONV_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPH_OK 0
#define SPH_ERR_INVALID (-1)     /* bad argument (null pointer, non-positive size, inconsistent shapes) */
#define SPH_ERR_UNSUPPORTED (-2) /* valid request this build does not implement (e.g. an operand shape) */
#define SPH_ERR_CUDA (-3)        /* a CUDA runtime call failed; see sph_last_error() */
#define SPH_ERR_LIMIT (-4)       /* size beyond a documented maximum */

/* bits of the device status word the kernels OR into (*d_status); 0 means clean */
#define SPH_STATUS_RULE_OVERFLOW 1 /* a (tile,k) list exceeded tile_n_max; extra pairs were not stored */
#define SPH_STATUS_BAD_INDEX 2     /* a z index / row id outside its valid range was met and skipped */
#define SPH_STATUS_TIMEOUT 4       /* a bounded device-side wait ran out */

enum sph_dtype { SPH_F32 = 0, SPH_F16 = 1, SPH_BF16 = 2, SPH_I8 = 3 };

/* Geometry of one convolution layer.  ref: argument list of get_rules / get_rules_subm,
 * include/sphconv/rules.h:8-32 (batchSize, spatialShape, outSpatialShape, kernelSize, stride, padding, tileSize). */
typedef struct sph_geom {
  int32_t B;
  int32_t in_shape[3];  /* H, W, D */
  int32_t out_shape[3]; /* oH, oW, oD */
  int32_t ksize[3];
  int32_t stride[3];
  int32_t padding[3];
  int32_t tile[2]; /* output tile (tH, tW); default of the reference is {2,2}, sphconv/conv.py:105 */
  /* Kernel offset k reads input o*stride - padding + k*dilation.  {1,1,1} is the reference: its kernels ignore the
   * argument (src/sphconv/rules.cu:40-41) while its out_spatial honours it (sphconv/utils/__init__.py:40-42), so other
   * values have no reference behaviour; here they give the dilated convolution out_spatial describes.  0 reads as 1. */
  int32_t dilation[3];
} sph_geom;

const char* sph_last_error(void);
int sph_version(void);
/* Kernels this library has launched so far in the process (all threads); for launch accounting in benchmarks. */
int64_t sph_kernel_launches(void);

/* ---- host-side geometry helpers --------------------------------------------------------------- */

/* ref: out_spatial, sphconv/utils/__init__.py:27-44: floor((i + 2p - d(k-1) - 1)/s + 1); dilation may be null (= 1). */
int sph_out_spatial(const int32_t in_shape[3], const int32_t ksize[3], const int32_t stride[3],
                    const int32_t padding[3], const int32_t dilation[3], int32_t out_shape[3]);

/* ref: huristic_tile_n_max + getInTileSize, src/sphconv/rules.cu:21-34; bit-identical result. */
int sph_tile_n_max(const sph_geom* g, int64_t nnz);

/* Number of tiles, ref: src/sphconv/rules.cu:353 and get_tile_grid_shape, sphconv/conv.py:32-38. */
int sph_num_tiles(const sph_geom* g);

/* ---- rule generation -------------------------------------------------------------------------- */

/* Submanifold rules.  ref: get_rules_subm, src/sphconv/rules.cu:326-390.
 *   d_rules      int32 [NTile, KV, 2, tile_n_max]  (may be null: only the neighbour tables are produced)
 *   d_rule_size  int32 [NTile, KV]                  (may be null together with d_rules)
 *   d_nbr        int32 [KV, nnz]: d_nbr[k][o] = input row paired with output row o at offset k, or -1 (may be null)
 *   fill_unused  != 0: entries of d_rules past rule_size are set to -1 as the reference does (rules.cu:364-366)
 *   d_scratch    sph_rules_subm_scratch_bytes(g, nnz) bytes (0 for sparse inputs: then it may be null); holds a
 *                per-column depth-bitmask index of the input, built when columns are long
 * The pair multiset of every (tile,k) list equals the reference's; the order inside a list is unspecified
 * there (atomics) and deterministic here. */
int64_t sph_rules_subm_scratch_bytes(const sph_geom* g, int64_t nnz);
int sph_rules_subm(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* g,
                   void* d_scratch, int32_t tile_n_max, int32_t* d_rules, int32_t* d_rule_size, int32_t* d_nbr,
                   int fill_unused, int32_t* d_status, void* stream);

/* Same operation as sph_rules_subm, for callers that must not allocate device memory: plug-ins running inside
 * a host application that owns the allocator, real-time loops with a no-malloc rule, or language runtimes
 * whose buffers cannot be handed out as scratch.  It has no
 * counterpart in the reference (whose ops allocate freely through ATen).  The scratch (the per-column depth
 * index built for inputs with long columns) is a fixed array inside the library of
 * SPH_RULES_SUBM_STATIC_SCRATCH_BYTES bytes; every device that loads the library keeps that much memory
 * reserved until the process exits.  Inputs that would need more are rejected with SPH_ERR_LIMIT and a
 * message naming both sizes (sph_rules_subm_scratch_bytes() tells the need in advance).  The function never
 * calls cudaMalloc / cudaFree or any allocating routine.
 *  - The first call on each device looks up the array's device address; make that call outside of any stream
 *    capture, with the device current.
 *  - All calls on a device share the one array: the index is cleared and rebuilt by every call, and two calls
 *    whose kernels can overlap on the GPU (different streams, no ordering between them) race on it. */
#define SPH_RULES_SUBM_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int sph_rules_subm_static(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* g,
                          int32_t tile_n_max, int32_t* d_rules, int32_t* d_rule_size, int32_t* d_nbr,
                          int fill_unused, int32_t* d_status, void* stream);

/* Strided ("regular") sparse conv, step 1: output sparsity pattern.
 * ref: get_rules, src/sphconv/rules.cu:405-462 (prepareGridKernel + the cumsum/roll scans).
 *   d_scratch   sph_rules_strided_scratch_bytes(g, nnz) bytes; must be kept untouched until step 2 has run
 *   d_oz_ptr    int32 [B,oH,oW], inclusive prefix like z_ptr
 *   d_out_nnz   int32 [1] on the device (= oz_ptr[-1])
 *   h_out_nnz   optional host pointer: when non-null the call synchronises `stream` and stores the
 *               count there (the same device->host read the reference does at rules.cu:461).  The kernel
 *               hands the count over through a word of mapped pinned host memory, not a memcpy, so the read
 *               does not queue behind bulk copies on the copy engines; the first such call on a device
 *               allocates 1 KiB of pinned host memory that lives until the process ends. */
int64_t sph_rules_strided_scratch_bytes(const sph_geom* g, int64_t nnz);
int sph_rules_strided_count(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* g,
                            void* d_scratch, int32_t* d_oz_ptr, int32_t* d_out_nnz, int32_t* h_out_nnz,
                            void* stream);
/* The same without the synchronisation: enqueues step 1 and returns in *h_count_word the address of the mapped host
 * word the count will be written to; it may be read once work enqueued on `stream` up to this call has completed
 * (e.g. after cudaEventSynchronize on an event recorded right after the call).  Lets a caller enqueue other work
 * behind step 1 - the convolution of the layer before - so that the GPU is busy during the host's round trip.
 * At most 256 such words per device are in use at a time (a ring): read the count before 255 further calls. */
int sph_rules_strided_count_async(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* g,
                                  void* d_scratch, int32_t* d_oz_ptr, int32_t* d_out_nnz,
                                  const int32_t** h_count_word, void* stream);

/* Strided sparse conv, step 2: output depth indices, rules and neighbour tables.
 * ref: getOzIndicesAndRulesKernel, src/sphconv/rules.cu:156-228,465-485.  Output rows are numbered in
 * ascending (b,oX,oY,oZ) exactly as rules.cu:434-443 numbers them.
 *   d_oz_idx  int32 [out_nnz]
 *   d_nbr     int32 [KV, out_nnz]  input row per (offset, output row) or -1          (may be null)
 *   d_nbr_t   int32 [KV, nnz]      output row per (offset, input row) or -1, for dgrad (may be null) */
int sph_rules_strided_fill(const int32_t* d_z_idx, const int32_t* d_z_ptr, int64_t nnz, const sph_geom* g,
                           const void* d_scratch, const int32_t* d_oz_ptr, int64_t out_nnz,
                           int32_t tile_n_max, int32_t* d_oz_idx, int32_t* d_rules, int32_t* d_rule_size,
                           int32_t* d_nbr, int32_t* d_nbr_t, int fill_unused, int32_t* d_status, void* stream);

/* The reference-format pair lists of a rule set from its finished neighbour table: what sph_rules_subm /
 * sph_rules_strided_fill write into d_rules / d_rule_size, as a step of its own, so that a caller whose convolution
 * reads only the table can call those with d_rules = NULL and run this step on another stream, beside the convolution.
 *   d_oz_ptr   int32 [B,oH,oW] of the OUTPUT tensor (z_ptr itself for a submanifold layer)
 *   d_nbr      int32 [KV, out_nnz]   tile_n_max, d_rules, d_rule_size, fill_unused: as for sph_rules_subm
 * Lists come out in ascending output row per batch, whatever the order inside the columns.
 * With d_rules = NULL only d_rule_size is written: the exact length of every list.  Its maximum is the tile_n_max
 * that cannot overflow (the reference sizes the lists with a heuristic, rules.cu:21-28, and drops pairs silently
 * when it is too small, rules.cu:217-224): count, read the maximum, allocate, call again. */
int sph_rule_lists(const int32_t* d_oz_ptr, const sph_geom* g, int64_t out_nnz, const int32_t* d_nbr,
                   int32_t tile_n_max, int32_t* d_rules, int32_t* d_rule_size, int fill_unused, int32_t* d_status,
                   void* stream);

/* Neighbour tables from a reference-format rules tensor (for rules that did not come from this library).
 * ref: the consumer side of the format, include/sphconv/iterator.cu.h:147-181 (reads rules[t][k][0|1][v], v < ruleSize).
 *   d_nbr   int32 [KV, out_rows] (may be null)   d_nbr_t int32 [KV, in_rows] (may be null) */
int sph_rules_to_nbr(const int32_t* d_rules, const int32_t* d_rule_size, int32_t n_tile, int32_t kv,
                     int32_t tile_n_max, int64_t in_rows, int64_t out_rows, int32_t* d_nbr, int32_t* d_nbr_t,
                     int32_t* d_status, void* stream);

/* ---- convolution ------------------------------------------------------------------------------ */

/* Weight image for the tensor-core kernels.  d_weight is [KV, K, N] row-major in `dtype`
 * (K = channels of the gathered rows, N = channels produced).  The packed image has
 * sph_packed_weight_bytes() bytes. */
int64_t sph_packed_weight_bytes(int dtype, int32_t kv, int32_t k_ch, int32_t n_ch);
int sph_pack_weight(const void* d_weight, int dtype, int32_t kv, int32_t k_ch, int32_t n_ch, void* d_packed,
                    void* stream);

/* 1 when sph_conv_gather runs the tcgen05 kernel for this combination, 0 when it runs a CUDA-core kernel. */
int sph_conv_uses_tensor_cores(int dtype, int32_t k_ch, int32_t n_ch);
/* Which CUDA-core kernel runs when the tensor-core kernels do not take the combination (27 offsets assumed, operands
 * 16-byte aligned): 1 = the pair-compacting kernel for sparse levels (rows of 4 / 8 / 16 / 32 channels in and out, the
 * fp32 filter within its shared-memory limit), 0 = the row-walking kernel (any shape).  No reference counterpart. */
int sph_conv_uses_pair_kernel(int dtype, int32_t k_ch, int32_t n_ch);
/* Which kernel sph_conv_wgrad runs for the combination (27 offsets assumed, operands 16-byte aligned): 1 = tcgen05,
 * 2 = the pair-compacting CUDA-core kernel (narrow rows, small fp32 layers), 0 = the general CUDA-core kernel.
 * No reference counterpart. */
int sph_conv_wgrad_kernel(int dtype, int32_t k_ch, int32_t n_ch);

/* out[r,:] = epilogue( sum_k rows[ nbr[k][r], : ] @ weight[k] )   for r in [0, n_out)
 * forward: ref rule_conv, src/sphconv/rule_conv.cu:286-336 (rows = feature, nbr = d_nbr, weight [KV,iC,oC]).
 * dgrad:   ref rule_conv_d_feature, src/sphconv/rule_conv.cu:520-575 (rows = d_out, nbr = d_nbr_t,
 *          weight = the [KV,oC,iC] transpose the reference's caller passes, sphconv/functional.py:70-74).
 *   d_rows      [n_rows, k_ch] in `dtype`
 *   d_weight    [KV, k_ch, n_ch] in `dtype` (CUDA-core kernel) ; d_packed: image from sph_pack_weight (tensor-core
 *               kernel; may be null, then the CUDA-core kernel runs)
 *   d_nbr       int32 [KV, n_out]
 *   flip_k      != 0: offset k reads table row KV-1-k (dgrad of an odd-kernel submanifold layer reuses the
 *               forward table this way)
 *   d_scale/d_bias  float [n_ch] or null; relu != 0 applies max(0,.) ; epilogue = relu(acc*scale + bias)
 *   out_dtype   dtype of d_out [n_out, n_ch]; F32/F16/BF16 accumulate in fp32, I8 accumulates in int32
 *               and converts to float before the epilogue; I8 output rounds to nearest and saturates. */
int sph_conv_gather(const void* d_rows, int dtype, int64_t n_rows, const void* d_weight, const void* d_packed,
                    const int32_t* d_nbr, int64_t n_out, int32_t kv, int32_t k_ch, int32_t n_ch, int flip_k,
                    const float* d_scale, const float* d_bias, int relu, void* d_out, int out_dtype,
                    int32_t* d_status, void* stream);

/* d_weight[k] (+)= rows[nbr[k][r], :]^T @ d_out[r, :] summed over r.
 * ref: rule_conv_d_weight, src/sphconv/rule_conv.cu:469-518 (per-tile partials + torch::sum there; one fp32
 * accumulation buffer here).
 *   d_dweight   float [KV, k_ch, n_ch]; zeroed first when zero_init != 0, else accumulated into */
int sph_conv_wgrad(const void* d_rows, const void* d_dout, int dtype, int64_t n_rows, const int32_t* d_nbr,
                   int64_t n_out, int32_t kv, int32_t k_ch, int32_t n_ch, float* d_dweight, int zero_init,
                   int32_t* d_status, void* stream);

/* ---- tensor operations on either side of the path: COO -> range-voxel, range-voxel <-> dense ----------------------
 * Rows are moved as bytes (`row_bytes` = channels x element size), so every dtype takes the same entry points.
 *
 * sph_init_tensor  ref: init_tensor, src/sphconv/tensor.cu:78-127 (fillGridKernel, the sum/cumsum, reorderFeatureKernel).
 *   d_indices      int32 [nnz,4] = (b, s0, s1, s2) per COO row, 16-byte aligned, no voxel listed twice
 *   d_scratch      sph_init_tensor_scratch_bytes(B, shape) bytes
 *   d_out_feature  [nnz, row_bytes]   d_z_idx int32 [nnz]   d_z_ptr int32 [B,s0,s1] (inclusive prefix)
 *   d_permutation  int32 [nnz]: new row of COO row n (-1 for a row whose coordinates are out of range: status bit
 *                  SPH_STATUS_BAD_INDEX).  Rows of a column come out in ascending depth (the reference's order is the
 *                  arrival order of its atomics).
 * sph_permute_rows ref: init_tensor_backward, tensor.cu:147-162, with gather = 1: d_dst[n] = d_src[permutation[n]];
 *                  gather = 0 is the forward reorder d_dst[permutation[n]] = d_src[n].
 * sph_to_dense     ref: to_dense / to_dense_backward, tensor.cu:222-309.  d_dense is [B,s0,s1,s2,row_bytes]; backward = 0
 *                  copies every row to its voxel (the other voxels of d_dense are left as they are, as in the
 *                  reference: the caller zero-fills), backward = 1 copies the voxels' values back into d_rows. */
int64_t sph_init_tensor_scratch_bytes(int32_t B, const int32_t shape[3]);
int sph_init_tensor(const void* d_feature, int32_t row_bytes, int64_t nnz, const int32_t* d_indices, int32_t B,
                    const int32_t shape[3], void* d_scratch, void* d_out_feature, int32_t* d_z_idx,
                    int32_t* d_z_ptr, int32_t* d_permutation, int32_t* d_status, void* stream);
int sph_permute_rows(const void* d_src, int32_t row_bytes, int64_t n_rows, const int32_t* d_permutation, int gather,
                     void* d_dst, void* stream);
int sph_to_dense(void* d_rows, int32_t row_bytes, int64_t nnz, const int32_t* d_z_idx, const int32_t* d_z_ptr,
                 int32_t B, const int32_t shape[3], void* d_dense, int backward, int32_t* d_status, void* stream);

/* Backward of the fused epilogue relu(acc + bias) of sph_conv_gather (an extension: the reference applies no bias or
 * activation).  d_dpre[r][c] = d_out[r][c] > 0 ? d_dout[r][c] : 0 (relu != 0; else a copy) and
 * d_dbias[c] = sum over rows of d_dpre[r][c] (fp32 [channels], overwritten; may be null, as may d_dpre).
 * dtype SPH_F32 / SPH_F16 / SPH_BF16; at most 256 channels. */
int sph_epilogue_backward(const void* d_dout, const void* d_out, int dtype, int64_t n, int32_t channels, int relu,
                          void* d_dpre, float* d_dbias, void* stream);

/* ---- points -> range-voxel tensor (the step in front of the path; the reference does it on the host) -------------
 * Replaces include/point2voxel.h:411-511 (points_to_voxel_3d) with its driver sphconv/utils/voxelize.py:122-219, the
 * transforms of sphconv/utils/coord_transform.py:8-127, the mean of sphconv/vfe.py:223-228 and the init_tensor call
 * behind them, for a batch of scans at once.
 *
 * sph_voxel_transform   d_points float [n, point_stride] (x, y, z, intensity, ...) -> d_sys_points float [n,4] =
 *                       (first, second, third system coordinate, intensity), 16-byte aligned.  `system`:
 *                       0 spherical (r, phi, theta)  1 l-spherical (log r, ...)  2 cylinder (d, phi, z)
 *                       3 l-cylinder  4 hybrid (d, phi, theta)  5 l-hybrid.
 * sph_voxel_grid        cells[i] / range[i], range[3+i]: cell count and low / high bound of system coordinate i
 *                       (angles in radians, logarithms taken for the l- systems: what the reference's transform
 *                       functions return as the system range); max_points kept per voxel (1..64), max_voxels per
 *                       scan, append_mode 0 point features, 1 point features + system coordinates, 2 system
 *                       coordinates + intensity (point2voxel.h:478-503).
 * The tensor has columns (b, c0, c1) = cells of the third and second coordinate and depth c2 = cell of the first:
 * z_ptr is [B, cells[2], cells[1]], z_idx < cells[0] (init_tensor reads coordinate rows this way, tensor.cu:30-33).
 * Points of scan b are rows d_scan_ptr[b] .. d_scan_ptr[b+1]-1 (int32 [B+1], [0] = 0, [B] = n_points); their order is
 * the order of the reference's walk: a voxel keeps its first max_points points, and a scan that would open more than
 * max_voxels voxels loses every point from the one that would open voxel max_voxels + 1.
 *
 * sph_voxelize_count    fills d_z_ptr and the scratch, writes the row count to *h_nnz (synchronises the stream).
 * sph_voxelize_fill     d_feature float [nnz, sph_voxel_feature_count(point_stride, append_mode)] = mean of the kept
 *                       points; d_z_idx int32 [nnz]; optional d_coordinates int32 [nnz,4] = (b, c0, c1, c2), 16-byte
 *                       aligned, and d_num_points int32 [nnz] (kept points per voxel).  Rows are in range-voxel order
 *                       (ascending b, c0, c1, c2), not in the reference's first-come order. */
typedef struct sph_voxel_grid {
  int32_t B;
  int32_t cells[3];
  float range[6];
  int32_t max_points;
  int32_t max_voxels;
  int32_t append_mode;
} sph_voxel_grid;

int sph_voxel_transform(const float* d_points, int32_t point_stride, int64_t n_points, int system,
                        float* d_sys_points, void* stream);
int sph_voxel_feature_count(int32_t point_stride, int append_mode);
int64_t sph_voxelize_scratch_bytes(const sph_voxel_grid* grid, int64_t n_points);
int sph_voxelize_count(const float* d_sys_points, const int32_t* d_scan_ptr, int64_t n_points,
                       const sph_voxel_grid* grid, void* d_scratch, int32_t* d_z_ptr, int32_t* h_nnz, void* stream);
int sph_voxelize_fill(const float* d_points, int32_t point_stride, const float* d_sys_points,
                      const int32_t* d_scan_ptr, int64_t n_points, const sph_voxel_grid* grid, const void* d_scratch,
                      int64_t nnz, float* d_feature, int32_t* d_z_idx, int32_t* d_coordinates, int32_t* d_num_points,
                      void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPHCONV_B200_H_ */
