/*
 * robocache_b200.h — C ABI of the B200 (sm_100a) preprocessing library.
 *
 * One shared object, plain pointers and sizes, no torch types.  Each entry point names
 * the reference interface it replaces (paths are relative to the reference project).
 *
 * Conventions
 *   - All data pointers are DEVICE pointers on `device`, unless a name ends in _host.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *     The operators only enqueue work; they never synchronise and never allocate device memory
 *     (rc_peer_alloc / rc_peer_open are set-up calls, not operators).
 *     (rc_bulk_wait_timeouts, a diagnostic, copies a counter back and therefore synchronises.)
 *   - Tensors are dense row-major.  Timestamps are fp32.
 *   - Every function returns an rc_status (0 = ok).  rc_strerror() names a code;
 *     rc_last_cuda_error() gives the cudaError_t behind RC_ERR_CUDA for this thread.
 *   - The library is re-entrant.  State kept between calls: the switches of rc_set_option, a
 *     per-device record of shared-memory limits already raised, and the counter array of
 *     rc_voxelize_mean_static (see there).
 */
#ifndef ROBOCACHE_B200_H
#define ROBOCACHE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RC_ABI_VERSION 1

/* exported symbols (the library is built with hidden default visibility) */
#if defined(__GNUC__)
#define RC_API __attribute__((visibility("default")))
#else
#define RC_API
#endif
#define RC_MAX_STREAMS 8

typedef enum rc_status {
    RC_OK = 0,
    RC_ERR_NULL_POINTER = 1,   /* a required pointer is NULL */
    RC_ERR_BAD_SHAPE = 2,      /* negative size, S == 0 with T > 0, too many streams, ... */
    RC_ERR_BAD_DTYPE = 3,      /* dtype is not RC_DTYPE_F32 / RC_DTYPE_BF16 */
    RC_ERR_BAD_ALIGNMENT = 4,  /* a pointer is not aligned to its element size */
    RC_ERR_BAD_MODE = 5,       /* unknown voxel mode, or features missing for mean mode */
    RC_ERR_CUDA = 6,           /* a CUDA runtime call failed; see rc_last_cuda_error() */
    RC_ERR_TOO_LARGE = 7,      /* a size exceeds what the kernels index (see each call) */
    RC_ERR_BAD_DEVICE = 8,     /* device index out of range */
    RC_ERR_BAD_VALUE = 9       /* voxel_size <= 0 or not finite */
} rc_status;

typedef enum rc_dtype { RC_DTYPE_F32 = 0, RC_DTYPE_BF16 = 1 } rc_dtype;

/* numbering of the reference's VoxelMode, robocache/csrc/cuda/voxelize_kernel.cu:20-25 */
typedef enum rc_voxel_mode {
    RC_VOXEL_COUNT = 0,        /* int32 points per voxel */
    RC_VOXEL_OCCUPANCY = 1,    /* int32 0/1 */
    RC_VOXEL_MEAN = 2,         /* fp32 [.., F] feature mean + int32 counts */
    RC_VOXEL_MAX = 3,          /* fp32 [.., F] feature maximum, empty voxels 0 */
    RC_VOXEL_OCCUPANCY_U8 = 4  /* uint8 0/1 (harness format; payload of the multi-GPU max-reduce) */
} rc_voxel_mode;

/* flags of rc_voxelize */
#define RC_VOXEL_ZERO_INIT   1u  /* clear grid (and counts) on `stream` before binning */
#define RC_VOXEL_NO_NORMALIZE 2u /* mean mode: leave feature SUMS in grid (multi-GPU partials) */
#define RC_VOXEL_WARP_AGGREGATE 4u /* merge equal voxel ids inside a warp before the atomic */
#define RC_VOXEL_SPARSE_OCCUPANCY 8u /* rc_voxel_sparse_merge, count mode: store 1 for every received voxel instead of adding its count */

/* one timestamped feature stream: data [B,S,D] (dtype of the call), times [B,S] fp32 */
typedef struct rc_stream_desc {
    const void*  data;
    const float* times;
    int64_t      S;
    int64_t      D;
} rc_stream_desc;

/*
 * Timestamp-aligned resampling: out[b,t,:] = lerp of the two source rows that bracket
 * target_times[b,t] (lower-bound search, clamped at both ends).
 * Replaces launch_resample_bf16 / launch_resample_fp32
 * (robocache/csrc/cuda/resample_kernel.cu:127-174) behind
 * resample_trajectories_cuda (robocache/csrc/cpp/resample_ops.cpp:31-90).
 * src [B,S,D], source_times [B,S], target_times [B,T], out [B,T,D]; out dtype = dtype.
 * Limits: S and T below 2^31; S >= 1 when T > 0.
 */
RC_API int rc_resample(const void* src, const float* source_times, const float* target_times, void* out,
                int64_t B, int64_t S, int64_t T, int64_t D, int dtype, int device, void* stream);

/*
 * Resampling of variable-length items without padding.  The source rows of all items are packed
 * back to back: src_rows [sum S_b, D], source_times [sum S_b], and item b owns rows
 * [row_offsets[b], row_offsets[b+1]) (row_offsets: B+1 int64 on the device, ascending).  max_len is
 * an upper bound of the item lengths (host value; it sizes the shared-memory staging): an item longer than
 * max_len is cut to its first max_len rows, and an item whose offsets do not ascend counts as empty.  Every
 * row_offsets[b] must lie inside the packed rows (the library does not know their number).
 * The result equals padding every item to a common length by repeating its last step — what the
 * reference's loader does before batching (robocache/python/robocache/datasets/rtx_loader.py:214-221)
 * — and calling rc_resample, without materialising the padded batch.  Items with no rows yield zeros.
 */
RC_API int rc_resample_ragged(const void* src_rows, const float* source_times, const int64_t* row_offsets,
                              int64_t max_len, const float* target_times, void* out, int64_t B, int64_t T,
                              int64_t D, int dtype, int device, void* stream);

/*
 * N-stream temporal fusion in one launch: every stream is resampled to target_times and
 * written into its column slice of out [B,T,sum(D_k)] (slice order = stream order).
 * Replaces multimodal_fusion_cuda (robocache/csrc/cuda/multimodal_kernel.cu:201-251) behind
 * fuse_multimodal_cuda (robocache/csrc/cpp/multimodal_ops.cpp:28-119); n_streams = 3 there.
 */
RC_API int rc_fuse(const rc_stream_desc* streams, int n_streams, const float* target_times, void* out,
            int64_t B, int64_t T, int dtype, int device, void* stream);

/*
 * rc_resample / rc_fuse with explicit row strides for the timestamp tensors, in floats: the distance
 * between the time rows of consecutive batch items.  0 means one row shared by the whole batch — what
 * `linspace(...).expand(B, -1)` is in the reference's examples and tests — so such views need no
 * materialised copy; otherwise the stride must be at least the row length.  Feature data and the output
 * stay dense.  No counterpart in the reference (its bindings copy, or misread, expanded time tensors).
 */
RC_API int rc_resample_strided(const void* src, const float* source_times, int64_t source_time_stride,
                               const float* target_times, int64_t target_time_stride, void* out, int64_t B,
                               int64_t S, int64_t T, int64_t D, int dtype, int device, void* stream);
RC_API int rc_fuse_strided(const rc_stream_desc* streams, const int64_t* time_strides, int n_streams,
                           const float* target_times, int64_t target_time_stride, void* out, int64_t B,
                           int64_t T, int dtype, int device, void* stream);

/*
 * Bracket rows and weights only (no feature traffic): left/right int32 [B,T], weight fp32 [B,T].
 * Plays the role of compute_all_indices
 * (robocache/kernels/cutlass/trajectory_resample_bulk.cu:37-95); used for the bit-exact
 * bracket check.  Any of the three outputs may be NULL.
 */
RC_API int rc_resample_brackets(const float* source_times, const float* target_times, int64_t B, int64_t S,
                         int64_t T, int32_t* left, int32_t* right, float* weight, int device,
                         void* stream);

/*
 * Point-cloud voxelisation.  points [N,3] fp32, features [N,F] fp32 (mean / max modes).
 * A point is binned at floor((p - grid_min) / voxel_size) per axis (fp32, IEEE) and dropped
 * if any axis falls outside the grid; flat voxel id = vz*gx*gy + vy*gx + vx.
 *   grid   : int32 [gx*gy*gz] (count, occupancy), uint8 (occupancy_u8), fp32 [gx*gy*gz*F] (mean, max)
 *   counts : int32 [gx*gy*gz], required for mean mode, ignored otherwise
 * Replaces voxelize_cuda (robocache/csrc/cuda/voxelize_kernel.cu:210-277) behind
 * voxelize_pointcloud_cuda (robocache/csrc/cpp/voxelize_ops.cpp:31-133).
 * Limits: gx*gy*gz*max(F,1) below 2^40; each grid extent below 2^24.
 */
RC_API int rc_voxelize(const float* points, const float* features, void* grid, int32_t* counts, int64_t N,
                int32_t F, const float grid_min_host[3], float voxel_size,
                const int32_t grid_size_host[3], int mode, uint32_t flags, int device, void* stream);

/*
 * rc_voxelize with an optional device scratch buffer.  Mean mode on grids whose accumulators do not
 * fit in L2 then runs in phases that keep the atomics L2-resident: with four feature channels the
 * points are first bucketed by slab of the grid into (voxel id, feature row) records in the scratch
 * and the slabs are then accumulated one after the other from those records; with other widths the
 * voxel ids are written once to the scratch and several passes each scatter into one slab.  Results
 * are the same as rc_voxelize's (counts exact, sums equal up to fp32 summation order).
 *   scratch, scratch_bytes : device buffer, 256-byte aligned, at least rc_voxelize_scratch_bytes()
 *                            (about 21.5 bytes per point for four channels, 4 bytes per point for other
 *                            widths, 0 when the plain path applies); may be NULL (plain path).
 * The scratch is only used during the call's own work on `stream`.  No counterpart in the reference.
 */
RC_API uint64_t rc_voxelize_scratch_bytes(int64_t N, int32_t F, const int32_t grid_size_host[3], int mode);
RC_API int rc_voxelize_ex(const float* points, const float* features, void* grid, int32_t* counts, int64_t N,
                          int32_t F, const float grid_min_host[3], float voxel_size,
                          const int32_t grid_size_host[3], int mode, uint32_t flags, void* scratch,
                          uint64_t scratch_bytes, int device, void* stream);

/*
 * Second pass of mean mode on voxels [voxel_begin, voxel_end): grid[v,:] *= 1.0f / counts[v]
 * where counts[v] > 0.  Replaces normalize_mean_kernel
 * (robocache/csrc/cuda/voxelize_kernel.cu:145-163); the range lets each rank of the
 * multi-GPU harness normalise only its own slab after the partial grids are reduced.
 */
RC_API int rc_voxel_normalize(float* grid, const int32_t* counts, int64_t voxel_begin, int64_t voxel_end,
                       int32_t F, int device, void* stream);

/*
 * Batched voxel grids in one launch: points [B,N,3] fp32 -> grid fp32 [B, D, H, W] (occupancy 0/1, density =
 * points per voxel) or [B, D, H, W, F] (feature mean; features [B,N,F] fp32, counts int32 [B, D, H, W] as work
 * space and second output; feature max = max(0, largest feature), what the reference's kernel computes by
 * taking fmaxf against a zero-filled grid, counts unused).  depth/height/width are the z/y/x extents; cell (vz, vy, vx) of item b sits at
 * ((b*D + vz)*H + vy)*W + vx, the item index being folded into the voxel id so that one launch bins the whole batch.
 * Cell arithmetic, dropping of out-of-grid points and flags as rc_voxelize.
 * Replaces voxelize_occupancy / voxelize_density / voxelize_feature_max / voxelize_feature_mean
 * (robocache/kernels/cutlass/point_cloud_voxelization.h:59-136; kernels point_cloud_voxelization.cu:41-300).
 * RC_VOXEL_ZERO_INIT is required for feature max unless the caller cleared the grid.
 * rc_point_cloud_bounds: per item the minimum and maximum of every coordinate, [B,3] each, starting from +-1e10
 * (compute_point_cloud_bounds, point_cloud_voxelization.h:218-227, .cu:386-449).
 */
typedef enum rc_batched_mode {
    RC_BATCHED_OCCUPANCY = 0, RC_BATCHED_DENSITY = 1, RC_BATCHED_FEATURE_MEAN = 2, RC_BATCHED_FEATURE_MAX = 3
} rc_batched_mode;
RC_API int rc_voxelize_batched(const float* points, const float* features, float* grid, int32_t* counts, int64_t B,
                               int64_t N, int32_t F, const float origin_host[3], float voxel_size,
                               const int32_t dhw_host[3], int mode, uint32_t flags, int device, void* stream);
RC_API int rc_point_cloud_bounds(const float* points, float* min_bounds, float* max_bounds, int64_t B, int64_t N,
                                 int device, void* stream);

/*
 * Truncated signed distance grids: points [B,N,3] fp32, normals [B,N,3] fp32 or NULL -> tsdf_grid fp32 [B,D,H,W] and
 * weight_grid fp32 [B,D,H,W]; both are cleared by the call.  For every voxel whose centre
 * origin + (v + 0.5) * voxel_size lies closer than truncation_distance to some point: tsdf = min over those points of
 * distance / truncation_distance, negative when the closest point's normal has a positive dot product with
 * (centre - point), which is the reference's sign rule; weight = the number of such points; other voxels 0 / 0.
 * Distances are single fp32 operations (subtract, multiply, add left to right, sqrt, multiply by 1/truncation).
 * Replaces voxelize_tsdf (robocache/kernels/cutlass/point_cloud_voxelization.h:146-173, kernel .cu:278-376), whose
 * compare-and-swap update keeps the sign of whichever point reached the voxel first; the two agree wherever the
 * reference's result does not depend on thread order.  truncation_distance / voxel_size may not exceed 510.
 */
RC_API int rc_voxelize_tsdf(const float* points, const float* normals, float* tsdf_grid, float* weight_grid, int64_t B,
                            int64_t N, const float origin_host[3], float voxel_size, const int32_t dhw_host[3],
                            float truncation_distance, int device, void* stream);

/*
 * Point exchange for multi-GPU voxelisation: instead of reducing dense partial grids, every rank
 * buckets its points by the rank that owns their voxel, the buckets travel to their owners (an
 * all-to-all by the caller, or written by the partition kernel straight into the owners' memory),
 * and each owner accumulates what it received into its own slab of the grid.  No counterpart in the
 * reference, whose multi-GPU test all-reduces dense grids (robocache/tests/test_multi_gpu.py:76).
 *
 * Parts.  The voxel ids [0, V) are cut into n_groups contiguous ranges of ceil(V / n_groups) ids (one per
 * owner; blocks of z-planes when gz divides), and each range into parts_per_group sub-ranges of
 * ceil(range / parts_per_group) ids.  part = group * parts_per_group + sub; n_groups * parts_per_group <= 64.
 * Sub-ranges let the owner accumulate one L2-sized piece of its slab at a time.
 *
 * rc_voxel_partition_count: points per part.
 *   part_counts : int64 [n_groups * parts_per_group] on the device
 *   scratch     : device buffer of rc_voxel_partition_scratch_bytes(N, n_parts, device) bytes, 16-byte
 *                 aligned; it carries the per-block offsets from the count to the move and must stay
 *                 untouched in between
 * rc_voxel_partition_move: stable partition (input order kept inside a part; dropped points vanish).
 *   Part p's points are written as voxel ids (global, z-major; int32) to dest_ids[p] and as feature rows
 *   (fp32 [., F]) to dest_features[p], from slot dest_start[p] on.  The destinations are device pointers
 *   given in HOST arrays of n_parts entries and may be buffers of other GPUs mapped with rc_peer_open;
 *   the caller guarantees room for the counted points.  With dest_start == NULL the parts are packed
 *   back to back in part order using part_counts_device (then all destinations are normally the same
 *   buffer).  dest_features may be NULL (ids only).  flags: RC_PARTITION_REMOTE_DESTINATIONS when destinations
 *   lie on other GPUs - the kernel then shapes every warp store as one 128-byte-aligned group (see
 *   RC_OPT_PART_ALIGNED_STORE); the bytes written are the same either way.
 * rc_voxel_partition: count + move into local buffers ids_out [N] / features_out [N, F], parts back to
 *   back; only the first sum(part_counts) entries are written.
 * Limits: N at most 2^31 - 4096, gx*gy*gz below 2^31.  Everything runs on `stream`.
 *
 * rc_voxel_scatter_ids: accumulates points given as (voxel id, feature row) into the slab of
 * voxels [id_begin, id_end); ids outside the range (and -1) are ignored.
 *   grid   : first cell of voxel id_begin: int32 [id_end-id_begin] (count, occupancy) or
 *            fp32 [id_end-id_begin, F] (mean);  counts : int32 [id_end-id_begin], mean mode only
 *   mode   : RC_VOXEL_COUNT, RC_VOXEL_OCCUPANCY or RC_VOXEL_MEAN;  flags as rc_voxelize
 *   ids must be 16-byte aligned.
 * rc_voxel_scatter_runs: the same for records that arrive as runs (host arrays run_begin / run_count, in
 *   records; run_pass[r] in [0, n_passes)): the runs of pass 0 are accumulated first, then pass 1, ...
 *   Give every sub-range of the slab its own pass and the atomics of a pass stay within that sub-range.
 */
#define RC_PARTITION_REMOTE_DESTINATIONS 1u
RC_API uint64_t rc_voxel_partition_scratch_bytes(int64_t N, int32_t n_parts, int device);
RC_API int rc_voxel_partition_count(const float* points, int64_t N, const float grid_min_host[3], float voxel_size,
                                    const int32_t grid_size_host[3], int32_t n_groups, int32_t parts_per_group,
                                    int64_t* part_counts, void* scratch, uint64_t scratch_bytes, int device,
                                    void* stream);
RC_API int rc_voxel_partition_move(const float* points, const float* features, int64_t N, int32_t F,
                                   const float grid_min_host[3], float voxel_size, const int32_t grid_size_host[3],
                                   int32_t n_groups, int32_t parts_per_group, void* const* dest_ids,
                                   void* const* dest_features, const int64_t* dest_start,
                                   const int64_t* part_counts_device, uint32_t flags, const void* scratch,
                                   uint64_t scratch_bytes, int device, void* stream);
RC_API int rc_voxel_partition(const float* points, const float* features, int64_t N, int32_t F,
                              const float grid_min_host[3], float voxel_size, const int32_t grid_size_host[3],
                              int32_t n_groups, int32_t parts_per_group, int32_t* ids_out, float* features_out,
                              int64_t* part_counts, void* scratch, uint64_t scratch_bytes, int device, void* stream);
RC_API int rc_voxel_scatter_ids(const int32_t* ids, const float* features, void* grid, int32_t* counts,
                                int64_t M, int32_t F, int64_t id_begin, int64_t id_end, int mode,
                                uint32_t flags, int device, void* stream);
RC_API int rc_voxel_scatter_runs(const int32_t* ids, const float* features, void* grid, int32_t* counts, int32_t F,
                                 int64_t id_begin, int64_t id_end, const int64_t* run_begin,
                                 const int64_t* run_count, const int32_t* run_pass, int32_t n_runs,
                                 int32_t n_passes, int mode, uint32_t flags, int device, void* stream);

/*
 * Point exchange by buckets (mean mode, four feature channels): the multi-GPU form of the slab-ordered run path,
 * with no counting pass and no host synchronisation.  The voxel ids are cut into n_groups owner ranges of
 * ceil(V / n_groups) ids and each range into parts_per_group sub-ranges; n_groups * parts_per_group <= 16.
 * A record pool is a sequence of blocks of rc_voxel_bucket_block_records() records (ids int32 and feature rows
 * fp32 [., 4] in two buffers, 128-byte aligned) with a run table uint32 [parts_per_group][pool_blocks] beside it.
 * rc_voxel_bucket_exchange: sorts each 1024-point chunk of the cloud by (owner, sub-range) and stores owner d's
 *   segment of chunk c into block first_block + c of pool d, and the sub-ranges' (first slot, length) into table d.
 *   dest_ids / dest_features / dest_runs are HOST arrays of n_groups device pointers; pool_blocks is the number of
 *   blocks of every pool (the row length of its table).  Two layouts are in use: the owners' pools in the owners'
 *   memory, mapped here with rc_peer_open (plain stores over NVLink; first_block = rank * chunks, pool_blocks =
 *   n_groups * chunks), or n_groups pools in this GPU's own memory that the owners read later (first_block = 0,
 *   pool_blocks = chunks).  N <= chunks * 1024; all `chunks` blocks are written on every call (empty ones as
 *   empty).  Nothing is read from a peer, no multicast.  ctas_per_sm (1..8, 0 = 8) sizes the grid: the kernel's
 *   remote stores are bound by NVLink, not by the SMs, and a small grid (2) leaves SMs to the accumulation of an
 *   earlier slice running on another stream.
 * rc_voxel_scatter_buckets: an owner accumulates the pools of n_sources sources (HOST arrays of device pointers
 *   to ids, feature rows and tables of blocks_per_source blocks each; they may lie in other GPUs' memory and are
 *   then read with plain loads over NVLink) into its slab [id_begin, id_end) of the grid (fp32 [., 4], first cell of
 *   voxel id_begin) and counts, one sub-range after the other; flags as rc_voxelize.  table_row_blocks is the row
 *   length of the sources' run tables (0: blocks_per_source); a larger value lets a "source" be a window of
 *   blocks_per_source blocks inside a bigger pool - a slice of the cloud that has already arrived while the next
 *   slice is still travelling.  With n_sources = 0 the call only clears and / or normalises the slab as flags say.
 * The caller orders writers against readers with a barrier on the stream before and after the exchange call.
 * No counterpart in the reference.
 */
RC_API int32_t rc_voxel_bucket_block_records(int32_t parts_per_group);
RC_API int rc_voxel_bucket_exchange(const float* points, const float* features, int64_t N, const float grid_min_host[3],
                                    float voxel_size, const int32_t grid_size_host[3], int32_t n_groups,
                                    int32_t parts_per_group, int64_t chunks, int64_t first_block, int64_t pool_blocks,
                                    void* const* dest_ids, void* const* dest_features, void* const* dest_runs,
                                    int32_t ctas_per_sm, int device, void* stream);
RC_API int rc_voxel_scatter_buckets(const void* const* pool_ids, const void* const* pool_features, const void* const* runs,
                                    int32_t n_sources, int64_t blocks_per_source, int64_t table_row_blocks,
                                    int32_t parts_per_group, float* grid, int32_t* counts, int64_t id_begin,
                                    int64_t id_end, uint32_t flags, int device, void* stream);

/*
 * Sparse reduction of partial grids (mean mode, four feature channels): when a cloud puts many points into every
 * occupied voxel, a rank that has binned its own points into a private full-size grid (feature sums + counts, not
 * normalised) sends every other rank only the occupied voxels of that rank's slab - 24 bytes per occupied voxel
 * instead of 20 bytes per point.
 * rc_voxel_sparse_send: for each of n_dest (<= 16) voxel ranges [id_begin_host[r], id_end_host[r]) of grid (fp32
 *   [V,4] sums) / counts (int32 [V]), appends (voxel id, sums, count) of every voxel with a non-zero count to record
 *   list r: dest_ids[r] int32 [capacity], dest_sums[r] fp32 [capacity,4], dest_counts[r] int32 [capacity] (HOST
 *   arrays of device pointers; the lists may lie in peer memory and are written with plain stores), in no particular
 *   order; then stores the number of records to *dest_nrec[r].  Records beyond `capacity` are dropped - the stored
 *   number still counts them, and *overflow (int32 on this GPU, may be NULL; set to 1, never cleared by the library)
 *   tells the sender; the owner learns of it in rc_voxel_sparse_merge.  cursors: int32 [n_dest] scratch on this GPU.
 * rc_voxel_sparse_merge: the owner adds the record lists of n_src sources (HOST arrays of device pointers; the
 *   record numbers are read on the device from *src_nrec[i], clamped to capacity) to its slab [id_begin, id_end) of
 *   its own partial grid (grid / counts point at voxel id_begin) and normalises the slab unless flags has
 *   RC_VOXEL_NO_NORMALIZE; a record number above the capacity sets *overflow (int32 on this GPU, may be NULL, not
 *   cleared by this call) to 1: the owner learns by itself that its slab is incomplete.
 * Count mode: grid = NULL in both calls and NULL entries in dest_sums / src_sums - records are (voxel id, count) only;
 * with RC_VOXEL_SPARSE_OCCUPANCY the merge stores 1 for every received voxel (occupancy grids).
 * The lists an owner merges may lie in the sources' own memory (plain loads over NVLink): with one list per rank that
 * holds the occupied voxels of that rank's WHOLE grid, every rank can merge all the others' lists into its own full
 * grid - the result of an all-reduce of the dense partial grids, for the price of the occupied voxels.
 * The caller orders senders against owners with a barrier on the stream between the two calls and before the next
 * send.  No counterpart in the reference.
 */
RC_API int rc_voxel_sparse_send(const float* grid, const int32_t* counts, int32_t n_dest, const int64_t* id_begin_host,
                                const int64_t* id_end_host, int64_t capacity, void* const* dest_ids,
                                void* const* dest_sums, void* const* dest_counts, void* const* dest_nrec,
                                int32_t* cursors, int32_t* overflow, int device, void* stream);
RC_API int rc_voxel_sparse_merge(int32_t n_src, const void* const* src_ids, const void* const* src_sums,
                                 const void* const* src_counts, const void* const* src_nrec, int64_t capacity,
                                 float* grid, int32_t* counts, int64_t id_begin, int64_t id_end, int32_t* overflow,
                                 uint32_t flags, int device, void* stream);

/*
 * Device buffers that the other processes of a node can map, for rc_voxel_partition_move's remote
 * destinations.  rc_peer_alloc allocates `bytes` on `device` (cudaMalloc) and fills the 64-byte CUDA IPC
 * handle to hand to the other processes (the buffer is zero-filled); rc_peer_open maps such a handle into this process on `device`
 * with peer access enabled; rc_peer_close unmaps, rc_peer_free releases (close every mapping first).
 * These are set-up calls: none of them belongs on a hot path.  No counterpart in the reference.
 */
RC_API int rc_peer_alloc(uint64_t bytes, int device, void** ptr, unsigned char handle[64]);
/*
 * Barrier among the n (<= 16) GPUs of a node, enqueued on `stream`: work enqueued after it on any of the ranks'
 * streams sees everything the ranks' streams did before it, plain stores into peers' memory included.  flags is a
 * HOST array of n device pointers: rank p's flag array (uint32 [n], from rc_peer_alloc, which zero-fills) as mapped
 * into this process; epoch must grow by one from call to call, the same on every rank.  One 32-thread kernel: each
 * thread stores the epoch into one peer's array (release, system scope) and polls this rank's own array for that
 * peer's (acquire).  The wait is bounded: after poll_limit polls of 0.26 us (0 = 2^25, about 8 s) *status (int32 on this
 * GPU, may be NULL) is set to 1 and the kernel returns - the caller reads it before trusting what follows.
 * Replaces a 4-byte NCCL all-reduce used as a barrier (0.09 ms per barrier on 8 GPUs).  No counterpart in the reference.
 */
RC_API int rc_peer_barrier(void* const* flags, int32_t n, int32_t rank, uint32_t epoch, int32_t* status,
                           int64_t poll_limit, int device, void* stream);
RC_API int rc_peer_open(const unsigned char handle[64], int device, void** ptr);
RC_API int rc_peer_close(void* ptr, int device);
RC_API int rc_peer_free(void* ptr, int device);

/*
 * Mean-mode voxelisation that allocates nothing. No counterpart in the reference: its binding
 * always allocates the counter plane with torch (robocache/csrc/cpp/voxelize_ops.cpp:91-100).
 *
 * For callers that cannot call cudaMalloc: code inside an allocator or memory-pool callback, a
 * control loop that forbids driver allocations once it is running, or a host that owns only the
 * input and output buffers it was given.  The per-voxel counters that mean mode needs live in a
 * fixed array inside the library (RC_STATIC_MAX_VOXELS int32 = 8 MiB, held by every GPU that
 * loads the library until the process exits), so the caller passes only points, features and the
 * fp32 output grid [gx*gy*gz*F]; the counters are not returned.
 *
 *   - gx*gy*gz above RC_STATIC_MAX_VOXELS is rejected with RC_ERR_TOO_LARGE.
 *   - The grid and the counters are cleared on `stream` by every call.
 *   - All calls on a device share the one counter array: two calls that overlap on the GPU
 *     (different streams, or different threads) race.  Serialise them on one stream.
 *   - The first call on each device looks up the array's device address; make that call before
 *     any stream capture begins.  Under CUDA's lazy module loading that first call (or the first
 *     launch of any kernel of this library on the device) is also what makes the driver place the
 *     library's image, the 8 MiB array included, on the GPU: a caller with a no-allocation region
 *     makes one warm-up call before entering it.
 *   - Apart from that one-time module load, no cudaMalloc, cudaFree or other allocating routine is
 *     called, by this function or on its behalf.
 * Results equal rc_voxelize(..., RC_VOXEL_MEAN, RC_VOXEL_ZERO_INIT) up to fp32 summation order.
 */
#define RC_STATIC_MAX_VOXELS (1 << 21)
RC_API int rc_voxelize_mean_static(const float* points, const float* features, float* grid, int64_t N,
                                   int32_t F, const float grid_min_host[3], float voxel_size,
                                   const int32_t grid_size_host[3], int device, void* stream);

/*
 * Process-wide switches, for tests and profiling.  RC_OPT_BLOCK_KERNEL (default 1): let
 * rc_resample / rc_fuse use the TMA-staged kernel when the shapes qualify; 0 forces the
 * row-gather kernel.  Both kernels produce identical bits.
 * RC_OPT_VOXEL_PASSES (default 0 = choose automatically): number of slab passes of the count /
 * mean / max scatter; each pass re-reads the coordinates but scatters into only 1/passes of the
 * grid, which keeps the touched part of large sparse grids resident in L2.
 * RC_OPT_PART_ALIGNED_STORE: how rc_voxel_partition_move lays its warp stores.  1 (default): when the call
 * carries RC_PARTITION_REMOTE_DESTINATIONS every warp store covers one 32-record-aligned group of the destination
 * (full 128-byte lines; records that do not fill a group yet wait in shared memory for the next chunk),
 * otherwise the sorted chunk is written as it lies; 0: never aligned; 2: always aligned.  All produce
 * identical bytes.
 * RC_OPT_BULK_WAIT_LIMIT (default -1 = built-in limit of 2^22 polls): how many times the TMA-staged kernel
 * polls for its bulk copies before it gives up, counts the event (rc_bulk_wait_timeouts) and fetches the same
 * bytes with ordinary loads.  0 makes every CTA give up at once - the way to exercise that fallback without
 * anything going wrong on the GPU; results are identical.  After the fallback a CTA still waits, with the
 * built-in limit, for its copies to land before it exits.
 * RC_OPT_GATHER_BULK_STAGE (default 1): the row-gather kernel stages its timestamp rows with bulk asynchronous
 * copies (TMA; one per row, issued by one thread, completed on an mbarrier with the same bounded wait and
 * fallback as the staged kernel) where every row is a whole number of 16-byte pieces at a 16-byte aligned
 * address; 0: ordinary loads by all threads.  Same bits either way; 205.0 against 206.1 us on the bf16
 * B=4096 S=500 D=256 T=250 case.
 * RC_OPT_BUCKET_BULK_STORE (default 1): the bucket kernel (mean mode's run path in rc_voxelize_ex, and
 * rc_voxel_bucket_exchange) sends every sorted chunk - every owner's segment of it - from shared memory with bulk
 * asynchronous copies (TMA stores issued by one thread per destination) instead of ordinary stores by all threads.
 * Same bytes either way; 2.17 against 2.21 ms on the 2^26-point mean case.
 * RC_OPT_SCATTER_OVERLAP (default 1): the per-slab accumulation launches of mean mode's run path are issued as
 * programmatic dependent launches, so that a slab's first CTAs fill the SMs the previous slab's last CTAs leave
 * idle (the launches depend on one another's order for L2 locality only, not on results); 0: ordinary launches.
 * No counterpart in the reference.
 */
#define RC_OPT_BLOCK_KERNEL 0
#define RC_OPT_SCATTER_OVERLAP 6
#define RC_OPT_BUCKET_BULK_STORE 5
#define RC_OPT_GATHER_BULK_STAGE 4
#define RC_OPT_BULK_WAIT_LIMIT 3
#define RC_OPT_VOXEL_PASSES 1
#define RC_OPT_PART_ALIGNED_STORE 2
RC_API int rc_set_option(int option, int value);

/*
 * Number of CTAs, since the library was loaded on `device`, whose bounded wait for a bulk
 * (TMA) copy ran out and which fetched their inputs with ordinary loads instead.  Expected
 * to stay 0; synchronises the device.  No counterpart in the reference.
 */
RC_API int rc_bulk_wait_timeouts(int device, unsigned int* count_host);

RC_API const char* rc_strerror(int status);
RC_API int rc_last_cuda_error(void);
RC_API int rc_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ROBOCACHE_B200_H */
