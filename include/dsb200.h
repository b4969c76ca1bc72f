/*
 * dsb200 -- C ABI of the sm_100a Gaussian-splat rasterizer.
 *
 * Plain pointers and sizes only: every buffer is caller-owned DEVICE memory unless a parameter says
 * "host"; every call enqueues its work on `stream` (a cudaStream_t passed as void*) and returns an int
 * status (0 = ok, negative = error, text from dsb_last_error()).  The library keeps no state between
 * calls except the last error string, a launch counter and one status word per device (see
 * dsb_take_device_status).
 *
 * Each entry point replaces one function of the reference's torch extension `ds_splat_cuda`
 * (bound in cpp/rasterizer_python.cpp:3-23); the comment above it cites that function.
 */
#ifndef DSB200_H_
#define DSB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSB_OK 0
#define DSB_ERR_INVALID_ARGUMENT (-1)
#define DSB_ERR_CUDA (-2)
#define DSB_ERR_WORKSPACE_TOO_SMALL (-3)
#define DSB_ERR_TOO_MANY_PAIRS (-4)
#define DSB_ERR_DEVICE_WAIT_EXPIRED (-5)
#define DSB_ERR_UNSUPPORTED (-6)
/* Positive values of the device status word are notes, not errors: results are valid. */
#define DSB_STATUS_COPY_WAIT_FELL_BACK 1 /* a preprocess block gave up waiting for its bulk copies and read its rows with plain loads */

/* The reference never emits (tile, splat) pairs for the splat with the highest index: it takes the
 * exclusive prefix of the last splat as the pair total (cpp/rasterizer_torch.cu:97-104).  With this
 * flag set the library reproduces that, which bit-exact parity of the sorted lists needs. */
#define DSB_FLAG_DROP_LAST_SPLAT 1
/* Pairs only for the tiles a splat can contribute to.  The reference pairs a splat with every tile of the
 * square around its 3-sigma circle (cpp/rasterizer_kernels.cu:233-250); most of those pairs end in the
 * per-pixel "alpha < 1/255" skip.  With this flag the tile rectangle kept in the record and counted in
 * tiles_touched is the square intersected with the bounding box of the region where opacity * exp(-q) can
 * reach 1/255, so the pair list, K and the ranges are those of a SUBSET of the reference's list; image, radii
 * and gradients are unchanged (the dropped pairs never pass the per-pixel test).  Off: lists, counts and
 * ranges are exactly the reference's. */
#define DSB_FLAG_TIGHT_TILES 2

/* How the fused render (dsb_forward_plan / dsb_forward_render / dsb_plan_views) gets from depth-ordered splats to the
 * sorted pair list.  Off: it writes the k pairs in depth order and sorts them on their tile bits (two radix passes at
 * 1080p and 4K).  On, for images of at most 256 x 509 tiles: "row binning" -- one 8-byte item per (splat, tile row),
 * sorted by row, then ONE pass over the k pairs that expands, ranks and places them.  Same list either way.  Measured
 * on B200: row binning is the faster of the two when splats are wide (row items under about an eighth of the pairs,
 * as in the high-overlap stress configuration) and the slower one on the 1M and 6M clouds, whose splats are about 3.5
 * tiles wide; hence off by default.  Every view of one call, and the plan and render calls of one view, must agree. */
#define DSB_FLAG_ROW_BINNING 4

/* Bands.  One view may hold at most DSB_MAX_PAIRS - 1 pairs (positions in the list are 32-bit, as in the reference,
 * whose own 32-bit pair count wraps at 2^31, cpp/rasterizer_torch.cu:101-107).  A view with more is rendered in BANDS of
 * tile rows: with tile_row_band set, the preprocess clips every splat's tile rectangle to the band, so plan, pair list
 * and ranges cover only the band's pairs, the forward blend writes only the band's pixels, and the backward blend only
 * adds the band's contributions to grad_acc (dsb_backward_blend with keep_grad_acc).  The bands of a view tile the image,
 * share image, final_T, final_idx and grad_acc, and each keeps its own pair list and ranges until the backward.
 * Rendering in bands changes nothing in the image; gradients agree up to the order of the atomic sums. */
#define DSB_RECORD_FLOATS 12  /* packed per-splat record: 3 x float4, see DsbCamera notes below   */
#define DSB_MAX_BATCH_VIEWS 8 /* views one dsb_geometry_backward_views call takes                  */
#define DSB_GRAD_FLOATS 12    /* per-splat accumulator row written by dsb_blend_backward          */
#define DSB_MAX_PAIRS ((int64_t)1 << 30)

/*
 * Camera and render settings: the fields of the reference's TorchRasterizationSettings
 * (cpp/ds_cuda_rasterizer/rasterizer_torch.hpp:7-22).  The struct lives in HOST memory; the four
 * pointers inside it point to DEVICE memory (as the reference's settings tensors do).
 *   matrices_transposed = 0: viewmatrix/projmatrix are row-major [R|t] and P*V, the form the reference
 *                            kernels read after ds_splat/rasterizer.py:147-148 transposed them;
 *   matrices_transposed = 1: they are still in the caller's (graphdeco) transposed form, and the
 *                            kernels index them accordingly -- saves the two transposes per call.
 * prefiltered / debug of the reference are accepted by the Python layer and, like there, unused.
 */
typedef struct DsbCamera {
    int32_t image_height;
    int32_t image_width;
    float tanfovx;
    float tanfovy;
    float scale_modifier;
    int32_t sh_degree;            /* active degree, 0..3                                          */
    int32_t max_sh_degree;        /* degree the shs tensor is laid out for: (max+1)^2 rows of 3   */
    int32_t matrices_transposed;
    int32_t flags;                /* DSB_FLAG_*                                                   */
    int32_t tile_row_band;        /* 0: the whole image; else (first tile row) | (one past the last) << 16: only this band of
                                     tile rows gets pairs and pixels, see "bands" below                                */
    const float* viewmatrix;      /* device, 16 floats */
    const float* projmatrix;      /* device, 16 floats */
    const float* campos;          /* device, 3 floats  */
    const float* bg;              /* device, 3 floats, or NULL for black                          */
} DsbCamera;

const char* dsb_last_error(void);
int32_t dsb_version(void);
/* Number of kernels this library has launched in this process (monotonic). */
int64_t dsb_launch_count(void);

/* ---- device status word (no reference counterpart: the reference checks no CUDA error after any launch and
 * defines a CUDA_CALL macro it never uses, cpp/gsplat/config.h:6-17) ------------------------------------
 * Every wait inside a kernel of this library (the look-back of the sorts and of the scan, the wait for bulk
 * copies) is bounded: when it runs out the kernel records DSB_ERR_DEVICE_WAIT_EXPIRED in a per-device status
 * word and finishes, so a logic error or a lost predecessor can never hang the GPU -- but the lists such a
 * kernel wrote are incomplete and everything rendered from them since is invalid.  The word is sticky until the
 * host takes it:
 *   - dsb_plan_pairs / dsb_forward_plan / dsb_plan_views / dsb_plan_totals_views, which synchronise the
 *     stream anyway to read the pair count, fetch it in the same synchronisation and return
 *     DSB_ERR_DEVICE_WAIT_EXPIRED when an earlier call on the device (for instance the tile sort inside the
 *     previous dsb_forward_render) recorded it;
 *   - dsb_take_device_status() synchronises `stream`, writes the word to *status_host (HOST int, may be NULL),
 *     clears it, and returns DSB_OK, or the error code the word held.  Callers of the sort entry points, which
 *     never synchronise by themselves, call it after their own synchronisation point.
 * Positive values (DSB_STATUS_*) are notes about a slower path taken with valid results; they are reported
 * through *status_host only (the plan calls leave them in place). */
int dsb_take_device_status(int32_t* status_host, void* stream);

/* ---- test hooks for the bounded waits (no reference counterpart) ----------------------------------------
 * Each runs ONE kernel of the normal path on well-formed input in a configuration where one wait can never be
 * satisfied, with a poll limit of a few hundred, so that a test can check that the kernel returns, the status
 * words are set and the host reports DSB_ERR_DEVICE_WAIT_EXPIRED.  Nothing faults or hangs: the starved block
 * gives up after spin_limit polls (1..100000) and finishes like the others.
 *   dsb_debug_expire_scan_wait: the offset scan of dsb_plan_pairs over n >= 2048 splats with the first tile of the
 *       look-back chain left out; workspace as for dsb_plan_pairs (dsb_plan_workspace_bytes(n)), on which
 *       dsb_plan_totals_views(1, n, ...) then reports the expiry.
 *   dsb_debug_expire_sort_wait: one radix pass (end_bit - begin_bit <= 8) of dsb_sort_pairs over k >= 8192 items
 *       with the first tile left out; items_alt receives an incomplete list.  dsb_take_device_status() reports it.
 *   dsb_debug_set_copy_wait_polls: how often the preprocess kernel polls for its bulk copies before it falls back
 *       to plain loads (0 restores the default); with 1 every block falls back, results must not change, and the
 *       status word holds DSB_STATUS_COPY_WAIT_FELL_BACK afterwards. */
int dsb_debug_expire_scan_wait(const DsbCamera* cam, int32_t n, const int32_t* tiles_touched,
                               const uint64_t* depth_keys_sorted, uint32_t* offsets, void* workspace,
                               int64_t workspace_bytes, uint32_t spin_limit, void* stream);
int dsb_debug_expire_sort_wait(uint64_t* items, uint64_t* items_alt, int64_t k, int32_t begin_bit, int32_t end_bit,
                               void* workspace, int64_t workspace_bytes, uint32_t spin_limit, void* stream);
int dsb_debug_set_copy_wait_polls(uint32_t polls);

/* ---- measurement hook: the forward blend with another way of fetching the records (no reference counterpart) -----
 * dsb_blend_forward's kernel fetches a chunk of 32 list entries with three 16-byte loads per lane (variant 0).  The
 * alternatives that were weighed against it stay callable so that the comparison can be repeated and so that a test
 * can check that all of them render the same image bit for bit:
 *   1  every lane asks the bulk copy engine (cp.async.bulk, global -> shared, this GPU's memory only, no multicast)
 *      for its 48-byte record, all of a chunk's copies completing on the warp's mbarrier (bounded wait);
 *   2  a gather pass first writes the records in list order into `scratch` (k x 48 bytes); a chunk is then ONE
 *      contiguous bulk copy of up to 1536 bytes;
 *   3  variant 0 with the cull's per-splat constants (ln(255 opacity) + margin, -b/c) read from a copy of the records
 *      in `scratch` (n x 48 bytes) instead of being recomputed by every warp that meets the splat.
 * tile_order may be NULL. */
int dsb_debug_blend_forward_variant(const DsbCamera* cam, int32_t variant, int32_t n, int64_t k, const float* records,
                                    const uint64_t* sorted_pairs, const int32_t* ranges, float* image, float* final_T,
                                    int32_t* final_idx, const int32_t* tile_order, void* scratch, int64_t scratch_bytes,
                                    void* stream);

/* ---- per-stage device timing (no reference counterpart: the reference times with std::chrono in
 * its tests, tests/rasterizer_test.cpp:112-143) --------------------------------------------------
 * While enabled, every stage inside the calls below is bracketed by a cudaEvent pair on the caller's
 * stream.  dsb_stage_timing_read() waits for the recorded events, writes the summed milliseconds and
 * call counts per stage (arrays of at least dsb_stage_count() entries, HOST memory) and clears them. */
int dsb_stage_timing_enable(int32_t on);
int32_t dsb_stage_count(void);
const char* dsb_stage_name(int32_t stage);
int dsb_stage_timing_read(int32_t stage_count, double* ms_total, int64_t* calls);

/* ---- workspace sizes (host arithmetic only) ------------------------------------------------- */
/* Scratch for dsb_plan_pairs (depth ordering of n splats + scan). */
int64_t dsb_plan_workspace_bytes(int32_t n);
/* Scratch for dsb_sort_pairs / dsb_sort_by_keys over k items (excludes the alternate buffers). */
int64_t dsb_sort_workspace_bytes(int64_t k);
/* Size of the tile_marks grid shared by dsb_forward_plan and dsb_forward_render:
 * (tiles_y + 1) x (tiles_x + 1) int32, rounded up to 256 bytes. */
int64_t dsb_tile_marks_bytes(int32_t image_height, int32_t image_width);

/* ---- stage (a) ------------------------------------------------------------------------------
 * Replaces rasterizer_forward_preprocessing + rasterizer_preprocessing_kernel
 * (cpp/rasterizer_torch.cu:115-168, cpp/rasterizer_kernels.cu:57-161).
 * shs may be NULL when colors_precomp is given; scales/rotations may be NULL when cov3d_precomp is.
 * Outputs: records [n][12] = (x_pix, y_pix, conic_a, conic_b | conic_c, opacity, r, g | b, depth,
 * rect_x, rect_y) with rect_* = (lo | hi << 16) tile bounds as integer bits; radii [n] int32;
 * tiles_touched [n] int32; cov3d [n][6]; depth_keys [n] = (depth bits << 32) | splat id. */
int dsb_preprocess(const DsbCamera* cam, int32_t n, const float* means3d, const float* shs,
                   const float* colors_precomp, const float* opacities, const float* scales,
                   const float* rotations, const float* cov3d_precomp, float* records, int32_t* radii,
                   int32_t* tiles_touched, float* cov3d, uint64_t* depth_keys, void* stream);

/* ---- stage (b), first half ------------------------------------------------------------------
 * Replaces the thrust::exclusive_scan + the two host read-backs of duplicate_keys
 * (cpp/rasterizer_torch.cu:83-104).  Orders the splats by (depth, id) with the radix sort of stage
 * (c), scans tiles_touched in that order and returns the pair total through *k_host (HOST pointer;
 * the call synchronises `stream` once to read it).  depth_keys is sorted in place (depth_keys_alt is
 * an equally sized scratch buffer); offsets [n] receives each ordered splat's first pair position. */
int dsb_plan_pairs(const DsbCamera* cam, int32_t n, const int32_t* tiles_touched, uint64_t* depth_keys,
                   uint64_t* depth_keys_alt, uint32_t* offsets, void* workspace, int64_t workspace_bytes,
                   int64_t* k_host, void* stream);

/* ---- stage (b), second half -----------------------------------------------------------------
 * Replaces calculate_keys_and_indices_kernel (cpp/rasterizer_kernels.cu:252-306).  Writes k packed
 * pairs (tile id << 32 | splat id), splats in (depth, id) order, each rectangle row-major.  k must be the
 * total dsb_plan_pairs returned for these offsets: a splat's pair count is taken as the distance to the next
 * splat's offset, the last one's as k minus its offset (tiles_touched is not read). */
int dsb_emit_pairs(const DsbCamera* cam, int32_t n, int64_t k, const float* records,
                   const int32_t* tiles_touched, const uint64_t* depth_keys_sorted, const uint32_t* offsets,
                   uint64_t* pairs, void* stream);

/* ---- stage (c) ------------------------------------------------------------------------------
 * Replaces sort_by_keys / thrust::sort_by_key (cpp/rasterizer_torch.cu:70-76).
 * dsb_sort_pairs: stable LSD radix sort of k 64-bit words on bits [begin_bit, end_bit); the sorted
 * data ends in `items` when *sorted_in_alt_host (HOST int) is 0, else in `items_alt`.
 * dsb_sort_by_keys: the reference's interface -- (int64 key, int32 value) pairs, keys compared as
 * signed when end_bit == 64 -- sorted on the given bit range; same ping-pong convention. */
int dsb_sort_pairs(uint64_t* items, uint64_t* items_alt, int64_t k, int32_t begin_bit, int32_t end_bit,
                   void* workspace, int64_t workspace_bytes, int32_t* sorted_in_alt_host, void* stream);
int dsb_sort_by_keys(int64_t* keys, int64_t* keys_alt, int32_t* values, int32_t* values_alt, int64_t k,
                     int32_t begin_bit, int32_t end_bit, void* workspace, int64_t workspace_bytes,
                     int32_t* sorted_in_alt_host, void* stream);

/* dsb_sort_pairs_static: dsb_sort_pairs for callers that cannot allocate.  It has no counterpart in
 * the reference (whose sort, thrust::sort_by_key, allocates its temporary storage with cudaMalloc on
 * every call).  Meant for hosts where the library is a guest: a renderer plugged into another engine's
 * frame loop that owns all device memory, or a latency-critical loop in which cudaMalloc -- which stalls
 * the whole device -- is off limits.  The caller passes only the list and an equally sized alternate
 * buffer; the histograms, tile counters and look-back words the sort needs come out of a fixed array
 * compiled into the library (about 4 MB of every GPU that loads it, held until the process exits).
 *   - k may be at most DSB_STATIC_SORT_MAX_ITEMS; larger lists are refused with
 *     DSB_ERR_WORKSPACE_TOO_SMALL and a message naming the limit.
 *   - The call issues memset and kernel launches only: no cudaMalloc, cudaFree or other allocating routine.
 *   - The first call on each device looks up that device's address of the built-in array (the device must
 *     be current); make that first call during start-up, before any stream capture is begun.
 *   - All calls on a device share the one array.  Each call clears what it needs first, so leftovers of
 *     the previous call are harmless, but two calls whose kernels overlap on the GPU (different streams)
 *     would corrupt each other: keep calls on one device ordered.
 * Results are identical to dsb_sort_pairs. */
#define DSB_STATIC_SORT_MAX_ITEMS ((int64_t)1 << 21)
int dsb_sort_pairs_static(uint64_t* items, uint64_t* items_alt, int64_t k, int32_t begin_bit, int32_t end_bit,
                          int32_t* sorted_in_alt_host, void* stream);

/* ---- stage (d) ------------------------------------------------------------------------------
 * Replaces identify_tile_ranges (cpp/rasterizer_torch.cu:23-42, kernel cpp/rasterizer_kernels.cu:
 * 308-323).  `sorted` holds k 64-bit words whose high 32 bits are the tile id (the reference's keys
 * and this library's packed pairs both qualify).  ranges [tiles+1] int32: tile t owns [r[t], r[t+1]).
 * One habit of the reference is kept because the result must be its array bit for bit: it marks the end of a tile
 * only where the next item belongs to another tile and fills the gaps with a running maximum, so when EMPTY tiles
 * follow the last non-empty tile, that tile's end is never marked -- its range comes out empty and its items belong
 * to the final tile, whose end is K.  (The fused render does the same when its pair list is the reference's, i.e.
 * with DSB_FLAG_DROP_LAST_SPLAT and without DSB_FLAG_TIGHT_TILES; otherwise its ranges are a clean partition.) */
int dsb_identify_tile_ranges(const uint64_t* sorted, int64_t k, int32_t image_height, int32_t image_width,
                             int32_t* ranges, void* stream);

/* ---- stage (e) ------------------------------------------------------------------------------
 * Replaces rasterizer_cuda_forward + render_image_kernel (cpp/rasterizer_torch.cu:44-68,
 * cpp/rasterizer_kernels.cu:341-431).  image [H][W][3], final_T [H][W], final_idx [H][W] int32.
 * depth [H][W] may be NULL; when given it receives sum_i z_i alpha_i T_i, the view-space depth of the
 * splats blended like a fourth colour channel (no reference counterpart: the reference returns colour
 * and radii only). */
int dsb_blend_forward(const DsbCamera* cam, const float* records, const uint64_t* sorted_pairs,
                      const int32_t* ranges, float* image, float* final_T, int32_t* final_idx, float* depth,
                      void* stream);

/* ---- stage (f1) -----------------------------------------------------------------------------
 * Replaces rasterize_backward_tensor + rasterize_backward_kernel (cpp/gsplat/bindings.cu:140-194,
 * cpp/gsplat/backward.cu:25-202).  grad_acc [n][12] must be zero on entry; on exit row i holds
 * (v_x, v_y, v_conic_a, v_conic_b | v_conic_c, v_opacity, v_r, v_g | v_b, v_z, 0, 0).
 * v_depth [H][W] may be NULL; when given it is the gradient of dsb_blend_forward's depth map, it takes
 * part in the opacity / mean / conic gradients, and v_z = sum alpha T v_depth is what dsb_geometry_backward
 * feeds to the mean through the v_depth slot of the reference's projection backward
 * (cpp/gsplat/backward.cu:253-259).  Without it v_z stays 0, which is what the reference always passes. */
int dsb_blend_backward(const DsbCamera* cam, const float* records, const uint64_t* sorted_pairs,
                       const int32_t* ranges, const float* final_T, const int32_t* final_idx,
                       const float* v_image, const float* v_depth, float* grad_acc, void* stream);

/* ---- stage (f2) -----------------------------------------------------------------------------
 * Replaces compute_sh_backward_tensor, project_gaussians_backward_tensor and the host glue of
 * rasterizer_backward_deepsense (cpp/gsplat/bindings.cu:22-131, cpp/rasterizer_torch.cu:263-316).
 * Writes the reference's eight gradients: v_means3d [n][3], v_means2d [n][3] (third column zero),
 * v_shs [n][(max+1)^2][3], v_colors [n][3], v_opacities [n][1], v_scales [n][3], v_rotations [n][4],
 * v_cov3d [n][6].  Any output pointer may be NULL.  accumulate != 0 adds into the outputs instead of
 * overwriting them (multi-view gradient accumulation). */
int dsb_geometry_backward(const DsbCamera* cam, int32_t n, const float* means3d, const float* scales,
                          const float* rotations, const float* records, const float* cov3d,
                          const int32_t* radii, const float* grad_acc, float* v_means3d, float* v_means2d,
                          float* v_shs, float* v_colors, float* v_opacities, float* v_scales,
                          float* v_rotations, float* v_cov3d, int32_t accumulate, void* stream);

/* ---- fused calls the Python operator uses ----------------------------------------------------
 * dsb_forward_plan   = the first half of rasterizer_forward_deepsense (cpp/rasterizer_torch.cu:170-196): preprocess,
 *                      then -- from a small grid in which the preprocess kernel marked the corners of every splat's
 *                      tile rectangle, and whose 2-D prefix sum is the number of pairs per tile -- the tile ranges
 *                      (`ranges`, [tiles+1]), the tile order (left in tile_marks: tile ids by falling pair count, which
 *                      the blend kernels and dsb_backward accept as tile_order) and a 1024-word `layout` block for the
 *                      render; then the depth order of the splats and a scan over it.  One host synchronisation
 *                      reads back *k_host (pairs) and *k_rows_host (row items, see below).
 *                      tile_marks: dsb_tile_marks_bytes(H, W); workspace: dsb_plan_workspace_bytes(n).
 *                      The layout step is one thread block and nothing before the pair emission reads what it
 *                      writes, so it runs beside the depth sort and the scan on a stream of the library's own (one
 *                      per device, created on first use; fork and join are events, and `stream` has joined it when
 *                      the call returns: whatever the caller enqueues on `stream` afterwards sees ranges, tile order
 *                      and layout).  Row-binned views and calls made while stage timing is on stay on `stream`.
 * dsb_forward_render = the second half (:196-207): from the depth-ordered splats to the sorted pair list in `pairs`
 *                      (k words) and the blended image.  By default the pairs are written in depth order and sorted
 *                      on their tile bits as the per-stage calls do (`offsets` = first pair of every depth-ordered
 *                      splat, k_rows = 0).  With DSB_FLAG_ROW_BINNING, images of at most 256 x 509 tiles (4096 x
 *                      8144 pixels) are "row-binned": every (splat, tile row) of a splat's rectangle becomes one
 *                      8-byte row item, the k_rows row items are sorted by row (one radix pass), a scan of their
 *                      widths gives each its first position in the list, and ONE pass over the k pairs expands them,
 *                      ranks them by tile column and writes each pair to its final place.  `offsets` is then the
 *                      first ROW ITEM of every depth-ordered splat.  The list is the same either way: the one the
 *                      reference's sort produces.
 *                      workspace: dsb_render_workspace_bytes(H, W, k, k_rows), 256-byte aligned.
 * dsb_forward        = dsb_forward_plan, then -- without returning to the caller in between -- dsb_forward_render
 *                      when the counts fit the buffers the caller brought (pairs holds pair_capacity words, the render
 *                      workspace is large enough).  *rendered_host (HOST int) tells which: 0 means the caller grows
 *                      its buffers and calls dsb_forward_render itself (everything the plan wrote stays valid).  A
 *                      caller that sizes the buffers from the previous call's counts with some slack pays the one
 *                      host synchronisation of a forward without any host work of its own between the two halves.
 * dsb_backward       = dsb_blend_backward + dsb_geometry_backward (rasterizer_backward_deepsense,
 *                      cpp/rasterizer_torch.cu:263-316); grad_acc is zeroed inside. */
int64_t dsb_render_workspace_bytes(int32_t image_height, int32_t image_width, int64_t k, int64_t k_rows);
int32_t dsb_row_binning_supported(int32_t image_height, int32_t image_width);   /* image size within the limits of DSB_FLAG_ROW_BINNING */
int dsb_forward_plan(const DsbCamera* cam, int32_t n, const float* means3d, const float* shs,
                     const float* colors_precomp, const float* opacities, const float* scales,
                     const float* rotations, const float* cov3d_precomp, float* records, int32_t* radii,
                     int32_t* tiles_touched, float* cov3d, uint64_t* depth_keys, uint64_t* depth_keys_alt,
                     uint32_t* offsets, int32_t* tile_marks, int32_t* ranges, uint32_t* layout /* [1024] */,
                     void* workspace, int64_t workspace_bytes, int64_t* k_host, int64_t* k_rows_host, void* stream);
int dsb_forward_render(const DsbCamera* cam, int32_t n, int64_t k, int64_t k_rows, const float* records,
                       const int32_t* tiles_touched, const uint64_t* depth_keys_sorted, const uint32_t* offsets,
                       uint64_t* pairs, const int32_t* tile_marks, const int32_t* ranges, const uint32_t* layout,
                       void* workspace, int64_t workspace_bytes, float* image, float* final_T, int32_t* final_idx,
                       float* depth /* may be NULL */, void* stream);
int dsb_forward(const DsbCamera* cam, int32_t n, const float* means3d, const float* shs, const float* colors_precomp,
                const float* opacities, const float* scales, const float* rotations, const float* cov3d_precomp,
                float* records, int32_t* radii, int32_t* tiles_touched, float* cov3d, uint64_t* depth_keys,
                uint64_t* depth_keys_alt, uint32_t* offsets, int32_t* tile_marks, int32_t* ranges, uint32_t* layout,
                void* plan_workspace, int64_t plan_workspace_bytes, uint64_t* pairs, int64_t pair_capacity,
                void* render_workspace, int64_t render_workspace_bytes, float* image, float* final_T,
                int32_t* final_idx, float* depth /* may be NULL */, int64_t* k_host, int64_t* k_rows_host,
                int32_t* rendered_host, void* stream);
int dsb_backward(const DsbCamera* cam, int32_t n, const float* means3d, const float* scales,
                 const float* rotations, const float* records, const float* cov3d, const int32_t* radii,
                 const uint64_t* sorted_pairs, const int32_t* ranges, const float* final_T,
                 const int32_t* final_idx, const float* v_image, const float* v_depth /* may be NULL */,
                 const int32_t* tile_order /* tile_marks as dsb_forward_render left it, or NULL */,
                 float* grad_acc, float* v_means3d,
                 float* v_means2d, float* v_shs, float* v_colors, float* v_opacities, float* v_scales,
                 float* v_rotations, float* v_cov3d, int32_t accumulate, void* stream);

/* ---- multi-view step ----------------------------------------------------------------------------
 * A training step renders several cameras against the same splats and needs the SUM of their gradients
 * (no reference counterpart: the reference is called once per camera and autograd adds the results).
 * Splitting dsb_backward lets the per-splat part run once per step instead of once per view:
 *   per step:   dsb_preprocess_views          (= the preprocess half of dsb_forward_plan for up to
 *                                              DSB_MAX_BATCH_VIEWS cameras: the splat parameters are read once,
 *                                              the 3-D covariance computed once; clears and fills each
 *                                              view's tile_marks; when ranges and layout (1024
 *                                              uint32 per view) are given it also makes every view's tile
 *                                              layout, as dsb_forward_plan does for one view)
 *               dsb_plan_views                (= the plan half of dsb_forward_plan for all those views in the same
 *                                              launches and with ONE host synchronisation: tiles_touched,
 *                                              depth_keys, depth_keys_alt and offsets hold one row of n entries
 *                                              per view, row_stride entries apart; records and layout are the
 *                                              views' record buffers and layout blocks; k_host and k_rows_host
 *                                              receive num_views totals each; workspace:
 *                                              dsb_plan_workspace_bytes_views)
 *   per view:   dsb_forward_render, then
 *               dsb_backward_blend            (= first half of dsb_backward: zero grad_acc unless told to keep it,
 *                                              backward blend)
 *   per step:   dsb_geometry_backward_views   over up to DSB_MAX_BATCH_VIEWS views at a time
 * records, radii, tiles_touched, depth_keys, tile_marks and grad_acc are HOST arrays of num_views device pointers (one buffer per view, all of the
 * layouts dsb_preprocess / dsb_blend_backward use); cams is a host array of num_views cameras that must
 * share sh_degree, max_sh_degree and scale_modifier (and, for dsb_preprocess_views, the image size); cov3d is
 * the splats' own (any view's).  The outputs
 * receive the sum over the views (added to their contents when accumulate != 0); v_means2d, too, is the
 * sum over views.  Results equal num_views calls of dsb_geometry_backward with accumulate, up to
 * floating-point summation order. */
int dsb_preprocess_views(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d,
                         const float* shs, const float* colors_precomp, const float* opacities,
                         const float* scales, const float* rotations, const float* cov3d_precomp,
                         float* const* records, int32_t* const* radii, int32_t* const* tiles_touched,
                         float* cov3d, uint64_t* const* depth_keys, int32_t* const* tile_marks,
                         int32_t* const* ranges /* may be NULL */, uint32_t* const* layout /* 1024 words per view; may be NULL */,
                         void* stream);
int64_t dsb_plan_workspace_bytes_views(int32_t n, int32_t num_views);
int dsb_plan_views(const DsbCamera* cam /* any of the views: its flags and image size are used */, int32_t num_views,
                   int32_t n, int64_t row_stride, const float* const* records, const int32_t* tiles_touched,
                   uint64_t* depth_keys, uint64_t* depth_keys_alt, uint32_t* offsets, const uint32_t* const* layout,
                   void* workspace, int64_t workspace_bytes, int64_t* k_host, int64_t* k_rows_host, void* stream);
/* dsb_plan_views with k_host == NULL only launches (no host synchronisation); dsb_plan_totals_views then fetches the
 * totals of that plan from the same workspace on the same stream (one synchronisation of that stream) and reports an
 * expired device-side wait.  Lets a caller queue other work, or a second batch on another stream, between the two.
 * k_rows_host may be NULL. */
int dsb_plan_totals_views(int32_t num_views, int32_t n, const void* workspace, int64_t workspace_bytes,
                          int64_t* k_host, int64_t* k_rows_host, void* stream);
int dsb_backward_blend(const DsbCamera* cam, int32_t n, const float* records, const uint64_t* sorted_pairs,
                       const int32_t* ranges, const float* final_T, const int32_t* final_idx,
                       const float* v_image, const float* v_depth /* may be NULL */,
                       const int32_t* tile_order /* may be NULL */, float* grad_acc,
                       int32_t keep_grad_acc /* 0: grad_acc is zeroed first; else added to (further bands of a view) */,
                       void* stream);
int dsb_geometry_backward_views(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d,
                                const float* scales, const float* rotations, const float* cov3d,
                                const float* const* records, const int32_t* const* radii,
                                const float* const* grad_acc, float* v_means3d, float* v_means2d, float* v_shs,
                                float* v_colors, float* v_opacities, float* v_scales, float* v_rotations,
                                float* v_cov3d, int32_t accumulate, void* stream);
/* The same call, which also keeps the per-splat statistics a 3-D Gaussian Splatting training loop consults when it
 * densifies (clone / split / prune), so that the loop does not read radii and v_means2d again after every view.
 * For every view of the call in which splat i has radius > 0:
 *     grad_norm_sum[i] += sqrt((norm_scale_x * v_x)^2 + (norm_scale_y * v_y)^2)
 *     visible_count[i] += 1
 *     max_radius[i]     = max(max_radius[i], radius)
 * with (v_x, v_y) THAT view's gradient of the pixel mean (the first two columns of the v_means2d a single-view
 * backward returns; the reference returns it in pixel units, cpp/rasterizer_torch.cu:287-315).
 * norm_scale = (1, 1) keeps pixel units; (W/2, H/2) gives the normalised-device-coordinate units of training
 * loops written for the original 3DGS rasterizer.  The three arrays are float[n], are always added to (never
 * overwritten, whatever `accumulate` says) and are cleared by the caller when it densifies.  Not part of the
 * reference. */
int dsb_geometry_backward_views_stats(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d,
                                      const float* scales, const float* rotations, const float* cov3d,
                                      const float* const* records, const int32_t* const* radii,
                                      const float* const* grad_acc, float* v_means3d, float* v_means2d, float* v_shs,
                                      float* v_colors, float* v_opacities, float* v_scales, float* v_rotations,
                                      float* v_cov3d, int32_t accumulate, float norm_scale_x, float norm_scale_y,
                                      float* grad_norm_sum, float* visible_count, float* max_radius, void* stream);

/* ---- torch-free forward ---------------------------------------------------------------------------
 * Same argument list as the reference's C++ entry rasterizer_forward_core_deepsense
 * (cpp/ds_cuda_rasterizer/rasterizer_cuda.hpp:4-9, cpp/rasterizer_cuda.cu:128-158) plus the stream: all
 * pointers are device pointers, view_matrix is the row-major [R|t], proj_matrix the row-major P*V,
 * output_image [H][W][3].  Intermediates come from the stream-ordered allocator (cudaMallocAsync) and
 * are returned to it before the call ends; the call synchronises the stream once (pair count).
 * include/dsb200.hpp wraps it under the reference's own function name. */
int dsb_forward_core(const float* means3d, const float* shs, const float* opacities, const float* scales,
                     const float* rotations, int32_t n, const float* view_matrix, const float* proj_matrix,
                     const float* camera_position, int32_t image_width, int32_t image_height, float tan_fovx,
                     float tan_fovy, float scale_modifier, int32_t max_sh_degree, int32_t sh_degree,
                     float* output_image, void* stream);

/* ---- the step before the operator's backward ----------------------------------------------------------
 * Photometric loss of 3-D Gaussian Splatting training and its gradient with respect to the rendered image
 * (no reference counterpart: users of the reference compose it from torch operations and autograd):
 *     L = (1 - lambda) * mean|image - target| + lambda * (1 - mean SSIM(image, target))
 * SSIM per channel, 11x11 Gaussian window (sigma 1.5), zero padding, C1 = 0.01^2, C2 = 0.03^2.
 * image, target, v_image: [H][W][3] floats on the device; v_image receives dL/dimage, ready to be passed to
 * dsb_backward / dsb_backward_blend; loss (may be NULL) receives L as one float on the device (no host
 * synchronisation).  workspace: dsb_image_loss_workspace_bytes(H, W). */
int64_t dsb_image_loss_workspace_bytes(int32_t image_height, int32_t image_width);
int dsb_image_loss_backward(const float* image, const float* target, int32_t image_height, int32_t image_width,
                            float lambda_dssim, void* workspace, int64_t workspace_bytes, float* v_image, float* loss,
                            void* stream);
/* The same with lambda_dssim = 0 (plain L1, which dsb_image_loss_backward computes in one pass without touching its
 * workspace) against an 8-bit target as datasets hold images: target [H][W][3] bytes standing for value / 255. */
int dsb_l1_loss_backward_u8(const float* image, const uint8_t* target, int32_t image_height, int32_t image_width,
                            float* v_image, float* loss, void* stream);

/* ---- the step after the operator -------------------------------------------------------------------
 * Adam on one parameter tensor (no reference counterpart: users of the reference call torch.optim.Adam;
 * this is that update -- no weight decay, no amsgrad -- in one pass over memory):
 *     g' = grad_scale * g;  m <- b1 m + (1-b1) g';  v <- b2 v + (1-b2) g'^2
 *     p <- p - lr / (1 - b1^step) * m / (sqrt(v) / sqrt(1 - b2^step) + eps)
 * params, exp_avg and exp_avg_sq are float tensors updated in place; step counts from 1.  The hyper-parameters are
 * doubles and are combined in double before rounding (1 - beta, the bias corrections), as torch does.  grad_scale lets the caller
 * turn the summed gradient of a multi-view step into a mean without another pass. */
int dsb_adam_step(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, int64_t count, double lr,
                  double beta1, double beta2, double eps, int32_t step, double grad_scale, void* stream);

/* Test/export helper: rebuild the reference-format sorted lists from this library's packed pairs:
 * keys[i] = (tile << 32) | sign-extended depth bits of the splat, ids[i] = splat id
 * (the layout cpp/rasterizer_kernels.cu:283,299-301 produces and thrust sorts). */
int dsb_export_reference_lists(const uint64_t* sorted_pairs, int64_t k, const float* records, int64_t* keys,
                               int32_t* ids, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSB200_H_ */
