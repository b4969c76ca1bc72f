// Shared declarations of the sm_100a splat pipeline: error plumbing, the device-side camera block,
// the packed per-splat record and the kernel launchers each stage file exports to capi.cu.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "../../include/dsb200.h"

namespace dsb {

constexpr int kTile = 16;            // tile edge in pixels (cpp/rasterizer_kernels.cuh:6 in the reference)
constexpr int kTilePixels = 256;

typedef unsigned long long u64;
typedef unsigned int u32;

// ---- host-side error plumbing -------------------------------------------------------------------
void set_error(const char* fmt, ...);
void count_launch(int n = 1);

#define DSB_CUDA_CHECK(expr)                                                                  \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            ::dsb::set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__, cudaGetErrorString(e__)); \
            return DSB_ERR_CUDA;                                                              \
        }                                                                                     \
    } while (0)

#define DSB_LAUNCH_CHECK()                                                                    \
    do {                                                                                      \
        ::dsb::count_launch();                                                                \
        cudaError_t e__ = cudaPeekAtLastError();                                              \
        if (e__ != cudaSuccess) {                                                             \
            ::dsb::set_error("kernel launch failed at %s:%d: %s", __FILE__, __LINE__, cudaGetErrorString(e__)); \
            return DSB_ERR_CUDA;                                                              \
        }                                                                                     \
    } while (0)

#define DSB_REQUIRE(cond, ...)                                                                \
    do {                                                                                      \
        if (!(cond)) {                                                                        \
            ::dsb::set_error(__VA_ARGS__);                                                    \
            return DSB_ERR_INVALID_ARGUMENT;                                                  \
        }                                                                                     \
    } while (0)

// ---- optional per-stage device timing -------------------------------------------------------------
// When enabled through dsb_stage_timing_enable(), a StageScope records a cudaEvent pair on the caller's
// stream around the kernels of one stage; dsb_stage_timing_read() sums the elapsed times.  Disabled
// scopes cost one branch.
enum Stage { kStagePreprocess = 0, kStageDepthSort, kStageScan, kStageEmit, kStageTileSort, kStageRanges,
             kStageBlendForward, kStageBlendBackward, kStageGeometryBackward, kStageCount };
struct StageScope {
    StageScope(int stage, cudaStream_t s);
    ~StageScope();
    int stage_;
    cudaStream_t stream_;
    void* slot_;
};

// ---- camera block handed to kernels by value ------------------------------------------------------
struct CamParams {
    const float* view;    // device
    const float* proj;    // device
    const float* campos;  // device
    const float* bg;      // device or null
    int H, W, tiles_x, tiles_y;
    float tanfovx, tanfovy;
    float fx, fy, cx, cy;        // forward focal / principal point
    float fx_bwd, fy_bwd;        // backward recomputes focal through atan/tan
    float scale_modifier;
    int sh_degree, max_coeff;
    int transposed;              // matrices still in the caller's transposed layout
    int drop_last;
    int tight_tiles;             // tile rectangles shrunk to where the splat can contribute
    int row_binning;             // the fused render builds its pair list by row binning (row_binning.cu)
    int band_y0, band_y1;        // tile rows [band_y0, band_y1) that get pairs and pixels (the whole image: 0, tiles_y)
};

int make_cam_params(const DsbCamera* cam, CamParams* out);

// Element (r, c) of a 4x4 stored row-major, or transposed when the caller skipped the transposes.
__device__ __forceinline__ float mat_at(const float* m, int r, int c, int transposed) {
    return transposed ? m[c * 4 + r] : m[r * 4 + c];
}

// ---- packed per-splat record: three float4 lanes ------------------------------------------------
//   q0 = (x_pix, y_pix, conic_a, conic_b)   q1 = (conic_c, opacity, r, g)   q2 = (b, depth, rect_x, rect_y)
// rect_* hold (lo | hi << 16) tile bounds as integer bits.
__device__ __forceinline__ u32 pack_rect(int lo, int hi) { return (u32)lo | ((u32)hi << 16); }

// ---- bounded waits -----------------------------------------------------------------------------
// Every spin in this library gives up after a fixed number of polls, records why in a status word and
// returns, so a logic error can never hang the GPU.  The limit travels to the kernels as an argument
// (kSpinLimit in normal use; the dsb_debug_* entry points pass a few hundred so that a test can watch a wait
// run out in microseconds).
constexpr u32 kSpinLimit = 1u << 22;
constexpr u32 kCopyWaitPolls = 1u << 20;   // polls of an mbarrier that counts bulk copies in

// One int per device that keeps the first DSB_ERR_* code any kernel of this library recorded since the host last
// took it: kernels receive its address and atomicExch the code in when a bounded wait gives up.  It lives in
// the library image (no allocation), its device address is looked up once per device with that device current.
// Calls that synchronise anyway (the pair-count read-back of a plan) fetch it in the same synchronisation;
// dsb_take_device_status() fetches it on demand.
int device_status_address(int** out);
// Copies the word to *host on stream s (no synchronisation); the caller synchronises, then calls
// finish_device_status(value, s), which clears the word when it was set and returns the DSB_ code to report.
int begin_device_status_read(int* host, cudaStream_t s);
int finish_device_status_read(int value, cudaStream_t s);
u32 copy_wait_polls();   // polls preprocess gives its bulk copies (kCopyWaitPolls unless a test lowered it)

// ---- launchers (one per stage file) -----------------------------------------------------------------
int launch_preprocess(const CamParams& cp, int n, const float* means, const float* shs, const float* colors_precomp,
                      const float* opac, const float* scales, const float* rots, const float* cov3d_precomp,
                      float* records, int32_t* radii, int32_t* tiles, float* cov3d, u64* depth_keys, int* tile_marks,
                      cudaStream_t s);

int launch_preprocess_views(const CamParams* cps, int count, int n, const float* means, const float* shs,
                            const float* colors_precomp, const float* opac, const float* scales, const float* rots,
                            const float* cov3d_precomp, float* const* records, int32_t* const* radii,
                            int32_t* const* tiles, float* cov3d, u64* const* depth_keys, int* const* tile_marks,
                            cudaStream_t s);

// Radix-sort pass layout: which bits each pass looks at.  flip is XORed into the digit (sign bit of signed keys).
constexpr int kMaxSortPasses = 8;
struct SortPlan {
    int npass;
    int shift[kMaxSortPasses];
    int bits[kMaxSortPasses];   // digit width of the pass, 1..8
    u32 mask[kMaxSortPasses];
    u32 flip[kMaxSortPasses];
    int tile_items;             // items per block; 0 = chosen from the list length
};
__device__ __forceinline__ u32 sort_digit(u64 key, int shift, u32 mask, u32 flip) {
    return ((u32)(key >> shift) & mask) ^ flip;
}
SortPlan make_sort_plan(int begin_bit, int end_bit, bool signed_top);

int64_t sort_workspace_bytes(int64_t k);
int64_t sort_status_offset();  // byte offset of the int status word inside a sort workspace
int launch_sort(u64* items, u64* items_alt, u32* vals, u32* vals_alt, int64_t k, int begin_bit, int end_bit,
                void* ws, int64_t ws_bytes, int* in_alt, cudaStream_t s, bool large_tiles_only = false, int batch = 1,
                int64_t item_stride = 0);
int64_t sort_batch_stride_bytes(int64_t k);  // workspace slice per list when `batch` lists are sorted together
// Two-step form for producers that count the digits themselves while writing the items:
// sort_begin clears the workspace and returns the histogram to fill, sort_passes runs the passes.
int sort_begin(int64_t k, const SortPlan& plan, void* ws, int64_t ws_bytes, u32** hist_out, cudaStream_t s, int batch = 1);
int sort_passes(u64* items, u64* items_alt, u32* vals, u32* vals_alt, int64_t k, const SortPlan& plan, void* ws,
                int* in_alt, cudaStream_t s, int batch = 1, int64_t item_stride = 0);

// ---- row binning (row_binning.cu): the fused render's way from depth-ordered splats to the sorted pair list ----
// Row item: one (splat, tile row) of a splat's tile rectangle, 64 bits: row | first column | width | splat id.
constexpr int kRowItemRowShift = 52, kRowItemX0Shift = 42, kRowItemWShift = 32;
constexpr u32 kRowItemFieldMask = 1023u;
constexpr int kRowScatterItems = 16;                // pairs per thread of the scatter pass
constexpr int kRowTile = 256 * kRowScatterItems;    // pairs per block of the scatter pass
// What tile_layout_kernel leaves in a view's 1024-word layout block when the view is row-binned:
//   [0 .. tiles_y]                      blocks of the scatter pass before each tile row (and their total)
//   [kRowInfoStarts .. + tiles_y]       first final-list position of each tile row (and K)
//   [kRowInfoTotal, kRowInfoTotal + 1]  K as 64 bits (exact even where 32-bit positions would wrap)
constexpr int kRowInfoStarts = 512, kRowInfoTotal = 1022;
constexpr int kLayoutWords = 1024;
bool row_binning_supported(const CamParams& cp);   // image size within the limits
bool row_binned(const CamParams& cp);                // asked for and within the limits
int64_t row_workspace_bytes(int64_t k, int64_t k_rows);
int launch_row_binning(const CamParams& cp, int n, int64_t k, int64_t k_rows, const float* records, const int32_t* tiles,
                       const u64* depth_keys_sorted, const u32* row_offsets, const int32_t* ranges, const u32* row_info,
                       u64* pairs, void* ws, int64_t ws_bytes, cudaStream_t s);

int64_t plan_workspace_bytes(int n);
int64_t plan_workspace_bytes_views(int n, int views);
// records / row_info: null for the per-stage plan (offsets = first PAIR of every depth-ordered splat), else one
// pointer per view (offsets = first ROW ITEM of every depth-ordered splat; the pair total comes from row_info).
int launch_plan_views(const CamParams& cp, int views, int n, int64_t item_stride, const int32_t* tiles, u64* depth_keys,
                      u64* depth_keys_alt, u32* offsets, void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s,
                      const float* const* records = nullptr, const u32* const* row_info = nullptr, int64_t* k_rows_host = nullptr);
int read_plan_totals_views(int views, int n, const void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s,
                           int64_t* k_rows_host = nullptr);
int launch_plan(const CamParams& cp, int n, const int32_t* tiles, u64* depth_keys, u64* depth_keys_alt, u32* offsets,
                void* ws, int64_t ws_bytes, int64_t* k_host, cudaStream_t s);
// Test hooks: one scan / one sort pass in which the first tile of the look-back chain is never processed, so the
// second tile's bounded wait runs out after `spin_limit` polls (see dsb_debug_expire_*_wait in the header).
int debug_expire_scan_wait(const CamParams& cp, int n, const int32_t* tiles, const u64* depth_keys_sorted, u32* offsets,
                           void* ws, int64_t ws_bytes, u32 spin_limit, cudaStream_t s);
int debug_expire_sort_wait(u64* items, u64* items_alt, int64_t k, int begin_bit, int end_bit, void* ws, int64_t ws_bytes,
                           u32 spin_limit, cudaStream_t s);
int launch_emit(const CamParams& cp, int n, int64_t k, const float* records, const int32_t* tiles,
                const u64* depth_keys_sorted, const u32* offsets, u64* pairs, cudaStream_t s);
// Grid of rectangle corner marks filled by the preprocess kernel; launch_tile_layout turns it into tile ranges
// and the tile sort's digit counts.
// The grid is kept in kMarkCopies copies, one per residue of the marking block's index, so that the marks of
// splats that share a tile corner do not all queue up on one L2 word; the layout kernel adds the copies.
#ifndef DSB_MARK_COPIES
#define DSB_MARK_COPIES 4
#endif
constexpr int kMarkCopies = DSB_MARK_COPIES;
int64_t tile_marks_bytes(int H, int W);
int64_t tile_marks_copy_ints(int H, int W);   // distance between two copies, in ints
int launch_tile_layout(const CamParams& cp, int* tile_marks, const SortPlan& plan, u32* hist, int32_t* ranges,
                       int* has_order, cudaStream_t s);
// hist: per view kLayoutWords words that receive the tile sort's digit counts, or the row-binning block (see above)
// when the image is row-binned.
int launch_tile_layout_views(const CamParams& cp, int count, int* const* tile_marks, const SortPlan& plan, u32* const* hist,
                             int32_t* const* ranges, int* has_order, cudaStream_t s);
SortPlan tile_sort_plan(const CamParams& cp);
bool tile_order_available(int H, int W);  // whether launch_tile_layout leaves the tile order for this image size
int launch_ranges(const u64* sorted, int64_t k, int H, int W, int32_t* ranges, cudaStream_t s, int trailing_quirk = 1);
int launch_export(const u64* sorted, int64_t k, const float* records, int64_t* keys, int32_t* ids, cudaStream_t s);

int launch_blend_forward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                         float* image, float* final_T, int32_t* final_idx, float* depth, const int32_t* tile_order,
                         cudaStream_t s);
int launch_blend_forward_variant(const CamParams& cp, int variant, int n, int64_t k, const float* records, const u64* sorted,
                                 const int32_t* ranges, float* image, float* final_T, int32_t* final_idx,
                                 const int32_t* tile_order, void* scratch, int64_t scratch_bytes, cudaStream_t s);
int launch_blend_backward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                          const float* final_T, const int32_t* final_idx, const float* v_image, const float* v_depth,
                          float* grad_acc, const int32_t* tile_order, cudaStream_t s);
int launch_geometry_backward(const CamParams& cp, int n, const float* means, const float* scales, const float* rots,
                             const float* records, const float* cov3d, const int32_t* radii, const float* grad_acc,
                             float* v_means3d, float* v_means2d, float* v_shs, float* v_colors, float* v_opac,
                             float* v_scales, float* v_rots, float* v_cov3d, int accumulate, cudaStream_t s);

// Per-splat statistics a training loop keeps between two densification rounds; the per-splat backward adds a
// step's views to them when the pointers are set.  For every view in which splat i has radius > 0:
//   grad_norm_sum[i] += sqrt((scale_x * v_x)^2 + (scale_y * v_y)^2)   (v_x, v_y: that view's pixel-mean gradient)
//   visible_count[i] += 1,   max_radius[i] = max(max_radius[i], radius)
struct DensifyStats {
    float* grad_norm_sum = nullptr;
    float* visible_count = nullptr;
    float* max_radius = nullptr;
    float scale_x = 1.f, scale_y = 1.f;
};

int launch_geometry_backward_views(const CamParams* cps, int count, int n, const float* means, const float* scales,
                                   const float* rots, const float* cov3d, const float* const* records,
                                   const int32_t* const* radii, const float* const* grad_acc, float* v_means3d,
                                   float* v_means2d, float* v_shs, float* v_colors, float* v_opac, float* v_scales,
                                   float* v_rots, float* v_cov3d, int accumulate, cudaStream_t s,
                                   const DensifyStats* stats = nullptr);

int64_t image_loss_workspace_bytes(int H, int W);
int launch_l1_loss_u8(const float* image, const unsigned char* target, int H, int W, float* v_image, float* loss, cudaStream_t s);
int launch_image_loss(const float* image, const float* target, int H, int W, float lambda_dssim, void* workspace,
                      int64_t workspace_bytes, float* v_image, float* loss, cudaStream_t s);
int launch_adam(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, int64_t count, double lr, double beta1,
                double beta2, double eps, int step, double grad_scale, cudaStream_t s);

}  // namespace dsb
