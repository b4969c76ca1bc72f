// extern "C" surface of the library (declared in include/dsb200.h): argument checks, the camera block,
// the last-error string and the fused forward/backward calls the Python operator uses.
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace dsb {

static thread_local char g_error[1024] = "";
static std::atomic<long long> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// ---- device status word ------------------------------------------------------------------------
static __device__ int g_device_status;            // first DSB_ERR_* a kernel recorded since the host last took it
constexpr int kMaxStatusDevices = 64;
static int* g_device_status_address[kMaxStatusDevices] = {};
static std::mutex g_device_status_mutex;
static std::atomic<unsigned> g_copy_wait_polls{kCopyWaitPolls};

int device_status_address(int** out) {
    int dev = -1;
    DSB_CUDA_CHECK(cudaGetDevice(&dev));
    DSB_REQUIRE(dev >= 0 && dev < kMaxStatusDevices, "device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_device_status_mutex);
    if (!g_device_status_address[dev]) {
        // In host code the symbol's name is only a handle; the address a kernel can use differs per GPU.
        void* p = nullptr;
        DSB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_device_status));
        DSB_REQUIRE(p != nullptr, "the device status word has no device address");
        g_device_status_address[dev] = static_cast<int*>(p);
    }
    *out = g_device_status_address[dev];
    return DSB_OK;
}

int begin_device_status_read(int* host, cudaStream_t s) {
    int* word = nullptr;
    const int rc = device_status_address(&word);
    if (rc != DSB_OK) return rc;
    DSB_CUDA_CHECK(cudaMemcpyAsync(host, word, sizeof(int), cudaMemcpyDeviceToHost, s));
    return DSB_OK;
}

int finish_device_status_read(int value, cudaStream_t s) {
    if (value >= 0) return DSB_OK;   // 0: nothing recorded; positive: a note about a slower path, results valid
    int* word = nullptr;
    const int rc = device_status_address(&word);
    if (rc != DSB_OK) return rc;
    DSB_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(int), s));   // taken: the next report starts from a clean word
    set_error("a bounded device-side wait of an earlier call on this device expired (status %d): results of the calls "
              "enqueued since the last status check are not valid", value);
    return value == DSB_ERR_DEVICE_WAIT_EXPIRED ? DSB_ERR_DEVICE_WAIT_EXPIRED : DSB_ERR_CUDA;
}

u32 copy_wait_polls() { return g_copy_wait_polls.load(std::memory_order_relaxed); }

// ---- side lane -----------------------------------------------------------------------------------
// One extra stream and two events per device, created on first use and kept for the life of the process.  The
// single-view plan runs the tile layout on it: the layout is one thread block (its duration is that block's
// latency, about 28 us at 1080p) and nothing before the pair emission needs its results, so it runs beside the
// depth sort and the offset scan instead of in front of them.  Fork and join are events; no kernel waits on a
// kernel.  Calls from several host threads share the lane: its stream is first-in first-out, so a join recorded
// later also covers every layout launched earlier.
struct SideLane { cudaStream_t stream; cudaEvent_t fork, join; bool ready; };
static SideLane g_side_lane[kMaxStatusDevices] = {};
static std::mutex g_side_lane_mutex;

static SideLane* side_lane_locked() {   // g_side_lane_mutex held
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxStatusDevices) return nullptr;
    SideLane& lane = g_side_lane[dev];
    if (!lane.ready) {
        if (cudaStreamCreateWithFlags(&lane.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&lane.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&lane.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        lane.ready = true;
    }
    return &lane;
}

// ---- stage timing ------------------------------------------------------------------------------
struct EventPair { cudaEvent_t a, b; int stage; };
static bool g_timing = false;
static std::vector<EventPair*> g_pending;
static std::mutex g_timing_mutex;
static const char* kStageNames[kStageCount] = {"preprocess", "depth_sort", "scan", "emit_pairs", "tile_sort", "tile_ranges",
                                               "blend_forward", "blend_backward", "geometry_backward"};

StageScope::StageScope(int stage, cudaStream_t s) : stage_(stage), stream_(s), slot_(nullptr) {
    if (!g_timing) return;
    EventPair* p = new EventPair;
    p->stage = stage;
    if (cudaEventCreate(&p->a) != cudaSuccess || cudaEventCreate(&p->b) != cudaSuccess) { delete p; return; }
    cudaEventRecord(p->a, s);
    slot_ = p;
}

StageScope::~StageScope() {
    if (!slot_) return;
    EventPair* p = static_cast<EventPair*>(slot_);
    cudaEventRecord(p->b, stream_);
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    g_pending.push_back(p);
}

int make_cam_params(const DsbCamera* cam, CamParams* out) {
    DSB_REQUIRE(cam, "camera is null");
    DSB_REQUIRE(cam->image_height > 0 && cam->image_width > 0, "image size must be positive (got %d x %d)",
                cam->image_width, cam->image_height);
    DSB_REQUIRE(cam->image_height <= 16 * 65535 && cam->image_width <= 16 * 65535, "image too large for 16-bit tile bounds");
    DSB_REQUIRE(cam->viewmatrix && cam->projmatrix && cam->campos, "camera matrices / position are null");
    DSB_REQUIRE(cam->sh_degree >= 0 && cam->sh_degree <= 4, "sh_degree must be in 0..4 (got %d)", cam->sh_degree);
    DSB_REQUIRE(cam->max_sh_degree >= 0 && cam->max_sh_degree <= 3, "max_sh_degree must be in 0..3 (got %d)", cam->max_sh_degree);
    DSB_REQUIRE(cam->tanfovx > 0.f && cam->tanfovy > 0.f, "tanfov must be positive");
    CamParams p;
    p.view = cam->viewmatrix; p.proj = cam->projmatrix; p.campos = cam->campos; p.bg = cam->bg;
    p.H = cam->image_height; p.W = cam->image_width;
    p.tiles_x = (p.W + kTile - 1) / kTile; p.tiles_y = (p.H + kTile - 1) / kTile;
    p.tanfovx = cam->tanfovx; p.tanfovy = cam->tanfovy;
    // Forward focal: size / (2 tanfov) in single precision (cpp/rasterizer_torch.cu:144-147 in the reference).
    p.fx = p.W / (2 * cam->tanfovx); p.fy = p.H / (2 * cam->tanfovy);
    p.cx = p.W / 2.0f; p.cy = p.H / 2.0f;
    // Backward focal goes through atan and tan again (cpp/rasterizer_torch.cu:78-81,297-298).
    p.fx_bwd = (float)p.W / (2.0f * tanf((2 * atanf(cam->tanfovx)) / 2.0f));
    p.fy_bwd = (float)p.H / (2.0f * tanf((2 * atanf(cam->tanfovy)) / 2.0f));
    p.scale_modifier = cam->scale_modifier;
    p.sh_degree = cam->sh_degree;
    p.max_coeff = (cam->max_sh_degree + 1) * (cam->max_sh_degree + 1);
    p.transposed = cam->matrices_transposed != 0;
    p.drop_last = (cam->flags & DSB_FLAG_DROP_LAST_SPLAT) != 0;
    p.tight_tiles = (cam->flags & DSB_FLAG_TIGHT_TILES) != 0;
    p.row_binning = (cam->flags & DSB_FLAG_ROW_BINNING) != 0;
    p.band_y0 = 0; p.band_y1 = p.tiles_y;
    if (cam->tile_row_band != 0) {
        const int lo = cam->tile_row_band & 0xffff, hi = (int)(((uint32_t)cam->tile_row_band) >> 16);
        DSB_REQUIRE(lo < hi && hi <= p.tiles_y, "tile_row_band [%d, %d) is not a band of the image's %d tile rows", lo, hi, p.tiles_y);
        p.band_y0 = lo; p.band_y1 = hi;
    }
    *out = p;
    return DSB_OK;
}

}  // namespace dsb

using namespace dsb;

#define CAM_OR_RETURN(cam, cp)                   \
    CamParams cp;                                \
    {                                            \
        const int rc__ = make_cam_params(cam, &cp); \
        if (rc__ != DSB_OK) return rc__;         \
    }

extern "C" {

const char* dsb_last_error(void) { return g_error; }
int32_t dsb_version(void) { return 100; }
int64_t dsb_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

int dsb_stage_timing_enable(int32_t on) {
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    for (EventPair* p : g_pending) { cudaEventDestroy(p->a); cudaEventDestroy(p->b); delete p; }
    g_pending.clear();
    g_timing = on != 0;
    return DSB_OK;
}

int dsb_take_device_status(int32_t* status_host, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    int value = 0;
    int rc = begin_device_status_read(&value, s);
    if (rc != DSB_OK) return rc;
    DSB_CUDA_CHECK(cudaStreamSynchronize(s));
    if (status_host) *status_host = value;
    if (value > 0) {   // a note: hand it over once
        int* word = nullptr;
        rc = device_status_address(&word);
        if (rc != DSB_OK) return rc;
        DSB_CUDA_CHECK(cudaMemsetAsync(word, 0, sizeof(int), s));
    }
    return finish_device_status_read(value, s);
}

int dsb_debug_set_copy_wait_polls(uint32_t polls) {
    g_copy_wait_polls.store(polls ? polls : kCopyWaitPolls, std::memory_order_relaxed);
    return DSB_OK;
}

int dsb_debug_expire_scan_wait(const DsbCamera* cam, int32_t n, const int32_t* tiles_touched,
                               const uint64_t* depth_keys_sorted, uint32_t* offsets, void* workspace,
                               int64_t workspace_bytes, uint32_t spin_limit, void* stream) {
    CAM_OR_RETURN(cam, cp);
    return debug_expire_scan_wait(cp, n, tiles_touched, reinterpret_cast<const u64*>(depth_keys_sorted), offsets, workspace,
                                  workspace_bytes, spin_limit, (cudaStream_t)stream);
}

int dsb_debug_expire_sort_wait(uint64_t* items, uint64_t* items_alt, int64_t k, int32_t begin_bit, int32_t end_bit,
                               void* workspace, int64_t workspace_bytes, uint32_t spin_limit, void* stream) {
    return debug_expire_sort_wait(reinterpret_cast<u64*>(items), reinterpret_cast<u64*>(items_alt), k, begin_bit, end_bit,
                                  workspace, workspace_bytes, spin_limit, (cudaStream_t)stream);
}

int32_t dsb_stage_count(void) { return kStageCount; }
const char* dsb_stage_name(int32_t stage) { return (stage >= 0 && stage < kStageCount) ? kStageNames[stage] : ""; }

int dsb_stage_timing_read(int32_t stage_count, double* ms_total, int64_t* calls) {
    DSB_REQUIRE(ms_total && calls && stage_count >= kStageCount, "stage_timing_read: need room for %d stages", (int)kStageCount);
    for (int i = 0; i < stage_count; ++i) { ms_total[i] = 0.0; calls[i] = 0; }
    std::lock_guard<std::mutex> lock(g_timing_mutex);
    for (EventPair* p : g_pending) {
        DSB_CUDA_CHECK(cudaEventSynchronize(p->b));
        float ms = 0.f;
        DSB_CUDA_CHECK(cudaEventElapsedTime(&ms, p->a, p->b));
        ms_total[p->stage] += ms;
        calls[p->stage] += 1;
        cudaEventDestroy(p->a); cudaEventDestroy(p->b);
        delete p;
    }
    g_pending.clear();
    return DSB_OK;
}

int64_t dsb_plan_workspace_bytes(int32_t n) { return plan_workspace_bytes(n < 0 ? 0 : n); }
int64_t dsb_sort_workspace_bytes(int64_t k) { return sort_workspace_bytes(k < 0 ? 0 : k); }
int64_t dsb_tile_marks_bytes(int32_t image_height, int32_t image_width) {
    return (image_height > 0 && image_width > 0) ? tile_marks_bytes(image_height, image_width) : 0;
}

int dsb_preprocess(const DsbCamera* cam, int32_t n, const float* means3d, const float* shs, const float* colors_precomp,
                   const float* opacities, const float* scales, const float* rotations, const float* cov3d_precomp,
                   float* records, int32_t* radii, int32_t* tiles_touched, float* cov3d, uint64_t* depth_keys,
                   void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    StageScope scope(kStagePreprocess, (cudaStream_t)stream);
    return launch_preprocess(cp, n, means3d, shs, colors_precomp, opacities, scales, rotations, cov3d_precomp, records,
                             radii, tiles_touched, cov3d, reinterpret_cast<u64*>(depth_keys), nullptr,
                             (cudaStream_t)stream);
}

int dsb_plan_pairs(const DsbCamera* cam, int32_t n, const int32_t* tiles_touched, uint64_t* depth_keys,
                   uint64_t* depth_keys_alt, uint32_t* offsets, void* workspace, int64_t workspace_bytes,
                   int64_t* k_host, void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    DSB_REQUIRE(k_host, "plan: k_host is null");
    return launch_plan(cp, n, tiles_touched, reinterpret_cast<u64*>(depth_keys), reinterpret_cast<u64*>(depth_keys_alt),
                       offsets, workspace, workspace_bytes, k_host, (cudaStream_t)stream);
}

int64_t dsb_plan_workspace_bytes_views(int32_t n, int32_t num_views) {
    return (n >= 0 && num_views >= 1 && num_views <= DSB_MAX_BATCH_VIEWS) ? plan_workspace_bytes_views(n, num_views) : 0;
}

int dsb_plan_views(const DsbCamera* cam, int32_t num_views, int32_t n, int64_t row_stride, const float* const* records,
                   const int32_t* tiles_touched, uint64_t* depth_keys, uint64_t* depth_keys_alt, uint32_t* offsets,
                   const uint32_t* const* layout, void* workspace, int64_t workspace_bytes, int64_t* k_host,
                   int64_t* k_rows_host, void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    const bool rows = row_binned(cp);
    DSB_REQUIRE(!rows || (records && layout), "plan_views: row binning needs the views' records and layout blocks");
    return launch_plan_views(cp, num_views, n, row_stride, tiles_touched, reinterpret_cast<u64*>(depth_keys),
                             reinterpret_cast<u64*>(depth_keys_alt), offsets, workspace, workspace_bytes, k_host,
                             (cudaStream_t)stream, rows ? records : nullptr, rows ? layout : nullptr, k_rows_host);
}

int dsb_plan_totals_views(int32_t num_views, int32_t n, const void* workspace, int64_t workspace_bytes, int64_t* k_host,
                          int64_t* k_rows_host, void* stream) {
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    return read_plan_totals_views(num_views, n, workspace, workspace_bytes, k_host, (cudaStream_t)stream, k_rows_host);
}

int32_t dsb_row_binning_supported(int32_t image_height, int32_t image_width) {
    if (image_height <= 0 || image_width <= 0) return 0;
    CamParams cp = {};
    cp.H = image_height; cp.W = image_width;
    cp.tiles_x = (cp.W + kTile - 1) / kTile; cp.tiles_y = (cp.H + kTile - 1) / kTile;
    return row_binning_supported(cp) ? 1 : 0;
}

int64_t dsb_render_workspace_bytes(int32_t image_height, int32_t image_width, int64_t k, int64_t k_rows) {
    if (k < 0) k = 0;
    if (k_rows < 0) k_rows = 0;
    // k_rows > 0: the plan row-binned the view
    if (k_rows > 0 && dsb_row_binning_supported(image_height, image_width)) return row_workspace_bytes(k, k_rows);
    return ((k * 8 + 255) / 256) * 256 + sort_workspace_bytes(k);   // alternate pair buffer + tile sort scratch
}

int dsb_emit_pairs(const DsbCamera* cam, int32_t n, int64_t k, const float* records, const int32_t* tiles_touched,
                   const uint64_t* depth_keys_sorted, const uint32_t* offsets, uint64_t* pairs, void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0 && k >= 0, "n and k must be non-negative");
    return launch_emit(cp, n, k, records, tiles_touched, reinterpret_cast<const u64*>(depth_keys_sorted), offsets,
                       reinterpret_cast<u64*>(pairs), (cudaStream_t)stream);
}

int dsb_sort_pairs(uint64_t* items, uint64_t* items_alt, int64_t k, int32_t begin_bit, int32_t end_bit, void* workspace,
                   int64_t workspace_bytes, int32_t* sorted_in_alt_host, void* stream) {
    DSB_REQUIRE(k >= 0, "k must be non-negative");
    int in_alt = 0;
    const int rc = launch_sort(reinterpret_cast<u64*>(items), reinterpret_cast<u64*>(items_alt), nullptr, nullptr, k,
                               begin_bit, end_bit, workspace, workspace_bytes, &in_alt, (cudaStream_t)stream);
    if (sorted_in_alt_host) *sorted_in_alt_host = in_alt;
    return rc;
}

int dsb_sort_by_keys(int64_t* keys, int64_t* keys_alt, int32_t* values, int32_t* values_alt, int64_t k,
                     int32_t begin_bit, int32_t end_bit, void* workspace, int64_t workspace_bytes,
                     int32_t* sorted_in_alt_host, void* stream) {
    DSB_REQUIRE(k >= 0, "k must be non-negative");
    DSB_REQUIRE(values && values_alt, "sort_by_keys: values are required");
    int in_alt = 0;
    const int rc = launch_sort(reinterpret_cast<u64*>(keys), reinterpret_cast<u64*>(keys_alt),
                               reinterpret_cast<u32*>(values), reinterpret_cast<u32*>(values_alt), k, begin_bit, end_bit,
                               workspace, workspace_bytes, &in_alt, (cudaStream_t)stream);
    if (sorted_in_alt_host) *sorted_in_alt_host = in_alt;
    return rc;
}

int dsb_identify_tile_ranges(const uint64_t* sorted, int64_t k, int32_t image_height, int32_t image_width,
                             int32_t* ranges, void* stream) {
    DSB_REQUIRE(k >= 0, "k must be non-negative");
    return launch_ranges(reinterpret_cast<const u64*>(sorted), k, image_height, image_width, ranges, (cudaStream_t)stream);
}

int dsb_blend_forward(const DsbCamera* cam, const float* records, const uint64_t* sorted_pairs, const int32_t* ranges,
                      float* image, float* final_T, int32_t* final_idx, float* depth, void* stream) {
    CAM_OR_RETURN(cam, cp);
    return launch_blend_forward(cp, records, reinterpret_cast<const u64*>(sorted_pairs), ranges, image, final_T,
                                final_idx, depth, nullptr, (cudaStream_t)stream);
}

int dsb_debug_blend_forward_variant(const DsbCamera* cam, int32_t variant, int32_t n, int64_t k, const float* records,
                                    const uint64_t* sorted_pairs, const int32_t* ranges, float* image, float* final_T,
                                    int32_t* final_idx, const int32_t* tile_order, void* scratch, int64_t scratch_bytes,
                                    void* stream) {
    CAM_OR_RETURN(cam, cp);
    return launch_blend_forward_variant(cp, variant, n, k, records, reinterpret_cast<const u64*>(sorted_pairs), ranges, image,
                                        final_T, final_idx, tile_order, scratch, scratch_bytes, (cudaStream_t)stream);
}

int dsb_blend_backward(const DsbCamera* cam, const float* records, const uint64_t* sorted_pairs, const int32_t* ranges,
                       const float* final_T, const int32_t* final_idx, const float* v_image, const float* v_depth,
                       float* grad_acc, void* stream) {
    CAM_OR_RETURN(cam, cp);
    return launch_blend_backward(cp, records, reinterpret_cast<const u64*>(sorted_pairs), ranges, final_T, final_idx,
                                 v_image, v_depth, grad_acc, nullptr, (cudaStream_t)stream);
}

int dsb_geometry_backward(const DsbCamera* cam, int32_t n, const float* means3d, const float* scales,
                          const float* rotations, const float* records, const float* cov3d, const int32_t* radii,
                          const float* grad_acc, float* v_means3d, float* v_means2d, float* v_shs, float* v_colors,
                          float* v_opacities, float* v_scales, float* v_rotations, float* v_cov3d, int32_t accumulate,
                          void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    return launch_geometry_backward(cp, n, means3d, scales, rotations, records, cov3d, radii, grad_acc, v_means3d,
                                    v_means2d, v_shs, v_colors, v_opacities, v_scales, v_rotations, v_cov3d, accumulate,
                                    (cudaStream_t)stream);
}

int dsb_forward_plan(const DsbCamera* cam, int32_t n, const float* means3d, const float* shs, const float* colors_precomp,
                     const float* opacities, const float* scales, const float* rotations, const float* cov3d_precomp,
                     float* records, int32_t* radii, int32_t* tiles_touched, float* cov3d, uint64_t* depth_keys,
                     uint64_t* depth_keys_alt, uint32_t* offsets, int32_t* tile_marks, int32_t* ranges, uint32_t* layout,
                     void* workspace, int64_t workspace_bytes, int64_t* k_host, int64_t* k_rows_host, void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    DSB_REQUIRE(tile_marks && ranges && layout, "forward_plan: null tile_marks, ranges or layout");
    DSB_REQUIRE(k_host && k_rows_host, "forward_plan: k_host or k_rows_host is null");
    *k_host = 0; *k_rows_host = 0;
    cudaStream_t s = (cudaStream_t)stream;
    {
        StageScope scope(kStagePreprocess, s);
        DSB_CUDA_CHECK(cudaMemsetAsync(tile_marks, 0, (size_t)tile_marks_bytes(cp.H, cp.W), s));
        const int rc = launch_preprocess(cp, n, means3d, shs, colors_precomp, opacities, scales, rotations, cov3d_precomp,
                                         records, radii, tiles_touched, cov3d, reinterpret_cast<u64*>(depth_keys),
                                         tile_marks, s);
        if (rc != DSB_OK) return rc;
    }
    // Tile ranges, tile order and the tile sort's digit counts (or the row-binning block) from the corner marks.  The
    // depth sort and the scan below do not read them (the scan of a row-binned view does), so the layout goes to the
    // side lane; the caller's stream joins it after the plan.  With stage timing on everything stays on one stream,
    // so that a stage's events bracket that stage alone.
    const bool rows = row_binned(cp);
    cudaEvent_t join = nullptr;
    {
        StageScope scope(kStageRanges, s);
        int has_order = 0;
        bool beside = false;
        if (!rows && n > 0 && !g_timing) {
            std::lock_guard<std::mutex> lock(g_side_lane_mutex);
            SideLane* lane = side_lane_locked();
            if (lane) {
                DSB_CUDA_CHECK(cudaEventRecord(lane->fork, s));
                DSB_CUDA_CHECK(cudaStreamWaitEvent(lane->stream, lane->fork, 0));
                const int rc = launch_tile_layout(cp, tile_marks, tile_sort_plan(cp), layout, ranges, &has_order, lane->stream);
                // joined whatever the launch said, so that the caller's stream never runs ahead of the side lane
                DSB_CUDA_CHECK(cudaEventRecord(lane->join, lane->stream));
                if (rc != DSB_OK) {
                    cudaStreamWaitEvent(s, lane->join, 0);
                    return rc;
                }
                join = lane->join;
                beside = true;
            }
        }
        if (!beside) {
            const int rc = launch_tile_layout(cp, tile_marks, tile_sort_plan(cp), layout, ranges, &has_order, s);
            if (rc != DSB_OK) return rc;
        }
    }
    if (n == 0) return DSB_OK;
    const float* rec = records;
    const u32* info = layout;
    const int rc = launch_plan_views(cp, 1, n, n, tiles_touched, reinterpret_cast<u64*>(depth_keys),
                                     reinterpret_cast<u64*>(depth_keys_alt), offsets, workspace, workspace_bytes, k_host, s,
                                     rows ? &rec : nullptr, rows ? &info : nullptr, k_rows_host);
    if (join) {   // everything the caller enqueues on its stream from here on sees the layout
        const cudaError_t e = cudaStreamWaitEvent(s, join, 0);
        if (rc == DSB_OK) DSB_CUDA_CHECK(e);
    }
    return rc;
}

int dsb_forward_render(const DsbCamera* cam, int32_t n, int64_t k, int64_t k_rows, const float* records,
                       const int32_t* tiles_touched, const uint64_t* depth_keys_sorted, const uint32_t* offsets, uint64_t* pairs,
                       const int32_t* tile_marks, const int32_t* ranges, const uint32_t* layout, void* workspace,
                       int64_t workspace_bytes, float* image, float* final_T, int32_t* final_idx, float* depth, void* stream) {
    CAM_OR_RETURN(cam, cp);
    cudaStream_t s = (cudaStream_t)stream;
    DSB_REQUIRE(k >= 0 && k < DSB_MAX_PAIRS, "too many pairs");
    DSB_REQUIRE(tile_marks && ranges && layout, "forward_render: null tile_marks, ranges or layout");
    DSB_REQUIRE(k == 0 || (pairs && workspace), "forward_render: null pair buffer or workspace");
    const int has_order = tile_order_available(cp.H, cp.W);
    int rc = DSB_OK;
    if (row_binned(cp)) {
        // depth-ordered splats -> row items -> ONE pass over the pairs (row_binning.cu)
        rc = launch_row_binning(cp, n, k, k_rows, records, tiles_touched, reinterpret_cast<const u64*>(depth_keys_sorted), offsets,
                                ranges, layout, reinterpret_cast<u64*>(pairs), workspace, workspace_bytes, s);
        if (rc != DSB_OK) return rc;
    } else if (k > 0) {
        // Pairs written in depth order, then a stable sort on their tile bits with the digit counts the layout left;
        // the workspace holds the alternate buffer and the sort's scratch.
        const int64_t alt_bytes = ((k * 8 + 255) / 256) * 256;
        DSB_REQUIRE(workspace_bytes >= alt_bytes + sort_workspace_bytes(k), "forward_render: workspace too small");
        u64* pairs_alt = reinterpret_cast<u64*>(workspace);
        void* sort_ws = reinterpret_cast<unsigned char*>(workspace) + alt_bytes;
        const SortPlan plan = tile_sort_plan(cp);
        u32* hist = nullptr;
        {
            StageScope scope(kStageEmit, s);
            rc = sort_begin(k, plan, sort_ws, workspace_bytes - alt_bytes, &hist, s);
            if (rc != DSB_OK) return rc;
            rc = launch_emit(cp, n, k, records, tiles_touched, reinterpret_cast<const u64*>(depth_keys_sorted), offsets,
                             reinterpret_cast<u64*>(pairs), s);
            if (rc != DSB_OK) return rc;
        }
        if (hist)
            DSB_CUDA_CHECK(cudaMemcpyAsync(hist, layout, (size_t)plan.npass * 256 * sizeof(u32), cudaMemcpyDeviceToDevice, s));
        int in_alt = 0;
        StageScope scope(kStageTileSort, s);
        rc = sort_passes(reinterpret_cast<u64*>(pairs), pairs_alt, nullptr, nullptr, k, plan, sort_ws, &in_alt, s);
        if (rc != DSB_OK) return rc;
        if (in_alt) DSB_CUDA_CHECK(cudaMemcpyAsync(pairs, pairs_alt, (size_t)k * 8, cudaMemcpyDeviceToDevice, s));
    }
    StageScope scope(kStageBlendForward, s);
    return launch_blend_forward(cp, records, reinterpret_cast<const u64*>(pairs), ranges, image, final_T, final_idx, depth,
#ifdef DSB_NO_TILE_ORDER
                                nullptr, s);
#else
                                has_order ? tile_marks : nullptr, s);
#endif
}

int dsb_forward(const DsbCamera* cam, int32_t n, const float* means3d, const float* shs, const float* colors_precomp,
                const float* opacities, const float* scales, const float* rotations, const float* cov3d_precomp,
                float* records, int32_t* radii, int32_t* tiles_touched, float* cov3d, uint64_t* depth_keys,
                uint64_t* depth_keys_alt, uint32_t* offsets, int32_t* tile_marks, int32_t* ranges, uint32_t* layout,
                void* plan_workspace, int64_t plan_workspace_bytes, uint64_t* pairs, int64_t pair_capacity,
                void* render_workspace, int64_t render_workspace_bytes, float* image, float* final_T, int32_t* final_idx,
                float* depth, int64_t* k_host, int64_t* k_rows_host, int32_t* rendered_host, void* stream) {
    DSB_REQUIRE(k_host && k_rows_host && rendered_host, "forward: k_host, k_rows_host or rendered_host is null");
    *rendered_host = 0;
    int rc = dsb_forward_plan(cam, n, means3d, shs, colors_precomp, opacities, scales, rotations, cov3d_precomp, records, radii,
                              tiles_touched, cov3d, depth_keys, depth_keys_alt, offsets, tile_marks, ranges, layout,
                              plan_workspace, plan_workspace_bytes, k_host, k_rows_host, stream);
    if (rc != DSB_OK) return rc;
    const int64_t k = *k_host;
    if (k > pair_capacity ||
        (k > 0 && render_workspace_bytes < dsb_render_workspace_bytes(cam->image_height, cam->image_width, k, *k_rows_host)))
        return DSB_OK;   // the caller grows its buffers and renders
    rc = dsb_forward_render(cam, n, k, *k_rows_host, records, tiles_touched, depth_keys, offsets, pairs, tile_marks, ranges,
                            layout, render_workspace, render_workspace_bytes, image, final_T, final_idx, depth, stream);
    if (rc == DSB_OK) *rendered_host = 1;
    return rc;
}

int dsb_backward(const DsbCamera* cam, int32_t n, const float* means3d, const float* scales, const float* rotations,
                 const float* records, const float* cov3d, const int32_t* radii, const uint64_t* sorted_pairs,
                 const int32_t* ranges, const float* final_T, const int32_t* final_idx, const float* v_image,
                 const float* v_depth, const int32_t* tile_order, float* grad_acc, float* v_means3d, float* v_means2d, float* v_shs, float* v_colors, float* v_opacities,
                 float* v_scales, float* v_rotations, float* v_cov3d, int32_t accumulate, void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    if (n == 0) return DSB_OK;
    DSB_REQUIRE(grad_acc, "backward: grad_acc is null");
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    {
        StageScope scope(kStageBlendBackward, s);
        DSB_CUDA_CHECK(cudaMemsetAsync(grad_acc, 0, (size_t)n * DSB_GRAD_FLOATS * sizeof(float), s));
        rc = launch_blend_backward(cp, records, reinterpret_cast<const u64*>(sorted_pairs), ranges, final_T, final_idx,
                                   v_image, v_depth, grad_acc,
#ifdef DSB_NO_TILE_ORDER
                                   nullptr, s);
#else
                                   tile_order && tile_order_available(cp.H, cp.W) ? tile_order : nullptr, s);
#endif
    }
    if (rc != DSB_OK) return rc;
    StageScope scope(kStageGeometryBackward, s);
    return launch_geometry_backward(cp, n, means3d, scales, rotations, records, cov3d, radii, grad_acc, v_means3d,
                                    v_means2d, v_shs, v_colors, v_opacities, v_scales, v_rotations, v_cov3d, accumulate, s);
}

int dsb_preprocess_views(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d, const float* shs,
                         const float* colors_precomp, const float* opacities, const float* scales, const float* rotations,
                         const float* cov3d_precomp, float* const* records, int32_t* const* radii,
                         int32_t* const* tiles_touched, float* cov3d, uint64_t* const* depth_keys,
                         int32_t* const* tile_marks, int32_t* const* ranges, uint32_t* const* layout_hist, void* stream) {
    DSB_REQUIRE(cams && num_views >= 0 && num_views <= DSB_MAX_BATCH_VIEWS,
                "preprocess_views: between 0 and %d views per call", DSB_MAX_BATCH_VIEWS);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    if (num_views == 0) return DSB_OK;
    DSB_REQUIRE(records && radii && tiles_touched && depth_keys && tile_marks, "preprocess_views: null pointer array");
    CamParams cps[DSB_MAX_BATCH_VIEWS];
    u64* keys[DSB_MAX_BATCH_VIEWS];
    cudaStream_t s = (cudaStream_t)stream;
    for (int v = 0; v < num_views; ++v) {
        const int rc = make_cam_params(&cams[v], &cps[v]);
        if (rc != DSB_OK) return rc;
        DSB_REQUIRE(tile_marks[v], "preprocess_views: tile_marks of view %d is null", v);
        DSB_CUDA_CHECK(cudaMemsetAsync(tile_marks[v], 0, (size_t)tile_marks_bytes(cps[v].H, cps[v].W), s));
        keys[v] = reinterpret_cast<u64*>(depth_keys[v]);
    }
    DSB_REQUIRE(!ranges == !layout_hist, "preprocess_views: ranges and layout_hist go together");
    {
        StageScope scope(kStagePreprocess, s);
        const int rc = launch_preprocess_views(cps, num_views, n, means3d, shs, colors_precomp, opacities, scales, rotations,
                                               cov3d_precomp, records, radii, tiles_touched, cov3d, keys, tile_marks, s);
        if (rc != DSB_OK || !ranges) return rc;
    }
    // tile layout of all views at once (one block each): ranges, the tile sort's digit counts, the tile order
    StageScope scope(kStageRanges, s);
    int has_order = 0;
    return launch_tile_layout_views(cps[0], num_views, tile_marks, tile_sort_plan(cps[0]), layout_hist, ranges, &has_order, s);
}

int dsb_backward_blend(const DsbCamera* cam, int32_t n, const float* records, const uint64_t* sorted_pairs,
                       const int32_t* ranges, const float* final_T, const int32_t* final_idx, const float* v_image,
                       const float* v_depth, const int32_t* tile_order, float* grad_acc, int32_t keep_grad_acc, void* stream) {
    CAM_OR_RETURN(cam, cp);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    if (n == 0) return DSB_OK;
    DSB_REQUIRE(grad_acc, "backward_blend: grad_acc is null");
    cudaStream_t s = (cudaStream_t)stream;
    StageScope scope(kStageBlendBackward, s);
    if (!keep_grad_acc) DSB_CUDA_CHECK(cudaMemsetAsync(grad_acc, 0, (size_t)n * DSB_GRAD_FLOATS * sizeof(float), s));
    return launch_blend_backward(cp, records, reinterpret_cast<const u64*>(sorted_pairs), ranges, final_T, final_idx,
                                 v_image, v_depth, grad_acc,
#ifdef DSB_NO_TILE_ORDER
                                 nullptr, s);
#else
                                 tile_order && tile_order_available(cp.H, cp.W) ? tile_order : nullptr, s);
#endif
}

namespace {
int geometry_backward_views(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d, const float* scales,
                            const float* rotations, const float* cov3d, const float* const* records,
                            const int32_t* const* radii, const float* const* grad_acc, float* v_means3d, float* v_means2d,
                            float* v_shs, float* v_colors, float* v_opacities, float* v_scales, float* v_rotations,
                            float* v_cov3d, int32_t accumulate, const DensifyStats* stats, void* stream) {
    DSB_REQUIRE(cams && num_views >= 0 && num_views <= DSB_MAX_BATCH_VIEWS,
                "geometry_backward_views: between 0 and %d views per call", DSB_MAX_BATCH_VIEWS);
    DSB_REQUIRE(n >= 0, "n must be non-negative");
    if (n == 0 || num_views == 0) return DSB_OK;
    CamParams cps[DSB_MAX_BATCH_VIEWS];
    for (int v = 0; v < num_views; ++v) {
        const int rc = make_cam_params(&cams[v], &cps[v]);
        if (rc != DSB_OK) return rc;
    }
    cudaStream_t s = (cudaStream_t)stream;
    StageScope scope(kStageGeometryBackward, s);
    return launch_geometry_backward_views(cps, num_views, n, means3d, scales, rotations, cov3d, records, radii, grad_acc,
                                          v_means3d, v_means2d, v_shs, v_colors, v_opacities, v_scales, v_rotations, v_cov3d,
                                          accumulate, s, stats);
}
}  // namespace

int dsb_geometry_backward_views(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d,
                                const float* scales, const float* rotations, const float* cov3d,
                                const float* const* records, const int32_t* const* radii, const float* const* grad_acc,
                                float* v_means3d, float* v_means2d, float* v_shs, float* v_colors, float* v_opacities,
                                float* v_scales, float* v_rotations, float* v_cov3d, int32_t accumulate, void* stream) {
    return geometry_backward_views(cams, num_views, n, means3d, scales, rotations, cov3d, records, radii, grad_acc,
                                   v_means3d, v_means2d, v_shs, v_colors, v_opacities, v_scales, v_rotations, v_cov3d,
                                   accumulate, nullptr, stream);
}

int dsb_geometry_backward_views_stats(const DsbCamera* cams, int32_t num_views, int32_t n, const float* means3d,
                                      const float* scales, const float* rotations, const float* cov3d,
                                      const float* const* records, const int32_t* const* radii,
                                      const float* const* grad_acc, float* v_means3d, float* v_means2d, float* v_shs,
                                      float* v_colors, float* v_opacities, float* v_scales, float* v_rotations,
                                      float* v_cov3d, int32_t accumulate, float norm_scale_x, float norm_scale_y,
                                      float* grad_norm_sum, float* visible_count, float* max_radius, void* stream) {
    DSB_REQUIRE(grad_norm_sum && visible_count && max_radius, "geometry_backward_views_stats: null statistics array");
    DensifyStats st;
    st.grad_norm_sum = grad_norm_sum; st.visible_count = visible_count; st.max_radius = max_radius;
    st.scale_x = norm_scale_x; st.scale_y = norm_scale_y;
    return geometry_backward_views(cams, num_views, n, means3d, scales, rotations, cov3d, records, radii, grad_acc,
                                   v_means3d, v_means2d, v_shs, v_colors, v_opacities, v_scales, v_rotations, v_cov3d,
                                   accumulate, &st, stream);
}

// Torch-free forward with the argument list of the reference's rasterizer_forward_core_deepsense
// (cpp/ds_cuda_rasterizer/rasterizer_cuda.hpp:4-9): device pointers in, device image out, every intermediate
// taken from and returned to the stream-ordered allocator inside the call.
int dsb_forward_core(const float* means3d, const float* shs, const float* opacities, const float* scales,
                     const float* rotations, int32_t n, const float* view_matrix, const float* proj_matrix,
                     const float* camera_position, int32_t image_width, int32_t image_height, float tan_fovx,
                     float tan_fovy, float scale_modifier, int32_t max_sh_degree, int32_t sh_degree, float* output_image,
                     void* stream) {
    DSB_REQUIRE(n >= 0 && output_image, "forward_core: bad arguments");
    DsbCamera cam = {};
    cam.image_height = image_height; cam.image_width = image_width;
    cam.tanfovx = tan_fovx; cam.tanfovy = tan_fovy; cam.scale_modifier = scale_modifier;
    cam.sh_degree = sh_degree; cam.max_sh_degree = max_sh_degree;
    cam.matrices_transposed = 0;                 // row-major [R|t] and P*V, as the reference's C++ entry takes them
    cam.flags = DSB_FLAG_DROP_LAST_SPLAT;        // what the reference's pair count does (cpp/rasterizer_torch.cu:97-104)
    cam.viewmatrix = view_matrix; cam.projmatrix = proj_matrix; cam.campos = camera_position; cam.bg = nullptr;
    CAM_OR_RETURN(&cam, cp);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t pixels = (size_t)image_height * image_width;
    if (n == 0) {
        DSB_CUDA_CHECK(cudaMemsetAsync(output_image, 0, pixels * 3 * sizeof(float), s));
        return DSB_OK;
    }
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    const size_t nn = (size_t)n;
    const size_t b_records = up(nn * 48), b_i32 = up(nn * 4), b_cov = up(nn * 24), b_keys = up(nn * 8);
    const size_t b_marks = up((size_t)tile_marks_bytes(cp.H, cp.W)), b_plan = up((size_t)plan_workspace_bytes(n));
    const size_t b_ranges = up(((size_t)cp.tiles_x * cp.tiles_y + 1) * 4), b_pix = up(pixels * 4), b_layout = up(kLayoutWords * 4);
    unsigned char* a = nullptr;   // arena 1: everything whose size is known before the pair count
    const size_t bytes1 = b_records + 3 * b_i32 + b_cov + 2 * b_keys + b_marks + b_plan + b_ranges + b_layout + 2 * b_pix;
    DSB_CUDA_CHECK(cudaMallocAsync(reinterpret_cast<void**>(&a), bytes1, s));
    unsigned char* p = a;
    auto take = [&p](size_t b) { unsigned char* r = p; p += b; return r; };
    float* records = reinterpret_cast<float*>(take(b_records));
    int32_t* radii = reinterpret_cast<int32_t*>(take(b_i32));
    int32_t* tiles = reinterpret_cast<int32_t*>(take(b_i32));
    uint32_t* offsets = reinterpret_cast<uint32_t*>(take(b_i32));
    float* cov3d = reinterpret_cast<float*>(take(b_cov));
    uint64_t* keys = reinterpret_cast<uint64_t*>(take(b_keys));
    uint64_t* keys_alt = reinterpret_cast<uint64_t*>(take(b_keys));
    int32_t* marks = reinterpret_cast<int32_t*>(take(b_marks));
    void* plan_ws = take(b_plan);
    int32_t* ranges = reinterpret_cast<int32_t*>(take(b_ranges));
    uint32_t* layout = reinterpret_cast<uint32_t*>(take(b_layout));
    float* final_T = reinterpret_cast<float*>(take(b_pix));
    int32_t* final_idx = reinterpret_cast<int32_t*>(take(b_pix));
    int64_t k = 0, k_rows = 0;
    int rc = dsb_forward_plan(&cam, n, means3d, shs, nullptr, opacities, scales, rotations, nullptr, records, radii, tiles, cov3d,
                              keys, keys_alt, offsets, marks, ranges, layout, plan_ws, (int64_t)b_plan, &k, &k_rows, stream);
    unsigned char* b = nullptr;   // arena 2: pair list and render workspace
    if (rc == DSB_OK) {
        const size_t b_pairs = up((size_t)(k > 0 ? k : 1) * 8);
        const size_t b_render = up((size_t)dsb_render_workspace_bytes(image_height, image_width, k, k_rows));
        const cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&b), b_pairs + b_render, s);
        if (e != cudaSuccess) {
            set_error("forward_core: cudaMallocAsync of the pair list failed: %s", cudaGetErrorString(e));
            rc = DSB_ERR_CUDA;
        } else {
            rc = dsb_forward_render(&cam, n, k, k_rows, records, tiles, keys, offsets, reinterpret_cast<uint64_t*>(b), marks, ranges,
                                    layout, b + b_pairs, (int64_t)b_render, output_image, final_T, final_idx, nullptr, stream);
        }
    }
    if (b) cudaFreeAsync(b, s);
    cudaFreeAsync(a, s);
    return rc;
}

int64_t dsb_image_loss_workspace_bytes(int32_t image_height, int32_t image_width) {
    return (image_height > 0 && image_width > 0) ? image_loss_workspace_bytes(image_height, image_width) : 0;
}

int dsb_image_loss_backward(const float* image, const float* target, int32_t image_height, int32_t image_width,
                            float lambda_dssim, void* workspace, int64_t workspace_bytes, float* v_image, float* loss,
                            void* stream) {
    return launch_image_loss(image, target, image_height, image_width, lambda_dssim, workspace, workspace_bytes, v_image, loss,
                             (cudaStream_t)stream);
}

int dsb_l1_loss_backward_u8(const float* image, const uint8_t* target, int32_t image_height, int32_t image_width,
                            float* v_image, float* loss, void* stream) {
    return launch_l1_loss_u8(image, target, image_height, image_width, v_image, loss, (cudaStream_t)stream);
}

int dsb_adam_step(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, int64_t count, double lr,
                  double beta1, double beta2, double eps, int32_t step, double grad_scale, void* stream) {
    return launch_adam(params, grads, exp_avg, exp_avg_sq, count, lr, beta1, beta2, eps, step, grad_scale, (cudaStream_t)stream);
}

int dsb_export_reference_lists(const uint64_t* sorted_pairs, int64_t k, const float* records, int64_t* keys, int32_t* ids,
                               void* stream) {
    DSB_REQUIRE(k >= 0, "k must be non-negative");
    return launch_export(reinterpret_cast<const u64*>(sorted_pairs), k, records, keys, ids, (cudaStream_t)stream);
}

}  // extern "C"
