// Stage (e): per-tile front-to-back alpha blending.
//
// Takes the place of the reference's render_image_kernel (cpp/rasterizer_kernels.cu:341-431), which runs
// one 256-thread block per 16x16 tile in lock step: rounds of 256 list entries, two block barriers per
// round, every entry evaluated for every pixel until all 256 pixels have stopped.
//
// Here each WARP is on its own (as in the backward blend): a warp owns a compact 8x4-pixel block of a tile
// (blend_common.cuh) and walks the tile's depth-ordered list in chunks of 32 entries, with no block barrier
// anywhere, so a warp stops as soon as ITS 32 pixels have stopped.  (Several pixels per lane, which pays in
// the backward blend, does not here: measured 0.31-0.35 ms against 0.30 ms at 1M splats / 1080p, because
// a larger block keeps running until its slowest pixel saturates -- and the changed floating-point
// contraction of the unrolled loop moved isolated pixels by 5e-5, outside the 1e-5 bound.)
//   * fetch + cull: lane l fetches entry l of the chunk (48-byte record) and tests in closed form whether
//     the splat can reach the warp's pixels at all; a ballot gives the survivors;
//   * blend: survivors are parked in the warp's private shared-memory slice and each pixel consumes them
//     in list order until its transmittance would fall under 1e-4.
//
// Per-pixel arithmetic (order of operations, 0.999 alpha clamp, 1/255 skip, no background term) is the
// reference's and the cull test is conservative, so images agree to rounding and final_idx exactly.
//
// Optional depth map (the reference has none): the DEPTH instantiation blends the splat's view-space z like
// a fourth colour channel, depth = sum z_i alpha_i T_i.
#include "blend_common.cuh"
#include "tma.cuh"

namespace dsb {

namespace {

// How a warp gets the records of a chunk of 32 list entries.  Variant 0 is the product path; the others exist so that
// the alternatives can be measured against it on the same lists (dsb_debug_blend_forward_variant) and are checked to
// render bit-identical images:
//   0  three 16-byte loads per lane through the read-only path, survivors parked with ordinary shared stores;
//   1  every lane asks the bulk copy engine for its 48-byte record (cp.async.bulk global -> shared) onto the warp's
//      mbarrier, then reads it back from shared memory for the cull (bounded wait);
//   2  a gather pass first writes the records in LIST order into a packed stream (K x 48 bytes), so that a chunk is
//      ONE contiguous bulk copy of up to 1536 bytes issued by lane 0;
//   3  variant 0 with the two per-splat constants of the cull, ln(255 opacity) + margin and -b/c, read from the
//      record (lanes rect_x / rect_y of a copy of the records) instead of being recomputed by every warp.
constexpr int kVariants = 4;

// Warps never synchronise with each other and stop at different list positions; small thread blocks give a
// finished warp's slots back to the scheduler instead of holding them until the block's slowest warp ends.
#ifndef DSB_FWD_THREADS
#define DSB_FWD_THREADS 64
#endif
constexpr int kThreads = DSB_FWD_THREADS;
constexpr int kWarps = kThreads / 32;
constexpr int kWarpsPerTile = kTilePixels / 32;
#ifndef DSB_FWD_PREFETCH
#define DSB_FWD_PREFETCH 0  // 1: fetch the next chunk's records while the current chunk is blended (costs occupancy)
#endif

struct Fetched {
    float4 q0, q1;
    float blue, z, e0, e1;   // e0, e1: the record's last two lanes (tile rectangle; cull constants in variant 3)
    bool have;
};

__device__ __forceinline__ Fetched fetch_entry(const float4* __restrict__ records, const u64* __restrict__ sorted,
                                               const int pos, const int end) {
    Fetched f;
    f.q0 = make_float4(0, 0, 0, 0); f.q1 = f.q0; f.blue = 0.f; f.z = 0.f; f.e0 = 0.f; f.e1 = 0.f;
    f.have = pos < end;
    if (f.have) {
        const u32 id = (u32)sorted[pos];
        const float4* r = records + (size_t)id * 3;
        f.q0 = __ldg(r); f.q1 = __ldg(r + 1);
        const float4 q2 = __ldg(r + 2);
        f.blue = q2.x; f.z = q2.y; f.e0 = q2.z; f.e1 = q2.w;
    }
    return f;
}

template <bool DEPTH, int VARIANT>
__global__ void __launch_bounds__(kThreads)
blend_forward_kernel(const int W, const int H, const int tiles_x, const int num_tiles,
                     const float4* __restrict__ records, const u64* __restrict__ sorted,
                     const int32_t* __restrict__ ranges, float* __restrict__ image, float* __restrict__ final_T,
                     int32_t* __restrict__ final_idx, float* __restrict__ depth, const int32_t* __restrict__ tile_order,
                     int* __restrict__ device_status, const int band_tile0, const int band_tile1) {
    constexpr bool kBulk = VARIANT == 1 || VARIANT == 2;
    __shared__ float4 s_q0[kBulk ? 1 : kWarps][32];  // x, y, conic a, conic b
    __shared__ float4 s_q1[kBulk ? 1 : kWarps][32];  // conic c, opacity, r, g
    __shared__ float s_b[kBulk ? 1 : kWarps][32];    // b
    __shared__ float s_z[DEPTH ? kWarps : 1][32];  // view-space depth
    __shared__ __align__(16) float4 s_raw[kBulk ? kWarps : 1][32][3];   // whole records as the copy engine delivers them
    __shared__ __align__(8) uint64_t s_bar[kBulk ? kWarps : 1];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wb = blockIdx.x * kWarps + warp;   // warp-level pixel block: 8 per tile
    const int slot = wb / kWarpsPerTile;
    if (slot >= num_tiles) return;               // whole warps only; no block-wide barrier below
    const int tile = tile_order ? tile_order[slot] : slot;   // longest lists first when the order is known
    if ((unsigned)tile >= (unsigned)num_tiles) return;       // a caller's stale order must not index outside the ranges
    if (tile < band_tile0 || tile >= band_tile1) return;     // a view rendered in bands: the other bands' pixels are not touched
    const WarpPixels wp = warp_pixels(tile % tiles_x, tile / tiles_x, wb % kWarpsPerTile, lane);
    const int x = wp.x, y = wp.y;
    const bool inside = x < W && y < H;
    const int start = ranges[tile], end = ranges[tile + 1];
    const float pxf = x + 0.5f, pyf = y + 0.5f;

    float T = 1.0f, c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, cz = 0.0f;
    int last = 0;
    bool done = !inside;

    float4* q0s = s_q0[kBulk ? 0 : warp];
    float4* q1s = s_q1[kBulk ? 0 : warp];
    float* bs = s_b[kBulk ? 0 : warp];
    float* zs = s_z[DEPTH ? warp : 0];
    float4 (*raw)[3] = s_raw[kBulk ? warp : 0];
    uint64_t* bar = &s_bar[kBulk ? warp : 0];
    u32 phase = 0;
    bool copies_lost = false;
    if (kBulk) {
        if (lane == 0) mbar_init(bar, 1);
        __syncwarp();
    }

#if DSB_FWD_PREFETCH
    Fetched nxt = fetch_entry(records, sorted, start + lane, end);
#endif
    for (int base = start; base < end; base += 32) {
        if (__all_sync(0xffffffffu, done)) break;
        Fetched cur;
        if (kBulk) {
            // the chunk's records through the copy engine onto the warp's mbarrier
            const int pos = base + lane;
            cur.have = pos < end;
            const int cnt = min(32, end - base);
            if (lane == 0) mbar_arrive_expect_tx(bar, 48u * (u32)cnt);
            __syncwarp();
            if (VARIANT == 1) {
                if (cur.have) bulk_load(&raw[lane][0], records + (size_t)(u32)sorted[pos] * 3, 48u, bar);
            } else {
                if (lane == 0) bulk_load(&raw[0][0], records + (size_t)base * 3, 48u * (u32)cnt, bar);   // records = packed stream
            }
            const bool ok = mbar_wait_bounded(bar, phase);
            phase ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {   // never seen; the image is incomplete and the host is told
                if (lane == 0) atomicExch(device_status, DSB_ERR_DEVICE_WAIT_EXPIRED);
                copies_lost = true;
                break;
            }
            cur.q0 = raw[lane][0]; cur.q1 = raw[lane][1];
            cur.blue = raw[lane][2].x; cur.z = raw[lane][2].y;
        } else {
#if DSB_FWD_PREFETCH
            cur = nxt;
            nxt = fetch_entry(records, sorted, base + 32 + lane, end);
#else
            cur = fetch_entry(records, sorted, base + lane, end);
#endif
        }
        bool hit = false;
        if (cur.have) {
            if (VARIANT == 3) {
                hit = splat_reaches_block_pre(cur.q0.x, cur.q0.y, cur.q0.z, cur.q0.w, cur.q1.x, cur.e0, cur.e1, wp.x0, wp.y0);
            } else {
                const float thr = __logf(255.0f * cur.q1.y) + kCullMargin;
                hit = splat_reaches_block(cur.q0.x, cur.q0.y, cur.q0.z, cur.q0.w, cur.q1.x, thr, wp.x0, wp.y0);
            }
        }
        const u32 todo = __ballot_sync(0xffffffffu, hit);
        if (todo == 0) continue;
        if (!kBulk) {
            q0s[lane] = cur.q0; q1s[lane] = cur.q1; bs[lane] = cur.blue;
        }
        if (DEPTH) zs[lane] = cur.z;
        __syncwarp();
        for (u32 m = todo; m != 0 && !done; m &= m - 1) {
            const int t = __ffs(m) - 1;
            const float4 a = kBulk ? raw[t][0] : q0s[t];
            const float4 b = kBulk ? raw[t][1] : q1s[t];
            const float dx = pxf - a.x, dy = pyf - a.y;
            const float power = -0.5f * (a.z * dx * dx + b.x * dy * dy) - a.w * dx * dy;
            const float alpha = min(0.999f, b.y * __expf(power));
            if (power >= 0.f || alpha < 1.0f / 255.0f) continue;
            const float Tn = (1.0f - alpha) * T;
            if (!(Tn >= 0.0001f)) { done = true; break; }
            const float wgt = alpha * T;
            c0 += wgt * b.z; c1 += wgt * b.w; c2 += wgt * (kBulk ? raw[t][2].x : bs[t]);
            if (DEPTH) cz += wgt * zs[t];
            T = Tn;
            last = base + t;
        }
        __syncwarp();  // the slice is reused by the next chunk
    }
    if (kBulk && copies_lost) {   // do not retire with copies of this warp in flight: one more bounded wait
        for (u32 poll = 0; poll < (1u << 20); ++poll) {
            if (mbar_try_wait(bar, phase ^ 1u)) break;
            __nanosleep(64);
        }
    }
    if (inside) {
        const size_t pix = (size_t)y * W + x;
        image[3 * pix] = c0; image[3 * pix + 1] = c1; image[3 * pix + 2] = c2;
        final_T[pix] = T;
        final_idx[pix] = last;
        if (DEPTH) depth[pix] = cz;
    }
}

// Records in list order, 48 bytes per list entry (variant 2): three threads per entry, 16 bytes each.
__global__ void pack_records_kernel(const u64* __restrict__ sorted, const u32 k, const float4* __restrict__ records,
                                    float4* __restrict__ packed) {
    const u32 i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 3u * k) return;
    const u32 e = i / 3u, q = i - 3u * e;
    packed[i] = __ldg(records + (size_t)(u32)sorted[e] * 3 + q);
}

// A copy of the records whose last two lanes hold the cull's per-splat constants (variant 3).
__global__ void cull_lanes_kernel(const float4* __restrict__ records, const int n, float4* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float4 q0 = records[(size_t)i * 3], q1 = records[(size_t)i * 3 + 1];
    float4 q2 = records[(size_t)i * 3 + 2];
    q2.z = __logf(255.0f * q1.y) + kCullMargin;
    q2.w = -q0.w / q1.x;
    out[(size_t)i * 3] = q0; out[(size_t)i * 3 + 1] = q1; out[(size_t)i * 3 + 2] = q2;
}

template <bool DEPTH, int VARIANT>
int launch_variant(const CamParams& cp, const float4* records, const u64* sorted, const int32_t* ranges, float* image,
                   float* final_T, int32_t* final_idx, float* depth, const int32_t* tile_order, cudaStream_t s) {
    const int num_tiles = cp.tiles_x * cp.tiles_y;
    const int grid = (num_tiles * kWarpsPerTile + kWarps - 1) / kWarps;
    int* device_status = nullptr;
    const int rc = device_status_address(&device_status);
    if (rc != DSB_OK) return rc;
    blend_forward_kernel<DEPTH, VARIANT><<<grid, kThreads, 0, s>>>(cp.W, cp.H, cp.tiles_x, num_tiles, records, sorted, ranges, image,
                                                                 final_T, final_idx, depth, tile_order, device_status,
                                                                 cp.band_y0 * cp.tiles_x, cp.band_y1 * cp.tiles_x);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace

// depth may be null (no depth map wanted); tile_order may be null (tiles are then taken in index order).
int launch_blend_forward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                         float* image, float* final_T, int32_t* final_idx, float* depth, const int32_t* tile_order,
                         cudaStream_t s) {
    DSB_REQUIRE(ranges && image && final_T && final_idx, "blend_forward: null pointer");
    const float4* rec = reinterpret_cast<const float4*>(records);
    if (depth) return launch_variant<true, 0>(cp, rec, sorted, ranges, image, final_T, final_idx, depth, tile_order, s);
    return launch_variant<false, 0>(cp, rec, sorted, ranges, image, final_T, final_idx, nullptr, tile_order, s);
}

// The forward blend with another way of fetching the records (see the head of this file), for measurements and for
// the test that all of them render the same image.  scratch: k x 48 bytes for variant 2, n x 48 bytes for variant 3.
int launch_blend_forward_variant(const CamParams& cp, int variant, int n, int64_t k, const float* records, const u64* sorted,
                                 const int32_t* ranges, float* image, float* final_T, int32_t* final_idx,
                                 const int32_t* tile_order, void* scratch, int64_t scratch_bytes, cudaStream_t s) {
    DSB_REQUIRE(ranges && image && final_T && final_idx && records, "blend_forward: null pointer");
    DSB_REQUIRE(variant >= 0 && variant < kVariants, "blend_forward: variants are 0..%d", kVariants - 1);
    DSB_REQUIRE(k >= 0 && k < DSB_MAX_PAIRS && n >= 0, "blend_forward: bad counts");
    const float4* rec = reinterpret_cast<const float4*>(records);
    if (variant == 2 && k > 0) {
        DSB_REQUIRE(scratch && scratch_bytes >= k * 48 && ((uintptr_t)scratch & 15) == 0, "blend_forward: variant 2 needs k x 48 bytes of scratch");
        pack_records_kernel<<<(unsigned)((3 * k + 255) / 256), 256, 0, s>>>(sorted, (u32)k, rec, reinterpret_cast<float4*>(scratch));
        DSB_LAUNCH_CHECK();
        rec = reinterpret_cast<const float4*>(scratch);
    }
    if (variant == 3 && n > 0) {
        DSB_REQUIRE(scratch && scratch_bytes >= (int64_t)n * 48 && ((uintptr_t)scratch & 15) == 0, "blend_forward: variant 3 needs n x 48 bytes of scratch");
        cull_lanes_kernel<<<(n + 255) / 256, 256, 0, s>>>(rec, n, reinterpret_cast<float4*>(scratch));
        DSB_LAUNCH_CHECK();
        rec = reinterpret_cast<const float4*>(scratch);
    }
    StageScope scope(kStageBlendForward, s);
    switch (variant) {
        case 1: return launch_variant<false, 1>(cp, rec, sorted, ranges, image, final_T, final_idx, nullptr, tile_order, s);
        case 2: return launch_variant<false, 2>(cp, rec, sorted, ranges, image, final_T, final_idx, nullptr, tile_order, s);
        case 3: return launch_variant<false, 3>(cp, rec, sorted, ranges, image, final_T, final_idx, nullptr, tile_order, s);
        default: return launch_variant<false, 0>(cp, rec, sorted, ranges, image, final_T, final_idx, nullptr, tile_order, s);
    }
}

}  // namespace dsb
