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

namespace dsb {

namespace {

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
    float blue, z;
    bool have;
};

__device__ __forceinline__ Fetched fetch_entry(const float4* __restrict__ records, const u64* __restrict__ sorted,
                                               const int pos, const int end) {
    Fetched f;
    f.q0 = make_float4(0, 0, 0, 0); f.q1 = f.q0; f.blue = 0.f; f.z = 0.f;
    f.have = pos < end;
    if (f.have) {
        const u32 id = (u32)sorted[pos];
        const float4* r = records + (size_t)id * 3;
        f.q0 = __ldg(r); f.q1 = __ldg(r + 1);
        const float4 q2 = __ldg(r + 2);
        f.blue = q2.x; f.z = q2.y;
    }
    return f;
}

template <bool DEPTH>
__global__ void __launch_bounds__(kThreads)
blend_forward_kernel(const int W, const int H, const int tiles_x, const int num_tiles,
                     const float4* __restrict__ records, const u64* __restrict__ sorted,
                     const int32_t* __restrict__ ranges, float* __restrict__ image, float* __restrict__ final_T,
                     int32_t* __restrict__ final_idx, float* __restrict__ depth, const int32_t* __restrict__ tile_order) {
    __shared__ float4 s_q0[kWarps][32];  // x, y, conic a, conic b
    __shared__ float4 s_q1[kWarps][32];  // conic c, opacity, r, g
    __shared__ float s_b[kWarps][32];    // b
    __shared__ float s_z[DEPTH ? kWarps : 1][32];  // view-space depth

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wb = blockIdx.x * kWarps + warp;   // warp-level pixel block: 8 per tile
    const int slot = wb / kWarpsPerTile;
    if (slot >= num_tiles) return;               // whole warps only; no block-wide barrier below
    const int tile = tile_order ? tile_order[slot] : slot;   // longest lists first when the order is known
    if ((unsigned)tile >= (unsigned)num_tiles) return;       // a caller's stale order must not index outside the ranges
    const WarpPixels wp = warp_pixels(tile % tiles_x, tile / tiles_x, wb % kWarpsPerTile, lane);
    const int x = wp.x, y = wp.y;
    const bool inside = x < W && y < H;
    const int start = ranges[tile], end = ranges[tile + 1];
    const float pxf = x + 0.5f, pyf = y + 0.5f;

    float T = 1.0f, c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, cz = 0.0f;
    int last = 0;
    bool done = !inside;

    float4* q0s = s_q0[warp];
    float4* q1s = s_q1[warp];
    float* bs = s_b[warp];
    float* zs = s_z[DEPTH ? warp : 0];

#if DSB_FWD_PREFETCH
    Fetched nxt = fetch_entry(records, sorted, start + lane, end);
#endif
    for (int base = start; base < end; base += 32) {
        if (__all_sync(0xffffffffu, done)) break;
#if DSB_FWD_PREFETCH
        const Fetched cur = nxt;
        nxt = fetch_entry(records, sorted, base + 32 + lane, end);
#else
        const Fetched cur = fetch_entry(records, sorted, base + lane, end);
#endif
        bool hit = false;
        if (cur.have) {
            const float thr = __logf(255.0f * cur.q1.y) + kCullMargin;
            hit = splat_reaches_block(cur.q0.x, cur.q0.y, cur.q0.z, cur.q0.w, cur.q1.x, thr, wp.x0, wp.y0);
        }
        const u32 todo = __ballot_sync(0xffffffffu, hit);
        if (todo == 0) continue;
        q0s[lane] = cur.q0; q1s[lane] = cur.q1; bs[lane] = cur.blue;
        if (DEPTH) zs[lane] = cur.z;
        __syncwarp();
        for (u32 m = todo; m != 0 && !done; m &= m - 1) {
            const int t = __ffs(m) - 1;
            const float4 a = q0s[t];
            const float4 b = q1s[t];
            const float dx = pxf - a.x, dy = pyf - a.y;
            const float power = -0.5f * (a.z * dx * dx + b.x * dy * dy) - a.w * dx * dy;
            const float alpha = min(0.999f, b.y * __expf(power));
            if (power >= 0.f || alpha < 1.0f / 255.0f) continue;
            const float Tn = (1.0f - alpha) * T;
            if (!(Tn >= 0.0001f)) { done = true; break; }
            const float wgt = alpha * T;
            c0 += wgt * b.z; c1 += wgt * b.w; c2 += wgt * bs[t];
            if (DEPTH) cz += wgt * zs[t];
            T = Tn;
            last = base + t;
        }
        __syncwarp();  // the slice is reused by the next chunk
    }
    if (inside) {
        const size_t pix = (size_t)y * W + x;
        image[3 * pix] = c0; image[3 * pix + 1] = c1; image[3 * pix + 2] = c2;
        final_T[pix] = T;
        final_idx[pix] = last;
        if (DEPTH) depth[pix] = cz;
    }
}

}  // namespace

// depth may be null (no depth map wanted); tile_order may be null (tiles are then taken in index order).
int launch_blend_forward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                         float* image, float* final_T, int32_t* final_idx, float* depth, const int32_t* tile_order,
                         cudaStream_t s) {
    DSB_REQUIRE(ranges && image && final_T && final_idx, "blend_forward: null pointer");
    const int num_tiles = cp.tiles_x * cp.tiles_y;
    const int grid = (num_tiles * kWarpsPerTile + kWarps - 1) / kWarps;
    if (depth)
        blend_forward_kernel<true><<<grid, kThreads, 0, s>>>(cp.W, cp.H, cp.tiles_x, num_tiles,
                                                            reinterpret_cast<const float4*>(records), sorted, ranges, image,
                                                            final_T, final_idx, depth, tile_order);
    else
        blend_forward_kernel<false><<<grid, kThreads, 0, s>>>(cp.W, cp.H, cp.tiles_x, num_tiles,
                                                             reinterpret_cast<const float4*>(records), sorted, ranges, image,
                                                             final_T, final_idx, nullptr, tile_order);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace dsb
