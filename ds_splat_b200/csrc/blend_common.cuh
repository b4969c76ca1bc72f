// Shared by the forward and backward blend kernels: how a tile's 256 pixels map to warps, and the test
// "can this splat reach this warp's pixels at all?".
//
// Warps work independently.  In the forward blend a warp owns a compact 8x4 block of a 16x16 tile (not a 16x2
// strip: for a splat of a given size the compact shape is met about 15% less often and has more live pixels
// when it is met); block w of a tile sits at column (w & 1), row (w >> 1) of the 2x4 arrangement and lane l is
// pixel (l & 7, l >> 3).  The backward blend uses larger blocks (several pixels per lane) and the same test
// through splat_reaches_rect.
//
// A pixel receives a splat only if opacity * exp(-q) >= 1/255, i.e. q <= tau = ln(255 * opacity), where
// q(d) = 0.5 (a dx^2 + c dy^2) + b dx dy is the conic form at the pixel's offset d from the splat centre.
// The exact minimum of q over the warp's rectangle of pixel centres is computed in closed form (q is
// convex, so the minimum over a rectangle that does not contain the centre lies on one of the at most
// two edges facing it) and compared with tau plus a margin.  The margin makes the test conservative
// against rounding: a splat is dropped only when no pixel of the warp could pass the per-pixel test, so
// results are exactly those of testing every pixel, and the per-pixel test stays in place.
//
// The reference fetches and evaluates every splat of the tile's list for all 256 pixels
// (cpp/rasterizer_kernels.cu:386-414, cpp/gsplat/backward.cu:112-145); its lists come from the 3-sigma
// circle's bounding square, so for elongated or faint splats most of those evaluations end in a skip.
#pragma once
#include "common.cuh"

namespace dsb {

constexpr float kCullMargin = 0.02f;
constexpr int kWarpPixelsX = 8, kWarpPixelsY = 4;

struct WarpPixels {
    int x, y;        // this lane's pixel
    float x0, y0;    // pixel-coordinate origin of the warp's 8x4 block
};

__device__ __forceinline__ WarpPixels warp_pixels(const int tile_x, const int tile_y, const int warp, const int lane) {
    WarpPixels p;
    const int bx = tile_x * kTile + (warp & 1) * kWarpPixelsX, by = tile_y * kTile + (warp >> 1) * kWarpPixelsY;
    p.x = bx + (lane & 7);
    p.y = by + (lane >> 3);
    p.x0 = (float)bx;
    p.y0 = (float)by;
    return p;
}

// True when some pixel centre of the BX x BY block at origin (x0, y0) may have q <= thr.
// (gx, gy) splat centre in pixels, (a, b, c) conic.
template <int BX, int BY>
__device__ __forceinline__ bool splat_reaches_rect(const float gx, const float gy, const float a, const float b,
                                                   const float c, const float thr, const float x0, const float y0) {
    // Anything that is not a proper ellipse with a finite threshold is left to the per-pixel test.
    if (!(a > 0.f && c > 0.f && a * c > b * b) || !(thr == thr)) return true;
    const float dxl = x0 + 0.5f - gx, dxh = dxl + (float)(BX - 1);
    const float dyl = y0 + 0.5f - gy, dyh = dyl + (float)(BY - 1);
    const float ex = fminf(fmaxf(0.f, dxl), dxh);  // offset of the block's nearest column / row to the centre
    const float ey = fminf(fmaxf(0.f, dyl), dyh);
    const bool in_x = ex == 0.f, in_y = ey == 0.f;
    if (in_x && in_y) return !(0.f > thr);
    float q1 = 3.0e38f, q2 = 3.0e38f;
    if (!in_x) {  // edge dx = ex, best dy on it
        const float dy = fminf(fmaxf(-b / c * ex, dyl), dyh);
        q1 = 0.5f * (a * ex * ex + c * dy * dy) + b * ex * dy;
    }
    if (!in_y) {  // edge dy = ey, best dx on it
        const float dx = fminf(fmaxf(-b / a * ey, dxl), dxh);
        q2 = 0.5f * (a * dx * dx + c * ey * ey) + b * dx * ey;
    }
    return !(fminf(q1, q2) > thr);
}

// The same test with the two per-splat constants handed in: thr = ln(255 opacity) + margin and nbc = -b / c.
template <int BX, int BY>
__device__ __forceinline__ bool splat_reaches_rect_pre(const float gx, const float gy, const float a, const float b,
                                                       const float c, const float thr, const float nbc, const float x0,
                                                       const float y0) {
    if (!(a > 0.f && c > 0.f && a * c > b * b) || !(thr == thr)) return true;
    const float dxl = x0 + 0.5f - gx, dxh = dxl + (float)(BX - 1);
    const float dyl = y0 + 0.5f - gy, dyh = dyl + (float)(BY - 1);
    const float ex = fminf(fmaxf(0.f, dxl), dxh);
    const float ey = fminf(fmaxf(0.f, dyl), dyh);
    const bool in_x = ex == 0.f, in_y = ey == 0.f;
    if (in_x && in_y) return !(0.f > thr);
    float q1 = 3.0e38f, q2 = 3.0e38f;
    if (!in_x) {
        const float dy = fminf(fmaxf(nbc * ex, dyl), dyh);
        q1 = 0.5f * (a * ex * ex + c * dy * dy) + b * ex * dy;
    }
    if (!in_y) {
        const float dx = fminf(fmaxf(-b / a * ey, dxl), dxh);
        q2 = 0.5f * (a * dx * dx + c * ey * ey) + b * dx * ey;
    }
    return !(fminf(q1, q2) > thr);
}
__device__ __forceinline__ bool splat_reaches_block_pre(const float gx, const float gy, const float a, const float b,
                                                        const float c, const float thr, const float nbc, const float x0,
                                                        const float y0) {
    return splat_reaches_rect_pre<kWarpPixelsX, kWarpPixelsY>(gx, gy, a, b, c, thr, nbc, x0, y0);
}

// The 8x4 block of warp_pixels().
__device__ __forceinline__ bool splat_reaches_block(const float gx, const float gy, const float a, const float b,
                                                    const float c, const float thr, const float x0, const float y0) {
    return splat_reaches_rect<kWarpPixelsX, kWarpPixelsY>(gx, gy, a, b, c, thr, x0, y0);
}

}  // namespace dsb
