// Shared by the forward and backward blend kernels: which 16x2-pixel strips of a tile can a splat reach?
//
// A 256-thread block owns a 16x16 tile; warp w owns the strip of rows 2w and 2w+1.  A pixel receives a
// splat only if opacity * exp(-q) >= 1/255, i.e. q <= tau = ln(255 * opacity), where
// q(d) = 0.5 (a dx^2 + c dy^2) + b dx dy is the conic form at the pixel's offset d from the splat centre.
// For each strip the exact minimum of q over the strip's pixel-centre rectangle is computed in closed
// form (q is convex, so the minimum over a rectangle that does not contain the centre lies on one of
// the at most two edges facing it) and compared with tau plus a margin.  The margin makes the test
// conservative against rounding: a strip is dropped only when no pixel in it could pass the per-pixel
// test, so results are exactly those of testing every pixel, and the per-pixel test stays in place.
//
// The reference fetches and evaluates every splat of the tile's list for all 256 pixels
// (cpp/rasterizer_kernels.cu:386-414, cpp/gsplat/backward.cu:112-145); its lists come from the 3-sigma
// circle's bounding square, so for elongated or faint splats most of those evaluations end in a skip.
#pragma once
#include "common.cuh"

namespace dsb {

constexpr float kStripMargin = 0.02f;

// Bit w of the result is set when strip w of the tile at pixel origin (X0, Y0) may contain a pixel whose
// q is <= thr.  (gx, gy) splat centre in pixels, (a, b, c) conic.
__device__ __forceinline__ u32 strip_mask8(const float gx, const float gy, const float a, const float b, const float c,
                                           const float thr, const float X0, const float Y0, const int first = 0,
                                           const int count = 8) {
    // Anything that is not a proper ellipse with a finite threshold is left to the per-pixel test.
    if (!(a > 0.f && c > 0.f && a * c > b * b) || !(thr == thr)) return 0xffu;
    const float dxl = X0 + 0.5f - gx, dxh = dxl + 15.0f;
    const float ex = fminf(fmaxf(0.f, dxl), dxh);
    const bool in_x = ex == 0.f;
    const float kc = -b / c, ka = -b / a;
    const float q_ex = 0.5f * a * ex * ex;
    u32 mask = 0;
#pragma unroll
    for (int w = first; w < first + count; ++w) {
        const float dyl = Y0 + (float)(2 * w) + 0.5f - gy, dyh = dyl + 1.0f;
        const float ey = fminf(fmaxf(0.f, dyl), dyh);
        const bool in_y = ey == 0.f;
        float minq = 0.f;
        if (!(in_x && in_y)) {
            float q1 = 3.0e38f, q2 = 3.0e38f;
            if (!in_x) {  // edge dx = ex, best dy on it
                const float dy = fminf(fmaxf(kc * ex, dyl), dyh);
                q1 = q_ex + 0.5f * c * dy * dy + b * ex * dy;
            }
            if (!in_y) {  // edge dy = ey, best dx on it
                const float dx = fminf(fmaxf(ka * ey, dxl), dxh);
                q2 = 0.5f * (a * dx * dx + c * ey * ey) + b * dx * ey;
            }
            minq = fminf(q1, q2);
        }
        if (!(minq > thr)) mask |= 1u << w;
    }
    return mask;
}

}  // namespace dsb
