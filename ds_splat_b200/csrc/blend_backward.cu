// Stage (f1): reverse-order blend, per-splat gradient accumulation.
//
// Takes the place of the reference's rasterize_backward_kernel (cpp/gsplat/backward.cu:25-202).  The
// reference runs one 256-thread block per 16x16 tile that marches through the tile's list in lock step
// (two block barriers per 256 entries), evaluates every entry for every pixel, reduces 9 values with 9
// full warp reductions (45 shuffles) and issues 9 scalar atomics per warp per entry.
//
// Here each WARP is on its own.  A warp owns a compact block of kPix * 32 pixels of a tile (8 x 16 by default)
// and every lane works on kPix pixels of one column (rows y, y + 4, ...).  The warp walks the tile's list back
// to front in chunks of 32 entries, with no block barrier anywhere, so a warp whose pixels ended early is
// finished early and nobody waits for the slowest warp; thread blocks are small (two warps) so that a
// finished warp's registers go back to the scheduler at once.
//   * fetch + cull: lane l fetches entry l of the chunk (48-byte record) and tests in closed form whether
//     the splat can reach the warp's pixels at all; a ballot gives the survivors;
//   * blend: survivors are parked in the warp's private shared-memory slice and processed one by one.
//     exp is only evaluated for pixels with q <= ln(255 opacity) + margin, after which the reference's own
//     test (clamped alpha < 1/255) decides.  Per pixel the nine sums are moments that need few multiplies,
//         S0 = sum v_s, Sx = sum v_s dx, Sy = sum v_s dy, Sxx, Sxy, Syy, and the three colour sums;
//     a lane adds the moments of its kPix pixels in registers, then the warp reduces them with a transposing
//     butterfly (8 values in 4+2+1+1+1 shuffles, the ninth in 5) into the entry's row of the warp's
//     accumulator slice -- so the reduction, the record reads and the loop control are paid once per
//     kPix * 32 pixels, and the kPix independent transmittance chains of a lane hide each other's latency;
//   * flush: lane l, which still holds entry l's record in registers, turns its row of moments into
//         v_xy = (a Sx + b Sy, b Sx + c Sy), v_conic = (Sxx/2, Sxy, Syy/2), v_opacity = -S0 / opacity
//     and issues two red.global.add.v4.f32 and one scalar red: 3 vector atomics per (warp, splat) that
//     received anything, instead of 9 scalar ones.
//
// The per-pixel arithmetic follows the reference: alpha clamp 0.99, 1/255 skip, opacity and visibility
// gradients without clamp masking, and the background term in v_alpha.  One regrouping: the reference keeps the
// colour blended behind the current entry per channel (b_c) and forms
//     v_alpha = sum_c (colour_c T - b_c / (1 - alpha)) v_out_c - T_final (bg . v_out) / (1 - alpha);
// only the dot products with the pixel's upstream gradient are ever used, so a lane carries the scalar
//     B = sum_c b_c v_out_c + T_final (bg . v_out),   v_alpha = T P - B / (1 - alpha),   B += alpha T P,
// with P = colour . v_out of the entry: one running value per pixel instead of three (a fourth with the depth
// channel) and 6 instead of 13 instructions per blended pixel.
//
// Optional depth gradient (the reference has no depth map): in the DEPTH instantiation the splat's view-space
// z acts as a fourth colour channel without background.  Its upstream gradient joins v_alpha, and a tenth
// sum, v_z = sum alpha T v_depth, lands in slot 9 of the splat's accumulator row, from where the per-splat
// backward feeds it to the mean exactly where the reference's projection backward takes its v_depth
// (cpp/gsplat/backward.cu:253-259).
#include "blend_common.cuh"

namespace dsb {

namespace {


__device__ __forceinline__ void red_add_v4(float4* addr, const float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}

__device__ __forceinline__ void red_add_v2(float* addr, const float a, const float b) {
    asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(a), "f"(b) : "memory");
}

__device__ __forceinline__ void red_add(float* addr, const float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// Sum of v[j] over the warp lands in lane 4*j (j = 0..7); 9 shuffles.
__device__ __forceinline__ float butterfly8(const float (&v)[8], const int lane) {
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
    float a0 = h16 ? v[4] : v[0], a1 = h16 ? v[5] : v[1], a2 = h16 ? v[6] : v[2], a3 = h16 ? v[7] : v[3];
    const float s0 = h16 ? v[0] : v[4], s1 = h16 ? v[1] : v[5], s2 = h16 ? v[2] : v[6], s3 = h16 ? v[3] : v[7];
    a0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    a1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    a2 += __shfl_xor_sync(0xffffffffu, s2, 16);
    a3 += __shfl_xor_sync(0xffffffffu, s3, 16);
    float b0 = h8 ? a2 : a0, b1 = h8 ? a3 : a1;
    const float t0 = h8 ? a0 : a2, t1 = h8 ? a1 : a3;
    b0 += __shfl_xor_sync(0xffffffffu, t0, 8);
    b1 += __shfl_xor_sync(0xffffffffu, t1, 8);
    float c = h4 ? b1 : b0;
    const float u = h4 ? b0 : b1;
    c += __shfl_xor_sync(0xffffffffu, u, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}

__device__ __forceinline__ float butterfly1(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- mapping of pixels to warps and lanes ------------------------------------------------------------------
// Measured on B200 (1M splats at 1080p / 3M at 4K / 2M wide splats, ms): one pixel per lane in 256-thread
// blocks 0.71 / 3.93 / 0.97; 2 pixels, 8x8 block, 64 threads 0.57 / 2.95 / 0.80; 4 pixels, 8x16 block,
// 64 threads 0.55 / 2.74 / 0.85 (the default); 16-wide blocks and 32- or 256-thread blocks are slower.
#ifndef DSB_BWD_PIX
#define DSB_BWD_PIX 4   // pixels per lane: 1, 2, 4 or 8
#endif
#ifndef DSB_BWD_BLOCK_W
#define DSB_BWD_BLOCK_W 8    // width of a warp's pixel block: 16 or 8
#endif
constexpr int kPix = DSB_BWD_PIX;
constexpr int kBlockW = DSB_BWD_BLOCK_W;
constexpr int kRowsPerPass = 32 / kBlockW;               // rows the 32 lanes cover at once
constexpr int kBlockH = kRowsPerPass * kPix;             // pixel block of one warp is kBlockW x kBlockH
constexpr int kBlocksPerTileX = kTile / kBlockW, kBlocksPerTileY = kTile / kBlockH;
constexpr int kBlocksPerTile = kBlocksPerTileX * kBlocksPerTileY;
static_assert(kBlockH <= kTile && kTile % kBlockH == 0, "a warp's pixel block must tile the 16x16 tile");
// Warps never synchronise with each other, and their lists differ in length; small thread blocks give the
// slots of a finished warp back to the scheduler instead of holding them until the block's slowest warp ends.
#ifndef DSB_BWD_THREADS
#define DSB_BWD_THREADS 64
#endif
#ifndef DSB_BWD_MIN_BLOCKS
#define DSB_BWD_MIN_BLOCKS 14  // 72 registers, nothing spilled; measured 12 / 14 / 16 blocks: 0.434 / 0.418 / 0.436 ms (16 spills)
#endif
constexpr int kThreads = DSB_BWD_THREADS, kWarps = kThreads / 32;

template <bool DEPTH>
__global__ void __launch_bounds__(kThreads, DSB_BWD_MIN_BLOCKS)
blend_backward_kernel(const int W, const int H, const int tiles_x, const int num_tiles, const float* __restrict__ bg,
                            const float4* __restrict__ records, const u64* __restrict__ sorted,
                            const int32_t* __restrict__ ranges, const float* __restrict__ final_T,
                            const int32_t* __restrict__ final_idx, const float* __restrict__ v_image,
                            const float* __restrict__ v_depth, float4* __restrict__ grad_acc,
                            const int32_t* __restrict__ tile_order) {
    __shared__ float4 s_rec[kWarps][32][3];   // x,y,a,b | c,opacity,r,g | blue, threshold, z, -
    __shared__ float s_acc[kWarps][32][12];   // moments of the chunk's entries

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wb = blockIdx.x * kWarps + warp;             // warp-level pixel block
    const int slot = wb / kBlocksPerTile;
    if (slot >= num_tiles) return;                         // whole warps only; no block-wide barrier below
    const int sub = wb - slot * kBlocksPerTile;
    const int tile = tile_order ? tile_order[slot] : slot; // longest lists first when the order is known
    if ((unsigned)tile >= (unsigned)num_tiles) return;     // a caller's stale order must not index outside the ranges
    const int tile_x = tile % tiles_x, tile_y = tile / tiles_x;
    const int bx = tile_x * kTile + (sub % kBlocksPerTileX) * kBlockW, by = tile_y * kTile + (sub / kBlocksPerTileX) * kBlockH;
    const int x = bx + (lane % kBlockW), y0 = by + (lane / kBlockW);
    const float px = (float)x + 0.5f, py0 = (float)y0 + 0.5f;
    const int start = ranges[tile], end = ranges[tile + 1];

    float T[kPix], B[kPix], vo0[kPix], vo1[kPix], vo2[kPix], vod[kPix];
    int fin[kPix];
    int fin_max = -1;
#pragma unroll
    for (int p = 0; p < kPix; ++p) {
        const int y = y0 + kRowsPerPass * p;
        T[p] = 1.0f; B[p] = 0.0f;
        vo0[p] = vo1[p] = vo2[p] = vod[p] = 0.0f;
        fin[p] = -1;                                       // outside the image: never valid
        if (x < W && y < H) {
            const size_t pix = (size_t)y * W + x;
            T[p] = final_T[pix];
            fin[p] = final_idx[pix];
            vo0[p] = v_image[3 * pix]; vo1[p] = v_image[3 * pix + 1]; vo2[p] = v_image[3 * pix + 2];
            if (DEPTH) vod[p] = v_depth[pix];
            const float bgdot = bg ? (bg[0] * vo0[p] + bg[1] * vo1[p] + bg[2] * vo2[p]) : 0.0f;
            B[p] = T[p] * bgdot;
        }
        fin_max = max(fin_max, fin[p]);
    }
    // Entries after the last one any pixel of the warp blended cannot contribute.
    const int top = min(end - 1, __reduce_max_sync(0xffffffffu, fin_max));

    float4 (*rec)[3] = s_rec[warp];
    float (*acc)[12] = s_acc[warp];

    for (int base = top; base >= start; base -= 32) {
        // ---- fetch + cull: lane l takes the entry at list position base - l
        const int my_pos = base - lane;
        u32 id = 0;
        float4 q0 = make_float4(0, 0, 0, 0), q1 = q0;
        float blue = 0.f, thr = 0.f, zview = 0.f;
        bool hit = false;
        if (my_pos >= start) {
            id = (u32)sorted[my_pos];
            const float4* r = records + (size_t)id * 3;
            q0 = __ldg(r); q1 = __ldg(r + 1);
            const float4 q2 = __ldg(r + 2);
            blue = q2.x; zview = q2.y;
            thr = __logf(255.0f * q1.y) + kCullMargin;
            hit = splat_reaches_rect<kBlockW, kBlockH>(q0.x, q0.y, q0.z, q0.w, q1.x, thr, (float)bx, (float)by);
        }
        u32 todo = __ballot_sync(0xffffffffu, hit);
        if (todo == 0) continue;
        rec[lane][0] = q0; rec[lane][1] = q1; rec[lane][2] = make_float4(blue, thr, zview, 0.f);
        __syncwarp();

        // ---- blend the survivors, nearest list position last (ascending lane = descending position)
        u32 touched = 0;
        while (todo) {
            const int t = __ffs(todo) - 1;
            todo &= todo - 1;
            const int pos = base - t;
            const float4 qa = rec[t][0];
            const float4 qb = rec[t][1];
            const float4 qc = rec[t][2];
            const float dx = qa.x - px;
            float dy[kPix], sigma[kPix];
            bool valid[kPix], any = false;
#pragma unroll
            for (int p = 0; p < kPix; ++p) {
                dy[p] = qa.y - (py0 + (float)(kRowsPerPass * p));
                sigma[p] = 0.5f * (qa.z * dx * dx + qb.x * dy[p] * dy[p]) + qa.w * dx * dy[p];
                valid[p] = pos <= fin[p] && sigma[p] >= 0.f && sigma[p] <= qc.y;
                any = any || valid[p];
            }
            if (!__any_sync(0xffffffffu, any)) continue;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, cr = 0.f, cg = 0.f, cb = 0.f, cz = 0.f;
#pragma unroll
            for (int p = 0; p < kPix; ++p) {
                if (valid[p]) {
                    const float vis = __expf(-sigma[p]);
                    const float alpha = min(0.99f, qb.y * vis);
                    if (!(alpha < 1.f / 255.f)) {
                        const float ra = 1.f / (1.f - alpha);
                        T[p] *= ra;
                        const float fac = alpha * T[p];
                        float P = qb.z * vo0[p] + qb.w * vo1[p] + qc.x * vo2[p];
                        if (DEPTH) {
                            P += qc.z * vod[p];
                            cz += fac * vod[p];
                        }
                        const float v_alpha = T[p] * P - ra * B[p];
                        B[p] += fac * P;
                        const float v_sigma = -qb.y * vis * v_alpha;
                        s0 += v_sigma;
                        s1 += v_sigma * dy[p];
                        s2 += v_sigma * dy[p] * dy[p];
                        cr += fac * vo0[p]; cg += fac * vo1[p]; cb += fac * vo2[p];
                    }
                }
            }
            const float sx = s0 * dx;
            const float v[8] = {sx, s1, sx * dx, s1 * dx, s2, s0, cr, cg};   // Sx, Sy, Sxx, Sxy, Syy, S0, r, g
            const float sum = butterfly8(v, lane);
            const float sum8 = butterfly1(cb);
            if ((lane & 3) == 0) acc[t][lane >> 2] = sum;
            if (lane == 0) acc[t][8] = sum8;
            if (DEPTH) {
                const float sum9 = butterfly1(cz);
                if (lane == 0) acc[t][9] = sum9;
            }
            touched |= 1u << t;
        }
        __syncwarp();

        // ---- flush: lane l owns entry l of the chunk and still has its record in registers
        if ((touched >> lane) & 1u) {
            const float4 m0 = *reinterpret_cast<const float4*>(&acc[lane][0]);  // Sx, Sy, Sxx, Sxy
            const float4 m1 = *reinterpret_cast<const float4*>(&acc[lane][4]);  // Syy, S0, r, g
            const float m2 = acc[lane][8];                                      // b
            float4* dst = grad_acc + (size_t)id * 3;
            red_add_v4(dst, make_float4(q0.z * m0.x + q0.w * m0.y, q0.w * m0.x + q1.x * m0.y, 0.5f * m0.z, m0.w));
            red_add_v4(dst + 1, make_float4(0.5f * m1.x, -m1.y / q1.y, m1.z, m1.w));
            if (DEPTH) red_add_v2(reinterpret_cast<float*>(dst + 2), m2, acc[lane][9]);
            else red_add(reinterpret_cast<float*>(dst + 2), m2);
        }
        __syncwarp();  // the slices are reused by the next chunk
    }
}

}  // namespace

// v_depth may be null (no depth map was rendered, or nothing depends on it); tile_order may be null.
int launch_blend_backward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                          const float* final_T, const int32_t* final_idx, const float* v_image, const float* v_depth,
                          float* grad_acc, const int32_t* tile_order, cudaStream_t s) {
    DSB_REQUIRE(ranges && final_T && final_idx && v_image && grad_acc, "blend_backward: null pointer");
    DSB_REQUIRE(((uintptr_t)grad_acc & 15) == 0, "blend_backward: grad_acc must be 16-byte aligned");
    const int num_tiles = cp.tiles_x * cp.tiles_y;
    const int blocks = (num_tiles * kBlocksPerTile + kWarps - 1) / kWarps;
    if (v_depth)
        blend_backward_kernel<true><<<blocks, kThreads, 0, s>>>(cp.W, cp.H, cp.tiles_x, num_tiles, cp.bg,
                                                                     reinterpret_cast<const float4*>(records), sorted, ranges,
                                                                     final_T, final_idx, v_image, v_depth,
                                                                     reinterpret_cast<float4*>(grad_acc), tile_order);
    else
        blend_backward_kernel<false><<<blocks, kThreads, 0, s>>>(cp.W, cp.H, cp.tiles_x, num_tiles, cp.bg,
                                                                      reinterpret_cast<const float4*>(records), sorted, ranges,
                                                                      final_T, final_idx, v_image, nullptr,
                                                                      reinterpret_cast<float4*>(grad_acc), tile_order);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace dsb
