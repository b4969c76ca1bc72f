// Stage (e): per-tile front-to-back alpha blending.
//
// Takes the place of the reference's render_image_kernel (cpp/rasterizer_kernels.cu:341-431).  One
// 256-thread block per 16x16 tile, one pixel per thread, warp w = rows 2w, 2w+1 of the tile.  The tile's
// depth-ordered list is consumed in rounds of 256 entries:
//   * staging: thread i fetches entry i's 48-byte record (the next round's records are already in flight
//     in registers while the current round is blended), works out which of the 8 warp strips the splat can
//     reach at all (blend_common.cuh) and the round's survivors are compacted into shared memory in list
//     order -- splats that cannot reach any pixel of the tile cost nothing further;
//   * blending: every warp walks the compacted round; one shared-memory word tells it whether the splat
//     can reach its strip, and only then are the record and the per-pixel arithmetic touched.
// A pixel stops at the first splat that would push its transmittance under 1e-4; a warp whose 32 pixels
// have all stopped leaves the inner loop; the tile stops fetching rounds once all 256 pixels have stopped.
//
// Per-pixel arithmetic (order of operations, 0.999 alpha clamp, 1/255 skip, no background term) is the
// reference's and the strip test is conservative, so images agree to rounding and final_idx exactly.
#include "blend_common.cuh"

namespace dsb {

namespace {

constexpr int kThreads = kTilePixels;
constexpr int kWarps = kThreads / 32;

__global__ void __launch_bounds__(kThreads)
blend_forward_kernel(const int W, const int H, const float4* __restrict__ records, const u64* __restrict__ sorted,
                     const int32_t* __restrict__ ranges, float* __restrict__ image, float* __restrict__ final_T,
                     int32_t* __restrict__ final_idx) {
    __shared__ float4 s_q0[kThreads];  // x, y, conic a, conic b
    __shared__ float4 s_q1[kThreads];  // conic c, opacity, r, g
    __shared__ float s_b[kThreads];    // b
    __shared__ u32 s_mp[kThreads];     // (position inside the round << 8) | strip mask
    __shared__ int s_wcount[kWarps];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int x = blockIdx.x * kTile + (tid & (kTile - 1));
    const int y = blockIdx.y * kTile + (tid >> 4);
    const bool inside = x < W && y < H;
    const int start = ranges[tile], end = ranges[tile + 1];
    const float pxf = x + 0.5f, pyf = y + 0.5f;
    const float X0 = (float)(blockIdx.x * kTile), Y0 = (float)(blockIdx.y * kTile);

    float T = 1.0f, c0 = 0.0f, c1 = 0.0f, c2 = 0.0f;
    int last = 0;
    bool done = !inside;

    float4 n0 = make_float4(0, 0, 0, 0), n1 = n0;
    float nb = 0.0f;
    bool have = start + tid < end;
    if (have) {
        const u32 id = (u32)sorted[start + tid];
        const float4* r = records + (size_t)id * 3;
        n0 = __ldg(r); n1 = __ldg(r + 1); nb = __ldg(r + 2).x;
    }
    const int rounds = (end - start + kThreads - 1) / kThreads;
    for (int s = 0; s < rounds; ++s) {
        // Also the barrier that lets the previous round's shared memory be overwritten.
        if (__syncthreads_count(done) == kThreads) break;
        u32 mask = 0;
        if (have) mask = strip_mask8(n0.x, n0.y, n0.z, n0.w, n1.x, __logf(255.0f * n1.y) + kStripMargin, X0, Y0);
        const u32 keep = __ballot_sync(0xffffffffu, mask != 0);
        if (lane == 0) s_wcount[warp] = __popc(keep);
        __syncthreads();
        int slot = __popc(keep & ((1u << lane) - 1u)), total = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const int cw = s_wcount[w];
            slot += (w < warp) ? cw : 0;
            total += cw;
        }
        if (mask) {
            s_q0[slot] = n0; s_q1[slot] = n1; s_b[slot] = nb;
            s_mp[slot] = ((u32)tid << 8) | mask;
        }
        __syncthreads();
        const int round_base = start + s * kThreads;
        const int next = round_base + kThreads + tid;
        have = next < end;
        if (have) {
            const u32 id = (u32)sorted[next];
            const float4* r = records + (size_t)id * 3;
            n0 = __ldg(r); n1 = __ldg(r + 1); nb = __ldg(r + 2).x;
        }
        for (int i = 0; i < total && !done; ++i) {
            const u32 mp = s_mp[i];
            if (!((mp >> warp) & 1u)) continue;  // this splat cannot reach the warp's strip
            const float4 a = s_q0[i];
            const float4 b = s_q1[i];
            const float dx = pxf - a.x, dy = pyf - a.y;
            const float power = -0.5f * (a.z * dx * dx + b.x * dy * dy) - a.w * dx * dy;
            const float alpha = min(0.999f, b.y * __expf(power));
            if (power >= 0.f || alpha < 1.0f / 255.0f) continue;
            const float Tn = (1.0f - alpha) * T;
            if (!(Tn >= 0.0001f)) { done = true; break; }
            const float wgt = alpha * T;
            c0 += wgt * b.z; c1 += wgt * b.w; c2 += wgt * s_b[i];
            T = Tn;
            last = round_base + (int)(mp >> 8);
        }
    }
    if (inside) {
        const size_t pix = (size_t)y * W + x;
        image[3 * pix] = c0; image[3 * pix + 1] = c1; image[3 * pix + 2] = c2;
        final_T[pix] = T;
        final_idx[pix] = last;
    }
}

}  // namespace

int launch_blend_forward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                         float* image, float* final_T, int32_t* final_idx, cudaStream_t s) {
    DSB_REQUIRE(ranges && image && final_T && final_idx, "blend_forward: null pointer");
    const dim3 grid(cp.tiles_x, cp.tiles_y);
    blend_forward_kernel<<<grid, kThreads, 0, s>>>(cp.W, cp.H, reinterpret_cast<const float4*>(records), sorted, ranges,
                                                  image, final_T, final_idx);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace dsb
