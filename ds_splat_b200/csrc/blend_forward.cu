// Stage (e): per-tile front-to-back alpha blending.
//
// Takes the place of the reference's render_image_kernel (cpp/rasterizer_kernels.cu:341-431).  One
// 256-thread block per 16x16 tile, one pixel per thread.  The tile's depth-ordered splats are consumed
// in rounds of 256: while a round is being blended out of shared memory, the next round's records are
// already in flight into registers, so the gather latency hides behind the arithmetic.  A pixel stops
// at the first splat that would push its transmittance under 1e-4; a warp whose 32 pixels have all
// stopped leaves the inner loop, and the tile stops fetching rounds once all 256 pixels have stopped.
//
// Per-pixel arithmetic (order of operations, 0.999 alpha clamp, 1/255 skip, no background term) is the
// reference's, so images agree to rounding and final_idx agrees exactly.
#include "common.cuh"

namespace dsb {

namespace {

constexpr int kThreads = kTilePixels;

__global__ void __launch_bounds__(kThreads)
blend_forward_kernel(const int W, const int H, const float4* __restrict__ records, const u64* __restrict__ sorted,
                     const int32_t* __restrict__ ranges, float* __restrict__ image, float* __restrict__ final_T,
                     int32_t* __restrict__ final_idx) {
    __shared__ float4 s_q0[kThreads];  // x, y, conic a, conic b
    __shared__ float4 s_q1[kThreads];  // conic c, opacity, r, g
    __shared__ float s_b[kThreads];    // b

    const int tid = threadIdx.x;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int x = blockIdx.x * kTile + (tid & (kTile - 1));
    const int y = blockIdx.y * kTile + (tid >> 4);
    const bool inside = x < W && y < H;
    const int start = ranges[tile], end = ranges[tile + 1];
    const float pxf = x + 0.5f, pyf = y + 0.5f;

    float T = 1.0f, c0 = 0.0f, c1 = 0.0f, c2 = 0.0f;
    int last = 0;
    bool done = !inside;

    float4 n0 = make_float4(0, 0, 0, 0), n1 = n0;
    float nb = 0.0f;
    if (start + tid < end) {
        const u32 id = (u32)sorted[start + tid];
        const float4* r = records + (size_t)id * 3;
        n0 = __ldg(r); n1 = __ldg(r + 1); nb = __ldg(r + 2).x;
    }
    const int rounds = (end - start + kThreads - 1) / kThreads;
    for (int s = 0; s < rounds; ++s) {
        // Also the barrier that lets the previous round's shared memory be overwritten.
        if (__syncthreads_count(done) == kThreads) break;
        s_q0[tid] = n0; s_q1[tid] = n1; s_b[tid] = nb;
        __syncthreads();
        const int round_base = start + s * kThreads;
        const int next = round_base + kThreads + tid;
        if (next < end) {
            const u32 id = (u32)sorted[next];
            const float4* r = records + (size_t)id * 3;
            n0 = __ldg(r); n1 = __ldg(r + 1); nb = __ldg(r + 2).x;
        }
        const int cnt = min(kThreads, end - round_base);
        for (int i = 0; i < cnt && !done; ++i) {
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
            last = round_base + i;
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
