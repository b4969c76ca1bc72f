// Stage (f1): reverse-order blend, per-splat gradient accumulation.
//
// Takes the place of the reference's rasterize_backward_kernel (cpp/gsplat/backward.cu:25-202).  One
// 256-thread block per 16x16 tile walks the tile's list back to front in rounds of 64 splats; each pixel
// recovers its transmittance by dividing by (1 - alpha) and produces nine partial derivatives per splat
// (pixel mean 2, conic 3, opacity 1, colour 3).
//
// The reduction over pixels is where the reference spends its time (9 full warp reductions and 9
// scalar atomics per warp per splat).  Here:
//   * a warp reduces the 9 values with a transposing butterfly -- at each step half of the values move
//     to the partner lane, so 8 values cost 4+2+1+1+1 shuffles instead of 40 -- and the ninth with a
//     plain butterfly: 14 shuffles in all;
//   * each warp parks its sums in its own shared-memory slot (plain stores, no shared atomics);
//   * after the round the block adds the 8 warps' slots and issues ONE vector reduction per splat and
//     row quarter to global memory (red.global.add.v4.f32), i.e. 3 global atomics per (tile, splat)
//     instead of 72.
//
// The per-pixel arithmetic follows the reference: alpha clamp 0.99, 1/255 skip, opacity and visibility
// gradients without clamp masking, and the background term in v_alpha.
#include "common.cuh"

namespace dsb {

namespace {

constexpr int kThreads = kTilePixels;
constexpr int kWarps = kThreads / 32;
constexpr int kRound = 64;  // splats per round

__device__ __forceinline__ void red_add_v4(float4* addr, const float4 v) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
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

__global__ void __launch_bounds__(kThreads)
blend_backward_kernel(const int W, const int H, const float* __restrict__ bg, const float4* __restrict__ records,
                      const u64* __restrict__ sorted, const int32_t* __restrict__ ranges,
                      const float* __restrict__ final_T, const int32_t* __restrict__ final_idx,
                      const float* __restrict__ v_image, float4* __restrict__ grad_acc) {
    __shared__ float4 s_rec[kRound][3];
    __shared__ u32 s_id[kRound];
    __shared__ float s_acc[kWarps][kRound][12];
    __shared__ u64 s_touched[kWarps];
    __shared__ int s_wmax[kWarps];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int x = blockIdx.x * kTile + (tid & (kTile - 1));
    const int y = blockIdx.y * kTile + (tid >> 4);
    const bool inside = x < W && y < H;
    const float px = (float)x + 0.5f, py = (float)y + 0.5f;
    const int start = ranges[tile], end = ranges[tile + 1];

    float Tf = 1.0f, vo0 = 0.0f, vo1 = 0.0f, vo2 = 0.0f;
    int fin = -1;
    if (inside) {
        const size_t pix = (size_t)y * W + x;
        Tf = final_T[pix];
        fin = final_idx[pix];
        vo0 = v_image[3 * pix]; vo1 = v_image[3 * pix + 1]; vo2 = v_image[3 * pix + 2];
    }
    const float bgdot = bg ? (bg[0] * vo0 + bg[1] * vo1 + bg[2] * vo2) : 0.0f;
    const int warp_max = __reduce_max_sync(0xffffffffu, fin);
    if (lane == 0) s_wmax[warp] = warp_max;
    __syncthreads();
    int block_max = s_wmax[0];
#pragma unroll
    for (int w = 1; w < kWarps; ++w) block_max = max(block_max, s_wmax[w]);
    const int top = min(end - 1, block_max);
    if (top < start) return;  // uniform: nothing in this tile reached any pixel
    const int rounds = (top - start + kRound) / kRound;

    float T = Tf, b0 = 0.0f, b1 = 0.0f, b2 = 0.0f;

    // Staging: 4 threads per splat, three of them carry one float4 of its record.
    const int g = tid >> 2, part = tid & 3;
    float4 nv = make_float4(0, 0, 0, 0);
    u32 nid = 0;
    {
        const int pos = top - g;
        if (pos >= start && part < 3) {
            nid = (u32)sorted[pos];
            nv = __ldg(records + (size_t)nid * 3 + part);
        }
    }
    for (int r = 0; r < rounds; ++r) {
        __syncthreads();  // the previous round's flush has finished with the shared arrays
        if (part < 3) s_rec[g][part] = nv;
        if (part == 0) s_id[g] = nid;
        __syncthreads();
        const int round_top = top - r * kRound;
        {
            const int pos = round_top - kRound - g;
            if (pos >= start && part < 3) {
                nid = (u32)sorted[pos];
                nv = __ldg(records + (size_t)nid * 3 + part);
            }
        }
        const int cnt = min(kRound, round_top - start + 1);
        u64 touched = 0;
        for (int t = max(0, round_top - warp_max); t < cnt; ++t) {
            const int pos = round_top - t;
            bool valid = inside && pos <= fin;
            const float4 qa = s_rec[t][0];  // x, y, conic a, conic b
            const float4 qb = s_rec[t][1];  // conic c, opacity, r, g
            const float dx = qa.x - px, dy = qa.y - py;
            const float sigma = 0.5f * (qa.z * dx * dx + qb.x * dy * dy) + qa.w * dx * dy;
            const float vis = __expf(-sigma);
            const float alpha = min(0.99f, qb.y * vis);
            valid = valid && !(sigma < 0.f || alpha < 1.f / 255.f);
            if (!__any_sync(0xffffffffu, valid)) continue;
            float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float v8 = 0.f;
            if (valid) {
                const float blue = s_rec[t][2].x;
                const float ra = 1.f / (1.f - alpha);
                T *= ra;
                const float fac = alpha * T;
                float v_alpha = 0.f;
                v_alpha += (qb.z * T - b0 * ra) * vo0;
                v_alpha += (qb.w * T - b1 * ra) * vo1;
                v_alpha += (blue * T - b2 * ra) * vo2;
                v_alpha += -Tf * ra * bgdot;
                b0 += qb.z * fac; b1 += qb.w * fac; b2 += blue * fac;
                const float v_sigma = -qb.y * vis * v_alpha;
                v[0] = v_sigma * (qa.z * dx + qa.w * dy);
                v[1] = v_sigma * (qa.w * dx + qb.x * dy);
                v[2] = 0.5f * v_sigma * dx * dx;
                v[3] = v_sigma * dx * dy;
                v[4] = 0.5f * v_sigma * dy * dy;
                v[5] = vis * v_alpha;
                v[6] = fac * vo0;
                v[7] = fac * vo1;
                v8 = fac * vo2;
            }
            const float sum = butterfly8(v, lane);
            const float sum8 = butterfly1(v8);
            if ((lane & 3) == 0) s_acc[warp][t][lane >> 2] = sum;
            if (lane == 0) s_acc[warp][t][8] = sum8;
            touched |= 1ull << t;
        }
        if (lane == 0) s_touched[warp] = touched;
        __syncthreads();
        // Flush: thread (g, part) adds the warps' slots of float4 `part` of splat g and issues one reduction.
        if (g < cnt && part < 3) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            bool any = false;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                if ((s_touched[w] >> g) & 1ull) {
                    const float4 p = *reinterpret_cast<const float4*>(&s_acc[w][g][4 * part]);
                    acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                    any = true;
                }
            }
            if (any) {
                float4* dst = grad_acc + (size_t)s_id[g] * 3 + part;
                if (part < 2) red_add_v4(dst, acc);
                else red_add(reinterpret_cast<float*>(dst), acc.x);
            }
        }
    }
}

}  // namespace

int launch_blend_backward(const CamParams& cp, const float* records, const u64* sorted, const int32_t* ranges,
                          const float* final_T, const int32_t* final_idx, const float* v_image, float* grad_acc,
                          cudaStream_t s) {
    DSB_REQUIRE(ranges && final_T && final_idx && v_image && grad_acc, "blend_backward: null pointer");
    DSB_REQUIRE(((uintptr_t)grad_acc & 15) == 0, "blend_backward: grad_acc must be 16-byte aligned");
    const dim3 grid(cp.tiles_x, cp.tiles_y);
    blend_backward_kernel<<<grid, kThreads, 0, s>>>(cp.W, cp.H, cp.bg, reinterpret_cast<const float4*>(records), sorted,
                                                   ranges, final_T, final_idx, v_image,
                                                   reinterpret_cast<float4*>(grad_acc));
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace dsb
