// The step before the operator's backward in a training loop: the photometric loss of 3-D Gaussian Splatting
// training and its gradient with respect to the rendered image, in two launches.
//
//     L = (1 - lambda) * mean |x - y|  +  lambda * (1 - mean SSIM(x, y))
//
// x the rendered image, y the target, both [H][W][3]; SSIM per channel with an 11x11 Gaussian window (sigma 1.5),
// zero padding, C1 = 0.01^2, C2 = 0.03^2 (Wang et al., "Image quality assessment: from error visibility to
// structural similarity", 2004, in the form 3DGS training code uses).  Not part of the reference, whose users
// build this loss from ~20 torch operations and let autograd differentiate them.
//
// With w the window, m1 = w*x, m2 = w*y, e11 = w*x^2, e22 = w*y^2, e12 = w*(xy) (* = zero-padded correlation):
//     s11 = e11 - m1^2, s22 = e22 - m2^2, s12 = e12 - m1 m2
//     A1 = 2 m1 m2 + C1, A2 = 2 s12 + C2, B1 = m1^2 + m2^2 + C1, B2 = s11 + s22 + C2, S = A1 A2 / (B1 B2)
// S depends on x through m1, e11 and e12; the window is symmetric, so
//     dL/dx = w*(g dS/dm1) + 2 x . w*(g dS/de11) + y . w*(g dS/de12) + (1 - lambda)/(3HW) sign(x - y),  g = -lambda/(3HW)
//     dS/dm1  = [2 m2 (A2 - A1) B1 B2 - A1 A2 2 m1 (B2 - B1)] / (B1 B2)^2
//     dS/de11 = -A1 A2 / (B1 B2^2)          dS/de12 = 2 A1 / (B1 B2)
// Kernel 1 computes the five windowed moments per pixel (separable, through shared memory), the loss sums and the
// three maps g dS/d.; kernel 2 correlates the maps with the window again and assembles dL/dx.
#include <cmath>

#include "common.cuh"

namespace dsb {

namespace {

constexpr int kWin = 11, kHalf = 5;
// A block of 256 threads produces a 32 x 32 pixel tile of one channel at a time.  Both passes of the separable window
// slide over registers: a thread of the horizontal pass turns 14 neighbouring values of a row into 4 neighbouring
// outputs, a thread of the vertical pass 14 values of a column into 4 outputs, so a value is read from shared memory
// 1.2 times per tap instead of once per tap and output.  Row strides are odd, which keeps the row-major work items of
// the horizontal pass (consecutive lanes = consecutive rows) and the column-major threads of the vertical pass free of
// bank conflicts.
constexpr int kPatch = 32, kLossThreads = 256, kOut = 4;
constexpr int kPad = kPatch + 2 * kHalf;          // 42 rows / columns with the halo
constexpr int kInStride = kPad + 1;              // 43
constexpr int kHStride = kPatch + 1;              // 33
constexpr int kGroups = kPatch / kOut;            // 8 four-column groups per row
constexpr int kSpan = kOut + kWin - 1;           // 14 inputs for 4 outputs
static_assert(kLossThreads == kPatch * (kPatch / kOut), "the vertical pass gives every thread one column and four rows");

struct Window { float w[kWin]; };

// acc[j] += w[k - j] * v for the outputs j that input k of the span reaches (k is a compile-time constant after unrolling)
__device__ __forceinline__ void slide(float (&acc)[kOut], const float v, const int k, const Window& win) {
#pragma unroll
    for (int j = 0; j < kOut; ++j) {
        const int t = k - j;
        if (t >= 0 && t < kWin) acc[j] = fmaf(win.w[t], v, acc[j]);
    }
}

__device__ __forceinline__ float block_sum(float v, float* s_red) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int tid = threadIdx.x;
    if ((tid & 31) == 0) s_red[tid >> 5] = v;
    __syncthreads();
    float total = 0.f;
    if (tid == 0)
        for (int k = 0; k < kLossThreads / 32; ++k) total += s_red[k];
    __syncthreads();
    return total;   // valid in thread 0
}

// maps: [3][H][W][3] (g dS/dm1, g dS/de11, g dS/de12); sums: [0] += sum |x - y|, [1] += sum SSIM
__global__ void __launch_bounds__(kLossThreads)
ssim_moments_kernel(const float* __restrict__ x, const float* __restrict__ y, const int H, const int W, const Window win,
                    const float g, float* __restrict__ maps, float* __restrict__ sums) {
    __shared__ float s_x[kPad][kInStride], s_y[kPad][kInStride];
    __shared__ float s_h[5][kPad][kHStride];   // horizontally filtered x, y, x^2, y^2, xy
    __shared__ float s_red[kLossThreads / 32];
    const int tid = threadIdx.x;
    const int x0 = blockIdx.x * kPatch, y0 = blockIdx.y * kPatch;
    const int tx = tid % kPatch, r0 = (tid / kPatch) * kOut;   // the vertical pass: column tx, rows r0 .. r0 + 3
    const int px = x0 + tx;
    const size_t plane = (size_t)H * W * 3;
    float l1_sum = 0.f, ssim_sum = 0.f;
    for (int c = 0; c < 3; ++c) {
        for (int k = tid; k < kPad * kPad; k += kLossThreads) {
            const int ry = k / kPad, rx = k - ry * kPad;
            const int gy = y0 + ry - kHalf, gx = x0 + rx - kHalf;
            const bool ok = gy >= 0 && gy < H && gx >= 0 && gx < W;   // zero padding outside the image
            const size_t idx = ((size_t)gy * W + gx) * 3 + c;
            s_x[ry][rx] = ok ? x[idx] : 0.f;
            s_y[ry][rx] = ok ? y[idx] : 0.f;
        }
        __syncthreads();
        for (int item = tid; item < kPad * kGroups; item += kLossThreads) {
            const int ry = item % kPad, cx = (item / kPad) * kOut;
            float a[kOut] = {}, b[kOut] = {}, aa[kOut] = {}, bb[kOut] = {}, ab[kOut] = {};
#pragma unroll
            for (int k = 0; k < kSpan; ++k) {
                const float xv = s_x[ry][cx + k], yv = s_y[ry][cx + k];
                slide(a, xv, k, win); slide(b, yv, k, win);
                slide(aa, xv * xv, k, win); slide(bb, yv * yv, k, win); slide(ab, xv * yv, k, win);
            }
#pragma unroll
            for (int j = 0; j < kOut; ++j) {
                s_h[0][ry][cx + j] = a[j]; s_h[1][ry][cx + j] = b[j]; s_h[2][ry][cx + j] = aa[j];
                s_h[3][ry][cx + j] = bb[j]; s_h[4][ry][cx + j] = ab[j];
            }
        }
        __syncthreads();
        float m1[kOut] = {}, m2[kOut] = {}, e11[kOut] = {}, e22[kOut] = {}, e12[kOut] = {};
#pragma unroll
        for (int k = 0; k < kSpan; ++k) {
            slide(m1, s_h[0][r0 + k][tx], k, win); slide(m2, s_h[1][r0 + k][tx], k, win);
            slide(e11, s_h[2][r0 + k][tx], k, win); slide(e22, s_h[3][r0 + k][tx], k, win);
            slide(e12, s_h[4][r0 + k][tx], k, win);
        }
#pragma unroll
        for (int j = 0; j < kOut; ++j) {
            const int py = y0 + r0 + j;
            if (px < W && py < H) {
                const float C1 = 0.01f * 0.01f, C2 = 0.03f * 0.03f;
                const float s11 = e11[j] - m1[j] * m1[j], s22 = e22[j] - m2[j] * m2[j], s12 = e12[j] - m1[j] * m2[j];
                const float A1 = 2.f * m1[j] * m2[j] + C1, A2 = 2.f * s12 + C2;
                const float B1 = m1[j] * m1[j] + m2[j] * m2[j] + C1, B2 = s11 + s22 + C2;
                const float inv = 1.f / (B1 * B2);
                const float S = A1 * A2 * inv;
                const float dS_dm1 = (2.f * m2[j] * (A2 - A1) * B1 * B2 - A1 * A2 * 2.f * m1[j] * (B2 - B1)) * inv * inv;
                const float dS_de11 = -A1 * A2 * inv / B2;
                const float dS_de12 = 2.f * A1 * inv;
                const size_t idx = ((size_t)py * W + px) * 3 + c;
                maps[idx] = g * dS_dm1; maps[plane + idx] = g * dS_de11; maps[2 * plane + idx] = g * dS_de12;
                ssim_sum += S;
                l1_sum += fabsf(s_x[r0 + j + kHalf][tx + kHalf] - s_y[r0 + j + kHalf][tx + kHalf]);
            }
        }
        __syncthreads();   // the tiles are reloaded for the next channel
    }
    const float l1_total = block_sum(l1_sum, s_red);
    const float ssim_total = block_sum(ssim_sum, s_red);
    if (tid == 0) { atomicAdd(sums, l1_total); atomicAdd(sums + 1, ssim_total); }
}

__global__ void __launch_bounds__(kLossThreads)
ssim_gradient_kernel(const float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ maps, const int H,
                     const int W, const Window win, const float l1_weight, float* __restrict__ v_image) {
    __shared__ float s_m[3][kPad][kInStride];
    __shared__ float s_h[3][kPad][kHStride];
    const int tid = threadIdx.x;
    const int x0 = blockIdx.x * kPatch, y0 = blockIdx.y * kPatch;
    const int tx = tid % kPatch, r0 = (tid / kPatch) * kOut;
    const int px = x0 + tx;
    const size_t plane = (size_t)H * W * 3;
    for (int c = 0; c < 3; ++c) {
        for (int k = tid; k < kPad * kPad; k += kLossThreads) {
            const int ry = k / kPad, rx = k - ry * kPad;
            const int gy = y0 + ry - kHalf, gx = x0 + rx - kHalf;
            const bool ok = gy >= 0 && gy < H && gx >= 0 && gx < W;
            const size_t idx = ((size_t)gy * W + gx) * 3 + c;
#pragma unroll
            for (int q = 0; q < 3; ++q) s_m[q][ry][rx] = ok ? maps[q * plane + idx] : 0.f;
        }
        __syncthreads();
        for (int item = tid; item < kPad * kGroups; item += kLossThreads) {
            const int ry = item % kPad, cx = (item / kPad) * kOut;
            float a0[kOut] = {}, a1[kOut] = {}, a2[kOut] = {};
#pragma unroll
            for (int k = 0; k < kSpan; ++k) {
                slide(a0, s_m[0][ry][cx + k], k, win); slide(a1, s_m[1][ry][cx + k], k, win);
                slide(a2, s_m[2][ry][cx + k], k, win);
            }
#pragma unroll
            for (int j = 0; j < kOut; ++j) { s_h[0][ry][cx + j] = a0[j]; s_h[1][ry][cx + j] = a1[j]; s_h[2][ry][cx + j] = a2[j]; }
        }
        __syncthreads();
        float c0[kOut] = {}, c1[kOut] = {}, c2[kOut] = {};
#pragma unroll
        for (int k = 0; k < kSpan; ++k) {
            slide(c0, s_h[0][r0 + k][tx], k, win); slide(c1, s_h[1][r0 + k][tx], k, win);
            slide(c2, s_h[2][r0 + k][tx], k, win);
        }
#pragma unroll
        for (int j = 0; j < kOut; ++j) {
            const int py = y0 + r0 + j;
            if (px < W && py < H) {
                const size_t idx = ((size_t)py * W + px) * 3 + c;
                const float xv = x[idx], yv = y[idx];
                const float d = xv - yv;
                const float sign = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
                v_image[idx] = c0[j] + 2.f * xv * c1[j] + yv * c2[j] + l1_weight * sign;
            }
        }
        __syncthreads();
    }
}

// lambda = 0: the loss is the plain L1 term and needs none of the windowed sums.  One pass: dL/dx = sign(x - y) / count,
// the block's share of mean|x - y| added to the loss.  VEC: all arrays aligned for 4-element accesses.  U8: the
// target is 8-bit (the form datasets hold images in) and stands for value / 255.
template <bool VEC, bool U8>
__global__ void __launch_bounds__(kLossThreads)
l1_gradient_kernel(const float* __restrict__ x, const void* __restrict__ target, const long long count, const float inv_count,
                   float* __restrict__ v_image, float* __restrict__ loss) {
    const float* yf = static_cast<const float*>(target);
    const unsigned char* yb = static_cast<const unsigned char*>(target);
    const long long stride = (long long)gridDim.x * kLossThreads;
    const long long first = (long long)blockIdx.x * kLossThreads + threadIdx.x;
    float acc = 0.f;
    auto one = [&](const float a, const float b) {
        const float d = a - b;
        acc += fabsf(d);
        return d > 0.f ? inv_count : (d < 0.f ? -inv_count : 0.f);
    };
    auto target_at = [&](const long long i) { return U8 ? (float)yb[i] * (1.0f / 255.0f) : yf[i]; };
    if (VEC) {
        const long long quads = count / 4;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        float4* v4 = reinterpret_cast<float4*>(v_image);
        for (long long i = first; i < quads; i += stride) {
            const float4 a = __ldg(x4 + i);
            float4 b;
            if (U8) {
                const uchar4 q = __ldg(reinterpret_cast<const uchar4*>(yb) + i);
                b = make_float4(q.x * (1.0f / 255.0f), q.y * (1.0f / 255.0f), q.z * (1.0f / 255.0f), q.w * (1.0f / 255.0f));
            } else {
                b = __ldg(reinterpret_cast<const float4*>(yf) + i);
            }
            v4[i] = make_float4(one(a.x, b.x), one(a.y, b.y), one(a.z, b.z), one(a.w, b.w));
        }
        for (long long i = quads * 4 + first; i < count; i += stride) v_image[i] = one(x[i], target_at(i));   // at most three
    } else {
        for (long long i = first; i < count; i += stride) v_image[i] = one(x[i], target_at(i));
    }
    __shared__ float s_red[kLossThreads / 32];
    const float total = block_sum(acc, s_red);
    if (threadIdx.x == 0 && loss) atomicAdd(loss, total * inv_count);
}

static int launch_l1(const float* image, const void* target, bool u8, int H, int W, float* v_image, float* loss, cudaStream_t s) {
    const long long elements = (long long)H * W * 3;
    const float inv_count = 1.f / (float)((double)H * W * 3);
    if (loss) DSB_CUDA_CHECK(cudaMemsetAsync(loss, 0, sizeof(float), s));
    const long long want = (elements / 4 + kLossThreads - 1) / kLossThreads;
    const int blocks = (int)(want < 148 * 8 ? (want > 0 ? want : 1) : 148 * 8);
    const bool vec = (((uintptr_t)image | (uintptr_t)v_image) & 15) == 0 && ((uintptr_t)target & (u8 ? 3 : 15)) == 0;
    if (u8) {
        if (vec) l1_gradient_kernel<true, true><<<blocks, kLossThreads, 0, s>>>(image, target, elements, inv_count, v_image, loss);
        else l1_gradient_kernel<false, true><<<blocks, kLossThreads, 0, s>>>(image, target, elements, inv_count, v_image, loss);
    } else {
        if (vec) l1_gradient_kernel<true, false><<<blocks, kLossThreads, 0, s>>>(image, target, elements, inv_count, v_image, loss);
        else l1_gradient_kernel<false, false><<<blocks, kLossThreads, 0, s>>>(image, target, elements, inv_count, v_image, loss);
    }
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

__global__ void finish_loss_kernel(const float* __restrict__ sums, const float inv_count, const float lambda, float* __restrict__ loss) {
    loss[0] = (1.f - lambda) * sums[0] * inv_count + lambda * (1.f - sums[1] * inv_count);
}

}  // namespace

int64_t image_loss_workspace_bytes(int H, int W) { return ((int64_t)H * W * 3 * 3 + 2) * (int64_t)sizeof(float); }

// workspace: image_loss_workspace_bytes(H, W); loss: one float on the device (may be null); v_image: [H][W][3].
int launch_image_loss(const float* image, const float* target, int H, int W, float lambda_dssim, void* workspace,
                      int64_t workspace_bytes, float* v_image, float* loss, cudaStream_t s) {
    DSB_REQUIRE(H > 0 && W > 0, "image_loss: bad image size");
    DSB_REQUIRE(image && target && v_image && workspace, "image_loss: null pointer");
    DSB_REQUIRE(lambda_dssim >= 0.f && lambda_dssim <= 1.f, "image_loss: lambda must lie in [0, 1]");
    const int64_t need = image_loss_workspace_bytes(H, W);
    if (workspace_bytes < need) {
        set_error("image_loss: workspace of %lld bytes is smaller than the %lld needed", (long long)workspace_bytes, (long long)need);
        return DSB_ERR_WORKSPACE_TOO_SMALL;
    }
    const float count = (float)((double)H * W * 3);
    if (lambda_dssim == 0.f) return launch_l1(image, target, false, H, W, v_image, loss, s);   // plain L1: one pass
    Window win;
    double sum = 0.0, raw[kWin];
    for (int t = 0; t < kWin; ++t) { raw[t] = std::exp(-(double)((t - kHalf) * (t - kHalf)) / (2.0 * 1.5 * 1.5)); sum += raw[t]; }
    for (int t = 0; t < kWin; ++t) win.w[t] = (float)(raw[t] / sum);
    float* maps = reinterpret_cast<float*>(workspace);
    float* sums = maps + (size_t)H * W * 3 * 3;
    DSB_CUDA_CHECK(cudaMemsetAsync(sums, 0, 2 * sizeof(float), s));
    const dim3 grid((W + kPatch - 1) / kPatch, (H + kPatch - 1) / kPatch), block(kLossThreads);
    ssim_moments_kernel<<<grid, block, 0, s>>>(image, target, H, W, win, -lambda_dssim / count, maps, sums);
    DSB_LAUNCH_CHECK();
    ssim_gradient_kernel<<<grid, block, 0, s>>>(image, target, maps, H, W, win, (1.f - lambda_dssim) / count, v_image);
    DSB_LAUNCH_CHECK();
    if (loss) {
        finish_loss_kernel<<<1, 1, 0, s>>>(sums, 1.f / count, lambda_dssim, loss);
        DSB_LAUNCH_CHECK();
    }
    return DSB_OK;
}

// L1 loss against an 8-bit target (value / 255): loss = mean|image - target|, v_image = dL/dimage.
int launch_l1_loss_u8(const float* image, const unsigned char* target, int H, int W, float* v_image, float* loss, cudaStream_t s) {
    DSB_REQUIRE(H > 0 && W > 0, "l1_loss: bad image size");
    DSB_REQUIRE(image && target && v_image, "l1_loss: null pointer");
    return launch_l1(image, target, true, H, W, v_image, loss, s);
}

}  // namespace dsb
