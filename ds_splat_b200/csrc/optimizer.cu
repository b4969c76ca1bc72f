// The step after the operator in a training loop: Adam on a parameter tensor and its gradient.
//
// Not part of the reference (its users call torch.optim.Adam, as graphdeco's train.py does); it follows the
// published algorithm (Kingma & Ba, "Adam: A Method for Stochastic Optimization", algorithm 1) in the form
// torch.optim.Adam applies it without weight decay or amsgrad:
//     m <- b1 m + (1 - b1) g            v <- b2 v + (1 - b2) g^2
//     p <- p - (lr / (1 - b1^t)) * m / (sqrt(v) / sqrt(1 - b2^t) + eps)
// One pass over memory: 16 bytes read (p, g, m, v) and 12 written (p, m, v) per element, so the kernel is bound
// by HBM bandwidth; it moves four elements per thread and trip as float4 when the tensors allow it.
#include <cmath>

#include "common.cuh"

namespace dsb {

namespace {

constexpr int kThreads = 256;

struct AdamConstants {
    float b1, b2, one_minus_b1, one_minus_b2, step_size, inv_bias2_sqrt, eps, grad_scale;
};

__device__ __forceinline__ void adam_one(float& p, const float g_raw, float& m, float& v, const AdamConstants& c) {
    const float g = g_raw * c.grad_scale;
    m = c.b1 * m + c.one_minus_b1 * g;
    v = c.b2 * v + c.one_minus_b2 * g * g;
    const float denom = sqrtf(v) * c.inv_bias2_sqrt + c.eps;
    p -= c.step_size * (m / denom);
}

template <bool VEC4>
__global__ void __launch_bounds__(kThreads)
adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
            const long long count, const AdamConstants c) {
    const long long stride = (long long)gridDim.x * kThreads;
    if (VEC4) {
        float4* p4 = reinterpret_cast<float4*>(p);
        const float4* g4 = reinterpret_cast<const float4*>(g);
        float4* m4 = reinterpret_cast<float4*>(m);
        float4* v4 = reinterpret_cast<float4*>(v);
        const long long n4 = count >> 2;
        for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < n4; i += stride) {
            float4 pp = p4[i], mm = m4[i], vv = v4[i];
            const float4 gg = g4[i];
            adam_one(pp.x, gg.x, mm.x, vv.x, c); adam_one(pp.y, gg.y, mm.y, vv.y, c);
            adam_one(pp.z, gg.z, mm.z, vv.z, c); adam_one(pp.w, gg.w, mm.w, vv.w, c);
            p4[i] = pp; m4[i] = mm; v4[i] = vv;
        }
        for (long long i = (n4 << 2) + (long long)blockIdx.x * kThreads + threadIdx.x; i < count; i += stride)
            adam_one(p[i], g[i], m[i], v[i], c);
    } else {
        for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < count; i += stride)
            adam_one(p[i], g[i], m[i], v[i], c);
    }
}

}  // namespace

// Hyper-parameters arrive as doubles and are combined in double (1 - beta, the bias corrections) before they are
// rounded to float, as torch does with its Python floats: 1.f - 0.999f is off by 1.3e-5 relative.
int launch_adam(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, int64_t count, double lr, double beta1,
                double beta2, double eps, int step, double grad_scale, cudaStream_t s) {
    DSB_REQUIRE(count >= 0, "adam: negative element count");
    if (count == 0) return DSB_OK;
    DSB_REQUIRE(params && grads && exp_avg && exp_avg_sq, "adam: null pointer");
    DSB_REQUIRE(step >= 1, "adam: the step counter starts at 1");
    DSB_REQUIRE(beta1 >= 0.0 && beta1 < 1.0 && beta2 >= 0.0 && beta2 < 1.0 && eps >= 0.0, "adam: bad hyper-parameters");
    AdamConstants c;
    c.b1 = (float)beta1; c.b2 = (float)beta2; c.one_minus_b1 = (float)(1.0 - beta1); c.one_minus_b2 = (float)(1.0 - beta2);
    const double bias1 = 1.0 - std::pow(beta1, (double)step), bias2 = 1.0 - std::pow(beta2, (double)step);
    c.step_size = (float)(lr / bias1);
    c.inv_bias2_sqrt = (float)(1.0 / std::sqrt(bias2));
    c.eps = (float)eps; c.grad_scale = (float)grad_scale;
    const bool vec4 = (((uintptr_t)params | (uintptr_t)grads | (uintptr_t)exp_avg | (uintptr_t)exp_avg_sq) & 15) == 0;
    const long long work = vec4 ? (count + 3) / 4 : count;
    long long blocks = (work + kThreads - 1) / kThreads;
    if (blocks > 148 * 16) blocks = 148 * 16;   // grid-stride loop beyond sixteen blocks per SM
    if (vec4) adam_kernel<true><<<(unsigned)blocks, kThreads, 0, s>>>(params, grads, exp_avg, exp_avg_sq, count, c);
    else adam_kernel<false><<<(unsigned)blocks, kThreads, 0, s>>>(params, grads, exp_avg, exp_avg_sq, count, c);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

}  // namespace dsb
