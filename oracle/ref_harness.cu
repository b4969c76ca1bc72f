// Driver for the REFERENCE's own CUDA kernels, used only as a test checker and as the "reference on
// the same GPU" timing arm.  TEST INFRASTRUCTURE ONLY; never linked into the product library.
//
// oracle/Makefile compiles this file together with the reference's kernel sources where they lie
// (cpp/rasterizer_kernels.cu, cpp/gsplat/backward.cu; cpp/gsplat/sh.cuh is included below) into
// oracle/_ref/libref_splat.so, with the reference's own pip flags (-O3 --use_fast_math, setup.py:8).
// The reference's host orchestration lives in a torch extension (cpp/rasterizer_torch.cu,
// cpp/gsplat/bindings.cu); this file restates that orchestration on raw device buffers so that the
// kernels can be launched without torch: same launch shapes, same thrust calls, same two host
// read-backs, same zero fills.  Buffers are allocated once per call rather than per stage, which
// only favours the reference's timings.
#include <cstdint>
#include <cstdio>
#include <cmath>
#include <cuda_runtime.h>
#include <thrust/device_ptr.h>
#include <thrust/scan.h>
#include <thrust/sort.h>
#include <thrust/functional.h>

#include "rasterizer_kernels.cuh"
#include "gsplat/backward.cuh"
#include "gsplat/config.h"
#include "gsplat/sh.cuh"

#define CK(x)                                                                                   \
    do {                                                                                        \
        cudaError_t e_ = (x);                                                                   \
        if (e_ != cudaSuccess) {                                                                \
            std::snprintf(g_err, sizeof(g_err), "%s:%d %s", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return -1;                                                                          \
        }                                                                                       \
    } while (0)

static char g_err[512] = "";

struct RefArgs {
    int32_t N, H, W, sh_degree, max_sh_degree;
    float tanfovx, tanfovy, scale_modifier;
    // host inputs
    const float *means, *shs, *opac, *scales, *rots, *view, *proj, *campos, *bg, *v_image;
    // host outputs (any may be null)
    int32_t* radii;
    uint8_t* gaussians;  // N * 48 bytes, the reference's packed record
    float* cov3d;
    int64_t* keys_sorted;
    int32_t* ids_sorted;
    int64_t k_capacity;  // capacity of keys_sorted / ids_sorted
    int32_t* tile_indices;
    float* image;
    float* final_T;
    int32_t* final_idx;
    float *v_mean, *v_xy, *v_conic, *v_colors, *v_opacity, *v_sh, *v_scale, *v_rot, *v_cov3d;
    int64_t k_out;
    int32_t iters, warmup, do_backward;
    float ms[8];  // preprocess, keys (scan + 2 read-backs + kernel), sort, ranges, blend, bwd blend, bwd sh, bwd projection
    float ms_forward, ms_backward;
};

__global__ void ref_viewdirs_kernel(const float* means, const float* campos, float* out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < 3 * n) out[i] = means[i] - campos[i % 3];  // cpp/rasterizer_torch.cu:291
}

__global__ void ref_tile_bins_kernel(const int32_t* ti, int32_t* bins, int t) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < t) { bins[2 * i] = ti[i]; bins[2 * i + 1] = ti[i + 1]; }  // cpp/rasterizer_torch.cu:277-283
}

static float fov_to_focal(float fov, float pixels) { return pixels / (2.0f * tanf(fov / 2.0f)); }  // cpp/rasterizer_torch.cu:78-81

template <class T> static cudaError_t dmalloc(T** p, size_t n) { return cudaMalloc((void**)p, n ? n * sizeof(T) : sizeof(T)); }

extern "C" const char* ref_last_error() { return g_err; }

extern "C" int ref_run(RefArgs* a) {
    const int N = a->N, H = a->H, W = a->W;
    if (N <= 0 || H <= 0 || W <= 0) { std::snprintf(g_err, sizeof(g_err), "empty problem"); return -2; }
    if (a->max_sh_degree != 3) { std::snprintf(g_err, sizeof(g_err), "reference asserts max_sh_degree == 3"); return -2; }
    const int threads = 768;  // cpp/rasterizer_torch.cu:131
    const int blocks = (N + threads - 1) / threads;
    const int tw = (W + TILE_SIZE - 1) / TILE_SIZE, th = (H + TILE_SIZE - 1) / TILE_SIZE, T = tw * th;
    const int max_coeff = (a->max_sh_degree + 1) * (a->max_sh_degree + 1);

    float *d_means, *d_shs, *d_opac, *d_scales, *d_rots, *d_view, *d_proj, *d_campos, *d_bg, *d_vimg;
    CK(dmalloc(&d_means, (size_t)N * 3)); CK(dmalloc(&d_shs, (size_t)N * 3 * max_coeff)); CK(dmalloc(&d_opac, (size_t)N));
    CK(dmalloc(&d_scales, (size_t)N * 3)); CK(dmalloc(&d_rots, (size_t)N * 4)); CK(dmalloc(&d_view, 16)); CK(dmalloc(&d_proj, 16));
    CK(dmalloc(&d_campos, 3)); CK(dmalloc(&d_bg, 4)); CK(dmalloc(&d_vimg, (size_t)H * W * 3));
    CK(cudaMemcpy(d_means, a->means, (size_t)N * 12, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_shs, a->shs, (size_t)N * 12 * max_coeff, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_opac, a->opac, (size_t)N * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_scales, a->scales, (size_t)N * 12, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_rots, a->rots, (size_t)N * 16, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_view, a->view, 64, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_proj, a->proj, 64, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_campos, a->campos, 12, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_bg, a->bg, 12, cudaMemcpyHostToDevice));
    if (a->v_image) CK(cudaMemcpy(d_vimg, a->v_image, (size_t)H * W * 12, cudaMemcpyHostToDevice));
    else CK(cudaMemset(d_vimg, 0, (size_t)H * W * 12));

    int32_t *d_radii, *d_block_sums, *d_tile_indices, *d_final_idx, *d_tile_bins, *d_ids = nullptr;
    int64_t* d_keys = nullptr;
    Gaussian* d_g;
    float *d_cov3d, *d_image, *d_final_T;
    CK(dmalloc(&d_radii, (size_t)N)); CK(dmalloc(&d_block_sums, (size_t)blocks)); CK(dmalloc(&d_tile_indices, (size_t)T + 1));
    CK(dmalloc(&d_final_idx, (size_t)H * W)); CK(dmalloc(&d_tile_bins, (size_t)T * 2)); CK(dmalloc(&d_g, (size_t)N));
    CK(dmalloc(&d_cov3d, (size_t)N * 6)); CK(dmalloc(&d_image, (size_t)H * W * 3)); CK(dmalloc(&d_final_T, (size_t)H * W));
    float *d_v_alpha, *d_v_xy, *d_v_conic, *d_v_colors, *d_v_opacity, *d_viewdirs, *d_v_sh, *d_v_depth, *d_v_cov2d,
        *d_v_cov3d, *d_v_mean, *d_v_scale, *d_v_quat;
    CK(dmalloc(&d_v_alpha, (size_t)H * W)); CK(dmalloc(&d_v_xy, (size_t)N * 2)); CK(dmalloc(&d_v_conic, (size_t)N * 3));
    CK(dmalloc(&d_v_colors, (size_t)N * 3)); CK(dmalloc(&d_v_opacity, (size_t)N)); CK(dmalloc(&d_viewdirs, (size_t)N * 3));
    CK(dmalloc(&d_v_sh, (size_t)N * 48)); CK(dmalloc(&d_v_depth, (size_t)N)); CK(dmalloc(&d_v_cov2d, (size_t)N * 3));
    CK(dmalloc(&d_v_cov3d, (size_t)N * 6)); CK(dmalloc(&d_v_mean, (size_t)N * 3)); CK(dmalloc(&d_v_scale, (size_t)N * 3));
    CK(dmalloc(&d_v_quat, (size_t)N * 4));

    const float focal_y = H / (2 * a->tanfovy), focal_x = W / (2 * a->tanfovx);  // cpp/rasterizer_torch.cu:144-147
    const float c_x = W / 2.0f, c_y = H / 2.0f;

    cudaEvent_t ev[10];
    for (auto& e : ev) CK(cudaEventCreate(&e));
    for (float& m : a->ms) m = 0.f;
    a->ms_forward = a->ms_backward = 0.f;
    int64_t k_alloc = 0;
    int32_t K = 0;
    const int total_iters = a->warmup + (a->iters > 0 ? a->iters : 1);

    for (int it = 0; it < total_iters; ++it) {
        const bool timed = it >= a->warmup;
        // ---- forward: cpp/rasterizer_torch.cu:170-208
        CK(cudaEventRecord(ev[0]));
        rasterizer_preprocessing_kernel<<<blocks, threads, threads * sizeof(int)>>>(
            d_means, d_shs, d_scales, d_rots, d_proj, d_view, d_campos, d_opac, nullptr, nullptr, a->scale_modifier,
            max_coeff, a->sh_degree, N, focal_x, focal_y, a->tanfovx, a->tanfovy, c_x, c_y, W, H, d_radii, d_block_sums,
            d_g, d_cov3d);
        CK(cudaEventRecord(ev[1]));
        {  // duplicate_keys, :83-113
            thrust::device_ptr<int32_t> bs(d_block_sums);
            thrust::exclusive_scan(bs, bs + blocks, bs);
            int32_t total = 0, last_block = 0;
            CK(cudaMemcpy(&total, reinterpret_cast<uint8_t*>(d_g) + (size_t)(N - 1) * sizeof(Gaussian) + offsetof(Gaussian, size_occupied_tiles),
                          4, cudaMemcpyDeviceToHost));
            CK(cudaMemcpy(&last_block, d_block_sums + blocks - 1, 4, cudaMemcpyDeviceToHost));
            K = total + last_block;
            if (K <= 0) { std::snprintf(g_err, sizeof(g_err), "no (tile, splat) pairs (K=%d)", K); return -3; }
            if (K > k_alloc) {
                if (d_keys) { cudaFree(d_keys); cudaFree(d_ids); }
                CK(dmalloc(&d_keys, (size_t)K)); CK(dmalloc(&d_ids, (size_t)K));
                k_alloc = K;
            }
            calculate_keys_and_indices_kernel<<<blocks, threads>>>(d_g, d_block_sums, d_radii, d_keys, d_ids, N, K, W, H);
        }
        CK(cudaEventRecord(ev[2]));
        {  // sort_by_keys, :70-76
            thrust::device_ptr<int64_t> k(d_keys);
            thrust::device_ptr<int32_t> v(d_ids);
            thrust::sort_by_key(k, k + K, v);
        }
        CK(cudaEventRecord(ev[3]));
        {  // identify_tile_ranges, :23-42
            CK(cudaMemsetAsync(d_tile_indices, 0, (size_t)(T + 1) * 4));
            CK(cudaMemcpy(d_tile_indices + T, &K, 4, cudaMemcpyHostToDevice));
            identify_tile_ranges_kernel<<<(K + threads - 1) / threads, threads>>>(d_keys, d_tile_indices, K);
            thrust::device_ptr<int32_t> ti(d_tile_indices);
            thrust::inclusive_scan(ti, ti + T + 1, ti, thrust::maximum<int32_t>());
        }
        CK(cudaEventRecord(ev[4]));
        {  // rasterizer_cuda_forward, :44-68
            dim3 block(TILE_SIZE, TILE_SIZE), grid(tw, th);
            render_image_kernel<<<grid, block>>>(d_g, d_ids, d_tile_indices, d_image, W, H, d_final_T, d_final_idx);
        }
        CK(cudaEventRecord(ev[5]));
        if (a->do_backward) {
            // ---- backward: cpp/rasterizer_torch.cu:263-316 with cpp/gsplat/bindings.cu:22-194
            ref_tile_bins_kernel<<<(T + 255) / 256, 256>>>(d_tile_indices, d_tile_bins, T);
            CK(cudaMemsetAsync(d_v_alpha, 0, (size_t)H * W * 4));
            CK(cudaMemsetAsync(d_v_xy, 0, (size_t)N * 8)); CK(cudaMemsetAsync(d_v_conic, 0, (size_t)N * 12));
            CK(cudaMemsetAsync(d_v_colors, 0, (size_t)N * 12)); CK(cudaMemsetAsync(d_v_opacity, 0, (size_t)N * 4));
            {
                const dim3 tile_bounds(tw, th, 1), block(TILE_SIZE, TILE_SIZE, 1), img_size(W, H, 1);
                rasterize_backward_kernel<<<tile_bounds, block>>>(
                    tile_bounds, img_size, d_ids, (int2*)d_tile_bins, d_g, d_opac, *(float3*)d_bg, d_final_T, d_final_idx,
                    (float3*)d_vimg, d_v_alpha, (float2*)d_v_xy, (float3*)d_v_conic, (float3*)d_v_colors, d_v_opacity);
            }
            CK(cudaEventRecord(ev[6]));
            ref_viewdirs_kernel<<<(3 * N + 255) / 256, 256>>>(d_means, d_campos, d_viewdirs, N);
            CK(cudaMemsetAsync(d_v_sh, 0, (size_t)N * 48 * 4));
            compute_sh_backward_kernel<<<(N + N_THREADS - 1) / N_THREADS, N_THREADS>>>(
                N, 3, a->sh_degree, (float3*)d_viewdirs, d_v_colors, d_v_sh);
            CK(cudaEventRecord(ev[7]));
            const float fx = fov_to_focal(2 * atanf(a->tanfovx), W), fy = fov_to_focal(2 * atanf(a->tanfovy), H);
            CK(cudaMemsetAsync(d_v_depth, 0, (size_t)N * 4)); CK(cudaMemsetAsync(d_v_cov2d, 0, (size_t)N * 12));
            CK(cudaMemsetAsync(d_v_cov3d, 0, (size_t)N * 24)); CK(cudaMemsetAsync(d_v_mean, 0, (size_t)N * 12));
            CK(cudaMemsetAsync(d_v_scale, 0, (size_t)N * 12)); CK(cudaMemsetAsync(d_v_quat, 0, (size_t)N * 16));
            {
                const float4 intrins = {fx, fy, c_x, c_y};
                const dim3 img_size(W, H, 1);
                project_gaussians_backward_kernel<<<(N + N_THREADS - 1) / N_THREADS, N_THREADS>>>(
                    N, (float3*)d_means, (float3*)d_scales, a->scale_modifier, (float4*)d_rots, d_view, intrins, img_size,
                    d_g, d_cov3d, d_radii, (float2*)d_v_xy, d_v_depth, (float3*)d_v_conic, (float3*)d_v_cov2d, d_v_cov3d,
                    (float3*)d_v_mean, (float3*)d_v_scale, (float4*)d_v_quat);
            }
            CK(cudaEventRecord(ev[8]));
        }
        CK(cudaDeviceSynchronize());
        CK(cudaGetLastError());
        if (timed) {
            float t;
            for (int s = 0; s < 5; ++s) { CK(cudaEventElapsedTime(&t, ev[s], ev[s + 1])); a->ms[s] += t; }
            CK(cudaEventElapsedTime(&t, ev[0], ev[5])); a->ms_forward += t;
            if (a->do_backward) {
                for (int s = 5; s < 8; ++s) { CK(cudaEventElapsedTime(&t, ev[s], ev[s + 1])); a->ms[s] += t; }
                CK(cudaEventElapsedTime(&t, ev[5], ev[8])); a->ms_backward += t;
            }
        }
    }
    const float inv = 1.0f / (a->iters > 0 ? a->iters : 1);
    for (float& m : a->ms) m *= inv;
    a->ms_forward *= inv; a->ms_backward *= inv;
    a->k_out = K;

    if (a->radii) CK(cudaMemcpy(a->radii, d_radii, (size_t)N * 4, cudaMemcpyDeviceToHost));
    if (a->gaussians) CK(cudaMemcpy(a->gaussians, d_g, (size_t)N * sizeof(Gaussian), cudaMemcpyDeviceToHost));
    if (a->cov3d) CK(cudaMemcpy(a->cov3d, d_cov3d, (size_t)N * 24, cudaMemcpyDeviceToHost));
    if (a->keys_sorted && a->k_capacity >= K) CK(cudaMemcpy(a->keys_sorted, d_keys, (size_t)K * 8, cudaMemcpyDeviceToHost));
    if (a->ids_sorted && a->k_capacity >= K) CK(cudaMemcpy(a->ids_sorted, d_ids, (size_t)K * 4, cudaMemcpyDeviceToHost));
    if (a->tile_indices) CK(cudaMemcpy(a->tile_indices, d_tile_indices, (size_t)(T + 1) * 4, cudaMemcpyDeviceToHost));
    if (a->image) CK(cudaMemcpy(a->image, d_image, (size_t)H * W * 12, cudaMemcpyDeviceToHost));
    if (a->final_T) CK(cudaMemcpy(a->final_T, d_final_T, (size_t)H * W * 4, cudaMemcpyDeviceToHost));
    if (a->final_idx) CK(cudaMemcpy(a->final_idx, d_final_idx, (size_t)H * W * 4, cudaMemcpyDeviceToHost));
    if (a->do_backward) {
        if (a->v_mean) CK(cudaMemcpy(a->v_mean, d_v_mean, (size_t)N * 12, cudaMemcpyDeviceToHost));
        if (a->v_xy) CK(cudaMemcpy(a->v_xy, d_v_xy, (size_t)N * 8, cudaMemcpyDeviceToHost));
        if (a->v_conic) CK(cudaMemcpy(a->v_conic, d_v_conic, (size_t)N * 12, cudaMemcpyDeviceToHost));
        if (a->v_colors) CK(cudaMemcpy(a->v_colors, d_v_colors, (size_t)N * 12, cudaMemcpyDeviceToHost));
        if (a->v_opacity) CK(cudaMemcpy(a->v_opacity, d_v_opacity, (size_t)N * 4, cudaMemcpyDeviceToHost));
        if (a->v_sh) CK(cudaMemcpy(a->v_sh, d_v_sh, (size_t)N * 192, cudaMemcpyDeviceToHost));
        if (a->v_scale) CK(cudaMemcpy(a->v_scale, d_v_scale, (size_t)N * 12, cudaMemcpyDeviceToHost));
        if (a->v_rot) CK(cudaMemcpy(a->v_rot, d_v_quat, (size_t)N * 16, cudaMemcpyDeviceToHost));
        if (a->v_cov3d) CK(cudaMemcpy(a->v_cov3d, d_v_cov3d, (size_t)N * 24, cudaMemcpyDeviceToHost));
    }
    for (auto& e : ev) cudaEventDestroy(e);
    void* frees[] = {d_means, d_shs, d_opac, d_scales, d_rots, d_view, d_proj, d_campos, d_bg, d_vimg, d_radii, d_block_sums,
                     d_tile_indices, d_final_idx, d_tile_bins, d_g, d_cov3d, d_image, d_final_T, d_v_alpha, d_v_xy, d_v_conic,
                     d_v_colors, d_v_opacity, d_viewdirs, d_v_sh, d_v_depth, d_v_cov2d, d_v_cov3d, d_v_mean, d_v_scale,
                     d_v_quat, d_keys, d_ids};
    for (void* p : frees) if (p) cudaFree(p);
    return 0;
}
