// Stage (f2): per-splat backward -- colour to SH coefficients, pixel mean / conic to 3-D mean, scale and
// rotation -- fused into one pass that also writes every gradient tensor the operator returns.
//
// Takes the place of, in the reference: compute_sh_backward_kernel (cpp/gsplat/sh.cuh:95-203),
// project_gaussians_backward_kernel with project_cov3d_ewa_vjp and scale_rot_to_cov3d_vjp
// (cpp/gsplat/backward.cu:216-393, helpers cpp/gsplat/helpers.cuh:68-220), and the ~25 small tensor
// operations of rasterizer_backward_deepsense (cpp/rasterizer_torch.cu:263-316: zero fills, the
// view-direction subtraction, the colour mask multiply, the column padding of v_xy).  Work the reference
// does and then discards (compensation, AoS->SoA unpack, v_depth) is not reproduced.
//
// Gradient conventions kept from the reference: no gradient from colour to the mean through the view
// direction, no mask for the max(.,0) colour clamp, the EWA VJP ignores the 1.3*tanfov clamp, the
// rotation VJP uses the quaternion as stored (assumed unit), focal lengths are recomputed via atan/tan,
// and only splats with radius > 0 receive geometry gradients.
//
// The 192-byte SH gradient rows -- 60% of all bytes this stage writes -- leave through shared memory
// as contiguous 128-byte warp stores.
#include "common.cuh"

namespace dsb {

namespace {

#ifndef DSB_GEO_THREADS
#define DSB_GEO_THREADS 128
#endif
constexpr int kThreads = DSB_GEO_THREADS;
constexpr int kWarps = kThreads / 32;
constexpr int kShStride = 49;  // odd stride: conflict-free row-per-lane writes

// In accumulate mode a zero contribution costs nothing: no load, no store (most splats are outside any given view).
__device__ __forceinline__ void put(float* p, float v, int accumulate) {
    if (!accumulate) *p = v;
    else if (v != 0.f) *p += v;
}

// Per-view inputs of one launch.  All views share the splat parameters (means, scales, rotations, cov3d);
// each view brings its camera, its records (for the conic), its radii and its accumulator rows.
struct GeoViews {
    int count;
    CamParams cam[DSB_MAX_BATCH_VIEWS];
    const float4* records[DSB_MAX_BATCH_VIEWS];
    const int32_t* radii[DSB_MAX_BATCH_VIEWS];
    const float4* grad_acc[DSB_MAX_BATCH_VIEWS];
};

// One thread per splat.  The contributions of all views of the launch are added in registers (and, for the SH
// rows, in shared memory) and every gradient is written once: a step over V views reads the shared splat
// parameters once and touches the 236 bytes of gradients per splat once instead of V times.  The chain from
// the 3-D covariance to scale and rotation is linear in v_cov3d, so it runs once on the summed v_cov3d.
__global__ void __launch_bounds__(kThreads)
geometry_backward_kernel(const GeoViews gv, const int n, const float* __restrict__ means, const float* __restrict__ scales,
                         const float* __restrict__ rots, const float* __restrict__ cov3d, float* __restrict__ v_means3d,
                         float* __restrict__ v_means2d, float* __restrict__ v_shs, float* __restrict__ v_colors,
                         float* __restrict__ v_opac, float* __restrict__ v_scales, float* __restrict__ v_rots,
                         float* __restrict__ v_cov3d, const int accumulate, const DensifyStats st) {
    __shared__ float s_sh[kWarps][32 * kShStride];
    __shared__ float s_cam[DSB_MAX_BATCH_VIEWS][16];  // per view: view rows 0..2 (12) + camera centre (3)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int k = tid; k < gv.count * 16; k += kThreads) {
        const int v = k >> 4, e = k & 15;
        const CamParams& c = gv.cam[v];
        s_cam[v][e] = e < 12 ? mat_at(c.view, e >> 2, e & 3, c.transposed) : (e < 15 ? c.campos[e - 12] : 0.f);
    }
    __syncthreads();
    const CamParams& cp = gv.cam[0];   // degree, coefficient count and scale modifier are common to the views
    const int i = blockIdx.x * kThreads + tid;
    const int warp_first = blockIdx.x * kThreads + warp * 32;
    const bool live = i < n;

    float mx = 0.f, my = 0.f, mz = 0.f;
    float S[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) {
        mx = means[(size_t)i * 3]; my = means[(size_t)i * 3 + 1]; mz = means[(size_t)i * 3 + 2];
#pragma unroll
        for (int k = 0; k < 6; ++k) S[k] = cov3d[(size_t)i * 6 + k];
    }
    const int row_floats = 3 * cp.max_coeff;
    float* row = &s_sh[warp][lane * kShStride];
    const int active = min((cp.sh_degree + 1) * (cp.sh_degree + 1), cp.max_coeff);

    float vm0 = 0.f, vm1 = 0.f, vm2 = 0.f, vs0 = 0.f, vs1 = 0.f, vs2 = 0.f, vq0 = 0.f, vq1 = 0.f, vq2 = 0.f, vq3 = 0.f;
    float vc[6] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float m2x = 0.f, m2y = 0.f, col_r = 0.f, col_g = 0.f, col_b = 0.f, vop = 0.f;
    bool any_geometry = false;
    float st_norm = 0.f, st_seen = 0.f, st_radius = 0.f;

    for (int view = 0; view < gv.count; ++view) {
        const float* V = s_cam[view];
        float4 g0 = make_float4(0, 0, 0, 0), g1 = g0;
        float gb = 0.f, gz = 0.f;
        int radius = 0;
        if (live) {
            const float4* ga = gv.grad_acc[view] + (size_t)i * 3;
            g0 = ga[0];                 // v_x, v_y, v_conic_a, v_conic_b
            g1 = ga[1];                 // v_conic_c, v_opacity, v_r, v_g
            const float4 g2 = ga[2];    // v_b, v_z (zero unless a depth map's gradient came in), -, -
            gb = g2.x; gz = g2.y;
            radius = gv.radii[view][i];
        }
        m2x += g0.x; m2y += g0.y; col_r += g1.z; col_g += g1.w; col_b += gb; vop += g1.y;

        // ---- colour gradient -> SH coefficients (rows collected in shared memory, written after the loop)
        if (v_shs) {
            float basis[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) basis[k] = 0.f;
            basis[0] = 0.28209479177387814f;
            if (cp.sh_degree >= 1) {
                float dx = mx - V[12], dy = my - V[13], dz = mz - V[14];
                const float inv = rsqrtf(dx * dx + dy * dy + dz * dz);
                const float x = dx * inv, y = dy * inv, z = dz * inv;
                basis[1] = -0.4886025119029199f * y; basis[2] = 0.4886025119029199f * z; basis[3] = -0.4886025119029199f * x;
                if (cp.sh_degree >= 2) {
                    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
                    basis[4] = 1.0925484305920792f * xy;
                    basis[5] = -1.0925484305920792f * yz;
                    basis[6] = 0.31539156525252005f * (2.f * zz - xx - yy);
                    basis[7] = -1.0925484305920792f * xz;
                    basis[8] = 0.5462742152960396f * (xx - yy);
                    if (cp.sh_degree >= 3) {
                        basis[9] = -0.5900435899266435f * y * (3.f * xx - yy);
                        basis[10] = 2.890611442640554f * xy * z;
                        basis[11] = -0.4570457994644658f * y * (4.f * zz - xx - yy);
                        basis[12] = 0.3731763325901154f * z * (2.f * zz - 3.f * xx - 3.f * yy);
                        basis[13] = -0.4570457994644658f * x * (4.f * zz - xx - yy);
                        basis[14] = 1.445305721320277f * z * (xx - yy);
                        basis[15] = -0.5900435899266435f * x * (xx - 3.f * yy);
                    }
                }
            }
            const bool colour = live && (g1.z != 0.f || g1.w != 0.f || gb != 0.f);
            if (view == 0) {
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    if (k < cp.max_coeff) {
                        const float bk = (k < active && live) ? basis[k] : 0.f;
                        row[3 * k] = bk * g1.z; row[3 * k + 1] = bk * g1.w; row[3 * k + 2] = bk * gb;
                    }
                }
            } else if (colour) {
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    if (k < active) {
                        row[3 * k] += basis[k] * g1.z; row[3 * k + 1] += basis[k] * g1.w; row[3 * k + 2] += basis[k] * gb;
                    }
                }
            }
        }

        // ---- geometry of this view
        if (live && radius > 0) {
            any_geometry = true;
            {
                const float sx = st.scale_x * g0.x, sy = st.scale_y * g0.y;
                st_norm += sqrtf(sx * sx + sy * sy);
                st_seen += 1.f;
                st_radius = fmaxf(st_radius, (float)radius);
            }
            const float fx = gv.cam[view].fx_bwd, fy = gv.cam[view].fy_bwd;
            const float tx = V[0] * mx + V[1] * my + V[2] * mz + V[3];
            const float ty = V[4] * mx + V[5] * my + V[6] * mz + V[7];
            const float tz = V[8] * mx + V[9] * my + V[10] * mz + V[11];
            // pixel mean -> view point -> world (rotation transposed)
            {
                const float rw = 1.f / (tz + 1e-6f);
                const float vpx = fx * g0.x, vpy = fy * g0.y;
                const float a = vpx * rw, b = vpy * rw, c = -(vpx * tx + vpy * ty) * rw * rw;
                vm0 += V[0] * a + V[4] * b + V[8] * c;
                vm1 += V[1] * a + V[5] * b + V[9] * c;
                vm2 += V[2] * a + V[6] * b + V[10] * c;
            }
            // view-space depth gradient (cpp/gsplat/backward.cu:253-259; the reference always feeds zeros here)
            vm0 += V[8] * gz; vm1 += V[9] * gz; vm2 += V[10] * gz;
            // conic -> 2-D covariance: v_Sigma = -X G X with X the conic, G the symmetrised conic gradient
            float s00, s01, s11;
            {
                const float4 q0 = gv.records[view][(size_t)i * 3];
                const float cc = gv.records[view][(size_t)i * 3 + 1].x;
                const float a = q0.z, b = q0.w, d = cc;
                const float ga = g0.z, gh = g0.w * 0.5f, gd = g1.x;
                const float m00 = a * ga + b * gh, m01 = a * gh + b * gd, m10 = b * ga + d * gh, m11 = b * gh + d * gd;
                s00 = -(m00 * a + m01 * b);
                s01 = -(m00 * b + m01 * d) - (m10 * a + m11 * b);  // both off-diagonal entries
                s11 = -(m10 * b + m11 * d);
            }
            // EWA VJP: cov2d = T Sigma T^T, T = J R (top two rows matter), no clamp on t here
            {
                const float rz = 1.f / tz, rz2 = rz * rz, rz3 = rz2 * rz;
                const float j00 = fx * rz, j02 = -fx * tx * rz2, j11 = fy * rz, j12 = -fy * ty * rz2;
                float Tm[2][3];
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    Tm[0][c] = j00 * V[c] + j02 * V[8 + c];
                    Tm[1][c] = j11 * V[4 + c] + j12 * V[8 + c];
                }
                const float h = 0.5f * s01;
                float GT[2][3];  // G T
#pragma unroll
                for (int c = 0; c < 3; ++c) {
                    GT[0][c] = s00 * Tm[0][c] + h * Tm[1][c];
                    GT[1][c] = h * Tm[0][c] + s11 * Tm[1][c];
                }
                float vV[3][3];  // T^T G T
#pragma unroll
                for (int r = 0; r < 3; ++r)
#pragma unroll
                    for (int c = 0; c < 3; ++c) vV[r][c] = Tm[0][r] * GT[0][c] + Tm[1][r] * GT[1][c];
                vc[0] += vV[0][0]; vc[1] += vV[0][1] + vV[1][0]; vc[2] += vV[0][2] + vV[2][0];
                vc[3] += vV[1][1]; vc[4] += vV[1][2] + vV[2][1]; vc[5] += vV[2][2];
                const float Sm[3][3] = {{S[0], S[1], S[2]}, {S[1], S[3], S[4]}, {S[2], S[4], S[5]}};
                float vT[2][3];  // 2 G T Sigma
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int c = 0; c < 3; ++c)
                        vT[r][c] = 2.f * (GT[r][0] * Sm[0][c] + GT[r][1] * Sm[1][c] + GT[r][2] * Sm[2][c]);
                float vJ[2][3];  // v_T R^T
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int c = 0; c < 3; ++c) vJ[r][c] = vT[r][0] * V[4 * c] + vT[r][1] * V[4 * c + 1] + vT[r][2] * V[4 * c + 2];
                const float vt0 = -fx * rz2 * vJ[0][2];
                const float vt1 = -fy * rz2 * vJ[1][2];
                const float vt2 = -fx * rz2 * vJ[0][0] + 2.f * fx * tx * rz3 * vJ[0][2] - fy * rz2 * vJ[1][1] + 2.f * fy * ty * rz3 * vJ[1][2];
                vm0 += vt0 * V[0] + vt1 * V[4] + vt2 * V[8];
                vm1 += vt0 * V[1] + vt1 * V[5] + vt2 * V[9];
                vm2 += vt0 * V[2] + vt1 * V[6] + vt2 * V[10];
            }
        }
    }

    // 3-D covariance -> scale and rotation: Sigma = M M^T, M = R(q) diag(s); once, on the summed v_cov3d
    if (any_geometry && scales && rots) {
        const float4 q = *reinterpret_cast<const float4*>(rots + (size_t)i * 4);
        const float w = q.x, x = q.y, y = q.z, z = q.w;
        const float R[3][3] = {{1.f - 2.f * (y * y + z * z), 2.f * (x * y - w * z), 2.f * (x * z + w * y)},
                               {2.f * (x * y + w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - w * x)},
                               {2.f * (x * z - w * y), 2.f * (y * z + w * x), 1.f - 2.f * (x * x + y * y)}};
        const float gs = cp.scale_modifier;
        const float sc[3] = {gs * scales[(size_t)i * 3], gs * scales[(size_t)i * 3 + 1], gs * scales[(size_t)i * 3 + 2]};
        const float G[3][3] = {{vc[0], 0.5f * vc[1], 0.5f * vc[2]}, {0.5f * vc[1], vc[3], 0.5f * vc[4]}, {0.5f * vc[2], 0.5f * vc[4], vc[5]}};
        float vM[3][3], vR[3][3];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int c = 0; c < 3; ++c)
                vM[r][c] = 2.f * (G[r][0] * R[0][c] + G[r][1] * R[1][c] + G[r][2] * R[2][c]) * sc[c];
        vs0 = (R[0][0] * vM[0][0] + R[1][0] * vM[1][0] + R[2][0] * vM[2][0]) * gs;
        vs1 = (R[0][1] * vM[0][1] + R[1][1] * vM[1][1] + R[2][1] * vM[2][1]) * gs;
        vs2 = (R[0][2] * vM[0][2] + R[1][2] * vM[1][2] + R[2][2] * vM[2][2]) * gs;
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int c = 0; c < 3; ++c) vR[r][c] = vM[r][c] * sc[c];
        vq0 = 2.f * (x * (vR[2][1] - vR[1][2]) + y * (vR[0][2] - vR[2][0]) + z * (vR[1][0] - vR[0][1]));
        vq1 = 2.f * (-2.f * x * (vR[1][1] + vR[2][2]) + y * (vR[1][0] + vR[0][1]) + z * (vR[2][0] + vR[0][2]) + w * (vR[2][1] - vR[1][2]));
        vq2 = 2.f * (x * (vR[1][0] + vR[0][1]) - 2.f * y * (vR[0][0] + vR[2][2]) + z * (vR[2][1] + vR[1][2]) + w * (vR[0][2] - vR[2][0]));
        vq3 = 2.f * (x * (vR[2][0] + vR[0][2]) + y * (vR[2][1] + vR[1][2]) - 2.f * z * (vR[0][0] + vR[1][1]) + w * (vR[1][0] - vR[0][1]));
    }

    if (live && st.grad_norm_sum && st_seen > 0.f) {   // always added: the caller clears them when it densifies
        st.grad_norm_sum[i] += st_norm;
        st.visible_count[i] += st_seen;
        st.max_radius[i] = fmaxf(st.max_radius[i], st_radius);
    }
    if (live) {
        if (v_means3d) { float* p = v_means3d + (size_t)i * 3; put(p, vm0, accumulate); put(p + 1, vm1, accumulate); put(p + 2, vm2, accumulate); }
        if (v_means2d) { float* p = v_means2d + (size_t)i * 3; put(p, m2x, accumulate); put(p + 1, m2y, accumulate); put(p + 2, 0.f, accumulate); }
        if (v_colors) { float* p = v_colors + (size_t)i * 3; put(p, col_r, accumulate); put(p + 1, col_g, accumulate); put(p + 2, col_b, accumulate); }
        if (v_opac) put(v_opac + i, vop, accumulate);
        if (v_scales) { float* p = v_scales + (size_t)i * 3; put(p, vs0, accumulate); put(p + 1, vs1, accumulate); put(p + 2, vs2, accumulate); }
        if (v_rots) {
            float4* p = reinterpret_cast<float4*>(v_rots + (size_t)i * 4);
            float4 o = make_float4(vq0, vq1, vq2, vq3);
            if (!accumulate) {
                *p = o;
            } else if (vq0 != 0.f || vq1 != 0.f || vq2 != 0.f || vq3 != 0.f) {
                const float4 c = *p;
                o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
                *p = o;
            }
        }
        if (v_cov3d) {
            float* p = v_cov3d + (size_t)i * 6;
#pragma unroll
            for (int k = 0; k < 6; ++k) put(p + k, vc[k], accumulate);
        }
    }

    if (v_shs) {
        __syncwarp();
        const int rows = min(32, n - warp_first);
        if (rows > 0) {
            float* out = v_shs + (size_t)warp_first * row_floats;
            const int total = rows * row_floats;
            for (int k = lane; k < total; k += 32) {
                const int r = k / row_floats;
                const float val = s_sh[warp][r * kShStride + (k - r * row_floats)];
                if (!accumulate) out[k] = val;
                else if (val != 0.f) out[k] += val;
            }
        }
    }
}

}  // namespace

// views: `count` cameras with their records, radii and accumulator rows (count <= DSB_MAX_BATCH_VIEWS).
int launch_geometry_backward_views(const CamParams* cps, int count, int n, const float* means, const float* scales,
                                   const float* rots, const float* cov3d, const float* const* records,
                                   const int32_t* const* radii, const float* const* grad_acc, float* v_means3d,
                                   float* v_means2d, float* v_shs, float* v_colors, float* v_opac, float* v_scales,
                                   float* v_rots, float* v_cov3d, int accumulate, cudaStream_t s,
                                   const DensifyStats* stats) {
    if (n == 0 || count == 0) return DSB_OK;
    DensifyStats st;
    if (stats) {
        st = *stats;
        DSB_REQUIRE(st.grad_norm_sum && st.visible_count && st.max_radius,
                    "geometry_backward: the three statistics arrays come together");
    }
    DSB_REQUIRE(count > 0 && count <= DSB_MAX_BATCH_VIEWS, "geometry_backward: %d views in one call (at most %d)", count,
                DSB_MAX_BATCH_VIEWS);
    DSB_REQUIRE(means && cov3d && records && radii && grad_acc, "geometry_backward: null required pointer");
    DSB_REQUIRE(!v_rots || ((uintptr_t)v_rots & 15) == 0, "geometry_backward: v_rotations must be 16-byte aligned");
    DSB_REQUIRE(!rots || ((uintptr_t)rots & 15) == 0, "geometry_backward: rotations must be 16-byte aligned");
    GeoViews gv;
    gv.count = count;
    for (int v = 0; v < count; ++v) {
        DSB_REQUIRE(records[v] && radii[v] && grad_acc[v], "geometry_backward: null pointer for view %d", v);
        DSB_REQUIRE(cps[v].max_coeff <= 16, "geometry_backward: at most 16 SH coefficients");
        DSB_REQUIRE(cps[v].max_coeff == cps[0].max_coeff && cps[v].sh_degree == cps[0].sh_degree &&
                        cps[v].scale_modifier == cps[0].scale_modifier,
                    "geometry_backward: the views of one call must share SH degree and scale modifier");
        gv.cam[v] = cps[v];
        gv.records[v] = reinterpret_cast<const float4*>(records[v]);
        gv.radii[v] = radii[v];
        gv.grad_acc[v] = reinterpret_cast<const float4*>(grad_acc[v]);
    }
    geometry_backward_kernel<<<(n + kThreads - 1) / kThreads, kThreads, 0, s>>>(gv, n, means, scales, rots, cov3d, v_means3d,
                                                                              v_means2d, v_shs, v_colors, v_opac, v_scales,
                                                                              v_rots, v_cov3d, accumulate, st);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int launch_geometry_backward(const CamParams& cp, int n, const float* means, const float* scales, const float* rots,
                             const float* records, const float* cov3d, const int32_t* radii, const float* grad_acc,
                             float* v_means3d, float* v_means2d, float* v_shs, float* v_colors, float* v_opac,
                             float* v_scales, float* v_rots, float* v_cov3d, int accumulate, cudaStream_t s) {
    return launch_geometry_backward_views(&cp, 1, n, means, scales, rots, cov3d, &records, &radii, &grad_acc, v_means3d,
                                          v_means2d, v_shs, v_colors, v_opac, v_scales, v_rots, v_cov3d, accumulate, s);
}

}  // namespace dsb
