// Stage (a): per-splat projection, 3-D -> 2-D covariance, conic, SH colour, radius and tile rectangle.
//
// Takes the place of the reference's rasterizer_preprocessing_kernel (cpp/rasterizer_kernels.cu:57-161)
// and its device helpers (:7-55, :163-250, :325-337, :433-659).  One thread per splat; every input
// tensor of a 256-splat block is brought into shared memory with fully coalesced 16-byte loads (the
// caller's tensors are row-per-splat, so a direct per-thread read would stride by 12..192 bytes), and
// every output row goes back out through shared memory as contiguous float4 streams.
//
// Arithmetic note: radii, tile rectangles and depth bits feed integer stages that must agree bit for
// bit with the reference's --use_fast_math build, so the expressions below keep the reference's
// association and this file is compiled with the same flag (same approximate rcp/sqrt/rsqrt and the
// same FMA contraction rules).
#include "common.cuh"
#include "tma.cuh"

namespace dsb {

namespace {

#ifndef DSB_PRE_THREADS
#define DSB_PRE_THREADS 256
#endif
constexpr int kThreads = DSB_PRE_THREADS;
constexpr int kShRow4 = 13;  // padded SH row in float4 units (12 used): conflict-free 16-byte shared loads

__device__ __forceinline__ float sh_channel(const float* f, int ch, int degree, float x, float y, float z) {
    // f = 48 coefficients of one splat, coefficient-major / channel-minor.
    float res = 0.0f;
    res += 0.28209479177387814f * f[ch];
    if (degree >= 1) {
        res += 0.4886025119029199f * (-y * f[3 + ch] + z * f[6 + ch] - x * f[9 + ch]);
        if (degree >= 2) {
            const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
            res += 1.0925484305920792f * xy * f[12 + ch] + -1.0925484305920792f * yz * f[15 + ch] +
                   0.31539156525252005f * (2.0f * zz - xx - yy) * f[18 + ch] + -1.0925484305920792f * xz * f[21 + ch] +
                   0.5462742152960396f * (xx - yy) * f[24 + ch];
            if (degree >= 3) {
                res += -0.5900435899266435f * y * (3 * xx - yy) * f[27 + ch] + 2.890611442640554f * xy * z * f[30 + ch] +
                       -0.4570457994644658f * y * (4 * zz - xx - yy) * f[33 + ch] +
                       0.3731763325901154f * z * (2 * zz - 3 * xx - 3 * yy) * f[36 + ch] +
                       -0.4570457994644658f * x * (4 * zz - xx - yy) * f[39 + ch] + 1.445305721320277f * z * (xx - yy) * f[42 + ch] +
                       -0.5900435899266435f * x * (xx - 3 * yy) * f[45 + ch];
            }
        }
    }
    return fmaxf(res + 0.5f, 0.0f);
}

// a a' + b b' + c c' with the fusion into multiply-adds fixed (intrinsics with explicit rounding are never re-fused):
__device__ __forceinline__ float dot3_first_plain(float a, float a2, float b, float b2, float c, float c2) {
    return __fmaf_rn(c, c2, __fmaf_rn(b, b2, __fmul_rn(a, a2)));
}
__device__ __forceinline__ float dot3_second_plain(float a, float a2, float b, float b2, float c, float c2) {
    return __fmaf_rn(c, c2, __fmaf_rn(a, a2, __fmul_rn(b, b2)));
}

// Cooperative copy of `count` floats from global to shared (coalesced 4-byte lanes).
__device__ __forceinline__ void stage_floats(float* dst, const float* src, int count, int tid) {
    for (int k = tid; k < count; k += kThreads) dst[k] = src[k];
}

// Per-view part of one launch: camera and output buffers.  All views share the splat parameters, which a block
// brings into shared memory once; the 3-D covariance, too, is computed once.
struct PreViews {
    int count;
    CamParams cam[DSB_MAX_BATCH_VIEWS];
    float4* records[DSB_MAX_BATCH_VIEWS];
    int32_t* radii[DSB_MAX_BATCH_VIEWS];
    int32_t* tiles[DSB_MAX_BATCH_VIEWS];
    u64* depth_keys[DSB_MAX_BATCH_VIEWS];
    int* tile_marks[DSB_MAX_BATCH_VIEWS];   // may be null
};

__global__ void __launch_bounds__(kThreads, 768 / kThreads)
preprocess_kernel(const PreViews pv, const int n, const float* __restrict__ means, const float* __restrict__ shs,
                  const float* __restrict__ colors_precomp, const float* __restrict__ opac,
                  const float* __restrict__ scales, const float* __restrict__ rots,
                  const float* __restrict__ cov3d_precomp, float* __restrict__ cov3d, const int sh_vec4, const int use_bulk,
                  const int marks_copy_ints, const u32 copy_polls, int* __restrict__ device_status) {
    extern __shared__ __align__(16) float4 dyn4[];
    __shared__ float s_cams[DSB_MAX_BATCH_VIEWS][32];   // per view: view rows 0..2 (12), projection (16), camera centre (3)
    __shared__ __align__(16) float s_means[kThreads * 3];
    __shared__ __align__(16) float s_scales[kThreads * 3];
    __shared__ __align__(16) float4 s_rec[kThreads * 3];   // output rows of the view being written
    __shared__ __align__(8) uint64_t s_bar;
    const CamParams& cp = pv.cam[0];   // SH degree, coefficient count and scale modifier are common to the views

    const int tid = threadIdx.x;
    const int base = blockIdx.x * kThreads;
    const int cnt = min(kThreads, n - base);
    const int i = base + tid;

    for (int k = tid; k < pv.count * 32; k += kThreads) {
        const int v = k >> 5, e = k & 31;
        const CamParams& c = pv.cam[v];
        s_cams[v][e] = e < 12 ? mat_at(c.view, e >> 2, e & 3, c.transposed)
                     : e < 28 ? mat_at(c.proj, (e - 12) >> 2, (e - 12) & 3, c.transposed)
                     : e < 31 ? c.campos[e - 28] : 0.f;
    }

    // Full blocks with 16-byte aligned inputs are staged by the bulk copy engine (TMA): every thread asks for
    // its own 192-byte SH row (into the padded row layout), one thread asks for the block's 3 KB of means
    // and of scales, and one mbarrier counts the bytes in.  No registers or load instructions are spent on
    // the 54 KB a block brings in.  The wait is bounded.  A block whose wait runs out goes `direct`: it never
    // touches the buffers the copies may still be writing, reads its rows straight from global memory instead,
    // leaves a note in the device status word, and before it exits waits once more (bounded again) so that it
    // does not retire with copies of its own in flight.
    bool staged = false, direct = false;
    if (use_bulk && cnt == kThreads) {
        if (tid == 0) mbar_init(&s_bar, 1);
        __syncthreads();
        if (tid == 0) {
            mbar_arrive_expect_tx(&s_bar, kThreads * 192u + 2u * kThreads * 12u);
            bulk_load(s_means, means + (size_t)base * 3, kThreads * 12u, &s_bar);
            bulk_load(s_scales, scales + (size_t)base * 3, kThreads * 12u, &s_bar);
        }
        bulk_load(dyn4 + tid * kShRow4, shs + (size_t)i * 48, 192u, &s_bar);
        const bool ok = mbar_wait_bounded(&s_bar, 0, copy_polls);
        staged = __syncthreads_and(ok);
        direct = !staged;
        if (direct && tid == 0) atomicCAS(device_status, 0, DSB_STATUS_COPY_WAIT_FELL_BACK);   // never hides an error code
    }
    if (!staged && !direct) {
        stage_floats(s_means, means + (size_t)base * 3, cnt * 3, tid);
        if (scales) stage_floats(s_scales, scales + (size_t)base * 3, cnt * 3, tid);
    }

    const int row_floats = 3 * cp.max_coeff;
    float* s_sh = reinterpret_cast<float*>(dyn4);
    if (shs && !colors_precomp && !staged && !direct) {
        if (sh_vec4) {  // 16 coefficients, 16-byte aligned rows: float4 in, padded float4 rows in shared memory
            const float4* g = reinterpret_cast<const float4*>(shs + (size_t)base * 48);
            const int total4 = cnt * 12;
#pragma unroll
            for (int r = 0; r < 12; ++r) {
                const int k = r * kThreads + tid;
                if (k < total4) {
                    const int row = k / 12;
                    dyn4[row * kShRow4 + (k - row * 12)] = __ldg(g + k);
                }
            }
        } else {  // any other layout: scalar lanes, odd row stride
            const int stride = row_floats | 1;
            const float* g = shs + (size_t)base * row_floats;
            for (int k = tid; k < cnt * row_floats; k += kThreads) {
                const int row = k / row_floats;
                s_sh[row * stride + (k - row * row_floats)] = g[k];
            }
        }
    }
    __syncthreads();

    float S[6] = {0, 0, 0, 0, 0, 0};
    float mx = 0.f, my = 0.f, mz = 0.f, opacity = 0.f;
    const bool live = tid < cnt;
    if (live) {
        const float* mrow = direct ? means + (size_t)i * 3 : s_means + 3 * tid;
        mx = mrow[0]; my = mrow[1]; mz = mrow[2];
        opacity = opac[i];
        // 3-D covariance from scale and rotation (or taken as given).
        if (cov3d_precomp) {
#pragma unroll
            for (int k = 0; k < 6; ++k) S[k] = cov3d_precomp[(size_t)i * 6 + k];
        } else {
            const float4 q = *reinterpret_cast<const float4*>(rots + (size_t)i * 4);
            float r = q.x, x = q.y, y = q.z, z = q.w;
            const float inv_norm = rsqrtf(r * r + x * x + y * y + z * z);
            r = r * inv_norm; x = x * inv_norm; y = y * inv_norm; z = z * inv_norm;
            const float* srow = direct ? scales + (size_t)i * 3 : s_scales + 3 * tid;
            const float sx = srow[0] * cp.scale_modifier, sy = srow[1] * cp.scale_modifier, sz = srow[2] * cp.scale_modifier;
            const float r00 = 1.0f - 2.0f * (y * y + z * z), r01 = 2.0f * (x * y - r * z), r02 = 2.0f * (x * z + r * y);
            const float r10 = 2.0f * (x * y + r * z), r11 = 1.0f - 2.0f * (x * x + z * z), r12 = 2.0f * (y * z - r * x);
            const float r20 = 2.0f * (x * z - r * y), r21 = 2.0f * (y * z + r * x), r22 = 1.0f - 2.0f * (x * x + y * y);
            const float m00 = sx * r00, m01 = sy * r01, m02 = sz * r02;
            const float m10 = sx * r10, m11 = sy * r11, m12 = sz * r12;
            const float m20 = sx * r20, m21 = sy * r21, m22 = sz * r22;
            // Sigma = M M^T.  Which two of the three products of a sum the compiler fuses into multiply-adds depends
            // on the code around the expression, and the integer stages downstream (radius, tile rectangle) must
            // agree bit for bit with the reference's build, so the fusion that build was measured to use is spelled
            // out: entries xx and xz keep the FIRST product as the plain multiply, the other four the SECOND.
            S[0] = dot3_first_plain(m00, m00, m01, m01, m02, m02);
            S[1] = dot3_second_plain(m00, m10, m01, m11, m02, m12);
            S[2] = dot3_first_plain(m00, m20, m01, m21, m02, m22);
            S[3] = dot3_second_plain(m10, m10, m11, m11, m12, m12);
            S[4] = dot3_second_plain(m10, m20, m11, m21, m12, m22);
            S[5] = dot3_second_plain(m20, m20, m21, m21, m22, m22);
        }

    }

    for (int view = 0; view < pv.count; ++view) {
        const CamParams& cv = pv.cam[view];
        const float* s_cam = s_cams[view];
        float4 q0 = make_float4(0, 0, 0, 0), q1 = q0, q2 = q0;
        if (live) {
            const float* V = s_cam;
            const float* P = s_cam + 12;
            int radius = 0, count = 0;
            float tz = 0.0f;
            // Colour.
            float cr, cg, cb;
            if (colors_precomp) {
                cr = colors_precomp[(size_t)i * 3]; cg = colors_precomp[(size_t)i * 3 + 1]; cb = colors_precomp[(size_t)i * 3 + 2];
            } else if (cp.sh_degree > 3) {
                cr = cg = cb = 0.0f;
            } else {
                float dx = mx - s_cam[28], dy = my - s_cam[29], dz = mz - s_cam[30];
                const float inv_norm = rsqrtf(dx * dx + dy * dy + dz * dz);
                dx = dx * inv_norm; dy = dy * inv_norm; dz = dz * inv_norm;
                float f[48];
                if (sh_vec4) {
                    // direct blocks (use_bulk implies 16-byte aligned rows) read the row where it lies
                    const float4* row = direct ? reinterpret_cast<const float4*>(shs) + (size_t)i * 12 : dyn4 + tid * kShRow4;
    #pragma unroll
                    for (int j = 0; j < 12; ++j) {
                        const float4 v = row[j];
                        f[4 * j] = v.x; f[4 * j + 1] = v.y; f[4 * j + 2] = v.z; f[4 * j + 3] = v.w;
                    }
                } else {
                    const float* row = s_sh + tid * (row_floats | 1);
                    const int have = min(row_floats, 3 * (cp.sh_degree + 1) * (cp.sh_degree + 1));
    #pragma unroll
                    for (int j = 0; j < 48; ++j) f[j] = j < have ? row[j] : 0.0f;
                }
                cr = sh_channel(f, 0, cp.sh_degree, dx, dy, dz);
                cg = sh_channel(f, 1, cp.sh_degree, dx, dy, dz);
                cb = sh_channel(f, 2, cp.sh_degree, dx, dy, dz);
            }

            // Frustum test on the projected centre (strict bounds, z_ndc > 0.1).
            const float inv_w = 1.f / (P[12] * mx + P[13] * my + P[14] * mz + P[15]);
            const float ndc_x = inv_w * (P[0] * mx + P[1] * my + P[2] * mz + P[3]);
            const float ndc_y = inv_w * (P[4] * mx + P[5] * my + P[6] * mz + P[7]);
            const float ndc_z = inv_w * (P[8] * mx + P[9] * my + P[10] * mz + P[11]);
            const int in_frustum = ndc_x > -1.f && ndc_x < 1.f && ndc_y > -1.f && ndc_y < 1.f && ndc_z > 0.1f;

            // View-space centre.
            const float tx = V[0] * mx + V[1] * my + V[2] * mz + V[3];
            const float ty = V[4] * mx + V[5] * my + V[6] * mz + V[7];
            tz = V[8] * mx + V[9] * my + V[10] * mz + V[11];

            // EWA projection of the covariance: cov2d = (W J^T)^T Sigma (W J^T), W = view rotation columns.
            const float limx = 1.3f * cv.tanfovx, limy = 1.3f * cv.tanfovy;
            const float txtz = tx / tz, tytz = ty / tz;
            const float t0 = min(limx, max(-limx, txtz)) * tz, t1 = min(limy, max(-limy, tytz)) * tz, t2 = tz;
            const float J[3][3] = {{cv.fx / t2, 0, -(cv.fx * t0) / (t2 * t2)}, {0, cv.fy / t2, -(cv.fy * t1) / (t2 * t2)}, {0, 0, 0}};
            const float Wc[3][3] = {{V[0], V[4], V[8]}, {V[1], V[5], V[9]}, {V[2], V[6], V[10]}};
            float Tm[3][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
    #pragma unroll
            for (int a = 0; a < 3; ++a)
    #pragma unroll
                for (int b = 0; b < 3; ++b)
    #pragma unroll
                    for (int k = 0; k < 3; ++k) Tm[a][b] += Wc[a][k] * J[b][k];
            const float Sm[3][3] = {{S[0], S[1], S[2]}, {S[1], S[3], S[4]}, {S[2], S[4], S[5]}};
            float half[3][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
    #pragma unroll
            for (int a = 0; a < 3; ++a)
    #pragma unroll
                for (int b = 0; b < 3; ++b)
    #pragma unroll
                    for (int k = 0; k < 3; ++k) half[a][b] += Tm[k][a] * Sm[k][b];
            float c2[2][2] = {{0, 0}, {0, 0}};
    #pragma unroll
            for (int a = 0; a < 2; ++a)
    #pragma unroll
                for (int b = 0; b < 2; ++b)
    #pragma unroll
                    for (int k = 0; k < 3; ++k) c2[a][b] += half[a][k] * Tm[k][b];
            const float ca = c2[0][0] + 0.3f, cb2 = c2[0][1], cc = c2[1][1] + 0.3f;

            // Pixel centre.
            const float z_inv = 1.f / (tz + 1e-6f);
            const float px = cv.fx * tx * z_inv + cv.cx, py = cv.fy * ty * z_inv + cv.cy;

            // Radius from the larger eigenvalue, 3 sigma, rounded up.
// a c - b^2 as the reference's build fuses it (checked bit for bit on 6M splats); spelled out like Sigma above
            const float det = __fmaf_rn(ca, cc, -__fmul_rn(cb2, cb2));
            const float mid = 0.5f * (ca + cc);
            const float diff = mid * mid - det;
            const float lambda1 = mid + sqrtf(max(0.1f, diff));
            const float lambda2 = mid - sqrtf(max(0.1f, diff));
            radius = ceilf(3 * sqrtf(max(lambda1, lambda2))) * (det > 1e-6f && in_frustum > 0);

            // Tile rectangle (float -> int conversion truncates toward zero) and its size.
            const float cxt = px / kTile, cyt = py / kTile, dt = radius / (float)kTile;
            int x0 = min(max(0, (int)(cxt - dt)), cv.tiles_x), x1 = min(max(0, (int)(cxt + dt + 1)), cv.tiles_x);
            int y0 = min(max(0, (int)(cyt - dt)), cv.tiles_y), y1 = min(max(0, (int)(cyt + dt + 1)), cv.tiles_y);
            if (cv.tight_tiles) {
                // A pixel blends the splat only if opacity * exp(-q) >= 1/255, q = 0.5 d^T conic d, i.e. inside the
                // ellipse q <= ln(255 opacity).  Its bounding box has half-widths sqrt(2 tau cov_xx), sqrt(2 tau cov_yy)
                // with cov the dilated 2-D covariance; tau carries the margin of the blend kernels' cull, the factor
                // (det + 1e-6) / det undoes the shrink the conic gets from its regularised inverse, and half a pixel
                // is added on every side, so the box can only be too large.  Tile t holds pixel centres
                // 16 t + 0.5 .. 16 t + 15.5; tiles outside the box are dropped from the rectangle.
                const float tau = __logf(255.0f * opacity) + 0.02f;
                if (!(tau > 0.f)) {
                    x1 = x0; y1 = y0;   // too faint to reach 1/255 anywhere
                } else if (det > 1e-6f) {
                    const float grow = 2.0f * tau * (1.0f + 1e-6f / det) * 1.001f;
                    const float wx = sqrtf(grow * ca) + 0.5f, wy = sqrtf(grow * cc) + 0.5f;
                    const float fx0 = floorf((px - wx - 15.5f) * (1.0f / kTile)) + 1.0f, fx1 = floorf((px + wx - 0.5f) * (1.0f / kTile)) + 1.0f;
                    const float fy0 = floorf((py - wy - 15.5f) * (1.0f / kTile)) + 1.0f, fy1 = floorf((py + wy - 0.5f) * (1.0f / kTile)) + 1.0f;
                    // compare as floats first: a huge splat must not overflow the conversion
                    if (fx0 > (float)x0) x0 = min((int)fx0, x1);
                    if (fx1 < (float)x1) x1 = max((int)fx1, x0);
                    if (fy0 > (float)y0) y0 = min((int)fy0, y1);
                    if (fy1 < (float)y1) y1 = max((int)fy1, y0);
                }
            }
            // A centre behind the camera can pass the frustum test (w < 0 flips both signs).  The reference
            // still reports its radius but, because the negative depth bits spill over the tile id of its
            // keys, never draws it; here it simply gets no pairs.
            // a view rendered in bands of tile rows: only the band's part of the rectangle gets pairs
            y0 = min(max(y0, cv.band_y0), cv.band_y1); y1 = max(min(y1, cv.band_y1), y0);
            count = (x1 - x0) * (y1 - y0) * (radius > 0 && tz > 0.f);
            // Corner marks of the tile rectangle (+1, -1, -1, +1) in a (tiles_y + 1) x (tiles_x + 1) grid: its 2-D
            // prefix sum is the number of (tile, splat) pairs per tile, from which tile ranges and the tile sort's
            // digit counts follow without a pass over the pairs.  Fire-and-forget reductions, hidden behind the
            // kernel's memory traffic.
            if (pv.tile_marks[view] && count > 0 && !(cv.drop_last && i == n - 1)) {
                const int stride = cv.tiles_x + 1;
                int* m = pv.tile_marks[view] + (size_t)(blockIdx.x % kMarkCopies) * marks_copy_ints;
                atomicAdd(m + y0 * stride + x0, 1);
                atomicAdd(m + y0 * stride + x1, -1);
                atomicAdd(m + y1 * stride + x0, -1);
                atomicAdd(m + y1 * stride + x1, 1);
            }

            // Conic = inverse of the dilated 2-D covariance.
            const float det_inv = 1.0f / (det + 1e-6f);
            q0 = make_float4(px, py, cc * det_inv, -cb2 * det_inv);
            q1 = make_float4(ca * det_inv, opacity, cr, cg);
            q2 = make_float4(cb, tz, __uint_as_float(pack_rect(x0, x1)), __uint_as_float(pack_rect(y0, y1)));

            pv.radii[view][i] = radius;
            pv.tiles[view][i] = count;
            pv.depth_keys[view][i] = ((u64)__float_as_uint(tz) << 32) | (u32)i;
        }

        // Records leave through shared memory so that global stores are contiguous 16-byte lanes.
        s_rec[tid * 3] = q0; s_rec[tid * 3 + 1] = q1; s_rec[tid * 3 + 2] = q2;
        __syncthreads();
        float4* grec = pv.records[view] + (size_t)base * 3;
        for (int k = tid; k < cnt * 3; k += kThreads) grec[k] = s_rec[k];
        __syncthreads();   // s_rec is reused by the next view
    }

    if (cov3d && !cov3d_precomp) {   // the covariance does not depend on the view: written once
        float* s_cov = reinterpret_cast<float*>(s_rec);  // [256][6]
#pragma unroll
        for (int k = 0; k < 6; ++k) s_cov[tid * 6 + k] = S[k];
        __syncthreads();
        float* gcov = cov3d + (size_t)base * 6;
        for (int k = tid; k < cnt * 6; k += kThreads) gcov[k] = s_cov[k];
    }
    if (direct) {   // block-uniform: the copies this block asked for must have landed before it retires
        bool ok = false;
        for (u32 poll = 0; poll < kCopyWaitPolls && !ok; ++poll) {
            ok = mbar_try_wait(&s_bar, 0);
            if (!ok) __nanosleep(64);
        }
        if (!ok && tid == 0) atomicExch(device_status, DSB_ERR_DEVICE_WAIT_EXPIRED);
    }
}

}  // namespace

// views: `count` cameras with their output buffers (count <= DSB_MAX_BATCH_VIEWS); cov3d is written once.
int launch_preprocess_views(const CamParams* cps, int count, int n, const float* means, const float* shs,
                            const float* colors_precomp, const float* opac, const float* scales, const float* rots,
                            const float* cov3d_precomp, float* const* records, int32_t* const* radii,
                            int32_t* const* tiles, float* cov3d, u64* const* depth_keys, int* const* tile_marks,
                            cudaStream_t s) {
    if (n == 0 || count == 0) return DSB_OK;
    DSB_REQUIRE(count > 0 && count <= DSB_MAX_BATCH_VIEWS, "preprocess: %d views in one call (at most %d)", count,
                DSB_MAX_BATCH_VIEWS);
    DSB_REQUIRE(means && opac && records && radii && tiles && depth_keys, "preprocess: null required pointer");
    DSB_REQUIRE(colors_precomp || shs, "preprocess: need shs or colors_precomp");
    DSB_REQUIRE(cov3d_precomp || (scales && rots), "preprocess: need scales and rotations, or cov3d_precomp");
    DSB_REQUIRE(!rots || ((uintptr_t)rots & 15) == 0, "preprocess: rotations must be 16-byte aligned");
    const CamParams& cp = cps[0];
    PreViews pv;
    pv.count = count;
    for (int v = 0; v < count; ++v) {
        DSB_REQUIRE(records[v] && radii[v] && tiles[v] && depth_keys[v], "preprocess: null output pointer for view %d", v);
        DSB_REQUIRE(((uintptr_t)records[v] & 15) == 0, "preprocess: records must be 16-byte aligned");
        DSB_REQUIRE(cps[v].max_coeff == cp.max_coeff && cps[v].sh_degree == cp.sh_degree &&
                        cps[v].scale_modifier == cp.scale_modifier,
                    "preprocess: the views of one call must share SH degree and scale modifier");
        DSB_REQUIRE(cps[v].H == cp.H && cps[v].W == cp.W, "preprocess: the views of one call must share the image size");
        pv.cam[v] = cps[v];
        pv.records[v] = reinterpret_cast<float4*>(records[v]);
        pv.radii[v] = radii[v];
        pv.tiles[v] = tiles[v];
        pv.depth_keys[v] = depth_keys[v];
        pv.tile_marks[v] = tile_marks ? tile_marks[v] : nullptr;
    }
    const int sh_vec4 = shs && cp.max_coeff == 16 && ((uintptr_t)shs & 15) == 0;
    // bulk-copy staging needs every streamed input 16-byte aligned and the default input form
#ifndef DSB_PRE_BULK
#define DSB_PRE_BULK 1   // 0: stage with ordinary 16-byte loads (kept for measurements)
#endif
    const int use_bulk = DSB_PRE_BULK && sh_vec4 && !colors_precomp && !cov3d_precomp && scales && ((uintptr_t)means & 15) == 0 &&
                         ((uintptr_t)scales & 15) == 0;
    // dynamic shared memory: the padded SH rows
    const size_t dyn = sh_vec4 ? (size_t)kThreads * kShRow4 * 16 : (size_t)kThreads * ((3 * cp.max_coeff) | 1) * 4;
    DSB_REQUIRE(dyn <= 64 * 1024, "preprocess: SH layout too large for shared memory");
    // the attribute belongs to the current device's context, so it is set at every launch rather than cached
    DSB_CUDA_CHECK(cudaFuncSetAttribute(preprocess_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
    const int blocks = (n + kThreads - 1) / kThreads;
    int* device_status = nullptr;
    {
        const int rc = device_status_address(&device_status);
        if (rc != DSB_OK) return rc;
    }
    preprocess_kernel<<<blocks, kThreads, dyn, s>>>(pv, n, means, shs, colors_precomp, opac, scales, rots, cov3d_precomp, cov3d,
                                                   sh_vec4, use_bulk, (int)tile_marks_copy_ints(cp.H, cp.W), copy_wait_polls(),
                                                   device_status);
    DSB_LAUNCH_CHECK();
    return DSB_OK;
}

int launch_preprocess(const CamParams& cp, int n, const float* means, const float* shs, const float* colors_precomp,
                      const float* opac, const float* scales, const float* rots, const float* cov3d_precomp,
                      float* records, int32_t* radii, int32_t* tiles, float* cov3d, u64* depth_keys, int* tile_marks,
                      cudaStream_t s) {
    return launch_preprocess_views(&cp, 1, n, means, shs, colors_precomp, opac, scales, rots, cov3d_precomp, &records, &radii,
                                   &tiles, cov3d, &depth_keys, tile_marks ? &tile_marks : nullptr, s);
}

}  // namespace dsb
