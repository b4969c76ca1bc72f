// CPU oracle for the ds-splat Gaussian rasterizer hot path (forward + backward).
//
// TEST INFRASTRUCTURE ONLY.  This file is a plain C++17/OpenMP restatement of the arithmetic the
// reference performs in its CUDA kernels.  It exists so that the sm_100a kernels of this repository
// can be checked stage by stage on identical inputs and so that a CPU baseline can be timed beside
// them.  Nothing in the product path links, imports or executes it.
//
// Parity status: the tile-range stage is pinned by the reference's two known-answer tests
// (tests/rasterizer_test.cpp:66-110).  Every other stage has no golden vector in the reference
// ("parity unpinned" by reference tests); those stages are pinned instead by running the reference's
// own CUDA kernels (oracle/_ref, built by oracle/Makefile) on a B200 against this file.
//
// Each function cites the reference file:line whose arithmetic it follows.  fp32 throughout, with
// the reference's operation order; libm expf/sqrtf replace the GPU's approximate intrinsics, so
// results agree with a --use_fast_math GPU build to a few ulp, not bit for bit.
//
// Build: g++ -O3 -march=native -fopenmp -shared -fPIC gs_oracle.cpp -o _build/libgs_oracle.so

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#include <parallel/algorithm>
#endif

namespace {

constexpr int kTile = 16;  // cpp/rasterizer_kernels.cuh:6

struct Cam {
    float view[16];   // row-major world->camera [R|t] (after the Python-side transpose, ds_splat/rasterizer.py:147)
    float proj[16];   // row-major full projection P*V (ds_splat/rasterizer.py:148)
    float campos[3];
    float tanfovx, tanfovy, scale_modifier;
    float bg[3];
    int H, W, sh_degree, max_sh_degree;
};

// GPU float->int conversion saturates and maps NaN to 0; plain C++ casts are undefined there.
inline int f2i_trunc(float v) {
    if (!(v == v)) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int)v;
}

inline int tiles_x(const Cam& c) { return (c.W + kTile - 1) / kTile; }
inline int tiles_y(const Cam& c) { return (c.H + kTile - 1) / kTile; }

// cpp/rasterizer_kernels.cu:615-659
inline void cov3d_from_scale_rot(const float* s, const float* q, float mod, float out[6]) {
    float r = q[0], x = q[1], y = q[2], z = q[3];
    const float inv = 1.0f / std::sqrt(r * r + x * x + y * y + z * z);
    r *= inv; x *= inv; y *= inv; z *= inv;
    const float sx = s[0] * mod, sy = s[1] * mod, sz = s[2] * mod;
    const float r00 = 1.0f - 2.0f * (y * y + z * z), r01 = 2.0f * (x * y - r * z), r02 = 2.0f * (x * z + r * y);
    const float r10 = 2.0f * (x * y + r * z), r11 = 1.0f - 2.0f * (x * x + z * z), r12 = 2.0f * (y * z - r * x);
    const float r20 = 2.0f * (x * z - r * y), r21 = 2.0f * (y * z + r * x), r22 = 1.0f - 2.0f * (x * x + y * y);
    const float m00 = sx * r00, m01 = sy * r01, m02 = sz * r02;
    const float m10 = sx * r10, m11 = sy * r11, m12 = sz * r12;
    const float m20 = sx * r20, m21 = sy * r21, m22 = sz * r22;
    out[0] = m00 * m00 + m01 * m01 + m02 * m02;
    out[1] = m00 * m10 + m01 * m11 + m02 * m12;
    out[2] = m00 * m20 + m01 * m21 + m02 * m22;
    out[3] = m10 * m10 + m11 * m11 + m12 * m12;
    out[4] = m10 * m20 + m11 * m21 + m12 * m22;
    out[5] = m20 * m20 + m21 * m21 + m22 * m22;
}

// Real spherical-harmonic basis values for a unit direction, degrees 0..3, in the coefficient order
// and with the signs of cpp/rasterizer_kernels.cu:433-554 (forward) and cpp/gsplat/sh.cuh:95-160 (backward).
inline void sh_basis(int degree, float x, float y, float z, float b[16]) {
    for (int k = 0; k < 16; ++k) b[k] = 0.0f;
    b[0] = 0.28209479177387814f;
    if (degree < 1) return;
    const float C1 = 0.4886025119029199f;
    b[1] = -C1 * y; b[2] = C1 * z; b[3] = -C1 * x;
    if (degree < 2) return;
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
    b[4] = 1.0925484305920792f * xy;
    b[5] = -1.0925484305920792f * yz;
    b[6] = 0.31539156525252005f * (2.0f * zz - xx - yy);
    b[7] = -1.0925484305920792f * xz;
    b[8] = 0.5462742152960396f * (xx - yy);
    if (degree < 3) return;
    b[9] = -0.5900435899266435f * y * (3.0f * xx - yy);
    b[10] = 2.890611442640554f * xy * z;
    b[11] = -0.4570457994644658f * y * (4.0f * zz - xx - yy);
    b[12] = 0.3731763325901154f * z * (2.0f * zz - 3.0f * xx - 3.0f * yy);
    b[13] = -0.4570457994644658f * x * (4.0f * zz - xx - yy);
    b[14] = 1.445305721320277f * z * (xx - yy);
    b[15] = -0.5900435899266435f * x * (xx - 3.0f * yy);
}

// Tile rectangle of a splat: cpp/rasterizer_kernels.cu:233-250 and :286-292.
inline void tile_rect(const Cam& c, float px, float py, int radius, int r[4]) {
    const float cx = px / kTile, cy = py / kTile, d = radius / (float)kTile;
    const int tw = tiles_x(c), th = tiles_y(c);
    r[0] = std::min(std::max(0, f2i_trunc(cx - d)), tw);
    r[1] = std::min(std::max(0, f2i_trunc(cx + d + 1)), tw);
    r[2] = std::min(std::max(0, f2i_trunc(cy - d)), th);
    r[3] = std::min(std::max(0, f2i_trunc(cy + d + 1)), th);
}

}  // namespace

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Number of hardware threads the host offers (what omp would use if nothing capped it).
int orc_num_procs() {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

// Thread count of all following stages; n <= 0 means every hardware thread.  Launchers such as torchrun
// export OMP_NUM_THREADS=1 to their workers, which would otherwise turn the timed CPU baseline into a
// one-core run without saying so.
void orc_set_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n > 0 ? n : omp_get_num_procs());
#else
    (void)n;
#endif
}

// Stage (a).  cpp/rasterizer_kernels.cu:57-161 with helpers :7-55, :163-250, :325-337, :433-659.
// Outputs per splat: xy (pixel mean), depth (view-space z), conic, rgb, radius, tile count, tile rect
// (x0,x1,y0,y1) and the 6-float 3-D covariance.
void orc_preprocess(const Cam* cam, int N, const float* means, const float* shs, const float* colors_precomp,
                    const float* opacities, const float* scales, const float* rots, const float* cov3d_precomp,
                    float* xy, float* depth, float* conic, float* rgb, int32_t* radii, int32_t* tiles,
                    int32_t* rect, float* cov3d_out) {
    const Cam& c = *cam;
    const float fx = c.W / (2 * c.tanfovx), fy = c.H / (2 * c.tanfovy);  // cpp/rasterizer_torch.cu:144-145
    const float cx = c.W / 2.0f, cy = c.H / 2.0f;
    const int max_coeff = (c.max_sh_degree + 1) * (c.max_sh_degree + 1);
    const float* V = c.view;
    const float* P = c.proj;
    (void)opacities;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; ++i) {
        float S[6];
        if (cov3d_precomp) std::memcpy(S, cov3d_precomp + 6 * (size_t)i, sizeof(S));
        else cov3d_from_scale_rot(scales + 3 * (size_t)i, rots + 4 * (size_t)i, c.scale_modifier, S);
        std::memcpy(cov3d_out + 6 * (size_t)i, S, sizeof(S));
        const float mx = means[3 * (size_t)i], my = means[3 * (size_t)i + 1], mz = means[3 * (size_t)i + 2];

        // colour: :26-42, :556-613
        float col[3];
        if (colors_precomp) {
            for (int k = 0; k < 3; ++k) col[k] = colors_precomp[3 * (size_t)i + k];
        } else if (c.sh_degree > 3) {
            col[0] = col[1] = col[2] = 0.0f;
        } else {
            float b[16];
            float dx = mx - c.campos[0], dy = my - c.campos[1], dz = mz - c.campos[2];
            const float inv = 1.0f / std::sqrt(dx * dx + dy * dy + dz * dz);
            dx *= inv; dy *= inv; dz *= inv;
            sh_basis(c.sh_degree, dx, dy, dz, b);
            const float* f = shs + (size_t)i * 3 * max_coeff;
            const int nb = (c.sh_degree + 1) * (c.sh_degree + 1);
            for (int ch = 0; ch < 3; ++ch) {
                float acc = 0.0f;
                for (int k = 0; k < nb; ++k) acc += b[k] * f[3 * k + ch];
                col[ch] = std::max(acc + 0.5f, 0.0f);
            }
        }
        // frustum mask: :7-24
        const float inv_w = 1.0f / (P[12] * mx + P[13] * my + P[14] * mz + P[15]);
        const float nx = inv_w * (P[0] * mx + P[1] * my + P[2] * mz + P[3]);
        const float ny = inv_w * (P[4] * mx + P[5] * my + P[6] * mz + P[7]);
        const float nz = inv_w * (P[8] * mx + P[9] * my + P[10] * mz + P[11]);
        const int mask = nx > -1.0f && nx < 1.0f && ny > -1.0f && ny < 1.0f && nz > 0.1f;
        // view-space point: :325-330
        const float tx = V[0] * mx + V[1] * my + V[2] * mz + V[3];
        const float ty = V[4] * mx + V[5] * my + V[6] * mz + V[7];
        const float tz = V[8] * mx + V[9] * my + V[10] * mz + V[11];
        // EWA 2-D covariance: :174-231
        const float limx = 1.3f * c.tanfovx, limy = 1.3f * c.tanfovy;
        const float t0 = std::min(limx, std::max(-limx, tx / tz)) * tz;
        const float t1 = std::min(limy, std::max(-limy, ty / tz)) * tz;
        const float J[3][3] = {{fx / tz, 0, -(fx * t0) / (tz * tz)}, {0, fy / tz, -(fy * t1) / (tz * tz)}, {0, 0, 0}};
        const float Wm[3][3] = {{V[0], V[4], V[8]}, {V[1], V[5], V[9]}, {V[2], V[6], V[10]}};
        float T[3][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
        for (int a = 0; a < 3; ++a)
            for (int b2 = 0; b2 < 3; ++b2)
                for (int k = 0; k < 3; ++k) T[a][b2] += Wm[a][k] * J[b2][k];
        const float Vr[3][3] = {{S[0], S[1], S[2]}, {S[1], S[3], S[4]}, {S[2], S[4], S[5]}};
        float tmp[3][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
        for (int a = 0; a < 3; ++a)
            for (int b2 = 0; b2 < 3; ++b2)
                for (int k = 0; k < 3; ++k) tmp[a][b2] += T[k][a] * Vr[k][b2];
        float cov[2][2] = {{0, 0}, {0, 0}};
        for (int a = 0; a < 2; ++a)
            for (int b2 = 0; b2 < 2; ++b2)
                for (int k = 0; k < 3; ++k) cov[a][b2] += tmp[a][k] * T[k][b2];
        const float ca = cov[0][0] + 0.3f, cb = cov[0][1], cc = cov[1][1] + 0.3f;
        // pixel mean: :332-337
        const float zinv = 1.0f / (tz + 1e-6f);
        const float px = fx * tx * zinv + cx, py = fy * ty * zinv + cy;
        // radius: :163-172
        const float det = ca * cc - cb * cb;
        const float mid = 0.5f * (ca + cc);
        const float diff = mid * mid - det;
        const float l1 = mid + std::sqrt(std::max(0.1f, diff)), l2 = mid - std::sqrt(std::max(0.1f, diff));
        const int radius = (int)(std::ceil(3 * std::sqrt(std::max(l1, l2))) * (float)(det > 1e-6f && mask > 0));
        // tile rect and count: :233-250
        int r[4];
        tile_rect(c, px, py, radius, r);
        const int count = (r[1] - r[0]) * (r[3] - r[2]) * (radius > 0);
        // conic: :49-55
        const float dinv = 1.0f / (det + 1e-6f);
        xy[2 * (size_t)i] = px; xy[2 * (size_t)i + 1] = py;
        depth[i] = tz;
        conic[3 * (size_t)i] = cc * dinv; conic[3 * (size_t)i + 1] = -cb * dinv; conic[3 * (size_t)i + 2] = ca * dinv;
        rgb[3 * (size_t)i] = col[0]; rgb[3 * (size_t)i + 1] = col[1]; rgb[3 * (size_t)i + 2] = col[2];
        radii[i] = radius; tiles[i] = count;
        for (int k = 0; k < 4; ++k) rect[4 * (size_t)i + k] = r[k];
    }
}

// Number of (tile, splat) pairs.  The reference takes the EXCLUSIVE prefix of the last splat as the
// total (cpp/rasterizer_torch.cu:97-104), so the last splat never emits a pair; drop_last=1 keeps that.
int64_t orc_count_pairs(int N, const int32_t* tiles, int drop_last) {
    int64_t k = 0;
    const int n = drop_last ? N - 1 : N;
    for (int i = 0; i < n; ++i) k += tiles[i];
    return k;
}

// Stage (b).  cpp/rasterizer_kernels.cu:252-306: key = (tile << 32) | sign-extended depth bits,
// value = splat id, rectangle scanned row-major, splats in ascending id.
void orc_duplicate_keys(const Cam* cam, int N, const float* xy, const float* depth, const int32_t* radii,
                        const int32_t* tiles, int drop_last, int64_t* keys, int32_t* ids) {
    const Cam& c = *cam;
    const int tw = tiles_x(c);
    const int n = drop_last ? N - 1 : N;
    int64_t pos = 0;
    for (int i = 0; i < n; ++i) {
        if (tiles[i] <= 0) continue;
        int r[4];
        tile_rect(c, xy[2 * (size_t)i], xy[2 * (size_t)i + 1], radii[i], r);
        int32_t bits;
        std::memcpy(&bits, depth + i, 4);
        const int64_t d = (int64_t)bits;
        for (int ty = r[2]; ty < r[3]; ++ty)
            for (int tx = r[0]; tx < r[1]; ++tx) {
                const int64_t tile = (int64_t)ty * tw + tx;
                keys[pos] = (tile << 32) | d;
                ids[pos] = i;
                ++pos;
            }
    }
}

// Stage (c).  cpp/rasterizer_torch.cu:70-76: ascending signed 64-bit keys; an LSD radix sort is
// stable, so equal keys keep their emission order.
void orc_sort_pairs(int64_t K, int64_t* keys, int32_t* ids) {
    std::vector<int64_t> order(K);
    std::iota(order.begin(), order.end(), (int64_t)0);
#ifdef _OPENMP
    __gnu_parallel::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return keys[a] < keys[b]; });
#else
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return keys[a] < keys[b]; });
#endif
    std::vector<int64_t> k2(K);
    std::vector<int32_t> v2(K);
    for (int64_t i = 0; i < K; ++i) { k2[i] = keys[order[i]]; v2[i] = ids[order[i]]; }
    std::memcpy(keys, k2.data(), K * sizeof(int64_t));
    std::memcpy(ids, v2.data(), K * sizeof(int32_t));
}

// Stage (d).  cpp/rasterizer_torch.cu:23-42 + cpp/rasterizer_kernels.cu:308-323: mark the end of each
// tile's run at [tile+1], put K in the last slot, then a running maximum fills empty tiles.
void orc_tile_ranges(int64_t K, const int64_t* keys, int H, int W, int32_t* out) {
    const int T = ((W + kTile - 1) / kTile) * ((H + kTile - 1) / kTile);
    for (int t = 0; t <= T; ++t) out[t] = 0;
    out[T] = (int32_t)K;
    for (int64_t i = 0; i + 1 < K; ++i) {
        const int32_t a = (int32_t)(keys[i] >> 32), b = (int32_t)(keys[i + 1] >> 32);
        if (a != b && a + 1 >= 0 && a + 1 <= T) out[a + 1] = (int32_t)(i + 1);
    }
    for (int t = 1; t <= T; ++t) out[t] = std::max(out[t], out[t - 1]);
}

// Stage (e).  cpp/rasterizer_kernels.cu:341-431.  Per pixel, front to back over its tile's run.
// pairs_out[0] = (pixel, splat) pairs evaluated, each pixel stopping on its own.
// Optional depth map (no reference counterpart: the reference returns colour only): when z (per-splat
// view-space depth) and depth_out are given, depth_out = sum_i z_i alpha_i T_i, i.e. z blended exactly
// like a fourth colour channel.
void orc_blend_forward(const Cam* cam, const int32_t* ids, const int32_t* ranges, const float* xy,
                       const float* conic, const float* rgb, const float* opac, float* image, float* final_T,
                       int32_t* final_idx, int64_t* pairs_out, const float* z, float* depth_out) {
    const Cam& c = *cam;
    const int tw = tiles_x(c), th = tiles_y(c);
    int64_t pairs = 0;
#pragma omp parallel for schedule(dynamic, 4) reduction(+ : pairs)
    for (int tile = 0; tile < tw * th; ++tile) {
        const int s = ranges[tile], e = ranges[tile + 1];
        const int tx0 = (tile % tw) * kTile, ty0 = (tile / tw) * kTile;
        for (int ly = 0; ly < kTile; ++ly)
            for (int lx = 0; lx < kTile; ++lx) {
                const int x = tx0 + lx, y = ty0 + ly;
                if (x >= c.W || y >= c.H) continue;
                float T = 1.0f, C0 = 0, C1 = 0, C2 = 0, D = 0;
                int last = 0;
                for (int p = s; p < e; ++p) {
                    ++pairs;
                    const int g = ids[p];
                    const float dx = x + 0.5f - xy[2 * (size_t)g], dy = y + 0.5f - xy[2 * (size_t)g + 1];
                    const float* q = conic + 3 * (size_t)g;
                    const float power = -0.5f * (q[0] * dx * dx + q[2] * dy * dy) - q[1] * dx * dy;
                    const float alpha = std::min(0.999f, opac[g] * std::exp(power));
                    if (power >= 0.0f || alpha < 1.0f / 255.0f) continue;
                    const float Tn = (1.0f - alpha) * T;
                    if (!(Tn >= 0.0001f)) break;
                    const float w = alpha * T;
                    C0 += w * rgb[3 * (size_t)g]; C1 += w * rgb[3 * (size_t)g + 1]; C2 += w * rgb[3 * (size_t)g + 2];
                    if (z) D += w * z[g];
                    T = Tn;
                    last = p;
                }
                const size_t pix = (size_t)y * c.W + x;
                image[3 * pix] = C0; image[3 * pix + 1] = C1; image[3 * pix + 2] = C2;  // no background: kernel has no bg argument
                final_T[pix] = T;
                final_idx[pix] = last;
                if (z && depth_out) depth_out[pix] = D;
            }
    }
    if (pairs_out) pairs_out[0] = pairs;
}

// Stage (f1).  cpp/gsplat/backward.cu:25-202.  Per pixel, back to front from final_idx; per-splat sums
// are accumulated in double (the GPU's atomic order is not deterministic, so no fp32 order exists to follow).
// Optional depth gradient (no reference counterpart): with z, v_depth_img (dL/d depth map) and v_z given,
// z takes part as a fourth colour channel without background -- its term joins v_alpha and
// v_z[g] = sum over pixels of alpha T v_depth, the quantity cpp/gsplat/backward.cu:253-259 expects as v_depth.
void orc_blend_backward(const Cam* cam, int N, const int32_t* ids, const int32_t* ranges, const float* xy,
                        const float* conic, const float* rgb, const float* opac, const float* final_T,
                        const int32_t* final_idx, const float* v_image, float* v_xy, float* v_conic, float* v_rgb,
                        float* v_opac, int64_t* pairs_out, const float* z, const float* v_depth_img, float* v_z) {
    const Cam& c = *cam;
    const int tw = tiles_x(c), th = tiles_y(c);
    const bool with_depth = z && v_depth_img && v_z;
    constexpr int kA = 10;  // 9 reference sums + v_z
    std::vector<double> acc((size_t)N * kA, 0.0);
    int64_t pairs = 0;
#pragma omp parallel reduction(+ : pairs)
    {
        std::vector<double> loc;
#pragma omp for schedule(dynamic, 4)
        for (int tile = 0; tile < tw * th; ++tile) {
            const int s = ranges[tile], e = ranges[tile + 1];
            if (e <= s) continue;
            loc.assign((size_t)(e - s) * kA, 0.0);
            const int tx0 = (tile % tw) * kTile, ty0 = (tile / tw) * kTile;
            for (int ly = 0; ly < kTile; ++ly)
                for (int lx = 0; lx < kTile; ++lx) {
                    const int x = tx0 + lx, y = ty0 + ly;
                    if (x >= c.W || y >= c.H) continue;
                    const size_t pix = (size_t)y * c.W + x;
                    const float px = (float)x + 0.5f, py = (float)y + 0.5f;
                    const float Tf = final_T[pix];
                    float T = Tf, b0 = 0, b1 = 0, b2 = 0, bz = 0;
                    const float vo0 = v_image[3 * pix], vo1 = v_image[3 * pix + 1], vo2 = v_image[3 * pix + 2];
                    const float vod = with_depth ? v_depth_img[pix] : 0.0f;
                    const int fin = final_idx[pix];
                    for (int p = std::min(e - 1, fin); p >= s; --p) {
                        ++pairs;
                        const int g = ids[p];
                        const float* q = conic + 3 * (size_t)g;
                        const float dx = xy[2 * (size_t)g] - px, dy = xy[2 * (size_t)g + 1] - py;
                        const float sigma = 0.5f * (q[0] * dx * dx + q[2] * dy * dy) + q[1] * dx * dy;
                        const float vis = std::exp(-sigma);
                        const float o = opac[g];
                        const float alpha = std::min(0.99f, o * vis);
                        if (sigma < 0.0f || alpha < 1.0f / 255.0f) continue;
                        const float ra = 1.0f / (1.0f - alpha);
                        T *= ra;
                        const float fac = alpha * T;
                        const float* col = rgb + 3 * (size_t)g;
                        float va = 0.0f;
                        va += (col[0] * T - b0 * ra) * vo0;
                        va += (col[1] * T - b1 * ra) * vo1;
                        va += (col[2] * T - b2 * ra) * vo2;
                        va += -Tf * ra * c.bg[0] * vo0;
                        va += -Tf * ra * c.bg[1] * vo1;
                        va += -Tf * ra * c.bg[2] * vo2;
                        if (with_depth) {
                            va += (z[g] * T - bz * ra) * vod;
                            bz += z[g] * fac;
                        }
                        b0 += col[0] * fac; b1 += col[1] * fac; b2 += col[2] * fac;
                        const float vs = -o * vis * va;
                        double* a = loc.data() + (size_t)(p - s) * kA;
                        a[0] += vs * (q[0] * dx + q[1] * dy);
                        a[1] += vs * (q[1] * dx + q[2] * dy);
                        a[2] += 0.5f * vs * dx * dx;
                        a[3] += vs * dx * dy;
                        a[4] += 0.5f * vs * dy * dy;
                        a[5] += fac * vo0; a[6] += fac * vo1; a[7] += fac * vo2;
                        a[8] += vis * va;
                        if (with_depth) a[9] += fac * vod;
                    }
                }
            for (int p = s; p < e; ++p) {
                const double* a = loc.data() + (size_t)(p - s) * kA;
                double* d = acc.data() + (size_t)ids[p] * kA;
                for (int k = 0; k < kA; ++k)
                    if (a[k] != 0.0) {
#pragma omp atomic
                        d[k] += a[k];
                    }
            }
        }
    }
    for (int i = 0; i < N; ++i) {
        const double* a = acc.data() + (size_t)i * kA;
        if (with_depth) v_z[i] = (float)a[9];
        v_xy[2 * (size_t)i] = (float)a[0]; v_xy[2 * (size_t)i + 1] = (float)a[1];
        v_conic[3 * (size_t)i] = (float)a[2]; v_conic[3 * (size_t)i + 1] = (float)a[3]; v_conic[3 * (size_t)i + 2] = (float)a[4];
        v_rgb[3 * (size_t)i] = (float)a[5]; v_rgb[3 * (size_t)i + 1] = (float)a[6]; v_rgb[3 * (size_t)i + 2] = (float)a[7];
        v_opac[i] = (float)a[8];
    }
    if (pairs_out) pairs_out[0] = pairs;
}

// Stage (f2), colour part.  cpp/gsplat/sh.cuh:95-203 driven by cpp/rasterizer_torch.cu:291-295:
// v_sh[k][c] = basis_k(normalise(mean - campos)) * v_rgb[c] for the active bands, zero elsewhere.
void orc_sh_backward(const Cam* cam, int N, int num_bases, const float* means, const float* v_rgb, float* v_sh) {
    const Cam& c = *cam;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; ++i) {
        float* out = v_sh + (size_t)i * num_bases * 3;
        for (int k = 0; k < num_bases * 3; ++k) out[k] = 0.0f;
        float dx = means[3 * (size_t)i] - c.campos[0], dy = means[3 * (size_t)i + 1] - c.campos[1],
              dz = means[3 * (size_t)i + 2] - c.campos[2];
        float b[16];
        if (c.sh_degree >= 1) {
            const float n = std::sqrt(dx * dx + dy * dy + dz * dz);
            dx /= n; dy /= n; dz /= n;
        }
        sh_basis(std::min(c.sh_degree, 3), dx, dy, dz, b);
        const int nb = std::min((c.sh_degree + 1) * (c.sh_degree + 1), num_bases);
        for (int k = 0; k < nb; ++k)
            for (int ch = 0; ch < 3; ++ch) out[3 * k + ch] = b[k] * v_rgb[3 * (size_t)i + ch];
    }
}

// Stage (f2), geometry part.  cpp/gsplat/backward.cu:216-393 with cpp/gsplat/helpers.cuh:68-79,97-147,
// 149-220; focal lengths recomputed the way cpp/rasterizer_torch.cu:78-81,297-298 does.
// Only splats with radius > 0 get gradients; every output row of the others is zero.
void orc_project_backward(const Cam* cam, int N, const float* means, const float* scales, const float* rots,
                          const float* conic, const float* cov3d, const int32_t* radii, const float* v_xy,
                          const float* v_conic, float* v_mean, float* v_scale, float* v_rot, float* v_cov3d,
                          const float* v_z) {
    const Cam& c = *cam;
    const float fx = c.W / (2.0f * std::tan((2 * std::atan(c.tanfovx)) / 2.0f));
    const float fy = c.H / (2.0f * std::tan((2 * std::atan(c.tanfovy)) / 2.0f));
    const float* V = c.view;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; ++i) {
        float* vm = v_mean + 3 * (size_t)i;
        float* vsc = v_scale + 3 * (size_t)i;
        float* vq = v_rot + 4 * (size_t)i;
        float* vc3 = v_cov3d + 6 * (size_t)i;
        vm[0] = vm[1] = vm[2] = 0; vsc[0] = vsc[1] = vsc[2] = 0; vq[0] = vq[1] = vq[2] = vq[3] = 0;
        for (int k = 0; k < 6; ++k) vc3[k] = 0;
        if (radii[i] <= 0) continue;
        const float mx = means[3 * (size_t)i], my = means[3 * (size_t)i + 1], mz = means[3 * (size_t)i + 2];
        const float tx = V[0] * mx + V[1] * my + V[2] * mz + V[3];
        const float ty = V[4] * mx + V[5] * my + V[6] * mz + V[7];
        const float tz = V[8] * mx + V[9] * my + V[10] * mz + V[11];
        // pixel-mean VJP: helpers.cuh:138-147, then R^T: :97-104
        {
            const float rw = 1.0f / (tz + 1e-6f);
            const float vpx = fx * v_xy[2 * (size_t)i], vpy = fy * v_xy[2 * (size_t)i + 1];
            const float vv[3] = {vpx * rw, vpy * rw, -(vpx * tx + vpy * ty) * rw * rw};
            vm[0] = V[0] * vv[0] + V[4] * vv[1] + V[8] * vv[2];
            vm[1] = V[1] * vv[0] + V[5] * vv[1] + V[9] * vv[2];
            vm[2] = V[2] * vv[0] + V[6] * vv[1] + V[10] * vv[2];
        }
        // view-space depth gradient: backward.cu:253-259 (the reference always passes zeros here)
        if (v_z) {
            vm[0] += V[8] * v_z[i]; vm[1] += V[9] * v_z[i]; vm[2] += V[10] * v_z[i];
        }
        // conic -> cov2d: helpers.cuh:68-79  (v_Sigma = -X G X)
        float vcov2[3];
        {
            const float a = conic[3 * (size_t)i], b = conic[3 * (size_t)i + 1], d = conic[3 * (size_t)i + 2];
            const float ga = v_conic[3 * (size_t)i], gb = v_conic[3 * (size_t)i + 1] / 2.0f, gd = v_conic[3 * (size_t)i + 2];
            // X G
            const float m00 = a * ga + b * gb, m01 = a * gb + b * gd, m10 = b * ga + d * gb, m11 = b * gb + d * gd;
            const float s00 = -(m00 * a + m01 * b), s01 = -(m00 * b + m01 * d), s10 = -(m10 * a + m11 * b), s11 = -(m10 * b + m11 * d);
            vcov2[0] = s00; vcov2[1] = s01 + s10; vcov2[2] = s11;
        }
        // EWA VJP: backward.cu:291-366 (no 1.3*tanfov clamp here)
        {
            const float R[3][3] = {{V[0], V[1], V[2]}, {V[4], V[5], V[6]}, {V[8], V[9], V[10]}};
            const float rz = 1.0f / tz, rz2 = rz * rz, rz3 = rz2 * rz;
            const float J[3][3] = {{fx * rz, 0, -fx * tx * rz2}, {0, fy * rz, -fy * ty * rz2}, {0, 0, 0}};
            const float* S = cov3d + 6 * (size_t)i;
            const float Vm[3][3] = {{S[0], S[1], S[2]}, {S[1], S[3], S[4]}, {S[2], S[4], S[5]}};
            const float G[3][3] = {{vcov2[0], 0.5f * vcov2[1], 0}, {0.5f * vcov2[1], vcov2[2], 0}, {0, 0, 0}};
            float T[3][3], GT[3][3], vV[3][3], GTV[3][3], vT[3][3], vJ[3][3];
            auto mul = [](const float A[3][3], const float B[3][3], float C[3][3]) {
                for (int r = 0; r < 3; ++r)
                    for (int q = 0; q < 3; ++q) C[r][q] = A[r][0] * B[0][q] + A[r][1] * B[1][q] + A[r][2] * B[2][q];
            };
            mul(J, R, T);
            mul(G, T, GT);
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) vV[r][q] = T[0][r] * GT[0][q] + T[1][r] * GT[1][q] + T[2][r] * GT[2][q];
            mul(GT, Vm, GTV);
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) vT[r][q] = GTV[r][q] + GTV[r][q];  // G T V^T + G^T T V, all symmetric
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) vJ[r][q] = vT[r][0] * R[q][0] + vT[r][1] * R[q][1] + vT[r][2] * R[q][2];
            vc3[0] = vV[0][0]; vc3[1] = vV[0][1] + vV[1][0]; vc3[2] = vV[0][2] + vV[2][0];
            vc3[3] = vV[1][1]; vc3[4] = vV[1][2] + vV[2][1]; vc3[5] = vV[2][2];
            const float vt[3] = {-fx * rz2 * vJ[0][2], -fy * rz2 * vJ[1][2],
                                 -fx * rz2 * vJ[0][0] + 2.0f * fx * tx * rz3 * vJ[0][2] - fy * rz2 * vJ[1][1] +
                                     2.0f * fy * ty * rz3 * vJ[1][2]};
            vm[0] += vt[0] * R[0][0] + vt[1] * R[1][0] + vt[2] * R[2][0];
            vm[1] += vt[0] * R[0][1] + vt[1] * R[1][1] + vt[2] * R[2][1];
            vm[2] += vt[0] * R[0][2] + vt[1] * R[1][2] + vt[2] * R[2][2];
        }
        // scale / rotation VJP: backward.cu:370-393, helpers.cuh:149-220; quaternion used as stored.
        if (scales && rots) {
            const float w = rots[4 * (size_t)i], x = rots[4 * (size_t)i + 1], y = rots[4 * (size_t)i + 2], z = rots[4 * (size_t)i + 3];
            const float R[3][3] = {{1.f - 2.f * (y * y + z * z), 2.f * (x * y - w * z), 2.f * (x * z + w * y)},
                                   {2.f * (x * y + w * z), 1.f - 2.f * (x * x + z * z), 2.f * (y * z - w * x)},
                                   {2.f * (x * z - w * y), 2.f * (y * z + w * x), 1.f - 2.f * (x * x + y * y)}};
            const float gs = c.scale_modifier;
            const float sc[3] = {gs * scales[3 * (size_t)i], gs * scales[3 * (size_t)i + 1], gs * scales[3 * (size_t)i + 2]};
            const float vV[3][3] = {{vc3[0], 0.5f * vc3[1], 0.5f * vc3[2]}, {0.5f * vc3[1], vc3[3], 0.5f * vc3[4]}, {0.5f * vc3[2], 0.5f * vc3[4], vc3[5]}};
            float M[3][3], vM[3][3], vR[3][3];
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) M[r][q] = R[r][q] * sc[q];
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) vM[r][q] = 2.0f * (vV[r][0] * M[0][q] + vV[r][1] * M[1][q] + vV[r][2] * M[2][q]);
            for (int q = 0; q < 3; ++q) vsc[q] = (R[0][q] * vM[0][q] + R[1][q] * vM[1][q] + R[2][q] * vM[2][q]) * gs;
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) vR[r][q] = vM[r][q] * sc[q];
            vq[0] = 2.f * (x * (vR[2][1] - vR[1][2]) + y * (vR[0][2] - vR[2][0]) + z * (vR[1][0] - vR[0][1]));
            vq[1] = 2.f * (-2.f * x * (vR[1][1] + vR[2][2]) + y * (vR[1][0] + vR[0][1]) + z * (vR[2][0] + vR[0][2]) + w * (vR[2][1] - vR[1][2]));
            vq[2] = 2.f * (x * (vR[1][0] + vR[0][1]) - 2.f * y * (vR[0][0] + vR[2][2]) + z * (vR[2][1] + vR[1][2]) + w * (vR[0][2] - vR[2][0]));
            vq[3] = 2.f * (x * (vR[2][0] + vR[0][2]) + y * (vR[2][1] + vR[1][2]) - 2.f * z * (vR[0][0] + vR[1][1]) + w * (vR[1][0] - vR[0][1]));
        }
    }
}

}  // extern "C"
