// Per-Gaussian stage: camera set-up, unscented-transform projection, tile counting, SH colour and
// the packed rasterizer record. Compile this file with --fmad=false: means2d / radii / depths feed
// integer tile lists and sort keys that must not depend on contraction choices.
//
// Replaces gsplat/ProjectionUT3DGSFused.cu:17 (K1), the first pass of gsplat/IntersectTile.cu:24,
// gsplat/SphericalHarmonicsCUDA.cu:374 and the activation / clamp glue of
// src/core/splat_data.cpp:267-286 and gsplat/Rasterization.cpp:358-378 in the fused path.
#include "gsmath.cuh"
#include "projection.cuh"

namespace lfs {

// ---------------------------------------------------------------------------------------------
// quaternion of the rotation block of a row-major 4x4 matrix: the branch with the largest of (trace, +-diagonal sums)
__device__ __forceinline__ void quat_of_viewmat(const float* __restrict__ vm, float& qw, float& qx, float& qy, float& qz) {
    const float R00 = vm[0], R01 = vm[1], R02 = vm[2];
    const float R10 = vm[4], R11 = vm[5], R12 = vm[6];
    const float R20 = vm[8], R21 = vm[9], R22 = vm[10];
    const float fx4 = R00 - R11 - R22, fy4 = R11 - R00 - R22, fz4 = R22 - R00 - R11, fw4 = R00 + R11 + R22;
    int big = 0;
    float fb = fw4;
    if (fx4 > fb) { fb = fx4; big = 1; }
    if (fy4 > fb) { fb = fy4; big = 2; }
    if (fz4 > fb) { fb = fz4; big = 3; }
    const float bv = sqrtf(fb + 1.0f) * 0.5f;
    const float mult = 0.25f / bv;
    if (big == 0)      { qw = bv; qx = (R21 - R12) * mult; qy = (R02 - R20) * mult; qz = (R10 - R01) * mult; }
    else if (big == 1) { qw = (R21 - R12) * mult; qx = bv; qy = (R10 + R01) * mult; qz = (R02 + R20) * mult; }
    else if (big == 2) { qw = (R02 - R20) * mult; qx = (R10 + R01) * mult; qy = bv; qz = (R21 + R12) * mult; }
    else               { qw = (R10 - R01) * mult; qx = (R02 + R20) * mult; qy = (R21 + R12) * mult; qz = bv; }
}

__device__ __forceinline__ CamDev make_cam(const float* __restrict__ vm, const float* __restrict__ vm1, int rs_type,
                                           const float* __restrict__ K, const float* __restrict__ radial4,
                                           const float* __restrict__ dist12, int W, int H, int model) {
    CamDev c;
    for (int i = 0; i < 12; ++i) c.dist[i] = dist12 ? dist12[i] : 0.f;
    float qw, qx, qy, qz;
    quat_of_viewmat(vm, qw, qx, qy, qz);
    c.qw = qw; c.qx = qx; c.qy = qy; c.qz = qz;
    c.tx = vm[3]; c.ty = vm[7]; c.tz = vm[11];
    // inverse quaternion -> rotation matrix -> ray origin
    const float d = qx * qx + qy * qy + qz * qz + qw * qw;
    quat_to_mat_unit(qw / d, -qx / d, -qy / d, -qz / d, c.Rinv);
    for (int i = 0; i < 3; ++i)
        c.ro[i] = (-c.Rinv[i * 3 + 0]) * c.tx + (-c.Rinv[i * 3 + 1]) * c.ty + (-c.Rinv[i * 3 + 2]) * c.tz;
    for (int i = 0; i < 3; ++i)
        c.campos[i] = (float)(-((double)vm[0 * 4 + i] * vm[3] + (double)vm[1 * 4 + i] * vm[7] + (double)vm[2 * 4 + i] * vm[11]));
    c.fx = K[0]; c.fy = K[4]; c.cx = K[2]; c.cy = K[5];
    c.W = W; c.H = H; c.model = model;
    // rolling shutter: end pose and the centre-of-frame pose (equal to the start pose without an end pose)
    c.rs_type = rs_type;
    c.has_end = vm1 != nullptr;
    c.q1w = qw; c.q1x = qx; c.q1y = qy; c.q1z = qz; c.t1x = c.tx; c.t1y = c.ty; c.t1z = c.tz;
    c.qcw = qw; c.qcx = qx; c.qcy = qy; c.qcz = qz; c.tcx = c.tx; c.tcy = c.ty; c.tcz = c.tz;
    if (vm1) {
        quat_of_viewmat(vm1, c.q1w, c.q1x, c.q1y, c.q1z);
        c.t1x = vm1[3]; c.t1y = vm1[7]; c.t1z = vm1[11];
        const PoseQ pc = shutter_pose(c, 0.5f);
        c.qcw = pc.w; c.qcx = pc.x; c.qcy = pc.y; c.qcz = pc.z; c.tcx = pc.t.x; c.tcy = pc.t.y; c.tcz = pc.t.z;
    }
    for (int i = 0; i < 4; ++i) c.k[i] = radial4 ? radial4[i] : 0.f;
    c.max_angle = 0.f; c.approx_b1 = 0.f;
    if (model == LFS_FISHEYE) {
        const float mdx = fmaxf((float)W - c.cx, c.cx), mdy = fmaxf((float)H - c.cy, c.cy);
        const float max_radius_pixels = sqrtf(mdx * mdx + mdy * mdy);
        // Largest usable angle of the OpenCV fisheye polynomial, in the operation order of compute_opencv_fisheye_max_angle
        // (gsplat/Cameras.cuh:760-815), since the clamp feeds the bit-exact tile lists:
        // smallest positive root of 1 + a x + b x^2 + c x^3 (x = theta^2), k4 == 0 only
        const float a = 3.f * c.k[0], b = 5.f * c.k[1], cc = 7.f * c.k[2];
        float root = FLT_MAX;
        if (cc == 0.0f) {
            if (b == 0.0f) {
                if (a < 0.0f) root = -1.0f / a;
            } else {
                float delta = a * a - 4.0f * b;
                if (delta >= 0.0f) {
                    delta = sqrtf(delta) - a;
                    if (delta > 0.0f) root = 2.0f / delta;
                }
            }
        } else {
            const float boc = b / cc, boc2 = boc * boc;
            const float t1 = (9.0f * a * boc - 2.0f * b * boc2 - 27.0f) / cc;
            const float t2 = 3.0f * a / cc - boc2;
            const float delta = t1 * t1 + 4.0f * t2 * t2 * t2;
            if (delta >= 0.0f) {
                const float d2 = sqrtf(delta);
                const float cube_root = cbrtf((d2 + t1) / 2.0f);
                if (cube_root != 0.0f) {
                    const float soln = (cube_root - (t2 / cube_root) - boc) / 3.0f;
                    if (soln > 0.0f) root = soln;
                }
            } else {
                const float theta = atan2f(sqrtf(-delta), t1) / 3.0f;
                const float two_third_pi = 2.0f * 3.14159265358979323846f / 3.0f;
                const float t3 = 2.0f * sqrtf(-t2);
                float soln = FLT_MAX;
                for (int i = -1; i <= 1; ++i) {
                    const float s = (t3 * cosf(theta + i * two_third_pi) - boc) / 3.0f;
                    if (s > 0.0f) soln = fminf(soln, s);
                }
                root = soln;
            }
        }
        float max_angle = sqrtf(root);
        max_angle = fminf(max_angle, fmaxf(max_radius_pixels / c.fx, max_radius_pixels / c.fy));
        c.max_angle = max_angle;
        const float max_norm_dist = fmaxf((float)W / 2.f / c.fx, (float)H / 2.f / c.fy);
        c.approx_b1 = max_angle / max_norm_dist;
    }
    return c;
}

__global__ void camera_setup_kernel(int C, const float* __restrict__ viewmats, const float* __restrict__ viewmats1, int rs_type,
                                    const float* __restrict__ Ks, const float* __restrict__ radial,
                                    const float* __restrict__ tangential, const float* __restrict__ thin_prism, int W, int H,
                                    int model, CamDev* cams) {
    const int cid = blockIdx.x * blockDim.x + threadIdx.x;
    if (cid >= C) return;
    const float* vm1 = viewmats1 ? viewmats1 + cid * 16 : nullptr;
    if (model == LFS_PINHOLE_OPENCV) {
        float d[12];
        for (int i = 0; i < 6; ++i) d[i] = radial ? radial[cid * 6 + i] : 0.f;
        for (int i = 0; i < 2; ++i) d[6 + i] = tangential ? tangential[cid * 2 + i] : 0.f;
        for (int i = 0; i < 4; ++i) d[8 + i] = thin_prism ? thin_prism[cid * 4 + i] : 0.f;
        cams[cid] = make_cam(viewmats + cid * 16, vm1, rs_type, Ks + cid * 9, nullptr, d, W, H, model);
    } else {
        cams[cid] = make_cam(viewmats + cid * 16, vm1, rs_type, Ks + cid * 9,
                             (radial && model == LFS_FISHEYE) ? radial + cid * 4 : nullptr, nullptr, W, H, model);
    }
}

int launch_camera_setup(int C, const float* viewmats, const float* viewmats1, int rs_type, const float* Ks, const float* radial,
                        const float* tangential, const float* thin_prism, int W, int H, int model, CamDev* cams,
                        cudaStream_t st) {
    camera_setup_kernel<<<(C + 31) / 32, 32, 0, st>>>(C, viewmats, viewmats1, rs_type, Ks, radial, tangential, thin_prism, W, H,
                                                      effective_model(model, radial, tangential, thin_prism), cams);
    return check_launch("camera_setup");
}

// ---------------------------------------------------------------------------------------------
// Unscented-transform projection of one Gaussian (activated quaternion / scale / opacity).
// Returns false when culled. Operation order is fixed; see the file header.
// ---------------------------------------------------------------------------------------------
struct ProjOut {
    float mx, my, depth;
    float c00, c01, c11;  // blurred 2-D covariance
    float det, compensation;
    int rx, ry;
};

template <int MODEL, bool RS>
__device__ __forceinline__ bool project_gaussian(const CamDev& cam, const ProjParams& pp, f3 mean, float qw, float qx,
                                                 float qy, float qz, f3 scale, bool has_opacity, float opacity_in,
                                                 ProjOut& o) {
    // unit quaternion (identity for a zero quaternion)
    {
        const float len = sqrtf(qx * qx + qy * qy + qz * qz + qw * qw);
        if (len <= 0.0f) { qw = 1.f; qx = 0.f; qy = 0.f; qz = 0.f; }
        else { const float inv = 1.0f / len; qw *= inv; qx *= inv; qy *= inv; qz *= inv; }
    }
    // depth and culling with the centre-of-frame pose (the start pose for a global shutter)
    const f3 mean_c = RS ? quat_rotate(cam.qcw, cam.qcx, cam.qcy, cam.qcz, mean) + f3{cam.tcx, cam.tcy, cam.tcz}
                         : quat_rotate(cam.qw, cam.qx, cam.qy, cam.qz, mean) + f3{cam.tx, cam.ty, cam.tz};
    // the equirectangular model sees the whole sphere: no near-plane cull (gsplat/ProjectionUT3DGSFused.cu:78)
    if ((mean_c.z < pp.near_plane && MODEL != LFS_EQUIRECTANGULAR) || mean_c.z > pp.far_plane) return false;
    o.depth = mean_c.z;

    const float D = 3.0f;
    const float lambda = pp.alpha * pp.alpha * (D + pp.kappa) - D;
    float R[9];
    quat_to_mat_unit(qw, qx, qy, qz, R);
    const float sq = sqrtf(D + lambda);
    const float wm0 = lambda / (D + lambda);
    const float wc0 = lambda / (D + lambda) + (1.0f - pp.alpha * pp.alpha + pp.beta);
    const float wi = 1.0f / (2.0f * (D + lambda));
    const float sc[3] = {scale.x, scale.y, scale.z};

    float ipx[7], ipy[7];
    float m2x = 0.f, m2y = 0.f;
    bool valid = pp.require_all;
#pragma unroll
    for (int i = 0; i < 7; ++i) {
        f3 p = mean;
        if (i > 0) {
            const int a = (i - 1) % 3;
            const float f = sq * sc[a];
            const f3 delta = f * f3{R[0 * 3 + a], R[1 * 3 + a], R[2 * 3 + a]};
            p = (i <= 3) ? (mean + delta) : (mean - delta);
        }
        float px, py;
        const bool pv = world_point_to_image<MODEL, RS>(cam, p, pp.margin, px, py);
        if (pp.require_all) {
            valid &= pv;
            if (!pv) return false;
        } else {
            valid |= pv;
        }
        ipx[i] = px; ipy[i] = py;
        const float w = (i == 0) ? wm0 : wi;
        m2x += w * px;
        m2y += w * py;
    }
    if (!valid) return false;
    float c00 = 0.f, c01 = 0.f, c11 = 0.f;
#pragma unroll
    for (int i = 0; i < 7; ++i) {
        const float dx = ipx[i] - m2x, dy = ipy[i] - m2y;
        const float w = (i == 0) ? wc0 : wi;
        c00 += w * (dx * dx);
        c01 += w * (dx * dy);
        c11 += w * (dy * dy);
    }
    const float det_orig = c00 * c11 - c01 * c01;
    c00 += pp.eps2d; c11 += pp.eps2d;
    const float det = c00 * c11 - c01 * c01;
    const float compensation = sqrtf(fmaxf(0.f, det_orig / det));
    if (det <= 0.f) return false;

    float extend = 3.33f;
    if (has_opacity) {
        const float opacity = opacity_in * compensation;
        const float ALPHA_THRESHOLD = 1.f / 255.f;
        if (opacity < ALPHA_THRESHOLD) return false;
        // log in double, rounded once: reproducible across math libraries
        const float lg = (float)log((double)(opacity / ALPHA_THRESHOLD));
        extend = fminf(extend, sqrtf(2.0f * lg));
    }
    const float b = 0.5f * (c00 + c11);
    const float tmp = sqrtf(fmaxf(0.01f, b * b - det));
    const float v1 = b + tmp;
    const float r1 = extend * sqrtf(v1);
    const float radius_x = ceilf(fminf(extend * sqrtf(c00), r1));
    const float radius_y = ceilf(fminf(extend * sqrtf(c11), r1));
    if (radius_x <= pp.radius_clip && radius_y <= pp.radius_clip) return false;
    if (m2x + radius_x <= 0 || m2x - radius_x >= (float)cam.W || m2y + radius_y <= 0 || m2y - radius_y >= (float)cam.H)
        return false;
    o.mx = m2x; o.my = m2y;
    o.c00 = c00; o.c01 = c01; o.c11 = c11;
    o.det = det; o.compensation = compensation;
    o.rx = (int)radius_x; o.ry = (int)radius_y;
    return true;
}

// ---------------------------------------------------------------------------------------------
// Operator-level projection kernel: [C,N] outputs in the reference layouts.
// ---------------------------------------------------------------------------------------------
template <int MODEL, bool RS>
__global__ void __launch_bounds__(256) projection_ut_kernel(
    int C, int N, const float* __restrict__ means, const float* __restrict__ quats, const float* __restrict__ scales,
    const float* __restrict__ opacities, const float* __restrict__ viewmats, const float* __restrict__ viewmats1, int rs_type,
    const float* __restrict__ Ks,
    const float* __restrict__ radial, const float* __restrict__ tangential, const float* __restrict__ thin_prism, int W, int H,
    ProjParams pp, int32_t* __restrict__ radii, float* __restrict__ means2d, float* __restrict__ depths,
    float* __restrict__ conics, float* __restrict__ compensations) {
    const int64_t total = (int64_t)C * N;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int cid = (int)(idx / N);
        const int gid = (int)(idx % N);
        CamDev cam;
        if (MODEL == LFS_PINHOLE_OPENCV) {
            float d[12];
            for (int i = 0; i < 6; ++i) d[i] = radial ? radial[cid * 6 + i] : 0.f;
            for (int i = 0; i < 2; ++i) d[6 + i] = tangential ? tangential[cid * 2 + i] : 0.f;
            for (int i = 0; i < 4; ++i) d[8 + i] = thin_prism ? thin_prism[cid * 4 + i] : 0.f;
            cam = make_cam(viewmats + cid * 16, viewmats1 ? viewmats1 + cid * 16 : nullptr, rs_type, Ks + cid * 9, nullptr, d, W, H, MODEL);
        } else {
            cam = make_cam(viewmats + cid * 16, viewmats1 ? viewmats1 + cid * 16 : nullptr, rs_type, Ks + cid * 9,
                           (radial && MODEL == LFS_FISHEYE) ? radial + cid * 4 : nullptr, nullptr, W, H, MODEL);
        }
        const f3 mean{means[gid * 3], means[gid * 3 + 1], means[gid * 3 + 2]};
        const f3 scale{scales[gid * 3], scales[gid * 3 + 1], scales[gid * 3 + 2]};
        const float4 q = reinterpret_cast<const float4*>(quats)[gid];
        ProjOut o;
        const bool vis = project_gaussian<MODEL, RS>(cam, pp, mean, q.x, q.y, q.z, q.w, scale, opacities != nullptr,
                                                     opacities ? opacities[gid] : 0.f, o);
        if (!vis) {
            radii[idx * 2] = 0;
            radii[idx * 2 + 1] = 0;
            continue;
        }
        radii[idx * 2] = o.rx;
        radii[idx * 2 + 1] = o.ry;
        means2d[idx * 2] = o.mx;
        means2d[idx * 2 + 1] = o.my;
        depths[idx] = o.depth;
        const float ood = 1.0f / (o.c00 * o.c11 - o.c01 * o.c01);
        conics[idx * 3] = o.c11 * ood;
        conics[idx * 3 + 1] = -o.c01 * ood;
        conics[idx * 3 + 2] = o.c00 * ood;
        if (compensations) compensations[idx] = o.compensation;
    }
}

int launch_projection_ut(int C, int N, const float* means, const float* quats, const float* scales,
                         const float* opacities, const float* viewmats, const float* viewmats1, int rs_type, const float* Ks,
                         const float* radial, const float* tangential, const float* thin_prism, int W, int H,
                         const ProjParams& pp, int model, int32_t* radii,
                         float* means2d, float* depths, float* conics, float* compensations, cudaStream_t st) {
    const int64_t total = (int64_t)C * N;
    if (total == 0) return LFS_OK;
    const int grid = grid_for(total, 256);
    LFS_TIMED("projection_ut", st);
    const bool rs = rs_type != LFS_SHUTTER_GLOBAL || viewmats1 != nullptr;
#define LFS_PROJ2(MODEL, RS)                                                                                                  \
    projection_ut_kernel<MODEL, RS><<<grid, 256, 0, st>>>(C, N, means, quats, scales, opacities, viewmats, viewmats1, rs_type, Ks, \
                                                          radial, tangential, thin_prism, W, H, pp, radii, means2d, depths,   \
                                                          conics, compensations)
#define LFS_PROJ(MODEL) do { if (rs) LFS_PROJ2(MODEL, true); else LFS_PROJ2(MODEL, false); } while (0)
    switch (effective_model(model, radial, tangential, thin_prism)) {
        case LFS_PINHOLE: LFS_PROJ(LFS_PINHOLE); break;
        case LFS_PINHOLE_OPENCV: LFS_PROJ(LFS_PINHOLE_OPENCV); break;
        case LFS_EQUIRECTANGULAR: LFS_PROJ(LFS_EQUIRECTANGULAR); break;
        default: LFS_PROJ(LFS_FISHEYE); break;
    }
#undef LFS_PROJ
#undef LFS_PROJ2
    return check_launch("projection_ut");
}

// ---------------------------------------------------------------------------------------------
// Rasterizer record from activated parameters: M = diag(1/s) R^T with the quaternion
// re-normalised, gro = M (ray_origin - mean).
// ---------------------------------------------------------------------------------------------
// Also computes the exact screen-space bounding box (in whole pixels, inclusive, clamped to 16 bits) of the
// pixels whose ray can reach alpha >= 1/255: alpha = opacity * exp(-d^2/2) with d the distance from the ray to
// the centre in the whitened frame, so those rays are exactly the ones that hit the ellipsoid
// (x-mu)^T M^T M (x-mu) <= rho^2, rho^2 = 2 ln(255 opacity). Under a pinhole camera its outline is a conic whose
// axis-aligned tangents follow from the dual quadric B = mu_c mu_c^T - Sigma_c:
// x_n = (B02 -+ sqrt(B02^2 - B00 B22)) / B22 (same with index 1 for y). A margin keeps the box conservative under
// rounding; when the ellipsoid reaches the camera plane (B22 <= 0) or the camera is not a pinhole the box is the
// whole image. The rasterizer uses it only to skip (warp patch, Gaussian) pairs that cannot contribute.
__device__ __forceinline__ void make_record(const CamDev& cam, f3 mean, float qw, float qx, float qy, float qz,
                                            f3 scale, float r, float g, float b, float opacity, float extra, float4* rec,
                                            uint4& box) {
    float R[9], inv_norm, qn[4];
    quat_to_rotmat_renorm(qw, qx, qy, qz, R, inv_norm, qn);
    // exponent below which opacity * exp(p) < 1/255 for certain, as float bits in .z
    const uint32_t thr_bits = __float_as_uint(-logf(fmaxf(255.0f * opacity, 1e-30f)) - 0.02f);
    const uint32_t extra_bits = __float_as_uint(extra);  // blended into the last channel of 1- and 4-channel renders
    box = make_uint4(0xFFFF0000u, 0xFFFF0000u, thr_bits, extra_bits);  // (lo | hi << 16) per axis: everything
    if (cam.model == LFS_PINHOLE && cam.rs_type == LFS_SHUTTER_GLOBAL && !cam.has_end) {   // one pose for every pixel
        const float rho2 = 2.0f * (logf(fmaxf(255.0f * opacity, 1.0f)) + 0.03f);
        // V = R_c R with R_c = Rinv^T ; Sigma_c = rho2 V S^2 V^T ; mu_c = R_c mean + t
        float V[9];
#pragma unroll
        for (int a = 0; a < 3; ++a)
#pragma unroll
            for (int c = 0; c < 3; ++c)
                V[a * 3 + c] = cam.Rinv[0 * 3 + a] * R[0 * 3 + c] + cam.Rinv[1 * 3 + a] * R[1 * 3 + c] + cam.Rinv[2 * 3 + a] * R[2 * 3 + c];
        const float s2[3] = {rho2 * scale.x * scale.x, rho2 * scale.y * scale.y, rho2 * scale.z * scale.z};
        const float mc[3] = {cam.Rinv[0] * mean.x + cam.Rinv[3] * mean.y + cam.Rinv[6] * mean.z + cam.tx,
                             cam.Rinv[1] * mean.x + cam.Rinv[4] * mean.y + cam.Rinv[7] * mean.z + cam.ty,
                             cam.Rinv[2] * mean.x + cam.Rinv[5] * mean.y + cam.Rinv[8] * mean.z + cam.tz};
        auto sig = [&](int a, int c) { return V[a * 3] * s2[0] * V[c * 3] + V[a * 3 + 1] * s2[1] * V[c * 3 + 1] + V[a * 3 + 2] * s2[2] * V[c * 3 + 2]; };
        const float B22 = mc[2] * mc[2] - sig(2, 2);
        if (mc[2] > 0.f && B22 > 0.02f * mc[2] * mc[2]) {
            uint32_t packed[2];
            const float f[2] = {cam.fx, cam.fy}, c0[2] = {cam.cx, cam.cy};
#pragma unroll
            for (int ax = 0; ax < 2; ++ax) {
                const float Ba2 = mc[ax] * mc[2] - sig(ax, 2);
                const float Baa = mc[ax] * mc[ax] - sig(ax, ax);
                const float disc = sqrtf(fmaxf(0.f, Ba2 * Ba2 - Baa * B22));
                const float lo_n = (Ba2 - disc) / B22, hi_n = (Ba2 + disc) / B22;
                const float fl = fabsf(f[ax]);
                const float lo_px = fminf(f[ax] * lo_n, f[ax] * hi_n) + c0[ax], hi_px = fmaxf(f[ax] * lo_n, f[ax] * hi_n) + c0[ax];
                const float margin = 0.75f + 2e-4f * (fabsf(lo_px) + fabsf(hi_px)) + 1e-3f * fl * (hi_n - lo_n);
                // pixel j has its centre at j + 0.5
                const float lo_j = floorf(lo_px - 0.5f - margin), hi_j = ceilf(hi_px - 0.5f + margin);
                const uint32_t lo_u = (uint32_t)fminf(fmaxf(lo_j, 0.f), 65535.f), hi_u = (uint32_t)fminf(fmaxf(hi_j, 0.f), 65535.f);
                packed[ax] = lo_u | (hi_u << 16);
            }
            box = make_uint4(packed[0], packed[1], thr_bits, extra_bits);
        }
    }
    const float is[3] = {1.0f / scale.x, 1.0f / scale.y, 1.0f / scale.z};
    float M[9];
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int c = 0; c < 3; ++c) M[a * 3 + c] = is[a] * R[c * 3 + a];
    const f3 om{cam.ro[0] - mean.x, cam.ro[1] - mean.y, cam.ro[2] - mean.z};
    const float g0 = M[0] * om.x + M[1] * om.y + M[2] * om.z;
    const float g1 = M[3] * om.x + M[4] * om.y + M[5] * om.z;
    const float g2 = M[6] * om.x + M[7] * om.y + M[8] * om.z;
    rec[0] = make_float4(M[0], M[1], M[2], g0);
    rec[1] = make_float4(M[3], M[4], M[5], g1);
    rec[2] = make_float4(M[6], M[7], M[8], g2);
    rec[3] = make_float4(r, g, b, opacity);
}

__global__ void __launch_bounds__(256) pack_records_kernel(
    int N, const float* __restrict__ means, const float* __restrict__ quats, const float* __restrict__ scales,
    const float* __restrict__ colors, int channels, const float* __restrict__ opacities, const CamDev* __restrict__ cams,
    float4* __restrict__ records, uint4* __restrict__ bounds, float4* __restrict__ accum, float* __restrict__ accum_extra) {
    const CamDev cam = cams[0];
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < N; g += gridDim.x * blockDim.x) {
        const f3 mean{means[g * 3], means[g * 3 + 1], means[g * 3 + 2]};
        const f3 scale{scales[g * 3], scales[g * 3 + 1], scales[g * 3 + 2]};
        const float4 q = reinterpret_cast<const float4*>(quats)[g];
        float4 rec[4];
        uint4 box;
        // colours [N, channels]: channels 3 = rgb; 4 = rgb + extra; 1 = extra only
        const float* col = colors + (size_t)g * channels;
        const bool has_rgb = channels >= 3;
        make_record(cam, mean, q.x, q.y, q.z, q.w, scale, has_rgb ? col[0] : 0.f, has_rgb ? col[1] : 0.f, has_rgb ? col[2] : 0.f,
                    opacities[g], channels != 3 ? col[channels - 1] : 0.f, rec, box);
#pragma unroll
        for (int k = 0; k < 4; ++k) records[(size_t)g * 4 + k] = rec[k];
        bounds[g] = box;
        if (accum) {
#pragma unroll
            for (int k = 0; k < 4; ++k) accum[(size_t)g * 4 + k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (accum_extra) accum_extra[g] = 0.f;
    }
}

int launch_pack_records(int N, const float* means, const float* quats, const float* scales, const float* colors, int channels,
                        const float* opacities, const CamDev* cam, float4* records, uint4* bounds, float4* accum,
                        float* accum_extra, cudaStream_t st) {
    if (N == 0) return LFS_OK;
    LFS_TIMED("pack_records", st);
    pack_records_kernel<<<grid_for(N, 256), 256, 0, st>>>(N, means, quats, scales, colors, channels, opacities, cam, records,
                                                          bounds, accum, accum_extra);
    return check_launch("pack_records");
}

// ---------------------------------------------------------------------------------------------
// Fused per-Gaussian forward stage of the training path (one camera): activations, projection,
// tile count, depth sort key, SH colour (+0.5, clamped at 0), packed record, zeroed gradient
// accumulator row. Invisible Gaussians get radii 0, tile count 0 and the sort key 0xFFFFFFFF.
// ---------------------------------------------------------------------------------------------
template <int MODEL, bool RS>
__global__ void __launch_bounds__(256, 3) project_pack_kernel(
    int N, int K, int sh_degree, const float* __restrict__ means, const float* __restrict__ sh0,
    const float* __restrict__ shN, const float* __restrict__ scaling_raw, const float* __restrict__ rotation_raw,
    const float* __restrict__ opacity_raw, const CamDev* __restrict__ cams, ProjParams pp, PackOptions opt, float tile_size,
    uint32_t tw, uint32_t th,
    int32_t* __restrict__ radii, float* __restrict__ means2d, float* __restrict__ depths,
    int32_t* __restrict__ tiles, uint32_t* __restrict__ sort_keys, uint32_t* __restrict__ sort_vals,
    float4* __restrict__ records, uint4* __restrict__ bounds, float4* __restrict__ accum, int32_t* __restrict__ n_visible) {
    // Each warp handles 32 consecutive Gaussians per iteration. Their higher-order SH rows ((K-1)*3 floats
    // each, contiguous in memory) are fetched as one coalesced run into shared memory when any of the 32
    // is visible, and every visible lane then reads its own row from there.
    extern __shared__ __align__(16) float s_rows[];
    const CamDev cam = cams[0];
    const int rest = (K - 1) * 3;
    const int nb = (sh_degree + 1) * (sh_degree + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my = s_rows + (size_t)warp * 32 * rest;
    const int n_chunks = (N + 31) / 32;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const bool sh_aligned = (reinterpret_cast<uintptr_t>(shN) & 15) == 0 && ((32 * rest) & 3) == 0;
    int local_visible = 0;
    for (int chunk = blockIdx.x * (blockDim.x >> 5) + warp; chunk < n_chunks; chunk += warps_total) {
        const int g = chunk * 32 + lane;
        const bool in_range = g < N;
        bool vis = false;
        ProjOut o;
        f3 mean{0.f, 0.f, 0.f}, scale{1.f, 1.f, 1.f};
        float opacity = 0.f, qw = 1.f, qx = 0.f, qy = 0.f, qz = 0.f;
        if (in_range) {
            mean = f3{means[g * 3], means[g * 3 + 1], means[g * 3 + 2]};
            // activations: sigmoid / exp through double, rounded once; F.normalize-style quaternion
            opacity = (float)(1.0 / (1.0 + exp(-(double)opacity_raw[g])));
            scale = f3{(float)exp((double)scaling_raw[g * 3]), (float)exp((double)scaling_raw[g * 3 + 1]),
                       (float)exp((double)scaling_raw[g * 3 + 2])};
            if (opt.scaling_modifier != 1.0f) { scale.x *= opt.scaling_modifier; scale.y *= opt.scaling_modifier; scale.z *= opt.scaling_modifier; }
            const float4 qr = reinterpret_cast<const float4*>(rotation_raw)[g];
            const float n2 = ((qr.x * qr.x + qr.y * qr.y) + qr.z * qr.z) + qr.w * qr.w;
            const float nrm = fmaxf(sqrtf(n2), 1e-12f);
            qw = qr.x / nrm; qx = qr.y / nrm; qy = qr.z / nrm; qz = qr.w / nrm;
            vis = project_gaussian<MODEL, RS>(cam, pp, mean, qw, qx, qy, qz, scale, true, opacity, o);
            sort_vals[g] = (uint32_t)g;
            if (!vis) {
                radii[g * 2] = 0; radii[g * 2 + 1] = 0;
                tiles[g] = 0;
                sort_keys[g] = 0xFFFFFFFFu;
            }
        }
        const bool any_vis = __any_sync(0xffffffffu, vis);
        if (any_vis && nb > 1 && opt.want_rgb) {
            // one batch of asynchronous 16-byte copies (a single round trip instead of one per row slice); the
            // chunk starts 16-byte aligned because it begins at a multiple of 32 rows
            const int n_rows = min(32, N - chunk * 32);
            const int total = n_rows * rest;
            const float* src = shN + (size_t)chunk * 32 * rest;
            const int total16 = sh_aligned ? (total >> 2) : 0;
            for (int i = lane; i < total16; i += 32) {
                const unsigned dst = (unsigned)__cvta_generic_to_shared(my + i * 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src + i * 4));
            }
            asm volatile("cp.async.commit_group;\n" ::);
            for (int i = total16 * 4 + lane; i < total; i += 32) my[i] = src[i];
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncwarp();
        if (vis) {
            radii[g * 2] = o.rx; radii[g * 2 + 1] = o.ry;
            means2d[g * 2] = o.mx; means2d[g * 2 + 1] = o.my;
            depths[g] = o.depth;
            uint32_t x0, y0, x1, y1;
            tile_rect(o.mx, o.my, o.rx, o.ry, tile_size, tw, th, x0, y0, x1, y1);
            const int nt = (int)((y1 - y0) * (x1 - x0));
            tiles[g] = nt;
            sort_keys[g] = nt > 0 ? __float_as_uint(o.depth) : 0xFFFFFFFFu;
            ++local_visible;

            // colour from SH along (mean - camera position)
            float rgb[3] = {0.f, 0.f, 0.f};
            if (opt.want_rgb) {
                float B[25];
                sh_basis(sh_degree, mean.x - cam.campos[0], mean.y - cam.campos[1], mean.z - cam.campos[2], B);
#pragma unroll
                for (int c = 0; c < 3; ++c) rgb[c] = B[0] * sh0[g * 3 + c];
                const float* row = my + lane * rest;
                for (int k = 1; k < nb; ++k) {
#pragma unroll
                    for (int c = 0; c < 3; ++c) rgb[c] += B[k] * row[(k - 1) * 3 + c];
                }
#pragma unroll
                for (int c = 0; c < 3; ++c) rgb[c] = fmaxf(rgb[c] + 0.5f, 0.0f);
            }
            // antialiased mode: the blended opacity carries the blur compensation (gsplat/Rasterization.cpp:396-399)
            if (opt.calc_compensations) opacity *= o.compensation;

            float4 rec[4];
            uint4 box;
            make_record(cam, mean, qw, qx, qy, qz, scale, rgb[0], rgb[1], rgb[2], opacity, o.depth, rec, box);
#pragma unroll
            for (int k = 0; k < 4; ++k) records[(size_t)g * 4 + k] = rec[k];
            bounds[g] = box;
#pragma unroll
            for (int k = 0; k < 4; ++k) accum[(size_t)g * 4 + k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        __syncwarp();
    }
    // visible count (statistics only)
    local_visible = __reduce_add_sync(0xffffffffu, local_visible);
    if (lane == 0 && local_visible) atomicAdd(n_visible, local_visible);
}

// Colours of the visible Gaussians into their packed records, for callers that build the tile lists first
// (project_pack with want_rgb = 0) and shade later, e.g. while the SH coefficients are still being updated on another
// stream. Same arithmetic and staging as the colour part of project_pack_kernel.
__global__ void __launch_bounds__(256) sh_color_kernel(int N, int K, int sh_degree, const float* __restrict__ means,
                                                       const float* __restrict__ sh0, const float* __restrict__ shN,
                                                       const CamDev* __restrict__ cams, const int32_t* __restrict__ radii,
                                                       float4* __restrict__ records) {
    extern __shared__ __align__(16) float s_rows[];
    const float cx = cams[0].campos[0], cy = cams[0].campos[1], cz = cams[0].campos[2];
    const int rest = (K - 1) * 3;
    const int nb = (sh_degree + 1) * (sh_degree + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my = s_rows + (size_t)warp * 32 * rest;
    const int n_chunks = (N + 31) / 32;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const bool sh_aligned = (reinterpret_cast<uintptr_t>(shN) & 15) == 0 && ((32 * rest) & 3) == 0;
    for (int chunk = blockIdx.x * (blockDim.x >> 5) + warp; chunk < n_chunks; chunk += warps_total) {
        const int g = chunk * 32 + lane;
        const bool vis = g < N && radii[g * 2] > 0 && radii[g * 2 + 1] > 0;
        if (!__any_sync(0xffffffffu, vis)) continue;
        if (nb > 1) {
            const int total = min(32, N - chunk * 32) * rest;
            const float* src = shN + (size_t)chunk * 32 * rest;
            const int total16 = sh_aligned ? (total >> 2) : 0;
            for (int i = lane; i < total16; i += 32) {
                const unsigned dst = (unsigned)__cvta_generic_to_shared(my + i * 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src + i * 4));
            }
            asm volatile("cp.async.commit_group;\n" ::);
            for (int i = total16 * 4 + lane; i < total; i += 32) my[i] = src[i];
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncwarp();
        if (vis) {
            float B[25];
            sh_basis(sh_degree, means[g * 3] - cx, means[g * 3 + 1] - cy, means[g * 3 + 2] - cz, B);
            float rgb[3];
#pragma unroll
            for (int c = 0; c < 3; ++c) rgb[c] = B[0] * sh0[g * 3 + c];
            const float* row = my + lane * rest;
            for (int k = 1; k < nb; ++k) {
#pragma unroll
                for (int c = 0; c < 3; ++c) rgb[c] += B[k] * row[(k - 1) * 3 + c];
            }
            float* out = reinterpret_cast<float*>(records + (size_t)g * 4 + 3);
#pragma unroll
            for (int c = 0; c < 3; ++c) out[c] = fmaxf(rgb[c] + 0.5f, 0.0f);
        }
        __syncwarp();
    }
}

int launch_sh_color(int N, int K, int sh_degree, const lfs_splats& p, const CamDev* cam, const int32_t* radii, float4* records,
                    cudaStream_t st) {
    if (N == 0) return LFS_OK;
    const size_t smem = (size_t)8 * 32 * (K - 1) * 3 * sizeof(float);
    if (smem > 200 * 1024) { set_error("sh_color: too many SH coefficients"); return LFS_EINVAL; }
    if (smem > 48 * 1024) cudaFuncSetAttribute(sh_color_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    LFS_TIMED("sh_color", st);
    sh_color_kernel<<<grid_for(N, 256), 256, smem, st>>>(N, K, sh_degree, p.means, p.sh0, p.shN, cam, radii, records);
    return check_launch("sh_color");
}

int launch_project_pack(int N, int K, int sh_degree, const lfs_splats& p, const CamDev* cam, const ProjParams& pp,
                        const PackOptions& opt, int model, int rolling, int tile_size, int tw, int th, int32_t* radii, float* means2d, float* depths,
                        int32_t* tiles, uint32_t* sort_keys, uint32_t* sort_vals, float4* records, uint4* bounds, float4* accum,
                        int32_t* n_visible, cudaStream_t st) {
    if (N == 0) return LFS_OK;
    const int grid = grid_for(N, 256);
    const size_t smem = (size_t)8 * 32 * (K - 1) * 3 * sizeof(float);
    if (smem > 200 * 1024) { set_error("project_pack: too many SH coefficients"); return LFS_EINVAL; }
    if (smem > 48 * 1024) {
#define LFS_PACK_ATTR(MODEL)                                                                                        \
    cudaFuncSetAttribute(project_pack_kernel<MODEL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    cudaFuncSetAttribute(project_pack_kernel<MODEL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        LFS_PACK_ATTR(LFS_PINHOLE); LFS_PACK_ATTR(LFS_FISHEYE); LFS_PACK_ATTR(LFS_PINHOLE_OPENCV); LFS_PACK_ATTR(LFS_EQUIRECTANGULAR);
#undef LFS_PACK_ATTR
    }
    LFS_TIMED("project_pack", st);
#define LFS_PACK2(MODEL, RS)                                                                                                       \
    project_pack_kernel<MODEL, RS><<<grid, 256, smem, st>>>(N, K, sh_degree, p.means, p.sh0, p.shN, p.scaling_raw, p.rotation_raw,  \
                                                            p.opacity_raw, cam, pp, opt, (float)tile_size, tw, th, radii, means2d, \
                                                            depths, tiles, sort_keys, sort_vals, records, bounds, accum, n_visible)
#define LFS_PACK(MODEL) do { if (rolling) LFS_PACK2(MODEL, true); else LFS_PACK2(MODEL, false); } while (0)
    switch (model) {
        case LFS_PINHOLE: LFS_PACK(LFS_PINHOLE); break;
        case LFS_PINHOLE_OPENCV: LFS_PACK(LFS_PINHOLE_OPENCV); break;
        case LFS_EQUIRECTANGULAR: LFS_PACK(LFS_EQUIRECTANGULAR); break;
        default: LFS_PACK(LFS_FISHEYE); break;
    }
#undef LFS_PACK
#undef LFS_PACK2
    return check_launch("project_pack");
}

// ---------------------------------------------------------------------------------------------
// Operator-level tile count: tiles_per_gauss [C*N] (0 where a radius is <= 0).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) tile_count_kernel(int64_t total, const float* __restrict__ means2d,
                                                         const int32_t* __restrict__ radii, float tile_size,
                                                         uint32_t tw, uint32_t th, int32_t* __restrict__ tiles) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int rx = radii[idx * 2], ry = radii[idx * 2 + 1];
        int nt = 0;
        if (!(rx <= 0 || ry <= 0)) {
            uint32_t x0, y0, x1, y1;
            tile_rect(means2d[idx * 2], means2d[idx * 2 + 1], rx, ry, tile_size, tw, th, x0, y0, x1, y1);
            nt = (int)((y1 - y0) * (x1 - x0));
        }
        tiles[idx] = nt;
    }
}

int launch_tile_count(int64_t total, const float* means2d, const int32_t* radii, int tile_size, int tw, int th,
                      int32_t* tiles, cudaStream_t st) {
    if (total == 0) return LFS_OK;
    tile_count_kernel<<<grid_for(total, 256), 256, 0, st>>>(total, means2d, radii, (float)tile_size, tw, th, tiles);
    return check_launch("tile_count");
}

}  // namespace lfs
