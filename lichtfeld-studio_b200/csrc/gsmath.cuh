// Device math shared by the kernels: quaternion / pose helpers, camera models, SH basis.
// The projection translation unit is compiled with --fmad=false so that these functions give
// bit-identical results to a plain IEEE float32 evaluation in the same operation order; the
// rasterizer units use the default contraction.
#pragma once

#include <cuda_runtime.h>
#include <float.h>
#include <math.h>

#include "common.cuh"

namespace lfs {

struct f3 { float x, y, z; };

__device__ __forceinline__ f3 operator+(f3 a, f3 b) { return {a.x + b.x, a.y + b.y, a.z + b.z}; }
__device__ __forceinline__ f3 operator-(f3 a, f3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
__device__ __forceinline__ f3 operator*(f3 a, float s) { return {a.x * s, a.y * s, a.z * s}; }
__device__ __forceinline__ f3 operator*(float s, f3 a) { return {a.x * s, a.y * s, a.z * s}; }
__device__ __forceinline__ float dot3(f3 a, f3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ f3 cross3(f3 a, f3 b) {
    return {a.y * b.z - b.y * a.z, a.z * b.x - b.z * a.x, a.x * b.y - b.x * a.y};
}

// Rotation of v by the quaternion (w; x,y,z): v + 2 (w (q x v) + q x (q x v)).
__device__ __forceinline__ f3 quat_rotate(float qw, float qx, float qy, float qz, f3 v) {
    const f3 qv{qx, qy, qz};
    const f3 uv = cross3(qv, v);
    const f3 uuv = cross3(qv, uv);
    return v + ((uv * qw) + uuv) * 2.0f;
}

// Rotation matrix (row-major m[r*3+c]) of a quaternion assumed to be unit length.
__device__ __forceinline__ void quat_to_mat_unit(float w, float x, float y, float z, float* m) {
    const float qxx = x * x, qyy = y * y, qzz = z * z;
    const float qxz = x * z, qxy = x * y, qyz = y * z;
    const float qwx = w * x, qwy = w * y, qwz = w * z;
    m[0] = 1.0f - 2.0f * (qyy + qzz);
    m[3] = 2.0f * (qxy + qwz);
    m[6] = 2.0f * (qxz - qwy);
    m[1] = 2.0f * (qxy - qwz);
    m[4] = 1.0f - 2.0f * (qxx + qzz);
    m[7] = 2.0f * (qyz + qwx);
    m[2] = 2.0f * (qxz + qwy);
    m[5] = 2.0f * (qyz - qwx);
    m[8] = 1.0f - 2.0f * (qxx + qyy);
}

// Rotation matrix of a quaternion that is re-normalised first with an approximate reciprocal
// square root (the rasterizer's convention). Also returns the normalised components.
__device__ __forceinline__ void quat_to_rotmat_renorm(float w, float x, float y, float z, float* m,
                                                      float& inv_norm, float* qn) {
    inv_norm = rsqrtf(x * x + y * y + z * z + w * w);
    x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
    qn[0] = w; qn[1] = x; qn[2] = y; qn[3] = z;
    const float x2 = x * x, y2 = y * y, z2 = z * z;
    const float xy = x * y, xz = x * z, yz = y * z;
    const float wx = w * x, wy = w * y, wz = w * z;
    m[0] = 1.f - 2.f * (y2 + z2); m[1] = 2.f * (xy - wz);       m[2] = 2.f * (xz + wy);
    m[3] = 2.f * (xy + wz);       m[4] = 1.f - 2.f * (x2 + z2); m[5] = 2.f * (yz - wx);
    m[6] = 2.f * (xz - wy);       m[7] = 2.f * (yz + wx);       m[8] = 1.f - 2.f * (x2 + y2);
}

// ---------------------------------------------------------------------------------------------
// Camera models (global shutter): pinhole without distortion, OpenCV pinhole (radial, tangential, thin prism)
// and the OpenCV fisheye model.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool in_bounds_margin(float px, float py, const CamDev& c, float margin) {
    const float mx = (float)c.W * margin, my = (float)c.H * margin;
    bool valid = true;
    valid &= (-mx) <= px && px < ((float)c.W + mx);
    valid &= (-my) <= py && py < ((float)c.H + my);
    return valid;
}

__device__ __forceinline__ float stable_norm2(float x, float y) {
    const float ax = fabsf(x), ay = fabsf(y);
    const float mn = fminf(ax, ay), mx = fmaxf(ax, ay);
    if (mx <= 0.f) return 0.f;
    const float r = mn / mx;
    return mx * sqrtf(1.f + r * r);
}

__device__ __forceinline__ float fisheye_poly_odd(const float* k, float x) {
    const float x2 = x * x;
    float y = 0.f;
    y = x2 * y + k[3];
    y = x2 * y + k[2];
    y = x2 * y + k[1];
    y = x2 * y + k[0];
    y = x2 * y + 1.f;
    return x * y;
}
__device__ __forceinline__ float fisheye_dpoly_even(const float* k, float x) {
    const float x2 = x * x;
    float y = 0.f;
    y = x2 * y + 9 * k[3];
    y = x2 * y + 7 * k[2];
    y = x2 * y + 5 * k[1];
    y = x2 * y + 3 * k[0];
    y = x2 * y + 1.f;
    return y;
}

// Camera-space point -> image point. Returns validity (inside the image with margin, in front
// of the camera, inside the fisheye cone). atan2 is evaluated in double and rounded so that a
// host evaluation of the same expression gives the same float.
// OpenCV pinhole distortion of a normalised point (gsplat/Cameras.cuh:504-533): radial factor and
// tangential + thin-prism offset.
__device__ __forceinline__ void opencv_distortion(const CamDev& c, float u, float v, float& icD, float& dx, float& dy) {
    const float* k = c.dist;
    const float u2 = u * u, v2 = v * v;
    const float r2 = u2 + v2;
    const float a1 = 2.f * u * v;
    const float a2 = r2 + 2.f * u2;
    const float a3 = r2 + 2.f * v2;
    const float num = 1.f + r2 * (k[0] + r2 * (k[1] + r2 * k[2]));
    const float den = 1.f + r2 * (k[3] + r2 * (k[4] + r2 * k[5]));
    icD = num / den;
    dx = k[6] * a1 + k[7] * a2 + r2 * (k[8] + r2 * k[9]);
    dy = k[6] * a3 + k[7] * a1 + r2 * (k[10] + r2 * k[11]);
}

template <int MODEL>
__device__ __forceinline__ bool cam_point_to_image(const CamDev& c, f3 p, float margin, float& ox, float& oy) {
    ox = 0.f; oy = 0.f;
    if (MODEL == LFS_EQUIRECTANGULAR) {
        // gsplat/Cameras.cuh:1013-1026: azimuth / elevation of the camera-space point, the whole sphere on the image; the
        // reference computes the bounds check and then reports every point valid, behind the camera included
        const float azimuth = atan2f(p.x, p.z);
        const float elevation = asinf(p.y / sqrtf(p.x * p.x + p.y * p.y + p.z * p.z));
        ox = (azimuth / (2.0f * 3.14159265358979323846f) + 0.5f) * (float)c.W;
        oy = (elevation / 3.14159265358979323846f + 0.5f) * (float)c.H;
        return true;
    }
    if (p.z <= 0.f) return false;
    if (MODEL == LFS_PINHOLE_OPENCV) {
        // gsplat/Cameras.cuh:535-597: points whose radial factor comes close to flipping are invalid
        const float u = p.x / p.z, v = p.y / p.z;
        float icD, dx, dy;
        opencv_distortion(c, u, v, icD, dx, dy);
        ox = (icD * u + dx) * c.fx + c.cx;
        oy = (icD * v + dy) * c.fy + c.cy;
        return icD > 0.8f && in_bounds_margin(ox, oy, c, margin);
    } else if (MODEL == LFS_PINHOLE) {
        ox = (p.x / p.z) * c.fx + c.cx;
        oy = (p.y / p.z) * c.fy + c.cy;
        return in_bounds_margin(ox, oy, c, margin);
    } else {
        float n = stable_norm2(p.x, p.y);
        if (n <= 0.f) n = FLT_EPSILON;
        const float theta_full = (float)atan2((double)n, (double)p.z);
        const float theta = theta_full < c.max_angle ? theta_full : c.max_angle;
        const float delta = fisheye_poly_odd(c.k, theta) / n;
        if (delta <= 0.f) return false;
        ox = c.fx * delta * p.x + c.cx;
        oy = c.fy * delta * p.y + c.cy;
        bool valid = in_bounds_margin(ox, oy, c, margin);
        valid &= theta <= c.max_angle;
        return valid;
    }
}

// Pixel centre -> unit camera ray. Fisheye inverts the forward polynomial with up to 20 Newton steps.
template <int MODEL>
__device__ __forceinline__ bool image_to_cam_ray(const CamDev& c, float px, float py, f3& ray) {
    if (MODEL == LFS_EQUIRECTANGULAR) {
        // gsplat/Cameras.cuh:1028-1037: the angles and the trigonometry are double in the reference (2.0 * PI * ...)
        const double kPi = (double)3.14159265358979323846f;
        const double azimuth = 2.0 * kPi * (px / (float)c.W - 0.5);
        const double elevation = kPi * (py / (float)c.H - 0.5);
        const float dx = (float)(cos(elevation) * sin(azimuth));
        const float dy = (float)sin(elevation);
        const float dz = (float)(cos(azimuth) * cos(elevation));
        const float len = sqrtf(dx * dx + dy * dy + dz * dz);
        ray = {dx / len, dy / len, dz / len};
        return true;
    }
    const float ux = (px - c.cx) / c.fx;
    const float uy = (py - c.cy) / c.fy;
    if (MODEL == LFS_PINHOLE_OPENCV) {
        // Newton inversion of the distortion, at most 5 steps (gsplat/Cameras.cuh:635-754). Once per pixel, so
        // the Jacobian keeps the reference's mixed float / double literal arithmetic.
        const float k1 = c.dist[0], k2 = c.dist[1], k3 = c.dist[2], k4 = c.dist[3], k5 = c.dist[4], k6 = c.dist[5];
        const float p1 = c.dist[6], p2 = c.dist[7], s1 = c.dist[8], s2 = c.dist[9], s3 = c.dist[10], s4 = c.dist[11];
        const float xd = ux, yd = uy;
        float x = xd, y = yd;
        bool converged = false;
        for (int iter = 0; iter < 5; ++iter) {
            const float r = x * x + y * y;
            const float r2 = r * r;
            const float alpha = 1.0f + r * (k1 + r * (k2 + r * k3));
            const float beta = 1.0f + r * (k4 + r * (k5 + r * k6));
            const float d = alpha / beta;
            if (d <= 0.f) break;
            const float fx = d * x + 2 * p1 * x * y + p2 * (r + 2 * x * x) + s1 * r + s2 * r2 - xd;
            const float fy = d * y + 2 * p2 * x * y + p1 * (r + 2 * y * y) + s3 * r + s4 * r2 - yd;
            const float alpha_r = (float)(k1 + r * (2.0 * k2 + r * (3.0 * k3)));
            const float beta_r = (float)(k4 + r * (2.0 * k5 + r * (3.0 * k6)));
            const float d_r = (alpha_r * beta - alpha * beta_r) / (beta * beta);
            const float d_x = (float)(2.0 * x * d_r);
            const float d_y = (float)(2.0 * y * d_r);
            float fx_x = (float)(d + d_x * x + 2.0 * p1 * y + 6.0 * p2 * x);
            fx_x = (float)(fx_x + 2.0 * x * (s1 + 2.0 * s2 * r));
            float fx_y = (float)(d_y * x + 2.0 * p1 * x + 2.0 * p2 * y);
            fx_y = (float)(fx_y + 2.0 * y * (s1 + 2.0 * s2 * r));
            float fy_x = (float)(d_x * y + 2.0 * p2 * y + 2.0 * p1 * x);
            fy_x = (float)(fy_x + 2.0 * x * (s3 + 2.0 * s4 * r));
            float fy_y = (float)(d + d_y * y + 2.0 * p2 * x + 6.0 * p1 * y);
            fy_y = (float)(fy_y + 2.0 * y * (s3 + 2.0 * s4 * r));
            const float det = fx_y * fy_x - fx_x * fy_y;
            if (fabsf(det) < 1e-6f) break;
            const float dx = (fx * fy_y - fy * fx_y) / det;
            const float dy = (fy * fx_x - fx * fy_x) / det;
            x += dx;
            y += dy;
            if (fabsf(dx) < 1e-6f && fabsf(dy) < 1e-6f) { converged = true; break; }
        }
        const float len = sqrtf(x * x + y * y + 1.f);
        ray = {x / len, y / len, 1.f / len};
        return converged;
    } else if (MODEL == LFS_PINHOLE) {
        const float len = sqrtf(ux * ux + uy * uy + 1.f);
        ray = {ux / len, uy / len, 1.f / len};
        return true;
    } else {
        const float delta = sqrtf(ux * ux + uy * uy);
        bool converged = false;
        float x = delta * c.approx_b1 + 0.f;
        for (int j = 0; j < 20; ++j) {
            const float dfdx = fisheye_dpoly_even(c.k, x);
            const float residual = fisheye_poly_odd(c.k, x) - delta;
            const float dx = residual / dfdx;
            x -= dx;
            if (fabsf(dx) < 1e-6f) { converged = true; break; }
        }
        const float theta = x;
        if (theta < 0.f || theta >= c.max_angle || !converged) { ray = {0.f, 0.f, 1.f}; return false; }
        if (delta >= 1e-6f) {
            const float sf = (float)sin((double)theta) / delta;
            ray = {sf * ux, sf * uy, (float)cos((double)theta)};
            return true;
        }
        ray = {0.f, 0.f, 1.f};
        return true;
    }
}

// World-space ray direction of a pixel centre.
template <int MODEL>
__device__ __forceinline__ bool pixel_world_dir(const CamDev& c, float px, float py, f3& d) {
    f3 cr;
    const bool valid = image_to_cam_ray<MODEL>(c, px, py, cr);
    d.x = c.Rinv[0] * cr.x + c.Rinv[1] * cr.y + c.Rinv[2] * cr.z;
    d.y = c.Rinv[3] * cr.x + c.Rinv[4] * cr.y + c.Rinv[5] * cr.z;
    d.z = c.Rinv[6] * cr.x + c.Rinv[7] * cr.y + c.Rinv[8] * cr.z;
    return valid;
}

// ---------------------------------------------------------------------------------------------
// Rolling shutter (gsplat/Cameras.cuh:33-71, :253-413): the pose is interpolated between a start and an end pose
// by the frame time of the image row / column.
// ---------------------------------------------------------------------------------------------
struct PoseQ { float w, x, y, z; f3 t; };

// glm::slerp; acos / sin through double and rounded once, like the host restatement
__device__ __forceinline__ void quat_slerp(float xw, float xx, float xy, float xz, float yw, float yx, float yy, float yz, float a,
                                           float& ow, float& ox, float& oy, float& oz) {
    float cosTheta = xx * yx + xy * yy + xz * yz + xw * yw;
    if (cosTheta < 0.f) { yw = -yw; yx = -yx; yy = -yy; yz = -yz; cosTheta = -cosTheta; }
    if (cosTheta > 1.f - FLT_EPSILON) {
        ow = xw * (1.f - a) + yw * a; ox = xx * (1.f - a) + yx * a; oy = xy * (1.f - a) + yy * a; oz = xz * (1.f - a) + yz * a;
        return;
    }
    const float angle = (float)acos((double)cosTheta);
    const float s0 = (float)sin((double)((1.f - a) * angle)), s1 = (float)sin((double)(a * angle)), sn = (float)sin((double)angle);
    ow = (s0 * xw + s1 * yw) / sn; ox = (s0 * xx + s1 * yx) / sn; oy = (s0 * xy + s1 * yy) / sn; oz = (s0 * xz + s1 * yz) / sn;
}

__device__ __forceinline__ PoseQ shutter_pose(const CamDev& c, float t) {
    PoseQ p;
    if (!c.has_end) { p.w = c.qw; p.x = c.qx; p.y = c.qy; p.z = c.qz; p.t = f3{c.tx, c.ty, c.tz}; return p; }
    p.t = (1.f - t) * f3{c.tx, c.ty, c.tz} + t * f3{c.t1x, c.t1y, c.t1z};
    quat_slerp(c.qw, c.qx, c.qy, c.qz, c.q1w, c.q1x, c.q1y, c.q1z, t, p.w, p.x, p.y, p.z);
    return p;
}

__device__ __forceinline__ float shutter_time(const CamDev& c, float px, float py) {
    switch (c.rs_type) {
        case 0: return floorf(py) / (float)(c.H - 1);
        case 1: return floorf(px) / (float)(c.W - 1);
        case 2: return ((float)c.H - ceilf(py)) / (float)(c.H - 1);
        case 3: return ((float)c.W - ceilf(px)) / (float)(c.W - 1);
        default: return 0.f;
    }
}

// World point -> image point. RS = false: the start pose. RS = true: start (else end) projection as the initial
// guess, then ten rounds of pixel -> frame time -> pose -> projection (Cameras.cuh:346-413).
template <int MODEL, bool RS>
__device__ __forceinline__ bool world_point_to_image(const CamDev& c, f3 world, float margin, float& ox, float& oy) {
    const f3 t0{c.tx, c.ty, c.tz};
    const bool v0 = cam_point_to_image<MODEL>(c, quat_rotate(c.qw, c.qx, c.qy, c.qz, world) + t0, margin, ox, oy);
    if (!RS || c.rs_type == LFS_SHUTTER_GLOBAL) return v0;
    float ex, ey;
    const bool v1 = cam_point_to_image<MODEL>(c, quat_rotate(c.q1w, c.q1x, c.q1y, c.q1z, world) + f3{c.t1x, c.t1y, c.t1z}, margin, ex, ey);
    if (!v0) {
        ox = ex; oy = ey;
        if (!v1) return false;
    }
    for (int j = 0; j < 10; ++j) {
        const PoseQ p = shutter_pose(c, shutter_time(c, ox, oy));
        cam_point_to_image<MODEL>(c, quat_rotate(p.w, p.x, p.y, p.z, world) + p.t, margin, ox, oy);
    }
    return true;
}

// Rolling-shutter pixel ray: direction and the offset of its origin from the start-pose origin c.ro
// (image_point_to_world_ray_shutter_pose, Cameras.cuh:322-339).
template <int MODEL>
__device__ __forceinline__ bool pixel_world_ray_rs(const CamDev& c, float px, float py, f3& d, f3& origin_offset) {
    f3 cr;
    const bool valid = image_to_cam_ray<MODEL>(c, px, py, cr);
    const PoseQ p = shutter_pose(c, shutter_time(c, px, py));
    const float dq = p.x * p.x + p.y * p.y + p.z * p.z + p.w * p.w;
    float Ri[9];
    quat_to_mat_unit(p.w / dq, -p.x / dq, -p.y / dq, -p.z / dq, Ri);
    d.x = Ri[0] * cr.x + Ri[1] * cr.y + Ri[2] * cr.z;
    d.y = Ri[3] * cr.x + Ri[4] * cr.y + Ri[5] * cr.z;
    d.z = Ri[6] * cr.x + Ri[7] * cr.y + Ri[8] * cr.z;
    origin_offset.x = ((-Ri[0]) * p.t.x + (-Ri[1]) * p.t.y + (-Ri[2]) * p.t.z) - c.ro[0];
    origin_offset.y = ((-Ri[3]) * p.t.x + (-Ri[4]) * p.t.y + (-Ri[5]) * p.t.z) - c.ro[1];
    origin_offset.z = ((-Ri[6]) * p.t.x + (-Ri[7]) * p.t.y + (-Ri[8]) * p.t.z) - c.ro[2];
    return valid;
}

// ---------------------------------------------------------------------------------------------
// Real SH basis up to degree 4 at a direction that is normalised here (Sloan's recurrences).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void sh_basis(int degree, float dx, float dy, float dz, float* B) {
    B[0] = 0.2820947917738781f;
    if (degree < 1) return;
    const float inorm = rsqrtf(dx * dx + dy * dy + dz * dz);
    const float x = dx * inorm, y = dy * inorm, z = dz * inorm;
    B[1] = -0.48860251190292f * y;
    B[2] = 0.48860251190292f * z;
    B[3] = -0.48860251190292f * x;
    if (degree < 2) return;
    const float z2 = z * z;
    const float fTmp0B = -1.092548430592079f * z;
    const float fC1 = x * x - y * y;
    const float fS1 = 2.f * x * y;
    B[6] = (0.9461746957575601f * z2 - 0.3153915652525201f);
    B[7] = fTmp0B * x;
    B[5] = fTmp0B * y;
    B[8] = 0.5462742152960395f * fC1;
    B[4] = 0.5462742152960395f * fS1;
    if (degree < 3) return;
    const float fTmp0C = -2.285228997322329f * z2 + 0.4570457994644658f;
    const float fTmp1B = 1.445305721320277f * z;
    const float fC2 = x * fC1 - y * fS1;
    const float fS2 = x * fS1 + y * fC1;
    B[12] = z * (1.865881662950577f * z2 - 1.119528997770346f);
    B[13] = fTmp0C * x;
    B[11] = fTmp0C * y;
    B[14] = fTmp1B * fC1;
    B[10] = fTmp1B * fS1;
    B[15] = -0.5900435899266435f * fC2;
    B[9] = -0.5900435899266435f * fS2;
    if (degree < 4) return;
    const float fTmp0D = z * (-4.683325804901025f * z2 + 2.007139630671868f);
    const float fTmp1C = 3.31161143515146f * z2 - 0.47308734787878f;
    const float fTmp2B = -1.770130769779931f * z;
    const float fC3 = x * fC2 - y * fS2;
    const float fS3 = x * fS2 + y * fC2;
    B[20] = (1.984313483298443f * z * B[12] - 1.006230589874905f * B[6]);
    B[21] = fTmp0D * x;
    B[19] = fTmp0D * y;
    B[22] = fTmp1C * fC1;
    B[18] = fTmp1C * fS1;
    B[23] = fTmp2B * fC2;
    B[17] = fTmp2B * fS2;
    B[24] = 0.6258357354491763f * fC3;
    B[16] = 0.6258357354491763f * fS3;
}

// Tile rectangle covered by a projected Gaussian: [x0,x1) x [y0,y1) in tile units. The float ->
// unsigned conversion saturates (negative -> 0), which is what clips boxes that start left of /
// above the image.
__device__ __forceinline__ void tile_rect(float mx, float my, int rx, int ry, float tile_size, uint32_t tw,
                                          uint32_t th, uint32_t& x0, uint32_t& y0, uint32_t& x1, uint32_t& y1) {
    const float trx = (float)rx / tile_size, try_ = (float)ry / tile_size;
    const float tx = mx / tile_size, ty = my / tile_size;
    x0 = min((uint32_t)floorf(tx - trx), tw);
    y0 = min((uint32_t)floorf(ty - try_), th);
    x1 = min((uint32_t)ceilf(tx + trx), tw);
    y1 = min((uint32_t)ceilf(ty + try_), th);
}

}  // namespace lfs
