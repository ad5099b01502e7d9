// TEST INFRASTRUCTURE — not product code.
//
// Scalar CPU restatement of the LichtFeld Studio Gaussian-splatting training-step
// operators (the gsplat/3DGUT path). It exists only so that tests, the smoke check
// and the benchmark's CPU baseline can check / time-compare the CUDA library.
// Nothing in the shipped library links or calls this file.
//
// Parity status: PARITY UNPINNED by the reference's own tests. The reference has no
// golden vectors, known-answer tests or fixtures for any operator on this path
// (tests/test_render_modes.cpp checks shapes only), and it has no CPU
// implementation, so this restatement is pinned only by hand-derived analytic cases,
// finite-difference gradient checks and self-consistency, not by reference outputs.
//
// Third-party arithmetic that is not part of the reference tree and is restated
// here from its published definition: glm (vcpkg baseline 4334d8b4c8, version
// not resolvable offline) — quat_cast, quat*vec3 rotate, mat3_cast, inverse(quat),
// inverse(mat2), outerProduct, column-major mat*vec.
//
// Every function cites the reference file:line it follows (paths are relative to
// the reference project root). Arithmetic is IEEE float32 in the reference's
// operation order; this file must be compiled with -ffp-contract=off and without
// -ffast-math so that +,-,*,/,sqrt are correctly rounded single operations.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -fopenmp -shared -fPIC lfs_oracle.cpp

#include <algorithm>
#include <array>
#include <limits>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

struct V2 { float x, y; };
struct V3 { float x, y, z; };
struct Q4 { float w, x, y, z; };
// Math-convention 3x3 matrix, m[row][col].
struct M3 { float m[3][3]; };

inline V3 operator+(V3 a, V3 b) { return {a.x + b.x, a.y + b.y, a.z + b.z}; }
inline V3 operator-(V3 a, V3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
inline V3 operator*(V3 a, float s) { return {a.x * s, a.y * s, a.z * s}; }
inline V3 operator*(float s, V3 a) { return {a.x * s, a.y * s, a.z * s}; }
inline float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
// glm::cross: (x.y*y.z - y.y*x.z, x.z*y.x - y.z*x.x, x.x*y.y - y.x*x.y)
inline V3 cross(V3 a, V3 b) {
    return {a.y * b.z - b.y * a.z, a.z * b.x - b.z * a.x, a.x * b.y - b.x * a.y};
}
// glm mat*vec for a math matrix m[row][col]: row r = m[r][0]*v.x + m[r][1]*v.y + m[r][2]*v.z
inline V3 mul(const M3& a, V3 v) {
    return {a.m[0][0] * v.x + a.m[0][1] * v.y + a.m[0][2] * v.z,
            a.m[1][0] * v.x + a.m[1][1] * v.y + a.m[1][2] * v.z,
            a.m[2][0] * v.x + a.m[2][1] * v.y + a.m[2][2] * v.z};
}

// glm::quat_cast(mat3) restated for a math-convention rotation R[row][col]
// (glm m[c][r] == R[r][c]). Call site: gsplat/Cameras.cuh:42-51.
inline Q4 quat_cast(const float* se3 /* row-major 4x4 */) {
    const float R00 = se3[0], R01 = se3[1], R02 = se3[2];
    const float R10 = se3[4], R11 = se3[5], R12 = se3[6];
    const float R20 = se3[8], R21 = se3[9], R22 = se3[10];
    const float fx = R00 - R11 - R22;
    const float fy = R11 - R00 - R22;
    const float fz = R22 - R00 - R11;
    const float fw = R00 + R11 + R22;
    int big = 0;
    float fb = fw;
    if (fx > fb) { fb = fx; big = 1; }
    if (fy > fb) { fb = fy; big = 2; }
    if (fz > fb) { fb = fz; big = 3; }
    const float bv = std::sqrt(fb + 1.0f) * 0.5f;
    const float mult = 0.25f / bv;
    // glm m[1][2] = R21, m[2][1] = R12, m[2][0] = R02, m[0][2] = R20, m[0][1] = R10, m[1][0] = R01
    switch (big) {
    case 0: return {bv, (R21 - R12) * mult, (R02 - R20) * mult, (R10 - R01) * mult};
    case 1: return {(R21 - R12) * mult, bv, (R10 + R01) * mult, (R02 + R20) * mult};
    case 2: return {(R02 - R20) * mult, (R10 + R01) * mult, bv, (R21 + R12) * mult};
    default: return {(R10 - R01) * mult, (R02 + R20) * mult, (R21 + R12) * mult, bv};
    }
}

// glm operator*(quat, vec3), used as glm::rotate(q, v). Call sites: Cameras.cuh:364,
// ProjectionUT3DGSFused.cu:77.
inline V3 quat_rotate(Q4 q, V3 v) {
    const V3 qv{q.x, q.y, q.z};
    const V3 uv = cross(qv, v);
    const V3 uuv = cross(qv, uv);
    return v + ((uv * q.w) + uuv) * 2.0f;
}

// glm::mat3_cast(quat) as a math matrix (glm Result[c][r] -> m[r][c]).
inline M3 mat3_cast(Q4 q) {
    const float qxx = q.x * q.x, qyy = q.y * q.y, qzz = q.z * q.z;
    const float qxz = q.x * q.z, qxy = q.x * q.y, qyz = q.y * q.z;
    const float qwx = q.w * q.x, qwy = q.w * q.y, qwz = q.w * q.z;
    M3 r;
    r.m[0][0] = 1.0f - 2.0f * (qyy + qzz);
    r.m[1][0] = 2.0f * (qxy + qwz);
    r.m[2][0] = 2.0f * (qxz - qwy);
    r.m[0][1] = 2.0f * (qxy - qwz);
    r.m[1][1] = 1.0f - 2.0f * (qxx + qzz);
    r.m[2][1] = 2.0f * (qyz + qwx);
    r.m[0][2] = 2.0f * (qxz + qwy);
    r.m[1][2] = 2.0f * (qyz - qwx);
    r.m[2][2] = 1.0f - 2.0f * (qxx + qyy);
    return r;
}

// glm::inverse(quat) = conjugate(q) / dot(q, q)
inline Q4 quat_inverse(Q4 q) {
    const float d = q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;  // glm dot order x,y,z,w
    return {q.w / d, -q.x / d, -q.y / d, -q.z / d};
}

// glm::normalize(quat): identity for zero length, else q * (1/len).
// Call site: ProjectionUT3DGSFused.cu:63.
inline Q4 quat_normalize(Q4 q) {
    const float len = std::sqrt(q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w);
    if (len <= 0.0f) return {1.0f, 0.0f, 0.0f, 0.0f};
    const float inv = 1.0f / len;
    return {q.w * inv, q.x * inv, q.y * inv, q.z * inv};
}

// gsplat/Utils.cuh:80-102 quat_to_rotmat (re-normalises with rsqrt).
inline M3 quat_to_rotmat(Q4 q) {
    float w = q.w, x = q.x, y = q.y, z = q.z;
    const float inv_norm = 1.0f / std::sqrt(x * x + y * y + z * z + w * w);
    x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
    const float x2 = x * x, y2 = y * y, z2 = z * z;
    const float xy = x * y, xz = x * z, yz = y * z;
    const float wx = w * x, wy = w * y, wz = w * z;
    M3 r;
    r.m[0][0] = 1.f - 2.f * (y2 + z2); r.m[0][1] = 2.f * (xy - wz);       r.m[0][2] = 2.f * (xz + wy);
    r.m[1][0] = 2.f * (xy + wz);       r.m[1][1] = 1.f - 2.f * (x2 + z2); r.m[1][2] = 2.f * (yz - wx);
    r.m[2][0] = 2.f * (xz - wy);       r.m[2][1] = 2.f * (yz + wx);       r.m[2][2] = 1.f - 2.f * (x2 + y2);
    return r;
}

struct Pose { Q4 q; V3 t; };

// RollingShutterParameters for a global shutter (Cameras.cuh:33-71): q = quat_cast(R),
// t = last column. slerp(q, q, a) of two identical quaternions is q, so the centre and
// start poses coincide (Cameras.cuh:268-280).
inline Pose pose_from_viewmat(const float* vm) {
    return {quat_cast(vm), V3{vm[3], vm[7], vm[11]}};
}

// ---- rolling shutter (Cameras.cuh:33-71, :253-413) ------------------------------------------------------
// ShutterType of gsplat/Cameras.h
enum Shutter { ROLLING_TOP_TO_BOTTOM = 0, ROLLING_LEFT_TO_RIGHT = 1, ROLLING_BOTTOM_TO_TOP = 2, ROLLING_RIGHT_TO_LEFT = 3, GLOBAL = 4 };

struct ShutterCtx {   // set by orc_set_shutter for the calls that follow (test infrastructure: one global context)
    bool has_end = false;
    float vm1[16] = {0};
    int type = GLOBAL;
};
ShutterCtx g_shutter;

struct RSPose { Pose start, end; bool has_end; int type; };

// glm::slerp(x, y, a). acos / sin go through double and are rounded once (the CUDA library does the same).
inline Q4 quat_slerp(Q4 x, Q4 y, float a) {
    Q4 z = y;
    float cosTheta = x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;   // glm dot order x, y, z, w
    if (cosTheta < 0.f) { z = {-y.w, -y.x, -y.y, -y.z}; cosTheta = -cosTheta; }
    if (cosTheta > 1.f - std::numeric_limits<float>::epsilon()) {
        auto mix = [a](float u, float v) { return u * (1.f - a) + v * a; };
        return {mix(x.w, z.w), mix(x.x, z.x), mix(x.y, z.y), mix(x.z, z.z)};
    }
    const float angle = (float)std::acos((double)cosTheta);
    const float s0 = (float)std::sin((double)((1.f - a) * angle)), s1 = (float)std::sin((double)(a * angle));
    const float sn = (float)std::sin((double)angle);
    return {(s0 * x.w + s1 * z.w) / sn, (s0 * x.x + s1 * z.x) / sn, (s0 * x.y + s1 * z.y) / sn, (s0 * x.z + s1 * z.z) / sn};
}

// interpolate_shutter_pose (Cameras.cuh:268-280). Without an end pose both poses coincide and the start pose is
// returned unchanged (slerp(q, q, a) is taken as q).
inline Pose shutter_pose(const RSPose& rs, float t) {
    if (!rs.has_end) return rs.start;
    const V3 tr = (1.f - t) * rs.start.t + t * rs.end.t;
    return {quat_slerp(rs.start.q, rs.end.q, t), tr};
}

enum CameraModel { PINHOLE = 0, ORTHO = 1, FISHEYE = 2, EQUIRECTANGULAR = 3 };

struct Camera {
    int model;
    float fx, fy, cx, cy;
    uint32_t W, H;
    // fisheye (Cameras.cuh:830-885)
    float k[4];
    float max_angle;
    float approx_b1;  // approx_backward_poly = {0, approx_b1}
    // OpenCV pinhole distortion (Cameras.cuh:481-486): used when `distorted`
    bool distorted;
    float radial[6], tangential[2], thin_prism[4];
};

inline float numerically_stable_norm2(float x, float y) {  // Cameras.cuh:77-89
    const float ax = std::fabs(x), ay = std::fabs(y);
    const float mn = std::fmin(ax, ay), mx = std::fmax(ax, ay);
    if (mx <= 0.f) return 0.f;
    const float r = mn / mx;
    return mx * std::sqrt(1.f + r * r);
}

// Cameras.cuh:760-815 compute_opencv_fisheye_max_angle, only the branches reachable
// with k4 == 0.
float fisheye_max_angle_poly(float a, float b, float c) {
    const float INF = std::numeric_limits<float>::max();
    const float PI = 3.14159265358979323846f;
    if (c == 0.0f) {
        if (b == 0.0f) {
            if (a >= 0.0f) return INF;
            return -1.0f / a;
        }
        float delta = a * a - 4.0f * b;
        if (delta >= 0.0f) {
            delta = std::sqrt(delta) - a;
            if (delta > 0.0f) return 2.0f / delta;
        }
    } else {
        const float boc = b / c;
        const float boc2 = boc * boc;
        const float t1 = (9.0f * a * boc - 2.0f * b * boc2 - 27.0f) / c;
        const float t2 = 3.0f * a / c - boc2;
        const float delta = t1 * t1 + 4.0f * t2 * t2 * t2;
        if (delta >= 0.0f) {
            const float d2 = std::sqrt(delta);
            const float cube_root = std::cbrt((d2 + t1) / 2.0f);
            if (cube_root != 0.0f) {
                const float soln = (cube_root - (t2 / cube_root) - boc) / 3.0f;
                if (soln > 0.0f) return soln;
            }
        } else {
            const float theta = std::atan2(std::sqrt(-delta), t1) / 3.0f;
            const float two_third_pi = 2.0f * PI / 3.0f;
            const float t3 = 2.0f * std::sqrt(-t2);
            float soln = INF;
            for (int i : {-1, 0, 1}) {
                const float angle = theta + i * two_third_pi;
                const float s = (t3 * std::cos(angle) - boc) / 3.0f;
                if (s > 0.0f) soln = std::min(soln, s);
            }
            return soln;
        }
    }
    return INF;
}

Camera make_camera(int model, const float* K, uint32_t W, uint32_t H, const float* radial) {
    Camera c{};
    c.model = model;
    c.fx = K[0]; c.fy = K[4]; c.cx = K[2]; c.cy = K[5];
    c.W = W; c.H = H;
    // `radial` is model dependent: FISHEYE -> 4 radial coefficients; PINHOLE -> 12 floats
    // (k1..k6, p1, p2, s1..s4), whose presence selects OpenCVPinholeCameraModel like any of the three optional
    // tensors does in gsplat/ProjectionUT3DGSFused.cu:91-113
    if (model == PINHOLE && radial) {
        c.distorted = true;
        for (int i = 0; i < 6; ++i) c.radial[i] = radial[i];
        for (int i = 0; i < 2; ++i) c.tangential[i] = radial[6 + i];
        for (int i = 0; i < 4; ++i) c.thin_prism[i] = radial[8 + i];
    }
    for (int i = 0; i < 4; ++i) c.k[i] = (radial && model == FISHEYE) ? radial[i] : 0.f;
    if (model == FISHEYE) {
        const float mdx = std::max((float)W - c.cx, c.cx);
        const float mdy = std::max((float)H - c.cy, c.cy);
        const float max_radius_pixels = std::sqrt(mdx * mdx + mdy * mdy);
        float max_angle;
        if (c.k[3] == 0.f) {
            max_angle = std::sqrt(fisheye_max_angle_poly(3.f * c.k[0], 5.f * c.k[1], 7.f * c.k[2]));
        } else {
            max_angle = std::numeric_limits<float>::max();  // k4 != 0 is outside the covered scope
        }
        max_angle = std::min(max_angle, std::max(max_radius_pixels / c.fx, max_radius_pixels / c.fy));
        c.max_angle = max_angle;
        const float max_norm_dist = std::max((float)W / 2.f / c.fx, (float)H / 2.f / c.fy);
        c.approx_b1 = max_angle / max_norm_dist;
    }
    return c;
}

inline bool in_bounds_margin(V2 p, const Camera& c, float margin) {  // Cameras.cuh:228-240
    const float mx = (float)c.W * margin, my = (float)c.H * margin;
    bool valid = true;
    valid &= (-mx) <= p.x && p.x < ((float)c.W + mx);
    valid &= (-my) <= p.y && p.y < ((float)c.H + my);
    return valid;
}

inline float poly_odd5(const float* k, float x) {  // x*(1 + k1 x^2 + ... ) Horner, Cameras.cuh:93-124
    const float x2 = x * x;
    float y = 0.f;
    const float co[5] = {1.f, k[0], k[1], k[2], k[3]};
    for (int i = 4; i >= 0; --i) y = x2 * y + co[i];
    return x * y;
}
inline float poly_even5_d(const float* k, float x) {  // 1 + 3k1 x^2 + 5k2 x^4 + ...
    const float x2 = x * x;
    float y = 0.f;
    const float co[5] = {1.f, 3 * k[0], 5 * k[1], 7 * k[2], 9 * k[3]};
    for (int i = 4; i >= 0; --i) y = x2 * y + co[i];
    return y;
}

inline RSPose rs_from_viewmat(const float* vm) {
    RSPose r;
    r.start = pose_from_viewmat(vm);
    r.has_end = g_shutter.has_end;
    r.end = g_shutter.has_end ? pose_from_viewmat(g_shutter.vm1) : r.start;
    r.type = g_shutter.type;
    return r;
}

// shutter_relative_frame_time (Cameras.cuh:293-320)
inline float shutter_time(int type, float px, float py, uint32_t W, uint32_t H) {
    switch (type) {
    case ROLLING_TOP_TO_BOTTOM: return std::floor(py) / (float)(H - 1);
    case ROLLING_LEFT_TO_RIGHT: return std::floor(px) / (float)(W - 1);
    case ROLLING_BOTTOM_TO_TOP: return ((float)H - std::ceil(py)) / (float)(H - 1);
    case ROLLING_RIGHT_TO_LEFT: return ((float)W - std::ceil(px)) / (float)(W - 1);
    default: return 0.f;
    }
}

// camera_ray_to_image_point. Pinhole: Cameras.cuh:431-455. Fisheye: :894-959.
// The two transcendental calls of the fisheye model (atan2) are evaluated in double and
// rounded to float: the CUDA library does the same so that both sides agree bit for bit.
// OpenCVPinholeCameraModel::compute_distortion, Cameras.cuh:504-533
inline void opencv_distortion(const Camera& c, float u, float v, float& icD, float& dx, float& dy) {
    const float u2 = u * u, v2 = v * v;
    const float r2 = u2 + v2;
    const float a1 = 2.f * u * v;
    const float a2 = r2 + 2.f * u2;
    const float a3 = r2 + 2.f * v2;
    const float num = 1.f + r2 * (c.radial[0] + r2 * (c.radial[1] + r2 * c.radial[2]));
    const float den = 1.f + r2 * (c.radial[3] + r2 * (c.radial[4] + r2 * c.radial[5]));
    icD = num / den;
    dx = c.tangential[0] * a1 + c.tangential[1] * a2 + r2 * (c.thin_prism[0] + r2 * c.thin_prism[1]);
    dy = c.tangential[0] * a3 + c.tangential[1] * a1 + r2 * (c.thin_prism[2] + r2 * c.thin_prism[3]);
}

inline bool cam_point_to_image(const Camera& c, V3 p, float margin, V2& out) {
    out = {0.f, 0.f};
    if (c.model == PINHOLE && c.distorted) {  // Cameras.cuh:535-597
        if (p.z <= 0.f) return false;
        const float u = p.x / p.z, v = p.y / p.z;
        float icD, dx, dy;
        opencv_distortion(c, u, v, icD, dx, dy);
        const bool valid_radial = icD > 0.8f;
        out.x = (icD * u + dx) * c.fx + c.cx;
        out.y = (icD * v + dy) * c.fy + c.cy;
        return valid_radial && in_bounds_margin(out, c, margin);
    }
    if (c.model == PINHOLE) {
        if (p.z <= 0.f) return false;
        out.x = (p.x / p.z) * c.fx + c.cx;
        out.y = (p.y / p.z) * c.fy + c.cy;
        return in_bounds_margin(out, c, margin);
    }
    if (c.model == EQUIRECTANGULAR) {
        // EquirectangularCameraModel::camera_ray_to_image_point (Cameras.cuh:1013-1026): azimuth / elevation of the point,
        // the whole sphere on the image; the bounds check is computed and dropped, every point is valid
        const float kPi = 3.14159265358979323846f;
        const float azimuth = std::atan2(p.x, p.z);
        const float elevation = std::asin(p.y / std::sqrt(p.x * p.x + p.y * p.y + p.z * p.z));
        out.x = (azimuth / (2.0f * kPi) + 0.5f) * (float)c.W;
        out.y = (elevation / kPi + 0.5f) * (float)c.H;
        return true;
    }
    if (c.model == FISHEYE) {
        if (p.z <= 0.f) return false;
        float n = numerically_stable_norm2(p.x, p.y);
        if (n <= 0.f) n = std::numeric_limits<float>::epsilon();
        const float theta_full = (float)std::atan2((double)n, (double)p.z);
        const float theta = theta_full < c.max_angle ? theta_full : c.max_angle;
        const float delta = poly_odd5(c.k, theta) / n;
        if (delta <= 0.f) return false;
        out.x = c.fx * delta * p.x + c.cx;
        out.y = c.fy * delta * p.y + c.cy;
        bool valid = in_bounds_margin(out, c, margin);
        valid &= theta <= c.max_angle;
        return valid;
    }
    return false;
}

// image_point_to_camera_ray. Pinhole: Cameras.cuh:457-470. Fisheye: :961-1000 with
// eval_poly_inverse_horner_newton<20> (:169-206).
inline bool image_to_cam_ray(const Camera& c, float px, float py, V3& ray) {
    if (c.model == EQUIRECTANGULAR) {
        // image_point_to_camera_ray (Cameras.cuh:1028-1037): the literals 2.0 and 0.5 make the angles and the trigonometry
        // double; the direction is rounded to float and normalised
        const double kPi = (double)3.14159265358979323846f;
        const double azimuth = 2.0 * kPi * (px / (float)c.W - 0.5);
        const double elevation = kPi * (py / (float)c.H - 0.5);
        const float dx = (float)(std::cos(elevation) * std::sin(azimuth));
        const float dy = (float)std::sin(elevation);
        const float dz = (float)(std::cos(azimuth) * std::cos(elevation));
        const float len = std::sqrt(dx * dx + dy * dy + dz * dz);
        ray = {dx / len, dy / len, dz / len};
        return true;
    }
    const float ux = (px - c.cx) / c.fx;
    const float uy = (py - c.cy) / c.fy;
    if (c.model == PINHOLE && c.distorted) {
        // compute_undistortion_newton with at most 5 iterations (Cameras.cuh:635-754); the Jacobian expressions mix
        // float and double literals exactly as written there
        const float k1 = c.radial[0], k2 = c.radial[1], k3 = c.radial[2], k4 = c.radial[3], k5 = c.radial[4], k6 = c.radial[5];
        const float p1 = c.tangential[0], p2 = c.tangential[1];
        const float s1 = c.thin_prism[0], s2 = c.thin_prism[1], s3 = c.thin_prism[2], s4 = c.thin_prism[3];
        const float xd = ux, yd = uy;
        float x = xd, y = yd;
        const float eps = 1e-6f;
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
            if (std::fabs(det) < eps) break;
            const float dx = (fx * fy_y - fy * fx_y) / det;
            const float dy = (fy * fx_x - fx * fy_x) / det;
            x += dx;
            y += dy;
            if (std::fabs(dx) < eps && std::fabs(dy) < eps) { converged = true; break; }
        }
        const float len = std::sqrt(x * x + y * y + 1.f * 1.f);
        ray = {x / len, y / len, 1.f / len};
        return converged;
    }
    if (c.model == PINHOLE) {
        const float len = std::sqrt(ux * ux + uy * uy + 1.f * 1.f);
        ray = {ux / len, uy / len, 1.f / len};
        return true;
    }
    if (c.model == FISHEYE) {
        const float delta = std::sqrt(ux * ux + uy * uy);
        bool converged = false;
        float x = delta * c.approx_b1 + 0.f;  // Horner of {0, b1}: y = x*0 + b1; y = x*y + 0
        for (int j = 0; j < 20; ++j) {
            const float dfdx = poly_even5_d(c.k, x);
            const float residual = poly_odd5(c.k, x) - delta;
            const float dx = residual / dfdx;
            x -= dx;
            if (std::fabs(dx) < 1e-6f) { converged = true; break; }
        }
        const float theta = x;
        if (theta < 0.f || theta >= c.max_angle || !converged) { ray = {0.f, 0.f, 1.f}; return false; }
        if (delta >= 1e-6f) {
            const float sf = (float)std::sin((double)theta) / delta;
            ray = {sf * ux, sf * uy, (float)std::cos((double)theta)};
            return true;
        }
        ray = {0.f, 0.f, 1.f};
        return true;
    }
    ray = {0.f, 0.f, 1.f};
    return false;
}

// world_point_to_image_point_shutter_pose (Cameras.cuh:346-413): project with the start pose; for a rolling shutter
// take the start (else the end) projection as the initial guess and iterate 10 times pixel -> frame time -> pose ->
// projection. The result of the last iteration is returned as valid whatever its own validity was, as in the reference.
inline bool world_point_to_image(const Camera& c, const RSPose& rs, V3 world, float margin, V2& out) {
    V2 p0;
    const bool v0 = cam_point_to_image(c, quat_rotate(rs.start.q, world) + rs.start.t, margin, p0);
    if (rs.type == GLOBAL) { out = p0; return v0; }
    V2 p1;
    const bool v1 = cam_point_to_image(c, quat_rotate(rs.end.q, world) + rs.end.t, margin, p1);
    V2 prev;
    if (v0) prev = p0;
    else if (v1) prev = p1;
    else { out = p1; return false; }
    for (int j = 0; j < 10; ++j) {
        const float t = shutter_time(rs.type, prev.x, prev.y, c.W, c.H);
        const Pose ps = shutter_pose(rs, t);
        V2 pj;
        cam_point_to_image(c, quat_rotate(ps.q, world) + ps.t, margin, pj);
        prev = pj;
    }
    out = prev;
    return true;
}

}  // namespace

extern "C" {

// Rolling-shutter context for the calls that follow: viewmat1 (row-major 4x4 end-of-frame pose, may be null = same as
// the start pose) and the ShutterType (4 = GLOBAL). Not thread safe; tests set it, call, and reset it.
void orc_set_shutter(const float* viewmat1, int rs_type) {
    g_shutter.has_end = viewmat1 != nullptr;
    if (viewmat1) std::memcpy(g_shutter.vm1, viewmat1, 16 * sizeof(float));
    g_shutter.type = rs_type;
}

// ---------------------------------------------------------------------------------------------
// Projection: gsplat/ProjectionUT3DGSFused.cu:17-210, Cameras.cuh:1070-1186, Utils.cuh:171-179.
// Inputs are ACTIVATED quantities exactly as the operator receives them. Outputs for culled
// Gaussians are left untouched (the reference leaves them uninitialised) except radii = 0.
// ut = {alpha, beta, kappa, in_image_margin_factor, require_all_sigma_points_valid}.
// ---------------------------------------------------------------------------------------------
void orc_projection_ut_3dgs_fused(
    int C, int N,
    const float* means, const float* quats, const float* scales, const float* opacities /*nullable*/,
    const float* viewmats, const float* Ks, int W, int H,
    float eps2d, float near_plane, float far_plane, float radius_clip,
    int camera_model, const float* ut, const float* radial_coeffs /*nullable: fisheye [C,4]; pinhole [C,12] = k1..k6 p1 p2 s1..s4*/,
    int32_t* radii, float* means2d, float* depths, float* conics, float* compensations /*nullable*/) {
    const float alpha = ut[0], beta = ut[1], kappa = ut[2], margin = ut[3];
    const bool require_all = ut[4] != 0.f;
    const float ALPHA_THRESHOLD = 1.f / 255.f;
    for (int cid = 0; cid < C; ++cid) {
        const RSPose rs = rs_from_viewmat(viewmats + cid * 16);
        const Pose pose = shutter_pose(rs, 0.5f);   // centre-of-frame pose for depth and culling (ProjectionUT3DGSFused.cu:73-77)
        const Camera cam = make_camera(camera_model, Ks + cid * 9, W, H,
                                       radial_coeffs ? radial_coeffs + cid * (camera_model == PINHOLE ? 12 : 4) : nullptr);
#pragma omp parallel for schedule(static)
        for (int gid = 0; gid < N; ++gid) {
            const size_t idx = (size_t)cid * N + gid;
            auto cull = [&]() { radii[idx * 2] = 0; radii[idx * 2 + 1] = 0; };
            const V3 mean{means[gid * 3], means[gid * 3 + 1], means[gid * 3 + 2]};
            const V3 scale{scales[gid * 3], scales[gid * 3 + 1], scales[gid * 3 + 2]};
            const Q4 quat = quat_normalize(Q4{quats[gid * 4], quats[gid * 4 + 1], quats[gid * 4 + 2], quats[gid * 4 + 3]});
            const V3 mean_c = quat_rotate(pose.q, mean) + pose.t;
            if ((mean_c.z < near_plane && camera_model != EQUIRECTANGULAR) || mean_c.z > far_plane) { cull(); continue; }

            // sigma points, Cameras.cuh:1070-1119
            const float D = 3.0f;
            const float lambda = alpha * alpha * (D + kappa) - D;
            const M3 R = mat3_cast(quat);
            V3 pts[7];
            float wm[7], wc[7];
            pts[0] = mean;
            const float sq = std::sqrt(D + lambda);
            const float sc[3] = {scale.x, scale.y, scale.z};
            for (int i = 0; i < 3; ++i) {
                const float f = sq * sc[i];
                const V3 col{R.m[0][i], R.m[1][i], R.m[2][i]};
                const V3 delta = f * col;
                pts[i + 1] = mean + delta;
                pts[i + 4] = mean - delta;
            }
            wm[0] = lambda / (D + lambda);
            wc[0] = lambda / (D + lambda) + (1.0f - alpha * alpha + beta);
            for (int i = 0; i < 6; ++i) { wm[i + 1] = 1.0f / (2.0f * (D + lambda)); wc[i + 1] = wm[i + 1]; }

            // Cameras.cuh:1145-1185
            bool valid = require_all;
            V2 ip[7];
            V2 m2{0.f, 0.f};
            bool early = false;
            for (int i = 0; i < 7; ++i) {
                V2 p;
                const bool pv = world_point_to_image(cam, rs, pts[i], margin, p);
                if (require_all) {
                    valid &= pv;
                    if (!pv) { early = true; break; }
                } else {
                    valid |= pv;
                }
                ip[i] = p;
                m2.x += wm[i] * p.x;
                m2.y += wm[i] * p.y;
            }
            if (early || !valid) { cull(); continue; }
            float c00 = 0.f, c01 = 0.f, c11 = 0.f;
            for (int i = 0; i < 7; ++i) {
                const float dx = ip[i].x - m2.x, dy = ip[i].y - m2.y;
                c00 += wc[i] * (dx * dx);
                c01 += wc[i] * (dx * dy);
                c11 += wc[i] * (dy * dy);
            }
            // add_blur, Utils.cuh:171-179
            const float det_orig = c00 * c11 - c01 * c01;
            c00 += eps2d; c11 += eps2d;
            const float det = c00 * c11 - c01 * c01;
            const float compensation = std::sqrt(std::max(0.f, det_orig / det));
            if (det <= 0.f) { cull(); continue; }
            // glm::inverse(mat2)
            const float ood = 1.0f / (c00 * c11 - c01 * c01);
            const float i00 = c11 * ood, i01 = -c01 * ood, i11 = c00 * ood;

            float extend = 3.33f;
            if (opacities != nullptr) {
                float opacity = opacities[gid];
                opacity *= compensation;
                if (opacity < ALPHA_THRESHOLD) { cull(); continue; }
                // log evaluated in double, rounded to float (the CUDA library does the same)
                const float lg = (float)std::log((double)(opacity / ALPHA_THRESHOLD));
                extend = std::min(extend, std::sqrt(2.0f * lg));
            }
            const float b = 0.5f * (c00 + c11);
            const float tmp = std::sqrt(std::max(0.01f, b * b - det));
            const float v1 = b + tmp;
            const float r1 = extend * std::sqrt(v1);
            const float radius_x = std::ceil(std::min(extend * std::sqrt(c00), r1));
            const float radius_y = std::ceil(std::min(extend * std::sqrt(c11), r1));
            if (radius_x <= radius_clip && radius_y <= radius_clip) { cull(); continue; }
            if (m2.x + radius_x <= 0 || m2.x - radius_x >= (float)W || m2.y + radius_y <= 0 || m2.y - radius_y >= (float)H) { cull(); continue; }
            radii[idx * 2] = (int32_t)radius_x;
            radii[idx * 2 + 1] = (int32_t)radius_y;
            means2d[idx * 2] = m2.x;
            means2d[idx * 2 + 1] = m2.y;
            depths[idx] = mean_c.z;
            conics[idx * 3] = i00;
            conics[idx * 3 + 1] = i01;
            conics[idx * 3 + 2] = i11;
            if (compensations) compensations[idx] = compensation;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Spherical harmonics: gsplat/SphericalHarmonicsCUDA.cu:21-110 (forward), :113-371 (backward,
// v_dirs branch not restated: the training path calls it with compute_v_dirs=false,
// gsplat/Rasterization.cpp:620).
// ---------------------------------------------------------------------------------------------
static void sh_basis(int degree, float dx, float dy, float dz, float* B /*[25]*/) {
    B[0] = 0.2820947917738781f;
    if (degree < 1) return;
    const float inorm = 1.0f / std::sqrt(dx * dx + dy * dy + dz * dz);
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

void orc_spherical_harmonics_fwd(int n, int K, int degree, const float* dirs, const float* coeffs,
                                 const uint8_t* masks /*nullable*/, float* colors) {
#pragma omp parallel for schedule(static)
    for (int e = 0; e < n; ++e) {
        if (masks && !masks[e]) continue;
        float B[25];
        sh_basis(degree, dirs[e * 3], dirs[e * 3 + 1], dirs[e * 3 + 2], B);
        const float* cf = coeffs + (size_t)e * K * 3;
        for (int c = 0; c < 3; ++c) {
            // summation grouping of the reference: per-degree partial sums added to result
            float result = B[0] * cf[c];
            if (degree >= 1) {
                // 0.4886*(-y*c1 + z*c2 - x*c3); B already holds the products with the constant,
                // so regroup as the reference writes it
                const float inorm = 1.0f / std::sqrt(dirs[e * 3] * dirs[e * 3] + dirs[e * 3 + 1] * dirs[e * 3 + 1] + dirs[e * 3 + 2] * dirs[e * 3 + 2]);
                const float x = dirs[e * 3] * inorm, y = dirs[e * 3 + 1] * inorm, z = dirs[e * 3 + 2] * inorm;
                result += 0.48860251190292f * (-y * cf[1 * 3 + c] + z * cf[2 * 3 + c] - x * cf[3 * 3 + c]);
            }
            if (degree >= 2) {
                result += B[4] * cf[4 * 3 + c] + B[5] * cf[5 * 3 + c] + B[6] * cf[6 * 3 + c] + B[7] * cf[7 * 3 + c] + B[8] * cf[8 * 3 + c];
            }
            if (degree >= 3) {
                result += B[9] * cf[9 * 3 + c] + B[10] * cf[10 * 3 + c] + B[11] * cf[11 * 3 + c] + B[12] * cf[12 * 3 + c] +
                          B[13] * cf[13 * 3 + c] + B[14] * cf[14 * 3 + c] + B[15] * cf[15 * 3 + c];
            }
            if (degree >= 4) {
                result += B[16] * cf[16 * 3 + c] + B[17] * cf[17 * 3 + c] + B[18] * cf[18 * 3 + c] + B[19] * cf[19 * 3 + c] +
                          B[20] * cf[20 * 3 + c] + B[21] * cf[21 * 3 + c] + B[22] * cf[22 * 3 + c] + B[23] * cf[23 * 3 + c] +
                          B[24] * cf[24 * 3 + c];
            }
            colors[e * 3 + c] = result;
        }
    }
}

// v_coeffs must be pre-zeroed by the caller (the reference allocates zeros,
// gsplat/SphericalHarmonics.cpp:57); only (degree+1)^2 bases of unmasked elements are written.
void orc_spherical_harmonics_bwd(int n, int K, int degree, const float* dirs, const uint8_t* masks,
                                 const float* v_colors, float* v_coeffs) {
    const int nb = (degree + 1) * (degree + 1);
#pragma omp parallel for schedule(static)
    for (int e = 0; e < n; ++e) {
        if (masks && !masks[e]) continue;
        float B[25];
        sh_basis(degree, dirs[e * 3], dirs[e * 3 + 1], dirs[e * 3 + 2], B);
        float* vc = v_coeffs + (size_t)e * K * 3;
        for (int k = 0; k < nb; ++k)
            for (int c = 0; c < 3; ++c) vc[k * 3 + c] = B[k] * v_colors[e * 3 + c];
    }
}

// ---------------------------------------------------------------------------------------------
// Tile intersection: gsplat/IntersectTile.cu:24-113 (count / emit), gsplat/Intersect.cpp:41-121
// (bit widths, cumsum), IntersectTile.cu:290-328 (stable ascending sort over the low
// 32+tile_bits+cam_bits bits), IntersectTile.cu:206-252 (offsets).
// CUDA float->uint32 conversion saturates (negative -> 0); restated explicitly.
// ---------------------------------------------------------------------------------------------
static inline uint32_t f2u_sat(float f) {
    if (!(f > 0.f)) return 0u;  // negative, zero and NaN -> 0
    if (f >= 4294967296.f) return 0xffffffffu;
    return (uint32_t)f;
}

static inline void tile_range(const float* means2d, const int32_t* radii, size_t idx, uint32_t tile_size,
                              uint32_t tw, uint32_t th, uint32_t& x0, uint32_t& y0, uint32_t& x1, uint32_t& y1, bool& ok) {
    const float rx = (float)radii[idx * 2], ry = (float)radii[idx * 2 + 1];
    ok = !(rx <= 0 || ry <= 0);
    if (!ok) return;
    const float trx = rx / (float)tile_size, try_ = ry / (float)tile_size;
    const float tx = means2d[idx * 2] / (float)tile_size, ty = means2d[idx * 2 + 1] / (float)tile_size;
    x0 = std::min(f2u_sat(std::floor(tx - trx)), tw);
    y0 = std::min(f2u_sat(std::floor(ty - try_)), th);
    x1 = std::min(f2u_sat(std::ceil(tx + trx)), tw);
    y1 = std::min(f2u_sat(std::ceil(ty + try_)), th);
}

static inline uint32_t bit_width_floor_log2_plus1(uint32_t v) {  // (uint32_t)floor(log2(v)) + 1
    uint32_t b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

int64_t orc_intersect_count(int C, int N, const float* means2d, const int32_t* radii, uint32_t tile_size,
                            uint32_t tw, uint32_t th, int32_t* tiles_per_gauss) {
    int64_t total = 0;
    for (size_t idx = 0; idx < (size_t)C * N; ++idx) {
        uint32_t x0, y0, x1, y1; bool ok;
        tile_range(means2d, radii, idx, tile_size, tw, th, x0, y0, x1, y1, ok);
        const int32_t n = ok ? (int32_t)((y1 - y0) * (x1 - x0)) : 0;
        tiles_per_gauss[idx] = n;
        total += n;
    }
    return total;
}

// Emits unsorted (isect_ids, flatten_ids), then a stable sort on the masked key when sort != 0.
void orc_intersect_emit_sort(int C, int N, const float* means2d, const int32_t* radii, const float* depths,
                             uint32_t tile_size, uint32_t tw, uint32_t th, int sort,
                             int64_t n_isects, int64_t* isect_ids, int32_t* flatten_ids) {
    const uint32_t tile_n_bits = bit_width_floor_log2_plus1(tw * th);
    const uint32_t cam_n_bits = bit_width_floor_log2_plus1((uint32_t)C);
    int64_t cur = 0;
    for (size_t idx = 0; idx < (size_t)C * N; ++idx) {
        uint32_t x0, y0, x1, y1; bool ok;
        tile_range(means2d, radii, idx, tile_size, tw, th, x0, y0, x1, y1, ok);
        if (!ok) continue;
        const int64_t cid = (int64_t)(idx / N);
        const int64_t cid_enc = cid << (32 + tile_n_bits);
        uint32_t dbits;
        std::memcpy(&dbits, depths + idx, 4);
        const int64_t depth_enc = (int64_t)dbits;
        for (uint32_t i = y0; i < y1; ++i)
            for (uint32_t j = x0; j < x1; ++j) {
                const int64_t tile_id = (int64_t)i * tw + j;
                isect_ids[cur] = cid_enc | (tile_id << 32) | depth_enc;
                flatten_ids[cur] = (int32_t)idx;
                ++cur;
            }
    }
    if (sort && n_isects > 0) {
        const int nbits = 32 + tile_n_bits + cam_n_bits;
        const uint64_t mask = nbits >= 64 ? ~0ull : ((1ull << nbits) - 1ull);
        std::vector<int64_t> perm(n_isects);
        std::iota(perm.begin(), perm.end(), 0);
        std::stable_sort(perm.begin(), perm.end(), [&](int64_t a, int64_t b) {
            return ((uint64_t)isect_ids[a] & mask) < ((uint64_t)isect_ids[b] & mask);
        });
        std::vector<int64_t> k(n_isects);
        std::vector<int32_t> v(n_isects);
        for (int64_t i = 0; i < n_isects; ++i) { k[i] = isect_ids[perm[i]]; v[i] = flatten_ids[perm[i]]; }
        std::memcpy(isect_ids, k.data(), n_isects * 8);
        std::memcpy(flatten_ids, v.data(), n_isects * 4);
    }
}

void orc_intersect_offset(int64_t n_isects, const int64_t* isect_ids, int C, uint32_t tw, uint32_t th, int32_t* offsets) {
    const uint32_t n_tiles = tw * th;
    const uint32_t tile_n_bits = bit_width_floor_log2_plus1(n_tiles);
    if (n_isects == 0) { std::fill(offsets, offsets + (size_t)C * n_tiles, 0); return; }
    for (int64_t idx = 0; idx < n_isects; ++idx) {
        const int64_t cur = isect_ids[idx] >> 32;
        const int64_t id_curr = (cur >> tile_n_bits) * n_tiles + (cur & ((1 << tile_n_bits) - 1));
        if (idx == 0)
            for (int64_t i = 0; i < id_curr + 1; ++i) offsets[i] = (int32_t)idx;
        if (idx == n_isects - 1)
            for (int64_t i = id_curr + 1; i < (int64_t)C * n_tiles; ++i) offsets[i] = (int32_t)n_isects;
        if (idx > 0) {
            const int64_t prev = isect_ids[idx - 1] >> 32;
            if (prev == cur) continue;
            const int64_t id_prev = (prev >> tile_n_bits) * n_tiles + (prev & ((1 << tile_n_bits) - 1));
            for (int64_t i = id_prev + 1; i < id_curr + 1; ++i) offsets[i] = (int32_t)idx;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Rasterizer forward: gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu:58-285 (C = 1 per call as in
// the reference; the camera index only offsets the output planes). exp is libm expf.
// Also returns n_pairs = number of list entries visited (up to and including the terminating
// one), the implementation-independent work count used by the benchmark's flop figure.
// ---------------------------------------------------------------------------------------------
static void world_ray(const RSPose& rs, const Camera& cam, float px, float py, V3& ro, V3& rd, bool& valid) {
    V3 cr;
    valid = image_to_cam_ray(cam, px, py, cr);
    if (!valid) { ro = {0, 0, 0}; rd = {0, 0, 0}; return; }
    // image_point_to_world_ray_shutter_pose, Cameras.cuh:322-339: the pose of this pixel's row / column
    const Pose pose = shutter_pose(rs, shutter_time(rs.type, px, py, cam.W, cam.H));
    // ShutterPose::camera_ray_to_world_ray, Cameras.cuh:261-265
    const M3 Rinv = mat3_cast(quat_inverse(pose.q));
    M3 nR;
    for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) nR.m[i][j] = -Rinv.m[i][j];
    ro = mul(nR, pose.t);
    rd = mul(Rinv, cr);
}

static inline float safe_rsqrt_norm(V3 v, V3& out) {  // Utils.cuh:181-184
    const float l = v.x * v.x + v.y * v.y + v.z * v.z;
    if (l > 0.f) { const float il = 1.0f / std::sqrt(l); out = v * il; } else out = v;
    return l;
}

// CH colour channels (1..4; the reference instantiates 1, 3, 4 for the render modes D, RGB, RGB_D of
// gsplat/Rasterization.cpp:373-393) and optional per-tile masks (RasterizeToPixelsFromWorld3DGSFwd.cu:147-155:
// a tile labelled false gets the background colour; alpha and last_ids, which the reference leaves
// unwritten there, are written as 0).
int64_t orc_rasterize_fwd_ch(
    int N, int64_t n_isects, int CH,
    const float* means, const float* quats, const float* scales, const float* colors /*[N,CH]*/, const float* opacities,
    const float* background /*nullable [CH]*/, const uint8_t* masks /*nullable [th*tw]*/,
    int W, int H, int tile_size, const float* viewmat, const float* K, int camera_model, const float* radial,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* render_colors /*[H,W,CH]*/, float* render_alphas /*[H,W]*/, int32_t* last_ids /*[H,W]*/,
    int tile_lo, int tile_hi /* only tiles in [tile_lo, tile_hi) are rendered; pass 0, -1 for all */) {
    const int tw = (W + tile_size - 1) / tile_size, th = (H + tile_size - 1) / tile_size;
    const RSPose pose = rs_from_viewmat(viewmat);
    const Camera cam = make_camera(camera_model, K, W, H, radial);
    int64_t n_pairs = 0;
    if (tile_hi < 0) tile_hi = tw * th;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : n_pairs)
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int ty = tile / tw, tx = tile % tw;
        const int32_t range_start = tile_offsets[tile];
        const int32_t range_end = (tile == tw * th - 1) ? (int32_t)n_isects : tile_offsets[tile + 1];
        // per-entry precompute shared by the tile's pixels (the reference does it per batch)
        const int cnt = range_end - range_start;
        if (masks && !masks[tile]) {
            for (int ly = 0; ly < tile_size; ++ly)
                for (int lx = 0; lx < tile_size; ++lx) {
                    const int i = ty * tile_size + ly, j = tx * tile_size + lx;
                    if (i >= H || j >= W) continue;
                    const int pid = i * W + j;
                    for (int k = 0; k < CH; ++k) render_colors[pid * CH + k] = background ? background[k] : 0.0f;
                    render_alphas[pid] = 0.0f;
                    last_ids[pid] = 0;
                }
            continue;
        }
        std::vector<M3> Ms(cnt > 0 ? cnt : 0);
        for (int t = 0; t < cnt; ++t) {
            const int g = flatten_ids[range_start + t];
            const M3 R = quat_to_rotmat(Q4{quats[g * 4], quats[g * 4 + 1], quats[g * 4 + 2], quats[g * 4 + 3]});
            const float is[3] = {1.0f / scales[g * 3], 1.0f / scales[g * 3 + 1], 1.0f / scales[g * 3 + 2]};
            // iscl_rot = S * R^T
            for (int i = 0; i < 3; ++i) for (int j = 0; j < 3; ++j) Ms[t].m[i][j] = is[i] * R.m[j][i];
        }
        for (int ly = 0; ly < tile_size; ++ly)
            for (int lx = 0; lx < tile_size; ++lx) {
                const int i = ty * tile_size + ly, j = tx * tile_size + lx;
                if (i >= H || j >= W) continue;
                V3 ro, rd; bool rv;
                world_ray(pose, cam, (float)j + 0.5f, (float)i + 0.5f, ro, rd, rv);
                float T = 1.0f;
                uint32_t cur_idx = 0;
                float pix[4] = {0.f, 0.f, 0.f, 0.f};
                bool done = !rv;
                for (int t = 0; t < cnt && !done; ++t) {
                    ++n_pairs;
                    const int g = flatten_ids[range_start + t];
                    const V3 xyz{means[g * 3], means[g * 3 + 1], means[g * 3 + 2]};
                    const float opac = opacities[g];
                    const V3 gro = mul(Ms[t], ro - xyz);
                    V3 grd; safe_rsqrt_norm(mul(Ms[t], rd), grd);
                    const V3 gc = cross(grd, gro);
                    const float power = -0.5f * dot(gc, gc);
                    const float alpha = std::min(0.999f, opac * std::exp(power));
                    if (alpha < 1.f / 255.f) continue;
                    const float next_T = T * (1.0f - alpha);
                    if (next_T <= 1e-4f) { done = true; break; }
                    const float vis = alpha * T;
                    for (int k = 0; k < CH; ++k) pix[k] += colors[g * CH + k] * vis;
                    cur_idx = (uint32_t)(range_start + t);
                    T = next_T;
                }
                const int pid = i * W + j;
                render_alphas[pid] = 1.0f - T;
                for (int k = 0; k < CH; ++k)
                    render_colors[pid * CH + k] = background ? (pix[k] + T * background[k]) : pix[k];
                last_ids[pid] = (int32_t)cur_idx;
            }
    }
    return n_pairs;
}

int64_t orc_rasterize_fwd(
    int N, int64_t n_isects,
    const float* means, const float* quats, const float* scales, const float* colors, const float* opacities,
    const float* background /*nullable [3]*/,
    int W, int H, int tile_size, const float* viewmat, const float* K, int camera_model, const float* radial,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* render_colors /*[H,W,3]*/, float* render_alphas /*[H,W]*/, int32_t* last_ids /*[H,W]*/,
    int tile_lo, int tile_hi) {
    return orc_rasterize_fwd_ch(N, n_isects, 3, means, quats, scales, colors, opacities, background, nullptr, W, H, tile_size,
                                viewmat, K, camera_model, radial, tile_offsets, flatten_ids, render_colors, render_alphas,
                                last_ids, tile_lo, tile_hi);
}

// ---------------------------------------------------------------------------------------------
// Rasterizer backward: gsplat/RasterizeToPixelsFromWorld3DGSBwd.cu:63-378 with the VJPs of
// gsplat/Utils.cuh:104-194. Per-Gaussian sums are accumulated in double in a fixed order
// (tile by tile, pixel by pixel, back to front) so the result is run-to-run identical.
// Outputs must be pre-zeroed. Returns the number of (pixel, entry) pairs walked.
// ---------------------------------------------------------------------------------------------
int64_t orc_rasterize_bwd_ch(
    int N, int64_t n_isects, int CH,
    const float* means, const float* quats, const float* scales, const float* colors, const float* opacities,
    const float* background, const uint8_t* masks,
    int W, int H, int tile_size, const float* viewmat, const float* K, int camera_model, const float* radial,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    const float* render_alphas, const int32_t* last_ids, const float* v_render_colors, const float* v_render_alphas,
    float* v_means, float* v_quats, float* v_scales, float* v_colors, float* v_opacities,
    int tile_lo, int tile_hi /* only tiles in [tile_lo, tile_hi) contribute; pass 0, -1 for all */) {
    const int tw = (W + tile_size - 1) / tile_size, th = (H + tile_size - 1) / tile_size;
    const RSPose pose = rs_from_viewmat(viewmat);
    const Camera cam = make_camera(camera_model, K, W, H, radial);
    std::vector<double> acc((size_t)N * 15, 0.0);  // mean3 scale3 quat4 colour4 opac1
    int64_t n_pairs = 0;
    // Tiles are processed sequentially for a fixed summation order; pixels inside a tile in parallel
    // into per-thread buffers would reorder sums, so parallelism is over tiles with a merge in tile order.
    const int n_tiles = tw * th;
    std::vector<std::vector<std::pair<int, std::array<double, 15>>>> tile_out(n_tiles);
    if (tile_hi < 0) tile_hi = n_tiles;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : n_pairs)
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int ty = tile / tw, tx = tile % tw;
        const int32_t range_start = tile_offsets[tile];
        const int32_t range_end = (tile == n_tiles - 1) ? (int32_t)n_isects : tile_offsets[tile + 1];
        const int cnt = range_end - range_start;
        if (cnt <= 0) continue;
        if (masks && !masks[tile]) continue;  // ...Bwd.cu:84
        std::vector<std::array<double, 15>> loc(cnt);
        for (auto& a : loc) a.fill(0.0);
        std::vector<char> touched(cnt, 0);
        for (int ly = 0; ly < tile_size; ++ly)
            for (int lx = 0; lx < tile_size; ++lx) {
                const int i = ty * tile_size + ly, j = tx * tile_size + lx;
                if (i >= H || j >= W) continue;
                V3 ro, rd; bool rv;
                world_ray(pose, cam, (float)j + 0.5f, (float)i + 0.5f, ro, rd, rv);
                if (!rv) continue;
                const int pid = i * W + j;
                const float T_final = 1.0f - render_alphas[pid];
                float T = T_final;
                float buffer[4] = {0.f, 0.f, 0.f, 0.f};
                const int32_t bin_final = last_ids[pid];
                float vrc[4] = {0.f, 0.f, 0.f, 0.f};
                for (int k = 0; k < CH; ++k) vrc[k] = v_render_colors[pid * CH + k];
                const float vra = v_render_alphas[pid];
                for (int idx = std::min(range_end - 1, bin_final); idx >= range_start; --idx) {
                    ++n_pairs;
                    const int t = idx - range_start;
                    const int g = flatten_ids[idx];
                    const V3 xyz{means[g * 3], means[g * 3 + 1], means[g * 3 + 2]};
                    const float opac = opacities[g];
                    const V3 scale{scales[g * 3], scales[g * 3 + 1], scales[g * 3 + 2]};
                    const Q4 quat{quats[g * 4], quats[g * 4 + 1], quats[g * 4 + 2], quats[g * 4 + 3]};
                    const M3 R = quat_to_rotmat(quat);
                    const float is[3] = {1.0f / scale.x, 1.0f / scale.y, 1.0f / scale.z};
                    M3 Mt;  // (R*S)^T = S*R^T
                    for (int a = 0; a < 3; ++a) for (int b = 0; b < 3; ++b) Mt.m[a][b] = is[a] * R.m[b][a];
                    const V3 omu = ro - xyz;
                    const V3 gro = mul(Mt, omu);
                    const V3 grd = mul(Mt, rd);
                    V3 grd_n; safe_rsqrt_norm(grd, grd_n);
                    const V3 gc = cross(grd_n, gro);
                    const float gd = dot(gc, gc);
                    const float power = -0.5f * gd;
                    const float vis = std::exp(power);
                    const float alpha = std::min(0.999f, opac * vis);
                    if (power > 0.f || alpha < 1.f / 255.f) continue;

                    const float ra = 1.0f / (1.0f - alpha);
                    T *= ra;
                    const float fac = alpha * T;
                    float v_rgb[4] = {0.f, 0.f, 0.f, 0.f};
                    for (int k = 0; k < CH; ++k) v_rgb[k] = fac * vrc[k];
                    float v_alpha = 0.f;
                    for (int k = 0; k < CH; ++k) v_alpha += (colors[g * CH + k] * T - buffer[k] * ra) * vrc[k];
                    v_alpha += T_final * ra * vra;
                    if (background) {
                        float accum = 0.f;
                        for (int k = 0; k < CH; ++k) accum += background[k] * vrc[k];
                        v_alpha += -T_final * ra * accum;
                    }
                    V3 v_mean{0, 0, 0}, v_scale{0, 0, 0};
                    float v_quat[4] = {0, 0, 0, 0};
                    float v_opacity = 0.f;
                    if (opac * vis <= 0.999f) {
                        const float v_vis = opac * v_alpha;
                        const float v_gd = -0.5f * vis * v_vis;
                        const V3 v_gc = (2.0f * v_gd) * gc;
                        const V3 cr1 = cross(v_gc, gro);
                        const V3 v_grd_n{-cr1.x, -cr1.y, -cr1.z};
                        const V3 v_gro = cross(v_gc, grd_n);
                        // safe_normalize_bw, Utils.cuh:186-194
                        V3 v_grd;
                        {
                            const float l = grd.x * grd.x + grd.y * grd.y + grd.z * grd.z;
                            if (l > 0.f) {
                                const float il = 1.0f / std::sqrt(l);
                                const float il3 = il * il * il;
                                const float dd = dot(v_grd_n, grd);
                                v_grd = il * v_grd_n - (il3 * dd) * grd;
                            } else v_grd = v_grd_n;
                        }
                        // v_Mt = outer(v_grd, rd) + outer(v_gro, omu)  (math: column-vector times row-vector)
                        float vMt[3][3];
                        const float vg[3] = {v_grd.x, v_grd.y, v_grd.z}, vo[3] = {v_gro.x, v_gro.y, v_gro.z};
                        const float d3[3] = {rd.x, rd.y, rd.z}, o3[3] = {omu.x, omu.y, omu.z};
                        for (int a = 0; a < 3; ++a) for (int b = 0; b < 3; ++b) vMt[a][b] = vg[a] * d3[b] + vo[a] * o3[b];
                        // v_o_minus_mu = Mt^T * v_gro
                        const V3 v_omu{Mt.m[0][0] * vo[0] + Mt.m[1][0] * vo[1] + Mt.m[2][0] * vo[2],
                                       Mt.m[0][1] * vo[0] + Mt.m[1][1] * vo[1] + Mt.m[2][1] * vo[2],
                                       Mt.m[0][2] * vo[0] + Mt.m[1][2] * vo[1] + Mt.m[2][2] * vo[2]};
                        v_mean = V3{-v_omu.x, -v_omu.y, -v_omu.z};
                        // quat_scale_to_preci_half_vjp(quat, scale, R, v_M = v_Mt^T), Utils.cuh:128-158.
                        // v_M[a][b] = vMt[b][a]; v_R = v_M * S -> v_R[a][b] = v_M[a][b] * is[b]
                        float vR[3][3];
                        for (int a = 0; a < 3; ++a) for (int b = 0; b < 3; ++b) vR[a][b] = vMt[b][a] * is[b];
                        // quat_to_rotmat_vjp, Utils.cuh:104-126 (glm v_R[c][r] == vR[r][c])
                        float w = quat.w, x = quat.x, y = quat.y, z = quat.z;
                        const float inv_norm = 1.0f / std::sqrt(x * x + y * y + z * z + w * w);
                        x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
                        const float vqn[4] = {
                            2.f * (x * (vR[2][1] - vR[1][2]) + y * (vR[0][2] - vR[2][0]) + z * (vR[1][0] - vR[0][1])),
                            2.f * (-2.f * x * (vR[1][1] + vR[2][2]) + y * (vR[1][0] + vR[0][1]) + z * (vR[2][0] + vR[0][2]) + w * (vR[2][1] - vR[1][2])),
                            2.f * (x * (vR[1][0] + vR[0][1]) - 2.f * y * (vR[0][0] + vR[2][2]) + z * (vR[2][1] + vR[1][2]) + w * (vR[0][2] - vR[2][0])),
                            2.f * (x * (vR[2][0] + vR[0][2]) + y * (vR[2][1] + vR[1][2]) - 2.f * z * (vR[0][0] + vR[1][1]) + w * (vR[1][0] - vR[0][1]))};
                        const float qn[4] = {w, x, y, z};
                        const float dq = vqn[0] * qn[0] + vqn[1] * qn[1] + vqn[2] * qn[2] + vqn[3] * qn[3];
                        for (int k = 0; k < 4; ++k) v_quat[k] = (vqn[k] - dq * qn[k]) * inv_norm;
                        // v_scale[j] = -is[j]^2 * sum_a R[a][j] * v_M[a][j]
                        v_scale.x = -is[0] * is[0] * (R.m[0][0] * vMt[0][0] + R.m[1][0] * vMt[0][1] + R.m[2][0] * vMt[0][2]);
                        v_scale.y = -is[1] * is[1] * (R.m[0][1] * vMt[1][0] + R.m[1][1] * vMt[1][1] + R.m[2][1] * vMt[1][2]);
                        v_scale.z = -is[2] * is[2] * (R.m[0][2] * vMt[2][0] + R.m[1][2] * vMt[2][1] + R.m[2][2] * vMt[2][2]);
                        v_opacity = vis * v_alpha;
                    }
                    for (int k = 0; k < CH; ++k) buffer[k] += colors[g * CH + k] * fac;
                    auto& a = loc[t];
                    touched[t] = 1;
                    a[0] += v_mean.x; a[1] += v_mean.y; a[2] += v_mean.z;
                    a[3] += v_scale.x; a[4] += v_scale.y; a[5] += v_scale.z;
                    a[6] += v_quat[0]; a[7] += v_quat[1]; a[8] += v_quat[2]; a[9] += v_quat[3];
                    a[10] += v_rgb[0]; a[11] += v_rgb[1]; a[12] += v_rgb[2]; a[13] += v_rgb[3];
                    a[14] += v_opacity;
                }
            }
        auto& out = tile_out[tile];
        for (int t = 0; t < cnt; ++t)
            if (touched[t]) out.emplace_back(flatten_ids[range_start + t], loc[t]);
    }
    for (int tile = 0; tile < n_tiles; ++tile)
        for (auto& e : tile_out[tile])
            for (int k = 0; k < 15; ++k) acc[(size_t)e.first * 15 + k] += e.second[k];
    for (int g = 0; g < N; ++g) {
        const double* a = &acc[(size_t)g * 15];
        for (int k = 0; k < 3; ++k) v_means[g * 3 + k] += (float)a[k];
        for (int k = 0; k < 3; ++k) v_scales[g * 3 + k] += (float)a[3 + k];
        for (int k = 0; k < 4; ++k) v_quats[g * 4 + k] += (float)a[6 + k];
        for (int k = 0; k < CH; ++k) v_colors[g * CH + k] += (float)a[10 + k];
        v_opacities[g] += (float)a[14];
    }
    return n_pairs;
}

int64_t orc_rasterize_bwd(
    int N, int64_t n_isects,
    const float* means, const float* quats, const float* scales, const float* colors, const float* opacities,
    const float* background,
    int W, int H, int tile_size, const float* viewmat, const float* K, int camera_model, const float* radial,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    const float* render_alphas, const int32_t* last_ids, const float* v_render_colors, const float* v_render_alphas,
    float* v_means, float* v_quats, float* v_scales, float* v_colors, float* v_opacities, int tile_lo, int tile_hi) {
    return orc_rasterize_bwd_ch(N, n_isects, 3, means, quats, scales, colors, opacities, background, nullptr, W, H, tile_size,
                                viewmat, K, camera_model, radial, tile_offsets, flatten_ids, render_alphas, last_ids,
                                v_render_colors, v_render_alphas, v_means, v_quats, v_scales, v_colors, v_opacities, tile_lo,
                                tile_hi);
}

// ---------------------------------------------------------------------------------------------
// Fused SSIM: src/training/kernels/ssim.cu:16-27 (taps), :46-54 (zero padding), :90-275
// (forward, symmetric-pair accumulation), :310-423 (backward). Images are CHW [CH,H,W].
// ---------------------------------------------------------------------------------------------
static const float G11[11] = {
    0.001028380123898387f, 0.0075987582094967365f, 0.036000773310661316f, 0.10936068743467331f,
    0.21300552785396576f, 0.26601171493530273f, 0.21300552785396576f, 0.10936068743467331f,
    0.036000773310661316f, 0.0075987582094967365f, 0.001028380123898387f};

static inline float pix_or_zero(const float* img, int c, int y, int x, int H, int W) {
    if (x < 0 || x >= W || y < 0 || y >= H) return 0.f;
    return img[(size_t)c * H * W + (size_t)y * W + x];
}

void orc_fusedssim_fwd(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2,
                       float* ssim_map, float* dm_dmu1, float* dm_dsigma1_sq, float* dm_dsigma12) {
#pragma omp parallel for schedule(static)
    for (int cy = 0; cy < CH * H; ++cy) {
        const int c = cy / H, y = cy % H;
        std::vector<float> h((size_t)11 * W * 5);  // horizontal sums for rows y-5..y+5
        for (int r = 0; r < 11; ++r) {
            const int yy = y + r - 5;
            for (int x = 0; x < W; ++x) {
                float sX = 0, sX2 = 0, sY = 0, sY2 = 0, sXY = 0;
                for (int d = 1; d <= 5; ++d) {
                    const float w = G11[5 - d];
                    const float Xl = pix_or_zero(img1, c, yy, x - d, H, W), Yl = pix_or_zero(img2, c, yy, x - d, H, W);
                    const float Xr = pix_or_zero(img1, c, yy, x + d, H, W), Yr = pix_or_zero(img2, c, yy, x + d, H, W);
                    sX += (Xl + Xr) * w;
                    sX2 += ((Xl * Xl) + (Xr * Xr)) * w;
                    sY += (Yl + Yr) * w;
                    sY2 += ((Yl * Yl) + (Yr * Yr)) * w;
                    sXY += ((Xl * Yl) + (Xr * Yr)) * w;
                }
                const float cX = pix_or_zero(img1, c, yy, x, H, W), cY = pix_or_zero(img2, c, yy, x, H, W);
                const float wc = G11[5];
                sX += cX * wc; sX2 += (cX * cX) * wc; sY += cY * wc; sY2 += (cY * cY) * wc; sXY += (cX * cY) * wc;
                float* o = &h[((size_t)r * W + x) * 5];
                o[0] = sX; o[1] = sX2; o[2] = sY; o[3] = sY2; o[4] = sXY;
            }
        }
        for (int x = 0; x < W; ++x) {
            float out[5] = {0, 0, 0, 0, 0};
            for (int d = 1; d <= 5; ++d) {
                const float w = G11[5 - d];
                const float* top = &h[((size_t)(5 - d) * W + x) * 5];
                const float* bot = &h[((size_t)(5 + d) * W + x) * 5];
                for (int k = 0; k < 5; ++k) out[k] += (top[k] + bot[k]) * w;
            }
            const float* ctr = &h[((size_t)5 * W + x) * 5];
            for (int k = 0; k < 5; ++k) out[k] += ctr[k] * G11[5];
            const float mu1 = out[0], mu2 = out[2];
            const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
            const float sigma1_sq = out[1] - mu1_sq, sigma2_sq = out[3] - mu2_sq, sigma12 = out[4] - mu1 * mu2;
            const float A = mu1_sq + mu2_sq + C1, B = sigma1_sq + sigma2_sq + C2;
            const float C_ = 2.f * mu1 * mu2 + C1, D_ = 2.f * sigma12 + C2;
            const size_t gi = (size_t)c * H * W + (size_t)y * W + x;
            ssim_map[gi] = (C_ * D_) / (A * B);
            if (dm_dmu1) {
                dm_dmu1[gi] = ((mu2 * 2.f * D_) / (A * B) - (mu2 * 2.f * C_) / (A * B) - (mu1 * 2.f * C_ * D_) / (A * A * B) + (mu1 * 2.f * C_ * D_) / (A * B * B));
                dm_dsigma1_sq[gi] = (-C_ * D_) / (A * B * B);
                dm_dsigma12[gi] = (2.f * C_) / (A * B);
            }
        }
    }
}

void orc_fusedssim_bwd(int CH, int H, int W, const float* img1, const float* img2, const float* dL_dmap,
                       const float* dm_dmu1, const float* dm_dsigma1_sq, const float* dm_dsigma12, float* dL_dimg1) {
#pragma omp parallel for schedule(static)
    for (int cy = 0; cy < CH * H; ++cy) {
        const int c = cy / H, y = cy % H;
        std::vector<float> h((size_t)11 * W * 3);
        for (int r = 0; r < 11; ++r) {
            const int yy = y + r - 5;
            for (int x = 0; x < W; ++x) {
                float a[3] = {0, 0, 0};
                auto fused = [&](int xx, float* o) {
                    const float chain = pix_or_zero(dL_dmap, c, yy, xx, H, W);
                    o[0] = pix_or_zero(dm_dmu1, c, yy, xx, H, W) * chain;
                    o[1] = pix_or_zero(dm_dsigma1_sq, c, yy, xx, H, W) * chain;
                    o[2] = pix_or_zero(dm_dsigma12, c, yy, xx, H, W) * chain;
                };
                for (int d = 1; d <= 5; ++d) {
                    const float w = G11[5 - d];
                    float l[3], rr[3];
                    fused(x - d, l); fused(x + d, rr);
                    for (int k = 0; k < 3; ++k) a[k] += (l[k] + rr[k]) * w;
                }
                float cc[3];
                fused(x, cc);
                for (int k = 0; k < 3; ++k) a[k] += cc[k] * G11[5];
                for (int k = 0; k < 3; ++k) h[((size_t)r * W + x) * 3 + k] = a[k];
            }
        }
        for (int x = 0; x < W; ++x) {
            float s[3] = {0, 0, 0};
            for (int d = 1; d <= 5; ++d) {
                const float w = G11[5 - d];
                const float* top = &h[((size_t)(5 - d) * W + x) * 3];
                const float* bot = &h[((size_t)(5 + d) * W + x) * 3];
                for (int k = 0; k < 3; ++k) s[k] += (top[k] + bot[k]) * w;
            }
            const float* ctr = &h[((size_t)5 * W + x) * 3];
            for (int k = 0; k < 3; ++k) s[k] += ctr[k] * G11[5];
            const size_t gi = (size_t)c * H * W + (size_t)y * W + x;
            const float p1 = img1[gi], p2 = img2[gi];
            dL_dimg1[gi] = s[0] + (2.f * p1) * s[1] + (p2)*s[2];
        }
    }
}

// Photometric loss of the trainer and its gradient w.r.t. the UNCLAMPED HWC render:
// src/training/trainer.cpp:107-134 (0.8 L1 + 0.2 (1 - SSIM)), include/kernels/fused_ssim.cuh:59-67,
// :85-96, :117-122 ("valid" crop of 5 px when h,w > 10, then mean),
// src/training/rasterization/rasterizer.cpp:205 (clamp(0,1) + HWC->CHW permute).
// render: [H,W,3] unclamped; target: [3,H,W]. Returns loss; v_render [H,W,3].
float orc_photometric_loss(int H, int W, float lambda_dssim, const float* render_hwc, const float* target_chw,
                           float* v_render_hwc /*nullable*/, float* out_l1, float* out_ssim) {
    const size_t n = (size_t)3 * H * W;
    std::vector<float> img(n);
    for (int c = 0; c < 3; ++c)
        for (int y = 0; y < H; ++y)
            for (int x = 0; x < W; ++x)
                img[(size_t)c * H * W + (size_t)y * W + x] = std::min(1.f, std::max(0.f, render_hwc[((size_t)y * W + x) * 3 + c]));
    std::vector<float> map(n), d1(n), d2(n), d3(n);
    orc_fusedssim_fwd(3, H, W, (float)(0.01 * 0.01), (float)(0.03 * 0.03), img.data(), target_chw, map.data(), d1.data(), d2.data(), d3.data());
    const bool crop = (H > 10 && W > 10);
    const int y0 = crop ? 5 : 0, y1 = crop ? H - 5 : H, x0 = crop ? 5 : 0, x1 = crop ? W - 5 : W;
    double ssum = 0.0, l1sum = 0.0;
    for (int c = 0; c < 3; ++c)
        for (int y = y0; y < y1; ++y)
            for (int x = x0; x < x1; ++x) ssum += map[(size_t)c * H * W + (size_t)y * W + x];
    for (size_t i = 0; i < n; ++i) l1sum += std::fabs(img[i] - target_chw[i]);
    const double n_valid = 3.0 * (y1 - y0) * (x1 - x0);
    const float l1 = (float)(l1sum / (double)n);
    const float ssim = (float)(ssum / n_valid);
    if (out_l1) *out_l1 = l1;
    if (out_ssim) *out_ssim = ssim;
    const float loss = (1.f - lambda_dssim) * l1 + lambda_dssim * (1.f - ssim);
    if (v_render_hwc) {
        std::vector<float> dmap(n, 0.f), gimg(n);
        const float gs = (float)(-(double)lambda_dssim / n_valid);
        for (int c = 0; c < 3; ++c)
            for (int y = y0; y < y1; ++y)
                for (int x = x0; x < x1; ++x) dmap[(size_t)c * H * W + (size_t)y * W + x] = gs;
        orc_fusedssim_bwd(3, H, W, img.data(), target_chw, dmap.data(), d1.data(), d2.data(), d3.data(), gimg.data());
        const float gl = (float)((1.0 - (double)lambda_dssim) / (double)n);
        for (int c = 0; c < 3; ++c)
            for (int y = 0; y < H; ++y)
                for (int x = 0; x < W; ++x) {
                    const size_t ci = (size_t)c * H * W + (size_t)y * W + x;
                    const float diff = img[ci] - target_chw[ci];
                    const float sgn = diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f);
                    float g = gimg[ci] + gl * sgn;
                    const float r = render_hwc[((size_t)y * W + x) * 3 + c];
                    if (!(r >= 0.f && r <= 1.f)) g = 0.f;  // clamp backward passes inside [0,1] inclusive
                    v_render_hwc[((size_t)y * W + x) * 3 + c] = g;
                }
    }
    return loss;
}

// ---------------------------------------------------------------------------------------------
// Adam: src/training/fastgs/optimizer/include/adam_kernels.cuh:25-35. Bias terms are computed by
// the caller in double (src/training/optimizers/fused_adam.cpp:78-79).
// ---------------------------------------------------------------------------------------------
void orc_adam_step(int64_t n, float* param, float* exp_avg, float* exp_avg_sq, const float* grad,
                   float lr, float beta1, float beta2, float eps, float bc1_rcp, float bc2_sqrt_rcp) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const float g = grad[i];
        const float m1 = beta1 * exp_avg[i] + (1.0f - beta1) * g;
        const float m2 = beta2 * exp_avg_sq[i] + (1.0f - beta2) * g * g;
        const float denom = std::sqrt(m2) * bc2_sqrt_rcp + eps;
        const float step_size = lr * bc1_rcp;
        param[i] -= step_size * m1 / denom;
        exp_avg[i] = m1;
        exp_avg_sq[i] = m2;
    }
}

// ---------------------------------------------------------------------------------------------
// MCMC relocation, equation (9): gsplat/RelocationCUDA.cu:12-43.
// ---------------------------------------------------------------------------------------------
void orc_relocation(int n, const float* opacities, const float* scales, const int32_t* ratios,
                    const float* binoms, int n_max, float* new_opacities, float* new_scales) {
#pragma omp parallel for schedule(static)
    for (int idx = 0; idx < n; ++idx) {
        const int n_idx = ratios[idx];
        float denom_sum = 0.0f;
        new_opacities[idx] = 1.0f - std::pow(1.0f - opacities[idx], 1.0f / (float)n_idx);
        for (int i = 1; i <= n_idx; ++i)
            for (int k = 0; k <= (i - 1); ++k) {
                const float bin_coeff = binoms[(i - 1) * n_max + k];
                const float sign = (k & 1) ? -1.0f : 1.0f;
                const float term = (sign / std::sqrt((float)(k + 1))) * std::pow(new_opacities[idx], (float)(k + 1));
                denom_sum += (bin_coeff * term);
            }
        const float coeff = opacities[idx] / denom_sum;
        for (int i = 0; i < 3; ++i) new_scales[idx * 3 + i] = coeff * scales[idx * 3 + i];
    }
}

// MCMC noise: gsplat/RelocationCUDA.cu:88-143 (raw_quat_to_rotmat clamps inv_norm at 1e12).
void orc_add_noise(int n, const float* raw_opacities, const float* raw_scales, const float* raw_quats,
                   const float* noise, float* means, float current_lr) {
#pragma omp parallel for schedule(static)
    for (int idx = 0; idx < n; ++idx) {
        const float s2[3] = {std::exp(2.f * raw_scales[idx * 3]), std::exp(2.f * raw_scales[idx * 3 + 1]), std::exp(2.f * raw_scales[idx * 3 + 2])};
        float w = raw_quats[idx * 4], x = raw_quats[idx * 4 + 1], y = raw_quats[idx * 4 + 2], z = raw_quats[idx * 4 + 3];
        const float inv_norm = std::fmin(1.0f / std::sqrt(x * x + y * y + z * z + w * w), 1e+12f);
        x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
        const float x2 = x * x, y2 = y * y, z2 = z * z, xy = x * y, xz = x * z, yz = y * z, wx = w * x, wy = w * y, wz = w * z;
        const float R[3][3] = {{1.f - 2.f * (y2 + z2), 2.f * (xy - wz), 2.f * (xz + wy)},
                               {2.f * (xy + wz), 1.f - 2.f * (x2 + z2), 2.f * (yz - wx)},
                               {2.f * (xz - wy), 2.f * (yz + wx), 1.f - 2.f * (x2 + y2)}};
        // covariance = R * S2 * R^T, applied to the noise vector
        float cov[3][3];
        for (int a = 0; a < 3; ++a)
            for (int b = 0; b < 3; ++b) {
                float s = 0.f;
                for (int k = 0; k < 3; ++k) s += (R[a][k] * s2[k]) * R[b][k];
                cov[a][b] = s;
            }
        const float nz[3] = {noise[idx * 3], noise[idx * 3 + 1], noise[idx * 3 + 2]};
        const float opacity = 1.0f / (1.f + std::exp(-raw_opacities[idx]));
        const float op_sigmoid = 1.0f / (1.f + std::exp(100.f * opacity - 0.5f));
        const float nf = current_lr * op_sigmoid;
        for (int a = 0; a < 3; ++a)
            means[idx * 3 + a] += nf * (cov[a][0] * nz[0] + cov[a][1] * nz[1] + cov[a][2] * nz[2]);
    }
}

// gsplat/QuatToRotmatCUDA.cu:13: quats [N,4] -> row-major rotmats [N,3,3].
void orc_quats_to_rotmats(int n, const float* quats, float* rotmats) {
    for (int i = 0; i < n; ++i) {
        const M3 R = quat_to_rotmat(Q4{quats[i * 4], quats[i * 4 + 1], quats[i * 4 + 2], quats[i * 4 + 3]});
        for (int a = 0; a < 3; ++a) for (int b = 0; b < 3; ++b) rotmats[i * 9 + a * 3 + b] = R.m[a][b];
    }
}

// Camera position as the reference's glue derives it: inverse(viewmat)[:3,3]
// (gsplat/Rasterization.cpp:358-359). For a rigid [R|t] that is -R^T t; evaluated in double.
void orc_campos(const float* vm, float* out) {
    for (int i = 0; i < 3; ++i)
        out[i] = (float)(-((double)vm[0 * 4 + i] * vm[3] + (double)vm[1 * 4 + i] * vm[7] + (double)vm[2 * 4 + i] * vm[11]));
}

// Camera model in isolation (for pinning the restatement): camera-space point -> pixel and pixel -> unit camera ray.
// `dist` as in make_camera (fisheye: 4 floats; pinhole: 12 floats or null).
int orc_cam_point_to_image(int model, const float* K, int W, int H, const float* dist, const float* p, float margin, float* out) {
    const Camera cam = make_camera(model, K, W, H, dist);
    V2 o;
    const bool valid = cam_point_to_image(cam, V3{p[0], p[1], p[2]}, margin, o);
    out[0] = o.x; out[1] = o.y;
    return valid ? 1 : 0;
}
int orc_image_to_cam_ray(int model, const float* K, int W, int H, const float* dist, float px, float py, float* ray) {
    const Camera cam = make_camera(model, K, W, H, dist);
    V3 r;
    const bool valid = image_to_cam_ray(cam, px, py, r);
    ray[0] = r.x; ray[1] = r.y; ray[2] = r.z;
    return valid ? 1 : 0;
}

int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

}  // extern "C"
