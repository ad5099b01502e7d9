// TEST INFRASTRUCTURE, NOT PRODUCT CODE. PARITY UNPINNED (the reference has no golden vectors for this path
// and its CUDA sources cannot be run where this is built).
//
// CPU restatement of the reference's default (non --gut) rasterizer: EWA splatting with exact per-tile culling,
// src/training/fastgs/rasterization/ (include/kernels_forward.cuh, include/kernels_backward.cuh,
// include/kernel_utils.cuh, src/forward.cu, src/backward.cu) with the glue of
// src/training/rasterization/fast_rasterizer.cpp:13-71. Scalar IEEE float32 in the reference's operation order,
// compiled with -ffp-contract=off; gradient sums in double in a fixed order.
//
// Deliberate differences, shared with the CUDA library so that the two agree bit for bit on everything that
// decides a tile list: exp / log are evaluated in double and rounded once (the reference calls expf / logf);
// depth ties are broken by the Gaussian index (the reference's order of equal depths depends on the order in
// which atomicAdd hands out slots, kernels_forward.cuh:188-191).
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {

constexpr float kDilation = 0.3f;              // rasterization_config.h:14
constexpr float kMinAlphaRcp = 255.0f;         // :15
constexpr float kMinAlpha = 1.0f / 255.0f;     // :16
constexpr float kMaxAlpha = 0.999f;            // :17
constexpr float kTransmittanceMin = 1e-4f;     // :18
constexpr int kTile = 16;                      // :26-27

inline float exp_d(float x) { return (float)std::exp((double)x); }
inline float log_d(float x) { return (float)std::log((double)x); }
inline float clampf(float v, float lo, float hi) { return std::fmin(std::fmax(v, lo), hi); }
inline float saturate(float v) { return std::isnan(v) ? 0.0f : std::fmin(std::fmax(v, 0.0f), 1.0f); }  // __saturatef

struct Geo {                  // everything preprocess derives from one Gaussian and the camera
    bool active;
    float depth, x, y;        // camera z, normalised image coordinates
    float R[9], var[3];       // rotation (row-major), variances exp(2 raw_scale)
    float q[4], qn2;          // raw quaternion (r, x, y, z), squared norm
    float p[9];               // 2 q_a q_b / |q|^2: xx yy zz xy xz yz rx ry rz
    float cov3[6];            // 11 12 13 22 23 33
    float tx, ty, j11, j13, j22, j23;
    float A1[3], A2[3];       // rows of J W
    float B1[3], B2[3];       // rows of J W Sigma
    float a, b, c, det;       // dilated 2-D covariance
};

// kernels_forward.cuh:62-151 (and the identical recomputation of kernels_backward.cuh:60-124)
Geo geometry(const float* mean, const float* raw_scale, const float* rq, const float* w2c, float W, float H, float fx,
             float fy, float cx, float cy) {
    Geo g{};
    g.active = true;
    const float* r1 = w2c;
    const float* r2 = w2c + 4;
    const float* r3 = w2c + 8;
    g.depth = r3[0] * mean[0] + r3[1] * mean[1] + r3[2] * mean[2] + r3[3];
    for (int k = 0; k < 3; ++k) g.var[k] = exp_d(2.0f * raw_scale[k]);
    const float qr = rq[0], qx = rq[1], qy = rq[2], qz = rq[3];
    for (int k = 0; k < 4; ++k) g.q[k] = rq[k];
    const float rr = qr * qr, xx = qx * qx, yy = qy * qy, zz = qz * qz;
    g.qn2 = rr + xx + yy + zz;
    const float n = g.qn2;
    float* p = g.p;
    p[0] = 2.0f * xx / n; p[1] = 2.0f * yy / n; p[2] = 2.0f * zz / n;
    p[3] = 2.0f * qx * qy / n; p[4] = 2.0f * qx * qz / n; p[5] = 2.0f * qy * qz / n;
    p[6] = 2.0f * qr * qx / n; p[7] = 2.0f * qr * qy / n; p[8] = 2.0f * qr * qz / n;
    float* R = g.R;
    R[0] = 1.0f - (p[1] + p[2]); R[1] = p[3] - p[8];          R[2] = p[7] + p[4];
    R[3] = p[8] + p[3];          R[4] = 1.0f - (p[0] + p[2]); R[5] = p[5] - p[6];
    R[6] = p[4] - p[7];          R[7] = p[6] + p[5];          R[8] = 1.0f - (p[0] + p[1]);
    float RS[9];
    for (int i = 0; i < 3; ++i) for (int k = 0; k < 3; ++k) RS[i * 3 + k] = R[i * 3 + k] * g.var[k];
    auto rowdot = [&](int i, int j) { return RS[i * 3] * R[j * 3] + RS[i * 3 + 1] * R[j * 3 + 1] + RS[i * 3 + 2] * R[j * 3 + 2]; };
    g.cov3[0] = rowdot(0, 0); g.cov3[1] = rowdot(0, 1); g.cov3[2] = rowdot(0, 2);
    g.cov3[3] = rowdot(1, 1); g.cov3[4] = rowdot(1, 2); g.cov3[5] = rowdot(2, 2);
    g.x = (r1[0] * mean[0] + r1[1] * mean[1] + r1[2] * mean[2] + r1[3]) / g.depth;
    g.y = (r2[0] * mean[0] + r2[1] * mean[1] + r2[2] * mean[2] + r2[3]) / g.depth;
    const float clip_l = (-0.15f * W - cx) / fx, clip_r = (1.15f * W - cx) / fx;
    const float clip_t = (-0.15f * H - cy) / fy, clip_b = (1.15f * H - cy) / fy;
    g.tx = clampf(g.x, clip_l, clip_r);
    g.ty = clampf(g.y, clip_t, clip_b);
    g.j11 = fx / g.depth; g.j13 = -g.j11 * g.tx;
    g.j22 = fy / g.depth; g.j23 = -g.j22 * g.ty;
    for (int k = 0; k < 3; ++k) {
        g.A1[k] = g.j11 * r1[k] + g.j13 * r3[k];
        g.A2[k] = g.j22 * r2[k] + g.j23 * r3[k];
    }
    const float* S = g.cov3;
    auto symmul = [&](const float* v, float* o) {
        o[0] = v[0] * S[0] + v[1] * S[1] + v[2] * S[2];
        o[1] = v[0] * S[1] + v[1] * S[3] + v[2] * S[4];
        o[2] = v[0] * S[2] + v[1] * S[4] + v[2] * S[5];
    };
    symmul(g.A1, g.B1);
    symmul(g.A2, g.B2);
    auto d3 = [](const float* u, const float* v) { return u[0] * v[0] + u[1] * v[1] + u[2] * v[2]; };
    g.a = d3(g.B1, g.A1) + kDilation;
    g.b = d3(g.B1, g.A2);
    g.c = d3(g.B2, g.A2) + kDilation;
    g.det = g.a * g.c - g.b * g.b;
    return g;
}

// kernel_utils.cuh:103-139 will_primitive_contribute: does the ellipse {power <= threshold} reach the tile's pixel-centre
// rectangle? `mean` is the 2-D mean shifted by -0.5.
bool tile_contributes(float mx, float my, float ca, float cb, float cc, uint32_t tile_x, uint32_t tile_y, float power_threshold) {
    const float min_x = (float)(tile_x * kTile), min_y = (float)(tile_y * kTile);
    const float max_x = (float)((tile_x + 1) * kTile - 1), max_y = (float)((tile_y + 1) * kTile - 1);
    const float x_min_diff = min_x - mx;
    const float x_left = x_min_diff > 0.0f ? 1.0f : 0.0f;
    const float not_in_x = x_left + (mx > max_x ? 1.0f : 0.0f);
    const float y_min_diff = min_y - my;
    const float y_above = y_min_diff > 0.0f ? 1.0f : 0.0f;
    const float not_in_y = y_above + (my > max_y ? 1.0f : 0.0f);
    if (not_in_y + not_in_x == 0.0f) return true;
    const float corner_x = max_x + x_left * (min_x - max_x);
    const float corner_y = max_y + y_above * (min_y - max_y);
    const float diff_x = mx - corner_x, diff_y = my - corner_y;
    const float dx = std::copysign((float)(kTile - 1), x_min_diff), dy = std::copysign((float)(kTile - 1), y_min_diff);
    const float t_x = not_in_y * saturate((dx * ca * diff_x + dx * cb * diff_y) / (dx * ca * dx));
    const float t_y = not_in_x * saturate((dy * cb * diff_x + dy * cc * diff_y) / (dy * cc * dy));
    const float px = corner_x + t_x * dx, py = corner_y + t_y * dy;
    const float ex = mx - px, ey = my - py;
    const float power = 0.5f * (ca * ex * ex + cc * ey * ey) + cb * ex * ey;
    return power <= power_threshold;
}

// the 16 real SH basis values of kernel_utils.cuh:24-43 at a unit direction
void sh16(float x, float y, float z, float* B) {
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
    B[0] = 0.28209479177387814f;
    B[1] = -0.48860251190291987f * y; B[2] = 0.48860251190291987f * z; B[3] = -0.48860251190291987f * x;
    B[4] = 1.0925484305920792f * xy; B[5] = -1.0925484305920792f * yz; B[6] = 0.94617469575755997f * zz - 0.31539156525251999f;
    B[7] = -1.0925484305920792f * xz; B[8] = 0.54627421529603959f * xx - 0.54627421529603959f * yy;
    B[9] = 0.59004358992664352f * y * (-3.0f * xx + yy); B[10] = 2.8906114426405538f * xy * z;
    B[11] = 0.45704579946446572f * y * (1.0f - 5.0f * zz); B[12] = 0.3731763325901154f * z * (5.0f * zz - 3.0f);
    B[13] = 0.45704579946446572f * x * (1.0f - 5.0f * zz); B[14] = 1.4453057213202769f * z * (xx - yy);
    B[15] = 0.59004358992664352f * x * (-xx + 3.0f * yy);
}
// d B[k] / d (x, y, z) of the same closed forms (kernel_utils.cuh:62-95)
void sh16_grad(float x, float y, float z, float (*D)[3]) {
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
    for (int k = 0; k < 16; ++k) D[k][0] = D[k][1] = D[k][2] = 0.f;
    D[1][1] = -0.48860251190291987f; D[2][2] = 0.48860251190291987f; D[3][0] = -0.48860251190291987f;
    D[4][0] = 1.0925484305920792f * y; D[4][1] = 1.0925484305920792f * x;
    D[5][1] = -1.0925484305920792f * z; D[5][2] = -1.0925484305920792f * y;
    D[6][2] = 1.8923493915151202f * z;
    D[7][0] = -1.0925484305920792f * z; D[7][2] = -1.0925484305920792f * x;
    D[8][0] = 1.0925484305920792f * x; D[8][1] = -1.0925484305920792f * y;
    D[9][0] = -3.5402615395598609f * xy; D[9][1] = -1.7701307697799304f * xx + 1.7701307697799304f * yy;
    D[10][0] = 2.8906114426405538f * yz; D[10][1] = 2.8906114426405538f * xz; D[10][2] = 2.8906114426405538f * xy;
    D[11][1] = 0.45704579946446572f - 2.2852289973223288f * zz; D[11][2] = -4.5704579946446566f * yz;
    D[12][2] = 5.597644988851731f * zz - 1.1195289977703462f;
    D[13][0] = 0.45704579946446572f - 2.2852289973223288f * zz; D[13][2] = -4.5704579946446566f * xz;
    D[14][0] = 2.8906114426405538f * xz; D[14][1] = -2.8906114426405538f * yz; D[14][2] = 1.4453057213202769f * xx - 1.4453057213202769f * yy;
    D[15][0] = -1.7701307697799304f * xx + 1.7701307697799304f * yy; D[15][1] = 3.5402615395598609f * xy;
}

}  // namespace

extern "C" {

// preprocess_cu (kernels_forward.cuh:19-192). Outputs for culled Gaussians: n_touched = 0, the rest untouched.
// bounds [N,4] = (x_min, x_max, y_min, y_max) in tiles; conic_opacity [N,4]; color [N,3] UNCLAMPED; depth [N].
void orc_ewa_preprocess(int N, const float* means, const float* scales_raw, const float* rotations_raw, const float* opacities_raw,
                        const float* sh0, const float* shN, const float* w2c, const float* cam_position, int active_sh_bases,
                        int total_rest, int W, int H, float fx, float fy, float cx, float cy, float near_plane, float far_plane,
                        int32_t* n_touched, int32_t* bounds, float* mean2d, float* conic_opacity, float* color, float* depth) {
    const uint32_t gw = (W + kTile - 1) / kTile, gh = (H + kTile - 1) / kTile;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; ++i) {
        n_touched[i] = 0;
        const float* mean = means + (size_t)i * 3;
        const Geo g = geometry(mean, scales_raw + (size_t)i * 3, rotations_raw + (size_t)i * 4, w2c, (float)W, (float)H, fx, fy, cx, cy);
        if (g.depth < near_plane || g.depth > far_plane) continue;
        const float opacity = 1.0f / (1.0f + exp_d(-opacities_raw[i]));
        if (opacity < kMinAlpha) continue;
        if (g.qn2 < 1e-8f) continue;
        if (g.det < 1e-8f) continue;
        const float ca = g.c / g.det, cb = -g.b / g.det, cc = g.a / g.det;
        const float mx = g.x * fx + cx, my = g.y * fy + cy;
        const float power_threshold = log_d(opacity * kMinAlphaRcp);
        const float factor = std::sqrt(2.0f * power_threshold);
        const float ext_x = std::fmax(factor * std::sqrt(g.a) - 0.5f, 0.0f);
        const float ext_y = std::fmax(factor * std::sqrt(g.c) - 0.5f, 0.0f);
        // __float2int_rd / __float2int_ru saturate; keep the cast defined for huge extents
        auto sat = [](float v) { return (int)std::fmin(std::fmax(v, -1.0e9f), 1.0e9f); };
        auto lo = [&](float v, uint32_t cap) { return std::min(cap, (uint32_t)std::max(0, sat(std::floor(v)))); };
        auto hi = [&](float v, uint32_t cap) { return std::min(cap, (uint32_t)std::max(0, sat(std::ceil(v)))); };
        const uint32_t x0 = lo((mx - ext_x) / (float)kTile, gw), x1 = hi((mx + ext_x) / (float)kTile, gw);
        const uint32_t y0 = lo((my - ext_y) / (float)kTile, gh), y1 = hi((my + ext_y) / (float)kTile, gh);
        if ((x1 - x0) * (y1 - y0) == 0) continue;
        int cnt = 0;
        for (uint32_t ty = y0; ty < y1; ++ty)
            for (uint32_t tx = x0; tx < x1; ++tx)
                cnt += tile_contributes(mx - 0.5f, my - 0.5f, ca, cb, cc, tx, ty, power_threshold) ? 1 : 0;
        if (cnt == 0) continue;
        n_touched[i] = cnt;
        bounds[i * 4] = x0; bounds[i * 4 + 1] = x1; bounds[i * 4 + 2] = y0; bounds[i * 4 + 3] = y1;
        mean2d[i * 2] = mx; mean2d[i * 2 + 1] = my;
        conic_opacity[i * 4] = ca; conic_opacity[i * 4 + 1] = cb; conic_opacity[i * 4 + 2] = cc; conic_opacity[i * 4 + 3] = opacity;
        depth[i] = g.depth;
        // convert_sh_to_color (kernel_utils.cuh:15-45)
        float res[3];
        for (int c = 0; c < 3; ++c) res[c] = 0.5f + 0.28209479177387814f * sh0[(size_t)i * 3 + c];
        if (active_sh_bases > 1) {
            const float dx = mean[0] - cam_position[0], dy = mean[1] - cam_position[1], dz = mean[2] - cam_position[2];
            const float inv = 1.0f / std::sqrt(dx * dx + dy * dy + dz * dz);
            float B[16];
            sh16(dx * inv, dy * inv, dz * inv, B);
            const int nb = active_sh_bases > 9 ? 16 : active_sh_bases > 4 ? 9 : 4;
            const float* co = shN + (size_t)i * total_rest * 3;
            for (int k = 1; k < nb; ++k)
                for (int c = 0; c < 3; ++c) res[c] += B[k] * co[(k - 1) * 3 + c];
        }
        for (int c = 0; c < 3; ++c) color[(size_t)i * 3 + c] = res[c];
    }
}

// Depth order, instance creation with the per-tile test, stable tile sort, per-tile ranges
// (src/forward.cu:101-160, kernels_forward.cuh:194-334). instance_ids needs room for sum(n_touched) entries.
// tile_offsets [n_tiles + 1]. Returns the number of instances.
int64_t orc_ewa_lists(int N, const int32_t* n_touched, const int32_t* bounds, const float* mean2d, const float* conic_opacity,
                      const float* depth, int W, int H, int32_t* instance_ids, int32_t* tile_offsets) {
    const uint32_t gw = (W + kTile - 1) / kTile, gh = (H + kTile - 1) / kTile;
    std::vector<int> order;
    for (int i = 0; i < N; ++i) if (n_touched[i] > 0) order.push_back(i);
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
        uint32_t ka, kb;
        std::memcpy(&ka, &depth[a], 4); std::memcpy(&kb, &depth[b], 4);
        return ka < kb;
    });
    std::vector<std::vector<int32_t>> per_tile(gw * gh);
    for (int i : order) {
        const float ca = conic_opacity[i * 4], cb = conic_opacity[i * 4 + 1], cc = conic_opacity[i * 4 + 2];
        const float thr = log_d(conic_opacity[i * 4 + 3] * kMinAlphaRcp);
        for (uint32_t ty = bounds[i * 4 + 2]; ty < (uint32_t)bounds[i * 4 + 3]; ++ty)
            for (uint32_t tx = bounds[i * 4]; tx < (uint32_t)bounds[i * 4 + 1]; ++tx)
                if (tile_contributes(mean2d[i * 2] - 0.5f, mean2d[i * 2 + 1] - 0.5f, ca, cb, cc, tx, ty, thr))
                    per_tile[ty * gw + tx].push_back(i);
    }
    int64_t n = 0;
    for (uint32_t t = 0; t < gw * gh; ++t) {
        tile_offsets[t] = (int32_t)n;
        for (int32_t id : per_tile[t]) instance_ids[n++] = id;
    }
    tile_offsets[gw * gh] = (int32_t)n;
    return n;
}

// blend_cu (kernels_forward.cuh:336-459) plus the background of fast_rasterizer.cpp:67. image [3,H,W], alpha [H,W],
// n_contrib [H,W] = 1 + position (within the tile's list) of the last contributing entry, 0 if none.
void orc_ewa_blend_fwd(int W, int H, const int32_t* instance_ids, const int32_t* tile_offsets, const float* mean2d,
                       const float* conic_opacity, const float* color, const float* background /*nullable [3]*/, float* image,
                       float* alpha, int32_t* n_contrib) {
    const int gw = (W + kTile - 1) / kTile, gh = (H + kTile - 1) / kTile;
    const size_t np = (size_t)W * H;
#pragma omp parallel for schedule(dynamic, 1)
    for (int tile = 0; tile < gw * gh; ++tile) {
        const int x0 = (tile % gw) * kTile, y0 = (tile / gw) * kTile;
        const int beg = tile_offsets[tile], end = tile_offsets[tile + 1];
        for (int py = y0; py < std::min(H, y0 + kTile); ++py)
            for (int px = x0; px < std::min(W, x0 + kTile); ++px) {
                const float fx_ = (float)px + 0.5f, fy_ = (float)py + 0.5f;
                float T = 1.0f, col[3] = {0.f, 0.f, 0.f};
                int last = 0;
                for (int e = beg; e < end; ++e) {
                    const int g = instance_ids[e];
                    const float dx = mean2d[g * 2] - fx_, dy = mean2d[g * 2 + 1] - fy_;
                    const float ca = conic_opacity[g * 4], cb = conic_opacity[g * 4 + 1], cc = conic_opacity[g * 4 + 2];
                    const float sigma = 0.5f * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    if (sigma < 0.0f) continue;
                    const float a = std::fmin(conic_opacity[g * 4 + 3] * std::exp(-sigma), kMaxAlpha);
                    if (a < kMinAlpha) continue;
                    const float nT = T * (1.0f - a);
                    if (nT < kTransmittanceMin) break;
                    for (int c = 0; c < 3; ++c) col[c] += T * a * std::fmax(color[(size_t)g * 3 + c], 0.0f);
                    T = nT;
                    last = e - beg + 1;
                }
                const size_t pid = (size_t)py * W + px;
                for (int c = 0; c < 3; ++c) image[c * np + pid] = col[c] + (background ? T * background[c] : 0.0f);
                alpha[pid] = 1.0f - T;
                n_contrib[pid] = last;
            }
    }
}

// blend_backward_cu (kernels_backward.cuh:236-448), evaluated per pixel from the last contributor back to the
// first (the reference walks front to back from stored per-bucket states; the sums are the same).
// grad_image [3,H,W] and grad_alpha [H,W] are the gradients of the FINAL image (with background) and of alpha.
// Outputs (overwritten): grad_mean2d [N,2], grad_conic [N,3] (off-diagonal stored with the reference's factor 1/2),
// grad_raw_opacity [N], grad_color [N,3] (after the clamp-at-zero mask).
void orc_ewa_blend_bwd(int N, int W, int H, const int32_t* instance_ids, const int32_t* tile_offsets, const float* mean2d,
                       const float* conic_opacity, const float* color, const float* background, const float* alpha,
                       const int32_t* n_contrib, const float* grad_image, const float* grad_alpha, float* grad_mean2d,
                       float* grad_conic, float* grad_raw_opacity, float* grad_color) {
    const int gw = (W + kTile - 1) / kTile, gh = (H + kTile - 1) / kTile;
    const size_t np = (size_t)W * H;
    std::vector<double> acc((size_t)N * 9, 0.0);
    for (int tile = 0; tile < gw * gh; ++tile) {
        const int x0 = (tile % gw) * kTile, y0 = (tile / gw) * kTile;
        const int beg = tile_offsets[tile];
        for (int py = y0; py < std::min(H, y0 + kTile); ++py)
            for (int px = x0; px < std::min(W, x0 + kTile); ++px) {
                const size_t pid = (size_t)py * W + px;
                const float fx_ = (float)px + 0.5f, fy_ = (float)py + 0.5f;
                const float gi[3] = {grad_image[pid], grad_image[np + pid], grad_image[2 * np + pid]};
                const float T_final = 1.0f - alpha[pid];
                // d(final)/d(alpha map) through the background: image + (1 - alpha) bg
                float ga = grad_alpha ? grad_alpha[pid] : 0.0f;
                if (background) ga -= gi[0] * background[0] + gi[1] * background[1] + gi[2] * background[2];
                const float ga_common = ga * T_final;
                float T = T_final, after[3] = {0.f, 0.f, 0.f};
                for (int e = beg + n_contrib[pid] - 1; e >= beg; --e) {
                    const int g = instance_ids[e];
                    const float dx = mean2d[g * 2] - fx_, dy = mean2d[g * 2 + 1] - fy_;
                    const float ca = conic_opacity[g * 4], cb = conic_opacity[g * 4 + 1], cc = conic_opacity[g * 4 + 2];
                    const float sigma = 0.5f * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    if (sigma < 0.0f) continue;
                    const float a = std::fmin(conic_opacity[g * 4 + 3] * std::exp(-sigma), kMaxAlpha);
                    if (a < kMinAlpha) continue;
                    const float rcp = 1.0f / (1.0f - a);
                    T *= rcp;  // transmittance in front of this entry
                    const float w = T * a;
                    double* out = &acc[(size_t)g * 9];
                    float dL_da = ga_common * rcp;
                    for (int c = 0; c < 3; ++c) {
                        const float cu = color[(size_t)g * 3 + c];
                        const float cl = std::fmax(cu, 0.0f);
                        if (cu >= 0.0f) out[6 + c] += (double)(w * gi[c]);
                        dL_da += (T * cl - after[c] * rcp) * gi[c];
                        after[c] += w * cl;
                    }
                    out[5] += (double)(a * dL_da);
                    const float h = -a * dL_da;
                    out[2] += (double)(0.5f * h * dx * dx);
                    out[3] += (double)(0.5f * h * dx * dy);
                    out[4] += (double)(0.5f * h * dy * dy);
                    out[0] += (double)(h * (ca * dx + cb * dy));
                    out[1] += (double)(h * (cb * dx + cc * dy));
                }
            }
    }
    for (int g = 0; g < N; ++g) {
        const double* a = &acc[(size_t)g * 9];
        grad_mean2d[g * 2] = (float)a[0]; grad_mean2d[g * 2 + 1] = (float)a[1];
        grad_conic[g * 3] = (float)a[2]; grad_conic[g * 3 + 1] = (float)a[3]; grad_conic[g * 3 + 2] = (float)a[4];
        grad_raw_opacity[g] = (float)(a[5] * (1.0 - (double)conic_opacity[g * 4 + 3]));
        for (int c = 0; c < 3; ++c) grad_color[g * 3 + c] = (float)a[6 + c];
    }
}

// preprocess_backward_cu (kernels_backward.cuh:19-233); g_mean_cam [N,3] (nullable) receives the gradient of every
// camera-space mean, from which the caller sums the camera-pose gradient. Only Gaussians with
// n_touched > 0 are written; the others keep what the buffers held (the reference zero-fills them beforehand).
// densification_info [2,N] (nullable): row 0 += 1, row 1 += |grad_mean2d * (W/2, H/2)|.
void orc_ewa_preprocess_bwd(int N, const float* means, const float* scales_raw, const float* rotations_raw, const float* shN,
                            const float* w2c, const float* cam_position, const int32_t* n_touched, const float* grad_mean2d,
                            const float* grad_conic, const float* grad_color, int active_sh_bases, int total_rest, int W, int H,
                            float fx, float fy, float cx, float cy, float* g_means, float* g_scales_raw, float* g_rotations_raw,
                            float* g_sh0, float* g_shN, float* densification_info, float* g_mean_cam) {
    const float* r1 = w2c;
    const float* r2 = w2c + 4;
    const float* r3 = w2c + 8;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < N; ++i) {
        if (n_touched[i] == 0) continue;
        const float* mean = means + (size_t)i * 3;
        // ---- colour: coefficients and, through the view direction, the mean (kernel_utils.cuh:47-100)
        const float gc[3] = {grad_color[i * 3], grad_color[i * 3 + 1], grad_color[i * 3 + 2]};
        for (int c = 0; c < 3; ++c) g_sh0[(size_t)i * 3 + c] = 0.28209479177387814f * gc[c];
        float dmean_color[3] = {0.f, 0.f, 0.f};
        if (active_sh_bases > 1) {
            const float xr = mean[0] - cam_position[0], yr = mean[1] - cam_position[1], zr = mean[2] - cam_position[2];
            const float inv = 1.0f / std::sqrt(xr * xr + yr * yr + zr * zr);
            const float x = xr * inv, y = yr * inv, z = zr * inv;
            float B[16], D[16][3];
            sh16(x, y, z, B);
            sh16_grad(x, y, z, D);
            const int nb = active_sh_bases > 9 ? 16 : active_sh_bases > 4 ? 9 : 4;
            const float* co = shN + (size_t)i * total_rest * 3;
            float* gco = g_shN + (size_t)i * total_rest * 3;
            float gdir[3] = {0.f, 0.f, 0.f};
            for (int k = 1; k < nb; ++k) {
                float cg = 0.f;
                for (int c = 0; c < 3; ++c) {
                    gco[(k - 1) * 3 + c] = B[k] * gc[c];
                    cg += co[(k - 1) * 3 + c] * gc[c];
                }
                for (int a = 0; a < 3; ++a) gdir[a] += D[k][a] * cg;
            }
            const float xx = xr * xr, yy = yr * yr, zz = zr * zr, xy = xr * yr, xz = xr * zr, yz = yr * zr;
            const float n2 = xx + yy + zz;
            const float s = 1.0f / std::sqrt(n2 * n2 * n2);
            dmean_color[0] = ((yy + zz) * gdir[0] - xy * gdir[1] - xz * gdir[2]) * s;
            dmean_color[1] = (-xy * gdir[0] + (xx + zz) * gdir[1] - yz * gdir[2]) * s;
            dmean_color[2] = (-xz * gdir[0] - yz * gdir[1] + (xx + yy) * gdir[2]) * s;
        }
        // ---- geometry
        const Geo g = geometry(mean, scales_raw + (size_t)i * 3, rotations_raw + (size_t)i * 4, w2c, (float)W, (float)H, fx, fy, cx, cy);
        const float a = g.a, b = g.b, c = g.c;
        const float rcp = 1.0f / g.det, rcp2 = rcp * rcp;
        const float kx = grad_conic[i * 3], ky = grad_conic[i * 3 + 1], kz = grad_conic[i * 3 + 2];
        // d/d(cov2d) of conic = inverse(cov2d), symmetric-entry convention
        const float hx = rcp2 * (2.0f * (b * c) * ky - (c * c) * kx - (b * b) * kz);
        const float hy = rcp2 * ((b * c) * kx - ((a * c) + (b * b)) * ky + (a * b) * kz);
        const float hz = rcp2 * (2.0f * (a * b) * ky - (b * b) * kx - (a * a) * kz);
        const float* A1 = g.A1; const float* A2 = g.A2;
        // d/d(cov3d) = A^T H A, upper triangle 11 12 13 22 23 33
        float S[6];
        S[0] = (A1[0] * A1[0]) * hx + 2.0f * (A1[0] * A2[0]) * hy + (A2[0] * A2[0]) * hz;
        S[1] = (A1[0] * A1[1]) * hx + (A1[0] * A2[1] + A1[1] * A2[0]) * hy + (A2[0] * A2[1]) * hz;
        S[2] = (A1[0] * A1[2]) * hx + (A1[0] * A2[2] + A1[2] * A2[0]) * hy + (A2[0] * A2[2]) * hz;
        S[3] = (A1[1] * A1[1]) * hx + 2.0f * (A1[1] * A2[1]) * hy + (A2[1] * A2[1]) * hz;
        S[4] = (A1[1] * A1[2]) * hx + (A1[1] * A2[2] + A1[2] * A2[1]) * hy + (A2[1] * A2[2]) * hz;
        S[5] = (A1[2] * A1[2]) * hx + 2.0f * (A1[2] * A2[2]) * hy + (A2[2] * A2[2]) * hz;
        // d/d(A) = 2 H (A Sigma)
        float dA1[3], dA2[3];
        for (int k = 0; k < 3; ++k) {
            dA1[k] = 2.0f * (g.B1[k] * hx + g.B2[k] * hy);
            dA2[k] = 2.0f * (g.B1[k] * hy + g.B2[k] * hz);
        }
        const float dj11 = r1[0] * dA1[0] + r1[1] * dA1[1] + r1[2] * dA1[2];
        const float dj22 = r2[0] * dA2[0] + r2[1] * dA2[1] + r2[2] * dA2[2];
        const float dj13 = r3[0] * dA1[0] + r3[1] * dA1[1] + r3[2] * dA1[2];
        const float dj23 = r3[0] * dA2[0] + r3[1] * dA2[1] + r3[2] * dA2[2];
        const float hz1 = dj11 - 2.0f * g.tx * dj13;
        const float hz2 = dj22 - 2.0f * g.ty * dj23;
        const float m2x = grad_mean2d[i * 2], m2y = grad_mean2d[i * 2 + 1];
        const float dc[3] = {g.j11 * (m2x - dj13 / g.depth), g.j22 * (m2y - dj23 / g.depth),
                             -g.j11 * (g.x * m2x + hz1 / g.depth) - g.j22 * (g.y * m2y + hz2 / g.depth)};
        for (int k = 0; k < 3; ++k)
            g_means[(size_t)i * 3 + k] = (r1[k] * dc[0] + r2[k] * dc[1] + r3[k] * dc[2]) + dmean_color[k];
        if (g_mean_cam)   // the summands of the camera-pose gradient (kernels_backward.cuh:160-173)
            for (int k = 0; k < 3; ++k) g_mean_cam[(size_t)i * 3 + k] = dc[k];
        // variances: d/d(var_k) = r_k^T S r_k with r_k the k-th column of R
        const float* R = g.R;
        for (int k = 0; k < 3; ++k) {
            const float u = R[0 * 3 + k], v = R[1 * 3 + k], w = R[2 * 3 + k];
            const float dv = u * u * S[0] + v * v * S[3] + w * w * S[5] + 2.0f * (u * v * S[1] + u * w * S[2] + v * w * S[4]);
            g_scales_raw[(size_t)i * 3 + k] = 2.0f * g.var[k] * dv;
        }
        // rotation: d/dR = 2 S (R diag(var)), then through R(p) and p = 2 q_a q_b / |q|^2
        float RS[9], dR[9];
        for (int r = 0; r < 3; ++r) for (int k = 0; k < 3; ++k) RS[r * 3 + k] = R[r * 3 + k] * g.var[k];
        const float Sm[9] = {S[0], S[1], S[2], S[1], S[3], S[4], S[2], S[4], S[5]};
        for (int r = 0; r < 3; ++r)
            for (int k = 0; k < 3; ++k)
                dR[r * 3 + k] = 2.0f * (RS[0 * 3 + k] * Sm[r * 3 + 0] + RS[1 * 3 + k] * Sm[r * 3 + 1] + RS[2 * 3 + k] * Sm[r * 3 + 2]);
        const float dxx = -dR[4] - dR[8], dyy = -dR[0] - dR[8], dzz = -dR[0] - dR[4];
        const float dxy = dR[1] + dR[3], dxz = dR[2] + dR[6], dyz = dR[5] + dR[7];
        const float drx = dR[7] - dR[5], dry = dR[2] - dR[6], drz = dR[3] - dR[1];
        const float* p = g.p;
        const float nh = p[0] * dxx + p[1] * dyy + p[2] * dzz + p[3] * dxy + p[4] * dxz + p[5] * dyz + p[6] * drx + p[7] * dry + p[8] * drz;
        const float qr = g.q[0], qx = g.q[1], qy = g.q[2], qz = g.q[3];
        float* gq = g_rotations_raw + (size_t)i * 4;
        gq[0] = 2.0f * (qx * drx + qy * dry + qz * drz - qr * nh) / g.qn2;
        gq[1] = 2.0f * (2.0f * qx * dxx + qy * dxy + qz * dxz + qr * drx - qx * nh) / g.qn2;
        gq[2] = 2.0f * (2.0f * qy * dyy + qx * dxy + qz * dyz + qr * dry - qy * nh) / g.qn2;
        gq[3] = 2.0f * (2.0f * qz * dzz + qx * dxz + qy * dyz + qr * drz - qz * nh) / g.qn2;
        if (densification_info) {
            densification_info[i] += 1.0f;
            const float sx = m2x * (0.5f * (float)W), sy = m2y * (0.5f * (float)H);
            densification_info[N + i] += std::sqrt(sx * sx + sy * sy);
        }
    }
}

}  // extern "C"
