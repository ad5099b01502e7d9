// Shared pieces of the EWA (default, non --gut) rasterizer: constants of
// src/training/fastgs/rasterization/include/rasterization_config.h:12-30 and the ellipse-versus-rectangle test of
// include/kernel_utils.cuh:103-139 (will_primitive_contribute), generalised from a 16x16 tile to any pixel
// rectangle so that the blend kernels can use it on a warp's 8x4 patch as well.
#pragma once

#include "common.cuh"

namespace lfs {

constexpr float kEwaDilation = 0.3f;
constexpr float kEwaMinAlphaRcp = 255.0f;
constexpr float kEwaMinAlpha = 1.0f / 255.0f;
constexpr float kEwaMaxAlpha = 0.999f;
constexpr float kEwaMinTransmittance = 1e-4f;

// Packed per-Gaussian record of the EWA path, three float4:
//   r0 = (mean2d.x, mean2d.y, conic.xx, conic.xy)
//   r1 = (conic.yy, opacity, red, green)        colour already clamped at 0
//   r2 = (blue, colour-gradient mask bits (bit c set when the unclamped channel c >= 0), power threshold ln(255 opacity), 0)
constexpr int kEwaRecordVec4 = 3;

// Does the region {0.5 d^T conic d <= power_threshold} around (mx, my) reach the rectangle of pixel coordinates
// [min_x, max_x] x [min_y, max_y]? (mx, my) is the 2-D mean shifted by -0.5 so that pixel centres sit on integers.
// The point of the rectangle with the smallest exponent lies either inside (mean inside) or on the two edges that
// face the mean; each edge is searched by the closed-form minimiser of the quadratic along it, clamped to the edge.
__device__ __forceinline__ bool ewa_rect_contributes(float mx, float my, float ca, float cb, float cc, float min_x, float max_x,
                                                     float min_y, float max_y, float power_threshold) {
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
    const float dx = copysignf(max_x - min_x, x_min_diff), dy = copysignf(max_y - min_y, y_min_diff);
    const float t_x = not_in_y * __saturatef((dx * ca * diff_x + dx * cb * diff_y) / (dx * ca * dx));
    const float t_y = not_in_x * __saturatef((dy * cb * diff_x + dy * cc * diff_y) / (dy * cc * dy));
    const float px = corner_x + t_x * dx, py = corner_y + t_y * dy;
    const float ex = mx - px, ey = my - py;
    const float power = 0.5f * (ca * ex * ex + cc * ey * ey) + cb * ex * ey;
    return power <= power_threshold;
}

__device__ __forceinline__ bool ewa_tile_contributes(float mx, float my, float ca, float cb, float cc, uint32_t tile_x,
                                                     uint32_t tile_y, float power_threshold) {
    return ewa_rect_contributes(mx, my, ca, cb, cc, (float)(tile_x * 16u), (float)(tile_x * 16u + 15u), (float)(tile_y * 16u),
                                (float)(tile_y * 16u + 15u), power_threshold);
}

}  // namespace lfs
