// Per-Gaussian stage of the EWA rasterizer. Compile with --fmad=false: the tile bounds, the exact per-tile test and
// the depth keys feed integer tile lists that must not depend on contraction choices.
//
// Replaces preprocess_cu (src/training/fastgs/rasterization/include/kernels_forward.cuh:19-192). exp / log go through
// double and are rounded once (the reference calls expf / logf) so that a host evaluation gives the same floats.
#include "ewa.cuh"
#include "ewa_common.cuh"

namespace lfs {
namespace {

__device__ __forceinline__ float exp_d(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float log_d(float x) { return (float)log((double)x); }

// colour = 0.5 + sum_k basis_k(dir) coeff_k with the closed-form real SH basis up to degree 3
__device__ __forceinline__ void ewa_sh_basis(float x, float y, float z, int nb, float* B) {
    B[0] = 0.28209479177387814f;
    if (nb <= 1) return;
    B[1] = -0.48860251190291987f * y; B[2] = 0.48860251190291987f * z; B[3] = -0.48860251190291987f * x;
    if (nb <= 4) return;
    const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
    B[4] = 1.0925484305920792f * xy; B[5] = -1.0925484305920792f * yz; B[6] = 0.94617469575755997f * zz - 0.31539156525251999f;
    B[7] = -1.0925484305920792f * xz; B[8] = 0.54627421529603959f * xx - 0.54627421529603959f * yy;
    if (nb <= 9) return;
    B[9] = 0.59004358992664352f * y * (-3.0f * xx + yy); B[10] = 2.8906114426405538f * xy * z;
    B[11] = 0.45704579946446572f * y * (1.0f - 5.0f * zz); B[12] = 0.3731763325901154f * z * (5.0f * zz - 3.0f);
    B[13] = 0.45704579946446572f * x * (1.0f - 5.0f * zz); B[14] = 1.4453057213202769f * z * (xx - yy);
    B[15] = 0.59004358992664352f * x * (-xx + 3.0f * yy);
}

__global__ void __launch_bounds__(256, 4) ewa_preprocess_kernel(
    int N, const float* __restrict__ means, const float* __restrict__ sh0, const float* __restrict__ shN,
    const float* __restrict__ scaling_raw, const float* __restrict__ rotation_raw, const float* __restrict__ opacity_raw,
    EwaCamera cam, int32_t* __restrict__ n_touched, ushort4* __restrict__ bounds, float4* __restrict__ records,
    uint32_t* __restrict__ sort_keys, uint32_t* __restrict__ sort_vals, float4* __restrict__ accum, int32_t* __restrict__ n_visible) {
    int local_visible = 0;
    float r1[4], r2[4], r3[4], campos[3];
#pragma unroll
    for (int k = 0; k < 4; ++k) { r1[k] = cam.w2c[k]; r2[k] = cam.w2c[4 + k]; r3[k] = cam.w2c[8 + k]; }
#pragma unroll
    for (int k = 0; k < 3; ++k) campos[k] = cam.campos[k];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < N; i += gridDim.x * blockDim.x) {
        sort_vals[i] = (uint32_t)i;
        int count = 0;
        const float m0 = means[i * 3], m1 = means[i * 3 + 1], m2 = means[i * 3 + 2];
        const float depth = r3[0] * m0 + r3[1] * m1 + r3[2] * m2 + r3[3];
        bool active = !(depth < cam.near_plane || depth > cam.far_plane);
        float opacity = 0.f, ca = 0.f, cb = 0.f, cc = 0.f, mx = 0.f, my = 0.f, thr = 0.f;
        uint32_t x0 = 0, x1 = 0, y0 = 0, y1 = 0;
        if (active) {
            opacity = 1.0f / (1.0f + exp_d(-opacity_raw[i]));
            if (opacity < kEwaMinAlpha) active = false;
        }
        if (active) {
            const float var[3] = {exp_d(2.0f * scaling_raw[i * 3]), exp_d(2.0f * scaling_raw[i * 3 + 1]), exp_d(2.0f * scaling_raw[i * 3 + 2])};
            const float4 q = reinterpret_cast<const float4*>(rotation_raw)[i];
            const float qr = q.x, qx = q.y, qy = q.z, qz = q.w;
            const float n = qr * qr + qx * qx + qy * qy + qz * qz;
            if (n < 1e-8f) active = false;
            const float pxx = 2.0f * (qx * qx) / n, pyy = 2.0f * (qy * qy) / n, pzz = 2.0f * (qz * qz) / n;
            const float pxy = 2.0f * qx * qy / n, pxz = 2.0f * qx * qz / n, pyz = 2.0f * qy * qz / n;
            const float prx = 2.0f * qr * qx / n, pry = 2.0f * qr * qy / n, prz = 2.0f * qr * qz / n;
            const float R[9] = {1.0f - (pyy + pzz), pxy - prz, pry + pxz,
                                prz + pxy, 1.0f - (pxx + pzz), pyz - prx,
                                pxz - pry, prx + pyz, 1.0f - (pxx + pyy)};
            float RS[9];
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int k = 0; k < 3; ++k) RS[r * 3 + k] = R[r * 3 + k] * var[k];
            auto rowdot = [&](int a, int b) { return RS[a * 3] * R[b * 3] + RS[a * 3 + 1] * R[b * 3 + 1] + RS[a * 3 + 2] * R[b * 3 + 2]; };
            const float S[6] = {rowdot(0, 0), rowdot(0, 1), rowdot(0, 2), rowdot(1, 1), rowdot(1, 2), rowdot(2, 2)};
            const float x = (r1[0] * m0 + r1[1] * m1 + r1[2] * m2 + r1[3]) / depth;
            const float y = (r2[0] * m0 + r2[1] * m1 + r2[2] * m2 + r2[3]) / depth;
            const float Wf = (float)cam.W, Hf = (float)cam.H;
            const float tx = fminf(fmaxf(x, (-0.15f * Wf - cam.cx) / cam.fx), (1.15f * Wf - cam.cx) / cam.fx);
            const float ty = fminf(fmaxf(y, (-0.15f * Hf - cam.cy) / cam.fy), (1.15f * Hf - cam.cy) / cam.fy);
            const float j11 = cam.fx / depth, j13 = -j11 * tx, j22 = cam.fy / depth, j23 = -j22 * ty;
            float A1[3], A2[3], B1[3], B2[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) { A1[k] = j11 * r1[k] + j13 * r3[k]; A2[k] = j22 * r2[k] + j23 * r3[k]; }
            B1[0] = A1[0] * S[0] + A1[1] * S[1] + A1[2] * S[2];
            B1[1] = A1[0] * S[1] + A1[1] * S[3] + A1[2] * S[4];
            B1[2] = A1[0] * S[2] + A1[1] * S[4] + A1[2] * S[5];
            B2[0] = A2[0] * S[0] + A2[1] * S[1] + A2[2] * S[2];
            B2[1] = A2[0] * S[1] + A2[1] * S[3] + A2[2] * S[4];
            B2[2] = A2[0] * S[2] + A2[1] * S[4] + A2[2] * S[5];
            const float a = (B1[0] * A1[0] + B1[1] * A1[1] + B1[2] * A1[2]) + kEwaDilation;
            const float b = B1[0] * A2[0] + B1[1] * A2[1] + B1[2] * A2[2];
            const float c = (B2[0] * A2[0] + B2[1] * A2[1] + B2[2] * A2[2]) + kEwaDilation;
            const float det = a * c - b * b;
            if (det < 1e-8f) active = false;
            if (active) {
                ca = c / det; cb = -b / det; cc = a / det;
                mx = x * cam.fx + cam.cx;
                my = y * cam.fy + cam.cy;
                thr = log_d(opacity * kEwaMinAlphaRcp);
                const float factor = sqrtf(2.0f * thr);
                const float ex = fmaxf(factor * sqrtf(a) - 0.5f, 0.0f), ey = fmaxf(factor * sqrtf(c) - 0.5f, 0.0f);
                x0 = min((uint32_t)cam.tw, (uint32_t)max(0, __float2int_rd((mx - ex) / 16.0f)));
                x1 = min((uint32_t)cam.tw, (uint32_t)max(0, __float2int_ru((mx + ex) / 16.0f)));
                y0 = min((uint32_t)cam.th, (uint32_t)max(0, __float2int_rd((my - ey) / 16.0f)));
                y1 = min((uint32_t)cam.th, (uint32_t)max(0, __float2int_ru((my + ey) / 16.0f)));
                // exact number of tiles the ellipse reaches
                for (uint32_t tyi = y0; tyi < y1; ++tyi)
                    for (uint32_t txi = x0; txi < x1; ++txi)
                        count += ewa_tile_contributes(mx - 0.5f, my - 0.5f, ca, cb, cc, txi, tyi, thr) ? 1 : 0;
            }
        }
        n_touched[i] = count;
        if (count == 0) {
            sort_keys[i] = 0xFFFFFFFFu;
            continue;
        }
        ++local_visible;
        sort_keys[i] = __float_as_uint(depth);
        bounds[i] = make_ushort4((unsigned short)x0, (unsigned short)x1, (unsigned short)y0, (unsigned short)y1);
        // colour
        float rgb[3];
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) rgb[ch] = 0.5f + 0.28209479177387814f * sh0[i * 3 + ch];
        if (cam.active_sh_bases > 1) {
            const float dx = m0 - campos[0], dy = m1 - campos[1], dz = m2 - campos[2];
            const float inv = 1.0f / sqrtf(dx * dx + dy * dy + dz * dz);
            const int nb = cam.active_sh_bases > 9 ? 16 : cam.active_sh_bases > 4 ? 9 : 4;
            float B[16];
            ewa_sh_basis(dx * inv, dy * inv, dz * inv, nb, B);
            const float* co = shN + (size_t)i * cam.total_rest * 3;
            for (int k = 1; k < nb; ++k) {
#pragma unroll
                for (int ch = 0; ch < 3; ++ch) rgb[ch] += B[k] * co[(k - 1) * 3 + ch];
            }
        }
        const uint32_t mask = (rgb[0] >= 0.f ? 1u : 0u) | (rgb[1] >= 0.f ? 2u : 0u) | (rgb[2] >= 0.f ? 4u : 0u);
        records[(size_t)i * 3 + 0] = make_float4(mx, my, ca, cb);
        records[(size_t)i * 3 + 1] = make_float4(cc, opacity, fmaxf(rgb[0], 0.f), fmaxf(rgb[1], 0.f));
        records[(size_t)i * 3 + 2] = make_float4(fmaxf(rgb[2], 0.f), __uint_as_float(mask), thr, 0.f);
#pragma unroll
        for (int k = 0; k < 3; ++k) accum[(size_t)i * 3 + k] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    local_visible = __reduce_add_sync(0xffffffffu, local_visible);
    if ((threadIdx.x & 31) == 0 && local_visible) atomicAdd(n_visible, local_visible);
}

}  // namespace

int launch_ewa_preprocess(int N, const lfs_splats& p, const EwaCamera& cam, int32_t* n_touched,
                          ushort4* bounds, float4* records, uint32_t* sort_keys, uint32_t* sort_vals, float4* accum,
                          int32_t* n_visible, cudaStream_t st) {
    if (N == 0) return LFS_OK;
    LFS_TIMED("ewa_preprocess", st);
    ewa_preprocess_kernel<<<grid_for(N, 256), 256, 0, st>>>(N, p.means, p.sh0, p.shN, p.scaling_raw, p.rotation_raw, p.opacity_raw,
                                                            cam, n_touched, bounds, records, sort_keys, sort_vals, accum, n_visible);
    return check_launch("ewa_preprocess");
}

}  // namespace lfs
