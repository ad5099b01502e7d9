// Separable 11x11 Gaussian-window SSIM (forward with derivative maps, backward) and the fused
// photometric loss 0.8 L1 + 0.2 (1 - SSIM_valid) with its gradient w.r.t. the unclamped HWC render.
//
// Replaces src/training/kernels/ssim.cu:64 (K9) and :284 (K10), the crop / pad / mean glue of
// include/kernels/fused_ssim.cuh:59-67, :85-96, :117-122, torch::l1_loss of
// src/training/trainer.cpp:126 and the clamp + permute of src/training/rasterization/rasterizer.cpp:205.
// Stencil work: each CTA stages the 42x42 halo tile of a 32x32 output tile of one channel in shared memory and runs
// the 11-tap horizontal and vertical passes from register windows (4 outputs per 14 loaded values).
#include "common.cuh"
#include "loss.cuh"

namespace lfs {

namespace {

constexpr int kT = 32;             // output tile edge
constexpr int kHalo = 5;
constexpr int kS = kT + 2 * kHalo;   // 42: halo tile edge
constexpr int kSX = kS + 1;          // 43: row stride of the staged images (conflict-free for lanes that walk rows)
constexpr int kSH = kT + 1;          // 33: row stride of the horizontally filtered planes
constexpr int kThreadsLoss = 256;
constexpr int kColGroups = kT / 4;   // a horizontal work item filters 4 adjacent columns of one row

__constant__ float cTaps[11] = {
    0.001028380123898387f, 0.0075987582094967365f, 0.036000773310661316f, 0.10936068743467331f,
    0.21300552785396576f,  0.26601171493530273f,   0.21300552785396576f,  0.10936068743467331f,
    0.036000773310661316f, 0.0075987582094967365f, 0.001028380123898387f};

// FUSED: img1 is the unclamped HWC render (clamped to [0,1] on load); otherwise plain CHW.
template <bool FUSED>
__device__ __forceinline__ float load_img1(const float* img1, int c, int y, int x, int H, int W) {
    if (x < 0 || x >= W || y < 0 || y >= H) return 0.f;
    if (FUSED) return fminf(1.f, fmaxf(0.f, img1[((size_t)y * W + x) * 3 + c]));
    return img1[(size_t)c * H * W + (size_t)y * W + x];
}
__device__ __forceinline__ float load_chw(const float* img, int c, int y, int x, int H, int W) {
    if (x < 0 || x >= W || y < 0 || y >= H) return 0.f;
    return img[(size_t)c * H * W + (size_t)y * W + x];
}

// 11-tap filter at centre index ci of a register window, symmetric pairs first (the reference's order of additions)
__device__ __forceinline__ float tap11(const float* v, int ci) {
    float a = 0.f;
#pragma unroll
    for (int d = 1; d <= kHalo; ++d) a += (v[ci - d] + v[ci + d]) * cTaps[kHalo - d];
    return a + v[ci] * cTaps[kHalo];
}

// One CTA filters a 32x32 output tile of one channel (blockIdx.z). The 42x42 halo tile is staged in shared memory;
// the horizontal pass gives every thread 4 adjacent outputs of one row from a 14-value register window (7 shared
// loads per output instead of 44), the vertical pass 4 stacked outputs of one column from 14-value windows of the five
// filtered planes.
//
// Forward. Plain mode writes ssim_map and the three derivative maps. Fused mode writes the derivative maps already
// multiplied by dL/dmap (map_grad inside the valid crop, 0 outside) and accumulates sum(ssim over the crop) and
// sum(|img1 - img2|) into sums[0], sums[1].
template <bool FUSED>
__global__ void __launch_bounds__(kThreadsLoss) ssim_fwd_kernel(int CH, int H, int W, float C1, float C2,
                                                               const float* __restrict__ img1, const float* __restrict__ img2,
                                                               float* __restrict__ ssim_map, float* __restrict__ dm_dmu1,
                                                               float* __restrict__ dm_dsigma1_sq, float* __restrict__ dm_dsigma12,
                                                               float map_grad, int crop, double* __restrict__ sums) {
    __shared__ float sX[kS][kSX], sY[kS][kSX];
    __shared__ float sH[5][kS][kSH];
    __shared__ float red[2][kThreadsLoss / 32];
    const int tid = threadIdx.x, c = blockIdx.z;
    const int bx0 = blockIdx.x * kT, by0 = blockIdx.y * kT;
    for (int q = tid; q < kS * kS; q += kThreadsLoss) {
        const int ly = q / kS, lx = q - ly * kS;
        sX[ly][lx] = load_img1<FUSED>(img1, c, by0 + ly - kHalo, bx0 + lx - kHalo, H, W);
        sY[ly][lx] = load_chw(img2, c, by0 + ly - kHalo, bx0 + lx - kHalo, H, W);
    }
    __syncthreads();
    for (int item = tid; item < kS * kColGroups; item += kThreadsLoss) {
        const int cg = item / kS, row = item - cg * kS;
        float xv[14], yv[14], q[14];
#pragma unroll
        for (int j = 0; j < 14; ++j) { xv[j] = sX[row][cg * 4 + j]; yv[j] = sY[row][cg * 4 + j]; }
#pragma unroll
        for (int o = 0; o < 4; ++o) sH[0][row][cg * 4 + o] = tap11(xv, o + kHalo);
#pragma unroll
        for (int o = 0; o < 4; ++o) sH[2][row][cg * 4 + o] = tap11(yv, o + kHalo);
#pragma unroll
        for (int j = 0; j < 14; ++j) q[j] = xv[j] * xv[j];
#pragma unroll
        for (int o = 0; o < 4; ++o) sH[1][row][cg * 4 + o] = tap11(q, o + kHalo);
#pragma unroll
        for (int j = 0; j < 14; ++j) q[j] = yv[j] * yv[j];
#pragma unroll
        for (int o = 0; o < 4; ++o) sH[3][row][cg * 4 + o] = tap11(q, o + kHalo);
#pragma unroll
        for (int j = 0; j < 14; ++j) q[j] = xv[j] * yv[j];
#pragma unroll
        for (int o = 0; o < 4; ++o) sH[4][row][cg * 4 + o] = tap11(q, o + kHalo);
    }
    __syncthreads();
    const int col = tid & 31, strip = tid >> 5;
    float out[4][5];
#pragma unroll
    for (int k = 0; k < 5; ++k) {
        float h[14];
#pragma unroll
        for (int j = 0; j < 14; ++j) h[j] = sH[k][strip * 4 + j][col];
#pragma unroll
        for (int o = 0; o < 4; ++o) out[o][k] = tap11(h, o + kHalo);
    }
    float ssim_acc = 0.f, l1_acc = 0.f;
    const int x = bx0 + col;
#pragma unroll
    for (int o = 0; o < 4; ++o) {
        const int y = by0 + strip * 4 + o;
        if (x < W && y < H) {
            const float mu1 = out[o][0], mu2 = out[o][2];
            const float mu1_sq = mu1 * mu1, mu2_sq = mu2 * mu2;
            const float sigma1_sq = out[o][1] - mu1_sq, sigma2_sq = out[o][3] - mu2_sq, sigma12 = out[o][4] - mu1 * mu2;
            const float A = mu1_sq + mu2_sq + C1, B = sigma1_sq + sigma2_sq + C2;
            const float C_ = 2.f * mu1 * mu2 + C1, D_ = 2.f * sigma12 + C2;
            const float val = (C_ * D_) / (A * B);
            const float g_mu1 = ((mu2 * 2.f * D_) / (A * B) - (mu2 * 2.f * C_) / (A * B) -
                                 (mu1 * 2.f * C_ * D_) / (A * A * B) + (mu1 * 2.f * C_ * D_) / (A * B * B));
            const float g_s1 = (-C_ * D_) / (A * B * B);
            const float g_s12 = (2.f * C_) / (A * B);
            const size_t gi = (size_t)c * H * W + (size_t)y * W + x;
            if (FUSED) {
                const bool in_crop = !crop || (x >= kHalo && x < W - kHalo && y >= kHalo && y < H - kHalo);
                const float chain = in_crop ? map_grad : 0.f;
                dm_dmu1[gi] = g_mu1 * chain;
                dm_dsigma1_sq[gi] = g_s1 * chain;
                dm_dsigma12[gi] = g_s12 * chain;
                if (in_crop) ssim_acc += val;
                const int ly = strip * 4 + o + kHalo, lx = col + kHalo;
                l1_acc += fabsf(sX[ly][lx] - sY[ly][lx]);
            } else {
                ssim_map[gi] = val;
                if (dm_dmu1) { dm_dmu1[gi] = g_mu1; dm_dsigma1_sq[gi] = g_s1; dm_dsigma12[gi] = g_s12; }
            }
        }
    }
    if (FUSED) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ssim_acc += __shfl_xor_sync(0xffffffffu, ssim_acc, o);
            l1_acc += __shfl_xor_sync(0xffffffffu, l1_acc, o);
        }
        if ((tid & 31) == 0) { red[0][tid >> 5] = ssim_acc; red[1][tid >> 5] = l1_acc; }
        __syncthreads();
        if (tid == 0) {
            double s_ = 0.0, l_ = 0.0;
            for (int k = 0; k < kThreadsLoss / 32; ++k) { s_ += red[0][k]; l_ += red[1][k]; }
            atomicAdd(&sums[0], s_);
            atomicAdd(&sums[1], l_);
        }
    }
}

// Backward, same tiling. Plain mode: maps are multiplied by dL_dmap on load and dL_dimg1 is CHW. Fused mode: the maps
// are pre-multiplied, the L1 sign term and the clamp mask are applied and the output is the HWC gradient of the
// unclamped render, scaled by grad_scale.
template <bool FUSED>
__global__ void __launch_bounds__(kThreadsLoss) ssim_bwd_kernel(int CH, int H, int W, const float* __restrict__ img1,
                                                               const float* __restrict__ img2, const float* __restrict__ dL_dmap,
                                                               const float* __restrict__ dm_dmu1, const float* __restrict__ dm_dsigma1_sq,
                                                               const float* __restrict__ dm_dsigma12, float* __restrict__ dL_dimg1,
                                                               float l1_grad, float grad_scale) {
    __shared__ float sD[3][kS][kSX];
    __shared__ float sH[3][kS][kSH];
    const int tid = threadIdx.x, c = blockIdx.z;
    const int bx0 = blockIdx.x * kT, by0 = blockIdx.y * kT;
    for (int q = tid; q < kS * kS; q += kThreadsLoss) {
        const int ly = q / kS, lx = q - ly * kS;
        const int gy = by0 + ly - kHalo, gx = bx0 + lx - kHalo;
        const float chain = FUSED ? 1.f : load_chw(dL_dmap, c, gy, gx, H, W);
        sD[0][ly][lx] = load_chw(dm_dmu1, c, gy, gx, H, W) * chain;
        sD[1][ly][lx] = load_chw(dm_dsigma1_sq, c, gy, gx, H, W) * chain;
        sD[2][ly][lx] = load_chw(dm_dsigma12, c, gy, gx, H, W) * chain;
    }
    __syncthreads();
    for (int item = tid; item < kS * kColGroups; item += kThreadsLoss) {
        const int cg = item / kS, row = item - cg * kS;
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            float v[14];
#pragma unroll
            for (int j = 0; j < 14; ++j) v[j] = sD[k][row][cg * 4 + j];
#pragma unroll
            for (int o = 0; o < 4; ++o) sH[k][row][cg * 4 + o] = tap11(v, o + kHalo);
        }
    }
    __syncthreads();
    const int col = tid & 31, strip = tid >> 5;
    float s[4][3];
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        float h[14];
#pragma unroll
        for (int j = 0; j < 14; ++j) h[j] = sH[k][strip * 4 + j][col];
#pragma unroll
        for (int o = 0; o < 4; ++o) s[o][k] = tap11(h, o + kHalo);
    }
    const int x = bx0 + col;
#pragma unroll
    for (int o = 0; o < 4; ++o) {
        const int y = by0 + strip * 4 + o;
        if (x < W && y < H) {
            if (FUSED) {
                const float raw = img1[((size_t)y * W + x) * 3 + c];
                const float p1 = fminf(1.f, fmaxf(0.f, raw));
                const float p2 = img2[(size_t)c * H * W + (size_t)y * W + x];
                float g = s[o][0] + (2.f * p1) * s[o][1] + (p2)*s[o][2];
                const float diff = p1 - p2;
                g += l1_grad * (diff > 0.f ? 1.f : (diff < 0.f ? -1.f : 0.f));
                if (!(raw >= 0.f && raw <= 1.f)) g = 0.f;
                dL_dimg1[((size_t)y * W + x) * 3 + c] = g * grad_scale;
            } else {
                const size_t gi = (size_t)c * H * W + (size_t)y * W + x;
                const float p1 = img1[gi], p2 = img2[gi];
                dL_dimg1[gi] = s[o][0] + (2.f * p1) * s[o][1] + (p2)*s[o][2];
            }
        }
    }
}

__global__ void loss_finalize_kernel(const double* sums, double n_all, double n_valid, float lambda, float* loss) {
    const float l1 = (float)(sums[1] / n_all);
    const float ssim = (float)(sums[0] / n_valid);
    loss[0] = (1.f - lambda) * l1 + lambda * (1.f - ssim);
    loss[1] = l1;
    loss[2] = ssim;
}

}  // namespace

int launch_fusedssim(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2, float* ssim_map,
                     float* dm1, float* ds1, float* ds12, cudaStream_t st) {
    if (CH * H * W == 0) return LFS_OK;
    dim3 grid((W + kT - 1) / kT, (H + kT - 1) / kT, CH), block(kThreadsLoss);
    ssim_fwd_kernel<false><<<grid, block, 0, st>>>(CH, H, W, C1, C2, img1, img2, ssim_map, dm1, ds1, ds12, 0.f, 0, nullptr);
    return check_launch("fusedssim");
}

int launch_fusedssim_backward(int CH, int H, int W, const float* img1, const float* img2, const float* dL_dmap,
                              const float* dm1, const float* ds1, const float* ds12, float* dL_dimg1, cudaStream_t st) {
    if (CH * H * W == 0) return LFS_OK;
    dim3 grid((W + kT - 1) / kT, (H + kT - 1) / kT, CH), block(kThreadsLoss);
    ssim_bwd_kernel<false><<<grid, block, 0, st>>>(CH, H, W, img1, img2, dL_dmap, dm1, ds1, ds12, dL_dimg1, 0.f, 1.f);
    return check_launch("fusedssim_backward");
}

namespace {
// out[c] += sum over pixels of v_render[p, c] * (1 - alpha[p]); one double atomic per CTA and channel.
__global__ void __launch_bounds__(256) background_gradient_kernel(int64_t P, int CH, const float* __restrict__ v_render,
                                                                  const float* __restrict__ alpha, double* __restrict__ acc) {
    double s[4] = {0.0, 0.0, 0.0, 0.0};
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < P; p += (int64_t)gridDim.x * blockDim.x) {
        const float w = 1.0f - alpha[p];
        for (int c = 0; c < CH; ++c) s[c] += (double)(v_render[p * CH + c] * w);
    }
    __shared__ double red[8][4];
    for (int c = 0; c < CH; ++c) {
        double v = s[c];
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5][c] = v;
    }
    __syncthreads();
    if (threadIdx.x < CH) {
        double v = 0.0;
        for (int w = 0; w < 8; ++w) v += red[w][threadIdx.x];
        atomicAdd(acc + threadIdx.x, v);
    }
}
__global__ void background_gradient_finalize_kernel(int CH, const double* __restrict__ acc, float* __restrict__ out) {
    if (threadIdx.x < CH) out[threadIdx.x] = (float)acc[threadIdx.x];
}
}  // namespace

int launch_background_gradient(int H, int W, int CH, const float* v_render, const float* alpha, float* v_background,
                               void* workspace, cudaStream_t st) {
    double* acc = reinterpret_cast<double*>(workspace);
    cudaMemsetAsync(acc, 0, 4 * sizeof(double), st);
    const int64_t P = (int64_t)H * W;
    if (P > 0) {
        LFS_TIMED("background_gradient", st);
        background_gradient_kernel<<<grid_for(P, 256, 4), 256, 0, st>>>(P, CH, v_render, alpha, acc);
    }
    background_gradient_finalize_kernel<<<1, 32, 0, st>>>(CH, acc, v_background);
    return check_launch("background_gradient");
}

size_t photometric_workspace_bytes(int H, int W) { return 256 + (size_t)3 * 3 * H * W * sizeof(float); }

int launch_photometric_loss(int H, int W, float lambda, float grad_scale, const float* render_hwc, const float* target_chw,
                            float* v_render_hwc, float* loss_dev, void* workspace, cudaStream_t st) {
    double* sums = reinterpret_cast<double*>(workspace);
    float* maps = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 256);
    const size_t plane = (size_t)3 * H * W;
    float *d1 = maps, *d2 = maps + plane, *d3 = maps + 2 * plane;
    const int crop = (H > 10 && W > 10) ? 1 : 0;
    const double n_all = 3.0 * H * W;
    const double n_valid = crop ? 3.0 * (H - 10) * (W - 10) : n_all;
    const float map_grad = (float)(-(double)lambda / n_valid);
    const float l1_grad = (float)((1.0 - (double)lambda) / n_all);
    cudaMemsetAsync(sums, 0, 2 * sizeof(double), st);
    dim3 grid((W + kT - 1) / kT, (H + kT - 1) / kT, 3), block(kThreadsLoss);
    {
    LFS_TIMED("loss_fwd", st);
    ssim_fwd_kernel<true><<<grid, block, 0, st>>>(3, H, W, (float)(0.01 * 0.01), (float)(0.03 * 0.03), render_hwc,
                                                  target_chw, nullptr, d1, d2, d3, map_grad, crop, sums);
    }
    if (v_render_hwc) {
        LFS_TIMED("loss_bwd", st);
        ssim_bwd_kernel<true><<<grid, block, 0, st>>>(3, H, W, render_hwc, target_chw, nullptr, d1, d2, d3, v_render_hwc,
                                                      l1_grad, grad_scale);
    }
    loss_finalize_kernel<<<1, 1, 0, st>>>(sums, n_all, n_valid, lambda, loss_dev);
    return check_launch("photometric_loss");
}

}  // namespace lfs
