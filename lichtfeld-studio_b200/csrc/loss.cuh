// Launchers of the loss stage (loss.cu).
#pragma once

#include "common.cuh"

namespace lfs {

int launch_fusedssim(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2, float* ssim_map,
                     float* dm1, float* ds1, float* ds12, cudaStream_t st);
int launch_fusedssim_backward(int CH, int H, int W, const float* img1, const float* img2, const float* dL_dmap,
                              const float* dm1, const float* ds1, const float* ds12, float* dL_dimg1, cudaStream_t st);
// v_background[c] = sum_p v_render[p, c] (1 - alpha[p]); workspace: 32 bytes of device scratch.
int launch_background_gradient(int H, int W, int CH, const float* v_render, const float* alpha, float* v_background,
                               void* workspace, cudaStream_t st);
size_t photometric_workspace_bytes(int H, int W);
int launch_photometric_loss(int H, int W, float lambda, float grad_scale, const float* render_hwc, const float* target_chw,
                            float* v_render_hwc, float* loss_dev, void* workspace, cudaStream_t st);

}  // namespace lfs
