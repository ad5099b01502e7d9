// Launchers of the streaming kernels (elementwise.cu).
#pragma once

#include "common.cuh"

namespace lfs {

struct AdamGroup {
    float* p; float* m; float* v; const float* g;
    int64_t n;        // elements in this group (already restricted to the row range)
    float step_size;  // lr * bias_correction1_rcp
    int aligned;      // all four pointers 16-byte aligned
};
struct AdamGroups {
    AdamGroup g[6];
    int64_t prefix4[7];  // prefix sums of ceil(n / 4)
    int n_groups;
    float beta1, beta2, eps, bc2_sqrt_rcp, grad_scale;
};

int launch_adam_groups(const AdamGroups& G, cudaStream_t st);

constexpr int kMaxAdamSegments = 16;
struct AdamSegments {
    AdamGroup g[kMaxAdamSegments];
    int64_t prefix4[kMaxAdamSegments + 1];
    int n;
    float beta1, beta2, eps, bc2_sqrt_rcp, grad_scale;
};
int launch_adam_segments(const AdamSegments& S, int ctas_per_sm, cudaStream_t st);

constexpr int kMaxPeers = 8;
struct DpSegment {
    int64_t offset, n;
    float* m; float* v;
    float step_size;
};
struct DpArgs {
    const float* grads[kMaxPeers];
    float* params[kMaxPeers];
    float* mc_params;          // NVSwitch multicast address of the parameter buffer, or nullptr: plain peer stores
    DpSegment seg[6];
    int64_t prefix4[7];
    int world, n_segments;
    float beta1, beta2, eps, bc2_sqrt_rcp, grad_scale;
};
int launch_dp_reduce_adam_broadcast(const DpArgs& A, int ctas_per_sm, cudaStream_t st);
int launch_regularization(int N, const float* scaling_raw, const float* opacity_raw, float scale_weight, float opacity_weight,
                          float* g_scaling, float* g_opacity, float* loss, cudaStream_t st);
int launch_sh_fwd(int n, int K, int degree, const float* dirs, const float* coeffs, const uint8_t* masks, float* colors, cudaStream_t st);
int launch_sh_bwd(int n, int K, int degree, const float* dirs, const uint8_t* masks, const float* v_colors, float* v_coeffs, cudaStream_t st);
int launch_relocation(int n, const float* opacities, const float* scales, const int32_t* ratios, const float* binoms, int n_max,
                      float* new_opacities, float* new_scales, cudaStream_t st);
int launch_add_noise(int n, const float* raw_opacities, const float* raw_scales, const float* raw_quats, const float* noise,
                     float* means, float lr, cudaStream_t st);
int launch_quats_to_rotmats(int n, const float* quats, float* rotmats, cudaStream_t st);
int launch_ply_rows(int N, int K, const lfs_splats& p, float* rows, int unpack, cudaStream_t st);
int launch_mcmc_classify(int N, const float* opacity_raw, const float* rotation_raw, float min_opacity, int64_t* dead_indices,
                         int64_t* alive_indices, float* alive_opacities, int32_t* counts_dev, int32_t* flags, int32_t* offs,
                         int32_t* total_dev, const SortScratch& s, cudaStream_t st);
int launch_mcmc_map_indices(int n, const int64_t* local, const int64_t* map, int64_t* out, cudaStream_t st);
int launch_mcmc_gather_ratios(int N, int n, const int64_t* sampled, const float* opacity_raw, const float* scaling_raw, int n_max,
                              int32_t* counts, int32_t* ratios, float* s_opac, float* s_scales, cudaStream_t st);
int launch_mcmc_apply(int N, int K, int n, const int64_t* sampled, const int64_t* dst_indices, const float* new_opac,
                      const float* new_scales, float min_opacity, const lfs_splats& p, const lfs_splats* m, const lfs_splats* v,
                      cudaStream_t st);

// Flag-based ordering between ranks (see dp_signal_kernel / dp_wait_kernel). peer_flags[i]: rank i's flag array as mapped
// on this GPU (host array of `world` device pointers, entry own_rank is the local array).
int launch_dp_signal(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, cudaStream_t st);
int launch_dp_wait(int world, const int32_t* flags, int slot, int32_t value, uint64_t timeout_ns, int32_t* status, cudaStream_t st);
int launch_dp_barrier(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, uint64_t timeout_ns, int32_t* status,
                      cudaStream_t st);

}  // namespace lfs
