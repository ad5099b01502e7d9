/*
 * lfs_b200 — C ABI of the B200 (sm_100a) Gaussian-splatting training-step library.
 *
 * Drop-in boundary for the gsplat / 3DGUT path of LichtFeld Studio: every entry point replaces
 * one operator (or one fused group of operators) that the reference reaches through
 * gsplat/Ops.h, src/training/kernels/ssim.cu, src/training/fastgs/optimizer and
 * src/training/strategies/mcmc.cpp. The citation above each declaration names the reference
 * interface it replaces (paths relative to the reference project root).
 *
 * Conventions
 *  - All data pointers are DEVICE pointers to contiguous float32 / int32 / int64 arrays in the
 *    reference's layouts unless a parameter is documented as a host value.
 *  - Nothing here allocates: outputs and scratch ("workspace") are supplied by the caller; the
 *    *_workspace_bytes functions give the scratch size. Workspace pointers must be 256-byte aligned.
 *  - Every call is asynchronous on `stream` (a cudaStream_t passed as void*) and returns
 *    LFS_OK or a negative lfs_status. lfs_last_error() returns the message of the last failure on
 *    the calling thread. No call synchronises the device except where stated.
 *  - One camera per rasterize call, like the reference kernels (the camera index only selects the
 *    output plane); batches are loops over cameras.
 */
#ifndef LFS_B200_H
#define LFS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum lfs_status {
    LFS_OK = 0,
    LFS_EINVAL = -1,    /* bad argument (null pointer, unsupported size / mode) */
    LFS_ECAPACITY = -2, /* a caller-provided buffer or workspace is too small */
    LFS_ECUDA = -3,     /* a CUDA runtime call or kernel launch failed */
    LFS_EUNSUPPORTED = -4
} lfs_status;

/* gsplat/Common.h:46-51 */
typedef enum lfs_camera_model { LFS_PINHOLE = 0, LFS_ORTHO = 1, LFS_FISHEYE = 2, LFS_EQUIRECTANGULAR = 3 } lfs_camera_model;

/* gsplat/Cameras.h:27-45 (UnscentedTransformParameters, passed by value in the reference) */
typedef struct lfs_ut_params {
    float alpha;                        /* 0.1 */
    float beta;                         /* 2.0 */
    float kappa;                        /* 0.0 */
    float in_image_margin_factor;       /* 0.1 */
    int require_all_sigma_points_valid; /* 1 */
} lfs_ut_params;

const char* lfs_last_error(void);
/* Library version and the SM architecture the kernels were compiled for ("sm_100a"). */
const char* lfs_build_info(void);

/* Opt-in per-kernel timing (the reference only has wall-clock ScopedTimer logging,
 * include/core/logger.hpp:382-401). While enabled, every kernel launch of this library is bracketed by
 * two CUDA events on its stream. lfs_profile_collect waits for the recorded events and returns up to
 * max_records (name, milliseconds) pairs in launch order; every lfs_profile_enable call clears the list.
 * `on` is a set of bits: 1 = CUDA events, 2 = an NVTX range (nvtx3, same names) around every launch for timeline
 * tools (free unless a profiler is attached; records nothing for lfs_profile_collect). 0 switches both off.
 * Not thread-safe; bit 1 creates CUDA events, so leave it off in production and during graph capture. */
int lfs_profile_enable(int on);
int lfs_profile_collect(int max_records, const char** names, float* ms);

/* ------------------------------------------------------------------------------------------ */
/* Operator level (same inputs / outputs as the reference operators)                           */
/* ------------------------------------------------------------------------------------------ */

/* gsplat/Ops.h:67-95 projection_ut_3dgs_fused -> gsplat/ProjectionUT3DGSFused.cu:17.
 * Shutter: rs_type is the reference's ShutterType (0 top-to-bottom, 1 left-to-right, 2 bottom-to-top, 3 right-to-left,
 * 4 global, gsplat/Cameras.h); viewmats1 [C,4,4] (or NULL = the start pose) is the end-of-frame pose of a rolling
 * shutter (gsplat/Cameras.cuh:33-71, :346-413). camera_model FISHEYE: radial_coeffs [C,4] or NULL. camera_model PINHOLE: radial_coeffs [C,6],
 * tangential_coeffs [C,2], thin_prism_coeffs [C,4], each or NULL; all NULL is the distortion-free pinhole, any
 * present selects the OpenCV pinhole model (gsplat/ProjectionUT3DGSFused.cu:91-113, gsplat/Cameras.cuh:474-755).
 * opacities and compensations may be NULL. Outputs of culled Gaussians other than radii = 0 are
 * left untouched, like the reference. */
int lfs_projection_ut_3dgs_fused(
    int C, int N, const float* means, const float* quats, const float* scales, const float* opacities,
    const float* viewmats0, const float* viewmats1, const float* Ks, int image_width, int image_height,
    float eps2d, float near_plane, float far_plane, float radius_clip,
    int camera_model, lfs_ut_params ut_params, int rs_type, const float* radial_coeffs, const float* tangential_coeffs,
    const float* thin_prism_coeffs, int32_t* radii, float* means2d, float* depths, float* conics, float* compensations, void* stream);

/* gsplat/Ops.h:12-17 spherical_harmonics_fwd -> gsplat/SphericalHarmonicsCUDA.cu:374.
 * n elements, coeffs [n,K,3], masks (uint8, NULL = all), colors [n,3]. */
int lfs_spherical_harmonics_fwd(int n, int K, int degrees_to_use, const float* dirs, const float* coeffs,
                                const uint8_t* masks, float* colors, void* stream);

/* gsplat/Ops.h:18-25 spherical_harmonics_bwd (compute_v_dirs = false) -> SphericalHarmonicsCUDA.cu:445.
 * Writes the FULL v_coeffs [n,K,3] (zeros where masked or above the active degree). */
int lfs_spherical_harmonics_bwd(int n, int K, int degrees_to_use, const float* dirs, const uint8_t* masks,
                                const float* v_colors, float* v_coeffs, void* stream);

/* gsplat/Ops.h:28-38 intersect_tile, first pass (gsplat/Intersect.cpp:55-77): tiles_per_gauss [C,N]
 * and the total number of intersections written to *n_isects_dev (device int64). The caller reads
 * it back to size the outputs of lfs_intersect_tile_emit, exactly like the reference's .item(). */
int lfs_intersect_tile_count(int C, int N, const float* means2d, const int32_t* radii,
                             int tile_size, int tile_width, int tile_height,
                             int32_t* tiles_per_gauss, int64_t* n_isects_dev, void* stream);

size_t lfs_intersect_tile_workspace_bytes(int C, int N, int64_t n_isects);

/* gsplat/Ops.h:28-38 intersect_tile, second pass + sort (gsplat/Intersect.cpp:79-121,
 * gsplat/IntersectTile.cu:290-328). isect_ids [n_isects] int64 and flatten_ids [n_isects] int32 come
 * out in the order a stable ascending radix sort of the (camera | tile | depth-bits) key gives.
 * With sort == 0 they are written in emission order. */
int lfs_intersect_tile_emit(int C, int N, const float* means2d, const int32_t* radii, const float* depths,
                            const int32_t* tiles_per_gauss, int tile_size, int tile_width, int tile_height,
                            int sort, int64_t n_isects, int64_t* isect_ids, int32_t* flatten_ids,
                            void* workspace, size_t workspace_bytes, void* stream);

/* gsplat/Ops.h:39-43 intersect_offset -> gsplat/IntersectTile.cu:206. offsets [C,tile_h,tile_w]. */
int lfs_intersect_offset(int64_t n_isects, const int64_t* isect_ids, int C, int tile_width, int tile_height,
                         int32_t* offsets, void* stream);

size_t lfs_rasterize_workspace_bytes(int N);

/* gsplat/Ops.h:97-125 rasterize_to_pixels_from_world_3dgs_fwd ->
 * gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu:20, one camera. colors [N,channels] with channels 1, 3 or 4
 * (the CDIM instantiations the render modes use, gsplat/Rasterization.cpp:107-110, :373-393).
 * backgrounds [channels] or NULL. masks [tile_h*tile_w] bytes or NULL: a tile labelled 0 is filled with the
 * background (alpha and last_ids 0 there; the reference leaves those two unwritten).
 * renders [H,W,channels], alphas [H,W,1], last_ids [H,W]. */
int lfs_rasterize_to_pixels_from_world_3dgs_fwd(
    int N, int64_t n_isects, int channels, const float* means, const float* quats, const float* scales, const float* colors,
    const float* opacities, const float* backgrounds, const uint8_t* masks, int image_width, int image_height, int tile_size,
    const float* viewmat0, const float* viewmat1, const float* K, int camera_model, int rs_type, const float* radial_coeffs,
    const float* tangential_coeffs, const float* thin_prism_coeffs,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    float* renders, float* alphas, int32_t* last_ids, void* workspace, size_t workspace_bytes, void* stream);

/* gsplat/Ops.h:127-160 rasterize_to_pixels_from_world_3dgs_bwd ->
 * gsplat/RasterizeToPixelsFromWorld3DGSBwd.cu:17. Writes (not accumulates) v_means [N,3],
 * v_quats [N,4], v_scales [N,3], v_colors [N,channels], v_opacities [N]. Masked tiles contribute nothing. */
int lfs_rasterize_to_pixels_from_world_3dgs_bwd(
    int N, int64_t n_isects, int channels, const float* means, const float* quats, const float* scales, const float* colors,
    const float* opacities, const float* backgrounds, const uint8_t* masks, int image_width, int image_height, int tile_size,
    const float* viewmat0, const float* viewmat1, const float* K, int camera_model, int rs_type, const float* radial_coeffs,
    const float* tangential_coeffs, const float* thin_prism_coeffs,
    const int32_t* tile_offsets, const int32_t* flatten_ids,
    const float* render_alphas, const int32_t* last_ids, const float* v_render_colors, const float* v_render_alphas,
    float* v_means, float* v_quats, float* v_scales, float* v_colors, float* v_opacities,
    void* workspace, size_t workspace_bytes, void* stream);

/* src/training/kernels/ssim.cu:431 fusedssim (train = true). Images [CH,H,W]. */
int lfs_fusedssim(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2,
                  float* ssim_map, float* dm_dmu1, float* dm_dsigma1_sq, float* dm_dsigma12, void* stream);

/* src/training/kernels/ssim.cu:476 fusedssim_backward. */
int lfs_fusedssim_backward(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2,
                           const float* dL_dmap, const float* dm_dmu1, const float* dm_dsigma1_sq,
                           const float* dm_dsigma12, float* dL_dimg1, void* stream);

/* src/training/fastgs/optimizer/include/adam_api.h (adam_step_wrapper) ->
 * fastgs/optimizer/include/adam_kernels.cuh:13. */
int lfs_adam_step(float* param, float* exp_avg, float* exp_avg_sq, const float* grad, int64_t n_elements,
                  float lr, float beta1, float beta2, float eps, float bias_correction1_rcp,
                  float bias_correction2_sqrt_rcp, void* stream);

/* Data-parallel exchange of the higher-order SH gradient in rank-1 form, fused with the optimizer (no counterpart in
 * the reference). Every rank ran lfs_render_backward for ONE camera with LFS_BACKWARD_SH_FACTORS; this rank owns the
 * elements [lo, lo + n) of the shN tensor [N_capacity, K-1, 3]. For the rows that intersect them the kernel loads every
 * rank's 24-byte factor row through NVLink peer pointers, sums the outer products (SH basis of the direction) x (colour
 * gradient) in the order given, applies Adam with this rank's moments (exp_avg / exp_avg_sq are indexed from `lo`) and
 * stores the new coefficients into every rank's shN tensor. peer_factors[i] / peer_shN[i] (host arrays of `world` device
 * pointers) belong to rank (own_rank + i) % world, entry 0 is this rank's own. It moves 24 N / world bytes per peer in
 * instead of 12 (K-1) N / world; ordering against the other ranks as for lfs_dp_reduce_adam_broadcast. Rows >= N
 * (capacity padding) take a zero gradient. multicast_shN as multicast_params of lfs_dp_reduce_adam_broadcast (the address of
 * the same tensor inside the multicast mapping), or NULL. */
int lfs_dp_sh_rank1_adam_broadcast(int world, const float* const* peer_factors, float* const* peer_shN, float* multicast_shN,
                                   int N, int sh_coeffs, int sh_degree, int64_t lo, int64_t n, float* exp_avg, float* exp_avg_sq, float lr,
                                   double beta1, double beta2, double eps, int64_t step_count, float grad_scale,
                                   int ctas_per_sm, void* stream);

/* Ordering between the ranks of a data-parallel step by flags in peer-mapped memory, with bounded waits (no counterpart
 * in the reference). Every rank owns a flag array of LFS_DP_FLAG_WORDS int32 (zero-initialised, mapped on every peer):
 * word [slot * LFS_DP_MAX_WORLD + r] is written by rank r only. lfs_dp_signal, enqueued after a producer kernel, stores
 * `value` (a step number that only grows) into this rank's word of slot `slot` in EVERY rank's array (peer_flags: host
 * array of `world` device pointers indexed by rank). lfs_dp_wait, enqueued before a consumer kernel, spins on the local
 * array until all `world` words of the slot have reached `value`, for at most timeout_ns nanoseconds; when the time runs
 * out it sets status[0] = 1, status[1] = bit mask of the ranks that were missing, status[2] = slot, status[3] = value
 * (device int32[4], zeroed by the caller) and returns, so a rank that stopped stepping shows up as a status word, never
 * as a hung stream. The kernels that follow then run on incomplete data: the host must read the status before it trusts
 * the step. */
#define LFS_DP_MAX_WORLD 16
#define LFS_DP_FLAG_SLOTS 8
#define LFS_DP_FLAG_WORDS (LFS_DP_MAX_WORLD * LFS_DP_FLAG_SLOTS)
int lfs_dp_signal(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, void* stream);
int lfs_dp_wait(int world, const int32_t* flags, int slot, int32_t value, uint64_t timeout_ns, int32_t* status_dev, void* stream);
/* lfs_dp_signal followed by lfs_dp_wait on this rank's own array (peer_flags[own_rank]) in ONE launch: the rendezvous of the
 * data-parallel step ("no rank goes on before every rank got here"). status[2..3] keep the slot and value of the first wait
 * that ran out. */
int lfs_dp_barrier(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, uint64_t timeout_ns,
                   int32_t* status_dev, void* stream);

/* gsplat/Ops.h:50-57 relocation -> gsplat/RelocationCUDA.cu:12. */
int lfs_relocation(int n, const float* opacities, const float* scales, const int32_t* ratios, const float* binoms,
                   int n_max, float* new_opacities, float* new_scales, void* stream);

/* gsplat/Ops.h:59-65 add_noise -> gsplat/RelocationCUDA.cu:113 (in place on means). */
int lfs_add_noise(int n, const float* raw_opacities, const float* raw_scales, const float* raw_quats,
                  const float* noise, float* means, float current_lr, void* stream);

/* gsplat/Ops.h:45-48 quats_to_rotmats -> gsplat/QuatToRotmatCUDA.cu:13. rotmats [n,3,3] row-major. */
int lfs_quats_to_rotmats(int n, const float* quats, float* rotmats, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Fused training path (replaces the torch glue between the operators as well)                 */
/* ------------------------------------------------------------------------------------------ */

/* The six parameter tensors of SplatData (src/core/splat_data.hpp:104-109), or tensors of the same
 * shapes (gradients, Adam moments). */
typedef struct lfs_splats {
    float* means;        /* [N,3]      */
    float* sh0;          /* [N,1,3]    */
    float* shN;          /* [N,K-1,3]  */
    float* scaling_raw;  /* [N,3] log  */
    float* rotation_raw; /* [N,4] wxyz */
    float* opacity_raw;  /* [N,1] logit */
} lfs_splats;

/* RenderMode of src/training/rasterization/rasterizer.hpp: colour, accumulated depth, expected depth
 * (= accumulated / max(alpha, 1e-10), src/training/rasterization/rasterizer.cpp:186-198), and both. */
typedef enum lfs_render_mode {
    LFS_RENDER_RGB = 0, LFS_RENDER_D = 1, LFS_RENDER_ED = 2, LFS_RENDER_RGB_D = 3, LFS_RENDER_RGB_ED = 4
} lfs_render_mode;

/* Constants of src/training/rasterization/rasterizer.cpp:90-94 plus the per-call inputs. */
typedef struct lfs_render_config {
    int N;                 /* Gaussians */
    int sh_coeffs;         /* K = total SH bases stored per Gaussian (1 + shN rows) */
    int sh_degree;         /* active degree */
    int image_width, image_height;
    int tile_size;         /* 16 */
    int camera_model;      /* lfs_camera_model */
    float eps2d, near_plane, far_plane, radius_clip;
    lfs_ut_params ut;
    int64_t isect_capacity; /* room for intersections in the workspace; overflow -> LFS_ECAPACITY flag */
    /* FusedRasterizationSettings (src/training/rasterization/rasterizer_autograd.hpp); zero = the trainer's defaults */
    int render_mode;        /* lfs_render_mode: channels of `render` are 3, 1, 1, 4, 4 */
    int calc_compensations; /* `antialiased`: blended opacity = opacity * compensation (gsplat/Rasterization.cpp:396-399) */
    float scaling_modifier; /* scales are multiplied by it; 0 means 1.0 */
    const uint8_t* tile_masks; /* device [tile_h*tile_w] bytes or NULL (gsplat/Ops.h `masks`) */
    /* Lens distortion of this camera, device pointers or NULL. LFS_FISHEYE: radial_coeffs [4].
     * LFS_PINHOLE: radial_coeffs [6] (k1..k6), tangential_coeffs [2], thin_prism_coeffs [4]; any of the three
     * being non-NULL selects the OpenCV pinhole model (gsplat/ProjectionUT3DGSFused.cu:91-113). */
    const float* radial_coeffs;
    const float* tangential_coeffs;
    const float* thin_prism_coeffs;
    /* Rolling shutter: 0 = global (default), 1 = top-to-bottom, 2 = left-to-right, 3 = bottom-to-top, 4 = right-to-left
     * (the reference's ShutterType + 1, so that a zeroed config is a global shutter). viewmat_end: device [4,4]
     * end-of-frame world-to-camera matrix or NULL (= the start pose). */
    int shutter;
    const float* viewmat_end;
} lfs_render_config;

size_t lfs_render_workspace_bytes(const lfs_render_config* cfg);

/* Forward of FusedRasterizationWithSHFunction (src/training/rasterization/rasterizer_autograd.cpp:11)
 * = gsplat::rasterize_from_world_with_sh_fwd (gsplat/Rasterization.cpp:279) including the SplatData
 * activations (src/core/splat_data.cpp:267-286), for one camera. viewmat [4,4], K [3,3],
 * background [channels] or NULL are device pointers; the distortion coefficients are in cfg.
 * Outputs: render [H,W,channels] (unclamped; channels by render_mode: colour first, depth last; in the two
 * expected-depth modes the depth channel is already divided by max(alpha, 1e-10)), alpha [H,W,1].
 * The depth channel's background is background[channels-1]; the reference passes its 3-float colour
 * background to the 1-channel kernel (so depth gets the red value) and reads past it with 4 channels:
 * callers that want the same pictures pass {r} resp. {r,g,b,0}. Everything the backward needs stays in the
 * workspace. status_dev (device int32[4]): [0] overflow flag, [1] n_isects, [2] n_visible. */
int lfs_render_forward(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat,
                       const float* K, const float* background,
                       float* render, float* alpha, int32_t* status_dev,
                       void* workspace, size_t workspace_bytes, void* stream);

/* The same forward in two calls, for callers that overlap the optimizer with the next step: the tile lists depend
 * on means / scales / rotations / opacities only, so lfs_render_forward_lists can start as soon as those four
 * tensors are updated, while the SH tensors (three quarters of the parameter bytes) are still being updated on
 * another stream; lfs_render_forward_shade (SH colours into the per-Gaussian records, then blending) follows once
 * that stream is done. lists + shade on one workspace = lfs_render_forward, bit for bit. */
int lfs_render_forward_lists(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat,
                             const float* K, void* workspace, size_t workspace_bytes, void* stream);
/* lfs_render_forward_lists that also records `projected_event` (a cudaEvent_t of the caller, or NULL) on the stream right
 * after the per-Gaussian projection kernel and before the sorting kernels: work on another stream that should not run
 * next to the projection (the NVLink-bound colour exchange of a data-parallel step, whose queued peer stores slow it
 * threefold) waits for this event and runs next to the sorts instead. */
int lfs_render_forward_lists_event(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat,
                                   const float* K, void* projected_event, void* workspace, size_t workspace_bytes,
                                   void* stream);
int lfs_render_forward_shade(const lfs_render_config* cfg, const lfs_splats* params, const float* background,
                             float* render, float* alpha, int32_t* status_dev,
                             void* workspace, size_t workspace_bytes, void* stream);

/* Backward of the same node (rasterizer_autograd.cpp:105 -> gsplat/Rasterization.cpp:470) followed by
 * the activation backward, for the camera whose forward state is in the workspace. alpha is the
 * forward's alpha output, v_render [H,W,channels] and v_alpha [H,W,1] (may be NULL = zeros) the output
 * gradients (w.r.t. the divided depth in the expected-depth modes). As in the reference, the depth channel
 * only acts on the parameters through alpha (its per-Gaussian gradient is dropped, gsplat/Rasterization.cpp:575-590)
 * and the opacity gradient is not multiplied by the compensation.
 * Call it once per lfs_render_forward: it consumes the per-Gaussian accumulators that the forward zeroed.
 * grads: the six raw-parameter gradients. `accumulate` is a set of lfs_backward_flags: with LFS_BACKWARD_ACCUMULATE the
 * gradients are added to, else they are overwritten (all N rows, zeros for Gaussians that were not visible).
 * grads->shN may be NULL: that gradient is then not written (see lfs_adam_step_splats_rank1_sh). With
 * LFS_BACKWARD_SH_FACTORS the start of grads->shN receives, instead of the rows, their two factors as [N,6] floats
 * (clamped colour gradient, unit view direction) for lfs_dp_sh_rank1_adam_broadcast; not together with ACCUMULATE. */
typedef enum lfs_backward_flags {
    LFS_BACKWARD_ACCUMULATE = 1,
    LFS_BACKWARD_SH_FACTORS = 2
} lfs_backward_flags;
int lfs_render_backward(const lfs_render_config* cfg, const lfs_splats* params, const float* background,
                        const float* alpha, const float* v_render, const float* v_alpha, const lfs_splats* grads,
                        int accumulate, void* workspace, size_t workspace_bytes, void* stream);

/* Device pointers of the forward state kept in the workspace, valid after lfs_render_forward on the
 * same stream: the per-Gaussian outputs gsplat::rasterize_from_world_with_sh_fwd returns
 * (gsplat/Ops.h:171-185) — radii [N,2], means2d [N,2], depths [N] (meaningful where radii > 0) — plus
 * tiles_per_gauss [N], tile_offsets [tile_h*tile_w + 1] (last entry = n_isects), flatten_ids
 * [n_isects], last_ids [H,W] and the packed 16-float rasterizer records [N,16] whose floats 12..14
 * are the clamped colours. */
typedef struct lfs_render_view {
    const int32_t* radii;
    const float* means2d;
    const float* depths;
    const int32_t* tiles_per_gauss;
    const int32_t* tile_offsets;
    const int32_t* flatten_ids;
    const int32_t* last_ids;
    const float* records;
} lfs_render_view;
int lfs_render_workspace_view(const lfs_render_config* cfg, void* workspace, size_t workspace_bytes,
                              lfs_render_view* view);

size_t lfs_photometric_loss_workspace_bytes(int H, int W);

/* Trainer::compute_photometric_loss (src/training/trainer.cpp:107-134) on the clamped, permuted render
 * (rasterizer.cpp:205) with fused_ssim "valid" padding (include/kernels/fused_ssim.cuh:59-67, :117-122),
 * and its gradient w.r.t. the unclamped HWC render. target is CHW [3,H,W]. loss_dev (device float[4]):
 * [0] loss, [1] L1 mean, [2] SSIM mean. grad_scale multiplies the gradient (1/batch for batches). */
int lfs_photometric_loss(int H, int W, float lambda_dssim, float grad_scale, const float* render_hwc,
                         const float* target_chw, float* v_render_hwc, float* loss_dev,
                         void* workspace, size_t workspace_bytes, void* stream);

/* v_bg_color of the autograd node (src/training/rasterization/rasterizer_autograd.cpp:206-209):
 * v_background[c] = sum over pixels of v_render[p, c] * (1 - alpha[p]), for callers whose background colour is a trained
 * parameter. v_render [H,W,channels] (channels 1..4), alpha [H,W,1] the forward's alpha, v_background device float[channels].
 * workspace: 32 bytes of 8-byte aligned device scratch. */
int lfs_background_gradient(int H, int W, int channels, const float* v_render, const float* alpha, float* v_background,
                            void* workspace, size_t workspace_bytes, void* stream);

/* FusedAdam::step over all six groups in one launch (src/training/optimizers/fused_adam.cpp:22-95,
 * group order and learning rates of src/training/strategies/mcmc.cpp:487-492). lr[6] host values in
 * group order means, sh0, shN, scaling, rotation, opacity; step_count >= 1 is the optimizer step
 * index (beta1 / beta2 are doubles because the reference computes the bias corrections from the double
 * option values before narrowing, fused_adam.cpp:78-79); skip_shN != 0 reproduces the `iteration <= 1000`
 * skip. first_row/n_rows select a contiguous Gaussian range (optimizer-state sharding).
 * grad_scale multiplies the gradient on read. */
int lfs_adam_step_splats(int N, int sh_coeffs, const lfs_splats* params, const lfs_splats* exp_avg,
                         const lfs_splats* exp_avg_sq, const lfs_splats* grads, const float* lr,
                         double beta1, double beta2, double eps, int64_t step_count, int skip_shN,
                         int64_t first_row, int64_t n_rows, float grad_scale, void* stream);

/* lfs_render_backward and FusedAdam::step (src/training/optimizers/fused_adam.cpp:22-95) in one call, for steps of ONE
 * camera; no gradient tensor exists. The per-Gaussian gradient stage applies Adam to the five small groups (means, sh0,
 * scales, rotations, opacities) in place as it produces their gradients and leaves the two rank-1 factors of the shN
 * gradient (clamped colour gradient, unit view direction) in the workspace; a second kernel rebuilds the shN gradient rows
 * from them and streams the shN coefficients and moments through once. Arguments as in lfs_render_backward and
 * lfs_adam_step_splats (lr[6] host values in group order, bias corrections from the double betas, skip_shN for
 * `iteration <= 1000`, grad_scale multiplies the gradient). The result equals lfs_render_backward(accumulate = 0)
 * followed by lfs_adam_step_splats over all rows up to the rounding of the backward's atomic sums; Gaussians that were
 * not visible take a zero gradient (their moments decay). Not for batches of several cameras, data-parallel steps, or
 * callers that add regularisers or inspect gradients between the two reference calls. */
int lfs_render_backward_adam(const lfs_render_config* cfg, const lfs_splats* params, const float* background,
                             const float* alpha, const float* v_render, const float* v_alpha, const lfs_splats* exp_avg,
                             const lfs_splats* exp_avg_sq, const float* lr /* host[6] */, double beta1, double beta2,
                             double eps, int64_t step_count, int skip_shN, float grad_scale, void* workspace,
                             size_t workspace_bytes, void* stream);

/* FusedAdam::step (src/training/optimizers/fused_adam.cpp:22-95) after a ONE-camera lfs_render_backward whose
 * grads->shN was NULL: the higher-order SH gradient is never materialised. For one camera, row g of that gradient is the
 * outer product of the SH basis of Gaussian g's view direction with its clamped colour gradient, and grads->sh0 holds
 * Y_0 times that colour gradient (gsplat/SphericalHarmonicsCUDA.cu:113-371), so the kernel that updates shN rebuilds the
 * rows on the fly from grads->sh0, params->means and the camera of the forward state in `workspace` (the one the backward
 * used). The other five groups are updated from their gradient tensors as in lfs_adam_step_splats. Saves the write and the
 * read of 12 (K-1) N gradient bytes per step; the result equals backward-with-shN + lfs_adam_step_splats up to one
 * rounding of the colour gradient. Not for gradients accumulated over several cameras (their sum is no outer product), and
 * only while params->means are the means the forward used: a caller that moves them between backward and this call (the
 * MCMC noise, a relocation) must let the backward write grads->shN and use lfs_adam_step_splats. */
int lfs_adam_step_splats_rank1_sh(const lfs_render_config* cfg, const lfs_splats* params, const lfs_splats* exp_avg,
                                  const lfs_splats* exp_avg_sq, const lfs_splats* grads, const float* lr /* host[6] */,
                                  double beta1, double beta2, double eps, int64_t step_count, int skip_shN,
                                  float grad_scale, void* workspace, size_t workspace_bytes, void* stream);

/* src/training/kernels/regularization.cu:20 / :171 (compute_exp_l1_regularization_with_grad_cuda,
 * compute_sigmoid_l1_regularization_with_grad_cuda), both in one launch and without the host read:
 *   L_scale = scale_weight * mean(exp(scaling_raw)),     grad_scaling += scale_weight / (3N) * exp(scaling_raw)
 *   L_opac  = opacity_weight * mean(sigmoid(opacity_raw)), grad_opacity += opacity_weight / N * s (1 - s)
 * A weight of 0 skips that term (its gradient pointer may then be NULL). reg_loss_dev (device float[2])
 * receives (L_scale, L_opac). */
int lfs_regularization(int N, const float* scaling_raw, const float* opacity_raw, float scale_weight, float opacity_weight,
                       float* grad_scaling, float* grad_opacity, float* reg_loss_dev, void* stream);

/* Fused Adam over up to 16 arbitrary contiguous segments in one launch (each with its own learning rate).
 * lfs_adam_step_splats is the special case "six groups, one row range". Used for optimizer-state sharding
 * by flat element range: a shard of the group-major parameter buffer is at most six segments. */
typedef struct lfs_adam_segment {
    float* param;
    float* exp_avg;
    float* exp_avg_sq;
    const float* grad;
    int64_t n;
    float lr;
} lfs_adam_segment;
/* ctas_per_sm: launch footprint, 0 = default (16 CTAs of 256 threads per SM); a small value leaves thread slots for
 * kernels that run next to this one on other streams. */
int lfs_adam_step_segments(int n_segments, const lfs_adam_segment* segments /* host */, double beta1, double beta2,
                           double eps, int64_t step_count, float grad_scale, int ctas_per_sm, void* stream);

/* Data-parallel exchange fused with the optimizer (no counterpart in the reference, which is single-GPU):
 * ONE kernel that, for this rank's shard of the flat parameter buffer, loads the gradient of every rank
 * through NVLink peer pointers, sums them in rank order (deterministic), applies Adam with the local
 * moments, and stores the new parameters into every rank's parameter buffer. It replaces
 * ncclReduceScatter -> Adam -> ncclAllGather. peer_grads[i] / peer_params[i] (host arrays of `world` device
 * pointers) are the peer-mapped FULL flat buffers of rank (own_rank + i) % world, i.e. entry 0 is this
 * rank's own buffer (the parameters are read from it; the sum runs in that rotated order); offset / n / lr / moments per segment describe
 * the shard (offsets in elements from the start of the flat buffers; moments are shard-local buffers).
 * ctas_per_sm: launch footprint, 0 = default (16 CTAs of 256 threads per SM); the kernel is NVLink-bound and keeps its
 * speed with 2 - 4, which leaves thread slots for kernels running next to it on other streams.
 * The caller must order it against the other ranks: every rank's backward finished before, nobody reads
 * parameters or rewrites gradients until all ranks finished after (lfs_dp_barrier, or a stream-ordered collective).
 * multicast_params: NULL, or the address of the parameter buffer in an NVSwitch multicast mapping bound to the same memory
 * on all `world` GPUs (cuMulticast* / torch symmetric memory's multicast_ptr): the new parameters then leave this GPU as ONE
 * multimem.st per 16 bytes, which the switch replicates, instead of `world` peer stores (the broadcast's share of the NVLink
 * egress drops by the number of peers). Gradients are always read with plain peer loads. */
typedef struct lfs_dp_segment {
    int64_t offset;      /* first element of the segment in the flat buffers */
    int64_t n;           /* elements */
    float* exp_avg;      /* local moments of this segment */
    float* exp_avg_sq;
    float lr;
} lfs_dp_segment;
int lfs_dp_reduce_adam_broadcast(int world, const float* const* peer_grads, float* const* peer_params, float* multicast_params,
                                 int n_segments, const lfs_dp_segment* segments /* host */, double beta1, double beta2, double eps,
                                 int64_t step_count, float grad_scale, int ctas_per_sm, void* stream);

/* ------------------------------------------------------------------------------------------ */
/* MCMC densification index work (src/training/strategies/mcmc.cpp:112-347)                    */
/* ------------------------------------------------------------------------------------------ */

/* mcmc.cpp:121-131: dead = sigmoid(opacity_raw) <= min_opacity | |rotation_raw|^2 < 1e-8.
 * Writes ascending dead_indices / alive_indices (int64, capacity N each), alive_opacities (the
 * probabilities handed to multinomial, float32 1/(1+exp(-x)) like torch::sigmoid) and counts_dev (device int32[2]: n_dead, n_alive). */
size_t lfs_mcmc_workspace_bytes(int N);
int lfs_mcmc_classify(int N, const float* opacity_raw, const float* rotation_raw, float min_opacity,
                      int64_t* dead_indices, int64_t* alive_indices, float* alive_opacities,
                      int32_t* counts_dev, void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference. Same result as lfs_mcmc_classify, but for callers that must not
 * allocate device memory where they run the densification step (a trainer refining under the viewer's
 * render lock, where an allocation can stall the frame in flight; a plugin host with a budget fixed at
 * start-up). The scratch is a fixed array inside the library (about 2.1 MB per GPU, held until the
 * process exits), so N is limited to LFS_NOALLOC_MAX_GAUSSIANS; larger N returns LFS_ECAPACITY. The first
 * call on a device also looks up the array's device address; make that call before any stream capture.
 * The array used is the one of the device that is CURRENT when the call is made, so the device that owns `stream` must be
 * current (a stream of another device would be paired with the wrong copy of the array).
 * All calls on a device share the scratch: calls that overlap on the GPU race and corrupt each other. */
#define LFS_NOALLOC_MAX_GAUSSIANS 262144
int lfs_mcmc_classify_noalloc(int N, const float* opacity_raw, const float* rotation_raw, float min_opacity,
                              int64_t* dead_indices, int64_t* alive_indices, float* alive_opacities,
                              int32_t* counts_dev, void* stream);

/* mcmc.cpp:137: sampled = alive_indices.index_select(0, sampled_local): out[i] = index_map[local_indices[i]]. */
int lfs_mcmc_map_indices(int n, const int64_t* local_indices, const int64_t* index_map, int64_t* out, void* stream);

/* mcmc.cpp:139-150 / :221-228: ratios[i] = clamp(1 + #occurrences of sampled[i] in sampled, 1, n_max),
 * plus the gathered activated opacity / scale of each sampled Gaussian. counts is an int32[N] scratch. */
int lfs_mcmc_gather_ratios(int N, int n_sampled, const int64_t* sampled, const float* opacity_raw,
                           const float* scaling_raw, int n_max, int32_t* counts, int32_t* ratios,
                           float* sampled_opacities, float* sampled_scales, void* stream);

/* mcmc.cpp:160-187 (relocate, dst = dead indices) and :238-344 (add, dst = N..N+n-1 when dst_indices is
 * NULL): clamp new opacity to [min_opacity, 1-1e-7], write logit / log back at the sampled rows, copy
 * all six parameter rows sampled -> dst, zero the Adam moments at `sampled` (relocate) or at the
 * appended rows (add). The parameter / moment buffers must have capacity for N + n rows when adding. */
int lfs_mcmc_apply(int N, int sh_coeffs, int n_sampled, const int64_t* sampled, const int64_t* dst_indices,
                   const float* new_opacities, const float* new_scales, float min_opacity,
                   const lfs_splats* params, const lfs_splats* exp_avg, const lfs_splats* exp_avg_sq,
                   void* stream);

/* ---- EWA rasterizer: the default (non --gut) training path ------------------------------- */

/* FastGSSettings (src/training/fastgs/rasterization/include/rasterization_api.h:14-25) plus sizes. */
typedef struct lfs_ewa_config {
    int N;                 /* Gaussians */
    int sh_coeffs;         /* K = SH bases stored per Gaussian (1 + shN rows) */
    int active_sh_bases;   /* (active degree + 1)^2: 1, 4, 9 or 16 */
    int image_width, image_height;
    float focal_x, focal_y, center_x, center_y;
    float near_plane, far_plane;    /* fast_rasterizer.cpp:33-34 uses 0.01 and 1e10 */
    int64_t instance_capacity;      /* room for (Gaussian, tile) instances in the workspace */
} lfs_ewa_config;

size_t lfs_ewa_workspace_bytes(const lfs_ewa_config* cfg);

/* fast_rasterize (src/training/rasterization/fast_rasterizer.cpp:13-71) = FastGSRasterize::forward
 * (fast_rasterizer_autograd.cpp:8-86 -> fastgs/rasterization/src/forward.cu:17-199) plus the background blend, on the
 * raw SplatData tensors. w2c [4,4] row-major, cam_position [3], background [3] or NULL are device pointers.
 * Outputs: image [3,H,W] = blend + (1 - alpha) background, alpha [1,H,W]. status_dev (device int32[4], may be
 * NULL): [0] capacity overflow flag (nothing is drawn), [1] n_instances, [2] n_visible. Unlike the reference there
 * is no host synchronisation: counts stay on the device and the lists live in the caller's workspace.
 * exp / log of the per-Gaussian stage are evaluated in double and rounded once (the reference calls expf / logf),
 * and equal depths are ordered by Gaussian index (the reference's order there depends on atomic slot order). */
int lfs_ewa_forward(const lfs_ewa_config* cfg, const lfs_splats* params, const float* w2c, const float* cam_position,
                    const float* background, float* image, float* alpha, int32_t* status_dev,
                    void* workspace, size_t workspace_bytes, void* stream);

/* FastGSRasterize::backward (fast_rasterizer_autograd.cpp:88-165 -> fastgs/rasterization/src/backward.cu:12-116)
 * for the camera whose forward state is in the workspace; call once per lfs_ewa_forward. grad_image [3,H,W] is
 * the gradient of the FINAL image (the background term is folded in, pass the same background), grad_alpha
 * [1,H,W] or NULL. grads: the six raw-parameter gradients, overwritten (all N rows) or added to.
 * densification_info (device [2,N] or NULL): row 0 += 1 and row 1 += |d mean2d * (W/2, H/2)| for every Gaussian
 * that reached a tile (kernels_backward.cuh:228-232). grad_w2c (device [4,4] row-major or NULL): the camera-pose
 * gradient of kernels_backward.cuh:160-173, rows 0..2 = sum over those Gaussians of (gradient of the camera-space mean) x
 * (mean, 1), row 3 zero; overwritten, or added to with `accumulate`. Like the reference's it carries the mean term only
 * (not the pose's part in the covariance or the SH view direction). */
int lfs_ewa_backward(const lfs_ewa_config* cfg, const lfs_splats* params, const float* w2c, const float* cam_position,
                     const float* background, const float* alpha, const float* grad_image, const float* grad_alpha,
                     const lfs_splats* grads, int accumulate, float* densification_info, float* grad_w2c,
                     void* workspace, size_t workspace_bytes, void* stream);

/* FusedAdam::step after a ONE-camera lfs_ewa_backward whose grads->shN was NULL (that gradient is then not written):
 * the shN rows are updated from gradient rows rebuilt on the fly as (SH basis of the view direction from cam_position) x
 * (grads->sh0 / Y_0), the other five groups from their gradient tensors. Same contract as lfs_adam_step_splats_rank1_sh;
 * cam_position [3] is the device pointer given to the backward. */
int lfs_ewa_adam_step_rank1_sh(const lfs_ewa_config* cfg, const lfs_splats* params, const float* cam_position,
                               const lfs_splats* exp_avg, const lfs_splats* exp_avg_sq, const lfs_splats* grads,
                               const float* lr /* host[6] */, double beta1, double beta2, double eps, int64_t step_count,
                               int skip_shN, float grad_scale, void* stream);

/* Device pointers into a workspace that holds a finished lfs_ewa_forward (tests, inspection). */
typedef struct lfs_ewa_view {
    const int32_t* n_touched;     /* [N] tiles reached per Gaussian (0 = culled) */
    const uint16_t* bounds;       /* [N,4] x_min, x_max, y_min, y_max in tiles */
    const float* records;         /* [N,12] mean2d 2, conic 3 (xx, xy at [2..3], yy at [4]), opacity, rgb (clamped), mask, threshold */
    const uint32_t* instance_ids; /* [n_instances] */
    const int32_t* tile_offsets;  /* [tiles + 1] */
    const int32_t* n_contrib;     /* [H,W] */
} lfs_ewa_view;
int lfs_ewa_workspace_view(const lfs_ewa_config* cfg, void* workspace, size_t workspace_bytes, lfs_ewa_view* out);

/* ---- PLY export / import rows -------------------------------------------------------------- */

/* The vertex rows of SplatData::save_ply (src/core/splat_data.cpp:402-418 attribute names, :483-503
 * SplatData::to_point_cloud contents), built on the device in one pass instead of transpose / flatten /
 * normalize / .cpu() per tensor: rows [N, 14 + 3*sh_coeffs] float32 =
 *   x y z | nx ny nz = 0 | f_dc_0..2 | f_rest_0.. (channel-major: all R, then G, then B) |
 *   opacity (raw logit) | scale_0..2 (raw log) | rot_0..3 (normalised, q / max(|q|, 1e-12)).
 * Copy the buffer to the host and write it after the header: it is the binary_little_endian body. */
int lfs_ply_pack_rows(int N, int sh_coeffs, const lfs_splats* params, float* rows, void* stream);

/* Inverse (the layout src/loader/formats/ply.cpp reads): scatters rows into the six tensors; the normals
 * are ignored and the quaternion is stored as found. */
int lfs_ply_unpack_rows(int N, int sh_coeffs, const float* rows, const lfs_splats* params, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LFS_B200_H */
