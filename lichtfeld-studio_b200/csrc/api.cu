// extern "C" entry points declared in include/lfs_b200.h: argument checks, workspace carving and
// the launch sequences. No allocation happens here; every call is asynchronous on the caller's stream.
#include <cmath>
#include <cstddef>
#include <cstring>

#include "elementwise.cuh"
#include "loss.cuh"
#include "projection.cuh"
#include "raster.cuh"
#include "ewa.cuh"
#include "sort.cuh"

#define LFS_STR2(x) #x
#define LFS_STR(x) LFS_STR2(x)

namespace lfs {
const char* last_error();
void profile_enable(bool events, bool nvtx);
int profile_collect(int max_records, const char** names, float* ms);

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline cudaStream_t S_(void* s) { return reinterpret_cast<cudaStream_t>(s); }

struct Carver {
    char* base;
    size_t off = 0;
    explicit Carver(void* b) : base(reinterpret_cast<char*>(b)) {}
    template <typename T>
    T* take(size_t count) {
        off = (off + 255) & ~(size_t)255;
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += count * sizeof(T);
        return p;
    }
    size_t total() const { return (off + 255) & ~(size_t)255; }
};

uint32_t bit_width_u32(uint32_t v) {
    uint32_t b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

// which buffer of a ping-pong pair holds the result after sorting key_bits bits
int sorted_sel(int key_bits) { return ((key_bits + 7) / 8) & 1; }

SortScratch carve_scratch(Carver& c) {
    SortScratch s;
    s.hist = c.take<uint32_t>((size_t)kRadixBlocks * 256);
    s.block_sums = c.take<uint32_t>(kScanBlocks + 320);  // also holds the 256 digit totals of a radix pass
    return s;
}

// ---- fused render workspace -------------------------------------------------------------------
struct RenderWs {
    CamDev* cam;
    int32_t* counters;  // [0] overflow, [1] n_isects, [2] n_visible
    int32_t *radii, *tiles, *offs, *tile_offsets, *last_ids, *tile_order;
    float *means2d, *depths, *accum, *extra_sum;
    float4* records;
    uint4* bounds;
    uint32_t *gkeys[2], *gvals[2], *tkeys[2], *tvals[2];
    SortScratch scratch;
    size_t bytes;
};

RenderWs carve_render(const lfs_render_config& cfg, void* base) {
    Carver c(base);
    RenderWs w;
    const size_t N = (size_t)cfg.N;
    const size_t cap = (size_t)cfg.isect_capacity;
    const int tw = (cfg.image_width + cfg.tile_size - 1) / cfg.tile_size;
    const int th = (cfg.image_height + cfg.tile_size - 1) / cfg.tile_size;
    w.cam = c.take<CamDev>(1);
    w.counters = c.take<int32_t>(16);
    w.radii = c.take<int32_t>(N * 2);
    w.means2d = c.take<float>(N * 2);
    w.depths = c.take<float>(N);
    w.tiles = c.take<int32_t>(N);
    w.offs = c.take<int32_t>(N);
    for (int k = 0; k < 2; ++k) { w.gkeys[k] = c.take<uint32_t>(N); w.gvals[k] = c.take<uint32_t>(N); }
    w.records = c.take<float4>(N * 4);
    w.bounds = c.take<uint4>(N);
    w.accum = c.take<float>(N * 16);
    for (int k = 0; k < 2; ++k) { w.tkeys[k] = c.take<uint32_t>(cap); w.tvals[k] = c.take<uint32_t>(cap); }
    w.tile_offsets = c.take<int32_t>((size_t)tw * th + 1);
    w.tile_order = c.take<int32_t>((size_t)tw * th);
    w.last_ids = c.take<int32_t>((size_t)cfg.image_width * cfg.image_height);
    w.extra_sum = c.take<float>((size_t)cfg.image_width * cfg.image_height);  // blended depth before the division (ED modes)
    w.scratch = carve_scratch(c);
    w.bytes = c.total();
    return w;
}

// ---- EWA workspace ----------------------------------------------------------------------------
struct EwaWs {
    int32_t* counters;  // [0] overflow, [1] n_instances, [2] n_visible
    int32_t *n_touched, *offs, *tile_offsets, *n_contrib, *tile_order;
    ushort4* bounds;
    float4* records;
    float* accum;
    uint32_t *gkeys[2], *gvals[2], *tkeys[2], *tvals[2];
    SortScratch scratch;
    size_t bytes;
};

EwaWs carve_ewa(const lfs_ewa_config& cfg, void* base) {
    Carver c(base);
    EwaWs w;
    const size_t N = (size_t)cfg.N, cap = (size_t)cfg.instance_capacity;
    const int tw = (cfg.image_width + 15) / 16, th = (cfg.image_height + 15) / 16;
    w.counters = c.take<int32_t>(16);
    w.n_touched = c.take<int32_t>(N);
    w.offs = c.take<int32_t>(N);
    w.bounds = c.take<ushort4>(N);
    w.records = c.take<float4>(N * 3);
    w.accum = c.take<float>(N * 12);
    for (int k = 0; k < 2; ++k) { w.gkeys[k] = c.take<uint32_t>(N); w.gvals[k] = c.take<uint32_t>(N); }
    for (int k = 0; k < 2; ++k) { w.tkeys[k] = c.take<uint32_t>(cap); w.tvals[k] = c.take<uint32_t>(cap); }
    w.tile_offsets = c.take<int32_t>((size_t)tw * th + 1);
    w.n_contrib = c.take<int32_t>((size_t)cfg.image_width * cfg.image_height);
    w.tile_order = c.take<int32_t>((size_t)tw * th);
    w.scratch = carve_scratch(c);
    w.bytes = c.total();
    return w;
}

int check_ewa_cfg(const lfs_ewa_config* cfg) {
    LFS_REQUIRE(cfg != nullptr, "null config");
    LFS_REQUIRE(cfg->N >= 0 && cfg->image_width > 0 && cfg->image_height > 0, "bad sizes");
    LFS_REQUIRE(cfg->image_width <= 65535 * 16 && cfg->image_height <= 65535 * 16, "image too large");
    LFS_REQUIRE(cfg->sh_coeffs >= 1 && cfg->active_sh_bases >= 1 && cfg->active_sh_bases <= 16 && cfg->active_sh_bases <= cfg->sh_coeffs,
                "active_sh_bases must be in [1, min(16, sh_coeffs)]");
    LFS_REQUIRE(cfg->focal_x != 0.f && cfg->focal_y != 0.f, "zero focal length");
    LFS_REQUIRE(cfg->instance_capacity >= 0 && cfg->instance_capacity < ((int64_t)1 << 31), "instance_capacity out of range");
    return LFS_OK;
}

EwaCamera ewa_camera(const lfs_ewa_config& cfg, const float* w2c, const float* campos) {
    EwaCamera cam;
    cam.w2c = w2c; cam.campos = campos;
    cam.fx = cfg.focal_x; cam.fy = cfg.focal_y; cam.cx = cfg.center_x; cam.cy = cfg.center_y;
    cam.near_plane = cfg.near_plane; cam.far_plane = cfg.far_plane;
    cam.W = cfg.image_width; cam.H = cfg.image_height;
    cam.tw = (cfg.image_width + 15) / 16; cam.th = (cfg.image_height + 15) / 16;
    cam.active_sh_bases = cfg.active_sh_bases; cam.total_rest = cfg.sh_coeffs - 1;
    return cam;
}

int check_cfg(const lfs_render_config* cfg) {
    LFS_REQUIRE(cfg != nullptr, "null config");
    LFS_REQUIRE(cfg->N >= 0 && cfg->image_width > 0 && cfg->image_height > 0, "bad sizes");
    LFS_REQUIRE(cfg->tile_size == 16, "tile_size must be 16");
    LFS_REQUIRE(cfg->sh_degree >= 0 && cfg->sh_degree <= 4, "sh_degree must be in [0,4]");
    LFS_REQUIRE(cfg->sh_coeffs >= (cfg->sh_degree + 1) * (cfg->sh_degree + 1), "not enough SH coefficients for the degree");
    LFS_REQUIRE(cfg->camera_model == LFS_PINHOLE || cfg->camera_model == LFS_FISHEYE || cfg->camera_model == LFS_EQUIRECTANGULAR,
                "camera model must be PINHOLE, FISHEYE or EQUIRECTANGULAR");
    LFS_REQUIRE(cfg->camera_model != LFS_EQUIRECTANGULAR || (cfg->shutter == 0 && !cfg->viewmat_end && !cfg->radial_coeffs),
                "the equirectangular model has a global shutter and no distortion coefficients");
    LFS_REQUIRE(cfg->isect_capacity >= 0 && cfg->isect_capacity < ((int64_t)1 << 31), "isect_capacity out of range");
    LFS_REQUIRE(cfg->render_mode >= LFS_RENDER_RGB && cfg->render_mode <= LFS_RENDER_RGB_ED, "render_mode must be in [0,4]");
    LFS_REQUIRE(cfg->scaling_modifier >= 0.f, "scaling_modifier must be positive (0 = 1.0)");
    LFS_REQUIRE(cfg->shutter >= 0 && cfg->shutter <= 4, "shutter must be 0 (global) or 1..4 (rolling)");
    LFS_REQUIRE(cfg->camera_model == LFS_PINHOLE || (!cfg->tangential_coeffs && !cfg->thin_prism_coeffs),
                "tangential / thin-prism coefficients belong to the pinhole model");
    return LFS_OK;
}

int mode_channels(int render_mode) {
    return render_mode == LFS_RENDER_RGB ? 3 : (render_mode == LFS_RENDER_D || render_mode == LFS_RENDER_ED) ? 1 : 4;
}
int mode_normalize(int render_mode) { return render_mode == LFS_RENDER_ED || render_mode == LFS_RENDER_RGB_ED; }
int cfg_model(const lfs_render_config& cfg) {
    return effective_model(cfg.camera_model, cfg.radial_coeffs, cfg.tangential_coeffs, cfg.thin_prism_coeffs);
}
// cfg.shutter: 0 = global, 1..4 = the reference's ShutterType 0..3
int cfg_rs_type(const lfs_render_config& cfg) { return cfg.shutter == 0 ? LFS_SHUTTER_GLOBAL : cfg.shutter - 1; }
int cfg_rolling(const lfs_render_config& cfg) { return (cfg.shutter != 0 || cfg.viewmat_end != nullptr) ? 1 : 0; }
float cfg_modifier(const lfs_render_config& cfg) { return cfg.scaling_modifier > 0.f ? cfg.scaling_modifier : 1.0f; }

}  // namespace
}  // namespace lfs

using namespace lfs;

extern "C" {

const char* lfs_last_error(void) { return lfs::last_error(); }
int lfs_profile_enable(int on) {
    if (on < 0 || on > 3) { lfs::set_error("lfs_profile_enable: flags must be 0..3"); return LFS_EINVAL; }
    lfs::profile_enable((on & 1) != 0, (on & 2) != 0);
    return LFS_OK;
}
int lfs_profile_collect(int max_records, const char** names, float* ms) { return lfs::profile_collect(max_records, names, ms); }
const char* lfs_build_info(void) { return "lfs_b200 0.1 (sm_100a, CUDA " LFS_STR(CUDART_VERSION) ")"; }

// ---------------------------------------------------------------------------------------------
int lfs_projection_ut_3dgs_fused(int C, int N, const float* means, const float* quats, const float* scales,
                                 const float* opacities, const float* viewmats0, const float* viewmats1, const float* Ks, int W,
                                 int H, float eps2d, float near_plane, float far_plane, float radius_clip, int camera_model,
                                 lfs_ut_params ut, int rs_type, const float* radial_coeffs, const float* tangential_coeffs, const float* thin_prism_coeffs,
                                 int32_t* radii, float* means2d, float* depths, float* conics,
                                 float* compensations, void* stream) {
    LFS_REQUIRE(C >= 0 && N >= 0 && W > 0 && H > 0, "bad sizes");
    LFS_REQUIRE(camera_model == LFS_PINHOLE || camera_model == LFS_FISHEYE || camera_model == LFS_EQUIRECTANGULAR,
                "camera model must be PINHOLE, FISHEYE or EQUIRECTANGULAR");
    LFS_REQUIRE(camera_model != LFS_EQUIRECTANGULAR || (rs_type == LFS_SHUTTER_GLOBAL && !viewmats1 && !radial_coeffs),
                "the equirectangular model has a global shutter and no distortion coefficients");
    if ((int64_t)C * N == 0) return LFS_OK;
    LFS_REQUIRE(means && quats && scales && viewmats0 && Ks && radii && means2d && depths && conics, "null pointer");
    LFS_REQUIRE(aligned16(quats), "quats must be 16-byte aligned");
    LFS_REQUIRE(camera_model == LFS_PINHOLE || (!tangential_coeffs && !thin_prism_coeffs),
                "tangential / thin-prism coefficients belong to the pinhole model");
    LFS_REQUIRE(rs_type >= 0 && rs_type <= LFS_SHUTTER_GLOBAL, "rs_type must be a ShutterType (0..4)");
    return launch_projection_ut(C, N, means, quats, scales, opacities, viewmats0, viewmats1, rs_type, Ks, radial_coeffs, tangential_coeffs,
                                thin_prism_coeffs, W, H,
                                make_proj_params(eps2d, near_plane, far_plane, radius_clip, ut), camera_model, radii,
                                means2d, depths, conics, compensations, S(stream));
}

int lfs_spherical_harmonics_fwd(int n, int K, int degree, const float* dirs, const float* coeffs, const uint8_t* masks,
                                float* colors, void* stream) {
    LFS_REQUIRE(n >= 0 && degree >= 0 && degree <= 4 && K >= (degree + 1) * (degree + 1), "bad sizes");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(dirs && coeffs && colors, "null pointer");
    return launch_sh_fwd(n, K, degree, dirs, coeffs, masks, colors, S(stream));
}

int lfs_spherical_harmonics_bwd(int n, int K, int degree, const float* dirs, const uint8_t* masks, const float* v_colors,
                                float* v_coeffs, void* stream) {
    LFS_REQUIRE(n >= 0 && degree >= 0 && degree <= 4 && K >= (degree + 1) * (degree + 1), "bad sizes");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(dirs && v_colors && v_coeffs, "null pointer");
    return launch_sh_bwd(n, K, degree, dirs, masks, v_colors, v_coeffs, S(stream));
}

int lfs_intersect_tile_count(int C, int N, const float* means2d, const int32_t* radii, int tile_size, int tw, int th,
                             int32_t* tiles_per_gauss, int64_t* n_isects_dev, void* stream) {
    LFS_REQUIRE(C >= 0 && N >= 0 && tile_size > 0 && tw >= 0 && th >= 0, "bad sizes");
    LFS_REQUIRE(n_isects_dev != nullptr, "null pointer");
    const int64_t total = (int64_t)C * N;
    if (total > 0) LFS_REQUIRE(means2d && radii && tiles_per_gauss, "null pointer");
    int rc = launch_tile_count(total, means2d, radii, tile_size, tw, th, tiles_per_gauss, S(stream));
    if (rc != LFS_OK) return rc;
    return launch_sum_i32(total, tiles_per_gauss, n_isects_dev, S(stream));
}

static size_t isect_ws(int C, int N, int64_t n_isects, void* base, uint32_t** gk, uint32_t** gv, int32_t** offs,
                       int32_t** n_dev, uint32_t** tk, uint32_t** tv, SortScratch* s) {
    Carver c(base);
    const size_t total = (size_t)C * N, cap = (size_t)(n_isects > 0 ? n_isects : 1);
    for (int k = 0; k < 2; ++k) { gk[k] = c.take<uint32_t>(total); gv[k] = c.take<uint32_t>(total); }
    *offs = c.take<int32_t>(total);
    *n_dev = c.take<int32_t>(16);
    for (int k = 0; k < 2; ++k) { tk[k] = c.take<uint32_t>(cap); tv[k] = c.take<uint32_t>(cap); }
    *s = carve_scratch(c);
    return c.total();
}

size_t lfs_intersect_tile_workspace_bytes(int C, int N, int64_t n_isects) {
    uint32_t *gk[2], *gv[2], *tk[2], *tv[2];
    int32_t *offs, *n_dev;
    SortScratch s;
    return isect_ws(C, N, n_isects, nullptr, gk, gv, &offs, &n_dev, tk, tv, &s);
}

int lfs_intersect_tile_emit(int C, int N, const float* means2d, const int32_t* radii, const float* depths,
                            const int32_t* tiles_per_gauss, int tile_size, int tw, int th, int sort, int64_t n_isects,
                            int64_t* isect_ids, int32_t* flatten_ids, void* workspace, size_t workspace_bytes, void* stream) {
    LFS_REQUIRE(C >= 0 && N >= 0 && tile_size > 0 && n_isects >= 0 && n_isects < ((int64_t)1 << 31), "bad sizes");
    if (n_isects == 0 || (int64_t)C * N == 0) return LFS_OK;
    LFS_REQUIRE(means2d && radii && depths && tiles_per_gauss && isect_ids && flatten_ids && workspace, "null pointer");
    TileListArgs a{};
    const size_t need = isect_ws(C, N, n_isects, workspace, a.gkeys, a.gvals, &a.offs, &a.n_isects_dev, a.tkeys, a.tvals, &a.scratch);
    if (workspace_bytes < need) { set_error("lfs_intersect_tile_emit: workspace too small (%zu < %zu)", workspace_bytes, need); return LFS_ECAPACITY; }
    a.C = C; a.N = N; a.tw = tw; a.th = th; a.tile_size = tile_size; a.sort = sort ? 1 : 0; a.keys_ready = 0;
    a.means2d = means2d; a.radii = radii; a.depths = depths; a.tiles = tiles_per_gauss;
    a.capacity = n_isects; a.overflow = nullptr; a.tile_offsets = nullptr;
    int sel = 0;
    a.sel_out = &sel;
    int rc = build_tile_lists(a, S(stream));
    if (rc != LFS_OK) return rc;
    return launch_compose_isect_ids(n_isects, a.tkeys[sel], a.tvals[sel], depths, isect_ids, flatten_ids, S(stream));
}

int lfs_intersect_offset(int64_t n_isects, const int64_t* isect_ids, int C, int tw, int th, int32_t* offsets, void* stream) {
    LFS_REQUIRE(n_isects >= 0 && C >= 0 && tw >= 0 && th >= 0, "bad sizes");
    if ((int64_t)C * tw * th == 0) return LFS_OK;
    LFS_REQUIRE(offsets && (n_isects == 0 || isect_ids), "null pointer");
    return launch_isect_offset(n_isects, isect_ids, C, tw, th, offsets, S(stream));
}

// ---------------------------------------------------------------------------------------------
size_t lfs_rasterize_workspace_bytes(int N) {
    Carver c(nullptr);
    c.take<CamDev>(1);
    c.take<float4>((size_t)N * 4);
    c.take<uint4>((size_t)N);
    c.take<float>((size_t)N * 16);
    c.take<float>((size_t)N);
    return c.total();
}

static int raster_common(int N, int64_t n_isects, int channels, int W, int H, int tile_size, int camera_model,
                         const void* workspace, size_t workspace_bytes) {
    LFS_REQUIRE(N >= 0 && n_isects >= 0 && n_isects < ((int64_t)1 << 31) && W > 0 && H > 0, "bad sizes");
    LFS_REQUIRE(channels == 1 || channels == 3 || channels == 4, "colours must have 1, 3 or 4 channels");
    LFS_REQUIRE(tile_size == 16, "tile_size must be 16");
    LFS_REQUIRE(camera_model == LFS_PINHOLE || camera_model == LFS_FISHEYE || camera_model == LFS_EQUIRECTANGULAR,
                "camera model must be PINHOLE, FISHEYE or EQUIRECTANGULAR");
    LFS_REQUIRE(workspace != nullptr, "null workspace");
    if (workspace_bytes < lfs_rasterize_workspace_bytes(N)) { set_error("rasterize: workspace too small"); return LFS_ECAPACITY; }
    return LFS_OK;
}

int lfs_rasterize_to_pixels_from_world_3dgs_fwd(int N, int64_t n_isects, int channels, const float* means, const float* quats,
                                                const float* scales, const float* colors, const float* opacities,
                                                const float* backgrounds, const uint8_t* masks, int W, int H, int tile_size,
                                                const float* viewmat0, const float* viewmat1,
                                                const float* K, int camera_model, int rs_type, const float* radial_coeffs,
                                                const float* tangential_coeffs, const float* thin_prism_coeffs,
                                                const int32_t* tile_offsets, const int32_t* flatten_ids, float* renders,
                                                float* alphas, int32_t* last_ids, void* workspace, size_t workspace_bytes,
                                                void* stream) {
    int rc = raster_common(N, n_isects, channels, W, H, tile_size, camera_model, workspace, workspace_bytes);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(viewmat0 && K && tile_offsets && renders && alphas && last_ids, "null pointer");
    LFS_REQUIRE(aligned16(quats), "quats must be 16-byte aligned");
    Carver c(workspace);
    CamDev* cam = c.take<CamDev>(1);
    float4* records = c.take<float4>((size_t)N * 4);
    uint4* bounds = c.take<uint4>((size_t)N);
    LFS_REQUIRE(camera_model == LFS_PINHOLE || (!tangential_coeffs && !thin_prism_coeffs),
                "tangential / thin-prism coefficients belong to the pinhole model");
    LFS_REQUIRE(rs_type >= 0 && rs_type <= LFS_SHUTTER_GLOBAL, "rs_type must be a ShutterType (0..4)");
    rc = launch_camera_setup(1, viewmat0, viewmat1, rs_type, K, radial_coeffs, tangential_coeffs, thin_prism_coeffs, W, H, camera_model,
                             cam, S(stream));
    const int eff_model = effective_model(camera_model, radial_coeffs, tangential_coeffs, thin_prism_coeffs);
    const int rolling = (rs_type != LFS_SHUTTER_GLOBAL || viewmat1 != nullptr) ? 1 : 0;
    LFS_REQUIRE(camera_model != LFS_EQUIRECTANGULAR || (!rolling && !radial_coeffs),
                "the equirectangular model has a global shutter and no distortion coefficients");
    if (rc != LFS_OK) return rc;
    rc = launch_pack_records(N, means, quats, scales, colors, channels, opacities, cam, records, bounds, nullptr, nullptr, S(stream));
    if (rc != LFS_OK) return rc;
    RasterArgs a{cam, records, bounds, reinterpret_cast<const uint32_t*>(flatten_ids), tile_offsets, nullptr, n_isects, backgrounds,
                 nullptr, W, H, (W + 15) / 16, (H + 15) / 16, eff_model, channels, 0, masks, nullptr, rolling};
    return launch_raster_fwd(a, renders, alphas, last_ids, nullptr, S(stream));
}

int lfs_rasterize_to_pixels_from_world_3dgs_bwd(int N, int64_t n_isects, int channels, const float* means, const float* quats,
                                                const float* scales, const float* colors, const float* opacities,
                                                const float* backgrounds, const uint8_t* masks, int W, int H, int tile_size,
                                                const float* viewmat0, const float* viewmat1,
                                                const float* K, int camera_model, int rs_type, const float* radial_coeffs,
                                                const float* tangential_coeffs, const float* thin_prism_coeffs,
                                                const int32_t* tile_offsets, const int32_t* flatten_ids,
                                                const float* render_alphas, const int32_t* last_ids,
                                                const float* v_render_colors, const float* v_render_alphas, float* v_means,
                                                float* v_quats, float* v_scales, float* v_colors, float* v_opacities,
                                                void* workspace, size_t workspace_bytes, void* stream) {
    int rc = raster_common(N, n_isects, channels, W, H, tile_size, camera_model, workspace, workspace_bytes);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(viewmat0 && K && tile_offsets && render_alphas && last_ids && v_render_colors, "null pointer");
    LFS_REQUIRE(v_means && v_quats && v_scales && v_colors && v_opacities, "null output pointer");
    LFS_REQUIRE(aligned16(quats), "quats must be 16-byte aligned");
    Carver c(workspace);
    CamDev* cam = c.take<CamDev>(1);
    float4* records = c.take<float4>((size_t)N * 4);
    uint4* bounds = c.take<uint4>((size_t)N);
    float* accum = c.take<float>((size_t)N * 16);
    float* accum_extra = channels != 3 ? c.take<float>((size_t)N) : nullptr;
    LFS_REQUIRE(camera_model == LFS_PINHOLE || (!tangential_coeffs && !thin_prism_coeffs),
                "tangential / thin-prism coefficients belong to the pinhole model");
    LFS_REQUIRE(rs_type >= 0 && rs_type <= LFS_SHUTTER_GLOBAL, "rs_type must be a ShutterType (0..4)");
    rc = launch_camera_setup(1, viewmat0, viewmat1, rs_type, K, radial_coeffs, tangential_coeffs, thin_prism_coeffs, W, H, camera_model,
                             cam, S(stream));
    const int eff_model = effective_model(camera_model, radial_coeffs, tangential_coeffs, thin_prism_coeffs);
    const int rolling = (rs_type != LFS_SHUTTER_GLOBAL || viewmat1 != nullptr) ? 1 : 0;
    LFS_REQUIRE(camera_model != LFS_EQUIRECTANGULAR || (!rolling && !radial_coeffs),
                "the equirectangular model has a global shutter and no distortion coefficients");
    if (rc != LFS_OK) return rc;
    rc = launch_pack_records(N, means, quats, scales, colors, channels, opacities, cam, records, bounds,
                             reinterpret_cast<float4*>(accum), accum_extra, S(stream));
    if (rc != LFS_OK) return rc;
    RasterArgs a{cam, records, bounds, reinterpret_cast<const uint32_t*>(flatten_ids), tile_offsets, nullptr, n_isects, backgrounds,
                 nullptr, W, H, (W + 15) / 16, (H + 15) / 16, eff_model, channels, 0, masks, nullptr, rolling};
    rc = launch_raster_bwd(a, render_alphas, last_ids, nullptr, v_render_colors, v_render_alphas, accum, accum_extra, S(stream));
    if (rc != LFS_OK) return rc;
    return launch_grad_epilogue_op(N, cam, accum, means, quats, scales, channels, accum_extra, v_means, v_quats, v_scales,
                                   v_colors, v_opacities, S(stream));
}

// ---------------------------------------------------------------------------------------------
int lfs_fusedssim(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2, float* ssim_map,
                  float* dm_dmu1, float* dm_dsigma1_sq, float* dm_dsigma12, void* stream) {
    LFS_REQUIRE(CH >= 0 && H >= 0 && W >= 0, "bad sizes");
    if ((int64_t)CH * H * W == 0) return LFS_OK;
    LFS_REQUIRE(img1 && img2 && ssim_map, "null pointer");
    LFS_REQUIRE((dm_dmu1 == nullptr) == (dm_dsigma1_sq == nullptr) && (dm_dmu1 == nullptr) == (dm_dsigma12 == nullptr),
                "derivative maps must be all given or all null");
    return launch_fusedssim(CH, H, W, C1, C2, img1, img2, ssim_map, dm_dmu1, dm_dsigma1_sq, dm_dsigma12, S(stream));
}

int lfs_fusedssim_backward(int CH, int H, int W, float C1, float C2, const float* img1, const float* img2,
                           const float* dL_dmap, const float* dm_dmu1, const float* dm_dsigma1_sq, const float* dm_dsigma12,
                           float* dL_dimg1, void* stream) {
    (void)C1; (void)C2;
    LFS_REQUIRE(CH >= 0 && H >= 0 && W >= 0, "bad sizes");
    if ((int64_t)CH * H * W == 0) return LFS_OK;
    LFS_REQUIRE(img1 && img2 && dL_dmap && dm_dmu1 && dm_dsigma1_sq && dm_dsigma12 && dL_dimg1, "null pointer");
    return launch_fusedssim_backward(CH, H, W, img1, img2, dL_dmap, dm_dmu1, dm_dsigma1_sq, dm_dsigma12, dL_dimg1, S(stream));
}

size_t lfs_photometric_loss_workspace_bytes(int H, int W) { return photometric_workspace_bytes(H, W); }

int lfs_background_gradient(int H, int W, int channels, const float* v_render, const float* alpha, float* v_background,
                            void* workspace, size_t workspace_bytes, void* stream) {
    LFS_REQUIRE(H >= 0 && W >= 0 && channels >= 1 && channels <= 4, "bad size");
    LFS_REQUIRE(v_background && workspace, "null pointer");
    if ((int64_t)H * W > 0) LFS_REQUIRE(v_render && alpha, "null pointer");
    if (workspace_bytes < 32) { set_error("lfs_background_gradient: workspace too small (32 bytes)"); return LFS_ECAPACITY; }
    LFS_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 7) == 0, "workspace must be 8-byte aligned");
    return launch_background_gradient(H, W, channels, v_render, alpha, v_background, workspace, reinterpret_cast<cudaStream_t>(stream));
}

int lfs_photometric_loss(int H, int W, float lambda_dssim, float grad_scale, const float* render_hwc, const float* target_chw,
                         float* v_render_hwc, float* loss_dev, void* workspace, size_t workspace_bytes, void* stream) {
    LFS_REQUIRE(H > 0 && W > 0, "bad sizes");
    LFS_REQUIRE(render_hwc && target_chw && loss_dev && workspace, "null pointer");
    if (workspace_bytes < photometric_workspace_bytes(H, W)) { set_error("lfs_photometric_loss: workspace too small"); return LFS_ECAPACITY; }
    return launch_photometric_loss(H, W, lambda_dssim, grad_scale, render_hwc, target_chw, v_render_hwc, loss_dev, workspace, S(stream));
}

// ---------------------------------------------------------------------------------------------

int lfs_adam_step(float* param, float* exp_avg, float* exp_avg_sq, const float* grad, int64_t n, float lr, float beta1,
                  float beta2, float eps, float bc1_rcp, float bc2_sqrt_rcp, void* stream) {
    LFS_REQUIRE(n >= 0, "bad size");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(param && exp_avg && exp_avg_sq && grad, "null pointer");
    AdamGroups G{};
    G.n_groups = 1;
    G.g[0] = AdamGroup{param, exp_avg, exp_avg_sq, grad, n, lr * bc1_rcp,
                       aligned16(param) && aligned16(exp_avg) && aligned16(exp_avg_sq) && aligned16(grad)};
    G.prefix4[0] = 0;
    G.prefix4[1] = (n + 3) / 4;
    G.beta1 = beta1; G.beta2 = beta2; G.eps = eps; G.bc2_sqrt_rcp = bc2_sqrt_rcp; G.grad_scale = 1.0f;
    return launch_adam_groups(G, S(stream));
}

int lfs_adam_step_splats(int N, int K, const lfs_splats* params, const lfs_splats* exp_avg, const lfs_splats* exp_avg_sq,
                         const lfs_splats* grads, const float* lr, double beta1, double beta2, double eps, int64_t step_count,
                         int skip_shN, int64_t first_row, int64_t n_rows, float grad_scale, void* stream) {
    LFS_REQUIRE(params && exp_avg && exp_avg_sq && grads && lr, "null pointer");
    LFS_REQUIRE(N >= 0 && K >= 1 && step_count >= 1, "bad sizes");
    LFS_REQUIRE(first_row >= 0 && n_rows >= 0 && first_row + n_rows <= N, "row range outside [0, N)");
    if (n_rows == 0) return LFS_OK;
    const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
    const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
    float* P[6] = {params->means, params->sh0, params->shN, params->scaling_raw, params->rotation_raw, params->opacity_raw};
    float* M[6] = {exp_avg->means, exp_avg->sh0, exp_avg->shN, exp_avg->scaling_raw, exp_avg->rotation_raw, exp_avg->opacity_raw};
    float* V[6] = {exp_avg_sq->means, exp_avg_sq->sh0, exp_avg_sq->shN, exp_avg_sq->scaling_raw, exp_avg_sq->rotation_raw, exp_avg_sq->opacity_raw};
    float* Gd[6] = {grads->means, grads->sh0, grads->shN, grads->scaling_raw, grads->rotation_raw, grads->opacity_raw};
    const int width[6] = {3, 3, (K - 1) * 3, 3, 4, 1};
    AdamGroups G{};
    int ng = 0;
    G.prefix4[0] = 0;
    for (int k = 0; k < 6; ++k) {
        if (width[k] == 0) continue;
        if (k == 2 && skip_shN) continue;
        LFS_REQUIRE(P[k] && M[k] && V[k] && Gd[k], "null tensor in a parameter group");
        const int64_t off = first_row * width[k], n = n_rows * width[k];
        AdamGroup g{P[k] + off, M[k] + off, V[k] + off, Gd[k] + off, n, (float)((double)lr[k]) * (float)bc1, 0};
        g.aligned = aligned16(g.p) && aligned16(g.m) && aligned16(g.v) && aligned16(g.g);
        G.g[ng] = g;
        G.prefix4[ng + 1] = G.prefix4[ng] + (n + 3) / 4;
        ++ng;
    }
    G.n_groups = ng;
    G.beta1 = (float)beta1; G.beta2 = (float)beta2; G.eps = (float)eps; G.bc2_sqrt_rcp = (float)bc2; G.grad_scale = grad_scale;
    return launch_adam_groups(G, S(stream));
}

int lfs_regularization(int N, const float* scaling_raw, const float* opacity_raw, float scale_weight, float opacity_weight,
                       float* grad_scaling, float* grad_opacity, float* reg_loss_dev, void* stream) {
    LFS_REQUIRE(N >= 0 && reg_loss_dev != nullptr, "bad arguments");
    if (N > 0 && scale_weight != 0.f) LFS_REQUIRE(scaling_raw && grad_scaling, "null pointer");
    if (N > 0 && opacity_weight != 0.f) LFS_REQUIRE(opacity_raw && grad_opacity, "null pointer");
    return launch_regularization(N, scaling_raw, opacity_raw, scale_weight, opacity_weight, grad_scaling, grad_opacity,
                                 reg_loss_dev, S(stream));
}

int lfs_adam_step_segments(int n_segments, const lfs_adam_segment* segs, double beta1, double beta2, double eps,
                           int64_t step_count, float grad_scale, int ctas_per_sm, void* stream) {
    LFS_REQUIRE(ctas_per_sm >= 0 && ctas_per_sm <= 16, "ctas_per_sm must be in [0, 16]");
    LFS_REQUIRE(n_segments >= 0 && n_segments <= kMaxAdamSegments, "at most 16 segments");
    LFS_REQUIRE(step_count >= 1, "step_count must be >= 1");
    if (n_segments == 0) return LFS_OK;
    LFS_REQUIRE(segs != nullptr, "null pointer");
    const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
    const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
    AdamSegments S{};
    S.prefix4[0] = 0;
    int ng = 0;
    for (int k = 0; k < n_segments; ++k) {
        LFS_REQUIRE(segs[k].n >= 0, "negative segment size");
        if (segs[k].n == 0) continue;
        LFS_REQUIRE(segs[k].param && segs[k].exp_avg && segs[k].exp_avg_sq && segs[k].grad, "null tensor in a segment");
        AdamGroup g{segs[k].param, segs[k].exp_avg, segs[k].exp_avg_sq, segs[k].grad, segs[k].n, segs[k].lr * (float)bc1, 0};
        g.aligned = aligned16(g.p) && aligned16(g.m) && aligned16(g.v) && aligned16(g.g);
        S.g[ng] = g;
        S.prefix4[ng + 1] = S.prefix4[ng] + (g.n + 3) / 4;
        ++ng;
    }
    S.n = ng;
    S.beta1 = (float)beta1; S.beta2 = (float)beta2; S.eps = (float)eps; S.bc2_sqrt_rcp = (float)bc2; S.grad_scale = grad_scale;
    return launch_adam_segments(S, ctas_per_sm, S_(stream));
}

int lfs_dp_reduce_adam_broadcast(int world, const float* const* peer_grads, float* const* peer_params, float* multicast_params,
                                 int n_segments, const lfs_dp_segment* segs, double beta1, double beta2, double eps, int64_t step_count,
                                 float grad_scale, int ctas_per_sm, void* stream) {
    LFS_REQUIRE(world >= 1 && world <= kMaxPeers, "world must be in [1, 8]");
    LFS_REQUIRE(n_segments >= 0 && n_segments <= 6, "at most 6 segments");
    LFS_REQUIRE(step_count >= 1, "step_count must be >= 1");
    LFS_REQUIRE(peer_grads && peer_params, "null pointer");
    if (n_segments == 0) return LFS_OK;
    LFS_REQUIRE(segs != nullptr, "null pointer");
    const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
    const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
    DpArgs A{};
    A.world = world;
    for (int r = 0; r < world; ++r) {
        LFS_REQUIRE(peer_grads[r] && peer_params[r], "null peer pointer");
        LFS_REQUIRE(aligned16(peer_grads[r]) && aligned16(peer_params[r]), "peer buffers must be 16-byte aligned");
        A.grads[r] = peer_grads[r];
        A.params[r] = peer_params[r];
    }
    LFS_REQUIRE(aligned16(multicast_params), "the multicast address must be 16-byte aligned");
    A.mc_params = multicast_params;
    A.prefix4[0] = 0;
    int ns = 0;
    for (int k = 0; k < n_segments; ++k) {
        if (segs[k].n == 0) continue;
        LFS_REQUIRE(segs[k].n > 0 && segs[k].offset >= 0, "bad segment");
        LFS_REQUIRE(segs[k].n % 4 == 0 && segs[k].offset % 4 == 0, "segment offsets and sizes must be multiples of 4 elements");
        LFS_REQUIRE(segs[k].exp_avg && segs[k].exp_avg_sq && aligned16(segs[k].exp_avg) && aligned16(segs[k].exp_avg_sq),
                    "segment moments must be non-null and 16-byte aligned");
        A.seg[ns] = DpSegment{segs[k].offset, segs[k].n, segs[k].exp_avg, segs[k].exp_avg_sq, segs[k].lr * (float)bc1};
        A.prefix4[ns + 1] = A.prefix4[ns] + segs[k].n / 4;
        ++ns;
    }
    A.n_segments = ns;
    A.beta1 = (float)beta1; A.beta2 = (float)beta2; A.eps = (float)eps; A.bc2_sqrt_rcp = (float)bc2; A.grad_scale = grad_scale;
    LFS_REQUIRE(ctas_per_sm >= 0 && ctas_per_sm <= 16, "ctas_per_sm must be in [0, 16]");
    return launch_dp_reduce_adam_broadcast(A, ctas_per_sm, S_(stream));
}

int lfs_dp_sh_rank1_adam_broadcast(int world, const float* const* peer_factors, float* const* peer_shN, float* multicast_shN, int N,
                                   int sh_coeffs,
                                   int sh_degree, int64_t lo, int64_t n, float* exp_avg, float* exp_avg_sq, float lr,
                                   double beta1, double beta2, double eps, int64_t step_count, float grad_scale,
                                   int ctas_per_sm, void* stream) {
    LFS_REQUIRE(world >= 1 && world <= kRank1MaxPeers, "world must be in [1, 8]");
    LFS_REQUIRE(step_count >= 1, "step_count must be >= 1");
    LFS_REQUIRE(N >= 0 && sh_coeffs >= 1 && sh_degree >= 0 && (sh_degree + 1) * (sh_degree + 1) <= sh_coeffs, "bad sizes");
    LFS_REQUIRE(lo >= 0 && n >= 0, "bad element range");
    LFS_REQUIRE(ctas_per_sm >= 0 && ctas_per_sm <= 16, "ctas_per_sm must be in [0, 16]");
    if (n == 0 || sh_coeffs == 1) return LFS_OK;
    LFS_REQUIRE(peer_factors && peer_shN && exp_avg && exp_avg_sq, "null pointer");
    const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
    const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
    DpRank1 A{};
    A.world = world; A.N = N; A.lo = lo; A.n = n; A.m = exp_avg; A.v = exp_avg_sq;
    bool vec = lo % 4 == 0 && aligned16(exp_avg) && aligned16(exp_avg_sq);
    for (int r = 0; r < world; ++r) {
        LFS_REQUIRE(peer_factors[r] && peer_shN[r], "null peer pointer");
        LFS_REQUIRE((reinterpret_cast<uintptr_t>(peer_factors[r]) & 7) == 0, "factor buffers must be 8-byte aligned");
        A.factors[r] = peer_factors[r];
        A.shN[r] = peer_shN[r];
        vec = vec && aligned16(peer_shN[r]);
    }
    A.vec = vec && aligned16(multicast_shN);
    A.mc_shN = multicast_shN;
    A.adam = AdamRank1{nullptr, nullptr, nullptr, lr * (float)bc1, (float)beta1, (float)beta2, (float)eps, (float)bc2, grad_scale, 0};
    return launch_dp_sh_rank1(sh_coeffs, sh_degree, A, ctas_per_sm, S_(stream));
}

int lfs_dp_signal(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, void* stream) {
    LFS_REQUIRE(world >= 1 && world <= LFS_DP_MAX_WORLD && own_rank >= 0 && own_rank < world, "bad world / rank");
    LFS_REQUIRE(slot >= 0 && slot < LFS_DP_FLAG_SLOTS, "bad slot");
    LFS_REQUIRE(peer_flags != nullptr, "null pointer");
    for (int i = 0; i < world; ++i) LFS_REQUIRE(peer_flags[i] != nullptr, "null peer flag array");
    return launch_dp_signal(world, peer_flags, own_rank, slot, value, S(stream));
}

int lfs_dp_wait(int world, const int32_t* flags, int slot, int32_t value, uint64_t timeout_ns, int32_t* status_dev, void* stream) {
    LFS_REQUIRE(world >= 1 && world <= LFS_DP_MAX_WORLD, "bad world");
    LFS_REQUIRE(slot >= 0 && slot < LFS_DP_FLAG_SLOTS, "bad slot");
    LFS_REQUIRE(flags && status_dev, "null pointer");
    LFS_REQUIRE(timeout_ns > 0 && timeout_ns <= 60ull * 1000000000ull, "timeout must be in (0, 60 s]");
    return launch_dp_wait(world, flags, slot, value, timeout_ns, status_dev, S(stream));
}

int lfs_dp_barrier(int world, int32_t* const* peer_flags, int own_rank, int slot, int32_t value, uint64_t timeout_ns,
                   int32_t* status_dev, void* stream) {
    LFS_REQUIRE(world >= 1 && world <= LFS_DP_MAX_WORLD && own_rank >= 0 && own_rank < world, "bad world / rank");
    LFS_REQUIRE(slot >= 0 && slot < LFS_DP_FLAG_SLOTS, "bad slot");
    LFS_REQUIRE(peer_flags != nullptr && status_dev != nullptr, "null pointer");
    for (int i = 0; i < world; ++i) LFS_REQUIRE(peer_flags[i] != nullptr, "null peer flag array");
    LFS_REQUIRE(timeout_ns > 0 && timeout_ns <= 60ull * 1000000000ull, "timeout must be in (0, 60 s]");
    return launch_dp_barrier(world, peer_flags, own_rank, slot, value, timeout_ns, status_dev, S(stream));
}

int lfs_relocation(int n, const float* opacities, const float* scales, const int32_t* ratios, const float* binoms, int n_max,
                   float* new_opacities, float* new_scales, void* stream) {
    LFS_REQUIRE(n >= 0 && n_max > 0, "bad sizes");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(opacities && scales && ratios && binoms && new_opacities && new_scales, "null pointer");
    return launch_relocation(n, opacities, scales, ratios, binoms, n_max, new_opacities, new_scales, S(stream));
}

int lfs_add_noise(int n, const float* raw_opacities, const float* raw_scales, const float* raw_quats, const float* noise,
                  float* means, float current_lr, void* stream) {
    LFS_REQUIRE(n >= 0, "bad size");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(raw_opacities && raw_scales && raw_quats && noise && means, "null pointer");
    LFS_REQUIRE(aligned16(raw_quats), "raw_quats must be 16-byte aligned");
    return launch_add_noise(n, raw_opacities, raw_scales, raw_quats, noise, means, current_lr, S(stream));
}

int lfs_quats_to_rotmats(int n, const float* quats, float* rotmats, void* stream) {
    LFS_REQUIRE(n >= 0, "bad size");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(quats && rotmats, "null pointer");
    LFS_REQUIRE(aligned16(quats), "quats must be 16-byte aligned");
    return launch_quats_to_rotmats(n, quats, rotmats, S(stream));
}

// ---------------------------------------------------------------------------------------------
size_t lfs_ewa_workspace_bytes(const lfs_ewa_config* cfg) {
    if (check_ewa_cfg(cfg) != LFS_OK) return 0;
    return carve_ewa(*cfg, nullptr).bytes;
}

int lfs_ewa_forward(const lfs_ewa_config* cfg, const lfs_splats* params, const float* w2c, const float* cam_position,
                    const float* background, float* image, float* alpha, int32_t* status_dev, void* workspace,
                    size_t workspace_bytes, void* stream) {
    int rc = check_ewa_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && w2c && cam_position && image && alpha && workspace, "null pointer");
    LFS_REQUIRE(aligned16(params->rotation_raw), "rotation_raw must be 16-byte aligned");
    EwaWs w = carve_ewa(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_ewa_forward: workspace too small (%zu < %zu)", workspace_bytes, w.bytes); return LFS_ECAPACITY; }
    cudaStream_t st = S(stream);
    const EwaCamera cam = ewa_camera(*cfg, w2c, cam_position);
    cudaMemsetAsync(w.counters, 0, 16 * sizeof(int32_t), st);
    rc = launch_ewa_preprocess(cfg->N, *params, cam, w.n_touched, w.bounds, w.records, w.gkeys[0], w.gvals[0],
                               reinterpret_cast<float4*>(w.accum), w.counters + 2, st);
    if (rc != LFS_OK) return rc;
    TileListArgs a{};
    a.C = 1; a.N = cfg->N; a.tw = cam.tw; a.th = cam.th; a.tile_size = 16; a.sort = 1; a.keys_ready = 1;
    a.tiles = w.n_touched;
    for (int k = 0; k < 2; ++k) { a.gkeys[k] = w.gkeys[k]; a.gvals[k] = w.gvals[k]; a.tkeys[k] = w.tkeys[k]; a.tvals[k] = w.tvals[k]; }
    a.offs = w.offs; a.n_isects_dev = w.counters + 1; a.capacity = cfg->instance_capacity; a.overflow = w.counters + 0;
    int sel = 0;
    a.sel_out = &sel;
    a.tile_offsets = w.tile_offsets; a.scratch = w.scratch;
    a.ewa_bounds = w.bounds; a.ewa_records = w.records;
    rc = build_tile_lists(a, st);
    if (rc != LFS_OK) return rc;
    rc = launch_tile_order(cam.tw * cam.th, w.tile_offsets, w.tile_order, st);
    if (rc != LFS_OK) return rc;
    EwaBlendArgs b{w.records, w.tvals[sel], w.tile_offsets, w.counters + 0, background, cfg->image_width, cfg->image_height, cam.tw, cam.th,
                   w.tile_order};
    rc = launch_ewa_blend_fwd(b, image, alpha, w.n_contrib, st);
    if (rc != LFS_OK) return rc;
    if (status_dev) cudaMemcpyAsync(status_dev, w.counters, 4 * sizeof(int32_t), cudaMemcpyDeviceToDevice, st);
    return check_launch("lfs_ewa_forward");
}

int lfs_ewa_backward(const lfs_ewa_config* cfg, const lfs_splats* params, const float* w2c, const float* cam_position,
                     const float* background, const float* alpha, const float* grad_image, const float* grad_alpha,
                     const lfs_splats* grads, int accumulate, float* densification_info, float* grad_w2c, void* workspace,
                     size_t workspace_bytes, void* stream) {
    int rc = check_ewa_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && w2c && cam_position && alpha && grad_image && grads && workspace, "null pointer");
    LFS_REQUIRE(aligned16(params->rotation_raw) && aligned16(grads->rotation_raw), "rotation_raw tensors must be 16-byte aligned");
    EwaWs w = carve_ewa(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_ewa_backward: workspace too small"); return LFS_ECAPACITY; }
    cudaStream_t st = S(stream);
    const EwaCamera cam = ewa_camera(*cfg, w2c, cam_position);
    const int sel = sorted_sel((int)(bit_width_u32((uint32_t)cam.tw * cam.th) + 1));  // tile bits + one camera bit
    EwaBlendArgs b{w.records, w.tvals[sel], w.tile_offsets, w.counters + 0, background, cfg->image_width, cfg->image_height, cam.tw, cam.th,
                   w.tile_order};
    rc = launch_ewa_blend_bwd(b, alpha, w.n_contrib, grad_image, grad_alpha, w.accum, st);
    if (rc != LFS_OK) return rc;
    return launch_ewa_epilogue(cfg->N, cfg->sh_coeffs, *params, cam, w.n_touched, w.records, w.accum, *grads, accumulate,
                               densification_info, grad_w2c, st);
}

int lfs_ewa_adam_step_rank1_sh(const lfs_ewa_config* cfg, const lfs_splats* params, const float* cam_position,
                               const lfs_splats* exp_avg, const lfs_splats* exp_avg_sq, const lfs_splats* grads,
                               const float* lr, double beta1, double beta2, double eps, int64_t step_count, int skip_shN,
                               float grad_scale, void* stream) {
    int rc = check_ewa_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && exp_avg && exp_avg_sq && grads && lr && cam_position, "null pointer");
    LFS_REQUIRE(step_count >= 1, "step_count must be >= 1");
    // shN first: its gradient rows depend on the means, which the second launch updates
    if (!skip_shN && cfg->sh_coeffs > 1 && cfg->N > 0) {
        LFS_REQUIRE(params->shN && exp_avg->shN && exp_avg_sq->shN && grads->sh0 && params->means, "null tensor in a parameter group");
        int degree = 0;
        while ((degree + 1) * (degree + 1) < cfg->active_sh_bases) ++degree;
        const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
        const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
        rc = launch_adam_sh_rank1(cfg->N, cfg->sh_coeffs, degree, cam_position, params->means, grads->sh0, params->shN,
                                  exp_avg->shN, exp_avg_sq->shN, (float)((double)lr[2]) * (float)bc1, (float)beta1, (float)beta2,
                                  (float)eps, (float)bc2, grad_scale, S(stream));
        if (rc != LFS_OK) return rc;
    }
    return lfs_adam_step_splats(cfg->N, cfg->sh_coeffs, params, exp_avg, exp_avg_sq, grads, lr, beta1, beta2, eps, step_count,
                                /*skip_shN=*/1, 0, cfg->N, grad_scale, stream);
}

int lfs_ewa_workspace_view(const lfs_ewa_config* cfg, void* workspace, size_t workspace_bytes, lfs_ewa_view* out) {
    int rc = check_ewa_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(workspace && out, "null pointer");
    EwaWs w = carve_ewa(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_ewa_workspace_view: workspace too small"); return LFS_ECAPACITY; }
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    const int sel = sorted_sel((int)(bit_width_u32((uint32_t)tw * th) + 1));
    out->n_touched = w.n_touched;
    out->bounds = reinterpret_cast<const uint16_t*>(w.bounds);
    out->records = reinterpret_cast<const float*>(w.records);
    out->instance_ids = w.tvals[sel];
    out->tile_offsets = w.tile_offsets;
    out->n_contrib = w.n_contrib;
    return LFS_OK;
}

int lfs_ply_pack_rows(int N, int sh_coeffs, const lfs_splats* params, float* rows, void* stream) {
    LFS_REQUIRE(N >= 0 && sh_coeffs >= 1, "bad sizes");
    if (N == 0) return LFS_OK;
    LFS_REQUIRE(params && rows && params->means && params->sh0 && params->scaling_raw && params->rotation_raw && params->opacity_raw,
                "null pointer");
    LFS_REQUIRE(sh_coeffs == 1 || params->shN, "null shN");
    LFS_REQUIRE(aligned16(params->rotation_raw), "rotation_raw must be 16-byte aligned");
    return launch_ply_rows(N, sh_coeffs, *params, rows, 0, S(stream));
}

int lfs_ply_unpack_rows(int N, int sh_coeffs, const float* rows, const lfs_splats* params, void* stream) {
    LFS_REQUIRE(N >= 0 && sh_coeffs >= 1, "bad sizes");
    if (N == 0) return LFS_OK;
    LFS_REQUIRE(params && rows && params->means && params->sh0 && params->scaling_raw && params->rotation_raw && params->opacity_raw,
                "null pointer");
    LFS_REQUIRE(sh_coeffs == 1 || params->shN, "null shN");
    return launch_ply_rows(N, sh_coeffs, *params, const_cast<float*>(rows), 1, S(stream));
}

// ---------------------------------------------------------------------------------------------
size_t lfs_render_workspace_bytes(const lfs_render_config* cfg) {
    if (check_cfg(cfg) != LFS_OK) return 0;
    return carve_render(*cfg, nullptr).bytes;
}

// Shared body of the forward: per-Gaussian stage + tile lists (stage 1), shading + blending (stage 2).
static int render_forward_lists(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat, const float* K,
                                int with_colors, RenderWs& w, int* sel_out, cudaStream_t st, cudaEvent_t projected = nullptr) {
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    int rc = launch_camera_setup(1, viewmat, cfg->viewmat_end, cfg_rs_type(*cfg), K, cfg->radial_coeffs, cfg->tangential_coeffs,
                                 cfg->thin_prism_coeffs, cfg->image_width, cfg->image_height, cfg->camera_model, w.cam, st);
    if (rc != LFS_OK) return rc;
    cudaMemsetAsync(w.counters, 0, 16 * sizeof(int32_t), st);
    const ProjParams pp = make_proj_params(cfg->eps2d, cfg->near_plane, cfg->far_plane, cfg->radius_clip, cfg->ut);
    PackOptions opt;
    opt.scaling_modifier = cfg_modifier(*cfg);
    opt.calc_compensations = cfg->calc_compensations;
    opt.want_rgb = with_colors && mode_channels(cfg->render_mode) != 1;
    rc = launch_project_pack(cfg->N, cfg->sh_coeffs, cfg->sh_degree, *params, w.cam, pp, opt, cfg_model(*cfg), cfg_rolling(*cfg), cfg->tile_size, tw,
                             th, w.radii, w.means2d, w.depths, w.tiles, w.gkeys[0], w.gvals[0], w.records, w.bounds,
                             reinterpret_cast<float4*>(w.accum), w.counters + 2, st);
    if (rc != LFS_OK) return rc;
    if (projected && cudaEventRecord(projected, st) != cudaSuccess) { set_error("cudaEventRecord failed"); return LFS_ECUDA; }
    TileListArgs a{};
    a.C = 1; a.N = cfg->N; a.tw = tw; a.th = th; a.tile_size = cfg->tile_size; a.sort = 1; a.keys_ready = 1;
    a.means2d = w.means2d; a.radii = w.radii; a.depths = w.depths; a.tiles = w.tiles;
    for (int k = 0; k < 2; ++k) { a.gkeys[k] = w.gkeys[k]; a.gvals[k] = w.gvals[k]; a.tkeys[k] = w.tkeys[k]; a.tvals[k] = w.tvals[k]; }
    a.offs = w.offs; a.n_isects_dev = w.counters + 1; a.capacity = cfg->isect_capacity; a.overflow = w.counters + 0;
    a.sel_out = sel_out;
    a.tile_offsets = w.tile_offsets; a.scratch = w.scratch;
    rc = build_tile_lists(a, st);
    if (rc != LFS_OK) return rc;
    return launch_tile_order(tw * th, w.tile_offsets, w.tile_order, st);
}

static int render_forward_blend(const lfs_render_config* cfg, const float* background, float* render, float* alpha,
                                int32_t* status_dev, RenderWs& w, int sel, cudaStream_t st) {
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    RasterArgs ra{w.cam, w.records, w.bounds, w.tvals[sel], w.tile_offsets, w.counters + 1, 0, background, w.counters + 0,
                  cfg->image_width, cfg->image_height, tw, th, cfg_model(*cfg), mode_channels(cfg->render_mode),
                  mode_normalize(cfg->render_mode), cfg->tile_masks, w.tile_order, cfg_rolling(*cfg)};
    int rc = launch_raster_fwd(ra, render, alpha, w.last_ids, w.extra_sum, st);
    if (rc != LFS_OK) return rc;
    if (status_dev) cudaMemcpyAsync(status_dev, w.counters, 4 * sizeof(int32_t), cudaMemcpyDeviceToDevice, st);
    return LFS_OK;
}

int lfs_render_forward(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat, const float* K,
                       const float* background, float* render, float* alpha,
                       int32_t* status_dev, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && viewmat && K && render && alpha && workspace, "null pointer");
    LFS_REQUIRE(aligned16(params->rotation_raw), "rotation_raw must be 16-byte aligned");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_render_forward: workspace too small (%zu < %zu)", workspace_bytes, w.bytes); return LFS_ECAPACITY; }
    cudaStream_t st = S(stream);
    int sel = 0;
    rc = render_forward_lists(cfg, params, viewmat, K, 1, w, &sel, st);
    if (rc != LFS_OK) return rc;
    rc = render_forward_blend(cfg, background, render, alpha, status_dev, w, sel, st);
    if (rc != LFS_OK) return rc;
    return check_launch("lfs_render_forward");
}

int lfs_render_forward_lists_event(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat, const float* K,
                                   void* projected_event, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && viewmat && K && workspace, "null pointer");
    LFS_REQUIRE(aligned16(params->rotation_raw), "rotation_raw must be 16-byte aligned");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_render_forward_lists: workspace too small"); return LFS_ECAPACITY; }
    int sel = 0;
    rc = render_forward_lists(cfg, params, viewmat, K, 0, w, &sel, S(stream), reinterpret_cast<cudaEvent_t>(projected_event));
    if (rc != LFS_OK) return rc;
    return check_launch("lfs_render_forward_lists");
}

int lfs_render_forward_lists(const lfs_render_config* cfg, const lfs_splats* params, const float* viewmat, const float* K,
                             void* workspace, size_t workspace_bytes, void* stream) {
    return lfs_render_forward_lists_event(cfg, params, viewmat, K, nullptr, workspace, workspace_bytes, stream);
}

int lfs_render_forward_shade(const lfs_render_config* cfg, const lfs_splats* params, const float* background, float* render,
                             float* alpha, int32_t* status_dev, void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && render && alpha && workspace, "null pointer");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_render_forward_shade: workspace too small"); return LFS_ECAPACITY; }
    cudaStream_t st = S(stream);
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    const int sel = sorted_sel((int)(bit_width_u32((uint32_t)tw * th) + 1));
    if (mode_channels(cfg->render_mode) != 1) {
        rc = launch_sh_color(cfg->N, cfg->sh_coeffs, cfg->sh_degree, *params, w.cam, w.radii, w.records, st);
        if (rc != LFS_OK) return rc;
    }
    rc = render_forward_blend(cfg, background, render, alpha, status_dev, w, sel, st);
    if (rc != LFS_OK) return rc;
    return check_launch("lfs_render_forward_shade");
}

int lfs_render_backward(const lfs_render_config* cfg, const lfs_splats* params, const float* background, const float* alpha,
                        const float* v_render, const float* v_alpha, const lfs_splats* grads, int accumulate, void* workspace,
                        size_t workspace_bytes, void* stream) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && alpha && v_render && grads && workspace, "null pointer");
    LFS_REQUIRE(aligned16(params->rotation_raw) && aligned16(grads->rotation_raw), "rotation_raw tensors must be 16-byte aligned");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_render_backward: workspace too small"); return LFS_ECAPACITY; }
    cudaStream_t st = S(stream);
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    const int sel = sorted_sel((int)(bit_width_u32((uint32_t)tw * th) + 1));
    RasterArgs ra{w.cam, w.records, w.bounds, w.tvals[sel], w.tile_offsets, w.counters + 1, 0, background, w.counters + 0,
                  cfg->image_width, cfg->image_height, tw, th, cfg_model(*cfg), mode_channels(cfg->render_mode),
                  mode_normalize(cfg->render_mode), cfg->tile_masks, w.tile_order, cfg_rolling(*cfg)};
    rc = launch_raster_bwd(ra, alpha, w.last_ids, w.extra_sum, v_render, v_alpha, w.accum, nullptr, st);
    if (rc != LFS_OK) return rc;
    const int sh_factors = (accumulate & LFS_BACKWARD_SH_FACTORS) != 0;
    if (sh_factors) LFS_REQUIRE(!(accumulate & LFS_BACKWARD_ACCUMULATE), "the shN factors of several cameras cannot be accumulated");
    if (sh_factors && grads->shN) LFS_REQUIRE((reinterpret_cast<uintptr_t>(grads->shN) & 7) == 0, "grads->shN must be 8-byte aligned");
    return launch_grad_epilogue_fused(cfg->N, cfg->sh_coeffs, cfg->sh_degree, w.cam, w.accum, w.records, w.radii, *params,
                                      *grads, accumulate & LFS_BACKWARD_ACCUMULATE, cfg_modifier(*cfg), sh_factors, st);
}

int lfs_render_backward_adam(const lfs_render_config* cfg, const lfs_splats* params, const float* background,
                             const float* alpha, const float* v_render, const float* v_alpha, const lfs_splats* exp_avg,
                             const lfs_splats* exp_avg_sq, const float* lr, double beta1, double beta2, double eps,
                             int64_t step_count, int skip_shN, float grad_scale, void* workspace, size_t workspace_bytes,
                             void* stream) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && alpha && v_render && exp_avg && exp_avg_sq && lr && workspace, "null pointer");
    LFS_REQUIRE(step_count >= 1, "step_count must be >= 1");
    LFS_REQUIRE(aligned16(params->rotation_raw), "rotation_raw must be 16-byte aligned");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_render_backward_adam: workspace too small"); return LFS_ECAPACITY; }
    const int K = cfg->sh_coeffs;
    // the same host arithmetic as lfs_adam_step_splats
    const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
    const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
    float* P[5] = {params->means, params->sh0, params->scaling_raw, params->rotation_raw, params->opacity_raw};
    float* M[5] = {exp_avg->means, exp_avg->sh0, exp_avg->scaling_raw, exp_avg->rotation_raw, exp_avg->opacity_raw};
    float* V[5] = {exp_avg_sq->means, exp_avg_sq->sh0, exp_avg_sq->scaling_raw, exp_avg_sq->rotation_raw, exp_avg_sq->opacity_raw};
    const int lr_index[5] = {0, 1, 3, 4, 5};
    AdamSmall A{};
    for (int k = 0; k < 5; ++k) {
        if (cfg->N > 0) LFS_REQUIRE(P[k] && M[k] && V[k], "null tensor in a parameter group");
        A.p[k] = P[k]; A.m[k] = M[k]; A.v[k] = V[k];
        A.step_size[k] = (float)((double)lr[lr_index[k]]) * (float)bc1;
    }
    A.beta1 = (float)beta1; A.beta2 = (float)beta2; A.eps = (float)eps; A.bc2_sqrt_rcp = (float)bc2; A.grad_scale = grad_scale;
    const bool with_shN = !skip_shN && K > 1 && cfg->N > 0;
    if (with_shN) LFS_REQUIRE(params->shN && exp_avg->shN && exp_avg_sq->shN, "null tensor in a parameter group");
    cudaStream_t st = S(stream);
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    const int sel = sorted_sel((int)(bit_width_u32((uint32_t)tw * th) + 1));
    RasterArgs ra{w.cam, w.records, w.bounds, w.tvals[sel], w.tile_offsets, w.counters + 1, 0, background, w.counters + 0,
                  cfg->image_width, cfg->image_height, tw, th, cfg_model(*cfg), mode_channels(cfg->render_mode),
                  mode_normalize(cfg->render_mode), cfg->tile_masks, w.tile_order, cfg_rolling(*cfg)};
    rc = launch_raster_bwd(ra, alpha, w.last_ids, w.extra_sum, v_render, v_alpha, w.accum, nullptr, st);
    if (rc != LFS_OK) return rc;
    lfs_splats none{};
    rc = launch_grad_epilogue_fused(cfg->N, K, cfg->sh_degree, w.cam, w.accum, w.records, w.radii, *params, none, 0,
                                    cfg_modifier(*cfg), 1, st, &A);
    if (rc != LFS_OK || !with_shN) return rc;
    // the factors of the shN rows are now in the rows of the 16 sums (stride 16 floats)
    return launch_adam_sh_rank1(cfg->N, K, cfg->sh_degree, nullptr, nullptr, nullptr, params->shN, exp_avg->shN, exp_avg_sq->shN,
                                (float)((double)lr[2]) * (float)bc1, (float)beta1, (float)beta2, (float)eps, (float)bc2, grad_scale,
                                st, w.accum, 16);
}

int lfs_adam_step_splats_rank1_sh(const lfs_render_config* cfg, const lfs_splats* params, const lfs_splats* exp_avg,
                                  const lfs_splats* exp_avg_sq, const lfs_splats* grads, const float* lr, double beta1,
                                  double beta2, double eps, int64_t step_count, int skip_shN, float grad_scale,
                                  void* workspace, size_t workspace_bytes, void* stream) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(params && exp_avg && exp_avg_sq && grads && lr && workspace, "null pointer");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_adam_step_splats_rank1_sh: workspace too small"); return LFS_ECAPACITY; }
    // shN first: its gradient rows depend on the means, which the second launch updates
    if (!skip_shN && cfg->sh_coeffs > 1 && cfg->N > 0) {
        LFS_REQUIRE(params->shN && exp_avg->shN && exp_avg_sq->shN && grads->sh0 && params->means, "null tensor in a parameter group");
        const double bc1 = 1.0 / (1.0 - std::pow(beta1, (double)step_count));
        const double bc2 = 1.0 / std::sqrt(1.0 - std::pow(beta2, (double)step_count));
        const float* campos = reinterpret_cast<const float*>(reinterpret_cast<const char*>(w.cam) + offsetof(CamDev, campos));
        rc = launch_adam_sh_rank1(cfg->N, cfg->sh_coeffs, cfg->sh_degree, campos, params->means, grads->sh0, params->shN,
                                  exp_avg->shN, exp_avg_sq->shN, (float)((double)lr[2]) * (float)bc1, (float)beta1, (float)beta2,
                                  (float)eps, (float)bc2, grad_scale, S(stream));
        if (rc != LFS_OK) return rc;
    }
    // the five small groups from their gradient tensors, exactly as lfs_adam_step_splats does
    return lfs_adam_step_splats(cfg->N, cfg->sh_coeffs, params, exp_avg, exp_avg_sq, grads, lr, beta1, beta2, eps, step_count,
                                /*skip_shN=*/1, 0, cfg->N, grad_scale, stream);
}

int lfs_render_workspace_view(const lfs_render_config* cfg, void* workspace, size_t workspace_bytes, lfs_render_view* view) {
    int rc = check_cfg(cfg);
    if (rc != LFS_OK) return rc;
    LFS_REQUIRE(workspace && view, "null pointer");
    RenderWs w = carve_render(*cfg, workspace);
    if (workspace_bytes < w.bytes) { set_error("lfs_render_workspace_view: workspace too small"); return LFS_ECAPACITY; }
    const int tw = (cfg->image_width + 15) / 16, th = (cfg->image_height + 15) / 16;
    const int sel = sorted_sel((int)(bit_width_u32((uint32_t)tw * th) + 1));
    view->radii = w.radii; view->means2d = w.means2d; view->depths = w.depths; view->tiles_per_gauss = w.tiles;
    view->tile_offsets = w.tile_offsets; view->flatten_ids = reinterpret_cast<const int32_t*>(w.tvals[sel]);
    view->last_ids = w.last_ids; view->records = reinterpret_cast<const float*>(w.records);
    return LFS_OK;
}

// ---------------------------------------------------------------------------------------------
static size_t mcmc_ws(int N, void* base, int32_t** flags, int32_t** offs, int32_t** total, SortScratch* s) {
    Carver c(base);
    *flags = c.take<int32_t>((size_t)N);
    *offs = c.take<int32_t>((size_t)N);
    *total = c.take<int32_t>(16);
    *s = carve_scratch(c);
    return c.total();
}

size_t lfs_mcmc_workspace_bytes(int N) {
    int32_t *a, *b, *t;
    SortScratch s;
    return mcmc_ws(N, nullptr, &a, &b, &t, &s);
}

int lfs_mcmc_classify(int N, const float* opacity_raw, const float* rotation_raw, float min_opacity, int64_t* dead_indices,
                      int64_t* alive_indices, float* alive_opacities, int32_t* counts_dev, void* workspace,
                      size_t workspace_bytes, void* stream) {
    LFS_REQUIRE(N >= 0, "bad size");
    LFS_REQUIRE(counts_dev && workspace, "null pointer");
    if (N > 0) LFS_REQUIRE(opacity_raw && rotation_raw && dead_indices && alive_indices && alive_opacities, "null pointer");
    LFS_REQUIRE(aligned16(rotation_raw), "rotation_raw must be 16-byte aligned");
    int32_t *flags, *offs, *total;
    SortScratch s;
    if (workspace_bytes < mcmc_ws(N, workspace, &flags, &offs, &total, &s)) { set_error("lfs_mcmc_classify: workspace too small"); return LFS_ECAPACITY; }
    return launch_mcmc_classify(N, opacity_raw, rotation_raw, min_opacity, dead_indices, alive_indices, alive_opacities,
                                counts_dev, flags, offs, total, s, S(stream));
}

int lfs_mcmc_map_indices(int n, const int64_t* local_indices, const int64_t* index_map, int64_t* out, void* stream) {
    LFS_REQUIRE(n >= 0, "bad size");
    if (n == 0) return LFS_OK;
    LFS_REQUIRE(local_indices && index_map && out, "null pointer");
    return launch_mcmc_map_indices(n, local_indices, index_map, out, S(stream));
}

int lfs_mcmc_gather_ratios(int N, int n_sampled, const int64_t* sampled, const float* opacity_raw, const float* scaling_raw,
                           int n_max, int32_t* counts, int32_t* ratios, float* sampled_opacities, float* sampled_scales,
                           void* stream) {
    LFS_REQUIRE(N >= 0 && n_sampled >= 0 && n_max > 0, "bad sizes");
    LFS_REQUIRE(counts != nullptr || N == 0, "null pointer");
    if (n_sampled > 0) LFS_REQUIRE(sampled && opacity_raw && scaling_raw && ratios && sampled_opacities && sampled_scales, "null pointer");
    return launch_mcmc_gather_ratios(N, n_sampled, sampled, opacity_raw, scaling_raw, n_max, counts, ratios, sampled_opacities,
                                     sampled_scales, S(stream));
}

int lfs_mcmc_apply(int N, int K, int n_sampled, const int64_t* sampled, const int64_t* dst_indices, const float* new_opacities,
                   const float* new_scales, float min_opacity, const lfs_splats* params, const lfs_splats* exp_avg,
                   const lfs_splats* exp_avg_sq, void* stream) {
    LFS_REQUIRE(N >= 0 && K >= 1 && n_sampled >= 0, "bad sizes");
    if (n_sampled == 0) return LFS_OK;
    LFS_REQUIRE(sampled && new_opacities && new_scales && params, "null pointer");
    return launch_mcmc_apply(N, K, n_sampled, sampled, dst_indices, new_opacities, new_scales, min_opacity, *params, exp_avg,
                             exp_avg_sq, S(stream));
}

}  // extern "C"
