// Alpha-blend rasterizer by ray / Gaussian distance: forward, backward and the per-Gaussian
// gradient epilogues.
//
// Replaces gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu:20 (K7), gsplat/RasterizeToPixelsFromWorld3DGSBwd.cu:17
// (K8) with the VJPs of gsplat/Utils.cuh:104-194, gsplat/SphericalHarmonicsCUDA.cu:445 (K3) and the
// activation backward that autograd performs for src/core/splat_data.cpp:267-286.
//
// Design (instruction-issue bound, no tensor cores: the largest contraction is 3x3):
//  * one CTA per 16x16 tile, one thread per pixel, warps cover 8x4 pixel patches;
//  * the tile's depth-sorted Gaussians are staged in shared memory in batches (192 records forward, 64 backward) of
//    packed 64-byte records (M = S^-1 R^T, gro = M (o - mu), colour, opacity) built once per Gaussian,
//    so no quaternion -> matrix work is repeated per tile or per pixel;
//  * per warp, a ballot over the batch keeps the records whose screen-space box overlaps the warp's 8x4 patch;
//  * per pair the response is -0.5 |u x gro|^2 / |u|^2 with u = M d (same value as the normalised
//    cross-product form), preceded by an exp-free conservative rejection test;
//  * backward: every (warp, Gaussian) contribution is 16 numbers that are LINEAR in the per-pixel
//    terms (sum v_u (x) d, sum v_gro, v_rgb, v_opacity). They are summed over the warp by a transpose through
//    padded shared-memory rows (warp_reduce16), combined across the 8 warps by shared-memory atomics, and leave the
//    CTA as four float4 reductions per (tile, Gaussian). The nonlinear quaternion / scale VJP runs once per Gaussian
//    in the epilogue instead of once per pixel pair.
#include "gsmath.cuh"
#include "raster.cuh"

namespace lfs {

namespace {

constexpr int kBlock = 256;
constexpr float kAlphaMin = 1.f / 255.f;

__device__ __forceinline__ void pixel_of_thread(int tile, int tw, int& i, int& j) {
    // warps tile the 16x16 block as 2 x 4 patches of 8 x 4 pixels
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int lx = (warp & 1) * 8 + (lane & 7);
    const int ly = (warp >> 1) * 4 + (lane >> 3);
    i = (tile / tw) * 16 + ly;
    j = (tile % tw) * 16 + lx;
}

// Warp patch of 8x4 pixels: inclusive pixel bounds packed like the Gaussian boxes (lo | hi << 16).
__device__ __forceinline__ void warp_patch(int tile, int tw, uint32_t& px, uint32_t& py) {
    const int warp = threadIdx.x >> 5;
    const uint32_t x0 = (tile % tw) * 16 + (warp & 1) * 8, y0 = (tile / tw) * 16 + (warp >> 1) * 4;
    px = x0 | ((x0 + 7) << 16);
    py = y0 | ((y0 + 3) << 16);
}
__device__ __forceinline__ bool box_overlaps(uint2 box, uint32_t px, uint32_t py) {
    return (box.x & 0xFFFFu) <= (px >> 16) && (box.x >> 16) >= (px & 0xFFFFu) &&
           (box.y & 0xFFFFu) <= (py >> 16) && (box.y >> 16) >= (py & 0xFFFFu);
}

__device__ __forceinline__ int32_t load_count(const int32_t* n_dev, int64_t n_host) {
    return n_dev ? *n_dev : (int32_t)n_host;
}

// ---------------------------------------------------------------------------------------------
// Staging of one batch of tile entries into shared memory with 16-byte asynchronous copies
// (cp.async: the entries are a gather by Gaussian index, so each copy is one quarter record or one
// bounds row). Two buffers: batch b+1 is in flight while batch b is being blended.
template <int BATCH>
struct Stage {
    float4 rec[BATCH * 4];  // packed records
    uint4 box[BATCH];       // (x box, y box, rejection exponent as float bits, unused)
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Each thread owns kParts quarter-record slots q = k * kBlock + tid of a batch: entry q >> 2, part q & 3.
template <int BATCH>
struct StageIds {
    static constexpr int kParts = (BATCH * 4 + kBlock - 1) / kBlock;
    uint32_t g[kParts];
};

// ids of the batch whose first list position is `first` and which runs forward (step +1) or backward (-1)
template <int BATCH>
__device__ __forceinline__ void load_ids(StageIds<BATCH>& ids, const uint32_t* __restrict__ flatten_ids, int32_t first,
                                         int step, int batch_size) {
#pragma unroll
    for (int k = 0; k < StageIds<BATCH>::kParts; ++k) {
        const int e = (k * kBlock + threadIdx.x) >> 2;
        ids.g[k] = e < batch_size ? flatten_ids[first + step * e] : 0u;
    }
}

template <int BATCH>
__device__ __forceinline__ void issue_stage(Stage<BATCH>& st, uint32_t* sid, const StageIds<BATCH>& ids,
                                            const float4* __restrict__ records, const uint4* __restrict__ bounds,
                                            int batch_size) {
#pragma unroll
    for (int k = 0; k < StageIds<BATCH>::kParts; ++k) {
        const int q = k * kBlock + threadIdx.x;
        const int e = q >> 2, part = q & 3;
        if (e < batch_size) {
            cp_async16(&st.rec[q], records + (size_t)ids.g[k] * 4 + part);
            if (part == 0) {
                cp_async16(&st.box[e], bounds + ids.g[k]);
                if (sid) sid[e] = ids.g[k];
            }
        }
    }
    cp_async_commit();
}

// ---------------------------------------------------------------------------------------------
// EXTRA = false: three colour channels (render mode RGB). EXTRA = true: `channels` is 1 or 4 and the last
// channel blends the per-Gaussian value kept in bounds.w (the depth in the render modes D / ED / RGB_D /
// RGB_ED of gsplat/Rasterization.cpp:373-393); `normalize` divides it by max(alpha, 1e-10) on output (the
// expected-depth modes of src/training/rasterization/rasterizer.cpp:186-198) and keeps the undivided value
// in extra_sum for the backward.
// RS: rolling shutter. Every pixel has its own pose, hence its own ray origin; the record's gro = M (o_start - mu) is
// corrected per pair by M (o_pixel - o_start).
// The plain pinhole RGB instantiation fits 40 registers (12 bytes of spills outside the loop) and, with 192-record batches
// (30 KB for the two staging buffers), six CTAs per SM; the other instantiations keep their 48 - 64 registers.
template <int MODEL, bool EXTRA, bool RS>
__global__ void __launch_bounds__(kBlock, (MODEL == LFS_PINHOLE && !RS && !EXTRA) ? 6 : 4) raster_fwd_kernel(
    const CamDev* __restrict__ cams, const float4* __restrict__ records, const uint4* __restrict__ bounds,
    const uint32_t* __restrict__ flatten_ids,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ n_isects_dev, int64_t n_isects_host,
    const int32_t* __restrict__ overflow, const float* __restrict__ background, const uint8_t* __restrict__ masks,
    const int32_t* __restrict__ tile_order, int channels, int normalize, int W, int H, int tw, int n_tiles,
    float* __restrict__ render, float* __restrict__ alphas, int32_t* __restrict__ last_ids, float* __restrict__ extra_sum) {
    constexpr int BATCH = 192;
    __shared__ Stage<BATCH> stage[2];

    if (overflow && *overflow) return;
    const int tile = tile_order ? tile_order[blockIdx.x] : blockIdx.x;
    int i, j;
    pixel_of_thread(tile, tw, i, j);
    const bool inside = (i < H && j < W);
    if (masks && !masks[tile]) {
        // a tile labelled false shows the background (gsplat/RasterizeToPixelsFromWorld3DGSFwd.cu:147-155)
        if (inside) {
            const int pid = i * W + j;
            const int ch = EXTRA ? channels : 3;
            for (int k = 0; k < ch; ++k) render[pid * ch + k] = background ? background[k] : 0.f;
            alphas[pid] = 0.f;
            last_ids[pid] = 0;
            if (EXTRA && extra_sum) extra_sum[pid] = background ? background[ch - 1] : 0.f;
        }
        return;
    }
    const CamDev& cam = cams[0];
    f3 d, oo{0.f, 0.f, 0.f};
    const bool ray_ok = RS ? pixel_world_ray_rs<MODEL>(cam, (float)j + 0.5f, (float)i + 0.5f, d, oo)
                           : pixel_world_dir<MODEL>(cam, (float)j + 0.5f, (float)i + 0.5f, d);
    bool done = !inside || !ray_ok;
    uint32_t patch_x, patch_y;
    warp_patch(tile, tw, patch_x, patch_y);

    const int32_t n_isects = load_count(n_isects_dev, n_isects_host);
    const int32_t range_start = tile_offsets[tile];
    const int32_t range_end = (tile == n_tiles - 1) ? n_isects : tile_offsets[tile + 1];
    const int n_batches = (range_end - range_start + BATCH - 1) / BATCH;

    float T = 1.0f;
    uint32_t cur_idx = 0;
    float pr = 0.f, pg = 0.f, pb = 0.f, px = 0.f;

    StageIds<BATCH> ids;
    if (n_batches > 0) {
        load_ids(ids, flatten_ids, range_start, 1, min(BATCH, range_end - range_start));
        issue_stage(stage[0], nullptr, ids, records, bounds, min(BATCH, range_end - range_start));
        if (n_batches > 1) load_ids(ids, flatten_ids, range_start + BATCH, 1, min(BATCH, range_end - range_start - BATCH));
    }
    for (int b = 0; b < n_batches; ++b) {
        const int32_t batch_start = range_start + b * BATCH;
        const int32_t batch_size = min(BATCH, range_end - batch_start);
        // next batch into the other buffer (its previous contents were consumed before the barrier that ended
        // the previous iteration), then the ids of the batch after that
        if (b + 1 < n_batches) {
            issue_stage(stage[(b + 1) & 1], nullptr, ids, records, bounds, min(BATCH, range_end - batch_start - BATCH));
            if (b + 2 < n_batches)
                load_ids(ids, flatten_ids, batch_start + 2 * BATCH, 1, min(BATCH, range_end - batch_start - 2 * BATCH));
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        // everyone's copies of batch b have landed; leave early when every pixel of the tile is finished
        if (__syncthreads_count(done) >= kBlock) break;
        const Stage<BATCH>& st = stage[b & 1];
        if (!__all_sync(0xffffffffu, done)) {
            // entries of this batch whose box overlaps this warp's 8x4 patch: one ballot word per 32 entries
            uint32_t live[BATCH / 32];
#pragma unroll
            for (int w = 0; w < BATCH / 32; ++w) {
                const int e = w * 32 + (threadIdx.x & 31);
                bool ov = false;
                if (e < batch_size) { const uint4 bx = st.box[e]; ov = box_overlaps(make_uint2(bx.x, bx.y), patch_x, patch_y); }
                live[w] = __ballot_sync(0xffffffffu, ov);
            }
#pragma unroll
            for (int w = 0; w < BATCH / 32; ++w) {
                uint32_t bits = live[w];
                while (bits && !done) {
                    const int t = w * 32 + __ffs(bits) - 1;
                    bits &= bits - 1;
                    const float4 r0 = st.rec[t * 4 + 0], r1 = st.rec[t * 4 + 1], r2 = st.rec[t * 4 + 2];
                    const float ux = r0.x * d.x + r0.y * d.y + r0.z * d.z;
                    const float uy = r1.x * d.x + r1.y * d.y + r1.z * d.z;
                    const float uz = r2.x * d.x + r2.y * d.y + r2.z * d.z;
                    float gx = r0.w, gy = r1.w, gz = r2.w;
                    if (RS) {
                        gx += r0.x * oo.x + r0.y * oo.y + r0.z * oo.z;
                        gy += r1.x * oo.x + r1.y * oo.y + r1.z * oo.z;
                        gz += r2.x * oo.x + r2.y * oo.y + r2.z * oo.z;
                    }
                    const float cx = uy * gz - gy * uz;
                    const float cy = uz * gx - gz * ux;
                    const float cz = ux * gy - gx * uy;
                    const float cc = cx * cx + cy * cy + cz * cz;
                    const float uu = ux * ux + uy * uy + uz * uz;
                    // power = -0.5 cc / uu ; reject when power < thr  <=>  cc > -2 thr uu
                    if (cc > -2.0f * __uint_as_float(st.box[t].z) * uu) continue;
                    const float4 r3 = st.rec[t * 4 + 3];
                    const float power = -0.5f * __fdividef(cc, fmaxf(uu, 1e-37f));
                    const float alpha = fminf(0.999f, r3.w * __expf(power));
                    if (alpha < kAlphaMin) continue;
                    const float next_T = T * (1.0f - alpha);
                    if (next_T <= 1e-4f) { done = true; break; }
                    const float vis = alpha * T;
                    pr += r3.x * vis; pg += r3.y * vis; pb += r3.z * vis;
                    if (EXTRA) px += __uint_as_float(st.box[t].w) * vis;
                    cur_idx = (uint32_t)(batch_start + t);
                    T = next_T;
                }
            }
        }
        __syncthreads();  // buffer b & 1 may be refilled by the next iteration's issue
    }
    cp_async_wait<0>();
    if (inside) {
        const int pid = i * W + j;
        alphas[pid] = 1.0f - T;
        if (!EXTRA) {
            if (background) { pr += T * background[0]; pg += T * background[1]; pb += T * background[2]; }
            render[pid * 3 + 0] = pr;
            render[pid * 3 + 1] = pg;
            render[pid * 3 + 2] = pb;
        } else {
            if (channels == 4) {
                if (background) { pr += T * background[0]; pg += T * background[1]; pb += T * background[2]; }
                render[pid * 4 + 0] = pr;
                render[pid * 4 + 1] = pg;
                render[pid * 4 + 2] = pb;
            }
            if (background) px += T * background[channels - 1];
            if (extra_sum) extra_sum[pid] = px;
            render[pid * channels + channels - 1] = normalize ? px / fmaxf(1.0f - T, 1e-10f) : px;
        }
        last_ids[pid] = (int32_t)cur_idx;
    }
}

// ---------------------------------------------------------------------------------------------
// 16 values per lane -> per-value sums over the warp, value k left in lanes 2k and 2k+1.
// The transpose goes through shared memory owned by the warp instead of a shuffle butterfly (about 40 issue slots
// against 90): row k (36 floats, 32 used) holds value k of the 32 lanes. The row stride of 36 floats puts the 16-byte
// loads of one quarter-warp (lane = 2 k + h reads the 16 lanes of half h of row k) on eight different bank groups, and
// the scalar stores of one row are contiguous. The closing shuffle needs every lane's sum, hence every lane's loads,
// before any lane returns, so the next call may overwrite the rows.
constexpr int kRedStride = 36;
__device__ __forceinline__ float warp_reduce16(const float (&v)[16], float* __restrict__ red, int lane) {
#pragma unroll
    for (int k = 0; k < 16; ++k) red[k * kRedStride + lane] = v[k];
    __syncwarp();
    const float4* half = reinterpret_cast<const float4*>(red + (lane >> 1) * kRedStride + 16 * (lane & 1));
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 x = half[q];
        s += (x.x + x.y) + (x.z + x.w);
    }
    return s + __shfl_xor_sync(0xffffffffu, s, 1);
}

__device__ __forceinline__ float __reduce_add_sync_f32(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

template <int BATCH>
struct BwdShared {
    Stage<BATCH> stage[3];       // batch b is walked while b+1 and b+2 are in flight
    uint32_t sid[4][BATCH];      // Gaussian index per slot; four deep: batch b+2 is staged while batch b-1 is flushed
    float sacc[2][BATCH * 16];   // per-slot sums of the batch being walked / the batch being flushed
    float sextra[2][BATCH];
    int stouched[2][BATCH];
    float red[kBlock / 32][16 * kRedStride];  // per-warp transpose rows of warp_reduce16
};

// EXTRA: the output has 1 or 4 channels and its last one blends bounds.w (see the forward). XGRAD: also return
// the gradient of that per-Gaussian value in accum_extra [N] (operator-level colours with 1 or 4 channels;
// the fused render modes drop it like gsplat/Rasterization.cpp:575-590 does).
template <int MODEL, int BATCH, bool EXTRA, bool XGRAD, bool RS>
__global__ void __launch_bounds__(kBlock) raster_bwd_kernel(
    const CamDev* __restrict__ cams, const float4* __restrict__ records, const uint4* __restrict__ bounds,
    const uint32_t* __restrict__ flatten_ids,
    const int32_t* __restrict__ tile_offsets, const int32_t* __restrict__ n_isects_dev, int64_t n_isects_host,
    const int32_t* __restrict__ overflow, const float* __restrict__ background, const uint8_t* __restrict__ masks,
    const int32_t* __restrict__ tile_order, int channels, int normalize, int W, int H, int tw, int n_tiles,
    const float* __restrict__ render_alphas, const int32_t* __restrict__ last_ids, const float* __restrict__ extra_sum,
    const float* __restrict__ v_render, const float* __restrict__ v_alphas, float* __restrict__ accum,
    float* __restrict__ accum_extra) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdShared<BATCH>& sm = *reinterpret_cast<BwdShared<BATCH>*>(smem_raw);

    if (overflow && *overflow) return;
    const int tile = tile_order ? tile_order[blockIdx.x] : blockIdx.x;
    if (masks && !masks[tile]) return;  // gsplat/RasterizeToPixelsFromWorld3DGSBwd.cu:84
    int i, j;
    pixel_of_thread(tile, tw, i, j);
    const bool inside = (i < H && j < W);
    const CamDev& cam = cams[0];
    f3 d, oo{0.f, 0.f, 0.f};
    const bool ray_ok = RS ? pixel_world_ray_rs<MODEL>(cam, (float)j + 0.5f, (float)i + 0.5f, d, oo)
                           : pixel_world_dir<MODEL>(cam, (float)j + 0.5f, (float)i + 0.5f, d);
    const bool active = inside && ray_ok;
    const int pid = min(i * W + j, W * H - 1);
    uint32_t patch_x, patch_y;
    warp_patch(tile, tw, patch_x, patch_y);

    const int32_t n_isects = load_count(n_isects_dev, n_isects_host);
    const int32_t range_start = tile_offsets[tile];
    const int32_t range_end = (tile == n_tiles - 1) ? n_isects : tile_offsets[tile + 1];
    const int n_batches = (range_end - range_start + BATCH - 1) / BATCH;

    const float T_final = 1.0f - render_alphas[pid];
    float T = T_final;
    float bufr = 0.f, bufg = 0.f, bufb = 0.f, bufx = 0.f;
    const int32_t bin_final = active ? last_ids[pid] : 0;
    float vcr, vcg, vcb, vcx = 0.f;
    float v_a = v_alphas ? v_alphas[pid] : 0.f;
    if (!EXTRA) {
        vcr = v_render[pid * 3 + 0]; vcg = v_render[pid * 3 + 1]; vcb = v_render[pid * 3 + 2];
    } else {
        vcr = vcg = vcb = 0.f;
        if (channels == 4) { vcr = v_render[pid * 4 + 0]; vcg = v_render[pid * 4 + 1]; vcb = v_render[pid * 4 + 2]; }
        vcx = v_render[pid * channels + channels - 1];
        if (normalize) {
            // output = sum / max(alpha, 1e-10): chain rule of the division and of clamp_min
            const float a = 1.0f - T_final, ac = fmaxf(a, 1e-10f);
            if (a > 1e-10f) v_a -= extra_sum[pid] / (ac * ac) * vcx;
            vcx = vcx / ac;
        }
    }
    float bg_dot = 0.f;
    if (background) {
        if (!EXTRA || channels == 4) bg_dot = background[0] * vcr + background[1] * vcg + background[2] * vcb;
        if (EXTRA) bg_dot += background[channels - 1] * vcx;
    }
    const float tail_c = T_final * (v_a - bg_dot);
    const int32_t warp_bin_final = __reduce_max_sync(0xffffffffu, bin_final);
    const int lane = threadIdx.x & 31;
    float* red = sm.red[threadIdx.x >> 5];

    for (int e = threadIdx.x; e < 2 * BATCH; e += kBlock) {
#pragma unroll
        for (int k = 0; k < 16; ++k) (&sm.sacc[0][0])[e * 16 + k] = 0.f;
        (&sm.sextra[0][0])[e] = 0.f;
        (&sm.stouched[0][0])[e] = 0;
    }
    // flush the sums of batch k (four 16-byte reductions per touched Gaussian) and leave its buffers zeroed
    auto flush = [&](int k) {
        const int size_k = min(BATCH, range_end - k * BATCH - range_start);
        float* acc_k = sm.sacc[k & 1];
        for (int e = threadIdx.x; e < size_k; e += kBlock) {
            if (sm.stouched[k & 1][e]) {
                const uint32_t g = sm.sid[k & 3][e];
                float4* dst = reinterpret_cast<float4*>(accum) + (size_t)g * 4;
                float4* src = reinterpret_cast<float4*>(acc_k) + e * 4;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    atomicAdd(dst + q, src[q]);
                    src[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                if (XGRAD) { atomicAdd(accum_extra + g, sm.sextra[k & 1][e]); sm.sextra[k & 1][e] = 0.f; }
                sm.stouched[k & 1][e] = 0;
            }
        }
    };

    // batches run back to front: slot e of batch b holds list position batch_end - e
    StageIds<BATCH> ids;
    auto batch_count = [&](int k) { return min(BATCH, range_end - k * BATCH - range_start); };
    auto batch_top = [&](int k) { return range_end - 1 - k * BATCH; };
    if (n_batches > 0) {
        load_ids(ids, flatten_ids, batch_top(0), -1, batch_count(0));
        issue_stage(sm.stage[0], sm.sid[0], ids, records, bounds, batch_count(0));
        if (n_batches > 1) {
            load_ids(ids, flatten_ids, batch_top(1), -1, batch_count(1));
            issue_stage(sm.stage[1], sm.sid[1], ids, records, bounds, batch_count(1));
            if (n_batches > 2) load_ids(ids, flatten_ids, batch_top(2), -1, batch_count(2));
        }
    }
    // One barrier per batch: after it, batch b is in shared memory and every warp has finished walking batch b-1,
    // so batch b+2 may be staged over b-1's records and b-1's sums may be flushed while batch b is walked.
    for (int b = 0; b < n_batches; ++b) {
        const int32_t batch_end = batch_top(b);
        const int32_t batch_size = batch_count(b);
        if (b + 1 < n_batches) cp_async_wait<1>(); else cp_async_wait<0>();
        __syncthreads();
        if (b + 2 < n_batches) {
            issue_stage(sm.stage[(b + 2) % 3], sm.sid[(b + 2) & 3], ids, records, bounds, batch_count(b + 2));
            if (b + 3 < n_batches) load_ids(ids, flatten_ids, batch_top(b + 3), -1, batch_count(b + 3));
        }
        if (b > 0) flush(b - 1);
        float* sacc = sm.sacc[b & 1];
        const Stage<BATCH>& st = sm.stage[b % 3];
        // entries (back to front) that no pixel of this warp reaches (beyond its last contributor) or whose
        // box misses this warp's 8x4 patch are dropped up front: one ballot word per 32 entries
        const int t_begin = max(0, batch_end - warp_bin_final);
        uint32_t live[BATCH / 32];
#pragma unroll
        for (int w = 0; w < BATCH / 32; ++w) {
            const int e = w * 32 + lane;
            bool ov = false;
            if (e >= t_begin && e < batch_size) { const uint4 bx = st.box[e]; ov = box_overlaps(make_uint2(bx.x, bx.y), patch_x, patch_y); }
            live[w] = __ballot_sync(0xffffffffu, ov);
        }
#pragma unroll
        for (int w = 0; w < BATCH / 32; ++w) {
            uint32_t bits = live[w];
            while (bits) {
                const int t = w * 32 + __ffs(bits) - 1;
                bits &= bits - 1;
                // Every lane evaluates the pair (the record reads are warp-wide broadcasts); lanes that are outside
                // the image, beyond their last contributor or below the alpha threshold continue with alpha = vis = 0,
                // which makes every term they add exactly zero, so no per-lane branching is needed below.
                const float4 r0 = st.rec[t * 4 + 0], r1 = st.rec[t * 4 + 1], r2 = st.rec[t * 4 + 2];
                const float ux = r0.x * d.x + r0.y * d.y + r0.z * d.z;
                const float uy = r1.x * d.x + r1.y * d.y + r1.z * d.z;
                const float uz = r2.x * d.x + r2.y * d.y + r2.z * d.z;
                float gx = r0.w, gy = r1.w, gz = r2.w;
                if (RS) {
                    gx += r0.x * oo.x + r0.y * oo.y + r0.z * oo.z;
                    gy += r1.x * oo.x + r1.y * oo.y + r1.z * oo.z;
                    gz += r2.x * oo.x + r2.y * oo.y + r2.z * oo.z;
                }
                float cx = uy * gz - gy * uz;
                float cy = uz * gx - gz * ux;
                float cz = ux * gy - gx * uy;
                const float cc = cx * cx + cy * cy + cz * cz;
                const float uu = ux * ux + uy * uy + uz * uz;
                bool valid = active && (batch_end - t <= bin_final) && !(cc > -2.0f * __uint_as_float(st.box[t].z) * uu);
                if (!__any_sync(0xffffffffu, valid)) continue;
                const float4 r3 = st.rec[t * 4 + 3];
                const float inv = rsqrtf(fmaxf(uu, 1e-37f));
                cx *= inv; cy *= inv; cz *= inv;  // cross(normalised u, gro)
                const float power = -0.5f * (cx * cx + cy * cy + cz * cz);
                float vis = __expf(power);
                float alpha = fminf(0.999f, r3.w * vis);
                valid = valid && !(alpha < kAlphaMin);
                if (!__any_sync(0xffffffffu, valid)) continue;
                if (!valid) { vis = 0.f; alpha = 0.f; }
                float v[16];
                {
                    const float ra = __frcp_rn(1.0f - alpha);
                    T *= ra;
                    const float fac = alpha * T;
                    v[12] = fac * vcr; v[13] = fac * vcg; v[14] = fac * vcb;
                    float v_alpha = (r3.x * T - bufr * ra) * vcr + (r3.y * T - bufg * ra) * vcg + (r3.z * T - bufb * ra) * vcb;
                    float xval = 0.f;
                    if (EXTRA) {
                        xval = __uint_as_float(st.box[t].w);
                        v_alpha += (xval * T - bufx * ra) * vcx;
                    }
                    v_alpha += ra * tail_c;  // T_final * ra * (v_alpha_out - background . v_colour_out)
                    // geometry and opacity only while alpha is not clamped at 0.999
                    const float gate = (r3.w * vis <= 0.999f) ? vis : 0.f;
                    const float s = -gate * (r3.w * v_alpha);  // v_c = s * c with c = n x g
                    // with n = u / |u|, gn = g . n and w = gn n - g (minus the part of g orthogonal to n):
                    //   v_g = v_c x n = -s w,   v_u = (v_n - (v_n . n) n) / |u| = (s gn / |u|) w
                    const float nx = ux * inv, ny = uy * inv, nz = uz * inv;
                    const float gn = gx * nx + gy * ny + gz * nz;
                    const float wx = gn * nx - gx, wy = gn * ny - gy, wz = gn * nz - gz;
                    const float ku = s * gn * inv;
                    const float vux = ku * wx, vuy = ku * wy, vuz = ku * wz;
                    v[0] = vux * d.x; v[1] = vux * d.y; v[2] = vux * d.z;
                    v[3] = vuy * d.x; v[4] = vuy * d.y; v[5] = vuy * d.z;
                    v[6] = vuz * d.x; v[7] = vuz * d.y; v[8] = vuz * d.z;
                    v[9] = -s * wx; v[10] = -s * wy; v[11] = -s * wz;
                    if (RS) {
                        // g = M (o_start - mu) + M (o_pixel - o_start): the second term adds v_g (x) (o_pixel - o_start) to v_M
                        v[0] += v[9] * oo.x;  v[1] += v[9] * oo.y;  v[2] += v[9] * oo.z;
                        v[3] += v[10] * oo.x; v[4] += v[10] * oo.y; v[5] += v[10] * oo.z;
                        v[6] += v[11] * oo.x; v[7] += v[11] * oo.y; v[8] += v[11] * oo.z;
                    }
                    v[15] = gate * v_alpha;
                    bufr += r3.x * fac; bufg += r3.y * fac; bufb += r3.z * fac;
                    if (EXTRA) bufx += xval * fac;
                    if (XGRAD) {
                        const float xs = __reduce_add_sync_f32(fac * vcx);
                        if (lane == 0) atomicAdd(&sm.sextra[b & 1][t], xs);
                    }
                }
                const float total = warp_reduce16(v, red, lane);
                if ((lane & 1) == 0) atomicAdd(&sacc[t * 16 + (lane >> 1)], total);
                if (lane == 0) sm.stouched[b & 1][t] = 1;
            }
        }
    }
    __syncthreads();
    if (n_batches > 0) flush(n_batches - 1);
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// Per-Gaussian gradient from the 16 accumulated numbers. Outputs gradients w.r.t. the ACTIVATED
// mean / quaternion / scale / opacity and the colour.
// ---------------------------------------------------------------------------------------------
struct GaussGrad {
    float v_mean[3], v_quat[4], v_scale[3], v_opac, v_rgb[3];
};

__device__ __forceinline__ void gaussian_vjp(const CamDev& cam, const float* acc /*16*/, f3 mean, float qw, float qx,
                                             float qy, float qz, f3 scale, GaussGrad& o) {
    float R[9], inv_norm, qn[4];
    quat_to_rotmat_renorm(qw, qx, qy, qz, R, inv_norm, qn);
    const float is[3] = {1.0f / scale.x, 1.0f / scale.y, 1.0f / scale.z};
    const float omu[3] = {cam.ro[0] - mean.x, cam.ro[1] - mean.y, cam.ro[2] - mean.z};
    const float G[3] = {acc[9], acc[10], acc[11]};
    // v_Mt = A + G (x) (o - mu)
    float vMt[9];
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int b = 0; b < 3; ++b) vMt[a * 3 + b] = acc[a * 3 + b] + G[a] * omu[b];
    // v_(o-mu) = Mt^T G with Mt[a][b] = is[a] R[b][a]  ->  sum_a is[a] R[b][a] G[a]
#pragma unroll
    for (int b = 0; b < 3; ++b)
        o.v_mean[b] = -(is[0] * R[b * 3 + 0] * G[0] + is[1] * R[b * 3 + 1] * G[1] + is[2] * R[b * 3 + 2] * G[2]);
    // v_R[a][b] = v_M[a][b] is[b] with v_M = v_Mt^T
    float vR[9];
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int b = 0; b < 3; ++b) vR[a * 3 + b] = vMt[b * 3 + a] * is[b];
    const float w = qn[0], x = qn[1], y = qn[2], z = qn[3];
    const float vqn[4] = {
        2.f * (x * (vR[7] - vR[5]) + y * (vR[2] - vR[6]) + z * (vR[3] - vR[1])),
        2.f * (-2.f * x * (vR[4] + vR[8]) + y * (vR[3] + vR[1]) + z * (vR[6] + vR[2]) + w * (vR[7] - vR[5])),
        2.f * (x * (vR[3] + vR[1]) - 2.f * y * (vR[0] + vR[8]) + z * (vR[7] + vR[5]) + w * (vR[2] - vR[6])),
        2.f * (x * (vR[6] + vR[2]) + y * (vR[7] + vR[5]) - 2.f * z * (vR[0] + vR[4]) + w * (vR[3] - vR[1]))};
    const float dq = vqn[0] * qn[0] + vqn[1] * qn[1] + vqn[2] * qn[2] + vqn[3] * qn[3];
#pragma unroll
    for (int k = 0; k < 4; ++k) o.v_quat[k] = (vqn[k] - dq * qn[k]) * inv_norm;
    // v_scale[j] = -is[j]^2 sum_a R[a][j] v_M[a][j] = -is[j]^2 sum_a R[a][j] vMt[j][a]
#pragma unroll
    for (int jx = 0; jx < 3; ++jx)
        o.v_scale[jx] = -is[jx] * is[jx] * (R[0 * 3 + jx] * vMt[jx * 3 + 0] + R[1 * 3 + jx] * vMt[jx * 3 + 1] + R[2 * 3 + jx] * vMt[jx * 3 + 2]);
    o.v_rgb[0] = acc[12]; o.v_rgb[1] = acc[13]; o.v_rgb[2] = acc[14];
    o.v_opac = acc[15];
}

__global__ void __launch_bounds__(256) grad_epilogue_op_kernel(
    int N, const CamDev* __restrict__ cams, const float* __restrict__ accum, const float* __restrict__ means,
    const float* __restrict__ quats, const float* __restrict__ scales, int channels, const float* __restrict__ accum_extra,
    float* __restrict__ v_means, float* __restrict__ v_quats, float* __restrict__ v_scales, float* __restrict__ v_colors,
    float* __restrict__ v_opacities) {
    const CamDev& cam = cams[0];
    for (int g = blockIdx.x * blockDim.x + threadIdx.x; g < N; g += gridDim.x * blockDim.x) {
        float acc[16];
        const float4* a4 = reinterpret_cast<const float4*>(accum) + (size_t)g * 4;
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float4 t = a4[k]; acc[k * 4] = t.x; acc[k * 4 + 1] = t.y; acc[k * 4 + 2] = t.z; acc[k * 4 + 3] = t.w; }
        const float4 q = reinterpret_cast<const float4*>(quats)[g];
        GaussGrad o;
        gaussian_vjp(cam, acc, f3{means[g * 3], means[g * 3 + 1], means[g * 3 + 2]}, q.x, q.y, q.z, q.w,
                     f3{scales[g * 3], scales[g * 3 + 1], scales[g * 3 + 2]}, o);
#pragma unroll
        for (int k = 0; k < 3; ++k) { v_means[g * 3 + k] = o.v_mean[k]; v_scales[g * 3 + k] = o.v_scale[k]; }
        if (channels >= 3) {
#pragma unroll
            for (int k = 0; k < 3; ++k) v_colors[(size_t)g * channels + k] = o.v_rgb[k];
        }
        if (channels != 3) v_colors[(size_t)g * channels + channels - 1] = accum_extra[g];
#pragma unroll
        for (int k = 0; k < 4; ++k) v_quats[g * 4 + k] = o.v_quat[k];
        v_opacities[g] = o.v_opac;
    }
}

__device__ __forceinline__ void adam_small_update(float& p, float& m, float& v, float g, float step_size, const AdamSmall& A) {
    const float m1 = A.beta1 * m + (1.0f - A.beta1) * g;
    const float m2 = A.beta2 * v + (1.0f - A.beta2) * g * g;
    const float denom = sqrtf(m2) * A.bc2_sqrt_rcp + A.eps;
    p -= step_size * m1 / denom;
    m = m1;
    v = m2;
}
// One row of W floats of small group `gi` (index into AdamSmall): p_in are the parameter values already in registers.
template <int W>
__device__ __forceinline__ void adam_small_row(const AdamSmall& A, int gi, size_t row, const float* p_in, const float* grad) {
    float* mm = A.m[gi] + row * W;
    float* vv = A.v[gi] + row * W;
    float* pp = A.p[gi] + row * W;
    float p[W], m[W], v[W];
#pragma unroll
    for (int k = 0; k < W; ++k) { p[k] = p_in[k]; m[k] = mm[k]; v[k] = vv[k]; }
#pragma unroll
    for (int k = 0; k < W; ++k) adam_small_update(p[k], m[k], v[k], grad[k] * A.grad_scale, A.step_size[gi], A);
#pragma unroll
    for (int k = 0; k < W; ++k) { pp[k] = p[k]; mm[k] = m[k]; vv[k] = v[k]; }
}

// Fused-path epilogue: raw-parameter gradients (activation backward folded in) and the SH backward.
// Each warp handles 32 consecutive Gaussians per iteration; their shN gradient rows (the bulk of the
// output, (K-1)*3 floats each) are staged in shared memory and written as one contiguous run.
// ADAM: the five small groups (means, sh0, scales, rotations, opacities) are not written as gradients but applied at
// once, in place, with the moments in A (the parameter pointers below alias A.p, hence no __restrict__ on them); the
// shN gradient leaves as its two rank-1 factors (sh_factors) for adam_sh_rank1_kernel.
template <bool ADAM>
__global__ void __launch_bounds__(256, 4) grad_epilogue_fused_kernel(
    int N, int K, int sh_degree, const CamDev* __restrict__ cams, const float* accum /* ADAM: aliased by g_shN */,
    const float4* __restrict__ records, const int32_t* __restrict__ radii,
    const float* means, const float* sh0, const float* scaling_raw, const float* rotation_raw, const float* opacity_raw,
    float* __restrict__ g_means, float* __restrict__ g_sh0, float* g_shN, float* __restrict__ g_scaling,
    float* __restrict__ g_rotation, float* __restrict__ g_opacity, int accumulate, float scaling_modifier, int sh_factors,
    AdamSmall A) {
    extern __shared__ float s_rows[];
    const CamDev& cam = cams[0];
    const int rest = (K - 1) * 3;
    const int nb = (sh_degree + 1) * (sh_degree + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my = s_rows + (size_t)warp * 32 * rest;
    const int n_chunks = (N + 31) / 32;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int chunk = blockIdx.x * (blockDim.x >> 5) + warp; chunk < n_chunks; chunk += warps_total) {
        const int g = chunk * 32 + lane;
        const bool in_range = g < N;
        // Everything a visible Gaussian needs is requested together with its radii (one round trip to memory instead of
        // two); for the others the values are dropped.
        int2 rad = make_int2(0, 0);
        float4 a_in[4], qr = make_float4(1.f, 0.f, 0.f, 0.f), r3 = make_float4(0.f, 0.f, 0.f, 0.f);
        float m_in[3] = {0.f, 0.f, 0.f}, s_in[3] = {0.f, 0.f, 0.f}, o_in = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) a_in[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in_range) {
            rad = reinterpret_cast<const int2*>(radii)[g];
            if (rad.x > 0 && rad.y > 0) {   // culled Gaussians have no accumulator row: the projection zeroes visible rows only
                const float4* a4 = reinterpret_cast<const float4*>(accum) + (size_t)g * 4;
#pragma unroll
                for (int k = 0; k < 4; ++k) a_in[k] = a4[k];
            }
#pragma unroll
            for (int k = 0; k < 3; ++k) { m_in[k] = means[g * 3 + k]; s_in[k] = scaling_raw[g * 3 + k]; }
            o_in = opacity_raw[g];
            qr = reinterpret_cast<const float4*>(rotation_raw)[g];
            r3 = records[(size_t)g * 4 + 3];
        }
        const bool visible = in_range && rad.x > 0 && rad.y > 0;
        float gm[3] = {0.f, 0.f, 0.f}, g0[3] = {0.f, 0.f, 0.f}, gs[3] = {0.f, 0.f, 0.f}, gq[4] = {0.f, 0.f, 0.f, 0.f}, go = 0.f;
        float vc[3] = {0.f, 0.f, 0.f};
        float B[25];
#pragma unroll
        for (int k = 0; k < 25; ++k) B[k] = 0.f;
        if (visible) {
            float acc[16];
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float4 t = a_in[k]; acc[k * 4] = t.x; acc[k * 4 + 1] = t.y; acc[k * 4 + 2] = t.z; acc[k * 4 + 3] = t.w; }
            const f3 mean{m_in[0], m_in[1], m_in[2]};
            const float opacity = (float)(1.0 / (1.0 + exp(-(double)o_in)));
            // scale as blended: exp(raw) * modifier; d(scale)/d(raw) is the same product
            f3 scale{(float)exp((double)s_in[0]), (float)exp((double)s_in[1]), (float)exp((double)s_in[2])};
            if (scaling_modifier != 1.0f) { scale.x *= scaling_modifier; scale.y *= scaling_modifier; scale.z *= scaling_modifier; }
            const float n2 = ((qr.x * qr.x + qr.y * qr.y) + qr.z * qr.z) + qr.w * qr.w;
            const float nrm = fmaxf(sqrtf(n2), 1e-12f);
            const float q[4] = {qr.x / nrm, qr.y / nrm, qr.z / nrm, qr.w / nrm};
            GaussGrad o;
            gaussian_vjp(cam, acc, mean, q[0], q[1], q[2], q[3], scale, o);
            // activation backward: sigmoid, exp, x / max(|x|, eps)
            go = o.v_opac * (opacity * (1.0f - opacity));
            gs[0] = o.v_scale[0] * scale.x; gs[1] = o.v_scale[1] * scale.y; gs[2] = o.v_scale[2] * scale.z;
            const float dq = o.v_quat[0] * q[0] + o.v_quat[1] * q[1] + o.v_quat[2] * q[2] + o.v_quat[3] * q[3];
#pragma unroll
            for (int k = 0; k < 4; ++k) gq[k] = (o.v_quat[k] - q[k] * dq) / nrm;
#pragma unroll
            for (int k = 0; k < 3; ++k) gm[k] = o.v_mean[k];
            // colour clamp mask, then SH backward
            vc[0] = r3.x <= 0.f ? 0.f : o.v_rgb[0];
            vc[1] = r3.y <= 0.f ? 0.f : o.v_rgb[1];
            vc[2] = r3.z <= 0.f ? 0.f : o.v_rgb[2];
            sh_basis(sh_degree, mean.x - cam.campos[0], mean.y - cam.campos[1], mean.z - cam.campos[2], B);
#pragma unroll
            for (int k = 0; k < 3; ++k) g0[k] = B[0] * vc[k];
        }
        if (g_shN && sh_factors) {
            // the two factors of the rank-1 rows instead of the rows: [N,6] = (clamped colour gradient, unit view direction)
            // at the start of the shN gradient tensor, for the data-parallel exchange that sums the outer products
            if (in_range) {
                float dx = 0.f, dy = 0.f, dz = 0.f;
                if (visible) {
                    dx = m_in[0] - cam.campos[0]; dy = m_in[1] - cam.campos[1]; dz = m_in[2] - cam.campos[2];
                    const float inorm = rsqrtf(dx * dx + dy * dy + dz * dz);
                    dx *= inorm; dy *= inorm; dz *= inorm;
                }
                // ADAM: the factors go into the Gaussian's own (now consumed) row of 16 sums
                float2* f = ADAM ? reinterpret_cast<float2*>(g_shN) + (size_t)g * 8 : reinterpret_cast<float2*>(g_shN) + (size_t)g * 3;
                f[0] = make_float2(vc[0], vc[1]); f[1] = make_float2(vc[2], dx); f[2] = make_float2(dy, dz);
            }
        } else if (g_shN) {  // NULL: the caller forms these rows itself from the sh0 gradient (adam_sh_rank1_kernel)
            for (int k = 1; k < K; ++k) {
                const float w = k < nb ? B[k] : 0.f;
#pragma unroll
                for (int c = 0; c < 3; ++c) my[lane * rest + (k - 1) * 3 + c] = w * vc[c];
            }
            __syncwarp();
            const int n_rows = min(32, N - chunk * 32);
            const int total = n_rows * rest;
            float* dst = g_shN + (size_t)chunk * 32 * rest;
            if (accumulate) {
                if (__any_sync(0xffffffffu, visible))
                    for (int i = lane; i < total; i += 32) dst[i] += my[i];
            } else {
                for (int i = lane; i < total; i += 32) dst[i] = my[i];
            }
            __syncwarp();
        }
        if (ADAM) {
            if (in_range) {
                const float c_in[3] = {sh0[g * 3], sh0[g * 3 + 1], sh0[g * 3 + 2]};
                const float q_in[4] = {qr.x, qr.y, qr.z, qr.w};
                adam_small_row<3>(A, 0, (size_t)g, m_in, gm);
                adam_small_row<3>(A, 1, (size_t)g, c_in, g0);
                adam_small_row<3>(A, 2, (size_t)g, s_in, gs);
                adam_small_row<4>(A, 3, (size_t)g, q_in, gq);
                adam_small_row<1>(A, 4, (size_t)g, &o_in, &go);
            }
        } else if (in_range && (visible || !accumulate)) {
            if (accumulate) {
#pragma unroll
                for (int k = 0; k < 3; ++k) { g_means[g * 3 + k] += gm[k]; g_sh0[g * 3 + k] += g0[k]; g_scaling[g * 3 + k] += gs[k]; }
#pragma unroll
                for (int k = 0; k < 4; ++k) g_rotation[g * 4 + k] += gq[k];
                g_opacity[g] += go;
            } else {
#pragma unroll
                for (int k = 0; k < 3; ++k) { g_means[g * 3 + k] = gm[k]; g_sh0[g * 3 + k] = g0[k]; g_scaling[g * 3 + k] = gs[k]; }
                reinterpret_cast<float4*>(g_rotation)[g] = make_float4(gq[0], gq[1], gq[2], gq[3]);
                g_opacity[g] = go;
            }
        }
    }
}

// Adam on the higher-order SH coefficients without a gradient tensor. For one camera the gradient row of a Gaussian
// is the outer product of the SH basis of its view direction with the clamped colour gradient vc, and the sh0
// gradient already holds Y00 * vc; so the rows are rebuilt here, 32 Gaussians per warp in shared memory, and the
// parameter / moment rows (one contiguous run per warp) are streamed through once, 16 bytes per lane and U vectors of
// each tensor in flight. Same update arithmetic as the optimizer kernels.
__device__ __forceinline__ void adam_rank1_update(float& p, float& m, float& v, float g, const AdamRank1& A) {
    const float m1 = A.beta1 * m + (1.0f - A.beta1) * g;
    const float m2 = A.beta2 * v + (1.0f - A.beta2) * g * g;
    const float denom = sqrtf(m2) * A.bc2_sqrt_rcp + A.eps;
    p -= A.step_size * m1 / denom;
    m = m1;
    v = m2;
}
// KT: the number of SH coefficients when known at compile time (16 = degree 3, the training default; the row loop
// then unrolls and the basis stays in registers), 0 = generic.
template <int KT>
__global__ void __launch_bounds__(256, 4) adam_sh_rank1_kernel(int N, int K_rt, int sh_degree, const float* __restrict__ campos,
                                                               const float* __restrict__ means, const float* __restrict__ g_sh0,
                                                               const float* __restrict__ factors, int factor_stride, AdamRank1 A) {
    extern __shared__ __align__(16) float s_rows[];
    constexpr int U = 3;
    const int K = KT ? KT : K_rt;
    float cx = 0.f, cy = 0.f, cz = 0.f;
    if (!factors) { cx = campos[0]; cy = campos[1]; cz = campos[2]; }
    const int rest = (K - 1) * 3;
    const int nb = (sh_degree + 1) * (sh_degree + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my = s_rows + (size_t)warp * 32 * rest;
    const int n_chunks = (N + 31) / 32;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int chunk = blockIdx.x * (blockDim.x >> 5) + warp; chunk < n_chunks; chunk += warps_total) {
        const int g = chunk * 32 + lane;
        float vc[3] = {0.f, 0.f, 0.f}, dir[3] = {0.f, 0.f, 0.f};
        if (g < N) {
            if (factors) {
                // written by the gradient stage: (clamped colour gradient, unit view direction)
                const float2* f = reinterpret_cast<const float2*>(factors + (size_t)g * factor_stride);
                const float2 f0 = f[0], f1 = f[1], f2 = f[2];
                vc[0] = f0.x; vc[1] = f0.y; vc[2] = f1.x; dir[0] = f1.y; dir[1] = f2.x; dir[2] = f2.y;
            } else {
#pragma unroll
                for (int c = 0; c < 3; ++c) vc[c] = g_sh0[g * 3 + c] / 0.2820947917738781f;
            }
        }
        float B[25];
#pragma unroll
        for (int k = 0; k < 25; ++k) B[k] = 0.f;
        if (vc[0] != 0.f || vc[1] != 0.f || vc[2] != 0.f) {
            if (!factors) { dir[0] = means[g * 3] - cx; dir[1] = means[g * 3 + 1] - cy; dir[2] = means[g * 3 + 2] - cz; }
            sh_basis(sh_degree, dir[0], dir[1], dir[2], B);
        }
        if (KT) {
#pragma unroll
            for (int k = 1; k < (KT ? KT : 1); ++k) {
                const float w = k < nb ? B[k] : 0.f;
#pragma unroll
                for (int c = 0; c < 3; ++c) my[lane * rest + (k - 1) * 3 + c] = w * vc[c];
            }
        } else {
            for (int k = 1; k < K; ++k) {
                const float w = k < nb ? B[k] : 0.f;
#pragma unroll
                for (int c = 0; c < 3; ++c) my[lane * rest + (k - 1) * 3 + c] = w * vc[c];
            }
        }
        __syncwarp();
        const int total = min(32, N - chunk * 32) * rest;
        const size_t base = (size_t)chunk * 32 * rest;
        float* __restrict__ pp = A.p + base;
        float* __restrict__ mm = A.m + base;
        float* __restrict__ vv = A.v + base;
        int done = 0;
        if (A.vec) {
            const int total4 = total >> 2;
            float4* __restrict__ p4 = reinterpret_cast<float4*>(pp);
            float4* __restrict__ m4 = reinterpret_cast<float4*>(mm);
            float4* __restrict__ v4 = reinterpret_cast<float4*>(vv);
            const float4* __restrict__ g4 = reinterpret_cast<const float4*>(my);
            for (int i0 = lane; i0 < total4; i0 += 32 * U) {
                float4 p[U], m[U], v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + 32 * u;
                    if (i < total4) { p[u] = p4[i]; m[u] = m4[i]; v[u] = v4[i]; }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + 32 * u;
                    if (i < total4) {
                        const float4 gr = g4[i];
                        adam_rank1_update(p[u].x, m[u].x, v[u].x, gr.x * A.grad_scale, A);
                        adam_rank1_update(p[u].y, m[u].y, v[u].y, gr.y * A.grad_scale, A);
                        adam_rank1_update(p[u].z, m[u].z, v[u].z, gr.z * A.grad_scale, A);
                        adam_rank1_update(p[u].w, m[u].w, v[u].w, gr.w * A.grad_scale, A);
                        p4[i] = p[u]; m4[i] = m[u]; v4[i] = v[u];
                    }
                }
            }
            done = total4 << 2;
        }
        for (int i = done + lane; i < total; i += 32) {
            float p = pp[i], m = mm[i], v = vv[i];
            adam_rank1_update(p, m, v, my[i] * A.grad_scale, A);
            pp[i] = p; mm[i] = m; vv[i] = v;
        }
        __syncwarp();
    }
}

// Data-parallel form of adam_sh_rank1_kernel: this rank owns the elements [lo, lo + n) of the shN tensor. For the rows
// that intersect them, the gradient row is the sum over ranks of (SH basis of that rank's view direction) x (that
// rank's clamped colour gradient), both read from the rank's factor buffer [N,6] through its peer pointer (24 bytes per
// row and rank instead of the 12 (K-1) bytes of a materialised row); then Adam with the shard-local moments and 16-byte
// stores of the new coefficients into every rank's parameter buffer (plain peer stores, or one multimem.st through the
// NVSwitch multicast address of the tensor). Plain peer loads; the caller orders the launch against the other ranks.
template <int KT>
__global__ void __launch_bounds__(256) dp_sh_rank1_kernel(int K_rt, int sh_degree, DpRank1 A) {
    extern __shared__ __align__(16) float s_rows[];
    constexpr int U = 2;
    constexpr int kPre = 4;
    const int K = KT ? KT : K_rt;
    const int rest = (K - 1) * 3;
    const int nb = (sh_degree + 1) * (sh_degree + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my = s_rows + (size_t)warp * 32 * rest;
    const int64_t hi = A.lo + A.n;
    const int64_t chunk_elems = (int64_t)32 * rest;
    const int64_t first_chunk = A.lo / chunk_elems, last_chunk = (hi - 1) / chunk_elems;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int64_t chunk = first_chunk + blockIdx.x * (blockDim.x >> 5) + warp; chunk <= last_chunk; chunk += warps_total) {
        const int64_t g = chunk * 32 + lane;
        for (int j = 0; j < rest; ++j) my[lane * rest + j] = 0.f;
        if (g < A.N) {
            // kPre ranks' factors are in flight at a time (a peer load takes microseconds)
            for (int r0 = 0; r0 < A.world; r0 += kPre) {
                float2 F[kPre][3];
#pragma unroll
                for (int q = 0; q < kPre; ++q) {
                    if (r0 + q < A.world) {
                        const float2* f = reinterpret_cast<const float2*>(A.factors[r0 + q]) + g * 3;
                        F[q][0] = f[0]; F[q][1] = f[1]; F[q][2] = f[2];
                    } else {
                        F[q][0] = F[q][1] = F[q][2] = make_float2(0.f, 0.f);
                    }
                }
#pragma unroll
                for (int q = 0; q < kPre; ++q) {
                    const float vc[3] = {F[q][0].x, F[q][0].y, F[q][1].x};
                    if (vc[0] == 0.f && vc[1] == 0.f && vc[2] == 0.f) continue;
                    float B[25];
#pragma unroll
                    for (int k = 0; k < 25; ++k) B[k] = 0.f;
                    sh_basis(sh_degree, F[q][1].y, F[q][2].x, F[q][2].y, B);
                    if (KT) {
#pragma unroll
                        for (int k = 1; k < (KT ? KT : 1); ++k) {
                            const float w = k < nb ? B[k] : 0.f;
#pragma unroll
                            for (int c = 0; c < 3; ++c) my[lane * rest + (k - 1) * 3 + c] += w * vc[c];
                        }
                    } else {
                        for (int k = 1; k < K; ++k) {
                            const float w = k < nb ? B[k] : 0.f;
#pragma unroll
                            for (int c = 0; c < 3; ++c) my[lane * rest + (k - 1) * 3 + c] += w * vc[c];
                        }
                    }
                }
            }
        }
        __syncwarp();
        const int64_t c0 = chunk * chunk_elems;
        const int64_t e0 = max(A.lo, c0), e1 = min(hi, c0 + chunk_elems);
        const int total = (int)(e1 - e0);
        const float* __restrict__ grad = my + (e0 - c0);
        const float* __restrict__ pp = A.shN[0] + e0;   // every rank holds the same coefficients; read the local copy
        float* __restrict__ mm = A.m + (e0 - A.lo);
        float* __restrict__ vv = A.v + (e0 - A.lo);
        int done = 0;
        if (A.vec) {
            const int total4 = total >> 2;
            const float4* __restrict__ p4 = reinterpret_cast<const float4*>(pp);
            float4* __restrict__ m4 = reinterpret_cast<float4*>(mm);
            float4* __restrict__ v4 = reinterpret_cast<float4*>(vv);
            const float4* __restrict__ g4 = reinterpret_cast<const float4*>(grad);
            for (int i0 = lane; i0 < total4; i0 += 32 * U) {
                float4 p[U], m[U], v[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + 32 * u;
                    if (i < total4) { p[u] = p4[i]; m[u] = m4[i]; v[u] = v4[i]; }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int i = i0 + 32 * u;
                    if (i < total4) {
                        const float4 gr = g4[i];
                        adam_rank1_update(p[u].x, m[u].x, v[u].x, gr.x * A.adam.grad_scale, A.adam);
                        adam_rank1_update(p[u].y, m[u].y, v[u].y, gr.y * A.adam.grad_scale, A.adam);
                        adam_rank1_update(p[u].z, m[u].z, v[u].z, gr.z * A.adam.grad_scale, A.adam);
                        adam_rank1_update(p[u].w, m[u].w, v[u].w, gr.w * A.adam.grad_scale, A.adam);
                        m4[i] = m[u]; v4[i] = v[u];
                        if (A.mc_shN) {
                            multimem_st4(A.mc_shN + e0 + 4 * (int64_t)i, p[u]);
                        } else {
                            for (int r = 0; r < A.world; ++r) reinterpret_cast<float4*>(A.shN[r] + e0)[i] = p[u];
                        }
                    }
                }
            }
            done = total4 << 2;
        }
        for (int i = done + lane; i < total; i += 32) {
            float p = pp[i], m = mm[i], v = vv[i];
            adam_rank1_update(p, m, v, grad[i] * A.adam.grad_scale, A.adam);
            mm[i] = m; vv[i] = v;
            if (A.mc_shN) {
                multimem_st1(A.mc_shN + e0 + i, p);
            } else {
                for (int r = 0; r < A.world; ++r) A.shN[r][e0 + i] = p;
            }
        }
        __syncwarp();
    }
}

}  // namespace

int launch_raster_fwd(const RasterArgs& a, float* render, float* alphas, int32_t* last_ids, float* extra_sum, cudaStream_t st) {
    const int n_tiles = a.tw * a.th;
    if (n_tiles == 0) return LFS_OK;
    if (a.channels != 1 && a.channels != 3 && a.channels != 4) { set_error("raster_fwd: channels must be 1, 3 or 4"); return LFS_EINVAL; }
    LFS_TIMED("raster_fwd", st);
#define LFS_FWD3(MODEL, EXTRA, RS)                                                                                         \
    raster_fwd_kernel<MODEL, EXTRA, RS><<<n_tiles, kBlock, 0, st>>>(a.cam, a.records, a.bounds, a.flatten_ids, a.tile_offsets,   \
                                                                    a.n_isects_dev, a.n_isects_host, a.overflow, a.background,  \
                                                                    a.masks, a.tile_order, a.channels, a.normalize, a.W, a.H,   \
                                                                    a.tw, n_tiles, render, alphas, last_ids, extra_sum)
#define LFS_FWD(MODEL, EXTRA) do { if (a.rolling) LFS_FWD3(MODEL, EXTRA, true); else LFS_FWD3(MODEL, EXTRA, false); } while (0)
    const bool extra = a.channels != 3;
    if (a.model == LFS_PINHOLE) { if (extra) LFS_FWD(LFS_PINHOLE, true); else LFS_FWD(LFS_PINHOLE, false); }
    else if (a.model == LFS_PINHOLE_OPENCV) { if (extra) LFS_FWD(LFS_PINHOLE_OPENCV, true); else LFS_FWD(LFS_PINHOLE_OPENCV, false); }
    else if (a.model == LFS_EQUIRECTANGULAR) { if (extra) LFS_FWD3(LFS_EQUIRECTANGULAR, true, false); else LFS_FWD3(LFS_EQUIRECTANGULAR, false, false); }
    else { if (extra) LFS_FWD(LFS_FISHEYE, true); else LFS_FWD(LFS_FISHEYE, false); }
#undef LFS_FWD3
#undef LFS_FWD
    return check_launch("raster_fwd");
}

int launch_raster_bwd(const RasterArgs& a, const float* render_alphas, const int32_t* last_ids, const float* extra_sum,
                      const float* v_render, const float* v_alphas, float* accum, float* accum_extra, cudaStream_t st) {
    const int n_tiles = a.tw * a.th;
    if (n_tiles == 0) return LFS_OK;
    if (a.channels != 1 && a.channels != 3 && a.channels != 4) { set_error("raster_bwd: channels must be 1, 3 or 4"); return LFS_EINVAL; }
    if (a.normalize && !extra_sum) { set_error("raster_bwd: expected-depth modes need the forward's blended sum"); return LFS_EINVAL; }
    LFS_TIMED("raster_bwd", st);
#ifndef LFS_BWD_BATCH
#define LFS_BWD_BATCH 64
#endif
    constexpr int kBwdBatch = LFS_BWD_BATCH;
    const size_t smem = sizeof(BwdShared<kBwdBatch>);
    static bool attr_set = false;
#define LFS_BWD_ATTR(MODEL, EXTRA, XGRAD)                                                                                     \
    cudaFuncSetAttribute(raster_bwd_kernel<MODEL, kBwdBatch, EXTRA, XGRAD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                         (int)smem);                                                                                           \
    cudaFuncSetAttribute(raster_bwd_kernel<MODEL, kBwdBatch, EXTRA, XGRAD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                         (int)smem)
    if (!attr_set) {
        LFS_BWD_ATTR(LFS_PINHOLE, false, false); LFS_BWD_ATTR(LFS_PINHOLE, true, false); LFS_BWD_ATTR(LFS_PINHOLE, true, true);
        LFS_BWD_ATTR(LFS_FISHEYE, false, false); LFS_BWD_ATTR(LFS_FISHEYE, true, false); LFS_BWD_ATTR(LFS_FISHEYE, true, true);
        LFS_BWD_ATTR(LFS_PINHOLE_OPENCV, false, false); LFS_BWD_ATTR(LFS_PINHOLE_OPENCV, true, false);
        LFS_BWD_ATTR(LFS_PINHOLE_OPENCV, true, true);
        LFS_BWD_ATTR(LFS_EQUIRECTANGULAR, false, false); LFS_BWD_ATTR(LFS_EQUIRECTANGULAR, true, false); LFS_BWD_ATTR(LFS_EQUIRECTANGULAR, true, true);
        attr_set = true;
    }
#undef LFS_BWD_ATTR
#define LFS_BWD4(MODEL, EXTRA, XGRAD, RS)                                                                                     \
    raster_bwd_kernel<MODEL, kBwdBatch, EXTRA, XGRAD, RS><<<n_tiles, kBlock, smem, st>>>(                                      \
        a.cam, a.records, a.bounds, a.flatten_ids, a.tile_offsets, a.n_isects_dev, a.n_isects_host, a.overflow, a.background, \
        a.masks, a.tile_order, a.channels, a.normalize, a.W, a.H, a.tw, n_tiles, render_alphas, last_ids, extra_sum, v_render, \
        v_alphas, accum, accum_extra)
#define LFS_BWD(MODEL, EXTRA, XGRAD) do { if (a.rolling) LFS_BWD4(MODEL, EXTRA, XGRAD, true); else LFS_BWD4(MODEL, EXTRA, XGRAD, false); } while (0)
    const bool extra = a.channels != 3, xgrad = extra && accum_extra != nullptr;
    if (a.model == LFS_PINHOLE) {
        if (!extra) LFS_BWD(LFS_PINHOLE, false, false); else if (!xgrad) LFS_BWD(LFS_PINHOLE, true, false); else LFS_BWD(LFS_PINHOLE, true, true);
    } else if (a.model == LFS_PINHOLE_OPENCV) {
        if (!extra) LFS_BWD(LFS_PINHOLE_OPENCV, false, false); else if (!xgrad) LFS_BWD(LFS_PINHOLE_OPENCV, true, false);
        else LFS_BWD(LFS_PINHOLE_OPENCV, true, true);
    } else if (a.model == LFS_EQUIRECTANGULAR) {
        if (!extra) LFS_BWD4(LFS_EQUIRECTANGULAR, false, false, false); else if (!xgrad) LFS_BWD4(LFS_EQUIRECTANGULAR, true, false, false);
        else LFS_BWD4(LFS_EQUIRECTANGULAR, true, true, false);
    } else {
        if (!extra) LFS_BWD(LFS_FISHEYE, false, false); else if (!xgrad) LFS_BWD(LFS_FISHEYE, true, false); else LFS_BWD(LFS_FISHEYE, true, true);
    }
#undef LFS_BWD4
#undef LFS_BWD
    return check_launch("raster_bwd");
}

int launch_grad_epilogue_op(int N, const CamDev* cam, const float* accum, const float* means, const float* quats,
                            const float* scales, int channels, const float* accum_extra, float* v_means, float* v_quats,
                            float* v_scales, float* v_colors, float* v_opacities, cudaStream_t st) {
    if (N == 0) return LFS_OK;
    LFS_TIMED("grad_epilogue", st);
    grad_epilogue_op_kernel<<<grid_for(N, 256), 256, 0, st>>>(N, cam, accum, means, quats, scales, channels, accum_extra,
                                                              v_means, v_quats, v_scales, v_colors, v_opacities);
    return check_launch("grad_epilogue_op");
}

int launch_grad_epilogue_fused(int N, int K, int sh_degree, const CamDev* cam, const float* accum,
                               const float4* records, const int32_t* radii, const lfs_splats& p, const lfs_splats& g,
                               int accumulate, float scaling_modifier, int sh_factors, cudaStream_t st, const AdamSmall* adam) {
    if (N == 0) return LFS_OK;
    LFS_TIMED(adam ? "grad_epilogue_adam" : "grad_epilogue", st);
    const size_t smem = (size_t)8 * 32 * (K - 1) * 3 * sizeof(float);
    if (smem > 200 * 1024) { set_error("grad_epilogue_fused: too many SH coefficients"); return LFS_EINVAL; }
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(grad_epilogue_fused_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(grad_epilogue_fused_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    if (adam)
        grad_epilogue_fused_kernel<true><<<grid_for(N, 256), 256, smem, st>>>(
            N, K, sh_degree, cam, accum, records, radii, p.means, p.sh0, p.scaling_raw, p.rotation_raw, p.opacity_raw, nullptr,
            nullptr, const_cast<float*>(accum), nullptr, nullptr, nullptr, 0, scaling_modifier, 1, *adam);
    else
        grad_epilogue_fused_kernel<false><<<grid_for(N, 256), 256, smem, st>>>(
            N, K, sh_degree, cam, accum, records, radii, p.means, p.sh0, p.scaling_raw, p.rotation_raw, p.opacity_raw, g.means,
            g.sh0, g.shN, g.scaling_raw, g.rotation_raw, g.opacity_raw, accumulate, scaling_modifier, sh_factors, AdamSmall{});
    return check_launch("grad_epilogue_fused");
}

int launch_adam_sh_rank1(int N, int K, int sh_degree, const float* campos, const float* means, const float* g_sh0, float* p,
                         float* m, float* v, float step_size, float beta1, float beta2, float eps, float bc2_sqrt_rcp,
                         float grad_scale, cudaStream_t st, const float* factors, int factor_stride) {
    if (N == 0 || K <= 1) return LFS_OK;
    LFS_TIMED("adam_sh_rank1", st);
    const size_t smem = (size_t)8 * 32 * (K - 1) * 3 * sizeof(float);
    if (smem > 200 * 1024) { set_error("adam_sh_rank1: too many SH coefficients"); return LFS_EINVAL; }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(adam_sh_rank1_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    AdamRank1 A{p, m, v, step_size, beta1, beta2, eps, bc2_sqrt_rcp, grad_scale,
                (int)(((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) == 0)};
    if (K == 16) adam_sh_rank1_kernel<16><<<grid_for(N, 256), 256, smem, st>>>(N, K, sh_degree, campos, means, g_sh0, factors, factor_stride, A);
    else adam_sh_rank1_kernel<0><<<grid_for(N, 256), 256, smem, st>>>(N, K, sh_degree, campos, means, g_sh0, factors, factor_stride, A);
    return check_launch("adam_sh_rank1");
}

int launch_dp_sh_rank1(int K, int sh_degree, const DpRank1& A, int ctas_per_sm, cudaStream_t st) {
    if (A.n == 0 || K <= 1) return LFS_OK;
    LFS_TIMED("dp_exchange_side_sh_rank1", st);
    const size_t smem = (size_t)8 * 32 * (K - 1) * 3 * sizeof(float);
    if (smem > 200 * 1024) { set_error("dp_sh_rank1: too many SH coefficients"); return LFS_EINVAL; }
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(dp_sh_rank1_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int64_t chunks = (A.lo + A.n - 1) / (32 * (K - 1) * 3) - A.lo / (32 * (K - 1) * 3) + 1;
    const int grid = grid_for(chunks * 32, 256, ctas_per_sm > 0 ? ctas_per_sm : 4);
    if (K == 16) dp_sh_rank1_kernel<16><<<grid, 256, smem, st>>>(K, sh_degree, A);
    else dp_sh_rank1_kernel<0><<<grid, 256, smem, st>>>(K, sh_degree, A);
    return check_launch("dp_sh_rank1");
}

}  // namespace lfs
