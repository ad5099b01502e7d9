// Blend stage of the EWA (default, non --gut) rasterizer and its per-Gaussian gradient stage.
//
// Replaces blend_cu (src/training/fastgs/rasterization/include/kernels_forward.cuh:336-459), blend_backward_cu
// (include/kernels_backward.cuh:236-448), preprocess_backward_cu (:19-233) and the background blend of
// src/training/rasterization/fast_rasterizer.cpp:67.
//
// Design: one CTA per 16x16 tile, one thread per pixel, warps cover 8x4 pixel patches. The tile's depth-sorted
// Gaussians are staged in shared memory as packed 48-byte records by 16-byte asynchronous copies, double buffered.
// Each warp first tests 32 staged entries at a time against its own patch with the same ellipse-versus-rectangle
// test that built the tile lists, and then walks only the entries that can reach it. The backward walks the lists
// from each pixel's last contributor to the front (transmittance is recovered by division, so no per-bucket state
// is stored by the forward, unlike the reference) and reduces the nine per-pair gradient terms per (warp, Gaussian)
// with a halving shuffle butterfly before they leave the CTA as three 16-byte atomic adds per (tile, Gaussian).
#include "ewa.cuh"
#include "ewa_common.cuh"

namespace lfs {
namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void pixel_of_thread(int tile, int tw, int& i, int& j) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    j = (tile % tw) * 16 + (warp & 1) * 8 + (lane & 7);
    i = (tile / tw) * 16 + (warp >> 1) * 4 + (lane >> 3);
}

// Stage `count` entries whose list positions are first, first + step, ... into rec[0 .. 3 * count): every thread
// issues the quarter-records q = k * kBlock + tid (entry q / 3, part q % 3) and records the Gaussian index.
template <int BATCH>
__device__ __forceinline__ void stage_batch(float4* rec, uint32_t* sid, const float4* __restrict__ records,
                                            const uint32_t* __restrict__ ids, int32_t first, int step, int count) {
    constexpr int kParts = (BATCH * 3 + kBlock - 1) / kBlock;
#pragma unroll
    for (int k = 0; k < kParts; ++k) {
        const int q = k * kBlock + threadIdx.x;
        const int e = q / 3, part = q - e * 3;
        if (e < count) {
            const uint32_t g = ids[first + step * e];
            cp_async16(&rec[q], records + (size_t)g * 3 + part);
            if (sid && part == 0) sid[e] = g;
        }
    }
    cp_async_commit();
}

// one ballot word per 32 staged entries: which of them can reach this warp's patch
template <int BATCH>
__device__ __forceinline__ void cull_batch(const float4* rec, int lo, int hi, float px0, float py0, uint32_t* live) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int w = 0; w < BATCH / 32; ++w) {
        const int e = w * 32 + lane;
        bool ok = false;
        if (e >= lo && e < hi) {
            const float4 r0 = rec[e * 3], r1 = rec[e * 3 + 1], r2 = rec[e * 3 + 2];
            // a small margin on the threshold keeps the test conservative under rounding
            ok = ewa_rect_contributes(r0.x - 0.5f, r0.y - 0.5f, r0.z, r0.w, r1.x, px0, px0 + 7.0f, py0, py0 + 3.0f, r2.z + 0.01f);
        }
        live[w] = __ballot_sync(0xffffffffu, ok);
    }
}

// 48 registers (instead of the 64 the compiler takes unasked) let five CTAs share an SM
__global__ void __launch_bounds__(kBlock, 5) ewa_blend_fwd_kernel(
    const float4* __restrict__ records, const uint32_t* __restrict__ ids, const int32_t* __restrict__ tile_offsets,
    const int32_t* __restrict__ overflow, const float* __restrict__ background, const int32_t* __restrict__ tile_order,
    int W, int H, int tw, float* __restrict__ image, float* __restrict__ alpha_map, int32_t* __restrict__ n_contrib) {
    constexpr int BATCH = 256;
    __shared__ float4 rec[2][BATCH * 3];
    const int tile = tile_order ? tile_order[blockIdx.x] : blockIdx.x;
    int i, j;
    pixel_of_thread(tile, tw, i, j);
    const bool inside = i < H && j < W;
    const bool dead = overflow && *overflow;
    const int32_t range_start = dead ? 0 : tile_offsets[tile];
    const int32_t range_end = dead ? 0 : tile_offsets[tile + 1];
    const int n_batches = (range_end - range_start + BATCH - 1) / BATCH;
    const float px = (float)j + 0.5f, py = (float)i + 0.5f;
    const int warp = threadIdx.x >> 5;
    const float patch_x = (float)((tile % tw) * 16 + (warp & 1) * 8), patch_y = (float)((tile / tw) * 16 + (warp >> 1) * 4);

    float T = 1.0f, cr = 0.f, cg = 0.f, cb_ = 0.f;
    int32_t last = 0;
    bool done = !inside;
    if (n_batches > 0) stage_batch<BATCH>(rec[0], nullptr, records, ids, range_start, 1, min(BATCH, range_end - range_start));
    for (int b = 0; b < n_batches; ++b) {
        const int32_t batch_start = range_start + b * BATCH;
        const int batch_size = min(BATCH, range_end - batch_start);
        if (b + 1 < n_batches) {
            stage_batch<BATCH>(rec[(b + 1) & 1], nullptr, records, ids, batch_start + BATCH, 1, min(BATCH, range_end - batch_start - BATCH));
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        if (__syncthreads_count(done) >= kBlock) break;
        const float4* st = rec[b & 1];
        if (!__all_sync(0xffffffffu, done)) {
            uint32_t live[BATCH / 32];
            cull_batch<BATCH>(st, 0, batch_size, patch_x, patch_y, live);
#pragma unroll
            for (int w = 0; w < BATCH / 32; ++w) {
                uint32_t bits = live[w];
                while (bits && !done) {
                    const int t = w * 32 + __ffs(bits) - 1;
                    bits &= bits - 1;
                    const float4 r0 = st[t * 3], r1 = st[t * 3 + 1];
                    const float dx = r0.x - px, dy = r0.y - py;
                    const float sigma = 0.5f * (r0.z * dx * dx + r1.x * dy * dy) + r0.w * dx * dy;
                    if (sigma < 0.0f) continue;
                    const float a = fminf(r1.y * __expf(-sigma), kEwaMaxAlpha);
                    if (a < kEwaMinAlpha) continue;
                    const float nT = T * (1.0f - a);
                    if (nT < kEwaMinTransmittance) { done = true; break; }
                    const float wgt = T * a;
                    cr += wgt * r1.z; cg += wgt * r1.w; cb_ += wgt * st[t * 3 + 2].x;
                    T = nT;
                    last = batch_start - range_start + t + 1;
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (inside) {
        const size_t pid = (size_t)i * W + j, np = (size_t)W * H;
        if (background) { cr += T * background[0]; cg += T * background[1]; cb_ += T * background[2]; }
        image[pid] = cr;
        image[np + pid] = cg;
        image[2 * np + pid] = cb_;
        alpha_map[pid] = 1.0f - T;
        n_contrib[pid] = last;
    }
}

// 9 values per lane -> per-value sums over the warp, value k left in lanes 2k and 2k+1 (lanes 18..31 repeat value 8).
// The transpose goes through shared memory owned by the warp instead of a shuffle butterfly: row k (36 floats, 32 used)
// holds value k of the 32 lanes. The row stride of 36 floats puts the 16-byte loads of one quarter-warp (lane = 2 k + h
// reads the 16 lanes of half h of row k) on eight different bank groups, and the scalar stores of one row are contiguous.
// The closing shuffle needs every lane's sum, hence every lane's loads, before any lane returns, so the next call may
// overwrite the rows.
constexpr int kRedStride = 36;
__device__ __forceinline__ float warp_reduce9(const float (&v)[9], float* __restrict__ red, int lane) {
#pragma unroll
    for (int k = 0; k < 9; ++k) red[k * kRedStride + lane] = v[k];
    __syncwarp();
    const int k = min(lane >> 1, 8), h = lane & 1;
    const float4* half = reinterpret_cast<const float4*>(red + k * kRedStride + 16 * h);
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 x = half[q];
        s += (x.x + x.y) + (x.z + x.w);
    }
    return s + __shfl_xor_sync(0xffffffffu, s, 1);
}

__global__ void __launch_bounds__(kBlock, 4) ewa_blend_bwd_kernel(
    const float4* __restrict__ records, const uint32_t* __restrict__ ids, const int32_t* __restrict__ tile_offsets,
    const int32_t* __restrict__ overflow, const float* __restrict__ background, const int32_t* __restrict__ tile_order,
    int W, int H, int tw, const float* __restrict__ alpha_map, const int32_t* __restrict__ n_contrib,
    const float* __restrict__ grad_image,
    const float* __restrict__ grad_alpha, float* __restrict__ accum) {
    constexpr int BATCH = 128;
    __shared__ float4 rec[2][BATCH * 3];
    __shared__ uint32_t sid[3][BATCH];                  // three deep: batch b+1 is staged while batch b-1 is flushed
    __shared__ __align__(16) float sacc_all[2][BATCH * 12];
    __shared__ int stouched_all[2][BATCH];
    __shared__ __align__(16) float red_all[kBlock / 32][9 * kRedStride];  // per-warp transpose rows of warp_reduce9
    if (overflow && *overflow) return;
    const int tile = tile_order ? tile_order[blockIdx.x] : blockIdx.x;
    int i, j;
    pixel_of_thread(tile, tw, i, j);
    const bool inside = i < H && j < W;
    const size_t pid = inside ? (size_t)i * W + j : 0, np = (size_t)W * H;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float px = (float)j + 0.5f, py = (float)i + 0.5f;
    const float patch_x = (float)((tile % tw) * 16 + (warp & 1) * 8), patch_y = (float)((tile / tw) * 16 + (warp >> 1) * 4);
    const int32_t range_start = tile_offsets[tile];

    const float gr = inside ? grad_image[pid] : 0.f, gg = inside ? grad_image[np + pid] : 0.f, gb = inside ? grad_image[2 * np + pid] : 0.f;
    const float T_final = inside ? 1.0f - alpha_map[pid] : 1.0f;
    float ga = (inside && grad_alpha) ? grad_alpha[pid] : 0.f;
    if (background) ga -= gr * background[0] + gg * background[1] + gb * background[2];  // image = blend + (1 - alpha) bg
    const float ga_common = ga * T_final;
    const int32_t my_last = inside ? n_contrib[pid] : 0;  // entries at list positions < my_last can contribute
    // the tile is walked from its deepest contributor to the front
    int32_t tile_last = __reduce_max_sync(0xffffffffu, my_last);
    __shared__ int32_t s_last[kBlock / 32];
    if (lane == 0) s_last[warp] = tile_last;
    for (int e = threadIdx.x; e < 2 * BATCH; e += kBlock) {
#pragma unroll
        for (int k = 0; k < 12; ++k) (&sacc_all[0][0])[e * 12 + k] = 0.f;
        (&stouched_all[0][0])[e] = 0;
    }
    __syncthreads();
    const int32_t warp_last = tile_last;
    tile_last = 0;
#pragma unroll
    for (int w = 0; w < kBlock / 32; ++w) tile_last = max(tile_last, s_last[w]);
    const int n_batches = (tile_last + BATCH - 1) / BATCH;
    const int32_t top = range_start + tile_last - 1;  // list position of the first entry walked

    float T = T_final, ar = 0.f, ag = 0.f, ab = 0.f;
    // flush the sums of batch k (three 16-byte reductions per touched Gaussian) and leave its buffers zeroed
    auto flush = [&](int k) {
        const int size_k = min(BATCH, tile_last - k * BATCH);
        for (int e = threadIdx.x; e < size_k; e += kBlock) {
            if (stouched_all[k & 1][e]) {
                float4* dst = reinterpret_cast<float4*>(accum) + (size_t)sid[k % 3][e] * 3;
                float4* src = reinterpret_cast<float4*>(sacc_all[k & 1]) + e * 3;
#pragma unroll
                for (int q = 0; q < 3; ++q) {
                    atomicAdd(dst + q, src[q]);
                    src[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
                stouched_all[k & 1][e] = 0;
            }
        }
    };
    if (n_batches > 0) stage_batch<BATCH>(rec[0], sid[0], records, ids, top, -1, min(BATCH, tile_last));
    // One barrier per batch: after it, batch b is in shared memory and every warp has finished walking batch b-1,
    // so batch b+1 may be staged over b-1's records and b-1's sums may be flushed while batch b is walked.
    for (int b = 0; b < n_batches; ++b) {
        const int32_t batch_top = top - b * BATCH;                    // slot t holds list position batch_top - t
        const int batch_size = min(BATCH, tile_last - b * BATCH);
        cp_async_wait<0>();
        __syncthreads();
        if (b + 1 < n_batches)
            stage_batch<BATCH>(rec[(b + 1) & 1], sid[(b + 1) % 3], records, ids, batch_top - BATCH, -1, min(BATCH, tile_last - (b + 1) * BATCH));
        if (b > 0) flush(b - 1);
        float* sacc = sacc_all[b & 1];
        int* stouched = stouched_all[b & 1];
        const float4* st = rec[b & 1];
        // slots whose tile-local position is at or beyond this warp's deepest contributor are dropped up front
        const int t_begin = max(0, (batch_top - range_start) - (warp_last - 1));
        uint32_t live[BATCH / 32];
        cull_batch<BATCH>(st, t_begin, batch_size, patch_x, patch_y, live);
#pragma unroll
        for (int w = 0; w < BATCH / 32; ++w) {
            uint32_t bits = live[w];
            while (bits) {
                const int t = w * 32 + __ffs(bits) - 1;
                bits &= bits - 1;
                const float4 r0 = st[t * 3], r1 = st[t * 3 + 1];
                const float dx = r0.x - px, dy = r0.y - py;
                const float sigma = 0.5f * (r0.z * dx * dx + r1.x * dy * dy) + r0.w * dx * dy;
                float a = fminf(r1.y * __expf(-sigma), kEwaMaxAlpha);
                const bool valid = inside && (batch_top - range_start - t) < my_last && !(sigma < 0.0f) && !(a < kEwaMinAlpha);
                if (!__any_sync(0xffffffffu, valid)) continue;
                if (!valid) a = 0.f;  // every term below is then exactly zero for this lane
                const float blue = st[t * 3 + 2].x;
                const float rcp = __frcp_rn(1.0f - a);
                T *= rcp;  // transmittance in front of this entry
                const float wgt = T * a;
                const float dL_da = ga_common * rcp + (T * r1.z - ar * rcp) * gr + (T * r1.w - ag * rcp) * gg + (T * blue - ab * rcp) * gb;
                ar += wgt * r1.z; ag += wgt * r1.w; ab += wgt * blue;
                const float h = -a * dL_da;
                float v[9];
                v[0] = h * (r0.z * dx + r0.w * dy);
                v[1] = h * (r0.w * dx + r1.x * dy);
                v[2] = 0.5f * h * dx * dx;
                v[3] = 0.5f * h * dx * dy;
                v[4] = 0.5f * h * dy * dy;
                v[5] = a * dL_da;
                v[6] = wgt * gr;
                v[7] = wgt * gg;
                v[8] = wgt * gb;
                const float total = warp_reduce9(v, red_all[warp], lane);
                if ((lane & 1) == 0 && lane < 18) atomicAdd(&sacc[t * 12 + (lane >> 1)], total);
                if (lane == 0) stouched[t] = 1;
            }
        }
    }
    __syncthreads();
    if (n_batches > 0) flush(n_batches - 1);
    cp_async_wait<0>();
}

// ---------------------------------------------------------------------------------------------
// Per-Gaussian gradient stage: from (d mean2d, d conic, sum alpha dL/dalpha, d colour) to the six raw tensors.
// cov2d = A Sigma A^T + 0.3 I with A = J W (2x3), Sigma = R diag(exp(2 s)) R^T, conic = cov2d^-1.
// ---------------------------------------------------------------------------------------------
// Each warp handles 32 consecutive Gaussians per iteration: their shN rows ((K-1)*3 floats each, contiguous in
// memory) are read as one coalesced run into shared memory, every lane then works on its own row in place
// (coefficient in, gradient out), and the 32 gradient rows leave as one coalesced run.
// capped at 64 registers (the compiler takes 114 unasked): this stage is latency bound and wants the fourth resident CTA
// W2C: also the camera-pose gradient of kernels_backward.cuh:160-173, sum over the Gaussians that reached a tile of
// (gradient of the camera-space mean) x (mean, 1), rows 0..2 of a [4,4] matrix: per warp a shuffle reduction, per CTA 12
// shared sums, 12 atomics per CTA at the end. A separate instantiation, so the default one keeps its registers.
template <bool W2C>
__global__ void __launch_bounds__(256, 4) ewa_epilogue_kernel(
    int N, int K, const float* __restrict__ means, const float* __restrict__ shN, const float* __restrict__ scaling_raw,
    const float* __restrict__ rotation_raw, EwaCamera cam, const int32_t* __restrict__ n_touched, const float4* __restrict__ records,
    const float* __restrict__ accum, float* __restrict__ g_means, float* __restrict__ g_sh0, float* __restrict__ g_shN,
    float* __restrict__ g_scaling, float* __restrict__ g_rotation, float* __restrict__ g_opacity, int accumulate,
    float* __restrict__ densification_info, float* __restrict__ grad_w2c) {
    extern __shared__ float s_rows[];
    __shared__ float s_pose[8][12];
    if (W2C) {
        if (threadIdx.x < 96) s_pose[threadIdx.x / 12][threadIdx.x % 12] = 0.f;
        __syncthreads();
    }
    float r1[4], r2[4], r3[4], campos[3];
#pragma unroll
    for (int k = 0; k < 4; ++k) { r1[k] = cam.w2c[k]; r2[k] = cam.w2c[4 + k]; r3[k] = cam.w2c[8 + k]; }
#pragma unroll
    for (int k = 0; k < 3; ++k) campos[k] = cam.campos[k];
    const int rest = (K - 1) * 3;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* my = s_rows + (size_t)warp * 32 * rest;
    const int n_chunks = (N + 31) / 32;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const int nb = cam.active_sh_bases > 9 ? 16 : cam.active_sh_bases > 4 ? 9 : cam.active_sh_bases > 1 ? 4 : 1;
    for (int chunk = blockIdx.x * (blockDim.x >> 5) + warp; chunk < n_chunks; chunk += warps_total) {
        const int i = chunk * 32 + lane;
        const bool in_range = i < N;
        const bool visible = in_range && n_touched[i] > 0;
        const bool any_visible = __any_sync(0xffffffffu, visible);
        const int n_rows = min(32, N - chunk * 32);
        const int total = n_rows * rest;
        float* dst_rows = g_shN + (size_t)chunk * 32 * rest;
        if (!any_visible) {
            // nothing in this chunk reached a tile: zeros (or untouched when accumulating)
            if (!accumulate) {
                if (g_shN) for (int k = lane; k < total; k += 32) dst_rows[k] = 0.f;
                if (in_range) {
#pragma unroll
                    for (int k = 0; k < 3; ++k) { g_means[i * 3 + k] = 0.f; g_sh0[i * 3 + k] = 0.f; g_scaling[i * 3 + k] = 0.f; }
                    reinterpret_cast<float4*>(g_rotation)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    g_opacity[i] = 0.f;
                }
            }
            continue;
        }
        if (nb > 1) {
            const float* src_rows = shN + (size_t)chunk * 32 * rest;
            for (int k = lane; k < total; k += 32) my[k] = src_rows[k];
        }
        __syncwarp();
        float* out_rest = my + lane * rest;   // this lane's row: coefficients now, gradients afterwards
        float gm[3] = {0.f, 0.f, 0.f}, gs[3] = {0.f, 0.f, 0.f}, gq[4] = {0.f, 0.f, 0.f, 0.f}, g0[3] = {0.f, 0.f, 0.f}, go = 0.f;
        float pose[12];
        if (W2C) {
#pragma unroll
            for (int k = 0; k < 12; ++k) pose[k] = 0.f;
        }
        if (!visible) {
            for (int k = 0; k < rest; ++k) out_rest[k] = 0.f;
        } else {
        float acc[12];
        const float4* a4 = reinterpret_cast<const float4*>(accum) + (size_t)i * 3;
#pragma unroll
        for (int k = 0; k < 3; ++k) { const float4 t = a4[k]; acc[k * 4] = t.x; acc[k * 4 + 1] = t.y; acc[k * 4 + 2] = t.z; acc[k * 4 + 3] = t.w; }
        const float4 rc1 = records[(size_t)i * 3 + 1], rc2 = records[(size_t)i * 3 + 2];
        const uint32_t mask = __float_as_uint(rc2.y);
        const float gc[3] = {(mask & 1u) ? acc[6] : 0.f, (mask & 2u) ? acc[7] : 0.f, (mask & 4u) ? acc[8] : 0.f};
        go = acc[5] * (1.0f - rc1.y);
        const float m0 = means[i * 3], m1 = means[i * 3 + 1], m2 = means[i * 3 + 2];
        // ---- colour: SH coefficients and, through the view direction, the mean
#pragma unroll
        for (int ch = 0; ch < 3; ++ch) g0[ch] = 0.28209479177387814f * gc[ch];
        float dmc[3] = {0.f, 0.f, 0.f};
        if (nb > 1) {
            const float xr = m0 - campos[0], yr = m1 - campos[1], zr = m2 - campos[2];
            const float inv = rsqrtf(xr * xr + yr * yr + zr * zr);
            const float x = xr * inv, y = yr * inv, z = zr * inv;
            const float xx = x * x, yy = y * y, zz = z * z, xy = x * y, xz = x * z, yz = y * z;
            const float* co = out_rest;
            float gd[3] = {0.f, 0.f, 0.f};
            // basis value B and its derivative (Dx, Dy, Dz) with respect to the unit direction, one row at a time
            auto row = [&](int k, float B, float Dx, float Dy, float Dz) {
                const float c0 = co[(k - 1) * 3], c1 = co[(k - 1) * 3 + 1], c2 = co[(k - 1) * 3 + 2];
                const float cgd = c0 * gc[0] + c1 * gc[1] + c2 * gc[2];
                gd[0] += Dx * cgd; gd[1] += Dy * cgd; gd[2] += Dz * cgd;
                out_rest[(k - 1) * 3] = B * gc[0]; out_rest[(k - 1) * 3 + 1] = B * gc[1]; out_rest[(k - 1) * 3 + 2] = B * gc[2];
            };
            row(1, -0.48860251190291987f * y, 0.f, -0.48860251190291987f, 0.f);
            row(2, 0.48860251190291987f * z, 0.f, 0.f, 0.48860251190291987f);
            row(3, -0.48860251190291987f * x, -0.48860251190291987f, 0.f, 0.f);
            if (nb > 4) {
                row(4, 1.0925484305920792f * xy, 1.0925484305920792f * y, 1.0925484305920792f * x, 0.f);
                row(5, -1.0925484305920792f * yz, 0.f, -1.0925484305920792f * z, -1.0925484305920792f * y);
                row(6, 0.94617469575755997f * zz - 0.31539156525251999f, 0.f, 0.f, 1.8923493915151202f * z);
                row(7, -1.0925484305920792f * xz, -1.0925484305920792f * z, 0.f, -1.0925484305920792f * x);
                row(8, 0.54627421529603959f * xx - 0.54627421529603959f * yy, 1.0925484305920792f * x, -1.0925484305920792f * y, 0.f);
            }
            if (nb > 9) {
                row(9, 0.59004358992664352f * y * (-3.0f * xx + yy), -3.5402615395598609f * xy, -1.7701307697799304f * xx + 1.7701307697799304f * yy, 0.f);
                row(10, 2.8906114426405538f * xy * z, 2.8906114426405538f * yz, 2.8906114426405538f * xz, 2.8906114426405538f * xy);
                row(11, 0.45704579946446572f * y * (1.0f - 5.0f * zz), 0.f, 0.45704579946446572f - 2.2852289973223288f * zz, -4.5704579946446566f * yz);
                row(12, 0.3731763325901154f * z * (5.0f * zz - 3.0f), 0.f, 0.f, 5.597644988851731f * zz - 1.1195289977703462f);
                row(13, 0.45704579946446572f * x * (1.0f - 5.0f * zz), 0.45704579946446572f - 2.2852289973223288f * zz, 0.f, -4.5704579946446566f * xz);
                row(14, 1.4453057213202769f * z * (xx - yy), 2.8906114426405538f * xz, -2.8906114426405538f * yz, 1.4453057213202769f * xx - 1.4453057213202769f * yy);
                row(15, 0.59004358992664352f * x * (-xx + 3.0f * yy), -1.7701307697799304f * xx + 1.7701307697799304f * yy, 3.5402615395598609f * xy, 0.f);
            }
            for (int k = (nb - 1) * 3; k < rest; ++k) out_rest[k] = 0.f;
            // through the normalisation: (|r|^2 I - r r^T) gd / |r|^3
            const float xxr = xr * xr, yyr = yr * yr, zzr = zr * zr, xyr = xr * yr, xzr = xr * zr, yzr = yr * zr;
            const float n2 = xxr + yyr + zzr;
            const float s = rsqrtf(n2 * n2 * n2);
            dmc[0] = ((yyr + zzr) * gd[0] - xyr * gd[1] - xzr * gd[2]) * s;
            dmc[1] = (-xyr * gd[0] + (xxr + zzr) * gd[1] - yzr * gd[2]) * s;
            dmc[2] = (-xzr * gd[0] - yzr * gd[1] + (xxr + yyr) * gd[2]) * s;
        } else {
            for (int k = 0; k < rest; ++k) out_rest[k] = 0.f;
        }
        // ---- geometry, recomputed as in the forward
        const float depth = r3[0] * m0 + r3[1] * m1 + r3[2] * m2 + r3[3];
        const float x = (r1[0] * m0 + r1[1] * m1 + r1[2] * m2 + r1[3]) / depth;
        const float y = (r2[0] * m0 + r2[1] * m1 + r2[2] * m2 + r2[3]) / depth;
        const float var[3] = {expf(2.0f * scaling_raw[i * 3]), expf(2.0f * scaling_raw[i * 3 + 1]), expf(2.0f * scaling_raw[i * 3 + 2])};
        const float4 q = reinterpret_cast<const float4*>(rotation_raw)[i];
        const float qr = q.x, qx = q.y, qy = q.z, qz = q.w;
        const float n = qr * qr + qx * qx + qy * qy + qz * qz;
        const float pxx = 2.0f * qx * qx / n, pyy = 2.0f * qy * qy / n, pzz = 2.0f * qz * qz / n;
        const float pxy = 2.0f * qx * qy / n, pxz = 2.0f * qx * qz / n, pyz = 2.0f * qy * qz / n;
        const float prx = 2.0f * qr * qx / n, pry = 2.0f * qr * qy / n, prz = 2.0f * qr * qz / n;
        const float R[9] = {1.0f - (pyy + pzz), pxy - prz, pry + pxz, prz + pxy, 1.0f - (pxx + pzz), pyz - prx, pxz - pry, prx + pyz, 1.0f - (pxx + pyy)};
        float RS[9];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int k = 0; k < 3; ++k) RS[r * 3 + k] = R[r * 3 + k] * var[k];
        auto rowdot = [&](int a, int b) { return RS[a * 3] * R[b * 3] + RS[a * 3 + 1] * R[b * 3 + 1] + RS[a * 3 + 2] * R[b * 3 + 2]; };
        const float Sg[6] = {rowdot(0, 0), rowdot(0, 1), rowdot(0, 2), rowdot(1, 1), rowdot(1, 2), rowdot(2, 2)};
        const float Wf = (float)cam.W, Hf = (float)cam.H;
        const float tx = fminf(fmaxf(x, (-0.15f * Wf - cam.cx) / cam.fx), (1.15f * Wf - cam.cx) / cam.fx);
        const float ty = fminf(fmaxf(y, (-0.15f * Hf - cam.cy) / cam.fy), (1.15f * Hf - cam.cy) / cam.fy);
        const float j11 = cam.fx / depth, j13 = -j11 * tx, j22 = cam.fy / depth, j23 = -j22 * ty;
        float A1[3], A2[3], B1[3], B2[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) { A1[k] = j11 * r1[k] + j13 * r3[k]; A2[k] = j22 * r2[k] + j23 * r3[k]; }
        B1[0] = A1[0] * Sg[0] + A1[1] * Sg[1] + A1[2] * Sg[2];
        B1[1] = A1[0] * Sg[1] + A1[1] * Sg[3] + A1[2] * Sg[4];
        B1[2] = A1[0] * Sg[2] + A1[1] * Sg[4] + A1[2] * Sg[5];
        B2[0] = A2[0] * Sg[0] + A2[1] * Sg[1] + A2[2] * Sg[2];
        B2[1] = A2[0] * Sg[1] + A2[1] * Sg[3] + A2[2] * Sg[4];
        B2[2] = A2[0] * Sg[2] + A2[1] * Sg[4] + A2[2] * Sg[5];
        const float a = (B1[0] * A1[0] + B1[1] * A1[1] + B1[2] * A1[2]) + kEwaDilation;
        const float b = B1[0] * A2[0] + B1[1] * A2[1] + B1[2] * A2[2];
        const float c = (B2[0] * A2[0] + B2[1] * A2[1] + B2[2] * A2[2]) + kEwaDilation;
        const float rcp = 1.0f / (a * c - b * b), rcp2 = rcp * rcp;
        // gradient of conic = cov2d^-1 (symmetric-entry convention: the off-diagonal sum was accumulated with 1/2)
        const float kx = acc[2], ky = acc[3], kz = acc[4];
        const float hx = rcp2 * (2.0f * (b * c) * ky - (c * c) * kx - (b * b) * kz);
        const float hy = rcp2 * ((b * c) * kx - ((a * c) + (b * b)) * ky + (a * b) * kz);
        const float hz = rcp2 * (2.0f * (a * b) * ky - (b * b) * kx - (a * a) * kz);
        // d/d Sigma = A^T H A
        float S[6];
        S[0] = (A1[0] * A1[0]) * hx + 2.0f * (A1[0] * A2[0]) * hy + (A2[0] * A2[0]) * hz;
        S[1] = (A1[0] * A1[1]) * hx + (A1[0] * A2[1] + A1[1] * A2[0]) * hy + (A2[0] * A2[1]) * hz;
        S[2] = (A1[0] * A1[2]) * hx + (A1[0] * A2[2] + A1[2] * A2[0]) * hy + (A2[0] * A2[2]) * hz;
        S[3] = (A1[1] * A1[1]) * hx + 2.0f * (A1[1] * A2[1]) * hy + (A2[1] * A2[1]) * hz;
        S[4] = (A1[1] * A1[2]) * hx + (A1[1] * A2[2] + A1[2] * A2[1]) * hy + (A2[1] * A2[2]) * hz;
        S[5] = (A1[2] * A1[2]) * hx + 2.0f * (A1[2] * A2[2]) * hy + (A2[2] * A2[2]) * hz;
        // d/d A = 2 H (A Sigma), then the four non-constant entries of J
        float dA1[3], dA2[3];
#pragma unroll
        for (int k = 0; k < 3; ++k) { dA1[k] = 2.0f * (B1[k] * hx + B2[k] * hy); dA2[k] = 2.0f * (B1[k] * hy + B2[k] * hz); }
        const float dj11 = r1[0] * dA1[0] + r1[1] * dA1[1] + r1[2] * dA1[2];
        const float dj22 = r2[0] * dA2[0] + r2[1] * dA2[1] + r2[2] * dA2[2];
        const float dj13 = r3[0] * dA1[0] + r3[1] * dA1[1] + r3[2] * dA1[2];
        const float dj23 = r3[0] * dA2[0] + r3[1] * dA2[1] + r3[2] * dA2[2];
        const float m2x = acc[0], m2y = acc[1];
        const float dcx = j11 * (m2x - dj13 / depth), dcy = j22 * (m2y - dj23 / depth);
        const float dcz = -j11 * (x * m2x + (dj11 - 2.0f * tx * dj13) / depth) - j22 * (y * m2y + (dj22 - 2.0f * ty * dj23) / depth);
#pragma unroll
        for (int k = 0; k < 3; ++k) gm[k] = (r1[k] * dcx + r2[k] * dcy + r3[k] * dcz) + dmc[k];
        if (W2C) {
            const float dc[3] = {dcx, dcy, dcz}, mh[4] = {m0, m1, m2, 1.0f};
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int k = 0; k < 4; ++k) pose[r * 4 + k] = dc[r] * mh[k];
        }
        // variances (columns of R) and the log-scale chain
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            const float u = R[k], v = R[3 + k], w = R[6 + k];
            gs[k] = 2.0f * var[k] * (u * u * S[0] + v * v * S[3] + w * w * S[5] + 2.0f * (u * v * S[1] + u * w * S[2] + v * w * S[4]));
        }
        // rotation: d/dR = 2 S (R diag(var)), R is linear in the products p_ab = 2 q_a q_b / |q|^2
        const float Sm[9] = {S[0], S[1], S[2], S[1], S[3], S[4], S[2], S[4], S[5]};
        float dR[9];
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int k = 0; k < 3; ++k) dR[r * 3 + k] = 2.0f * (RS[k] * Sm[r * 3] + RS[3 + k] * Sm[r * 3 + 1] + RS[6 + k] * Sm[r * 3 + 2]);
        const float dxx = -dR[4] - dR[8], dyy = -dR[0] - dR[8], dzz = -dR[0] - dR[4];
        const float dxy = dR[1] + dR[3], dxz = dR[2] + dR[6], dyz = dR[5] + dR[7];
        const float drx = dR[7] - dR[5], dry = dR[2] - dR[6], drz = dR[3] - dR[1];
        const float nh = pxx * dxx + pyy * dyy + pzz * dzz + pxy * dxy + pxz * dxz + pyz * dyz + prx * drx + pry * dry + prz * drz;
        gq[0] = 2.0f * (qx * drx + qy * dry + qz * drz - qr * nh) / n;
        gq[1] = 2.0f * (2.0f * qx * dxx + qy * dxy + qz * dxz + qr * drx - qx * nh) / n;
        gq[2] = 2.0f * (2.0f * qy * dyy + qx * dxy + qz * dyz + qr * dry - qy * nh) / n;
        gq[3] = 2.0f * (2.0f * qz * dzz + qx * dxz + qy * dyz + qr * drz - qz * nh) / n;
        if (densification_info) {
            densification_info[i] += 1.0f;
            const float sx = m2x * (0.5f * Wf), sy = m2y * (0.5f * Hf);
            densification_info[N + i] += sqrtf(sx * sx + sy * sy);
        }
        }  // visible
        __syncwarp();
        if (W2C) {
#pragma unroll
            for (int k = 0; k < 12; ++k) {
                float v = pose[k];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == 0) s_pose[warp][k] += v;
            }
        }
        if (!g_shN) {
            // the caller rebuilds these rows from the sh0 gradient (lfs_ewa_adam_step_rank1_sh)
        } else if (accumulate) {
            for (int k = lane; k < total; k += 32) dst_rows[k] += my[k];
        } else {
            for (int k = lane; k < total; k += 32) dst_rows[k] = my[k];
        }
        __syncwarp();
        if (in_range && (visible || !accumulate)) {
            if (accumulate) {
#pragma unroll
                for (int k = 0; k < 3; ++k) { g_means[i * 3 + k] += gm[k]; g_sh0[i * 3 + k] += g0[k]; g_scaling[i * 3 + k] += gs[k]; }
#pragma unroll
                for (int k = 0; k < 4; ++k) g_rotation[i * 4 + k] += gq[k];
                g_opacity[i] += go;
            } else {
#pragma unroll
                for (int k = 0; k < 3; ++k) { g_means[i * 3 + k] = gm[k]; g_sh0[i * 3 + k] = g0[k]; g_scaling[i * 3 + k] = gs[k]; }
                reinterpret_cast<float4*>(g_rotation)[i] = make_float4(gq[0], gq[1], gq[2], gq[3]);
                g_opacity[i] = go;
            }
        }
    }
    if (W2C) {
        __syncthreads();
        if (threadIdx.x < 12) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += s_pose[w][threadIdx.x];
            if (v != 0.f) atomicAdd(grad_w2c + threadIdx.x, v);
        }
    }
}

}  // namespace

int launch_ewa_blend_fwd(const EwaBlendArgs& a, float* image, float* alpha, int32_t* n_contrib, cudaStream_t st) {
    const int n_tiles = a.tw * a.th;
    if (n_tiles == 0) return LFS_OK;
    LFS_TIMED("ewa_blend_fwd", st);
    ewa_blend_fwd_kernel<<<n_tiles, kBlock, 0, st>>>(a.records, a.instance_ids, a.tile_offsets, a.overflow, a.background, a.tile_order,
                                                     a.W, a.H, a.tw, image, alpha, n_contrib);
    return check_launch("ewa_blend_fwd");
}

int launch_ewa_blend_bwd(const EwaBlendArgs& a, const float* alpha, const int32_t* n_contrib, const float* grad_image,
                         const float* grad_alpha, float* accum, cudaStream_t st) {
    const int n_tiles = a.tw * a.th;
    if (n_tiles == 0) return LFS_OK;
    LFS_TIMED("ewa_blend_bwd", st);
    ewa_blend_bwd_kernel<<<n_tiles, kBlock, 0, st>>>(a.records, a.instance_ids, a.tile_offsets, a.overflow, a.background, a.tile_order,
                                                     a.W, a.H, a.tw, alpha, n_contrib, grad_image, grad_alpha, accum);
    return check_launch("ewa_blend_bwd");
}

int launch_ewa_epilogue(int N, int K, const lfs_splats& p, const EwaCamera& cam, const int32_t* n_touched, const float4* records,
                        const float* accum, const lfs_splats& g, int accumulate, float* densification_info, float* grad_w2c,
                        cudaStream_t st) {
    if (grad_w2c && !accumulate) cudaMemsetAsync(grad_w2c, 0, 16 * sizeof(float), st);
    if (N == 0) return LFS_OK;
    LFS_TIMED("ewa_epilogue", st);
    const size_t smem = (size_t)8 * 32 * (K - 1) * 3 * sizeof(float);
    if (smem > 200 * 1024) { set_error("ewa_epilogue: too many SH coefficients"); return LFS_EINVAL; }
    if (smem > 48 * 1024) {
        cudaFuncSetAttribute(ewa_epilogue_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(ewa_epilogue_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
#define LFS_EWA_EPILOGUE(W2C)                                                                                                       \
    ewa_epilogue_kernel<W2C><<<grid_for(N, 256), 256, smem, st>>>(N, K, p.means, p.shN, p.scaling_raw, p.rotation_raw, cam, n_touched, \
                                                                 records, accum, g.means, g.sh0, g.shN, g.scaling_raw, g.rotation_raw, \
                                                                 g.opacity_raw, accumulate, densification_info, grad_w2c)
    if (grad_w2c) LFS_EWA_EPILOGUE(true); else LFS_EWA_EPILOGUE(false);
#undef LFS_EWA_EPILOGUE
    return check_launch("ewa_epilogue");
}

}  // namespace lfs
