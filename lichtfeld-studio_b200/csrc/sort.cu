// Tile-list construction: prefix sums, a stable LSD radix sort on (uint32 key, uint32 value) pairs,
// instance emission and per-tile offsets.
//
// Replaces gsplat/IntersectTile.cu:24 (second pass), the at::cumsum + CUB DeviceRadixSort::SortPairs
// call of gsplat/Intersect.cpp:75 / gsplat/IntersectTile.cu:290-328, and gsplat/IntersectTile.cu:206.
//
// The reference sorts n_isects 12-byte (int64 key, int32 value) pairs over 32 + tile_bits + cam_bits
// bits. The same order (camera, tile, depth bits, ties by ascending flattened Gaussian index) is
// produced here with far less traffic: the Gaussians are sorted once by their 32 depth bits, the
// instances are emitted in that order, and a stable sort on the (camera, tile) key alone finishes.
// All passes are HBM-bound integer work; nothing here is shaped for tensor cores.
#include "gsmath.cuh"
#include "sort.cuh"
#include "ewa_common.cuh"

namespace lfs {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kItems = 8;
constexpr int kTile = kThreads * kItems;

__device__ __forceinline__ int warp_incl_scan(int v) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) >= o) v += t;
    }
    return v;
}

// Exclusive scan over the block (any multiple of 32 threads up to 1024); returns the block total.
__device__ __forceinline__ int block_excl_scan(int v, int& total, int* smem /*[33]*/) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int incl = warp_incl_scan(v);
    if (lane == 31) smem[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int s = lane < nw ? smem[lane] : 0;
        const int si = warp_incl_scan(s);
        smem[lane] = si - s;
        if (lane == 31) smem[32] = si;
    }
    __syncthreads();
    const int base = smem[warp];
    total = smem[32];
    __syncthreads();
    return base + incl - v;
}

__device__ __forceinline__ int64_t device_count(const int32_t* n_dev, int64_t n_max) {
    if (n_dev == nullptr) return n_max;
    int64_t n = *n_dev;
    if (n > n_max) n = n_max;
    if (n < 0) n = 0;
    return n;
}

// ---- prefix sum -----------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) scan_reduce_kernel(const int32_t* __restrict__ src, const uint32_t* __restrict__ idx,
                                                               int64_t n, int64_t chunk, uint32_t* __restrict__ block_sums) {
    __shared__ int sm[33];
    const int64_t lo = (int64_t)blockIdx.x * chunk, hi = min(n, lo + chunk);
    int s = 0;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) s += idx ? src[idx[i]] : src[i];
    int total;
    block_excl_scan(s, total, sm);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = (uint32_t)total;
}

__global__ void __launch_bounds__(1024) scan_block_sums_kernel(uint32_t* __restrict__ sums, int n, int32_t* __restrict__ total_dev) {
    __shared__ int sm[33];
    __shared__ int carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const int v = i < n ? (int)sums[i] : 0;
        int total;
        const int ex = block_excl_scan(v, total, sm);
        if (i < n) sums[i] = (uint32_t)(carry + ex);
        __syncthreads();
        if (threadIdx.x == 0) carry += total;
        __syncthreads();
    }
    if (threadIdx.x == 0 && total_dev) *total_dev = carry;
}

__global__ void __launch_bounds__(kThreads) scan_apply_kernel(const int32_t* __restrict__ src, const uint32_t* __restrict__ idx,
                                                              int64_t n, int64_t chunk, const uint32_t* __restrict__ block_sums,
                                                              int32_t* __restrict__ out) {
    __shared__ int sm[33];
    const int64_t lo = (int64_t)blockIdx.x * chunk, hi = min(n, lo + chunk);
    int carry = (int)block_sums[blockIdx.x];
    for (int64_t base = lo; base < hi; base += kThreads) {
        const int64_t i = base + threadIdx.x;
        const int v = i < hi ? (idx ? src[idx[i]] : src[i]) : 0;
        int total;
        const int ex = block_excl_scan(v, total, sm);
        if (i < hi) out[i] = carry + ex;
        carry += total;
    }
}

// ---- radix sort -------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) radix_hist_kernel(const uint32_t* __restrict__ keys, const int32_t* n_dev,
                                                              int64_t n_max, int shift, uint32_t mask, int nb,
                                                              uint32_t* __restrict__ hist) {
    __shared__ uint32_t h[256];
    const int64_t n = device_count(n_dev, n_max);
    const int64_t chunk = (n + nb - 1) / nb;
    const int64_t lo = (int64_t)blockIdx.x * chunk, hi = min(n, lo + chunk);
    h[threadIdx.x] = 0;
    __syncthreads();
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) atomicAdd(&h[(keys[i] >> shift) & mask], 1u);
    __syncthreads();
    hist[(size_t)threadIdx.x * nb + blockIdx.x] = h[threadIdx.x];
}

// One CTA per digit: exclusive scan of that digit's per-block counts (row d of the digit-major table)
// and the digit total. The prefix over digits is taken by every scatter CTA from the 256 totals.
__global__ void __launch_bounds__(kThreads) radix_scan_kernel(uint32_t* __restrict__ hist, int nb,
                                                              uint32_t* __restrict__ digit_totals) {
    __shared__ int sm[33];
    uint32_t* row = hist + (size_t)blockIdx.x * nb;
    int carry = 0;
    for (int base = 0; base < nb; base += kThreads) {
        const int i = base + threadIdx.x;
        const int v = i < nb ? (int)row[i] : 0;
        int total;
        const int ex = block_excl_scan(v, total, sm);
        if (i < nb) row[i] = (uint32_t)(carry + ex);
        carry += total;
    }
    if (threadIdx.x == 0) digit_totals[blockIdx.x] = (uint32_t)carry;
}

// Stable scatter of one radix pass. A CTA walks its chunk in tiles of 2048 pairs: every item gets its rank among
// the equal digits of the tile (warp match + per-warp counters), the tile is reordered by digit in shared memory,
// and then consecutive threads write consecutive addresses of each digit's output run, so the global stores are
// contiguous runs instead of 4-byte scatters.
__global__ void __launch_bounds__(kThreads) radix_scatter_kernel(
    const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in, uint32_t* __restrict__ keys_out,
    uint32_t* __restrict__ vals_out, const int32_t* n_dev, int64_t n_max, int shift, uint32_t mask, int nb,
    const uint32_t* __restrict__ hist, const uint32_t* __restrict__ digit_totals) {
    __shared__ uint32_t cnt[kWarps][256];   // per-warp digit counts, then per-warp start inside the tile
    __shared__ uint32_t gbase[256];         // where the next item of digit d from this CTA goes
    __shared__ uint32_t tstart[256];        // start of digit d inside the reordered tile
    __shared__ uint32_t skeys[kTile], svals[kTile];
    __shared__ int sm[33];
    const int64_t n = device_count(n_dev, n_max);
    const int64_t chunk = (n + nb - 1) / nb;
    const int64_t lo = (int64_t)blockIdx.x * chunk, hi = min(n, lo + chunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lt_mask = (1u << lane) - 1u;
    {
        // start of digit d = totals of the smaller digits + this digit's counts in the earlier blocks
        int total;
        const int digit_base = block_excl_scan((int)digit_totals[threadIdx.x], total, sm);
        gbase[threadIdx.x] = (uint32_t)digit_base + hist[(size_t)threadIdx.x * nb + blockIdx.x];
    }
    for (int64_t tile_lo = lo; tile_lo < hi; tile_lo += kTile) {
        const int tile_n = (int)min((int64_t)kTile, hi - tile_lo);
#pragma unroll
        for (int w = 0; w < kWarps; ++w) cnt[w][threadIdx.x] = 0;
        __syncthreads();
        uint32_t key[kItems], val[kItems], rank[kItems];
        const int64_t wbase = tile_lo + (int64_t)warp * (32 * kItems);
#pragma unroll
        for (int r = 0; r < kItems; ++r) {
            const int64_t i = wbase + r * 32 + lane;
            const bool ok = i < hi;
            key[r] = ok ? keys_in[i] : 0u;
            val[r] = ok ? vals_in[i] : 0u;
        }
#pragma unroll
        for (int r = 0; r < kItems; ++r) {
            const int64_t i = wbase + r * 32 + lane;
            const bool ok = i < hi;
            const uint32_t d = ok ? ((key[r] >> shift) & mask) : 0xFFFFFFFFu;
            const uint32_t peers = __match_any_sync(0xffffffffu, d);
            uint32_t prev = 0;
            if (ok) prev = cnt[warp][d];
            __syncwarp();
            if (ok && (peers & lt_mask) == 0) cnt[warp][d] = prev + __popc(peers);
            __syncwarp();
            rank[r] = prev + __popc(peers & lt_mask);
        }
        __syncthreads();
        {
            // digit threadIdx.x: exclusive prefix over the warps and the digit's total in this tile
            uint32_t run = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                const uint32_t c = cnt[w][threadIdx.x];
                cnt[w][threadIdx.x] = run;
                run += c;
            }
            int total;
            const int start = block_excl_scan((int)run, total, sm);  // start of this digit inside the tile
            tstart[threadIdx.x] = (uint32_t)start;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) cnt[w][threadIdx.x] += (uint32_t)start;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kItems; ++r) {
            const int64_t i = wbase + r * 32 + lane;
            if (i < hi) {
                const uint32_t d = (key[r] >> shift) & mask;
                const uint32_t pos = cnt[warp][d] + rank[r];
                skeys[pos] = key[r];
                svals[pos] = val[r];
            }
        }
        __syncthreads();
        // write out: item j of the reordered tile belongs to digit d = digit(skeys[j]) and goes to
        // gbase[d] + (j - tstart[d]); neighbouring j of one digit are neighbouring addresses
#pragma unroll
        for (int r = 0; r < kItems; ++r) {
            const int j = r * kThreads + threadIdx.x;
            if (j < tile_n) {
                const uint32_t k = skeys[j];
                const uint32_t d = (k >> shift) & mask;
                const uint32_t pos = gbase[d] + ((uint32_t)j - tstart[d]);
                keys_out[pos] = k;
                vals_out[pos] = svals[j];
            }
        }
        __syncthreads();
        {
            // advance the global bases by this tile's digit totals
            const uint32_t next = threadIdx.x + 1 < 256 ? tstart[threadIdx.x + 1] : (uint32_t)tile_n;
            gbase[threadIdx.x] += next - tstart[threadIdx.x];
        }
        __syncthreads();
    }
}

// ---- instance emission ----------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads) emit_instances_kernel(
    int64_t total, int N, const uint32_t* __restrict__ order, const int32_t* __restrict__ tiles,
    const int32_t* __restrict__ offs, const float* __restrict__ means2d, const int32_t* __restrict__ radii,
    float tile_size, uint32_t tw, uint32_t th, uint32_t tile_n_bits, int64_t capacity,
    uint32_t* __restrict__ tkeys, uint32_t* __restrict__ tvals, int32_t* __restrict__ overflow) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < total; r += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t idx = order ? order[r] : (uint32_t)r;
        const int nt = tiles[idx];
        if (nt <= 0) continue;
        const int64_t base = offs[r];
        if (base + nt > capacity) {
            if (overflow) atomicExch(overflow, 1);
            continue;
        }
        uint32_t x0, y0, x1, y1;
        tile_rect(means2d[(size_t)idx * 2], means2d[(size_t)idx * 2 + 1], radii[(size_t)idx * 2],
                              radii[(size_t)idx * 2 + 1], tile_size, tw, th, x0, y0, x1, y1);
        const uint32_t cid = idx / (uint32_t)N;
        const uint32_t cenc = cid << tile_n_bits;
        int64_t cur = base;
        for (uint32_t i = y0; i < y1; ++i)
            for (uint32_t j = x0; j < x1; ++j) {
                tkeys[cur] = cenc | (i * tw + j);
                tvals[cur] = idx;
                ++cur;
            }
    }
}

// EWA path: one instance per tile of the bounds rectangle that the ellipse reaches (create_instances_cu,
// src/training/fastgs/rasterization/include/kernels_forward.cuh:205-309), in row-major tile order.
__global__ void __launch_bounds__(kThreads) ewa_emit_instances_kernel(
    int64_t total, const uint32_t* __restrict__ order, const int32_t* __restrict__ tiles, const int32_t* __restrict__ offs,
    const ushort4* __restrict__ ewa_bounds, const float4* __restrict__ rec, uint32_t tw, int64_t capacity,
    uint32_t* __restrict__ tkeys, uint32_t* __restrict__ tvals, int32_t* __restrict__ overflow) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < total; r += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t idx = order ? order[r] : (uint32_t)r;
        const int nt = tiles[idx];
        if (nt <= 0) continue;
        const int64_t base = offs[r];
        if (base + nt > capacity) {
            if (overflow) atomicExch(overflow, 1);
            continue;
        }
        const ushort4 b = ewa_bounds[idx];
        const float4 r0 = rec[(size_t)idx * 3], r1 = rec[(size_t)idx * 3 + 1], r2 = rec[(size_t)idx * 3 + 2];
        int64_t cur = base;
        for (uint32_t ty = b.z; ty < b.w; ++ty)
            for (uint32_t tx = b.x; tx < b.y; ++tx)
                if (ewa_tile_contributes(r0.x - 0.5f, r0.y - 0.5f, r0.z, r0.w, r1.x, tx, ty, r2.z) && cur < base + nt) {
                    tkeys[cur] = ty * tw + tx;
                    tvals[cur] = idx;
                    ++cur;
                }
    }
}

// offsets[t] = first sorted instance whose (camera, tile) id >= t, for t in [0, n_ids]; entry n_ids
// (one past the last tile) holds the instance count. Keys hold (cid << tile_n_bits) | tile.
// When the overflow flag is set the instance list is incomplete (some slots were never written), so
// the keys cannot be trusted: all offsets are zeroed and the rasterizer draws nothing. Ids are clamped to
// n_ids in any case so that no key value can direct a store outside the offsets array.
__global__ void __launch_bounds__(kThreads) tile_offsets_kernel(const uint32_t* __restrict__ tkeys, const int32_t* n_dev,
                                                                int64_t n_max, uint32_t n_tiles, uint32_t tile_n_bits,
                                                                int64_t n_ids, const int32_t* __restrict__ overflow,
                                                                int32_t* __restrict__ offsets) {
    const int64_t n = (overflow && *overflow) ? 0 : device_count(n_dev, n_max);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n == 0) {
        for (int64_t i = tid; i <= n_ids; i += stride) offsets[i] = 0;
        return;
    }
    const uint32_t tmask = (1u << tile_n_bits) - 1u;
    for (int64_t i = tid; i < n; i += stride) {
        const uint32_t k = tkeys[i];
        const int64_t id_curr = min((int64_t)(k >> tile_n_bits) * n_tiles + (k & tmask), n_ids - 1);
        if (i == 0)
            for (int64_t t = 0; t <= id_curr; ++t) offsets[t] = 0;
        if (i == n - 1)
            for (int64_t t = id_curr + 1; t <= n_ids; ++t) offsets[t] = (int32_t)n;
        if (i > 0) {
            const uint32_t kp = tkeys[i - 1];
            if (kp != k) {
                const int64_t id_prev = min((int64_t)(kp >> tile_n_bits) * n_tiles + (kp & tmask), n_ids - 1);
                for (int64_t t = id_prev + 1; t <= id_curr; ++t) offsets[t] = (int32_t)i;
            }
        }
    }
}

// Operator-level output: 64-bit keys (camera | tile | depth bits) and int32 flattened ids.
__global__ void __launch_bounds__(kThreads) compose_isect_ids_kernel(int64_t n, const uint32_t* __restrict__ tkeys,
                                                                     const uint32_t* __restrict__ tvals,
                                                                     const float* __restrict__ depths,
                                                                     int64_t* __restrict__ isect_ids,
                                                                     int32_t* __restrict__ flatten_ids) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t v = tvals[i];
        isect_ids[i] = ((int64_t)tkeys[i] << 32) | (int64_t)__float_as_uint(depths[v]);
        flatten_ids[i] = (int32_t)v;
    }
}

// Operator-level intersect_offset on 64-bit keys.
__global__ void __launch_bounds__(kThreads) isect_offset_kernel(int64_t n, const int64_t* __restrict__ isect_ids, int64_t n_ids,
                                                                uint32_t n_tiles, uint32_t tile_n_bits,
                                                                int32_t* __restrict__ offsets) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (n == 0) {
        for (int64_t i = tid; i < n_ids; i += stride) offsets[i] = 0;
        return;
    }
    const int64_t tmask = ((int64_t)1 << tile_n_bits) - 1;
    for (int64_t i = tid; i < n; i += stride) {
        const int64_t cur = isect_ids[i] >> 32;
        const int64_t id_curr = (cur >> tile_n_bits) * n_tiles + (cur & tmask);
        if (i == 0)
            for (int64_t t = 0; t <= id_curr && t < n_ids; ++t) offsets[t] = 0;
        if (i == n - 1)
            for (int64_t t = id_curr + 1; t < n_ids; ++t) offsets[t] = (int32_t)n;
        if (i > 0) {
            const int64_t prev = isect_ids[i - 1] >> 32;
            if (prev != cur) {
                const int64_t id_prev = (prev >> tile_n_bits) * n_tiles + (prev & tmask);
                for (int64_t t = id_prev + 1; t <= id_curr && t < n_ids; ++t) offsets[t] = (int32_t)i;
            }
        }
    }
}

__global__ void depth_keys_kernel(int64_t total, const float* __restrict__ depths, const int32_t* __restrict__ tiles,
                                  uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        keys[i] = tiles[i] > 0 ? __float_as_uint(depths[i]) : 0xFFFFFFFFu;
        vals[i] = (uint32_t)i;
    }
}

__global__ void total_to_i64_kernel(const int32_t* total, int64_t* out) { *out = (int64_t)*total; }

__global__ void __launch_bounds__(kThreads) sum_i32_kernel(int64_t n, const int32_t* __restrict__ src, unsigned long long* out) {
    long long s = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) s += src[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0 && s) atomicAdd(out, (unsigned long long)s);
}

}  // namespace

size_t sort_scratch_bytes() { return ((size_t)kRadixBlocks * 256 + kScanBlocks + 320) * sizeof(uint32_t); }

int exclusive_scan_gather(const int32_t* src, const uint32_t* idx, int64_t n, int32_t* out, int32_t* total_dev,
                          const SortScratch& s, cudaStream_t st) {
    if (n <= 0) {
        if (total_dev) cudaMemsetAsync(total_dev, 0, sizeof(int32_t), st);
        return LFS_OK;
    }
    int nb = (int)((n + kTile - 1) / kTile);
    nb = min(nb, min(4 * num_sms(), kScanBlocks));
    const int64_t chunk = (n + nb - 1) / nb;
    LFS_TIMED("exclusive_scan", st);
    scan_reduce_kernel<<<nb, kThreads, 0, st>>>(src, idx, n, chunk, s.block_sums);
    scan_block_sums_kernel<<<1, 1024, 0, st>>>(s.block_sums, nb, total_dev);
    scan_apply_kernel<<<nb, kThreads, 0, st>>>(src, idx, n, chunk, s.block_sums, out);
    return check_launch("exclusive_scan");
}

int radix_sort_pairs(uint32_t* keys[2], uint32_t* vals[2], const int32_t* n_dev, int64_t n_max, int key_bits,
                     const SortScratch& s, cudaStream_t st) {
    if (n_max <= 0 || key_bits <= 0) return 0;
    const int passes = (key_bits + 7) / 8;
    const int bits = (key_bits + passes - 1) / passes;
    int nb = (int)((n_max + kTile - 1) / kTile);
    nb = min(nb, min(4 * num_sms(), kRadixBlocks));
    int cur = 0;
    LFS_TIMED(key_bits == 32 ? "radix_sort_depth" : "radix_sort_tile", st);
    for (int p = 0; p < passes; ++p) {
        const int shift = p * bits;
        const int nbits = (shift + bits > key_bits) ? (key_bits - shift) : bits;
        const uint32_t mask = (1u << nbits) - 1u;
        radix_hist_kernel<<<nb, kThreads, 0, st>>>(keys[cur], n_dev, n_max, shift, mask, nb, s.hist);
        radix_scan_kernel<<<256, kThreads, 0, st>>>(s.hist, nb, s.block_sums);
        radix_scatter_kernel<<<nb, kThreads, 0, st>>>(keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], n_dev, n_max,
                                                      shift, mask, nb, s.hist, s.block_sums);
        cur ^= 1;
    }
    if (check_launch("radix_sort") != LFS_OK) return -1;
    return cur;
}

static uint32_t bit_width_u32(uint32_t v) {
    uint32_t b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

int build_tile_lists(const TileListArgs& a, cudaStream_t st) {
    const int64_t total = (int64_t)a.C * a.N;
    const uint32_t n_tiles = (uint32_t)a.tw * a.th;
    const uint32_t tile_n_bits = bit_width_u32(n_tiles);
    const uint32_t cam_n_bits = bit_width_u32((uint32_t)a.C);
    if (tile_n_bits + cam_n_bits > 32) {
        set_error("build_tile_lists: tile and camera ids need more than 32 bits");
        return LFS_EINVAL;
    }
    SortScratch s = a.scratch;
    const uint32_t* order = nullptr;
    if (a.sort) {
        if (!a.keys_ready) {
            depth_keys_kernel<<<grid_for(total, 256), 256, 0, st>>>(total, a.depths, a.tiles, a.gkeys[0], a.gvals[0]);
        }
        uint32_t* k[2] = {a.gkeys[0], a.gkeys[1]};
        uint32_t* v[2] = {a.gvals[0], a.gvals[1]};
        const int sel = radix_sort_pairs(k, v, nullptr, total, 32, s, st);
        if (sel < 0) return LFS_ECUDA;
        order = v[sel];
    }
    int rc = exclusive_scan_gather(a.tiles, order, total, a.offs, a.n_isects_dev, s, st);
    if (rc != LFS_OK) return rc;
    if (total > 0) {
        LFS_TIMED("emit_instances", st);
        if (a.ewa_bounds)
            ewa_emit_instances_kernel<<<grid_for(total, 256), 256, 0, st>>>(total, order, a.tiles, a.offs, a.ewa_bounds, a.ewa_records,
                                                                            (uint32_t)a.tw, a.capacity, a.tkeys[0], a.tvals[0],
                                                                            a.overflow);
        else
        emit_instances_kernel<<<grid_for(total, 256), 256, 0, st>>>(total, a.N, order, a.tiles, a.offs, a.means2d, a.radii,
                                                                    (float)a.tile_size, (uint32_t)a.tw, (uint32_t)a.th,
                                                                    tile_n_bits, a.capacity, a.tkeys[0], a.tvals[0],
                                                                    a.overflow);
    }
    int sel = 0;
    if (a.sort && a.capacity > 0) {
        uint32_t* k[2] = {a.tkeys[0], a.tkeys[1]};
        uint32_t* v[2] = {a.tvals[0], a.tvals[1]};
        sel = radix_sort_pairs(k, v, a.n_isects_dev, a.capacity, (int)(tile_n_bits + cam_n_bits), s, st);
        if (sel < 0) return LFS_ECUDA;
    }
    if (a.sel_out) *a.sel_out = sel;
    if (a.tile_offsets) {
        const int64_t n_ids = (int64_t)a.C * n_tiles;
        LFS_TIMED("tile_offsets", st);
        tile_offsets_kernel<<<grid_for(a.capacity > 0 ? a.capacity : 1, 256), 256, 0, st>>>(
            a.tkeys[sel], a.n_isects_dev, a.capacity, n_tiles, tile_n_bits, n_ids, a.overflow, a.tile_offsets);
    }
    return check_launch("build_tile_lists");
}

// Launch order of the tile CTAs: tiles with the longest lists first, so that the last wave of a rasterizer launch
// is made of short tiles. 132 buckets by the leading one and the next two bits of the list length (a
// floating-point-like key with a 2-bit mantissa); the order inside a bucket is arbitrary. offsets has n_tiles + 1
// entries.
__device__ __forceinline__ int tile_order_bucket(int c) {
    if (c <= 0) return 131;
    const int lz = __clz(c);                              // 0 .. 31, small = long list
    const int shift = max(0, 29 - lz);                    // bring the two bits below the leading one down
    const int mant = (c >> shift) & 3;
    return lz * 4 + (3 - mant);
}

__global__ void __launch_bounds__(1024) tile_order_kernel(int n_tiles, const int32_t* __restrict__ offsets,
                                                          int32_t* __restrict__ order) {
    __shared__ int hist[132], cursor[132];
    if (threadIdx.x < 132) hist[threadIdx.x] = 0;
    __syncthreads();
    for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) atomicAdd(&hist[tile_order_bucket(offsets[t + 1] - offsets[t])], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int b = 0; b < 132; ++b) { cursor[b] = run; run += hist[b]; }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n_tiles; t += blockDim.x)
        order[atomicAdd(&cursor[tile_order_bucket(offsets[t + 1] - offsets[t])], 1)] = t;
}

int launch_tile_order(int n_tiles, const int32_t* offsets, int32_t* order, cudaStream_t st) {
    if (n_tiles <= 0) return LFS_OK;
    LFS_TIMED("tile_order", st);
    tile_order_kernel<<<1, 1024, 0, st>>>(n_tiles, offsets, order);
    return check_launch("tile_order");
}

int launch_compose_isect_ids(int64_t n, const uint32_t* tkeys, const uint32_t* tvals, const float* depths,
                             int64_t* isect_ids, int32_t* flatten_ids, cudaStream_t st) {
    if (n <= 0) return LFS_OK;
    compose_isect_ids_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, tkeys, tvals, depths, isect_ids, flatten_ids);
    return check_launch("compose_isect_ids");
}

int launch_isect_offset(int64_t n, const int64_t* isect_ids, int C, int tw, int th, int32_t* offsets, cudaStream_t st) {
    const uint32_t n_tiles = (uint32_t)tw * th;
    const int64_t n_ids = (int64_t)C * n_tiles;
    isect_offset_kernel<<<grid_for(n > 0 ? n : n_ids, 256), 256, 0, st>>>(n, isect_ids, n_ids, n_tiles,
                                                                          bit_width_u32(n_tiles), offsets);
    return check_launch("isect_offset");
}

int launch_sum_i32(int64_t n, const int32_t* src, int64_t* out_dev, cudaStream_t st) {
    cudaMemsetAsync(out_dev, 0, sizeof(int64_t), st);
    if (n > 0) sum_i32_kernel<<<grid_for(n, 256), 256, 0, st>>>(n, src, reinterpret_cast<unsigned long long*>(out_dev));
    return check_launch("sum_i32");
}

int launch_total_to_i64(const int32_t* total, int64_t* out, cudaStream_t st) {
    total_to_i64_kernel<<<1, 1, 0, st>>>(total, out);
    return check_launch("total_to_i64");
}

}  // namespace lfs
