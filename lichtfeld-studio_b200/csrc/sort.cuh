// Launchers of the tile-list stage (sort.cu).
#pragma once

#include "common.cuh"

namespace lfs {

struct TileListArgs {
    int C, N;            // cameras, Gaussians per camera (flattened index = cid * N + gid)
    int tw, th, tile_size;
    int sort;            // 0: emission order, 1: (camera, tile, depth, index) order
    int keys_ready;      // gkeys[0] / gvals[0] already hold (depth bits | 0xFFFFFFFF, index)
    const float* means2d;
    const int32_t* radii;
    const float* depths;
    const int32_t* tiles;  // [C*N] tiles per Gaussian
    uint32_t* gkeys[2];    // [C*N] each
    uint32_t* gvals[2];    // [C*N] each
    int32_t* offs;         // [C*N] exclusive prefix of tiles in emission order
    int32_t* n_isects_dev; // device int32: total number of instances
    int64_t capacity;      // room in tkeys / tvals
    uint32_t* tkeys[2];
    uint32_t* tvals[2];
    int32_t* overflow;     // device flag set when an instance does not fit (may be null)
    int* sel_out;          // host: which of tkeys/tvals holds the result
    int32_t* tile_offsets; // [C*tw*th + 1] or null
    SortScratch scratch;
    // EWA path (C = 1): when set, a Gaussian's instances are the tiles of its bounds rectangle that pass the exact
    // ellipse test (`tiles` holds that count); means2d / radii are unused
    const ushort4* ewa_bounds = nullptr;  // [N] (x_min, x_max, y_min, y_max) in tiles
    const float4* ewa_records = nullptr;  // [N*3], see ewa_common.cuh
};

int build_tile_lists(const TileListArgs& a, cudaStream_t st);

// order [n_tiles]: tile indices, longest lists first; offsets [n_tiles + 1]
int launch_tile_order(int n_tiles, const int32_t* offsets, int32_t* order, cudaStream_t st);
int launch_compose_isect_ids(int64_t n, const uint32_t* tkeys, const uint32_t* tvals, const float* depths,
                             int64_t* isect_ids, int32_t* flatten_ids, cudaStream_t st);
int launch_isect_offset(int64_t n, const int64_t* isect_ids, int C, int tw, int th, int32_t* offsets, cudaStream_t st);
int launch_total_to_i64(const int32_t* total, int64_t* out, cudaStream_t st);
int launch_sum_i32(int64_t n, const int32_t* src, int64_t* out_dev, cudaStream_t st);

}  // namespace lfs
