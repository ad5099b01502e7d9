// Test infrastructure, not part of the product: times the sort call of the reference's tile-list stage on this GPU.
//
// The reference sorts the (tile id << 32 | depth bits) keys of all tile intersections with ONE
// cub::DeviceRadixSort::SortPairs over int64 keys and int32 values, bits [0, 32 + tile bits)
// (gsplat/IntersectTile.cu:290-316). This program issues that call on random keys with the instance counts, tile
// counts and key widths of the benchmark workloads, so that the tile-list stage of this library (depth sort + scan +
// emit + tile sort + offsets, `roofline_tile_lists.ms` of bench.py) has the reference's own sort as its bar.
//
//   nvcc -O3 -gencode arch=compute_100a,code=sm_100a oracle/sort_bar/cub_sortpairs_bar.cu -o oracle/_ref/cub_sortpairs_bar
//   oracle/_ref/cub_sortpairs_bar
#include <cub/cub.cuh>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

int main() {
    struct Case { size_t n; int tiles; int bits; const char* name; } cases[] = {
        {4206111, 4293, 46, "train_1m"}, {7953440, 32400, 48, "wide_4k"}, {9932648, 14400, 47, "wide_fisheye"}};
    for (auto& c : cases) {
        const size_t n = c.n;
        std::vector<int64_t> hk(n);
        std::vector<int32_t> hv(n);
        for (size_t i = 0; i < n; i++) {
            const float d = 1.0f + (rand() % 100000) * 1e-4f;
            uint32_t db;
            memcpy(&db, &d, 4);
            hk[i] = ((int64_t)(rand() % c.tiles) << 32) | db;
            hv[i] = (int32_t)(rand() % 1000000);
        }
        int64_t *k0, *k1;
        int32_t *v0, *v1;
        cudaMalloc(&k0, n * 8); cudaMalloc(&k1, n * 8); cudaMalloc(&v0, n * 4); cudaMalloc(&v1, n * 4);
        cudaMemcpy(k0, hk.data(), n * 8, cudaMemcpyHostToDevice);
        cudaMemcpy(v0, hv.data(), n * 4, cudaMemcpyHostToDevice);
        size_t ws = 0;
        void* d = nullptr;
        cub::DeviceRadixSort::SortPairs(d, ws, k0, k1, v0, v1, (int)n, 0, c.bits);
        cudaMalloc(&d, ws);
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        float best = 1e9f;
        for (int rep = 0; rep < 10; rep++) {
            cudaEventRecord(e0);
            cub::DeviceRadixSort::SortPairs(d, ws, k0, k1, v0, v1, (int)n, 0, c.bits);
            cudaEventRecord(e1);
            cudaEventSynchronize(e1);
            float ms;
            cudaEventElapsedTime(&ms, e0, e1);
            if (rep >= 3 && ms < best) best = ms;
        }
        printf("%s: cub::DeviceRadixSort::SortPairs int64 keys / int32 values, n = %zu, bits [0, %d): %.3f ms (best of 7 after 3 warm-up)\n",
               c.name, n, c.bits, best);
        cudaFree(k0); cudaFree(k1); cudaFree(v0); cudaFree(v1); cudaFree(d);
    }
    return 0;
}
