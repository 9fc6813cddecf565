// Layout of the convolution gather plan shared by its builder and the kernel that reads
// it: int2 tile_info[tiles + 1] (256-byte padded; the last entry holds the number of
// tiles that use any offset, and the vector total), int32 tile_order[tiles] (256-byte
// padded: the tiles by falling number of used offsets, tiles without any last), then int32
// row vectors of 256 entries.
#pragma once

#include <algorithm>

#include "common.cuh"

namespace lat {

constexpr int kPlanTileRows = 256;

inline int plan_tiles(int out_capacity) {
    return (std::max(out_capacity, 0) + kPlanTileRows - 1) / kPlanTileRows;
}

inline size_t plan_info_bytes(int tiles) {
    return align_up(sizeof(int2) * (static_cast<size_t>(std::max(tiles, 0)) + 1));
}

inline size_t plan_order_bytes(int tiles) {
    return align_up(sizeof(int32_t) * static_cast<size_t>(std::max(tiles, 1)));
}

// byte offset of the row vectors inside the plan
inline size_t plan_vectors_offset(int tiles) { return plan_info_bytes(tiles) + plan_order_bytes(tiles); }

// The convolution hands out tiles in the plan's tile order, CTA b of G taking positions
// b, 2G - 1 - b, 2G + b, ... (a serpentine over the order): with the tiles sorted by cost,
// every pair of rounds gives each CTA about the same work.
__host__ __device__ inline int plan_position(int turn, int cta, int grid) {
    return turn * grid + ((turn & 1) ? grid - 1 - cta : cta);
}

// position of tile row r inside a row vector
__host__ __device__ inline int plan_slot(int r) { return (r & 31) * 8 + (r >> 5); }

} // namespace lat
