// Layout of the convolution gather plan shared by its builder and the kernel that reads
// it: int2 tile_info[tiles + 1] (256-byte padded; the last entry holds the number of
// leading tiles up to the last one that uses any offset, and the vector total), then
// int32 row vectors of 256 entries.
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

// position of tile row r inside a row vector
__host__ __device__ inline int plan_slot(int r) { return (r & 31) * 8 + (r >> 5); }

} // namespace lat
