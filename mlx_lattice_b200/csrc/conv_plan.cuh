// Layout of the convolution gather plan shared by its builder and the kernel that reads
// it: int2 tile_info[tiles + 1] (256-byte padded; the last entry holds the number of
// leading tiles up to the last one that uses any offset, and the vector total), the
// builder's scratch, then int32 row vectors of 256 entries.
#pragma once

#include <algorithm>

#include "common.cuh"

namespace lat {

constexpr int kPlanTileRows = 256;

inline int plan_tiles(int out_capacity) {
    return (std::max(out_capacity, 0) + kPlanTileRows - 1) / kPlanTileRows;
}

// tile_info[tiles + 1], then the builder's scratch (one 8-byte look-back word per tile
// and a ticket counter), each padded to 256 bytes
inline size_t plan_tile_info_bytes(int tiles) {
    return align_up(sizeof(int2) * (static_cast<size_t>(std::max(tiles, 0)) + 1));
}

inline size_t plan_info_bytes(int tiles) {
    return plan_tile_info_bytes(tiles) +
           align_up(sizeof(unsigned long long) * (static_cast<size_t>(std::max(tiles, 0)) + 1));
}

// position of tile row r inside a row vector
__host__ __device__ inline int plan_slot(int r) { return (r & 31) * 8 + (r >> 5); }

} // namespace lat
