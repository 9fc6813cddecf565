// Test infrastructure only: IEEE binary16 through the compiler's _Float16
// (round-to-nearest-even conversions, like MLX's float16_t on the CPU).
#pragma once

namespace mlx::core {

using float16_t = _Float16;

} // namespace mlx::core
