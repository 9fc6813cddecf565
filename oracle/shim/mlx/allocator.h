// Test infrastructure only: host malloc behind the MLX allocator names.
#pragma once

#include <cstddef>
#include <cstdlib>

namespace mlx::core::allocator {

class Buffer {
  public:
    explicit Buffer(void* ptr) : ptr_(ptr) {}
    void* raw_ptr() const { return ptr_; }
    void* ptr() const { return ptr_; }

  private:
    void* ptr_;
};

inline Buffer malloc(std::size_t bytes) {
    return Buffer(std::malloc(bytes == 0 ? 1 : bytes));
}

inline void free(Buffer buffer) { std::free(buffer.raw_ptr()); }

} // namespace mlx::core::allocator
