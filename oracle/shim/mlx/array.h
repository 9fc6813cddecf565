// Test infrastructure only: a minimal stand-in for the MLX C++ array type, just
// wide enough for the reference project's CPU algorithm files to compile
// unmodified. Arrays are plain host buffers with a shape, row-major strides and a
// dtype tag. Nothing here is part of the shipped library.
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <memory>
#include <vector>

#include "mlx/allocator.h"
#include "mlx/stream.h"
#include "mlx/types/half_types.h"

namespace mlx::core {

using Shape = std::vector<int>;
using Strides = std::vector<std::ptrdiff_t>;

struct Dtype {
    enum class Val : std::uint8_t { u32, i32, i64, f16, f32 };
    Val val;
    std::uint8_t size;
    constexpr bool operator==(const Dtype& other) const { return val == other.val; }
    constexpr bool operator!=(const Dtype& other) const { return val != other.val; }
};

inline constexpr Dtype uint32{Dtype::Val::u32, 4};
inline constexpr Dtype int32{Dtype::Val::i32, 4};
inline constexpr Dtype int64{Dtype::Val::i64, 8};
inline constexpr Dtype float16{Dtype::Val::f16, 2};
inline constexpr Dtype float32{Dtype::Val::f32, 4};

class array {
  public:
    array(Shape shape, Dtype dtype) : state_(std::make_shared<State>()) {
        state_->shape = std::move(shape);
        state_->dtype = dtype;
        reset_strides();
    }

    // Wrap caller-owned memory (not freed here).
    array(void* data, Shape shape, Dtype dtype) : array(std::move(shape), dtype) {
        state_->data = data;
    }

    array(void* data, Shape shape, Strides strides, Dtype dtype)
        : array(std::move(shape), dtype) {
        state_->data = data;
        state_->strides = std::move(strides);
    }

    int shape(int axis) const { return state_->shape[norm(axis)]; }
    const Shape& shape() const { return state_->shape; }
    std::ptrdiff_t strides(int axis) const { return state_->strides[norm(axis)]; }
    const Strides& strides() const { return state_->strides; }
    int ndim() const { return int(state_->shape.size()); }
    Dtype dtype() const { return state_->dtype; }
    std::size_t itemsize() const { return state_->dtype.size; }

    std::size_t size() const {
        std::size_t total = 1;
        for (auto dim : state_->shape) {
            total *= std::size_t(dim);
        }
        return total;
    }

    std::size_t nbytes() const { return size() * itemsize(); }

    // The reference allocates every output itself; when the harness already
    // attached caller-owned memory the fresh buffer is dropped again so results
    // land where the caller can read them.
    void set_data(allocator::Buffer buffer) {
        if (state_->data != nullptr) {
            allocator::free(buffer);
            return;
        }
        state_->data = buffer.raw_ptr();
        state_->owned = buffer;
    }

    template <typename T> T* data() { return static_cast<T*>(state_->data); }
    template <typename T> const T* data() const {
        return static_cast<const T*>(state_->data);
    }

  private:
    struct State {
        Shape shape;
        Strides strides;
        Dtype dtype{Dtype::Val::f32, 4};
        void* data = nullptr;
        allocator::Buffer owned{nullptr};
        ~State() {
            if (owned.raw_ptr() != nullptr) {
                allocator::free(owned);
            }
        }
    };

    int norm(int axis) const { return axis < 0 ? axis + ndim() : axis; }

    void reset_strides() {
        state_->strides.assign(state_->shape.size(), 1);
        std::ptrdiff_t run = 1;
        for (int axis = ndim() - 1; axis >= 0; --axis) {
            state_->strides[axis] = run;
            run *= state_->shape[axis];
        }
    }

    std::shared_ptr<State> state_;
};

} // namespace mlx::core
