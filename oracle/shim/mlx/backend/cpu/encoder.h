// Test infrastructure only: the command encoder runs each task immediately on
// the calling thread instead of queueing it on a stream worker.
#pragma once

#include <utility>

#include "mlx/array.h"
#include "mlx/stream.h"

namespace mlx::core::cpu {

struct CommandEncoder {
    void set_input_array(const array&) {}
    void set_output_array(array&) {}
    template <typename Fn> void dispatch(Fn&& fn) { std::forward<Fn>(fn)(); }
};

inline CommandEncoder& get_command_encoder(const Stream&) {
    static thread_local CommandEncoder encoder;
    return encoder;
}

} // namespace mlx::core::cpu
