// Test infrastructure only: a stream is just a tag; work runs inline.
#pragma once

namespace mlx::core {

struct Device {
    enum DeviceType { cpu, gpu };
    DeviceType type = cpu;
    int index = 0;
};

struct Stream {
    int index = 0;
    Device device{};
};

} // namespace mlx::core
