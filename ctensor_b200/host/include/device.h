// Device tag of a tensor's storage — same names and meaning as the reference's
// src/core/device.h:5-25, so callers that say Device(DeviceType::CUDA, 0) compile unchanged.
#pragma once
#include <string>

enum class DeviceType { CPU, CUDA };

struct Device {
    DeviceType type;
    int index;

    Device(DeviceType t = DeviceType::CPU, int i = -1) : type(t), index(i) {}

    bool is_cpu() const { return type == DeviceType::CPU; }
    bool is_cuda() const { return type == DeviceType::CUDA; }

    std::string str() const {
        std::string s = is_cpu() ? "cpu" : "cuda";
        if (index >= 0) s += ":" + std::to_string(index);
        return s;
    }

    bool operator==(const Device& o) const { return type == o.type && index == o.index; }
    bool operator!=(const Device& o) const { return !(*this == o); }
};
