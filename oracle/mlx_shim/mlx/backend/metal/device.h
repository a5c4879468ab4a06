// Stand-in for mlx/backend/metal/device.h.  There is no Metal here; every entry
// point throws.  Present only so the reference's dequantizer.cpp compiles.
#pragma once
#include "mlx/mlx.h"

namespace MTL {
struct Size {
    size_t width, height, depth;
    Size(size_t w, size_t h, size_t d) : width(w), height(h), depth(d) {}
};
struct Library {};
struct ComputePipelineState {};
}  // namespace MTL

namespace mlx {
namespace core {
namespace metal {

struct CommandEncoder {
    void set_compute_pipeline_state(MTL::ComputePipelineState*) {}
    void set_input_array(const array&, int) {}
    void set_output_array(array&, int) {}
    void dispatch_threadgroups(MTL::Size, MTL::Size) {}
};

struct Device {
    MTL::Library* get_library(const std::string&, const std::string&) {
        throw std::runtime_error("mlx shim: no Metal device");
    }
    MTL::ComputePipelineState* get_kernel(const std::string&, MTL::Library*) {
        throw std::runtime_error("mlx shim: no Metal device");
    }
    CommandEncoder& get_command_encoder(int) { throw std::runtime_error("mlx shim: no Metal device"); }
};

inline Device& device(mlx::core::Device) {
    static Device d;
    return d;
}

}  // namespace metal
}  // namespace core
}  // namespace mlx
