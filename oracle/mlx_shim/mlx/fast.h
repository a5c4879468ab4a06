// Stand-in for mlx/fast.h: the reference only reaches these entry points on its
// Metal path, which the checker build never takes (force_cpu is always set).
// They exist so the translation units compile; calling one is an error.
#pragma once
#include "mlx/mlx.h"

namespace mlx {
namespace core {
namespace fast {

using CustomKernelFunction = std::function<std::vector<array>(
    const std::vector<array>&,
    const std::vector<Shape>&,
    const std::vector<Dtype>&,
    std::tuple<int, int, int>,
    std::tuple<int, int, int>,
    std::vector<std::pair<std::string, int>>,
    std::optional<float>,
    bool,
    Stream)>;

inline CustomKernelFunction metal_kernel(
    const std::string& name,
    const std::vector<std::string>&,
    const std::vector<std::string>&,
    const std::string&,
    const std::string& = "",
    bool = true,
    bool = false) {
    return [name](const std::vector<array>&, const std::vector<Shape>&, const std::vector<Dtype>&,
                  std::tuple<int, int, int>, std::tuple<int, int, int>,
                  std::vector<std::pair<std::string, int>>, std::optional<float>, bool,
                  Stream) -> std::vector<array> {
        throw std::runtime_error("mlx shim: Metal kernel '" + name + "' cannot run on this host");
    };
}

inline array scaled_dot_product_attention(const array&, const array&, const array&, float) {
    throw std::runtime_error("mlx shim: SDPA is restated in the C oracle, not provided here");
}

}  // namespace fast
}  // namespace core
}  // namespace mlx
