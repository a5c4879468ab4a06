// Stand-in for mlx/primitives.h: just enough of the Primitive base class for the
// reference's FusedDequantMatmulPrimitive to compile.  Never evaluated.
#pragma once
#include "mlx/mlx.h"

namespace mlx {
namespace core {

class Primitive {
public:
    explicit Primitive(Stream s) : stream_(s) {}
    virtual ~Primitive() = default;
    virtual void eval_cpu(const std::vector<array>& inputs, std::vector<array>& outputs) = 0;
    virtual void eval_gpu(const std::vector<array>& inputs, std::vector<array>& outputs) = 0;
    virtual const char* name() const { return "Primitive"; }
    virtual bool is_equivalent(const Primitive&) const { return false; }
    const Stream& stream() const { return stream_; }

private:
    Stream stream_;
};

}  // namespace core
}  // namespace mlx
