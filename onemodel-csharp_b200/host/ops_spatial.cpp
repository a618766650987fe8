// Convolution, pooling, recurrent and CTC forward operations
// (src/OneModel/Tensors/Ops.Layers.cs:279-461, Ops.cs:146-178, Ops.Recurrent.cs:40-146, CtcLoss.cs:40-153).
#include "omh.hpp"

namespace omh {

static Tensor NotYet(const char* what) { throw InvalidOperationException(std::string(what) + " is not available in this build."); }

Tensor Ops::Conv2d(const Tensor&, const Tensor&, const Tensor&, const Conv2dParams&) { return NotYet("Conv2d"); }
Tensor Ops::MaxPool2d(const Tensor&, int, int, int, int, int, int) { return NotYet("MaxPool2d"); }
Tensor Ops::AvgPool2d(const Tensor&, int, int, int, int, int, int, bool) { return NotYet("AvgPool2d"); }
Tensor Ops::LstmLayer(const Tensor&, const Tensor&, const Tensor&, const Tensor&, const Tensor&, bool, Tensor*, Tensor*) { return NotYet("LstmLayer"); }
Tensor Ops::CtcLoss(const Tensor&, const Tensor&, const Tensor&, const Tensor&, int, int, bool) { return NotYet("CtcLoss"); }
Recurrent::Recurrent(int, int hidden, int layers, bool bidirectional, Generator&) : Hidden(hidden), Layers(layers), Bidirectional(bidirectional) {}
Tensor Recurrent::Forward(const Tensor&) { return NotYet("Recurrent"); }

}  // namespace omh
