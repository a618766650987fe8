// Backward functions of the convolution, pooling, recurrent and CTC records
// (src/OneModel/Tensors/Autograd/BackwardNn.cs:317-506, BackwardOps.cs:285-298, BackwardRecurrent.cs:10-296).
#include "omh.hpp"

namespace omh {

static om_ctx* C() { return Device::Current(); }

// Destination of a parameter gradient: the leaf's own buffer when there is one, else a fresh tensor that is emitted.
struct GradSlot {
  float* ptr = nullptr;
  bool accumulate = false, leaf = false, needed = false;
  Tensor tmp;
  GradSlot(BackwardRecord& r, int i) {
    if (i >= r.InputCount() || !r.NeedsInputGrad(i)) return;
    needed = true;
    leaf = Engine::LeafTarget(r, i, &ptr, &accumulate);
    if (!leaf) {
      tmp = Tensor::Create(DType::F32, r.InputShapes[i]);
      ptr = tmp.Data();
    }
  }
  void Done(BackwardRecord& r, int i) {
    if (!needed) return;
    if (leaf) Engine::LeafWritten(r, i); else Engine::Emit(r, i, tmp, true);
  }
};

static void ConvBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor &x = r.Saved(0), &w = r.Saved(1);
  om_conv_shape s;
  s.n = x.GetShape()[0]; s.cin = x.GetShape()[1]; s.h = x.GetShape()[2]; s.w = x.GetShape()[3];
  s.cout = w.GetShape()[0]; s.kh = w.GetShape()[2]; s.kw = w.GetShape()[3];
  s.stride_h = (int)r.Ints[0]; s.stride_w = (int)r.Ints[1]; s.pad_top = (int)r.Ints[2]; s.pad_left = (int)r.Ints[3];
  s.pad_bottom = (int)r.Ints[4]; s.pad_right = (int)r.Ints[5]; s.dil_h = (int)r.Ints[6]; s.dil_w = (int)r.Ints[7]; s.groups = (int)r.Ints[8];
  Tensor gc = g.Contiguous();
  // Order of the reference: bias, weights, input.
  GradSlot db(r, 2);
  if (db.needed) Check(om_conv2d_dbias(C(), &s, gc.Data(), db.ptr, db.accumulate));
  db.Done(r, 2);
  GradSlot dw(r, 1);
  if (dw.needed) Check(om_conv2d_wgrad(C(), &s, gc.Data(), x.Data(), dw.ptr, dw.accumulate));
  dw.Done(r, 1);
  if (r.NeedsInputGrad(0)) {
    Tensor dx = Tensor::Create(DType::F32, x.GetShape());
    Check(om_conv2d_dgrad(C(), &s, gc.Data(), w.Data(), dx.Data()));
    Engine::Emit(r, 0, dx, true);
  }
}

// The record of Ops::LstmBidirectional: inputs x, then (wIh, wHh, bIh, bHh) per direction; slots 0 x, then per direction
// wIh, wHh, gates, c, tanh c, y.
static void LstmBidirectionalBackward(BackwardRecord& r, const Tensor& gy) {
  const Tensor& x = r.Saved(0);
  int steps = (int)r.Ints[1], batch = (int)r.Ints[2], inSize = (int)r.Ints[3], h = (int)r.Ints[4];
  Tensor g[2], dx[2];
  for (int d = 0; d < 2; d++) {
    g[d] = gy.Slice(2, d * h, (d + 1) * h).Contiguous();
    if (r.NeedsInputGrad(0)) dx[d] = Tensor::Create(DType::F32, x.GetShape());
  }
  std::vector<GradSlot> slots;
  slots.reserve(8);
  for (int k = 0; k < 8; k++) slots.emplace_back(r, 1 + k);
  for (int k = 0; k < 8; k++) {
    GradSlot& s = slots[k];
    if (s.needed && s.leaf && s.accumulate) {      // the kernels overwrite: go through a temporary and add
      s.leaf = false;
      s.tmp = Tensor::Create(DType::F32, r.InputShapes[1 + k]);
      s.ptr = s.tmp.Data();
    }
  }
  const float *gp[2] = {g[0].Data(), g[1].Data()}, *yp[2] = {r.Saved(6).Data(), r.Saved(12).Data()};
  const float *wih[2] = {r.Saved(1).Data(), r.Saved(7).Data()}, *whh[2] = {r.Saved(2).Data(), r.Saved(8).Data()};
  const float *gt[2] = {r.Saved(3).Data(), r.Saved(9).Data()}, *cs[2] = {r.Saved(4).Data(), r.Saved(10).Data()};
  const float* tc[2] = {r.Saved(5).Data(), r.Saved(11).Data()};
  float* dxp[2] = {dx[0].IsEmpty() ? nullptr : dx[0].Data(), dx[1].IsEmpty() ? nullptr : dx[1].Data()};
  float *dwi[2] = {slots[0].ptr, slots[4].ptr}, *dwh[2] = {slots[1].ptr, slots[5].ptr}, *dbi[2] = {slots[2].ptr, slots[6].ptr},
        *dbh[2] = {slots[3].ptr, slots[7].ptr};
  Check(om_lstm_bilayer_bwd(C(), steps, batch, inSize, h, gp, x.Data(), yp, wih, whh, gt, cs, tc, dxp, dwi, dwh, dbi, dbh));
  if (!dx[0].IsEmpty()) {
    Check(om_add_into(C(), dx[0].Data(), dx[1].Data(), dx[0].Length()));   // forward direction's share first, then the reverse one
    Engine::Emit(r, 0, dx[0], true);
  }
  for (int k = 0; k < 8; k++) slots[k].Done(r, 1 + k);
}

static void LstmBackward(BackwardRecord& r, const Tensor& gy) {
  if (r.Ints[0] == 2) return LstmBidirectionalBackward(r, gy);
  const Tensor &x = r.Saved(0), &wIh = r.Saved(1), &wHh = r.Saved(2), &gates = r.Saved(3), &cseq = r.Saved(4), &tanhC = r.Saved(5), &y = r.Saved(6);
  bool reverse = r.Ints[0] != 0;
  int steps = (int)r.Ints[1], batch = (int)r.Ints[2], inSize = (int)r.Ints[3], h = (int)r.Ints[4];
  Tensor gc = gy.Contiguous();
  Tensor dx;
  if (r.NeedsInputGrad(0)) dx = Tensor::Create(DType::F32, x.GetShape());
  GradSlot dwi(r, 1), dwh(r, 2), dbi(r, 3), dbh(r, 4);
  // The kernels overwrite their outputs; when a leaf buffer already holds a gradient, go through a temporary and add.
  auto Plain = [&](GradSlot& s, int i) {
    if (s.needed && s.leaf && s.accumulate) {
      s.leaf = false;
      s.tmp = Tensor::Create(DType::F32, r.InputShapes[i]);
      s.ptr = s.tmp.Data();
    }
  };
  Plain(dwi, 1); Plain(dwh, 2); Plain(dbi, 3); Plain(dbh, 4);
  Check(om_lstm_layer_bwd(C(), reverse, steps, batch, inSize, h, gc.Data(), nullptr, nullptr, x.Data(), y.Data(), wIh.Data(), wHh.Data(),
                          nullptr, nullptr, gates.Data(), cseq.Data(), tanhC.Data(), dx.IsEmpty() ? nullptr : dx.Data(), dwi.ptr, dwh.ptr,
                          dbi.ptr, dbh.ptr, nullptr, nullptr));
  if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  dwi.Done(r, 1); dwh.Done(r, 2); dbi.Done(r, 3); dbh.Done(r, 4);
}

static void GruBackward(BackwardRecord& r, const Tensor& gy) {
  const Tensor &x = r.Saved(0), &wIh = r.Saved(1), &wHh = r.Saved(2), &gates = r.Saved(3), &hn = r.Saved(4), &y = r.Saved(5), &h0 = r.Saved(6);
  bool reverse = r.Ints[0] != 0;
  int steps = (int)r.Ints[1], batch = (int)r.Ints[2], inSize = (int)r.Ints[3], h = (int)r.Ints[4];
  Tensor gc = gy.Contiguous();
  Tensor dx, dh0;
  if (r.NeedsInputGrad(0)) dx = Tensor::Create(DType::F32, x.GetShape());
  if (r.NeedsInputGrad(5)) dh0 = Tensor::Create(DType::F32, Shape{batch, h});
  GradSlot dwi(r, 1), dwh(r, 2), dbi(r, 3), dbh(r, 4);
  auto Plain = [&](GradSlot& s, int i) {
    if (s.needed && s.leaf && s.accumulate) {
      s.leaf = false;
      s.tmp = Tensor::Create(DType::F32, r.InputShapes[i]);
      s.ptr = s.tmp.Data();
    }
  };
  Plain(dwi, 1); Plain(dwh, 2); Plain(dbi, 3); Plain(dbh, 4);
  Check(om_gru_layer_bwd(C(), reverse, steps, batch, inSize, h, gc.Data(), x.Data(), y.Data(), wIh.Data(), wHh.Data(),
                         h0.IsEmpty() ? nullptr : h0.Data(), gates.Data(), hn.Data(), dx.IsEmpty() ? nullptr : dx.Data(), dwi.ptr, dwh.ptr,
                         dbi.ptr, dbh.ptr, dh0.IsEmpty() ? nullptr : dh0.Data()));
  if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  dwi.Done(r, 1); dwh.Done(r, 2); dbi.Done(r, 3); dbh.Done(r, 4);
  if (!dh0.IsEmpty()) Engine::Emit(r, 5, dh0, true);
}

void RunSpatialBackward(Engine& e, BackwardRecord& r, const Tensor& g) {
  (void)e;
  switch (r.Op) {
    case OpKind::Conv2d: ConvBackward(r, g); break;
    case OpKind::MaxPool2d: {
      const Tensor& idx = r.Saved(0);
      const Shape& in = r.InputShapes[0];
      Tensor gc = g.Contiguous();
      Tensor dx = Tensor::Create(DType::F32, in);
      Check(om_maxpool_bwd(C(), gc.Data(), (const int32_t*)idx.RawData(), in[0] * in[1], in[2], in[3], g.GetShape()[2], g.GetShape()[3],
                           (int)r.Ints[0], (int)r.Ints[1], (int)r.Ints[2], (int)r.Ints[3], (int)r.Ints[4], (int)r.Ints[5], dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::AvgPool2d: {
      const Shape& in = r.InputShapes[0];
      Tensor gc = g.Contiguous();
      Tensor dx = Tensor::Create(DType::F32, in);
      Check(om_avgpool_bwd(C(), gc.Data(), in[0] * in[1], in[2], in[3], (int)r.Ints[0], (int)r.Ints[1], (int)r.Ints[2], (int)r.Ints[3],
                           (int)r.Ints[4], (int)r.Ints[5], (int)r.Ints[6], dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Lstm: LstmBackward(r, g); break;
    case OpKind::Gru: GruBackward(r, g); break;
    case OpKind::CtcLoss: {
      const Tensor &lp = r.Saved(0), &targets = r.Saved(1), &ilen = r.Saved(2), &tlen = r.Saved(3);
      Tensor gc = g.Contiguous();
      Tensor dx = Tensor::Create(DType::F32, lp.GetShape());
      Check(om_ctc_grad(C(), gc.Data(), lp.Data(), lp.GetShape()[0], lp.GetShape()[1], lp.GetShape()[2], (const int32_t*)targets.RawData(),
                        (const int32_t*)tlen.RawData(), (const int32_t*)ilen.RawData(), nullptr, (int)r.Ints[0], (int)r.Ints[2],
                        (int)r.Ints[1], dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    default: RunGraphBackward(r, g); break;
  }
}

}  // namespace omh
