// Convolution, pooling, recurrent and CTC forward operations
// (src/OneModel/Tensors/Ops.Layers.cs:279-461, Ops.cs:146-178, Ops.Recurrent.cs:40-146, CtcLoss.cs:40-153).
#include <math.h>

#include "omh.hpp"

namespace omh {

static om_ctx* C() { return Device::Current(); }

static Tensor NewOut(const Shape& s) {
  Tensor r = Tensor::Create(DType::F32, s);
  ActivationScope::Track(r);
  return r;
}

static om_conv_shape ConvShapeOf(const Tensor& x, const Tensor& w, const Conv2dParams& p) {
  om_conv_shape s;
  s.n = x.GetShape()[0]; s.cin = x.GetShape()[1]; s.h = x.GetShape()[2]; s.w = x.GetShape()[3];
  s.cout = w.GetShape()[0]; s.kh = w.GetShape()[2]; s.kw = w.GetShape()[3];
  s.stride_h = p.strideH; s.stride_w = p.strideW; s.pad_top = p.padTop; s.pad_left = p.padLeft;
  s.pad_bottom = p.padBottom; s.pad_right = p.padRight; s.dil_h = p.dilH; s.dil_w = p.dilW; s.groups = p.groups;
  return s;
}

Tensor Ops::Conv2d(const Tensor& x, const Tensor& weight, const Tensor& bias, const Conv2dParams& pin) {
  Conv2dParams p = pin;
  if (p.strideH == 0) p.strideH = 1;
  if (p.strideW == 0) p.strideW = 1;
  if (p.dilH == 0) p.dilH = 1;
  if (p.dilW == 0) p.dilW = 1;
  if (p.groups == 0) p.groups = 1;
  if (x.Rank() != 4 || weight.Rank() != 4)
    throw TensorShapeException("Conv2d needs an (N,C,H,W) input and (O,I,KH,KW) weights, not " + x.GetShape().ToString() + " and " + weight.GetShape().ToString() + ".");
  if (p.groups < 1 || x.GetShape()[1] % p.groups != 0 || weight.GetShape()[0] % p.groups != 0 || weight.GetShape()[1] != x.GetShape()[1] / p.groups)
    throw TensorShapeException("Weights " + weight.GetShape().ToString() + " do not fit input " + x.GetShape().ToString() + " with " + std::to_string(p.groups) + " groups.");
  if (!bias.IsEmpty() && (bias.Rank() != 1 || bias.GetShape()[0] != weight.GetShape()[0]))
    throw TensorShapeException("The bias must have shape [" + std::to_string(weight.GetShape()[0]) + "], not " + bias.GetShape().ToString() + ".");
  om_conv_shape s = ConvShapeOf(x, weight, p);
  int oh = (s.h + s.pad_top + s.pad_bottom - s.dil_h * (s.kh - 1) - 1) / s.stride_h + 1;
  int ow = (s.w + s.pad_left + s.pad_right - s.dil_w * (s.kw - 1) - 1) / s.stride_w + 1;
  if (p.strideH < 1 || p.strideW < 1 || p.dilH < 1 || p.dilW < 1 || p.padTop < 0 || p.padLeft < 0 || oh < 1 || ow < 1)
    throw TensorShapeException("Invalid convolution geometry for input " + x.GetShape().ToString() + " and kernel " + weight.GetShape().ToString() + ".");
  Tensor xc = x.Contiguous(), wc = weight.Contiguous();
  Tensor bc = bias.IsEmpty() ? Tensor() : bias.Contiguous();
  Tensor r = NewOut(Shape{s.n, s.cout, oh, ow});
  Check(om_conv2d_fwd(C(), &s, xc.Data(), wc.Data(), bc.IsEmpty() ? nullptr : bc.Data(), r.Data()));
  if (!Recording({&x, &weight, &bias})) return r;
  auto br = bias.IsEmpty() ? BackwardRecord::Create(OpKind::Conv2d, 2, {&x, &weight}) : BackwardRecord::Create(OpKind::Conv2d, 2, {&x, &weight, &bias});
  br->Save(0, xc.Detach());
  br->Save(1, wc.Detach());
  br->Ints = {p.strideH, p.strideW, p.padTop, p.padLeft, p.padBottom, p.padRight, p.dilH, p.dilW, p.groups};
  return br->Attach(r);
}

static int PoolOut(int size, int kernel, int stride, int pad) {
  if (kernel < 1 || stride < 1 || pad < 0 || pad >= kernel)
    throw TensorShapeException("Invalid pooling window (kernel " + std::to_string(kernel) + ", stride " + std::to_string(stride) + ", pad " + std::to_string(pad) + ").");
  int64_t span = (int64_t)size + 2LL * pad - kernel;
  if (span < 0) throw TensorShapeException("The pooling window is larger than the padded input.");
  return (int)(span / stride) + 1;
}

Tensor Ops::MaxPool2d(const Tensor& x, int kh, int kw, int sh, int sw, int ph, int pw) {
  if (x.Rank() != 4) throw TensorShapeException("MaxPool2d needs an (N,C,H,W) input, not " + x.GetShape().ToString() + ".");
  int n = x.GetShape()[0], c = x.GetShape()[1], h = x.GetShape()[2], w = x.GetShape()[3];
  int oh = PoolOut(h, kh, sh, ph), ow = PoolOut(w, kw, sw, pw);
  Tensor xc = x.Contiguous();
  Tensor r = NewOut(Shape{n, c, oh, ow});
  bool track = Recording({&x});
  Tensor idx = track ? Tensor::Create(DType::I32, Shape{n, c, oh, ow}) : Tensor();
  Check(om_maxpool_fwd(C(), xc.Data(), n * c, h, w, kh, kw, sh, sw, ph, pw, r.Data(), track ? (int32_t*)idx.RawData() : nullptr));
  if (!track) return r;
  auto rec = BackwardRecord::Create(OpKind::MaxPool2d, 1, {&x});
  rec->Save(0, idx);
  rec->Ints = {kh, kw, sh, sw, ph, pw};
  return rec->Attach(r);
}

Tensor Ops::AvgPool2d(const Tensor& x, int kh, int kw, int sh, int sw, int ph, int pw, bool countIncludePad) {
  if (x.Rank() != 4) throw TensorShapeException("AvgPool2d needs an (N,C,H,W) input, not " + x.GetShape().ToString() + ".");
  int n = x.GetShape()[0], c = x.GetShape()[1], h = x.GetShape()[2], w = x.GetShape()[3];
  int oh = PoolOut(h, kh, sh, ph), ow = PoolOut(w, kw, sw, pw);
  Tensor xc = x.Contiguous();
  Tensor r = NewOut(Shape{n, c, oh, ow});
  Check(om_avgpool_fwd(C(), xc.Data(), n * c, h, w, kh, kw, sh, sw, ph, pw, countIncludePad, r.Data()));
  if (!Recording({&x})) return r;
  auto rec = BackwardRecord::Create(OpKind::AvgPool2d, 0, {&x});
  rec->Ints = {kh, kw, sh, sw, ph, pw, countIncludePad ? 1 : 0};
  return rec->Attach(r);
}

// One LSTM layer direction over x [T,B,I] with zero initial state. Record slots as the reference: x, wIh, wHh, gates,
// c, tanh(c), y; Ints = [reverse, T, B, I, H] (Ops.Recurrent.cs:125-146).
Tensor Ops::LstmLayer(const Tensor& x, const Tensor& wIh, const Tensor& wHh, const Tensor& bIh, const Tensor& bHh, bool reverse,
                      Tensor* hn, Tensor* cn) {
  if (x.Rank() != 3 || wIh.Rank() != 2 || wHh.Rank() != 2 || wIh.GetShape()[0] % 4 != 0 || wIh.GetShape()[1] != x.GetShape()[2] ||
      wHh.GetShape()[0] != wIh.GetShape()[0] || wHh.GetShape()[1] * 4 != wHh.GetShape()[0])
    throw TensorShapeException("LstmLayer needs x [T,B,I], wIh [4H,I], wHh [4H,H], not " + x.GetShape().ToString() + ", " +
                               wIh.GetShape().ToString() + ", " + wHh.GetShape().ToString() + ".");
  int steps = x.GetShape()[0], batch = x.GetShape()[1], inSize = x.GetShape()[2], h = wHh.GetShape()[1];
  for (const Tensor* b : {&bIh, &bHh})
    if (!b->IsEmpty() && (b->Rank() != 1 || b->GetShape()[0] != 4 * h)) throw TensorShapeException("LstmLayer biases must have shape [4H].");
  Tensor xc = x.Contiguous(), wi = wIh.Contiguous(), wh = wHh.Contiguous();
  Tensor bi = bIh.IsEmpty() ? Tensor() : bIh.Contiguous(), bh = bHh.IsEmpty() ? Tensor() : bHh.Contiguous();
  Tensor y = NewOut(Shape{steps, batch, h});
  Tensor gates = Tensor::Create(DType::F32, Shape{steps, batch, 4 * h});
  Tensor cseq = Tensor::Create(DType::F32, Shape{steps, batch, h});
  Tensor tanhC = Tensor::Create(DType::F32, Shape{steps, batch, h});
  Check(om_lstm_layer_fwd(C(), reverse, steps, batch, inSize, h, xc.Data(), wi.Data(), wh.Data(), bi.IsEmpty() ? nullptr : bi.Data(),
                          bh.IsEmpty() ? nullptr : bh.Data(), nullptr, nullptr, y.Data(), gates.Data(), cseq.Data(), tanhC.Data()));
  if (hn && steps > 0) *hn = y.Select(0, reverse ? 0 : steps - 1).Detach();
  if (cn && steps > 0) *cn = cseq.Select(0, reverse ? 0 : steps - 1);
  std::vector<Tensor> ins = {x, wIh, wHh};
  if (!bIh.IsEmpty() || !bHh.IsEmpty()) {
    ins.push_back(bIh);
    ins.push_back(bHh);
  }
  bool rec = GradMode::Enabled();
  if (rec) {
    rec = false;
    for (const Tensor& t : ins) rec = rec || (!t.IsEmpty() && t.RequiresGrad());
  }
  if (!rec) return y;
  auto br = BackwardRecord::Create(OpKind::Lstm, 7, ins);
  br->Save(0, xc.Detach());
  br->Save(1, wi.Detach());
  br->Save(2, wh.Detach());
  br->Save(3, gates);
  br->Save(4, cseq);
  br->Save(5, tanhC);
  br->Save(6, y.Detach());
  br->Ints = {reverse ? 1 : 0, steps, batch, inSize, h};
  return br->Attach(y);
}

Tensor Ops::LstmBidirectional(const Tensor& x, const std::vector<Tensor>& w) {
  if (w.size() != 8) throw std::invalid_argument("LstmBidirectional needs wIh, wHh, bIh, bHh for both directions.");
  if (x.Rank() != 3) throw TensorShapeException("LstmLayer needs x [T,B,I], not " + x.GetShape().ToString() + ".");
  int steps = x.GetShape()[0], batch = x.GetShape()[1], inSize = x.GetShape()[2], h = w[1].GetShape()[1];
  for (int d = 0; d < 2; d++) {
    const Tensor &wi = w[4 * d], &wh = w[4 * d + 1], &bi = w[4 * d + 2], &bh = w[4 * d + 3];
    if (wi.Rank() != 2 || wh.Rank() != 2 || wi.GetShape()[0] != 4 * h || wi.GetShape()[1] != inSize || wh.GetShape()[0] != 4 * h ||
        wh.GetShape()[1] != h)
      throw TensorShapeException("LstmLayer needs x [T,B,I], wIh [4H,I], wHh [4H,H], not " + x.GetShape().ToString() + ", " +
                                 wi.GetShape().ToString() + ", " + wh.GetShape().ToString() + ".");
    if (bi.IsEmpty() != bh.IsEmpty() || (!bi.IsEmpty() && (bi.Length() != 4 * h || bh.Length() != 4 * h)))
      throw TensorShapeException("LstmLayer biases must have shape [4H] (both or none).");
  }
  Tensor xc = x.Contiguous();
  Tensor wc[8];
  for (int k = 0; k < 8; k++) wc[k] = w[k].IsEmpty() ? Tensor() : w[k].Contiguous();
  Tensor y[2], gates[2], cseq[2], tanhC[2];
  for (int d = 0; d < 2; d++) {
    y[d] = Tensor::Create(DType::F32, Shape{steps, batch, h});
    gates[d] = Tensor::Create(DType::F32, Shape{steps, batch, 4 * h});
    cseq[d] = Tensor::Create(DType::F32, Shape{steps, batch, h});
    tanhC[d] = Tensor::Create(DType::F32, Shape{steps, batch, h});
  }
  const bool hasBias = !wc[2].IsEmpty() && !wc[6].IsEmpty();
  const float *wih[2] = {wc[0].Data(), wc[4].Data()}, *whh[2] = {wc[1].Data(), wc[5].Data()};
  const float *bih[2] = {hasBias ? wc[2].Data() : nullptr, hasBias ? wc[6].Data() : nullptr};
  const float *bhh[2] = {hasBias ? wc[3].Data() : nullptr, hasBias ? wc[7].Data() : nullptr};
  float *yp[2] = {y[0].Data(), y[1].Data()}, *gp[2] = {gates[0].Data(), gates[1].Data()}, *cp[2] = {cseq[0].Data(), cseq[1].Data()},
        *tp[2] = {tanhC[0].Data(), tanhC[1].Data()};
  if (!hasBias && (!wc[2].IsEmpty() || !wc[6].IsEmpty()))
    throw TensorShapeException("LstmBidirectional: either both directions have biases or neither.");
  Check(om_lstm_bilayer_fwd(C(), steps, batch, inSize, h, xc.Data(), wih, whh, hasBias ? bih : nullptr, hasBias ? bhh : nullptr, yp, gp, cp, tp));
  // [T,B,2H]: the two outputs side by side on the feature axis.
  Tensor r = NewOut(Shape{steps, batch, 2 * h});
  for (int d = 0; d < 2; d++) {
    Tensor dst = r.Slice(2, d * h, (d + 1) * h).Detach();
    Check(om_strided_copy(C(), 3, y[d].GetShape().d.data(), y[d].Data(), y[d].Strides().data(), dst.Data(), dst.Strides().data()));
  }
  std::vector<Tensor> ins = {x};
  for (int k = 0; k < 8; k++) ins.push_back(w[k]);
  bool rec = false;
  if (GradMode::Enabled())
    for (const Tensor& t : ins) rec = rec || (!t.IsEmpty() && t.RequiresGrad());
  if (!rec) return r;
  auto br = BackwardRecord::Create(OpKind::Lstm, 13, ins);
  br->Save(0, xc.Detach());
  for (int d = 0; d < 2; d++) {
    br->Save(1 + 6 * d, wc[4 * d].Detach());
    br->Save(2 + 6 * d, wc[4 * d + 1].Detach());
    br->Save(3 + 6 * d, gates[d]);
    br->Save(4 + 6 * d, cseq[d]);
    br->Save(5 + 6 * d, tanhC[d]);
    br->Save(6 + 6 * d, y[d]);
  }
  br->Ints = {2, steps, batch, inSize, h};     // Ints[0] == 2 marks the bidirectional record
  return br->Attach(r);
}

Tensor Ops::GruLayer(const Tensor& x, const Tensor& wIh, const Tensor& wHh, const Tensor& bIh, const Tensor& bHh, const Tensor& h0,
                     bool reverse) {
  if (x.Rank() != 3 || wIh.Rank() != 2 || wHh.Rank() != 2 || wIh.GetShape()[0] % 3 != 0 || wIh.GetShape()[1] != x.GetShape()[2] ||
      wHh.GetShape()[0] != wIh.GetShape()[0] || wHh.GetShape()[1] * 3 != wHh.GetShape()[0])
    throw TensorShapeException("GruLayer needs x [T,B,I], wIh [3H,I], wHh [3H,H], not " + x.GetShape().ToString() + ", " +
                               wIh.GetShape().ToString() + ", " + wHh.GetShape().ToString() + ".");
  int steps = x.GetShape()[0], batch = x.GetShape()[1], inSize = x.GetShape()[2], h = wHh.GetShape()[1];
  for (const Tensor* b : {&bIh, &bHh})
    if (!b->IsEmpty() && (b->Rank() != 1 || b->GetShape()[0] != 3 * h)) throw TensorShapeException("GruLayer biases must have shape [3H].");
  if (!h0.IsEmpty() && (h0.Rank() != 2 || h0.GetShape()[0] != batch || h0.GetShape()[1] != h))
    throw TensorShapeException("GruLayer: the initial state must be [B,H], not " + h0.GetShape().ToString() + ".");
  Tensor xc = x.Contiguous(), wi = wIh.Contiguous(), wh = wHh.Contiguous();
  Tensor bi = bIh.IsEmpty() ? Tensor() : bIh.Contiguous(), bh = bHh.IsEmpty() ? Tensor() : bHh.Contiguous();
  Tensor h0c = h0.IsEmpty() ? Tensor() : h0.Contiguous();
  Tensor y = NewOut(Shape{steps, batch, h});
  Tensor gates = Tensor::Create(DType::F32, Shape{steps, batch, 3 * h});
  Tensor hn = Tensor::Create(DType::F32, Shape{steps, batch, h});
  Check(om_gru_layer_fwd(C(), reverse, steps, batch, inSize, h, xc.Data(), wi.Data(), wh.Data(), bi.IsEmpty() ? nullptr : bi.Data(),
                         bh.IsEmpty() ? nullptr : bh.Data(), h0c.IsEmpty() ? nullptr : h0c.Data(), y.Data(), gates.Data(), hn.Data()));
  // Record inputs: x, wIh, wHh, bIh, bHh, h0 (the reference's order); absent ones are empty tensors.
  std::vector<Tensor> ins = {x, wIh, wHh, bIh, bHh, h0};
  bool rec = false;
  if (GradMode::Enabled())
    for (const Tensor& t : ins) rec = rec || (!t.IsEmpty() && t.RequiresGrad());
  if (!rec) return y;
  auto br = BackwardRecord::Create(OpKind::Gru, 7, ins);
  br->Save(0, xc.Detach());
  br->Save(1, wi.Detach());
  br->Save(2, wh.Detach());
  br->Save(3, gates);
  br->Save(4, hn);
  br->Save(5, y.Detach());
  if (!h0c.IsEmpty()) br->Save(6, h0c.Detach());
  br->Ints = {reverse ? 1 : 0, steps, batch, inSize, h};
  return br->Attach(y);
}

// logProbs [T,B,C]; targets (Int32, concatenated), inputLengths and targetLengths (Int32 [B]) live on the device.
// reduction: 0 none, 1 mean, 2 sum (CtcReduction of the reference).
Tensor Ops::CtcLoss(const Tensor& logProbs, const Tensor& targets, const Tensor& inputLengths, const Tensor& targetLengths,
                    int blank, int reduction, bool zeroInfinity) {
  if (logProbs.Rank() != 3) throw TensorShapeException("CtcLoss needs log-probabilities [T,B,C], not " + logProbs.GetShape().ToString() + ".");
  int steps = logProbs.GetShape()[0], batch = logProbs.GetShape()[1], classes = logProbs.GetShape()[2];
  if (inputLengths.Length() != batch || targetLengths.Length() != batch || inputLengths.GetDType() != DType::I32 ||
      targetLengths.GetDType() != DType::I32 || targets.GetDType() != DType::I32)
    throw std::invalid_argument("Expected " + std::to_string(batch) + " Int32 input and target lengths and Int32 targets.");
  if (blank < 0 || blank >= classes) throw std::invalid_argument("The blank index " + std::to_string(blank) + " is outside [0, " + std::to_string(classes) + ").");
  Tensor lpc = logProbs.Contiguous();
  Tensor result = NewOut(reduction == 0 ? Shape{batch} : Shape{});
  Tensor nll = Tensor::Create(DType::F32, Shape{batch});
  Check(om_ctc_loss(C(), lpc.Data(), steps, batch, classes, (const int32_t*)targets.RawData(), (const int32_t*)targetLengths.RawData(),
                    (const int32_t*)inputLengths.RawData(), blank, reduction, zeroInfinity, reduction == 0 ? result.Data() : nll.Data(),
                    reduction == 0 ? nullptr : result.Data()));
  if (!Recording({&logProbs})) return result;
  auto br = BackwardRecord::Create(OpKind::CtcLoss, 4, {&logProbs});
  br->Save(0, lpc.Detach());
  br->Save(1, targets);
  br->Save(2, inputLengths);
  br->Save(3, targetLengths);
  br->Ints = {blank, zeroInfinity ? 1 : 0, reduction, batch};
  return br->Attach(result);
}

// Stacked (bi)directional LSTM (src/OneModel.Training/Recurrent.cs:13-67): per layer the forward and reverse
// directions run over the same input and are concatenated on the feature axis.
Recurrent::Recurrent(int input, int hidden, int layers, bool bidirectional, Generator& g)
    : Hidden(hidden), Layers(layers), Bidirectional(bidirectional) {
  Init(input, g);
}

Recurrent::Recurrent(bool gru, int input, int hidden, Generator& g, int layers, bool bidirectional, bool batchFirst)
    : Hidden(hidden), Layers(layers), Bidirectional(bidirectional), Gru(gru), BatchFirst(batchFirst) {
  Init(input, g);
}

void Recurrent::Init(int input, Generator& g) {
  if (input < 1 || Hidden < 1 || Layers < 1) throw ArgumentOutOfRangeException("A recurrent stack needs positive sizes and at least one layer.");
  float bound = 1.0f / sqrtf((float)Hidden);
  int dirs = Bidirectional ? 2 : 1, gates = Gru ? 3 : 4;
  for (int l = 0; l < Layers; l++) {
    int in = l == 0 ? input : Hidden * dirs;
    for (int d = 0; d < dirs; d++) {
      std::string suffix = "_l" + std::to_string(l) + (d ? "_reverse" : "");
      auto init = [&](const Shape& s) {
        std::vector<float> hbuf((size_t)s.Length());
        for (float& v : hbuf) v = g.Uniform(-bound, bound);
        return Tensor::FromHost(hbuf.data(), s);
      };
      WIh.push_back(RegisterParameter("weight_ih" + suffix, init(Shape{gates * Hidden, in})));
      WHh.push_back(RegisterParameter("weight_hh" + suffix, init(Shape{gates * Hidden, Hidden})));
      BIh.push_back(RegisterParameter("bias_ih" + suffix, init(Shape{gates * Hidden})));
      BHh.push_back(RegisterParameter("bias_hh" + suffix, init(Shape{gates * Hidden})));
    }
  }
}

Tensor Recurrent::RunLayer(const Tensor& x, int k, bool reverse) const {
  return Gru ? Ops::GruLayer(x, WIh[k], WHh[k], BIh[k], BHh[k], Tensor(), reverse) : Ops::LstmLayer(x, WIh[k], WHh[k], BIh[k], BHh[k], reverse);
}

Tensor Recurrent::Forward(const Tensor& x, const std::vector<int>& lengths) {
  if (x.Rank() != 3) throw TensorShapeException("A recurrent network needs a rank-3 input, not " + x.GetShape().ToString() + ".");
  Tensor cur = BatchFirst ? x.Transpose(0, 1) : x;
  const int steps = cur.GetShape()[0], batch = cur.GetShape()[1], dirs = Bidirectional ? 2 : 1;
  const bool packed = !lengths.empty();
  Tensor map, mask;
  if (packed) {
    if ((int)lengths.size() != batch) throw std::invalid_argument("Expected " + std::to_string(batch) + " lengths, got " + std::to_string(lengths.size()) + ".");
    // map[t*B+b]: the row of the flattened [T*B] sequence that step t of row b's reversed sequence reads (its own
    // inverse); steps past the row's length stay where they are.
    std::vector<int32_t> idx((size_t)steps * batch);
    std::vector<float> keep((size_t)steps * batch);
    for (int b = 0; b < batch; b++) {
      int len = lengths[(size_t)b];
      if (len < 1 || len > steps)
        throw std::invalid_argument("Length " + std::to_string(len) + " of row " + std::to_string(b) + " is outside [1, " + std::to_string(steps) + "].");
      for (int t = 0; t < steps; t++) {
        idx[(size_t)t * batch + b] = (t < len ? len - 1 - t : t) * batch + b;
        keep[(size_t)t * batch + b] = t < len ? 1.f : 0.f;
      }
    }
    map = Tensor::FromHostInt32(idx.data(), Shape{steps * batch});
    mask = Tensor::FromHost(keep.data(), Shape{steps, batch, 1});
  }
  for (int l = 0; l < Layers; l++) {
    Tensor next;
    if (dirs == 2 && !packed && !Gru) {
      // Both directions in one record: they run concurrently on two streams, forward and backward.
      int k = l * 2;
      next = Ops::LstmBidirectional(cur, {WIh[k], WHh[k], BIh[k], BHh[k], WIh[k + 1], WHh[k + 1], BIh[k + 1], BHh[k + 1]});
    } else {
      next = RunLayer(cur, l * dirs, false);
      if (dirs == 2) {
        Tensor back;
        if (packed) {
          int width = cur.GetShape()[2];
          Tensor rev = Ops::Embedding(cur.Reshape(Shape{steps * batch, width}), map, -1).Reshape(Shape{steps, batch, width});
          Tensor run = RunLayer(rev, l * dirs + 1, false);
          back = Ops::Embedding(run.Reshape(Shape{steps * batch, Hidden}), map, -1).Reshape(Shape{steps, batch, Hidden});
        } else {
          back = RunLayer(cur, l * dirs + 1, true);
        }
        next = Ops::Concat({next, back}, 2);
      }
    }
    if (packed) next = Ops::Mul(next, mask);
    cur = next;
  }
  return BatchFirst ? cur.Transpose(0, 1) : cur;
}

}  // namespace omh
