// Eager forward operations. Each computes on the device through the C ABI and, when an input requires a gradient
// and recording is on, attaches a BackwardRecord with the same saved slots, Ints and Floats as the reference's
// Ops.* (src/OneModel/Tensors/Ops.cs, Ops.Nn.cs, Ops.Layers.cs, Ops.Recurrent.cs, CtcLoss.cs).
#include <math.h>

#include "omh.hpp"

namespace omh {

static om_ctx* C() { return Device::Current(); }

bool Ops::Recording(std::initializer_list<const Tensor*> inputs) {
  if (!GradMode::Enabled()) return false;
  for (const Tensor* t : inputs)
    if (t && !t->IsEmpty() && t->RequiresGrad()) return true;
  return false;
}

// Products with bfloat16 operands (the context's OM_BF16_OPERANDS tier): every operand is read from the bfloat16 copy of
// its storage. The product kernels address operands through TMA, which wants pitches of 16-byte multiples (8 elements)
// and views that start on such a boundary; a Linear that does not fit keeps its fp32 operands.
bool Bf16Products() {
  uint32_t flags = 0;
  Check(om_ctx_get_flags(C(), &flags));
  return (flags & OM_BF16_OPERANDS) != 0 && (flags & OM_TF32) != 0;
}
bool Bf16Operand(const Tensor& t, int64_t pitch) { return t.GetDType() == DType::F32 && pitch % 8 == 0 && t.Offset() % 8 == 0; }

static void RequireFloat32(const Tensor& t) {
  if (t.GetDType() != DType::F32) throw TensorShapeException("A float32 tensor is required.");
}

static Tensor NewOut(const Shape& s) {
  Tensor r = Tensor::Create(DType::F32, s);
  ActivationScope::Track(r);
  return r;
}

// Broadcast shape of a and b, and each operand's strides over it (0 on broadcast axes).
static Shape Broadcast(const Tensor& a, const Tensor& b, std::array<int64_t, kMaxRank>& sa, std::array<int64_t, kMaxRank>& sb) {
  Shape s;
  s.rank = std::max(a.Rank(), b.Rank());
  for (int i = 0; i < s.rank; i++) {
    int ia = i - (s.rank - a.Rank()), ib = i - (s.rank - b.Rank());
    int da = ia >= 0 ? a.GetShape()[ia] : 1, db = ib >= 0 ? b.GetShape()[ib] : 1;
    if (da != db && da != 1 && db != 1)
      throw TensorShapeException("Shapes " + a.GetShape().ToString() + " and " + b.GetShape().ToString() + " do not broadcast.");
    s.d[i] = da == 1 ? db : da;
    sa[i] = (ia >= 0 && da != 1) ? a.Strides()[ia] : 0;
    sb[i] = (ib >= 0 && db != 1) ? b.Strides()[ib] : 0;
  }
  return s;
}

static Tensor Binary(OpKind kind, om_binary_op op, const Tensor& a, const Tensor& b) {
  RequireFloat32(a);
  RequireFloat32(b);
  std::array<int64_t, kMaxRank> sa{}, sb{};
  Shape s = Broadcast(a, b, sa, sb);
  Tensor r = NewOut(s);
  Check(om_binary(C(), op, s.rank, s.d.data(), a.Data(), sa.data(), b.Data(), sb.data(), r.Data()));
  if (!Ops::Recording({&a, &b})) return r;
  bool saves = kind == OpKind::Mul || kind == OpKind::Div;
  auto rec = BackwardRecord::Create(kind, saves ? 2 : 0, {&a, &b});
  if (saves) {
    rec->Save(0, a.Detach());
    rec->Save(1, b.Detach());
  }
  return rec->Attach(r);
}

Tensor Ops::Add(const Tensor& a, const Tensor& b) { return Binary(OpKind::Add, OM_ADD, a, b); }
Tensor Ops::Sub(const Tensor& a, const Tensor& b) { return Binary(OpKind::Sub, OM_SUB, a, b); }
Tensor Ops::Mul(const Tensor& a, const Tensor& b) { return Binary(OpKind::Mul, OM_MUL, a, b); }
Tensor Ops::Div(const Tensor& a, const Tensor& b) { return Binary(OpKind::Div, OM_DIV, a, b); }

// saved: 0 = nothing, 1 = output, 2 = input
static Tensor Unary(OpKind kind, om_unary_op op, const Tensor& x, int saved, std::vector<int64_t> ints = {}) {
  RequireFloat32(x);
  Tensor xc = x.Contiguous();
  Tensor r = NewOut(x.GetShape());
  // The activation between two Linear layers: its result is a product operand, so under bfloat16 products the copy is
  // written here instead of by a cast pass.
  if (kind == OpKind::Gelu && Bf16Products()) {
    Check(om_unary_b16(C(), op, xc.Data(), r.Data(), r.Bf16ForWrite(), r.Length()));
    r.Bf16Written();
  } else {
    Check(om_unary(C(), op, xc.Data(), r.Data(), r.Length()));
  }
  if (!Ops::Recording({&x})) return r;
  auto rec = BackwardRecord::Create(kind, saved ? 1 : 0, {&x});
  if (saved == 1) rec->Save(0, r.Detach());
  if (saved == 2) rec->Save(0, xc.Detach());
  rec->Ints = std::move(ints);
  return rec->Attach(r);
}

Tensor Ops::Neg(const Tensor& x) { return Unary(OpKind::Neg, OM_NEG, x, 0); }
Tensor Ops::Relu(const Tensor& x) { return Unary(OpKind::Relu, OM_RELU, x, 1); }
Tensor Ops::Gelu(const Tensor& x, bool tanhForm) {
  return Unary(OpKind::Gelu, tanhForm ? OM_GELU_TANH : OM_GELU_ERF, x, 2, {tanhForm ? 1 : 0});
}
Tensor Ops::Sigmoid(const Tensor& x) { return Unary(OpKind::Sigmoid, OM_SIGMOID, x, 1); }
Tensor Ops::Tanh(const Tensor& x) { return Unary(OpKind::Tanh, OM_TANH, x, 1); }

// Leading dimension and transposition of a 2-D view that the GEMM can read in place; false if it needs a copy.
static bool GemmLayout(const Tensor& t, int* trans, int* ld) {
  int64_t s0 = t.Strides()[0], s1 = t.Strides()[1];
  int r = t.GetShape()[0], c = t.GetShape()[1];
  if ((s1 == 1 || c == 1) && (s0 >= c || r == 1)) {
    *trans = 0;
    *ld = (int)(r == 1 ? std::max<int64_t>(c, 1) : s0);
    return true;
  }
  if ((s0 == 1 || r == 1) && (s1 >= r || c == 1)) {
    *trans = 1;
    *ld = (int)(c == 1 ? std::max<int64_t>(r, 1) : s1);
    return true;
  }
  return false;
}

Tensor Ops::MatMul(const Tensor& a, const Tensor& b) {
  RequireFloat32(a);
  RequireFloat32(b);
  if (a.Rank() != 2 || b.Rank() != 2 || a.GetShape()[1] != b.GetShape()[0])
    throw TensorShapeException("MatMul needs [M,K] and [K,N], not " + a.GetShape().ToString() + " and " + b.GetShape().ToString());
  int m = a.GetShape()[0], k = a.GetShape()[1], n = b.GetShape()[1];
  Tensor av = a, bv = b;
  int ta, tb, lda, ldb;
  if (!GemmLayout(av, &ta, &lda)) {
    av = a.Contiguous();
    GemmLayout(av, &ta, &lda);
  }
  if (!GemmLayout(bv, &tb, &ldb)) {
    bv = b.Contiguous();
    GemmLayout(bv, &tb, &ldb);
  }
  Tensor r = NewOut(Shape{m, n});
  Check(om_matmul(C(), ta, tb, m, n, k, av.Data(), lda, bv.Data(), ldb, r.Data(), n, 0));
  if (!Recording({&a, &b})) return r;
  auto rec = BackwardRecord::Create(OpKind::MatMul, 2, {&a, &b});
  rec->Save(0, av.Detach());
  rec->Save(1, bv.Detach());
  return rec->Attach(r);
}

static Tensor Reduce(OpKind kind, const Tensor& x, int axis, bool keepDim, bool all) {
  RequireFloat32(x);
  Tensor xc = x.Contiguous();
  int64_t outer = 1, n = xc.Length(), inner = 1;
  int ax = -1;
  Shape os;
  if (!all) {
    ax = axis < 0 ? axis + x.Rank() : axis;
    if (ax < 0 || ax >= x.Rank()) throw TensorShapeException("Axis out of range.");
    n = x.GetShape()[ax];
    for (int i = 0; i < ax; i++) outer *= x.GetShape()[i];
    for (int i = ax + 1; i < x.Rank(); i++) inner *= x.GetShape()[i];
    for (int i = 0; i < x.Rank(); i++) {
      if (i != ax) os.d[os.rank++] = x.GetShape()[i];
      else if (keepDim) os.d[os.rank++] = 1;
    }
  }
  Tensor r = NewOut(os);
  Check(om_reduce_fwd(C(), xc.Data(), outer, n, inner, kind == OpKind::Mean, r.Data()));
  if (!Ops::Recording({&x})) return r;
  auto rec = BackwardRecord::Create(kind, 0, {&x});
  rec->Ints = {all ? -1 : ax, keepDim ? 1 : 0};
  return rec->Attach(r);
}

Tensor Ops::Sum(const Tensor& x) { return Reduce(OpKind::Sum, x, 0, false, true); }
Tensor Ops::Sum(const Tensor& x, int axis, bool keepDim) { return Reduce(OpKind::Sum, x, axis, keepDim, false); }
Tensor Ops::Mean(const Tensor& x) { return Reduce(OpKind::Mean, x, 0, false, true); }
Tensor Ops::Mean(const Tensor& x, int axis, bool keepDim) { return Reduce(OpKind::Mean, x, axis, keepDim, false); }

static Tensor SoftmaxLike(OpKind kind, const Tensor& x, int axis) {
  RequireFloat32(x);
  int ax = axis < 0 ? axis + x.Rank() : axis;
  if (ax != x.Rank() - 1) {
    Tensor t = x.Transpose(ax, x.Rank() - 1);
    Tensor y = kind == OpKind::Softmax ? Ops::Softmax(t, -1) : Ops::LogSoftmax(t, -1);
    return y.Transpose(ax, x.Rank() - 1);
  }
  Tensor xc = x.Contiguous();
  Tensor r = NewOut(x.GetShape());
  int cols = x.GetShape()[ax];
  int rows = cols == 0 ? 0 : (int)(x.Length() / cols);
  if (kind == OpKind::Softmax) Check(om_softmax_fwd(C(), xc.Data(), rows, cols, r.Data()));
  else Check(om_logsoftmax_fwd(C(), xc.Data(), rows, cols, r.Data()));
  if (!Ops::Recording({&x})) return r;
  auto rec = BackwardRecord::Create(kind, 1, {&x});
  rec->Save(0, r.Detach());
  return rec->Attach(r);
}
Tensor Ops::Softmax(const Tensor& x, int axis) { return SoftmaxLike(OpKind::Softmax, x, axis); }
Tensor Ops::LogSoftmax(const Tensor& x, int axis) { return SoftmaxLike(OpKind::LogSoftmax, x, axis); }

Tensor Ops::LayerNorm(const Tensor& x, const Tensor& gamma, const Tensor& beta, float eps) {
  int cols = x.GetShape()[x.Rank() - 1];
  if (gamma.Rank() != 1 || beta.Rank() != 1 || gamma.GetShape()[0] != cols || beta.GetShape()[0] != cols)
    throw TensorShapeException("LayerNorm over " + std::to_string(cols) + " features needs gamma and beta of shape [" +
                               std::to_string(cols) + "], not " + gamma.GetShape().ToString() + " and " + beta.GetShape().ToString() + ".");
  int rows = cols == 0 ? 0 : (int)(x.Length() / cols);
  Tensor xc = x.Contiguous(), gc = gamma.Contiguous(), bc = beta.Contiguous();
  Tensor r = NewOut(x.GetShape());
  bool rec = Recording({&x, &gamma, &beta});
  Tensor mean, inv;
  if (rec) {
    mean = Tensor::Create(DType::F32, Shape{rows});
    inv = Tensor::Create(DType::F32, Shape{rows});
  }
  if (Bf16Products() && cols <= 1024) {
    Check(om_layernorm_fwd_b16(C(), xc.Data(), gc.Data(), bc.Data(), rows, cols, eps, r.Data(), r.Bf16ForWrite(), rec ? mean.Data() : nullptr,
                               rec ? inv.Data() : nullptr));
    r.Bf16Written();
  } else {
    Check(om_layernorm_fwd(C(), xc.Data(), gc.Data(), bc.Data(), rows, cols, eps, r.Data(), rec ? mean.Data() : nullptr,
                           rec ? inv.Data() : nullptr));
  }
  if (!rec) return r;
  auto br = BackwardRecord::Create(OpKind::LayerNorm, 4, {&x, &gamma, &beta});
  br->Save(0, xc.Detach());
  br->Save(1, gc.Detach());
  br->Save(2, mean);
  br->Save(3, inv);
  br->Floats = {eps};
  return br->Attach(r);
}

// LayerNorm(Add(a, b)) with the sum formed inside the layer norm's kernel. The tape holds the same two records as the two
// separate ops (an Add whose result is the sum, a LayerNorm over it), so the backward pass is theirs.
Tensor Ops::AddLayerNorm(const Tensor& a, const Tensor& b, const Tensor& gamma, const Tensor& beta, float eps) {
  const int cols = a.Rank() > 0 ? a.GetShape()[a.Rank() - 1] : 0;
  const bool fused = a.GetDType() == DType::F32 && b.GetDType() == DType::F32 && a.GetShape() == b.GetShape() && a.IsContiguous() && b.IsContiguous() &&
                     cols > 0 && cols <= 1024 && gamma.Rank() == 1 && beta.Rank() == 1 && gamma.GetShape()[0] == cols && beta.GetShape()[0] == cols;
  if (!fused) return LayerNorm(Add(a, b), gamma, beta, eps);
  const int rows = (int)(a.Length() / cols);
  Tensor gc = gamma.Contiguous(), bc = beta.Contiguous();
  Tensor sum = NewOut(a.GetShape()), r = NewOut(a.GetShape());
  const bool rec_add = Recording({&a, &b});
  if (rec_add) sum = BackwardRecord::Create(OpKind::Add, 0, {&a, &b})->Attach(sum);
  const bool rec = Recording({&sum, &gamma, &beta});
  Tensor mean, inv;
  if (rec) {
    mean = Tensor::Create(DType::F32, Shape{rows});
    inv = Tensor::Create(DType::F32, Shape{rows});
  }
  const bool b16 = Bf16Products();
  Check(om_add_layernorm_fwd_b16(C(), a.Data(), b.Data(), sum.Data(), gc.Data(), bc.Data(), rows, cols, eps, r.Data(), b16 ? r.Bf16ForWrite() : nullptr,
                                 rec ? mean.Data() : nullptr, rec ? inv.Data() : nullptr));
  if (b16) r.Bf16Written();
  if (!rec) return r;
  auto br = BackwardRecord::Create(OpKind::LayerNorm, 4, {&sum, &gamma, &beta});
  br->Save(0, sum.Detach());
  br->Save(1, gc.Detach());
  br->Save(2, mean);
  br->Save(3, inv);
  br->Floats = {eps};
  return br->Attach(r);
}

Tensor Ops::BatchNorm2d(const Tensor& x, const Tensor& gamma, const Tensor& beta, const Tensor& runningMean,
                        const Tensor& runningVar, bool training, float momentum, float eps) {
  RequireFloat32(x);
  if (x.Rank() != 4) throw TensorShapeException("BatchNorm2d needs an (N,C,H,W) input, not " + x.GetShape().ToString() + ".");
  int n = x.GetShape()[0], c = x.GetShape()[1], plane = x.GetShape()[2] * x.GetShape()[3];
  for (const Tensor* t : {&gamma, &beta, &runningMean, &runningVar})
    if (t->Rank() != 1 || t->GetShape()[0] != c)
      throw TensorShapeException("BatchNorm2d over " + std::to_string(c) + " channels needs per-channel tensors of shape [" + std::to_string(c) + "].");
  Tensor xc = x.Contiguous(), gc = gamma.Contiguous(), bc = beta.Contiguous();
  Tensor mean = Tensor::Create(DType::F32, Shape{c}), inv = Tensor::Create(DType::F32, Shape{c});
  Tensor r = NewOut(x.GetShape());
  Check(om_batchnorm_fwd(C(), xc.Data(), gc.Data(), bc.Data(), runningMean.Data(), runningVar.Data(), n, c, plane,
                         training, momentum, eps, r.Data(), mean.Data(), inv.Data()));
  if (!Recording({&x, &gamma, &beta})) return r;
  auto br = BackwardRecord::Create(OpKind::BatchNorm, 4, {&x, &gamma, &beta});
  br->Save(0, xc.Detach());
  br->Save(1, gc.Detach());
  br->Save(2, mean);
  br->Save(3, inv);
  br->Ints = {training ? 1 : 0};
  br->Floats = {eps};
  return br->Attach(r);
}

Tensor Ops::Embedding(const Tensor& table, const Tensor& ids, int paddingIndex, bool sparse) {
  RequireFloat32(table);
  if (table.Rank() != 2 || (ids.GetDType() != DType::I32 && ids.GetDType() != DType::I64))
    throw TensorShapeException("Embedding needs a [V, D] float32 table and Int32 or Int64 ids.");
  if (ids.Rank() + 1 > kMaxRank) throw TensorShapeException("Too many dimensions.");
  Tensor tc = table.Contiguous();
  Tensor ic = ids.IsContiguous() ? ids : ids.Clone();
  int v = table.GetShape()[0], dim = table.GetShape()[1];
  Shape os = ids.GetShape();
  os.d[os.rank++] = dim;
  Tensor r = NewOut(os);
  Check(om_embedding_fwd(C(), tc.Data(), v, dim, ic.RawData(), (int32_t)ic.GetDType(), ids.Length(), r.Data()));
  if (!Recording({&table})) return r;
  auto rec = BackwardRecord::Create(OpKind::Embedding, 1, {&table});
  rec->Save(0, ic.Detach());
  rec->Ints = {paddingIndex, sparse ? 1 : 0};
  return rec->Attach(r);
}

Tensor Ops::NllLoss(const Tensor& logProbs, const Tensor& targets, bool mean, int ignoreIndex) {
  RequireFloat32(logProbs);
  if (logProbs.Rank() != 2 || targets.Rank() != 1 || targets.GetShape()[0] != logProbs.GetShape()[0] ||
      (targets.GetDType() != DType::I32 && targets.GetDType() != DType::I64))
    throw TensorShapeException("NllLoss needs [N, C] log-probabilities and [N] Int32 or Int64 targets, not " +
                               logProbs.GetShape().ToString() + " and " + targets.GetShape().ToString() + ".");
  int rows = logProbs.GetShape()[0], cols = logProbs.GetShape()[1];
  Tensor lc = logProbs.Contiguous();
  Tensor tc = targets.IsContiguous() ? targets : targets.Clone();
  Tensor r = NewOut(Shape{});
  Check(om_nll_fwd(C(), lc.Data(), tc.RawData(), (int32_t)tc.GetDType(), rows, cols, mean, ignoreIndex, r.Data(), nullptr));
  if (!Recording({&logProbs})) return r;
  auto rec = BackwardRecord::Create(OpKind::NllLoss, 1, {&logProbs});
  rec->Save(0, tc.Detach());
  rec->Ints = {mean ? 1 : 0, ignoreIndex};
  return rec->Attach(r);
}

Tensor Ops::CrossEntropy(const Tensor& logits, const Tensor& targets, bool mean, int ignoreIndex, float denominator) {
  RequireFloat32(logits);
  if (logits.Rank() != 2 || targets.Rank() != 1 || targets.GetShape()[0] != logits.GetShape()[0] ||
      (targets.GetDType() != DType::I32 && targets.GetDType() != DType::I64))
    throw TensorShapeException("CrossEntropy needs [N, C] logits and [N] Int32 or Int64 targets, not " +
                               logits.GetShape().ToString() + " and " + targets.GetShape().ToString() + ".");
  int rows = logits.GetShape()[0], cols = logits.GetShape()[1];
  Tensor tc = targets.IsContiguous() ? targets : targets.Clone();
  // Row-pitched logits (see Ops::Linear) are read in place; logp and the gradient keep the same pitch.
  int ld = cols;
  Tensor lc;
  if (rows > 1 && logits.Strides()[1] == 1 && logits.Strides()[0] > cols) {
    lc = logits;
    ld = (int)logits.Strides()[0];
  } else {
    lc = logits.Contiguous();
  }
  Tensor logp = ld == cols ? Tensor::Create(DType::F32, logits.GetShape())
                           : Tensor::Create(DType::F32, Shape{rows, ld}).View(logits.GetShape(), {(int64_t)ld, 1}, 0);
  Tensor r = NewOut(Shape{});
  Check(om_cross_entropy_fwd_ld(C(), lc.Data(), tc.RawData(), (int32_t)tc.GetDType(), rows, cols, ld, mean, ignoreIndex,
                                denominator, logp.Data(), r.Data(), nullptr));
  if (!Recording({&logits})) return r;
  auto rec = BackwardRecord::Create(OpKind::CrossEntropy, 2, {&logits});
  rec->Save(0, logp);
  rec->Save(1, tc.Detach());
  rec->Ints = {mean ? 1 : 0, ignoreIndex, ld};
  rec->Floats = {denominator};
  return rec->Attach(r);
}

Tensor Ops::Linear(const Tensor& x, const Tensor& weight, const Tensor& bias) {
  if (weight.Rank() != 2 || x.Rank() < 1 || x.GetShape()[x.Rank() - 1] != weight.GetShape()[1])
    throw TensorShapeException("Linear: input " + x.GetShape().ToString() + " does not fit weights " + weight.GetShape().ToString() + " ([out, in]).");
  int inF = weight.GetShape()[1], outF = weight.GetShape()[0];
  int rows = (int)(x.Length() / std::max(1, inF));
  Tensor xc = x.Contiguous(), wc = weight.Contiguous();
  Tensor bc = bias.IsEmpty() ? Tensor() : bias.Contiguous();
  Shape os = x.GetShape();
  os.d[os.rank - 1] = outF;
  // A wide rank-2 output whose width is not a multiple of four (the vocabulary logits) gets a row pitch that is, so
  // that the backward products can read it with TMA; consumers see an ordinary strided view.
  // (a multiple of eight, so that the bfloat16 copy of the gradient has a 16-byte pitch as well)
  const bool pitched = os.rank == 2 && (outF & 7) != 0 && (int64_t)rows * outF >= (1 << 20);
  const int ld = pitched ? ((outF + 7) & ~7) : outF;
  Tensor r = pitched ? Tensor::Create(DType::F32, Shape{rows, ld}).View(os, {(int64_t)ld, 1}, 0) : NewOut(os);
  if (Bf16Products() && rows > 0 && Bf16Operand(xc, inF) && Bf16Operand(wc, inF) && (ld & 3) == 0)
    Check(om_linear_fwd_bf16(C(), xc.Bf16(), wc.Bf16(), bc.IsEmpty() ? nullptr : bc.Data(), rows, inF, outF, r.Data(), ld));
  else
    Check(om_linear_fwd_ld(C(), xc.Data(), wc.Data(), bc.IsEmpty() ? nullptr : bc.Data(), rows, inF, outF, r.Data(), ld));
  if (!Recording({&x, &weight, &bias})) return r;
  Tensor none;
  auto rec = bias.IsEmpty() ? BackwardRecord::Create(OpKind::Linear, 2, {&x, &weight})
                            : BackwardRecord::Create(OpKind::Linear, 2, {&x, &weight, &bias});
  rec->Save(0, xc.Detach());
  rec->Save(1, wc.Detach());
  rec->Ints = {rows, inF, outF};
  return rec->Attach(r);
}

Tensor Ops::FeedForward(const Tensor& x, const Tensor& w1, const Tensor& b1, const Tensor& w2, const Tensor& b2, bool tanhForm) {
  const int op = tanhForm ? OM_GELU_TANH : OM_GELU_ERF;
  bool fused = Bf16Products() && !b1.IsEmpty() && !b2.IsEmpty() && w1.Rank() == 2 && w2.Rank() == 2 && x.Rank() >= 1 &&
               x.GetDType() == DType::F32 && x.GetShape()[x.Rank() - 1] == w1.GetShape()[1] && w2.GetShape()[1] == w1.GetShape()[0];
  int inF = 0, ff = 0, outF = 0, rows = 0;
  Tensor xc, w1c, w2c;
  if (fused) {
    inF = w1.GetShape()[1], ff = w1.GetShape()[0], outF = w2.GetShape()[0];
    rows = (int)(x.Length() / std::max(1, inF));
    xc = x.Contiguous(), w1c = w1.Contiguous(), w2c = w2.Contiguous();
    fused = rows > 0 && Bf16Operand(xc, inF) && Bf16Operand(w1c, inF) && Bf16Operand(w2c, ff) && (outF & 7) == 0 &&
            om_linear_act_bf16_supported(C(), rows, inF, ff, op, 0) == 1 && om_linear_act_bf16_supported(C(), rows, ff, outF, op, 1) == 1;
  }
  if (!fused) return Linear(Gelu(Linear(x, w1, b1), tanhForm), w2, b2);
  Tensor b1c = b1.Contiguous(), b2c = b2.Contiguous();
  Shape os = x.GetShape();
  os.d[os.rank - 1] = outF;
  // The activation's derivative at the first layer's result (IEEE half: what the backward pass multiplies by; when nothing
  // is recorded it is scratch) and the activation's result as bfloat16 only, each two per 32-bit word of an integer tensor:
  // nothing but the backward epilogue reads the first, nothing but the second product the other.
  Tensor pre = Tensor::Create(DType::I32, Shape{rows, ff / 2});
  Tensor act16 = Tensor::Create(DType::I32, Shape{rows, ff / 2});
  ActivationScope::Track(pre);
  ActivationScope::Track(act16);
  Check(om_linear_fwd_bf16_actd(C(), xc.Bf16(), w1c.Bf16(), b1c.Data(), rows, inF, ff, op, (uint16_t*)pre.RawData(), (uint16_t*)act16.RawData(), ff));
  Tensor r = NewOut(os);
  Check(om_linear_fwd_bf16(C(), (const uint16_t*)act16.RawData(), w2c.Bf16(), b2c.Data(), rows, ff, outF, r.Data(), outF));
  if (!Recording({&x, &w1, &b1, &w2, &b2})) return r;
  auto rec = BackwardRecord::Create(OpKind::FeedForward, 5, {&x, &w1, &b1, &w2, &b2});
  rec->Save(0, xc.Detach());
  rec->Save(1, w1c.Detach());
  rec->Save(2, w2c.Detach());
  rec->Save(3, pre);
  rec->Save(4, act16);
  rec->Ints = {rows, inF, ff, outF, op};
  return rec->Attach(r);
}

Tensor Ops::Attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, float scale) {
  if (q.Rank() != 4 || k.Rank() != 4 || v.Rank() != 4 || k.GetShape() != v.GetShape() || q.GetShape()[0] != k.GetShape()[0] ||
      q.GetShape()[1] != k.GetShape()[1] || q.GetShape()[3] != k.GetShape()[3] || q.GetShape()[3] % 2 != 0)
    throw TensorShapeException("Attention needs [B,H,L,D] tensors with matching batch, heads and even D, not " +
                               q.GetShape().ToString() + ", " + k.GetShape().ToString() + ", " + v.GetShape().ToString() + ".");
  int b = q.GetShape()[0], h = q.GetShape()[1], lq = q.GetShape()[2], lk = k.GetShape()[2], d = q.GetShape()[3];
  int64_t maskStride = 0;
  Tensor mc;
  if (!mask.IsEmpty()) {
    RequireFloat32(mask);
    bool ok = (mask.Rank() == 2 && mask.GetShape()[0] == lq && mask.GetShape()[1] == lk) ||
              (mask.Rank() == 3 && mask.GetShape()[0] == b && mask.GetShape()[1] == lq && mask.GetShape()[2] == lk);
    if (!ok) throw TensorShapeException("The mask must be [" + std::to_string(lq) + "," + std::to_string(lk) + "] or [" +
                                        std::to_string(b) + "," + std::to_string(lq) + "," + std::to_string(lk) + "], not " + mask.GetShape().ToString() + ".");
    mc = mask.Contiguous().Detach();
    maskStride = mask.Rank() == 2 ? 0 : (int64_t)lq * lk;
  }
  if (scale == 0.f || isnan(scale)) scale = 1.0f / sqrtf((float)d);
  Tensor qc = q.Contiguous(), kc = k.Contiguous(), vc = v.Contiguous();
  Tensor r = NewOut(q.GetShape());
  const bool recording = Recording({&q, &k, &v});
  Tensor lse = recording ? Tensor::Create(DType::F32, Shape{b, h, lq}) : Tensor();   // row log-sum-exp, kept for the backward
  Check(om_attention_fwd(C(), qc.Data(), kc.Data(), vc.Data(), mc.IsEmpty() ? nullptr : mc.Data(), maskStride, b, h, lq, lk,
                         d, scale, r.Data(), lse.IsEmpty() ? nullptr : lse.Data()));
  if (!recording) return r;
  auto rec = BackwardRecord::Create(OpKind::Attention, 6, {&q, &k, &v});
  rec->Save(4, lse);
  rec->Save(5, r.Detach());   // the output: the backward takes the row dots from rowsum(dO O)
  rec->Save(0, qc.Detach());
  rec->Save(1, kc.Detach());
  rec->Save(2, vc.Detach());
  if (!mc.IsEmpty()) rec->Save(3, mc);
  rec->Floats = {scale};
  rec->Ints = {maskStride};
  return rec->Attach(r);
}

// Row-pitched [B, L, D] activation (innermost stride 1, row stride >= D) usable in place, else a contiguous clone.
static Tensor HeadsOperand(const Tensor& t) {
  const auto& st = t.Strides();
  if (t.GetShape()[2] > 0 && st[2] == 1 && st[1] >= t.GetShape()[2] && st[0] >= 0) return t;
  return t.Contiguous();
}
static om_head_strides HeadStridesOf(const Tensor& t, int dh) { return om_head_strides{t.Strides()[0], (int64_t)dh, t.Strides()[1]}; }

// Attention over activations that are still [batch, length, heads * d]: the Reshape + Permute(0, 2, 1, 3) pairs that
// MultiHeadAttention.Forward (Layers.cs:503-520 of the reference) wraps around Ops.Attention are folded into the
// kernels' addressing, forward and backward, so the four head-split copies and their four inverse copies per layer
// disappear. Same arithmetic per (batch, head) as Ops::Attention.
Tensor Ops::AttentionHeads(const Tensor& q, const Tensor& k, const Tensor& v, int heads, const Tensor& mask, float scale) {
  if (q.Rank() != 3 || k.Rank() != 3 || v.Rank() != 3 || k.GetShape() != v.GetShape() || q.GetShape()[0] != k.GetShape()[0] ||
      q.GetShape()[2] != k.GetShape()[2] || heads < 1 || q.GetShape()[2] % heads != 0 || (q.GetShape()[2] / heads) % 2 != 0)
    throw TensorShapeException("Attention over heads needs [B,L,H*D] tensors with matching batch and width and even D, not " +
                               q.GetShape().ToString() + ", " + k.GetShape().ToString() + ", " + v.GetShape().ToString() + ".");
  RequireFloat32(q);
  RequireFloat32(k);
  RequireFloat32(v);
  int b = q.GetShape()[0], lq = q.GetShape()[1], lk = k.GetShape()[1], width = q.GetShape()[2], d = width / heads;
  int64_t maskStride = 0;
  Tensor mc;
  if (!mask.IsEmpty()) {
    RequireFloat32(mask);
    bool ok = (mask.Rank() == 2 && mask.GetShape()[0] == lq && mask.GetShape()[1] == lk) ||
              (mask.Rank() == 3 && mask.GetShape()[0] == b && mask.GetShape()[1] == lq && mask.GetShape()[2] == lk);
    if (!ok) throw TensorShapeException("The mask must be [" + std::to_string(lq) + "," + std::to_string(lk) + "] or [" +
                                        std::to_string(b) + "," + std::to_string(lq) + "," + std::to_string(lk) + "], not " + mask.GetShape().ToString() + ".");
    mc = mask.Contiguous().Detach();
    maskStride = mask.Rank() == 2 ? 0 : (int64_t)lq * lk;
  }
  if (scale == 0.f || isnan(scale)) scale = 1.0f / sqrtf((float)d);
  Tensor qc = HeadsOperand(q), kc = HeadsOperand(k), vc = HeadsOperand(v);
  Tensor r = NewOut(q.GetShape());
  om_head_strides qs = HeadStridesOf(qc, d), ks = HeadStridesOf(kc, d), vs = HeadStridesOf(vc, d), os = HeadStridesOf(r, d);
  const bool recording = Recording({&q, &k, &v});
  Tensor lse = recording ? Tensor::Create(DType::F32, Shape{b, heads, lq}) : Tensor();
  Check(om_attention_fwd_strided(C(), qc.Data(), &qs, kc.Data(), &ks, vc.Data(), &vs, mc.IsEmpty() ? nullptr : mc.Data(), maskStride,
                                 b, heads, lq, lk, d, scale, r.Data(), &os, lse.IsEmpty() ? nullptr : lse.Data()));
  if (!recording) return r;
  auto rec = BackwardRecord::Create(OpKind::Attention, 6, {&q, &k, &v});
  rec->Save(4, lse);
  rec->Save(5, r.Detach());   // the output: the backward takes the row dots from rowsum(dO O)
  rec->Save(0, qc.Detach());
  rec->Save(1, kc.Detach());
  rec->Save(2, vc.Detach());
  if (!mc.IsEmpty()) rec->Save(3, mc);
  rec->Floats = {scale};
  rec->Ints = {maskStride, heads};
  return rec->Attach(r);
}

bool Ops::Adjacent(const std::vector<Tensor>& parts) {
  for (size_t i = 0; i < parts.size(); i++) {
    if (parts[i].IsEmpty() || !parts[i].IsContiguous() || parts[i].GetDType() != DType::F32) return false;
    if (i > 0 && parts[i].Data() != parts[i - 1].Data() + parts[i - 1].Length()) return false;
  }
  return !parts.empty();
}

Tensor Ops::LinearPacked(const Tensor& x, const std::vector<Tensor>& weights, const std::vector<Tensor>& biases, bool bf16_only_result) {
  if (weights.empty() || weights.size() > 3 || (!biases.empty() && biases.size() != weights.size()))
    throw TensorShapeException("LinearPacked needs one to three weight matrices and as many biases (or none).");
  if (!Adjacent(weights) || (!biases.empty() && !Adjacent(biases)))
    throw InvalidOperationException("LinearPacked: the parameters are not adjacent in memory.");
  int inF = weights[0].GetShape()[1], outF = 0;
  for (size_t i = 0; i < weights.size(); i++) {
    if (weights[i].Rank() != 2 || weights[i].GetShape()[1] != inF || (!biases.empty() && biases[i].Length() != weights[i].GetShape()[0]))
      throw TensorShapeException("LinearPacked: the weight matrices must share the input width and match their biases.");
    outF += weights[i].GetShape()[0];
  }
  if (x.Rank() < 1 || x.GetShape()[x.Rank() - 1] != inF)
    throw TensorShapeException("Linear: input " + x.GetShape().ToString() + " does not fit weights [" + std::to_string(outF) + "," + std::to_string(inF) + "] ([out, in]).");
  int rows = (int)(x.Length() / std::max(1, inF));
  Tensor xc = x.Contiguous();
  Shape os = x.GetShape();
  os.d[os.rank - 1] = outF;
  const bool route16 = Bf16Products() && rows > 0 && Bf16Operand(xc, inF) && Bf16Operand(weights[0], inF) && (outF & 3) == 0;
  bool parts8 = (inF % 8) == 0;
  for (auto& w : weights) parts8 = parts8 && (w.GetShape()[0] % 8) == 0;
  // Without an fp32 result the product may not split k (the slices are summed in fp32): the same rule the kernel applies.
  const bool only16 = bf16_only_result && route16 && parts8 && om_linear_act_bf16_supported(C(), rows, inF, outF, OM_GELU_ERF, 0) == 1;
  Tensor r = only16 ? Tensor::CreateBf16Only(os) : NewOut(os);
  if (only16) {
    ActivationScope::Track(r);
    Check(om_linear_fwd_bf16_b16(C(), xc.Bf16(), weights[0].Bf16(), biases.empty() ? nullptr : biases[0].Data(), rows, inF, outF, nullptr, r.Bf16ForWrite(), outF));
  } else if (route16) {
    // The packed q | k | v projections feed the attention kernels, which read them as bfloat16 under this tier: the
    // product's epilogue writes that copy along.
    uint16_t* y16 = outF % 8 == 0 ? r.Bf16ForWrite() : nullptr;
    Check(om_linear_fwd_bf16_b16(C(), xc.Bf16(), weights[0].Bf16(), biases.empty() ? nullptr : biases[0].Data(), rows, inF, outF, r.Data(), y16, outF));
    if (y16) r.Bf16Written();
  } else
    Check(om_linear_fwd_ld(C(), xc.Data(), weights[0].Data(), biases.empty() ? nullptr : biases[0].Data(), rows, inF, outF, r.Data(), outF));
  std::vector<Tensor> ins = {x};
  for (auto& w : weights) ins.push_back(w);
  for (auto& b : biases) ins.push_back(b);
  bool rec_needed = false;
  for (auto& t : ins) rec_needed = rec_needed || t.RequiresGrad();
  if (!GradMode::Enabled() || !rec_needed) return r;
  auto rec = BackwardRecord::Create(OpKind::Linear, 1 + (int)weights.size(), ins);
  rec->Save(0, xc.Detach());
  for (size_t i = 0; i < weights.size(); i++) rec->Save(1 + (int)i, weights[i].Detach());
  rec->Ints = {rows, inF, outF, (int64_t)weights.size(), biases.empty() ? 0 : 1};
  // On the bfloat16 route every gradient this record computes reads the bfloat16 copy of the incoming gradient.
  rec->TakesBf16OnlyGrad = route16 && parts8;
  return rec->Attach(r);
}

bool Ops::AttentionPackedReadsBf16Only(const Tensor& input, int width, int heads) {
  if (!Bf16Products() || input.Rank() != 3 || heads < 1 || width % heads != 0 || width % 8 != 0) return false;
  const int b = input.GetShape()[0], l = input.GetShape()[1], d = width / heads;
  const float scale = 1.0f / sqrtf((float)d);
  return l > 128 && om_attention_fwd_bf16_supported(C(), b, heads, l, l, d, scale) == 1 && om_attention_bwd_bf16_supported(C(), b, heads, l, l, d) == 1;
}

Tensor Ops::AttentionPacked(const Tensor& qkv, int heads, const Tensor& mask, float scale) {
  if (qkv.Rank() != 3 || heads < 1 || qkv.GetShape()[2] % (3 * heads) != 0 || (qkv.GetShape()[2] / (3 * heads)) % 2 != 0)
    throw TensorShapeException("Packed attention needs [B, L, 3*H*D] with even D, not " + qkv.GetShape().ToString() + ".");
  RequireFloat32(qkv);
  int b = qkv.GetShape()[0], l = qkv.GetShape()[1], width = qkv.GetShape()[2] / 3, d = width / heads;
  int64_t maskStride = 0;
  Tensor mc;
  if (!mask.IsEmpty()) {
    RequireFloat32(mask);
    bool ok = (mask.Rank() == 2 && mask.GetShape()[0] == l && mask.GetShape()[1] == l) ||
              (mask.Rank() == 3 && mask.GetShape()[0] == b && mask.GetShape()[1] == l && mask.GetShape()[2] == l);
    if (!ok) throw TensorShapeException("The mask must be [" + std::to_string(l) + "," + std::to_string(l) + "] or [" +
                                        std::to_string(b) + "," + std::to_string(l) + "," + std::to_string(l) + "], not " + mask.GetShape().ToString() + ".");
    mc = mask.Contiguous().Detach();
    maskStride = mask.Rank() == 2 ? 0 : (int64_t)l * l;
  }
  if (scale == 0.f || isnan(scale)) scale = 1.0f / sqrtf((float)d);
  Tensor pc = qkv.Contiguous();
  Tensor r = NewOut(Shape{b, l, width});
  om_head_strides ps{(int64_t)l * 3 * width, (int64_t)d, (int64_t)3 * width}, os{(int64_t)l * width, (int64_t)d, (int64_t)width};
  const bool recording = Recording({&qkv});
  Tensor lse = recording ? Tensor::Create(DType::F32, Shape{b, heads, l}) : Tensor();
  // Under bfloat16 products a sequence of several tiles runs on the bfloat16 forward: it reads the copy of q | k | v that the
  // packed projection wrote and writes the copy of its result that the output projection reads.
  if (Bf16Products() && l > 128 && Bf16Operand(pc, 3 * width) && width % 8 == 0 && om_attention_fwd_bf16_supported(C(), b, heads, l, l, d, scale) == 1) {
    const uint16_t* p16 = pc.Bf16();
    Check(om_attention_fwd_bf16(C(), p16, &ps, p16 + width, &ps, p16 + 2 * width, &ps, mc.IsEmpty() ? nullptr : mc.Data(), maskStride, b, heads, l, l, d,
                                scale, r.Data(), r.Bf16ForWrite(), &os, lse.IsEmpty() ? nullptr : lse.Data()));
    r.Bf16Written();
  } else {
    Check(om_attention_fwd_strided(C(), pc.Data(), &ps, pc.Data() + width, &ps, pc.Data() + 2 * width, &ps, mc.IsEmpty() ? nullptr : mc.Data(),
                                   maskStride, b, heads, l, l, d, scale, r.Data(), &os, lse.IsEmpty() ? nullptr : lse.Data()));
  }
  if (!recording) return r;
  auto rec = BackwardRecord::Create(OpKind::Attention, 6, {&qkv});
  rec->Save(4, lse);
  rec->Save(5, r.Detach());
  rec->Save(0, pc.Detach());
  if (!mc.IsEmpty()) rec->Save(3, mc);
  rec->Floats = {scale};
  rec->Ints = {maskStride, heads, 1};
  return rec->Attach(r);
}

Tensor Ops::Concat(const std::vector<Tensor>& xs, int axis) {
  if (xs.empty()) throw TensorShapeException("Concat needs at least one tensor.");
  int rank = xs[0].Rank();
  int ax = axis < 0 ? axis + rank : axis;
  Shape os = xs[0].GetShape();
  int total = 0;
  for (const Tensor& t : xs) {
    RequireFloat32(t);
    if (t.Rank() != rank) throw TensorShapeException("Concat needs tensors of one rank.");
    for (int i = 0; i < rank; i++)
      if (i != ax && t.GetShape()[i] != os[i]) throw TensorShapeException("Concat: shapes differ off the axis.");
    total += t.GetShape()[ax];
  }
  os.d[ax] = total;
  Tensor r = NewOut(os);
  int start = 0;
  bool any = false;
  for (const Tensor& t : xs) {
    int len = t.GetShape()[ax];
    Tensor dst = r.Slice(ax, start, start + len);
    Check(om_strided_copy(C(), rank, t.GetShape().d.data(), t.Data(), t.Strides().data(), dst.Data(), dst.Strides().data()));
    start += len;
    any = any || t.RequiresGrad();
  }
  if (!GradMode::Enabled() || !any) return r;
  auto rec = BackwardRecord::Create(OpKind::Concat, 0, xs);
  rec->Ints = {ax};
  return rec->Attach(r);
}

Tensor Ops::GlobalAvgPool2d(const Tensor& x) {
  if (x.Rank() != 4) throw TensorShapeException("GlobalAvgPool2d needs an (N,C,H,W) input.");
  int n = x.GetShape()[0], c = x.GetShape()[1], plane = x.GetShape()[2] * x.GetShape()[3];
  // Mean over the flattened plane, kept as [N, C, 1, 1] like the reference (Ops.Layers.cs:463-478).
  Tensor flat = x.Reshape(Shape{n, c, plane});
  return Mean(flat, 2, false).Reshape(Shape{n, c, 1, 1});
}

}  // namespace omh
