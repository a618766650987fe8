// The graph-op family of the reference (Ops.GraphOps.cs) and its backward functions (BackwardGraphOps.cs): batched matrix
// product with broadcast batch axes, Erf / Exp / Sqrt / Pow, Where, Gather.
#include <math.h>

#include "omh.hpp"

namespace omh {

static om_ctx* Ctx() { return Device::Current(); }

static void RequireF32(const Tensor& t) {
  if (t.GetDType() != DType::F32) throw TensorShapeException("A float32 tensor is required.");
}

static Tensor UnaryGraph(OpKind kind, om_unary_op op, const Tensor& x, bool saveOutput) {
  RequireF32(x);
  Tensor xc = x.Contiguous();
  Tensor r = Tensor::Create(DType::F32, x.GetShape());
  Check(om_unary(Ctx(), op, xc.Data(), r.Data(), r.Length()));
  if (!Ops::Recording({&x})) return r;
  auto rec = BackwardRecord::Create(kind, 1, {&x});
  rec->Save(0, saveOutput ? r.Detach() : xc.Detach());
  return rec->Attach(r);
}

// Erf saves its input, Exp and Sqrt their output (Ops.GraphOps.cs:125-172).
Tensor Ops::Erf(const Tensor& x) { return UnaryGraph(OpKind::Erf, OM_ERF, x, false); }
Tensor Ops::Exp(const Tensor& x) { return UnaryGraph(OpKind::Exp, OM_EXP, x, true); }
Tensor Ops::Sqrt(const Tensor& x) { return UnaryGraph(OpKind::Sqrt, OM_SQRT, x, true); }

Tensor Ops::Pow(const Tensor& x, float exponent) {
  RequireF32(x);
  Tensor xc = x.Contiguous();
  Tensor r = Tensor::Create(DType::F32, x.GetShape());
  Check(om_pow(Ctx(), xc.Data(), exponent, r.Data(), r.Length()));
  if (!Recording({&x})) return r;
  auto rec = BackwardRecord::Create(OpKind::Pow, 1, {&x});
  rec->Save(0, xc.Detach());
  rec->Floats = {exponent};
  return rec->Attach(r);
}

// Dropout: the record keeps the call number the forward used (a device Int64 [1] written by the kernel), not the mask;
// the backward forms the mask bits again from it.
Tensor Ops::Dropout(const Tensor& x, float p, uint64_t seed, const Tensor& draws) {
  RequireF32(x);
  if (!(p >= 0.f && p < 1.f)) throw ArgumentOutOfRangeException("Dropout probability must be in [0, 1).");
  if (draws.GetDType() != DType::I64 || draws.Length() != 1) throw TensorShapeException("The draw counter must be Int64 [1].");
  Tensor xc = x.Contiguous();
  Tensor r = Tensor::Create(DType::F32, x.GetShape());
  bool record = Recording({&x});
  Tensor used = record ? Tensor::Create(DType::I64, Shape{1}) : Tensor();
  Check(om_dropout_fwd(Ctx(), xc.Data(), r.Length(), p, seed, (int64_t*)draws.RawData(), record ? (int64_t*)used.RawData() : nullptr,
                       r.Data(), nullptr));
  if (!record) return r;
  auto rec = BackwardRecord::Create(OpKind::Dropout, 1, {&x});
  rec->Save(0, used);
  rec->Floats = {p};
  rec->Ints = {(int64_t)seed};
  return rec->Attach(r);
}

static Shape BroadcastShapes(const Shape& a, const Shape& b) {
  Shape s;
  s.rank = std::max(a.rank, b.rank);
  for (int i = 0; i < s.rank; i++) {
    int ia = i - (s.rank - a.rank), ib = i - (s.rank - b.rank);
    int da = ia >= 0 ? a.d[ia] : 1, db = ib >= 0 ? b.d[ib] : 1;
    if (da != db && da != 1 && db != 1) throw TensorShapeException("Shapes " + a.ToString() + " and " + b.ToString() + " do not broadcast.");
    s.d[i] = da == 1 ? db : da;
  }
  return s;
}

// condition is Int32 (non-zero = true): the device ABI has no one-byte tensor type.
Tensor Ops::Where(const Tensor& condition, const Tensor& x, const Tensor& y) {
  RequireF32(x);
  RequireF32(y);
  if (condition.IsEmpty() || condition.GetDType() != DType::I32) throw std::invalid_argument("Where needs an Int32 condition (non-zero = true).");
  Shape s = BroadcastShapes(BroadcastShapes(condition.GetShape(), x.GetShape()), y.GetShape());
  Tensor cc, xc, yc;
  {
    GradMode::NoGrad ng;
    cc = condition.Expand(s).Contiguous();
    xc = x.Expand(s).Contiguous();
    yc = y.Expand(s).Contiguous();
  }
  Tensor r = Tensor::Create(DType::F32, s);
  Check(om_where(Ctx(), (const int32_t*)cc.RawData(), xc.Data(), yc.Data(), r.Data(), r.Length()));
  if (!Recording({&x, &y})) return r;
  auto rec = BackwardRecord::Create(OpKind::Where, 1, {&condition, &x, &y});
  rec->Save(0, cc.Detach());
  return rec->Attach(r);
}

Tensor Ops::Gather(const Tensor& data, const Tensor& indices, int axis) {
  RequireF32(data);
  if (indices.IsEmpty() || (indices.GetDType() != DType::I32 && indices.GetDType() != DType::I64))
    throw std::invalid_argument("Gather needs Int32 or Int64 indices.");
  int ax = axis < 0 ? axis + data.Rank() : axis;
  if (ax < 0 || ax >= data.Rank()) throw TensorShapeException("Gather: axis out of range.");
  if (data.Rank() - 1 + indices.Rank() > kMaxRank) throw TensorShapeException("The gathered tensor would exceed the maximum rank.");
  Shape os;
  int64_t outer = 1, inner = 1, n = data.GetShape()[ax];
  for (int i = 0; i < ax; i++) { os.d[os.rank++] = data.GetShape()[i]; outer *= data.GetShape()[i]; }
  for (int i = 0; i < indices.Rank(); i++) os.d[os.rank++] = indices.GetShape()[i];
  for (int i = ax + 1; i < data.Rank(); i++) { os.d[os.rank++] = data.GetShape()[i]; inner *= data.GetShape()[i]; }
  Tensor dc = data.Contiguous();
  Tensor ic = indices.IsContiguous() ? indices : indices.Clone();
  Tensor r = Tensor::Create(DType::F32, os);
  Check(om_gather_fwd(Ctx(), dc.Data(), ic.RawData(), (int32_t)ic.GetDType(), outer, ic.Length(), n, inner, r.Data()));
  if (!Recording({&data})) return r;
  auto rec = BackwardRecord::Create(OpKind::Gather, 1, {&data});
  rec->Save(0, ic.Detach());
  rec->Ints = {ax};
  return rec->Attach(r);
}

// Flattens the batch axes of a contiguous [..., r, c] tensor: count and matrix size.
static int64_t BatchOf(const Tensor& t) {
  int64_t b = 1;
  for (int i = 0; i < t.Rank() - 2; i++) b *= t.GetShape()[i];
  return b;
}

// c[batch] = op(a[batch]) op(b[batch]) on contiguous operands with equal batch axes.
static void BatchedProduct(const Tensor& a, bool ta, const Tensor& b, bool tb, Tensor& c) {
  int64_t batch = BatchOf(c);
  int m = c.GetShape()[c.Rank() - 2], n = c.GetShape()[c.Rank() - 1];
  int k = ta ? a.GetShape()[a.Rank() - 2] : a.GetShape()[a.Rank() - 1];
  int lda = a.GetShape()[a.Rank() - 1], ldb = b.GetShape()[b.Rank() - 1];
  int64_t sa = (int64_t)a.GetShape()[a.Rank() - 2] * lda, sb = (int64_t)b.GetShape()[b.Rank() - 2] * ldb;
  for (int64_t z0 = 0; z0 < batch; z0 += 65535) {
    int nb = (int)std::min<int64_t>(65535, batch - z0);
    Check(om_matmul_batched(Ctx(), ta, tb, m, n, k, a.Data() + z0 * sa, lda, sa, b.Data() + z0 * sb, ldb, sb, c.Data() + z0 * (int64_t)m * n, n,
                            (int64_t)m * n, nb, 0));
  }
}

Tensor Ops::MatMulBatched(const Tensor& a, const Tensor& b) {
  RequireF32(a);
  RequireF32(b);
  if (a.Rank() < 2 || b.Rank() < 2) throw TensorShapeException("MatMulBatched needs rank 2 or more, not " + a.GetShape().ToString() + " and " + b.GetShape().ToString() + ".");
  int m = a.GetShape()[a.Rank() - 2], k = a.GetShape()[a.Rank() - 1], n = b.GetShape()[b.Rank() - 1];
  if (b.GetShape()[b.Rank() - 2] != k) throw TensorShapeException("Cannot multiply " + a.GetShape().ToString() + " by " + b.GetShape().ToString() + ".");
  if (b.Rank() == 2) {
    if (a.Rank() == 2) return MatMul(a, b);
    // Rows of every batch share the one right operand: a single product over the flattened rows.
    Tensor flat = MatMul(a.Reshape(Shape{(int)(a.Length() / std::max(1, k)), k}), b);
    Shape os = a.GetShape();
    os.d[os.rank - 1] = n;
    return flat.Reshape(os);
  }
  int rank = std::max(a.Rank(), b.Rank());
  Shape sa, sb, so;
  sa.rank = sb.rank = so.rank = rank;
  for (int i = 0; i < rank - 2; i++) {
    int ia = i - (rank - a.Rank()), ib = i - (rank - b.Rank());
    int da = ia >= 0 ? a.GetShape()[ia] : 1, db = ib >= 0 ? b.GetShape()[ib] : 1;
    if (da != db && da != 1 && db != 1)
      throw TensorShapeException("The batch axes of " + a.GetShape().ToString() + " and " + b.GetShape().ToString() + " do not broadcast.");
    sa.d[i] = sb.d[i] = so.d[i] = da == 1 ? db : da;
  }
  sa.d[rank - 2] = m; sa.d[rank - 1] = k;
  sb.d[rank - 2] = k; sb.d[rank - 1] = n;
  so.d[rank - 2] = m; so.d[rank - 1] = n;
  Tensor ae, be;
  {
    GradMode::NoGrad ng;
    ae = a.Expand(sa).Contiguous();
    be = b.Expand(sb).Contiguous();
  }
  Tensor r = Tensor::Create(DType::F32, so);
  BatchedProduct(ae, false, be, false, r);
  if (!Recording({&a, &b})) return r;
  auto rec = BackwardRecord::Create(OpKind::BatchMatMul, 2, {&a, &b});
  if (b.RequiresGrad()) rec->Save(0, ae.Detach());
  if (a.RequiresGrad()) rec->Save(1, be.Detach());
  return rec->Attach(r);
}

// The convolution whose adjoint the transposed convolution is: input = the transposed convolution's OUTPUT
// [N, Cout, OH, OW], output = its input [N, Cin, H, W], weights as they are ([Cin, Cout/G, KH, KW] is [conv out, conv in / G]).
static om_conv_shape AdjointShape(const Shape& xs, const Shape& ws, int oh, int ow, const ConvTranspose2dParams& p) {
  om_conv_shape s;
  s.n = xs.d[0]; s.cin = ws.d[1] * p.groups; s.h = oh; s.w = ow; s.cout = xs.d[1]; s.kh = ws.d[2]; s.kw = ws.d[3];
  s.stride_h = p.strideH; s.stride_w = p.strideW; s.pad_top = p.padH; s.pad_left = p.padW; s.pad_bottom = p.padH; s.pad_right = p.padW;
  s.dil_h = p.dilH; s.dil_w = p.dilW; s.groups = p.groups;
  return s;
}

// The reference runs Conv1d on its 2-D kernels with a height of 1 and differentiates it with the 2-D backward on the
// height-1 view; here the views are explicit (reshapes are free and differentiable) and Conv2d does the rest, so forward,
// dx, dW and dbias are exactly those of the 2-D path.
Tensor Ops::Conv1d(const Tensor& x, const Tensor& weight, const Tensor& bias, const Conv1dParams& p0) {
  RequireF32(x);
  RequireF32(weight);
  Conv1dParams p = p0;
  if (p.stride == 0) p.stride = 1;
  if (p.dilation == 0) p.dilation = 1;
  if (p.groups == 0) p.groups = 1;
  if (x.Rank() != 3 || weight.Rank() != 3)
    throw TensorShapeException("Conv1d needs an (N,C,L) input and (O,I,K) weights, not " + x.GetShape().ToString() + " and " +
                               weight.GetShape().ToString() + ".");
  if (p.groups < 1 || x.GetShape()[1] % p.groups != 0 || weight.GetShape()[0] % p.groups != 0 ||
      weight.GetShape()[1] != x.GetShape()[1] / p.groups)
    throw TensorShapeException("Weights " + weight.GetShape().ToString() + " do not fit input " + x.GetShape().ToString() + " with " +
                               std::to_string(p.groups) + " groups.");
  if (!bias.IsEmpty() && (bias.Rank() != 1 || bias.GetShape()[0] != weight.GetShape()[0]))
    throw TensorShapeException("The bias must have shape [" + std::to_string(weight.GetShape()[0]) + "], not " + bias.GetShape().ToString() + ".");
  const int n = x.GetShape()[0], c = x.GetShape()[1], l = x.GetShape()[2], o = weight.GetShape()[0], k = weight.GetShape()[2];
  const long long span = (long long)p.dilation * (k - 1) + 1;
  const long long outw = p.stride >= 1 ? ((long long)l + p.padLeft + p.padRight - span) / p.stride + 1 : 0;
  if (p.stride < 1 || p.dilation < 1 || p.padLeft < 0 || p.padRight < 0 || (long long)l + p.padLeft + p.padRight < span || outw < 1)
    throw TensorShapeException("Invalid convolution geometry for input " + x.GetShape().ToString() + " and kernel " + weight.GetShape().ToString() + ".");
  Conv2dParams q;
  q.strideH = 1; q.strideW = p.stride;
  q.padTop = 0; q.padBottom = 0; q.padLeft = p.padLeft; q.padRight = p.padRight;
  q.dilH = 1; q.dilW = p.dilation; q.groups = p.groups;
  Tensor y = Conv2d(x.Reshape(Shape{n, c, 1, l}), weight.Reshape(Shape{o, weight.GetShape()[1], 1, k}), bias, q);
  return y.Reshape(Shape{n, o, y.GetShape()[3]});
}

Tensor Ops::ConvTranspose2d(const Tensor& x, const Tensor& weight, const Tensor& bias, const ConvTranspose2dParams& p) {
  RequireF32(x);
  RequireF32(weight);
  if (x.Rank() != 4 || weight.Rank() != 4 || p.groups < 1 || x.GetShape()[1] != weight.GetShape()[0] || x.GetShape()[1] % p.groups != 0)
    throw TensorShapeException("ConvTranspose2d needs an (N,C,H,W) input and (Cin,Cout/G,KH,KW) weights, not " + x.GetShape().ToString() +
                               " and " + weight.GetShape().ToString() + ".");
  if (p.strideH < 1 || p.strideW < 1 || p.dilH < 1 || p.dilW < 1 || p.padH < 0 || p.padW < 0 || p.outPadH < 0 || p.outPadW < 0 ||
      p.outPadH >= p.strideH || p.outPadW >= p.strideW)
    throw TensorShapeException("ConvTranspose2d: invalid stride, padding, output padding or dilation.");
  int cout = weight.GetShape()[1] * p.groups;
  int oh = (x.GetShape()[2] - 1) * p.strideH - 2 * p.padH + p.dilH * (weight.GetShape()[2] - 1) + p.outPadH + 1;
  int ow = (x.GetShape()[3] - 1) * p.strideW - 2 * p.padW + p.dilW * (weight.GetShape()[3] - 1) + p.outPadW + 1;
  if (oh < 1 || ow < 1) throw TensorShapeException("ConvTranspose2d: the output would be empty.");
  if (!bias.IsEmpty() && (bias.Rank() != 1 || bias.GetShape()[0] != cout)) throw TensorShapeException("ConvTranspose2d: the bias must be [Cout].");
  Tensor xc = x.Contiguous(), wc = weight.Contiguous();
  om_conv_shape s = AdjointShape(x.GetShape(), weight.GetShape(), oh, ow, p);
  Tensor r = Tensor::Create(DType::F32, Shape{x.GetShape()[0], cout, oh, ow});
  Check(om_conv2d_dgrad(Ctx(), &s, xc.Data(), wc.Data(), r.Data()));
  if (!bias.IsEmpty()) {
    GradMode::NoGrad ng;
    r = Ops::Add(r, bias.Detach().Reshape(Shape{1, cout, 1, 1}));
  }
  if (!Recording({&x, &weight, &bias})) return r;
  auto rec = bias.IsEmpty() ? BackwardRecord::Create(OpKind::ConvTranspose2d, 2, {&x, &weight})
                            : BackwardRecord::Create(OpKind::ConvTranspose2d, 2, {&x, &weight, &bias});
  rec->Save(0, xc.Detach());
  rec->Save(1, wc.Detach());
  rec->Ints = {p.strideH, p.strideW, p.padH, p.padW, p.padH, p.padW, p.dilH, p.dilW, p.groups};
  return rec->Attach(r);
}

Tensor Ops::Resize2d(const Tensor& x, int outH, int outW, int mode, bool alignCorners) {
  RequireF32(x);
  if (x.Rank() != 4 || outH < 1 || outW < 1 || x.GetShape()[2] < 1 || x.GetShape()[3] < 1 || mode < 0 || mode > 1)
    throw TensorShapeException("Resize2d needs an (N,C,H,W) input and a positive output size, not " + x.GetShape().ToString() + " and " +
                               std::to_string(outH) + "x" + std::to_string(outW) + ".");
  Tensor xc = x.Contiguous();
  bool align = alignCorners && mode == 1;
  Tensor r = Tensor::Create(DType::F32, Shape{x.GetShape()[0], x.GetShape()[1], outH, outW});
  Check(om_resize2d_fwd(Ctx(), xc.Data(), (int64_t)x.GetShape()[0] * x.GetShape()[1], x.GetShape()[2], x.GetShape()[3], outH, outW, mode, align, r.Data()));
  if (!Recording({&x})) return r;
  auto rec = BackwardRecord::Create(OpKind::Resize2d, 0, {&x});
  rec->Ints = {mode, align ? 1 : 0, outH, outW};
  return rec->Attach(r);
}

// Sum of g over the axes that `target` broadcast (leading axes it lacks, axes where it is 1): Sum keeps the double
// accumulation of om_reduce_fwd. Only called when the shapes differ.
static Tensor SumToShape(Tensor g, const Shape& target) {
  GradMode::NoGrad ng;
  while (g.Rank() > target.rank) g = Ops::Sum(g, 0, false);
  for (int i = 0; i < target.rank; i++)
    if (target.d[i] == 1 && g.GetShape()[i] != 1) g = Ops::Sum(g, i, true);
  return g.Contiguous();
}

void RunGraphBackward(BackwardRecord& r, const Tensor& g) {
  Tensor gc = g.Contiguous();
  switch (r.Op) {
    case OpKind::BatchMatMul: {
      // dA = g b^T, dB = a^T g over the broadcast batch, then summed back to the operand's own batch axes.
      for (int side = 0; side < 2; side++) {
        if (!r.NeedsInputGrad(side)) continue;
        const Tensor& other = r.Saved(1 - side);
        Shape full = g.GetShape();
        if (side == 0) full.d[full.rank - 1] = other.GetShape()[other.Rank() - 2];
        else full.d[full.rank - 2] = other.GetShape()[other.Rank() - 1];
        Tensor t = Tensor::Create(DType::F32, full);
        if (side == 0) BatchedProduct(gc, false, other, true, t);
        else BatchedProduct(other, true, gc, false, t);
        Engine::Emit(r, side, t.GetShape() == r.InputShapes[side] ? t : SumToShape(t, r.InputShapes[side]).Reshape(r.InputShapes[side]), true);
      }
      break;
    }
    case OpKind::ConvTranspose2d: {
      const Tensor &x = r.Saved(0), &w = r.Saved(1);
      ConvTranspose2dParams p;
      p.strideH = (int)r.Ints[0]; p.strideW = (int)r.Ints[1]; p.padH = (int)r.Ints[2]; p.padW = (int)r.Ints[3];
      p.dilH = (int)r.Ints[6]; p.dilW = (int)r.Ints[7]; p.groups = (int)r.Ints[8];
      om_conv_shape s = AdjointShape(x.GetShape(), w.GetShape(), g.GetShape()[2], g.GetShape()[3], p);
      if (r.NeedsInputGrad(0)) {
        // dx = Conv2d(g, W)
        Tensor dx = Tensor::Create(DType::F32, x.GetShape());
        Check(om_conv2d_fwd(Ctx(), &s, gc.Data(), w.Data(), nullptr, dx.Data()));
        Engine::Emit(r, 0, dx, true);
      }
      if (r.NeedsInputGrad(1)) {
        // dW = x . im2col(g)^T per group: the weight gradient of the adjoint convolution with x in the role of its output gradient.
        Tensor dw = Tensor::Create(DType::F32, w.GetShape());
        Check(om_conv2d_wgrad(Ctx(), &s, x.Data(), gc.Data(), dw.Data(), 0));
        Engine::Emit(r, 1, dw, true);
      }
      if (r.InputCount() > 2 && r.NeedsInputGrad(2)) {
        om_conv_shape b{};
        b.n = g.GetShape()[0]; b.cin = 1; b.h = g.GetShape()[2]; b.w = g.GetShape()[3]; b.cout = g.GetShape()[1]; b.kh = b.kw = 1;
        b.stride_h = b.stride_w = b.dil_h = b.dil_w = b.groups = 1;
        Tensor db = Tensor::Create(DType::F32, r.InputShapes[2]);
        Check(om_conv2d_dbias(Ctx(), &b, gc.Data(), db.Data(), 0));
        Engine::Emit(r, 2, db, true);
      }
      break;
    }
    case OpKind::Resize2d: {
      const Shape& xs = r.InputShapes[0];
      Tensor dx = Tensor::Create(DType::F32, xs);
      Check(om_resize2d_bwd(Ctx(), gc.Data(), (int64_t)xs.d[0] * xs.d[1], xs.d[2], xs.d[3], (int)r.Ints[2], (int)r.Ints[3], (int)r.Ints[0],
                            (int)r.Ints[1], dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Erf:
    case OpKind::Exp:
    case OpKind::Sqrt: {
      const Tensor& saved = r.Saved(0);
      Tensor dx = Tensor::Create(DType::F32, saved.GetShape());
      om_unary_op op = r.Op == OpKind::Erf ? OM_ERF : r.Op == OpKind::Exp ? OM_EXP : OM_SQRT;
      Check(om_unary_bwd(Ctx(), op, gc.Data(), saved.Data(), dx.Data(), dx.Length()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Pow: {
      const Tensor& x = r.Saved(0);
      Tensor dx = Tensor::Create(DType::F32, x.GetShape());
      Check(om_pow_bwd(Ctx(), gc.Data(), x.Data(), (float)r.Floats[0], dx.Data(), dx.Length()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Dropout: {
      Tensor dx = Tensor::Create(DType::F32, r.InputShapes[0]);
      Check(om_dropout_bwd(Ctx(), gc.Data(), dx.Length(), (float)r.Floats[0], (uint64_t)r.Ints[0], (const int64_t*)r.Saved(0).RawData(),
                           dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Where: {
      const Tensor& c = r.Saved(0);
      for (int side = 0; side < 2; side++) {
        int input = side + 1;
        if (!r.NeedsInputGrad(input)) continue;
        Tensor t = Tensor::Create(DType::F32, g.GetShape());
        Check(om_where_bwd(Ctx(), (const int32_t*)c.RawData(), gc.Data(), side == 0 ? 1 : 0, t.Data(), t.Length()));
        Engine::Emit(r, input, t.GetShape() == r.InputShapes[input] ? t : SumToShape(t, r.InputShapes[input]).Reshape(r.InputShapes[input]), true);
      }
      break;
    }
    case OpKind::Gather: {
      const Tensor& idx = r.Saved(0);
      const Shape& ds = r.InputShapes[0];
      int ax = (int)r.Ints[0];
      int64_t outer = 1, inner = 1, n = ds.d[ax];
      for (int i = 0; i < ax; i++) outer *= ds.d[i];
      for (int i = ax + 1; i < ds.rank; i++) inner *= ds.d[i];
      Tensor dx = Tensor::Create(DType::F32, ds);
      Check(om_gather_bwd(Ctx(), gc.Data(), idx.RawData(), (int32_t)idx.GetDType(), outer, idx.Length(), n, inner, dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    default:
      throw InvalidOperationException("No backward function for op kind " + std::to_string((int)r.Op) + ".");
  }
}

}  // namespace omh
