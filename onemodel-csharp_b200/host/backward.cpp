// The backward function of every OpKind: reads the record and the incoming gradient (contiguous, the output's shape)
// and emits one gradient per input that needs one, as BackwardOps.Run / RunNn do in the reference
// (src/OneModel/Tensors/Autograd/BackwardOps.cs:13-145, BackwardNn.cs:7-143). All arithmetic runs on the device.
#include "omh.hpp"

namespace omh {

static om_ctx* C() { return Device::Current(); }

void RunSpatialBackward(Engine& e, BackwardRecord& r, const Tensor& g);  // backward_spatial.cpp

// Sums g down to `target` (undoing a broadcast). Returns g itself with same = true when the shapes already match
// (BackwardOps.SumTo, BackwardOps.cs:201-269).
static Tensor SumTo(const Tensor& g, const Shape& target, bool* same) {
  *same = g.GetShape() == target;
  if (*same) return g;
  int rank = g.Rank(), lead = rank - target.rank;
  if (lead < 0) throw TensorShapeException("Cannot sum " + g.GetShape().ToString() + " down to " + target.ToString() + ".");
  std::array<int64_t, kMaxRank> ts{};
  int64_t acc = 1;
  for (int ax = rank - 1; ax >= 0; ax--) {
    int t = ax - lead;
    if (t < 0 || target[t] == 1) {
      ts[ax] = 0;
    } else {
      ts[ax] = acc;
      acc *= target[t];
    }
  }
  Tensor gc = g.Contiguous();
  Tensor out = Tensor::Create(DType::F32, target);
  Check(om_sum_to(C(), rank, gc.GetShape().d.data(), gc.Data(), ts.data(), out.Data(), out.Length()));
  return out;
}

static Tensor UnaryGrad(om_unary_op op, const Tensor& g, const Tensor& saved) {
  Tensor gc = g.Contiguous();
  Tensor dx = Tensor::Create(DType::F32, saved.GetShape());
  // The gradient of the activation between two Linear layers is the first layer's output gradient: a product operand.
  if ((op == OM_GELU_ERF || op == OM_GELU_TANH) && Bf16Products()) {
    Check(om_unary_bwd_b16(C(), op, gc.Data(), saved.Data(), dx.Data(), dx.Bf16ForWrite(), dx.Length()));
    dx.Bf16Written();
  } else {
    Check(om_unary_bwd(C(), op, gc.Data(), saved.Data(), dx.Data(), dx.Length()));
  }
  return dx;
}

static Tensor NegOf(const Tensor& g) {
  Tensor gc = g.Contiguous();
  Tensor r = Tensor::Create(DType::F32, g.GetShape());
  Check(om_unary(C(), OM_NEG, gc.Data(), r.Data(), r.Length()));
  return r;
}

// Add and Sub: the output gradient summed down to each input's shape; Sub negates the second (BackwardOps.cs:156-194).
static void EmitSummed(Engine& e, BackwardRecord& r, const Tensor& g, bool negateSecond) {
  bool need0 = r.NeedsInputGrad(0), need1 = r.NeedsInputGrad(1);
  if (need0) {
    bool same;
    Tensor s = SumTo(g, r.InputShapes[0], &same);
    if (!same) Engine::Emit(r, 0, s, true);
    else if (!need1) e.EmitAliased(r, 0, g);
    else Engine::Emit(r, 0, g, false);       // both inputs take g itself: shared, copied only if something is added into it
  }
  if (need1) {
    bool same;
    Tensor s = SumTo(g, r.InputShapes[1], &same);
    if (negateSecond) Engine::Emit(r, 1, NegOf(s), true);
    else if (!same) Engine::Emit(r, 1, s, true);
    else if (need0 && r.InputShapes[0] == r.InputShapes[1]) Engine::Emit(r, 1, g, false);
    else e.EmitAliased(r, 1, g);
  }
}

// One call of the Linear backward on fp32 operands, or on their bfloat16 copies when the context asks for bfloat16 products
// and the three operands fit (g: the gradient with pitch ldg, possibly a column slice `col` of a wider gradient; x: the
// saved input; w: the saved weights, `col` rows in). The bias gradient always sums the fp32 gradient.
static void LinearBwdCall(const Tensor& g, int col, int ldg, const Tensor& x, const Tensor& w, int rows, int inF, int outF, float* dx, float* dw,
                          float* db, int acc, const Tensor* dx_tensor = nullptr) {
  if (!dx && !dw && !db) return;
  auto aligned16 = [](const float* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (Bf16Products() && rows > 0 && (dx || dw) && Bf16Operand(g, ldg) && col % 8 == 0 && Bf16Operand(x, inF) && Bf16Operand(w, inF) && (inF & 3) == 0 &&
      aligned16(dx) && aligned16(dw)) {
    // dx_tensor: the caller wants the bfloat16 copy of the input gradient from the product's epilogue (its consumer reads
    // bfloat16: the attention backward).
    uint16_t* dx16 = (dx && dx_tensor && inF % 8 == 0 && !(acc & 2)) ? dx_tensor->Bf16ForWrite() : nullptr;
    // The bias gradient g^T 1 reads the same bfloat16 copy of g as the weight gradient g^T x (no fp32 gradient is passed).
    Check(om_linear_bwd_bf16_b16(C(), g.Bf16() + col, nullptr, ldg, x.Bf16(), w.Bf16() + (size_t)col * inF, rows, inF, outF, dx, dx16, dw, db, acc));
    if (dx16) dx_tensor->Bf16Written();
    return;
  }
  // (A gradient that exists as bfloat16 only cannot take this route: its Data() throws.)
  Check(om_linear_bwd_ld(C(), g.Data() + col, ldg, x.Data(), w.Data() + (size_t)col * inF, rows, inF, outF, dx, dw, db, acc));
}

// The input gradient of a Linear layer whose input already holds another branch's gradient. Returns the tensor the product
// must ADD into (in place), or an empty tensor when nothing is left to do because the sum residual + g W was formed out of
// place by the product's epilogue and installed as the pending gradient (bfloat16 products on shapes the fused kernel takes:
// the shared gradient of a residual connection is then never copied). A shared gradient that cannot take that route is
// copied first, as the engine would have done on arrival.
static Tensor AddIntoPending(BackwardRecord& r, const uint16_t* g16, int ldg, const Tensor& w, int rows, int inF, int outF, const Tensor& pending,
                             bool shared) {
  if (!shared) return pending;
  auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (g16 && Bf16Products() && rows > 0 && ldg % 8 == 0 && aligned16(g16) && Bf16Operand(w, inF) && (inF & 7) == 0 && aligned16(pending.Data()) &&
      om_linear_dgrad_bf16_add_supported(C(), rows, inF, outF) == 1) {
    Tensor sum = Tensor::Create(DType::F32, pending.GetShape());
    Check(om_linear_dgrad_bf16_add(C(), g16, ldg, w.Bf16(), rows, inF, outF, pending.Data(), inF, sum.Data(), nullptr));
    Engine::PendingReplace(r, 0, sum);
    return Tensor();
  }
  return Engine::PendingOwn(r, 0);
}

// The record of Ops::LinearPacked (Ints = {rows, inF, outF, parts, hasBias}; inputs x, weights..., biases...): the input
// gradient is one product over the packed weights; the weight and bias gradients are one product and one column sum
// when the leaves' gradient buffers are adjacent like the parameters, else one per part on column slices of g.
static void LinearPackedBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor& x = r.Saved(0);
  const int rows = (int)r.Ints[0], inF = (int)r.Ints[1], outF = (int)r.Ints[2], parts = (int)r.Ints[3];
  const bool hasBias = r.Ints[4] != 0;
  Tensor gc = g.Contiguous();
  const Tensor& wpacked = r.Saved(1);
  Tensor dx;
  bool dx_into_pending = false;   // the input already has the residual branch's gradient: the product adds into it
  if (r.NeedsInputGrad(0)) {
    bool shared = false;
    dx_into_pending = Engine::PendingTarget(r, 0, &dx, &shared);
    if (dx_into_pending) {
      dx = AddIntoPending(r, (shared && Bf16Products() && Bf16Operand(gc, outF)) ? gc.Bf16() : nullptr, outF, wpacked, rows, inF, outF, dx, shared);
      dx_into_pending = !dx.IsEmpty();      // empty: the sum is already in place
    } else {
      dx = Tensor::Create(DType::F32, r.InputShapes[0]);
    }
  }
  const int accx = dx_into_pending ? 2 : 0;
  std::vector<float*> wp(parts, nullptr), bp(parts, nullptr);
  std::vector<bool> wacc(parts, false), bacc(parts, false), wleaf(parts, false), bleaf(parts, false);
  std::vector<Tensor> wtmp(parts), btmp(parts);
  std::vector<int> outs(parts);
  for (int i = 0; i < parts; i++) {
    outs[i] = r.InputShapes[1 + i][0];
    if (r.NeedsInputGrad(1 + i)) {
      bool acc = false;
      wleaf[i] = Engine::LeafTarget(r, 1 + i, &wp[i], &acc);
      wacc[i] = acc;
      if (!wleaf[i]) {
        wtmp[i] = Tensor::Create(DType::F32, r.InputShapes[1 + i]);
        wp[i] = wtmp[i].Data();
      }
    }
    if (hasBias && r.NeedsInputGrad(1 + parts + i)) {
      bool acc = false;
      bleaf[i] = Engine::LeafTarget(r, 1 + parts + i, &bp[i], &acc);
      bacc[i] = acc;
      if (!bleaf[i]) {
        btmp[i] = Tensor::Create(DType::F32, r.InputShapes[1 + parts + i]);
        bp[i] = btmp[i].Data();
      }
    }
  }
  auto packed = [&](const std::vector<float*>& ptr, const std::vector<bool>& acc, bool weights) {
    for (int i = 0; i < parts; i++) {
      if (!ptr[i] || acc[i] != acc[0]) return false;
      if (i > 0 && ptr[i] != ptr[i - 1] + (size_t)outs[i - 1] * (weights ? inF : 1)) return false;
    }
    return true;
  };
  const bool wp_one = packed(wp, wacc, true), bp_one = hasBias && packed(bp, bacc, false);
  // Input gradient (+ the packed weight / bias gradients when they can ride along).
  if (!dx.IsEmpty() || wp_one || bp_one) {
    if (wp_one && bp_one && wacc[0] != bacc[0]) {
      LinearBwdCall(gc, 0, outF, x, wpacked, rows, inF, outF, dx.IsEmpty() ? nullptr : dx.Data(), wp[0], nullptr, (wacc[0] ? 1 : 0) | accx);
      LinearBwdCall(gc, 0, outF, x, wpacked, rows, inF, outF, nullptr, nullptr, bp[0], bacc[0] ? 1 : 0);
    } else {
      LinearBwdCall(gc, 0, outF, x, wpacked, rows, inF, outF, dx.IsEmpty() ? nullptr : dx.Data(), wp_one ? wp[0] : nullptr,
                    bp_one ? bp[0] : nullptr, ((wp_one ? wacc[0] : (bp_one && bacc[0])) ? 1 : 0) | accx);
    }
  }
  int col = 0;
  for (int i = 0; i < parts; i++) {
    if (!wp_one && wp[i]) LinearBwdCall(gc, col, outF, x, wpacked, rows, inF, outs[i], nullptr, wp[i], nullptr, wacc[i] ? 1 : 0);
    if (hasBias && !bp_one && bp[i]) LinearBwdCall(gc, col, outF, x, wpacked, rows, inF, outs[i], nullptr, nullptr, bp[i], bacc[i] ? 1 : 0);
    col += outs[i];
  }
  // Emission order as for the single layer, part by part: bias, (input once), weight.
  for (int i = 0; i < parts; i++)
    if (hasBias && r.NeedsInputGrad(1 + parts + i)) {
      if (bleaf[i]) Engine::LeafWritten(r, 1 + parts + i); else Engine::Emit(r, 1 + parts + i, btmp[i], true);
    }
  if (dx_into_pending) Engine::PendingWritten(r, 0);
  else if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  for (int i = 0; i < parts; i++)
    if (r.NeedsInputGrad(1 + i)) {
      if (wleaf[i]) Engine::LeafWritten(r, 1 + i); else Engine::Emit(r, 1 + i, wtmp[i], true);
    }
}

static void LinearBackward(Engine& e, BackwardRecord& r, const Tensor& g) {
  if (r.Ints.size() == 5) return LinearPackedBackward(r, g);
  const Tensor& x = r.Saved(0);
  const Tensor& w = r.Saved(1);
  int rows = (int)r.Ints[0], inF = (int)r.Ints[1], outF = (int)r.Ints[2];
  // A row-pitched rank-2 gradient (unit inner stride) is read in place.
  int ldg = outF;
  Tensor gc;
  if (g.Rank() == 2 && rows > 1 && g.Strides()[1] == 1 && g.Strides()[0] > outF) {
    gc = g;
    ldg = (int)g.Strides()[0];
  } else {
    gc = g.Contiguous();
  }
  bool hasBias = r.InputCount() == 3;
  Tensor dx;
  // When the input already has a gradient from another branch (the residual connection), the product adds into it.
  bool dx_into_pending = false;
  if (r.NeedsInputGrad(0)) {
    bool shared = false;
    dx_into_pending = Engine::PendingTarget(r, 0, &dx, &shared);
    if (dx_into_pending) {
      dx = AddIntoPending(r, (shared && Bf16Products() && Bf16Operand(gc, ldg)) ? gc.Bf16() : nullptr, ldg, w, rows, inF, outF, dx, shared);
      dx_into_pending = !dx.IsEmpty();
    } else {
      dx = Tensor::Create(DType::F32, r.InputShapes[0]);
    }
  }
  const int accx = dx_into_pending ? 2 : 0;
  // Weight and bias gradients go straight into the leaf's gradient buffer when there is one.
  float *dwp = nullptr, *dbp = nullptr;
  bool accw = false, accb = false, wleaf = false, bleaf = false;
  Tensor dw, db;
  if (r.NeedsInputGrad(1)) {
    wleaf = Engine::LeafTarget(r, 1, &dwp, &accw);
    if (!wleaf) {
      dw = Tensor::Create(DType::F32, r.InputShapes[1]);
      dwp = dw.Data();
    }
  }
  if (hasBias && r.NeedsInputGrad(2)) {
    bleaf = Engine::LeafTarget(r, 2, &dbp, &accb);
    if (!bleaf) {
      db = Tensor::Create(DType::F32, r.InputShapes[2]);
      dbp = db.Data();
    }
  }
  // The gradient of an attention output is read as bfloat16 by the attention backward: ask the product for the copy.
  const bool to_attention = !dx.IsEmpty() && r.Inputs[0] && r.Inputs[0]->GradFn && r.Inputs[0]->GradFn->Op == OpKind::Attention;
  const Tensor* dxt = to_attention ? &dx : nullptr;
  if (accw == accb || !dwp || !dbp) {
    LinearBwdCall(gc, 0, ldg, x, w, rows, inF, outF, dx.IsEmpty() ? nullptr : dx.Data(), dwp, dbp, ((dwp ? accw : accb) ? 1 : 0) | accx, dxt);
  } else {
    LinearBwdCall(gc, 0, ldg, x, w, rows, inF, outF, dx.IsEmpty() ? nullptr : dx.Data(), dwp, nullptr, (accw ? 1 : 0) | accx, dxt);
    LinearBwdCall(gc, 0, ldg, x, w, rows, inF, outF, nullptr, nullptr, dbp, accb ? 1 : 0);
  }
  // Emission order of the reference's record chain: bias (Add record), then input and weight (MatMul record).
  if (hasBias && r.NeedsInputGrad(2)) {
    if (bleaf) Engine::LeafWritten(r, 2); else Engine::Emit(r, 2, db, true);
  }
  if (dx_into_pending) Engine::PendingWritten(r, 0);
  else if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  if (r.NeedsInputGrad(1)) {
    if (wleaf) Engine::LeafWritten(r, 1); else Engine::Emit(r, 1, dw, true);
  }
}

// The record of Ops::FeedForward (inputs x, w1, b1, w2, b2; saved x, w1, w2, the activation's derivative at the first layer's
// result, the activation's result as bfloat16; Ints = {rows, in, ff, out, op}). The second layer's input gradient comes
// out of its product already multiplied by the activation's derivative, as fp32 (the first layer's bias gradient sums it)
// and as bfloat16 (the operand of the first layer's two gradient products).
static void FeedForwardBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor& x = r.Saved(0);
  const Tensor& w1 = r.Saved(1);
  const Tensor& w2 = r.Saved(2);
  const Tensor& pre = r.Saved(3);      // the activation's derivative (see Ops::FeedForward)
  const Tensor& act16 = r.Saved(4);
  const int rows = (int)r.Ints[0], inF = (int)r.Ints[1], ff = (int)r.Ints[2], outF = (int)r.Ints[3];
  Tensor gc = g.Contiguous();
  struct Leaf {
    float* p = nullptr;
    bool acc = false, leaf = false, need = false;
    Tensor t;
  };
  auto target = [&](int i) {
    Leaf l;
    l.need = r.NeedsInputGrad(i);
    if (!l.need) return l;
    l.leaf = Engine::LeafTarget(r, i, &l.p, &l.acc);
    if (!l.leaf) {
      l.t = Tensor::Create(DType::F32, r.InputShapes[i]);
      l.p = l.t.Data();
    }
    return l;
  };
  auto done = [&](int i, Leaf& l) {
    if (!l.need) return;
    if (l.leaf) Engine::LeafWritten(r, i); else Engine::Emit(r, i, l.t, true);
  };
  Leaf dw1 = target(1), db1 = target(2), dw2 = target(3), db2 = target(4);
  const uint16_t* g16 = gc.Bf16();
  // Second layer: weight and bias gradients, then the input gradient through the activation.
  if (dw2.p && db2.p && dw2.acc == db2.acc) {
    // one call: with OM_TWO_STREAMS the bias sum then runs beside the weight-gradient product
    Check(om_linear_bwd_bf16_b16(C(), g16, nullptr, outF, (const uint16_t*)act16.RawData(), w2.Bf16(), rows, ff, outF, nullptr, nullptr, dw2.p, db2.p, dw2.acc ? 1 : 0));
  } else {
    if (dw2.p) Check(om_linear_bwd_bf16_b16(C(), g16, nullptr, outF, (const uint16_t*)act16.RawData(), w2.Bf16(), rows, ff, outF, nullptr, nullptr, dw2.p, nullptr, dw2.acc ? 1 : 0));
    if (db2.p) Check(om_linear_bwd_bf16_b16(C(), g16, nullptr, outF, (const uint16_t*)act16.RawData(), w2.Bf16(), rows, ff, outF, nullptr, nullptr, nullptr, db2.p, db2.acc ? 1 : 0));
  }
  done(4, db2);
  done(3, dw2);
  if (!dw1.p && !db1.p && !r.NeedsInputGrad(0)) return;
  // The gradient in front of the activation exists as bfloat16 only (two per 32-bit word of an integer tensor): the three
  // gradients of the first layer are products that read it as an operand (the bias gradient is g^T 1).
  Tensor dpre16 = Tensor::Create(DType::I32, Shape{rows, ff / 2});
  const uint16_t* d16 = (const uint16_t*)dpre16.RawData();
  Check(om_linear_dgrad_bf16_mul(C(), g16, outF, w2.Bf16(), rows, ff, outF, (const uint16_t*)pre.RawData(), ff, nullptr, (uint16_t*)dpre16.RawData()));
  // First layer.
  Tensor dx;
  bool dx_into_pending = false;
  if (r.NeedsInputGrad(0)) {
    bool shared = false;
    dx_into_pending = Engine::PendingTarget(r, 0, &dx, &shared);
    if (dx_into_pending) {
      dx = AddIntoPending(r, d16, ff, w1, rows, inF, ff, dx, shared);
      dx_into_pending = !dx.IsEmpty();
    } else {
      dx = Tensor::Create(DType::F32, r.InputShapes[0]);
    }
  }
  const int accx = dx_into_pending ? 2 : 0;
  float* dxp = dx.IsEmpty() ? nullptr : dx.Data();
  if (dw1.acc == db1.acc || !dw1.p || !db1.p) {
    if (dxp || dw1.p || db1.p)
      Check(om_linear_bwd_bf16_b16(C(), d16, nullptr, ff, x.Bf16(), w1.Bf16(), rows, inF, ff, dxp, nullptr, dw1.p, db1.p, ((dw1.p ? dw1.acc : db1.acc) ? 1 : 0) | accx));
  } else {
    Check(om_linear_bwd_bf16_b16(C(), d16, nullptr, ff, x.Bf16(), w1.Bf16(), rows, inF, ff, dxp, nullptr, dw1.p, nullptr, (dw1.acc ? 1 : 0) | accx));
    Check(om_linear_bwd_bf16_b16(C(), d16, nullptr, ff, x.Bf16(), w1.Bf16(), rows, inF, ff, nullptr, nullptr, nullptr, db1.p, db1.acc ? 1 : 0));
  }
  done(2, db1);
  if (dx_into_pending) Engine::PendingWritten(r, 0);
  else if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  done(1, dw1);
}

static bool GemmLayout(const Tensor& t, int* trans, int* ld) {
  int64_t s0 = t.Strides()[0], s1 = t.Strides()[1];
  int rr = t.GetShape()[0], c = t.GetShape()[1];
  if ((s1 == 1 || c == 1) && (s0 >= c || rr == 1)) {
    *trans = 0;
    *ld = (int)(rr == 1 ? std::max<int64_t>(c, 1) : s0);
    return true;
  }
  if ((s0 == 1 || rr == 1) && (s1 >= rr || c == 1)) {
    *trans = 1;
    *ld = (int)(c == 1 ? std::max<int64_t>(rr, 1) : s1);
    return true;
  }
  return false;
}

// dA = g B^T, dB = A^T g (BackwardOps.cs:69-82); the saved operands may be transposed views, read in place.
static void MatMulBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor& a = r.Saved(0);
  const Tensor& b = r.Saved(1);
  Tensor gc = g.Contiguous();
  int m = a.GetShape()[0], k = a.GetShape()[1], n = b.GetShape()[1];
  int ta, tb, lda, ldb;
  GemmLayout(a, &ta, &lda);
  GemmLayout(b, &tb, &ldb);
  if (r.NeedsInputGrad(0)) {
    Tensor da = Tensor::Create(DType::F32, Shape{m, k});
    // da[m,k] = g[m,n] * op(b)^T : B operand of the product is op(b)^T, i.e. transposed flag flipped.
    Check(om_matmul(C(), 0, !tb, m, k, n, gc.Data(), n, b.Data(), ldb, da.Data(), k, 0));
    Engine::Emit(r, 0, da, true);
  }
  if (r.NeedsInputGrad(1)) {
    Tensor db = Tensor::Create(DType::F32, Shape{k, n});
    Check(om_matmul(C(), !ta, 0, k, n, m, a.Data(), lda, gc.Data(), n, db.Data(), n, 0));
    Engine::Emit(r, 1, db, true);
  }
}

static void ReduceBackward(BackwardRecord& r, const Tensor& g) {
  const Shape& in = r.InputShapes[0];
  int axis = (int)r.Ints[0];
  int64_t outer = 1, n = 1, inner = 1;
  if (axis < 0) {
    n = in.Length();
  } else {
    n = in[axis];
    for (int i = 0; i < axis; i++) outer *= in[i];
    for (int i = axis + 1; i < in.rank; i++) inner *= in[i];
  }
  Tensor gc = g.Contiguous();
  Tensor dx = Tensor::Create(DType::F32, in);
  Check(om_reduce_bwd(C(), gc.Data(), outer, n, inner, r.Op == OpKind::Mean, dx.Data()));
  Engine::Emit(r, 0, dx, true);
}

static void NormParamGrads(BackwardRecord& r, float** dg, float** db, bool* acc, Tensor* tg, Tensor* tb, bool* gleaf, bool* bleaf) {
  bool ag = false, ab = false;
  *dg = *db = nullptr;
  *gleaf = *bleaf = false;
  if (r.NeedsInputGrad(1)) {
    *gleaf = Engine::LeafTarget(r, 1, dg, &ag);
    if (!*gleaf) {
      *tg = Tensor::Create(DType::F32, r.InputShapes[1]);
      *dg = tg->Data();
    }
  }
  if (r.NeedsInputGrad(2)) {
    *bleaf = Engine::LeafTarget(r, 2, db, &ab);
    if (!*bleaf) {
      *tb = Tensor::Create(DType::F32, r.InputShapes[2]);
      *db = tb->Data();
    }
  }
  if (*dg && *db && ag != ab) {
    // Mixed accumulate states cannot share one launch: fall back to temporaries and Emit.
    if (*gleaf) { *tg = Tensor::Create(DType::F32, r.InputShapes[1]); *dg = tg->Data(); *gleaf = false; }
    if (*bleaf) { *tb = Tensor::Create(DType::F32, r.InputShapes[2]); *db = tb->Data(); *bleaf = false; }
    ag = ab = false;
  }
  *acc = *dg ? ag : ab;
}

static void EmitNormParams(BackwardRecord& r, const Tensor& tg, const Tensor& tb, bool gleaf, bool bleaf) {
  if (r.NeedsInputGrad(1)) {
    if (gleaf) Engine::LeafWritten(r, 1); else Engine::Emit(r, 1, tg, true);
  }
  if (r.NeedsInputGrad(2)) {
    if (bleaf) Engine::LeafWritten(r, 2); else Engine::Emit(r, 2, tb, true);
  }
}

static void LayerNormBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor &x = r.Saved(0), &gamma = r.Saved(1), &mean = r.Saved(2), &inv = r.Saved(3);
  int cols = x.GetShape()[x.Rank() - 1];
  int rows = cols == 0 ? 0 : (int)(x.Length() / cols);
  Tensor gc = g.Contiguous();
  Tensor dx;
  if (r.NeedsInputGrad(0)) dx = Tensor::Create(DType::F32, x.GetShape());
  float *dg, *db;
  bool acc, gleaf, bleaf;
  Tensor tg, tb;
  NormParamGrads(r, &dg, &db, &acc, &tg, &tb, &gleaf, &bleaf);
  if (Bf16Products() && !dx.IsEmpty()) {
    Check(om_layernorm_bwd_b16(C(), gc.Data(), x.Data(), gamma.Data(), mean.Data(), inv.Data(), rows, cols, dx.Data(), dx.Bf16ForWrite(), dg, db, acc));
    dx.Bf16Written();
  } else {
    Check(om_layernorm_bwd(C(), gc.Data(), x.Data(), gamma.Data(), mean.Data(), inv.Data(), rows, cols,
                           dx.IsEmpty() ? nullptr : dx.Data(), dg, db, acc));
  }
  if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  EmitNormParams(r, tg, tb, gleaf, bleaf);
}

static void BatchNormBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor &x = r.Saved(0), &gamma = r.Saved(1), &mean = r.Saved(2), &inv = r.Saved(3);
  int n = x.GetShape()[0], c = x.GetShape()[1], plane = (int)(x.Length() / std::max(1, n * c));
  Tensor gc = g.Contiguous();
  Tensor dx;
  if (r.NeedsInputGrad(0)) dx = Tensor::Create(DType::F32, x.GetShape());
  float *dg, *db;
  bool acc, gleaf, bleaf;
  Tensor tg, tb;
  NormParamGrads(r, &dg, &db, &acc, &tg, &tb, &gleaf, &bleaf);
  Check(om_batchnorm_bwd(C(), gc.Data(), x.Data(), gamma.Data(), mean.Data(), inv.Data(), n, c, plane, r.Ints[0] != 0,
                         dx.IsEmpty() ? nullptr : dx.Data(), dg, db, acc));
  if (!dx.IsEmpty()) Engine::Emit(r, 0, dx, true);
  EmitNormParams(r, tg, tb, gleaf, bleaf);
}

// Row-sparse table gradient (EmbeddingSparseBackward, BackwardNn.cs:548-600): the looked-up rows in ascending order and, for
// each, the sum of its lookups' output gradients in increasing position order from zero - the dense gradient's rows bit for
// bit. The row count stays on the device; a lookup of nothing but padding leaves a gradient without rows, which
// Tensor::SparseGrad reports as none.
static void EmbeddingSparseBackward(BackwardRecord& r, const Tensor& g, const Tensor& ids, const Shape& ts) {
  if (ids.Length() == 0) return;
  Tensor gc = g.Contiguous();
  const int cap = (int)std::min<int64_t>(ids.Length(), ts[0]);
  Tensor rows = Tensor::Create(DType::I32, Shape{cap}), values = Tensor::Create(DType::F32, Shape{cap, ts[1]}), count = Tensor::Create(DType::I32, Shape{1});
  Check(om_embedding_bwd_sparse(C(), gc.Data(), ids.RawData(), (int32_t)ids.GetDType(), ids.Length(), ts[0], ts[1], r.Ints[0], (int32_t*)rows.RawData(),
                                values.Data(), cap, (int32_t*)count.RawData()));
  Engine::EmitSparse(r, 0, std::make_shared<RowSparseGradient>(ts, rows, values, count));
}

static void EmbeddingBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor& ids = r.Saved(0);
  const Shape& ts = r.InputShapes[0];
  if (r.Ints.size() > 1 && r.Ints[1] != 0 && r.Inputs[0] && !r.Inputs[0]->GradFn) {
    EmbeddingSparseBackward(r, g, ids, ts);
    return;
  }
  Tensor gc = g.Contiguous();
  float* dt = nullptr;
  bool acc = false;
  Tensor tmp;
  bool leaf = Engine::LeafTarget(r, 0, &dt, &acc);
  if (!leaf) {
    tmp = Tensor::Create(DType::F32, ts);
    dt = tmp.Data();
  }
  Check(om_embedding_bwd(C(), gc.Data(), ids.RawData(), (int32_t)ids.GetDType(), ids.Length(), ts[0], ts[1], r.Ints[0], dt, acc));
  if (leaf) Engine::LeafWritten(r, 0); else Engine::Emit(r, 0, tmp, true);
}

// The record of Ops::AttentionHeads (Ints = {maskStride, heads}): activations [B, L, H*D], possibly row-pitched.
static void AttentionHeadsBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor &q = r.Saved(0), &k = r.Saved(1), &v = r.Saved(2), &mask = r.Saved(3);
  int heads = (int)r.Ints[1];
  int b = q.GetShape()[0], lq = q.GetShape()[1], lk = k.GetShape()[1], d = q.GetShape()[2] / heads;
  Tensor gc = g.Contiguous();
  Tensor dq, dk, dv;
  if (r.NeedsInputGrad(0)) dq = Tensor::Create(DType::F32, q.GetShape());
  if (r.NeedsInputGrad(1)) dk = Tensor::Create(DType::F32, k.GetShape());
  if (r.NeedsInputGrad(2)) dv = Tensor::Create(DType::F32, v.GetShape());
  auto strides = [&](const Tensor& t) { return om_head_strides{t.Strides()[0], (int64_t)d, t.Strides()[1]}; };
  om_head_strides gs = strides(gc), qs = strides(q), ks = strides(k), vs = strides(v), dqs{}, dks{}, dvs{};
  if (!dq.IsEmpty()) dqs = strides(dq);
  if (!dk.IsEmpty()) dks = strides(dk);
  if (!dv.IsEmpty()) dvs = strides(dv);
  const Tensor& out = r.Saved(5);
  om_head_strides os{};
  if (!out.IsEmpty()) os = strides(out);
  Check(om_attention_bwd_strided_out(C(), gc.Data(), &gs, q.Data(), &qs, k.Data(), &ks, v.Data(), &vs, out.IsEmpty() ? nullptr : out.Data(), &os,
                                     mask.IsEmpty() ? nullptr : mask.Data(), r.Ints[0], r.Saved(4).IsEmpty() ? nullptr : r.Saved(4).Data(), b, heads,
                                     lq, lk, d, (float)r.Floats[0], dq.IsEmpty() ? nullptr : dq.Data(), &dqs, dk.IsEmpty() ? nullptr : dk.Data(), &dks,
                                     dv.IsEmpty() ? nullptr : dv.Data(), &dvs));
  if (!dq.IsEmpty()) Engine::Emit(r, 0, dq, true);
  if (!dk.IsEmpty()) Engine::Emit(r, 1, dk, true);
  if (!dv.IsEmpty()) Engine::Emit(r, 2, dv, true);
}

// The record of Ops::AttentionPacked (Ints = {maskStride, heads, 1}): q | k | v packed along the last axis of one tensor.
static void AttentionPackedBackward(BackwardRecord& r, const Tensor& g) {
  const Tensor &qkv = r.Saved(0), &mask = r.Saved(3);
  const int heads = (int)r.Ints[1];
  const int b = qkv.GetShape()[0], l = qkv.GetShape()[1], width = qkv.GetShape()[2] / 3, d = width / heads;
  if (!r.NeedsInputGrad(0)) return;
  Tensor gc = g.Contiguous();
  om_head_strides ps{(int64_t)l * 3 * width, (int64_t)d, (int64_t)3 * width}, gs{(int64_t)l * width, (int64_t)d, (int64_t)width};
  const Tensor& out = r.Saved(5);
  if (Bf16Products() && !out.IsEmpty() && !r.Saved(4).IsEmpty() && l > 128 && om_attention_bwd_bf16_supported(C(), b, heads, l, l, d) &&
      Bf16Operand(qkv, 3 * width) && Bf16Operand(gc, width) && width % 8 == 0) {
    // Several tiles under bfloat16 products: the fully fused kernel on the bfloat16 copies of the packed projections and of
    // the gradient; it also writes the bfloat16 copy of dqkv, the next product's operand.
    const uint16_t* p16 = qkv.Bf16();
    const uint16_t* g16 = gc.Bf16();
    // When the packed projection that made q | k | v reads its gradient as bfloat16 only and nothing else has contributed
    // to that gradient, dqkv is written as bfloat16 alone (a third of the bytes).
    BackwardRecord* producer = r.Inputs[0] ? r.Inputs[0]->GradFn.get() : nullptr;
    const bool only16 = producer && producer->TakesBf16OnlyGrad && producer->PendingGrad.IsEmpty();
    Tensor dqkv = only16 ? Tensor::CreateBf16Only(qkv.GetShape()) : Tensor::Create(DType::F32, qkv.GetShape());
    uint16_t* d16 = dqkv.Bf16ForWrite();
    float* d32 = only16 ? nullptr : dqkv.Data();
    Check(om_attention_bwd_bf16(C(), g16, gc.Data(), &gs, p16, &ps, p16 + width, &ps, p16 + 2 * width, &ps, out.Data(), &gs,
                                mask.IsEmpty() ? nullptr : mask.Data(), r.Ints[0], r.Saved(4).Data(), b, heads, l, l, d, (float)r.Floats[0], d32, d16, &ps,
                                d32 ? d32 + width : nullptr, d16 + width, &ps, d32 ? d32 + 2 * width : nullptr, d16 + 2 * width, &ps));
    dqkv.Bf16Written();
    Engine::Emit(r, 0, dqkv, true);
    return;
  }
  Tensor dqkv = Tensor::Create(DType::F32, qkv.GetShape());
  Check(om_attention_bwd_strided_out(C(), gc.Data(), &gs, qkv.Data(), &ps, qkv.Data() + width, &ps, qkv.Data() + 2 * width, &ps,
                                     out.IsEmpty() ? nullptr : out.Data(), &gs, mask.IsEmpty() ? nullptr : mask.Data(), r.Ints[0],
                                     r.Saved(4).IsEmpty() ? nullptr : r.Saved(4).Data(), b, heads, l, l, d, (float)r.Floats[0], dqkv.Data(), &ps,
                                     dqkv.Data() + width, &ps, dqkv.Data() + 2 * width, &ps));
  Engine::Emit(r, 0, dqkv, true);
}

static void AttentionBackward(BackwardRecord& r, const Tensor& g) {
  if (r.Ints.size() > 2) return AttentionPackedBackward(r, g);
  if (r.Ints.size() > 1) return AttentionHeadsBackward(r, g);
  const Tensor &q = r.Saved(0), &k = r.Saved(1), &v = r.Saved(2), &mask = r.Saved(3);
  int b = q.GetShape()[0], h = q.GetShape()[1], lq = q.GetShape()[2], d = q.GetShape()[3], lk = k.GetShape()[2];
  Tensor gc = g.Contiguous();
  Tensor dq, dk, dv;
  if (r.NeedsInputGrad(0)) dq = Tensor::Create(DType::F32, q.GetShape());
  if (r.NeedsInputGrad(1)) dk = Tensor::Create(DType::F32, k.GetShape());
  if (r.NeedsInputGrad(2)) dv = Tensor::Create(DType::F32, v.GetShape());
  const om_head_strides sq{(int64_t)h * lq * d, (int64_t)lq * d, (int64_t)d}, sk{(int64_t)h * lk * d, (int64_t)lk * d, (int64_t)d};
  const Tensor& out = r.Saved(5);
  Check(om_attention_bwd_strided_out(C(), gc.Data(), &sq, q.Data(), &sq, k.Data(), &sk, v.Data(), &sk, out.IsEmpty() ? nullptr : out.Data(), &sq,
                                     mask.IsEmpty() ? nullptr : mask.Data(), r.Ints[0], r.Saved(4).IsEmpty() ? nullptr : r.Saved(4).Data(), b, h, lq,
                                     lk, d, (float)r.Floats[0], dq.IsEmpty() ? nullptr : dq.Data(), &sq, dk.IsEmpty() ? nullptr : dk.Data(), &sk,
                                     dv.IsEmpty() ? nullptr : dv.Data(), &sk));
  if (!dq.IsEmpty()) Engine::Emit(r, 0, dq, true);
  if (!dk.IsEmpty()) Engine::Emit(r, 1, dk, true);
  if (!dv.IsEmpty()) Engine::Emit(r, 2, dv, true);
}

void RunBackwardOp(Engine& e, BackwardRecord& r, const Tensor& g) {
  switch (r.Op) {
    case OpKind::Add: EmitSummed(e, r, g, false); break;
    case OpKind::Sub: EmitSummed(e, r, g, true); break;
    case OpKind::Mul:
      for (int i = 0; i < 2; i++)
        if (r.NeedsInputGrad(i)) {
          GradMode::NoGrad ng;
          Tensor t = Ops::Mul(g, r.Saved(1 - i));
          bool same;
          Engine::Emit(r, i, SumTo(t, r.InputShapes[i], &same), true);
        }
      break;
    case OpKind::Div:
      if (r.NeedsInputGrad(0)) {
        Tensor t = Ops::Div(g, r.Saved(1));
        bool same;
        Engine::Emit(r, 0, SumTo(t, r.InputShapes[0], &same), true);
      }
      if (r.NeedsInputGrad(1)) {
        // d(a/b)/db = -a/b^2
        const Tensor& b = r.Saved(1);
        Tensor t = Ops::Neg(Ops::Div(Ops::Mul(g, r.Saved(0)), Ops::Mul(b, b)));
        bool same;
        Engine::Emit(r, 1, SumTo(t, r.InputShapes[1], &same), true);
      }
      break;
    case OpKind::Neg: Engine::Emit(r, 0, NegOf(g), true); break;
    case OpKind::Relu: Engine::Emit(r, 0, UnaryGrad(OM_RELU, g, r.Saved(0)), true); break;
    case OpKind::Gelu: Engine::Emit(r, 0, UnaryGrad(r.Ints[0] == 1 ? OM_GELU_TANH : OM_GELU_ERF, g, r.Saved(0)), true); break;
    case OpKind::Sigmoid: Engine::Emit(r, 0, UnaryGrad(OM_SIGMOID, g, r.Saved(0)), true); break;
    case OpKind::Tanh: Engine::Emit(r, 0, UnaryGrad(OM_TANH, g, r.Saved(0)), true); break;
    case OpKind::MatMul: MatMulBackward(r, g); break;
    case OpKind::Linear: LinearBackward(e, r, g); break;
    case OpKind::FeedForward: FeedForwardBackward(r, g); break;
    case OpKind::Slice: {
      Tensor dx = Tensor::Zeros(DType::F32, r.InputShapes[0]);
      Tensor dst = dx.Slice((int)r.Ints[0], (int)r.Ints[1], (int)r.Ints[2], (int)r.Ints[3]);
      Check(om_strided_copy(C(), g.Rank(), g.GetShape().d.data(), g.Data(), g.Strides().data(), dst.Data(), dst.Strides().data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Select: {
      Tensor dx = Tensor::Zeros(DType::F32, r.InputShapes[0]);
      Tensor dst = dx.Select((int)r.Ints[0], (int)r.Ints[1]);
      Check(om_strided_copy(C(), g.Rank(), g.GetShape().d.data(), g.Data(), g.Strides().data(), dst.Data(), dst.Strides().data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::Permute: {
      std::vector<int> inv(r.Ints.size());
      for (size_t i = 0; i < r.Ints.size(); i++) inv[(size_t)r.Ints[i]] = (int)i;
      Engine::Emit(r, 0, g.Permute(inv).Clone(), true);
      break;
    }
    case OpKind::Reshape: e.EmitAliased(r, 0, g.Contiguous().Reshape(r.InputShapes[0])); break;
    case OpKind::Expand: {
      bool same;
      Tensor s = SumTo(g, r.InputShapes[0], &same);
      if (same) e.EmitAliased(r, 0, g); else Engine::Emit(r, 0, s, true);
      break;
    }
    case OpKind::Flip: Engine::Emit(r, 0, g.Flip((int)r.Ints[0]).Clone(), true); break;
    case OpKind::Sum:
    case OpKind::Mean: ReduceBackward(r, g); break;
    case OpKind::Softmax: {
      const Tensor& y = r.Saved(0);
      int cols = y.GetShape()[y.Rank() - 1];
      int rows = cols == 0 ? 0 : (int)(y.Length() / cols);
      Tensor gc = g.Contiguous();
      Tensor dx = Tensor::Create(DType::F32, y.GetShape());
      Check(om_softmax_bwd(C(), gc.Data(), y.Data(), rows, cols, dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::LogSoftmax: {
      const Tensor& y = r.Saved(0);
      int cols = y.GetShape()[y.Rank() - 1];
      int rows = cols == 0 ? 0 : (int)(y.Length() / cols);
      Tensor gc = g.Contiguous();
      Tensor dx = Tensor::Create(DType::F32, y.GetShape());
      Check(om_logsoftmax_bwd(C(), gc.Data(), y.Data(), rows, cols, dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::NllLoss: {
      const Tensor& t = r.Saved(0);
      const Shape& ls = r.InputShapes[0];
      Tensor gc = g.Contiguous();
      Tensor dx = Tensor::Create(DType::F32, ls);
      Check(om_nll_bwd(C(), gc.Data(), t.RawData(), (int32_t)t.GetDType(), ls[0], ls[1], r.Ints[0] != 0, r.Ints[1], dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::CrossEntropy: {
      const Tensor &logp = r.Saved(0), &t = r.Saved(1);
      const Shape& ls = r.InputShapes[0];
      Tensor gc = g.Contiguous();
      int ld = (int)r.Ints[2];
      Tensor dx = ld == ls[1] ? Tensor::Create(DType::F32, ls)
                              : Tensor::Create(DType::F32, Shape{ls[0], ld}).View(ls, {(int64_t)ld, 1}, 0);
      Check(om_cross_entropy_bwd_ld(C(), gc.Data(), logp.Data(), t.RawData(), (int32_t)t.GetDType(), ls[0], ls[1], ld,
                                    r.Ints[0] != 0, r.Ints[1], (float)r.Floats[0], dx.Data()));
      Engine::Emit(r, 0, dx, true);
      break;
    }
    case OpKind::LayerNorm: LayerNormBackward(r, g); break;
    case OpKind::BatchNorm: BatchNormBackward(r, g); break;
    case OpKind::Embedding: EmbeddingBackward(r, g); break;
    case OpKind::Attention: AttentionBackward(r, g); break;
    case OpKind::Concat: {
      int axis = (int)r.Ints[0];
      int start = 0;
      for (int i = 0; i < r.InputCount(); i++) {
        int len = r.InputShapes[i][axis];
        if (r.NeedsInputGrad(i)) Engine::Emit(r, i, g.Slice(axis, start, start + len).Clone(), true);
        start += len;
      }
      break;
    }
    default: RunSpatialBackward(e, r, g); break;
  }
}

}  // namespace omh
