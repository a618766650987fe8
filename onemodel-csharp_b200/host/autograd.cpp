// The tape and the reverse-mode engine: the same traversal and accumulation order as the reference's
// Backprop.Run / Engine.Execute / Emit / AccumulateLeaf (src/OneModel/Tensors/Autograd/Engine.cs:28-344).
#include <atomic>

#include "omh.hpp"

namespace omh {

static thread_local bool t_grad_enabled = true;
static thread_local ActivationScope* t_scope = nullptr;
static std::atomic<int> s_pass{0};
std::function<void(AutogradMeta*)> Backprop::GradReadyHook;

bool GradMode::Enabled() { return t_grad_enabled; }
GradMode::NoGrad::NoGrad() : prev(t_grad_enabled) { t_grad_enabled = false; }
GradMode::NoGrad::~NoGrad() { t_grad_enabled = prev; }

ActivationScope::ActivationScope() : outer(t_scope) { t_scope = this; }
ActivationScope::~ActivationScope() {
  tracked.clear();
  t_scope = outer;
}
void ActivationScope::Track(const Tensor& t) {
  if (t_scope) t_scope->tracked.push_back(t);
}

std::shared_ptr<BackwardRecord> BackwardRecord::Create(OpKind op, int savedSlots, const std::vector<Tensor>& inputs) {
  auto rec = std::make_shared<BackwardRecord>();
  rec->Op = op;
  rec->SavedSlots.resize(savedSlots);
  rec->SavedVersions.assign(savedSlots, 0);
  for (const Tensor& t : inputs) {
    rec->Inputs.push_back(t.RequiresGrad() ? t.Autograd() : nullptr);
    rec->InputShapes.push_back(t.GetShape());
    rec->InputTypes.push_back(t.GetDType());
  }
  return rec;
}

std::shared_ptr<BackwardRecord> BackwardRecord::Create(OpKind op, int savedSlots, std::initializer_list<const Tensor*> inputs) {
  std::vector<Tensor> v;
  for (const Tensor* t : inputs) v.push_back(*t);
  return Create(op, savedSlots, v);
}

Tensor BackwardRecord::Attach(const Tensor& output, int outputIndex) {
  auto meta = std::make_shared<AutogradMeta>();
  meta->RequiresGrad = true;
  meta->GradFn = shared_from_this();
  meta->OutputIndex = outputIndex;
  return output.WithAutograd(meta);
}

const Tensor& BackwardRecord::Saved(int slot) const {
  const Tensor& t = SavedSlots[slot];
  if (!t.IsEmpty() && t.Version() != SavedVersions[slot])
    throw TensorVersionException("A tensor saved for the backward pass was modified in place (saved at version " +
                                 std::to_string(SavedVersions[slot]) + ", now " + std::to_string(t.Version()) + ").");
  return t;
}

void BackwardRecord::Release() {
  IsReleased = true;
  for (Tensor& t : SavedSlots) t = Tensor();
}

void Backprop::Run(const Tensor& root, const Tensor* gradient, bool retainGraph) {
  if (root.IsEmpty() || !root.RequiresGrad()) throw InvalidOperationException("Backward needs a tensor that requires gradients.");
  Tensor g;
  if (gradient) {
    if (gradient->GetShape() != root.GetShape())
      throw TensorShapeException("The gradient has shape " + gradient->GetShape().ToString() + ", the tensor " + root.GetShape().ToString() + ".");
    g = gradient->Clone();
  } else {
    if (root.Length() != 1) throw TensorShapeException("Backward without a gradient needs a one-element tensor.");
    g = Tensor::Create(DType::F32, root.GetShape());
    g.Fill(1.f);
  }
  auto meta = root.Autograd();
  GradMode::NoGrad noGrad;
  Engine engine;
  if (!meta->GradFn) {
    Engine::AccumulateLeaf(*meta, g, true);
    return;
  }
  engine.Execute(meta->GradFn, g, retainGraph);
}

// A row-sparse gradient is freed instead of zeroed: zero is the absence of rows (Engine.cs:75-90).
void Backprop::ZeroGrad(const Tensor& leaf) {
  auto& m = leaf.Autograd();
  if (m) m->SparseGrad.reset();
  if (m && !m->Grad.IsEmpty()) m->GradIsZero = true;
}

void Backprop::ClearGrad(const Tensor& leaf) {
  auto& m = leaf.Autograd();
  if (m) {
    m->SparseGrad.reset();
    m->Grad = Tensor();
    m->GradIsZero = false;
  }
}

// Leaves reached by the traversal, with the number of tape edges that will deliver a gradient to each: when the
// count reaches zero the leaf's gradient is final for this pass.
static thread_local std::vector<std::pair<AutogradMeta*, int>>* t_leaf_edges = nullptr;

static void leaf_arrived(AutogradMeta* leaf) {
  if (!t_leaf_edges) return;
  for (auto& kv : *t_leaf_edges) {
    if (kv.first == leaf) {
      if (--kv.second == 0 && Backprop::GradReadyHook) Backprop::GradReadyHook(leaf);
      return;
    }
  }
}

void Engine::Execute(const std::shared_ptr<BackwardRecord>& root, Tensor rootGrad, bool retain) {
  int mark = ++s_pass;
  std::vector<BackwardRecord*> order;
  std::vector<std::pair<BackwardRecord*, int>> stack;
  std::vector<std::pair<AutogradMeta*, int>> leaf_edges;
  root->VisitMark = mark;
  stack.emplace_back(root.get(), 0);
  while (!stack.empty()) {
    BackwardRecord* rec = stack.back().first;
    int next = stack.back().second;
    if (rec->IsReleased)
      throw InvalidOperationException(
          "Backward ran through a graph whose saved tensors were already freed by an earlier backward. Pass retainGraph: true to the first call.");
    if (next < rec->InputCount()) {
      stack.back().second = next + 1;
      AutogradMeta* in = rec->Inputs[next].get();
      if (in && in->GradFn) {
        BackwardRecord* producer = in->GradFn.get();
        if (producer->VisitMark != mark) {
          producer->VisitMark = mark;
          stack.emplace_back(producer, 0);
        }
      } else if (in && in->RequiresGrad) {
        bool found = false;
        for (auto& kv : leaf_edges)
          if (kv.first == in) {
            kv.second++;
            found = true;
            break;
          }
        if (!found) leaf_edges.emplace_back(in, 1);
      }
    } else {
      order.push_back(rec);
      stack.pop_back();
    }
  }

  root->PendingGrad = rootGrad;
  t_leaf_edges = &leaf_edges;
  struct Cleanup {
    std::vector<BackwardRecord*>& order;
    ~Cleanup() {
      for (BackwardRecord* r : order) {
        r->PendingGrad = Tensor();
        r->PendingShared = false;
      }
      t_leaf_edges = nullptr;
    }
  } cleanup{order};
  for (int i = (int)order.size() - 1; i >= 0; i--) {
    BackwardRecord* rec = order[i];
    Tensor g = rec->PendingGrad;
    rec->PendingGrad = Tensor();
    current_shared_ = rec->PendingShared;
    rec->PendingShared = false;
    if (g.IsEmpty()) {
      // No gradient reached this record: its leaf inputs still count as served.
      for (auto& in : rec->Inputs)
        if (in && !in->GradFn) leaf_arrived(in.get());
      continue;
    }
    RunBackwardOp(*this, *rec, g);
    if (!retain) rec->Release();
  }
}

void Engine::Emit(BackwardRecord& rec, int i, const Tensor& grad, bool owned) {
  AutogradMeta* meta = rec.Inputs[i].get();
  if (!meta) return;
  if (!meta->GradFn) {
    AccumulateLeaf(*meta, grad, owned);
    leaf_arrived(meta);
    return;
  }
  BackwardRecord& p = *meta->GradFn;
  if (p.PendingGrad.IsEmpty()) {
    // The first gradient to arrive is adopted as it is; one that its sender does not give away stays shared and is copied only
    // if something has to be added into it.
    p.PendingGrad = grad;
    p.PendingShared = !owned;
  } else {
    if (p.PendingShared) {
      p.PendingGrad = p.PendingGrad.Clone();
      p.PendingShared = false;
    }
    AddInto(p.PendingGrad, grad);
  }
}

void Engine::EmitSparse(BackwardRecord& rec, int i, std::shared_ptr<RowSparseGradient> grad) {
  AutogradMeta* meta = rec.Inputs[i].get();
  if (!meta) return;
  if (meta->GradFn) {
    // The table is itself computed (not a leaf): later operations want a dense gradient.
    Emit(rec, i, grad->ToDense(), true);
    return;
  }
  if (!meta->RequiresGrad) return;
  if (!meta->Grad.IsEmpty()) {
    if (meta->GradIsZero) {
      meta->Grad.Fill(0.f);
      meta->GradIsZero = false;
    }
    grad->AddTo(meta->Grad);
  } else if (!meta->SparseGrad) {
    meta->SparseGrad = std::move(grad);
  } else {
    meta->SparseGrad = RowSparseGradient::Merge(*meta->SparseGrad, *grad);
  }
  leaf_arrived(meta);
}

void Engine::AccumulateLeaf(AutogradMeta& leaf, const Tensor& grad, bool owned) {
  if (!leaf.RequiresGrad) return;
  if (leaf.SparseGrad) {
    // A dense gradient arrives for a leaf that already has a sparse one (a table used by a lookup and by something
    // else): go dense (Engine.cs:305-311).
    leaf.Grad = leaf.SparseGrad->ToDense();
    leaf.GradIsZero = false;
    leaf.SparseGrad.reset();
  }
  if (leaf.Grad.IsEmpty()) {
    // A view (aliased gradient) must not be adopted: the leaf's gradient outlives the step.
    leaf.Grad = (owned && grad.IsContiguous() && grad.Offset() == 0) ? grad.Detach() : grad.Clone();
    leaf.GradIsZero = false;
  } else if (leaf.GradIsZero) {
    // Logically 0 + grad: overwrite instead of zero-fill then add.
    Tensor src = grad.Contiguous();
    Check(om_memcpy_d2d(Device::Current(), leaf.Grad.RawData(), src.RawData(), (size_t)src.Length() * 4));
    leaf.Grad.MarkModified();
    leaf.GradIsZero = false;
  } else {
    AddInto(leaf.Grad, grad);
  }
}

bool Engine::LeafTarget(BackwardRecord& rec, int i, float** ptr, bool* accumulate) {
  AutogradMeta* meta = rec.Inputs[i].get();
  if (!meta || meta->GradFn || !meta->RequiresGrad) return false;
  if (meta->Grad.IsEmpty()) {
    meta->Grad = Tensor::Create(DType::F32, rec.InputShapes[i]);
    meta->GradIsZero = true;
  }
  if (meta->Grad.GetShape() != rec.InputShapes[i]) return false;
  *ptr = meta->Grad.Data();
  *accumulate = !meta->GradIsZero;
  return true;
}

void Engine::LeafWritten(BackwardRecord& rec, int i) {
  AutogradMeta* meta = rec.Inputs[i].get();
  meta->GradIsZero = false;
  meta->Grad.MarkModified();
  leaf_arrived(meta);
}

bool Engine::PendingTarget(BackwardRecord& rec, int i, Tensor* pending, bool* shared) {
  AutogradMeta* meta = rec.Inputs[i].get();
  if (!meta || !meta->GradFn) return false;
  const Tensor& p = meta->GradFn->PendingGrad;
  if (p.IsEmpty() || !p.IsContiguous() || p.GetDType() != DType::F32 || p.GetShape() != rec.InputShapes[i]) return false;
  *pending = p;
  *shared = meta->GradFn->PendingShared;
  return true;
}

void Engine::PendingReplace(BackwardRecord& rec, int i, const Tensor& sum) {
  BackwardRecord& p = *rec.Inputs[i]->GradFn;
  p.PendingGrad = sum;
  p.PendingShared = false;
}

Tensor Engine::PendingOwn(BackwardRecord& rec, int i) {
  BackwardRecord& p = *rec.Inputs[i]->GradFn;
  if (p.PendingShared) {
    p.PendingGrad = p.PendingGrad.Clone();
    p.PendingShared = false;
  }
  return p.PendingGrad;
}

void Engine::PendingWritten(BackwardRecord& rec, int i) { rec.Inputs[i]->GradFn->PendingGrad.MarkModified(); }

void Engine::AddInto(const Tensor& dst, const Tensor& src) {
  if (dst.GetShape() != src.GetShape())
    throw TensorShapeException("Gradient shape " + src.GetShape().ToString() + " does not match " + dst.GetShape().ToString() + ".");
  Tensor s = src.Contiguous();
  Check(om_add_into(Device::Current(), dst.Data(), s.Data(), dst.Length()));
  dst.MarkModified();
}

// ---- RowSparseGradient (RowSparseGradient.cs:14-120) --------------------------------------------------------------------
int RowSparseGradient::RowCount() const {
  int32_t n = 0;
  count_.CopyToHost(&n);
  return n;
}

std::vector<int32_t> RowSparseGradient::Rows() const {
  const int n = RowCount();
  std::vector<int32_t> all((size_t)Capacity());
  rows_.CopyToHost(all.data());
  all.resize((size_t)n);
  return all;
}

Tensor RowSparseGradient::Values() const { return values_.Slice(0, 0, RowCount()); }

void RowSparseGradient::AddTo(const Tensor& dense) const {
  if (dense.GetDType() != DType::F32 || dense.GetShape() != dense_shape_ || !dense.IsContiguous())
    throw TensorShapeException("A row-sparse gradient of a " + dense_shape_.ToString() + " table cannot be added to " + dense.GetShape().ToString() + ".");
  Check(om_rowsparse_add_to(Device::Current(), (const int32_t*)rows_.RawData(), values_.Data(), (const int32_t*)count_.RawData(), Capacity(),
                            dense_shape_[1], dense.Data(), dense_shape_[0]));
  dense.MarkModified();
}

Tensor RowSparseGradient::ToDense() const {
  Tensor dense = Tensor::Zeros(DType::F32, dense_shape_);
  AddTo(dense);
  return dense;
}

std::shared_ptr<RowSparseGradient> RowSparseGradient::Merge(const RowSparseGradient& a, const RowSparseGradient& b) {
  if (a.dense_shape_ != b.dense_shape_) throw TensorShapeException("Row-sparse gradients of different tables cannot be merged.");
  const int v = a.dense_shape_[0], width = a.dense_shape_[1];
  const int cap = (int)std::min<int64_t>((int64_t)a.Capacity() + b.Capacity(), v);
  Tensor rows = Tensor::Create(DType::I32, Shape{cap}), values = Tensor::Create(DType::F32, Shape{cap, width}), count = Tensor::Create(DType::I32, Shape{1});
  Check(om_rowsparse_merge(Device::Current(), (const int32_t*)a.rows_.RawData(), a.values_.Data(), (const int32_t*)a.count_.RawData(), a.Capacity(),
                           (const int32_t*)b.rows_.RawData(), b.values_.Data(), (const int32_t*)b.count_.RawData(), b.Capacity(), v, width,
                           (int32_t*)rows.RawData(), values.Data(), cap, (int32_t*)count.RawData()));
  return std::make_shared<RowSparseGradient>(a.dense_shape_, rows, values, count);
}

}  // namespace omh
