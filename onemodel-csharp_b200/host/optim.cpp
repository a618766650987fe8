// Optimizers, gradient clipping and learning-rate schedules, after src/OneModel.Training/{Optimizers,Schedules}.cs.
// The per-step scalars are computed here on the host in double exactly as the reference does; the per-element
// update runs in one fused multi-tensor launch on the device.
#include <math.h>

#include <map>

#include "omh.hpp"

namespace omh {

static om_ctx* C() { return Device::Current(); }

Optimizer::Optimizer(std::vector<Tensor> parameters) : params_(std::move(parameters)) {
  for (const Tensor& p : params_) {
    if (p.GetDType() != DType::F32 || !p.IsContiguous())
      throw TensorShapeException("Optimizers need contiguous float32 parameters.");
  }
}

void Optimizer::ZeroGrad() {
  for (const Tensor& p : params_) Backprop::ZeroGrad(p);
}

// The parameters of the running launch that are product operands under bfloat16 products (their storage has a bfloat16
// copy) get that copy refreshed by the launch itself, when the launch covers the whole storage.
void Optimizer::OfferBf16Copies() {
  p16_.assign(index_.size(), nullptr);
  if (!WritesBf16Copies()) return;
  std::map<const Buffer*, int64_t> covered;
  for (int i : index_) {
    const Tensor& t = params_[(size_t)i];
    if (t.HasBf16Storage()) covered[t.Storage().get()] += t.Length();
  }
  for (size_t k = 0; k < index_.size(); k++) {
    const Tensor& t = params_[(size_t)index_[k]];
    if (t.HasBf16Storage() && covered[t.Storage().get()] == (int64_t)(t.Storage()->bytes / 4)) p16_[k] = t.Bf16ForWrite();
  }
}

void Optimizer::Bf16CopiesWritten() {
  for (size_t k = 0; k < index_.size(); k++)
    if (p16_[k]) params_[(size_t)index_[k]].Bf16Written();
}

void Optimizer::UpdateSparse(int index, const Tensor&, const RowSparseGradient&) {
  throw InvalidOperationException("Parameter " + std::to_string(index) + " has a row-sparse gradient, which this optimizer (" + Kind() +
                                  ") does not support; use Sgd without momentum or SparseAdam for it.");
}

// Optimizer.Step (Optimizers.cs:184-219): parameters without a gradient are skipped; one with a row-sparse gradient goes
// through UpdateSparse.
void Optimizer::Step() {
  BeginStep();
  std::vector<float*> p;
  std::vector<const float*> g;
  std::vector<int64_t> len;
  index_.clear();
  for (size_t i = 0; i < params_.size(); i++) {
    const Tensor& t = params_[i];
    if (!t.RequiresGrad()) continue;
    if (t.Autograd() && t.Autograd()->SparseGrad) {
      UpdateSparse((int)i, t, *t.Autograd()->SparseGrad);
      t.MarkModified();
      continue;
    }
    Tensor grad = t.Grad();  // materialises zeros if the step produced no gradient for this parameter
    if (grad.IsEmpty()) continue;
    p.push_back(t.Data());
    g.push_back(grad.Data());
    len.push_back(t.Length());
    index_.push_back((int)i);
  }
  OfferBf16Copies();
  Launch(p, g, len);
  for (int i : index_) params_[(size_t)i].MarkModified();   // written in place: saved copies and bfloat16 copies are stale
  Bf16CopiesWritten();                                      // ... except the copies the launch itself refreshed
  StepCount++;
}

void Optimizer::StepGroups(const std::vector<std::vector<int>>& groups, const std::function<void(int)>& before) {
  BeginStep();
  for (size_t gi = 0; gi < groups.size(); gi++) {
    std::vector<float*> p;
    std::vector<const float*> g;
    std::vector<int64_t> len;
    index_.clear();
    for (int i : groups[gi]) {
      const Tensor& t = params_[(size_t)i];
      if (!t.RequiresGrad()) continue;
      if (t.Autograd() && t.Autograd()->SparseGrad) {
        UpdateSparse(i, t, *t.Autograd()->SparseGrad);
        t.MarkModified();
        continue;
      }
      Tensor grad = t.Grad();
      if (grad.IsEmpty()) continue;
      p.push_back(t.Data());
      g.push_back(grad.Data());
      len.push_back(t.Length());
      index_.push_back(i);
    }
    if (before) before((int)gi);
    OfferBf16Copies();
    if (!p.empty()) Launch(p, g, len);
    for (int i : index_) params_[(size_t)i].MarkModified();
    Bf16CopiesWritten();
  }
  StepCount++;
}

// ---- SGD ------------------------------------------------------------------------------------------------------------
Sgd::Sgd(std::vector<Tensor> parameters, float lr, float momentum, float dampening, float weightDecay, bool nesterov)
    : Optimizer(std::move(parameters)), momentum_(momentum), dampening_(dampening), nesterov_(nesterov) {
  LearningRate = lr;
  WeightDecay = weightDecay;
  if (nesterov && (momentum <= 0.f || dampening != 0.f))
    throw std::invalid_argument("Nesterov momentum needs a positive momentum and zero dampening.");
  if (momentum != 0.f) {
    for (const Tensor& p : params_) buffers_.push_back(Tensor::Zeros(DType::F32, p.GetShape()));
    initialized_.assign(params_.size(), 0);
  }
}

// Optimizers.cs:317-318 and 300-311: flags first, then the momentum buffers.
std::vector<std::pair<std::string, float>> Sgd::HyperParameters() const {
  return {{"lr", LearningRate}, {"momentum", momentum_}, {"dampening", dampening_}, {"weight_decay", WeightDecay}, {"nesterov", nesterov_ ? 1.f : 0.f}};
}
std::vector<Optimizer::StateEntry> Sgd::NamedState() {
  if (initialized_.size() != params_.size()) initialized_.resize(params_.size(), 0);
  std::vector<StateEntry> out;
  StateEntry flags;
  flags.name = "initialized";
  flags.flags = &initialized_;
  out.push_back(flags);
  for (size_t i = 0; i < buffers_.size(); i++) out.push_back({"momentum_buffer." + std::to_string(i), buffers_[i], nullptr});
  return out;
}

void Sgd::FillHyper(void* host, int64_t) const {
  om_sgd_hyper* h = (om_sgd_hyper*)host;
  h->lr = LearningRate;
  h->weight_decay = WeightDecay;
  h->momentum = momentum_;
  h->dampening = dampening_;
  h->grad_scale = GradScale;
  h->nesterov = nesterov_;
  h->has_momentum = momentum_ != 0.f;
}

void Sgd::Launch(const std::vector<float*>& p, const std::vector<const float*>& g, const std::vector<int64_t>& len) {
  om_sgd_hyper h;
  FillHyper(&h, StepCount + 1);
  std::vector<float*> buf;
  std::vector<int32_t> first;
  if (h.has_momentum) {
    for (int i : index_) {
      buf.push_back(buffers_[i].Data());
      first.push_back(initialized_[i] == 0);
      initialized_[i] = 1;
    }
  }
  Check(om_optim_sgd_step(C(), (int32_t)p.size(), p.data(), g.data(), h.has_momentum ? buf.data() : nullptr,
                          h.has_momentum ? first.data() : nullptr, len.data(), &h, (const om_sgd_hyper*)HyperDevice));
}

void Sgd::UpdateSparse(int, const Tensor& parameter, const RowSparseGradient& gradient) {
  if (momentum_ != 0.f || WeightDecay != 0.f)
    throw NotSupportedException("Sgd supports row-sparse gradients only without momentum and weight decay.");
  const Shape& ds = gradient.DenseShape();
  Check(om_optim_sparse_sgd_step_rows(C(), parameter.Data(), (const int32_t*)gradient.RowsStorage().RawData(), gradient.ValuesStorage().Data(),
                                      (const int32_t*)gradient.CountStorage().RawData(), gradient.Capacity(), ds[0], ds[1], LearningRate));
}

// ---- Adam -----------------------------------------------------------------------------------------------------------
Adam::Adam(std::vector<Tensor> parameters, float lr, float beta1, float beta2, float eps, float weightDecay, bool decoupled,
           bool amsgrad)
    : Optimizer(std::move(parameters)), beta1_(beta1), beta2_(beta2), eps_(eps), decoupled_(decoupled), amsgrad_(amsgrad) {
  LearningRate = lr;
  WeightDecay = weightDecay;
  for (const Tensor& p : params_) {
    m_.push_back(Tensor::Zeros(DType::F32, p.GetShape()));
    v_.push_back(Tensor::Zeros(DType::F32, p.GetShape()));
    if (amsgrad) vmax_.push_back(Tensor::Zeros(DType::F32, p.GetShape()));
  }
}

std::vector<Tensor> Adam::StateTensors() const {
  std::vector<Tensor> s = m_;
  s.insert(s.end(), v_.begin(), v_.end());
  s.insert(s.end(), vmax_.begin(), vmax_.end());
  return s;
}

// Optimizers.cs:466-467; state slots exp_avg, exp_avg_sq (and max_exp_avg_sq with amsgrad), each named slot.index.
std::vector<std::pair<std::string, float>> Adam::HyperParameters() const {
  return {{"lr", LearningRate}, {"beta1", beta1_}, {"beta2", beta2_}, {"epsilon", eps_}, {"weight_decay", WeightDecay}, {"amsgrad", amsgrad_ ? 1.f : 0.f}};
}
std::vector<Optimizer::StateEntry> Adam::NamedState() {
  std::vector<StateEntry> out;
  for (size_t i = 0; i < m_.size(); i++) out.push_back({"exp_avg." + std::to_string(i), m_[i], nullptr});
  for (size_t i = 0; i < v_.size(); i++) out.push_back({"exp_avg_sq." + std::to_string(i), v_[i], nullptr});
  for (size_t i = 0; i < vmax_.size(); i++) out.push_back({"max_exp_avg_sq." + std::to_string(i), vmax_[i], nullptr});
  return out;
}

// Adam.IntPow: binary powering in double (Optimizers.cs:483-499).
static double IntPow(double b, int64_t n) {
  double result = 1.0;
  while (n > 0) {
    if (n & 1) result *= b;
    b *= b;
    n >>= 1;
  }
  return result;
}

// Adam.BeginStep (Optimizers.cs:501-508).
void Adam::FillHyper(void* host, int64_t t) const {
  om_adam_hyper* h = (om_adam_hyper*)host;
  double bc1 = 1.0 - IntPow((double)beta1_, t);
  double bc2 = 1.0 - IntPow((double)beta2_, t);
  h->lr = LearningRate;
  h->beta1 = beta1_;
  h->beta2 = beta2_;
  h->eps = eps_;
  h->weight_decay = WeightDecay;
  h->step_size = (float)((double)LearningRate / bc1);
  h->sqrt_bc2 = (float)sqrt(bc2);
  h->grad_scale = GradScale;
  h->decoupled = decoupled_;
  h->amsgrad = amsgrad_;
}

void Adam::Launch(const std::vector<float*>& p, const std::vector<const float*>& g, const std::vector<int64_t>& len) {
  om_adam_hyper h;
  FillHyper(&h, StepCount + 1);
  std::vector<float*> m, v, vm;
  for (int i : index_) {
    m.push_back(m_[i].Data());
    v.push_back(v_[i].Data());
    if (amsgrad_) vm.push_back(vmax_[i].Data());
  }
  Check(om_optim_adam_step_b16(C(), (int32_t)p.size(), p.data(), g.data(), m.data(), v.data(), amsgrad_ ? vm.data() : nullptr,
                               p16_.size() == p.size() ? p16_.data() : nullptr, len.data(), &h, (const om_adam_hyper*)HyperDevice));
}

// ---- SparseAdam (Optimizers.cs:625-722) ------------------------------------------------------------------------------
SparseAdam::SparseAdam(std::vector<Tensor> parameters, float lr, float beta1, float beta2, float eps)
    : Optimizer(std::move(parameters)), beta1_(beta1), beta2_(beta2), eps_(eps) {
  LearningRate = lr;
  if (!(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f)) throw ArgumentOutOfRangeException("Betas must be in [0, 1).");
  if (!(eps > 0.f) || !std::isfinite(eps)) throw ArgumentOutOfRangeException("Epsilon must be positive and finite.");
  for (const Tensor& p : params_) {
    if (p.Rank() != 2) throw std::invalid_argument("SparseAdam parameters must be rank 2 ([rows, width]) tables.");
    m_.push_back(Tensor::Zeros(DType::F32, p.GetShape()));
    v_.push_back(Tensor::Zeros(DType::F32, p.GetShape()));
  }
}

std::vector<Tensor> SparseAdam::StateTensors() const {
  std::vector<Tensor> out = m_;
  out.insert(out.end(), v_.begin(), v_.end());
  return out;
}
std::vector<std::pair<std::string, float>> SparseAdam::HyperParameters() const {
  return {{"lr", LearningRate}, {"beta1", beta1_}, {"beta2", beta2_}, {"epsilon", eps_}};
}
std::vector<Optimizer::StateEntry> SparseAdam::NamedState() {
  std::vector<StateEntry> out;
  for (size_t i = 0; i < m_.size(); i++) out.push_back({"exp_avg." + std::to_string(i), m_[i], nullptr});
  for (size_t i = 0; i < v_.size(); i++) out.push_back({"exp_avg_sq." + std::to_string(i), v_[i], nullptr});
  return out;
}

// lr * sqrt(1 - beta2^t) / (1 - beta1^t) in double, rounded once (SparseAdam.BeginStep, Optimizers.cs:684-690).
void SparseAdam::BeginStep() {
  const int64_t t = StepCount + 1;
  const double bc1 = 1.0 - IntPow((double)beta1_, t), bc2 = 1.0 - IntPow((double)beta2_, t);
  step_size_ = (float)((double)LearningRate * sqrt(bc2) / bc1);
}

void SparseAdam::Launch(const std::vector<float*>& p, const std::vector<const float*>&, const std::vector<int64_t>&) {
  if (p.empty()) return;
  throw InvalidOperationException("SparseAdam got a dense gradient for parameter " + std::to_string(index_.empty() ? 0 : index_[0]) +
                                  "; it only handles row-sparse gradients (build the Embedding with sparse: true, or use Adam).");
}

void SparseAdam::UpdateSparse(int index, const Tensor& parameter, const RowSparseGradient& gradient) {
  const Shape& ds = gradient.DenseShape();
  Check(om_optim_sparse_adam_step_rows(C(), parameter.Data(), (const int32_t*)gradient.RowsStorage().RawData(), gradient.ValuesStorage().Data(),
                                       (const int32_t*)gradient.CountStorage().RawData(), gradient.Capacity(), m_[(size_t)index].Data(),
                                       v_[(size_t)index].Data(), ds[0], ds[1], beta1_, beta2_, eps_, step_size_));
  m_[(size_t)index].MarkModified();
  v_[(size_t)index].MarkModified();
}

// ---- clipping -------------------------------------------------------------------------------------------------------
// The values of a row-sparse gradient stand in for the gradient, each row counted once (Schedules.cs:33,72,130); the entries
// behind its row count are zero, so the whole storage is normed and scaled.
static void CollectGrads(const std::vector<Tensor>& parameters, std::vector<float*>& g, std::vector<int64_t>& len) {
  for (const Tensor& p : parameters) {
    if (p.Autograd() && p.Autograd()->SparseGrad) {
      const Tensor& values = p.Autograd()->SparseGrad->ValuesStorage();
      g.push_back(values.Data());
      len.push_back(values.Length());
      continue;
    }
    Tensor grad = p.Grad();
    if (grad.IsEmpty()) continue;
    g.push_back(grad.Data());
    len.push_back(grad.Length());
  }
}

void GradClip::ClipNormAsync(const std::vector<Tensor>& parameters, float maxNorm, bool infinityNorm, float* norm_out) {
  if (!(maxNorm > 0.f)) throw ArgumentOutOfRangeException("The maximum norm must be positive.");
  std::vector<float*> g;
  std::vector<int64_t> len;
  CollectGrads(parameters, g, len);
  Check(om_grad_norm_clip(C(), (int32_t)g.size(), g.data(), len.data(), maxNorm, infinityNorm, norm_out));
}

float GradClip::ClipNorm(const std::vector<Tensor>& parameters, float maxNorm, bool infinityNorm) {
  Tensor norm = Tensor::Create(DType::F32, Shape{});
  ClipNormAsync(parameters, maxNorm, infinityNorm, norm.Data());
  return norm.Item();
}

void GradClip::ClipValue(const std::vector<Tensor>& parameters, float clipValue) {
  if (!(clipValue >= 0.f)) throw ArgumentOutOfRangeException("The bound must not be negative.");
  std::vector<float*> g;
  std::vector<int64_t> len;
  CollectGrads(parameters, g, len);
  Check(om_grad_clip_value(C(), (int32_t)g.size(), g.data(), len.data(), clipValue));
}

// ---- schedules (Schedules.cs:151-422) ------------------------------------------------------------------------------
void LrSchedule::Apply(Optimizer& optimizer) const { optimizer.LearningRate = LrAt(optimizer.StepCount); }

double LrSchedule::Cos(double t) {
  if (!(t > 0.0)) return 1.0;
  if (t >= 1.0) return -1.0;
  const bool mirrored = t > 0.5;
  const double angle = 3.14159265358979323846 * (mirrored ? 1.0 - t : t);
  const double sq = angle * angle;
  double series = 1.0;
  for (int term = 13; term >= 1; term--) series = 1.0 - sq / ((2.0 * term - 1.0) * (2.0 * term)) * series;
  return mirrored ? -series : series;
}

namespace {

int64_t NotNegative(int64_t step) { return step < 0 ? 0 : step; }

struct ConstantRate final : LrSchedule {
  float lr;
  explicit ConstantRate(float v) : lr(v) {}
  float LrAt(int64_t) const override { return lr; }
};

struct StepRate final : LrSchedule {
  double base, gamma;
  int64_t every;
  StepRate(float b, int64_t e, float g) : base(b), gamma(g), every(e) {}
  float LrAt(int64_t step) const override {
    double rate = base, factor = gamma;
    for (int64_t drops = NotNegative(step) / every; drops > 0; drops >>= 1) {
      if (drops & 1) rate *= factor;
      factor *= factor;
    }
    return (float)rate;
  }
};

struct CosineRate final : LrSchedule {
  double base, floor;
  int64_t total;
  CosineRate(float b, int64_t t, float m) : base(b), floor(m), total(t) {}
  float LrAt(int64_t step) const override {
    const int64_t s = NotNegative(step);
    const double t = s >= total ? 1.0 : (double)s / (double)total;
    return (float)(floor + (base - floor) * (1.0 + Cos(t)) / 2.0);
  }
};

struct WarmupRate final : LrSchedule {
  std::shared_ptr<LrSchedule> after;
  int64_t warmup;
  double start;
  WarmupRate(std::shared_ptr<LrSchedule> a, int64_t w, float s) : after(std::move(a)), warmup(w), start(s) {}
  float LrAt(int64_t step) const override {
    const int64_t s = NotNegative(step);
    if (s >= warmup) return after->LrAt(s - warmup);
    const double first = after->LrAt(0);
    return (float)(first * (start + (1.0 - start) * ((double)s / (double)warmup)));
  }
};

struct WarmupCosineRate final : LrSchedule {
  double base, floor;
  int64_t warmup, total;
  WarmupCosineRate(float b, int64_t w, int64_t t, float f) : base(b), floor(f), warmup(w), total(t) {}
  float LrAt(int64_t step) const override {
    const int64_t s = NotNegative(step);
    if (s < warmup) return (float)(base * (double)(s + 1) / (double)warmup);
    const int64_t span = total - warmup > 1 ? total - warmup : 1;
    double p = (double)(s - warmup) / (double)span;
    if (p > 1.0) p = 1.0;
    return (float)(base * (floor + ((1.0 - floor) * 0.5 * (1.0 + Cos(p)))));
  }
};

struct OneCycleRate final : LrSchedule {
  double peak, first, last, up_end, down_end;
  OneCycleRate(float maxLr, int64_t total, float pct, float div, float finalDiv)
      : peak(maxLr), first((double)maxLr / div), last(first / finalDiv), up_end((double)pct * (double)total - 1.0),
        down_end((double)total - 1.0) {}
  static double Anneal(double from, double to, double pct) { return to + (from - to) / 2.0 * (Cos(pct) + 1.0); }
  float LrAt(int64_t step) const override {
    double s = (double)NotNegative(step);
    if (s > down_end) s = down_end;
    return s <= up_end ? (float)Anneal(first, peak, s / up_end) : (float)Anneal(peak, last, (s - up_end) / (down_end - up_end));
  }
};

}  // namespace

std::shared_ptr<LrSchedule> LrSchedule::Constant(float lr) { return std::make_shared<ConstantRate>(lr); }

std::shared_ptr<LrSchedule> LrSchedule::Step(float baseLr, int64_t stepSize, float gamma) {
  if (stepSize < 1) throw ArgumentOutOfRangeException("The step size must be at least 1.");
  return std::make_shared<StepRate>(baseLr, stepSize, gamma);
}

std::shared_ptr<LrSchedule> LrSchedule::Cosine(float baseLr, int64_t totalSteps, float minLr) {
  if (totalSteps < 1) throw ArgumentOutOfRangeException("The number of steps must be at least 1.");
  return std::make_shared<CosineRate>(baseLr, totalSteps, minLr);
}

std::shared_ptr<LrSchedule> LrSchedule::Warmup(std::shared_ptr<LrSchedule> after, int64_t warmupSteps, float startFactor) {
  if (!after) throw std::invalid_argument("A warm-up needs the schedule that follows it.");
  if (warmupSteps < 1) throw ArgumentOutOfRangeException("The warm-up must last at least 1 step.");
  return std::make_shared<WarmupRate>(std::move(after), warmupSteps, startFactor);
}

std::shared_ptr<LrSchedule> LrSchedule::WarmupCosine(float baseLr, int64_t warmupSteps, int64_t totalSteps, float floorFraction) {
  if (warmupSteps < 1) throw ArgumentOutOfRangeException("The warm-up must last at least 1 step.");
  if (totalSteps <= warmupSteps) throw ArgumentOutOfRangeException("The total must exceed the warm-up.");
  if (!(floorFraction >= 0.f && floorFraction <= 1.f)) throw ArgumentOutOfRangeException("The floor fraction must be in [0, 1].");
  return std::make_shared<WarmupCosineRate>(baseLr, warmupSteps, totalSteps, floorFraction);
}

std::shared_ptr<LrSchedule> LrSchedule::OneCycle(float maxLr, int64_t totalSteps, float pctStart, float divFactor, float finalDivFactor) {
  if (totalSteps < 2) throw ArgumentOutOfRangeException("One cycle needs at least 2 steps.");
  if (!(pctStart > 0.f && pctStart < 1.f)) throw ArgumentOutOfRangeException("pctStart must be in (0, 1).");
  return std::make_shared<OneCycleRate>(maxLr, totalSteps, pctStart, divFactor, finalDivFactor);
}

}  // namespace omh
