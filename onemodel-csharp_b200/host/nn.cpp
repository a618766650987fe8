// Modules and initialisation, after src/OneModel.Training/{NnModule,Layers,Recurrent,Generator,Losses}.cs.
#include <math.h>

#include "omh.hpp"

namespace omh {

uint64_t Generator::NextUInt64() {
  state_ += 0x9E3779B97F4A7C15ULL;
  uint64_t z = state_;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

// Init.Uniform (Layers.cs:11-21): uniform in [-bound, bound), drawn in row-major order.
static Tensor InitUniform(Generator& g, float bound, const Shape& s) {
  std::vector<float> h((size_t)s.Length());
  for (float& v : h) v = g.Uniform(-bound, bound);
  return Tensor::FromHost(h.data(), s);
}

static Tensor InitConstant(float value, const Shape& s) {
  Tensor t = Tensor::Create(DType::F32, s);
  t.Fill(value);
  return t;
}

Tensor NnModule::RegisterParameter(const std::string& name, Tensor t) {
  t.SetRequiresGrad(true);
  params_.emplace_back(name, t);
  return t;
}

std::vector<std::pair<std::string, Tensor>> NnModule::NamedParameters(const std::string& prefix) const {
  std::vector<std::pair<std::string, Tensor>> out;
  for (auto& p : params_) out.emplace_back(prefix + p.first, p.second);
  for (auto& c : children_) {
    auto sub = c.second->NamedParameters(prefix + c.first + ".");
    out.insert(out.end(), sub.begin(), sub.end());
  }
  return out;
}

Tensor NnModule::RegisterBuffer(const std::string& name, Tensor t) {
  buffers_.emplace_back(name, t);
  return t;
}

std::vector<std::pair<std::string, Tensor>> NnModule::StateDict(const std::string& prefix) const {
  std::vector<std::pair<std::string, Tensor>> out;
  for (auto& p : params_) out.emplace_back(prefix + p.first, p.second);
  for (auto& b : buffers_) out.emplace_back(prefix + b.first, b.second);
  for (auto& c : children_) {
    auto sub = c.second->StateDict(prefix + c.first + ".");
    out.insert(out.end(), sub.begin(), sub.end());
  }
  return out;
}

std::vector<Tensor> NnModule::Parameters() const {
  std::vector<Tensor> out;
  for (auto& p : NamedParameters()) out.push_back(p.second);
  return out;
}

std::vector<std::pair<std::string, Tensor>> NnModule::NamedBuffers(const std::string& prefix) const {
  std::vector<std::pair<std::string, Tensor>> out;
  for (auto& b : buffers_) out.emplace_back(prefix + b.first, b.second);
  for (auto& c : children_) {
    auto sub = c.second->NamedBuffers(prefix + c.first + ".");
    out.insert(out.end(), sub.begin(), sub.end());
  }
  return out;
}

std::vector<std::pair<std::string, Tensor>> NnModule::NamedTrainableParameters() const {
  std::vector<std::pair<std::string, Tensor>> out;
  for (auto& p : NamedParameters())
    if (p.second.RequiresGrad()) out.push_back(p);
  return out;
}

std::vector<Tensor> NnModule::TrainableParameters() const {
  std::vector<Tensor> out;
  for (auto& p : NamedTrainableParameters()) out.push_back(p.second);
  return out;
}

int NnModule::SetTrainable(const std::function<bool(const std::string&, const Tensor&)>& predicate, bool trainable) {
  if (!predicate) throw std::invalid_argument("A predicate is required.");
  int changed = 0;
  for (auto& p : NamedParameters()) {
    if (predicate(p.first, p.second) && p.second.RequiresGrad() != trainable) {
      p.second.SetRequiresGrad(trainable);   // the handle shares the parameter's autograd state
      changed++;
    }
  }
  return changed;
}

int NnModule::SetTrainable(const std::string& nameOrPrefix, bool trainable) {
  if (nameOrPrefix.empty()) throw std::invalid_argument("A parameter name or module path is required.");
  const std::string prefix = nameOrPrefix + ".";
  bool found = false;
  int changed = SetTrainable([&](const std::string& n, const Tensor&) {
    bool hit = n == nameOrPrefix || n.compare(0, prefix.size(), prefix) == 0;
    found |= hit;
    return hit;
  }, trainable);
  if (!found) throw std::invalid_argument("No parameter is named '" + nameOrPrefix + "' or lies under a module of that path.");
  return changed;
}

int NnModule::Freeze() { return SetTrainable([](const std::string&, const Tensor&) { return true; }, false); }
int NnModule::Freeze(const std::string& nameOrPrefix) { return SetTrainable(nameOrPrefix, false); }
int NnModule::Freeze(const std::function<bool(const std::string&, const Tensor&)>& predicate) { return SetTrainable(predicate, false); }
int NnModule::Unfreeze() { return SetTrainable([](const std::string&, const Tensor&) { return true; }, true); }
int NnModule::Unfreeze(const std::string& nameOrPrefix) { return SetTrainable(nameOrPrefix, true); }
int NnModule::Unfreeze(const std::function<bool(const std::string&, const Tensor&)>& predicate) { return SetTrainable(predicate, true); }

bool NnModule::IsFrozen(const std::string& name) const {
  for (auto& p : NamedParameters())
    if (p.first == name) return !p.second.RequiresGrad();
  throw std::invalid_argument("No parameter named '" + name + "'.");
}

void NnModule::LoadStateDict(const std::vector<std::pair<std::string, Tensor>>& state) {
  std::vector<std::pair<std::string, Tensor>> mine = StateDict();
  auto find = [&](const std::string& n) -> const Tensor* {
    const Tensor* hit = nullptr;
    for (auto& e : state) {
      if (e.first != n) continue;
      if (hit) throw std::invalid_argument("State name '" + n + "' appears twice.");
      hit = &e.second;
    }
    return hit;
  };
  for (auto& e : state) find(e.first);   // duplicates anywhere in the given state are an error
  for (auto& m : mine) {
    const Tensor* src = find(m.first);
    if (!src) throw std::invalid_argument("State has no entry '" + m.first + "'.");
    if (src->GetDType() != m.second.GetDType() || !(src->GetShape() == m.second.GetShape()))
      throw std::invalid_argument("State entry '" + m.first + "' is " + src->GetShape().ToString() + ", the module has " +
                                  m.second.GetShape().ToString() + ".");
  }
  if (state.size() != mine.size())
    throw std::invalid_argument("State has " + std::to_string(state.size()) + " entries, the module has " + std::to_string(mine.size()) + ".");
  for (auto& m : mine) {
    Tensor src = find(m.first)->Contiguous();
    if (!m.second.IsContiguous()) throw TensorShapeException("Module state must be contiguous.");
    if (m.second.Length())
      Check(om_memcpy_d2d(Device::Current(), m.second.RawData(), src.RawData(), (size_t)m.second.Length() * SizeOf(m.second.GetDType())));
  }
}

void NnModule::ZeroGrad() {
  for (auto& p : NamedParameters()) Backprop::ZeroGrad(p.second);
}

void NnModule::Train(bool on) {
  Training = on;
  for (auto& c : children_) c.second->Train(on);
}

Linear::Linear(int inFeatures, int outFeatures, Generator& g, bool bias) {
  if (inFeatures < 1 || outFeatures < 1) throw ArgumentOutOfRangeException("Linear needs positive feature counts.");
  float bound = 1.0f / sqrtf((float)inFeatures);
  Weight = RegisterParameter("weight", InitUniform(g, bound, Shape{outFeatures, inFeatures}));
  if (bias) Bias = RegisterParameter("bias", InitUniform(g, bound, Shape{outFeatures}));
}

Linear::Linear(Tensor weight, Tensor bias) {
  if (weight.Rank() != 2) throw TensorShapeException("Linear weights are [out, in].");
  Weight = RegisterParameter("weight", weight);
  if (!bias.IsEmpty()) Bias = RegisterParameter("bias", bias);
}

LayerNorm::LayerNorm(int width, float eps) : Epsilon(eps) {
  Gamma = RegisterParameter("weight", InitConstant(1.f, Shape{width}));
  Beta = RegisterParameter("bias", InitConstant(0.f, Shape{width}));
}

// Embedding rows are uniform in [-1, 1) (Layers.cs:268-313).
Embedding::Embedding(int count, int width, Generator& g, int paddingIndex, bool sparse) : PaddingIndex(paddingIndex), IsSparse(sparse) {
  Weight = RegisterParameter("weight", InitUniform(g, 1.0f, Shape{count, width}));
}

Conv2d::Conv2d(int inCh, int outCh, int kernel, Generator& g, int stride, int padding, bool bias) {
  float bound = 1.0f / sqrtf((float)(inCh * kernel * kernel));
  Weight = RegisterParameter("weight", InitUniform(g, bound, Shape{outCh, inCh, kernel, kernel}));
  if (bias) Bias = RegisterParameter("bias", InitUniform(g, bound, Shape{outCh}));
  P.strideH = P.strideW = stride;
  P.padTop = P.padLeft = P.padBottom = P.padRight = padding;
}

BatchNorm2d::BatchNorm2d(int channels, float momentum, float eps) : Momentum(momentum), Epsilon(eps) {
  Gamma = RegisterParameter("weight", InitConstant(1.f, Shape{channels}));
  Beta = RegisterParameter("bias", InitConstant(0.f, Shape{channels}));
  RunningMean = RegisterBuffer("running_mean", InitConstant(0.f, Shape{channels}));
  RunningVar = RegisterBuffer("running_var", InitConstant(1.f, Shape{channels}));
}

MultiHeadAttention::MultiHeadAttention(int width, int heads, Generator& g) : Heads(heads) {
  if (heads < 1) throw ArgumentOutOfRangeException("heads must be at least 1.");
  if (width < 1 || width % heads != 0)
    throw std::invalid_argument("Width " + std::to_string(width) + " must be positive and divisible by the head count " + std::to_string(heads) + ".");
  // The three input projections live in one [3 * width, width] allocation (and one [3 * width] bias) so that they run
  // as a single product; q, k, v stay separate parameters (views), drawn in the reference's order: q.weight, q.bias,
  // k.weight, k.bias, v.weight, v.bias (Layers.cs:479-492).
  const float bound = 1.0f / sqrtf((float)width);
  std::vector<float> hw((size_t)3 * width * width), hb((size_t)3 * width);
  for (int i = 0; i < 3; i++) {
    for (size_t j = 0; j < (size_t)width * width; j++) hw[(size_t)i * width * width + j] = g.Uniform(-bound, bound);
    for (int j = 0; j < width; j++) hb[(size_t)i * width + j] = g.Uniform(-bound, bound);
  }
  Tensor pw = Tensor::FromHost(hw.data(), Shape{3 * width, width}), pb = Tensor::FromHost(hb.data(), Shape{3 * width});
  Linear** slots[3] = {&Q, &K, &V};
  const char* names[3] = {"q", "k", "v"};
  for (int i = 0; i < 3; i++)
    *slots[i] = RegisterModule(names[i], new Linear(pw.Slice(0, i * width, (i + 1) * width), pb.Slice(0, i * width, (i + 1) * width)));
  O = RegisterModule("o", new Linear(width, width, g));
}

Tensor MultiHeadAttention::Forward(const Tensor& input, const Tensor& mask) {
  if (input.Rank() != 3) throw TensorShapeException("MultiHeadAttention needs [batch, length, width], not " + input.GetShape().ToString() + ".");
  // The head split and merge (Reshape + Permute(0, 2, 1, 3) around Ops.Attention in the reference) are folded into the
  // attention kernels' addressing: q, k, v stay [batch, length, width] and so does the result.
  Tensor a;
  if (Ops::Adjacent({Q->Weight, K->Weight, V->Weight}) && Ops::Adjacent({Q->Bias, K->Bias, V->Bias}))
    // (the attention kernels of the bfloat16 tier read q | k | v as bfloat16 only: the projection then writes nothing else)
    a = Ops::AttentionPacked(Ops::LinearPacked(input, {Q->Weight, K->Weight, V->Weight}, {Q->Bias, K->Bias, V->Bias},
                                               Ops::AttentionPackedReadsBf16Only(input, Q->Weight.GetShape()[0], Heads)),
                             Heads, mask);
  else
    a = Ops::AttentionHeads(Q->Forward(input), K->Forward(input), V->Forward(input), Heads, mask);
  return O->Forward(a);
}

TransformerEncoderLayer::TransformerEncoderLayer(int width, int heads, int ff, Generator& g) {
  Attn = RegisterModule("attn", new MultiHeadAttention(width, heads, g));
  Norm1 = RegisterModule("norm1", new LayerNorm(width));
  Ff1 = RegisterModule("ff1", new Linear(width, ff, g));
  Ff2 = RegisterModule("ff2", new Linear(ff, width, g));
  Norm2 = RegisterModule("norm2", new LayerNorm(width));
}

Tensor TransformerEncoderLayer::Forward(const Tensor& input, const Tensor& mask) {
  Tensor a = Attn->Forward(input, mask);
  Tensor x1 = Ops::AddLayerNorm(input, a, Norm1->Gamma, Norm1->Beta, Norm1->Epsilon);
  Tensor f = Ops::FeedForward(x1, Ff1->Weight, Ff1->Bias, Ff2->Weight, Ff2->Bias);
  return Ops::AddLayerNorm(x1, f, Norm2->Gamma, Norm2->Beta, Norm2->Epsilon);
}

void Conv1d::Init(int inCh, int outCh, int kernel, Generator& g, bool bias) {
  if (kernel < 1 || P.groups < 1) throw ArgumentOutOfRangeException("Conv1d needs a positive kernel size and group count.");
  if (inCh < 1 || outCh < 1 || inCh % P.groups != 0 || outCh % P.groups != 0)
    throw std::invalid_argument("Channels must be positive and divisible by the groups.");
  float bound = 1.0f / sqrtf((float)(inCh / P.groups * kernel));
  Weight = RegisterParameter("weight", InitUniform(g, bound, Shape{outCh, inCh / P.groups, kernel}));
  if (bias) Bias = RegisterParameter("bias", InitUniform(g, bound, Shape{outCh}));
}

Conv1d::Conv1d(int inCh, int outCh, int kernel, Generator& g, int stride, int padding, int dilation, int groups, bool bias) {
  P.stride = stride;
  P.padLeft = P.padRight = padding;
  P.dilation = dilation;
  P.groups = groups;
  Init(inCh, outCh, kernel, g, bias);
}

// "same": the total dilation*(kernel-1) is split with the odd zero on the right; "valid": no padding (Ops.Nn.cs:12-26).
Conv1d::Conv1d(int inCh, int outCh, int kernel, Generator& g, const std::string& padding, int dilation, int groups, bool bias) {
  if (kernel < 1) throw ArgumentOutOfRangeException("Conv1d needs a positive kernel size.");
  P.stride = 1;
  P.dilation = dilation;
  P.groups = groups;
  if (padding == "same") {
    int total = (dilation > 1 ? dilation : 1) * (kernel - 1);
    P.padLeft = total / 2;
    P.padRight = total - total / 2;
  } else if (padding != "valid") {
    throw std::invalid_argument("Padding must be \"same\" or \"valid\", not \"" + padding + "\".");
  }
  Init(inCh, outCh, kernel, g, bias);
}

ConvTranspose2d::ConvTranspose2d(int inCh, int outCh, int kernel, Generator& g, int stride, int padding, int outputPadding, int dilation,
                                 int groups, bool bias) {
  if (kernel < 1 || groups < 1) throw ArgumentOutOfRangeException("ConvTranspose2d needs a positive kernel size and group count.");
  if (inCh < 1 || outCh < 1 || inCh % groups != 0 || outCh % groups != 0)
    throw std::invalid_argument("Channels must be positive and divisible by the groups.");
  P.strideH = P.strideW = stride;
  P.padH = P.padW = padding;
  P.outPadH = P.outPadW = outputPadding;
  P.dilH = P.dilW = dilation;
  P.groups = groups;
  float bound = 1.0f / sqrtf((float)(outCh / groups * kernel * kernel));
  Weight = RegisterParameter("weight", InitUniform(g, bound, Shape{inCh, outCh / groups, kernel, kernel}));
  if (bias) Bias = RegisterParameter("bias", InitUniform(g, bound, Shape{outCh}));
}

Dropout::Dropout(float p, uint64_t seed) : P(p), Seed(seed) {
  if (!(p >= 0.f && p < 1.f)) throw ArgumentOutOfRangeException("Dropout probability must be in [0, 1).");
  Counter = RegisterBuffer("draws", Tensor::Zeros(DType::I64, Shape{1}));
}

int64_t Dropout::Draws() const {
  int64_t v = 0;
  Counter.CopyToHost(&v);
  return v;
}

// ---- losses (Losses.cs:14-129) ------------------------------------------------------------------------------------------
Tensor Losses::CrossEntropy(const Tensor& logits, const Tensor& targets, float labelSmoothing, int ignoreIndex, bool mean) {
  if (!(labelSmoothing >= 0.f && labelSmoothing <= 1.f)) throw ArgumentOutOfRangeException("Label smoothing must be in [0, 1].");
  if (labelSmoothing == 0.f) return Ops::CrossEntropy(logits, targets, mean, ignoreIndex);
  if (logits.Rank() != 2) throw TensorShapeException("CrossEntropy needs [rows, classes] logits, not " + logits.GetShape().ToString() + ".");
  Tensor logp = Ops::LogSoftmax(logits);
  Tensor nll = Ops::NllLoss(logp, targets, mean, ignoreIndex);
  // The smoothing term, per row -mean_c(logp), over the counted rows. The mask of counted rows is formed on the device.
  int rows = logits.GetShape()[0];
  Tensor tc = targets.Contiguous();
  Tensor mask = Tensor::Create(DType::F32, Shape{rows});
  Check(om_target_mask(Device::Current(), tc.RawData(), (int32_t)tc.GetDType(), rows, ignoreIndex, mask.Data()));
  Tensor perRow = Ops::Neg(Ops::Mean(logp, 1));
  Tensor smooth = Ops::Sum(Ops::Mul(perRow, mask));
  if (mean) {
    // 1 / counted as a float (0 rows: 1/0 = inf, and 0 * inf = NaN like the reference's NaN factor), then one product.
    Tensor one = Tensor::Create(DType::F32, Shape{});
    one.Fill(1.f);
    smooth = Ops::Mul(smooth, Ops::Div(one, Ops::Sum(mask)));
  }
  Tensor keep = Tensor::Create(DType::F32, Shape{}), share = Tensor::Create(DType::F32, Shape{});
  keep.Fill(1.f - labelSmoothing);
  share.Fill(labelSmoothing);
  return Ops::Add(Ops::Mul(nll, keep), Ops::Mul(smooth, share));
}

Tensor Losses::Mse(const Tensor& prediction, const Tensor& target, bool mean) {
  Tensor d = Ops::Sub(prediction, target);
  Tensor sq = Ops::Mul(d, d);
  return mean ? Ops::Mean(sq) : Ops::Sum(sq);
}

Tensor Losses::L1(const Tensor& prediction, const Tensor& target, bool mean) {
  Tensor d = Ops::Sub(prediction, target);
  Tensor magnitude = Ops::Add(Ops::Relu(d), Ops::Relu(Ops::Neg(d)));
  return mean ? Ops::Mean(magnitude) : Ops::Sum(magnitude);
}

Tensor Losses::BceWithLogits(const Tensor& logits, const Tensor& targets, bool mean) {
  if (!(logits.GetShape() == targets.GetShape()))
    throw TensorShapeException("BceWithLogits needs equal shapes, not " + logits.GetShape().ToString() + " and " + targets.GetShape().ToString() + ".");
  int count = (int)logits.Length();
  Tensor x = logits.Reshape(Shape{count, 1});
  Tensor zeros = Tensor::Zeros(DType::F32, Shape{count, 1});
  Tensor logSoftmax = Ops::LogSoftmax(Ops::Concat({x, zeros}, 1));
  Tensor softplus = Ops::Neg(logSoftmax.Select(1, 1));
  Tensor xt = Ops::Mul(logits.Reshape(Shape{count}), targets.Reshape(Shape{count}));
  Tensor perElement = Ops::Sub(softplus, xt);
  return mean ? Ops::Mean(perElement) : Ops::Sum(perElement);
}

}  // namespace omh
