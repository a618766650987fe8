// Training-step drivers for the benchmark configurations, written against the host mirror exactly as a user of the
// reference writes a loop (tests/GuideSamples/TrainingGuide.cs:48-67 of the reference):
//   scope; loss = model.Forward(x); opt.ZeroGrad(); loss.Backward(); opt.Step();
// plus what the reference does not have: whole-step CUDA graph replay and data-parallel gradient buckets.
#include <math.h>
#include <string.h>

#include <map>

#include "omh.hpp"

using namespace omh;

#define OMH_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string t_error;

template <class F>
int32_t Guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const TensorShapeException& e) {
    t_error = e.what();
    return 1;
  } catch (const ArgumentOutOfRangeException& e) {
    t_error = e.what();
    return 2;
  } catch (const BackendException& e) {
    t_error = e.what();
    return 100 + e.status;
  } catch (const std::exception& e) {
    t_error = e.what();
    return 10;
  }
}

// ---- models ----------------------------------------------------------------------------------------------------------

// Config 1: 784 -> 512 -> ReLU -> 512 -> ReLU -> 10, softmax cross-entropy.
struct Mlp : NnModule {
  std::vector<Linear*> layers;
  Mlp(const std::vector<int>& widths, Generator& g) {
    for (size_t i = 0; i + 1 < widths.size(); i++)
      layers.push_back(RegisterModule(std::to_string(2 * i), new Linear(widths[i], widths[i + 1], g)));
  }
  Tensor Forward(const Tensor& x) override {
    Tensor h = x;
    for (size_t i = 0; i < layers.size(); i++) {
      h = layers[i]->Forward(h);
      if (i + 1 < layers.size()) h = Ops::Relu(h);
    }
    return h;
  }
};

// Configs 3 and 5: token + learned position embeddings, N post-norm encoder layers, masked-LM head on gathered rows.
struct MlmEncoder : NnModule {
  Embedding *Tok, *Pos;
  std::vector<TransformerEncoderLayer*> layers;
  Linear* Head;
  int Width;
  MlmEncoder(int nLayers, int width, int heads, int ff, int vocab, int seq, Generator& g) : Width(width) {
    Tok = RegisterModule("tok", new Embedding(vocab, width, g));
    Pos = RegisterModule("pos", new Embedding(seq, width, g));
    for (int i = 0; i < nLayers; i++)
      layers.push_back(RegisterModule("layers." + std::to_string(i), new TransformerEncoderLayer(width, heads, ff, g)));
    Head = RegisterModule("head", new Linear(width, vocab, g));
  }
  Tensor Forward(const Tensor&) override { throw InvalidOperationException("use Logits(ids, positions, rows)"); }
  // ids [B,S]; positions [S] = 0..S-1; rows [R] = flat indices of the masked positions. Returns logits [R, vocab].
  Tensor Logits(const Tensor& ids, const Tensor& positions, const Tensor& rows) {
    Tensor x = Ops::Add(Tok->Forward(ids), Pos->Forward(positions));
    for (auto* l : layers) x = l->Forward(x);
    int b = ids.GetShape()[0], s = ids.GetShape()[1];
    Tensor hidden = x.Reshape(Shape{b * s, Width});
    // Row gather on an activation, the idiom of Ops.Recurrent.cs:362 in the reference.
    Tensor picked = Ops::Embedding(hidden, rows);
    return Head->Forward(picked);
  }
};

// 12-uniform Irwin-Hall normal on the generator's stream (the reference's SampleRng.NextNormal, Data/SampleRng.cs:83-88).
static float NextNormal(Generator& g) {
  float acc = 0.f;
  for (int i = 0; i < 12; i++) acc += g.NextSingle();
  return acc - 6.0f;
}
// He-normal weights, N(0, 2 / fanIn); the reference has no normal initialiser, the CNN configuration asks for one.
static void HeNormal(Tensor& w, int fanIn, Generator& g) {
  std::vector<float> h((size_t)w.Length());
  float scale = sqrtf(2.0f / (float)fanIn);
  for (float& v : h) v = NextNormal(g) * scale;
  w.CopyFromHost(h.data());
}
static void ZeroFill(Tensor& t) {
  std::vector<float> h((size_t)t.Length(), 0.f);
  t.CopyFromHost(h.data());
}

// Config 2: [Conv 3x3 pad 1 (bias) + BatchNorm + ReLU] x n with per-conv stride, global average pool, Linear.
struct SmallCnn : NnModule {
  std::vector<Conv2d*> convs;
  std::vector<BatchNorm2d*> norms;
  Linear* Fc;
  SmallCnn(int inCh, const std::vector<int>& channels, const std::vector<int>& strides, int classes, Generator& g) {
    int c = inCh;
    for (size_t i = 0; i < channels.size(); i++) {
      convs.push_back(RegisterModule("conv" + std::to_string(i), new Conv2d(c, channels[i], 3, g, strides[i], 1, true)));
      norms.push_back(RegisterModule("bn" + std::to_string(i), new BatchNorm2d(channels[i])));
      HeNormal(convs.back()->Weight, c * 9, g);
      ZeroFill(convs.back()->Bias);
      c = channels[i];
    }
    Fc = RegisterModule("fc", new Linear(c, classes, g));
    HeNormal(Fc->Weight, c, g);
    ZeroFill(Fc->Bias);
  }
  Tensor Forward(const Tensor& x) override {
    Tensor h = x;
    for (size_t i = 0; i < convs.size(); i++) h = Ops::Relu(norms[i]->Forward(convs[i]->Forward(h)));
    Tensor pooled = Ops::GlobalAvgPool2d(h);
    return Fc->Forward(pooled.Reshape(Shape{pooled.GetShape()[0], pooled.GetShape()[1]}));
  }
};

// Config 4: four Conv 3x3 + ReLU + MaxPool stages that reduce the height to 1, a 2-layer bidirectional LSTM over the
// width axis, Linear to the classes, log-softmax. Returns log-probabilities [T, B, classes].
struct Crnn : NnModule {
  Conv2d* Convs[4];
  Recurrent* Rnn;
  Linear* Fc;
  Crnn(const int channels[4], int hidden, int classes, Generator& g) {
    int c = 1;
    for (int i = 0; i < 4; i++) {
      Convs[i] = RegisterModule("conv" + std::to_string(i), new Conv2d(c, channels[i], 3, g, 1, 1, true));
      c = channels[i];
    }
    Rnn = RegisterModule("lstm", new Recurrent(c, hidden, 2, true, g));
    Fc = RegisterModule("fc", new Linear(2 * hidden, classes, g));
  }
  Tensor Forward(const Tensor& x) override {
    static const int pool[4][2] = {{2, 2}, {2, 2}, {2, 1}, {4, 1}};
    Tensor h = x;
    for (int i = 0; i < 4; i++) h = Ops::MaxPool2d(Ops::Relu(Convs[i]->Forward(h)), pool[i][0], pool[i][1], pool[i][0], pool[i][1]);
    if (h.GetShape()[2] != 1) throw TensorShapeException("The CRNN needs an input height of 32, got a feature map " + h.GetShape().ToString() + ".");
    int b = h.GetShape()[0], c = h.GetShape()[1], t = h.GetShape()[3];
    Tensor seq = h.Reshape(Shape{b, c, t}).Permute({2, 0, 1});   // [T, B, C]
    Tensor y = Rnn->Forward(seq);
    return Ops::LogSoftmax(Fc->Forward(y), -1);
  }
};

}  // namespace

struct omh_trainer {
  int kind = 0;
  std::vector<int64_t> cfg;
  std::unique_ptr<NnModule> model;
  std::unique_ptr<Optimizer> opt;
  std::vector<std::pair<std::string, Tensor>> params;
  // persistent device inputs
  std::vector<Tensor> inputs;
  Tensor positions;
  Tensor input_lengths;   // CRNN: every sequence spans all frames
  Tensor loss_out;     // device scalar that survives the step
  Tensor flat_grads;   // all gradients, contiguous, in reverse registration order
  float ce_denominator = 0.f;
  Tensor dp_loss_scale;   // scalar 1 / world for losses that are means over the local batch (CTC)
  float clip_norm = 0.f;
  // graph replay
  void* graph = nullptr;
  Tensor hyper_dev;
  std::vector<uint8_t> hyper_host;
  int64_t steps_done = 0;
  // data parallel
  int world = 1, rank = 0;
  int dp_timeout_ms = 0;   // host deadline for the gradient exchange of a step (0: the step is not waited for)
  struct BucketInfo { int64_t begin, end; int pending; int total; };
  std::vector<BucketInfo> buckets;
  std::map<AutogradMeta*, int> bucket_of;
  std::vector<std::vector<int>> bucket_params;   // positions in the optimizer's parameter list, per bucket
  int loss_bucket = -1;                          // the loss scalar rides on the communication stream as a bucket of one
  // Batches staged ahead of their step (DataLoader's prefetch ring on the device): per slot the inputs on the device and a
  // pinned host copy the asynchronous transfer reads from, so the caller's memory is free again when prefetch returns.
  int stage_depth = 0;
  std::vector<std::vector<Tensor>> stage_dev;
  std::vector<std::vector<void*>> stage_host;
  int64_t staged = 0, taken = 0;                 // batches put into / taken out of the ring
};

static void BuildFlatGrads(omh_trainer* t) {
  int64_t total = 0;
  for (auto& p : t->params) total += p.second.Length() + 63;   // room for the alignment of each gradient
  t->flat_grads = Tensor::Zeros(DType::F32, Shape{(int)std::min<int64_t>(total, INT32_MAX)});
  if (total > INT32_MAX) throw TensorShapeException("more than 2^31-1 parameters");
  // Reverse registration order: the gradients that become final first (last layers) sit at the front, so the first
  // buckets complete early in the backward sweep.
  int64_t off = 0;
  const int64_t bucket_elems = 6 * 1024 * 1024;  // ~25 MB of fp32
  int64_t bucket_begin = 0;
  // Parameters that are adjacent views of one allocation (the packed q, k, v projections) get gradients that are adjacent in the same
  // order, so that their weight gradient can be written by one product.
  const int np = (int)t->params.size();
  std::vector<bool> placed(np, false);
  auto place = [&](int i, bool group_start) {
    Tensor& p = t->params[i].second;
    // Every gradient (every group of adjacent ones) starts on a 256-byte boundary: the product kernels write weight
    // gradients through TMA, which wants 16-byte aligned rows. The padding words stay zero and ride along in the buckets.
    if (group_start) off = (off + 63) & ~(int64_t)63;
    auto meta = p.Autograd();
    Tensor view = t->flat_grads.View(p.GetShape(), ContiguousStrides(p.GetShape()), off);
    meta->Grad = view;
    meta->GradIsZero = true;
    int64_t len = p.Length();
    if (off + len - bucket_begin > bucket_elems && off > bucket_begin) {
      t->buckets.push_back({bucket_begin, off, 0, 0});
      bucket_begin = off;
    }
    t->bucket_of[meta.get()] = (int)t->buckets.size();
    off += len;
    placed[i] = true;
  };
  auto before = [&](int i) {   // the parameter whose storage ends where parameter i starts, or -1
    for (int j = 0; j < np; j++)
      if (j != i && !placed[j] && t->params[j].second.Storage() == t->params[i].second.Storage() &&
          t->params[j].second.Data() + t->params[j].second.Length() == t->params[i].second.Data()) return j;
    return -1;
  };
  auto after = [&](int i) {
    for (int j = 0; j < np; j++)
      if (j != i && !placed[j] && t->params[j].second.Storage() == t->params[i].second.Storage() &&
          t->params[i].second.Data() + t->params[i].second.Length() == t->params[j].second.Data()) return j;
    return -1;
  };
  for (int i = np - 1; i >= 0; i--) {
    if (placed[i]) continue;
    int first = i;
    for (int guard = 0, j; guard < np && (j = before(first)) >= 0; guard++) first = j;
    for (int cur = first; cur >= 0;) {
      int nxt = after(cur);
      place(cur, cur == first);
      cur = nxt;
    }
  }
  t->buckets.push_back({bucket_begin, off, 0, 0});
  for (auto& kv : t->bucket_of) t->buckets[kv.second].total++;
}

static Tensor Forward(omh_trainer* t) {
  if (t->kind == 1) {
    Tensor logits = t->model->Forward(t->inputs[0]);
    return Ops::CrossEntropy(logits, t->inputs[1], true, -100, t->ce_denominator);
  }
  if (t->kind == 2) {
    Tensor logits = t->model->Forward(t->inputs[0]);
    return Ops::CrossEntropy(logits, t->inputs[1], true, -100, t->ce_denominator);
  }
  if (t->kind == 4) {
    Tensor lp = t->model->Forward(t->inputs[0]);
    Tensor loss = Ops::CtcLoss(lp, t->inputs[1], t->input_lengths, t->inputs[2], 0, 1, true);
    // The CTC mean is a mean over sequences of (loss / target length): with equal shards the global mean is the mean of
    // the shard means, so each shard contributes its mean divided by the world size and the sum over ranks (of the loss
    // and of every gradient) is the single-process value.
    if (t->world > 1) loss = Ops::Mul(loss, t->dp_loss_scale);
    return loss;
  }
  auto* m = static_cast<MlmEncoder*>(t->model.get());
  Tensor logits = m->Logits(t->inputs[0], t->positions, t->inputs[1]);
  return Ops::CrossEntropy(logits, t->inputs[2], true, -100, t->ce_denominator);
}

// One training step on the device inputs; leaves the loss in t->loss_out.
static void StepBody(omh_trainer* t) {
  om_ctx* ctx = Device::Current();
  ActivationScope scope;
  Tensor loss = Forward(t);
  Check(om_memcpy_d2d(ctx, t->loss_out.RawData(), loss.RawData(), 4));
  if (t->world > 1) Check(om_dp_allreduce_bucket(ctx, t->loss_bucket));   // summed beside the backward pass
  t->opt->ZeroGrad();
  if (t->world > 1) {
    for (auto& b : t->buckets) b.pending = b.total;
    Backprop::GradReadyHook = [t, ctx](AutogradMeta* leaf) {
      auto it = t->bucket_of.find(leaf);
      if (it == t->bucket_of.end()) return;
      auto& b = t->buckets[it->second];
      if (--b.pending == 0) Check(om_dp_allreduce_bucket(ctx, it->second));
    };
  }
  loss.Backward();
  if (t->world > 1) {
    Backprop::GradReadyHook = nullptr;
    // Buckets whose parameters got no gradient this step are still exchanged so that all ranks agree.
    for (size_t i = 0; i < t->buckets.size(); i++)
      if (t->buckets[i].pending > 0) Check(om_dp_allreduce_bucket(ctx, (int32_t)i));
    if (t->clip_norm <= 0.f) {
      // No global norm to wait for: each bucket's parameters are updated as soon as that bucket's sum has arrived, while
      // the later buckets (the embedding table comes last) are still on the wire.
      t->opt->StepGroups(t->bucket_params, [&](int b) { Check(om_dp_wait_bucket(ctx, b)); });
      Check(om_dp_wait(ctx, t->dp_timeout_ms));
      return;
    }
    Check(om_dp_wait(ctx, t->dp_timeout_ms));
  }
  if (t->clip_norm > 0.f) GradClip::ClipNormAsync(t->opt->Parameters(), t->clip_norm, false, nullptr);
  t->opt->Step();
}

OMH_API int32_t omh_trainer_last_error(char* buf, size_t n) {
  size_t len = std::min(n - 1, t_error.size());
  memcpy(buf, t_error.data(), len);
  buf[len] = 0;
  return 0;
}

// kind 1 (MLP, AdamW): cfg = [batch, in, h1, h2, out]. kind 2 (CNN, SGD momentum 0.9) and kind 4 (CRNN + CTC, Adam): see
// below. kind 3 (masked-LM encoder, AdamW): cfg = [batch, seq, layers, width, heads,
// ff, vocab, masked_rows]. hyper = [lr, weight_decay, clip_norm (0 = off)].
OMH_API int32_t omh_trainer_create(int32_t kind, const int64_t* cfg, int32_t ncfg, uint64_t seed, const double* hyper,
                                   omh_trainer** out) {
  return Guard([&] {
    auto t = std::make_unique<omh_trainer>();
    t->kind = kind;
    t->cfg.assign(cfg, cfg + ncfg);
    Generator g(seed);
    if (kind == 1) {
      if (ncfg < 3) throw TensorShapeException("MLP config needs [batch, widths...]");
      std::vector<int> widths;
      for (int i = 1; i < ncfg; i++) widths.push_back((int)cfg[i]);
      t->model.reset(new Mlp(widths, g));
      t->inputs.push_back(Tensor::Zeros(DType::F32, Shape{(int)cfg[0], widths[0]}));
      t->inputs.push_back(Tensor::Zeros(DType::I64, Shape{(int)cfg[0]}));
    } else if (kind == 3) {
      if (ncfg != 8) throw TensorShapeException("encoder config needs 8 integers");
      int batch = (int)cfg[0], seq = (int)cfg[1], rows = (int)cfg[7];
      t->model.reset(new MlmEncoder((int)cfg[2], (int)cfg[3], (int)cfg[4], (int)cfg[5], (int)cfg[6], seq, g));
      t->inputs.push_back(Tensor::Zeros(DType::I32, Shape{batch, seq}));
      t->inputs.push_back(Tensor::Zeros(DType::I32, Shape{rows}));
      t->inputs.push_back(Tensor::Zeros(DType::I64, Shape{rows}));
      std::vector<int32_t> pos(seq);
      for (int i = 0; i < seq; i++) pos[i] = i;
      t->positions = Tensor::FromHostInt32(pos.data(), Shape{seq});
    } else if (kind == 2) {
      // [batch, in_channels, height, width, classes, n, channels x n, strides x n]
      if (ncfg < 6 || ncfg != 6 + 2 * cfg[5]) throw TensorShapeException("CNN config needs [batch, in_ch, h, w, classes, n, channels..., strides...]");
      int n = (int)cfg[5];
      std::vector<int> ch, st;
      for (int i = 0; i < n; i++) ch.push_back((int)cfg[6 + i]);
      for (int i = 0; i < n; i++) st.push_back((int)cfg[6 + n + i]);
      t->model.reset(new SmallCnn((int)cfg[1], ch, st, (int)cfg[4], g));
      t->inputs.push_back(Tensor::Zeros(DType::F32, Shape{(int)cfg[0], (int)cfg[1], (int)cfg[2], (int)cfg[3]}));
      t->inputs.push_back(Tensor::Zeros(DType::I64, Shape{(int)cfg[0]}));
    } else if (kind == 4) {
      // [batch, height, width, classes, hidden, max_label, c1, c2, c3, c4]
      if (ncfg != 10) throw TensorShapeException("CRNN config needs 10 integers");
      int batch = (int)cfg[0], frames = (int)cfg[2] / 4;
      const int ch[4] = {(int)cfg[6], (int)cfg[7], (int)cfg[8], (int)cfg[9]};
      t->model.reset(new Crnn(ch, (int)cfg[4], (int)cfg[3], g));
      t->inputs.push_back(Tensor::Zeros(DType::F32, Shape{batch, 1, (int)cfg[1], (int)cfg[2]}));
      t->inputs.push_back(Tensor::Zeros(DType::I32, Shape{batch * (int)cfg[5]}));   // labels, concatenated
      t->inputs.push_back(Tensor::Zeros(DType::I32, Shape{batch}));                 // label lengths
      std::vector<int32_t> il(batch, frames);
      t->input_lengths = Tensor::FromHostInt32(il.data(), Shape{batch});
    } else {
      throw InvalidOperationException("unknown trainer kind");
    }
    t->params = t->model->NamedParameters();
    std::vector<Tensor> ps;
    for (auto& p : t->params) ps.push_back(p.second);
    if (kind == 2) t->opt.reset(new Sgd(ps, (float)hyper[0], 0.9f, 0.f, (float)hyper[1], false));
    else if (kind == 4) t->opt.reset(new Adam(ps, (float)hyper[0], 0.9f, 0.999f, 1e-8f, (float)hyper[1]));
    else t->opt.reset(new AdamW(ps, (float)hyper[0], 0.9f, 0.999f, 1e-8f, (float)hyper[1]));
    t->clip_norm = (float)hyper[2];
    t->loss_out = Tensor::Zeros(DType::F32, Shape{});
    t->hyper_host.assign(t->opt->HyperBytes(), 0);
    t->hyper_dev = Tensor::Zeros(DType::F32, Shape{(int)(t->opt->HyperBytes() + 3) / 4});
    BuildFlatGrads(t.get());
    *out = t.release();
  });
}

OMH_API int32_t omh_trainer_free(omh_trainer* t) {
  if (t && t->graph) om_graph_destroy(Device::Current(), t->graph);
  if (t) {
    om_ctx* ctx = Device::Current();
    om_sync(ctx);
    for (auto& slot : t->stage_host)
      for (void* h : slot) om_host_free_pinned(ctx, h);
  }
  delete t;
  return 0;
}

OMH_API int32_t omh_trainer_param_count(omh_trainer* t) { return (int32_t)t->params.size(); }

OMH_API int32_t omh_trainer_param_info(omh_trainer* t, int32_t i, char* name, size_t n, int32_t* rank, int32_t* shape) {
  if (i < 0 || i >= (int)t->params.size()) return 1;
  strncpy(name, t->params[i].first.c_str(), n - 1);
  name[n - 1] = 0;
  *rank = t->params[i].second.Rank();
  for (int k = 0; k < *rank; k++) shape[k] = t->params[i].second.GetShape()[k];
  return 0;
}

OMH_API int32_t omh_trainer_get_param(omh_trainer* t, int32_t i, float* dst) {
  return Guard([&] { t->params[i].second.CopyToHost(dst); });
}
OMH_API int32_t omh_trainer_set_param(omh_trainer* t, int32_t i, const float* src) {
  return Guard([&] { t->params[i].second.CopyFromHost(src); });
}
OMH_API int32_t omh_trainer_get_grad(omh_trainer* t, int32_t i, float* dst) {
  return Guard([&] {
    Tensor g = t->params[i].second.Grad();
    if (g.IsEmpty()) throw InvalidOperationException("no gradient yet");
    g.CopyToHost(dst);
  });
}

OMH_API int32_t omh_trainer_input_count(omh_trainer* t) { return (int32_t)t->inputs.size(); }
OMH_API int64_t omh_trainer_input_bytes(omh_trainer* t, int32_t i) {
  return t->inputs[i].Length() * (int64_t)SizeOf(t->inputs[i].GetDType());
}

// Joins a data-parallel group; the cross-entropy then divides by `global_rows` (the counted rows of all ranks) so that
// the summed gradients are the gradient of the global mean.
OMH_API int32_t omh_trainer_dp_init(omh_trainer* t, const uint8_t* id128, int32_t rank, int32_t world, int64_t global_rows) {
  return Guard([&] {
    om_ctx* ctx = Device::Current();
    Check(om_dp_init(ctx, id128, rank, world));
    t->world = world;
    t->rank = rank;
    t->ce_denominator = (float)global_rows;
    const float inv_world = 1.0f / (float)world;
    t->dp_loss_scale = Tensor::FromHost(&inv_world, Shape{});
    for (size_t i = 0; i < t->buckets.size(); i++)
      Check(om_dp_register_bucket(ctx, (int32_t)i, t->flat_grads.Data() + t->buckets[i].begin, t->buckets[i].end - t->buckets[i].begin));
    t->loss_bucket = (int)t->buckets.size();
    Check(om_dp_register_bucket(ctx, t->loss_bucket, t->loss_out.Data(), 1));
    t->bucket_params.assign(t->buckets.size(), {});
    for (size_t i = 0; i < t->params.size(); i++) {
      auto it = t->bucket_of.find(t->params[i].second.Autograd().get());
      if (it != t->bucket_of.end()) t->bucket_params[(size_t)it->second].push_back((int)i);
    }
  });
}

// Sets the host deadline under which every later step waits for its gradient exchange (0 switches the wait off: the
// step is then only enqueued, and a peer that stopped shows at the next synchronisation).
OMH_API int32_t omh_trainer_set_dp_timeout_ms(omh_trainer* t, int32_t ms) {
  return Guard([&] {
    if (ms < 0) throw ArgumentOutOfRangeException("The deadline must not be negative.");
    t->dp_timeout_ms = ms;
  });
}

static void CopyInputs(omh_trainer* t, const void* const* inputs_host) {
  om_ctx* ctx = Device::Current();
  for (size_t i = 0; i < t->inputs.size(); i++) {
    Check(om_memcpy_h2d(ctx, t->inputs[i].RawData(), inputs_host[i], (size_t)omh_trainer_input_bytes(t, (int32_t)i)));
    t->inputs[i].MarkModified();   // a new batch: a bfloat16 copy of the old one is stale
  }
}

static void RunStep(omh_trainer* t) {
  om_ctx* ctx = Device::Current();
  if (t->graph) {
    // Per-step scalars of the optimizer for this step, written where the captured kernels read them.
    t->opt->FillHyper(t->hyper_host.data(), t->steps_done + 1);
    Check(om_memcpy_h2d(ctx, t->hyper_dev.RawData(), t->hyper_host.data(), t->hyper_host.size()));
    Check(om_graph_launch(ctx, t->graph));
    // A replayed step contains its collectives; with a deadline set, the host waits for the step under that deadline and
    // looks at the communicator, so that a peer that stopped shows as an error here and not as an endless wait later.
    if (t->world > 1 && t->dp_timeout_ms > 0) Check(om_dp_wait(ctx, t->dp_timeout_ms));
    t->opt->StepCount = t->steps_done + 1;
  } else {
    StepBody(t);
  }
  t->steps_done++;
}

// The call a user makes: host batch in, loss out. inputs_host[i] should be pinned for an asynchronous copy.
OMH_API int32_t omh_trainer_step(omh_trainer* t, const void* const* inputs_host, float* loss) {
  return Guard([&] {
    CopyInputs(t, inputs_host);
    RunStep(t);
    if (loss) Check(om_memcpy_d2h(Device::Current(), loss, t->loss_out.RawData(), 4));
  });
}

// ---- batches staged ahead of their step ----------------------------------------------------------------------------------
// omh_trainer_prefetch(batch) puts the next batch into the ring: a copy into the slot's pinned buffer (the caller's memory
// is free when the call returns) and an asynchronous transfer on the copy stream, which runs under the steps already
// queued. omh_trainer_step_prefetched() runs a step on the oldest staged batch: the compute stream waits for that slot's
// transfer (the host does not), takes the batch with device-to-device copies into the inputs the step (and its captured
// graph) reads, and frees the slot. Batches are consumed in the order they were staged (docs/data-loading.md section 1 of
// the reference: a batch waits in slot `step mod Prefetch` until the consumer reaches it).
OMH_API int32_t omh_trainer_prefetch_depth(omh_trainer* t, int32_t depth) {
  return Guard([&] {
    if (depth < 1 || depth > 16) throw ArgumentOutOfRangeException("The prefetch depth must be between 1 and 16.");
    if (t->stage_depth != 0) throw InvalidOperationException("The prefetch depth is already set.");
    om_ctx* ctx = Device::Current();
    t->stage_depth = depth;
    t->stage_dev.resize(depth);
    t->stage_host.resize(depth);
    for (int s = 0; s < depth; s++)
      for (size_t i = 0; i < t->inputs.size(); i++) {
        t->stage_dev[s].push_back(Tensor::Zeros(t->inputs[i].GetDType(), t->inputs[i].GetShape()));
        void* h = nullptr;
        Check(om_host_alloc_pinned(ctx, (size_t)omh_trainer_input_bytes(t, (int32_t)i), &h));
        t->stage_host[s].push_back(h);
      }
  });
}

OMH_API int32_t omh_trainer_prefetch(omh_trainer* t, const void* const* inputs_host) {
  return Guard([&] {
    if (t->stage_depth == 0) throw InvalidOperationException("Set the prefetch depth first.");
    if (t->staged - t->taken >= t->stage_depth) throw InvalidOperationException("The prefetch ring is full: take a step first.");
    om_ctx* ctx = Device::Current();
    const int slot = (int)(t->staged % t->stage_depth);
    // The pinned buffer of this slot was last read by the transfer of the batch staged stage_depth batches ago, whose step
    // has been queued since; the transfer itself has long run by the time its step was taken, except when the caller
    // stages faster than the device steps: then wait for that step's take (a host wait on purpose: back-pressure).
    if (t->staged >= t->stage_depth) Check(om_stage_wait_taken(ctx, slot));
    for (size_t i = 0; i < t->inputs.size(); i++) {
      const size_t bytes = (size_t)omh_trainer_input_bytes(t, (int32_t)i);
      memcpy(t->stage_host[slot][i], inputs_host[i], bytes);
      Check(om_stage_h2d(ctx, slot, t->stage_dev[slot][i].RawData(), t->stage_host[slot][i], bytes));
    }
    Check(om_stage_commit(ctx, slot));
    t->staged++;
  });
}

OMH_API int32_t omh_trainer_step_prefetched(omh_trainer* t, float* loss) {
  return Guard([&] {
    if (t->taken >= t->staged) throw InvalidOperationException("No batch is staged.");
    om_ctx* ctx = Device::Current();
    const int slot = (int)(t->taken % t->stage_depth);
    Check(om_stage_acquire(ctx, slot));
    for (size_t i = 0; i < t->inputs.size(); i++) {
      Check(om_memcpy_d2d(ctx, t->inputs[i].RawData(), t->stage_dev[slot][i].RawData(), (size_t)omh_trainer_input_bytes(t, (int32_t)i)));
      t->inputs[i].MarkModified();
    }
    Check(om_stage_release(ctx, slot));
    t->taken++;
    RunStep(t);
    if (loss) Check(om_memcpy_d2h(ctx, loss, t->loss_out.RawData(), 4));
  });
}

// Copies a batch to the device without stepping, and steps on the resident batch without copies or read-back.
OMH_API int32_t omh_trainer_load_inputs(omh_trainer* t, const void* const* inputs_host) {
  return Guard([&] {
    CopyInputs(t, inputs_host);
    Check(om_sync(Device::Current()));
  });
}
OMH_API int32_t omh_trainer_step_resident(omh_trainer* t) {
  return Guard([&] { RunStep(t); });
}
OMH_API int32_t omh_trainer_read_loss(omh_trainer* t, float* loss) {
  return Guard([&] { Check(om_memcpy_d2h(Device::Current(), loss, t->loss_out.RawData(), 4)); });
}
OMH_API int32_t omh_trainer_sync(omh_trainer*) {
  return Guard([&] { Check(om_sync(Device::Current())); });
}

// Captures one step into a CUDA graph; later steps replay it. At least one eager step must have run so that the memory
// pool already holds every block the step needs.
OMH_API int32_t omh_trainer_enable_graph(omh_trainer* t) {
  return Guard([&] {
    if (t->graph) return;
    if (t->steps_done < 1) throw InvalidOperationException("run at least one eager step before capturing");
    om_ctx* ctx = Device::Current();
    t->opt->HyperDevice = t->hyper_dev.RawData();
    Check(om_sync(ctx));
    int64_t saved_count = t->opt->StepCount;
    // The batch changes between replays without the host code of the step running again: whatever the step derives from
    // the inputs (a bfloat16 copy) must be derived inside the captured step, so it is made stale before the capture.
    for (auto& in : t->inputs) in.MarkModified();
    Check(om_graph_begin(ctx));
    int32_t st = 0;
    try {
      StepBody(t);
    } catch (...) {
      void* g = nullptr;
      om_graph_end(ctx, &g);
      if (g) om_graph_destroy(ctx, g);
      t->opt->HyperDevice = nullptr;
      throw;
    }
    (void)st;
    Check(om_graph_end(ctx, &t->graph));
    t->opt->StepCount = saved_count;  // capturing executed nothing
  });
}

OMH_API int64_t omh_trainer_steps_done(omh_trainer* t) { return t->steps_done; }

// ---- what a checkpoint reads and writes (Checkpoint.cs of the reference; the file format lives in checkpoint.py) -------
OMH_API int32_t omh_trainer_model_state_count(omh_trainer* t) { return (int32_t)t->model->StateDict().size(); }
OMH_API int32_t omh_trainer_model_state_info(omh_trainer* t, int32_t i, char* name, size_t n, int32_t* dtype, int32_t* rank, int32_t* shape) {
  auto st = t->model->StateDict();
  if (i < 0 || i >= (int)st.size()) return 1;
  strncpy(name, st[i].first.c_str(), n - 1);
  name[n - 1] = 0;
  *dtype = (int32_t)st[i].second.GetDType();
  *rank = st[i].second.Rank();
  for (int k = 0; k < *rank; k++) shape[k] = st[i].second.GetShape()[k];
  return 0;
}
OMH_API int32_t omh_trainer_model_state_get(omh_trainer* t, int32_t i, void* dst) {
  return Guard([&] { t->model->StateDict().at(i).second.CopyToHost(dst); });
}
OMH_API int32_t omh_trainer_model_state_set(omh_trainer* t, int32_t i, const void* src) {
  return Guard([&] { t->model->StateDict().at(i).second.CopyFromHost(src); });
}
OMH_API int32_t omh_trainer_opt_kind(omh_trainer* t, char* buf, size_t n) {
  std::string k = t->opt->Kind();
  strncpy(buf, k.c_str(), n - 1);
  buf[n - 1] = 0;
  return 0;
}
OMH_API int32_t omh_trainer_hyper_count(omh_trainer* t) { return (int32_t)t->opt->HyperParameters().size(); }
OMH_API int32_t omh_trainer_hyper_info(omh_trainer* t, int32_t i, char* name, size_t n, float* value) {
  auto h = t->opt->HyperParameters();
  if (i < 0 || i >= (int)h.size()) return 1;
  strncpy(name, h[i].first.c_str(), n - 1);
  name[n - 1] = 0;
  *value = h[i].second;
  return 0;
}
OMH_API int32_t omh_trainer_state_count(omh_trainer* t) { return (int32_t)t->opt->NamedState().size(); }
OMH_API int32_t omh_trainer_state_info(omh_trainer* t, int32_t i, char* name, size_t n, int32_t* dtype, int32_t* rank, int32_t* shape) {
  auto st = t->opt->NamedState();
  if (i < 0 || i >= (int)st.size()) return 1;
  strncpy(name, st[i].name.c_str(), n - 1);
  name[n - 1] = 0;
  if (st[i].flags) {
    *dtype = OM_I32;
    *rank = 1;
    shape[0] = (int32_t)st[i].flags->size();
  } else {
    *dtype = OM_F32;
    *rank = st[i].tensor.Rank();
    for (int k = 0; k < *rank; k++) shape[k] = st[i].tensor.GetShape()[k];
  }
  return 0;
}
OMH_API int32_t omh_trainer_state_get(omh_trainer* t, int32_t i, void* dst) {
  return Guard([&] {
    auto st = t->opt->NamedState();
    if (st.at(i).flags) memcpy(dst, st[i].flags->data(), st[i].flags->size() * 4);
    else st[i].tensor.CopyToHost(dst);
  });
}
OMH_API int32_t omh_trainer_state_set(omh_trainer* t, int32_t i, const void* src) {
  return Guard([&] {
    auto st = t->opt->NamedState();
    if (st.at(i).flags) memcpy(st[i].flags->data(), src, st[i].flags->size() * 4);
    else st[i].tensor.CopyFromHost(src);
  });
}
// Restores the step count, the learning rate and the weight decay (Optimizer.RestoreStepCount / SetHyperParameters); the fixed settings
// (betas, epsilon, momentum ...) are compared by the loader, not changed.
OMH_API int32_t omh_trainer_restore(omh_trainer* t, int64_t steps, float lr, float weight_decay) {
  return Guard([&] {
    if (steps < 0) throw ArgumentOutOfRangeException("The step count must not be negative.");
    if (t->graph) throw InvalidOperationException("Restore a checkpoint before capturing the step.");
    t->opt->StepCount = steps;
    t->steps_done = steps;
    t->opt->LearningRate = lr;
    t->opt->WeightDecay = weight_decay;
  });
}
