// Plain-C surface of the host mirror (libonemodel_b200_host.so), used by the Python tests and the bench through
// ctypes: tensors are opaque handles, operations are dispatched by name, and every C++ exception becomes a status
// code (1 shape, 2 index, 9 invalid operation, 11 a saved tensor changed in place, 12 not supported, 10 other) with the message kept for omh_last_error.
#include <stdio.h>
#include <string.h>

#include <map>

#include "omh.hpp"

using namespace omh;

#define OMH_API extern "C" __attribute__((visibility("default")))

static thread_local std::string t_error;

template <class F>
static int32_t Guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const TensorShapeException& e) {
    t_error = e.what();
    return 1;
  } catch (const ArgumentOutOfRangeException& e) {
    t_error = e.what();
    return 2;
  } catch (const TensorVersionException& e) {
    t_error = e.what();
    return 11;
  } catch (const InvalidOperationException& e) {
    t_error = e.what();
    return 9;
  } catch (const NotSupportedException& e) {
    t_error = e.what();
    return 12;
  } catch (const BackendException& e) {
    t_error = e.what();
    return 100 + e.status;
  } catch (const std::exception& e) {
    t_error = e.what();
    return 10;
  }
}

struct omh_tensor { Tensor t; };
static omh_tensor* Box(const Tensor& t) { return t.IsEmpty() ? nullptr : new omh_tensor{t}; }
static Tensor Unbox(const omh_tensor* h) { return h ? h->t : Tensor(); }

OMH_API int32_t omh_last_error(char* buf, size_t n) {
  if (!buf || !n) return 1;
  size_t len = std::min(n - 1, t_error.size());
  memcpy(buf, t_error.data(), len);
  buf[len] = 0;
  return 0;
}

OMH_API int32_t omh_init(int32_t device, uint32_t flags, om_ctx** out) {
  om_ctx* ctx = nullptr;
  int32_t s = om_ctx_create(device, flags, &ctx);
  if (s != OM_OK) {
    char buf[512];
    om_last_error(nullptr, buf, sizeof buf);
    t_error = buf;
    return 100 + s;
  }
  Device::SetCurrent(ctx);
  if (out) *out = ctx;
  return 0;
}

OMH_API int32_t omh_set_current(om_ctx* ctx) {
  Device::SetCurrent(ctx);
  return 0;
}

OMH_API int32_t omh_tensor_from_host(int32_t dtype, int32_t rank, const int32_t* shape, const void* data, omh_tensor** out) {
  return Guard([&] {
    Shape s;
    if (rank > kMaxRank) throw TensorShapeException("Too many dimensions.");
    s.rank = rank;
    for (int i = 0; i < rank; i++) s.d[i] = shape[i];
    Tensor t = Tensor::Create((DType)dtype, s);
    if (data && t.Length() > 0) t.CopyFromHost(data);
    *out = new omh_tensor{t};
  });
}

OMH_API int32_t omh_tensor_free(omh_tensor* h) {
  delete h;
  return 0;
}

OMH_API int32_t omh_tensor_info(const omh_tensor* h, int32_t* dtype, int32_t* rank, int32_t* shape, int64_t* strides) {
  if (!h) return 1;
  *dtype = (int32_t)h->t.GetDType();
  *rank = h->t.Rank();
  for (int i = 0; i < h->t.Rank(); i++) {
    shape[i] = h->t.GetShape()[i];
    if (strides) strides[i] = h->t.Strides()[i];
  }
  return 0;
}

OMH_API int32_t omh_tensor_to_host(const omh_tensor* h, void* dst) {
  return Guard([&] { h->t.CopyToHost(dst); });
}

OMH_API int32_t omh_tensor_copy_from_host(omh_tensor* h, const void* src) {
  return Guard([&] { h->t.CopyFromHost(src); });
}

OMH_API void* omh_tensor_data(const omh_tensor* h) { return h ? h->t.RawData() : nullptr; }

OMH_API int32_t omh_tensor_set_requires_grad(omh_tensor* h, int32_t on) {
  return Guard([&] { h->t.SetRequiresGrad(on != 0); });
}

OMH_API int32_t omh_tensor_requires_grad(const omh_tensor* h) { return h && h->t.RequiresGrad(); }

OMH_API int32_t omh_tensor_grad(const omh_tensor* h, omh_tensor** out) {
  return Guard([&] { *out = Box(h->t.Grad()); });
}

// The leaf's row-sparse gradient (Tensor.SparseGrad): *row_count = 0 and null handles when there is none; otherwise the row
// count, the row numbers (Int32 [row_count]) and the values (float32 [row_count, width], a view of the gradient's storage).
OMH_API int32_t omh_tensor_sparse_grad(const omh_tensor* h, int32_t* row_count, omh_tensor** rows, omh_tensor** values) {
  return Guard([&] {
    *row_count = 0;
    *rows = *values = nullptr;
    auto sg = h->t.SparseGrad();
    if (!sg) return;
    *row_count = sg->RowCount();
    *rows = Box(sg->RowsStorage().Slice(0, 0, *row_count));
    *values = Box(sg->Values());
  });
}
// RowSparseGradient.ToDense (add_to null: a new tensor in *out) or AddTo (dense[row] += values[k] into add_to). Merge has no
// entry of its own: it runs when two sparse lookups of one table meet in a backward pass.
OMH_API int32_t omh_tensor_sparse_grad_to_dense(const omh_tensor* h, omh_tensor* add_to, omh_tensor** out) {
  return Guard([&] {
    auto sg = h->t.SparseGrad();
    if (!sg) throw InvalidOperationException("The tensor has no row-sparse gradient.");
    if (add_to) {
      sg->AddTo(add_to->t);
      if (out) *out = nullptr;
    } else {
      *out = Box(sg->ToDense());
    }
  });
}

OMH_API int32_t omh_tensor_zero_grad(const omh_tensor* h) {
  return Guard([&] { Backprop::ZeroGrad(h->t); });
}

OMH_API int32_t omh_tensor_clear_grad(const omh_tensor* h) {
  return Guard([&] { Backprop::ClearGrad(h->t); });
}

OMH_API int32_t omh_backward(const omh_tensor* h, const omh_tensor* gradient, int32_t retain) {
  return Guard([&] {
    Tensor g = Unbox(gradient);
    h->t.Backward(gradient ? &g : nullptr, retain != 0);
  });
}

OMH_API int32_t omh_no_grad(int32_t on) {
  static thread_local std::vector<GradMode::NoGrad*> stack;
  if (on) stack.push_back(new GradMode::NoGrad());
  else if (!stack.empty()) {
    delete stack.back();
    stack.pop_back();
  }
  return 0;
}

// One entry for every operation and view: inputs are handles (null = empty tensor), plus integer and float arguments.
OMH_API int32_t omh_call(const char* op, int32_t n_in, omh_tensor* const* in, int32_t n_ints, const int64_t* ints,
                         int32_t n_floats, const double* fl, omh_tensor** out) {
  return Guard([&] {
    std::string name = op;
    auto T = [&](int i) { return i < n_in ? Unbox(in[i]) : Tensor(); };
    auto I = [&](int i, int64_t dflt = 0) { return i < n_ints ? ints[i] : dflt; };
    auto F = [&](int i, double dflt = 0) { return i < n_floats ? fl[i] : dflt; };
    auto ShapeFromInts = [&](int from) {
      Shape s;
      for (int i = from; i < n_ints; i++) s.d[s.rank++] = (int)ints[i];
      return s;
    };
    Tensor r;
    if (name == "add") r = Ops::Add(T(0), T(1));
    else if (name == "sub") r = Ops::Sub(T(0), T(1));
    else if (name == "mul") r = Ops::Mul(T(0), T(1));
    else if (name == "div") r = Ops::Div(T(0), T(1));
    else if (name == "neg") r = Ops::Neg(T(0));
    else if (name == "relu") r = Ops::Relu(T(0));
    else if (name == "gelu") r = Ops::Gelu(T(0), I(0) != 0);
    else if (name == "sigmoid") r = Ops::Sigmoid(T(0));
    else if (name == "tanh") r = Ops::Tanh(T(0));
    else if (name == "matmul") r = Ops::MatMul(T(0), T(1));
    else if (name == "sum") r = n_ints ? Ops::Sum(T(0), (int)I(0), I(1) != 0) : Ops::Sum(T(0));
    else if (name == "mean") r = n_ints ? Ops::Mean(T(0), (int)I(0), I(1) != 0) : Ops::Mean(T(0));
    else if (name == "softmax") r = Ops::Softmax(T(0), (int)I(0, -1));
    else if (name == "log_softmax") r = Ops::LogSoftmax(T(0), (int)I(0, -1));
    else if (name == "layer_norm") r = Ops::LayerNorm(T(0), T(1), T(2), (float)F(0, 1e-5));
    else if (name == "add_layer_norm") r = Ops::AddLayerNorm(T(0), T(1), T(2), T(3), (float)F(0, 1e-5));
    else if (name == "batch_norm2d") r = Ops::BatchNorm2d(T(0), T(1), T(2), T(3), T(4), I(0) != 0, (float)F(0, 0.1), (float)F(1, 1e-5));
    else if (name == "embedding") r = Ops::Embedding(T(0), T(1), (int)I(0, -1), I(1, 0) != 0);
    else if (name == "nll_loss") r = Ops::NllLoss(T(0), T(1), I(0, 1) != 0, (int)I(1, -100));
    else if (name == "cross_entropy") r = Ops::CrossEntropy(T(0), T(1), I(0, 1) != 0, (int)I(1, -100), (float)F(0, 0));
    else if (name == "cross_entropy_smoothed") r = Losses::CrossEntropy(T(0), T(1), (float)F(0, 0), (int)I(1, -100), I(0, 1) != 0);
    else if (name == "mse_loss") r = Losses::Mse(T(0), T(1), I(0, 1) != 0);
    else if (name == "l1_loss") r = Losses::L1(T(0), T(1), I(0, 1) != 0);
    else if (name == "bce_with_logits") r = Losses::BceWithLogits(T(0), T(1), I(0, 1) != 0);
    else if (name == "dropout") r = Ops::Dropout(T(0), (float)F(0, 0.5), (uint64_t)I(0), T(1));
    else if (name == "linear") r = Ops::Linear(T(0), T(1), T(2));
    else if (name == "feed_forward") r = Ops::FeedForward(T(0), T(1), T(2), T(3), T(4), I(0) != 0);
    else if (name == "attention") r = Ops::Attention(T(0), T(1), T(2), T(3), (float)F(0, 0));
    else if (name == "attention_heads") r = Ops::AttentionHeads(T(0), T(1), T(2), (int)I(0, 1), T(3), (float)F(0, 0));
    else if (name == "concat") {
      std::vector<Tensor> xs;
      for (int i = 0; i < n_in; i++) xs.push_back(T(i));
      r = Ops::Concat(xs, (int)I(0));
    } else if (name == "global_avg_pool2d") r = Ops::GlobalAvgPool2d(T(0));
    else if (name == "conv2d") {
      Conv2dParams p;
      p.strideH = (int)I(0, 1); p.strideW = (int)I(1, 1);
      p.padTop = (int)I(2); p.padLeft = (int)I(3); p.padBottom = (int)I(4); p.padRight = (int)I(5);
      p.dilH = (int)I(6, 1); p.dilW = (int)I(7, 1); p.groups = (int)I(8, 1);
      r = Ops::Conv2d(T(0), T(1), T(2), p);
    } else if (name == "max_pool2d") r = Ops::MaxPool2d(T(0), (int)I(0), (int)I(1), (int)I(2), (int)I(3), (int)I(4), (int)I(5));
    else if (name == "avg_pool2d") r = Ops::AvgPool2d(T(0), (int)I(0), (int)I(1), (int)I(2), (int)I(3), (int)I(4), (int)I(5), I(6) != 0);
    else if (name == "lstm_layer") r = Ops::LstmLayer(T(0), T(1), T(2), T(3), T(4), I(0) != 0);
    else if (name == "conv1d") {
      Conv1dParams p;
      p.stride = (int)I(0, 1); p.padLeft = (int)I(1); p.padRight = (int)I(2); p.dilation = (int)I(3, 1); p.groups = (int)I(4, 1);
      r = Ops::Conv1d(T(0), T(1), T(2), p);
    } else if (name == "conv_transpose2d") {
      ConvTranspose2dParams p;
      p.strideH = (int)I(0, 1); p.strideW = (int)I(1, 1); p.padH = (int)I(2); p.padW = (int)I(3); p.outPadH = (int)I(4); p.outPadW = (int)I(5);
      p.dilH = (int)I(6, 1); p.dilW = (int)I(7, 1); p.groups = (int)I(8, 1);
      r = Ops::ConvTranspose2d(T(0), T(1), T(2), p);
    } else if (name == "resize2d") r = Ops::Resize2d(T(0), (int)I(0), (int)I(1), (int)I(2), I(3) != 0);
    else if (name == "matmul_batched") r = Ops::MatMulBatched(T(0), T(1));
    else if (name == "erf") r = Ops::Erf(T(0));
    else if (name == "exp") r = Ops::Exp(T(0));
    else if (name == "sqrt") r = Ops::Sqrt(T(0));
    else if (name == "pow") r = Ops::Pow(T(0), (float)F(0, 1));
    else if (name == "where") r = Ops::Where(T(0), T(1), T(2));
    else if (name == "gather") r = Ops::Gather(T(0), T(1), (int)I(0));
    else if (name == "lstm_bidirectional") {
      std::vector<Tensor> ws;
      for (int k = 1; k < 9; k++) ws.push_back(T(k));
      r = Ops::LstmBidirectional(T(0), ws);
    } else if (name == "gru_layer") r = Ops::GruLayer(T(0), T(1), T(2), T(3), T(4), T(5), I(0) != 0);
    else if (name == "ctc_loss") r = Ops::CtcLoss(T(0), T(1), T(2), T(3), (int)I(0), (int)I(1, 1), I(2) != 0);
    else if (name == "reshape") r = T(0).Reshape(ShapeFromInts(0));
    else if (name == "permute") {
      std::vector<int> axes;
      for (int i = 0; i < n_ints; i++) axes.push_back((int)ints[i]);
      r = T(0).Permute(axes);
    } else if (name == "t") r = T(0).T();
    else if (name == "slice") r = T(0).Slice((int)I(0), (int)I(1), (int)I(2), (int)I(3, 1));
    else if (name == "select") r = T(0).Select((int)I(0), (int)I(1));
    else if (name == "expand") r = T(0).Expand(ShapeFromInts(0));
    else if (name == "flip") r = T(0).Flip((int)I(0));
    else if (name == "clone") r = T(0).Clone();
    else if (name == "contiguous") r = T(0).Contiguous();
    else if (name == "detach") r = T(0).Detach();
    else throw InvalidOperationException("Unknown operation '" + name + "'.");
    *out = Box(r);
  });
}

// ---- optimizers -----------------------------------------------------------------------------------------------------
struct omh_optim { std::unique_ptr<Optimizer> o; };

// kind: 0 SGD (f: lr, momentum, dampening, weight_decay; i: nesterov), 1 Adam, 2 AdamW (f: lr, beta1, beta2, eps,
// weight_decay; i: amsgrad), 3 SparseAdam (f: lr, beta1, beta2, eps).
OMH_API int32_t omh_optim_create(int32_t kind, int32_t n, omh_tensor* const* params, const double* f, const int64_t* i,
                                 omh_optim** out) {
  return Guard([&] {
    std::vector<Tensor> ps;
    for (int k = 0; k < n; k++) ps.push_back(params[k]->t);
    std::unique_ptr<Optimizer> o;
    if (kind == 0) o.reset(new Sgd(ps, (float)f[0], (float)f[1], (float)f[2], (float)f[3], i[0] != 0));
    else if (kind == 1) o.reset(new Adam(ps, (float)f[0], (float)f[1], (float)f[2], (float)f[3], (float)f[4], false, i[0] != 0));
    else if (kind == 2) o.reset(new AdamW(ps, (float)f[0], (float)f[1], (float)f[2], (float)f[3], (float)f[4], i[0] != 0));
    else if (kind == 3) o.reset(new SparseAdam(ps, (float)f[0], (float)f[1], (float)f[2], (float)f[3]));
    else throw InvalidOperationException("Unknown optimizer kind.");
    *out = new omh_optim{std::move(o)};
  });
}
OMH_API int32_t omh_optim_free(omh_optim* o) {
  delete o;
  return 0;
}
OMH_API int32_t omh_optim_step(omh_optim* o) {
  return Guard([&] { o->o->Step(); });
}
OMH_API int32_t omh_optim_zero_grad(omh_optim* o) {
  return Guard([&] { o->o->ZeroGrad(); });
}
OMH_API int32_t omh_optim_set_lr(omh_optim* o, float lr) {
  o->o->LearningRate = lr;
  return 0;
}
OMH_API int32_t omh_clip_norm(int32_t n, omh_tensor* const* params, float max_norm, int32_t infinity, float* total) {
  return Guard([&] {
    std::vector<Tensor> ps;
    for (int k = 0; k < n; k++) ps.push_back(params[k]->t);
    *total = GradClip::ClipNorm(ps, max_norm, infinity != 0);
  });
}
OMH_API int32_t omh_clip_value(int32_t n, omh_tensor* const* params, float clip) {
  return Guard([&] {
    std::vector<Tensor> ps;
    for (int k = 0; k < n; k++) ps.push_back(params[k]->t);
    GradClip::ClipValue(ps, clip);
  });
}
// ---- modules (NnModule, Layers.cs, Recurrent.cs) -----------------------------------------------------------------------
// A module handle owns its module; a Sequential takes over the modules handed to it (their handles become empty and only
// need omh_module_free). `ints` / `floats` per kind:
//   linear [in, out, bias]; conv1d [in, out, kernel, stride, padding, dilation, groups, bias]; conv1d_same / conv1d_valid
//   [in, out, kernel, dilation, groups, bias]; conv2d [in, out, kernel, stride, padding, bias]; conv_transpose2d [in, out,
//   kernel, stride, padding, output padding, dilation, groups, bias]; batch_norm2d [channels] {momentum, eps}; layer_norm
//   [width] {eps}; embedding [count, width, padding index, sparse]; dropout [seed] {p}; recurrent [gru, input, hidden, layers,
//   bidirectional, batch first]; relu, sigmoid, tanh, flatten,
//   global_avg_pool2d []; gelu [tanh form]; max_pool2d / avg_pool2d [kernel, stride, padding]; mean [axis].
// The generator state (SplitMix64, Generator.cs:10-48) is passed in and out so that several modules draw their initial
// weights from one stream as the reference's constructors do.
struct omh_module { std::unique_ptr<NnModule> m; };
OMH_API int32_t omh_module_create(const char* kind, uint64_t* generator_state, int32_t n_ints, const int64_t* ints, int32_t n_floats,
                                  const double* fl, omh_module** out) {
  return Guard([&] {
    std::string k = kind;
    auto I = [&](int i, int64_t dflt = 0) { return i < n_ints ? ints[i] : dflt; };
    auto F = [&](int i, double dflt = 0) { return i < n_floats ? fl[i] : dflt; };
    Generator g(generator_state ? *generator_state : 0);
    NnModule* m = nullptr;
    if (k == "linear") m = new Linear((int)I(0), (int)I(1), g, I(2, 1) != 0);
    else if (k == "conv1d") m = new Conv1d((int)I(0), (int)I(1), (int)I(2), g, (int)I(3, 1), (int)I(4, 0), (int)I(5, 1), (int)I(6, 1), I(7, 1) != 0);
    else if (k == "conv1d_same" || k == "conv1d_valid")
      m = new Conv1d((int)I(0), (int)I(1), (int)I(2), g, std::string(k == "conv1d_same" ? "same" : "valid"), (int)I(3, 1), (int)I(4, 1), I(5, 1) != 0);
    else if (k == "conv2d") m = new Conv2d((int)I(0), (int)I(1), (int)I(2), g, (int)I(3, 1), (int)I(4, 0), I(5, 1) != 0);
    else if (k == "conv_transpose2d")
      m = new ConvTranspose2d((int)I(0), (int)I(1), (int)I(2), g, (int)I(3, 1), (int)I(4, 0), (int)I(5, 0), (int)I(6, 1), (int)I(7, 1), I(8, 1) != 0);
    else if (k == "batch_norm2d") m = new BatchNorm2d((int)I(0), (float)F(0, 0.1), (float)F(1, 1e-5));
    else if (k == "layer_norm") m = new LayerNorm((int)I(0), (float)F(0, 1e-5));
    else if (k == "embedding") m = new Embedding((int)I(0), (int)I(1), g, (int)I(2, -1), I(3, 0) != 0);
    else if (k == "dropout") m = new Dropout((float)F(0, 0.5), (uint64_t)I(0));
    else if (k == "recurrent") m = new Recurrent(I(0) != 0, (int)I(1), (int)I(2), g, (int)I(3, 1), I(4) != 0, I(5) != 0);
    else if (k == "relu") m = Lambda::Relu();
    else if (k == "gelu") m = Lambda::Gelu(I(0) != 0);
    else if (k == "sigmoid") m = Lambda::Sigmoid();
    else if (k == "tanh") m = Lambda::Tanh();
    else if (k == "max_pool2d") m = Lambda::MaxPool2d((int)I(0), (int)I(1, 0), (int)I(2, 0));
    else if (k == "avg_pool2d") m = Lambda::AvgPool2d((int)I(0), (int)I(1, 0), (int)I(2, 0));
    else if (k == "global_avg_pool2d") m = Lambda::GlobalAvgPool2d();
    else if (k == "flatten") m = Lambda::Flatten();
    else if (k == "mean") m = Lambda::Mean((int)I(0));
    else throw InvalidOperationException("Unknown module kind '" + k + "'.");
    if (generator_state) *generator_state = g.State();
    *out = new omh_module{std::unique_ptr<NnModule>(m)};
  });
}
OMH_API int32_t omh_sequential_create(int32_t n, omh_module* const* layers, omh_module** out) {
  return Guard([&] {
    std::vector<NnModule*> ls;
    for (int i = 0; i < n; i++) {
      if (!layers[i] || !layers[i]->m) throw InvalidOperationException("A layer handle is empty.");
      ls.push_back(layers[i]->m.get());
    }
    for (int i = 0; i < n; i++) layers[i]->m.release();
    *out = new omh_module{std::unique_ptr<NnModule>(new Sequential(ls))};
  });
}
OMH_API void omh_module_free(omh_module* m) { delete m; }
OMH_API int32_t omh_module_forward(omh_module* m, omh_tensor* x, omh_tensor** out) {
  return Guard([&] { *out = Box(m->m->Forward(Unbox(x))); });
}
// A Recurrent stack over rows of different lengths padded to a common T (packed-sequence semantics).
OMH_API int32_t omh_module_forward_lengths(omh_module* m, omh_tensor* x, int32_t n, const int32_t* lengths, omh_tensor** out) {
  return Guard([&] {
    auto* r = dynamic_cast<Recurrent*>(m->m.get());
    if (!r) throw InvalidOperationException("Only a recurrent stack takes lengths.");
    *out = Box(r->Forward(Unbox(x), std::vector<int>(lengths, lengths + n)));
  });
}
OMH_API int32_t omh_module_train(omh_module* m, int32_t on) {
  return Guard([&] { m->m->Train(on != 0); });
}
OMH_API int32_t omh_module_zero_grad(omh_module* m) {
  return Guard([&] { m->m->ZeroGrad(); });
}
// which: 0 the state dict (parameters, buffers, children), 1 parameters, 2 trainable parameters, 3 buffers.
static std::vector<std::pair<std::string, Tensor>> ModuleList(omh_module* m, int32_t which) {
  switch (which) {
    case 0: return m->m->StateDict();
    case 1: return m->m->NamedParameters();
    case 2: return m->m->NamedTrainableParameters();
    case 3: return m->m->NamedBuffers();
    default: throw ArgumentOutOfRangeException("Unknown list.");
  }
}
OMH_API int32_t omh_module_count(omh_module* m, int32_t which, int32_t* count) {
  return Guard([&] { *count = (int32_t)ModuleList(m, which).size(); });
}
OMH_API int32_t omh_module_entry(omh_module* m, int32_t which, int32_t index, char* name, int32_t name_capacity, omh_tensor** tensor) {
  return Guard([&] {
    auto list = ModuleList(m, which);
    if (index < 0 || index >= (int32_t)list.size()) throw ArgumentOutOfRangeException("No such entry.");
    snprintf(name, (size_t)name_capacity, "%s", list[(size_t)index].first.c_str());
    *tensor = Box(list[(size_t)index].second);
  });
}
// name null or empty: every parameter. The count of parameters that changed is returned in `changed`.
OMH_API int32_t omh_module_set_frozen(omh_module* m, const char* name_or_prefix, int32_t frozen, int32_t* changed) {
  return Guard([&] {
    bool all = !name_or_prefix || !*name_or_prefix;
    *changed = frozen ? (all ? m->m->Freeze() : m->m->Freeze(std::string(name_or_prefix)))
                      : (all ? m->m->Unfreeze() : m->m->Unfreeze(std::string(name_or_prefix)));
  });
}
OMH_API int32_t omh_module_is_frozen(omh_module* m, const char* name, int32_t* frozen) {
  return Guard([&] { *frozen = m->m->IsFrozen(name) ? 1 : 0; });
}
OMH_API int32_t omh_module_load_state(omh_module* m, int32_t n, const char* const* names, omh_tensor* const* tensors) {
  return Guard([&] {
    std::vector<std::pair<std::string, Tensor>> state;
    for (int i = 0; i < n; i++) state.emplace_back(names[i], Unbox(tensors[i]));
    m->m->LoadStateDict(state);
  });
}

// Learning-rate schedules. kind: 0 constant {lr}; 1 step {base, gamma} [step size]; 2 cosine {base, min} [total];
// 3 warm-up {start factor} [warm-up steps] in front of `after`; 4 warm-up + cosine {base, floor fraction} [warm-up, total];
// 5 one cycle {max, pct start, div factor, final div factor} [total].
struct omh_schedule { std::shared_ptr<LrSchedule> s; };
OMH_API int32_t omh_schedule_create(int32_t kind, const float* f, const int64_t* n, const omh_schedule* after, omh_schedule** out) {
  return Guard([&] {
    std::shared_ptr<LrSchedule> s;
    switch (kind) {
      case 0: s = LrSchedule::Constant(f[0]); break;
      case 1: s = LrSchedule::Step(f[0], n[0], f[1]); break;
      case 2: s = LrSchedule::Cosine(f[0], n[0], f[1]); break;
      case 3: s = LrSchedule::Warmup(after ? after->s : nullptr, n[0], f[0]); break;
      case 4: s = LrSchedule::WarmupCosine(f[0], n[0], n[1], f[1]); break;
      case 5: s = LrSchedule::OneCycle(f[0], n[0], f[1], f[2], f[3]); break;
      default: throw ArgumentOutOfRangeException("Unknown schedule kind.");
    }
    *out = new omh_schedule{std::move(s)};
  });
}
OMH_API float omh_schedule_lr_at(const omh_schedule* h, int64_t step) { return h->s->LrAt(step); }
OMH_API void omh_schedule_free(omh_schedule* h) { delete h; }
OMH_API double omh_schedule_cos(double t) { return LrSchedule::Cos(t); }
