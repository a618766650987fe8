// C++ mirror of the reference's managed training API for the autograd hot path, written above the C ABI of
// libonemodel_b200.so. Names and semantics follow RecursiveAI.OneModel.Tensors / RecursiveAI.OneModel.Training:
//   Tensor (strided view + autograd meta)       src/OneModel/Tensors/Tensor.cs:29-50,396-473
//   BackwardRecord / AutogradMeta / OpKind       src/OneModel/Tensors/Autograd/{BackwardRecord,Autograd}.cs
//   Backprop / Engine                            src/OneModel/Tensors/Autograd/Engine.cs:21-344
//   Ops.*                                        src/OneModel/Tensors/Ops*.cs
//   NnModule, layers, Losses, optimizers         src/OneModel.Training/*.cs
// Every tensor lives in device memory; every op calls the C ABI and nothing here computes on the host except
// scalar bookkeeping (shapes, schedules, Adam's per-step bias corrections in double).
#pragma once
#include <stdint.h>

#include <array>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "onemodel_b200.h"

namespace omh {

// ---- errors (the reference's exception types) -----------------------------------------------------------------------
struct TensorShapeException : std::runtime_error { using std::runtime_error::runtime_error; };
struct ArgumentOutOfRangeException : std::runtime_error { using std::runtime_error::runtime_error; };
struct InvalidOperationException : std::runtime_error { using std::runtime_error::runtime_error; };
struct NotSupportedException : std::runtime_error { using std::runtime_error::runtime_error; };
// A tensor saved for the backward pass was modified in place before the pass read it (Autograd.cs:188-192).
struct TensorVersionException : InvalidOperationException { using InvalidOperationException::InvalidOperationException; };
struct BackendException : std::runtime_error {
  int32_t status;
  BackendException(int32_t s, const std::string& m) : std::runtime_error(m), status(s) {}
};

// ---- device ----------------------------------------------------------------------------------------------------------
// The process-wide compute selection of the reference (TensorCompute, Autograd/TensorCompute.cs:22-78) becomes the
// current device context.
struct Device {
  static om_ctx* Current();
  static void SetCurrent(om_ctx* ctx);
};
void Check(int32_t status);  // throws the mapped exception with om_last_error's text

// ---- shape -------------------------------------------------------------------------------------------------------------
constexpr int kMaxRank = 8;
struct Shape {
  int rank = 0;
  std::array<int32_t, kMaxRank> d{};
  Shape() = default;
  Shape(std::initializer_list<int> dims);
  explicit Shape(const std::vector<int>& dims);
  int operator[](int i) const { return d[i]; }
  int64_t Length() const;
  bool operator==(const Shape& o) const;
  bool operator!=(const Shape& o) const { return !(*this == o); }
  std::string ToString() const;
};

enum class DType : int32_t { F32 = OM_F32, I32 = OM_I32, I64 = OM_I64 };
inline size_t SizeOf(DType t) { return t == DType::I64 ? 8 : 4; }

struct Buffer {
  om_ctx* ctx = nullptr;
  void* ptr = nullptr;
  size_t bytes = 0;
  bool owned = true;
  // Counts the in-place writes to the storage (TensorBuffer.Version in the reference): a tensor saved for the backward
  // pass remembers the count it saw, and the bfloat16 copy below remembers the count it was made at.
  int64_t version = 0;
  // The bfloat16 copy of the whole storage, element i of the copy being element i of the fp32 storage rounded to nearest
  // even: the operand the products read under OM_BF16_OPERANDS. Made on first use, refreshed when the storage changed.
  std::shared_ptr<Buffer> shadow;
  int64_t shadow_version = -1;
  // The tensor exists as its bfloat16 copy only (an intermediate between two kernels that both work on bfloat16: the packed
  // q | k | v projections in front of the attention kernels, their gradient behind them). The fp32 storage is a stub and
  // any access to it throws, so a consumer that would need fp32 fails loudly instead of reading memory nobody wrote.
  bool fp32_absent = false;
  Buffer(om_ctx* c, size_t n, bool zero);
  Buffer(om_ctx* c, void* external, size_t n) : ctx(c), ptr(external), bytes(n), owned(false) {}
  ~Buffer();
  Buffer(const Buffer&) = delete;
  Buffer& operator=(const Buffer&) = delete;
};

struct BackwardRecord;
struct AutogradMeta;
class Tensor;
class RowSparseGradient;

// ---- tensor ------------------------------------------------------------------------------------------------------------
class Tensor {
 public:
  Tensor() = default;
  static Tensor Create(DType t, const Shape& s, bool zero = false);
  static Tensor Zeros(DType t, const Shape& s) { return Create(t, s, true); }
  static Tensor FromHost(const float* data, const Shape& s);
  static Tensor FromHostInt32(const int32_t* data, const Shape& s);
  static Tensor FromHostInt64(const int64_t* data, const Shape& s);
  // A tensor over caller-owned device memory (not freed by the tensor).
  static Tensor Wrap(void* device_ptr, DType t, const Shape& s);
  // A float32-typed tensor of this shape that holds its values as bfloat16 only (see Buffer::fp32_absent): Bf16() and
  // Bf16ForWrite() work, Data() throws.
  static Tensor CreateBf16Only(const Shape& s);
  bool Fp32Absent() const { return buf_ && buf_->fp32_absent; }

  bool IsEmpty() const { return !buf_; }
  const Shape& GetShape() const { return shape_; }
  int Rank() const { return shape_.rank; }
  int64_t Length() const { return IsEmpty() ? 0 : shape_.Length(); }
  DType GetDType() const { return dtype_; }
  const std::array<int64_t, kMaxRank>& Strides() const { return strides_; }
  bool IsContiguous() const;
  float* Data() const;  // device pointer to the first element
  void* RawData() const;
  // The storage's version counter; 0 for an empty tensor (Tensor.cs:190-191).
  int64_t Version() const { return buf_ ? buf_->version : 0; }
  // Tells the tensor that a kernel wrote into its storage in place (what MutableData does in the reference, Tensor.cs:292).
  void MarkModified() const {
    if (buf_) buf_->version++;
  }
  // Device pointer to this view's first element in the storage's bfloat16 copy (fp32 tensors only; the view's offset must
  // be a multiple of 8 elements for the copy to be usable as a product operand). Casts the storage when the copy is older
  // than the storage.
  const uint16_t* Bf16() const;
  // True when the storage has a bfloat16 copy at all (current or not): the tensor is used as a product operand.
  bool HasBf16Storage() const { return buf_ && buf_->shadow != nullptr; }
  // True when the storage already has an up-to-date bfloat16 copy.
  bool HasBf16() const { return buf_ && buf_->shadow && buf_->shadow_version == buf_->version; }
  // Storage for the bfloat16 copy, for a kernel that writes it together with the fp32 values; the caller then marks it current.
  uint16_t* Bf16ForWrite() const;
  void Bf16Written() const {
    if (buf_) buf_->shadow_version = buf_->version;
  }

  // views (each records a view record when the source requires grad; Tensor.Views.cs:11-21)
  Tensor Reshape(const Shape& s) const;
  Tensor Permute(const std::vector<int>& axes) const;
  Tensor T() const;
  Tensor Transpose(int a, int b) const;
  Tensor Slice(int axis, int start, int end, int step = 1) const;
  Tensor Select(int axis, int index) const;
  Tensor Expand(const Shape& s) const;
  Tensor Flip(int axis) const;
  Tensor Clone() const;        // contiguous copy, no autograd link
  Tensor Contiguous() const;   // this if contiguous, else Clone
  Tensor Detach() const;
  void Fill(float v) const;
  void CopyFromHost(const void* src) const;  // contiguous only
  void CopyToHost(void* dst) const;          // any layout (clones when strided); synchronises
  std::vector<float> ToVector() const;
  float Item() const;

  // autograd surface (Tensor.cs:396-473)
  bool RequiresGrad() const;
  Tensor& SetRequiresGrad(bool on = true);
  Tensor Grad() const;
  // The row-sparse gradient a sparse Embedding lookup left on this leaf (Tensor.cs:408), or null: none, or one without rows
  // (nothing but padding was looked up). Reads the row count from the device.
  std::shared_ptr<RowSparseGradient> SparseGrad() const;
  void Backward(const Tensor* gradient = nullptr, bool retainGraph = false) const;
  const std::shared_ptr<AutogradMeta>& Autograd() const { return meta_; }
  Tensor WithAutograd(std::shared_ptr<AutogradMeta> m) const;

  // internal: same storage with a different view
  Tensor View(const Shape& s, const std::array<int64_t, kMaxRank>& strides, int64_t offset) const;
  int64_t Offset() const { return offset_; }
  const std::shared_ptr<Buffer>& Storage() const { return buf_; }

 private:
  std::shared_ptr<Buffer> buf_;
  int64_t offset_ = 0;  // elements
  Shape shape_;
  std::array<int64_t, kMaxRank> strides_{};
  DType dtype_ = DType::F32;
  std::shared_ptr<AutogradMeta> meta_;
};

std::array<int64_t, kMaxRank> ContiguousStrides(const Shape& s);

// ---- autograd types ---------------------------------------------------------------------------------------------------
// The reference's 43 kinds (Autograd.cs:7-97) plus the fused kinds this backend records in their place: Linear for
// the Reshape/MatMul/Add chain of Ops.Linear, CrossEntropy for LogSoftmax+NllLoss, GlobalAvgPool for Mean over planes,
// FeedForward for Linear -> Gelu -> Linear when the activation rides in the products' epilogues.
enum class OpKind {
  None = 0, Add, Sub, Mul, Div, Neg, Relu, MatMul, MaxPool2d, Cast, Slice, Permute, Reshape, Expand, Flip, Select, Gelu,
  Sigmoid, Tanh, Sum, Mean, Softmax, LogSoftmax, LayerNorm, BatchNorm, Conv2d, AvgPool2d, Concat, Embedding, NllLoss,
  Attention, Lstm, Gru, CtcLoss, ConvTranspose2d, Resize2d, Conv1d, BatchMatMul, Erf, Exp, Sqrt, Pow, Where, Gather,
  Linear, CrossEntropy, Dropout, FeedForward
};

struct AutogradMeta {
  bool RequiresGrad = false;
  std::shared_ptr<BackwardRecord> GradFn;  // null for a leaf
  int OutputIndex = 0;
  Tensor Grad;
  // The gradient buffer is kept across steps; after ZeroGrad its contents are logically zero and are overwritten by
  // the first gradient that arrives instead of being zero-filled and then added to.
  bool GradIsZero = false;
  // Set instead of Grad by a sparse Embedding lookup on a leaf table (Autograd.cs:128).
  std::shared_ptr<RowSparseGradient> SparseGrad;
  bool IsLeaf() const { return !GradFn; }
};

// The gradient of a [rows, width] table that touches only some rows (RowSparseGradient.cs:14-120): the touched row numbers in
// ascending order, each once, and their gradients, row k of the values belonging to Rows()[k]; the values are the dense
// gradient's rows bit for bit. The arrays live on the device with a fixed capacity and a device-side row count (entries
// behind the count: row -1, zero values), so backward, clipping and the optimizers never read the count back; RowCount(),
// Rows() and Values() do.
class RowSparseGradient {
 public:
  RowSparseGradient(const Shape& denseShape, Tensor rows, Tensor values, Tensor count)
      : dense_shape_(denseShape), rows_(std::move(rows)), values_(std::move(values)), count_(std::move(count)) {}
  const Shape& DenseShape() const { return dense_shape_; }
  int Capacity() const { return rows_.GetShape()[0]; }
  int RowCount() const;                   // synchronises
  std::vector<int32_t> Rows() const;      // strictly ascending, each in [0, rows); synchronises
  Tensor Values() const;                  // float32 [RowCount, width], a view: writable (gradient clipping scales it); synchronises
  const Tensor& RowsStorage() const { return rows_; }      // Int32 [capacity]
  const Tensor& ValuesStorage() const { return values_; }  // float32 [capacity, width], zero behind the row count
  const Tensor& CountStorage() const { return count_; }    // Int32 [1]
  int64_t ByteCount() const { return (int64_t)RowCount() * (dense_shape_[1] * 4 + 4); }
  Tensor ToDense() const;                 // a new zeroed dense tensor with the rows scattered into it
  void AddTo(const Tensor& dense) const;  // dense[row] += values[k]
  // a + b: the union of the rows; a row in both gets a's values plus b's (a first).
  static std::shared_ptr<RowSparseGradient> Merge(const RowSparseGradient& a, const RowSparseGradient& b);

 private:
  Shape dense_shape_;
  Tensor rows_, values_, count_;
};

struct BackwardRecord : std::enable_shared_from_this<BackwardRecord> {
  OpKind Op = OpKind::None;
  std::vector<std::shared_ptr<AutogradMeta>> Inputs;  // null where the input needs no gradient
  std::vector<Shape> InputShapes;
  std::vector<DType> InputTypes;
  std::vector<Tensor> SavedSlots;
  std::vector<int64_t> SavedVersions;   // the storage version of each saved tensor when it was saved
  std::vector<int64_t> Ints;
  std::vector<double> Floats;
  Tensor PendingGrad;
  // The pending gradient's storage is also held by another record's pending gradient (a gradient that an Add hands to both
  // of its inputs is not copied): it is read freely but copied before anything is added into it.
  bool PendingShared = false;
  // This record's backward reads its incoming gradient as bfloat16 only (a packed Linear on the bfloat16 route): the
  // producer of that gradient may hand over a tensor made by Tensor::CreateBf16Only.
  bool TakesBf16OnlyGrad = false;
  int VisitMark = 0;
  bool IsReleased = false;

  static std::shared_ptr<BackwardRecord> Create(OpKind op, int savedSlots, std::initializer_list<const Tensor*> inputs);
  static std::shared_ptr<BackwardRecord> Create(OpKind op, int savedSlots, const std::vector<Tensor>& inputs);
  int InputCount() const { return (int)Inputs.size(); }
  bool NeedsInputGrad(int i) const { return Inputs[i] != nullptr; }
  // The saved tensor after checking that its storage was not written in place since it was saved
  // (SavedTensor.Unpack, Autograd.cs:198-238); an empty slot comes back empty.
  const Tensor& Saved(int slot) const;
  void Save(int slot, const Tensor& t) {
    SavedSlots[slot] = t;
    SavedVersions[slot] = t.Version();
  }
  Tensor Attach(const Tensor& output, int outputIndex = 0);
  void Release();
};

// RAII no-grad scope (GradMode.NoGrad, Autograd.cs:149).
struct GradMode {
  static bool Enabled();
  struct NoGrad {
    bool prev;
    NoGrad();
    ~NoGrad();
  };
};

// The reference frees every step temporary when the scope is disposed (ActivationScope.cs:18-106). Device buffers here
// are reference counted, so disposing the scope only drops the scope's own references; it is kept so that training
// loops read the same.
struct ActivationScope {
  ActivationScope();
  ~ActivationScope();
  static void Track(const Tensor& t);
  std::vector<Tensor> tracked;
  ActivationScope* outer;
};

struct Backprop {
  static void Run(const Tensor& root, const Tensor* gradient = nullptr, bool retainGraph = false);
  static void ZeroGrad(const Tensor& leaf);
  static void ClearGrad(const Tensor& leaf);
  // Called when the last gradient of a leaf has arrived in the running backward pass (data-parallel bucket trigger).
  static std::function<void(AutogradMeta*)> GradReadyHook;
};

class Engine {
 public:
  void Execute(const std::shared_ptr<BackwardRecord>& root, Tensor rootGrad, bool retain);
  static void Emit(BackwardRecord& rec, int i, const Tensor& grad, bool owned);
  // A view of the gradient this record received: owned by the receiver unless that gradient is itself shared.
  void EmitAliased(BackwardRecord& rec, int i, const Tensor& view) { Emit(rec, i, view, !current_shared_); }
  // The gradient the running record received is shared with another record (see BackwardRecord::PendingShared).
  bool CurrentShared() const { return current_shared_; }
  static void AccumulateLeaf(AutogradMeta& leaf, const Tensor& grad, bool owned);
  // Sends a row-sparse gradient to input i, a table the record gathered rows from (Engine.EmitSparse, Engine.cs:252-290): a
  // computed table gets it as a dense gradient; a leaf that already holds a dense gradient has it added in; otherwise it
  // becomes (or is merged into) the leaf's SparseGrad.
  static void EmitSparse(BackwardRecord& rec, int i, std::shared_ptr<RowSparseGradient> grad);
  // If input i is a leaf that keeps a gradient buffer, returns that buffer and whether the kernel must add to it
  // (accumulate) or overwrite it; the caller then calls LeafWritten instead of Emit.
  static bool LeafTarget(BackwardRecord& rec, int i, float** ptr, bool* accumulate);
  static void LeafWritten(BackwardRecord& rec, int i);
  // If input i's producer already holds a gradient from another branch (contiguous, of the input's shape), returns it: the
  // backward kernel then adds into it (what Emit would do with AddInto in a pass of its own) and calls PendingWritten.
  // *shared: that gradient's storage is shared and must not be written; the caller either forms the sum out of place and
  // installs it with PendingReplace, or asks for a private copy with PendingOwn and adds into that.
  static bool PendingTarget(BackwardRecord& rec, int i, Tensor* pending, bool* shared);
  static void PendingWritten(BackwardRecord& rec, int i);
  static void PendingReplace(BackwardRecord& rec, int i, const Tensor& sum);
  static Tensor PendingOwn(BackwardRecord& rec, int i);
  static void AddInto(const Tensor& dst, const Tensor& src);

 private:
  bool current_shared_ = false;
};

// True when the current context multiplies bfloat16 copies of the operands (OM_BF16_OPERANDS with OM_TF32), and whether a
// tensor with the given row pitch can be such an operand.
bool Bf16Products();
bool Bf16Operand(const Tensor& t, int64_t pitch);

void RunBackwardOp(Engine& e, BackwardRecord& r, const Tensor& g);
void RunGraphBackward(BackwardRecord& r, const Tensor& g);

// ---- ops ---------------------------------------------------------------------------------------------------------------
struct Conv2dParams {
  int strideH = 1, strideW = 1, padTop = 0, padLeft = 0, padBottom = 0, padRight = 0, dilH = 1, dilW = 1, groups = 1;
};

// Conv1dParams of the reference (Ops.Nn.cs:12-25): zero stride, dilation or groups mean 1.
struct Conv1dParams {
  int stride = 1, padLeft = 0, padRight = 0, dilation = 1, groups = 1;
};

struct ConvTranspose2dParams {
  int strideH = 1, strideW = 1, padH = 0, padW = 0, outPadH = 0, outPadW = 0, dilH = 1, dilW = 1, groups = 1;
};

struct Ops {
  static Tensor Add(const Tensor& a, const Tensor& b);
  static Tensor Sub(const Tensor& a, const Tensor& b);
  static Tensor Mul(const Tensor& a, const Tensor& b);
  static Tensor Div(const Tensor& a, const Tensor& b);
  static Tensor Neg(const Tensor& x);
  static Tensor Relu(const Tensor& x);
  static Tensor MatMul(const Tensor& a, const Tensor& b);
  static Tensor Gelu(const Tensor& x, bool approximateTanh = false);
  static Tensor Sigmoid(const Tensor& x);
  static Tensor Tanh(const Tensor& x);
  static Tensor Sum(const Tensor& x);
  static Tensor Sum(const Tensor& x, int axis, bool keepDim = false);
  static Tensor Mean(const Tensor& x);
  static Tensor Mean(const Tensor& x, int axis, bool keepDim = false);
  static Tensor Softmax(const Tensor& x, int axis = -1);
  static Tensor LogSoftmax(const Tensor& x, int axis = -1);
  static Tensor LayerNorm(const Tensor& x, const Tensor& gamma, const Tensor& beta, float epsilon = 1e-5f);
  // LayerNorm(Add(a, b), gamma, beta) in one pass over a and b (the residual connection in front of a layer norm).
  static Tensor AddLayerNorm(const Tensor& a, const Tensor& b, const Tensor& gamma, const Tensor& beta, float epsilon = 1e-5f);
  static Tensor BatchNorm2d(const Tensor& x, const Tensor& gamma, const Tensor& beta, const Tensor& runningMean,
                            const Tensor& runningVar, bool training, float momentum = 0.1f, float epsilon = 1e-5f);
  static Tensor Conv2d(const Tensor& x, const Tensor& weight, const Tensor& bias, const Conv2dParams& p);
  static Tensor MaxPool2d(const Tensor& x, int kh, int kw, int sh, int sw, int ph = 0, int pw = 0);
  static Tensor AvgPool2d(const Tensor& x, int kh, int kw, int sh, int sw, int ph = 0, int pw = 0, bool countIncludePad = false);
  static Tensor GlobalAvgPool2d(const Tensor& x);
  static Tensor Concat(const std::vector<Tensor>& xs, int axis);
  // sparse: when the table is a gradient leaf, backward leaves Tensor::SparseGrad (only the looked-up rows) instead of a
  // dense gradient (Ops.Layers.cs:554).
  static Tensor Embedding(const Tensor& table, const Tensor& ids, int paddingIndex = -1, bool sparse = false);
  static Tensor NllLoss(const Tensor& logProbs, const Tensor& targets, bool mean = true, int ignoreIndex = -100);
  static Tensor CrossEntropy(const Tensor& logits, const Tensor& targets, bool mean = true, int ignoreIndex = -100,
                             float denominator = 0.f);
  static Tensor Linear(const Tensor& x, const Tensor& weight, const Tensor& bias);
  static Tensor Attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& mask, float scale = 0.f);
  static Tensor AttentionHeads(const Tensor& q, const Tensor& k, const Tensor& v, int heads, const Tensor& mask, float scale = 0.f);
  // Several Linear layers over the same input whose weights (and biases) are adjacent in memory, as one product:
  // returns [..., sum of out features]. Throws when the parameters are not adjacent.
  // bf16_only_result: the caller consumes the result as bfloat16 only (the attention kernels of the bfloat16 tier); under
  // bfloat16 products the result is then made by Tensor::CreateBf16Only and no fp32 copy is written.
  static Tensor LinearPacked(const Tensor& x, const std::vector<Tensor>& weights, const std::vector<Tensor>& biases, bool bf16_only_result = false);
  // True when AttentionPacked on the packed projections of `input` ([B, L, .]) with this width and head count will take the
  // bfloat16 kernels, forward and backward, and so never read the projections as fp32.
  static bool AttentionPackedReadsBf16Only(const Tensor& input, int width, int heads);
  // Linear(Gelu(Linear(x, w1, b1)), w2, b2), the feed-forward block of an encoder layer. Under bfloat16 products (and
  // shapes the fused kernels take) the activation and its derivative are applied in the epilogues of the first forward
  // product and of the second layer's input-gradient product; the values are those of the three separate ops, which is
  // what runs otherwise.
  static Tensor FeedForward(const Tensor& x, const Tensor& w1, const Tensor& b1, const Tensor& w2, const Tensor& b2, bool approximateTanh = false);
  static bool Adjacent(const std::vector<Tensor>& parts);
  // Self-attention over the packed projections [B, L, 3 * H * D] (q | k | v along the last axis).
  static Tensor AttentionPacked(const Tensor& qkv, int heads, const Tensor& mask, float scale = 0.f);
  // One LSTM layer direction: returns y [T,B,H]; hn/cn receive the final states when not null.
  static Tensor LstmLayer(const Tensor& x, const Tensor& wIh, const Tensor& wHh, const Tensor& bIh, const Tensor& bHh,
                          bool reverse, Tensor* hn = nullptr, Tensor* cn = nullptr);
  // Both directions of a bidirectional LSTM layer, concatenated on the feature axis: [T,B,2H]. w[0..3] = forward
  // direction (wIh, wHh, bIh, bHh), w[4..7] = reverse direction; biases may be empty (both or none per direction).
  static Tensor LstmBidirectional(const Tensor& x, const std::vector<Tensor>& w);
  // One GRU layer direction (Ops.Recurrent.cs:148-260): returns y [T,B,H]; h0 [B,H] may be empty (zeros).
  static Tensor GruLayer(const Tensor& x, const Tensor& wIh, const Tensor& wHh, const Tensor& bIh, const Tensor& bHh,
                         const Tensor& h0, bool reverse);
  // Graph-op family (Ops.GraphOps.cs of the reference).
  static Tensor MatMulBatched(const Tensor& a, const Tensor& b);
  static Tensor Erf(const Tensor& x);
  static Tensor Exp(const Tensor& x);
  static Tensor Sqrt(const Tensor& x);
  static Tensor Pow(const Tensor& x, float exponent);
  // y = x * mask, the mask of call number draws[0] of the stream `seed` (kept elements scaled by 1/(1-p)); advances the
  // device counter `draws` (Int64 [1]) by one. The product of the reference's Dropout.Forward (Layers.cs:339-370).
  static Tensor Dropout(const Tensor& x, float p, uint64_t seed, const Tensor& draws);
  static Tensor Where(const Tensor& condition, const Tensor& x, const Tensor& y);
  static Tensor Gather(const Tensor& data, const Tensor& indices, int axis);
  // 1-D cross-correlation of an NCL input with OIK weights on the 2-D kernels with a height of 1 (Ops.Layers.cs:338-402;
  // backward BackwardNn.cs:313-321: the 2-D backward on the height-1 view).
  static Tensor Conv1d(const Tensor& x, const Tensor& weight, const Tensor& bias, const Conv1dParams& p);
  // Transposed convolution, the adjoint of Conv2d (Ops.Spatial.cs:43-130): x [N,Cin,H,W], weight [Cin,Cout/G,KH,KW].
  static Tensor ConvTranspose2d(const Tensor& x, const Tensor& weight, const Tensor& bias, const ConvTranspose2dParams& p);
  // mode 0 nearest, 1 bilinear (Ops.Spatial.cs:148-197).
  static Tensor Resize2d(const Tensor& x, int outH, int outW, int mode, bool alignCorners);
  static Tensor CtcLoss(const Tensor& logProbs, const Tensor& targets, const Tensor& inputLengths,
                        const Tensor& targetLengths, int blank, int reduction, bool zeroInfinity);
  static bool Recording(std::initializer_list<const Tensor*> inputs);
};

// ---- modules, losses, optimizers -------------------------------------------------------------------------------------
class Generator {  // SplitMix64, src/OneModel.Training/Generator.cs:10-48
 public:
  explicit Generator(uint64_t seed) : state_(seed) {}
  uint64_t NextUInt64();
  float NextSingle() { return (float)(NextUInt64() >> 40) * (1.0f / 16777216.0f); }
  float Uniform(float low, float high) { return low + (high - low) * NextSingle(); }
  uint64_t State() const { return state_; }
  void Restore(uint64_t state) { state_ = state; }
 private:
  uint64_t state_;
};

class NnModule {
 public:
  virtual ~NnModule() = default;
  virtual Tensor Forward(const Tensor& input) = 0;
  // Parameters in registration order, children after own parameters (NnModule.cs:139-311).
  std::vector<std::pair<std::string, Tensor>> NamedParameters(const std::string& prefix = "") const;
  std::vector<Tensor> Parameters() const;
  // The state order of the reference (docs/training.md section 1): a module's parameters, then its buffers, then each
  // child with a dotted path. Checkpoints store the model in this order.
  std::vector<std::pair<std::string, Tensor>> StateDict(const std::string& prefix = "") const;
  std::vector<std::pair<std::string, Tensor>> NamedBuffers(const std::string& prefix = "") const;
  // Parameters that still require gradients: the list an optimizer gets after Freeze (NnModule.cs:160-200).
  std::vector<std::pair<std::string, Tensor>> NamedTrainableParameters() const;
  std::vector<Tensor> TrainableParameters() const;
  // Freeze / Unfreeze switch RequiresGrad of the named parameter, of every parameter under a module path (a prefix ends
  // at a dot), of those a predicate picks, or of all; they return how many changed and throw when a name matches
  // nothing. A frozen parameter receives no gradient (its stored gradient is dropped) and costs no optimizer state.
  int Freeze();
  int Freeze(const std::string& nameOrPrefix);
  int Freeze(const std::function<bool(const std::string&, const Tensor&)>& predicate);
  int Unfreeze();
  int Unfreeze(const std::string& nameOrPrefix);
  int Unfreeze(const std::function<bool(const std::string&, const Tensor&)>& predicate);
  bool IsFrozen(const std::string& name) const;
  // Copies every entry of `state` into the module's own tensors (device to device) after checking that names, dtypes and
  // shapes match one to one (NnModule.cs:316-352).
  void LoadStateDict(const std::vector<std::pair<std::string, Tensor>>& state);
  void ZeroGrad();
  void Train(bool on = true);
  void Eval() { Train(false); }
  bool Training = true;
  const std::vector<std::pair<std::string, std::unique_ptr<NnModule>>>& Children() const { return children_; }
 protected:
  int SetTrainable(const std::function<bool(const std::string&, const Tensor&)>& predicate, bool trainable);
  int SetTrainable(const std::string& nameOrPrefix, bool trainable);
  Tensor RegisterParameter(const std::string& name, Tensor t);
  Tensor RegisterBuffer(const std::string& name, Tensor t);
  template <class M> M* RegisterModule(const std::string& name, M* m) {
    children_.emplace_back(name, std::unique_ptr<NnModule>(m));
    return m;
  }
  std::vector<std::pair<std::string, Tensor>> params_;
  std::vector<std::pair<std::string, Tensor>> buffers_;
  std::vector<std::pair<std::string, std::unique_ptr<NnModule>>> children_;
};

struct Linear : NnModule {
  Tensor Weight, Bias;
  Linear(int inFeatures, int outFeatures, Generator& g, bool bias = true);
  // Adopts existing storage (views into a packed allocation) as the parameters.
  Linear(Tensor weight, Tensor bias);
  Tensor Forward(const Tensor& x) override { return Ops::Linear(x, Weight, Bias); }
};
struct LayerNorm : NnModule {
  Tensor Gamma, Beta;
  float Epsilon;
  explicit LayerNorm(int width, float eps = 1e-5f);
  Tensor Forward(const Tensor& x) override { return Ops::LayerNorm(x, Gamma, Beta, Epsilon); }
};
// Inverted dropout with a seeded counter-based mask (Layers.cs:308-371). The call counter is the module's only buffer
// ("draws", Int64 [1], in device memory): restoring it from a checkpoint restores the stream of masks.
struct Dropout : NnModule {
  float P;
  uint64_t Seed;
  Tensor Counter;
  Dropout(float p, uint64_t seed);
  int64_t Draws() const;   // reads the counter back (synchronises)
  Tensor Forward(const Tensor& x) override { return (!Training || P == 0.f) ? x : Ops::Dropout(x, P, Seed, Counter); }
};
struct Embedding : NnModule {
  Tensor Weight;
  int PaddingIndex;
  // sparse: backward produces a row-sparse gradient (use with Sgd without momentum or SparseAdam; Layers.cs:276-294).
  bool IsSparse;
  Embedding(int count, int width, Generator& g, int paddingIndex = -1, bool sparse = false);
  Tensor Forward(const Tensor& ids) override { return Ops::Embedding(Weight, ids, PaddingIndex, IsSparse); }
};
struct Conv2d : NnModule {
  Tensor Weight, Bias;
  Conv2dParams P;
  Conv2d(int inCh, int outCh, int kernel, Generator& g, int stride = 1, int padding = 0, bool bias = true);
  Tensor Forward(const Tensor& x) override { return Ops::Conv2d(x, Weight, Bias, P); }
};
// Conv1d over [N, C, L] (Layers.cs:119-186): symmetric padding, or "same" / "valid" by name (stride 1).
struct Conv1d : NnModule {
  Tensor Weight, Bias;
  Conv1dParams P;
  Conv1d(int inCh, int outCh, int kernel, Generator& g, int stride = 1, int padding = 0, int dilation = 1, int groups = 1, bool bias = true);
  Conv1d(int inCh, int outCh, int kernel, Generator& g, const std::string& padding, int dilation = 1, int groups = 1, bool bias = true);
  Tensor Forward(const Tensor& x) override { return Ops::Conv1d(x, Weight, Bias, P); }
 private:
  void Init(int inCh, int outCh, int kernel, Generator& g, bool bias);
};
// Transposed convolution, weights [in, out/groups, k, k] (Recurrent.cs:71-115).
struct ConvTranspose2d : NnModule {
  Tensor Weight, Bias;
  ConvTranspose2dParams P;
  ConvTranspose2d(int inCh, int outCh, int kernel, Generator& g, int stride = 1, int padding = 0, int outputPadding = 0, int dilation = 1,
                  int groups = 1, bool bias = true);
  Tensor Forward(const Tensor& x) override { return Ops::ConvTranspose2d(x, Weight, Bias, P); }
};
// A parameter-free step of a Sequential (Layers.cs:373-426).
struct Lambda : NnModule {
  std::function<Tensor(const Tensor&)> Fn;
  explicit Lambda(std::function<Tensor(const Tensor&)> fn) : Fn(std::move(fn)) {}
  static Lambda* Relu() { return new Lambda([](const Tensor& x) { return Ops::Relu(x); }); }
  static Lambda* Gelu(bool approximateTanh = false) { return new Lambda([=](const Tensor& x) { return Ops::Gelu(x, approximateTanh); }); }
  static Lambda* Sigmoid() { return new Lambda([](const Tensor& x) { return Ops::Sigmoid(x); }); }
  static Lambda* Tanh() { return new Lambda([](const Tensor& x) { return Ops::Tanh(x); }); }
  static Lambda* MaxPool2d(int kernel, int stride = 0, int padding = 0) {
    int s = stride == 0 ? kernel : stride;
    return new Lambda([=](const Tensor& x) { return Ops::MaxPool2d(x, kernel, kernel, s, s, padding, padding); });
  }
  static Lambda* AvgPool2d(int kernel, int stride = 0, int padding = 0) {
    int s = stride == 0 ? kernel : stride;
    return new Lambda([=](const Tensor& x) { return Ops::AvgPool2d(x, kernel, kernel, s, s, padding, padding); });
  }
  static Lambda* GlobalAvgPool2d() { return new Lambda([](const Tensor& x) { return Ops::GlobalAvgPool2d(x); }); }
  static Lambda* Flatten() {
    return new Lambda([](const Tensor& x) {
      int rows = x.GetShape()[0];
      return x.Reshape(Shape{rows, (int)(x.Length() / (rows > 0 ? rows : 1))});
    });
  }
  static Lambda* Mean(int axis) { return new Lambda([=](const Tensor& x) { return Ops::Mean(x, axis); }); }
  Tensor Forward(const Tensor& x) override { return Fn(x); }
};
// Children named "0", "1", ... applied in order; takes ownership of the layers (Layers.cs:428-453).
struct Sequential : NnModule {
  explicit Sequential(std::vector<NnModule*> layers) {
    for (size_t i = 0; i < layers.size(); i++) RegisterModule(std::to_string(i), layers[i]);
  }
  Tensor Forward(const Tensor& x) override {
    Tensor h = x;
    for (auto& c : children_) h = c.second->Forward(h);
    return h;
  }
};
struct BatchNorm2d : NnModule {
  Tensor Gamma, Beta, RunningMean, RunningVar;
  float Momentum, Epsilon;
  explicit BatchNorm2d(int channels, float momentum = 0.1f, float eps = 1e-5f);
  Tensor Forward(const Tensor& x) override {
    return Ops::BatchNorm2d(x, Gamma, Beta, RunningMean, RunningVar, Training, Momentum, Epsilon);
  }
};
struct MultiHeadAttention : NnModule {
  Linear *Q, *K, *V, *O;
  int Heads;
  MultiHeadAttention(int width, int heads, Generator& g);
  Tensor Forward(const Tensor& x) override { return Forward(x, Tensor()); }
  Tensor Forward(const Tensor& x, const Tensor& mask);
};
struct TransformerEncoderLayer : NnModule {
  MultiHeadAttention* Attn;
  LayerNorm *Norm1, *Norm2;
  Linear *Ff1, *Ff2;
  TransformerEncoderLayer(int width, int heads, int ff, Generator& g);
  Tensor Forward(const Tensor& x) override { return Forward(x, Tensor()); }
  Tensor Forward(const Tensor& x, const Tensor& mask);
};
// Stacked (bi)directional LSTM or GRU over [T,B,I] ([B,T,I] when batchFirst) (src/OneModel.Training/Recurrent.cs:13-67).
// With `lengths` (one per batch row, each in [1, T]) the rows are sequences of different lengths padded to T, with the
// semantics of a packed sequence (Ops.Recurrent.cs:280-372): a row's reverse direction starts at its own last step from
// the zero state, and outputs at padded steps are exactly zero with zero gradient.
struct Recurrent : NnModule {
  int Hidden, Layers;
  bool Bidirectional, Gru = false, BatchFirst = false;
  std::vector<Tensor> WIh, WHh, BIh, BHh;  // per layer and direction
  Recurrent(int input, int hidden, int layers, bool bidirectional, Generator& g);
  Recurrent(bool gru, int input, int hidden, Generator& g, int layers = 1, bool bidirectional = false, bool batchFirst = false);
  Tensor Forward(const Tensor& x) override { return Forward(x, {}); }
  Tensor Forward(const Tensor& x, const std::vector<int>& lengths);
 private:
  void Init(int input, Generator& g);
  Tensor RunLayer(const Tensor& x, int k, bool reverse) const;
};

// Losses.cs:14-129 of the reference: thin compositions of Ops, so their gradients come from the records of those ops.
struct Losses {
  static Tensor CrossEntropy(const Tensor& logits, const Tensor& targets, bool mean = true, int ignoreIndex = -100) {
    return Ops::CrossEntropy(logits, targets, mean, ignoreIndex);
  }
  // With label smoothing: (1 - s) * NLL + s * (sum over counted rows of -mean_c(logp)), the second term divided by the
  // number of counted rows when `mean` (NaN when no row counts, as in the reference).
  static Tensor CrossEntropy(const Tensor& logits, const Tensor& targets, float labelSmoothing, int ignoreIndex, bool mean);
  static Tensor NllLoss(const Tensor& logp, const Tensor& targets, bool mean = true, int ignoreIndex = -100) {
    return Ops::NllLoss(logp, targets, mean, ignoreIndex);
  }
  static Tensor Ctc(const Tensor& logProbs, const Tensor& targets, const Tensor& inputLengths, const Tensor& targetLengths, int blank = 0,
                    int reduction = 1, bool zeroInfinity = false) {
    return Ops::CtcLoss(logProbs, targets, inputLengths, targetLengths, blank, reduction, zeroInfinity);
  }
  static Tensor Mse(const Tensor& prediction, const Tensor& target, bool mean = true);
  static Tensor L1(const Tensor& prediction, const Tensor& target, bool mean = true);
  // Mean or sum of softplus(x) - x*t, the softplus taken as -LogSoftmax([x, 0])[1] as the reference does.
  static Tensor BceWithLogits(const Tensor& logits, const Tensor& targets, bool mean = true);
};

class Optimizer {
 public:
  explicit Optimizer(std::vector<Tensor> parameters);
  virtual ~Optimizer() = default;
  void Step();      // Optimizers.cs:184-219
  void ZeroGrad();  // Optimizers.cs:222-228
  float LearningRate = 1e-3f;
  float WeightDecay = 0.f;
  int64_t StepCount = 0;
  const std::vector<Tensor>& Parameters() const { return params_; }
  // When set, the fused kernels read their per-step scalars from this device struct (graph replay).
  void* HyperDevice = nullptr;
  virtual size_t HyperBytes() const = 0;
  virtual void FillHyper(void* host, int64_t step) const = 0;  // scalars for the given 1-based step
  virtual std::vector<Tensor> StateTensors() const = 0;
  // Step() in groups of parameters (positions in Parameters()): `before(g)` runs before group g is launched. The data-parallel
  // trainer waits there for the group's gradient bucket, so that the update of early buckets overlaps the reduction of the
  // late ones. Every parameter gets the same update as from Step().
  void StepGroups(const std::vector<std::vector<int>>& groups, const std::function<void(int)>& before);
  // What a checkpoint stores (Checkpoint.cs, docs/training.md section 6 of the reference): the kind string, the
  // hyper-parameters in the reference's order, and the state tensors named slot.index in the reference's order. An entry
  // with a null tensor is the Int32 flag vector `flags` (Sgd's "initialized").
  struct StateEntry {
    std::string name;
    Tensor tensor;
    std::vector<int32_t>* flags = nullptr;
  };
  virtual std::string Kind() const = 0;
  virtual std::vector<std::pair<std::string, float>> HyperParameters() const = 0;
  virtual std::vector<StateEntry> NamedState() = 0;
 protected:
  virtual void BeginStep() {}
  // The update of parameter `index` from a row-sparse gradient (Optimizer.UpdateSparse, Optimizers.cs:184-219): an
  // optimizer without sparse semantics throws InvalidOperationException.
  virtual void UpdateSparse(int index, const Tensor& parameter, const RowSparseGradient& gradient);
  virtual void Launch(const std::vector<float*>& p, const std::vector<const float*>& g, const std::vector<int64_t>& len) = 0;
  std::vector<Tensor> params_;
  std::vector<int> index_;  // positions in params_ of the tensors of the running Step
  // For the tensors of the running Step, the bfloat16 copy to refresh in the same launch (null: none). A copy is offered
  // only where the launch updates every element of the copy's storage, so that the copy is current as a whole afterwards.
  std::vector<uint16_t*> p16_;
  // True for an optimizer whose Launch writes p16_ (Adam); the others leave the copies to the cast on next use.
  virtual bool WritesBf16Copies() const { return false; }
 private:
  void OfferBf16Copies();
  void Bf16CopiesWritten();
};

class Sgd : public Optimizer {
 public:
  Sgd(std::vector<Tensor> parameters, float lr, float momentum = 0.f, float dampening = 0.f, float weightDecay = 0.f,
      bool nesterov = false);
  size_t HyperBytes() const override { return sizeof(om_sgd_hyper); }
  void FillHyper(void* host, int64_t step) const override;
  std::vector<Tensor> StateTensors() const override { return buffers_; }
  std::string Kind() const override { return "sgd"; }
  std::vector<std::pair<std::string, float>> HyperParameters() const override;
  std::vector<StateEntry> NamedState() override;
  float GradScale = 1.f;
 protected:
  void Launch(const std::vector<float*>& p, const std::vector<const float*>& g, const std::vector<int64_t>& len) override;
  // p -= lr * g on the touched rows; NotSupportedException with momentum or weight decay (Optimizers.cs:377-397).
  void UpdateSparse(int index, const Tensor& parameter, const RowSparseGradient& gradient) override;
 private:
  float momentum_, dampening_;
  bool nesterov_;
  std::vector<Tensor> buffers_;
  std::vector<int32_t> initialized_;
};

class Adam : public Optimizer {
 public:
  Adam(std::vector<Tensor> parameters, float lr = 1e-3f, float beta1 = 0.9f, float beta2 = 0.999f, float eps = 1e-8f,
       float weightDecay = 0.f, bool decoupled = false, bool amsgrad = false);
  size_t HyperBytes() const override { return sizeof(om_adam_hyper); }
  void FillHyper(void* host, int64_t step) const override;
  std::vector<Tensor> StateTensors() const override;
  std::string Kind() const override { return decoupled_ ? "adamw" : "adam"; }
  std::vector<std::pair<std::string, float>> HyperParameters() const override;
  std::vector<StateEntry> NamedState() override;
  float GradScale = 1.f;
 protected:
  bool WritesBf16Copies() const override { return true; }
 
  void Launch(const std::vector<float*>& p, const std::vector<const float*>& g, const std::vector<int64_t>& len) override;
 private:
  float beta1_, beta2_, eps_;
  bool decoupled_, amsgrad_;
  std::vector<Tensor> m_, v_, vmax_;
};

class AdamW : public Adam {
 public:
  AdamW(std::vector<Tensor> parameters, float lr = 1e-3f, float beta1 = 0.9f, float beta2 = 0.999f, float eps = 1e-8f,
        float weightDecay = 0.01f, bool amsgrad = false)
      : Adam(std::move(parameters), lr, beta1, beta2, eps, weightDecay, true, amsgrad) {}
};

// Adam with lazy moments for row-sparse gradients (SparseAdam, Optimizers.cs:625-722): only the rows in a step's gradient have
// their moments and values updated; moments of untouched rows neither decay nor move; no weight decay, no AMSGrad; the step
// number is the optimizer's global one. A dense gradient throws InvalidOperationException.
class SparseAdam : public Optimizer {
 public:
  SparseAdam(std::vector<Tensor> parameters, float lr = 1e-3f, float beta1 = 0.9f, float beta2 = 0.999f, float eps = 1e-8f);
  size_t HyperBytes() const override { return 0; }
  void FillHyper(void*, int64_t) const override {}
  std::vector<Tensor> StateTensors() const override;
  std::string Kind() const override { return "sparseadam"; }
  std::vector<std::pair<std::string, float>> HyperParameters() const override;
  std::vector<StateEntry> NamedState() override;
 protected:
  void BeginStep() override;
  void Launch(const std::vector<float*>& p, const std::vector<const float*>& g, const std::vector<int64_t>& len) override;
  void UpdateSparse(int index, const Tensor& parameter, const RowSparseGradient& gradient) override;
 private:
  float beta1_, beta2_, eps_, step_size_ = 0.f;
  std::vector<Tensor> m_, v_;
};

struct GradClip {
  // Returns the total norm (synchronises to read it).
  static float ClipNorm(const std::vector<Tensor>& parameters, float maxNorm, bool infinityNorm = false);
  // Same without the read-back; norm_out (device float, may be null) receives the norm.
  static void ClipNormAsync(const std::vector<Tensor>& parameters, float maxNorm, bool infinityNorm, float* norm_out);
  static void ClipValue(const std::vector<Tensor>& parameters, float clipValue);
};

// Learning-rate schedules: pure host functions of the step index, 0 for the first step; a negative step counts as 0
// (Schedules.cs:151-422 of the reference). All arithmetic is in double and rounded to float once.
class LrSchedule {
 public:
  virtual ~LrSchedule() = default;
  virtual float LrAt(int64_t stepNumber) const = 0;
  // Sets the optimizer's learning rate to the rate for its current step count.
  void Apply(Optimizer& optimizer) const;
  // cos(pi t) for t in [0, 1] (clamped) from IEEE double operations only: reflected about 1/2 onto [0, pi/2] and summed as
  // the Maclaurin series up to degree 26 by Horner's rule, so that every platform gets the same rates (Schedules.cs:165-203).
  static double Cos(double t);

  static std::shared_ptr<LrSchedule> Constant(float lr);
  // base * gamma^(step / stepSize), the power by repeated squaring.
  static std::shared_ptr<LrSchedule> Step(float baseLr, int64_t stepSize, float gamma = 0.1f);
  // min + (base - min) (1 + cos(pi step / total)) / 2, held at min from `total` on.
  static std::shared_ptr<LrSchedule> Cosine(float baseLr, int64_t totalSteps, float minLr = 0.f);
  // after(0) * (start + (1 - start) step / warmup) for step < warmup, then after(step - warmup).
  static std::shared_ptr<LrSchedule> Warmup(std::shared_ptr<LrSchedule> after, int64_t warmupSteps, float startFactor = 0.f);
  // base (step + 1) / warmup, then base (floor + (1 - floor) (1 + cos(pi p)) / 2), p = (step - warmup) / (total - warmup).
  static std::shared_ptr<LrSchedule> WarmupCosine(float baseLr, int64_t warmupSteps, int64_t totalSteps, float floorFraction = 0.f);
  // Two cosine phases: max/div -> max over pctStart*total - 1 steps, then max -> max/div/finalDiv up to step total - 1.
  static std::shared_ptr<LrSchedule> OneCycle(float maxLr, int64_t totalSteps, float pctStart = 0.3f, float divFactor = 25.f,
                                              float finalDivFactor = 1e4f);
};

}  // namespace omh
