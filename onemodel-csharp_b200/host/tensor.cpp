// Tensor: a strided view over reference-counted device memory, with the view operations that the reference
// records on the tape (src/OneModel/Tensors/Tensor.cs, Tensor.Views.cs:11-21,314-318, Tensor.Copy.cs).
#include <string.h>

#include "omh.hpp"

namespace omh {

static thread_local om_ctx* t_ctx = nullptr;

om_ctx* Device::Current() {
  if (!t_ctx) throw InvalidOperationException("No device context is current: call Device::SetCurrent first.");
  return t_ctx;
}
void Device::SetCurrent(om_ctx* ctx) { t_ctx = ctx; }

void Check(int32_t status) {
  if (status == OM_OK) return;
  char buf[512] = {0};
  om_last_error(t_ctx, buf, sizeof buf);
  std::string msg = buf[0] ? buf : "backend call failed";
  switch (status) {
    case OM_ERR_SHAPE: throw TensorShapeException(msg);
    case OM_ERR_INDEX: throw ArgumentOutOfRangeException(msg);
    default: throw BackendException(status, msg);
  }
}

Shape::Shape(std::initializer_list<int> dims) {
  if (dims.size() > (size_t)kMaxRank) throw TensorShapeException("Too many dimensions.");
  for (int v : dims) d[rank++] = v;
}
Shape::Shape(const std::vector<int>& dims) {
  if (dims.size() > (size_t)kMaxRank) throw TensorShapeException("Too many dimensions.");
  for (int v : dims) d[rank++] = v;
}
int64_t Shape::Length() const {
  int64_t n = 1;
  for (int i = 0; i < rank; i++) n *= d[i];
  return n;
}
bool Shape::operator==(const Shape& o) const {
  if (rank != o.rank) return false;
  for (int i = 0; i < rank; i++)
    if (d[i] != o.d[i]) return false;
  return true;
}
std::string Shape::ToString() const {
  std::string s = "[";
  for (int i = 0; i < rank; i++) s += (i ? "," : "") + std::to_string(d[i]);
  return s + "]";
}

Buffer::Buffer(om_ctx* c, size_t n, bool zero) : ctx(c), bytes(n) {
  Check(om_alloc(c, n == 0 ? 4 : n, zero ? 1 : 0, &ptr));
}
Buffer::~Buffer() {
  if (owned && ptr) om_free(ctx, ptr);
}

std::array<int64_t, kMaxRank> ContiguousStrides(const Shape& s) {
  std::array<int64_t, kMaxRank> st{};
  int64_t acc = 1;
  for (int i = s.rank - 1; i >= 0; i--) {
    st[i] = acc;
    acc *= s.d[i];
  }
  return st;
}

Tensor Tensor::Create(DType t, const Shape& s, bool zero) {
  Tensor r;
  for (int i = 0; i < s.rank; i++)
    if (s.d[i] < 0) throw TensorShapeException("Negative extent in " + s.ToString());
  r.buf_ = std::make_shared<Buffer>(Device::Current(), (size_t)s.Length() * SizeOf(t), zero);
  r.shape_ = s;
  r.strides_ = ContiguousStrides(s);
  r.dtype_ = t;
  return r;
}

Tensor Tensor::CreateBf16Only(const Shape& s) {
  Tensor r;
  for (int i = 0; i < s.rank; i++)
    if (s.d[i] < 0) throw TensorShapeException("Negative extent in " + s.ToString());
  // A stub of fp32 storage (never read or written) whose bfloat16 copy is the tensor.
  r.buf_ = std::make_shared<Buffer>(Device::Current(), (size_t)16, false);
  r.buf_->shadow = std::make_shared<Buffer>(Device::Current(), (((size_t)s.Length() * 2) + 15) & ~(size_t)15, false);
  r.buf_->fp32_absent = true;
  r.buf_->shadow_version = r.buf_->version;
  r.shape_ = s;
  r.strides_ = ContiguousStrides(s);
  r.dtype_ = DType::F32;
  return r;
}

Tensor Tensor::Wrap(void* device_ptr, DType t, const Shape& s) {
  Tensor r;
  r.buf_ = std::make_shared<Buffer>(Device::Current(), device_ptr, (size_t)s.Length() * SizeOf(t));
  r.shape_ = s;
  r.strides_ = ContiguousStrides(s);
  r.dtype_ = t;
  return r;
}

Tensor Tensor::FromHost(const float* data, const Shape& s) {
  Tensor r = Create(DType::F32, s);
  r.CopyFromHost(data);
  return r;
}
Tensor Tensor::FromHostInt32(const int32_t* data, const Shape& s) {
  Tensor r = Create(DType::I32, s);
  r.CopyFromHost(data);
  return r;
}
Tensor Tensor::FromHostInt64(const int64_t* data, const Shape& s) {
  Tensor r = Create(DType::I64, s);
  r.CopyFromHost(data);
  return r;
}

bool Tensor::IsContiguous() const {
  int64_t acc = 1;
  for (int i = shape_.rank - 1; i >= 0; i--) {
    if (shape_.d[i] != 1 && strides_[i] != acc) return false;
    acc *= shape_.d[i];
  }
  return true;
}

void* Tensor::RawData() const {
  if (IsEmpty()) return nullptr;
  if (buf_->fp32_absent) throw InvalidOperationException("This tensor exists as bfloat16 only; a consumer asked for its float32 values.");
  return (char*)buf_->ptr + offset_ * (int64_t)SizeOf(dtype_);
}
float* Tensor::Data() const { return (float*)RawData(); }

Tensor Tensor::View(const Shape& s, const std::array<int64_t, kMaxRank>& strides, int64_t offset) const {
  Tensor r;
  r.buf_ = buf_;
  r.offset_ = offset;
  r.shape_ = s;
  r.strides_ = strides;
  r.dtype_ = dtype_;
  return r;
}

Tensor Tensor::WithAutograd(std::shared_ptr<AutogradMeta> m) const {
  Tensor r = *this;
  r.meta_ = std::move(m);
  return r;
}

// A view of a tensor that requires grad carries a record of the view's kind (Tensor.Derive in the reference).
static Tensor Derive(const Tensor& src, Tensor view, OpKind op, std::vector<int64_t> ints) {
  if (!GradMode::Enabled() || !src.RequiresGrad()) return view;
  auto rec = BackwardRecord::Create(op, 0, {&src});
  rec->Ints = std::move(ints);
  return rec->Attach(view);
}

Tensor Tensor::Reshape(const Shape& s) const {
  if (s.Length() != Length()) throw TensorShapeException("Cannot reshape " + shape_.ToString() + " to " + s.ToString());
  // A strided source is copied first; Contiguous() keeps the copy on the tape.
  Tensor base = IsContiguous() ? *this : Contiguous();
  Tensor v = base.View(s, ContiguousStrides(s), base.offset_);
  return Derive(base, v, OpKind::Reshape, {});
}

Tensor Tensor::Permute(const std::vector<int>& axes) const {
  if ((int)axes.size() != shape_.rank) throw TensorShapeException("Permute needs one axis per dimension.");
  Shape s;
  s.rank = shape_.rank;
  std::array<int64_t, kMaxRank> st{};
  std::vector<int64_t> ints;
  bool seen[kMaxRank] = {false};
  for (int i = 0; i < shape_.rank; i++) {
    int a = axes[i] < 0 ? axes[i] + shape_.rank : axes[i];
    if (a < 0 || a >= shape_.rank || seen[a]) throw TensorShapeException("Permute axes must be a permutation.");
    seen[a] = true;
    s.d[i] = shape_.d[a];
    st[i] = strides_[a];
    ints.push_back(a);
  }
  return Derive(*this, View(s, st, offset_), OpKind::Permute, ints);
}

Tensor Tensor::T() const {
  if (shape_.rank != 2) throw TensorShapeException("T() needs a matrix, not " + shape_.ToString());
  return Permute({1, 0});
}

Tensor Tensor::Transpose(int a, int b) const {
  std::vector<int> axes(shape_.rank);
  for (int i = 0; i < shape_.rank; i++) axes[i] = i;
  if (a < 0) a += shape_.rank;
  if (b < 0) b += shape_.rank;
  std::swap(axes[a], axes[b]);
  return Permute(axes);
}

Tensor Tensor::Slice(int axis, int start, int end, int step) const {
  if (axis < 0) axis += shape_.rank;
  if (axis < 0 || axis >= shape_.rank || step < 1 || start < 0 || end > shape_.d[axis] || start > end)
    throw TensorShapeException("Slice out of range for " + shape_.ToString());
  Shape s = shape_;
  s.d[axis] = (end - start + step - 1) / step;
  auto st = strides_;
  st[axis] *= step;
  return Derive(*this, View(s, st, offset_ + start * strides_[axis]), OpKind::Slice, {axis, start, end, step});
}

Tensor Tensor::Select(int axis, int index) const {
  if (axis < 0) axis += shape_.rank;
  if (axis < 0 || axis >= shape_.rank || index < 0 || index >= shape_.d[axis])
    throw TensorShapeException("Select out of range for " + shape_.ToString());
  Shape s;
  std::array<int64_t, kMaxRank> st{};
  for (int i = 0; i < shape_.rank; i++) {
    if (i == axis) continue;
    s.d[s.rank] = shape_.d[i];
    st[s.rank] = strides_[i];
    s.rank++;
  }
  return Derive(*this, View(s, st, offset_ + index * strides_[axis]), OpKind::Select, {axis, index});
}

Tensor Tensor::Expand(const Shape& s) const {
  int lead = s.rank - shape_.rank;
  if (lead < 0) throw TensorShapeException("Cannot expand " + shape_.ToString() + " to " + s.ToString());
  std::array<int64_t, kMaxRank> st{};
  for (int i = 0; i < s.rank; i++) {
    int j = i - lead;
    if (j < 0) st[i] = 0;
    else if (shape_.d[j] == s.d[i]) st[i] = strides_[j];
    else if (shape_.d[j] == 1) st[i] = 0;
    else throw TensorShapeException("Cannot expand " + shape_.ToString() + " to " + s.ToString());
  }
  return Derive(*this, View(s, st, offset_), OpKind::Expand, {});
}

Tensor Tensor::Flip(int axis) const {
  if (axis < 0) axis += shape_.rank;
  if (axis < 0 || axis >= shape_.rank) throw TensorShapeException("Flip axis out of range.");
  auto st = strides_;
  int64_t off = offset_ + (shape_.d[axis] > 0 ? (shape_.d[axis] - 1) * strides_[axis] : 0);
  st[axis] = -st[axis];
  return Derive(*this, View(shape_, st, off), OpKind::Flip, {axis});
}

Tensor Tensor::Clone() const {
  if (IsEmpty()) return Tensor();
  Tensor r = Create(dtype_, shape_);
  if (Length() == 0) return r;
  if (dtype_ == DType::I64) {
    if (!IsContiguous()) throw TensorShapeException("Strided Int64 tensors cannot be copied on the device.");
    Check(om_memcpy_d2d(Device::Current(), r.RawData(), RawData(), (size_t)Length() * 8));
    return r;
  }
  // Int32 shares the 4-byte strided copy kernel.
  auto dst = ContiguousStrides(shape_);
  Check(om_strided_copy(Device::Current(), shape_.rank, shape_.d.data(), (const float*)RawData(), strides_.data(),
                        (float*)r.RawData(), dst.data()));
  return r;
}

Tensor Tensor::Contiguous() const {
  if (IsContiguous()) return *this;
  Tensor c = Clone();
  // The copy of a strided view is gradient-transparent: record it as a Reshape of the source view (the gradient is
  // reshaped to the source's shape, and the source view's own record routes it further).
  if (GradMode::Enabled() && RequiresGrad()) {
    auto rec = BackwardRecord::Create(OpKind::Reshape, 0, {this});
    return rec->Attach(c);
  }
  return c;
}

Tensor Tensor::Detach() const {
  Tensor r = *this;
  r.meta_.reset();
  return r;
}

// After an in-place write from the host side: the storage has a new version, and a bfloat16 copy that exists is brought up
// to date at once, because a captured step reads the copy without looking at versions.
static void StorageWritten(const Tensor& t) {
  t.MarkModified();
  if (t.GetDType() == DType::F32 && t.Storage()->shadow) t.Bf16();
}

void Tensor::Fill(float v) const {
  if (!IsContiguous()) throw TensorShapeException("Fill needs a contiguous tensor.");
  if (v == 0.f) Check(om_memset(Device::Current(), RawData(), 0, (size_t)Length() * SizeOf(dtype_)));
  else Check(om_fill(Device::Current(), Data(), v, Length()));
  StorageWritten(*this);
}

uint16_t* Tensor::Bf16ForWrite() const {
  if (IsEmpty() || dtype_ != DType::F32) throw InvalidOperationException("A bfloat16 copy exists for float32 tensors only.");
  Buffer& b = *buf_;
  if (!b.shadow) b.shadow = std::make_shared<Buffer>(b.ctx, ((b.bytes / 4) * 2 + 15) & ~(size_t)15, false);
  return (uint16_t*)b.shadow->ptr + offset_;
}

const uint16_t* Tensor::Bf16() const {
  uint16_t* p = Bf16ForWrite();
  Buffer& b = *buf_;
  if (b.fp32_absent) return p;     // the copy is the tensor
  if (b.shadow_version != b.version) {
    Check(om_cast_bf16(b.ctx, (const float*)b.ptr, (uint16_t*)b.shadow->ptr, (int64_t)(b.bytes / 4)));
    b.shadow_version = b.version;
  }
  return p;
}

void Tensor::CopyFromHost(const void* src) const {
  if (!IsContiguous()) throw TensorShapeException("CopyFromHost needs a contiguous tensor.");
  Check(om_memcpy_h2d(Device::Current(), RawData(), src, (size_t)Length() * SizeOf(dtype_)));
  StorageWritten(*this);
  // The source is pageable caller memory: finish the copy before returning so the caller may reuse it.
  Check(om_sync(Device::Current()));
}

void Tensor::CopyToHost(void* dst) const {
  Tensor c = IsContiguous() ? *this : Clone();
  Check(om_memcpy_d2h(Device::Current(), dst, c.RawData(), (size_t)Length() * SizeOf(dtype_)));
}

std::vector<float> Tensor::ToVector() const {
  std::vector<float> v((size_t)Length());
  if (!v.empty()) CopyToHost(v.data());
  return v;
}

float Tensor::Item() const {
  if (Length() != 1) throw TensorShapeException("Item needs a one-element tensor.");
  float v = 0;
  CopyToHost(&v);
  return v;
}

bool Tensor::RequiresGrad() const { return meta_ && meta_->RequiresGrad; }

Tensor& Tensor::SetRequiresGrad(bool on) {
  if (meta_ && meta_->GradFn) throw InvalidOperationException("Only a leaf's RequiresGrad flag can be changed.");
  if (!meta_) meta_ = std::make_shared<AutogradMeta>();
  if (meta_->RequiresGrad == on) return *this;
  meta_->RequiresGrad = on;
  if (!on) {  // a frozen leaf drops its stored gradient, dense or row-sparse (Tensor.cs:418-452)
    meta_->Grad = Tensor();
    meta_->GradIsZero = false;
    meta_->SparseGrad.reset();
  }
  return *this;
}

Tensor Tensor::Grad() const {
  if (!meta_ || meta_->Grad.IsEmpty()) return Tensor();
  if (meta_->GradIsZero) {
    meta_->Grad.Fill(0.f);
    meta_->GradIsZero = false;
  }
  return meta_->Grad;
}

std::shared_ptr<RowSparseGradient> Tensor::SparseGrad() const {
  if (!meta_ || !meta_->SparseGrad || meta_->SparseGrad->RowCount() == 0) return nullptr;
  return meta_->SparseGrad;
}

void Tensor::Backward(const Tensor* gradient, bool retainGraph) const { Backprop::Run(*this, gradient, retainGraph); }

}  // namespace omh
