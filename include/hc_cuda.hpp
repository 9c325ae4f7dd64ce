// hc_cuda.hpp - C++ mirror of the part of Honeycrisp's `Backend` interface that libhccuda
// serves, header-only over the C ABI in hc_cuda.h.
//
// The reference's host language is Swift; where no Swift toolchain exists this is the compiled
// host side.  Names and argument meaning follow the reference:
//   Backend::matmul / batchedMatmul          Sources/Honeycrisp/Backend.swift:650-669
//   Backend::constant, cast                  Backend.swift:787-791, 489-494
//   add, columnSum, transpose, linear        what a Linear layer needs either side of its product
//                                            (Trainable.swift:530-546; Backend.swift:178-209, 524-531;
//                                            Index.swift:359-362), in the shapes it needs them
//   TensorData (byteCount, wait, onCPU)      Sources/Honeycrisp/Tensor.swift:69-85
//   BackendError (allocationFailed, kernelFailed, notImplemented)   Backend.swift:6-16
// A primitive a backend does not override throws BackendError::notImplemented, the reference's
// convention for partial backends.
#ifndef HC_CUDA_HPP_
#define HC_CUDA_HPP_

#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "hc_cuda.h"

namespace honeycrisp {

enum class DType { float16, float32, int64 };

inline size_t byteSize(DType t) { return t == DType::float16 ? 2 : t == DType::float32 ? 4 : 8; }

struct BackendError : std::runtime_error {
  enum class Kind { allocationFailed, kernelFailed, notImplemented } kind;
  BackendError(Kind k, const std::string& what) : std::runtime_error(what), kind(k) {}
  static BackendError notImplemented(const std::string& op) { return {Kind::notImplemented, "not implemented: " + op}; }
};

class Backend;

/// A buffer of tensor data owned by a backend (Tensor.Data).
class TensorData {
 public:
  virtual ~TensorData() = default;
  virtual size_t byteCount() const = 0;
  virtual void wait() = 0;
  /// The bytes on the host.
  virtual std::vector<unsigned char> onCPU() = 0;
};

/// The operator table.  Every primitive defaults to notImplemented (Backend.swift:28-892).
class Backend {
 public:
  virtual ~Backend() = default;
  virtual std::shared_ptr<TensorData> collection(const void* host, size_t count, DType) {
    (void)host; (void)count;
    throw BackendError::notImplemented("collection");
  }
  virtual std::shared_ptr<TensorData> matmul(const std::shared_ptr<TensorData>& a, bool transA,
                                             const std::shared_ptr<TensorData>& b, bool transB, bool transOut,
                                             int64_t rows, int64_t inner, int64_t cols, DType dtype) {
    (void)a; (void)transA; (void)b; (void)transB; (void)transOut; (void)rows; (void)inner; (void)cols; (void)dtype;
    throw BackendError::notImplemented("matmul");
  }
  virtual std::shared_ptr<TensorData> batchedMatmul(int64_t matrixCount, const std::shared_ptr<TensorData>& a,
                                                    bool transA, const std::shared_ptr<TensorData>& b, bool transB,
                                                    bool transOut, int64_t rows, int64_t inner, int64_t cols,
                                                    DType dtype) {
    (void)matrixCount; (void)a; (void)transA; (void)b; (void)transB; (void)transOut; (void)rows; (void)inner;
    (void)cols; (void)dtype;
    throw BackendError::notImplemented("batchedMatmul");
  }
  /// `count` elements equal to `value` (Backend.swift:787-791).
  virtual std::shared_ptr<TensorData> constant(float value, size_t count, DType dtype) {
    (void)value; (void)count; (void)dtype;
    throw BackendError::notImplemented("constant");
  }
  /// Elementwise conversion between element types (Backend.swift:489-494).
  virtual std::shared_ptr<TensorData> cast(const std::shared_ptr<TensorData>& a, size_t count, DType inType,
                                           DType outType) {
    (void)a; (void)count; (void)inType; (void)outType;
    throw BackendError::notImplemented("cast");
  }
  /// binaryOp(.add) on two buffers of equal shape (Backend.swift:178-209): gradient accumulation.
  virtual std::shared_ptr<TensorData> add(const std::shared_ptr<TensorData>& a, const std::shared_ptr<TensorData>& b,
                                          size_t count, DType dtype) {
    (void)a; (void)b; (void)count; (void)dtype;
    throw BackendError::notImplemented("add");
  }
  /// reduce(.sum) over the leading axis of a [rows, cols] buffer (Backend.swift:524-531): a bias gradient.
  virtual std::shared_ptr<TensorData> columnSum(const std::shared_ptr<TensorData>& a, int64_t rows, int64_t cols,
                                                DType dtype) {
    (void)a; (void)rows; (void)cols; (void)dtype;
    throw BackendError::notImplemented("columnSum");
  }
  /// The materialised `t()` of the last two axes (Index.swift:359-362).
  virtual std::shared_ptr<TensorData> transpose(const std::shared_ptr<TensorData>& a, int64_t matrixCount, int64_t rows,
                                                int64_t cols, DType dtype) {
    (void)a; (void)matrixCount; (void)rows; (void)cols; (void)dtype;
    throw BackendError::notImplemented("transpose");
  }
  /// x[rows, inCount] * weight[inCount, outCount] + bias[outCount]; `bias` may be null
  /// (Linear.callAsFunction, Trainable.swift:530-546).
  virtual std::shared_ptr<TensorData> linear(const std::shared_ptr<TensorData>& x, const std::shared_ptr<TensorData>& weight,
                                             const std::shared_ptr<TensorData>& bias, int64_t rows, int64_t inCount,
                                             int64_t outCount, DType dtype) {
    (void)x; (void)weight; (void)bias; (void)rows; (void)inCount; (void)outCount; (void)dtype;
    throw BackendError::notImplemented("linear");
  }
};

class CUDABackend;

class CUDAData : public TensorData {
 public:
  CUDAData(hc_ctx* ctx, size_t bytes) : ctx_(ctx), bytes_(bytes) {
    if (hc_alloc(ctx_, bytes_, &ptr_) != HC_OK) throw BackendError(BackendError::Kind::allocationFailed, "allocation failed");
  }
  ~CUDAData() override {
    if (event_) hc_event_destroy(event_);
    hc_free(ctx_, ptr_);
  }
  size_t byteCount() const override { return bytes_; }
  void* pointer() const { return ptr_; }
  void mark() {
    if (event_) hc_event_destroy(event_);
    event_ = nullptr;
    if (hc_event_record(ctx_, &event_) != HC_OK) throw BackendError(BackendError::Kind::kernelFailed, hc_last_error(ctx_));
  }
  void wait() override {
    const hc_status st = event_ ? hc_event_wait(event_) : hc_sync(ctx_);
    if (st != HC_OK) throw BackendError(BackendError::Kind::kernelFailed, hc_last_error(ctx_));
    inputs_.clear();
  }
  std::vector<unsigned char> onCPU() override {
    std::vector<unsigned char> host(bytes_ ? bytes_ : 1);
    if (bytes_ && (hc_d2h(ctx_, host.data(), ptr_, bytes_) != HC_OK || hc_sync(ctx_) != HC_OK))
      throw BackendError(BackendError::Kind::kernelFailed, hc_last_error(ctx_));
    wait();
    host.resize(bytes_);
    return host;
  }
  /// Start reading this buffer into (pinned) host memory on a side stream; later products keep
  /// running.  Wait on the returned marker with hc_event_wait and release it with hc_event_destroy.
  hc_event* readInto(void* host, size_t bytes) {
    hc_event* done = nullptr;
    if (bytes > bytes_ || hc_d2h_async(ctx_, host, ptr_, bytes, &done) != HC_OK)
      throw BackendError(BackendError::Kind::kernelFailed, hc_last_error(ctx_));
    return done;
  }
  /// Start filling this buffer from (pinned) host memory on a side stream; with `order` the work
  /// enqueued afterwards waits for the copy on the device.
  hc_event* writeFrom(const void* host, size_t bytes, bool order = true) {
    hc_event* done = nullptr;
    if (bytes > bytes_ || hc_h2d_async(ctx_, ptr_, host, bytes, &done) != HC_OK ||
        (order && hc_enqueue_wait(ctx_, done) != HC_OK))
      throw BackendError(BackendError::Kind::kernelFailed, hc_last_error(ctx_));
    return done;
  }
  void keep(std::shared_ptr<TensorData> a, std::shared_ptr<TensorData> b = nullptr, std::shared_ptr<TensorData> c = nullptr) {
    inputs_ = {std::move(a), std::move(b), std::move(c)};
  }

 private:
  hc_ctx* ctx_;
  size_t bytes_;
  void* ptr_ = nullptr;
  hc_event* event_ = nullptr;
  std::vector<std::shared_ptr<TensorData>> inputs_;   // operands stay alive until the product has run
};

/// `Backend.defaultBackend = try CUDABackend()` in the reference's terms.
class CUDABackend : public Backend {
 public:
  explicit CUDABackend(int device = 0) {
    const hc_status st = hc_init(device, &ctx_);
    if (st != HC_OK) throw BackendError(BackendError::Kind::kernelFailed, std::string("hc_init: ") + hc_status_string(st));
  }
  ~CUDABackend() override { hc_destroy(ctx_); }
  CUDABackend(const CUDABackend&) = delete;
  CUDABackend& operator=(const CUDABackend&) = delete;

  std::shared_ptr<TensorData> collection(const void* host, size_t count, DType dtype) override {
    auto d = std::make_shared<CUDAData>(ctx_, count * byteSize(dtype));
    check(hc_h2d(ctx_, d->pointer(), host, count * byteSize(dtype)));
    check(hc_sync(ctx_));
    return d;
  }

  std::shared_ptr<TensorData> matmul(const std::shared_ptr<TensorData>& a, bool transA,
                                     const std::shared_ptr<TensorData>& b, bool transB, bool transOut, int64_t rows,
                                     int64_t inner, int64_t cols, DType dtype) override {
    return batchedMatmul(1, a, transA, b, transB, transOut, rows, inner, cols, dtype);
  }

  std::shared_ptr<TensorData> batchedMatmul(int64_t matrixCount, const std::shared_ptr<TensorData>& a, bool transA,
                                            const std::shared_ptr<TensorData>& b, bool transB, bool transOut,
                                            int64_t rows, int64_t inner, int64_t cols, DType dtype) override {
    if (dtype != DType::float16 && dtype != DType::float32) throw BackendError::notImplemented("matmul for int64");
    auto da = std::dynamic_pointer_cast<CUDAData>(a), db = std::dynamic_pointer_cast<CUDAData>(b);
    // Operands of another backend's data type are staged through onCPU, as the reference's GPU
    // backend does (Sources/Honeycrisp/BackendMPS.swift:585-620).
    if (!da) { auto h = a->onCPU(); da = std::static_pointer_cast<CUDAData>(collection(h.data(), h.size() / byteSize(dtype), dtype)); }
    if (!db) { auto h = b->onCPU(); db = std::static_pointer_cast<CUDAData>(collection(h.data(), h.size() / byteSize(dtype), dtype)); }
    const size_t eb = byteSize(dtype);
    if (da->byteCount() < (size_t)(matrixCount * rows * inner) * eb || db->byteCount() < (size_t)(matrixCount * inner * cols) * eb)
      throw std::invalid_argument("matmul: operand smaller than its stated shape");
    auto out = std::make_shared<CUDAData>(ctx_, (size_t)(matrixCount * rows * cols) * eb);
    check(hc_batched_matmul(ctx_, dtype == DType::float16 ? HC_F16 : HC_F32, matrixCount, da->pointer(), transA,
                            db->pointer(), transB, transOut, rows, inner, cols, out->pointer()));
    out->mark();
    out->keep(da, db);
    return out;
  }

  std::shared_ptr<TensorData> constant(float value, size_t count, DType dtype) override {
    auto out = std::make_shared<CUDAData>(ctx_, count * byteSize(dtype));
    check(hc_constant(ctx_, hcType(dtype, "constant"), value, (int64_t)count, out->pointer()));
    out->mark();
    return out;
  }

  std::shared_ptr<TensorData> cast(const std::shared_ptr<TensorData>& a, size_t count, DType inType,
                                   DType outType) override {
    const hc_dtype from = hcType(inType, "cast"), to = hcType(outType, "cast");
    auto da = onDevice(a, count, inType);
    auto out = std::make_shared<CUDAData>(ctx_, count * byteSize(outType));
    check(hc_cast(ctx_, from, to, da->pointer(), (int64_t)count, out->pointer()));
    out->mark();
    out->keep(da);
    return out;
  }

  std::shared_ptr<TensorData> add(const std::shared_ptr<TensorData>& a, const std::shared_ptr<TensorData>& b, size_t count,
                                  DType dtype) override {
    const hc_dtype dt = hcType(dtype, "add");
    auto da = onDevice(a, count, dtype), db = onDevice(b, count, dtype);
    auto out = std::make_shared<CUDAData>(ctx_, count * byteSize(dtype));
    check(hc_add(ctx_, dt, da->pointer(), db->pointer(), (int64_t)count, out->pointer()));
    out->mark();
    out->keep(da, db);
    return out;
  }

  std::shared_ptr<TensorData> columnSum(const std::shared_ptr<TensorData>& a, int64_t rows, int64_t cols,
                                        DType dtype) override {
    const hc_dtype dt = hcType(dtype, "columnSum");
    auto da = onDevice(a, (size_t)(rows * cols), dtype);
    auto out = std::make_shared<CUDAData>(ctx_, (size_t)cols * byteSize(dtype));
    check(hc_column_sum(ctx_, dt, da->pointer(), rows, cols, out->pointer()));
    out->mark();
    out->keep(da);
    return out;
  }

  std::shared_ptr<TensorData> transpose(const std::shared_ptr<TensorData>& a, int64_t matrixCount, int64_t rows,
                                        int64_t cols, DType dtype) override {
    const hc_dtype dt = hcType(dtype, "transpose");
    auto da = onDevice(a, (size_t)(matrixCount * rows * cols), dtype);
    auto out = std::make_shared<CUDAData>(ctx_, (size_t)(matrixCount * rows * cols) * byteSize(dtype));
    check(hc_transpose(ctx_, dt, matrixCount, da->pointer(), rows, cols, out->pointer()));
    out->mark();
    out->keep(da);
    return out;
  }

  std::shared_ptr<TensorData> linear(const std::shared_ptr<TensorData>& x, const std::shared_ptr<TensorData>& weight,
                                     const std::shared_ptr<TensorData>& bias, int64_t rows, int64_t inCount,
                                     int64_t outCount, DType dtype) override {
    const hc_dtype dt = hcType(dtype, "linear");
    auto dx = onDevice(x, (size_t)(rows * inCount), dtype), dw = onDevice(weight, (size_t)(inCount * outCount), dtype);
    std::shared_ptr<CUDAData> db = bias ? onDevice(bias, (size_t)outCount, dtype) : nullptr;
    auto out = std::make_shared<CUDAData>(ctx_, (size_t)(rows * outCount) * byteSize(dtype));
    check(hc_linear_forward(ctx_, dt, dx->pointer(), dw->pointer(), db ? db->pointer() : nullptr, rows, inCount, outCount,
                            out->pointer()));
    out->mark();
    out->keep(dx, dw, db);
    return out;
  }

  hc_ctx* context() const { return ctx_; }

 private:
  static hc_dtype hcType(DType t, const char* op) {
    if (t == DType::float16) return HC_F16;
    if (t == DType::float32) return HC_F32;
    throw BackendError::notImplemented(std::string(op) + " for int64");
  }
  /// The operand as a buffer of this backend holding at least `count` elements; another backend's
  /// data is staged through onCPU (Sources/Honeycrisp/BackendMPS.swift:585-620).
  std::shared_ptr<CUDAData> onDevice(const std::shared_ptr<TensorData>& a, size_t count, DType dtype) {
    auto d = std::dynamic_pointer_cast<CUDAData>(a);
    if (!d) {
      auto h = a->onCPU();
      d = std::static_pointer_cast<CUDAData>(collection(h.data(), h.size() / byteSize(dtype), dtype));
    }
    if (d->byteCount() < count * byteSize(dtype)) throw std::invalid_argument("operand smaller than its stated shape");
    return d;
  }
  void check(hc_status st) {
    if (st == HC_OK) return;
    const std::string msg = hc_last_error(ctx_);
    if (st == HC_ERR_ALLOCATION_FAILED) throw BackendError(BackendError::Kind::allocationFailed, msg);
    if (st == HC_ERR_NOT_IMPLEMENTED) throw BackendError(BackendError::Kind::notImplemented, msg);
    if (st == HC_ERR_INVALID_ARGUMENT) throw std::invalid_argument(msg);
    throw BackendError(BackendError::Kind::kernelFailed, msg.empty() ? hc_status_string(st) : msg);
  }
  hc_ctx* ctx_ = nullptr;
};

}  // namespace honeycrisp
#endif  // HC_CUDA_HPP_
