// Implementation of the host-side mirror (host.hpp) and the handle-based C entry points that
// language bindings use to reach it. Everything numeric goes through the kernel-level C ABI.
#include "host.hpp"

#include <cuda_runtime.h>

#include <cstddef>
#include <cstring>

#include "../../include/fuelq.h"
#include "../../include/fuelq_seam.h"

namespace fuelq {

namespace {
void check(int32_t status, const char* op) {
  if (status != FUELQ_OK) throw Error(std::string(op) + ": " + fuelq_status_string(status), status);
}
void cuda_check(cudaError_t e, const char* op) {
  if (e != cudaSuccess) throw Error(std::string(op) + ": " + cudaGetErrorString(e), FUELQ_LAUNCH_FAILURE);
}
cudaStream_t cs(const Device& d) { return static_cast<cudaStream_t>(d.stream()); }
}  // namespace

size_t type_size(GgmlDType t) {
  switch (t) {
    case GgmlDType::F32: return 4;
    case GgmlDType::F16: case GgmlDType::BF16: return 2;
    default: {
      const int b = fuelq_block_bytes((int32_t)t);
      if (!b) throw Error("unknown dtype", FUELQ_NOT_SUPPORTED);
      return (size_t)b;
    }
  }
}
size_t block_size(GgmlDType t) {
  switch (t) {
    case GgmlDType::F32: case GgmlDType::F16: case GgmlDType::BF16: return 1;
    default: {
      const int b = fuelq_block_elems((int32_t)t);
      if (!b) throw Error("unknown dtype", FUELQ_NOT_SUPPORTED);
      return (size_t)b;
    }
  }
}
int64_t elem_count(const Shape& s) {
  int64_t n = 1;
  for (int64_t d : s) n *= d;
  return n;
}

void Device::make_current() const { cuda_check(cudaSetDevice(ordinal_), "cudaSetDevice"); }
void Device::synchronize() const {
  make_current();
  cuda_check(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)), "cudaStreamSynchronize");
}

DeviceBuffer::DeviceBuffer(const Device& dev, size_t bytes, bool zero) : bytes_(bytes), ordinal_(dev.ordinal()) {
  dev.make_current();
  cuda_check(cudaMalloc(&ptr_, bytes ? bytes : 16), "cudaMalloc");
  if (zero && bytes) cuda_check(cudaMemsetAsync(ptr_, 0, bytes, static_cast<cudaStream_t>(dev.stream())), "cudaMemset");
}
DeviceBuffer::~DeviceBuffer() {
  if (ptr_) {
    cudaSetDevice(ordinal_);
    cudaFree(ptr_);
  }
}
DeviceBuffer::DeviceBuffer(DeviceBuffer&& o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_), ordinal_(o.ordinal_) {
  o.ptr_ = nullptr;
  o.bytes_ = 0;
}
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& o) noexcept {
  if (this != &o) {
    if (ptr_) {
      cudaSetDevice(ordinal_);
      cudaFree(ptr_);
    }
    ptr_ = o.ptr_, bytes_ = o.bytes_, ordinal_ = o.ordinal_;
    o.ptr_ = nullptr, o.bytes_ = 0;
  }
  return *this;
}

// ---------------------------------------------------------------- QStorage
QStorage QStorage::zeros(const Device& dev, size_t el_count, GgmlDType dtype) {
  const size_t bs = fuelq::block_size(dtype);
  const size_t len = (el_count + bs - 1) / bs * type_size(dtype);
  QStorage s(dev, dtype, len);
  s.buf_ = DeviceBuffer(dev, len, true);
  return s;
}

QStorage QStorage::load_quantized(const Device& dev, GgmlDType dtype, const void* host_bytes, size_t len) {
  if (len % type_size(dtype)) throw Error("load_quantized: byte length is not a multiple of the block size", FUELQ_INVALID_PROBLEM);
  QStorage s(dev, dtype, len);
  s.buf_ = DeviceBuffer(dev, len, false);
  if (len) cuda_check(cudaMemcpyAsync(s.buf_.ptr(), host_bytes, len, cudaMemcpyHostToDevice, cs(dev)), "cudaMemcpyAsync");
  dev.synchronize();  // the host buffer may go away as soon as we return
  return s;
}

void QStorage::quantize(const float* device_src, size_t el_count) {
  dev_.make_current();
  const size_t bs = fuelq::block_size(dtype_);
  if (el_count % bs) throw Error("quantize: element count is not a multiple of the block size", FUELQ_INVALID_PROBLEM);
  const size_t len = el_count / bs * type_size(dtype_);
  if (len != len_) {
    buf_ = DeviceBuffer(dev_, len, false);
    len_ = len;
  }
  check(fuelq_quantize_weights((int32_t)dtype_, (int64_t)el_count, device_src, buf_.ptr(), dev_.stream()),
        "fuelq_quantize_weights");
}

void QStorage::quantize_onto(const float* host_src, size_t el_count) {
  dev_.make_current();
  DeviceBuffer tmp(dev_, el_count * sizeof(float), false);
  cuda_check(cudaMemcpyAsync(tmp.ptr(), host_src, el_count * sizeof(float), cudaMemcpyHostToDevice, cs(dev_)),
             "cudaMemcpyAsync");
  quantize(static_cast<const float*>(tmp.ptr()), el_count);
  dev_.synchronize();  // tmp is released on return
}

void QStorage::quantize_imatrix(const float*, size_t, const float*, size_t) {
  throw Error("quantize_imatrix is not supported on this backend", FUELQ_NOT_SUPPORTED);
}

DeviceBuffer QStorage::dequantize(size_t n) const {
  dev_.make_current();
  DeviceBuffer out(dev_, n * sizeof(float), false);
  check(fuelq_dequantize((int32_t)dtype_, (int64_t)n, buf_.ptr(), out.ptr(), FUELQ_TYPE_F32, dev_.stream()), "fuelq_dequantize");
  return out;
}
DeviceBuffer QStorage::dequantize_f16(size_t n) const {
  dev_.make_current();
  DeviceBuffer out(dev_, n * 2, false);
  check(fuelq_dequantize((int32_t)dtype_, (int64_t)n, buf_.ptr(), out.ptr(), FUELQ_TYPE_F16, dev_.stream()), "fuelq_dequantize");
  return out;
}

std::vector<uint8_t> QStorage::data() const {
  std::vector<uint8_t> out(len_);
  dev_.make_current();
  if (len_) cuda_check(cudaMemcpyAsync(out.data(), buf_.ptr(), len_, cudaMemcpyDeviceToHost, cs(dev_)), "cudaMemcpyAsync");
  dev_.synchronize();
  return out;
}

void QStorage::ensure_workspace(size_t bytes) const {
  if (workspace_.bytes() < bytes) {
    dev_.synchronize();  // an earlier call may still be reading the old one
    workspace_ = DeviceBuffer(dev_, bytes, false);
  }
}

void QStorage::fwd_into(const Shape& self_shape, const float* x, const Shape& in_shape, float* y) const {
  if (self_shape.size() != 2) throw Error("qmatmul: weight shape must be [n, k]", FUELQ_INVALID_PROBLEM);
  const int64_t n = self_shape[0], k = self_shape[1];
  if (in_shape.size() < 2) throw Error("input tensor has only one dimension", FUELQ_INVALID_PROBLEM);
  if (in_shape.back() != k) throw Error("input tensor incompatible with the weight shape", FUELQ_INVALID_PROBLEM);
  const int64_t m = elem_count(in_shape) / (k ? k : 1);
  dev_.make_current();
  const size_t need = fuelq_qmatmul_workspace_bytes((int32_t)dtype_, m, n, k);
  ensure_workspace(need ? need : 16);
  check(fuelq_qmatmul((int32_t)dtype_, m, n, k, buf_.ptr(), x, y, workspace_.ptr(), workspace_.bytes(), dev_.stream()),
        "fuelq_qmatmul");
}

std::pair<DeviceBuffer, Shape> QStorage::fwd(const Shape& self_shape, const float* x, const Shape& in_shape) const {
  if (self_shape.size() != 2 || in_shape.size() < 2 || in_shape.back() != self_shape[1])
    throw Error("input tensor incompatible with the weight shape", FUELQ_INVALID_PROBLEM);
  Shape out_shape(in_shape);
  out_shape.back() = self_shape[0];
  DeviceBuffer out(dev_, (size_t)elem_count(out_shape) * sizeof(float), false);
  fwd_into(self_shape, x, in_shape, static_cast<float*>(out.ptr()));
  return {std::move(out), out_shape};
}

// ---------------------------------------------------------------- QTensor / QMatMul
QTensor::QTensor(QStorage storage, Shape shape) : storage_(std::move(storage)), shape_(std::move(shape)) {
  if (shape_.empty()) throw Error("QTensor: empty shape", FUELQ_INVALID_PROBLEM);
  const size_t bs = storage_.block_size();
  if ((size_t)shape_.back() % bs) throw Error("QTensor: last dimension is not a multiple of the block size", FUELQ_INVALID_PROBLEM);
  if ((size_t)elem_count(shape_) / bs * type_size(storage_.dtype()) != storage_.storage_size_in_bytes())
    throw Error("QTensor: storage size does not match the shape", FUELQ_INVALID_PROBLEM);
}

QTensor QTensor::quantize(const Device& dev, const float* host_src, const Shape& shape, GgmlDType dtype) {
  if (shape.empty() || (size_t)shape.back() % fuelq::block_size(dtype))
    throw Error("quantize: last dimension is not a multiple of the block size", FUELQ_INVALID_PROBLEM);
  QStorage s = QStorage::zeros(dev, (size_t)elem_count(shape), dtype);
  s.quantize_onto(host_src, (size_t)elem_count(shape));
  return QTensor(std::move(s), shape);
}

void QMatMul::forward_into(const float* xs, const Shape& xs_shape, float* out) const {
  w_->storage().fwd_into(w_->shape(), xs, xs_shape, out);
}
std::pair<DeviceBuffer, Shape> QMatMul::forward(const float* xs, const Shape& xs_shape) const {
  return w_->storage().fwd(w_->shape(), xs, xs_shape);
}
std::vector<float> QMatMul::forward_host(const float* host_xs, const Shape& xs_shape) const {
  const Device& dev = w_->storage().device();
  dev.make_current();
  const size_t nx = (size_t)elem_count(xs_shape);
  DeviceBuffer x(dev, nx * sizeof(float), false);
  cuda_check(cudaMemcpyAsync(x.ptr(), host_xs, nx * sizeof(float), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(dev.stream())),
             "cudaMemcpyAsync");
  auto r = forward(static_cast<const float*>(x.ptr()), xs_shape);
  std::vector<float> out((size_t)elem_count(r.second));
  cuda_check(cudaMemcpyAsync(out.data(), r.first.ptr(), out.size() * sizeof(float), cudaMemcpyDeviceToHost,
                             static_cast<cudaStream_t>(dev.stream())),
             "cudaMemcpyAsync");
  dev.synchronize();
  return out;
}

}  // namespace fuelq

// ---------------------------------------------------------------- handle-based C entry points
using namespace fuelq;

namespace {
thread_local std::string g_last_error;
template <typename F>
int32_t guarded(F&& f) {
  try {
    f();
    return FUELQ_OK;
  } catch (const Error& e) {
    g_last_error = e.what();
    return e.status();
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return FUELQ_LAUNCH_FAILURE;
  }
}
struct QTensorHandle {
  std::shared_ptr<QTensor> t;
};
}  // namespace

void fuelq::set_last_error(const std::string& message) { g_last_error = message; }

static_assert(sizeof(fuelq_seam_hello_t) == 56 && offsetof(fuelq_seam_hello_t, envelope_version) == 4 &&
                  offsetof(fuelq_seam_hello_t, profiles_len) == 8 && offsetof(fuelq_seam_hello_t, profiles) == 10 &&
                  offsetof(fuelq_seam_hello_t, reserved1) == 42 && offsetof(fuelq_seam_hello_t, capabilities) == 48,
              "the handshake envelope is a frozen 56-byte layout");

extern "C" {

int fuelq_seam_hello(fuelq_seam_hello_t* out) {
  if (!out) return 2;
  std::memset(out, 0, sizeof(*out));
  out->magic = FUELQ_SEAM_MAGIC;
  out->envelope_version = FUELQ_SEAM_ENVELOPE_VERSION;
  out->profiles_len = 1;
  out->profiles[0] = FUELQ_SEAM_PROFILE_V1;
  out->capabilities = FUELQ_SEAM_CAP_FDX_V1 | FUELQ_SEAM_CAP_FDX_GGML;
  return 0;
}

const char* fuelq_last_error(void) { return g_last_error.c_str(); }

int32_t fuelq_qtensor_load(int32_t device, void* stream, int32_t ggml_type, int64_t n, int64_t k, const void* host_blocks,
                           size_t len, void** out) {
  return guarded([&] {
    if (!out) throw Error("null output handle", FUELQ_INVALID_PROBLEM);
    Device dev(device, stream);
    QStorage s = QStorage::load_quantized(dev, (GgmlDType)ggml_type, host_blocks, len);
    *out = new QTensorHandle{std::make_shared<QTensor>(std::move(s), Shape{n, k})};
  });
}

int32_t fuelq_qtensor_quantize(int32_t device, void* stream, int32_t ggml_type, int64_t n, int64_t k, const float* src,
                               int32_t src_on_device, void** out) {
  return guarded([&] {
    if (!out) throw Error("null output handle", FUELQ_INVALID_PROBLEM);
    Device dev(device, stream);
    if ((size_t)k % fuelq::block_size((GgmlDType)ggml_type)) throw Error("k is not a multiple of the block size", FUELQ_INVALID_PROBLEM);
    QStorage s = QStorage::zeros(dev, (size_t)(n * k), (GgmlDType)ggml_type);
    if (src_on_device)
      s.quantize(src, (size_t)(n * k));
    else
      s.quantize_onto(src, (size_t)(n * k));
    *out = new QTensorHandle{std::make_shared<QTensor>(std::move(s), Shape{n, k})};
  });
}

int32_t fuelq_qtensor_free(void* h) {
  delete static_cast<QTensorHandle*>(h);
  return FUELQ_OK;
}

int32_t fuelq_qtensor_info(const void* h, int32_t* ggml_type, int64_t* n, int64_t* k, size_t* storage_bytes, const void** device_ptr) {
  return guarded([&] {
    if (!h) throw Error("null handle", FUELQ_INVALID_PROBLEM);
    const QTensor& t = *static_cast<const QTensorHandle*>(h)->t;
    if (ggml_type) *ggml_type = (int32_t)t.dtype();
    if (n) *n = t.shape()[0];
    if (k) *k = t.shape()[1];
    if (storage_bytes) *storage_bytes = t.storage_size_in_bytes();
    if (device_ptr) *device_ptr = t.storage().device_ptr();
  });
}

int32_t fuelq_qtensor_data(const void* h, void* host_out, size_t len) {
  return guarded([&] {
    if (!h || !host_out) throw Error("null argument", FUELQ_INVALID_PROBLEM);
    const std::vector<uint8_t> d = static_cast<const QTensorHandle*>(h)->t->data();
    if (len != d.size()) throw Error("data: output length does not match the storage size", FUELQ_INVALID_PROBLEM);
    std::memcpy(host_out, d.data(), len);
  });
}

int32_t fuelq_qtensor_dequantize(const void* h, void* device_out, int32_t out_type) {
  return guarded([&] {
    if (!h || !device_out) throw Error("null argument", FUELQ_INVALID_PROBLEM);
    const QTensor& t = *static_cast<const QTensorHandle*>(h)->t;
    const Device& dev = t.storage().device();
    dev.make_current();
    check(fuelq_dequantize((int32_t)t.dtype(), elem_count(t.shape()), t.storage().device_ptr(), device_out, out_type,
                           dev.stream()),
          "fuelq_dequantize");
  });
}

int32_t fuelq_qmatmul_forward(const void* h, const float* device_x, int64_t m, float* device_y) {
  return guarded([&] {
    if (!h) throw Error("null handle", FUELQ_INVALID_PROBLEM);
    const QTensor& t = *static_cast<const QTensorHandle*>(h)->t;
    t.storage().fwd_into(t.shape(), device_x, Shape{m, t.shape()[1]}, device_y);
  });
}

int32_t fuelq_qmatmul_forward_host(const void* h, const float* host_x, int64_t m, float* host_y) {
  return guarded([&] {
    if (!h || !host_x || !host_y) throw Error("null argument", FUELQ_INVALID_PROBLEM);
    auto t = static_cast<const QTensorHandle*>(h)->t;
    const std::vector<float> y = QMatMul::from_qtensor(t).forward_host(host_x, Shape{m, t->shape()[1]});
    std::memcpy(host_y, y.data(), y.size() * sizeof(float));
  });
}

}  // extern "C"
