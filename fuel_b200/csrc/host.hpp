// Host-side mirror of the reference's quantized-tensor interface, above the C ABI.
//
// The reference is Rust; where no Rust toolchain is available this C++ layer plays the part
// of its storage and module types so that callers (and the tests) read like the reference's:
//   QStorage  <-> QCudaStorage / DynQuantizedStorage   fuel-cuda-backend/src/quantized.rs:306-609,
//                                                      fuel-backend-contract/src/quantized.rs:29-103
//   QTensor   <-> QTensor { storage, shape }           (the eager facade the reference removed,
//   QMatMul   <-> QMatMul::from_qtensor / forward       fuel-core/src/quantized/mod.rs:14-24; its
//                                                       forward is DynQuantizedStorage::fwd)
// Same names, same argument meaning, same error behaviour (every failure is an exception
// carrying the FFI status code; nothing aborts). Device memory is owned here with
// cudaMalloc/cudaFree, as the reference's storage owns its buffers; the kernels underneath
// never allocate.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace fuelq {

// fuel-ir/src/quantized.rs:16-104
enum class GgmlDType : int32_t {
  F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9, Q2K = 10, Q3K = 11, Q4K = 12, Q5K = 13, Q6K = 14,
  Q8K = 15, BF16 = 30
};
size_t type_size(GgmlDType t);
size_t block_size(GgmlDType t);

class Error : public std::runtime_error {
 public:
  Error(const std::string& what, int32_t status) : std::runtime_error(what), status_(status) {}
  int32_t status() const { return status_; }

 private:
  int32_t status_;
};

// message of the calling thread's last failure, as fuelq_last_error() returns it
void set_last_error(const std::string& message);

using Shape = std::vector<int64_t>;
int64_t elem_count(const Shape& s);

// One device + the single stream its work is ordered on (fuel-cuda-backend/src/device.rs:172-190).
class Device {
 public:
  explicit Device(int ordinal, void* stream = nullptr) : ordinal_(ordinal), stream_(stream) {}
  int ordinal() const { return ordinal_; }
  void* stream() const { return stream_; }
  void make_current() const;
  void synchronize() const;

 private:
  int ordinal_;
  void* stream_;
};

// Owning device allocation.
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  DeviceBuffer(const Device& dev, size_t bytes, bool zero);
  ~DeviceBuffer();
  DeviceBuffer(DeviceBuffer&& o) noexcept;
  DeviceBuffer& operator=(DeviceBuffer&& o) noexcept;
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  void* ptr() const { return ptr_; }
  size_t bytes() const { return bytes_; }

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
  int ordinal_ = 0;
};

class QStorage {
 public:
  // QCudaStorage::zeros, fuel-cuda-backend/src/quantized.rs:307-320
  static QStorage zeros(const Device& dev, size_t el_count, GgmlDType dtype);
  // load_quantized_bytes, quantized.rs:593-609 (pre-quantized GGUF block bytes from the host)
  static QStorage load_quantized(const Device& dev, GgmlDType dtype, const void* host_bytes, size_t len);

  GgmlDType dtype() const { return dtype_; }
  size_t block_size() const { return fuelq::block_size(dtype_); }
  size_t storage_size_in_bytes() const { return len_; }
  const Device& device() const { return dev_; }

  // quantize: device-resident f32 source (quantized.rs:414-420; done on the device here)
  void quantize(const float* device_src, size_t el_count);
  // quantize_onto: host f32 source (quantized.rs:444-446)
  void quantize_onto(const float* host_src, size_t el_count);
  // importance-matrix variants are outside this library
  void quantize_imatrix(const float*, size_t, const float*, size_t);

  // dequantize / dequantize_f16, quantized.rs:330-385. Returns f32 (or f16) device memory.
  DeviceBuffer dequantize(size_t elem_count) const;
  DeviceBuffer dequantize_f16(size_t elem_count) const;

  // data(): the original block bytes back on the host (quantized.rs:475-480)
  std::vector<uint8_t> data() const;
  const uint8_t* device_ptr() const { return static_cast<const uint8_t*>(buf_.ptr()); }

  // fwd: QMatMul forward, quantized.rs:452-473. self_shape = [n, k]; input is contiguous f32 on the
  // device with rank >= 2 and last dim k; the result has the input's shape with k replaced by n.
  std::pair<DeviceBuffer, Shape> fwd(const Shape& self_shape, const float* device_input, const Shape& input_shape) const;
  // same, into caller-owned output (what a graph executor with pre-allocated outputs calls)
  void fwd_into(const Shape& self_shape, const float* device_input, const Shape& input_shape, float* device_out) const;

 private:
  QStorage(const Device& dev, GgmlDType dtype, size_t len) : dev_(dev), dtype_(dtype), len_(len) {}
  void ensure_workspace(size_t bytes) const;
  Device dev_;
  GgmlDType dtype_;
  size_t len_ = 0;
  DeviceBuffer buf_;
  mutable DeviceBuffer workspace_;  // activation blocks for fwd; grown on demand, reused across calls
};

class QTensor {
 public:
  QTensor(QStorage storage, Shape shape);
  // QTensor::quantize: host f32 [.., k] -> blocks (last dim must be a multiple of the block size)
  static QTensor quantize(const Device& dev, const float* host_src, const Shape& shape, GgmlDType dtype);
  GgmlDType dtype() const { return storage_.dtype(); }
  const Shape& shape() const { return shape_; }
  size_t rank() const { return shape_.size(); }
  size_t storage_size_in_bytes() const { return storage_.storage_size_in_bytes(); }
  DeviceBuffer dequantize() const { return storage_.dequantize((size_t)elem_count(shape_)); }
  DeviceBuffer dequantize_f16() const { return storage_.dequantize_f16((size_t)elem_count(shape_)); }
  std::vector<uint8_t> data() const { return storage_.data(); }
  const QStorage& storage() const { return storage_; }

 private:
  QStorage storage_;
  Shape shape_;
};

// Module: forward(xs) = xs . W^T
class QMatMul {
 public:
  static QMatMul from_qtensor(std::shared_ptr<QTensor> w) { return QMatMul(std::move(w)); }
  std::pair<DeviceBuffer, Shape> forward(const float* device_xs, const Shape& xs_shape) const;
  void forward_into(const float* device_xs, const Shape& xs_shape, float* device_out) const;
  // host in / host out convenience (synchronizes)
  std::vector<float> forward_host(const float* host_xs, const Shape& xs_shape) const;
  const QTensor& weight() const { return *w_; }

 private:
  explicit QMatMul(std::shared_ptr<QTensor> w) : w_(std::move(w)) {}
  std::shared_ptr<QTensor> w_;
};

}  // namespace fuelq
