/* fuelq — object-level C entry points over the host-side mirror of the reference's quantized
 * tensor types (fuel_b200/csrc/host.hpp). These are what a language binding holds on to: an
 * opaque handle to a weight tensor living on the device, and QMatMul::forward on it.
 * Status codes as in fuelq.h; fuelq_last_error() returns the message of the calling thread's
 * last failure. Unlike the kernel-level entry points in fuelq.h these own device memory
 * (the weight blocks and a reusable activation workspace), like the reference's storage types.
 */
#ifndef FUELQ_HOST_H_
#define FUELQ_HOST_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* fuelq_last_error(void);

/* QuantizedDeviceKernels::load_quantized (fuel-backend-contract/src/quantized.rs:112-119;
 * fuel-cuda-backend/src/quantized.rs:593-609): GGUF block bytes on the host -> a [n, k] weight on
 * device `device`, ordered on `stream` (a cudaStream_t, may be null). */
int32_t fuelq_qtensor_load(int32_t device, void* stream, int32_t ggml_type, int64_t n, int64_t k,
                           const void* host_blocks, size_t len, void** out_handle);

/* qzeros + quantize / quantize_onto (fuel-backend-contract/src/quantized.rs:34-35,45-46,108-110;
 * fuel-cuda-backend/src/quantized.rs:414-446): f32 [n, k] from the device (src_on_device != 0) or the
 * host -> blocks, byte-identical to the reference's quantizer. */
int32_t fuelq_qtensor_quantize(int32_t device, void* stream, int32_t ggml_type, int64_t n, int64_t k,
                               const float* src, int32_t src_on_device, void** out_handle);

int32_t fuelq_qtensor_free(void* handle);

/* dtype / shape / storage_size_in_bytes / device_ptr (fuel-backend-contract/src/quantized.rs:30-32,67-70). */
int32_t fuelq_qtensor_info(const void* handle, int32_t* ggml_type, int64_t* n, int64_t* k, size_t* storage_bytes,
                           const void** device_ptr);

/* data(): the original block bytes (fuel-backend-contract/src/quantized.rs:64-65). len must equal the storage size. */
int32_t fuelq_qtensor_data(const void* handle, void* host_out, size_t len);

/* dequantize / dequantize_f16 (quantized.rs:56-62) into caller-owned device memory; out_type as in fuelq_dequantize. */
int32_t fuelq_qtensor_dequantize(const void* handle, void* device_out, int32_t out_type);

/* QMatMul::forward == DynQuantizedStorage::fwd (fuel-backend-contract/src/quantized.rs:72-80):
 * y[m, n] = x[m, k] . W^T, device f32 in and out, enqueued on the tensor's stream. */
int32_t fuelq_qmatmul_forward(const void* handle, const float* device_x, int64_t m, float* device_y);

/* The same with host buffers; copies in, runs, copies out and synchronizes. */
int32_t fuelq_qmatmul_forward_host(const void* handle, const float* host_x, int64_t m, float* host_y);

#ifdef __cplusplus
}
#endif
#endif /* FUELQ_HOST_H_ */
