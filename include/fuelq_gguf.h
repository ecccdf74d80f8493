/* fuelq — GGUF container reader: the file format quantized checkpoints arrive in, so that Q4_K / Q6_K / Q8_0
 * tensors go from the file mapping straight into device buffers, unchanged.
 *
 * Replaces, for this path, the reference's header parser `Content::read` (fuel-formats/src/gguf.rs:385-462:
 * magic "GGUF" in either byte order of the tag, versions 1-3 — v1 counts and string lengths are u32, v2/v3 u64 —,
 * the key/value metadata table, the tensor-info table with each dimension list REVERSED on read (:431), and the
 * start of the tensor data rounded up to `general.alignment`, default 32, :443-453) and the mapped-file tensor
 * slicing of the model loaders (fuel-core/src/lazy_quantized_llama.rs:251-260: bytes
 * [data_offset + offset, + elem_count / block_size * type_size)).
 *
 * Status codes as in fuelq.h (2 = the file is not a readable GGUF file, 3 = valid but not supported);
 * fuelq_last_error() (fuelq_host.h) holds the message, worded like the reference's where it has one.
 * Every pointer handed out points into memory owned by the handle and dies with fuelq_gguf_close.
 */
#ifndef FUELQ_GGUF_H_
#define FUELQ_GGUF_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fuelq_gguf fuelq_gguf;

/* metadata value types (gguf.rs:93-160) */
#define FUELQ_GGUF_U8 0
#define FUELQ_GGUF_I8 1
#define FUELQ_GGUF_U16 2
#define FUELQ_GGUF_I16 3
#define FUELQ_GGUF_U32 4
#define FUELQ_GGUF_I32 5
#define FUELQ_GGUF_F32 6
#define FUELQ_GGUF_BOOL 7
#define FUELQ_GGUF_STRING 8
#define FUELQ_GGUF_ARRAY 9
#define FUELQ_GGUF_U64 10
#define FUELQ_GGUF_I64 11
#define FUELQ_GGUF_F64 12

/* TensorInfo (gguf.rs:62-66) plus where its bytes are. */
typedef struct {
  const char* name;   /* NUL-terminated */
  int32_t ggml_type;  /* on-disk id (GgmlDType::from_u32, fuel-ir/src/quantized.rs:35-56) */
  int32_t n_dims;     /* at most 8 */
  int64_t dims[8];    /* outermost first, i.e. the file's order reversed: a linear weight reads [n_out, k_in] */
  uint64_t offset;    /* from the start of the tensor data */
  uint64_t nbytes;    /* elem_count / block_size * type_size */
  const void* data;   /* the bytes, inside the mapping */
} fuelq_gguf_tensor;

/* One metadata value. Integers (and bool) in `i` (u64 values as their bit pattern), floats in `f`, a string in
 * `s`/`len` (not NUL-terminated; trailing NULs of the file already dropped, gguf.rs:78-81). An array reports its
 * element type and count; `array` points at its packed little-endian elements when they are fixed-size scalars
 * (possibly unaligned), and is null for arrays of strings (fuelq_gguf_meta_array_string) or of arrays. */
typedef struct {
  const char* key; /* NUL-terminated */
  int32_t type;
  int32_t elem_type;
  uint64_t len;
  int64_t i;
  double f;
  const char* s;
  const void* array;
} fuelq_gguf_value;

/* Map `path` read-only and parse its header. */
int32_t fuelq_gguf_open(const char* path, fuelq_gguf** out);
/* Parse a file image the caller keeps alive until close (no copy is made). */
int32_t fuelq_gguf_open_memory(const void* bytes, size_t len, fuelq_gguf** out);
int32_t fuelq_gguf_close(fuelq_gguf* g);

int32_t fuelq_gguf_version(const fuelq_gguf* g);               /* 1, 2 or 3 */
uint64_t fuelq_gguf_alignment(const fuelq_gguf* g);            /* general.alignment, else 32 */
uint64_t fuelq_gguf_tensor_data_offset(const fuelq_gguf* g);   /* Content::tensor_data_offset */

int64_t fuelq_gguf_tensor_count(const fuelq_gguf* g);          /* distinct names; a repeated name keeps its last entry */
int64_t fuelq_gguf_find_tensor(const fuelq_gguf* g, const char* name); /* index, or -1 */
int32_t fuelq_gguf_tensor_at(const fuelq_gguf* g, int64_t index, fuelq_gguf_tensor* out);

int64_t fuelq_gguf_meta_count(const fuelq_gguf* g);
int64_t fuelq_gguf_find_meta(const fuelq_gguf* g, const char* key); /* index, or -1 */
int32_t fuelq_gguf_meta_at(const fuelq_gguf* g, int64_t index, fuelq_gguf_value* out);
int32_t fuelq_gguf_meta_array_string(const fuelq_gguf* g, int64_t index, uint64_t elem, const char** s, uint64_t* len);

/* Enqueue the copy of bytes [byte_offset, byte_offset + nbytes) of tensor `index` to device memory (whole weight
 * rows are contiguous in the file, so a tensor-parallel rank loads just its rows). The mapping must stay open
 * until the stream has passed the copy. */
int32_t fuelq_gguf_load_tensor(const fuelq_gguf* g, int64_t index, uint64_t byte_offset, uint64_t nbytes, void* device_dst,
                               void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FUELQ_GGUF_H_ */
