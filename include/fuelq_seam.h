/* fuelq — the provider handshake of fuel's kernel seam.
 *
 * Before fuel dispatches to an external kernel provider it asks the provider which interface profiles it
 * speaks: the provider fills a caller-allocated, fixed 56-byte envelope through an out-parameter entry point
 * `int <provider>_seam_hello(SeamHello* out)` that never allocates and returns 0 on success
 * (docs/specs/kernel-seam-interop.md:95-118; the Rust mirror of the struct is
 * fuel-kernel-seam-announce/src/lib.rs:30-90). fuel then picks the highest profile both sides list and the
 * intersection of the capability bits (kernel-seam-interop.md:127-133).
 *
 * The layout below is that frozen envelope, field for field; offsets are asserted at compile time in
 * fuel_b200/csrc/host.cpp and again in tests/test_seam.py.
 */
#ifndef FUELQ_SEAM_H_
#define FUELQ_SEAM_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FUELQ_SEAM_MAGIC 0x4D414553u      /* little-endian bytes "SEAM" (fuel-kernel-seam-announce/src/lib.rs:31) */
#define FUELQ_SEAM_ENVELOPE_VERSION 1     /* lib.rs:33 */
#define FUELQ_SEAM_MAX_PROFILES 16        /* lib.rs:35 */
#define FUELQ_SEAM_PROFILE_V1 1           /* the bundled FDX + FKC version, lib.rs:39 */
#define FUELQ_SEAM_CAP_FDX_V1 (1ull << 0)    /* base tensor sidecar, lib.rs:47 */
#define FUELQ_SEAM_CAP_FDX_GGML (1ull << 2)  /* GGML inline-block quantized operands, lib.rs:51 */

typedef struct fuelq_seam_hello_t {
  uint32_t magic;                                /* offset 0 */
  uint8_t envelope_version;                      /* 4 */
  uint8_t reserved[3];                           /* 5, zero */
  uint16_t profiles_len;                         /* 8 */
  uint16_t profiles[FUELQ_SEAM_MAX_PROFILES];    /* 10, ascending, unused entries zero */
  uint8_t reserved1[6];                          /* 42, zero */
  uint64_t capabilities;                         /* 48 */
} fuelq_seam_hello_t;                            /* 56 bytes */

/* Fills *out with this library's envelope: profile 1, capabilities FDX_V1 | FDX_GGML (its weight operands are
 * GGML blocks with inline scales and nothing else). Returns 0, or 2 (invalid problem) for a null pointer.
 * Touches no device and allocates nothing. */
int fuelq_seam_hello(fuelq_seam_hello_t* out);

#ifdef __cplusplus
}
#endif
#endif /* FUELQ_SEAM_H_ */
