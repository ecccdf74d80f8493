"""The provider handshake (include/fuelq_seam.h): a fixed 56-byte envelope with frozen offsets, filled through an
out-parameter, validated and negotiated the way fuel does it (fuel-kernel-seam-announce/src/lib.rs:30-90 for the
layout; validation rules :92-130 of the same file's SeamError; negotiation = highest common profile and the AND of
the capability bits, docs/specs/kernel-seam-interop.md:127-133). No device is touched."""
import ctypes
import struct


def _hello():
    from fuel_b200 import _lib
    buf = ctypes.create_string_buffer(b"\xff" * 64, 64)   # garbage first: every byte of the envelope must be written
    assert _lib.lib.fuelq_seam_hello(ctypes.addressof(buf)) == 0
    assert buf.raw[56:] == b"\xff" * 8                    # nothing past 56 bytes is touched
    return buf.raw[:56]


def test_envelope_layout_and_contents():
    raw = _hello()
    assert raw[:4] == b"SEAM"                             # the magic reads as ASCII on the wire
    magic, version, r0, r1, r2, n = struct.unpack_from("<IBBBBH", raw, 0)
    assert magic == 0x4D414553 and version == 1 and (r0, r1, r2) == (0, 0, 0)
    profiles = struct.unpack_from("<16H", raw, 10)
    assert n == 1 and profiles[0] == 1 and not any(profiles[1:])
    assert raw[42:48] == bytes(6)
    (caps,) = struct.unpack_from("<Q", raw, 48)
    assert caps == (1 << 0) | (1 << 2)                    # FDX base sidecar + GGML inline-block operands


def test_envelope_passes_the_consumer_side_checks_and_negotiates():
    raw = _hello()
    magic, version = struct.unpack_from("<IB", raw, 0)
    (n,) = struct.unpack_from("<H", raw, 8)
    profiles = list(struct.unpack_from("<16H", raw, 10))[:n]
    (caps,) = struct.unpack_from("<Q", raw, 48)
    # what the consumer rejects: bad magic, unknown envelope, too many profiles, not strictly ascending, nonzero reserved
    assert magic == 0x4D414553 and version == 1 and n <= 16
    assert all(a < b for a, b in zip(profiles, profiles[1:]))
    assert raw[5:8] == bytes(3) and raw[42:48] == bytes(6)
    # negotiation against a consumer that speaks profiles [1] with every FDX capability and JIT-on-request
    local_profiles, local_caps = [1], 0x3F | (1 << 16)
    common = sorted(set(local_profiles) & set(profiles))
    assert common and common[-1] == 1
    assert caps & local_caps == (1 << 0) | (1 << 2)
    # disjoint profile sets must not negotiate
    assert not (set([2, 3]) & set(profiles))


def test_null_pointer_is_a_status_not_a_crash():
    from fuel_b200 import _lib
    assert _lib.lib.fuelq_seam_hello(None) == 2
