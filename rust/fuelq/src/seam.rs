//! Handshake with the provider before anything is dispatched to it
//! (`docs/specs/kernel-seam-interop.md:95-133`).

use fuel_kernel_seam_announce::{negotiate, Negotiated, SeamError, SeamHello, PROFILE_V1, SEAM_CAP_FDX_GGML, SEAM_CAP_FDX_V1};

/// Asks `libfuelq.so` for its envelope and negotiates it against what this build of fuel speaks.
pub fn negotiate_with_provider() -> Result<Negotiated, SeamError> {
    let mut raw = fuelq_sys::fuelq_seam_hello_t::default();
    let rc = unsafe { fuelq_sys::fuelq_seam_hello(&mut raw) };
    assert_eq!(rc, 0, "fuelq_seam_hello fills a caller-owned struct and cannot fail for a valid pointer");
    // same layout, field for field (both sides assert 56 bytes and the offsets)
    let remote: SeamHello = unsafe { std::mem::transmute(raw) };
    let local = SeamHello::advertise(&[PROFILE_V1], SEAM_CAP_FDX_V1 | SEAM_CAP_FDX_GGML);
    negotiate(&local, &remote)
}
