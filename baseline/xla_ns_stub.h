// Force-included when building the reference's launch shim without jaxlib headers: its
// Torch-only build (-DPYPTX_NO_XLA_FFI) still names `xla::ffi` once in a namespace alias
// (pyptx/_shim/pyptx_launch.cc:197), so the empty namespaces have to exist.
namespace xla { namespace ffi {} }
