// Intentionally empty: stands in for the HIP-only rocWMMA internal header of the same name
// so that the reference's CPU-only test/reference_impl.hpp can be compiled with g++.
// The few declarations that header needs are provided by oracle/ref_shim/ref_wrap.cpp.
