// C entry points around the REFERENCE's own Q8_0 codec, so the Python oracle can call it through
// ctypes.  This file only declares the reference's functions (minfer::impl::quant_row_q8_0 and
// dequant_row_q8_0<T>, src/minfer/kernels/torch_ext/csrc/quants/impl.cpp:1153-1193) and forwards to
// them; the implementation is compiled from the reference tree where it lies (see Makefile).
// Test infrastructure only.
#include <cstdint>

#include "common/types.hpp"  // the reference's header: half_t, block_q8_0

namespace minfer::impl {
void quant_row_q8_0(const float* __restrict__ x, uint8_t* __restrict__ yr, int64_t k);
template <typename T>
void dequant_row_q8_0(const uint8_t* __restrict__ xr, T* __restrict__ y, int64_t k);
}  // namespace minfer::impl

extern "C" {
void ref_quant_row_q8_0(const float* x, uint8_t* y, int64_t k) { minfer::impl::quant_row_q8_0(x, y, k); }
void ref_dequant_row_q8_0_f32(const uint8_t* x, float* y, int64_t k) { minfer::impl::dequant_row_q8_0<float>(x, y, k); }
void ref_dequant_row_q8_0_f16(const uint8_t* x, void* y, int64_t k) {
  minfer::impl::dequant_row_q8_0<half_t>(x, static_cast<half_t*>(y), k);
}
}
