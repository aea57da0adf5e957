// Operator schemas of the attention path, registered through LibTorch's stable ABI, and the
// empty Python module that lets `from . import _C` load this shared object.
//
// Same mechanism as the reference's registration unit
// (src/minfer/kernels/torch_ext/csrc/reg.cpp:7-33 of dsuarez01/minfer-python): STABLE_TORCH_LIBRARY
// with one m.def per schema string, PyInit__C returning a module without methods.  The schema of
// flash_attn is the reference's, character for character (reg.cpp:30), and so are il_rope / neox_rope
// (reg.cpp:25-26); the other ops are this package's additions.  The CUDA implementations are
// bound in reg_cuda.cpp; ops that have none there receive theirs from Python (ops.py).
#include <Python.h>

#include <torch/csrc/stable/library.h>

extern "C" {
PyObject* PyInit__C(void) {
  static struct PyModuleDef module_def = {
      PyModuleDef_HEAD_INIT, "_C", NULL, -1, NULL,
  };
  return PyModule_Create(&module_def);
}
}

namespace minfer {

STABLE_TORCH_LIBRARY(minfer, m) {
  m.def("flash_attn(int qtype_int, int qblock_size, int qtype_size, Tensor q, Tensor k, Tensor v, Tensor(a!) mask, Tensor(a!) out) -> ()");
  m.def("il_rope(int rotary_dim, int start_pos, float freq_base, Tensor(a!) x) -> ()");
  m.def("neox_rope(int rotary_dim, int start_pos, float freq_base, Tensor(a!) x) -> ()");
  m.def("flash_attn_causal(Tensor q, Tensor k, Tensor v, Tensor(a!) out) -> ()");
  m.def("flash_attn_decode(Tensor q, Tensor k_cache, Tensor v_cache, Tensor lens, Tensor(a!) out) -> ()");
  m.def("flash_attn_decode_q8(Tensor q, Tensor k_cache, Tensor v_cache, Tensor lens, Tensor(a!) out) -> ()");
  m.def("flash_attn_decode_paged(Tensor q, Tensor k_pages, Tensor v_pages, Tensor block_table, Tensor lens, Tensor(a!) out) -> ()");
  m.def("rope_kv_append(int rotary_dim, float freq_base, int style, Tensor(a!) q, Tensor k, Tensor v, Tensor(a!) k_cache, Tensor(a!) v_cache, Tensor start) -> ()");
  m.def("rope_kv_append_q8(int rotary_dim, float freq_base, int style, Tensor(a!) q, Tensor k, Tensor v, Tensor(a!) k_cache, Tensor(a!) v_cache, Tensor start) -> ()");
  m.def("rope_kv_append_paged(int rotary_dim, float freq_base, int style, Tensor(a!) q, Tensor k, Tensor v, Tensor(a!) k_pages, Tensor(a!) v_pages, Tensor block_table, Tensor start) -> ()");
  // housekeeping of this binding: the device's status word, and the grid limit of later prefill calls
  m.def("attn_status_word(Tensor like) -> Tensor");
  m.def("attn_set_prefill_cta_limit(Tensor like, int max_ctas) -> ()");
}

}  // namespace minfer
