// pybind11 binding used ONLY to pin the CPU oracle against the reference's own CUDA kernels.
// It binds the four all-in-one attention entry points and the KNN entry point that the
// reference declares in Swin3D/src/attn/self_attn_aio_fwd.h:11-26,
// Swin3D/src/attn/self_attn_aio_bwd.h:9-32 and Swin3D/src/knn/knn_cuda_kernel.h:5-12.
// The reference sources are compiled where they lie (see build_ref.py); nothing of them is
// copied into this repository.  Test infrastructure: never imported by the product path.
#include <torch/extension.h>
#include "attn/self_attn_aio_fwd.h"
#include "attn/self_attn_aio_bwd.h"
#include "knn/knn_cuda_kernel.h"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("cal_max_coffs", &cal_max_coffs);
  m.def("self_attn_forward", &self_attn_cuda_forward);
  m.def("cal_exp_sum_grads", &cal_exp_sum_grads);
  m.def("self_attn_indir_backward", &self_attn_cuda_backward);
  m.def("knn_cuda", &knn_cuda);
}
