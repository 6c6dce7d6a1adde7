// Thin harness around the REFERENCE's own page-copy launchers.  TEST INFRASTRUCTURE ONLY.
//
// Compiled by oracle/build_ref.py together with the reference's copy_kernel.cu, taken
// from the reference checkout where it lies (nothing of it is copied into this
// repository).  The reference's Python binding can only reach its kernels through a
// CUDA-IPC channel set up between two processes (producer_init / consumer_init,
// SharedMemory/CUDA_Shared/ipc_service.cpp:20-110); this harness instead hands
// cuda_producer_copy_pages (copy_kernel.cu:68-129) and cuda_producer_zero_copy_pages
// (copy_kernel.cu:133-196) a private control block and a caller-provided output tensor
// as the "shared" buffer, so that one process can run the reference kernel on chosen
// inputs and read its output.
#include "ipc_wrapper.h"

#include <cstring>

namespace {

struct Control {
  SharedControl ctrl;
  Control(size_t bytes) {
    std::memset(&ctrl, 0, sizeof(ctrl));
    sem_init(&ctrl.sem_start, 0, 0);
    sem_init(&ctrl.sem_complete, 0, 0);
    ctrl.buffer_size = bytes;
    ctrl.current_offset = 0;
  }
  ~Control() {
    sem_destroy(&ctrl.sem_start);
    sem_destroy(&ctrl.sem_complete);
  }
};

TensorDims make_dims(int64_t tokens, int64_t head_size, int64_t kv_heads, int64_t layers, int64_t kv_pair) {
  TensorDims d;
  d.total_tokens = tokens;
  d.head_size = head_size;
  d.num_kv_heads = kv_heads;
  d.num_layers = layers;
  d.kv_pair = kv_pair;
  return d;
}

// Runs the reference gather into `out` (a CUDA tensor at least as large as the
// transfer); returns the 5-D shape the reference records for the consumer.
std::vector<int64_t> ref_copy_pages(torch::Tensor cache, torch::Tensor src_off, torch::Tensor dst_off,
                                    torch::Tensor out, int64_t page_size, int64_t head_size,
                                    int64_t kv_heads, int64_t layers, int64_t kv_pair) {
  Control c(out.nbytes());
  TensorDims dims = make_dims(src_off.size(0) * page_size, head_size, kv_heads, layers, kv_pair);
  cuda_producer_copy_pages(cache, src_off, dst_off, &c.ctrl, out.data_ptr(), (int)page_size, dims);
  return std::vector<int64_t>(c.ctrl.tensor_shape, c.ctrl.tensor_shape + c.ctrl.tensor_dim);
}

std::vector<int64_t> ref_zero_copy_pages(torch::Tensor pinned, torch::Tensor src_off, torch::Tensor dst_off,
                                         torch::Tensor out, int64_t page_size, int64_t head_size,
                                         int64_t kv_heads, int64_t layers, int64_t kv_pair) {
  Control c(out.nbytes());
  TensorDims dims = make_dims(src_off.size(0) * page_size, head_size, kv_heads, layers, kv_pair);
  cuda_producer_zero_copy_pages(pinned, src_off, dst_off, &c.ctrl, out.data_ptr(), (int)page_size, dims);
  return std::vector<int64_t>(c.ctrl.tensor_shape, c.ctrl.tensor_shape + c.ctrl.tensor_dim);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("ref_copy_pages", &ref_copy_pages, "reference block_per_page_copy_kernel via cuda_producer_copy_pages");
  m.def("ref_zero_copy_pages", &ref_zero_copy_pages, "reference zero_copy_page_kernel");
}
