// Buffers that the other ranks of one node can write: the receiving side of the fused
// pooling + exchange step.  A rank allocates its receive buffer here, hands the 64-byte
// handle to its peers (over any host channel), and each peer maps the buffer into its own
// address space.  The mapped pointer is an ordinary device pointer: the bag kernel of a
// row-sharded table is given it as its output and stores its partial sums straight into the
// owner's memory over NVLink, so no separate all-to-all pass reads and rewrites them.
// Plain CUDA IPC: no multicast object is created or bound anywhere.
#include <cuda_runtime.h>

#include <cstring>

#include "common.h"

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size is part of the C ABI");

extern "C" {

int annc_peer_buffer_create(size_t bytes, void** dev_ptr, void* handle64) {
  ANNC_REQUIRE(bytes > 0 && dev_ptr && handle64, ANNC_ERR_INVALID_ARGUMENT, "bad peer buffer request");
  void* p = nullptr;
  ANNC_CUDA(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return annc::cuda_fail(e, "cudaIpcGetMemHandle");
  }
  memcpy(handle64, &h, sizeof(h));
  *dev_ptr = p;
  return ANNC_OK;
}

int annc_peer_buffer_open(const void* handle64, void** dev_ptr) {
  ANNC_REQUIRE(handle64 && dev_ptr, ANNC_ERR_INVALID_ARGUMENT, "bad peer handle");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  ANNC_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *dev_ptr = p;
  return ANNC_OK;
}

int annc_peer_copy_dev(void* dst, const void* src, size_t bytes, void* stream) {
  if (bytes == 0) return ANNC_OK;
  ANNC_REQUIRE(dst && src, ANNC_ERR_INVALID_ARGUMENT, "null copy argument");
  ANNC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
  return ANNC_OK;
}

int annc_peer_buffer_close(void* dev_ptr) {
  if (dev_ptr) ANNC_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  return ANNC_OK;
}

int annc_peer_buffer_destroy(void* dev_ptr) {
  if (dev_ptr) ANNC_CUDA(cudaFree(dev_ptr));
  return ANNC_OK;
}

}  // extern "C"
