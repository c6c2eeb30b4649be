// Peer mapping of one device buffer per rank through CUDA IPC memory handles.
//
// Each rank allocates its symmetric buffer with cudaMalloc, exports a 64-byte handle that the ranks
// exchange as plain bytes over the process group, and opens every peer's handle; the returned
// pointers address the peers' buffers over NVLink and are what the fused GEMM+collective kernels
// store to, poll and TMA-load from.  No file descriptors are passed between processes.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" int fi_symm_alloc(void** out, long nbytes) {
  cudaError_t e = cudaMalloc(out, static_cast<size_t>(nbytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*out, 0, static_cast<size_t>(nbytes)));
}

extern "C" int fi_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }

// handle_out: 64 bytes
extern "C" int fi_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}

extern "C" int fi_ipc_open_handle(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int fi_ipc_close_handle(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

extern "C" int fi_ipc_handle_size() { return static_cast<int>(sizeof(cudaIpcMemHandle_t)); }
