// Set-up helpers for buffers that several ranks (one process per GPU on one node)
// address directly: allocation with an exportable handle, and mapping of a peer's
// allocation.  These are the only entry points of the library that allocate; they
// run once, before the simulation, never on the hot path.
#include <string.h>

#include "common.cuh"

using namespace bsx;

extern "C" {

int bsx_ipc_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return fail(BSX_ERR_INVALID_ARG, "bsx_ipc_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  BSX_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "bsx_ipc_alloc");
  }
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return BSX_OK;
}

int bsx_ipc_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return fail(BSX_ERR_INVALID_ARG, "bsx_ipc_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  BSX_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return BSX_OK;
}

int bsx_ipc_close(void* ptr) {
  if (!ptr) return BSX_OK;
  BSX_CUDA(cudaIpcCloseMemHandle(ptr));
  return BSX_OK;
}

int bsx_ipc_free(void* ptr) {
  if (!ptr) return BSX_OK;
  BSX_CUDA(cudaFree(ptr));
  return BSX_OK;
}

}  // extern "C"
