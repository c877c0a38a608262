// Device arenas that other processes (one per GPU) can map: allocation, CUDA IPC export/import, peer access.
//
// The reference exchanges tensors between peers as protobuf messages over libp2p streams
// (hivemind/averaging/allreduce.py:216-234). On one NVLink box peers instead exchange one 64-byte IPC handle per
// arena at group assembly and afterwards read each other's memory directly from kernels.
// A mapping opened here stays valid until hm_ipc_close, i.e. a peer that leaves a group can never turn another
// peer's in-flight kernel into a faulting one: mappings are closed only at endpoint shutdown.
#include "hm_common.cuh"

HM_API int hm_arena_alloc(void** out, unsigned long long bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}
HM_API int hm_arena_free(void* ptr) { return (int)cudaFree(ptr); }

HM_API int hm_ipc_export(void* ptr, void* handle_out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out64, &h, sizeof(h));
  return 0;
}
HM_API int hm_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
HM_API int hm_ipc_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
HM_API int hm_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }

// Same-process peers on different devices: enable direct access from `dev` to `peer` (idempotent).
HM_API int hm_enable_peer_access(int dev, int peer) {
  if (dev == peer) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer);
  if (e != cudaSuccess) return (int)e;
  if (!can) return -1;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(dev);
  e = cudaDeviceEnablePeerAccess(peer, 0);
  cudaSetDevice(prev);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return 0; }
  return (int)e;
}
HM_API int hm_memset_async(void* ptr, int value, unsigned long long bytes, cudaStream_t stream) {
  return (int)cudaMemsetAsync(ptr, value, bytes, stream);
}
HM_API int hm_memcpy_h2d_async(void* dst, const void* src, unsigned long long bytes, cudaStream_t stream) {
  return (int)cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream);
}
HM_API int hm_memcpy_d2h(void* dst, const void* src, unsigned long long bytes, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);
}
HM_API int hm_stream_create(cudaStream_t* out) { return (int)cudaStreamCreateWithFlags(out, cudaStreamNonBlocking); }
HM_API int hm_stream_sync(cudaStream_t s) { return (int)cudaStreamSynchronize(s); }
HM_API int hm_stream_destroy(cudaStream_t s) { return (int)cudaStreamDestroy(s); }
