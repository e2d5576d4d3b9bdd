// Device-memory helpers for a host layer that includes no CUDA header (the C++ shim carries streams as void*): plain
// allocations, host <-> device copies and a fill kernel.  Counterparts of the reference's Device::alloc / Buffer::cpu
// (src/core/metal.hpp:11-40; shared storage there, explicit copies here) and of its fill dispatches
// (src/model/dec_layer.mm: fill0).
#include "msb_common.cuh"

namespace msb {

__global__ void fill_f32_kernel(float* p, float v, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) p[i] = v;
}

int device_alloc(size_t bytes, void** out) {
  if (!out) return fail(kErrArg, "device_alloc: null out");
  void* d = nullptr;
  MSB_CUDA(cudaMalloc(&d, bytes ? bytes : 16));
  cudaError_t e = cudaMemset(d, 0, bytes ? bytes : 16);
  if (e != cudaSuccess) { cudaFree(d); return cuda_fail(e, "device_alloc"); }
  *out = d;
  return kOk;
}
int device_free(void* p) {
  if (p) MSB_CUDA(cudaFree(p));
  return kOk;
}
int copy_to_device(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  if (bytes && (!dst || !src)) return fail(kErrArg, "copy_to_device: null pointer");
  MSB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st));
  MSB_CUDA(cudaStreamSynchronize(st));
  return kOk;
}
int copy_to_host(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  if (bytes && (!dst || !src)) return fail(kErrArg, "copy_to_host: null pointer");
  MSB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, st));
  MSB_CUDA(cudaStreamSynchronize(st));
  return kOk;
}
int copy_device(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  if (bytes == 0) return kOk;
  if (!dst || !src) return fail(kErrArg, "copy_device: null pointer");
  MSB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st));
  return kOk;
}
int fill_f32(float* p, float v, size_t n, cudaStream_t st) {
  if (n == 0) return kOk;
  if (!p) return fail(kErrArg, "fill_f32: null pointer");
  const int blocks = (int)((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024);
  MSB_CUDA(launch_pdl(fill_f32_kernel, dim3(blocks), dim3(256), 0, st, p, v, n));
  MSB_LAUNCH_CHECK("fill_f32_kernel");
  return kOk;
}

}  // namespace msb
