// Fused optimizer step over one flat gradient bucket.
//
// The data-parallel engine keeps every bucket as four flat arrays: bf16 (or fp32)
// parameters, their gradients, fp32 master weights and fp32 momentum.  The daemon's
// all-reduce already wrote the averaged gradient in fp32 (scale and cast fused into
// the collective), so the whole update of a bucket is one streaming pass:
//   g = grad + wd * w ; m = mu * m + g ; w -= lr * m ; param = cast(w)
// 16 bytes in flight per array per thread, grid sized to the SM count.  No
// counterpart in the reference, which has no optimizer (it is a collective library);
// this kernel exists so that the gradient path of the benchmarks never leaves flat,
// heap-resident buffers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "dfccl.h"

namespace {

template <typename P>
__global__ void __launch_bounds__(256) sgdKernel(float* __restrict__ master, const float* __restrict__ grad,
                                                 float* __restrict__ mom, P* __restrict__ param, size_t n, float lr,
                                                 float mu, float wd, int firstStep) {
  const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 w = *reinterpret_cast<const float4*>(master + i);
      float4 g = *reinterpret_cast<const float4*>(grad + i);
      float4 m = firstStep ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(mom + i);
      g.x += wd * w.x; g.y += wd * w.y; g.z += wd * w.z; g.w += wd * w.w;
      m.x = mu * m.x + g.x; m.y = mu * m.y + g.y; m.z = mu * m.z + g.z; m.w = mu * m.w + g.w;
      w.x -= lr * m.x; w.y -= lr * m.y; w.z -= lr * m.z; w.w -= lr * m.w;
      *reinterpret_cast<float4*>(master + i) = w;
      *reinterpret_cast<float4*>(mom + i) = m;
      if (sizeof(P) == 2) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(param + i) = pk;
      } else {
        *reinterpret_cast<float4*>(param + i) = w;
      }
    } else {
      for (size_t k = i; k < n; ++k) {
        float w = master[k], g = grad[k] + wd * master[k];
        float m = (firstStep ? 0.f : mu * mom[k]) + g;
        w -= lr * m;
        master[k] = w; mom[k] = m;
        if (sizeof(P) == 2) param[k] = (P)__float2bfloat16_rn(w); else reinterpret_cast<float*>(param)[k] = w;
      }
    }
  }
}

}  // namespace

// paramType: ncclBfloat16 or ncclFloat32 (then `param` may alias `master`).  All arrays 16-byte aligned.
extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclFusedSgdStep(void* master, const void* grad, void* momentum, void* param, size_t n, int paramType,
                               float lr, float mu, float wd, int firstStep, cudaStream_t stream) {
  if (n == 0) return ncclSuccess;
  if (!master || !grad || !momentum || !param) return ncclInvalidArgument;
  if ((((uintptr_t)master | (uintptr_t)grad | (uintptr_t)momentum | (uintptr_t)param) & 15) != 0) return ncclInvalidArgument;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  size_t want = (n / 4 + 255) / 256;
  int grid = (int)(want < (size_t)sms * 8 ? (want ? want : 1) : (size_t)sms * 8);
  if (paramType == ncclBfloat16)
    sgdKernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((float*)master, (const float*)grad, (float*)momentum, (__nv_bfloat16*)param, n, lr, mu, wd, firstStep);
  else if (paramType == ncclFloat32)
    sgdKernel<float><<<grid, 256, 0, stream>>>((float*)master, (const float*)grad, (float*)momentum, (float*)param, n, lr, mu, wd, firstStep);
  else
    return ncclInvalidArgument;
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

// Load the kernels of this file into the current context without launching them.
extern "C" __attribute__((visibility("default"))) ncclResult_t dfcclOpsWarm(void) {
  cudaFuncAttributes a;
  if (cudaFuncGetAttributes(&a, sgdKernel<__nv_bfloat16>) != cudaSuccess) return ncclUnhandledCudaError;
  if (cudaFuncGetAttributes(&a, sgdKernel<float>) != cudaSuccess) return ncclUnhandledCudaError;
  return ncclSuccess;
}
