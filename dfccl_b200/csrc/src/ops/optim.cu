// Fused optimizer step over one flat gradient bucket.
//
// The data-parallel engine keeps every bucket as four flat arrays: bf16 (or fp32)
// parameters, their gradients, fp32 master weights and fp32 momentum.  The daemon's
// all-reduce already wrote the averaged gradient in fp32 (scale and cast fused into
// the collective), so the whole update of a bucket is one streaming pass:
//   g = grad + wd * w ; m = mu * m + g ; w -= lr * m ; param = cast(w)
// (SGD with momentum; an AdamW variant of the same shape follows it)
// 16 bytes in flight per array per thread, grid sized to the SM count.  No
// counterpart in the reference, which has no optimizer (it is a collective library);
// this kernel exists so that the gradient path of the benchmarks never leaves flat,
// heap-resident buffers.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
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

// AdamW over the same flat arrays (decoupled weight decay; bias correction folded into the two scalars the host
// passes: stepSize = lr / (1 - beta1^t), invBias2Sqrt = 1 / sqrt(1 - beta2^t)):
//   m = b1 m + (1 - b1) g ; v = b2 v + (1 - b2) g^2 ; w = w (1 - lr wd) - stepSize * m / (sqrt(v) * invBias2Sqrt + eps)
__device__ __forceinline__ void adamwOne(float& w, float g, float& m, float& v, float b1, float b2, float eps, float decay,
                                         float stepSize, float invBias2Sqrt) {
  m = b1 * m + (1.f - b1) * g;
  v = b2 * v + (1.f - b2) * g * g;
  // one square root and one fast division per element: the IEEE division's slow path costs more registers and
  // instructions than the whole rest of the update and made the kernel instruction-bound (2 ulp is irrelevant here)
  w = w * decay - stepSize * __fdividef(m, __fsqrt_rn(v) * invBias2Sqrt + eps);
}

template <typename P>
__global__ void __launch_bounds__(256) adamwKernel(float* __restrict__ master, const float* __restrict__ grad,
                                                   float* __restrict__ m1, float* __restrict__ m2, P* __restrict__ param, size_t n,
                                                   float lr, float b1, float b2, float eps, float wd, float stepSize, float invBias2Sqrt) {
  const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
  const float decay = 1.f - lr * wd;
  const size_t nFull = n & ~(size_t)3;
  for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < nFull; i += stride) {
    float4 w = *reinterpret_cast<const float4*>(master + i);
    const float4 g = *reinterpret_cast<const float4*>(grad + i);
    float4 m = *reinterpret_cast<const float4*>(m1 + i);
    float4 v = *reinterpret_cast<const float4*>(m2 + i);
    adamwOne(w.x, g.x, m.x, v.x, b1, b2, eps, decay, stepSize, invBias2Sqrt);
    adamwOne(w.y, g.y, m.y, v.y, b1, b2, eps, decay, stepSize, invBias2Sqrt);
    adamwOne(w.z, g.z, m.z, v.z, b1, b2, eps, decay, stepSize, invBias2Sqrt);
    adamwOne(w.w, g.w, m.w, v.w, b1, b2, eps, decay, stepSize, invBias2Sqrt);
    *reinterpret_cast<float4*>(master + i) = w;
    *reinterpret_cast<float4*>(m1 + i) = m;
    *reinterpret_cast<float4*>(m2 + i) = v;
    if (sizeof(P) == 2) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(w.x, w.y), hi = __floats2bfloat162_rn(w.z, w.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(param + i) = pk;
    } else {
      *reinterpret_cast<float4*>(param + i) = w;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {             // up to three elements past the last full pack
    for (size_t k = nFull; k < n; ++k) {
      float w = master[k], m = m1[k], v = m2[k];
      adamwOne(w, grad[k], m, v, b1, b2, eps, decay, stepSize, invBias2Sqrt);
      master[k] = w; m1[k] = m; m2[k] = v;
      if (sizeof(P) == 2) param[k] = (P)__float2bfloat16_rn(w); else reinterpret_cast<float*>(param)[k] = w;
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

// `step` counts from 1.  State arrays (first and second moment) start at zero.
extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclFusedAdamWStep(void* master, const void* grad, void* moment1, void* moment2, void* param, size_t n, int paramType,
                                 float lr, float beta1, float beta2, float eps, float wd, int step, cudaStream_t stream) {
  if (n == 0) return ncclSuccess;
  if (!master || !grad || !moment1 || !moment2 || !param || step < 1) return ncclInvalidArgument;
  if ((((uintptr_t)master | (uintptr_t)grad | (uintptr_t)moment1 | (uintptr_t)moment2 | (uintptr_t)param) & 15) != 0) return ncclInvalidArgument;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  size_t want = (n / 4 + 255) / 256;
  int grid = (int)(want < (size_t)sms * 8 ? (want ? want : 1) : (size_t)sms * 8);
  const float stepSize = lr / (1.f - powf(beta1, (float)step));
  const float invBias2Sqrt = 1.f / sqrtf(1.f - powf(beta2, (float)step));
  if (paramType == ncclBfloat16)
    adamwKernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((float*)master, (const float*)grad, (float*)moment1, (float*)moment2, (__nv_bfloat16*)param, n,
                                                         lr, beta1, beta2, eps, wd, stepSize, invBias2Sqrt);
  else if (paramType == ncclFloat32)
    adamwKernel<float><<<grid, 256, 0, stream>>>((float*)master, (const float*)grad, (float*)moment1, (float*)moment2, (float*)param, n,
                                                 lr, beta1, beta2, eps, wd, stepSize, invBias2Sqrt);
  else
    return ncclInvalidArgument;
  return cudaGetLastError() == cudaSuccess ? ncclSuccess : ncclUnhandledCudaError;
}

// Load the kernels of this file into the current context without launching them.
extern "C" __attribute__((visibility("default"))) ncclResult_t dfcclOpsWarm(void) {
  cudaFuncAttributes a;
  if (cudaFuncGetAttributes(&a, sgdKernel<__nv_bfloat16>) != cudaSuccess) return ncclUnhandledCudaError;
  if (cudaFuncGetAttributes(&a, sgdKernel<float>) != cudaSuccess) return ncclUnhandledCudaError;
  if (cudaFuncGetAttributes(&a, adamwKernel<__nv_bfloat16>) != cudaSuccess) return ncclUnhandledCudaError;
  if (cudaFuncGetAttributes(&a, adamwKernel<float>) != cudaSuccess) return ncclUnhandledCudaError;
  return ncclSuccess;
}
