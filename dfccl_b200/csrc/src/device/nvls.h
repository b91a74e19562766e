// NVLS bodies.  All-reduce: every rank owns a slice; it reads the slice reduced over all members with
// multimem.ld_reduce (the NVLink switch adds the members' copies on the way), applies the scale and
// the output cast, and writes the result to all members with multimem.st.  Sum only, on f32, bf16
// and f16 inputs (bf16 / f16 accumulate in fp32 inside the switch); the output may be fp32.
// Addresses are byte offsets into the arena; every access is 16 bytes.
//
// On the host backend there is no switch: the "multicast" view is a loop over the members'
// blocks, so the schedule around it runs in the CPU tests unchanged.
//
// The reference has no counterpart (its NCCL generation predates NVLS).
#pragma once
#include "datapath.h"

namespace dfccl {

template <typename T> struct MmRed;
#if DF_DEVICE_CODE
template <> struct MmRed<float> {
  static __device__ __forceinline__ uint4 ld(const char* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct MmRed<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld(const char* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct MmRed<__half> {
  static __device__ __forceinline__ uint4 ld(const char* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
__device__ __forceinline__ void mmStore(char* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
#endif

template <typename Tin>
DF_HD uint4 nvlsLoad(const char* mc, char* const* peers, int n, uint64_t off) {
#if DF_DEVICE_CODE
  if (mc) return MmRed<Tin>::ld(mc + off);
#endif
  constexpr int V = 16 / (int)sizeof(Tin);
  float acc[V];
  for (int k = 0; k < V; ++k) acc[k] = 0.f;
  for (int j = 0; j < n; ++j) {
    uint4 v = ld16(peers[j] + off);
    for (int k = 0; k < V; ++k) acc[k] += (float)Lane<Tin>::get(v, k);
  }
  uint4 o;
  for (int k = 0; k < V; ++k) Lane<Tin>::put(o, k, acc[k]);
  return o;
}

DF_HD void nvlsStore(char* mc, char* const* peers, int n, uint64_t off, uint4 v) {
#if DF_DEVICE_CODE
  if (mc) { mmStore(mc + off, v); return; }
#endif
  for (int j = 0; j < n; ++j) st16(peers[j] + off, v);
}

// nElems elements starting at byte offsets inOff / outOff; nElems * sizeof(Tin) is a multiple of 16.
template <typename Tin, typename Tout>
DF_HD void nvlsSlice(char* mc, char* const* peers, int n, uint64_t inOff, uint64_t outOff, uint64_t nElems, float scale) {
  constexpr int V = 16 / (int)sizeof(Tin);                 // elements per input pack
  constexpr int W = (int)(sizeof(Tout) / sizeof(Tin));     // output packs per input pack (1 or 2)
  constexpr int U = 8;                                     // reductions in flight per thread: a round trip through the switch is long
  const uint64_t packs = nElems / V;
  const bool plain = scale == 1.0f && W == 1;
  for (uint64_t p0 = (uint64_t)df_tid() ; p0 < packs; p0 += (uint64_t)df_nthreads() * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t p = p0 + (uint64_t)u * df_nthreads();
      if (p < packs) v[u] = nvlsLoad<Tin>(mc, peers, n, inOff + p * 16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t p = p0 + (uint64_t)u * df_nthreads();
      if (p >= packs) continue;
      if (plain) { nvlsStore(mc, peers, n, outOff + p * 16, v[u]); continue; }
      uint4 o[W];
#pragma unroll
      for (int w = 0; w < W; ++w) o[w] = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float x = (float)Lane<Tin>::get(v[u], k) * scale;
        Lane<Tout>::put(o[k / (V / W)], k % (V / W), x);
      }
#pragma unroll
      for (int w = 0; w < W; ++w) nvlsStore(mc, peers, n, outOff + (p * W + w) * 16, o[w]);
    }
  }
}

// Reduce-scatter form: the reduced slice is kept locally (plain 16-byte stores to `dst`) instead of being broadcast.
template <typename Tin, typename Tout>
DF_HD void nvlsSliceToLocal(char* mc, char* const* peers, int n, uint64_t inOff, char* dst, uint64_t nElems, float scale) {
  constexpr int V = 16 / (int)sizeof(Tin);
  constexpr int W = (int)(sizeof(Tout) / sizeof(Tin));
  constexpr int U = 8;
  const uint64_t packs = nElems / V;
  const bool plain = scale == 1.0f && W == 1;
  for (uint64_t p0 = (uint64_t)df_tid(); p0 < packs; p0 += (uint64_t)df_nthreads() * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t p = p0 + (uint64_t)u * df_nthreads();
      if (p < packs) v[u] = nvlsLoad<Tin>(mc, peers, n, inOff + p * 16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t p = p0 + (uint64_t)u * df_nthreads();
      if (p >= packs) continue;
      if (plain) { st16(dst + p * 16, v[u]); continue; }
      uint4 o[W];
#pragma unroll
      for (int w = 0; w < W; ++w) o[w] = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < V; ++k) Lane<Tout>::put(o[k / (V / W)], k % (V / W), (float)Lane<Tin>::get(v[u], k) * scale);
#pragma unroll
      for (int w = 0; w < W; ++w) st16(dst + (p * W + w) * 16, o[w]);
    }
  }
}

// All-gather form: `bytes` (a multiple of 16) from local `src` to offset `outOff` of every member's arena.
DF_HD void nvlsBroadcastBytes(char* mc, char* const* peers, int n, const char* src, uint64_t outOff, uint64_t bytes) {
  constexpr int U = 8;
  const uint64_t packs = bytes / 16;
  for (uint64_t p0 = (uint64_t)df_tid(); p0 < packs; p0 += (uint64_t)df_nthreads() * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t p = p0 + (uint64_t)u * df_nthreads();
      if (p < packs) v[u] = ld16(src + p * 16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint64_t p = p0 + (uint64_t)u * df_nthreads();
      if (p < packs) nvlsStore(mc, peers, n, outOff + p * 16, v[u]);
    }
  }
}

// Which (input, output) pairs the schedule exists for.
DF_HD bool nvlsTypesOk(int inType, int outType) {
  if (inType == ncclFloat32) return outType == ncclFloat32;
  if (inType == ncclBfloat16 || inType == ncclFloat16) return outType == inType || outType == ncclFloat32;
  return false;
}

DF_HD bool nvlsDispatch(int inType, int outType, char* mc, char* const* peers, int n, uint64_t inOff, uint64_t outOff, uint64_t nElems, float scale) {
  if (inType == ncclFloat32 && outType == ncclFloat32) nvlsSlice<float, float>(mc, peers, n, inOff, outOff, nElems, scale);
  else if (inType == ncclBfloat16 && outType == ncclBfloat16) nvlsSlice<__nv_bfloat16, __nv_bfloat16>(mc, peers, n, inOff, outOff, nElems, scale);
  else if (inType == ncclBfloat16 && outType == ncclFloat32) nvlsSlice<__nv_bfloat16, float>(mc, peers, n, inOff, outOff, nElems, scale);
  else if (inType == ncclFloat16 && outType == ncclFloat16) nvlsSlice<__half, __half>(mc, peers, n, inOff, outOff, nElems, scale);
  else if (inType == ncclFloat16 && outType == ncclFloat32) nvlsSlice<__half, float>(mc, peers, n, inOff, outOff, nElems, scale);
  else return false;
  return true;
}

DF_HD bool nvlsDispatchToLocal(int inType, int outType, char* mc, char* const* peers, int n, uint64_t inOff, char* dst, uint64_t nElems, float scale) {
  if (inType == ncclFloat32 && outType == ncclFloat32) nvlsSliceToLocal<float, float>(mc, peers, n, inOff, dst, nElems, scale);
  else if (inType == ncclBfloat16 && outType == ncclBfloat16) nvlsSliceToLocal<__nv_bfloat16, __nv_bfloat16>(mc, peers, n, inOff, dst, nElems, scale);
  else if (inType == ncclBfloat16 && outType == ncclFloat32) nvlsSliceToLocal<__nv_bfloat16, float>(mc, peers, n, inOff, dst, nElems, scale);
  else if (inType == ncclFloat16 && outType == ncclFloat16) nvlsSliceToLocal<__half, __half>(mc, peers, n, inOff, dst, nElems, scale);
  else if (inType == ncclFloat16 && outType == ncclFloat32) nvlsSliceToLocal<__half, float>(mc, peers, n, inOff, dst, nElems, scale);
  else return false;
  return true;
}

}  // namespace dfccl
