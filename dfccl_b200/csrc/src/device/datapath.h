// Element-wise data path: N sources -> reduce -> scale / divide -> cast -> M destinations.
//
// Role of the reference's ReduceOrCopyMulti and its functors
// (src/include/common_kernel.h:490-690, src/include/reduce_kernel.h:15-705), built
// differently: sources and destinations are plain pointers into this GPU's or a
// peer's symmetric heap (no FIFO slots), 16/32-bit floating inputs accumulate in
// fp32 in a fixed rank order so every rank computes bit-identical results, and
// the scale (gradient averaging, user PreMulSum scalar) and the output cast are
// applied in registers before the only store - the "fused scale / cast".
// The 16-byte packs are the unit of every vector access; a range whose pointers
// are not 16-byte aligned takes the scalar path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "dfccl.h"
#include "platform.h"
#include "types.h"

namespace dfccl {

enum RedOp : int { OP_SUM = 0, OP_PROD = 1, OP_MAX = 2, OP_MIN = 3 };

struct DataArgs {
  int nsrc, ndst;
  const char* src[DF_MAX_RANKS];
  char* dst[DF_MAX_RANKS];
  uint64_t n;            // elements
  double scale;          // 1.0 = none
  int postDiv;           // 0 = none
};

template <int N> struct BitsOf;
template <> struct BitsOf<1> { typedef uint8_t type; };
template <> struct BitsOf<2> { typedef uint16_t type; };
template <> struct BitsOf<4> { typedef uint32_t type; };
template <> struct BitsOf<8> { typedef uint64_t type; };

template <typename T> DF_HD T ld_elem(const T* p) {
  typedef typename BitsOf<sizeof(T)>::type B;
  B b = *(const volatile B*)p;
  T v;
  __builtin_memcpy(&v, &b, sizeof(T));
  return v;
}
template <typename T> DF_HD void st_elem(T* p, T v) {
  typedef typename BitsOf<sizeof(T)>::type B;
  B b;
  __builtin_memcpy(&b, &v, sizeof(T));
  *(volatile B*)p = b;
}

// accumulator type and conversions
template <typename T> struct Elem { typedef T Acc; static DF_HD Acc up(T v) { return v; } static DF_HD T down(Acc a) { return a; } enum { isFloat = 0, isBf16 = 0 }; };
template <> struct Elem<int8_t> { typedef int32_t Acc; static DF_HD Acc up(int8_t v) { return v; } static DF_HD int8_t down(Acc a) { return (int8_t)a; } enum { isFloat = 0, isBf16 = 0 }; };
template <> struct Elem<uint8_t> { typedef uint32_t Acc; static DF_HD Acc up(uint8_t v) { return v; } static DF_HD uint8_t down(Acc a) { return (uint8_t)a; } enum { isFloat = 0, isBf16 = 0 }; };
template <> struct Elem<float> { typedef float Acc; static DF_HD Acc up(float v) { return v; } static DF_HD float down(Acc a) { return a; } enum { isFloat = 1, isBf16 = 0 }; };
template <> struct Elem<double> { typedef double Acc; static DF_HD Acc up(double v) { return v; } static DF_HD double down(Acc a) { return a; } enum { isFloat = 1, isBf16 = 0 }; };
template <> struct Elem<__half> { typedef float Acc; static DF_HD Acc up(__half v) { return __half2float(v); } static DF_HD __half down(Acc a) { return __float2half_rn(a); } enum { isFloat = 1, isBf16 = 0 }; };
template <> struct Elem<__nv_bfloat16> { typedef float Acc; static DF_HD Acc up(__nv_bfloat16 v) { return __bfloat162float(v); } static DF_HD __nv_bfloat16 down(Acc a) { return __float2bfloat16_rn(a); } enum { isFloat = 1, isBf16 = 1 }; };

template <int OP, typename A> DF_HD A red(A a, A b) {
  if (OP == OP_SUM) return a + b;
  if (OP == OP_PROD) return a * b;
  if (OP == OP_MAX) return a > b ? a : b;
  return a < b ? a : b;
}

template <typename Tin, typename Tout, typename A>
DF_HD typename Elem<Tout>::Acc finish(A a, double scale, int postDiv) {
  typedef typename Elem<Tout>::Acc AO;
  if (Elem<Tin>::isFloat) {
    if (scale != 1.0) a = (A)(a * (A)scale);
  } else if (postDiv) {
    a = a / (A)postDiv;
  } else if (scale != 1.0) {
    a = (A)((double)a * scale);
  }
  return (AO)a;
}

DF_HD void st8(void* p, uint2 v) {
#if DF_DEVICE_CODE
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
#else
  __builtin_memcpy(p, &v, 8);
#endif
}

// ---- 16-byte pack <-> V accumulators, in registers only on the device.  (Going through a local
// array and memcpy is what the host build does; on the device an address-taken array can end up in
// local memory, and a load whose result is stored right away cannot overlap with the next load.)
DF_HD uint32_t packWord(const uint4& v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }
DF_HD void setWord(uint4& v, int i, uint32_t w) { if (i == 0) v.x = w; else if (i == 1) v.y = w; else if (i == 2) v.z = w; else v.w = w; }

template <typename T> struct Lane;     // element k of a 16-byte pack <-> accumulator
#if DF_DEVICE_CODE
template <> struct Lane<float> {
  static DF_HD float get(const uint4& v, int k) { return __uint_as_float(packWord(v, k)); }
  static DF_HD void put(uint4& v, int k, float a) { setWord(v, k, __float_as_uint(a)); }
};
template <> struct Lane<int32_t> {
  static DF_HD int32_t get(const uint4& v, int k) { return (int32_t)packWord(v, k); }
  static DF_HD void put(uint4& v, int k, int32_t a) { setWord(v, k, (uint32_t)a); }
};
template <> struct Lane<uint32_t> {
  static DF_HD uint32_t get(const uint4& v, int k) { return packWord(v, k); }
  static DF_HD void put(uint4& v, int k, uint32_t a) { setWord(v, k, a); }
};
template <> struct Lane<__nv_bfloat16> {
  static DF_HD float get(const uint4& v, int k) { uint32_t w = packWord(v, k >> 1); return __uint_as_float((k & 1) ? (w & 0xffff0000u) : (w << 16)); }
  static DF_HD void put(uint4& v, int k, float a) {
    uint32_t h = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(a));
    uint32_t w = packWord(v, k >> 1);
    setWord(v, k >> 1, (k & 1) ? ((w & 0x0000ffffu) | (h << 16)) : ((w & 0xffff0000u) | h));
  }
};
template <> struct Lane<__half> {
  static DF_HD float get(const uint4& v, int k) { uint32_t w = packWord(v, k >> 1); return __half2float(__ushort_as_half((unsigned short)((k & 1) ? (w >> 16) : (w & 0xffffu)))); }
  static DF_HD void put(uint4& v, int k, float a) {
    uint32_t h = (uint32_t)__half_as_ushort(__float2half_rn(a));
    uint32_t w = packWord(v, k >> 1);
    setWord(v, k >> 1, (k & 1) ? ((w & 0x0000ffffu) | (h << 16)) : ((w & 0xffff0000u) | h));
  }
};
template <> struct Lane<int8_t> {
  static DF_HD int32_t get(const uint4& v, int k) { return (int32_t)(int8_t)(packWord(v, k >> 2) >> (8 * (k & 3))); }
  static DF_HD void put(uint4& v, int k, int32_t a) { uint32_t sh = 8 * (k & 3), w = packWord(v, k >> 2); setWord(v, k >> 2, (w & ~(0xffu << sh)) | (((uint32_t)a & 0xffu) << sh)); }
};
template <> struct Lane<uint8_t> {
  static DF_HD uint32_t get(const uint4& v, int k) { return (packWord(v, k >> 2) >> (8 * (k & 3))) & 0xffu; }
  static DF_HD void put(uint4& v, int k, uint32_t a) { uint32_t sh = 8 * (k & 3), w = packWord(v, k >> 2); setWord(v, k >> 2, (w & ~(0xffu << sh)) | ((a & 0xffu) << sh)); }
};
template <> struct Lane<double> {
  static DF_HD double get(const uint4& v, int k) { return __hiloint2double((int)packWord(v, 2 * k + 1), (int)packWord(v, 2 * k)); }
  static DF_HD void put(uint4& v, int k, double a) { setWord(v, 2 * k, (uint32_t)__double2loint(a)); setWord(v, 2 * k + 1, (uint32_t)__double2hiint(a)); }
};
template <> struct Lane<int64_t> {
  static DF_HD int64_t get(const uint4& v, int k) { return (int64_t)(((uint64_t)packWord(v, 2 * k + 1) << 32) | packWord(v, 2 * k)); }
  static DF_HD void put(uint4& v, int k, int64_t a) { setWord(v, 2 * k, (uint32_t)(uint64_t)a); setWord(v, 2 * k + 1, (uint32_t)((uint64_t)a >> 32)); }
};
template <> struct Lane<uint64_t> {
  static DF_HD uint64_t get(const uint4& v, int k) { return ((uint64_t)packWord(v, 2 * k + 1) << 32) | packWord(v, 2 * k); }
  static DF_HD void put(uint4& v, int k, uint64_t a) { setWord(v, 2 * k, (uint32_t)a); setWord(v, 2 * k + 1, (uint32_t)(a >> 32)); }
};
#else
template <typename T> struct Lane {
  typedef typename Elem<T>::Acc A;
  static A get(const uint4& v, int k) { T e; __builtin_memcpy(&e, (const char*)&v + k * sizeof(T), sizeof(T)); return Elem<T>::up(e); }
  static void put(uint4& v, int k, A a) { T e = Elem<T>::down(a); __builtin_memcpy((char*)&v + k * sizeof(T), &e, sizeof(T)); }
};
#endif

// ---- whole-pack conversions: V accumulators <-> 16-byte words, few instructions per element
template <typename Tout, typename A, int V>
DF_HD void packAll(uint4* ow, const A* r) {
#if DF_DEVICE_CODE
  if (sizeof(Tout) == 2 && sizeof(A) == 4) {            // bf16 / fp16 from fp32: one convert per pair
#pragma unroll
    for (int k = 0; k < V; k += 2) {
      uint32_t word;
      if (Elem<Tout>::isBf16) { __nv_bfloat162 h = __floats2bfloat162_rn((float)r[k], (float)r[k + 1]); word = *reinterpret_cast<uint32_t*>(&h); }
      else { __half2 h = __floats2half2_rn((float)r[k], (float)r[k + 1]); word = *reinterpret_cast<uint32_t*>(&h); }
      setWord(ow[(k / 2) / 4], (k / 2) % 4, word);
    }
    return;
  }
#endif
  constexpr int VO = 16 / (int)sizeof(Tout);
#pragma unroll
  for (int k = 0; k < V; ++k) Lane<Tout>::put(ow[k / VO], k % VO, (typename Elem<Tout>::Acc)r[k]);
}

// ---- sources that are not 16-byte aligned.  All sources of one call share one misalignment (they are the same offset
// into symmetric buffers), so a logical pack is 16 bytes that straddle two aligned packs: bytes [shift, shift + 16) of
// lo:hi.  The aligned packs are loaded as usual and shifted in registers; in a full trip the upper pack of a thread is
// the lower pack of its neighbour lane and comes by shuffle, so the memory traffic stays that of an aligned copy.
// (Role of the reference's misaligned-load helpers, src/collectives/device/op128.h:40-68.)
DF_HD uint4 shiftPack(const uint4& lo, const uint4& hi, uint32_t shift) {
#if DF_DEVICE_CODE
  const uint32_t bs = (shift & 3u) * 8u;
  uint32_t w0, w1, w2, w3, w4;
  switch (shift >> 2) {
    case 0: w0 = lo.x; w1 = lo.y; w2 = lo.z; w3 = lo.w; w4 = hi.x; break;
    case 1: w0 = lo.y; w1 = lo.z; w2 = lo.w; w3 = hi.x; w4 = hi.y; break;
    case 2: w0 = lo.z; w1 = lo.w; w2 = hi.x; w3 = hi.y; w4 = hi.z; break;
    default: w0 = lo.w; w1 = hi.x; w2 = hi.y; w3 = hi.z; w4 = hi.w; break;
  }
  return make_uint4(__funnelshift_r(w0, w1, bs), __funnelshift_r(w1, w2, bs), __funnelshift_r(w2, w3, bs), __funnelshift_r(w3, w4, bs));
#else
  unsigned char b[32];
  __builtin_memcpy(b, &lo, 16);
  __builtin_memcpy(b + 16, &hi, 16);
  uint4 o;
  __builtin_memcpy(&o, b + shift, 16);
  return o;
#endif
}

// U logical packs of one source for this thread; pack u starts `u * strideB` bytes after `s`, `shift` = s & 15.
// SHIFT = false: s is aligned.  FULL: every thread of the block loads all of its U packs (warp shuffles are safe).
template <bool FULL, bool SHIFT, int U>
DF_HD void loadPacks(uint4* out, const char* s, uint32_t strideB, uint32_t shift, uint64_t p0, uint32_t stride, uint64_t nPacks) {
  if (!SHIFT) {
#pragma unroll
    for (int u = 0; u < U; ++u) if (FULL || p0 + (uint64_t)u * stride < nPacks) out[u] = ld16(s + (uint64_t)u * strideB);
    return;
  }
  const char* a = s - shift;                       // aligned; every aligned pack touched holds at least one wanted byte
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (!(FULL || p0 + (uint64_t)u * stride < nPacks)) continue;
    const uint4 lo = ld16(a + (uint64_t)u * strideB);
    uint4 hi;
#if DF_DEVICE_CODE
    if (FULL) {
      hi.x = __shfl_down_sync(0xffffffffu, lo.x, 1); hi.y = __shfl_down_sync(0xffffffffu, lo.y, 1);
      hi.z = __shfl_down_sync(0xffffffffu, lo.z, 1); hi.w = __shfl_down_sync(0xffffffffu, lo.w, 1);
      if ((threadIdx.x & 31) == 31) hi = ld16(a + (uint64_t)u * strideB + 16);
    } else
#endif
      hi = ld16(a + (uint64_t)u * strideB + 16);
    out[u] = shiftPack(lo, hi, shift);
  }
}

// One noinline body per (input type, output type, operator): the daemon's register
// budget is the maximum over what it inlines, so the variants stay out of line.
// The hot loop is written for instruction count (it was issue-bound at 150 warp instructions
// per 16-byte pack in its first form): pointers are read from shared memory once per source
// and trip, indices are a base plus compile-time multiples of the stride, the bounds test is
// hoisted out of full trips, the scale is a float decided once, outputs are packed pairwise.
template <typename Tin, typename Tout, int OP, bool FULL, bool SHIFT, int U>
DF_HD void reduceTrip(const DataArgs* a, uint64_t p0, uint64_t nPacks, uint32_t strideB, int nsrc, int ndst,
                      typename Elem<Tin>::Acc mul, bool doMul, int postDiv, double dscale,
                      uint64_t srcOff, uint64_t dstOff, uint32_t shift) {
  typedef typename Elem<Tin>::Acc A;
  constexpr int V = 16 / (int)sizeof(Tin);
  constexpr int OUTB = V * (int)sizeof(Tout);
  constexpr int NW = (OUTB + 15) / 16;
  const uint32_t stride = strideB >> 4;
  const uint64_t off = srcOff + p0 * 16;
  A acc[U][V];
  uint4 cur[U], nxt[U];
  loadPacks<FULL, SHIFT, U>(cur, a->src[0] + off, strideB, shift, p0, stride, nPacks);
  for (int j = 1; j <= nsrc; ++j) {
    if (j < nsrc) loadPacks<FULL, SHIFT, U>(nxt, a->src[j] + off, strideB, shift, p0, stride, nPacks);
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const A e = (A)Lane<Tin>::get(cur[u], k);
        acc[u][k] = j == 1 ? e : red<OP>(acc[u][k], e);
      }
    }
    if (j < nsrc) {
#pragma unroll
      for (int u = 0; u < U; ++u) cur[u] = nxt[u];
    }
  }
  uint4 ow[U][NW];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (Elem<Tin>::isFloat) {
      if (doMul) {
#pragma unroll
        for (int k = 0; k < V; ++k) acc[u][k] = acc[u][k] * mul;
      }
    } else if (postDiv) {
#pragma unroll
      for (int k = 0; k < V; ++k) acc[u][k] = acc[u][k] / (A)postDiv;
    } else if (doMul) {
#pragma unroll
      for (int k = 0; k < V; ++k) acc[u][k] = (A)((double)acc[u][k] * dscale);
    }
#pragma unroll
    for (int w = 0; w < NW; ++w) ow[u][w] = make_uint4(0u, 0u, 0u, 0u);
    packAll<Tout, A, V>(ow[u], acc[u]);
  }
  for (int d = 0; d < ndst; ++d) {
    char* o = a->dst[d] + dstOff + p0 * OUTB;
#pragma unroll
    for (int u = 0; u < U; ++u) if (FULL || p0 + (uint64_t)u * stride < nPacks) {
      char* ou = o + (uint64_t)u * stride * OUTB;
      if (OUTB == 8) st8(ou, make_uint2(ow[u][0].x, ow[u][0].y));
      else {
#pragma unroll
        for (int w = 0; w < OUTB / 16; ++w) st16(ou + 16 * w, ow[u][w]);
      }
    }
  }
}

// The unrolled trips of one call, for aligned (SHIFT = false) or uniformly misaligned sources.
template <typename Tin, typename Tout, int OP, bool SHIFT>
DF_HD void reduceTrips(const DataArgs* a, uint64_t nPacks, int nsrc, int ndst, typename Elem<Tin>::Acc mul, bool doMul, int postDiv,
                       double scale, uint64_t srcOff, uint64_t dstOff, uint32_t shift) {
  constexpr int U = OP == OP_SUM ? 4 : 2;     // the sum carries the traffic; the rarer operators trade speed for code size
  const int tid = df_tid(), nt = df_nthreads();
  // Software-pipelined over the sources inside a trip: the U loads of source j+1 are issued before
  // the U packs of source j are consumed, so up to 2*U 16-byte loads are in flight per thread.
  const uint64_t step = (uint64_t)nt * U;
  const uint32_t strideB = (uint32_t)nt * 16u;
  uint64_t base = 0;
  for (; base + step <= nPacks; base += step)
    reduceTrip<Tin, Tout, OP, true, SHIFT, U>(a, base + tid, nPacks, strideB, nsrc, ndst, mul, doMul, postDiv, scale, srcOff, dstOff, shift);
  // what the unrolled trips leave: one pack per thread per trip, the last trip partly filled
  for (; base + nt <= nPacks; base += nt)
    reduceTrip<Tin, Tout, OP, true, SHIFT, 1>(a, base + tid, nPacks, strideB, nsrc, ndst, mul, doMul, postDiv, scale, srcOff, dstOff, shift);
  if (base + tid < nPacks)
    reduceTrip<Tin, Tout, OP, false, SHIFT, 1>(a, base + tid, nPacks, strideB, nsrc, ndst, mul, doMul, postDiv, scale, srcOff, dstOff, shift);
}

template <typename Tin, typename Tout, int OP>
DF_HD_NOINLINE void reduce_copy(const DataArgs* a) {
  typedef typename Elem<Tin>::Acc A;
  constexpr int V = 16 / (int)sizeof(Tin);
  constexpr int OUTB = V * (int)sizeof(Tout);
  constexpr int DA = OUTB >= 16 ? 16 : OUTB;          // alignment the vector stores need
  const int tid = df_tid(), nt = df_nthreads();
  const int nsrc = a->nsrc, ndst = a->ndst;
  const uint64_t n = a->n;
  const double scale = a->scale;
  const int postDiv = a->postDiv;
  const bool doMul = scale != 1.0;
  const A mul = (A)scale;

  // The vector path needs all sources at one misalignment and all destinations at one misalignment (true for equal
  // offsets into symmetric buffers): `head` elements bring the destinations to their alignment, from there on the
  // sources are read as packs shifted by `shift` bytes.  Anything else goes element by element.
  const uint32_t sphase = (uint32_t)((uintptr_t)a->src[0] & 15), dphase = (uint32_t)((uintptr_t)a->dst[0] & (DA - 1));
  bool vec = (dphase % sizeof(Tout)) == 0 && (sphase % sizeof(Tin)) == 0;
  for (int j = 1; j < nsrc; ++j) vec &= ((uintptr_t)a->src[j] & 15) == sphase;
  for (int j = 1; j < ndst; ++j) vec &= ((uintptr_t)a->dst[j] & (DA - 1)) == dphase;
  uint64_t head = vec ? ((DA - dphase) % DA) / sizeof(Tout) : 0;
  if (head > n) head = n;
  const uint32_t shift = (uint32_t)((sphase + head * sizeof(Tin)) & 15);
  const uint64_t nPacks = vec ? (n - head) / V : 0;
  const uint64_t srcOff = head * sizeof(Tin), dstOff = head * sizeof(Tout);
  if (nPacks) {
    if (shift == 0) reduceTrips<Tin, Tout, OP, false>(a, nPacks, nsrc, ndst, mul, doMul, postDiv, scale, srcOff, dstOff, 0);
    else reduceTrips<Tin, Tout, OP, true>(a, nPacks, nsrc, ndst, mul, doMul, postDiv, scale, srcOff, dstOff, shift);
  }
  // the head, the ragged tail, or everything when the pointers do not line up: element by element
  const uint64_t tail0 = head + nPacks * V;
  for (uint64_t i = tid; i < head + (n - tail0); i += nt) {
    const uint64_t e = i < head ? i : tail0 + (i - head);
    A acc = Elem<Tin>::up(ld_elem((const Tin*)a->src[0] + e));
    for (int j = 1; j < nsrc; ++j) acc = red<OP>(acc, Elem<Tin>::up(ld_elem((const Tin*)a->src[j] + e)));
    Tout o = Elem<Tout>::down(finish<Tin, Tout>(acc, scale, postDiv));
    for (int d = 0; d < ndst; ++d) st_elem((Tout*)a->dst[d] + e, o);
  }
}

// Byte copy of one source to M destinations (AllGather, Broadcast, staging).
template <bool FULL, bool SHIFT, int U>
DF_HD void copyTrip(const DataArgs* a, uint64_t p0, uint64_t nPacks, uint32_t strideB, int ndst, uint64_t off, uint32_t shift) {
  const uint32_t stride = strideB >> 4;
  uint4 raw[U];
  loadPacks<FULL, SHIFT, U>(raw, a->src[0] + off + p0 * 16, strideB, shift, p0, stride, nPacks);
  for (int d = 0; d < ndst; ++d) {
    char* o = a->dst[d] + off + p0 * 16;
#pragma unroll
    for (int u = 0; u < U; ++u) if (FULL || p0 + (uint64_t)u * stride < nPacks) st16(o + (uint64_t)u * strideB, raw[u]);
  }
}

template <bool SHIFT>
DF_HD void copyTrips(const DataArgs* a, uint64_t nPacks, int ndst, uint64_t off, uint32_t shift) {
  constexpr int U = 8;
  const int tid = df_tid(), nt = df_nthreads();
  const uint64_t step = (uint64_t)nt * U;
  const uint32_t strideB = (uint32_t)nt * 16u;
  uint64_t base = 0;
  for (; base + step <= nPacks; base += step) copyTrip<true, SHIFT, U>(a, base + tid, nPacks, strideB, ndst, off, shift);
  for (; base + nt <= nPacks; base += nt) copyTrip<true, SHIFT, 1>(a, base + tid, nPacks, strideB, ndst, off, shift);
  if (base + tid < nPacks) copyTrip<false, SHIFT, 1>(a, base + tid, nPacks, strideB, ndst, off, shift);
}

#ifdef DF_DATAPATH_IMPL
__host__ __device__ void copy_multi(const DataArgs* a) {
  const int tid = df_tid(), nt = df_nthreads();
  const int ndst = a->ndst;
  const uint64_t nbytes = a->n;
  // destinations at one misalignment: `head` bytes bring them to 16, from there the source is read as shifted packs
  const uint32_t dphase = ndst ? (uint32_t)((uintptr_t)a->dst[0] & 15) : 0;
  bool vec = ndst > 0;
  for (int j = 1; j < ndst; ++j) vec &= ((uintptr_t)a->dst[j] & 15) == dphase;
  uint64_t head = vec ? (16 - dphase) % 16 : 0;
  if (head > nbytes) head = nbytes;
  const uint32_t shift = (uint32_t)(((uintptr_t)a->src[0] + head) & 15);
  const uint64_t nPacks = vec ? (nbytes - head) / 16 : 0;
  if (nPacks) {
    if (shift == 0) copyTrips<false>(a, nPacks, ndst, head, 0);
    else copyTrips<true>(a, nPacks, ndst, head, shift);
  }
  const uint64_t tail0 = head + nPacks * 16;
  for (uint64_t i = tid; i < head + (nbytes - tail0); i += nt) {
    const uint64_t e = i < head ? i : tail0 + (i - head);
    uint8_t b = ld_elem((const uint8_t*)a->src[0] + e);
    for (int d = 0; d < ndst; ++d) st_elem((uint8_t*)a->dst[d] + e, b);
  }
}

#else
__host__ __device__ void copy_multi(const DataArgs* a);
#endif

DF_HD int dtypeSize(int t) {
  switch (t) {
    case ncclInt8: case ncclUint8: return 1;
    case ncclFloat16: case ncclBfloat16: return 2;
    case ncclInt32: case ncclUint32: case ncclFloat32: return 4;
    default: return 8;
  }
}

#ifdef DF_DATAPATH_IMPL
template <typename T>
DF_HD void reduce_same(int op, const DataArgs* a) {
  switch (op) {
    case OP_SUM: reduce_copy<T, T, OP_SUM>(a); break;
    case OP_PROD: reduce_copy<T, T, OP_PROD>(a); break;
    case OP_MAX: reduce_copy<T, T, OP_MAX>(a); break;
    default: reduce_copy<T, T, OP_MIN>(a); break;
  }
}

// Returns false when the (in, out, op) combination is not instantiated.
__host__ __device__ bool reduce_dispatch(int inType, int outType, int op, const DataArgs* a) {
  if (inType == outType) {
    switch (inType) {
#ifndef DF_FAST_BUILD
      case ncclInt8: reduce_same<int8_t>(op, a); return true;
      case ncclUint8: reduce_same<uint8_t>(op, a); return true;
      case ncclInt32: reduce_same<int32_t>(op, a); return true;
      case ncclUint32: reduce_same<uint32_t>(op, a); return true;
      case ncclInt64: reduce_same<int64_t>(op, a); return true;
      case ncclUint64: reduce_same<uint64_t>(op, a); return true;
      case ncclFloat16: reduce_same<__half>(op, a); return true;
      case ncclFloat64: reduce_same<double>(op, a); return true;
#endif
      case ncclFloat32: reduce_same<float>(op, a); return true;
      case ncclBfloat16: reduce_same<__nv_bfloat16>(op, a); return true;
      default: return false;
    }
  }
  if (op != OP_SUM) return false;   // fused casts exist for the gradient path only
  if (inType == ncclBfloat16 && outType == ncclFloat32) { reduce_copy<__nv_bfloat16, float, OP_SUM>(a); return true; }
  if (inType == ncclFloat16 && outType == ncclFloat32) { reduce_copy<__half, float, OP_SUM>(a); return true; }
  if (inType == ncclFloat32 && outType == ncclBfloat16) { reduce_copy<float, __nv_bfloat16, OP_SUM>(a); return true; }
  if (inType == ncclFloat32 && outType == ncclFloat16) { reduce_copy<float, __half, OP_SUM>(a); return true; }
  return false;
}

#else
// Defined once, in device/datapath.cu (relocatable device code): every kernel of the library calls the
// same out-of-line bodies instead of compiling its own copy of the 44 variants.
// Returns false when the (in, out, op) combination is not instantiated.
__host__ __device__ bool reduce_dispatch(int inType, int outType, int op, const DataArgs* a);
#endif

// Host-callable check used at prepare time.
inline bool reduceSupported(int inType, int outType, int op) {
  if (inType < 0 || inType >= ncclNumTypes || outType < 0 || outType >= ncclNumTypes) return false;
  if (inType == outType) return op >= OP_SUM && op <= OP_MIN;
  if (op != OP_SUM) return false;
  return ((inType == ncclBfloat16 || inType == ncclFloat16) && outType == ncclFloat32) ||
         (inType == ncclFloat32 && (outType == ncclBfloat16 || outType == ncclFloat16));
}

}  // namespace dfccl
