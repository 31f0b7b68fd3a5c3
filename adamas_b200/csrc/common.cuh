// Shared device helpers for the Adamas decode-path kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace adamas {

// One sequence of a batched decode step: its caches and page tables.  An array of these lives in device
// memory (one entry per sequence); a kernel of a batched launch picks its entry by a grid coordinate.
// Everything else of a batched step (q, k, v, o, query codes, distances, histogram scratch, index lists)
// is one contiguous array over (sequence, head) rows, and the sequence lengths are an int32 array.
struct SeqDesc {
  void* kv_data;
  void* code_data;
  const int32_t* kv_table;
  const int32_t* code_table;
};


constexpr int kHeadDim = 128;           // the only head dimension the path supports
constexpr int kCodeWords = kHeadDim / 8;  // 16-bit words per (token, head) code = 32 bytes

// ---- 16-byte global loads / stores ---------------------------------------------------------
// Streaming read of data that is read once (code cache): bypass L1 allocation.
__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// ---- cp.async (16 B, L2 only) --------------------------------------------------------------
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  unsigned s = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// ---- programmatic dependent launch -----------------------------------------------------------
// A kernel launched with the programmatic-serialization attribute may start while its predecessor in
// the stream is still running.  grid_dependency_wait() returns once the predecessor has completed
// and its writes are visible; everything before it may only touch data that was final before the
// predecessor started.  grid_launch_dependents() lets the successor's blocks be scheduled as this
// grid's blocks retire.  Both are no-ops for a normal launch.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- mbarrier + bulk (TMA) copy, global -> shared ---------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One poll: the thread may sleep inside the instruction until the phase completes or about kMbarSuspendNs
// have passed (a hint), so that waiting warps do not fill the issue slots of the working ones with polls.
constexpr unsigned kMbarSuspendNs = 1000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kMbarSuspendNs)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself suspend for a while) and reports
// failure instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, unsigned limit) {
  for (unsigned spin = 0; spin < limit; ++spin)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// 1-D bulk copy of `bytes` (multiple of 16; src and dst 16-byte aligned); completion is signalled on
// `bar` as transaction bytes.
__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gmem_src, unsigned bytes,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---- element conversion: 8 x 16-bit storage <-> 8 x fp32 -----------------------------------
template <typename T>
struct Elem;
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float2 to_f2(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
  }
  static __device__ __forceinline__ uint32_t from_f2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float round(float a) { return __half2float(__float2half_rn(a)); }
  // c + a.lo * b.lo + a.hi * b.hi on two packed pairs, in that order, each step one fused multiply-add
  // in fp32 on the 16-bit operands (mixed-precision fma of sm_100: the same result as converting
  // first, without the conversions)
  static __device__ __forceinline__ float dot2(uint32_t a, uint32_t b, float c) {
    float d;
    asm("{\n\t.reg .b16 alo, ahi, blo, bhi;\n\t"
        "mov.b32 {alo, ahi}, %1;\n\t"
        "mov.b32 {blo, bhi}, %2;\n\t"
        "fma.rn.f32.f16 %0, alo, blo, %3;\n\t"
        "fma.rn.f32.f16 %0, ahi, bhi, %0;\n\t}"
        : "=f"(d)
        : "r"(a), "r"(b), "f"(c));
    return d;
  }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float2 to_f2(uint32_t u) {
    // bf16 -> fp32 is a 16-bit shift
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
  }
  static __device__ __forceinline__ uint32_t from_f2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float round(float a) {
    return __bfloat162float(__float2bfloat16_rn(a));
  }
  static __device__ __forceinline__ float dot2(uint32_t a, uint32_t b, float c) {
    float d;
    asm("{\n\t.reg .b16 alo, ahi, blo, bhi;\n\t"
        "mov.b32 {alo, ahi}, %1;\n\t"
        "mov.b32 {blo, bhi}, %2;\n\t"
        "fma.rn.f32.bf16 %0, alo, blo, %3;\n\t"
        "fma.rn.f32.bf16 %0, ahi, bhi, %0;\n\t}"
        : "=f"(d)
        : "r"(a), "r"(b), "f"(c));
    return d;
  }
};

template <typename T>
__device__ __forceinline__ void unpack8(uint4 v, float (&x)[8]) {
  float2 a = Elem<T>::to_f2(v.x), b = Elem<T>::to_f2(v.y), c = Elem<T>::to_f2(v.z),
         d = Elem<T>::to_f2(v.w);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
  x[4] = c.x; x[5] = c.y; x[6] = d.x; x[7] = d.y;
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  uint4 v;
  v.x = Elem<T>::from_f2(x[0], x[1]);
  v.y = Elem<T>::from_f2(x[2], x[3]);
  v.z = Elem<T>::from_f2(x[4], x[5]);
  v.w = Elem<T>::from_f2(x[6], x[7]);
  return v;
}

// Device-side error flags, readable through adamas_device_error().  A kernel that gives up on a
// bounded wait sets a bit here and finishes normally.
__device__ unsigned g_adamas_error = 0;
constexpr unsigned kErrEstimateTimeout = 1u;
constexpr unsigned kErrDecodeTimeout = 2u;
constexpr unsigned kErrGatherTimeout = 4u;
constexpr unsigned kErrHistogram = 8u;   // select_attend found histograms that do not describe its row

struct Thresholds {
  float t0, t1, t2;
};

}  // namespace adamas
