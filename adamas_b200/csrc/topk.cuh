// Stage 3 of the decode path: per row, the k smallest of n 16-bit values, ties resolved towards
// the lower position, results emitted in ascending position order (deterministic).
//
// One thread block per row.  The row is staged once into shared memory (when it fits) as raw
// 16-byte granules; a value's sort key is an order-preserving map to uint16.  Selection is a
// two-pass radix select on the key (high byte, then low byte) with warp-aggregated shared-memory
// histogram updates (match.any), followed by an ordered compaction: every warp owns a contiguous
// range of granules, counts its (key < cut) and (key == cut) elements, a block scan of the 32 warp
// totals gives each warp its output base, and a second sweep writes the winners using warp prefix
// sums only.  No global scratch memory and no atomics on global memory are used.
#pragma once
#include "common.cuh"

namespace adamas {

constexpr int kTopkThreads = 1024;
constexpr int kTopkWarps = kTopkThreads / 32;

template <int FORMAT>
__device__ __forceinline__ unsigned to_key(unsigned raw) {
  if (FORMAT == 0) {  // fp16: fold -0 onto +0, flip negatives, set the sign bit of the rest
    if (raw == 0x8000u) raw = 0;
    return (raw & 0x8000u) ? (~raw & 0xffffu) : (raw | 0x8000u);
  }
  return raw;
}

struct TopkShared {
  unsigned hist[256];
  unsigned warp_lt[kTopkWarps];
  unsigned warp_eq[kTopkWarps];
  unsigned bucket;
  unsigned before;
};

// Executed by warp 0: smallest bucket b with sum(hist[0..b]) >= want; writes bucket and the count
// strictly before it.
__device__ __forceinline__ void find_bucket(TopkShared& sh, unsigned want) {
  const unsigned lane = threadIdx.x & 31;
  unsigned c[8];
  unsigned s = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    c[i] = sh.hist[lane * 8 + i];
    s += c[i];
  }
  unsigned incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const unsigned excl = incl - s;
  const unsigned hit = __ballot_sync(0xffffffffu, incl >= want);
  const unsigned first = __ffs(hit) - 1;  // hit != 0 because want <= total
  if (lane == first) {
    unsigned run = excl;
    int b = 7;
    bool found = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!found) {
        if (run + c[i] >= want) {
          b = i;
          found = true;
        } else {
          run += c[i];
        }
      }
    }
    // found is guaranteed since excl + sum(c) >= want
    sh.bucket = lane * 8 + b;
    sh.before = run;
  }
}

// values: row-major 16-bit; rows may start at any 2-byte boundary.
template <int FORMAT>
__global__ void __launch_bounds__(kTopkThreads)
topk_kernel(const uint16_t* __restrict__ values, int64_t value_stride, int n,
            const int32_t* __restrict__ in_idx, int64_t in_idx_stride, int idx_page_size, int k,
            uint16_t* __restrict__ out_values, int32_t* __restrict__ out_idx, int64_t out_stride,
            int smem_granules) {
  extern __shared__ uint4 staged[];
  __shared__ TopkShared sh;

  const int row = blockIdx.x;
  const unsigned lane = threadIdx.x & 31;
  const unsigned warp = threadIdx.x >> 5;

  const uint16_t* rowp = values + static_cast<int64_t>(row) * value_stride;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(rowp);
  const int lead = static_cast<int>((addr & 15) >> 1);  // elements of the first granule before the row
  const uint4* gbase = reinterpret_cast<const uint4*>(addr & ~static_cast<uintptr_t>(15));
  const int G = (lead + n + 7) >> 3;  // granules covering the row
  const int end = lead + n;           // valid granule-space element range is [lead, end)

  const uint4* src = gbase;
  if (G <= smem_granules) {
    for (int g = threadIdx.x; g < G; g += kTopkThreads) staged[g] = ld_16(gbase + g);
    src = staged;
  }
  for (int i = threadIdx.x; i < 256; i += kTopkThreads) sh.hist[i] = 0;
  __syncthreads();

  // ---- radix pass on the high byte, then on the low byte within the chosen bucket -------------
  unsigned prefix_hi = 0;
  unsigned want = static_cast<unsigned>(k);
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    const int G32 = (G + 31) & ~31;
    for (int g = threadIdx.x; g < G32; g += kTopkThreads) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (g < G) v = src[g];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = g * 8 + j;
        const unsigned key = to_key<FORMAT>((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
        bool ok = (g < G) && e >= lead && e < end;
        unsigned bin;
        if (pass == 0) {
          bin = key >> 8;
        } else {
          ok = ok && (key >> 8) == prefix_hi;
          bin = key & 0xffu;
        }
        const unsigned tag = ok ? bin : (0x100u + lane);
        const unsigned peers = __match_any_sync(0xffffffffu, tag);
        if (ok && lane == static_cast<unsigned>(__ffs(peers) - 1)) atomicAdd(&sh.hist[bin], __popc(peers));
      }
    }
    __syncthreads();
    if (warp == 0) find_bucket(sh, want);
    __syncthreads();
    const unsigned bucket = sh.bucket;
    want -= sh.before;
    if (pass == 0) {
      prefix_hi = bucket;
      __syncthreads();
      for (int i = threadIdx.x; i < 256; i += kTopkThreads) sh.hist[i] = 0;
      __syncthreads();
    } else {
      prefix_hi = (prefix_hi << 8) | bucket;
    }
  }
  const unsigned cut = prefix_hi;   // key of the k-th smallest element
  const unsigned need_eq = want;    // how many elements equal to the cut are taken (>= 1)

  // ---- ordered compaction ------------------------------------------------------------------------
  const int Gw = (G + kTopkWarps - 1) / kTopkWarps;  // granules per warp (contiguous range)
  const int g0 = warp * Gw;
  const int iters = (Gw + 31) >> 5;

  unsigned my_lt = 0, my_eq = 0;
  for (int it = 0; it < iters; ++it) {
    const int gi = it * 32 + lane;
    const int g = g0 + gi;
    if (gi < Gw && g < G) {
      const uint4 v = src[g];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = g * 8 + j;
        const unsigned key = to_key<FORMAT>((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
        const bool ok = e >= lead && e < end;
        my_lt += (ok && key < cut);
        my_eq += (ok && key == cut);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    my_lt += __shfl_xor_sync(0xffffffffu, my_lt, o);
    my_eq += __shfl_xor_sync(0xffffffffu, my_eq, o);
  }
  if (lane == 0) {
    sh.warp_lt[warp] = my_lt;
    sh.warp_eq[warp] = my_eq;
  }
  __syncthreads();
  unsigned base_lt = 0, base_eq = 0;
  for (unsigned w2 = 0; w2 < warp; ++w2) {
    base_lt += sh.warp_lt[w2];
    base_eq += sh.warp_eq[w2];
  }

  const int32_t* idx_row = in_idx ? in_idx + static_cast<int64_t>(row) * in_idx_stride : nullptr;
  int32_t* oi = out_idx + static_cast<int64_t>(row) * out_stride;
  uint16_t* ov = out_values ? out_values + static_cast<int64_t>(row) * out_stride : nullptr;

  for (int it = 0; it < iters; ++it) {
    const int gi = it * 32 + lane;
    const int g = g0 + gi;
    const bool have = gi < Gw && g < G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (have) v = src[g];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    unsigned c_lt = 0, c_eq = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = g * 8 + j;
      const unsigned key = to_key<FORMAT>((w[j >> 1] >> ((j & 1) * 16)) & 0xffffu);
      const bool ok = have && e >= lead && e < end;
      c_lt += (ok && key < cut);
      c_eq += (ok && key == cut);
    }
    // warp exclusive scan of both counts (each <= 8 per lane, <= 256 per warp: 16 bits suffice)
    const unsigned packed = c_lt | (c_eq << 16);
    unsigned incl = packed;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned excl = incl - packed;
    const unsigned total = __shfl_sync(0xffffffffu, incl, 31);
    unsigned run_lt = base_lt + (excl & 0xffffu);
    unsigned run_eq = base_eq + (excl >> 16);
    if (c_lt | c_eq) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = g * 8 + j;
        const unsigned raw = (w[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        const unsigned key = to_key<FORMAT>(raw);
        const bool ok = e >= lead && e < end;
        if (ok && key <= cut) {
          int pos = -1;
          if (key < cut) {
            pos = static_cast<int>(run_lt + min(run_eq, need_eq));
            ++run_lt;
          } else {
            if (run_eq < need_eq) pos = static_cast<int>(run_lt + run_eq);
            ++run_eq;
          }
          if (pos >= 0) {
            const int p = e - lead;
            int32_t id = p;
            if (idx_row) {
              const int pg = p / idx_page_size;
              id = __ldg(idx_row + pg) * idx_page_size + (p - pg * idx_page_size);
            }
            oi[pos] = id;
            if (ov) ov[pos] = static_cast<uint16_t>(raw);
          }
        }
      }
    }
    base_lt += total & 0xffffu;
    base_eq += total >> 16;
  }
}

}  // namespace adamas
