// Stage 3 of the decode path: per row, the k smallest of n 16-bit values, ties resolved towards
// the lower position, results emitted in ascending position order (deterministic).
//
// Two kernels.  topk_cluster_kernel (rows up to 262144 values) spreads a row over a thread-block
// cluster and keeps every value in registers; it is described at its definition.  topk_kernel is
// the single-block fallback for longer rows:
//
// One thread block per row.  The row is staged once into shared memory (when it fits) as raw
// 16-byte granules; a value's sort key is an order-preserving map to uint16.  Selection is a
// two-pass radix select on the key (high byte, then low byte) into per-warp private shared-memory
// histograms (no contention between warps; a warp whose 32 elements fall into one bin adds them with
// a single update), followed by an ordered compaction: every warp owns a contiguous
// range of granules, counts its (key < cut) and (key == cut) elements, a block scan of the 32 warp
// totals gives each warp its output base, and a second sweep writes the winners using warp prefix
// sums only.  No global scratch memory and no atomics on global memory are used.
#pragma once
#include <cooperative_groups.h>

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
  unsigned whist[kTopkWarps][256];   // per-warp private histograms
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
  __syncthreads();

  // ---- radix pass on the high byte, then on the low byte within the chosen bucket -------------
  unsigned prefix_hi = 0;
  unsigned want = static_cast<unsigned>(k);
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    for (int i = lane; i < 256; i += 32) sh.whist[warp][i] = 0;
    __syncwarp();
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
        const unsigned tag = ok ? bin : 0xffffu;
        const unsigned first = __shfl_sync(0xffffffffu, tag, 0);
        if (__all_sync(0xffffffffu, tag == first)) {
          if (lane == 0 && first != 0xffffu) atomicAdd(&sh.whist[warp][first], 32u);
        } else if (ok) {
          atomicAdd(&sh.whist[warp][bin], 1u);
        }
      }
    }
    __syncthreads();
    if (threadIdx.x < 256) {
      unsigned s = 0;
#pragma unroll
      for (int w2 = 0; w2 < kTopkWarps; ++w2) s += sh.whist[w2][threadIdx.x];
      sh.hist[threadIdx.x] = s;
    }
    __syncthreads();
    if (warp == 0) find_bucket(sh, want);
    __syncthreads();
    const unsigned bucket = sh.bucket;
    want -= sh.before;
    prefix_hi = (pass == 0) ? bucket : ((prefix_hi << 8) | bucket);
    __syncthreads();
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


// -------------------------------------------------------------------------------------------------
// Cluster kernel.  A row is split over the CL thread blocks of a cluster (CL = 1, 2, 4 or 8); block
// `cr` owns a contiguous range of 16-byte granules and every thread holds ITEMS consecutive
// granules (8 values each) in registers for the whole kernel.
//   1. histogram of the top 12 key bits in shared memory (4096 bins); cluster barrier; every block
//      sums the CL histograms through distributed shared memory and scans them to find the bin that
//      holds the k-th smallest key;
//   2. histogram of the low 4 key bits inside that bin (16 bins); cluster barrier; same reduction:
//      the exact cut key and the number of cut-valued elements to take;
//   3. per-thread counts of (key < cut) and (key == cut), warp scan, block scan, cluster barrier,
//      sum of the totals of the lower-ranked blocks: every thread knows the output position of each
//      of its winners and writes them (ascending position order, lower position wins ties).
// A final cluster barrier keeps every block's shared memory alive until its peers have read it.
// -------------------------------------------------------------------------------------------------
struct TopkClusterShared {
  unsigned hist[4096];
  unsigned hist2[16];
  unsigned warp_a[kTopkWarps];
  unsigned warp_b[kTopkWarps];
  unsigned tot_lt;
  unsigned tot_eq;
  unsigned bucket;
  unsigned before;
};

struct TopkParams {
  const uint16_t* values;
  int64_t value_stride;
  int n;
  const int32_t* in_idx;
  int64_t in_idx_stride;
  int idx_page_size;
  int idx_ps_shift;   // log2(idx_page_size) or -1
  int k;
  uint16_t* out_values;
  int32_t* out_idx;
  int64_t out_stride;
  int granules_per_block;
};

template <int FORMAT, int ITEMS>
__global__ void __launch_bounds__(kTopkThreads) topk_cluster_kernel(const TopkParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ TopkClusterShared sh;

  const unsigned CL = cluster.num_blocks();
  const unsigned cr = cluster.block_rank();
  const int row = blockIdx.x / CL;
  const int tid = threadIdx.x;
  const unsigned lane = tid & 31;
  const unsigned warp = tid >> 5;

  const uint16_t* rowp = p.values + static_cast<int64_t>(row) * p.value_stride;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(rowp);
  const int lead = static_cast<int>((addr & 15) >> 1);
  const uint4* gbase = reinterpret_cast<const uint4*>(addr & ~static_cast<uintptr_t>(15));
  const int G = (lead + p.n + 7) >> 3;
  const int end = lead + p.n;

  // this thread's granules: g0 .. g0 + ITEMS - 1 (inside the block's range and the row)
  const int blk_first = cr * p.granules_per_block;
  const int blk_end = min(G, blk_first + p.granules_per_block);
  const int g0 = blk_first + tid * ITEMS;
  uint4 v[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    v[i] = make_uint4(0, 0, 0, 0);
    if (g0 + i < blk_end) v[i] = ld_16(gbase + g0 + i);
  }
  for (int i = tid; i < 4096; i += kTopkThreads) sh.hist[i] = 0;
  if (tid < 16) sh.hist2[tid] = 0;
  __syncthreads();

  // element accessors
  auto raw_of = [&](int i, int j) -> unsigned {
    const uint32_t w = (j >> 1) == 0 ? v[i].x : (j >> 1) == 1 ? v[i].y : (j >> 1) == 2 ? v[i].z : v[i].w;
    return (w >> ((j & 1) * 16)) & 0xffffu;
  };
  auto valid = [&](int i, int j) -> bool {
    const int e = (g0 + i) * 8 + j;
    return (g0 + i < blk_end) && e >= lead && e < end;
  };

  // ---- pass 1: top 12 bits ------------------------------------------------------------------
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    // a whole warp holding one single value (degenerate inputs) adds it with one update
    const bool full = (g0 + i < blk_end) && (g0 + i) * 8 >= lead && (g0 + i) * 8 + 8 <= end;
    const bool same = full && v[i].x == v[i].y && v[i].y == v[i].z && v[i].z == v[i].w &&
                      (v[i].x >> 16) == (v[i].x & 0xffffu);
    const unsigned first = __shfl_sync(0xffffffffu, v[i].x, 0);
    if (__all_sync(0xffffffffu, same && v[i].x == first)) {
      if (lane == 0) atomicAdd(&sh.hist[to_key<FORMAT>(first & 0xffffu) >> 4], 256u);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (valid(i, j)) atomicAdd(&sh.hist[to_key<FORMAT>(raw_of(i, j)) >> 4], 1u);
    }
  }
  cluster.sync();

  // cluster-wide histogram of this thread's 4 bins, block scan, locate the k-th key's bin
  {
    unsigned c[4] = {0, 0, 0, 0};
    for (unsigned r = 0; r < CL; ++r) {
      const unsigned* rh = cluster.map_shared_rank(sh.hist, r);
      const uint4 t = *reinterpret_cast<const uint4*>(rh + tid * 4);
      c[0] += t.x; c[1] += t.y; c[2] += t.z; c[3] += t.w;
    }
    const unsigned s = c[0] + c[1] + c[2] + c[3];
    unsigned incl = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) sh.warp_a[warp] = incl;
    __syncthreads();
    unsigned wbase = 0;
    for (unsigned w2 = 0; w2 < warp; ++w2) wbase += sh.warp_a[w2];
    const unsigned excl = wbase + incl - s;
    const unsigned want = static_cast<unsigned>(p.k);
    if (excl < want && excl + s >= want) {   // exactly one thread
      unsigned run = excl;
      int b = 3;
      bool found = false;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (!found) {
          if (run + c[i] >= want) { b = i; found = true; } else { run += c[i]; }
        }
      }
      sh.bucket = tid * 4 + b;
      sh.before = run;
    }
    __syncthreads();
  }
  const unsigned bucket12 = sh.bucket;
  unsigned want = static_cast<unsigned>(p.k) - sh.before;

  // ---- pass 2: low 4 bits inside the bin ----------------------------------------------------------
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned key = to_key<FORMAT>(raw_of(i, j));
      if (valid(i, j) && (key >> 4) == bucket12) atomicAdd(&sh.hist2[key & 15u], 1u);
    }
  }
  cluster.sync();
  if (warp == 0) {
    unsigned c = 0;
    if (lane < 16)
      for (unsigned r = 0; r < CL; ++r) c += cluster.map_shared_rank(sh.hist2, r)[lane];
    unsigned incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, incl >= want);
    const unsigned firstl = __ffs(hit) - 1;
    if (lane == firstl) {
      sh.bucket = (bucket12 << 4) | lane;
      sh.before = incl - c;
    }
  }
  __syncthreads();
  const unsigned cut = sh.bucket;
  const unsigned need_eq = want - sh.before;

  // ---- counts, scans ---------------------------------------------------------------------------------
  unsigned c_lt = 0, c_eq = 0;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned key = to_key<FORMAT>(raw_of(i, j));
      const bool ok = valid(i, j);
      c_lt += (ok && key < cut);
      c_eq += (ok && key == cut);
    }
  }
  unsigned i_lt = c_lt, i_eq = c_eq;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned a = __shfl_up_sync(0xffffffffu, i_lt, o);
    const unsigned b = __shfl_up_sync(0xffffffffu, i_eq, o);
    if (lane >= o) { i_lt += a; i_eq += b; }
  }
  __syncthreads();   // warp_a is reused
  if (lane == 31) { sh.warp_a[warp] = i_lt; sh.warp_b[warp] = i_eq; }
  __syncthreads();
  unsigned base_lt = 0, base_eq = 0, blk_lt = 0, blk_eq = 0;
  for (unsigned w2 = 0; w2 < kTopkWarps; ++w2) {
    const unsigned a = sh.warp_a[w2], b = sh.warp_b[w2];
    if (w2 < warp) { base_lt += a; base_eq += b; }
    blk_lt += a; blk_eq += b;
  }
  if (tid == 0) { sh.tot_lt = blk_lt; sh.tot_eq = blk_eq; }
  cluster.sync();
  for (unsigned r = 0; r < cr; ++r) {
    base_lt += *cluster.map_shared_rank(&sh.tot_lt, r);
    base_eq += *cluster.map_shared_rank(&sh.tot_eq, r);
  }
  unsigned run_lt = base_lt + i_lt - c_lt;
  unsigned run_eq = base_eq + i_eq - c_eq;

  // ---- emit -------------------------------------------------------------------------------------------
  if (c_lt | c_eq) {
    const int32_t* idx_row = p.in_idx ? p.in_idx + static_cast<int64_t>(row) * p.in_idx_stride : nullptr;
    int32_t* oi = p.out_idx + static_cast<int64_t>(row) * p.out_stride;
    uint16_t* ov = p.out_values ? p.out_values + static_cast<int64_t>(row) * p.out_stride : nullptr;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const unsigned raw = raw_of(i, j);
        const unsigned key = to_key<FORMAT>(raw);
        if (valid(i, j) && key <= cut) {
          int pos = -1;
          if (key < cut) {
            pos = static_cast<int>(run_lt + min(run_eq, need_eq));
            ++run_lt;
          } else {
            if (run_eq < need_eq) pos = static_cast<int>(run_lt + run_eq);
            ++run_eq;
          }
          if (pos >= 0) {
            const int pp = (g0 + i) * 8 + j - lead;
            int32_t id = pp;
            if (idx_row) {
              int pg, off;
              if (p.idx_ps_shift >= 0) {
                pg = pp >> p.idx_ps_shift;
                off = pp & (p.idx_page_size - 1);
              } else {
                pg = pp / p.idx_page_size;
                off = pp - pg * p.idx_page_size;
              }
              id = __ldg(idx_row + pg) * p.idx_page_size + off;
            }
            oi[pos] = id;
            if (ov) ov[pos] = static_cast<uint16_t>(raw);
          }
        }
      }
    }
  }
  cluster.sync();   // peers may still be reading this block's totals
}

}  // namespace adamas
