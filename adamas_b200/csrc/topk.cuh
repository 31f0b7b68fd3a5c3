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
// granules (8 values each) in registers for the whole kernel, together with their sort keys.
// Blocks never read each other's shared memory (remote loads are slow); they push:
//   0. every block zeroes its accumulators; cluster barrier (all blocks have started);
//   1. local histogram of the high key byte; the non-zero bins are added into the `total` array of
//      EVERY block of the cluster with remote shared-memory reductions; cluster barrier; now each
//      block holds the row's histogram and finds the bin of the k-th smallest key by itself;
//   2. the same for the low key byte of the elements inside that bin: the exact cut key and the
//      number of cut-valued elements to take;
//   3. per-thread counts of (key < cut) and (key == cut), warp scan, block scan; every block adds
//      its totals to the `base` of the higher-ranked blocks; cluster barrier; every thread knows the
//      output position of each of its winners and writes them (ascending position order, lower
//      position wins ties).
// -------------------------------------------------------------------------------------------------
constexpr int kTopkClThreads = 256;          // default block size; long rows use 1024
constexpr int kTopkClMaxWarps = 32;

struct TopkClusterShared {
  unsigned local[256];      // this block's histogram of the current pass
  unsigned total[2][256];   // row histogram of pass 0 / pass 1 (filled by all blocks of the cluster)
  unsigned warp_a[kTopkClMaxWarps];
  unsigned warp_b[kTopkClMaxWarps];
  unsigned base_lt;         // winners below the cut in lower-ranked blocks (filled by them)
  unsigned base_eq;
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

// two packed 16-bit values -> two packed sort keys
template <int FORMAT>
__device__ __forceinline__ uint32_t to_key2(uint32_t w) {
  if (FORMAT == 0) {
    if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;          // -0 -> +0
    if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
    const uint32_t neg = ((w >> 15) & 0x00010001u) * 0xffffu;  // 0xffff in the lanes with the sign set
    return w ^ (neg | 0x80008000u);
  }
  return w;
}

// Executed by warp 0 on a 256-bin histogram in shared memory: smallest bin b with
// sum(hist[0..b]) >= want; stores the bin and the count strictly before it.
__device__ __forceinline__ void find_bin256(const unsigned* hist, unsigned want, unsigned* bucket,
                                            unsigned* before) {
  const unsigned lane = threadIdx.x & 31;
  unsigned c[8];
  unsigned s = 0;
  const uint4 a = reinterpret_cast<const uint4*>(hist)[lane * 2];
  const uint4 b = reinterpret_cast<const uint4*>(hist)[lane * 2 + 1];
  c[0] = a.x; c[1] = a.y; c[2] = a.z; c[3] = a.w; c[4] = b.x; c[5] = b.y; c[6] = b.z; c[7] = b.w;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += c[i];
  unsigned incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const unsigned hit = __ballot_sync(0xffffffffu, incl >= want);
  const unsigned first = __ffs(hit) - 1;   // hit != 0: the histogram holds at least `want` elements
  if (lane == first) {
    unsigned run = incl - s;
    int bsel = 7;
    bool found = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (!found) {
        if (run + c[i] >= want) { bsel = i; found = true; } else { run += c[i]; }
      }
    }
    *bucket = lane * 8 + bsel;
    *before = run;
  }
}

template <int FORMAT, int ITEMS, int NT = kTopkClThreads>
__global__ void __launch_bounds__(NT) topk_cluster_kernel(const TopkParams p) {
  constexpr int kWarps = NT / 32;
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ __align__(16) TopkClusterShared sh;

  const unsigned CL = cluster.num_blocks();
  const unsigned cr = cluster.block_rank();
  const int row = blockIdx.x / CL;
  const int tid = threadIdx.x;
  const unsigned lane = tid & 31;
  const unsigned warp = tid >> 5;

  // zero the accumulators that peers will add into, then make sure every block has done so; all of
  // this can run while the kernel that produces `values` is still finishing
  if (tid < 256) {
    sh.local[tid] = 0;
    sh.total[0][tid] = 0;
    sh.total[1][tid] = 0;
  }
  if (tid == 0) { sh.base_lt = 0; sh.base_eq = 0; }

  const uint16_t* rowp = p.values + static_cast<int64_t>(row) * p.value_stride;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(rowp);
  const int lead = static_cast<int>((addr & 15) >> 1);
  const uint4* gbase = reinterpret_cast<const uint4*>(addr & ~static_cast<uintptr_t>(15));
  const int G = (lead + p.n + 7) >> 3;
  const int end = lead + p.n;
  const int blk_first = cr * p.granules_per_block;
  const int blk_end = min(G, blk_first + p.granules_per_block);
  const int g0 = blk_first + tid * ITEMS;
  cluster.sync();
  grid_dependency_wait();
  grid_launch_dependents();

  // this thread's granules: g0 .. g0 + ITEMS - 1 (inside the block's range and the row)
  uint32_t raw[ITEMS][4];
  uint32_t key[ITEMS][4];
  unsigned vmask[ITEMS];   // bit j: element j of the granule belongs to the row
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    uint4 v = make_uint4(0, 0, 0, 0);
    unsigned m = 0;
    const int g = g0 + i;
    if (g < blk_end) {
      v = ld_16(gbase + g);
      const int e0 = g * 8;
      m = 0xffu;
      if (e0 < lead) m &= 0xffu << (lead - e0);
      if (e0 + 8 > end) m &= 0xffu >> (e0 + 8 - end);
    }
    raw[i][0] = v.x; raw[i][1] = v.y; raw[i][2] = v.z; raw[i][3] = v.w;
#pragma unroll
    for (int q = 0; q < 4; ++q) key[i][q] = to_key2<FORMAT>(raw[i][q]);
    vmask[i] = m;
  }

  unsigned prefix = 0;                              // key bits decided so far
  unsigned want = static_cast<unsigned>(p.k);
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    // local histogram of the pass's byte
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      if (pass == 0) {
        // a whole warp holding one single value (degenerate inputs) adds it with one update
        const bool same = vmask[i] == 0xffu && key[i][0] == key[i][1] && key[i][1] == key[i][2] &&
                          key[i][2] == key[i][3] && (key[i][0] >> 16) == (key[i][0] & 0xffffu);
        const unsigned first = __shfl_sync(0xffffffffu, key[i][0], 0);
        if (__all_sync(0xffffffffu, same && key[i][0] == first)) {
          if (lane == 0) atomicAdd(&sh.local[(first >> 8) & 0xffu], 256u);
          continue;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const unsigned k16 = (key[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        bool ok = (vmask[i] >> j) & 1u;
        unsigned bin = k16 >> 8;
        if (pass == 1) {
          ok = ok && bin == prefix;
          bin = k16 & 0xffu;
        }
        if (ok) atomicAdd(&sh.local[bin], 1u);
      }
    }
    __syncthreads();
    // push the non-zero bins to every block of the cluster (including this one)
    if (tid < 256) {
      const unsigned c = sh.local[tid];
      if (c != 0) {
        for (unsigned r = 0; r < CL; ++r) atomicAdd(cluster.map_shared_rank(&sh.total[pass][tid], r), c);
      }
      sh.local[tid] = 0;
    }
    cluster.sync();
    if (warp == 0) find_bin256(sh.total[pass], want, &sh.bucket, &sh.before);
    __syncthreads();
    prefix = (prefix << 8) | sh.bucket;
    want -= sh.before;
    __syncthreads();   // bucket / before are rewritten in the next pass
  }
  const unsigned cut = prefix;
  const unsigned need_eq = want;

  // ---- counts, scans ---------------------------------------------------------------------------------
  unsigned c_lt = 0, c_eq = 0;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned k16 = (key[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu;
      const bool ok = (vmask[i] >> j) & 1u;
      c_lt += (ok && k16 < cut);
      c_eq += (ok && k16 == cut);
    }
  }
  unsigned i_lt = c_lt, i_eq = c_eq;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned a = __shfl_up_sync(0xffffffffu, i_lt, o);
    const unsigned b = __shfl_up_sync(0xffffffffu, i_eq, o);
    if (lane >= o) { i_lt += a; i_eq += b; }
  }
  if (lane == 31) { sh.warp_a[warp] = i_lt; sh.warp_b[warp] = i_eq; }
  __syncthreads();
  unsigned base_lt = 0, base_eq = 0, blk_lt = 0, blk_eq = 0;
#pragma unroll
  for (unsigned w2 = 0; w2 < kWarps; ++w2) {
    const unsigned a = sh.warp_a[w2], b = sh.warp_b[w2];
    if (w2 < warp) { base_lt += a; base_eq += b; }
    blk_lt += a; blk_eq += b;
  }
  // this block's totals go to the bases of all higher-ranked blocks
  if (tid < 2) {
    const unsigned v = tid == 0 ? blk_lt : blk_eq;
    if (v != 0)
      for (unsigned r = cr + 1; r < CL; ++r)
        atomicAdd(cluster.map_shared_rank(tid == 0 ? &sh.base_lt : &sh.base_eq, r), v);
  }
  cluster.sync();
  unsigned run_lt = sh.base_lt + base_lt + i_lt - c_lt;
  unsigned run_eq = sh.base_eq + base_eq + i_eq - c_eq;

  // ---- emit -------------------------------------------------------------------------------------------
  if (c_lt | c_eq) {
    const int32_t* idx_row = p.in_idx ? p.in_idx + static_cast<int64_t>(row) * p.in_idx_stride : nullptr;
    int32_t* oi = p.out_idx + static_cast<int64_t>(row) * p.out_stride;
    uint16_t* ov = p.out_values ? p.out_values + static_cast<int64_t>(row) * p.out_stride : nullptr;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const unsigned k16 = (key[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        if (((vmask[i] >> j) & 1u) && k16 <= cut) {
          int pos = -1;
          if (k16 < cut) {
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
            if (ov) ov[pos] = static_cast<uint16_t>((raw[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu);
          }
        }
      }
    }
  }
}

}  // namespace adamas
