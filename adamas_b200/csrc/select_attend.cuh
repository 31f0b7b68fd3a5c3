// Stages 3 + 4 of the decode path in one kernel: per head, pick the k smallest of n integer distances
// (ties to the lower position) and run the decode attention over the picked tokens plus the newest
// token.  Used by the fused decode step; the separate top-k and decode kernels remain for callers
// that want the stages one by one.
//
// One thread-block cluster (CL <= 8 blocks x 512 threads) per head.  Block `cr` owns a contiguous
// slice of the head's distance row, keeps it in registers, and later attends over the winners that
// lie in its own slice, so the selected indices never travel between blocks:
//   pre   clear the local histogram and ARRIVE at a cluster barrier without waiting ("I have
//         started"); all of this may overlap the tail of the estimate kernel (programmatic dependent
//         launch);
//   1     histogram of the block's distances (values < 512: a distance is at most 3 * 128); the wait
//         half of the start-up barrier (every peer is running by now); the whole histogram, packed
//         to 16-bit counts, is STORED into slot `cr` of every peer's per-source table with one
//         16-byte remote store per thread (nothing has to be zeroed); cluster barrier.  Every block
//         now holds all CL histograms and derives by itself: the cut distance, how many cut-valued
//         elements are taken in all, how many of them and how many smaller elements lie in
//         lower-ranked slices (= its tie quota and its offset in the output list);
//   2     ordered compaction of the block's winners into a shared-memory list (and, optionally, to
//         the global index list at the right offset);
//   3     attention over the list in tiles of `tile_cap` (64, 128 or 192) tokens, chosen by the host so
//         that a block's winners almost always fit one tile: K/V rows gathered with one 256-byte
//         bulk (TMA) copy per row, counted by an mbarrier (bounded wait), four threads per token
//         for q.K (odd and even tokens walk their chunks in different orders, which keeps the
//         un-padded rows free of bank conflicts), online softmax in base 2, one thread per (group
//         of tile_cap/32 tokens, 8-dim chunk) for P.V;
//   4     the partial (o, m, l) is stored into slot `cr` of rank 0's shared memory; cluster barrier;
//         rank 0 merges the CL partials and writes the head's output.
// Only two cluster barriers sit on the critical path.  The histogram tables and the per-warp partial
// outputs live in the K/V tile memory, which is idle before and after phase 3.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace adamas {

constexpr int kSaThreads = 512;
constexpr int kSaMaxWarps = kSaThreads / 32;
constexpr int kSaBins = 512;
constexpr int kSaTile = 128;          // planning unit of the host (winners per block it aims for)
constexpr int kSaMaxTpg = 6;          // tokens per P.V group at most
constexpr int kSaTileMax = kSaMaxTpg * kSaThreads / 16;   // largest attention tile: 192 tokens
constexpr int kSaMaxCluster = 8;      // portable cluster size
constexpr int kSaBigCluster = 16;     // non-portable: long rows of few heads (see the host code)

struct SelectAttendParams {
  const uint16_t* dist;     // [H, dist_stride] u16 distances, rows 16-byte aligned
  int64_t dist_stride;
  int n;                    // distances per head (tokens 0 .. n-1)
  int k;                    // winners per head, 1 <= k <= n
  const void* q;            // [H, 128]; read after the preceding kernel has completed
  void* o;                  // [H, 128]
  float* lse;               // [H] or null (base 2)
  const void* kv;           // [pages, 2, page_size, H, 128]
  const int32_t* kv_table;  // logical page -> physical page
  int page_size;
  int ps_shift;             // log2(page_size) or -1
  int H;
  unsigned tail_slot;       // physical slot of the newest token (always attended)
  int32_t* out_idx;         // optional [H, out_stride]: physical slots of the winners, ascending position
  int64_t out_stride;
  int granules_per_block;   // 16-byte granules (8 distances) of a row per block
  int list_capacity;        // entries of the shared-memory winner list
  int tile_cap;             // tokens per attention tile: 64, 128 or 192
  int trace_tag;            // launch number, used by builds with phase timing only
  float scale_log2;
};

struct SaShared {
  float s_logit[kSaTileMax];
  float s_p[kSaTileMax];
  float s_red[kSaMaxWarps];
  float s_sum[kSaTileMax / 32];
  unsigned warp_a[kSaMaxWarps];
  unsigned warp_b[kSaMaxWarps];
  unsigned cut, before, lt_before, eq_before;
};

// The two halves of a cluster barrier (all threads of all blocks of the cluster execute both).
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Dynamic shared memory: K tile (tile_cap * 256 B) | V tile (same) | winner list (list_capacity * 4 B,
// rounded up to 16) | rank 0's table of the blocks' partial results (CL * 130 floats).
// The first 2 KB + CL KB double as the histogram tables (local: 512 x u32; per source block: CL x 512 x
// u16) until phase 3 starts, the first 8 KB as the warps' partial outputs after it has ended.
template <typename T, int ITEMS>
__global__ void __launch_bounds__(kSaThreads, 2) select_attend_kernel(const SelectAttendParams p) {
  constexpr int NT = kSaThreads;
  static_assert(NT >= kSaBins, "one histogram bin per thread");
  constexpr int kWarps = NT / 32;
  constexpr int kGroups = NT / 16;        // P.V token groups per tile
  constexpr int kQkTokens = NT / 4;       // tokens per q.K pass
  constexpr int kCapMax = kSaMaxTpg * kGroups;
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ __align__(16) uint8_t sa_smem[];
  __shared__ __align__(16) SaShared sh;
  __shared__ __align__(8) uint64_t gather_bar;

  const unsigned CL = cluster.num_blocks();
  const unsigned cr = cluster.block_rank();
  const int head = blockIdx.x / CL;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int H = p.H;
  const int cap = p.tile_cap;

  uint8_t* sk = sa_smem;
  uint8_t* sv = sa_smem + cap * 256;
  int32_t* s_list = reinterpret_cast<int32_t*>(sa_smem + 2 * cap * 256);
  float* part_o = reinterpret_cast<float*>(sa_smem + 2 * cap * 256 + ((p.list_capacity * 4 + 15) & ~15));  // [CL][128]
  float* part_ml = part_o + CL * kHeadDim;                                                                  // [CL][2]
  unsigned* h_local = reinterpret_cast<unsigned*>(sa_smem);
  uint16_t* h_src = reinterpret_cast<uint16_t*>(sa_smem + kSaBins * 4);
  float(*s_o)[kHeadDim] = reinterpret_cast<float(*)[kHeadDim]>(sa_smem);

  // ---- pre ------------------------------------------------------------------------------------------
  ADAMAS_STAMP(1, 0, tid == 0);
  ADAMAS_TRACE(1, p.trace_tag, 0, tid == 0);
  ADAMAS_CHAIN(2, 0, false, blockIdx.x == 0 && tid == 0);
  if (tid < kSaBins) h_local[tid] = 0;
  if (tid == 0) {
    mbar_init(&gather_bar, NT);
    mbar_fence_init();
  }
  cluster_arrive_release();   // start-up barrier, first half: this block is running
  __syncthreads();
  grid_dependency_wait();
  grid_launch_dependents();
  ADAMAS_STAMP(1, 1, tid == 0);
  ADAMAS_CHAIN(2, 1, false, blockIdx.x == 0 && tid == 0);

  // q.K mapping: four threads per token (tl = tid / 4, quarter = tid % 4); step i of a thread reads
  // chunk 4*quarter + ((i + quarter + tl) & 3).  A quarter-warp covers an even and an odd token; the
  // rows are 256 bytes apart (the same banks), and with this order the two tokens' four chunks fall
  // on complementary 16-byte bank groups, so the 8 lanes hit 8 different ones.  The query chunks stay
  // packed in registers, in the thread's own order.  Short rows fetch them
  // now (the latency hides behind the selection); long rows hold 16 to 64 distances per thread through
  // the selection phases and fetch the query after them, so that it does not push distances out of the
  // registers.
  const int qk_tl = tid >> 2;
  const int quarter = tid & 3;
  uint4 qpk[4];
  auto load_query = [&]() {
    const T* qp = static_cast<const T*>(p.q) + static_cast<int64_t>(head) * kHeadDim;
#pragma unroll
    for (int i = 0; i < 4; ++i) qpk[i] = ld_16(qp + (4 * quarter + ((i + quarter + qk_tl) & 3)) * 8);
  };
  if (ITEMS == 1) load_query();

  // ---- 1: this block's slice of the row, histogram, exchange --------------------------------------
  const uint16_t* rowp = p.dist + static_cast<int64_t>(head) * p.dist_stride;
  const uint4* gbase = reinterpret_cast<const uint4*>(rowp);
  const int G = (p.n + 7) >> 3;
  const int blk_first = cr * p.granules_per_block;
  const int blk_end = min(G, blk_first + p.granules_per_block);
  const int g0 = blk_first + tid * ITEMS;
  uint32_t raw[ITEMS][4];
  unsigned vmask[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    uint4 v = make_uint4(0, 0, 0, 0);
    unsigned m = 0;
    const int g = g0 + i;
    if (g < blk_end) {
      v = ld_16(gbase + g);
      m = 0xffu;
      if (g * 8 + 8 > p.n) m = 0xffu >> (g * 8 + 8 - p.n);
    }
    raw[i][0] = v.x; raw[i][1] = v.y; raw[i][2] = v.z; raw[i][3] = v.w;
    vmask[i] = m;
  }
  // With pages of 8 tokens or more (a power of two) a granule lies inside one page: fetch its
  // physical page number now, long before the winners are known.
  const bool page_per_granule = p.ps_shift >= 3;
  int granule_page[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    granule_page[i] = 0;
    if (page_per_granule && g0 + i < blk_end) granule_page[i] = __ldg(p.kv_table + (((g0 + i) * 8) >> p.ps_shift));
  }
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned d = (raw[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu;
      if ((vmask[i] >> j) & 1u) atomicAdd(&h_local[min(d, static_cast<unsigned>(kSaBins - 1))], 1u);
    }
  }
  __syncthreads();
  cluster_wait_acquire();     // start-up barrier, second half: every peer is running
  ADAMAS_STAMP(1, 2, tid == 0);
  {
    // thread -> (8 bins, peer): a block's count of one bin is at most 8 * 512 * ITEMS <= 32768
    const int vec = tid & 63;
    const uint4 a = *reinterpret_cast<const uint4*>(h_local + 8 * vec);
    const uint4 b = *reinterpret_cast<const uint4*>(h_local + 8 * vec + 4);
    const uint4 pk = make_uint4(a.x | (a.y << 16), a.z | (a.w << 16), b.x | (b.y << 16), b.z | (b.w << 16));
    for (unsigned peer = static_cast<unsigned>(tid) >> 6; peer < CL; peer += NT / 64) {
      uint16_t* dst = cluster.map_shared_rank(h_src + cr * kSaBins + 8 * vec, peer);
      *reinterpret_cast<uint4*>(dst) = pk;
    }
  }
  cluster_arrive_release();
  cluster_wait_acquire();
  ADAMAS_STAMP(1, 3, tid == 0);

  // every block: total histogram, cut, counts in lower-ranked slices (one bin per thread)
  {
    unsigned tot = 0, low = 0;
    if (tid < kSaBins) {
      for (unsigned r = 0; r < CL; ++r) {
        const unsigned c = h_src[r * kSaBins + tid];
        tot += c;
        if (r < cr) low += c;
      }
    }
    unsigned it = tot, il = low;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned t = __shfl_up_sync(0xffffffffu, it, o);
      const unsigned u = __shfl_up_sync(0xffffffffu, il, o);
      if (lane >= o) {
        it += t;
        il += u;
      }
    }
    if (lane == 31) {
      sh.warp_a[warp] = it;
      sh.warp_b[warp] = il;
    }
    __syncthreads();
    unsigned wa = 0, wb = 0;
#pragma unroll
    for (int w2 = 0; w2 < kWarps; ++w2) {
      wa += (w2 < warp) ? sh.warp_a[w2] : 0u;
      wb += (w2 < warp) ? sh.warp_b[w2] : 0u;
    }
    const unsigned excl = wa + it - tot;
    const unsigned want = static_cast<unsigned>(p.k);
    if (excl < want && excl + tot >= want) {   // exactly one thread
      sh.cut = tid;
      sh.before = excl;
      sh.lt_before = wb + il - low;            // smaller-valued elements in lower-ranked slices
      sh.eq_before = low;                      // cut-valued elements in lower-ranked slices
    }
    __syncthreads();
  }
  const unsigned cut = sh.cut;
  ADAMAS_STAMP(1, 4, tid == 0);
  const unsigned need_eq = static_cast<unsigned>(p.k) - sh.before;       // cut-valued winners in all
  const unsigned eq_before = sh.eq_before;
  const unsigned take_eq = need_eq > eq_before ? need_eq - eq_before : 0u;  // this slice's tie quota
  const unsigned out_base = sh.lt_before + min(eq_before, need_eq);      // winners in lower slices

  // ---- 2: ordered compaction of this block's winners ------------------------------------------------
  unsigned c_lt = 0, c_eq = 0;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned d = (raw[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu;
      const bool ok = (vmask[i] >> j) & 1u;
      c_lt += (ok && d < cut);
      c_eq += (ok && d == cut);
    }
  }
  const unsigned packed = c_lt | (c_eq << 16);
  unsigned incl = packed;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) sh.warp_a[warp] = incl;
  __syncthreads();
  unsigned wbase = 0, blk_tot = 0;
#pragma unroll
  for (int w2 = 0; w2 < kWarps; ++w2) {
    const unsigned a = sh.warp_a[w2];
    wbase += (w2 < warp) ? a : 0u;
    blk_tot += a;
  }
  const unsigned excl = wbase + incl - packed;
  unsigned run_lt = excl & 0xffffu, run_eq = excl >> 16;
  const unsigned blk_lt = blk_tot & 0xffffu, blk_eq = blk_tot >> 16;
  int n_loc = static_cast<int>(blk_lt + min(blk_eq, take_eq));
  int32_t* oi = p.out_idx ? p.out_idx + static_cast<int64_t>(head) * p.out_stride + out_base : nullptr;
  if (c_lt | c_eq) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const unsigned d = (raw[i][j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        if (((vmask[i] >> j) & 1u) && d <= cut) {
          int pos = -1;
          if (d < cut) {
            pos = static_cast<int>(run_lt + min(run_eq, take_eq));
            ++run_lt;
          } else {
            if (run_eq < take_eq) pos = static_cast<int>(run_lt + run_eq);
            ++run_eq;
          }
          if (pos >= 0) {
            const unsigned t = static_cast<unsigned>((g0 + i) * 8 + j);   // logical token position
            int32_t slot;
            if (page_per_granule) {
              slot = granule_page[i] * p.page_size + static_cast<int32_t>(t & (p.page_size - 1));
            } else {
              unsigned pg, e;
              if (p.ps_shift >= 0) {
                pg = t >> p.ps_shift;
                e = t & (p.page_size - 1);
              } else {
                pg = t / p.page_size;
                e = t - pg * p.page_size;
              }
              slot = __ldg(p.kv_table + pg) * p.page_size + static_cast<int32_t>(e);
            }
            if (pos < p.list_capacity) s_list[pos] = slot;
            if (oi) oi[pos] = slot;
          }
        }
      }
    }
  }
  if (cr == CL - 1) {   // the newest token rides with the last slice
    if (tid == 0 && n_loc < p.list_capacity) s_list[n_loc] = static_cast<int32_t>(p.tail_slot);
    n_loc += 1;
  }
  n_loc = min(n_loc, p.list_capacity);
  __syncthreads();
  ADAMAS_STAMP(1, 5, tid == 0);

  // ---- 3: attention over the block's winners ------------------------------------------------------------
  if (ITEMS > 1) load_query();
  const T* kvp = static_cast<const T*>(p.kv);
  const int64_t v_delta = static_cast<int64_t>(p.page_size) * H * kHeadDim;
  float m_run = -INFINITY, l_run = 0.f;
  float o_acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) o_acc[d] = 0.f;
  const int tpg = cap / kGroups;   // tokens per P.V group
  const int pv_g = tid >> 4;   // token group: tokens pv_g*tpg .. pv_g*tpg+tpg-1 of the tile
  const int pv_c = tid & 15;   // 8-dim chunk
  const unsigned ps = static_cast<unsigned>(p.page_size);

  // The tile memory held the histogram tables, written through the generic proxy (by this block and
  // by its peers); the bulk copies write it through the async proxy.
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  unsigned gather_parity = 0;
  for (int t0 = 0; t0 < n_loc; t0 += cap) {
    const int tile_tokens = min(cap, n_loc - t0);
    // gather: thread -> (token tl = tid / 2, K or V row), one 256-byte bulk copy each; every thread
    // arrives at the barrier once, with the bytes it asked for
    {
      const int tl = tid >> 1;
      const int is_v = tid & 1;
      if (tl < tile_tokens) {
        const unsigned slot = static_cast<unsigned>(s_list[t0 + tl]);
        unsigned page, e;
        if (p.ps_shift >= 0) {
          page = slot >> p.ps_shift;
          e = slot & (ps - 1);
        } else {
          page = slot / ps;
          e = slot - page * ps;
        }
        const int64_t row = static_cast<int64_t>(page) * (2 * ps) + e;
        const T* src = kvp + (row * H + head) * kHeadDim + (is_v ? v_delta : 0);
        mbar_arrive_expect_tx(&gather_bar, kHeadDim * 2);
        bulk_copy_g2s((is_v ? sv : sk) + tl * 256, src, kHeadDim * 2, &gather_bar);
      } else {
        mbar_arrive(&gather_bar);
      }
      if (!mbar_wait_bounded(&gather_bar, gather_parity, 1u << 22)) atomicOr(&g_adamas_error, kErrGatherTimeout);
      gather_parity ^= 1u;
    }
    ADAMAS_STAMP(1, 6, tid == 0 && t0 == 0);
    ADAMAS_STAMP(1, 10, tid == 0 && t0 != 0);

    // q.K: tokens qk_tl (all threads) and NT/4 + qk_tl (tiles of more than NT/4 tokens)
    float wmax = -INFINITY;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      if (pass == 1 && tile_tokens <= kQkTokens) break;   // block-uniform
      const int tl = qk_tl + kQkTokens * pass;
      float acc = 0.f;
      const bool live = tl < tile_tokens;
      if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int lc = 4 * quarter + ((i + quarter + qk_tl) & 3);   // tl and qk_tl have the same parity
          float kf[8], qf[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(sk + tl * 256 + lc * 16), kf);
          unpack8<T>(qpk[i], qf);
#pragma unroll
          for (int d = 0; d < 8; ++d) acc = fmaf(qf[d], kf[d], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      const float logit = live ? acc * p.scale_log2 : -INFINITY;
      if (quarter == 0 && tl < kCapMax) sh.s_logit[tl] = logit;
      wmax = fmaxf(wmax, logit);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
    if (lane == 0) sh.s_red[warp] = wmax;
    __syncthreads();
    float m_tile = sh.s_red[0];
#pragma unroll
    for (int w2 = 1; w2 < kWarps; ++w2) m_tile = fmaxf(m_tile, sh.s_red[w2]);
    const float m_new = fmaxf(m_run, m_tile);
    const float rescale = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
    if (tid < kCapMax) {   // the first kCapMax / 32 warps
      float psum = 0.f;
      if (tid < tile_tokens) {
        const float lg = sh.s_logit[tid];
        const float pr = (lg == -INFINITY) ? 0.f : exp2f(lg - m_new);
        sh.s_p[tid] = pr;
        psum = pr;
      } else {
        sh.s_p[tid] = 0.f;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
      if (lane == 0) sh.s_sum[warp] = psum;
    }
    __syncthreads();
    {
      float tile_sum = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < kCapMax / 32; ++w2) tile_sum += sh.s_sum[w2];
      l_run = l_run * rescale + tile_sum;
    }
    m_run = m_new;
#pragma unroll
    for (int d = 0; d < 8; ++d) o_acc[d] *= rescale;
#pragma unroll
    for (int i = 0; i < kSaMaxTpg; ++i) {
      if (i < tpg) {
        const int tl = pv_g * tpg + i;
        const float pr = sh.s_p[tl];
        if (pr != 0.f) {
          float vf[8];
          unpack8<T>(*reinterpret_cast<const uint4*>(sv + tl * 256 + pv_c * 16), vf);
#pragma unroll
          for (int d = 0; d < 8; ++d) o_acc[d] = fmaf(pr, vf[d], o_acc[d]);
        }
      }
    }
    __syncthreads();
  }

  // ---- 4: partial to rank 0, merge -----------------------------------------------------------------------
  ADAMAS_STAMP(1, 7, tid == 0);
#pragma unroll
  for (int d = 0; d < 8; ++d) o_acc[d] += __shfl_xor_sync(0xffffffffu, o_acc[d], 16);   // the warp's two groups
  if (lane < 16) {
#pragma unroll
    for (int d = 0; d < 8; ++d) s_o[warp][pv_c * 8 + d] = o_acc[d];
  }
  __syncthreads();
  if (tid < kHeadDim) {
    float od = 0.f;
#pragma unroll
    for (int g = 0; g < kWarps; ++g) od += s_o[g][tid];
    *cluster.map_shared_rank(part_o + cr * kHeadDim + tid, 0) = od;
  }
  if (tid == 0) {
    float* ml = cluster.map_shared_rank(part_ml + cr * 2, 0);
    ml[0] = m_run;
    ml[1] = l_run;
  }
  cluster_arrive_release();
  cluster_wait_acquire();
  ADAMAS_STAMP(1, 8, tid == 0);
  ADAMAS_TRACE(1, p.trace_tag, 1, tid == 0);
#ifdef ADAMAS_PHASE_TIMING
  if (tid == 0 && blockIdx.x < kTimingBlocks) g_phase_timing[1][blockIdx.x][11] = static_cast<unsigned long long>(n_loc);
#endif
  if (cr != 0 || tid >= kHeadDim) return;
  float M = -INFINITY;
  for (unsigned r = 0; r < CL; ++r) M = fmaxf(M, part_ml[r * 2]);
  float accd = 0.f, L = 0.f;
  for (unsigned r = 0; r < CL; ++r) {
    const float m = part_ml[r * 2];
    const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
    L += w * part_ml[r * 2 + 1];
    accd += w * part_o[r * kHeadDim + tid];
  }
  const float res = L > 0.f ? accd / L : 0.f;
  const float res1 = __shfl_down_sync(0xffffffffu, res, 1);
  T* op = static_cast<T*>(p.o) + static_cast<int64_t>(head) * kHeadDim;
  if ((tid & 1) == 0) reinterpret_cast<uint32_t*>(op)[tid >> 1] = Elem<T>::from_f2(res, res1);
  if (tid == 0 && p.lse) p.lse[head] = L > 0.f ? M + log2f(L) : -INFINITY;
  ADAMAS_STAMP(1, 9, tid == 0);
  ADAMAS_CHAIN(2, 2, true, blockIdx.x == 0 && tid == 0);
#ifdef ADAMAS_PHASE_TIMING
  if (tid == 0 && blockIdx.x < kTimingBlocks) g_phase_timing[1][blockIdx.x][11] = static_cast<unsigned long long>(n_loc);
#endif
}

}  // namespace adamas
