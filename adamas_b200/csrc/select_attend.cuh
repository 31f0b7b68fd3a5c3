// Stages 3 + 4 of the decode path in one kernel: per head, pick the k smallest of n integer distances
// (ties to the lower position) and run the decode attention over the picked tokens plus the newest
// token.  Used by the fused decode step; the separate top-k and decode kernels remain for callers
// that want the stages one by one.
//
// The kernel does not count anything itself.  The estimate kernels (or dist_histogram_kernel, for a
// caller that only has a distance row) leave, per head, one 512-bin histogram per SLICE of the row
// in a global table [H][kSaMaxSlices][512] u32: slice r covers the granules (8 distances) that block
// r of the head's cluster owns.  A distance is at most 3 * 128 = 384; larger values count as 511.
//
// CL <= 16 blocks x 512 threads per head (grid (CL, H)); the blocks of a head never wait for one another.
// Block `cr`:
//   load   its slice of the distance row (registers), the head's CL histograms (one bin per thread)
//          and the query chunks, all in flight together;
//   cut    block-wide scan of the summed histogram: the cut distance, how many cut-valued elements
//          are taken in all, how many of them and how many smaller elements lie in lower-ranked
//          slices (= this slice's tie quota and its offset in the output list).  Every block
//          derives this by itself from the same table: no exchange between blocks;
//   pick   ordered compaction of the block's winners into a list in shared memory;
//   attend the rows of the list are dealt out evenly to the 16 warps; a warp gathers the K and V rows of
//          its tokens itself (16-byte asynchronous copies, a half-warp per 256-byte row, into its own
//          part of the tile; K rows as one group, V rows as a second), computes q.K with four lanes per token, a
//          softmax in base 2 over its tokens and P.V with four dimensions per lane: no block barrier
//          inside the attention;
//   merge  the 16 warps' partial (o, m, l) are merged in shared memory and the block's partial goes to
//          the head's slot table in global scratch; the block that arrives LAST at the head's counter
//          merges the CL partials, writes the head's output, clears the head's histogram rows and the
//          counter.  Every other block is gone by then: its SM is free for the next kernel's blocks
//          while the slowest block of the head still works (with a cluster barrier at this point all
//          blocks of a head stayed resident until the slowest had finished, 2 us at 32K / 1024).
#pragma once
#include "common.cuh"
#include "hadamard_append.cuh"

namespace adamas {

constexpr int kSaThreads = 512;
constexpr int kSaWarps = kSaThreads / 32;
constexpr int kSaBins = 512;
constexpr int kSaMaxSlices = 16;      // histogram rows per head = largest cluster
constexpr int kSaTile = 128;          // planning unit of the host (winners per block it aims for)
constexpr int kSaWarpRows = 12;       // rows a warp gathers per round (its part of the tile: 12 K + 12 V rows)
constexpr int kSaMaxCluster = 8;      // blocks per head by default (more, up to 16, while all blocks are resident at once)
constexpr int kSaBigCluster = 16;     // long rows of few heads (see the host code)
// Scratch words (32 bit) per head: kSaMaxSlices histogram rows of 512 counts, then kSaMaxSlices slots of
// kSaSlotWords floats for the blocks' partial results (128 outputs, running max, running sum; word 130
// of slot 0 is the head's arrival counter).
constexpr int kSaSlotWords = 132;
constexpr int kSaScratchWordsPerHead = kSaMaxSlices * kSaBins + kSaMaxSlices * kSaSlotWords;

// Granules (8 distances) of a row that each of `cl` blocks owns: a multiple of 4, so that a slice
// starts on a multiple of 32 tokens and no 32-token tile of an estimate kernel straddles two slices.
__host__ __device__ __forceinline__ int sa_granules_per_block(int n, int cl) {
  const int g = ((n + 7) >> 3);
  return (((g + cl - 1) / cl) + 3) & ~3;
}

struct SelectAttendParams {
  const uint16_t* dist;     // [H, dist_stride] u16 distances, rows 16-byte aligned
  int64_t dist_stride;
  uint32_t* hist;           // [H][kSaScratchWordsPerHead]: per-slice histograms of the rows (cleared on exit),
                            // then the slots of the blocks' partial results and the arrival counter
  const int2* ext_cut;      // optional [H]: (cut distance, cut-valued winners this call takes), decided
                            // elsewhere (sequence shards); k is then unused
  const int32_t* seq_len_dev;  // optional: n = *seq_len_dev - 1 and the newest token sits at position n
  const SeqDesc* seqs;      // optional (needs seq_len_dev): a batch of sequences, grid.z = sequence; dist, hist, q, o,
                            // lse and out_idx have one row per (sequence, head); cache, page table and length are the sequence's
  int n;                    // distances per head (tokens 0 .. n-1) when seq_len_dev is null
  int k;                    // winners per head, 1 <= k <= n
  const void* q;            // [H, 128]; read after the preceding kernel has completed
  void* o;                  // [H, 128] in the cache's element type, or null
  float* o_f32;             // [H, 128] fp32 (partial result of a sequence shard), or null
  float* lse;               // [H] or null (base 2)
  const void* kv;           // [pages, 2, page_size, H, 128]
  const int32_t* kv_table;  // logical page -> physical page
  int page_size;
  int ps_shift;             // log2(page_size) or -1
  int H;                    // heads of the KV cache
  int q_group;              // query heads per cache head (grouped-query attention; 1 otherwise): the grid, dist,
                            // hist, q, o, lse and out_idx have H * q_group rows; row r attends cache head r / q_group
  int tail_mode;            // 0: no newest token; 1: it is at tail_slot; 2: at logical position n
  unsigned tail_slot;       // physical slot of the newest token (tail_mode 1)
  int32_t* out_idx;         // optional [H, out_stride]: physical slots of the winners, ascending position
  int64_t out_stride;
  int list_capacity;        // entries of the shared-memory winner list (a block's winners at most, plus the newest token)
  float scale_log2;
  // q arrives un-rotated (the append-fused estimate in front of this launch has coded the rotated query but left
  // q alone): every block rotates it for position n for its own use, the block that finishes a head writes
  // the rotated row back into q
  int rope_on;
  RopeParams rope;
};

struct SaShared {
  float ml[kSaWarps][2];
  unsigned warp_a[kSaWarps];
  unsigned warp_b[kSaWarps];
  unsigned cut, need_eq, lt_before, eq_before;
  unsigned last;   // this block arrived last at the head's counter
  uint4 q[16];     // the head's query row
  float2 cs[kHeadDim / 2];   // rope_on: (cos, sin) of the position
};

// Dynamic shared memory: the tile (16 warps x (12 K rows + 12 V rows) x 256 B; a warp parks its partial
// output in its own K rows at the end) | winner list (list_capacity * 4 B).
template <typename T, int ITEMS>
__global__ void __launch_bounds__(kSaThreads, 2) select_attend_kernel(const SelectAttendParams p) {
  constexpr int NT = kSaThreads;
  static_assert(NT >= kSaBins, "one histogram bin per thread");
  extern __shared__ __align__(16) uint8_t sa_smem[];
  __shared__ __align__(16) SaShared sh;

  const unsigned CL = gridDim.x;
  const unsigned cr = blockIdx.x;
  const int head = blockIdx.z * gridDim.y + blockIdx.y;   // row of dist, hist, q, o, lse, out_idx: (sequence, query head)
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int H = p.H;
  const int head_kv = p.q_group == 1 ? blockIdx.y : blockIdx.y / p.q_group;
  const int32_t* kv_table = p.kv_table;
  const void* kv_base = p.kv;
  const int32_t* seq_len_dev = p.seq_len_dev;
  if (p.seqs) {   // (the table of sequences is set up once, long before this launch)
    kv_table = p.seqs[blockIdx.z].kv_table;
    kv_base = p.seqs[blockIdx.z].kv_data;
    seq_len_dev += blockIdx.z;
  }

  uint8_t* sa_tile = sa_smem;                                                         // [16 warps][K rows | V rows]
  int32_t* s_list = reinterpret_cast<int32_t*>(sa_smem + kSaWarps * 2 * kSaWarpRows * 256);   // the block's winners, in position order
  uint32_t* head_scratch = p.hist + static_cast<size_t>(head) * kSaScratchWordsPerHead;
  float* slots = reinterpret_cast<float*>(head_scratch + kSaMaxSlices * kSaBins);     // [CL][kSaSlotWords]
  uint4* s_q = sh.q;

  // ---- set-up that needs no input (overlaps the tail of the preceding kernel) -----------------------
  if (tid == 0) sh.cut = 0xffffffffu;
  __syncthreads();
  grid_dependency_wait();
  grid_launch_dependents();

  // ---- loads: distances, histograms, query, page numbers --------------------------------------------
  const int n = seq_len_dev ? (__ldg(seq_len_dev) - 1) : p.n;
  const int G = (n + 7) >> 3;
  const int gpb = sa_granules_per_block(n, static_cast<int>(CL));
  const int blk_first = cr * gpb;
  // (rope_on: warps 2 and 3 form the position's cos / sin pairs; the block barriers of the cut phase order
  // them before the query is rotated)
  const bool rope_thread = p.rope_on && tid >= kHeadDim / 2 && tid < kHeadDim;
  const int blk_end = min(G, blk_first + gpb);
  const int g0 = blk_first + tid * ITEMS;
  const uint4* gbase = reinterpret_cast<const uint4*>(p.dist + static_cast<int64_t>(head) * p.dist_stride);
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
      if (g * 8 + 8 > n) m = 0xffu >> (g * 8 + 8 - n);
    }
    raw[i][0] = v.x; raw[i][1] = v.y; raw[i][2] = v.z; raw[i][3] = v.w;
    vmask[i] = m;
  }
  // (all loads are issued before the first count is used: one trip to L2, not one per slice)
  unsigned hcnt[kSaMaxSlices];
  {
    const uint32_t* hrow = head_scratch + tid;
#pragma unroll
    for (unsigned r = 0; r < kSaMaxSlices; ++r) hcnt[r] = r < CL ? __ldcg(hrow + r * kSaBins) : 0u;
  }
  // With pages of 8 tokens or more (a power of two) a granule lies inside one page: fetch its
  // physical page number now, long before the winners are known.
  const bool page_per_granule = p.ps_shift >= 3;
  int granule_page[ITEMS];
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    granule_page[i] = 0;
    if (page_per_granule && g0 + i < blk_end) granule_page[i] = __ldg(kv_table + (((g0 + i) * 8) >> p.ps_shift));
  }
  // the newest token rides with the last slice
  const bool tail_here = p.tail_mode != 0 && cr == CL - 1;
  unsigned tail_slot = p.tail_slot;
  if (tail_here && tid == 0 && p.tail_mode == 2) {
    const unsigned un = static_cast<unsigned>(n), ps = static_cast<unsigned>(p.page_size);
    const unsigned pg = p.ps_shift >= 0 ? (un >> p.ps_shift) : (un / ps);
    tail_slot = static_cast<unsigned>(__ldg(kv_table + pg)) * ps + (un - pg * ps);
  }
  if (rope_thread) sh.cs[tid - kHeadDim / 2] = rope_cos_sin(tid - kHeadDim / 2, static_cast<float>(n), p.rope);
  // ---- cut: one bin per thread ------------------------------------------------------------------------
  unsigned tot = 0, low = 0;
#pragma unroll
  for (unsigned r = 0; r < kSaMaxSlices; ++r) {
    tot += hcnt[r];
    low += r < cr ? hcnt[r] : 0u;
  }
  {
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
    for (int w2 = 0; w2 < kSaWarps; ++w2) {
      wa += (w2 < warp) ? sh.warp_a[w2] : 0u;
      wb += (w2 < warp) ? sh.warp_b[w2] : 0u;
    }
    const unsigned excl = wa + it - tot;        // elements of smaller value, whole row
    const unsigned excl_low = wb + il - low;    // ... in lower-ranked slices
    bool mine, all_win = false;
    unsigned need = 0;
    if (p.ext_cut) {
      // (a cut of 512, beyond every bin: the whole row wins; thread 511 stands in, there are no ties)
      const int2 e = __ldg(p.ext_cut + head);
      all_win = e.x >= kSaBins;
      mine = tid == min(e.x, kSaBins - 1);
      need = all_win ? 0u : static_cast<unsigned>(e.y);
    } else {
      const unsigned want = static_cast<unsigned>(p.k);
      mine = excl < want && excl + tot >= want;   // exactly one thread
      need = want - excl;
    }
    if (mine) {
      sh.cut = all_win ? static_cast<unsigned>(kSaBins) : static_cast<unsigned>(tid);
      sh.need_eq = need;                                  // cut-valued winners in all
      sh.lt_before = excl_low + (all_win ? low : 0u);     // smaller-valued elements in lower-ranked slices
      sh.eq_before = all_win ? 0u : low;                  // cut-valued elements in lower-ranked slices
    }
    __syncthreads();
  }
  unsigned cut = sh.cut;
  unsigned need_eq = sh.need_eq;
  if (cut == 0xffffffffu) {
    // the table does not describe this row (fewer than k entries): take nothing but the newest token
    if (tid == 0) atomicOr(&g_adamas_error, kErrHistogram);
    cut = 0;
    need_eq = 0;
  }
  const unsigned eq_before = (sh.cut == 0xffffffffu) ? 0u : sh.eq_before;
  const unsigned take_eq = need_eq > eq_before ? need_eq - eq_before : 0u;   // this slice's tie quota
  const unsigned out_base = ((sh.cut == 0xffffffffu) ? 0u : sh.lt_before) + min(eq_before, need_eq);

  // ---- pick: ordered compaction of this block's winners -----------------------------------------------
  // Two halfword-parallel compares per register give, per granule, the 8-bit masks of the elements below
  // the cut and at the cut (values of 511 and more count as 511).
  const unsigned cut2 = min(cut, 0xffffu) * 0x00010001u;
  unsigned m_lt[ITEMS], m_eq[ITEMS];
  unsigned c_lt = 0, c_eq = 0;
#pragma unroll
  for (int i = 0; i < ITEMS; ++i) {
    unsigned lt = 0, eq = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const unsigned x = __vminu2(raw[i][w], 0x01ff01ffu);
      const unsigned l = __vcmpltu2(x, cut2);   // 0xffff per halfword that is below the cut
      const unsigned e = __vcmpeq2(x, cut2);
      lt |= ((l & 1u) | ((l >> 15) & 2u)) << (2 * w);
      eq |= ((e & 1u) | ((e >> 15) & 2u)) << (2 * w);
    }
    m_lt[i] = lt & vmask[i];
    m_eq[i] = eq & vmask[i];
    c_lt += __popc(m_lt[i]);
    c_eq += __popc(m_eq[i]);
  }
  const unsigned packed = c_lt | (c_eq << 16);
  unsigned incl = packed;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) sh.warp_a[warp] = incl;   // (its readers of the cut phase are past a block barrier)
  __syncthreads();
  unsigned wbase = 0, blk_tot = 0;
#pragma unroll
  for (int w2 = 0; w2 < kSaWarps; ++w2) {
    const unsigned a = sh.warp_a[w2];
    wbase += (w2 < warp) ? a : 0u;
    blk_tot += a;
  }
  const unsigned excl = wbase + incl - packed;
  unsigned run_lt = excl & 0xffffu, run_eq = excl >> 16;
  const unsigned blk_lt = blk_tot & 0xffffu, blk_eq = blk_tot >> 16;
  const int n_win = static_cast<int>(blk_lt + min(blk_eq, take_eq));
  const int n_loc = min(n_win + (tail_here ? 1 : 0), p.list_capacity);

  const T* kvp = static_cast<const T*>(kv_base);
  const unsigned ps = static_cast<unsigned>(p.page_size);
  const int64_t v_delta = static_cast<int64_t>(p.page_size) * H * kHeadDim;
  // The winners go to a list in shared memory (a few instructions on a divergent path).
  int32_t* oi = p.out_idx ? p.out_idx + static_cast<int64_t>(head) * p.out_stride + out_base : nullptr;
  if (c_lt | c_eq) {
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      // only the elements at or below the cut are visited, in position order (a warp takes as many turns
      // as its busiest lane has candidates: one or two at the usual budgets)
      unsigned cand = m_lt[i] | m_eq[i];
      while (cand) {
        const int j = __ffs(cand) - 1;
        cand &= cand - 1;
        int pos = -1;
        if ((m_lt[i] >> j) & 1u) {
          pos = static_cast<int>(run_lt + min(run_eq, take_eq));
          ++run_lt;
        } else {
          if (run_eq < take_eq) pos = static_cast<int>(run_lt + run_eq);
          ++run_eq;
        }
        if (pos >= 0) {
          const unsigned t = static_cast<unsigned>((g0 + i) * 8 + j);   // logical token position
          unsigned slot;
          if (page_per_granule) {
            slot = static_cast<unsigned>(granule_page[i]) * ps + (t & (ps - 1));
          } else {
            unsigned pg, e;
            if (p.ps_shift >= 0) {
              pg = t >> p.ps_shift;
              e = t & (ps - 1);
            } else {
              pg = t / ps;
              e = t - pg * ps;
            }
            slot = static_cast<unsigned>(__ldg(kv_table + pg)) * ps + e;
          }
          if (pos < p.list_capacity) s_list[pos] = static_cast<int32_t>(slot);
          if (oi) oi[pos] = static_cast<int32_t>(slot);
        }
      }
    }
  }
  if (tail_here && tid == 0 && n_win < p.list_capacity) s_list[n_win] = static_cast<int32_t>(tail_slot);
  if (warp == 0) {
    // the query row: 16 lanes x 16 bytes (with rope_on rotated first: dimension pairs sit in lanes l and l ^ 8)
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (lane < 16) raw = ld_16(static_cast<const T*>(p.q) + static_cast<int64_t>(head) * kHeadDim + lane * 8);
    if (p.rope_on) {
      float x[8];
      unpack8<T>(raw, x);
      rope_halfwarp_cs<T>(x, lane & 15, sh.cs, p.rope.inv_freq != nullptr, p.rope.mscale);
      raw = pack8<T>(x);
    }
    if (lane < 16) s_q[lane] = raw;
  }

  // ---- attend: every warp over its own rows --------------------------------------------------------------
  // The rows are dealt out evenly: warp w owns rows w*rpw .. of the list.  It gathers them itself, kSaWarpRows
  // at a time, with 16-byte asynchronous copies (cp.async), a half-warp per 256-byte row, into the warp's own
  // part of the tile: first all K rows (one commit group), then all V rows (a second group); then q.K with
  // four lanes per token as soon as the K group has landed, a softmax in base 2 over its tokens and, after
  // the V group, P.V with four dimensions per lane.  Nothing in here is shared between warps: no block
  // barrier inside the attention.
  // Measured alternatives for the gather (select+attend alone, 32K / 1024): one 256-byte bulk (TMA) copy
  // per row with an mbarrier per warp 12.4-12.5 us against 12.2 with the 16-byte copies (a bulk copy with
  // a different address in every lane is issued lane after lane, about 45 ns each: 0.7 us for the 16 rows
  // of a warp); all bulk copies issued by the first n_loc / 16 warps 1.9 us instead of 0.7; plain vector
  // loads into registers instead of the tile (all rows cannot be in flight at once in 64 registers: the
  // second round of a warp pays the memory latency again) 4.5 us in this phase.
  __syncthreads();   // the list and the query are complete
  float m_run = -INFINITY, l_run = 0.f;   // l_run is kept by the lanes with quarter == 0
  float o_acc[4] = {0.f, 0.f, 0.f, 0.f};  // dimensions 4*lane .. 4*lane+3
  const int rpw = (n_loc + kSaWarps - 1) / kSaWarps;
  const int my_first = warp * rpw;
  const int my_total = max(0, min(rpw, n_loc - my_first));
  uint8_t* wk = sa_tile + warp * (2 * kSaWarpRows * 256);   // this warp's K rows, then its V rows
  uint8_t* wv = wk + kSaWarpRows * 256;
  // q.K mapping: four lanes per token (tq = lane / 4, quarter = lane % 4); step i of a lane reads chunk
  // 4*quarter + ((i + quarter + tq) & 3).  A quarter-warp covers an even and an odd token; the rows are
  // 256 bytes apart (the same banks), and with this order the two tokens' four chunks fall on
  // complementary 16-byte bank groups, so the 8 lanes hit 8 different ones.
  const int tq = lane >> 2;
  const int quarter = lane & 3;
  uint4 qpk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) qpk[i] = s_q[4 * quarter + ((i + quarter + tq) & 3)];
  constexpr int kGroups = (kSaWarpRows + 7) / 8;   // groups of 8 rows per round
  for (int done = 0; done < my_total; done += kSaWarpRows) {
    const int my_rows = min(kSaWarpRows, my_total - done);
    if (done > 0) __syncwarp();   // every lane has read the rows of the round before
    // 16-byte asynchronous copies, a half-warp per 256-byte row: all K rows of the round as one group, then
    // all V rows as a second one, so that the logits are formed while the V rows are still on their way.
    {
      const int half = lane >> 4, l16 = lane & 15;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        for (int r = half; r < my_rows; r += 2) {
          const unsigned slot = static_cast<unsigned>(s_list[my_first + done + r]);
          unsigned page, e;
          if (p.ps_shift >= 0) {
            page = slot >> p.ps_shift;
            e = slot & (ps - 1);
          } else {
            page = slot / ps;
            e = slot - page * ps;
          }
          const T* src = kvp + (static_cast<int64_t>(page * (2 * ps) + e) * H + head_kv) * kHeadDim + (kv ? v_delta : 0);
          cp_async_16((kv ? wv : wk) + r * 256 + l16 * 16, src + l16 * 8);
        }
        cp_async_commit();
      }
    }
    cp_async_wait<1>();
    __syncwarp();
    float logit[kGroups];
#pragma unroll
    for (int g = 0; g < kGroups; ++g) {
      const int row = g * 8 + tq;
      const bool live = row < my_rows;
      float acc = 0.f;
      if (live) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int lc = 4 * quarter + ((i + quarter + tq) & 3);
          const uint4 kk = *reinterpret_cast<const uint4*>(wk + row * 256 + lc * 16);
          acc = Elem<T>::dot2(qpk[i].x, kk.x, acc);
          acc = Elem<T>::dot2(qpk[i].y, kk.y, acc);
          acc = Elem<T>::dot2(qpk[i].z, kk.z, acc);
          acc = Elem<T>::dot2(qpk[i].w, kk.w, acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      logit[g] = live ? acc * p.scale_log2 : -INFINITY;
    }
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int g = 0; g < kGroups; ++g) {
      const int base = g * 8;
      if (base >= my_rows) break;   // warp-uniform
      const bool live = base + tq < my_rows;
      float m_new = logit[g];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) m_new = fmaxf(m_new, __shfl_xor_sync(0xffffffffu, m_new, o));
      m_new = fmaxf(m_new, m_run);      // finite: the first row of a group is live
      const float rescale = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
      const float pr = live ? exp2f(logit[g] - m_new) : 0.f;
      float psum = quarter == 0 ? pr : 0.f;
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
      l_run = l_run * rescale + psum;
      m_run = m_new;
#pragma unroll
      for (int d = 0; d < 4; ++d) o_acc[d] *= rescale;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pr, 4 * j);
        if (pj != 0.f) {   // warp-uniform; rows past the end are stale
          const uint2 vv = *reinterpret_cast<const uint2*>(wv + (base + j) * 256 + lane * 8);
          const float2 a = Elem<T>::to_f2(vv.x), b = Elem<T>::to_f2(vv.y);
          o_acc[0] = fmaf(pj, a.x, o_acc[0]);
          o_acc[1] = fmaf(pj, a.y, o_acc[1]);
          o_acc[2] = fmaf(pj, b.x, o_acc[2]);
          o_acc[3] = fmaf(pj, b.y, o_acc[3]);
        }
      }
    }
  }

  // ---- merge: warps -> block -> head ----------------------------------------------------------------------
  // a warp parks its partial output in its own K rows, which nobody else touches
  __syncwarp();
  reinterpret_cast<float4*>(wk)[lane] = make_float4(o_acc[0], o_acc[1], o_acc[2], o_acc[3]);
  if (lane == 0) {
    sh.ml[warp][0] = m_run;
    sh.ml[warp][1] = l_run;
  }
  __syncthreads();
  {
    // all 512 threads: thread (part = tid / 128, d = tid % 128) folds the partials of warps 4*part .. 4*part+3
    // for output d; the four parts are added by the first 128 threads
    float M = -INFINITY;
#pragma unroll
    for (int w2 = 0; w2 < kSaWarps; ++w2) M = fmaxf(M, sh.ml[w2][0]);
    const int d = tid & (kHeadDim - 1), part = tid >> 7;
    float od = 0.f, L = 0.f;
#pragma unroll
    for (int j = 0; j < kSaWarps / 4; ++j) {
      const int w2 = part * (kSaWarps / 4) + j;
      const float m = sh.ml[w2][0];
      const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
      L += w * sh.ml[w2][1];
      if (w != 0.f) od += w * reinterpret_cast<const float*>(sa_tile + w2 * (2 * kSaWarpRows * 256))[d];
    }
    float* fold = reinterpret_cast<float*>(sa_tile + kSaWarpRows * 256);   // [4][130], in warp 0's V rows (free by now)
    fold[part * 130 + d] = od;
    if (d == 0) fold[part * 130 + kHeadDim] = L;
    __syncthreads();
    if (tid < kHeadDim) {
      float* slot = slots + cr * kSaSlotWords;
      __stcg(slot + tid, (fold[tid] + fold[130 + tid]) + (fold[260 + tid] + fold[390 + tid]));
      if (tid == 0) {
        __stcg(slot + kHeadDim, M);
        __stcg(slot + kHeadDim + 1, (fold[kHeadDim] + fold[130 + kHeadDim]) + (fold[260 + kHeadDim] + fold[390 + kHeadDim]));
      }
    }
  }
  // the block that arrives last at the head's counter merges; nobody waits.  The block barrier orders
  // the slot stores of all threads before thread 0's release at the counter; the last block's acquire
  // there, followed by the second barrier, orders its loads of the slots after every block's stores.
  unsigned* counter = head_scratch + kSaMaxSlices * kSaBins + kHeadDim + 2;   // word 130 of slot 0
  __syncthreads();
  if (tid == 0) {
    unsigned ticket;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(counter) : "memory");
    sh.last = (ticket == CL - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (!sh.last) return;
  // every block of the head has read the histograms long ago: clear them and the counter for the next launch
#pragma unroll
  for (unsigned r = 0; r < kSaMaxSlices; ++r)
    if (r < CL) head_scratch[r * kSaBins + tid] = 0u;
  if (tid == 0) *counter = 0u;
  // (every block of the head has read the un-rotated query long ago)
  if (p.rope_on && tid < 16)
    st_16(static_cast<T*>(const_cast<void*>(p.q)) + static_cast<int64_t>(head) * kHeadDim + tid * 8, s_q[tid]);
  if (tid >= kHeadDim) return;
  // all loads of the CL partials are issued before the first is used: one trip to L2
  float pm[kSaMaxSlices], pl[kSaMaxSlices], po[kSaMaxSlices];
#pragma unroll
  for (unsigned r = 0; r < kSaMaxSlices; ++r) {
    pm[r] = -INFINITY;
    pl[r] = 0.f;
    po[r] = 0.f;
    if (r < CL) {
      pm[r] = __ldcg(slots + r * kSaSlotWords + kHeadDim);
      pl[r] = __ldcg(slots + r * kSaSlotWords + kHeadDim + 1);
      po[r] = __ldcg(slots + r * kSaSlotWords + tid);
    }
  }
  float M = -INFINITY;
#pragma unroll
  for (unsigned r = 0; r < kSaMaxSlices; ++r) M = fmaxf(M, pm[r]);
  float accd = 0.f, L = 0.f;
#pragma unroll
  for (unsigned r = 0; r < kSaMaxSlices; ++r) {
    const float w = (pm[r] == -INFINITY) ? 0.f : exp2f(pm[r] - M);
    L += w * pl[r];
    if (w != 0.f) accd += w * po[r];
  }
  const float res = L > 0.f ? accd / L : 0.f;
  const float res1 = __shfl_down_sync(0xffffffffu, res, 1);
  if (p.o_f32) p.o_f32[static_cast<int64_t>(head) * kHeadDim + tid] = res;
  if (p.o && (tid & 1) == 0)
    reinterpret_cast<uint32_t*>(static_cast<T*>(p.o) + static_cast<int64_t>(head) * kHeadDim)[tid >> 1] =
        Elem<T>::from_f2(res, res1);
  if (tid == 0 && p.lse) p.lse[head] = L > 0.f ? M + log2f(L) : -INFINITY;
}

// Per-slice histograms of distance rows, for callers of select_attend that did not get them from an
// estimate kernel: grid (cl, H); block (r, h) counts slice r of head h in shared memory and STORES the
// row (the table needs no clearing beforehand).
struct DistHistogramParams {
  const uint16_t* dist;
  int64_t dist_stride;
  uint32_t* hist;
  int n;                        // distances per row, or their upper bound with seq_len_dev
  int cl;
  const int32_t* seq_len_dev;   // optional: n = *seq_len_dev - 1 (grid.z = sequence: seq_len_dev[z], rows (z, y))
};

// Per-slice histograms of given distance rows: grid (slices, rows[, sequences]).  Used where the rows exist
// already (the stand-alone select_attend call) and, in the fused step, for launches with so many distances
// that one L2 atomic per distance from inside the estimate would bound it (3 M and more per launch): a
// block counts its slice in shared memory and stores 512 totals.
__global__ void __launch_bounds__(kSaThreads) dist_histogram_kernel(const DistHistogramParams p) {
  __shared__ unsigned h_local[kSaBins];
  const int tid = threadIdx.x;
  const int r = blockIdx.x;
  const int head = blockIdx.z * gridDim.y + blockIdx.y;
  h_local[tid] = 0;
  __syncthreads();
  grid_dependency_wait();
  grid_launch_dependents();
  const int n = p.seq_len_dev ? __ldg(p.seq_len_dev + blockIdx.z) - 1 : p.n;
  const int G = (n + 7) >> 3;
  const int gpb = sa_granules_per_block(n, p.cl);
  const int g_end = min(G, (r + 1) * gpb);
  const uint4* gbase = reinterpret_cast<const uint4*>(p.dist + static_cast<int64_t>(head) * p.dist_stride);
  for (int g = r * gpb + tid; g < g_end; g += kSaThreads) {
    const uint4 v = ld_16(gbase + g);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    const int valid = min(8, n - g * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const unsigned d = (w[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
      if (j < valid) atomicAdd(&h_local[min(d, static_cast<unsigned>(kSaBins - 1))], 1u);
    }
  }
  __syncthreads();
  p.hist[static_cast<size_t>(head) * kSaScratchWordsPerHead + r * kSaBins + tid] = h_local[tid];
}

// ---- a sequence split over several GPUs: one cut for all shards -----------------------------------------------
// Every shard counts its own distances (estimate kernel, per-slice histograms).  hist_rowsum_kernel adds
// a shard's slices to one 512-bin histogram per head; the shards exchange those ([G][H][512], one
// all-gather); global_cut_kernel then derives, identically on every shard, the cut distance of the k
// smallest distances of the whole sequence and this shard's share of the cut-valued elements (shards
// hold ascending token ranges, so "the lower position wins a tie" means: lower shards first): the
// ext_cut input of select_attend_kernel.  No candidate list ever crosses the link.
__global__ void __launch_bounds__(kSaBins) hist_rowsum_kernel(const uint32_t* __restrict__ scratch, int slices,
                                                              uint32_t* __restrict__ out) {
  const int head = blockIdx.x, tid = threadIdx.x;
  grid_dependency_wait();
  grid_launch_dependents();
  const uint32_t* rows = scratch + static_cast<size_t>(head) * kSaScratchWordsPerHead + tid;
  uint32_t c = 0;
  for (int r = 0; r < slices; ++r) c += __ldcg(rows + r * kSaBins);
  out[static_cast<size_t>(head) * kSaBins + tid] = c;
}

// all: [G][H][512] counts; ext_cut[h] = (cut distance, cut-valued elements shard `rank` takes).  If the
// whole sequence holds fewer than k distances every element wins: cut = 512, nothing to share out.
__global__ void __launch_bounds__(kSaBins) global_cut_kernel(const uint32_t* __restrict__ all, int G, int rank, int H,
                                                             int k, int2* __restrict__ ext_cut) {
  __shared__ unsigned warp_tot[kSaBins / 32];
  __shared__ int2 result;
  const int head = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) result = make_int2(kSaBins, 0);
  unsigned tot = 0, low = 0, own = 0;
  for (int g = 0; g < G; ++g) {
    const unsigned c = all[(static_cast<size_t>(g) * H + head) * kSaBins + tid];
    tot += c;
    if (g < rank) low += c;
    if (g == rank) own = c;
  }
  unsigned incl = tot;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  unsigned before = 0;
  for (int w2 = 0; w2 < warp; ++w2) before += warp_tot[w2];
  const unsigned excl = before + incl - tot;
  const unsigned want = static_cast<unsigned>(k);
  if (excl < want && excl + tot >= want) {   // exactly one thread, if the sequence holds k distances
    const unsigned need = want - excl;       // cut-valued winners in all
    const unsigned take = need > low ? min(need - low, own) : 0u;
    result = make_int2(tid, static_cast<int>(take));
  }
  __syncthreads();
  if (tid == 0) ext_cut[head] = result;
}

}  // namespace adamas
