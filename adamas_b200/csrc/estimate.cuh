// Stage 2 of the decode path: distance between the query's 2-bit code and every cached key code.
//
// The code of (token t, head h) is 32 bytes at ((page*page_size + entry)*H + h)*32 in the code
// cache, so one token's codes for all heads are H*32 contiguous bytes.  The kernel is persistent:
// gridDim.x blocks walk tiles of kEstTile = 32 consecutive tokens round-robin.
//   * One producer warp: each lane issues one bulk (TMA) copy per token of the tile (the token's H
//     codes) into a kEstStages-deep shared-memory ring; rows are padded by 16 bytes.  A "full"
//     mbarrier per slot counts the bytes, an "empty" mbarrier per slot collects one arrival per
//     consumer warp before the slot is refilled.
//   * 16 consumer warps: lane l owns token l of the tile, a warp owns a set of heads.  A lane reads
//     the two 16-byte halves of a code (the row padding makes the 32 lanes hit 32 different bank
//     groups), reduces them in registers and stores the distance: the 32 lanes of a warp write 32
//     consecutive tokens of one head, so the [H, n] output needs no transpose, no shuffle and no
//     block barrier; the warps run decoupled from one another.
// All mbarrier waits are bounded; a wait that runs out sets a device error flag and the kernel
// finishes (with wrong results, which the flag reports).
// The distance arithmetic on packed 2-bit codes is described at chunk_distance().
#pragma once
#include "common.cuh"
#include "hadamard_append.cuh"
#include "select_attend.cuh"

namespace adamas {

constexpr int kEstTile = 32;      // tokens per tile
constexpr int kEstConsumerWarps = 16;
constexpr int kEstProducerWarps = 2;   // token-copy kernels: see est_produce
constexpr int kEstThreads = (kEstConsumerWarps + kEstProducerWarps) * 32;
constexpr int kEstPagesThreads = (kEstConsumerWarps + 1) * 32;   // page-copy kernel: 16 consumer warps + 1 producer warp
constexpr int kEstStages = 3;     // ring depth (tiles in flight per block: kEstStages - 1)

struct QPlanes {
  uint32_t qw[4];   // the query's packed codes
  uint32_t qd[4];   // METRIC 0: (q_hi ^ q_lo) of every dimension, at the hi bit positions
};

__device__ __forceinline__ uint32_t lop3_70(uint32_t a, uint32_t b, uint32_t c) {  // a & ~(b & c)
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x70;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t lop3_e4(uint32_t a, uint32_t b, uint32_t c) {  // (a & c) | (b & ~c)
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xE4;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <int METRIC>
__device__ __forceinline__ QPlanes make_qplanes(uint4 q) {
  QPlanes p;
  p.qw[0] = q.x; p.qw[1] = q.y; p.qw[2] = q.z; p.qw[3] = q.w;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.qd[i] = ((p.qw[i] << 1) ^ p.qw[i]) & 0xAAAAAAAAu;
  return p;
}

// Distance contribution of one 16-byte chunk (64 dimensions), 25 integer instructions.
// With x = k ^ q per dimension (x1, x0):  |k - q| = x0 + 2*x1 - 2*[x1 & x0 & (q1 ^ q0)]
// (the correction fires exactly for the code pairs {1, 2}).  Clearing x1 where the bracket holds
// gives y with |k - q| = y0 + 2*y1, so a word contributes popc(y) + popc(y & HI); the second terms of
// two words share one popc.  The XOR metric of the reference's CUDA kernel is the same without the
// correction.
template <int METRIC>
__device__ __forceinline__ unsigned chunk_distance(uint4 kc, const QPlanes& q) {
  const uint32_t w[4] = {kc.x, kc.y, kc.z, kc.w};
  uint32_t y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t x = w[i] ^ q.qw[i];
    y[i] = (METRIC == 0) ? lop3_70(x, x << 1, q.qd[i]) : x;
  }
  const uint32_t z0 = lop3_e4(y[0], y[1] >> 1, 0xAAAAAAAAu);
  const uint32_t z1 = lop3_e4(y[2], y[3] >> 1, 0xAAAAAAAAu);
  return (__popc(y[0]) + __popc(y[1]) + __popc(y[2])) + (__popc(y[3]) + __popc(z0) + __popc(z1));
}

template <typename OutT>
__device__ __forceinline__ OutT dist_to_out(unsigned d);
template <>
__device__ __forceinline__ uint16_t dist_to_out<uint16_t>(unsigned d) {
  return static_cast<uint16_t>(d);
}
template <>
__device__ __forceinline__ __half dist_to_out<__half>(unsigned d) {
  return __uint2half_rn(d);  // exact: d <= 384
}

struct EstimateParams {
  const uint4* codes;
  const int32_t* page_table;
  const uint4* q_code;
  void* out;
  int64_t out_stride;
  int n_tokens;
  int H;            // heads of the code cache
  int q_group;      // query heads per cache head (grouped-query attention; 1 otherwise): q_code, out and hist
                    // have H * q_group rows, row r reads the codes of cache head r / q_group (generic kernel only)
  int page_size;
  int ps_shift;     // log2(page_size) or -1
  int groups;       // token groups of 32 per tile: 1, or 2 * 16 / H for H < 16 (generic kernel only): each
                    // of the 16 consumer warps takes one head of two token groups
  int num_tiles;
  // optional: the sequence length (tokens, the newest included) lives on the device; n_tokens is then
  // *seq_len_dev - 1 and num_tiles follows from it (the host values above are upper bounds that size
  // the grid).  Read before the kernel's dependency resolves: the value must be final before the
  // kernel that precedes this one in the stream starts.
  const int32_t* seq_len_dev;
  // optional: per-slice histograms of the distance rows for select_attend, in the histogram rows of its
  // scratch table ([H][kSaScratchWordsPerHead] u32, rows zero on entry); slice = token / (8 * sa_granules_per_block(n_tokens, hist_cl))
  uint32_t* hist;
  int hist_cl;
  // optional (needs seq_len_dev): a batch of sequences, grid.y = sequence, each with gridDim.x blocks.
  // q_code, out and hist have one row per (sequence, head); codes, page table and length are the sequence's.
  const SeqDesc* seqs;
};

// What a block works on: lengths from the host or from the device-resident sequence length, and, in a
// batched launch, its sequence's cache and first row.
struct EstGeom {
  int n_tokens;
  int num_tiles;
  int slice_tokens;   // tokens per histogram slice (a multiple of 32)
  const uint4* codes;
  const int32_t* page_table;
  int row0;           // first row of this sequence in q_code, out and hist
};
__device__ __forceinline__ EstGeom est_geom(const EstimateParams& p, int tile_span) {
  EstGeom g;
  g.n_tokens = p.n_tokens;
  g.num_tiles = p.num_tiles;
  g.codes = p.codes;
  g.page_table = p.page_table;
  g.row0 = 0;
  const int32_t* len = p.seq_len_dev;
  if (p.seqs) {   // (the table of sequences is set up once, long before this launch)
    const int b = blockIdx.y;
    g.codes = static_cast<const uint4*>(p.seqs[b].code_data);
    g.page_table = p.seqs[b].code_table;
    g.row0 = b * p.H * p.q_group;
    len += b;
  }
  if (len) {
    g.n_tokens = __ldg(len) - 1;
    g.num_tiles = (g.n_tokens + tile_span - 1) / tile_span;
  }
  g.slice_tokens = p.hist ? 8 * sa_granules_per_block(g.n_tokens, p.hist_cl) : 1;
  return g;
}

__device__ __forceinline__ void hist_count(uint32_t* hist, int head, int slice, unsigned d) {
  uint32_t* a = hist + static_cast<size_t>(head) * kSaScratchWordsPerHead + (slice << 9) + d;
  asm volatile("red.global.add.u32 [%0], 1;" ::"l"(a) : "memory");
}

// ---- the two halves of the copy pipeline, shared by the kernels below --------------------------------
// Geometry of the ring for H heads: a token's codes are 2H 16-byte chunks, padded by one chunk so
// that lanes reading one chunk position of 32 consecutive tokens hit 32 different bank groups.
struct EstRing {
  uint4* base;
  uint64_t* full_bar;
  uint64_t* empty_bar;
  int cpt;            // 16-byte chunks per token (2H)
  int row_chunks;     // padded row
  int stage_chunks;   // chunks per ring slot
};

__device__ __forceinline__ int est_tiles_of_block(int num_tiles) {
  return max(0, (num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                    static_cast<int>(gridDim.x));
}

// Producer warps: one bulk copy per token (its H codes) into the padded ring slot.  GROUPED: a tile
// holds p.groups groups of 32 tokens.
// A bulk copy with a different address in every lane is issued lane after lane, about 45 ns each
// (measured: the 32 copies of a tile kept a single producer warp busy for 1.4 us, so that it needed
// over 4 us to ask for the first three tiles and the ring was never ahead of the consumers; the SM's
// copy unit itself takes a request every 2 ns).  So the copies of a tile are split over
// kEstProducerWarps warps: producer `pw` issues the tokens tl with (tl / 16) % kEstProducerWarps == pw,
// 16 lanes at a time.  Producer 0 also announces the tile's bytes on the "full" barrier; a copy of
// another producer that lands before that announcement only makes the barrier's byte count negative
// for a moment, which it allows.
__device__ __forceinline__ void est_token_slot(const EstimateParams& p, int t, int* lp, int* e) {
  if (p.ps_shift >= 0) {
    *lp = t >> p.ps_shift;
    *e = t & (p.page_size - 1);
  } else {
    *lp = t / p.page_size;
    *e = t - *lp * p.page_size;
  }
}

template <bool GROUPED>
__device__ __forceinline__ void est_produce(const EstimateParams& p, const EstGeom& g, const EstRing& r, int my_tiles,
                                            int lane, int pw) {
  const unsigned token_bytes = static_cast<unsigned>(r.cpt) * 16u;
  const int tile_span = GROUPED ? kEstTile * p.groups : kEstTile;
  // this lane's tokens of a tile: tl = first_tl, first_tl + 16 * kEstProducerWarps * 2, ... (lanes 0-15 and
  // 16-31 of a producer take alternate 16-token runs of its share)
  const int first_tl = ((lane >> 4) * kEstProducerWarps + pw) * 16 + (lane & 15);
  int slot = 0;
  unsigned parity = 0;   // parity of the previous use of the slot, for the empty barrier
  for (int j = 0; j < my_tiles; ++j) {
    const int tile0 = (blockIdx.x + j * gridDim.x) * tile_span;
    const int tile_tokens = min(tile_span, g.n_tokens - tile0);
    // the physical page of the first token does not depend on the slot: fetch it before waiting
    int64_t tok_first = 0;
    if (first_tl < tile_tokens) {
      int lp, e;
      est_token_slot(p, tile0 + first_tl, &lp, &e);
      tok_first = static_cast<int64_t>(__ldg(g.page_table + lp)) * p.page_size + e;
    }
    if (j >= kEstStages) {
      // every consumer warp has finished reading the tile that used this slot before
      if (!mbar_wait_bounded(&r.empty_bar[slot], parity, 1u << 20)) atomicOr(&g_adamas_error, kErrEstimateTimeout);
    }
    if (pw == 0 && lane == 0) mbar_arrive_expect_tx(&r.full_bar[slot], static_cast<unsigned>(tile_tokens) * token_bytes);
    __syncwarp();
    for (int tl = first_tl; tl < tile_tokens; tl += 32 * kEstProducerWarps) {
      int64_t tok = tok_first;
      if (tl != first_tl) {
        int lp, e;
        est_token_slot(p, tile0 + tl, &lp, &e);
        tok = static_cast<int64_t>(__ldg(g.page_table + lp)) * p.page_size + e;
      }
      bulk_copy_g2s(r.base + slot * r.stage_chunks + tl * r.row_chunks, g.codes + tok * r.cpt, token_bytes,
                    &r.full_bar[slot]);
    }
    if (++slot == kEstStages) {
      slot = 0;
      if (j >= kEstStages) parity ^= 1u;
    }
  }
}

// Consumer warp: lane = token of the tile; the warp covers heads warp*HPW .. (query planes in
// registers, HPW > 0) or heads warp, warp + 16, ... (planes `sq` in shared memory, HPW == 0).
template <int METRIC, typename OutT, int HPW>
__device__ __forceinline__ void est_consume(const EstimateParams& p, const EstGeom& g, const EstRing& r, int my_tiles,
                                            int lane, int warp, const QPlanes (&qp)[HPW > 0 ? HPW : 1][2],
                                            const QPlanes* sq) {
  OutT* out = static_cast<OutT*>(p.out) + static_cast<int64_t>(g.row0) * p.out_stride;   // this sequence's rows
  uint32_t* hist = p.hist ? p.hist + static_cast<size_t>(g.row0) * kSaScratchWordsPerHead : nullptr;
  const int H = p.H;
  const int tile_span = (HPW == 0) ? kEstTile * p.groups : kEstTile;
  int slot = 0;
  unsigned parity = 0;
  for (int j = 0; j < my_tiles; ++j) {
    const int tile0 = (blockIdx.x + j * gridDim.x) * tile_span;
    const int tile_tokens = min(tile_span, g.n_tokens - tile0);
    const int slice = p.hist ? tile0 / g.slice_tokens : 0;   // a 32-token group never straddles two slices
    // bounded wait for this tile's bytes; on failure flag the error and carry on (results are then
    // wrong, which the flag reports, but nothing spins forever)
    if (!mbar_wait_bounded(&r.full_bar[slot], parity, 1u << 20)) atomicOr(&g_adamas_error, kErrEstimateTimeout);
    const uint4* row = r.base + slot * r.stage_chunks + lane * r.row_chunks;
    OutT* o = out + tile0 + lane;
    if (HPW > 0) {
      unsigned d[HPW > 0 ? HPW : 1];
#pragma unroll
      for (int hh = 0; hh < HPW; ++hh) {
        const int h = warp * HPW + hh;
        d[hh] = chunk_distance<METRIC>(row[2 * h], qp[hh][0]) + chunk_distance<METRIC>(row[2 * h + 1], qp[hh][1]);
      }
      if (lane < tile_tokens) {
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh)
          o[static_cast<int64_t>(warp * HPW + hh) * p.out_stride] = dist_to_out<OutT>(d[hh]);
        if (p.hist) {
#pragma unroll
          for (int hh = 0; hh < HPW; ++hh) hist_count(hist, warp * HPW + hh, slice, d[hh]);
        }
      }
    } else if (p.groups > 1) {
      // fewer than 16 heads: H * groups == 32; warp w takes head w % H of token groups w / H and
      // w / H + groups / 2 (two independent distances per lane and tile, as with 32 heads)
      const int h = warp % H;
      const QPlanes q0 = sq[2 * h], q1 = sq[2 * h + 1];
      unsigned d[2];
      int tl[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        tl[rr] = (warp / H + rr * (p.groups >> 1)) * kEstTile + lane;
        const uint4* grow = r.base + slot * r.stage_chunks + tl[rr] * r.row_chunks;
        d[rr] = chunk_distance<METRIC>(grow[2 * h], q0) + chunk_distance<METRIC>(grow[2 * h + 1], q1);
      }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
        if (tl[rr] < tile_tokens) {
          out[static_cast<int64_t>(h) * p.out_stride + tile0 + tl[rr]] = dist_to_out<OutT>(d[rr]);
          if (p.hist) hist_count(hist, h, (tile0 + tl[rr] - lane) / g.slice_tokens, d[rr]);
        }
    } else {
      const int rows = H * p.q_group;
      for (int h = warp; h < rows; h += kEstConsumerWarps) {
        const int hc = p.q_group == 1 ? h : h / p.q_group;   // the cache head this query head reads
        const unsigned d = chunk_distance<METRIC>(row[2 * hc], sq[2 * h]) + chunk_distance<METRIC>(row[2 * hc + 1], sq[2 * h + 1]);
        if (lane < tile_tokens) {
          o[static_cast<int64_t>(h) * p.out_stride] = dist_to_out<OutT>(d);
          if (p.hist) hist_count(hist, h, slice, d);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&r.empty_bar[slot]);
    if (++slot == kEstStages) {
      slot = 0;
      parity ^= 1u;
    }
  }
}

__device__ __forceinline__ EstRing est_ring_init(uint4* smem, uint64_t* full_bar, uint64_t* empty_bar, int H,
                                                 int tid, int groups = 1) {
  EstRing r;
  r.base = smem;
  r.full_bar = full_bar;
  r.empty_bar = empty_bar;
  r.cpt = 2 * H;
  r.row_chunks = r.cpt + 1;
  r.stage_chunks = kEstTile * groups * r.row_chunks;
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kEstStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kEstConsumerWarps);
    }
    mbar_fence_init();
  }
  return r;
}

// Dynamic shared memory: kEstStages * kEstTile * groups * (2H + 1) * 16 bytes (ring), plus 2H * q_group * 32
// bytes of query planes when HPW == 0.
// HPW > 0: H == kEstConsumerWarps * HPW and warp w keeps the query planes of heads w*HPW .. in
// registers.  HPW == 0: any H, warp w handles heads w, w + 16, ... with the planes in shared memory.
template <int METRIC, typename OutT, int HPW>
__global__ void __launch_bounds__(kEstThreads) estimate_kernel(const EstimateParams p) {
  extern __shared__ uint4 est_smem[];
  __shared__ __align__(8) uint64_t full_bar[kEstStages];
  __shared__ __align__(8) uint64_t empty_bar[kEstStages];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const EstRing ring = est_ring_init(est_smem, full_bar, empty_bar, p.H, tid, HPW == 0 ? p.groups : 1);
  QPlanes* sq = reinterpret_cast<QPlanes*>(est_smem + kEstStages * ring.stage_chunks);
  const EstGeom geom = est_geom(p, HPW == 0 ? kEstTile * p.groups : kEstTile);
  const uint4* q_code = p.q_code + 2 * geom.row0;   // this sequence's query codes
  if (HPW == 0) {
    // generic path: the query planes go through shared memory, so the query code (written by the
    // preceding append kernel) is needed before the block barrier
    grid_dependency_wait();
    for (int c = tid; c < ring.cpt * p.q_group; c += kEstThreads) sq[c] = make_qplanes<METRIC>(__ldg(q_code + c));
  }
  __syncthreads();
  const int my_tiles = est_tiles_of_block(geom.num_tiles);
  if (warp >= kEstConsumerWarps) {
    est_produce<HPW == 0>(p, geom, ring, my_tiles, lane, warp - kEstConsumerWarps);
    grid_launch_dependents();
    return;
  }
  // The cached codes the producers stream were final before the preceding kernel started; the query
  // code is that kernel's output, so the consumers wait for it here (the producers do not).
  grid_dependency_wait();
  grid_launch_dependents();
  QPlanes qp[HPW > 0 ? HPW : 1][2];
  if (HPW > 0) {
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
      qp[hh][0] = make_qplanes<METRIC>(__ldg(q_code + 2 * (warp * HPW + hh)));
      qp[hh][1] = make_qplanes<METRIC>(__ldg(q_code + 2 * (warp * HPW + hh) + 1));
    }
  }
  est_consume<METRIC, OutT, HPW>(p, geom, ring, my_tiles, lane, warp, qp, sq);
}

// ---- estimate with the decode append inside (stages 1 + 2 of a decode step in one launch) -------------
// Same pipeline; the consumer warps do not read a query code from memory but make it themselves: warp w
// loads the query rows of its HPW heads (one half-warp per row), transforms, buckets and packs them,
// and spreads the 16 code words of each head over the warp through shared memory.
// Every block does this redundantly (H rows of 256 bytes from L2), so no block waits for another.
// The last block (it has the fewest tiles) also does the append proper for the new token: K and V rows
// into the page slot, the key's code into the code cache, the query code to q_code_out.  None of this
// is read by the scan, which leaves the newest token out; the kernel after this one finds all of it
// complete.  q and k arrive rotated: a rotary embedding in here would be repeated by every block (a
// power and a sine/cosine per element), which costs far more than the append launch this kernel saves.
struct StepAppend {
  const void* q;           // [H,128]
  const void* k;           // [H,128]
  const void* v;           // [H,128]
  uint16_t* q_code_out;    // [H,16]
  PagedTarget tgt;
  int kv_last_page, kv_entry, code_last_page, code_entry;
  float scale;
  Thresholds th;
  RopeParams rp;           // ROPE: q and k arrive un-rotated
};

// ROPE: q and k arrive un-rotated.  Every block forms the position's 64 (cos, sin) pairs once (64 consumer
// threads, before the kernel's dependency resolves: the position does not depend on the preceding kernel) and
// each consumer warp rotates its query rows in registers before it codes them.  The block that appends also
// rotates the key, stores the rotated row into the cache and back into the caller's k.  The caller's q is NOT
// rotated here (other blocks are still reading it un-rotated): the select+attend launch that follows rotates
// it the same way for its own use and writes it back.
template <typename T, int HPW, bool ROPE>
__global__ void __launch_bounds__(kEstThreads) estimate_append_kernel(const EstimateParams p, const StepAppend a) {
  static_assert(HPW == 1 || HPW == 2 || HPW == 4, "heads per warp");
  extern __shared__ uint4 est_smem[];
  __shared__ __align__(8) uint64_t full_bar[kEstStages];
  __shared__ __align__(8) uint64_t empty_bar[kEstStages];
  __shared__ __align__(16) uint16_t s_code[kEstConsumerWarps][32];   // a warp's two rows of code words
  __shared__ float2 s_cs[ROPE ? kHeadDim / 2 : 1];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const EstRing ring = est_ring_init(est_smem, full_bar, empty_bar, p.H, tid);
  __syncthreads();
  const EstGeom geom = est_geom(p, kEstTile);
  const int my_tiles = est_tiles_of_block(geom.num_tiles);
  if (warp >= kEstConsumerWarps) {
    // the cached codes were final before the preceding kernel started: stream them right away
    est_produce<false>(p, geom, ring, my_tiles, lane, warp - kEstConsumerWarps);
    grid_launch_dependents();
    return;
  }
  if (ROPE) {
    // the new token sits at position n_tokens (= tokens before it)
    if (tid < kHeadDim / 2) s_cs[tid] = rope_cos_sin(tid, static_cast<float>(geom.n_tokens), a.rp);
    asm volatile("bar.sync 1, %0;" ::"n"(kEstConsumerWarps * 32) : "memory");   // the consumer warps only
  }
  // q, k, v are the preceding kernel's output
  grid_dependency_wait();
  grid_launch_dependents();

  const bool appender = blockIdx.x == gridDim.x - 1;
  // slot of the new token: from the host, or from the device-resident sequence length (position n)
  int kv_last_page = a.kv_last_page, kv_entry = a.kv_entry, code_last_page = a.code_last_page, code_entry = a.code_entry;
  if (p.seq_len_dev) {
    kv_last_page = code_last_page = geom.n_tokens / p.page_size;
    kv_entry = code_entry = geom.n_tokens - kv_last_page * p.page_size;
  }
  const unsigned l16 = lane & 15;
  const int half = lane >> 4;
  const int H = p.H;
  PagedTarget tgt = a.tgt;
  if (p.seqs) {
    const SeqDesc sd = p.seqs[blockIdx.y];
    tgt.kv_data = sd.kv_data;
    tgt.kv_table = sd.kv_table;
    tgt.code_data = static_cast<uint16_t*>(sd.code_data);
    tgt.code_table = sd.code_table;
  }
  QPlanes qp[HPW][2];
#pragma unroll
  for (int pass = 0; pass < (HPW + 1) / 2; ++pass) {
    // this half-warp's row: head warp*HPW + 2*pass + half (HPW == 1: both halves take the one head)
    const int hh_mine = (HPW == 1) ? 0 : 2 * pass + half;
    const int head = warp * HPW + hh_mine;
    const int64_t in_off = static_cast<int64_t>(geom.row0 + head) * kHeadDim + l16 * 8;   // rows of q, k, v: (sequence, head)
    const bool writer = appender && (HPW > 1 || half == 0);
    float x[8];
    unpack8<T>(ld_16(static_cast<const T*>(a.q) + in_off), x);
    if (ROPE) rope_halfwarp_cs<T>(x, l16, s_cs, a.rp.inv_freq != nullptr, a.rp.mscale);
    wht128_halfwarp(x, l16);
    scale_round<T>(x, a.scale);
    const unsigned word = bucketize_pack8(x, a.th);   // code word l16 of `head`
    if (writer) a.q_code_out[(geom.row0 + head) * kCodeWords + l16] = static_cast<uint16_t>(word);
    // spread the 16 code words of each row over the warp: through shared memory (one 2-byte store per
    // lane, two 16-byte broadcast loads per head)
    __syncwarp();
    s_code[warp][lane] = static_cast<uint16_t>(word);
    __syncwarp();
#pragma unroll
    for (int s = 0; s < (HPW == 1 ? 1 : 2); ++s) {
      const uint4* cw = reinterpret_cast<const uint4*>(&s_code[warp][16 * s]);
      const int hh = (HPW == 1) ? 0 : 2 * pass + s;
      qp[hh][0] = make_qplanes<0>(cw[0]);
      qp[hh][1] = make_qplanes<0>(cw[1]);
    }
    if (appender) {   // block-uniform
      const int kv_page = __ldg(tgt.kv_table + kv_last_page);
      const int code_page = __ldg(tgt.code_table + code_last_page);
      const int ps = tgt.page_size;
      T* kv = static_cast<T*>(tgt.kv_data);
      const int64_t k_off =
          ((static_cast<int64_t>(kv_page) * 2 * ps + kv_entry) * H + head) * kHeadDim + l16 * 8;
      const int64_t v_delta = static_cast<int64_t>(ps) * H * kHeadDim;
      uint4 kraw = ld_16(static_cast<const T*>(a.k) + in_off);
      const uint4 vraw = ld_16(static_cast<const T*>(a.v) + in_off);
      float b[8];
      unpack8<T>(kraw, b);
      if (ROPE) {
        rope_halfwarp_cs<T>(b, l16, s_cs, a.rp.inv_freq != nullptr, a.rp.mscale);
        kraw = pack8<T>(b);
        if (writer) st_16(static_cast<T*>(const_cast<void*>(a.k)) + in_off, kraw);
      }
      if (writer) {
        st_16(kv + k_off, kraw);
        st_16(kv + k_off + v_delta, vraw);
      }
      wht128_halfwarp(b, l16);
      scale_round<T>(b, a.scale);
      if (writer) {
        const int64_t c_off =
            ((static_cast<int64_t>(code_page) * ps + code_entry) * H + head) * kCodeWords + l16;
        tgt.code_data[c_off] = bucketize_pack8(b, a.th);
      }
    }
  }
  est_consume<0, uint16_t, HPW>(p, geom, ring, my_tiles, lane, warp, qp, nullptr);
}

// ---- few heads per GPU: whole pages per copy, one 16-byte chunk per lane ---------------------------------
// With H <= 16 heads (a head-sharded model) a token's codes are only H*32 bytes, and one bulk copy per
// token leaves the producer warp issuing thousands of 128- to 512-byte copies.  A page of the code cache
// is contiguous (page_size * H * 32 bytes), so this kernel copies whole pages and lays them out back to
// back in shared memory.  Consumers take one 16-byte chunk per lane: 32 consecutive chunks per warp
// step (conflict-free), lane l always holds half (l & 1) of head (l % 2H) / 2, so its query planes stay
// in registers; the two halves of a (token, head) are joined by one shuffle.  Needs 2H | 32.  Partial
// last units read a few chunks past the valid ones (the allocation has 512 spare bytes).
constexpr int kEstLookahead = 8;   // tiles whose page numbers the page-copy producer fetches together

struct EstimatePagesParams {
  const uint4* codes;
  const int32_t* page_table;
  const uint4* q_code;
  void* out;
  int64_t out_stride;
  int n_tokens;
  int H;
  int page_size;
  int pages_per_tile;
  int num_tiles;
  int stage_out;    // gather the distances of 8 tokens per head in shared memory before writing them
  const int32_t* seq_len_dev;   // optional device-resident sequence length, as in EstimateParams
  uint32_t* hist;               // optional per-slice histograms, as in EstimateParams
  int hist_cl;
  const SeqDesc* seqs;          // optional batch of sequences (grid.y = sequence), as in EstimateParams
};

template <int METRIC, typename OutT>
__global__ void __launch_bounds__(kEstPagesThreads, 2) estimate_pages_kernel(const EstimatePagesParams p) {
  extern __shared__ uint4 est_smem[];
  __shared__ __align__(8) uint64_t full_bar[kEstStages];
  __shared__ __align__(8) uint64_t empty_bar[kEstStages];
  __shared__ __align__(16) uint16_t s_stage[kEstConsumerWarps][16][16];   // per warp: [head][token of the unit]
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int H2 = 2 * p.H;                              // chunks per token
  const int page_chunks = p.page_size * H2;
  const int tile_chunks = p.pages_per_tile * page_chunks;
  const int tile_span = p.pages_per_tile * p.page_size;   // tokens per tile
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kEstStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kEstConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  int n_tokens = p.n_tokens, num_tiles = p.num_tiles;
  const uint4* codes = p.codes;
  const int32_t* page_table = p.page_table;
  const int32_t* len = p.seq_len_dev;
  int row0 = 0;
  if (p.seqs) {
    const int b = blockIdx.y;
    codes = static_cast<const uint4*>(p.seqs[b].code_data);
    page_table = p.seqs[b].code_table;
    len += b;
    row0 = b * p.H;
  }
  if (len) {
    n_tokens = __ldg(len) - 1;
    num_tiles = (n_tokens + tile_span - 1) / tile_span;
  }
  const int slice_tokens = p.hist ? 8 * sa_granules_per_block(n_tokens, p.hist_cl) : 1;
  const int my_tiles = est_tiles_of_block(num_tiles);

  if (warp == kEstConsumerWarps) {
    // ---- producer: one bulk copy per page of the tile (the last page of the row may be partial); the
    // page numbers of the next kEstLookahead tiles are fetched together, ahead of the copies
    int slot = 0;
    unsigned parity = 0;
    for (int j0 = 0; j0 < my_tiles; j0 += kEstLookahead) {
      int page[kEstLookahead];
#pragma unroll
      for (int u = 0; u < kEstLookahead; ++u) {
        const int tile = blockIdx.x + (j0 + u) * gridDim.x;
        const int tok0 = tile * tile_span;
        page[u] = 0;
        if (j0 + u < my_tiles && tok0 + lane * p.page_size < n_tokens)
          page[u] = __ldg(page_table + tile * p.pages_per_tile + lane);
      }
#pragma unroll
      for (int u = 0; u < kEstLookahead; ++u) {
        const int j = j0 + u;
        if (j >= my_tiles) break;
        const int tile = blockIdx.x + j * gridDim.x;
        const int tok0 = tile * tile_span;
        const int ntok = min(tile_span, n_tokens - tok0);
        if (j >= kEstStages) {
          if (!mbar_wait_bounded(&empty_bar[slot], parity, 1u << 20)) atomicOr(&g_adamas_error, kErrEstimateTimeout);
        }
        if (lane == 0) mbar_arrive_expect_tx(&full_bar[slot], static_cast<unsigned>(ntok) * H2 * 16u);
        __syncwarp();
        const int npages = (ntok + p.page_size - 1) / p.page_size;   // at most 32: one per lane
        if (lane < npages) {
          const int64_t phys = page[u];
          const int toks = min(p.page_size, ntok - lane * p.page_size);
          bulk_copy_g2s(est_smem + slot * tile_chunks + lane * page_chunks, codes + phys * page_chunks,
                        static_cast<unsigned>(toks) * H2 * 16u, &full_bar[slot]);
        }
        if (++slot == kEstStages) {
          slot = 0;
          if (j >= kEstStages) parity ^= 1u;
        }
      }
    }
    grid_launch_dependents();
    return;
  }

  // ---- consumers ------------------------------------------------------------------------------------
  grid_dependency_wait();
  grid_launch_dependents();
  const int half = lane & 1;
  const int h = (lane % H2) >> 1;
  const QPlanes qp = make_qplanes<METRIC>(__ldg(p.q_code + 2 * (row0 + h) + half));
  const int toks_per_step = 32 / H2;
  const int tok_in_step = lane / H2;
  // A warp works in units of 8 consecutive tokens (16 for one head).  With stage_out its lanes drop
  // their distances into a warp-private table [head][token], then one lane per head (and 8-token part)
  // writes 16 contiguous bytes of the head's output row: with 16 heads a step covers one token, and
  // isolated 2-byte stores to 16 different rows cost more than the scan itself.  With fewer heads a
  // step already writes runs of 2 to 16 tokens per row, and direct stores are faster.
  const int unit_tok = max(8, toks_per_step);
  const int steps_per_unit = unit_tok / toks_per_step;
  const int parts = unit_tok >> 3;
  uint16_t(*stage)[16] = s_stage[warp];
  OutT* out = static_cast<OutT*>(p.out) + static_cast<int64_t>(row0) * p.out_stride;   // this sequence's rows
  uint32_t* hist = p.hist ? p.hist + static_cast<size_t>(row0) * kSaScratchWordsPerHead : nullptr;
  const bool rows_aligned = ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0) && ((p.out_stride * sizeof(OutT)) % 16 == 0);
  int slot = 0;
  unsigned parity = 0;
  for (int j = 0; j < my_tiles; ++j) {
    const int tile = blockIdx.x + j * gridDim.x;
    const int tok0 = tile * tile_span;
    const int ntok = min(tile_span, n_tokens - tok0);
    const int slice0 = p.hist ? tok0 / slice_tokens : 0;
    const int off0 = tok0 - slice0 * slice_tokens;
    if (!mbar_wait_bounded(&full_bar[slot], parity, 1u << 20)) atomicOr(&g_adamas_error, kErrEstimateTimeout);
    const uint4* base = est_smem + slot * tile_chunks;
    const int units = (ntok + unit_tok - 1) / unit_tok;
    for (int u = warp; u < units; u += kEstConsumerWarps) {
      const uint4* ubase = base + u * steps_per_unit * 32 + lane;
#pragma unroll 4
      for (int st = 0; st < steps_per_unit; ++st) {
        unsigned d = chunk_distance<METRIC>(ubase[st * 32], qp);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        if (half == 0) {
          const OutT v = dist_to_out<OutT>(d);
          const int t = st * toks_per_step + tok_in_step;
          if (p.stage_out) {
            stage[h][t] = *reinterpret_cast<const uint16_t*>(&v);
          } else if (u * unit_tok + t < ntok) {
            out[static_cast<int64_t>(h) * p.out_stride + tok0 + u * unit_tok + t] = v;
          }
          if (p.hist && u * unit_tok + t < ntok) {
            const int off = off0 + u * unit_tok + t;
            hist_count(hist, h, slice0 + (off >= slice_tokens ? off / slice_tokens : 0), d);
          }
        }
      }
      if (!p.stage_out) continue;
      __syncwarp();
      if (lane < p.H * parts) {
        const int row = lane / parts;
        const int t_base = u * unit_tok + (lane % parts) * 8;
        if (t_base < ntok) {
          OutT* dst = out + static_cast<int64_t>(row) * p.out_stride + tok0 + t_base;
          const uint16_t* src = &stage[row][(lane % parts) * 8];
          if (rows_aligned && ((tok0 + t_base) & 7) == 0 && t_base + 8 <= ntok) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
          } else {
            for (int k = 0; k < 8 && t_base + k < ntok; ++k) reinterpret_cast<uint16_t*>(dst)[k] = src[k];
          }
        }
      }
      __syncwarp();
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[slot]);
    if (++slot == kEstStages) {
      slot = 0;
      parity ^= 1u;
    }
  }
}

}  // namespace adamas
