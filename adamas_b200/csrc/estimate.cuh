// Stage 2 of the decode path: distance between the query's 2-bit code and every cached key code.
//
// The code of (token t, head h) is 32 bytes at ((page*page_size + entry)*H + h)*32 in the code
// cache, so one token's codes for all heads are H*32 contiguous bytes.  The kernel is persistent:
// gridDim.x blocks walk the token tiles round-robin.  A tile is kEstTile consecutive tokens, i.e. a
// flat list of 16-byte chunks (2 per code).  Warp 0 is the producer: each of its lanes issues one
// bulk (TMA) copy per token of the tile (the token's H codes, contiguous) into a kEstStages-deep
// shared-memory ring, completion counted on one mbarrier per ring slot, so that several tiles are in
// flight per block while one is being reduced.  All warps consume: every thread owns fixed chunk
// positions of the tile; the two halves of a code sit in adjacent lanes and are summed with one
// shfl.xor.  Waits on the mbarriers are bounded (a timeout sets a device error flag).  Distances are transposed through a small
// double-buffered shared array so that the [H, n] output is written in runs along the token axis.
//
// The kernel is bound by integer instruction issue as much as by HBM, so index arithmetic is kept
// out of the inner loops: in the FAST variant (2H a power of two between 16 and the block size) a
// thread's chunk position inside a code is fixed and its token advances by a constant per round.
//
// The distance arithmetic on packed 2-bit codes is described at chunk_distance().
#pragma once
#include "common.cuh"

namespace adamas {

constexpr int kEstTile = 32;      // tokens per tile
constexpr int kEstThreads = 512;
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
  int H;
  int page_size;
  int ps_shift;     // log2(page_size) or -1
  int cpt_shift;    // log2(2H) or -1
  int num_tiles;
  int rounds;       // ceil(kEstTile * 2H / kEstThreads)
  int out_pairs_aligned;  // out rows start on 4-byte boundaries (stride even, base aligned)
};

// Dynamic shared memory: kEstStages * kEstTile * H * 32 (ring) + 2 * H * (kEstTile + 2) * 2.
// FAST requires cpt_shift >= 4 (H >= 8) and 2H <= kEstThreads.  ROUNDS > 0 makes the number of chunks per
// thread and tile a compile-time constant (it must then equal p.rounds).
template <int METRIC, typename OutT, bool FAST, int ROUNDS>
__global__ void __launch_bounds__(kEstThreads) estimate_kernel(const EstimateParams p) {
  extern __shared__ uint4 est_smem[];
  __shared__ __align__(8) uint64_t bars[kEstStages];
  constexpr int PAD = kEstTile + 2;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int H = p.H;
  const int cpt = 2 * H;  // 16-byte chunks per token
  const int rounds = ROUNDS > 0 ? ROUNDS : p.rounds;
  const int stage_chunks = kEstTile * cpt;
  uint16_t* sdist = reinterpret_cast<uint16_t*>(est_smem + kEstStages * stage_chunks);
  OutT* out = static_cast<OutT*>(p.out);

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kEstStages; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncthreads();

  // Producer (warp 0, one lane per token of the tile): one bulk copy of the token's H codes.
  auto produce = [&](int tile, int slot) {
    if (tile < p.num_tiles) {
      const int tile0 = tile * kEstTile;
      const int tile_tokens = min(kEstTile, p.n_tokens - tile0);
      const unsigned token_bytes = static_cast<unsigned>(cpt) * 16u;
      if (lane == 0) mbar_arrive_expect_tx(&bars[slot], static_cast<unsigned>(tile_tokens) * token_bytes);
      __syncwarp();
      if (lane < tile_tokens) {
        const int t = tile0 + lane;
        int lp, e;
        if (p.ps_shift >= 0) {
          lp = t >> p.ps_shift;
          e = t & (p.page_size - 1);
        } else {
          lp = t / p.page_size;
          e = t - lp * p.page_size;
        }
        const int64_t tok = static_cast<int64_t>(__ldg(p.page_table + lp)) * p.page_size + e;
        bulk_copy_g2s(est_smem + slot * stage_chunks + lane * cpt, p.codes + tok * cpt, token_bytes,
                      &bars[slot]);
      }
    }
  };

  // FAST: chunk position inside a code is fixed per thread, the token advances by tl_step per round
  const int c_fixed = FAST ? (tid & (cpt - 1)) : 0;
  const int tl_first = FAST ? (tid >> p.cpt_shift) : 0;
  const int tl_step = FAST ? (kEstThreads >> p.cpt_shift) : 0;
  const QPlanes qfix = make_qplanes<METRIC>(__ldg(p.q_code + c_fixed));
  const int sd_base = (c_fixed >> 1) * PAD + tl_first;  // FAST: transpose slot of round 0

  int tile = blockIdx.x;
  if (tid < 32) {
#pragma unroll
    for (int s = 0; s < kEstStages - 1; ++s) produce(tile + s * gridDim.x, s);
  }

  int it = 0;
  int slot = 0;
  unsigned parity = 0;
  for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
    int nslot = slot + (kEstStages - 1);
    if (nslot >= kEstStages) nslot -= kEstStages;
    if (tid < 32) produce(tile + (kEstStages - 1) * gridDim.x, nslot);

    // bounded wait for this tile's bytes; on failure flag the error and carry on (results are
    // then wrong, which the flag reports, but nothing spins forever)
    if (!mbar_wait_bounded(&bars[slot], parity, 1u << 22)) atomicOr(&g_adamas_error, kErrEstimateTimeout);

    const int tile0 = tile * kEstTile;
    const int tile_tokens = min(kEstTile, p.n_tokens - tile0);
    const uint4* srcp = est_smem + slot * stage_chunks + tid;
    uint16_t* sd = sdist + (it & 1) * H * PAD;
    if (FAST) {
      unsigned d[ROUNDS > 0 ? ROUNDS : 1];
      if (ROUNDS > 0) {
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) d[r] = chunk_distance<METRIC>(srcp[r * kEstThreads], qfix);
#pragma unroll
        for (int r = 0; r < ROUNDS; ++r) d[r] += __shfl_xor_sync(0xffffffffu, d[r], 1);
        if ((tid & 1) == 0) {
#pragma unroll
          for (int r = 0; r < ROUNDS; ++r) sd[sd_base + r * tl_step] = static_cast<uint16_t>(d[r]);
        }
      } else {
        for (int r = 0; r < rounds; ++r) {
          unsigned dd = chunk_distance<METRIC>(srcp[r * kEstThreads], qfix);
          dd += __shfl_xor_sync(0xffffffffu, dd, 1);
          if ((tid & 1) == 0) sd[sd_base + r * tl_step] = static_cast<uint16_t>(dd);
        }
      }
    } else {
      const int total = kEstTile * cpt;
      for (int r = 0; r < rounds; ++r) {
        const int f = r * kEstThreads + tid;
        const bool live = f < total;
        const int tl = f / cpt;
        const int c = f - tl * cpt;
        uint4 kc = make_uint4(0, 0, 0, 0);
        if (live) kc = srcp[r * kEstThreads];
        const QPlanes qp = make_qplanes<METRIC>(__ldg(p.q_code + (live ? c : 0)));
        unsigned d = chunk_distance<METRIC>(kc, qp);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        if (live && (c & 1) == 0) sd[(c >> 1) * PAD + tl] = static_cast<uint16_t>(d);
      }
    }
    __syncthreads();
    // write out[h, tile0 + tl]: one thread per pair of tokens, consecutive threads -> consecutive
    // pairs (tokens past the end of a partial tile hold stale bytes and are skipped)
    for (int i = tid; i < H * (kEstTile / 2); i += kEstThreads) {
      const int h = i / (kEstTile / 2);
      const int tl = (i & (kEstTile / 2 - 1)) * 2;
      const uint32_t two = *reinterpret_cast<const uint32_t*>(sd + h * PAD + tl);
      OutT* o = out + static_cast<int64_t>(h) * p.out_stride + tile0 + tl;
      const OutT lo = dist_to_out<OutT>(two & 0xffffu), hi = dist_to_out<OutT>(two >> 16);
      if (p.out_pairs_aligned && tl + 1 < tile_tokens) {
        uint32_t packed;
        const uint16_t lo16 = *reinterpret_cast<const uint16_t*>(&lo), hi16 = *reinterpret_cast<const uint16_t*>(&hi);
        packed = static_cast<uint32_t>(lo16) | (static_cast<uint32_t>(hi16) << 16);
        *reinterpret_cast<uint32_t*>(o) = packed;
      } else {
        if (tl < tile_tokens) o[0] = lo;
        if (tl + 1 < tile_tokens) o[1] = hi;
      }
    }
    if (++slot == kEstStages) {
      slot = 0;
      parity ^= 1u;
    }
  }
}

}  // namespace adamas
