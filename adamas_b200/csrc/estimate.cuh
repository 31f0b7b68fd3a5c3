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

namespace adamas {

constexpr int kEstTile = 32;      // tokens per tile
constexpr int kEstConsumerWarps = 16;
constexpr int kEstThreads = (kEstConsumerWarps + 1) * 32;   // 16 consumer warps + 1 producer warp
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
  int num_tiles;
};

// Dynamic shared memory: kEstStages * kEstTile * (2H + 1) * 16 bytes (ring), plus 2H * 32 bytes of
// query planes when HPW == 0.
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
  const int H = p.H;
  const int cpt = 2 * H;                      // 16-byte chunks per token
  const int row_chunks = cpt + 1;             // padded row: lanes reading one chunk position of 32
                                              // consecutive tokens hit 32 different bank groups
  const int stage_chunks = kEstTile * row_chunks;
  OutT* out = static_cast<OutT*>(p.out);

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kEstStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kEstConsumerWarps);
    }
    mbar_fence_init();
  }
  QPlanes* sq = reinterpret_cast<QPlanes*>(est_smem + kEstStages * stage_chunks);
  if (HPW == 0) {
    // generic path: the query planes go through shared memory, so the query code (written by the
    // preceding append kernel) is needed before the block barrier
    grid_dependency_wait();
    for (int c = tid; c < cpt; c += kEstThreads) sq[c] = make_qplanes<METRIC>(__ldg(p.q_code + c));
  }
  __syncthreads();

  const int my_tiles = (p.num_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);

  if (warp == kEstConsumerWarps) {
    // ---- producer warp: one bulk copy per token (its H codes) into the padded ring slot -----------
    const unsigned token_bytes = static_cast<unsigned>(cpt) * 16u;
    int slot = 0;
    unsigned parity = 0;   // parity of the previous use of the slot, for the empty barrier
    for (int j = 0; j < my_tiles; ++j) {
      const int tile0 = (blockIdx.x + j * gridDim.x) * kEstTile;
      const int tile_tokens = min(kEstTile, p.n_tokens - tile0);
      if (j >= kEstStages) {
        // every consumer warp has finished reading the tile that used this slot before
        if (!mbar_wait_bounded(&empty_bar[slot], parity, 1u << 22)) atomicOr(&g_adamas_error, kErrEstimateTimeout);
      }
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[slot], static_cast<unsigned>(tile_tokens) * token_bytes);
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
        bulk_copy_g2s(est_smem + slot * stage_chunks + lane * row_chunks, p.codes + tok * cpt, token_bytes,
                      &full_bar[slot]);
      }
      if (++slot == kEstStages) {
        slot = 0;
        if (j >= kEstStages) parity ^= 1u;
      }
    }
    grid_launch_dependents();
    return;
  }

  // ---- consumer warps: lane = token of the tile, a warp covers its heads -------------------------
  // The cached codes the producer streams were final before the preceding kernel started; the query
  // code is that kernel's output, so the consumers wait for it here (the producer does not).
  grid_dependency_wait();
  grid_launch_dependents();
  QPlanes qp[HPW > 0 ? HPW : 1][2];
  if (HPW > 0) {
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
      qp[hh][0] = make_qplanes<METRIC>(__ldg(p.q_code + 2 * (warp * HPW + hh)));
      qp[hh][1] = make_qplanes<METRIC>(__ldg(p.q_code + 2 * (warp * HPW + hh) + 1));
    }
  }
  int slot = 0;
  unsigned parity = 0;
  for (int j = 0; j < my_tiles; ++j) {
    const int tile0 = (blockIdx.x + j * gridDim.x) * kEstTile;
    const int tile_tokens = min(kEstTile, p.n_tokens - tile0);
    // bounded wait for this tile's bytes; on failure flag the error and carry on (results are then
    // wrong, which the flag reports, but nothing spins forever)
    if (!mbar_wait_bounded(&full_bar[slot], parity, 1u << 22)) atomicOr(&g_adamas_error, kErrEstimateTimeout);
    const uint4* row = est_smem + slot * stage_chunks + lane * row_chunks;
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
      }
    } else {
      for (int h = warp; h < H; h += kEstConsumerWarps) {
        const unsigned d = chunk_distance<METRIC>(row[2 * h], sq[2 * h]) + chunk_distance<METRIC>(row[2 * h + 1], sq[2 * h + 1]);
        if (lane < tile_tokens) o[static_cast<int64_t>(h) * p.out_stride] = dist_to_out<OutT>(d);
      }
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
