// Stage 2 of the decode path: distance between the query's 2-bit code and every cached key code.
//
// The code of (token t, head h) is 32 bytes at ((page*page_size + entry)*H + h)*32 in the code
// cache, so one token's codes for all heads are H*32 contiguous bytes.  The kernel is persistent:
// gridDim.x blocks walk the token tiles round-robin.  A tile is kEstTile consecutive tokens, i.e. a
// flat list of 16-byte chunks (2 per code).  Every thread owns fixed chunk positions of the tile and
// moves them global -> shared with 16-byte cp.async into a kEstStages-deep ring, so that several
// tiles are in flight per block while one is being reduced; a thread only ever reads back the
// chunks it copied itself, so the ring needs no block barrier.  The two halves of a code sit in
// adjacent lanes and are summed with one shfl.xor.  Distances are transposed through a small
// double-buffered shared array so that the [H, n] output is written in runs along the token axis.
//
// The kernel is bound by integer instruction issue as much as by HBM (about 35 integer instructions
// per 16 bytes at best), so index arithmetic is kept out of the inner loops: in the FAST variant
// (2H a power of two that divides the block size, page size a power of two) a thread's chunk
// position inside a code is fixed, its token advances by a constant per round, and all divisions
// are shifts.
//
// L1 distance on packed 2-bit codes, 16 dimensions per 32-bit word w (code c = 2*hi + lo):
//   s = (w >> 1) & 0x55555555          hi bits moved onto the lo positions
//   A = w | s                          lo position: c >= 1, hi position: c >= 2
//   B = w & s                          lo position: c >= 3
//   |c - c'| summed over the word = popc(A ^ A') + popc(B ^ B')     (thermometer code identity)
// The B planes of two words are merged into one popc (they only occupy the lo positions).
#pragma once
#include "common.cuh"

namespace adamas {

constexpr int kEstTile = 32;      // tokens per tile
constexpr int kEstThreads = 512;
constexpr int kEstStages = 3;     // ring depth (tiles in flight per block: kEstStages - 1)

struct QPlanes {
  uint32_t a[4];
  uint32_t b[2];
};

template <int METRIC>
__device__ __forceinline__ QPlanes make_qplanes(uint4 q) {
  QPlanes p;
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  if (METRIC == 0) {
    uint32_t bb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t s = (w[i] >> 1) & 0x55555555u;
      p.a[i] = w[i] | s;
      bb[i] = w[i] & s;
    }
    p.b[0] = bb[0] | (bb[1] << 1);
    p.b[1] = bb[2] | (bb[3] << 1);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) p.a[i] = w[i];
    p.b[0] = p.b[1] = 0;
  }
  return p;
}

// distance contribution of one 16-byte chunk (64 dimensions)
template <int METRIC>
__device__ __forceinline__ unsigned chunk_distance(uint4 kc, const QPlanes& q) {
  const uint32_t w[4] = {kc.x, kc.y, kc.z, kc.w};
  unsigned acc = 0;
  if (METRIC == 0) {
    uint32_t bb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t s = (w[i] >> 1) & 0x55555555u;
      acc += __popc((w[i] | s) ^ q.a[i]);
      bb[i] = w[i] & s;
    }
    acc += __popc((bb[0] | (bb[1] << 1)) ^ q.b[0]);
    acc += __popc((bb[2] | (bb[3] << 1)) ^ q.b[1]);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t x = w[i] ^ q.a[i];
      acc += __popc(x & 0x55555555u) + 2 * __popc(x & 0xAAAAAAAAu);
    }
  }
  return acc;
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
};

// Dynamic shared memory: kEstStages * rounds * kEstThreads * 16 (ring) + 2 * H * (kEstTile + 2) * 2.
// FAST requires cpt_shift >= 0, 2H <= kEstThreads and ps_shift >= 0.  ROUNDS > 0 makes the number of
// chunks per thread and tile a compile-time constant (it must then equal p.rounds).
template <int METRIC, typename OutT, bool FAST, int ROUNDS>
__global__ void __launch_bounds__(kEstThreads) estimate_kernel(const EstimateParams p) {
  extern __shared__ uint4 est_smem[];
  constexpr int PAD = kEstTile + 2;
  const int tid = threadIdx.x;
  const int H = p.H;
  const int cpt = 2 * H;  // chunks per token
  const int rounds = ROUNDS > 0 ? ROUNDS : p.rounds;
  const int stage_chunks = rounds * kEstThreads;
  uint16_t* sdist = reinterpret_cast<uint16_t*>(est_smem + kEstStages * stage_chunks);
  OutT* out = static_cast<OutT*>(p.out);

  // FAST: chunk position inside a code is fixed per thread, the token advances by tl_step per round
  const int c_fixed = FAST ? (tid & (cpt - 1)) : 0;
  const int tl_first = FAST ? (tid >> p.cpt_shift) : 0;
  const int tl_step = FAST ? (kEstThreads >> p.cpt_shift) : 0;
  QPlanes qfix = make_qplanes<METRIC>(__ldg(p.q_code + c_fixed));
  const int sd_base = (c_fixed >> 1) * PAD + tl_first;  // FAST: transpose slot of round 0

  auto issue = [&](int tile, int slot) {
    if (tile < p.num_tiles) {
      const int tile0 = tile * kEstTile;
      const int tile_tokens = min(kEstTile, p.n_tokens - tile0);
      uint4* dst = est_smem + slot * stage_chunks + tid;
      if (FAST) {
#pragma unroll
        for (int r = 0; r < rounds; ++r) {
          const int tl = tl_first + r * tl_step;
          if (tl < tile_tokens) {
            const int t = tile0 + tl;
            const int page = __ldg(p.page_table + (t >> p.ps_shift));
            const int64_t tok = (static_cast<int64_t>(page) << p.ps_shift) + (t & (p.page_size - 1));
            cp_async_16(dst + r * kEstThreads, p.codes + ((tok << p.cpt_shift) + c_fixed));
          }
        }
      } else {
        const int total = tile_tokens * cpt;
        for (int r = 0; r < rounds; ++r) {
          const int f = r * kEstThreads + tid;
          if (f < total) {
            const int tl = f / cpt;
            const int c = f - tl * cpt;
            const int t = tile0 + tl;
            const int lp = t / p.page_size;
            const int e = t - lp * p.page_size;
            const int64_t tok = static_cast<int64_t>(__ldg(p.page_table + lp)) * p.page_size + e;
            cp_async_16(dst + r * kEstThreads, p.codes + tok * cpt + c);
          }
        }
      }
    }
    cp_async_commit();
  };

  int tile = blockIdx.x;
#pragma unroll
  for (int s = 0; s < kEstStages - 1; ++s) issue(tile + s * gridDim.x, s);

  int it = 0;
  int slot = 0;
  for (; tile < p.num_tiles; tile += gridDim.x, ++it) {
    int nslot = slot + (kEstStages - 1);
    if (nslot >= kEstStages) nslot -= kEstStages;
    issue(tile + (kEstStages - 1) * gridDim.x, nslot);
    cp_async_wait<kEstStages - 1>();  // this thread's copies of `tile` have landed

    const int tile0 = tile * kEstTile;
    const int tile_tokens = min(kEstTile, p.n_tokens - tile0);
    const uint4* srcp = est_smem + slot * stage_chunks + tid;
    uint16_t* sd = sdist + (it & 1) * H * PAD;
    if (FAST) {
#pragma unroll
      for (int r = 0; r < rounds; ++r) {
        const bool live = tl_first + r * tl_step < tile_tokens;
        uint4 kc = make_uint4(0, 0, 0, 0);
        if (live) kc = srcp[r * kEstThreads];
        unsigned d = chunk_distance<METRIC>(kc, qfix);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        if (live && (tid & 1) == 0) sd[sd_base + r * tl_step] = static_cast<uint16_t>(d);
      }
    } else {
      const int total = tile_tokens * cpt;
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
    // write out[h, tile0 + tl]: consecutive threads -> consecutive tokens
    for (int i = tid; i < H * kEstTile; i += kEstThreads) {
      const int h = i / kEstTile;
      const int tl = i & (kEstTile - 1);
      if (tl < tile_tokens)
        out[static_cast<int64_t>(h) * p.out_stride + tile0 + tl] = dist_to_out<OutT>(sd[h * PAD + tl]);
    }
    slot = slot + 1 == kEstStages ? 0 : slot + 1;
  }
  cp_async_wait<0>();
}

}  // namespace adamas
