// Stage 2 of the decode path: distance between the query's 2-bit code and every cached key code.
//
// The code of (token t, head h) is 32 bytes at ((page*page_size + entry)*H + h)*32 in the code
// cache, so one token's codes for all heads are H*32 contiguous bytes.  A thread block takes a tile
// of TILE consecutive tokens; the tile is a flat list of 16-byte chunks (2 per code) which the
// threads read with coalesced 128-bit streaming loads, all issued before any is used.  The two
// halves of a code sit in adjacent lanes and are summed with one shfl.xor.  Distances are transposed
// through shared memory so that the [H, n] output is written in runs along the token axis.
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

constexpr int kEstTile = 32;      // tokens per thread block
constexpr int kEstThreads = 256;
constexpr int kEstBatch = 8;      // 16-byte loads in flight per thread

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

// grid.x = ceil(n_tokens / kEstTile).  Dynamic shared memory: H * (kEstTile + 2) uint16.
template <int METRIC, typename OutT>
__global__ void __launch_bounds__(kEstThreads)
estimate_kernel(const uint4* __restrict__ codes, const int32_t* __restrict__ page_table,
                const uint4* __restrict__ q_code, OutT* __restrict__ out, int64_t out_stride,
                int n_tokens, int H, int page_size) {
  extern __shared__ uint16_t sdist[];
  constexpr int PAD = kEstTile + 2;
  const int tile0 = blockIdx.x * kEstTile;
  const int chunks_per_token = 2 * H;
  const int tile_tokens = min(kEstTile, n_tokens - tile0);
  const int total = tile_tokens * chunks_per_token;

  for (int base = 0; base < total; base += kEstThreads * kEstBatch) {
    uint4 kc[kEstBatch];
    int cidx[kEstBatch];
    int tloc[kEstBatch];
    // issue all loads of the batch first
#pragma unroll
    for (int r = 0; r < kEstBatch; ++r) {
      const int f = base + r * kEstThreads + threadIdx.x;
      kc[r] = make_uint4(0, 0, 0, 0);
      tloc[r] = -1;
      cidx[r] = 0;
      if (f < total) {
        const int tl = f / chunks_per_token;
        const int c = f - tl * chunks_per_token;
        const int t = tile0 + tl;
        const int lp = t / page_size;
        const int e = t - lp * page_size;
        const int64_t slot = static_cast<int64_t>(__ldg(page_table + lp)) * page_size + e;
        kc[r] = ld_stream_16(codes + slot * chunks_per_token + c);
        tloc[r] = tl;
        cidx[r] = c;
      }
    }
#pragma unroll
    for (int r = 0; r < kEstBatch; ++r) {
      const QPlanes qp = make_qplanes<METRIC>(__ldg(q_code + cidx[r]));
      unsigned d = chunk_distance<METRIC>(kc[r], qp);
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      if (tloc[r] >= 0 && (cidx[r] & 1) == 0) {
        sdist[(cidx[r] >> 1) * PAD + tloc[r]] = static_cast<uint16_t>(d);
      }
    }
  }
  __syncthreads();
  // write out[h, tile0 + tl]: consecutive threads -> consecutive tokens
  for (int i = threadIdx.x; i < H * kEstTile; i += kEstThreads) {
    const int h = i / kEstTile;
    const int tl = i - h * kEstTile;
    if (tl < tile_tokens) {
      out[static_cast<int64_t>(h) * out_stride + tile0 + tl] = dist_to_out<OutT>(sdist[h * PAD + tl]);
    }
  }
}

}  // namespace adamas
