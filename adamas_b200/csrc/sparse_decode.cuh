// Stage 4 of the decode path: decode attention of one query row per head over a per-head list of
// selected token slots (plus an always-attended tail) in the paged KV cache.
//
// grid = (num_splits, H).  A thread block walks its share of the head's token list in tiles of
// kDecTile tokens.  For each tile it resolves the token slots from the index list, gathers the
// 256-byte K and V rows into shared memory with one bulk (TMA) copy per row (double buffered across
// tiles, one mbarrier per stage counting the bytes; waits are bounded), computes the logits with two
// threads per token, runs an online softmax in base 2, and accumulates P.V with one thread per (token
// group, 8-dim chunk).  Rows are padded to 272 bytes so that both access patterns are bank-conflict
// free.
//
// With more than one split per head each block writes an unnormalised partial (o, m, l) to global
// scratch, and the block that arrives last at the head's counter merges the partials and writes the
// output (no block ever waits for another).  The counter is left at zero for the next launch.
#pragma once
#include "common.cuh"

namespace adamas {

constexpr int kDecTile = 64;       // tokens per tile
constexpr int kDecThreads = 128;
constexpr int kDecRowBytes = kHeadDim * 2 + 16;             // a row plus 16 bytes of padding
constexpr int kDecStageBytes = 2 * kDecTile * kDecRowBytes;  // K + V rows of one tile (34 KB)

struct DecodeParams {
  const void* q;          // [H, 128]
  void* o;                // [H, 128] in the cache's element type, or null
  float* o_f32;           // [H, 128] fp32 output (partial results of a sequence shard), or null
  float* lse;             // [H] or null (base-2 log-sum-exp of the scaled logits)
  const void* kv;         // [pages, 2, page_size, H, 128]
  const int32_t* indices; // [H, idx_stride]
  int64_t idx_stride;
  int n_idx;              // indices used per head
  int idx_unit;           // token slots covered by one index
  int page_size;
  int H;                  // heads of the KV cache
  int q_group;            // query heads per cache head (1: multi-head attention); the grid has H * q_group rows
  unsigned tail_slot0;    // physical token slot of the first tail token
  int ps_shift;           // log2(page_size) or -1
  int n_tokens;           // n_idx * idx_unit + tail_len
  int tiles_per_block;
  int num_splits;
  float* partial_o;       // [H, num_splits, 128]
  float* partial_ml;      // [H, num_splits, 2]
  unsigned* counters;     // [H], zero on entry and on exit
  float scale_log2;       // sm_scale * log2(e)
  // optional: attend to EVERY token of a sequence whose length lives on the device (the dense layers
  // of a graph-captured decode step): `indices` is then the page table (idx_stride 0, idx_unit =
  // page_size) and n_idx, n_tokens, tail_slot0 and tiles_per_block are derived from *seq_len_dev here;
  // num_splits (the grid) was sized for the longest sequence.
  const int32_t* seq_len_dev;
  // optional (needs seq_len_dev): a batch of sequences, grid.z = sequence.  q, o, o_f32, lse and the
  // scratch have one row per (sequence, head); the cache, its page table and the length are the sequence's.
  const SeqDesc* seqs;
};

template <typename T>
__global__ void __launch_bounds__(kDecThreads, 4) sparse_decode_kernel(DecodeParams prm) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float s_logit[kDecTile];
  __shared__ unsigned char s_skip[2][kDecTile];   // per stage: token masked out (negative index)
  __shared__ float s_p[kDecTile];
  __shared__ float s_red[4];
  __shared__ float s_sum[4];
  __shared__ float s_o[8][kHeadDim];
  __shared__ unsigned s_last;
  __shared__ __align__(8) uint64_t full_bar[2];

  const int split = blockIdx.x;
  const int head = blockIdx.z * gridDim.y + blockIdx.y;   // row of q, o, lse and the scratch: (sequence, query head)
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int H = prm.H;
  const int head_kv = prm.q_group == 1 ? blockIdx.y : blockIdx.y / prm.q_group;

  const T* kvp = static_cast<const T*>(prm.kv);
  const int32_t* idx_row = prm.indices + static_cast<int64_t>(head) * prm.idx_stride;
  const int32_t* seq_len_dev = prm.seq_len_dev;
  if (prm.seqs) {   // (the table of sequences is set up once, long before this launch)
    kvp = static_cast<const T*>(prm.seqs[blockIdx.z].kv_data);
    idx_row = prm.seqs[blockIdx.z].kv_table;
    seq_len_dev += blockIdx.z;
  }
  const int64_t v_delta = static_cast<int64_t>(prm.page_size) * H * kHeadDim;

  // ---- gather one tile into a stage --------------------------------------------------------------
  // thread -> (token tl = tid / 2, K or V row): one 256-byte bulk copy each.  Every thread arrives at
  // the stage's barrier once, with the bytes it has asked for (none for a skipped or absent token).
  // Slots are < 2^31 (checked on the host), so the index arithmetic is 32-bit; only the final element
  // offset is 64-bit.
  if (tid == 0) {
    mbar_init(&full_bar[0], kDecThreads);
    mbar_init(&full_bar[1], kDecThreads);
    mbar_fence_init();
  }
  __syncthreads();
  // The index list, the query and a device-resident length are the preceding kernels' output (a
  // RoPE-fused append rotates q in place), so nothing of them is touched before the dependency has
  // resolved.
  grid_dependency_wait();
  grid_launch_dependents();
  int n_tokens = prm.n_tokens, tiles_per_block = prm.tiles_per_block, n_listed = prm.n_idx * prm.idx_unit;
  unsigned tail_slot0 = prm.tail_slot0;
  if (seq_len_dev) {
    const int len = __ldg(seq_len_dev);
    const int pages = (len + prm.page_size - 1) / prm.page_size;
    n_listed = (pages - 1) * prm.page_size;
    n_tokens = len;
    tail_slot0 = static_cast<unsigned>(__ldg(idx_row + pages - 1)) * static_cast<unsigned>(prm.page_size);
    const int tiles = (len + kDecTile - 1) / kDecTile;
    tiles_per_block = (tiles + prm.num_splits - 1) / prm.num_splits;
  }
  const int tok_begin = split * tiles_per_block * kDecTile;
  const int tok_end = min(n_tokens, tok_begin + tiles_per_block * kDecTile);
  const int n_tiles = max(0, (tok_end - tok_begin + kDecTile - 1) / kDecTile);
  auto issue_tile = [&](int tile, int stage) {
    uint8_t* sk = smem + stage * kDecStageBytes;
    uint8_t* sv = sk + kDecTile * kDecRowBytes;
    const int tl = tid >> 1;
    const int is_v = tid & 1;
    const int j = tok_begin + tile * kDecTile + tl;
    const unsigned ps = static_cast<unsigned>(prm.page_size);
    bool ok = j < tok_end;
    unsigned slot = 0;
    if (ok) {
      if (j < n_listed) {
        if (prm.idx_unit == 1) {
          const int32_t id = __ldg(idx_row + j);
          ok = id >= 0;   // a negative entry is a hole in the list: the token is skipped
          slot = static_cast<unsigned>(id);
        } else {  // page-granular list: idx_unit == page_size
          unsigned item, off;
          if (prm.ps_shift >= 0) {
            item = static_cast<unsigned>(j) >> prm.ps_shift;
            off = static_cast<unsigned>(j) & (ps - 1);
          } else {
            item = static_cast<unsigned>(j) / ps;
            off = static_cast<unsigned>(j) - item * ps;
          }
          slot = static_cast<unsigned>(__ldg(idx_row + item)) * ps + off;
        }
      } else {
        slot = tail_slot0 + static_cast<unsigned>(j - n_listed);
      }
    }
    if (is_v == 0) s_skip[stage][tl] = ok ? 0 : 1;
    if (ok) {
      unsigned page, e;
      if (prm.ps_shift >= 0) {
        page = slot >> prm.ps_shift;
        e = slot & (ps - 1);
      } else {
        page = slot / ps;
        e = slot - page * ps;
      }
      const int64_t row = static_cast<int64_t>(page) * (2 * ps) + e;
      const T* src = kvp + (row * H + head_kv) * kHeadDim + (is_v ? v_delta : 0);
      mbar_arrive_expect_tx(&full_bar[stage], kHeadDim * 2);
      bulk_copy_g2s((is_v ? sv : sk) + tl * kDecRowBytes, src, kHeadDim * 2, &full_bar[stage]);
    } else {
      mbar_arrive(&full_bar[stage]);
    }
  };

  issue_tile(0, 0);

  // ---- query: 64 dims per thread, in the order the thread walks its chunks ---------------------
  // thread pair (tl = tid / 2, half = tid % 2); step i reads logical chunk half*8 + (i ^ half*4)
  const int qk_tl = tid >> 1;
  const int half = tid & 1;
  float qreg[8][8];
  {
    const T* qp = static_cast<const T*>(prm.q) + static_cast<int64_t>(head) * kHeadDim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int lc = half * 8 + (i ^ (half * 4));
      unpack8<T>(ld_16(qp + lc * 8), qreg[i]);
#pragma unroll
      for (int d = 0; d < 8; ++d) qreg[i][d] *= prm.scale_log2;
    }
  }


  float m_run = -INFINITY, l_run = 0.f;
  float o_acc[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) o_acc[d] = 0.f;
  const int pv_g = tid >> 4;   // token group: tokens pv_g*8 .. pv_g*8+7 of the tile
  const int pv_c = tid & 15;   // 8-dim chunk

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) issue_tile(tile + 1, stage ^ 1);
    // bounded wait for this tile's bytes (a stage is used every other tile: its phase parity follows)
    if (!mbar_wait_bounded(&full_bar[stage], (tile >> 1) & 1, 1u << 20)) atomicOr(&g_adamas_error, kErrDecodeTimeout);
    __syncthreads();   // s_skip of this stage is visible to all threads
    const uint8_t* sk = smem + stage * kDecStageBytes;
    const uint8_t* sv = sk + kDecTile * kDecRowBytes;
    const int tile_tokens = min(kDecTile, tok_end - (tok_begin + tile * kDecTile));

    // logits
    float acc = 0.f;
    const bool qk_live = qk_tl < tile_tokens && s_skip[stage][qk_tl] == 0;
    if (qk_live) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int lc = half * 8 + (i ^ (half * 4));
        float kf[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(sk + qk_tl * kDecRowBytes + lc * 16), kf);
#pragma unroll
        for (int d = 0; d < 8; ++d) acc = fmaf(qreg[i][d], kf[d], acc);
      }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    const float logit = qk_live ? acc : -INFINITY;
    if (half == 0) s_logit[qk_tl] = logit;
    float wmax = logit;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
    if (lane == 0) s_red[warp] = wmax;
    __syncthreads();

    const float m_tile = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
    const float m_new = fmaxf(m_run, m_tile);
    const float rescale = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
    float psum = 0.f;
    if (tid < kDecTile) {
      const float lg = s_logit[tid];
      const float p = (lg == -INFINITY) ? 0.f : exp2f(lg - m_new);   // masked tokens weigh nothing
      s_p[tid] = p;
      psum = p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    if (lane == 0) s_sum[warp] = psum;
    __syncthreads();
    l_run = l_run * rescale + (s_sum[0] + s_sum[1]);
    m_run = m_new;

    // P.V for this thread's token group and chunk
#pragma unroll
    for (int d = 0; d < 8; ++d) o_acc[d] *= rescale;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int tl = pv_g * 8 + i;
      const float p = s_p[tl];
      if (p != 0.f) {   // masked or absent tokens: their rows in shared memory are stale
        float vf[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(sv + tl * kDecRowBytes + pv_c * 16), vf);
#pragma unroll
        for (int d = 0; d < 8; ++d) o_acc[d] = fmaf(p, vf[d], o_acc[d]);
      }
    }
    __syncthreads();  // the stage is free for the tile after next; s_logit / s_p reusable
  }

  // ---- reduce the 8 token groups ----------------------------------------------------------------
#pragma unroll
  for (int d = 0; d < 8; ++d) s_o[pv_g][pv_c * 8 + d] = o_acc[d];
  __syncthreads();
  float od = 0.f;
#pragma unroll
  for (int g = 0; g < 8; ++g) od += s_o[g][tid];

  T* op = static_cast<T*>(prm.o) + static_cast<int64_t>(head) * kHeadDim;
  if (prm.num_splits == 1) {
    const float r = l_run > 0.f ? od / l_run : 0.f;   // nothing attended: zeros and lse = -inf
    // pairs of threads share a 32-bit store
    const float r1 = __shfl_down_sync(0xffffffffu, r, 1);
    if (prm.o_f32) prm.o_f32[static_cast<int64_t>(head) * kHeadDim + tid] = r;
    if (prm.o && (tid & 1) == 0) reinterpret_cast<uint32_t*>(op)[tid >> 1] = Elem<T>::from_f2(r, r1);
    if (tid == 0 && prm.lse) prm.lse[head] = l_run > 0.f ? m_run + log2f(l_run) : -INFINITY;
    return;
  }

  const int64_t pidx = static_cast<int64_t>(head) * prm.num_splits + split;
  prm.partial_o[pidx * kHeadDim + tid] = od;
  if (tid == 0) {
    prm.partial_ml[pidx * 2] = m_run;
    prm.partial_ml[pidx * 2 + 1] = l_run;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned ticket = atomicAdd(prm.counters + head, 1u);
    s_last = (ticket == static_cast<unsigned>(prm.num_splits - 1));
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();

  // ---- merge by the last block of the head ---------------------------------------------------
  // (m, l) of every split -> shared memory (the stage buffers are free now), then one pass per dim.
  const int64_t p0 = static_cast<int64_t>(head) * prm.num_splits;
  float* s_w = reinterpret_cast<float*>(smem);       // num_splits weights (fits: checked on the host)
  float mloc = -INFINITY;
  for (int s = tid; s < prm.num_splits; s += kDecThreads)
    mloc = fmaxf(mloc, __ldcg(prm.partial_ml + (p0 + s) * 2));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, o));
  if (lane == 0) s_red[warp] = mloc;
  __syncthreads();
  const float M = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  float lloc = 0.f;
  for (int s = tid; s < prm.num_splits; s += kDecThreads) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(prm.partial_ml + (p0 + s) * 2));
    const float w = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - M);
    s_w[s] = w;
    lloc += w * ml.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lloc += __shfl_xor_sync(0xffffffffu, lloc, o);
  if (lane == 0) s_sum[warp] = lloc;
  __syncthreads();
  const float Lsum = (s_sum[0] + s_sum[1]) + (s_sum[2] + s_sum[3]);
  float accd = 0.f;
  const float* po = prm.partial_o + p0 * kHeadDim + tid;
  int s = 0;
  for (; s + 8 <= prm.num_splits; s += 8) {
    float t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) t[u] = __ldcg(po + static_cast<int64_t>(s + u) * kHeadDim);
#pragma unroll
    for (int u = 0; u < 8; ++u) accd = fmaf(s_w[s + u], t[u], accd);
  }
  for (; s < prm.num_splits; ++s) accd = fmaf(s_w[s], __ldcg(po + static_cast<int64_t>(s) * kHeadDim), accd);
  const float r = Lsum > 0.f ? accd / Lsum : 0.f;
  const float r1 = __shfl_down_sync(0xffffffffu, r, 1);
  if (prm.o_f32) prm.o_f32[static_cast<int64_t>(head) * kHeadDim + tid] = r;
  if (prm.o && (tid & 1) == 0) reinterpret_cast<uint32_t*>(op)[tid >> 1] = Elem<T>::from_f2(r, r1);
  if (tid == 0) {
    if (prm.lse) prm.lse[head] = Lsum > 0.f ? M + log2f(Lsum) : -INFINITY;
    prm.counters[head] = 0;
  }
}

// Merge P already-normalised partial results (o_parts [P,H,128] fp32, lse_parts [P,H] base 2).
template <typename T>
__global__ void __launch_bounds__(kHeadDim)
merge_states_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts, int P,
                    int H, T* __restrict__ o, float* __restrict__ lse) {
  const int head = blockIdx.x;
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int p = 0; p < P; ++p) M = fmaxf(M, lse_parts[static_cast<int64_t>(p) * H + head]);
  float acc = 0.f, den = 0.f;
  for (int p = 0; p < P; ++p) {
    const float l = lse_parts[static_cast<int64_t>(p) * H + head];
    const float w = (l == -INFINITY) ? 0.f : exp2f(l - M);
    den += w;
    if (w != 0.f) acc += w * o_parts[(static_cast<int64_t>(p) * H + head) * kHeadDim + d];
  }
  // every part empty (lse = -inf everywhere): zeros and lse = -inf, as the decode kernel itself writes
  const float r = den > 0.f ? acc / den : 0.f;
  const float r1 = __shfl_down_sync(0xffffffffu, r, 1);
  if ((d & 1) == 0)
    reinterpret_cast<uint32_t*>(o + static_cast<int64_t>(head) * kHeadDim)[d >> 1] =
        Elem<T>::from_f2(r, r1);
  if (d == 0 && lse) lse[head] = den > 0.f ? M + log2f(den) : -INFINITY;
}

}  // namespace adamas
