// Stage 1 of the decode path: 128-point Walsh-Hadamard transform, 2-bit bucketize, pack, and the
// append of new keys/values/codes to the paged caches.
//
// Work decomposition: one half-warp (16 lanes) per 128-element row, 8 elements (16 bytes) per lane.
// Butterfly strides 1,2,4 run inside a lane's registers, strides 8..64 through shfl.xor with lane
// masks 1,2,4,8.  Arithmetic is fp32 add/sub in a fixed order plus one multiply, then a round to
// the storage type, so the result is bit-identical to the CPU restatement.  After the transform
// lane w holds dimensions 8w..8w+7, which is exactly packed code word w.
#pragma once
#include "common.cuh"

namespace adamas {

// In-place 128-point WHT over the 16 lanes of a half-warp. `l16` = lane index within the half-warp.
__device__ __forceinline__ void wht128_halfwarp(float (&x)[8], unsigned l16) {
#pragma unroll
  for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if ((i & s) == 0) {
        float a = x[i], b = x[i + s];
        x[i] = __fadd_rn(a, b);
        x[i + s] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (unsigned m = 1; m < 16; m <<= 1) {
    // lower lane holds a and receives b: a + b; upper lane holds b and receives a: a - b.  Written as
    // one fused multiply-add with a factor of +-1: the product is exact, so the single rounding is that
    // of the plain add or subtract.
    const float sgn = (l16 & m) != 0 ? -1.0f : 1.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], m);
      x[i] = __fmaf_rn(x[i], sgn, other);
    }
  }
}

template <typename T>
__device__ __forceinline__ void scale_round(float (&x)[8], float scale) {
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = Elem<T>::round(__fmul_rn(x[i], scale));
}

// 8 values -> one packed word: value i at bits [2i, 2i+1]; bucket = #thresholds strictly below.
__device__ __forceinline__ uint16_t bucketize_pack8(const float (&x)[8], Thresholds th) {
  unsigned w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    unsigned b = (x[i] > th.t0) + (x[i] > th.t1) + (x[i] > th.t2);
    w |= b << (2 * i);
  }
  return static_cast<uint16_t>(w);
}

// Llama rotary embedding (rotate-half form) of one 128-dim row spread over a half-warp: element e of
// the first half pairs with e + 64, which lives in lane l16 ^ 8.  angle = pos * inv_freq(e % 64) with
// inv_freq(j) = (1 / rope_scale) / theta^(2j/128), all in fp32 as the reference's kernel and the HF
// module compute it (kernels/include/decode/decode_page.cuh:642-690).  The result is rounded to the
// storage type, as the in-place reference operator leaves it.
// With `inv_freq` (64 floats on the device: one rotation frequency per dimension pair, position scaling
// already folded in) the angle is pos * inv_freq[j] and the rotated values are multiplied by `mscale`:
// the form YaRN-scaled models use (per-dimension interpolation ramp, attention factor on cos and sin).
struct RopeParams {
  float rcp_scale;
  float theta;
  const float* inv_freq;
  float mscale;
};

template <typename T>
__device__ __forceinline__ void rope_halfwarp(float (&x)[8], unsigned l16, float pos, RopeParams rp) {
  const bool upper = (l16 & 8) != 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float other = __shfl_xor_sync(0xffffffffu, x[i], 8);
    const int j = static_cast<int>(l16 & 7) * 8 + i;
    const float inv_freq = rp.inv_freq ? __ldg(rp.inv_freq + j)
                                       : rp.rcp_scale / powf(rp.theta, static_cast<float>(2 * j) * (1.0f / kHeadDim));
    float sn, cs;
    sincosf(pos * inv_freq, &sn, &cs);
    // lower half: x*cos - partner*sin; upper half: x*cos + partner*sin
    float r = upper ? fmaf(other, sn, x[i] * cs) : fmaf(-other, sn, x[i] * cs);
    if (rp.inv_freq) r *= rp.mscale;
    x[i] = Elem<T>::round(r);
  }
}

// (cos, sin) of dimension pair j at position pos: the one expression every kernel that rotates a decode
// token uses, so that all of them produce the same bits.
__device__ __forceinline__ float2 rope_cos_sin(int j, float pos, const RopeParams& rp) {
  const float inv_freq = rp.inv_freq ? __ldg(rp.inv_freq + j)
                                     : rp.rcp_scale / powf(rp.theta, static_cast<float>(2 * j) * (1.0f / kHeadDim));
  float sn, cs;
  sincosf(pos * inv_freq, &sn, &cs);
  return make_float2(cs, sn);
}

// The same rotation with the 64 (cos, sin) pairs of the position given (shared memory): what the decode
// append uses, where every row of the launch sits at the same position.
template <typename T>
__device__ __forceinline__ void rope_halfwarp_cs(float (&x)[8], unsigned l16, const float2* cs_table, bool scaled,
                                                 float mscale) {
  const bool upper = (l16 & 8) != 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float other = __shfl_xor_sync(0xffffffffu, x[i], 8);
    const float2 cs = cs_table[static_cast<int>(l16 & 7) * 8 + i];
    float r = upper ? fmaf(other, cs.y, x[i] * cs.x) : fmaf(-other, cs.y, x[i] * cs.x);
    if (scaled) r *= mscale;
    x[i] = Elem<T>::round(r);
  }
}

// In-place rotary embedding of q [seq, Hq, 128] and k [seq, Hk, 128]; token s has position past_len + s.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ q, T* __restrict__ k, int64_t rows_q,
                                                   int64_t rows_k, int hq, int hk, int past_len,
                                                   RopeParams rp) {
  const unsigned l16 = threadIdx.x & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const bool valid = row < rows_q + rows_k;
  const bool is_k = row >= rows_q;
  const int64_t r = valid ? (is_k ? row - rows_q : row) : 0;
  T* base = (is_k && valid) ? k : q;
  const int heads = (is_k && valid) ? hk : hq;
  const float pos = static_cast<float>(past_len + r / heads);
  float v[8];
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (valid) raw = ld_16(base + r * kHeadDim + l16 * 8);
  unpack8<T>(raw, v);
  rope_halfwarp<T>(v, l16, pos, rp);
  if (valid) st_16(base + r * kHeadDim + l16 * 8, pack8<T>(v));
}

// y = round(scale * WHT(x)), rows x 128.
template <typename T>
__global__ void __launch_bounds__(256) hadamard_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                       int64_t rows, float scale) {
  const unsigned l16 = threadIdx.x & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const bool valid = row < rows;
  float v[8];
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (valid) raw = ld_16(x + row * kHeadDim + l16 * 8);
  unpack8<T>(raw, v);
  wht128_halfwarp(v, l16);
  scale_round<T>(v, scale);
  if (valid) st_16(y + row * kHeadDim + l16 * 8, pack8<T>(v));
}

// codes[row, w] = pack(bucketize(h[row, 8w..8w+7]))
template <typename T>
__global__ void __launch_bounds__(256) bucketize_pack_kernel(const T* __restrict__ h,
                                                             uint16_t* __restrict__ codes,
                                                             int64_t rows, Thresholds th) {
  const unsigned l16 = threadIdx.x & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  if (row >= rows) return;
  float v[8];
  unpack8<T>(ld_16(h + row * kHeadDim + l16 * 8), v);
  codes[row * kCodeWords + l16] = bucketize_pack8(v, th);
}

struct PagedTarget {
  void* kv_data;
  const int32_t* kv_table;
  uint16_t* code_data;
  const int32_t* code_table;
  int page_size;
  int num_heads;
};

// Decode append: one half-warp per head.  FUSED: qh = q, kh = k and the transform runs here;
// otherwise qh/kh point at rows 0/1 of the pre-transformed h.  Grouped-query attention (FUSED only):
// q has q_heads = group * H rows and the caches H; half-warp i takes query row i and K/V row i, each
// where it exists.  ROPE (needs FUSED): q and k arrive
// un-rotated; they are rotated for position `pos`, written back in place (the attention reads the
// rotated q, the caller's k stays consistent with the cache) and then coded.
template <typename T, bool FUSED, bool ROPE = false>
__global__ void __launch_bounds__(256)
append_decode_kernel(const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ qh,
                     const T* __restrict__ kh, uint16_t* __restrict__ q_code_out, PagedTarget tgt,
                     int kv_last_page, int kv_entry, int code_last_page, int code_entry, float scale,
                     Thresholds th, float pos, RopeParams rp, const int32_t* seq_len_dev, int q_heads,
                     const SeqDesc* seqs) {
  // The kernel after this one (the estimate) may become resident right away: its producer warps only
  // read the code cache as it was before this step, and its consumers wait for this grid to complete,
  // which in turn waits for the grid before it.  (Two appends to one cache back to back, followed by an
  // estimate, are outside this reasoning: the estimate's early reads could then see the first append's
  // slot unwritten.  A decode step appends once.)
  grid_launch_dependents();
  grid_dependency_wait();
  if (seqs) {
    // a batch of sequences (grid.y = sequence): rows of q, k, v and the query codes are (sequence, head)
    const int b = blockIdx.y;
    tgt.kv_data = seqs[b].kv_data;
    tgt.kv_table = seqs[b].kv_table;
    tgt.code_data = static_cast<uint16_t*>(seqs[b].code_data);
    tgt.code_table = seqs[b].code_table;
    const int64_t kv_rows = static_cast<int64_t>(b) * tgt.num_heads * kHeadDim;
    const int64_t q_rows = static_cast<int64_t>(b) * q_heads * kHeadDim;
    k += kv_rows;
    v += kv_rows;
    kh += FUSED ? kv_rows : 0;
    qh += q_rows;
    q_code_out += static_cast<int64_t>(b) * q_heads * kCodeWords;
    seq_len_dev += b;
  }
  if (seq_len_dev) {
    // the token being appended sits at position *seq_len_dev - 1 of both caches
    const int t = __ldg(seq_len_dev) - 1;
    kv_last_page = code_last_page = t / tgt.page_size;
    kv_entry = code_entry = t - kv_last_page * tgt.page_size;
    pos = static_cast<float>(t);
  }
  // ROPE: the 64 (cos, sin) pairs of the position, once per block (every row of the launch has the same
  // position; a sine/cosine of an angle beyond 1e5 rad takes the slow argument reduction, and eight of them
  // one after the other in every lane cost 6 us per layer at 128K tokens)
  __shared__ float2 s_cs[kHeadDim / 2];
  if (ROPE) {
    if (threadIdx.x < kHeadDim / 2) s_cs[threadIdx.x] = rope_cos_sin(threadIdx.x, pos, rp);
    __syncthreads();
  }
  // physical pages of the slot being written: last entries of the two page tables
  const int kv_page = __ldg(tgt.kv_table + kv_last_page);
  const int code_page = __ldg(tgt.code_table + code_last_page);
  const unsigned l16 = threadIdx.x & 15;
  const int head = (blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const int H = tgt.num_heads;
  const bool valid = head < H;            // a K/V row of the caches
  const bool valid_q = head < q_heads;    // a query row
  const int hh = valid ? head : 0;
  const int hq = valid_q ? head : 0;
  const int64_t in_off = static_cast<int64_t>(hh) * kHeadDim + l16 * 8;
  const int64_t q_off = static_cast<int64_t>(hq) * kHeadDim + l16 * 8;

  // copy K and V rows into the page slot
  T* kv = static_cast<T*>(tgt.kv_data);
  const int64_t k_off =
      ((static_cast<int64_t>(kv_page) * 2 * tgt.page_size + kv_entry) * H + hh) * kHeadDim + l16 * 8;
  const int64_t v_delta = static_cast<int64_t>(tgt.page_size) * H * kHeadDim;
  uint4 kraw = ld_16(k + in_off);
  uint4 vraw = ld_16(v + in_off);
  float a[8], b[8];
  unpack8<T>(ld_16(qh + q_off), a);
  if (ROPE) {
    unpack8<T>(kraw, b);
    rope_halfwarp_cs<T>(a, l16, s_cs, rp.inv_freq != nullptr, rp.mscale);
    rope_halfwarp_cs<T>(b, l16, s_cs, rp.inv_freq != nullptr, rp.mscale);
    kraw = pack8<T>(b);
    if (valid_q) st_16(const_cast<T*>(qh) + q_off, pack8<T>(a));
    if (valid) st_16(const_cast<T*>(k) + in_off, kraw);
  }
  if (valid) {
    st_16(kv + k_off, kraw);
    st_16(kv + k_off + v_delta, vraw);
  }

  if (FUSED) {
    unpack8<T>(kraw, b);
    wht128_halfwarp(a, l16);
    wht128_halfwarp(b, l16);
    scale_round<T>(a, scale);
    scale_round<T>(b, scale);
  } else {
    unpack8<T>(ld_16(kh + in_off), b);
  }
  if (valid_q) q_code_out[hq * kCodeWords + l16] = bucketize_pack8(a, th);
  if (valid) {
    const int64_t c_off =
        ((static_cast<int64_t>(code_page) * tgt.page_size + code_entry) * H + hh) * kCodeWords + l16;
    tgt.code_data[c_off] = bucketize_pack8(b, th);
  }
}

// Prefill append: one half-warp per (token, head) row; token n sits at position start_pos + n.
template <typename T, bool FUSED>
__global__ void __launch_bounds__(256)
append_prefill_kernel(const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ h,
                      int64_t rows, int64_t start_pos, PagedTarget tgt, float scale, Thresholds th) {
  const unsigned l16 = threadIdx.x & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const bool valid = row < rows;
  const int64_t r = valid ? row : 0;
  const int H = tgt.num_heads;
  const int64_t n = r / H;
  const int head = static_cast<int>(r - n * H);
  const int64_t pos = start_pos + n;
  const int64_t lp = pos / tgt.page_size;
  const int e = static_cast<int>(pos - lp * tgt.page_size);
  const int64_t in_off = r * kHeadDim + l16 * 8;

  uint4 kraw = ld_stream_16(k + in_off);
  uint4 vraw = ld_stream_16(v + in_off);
  const int64_t kv_page = tgt.kv_table[lp];
  T* kv = static_cast<T*>(tgt.kv_data);
  const int64_t k_off = ((kv_page * 2 * tgt.page_size + e) * H + head) * kHeadDim + l16 * 8;
  if (valid) {
    st_16(kv + k_off, kraw);
    st_16(kv + k_off + static_cast<int64_t>(tgt.page_size) * H * kHeadDim, vraw);
  }
  float x[8];
  if (FUSED) {
    unpack8<T>(kraw, x);
    wht128_halfwarp(x, l16);
    scale_round<T>(x, scale);
  } else {
    unpack8<T>(ld_stream_16(h + in_off), x);
  }
  if (valid) {
    const int64_t code_page = tgt.code_table[lp];
    tgt.code_data[((code_page * tgt.page_size + e) * H + head) * kCodeWords + l16] =
        bucketize_pack8(x, th);
  }
}

}  // namespace adamas
