// C ABI of the B200 Adamas decode path (see include/adamas_b200.h for the contract of every
// entry point and the reference interface each one replaces).  Host side only: argument checks,
// launch geometry, error reporting.  Kernels live in the .cuh files next to this one.
#include "../../include/adamas_b200.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstddef>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "common.cuh"
#include "estimate.cuh"
#include "hadamard_append.cuh"
#include "select_attend.cuh"
#include "sparse_decode.cuh"
#include "topk.cuh"

using namespace adamas;

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define ADAMAS_REQUIRE(cond, ...) \
  do {                            \
    if (!(cond)) return fail(ADAMAS_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define ADAMAS_CUDA(expr)                                                                   \
  do {                                                                                      \
    cudaError_t e_ = (expr);                                                                \
    if (e_ != cudaSuccess)                                                                  \
      return fail(ADAMAS_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_));         \
  } while (0)

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ADAMAS_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  return ADAMAS_OK;
}

inline cudaStream_t to_stream(adamas_stream_t s) { return static_cast<cudaStream_t>(s); }

Thresholds make_thresholds(const float* t) {
  Thresholds th;
  if (t) {
    th.t0 = t[0]; th.t1 = t[1]; th.t2 = t[2];
  } else {
    th.t0 = -10.f; th.t1 = 0.f; th.t2 = 10.f;
  }
  return th;
}

int check_common(int num_heads, int head_dim, int page_size, int dtype) {
  ADAMAS_REQUIRE(head_dim == kHeadDim, "head_dim must be 128 (got %d)", head_dim);
  ADAMAS_REQUIRE(num_heads >= 1 && num_heads <= 1024, "num_heads out of range (%d)", num_heads);
  ADAMAS_REQUIRE(page_size >= 1, "page_size must be >= 1 (got %d)", page_size);
  ADAMAS_REQUIRE(dtype == ADAMAS_F16 || dtype == ADAMAS_BF16, "unsupported dtype %d", dtype);
  return ADAMAS_OK;
}

// Grouped-query attention: num_q_heads query heads over num_heads cache heads, query head r reads cache
// head r / (num_q_heads / num_heads).  num_q_heads == num_heads is multi-head attention, all the
// reference knows (kernels/include/decode/decode_handler.cuh:83 asserts it).
int check_q_heads(int num_heads, int num_q_heads) {
  ADAMAS_REQUIRE(num_q_heads >= num_heads && num_q_heads <= 1024 && num_q_heads % num_heads == 0,
                 "num_q_heads (%d) must be a multiple of num_heads (%d)", num_q_heads, num_heads);
  return ADAMAS_OK;
}

constexpr int kEstAppendStatic = 1792;   // static shared memory of estimate_append_kernel (with the cos / sin table), rounded up
constexpr int kEstPagesStatic = 8448;    // static shared memory of estimate_pages_kernel, rounded up
constexpr int kSaMaxDynSmem = 160 * 1024;   // dynamic shared memory select_attend may ask for (a long winner list)

// Per-device facts and one-time kernel attributes.
struct DeviceInfo {
  bool ready = false;
  int num_sms = 0;
  int max_smem_optin = 0;
  int smem_per_sm = 0;
  int topk_dyn_smem = 0;
};

std::mutex g_init_mutex;   // first-use set-up may be reached from several host threads at once

int get_device_info(const DeviceInfo** out) {
  static DeviceInfo infos[64];
  int dev = 0;
  ADAMAS_CUDA(cudaGetDevice(&dev));
  ADAMAS_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_init_mutex);
  DeviceInfo& d = infos[dev];
  if (!d.ready) {
    ADAMAS_CUDA(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev));
    ADAMAS_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    ADAMAS_CUDA(cudaDeviceGetAttribute(&d.smem_per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
    d.topk_dyn_smem = d.max_smem_optin - static_cast<int>(sizeof(TopkShared)) - 1024;
    ADAMAS_CUDA(cudaFuncSetAttribute(topk_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, d.topk_dyn_smem));
    ADAMAS_CUDA(cudaFuncSetAttribute(topk_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, d.topk_dyn_smem));
    const int est_max = d.max_smem_optin - 1024;
#define EST_ATTR(M, OT, HPW)                                                                       \
  ADAMAS_CUDA(cudaFuncSetAttribute(estimate_kernel<M, OT, HPW>,                                    \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, est_max))
#define EST_ATTR_ALL(M, OT) \
  EST_ATTR(M, OT, 0);       \
  EST_ATTR(M, OT, 1);       \
  EST_ATTR(M, OT, 2);       \
  EST_ATTR(M, OT, 4)
    EST_ATTR_ALL(0, __half);
    EST_ATTR_ALL(0, uint16_t);
    EST_ATTR_ALL(1, __half);
    EST_ATTR_ALL(1, uint16_t);
#undef EST_ATTR_ALL
#undef EST_ATTR
#define ESTA_ATTR(T, HPW, R)                                                                           \
  ADAMAS_CUDA(cudaFuncSetAttribute((estimate_append_kernel<T, HPW, R>),                                \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, est_max - kEstAppendStatic)); \
  ADAMAS_CUDA(cudaFuncSetAttribute((estimate_append_kernel<T, HPW, R>),                                \
                                   cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared))
#define ESTA_ATTR_ALL(T)    \
  ESTA_ATTR(T, 1, false);   \
  ESTA_ATTR(T, 2, false);   \
  ESTA_ATTR(T, 4, false);   \
  ESTA_ATTR(T, 1, true);    \
  ESTA_ATTR(T, 2, true);    \
  ESTA_ATTR(T, 4, true)
    ESTA_ATTR_ALL(__half);
    ESTA_ATTR_ALL(__nv_bfloat16);
#undef ESTA_ATTR_ALL
#undef ESTA_ATTR
    ADAMAS_CUDA(cudaFuncSetAttribute(sparse_decode_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kDecStageBytes));
    ADAMAS_CUDA(cudaFuncSetAttribute(sparse_decode_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kDecStageBytes));
    // One shared-memory carve-out for every kernel of the decode step: a kernel that asks for a
    // different L1 / shared split than its predecessor cannot start until the SMs have drained.
#define SET_CARVEOUT(kern) \
  ADAMAS_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared))
    SET_CARVEOUT((append_decode_kernel<__half, true, false>));
    SET_CARVEOUT((append_decode_kernel<__half, false, false>));
    SET_CARVEOUT((append_decode_kernel<__nv_bfloat16, true, false>));
    SET_CARVEOUT((append_decode_kernel<__nv_bfloat16, false, false>));
    SET_CARVEOUT((append_decode_kernel<__half, true, true>));
    SET_CARVEOUT((append_decode_kernel<__nv_bfloat16, true, true>));
    SET_CARVEOUT((estimate_kernel<0, __half, 0>));
    SET_CARVEOUT((estimate_kernel<0, __half, 1>));
    SET_CARVEOUT((estimate_kernel<0, __half, 2>));
    SET_CARVEOUT((estimate_kernel<0, __half, 4>));
    SET_CARVEOUT((estimate_kernel<0, uint16_t, 0>));
    SET_CARVEOUT((estimate_kernel<0, uint16_t, 1>));
    SET_CARVEOUT((estimate_kernel<0, uint16_t, 2>));
    SET_CARVEOUT((estimate_kernel<0, uint16_t, 4>));
    SET_CARVEOUT((topk_cluster_kernel<0, 1, 256>));
    SET_CARVEOUT((topk_cluster_kernel<0, 2, 256>));
    SET_CARVEOUT((topk_cluster_kernel<0, 4, 256>));
    SET_CARVEOUT((topk_cluster_kernel<1, 1, 256>));
    SET_CARVEOUT((topk_cluster_kernel<1, 2, 256>));
    SET_CARVEOUT((topk_cluster_kernel<1, 4, 256>));
    SET_CARVEOUT((sparse_decode_kernel<__half>));
    SET_CARVEOUT((sparse_decode_kernel<__nv_bfloat16>));
#undef SET_CARVEOUT
    // select+attend: large dynamic shared memory
#define SA_ATTR(T, I)                                                                                          \
  ADAMAS_CUDA(cudaFuncSetAttribute(select_attend_kernel<T, I>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                   kSaMaxDynSmem));                                                            \
  ADAMAS_CUDA(cudaFuncSetAttribute(select_attend_kernel<T, I>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                                   cudaSharedmemCarveoutMaxShared))
#define SA_ATTR_ALL(T) \
  SA_ATTR(T, 1);       \
  SA_ATTR(T, 2);       \
  SA_ATTR(T, 4);       \
  SA_ATTR(T, 8)
    SA_ATTR_ALL(__half);
    SA_ATTR_ALL(__nv_bfloat16);
#undef SA_ATTR_ALL
#undef SA_ATTR
#define ESTP_ATTR(M, OT)                                                                                      \
  ADAMAS_CUDA(cudaFuncSetAttribute(estimate_pages_kernel<M, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                   d.max_smem_optin - 1024 - kEstPagesStatic));                               \
  ADAMAS_CUDA(cudaFuncSetAttribute(estimate_pages_kernel<M, OT>, cudaFuncAttributePreferredSharedMemoryCarveout, \
                                   cudaSharedmemCarveoutMaxShared))
    ESTP_ATTR(0, __half);
    ESTP_ATTR(0, uint16_t);
    ESTP_ATTR(1, __half);
    ESTP_ATTR(1, uint16_t);
#undef ESTP_ATTR
    d.ready = true;
  }
  *out = &d;
  return ADAMAS_OK;
}

// Process-wide settings.  Each is one atomic integer: a launch reads it once, so a change made by
// another thread applies to whole launches, never to half of one.  -1 = not yet read from the
// environment.
int setting(std::atomic<int>& v, const char* env, int dflt, int lo, int hi) {
  int cur = v.load(std::memory_order_relaxed);
  if (cur < 0) {
    const char* e = std::getenv(env);
    cur = e ? std::atoi(e) : dflt;
    if (cur < lo || cur > hi) cur = dflt;
    v.store(cur, std::memory_order_relaxed);
  }
  return cur;
}
// Programmatic dependent launch of the hot kernels (on unless ADAMAS_PDL=0 or adamas_set_pdl(0)).
std::atomic<int> g_pdl{-1};
bool pdl_enabled() { return setting(g_pdl, "ADAMAS_PDL", 1, 0, 1) != 0; }
// Whether adamas_decode_step folds the append into the estimate launch (on unless
// ADAMAS_FUSED_APPEND=0 or adamas_set_fused_append(0)).
std::atomic<int> g_fused_append{-1};
bool fused_append_enabled() { return setting(g_fused_append, "ADAMAS_FUSED_APPEND", 1, 0, 1) != 0; }
// Upper bound on the estimate kernel's resident blocks per SM (adamas_set_estimate_blocks_per_sm /
// ADAMAS_EST_BLOCKS_PER_SM): 2 by default, 1 leaves half of every SM to kernels of other streams.
std::atomic<int> g_est_blocks_per_sm{-1};
int est_blocks_per_sm() { return setting(g_est_blocks_per_sm, "ADAMAS_EST_BLOCKS_PER_SM", 2, 1, 2); }
// Upper bound on the cluster size of select_attend (adamas_set_max_cluster / ADAMAS_MAX_CLUSTER).
std::atomic<int> g_max_cluster{-1};
int max_cluster() {
  const int v = setting(g_max_cluster, "ADAMAS_MAX_CLUSTER", kSaMaxCluster, 1, kSaMaxCluster);
  return (v & (v - 1)) == 0 ? v : kSaMaxCluster;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                          int cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[3];
  unsigned n = 0;
  if (cluster > 1) {
    // By default the hardware spreads the blocks of a cluster over as many different SMs of a GPC.  With
    // two resident blocks per SM and nearly as many clusters as fit, blocks placed while the preceding
    // kernel drains then leave a GPC with enough free slots on too few SMs, and the last cluster
    // waits for another to finish (measured: a third of the select_attend launches took 9 us
    // longer).  Load balancing lets blocks of one cluster share an SM.
    attr[n].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
    attr[n].val.clusterSchedulingPolicyPreference = cudaClusterSchedulingPolicyLoadBalancing;
    ++n;
  }
  if (cluster >= 0 && pdl_enabled()) {   // cluster < 0: an ordinary, fully serialised launch
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

#define ADAMAS_LAUNCH(what, ...)                                                              \
  do {                                                                                        \
    cudaError_t le_ = launch_kernel(__VA_ARGS__);                                             \
    if (le_ != cudaSuccess)                                                                   \
      return fail(ADAMAS_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(le_));    \
  } while (0)

int log2_exact(int v) {
  if (v <= 0 || (v & (v - 1)) != 0) return -1;
  int s = 0;
  while ((1 << s) < v) ++s;
  return s;
}

inline unsigned rows_to_blocks(int64_t rows) { return static_cast<unsigned>((rows * 16 + 255) / 256); }

}  // namespace

extern "C" {

int adamas_abi_version(void) { return ADAMAS_ABI_VERSION; }

int adamas_set_pdl(int enable) {
  g_pdl.store(enable ? 1 : 0);
  return ADAMAS_OK;
}

int adamas_set_fused_append(int enable) {
  g_fused_append.store(enable ? 1 : 0);
  return ADAMAS_OK;
}

int adamas_set_estimate_blocks_per_sm(int blocks) {
  ADAMAS_REQUIRE(blocks == 1 || blocks == 2, "blocks per SM must be 1 or 2 (got %d)", blocks);
  g_est_blocks_per_sm.store(blocks);
  return ADAMAS_OK;
}

int adamas_set_max_cluster(int blocks) {
  ADAMAS_REQUIRE(blocks >= 1 && blocks <= kSaMaxCluster && (blocks & (blocks - 1)) == 0,
                 "cluster size must be a power of two between 1 and %d (got %d)", kSaMaxCluster, blocks);
  g_max_cluster.store(blocks);
  return ADAMAS_OK;
}

int adamas_device_error(unsigned* flags, int clear) {
  ADAMAS_REQUIRE(flags, "null pointer");
  ADAMAS_CUDA(cudaMemcpyFromSymbol(flags, g_adamas_error, sizeof(unsigned)));
  if (clear && *flags) {
    const unsigned zero = 0;
    ADAMAS_CUDA(cudaMemcpyToSymbol(g_adamas_error, &zero, sizeof(unsigned)));
  }
  return ADAMAS_OK;
}
const char* adamas_last_error(void) { return g_err; }

// ---------------------------------------------------------------------------------------------
int adamas_hadamard_transform(const void* x, void* y, int64_t rows, int head_dim, float scale,
                              int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(head_dim == kHeadDim, "head_dim must be 128 (got %d)", head_dim);
  ADAMAS_REQUIRE(dtype == ADAMAS_F16 || dtype == ADAMAS_BF16, "unsupported dtype %d", dtype);
  ADAMAS_REQUIRE(rows >= 0, "rows must be >= 0");
  if (rows == 0) return ADAMAS_OK;
  ADAMAS_REQUIRE(x && y, "null pointer");
  ADAMAS_REQUIRE(rows < (int64_t(1) << 31) * 16, "too many rows");
  const unsigned blocks = rows_to_blocks(rows);
  if (dtype == ADAMAS_F16)
    hadamard_kernel<__half><<<blocks, 256, 0, to_stream(stream)>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), rows, scale);
  else
    hadamard_kernel<__nv_bfloat16><<<blocks, 256, 0, to_stream(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, scale);
  return check_launch("hadamard_kernel");
}

int adamas_bucketize_pack(const void* h, void* codes, int64_t rows, int head_dim,
                          const float* thresholds3_host, int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(head_dim == kHeadDim, "head_dim must be 128 (got %d)", head_dim);
  ADAMAS_REQUIRE(dtype == ADAMAS_F16 || dtype == ADAMAS_BF16, "unsupported dtype %d", dtype);
  ADAMAS_REQUIRE(rows >= 0, "rows must be >= 0");
  if (rows == 0) return ADAMAS_OK;
  ADAMAS_REQUIRE(h && codes, "null pointer");
  const Thresholds th = make_thresholds(thresholds3_host);
  const unsigned blocks = rows_to_blocks(rows);
  if (dtype == ADAMAS_F16)
    bucketize_pack_kernel<__half><<<blocks, 256, 0, to_stream(stream)>>>(
        static_cast<const __half*>(h), static_cast<uint16_t*>(codes), rows, th);
  else
    bucketize_pack_kernel<__nv_bfloat16><<<blocks, 256, 0, to_stream(stream)>>>(
        static_cast<const __nv_bfloat16*>(h), static_cast<uint16_t*>(codes), rows, th);
  return check_launch("bucketize_pack_kernel");
}

// Rotary embedding of the append launch: off, the Llama form with linear position scaling, or a
// caller-supplied table of 64 rotation frequencies plus a factor on the rotated values (YaRN).
struct RopeSpec {
  bool on = false;
  float scale = 1.f, theta = 1e4f;
  const float* inv_freq = nullptr;   // device, 64 floats
  float mscale = 1.f;
};

// seq_len_dev (optional): the sequence length, new token included, lives on the device; the page
// counts and last-page lengths are then not used (pass the capacity's) and the slot and the position
// follow from the device value.
static RopeSpec linear_rope(float rope_scale, float rope_theta) {
  RopeSpec r;
  r.on = true;
  r.scale = rope_scale;
  r.theta = rope_theta;
  return r;
}

static int append_decode_impl(const void* k, const void* v, const void* qh, const void* kh, bool fused,
                              void* q_code_out, void* kv_data, const int32_t* kv_page_table,
                              int kv_num_pages, int kv_last_page_len, void* code_data,
                              const int32_t* code_page_table, int code_num_pages,
                              int code_last_page_len, int num_heads, int head_dim, int page_size,
                              float scale, const float* thresholds3_host, int dtype,
                              adamas_stream_t stream, const RopeSpec& rope = RopeSpec(),
                              const int32_t* seq_len_dev = nullptr, int q_heads = 0,
                              const SeqDesc* seqs = nullptr, int batch = 1) {
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  if (q_heads == 0) q_heads = num_heads;
  if (int rc = check_q_heads(num_heads, q_heads)) return rc;
  ADAMAS_REQUIRE(q_heads == num_heads || fused, "grouped-query attention needs the fused append (q, k, v)");
  ADAMAS_REQUIRE(k && v && qh && kh && q_code_out, "null pointer");
  ADAMAS_REQUIRE(seqs || (kv_data && code_data && kv_page_table && code_page_table), "null pointer");
  ADAMAS_REQUIRE(!seqs || (fused && seq_len_dev && batch >= 1), "a batched append needs the fused form and device lengths");
  ADAMAS_REQUIRE(!rope.on || rope.inv_freq || (rope.scale > 0.f && rope.theta > 0.f),
                 "rope_scale and rope_theta must be positive");
  ADAMAS_REQUIRE(!rope.on || fused, "the rotary embedding needs the fused append");
  if (!seq_len_dev) {
    ADAMAS_REQUIRE(kv_num_pages >= 1 && code_num_pages >= 1, "page tables must not be empty");
    ADAMAS_REQUIRE(kv_last_page_len >= 1 && kv_last_page_len <= page_size, "kv_last_page_len out of range");
    ADAMAS_REQUIRE(code_last_page_len >= 1 && code_last_page_len <= page_size,
                   "code_last_page_len out of range");
  }
  PagedTarget tgt{kv_data, kv_page_table, static_cast<uint16_t*>(code_data), code_page_table, page_size,
                  num_heads};
  const Thresholds th = make_thresholds(thresholds3_host);
  const unsigned blocks = rows_to_blocks(q_heads);
  cudaStream_t st = to_stream(stream);
  {
    const DeviceInfo* di = nullptr;
    if (int rc = get_device_info(&di)) return rc;
  }
  // position of the token being appended
  const float pos = static_cast<float>(static_cast<int64_t>(kv_num_pages - 1) * page_size + kv_last_page_len - 1);
  const RopeParams rp{rope.scale > 0.f ? 1.0f / rope.scale : 1.f, rope.theta, rope.inv_freq, rope.mscale};
#define LAUNCH_AD(T, F, R)                                                                            \
  ADAMAS_LAUNCH("append_decode_kernel", (append_decode_kernel<T, F, R>), dim3(blocks, seqs ? batch : 1), dim3(256), 0,  \
                st, 1, static_cast<const T*>(k), static_cast<const T*>(v), static_cast<const T*>(qh), \
                static_cast<const T*>(kh), static_cast<uint16_t*>(q_code_out), tgt, kv_num_pages - 1, \
                kv_last_page_len - 1, code_num_pages - 1, code_last_page_len - 1, scale, th, pos, rp, \
                seq_len_dev, q_heads, seqs)
  if (dtype == ADAMAS_F16) {
    if (rope.on) LAUNCH_AD(__half, true, true);
    else if (fused) LAUNCH_AD(__half, true, false);
    else LAUNCH_AD(__half, false, false);
  } else {
    if (rope.on) LAUNCH_AD(__nv_bfloat16, true, true);
    else if (fused) LAUNCH_AD(__nv_bfloat16, true, false);
    else LAUNCH_AD(__nv_bfloat16, false, false);
  }
#undef LAUNCH_AD
  return check_launch("append_decode_kernel");
}

int adamas_append_decode(const void* k, const void* v, const void* h, void* q_code_out, void* kv_data,
                         const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                         void* code_data, const int32_t* code_page_table, int code_num_pages,
                         int code_last_page_len, int num_heads, int head_dim, int page_size,
                         const float* thresholds3_host, int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(h, "null pointer");
  ADAMAS_REQUIRE(num_heads >= 1, "num_heads out of range");
  const size_t row_bytes = static_cast<size_t>(num_heads) * kHeadDim * 2;
  return append_decode_impl(k, v, h, static_cast<const uint8_t*>(h) + row_bytes, false, q_code_out,
                            kv_data, kv_page_table, kv_num_pages, kv_last_page_len, code_data,
                            code_page_table, code_num_pages, code_last_page_len, num_heads, head_dim,
                            page_size, 1.f, thresholds3_host, dtype, stream);
}

int adamas_append_decode_fused(const void* q, const void* k, const void* v, void* q_code_out,
                               void* kv_data, const int32_t* kv_page_table, int kv_num_pages,
                               int kv_last_page_len, void* code_data,
                               const int32_t* code_page_table, int code_num_pages,
                               int code_last_page_len, int num_heads, int num_q_heads, int head_dim,
                               int page_size, float scale, const float* thresholds3_host, int dtype,
                               adamas_stream_t stream) {
  return append_decode_impl(k, v, q, k, true, q_code_out, kv_data, kv_page_table, kv_num_pages,
                            kv_last_page_len, code_data, code_page_table, code_num_pages,
                            code_last_page_len, num_heads, head_dim, page_size, scale,
                            thresholds3_host, dtype, stream, RopeSpec(), nullptr, num_q_heads);
}

int adamas_append_decode_rope_fused(void* q, void* k, const void* v, void* q_code_out, void* kv_data,
                                    const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                                    void* code_data, const int32_t* code_page_table, int code_num_pages,
                                    int code_last_page_len, int num_heads, int num_q_heads, int head_dim,
                                    int page_size, float scale, const float* thresholds3_host, float rope_scale,
                                    float rope_theta, const float* rope_inv_freq, float rope_mscale, int dtype,
                                    adamas_stream_t stream) {
  RopeSpec rope = linear_rope(rope_scale, rope_theta);
  if (rope_inv_freq) {
    rope.inv_freq = rope_inv_freq;
    rope.mscale = rope_mscale;
  }
  return append_decode_impl(k, v, q, k, true, q_code_out, kv_data, kv_page_table, kv_num_pages,
                            kv_last_page_len, code_data, code_page_table, code_num_pages,
                            code_last_page_len, num_heads, head_dim, page_size, scale,
                            thresholds3_host, dtype, stream, rope, nullptr, num_q_heads);
}

int adamas_apply_rope_in_place(void* q, void* k, int64_t seq_len, int num_q_heads, int num_kv_heads,
                               int head_dim, int64_t past_kv_len, float rope_scale, float rope_theta,
                               int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(head_dim == kHeadDim, "head_dim must be 128 (got %d)", head_dim);
  ADAMAS_REQUIRE(dtype == ADAMAS_F16 || dtype == ADAMAS_BF16, "unsupported dtype %d", dtype);
  ADAMAS_REQUIRE(seq_len >= 0 && num_q_heads >= 1 && num_kv_heads >= 1, "bad shape");
  ADAMAS_REQUIRE(rope_scale > 0.f && rope_theta > 0.f, "rope_scale and rope_theta must be positive");
  ADAMAS_REQUIRE(past_kv_len >= 0 && past_kv_len + seq_len < (int64_t(1) << 24),
                 "positions must stay below 2^24 (exact in fp32)");
  if (seq_len == 0) return ADAMAS_OK;
  ADAMAS_REQUIRE(q && k, "null pointer");
  const int64_t rows_q = seq_len * num_q_heads, rows_k = seq_len * num_kv_heads;
  const unsigned blocks = rows_to_blocks(rows_q + rows_k);
  const RopeParams rp{1.0f / rope_scale, rope_theta, nullptr, 1.f};
  if (dtype == ADAMAS_F16)
    rope_kernel<__half><<<blocks, 256, 0, to_stream(stream)>>>(static_cast<__half*>(q), static_cast<__half*>(k),
                                                              rows_q, rows_k, num_q_heads, num_kv_heads,
                                                              static_cast<int>(past_kv_len), rp);
  else
    rope_kernel<__nv_bfloat16><<<blocks, 256, 0, to_stream(stream)>>>(
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), rows_q, rows_k, num_q_heads,
        num_kv_heads, static_cast<int>(past_kv_len), rp);
  return check_launch("rope_kernel");
}

int adamas_append_prefill(const void* k, const void* v, const void* h, int64_t n_tokens, void* kv_data,
                          const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                          void* code_data, const int32_t* code_page_table, int code_num_pages,
                          int code_last_page_len, int num_heads, int head_dim, int page_size,
                          float scale, const float* thresholds3_host, int dtype,
                          adamas_stream_t stream) {
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  ADAMAS_REQUIRE(n_tokens >= 0, "n_tokens must be >= 0");
  if (n_tokens == 0) return ADAMAS_OK;
  ADAMAS_REQUIRE(k && v && kv_data && code_data && kv_page_table && code_page_table, "null pointer");
  ADAMAS_REQUIRE(kv_num_pages >= 1 && code_num_pages >= 1, "page tables must not be empty");
  ADAMAS_REQUIRE(kv_last_page_len >= 1 && kv_last_page_len <= page_size, "kv_last_page_len out of range");
  ADAMAS_REQUIRE(code_last_page_len >= 1 && code_last_page_len <= page_size,
                 "code_last_page_len out of range");
  const int64_t seq_len = static_cast<int64_t>(kv_num_pages - 1) * page_size + kv_last_page_len;
  const int64_t code_len = static_cast<int64_t>(code_num_pages - 1) * page_size + code_last_page_len;
  ADAMAS_REQUIRE(seq_len == code_len, "KV cache holds %lld tokens but the code cache %lld",
                 static_cast<long long>(seq_len), static_cast<long long>(code_len));
  ADAMAS_REQUIRE(n_tokens <= seq_len, "n_tokens (%lld) exceeds the sequence length (%lld)",
                 static_cast<long long>(n_tokens), static_cast<long long>(seq_len));
  const int64_t rows = n_tokens * num_heads;
  ADAMAS_REQUIRE(rows < (int64_t(1) << 31) * 16, "too many rows");
  PagedTarget tgt{kv_data, kv_page_table, static_cast<uint16_t*>(code_data), code_page_table, page_size,
                  num_heads};
  const Thresholds th = make_thresholds(thresholds3_host);
  const unsigned blocks = rows_to_blocks(rows);
  const int64_t start = seq_len - n_tokens;
  cudaStream_t st = to_stream(stream);
#define LAUNCH_AP(T, F)                                                                            \
  append_prefill_kernel<T, F><<<blocks, 256, 0, st>>>(static_cast<const T*>(k),                    \
                                                      static_cast<const T*>(v),                    \
                                                      static_cast<const T*>(h), rows, start, tgt,  \
                                                      scale, th)
  if (dtype == ADAMAS_F16) {
    if (h) LAUNCH_AP(__half, false); else LAUNCH_AP(__half, true);
  } else {
    if (h) LAUNCH_AP(__nv_bfloat16, false); else LAUNCH_AP(__nv_bfloat16, true);
  }
#undef LAUNCH_AP
  return check_launch("append_prefill_kernel");
}

// ---------------------------------------------------------------------------------------------
// n: distances per head (host mode), or their upper bound when seq_len_dev gives the length on the
// device (the grid is then sized for n and each block derives its share from the device value).
// num_heads: heads of the code cache; q_heads: rows of q_code / out / hist (a multiple of num_heads).
static int estimate_impl(const void* q_code, const void* code_data, const int32_t* code_page_table, int n,
                         int page_size, int num_heads, int q_heads, void* out, int64_t out_stride, int out_format,
                         int metric, const int32_t* seq_len_dev, uint32_t* hist, int hist_cl, adamas_stream_t stream,
                         const SeqDesc* seqs = nullptr, int batch = 1) {
  if (int rc = check_q_heads(num_heads, q_heads)) return rc;
  if (!seqs) batch = 1;
  const int q_group = q_heads / num_heads;
  ADAMAS_REQUIRE(q_code && out && (seqs || (code_data && code_page_table)), "null pointer");
  ADAMAS_REQUIRE(!seqs || seq_len_dev, "a batched estimate needs device lengths");
  ADAMAS_REQUIRE(out_stride >= n, "out_stride (%lld) smaller than the row length (%d)",
                 static_cast<long long>(out_stride), n);
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(q_code) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(code_data) & 15) == 0,
                 "q_code and code_data must be 16-byte aligned");
  ADAMAS_REQUIRE(!hist || (hist_cl >= 1 && hist_cl <= kSaMaxSlices), "histogram slices out of range (%d)", hist_cl);
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  cudaStream_t st = to_stream(stream);
  // (8 and 16 heads with histograms go token by token: in the page-copy kernel the 16 lanes of a count
  // instruction hit the tables of different heads, one L2 transaction each, where a warp of the token-copy
  // kernel counts 32 tokens of ONE head into a few neighbouring bins.  Measured at 32K with the counts: 16
  // heads 13.9 us by pages, 6.0 by tokens; 8 heads 7.9 / 6.6; 4 heads 4.7 / 7.7)
  constexpr int kPagesMaxHeadsWithHist = 4;
  if (q_group == 1 && num_heads <= 16 && !(hist && num_heads > kPagesMaxHeadsWithHist) && 32 % (2 * num_heads) == 0 &&
      page_size * num_heads * 32 >= 512) {
    // few heads (a head-sharded model): whole pages per copy, one chunk per lane
    const int page_bytes = page_size * num_heads * 32;
    const int ppt = std::max(1, std::min(32, 32768 / page_bytes));
    const int pages = (n + page_size - 1) / page_size;
    const int num_tiles = (pages + ppt - 1) / ppt;
    // spare bytes: a partial last unit reads up to 8 tokens past the valid ones
    const size_t smem = static_cast<size_t>(kEstStages) * ppt * page_bytes + 4096 + 512;
    ADAMAS_REQUIRE(smem <= static_cast<size_t>(di->max_smem_optin - 1024 - kEstPagesStatic),
                   "page too large for the estimate kernel");
    const int per_sm = std::min(est_blocks_per_sm(),
                                (smem + 1024 + kEstPagesStatic) * 2 <= static_cast<size_t>(di->max_smem_optin) ? 2 : 1);
    const unsigned blocks = static_cast<unsigned>(std::min(num_tiles, std::max(1, di->num_sms * per_sm / batch)));
    EstimatePagesParams pp;
    pp.codes = static_cast<const uint4*>(code_data);
    pp.page_table = code_page_table;
    pp.q_code = static_cast<const uint4*>(q_code);
    pp.out = out;
    pp.out_stride = out_stride;
    pp.n_tokens = n;
    pp.H = num_heads;
    pp.page_size = page_size;
    pp.pages_per_tile = ppt;
    pp.num_tiles = num_tiles;
    pp.stage_out = num_heads >= 16 ? 1 : 0;
    pp.seq_len_dev = seq_len_dev;
    pp.hist = hist;
    pp.hist_cl = hist_cl;
    pp.seqs = seqs;
#define LAUNCH_ESTP(M, OT) \
  ADAMAS_LAUNCH("estimate_pages_kernel", (estimate_pages_kernel<M, OT>), dim3(blocks, batch), dim3(kEstPagesThreads), smem, st, 1, pp)
    if (metric == ADAMAS_METRIC_L1) {
      if (out_format == ADAMAS_VAL_F16) LAUNCH_ESTP(0, __half); else LAUNCH_ESTP(0, uint16_t);
    } else {
      if (out_format == ADAMAS_VAL_F16) LAUNCH_ESTP(1, __half); else LAUNCH_ESTP(1, uint16_t);
    }
#undef LAUNCH_ESTP
    return check_launch("estimate_pages_kernel");
  }
  const int hpw = (num_heads % kEstConsumerWarps == 0) ? num_heads / kEstConsumerWarps : 0;
  const bool in_regs = q_group == 1 && (hpw == 1 || hpw == 2 || hpw == 4);   // grouped queries: the generic kernel
  // fewer than 16 heads: a tile holds 32 / H groups of 32 tokens, so that all 16 consumer warps work,
  // each on one head of two token groups
  const int groups = (q_group == 1 && num_heads < kEstConsumerWarps && kEstConsumerWarps % num_heads == 0)
                         ? 2 * kEstConsumerWarps / num_heads : 1;
  const int tile_span = kEstTile * groups;
  const int num_tiles = (n + tile_span - 1) / tile_span;
  const size_t smem = static_cast<size_t>(kEstStages) * tile_span * (2 * num_heads + 1) * 16 +
                      (in_regs ? 0 : static_cast<size_t>(2 * q_heads) * sizeof(QPlanes));
  ADAMAS_REQUIRE(smem <= static_cast<size_t>(di->max_smem_optin - 1024),
                 "num_heads (%d) too large for the estimate kernel", num_heads);
  const int per_sm = std::min(est_blocks_per_sm(), (smem + 1024) * 2 <= static_cast<size_t>(di->max_smem_optin) ? 2 : 1);
  const unsigned blocks = static_cast<unsigned>(std::min(num_tiles, std::max(1, di->num_sms * per_sm / batch)));
  EstimateParams prm;
  prm.seqs = seqs;
  prm.codes = static_cast<const uint4*>(code_data);
  prm.page_table = code_page_table;
  prm.q_code = static_cast<const uint4*>(q_code);
  prm.out = out;
  prm.out_stride = out_stride;
  prm.n_tokens = n;
  prm.H = num_heads;
  prm.q_group = q_group;
  prm.page_size = page_size;
  prm.ps_shift = log2_exact(page_size);
  prm.groups = groups;
  prm.num_tiles = num_tiles;
  prm.seq_len_dev = seq_len_dev;
  prm.hist = hist;
  prm.hist_cl = hist_cl;
#define LAUNCH_EST(M, OT)                                                                      \
  do {                                                                                         \
    if (in_regs && hpw == 1)                                                                   \
      ADAMAS_LAUNCH("estimate_kernel", estimate_kernel<M, OT, 1>, dim3(blocks, batch), dim3(kEstThreads), smem, st, 1, prm);                       \
    else if (in_regs && hpw == 2)                                                              \
      ADAMAS_LAUNCH("estimate_kernel", estimate_kernel<M, OT, 2>, dim3(blocks, batch), dim3(kEstThreads), smem, st, 1, prm);                       \
    else if (in_regs && hpw == 4)                                                              \
      ADAMAS_LAUNCH("estimate_kernel", estimate_kernel<M, OT, 4>, dim3(blocks, batch), dim3(kEstThreads), smem, st, 1, prm);                       \
    else                                                                                       \
      ADAMAS_LAUNCH("estimate_kernel", estimate_kernel<M, OT, 0>, dim3(blocks, batch), dim3(kEstThreads), smem, st, 1, prm);                       \
  } while (0)
  if (metric == ADAMAS_METRIC_L1) {
    if (out_format == ADAMAS_VAL_F16) LAUNCH_EST(0, __half); else LAUNCH_EST(0, uint16_t);
  } else {
    if (out_format == ADAMAS_VAL_F16) LAUNCH_EST(1, __half); else LAUNCH_EST(1, uint16_t);
  }
#undef LAUNCH_EST
  return check_launch("estimate_kernel");
}

int adamas_estimate(const void* q_code, const void* code_data, const int32_t* code_page_table,
                    int code_num_pages, int code_last_page_len, int page_size, int num_heads,
                    int num_q_heads, int head_dim, void* out, int64_t out_stride, int out_format, int metric,
                    int exclude_last, uint32_t* hist, int hist_slices, adamas_stream_t stream) {
  if (int rc = check_common(num_heads, head_dim, page_size, ADAMAS_F16)) return rc;
  ADAMAS_REQUIRE(code_num_pages >= 1, "page table must not be empty");
  ADAMAS_REQUIRE(code_last_page_len >= 1 && code_last_page_len <= page_size,
                 "code_last_page_len out of range");
  ADAMAS_REQUIRE(out_format == ADAMAS_VAL_F16 || out_format == ADAMAS_VAL_U16, "bad out_format %d",
                 out_format);
  ADAMAS_REQUIRE(metric == ADAMAS_METRIC_L1 || metric == ADAMAS_METRIC_XOR, "bad metric %d", metric);
  ADAMAS_REQUIRE(exclude_last == 0 || exclude_last == 1, "exclude_last must be 0 or 1");
  const int64_t n64 =
      static_cast<int64_t>(code_num_pages - 1) * page_size + code_last_page_len - exclude_last;
  ADAMAS_REQUIRE(n64 < (int64_t(1) << 31) - kEstTile * kEstConsumerWarps * 2, "sequence too long");
  if (n64 == 0) return ADAMAS_OK;
  return estimate_impl(q_code, code_data, code_page_table, static_cast<int>(n64), page_size, num_heads, num_q_heads,
                       out, out_stride, out_format, metric, nullptr, hist, hist_slices, stream);
}

// ---------------------------------------------------------------------------------------------
int adamas_topk(const void* values, int value_format, int64_t value_stride, int n,
                const int32_t* in_idx, int64_t in_idx_stride, int idx_page_size, int num_rows, int k,
                void* out_values, int32_t* out_idx, int64_t out_stride, adamas_stream_t stream) {
  ADAMAS_REQUIRE(value_format == ADAMAS_VAL_F16 || value_format == ADAMAS_VAL_U16,
                 "bad value_format %d", value_format);
  ADAMAS_REQUIRE(num_rows >= 0, "num_rows must be >= 0");
  if (num_rows == 0) return ADAMAS_OK;
  ADAMAS_REQUIRE(values && out_idx, "null pointer");
  ADAMAS_REQUIRE(n >= 1 && n < (1 << 30), "n out of range (%d)", n);
  ADAMAS_REQUIRE(k >= 1 && k <= n, "k must satisfy 1 <= k <= n (k=%d, n=%d)", k, n);
  ADAMAS_REQUIRE(value_stride >= n || num_rows == 1, "value_stride smaller than n");
  ADAMAS_REQUIRE(out_stride >= k || num_rows == 1, "out_stride smaller than k");
  ADAMAS_REQUIRE(idx_page_size >= 1, "idx_page_size must be >= 1");
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(values) & 1) == 0, "values must be 2-byte aligned");
  cudaStream_t st = to_stream(stream);
  const uint16_t* vals = static_cast<const uint16_t*>(values);
  uint16_t* ov = static_cast<uint16_t*>(out_values);

  // Rows that all start on a 16-byte boundary need ceil(n/8) granules, others up to one more.
  const bool aligned = (reinterpret_cast<uintptr_t>(values) & 15) == 0 &&
                       (num_rows == 1 || (value_stride * 2) % 16 == 0);
  const int g_max = aligned ? (n + 7) / 8 : (n + 14) / 8;
  // smallest ITEMS (granules per thread) that lets a cluster of up to 8 blocks of 256 threads cover
  // the row; rows beyond 65536 values use blocks of 1024 threads with 2 or 4 granules per thread
  int cl = 0, items = 0, nt = kTopkClThreads;
  for (int it = 1; it <= 4 && cl == 0; it *= 2) {
    for (int c = 1; c <= 8; c *= 2) {
      if (static_cast<int64_t>(c) * it * kTopkClThreads >= g_max) {
        cl = c;
        items = it;
        break;
      }
    }
  }
  if (cl == 0) {
    for (int it = 2; it <= 4 && cl == 0; it *= 2) {
      if (static_cast<int64_t>(8) * it * 1024 >= g_max) {
        cl = 8;
        items = it;
        nt = 1024;
      }
    }
  }
  if (cl > 0) {
    TopkParams prm;
    prm.values = vals;
    prm.value_stride = value_stride;
    prm.n = n;
    prm.in_idx = in_idx;
    prm.in_idx_stride = in_idx_stride;
    prm.idx_page_size = idx_page_size;
    prm.idx_ps_shift = -1;
    if ((idx_page_size & (idx_page_size - 1)) == 0) {
      prm.idx_ps_shift = 0;
      while ((1 << prm.idx_ps_shift) < idx_page_size) ++prm.idx_ps_shift;
    }
    prm.k = k;
    prm.out_values = ov;
    prm.out_idx = out_idx;
    prm.out_stride = out_stride;
    prm.granules_per_block = (g_max + cl - 1) / cl;
    const dim3 tgrid(static_cast<unsigned>(num_rows) * cl);
#define LAUNCH_TK(F, I, N)                                                                      \
  ADAMAS_LAUNCH("topk_cluster_kernel", (topk_cluster_kernel<F, I, N>), tgrid, dim3(N), 0, st, cl, prm)
#define LAUNCH_TK_ITEMS(F)                                  \
  if (nt == 1024) {                                         \
    if (items == 2) LAUNCH_TK(F, 2, 1024); else LAUNCH_TK(F, 4, 1024); \
  } else {                                                  \
    switch (items) {                                        \
      case 1: LAUNCH_TK(F, 1, 256); break;                  \
      case 2: LAUNCH_TK(F, 2, 256); break;                  \
      default: LAUNCH_TK(F, 4, 256); break;                 \
    }                                                       \
  }
    if (value_format == ADAMAS_VAL_F16) {
      LAUNCH_TK_ITEMS(0)
    } else {
      LAUNCH_TK_ITEMS(1)
    }
#undef LAUNCH_TK_ITEMS
#undef LAUNCH_TK
    return check_launch("topk_cluster_kernel");
  }

  // long rows: one block per row, staged in shared memory when it fits
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  const int max_smem = di->topk_dyn_smem;
  const int granules = (n + 7) / 8 + 1;
  int smem_granules = 0;
  size_t smem = 0;
  if (static_cast<size_t>(granules) * 16 <= static_cast<size_t>(max_smem)) {
    smem_granules = granules;
    smem = static_cast<size_t>(granules) * 16;
  }
  if (value_format == ADAMAS_VAL_F16)
    topk_kernel<0><<<num_rows, kTopkThreads, smem, st>>>(vals, value_stride, n, in_idx, in_idx_stride,
                                                         idx_page_size, k, ov, out_idx, out_stride,
                                                         smem_granules);
  else
    topk_kernel<1><<<num_rows, kTopkThreads, smem, st>>>(vals, value_stride, n, in_idx, in_idx_stride,
                                                         idx_page_size, k, ov, out_idx, out_stride,
                                                         smem_granules);
  return check_launch("topk_kernel");
}

// ---------------------------------------------------------------------------------------------
struct adamas_decode_handler {
  void* scratch = nullptr;        // partial_o | partial_ml | counters
  size_t scratch_bytes = 0;
  int64_t cap_units = 0;          // H * max_splits the scratch was sized for
  int cap_heads = 0;
  int num_sms = 0;
  int device = -1;
  bool forward_started = false;
  int num_heads = 0, page_size = 0, dtype = 0;   // num_heads: query heads (rows of q, o and the index lists)
  int kv_heads = 0;                              // heads of the KV cache (num_heads / kv_heads query heads share one)
  int batch = 1;                                 // sequences a batched dense step may carry (sizes the scratch)
};

namespace {

struct SplitPlan {
  int tiles_per_block;
  int num_splits;
};

// One wave of resident blocks: up to 4 single-tile blocks per SM (34 KB of shared memory each) or 3
// double-buffered multi-tile blocks (68 KB each), over all heads; never more splits than tiles.
SplitPlan plan_splits(int64_t n_tokens, int num_heads, int num_sms) {
  const int64_t tiles = (n_tokens + kDecTile - 1) / kDecTile;
  const int64_t cap1 = std::max<int64_t>(1, (static_cast<int64_t>(num_sms) * 4 + num_heads - 1) / num_heads);
  SplitPlan p;
  if (tiles <= cap1) {
    p.tiles_per_block = 1;
    p.num_splits = static_cast<int>(tiles);
    return p;
  }
  const int64_t cap2 = std::max<int64_t>(1, static_cast<int64_t>(num_sms) * 3 / num_heads);
  p.tiles_per_block = static_cast<int>((tiles + cap2 - 1) / cap2);
  p.num_splits = static_cast<int>((tiles + p.tiles_per_block - 1) / p.tiles_per_block);
  return p;
}

size_t scratch_layout(int64_t units, int heads, size_t* off_ml, size_t* off_cnt) {
  size_t o = static_cast<size_t>(units) * kHeadDim * sizeof(float);
  *off_ml = o;
  o += static_cast<size_t>(units) * 2 * sizeof(float);
  o = (o + 255) & ~static_cast<size_t>(255);
  *off_cnt = o;
  o += static_cast<size_t>(heads) * sizeof(unsigned);
  return (o + 255) & ~static_cast<size_t>(255);
}

}  // namespace

int adamas_decode_handler_create(adamas_decode_handler_t** handler) {
  ADAMAS_REQUIRE(handler, "null pointer");
  adamas_decode_handler* h = new (std::nothrow) adamas_decode_handler();
  ADAMAS_REQUIRE(h, "out of host memory");
  *handler = h;
  return ADAMAS_OK;
}

int adamas_decode_handler_destroy(adamas_decode_handler_t* handler) {
  if (!handler) return ADAMAS_OK;
  if (handler->scratch) cudaFree(handler->scratch);
  delete handler;
  return ADAMAS_OK;
}

int adamas_decode_begin_forward(adamas_decode_handler_t* handler, int64_t max_tokens, int batch, int num_heads,
                                int num_q_heads, int head_dim, int page_size, int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(handler, "null handler");
  ADAMAS_REQUIRE(batch >= 1 && batch <= 1024, "batch out of range (%d)", batch);
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  if (int rc = check_q_heads(num_heads, num_q_heads)) return rc;
  const int kv_heads = num_heads;
  num_heads = num_q_heads;   // from here on: the rows of the launch
  ADAMAS_REQUIRE(max_tokens >= 1 && max_tokens < (int64_t(1) << 31) - kDecTile, "max_tokens out of range");
  int dev = 0;
  ADAMAS_CUDA(cudaGetDevice(&dev));
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  if (handler->device != dev) {
    ADAMAS_REQUIRE(handler->scratch == nullptr, "handler was planned on another device");
    handler->num_sms = di->num_sms;
    handler->device = dev;
  }
  // The planner never gives a head more than ceil(4 * SMs / H) splits, so H * splits <= 4 * SMs + H
  // whatever the length: sized once for that bound, the scratch never has to grow while the head count
  // stays (a regrow costs a stream synchronisation and a cudaFree / cudaMalloc pair).
  const int rows = num_heads * batch;
  const int64_t units = static_cast<int64_t>(4) * handler->num_sms + rows;
  if (units > handler->cap_units || rows > handler->cap_heads) {
    size_t off_ml, off_cnt;
    const int64_t new_units = units > handler->cap_units ? units : handler->cap_units;
    const int new_heads = rows > handler->cap_heads ? rows : handler->cap_heads;
    const size_t bytes = scratch_layout(new_units, new_heads, &off_ml, &off_cnt);
    if (handler->scratch) {
      // earlier launches on this stream may still use the old buffer
      ADAMAS_CUDA(cudaStreamSynchronize(to_stream(stream)));
      ADAMAS_CUDA(cudaFree(handler->scratch));
      handler->scratch = nullptr;
      handler->cap_units = 0;
      handler->cap_heads = 0;
    }
    ADAMAS_CUDA(cudaMalloc(&handler->scratch, bytes));
    ADAMAS_CUDA(cudaMemsetAsync(handler->scratch, 0, bytes, to_stream(stream)));
    handler->scratch_bytes = bytes;
    handler->cap_units = new_units;
    handler->cap_heads = new_heads;
  }
  handler->forward_started = true;
  handler->num_heads = num_heads;
  handler->kv_heads = kv_heads;
  handler->batch = batch;
  handler->page_size = page_size;
  handler->dtype = dtype;
  return ADAMAS_OK;
}

int adamas_decode_end_forward(adamas_decode_handler_t* handler) {
  ADAMAS_REQUIRE(handler, "null handler");
  handler->forward_started = false;
  return ADAMAS_OK;
}

// seq_len_dev (optional): attend to every token of a sequence whose length lives on the device; indices
// is then the page table, n_idx / tail_len describe the LONGEST sequence (they size the grid), and the
// kernel derives the actual lists from the device value.
static int decode_forward_impl(adamas_decode_handler_t* handler, const void* q, void* o, float* o_f32,
                               float* lse, const void* kv_data, const int32_t* indices,
                               int64_t idx_stride, int n_idx, int idx_unit, int last_page_idx,
                               int last_page_len, int tail_len, float sm_scale,
                               adamas_stream_t stream, const int32_t* seq_len_dev = nullptr,
                               const SeqDesc* seqs = nullptr, int batch = 1) {
  ADAMAS_REQUIRE(handler, "null handler");
  if (!handler->forward_started)
    return fail(ADAMAS_ERR_STATE, "decode forward called before begin_forward");
  ADAMAS_REQUIRE(q && (o || o_f32) && (kv_data || seqs), "null pointer");
  ADAMAS_REQUIRE(n_idx >= 0 && (n_idx == 0 || indices || seqs), "indices missing");
  ADAMAS_REQUIRE(!seqs || (seq_len_dev && batch >= 1 && batch <= handler->batch),
                 "a batched dense step needs device lengths and a handler planned for the batch");
  if (!seqs) batch = 1;
  const int ps = handler->page_size;
  ADAMAS_REQUIRE(idx_unit == 1 || idx_unit == ps, "idx_unit must be 1 or page_size");
  ADAMAS_REQUIRE(tail_len >= 0 && tail_len <= last_page_len && last_page_len <= ps,
                 "tail_len / last_page_len out of range");
  ADAMAS_REQUIRE(last_page_idx >= 0, "last_page_idx must be >= 0");
  const int64_t n_tokens = static_cast<int64_t>(n_idx) * idx_unit + tail_len;
  ADAMAS_REQUIRE(n_tokens >= 1, "nothing to attend to");
  ADAMAS_REQUIRE(n_tokens < (int64_t(1) << 31) - kDecTile, "too many tokens");
  ADAMAS_REQUIRE(idx_stride == 0 || idx_stride >= n_idx || handler->num_heads == 1,
                 "idx_stride must be 0 (shared row) or >= n_idx");
  const int H = handler->num_heads;
  const SplitPlan p = plan_splits(n_tokens, H * batch, handler->num_sms);
  if (static_cast<int64_t>(H) * batch * p.num_splits > handler->cap_units)
    return fail(ADAMAS_ERR_STATE,
                "decode forward needs %d splits per head but begin_forward planned for fewer tokens",
                p.num_splits);
  size_t off_ml, off_cnt;
  scratch_layout(handler->cap_units, handler->cap_heads, &off_ml, &off_cnt);
  DecodeParams prm;
  prm.q = q;
  prm.o = o;
  prm.o_f32 = o_f32;
  prm.lse = lse;
  prm.kv = kv_data;
  prm.indices = indices ? indices : reinterpret_cast<const int32_t*>(kv_data);
  prm.seqs = seqs;
  prm.idx_stride = idx_stride;
  prm.n_idx = n_idx;
  prm.idx_unit = idx_unit;
  prm.page_size = ps;
  prm.H = handler->kv_heads;
  prm.q_group = H / handler->kv_heads;
  const int64_t tail0 = static_cast<int64_t>(last_page_idx) * ps + (last_page_len - tail_len);
  ADAMAS_REQUIRE(tail0 + tail_len < (int64_t(1) << 31), "token slots must be below 2^31");
  prm.tail_slot0 = static_cast<unsigned>(tail0);
  prm.ps_shift = -1;
  if ((ps & (ps - 1)) == 0) {
    prm.ps_shift = 0;
    while ((1 << prm.ps_shift) < ps) ++prm.ps_shift;
  }
  prm.n_tokens = static_cast<int>(n_tokens);
  prm.tiles_per_block = p.tiles_per_block;
  prm.num_splits = p.num_splits;
  uint8_t* base = static_cast<uint8_t*>(handler->scratch);
  prm.partial_o = reinterpret_cast<float*>(base);
  prm.partial_ml = reinterpret_cast<float*>(base + off_ml);
  prm.counters = reinterpret_cast<unsigned*>(base + off_cnt);
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.seq_len_dev = seq_len_dev;
  // (with the length on the device a block may get more than one tile later on: two stages)
  const size_t smem = static_cast<size_t>(p.tiles_per_block > 1 || seq_len_dev ? 2 : 1) * kDecStageBytes;
  dim3 grid(p.num_splits, H, batch);
  if (handler->dtype == ADAMAS_F16)
    ADAMAS_LAUNCH("sparse_decode_kernel", sparse_decode_kernel<__half>, grid, dim3(kDecThreads), smem,
                  to_stream(stream), 1, prm);
  else
    ADAMAS_LAUNCH("sparse_decode_kernel", sparse_decode_kernel<__nv_bfloat16>, grid, dim3(kDecThreads), smem,
                  to_stream(stream), 1, prm);
  return check_launch("sparse_decode_kernel");
}

int adamas_decode_forward(adamas_decode_handler_t* handler, const void* q, void* o, float* lse,
                          const void* kv_data, const int32_t* indices, int64_t idx_stride, int n_idx,
                          int idx_unit, int last_page_idx, int last_page_len, int tail_len,
                          float sm_scale, adamas_stream_t stream) {
  return decode_forward_impl(handler, q, o, nullptr, lse, kv_data, indices, idx_stride, n_idx, idx_unit,
                             last_page_idx, last_page_len, tail_len, sm_scale, stream);
}

int adamas_decode_forward_partial(adamas_decode_handler_t* handler, const void* q, float* o_f32,
                                  float* lse, const void* kv_data, const int32_t* indices,
                                  int64_t idx_stride, int n_idx, int idx_unit, int last_page_idx,
                                  int last_page_len, int tail_len, float sm_scale,
                                  adamas_stream_t stream) {
  return decode_forward_impl(handler, q, nullptr, o_f32, lse, kv_data, indices, idx_stride, n_idx,
                             idx_unit, last_page_idx, last_page_len, tail_len, sm_scale, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the sparse decode.  Its split-KV scratch (partial outputs, running
// max / sum pairs and the per-head arrival counters) lives in the fixed array below instead of a
// handler-owned cudaMalloc buffer.  Every device that loads this library keeps the array until
// the process exits; all calls on a device share it.
constexpr int kStaticMaxUnits = 2048;   // heads x splits
constexpr int kStaticMaxHeads = 256;
constexpr size_t kStaticOffMl = static_cast<size_t>(kStaticMaxUnits) * kHeadDim * sizeof(float);
constexpr size_t kStaticOffCnt = kStaticOffMl + static_cast<size_t>(kStaticMaxUnits) * 2 * sizeof(float);
constexpr size_t kStaticBytes = kStaticOffCnt + static_cast<size_t>(kStaticMaxHeads) * sizeof(unsigned);
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticBytes];

int adamas_decode_forward_static(const void* q, void* o, float* lse, const void* kv_data,
                                 const int32_t* indices, int64_t idx_stride, int n_idx, int idx_unit,
                                 int num_heads, int head_dim, int page_size, int dtype,
                                 int last_page_idx, int last_page_len, int tail_len, float sm_scale,
                                 adamas_stream_t stream) {
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  ADAMAS_REQUIRE(q && o && kv_data, "null pointer");
  ADAMAS_REQUIRE(n_idx >= 0 && (n_idx == 0 || indices), "indices missing");
  ADAMAS_REQUIRE(idx_unit == 1 || idx_unit == page_size, "idx_unit must be 1 or page_size");
  ADAMAS_REQUIRE(tail_len >= 0 && tail_len <= last_page_len && last_page_len <= page_size,
                 "tail_len / last_page_len out of range");
  ADAMAS_REQUIRE(last_page_idx >= 0, "last_page_idx must be >= 0");
  const int64_t n_tokens = static_cast<int64_t>(n_idx) * idx_unit + tail_len;
  ADAMAS_REQUIRE(n_tokens >= 1, "nothing to attend to");
  ADAMAS_REQUIRE(n_tokens < (int64_t(1) << 31) - kDecTile, "too many tokens");
  ADAMAS_REQUIRE(idx_stride == 0 || idx_stride >= n_idx || num_heads == 1,
                 "idx_stride must be 0 (shared row) or >= n_idx");

  // Per-device set-up on the first call with that device current: the name of a __device__ array is
  // only a host-side handle, so the address the kernel needs is looked up once and kept.
  static void* scratch_ptr[64] = {};
  int dev = 0;
  ADAMAS_CUDA(cudaGetDevice(&dev));
  ADAMAS_REQUIRE(dev >= 0 && dev < 64, "device ordinal out of range");
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  std::unique_lock<std::mutex> init_lock(g_init_mutex);
  if (scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    ADAMAS_CUDA(cudaGetSymbolAddress(&ptr, g_static_decode_scratch));
    ADAMAS_REQUIRE(ptr != nullptr, "cudaGetSymbolAddress returned a null address");
    scratch_ptr[dev] = ptr;
  }
  init_lock.unlock();

  const SplitPlan p = plan_splits(n_tokens, num_heads, di->num_sms);
  ADAMAS_REQUIRE(num_heads <= kStaticMaxHeads,
                 "adamas_decode_forward_static supports at most %d heads (got %d)", kStaticMaxHeads,
                 num_heads);
  ADAMAS_REQUIRE(static_cast<int64_t>(num_heads) * p.num_splits <= kStaticMaxUnits,
                 "adamas_decode_forward_static: %d heads x %d splits exceeds the fixed scratch of %d "
                 "(head, split) units; use the handler-based adamas_decode_forward",
                 num_heads, p.num_splits, kStaticMaxUnits);

  uint8_t* base = static_cast<uint8_t*>(scratch_ptr[dev]);
  cudaStream_t st = to_stream(stream);
  // the arrival counters must start at zero whatever an earlier (possibly failed) call left behind
  ADAMAS_CUDA(cudaMemsetAsync(base + kStaticOffCnt, 0, static_cast<size_t>(num_heads) * sizeof(unsigned), st));

  DecodeParams prm;
  prm.q = q;
  prm.o = o;
  prm.o_f32 = nullptr;
  prm.lse = lse;
  prm.kv = kv_data;
  prm.indices = indices ? indices : reinterpret_cast<const int32_t*>(kv_data);
  prm.idx_stride = idx_stride;
  prm.n_idx = n_idx;
  prm.idx_unit = idx_unit;
  prm.page_size = page_size;
  prm.H = num_heads;
  prm.q_group = 1;
  prm.seqs = nullptr;
  const int64_t tail0 = static_cast<int64_t>(last_page_idx) * page_size + (last_page_len - tail_len);
  ADAMAS_REQUIRE(tail0 + tail_len < (int64_t(1) << 31), "token slots must be below 2^31");
  prm.tail_slot0 = static_cast<unsigned>(tail0);
  prm.ps_shift = -1;
  if ((page_size & (page_size - 1)) == 0) {
    prm.ps_shift = 0;
    while ((1 << prm.ps_shift) < page_size) ++prm.ps_shift;
  }
  prm.n_tokens = static_cast<int>(n_tokens);
  prm.tiles_per_block = p.tiles_per_block;
  prm.num_splits = p.num_splits;
  prm.partial_o = reinterpret_cast<float*>(base);
  prm.partial_ml = reinterpret_cast<float*>(base + kStaticOffMl);
  prm.counters = reinterpret_cast<unsigned*>(base + kStaticOffCnt);
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  prm.seq_len_dev = nullptr;
  const size_t smem = static_cast<size_t>(p.tiles_per_block > 1 ? 2 : 1) * kDecStageBytes;
  dim3 grid(p.num_splits, num_heads);
  if (dtype == ADAMAS_F16)
    sparse_decode_kernel<__half><<<grid, kDecThreads, smem, st>>>(prm);
  else
    sparse_decode_kernel<__nv_bfloat16><<<grid, kDecThreads, smem, st>>>(prm);
  return check_launch("sparse_decode_kernel (static scratch)");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
namespace {

template <typename T, int I>
int launch_select_attend_one(const SelectAttendParams& prm, int cl, int num_heads, int batch, size_t smem,
                             cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>(cl), static_cast<unsigned>(num_heads), static_cast<unsigned>(batch));
  ADAMAS_LAUNCH("select_attend_kernel", (select_attend_kernel<T, I>), grid, dim3(kSaThreads), smem, st, 1, prm);
  return check_launch("select_attend_kernel");
}

template <typename T>
int launch_select_attend(const SelectAttendParams& prm, int items, int cl, int num_heads, int batch, size_t smem,
                         cudaStream_t st) {
  switch (items) {
    case 1: return launch_select_attend_one<T, 1>(prm, cl, num_heads, batch, smem, st);
    case 2: return launch_select_attend_one<T, 2>(prm, cl, num_heads, batch, smem, st);
    case 4: return launch_select_attend_one<T, 4>(prm, cl, num_heads, batch, smem, st);
    case 8: return launch_select_attend_one<T, 8>(prm, cl, num_heads, batch, smem, st);
    default: break;
  }
  return fail(ADAMAS_ERR_INVALID, "unsupported row length for select_attend");
}

// Shape of a select_attend launch: blocks per head (= histogram slices), granules per thread, winner
// list and dynamic shared memory (the tile | winner list).  Planned for rows of up to n distances; shorter rows run in the same shape.
struct SaPlan {
  int cl, items, list_capacity;
  size_t smem;
};

void sa_shape(int n, int k, int cl, SaPlan* pl) {
  const int slice_tokens = std::min(n, sa_granules_per_block(n, cl) * 8);
  const int max_loc = std::min(k, slice_tokens) + 1;   // winners of one block at most, plus the newest token
  pl->list_capacity = max_loc;
  pl->smem = static_cast<size_t>(kSaWarps) * 2 * kSaWarpRows * 256 +
             ((static_cast<size_t>(pl->list_capacity) * 4 + 15) & ~static_cast<size_t>(15));
}

int sa_plan(int n, int k, int num_heads, const DeviceInfo* di, SaPlan* pl) {
  const int g_total = (n + 7) / 8;
  // Blocks per head: any number up to 16 (the blocks of a head do not wait for one another).  num_heads
  // counts the rows of the launch (query heads x sequences).  By default up to 8 blocks, or more as long as
  // every block of the launch is resident at once (a row a little beyond 8 * 512 granules then takes 9
  // blocks instead of two granules per thread, which would double the selection's work);
  // adamas_set_max_cluster lowers the bound.
  const int user_limit = max_cluster();
  const int resident_blocks = 2 * di->num_sms;
  const int resident = std::max(1, resident_blocks / num_heads);
  const int cl_limit = user_limit < kSaMaxCluster ? user_limit
                                                  : std::min(kSaBigCluster, std::max(kSaMaxCluster, resident));
  // As few granules per thread as possible while the whole launch is resident at once: a block's work is a
  // chain of short dependent steps that leaves the SM mostly idle, so a second wave of blocks costs a whole
  // chain again, while more granules per thread only lengthen the first steps (many rows, i.e. a batch of
  // sequences: 128 rows of 32K distances run as 2 blocks x 4 granules, not 8 x 1 in four waves).  If no
  // shape is resident at once, the one with the fewest blocks.
  int cl = 0, items = 0, fewest_cl = 0, fewest_items = 0;
  for (int it = 1; it <= 8 && cl == 0; it *= 2) {
    const int need = std::max(1, (g_total + it * kSaThreads - 1) / (it * kSaThreads));
    if (need > cl_limit) continue;
    fewest_cl = need;
    fewest_items = it;
    if (need * num_heads <= resident_blocks) {
      cl = need;
      items = it;
    }
  }
  if (cl == 0) {
    cl = fewest_cl;
    items = fewest_items;
  }
  ADAMAS_REQUIRE(cl > 0, "select_attend supports at most %d distances per head with %d blocks per head (got %d)",
                 cl_limit * 8 * kSaThreads * 8, cl_limit, n);
  // with several granules per thread, rather twice the blocks with half-filled threads than the fewest
  // blocks that cover the row, if they are still resident at once
  if (items >= 2) {
    const int twice = std::min(cl_limit, std::max(cl, (g_total + items * kSaThreads / 2 - 1) / (items * kSaThreads / 2)));
    if (twice * num_heads <= resident_blocks) cl = twice;
  }
  // a large budget on a short row: more blocks per head than the scan needs, so that each block
  // attends to about one tile of winners, as long as all blocks stay resident at once
  while (cl < std::min(cl_limit, kSaMaxCluster) && k > cl * kSaTile && 2 * cl * num_heads <= resident_blocks) cl *= 2;
  cl = std::min(cl, cl_limit);
  pl->cl = cl;
  pl->items = items;
  sa_shape(n, k, cl, pl);
  ADAMAS_REQUIRE(pl->smem <= static_cast<size_t>(kSaMaxDynSmem), "winner list too long for select_attend (k=%d)", k);
  return ADAMAS_OK;
}

// n: distances per head, or their upper bound when seq_len_dev is given.
// num_heads: heads of the KV cache; q_heads: rows of the launch (a multiple of num_heads).
int select_attend_impl(const void* dist, int64_t dist_stride, int n, int k, const void* q, void* o, float* o_f32,
                       float* lse, const void* kv_data, const int32_t* kv_page_table, int page_size, int num_heads,
                       int q_heads, int dtype, int tail_mode, unsigned tail_slot, uint32_t* hist, const int32_t* ext_cut,
                       const int32_t* seq_len_dev, int32_t* out_idx, int64_t out_stride, float sm_scale,
                       const SaPlan& pl, adamas_stream_t stream, const SeqDesc* seqs = nullptr, int batch = 1,
                       const RopeSpec* rope_q = nullptr) {
  SelectAttendParams prm;
  prm.rope_on = rope_q != nullptr && rope_q->on;
  prm.rope = RopeParams{1.f, 1e4f, nullptr, 1.f};
  if (prm.rope_on)
    prm.rope = RopeParams{rope_q->scale > 0.f ? 1.0f / rope_q->scale : 1.f, rope_q->theta, rope_q->inv_freq, rope_q->mscale};
  prm.seqs = seqs;
  if (!seqs) batch = 1;
  prm.dist = static_cast<const uint16_t*>(dist);
  prm.dist_stride = dist_stride;
  prm.hist = hist;
  prm.ext_cut = reinterpret_cast<const int2*>(ext_cut);
  prm.seq_len_dev = seq_len_dev;
  prm.n = n;
  prm.k = k;
  prm.q = q;
  prm.o = o;
  prm.o_f32 = o_f32;
  prm.lse = lse;
  prm.kv = kv_data;
  prm.kv_table = kv_page_table;
  prm.page_size = page_size;
  prm.ps_shift = log2_exact(page_size);
  prm.H = num_heads;
  prm.q_group = q_heads / num_heads;
  prm.tail_mode = tail_mode;
  prm.tail_slot = tail_slot;
  prm.out_idx = out_idx;
  prm.out_stride = out_stride;
  prm.list_capacity = pl.list_capacity;
  prm.scale_log2 = sm_scale * 1.4426950408889634f;
  if (dtype == ADAMAS_F16)
    return launch_select_attend<__half>(prm, pl.items, pl.cl, q_heads, batch, pl.smem, to_stream(stream));
  return launch_select_attend<__nv_bfloat16>(prm, pl.items, pl.cl, q_heads, batch, pl.smem, to_stream(stream));
}

static_assert(ADAMAS_HIST_WORDS_PER_HEAD == kSaScratchWordsPerHead, "scratch layout of select_attend");
size_t hist_bytes(int num_heads) {
  return static_cast<size_t>(num_heads) * ADAMAS_HIST_WORDS_PER_HEAD * sizeof(uint32_t);
}

__global__ void seq_len_advance_kernel(int32_t* seq_len, int count, int delta) {
  if (static_cast<int>(threadIdx.x) < count) seq_len[threadIdx.x] += delta;
}

}  // namespace

extern "C" {

int adamas_select_attend_slices(int n, int k, int num_heads, int* slices) {
  ADAMAS_REQUIRE(slices, "null pointer");
  ADAMAS_REQUIRE(n >= 1 && k >= 1 && k <= n && num_heads >= 1, "need 1 <= k <= n (k=%d, n=%d)", k, n);
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  SaPlan pl;
  if (int rc = sa_plan(n, k, num_heads, di, &pl)) return rc;
  *slices = pl.cl;
  return ADAMAS_OK;
}

int adamas_select_attend(const void* dist, int64_t dist_stride, int n, int k, const void* q, void* o,
                         float* o_f32, float* lse, const void* kv_data, const int32_t* kv_page_table,
                         int page_size, int num_heads, int num_q_heads, int head_dim, int dtype,
                         int last_page_idx, int last_page_len, uint32_t* hist, int hist_ready,
                         const int32_t* ext_cut, int32_t* out_idx, int64_t out_stride, float sm_scale,
                         adamas_stream_t stream) {
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  if (int rc = check_q_heads(num_heads, num_q_heads)) return rc;
  const int kv_heads = num_heads;
  num_heads = num_q_heads;   // rows of dist, q, o, hist, out_idx
  ADAMAS_REQUIRE(dist && q && (o || o_f32) && kv_data && kv_page_table && hist, "null pointer");
  ADAMAS_REQUIRE(!o_f32 || lse, "a partial result (o_f32) needs lse");
  ADAMAS_REQUIRE(n >= 1 && k >= 1 && k <= n, "need 1 <= k <= n (k=%d, n=%d)", k, n);
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(dist) & 15) == 0 && (num_heads == 1 || (dist_stride * 2) % 16 == 0),
                 "distance rows must start on 16-byte boundaries");
  ADAMAS_REQUIRE(dist_stride >= n || num_heads == 1, "dist_stride smaller than n");
  ADAMAS_REQUIRE(last_page_idx >= 0 && last_page_len >= 0 && last_page_len <= page_size,
                 "last page out of range");
  ADAMAS_REQUIRE(out_idx == nullptr || out_stride >= k || num_heads == 1, "out_stride smaller than k");
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(ext_cut) & 7) == 0, "ext_cut must be 8-byte aligned");
  const int64_t tail = static_cast<int64_t>(last_page_idx) * page_size + last_page_len - 1;
  ADAMAS_REQUIRE(tail < (int64_t(1) << 31), "token slots must be below 2^31");
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  SaPlan pl;
  if (int rc = sa_plan(n, k, num_heads, di, &pl)) return rc;
  if (!hist_ready) {
    DistHistogramParams hp;
    hp.dist = static_cast<const uint16_t*>(dist);
    hp.dist_stride = dist_stride;
    hp.hist = hist;
    hp.n = n;
    hp.cl = pl.cl;
    hp.seq_len_dev = nullptr;
    ADAMAS_LAUNCH("dist_histogram_kernel", dist_histogram_kernel, dim3(pl.cl, num_heads), dim3(kSaThreads), 0,
                  to_stream(stream), 1, hp);
  }
  return select_attend_impl(dist, dist_stride, n, k, q, o, o_f32, lse, kv_data, kv_page_table, page_size, kv_heads,
                            num_heads, dtype, last_page_len > 0 ? 1 : 0, static_cast<unsigned>(std::max<int64_t>(tail, 0)), hist,
                            ext_cut, nullptr, out_idx, out_stride, sm_scale, pl, stream);
}

int adamas_dist_histograms(const void* dist, int64_t dist_stride, int n, int num_heads, int slices, uint32_t* hist,
                           adamas_stream_t stream) {
  ADAMAS_REQUIRE(dist && hist, "null pointer");
  ADAMAS_REQUIRE(n >= 1 && num_heads >= 1 && slices >= 1 && slices <= kSaMaxSlices, "n / num_heads / slices out of range");
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(dist) & 15) == 0 && (num_heads == 1 || (dist_stride * 2) % 16 == 0),
                 "distance rows must start on 16-byte boundaries");
  ADAMAS_REQUIRE(dist_stride >= n || num_heads == 1, "dist_stride smaller than n");
  DistHistogramParams hp;
  hp.dist = static_cast<const uint16_t*>(dist);
  hp.dist_stride = dist_stride;
  hp.hist = hist;
  hp.n = n;
  hp.cl = slices;
  hp.seq_len_dev = nullptr;
  ADAMAS_LAUNCH("dist_histogram_kernel", dist_histogram_kernel, dim3(slices, num_heads), dim3(kSaThreads), 0,
                to_stream(stream), 1, hp);
  return check_launch("dist_histogram_kernel");
}

int adamas_hist_rowsum(const uint32_t* hist, int num_heads, int slices, uint32_t* out, adamas_stream_t stream) {
  ADAMAS_REQUIRE(hist && out, "null pointer");
  ADAMAS_REQUIRE(num_heads >= 1 && slices >= 1 && slices <= kSaMaxSlices, "num_heads / slices out of range");
  ADAMAS_LAUNCH("hist_rowsum_kernel", hist_rowsum_kernel, dim3(num_heads), dim3(kSaBins), 0, to_stream(stream), 1, hist,
                slices, out);
  return check_launch("hist_rowsum_kernel");
}

int adamas_global_cut(const uint32_t* all_hists, int num_shards, int shard, int num_heads, int k, int32_t* ext_cut,
                      adamas_stream_t stream) {
  ADAMAS_REQUIRE(all_hists && ext_cut, "null pointer");
  ADAMAS_REQUIRE(num_shards >= 1 && shard >= 0 && shard < num_shards && num_heads >= 1 && k >= 1,
                 "shard / num_shards / num_heads / k out of range");
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(ext_cut) & 7) == 0, "ext_cut must be 8-byte aligned");
  global_cut_kernel<<<num_heads, kSaBins, 0, to_stream(stream)>>>(all_hists, num_shards, shard, num_heads, k,
                                                                  reinterpret_cast<int2*>(ext_cut));
  return check_launch("global_cut_kernel");
}

int adamas_seq_len_advance(int32_t* seq_len_dev, int count, int delta, adamas_stream_t stream) {
  ADAMAS_REQUIRE(seq_len_dev, "null pointer");
  ADAMAS_REQUIRE(count >= 1 && count <= 1024, "count out of range (%d)", count);
  // an ordinary launch: it completes before anything that follows it in the stream starts
  ADAMAS_LAUNCH("seq_len_advance_kernel", seq_len_advance_kernel, dim3(1), dim3(static_cast<unsigned>((count + 31) / 32 * 32)),
                0, to_stream(stream), -1, seq_len_dev, count, delta);
  return check_launch("seq_len_advance_kernel");
}

// Stages 1 + 2 of a decode step in one launch (estimate_append_kernel); the caller has checked that
// num_heads is 16, 32 or 64.  n: distances per head (host mode) or their upper bound (seq_len_dev).
static int estimate_append_launch(const void* q, const void* k, const void* v, void* q_code, void* kv_data,
                                  const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                                  void* code_data, const int32_t* code_page_table, int code_num_pages,
                                  int code_last_page_len, int n, int num_heads, int page_size, int dtype, void* dist,
                                  int64_t dist_stride, float hadamard_scale, const float* thresholds3_host,
                                  const int32_t* seq_len_dev, uint32_t* hist, int hist_cl, adamas_stream_t stream,
                                  const SeqDesc* seqs = nullptr, int batch = 1, const RopeSpec& rope = RopeSpec()) {
  ADAMAS_REQUIRE(q && k && v && q_code && dist && (seqs || (kv_data && code_data && kv_page_table && code_page_table)),
                 "null pointer");
  if (!seqs) batch = 1;
  ADAMAS_REQUIRE(n >= 1 && n < 2147483647 - kEstTile, "sequence length out of range");
  ADAMAS_REQUIRE(dist_stride >= n, "dist_stride (%lld) smaller than the row length (%d)",
                 static_cast<long long>(dist_stride), n);
  ADAMAS_REQUIRE((seqs || (reinterpret_cast<uintptr_t>(code_data) & 15) == 0) && (reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(k) & 15) == 0 && (reinterpret_cast<uintptr_t>(v) & 15) == 0,
                 "q, k, v and code_data must be 16-byte aligned");
  ADAMAS_REQUIRE(!hist || (hist_cl >= 1 && hist_cl <= kSaMaxSlices), "histogram slices out of range (%d)", hist_cl);
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  const int num_tiles = (n + kEstTile - 1) / kEstTile;
  const int hpw = num_heads / kEstConsumerWarps;
  const size_t smem = static_cast<size_t>(kEstStages) * kEstTile * (2 * num_heads + 1) * 16;
  ADAMAS_REQUIRE(smem <= static_cast<size_t>(di->max_smem_optin - 1024 - kEstAppendStatic),
                 "num_heads (%d) too large", num_heads);
  const int per_sm = std::min(est_blocks_per_sm(),
                              (smem + 1024 + kEstAppendStatic) * 2 <= static_cast<size_t>(di->max_smem_optin) ? 2 : 1);
  const unsigned blocks = static_cast<unsigned>(std::min(num_tiles, std::max(1, di->num_sms * per_sm / batch)));
  EstimateParams prm;
  prm.seqs = seqs;
  prm.codes = static_cast<const uint4*>(code_data);
  prm.page_table = code_page_table;
  prm.q_code = nullptr;
  prm.out = dist;
  prm.out_stride = dist_stride;
  prm.n_tokens = n;
  prm.H = num_heads;
  prm.q_group = 1;
  prm.page_size = page_size;
  prm.ps_shift = log2_exact(page_size);
  prm.groups = 1;
  prm.num_tiles = num_tiles;
  prm.seq_len_dev = seq_len_dev;
  prm.hist = hist;
  prm.hist_cl = hist_cl;
  StepAppend ap;
  ap.q = q;
  ap.k = k;
  ap.v = v;
  ap.q_code_out = static_cast<uint16_t*>(q_code);
  ap.tgt = PagedTarget{kv_data, kv_page_table, static_cast<uint16_t*>(code_data), code_page_table, page_size,
                       num_heads};
  ap.kv_last_page = kv_num_pages - 1;
  ap.kv_entry = kv_last_page_len - 1;
  ap.code_last_page = code_num_pages - 1;
  ap.code_entry = code_last_page_len - 1;
  ap.scale = hadamard_scale;
  ap.th = make_thresholds(thresholds3_host);
  ap.rp = RopeParams{rope.scale > 0.f ? 1.0f / rope.scale : 1.f, rope.theta, rope.inv_freq, rope.mscale};
  cudaStream_t st = to_stream(stream);
#define LAUNCH_ESTA(T, HPW, R)                                                                        \
  ADAMAS_LAUNCH("estimate_append_kernel", (estimate_append_kernel<T, HPW, R>), dim3(blocks, batch),   \
                dim3(kEstThreads), smem, st, 1, prm, ap)
#define LAUNCH_ESTA_T(T)                                                        \
  do {                                                                          \
    if (rope.on) {                                                              \
      if (hpw == 1) LAUNCH_ESTA(T, 1, true);                                    \
      else if (hpw == 2) LAUNCH_ESTA(T, 2, true);                               \
      else LAUNCH_ESTA(T, 4, true);                                             \
    } else {                                                                    \
      if (hpw == 1) LAUNCH_ESTA(T, 1, false);                                   \
      else if (hpw == 2) LAUNCH_ESTA(T, 2, false);                              \
      else LAUNCH_ESTA(T, 4, false);                                            \
    }                                                                           \
  } while (0)
  if (dtype == ADAMAS_F16) LAUNCH_ESTA_T(__half); else LAUNCH_ESTA_T(__nv_bfloat16);
#undef LAUNCH_ESTA_T
#undef LAUNCH_ESTA
  return check_launch("estimate_append_kernel");
}

int adamas_append_estimate(const void* q, const void* k, const void* v, void* q_code, void* kv_data,
                           const int32_t* kv_page_table, int kv_num_pages, int kv_last_page_len,
                           void* code_data, const int32_t* code_page_table, int code_num_pages,
                           int code_last_page_len, int num_heads, int head_dim, int page_size, int dtype,
                           void* dist, int64_t dist_stride, float hadamard_scale,
                           const float* thresholds3_host, uint32_t* hist, int hist_slices,
                           adamas_stream_t stream) {
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  ADAMAS_REQUIRE(num_heads == 16 || num_heads == 32 || num_heads == 64,
                 "adamas_append_estimate supports 16, 32 or 64 heads (got %d); use adamas_append_decode_fused "
                 "and adamas_estimate", num_heads);
  ADAMAS_REQUIRE(kv_num_pages >= 1 && code_num_pages >= 1, "page tables must not be empty");
  ADAMAS_REQUIRE(kv_last_page_len >= 1 && kv_last_page_len <= page_size, "kv_last_page_len out of range");
  ADAMAS_REQUIRE(code_last_page_len >= 1 && code_last_page_len <= page_size,
                 "code_last_page_len out of range");
  const int64_t n64 = static_cast<int64_t>(code_num_pages - 1) * page_size + code_last_page_len - 1;
  ADAMAS_REQUIRE(n64 >= 1 && n64 < (int64_t(1) << 31) - kEstTile, "sequence length out of range");
  return estimate_append_launch(q, k, v, q_code, kv_data, kv_page_table, kv_num_pages, kv_last_page_len,
                                code_data, code_page_table, code_num_pages, code_last_page_len,
                                static_cast<int>(n64), num_heads, page_size, dtype, dist, dist_stride,
                                hadamard_scale, thresholds3_host, nullptr, hist, hist_slices, stream);
}

// One layer's decode step.  Host mode (seq_len_dev null): seq_len tokens are in the caches, the newest
// included.  Device mode: *seq_len_dev holds that number and seq_len is its upper bound, which sizes the
// launches.
static int decode_step_impl(void* q, void* k, const void* v, void* o, float* lse, void* q_code, void* kv_data,
                            const int32_t* kv_page_table, int kv_last_page_idx, void* code_data,
                            const int32_t* code_page_table, int64_t seq_len, const int32_t* seq_len_dev,
                            int num_heads, int q_heads, int head_dim, int page_size, int dtype, int budget,
                            void* dist_scratch,
                            int64_t dist_stride, uint32_t* hist, int32_t* out_idx, int64_t out_stride,
                            float hadamard_scale, const float* thresholds3_host, const RopeSpec& rope,
                            float sm_scale, adamas_stream_t stream, const SeqDesc* seqs = nullptr, int batch = 1) {
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  if (int rc = check_q_heads(num_heads, q_heads)) return rc;
  ADAMAS_REQUIRE(seqs || (kv_page_table && code_page_table), "page table missing");
  ADAMAS_REQUIRE(!seqs || (seq_len_dev && batch >= 1 && batch <= 1024), "a batched step needs device lengths");
  if (!seqs) batch = 1;
  ADAMAS_REQUIRE(budget >= 2 && seq_len > budget,
                 "a decode step needs budget >= 2 and a context longer than the budget (%lld vs %d); "
                 "shorter contexts attend to every page through adamas_decode_forward",
                 static_cast<long long>(seq_len), budget);
  ADAMAS_REQUIRE(seq_len - 1 < (int64_t(1) << 31) - kEstTile * kEstConsumerWarps * 2, "sequence too long");
  ADAMAS_REQUIRE(q && o && dist_scratch && q_code && hist, "null pointer");
  ADAMAS_REQUIRE((reinterpret_cast<uintptr_t>(dist_scratch) & 15) == 0 && (dist_stride * 2) % 16 == 0,
                 "distance rows must start on 16-byte boundaries");
  ADAMAS_REQUIRE(out_idx == nullptr || out_stride >= budget - 1 || q_heads * batch == 1, "out_stride smaller than budget - 1");
  const int n = static_cast<int>(seq_len - 1);
  const int pages = static_cast<int>((seq_len + page_size - 1) / page_size);
  const int last_len = static_cast<int>(seq_len - static_cast<int64_t>(pages - 1) * page_size);
  const DeviceInfo* di = nullptr;
  if (int rc = get_device_info(&di)) return rc;
  SaPlan pl;
  if (int rc = sa_plan(n, budget - 1, q_heads * batch, di, &pl)) return rc;
  int rc;
  // The histogram counts: one L2 atomic per distance from inside the estimate, or, for launches with 3 M
  // distances and more (a 128K context of 32 heads, three 32K sequences), a launch of their own that
  // counts in shared memory (measured: the estimate of one 128K sequence 31.7 us with the counts, 23.7
  // without).  Few heads per GPU keep the counts inside (the extra launch costs more than it saves).
  const bool count_apart = static_cast<int64_t>(q_heads) * batch * n >= (int64_t(3) << 20) && q_heads >= 16;
  uint32_t* est_hist = count_apart ? nullptr : hist;
  const bool two_launches = fused_append_enabled() && q_heads == num_heads &&
                            (num_heads == 16 || num_heads == 32 || num_heads == 64);
  if (two_launches) {
    // two launches: the estimate with the append (and, with RoPE, the rotation) inside, then select + attend
    rc = estimate_append_launch(q, k, v, q_code, kv_data, kv_page_table, pages, last_len, code_data,
                                code_page_table, pages, last_len, n, num_heads, page_size, dtype, dist_scratch,
                                dist_stride, hadamard_scale, thresholds3_host, seq_len_dev, est_hist, pl.cl, stream, seqs,
                                batch, rope);
    if (rc) return rc;
  } else {
    rc = append_decode_impl(k, v, q, k, true, q_code, kv_data, kv_page_table, pages, last_len, code_data,
                            code_page_table, pages, last_len, num_heads, head_dim, page_size, hadamard_scale,
                            thresholds3_host, dtype, stream, rope, seq_len_dev, q_heads, seqs, batch);
    if (rc) return rc;
    rc = estimate_impl(q_code, code_data, code_page_table, n, page_size, num_heads, q_heads, dist_scratch,
                       dist_stride, ADAMAS_VAL_U16, ADAMAS_METRIC_L1, seq_len_dev, est_hist, pl.cl, stream, seqs, batch);
    if (rc) return rc;
  }
  if (count_apart) {
    DistHistogramParams hp;
    hp.dist = static_cast<const uint16_t*>(dist_scratch);
    hp.dist_stride = dist_stride;
    hp.hist = hist;
    hp.n = n;
    hp.cl = pl.cl;
    hp.seq_len_dev = seq_len_dev;
    ADAMAS_LAUNCH("dist_histogram_kernel", dist_histogram_kernel, dim3(pl.cl, q_heads, batch), dim3(kSaThreads), 0,
                  to_stream(stream), 1, hp);
    if (int rc2 = check_launch("dist_histogram_kernel")) return rc2;
  }
  const int64_t tail = static_cast<int64_t>(kv_last_page_idx) * page_size + last_len - 1;
  rc = select_attend_impl(dist_scratch, dist_stride, n, budget - 1, q, o, nullptr, lse, kv_data, kv_page_table,
                          page_size, num_heads, q_heads, dtype, seq_len_dev ? 2 : 1, static_cast<unsigned>(tail), hist, nullptr,
                          seq_len_dev, out_idx, out_stride, sm_scale, pl, stream, seqs, batch,
                          two_launches ? &rope : nullptr);   // (after a separate append q is rotated already)
  if (rc) {
    // the estimate has filled the histogram table and nothing will clear it: restore the all-zero state
    cudaMemsetAsync(hist, 0, hist_bytes(q_heads * batch), to_stream(stream));
  }
  return rc;
}

static RopeSpec rope_from_args(float rope_scale, float rope_theta, const float* rope_inv_freq, float rope_mscale) {
  RopeSpec rope;
  if (rope_inv_freq) {
    rope.on = true;
    rope.inv_freq = rope_inv_freq;
    rope.mscale = rope_mscale;
  } else if (rope_scale > 0.f) {
    rope = linear_rope(rope_scale, rope_theta);
  }
  return rope;
}

int adamas_decode_step(void* q, void* k, const void* v, void* o, float* lse, void* q_code,
                       void* kv_data, const int32_t* kv_page_table, int kv_num_pages,
                       int kv_last_page_len, int kv_last_page_idx, void* code_data,
                       const int32_t* code_page_table, int code_num_pages, int code_last_page_len,
                       int num_heads, int num_q_heads, int head_dim, int page_size, int dtype, int budget,
                       void* dist_scratch, int64_t dist_stride, uint32_t* hist_scratch, int32_t* out_idx,
                       int64_t out_stride, float hadamard_scale, const float* thresholds3_host,
                       float rope_scale, float rope_theta, const float* rope_inv_freq, float rope_mscale,
                       float sm_scale, adamas_stream_t stream) {
  ADAMAS_REQUIRE(kv_num_pages >= 1 && code_num_pages >= 1, "page tables must not be empty");
  ADAMAS_REQUIRE(page_size >= 1, "page_size must be >= 1");
  ADAMAS_REQUIRE(kv_last_page_len >= 1 && kv_last_page_len <= page_size, "kv_last_page_len out of range");
  ADAMAS_REQUIRE(kv_num_pages == code_num_pages && kv_last_page_len == code_last_page_len,
                 "the KV cache and the code cache must hold the same number of tokens");
  ADAMAS_REQUIRE(kv_last_page_idx >= 0, "kv_last_page_idx must be >= 0");
  const int64_t seq_len = static_cast<int64_t>(kv_num_pages - 1) * page_size + kv_last_page_len;
  const RopeSpec rope = rope_from_args(rope_scale, rope_theta, rope_inv_freq, rope_mscale);
  return decode_step_impl(q, k, v, o, lse, q_code, kv_data, kv_page_table, kv_last_page_idx, code_data,
                          code_page_table, seq_len, nullptr, num_heads, num_q_heads, head_dim, page_size, dtype, budget,
                          dist_scratch, dist_stride, hist_scratch, out_idx, out_stride, hadamard_scale,
                          thresholds3_host, rope, sm_scale, stream);
}

int adamas_decode_step_dev(void* q, void* k, const void* v, void* o, float* lse, void* q_code, void* kv_data,
                           const int32_t* kv_page_table, void* code_data, const int32_t* code_page_table,
                           const int32_t* seq_len_dev, int max_seq_len, int num_heads, int num_q_heads,
                           int head_dim, int page_size, int dtype, int budget, void* dist_scratch, int64_t dist_stride,
                           uint32_t* hist_scratch, int32_t* out_idx, int64_t out_stride, float hadamard_scale,
                           const float* thresholds3_host, float rope_scale, float rope_theta,
                           const float* rope_inv_freq, float rope_mscale, float sm_scale,
                           adamas_stream_t stream) {
  ADAMAS_REQUIRE(seq_len_dev, "null pointer");
  ADAMAS_REQUIRE(page_size >= 1 && max_seq_len >= 1, "page_size and max_seq_len must be >= 1");
  return decode_step_impl(q, k, v, o, lse, q_code, kv_data, kv_page_table, 0, code_data, code_page_table,
                          max_seq_len, seq_len_dev, num_heads, num_q_heads, head_dim, page_size, dtype, budget, dist_scratch,
                          dist_stride, hist_scratch, out_idx, out_stride, hadamard_scale, thresholds3_host,
                          rope_from_args(rope_scale, rope_theta, rope_inv_freq, rope_mscale), sm_scale, stream);
}

int adamas_dense_step_dev(adamas_decode_handler_t* handler, void* q, void* k, const void* v, void* o, float* lse,
                          void* q_code, void* kv_data, const int32_t* kv_page_table, void* code_data,
                          const int32_t* code_page_table, const int32_t* seq_len_dev, int max_seq_len,
                          int num_heads, int num_q_heads, int head_dim, int page_size, int dtype,
                          float hadamard_scale, const float* thresholds3_host, float rope_scale, float rope_theta,
                          const float* rope_inv_freq, float rope_mscale, float sm_scale,
                          adamas_stream_t stream) {
  ADAMAS_REQUIRE(handler && seq_len_dev, "null pointer");
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  ADAMAS_REQUIRE(max_seq_len >= 1, "max_seq_len must be >= 1");
  ADAMAS_REQUIRE(q && k && v && o && q_code, "null pointer");
  if (!handler->forward_started)
    return fail(ADAMAS_ERR_STATE, "dense step called before begin_forward");
  ADAMAS_REQUIRE(handler->kv_heads == num_heads && handler->num_heads == num_q_heads &&
                     handler->page_size == page_size && handler->dtype == dtype,
                 "the handler was planned for another cache geometry");
  const int pages = (max_seq_len + page_size - 1) / page_size;
  const int last_len = max_seq_len - (pages - 1) * page_size;
  if (int rc = append_decode_impl(k, v, q, k, true, q_code, kv_data, kv_page_table, pages, last_len, code_data,
                                  code_page_table, pages, last_len, num_heads, head_dim, page_size, hadamard_scale,
                                  thresholds3_host, dtype, stream,
                                  rope_from_args(rope_scale, rope_theta, rope_inv_freq, rope_mscale), seq_len_dev,
                                  num_q_heads))
    return rc;
  return decode_forward_impl(handler, q, o, nullptr, lse, kv_data, kv_page_table, 0, pages - 1, page_size, 0,
                             last_len, last_len, sm_scale, stream, seq_len_dev);
}

static_assert(sizeof(adamas_seq_desc_t) == sizeof(SeqDesc) && offsetof(adamas_seq_desc_t, code_page_table) == offsetof(SeqDesc, code_table),
              "sequence descriptor layout");

int adamas_decode_step_batch_dev(void* q, void* k, const void* v, void* o, float* lse, void* q_code,
                                 const adamas_seq_desc_t* seqs_dev, const int32_t* seq_lens_dev, int batch,
                                 int max_seq_len, int num_heads, int num_q_heads, int head_dim, int page_size,
                                 int dtype, int budget, void* dist_scratch, int64_t dist_stride,
                                 uint32_t* hist_scratch, int32_t* out_idx, int64_t out_stride, float hadamard_scale,
                                 const float* thresholds3_host, float rope_scale, float rope_theta,
                                 const float* rope_inv_freq, float rope_mscale, float sm_scale,
                                 adamas_stream_t stream) {
  ADAMAS_REQUIRE(seqs_dev && seq_lens_dev, "null pointer");
  ADAMAS_REQUIRE(batch >= 1 && batch <= 1024, "batch out of range (%d)", batch);
  ADAMAS_REQUIRE(page_size >= 1 && max_seq_len >= 1, "page_size and max_seq_len must be >= 1");
  return decode_step_impl(q, k, v, o, lse, q_code, nullptr, nullptr, 0, nullptr, nullptr, max_seq_len, seq_lens_dev,
                          num_heads, num_q_heads, head_dim, page_size, dtype, budget, dist_scratch, dist_stride,
                          hist_scratch, out_idx, out_stride, hadamard_scale, thresholds3_host,
                          rope_from_args(rope_scale, rope_theta, rope_inv_freq, rope_mscale), sm_scale, stream,
                          reinterpret_cast<const SeqDesc*>(seqs_dev), batch);
}

int adamas_dense_step_batch_dev(adamas_decode_handler_t* handler, void* q, void* k, const void* v, void* o,
                                float* lse, void* q_code, const adamas_seq_desc_t* seqs_dev,
                                const int32_t* seq_lens_dev, int batch, int max_seq_len, int num_heads,
                                int num_q_heads, int head_dim, int page_size, int dtype, float hadamard_scale,
                                const float* thresholds3_host, float rope_scale, float rope_theta,
                                const float* rope_inv_freq, float rope_mscale, float sm_scale,
                                adamas_stream_t stream) {
  ADAMAS_REQUIRE(handler && seqs_dev && seq_lens_dev, "null pointer");
  if (int rc = check_common(num_heads, head_dim, page_size, dtype)) return rc;
  ADAMAS_REQUIRE(max_seq_len >= 1, "max_seq_len must be >= 1");
  ADAMAS_REQUIRE(q && k && v && o && q_code, "null pointer");
  if (!handler->forward_started)
    return fail(ADAMAS_ERR_STATE, "dense step called before begin_forward");
  ADAMAS_REQUIRE(handler->kv_heads == num_heads && handler->num_heads == num_q_heads &&
                     handler->page_size == page_size && handler->dtype == dtype,
                 "the handler was planned for another cache geometry");
  const SeqDesc* seqs = reinterpret_cast<const SeqDesc*>(seqs_dev);
  const int pages = (max_seq_len + page_size - 1) / page_size;
  const int last_len = max_seq_len - (pages - 1) * page_size;
  if (int rc = append_decode_impl(k, v, q, k, true, q_code, nullptr, nullptr, pages, last_len, nullptr, nullptr, pages,
                                  last_len, num_heads, head_dim, page_size, hadamard_scale, thresholds3_host, dtype,
                                  stream, rope_from_args(rope_scale, rope_theta, rope_inv_freq, rope_mscale),
                                  seq_lens_dev, num_q_heads, seqs, batch))
    return rc;
  return decode_forward_impl(handler, q, o, nullptr, lse, nullptr, nullptr, 0, pages - 1, page_size, 0, last_len,
                             last_len, sm_scale, stream, seq_lens_dev, seqs, batch);
}

int adamas_apply_rope_table_in_place(void* q, void* k, int64_t seq_len, int num_q_heads, int num_kv_heads,
                                     int head_dim, int64_t past_kv_len, const float* inv_freq_dev, float mscale,
                                     int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(head_dim == kHeadDim, "head_dim must be 128 (got %d)", head_dim);
  ADAMAS_REQUIRE(dtype == ADAMAS_F16 || dtype == ADAMAS_BF16, "unsupported dtype %d", dtype);
  ADAMAS_REQUIRE(seq_len >= 0 && num_q_heads >= 1 && num_kv_heads >= 1, "bad shape");
  ADAMAS_REQUIRE(past_kv_len >= 0 && past_kv_len + seq_len < (int64_t(1) << 24),
                 "positions must stay below 2^24 (exact in fp32)");
  if (seq_len == 0) return ADAMAS_OK;
  ADAMAS_REQUIRE(q && k && inv_freq_dev, "null pointer");
  const int64_t rows_q = seq_len * num_q_heads, rows_k = seq_len * num_kv_heads;
  const unsigned blocks = rows_to_blocks(rows_q + rows_k);
  const RopeParams rp{1.f, 1e4f, inv_freq_dev, mscale};
  if (dtype == ADAMAS_F16)
    rope_kernel<__half><<<blocks, 256, 0, to_stream(stream)>>>(static_cast<__half*>(q), static_cast<__half*>(k),
                                                              rows_q, rows_k, num_q_heads, num_kv_heads,
                                                              static_cast<int>(past_kv_len), rp);
  else
    rope_kernel<__nv_bfloat16><<<blocks, 256, 0, to_stream(stream)>>>(
        static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), rows_q, rows_k, num_q_heads,
        num_kv_heads, static_cast<int>(past_kv_len), rp);
  return check_launch("rope_kernel");
}

int adamas_merge_states(const float* o_parts, const float* lse_parts, int num_parts, int num_heads,
                        int head_dim, void* o, float* lse, int dtype, adamas_stream_t stream) {
  ADAMAS_REQUIRE(head_dim == kHeadDim, "head_dim must be 128 (got %d)", head_dim);
  ADAMAS_REQUIRE(dtype == ADAMAS_F16 || dtype == ADAMAS_BF16, "unsupported dtype %d", dtype);
  ADAMAS_REQUIRE(num_parts >= 1 && num_heads >= 1, "num_parts and num_heads must be >= 1");
  ADAMAS_REQUIRE(o_parts && lse_parts && o, "null pointer");
  if (dtype == ADAMAS_F16)
    merge_states_kernel<__half><<<num_heads, kHeadDim, 0, to_stream(stream)>>>(
        o_parts, lse_parts, num_parts, num_heads, static_cast<__half*>(o), lse);
  else
    merge_states_kernel<__nv_bfloat16><<<num_heads, kHeadDim, 0, to_stream(stream)>>>(
        o_parts, lse_parts, num_parts, num_heads, static_cast<__nv_bfloat16*>(o), lse);
  return check_launch("merge_states_kernel");
}

}  // extern "C"
