// C-ABI entry points (see include/fal_b200.h): argument validation, TMA
// descriptor construction and kernel launches.  This file is the counterpart
// of the reference's csrc/flash_attn_legacy.cpp, minus everything torch.
#include "../../include/fal_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "fal_common.h"
#include "fal_launch.h"

namespace {

thread_local int g_last_cuda_error = 0;

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return FAL_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Driver entry point for tensor-map encoding, fetched through the runtime so
// that the library has no link-time dependency on libcuda.
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

// fp16 tensor addressed as [batch, head, row, head_dim]; box = 64 x box_rows x 1 x 1,
// 128-byte swizzle, out-of-range elements read as zero.
int make_tensor_map(CUtensorMap* map, const void* base, int head_dim, int64_t rows, int64_t heads,
                    int64_t batch, const fal::RowStrides& st, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return FAL_ERR_TENSOR_MAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return FAL_ERR_INVALID_ARGUMENT;
  // Degenerate dimensions: the driver wants non-zero extents and 16-byte-multiple strides.
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim),
                              static_cast<cuuint64_t>(rows > 0 ? rows : 1),
                              static_cast<cuuint64_t>(heads > 0 ? heads : 1),
                              static_cast<cuuint64_t>(batch > 0 ? batch : 1)};
  // A dimension of extent <= 1 is never stepped along: any valid stride will do.  A longer one needs
  // a positive stride (a broadcast view, stride 0, cannot be described to the TMA unit).
  if ((rows > 1 && st.row <= 0) || (heads > 1 && st.head <= 0) || (batch > 1 && st.batch <= 0))
    return FAL_ERR_INVALID_ARGUMENT;
  auto fix = [&](int64_t s) -> cuuint64_t {
    if (s <= 0) s = head_dim;
    return static_cast<cuuint64_t>(s) * 2u;
  };
  const cuuint64_t strides[3] = {fix(st.row), fix(st.head), fix(st.batch)};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16u != 0) return FAL_ERR_INVALID_ARGUMENT;
  const cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(box_rows), 1u, 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = 100000 + static_cast<int>(r);  // driver (CUresult) codes are offset by 100000
    return FAL_ERR_TENSOR_MAP;
  }
  return FAL_OK;
}

// fp32 dQ accumulator addressed as [batch, head, row, head_dim] through strides in floats (rows of
// head_dim contiguous floats); box = 32 floats x 128 rows, 128-byte swizzle: the shape of one dQ
// staging box of the backward kernel.  `rows` is the extent reductions are clipped to.
int make_accum_tensor_map(CUtensorMap* map, const float* base, int head_dim, int64_t rows, int64_t heads,
                          int64_t batch, const fal::RowStrides& st) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return FAL_ERR_TENSOR_MAP;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return FAL_ERR_INVALID_ARGUMENT;
  if ((rows > 1 && st.row <= 0) || (heads > 1 && st.head <= 0) || (batch > 1 && st.batch <= 0))
    return FAL_ERR_INVALID_ARGUMENT;
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  auto fix = [&](int64_t s) -> cuuint64_t { return static_cast<cuuint64_t>(s > 0 ? s : head_dim) * 4u; };
  const cuuint64_t strides[3] = {fix(st.row), fix(st.head), fix(st.batch)};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16u != 0) return FAL_ERR_INVALID_ARGUMENT;
  const cuuint32_t box[4] = {32u, 128u, 1u, 1u};
  const cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = 100000 + static_cast<int>(r);
    return FAL_ERR_TENSOR_MAP;
  }
  return FAL_OK;
}

fal::RowStrides to_rs(const fal_strides* s) { return fal::RowStrides{s->batch, s->head, s->row}; }

int check_device() {
  static std::mutex mu;
  static int cached[64] = {};  // 0 unknown, 1 ok, -1 unsupported
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return FAL_ERR_UNSUPPORTED_DEVICE;
  // A host thread that has made no CUDA call yet (an autograd worker, say) has no context bound,
  // and the driver's tensor-map encoder refuses to run without one.  Re-selecting the current
  // device binds the primary context to this thread; it changes nothing else.
  thread_local int bound_device = -1;
  if (bound_device != dev) {
    e = cudaSetDevice(dev);
    if (e != cudaSuccess) return cuda_fail(e);
    bound_device = dev;
  }
  std::lock_guard<std::mutex> g(mu);
  if (cached[dev] == 0) {
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    cached[dev] = (major == 10) ? 1 : -1;
  }
  return cached[dev] == 1 ? FAL_OK : FAL_ERR_UNSUPPORTED_DEVICE;
}

// 32, 64, 96, 128 and 256 in every entry point.  64, 128 and 256 have kernels of their own (the
// head_dim-256 backward runs on column halves); 32 and 96 run on the 64 / 128 kernels: the TMA
// descriptors carry the real width, so the missing columns arrive as zeros (they add 0 to every
// score), and the kernels do not write output columns the tensors do not have.
bool head_dim_ok(int d) { return d == 32 || d == 64 || d == 96 || d == 128 || d == 256; }
int kernel_head_dim(int d) { return d == 32 ? 64 : (d == 96 ? 128 : d); }
// Number of SMs of the current device (cached per device; 0 if it cannot be read).
int sm_count() {
  static std::mutex mu;
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> g(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) cached[dev] = n;
  }
  return cached[dev];
}

// Forward kernel variant.  Two 128-row tiles per CTA let one tile's softmax run under the other's
// MMAs and fetch every K / V tile once for 256 query rows; a CTA of one tile (the softmax warpgroups
// take alternate key tiles of it) takes about 0.6 of the time of a two-tile CTA, measured on grids of
// many waves.  One tile per CTA is chosen where its larger number of shorter waves finishes first:
// grids that leave SMs without a two-tile CTA, or that end in a mostly empty wave.
std::atomic<int> g_fwd_variant{FAL_FWD_AUTO};  // fal_set_fwd_variant

int forward_cta_rows(int head_dim, int64_t blocks_of_256_rows, int64_t units) {
  const int forced = g_fwd_variant.load(std::memory_order_relaxed);
  bool one_tile = forced == FAL_FWD_ONE_TILE;
  if (forced == FAL_FWD_AUTO) {
    const int64_t sms = sm_count() > 0 ? sm_count() : 148;
    const int64_t ctas2 = blocks_of_256_rows * units;
    const int64_t waves2 = (ctas2 + sms - 1) / sms;
    const int64_t waves1 = (2 * ctas2 + sms - 1) / sms;
    one_tile = 6 * waves1 < 10 * waves2;
  }
  return fal::fwd_cta_rows(head_dim, one_tile);
}

int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// Backward scratch layout: [dq_accum fp32 batch*heads*padded_rows*d][delta fp32 batch*heads*padded_rows]
struct BwdWorkspace {
  int64_t padded_rows;
  size_t dq_bytes;
  size_t delta_bytes;
  size_t total() const { return dq_bytes + delta_bytes; }
};

BwdWorkspace bwd_workspace_layout(int batch, int heads_q, int rows, int head_dim) {
  head_dim = kernel_head_dim(head_dim);
  BwdWorkspace w;
  // One extra 128-row tile of slack: packed sequences start at arbitrary rows, and a tile's
  // reduction may touch (with zeros) up to 127 rows past the last query.
  w.padded_rows = round_up(rows, 128) + 128;
  w.dq_bytes = static_cast<size_t>(batch) * heads_q * w.padded_rows * head_dim * sizeof(float);
  w.delta_bytes = round_up(static_cast<int64_t>(batch) * heads_q * w.padded_rows * sizeof(float), 256);
  return w;
}

// Cache positions one split-K CTA streams.  1 024 keeps a small batch's CTAs fine-grained (8 entries:
// 0.081 ms per step against 0.089 with 2 048 or with 512); once the batch alone fills the GPU many
// times over, 2 048 halves the partials and the combine work (64 entries of up to 32 768 positions:
// 0.714 against 0.745 ms per step).
constexpr int kDecodeSplitLen = 1024;
int decode_split_len(int batch, int capacity) {
  const int64_t long_splits = static_cast<int64_t>(batch) * ((capacity + 2 * kDecodeSplitLen - 1) / (2 * kDecodeSplitLen));
  return long_splits >= 192 ? 2 * kDecodeSplitLen : kDecodeSplitLen;
}

// Decode scratch layout: [partial O fp32 rows*d][partial (max, sum) fp32 rows*2], rows =
// batch*heads_q*splits.  Nothing in it needs initialising.  (Sized for the shorter split length
// whichever is used, so the size a caller was told does not depend on the choice.)
struct DecodeWorkspace {
  int64_t splits;
  int split_len;
  size_t partial_bytes;
  size_t total() const { return partial_bytes; }
};

DecodeWorkspace decode_workspace_layout(int batch, int heads_q, int capacity, int head_dim) {
  head_dim = kernel_head_dim(head_dim);
  DecodeWorkspace w;
  w.split_len = decode_split_len(batch, capacity);
  w.splits = (capacity + w.split_len - 1) / w.split_len;
  const int64_t max_splits = (capacity + kDecodeSplitLen - 1) / kDecodeSplitLen;
  const int64_t rows = static_cast<int64_t>(batch) * heads_q * max_splits;
  w.partial_bytes = static_cast<size_t>(rows) * (head_dim + 2) * sizeof(float);
  return w;
}

// ---------------------------------------------------------------------------
// Optional event timing around the main kernels (off by default).
// ---------------------------------------------------------------------------
struct KernelTimer {
  static constexpr int kKinds = 3;
  static constexpr int kMaxRecords = 8192;
  std::mutex mu;
  bool enabled = false;
  struct Rec { cudaEvent_t a, b; };
  std::vector<Rec> recs[kKinds];

  // Returns the index of a new record with its start event recorded, or -1.
  int begin(int kind, cudaStream_t st) {
    std::lock_guard<std::mutex> g(mu);
    if (!enabled || static_cast<int>(recs[kind].size()) >= kMaxRecords) return -1;
    Rec r;
    if (cudaEventCreate(&r.a) != cudaSuccess) return -1;
    if (cudaEventCreate(&r.b) != cudaSuccess) { cudaEventDestroy(r.a); return -1; }
    cudaEventRecord(r.a, st);
    recs[kind].push_back(r);
    return static_cast<int>(recs[kind].size()) - 1;
  }
  void end(int kind, int idx, cudaStream_t st) {
    if (idx < 0) return;
    std::lock_guard<std::mutex> g(mu);
    if (idx < static_cast<int>(recs[kind].size())) cudaEventRecord(recs[kind][idx].b, st);
  }
};
KernelTimer g_timer;


}  // namespace

extern "C" {

const char* fal_strerror(int code) {
  switch (code) {
    case FAL_OK: return "ok";
    case FAL_ERR_INVALID_ARGUMENT: return "invalid argument (shape, stride, alignment or null pointer)";
    case FAL_ERR_UNSUPPORTED_HEAD_DIM: return "unsupported head_dim (32, 64, 96, 128 and 256 are built)";
    case FAL_ERR_WORKSPACE_TOO_SMALL: return "workspace too small";
    case FAL_ERR_CUDA: return "CUDA runtime error";
    case FAL_ERR_TENSOR_MAP: return "TMA descriptor could not be built";
    case FAL_ERR_UNSUPPORTED_DEVICE: return "device is not compute capability 10.x (B200)";
    case FAL_ERR_STATIC_SCRATCH_EXCEEDED:
      return "problem too large for fal_decode_static's fixed 8 MiB scratch "
             "(fal_decode_workspace_bytes(batch, heads_q, capacity, head_dim) must fit); use fal_decode";
    default: return "unknown error";
  }
}

int fal_last_cuda_error(void) { return g_last_cuda_error; }

const char* fal_version(void) { return "0.1.0"; }

namespace {

// The batched forward; `seqused_k` (device, one int per batch entry, or null) limits every entry to
// its own number of keys, seqlen_k then being the capacity the tensors are laid out for.
int fwd_batched(const void* q, const void* k, const void* v, void* o, float* lse,
                const int32_t* seqused_k, int batch, int heads_q, int heads_kv, int seqlen_q,
                int seqlen_k, int head_dim, const fal_strides* q_strides,
                const fal_strides* k_strides, const fal_strides* v_strides,
                const fal_strides* o_strides, float softmax_scale, int is_causal, int* status,
                void* stream) {
  if (!q || !k || !v || !o || !lse || !q_strides || !k_strides || !v_strides || !o_strides)
    return FAL_ERR_INVALID_ARGUMENT;
  if (batch <= 0 || heads_q <= 0 || heads_kv <= 0 || seqlen_q <= 0 || seqlen_k < 0)
    return FAL_ERR_INVALID_ARGUMENT;
  if (heads_q % heads_kv != 0 || !(softmax_scale > 0.f)) return FAL_ERR_INVALID_ARGUMENT;
  // The bottom-right-aligned mask is defined here for a query block that ends where the keys end
  // (with a length per entry, an entry shorter than the block leaves its first queries without keys).
  if (is_causal < 0 || is_causal > FAL_CAUSAL_BOTTOM_RIGHT) return FAL_ERR_INVALID_ARGUMENT;
  if (is_causal == FAL_CAUSAL_BOTTOM_RIGHT && seqused_k == nullptr && seqlen_k < seqlen_q)
    return FAL_ERR_INVALID_ARGUMENT;
  if (!head_dim_ok(head_dim)) return FAL_ERR_UNSUPPORTED_HEAD_DIM;
  if ((reinterpret_cast<uintptr_t>(o) & 15u) != 0 || o_strides->row % 8 != 0 ||
      o_strides->head % 8 != 0 || o_strides->batch % 8 != 0)
    return FAL_ERR_INVALID_ARGUMENT;
  int rc = check_device();
  if (rc != FAL_OK) return rc;

  CUtensorMap tq, tk, tv;
  if ((rc = make_tensor_map(&tq, q, head_dim, seqlen_q, heads_q, batch, to_rs(q_strides), 128)))
    return rc;
  if ((rc = make_tensor_map(&tk, k, head_dim, seqlen_k, heads_kv, batch, to_rs(k_strides), 128)))
    return rc;
  if ((rc = make_tensor_map(&tv, v, head_dim, seqlen_k, heads_kv, batch, to_rs(v_strides), 128)))
    return rc;

  // O leaves its CTA as whole tiles through TMA stores when its layout can be described to the TMA
  // unit (else row by row from registers).
  CUtensorMap to = tq;
  const bool o_by_tma = make_tensor_map(&to, o, head_dim, seqlen_q, heads_q, batch, to_rs(o_strides), 128) == FAL_OK;

  fal::FwdParams p{};
  p.store_by_tma = o_by_tma ? 1 : 0;
  p.o = o;
  p.lse = lse;
  p.o_strides = to_rs(o_strides);
  p.lse_strides = fal::RowStrides{static_cast<int64_t>(heads_q) * seqlen_q, seqlen_q, 1};
  p.cu_q = nullptr;
  p.cu_k = nullptr;
  p.num_seqs = 0;
  p.batch = batch;
  p.heads_q = heads_q;
  p.heads_kv = heads_kv;
  p.head_dim = head_dim;
  p.seqlen_q = seqlen_q;
  p.seqlen_k = seqlen_k;
  p.seqused_k = seqused_k;
  if (seqused_k == nullptr) p.causal_shift = is_causal == FAL_CAUSAL_BOTTOM_RIGHT ? seqlen_k - seqlen_q : 0;
  else p.shift_per_sequence = is_causal == FAL_CAUSAL_BOTTOM_RIGHT ? 1 : 0;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kdim = kernel_head_dim(head_dim);
  const int cta_rows = forward_cta_rows(kdim, (seqlen_q + 255) / 256, static_cast<int64_t>(batch) * heads_q);
  p.cta_rows = cta_rows;
  p.num_qblk = (seqlen_q + cta_rows - 1) / cta_rows;
  const int64_t grid = static_cast<int64_t>(p.num_qblk) * batch * heads_q;
  if (grid > 0x7fffffff) return FAL_ERR_INVALID_ARGUMENT;
  const int rec = g_timer.begin(FAL_KERNEL_FWD, st);
  cudaError_t e = fal::launch_fwd(kdim, is_causal != 0, tq, tk, tv, to, p, static_cast<int>(grid), st);
  g_timer.end(FAL_KERNEL_FWD, rec, st);
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

}  // namespace

int fal_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch,
            int heads_q, int heads_kv, int seqlen_q, int seqlen_k, int head_dim,
            const fal_strides* q_strides, const fal_strides* k_strides,
            const fal_strides* v_strides, const fal_strides* o_strides, float softmax_scale,
            int is_causal, int* status, void* stream) {
  return fwd_batched(q, k, v, o, lse, nullptr, batch, heads_q, heads_kv, seqlen_q, seqlen_k, head_dim,
                     q_strides, k_strides, v_strides, o_strides, softmax_scale, is_causal, status, stream);
}

int fal_fwd_kvcache(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                    const int32_t* cache_seqlens, int batch, int heads_q, int heads_kv, int seqlen_q,
                    int cache_capacity, int head_dim, const fal_strides* q_strides,
                    const fal_strides* k_strides, const fal_strides* v_strides,
                    const fal_strides* o_strides, float softmax_scale, int is_causal, int* status,
                    void* stream) {
  if (!cache_seqlens) return FAL_ERR_INVALID_ARGUMENT;
  return fwd_batched(q, k_cache, v_cache, o, lse, cache_seqlens, batch, heads_q, heads_kv, seqlen_q,
                     cache_capacity, head_dim, q_strides, k_strides, v_strides, o_strides,
                     softmax_scale, is_causal, status, stream);
}

int fal_fwd_varlen(const void* q, const void* k, const void* v, void* o, float* lse,
                   const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int num_seqs,
                   int total_q, int total_k, int max_seqlen_q, int max_seqlen_k, int heads_q,
                   int heads_kv, int head_dim, const fal_strides* q_strides,
                   const fal_strides* k_strides, const fal_strides* v_strides,
                   const fal_strides* o_strides, float softmax_scale, int is_causal, int* status,
                   void* stream) {
  (void)max_seqlen_q;
  (void)max_seqlen_k;
  if (!q || !k || !v || !o || !lse || !cu_seqlens_q || !cu_seqlens_k || !q_strides || !k_strides ||
      !v_strides || !o_strides)
    return FAL_ERR_INVALID_ARGUMENT;
  if (num_seqs <= 0 || total_q <= 0 || total_k < 0 || heads_q <= 0 || heads_kv <= 0)
    return FAL_ERR_INVALID_ARGUMENT;
  if (heads_q % heads_kv != 0 || !(softmax_scale > 0.f)) return FAL_ERR_INVALID_ARGUMENT;
  if (is_causal < 0 || is_causal > FAL_CAUSAL_BOTTOM_RIGHT) return FAL_ERR_INVALID_ARGUMENT;
  if (!head_dim_ok(head_dim)) return FAL_ERR_UNSUPPORTED_HEAD_DIM;
  if ((reinterpret_cast<uintptr_t>(o) & 15u) != 0 || o_strides->row % 8 != 0 ||
      o_strides->head % 8 != 0)
    return FAL_ERR_INVALID_ARGUMENT;
  int rc = check_device();
  if (rc != FAL_OK) return rc;

  CUtensorMap tq, tk, tv;
  fal::RowStrides qs = to_rs(q_strides), ks = to_rs(k_strides), vs = to_rs(v_strides);
  qs.batch = ks.batch = vs.batch = 0;
  if ((rc = make_tensor_map(&tq, q, head_dim, total_q, heads_q, 1, qs, 128))) return rc;
  if ((rc = make_tensor_map(&tk, k, head_dim, total_k, heads_kv, 1, ks, 128))) return rc;
  if ((rc = make_tensor_map(&tv, v, head_dim, total_k, heads_kv, 1, vs, 128))) return rc;

  fal::RowStrides os = to_rs(o_strides);
  os.batch = 0;
  CUtensorMap to = tq;
  const bool o_by_tma = make_tensor_map(&to, o, head_dim, total_q, heads_q, 1, os, 128) == FAL_OK;

  fal::FwdParams p{};
  p.store_by_tma = o_by_tma ? 1 : 0;
  p.o = o;
  p.lse = lse;
  p.o_strides = to_rs(o_strides);
  p.o_strides.batch = 0;
  p.lse_strides = fal::RowStrides{0, 1, heads_q};  // lse[token, head]
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.num_seqs = num_seqs;
  p.batch = 1;
  p.heads_q = heads_q;
  p.heads_kv = heads_kv;
  p.head_dim = head_dim;
  p.seqlen_q = 0;
  p.seqlen_k = 0;
  p.shift_per_sequence = is_causal == FAL_CAUSAL_BOTTOM_RIGHT ? 1 : 0;
  p.scale = softmax_scale;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The lengths stay on the device.  Every sequence rounds up to whole query blocks: at most one
  // extra block each.
  const int kdim = kernel_head_dim(head_dim);
  p.cta_rows = forward_cta_rows(kdim, total_q / 256 + num_seqs, heads_q);
  p.num_qblk = total_q / p.cta_rows + num_seqs;
  const int64_t grid = static_cast<int64_t>(p.num_qblk) * heads_q;
  if (grid > 0x7fffffff) return FAL_ERR_INVALID_ARGUMENT;
  const int rec = g_timer.begin(FAL_KERNEL_FWD, st);
  cudaError_t e = fal::launch_fwd(kdim, is_causal != 0, tq, tk, tv, to, p, static_cast<int>(grid), st);
  g_timer.end(FAL_KERNEL_FWD, rec, st);
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

size_t fal_bwd_workspace_bytes(int batch, int heads_q, int rows, int head_dim) {
  if (batch <= 0 || heads_q <= 0 || rows <= 0 || head_dim <= 0) return 0;
  return bwd_workspace_layout(batch, heads_q, rows, head_dim).total();
}

namespace {

// Shared tail of the batched and packed backward: pre-pass, main kernel, post-pass.
struct BwdCall {
  const void *d_out, *q, *k, *v, *o;
  const float* lse;
  void *dq, *dk, *dv;
  const int32_t *cu_q, *cu_k;
  int num_seqs;
  int batch, heads_q, heads_kv, rows_q, rows_k, head_dim;
  fal::RowStrides s_do, s_q, s_k, s_v, s_o, s_dq, s_dk, s_dv;
  fal::RowStrides s_lse;
  float scale;
  int causal;
  void* workspace;
  size_t workspace_bytes;
  int* status;
  cudaStream_t stream;
  // Partial mode (fal_bwd_partial): dQ is ADDED into the caller's fp32 accumulator (never zeroed, no
  // cast pass) and dK / dV leave as fp32; dq, dk, dv above are then unused.
  float* dq_acc = nullptr;
  float* dk_f32 = nullptr;
  float* dv_f32 = nullptr;
  fal::RowStrides s_dq_acc{};
};

int run_bwd(const BwdCall& c) {
  const bool partial = c.dq_acc != nullptr;
  if (!c.d_out || !c.q || !c.k || !c.v || !c.o || !c.lse || !c.workspace) return FAL_ERR_INVALID_ARGUMENT;
  if (partial ? (!c.dk_f32 || !c.dv_f32) : (!c.dq || !c.dk || !c.dv)) return FAL_ERR_INVALID_ARGUMENT;
  if (c.batch <= 0 || c.heads_q <= 0 || c.heads_kv <= 0 || c.rows_q <= 0 || c.rows_k <= 0)
    return FAL_ERR_INVALID_ARGUMENT;
  if (c.heads_q % c.heads_kv != 0 || !(c.scale > 0.f)) return FAL_ERR_INVALID_ARGUMENT;
  if (c.causal < 0 || c.causal > FAL_CAUSAL_BOTTOM_RIGHT) return FAL_ERR_INVALID_ARGUMENT;
  // the bottom-right-aligned mask is defined for a query block that ends where the keys end
  if (c.causal == FAL_CAUSAL_BOTTOM_RIGHT && c.cu_q == nullptr && c.rows_k < c.rows_q) return FAL_ERR_INVALID_ARGUMENT;
  if (!head_dim_ok(c.head_dim)) return FAL_ERR_UNSUPPORTED_HEAD_DIM;
  auto out_ok = [](const void* ptr, const fal::RowStrides& s) {
    return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && s.row % 8 == 0 && s.head % 8 == 0 &&
           s.batch % 8 == 0;
  };
  const int kdim = kernel_head_dim(c.head_dim);
  if (partial) {
    if (kdim != c.head_dim) return FAL_ERR_UNSUPPORTED_HEAD_DIM;  // fp32 partials: head_dim 64, 128, 256
    if (!out_ok(c.dk_f32, c.s_dk) || !out_ok(c.dv_f32, c.s_dv) || !out_ok(c.dq_acc, c.s_dq_acc) ||
        c.s_dq_acc.row != c.head_dim)
      return FAL_ERR_INVALID_ARGUMENT;
  } else if (!out_ok(c.dq, c.s_dq) || !out_ok(c.dk, c.s_dk) || !out_ok(c.dv, c.s_dv)) {
    return FAL_ERR_INVALID_ARGUMENT;
  }
  if (!out_ok(c.o, c.s_o) || !out_ok(c.d_out, c.s_do)) return FAL_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(c.workspace) & 255u) != 0) return FAL_ERR_INVALID_ARGUMENT;
  BwdWorkspace w = bwd_workspace_layout(c.batch, c.heads_q, c.rows_q, c.head_dim);
  if (partial) w.dq_bytes = 0;  // the accumulator is the caller's; the workspace holds delta only
  if (c.workspace_bytes < w.total()) return FAL_ERR_WORKSPACE_TOO_SMALL;
  int rc = check_device();
  if (rc != FAL_OK) return rc;

  float* dq_accum = partial ? c.dq_acc : static_cast<float*>(c.workspace);
  float* delta = reinterpret_cast<float*>(static_cast<char*>(c.workspace) + w.dq_bytes);
  const int64_t acc_head = partial ? c.s_dq_acc.head : w.padded_rows * kdim;
  const int64_t acc_batch = partial ? c.s_dq_acc.batch : acc_head * c.heads_q;
  const int64_t acc_rows = partial ? c.rows_q : w.padded_rows;

  CUtensorMap tq, tk, tv, tdo, tdq;
  if ((rc = make_tensor_map(&tq, c.q, c.head_dim, c.rows_q, c.heads_q, c.batch, c.s_q, 128))) return rc;
  if ((rc = make_tensor_map(&tdo, c.d_out, c.head_dim, c.rows_q, c.heads_q, c.batch, c.s_do, 128)))
    return rc;
  if ((rc = make_accum_tensor_map(&tdq, dq_accum, kdim, acc_rows, c.heads_q, c.batch,
                                  fal::RowStrides{acc_batch, acc_head, kdim})))
    return rc;
  if ((rc = make_tensor_map(&tk, c.k, c.head_dim, c.rows_k, c.heads_kv, c.batch, c.s_k, 128))) return rc;
  if ((rc = make_tensor_map(&tv, c.v, c.head_dim, c.rows_k, c.heads_kv, c.batch, c.s_v, 128))) return rc;
  // dK and dV leave their CTA as whole tiles through TMA stores when their layout can be described
  // to the TMA unit (else, and for the fp32 partials of a ring step, row by row from registers).
  CUtensorMap tdk = tk, tdv = tv;
  const bool store_by_tma = !partial &&
                            make_tensor_map(&tdk, c.dk, c.head_dim, c.rows_k, c.heads_kv, c.batch, c.s_dk, 128) == FAL_OK &&
                            make_tensor_map(&tdv, c.dv, c.head_dim, c.rows_k, c.heads_kv, c.batch, c.s_dv, 128) == FAL_OK;

  fal::BwdPrepParams pp{};
  pp.o = c.o;
  pp.d_o = c.d_out;
  pp.o_strides = c.s_o;
  pp.do_strides = c.s_do;
  pp.delta = delta;
  pp.delta_head_stride = w.padded_rows;
  pp.delta_batch_stride = w.padded_rows * c.heads_q;
  pp.dq_accum = partial ? nullptr : dq_accum;  // a caller-owned accumulator is continued, not cleared
  pp.dq_accum_head_stride = acc_head;
  pp.dq_accum_batch_stride = acc_batch;
  pp.batch = c.batch;
  pp.heads_q = c.heads_q;
  pp.rows = c.rows_q;
  pp.padded_rows = static_cast<int>(w.padded_rows);
  pp.head_dim = kdim;
  pp.head_dim_real = c.head_dim;
  cudaError_t e = fal::launch_bwd_prep(pp, c.stream);
  if (e != cudaSuccess) return cuda_fail(e);

  fal::BwdParams p{};
  p.dk = c.dk;
  p.dv = c.dv;
  p.dk_f32 = c.dk_f32;
  p.dv_f32 = c.dv_f32;
  p.store_by_tma = store_by_tma ? 1 : 0;
  p.dk_strides = c.s_dk;
  p.dv_strides = c.s_dv;
  p.dq_accum = dq_accum;
  p.dq_accum_head_stride = acc_head;
  p.dq_accum_batch_stride = acc_batch;
  p.lse = c.lse;
  p.lse_strides = c.s_lse;
  p.delta = delta;
  p.delta_head_stride = pp.delta_head_stride;
  p.delta_batch_stride = pp.delta_batch_stride;
  p.cu_q = c.cu_q;
  p.cu_k = c.cu_k;
  p.num_seqs = c.num_seqs;
  p.batch = c.batch;
  p.heads_q = c.heads_q;
  p.heads_kv = c.heads_kv;
  p.head_dim = c.head_dim;
  p.seqlen_q = c.cu_q ? 0 : c.rows_q;
  p.seqlen_k = c.cu_k ? 0 : c.rows_k;
  p.num_kvblk = c.cu_k ? (c.rows_k / 128 + c.num_seqs) : (c.rows_k + 127) / 128;
  p.causal_shift = (c.causal == FAL_CAUSAL_BOTTOM_RIGHT && !c.cu_k) ? c.rows_k - c.rows_q : 0;
  p.shift_per_sequence = (c.causal == FAL_CAUSAL_BOTTOM_RIGHT && c.cu_k) ? 1 : 0;
  p.scale = c.scale;
  p.scale_log2 = c.scale * 1.4426950408889634f;
  p.status = c.status;
  const int64_t grid = static_cast<int64_t>(p.num_kvblk) * c.batch * c.heads_kv;
  if (grid > 0x7fffffff) return FAL_ERR_INVALID_ARGUMENT;
  const int rec = g_timer.begin(FAL_KERNEL_BWD, c.stream);
  e = fal::launch_bwd(kdim, c.causal != 0, tq, tk, tv, tdo, tdq, tdk, tdv, p, static_cast<int>(grid),
                      c.stream);
  g_timer.end(FAL_KERNEL_BWD, rec, c.stream);
  if (e != cudaSuccess) return cuda_fail(e);
  if (partial) return FAL_OK;  // the caller casts its accumulator once, after the last partial call

  fal::BwdPostParams po{};
  po.dq_accum = dq_accum;
  po.dq_accum_head_stride = acc_head;
  po.dq_accum_batch_stride = acc_batch;
  po.dq = c.dq;
  po.dq_strides = c.s_dq;
  po.batch = c.batch;
  po.heads_q = c.heads_q;
  po.rows = c.rows_q;
  po.head_dim = kdim;
  po.head_dim_real = c.head_dim;
  po.scale = c.scale;
  e = fal::launch_bwd_post(po, c.stream);
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

}  // namespace

int fal_bwd(const void* d_out, const void* q, const void* k, const void* v, const void* o,
            const float* lse, void* dq, void* dk, void* dv, int batch, int heads_q, int heads_kv,
            int seqlen_q, int seqlen_k, int head_dim, const fal_strides* do_strides,
            const fal_strides* q_strides, const fal_strides* k_strides,
            const fal_strides* v_strides, const fal_strides* o_strides,
            const fal_strides* dq_strides, const fal_strides* dk_strides,
            const fal_strides* dv_strides, float softmax_scale, int is_causal, void* workspace,
            size_t workspace_bytes, int* status, void* stream) {
  if (!do_strides || !q_strides || !k_strides || !v_strides || !o_strides || !dq_strides ||
      !dk_strides || !dv_strides)
    return FAL_ERR_INVALID_ARGUMENT;
  BwdCall c{};
  c.d_out = d_out; c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse;
  c.dq = dq; c.dk = dk; c.dv = dv;
  c.cu_q = nullptr; c.cu_k = nullptr; c.num_seqs = 0;
  c.batch = batch; c.heads_q = heads_q; c.heads_kv = heads_kv;
  c.rows_q = seqlen_q; c.rows_k = seqlen_k; c.head_dim = head_dim;
  c.s_do = to_rs(do_strides); c.s_q = to_rs(q_strides); c.s_k = to_rs(k_strides);
  c.s_v = to_rs(v_strides); c.s_o = to_rs(o_strides); c.s_dq = to_rs(dq_strides);
  c.s_dk = to_rs(dk_strides); c.s_dv = to_rs(dv_strides);
  c.s_lse = fal::RowStrides{static_cast<int64_t>(heads_q) * seqlen_q, seqlen_q, 1};
  c.scale = softmax_scale; c.causal = is_causal;
  c.workspace = workspace; c.workspace_bytes = workspace_bytes;
  c.status = status; c.stream = static_cast<cudaStream_t>(stream);
  return run_bwd(c);
}

int fal_bwd_varlen(const void* d_out, const void* q, const void* k, const void* v, const void* o,
                   const float* lse, void* dq, void* dk, void* dv, const int32_t* cu_seqlens_q,
                   const int32_t* cu_seqlens_k, int num_seqs, int total_q, int total_k,
                   int max_seqlen_q, int max_seqlen_k, int heads_q, int heads_kv, int head_dim,
                   const fal_strides* do_strides, const fal_strides* q_strides,
                   const fal_strides* k_strides, const fal_strides* v_strides,
                   const fal_strides* o_strides, const fal_strides* dq_strides,
                   const fal_strides* dk_strides, const fal_strides* dv_strides,
                   float softmax_scale, int is_causal, void* workspace, size_t workspace_bytes,
                   int* status, void* stream) {
  (void)max_seqlen_q;
  (void)max_seqlen_k;
  if (!do_strides || !q_strides || !k_strides || !v_strides || !o_strides || !dq_strides ||
      !dk_strides || !dv_strides || !cu_seqlens_q || !cu_seqlens_k || num_seqs <= 0)
    return FAL_ERR_INVALID_ARGUMENT;
  BwdCall c{};
  c.d_out = d_out; c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse;
  c.dq = dq; c.dk = dk; c.dv = dv;
  c.cu_q = cu_seqlens_q; c.cu_k = cu_seqlens_k; c.num_seqs = num_seqs;
  c.batch = 1; c.heads_q = heads_q; c.heads_kv = heads_kv;
  c.rows_q = total_q; c.rows_k = total_k; c.head_dim = head_dim;
  auto packed = [](const fal_strides* s) { return fal::RowStrides{0, s->head, s->row}; };
  c.s_do = packed(do_strides); c.s_q = packed(q_strides); c.s_k = packed(k_strides);
  c.s_v = packed(v_strides); c.s_o = packed(o_strides); c.s_dq = packed(dq_strides);
  c.s_dk = packed(dk_strides); c.s_dv = packed(dv_strides);
  c.s_lse = fal::RowStrides{0, 1, heads_q};
  c.scale = softmax_scale; c.causal = is_causal;
  c.workspace = workspace; c.workspace_bytes = workspace_bytes;
  c.status = status; c.stream = static_cast<cudaStream_t>(stream);
  return run_bwd(c);
}

size_t fal_bwd_partial_workspace_bytes(int batch, int heads_q, int rows, int head_dim) {
  if (batch <= 0 || heads_q <= 0 || rows <= 0 || head_dim <= 0) return 0;
  return bwd_workspace_layout(batch, heads_q, rows, head_dim).delta_bytes;
}

int fal_bwd_partial(const void* d_out, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, float* dq_accum, float* dk_partial, float* dv_partial, int batch,
                    int heads_q, int heads_kv, int seqlen_q, int seqlen_k, int head_dim,
                    const fal_strides* do_strides, const fal_strides* q_strides, const fal_strides* k_strides,
                    const fal_strides* v_strides, const fal_strides* o_strides,
                    const fal_strides* dq_accum_strides, const fal_strides* dk_strides,
                    const fal_strides* dv_strides, const fal_strides* lse_strides, float softmax_scale,
                    int is_causal, void* workspace, size_t workspace_bytes, int* status, void* stream) {
  if (!do_strides || !q_strides || !k_strides || !v_strides || !o_strides || !dq_accum_strides ||
      !dk_strides || !dv_strides || !lse_strides || !dq_accum)
    return FAL_ERR_INVALID_ARGUMENT;
  BwdCall c{};
  c.d_out = d_out; c.q = q; c.k = k; c.v = v; c.o = o; c.lse = lse;
  c.dq = nullptr; c.dk = nullptr; c.dv = nullptr;
  c.dq_acc = dq_accum; c.dk_f32 = dk_partial; c.dv_f32 = dv_partial;
  c.cu_q = nullptr; c.cu_k = nullptr; c.num_seqs = 0;
  c.batch = batch; c.heads_q = heads_q; c.heads_kv = heads_kv;
  c.rows_q = seqlen_q; c.rows_k = seqlen_k; c.head_dim = head_dim;
  c.s_do = to_rs(do_strides); c.s_q = to_rs(q_strides); c.s_k = to_rs(k_strides);
  c.s_v = to_rs(v_strides); c.s_o = to_rs(o_strides); c.s_dq_acc = to_rs(dq_accum_strides);
  c.s_dk = to_rs(dk_strides); c.s_dv = to_rs(dv_strides);
  c.s_lse = to_rs(lse_strides);
  c.scale = softmax_scale; c.causal = is_causal;
  c.workspace = workspace; c.workspace_bytes = workspace_bytes;
  c.status = status; c.stream = static_cast<cudaStream_t>(stream);
  return run_bwd(c);
}

namespace {
bool elementwise_shape_ok(int batch, int heads, int rows, int head_dim) {
  return batch > 0 && heads > 0 && rows > 0 && head_dim > 0 && head_dim % 8 == 0 && head_dim <= 256;
}
// 16-byte accesses of 8 fp16 / 4 fp32 elements: base and every stride must keep that alignment.
bool vec_ok(const void* ptr, const fal_strides* s, int elem_bytes) {
  const int64_t per16 = 16 / elem_bytes;
  return ptr != nullptr && s != nullptr && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 &&
         s->row % per16 == 0 && s->head % per16 == 0 && s->batch % per16 == 0;
}
}  // namespace

int fal_merge_partial(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part, int batch,
                      int heads, int rows, int head_dim, const fal_strides* o_acc_strides,
                      const fal_strides* lse_acc_strides, const fal_strides* o_part_strides,
                      const fal_strides* lse_part_strides, int init, void* stream) {
  if (!elementwise_shape_ok(batch, heads, rows, head_dim) || !lse_acc || !lse_part || !lse_acc_strides ||
      !lse_part_strides || !vec_ok(o_acc, o_acc_strides, 4) || !vec_ok(o_part, o_part_strides, 2))
    return FAL_ERR_INVALID_ARGUMENT;
  int rc = check_device();
  if (rc != FAL_OK) return rc;
  fal::MergeParams p{};
  p.o_acc = o_acc; p.lse_acc = lse_acc; p.o_part = o_part; p.lse_part = lse_part;
  p.o_acc_strides = to_rs(o_acc_strides); p.lse_acc_strides = to_rs(lse_acc_strides);
  p.o_part_strides = to_rs(o_part_strides); p.lse_part_strides = to_rs(lse_part_strides);
  p.batch = batch; p.heads = heads; p.rows = rows; p.head_dim = head_dim; p.init = init != 0;
  cudaError_t e = fal::launch_merge_partial(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

int fal_accumulate_f32(float* dst, const float* src, int batch, int heads, int rows, int head_dim,
                       const fal_strides* dst_strides, const fal_strides* src_strides, void* stream) {
  if (!elementwise_shape_ok(batch, heads, rows, head_dim) || !vec_ok(dst, dst_strides, 4) ||
      !vec_ok(src, src_strides, 4))
    return FAL_ERR_INVALID_ARGUMENT;
  int rc = check_device();
  if (rc != FAL_OK) return rc;
  fal::AccumulateParams p{};
  p.dst = dst; p.src = src; p.dst_strides = to_rs(dst_strides); p.src_strides = to_rs(src_strides);
  p.batch = batch; p.heads = heads; p.rows = rows; p.head_dim = head_dim;
  cudaError_t e = fal::launch_accumulate(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

int fal_scale_cast_f16(void* dst, const float* src, int batch, int heads, int rows, int head_dim,
                       const fal_strides* dst_strides, const fal_strides* src_strides, float scale,
                       void* stream) {
  if (!elementwise_shape_ok(batch, heads, rows, head_dim) || !vec_ok(dst, dst_strides, 2) ||
      !vec_ok(src, src_strides, 4))
    return FAL_ERR_INVALID_ARGUMENT;
  int rc = check_device();
  if (rc != FAL_OK) return rc;
  fal::ScaleCastParams p{};
  p.dst = dst; p.src = src; p.dst_strides = to_rs(dst_strides); p.src_strides = to_rs(src_strides);
  p.batch = batch; p.heads = heads; p.rows = rows; p.head_dim = head_dim; p.scale = scale;
  cudaError_t e = fal::launch_scale_cast(p, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

size_t fal_decode_workspace_bytes(int batch, int heads_q, int capacity, int head_dim) {
  if (batch <= 0 || heads_q <= 0 || capacity <= 0 || head_dim <= 0) return 0;
  return decode_workspace_layout(batch, heads_q, capacity, head_dim).total();
}

namespace {
// Argument checks shared by every decode entry point (no CUDA call is made here).
int decode_check_args(const void* q, const void* k_cache, const void* v_cache, const fal_strides* k_strides,
                      const fal_strides* v_strides, const int32_t* cache_seqlens, const void* k_new,
                      const void* v_new, const void* o, int batch, int heads_q, int heads_kv, int capacity,
                      int head_dim, float softmax_scale) {
  if (!q || !k_cache || !v_cache || !k_strides || !v_strides || !cache_seqlens || !o)
    return FAL_ERR_INVALID_ARGUMENT;
  if ((k_new == nullptr) != (v_new == nullptr)) return FAL_ERR_INVALID_ARGUMENT;
  if (batch <= 0 || heads_q <= 0 || heads_kv <= 0 || capacity <= 0) return FAL_ERR_INVALID_ARGUMENT;
  if (heads_q % heads_kv != 0 || !(softmax_scale > 0.f)) return FAL_ERR_INVALID_ARGUMENT;
  if (!head_dim_ok(head_dim)) return FAL_ERR_UNSUPPORTED_HEAD_DIM;
  auto aligned16 = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(o) ||
      !aligned16(k_new) || !aligned16(v_new))
    return FAL_ERR_INVALID_ARGUMENT;
  const fal_strides* both[2] = {k_strides, v_strides};
  for (const fal_strides* s : both)
    if (s->row % 8 != 0 || s->head % 8 != 0 || s->batch % 8 != 0) return FAL_ERR_INVALID_ARGUMENT;
  return FAL_OK;
}

int decode_with_workspace(const void* q, void* k_cache, void* v_cache, const fal_strides* k_strides,
                          const fal_strides* v_strides, const int32_t* cache_starts,
                          const int32_t* cache_seqlens, const void* k_new, const void* v_new, void* o,
                          float* lse, int batch, int heads_q, int heads_kv, int capacity, int head_dim,
                          float softmax_scale, void* workspace, size_t workspace_bytes, int* status,
                          void* stream) {
  int rc = decode_check_args(q, k_cache, v_cache, k_strides, v_strides, cache_seqlens, k_new, v_new, o, batch,
                             heads_q, heads_kv, capacity, head_dim, softmax_scale);
  if (rc != FAL_OK) return rc;
  if (!workspace) return FAL_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return FAL_ERR_INVALID_ARGUMENT;
  const DecodeWorkspace w = decode_workspace_layout(batch, heads_q, capacity, head_dim);
  if (workspace_bytes < w.total()) return FAL_ERR_WORKSPACE_TOO_SMALL;
  rc = check_device();
  if (rc != FAL_OK) return rc;

  fal::DecodeParams p{};
  p.q = q;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.k_strides = to_rs(k_strides);
  p.v_strides = to_rs(v_strides);
  p.k_new = k_new;
  p.v_new = v_new;
  p.cache_seqlens = cache_seqlens;
  p.cache_starts = cache_starts;
  p.o = o;
  p.lse = lse;
  p.batch = batch;
  p.heads_q = heads_q;
  p.heads_kv = heads_kv;
  p.capacity = capacity;
  p.head_dim = kernel_head_dim(head_dim);
  p.head_dim_real = head_dim;
  p.split_len = w.split_len;
  p.splits = static_cast<int>(w.splits);
  p.scale = softmax_scale;
  p.status = status;
  p.part_o = static_cast<float*>(workspace);
  p.part_ml = p.part_o + static_cast<int64_t>(batch) * heads_q * p.splits * p.head_dim;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rec = g_timer.begin(FAL_KERNEL_DECODE_SPLITK, st);
  cudaError_t e = fal::launch_decode_splitk(p, st);
  g_timer.end(FAL_KERNEL_DECODE_SPLITK, rec, st);
  if (e != cudaSuccess) return cuda_fail(e);
  e = fal::launch_decode_combine(p, st);
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}
}  // namespace

int fal_decode(const void* q, void* k_cache, void* v_cache, const fal_strides* k_strides,
               const fal_strides* v_strides, const int32_t* cache_seqlens, const void* k_new,
               const void* v_new, void* o, float* lse, int batch, int heads_q, int heads_kv,
               int capacity, int head_dim, float softmax_scale, void* workspace,
               size_t workspace_bytes, int* status, void* stream) {
  return decode_with_workspace(q, k_cache, v_cache, k_strides, v_strides, nullptr, cache_seqlens, k_new,
                               v_new, o, lse, batch, heads_q, heads_kv, capacity, head_dim, softmax_scale,
                               workspace, workspace_bytes, status, stream);
}

int fal_decode_ranged(const void* q, void* k_cache, void* v_cache, const fal_strides* k_strides,
                      const fal_strides* v_strides, const int32_t* cache_starts,
                      const int32_t* cache_seqlens, const void* k_new, const void* v_new, void* o,
                      float* lse, int batch, int heads_q, int heads_kv, int capacity, int head_dim,
                      float softmax_scale, void* workspace, size_t workspace_bytes, int* status,
                      void* stream) {
  if (!cache_starts) return FAL_ERR_INVALID_ARGUMENT;
  return decode_with_workspace(q, k_cache, v_cache, k_strides, v_strides, cache_starts, cache_seqlens,
                               k_new, v_new, o, lse, batch, heads_q, heads_kv, capacity, head_dim,
                               softmax_scale, workspace, workspace_bytes, status, stream);
}

int fal_decode_static(const void* q, void* k_cache, void* v_cache, const fal_strides* k_strides,
                      const fal_strides* v_strides, const int32_t* cache_seqlens, const void* k_new,
                      const void* v_new, void* o, float* lse, int batch, int heads_q, int heads_kv,
                      int capacity, int head_dim, float softmax_scale, int* status, void* stream) {
  int rc = decode_check_args(q, k_cache, v_cache, k_strides, v_strides, cache_seqlens, k_new, v_new, o, batch,
                             heads_q, heads_kv, capacity, head_dim, softmax_scale);
  if (rc != FAL_OK) return rc;
  // The partials of this problem must fit the fixed array; nothing is launched otherwise.
  if (fal_decode_workspace_bytes(batch, heads_q, capacity, head_dim) > fal::kDecodeStaticScratchBytes)
    return FAL_ERR_STATIC_SCRATCH_EXCEEDED;
  rc = check_device();
  if (rc != FAL_OK) return rc;
  float* scratch = nullptr;
  cudaError_t e = fal::decode_static_scratch(&scratch);  // first call per device: address look-up
  if (e != cudaSuccess) return cuda_fail(e);
  return decode_with_workspace(q, k_cache, v_cache, k_strides, v_strides, nullptr, cache_seqlens, k_new, v_new,
                               o, lse, batch, heads_q, heads_kv, capacity, head_dim, softmax_scale, scratch,
                               fal::kDecodeStaticScratchBytes, status, stream);
}

int fal_set_fwd_variant(int variant) {
  if (variant < FAL_FWD_AUTO || variant > FAL_FWD_TWO_TILES) return FAL_ERR_INVALID_ARGUMENT;
  g_fwd_variant.store(variant, std::memory_order_relaxed);
  return FAL_OK;
}

int fal_selftest_wait_timeout(int barrier_id, int* status, int* waits_given_up, void* stream) {
  if (!status || barrier_id < 0 || barrier_id >= 1000) return FAL_ERR_INVALID_ARGUMENT;
  int rc = check_device();
  if (rc != FAL_OK) return rc;
  cudaError_t e = fal::launch_selftest_wait(barrier_id, status, waits_given_up, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FAL_OK : cuda_fail(e);
}

int fal_profile_enable(int on) {
  std::lock_guard<std::mutex> g(g_timer.mu);
  g_timer.enabled = on != 0;
  return FAL_OK;
}

int fal_profile_read(int kind, double* total_ms, int* launches) {
  if (kind < 0 || kind >= KernelTimer::kKinds || !total_ms || !launches) return FAL_ERR_INVALID_ARGUMENT;
  std::vector<KernelTimer::Rec> recs;
  {
    std::lock_guard<std::mutex> g(g_timer.mu);
    recs.swap(g_timer.recs[kind]);
  }
  double sum = 0.0;
  int n = 0;
  int rc = FAL_OK;
  for (auto& r : recs) {
    float ms = 0.f;
    cudaError_t e = cudaEventSynchronize(r.b);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, r.a, r.b);
    if (e == cudaSuccess) {
      sum += ms;
      ++n;
    } else {
      rc = cuda_fail(e);
    }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  *total_ms = sum;
  *launches = n;
  return rc;
}

}  // extern "C"
