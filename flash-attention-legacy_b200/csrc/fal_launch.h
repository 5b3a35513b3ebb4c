// Internal launcher declarations shared by the kernel files and the C-ABI layer.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "fal_common.h"

namespace fal {

// Runs a per-device set-up action (e.g. cudaFuncSetAttribute) once for each
// device that launches a kernel, under a mutex so that concurrent callers on
// different host threads are safe.
class DeviceOnce {
 public:
  template <class F>
  cudaError_t run(F&& f) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> g(mu_);
    if (done_[dev]) return cudaSuccess;
    e = f();
    if (e == cudaSuccess) done_[dev] = true;
    return e;
  }

 private:
  static constexpr int kMaxDevices = 64;
  std::mutex mu_;
  bool done_[kMaxDevices] = {};
};

// Forward: grid = number of (p.cta_rows-row block, batch*head) units.  fwd_cta_rows gives the rows
// a CTA takes: 256 (two query tiles) unless head_dim is 256 or the one-tile variant is asked for.
int fwd_cta_rows(int head_dim, bool one_tile);
cudaError_t launch_fwd(int head_dim, bool causal, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& to, const FwdParams& p, int grid,
                       cudaStream_t stream);

// Backward pre-pass: delta = rowsum(dO * O) and zero of the fp32 dQ accumulator.
struct BwdPrepParams {
  const void* o;
  const void* d_o;
  RowStrides o_strides;
  RowStrides do_strides;
  float* delta;
  int64_t delta_head_stride;
  int64_t delta_batch_stride;
  float* dq_accum;
  int64_t dq_accum_head_stride;
  int64_t dq_accum_batch_stride;
  int batch;       // 1 when packed
  int heads_q;
  int rows;        // batched: seqlen_q; packed: total_q
  int padded_rows; // rows of delta / dq_accum per (batch, head)
  int head_dim;      // kernel head_dim (64, 128, 256): row length of dq_accum
  int head_dim_real; // the tensors' head_dim (32 -> 64 and 96 -> 128 kernels read the rest as zeros)
};
cudaError_t launch_bwd_prep(const BwdPrepParams& p, cudaStream_t stream);

// Backward main kernel: grid = number of (128-key block, batch*kv_head) units.
// tdq: fp32 tensor map of the dQ accumulator (head_dim, padded rows, heads, batch), 32 x 128 boxes.
cudaError_t launch_bwd(int head_dim, bool causal, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdq,
                       const CUtensorMap& tdk, const CUtensorMap& tdv, const BwdParams& p, int grid,
                       cudaStream_t stream);

// Backward post-pass: dQ = fp16(scale * dq_accum).
struct BwdPostParams {
  const float* dq_accum;
  int64_t dq_accum_head_stride;
  int64_t dq_accum_batch_stride;
  void* dq;
  RowStrides dq_strides;
  int batch;
  int heads_q;
  int rows;
  int head_dim;      // kernel head_dim: row length of dq_accum
  int head_dim_real; // the tensors' head_dim: columns of dq that exist
  float scale;
};
cudaError_t launch_bwd_post(const BwdPostParams& p, cudaStream_t stream);

// One block waiting on a barrier that never completes (fal_selftest.cu): the bounded wait must end it.
cudaError_t launch_selftest_wait(int barrier_id, int* status, int* waits_given_up, cudaStream_t stream);

// Element-wise steps of a ring / context-parallel pass (fal_ring.cu).  Tensors are addressed as
// [batch, heads, rows, head_dim] through element strides; LSE tensors as [batch, heads, rows].
struct MergeParams {
  float* o_acc;          // fp32, in-out
  float* lse_acc;        // fp32, in-out
  const void* o_part;    // fp16
  const float* lse_part;
  RowStrides o_acc_strides, lse_acc_strides, o_part_strides, lse_part_strides;
  int batch, heads, rows, head_dim;
  int init;              // non-zero: the accumulators hold nothing yet and are overwritten
};
struct AccumulateParams {
  float* dst;
  const float* src;
  RowStrides dst_strides, src_strides;
  int batch, heads, rows, head_dim;
};
struct ScaleCastParams {
  void* dst;             // fp16
  const float* src;
  RowStrides dst_strides, src_strides;
  int batch, heads, rows, head_dim;
  float scale;
};
cudaError_t launch_merge_partial(const MergeParams& p, cudaStream_t stream);
cudaError_t launch_accumulate(const AccumulateParams& p, cudaStream_t stream);
cudaError_t launch_scale_cast(const ScaleCastParams& p, cudaStream_t stream);

// Decode over a KV cache: split-K streaming pass (which also appends the new row), then the
// log-sum-exp combine.
struct DecodeParams {
  const void* q;        // [batch, heads_q, head_dim] fp16, contiguous
  void* k_cache;        // fp16
  void* v_cache;        // fp16
  RowStrides k_strides; // batch / head / row(position) strides in elements
  RowStrides v_strides;
  const void* k_new;    // optional [batch, heads_kv, head_dim] fp16 to append, else nullptr
  const void* v_new;
  const int32_t* cache_seqlens;  // [batch] valid positions before the append
  const int32_t* cache_starts;   // optional [batch]: first position attended to (left padding), else nullptr
  void* o;              // [batch, heads_q, head_dim] fp16
  float* lse;           // optional [batch, heads_q]
  float* part_o;        // workspace [batch, heads_q, splits, head_dim] fp32
  float* part_ml;       // workspace [batch, heads_q, splits, 2] (max, sum)
  int batch;
  int heads_q;
  int heads_kv;
  int capacity;         // cache positions per batch entry
  int head_dim;         // kernel head_dim (64, 128, 256): row length of the partial results
  int head_dim_real;    // the tensors' head_dim (32 and 96 run on the 64 / 128 kernels)
  int split_len;        // positions per split (multiple of the key tile)
  int splits;           // ceil(capacity / split_len)
  float scale;
  int* status;
};
// Size of the library-resident scratch behind fal_decode_static, and its per-device address.
constexpr size_t kDecodeStaticScratchBytes = 8u << 20;
cudaError_t decode_static_scratch(float** ptr);

cudaError_t launch_decode_splitk(const DecodeParams& p, cudaStream_t stream);
cudaError_t launch_decode_combine(const DecodeParams& p, cudaStream_t stream);

}  // namespace fal
