// Host/device-shared parameter blocks for the attention kernels.
//
// These play the role of the reference's POD argument structs
// (csrc/include/flash_attn_common.h:25-147 in sirCamp/flash-attention-legacy):
// raw pointers, sizes, element strides, softmax scale and the causal flag.
// Strides are 64-bit here (the reference's are int32, which overflows on
// long-context inputs).
#pragma once

#include <stdint.h>

namespace fal {

// Where a [batch, head, row] coordinate lives inside a tensor whose last
// dimension (head_dim) is contiguous.  Strides are in elements.
struct RowStrides {
  int64_t batch;
  int64_t head;
  int64_t row;
};

struct FwdParams {
  void* o;     // fp16 output
  float* lse;  // natural-log LSE of the scaled scores
  RowStrides o_strides;
  RowStrides lse_strides;  // in floats; batched [B,Hq,N] or packed [total,Hq]
  const int32_t* cu_q;     // packed mode: cumulative lengths, else nullptr
  const int32_t* cu_k;
  int num_seqs;   // packed mode only
  int batch;      // batched mode only
  int heads_q;
  int heads_kv;
  int seqlen_q;   // batched mode only
  int seqlen_k;   // batched mode only
  int head_dim;   // the tensors' head_dim: 32 and 96 run on the 64 / 128 kernels (TMA fills the missing
                  // columns with zeros), output columns beyond it are not written
  int cta_rows;   // query rows per CTA: 256 (two tiles) or 128 (one tile, both softmax warpgroups on it)
  int num_qblk;   // batched: ceil(seqlen_q / cta_rows); packed: bound on all sequences' blocks
  int causal_shift;  // causal kernels, batched: query row i sees keys <= i + causal_shift (0: top-left aligned mask)
  int shift_per_sequence;  // causal kernels, packed: the shift of a sequence is its seqlen_k - seqlen_q
  int store_by_tma;  // O tiles leave through shared memory and TMA stores (the output's tensor map is valid)
  const int32_t* seqused_k;  // batched mode, optional: keys in use per batch entry (a cache filled to different
                             // lengths); seqlen_k is then the capacity, and shift_per_sequence applies per entry
  float scale;       // softmax scale
  float scale_log2;  // softmax scale * log2(e)
  int* status;       // device status word, may be nullptr
};

struct BwdParams {
  // outputs
  void* dk;  // fp16
  void* dv;  // fp16
  float* dk_f32;  // when set, dK and dV leave as unrounded fp32 here instead (same strides, in floats)
  float* dv_f32;
  int store_by_tma;  // dK / dV tiles leave through shared memory and TMA stores (the tensor maps are valid)
  RowStrides dk_strides;
  RowStrides dv_strides;
  float* dq_accum;  // fp32 [batch, heads_q, padded_q_rows, head_dim] (packed: [heads_q, padded_total, head_dim])
  int64_t dq_accum_head_stride;   // floats
  int64_t dq_accum_batch_stride;  // floats
  // per-row statistics, [batch, heads_q, rows] (packed: strides say where)
  const float* lse;
  RowStrides lse_strides;
  const float* delta;  // rowsum(dO * O), same indexing as dq_accum rows: [batch, heads_q, padded rows]
  int64_t delta_head_stride;
  int64_t delta_batch_stride;
  const int32_t* cu_q;
  const int32_t* cu_k;
  int num_seqs;
  int batch;
  int heads_q;
  int heads_kv;
  int seqlen_q;
  int seqlen_k;
  int head_dim;   // the tensors' head_dim (32 / 96 run on the 64 / 128 kernels); dK, dV columns beyond it are not written
  int num_kvblk;  // batched: ceil(seqlen_k / 128); packed: bound over all sequences
  int causal_shift;        // causal, batched: query row i sees keys <= i + causal_shift (0: top-left aligned mask)
  int shift_per_sequence;  // causal, packed: the shift of a sequence is its seqlen_k - seqlen_q
  float scale;
  float scale_log2;
  int* status;
};

}  // namespace fal
