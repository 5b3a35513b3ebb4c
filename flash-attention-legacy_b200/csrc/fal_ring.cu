// Element-wise steps between the attention kernels of a ring / context-parallel pass: the exact
// merge of two softmax partials, fp32 accumulation of gradient partials and the final fp32 -> fp16
// cast.  One small kernel each, so that a ring step costs its attention kernels plus one of these
// instead of a chain of framework tensor operations.
//
// The reference has no multi-GPU path (no NCCL, no torch.distributed anywhere in it); these kernels
// serve the long-sequence case its tests run on a single GPU (tests/test_flash_attn.py:486-547)
// when the sequence is sharded over several GPUs.
//
// All three are bound by HBM bandwidth: every thread moves 8 consecutive head_dim elements of one
// (batch, head, row) with 16-byte accesses, rows of a head are contiguous lines.
#include "fal_common.h"
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

constexpr int kRingThreads = 256;

struct RowIndex {
  int b, h, r, sub;
  bool ok;
};

// Thread -> (batch, head, row, 8-element chunk) for a [batch, heads, rows, head_dim] problem.
__device__ __forceinline__ RowIndex ring_row_index(int batch, int heads, int rows, int head_dim) {
  const int chunks = head_dim / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * kRingThreads + threadIdx.x;
  const int64_t total = static_cast<int64_t>(batch) * heads * rows * chunks;
  RowIndex x;
  x.ok = idx < total;
  const int64_t i = x.ok ? idx : 0;
  x.sub = static_cast<int>(i % chunks);
  const int64_t row_id = i / chunks;
  x.r = static_cast<int>(row_id % rows);
  const int64_t bh = row_id / rows;
  x.h = static_cast<int>(bh % heads);
  x.b = static_cast<int>(bh / heads);
  return x;
}

__device__ __forceinline__ int64_t ring_offset(const RowStrides& s, const RowIndex& x) {
  return x.b * s.batch + x.h * s.head + static_cast<int64_t>(x.r) * s.row;
}

// (O_acc, LSE_acc) <- exact merge with (O_part, LSE_part): both are softmax results of the same
// queries over disjoint key sets.  LSE_new = log(exp(LSE_acc) + exp(LSE_part)), O_new = the two
// outputs weighted by exp(LSE - LSE_new).  A side that saw no key (LSE = -inf) has weight 0.
__global__ void __launch_bounds__(kRingThreads) fal_merge_partial_kernel(const MergeParams p) {
  const RowIndex x = ring_row_index(p.batch, p.heads, p.rows, p.head_dim);
  if (!x.ok) return;
  const float lp = p.lse_part[ring_offset(p.lse_part_strides, x)];
  float* lse_acc = p.lse_acc + ring_offset(p.lse_acc_strides, x);
  float w_acc = 0.f, w_part = 1.f, lse_new = lp;
  if (!p.init) {
    const float la = *lse_acc;
    const float m = fmaxf(la, lp);
    if (m == -INFINITY) {
      w_part = 0.f;
      lse_new = -INFINITY;
    } else {
      const float ea = expf(la - m), ep = expf(lp - m);
      const float inv = 1.f / (ea + ep);
      lse_new = m + logf(ea + ep);
      w_acc = ea * inv;
      w_part = ep * inv;
    }
  } else if (lp == -INFINITY) {
    w_part = 0.f;
  }
  float* oa = p.o_acc + ring_offset(p.o_acc_strides, x) + x.sub * 8;
  const __half* op = static_cast<const __half*>(p.o_part) + ring_offset(p.o_part_strides, x) + x.sub * 8;
  const uint4 raw = *reinterpret_cast<const uint4*>(op);
  const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
  float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
  if (w_acc != 0.f) {  // an accumulator that does not count may hold anything
    a0 = *reinterpret_cast<const float4*>(oa);
    a1 = *reinterpret_cast<const float4*>(oa + 4);
  }
  const float2 p0 = __half22float2(h2[0]), p1 = __half22float2(h2[1]);
  const float2 p2 = __half22float2(h2[2]), p3 = __half22float2(h2[3]);
  a0 = make_float4(a0.x * w_acc + p0.x * w_part, a0.y * w_acc + p0.y * w_part, a0.z * w_acc + p1.x * w_part,
                   a0.w * w_acc + p1.y * w_part);
  a1 = make_float4(a1.x * w_acc + p2.x * w_part, a1.y * w_acc + p2.y * w_part, a1.z * w_acc + p3.x * w_part,
                   a1.w * w_acc + p3.y * w_part);
  *reinterpret_cast<float4*>(oa) = a0;
  *reinterpret_cast<float4*>(oa + 4) = a1;
  // The threads of a row (head_dim / 8 <= 32 of them) sit in one warp: all of them have read the old
  // LSE once the warp has passed this point, and only then does the row's first thread replace it.
  __syncwarp();
  if (x.sub == 0) *lse_acc = lse_new;
}

// dst (fp32) += src (fp32)
__global__ void __launch_bounds__(kRingThreads) fal_accumulate_kernel(const AccumulateParams p) {
  const RowIndex x = ring_row_index(p.batch, p.heads, p.rows, p.head_dim);
  if (!x.ok) return;
  float* d = p.dst + ring_offset(p.dst_strides, x) + x.sub * 8;
  const float* s = p.src + ring_offset(p.src_strides, x) + x.sub * 8;
  float4 d0 = *reinterpret_cast<const float4*>(d), d1 = *reinterpret_cast<const float4*>(d + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(s), s1 = *reinterpret_cast<const float4*>(s + 4);
  d0 = make_float4(d0.x + s0.x, d0.y + s0.y, d0.z + s0.z, d0.w + s0.w);
  d1 = make_float4(d1.x + s1.x, d1.y + s1.y, d1.z + s1.z, d1.w + s1.w);
  *reinterpret_cast<float4*>(d) = d0;
  *reinterpret_cast<float4*>(d + 4) = d1;
}

// dst (fp16) = scale * src (fp32)
__global__ void __launch_bounds__(kRingThreads) fal_scale_cast_kernel(const ScaleCastParams p) {
  const RowIndex x = ring_row_index(p.batch, p.heads, p.rows, p.head_dim);
  if (!x.ok) return;
  const float* s = p.src + ring_offset(p.src_strides, x) + x.sub * 8;
  const float4 a = *reinterpret_cast<const float4*>(s), b = *reinterpret_cast<const float4*>(s + 4);
  uint4 out;
  out.x = pack_half2(a.x * p.scale, a.y * p.scale);
  out.y = pack_half2(a.z * p.scale, a.w * p.scale);
  out.z = pack_half2(b.x * p.scale, b.y * p.scale);
  out.w = pack_half2(b.z * p.scale, b.w * p.scale);
  *reinterpret_cast<uint4*>(static_cast<__half*>(p.dst) + ring_offset(p.dst_strides, x) + x.sub * 8) = out;
}

unsigned ring_blocks(int batch, int heads, int rows, int head_dim) {
  const int64_t total = static_cast<int64_t>(batch) * heads * rows * (head_dim / 8);
  return static_cast<unsigned>((total + kRingThreads - 1) / kRingThreads);
}

}  // namespace

cudaError_t launch_merge_partial(const MergeParams& p, cudaStream_t stream) {
  fal_merge_partial_kernel<<<ring_blocks(p.batch, p.heads, p.rows, p.head_dim), kRingThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_accumulate(const AccumulateParams& p, cudaStream_t stream) {
  fal_accumulate_kernel<<<ring_blocks(p.batch, p.heads, p.rows, p.head_dim), kRingThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_scale_cast(const ScaleCastParams& p, cudaStream_t stream) {
  fal_scale_cast_kernel<<<ring_blocks(p.batch, p.heads, p.rows, p.head_dim), kRingThreads, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fal
