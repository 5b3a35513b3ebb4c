// Single-token decode against an fp16 KV cache: a split-K streaming kernel (which
// also appends the new token's K/V row) followed by a log-sum-exp combine.
//
// Stands in for the eager matmul -> softmax -> matmul fallback that the
// reference's attention hook uses whenever q_len != kv_len
// (flash_attn_legacy/integrations.py:77-98): softmax(q K^T * scale) V over the
// valid cache positions, no causal mask, GQA by head mapping instead of
// repeat_interleave.
//
// The pass is bound by HBM bandwidth (4 flops per cache byte), so the kernel is
// organised around keeping 16-byte loads in flight:
//   - grid (kv_head x head-chunk, split, batch); each CTA streams `split_len`
//     cache positions of one KV head exactly once for all the query heads that
//     share it (up to 16 per CTA);
//   - every warp runs its own cp.async pipeline over interleaved 16-key slices
//     (no block-level barrier inside the main loop), shared memory XOR-swizzled
//     for conflict-free ldmatrix;
//   - scores and PV use mma.sync m16n8k16 with the query heads as the M rows:
//     tensor throughput is irrelevant here, the MMA only keeps the issue slots
//     free for the loads;
//   - the CTA whose split holds the position the new token goes to writes that
//     row into the cache before it starts streaming (no separate append launch);
//   - each split writes an unnormalised fp32 partial (O, max, sum); the combine
//     kernel merges the splits that the sequence length actually reaches.  (Letting
//     the last split of an entry to finish do the merge instead -- an arrival
//     counter per entry, one launch in all -- was built and measured: every CTA then
//     ends with a fence and an atomic round trip to L2, which cost more than the
//     second launch saves, 84 against 80 us per step on an 8-entry batch replayed as
//     a CUDA graph and 0.797 against 0.787 ms at batch 64.)
// An optional first position per batch entry (cache_starts) skips a padded prefix
// of the cache: the entry's row pointers start there and its length shrinks.
#include "fal_common.h"
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kSliceKeys = 16;  // keys per warp step
constexpr int kDecStages = 3;   // per-warp pipeline depth
constexpr float kNegInfD = -INFINITY;

__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D (fp32, 16x8) += A (fp16, 16x16) * B (fp16, 16x8)
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------
// Append + split-K pass + merge by the last CTA to arrive.
// ---------------------------------------------------------------------------
// The keys entry b attends to: [start, start + len) of its cache, the appended token included when
// there is one and it fits.  `can_append`: a new token is given and position len_old is inside the
// cache.  A cache that is already full (or a negative length) cannot take the token: it is then
// neither stored nor attended to, and the status word says so.
struct DecodeRange {
  int len_old;
  int start;
  int len;
  bool can_append;
};
__device__ __forceinline__ DecodeRange decode_range(const DecodeParams& p, int b) {
  DecodeRange r;
  r.len_old = __ldg(p.cache_seqlens + b);
  r.can_append = p.k_new != nullptr && r.len_old >= 0 && r.len_old < p.capacity;
  int len = min(max(r.len_old + (r.can_append ? 1 : 0), 0), p.capacity);
  r.start = p.cache_starts ? min(max(__ldg(p.cache_starts + b), 0), len) : 0;
  r.len = len - r.start;
  return r;
}

template <int D>
struct DecSmem {
  static constexpr int kRowBytes = D * 2;
  static constexpr int kSliceBytes = kSliceKeys * kRowBytes;            // one K or V slice
  static constexpr int kStageBytes = 2 * kSliceBytes;                   // K then V
  static constexpr int kWarpBytes = kDecStages * kStageBytes;
  static constexpr int kPipeBytes = kDecWarps * kWarpBytes;
  // After the main loop the same memory holds the per-warp partials.
  static constexpr int kMergeBytes = kDecWarps * 16 * (D + 2) * 4;
  static constexpr int kBytes = kPipeBytes > kMergeBytes ? kPipeBytes : kMergeBytes;
};

template <int D>
__global__ void __launch_bounds__(kDecThreads)
fal_decode_splitk_kernel(const DecodeParams p) {
  using L = DecSmem<D>;
  constexpr int kChunks = D / 8;       // 16-byte chunks per row
  constexpr int kKSteps = D / 16;      // k-steps of the score MMA
  constexpr int kNTiles = D / 8;       // 8-wide output tiles of the PV MMA
  constexpr int kLoadsPerLane = kSliceKeys * kChunks / 32;

  extern __shared__ __align__(128) uint8_t dec_smem[];

  const int group = p.heads_q / p.heads_kv;          // query heads per KV head
  const int head_chunks = (group + 15) / 16;
  const int kv_head = blockIdx.x / head_chunks;
  const int head_chunk = blockIdx.x % head_chunks;
  const int split = blockIdx.y;
  const int b = blockIdx.z;

  const DecodeRange rg = decode_range(p, b);
  const int len_old = rg.len_old, start = rg.start, len = rg.len;
  const bool can_append = rg.can_append;
  if (p.k_new != nullptr && !can_append && split == 0 && blockIdx.x == 0 && threadIdx.x == 0 && p.status)
    atomicCAS(p.status, 0, kDevAppendOverflow);
  const int pos0 = split * p.split_len;

  const int rows_valid = min(16, group - head_chunk * 16);
  const int hq0 = kv_head * group + head_chunk * 16;  // first query head of this CTA

  // ---- append: the split that holds the new position stores the row, then streams it like any
  // other (split 0 stores it when the position lies before `start` and nobody attends to it) ----
  if (can_append) {
    const int new_local = len_old - start;
    const int store_split = new_local >= 0 ? new_local / p.split_len : 0;
    if (split == store_split) {
      const int real_chunks = p.head_dim_real / 8;  // head_dim 32 / 96 run on the 64 / 128 kernels
      for (int c = threadIdx.x; c < 2 * real_chunks; c += kDecThreads) {
        const bool is_v = c >= real_chunks;
        const int cc = is_v ? c - real_chunks : c;
        const __half* src = static_cast<const __half*>(is_v ? p.v_new : p.k_new) +
                            (static_cast<int64_t>(b) * p.heads_kv + kv_head) * p.head_dim_real + cc * 8;
        const RowStrides& st = is_v ? p.v_strides : p.k_strides;
        __half* dst = static_cast<__half*>(is_v ? p.v_cache : p.k_cache) + b * st.batch + kv_head * st.head +
                      static_cast<int64_t>(len_old) * st.row + cc * 8;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
      }
      __threadfence();   // the row is read back through L2 by this CTA's asynchronous copies
      __syncthreads();
    }
  }
  if (pos0 >= len) return;  // this split lies beyond the sequence
  const int pos_end = min(pos0 + p.split_len, len);
  const int num_slices = (pos_end - pos0 + kSliceKeys - 1) / kSliceKeys;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int t = lane & 3;

  // ---- query fragments (A operand: row = head, col = head_dim) ---------------
  uint32_t qa[kKSteps][4];
  {
    // (columns beyond the tensors' head_dim -- 32 and 96 run on the 64 / 128 kernels -- read as zero)
    const int dr = p.head_dim_real;
    const __half* qb = static_cast<const __half*>(p.q) + (static_cast<int64_t>(b) * p.heads_q + hq0) * dr;
#pragma unroll
    for (int ks = 0; ks < kKSteps; ++ks) {
      const int col = ks * 16 + 2 * t;
      qa[ks][0] = (g < rows_valid && col < dr) ? *reinterpret_cast<const uint32_t*>(qb + g * dr + col) : 0u;
      qa[ks][1] = (g + 8 < rows_valid && col < dr) ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * dr + col) : 0u;
      qa[ks][2] = (g < rows_valid && col + 8 < dr) ? *reinterpret_cast<const uint32_t*>(qb + g * dr + col + 8) : 0u;
      qa[ks][3] = (g + 8 < rows_valid && col + 8 < dr) ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * dr + col + 8) : 0u;
    }
  }

  const __half* kbase = static_cast<const __half*>(p.k_cache) + b * p.k_strides.batch +
                        kv_head * p.k_strides.head + static_cast<int64_t>(start) * p.k_strides.row;
  const __half* vbase = static_cast<const __half*>(p.v_cache) + b * p.v_strides.batch +
                        kv_head * p.v_strides.head + static_cast<int64_t>(start) * p.v_strides.row;
  const uint32_t wbase = smem_u32(dec_smem) + warp * L::kWarpBytes;
  const int real_chunks = p.head_dim_real / 8;

  // Issues the loads of this warp's i-th slice (keys pos0 + (i*4 + warp)*16 ...).
  auto issue_slice = [&](int i) {
    const int slice = i * kDecWarps + warp;
    if (slice < num_slices) {
      const uint32_t sb = wbase + (i % kDecStages) * L::kStageBytes;
      const int key0 = pos0 + slice * kSliceKeys;
#pragma unroll
      for (int it = 0; it < kLoadsPerLane; ++it) {
        const int idx = it * 32 + lane;
        const int row = idx / kChunks;
        const int ch = idx % kChunks;
        const int key = key0 + row;
        const bool ok = key < pos_end && ch < real_chunks;  // chunks past the tensors' head_dim fill with zeros
        const int64_t krow = static_cast<int64_t>(key < pos_end ? key : pos0);
        const int src_ch = ch < real_chunks ? ch : 0;
        const uint32_t soff = row * L::kRowBytes + ((ch ^ (row & 7)) << 4);
        cp_async_16_zfill(sb + soff, kbase + krow * p.k_strides.row + src_ch * 8, ok);
        cp_async_16_zfill(sb + L::kSliceBytes + soff, vbase + krow * p.v_strides.row + src_ch * 8, ok);
      }
    }
    cp_async_commit();  // always commit so that group counting stays uniform
  };

  float acc_o[kNTiles][4];
#pragma unroll
  for (int n = 0; n < kNTiles; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc_o[n][i] = 0.f;
  float m_run[2] = {kNegInfD, kNegInfD};  // rows g and g+8, log2 domain
  float l_run[2] = {0.f, 0.f};
  const float c2 = p.scale * 1.4426950408889634f;

  const int my_slices = (num_slices - warp + kDecWarps - 1) / kDecWarps;  // may be <= 0
#pragma unroll
  for (int i = 0; i < kDecStages - 1; ++i) issue_slice(i);

  for (int i = 0; i < my_slices; ++i) {
    issue_slice(i + kDecStages - 1);
    cp_async_wait<kDecStages - 1>();
    __syncwarp();
    const uint32_t sb = wbase + (i % kDecStages) * L::kStageBytes;
    const int key0 = pos0 + (i * kDecWarps + warp) * kSliceKeys;

    // ---- S = Q K^T (16 heads x 16 keys) ------------------------------------
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    {
      const int mi = lane >> 3;
      const int r = lane & 7;
      const int krow = (mi >> 1) * 8 + r;
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        const int ch = 2 * ks + (mi & 1);
        uint32_t b00, b01, b10, b11;
        ldmatrix_x4(sb + krow * L::kRowBytes + ((ch ^ (krow & 7)) << 4), b00, b01, b10, b11);
        mma_16816(s[0], qa[ks], b00, b01);
        mma_16816(s[1], qa[ks], b10, b11);
      }
    }
    // ---- online softmax (log2 domain) --------------------------------------
    const bool tail = key0 + kSliceKeys > pos_end;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * c2;
        if (tail && (key0 + nt * 8 + 2 * t + (e & 1) >= pos_end)) v = kNegInfD;
        s[nt][e] = v;
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mx = fmaxf(fmaxf(s[0][2 * h], s[0][2 * h + 1]), fmaxf(s[1][2 * h], s[1][2 * h + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[h], mx);
      const float m_use = (m_new == kNegInfD) ? 0.f : m_new;
      alpha[h] = fast_exp2(m_run[h] - m_use);  // exp2(-inf) = 0 on the first slice
      float sum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float p0 = fast_exp2(s[nt][2 * h] - m_use);
        const float p1 = fast_exp2(s[nt][2 * h + 1] - m_use);
        s[nt][2 * h] = p0;
        s[nt][2 * h + 1] = p1;
        sum += p0 + p1;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l_run[h] = l_run[h] * alpha[h] + sum;
      m_run[h] = m_new;
    }
    uint32_t pa[4];
    pa[0] = pack_half2(s[0][0], s[0][1]);
    pa[1] = pack_half2(s[0][2], s[0][3]);
    pa[2] = pack_half2(s[1][0], s[1][1]);
    pa[3] = pack_half2(s[1][2], s[1][3]);

    // ---- O = alpha * O + P V ----------------------------------------------
    {
      const int mi = lane >> 3;
      const int r = lane & 7;
      const int vrow = (mi & 1) * 8 + r;
      const uint32_t vb = sb + L::kSliceBytes + vrow * L::kRowBytes;
#pragma unroll
      for (int n = 0; n < kNTiles; n += 2) {
        const int ch = n + (mi >> 1);
        uint32_t b00, b01, b10, b11;
        ldmatrix_x4_trans(vb + ((ch ^ (vrow & 7)) << 4), b00, b01, b10, b11);
        acc_o[n][0] *= alpha[0];
        acc_o[n][1] *= alpha[0];
        acc_o[n][2] *= alpha[1];
        acc_o[n][3] *= alpha[1];
        acc_o[n + 1][0] *= alpha[0];
        acc_o[n + 1][1] *= alpha[0];
        acc_o[n + 1][2] *= alpha[1];
        acc_o[n + 1][3] *= alpha[1];
        mma_16816(acc_o[n], pa, b00, b01);
        mma_16816(acc_o[n + 1], pa, b10, b11);
      }
    }
    __syncwarp();  // all lanes are done with this stage before it is refilled
  }
  cp_async_wait<0>();
  __syncthreads();  // the pipeline memory is reused for the merge below

  // ---- merge the four warps' partials and write the split's result ----------
  float* mo = reinterpret_cast<float*>(dec_smem);               // [warp][16][D]
  float* mml = mo + kDecWarps * 16 * D;                         // [warp][16][2]
#pragma unroll
  for (int n = 0; n < kNTiles; ++n) {
    const int col = n * 8 + 2 * t;
    *reinterpret_cast<float2*>(mo + (warp * 16 + g) * D + col) = make_float2(acc_o[n][0], acc_o[n][1]);
    *reinterpret_cast<float2*>(mo + (warp * 16 + g + 8) * D + col) = make_float2(acc_o[n][2], acc_o[n][3]);
  }
  if (t == 0) {
    mml[(warp * 16 + g) * 2 + 0] = m_run[0];
    mml[(warp * 16 + g) * 2 + 1] = l_run[0];
    mml[(warp * 16 + g + 8) * 2 + 0] = m_run[1];
    mml[(warp * 16 + g + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_valid * D; idx += kDecThreads) {
    const int r = idx / D;
    const int c = idx % D;
    float mmax = kNegInfD;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mmax = fmaxf(mmax, mml[(w * 16 + r) * 2]);
    const float muse = (mmax == kNegInfD) ? 0.f : mmax;
    float o = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float sc = fast_exp2(mml[(w * 16 + r) * 2] - muse);
      o += sc * mo[(w * 16 + r) * D + c];
      lsum += sc * mml[(w * 16 + r) * 2 + 1];
    }
    const int64_t prow = (static_cast<int64_t>(b) * p.heads_q + hq0 + r) * p.splits + split;
    p.part_o[prow * D + c] = o;
    if (c == 0) {
      p.part_ml[prow * 2 + 0] = mmax;
      p.part_ml[prow * 2 + 1] = lsum;
    }
  }

}

// ---------------------------------------------------------------------------
// Combine: merge the splits a sequence actually reaches.
// ---------------------------------------------------------------------------
__global__ void fal_decode_combine_kernel(const DecodeParams p) {
  const int bh = blockIdx.x;
  const int b = bh / p.heads_q;
  const int D = p.head_dim;
  const int len = decode_range(p, b).len;
  const int n = (len + p.split_len - 1) / p.split_len;
  const float* ml = p.part_ml + static_cast<int64_t>(bh) * p.splits * 2;
  const float* po = p.part_o + static_cast<int64_t>(bh) * p.splits * D;

  float mmax = kNegInfD;
  for (int i = 0; i < n; ++i) mmax = fmaxf(mmax, ml[2 * i]);
  const float muse = (mmax == kNegInfD) ? 0.f : mmax;
  float lsum = 0.f;
  for (int i = 0; i < n; ++i) lsum += fast_exp2(ml[2 * i] - muse) * ml[2 * i + 1];
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  for (int c = threadIdx.x; c < p.head_dim_real; c += blockDim.x) {
    float o = 0.f;
    for (int i = 0; i < n; ++i) o += fast_exp2(ml[2 * i] - muse) * po[static_cast<int64_t>(i) * D + c];
    static_cast<__half*>(p.o)[static_cast<int64_t>(bh) * p.head_dim_real + c] = __float2half_rn(o * inv);
  }
  if (p.lse != nullptr && threadIdx.x == 0) {
    p.lse[bh] = (lsum > 0.f) ? (mmax + log2f(lsum)) * 0.6931471805599453f : kNegInfD;
  }
}

template <int D>
cudaError_t launch_splitk_t(const DecodeParams& p, cudaStream_t stream) {
  auto kern = fal_decode_splitk_kernel<D>;
  static DeviceOnce configured;
  cudaError_t e = configured.run([&] {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                DecSmem<D>::kBytes);
  });
  if (e != cudaSuccess) return e;
  const int group = p.heads_q / p.heads_kv;
  const int head_chunks = (group + 15) / 16;
  dim3 grid(p.heads_kv * head_chunks, p.splits, p.batch);
  kern<<<grid, kDecThreads, DecSmem<D>::kBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

// ---------------------------------------------------------------------------
// Fixed scratch for fal_decode_static: split-K partials for callers that cannot
// allocate device memory.  It lives in the library image, so every GPU that
// loads the library carries these bytes until the process exits.
// ---------------------------------------------------------------------------
namespace {
static __device__ __align__(256) float g_decode_static_scratch[kDecodeStaticScratchBytes / sizeof(float)];
}  // namespace

// In host code the array's name is only a handle for the runtime, not a device address, so the
// address is looked up once per device (with that device current) and cached.
cudaError_t decode_static_scratch(float** ptr) {
  static std::mutex mu;
  static float* cached[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
    if (e != cudaSuccess) return e;
    cached[dev] = static_cast<float*>(p);
  }
  *ptr = cached[dev];
  return cudaSuccess;
}

cudaError_t launch_decode_combine(const DecodeParams& p, cudaStream_t stream) {
  fal_decode_combine_kernel<<<p.batch * p.heads_q, p.head_dim, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_decode_splitk(const DecodeParams& p, cudaStream_t stream) {
  if (p.head_dim == 128) return launch_splitk_t<128>(p, stream);
  if (p.head_dim == 64) return launch_splitk_t<64>(p, stream);
  if (p.head_dim == 256) return launch_splitk_t<256>(p, stream);
  return cudaErrorInvalidValue;
}

}  // namespace fal
