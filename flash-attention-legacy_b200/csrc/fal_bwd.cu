// FlashAttention-2 backward for sm_100a: dK/dV/dQ with P recomputed from the
// forward's log-sum-exp, five tcgen05 GEMMs per (key tile, query tile) pair,
// all accumulators in TMEM.
//
// Replaces precompute_D_kernel, flash_attn_bwd_volta_kernel and the fp32->fp16
// dQ cast (csrc/kernels/flash_attn_bwd.cu:76-107, :425-647 and
// csrc/flash_attn_legacy.cpp:126,184 of the reference).  Same loop nest -- a
// CTA owns one 128-key tile of one KV head and sweeps the query heads of its
// group and their (causally reachable) query tiles -- and the same math:
//   P  = exp(S*scale - L)          dV += P^T dO
//   dP = dO V^T                    dS  = P o (dP - D)      (scale applied at the end)
//   dK += dS^T Q                   dQ += dS K
// with P and dS rounded to fp16 before they feed a GEMM.
//
// S, dP, dV and dK are computed transposed (keys on the 128 TMEM lanes), 128 queries per step,
// so that every MMA is a full M=128 x N=128 instruction (an N=64 instruction costs the same
// tensor-pipe time as an N=128 one):
//   S^T  = K Q^T      (M=128 keys, N=128 queries, K=head_dim)   smem x smem
//   dP^T = V dO^T     (same shape)                              smem x smem
//   dV  += P^T dO     (M=128, N=head_dim, K=128)                TMEM x smem
//   dK  += dS^T Q     (M=128, N=head_dim, K=128)                smem x smem
//   dQ   = dS K       (M=128 queries, N=head_dim, K=128)        smem x smem (dS^T read M-contiguous)
// P^T is produced in place over S^T, each compute thread owns one key row, and dS^T is
// written to shared memory once and serves both dK and dQ.  The dQ tile leaves TMEM through
// a swizzled shared-memory staging buffer and TMA tensor reductions (fp32 add) into the
// accumulator that the post-pass casts.
//
//   warps 0-7    compute (two per TMEM lane quarter, 64 query columns each)
//   warp  8      TMA producer
//   warp  9      tcgen05.mma issuer, TMEM owner
//   warps 10-13  dQ write-back
//   warp  14     LSE / delta staging (kept apart from the TMA producer so that neither waits
//                behind the other's global-memory latency)
//   warp  15     idle
//
// TMEM columns: S^T/P^T [0,128), dP^T/dQ [128,256) (the dQ tile of a step reuses the columns of
//               that step's consumed dP^T), dV [256,256+D), dK [256+D,256+2D).
// Shared memory at head_dim 128: K 32K, V 32K, Q 2 x 32K, dO 32K, dS^T 32K, dQ staging 2 x 16K.
//
// head_dim 256 (SPLIT = true) runs the head_dim-128 layout on column halves: two CTAs share a key
// tile, each owning 128 of the 256 columns of dV, dK and dQ.  The two score GEMMs contract over all
// 256 columns, so every step first loads the OTHER half of K, Q, V and dO into the (single) tile
// buffers and starts S^T and dP^T on it, then loads its own half over them and accumulates; from
// there the step is the head_dim-128 step.  K and V are therefore reloaded every step (they come
// from L2) and a step's loads and GEMMs run one after the other: it is the reference's head_dim
// 256 backward made available, not a tuned kernel.
#include "fal_common.h"
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

constexpr int kBwdThreads = 512;
constexpr int kKvTile = 128;
constexpr int kQTile = 128;
constexpr float kLog2e = 1.4426950408889634f;

enum BwdBarrier : int {
  kBbKFull = 100, kBbVFull = 101, kBbQFull = 110, kBbDoFull = 120, kBbStatFull = 130,
  kBbQEmpty = 140, kBbDoEmpty = 145, kBbSReady = 150, kBbDpReady = 160, kBbPReady = 161,
  kBbDsReady = 162, kBbDqReady = 164, kBbDqFree = 165, kBbAllDone = 166, kBbAFull = 170, kBbADone = 171,
};

template <int D>
struct BwdSmem {
  static constexpr int kQStages = 2;                           // Q tiles and row statistics
  static constexpr int kBoxes = D / 64;
  static constexpr int kBoxBytes = 128 * 128;                  // one 128-row x 128-byte box
  static constexpr int kTileBytes = kBoxes * kBoxBytes;        // K, V, Q and dO tiles are 128 x D
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kTileBytes;
  static constexpr int kQOff = 2 * kTileBytes;
  static constexpr int kDoOff = kQOff + kQStages * kTileBytes;  // single stage
  static constexpr int kDsOff = kDoOff + kTileBytes;            // [2 boxes][128 keys][64 queries] fp16
  static constexpr int kDsBytes = 2 * kBoxBytes;
  static constexpr int kStageOff = kDsOff + kDsBytes;           // dQ staging: 2 x [128 rows][32 fp32]
  static constexpr int kStageBytes = 2 * kBoxBytes;
  static constexpr int kStatOff = kStageOff + kStageBytes;      // per Q stage: lse2[128], delta[128]
  static constexpr int kStatBytes = kQStages * 2 * kQTile * 4;
  static constexpr int kBarOff = kStatOff + kStatBytes;
  // k_full v_full q_full[2] q_empty[2] stat_full[2] do_full do_empty
  // s_ready dp_ready dq_ready dq_free p_ready ds_ready all_done ds_free a_full a_done
  static constexpr int kNumBars = 2 + 6 + 2 + 8 + 2;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kBytes = kMiscOff + 16;
  // No slack for re-aligning the base: at head_dim 128 the layout fills the 227 KB limit, so the
  // kernel requires the dynamic shared memory window itself to be 1024-byte aligned and reports
  // an error otherwise.
  static constexpr int kAllocBytes = kBytes;
  static_assert(kAllocBytes <= 232448, "exceeds the per-CTA shared memory limit");
};

struct BwdWork {
  int batch;      // TMA batch coordinate
  int kv_head;
  int kvblk;      // 128-key block inside the sequence
  int q_row0;     // global row of the sequence's first query (packed), else 0
  int k_row0;
  int seqlen_q;
  int seqlen_k;
};

#ifndef FAL_BWD_WAVE_GROUPS
#define FAL_BWD_WAVE_GROUPS 8
#endif
constexpr int kWaveGroups = FAL_BWD_WAVE_GROUPS;

__device__ __forceinline__ bool bwd_decode_work(const BwdParams& p, int idx, BwdWork& w) {
  if (p.cu_k == nullptr) {
    // CTAs are numbered in waves of up to kWaveGroups (batch, KV head) groups; inside a wave the first key
    // blocks come first (under a causal mask they see the most queries).  The CTAs that run at the
    // same time then add into the fp32 dQ accumulators of a few groups only (8 MB per group at
    // 4 heads x 4096 rows), which stay in L2 between the 32 key tiles that touch them.
    const int bh_count = p.batch * p.heads_kv;
    const int nkvblk = (p.seqlen_k + kKvTile - 1) / kKvTile;
    // equal waves of at most kWaveGroups groups (a short last wave leaves SMs idle at the end)
    const int num_waves = (bh_count + kWaveGroups - 1) / kWaveGroups;
    const int wave_groups = (bh_count + num_waves - 1) / num_waves;
    const int wave = idx / (wave_groups * nkvblk);
    const int first_group = wave * wave_groups;
    const int groups_here = min(wave_groups, bh_count - first_group);
    const int r = idx - wave * wave_groups * nkvblk;
    w.kvblk = r / groups_here;
    const int bh = first_group + r % groups_here;
    w.batch = bh / p.heads_kv;
    w.kv_head = bh % p.heads_kv;
    w.q_row0 = 0;
    w.k_row0 = 0;
    w.seqlen_q = p.seqlen_q;
    w.seqlen_k = p.seqlen_k;
    return true;
  }
  const int slot = idx / p.heads_kv;
  w.kv_head = idx % p.heads_kv;
  w.batch = 0;
  // Which sequence owns key block `slot`: every warp scans the lengths 32 sequences at a time (one
  // coalesced load, a prefix sum of the block counts, a vote) instead of walking them one by one.
  const int lane = threadIdx.x & 31;
  int first = 0;
  for (int base = 0; base < p.num_seqs; base += 32) {
    const int s = base + lane;
    int a = 0, e = 0;
    if (s < p.num_seqs) {
      a = __ldg(p.cu_k + s);
      e = __ldg(p.cu_k + s + 1);
    }
    const int nblk = (e - a + kKvTile - 1) / kKvTile;
    int incl = nblk;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += t;
    }
    const int excl = first + incl - nblk;
    const unsigned hit = __ballot_sync(0xffffffffu, slot >= excl && slot < excl + nblk);
    if (hit != 0u) {
      const int src = __ffs(hit) - 1;
      w.kvblk = slot - __shfl_sync(0xffffffffu, excl, src);
      w.k_row0 = __shfl_sync(0xffffffffu, a, src);
      w.seqlen_k = __shfl_sync(0xffffffffu, e, src) - w.k_row0;
      w.q_row0 = __ldg(p.cu_q + base + src);
      w.seqlen_q = __ldg(p.cu_q + base + src + 1) - w.q_row0;
      return true;
    }
    first += __shfl_sync(0xffffffffu, incl, 31);
  }
  return false;
}

// Of every 8 consecutive score columns, this many take the FMA-pipe exp2 instead of the
// special-function unit (two compute warps per scheduler share 4 ex2 lanes per clock).
#ifndef FAL_BWD_EXP_EMU_PER8
#define FAL_BWD_EXP_EMU_PER8 0
#endif
template <int K>
__device__ __forceinline__ float bwd_exp2(int j, float x) {
  // j is a multiple of 4 under full unrolling, so the choice folds at compile time.
  return (((j + K) & 7) < FAL_BWD_EXP_EMU_PER8) ? exp2_fma(x) : fast_exp2(x);
}

// dQ(i) issued before dK(i) (1): the write-back warps drain dQ out of TMEM -- which the next
// step's dP^T needs gone -- while dK still runs.  0: dK first.
#ifndef FAL_BWD_DQ_FIRST
#define FAL_BWD_DQ_FIRST 1
#endif
// One elected lane per compute warp arrives on p_ready / ds_ready (1) or every thread (0).
#ifndef FAL_BWD_ELECT_ARRIVE
#define FAL_BWD_ELECT_ARRIVE 1
#endif

// fp32 add-reduction of one swizzled shared-memory box into a 4-D tensor (TMA).
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1,
                                                  int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// One swizzled shared-memory box into a 4-D tensor (TMA store; rows and columns past the tensor's
// extent are dropped).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src_smem, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int D, bool CAUSAL, bool SPLIT>
__global__ void __launch_bounds__(kBwdThreads, 1)
fal_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
               const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_dk,
               const __grid_constant__ CUtensorMap tm_dv, const BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int NS = SPLIT ? 1 : L::kQStages;
  // SPLIT: head_dim is 2 * D; CTAs 2n and 2n+1 share key tile n and own columns [0, D) and [D, 2D).
  const int col_own = SPLIT ? static_cast<int>(blockIdx.x & 1) * D : 0;
  const int col_other = SPLIT ? D - col_own : 0;

  BwdWork wk;
  if (!bwd_decode_work(p, SPLIT ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x), wk)) return;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t sbase = smem_u32(smem_raw);
  uint8_t* sgen = smem_raw;
  if ((sbase & 1023u) != 0) {  // the 128-byte swizzle needs 1024-byte aligned tiles
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, kDevWaitTimeout + 999);
    return;
  }
  const uint32_t bar0 = sbase + L::kBarOff;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  constexpr int iKFull = 0, iVFull = 1, iQFull = 2, iQEmpty = 4, iStatFull = 6, iDoFull = 8, iDoEmpty = 9,
                iSReady = 10, iDpReady = 11, iDqReady = 12, iDqFree = 13, iPReady = 14, iDsReady = 15,
                iAllDone = 16, iDsFree = 17, iAFull = 18, iADone = 19;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kMiscOff + 4);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int group = p.heads_q / p.heads_kv;
  const int kv0 = wk.kvblk * kKvTile;                       // local index of the tile's first key
  const int nqt = (wk.seqlen_q + kQTile - 1) / kQTile;
  // Keys the causal diagonal is moved by: query i sees keys <= i + cshift (0 = the reference's
  // top-left-aligned mask; seqlen_k - seqlen_q aligns it to the end of the keys).
  const int cshift = !CAUSAL ? 0
                     : (p.cu_k != nullptr ? (p.shift_per_sequence ? wk.seqlen_k - wk.seqlen_q : 0) : p.causal_shift);
  const int qt0 = CAUSAL ? min(max(kv0 - cshift, 0) / kQTile, nqt) : 0;  // first query tile that sees this key tile
  const int nq = nqt - qt0;                                  // query tiles per head
  const int n_iter = group * nq;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar(iKFull), 1);
    mbar_init(bar(iVFull), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(iQFull + s), 1);
      mbar_init(bar(iQEmpty + s), 1);
      mbar_init(bar(iStatFull + s), 32);
    }
    mbar_init(bar(iDoFull), 1);
    mbar_init(bar(iDoEmpty), 1);
    mbar_init(bar(iSReady), 1);
    mbar_init(bar(iDpReady), 1);
    mbar_init(bar(iDqReady), 1);
    mbar_init(bar(iDqFree), 128);
    mbar_init(bar(iPReady), FAL_BWD_ELECT_ARRIVE ? 8 : 256);
    mbar_init(bar(iDsReady), FAL_BWD_ELECT_ARRIVE ? 8 : 256);
    mbar_init(bar(iAllDone), 1);
    mbar_init(bar(iDsFree), 1);
    mbar_init(bar(iAFull), 1);
    mbar_init(bar(iADone), 1);
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColDpq = 128, kColDv = 256, kColDk = 256 + D;

  if (warp == 8) {
    // ===================== producer: TMA ======================================
    if constexpr (SPLIT) {
      if (lane == 0 && n_iter > 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_dq);
        const uint32_t k_s = sbase + L::kKOff, v_s = sbase + L::kVOff, q_s = sbase + L::kQOff,
                       do_s = sbase + L::kDoOff;
        for (int i = 0; i < n_iter; ++i) {
          const int head = wk.kv_head * group + i / nq;
          const int row = wk.q_row0 + (qt0 + i % nq) * kQTile;
          const int krow = wk.k_row0 + kv0;
          // every GEMM of the previous step has completed: all four tile buffers are free
          if (i >= 1) mbar_wait(bar(iQEmpty), (i - 1) & 1, wctx, kBbQEmpty);
          mbar_arrive_expect_tx(bar(iAFull), 4 * L::kTileBytes);
          for (int bx = 0; bx < L::kBoxes; ++bx) {
            const int x = col_other + bx * 64;
            tma_load_4d(k_s + bx * L::kBoxBytes, &tm_k, bar(iAFull), x, krow, wk.kv_head, wk.batch);
            tma_load_4d(q_s + bx * L::kBoxBytes, &tm_q, bar(iAFull), x, row, head, wk.batch);
            tma_load_4d(v_s + bx * L::kBoxBytes, &tm_v, bar(iAFull), x, krow, wk.kv_head, wk.batch);
            tma_load_4d(do_s + bx * L::kBoxBytes, &tm_do, bar(iAFull), x, row, head, wk.batch);
          }
          // the partial S^T and dP^T have read them: this CTA's own columns go over them
          mbar_wait(bar(iADone), i & 1, wctx, kBbADone);
          mbar_arrive_expect_tx(bar(iQFull), 2 * L::kTileBytes);
          for (int bx = 0; bx < L::kBoxes; ++bx) {
            const int x = col_own + bx * 64;
            tma_load_4d(k_s + bx * L::kBoxBytes, &tm_k, bar(iQFull), x, krow, wk.kv_head, wk.batch);
            tma_load_4d(q_s + bx * L::kBoxBytes, &tm_q, bar(iQFull), x, row, head, wk.batch);
          }
          mbar_arrive_expect_tx(bar(iDoFull), 2 * L::kTileBytes);
          for (int bx = 0; bx < L::kBoxes; ++bx) {
            const int x = col_own + bx * 64;
            tma_load_4d(v_s + bx * L::kBoxBytes, &tm_v, bar(iDoFull), x, krow, wk.kv_head, wk.batch);
            tma_load_4d(do_s + bx * L::kBoxBytes, &tm_do, bar(iDoFull), x, row, head, wk.batch);
          }
        }
      }
      __syncwarp();
    } else {
      if (lane == 0 && n_iter > 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_dq);
        mbar_arrive_expect_tx(bar(iKFull), L::kTileBytes);
        for (int bx = 0; bx < L::kBoxes; ++bx)
          tma_load_4d(sbase + L::kKOff + bx * L::kBoxBytes, &tm_k, bar(iKFull), bx * 64,
                      wk.k_row0 + kv0, wk.kv_head, wk.batch);
        mbar_arrive_expect_tx(bar(iVFull), L::kTileBytes);
        for (int bx = 0; bx < L::kBoxes; ++bx)
          tma_load_4d(sbase + L::kVOff + bx * L::kBoxBytes, &tm_v, bar(iVFull), bx * 64,
                      wk.k_row0 + kv0, wk.kv_head, wk.batch);
      }
      for (int i = 0; i < n_iter; ++i) {
        const int st = i % NS;
        const int head = wk.kv_head * group + i / nq;
        const int qt = qt0 + i % nq;
        const int row = wk.q_row0 + qt * kQTile;
        if (i >= NS) mbar_wait(bar(iQEmpty + st), ((i / NS) - 1) & 1, wctx, kBbQEmpty + st);
        if (lane == 0) {
          mbar_arrive_expect_tx(bar(iQFull + st), L::kTileBytes);
          for (int bx = 0; bx < L::kBoxes; ++bx)
            tma_load_4d(sbase + L::kQOff + st * L::kTileBytes + bx * L::kBoxBytes, &tm_q,
                        bar(iQFull + st), bx * 64, row, head, wk.batch);
        }
        // dO has a single buffer: it is reloaded as soon as dV of the previous step has read it.
        if (lane == 0) {
          if (i >= 1) mbar_wait(bar(iDoEmpty), (i - 1) & 1, wctx, kBbDoEmpty);
          mbar_arrive_expect_tx(bar(iDoFull), L::kTileBytes);
          for (int bx = 0; bx < L::kBoxes; ++bx)
            tma_load_4d(sbase + L::kDoOff + bx * L::kBoxBytes, &tm_do, bar(iDoFull), bx * 64, row, head,
                        wk.batch);
        }
        __syncwarp();
      }
    }
  } else if (warp == 14) {
    // ===================== per-row statistics: lse * log2(e) and delta ========
    for (int i = 0; i < n_iter; ++i) {
      const int st = i % NS;
      const int head = wk.kv_head * group + i / nq;
      const int qt = qt0 + i % nq;
      if (i >= NS) mbar_wait(bar(iQEmpty + st), ((i / NS) - 1) & 1, wctx, kBbQEmpty + st);
      float* stat = reinterpret_cast<float*>(sgen + L::kStatOff) + st * 2 * kQTile;
#pragma unroll
      for (int rr = 0; rr < kQTile / 32; ++rr) {
        const int r = lane + rr * 32;
        const int q_local = qt * kQTile + r;
        float lse2 = INFINITY;  // exp2(x - inf) = 0: rows past the sequence contribute nothing
        float dl = 0.f;
        if (q_local < wk.seqlen_q) {
          const int64_t grow = static_cast<int64_t>(wk.q_row0) + q_local;
          const float l = __ldg(p.lse + wk.batch * p.lse_strides.batch + head * p.lse_strides.head +
                                grow * p.lse_strides.row);
          if (l > -INFINITY) lse2 = l * kLog2e;
          dl = __ldg(p.delta + wk.batch * p.delta_batch_stride + head * p.delta_head_stride + grow);
        }
        stat[r] = lse2;
        stat[kQTile + r] = dl;
      }
      mbar_arrive(bar(iStatFull + st));
    }
  } else if (warp == 9) {
    // ===================== MMA issuer =========================================
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_st = make_idesc_f16(kKvTile, kQTile, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_dkv = make_idesc_f16(kKvTile, D, 0, 1);       // dV, dK
      constexpr uint32_t idesc_dq = make_idesc_f16(kQTile, D, 1, 1);         // dQ = dS K (queries on lanes)
      const uint32_t k_s = sbase + L::kKOff, v_s = sbase + L::kVOff, ds_s = sbase + L::kDsOff;
      // Descriptors are stepped with 32-bit adds on their low words (address field = addr >> 4).
      constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
      const uint32_t k_lo_k = smem_desc_lo(k_s, 16);                // K as K-major A of S^T
      const uint32_t v_lo_k = smem_desc_lo(v_s, 16);                // V as K-major A of dP^T
      const uint32_t k_lo_mn = smem_desc_lo(k_s, L::kBoxBytes);     // K^T, MN-major A of dQ^T
      const uint32_t ds_lo_k = smem_desc_lo(ds_s, 16);              // dS^T, K-major A of dK
      const uint32_t ds_lo_mn = smem_desc_lo(ds_s, L::kBoxBytes);   // dS^T, MN-major B of dQ^T

      // acc[128 keys x 128 queries] = X[keys x D] * Y[queries x D]^T, both head_dim-contiguous
      auto issue_xyT = [&](uint32_t d_col, uint32_t x_lo, uint32_t y_s, bool accumulate = false) {
        const uint32_t y_lo = smem_desc_lo(y_s, 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * L::kBoxBytes + (ks & 3) * 32) >> 4;
          umma_ss(tmem_base + d_col, smem_desc_join(x_lo + off, kHi), smem_desc_join(y_lo + off, kHi),
                  idesc_st, (accumulate || ks > 0) ? 1u : 0u);
        }
      };

      if constexpr (!SPLIT) {
        mbar_wait(bar(iKFull), 0, wctx, kBbKFull);
        mbar_wait(bar(iQFull + 0), 0, wctx, kBbQFull);
        tc_fence_after_sync();
        issue_xyT(kColS, k_lo_k, sbase + L::kQOff);
        tc_commit(bar(iSReady));
        mbar_wait(bar(iVFull), 0, wctx, kBbVFull);
        mbar_wait(bar(iDoFull), 0, wctx, kBbDoFull);
        tc_fence_after_sync();
        issue_xyT(kColDpq, v_lo_k, sbase + L::kDoOff);
        tc_commit(bar(iDpReady));
      }
      const uint32_t do_lo_mn = smem_desc_lo(sbase + L::kDoOff, L::kBoxBytes);

      for (int i = 0; i < n_iter; ++i) {
        const int st = i % NS;
        const int st1 = (i + 1) % NS;
        const uint32_t q_lo_mn = smem_desc_lo(sbase + L::kQOff + st * L::kTileBytes, L::kBoxBytes);
        if constexpr (SPLIT) {
          // S^T(i) and dP^T(i) in two parts: the other column half first, then this CTA's own, which
          // stays in the tile buffers for dV, dK and dQ.  S^T goes over P^T(i-1), which dV(i-1)
          // -- issued before -- has read; dP^T goes over dQ(i-1), which the write-back warps must
          // have read out.
          mbar_wait(bar(iAFull), i & 1, wctx, kBbAFull);
          tc_fence_after_sync();
          issue_xyT(kColS, k_lo_k, sbase + L::kQOff);
          if (i >= 1) {
            mbar_wait(bar(iDqFree), (i - 1) & 1, wctx, kBbDqFree);
            tc_fence_after_sync();
          }
          issue_xyT(kColDpq, v_lo_k, sbase + L::kDoOff);
          tc_commit(bar(iADone));
          mbar_wait(bar(iQFull), i & 1, wctx, kBbQFull);
          tc_fence_after_sync();
          issue_xyT(kColS, k_lo_k, sbase + L::kQOff, true);
          tc_commit(bar(iSReady));
          mbar_wait(bar(iDoFull), i & 1, wctx, kBbDoFull);
          tc_fence_after_sync();
          issue_xyT(kColDpq, v_lo_k, sbase + L::kDoOff, true);
          tc_commit(bar(iDpReady));
        }
        // dV += P^T(i) dO(i): P^T as packed fp16 in TMEM; query columns [0,64) at +0, [64,128) at +64
        mbar_wait(bar(iPReady), i & 1, wctx, kBbPReady);
        tc_fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < kQTile / 16; ++ks) {
          const uint32_t a_col = kColS + (ks >> 2) * 64 + (ks & 3) * 8;
          umma_ts(tmem_base + kColDv, tmem_base + a_col,
                  smem_desc_join(do_lo_mn + ((ks * 2048) >> 4), kHi), idesc_dkv,
                  (i > 0 || ks > 0) ? 1u : 0u);
        }
        tc_commit(bar(iDoEmpty));  // dO(i) has no reader left once dV(i) is done
        // S^T(i+1) overwrites P^T(i): issued after dV(i), which reads it.
        if (!SPLIT && i + 1 < n_iter) {
          mbar_wait(bar(iQFull + st1), ((i + 1) / NS) & 1, wctx, kBbQFull + st1);
          tc_fence_after_sync();
          issue_xyT(kColS, k_lo_k, sbase + L::kQOff + st1 * L::kTileBytes);
          tc_commit(bar(iSReady));
        }
        mbar_wait(bar(iDsReady), i & 1, wctx, kBbDsReady);
        tc_fence_after_sync();
        // dK += dS^T(i) Q(i)
        auto issue_dk = [&]() {
#pragma unroll
          for (int ks = 0; ks < kQTile / 16; ++ks) {
            const uint32_t a_off = ((ks >> 2) * L::kBoxBytes + (ks & 3) * 32) >> 4;
            umma_ss(tmem_base + kColDk, smem_desc_join(ds_lo_k + a_off, kHi),
                    smem_desc_join(q_lo_mn + ((ks * 2048) >> 4), kHi), idesc_dkv,
                    (i > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(bar(iQEmpty + st));  // Q(i) has no reader left once dK(i) is done
        };
        // dQ(i) = dS(i) K: the dS^T buffer read as an M-contiguous A operand; the result (queries on
        // the lanes, head_dim on the columns) goes into the columns of the consumed dP^T(i)
        auto issue_dq = [&]() {
#pragma unroll
          for (int ks = 0; ks < kKvTile / 16; ++ks) {
            umma_ss(tmem_base + kColDpq, smem_desc_join(ds_lo_mn + ((ks * 2048) >> 4), kHi),
                    smem_desc_join(k_lo_mn + ((ks * 2048) >> 4), kHi), idesc_dq, ks > 0 ? 1u : 0u);
          }
          tc_commit(bar(iDqReady));
        };
#if FAL_BWD_DQ_FIRST
        issue_dq();
        issue_dk();
#else
        issue_dk();
        issue_dq();
#endif
        tc_commit(bar(iDsFree));  // both readers of the dS^T buffer are done
        // dP^T(i+1) goes where dQ(i) is: the write-back warps must have read it out first.
        if (!SPLIT && i + 1 < n_iter) {
          mbar_wait(bar(iDoFull), (i + 1) & 1, wctx, kBbDoFull);
          mbar_wait(bar(iDqFree), i & 1, wctx, kBbDqFree);
          tc_fence_after_sync();
          issue_xyT(kColDpq, v_lo_k, sbase + L::kDoOff);
          tc_commit(bar(iDpReady));
        }
      }
      tc_commit(bar(iAllDone));
    }
    __syncwarp();
  } else if (warp < 8) {
    // ===================== compute ============================================
    const int quarter = warp & 3;
    const int half = warp >> 2;                       // query columns [64*half, 64*half+64)
    const int kv_row = quarter * 32 + lane;           // key row inside the tile (= TMEM lane)
    const int kv_local = kv0 + kv_row;
    const bool kv_ok = kv_local < wk.seqlen_k;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c2 = p.scale_log2;
    // this thread's dS^T row: box `half` (64 query columns = 128 bytes per key row)
    uint8_t* ds_row = sgen + L::kDsOff + half * L::kBoxBytes + kv_row * 128;

    for (int i = 0; i < n_iter; ++i) {
      const int st = i % NS;
      const int qt = qt0 + i % nq;
      const int q_col0 = qt * kQTile + half * 64;  // local query index of this thread's first column
      const float* stat = reinterpret_cast<const float*>(sgen + L::kStatOff) + st * 2 * kQTile + half * 64;
      const bool tile_mask = !kv_ok || (CAUSAL && (kv0 + kKvTile - 1 > qt * kQTile + cshift));

      mbar_wait(bar(iStatFull + st), (i / NS) & 1, wctx, kBbStatFull + st);
      mbar_wait(bar(iSReady), i & 1, wctx, kBbSReady);
      tc_fence_after_sync();

      // ---- P^T = exp2(S^T * c2 - lse2), kept as packed fp16 for the dS step ----
      uint32_t pk[32];
      {
        uint32_t r[2][32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColS + half * 64, r[0]);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColS + half * 64 + 32, r[1]);
        tmem_wait_ld();
        if (tile_mask) {  // hidden scores become -inf before the exponential (exp2(-inf) = 0)
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const bool vis = kv_ok && (!CAUSAL || kv_local <= q_col0 + cshift + c * 32 + j);
              r[c][j] = vis ? r[c][j] : 0xff800000u;
            }
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(stat + c * 32 + j);
#ifdef FAL_BWD_EXP_F16X2
            // exponent rounded to fp16 first, two exponentials per MUFU instruction
            pk[c * 16 + (j >> 1) + 0] = exp2_f16x2(pack_half2(fmaf(__uint_as_float(r[c][j + 0]), c2, -l4.x),
                                                              fmaf(__uint_as_float(r[c][j + 1]), c2, -l4.y)));
            pk[c * 16 + (j >> 1) + 1] = exp2_f16x2(pack_half2(fmaf(__uint_as_float(r[c][j + 2]), c2, -l4.z),
                                                              fmaf(__uint_as_float(r[c][j + 3]), c2, -l4.w)));
#else
            const float p0 = bwd_exp2<0>(j, fmaf(__uint_as_float(r[c][j + 0]), c2, -l4.x));
            const float p1 = bwd_exp2<1>(j, fmaf(__uint_as_float(r[c][j + 1]), c2, -l4.y));
            const float p2 = bwd_exp2<2>(j, fmaf(__uint_as_float(r[c][j + 2]), c2, -l4.z));
            const float p3 = bwd_exp2<3>(j, fmaf(__uint_as_float(r[c][j + 3]), c2, -l4.w));
            pk[c * 16 + (j >> 1) + 0] = pack_half2(p0, p1);
            pk[c * 16 + (j >> 1) + 1] = pack_half2(p2, p3);
#endif
          }
        }
        // P^T overwrites this thread's own S^T columns: 32 packed columns at [64*half, 64*half+32)
        tmem_st_32x32b_x32(tmem_base + lane_addr + kColS + half * 64, pk);
        tmem_wait_st();
      }
      tc_fence_before_sync();
#if FAL_BWD_ELECT_ARRIVE
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(iPReady));
#else
      mbar_arrive(bar(iPReady));
#endif

      // ---- dS^T = P^T o (dP^T - delta) ------------------------------------------
      mbar_wait(bar(iDpReady), i & 1, wctx, kBbDpReady);
      tc_fence_after_sync();
      uint32_t dsp[32];
      {
        uint32_t r[2][32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + half * 64, r[0]);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + half * 64 + 32, r[1]);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            // (dP - delta) in fp32 (it cancels), rounded to fp16, then one packed multiply by the
            // fp16 P: the product is the fp16 dS the GEMMs consume.
            const float4 d4 = *reinterpret_cast<const float4*>(stat + kQTile + c * 32 + j);
            const uint32_t e0 = pack_half2(__uint_as_float(r[c][j + 0]) - d4.x, __uint_as_float(r[c][j + 1]) - d4.y);
            const uint32_t e1 = pack_half2(__uint_as_float(r[c][j + 2]) - d4.z, __uint_as_float(r[c][j + 3]) - d4.w);
            dsp[c * 16 + (j >> 1) + 0] = hmul2_bits(pk[c * 16 + (j >> 1) + 0], e0);
            dsp[c * 16 + (j >> 1) + 1] = hmul2_bits(pk[c * 16 + (j >> 1) + 1], e1);
          }
        }
      }
      if (i > 0) mbar_wait(bar(iDsFree), (i - 1) & 1, wctx, kBbDqReady);
      // dS^T row -> shared memory, 128-byte XOR swizzle (16-byte chunk index ^ row % 8)
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        *reinterpret_cast<uint4*>(ds_row + ((c ^ (kv_row & 7)) << 4)) =
            make_uint4(dsp[4 * c + 0], dsp[4 * c + 1], dsp[4 * c + 2], dsp[4 * c + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
#if FAL_BWD_ELECT_ARRIVE
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(iDsReady));
#else
      mbar_arrive(bar(iDsReady));
#endif
    }

    // ---- epilogue: dV (warps 0-3) and dK (warps 4-7) -------------------------
    if (n_iter > 0) {
      mbar_wait(bar(iAllDone), 0, wctx, kBbAllDone);
      tc_fence_after_sync();
    }
    const bool is_dk = half == 1;
    const RowStrides& st_o = is_dk ? p.dk_strides : p.dv_strides;
    const int64_t out_off = wk.batch * st_o.batch + wk.kv_head * st_o.head +
                            (static_cast<int64_t>(wk.k_row0) + kv_local) * st_o.row + col_own;
    __half* out_row = static_cast<__half*>(is_dk ? p.dk : p.dv) + out_off;
    float* out_row32 = p.dk_f32 != nullptr ? (is_dk ? p.dk_f32 : p.dv_f32) + out_off : nullptr;
    const float mul = is_dk ? p.scale : 1.f;
    const uint32_t t_acc = tmem_base + lane_addr + (is_dk ? kColDk : kColDv);
    // Whole tiles leave through shared memory (the K buffer for dK, the V buffer for dV: every MMA that
    // read them has completed) and TMA stores: a thread owns a key row, and 32 threads storing 16
    // bytes each into 32 different rows of global memory is what takes microseconds here otherwise.
    // A packed sequence's last, partial tile keeps the row-by-row path (the rows behind it belong to
    // the next sequence, which a tile store would overwrite), and so do the fp32 partials.
    const bool by_tma = p.store_by_tma != 0 && out_row32 == nullptr &&
                        (p.cu_k == nullptr || wk.seqlen_k - kv0 >= kKvTile);
    uint8_t* stage_row = sgen + (is_dk ? L::kKOff : L::kVOff) + kv_row * 128;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      if (n_iter > 0) {
        tmem_ld_32x32b_x32(t_acc + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (by_tma) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 out;
          out.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * mul, __uint_as_float(r[v * 8 + 1]) * mul);
          out.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * mul, __uint_as_float(r[v * 8 + 3]) * mul);
          out.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * mul, __uint_as_float(r[v * 8 + 5]) * mul);
          out.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * mul, __uint_as_float(r[v * 8 + 7]) * mul);
          // box c / 2, 16-byte chunk (c % 2) * 4 + v of the row, 128-byte XOR swizzle
          *reinterpret_cast<uint4*>(stage_row + (c >> 1) * L::kBoxBytes + ((((c & 1) * 4 + v) ^ (kv_row & 7)) << 4)) = out;
        }
      } else if (kv_ok && out_row32 != nullptr) {
        // unrounded partial for a caller that sums the key shard's gradient over several calls
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<float4*>(out_row32 + c * 32 + v * 4) =
              make_float4(__uint_as_float(r[v * 4 + 0]) * mul, __uint_as_float(r[v * 4 + 1]) * mul,
                          __uint_as_float(r[v * 4 + 2]) * mul, __uint_as_float(r[v * 4 + 3]) * mul);
      } else if (kv_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          if (col_own + c * 32 + v * 8 >= p.head_dim) continue;  // head_dim 32 / 96: no such column
          uint4 out;
          out.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * mul, __uint_as_float(r[v * 8 + 1]) * mul);
          out.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * mul, __uint_as_float(r[v * 8 + 3]) * mul);
          out.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * mul, __uint_as_float(r[v * 8 + 5]) * mul);
          out.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * mul, __uint_as_float(r[v * 8 + 7]) * mul);
          *reinterpret_cast<uint4*>(out_row + c * 32 + v * 8) = out;
        }
      }
    }
    if (by_tma) {  // uniform over the CTA
      fence_proxy_async_smem();
      named_barrier_sync(2 + half, 128);
      if (quarter == 0 && lane == 0) {
        const uint32_t src = sbase + (is_dk ? L::kKOff : L::kVOff);
        for (int bx = 0; bx < L::kBoxes; ++bx)
          tma_store_4d(is_dk ? &tm_dk : &tm_dv, src + bx * L::kBoxBytes, col_own + bx * 64, wk.k_row0 + kv0,
                       wk.kv_head, wk.batch);
        bulk_commit_group();
        bulk_wait_group_read<0>();  // the boxes must have been read before the CTA's shared memory goes away
      }
    }
  } else if (warp < 14) {
    // ===================== dQ write-back ======================================
    // dQ tile: TMEM lane = query row, column = head_dim.  It leaves in 64-column halves.  For each
    // half a thread reads its row's 64 values, writes them as two 32-float slices into the two
    // swizzled [128 rows][128 bytes] staging boxes, and one thread issues two TMA tensor reductions
    // that add the boxes to the fp32 accumulator.  The second half is pulled into registers (and the
    // TMEM columns handed back to the issuer) before waiting for the first half's reductions.
    const int quarter = warp & 3;
    const int qrow = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const bool issuer = warp == 10 && lane == 0;
    uint8_t* box_row = sgen + L::kStageOff + qrow * 128;
    for (int i = 0; i < n_iter; ++i) {
      const int head = wk.kv_head * group + i / nq;
      const int qt = qt0 + i % nq;
      mbar_wait(bar(iDqReady), i & 1, wctx, kBbDqReady);
      tc_fence_after_sync();
      const int grow = wk.q_row0 + qt * kQTile;  // accumulator row of the tile's first query
#pragma unroll
      for (int hf = 0; hf < D / 64; ++hf) {
        uint32_t r[2][32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + hf * 64, r[0]);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + hf * 64 + 32, r[1]);
        tmem_wait_ld();
        if (hf == D / 64 - 1) {  // everything is in registers: the issuer may overwrite the columns
          tc_fence_before_sync();
          mbar_arrive(bar(iDqFree));
        }
        // Earlier reductions must be done reading the staging boxes.
        if (issuer) bulk_wait_group_read<0>();
        named_barrier_sync(1, 128);
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int v = 0; v < 8; ++v)
            *reinterpret_cast<uint4*>(box_row + c * L::kBoxBytes + ((v ^ (qrow & 7)) << 4)) =
                make_uint4(r[c][4 * v + 0], r[c][4 * v + 1], r[c][4 * v + 2], r[c][4 * v + 3]);
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (issuer) {
          tma_reduce_add_4d(&tm_dq, sbase + L::kStageOff, col_own + hf * 64, grow, head, wk.batch);
          tma_reduce_add_4d(&tm_dq, sbase + L::kStageOff + L::kBoxBytes, col_own + hf * 64 + 32, grow, head,
                            wk.batch);
          bulk_commit_group();
        }
      }
    }
    if (issuer) bulk_wait_group0();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------
// Pre-pass: delta[row] = sum_d dO*O  (precompute_D_kernel, bwd.cu:76-107 of the reference) and
// the zeroing of the fp32 dQ accumulator (dQ_fp32 = zeros at csrc/flash_attn_legacy.cpp:126).
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256) fal_bwd_prep_kernel(const BwdPrepParams p) {
  constexpr int kLanesPerRow = D / 8;
  constexpr int kRowsPerBlock = 256 / kLanesPerRow;
  const int sub = threadIdx.x % kLanesPerRow;
  const int64_t row_id = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + threadIdx.x / kLanesPerRow;
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.rows;
  float acc = 0.f;
  int b = 0, h = 0, r = 0;
  const bool ok = row_id < total;
  if (ok) {
    r = static_cast<int>(row_id % p.rows);
    const int64_t bh = row_id / p.rows;
    h = static_cast<int>(bh % p.heads_q);
    b = static_cast<int>(bh / p.heads_q);
    const __half* o = static_cast<const __half*>(p.o) + b * p.o_strides.batch + h * p.o_strides.head +
                      static_cast<int64_t>(r) * p.o_strides.row + sub * 8;
    const __half* d_o = static_cast<const __half*>(p.d_o) + b * p.do_strides.batch +
                        h * p.do_strides.head + static_cast<int64_t>(r) * p.do_strides.row + sub * 8;
    uint4 ov = make_uint4(0u, 0u, 0u, 0u), dv = ov;
    if (sub * 8 < p.head_dim_real) {  // head_dim 32 / 96: the columns beyond it do not exist
      ov = *reinterpret_cast<const uint4*>(o);
      dv = *reinterpret_cast<const uint4*>(d_o);
    }
    const __half2* oh = reinterpret_cast<const __half2*>(&ov);
    const __half2* dh = reinterpret_cast<const __half2*>(&dv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __half22float2(oh[j]);
      const float2 g = __half22float2(dh[j]);
      acc = fmaf(a.x, g.x, acc);
      acc = fmaf(a.y, g.y, acc);
    }
  }
#pragma unroll
  for (int off = kLanesPerRow / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (ok && sub == 0) p.delta[b * p.delta_batch_stride + h * p.delta_head_stride + r] = acc;
  // The fp32 dQ accumulator must start at zero (the main kernel only ever adds to it): this thread
  // clears the 8 columns of the row it has just read from O and dO.  Rows between p.rows and the
  // padded row count may be added into by partial tiles but are never read, so they stay as they are.
  if (ok && p.dq_accum != nullptr) {  // (a caller-owned accumulator that is being continued is left alone)
    float4* acc_row = reinterpret_cast<float4*>(p.dq_accum + b * p.dq_accum_batch_stride +
                                                h * p.dq_accum_head_stride + static_cast<int64_t>(r) * D + sub * 8);
    acc_row[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    acc_row[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// ---------------------------------------------------------------------------
// Post-pass: dQ = fp16(scale * accumulator)  (csrc/flash_attn_legacy.cpp:184 of the reference).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fal_bwd_post_kernel(const BwdPostParams p) {
  const int chunks = p.head_dim_real / 8;  // only the columns the tensors have
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.rows * chunks;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % chunks);
  const int64_t row_id = idx / chunks;
  const int r = static_cast<int>(row_id % p.rows);
  const int64_t bh = row_id / p.rows;
  const int h = static_cast<int>(bh % p.heads_q);
  const int b = static_cast<int>(bh / p.heads_q);
  const float* src = p.dq_accum + b * p.dq_accum_batch_stride + h * p.dq_accum_head_stride +
                     static_cast<int64_t>(r) * p.head_dim + c * 8;
  const float4 x = *reinterpret_cast<const float4*>(src);
  const float4 y = *reinterpret_cast<const float4*>(src + 4);
  uint4 out;
  out.x = pack_half2(x.x * p.scale, x.y * p.scale);
  out.y = pack_half2(x.z * p.scale, x.w * p.scale);
  out.z = pack_half2(y.x * p.scale, y.y * p.scale);
  out.w = pack_half2(y.z * p.scale, y.w * p.scale);
  __half* dst = static_cast<__half*>(p.dq) + b * p.dq_strides.batch + h * p.dq_strides.head +
                static_cast<int64_t>(r) * p.dq_strides.row + c * 8;
  *reinterpret_cast<uint4*>(dst) = out;
}

template <int D, bool CAUSAL, bool SPLIT = false>
cudaError_t launch_bwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const CUtensorMap& tdq, const CUtensorMap& tdk,
                         const CUtensorMap& tdv, const BwdParams& p, int grid, cudaStream_t stream) {
  auto kern = fal_bwd_kernel<D, CAUSAL, SPLIT>;
  static DeviceOnce configured;
  cudaError_t e = configured.run([&] {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                BwdSmem<D>::kAllocBytes);
  });
  if (e != cudaSuccess) return e;
  if (SPLIT && grid > 0x3fffffff) return cudaErrorInvalidValue;
  kern<<<SPLIT ? 2 * grid : grid, kBwdThreads, BwdSmem<D>::kAllocBytes, stream>>>(tq, tk, tv, tdo, tdq, tdk, tdv, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_prep(const BwdPrepParams& p, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.rows;
  if (p.head_dim == 256) {
    const int64_t blocks = (total + 7) / 8;
    fal_bwd_prep_kernel<256><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  } else if (p.head_dim == 128) {
    const int64_t blocks = (total + 15) / 16;
    fal_bwd_prep_kernel<128><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  } else if (p.head_dim == 64) {
    const int64_t blocks = (total + 31) / 32;
    fal_bwd_prep_kernel<64><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_bwd(int head_dim, bool causal, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdq,
                       const CUtensorMap& tdk, const CUtensorMap& tdv, const BwdParams& p, int grid,
                       cudaStream_t stream) {
  if (head_dim == 128) {
    return causal ? launch_bwd_t<128, true>(tq, tk, tv, tdo, tdq, tdk, tdv, p, grid, stream)
                  : launch_bwd_t<128, false>(tq, tk, tv, tdo, tdq, tdk, tdv, p, grid, stream);
  }
  if (head_dim == 64) {
    return causal ? launch_bwd_t<64, true>(tq, tk, tv, tdo, tdq, tdk, tdv, p, grid, stream)
                  : launch_bwd_t<64, false>(tq, tk, tv, tdo, tdq, tdk, tdv, p, grid, stream);
  }
  if (head_dim == 256) {  // two CTAs per key tile, 128 output columns each
    return causal ? launch_bwd_t<128, true, true>(tq, tk, tv, tdo, tdq, tdk, tdv, p, grid, stream)
                  : launch_bwd_t<128, false, true>(tq, tk, tv, tdo, tdq, tdk, tdv, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_bwd_post(const BwdPostParams& p, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.rows * (p.head_dim_real / 8);
  const int64_t blocks = (total + 255) / 256;
  fal_bwd_post_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fal
