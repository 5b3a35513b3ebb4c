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
// Everything is computed transposed, keys on the 128 TMEM lanes:
//   S^T  = K Q^T      (M=128 keys, N=64 queries, K=head_dim)   smem x smem
//   dP^T = V dO^T     (same shape)                             smem x smem
//   dV  += P^T dO     (M=128, N=head_dim, K=64)                TMEM x smem
//   dK  += dS^T Q     (M=128, N=head_dim, K=64)                smem x smem
//   dQ^T = K^T dS^T   (M=head_dim, N=64, K=128)                smem x smem
// so P^T is produced in place over S^T, each compute thread owns one key row,
// and dS^T is written to shared memory once and serves both dK and dQ.
// dQ^T tiles leave through a shared-memory transpose and one bulk fp32
// add-reduction per tile into the accumulator that the post-pass casts.
//
//   warps 0-7    compute (two per TMEM lane quarter, 32 query columns each)
//   warp  8      TMA producer, LSE / delta staging
//   warp  9      tcgen05.mma issuer, TMEM owner
//   warps 10-13  dQ tile write-back
//
// TMEM columns: S^T/P^T x2 [0,128), dP^T/dQ^T x2 [128,256) (dQ^T of a step reuses the
//               columns of that step's consumed dP^T), dV [256,256+D), dK [256+D,256+2D).
// Q/dO tiles and their row statistics go through a 3-deep shared-memory ring, and the
// issuer runs S^T and dP^T one step ahead of the compute warps.
#define FAL_WAIT_SLOW_PATH_INLINE  // measured: the out-of-line wait path is slower for this kernel
#include "fal_common.h"
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

constexpr int kBwdThreads = 448;
constexpr int kKvTile = 128;
constexpr int kQTile = 64;
constexpr float kLog2e = 1.4426950408889634f;

enum BwdBarrier : int {
  kBbKFull = 100, kBbVFull = 101, kBbQFull = 110, kBbDoFull = 120, kBbStatFull = 130,
  kBbStageEmpty = 140, kBbSReady = 150, kBbDpReady = 160, kBbPReady = 161, kBbDsReady = 162,
  kBbDsFree = 163, kBbDqReady = 164, kBbDqFree = 165, kBbAllDone = 166,
};

template <int D>
struct BwdSmem {
  static constexpr int kStages = 3;                            // Q / dO / statistics ring depth
  static constexpr int kBoxes = D / 64;
  static constexpr int kKvBoxBytes = kKvTile * 128;
  static constexpr int kKvTileBytes = kBoxes * kKvBoxBytes;
  static constexpr int kQBoxBytes = kQTile * 128;
  static constexpr int kQTileBytes = kBoxes * kQBoxBytes;
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kKvTileBytes;
  static constexpr int kQOff = 2 * kKvTileBytes;
  static constexpr int kDoOff = kQOff + kStages * kQTileBytes;
  static constexpr int kDsOff = kDoOff + kStages * kQTileBytes;  // [128 keys][64 queries] fp16
  static constexpr int kDsBytes = kKvTile * 128;
  static constexpr int kDqOff = kDsOff + kDsBytes;               // [64 queries][D] fp32
  static constexpr int kDqBytes = kQTile * D * 4;
  static constexpr int kStatOff = kDqOff + kDqBytes;             // per stage: lse2[64], delta[64]
  static constexpr int kStatBytes = kStages * 2 * kQTile * 4;
  static constexpr int kBarOff = kStatOff + kStatBytes;
  // k_full v_full q_full[3] do_full[3] stat_full[3] stage_empty[3] s_ready[2] dp_ready[2]
  // dq_ready[2] dq_free[2] p_ready ds_ready ds_free all_done
  static constexpr int kNumBars = 2 + 4 * kStages + 8 + 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kBytes = kMiscOff + 16;
  static constexpr int kAllocBytes = kBytes + 1024;
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

__device__ __forceinline__ bool bwd_decode_work(const BwdParams& p, BwdWork& w) {
  const int idx = blockIdx.x;
  if (p.cu_k == nullptr) {
    const int bh_count = p.batch * p.heads_kv;
    w.kvblk = idx / bh_count;  // first key blocks first: under a causal mask they see the most queries
    const int bh = idx % bh_count;
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
  int first = 0;
  for (int s = 0; s < p.num_seqs; ++s) {
    const int a = __ldg(p.cu_k + s);
    const int e = __ldg(p.cu_k + s + 1);
    const int nblk = (e - a + kKvTile - 1) / kKvTile;
    if (slot < first + nblk) {
      w.kvblk = slot - first;
      w.k_row0 = a;
      w.seqlen_k = e - a;
      w.q_row0 = __ldg(p.cu_q + s);
      w.seqlen_q = __ldg(p.cu_q + s + 1) - w.q_row0;
      return true;
    }
    first += nblk;
  }
  return false;
}

// Tuning aid, compiled in only with -DFAL_BWD_TIMING: cycles each role spends in each wait.
#ifdef FAL_BWD_TIMING
__device__ unsigned long long g_bwd_wait_cycles[32];
#define BWD_WAIT(slot, ...)                           \
  do {                                                \
    const long long _t0 = clock64();                  \
    mbar_wait(__VA_ARGS__);                           \
    tacc[slot] += clock64() - _t0;                    \
  } while (0)
#define BWD_TIMING_ONLY(x) x
#else
#define BWD_WAIT(slot, ...) mbar_wait(__VA_ARGS__)
#define BWD_TIMING_ONLY(x)
#endif

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <int D, bool CAUSAL>
__global__ void __launch_bounds__(kBwdThreads, 1)
fal_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
               const BwdParams p) {
  using L = BwdSmem<D>;

  BwdWork wk;
  if (!bwd_decode_work(p, wk)) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));
  const uint32_t bar0 = sbase + L::kBarOff;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  constexpr int NS = L::kStages;
  constexpr int iKFull = 0, iVFull = 1, iQFull = 2, iDoFull = 2 + NS, iStatFull = 2 + 2 * NS,
                iStageEmpty = 2 + 3 * NS, iSReady = 2 + 4 * NS, iDpReady = iSReady + 2,
                iDqReady = iSReady + 4, iDqFree = iSReady + 6, iPReady = iSReady + 8,
                iDsReady = iSReady + 9, iDsFree = iSReady + 10, iAllDone = iSReady + 11;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kMiscOff + 4);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  BWD_TIMING_ONLY(long long tacc[24] = {}; const long long t_cta0 = clock64();)

  const int group = p.heads_q / p.heads_kv;
  const int kv0 = wk.kvblk * kKvTile;                       // local index of the tile's first key
  const int nqt = (wk.seqlen_q + kQTile - 1) / kQTile;
  const int qt0 = CAUSAL ? min(kv0 / kQTile, nqt) : 0;      // first query tile that sees this key tile
  const int nq = nqt - qt0;                                  // query tiles per head
  const int n_iter = group * nq;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar(iKFull), 1);
    mbar_init(bar(iVFull), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(iQFull + s), 1);
      mbar_init(bar(iDoFull + s), 1);
      mbar_init(bar(iStatFull + s), 32);
      mbar_init(bar(iStageEmpty + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(iSReady + s), 1);
      mbar_init(bar(iDpReady + s), 1);
      mbar_init(bar(iDqReady + s), 1);
      mbar_init(bar(iDqFree + s), 128);
    }
    mbar_init(bar(iPReady), 256);
    mbar_init(bar(iDsReady), 256);
    mbar_init(bar(iDsFree), 1);
    mbar_init(bar(iAllDone), 1);
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
    // ===================== producer: TMA + per-row statistics =================
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      mbar_arrive_expect_tx(bar(iKFull), L::kKvTileBytes);
      for (int bx = 0; bx < L::kBoxes; ++bx)
        tma_load_4d(sbase + L::kKOff + bx * L::kKvBoxBytes, &tm_k, bar(iKFull), bx * 64,
                    wk.k_row0 + kv0, wk.kv_head, wk.batch);
      mbar_arrive_expect_tx(bar(iVFull), L::kKvTileBytes);
      for (int bx = 0; bx < L::kBoxes; ++bx)
        tma_load_4d(sbase + L::kVOff + bx * L::kKvBoxBytes, &tm_v, bar(iVFull), bx * 64,
                    wk.k_row0 + kv0, wk.kv_head, wk.batch);
    }
    for (int i = 0; i < n_iter; ++i) {
      const int st = i % NS;
      const int head = wk.kv_head * group + i / nq;
      const int qt = qt0 + i % nq;
      if (i >= NS) BWD_WAIT(0, bar(iStageEmpty + st), ((i / NS) - 1) & 1, wctx, kBbStageEmpty + st);
      if (lane == 0) {
        const int row = wk.q_row0 + qt * kQTile;
        mbar_arrive_expect_tx(bar(iQFull + st), L::kQTileBytes);
        for (int bx = 0; bx < L::kBoxes; ++bx)
          tma_load_4d(sbase + L::kQOff + st * L::kQTileBytes + bx * L::kQBoxBytes, &tm_q,
                      bar(iQFull + st), bx * 64, row, head, wk.batch);
        mbar_arrive_expect_tx(bar(iDoFull + st), L::kQTileBytes);
        for (int bx = 0; bx < L::kBoxes; ++bx)
          tma_load_4d(sbase + L::kDoOff + st * L::kQTileBytes + bx * L::kQBoxBytes, &tm_do,
                      bar(iDoFull + st), bx * 64, row, head, wk.batch);
      }
      float* stat = reinterpret_cast<float*>(sgen + L::kStatOff) + st * 2 * kQTile;
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
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
      constexpr uint32_t idesc_dq = make_idesc_f16(128, kQTile, 1, 1);       // dQ^T
      const uint32_t k_s = sbase + L::kKOff, v_s = sbase + L::kVOff, ds_s = sbase + L::kDsOff;

      // Descriptors are stepped with 32-bit adds on their low words (address field = addr >> 4).
      constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
      const uint32_t k_lo_k = smem_desc_lo(k_s, 16);                    // K as K-major operand
      const uint32_t v_lo_k = smem_desc_lo(v_s, 16);                    // V as K-major operand
      const uint32_t k_lo_mn = smem_desc_lo(k_s, L::kKvBoxBytes);       // K^T (MN-major A of dQ^T)
      const uint32_t ds_lo_k = smem_desc_lo(ds_s, 16);                  // dS^T as K-major A of dK
      const uint32_t ds_lo_mn = smem_desc_lo(ds_s, 16);                 // dS^T as MN-major B of dQ^T

      // acc[128 keys x 64 queries] = X[keys x D] * Y[queries x D]^T, both head_dim-contiguous
      auto issue_xyT = [&](uint32_t d_col, uint32_t x_lo, uint32_t y_s) {
        const uint32_t y_lo = smem_desc_lo(y_s, 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          umma_ss(tmem_base + d_col,
                  smem_desc_join(x_lo + (((ks >> 2) * L::kKvBoxBytes + (ks & 3) * 32) >> 4), kHi),
                  smem_desc_join(y_lo + (((ks >> 2) * L::kQBoxBytes + (ks & 3) * 32) >> 4), kHi),
                  idesc_st, ks > 0 ? 1u : 0u);
        }
      };

      // S^T and dP^T run one step ahead of the compute warps; each has two TMEM buffers.
      mbar_wait(bar(iKFull), 0, wctx, kBbKFull);
      mbar_wait(bar(iQFull + 0), 0, wctx, kBbQFull);
      tc_fence_after_sync();
      issue_xyT(kColS, k_lo_k, sbase + L::kQOff);
      tc_commit(bar(iSReady + 0));
      mbar_wait(bar(iVFull), 0, wctx, kBbVFull);
      mbar_wait(bar(iDoFull + 0), 0, wctx, kBbDoFull);
      tc_fence_after_sync();
      issue_xyT(kColDpq, v_lo_k, sbase + L::kDoOff);
      tc_commit(bar(iDpReady + 0));

      for (int i = 0; i < n_iter; ++i) {
        const int st = i % NS;
        const int sb = i & 1;
        const int st1 = (i + 1) % NS;
        const int sb1 = (i + 1) & 1;
        const uint32_t q_lo_mn = smem_desc_lo(sbase + L::kQOff + st * L::kQTileBytes, L::kQBoxBytes);
        const uint32_t do_lo_mn = smem_desc_lo(sbase + L::kDoOff + st * L::kQTileBytes, L::kQBoxBytes);
        // S^T(i+1): its buffer held P^T(i-1), which dV(i-1) (issued earlier) has read by then.
        if (i + 1 < n_iter) {
          BWD_WAIT(1, bar(iQFull + st1), ((i + 1) / NS) & 1, wctx, kBbQFull + st1);
          tc_fence_after_sync();
          BWD_TIMING_ONLY(const long long t_a = clock64();)
          issue_xyT(kColS + sb1 * kQTile, k_lo_k, sbase + L::kQOff + st1 * L::kQTileBytes);
          BWD_TIMING_ONLY(tacc[16] += clock64() - t_a;)
          tc_commit(bar(iSReady + sb1));
          BWD_TIMING_ONLY(tacc[20] += clock64() - t_a;)
        }
        // dV += P^T(i) dO(i): P^T as fp16 in TMEM, query columns [0,32) at +0, [32,64) at +32
        BWD_WAIT(2, bar(iPReady), i & 1, wctx, kBbPReady);
        tc_fence_after_sync();
        BWD_TIMING_ONLY(const long long t_b = clock64();)
#pragma unroll
        for (int ks = 0; ks < kQTile / 16; ++ks) {
          const uint32_t a_col = kColS + sb * kQTile + (ks >> 1) * 32 + (ks & 1) * 8;
          umma_ts(tmem_base + kColDv, tmem_base + a_col,
                  smem_desc_join(do_lo_mn + ((ks * 2048) >> 4), kHi), idesc_dkv,
                  (i > 0 || ks > 0) ? 1u : 0u);
        }
        BWD_TIMING_ONLY(tacc[17] += clock64() - t_b;)
        // dP^T(i+1): its buffer last held dQ^T(i-1), which the write-back warps must have drained.
        if (i + 1 < n_iter) {
          BWD_WAIT(3, bar(iDoFull + st1), ((i + 1) / NS) & 1, wctx, kBbDoFull + st1);
          if (i >= 1) BWD_WAIT(4, bar(iDqFree + sb1), ((i - 1) >> 1) & 1, wctx, kBbDqFree);
          tc_fence_after_sync();
          BWD_TIMING_ONLY(const long long t_c = clock64();)
          issue_xyT(kColDpq + sb1 * kQTile, v_lo_k, sbase + L::kDoOff + st1 * L::kQTileBytes);
          tc_commit(bar(iDpReady + sb1));
          BWD_TIMING_ONLY(tacc[18] += clock64() - t_c;)
        }
        // dK += dS^T(i) Q(i)
        BWD_WAIT(5, bar(iDsReady), i & 1, wctx, kBbDsReady);
        tc_fence_after_sync();
        BWD_TIMING_ONLY(const long long t_d = clock64();)
#pragma unroll
        for (int ks = 0; ks < kQTile / 16; ++ks) {
          umma_ss(tmem_base + kColDk, smem_desc_join(ds_lo_k + ((ks * 32) >> 4), kHi),
                  smem_desc_join(q_lo_mn + ((ks * 2048) >> 4), kHi), idesc_dkv,
                  (i > 0 || ks > 0) ? 1u : 0u);
        }
        // dQ^T(i) = K^T dS^T(i), into the columns of the consumed dP^T(i)
#pragma unroll
        for (int ks = 0; ks < kKvTile / 16; ++ks) {
          umma_ss(tmem_base + kColDpq + sb * kQTile,
                  smem_desc_join(k_lo_mn + ((ks * 2048) >> 4), kHi),
                  smem_desc_join(ds_lo_mn + ((ks * 2048) >> 4), kHi), idesc_dq, ks > 0 ? 1u : 0u);
        }
        BWD_TIMING_ONLY(tacc[19] += clock64() - t_d;)
        tc_commit(bar(iDqReady + sb));
        tc_commit(bar(iStageEmpty + st));
        tc_commit(bar(iDsFree));
        BWD_TIMING_ONLY(tacc[21] += clock64() - t_d;)
      }
      tc_commit(bar(iAllDone));
    }
    __syncwarp();
  } else if (warp < 8) {
    // ===================== compute ============================================
    const int quarter = warp & 3;
    const int half = warp >> 2;                       // query columns [32*half, 32*half+32)
    const int kv_row = quarter * 32 + lane;           // key row inside the tile (= TMEM lane)
    const int kv_local = kv0 + kv_row;
    const bool kv_ok = kv_local < wk.seqlen_k;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float c2 = p.scale_log2;
    uint8_t* ds_row = sgen + L::kDsOff + kv_row * 128;

    for (int i = 0; i < n_iter; ++i) {
      const int st = i % NS;
      const int sb = i & 1;
      const int qt = qt0 + i % nq;
      const int q_col0 = qt * kQTile + half * 32;  // local query index of this thread's first column
      const float* stat = reinterpret_cast<const float*>(sgen + L::kStatOff) + st * 2 * kQTile + half * 32;
      const bool tile_mask = !kv_ok || (CAUSAL && (kv0 + kKvTile - 1 > qt * kQTile));

      BWD_WAIT(6, bar(iStatFull + st), (i / NS) & 1, wctx, kBbStatFull + st);
      BWD_WAIT(7, bar(iSReady + sb), (i >> 1) & 1, wctx, kBbSReady + sb);
      tc_fence_after_sync();
      BWD_TIMING_ONLY(const long long t_p0 = clock64();)

      float pv[32];
      {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColS + sb * kQTile + half * 32, r);
        float4 l4[8];  // the statistics load overlaps the TMEM load's latency
#pragma unroll
        for (int j = 0; j < 8; ++j) l4[j] = *reinterpret_cast<const float4*>(stat + 4 * j);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          pv[j + 0] = fast_exp2(fmaf(__uint_as_float(r[j + 0]), c2, -l4[j >> 2].x));
          pv[j + 1] = fast_exp2(fmaf(__uint_as_float(r[j + 1]), c2, -l4[j >> 2].y));
          pv[j + 2] = fast_exp2(fmaf(__uint_as_float(r[j + 2]), c2, -l4[j >> 2].z));
          pv[j + 3] = fast_exp2(fmaf(__uint_as_float(r[j + 3]), c2, -l4[j >> 2].w));
        }
        if (tile_mask) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const bool vis = kv_ok && (!CAUSAL || kv_local <= q_col0 + j);
            pv[j] = vis ? pv[j] : 0.f;
          }
        }
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack_half2(pv[2 * j], pv[2 * j + 1]);
        // P^T overwrites this thread's own S^T columns: [32*half, 32*half+16)
        tmem_st_32x32b_x16(tmem_base + lane_addr + kColS + sb * kQTile + half * 32, pk);
        tmem_wait_st();
      }
      tc_fence_before_sync();
      mbar_arrive(bar(iPReady));
      BWD_TIMING_ONLY(tacc[22] += clock64() - t_p0;)

      BWD_WAIT(8, bar(iDpReady + sb), (i >> 1) & 1, wctx, kBbDpReady);
      tc_fence_after_sync();
      BWD_TIMING_ONLY(const long long t_s0 = clock64();)
      uint32_t dsp[16];
      {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + sb * kQTile + half * 32, r);
        float4 d4s[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) d4s[j] = *reinterpret_cast<const float4*>(stat + kQTile + 4 * j);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 d4 = d4s[j >> 2];
          const float a0 = pv[j + 0] * (__uint_as_float(r[j + 0]) - d4.x);
          const float a1 = pv[j + 1] * (__uint_as_float(r[j + 1]) - d4.y);
          const float a2 = pv[j + 2] * (__uint_as_float(r[j + 2]) - d4.z);
          const float a3 = pv[j + 3] * (__uint_as_float(r[j + 3]) - d4.w);
          dsp[(j >> 1) + 0] = pack_half2(a0, a1);
          dsp[(j >> 1) + 1] = pack_half2(a2, a3);
        }
      }
      if (i > 0) BWD_WAIT(9, bar(iDsFree), (i - 1) & 1, wctx, kBbDsFree);
      // dS^T row -> shared memory, 128-byte XOR swizzle (16-byte chunk index ^ row % 8)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int chunk = half * 4 + c;
        *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (kv_row & 7)) << 4)) =
            make_uint4(dsp[4 * c + 0], dsp[4 * c + 1], dsp[4 * c + 2], dsp[4 * c + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(bar(iDsReady));
      BWD_TIMING_ONLY(tacc[23] += clock64() - t_s0;)
    }

    // ---- epilogue: dV (warps 0-3) and dK (warps 4-7) -------------------------
    if (n_iter > 0) {
      mbar_wait(bar(iAllDone), 0, wctx, kBbAllDone);
      tc_fence_after_sync();
    }
    const bool is_dk = half == 1;
    const RowStrides& st_o = is_dk ? p.dk_strides : p.dv_strides;
    __half* out_row = static_cast<__half*>(is_dk ? p.dk : p.dv) + wk.batch * st_o.batch +
                      wk.kv_head * st_o.head +
                      (static_cast<int64_t>(wk.k_row0) + kv_local) * st_o.row;
    const float mul = is_dk ? p.scale : 1.f;
    const uint32_t t_acc = tmem_base + lane_addr + (is_dk ? kColDk : kColDv);
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
      if (kv_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 out;
          out.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * mul, __uint_as_float(r[v * 8 + 1]) * mul);
          out.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * mul, __uint_as_float(r[v * 8 + 3]) * mul);
          out.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * mul, __uint_as_float(r[v * 8 + 5]) * mul);
          out.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * mul, __uint_as_float(r[v * 8 + 7]) * mul);
          *reinterpret_cast<uint4*>(out_row + c * 32 + v * 8) = out;
        }
      }
    }
  } else {
    // ===================== dQ write-back ======================================
    const int quarter = warp & 3;
    const int drow = quarter * 32 + lane;  // head_dim index = TMEM lane of dQ^T
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    // The 64-row tile leaves in two 32-row halves, each with its own staging buffer, so that
    // the bulk reduction of one half reads shared memory while the other half is being written.
    float* stage_half[2] = {reinterpret_cast<float*>(sgen + L::kDqOff),
                            reinterpret_cast<float*>(sgen + L::kDqOff) + (kQTile / 2) * D};
    const bool issuer = warp == 10 && lane == 0;
    for (int i = 0; i < n_iter; ++i) {
      const int head = wk.kv_head * group + i / nq;
      const int qt = qt0 + i % nq;
      const int sb = i & 1;
      BWD_WAIT(10, bar(iDqReady + sb), (i >> 1) & 1, wctx, kBbDqReady);
      tc_fence_after_sync();
      uint32_t r[2][32];
      tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + sb * kQTile, r[0]);
      tmem_ld_32x32b_x32(tmem_base + lane_addr + kColDpq + sb * kQTile + 32, r[1]);
      tmem_wait_ld();
      tc_fence_before_sync();
      mbar_arrive(bar(iDqFree + sb));
      BWD_TIMING_ONLY(const long long t_red0 = clock64();)
      float* dst_tile = p.dq_accum + wk.batch * p.dq_accum_batch_stride + head * p.dq_accum_head_stride +
                        (static_cast<int64_t>(wk.q_row0) + qt * kQTile) * D;
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        // The reduction that last read this half's buffer (two groups ago) must be done with it.
        if (issuer) bulk_wait_group_read<1>();
        named_barrier_sync(1, 128);
        if (drow < D) {
#pragma unroll
          for (int j = 0; j < 32; ++j) stage_half[hf][j * D + drow] = __uint_as_float(r[hf][j]);
        }
        fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (issuer) {
          const int rows = min(kQTile / 2, wk.seqlen_q - qt * kQTile - hf * (kQTile / 2));
          if (rows > 0) {
            bulk_reduce_add_f32(dst_tile + hf * (kQTile / 2) * D,
                                sbase + L::kDqOff + hf * (kQTile / 2) * D * 4,
                                static_cast<uint32_t>(rows) * D * 4u);
          }
          bulk_commit_group();  // one group per half, empty or not: keeps the group count uniform
        }
      }
      BWD_TIMING_ONLY(tacc[11] += clock64() - t_red0;)
    }
    if (warp == 10 && lane == 0) bulk_wait_group0();
  }

#ifdef FAL_BWD_TIMING
  if (lane == 0 && (warp == 0 || warp == 8 || warp == 9 || warp == 10)) {
    for (int i = 0; i < 12; ++i)
      if (tacc[i]) atomicAdd(&g_bwd_wait_cycles[i], static_cast<unsigned long long>(tacc[i]));
    for (int i = 16; i < 24; ++i)
      if (tacc[i]) atomicAdd(&g_bwd_wait_cycles[i], static_cast<unsigned long long>(tacc[i]));
    if (warp == 0) {
      atomicAdd(&g_bwd_wait_cycles[12], static_cast<unsigned long long>(clock64() - t_cta0));
      atomicAdd(&g_bwd_wait_cycles[13], static_cast<unsigned long long>(n_iter));
      atomicAdd(&g_bwd_wait_cycles[14], 1ull);
    }
  }
#endif
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

#ifdef FAL_BWD_TIMING
}  // namespace
}  // namespace fal
extern "C" __attribute__((visibility("default"))) int fal_debug_bwd_waits(unsigned long long* out32, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out32, fal::g_bwd_wait_cycles, sizeof(unsigned long long) * 32);
  if (e == cudaSuccess && reset) {
    unsigned long long z[32] = {};
    e = cudaMemcpyToSymbol(fal::g_bwd_wait_cycles, z, sizeof(z));
  }
  return static_cast<int>(e);
}
namespace fal {
namespace {
#endif

// ---------------------------------------------------------------------------
// Pre-pass: delta[row] = sum_d dO*O  (precompute_D_kernel, bwd.cu:76-107 of the reference).
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
    const uint4 ov = *reinterpret_cast<const uint4*>(o);
    const uint4 dv = *reinterpret_cast<const uint4*>(d_o);
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
}

// ---------------------------------------------------------------------------
// Post-pass: dQ = fp16(scale * accumulator)  (csrc/flash_attn_legacy.cpp:184 of the reference).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) fal_bwd_post_kernel(const BwdPostParams p) {
  const int chunks = p.head_dim / 8;
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

template <int D, bool CAUSAL>
cudaError_t launch_bwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& tdo, const BwdParams& p, int grid, cudaStream_t stream) {
  auto kern = fal_bwd_kernel<D, CAUSAL>;
  static DeviceOnce configured;
  cudaError_t e = configured.run([&] {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                BwdSmem<D>::kAllocBytes);
  });
  if (e != cudaSuccess) return e;
  kern<<<grid, kBwdThreads, BwdSmem<D>::kAllocBytes, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_prep(const BwdPrepParams& p, cudaStream_t stream) {
  // The accumulator must start at zero: the main kernel only ever adds to it.
  const size_t acc_bytes = static_cast<size_t>(p.batch) * p.dq_accum_batch_stride * sizeof(float);
  cudaError_t e = cudaMemsetAsync(p.dq_accum, 0, acc_bytes, stream);
  if (e != cudaSuccess) return e;
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.rows;
  if (p.head_dim == 128) {
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
                       const CUtensorMap& tv, const CUtensorMap& tdo, const BwdParams& p, int grid,
                       cudaStream_t stream) {
  if (head_dim == 128) {
    return causal ? launch_bwd_t<128, true>(tq, tk, tv, tdo, p, grid, stream)
                  : launch_bwd_t<128, false>(tq, tk, tv, tdo, p, grid, stream);
  }
  if (head_dim == 64) {
    return causal ? launch_bwd_t<64, true>(tq, tk, tv, tdo, p, grid, stream)
                  : launch_bwd_t<64, false>(tq, tk, tv, tdo, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_bwd_post(const BwdPostParams& p, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads_q * p.rows * (p.head_dim / 8);
  const int64_t blocks = (total + 255) / 256;
  fal_bwd_post_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace fal
