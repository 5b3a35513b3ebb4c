// FlashAttention-2 forward for sm_100a, head_dim 128, on CTA pairs: the same algorithm and
// warp roles as fal_fwd.cu (which replaces csrc/kernels/flash_attn_fwd_volta.cu:170-345 and
// :350-523 of the reference), but two CTAs on neighbouring SMs form a cluster and every MMA is a
// pair MMA (tcgen05.mma.cta_group::2, M = 256).
//
// Why: with one CTA per MMA the S = Q K^T instruction reads 8 KB of shared memory (A and B) per
// 64 tensor-pipe cycles, which is all the shared-memory bandwidth an SM has; the TMA writes of
// the next K/V tiles and the V reads of P V come on top, so the tensor pipe starves.  In a pair
// MMA each CTA supplies its own 128 rows of A but only HALF of B, and loads only half of every
// K and V tile: per SM and key tile 80 KB of shared-memory traffic instead of 128 KB.
//
// A cluster owns 512 consecutive query rows of one (batch, head): two pair tiles of 256 rows;
// CTA r of the pair holds rows [128 r, 128 r + 128) of each.  Per CTA:
//
//   warps 0-3   softmax + output, pair tile 0 (its own 128 rows; TMEM lanes by warp % 4)
//   warps 4-7   softmax + output, pair tile 1
//   warp  8     TMA producer: its own Q rows, keys [64 r, 64 r + 64) of every K tile (B of
//               Q K^T splits along the keys), head-dim columns [64 r, 64 r + 64) of every V
//               tile (B of P V splits along the head dimension)
//   warp  9     TMEM owner; in the leader CTA (rank 0) one lane issues pair tile 0's MMAs
//   warp 10     leader CTA: one lane issues pair tile 1's MMAs; peer CTA: forwards "my half has
//               landed" to the leader's barriers
//   warp 11     idle
//
// Barriers: "full" barriers that the issuer waits on live in the leader and count two arrivals
// (leader's TMA transaction + the peer's forwarder); P-ready barriers live in the leader and
// count one elected arrival per softmax warp of both CTAs; everything the MMAs signal (S ready,
// O done, stage empty) is committed to the same barrier of BOTH CTAs.  A stage holds the K and
// the V half of one key tile and has one "empty" barrier per pair tile (each tile's issuer
// commits its own); a token barrier per tile keeps the two issuers strictly alternating.
// TMEM columns per CTA: S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P (fp16) overwrites
// the first 64 columns of its S tile and feeds the P V MMA straight from TMEM.
#define FAL_WAIT_SLOW_PATH_INLINE  // this kernel uses setmaxnreg, which rules out calls
#include "fal_common.h"
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

constexpr int kThreads = 384;
constexpr int kTileM = 128;  // query rows per CTA in a pair tile
constexpr int kTileN = 128;  // keys per step
constexpr int kD = 128;
constexpr int kPairRows = 2 * kTileM;
constexpr int kClusterRows = 2 * kPairRows;
constexpr int kStages = 4;
constexpr float kNegInf = -INFINITY;
constexpr float kRescaleThreshold = 8.0f;  // skip the O rescale while the maximum grows by < 2^8

// Register split after launch (see fal_fwd.cu): must not exceed what the CTA was launched with.
constexpr int kRegsSoftmax = 216;
constexpr int kRegsOther = 72;
static_assert(2 * 128 * kRegsSoftmax + 128 * kRegsOther <= 168 * kThreads,
              "setmaxnreg split exceeds the registers the CTA was launched with");

// P handed to the issuer in two halves (1) or at once (0).
#ifndef FAL_PAIR_SPLIT_P
#define FAL_PAIR_SPLIT_P 1
#endif

// Of every 4 score pairs, this many take the polynomial exp2 on the FMA pipe instead of the
// special-function unit (which both tiles' softmax warps share).
#ifndef FAL_PAIR_EMU_PAIRS
#define FAL_PAIR_EMU_PAIRS 0
#endif
template <int K>
__device__ __forceinline__ uint64_t pair_exp2(int i, uint64_t x) {
  const int q = ((i >> 1) + K) & 3;  // i is a multiple of 4 under full unrolling
  const bool emu = (FAL_PAIR_EMU_PAIRS == 1) ? (q == 0)
                 : (FAL_PAIR_EMU_PAIRS == 2) ? ((q & 1) == 0)
                 : (FAL_PAIR_EMU_PAIRS == 3) ? (q != 3)
                 : (FAL_PAIR_EMU_PAIRS >= 4);
  return emu ? exp2_pair_fma(x) : exp2_pair_mufu(x);
}

// Tuning aid, compiled in only with -DFAL_FWD_TIMING: cycles per role and phase, summed over CTAs.
#ifdef FAL_FWD_TIMING
__device__ unsigned long long g_fwd_pair_cycles[32];
#define PAIR_T(slot, stmt)                 \
  do {                                     \
    const long long _t0 = clock64();       \
    stmt;                                  \
    tacc[slot] += clock64() - _t0;         \
  } while (0)
#define PAIR_MARK(slot)                    \
  do {                                     \
    const long long _t1 = clock64();       \
    tacc[slot] += _t1 - tmark;             \
    tmark = _t1;                           \
  } while (0)
#else
#define PAIR_T(slot, stmt) stmt
#define PAIR_MARK(slot)
#endif

enum PairBarrier : int {  // labels for a wait that gave up
  kBarQFull = 100,
  kBarKFull = 110,
  kBarKEmpty = 120,
  kBarVFull = 130,
  kBarVEmpty = 140,
  kBarSReady = 150,
  kBarPReady = 160,
  kBarODone = 170,
};

struct PairSmem {
  static constexpr int kQBoxBytes = kTileM * 128;       // [128 rows][64 d]
  static constexpr int kQTileBytes = 2 * kQBoxBytes;    // 128 x 128
  static constexpr int kKBoxBytes = 64 * 128;           // [64 keys][64 d]
  static constexpr int kKHalfBytes = 2 * kKBoxBytes;    // this CTA's 64 keys x 128 d
  static constexpr int kVHalfBytes = kTileN * 128;      // [128 keys][this CTA's 64 d]
  static constexpr int kQOff = 0;
  static constexpr int kKOff = 2 * kQTileBytes;
  static constexpr int kVOff = kKOff + kStages * kKHalfBytes;
  static constexpr int kBarOff = kVOff + kStages * kVHalfBytes;
  // q_full[2] kv_full[S] kv_empty[2][S] s_ready[2] p_ready[2] o_done[2] p_half[2] token[2]
  static constexpr int kNumBars = 2 + 3 * kStages + 10;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;  // tmem slot, abort flag
  static constexpr int kBytes = kMiscOff + 16;
  static constexpr int kAllocBytes = kBytes + 1024;  // room to align the base to 1024
};

struct PairWork {
  int batch;  // TMA batch coordinate (0 when packed)
  int head;
  int kv_head;
  int blk;       // 512-row block inside the sequence
  int q_row0;    // TMA row coordinate of the sequence's first query
  int k_row0;    // TMA row coordinate of the sequence's first key
  int seqlen_q;
  int seqlen_k;
  int64_t o_base;
  int64_t lse_base;
};

// Maps a cluster (blockIdx.x / 2) to a unit of work; false when it has none.  Both CTAs of a
// cluster take the same decision.
__device__ __forceinline__ bool pair_decode_work(const FwdParams& p, PairWork& w) {
  const int idx = blockIdx.x >> 1;
  if (p.cu_q == nullptr) {
    const int bh_count = p.batch * p.heads_q;
    // Heaviest (last) query blocks first: under a causal mask they have the most keys.
    w.blk = p.num_qblk - 1 - idx / bh_count;
    const int bh = idx % bh_count;
    w.batch = bh / p.heads_q;
    w.head = bh % p.heads_q;
    w.q_row0 = 0;
    w.k_row0 = 0;
    w.seqlen_q = p.seqlen_q;
    w.seqlen_k = p.seqlen_k;
    w.o_base = w.batch * p.o_strides.batch + w.head * p.o_strides.head;
    w.lse_base = w.batch * p.lse_strides.batch + w.head * p.lse_strides.head;
  } else {
    const int slot = idx / p.heads_q;
    w.head = idx % p.heads_q;
    w.batch = 0;
    int first = 0;
    int seq = -1;
    int q_start = 0;
    for (int s = 0; s < p.num_seqs; ++s) {
      const int a = __ldg(p.cu_q + s);
      const int e = __ldg(p.cu_q + s + 1);
      const int nblk = (e - a + kClusterRows - 1) / kClusterRows;
      if (slot < first + nblk) {
        seq = s;
        q_start = a;
        w.seqlen_q = e - a;
        break;
      }
      first += nblk;
    }
    if (seq < 0) return false;
    w.blk = slot - first;
    w.q_row0 = q_start;
    w.k_row0 = __ldg(p.cu_k + seq);
    w.seqlen_k = __ldg(p.cu_k + seq + 1) - w.k_row0;
    w.o_base = w.head * p.o_strides.head + static_cast<int64_t>(q_start) * p.o_strides.row;
    w.lse_base = w.head * p.lse_strides.head + static_cast<int64_t>(q_start) * p.lse_strides.row;
  }
  w.kv_head = w.head / (p.heads_q / p.heads_kv);
  return true;
}

template <bool CAUSAL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fal_fwd_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using L = PairSmem;
  constexpr int NS = kStages;

  PairWork wk;
  if (!pair_decode_work(p, wk)) return;
  const uint32_t rank = cluster_cta_rank();

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));

  const uint32_t bar0 = sbase + L::kBarOff;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int iQFull = 0, iFull = 2, iEmpty = 2 + NS, iSReady = 2 + 3 * NS, iPReady = iSReady + 2,
            iODone = iSReady + 4, iPHalf = iSReady + 6, iToken = iSReady + 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kMiscOff + 4);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Key tiles each 256-row pair tile visits (the same number in both CTAs of the pair: under a
  // causal mask the leader's rows see one tile fewer, its last tile is then fully masked).
  const int nk_tiles = (wk.seqlen_k + kTileN - 1) / kTileN;
  int ntile[2];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int row0 = wk.blk * kClusterRows + w * kPairRows;
    int n = 0;
    if (row0 < wk.seqlen_q) {
      n = nk_tiles;
      if (CAUSAL) n = min(n, min(row0 + kPairRows - 1, wk.seqlen_q - 1) / kTileN + 1);
    }
    ntile[w] = n;
  }
  const int n_max = max(ntile[0], ntile[1]);

  // ---- one-time setup -------------------------------------------------------
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    const uint32_t full_count = (rank == 0) ? 2u : 1u;  // leader: own TMA + the peer's forwarder
    mbar_init(bar(iQFull + 0), full_count);
    mbar_init(bar(iQFull + 1), full_count);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(iFull + s), full_count);
      mbar_init(bar(iEmpty + s), 1);       // released by tile 0's issuer
      mbar_init(bar(iEmpty + NS + s), 1);  // released by tile 1's issuer
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar(iSReady + w), 1);
      mbar_init(bar(iPReady + w), 8);  // one elected lane per softmax warp, both CTAs
      mbar_init(bar(iPHalf + w), 8);
      mbar_init(bar(iODone + w), 1);
      mbar_init(bar(iToken + w), 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
  if (warp == 9) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t leader_bar0 = cluster_map_shared(bar0, 0);

  if (warp >= 8) {
    setmaxnreg_dec<kRegsOther>();
    if (warp == 8) {
      // ===================== TMA producer =====================================
      if (lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        for (int w = 0; w < 2; ++w) {
          if (ntile[w] == 0) continue;
          mbar_arrive_expect_tx(bar(iQFull + w), L::kQTileBytes);
          const int row = wk.q_row0 + wk.blk * kClusterRows + w * kPairRows + static_cast<int>(rank) * kTileM;
          for (int bx = 0; bx < 2; ++bx)
            tma_load_4d(sbase + L::kQOff + w * L::kQTileBytes + bx * L::kQBoxBytes, &tm_q,
                        bar(iQFull + w), bx * 64, row, wk.head, wk.batch);
        }
        for (int j = 0; j < n_max; ++j) {
          const int s = j % NS;
          const int use = j / NS;
          const int row = wk.k_row0 + j * kTileN;
          if (use > 0) {
            for (int w = 0; w < 2; ++w)
              if (j - NS < ntile[w]) mbar_wait(bar(iEmpty + w * NS + s), (use - 1) & 1, wctx, kBarKEmpty + s);
          }
          mbar_arrive_expect_tx(bar(iFull + s), L::kKHalfBytes + L::kVHalfBytes);
          for (int bx = 0; bx < 2; ++bx)
            tma_load_4d(sbase + L::kKOff + s * L::kKHalfBytes + bx * L::kKBoxBytes, &tm_k,
                        bar(iFull + s), bx * 64, row + static_cast<int>(rank) * 64, wk.kv_head, wk.batch);
          tma_load_4d(sbase + L::kVOff + s * L::kVHalfBytes, &tm_v, bar(iFull + s),
                      static_cast<int>(rank) * 64, row, wk.kv_head, wk.batch);
        }
      }
      __syncwarp();
    } else if (rank == 0 && (warp == 9 || warp == 10)) {
      // ===================== MMA issuers (leader CTA only): warp 9 tile 0, warp 10 tile 1 =====
      // The tensor pipe's queue is short: whatever the issuing thread does between MMAs (barrier
      // round trips, commits) is time the pipe mostly idles.  So each tile has its own issuer
      // and a token travels between them: a thread issues its tile's P V and next Q K^T only
      // while it holds the token -- which keeps the two tiles strictly alternating, one tile's
      // softmax under the other's MMAs -- and does its waiting and committing without it.
      const int w = warp - 9;
      const int nt = ntile[w];
      const int nt_other = ntile[w ^ 1];
      if (lane == 0 && nt > 0) {
        constexpr uint32_t idesc_qk = make_idesc_f16(kPairRows, kTileN, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc_f16(kPairRows, kD, 0, 1);
        constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
        const uint32_t q_lo = smem_desc_lo(sbase + L::kQOff + w * L::kQTileBytes, 16);
        const uint32_t tS_w = tmem_base + w * kTileN;
        const uint32_t tO_w = tmem_base + 256 + w * kD;
        const uint32_t peer_bar0 = cluster_map_shared(bar0, 1);
        // Arrive on barrier i of both CTAs once every MMA this thread issued so far has finished.
        auto commit_both = [&](int i) {
          tc_commit_pair(leader_bar0 + 8u * i);
          tc_commit_pair(peer_bar0 + 8u * i);
        };
        // S = Q K_j^T: A = each CTA's own 128 x 128 Q tile, B = each CTA's 64 keys, both K-major;
        // 16 head-dim elements (32 bytes inside the 128-byte swizzle row) per step.
        auto issue_qk = [&](int j) {
          const uint32_t k_lo = smem_desc_lo(sbase + L::kKOff + (j % NS) * L::kKHalfBytes, 16);
#pragma unroll
          for (int ks = 0; ks < kD / 16; ++ks) {
            const uint32_t a_off = ((ks >> 2) * L::kQBoxBytes + (ks & 3) * 32) >> 4;
            const uint32_t b_off = ((ks >> 2) * L::kKBoxBytes + (ks & 3) * 32) >> 4;
            umma_ss_pair(tS_w, smem_desc_join(q_lo + a_off, kHi), smem_desc_join(k_lo + b_off, kHi),
                         idesc_qk, ks > 0 ? 1u : 0u);
          }
        };
        // O += P V_j: A = P from each CTA's TMEM (8 columns of packed fp16 per 16 keys), B = each
        // CTA's 64 head-dim columns of V, MN-major: 16 keys = 2048 bytes per step, 8-key groups
        // 1024 bytes apart.
        auto issue_pv = [&](int j, int half) {
          const uint32_t v_lo = smem_desc_lo(sbase + L::kVOff + (j % NS) * L::kVHalfBytes, L::kVHalfBytes);
#pragma unroll
          for (int kk = 0; kk < kTileN / 32; ++kk) {
            const int ks = half * (kTileN / 32) + kk;
            umma_ts_pair(tO_w, tS_w + ks * 8, smem_desc_join(v_lo + ((ks * 2048) >> 4), kHi), idesc_pv,
                         (j > 0 || ks > 0) ? 1u : 0u);
          }
        };
        // Global issue order: QK(0,0) QK(1,0), then for every step j: block(0,j) block(1,j),
        // block(w,j) = PV(w,j) [+ QK(w,j+1)], leaving out what a tile does not have.  A block
        // takes the token from its predecessor and hands it to its successor where they exist.
        uint32_t takes = 0;  // tokens taken so far (phase of this tile's token barrier)
        auto take_token = [&]() {
          mbar_wait(bar(iToken + w), takes & 1, wctx, kBarPReady + 2 + w);
          ++takes;
        };
        auto pass_token = [&]() { mbar_arrive(bar(iToken + (w ^ 1))); };
#ifdef FAL_FWD_TIMING
        long long tacc[8] = {};
        const long long t_begin = clock64();
#endif
        mbar_wait_cluster(bar(iFull + 0), 0, wctx, kBarKFull);
        mbar_wait_cluster(bar(iQFull + w), 0, wctx, kBarQFull + w);
        if (w == 1) take_token();  // after QK(0,0)
        tc_fence_after_sync();
        issue_qk(0);
        if (w == 0 ? (nt_other > 0) : true) pass_token();  // to QK(1,0) / to block(0,0)
        commit_both(iSReady + w);
        for (int j = 0; j < nt; ++j) {
          const int s = j % NS;
          const bool more = j + 1 < nt;
#if FAL_PAIR_SPLIT_P
          PAIR_T(0, mbar_wait_cluster(bar(iPHalf + w), j & 1, wctx, kBarPReady + w));
#else
          PAIR_T(2, mbar_wait_cluster(bar(iPReady + w), j & 1, wctx, kBarPReady + w));
#endif
          if (more) PAIR_T(3, mbar_wait_cluster(bar(iFull + (j + 1) % NS), ((j + 1) / NS) & 1, wctx, kBarKFull));
          // predecessor: block(1,j-1) or QK(1,0) for tile 0; block(0,j) for tile 1
          const bool pred = (w == 0) ? (j == 0 ? nt_other > 0 : j - 1 < nt_other) : (j < nt_other);
          if (pred) PAIR_T(1, take_token());
          tc_fence_after_sync();
          PAIR_T(5, issue_pv(j, 0));
#if FAL_PAIR_SPLIT_P
          PAIR_T(2, mbar_wait_cluster(bar(iPReady + w), j & 1, wctx, kBarPReady + w));
          tc_fence_after_sync();
#endif
          PAIR_T(6, issue_pv(j, 1));
          if (more) PAIR_T(7, issue_qk(j + 1));
          // successor: block(1,j) for tile 0; block(0,j+1) for tile 1
          const bool succ = (w == 0) ? (j < nt_other) : (j + 1 < nt_other);
          if (succ) pass_token();
          commit_both(iEmpty + w * NS + s);
          commit_both(more ? iSReady + w : iODone + w);
        }
#ifdef FAL_FWD_TIMING
        for (int i = 0; i < 4; ++i) atomicAdd(&g_fwd_pair_cycles[i], static_cast<unsigned long long>(tacc[i]));
        for (int i = 5; i < 8; ++i) atomicAdd(&g_fwd_pair_cycles[18 + i], static_cast<unsigned long long>(tacc[i]));
        atomicAdd(&g_fwd_pair_cycles[4], static_cast<unsigned long long>(clock64() - t_begin));
        atomicAdd(&g_fwd_pair_cycles[5], static_cast<unsigned long long>(nt));
        if (w == 0) atomicAdd(&g_fwd_pair_cycles[6], 1ull);
#endif
      }
      __syncwarp();
    } else if (warp == 10) {
      // ===================== peer CTA: tell the leader that this half has landed ============
      if (lane == 0) {
        for (int w = 0; w < 2; ++w) {
          if (ntile[w] == 0) continue;
          mbar_wait(bar(iQFull + w), 0, wctx, kBarQFull + w);
          mbar_arrive_cluster(leader_bar0 + 8u * (iQFull + w));
        }
        for (int j = 0; j < n_max; ++j) {
          const int s = j % NS;
          const int use = j / NS;
          mbar_wait(bar(iFull + s), use & 1, wctx, kBarKFull + s);
          mbar_arrive_cluster(leader_bar0 + 8u * (iFull + s));
        }
      }
      __syncwarp();
    }
  } else {
    // ===================== softmax + output =================================
    setmaxnreg_inc<kRegsSoftmax>();
    const int wg = warp >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_tile0 = wk.blk * kClusterRows + wg * kPairRows + static_cast<int>(rank) * kTileM;
    const int q_local = q_tile0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + wg * kTileN;
    const uint32_t tO = tmem_base + lane_addr + 256 + wg * kD;
    const int nt = ntile[wg];
    const float c2 = p.scale_log2;
    // One lane per warp tells the leader's issuer that this warp's part of P is in TMEM.
    auto p_arrive = [&](int i) {
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (rank == 0) mbar_arrive(bar(i));
#ifdef FAL_PAIR_RELEASE_ARRIVE
        else mbar_arrive_cluster(leader_bar0 + 8u * i);
#else
        else mbar_arrive_cluster_relaxed(leader_bar0 + 8u * i);
#endif
      }
    };

    float m_ref = kNegInf;
    float l = 0.f;

#ifdef FAL_FWD_TIMING
    long long tacc[8] = {};
    long long tmark = clock64();
    const long long t_begin = tmark;
#endif
    for (int j = 0; j < nt; ++j) {
      PAIR_MARK(7);
      mbar_wait(bar(iSReady + wg), j & 1, wctx, kBarSReady + wg);
      tc_fence_after_sync();
      PAIR_MARK(0);
      const int kv0 = j * kTileN;
      int limit = wk.seqlen_k - kv0;  // columns c < limit are visible
      if (CAUSAL) limit = min(limit, q_local - kv0 + 1);
      const bool tile_mask =
          (kv0 + kTileN > wk.seqlen_k) || (CAUSAL && (kv0 + kTileN - 1 > q_tile0));

      // All 128 scores of this thread's row, one TMEM round trip.
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(tS + c * 32, sr[c]);
      tmem_wait_ld();
      PAIR_MARK(1);
      if (tile_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= limit) sr[c][i] = __float_as_uint(kNegInf);
      }
      // Row maximum: eight independent 3-input chains instead of one 128-long chain.
      float mx;
      {
        float part[8];
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int hlf = 0; hlf < 2; ++hlf) {
            const int b0 = hlf * 16;
            float a = fmax3(__uint_as_float(sr[c][b0]), __uint_as_float(sr[c][b0 + 1]),
                            __uint_as_float(sr[c][b0 + 2]));
#pragma unroll
            for (int i = 3; i + 1 < 16; i += 2)
              a = fmax3(a, __uint_as_float(sr[c][b0 + i]), __uint_as_float(sr[c][b0 + i + 1]));
            a = fmaxf(a, __uint_as_float(sr[c][b0 + 15]));
            part[c * 2 + hlf] = a;
          }
        mx = fmaxf(fmax3(part[0], part[1], part[2]), fmax3(part[3], part[4], part[5]));
        mx = fmax3(mx, part[6], part[7]);
      }
      const float m_new = fmaxf(m_ref, mx);
      PAIR_MARK(2);

      if (j == 0) {
        m_ref = m_new;
      } else {
        const bool need = (m_new - m_ref) * c2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O may be touched: "S of this step is ready" was committed after the previous step's
          // P V, and MMAs complete in order.
          const float alpha = (m_new == kNegInf) ? 1.f : fast_exp2((m_ref - m_new) * c2);
#pragma unroll
          for (int c = 0; c < kD / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tO + c * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32b_x32(tO + c * 32, r);
          }
          l *= alpha;
          m_ref = m_new;
        }
      }
      const float moff = (m_ref == kNegInf) ? 0.f : m_ref * c2;
      PAIR_MARK(3);

      // P = exp2(s * c2 - m * c2) from the registers with two-float instructions, fp16 P back
      // into TMEM over the first half of S.
      const uint64_t c2p = pack_f32x2(c2, c2);
      const uint64_t moffp = pack_f32x2(-moff, -moff);
      uint64_t sum_a = pack_f32x2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const uint64_t x01 = ffma2(pack_f32x2(__uint_as_float(sr[c][i + 0]), __uint_as_float(sr[c][i + 1])),
                                     c2p, moffp);
          const uint64_t x23 = ffma2(pack_f32x2(__uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3])),
                                     c2p, moffp);
          const uint64_t p01 = pair_exp2<0>(i, x01);
          const uint64_t p23 = pair_exp2<1>(i, x23);
          sum_a = fadd2(sum_a, p01);
          sum_b = fadd2(sum_b, p23);
          float p0, p1, p2, p3;
          unpack_f32x2(p01, p0, p1);
          unpack_f32x2(p23, p2, p3);
          pk[(i >> 1) + 0] = pack_half2(p0, p1);
          pk[(i >> 1) + 1] = pack_half2(p2, p3);
        }
        tmem_st_32x32b_x16(tS + c * 16, pk);
#if FAL_PAIR_SPLIT_P
        if (c == 1) {  // the first 64 keys of P: the PV MMA may start on them
          p_arrive(iPHalf + wg);
          PAIR_MARK(4);
        }
#endif
      }
      float sum0, sum1, sum2, sum3;
      unpack_f32x2(sum_a, sum0, sum1);
      unpack_f32x2(sum_b, sum2, sum3);
      l += (sum0 + sum1) + (sum2 + sum3);
      p_arrive(iPReady + wg);
      PAIR_MARK(5);
    }
#ifdef FAL_FWD_TIMING
#ifndef FAL_TIMING_RANK
#define FAL_TIMING_RANK rank
#endif
    if (lane == 0 && quarter == 0 && rank == (FAL_TIMING_RANK)) {
      for (int i = 0; i < 8; ++i)
        if (i != 6) atomicAdd(&g_fwd_pair_cycles[8 + i], static_cast<unsigned long long>(tacc[i]));
      atomicAdd(&g_fwd_pair_cycles[8 + 6], static_cast<unsigned long long>(clock64() - t_begin));
      atomicAdd(&g_fwd_pair_cycles[16], static_cast<unsigned long long>(nt));
    }
#endif

    // ---- epilogue: O / l -> fp16, LSE -----------------------------------------
    if (nt > 0) {
      mbar_wait(bar(iODone + wg), 0, wctx, kBarODone + wg);
      tc_fence_after_sync();
    }
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    const bool row_ok = q_local < wk.seqlen_q;
    __half* o_row = static_cast<__half*>(p.o) + wk.o_base +
                    static_cast<int64_t>(q_local) * p.o_strides.row;
#pragma unroll
    for (int c = 0; c < kD / 32; ++c) {
      uint32_t r[32];
      if (nt > 0) {
        tmem_ld_32x32b_x32(tO + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 out;
          out.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
          out.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
          out.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
          out.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(o_row + c * 32 + v * 8) = out;
        }
      }
    }
    if (row_ok) {
      const float lse = (nt > 0 && m_ref != kNegInf) ? m_ref * p.scale + logf(fmaxf(l, 1e-20f))
                                                      : kNegInf;
      p.lse[wk.lse_base + static_cast<int64_t>(q_local) * p.lse_strides.row] = lse;
    }
  }

  // ---- teardown: neither CTA leaves while the other may still reach into it -------------
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

#ifdef FAL_FWD_TIMING
}  // namespace
}  // namespace fal
extern "C" __attribute__((visibility("default"))) int fal_debug_fwd_pair_cycles(unsigned long long* out32, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out32, fal::g_fwd_pair_cycles, sizeof(unsigned long long) * 32);
  if (e == cudaSuccess && reset) {
    unsigned long long z[32] = {};
    e = cudaMemcpyToSymbol(fal::g_fwd_pair_cycles, z, sizeof(z));
  }
  return static_cast<int>(e);
}
namespace fal {
namespace {
#endif

template <bool CAUSAL>
cudaError_t launch_fwd_pair_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const FwdParams& p, int grid, cudaStream_t stream) {
  auto kern = fal_fwd_pair_kernel<CAUSAL>;
  static DeviceOnce configured;  // one per template instance
  cudaError_t e = configured.run([&] {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                PairSmem::kAllocBytes);
  });
  if (e != cudaSuccess) return e;
  kern<<<grid, kThreads, PairSmem::kAllocBytes, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd_pair(bool causal, const CUtensorMap& tq, const CUtensorMap& tk_half,
                            const CUtensorMap& tv, const FwdParams& p, int grid, cudaStream_t stream) {
  return causal ? launch_fwd_pair_t<true>(tq, tk_half, tv, p, grid, stream)
                : launch_fwd_pair_t<false>(tq, tk_half, tv, p, grid, stream);
}

}  // namespace fal
