// FlashAttention-2 forward for sm_100a: online-softmax QK^T / PV on tcgen05
// tensor cores with TMEM accumulators, TMA-staged 128B-swizzled shared memory
// and a warp-specialised producer / MMA-issuer / softmax pipeline.
//
// Replaces flash_attn_fwd_volta_kernel and its packed twin
// (csrc/kernels/flash_attn_fwd_volta.cu:170-345, :350-523 of the reference):
// same math -- s = (q.k) * scale, top-left-aligned causal mask (kv > q masked,
// local indices), fp32 online softmax with P rounded to fp16 before PV,
// O = acc / l, L = m + ln(l) -- on a different machine model.  A second causal
// instance (SHIFTED) moves the mask's diagonal by seqlen_k - seqlen_q keys for a
// chunk of new tokens behind a cached prefix, which the reference computes
// eagerly (flash_attn_legacy/integrations.py:77-98).
//
// Two CTA shapes, both 384 threads:
//
//   warps 0-3   softmax warpgroup 0 (TMEM lanes by warp % 4)
//   warps 4-7   softmax warpgroup 1
//   warp  8     TMA producer (one elected lane)
//   warp  9     tcgen05.mma issuer (one elected lane), TMEM owner
//   warps 10-11 idle (they complete the third warpgroup so that registers can be
//               moved from it to the softmax warpgroups with setmaxnreg)
//
// Two tiles (256 query rows of one (batch, head) per CTA): each softmax warpgroup owns a 128-row
// tile with its own S/P block and O accumulator in TMEM; the MMA-issuing thread interleaves the
// two tiles so that one tile's softmax overlaps the other's tensor-core work.
// TMEM columns: S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
//
// One tile (128 query rows per CTA; head_dim 256, and the smaller grids of 64 / 128): the two S
// blocks are two buffers of the one tile, key tiles alternate between them and between the
// warpgroups (warpgroup j % 2 takes key tile j), and there is one O accumulator.  The scores of
// key tile j + 2 are computed as soon as P V of tile j is issued, so a warpgroup finds its next
// scores waiting; the warpgroups share the running row maximum through shared memory (only that
// short part of a step is serial) and keep private row sums that are added in the epilogue.
// TMEM columns: S even [0,128) S odd [128,256) P even [256,320) P odd [320,384) O [384,384+D):
// P has columns of its own here, so a score buffer is free again as soon as its warpgroup has read it.
// (head_dim 256 has no columns left for this: one warpgroup takes every key tile, as in a two-tile CTA.)
//
// P (fp16) feeds the PV MMA straight from TMEM; in the two-tile CTA it overwrites the first 64
// columns of its S block.
#define FAL_WAIT_SLOW_PATH_INLINE  // this kernel uses setmaxnreg, which rules out calls
#include "fal_common.h"
#include "fal_launch.h"
#include "sm100_ptx.cuh"

namespace fal {

namespace {

// Kernel variants (ONE_TILE):
//   false  two query tiles per CTA, one softmax warpgroup per tile
//   true   one query tile per CTA, the softmax warpgroups take alternate key tiles of it
// A thread owns one 128-column score row either way.
// Built, measured on B4 Hq32 Hkv8 N4096 d128 causal and not kept:
//  - two tiles with two softmax warpgroups EACH (640 threads, 104 registers per softmax thread): 583
//    against 515 us; ncu: tensor pipe 45.7 % against 54.3 %, long-scoreboard stalls per issue 4.9
//    against 2.5: the register cut spills inside the exponential loop and five warps per scheduler
//    crowd the one MMA-issuing thread;
//  - one tile with both warpgroups on the SAME key tile, 64 score columns per thread and the row
//    maxima exchanged every step: 600 us even with two score buffers; the two warps of a scheduler
//    then run in lockstep (both load, both exponentiate) instead of filling each other's gaps.
constexpr int kFwdThreads = 384;
constexpr int kSmWarps = 8;  // softmax warps; then producer, issuer, 2 idle
constexpr int kTileM = 128;   // query rows per softmax warpgroup
constexpr int kTileN = 128;   // keys per step
constexpr float kNegInf = -INFINITY;
// Skip the O rescale while the running maximum grows by less than 2^8.
constexpr float kRescaleThreshold = 8.0f;

// The softmax arithmetic -- scale-and-subtract, the row sums and (for a share of the pairs) the
// exponential itself -- runs as two-float instructions.  FAL_FWD_EMU_PAIRS of every 4 pairs take the
// polynomial path on the FMA pipe instead of the special-function unit (0 = none: measured slower
// with 1, the kernel is bound by dependency latency, not by the special-function unit).
#ifndef FAL_FWD_EMU_PAIRS
#define FAL_FWD_EMU_PAIRS 0
#endif
template <int K>
__device__ __forceinline__ uint64_t tile_exp2_pair(int i, uint64_t x) {
  // pair index within its group of four; i is a multiple of 4 under full unrolling
  const int q = ((i >> 1) + K) & 3;
  const bool emu = (FAL_FWD_EMU_PAIRS == 1) ? (q == 0)
                 : (FAL_FWD_EMU_PAIRS == 2) ? ((q & 1) == 0)
                 : (FAL_FWD_EMU_PAIRS == 3) ? (q != 3)
                 : (FAL_FWD_EMU_PAIRS >= 4);
  return emu ? exp2_pair_fma(x) : exp2_pair_mufu(x);
}

// Register split after launch (setmaxnreg).  The kernel launches with 168 registers for each of
// its 384 threads = 64512; the two softmax warpgroups and the third warpgroup must not ask for
// more than that in total, or setmaxnreg.inc would wait forever.
#ifndef FAL_FWD_REGS_SOFTMAX
#define FAL_FWD_REGS_SOFTMAX 216
#endif
#ifndef FAL_FWD_REGS_OTHER
#define FAL_FWD_REGS_OTHER 72
#endif
constexpr int kRegsSoftmax = FAL_FWD_REGS_SOFTMAX;
constexpr int kRegsOther = FAL_FWD_REGS_OTHER;
static_assert(2 * 128 * kRegsSoftmax + 128 * kRegsOther <= 168 * 384,
              "setmaxnreg split exceeds the registers the CTA was launched with");
// Barrier ids (only used to label a wait that gave up).
enum FwdBarrier : int {
  kBarQFull = 0,
  kBarKFull = 10,
  kBarKEmpty = 20,
  kBarVFull = 30,
  kBarVEmpty = 40,
  kBarSReady = 50,
  kBarPReady = 60,
  kBarODone = 70,
};

template <int D, bool ONE_TILE>
struct FwdSmem {
  // One 128-row query tile per CTA: always at head_dim 256 (its O accumulator alone takes 256 of the
  // 512 TMEM columns; single K and V buffers, a 128 x 256 tile is 64 KB), and at head_dim 64 / 128
  // when two-tile CTAs would leave SMs without work.
  static_assert(ONE_TILE || D != 256, "head_dim 256 runs one query tile per CTA");
  static constexpr int kQTiles = ONE_TILE ? 1 : 2;
  // One tile at head_dim 64 / 128: the softmax warpgroups take alternate key tiles (kAlt).  At 256 there
  // is no TMEM left for that (P needs columns of its own), one warpgroup takes every key tile.
  static constexpr bool kAlt = ONE_TILE && D != 256;
  static constexpr int kCtaRows = kQTiles * kTileM;
  static constexpr int kStages = (D == 256) ? 1 : (D == 128) ? 2 : 4;
  static constexpr int kBoxes = D / 64;                 // 64-element (128-byte) column boxes
  static constexpr int kBoxBytes = kTileM * 128;        // one box of a 128-row tile
  static constexpr int kTileBytes = kBoxes * kBoxBytes;  // Q, K and V tiles are all 128 x D
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQTiles * kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kTileBytes;
  static constexpr int kBarOff = kVOff + kStages * kTileBytes;
  // barriers: q_full[2] k_full[S] k_empty[S] v_full[S] v_empty[S] s_ready[2] p_ready[2] o_done[2]
  //           p_half[2] s_free[2] v_fixed
  static constexpr int kNumBars = 2 + 4 * kStages + 11;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;  // tmem slot, abort flag
  // one tile: the running row maximum the warpgroups hand to each other, and their two row sums
  static constexpr int kXchOff = kMiscOff + 16;
  static constexpr int kXchBytes = kAlt ? 3 * kTileM * 4 : 0;
  static constexpr int kBytes = kXchOff + kXchBytes;
  static constexpr int kAllocBytes = kBytes + 1024;  // room to align the base to 1024
};

struct FwdWork {
  int batch;     // TMA batch coordinate (0 when packed)
  int head;
  int kv_head;
  int qblk;      // 256-row block inside the sequence
  int q_row0;    // TMA row coordinate of the sequence's first query
  int k_row0;    // TMA row coordinate of the sequence's first key
  int seqlen_q;
  int seqlen_k;
  int64_t o_base;    // element offset of (batch, head, sequence row 0)
  int64_t lse_base;  // float offset of the same
};

// Maps blockIdx.x to a unit of work.  Returns false when the block has none
// (packed mode launches an upper bound of blocks).
__device__ __forceinline__ bool fwd_decode_work(const FwdParams& p, int cta_rows, FwdWork& w) {
  const int idx = blockIdx.x;
  if (p.cu_q == nullptr) {
    const int bh_count = p.batch * p.heads_q;
    // Heaviest (last) query blocks first: under a causal mask they have the most keys.
    w.qblk = p.num_qblk - 1 - idx / bh_count;
    const int bh = idx % bh_count;
    w.batch = bh / p.heads_q;
    w.head = bh % p.heads_q;
    w.q_row0 = 0;
    w.k_row0 = 0;
    w.seqlen_q = p.seqlen_q;
    w.seqlen_k = p.seqused_k != nullptr ? max(min(__ldg(p.seqused_k + w.batch), p.seqlen_k), 0) : p.seqlen_k;
    w.o_base = w.batch * p.o_strides.batch + w.head * p.o_strides.head;
    w.lse_base = w.batch * p.lse_strides.batch + w.head * p.lse_strides.head;
  } else {
    const int slot = idx / p.heads_q;
    w.head = idx % p.heads_q;
    w.batch = 0;
    // Which sequence owns block `slot`: every warp scans the lengths 32 sequences at a time (one
    // coalesced load, a prefix sum of the block counts, a vote) instead of walking them one by one.
    const int lane = threadIdx.x & 31;
    int first = 0;
    int seq = -1;
    int q_start = 0;
    w.seqlen_q = 0;
    for (int base = 0; base < p.num_seqs && seq < 0; base += 32) {
      const int s = base + lane;
      int a = 0, e = 0;
      if (s < p.num_seqs) {
        a = __ldg(p.cu_q + s);
        e = __ldg(p.cu_q + s + 1);
      }
      const int nblk = (e - a + cta_rows - 1) / cta_rows;
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
        seq = base + src;
        q_start = __shfl_sync(0xffffffffu, a, src);
        w.seqlen_q = __shfl_sync(0xffffffffu, e, src) - q_start;
        first = __shfl_sync(0xffffffffu, excl, src);
      } else {
        first += __shfl_sync(0xffffffffu, incl, 31);
      }
    }
    if (seq < 0) return false;
    w.qblk = slot - first;
    w.q_row0 = q_start;
    w.k_row0 = __ldg(p.cu_k + seq);
    w.seqlen_k = __ldg(p.cu_k + seq + 1) - w.k_row0;
    w.o_base = w.head * p.o_strides.head + static_cast<int64_t>(q_start) * p.o_strides.row;
    w.lse_base = w.head * p.lse_strides.head + static_cast<int64_t>(q_start) * p.lse_strides.row;
  }
  w.kv_head = w.head / (p.heads_q / p.heads_kv);
  return true;
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

// SHIFTED (causal only): the mask's diagonal is moved by seqlen_k - seqlen_q keys (bottom-right
// alignment); the kernels of the reference's own top-left mask are compiled without it.
template <int D, bool CAUSAL, bool SHIFTED, bool ONE_TILE>
__global__ void __launch_bounds__(kFwdThreads, 1)
fal_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
               const FwdParams p) {
  using L = FwdSmem<D, ONE_TILE>;
  constexpr int NS = L::kStages;

  FwdWork wk;
  constexpr int kCtaRows = L::kCtaRows;
  if (!fwd_decode_work(p, kCtaRows, wk)) return;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sgen = smem_raw + (sbase - smem_u32(smem_raw));

  const uint32_t bar0 = sbase + L::kBarOff;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  const int iQFull = 0, iKFull = 2, iKEmpty = 2 + NS, iVFull = 2 + 2 * NS, iVEmpty = 2 + 3 * NS,
            iSReady = 2 + 4 * NS, iPReady = iSReady + 2, iODone = iSReady + 4, iPHalf = iSReady + 6,
            iSFree = iSReady + 8, iVFixed = iSReady + 10;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sgen + L::kMiscOff);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sgen + L::kMiscOff + 4);
  const WaitCtx wctx{abort_flag, p.status};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // SHIFTED: keys the causal diagonal is moved by (batched: one value; packed, or a cache with its
  // own length per entry: each sequence's seqlen_k - seqlen_q).
  const int cshift = SHIFTED ? ((p.cu_q != nullptr || p.seqused_k != nullptr) ? wk.seqlen_k - wk.seqlen_q
                                                                              : p.causal_shift)
                             : 0;
  // Number of key tiles each 128-row query tile visits.
  const int nk_tiles = (wk.seqlen_k + kTileN - 1) / kTileN;
  int ntile[2];
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const int row0 = wk.qblk * kCtaRows + w * kTileM;
    int n = 0;
    if (w < L::kQTiles && row0 < wk.seqlen_q) {
      n = nk_tiles;
      if (CAUSAL) n = min(n, SHIFTED ? max(row0 + kTileM - 1 + cshift, 0) / kTileN + 1 : row0 / kTileN + 1);
    }
    ntile[w] = n;
  }
  const int n_max = max(ntile[0], ntile[1]);
  // A cache entry shorter than its capacity: the rows behind its last key are memory the caller
  // never wrote.  Masked score columns take care of such K rows, but P = 0 times a V row that
  // happens to hold a NaN or an infinity would still poison O, so the V warp clears those rows of
  // the last tile in shared memory before the P V that reads them (v_fixed).
  const bool v_fix = p.seqused_k != nullptr && n_max == nk_tiles && (wk.seqlen_k % kTileN) != 0;

  // ---- one-time setup -------------------------------------------------------
  // The producer lane initialises the barriers and sends the first loads (Q, K_0, V_0) on their way
  // before the CTA-wide sync, so that their latency overlaps the TMEM allocation and the sync.
  auto load_q = [&](int w) {
    mbar_arrive_expect_tx(bar(iQFull + w), L::kTileBytes);
    const int row = wk.q_row0 + wk.qblk * kCtaRows + w * kTileM;
    for (int bx = 0; bx < L::kBoxes; ++bx)
      tma_load_4d(sbase + L::kQOff + w * L::kTileBytes + bx * L::kBoxBytes, &tm_q, bar(iQFull + w),
                  bx * 64, row, wk.head, wk.batch);
  };
  auto load_k = [&](int j) {
    const int s = j % NS;
    mbar_arrive_expect_tx(bar(iKFull + s), L::kTileBytes);
    for (int bx = 0; bx < L::kBoxes; ++bx)
      tma_load_4d(sbase + L::kKOff + s * L::kTileBytes + bx * L::kBoxBytes, &tm_k, bar(iKFull + s),
                  bx * 64, wk.k_row0 + j * kTileN, wk.kv_head, wk.batch);
  };
  auto load_v = [&](int j) {
    const int s = j % NS;
    mbar_arrive_expect_tx(bar(iVFull + s), L::kTileBytes);
    for (int bx = 0; bx < L::kBoxes; ++bx)
      tma_load_4d(sbase + L::kVOff + s * L::kTileBytes + bx * L::kBoxBytes, &tm_v, bar(iVFull + s),
                  bx * 64, wk.k_row0 + j * kTileN, wk.kv_head, wk.batch);
  };
  if (threadIdx.x == kSmWarps * 32) {
    *abort_flag = 0;
    mbar_init(bar(iQFull + 0), 1);
    mbar_init(bar(iQFull + 1), 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar(iKFull + s), 1);
      mbar_init(bar(iKEmpty + s), 1);
      mbar_init(bar(iVFull + s), 1);
      mbar_init(bar(iVEmpty + s), 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(bar(iSReady + w), 1);
      mbar_init(bar(iPReady + w), kTileM);
      mbar_init(bar(iPHalf + w), kTileM);
      mbar_init(bar(iODone + w), 1);
      mbar_init(bar(iSFree + w), kTileM);
    }
    mbar_init(bar(iVFixed), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int w = 0; w < 2; ++w)
      if (ntile[w] > 0) load_q(w);
    if (n_max > 0) {
      load_k(0);
      if (NS > 1 && n_max > 1) load_k(1);
      load_v(0);
    }
  }
  if (warp == kSmWarps + 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Register rebalancing between warpgroups (first statement of every role): the softmax warps
  // keep a whole 128-wide score row in registers, the producer / issuer warpgroup needs few.
  if (warp >= kSmWarps) {
    setmaxnreg_dec<kRegsOther>();
    if (warp == kSmWarps || warp == kSmWarps + 2) {
    // ===================== TMA producers ====================================
    // K tiles from warp 8, V tiles from warp 10: each ring refills as soon as its own stage is free
    // (the first tiles went out during setup).
    if (warp == kSmWarps) {
      if (lane == 0) {
        for (int j = (NS > 1) ? 2 : 1; j < n_max; ++j) {
          const int s = j % NS;
          const int use = j / NS;
          if (use > 0) mbar_wait(bar(iKEmpty + s), (use - 1) & 1, wctx, kBarKEmpty + s);
          load_k(j);
        }
      }
    } else {
      if (lane == 0) {
        for (int j = 1; j < n_max; ++j) {
          const int s = j % NS;
          const int use = j / NS;
          if (use > 0) mbar_wait(bar(iVEmpty + s), (use - 1) & 1, wctx, kBarVEmpty + s);
          load_v(j);
        }
      }
      __syncwarp();
      if (v_fix) {
        // Rows [valid, 128) of the last V tile, every 64-column box: whole 128-byte rows, so the
        // swizzle inside a row does not matter.
        const int j = n_max - 1;
        const int s = j % NS;
        mbar_wait(bar(iVFull + s), (j / NS) & 1, wctx, kBarVFull + s);
        const int valid = wk.seqlen_k - j * kTileN;
        const int chunks = (kTileM - valid) * 8;  // 16-byte pieces per box
        for (int bx = 0; bx < L::kBoxes; ++bx) {
          uint4* base = reinterpret_cast<uint4*>(sgen + L::kVOff + s * L::kTileBytes + bx * L::kBoxBytes + valid * 128);
          for (int i = lane; i < chunks; i += 32) base[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(iVFixed));
      }
    }
    __syncwarp();
  } else if (warp == kSmWarps + 1) {
    // ===================== MMA issuer =======================================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(kTileM, kTileN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(kTileM, D, 0, 1);
      // Descriptors are stepped with 32-bit adds on their low words (address field = addr >> 4).
      constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
      const uint32_t q_lo[2] = {smem_desc_lo(sbase + L::kQOff, 16),
                                smem_desc_lo(sbase + L::kQOff + L::kTileBytes, 16)};
      // S[w] = Q[w] K_j^T : both operands K-major (head_dim contiguous), 16 head-dim
      // elements (32 bytes inside the 128-byte swizzle row) per instruction.
      // sb = score buffer (TMEM columns [128 sb, +128)), qt = query tile in shared memory.
      auto issue_qk = [&](int sb, int qt, int j) {
        const uint32_t k_lo = smem_desc_lo(sbase + L::kKOff + (j % NS) * L::kTileBytes, 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * L::kBoxBytes + (ks & 3) * 32) >> 4;
          umma_ss(tmem_base + sb * kTileN, smem_desc_join(q_lo[qt] + off, kHi),
                  smem_desc_join(k_lo + off, kHi), idesc_qk, ks > 0 ? 1u : 0u);
        }
      };
      // O[w] += P[w] V_j : A = P from TMEM (8 columns of packed fp16 per 16 keys), B = V
      // MN-major (head_dim contiguous): 16 keys = 2048 bytes per step, 64-column halves
      // kBoxBytes apart (LBO), 8-key groups 1024 bytes apart (SBO).
      // sb = buffer that holds P, ot = output accumulator.
      auto issue_pv = [&](int sb, int ot, int j, int half) {
        const uint32_t v_lo = smem_desc_lo(sbase + L::kVOff + (j % NS) * L::kTileBytes, L::kBoxBytes);
        const uint32_t t_o = L::kAlt ? tmem_base + 384 : tmem_base + 256 + ot * D;
        const uint32_t t_p = L::kAlt ? tmem_base + 256 + sb * 64 : tmem_base + sb * kTileN;
#pragma unroll
        for (int kk = 0; kk < kTileN / 32; ++kk) {
          const int ks = half * (kTileN / 32) + kk;
          umma_ts(t_o, t_p + ks * 8,
                  smem_desc_join(v_lo + ((ks * 2048) >> 4), kHi), idesc_pv,
                  (j > 0 || ks > 0) ? 1u : 0u);
        }
      };

      if constexpr (L::kAlt) {
        // One query tile, two score buffers (barrier index = buffer, parity = (j / 2) % 2).  The scores
        // of key tile j + 2 are issued as soon as the warpgroup of tile j has read its scores out of
        // the buffer (s_free), so it finds the next ones waiting; the order below follows the order
        // the events come in when the two warpgroups run half a step apart.
        const int nt = ntile[0];
        auto next_scores = [&](int j) {  // scores of key tile j + 2 into the buffer of tile j
          if (j >= 0 && j + 2 < nt) {
            const int sb = j & 1;
            const int s2 = (j + 2) % NS;
            mbar_wait(bar(iSFree + sb), (j >> 1) & 1, wctx, kBarSReady + sb);
            mbar_wait(bar(iKFull + s2), ((j + 2) / NS) & 1, wctx, kBarKFull + s2);
            tc_fence_after_sync();
            issue_qk(sb, 0, j + 2);
            tc_commit(bar(iSReady + sb));
            tc_commit(bar(iKEmpty + s2));
          }
        };
        if (nt > 0) {
          mbar_wait(bar(iQFull), 0, wctx, kBarQFull);
          for (int j = 0; j < min(nt, 2); ++j) {
            mbar_wait(bar(iKFull + j % NS), (j / NS) & 1, wctx, kBarKFull + j % NS);
            tc_fence_after_sync();
            issue_qk(j, 0, j);
            tc_commit(bar(iSReady + j));
            tc_commit(bar(iKEmpty + j % NS));
          }
          next_scores(0);
        }
        for (int j = 0; j < nt; ++j) {
          const int sb = j & 1;
          const int s = j % NS;
          mbar_wait(bar(iPHalf + sb), (j >> 1) & 1, wctx, kBarPReady + sb);
          mbar_wait(bar(iVFull + s), (j / NS) & 1, wctx, kBarVFull + s);
          if (v_fix && j == nt - 1) mbar_wait(bar(iVFixed), 0, wctx, kBarVFull + s);
          tc_fence_after_sync();
          issue_pv(sb, 0, j, 0);
          next_scores(j + 1);
          mbar_wait(bar(iPReady + sb), (j >> 1) & 1, wctx, kBarPReady + sb);
          tc_fence_after_sync();
          issue_pv(sb, 0, j, 1);
          tc_commit(bar(iODone + sb));
          tc_commit(bar(iVEmpty + s));
        }
      } else {
      if (n_max > 0) {
        mbar_wait(bar(iKFull + 0), 0, wctx, kBarKFull);
        for (int w = 0; w < 2; ++w) {
          if (ntile[w] == 0) continue;
          mbar_wait(bar(iQFull + w), 0, wctx, kBarQFull + w);
          tc_fence_after_sync();
          issue_qk(w, w, 0);
          tc_commit(bar(iSReady + w));
        }
        tc_commit(bar(iKEmpty + 0));
      }
      for (int j = 0; j < n_max; ++j) {
        const int s = j % NS;
        const int use = j / NS;
        for (int w = 0; w < 2; ++w) {
          if (j >= ntile[w]) continue;
          // P arrives in two halves of 64 keys, so that PV starts while the softmax warps are
          // still exponentiating the second half.
          mbar_wait(bar(iPHalf + w), j & 1, wctx, kBarPReady + w);
          mbar_wait(bar(iVFull + s), use & 1, wctx, kBarVFull + s);
          if (v_fix && j == n_max - 1) mbar_wait(bar(iVFixed), 0, wctx, kBarVFull + s);
          tc_fence_after_sync();
          issue_pv(w, w, j, 0);
          mbar_wait(bar(iPReady + w), j & 1, wctx, kBarPReady + w);
          tc_fence_after_sync();
          issue_pv(w, w, j, 1);
          tc_commit(bar(iODone + w));
          if (w == 1 || j >= ntile[1]) tc_commit(bar(iVEmpty + s));
          if (j + 1 < ntile[w]) {
            const int s1 = (j + 1) % NS;
            mbar_wait(bar(iKFull + s1), ((j + 1) / NS) & 1, wctx, kBarKFull + s1);
            tc_fence_after_sync();
            issue_qk(w, w, j + 1);
            tc_commit(bar(iSReady + w));
            if (w == 1 || j + 1 >= ntile[1]) tc_commit(bar(iKEmpty + s1));
          }
        }
      }
      }
    }
    __syncwarp();
  }
  } else {
    // ===================== softmax + output =================================
    setmaxnreg_inc<kRegsSoftmax>();
    {
    // kAlt (one query tile): warpgroup wg takes key tiles wg, wg + 2, ... of the one tile, from score
    // buffer wg.  Otherwise warpgroup wg owns query tile wg and takes every key tile of it.
    constexpr bool kAlt = L::kAlt;
    const int wg = warp >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q_tile0 = wk.qblk * kCtaRows + (kAlt ? 0 : wg * kTileM);  // first row of this tile (local)
    const int q_local = q_tile0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + wg * kTileN;
    const uint32_t tO = tmem_base + lane_addr + (kAlt ? 384 : 256 + wg * D);
    const uint32_t tP = kAlt ? tmem_base + lane_addr + 256 + wg * 64 : tS;  // packed fp16 P
    const int nt = kAlt ? ntile[0] : ntile[wg];
    const float c2 = p.scale_log2;
    // kAlt: the reference maximum of a row travels between the two threads that own the row (same
    // quarter, same lane, other warpgroup) through xm[row]; named barrier 1 + 2 quarter + w says
    // "warpgroup w has published" (the publisher arrives, the reader syncs; the two strictly alternate).
    float* xm = reinterpret_cast<float*>(sgen + L::kXchOff);
    float* xl = xm + kTileM;  // [2][kTileM] row sums, added in the epilogue
    auto hand_over = [&](float m) {
      xm[row] = m;
      __threadfence_block();
      asm volatile("bar.arrive %0, 64;" ::"r"(1 + 2 * quarter + wg) : "memory");
    };
    auto take_over = [&]() -> float {
      asm volatile("bar.sync %0, 64;" ::"r"(1 + 2 * quarter + (wg ^ 1)) : "memory");
      return xm[row];
    };

    float m_ref = kNegInf;
    float l = 0.f;

    for (int j = kAlt ? wg : 0; j < nt; j += kAlt ? 2 : 1) {
      const int par = kAlt ? (j >> 1) & 1 : j & 1;
      mbar_wait(bar(iSReady + wg), par, wctx, kBarSReady + wg);
      tc_fence_after_sync();
      const int kv0 = j * kTileN;
      int limit = wk.seqlen_k - kv0;  // columns c < limit are visible
      if (CAUSAL) limit = min(limit, q_local + cshift - kv0 + 1);
      const bool tile_mask =
          (kv0 + kTileN > wk.seqlen_k) || (CAUSAL && (kv0 + kTileN - 1 > q_tile0 + cshift));

      // All 128 scores of this thread's row, one TMEM round trip.
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(tS + c * 32, sr[c]);
      tmem_wait_ld();
      if (kAlt) {  // the scores are in registers: the buffer may take those of key tile j + 2
        tc_fence_before_sync();
        mbar_arrive(bar(iSFree + wg));
      }
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
      if (kAlt && j > 0) {
        // The other warpgroup's reference after key tile j - 1: bring the private row sum onto it.
        const float m_other = take_over();
        if (m_other != m_ref) {
          l = (m_ref == kNegInf) ? 0.f : l * fast_exp2((m_ref - m_other) * c2);
          m_ref = m_other;
        }
      }
      const float m_new = fmaxf(m_ref, mx);

      if (j == 0) {
        m_ref = m_new;
      } else {
        const bool need = (m_new - m_ref) * c2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // PV of the previous step must have landed before O is touched.
          if (kAlt) mbar_wait(bar(iODone + (wg ^ 1)), ((j - 1) >> 1) & 1, wctx, kBarODone + (wg ^ 1));
          else mbar_wait(bar(iODone + wg), (j - 1) & 1, wctx, kBarODone + wg);
          tc_fence_after_sync();
          const float alpha = (m_new == kNegInf) ? 1.f : fast_exp2((m_ref - m_new) * c2);
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
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
      if (kAlt) {
        hand_over(m_ref);
        // P of key tile j - 2 sits where this step's P goes: its P V must have read it.
        if (j >= 2) {
          mbar_wait(bar(iODone + wg), ((j - 2) >> 1) & 1, wctx, kBarODone + wg);
          tc_fence_after_sync();
        }
      }
      const float moff = (m_ref == kNegInf) ? 0.f : m_ref * c2;

      // P = exp2(s * c2 - m * c2) from the registers, four independent row-sum chains,
      // fp16 P back into TMEM over the first half of S.
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
          const uint64_t p01 = tile_exp2_pair<0>(i, x01);
          const uint64_t p23 = tile_exp2_pair<1>(i, x23);
          sum_a = fadd2(sum_a, p01);
          sum_b = fadd2(sum_b, p23);
          float p0, p1, p2, p3;
          unpack_f32x2(p01, p0, p1);
          unpack_f32x2(p23, p2, p3);
          pk[(i >> 1) + 0] = pack_half2(p0, p1);
          pk[(i >> 1) + 1] = pack_half2(p2, p3);
        }
        tmem_st_32x32b_x16(tP + c * 16, pk);
        if (c == 1) {  // the first 64 keys of P are in TMEM: the PV MMA may start on them
          tmem_wait_st();
          tc_fence_before_sync();
          mbar_arrive(bar(iPHalf + wg));
        }
      }
      float sum0, sum1, sum2, sum3;
      unpack_f32x2(sum_a, sum0, sum1);
      unpack_f32x2(sum_b, sum2, sum3);
      const float sum_lo = sum0 + sum1, sum_hi = sum2 + sum3;
      const float sum01 = sum_lo + sum_hi;
      l += sum01;
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(bar(iPReady + wg));
    }

    // ---- epilogue: O / l -> fp16, LSE -----------------------------------------
    if (nt > 0) {
      if (kAlt) mbar_wait(bar(iODone + ((nt - 1) & 1)), ((nt - 1) >> 1) & 1, wctx, kBarODone + ((nt - 1) & 1));
      else mbar_wait(bar(iODone + wg), (nt - 1) & 1, wctx, kBarODone + wg);
      tc_fence_after_sync();
    }
    int col0 = 0;           // first output column this thread writes
    int ncol = D;           // and how many
    bool row_ok = wg < L::kQTiles && q_local < wk.seqlen_q;  // an unused second tile owns no rows
    if (kAlt) {
      // The warpgroup that did not take the last key tile picks up the final reference (the last
      // hand-over has no other reader); then the two row sums are added, and each warpgroup
      // writes one half of the output columns.
      if (nt > 0 && ((nt - 1) & 1) != wg) {
        const float m_other = take_over();
        if (m_other != m_ref) {
          l = (m_ref == kNegInf) ? 0.f : l * fast_exp2((m_ref - m_other) * c2);
          m_ref = m_other;
        }
      }
      xl[wg * kTileM + row] = l;
      asm volatile("bar.sync %0, 64;" ::"r"(9 + quarter) : "memory");
      l += xl[(wg ^ 1) * kTileM + row];
      col0 = wg * (D / 2);
      ncol = D / 2;
      row_ok = q_local < wk.seqlen_q;
    }
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    __half* o_row = static_cast<__half*>(p.o) + wk.o_base +
                    static_cast<int64_t>(q_local) * p.o_strides.row;
    // A whole tile leaves through shared memory (the tile's Q buffer: its last Q K^T has completed)
    // and TMA stores: a thread owns a row, and 32 threads storing 16 bytes each into 32 different
    // rows of global memory is slow.  A packed sequence's last, partial tile keeps the row-by-row
    // path (the rows behind it belong to the next sequence, which a tile store would overwrite).
    const bool tile_used = (kAlt || wg < L::kQTiles) && q_tile0 < wk.seqlen_q;
    // (Not at head_dim 256: measured 5 - 10 % slower there -- the CTA then waits for the TMA unit to read
    // 64 KB of staging before it can exit, where plain stores drain behind its back.)
    const bool by_tma = D != 256 && p.store_by_tma != 0 && tile_used &&
                        (p.cu_q == nullptr || q_tile0 + kTileM <= wk.seqlen_q);
    uint8_t* stage_row = sgen + L::kQOff + (kAlt ? 0 : wg * L::kTileBytes) + row * 128;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      if (c * 32 < col0 || c * 32 >= col0 + ncol) continue;
      uint32_t r[32];
      if (nt > 0) {
        tmem_ld_32x32b_x32(tO + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (by_tma) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          uint4 out;
          out.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
          out.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
          out.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
          out.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
          // box c / 2, 16-byte chunk (c % 2) * 4 + v of the row, 128-byte XOR swizzle
          *reinterpret_cast<uint4*>(stage_row + (c >> 1) * L::kBoxBytes + ((((c & 1) * 4 + v) ^ (row & 7)) << 4)) = out;
        }
      } else if (row_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          if (c * 32 + v * 8 >= p.head_dim) continue;  // head_dim 32 / 96: no such column
          uint4 out;
          out.x = pack_half2(__uint_as_float(r[v * 8 + 0]) * inv, __uint_as_float(r[v * 8 + 1]) * inv);
          out.y = pack_half2(__uint_as_float(r[v * 8 + 2]) * inv, __uint_as_float(r[v * 8 + 3]) * inv);
          out.z = pack_half2(__uint_as_float(r[v * 8 + 4]) * inv, __uint_as_float(r[v * 8 + 5]) * inv);
          out.w = pack_half2(__uint_as_float(r[v * 8 + 6]) * inv, __uint_as_float(r[v * 8 + 7]) * inv);
          *reinterpret_cast<uint4*>(o_row + c * 32 + v * 8) = out;
        }
      }
    }
    if (row_ok && (!kAlt || wg == 0)) {
      const float lse = (nt > 0 && m_ref != kNegInf) ? m_ref * p.scale + logf(fmaxf(l, 1e-20f))
                                                      : kNegInf;
      p.lse[wk.lse_base + static_cast<int64_t>(q_local) * p.lse_strides.row] = lse;
    }
    if (by_tma) {  // the same for every thread that wrote into the tile's staging buffer
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (kAlt) asm volatile("bar.sync 15, 256;" ::: "memory");
      else asm volatile("bar.sync %0, 128;" ::"r"(13 + wg) : "memory");
      if (quarter == 0 && lane == 0 && (!kAlt || wg == 0)) {
        const uint32_t src = sbase + L::kQOff + (kAlt ? 0 : wg * L::kTileBytes);
        for (int bx = 0; bx < L::kBoxes; ++bx)
          tma_store_4d(&tm_o, src + bx * L::kBoxBytes, bx * 64, wk.q_row0 + q_tile0, wk.head, wk.batch);
        bulk_commit_group();
        bulk_wait_group_read<0>();  // the boxes must have been read before the CTA's shared memory goes away
      }
    }
    }
  }

  // ---- teardown -------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kSmWarps + 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int D, bool CAUSAL, bool SHIFTED, bool ONE_TILE>
cudaError_t launch_fwd_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& to, const FwdParams& p, int grid, cudaStream_t stream) {
  auto kern = fal_fwd_kernel<D, CAUSAL, SHIFTED, ONE_TILE>;
  static DeviceOnce configured;  // one per template instance
  cudaError_t e = configured.run([&] {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                FwdSmem<D, ONE_TILE>::kAllocBytes);
  });
  if (e != cudaSuccess) return e;
  kern<<<grid, kFwdThreads, FwdSmem<D, ONE_TILE>::kAllocBytes, stream>>>(tq, tk, tv, to, p);
  return cudaGetLastError();
}

template <int D, bool ONE_TILE>
cudaError_t launch_fwd_d(bool causal, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                         const CUtensorMap& to, const FwdParams& p, int grid, cudaStream_t stream) {
  if (causal && (p.causal_shift != 0 || p.shift_per_sequence != 0))
    return launch_fwd_t<D, true, true, ONE_TILE>(tq, tk, tv, to, p, grid, stream);
  return causal ? launch_fwd_t<D, true, false, ONE_TILE>(tq, tk, tv, to, p, grid, stream)
                : launch_fwd_t<D, false, false, ONE_TILE>(tq, tk, tv, to, p, grid, stream);
}

}  // namespace

int fwd_cta_rows(int head_dim, bool one_tile) { return (head_dim == 256 || one_tile) ? 128 : 256; }

cudaError_t launch_fwd(int head_dim, bool causal, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& to, const FwdParams& p, int grid,
                       cudaStream_t stream) {
  const bool one_tile = p.cta_rows == 128;
  if (head_dim == 256) return one_tile ? launch_fwd_d<256, true>(causal, tq, tk, tv, to, p, grid, stream) : cudaErrorInvalidValue;
  if (head_dim == 128) {
    return one_tile ? launch_fwd_d<128, true>(causal, tq, tk, tv, to, p, grid, stream)
                    : launch_fwd_d<128, false>(causal, tq, tk, tv, to, p, grid, stream);
  }
  if (head_dim == 64) {
    return one_tile ? launch_fwd_d<64, true>(causal, tq, tk, tv, to, p, grid, stream)
                    : launch_fwd_d<64, false>(causal, tq, tk, tv, to, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace fal
