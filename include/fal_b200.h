/*
 * C ABI of the B200 (sm_100a) attention library: the native boundary behind
 * the Python module `flash_attn_legacy_cuda`.
 *
 * It replaces the pybind11/torch extension of sirCamp/flash-attention-legacy
 * (csrc/flash_attn_legacy.cpp): each entry point below names the reference
 * function it stands in for.  Differences by design:
 *   - plain pointers and sizes, no torch types; the caller owns every buffer,
 *     outputs and workspaces included -- the library never allocates or frees
 *     device memory;
 *   - element strides are passed per tensor, so [B,H,N,d] and [B,N,H,d] views
 *     work without copies (head_dim must be contiguous, rows 16-byte aligned);
 *   - functions return 0 or a negative fal_error code and never throw, print
 *     or exit; fal_strerror() names a code;
 *   - launches are asynchronous on the caller's stream, with the caller's
 *     device current; no call synchronises the device;
 *   - `status` is an optional device int the kernels set non-zero if an
 *     internal wait ran out (a bug indicator); read it after synchronising.
 *
 * All tensor data is fp16, statistics are fp32, index data int32.
 * Supported head_dim: 64, 128 and 256 in every entry point.
 */
#ifndef FAL_B200_H_
#define FAL_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define FAL_API __attribute__((visibility("default")))
#else
#define FAL_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum fal_error {
  FAL_OK = 0,
  FAL_ERR_INVALID_ARGUMENT = -1,  /* shape, stride, alignment or null-pointer problem */
  FAL_ERR_UNSUPPORTED_HEAD_DIM = -2,
  FAL_ERR_WORKSPACE_TOO_SMALL = -3,
  FAL_ERR_CUDA = -4,        /* a CUDA runtime call failed; see fal_last_cuda_error() */
  FAL_ERR_TENSOR_MAP = -5,  /* the driver rejected a TMA descriptor */
  FAL_ERR_UNSUPPORTED_DEVICE = -6, /* not compute capability 10.x */
  FAL_ERR_STATIC_SCRATCH_EXCEEDED = -7 /* fal_decode_static: problem needs more than its fixed scratch */
};

/* Human-readable name of a fal_error code. */
FAL_API const char* fal_strerror(int code);

/* cudaError_t value of the last failed CUDA runtime call on this host thread (0 if none);
 * after FAL_ERR_TENSOR_MAP, 100000 + the driver's CUresult. */
FAL_API int fal_last_cuda_error(void);

/* Library version, "major.minor.patch". */
FAL_API const char* fal_version(void);

/* Values of fal_fwd's `is_causal`.  0 and 1 are the reference's flag (no mask / its top-left-aligned
 * mask).  2 aligns the mask to the bottom-right corner instead: with Nk >= Nq, query i sees keys
 * j <= i + (Nk - Nq), i.e. the queries are the LAST Nq positions of the key sequence -- a prompt
 * chunk attending to a cache that already holds earlier chunks, which the reference leaves to its
 * eager fallback (flash_attn_legacy/integrations.py:63, :77-98).  Forward only. */
enum fal_causal {
  FAL_CAUSAL_NONE = 0,
  FAL_CAUSAL_TOP_LEFT = 1,
  FAL_CAUSAL_BOTTOM_RIGHT = 2
};

/* Element strides of a tensor addressed as [batch, head, row, head_dim]. */
typedef struct fal_strides {
  int64_t batch;
  int64_t head;
  int64_t row;
} fal_strides;

/*
 * Batched forward.  Stands in for flash_attn_forward
 * (csrc/flash_attn_legacy.cpp:42-98; bound as `forward` at :295-298).
 *   q [B,Hq,Nq,d], k/v [B,Hkv,Nk,d], o [B,Hq,Nq,d] fp16; lse [B,Hq,Nq] fp32 contiguous.
 *   Causal masking (is_causal = 1) is top-left aligned: key j is visible to query i iff j <= i;
 *   is_causal = 2 (FAL_CAUSAL_BOTTOM_RIGHT, needs Nk >= Nq) shifts the diagonal by Nk - Nq.
 *   lse = natural-log sum-exp of the scaled, masked scores.
 */
FAL_API int fal_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
            int batch, int heads_q, int heads_kv, int seqlen_q, int seqlen_k, int head_dim,
            const fal_strides* q_strides, const fal_strides* k_strides,
            const fal_strides* v_strides, const fal_strides* o_strides,
            float softmax_scale, int is_causal, int* status, void* stream);

/*
 * Forward kernel variants.  A thread block takes one or two 128-row query tiles:
 *   FAL_FWD_TWO_TILES        two tiles, one softmax warpgroup each (a thread owns a whole score row),
 *                            one tile's softmax running under the other tile's MMAs;
 *   FAL_FWD_ONE_TILE         one tile, the softmax warpgroups taking alternate key tiles of it from
 *                            two score buffers: twice as many, shorter blocks, for problems whose
 *                            two-tile grid would leave SMs without a block or end in a thin wave.
 * FAL_FWD_AUTO (default) chooses per call (one tile when its waves, at 0.6 of a two-tile wave each,
 * finish first; head_dim 256 always runs one tile).  fal_set_fwd_variant forces a variant for
 * every later call in the process: a tuning and test control -- the results agree within rounding.
 * The reference picks tile sizes from a compile-time table per architecture instead
 * (csrc/include/flash_attn_common.h:157-292).
 */
enum fal_fwd_variant {
  FAL_FWD_AUTO = 0,
  FAL_FWD_ONE_TILE = 1,
  FAL_FWD_TWO_TILES = 2
};
FAL_API int fal_set_fwd_variant(int variant);

/*
 * Forward of a chunk of query tokens against a key/value cache whose entries are filled to
 * different lengths: entry b attends to the first cache_seqlens[b] rows of its cache (device int32
 * [B]; clamped to [0, cache_capacity]).  Otherwise fal_fwd: q [B,Hq,Nq,d], caches [B,Hkv,capacity,d]
 * by strides (so [B,capacity,Hkv,d] memory works as well), o, lse as there.  is_causal = 2 aligns
 * the mask to the end of every entry's keys -- query i of the chunk sees keys <= cache_seqlens[b] -
 * Nq + i, the case of a chunk of new tokens already appended to the cache; a query left without
 * any key gets o = 0, lse = -inf.  The rows of a cache behind an entry's length are never used,
 * whatever they hold.  The reference has no counterpart: its hook sends every step with a cache to
 * eager attention over the whole, equally long cache (flash_attn_legacy/integrations.py:77-98).
 */
FAL_API int fal_fwd_kvcache(const void* q, const void* k_cache, const void* v_cache, void* o, float* lse,
                            const int32_t* cache_seqlens, int batch, int heads_q, int heads_kv,
                            int seqlen_q, int cache_capacity, int head_dim,
                            const fal_strides* q_strides, const fal_strides* k_strides,
                            const fal_strides* v_strides, const fal_strides* o_strides,
                            float softmax_scale, int is_causal, int* status, void* stream);

/*
 * Packed (variable-length) forward.  Stands in for flash_attn_forward_varlen
 * (csrc/flash_attn_legacy.cpp:193-290; bound as `forward_varlen` at :299-304).
 *   q [total_q,Hq,d], k/v [total_k,Hkv,d], o [total_q,Hq,d]; lse [total_q,Hq] contiguous.
 *   cu_seqlens_* are device int32 [num_seqs+1]; no host copy of them is made.
 *   Strides: `row` is the token stride, `head` the head stride, `batch` is ignored.
 */
FAL_API int fal_fwd_varlen(const void* q, const void* k, const void* v, void* o, float* lse,
                   const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int num_seqs,
                   int total_q, int total_k, int max_seqlen_q, int max_seqlen_k,
                   int heads_q, int heads_kv, int head_dim,
                   const fal_strides* q_strides, const fal_strides* k_strides,
                   const fal_strides* v_strides, const fal_strides* o_strides,
                   float softmax_scale, int is_causal, int* status, void* stream);

/*
 * Bytes of scratch the backward needs (fp32 dQ accumulator and the
 * rowsum(dO*O) vector).  `rows` is seqlen_q (batched) or total_q (packed, with
 * batch = 1).
 */
FAL_API size_t fal_bwd_workspace_bytes(int batch, int heads_q, int rows, int head_dim);

/*
 * Batched backward.  Stands in for flash_attn_backward
 * (csrc/flash_attn_legacy.cpp:105-186; bound as `backward` at :305-309), which
 * runs precompute_D, the dK/dV/dQ kernel and the fp32->fp16 dQ cast.
 *   d_out, q, o, dq [B,Hq,Nq,d]; k, v, dk, dv [B,Hkv,Nk,d]; lse [B,Hq,Nq] contiguous.
 *   dQ is accumulated with fp32 reductions whose order is not fixed, so dq can
 *   differ in the last bit between runs (the reference's atomics do the same).
 */
FAL_API int fal_bwd(const void* d_out, const void* q, const void* k, const void* v, const void* o,
            const float* lse, void* dq, void* dk, void* dv,
            int batch, int heads_q, int heads_kv, int seqlen_q, int seqlen_k, int head_dim,
            const fal_strides* do_strides, const fal_strides* q_strides,
            const fal_strides* k_strides, const fal_strides* v_strides,
            const fal_strides* o_strides, const fal_strides* dq_strides,
            const fal_strides* dk_strides, const fal_strides* dv_strides,
            float softmax_scale, int is_causal,
            void* workspace, size_t workspace_bytes, int* status, void* stream);

/*
 * Packed backward in one launch sequence.  Replaces the per-sequence Python
 * loop of FlashAttnVarlenFunc.backward (flash_attn_legacy/flash_attn.py:119-159).
 *   lse [total_q,Hq] contiguous, as written by fal_fwd_varlen.
 */
FAL_API int fal_bwd_varlen(const void* d_out, const void* q, const void* k, const void* v, const void* o,
                   const float* lse, void* dq, void* dk, void* dv,
                   const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int num_seqs,
                   int total_q, int total_k, int max_seqlen_q, int max_seqlen_k,
                   int heads_q, int heads_kv, int head_dim,
                   const fal_strides* do_strides, const fal_strides* q_strides,
                   const fal_strides* k_strides, const fal_strides* v_strides,
                   const fal_strides* o_strides, const fal_strides* dq_strides,
                   const fal_strides* dk_strides, const fal_strides* dv_strides,
                   float softmax_scale, int is_causal,
                   void* workspace, size_t workspace_bytes, int* status, void* stream);

/*
 * Steps of a ring / context-parallel pass over one long sequence whose rows are sharded over
 * several GPUs.  The reference has no multi-GPU code at all; its long-sequence case
 * (tests/test_flash_attn.py:486-547) runs on one GPU.  Per ring step a rank calls fal_fwd (or
 * fal_bwd_partial) on its query rows against the key shard it currently holds, then one of the
 * small element-wise kernels below; nothing else touches the data between the attention kernels.
 * All tensors are addressed as [batch, head, row, head_dim] through element strides, LSE tensors
 * as [batch, head, row].
 */

/* Bytes of scratch fal_bwd_partial needs (the rowsum(dO*O) vector only). */
FAL_API size_t fal_bwd_partial_workspace_bytes(int batch, int heads_q, int rows, int head_dim);

/*
 * Backward of ONE (query rows, key shard) pair of a larger problem: the same kernels as fal_bwd
 * with the outputs left unrounded, so that a caller can sum them over several calls.
 *   dq_accum  fp32 [B,Hq,Nq,d] (rows of d contiguous floats), IN-OUT: this pair's dQ, NOT yet
 *             multiplied by softmax_scale, is ADDED to it (the caller zeroes it before the first
 *             pair and applies scale * accumulator once at the end, e.g. with fal_scale_cast_f16);
 *   dk_partial, dv_partial  fp32 [B,Hkv,Nk,d], OUT: this pair's dK (scaled) and dV, overwritten;
 *   o, lse    the FINAL output and log-sum-exp of the query rows over ALL keys of the larger problem
 *             (P is recomputed from them), lse addressed through lse_strides;
 *   is_causal 0 or 1 (top-left aligned on this pair's rows, for the pair on the diagonal).
 */
FAL_API int fal_bwd_partial(const void* d_out, const void* q, const void* k, const void* v, const void* o,
                    const float* lse, float* dq_accum, float* dk_partial, float* dv_partial,
                    int batch, int heads_q, int heads_kv, int seqlen_q, int seqlen_k, int head_dim,
                    const fal_strides* do_strides, const fal_strides* q_strides,
                    const fal_strides* k_strides, const fal_strides* v_strides,
                    const fal_strides* o_strides, const fal_strides* dq_accum_strides,
                    const fal_strides* dk_strides, const fal_strides* dv_strides,
                    const fal_strides* lse_strides, float softmax_scale, int is_causal,
                    void* workspace, size_t workspace_bytes, int* status, void* stream);

/*
 * Exact merge of two softmax partials over disjoint key sets, in place:
 *   lse_new = log(exp(lse_acc) + exp(lse_part)),
 *   o_acc   = o_acc * exp(lse_acc - lse_new) + o_part * exp(lse_part - lse_new),  lse_acc = lse_new.
 * o_acc fp32, o_part fp16 (as fal_fwd writes it), LSEs fp32.  A side with lse = -inf has weight 0.
 * init != 0: the accumulators hold nothing yet and are overwritten with the partial.
 */
FAL_API int fal_merge_partial(float* o_acc, float* lse_acc, const void* o_part, const float* lse_part,
                      int batch, int heads, int rows, int head_dim,
                      const fal_strides* o_acc_strides, const fal_strides* lse_acc_strides,
                      const fal_strides* o_part_strides, const fal_strides* lse_part_strides,
                      int init, void* stream);

/* dst += src, both fp32 (a travelling dK / dV accumulator takes a rank's partial). */
FAL_API int fal_accumulate_f32(float* dst, const float* src, int batch, int heads, int rows, int head_dim,
                       const fal_strides* dst_strides, const fal_strides* src_strides, void* stream);

/* dst (fp16) = scale * src (fp32): the one rounding at the end of an accumulation. */
FAL_API int fal_scale_cast_f16(void* dst, const float* src, int batch, int heads, int rows, int head_dim,
                       const fal_strides* dst_strides, const fal_strides* src_strides, float scale,
                       void* stream);

/*
 * Bytes of scratch fal_decode needs for its split-K partial results (no initialisation needed;
 * 16-byte aligned; calls that use the same workspace must not overlap on the GPU).
 */
FAL_API size_t fal_decode_workspace_bytes(int batch, int heads_q, int capacity, int head_dim);

/*
 * Single-token decode against a KV cache (q_len = 1): a split-K streaming pass -- in which the
 * thread block whose split contains the new token's position first writes its K/V row -- plus
 * a log-sum-exp combine.  Stands in for the eager fallback branch of the
 * reference's attention hook (flash_attn_legacy/integrations.py:77-98): no
 * causal mask, GQA by head mapping, softmax over the cached positions.
 *   q, o [B,Hq,d] contiguous; caches addressed by strides as [B,Hkv,position,d];
 *   cache_seqlens device int32 [B] (positions already valid); if k_new/v_new
 *   ([B,Hkv,d] contiguous) are given they are first written at position
 *   cache_seqlens[b] and attended to as well.  lse [B,Hq] is optional.
 *   A new token for an entry whose cache is already full (cache_seqlens[b] >= capacity) is
 *   neither stored nor attended to; the kernel then sets *status to 2000 (append overflow).
 */
FAL_API int fal_decode(const void* q, void* k_cache, void* v_cache,
               const fal_strides* k_strides, const fal_strides* v_strides,
               const int32_t* cache_seqlens, const void* k_new, const void* v_new,
               void* o, float* lse,
               int batch, int heads_q, int heads_kv, int capacity, int head_dim,
               float softmax_scale, void* workspace, size_t workspace_bytes,
               int* status, void* stream);

/*
 * fal_decode for a left-padded batch: entry b attends to cache positions
 * [cache_starts[b], cache_seqlens[b]) only (device int32 [B]; plus the appended position).
 * Stands in for the same eager branch of the reference's hook when the batch carries padding
 * (flash_attn_legacy/integrations.py:77-98 with its additive mask at :88-89): decoder-only models
 * are padded on the left for generation, so the padded keys of an entry are a prefix of its cache.
 * Same workspace and arguments as fal_decode otherwise.
 */
FAL_API int fal_decode_ranged(const void* q, void* k_cache, void* v_cache,
               const fal_strides* k_strides, const fal_strides* v_strides,
               const int32_t* cache_starts, const int32_t* cache_seqlens,
               const void* k_new, const void* v_new, void* o, float* lse,
               int batch, int heads_q, int heads_kv, int capacity, int head_dim,
               float softmax_scale, void* workspace, size_t workspace_bytes,
               int* status, void* stream);

/*
 * Decode for callers that must not allocate device memory (no counterpart in the
 * reference).  Some hosts of this library cannot call cudaMalloc at the point where
 * they decode: a serving loop that was handed a fixed memory budget at start-up, a
 * plugin callback that only receives the tensors of the operator it implements, or
 * code that must stay free of the implicit device synchronisation an allocation
 * can cause.  fal_decode needs a caller-provided workspace for its split-K partial
 * results; this variant keeps those partials in a scratch array that is part of the
 * library image instead, and otherwise behaves exactly like fal_decode (same
 * arguments minus the workspace, same kernels, same results).
 *
 * Limits and rules:
 *   - the scratch is FAL_DECODE_STATIC_SCRATCH_BYTES (8 MiB) per GPU, held by every
 *     GPU that loads the library until the process exits; a problem is accepted only
 *     if fal_decode_workspace_bytes(batch, heads_q, capacity, head_dim) fits in it,
 *     otherwise the call returns FAL_ERR_STATIC_SCRATCH_EXCEEDED and launches nothing
 *     (8 MiB covers e.g. batch 8 x 32 heads x capacity 32768 x d 128);
 *   - the call performs no cudaMalloc / cudaFree and calls no allocating library
 *     routine; inputs and outputs are still the caller's buffers;
 *   - the first call on each device looks up the scratch's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture;
 *   - all calls on a device share the one array, which keeps whatever the last call
 *     left in it.  Nothing in it has to start at zero (every slot the combine step
 *     reads is written earlier in the same call), but two calls that overlap on the
 *     GPU -- different streams, or different host threads without ordering -- race
 *     on it and corrupt each other's results.  Serialise them on one stream.
 */
#define FAL_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
FAL_API int fal_decode_static(const void* q, void* k_cache, void* v_cache,
                      const fal_strides* k_strides, const fal_strides* v_strides,
                      const int32_t* cache_seqlens, const void* k_new, const void* v_new,
                      void* o, float* lse,
                      int batch, int heads_q, int heads_kv, int capacity, int head_dim,
                      float softmax_scale, int* status, void* stream);

/*
 * Self-test of the kernels' bounded waits (no counterpart in the reference, whose kernels only use
 * __syncthreads).  Launches one small thread block that waits on a barrier nothing will complete,
 * through the same wait routine and time limit (about one second) as the attention kernels.  The
 * kernel must end by itself: afterwards *status (device int, must be 0 before) holds
 * 1000 + barrier_id and *waits_given_up (device int, optional) the number of warps whose wait gave
 * up.  The device stays usable; nothing traps or faults.
 */
FAL_API int fal_selftest_wait_timeout(int barrier_id, int* status, int* waits_given_up, void* stream);

/*
 * Optional kernel timing, off by default.  While enabled, the library records a
 * CUDA event pair on the caller's stream around each launch of the kernel kinds
 * below (events only -- no synchronisation, no device memory).  fal_profile_read
 * waits for the recorded events, returns the summed device time and launch count
 * for one kind and clears that kind's records.  The reference has no counterpart;
 * its benchmarks time whole operator calls (benchmarks/benchmark.py:36-49).
 */
enum fal_kernel_kind {
  FAL_KERNEL_FWD = 0,          /* forward main kernel */
  FAL_KERNEL_BWD = 1,          /* backward dK/dV/dQ kernel (without pre/post passes) */
  FAL_KERNEL_DECODE_SPLITK = 2 /* decode streaming pass incl. the append (without the combine) */
};
FAL_API int fal_profile_enable(int on);
FAL_API int fal_profile_read(int kind, double* total_ms, int* launches);

#ifdef __cplusplus
}
#endif

#endif /* FAL_B200_H_ */
