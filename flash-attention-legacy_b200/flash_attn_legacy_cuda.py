"""ctypes binding of `lib/libfal_b200.so`, under the module name of the reference's extension.

The reference imports a pybind11 module `flash_attn_legacy_cuda`
(csrc/flash_attn_legacy.cpp:294-310 of sirCamp/flash-attention-legacy) exposing
`forward`, `forward_varlen` and `backward`.  This module keeps those three
functions with the same arguments and return conventions, and adds
`backward_varlen` and `decode`.  All compute happens in the shared library's
sm_100a kernels; there is no PyTorch or CPU fallback -- if the library is
missing the import fails, and if the device is not a B200 the calls raise.

PyTorch is used only to allocate outputs / workspaces and to hand over raw
device pointers and the current stream.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# FAL_B200_LIB selects another build of the same library (e.g. a tuning variant).
LIB_PATH = os.environ.get("FAL_B200_LIB") or os.path.join(_HERE, "lib", "libfal_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found. Build it with: python {os.path.join(_HERE, 'build.py')}"
    )

_lib = ctypes.CDLL(LIB_PATH)


class _Strides(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int64), ("head", ctypes.c_int64), ("row", ctypes.c_int64)]


_vp = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float
_sp = ctypes.POINTER(_Strides)

_lib.fal_strerror.restype = ctypes.c_char_p
_lib.fal_strerror.argtypes = [_i]
_lib.fal_last_cuda_error.restype = _i
_lib.fal_last_cuda_error.argtypes = []
_lib.fal_version.restype = ctypes.c_char_p
_lib.fal_version.argtypes = []

_lib.fal_fwd.restype = _i
_lib.fal_fwd.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _sp, _sp, _sp, _sp, _f, _i,
                         _vp, _vp]
_lib.fal_fwd_kvcache.restype = _i
_lib.fal_fwd_kvcache.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _sp, _sp, _sp, _sp, _f, _i,
                                 _vp, _vp]
_lib.fal_fwd_varlen.restype = _i
_lib.fal_fwd_varlen.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i,
                                _sp, _sp, _sp, _sp, _f, _i, _vp, _vp]
_lib.fal_bwd_workspace_bytes.restype = ctypes.c_size_t
_lib.fal_bwd_workspace_bytes.argtypes = [_i, _i, _i, _i]
_lib.fal_bwd.restype = _i
_lib.fal_bwd.argtypes = [_vp] * 9 + [_i] * 6 + [_sp] * 8 + [_f, _i, _vp, ctypes.c_size_t, _vp, _vp]
_lib.fal_bwd_varlen.restype = _i
_lib.fal_bwd_varlen.argtypes = ([_vp] * 9 + [_vp, _vp] + [_i] * 8 + [_sp] * 8 +
                                [_f, _i, _vp, ctypes.c_size_t, _vp, _vp])
_lib.fal_decode_workspace_bytes.restype = ctypes.c_size_t
_lib.fal_decode_workspace_bytes.argtypes = [_i, _i, _i, _i]
_lib.fal_decode.restype = _i
_lib.fal_decode.argtypes = [_vp, _vp, _vp, _sp, _sp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f,
                            _vp, ctypes.c_size_t, _vp, _vp]

_lib.fal_decode_ranged.restype = _i
_lib.fal_decode_ranged.argtypes = [_vp, _vp, _vp, _sp, _sp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f,
                                   _vp, ctypes.c_size_t, _vp, _vp]

_lib.fal_decode_static.restype = _i
_lib.fal_decode_static.argtypes = [_vp, _vp, _vp, _sp, _sp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f,
                                   _vp, _vp]
DECODE_STATIC_SCRATCH_BYTES = 8 << 20

_lib.fal_profile_enable.restype = _i
_lib.fal_profile_enable.argtypes = [_i]
_lib.fal_profile_read.restype = _i
_lib.fal_profile_read.argtypes = [_i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(_i)]

_lib.fal_bwd_partial_workspace_bytes.restype = ctypes.c_size_t
_lib.fal_bwd_partial_workspace_bytes.argtypes = [_i, _i, _i, _i]
_lib.fal_bwd_partial.restype = _i
_lib.fal_bwd_partial.argtypes = [_vp] * 9 + [_i] * 6 + [_sp] * 9 + [_f, _i, _vp, ctypes.c_size_t, _vp, _vp]
_lib.fal_merge_partial.restype = _i
_lib.fal_merge_partial.argtypes = [_vp] * 4 + [_i] * 4 + [_sp] * 4 + [_i, _vp]
_lib.fal_accumulate_f32.restype = _i
_lib.fal_accumulate_f32.argtypes = [_vp, _vp] + [_i] * 4 + [_sp, _sp, _vp]
_lib.fal_scale_cast_f16.restype = _i
_lib.fal_scale_cast_f16.argtypes = [_vp, _vp] + [_i] * 4 + [_sp, _sp, _f, _vp]

_lib.fal_selftest_wait_timeout.restype = _i
_lib.fal_selftest_wait_timeout.argtypes = [_i, _vp, _vp, _vp]
_lib.fal_set_fwd_variant.restype = _i
_lib.fal_set_fwd_variant.argtypes = [_i]

__version__ = _lib.fal_version().decode()

KERNEL_FWD, KERNEL_BWD, KERNEL_DECODE_SPLITK = 0, 1, 2


FWD_AUTO, FWD_ONE_TILE, FWD_TWO_TILES = 0, 1, 2


def set_forward_variant(variant=FWD_AUTO):
    """Forces a forward kernel variant for later calls (FWD_AUTO: chosen per call); see fal_b200.h."""
    _check(_lib.fal_set_fwd_variant(int(variant)))


def selftest_wait_timeout(barrier_id=7):
    """Runs the library's bounded-wait self-test on the current device and stream.

    A block waits (about one second) on a barrier that never completes; the wait must give up and
    report.  Returns (status word, warps whose wait gave up); the status word is left set to
    1000 + barrier_id until `reset_device_status()`.
    """
    dev = torch.device("cuda", torch.cuda.current_device())
    status = _status_word(dev)
    gave_up = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(_lib.fal_selftest_wait_timeout(int(barrier_id), status.data_ptr(), gave_up.data_ptr(),
                                          ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    torch.cuda.synchronize(dev)
    return int(status.item()), int(gave_up.item())


def profile_enable(on=True):
    """Turns the library's per-kernel event timing on or off (off by default)."""
    _check(_lib.fal_profile_enable(int(bool(on))))


def profile_read(kind):
    """Returns (total_ms, launches) recorded for one kernel kind since the last read."""
    total = ctypes.c_double(0.0)
    n = _i(0)
    _check(_lib.fal_profile_read(int(kind), ctypes.byref(total), ctypes.byref(n)))
    return total.value, n.value

# One device status word per GPU (a 4-byte tensor created on first use); kernels set it non-zero if
# an internal wait ran out (1000 + barrier id) or a decode append found its cache full (2000).
_status = {}


def _status_word(device):
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[idx] = t
    return t


def device_status(device=None):
    """Synchronises and returns the device status word (0 = no kernel reported a problem)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    t = _status_word(device)
    torch.cuda.synchronize(device)
    return int(t.item())


def reset_device_status(device=None):
    """Clears the device status word (and creates it if this is the first use on the device)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    _status_word(torch.device(device)).zero_()


def _check(rc):
    if rc != 0:
        msg = _lib.fal_strerror(rc).decode()
        if rc in (-4, -5):
            msg += f" (CUDA error code {_lib.fal_last_cuda_error()})"
        raise RuntimeError(f"flash_attn_legacy_cuda: {msg}")


def _bhn_strides(t):
    """Strides of a [B, H, N, d] view."""
    return _Strides(t.stride(0), t.stride(1), t.stride(2))


def _packed_strides(t):
    """Strides of a [total, H, d] view."""
    return _Strides(0, t.stride(1), t.stride(0))


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda_half(name, t, ndim):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be on CUDA")
    if t.dtype != torch.float16:
        raise RuntimeError(f"{name} must be float16")
    if t.dim() != ndim:
        raise RuntimeError(f"{name} must be {ndim}D")
    if t.stride(-1) != 1:
        raise RuntimeError(f"{name} must have a contiguous last dimension")


def _same_device(*ts):
    dev = ts[0].device
    for t in ts:
        if t is not None and t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    if dev.index != torch.cuda.current_device():
        raise RuntimeError("tensors must live on the current CUDA device")


def forward(Q, K, V, softmax_scale, is_causal=False, out=None, lse=None):
    """Batched forward.  Q [B,Hq,N,d], K/V [B,Hkv,N,d] fp16 -> [O [B,Hq,N,d] fp16, L [B,Hq,N] fp32].

    Same contract as the reference's `forward` (csrc/flash_attn_legacy.cpp:42-98),
    including its requirement that K and V have Q's sequence length.  `out` / `lse`
    let a caller supply preallocated outputs.
    """
    _require_cuda_half("Q", Q, 4)
    _require_cuda_half("K", K, 4)
    _require_cuda_half("V", V, 4)
    _same_device(Q, K, V)
    B, Hq, N, d = Q.shape
    Hkv = K.shape[1]
    if K.shape != (B, Hkv, N, d) or V.shape != K.shape:
        raise RuntimeError("K/V must be [B, H_kv, N, d] with Q's batch, sequence length and head_dim")
    if Hq % Hkv != 0:
        raise RuntimeError("H_q must be divisible by H_kv")
    O = torch.empty((B, Hq, N, d), dtype=torch.float16, device=Q.device) if out is None else out
    L = torch.empty((B, Hq, N), dtype=torch.float32, device=Q.device) if lse is None else lse
    _check(_lib.fal_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), L.data_ptr(),
                        B, Hq, Hkv, N, N, d,
                        _bhn_strides(Q), _bhn_strides(K), _bhn_strides(V), _bhn_strides(O),
                        float(softmax_scale), int(bool(is_causal)),
                        _status_word(Q.device).data_ptr(), _stream(Q)))
    return [O, L]


def forward_rect(Q, K, V, softmax_scale, is_causal=False, bottom_right=False, out=None, lse=None):
    """Forward with seqlen_k != seqlen_q allowed.

    The causal mask is top-left aligned (key j visible to query i iff j <= i, the reference's
    convention) unless `bottom_right` is set: then, with Nk >= Nq, the queries are the last Nq
    positions of the key sequence and query i sees keys j <= i + Nk - Nq (a prompt chunk attending
    to a cache that already holds the earlier chunks).  `out`: optional fp16 [B,Hq,Nq,d] tensor
    (any strides with a contiguous head_dim) to write into; `lse`: optional contiguous fp32 [B,Hq,Nq].
    """
    _require_cuda_half("Q", Q, 4)
    _require_cuda_half("K", K, 4)
    _require_cuda_half("V", V, 4)
    _same_device(Q, K, V)
    B, Hq, Nq, d = Q.shape
    Hkv, Nk = K.shape[1], K.shape[2]
    if bottom_right and Nk < Nq:
        raise RuntimeError("bottom-right causal alignment needs seqlen_k >= seqlen_q")
    if out is not None:
        _require_cuda_half("out", out, 4)
        if tuple(out.shape) != (B, Hq, Nq, d):
            raise RuntimeError("out must be [B, H_q, N_q, d]")
    O = out if out is not None else torch.empty((B, Hq, Nq, d), dtype=torch.float16, device=Q.device)
    if lse is not None and (lse.dtype != torch.float32 or tuple(lse.shape) != (B, Hq, Nq) or not lse.is_contiguous()):
        raise RuntimeError("lse must be contiguous float32 [B, H_q, N_q]")
    L = lse if lse is not None else torch.empty((B, Hq, Nq), dtype=torch.float32, device=Q.device)
    _check(_lib.fal_fwd(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), L.data_ptr(),
                        B, Hq, Hkv, Nq, Nk, d,
                        _bhn_strides(Q), _bhn_strides(K), _bhn_strides(V), _bhn_strides(O),
                        float(softmax_scale), (2 if bottom_right else 1) if is_causal else 0,
                        _status_word(Q.device).data_ptr(), _stream(Q)))
    return [O, L]


def forward_kvcache(Q, K_cache, V_cache, cache_seqlens, softmax_scale, is_causal=True, out=None):
    """A chunk of query tokens against caches filled to a different length per entry.

    Q [B,Hq,Nq,d]; caches [B,Hkv,S,d] (any strides with a contiguous head_dim, so a [B,S,Hkv,d] cache
    is passed as its transpose(1, 2) view); cache_seqlens int32 [B] on the device: entry b attends to
    its first cache_seqlens[b] rows.  With `is_causal` the mask is aligned to the end of each entry's
    keys (query i sees keys <= cache_seqlens[b] - Nq + i): the chunk's own keys are expected to be
    in the cache already.  Returns [O [B,Hq,Nq,d], L [B,Hq,Nq]].  No device-to-host copy of the
    lengths.  The reference has no such entry point (its hook computes every step with a cache
    eagerly, flash_attn_legacy/integrations.py:77-98).
    """
    _require_cuda_half("Q", Q, 4)
    _require_cuda_half("K_cache", K_cache, 4)
    _require_cuda_half("V_cache", V_cache, 4)
    _same_device(Q, K_cache, V_cache, cache_seqlens)
    B, Hq, Nq, d = Q.shape
    Hkv, S = K_cache.shape[1], K_cache.shape[2]
    if K_cache.shape[0] != B or tuple(V_cache.shape) != tuple(K_cache.shape) or K_cache.shape[3] != d:
        raise RuntimeError("caches must be [B, H_kv, S, d] with Q's batch and head_dim")
    if cache_seqlens.dtype != torch.int32 or tuple(cache_seqlens.shape) != (B,) or not cache_seqlens.is_contiguous():
        raise RuntimeError("cache_seqlens must be contiguous int32 [B]")
    if out is not None:
        _require_cuda_half("out", out, 4)
        if tuple(out.shape) != (B, Hq, Nq, d):
            raise RuntimeError("out must be [B, H_q, N_q, d]")
    O = out if out is not None else torch.empty((B, Hq, Nq, d), dtype=torch.float16, device=Q.device)
    L = torch.empty((B, Hq, Nq), dtype=torch.float32, device=Q.device)
    _check(_lib.fal_fwd_kvcache(Q.data_ptr(), K_cache.data_ptr(), V_cache.data_ptr(), O.data_ptr(), L.data_ptr(),
                                cache_seqlens.data_ptr(), B, Hq, Hkv, Nq, S, d,
                                _bhn_strides(Q), _bhn_strides(K_cache), _bhn_strides(V_cache), _bhn_strides(O),
                                float(softmax_scale), 2 if is_causal else 0,
                                _status_word(Q.device).data_ptr(), _stream(Q)))
    return [O, L]


def _causal_code(is_causal, bottom_right):
    return (2 if bottom_right else 1) if is_causal else 0


def forward_varlen(Q, K, V, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale,
                   is_causal=False, bottom_right=False):
    """Packed forward.  Q [total_q,Hq,d], K/V [total_k,Hkv,d] -> [O [total_q,Hq,d], L [total_q,Hq]].

    Same contract as the reference's `forward_varlen` (csrc/flash_attn_legacy.cpp:193-290), but
    cu_seqlens stay on the device: there is no device-to-host copy or synchronisation.
    `bottom_right` aligns each sequence's causal mask to the end of its keys (query i sees keys
    j <= i + len_k - len_q) instead of the reference's top-left alignment.
    """
    _require_cuda_half("Q", Q, 3)
    _require_cuda_half("K", K, 3)
    _require_cuda_half("V", V, 3)
    _same_device(Q, K, V, cu_seqlens_q, cu_seqlens_k)
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise RuntimeError("cu_seqlens must be int32")
    total_q, Hq, d = Q.shape
    total_k, Hkv = K.shape[0], K.shape[1]
    num_seqs = cu_seqlens_q.numel() - 1
    if cu_seqlens_k.numel() != num_seqs + 1:
        raise RuntimeError("cu_seqlens_q and cu_seqlens_k must have the same length")
    if Hq % Hkv != 0:
        raise RuntimeError("H_q must be divisible by H_kv")
    O = torch.empty((total_q, Hq, d), dtype=torch.float16, device=Q.device)
    L = torch.empty((total_q, Hq), dtype=torch.float32, device=Q.device)
    _check(_lib.fal_fwd_varlen(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), L.data_ptr(),
                               cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), num_seqs,
                               total_q, total_k, int(max_seqlen_q), int(max_seqlen_k), Hq, Hkv, d,
                               _packed_strides(Q), _packed_strides(K), _packed_strides(V),
                               _packed_strides(O), float(softmax_scale), _causal_code(is_causal, bottom_right),
                               _status_word(Q.device).data_ptr(), _stream(Q)))
    return [O, L]


def backward_workspace_bytes(B, Hq, rows, d):
    """Bytes of scratch `backward` needs for [B,Hq,rows,d] queries (packed: B=1, rows=total_q)."""
    return int(_lib.fal_bwd_workspace_bytes(B, Hq, rows, d))


def backward(dO, Q, K, V, O, L, softmax_scale, is_causal=False, out=None, workspace=None, bottom_right=False):
    """Batched backward -> [dQ [B,Hq,N,d], dK [B,Hkv,N,d], dV [B,Hkv,N,d]] fp16.

    Same contract as the reference's `backward` (csrc/flash_attn_legacy.cpp:105-186).
    `out` (a [dQ, dK, dV] list) and `workspace` (uint8, backward_workspace_bytes long,
    256-byte aligned) let a caller reuse buffers across calls.  `bottom_right`: the causal mask of
    `forward_rect(..., bottom_right=True)` (needs Nk >= Nq).
    """
    for name, t in (("dO", dO), ("Q", Q), ("K", K), ("V", V), ("O", O)):
        _require_cuda_half(name, t, 4)
    _same_device(dO, Q, K, V, O, L)
    B, Hq, Nq, d = Q.shape
    Hkv, Nk = K.shape[1], K.shape[2]
    if dO.shape != Q.shape or O.shape != Q.shape:
        raise RuntimeError("dO and O must have Q's shape")
    if L.dtype != torch.float32 or tuple(L.shape) != (B, Hq, Nq) or not L.is_contiguous():
        raise RuntimeError("L must be contiguous float32 [B, H_q, N]")
    if out is None:
        dQ = torch.empty((B, Hq, Nq, d), dtype=torch.float16, device=Q.device)
        dK = torch.empty((B, Hkv, Nk, d), dtype=torch.float16, device=Q.device)
        dV = torch.empty((B, Hkv, Nk, d), dtype=torch.float16, device=Q.device)
    else:
        dQ, dK, dV = out
    nbytes = _lib.fal_bwd_workspace_bytes(B, Hq, Nq, d)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=Q.device) if workspace is None else workspace
    if ws.numel() < nbytes:
        raise RuntimeError("workspace too small")
    _check(_lib.fal_bwd(dO.data_ptr(), Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(),
                        L.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(),
                        B, Hq, Hkv, Nq, Nk, d,
                        _bhn_strides(dO), _bhn_strides(Q), _bhn_strides(K), _bhn_strides(V),
                        _bhn_strides(O), _bhn_strides(dQ), _bhn_strides(dK), _bhn_strides(dV),
                        float(softmax_scale), _causal_code(is_causal, bottom_right),
                        ws.data_ptr(), nbytes, _status_word(Q.device).data_ptr(), _stream(Q)))
    return [dQ, dK, dV]


def backward_varlen(dO, Q, K, V, O, L, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                    softmax_scale, is_causal=False, bottom_right=False):
    """Packed backward in one native call -> [dQ [total_q,Hq,d], dK, dV [total_k,Hkv,d]] fp16.

    Replaces the per-sequence Python loop of the reference
    (flash_attn_legacy/flash_attn.py:133-157).
    """
    for name, t in (("dO", dO), ("Q", Q), ("K", K), ("V", V), ("O", O)):
        _require_cuda_half(name, t, 3)
    _same_device(dO, Q, K, V, O, L, cu_seqlens_q, cu_seqlens_k)
    total_q, Hq, d = Q.shape
    total_k, Hkv = K.shape[0], K.shape[1]
    num_seqs = cu_seqlens_q.numel() - 1
    if L.dtype != torch.float32 or tuple(L.shape) != (total_q, Hq) or not L.is_contiguous():
        raise RuntimeError("L must be contiguous float32 [total_q, H_q]")
    dQ = torch.empty((total_q, Hq, d), dtype=torch.float16, device=Q.device)
    dK = torch.empty((total_k, Hkv, d), dtype=torch.float16, device=Q.device)
    dV = torch.empty((total_k, Hkv, d), dtype=torch.float16, device=Q.device)
    nbytes = _lib.fal_bwd_workspace_bytes(1, Hq, total_q, d)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=Q.device)
    _check(_lib.fal_bwd_varlen(dO.data_ptr(), Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(),
                               L.data_ptr(), dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(),
                               cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), num_seqs,
                               total_q, total_k, int(max_seqlen_q), int(max_seqlen_k), Hq, Hkv, d,
                               _packed_strides(dO), _packed_strides(Q), _packed_strides(K),
                               _packed_strides(V), _packed_strides(O), _packed_strides(dQ),
                               _packed_strides(dK), _packed_strides(dV),
                               float(softmax_scale), _causal_code(is_causal, bottom_right),
                               ws.data_ptr(), nbytes, _status_word(Q.device).data_ptr(), _stream(Q)))
    return [dQ, dK, dV]


# ---------------------------------------------------------------------------------------------
# Steps of a ring / context-parallel pass (no counterpart in the reference, which is single-GPU)
# ---------------------------------------------------------------------------------------------
def _require_f32(name, t, ndim):
    if not t.is_cuda or t.dtype != torch.float32 or t.dim() != ndim:
        raise RuntimeError(f"{name} must be a float32 CUDA tensor with {ndim} dimensions")


def _lse_strides(t):
    """Strides of a [B, H, N] statistics view."""
    return _Strides(t.stride(0), t.stride(1), t.stride(2))


def backward_partial_workspace_bytes(B, Hq, rows, d):
    return int(_lib.fal_bwd_partial_workspace_bytes(B, Hq, rows, d))


def backward_partial(dO, Q, K, V, O, L, softmax_scale, is_causal, dq_accum, dk_partial, dv_partial,
                     workspace=None):
    """Backward of one (query rows, key shard) pair of a larger problem, outputs left in fp32.

    `dq_accum` fp32 [B,Hq,Nq,d] (rows contiguous) is ADDED to, without the softmax scale;
    `dk_partial` / `dv_partial` fp32 [B,Hkv,Nk,d] are overwritten with this pair's dK (scaled) and dV.
    `O`, `L` are the final output and log-sum-exp of the query rows over all keys.  Views with
    strides are read and written in place.
    """
    for name, t in (("dO", dO), ("Q", Q), ("K", K), ("V", V), ("O", O)):
        _require_cuda_half(name, t, 4)
    for name, t in (("dq_accum", dq_accum), ("dk_partial", dk_partial), ("dv_partial", dv_partial)):
        _require_f32(name, t, 4)
        if t.stride(-1) != 1:
            raise RuntimeError(f"{name} must have a contiguous last dimension")
    _require_f32("L", L, 3)
    _same_device(dO, Q, K, V, O, L, dq_accum, dk_partial, dv_partial)
    B, Hq, Nq, d = Q.shape
    Hkv, Nk = K.shape[1], K.shape[2]
    if dO.shape != Q.shape or O.shape != Q.shape or tuple(L.shape) != (B, Hq, Nq):
        raise RuntimeError("dO, O must have Q's shape and L must be [B, H_q, N_q]")
    if tuple(dq_accum.shape) != (B, Hq, Nq, d) or dq_accum.stride(2) != d:
        raise RuntimeError("dq_accum must be [B, H_q, N_q, d] with contiguous rows")
    if tuple(dk_partial.shape) != tuple(K.shape) or tuple(dv_partial.shape) != tuple(V.shape) or V.shape != K.shape:
        raise RuntimeError("dk_partial / dv_partial must have K's shape")
    nbytes = _lib.fal_bwd_partial_workspace_bytes(B, Hq, Nq, d)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=Q.device) if workspace is None else workspace
    if ws.numel() < nbytes:
        raise RuntimeError("workspace too small")
    _check(_lib.fal_bwd_partial(dO.data_ptr(), Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(),
                                L.data_ptr(), dq_accum.data_ptr(), dk_partial.data_ptr(), dv_partial.data_ptr(),
                                B, Hq, Hkv, Nq, Nk, d,
                                _bhn_strides(dO), _bhn_strides(Q), _bhn_strides(K), _bhn_strides(V),
                                _bhn_strides(O), _bhn_strides(dq_accum), _bhn_strides(dk_partial),
                                _bhn_strides(dv_partial), _lse_strides(L),
                                float(softmax_scale), int(bool(is_causal)),
                                ws.data_ptr(), ws.numel(), _status_word(Q.device).data_ptr(), _stream(Q)))


def merge_partial(o_acc, lse_acc, o_part, lse_part, init=False):
    """In place: (o_acc fp32, lse_acc) <- exact merge with (o_part fp16, lse_part); see fal_merge_partial."""
    _require_f32("o_acc", o_acc, 4)
    _require_cuda_half("o_part", o_part, 4)
    _require_f32("lse_acc", lse_acc, 3)
    _require_f32("lse_part", lse_part, 3)
    _same_device(o_acc, lse_acc, o_part, lse_part)
    B, H, N, d = o_acc.shape
    if tuple(o_part.shape) != (B, H, N, d) or tuple(lse_acc.shape) != (B, H, N) or tuple(lse_part.shape) != (B, H, N):
        raise RuntimeError("merge_partial: shapes must be [B,H,N,d] / [B,H,N]")
    if o_acc.stride(-1) != 1:
        raise RuntimeError("o_acc must have a contiguous last dimension")
    _check(_lib.fal_merge_partial(o_acc.data_ptr(), lse_acc.data_ptr(), o_part.data_ptr(), lse_part.data_ptr(),
                                  B, H, N, d, _bhn_strides(o_acc), _lse_strides(lse_acc), _bhn_strides(o_part),
                                  _lse_strides(lse_part), int(bool(init)), _stream(o_acc)))


def accumulate_f32(dst, src):
    """In place: dst += src, both fp32 [B,H,N,d] views."""
    _require_f32("dst", dst, 4)
    _require_f32("src", src, 4)
    _same_device(dst, src)
    if dst.shape != src.shape or dst.stride(-1) != 1 or src.stride(-1) != 1:
        raise RuntimeError("accumulate_f32: same shape and contiguous last dimensions needed")
    B, H, N, d = dst.shape
    _check(_lib.fal_accumulate_f32(dst.data_ptr(), src.data_ptr(), B, H, N, d, _bhn_strides(dst),
                                   _bhn_strides(src), _stream(dst)))


def scale_cast_f16(src, scale=1.0, out=None):
    """fp16(scale * src) for an fp32 [B,H,N,d] view; returns the fp16 tensor."""
    _require_f32("src", src, 4)
    if src.stride(-1) != 1:
        raise RuntimeError("src must have a contiguous last dimension")
    dst = torch.empty(src.shape, dtype=torch.float16, device=src.device) if out is None else out
    _same_device(src, dst)
    B, H, N, d = src.shape
    _check(_lib.fal_scale_cast_f16(dst.data_ptr(), src.data_ptr(), B, H, N, d, _bhn_strides(dst),
                                   _bhn_strides(src), float(scale), _stream(src)))
    return dst


_decode_ws = {}


def _decode_workspace(device, nbytes):
    """Split-K scratch of the current stream, kept across calls (decode loops call once per token).

    One workspace per (device, stream): calls on different streams may overlap on the GPU and must
    not share partial results.  A workspace is replaced when a call needs more room.
    """
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _decode_ws.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _decode_ws[key] = ws
    return ws


def _decode_args(q, k_cache, v_cache, cache_seqlens, k_new, v_new, cache_layout, out, lse, cache_starts=None):
    """Checks every buffer a decode call reads or writes; returns (B, Hq, Hkv, S, d, k strides, v strides)."""
    _require_cuda_half("q", q, 3)
    _require_cuda_half("k_cache", k_cache, 4)
    _require_cuda_half("v_cache", v_cache, 4)
    _same_device(q, k_cache, v_cache, cache_seqlens, k_new, v_new, cache_starts, out, lse)
    if not q.is_contiguous():
        raise RuntimeError("q must be contiguous [B, H_q, d]")
    B, Hq, d = q.shape
    if tuple(v_cache.shape) != tuple(k_cache.shape):
        raise RuntimeError("k_cache and v_cache must have the same shape")
    if cache_layout == "bshd":
        S, Hkv = k_cache.shape[1], k_cache.shape[2]
        ks = _Strides(k_cache.stride(0), k_cache.stride(2), k_cache.stride(1))
        vs = _Strides(v_cache.stride(0), v_cache.stride(2), v_cache.stride(1))
    elif cache_layout == "bhsd":
        Hkv, S = k_cache.shape[1], k_cache.shape[2]
        ks = _Strides(k_cache.stride(0), k_cache.stride(1), k_cache.stride(2))
        vs = _Strides(v_cache.stride(0), v_cache.stride(1), v_cache.stride(2))
    else:
        raise ValueError("cache_layout must be 'bshd' or 'bhsd'")
    if k_cache.shape[0] != B or k_cache.shape[3] != d:
        raise RuntimeError("the caches must have q's batch size and head_dim")
    if Hkv == 0 or Hq % Hkv != 0:
        raise RuntimeError("H_q must be divisible by H_kv")
    if cache_seqlens.dtype != torch.int32 or cache_seqlens.numel() != B or not cache_seqlens.is_contiguous():
        raise RuntimeError("cache_seqlens must be a contiguous int32 [B] tensor")
    if cache_starts is not None and (cache_starts.dtype != torch.int32 or cache_starts.numel() != B
                                     or not cache_starts.is_contiguous()):
        raise RuntimeError("cache_starts must be a contiguous int32 [B] tensor")
    if (k_new is None) != (v_new is None):
        raise RuntimeError("k_new and v_new go together")
    if k_new is not None:
        for name, t in (("k_new", k_new), ("v_new", v_new)):
            _require_cuda_half(name, t, 3)
            if tuple(t.shape) != (B, Hkv, d) or not t.is_contiguous():
                raise RuntimeError(f"{name} must be contiguous [B, H_kv, d]")
    if out is not None and (out.dtype != torch.float16 or tuple(out.shape) != (B, Hq, d) or not out.is_contiguous()):
        raise RuntimeError("out must be contiguous float16 [B, H_q, d]")
    if lse is not None and (lse.dtype != torch.float32 or tuple(lse.shape) != (B, Hq) or not lse.is_contiguous()):
        raise RuntimeError("lse must be contiguous float32 [B, H_q]")
    return B, Hq, Hkv, S, d, ks, vs


def decode(q, k_cache, v_cache, cache_seqlens, softmax_scale, k_new=None, v_new=None,
           cache_layout="bshd", return_lse=False, out=None, cache_starts=None):
    """Single-token decode.  q [B,Hq,d]; caches [B,S,Hkv,d] ("bshd") or [B,Hkv,S,d] ("bhsd").

    If k_new / v_new ([B,Hkv,d]) are given they are written into the caches at position
    cache_seqlens[b] first (an entry whose cache is full drops its new token and the device status
    word becomes 2000).  `cache_starts` (int32 [B], optional) is the first position each entry
    attends to -- the positions before it are padding (a left-padded batch).  The split-K scratch is
    kept per (device, stream) between calls.  Returns O [B,Hq,d] fp16 (and LSE [B,Hq] fp32 if asked).
    """
    B, Hq, Hkv, S, d, ks, vs = _decode_args(q, k_cache, v_cache, cache_seqlens, k_new, v_new, cache_layout,
                                            out, None, cache_starts)
    o = torch.empty((B, Hq, d), dtype=torch.float16, device=q.device) if out is None else out
    lse = torch.empty((B, Hq), dtype=torch.float32, device=q.device) if return_lse else None
    nbytes = _lib.fal_decode_workspace_bytes(B, Hq, S, d)
    ws = _decode_workspace(q.device, nbytes)
    tail = (k_new.data_ptr() if k_new is not None else None,
            v_new.data_ptr() if v_new is not None else None,
            o.data_ptr(), lse.data_ptr() if lse is not None else None,
            B, Hq, Hkv, S, d, float(softmax_scale), ws.data_ptr(), ws.numel(),
            _status_word(q.device).data_ptr(), _stream(q))
    if cache_starts is None:
        _check(_lib.fal_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), ks, vs,
                               cache_seqlens.data_ptr(), *tail))
    else:
        _check(_lib.fal_decode_ranged(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), ks, vs,
                                      cache_starts.data_ptr(), cache_seqlens.data_ptr(), *tail))
    return (o, lse) if return_lse else o


def decode_static(q, k_cache, v_cache, cache_seqlens, softmax_scale, out, k_new=None, v_new=None,
                  cache_layout="bshd", lse=None):
    """`decode` for callers that must not allocate on the device: binding of fal_decode_static.

    Some users of this library run where device allocation is off limits -- a serving loop with
    a memory budget fixed at start-up, an operator callback that only gets the operator's own
    tensors, code that cannot afford the device-wide synchronisation an allocation may imply.
    This call therefore allocates nothing in the library, and nothing here once the device's
    status word exists: the caller passes every buffer, `out` ([B,Hq,d] fp16) and the optional
    `lse` ([B,Hq] fp32) included, and the split-K scratch is an 8 MiB array inside the library.
    The status word is a 4-byte tensor this module creates on the first call of ANY of its
    functions on a device; a caller that cannot allocate even that once calls
    `reset_device_status()` during start-up.  Problems whose scratch does not fit
    (fal_decode_workspace_bytes > 8 MiB) raise RuntimeError.  Make the first call on a device
    outside stream capture (it looks up the scratch address once), and do not let two calls
    overlap on the GPU: they share the scratch.  Returns `out`.
    """
    B, Hq, Hkv, S, d, ks, vs = _decode_args(q, k_cache, v_cache, cache_seqlens, k_new, v_new, cache_layout,
                                            out, lse)
    _check(_lib.fal_decode_static(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), ks, vs,
                                  cache_seqlens.data_ptr(),
                                  k_new.data_ptr() if k_new is not None else None,
                                  v_new.data_ptr() if v_new is not None else None,
                                  out.data_ptr(), lse.data_ptr() if lse is not None else None,
                                  B, Hq, Hkv, S, d, float(softmax_scale),
                                  _status_word(q.device).data_ptr(), _stream(q)))
    return out
