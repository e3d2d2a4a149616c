"""ctypes binding of libspf_b200.so (C ABI in include/spf_b200.h).

torch is used here for device memory and the current CUDA stream only; every
computation is a call into the library.  There is no CPU fallback: if the
library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libspf_b200.so")

HEAD_QUERY_AWARE = 1
HEAD_PIVOT = 2
HEAD_SHARED = 4

_lib = None
# kernels of this library launched so far by this process (counted per wrapper call)
LAUNCH_COUNT = 0


def _launched(n: int):
    global LAUNCH_COUNT
    LAUNCH_COUNT += n

_P, _I, _L, _D = C.c_void_p, C.c_int, C.c_int64, C.c_double

# name -> (restype, argtypes); must list every symbol include/spf_b200.h declares
SIGNATURES = {
    "spf_status_string": (C.c_char_p, [_I]),
    "spf_last_cuda_error": (C.c_char_p, []),
    "spf_version": (_I, []),
    "spf_pool_qk": (_I, [_P, _L, _L, _P, _L, _L, _I, _I, _I, _I, _I, _P, _P, _P]),
    "spf_lastblock_scratch_bytes": (_L, [_I, _I, _I]),
    "spf_lastblock_profile": (_I, [_P, _L, _L, _P, _L, _L, _I, _I, _I, _I, _I, _P, _P, _P, _L, _P]),
    "spf_lastblock_profile_static": (_I, [_P, _L, _L, _P, _L, _L, _I, _I, _I, _I, _I, _P, _P, _P]),
    "spf_profile_budgets": (_I, [_P, _P, _I, _I, _I, _D, _I, _I, _P, _P, _P, _P, _P]),
    "spf_pooled_last_row": (_I, [_P, _L, _L, _P, _I, _I, _I, _I, _I, _P, _P]),
    "spf_sharing_state_bytes": (_L, [_I, _I]),
    "spf_sharing_state_reset": (_I, [_P, _I, _I, _P]),
    "spf_sharing_state_layout": (_I, [_I, _I, C.POINTER(C.c_int64)]),
    "spf_classify_heads": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P]),
    "spf_pairwise_sqrt_jsd": (_I, [_P, _I, _I, _P, _P]),
    "spf_elect_and_share": (_I, [_P, _P, _I, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _D, _D, _D, _I,
                                 _P, _P, _P, _P]),
    "spf_build_vs_bitmap": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P]),
    "spf_query_aware_scores": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P]),
    "spf_query_aware_select": (_I, [_P, _P, _I, _I, _D, _P, _P]),
    "spf_bitmap_row_counts": (_I, [_P, _I, _I, _P, _P, _P]),
    "spf_sparse_attention": (_I, [_P, _L, _L, _P, _L, _L, _P, _L, _L, _I, _I, _I, _I, _I, _D, _P, _P, _P,
                                  _P, _I, _P, _P]),
    "spf_device_timeouts": (_I, []),
    "spf_reset_device_timeouts": (_I, []),
    "spf_set_device_wait_limit_ns": (_I, [C.c_uint64]),
    "spf_wait_limit_selftest": (_I, [_P]),
    "spf_force_generic_kernels": (_I, [_I, _I]),
    "spf_pivot_summary_width": (_L, [_I]),
    "spf_pack_pivot_summaries": (_I, [_P, _I, _I, _I, _I, _I, _P, _P]),
    "spf_merge_pivot_summaries": (_I, [_P, _I, _I, _P, _I, _P]),
    "spf_decode_scratch_bytes": (_L, [_I, _I, _I, _I]),
    "spf_decode_attention": (_I, [_P, _L, _P, _L, _L, _P, _L, _L, _I, _I, _I, _I, _D, _P, _P, _L, _P]),
    "spf_update_pivots": (_I, [_P, _P, _P, _I, _I, _I, _D, _P]),
}


class SpfError(RuntimeError):
    pass


def load(path: Optional[str] = None):
    """Load the shared library (once) and attach argument types."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise SpfError(
            f"{path} not found: build it with `python -m shareprefill_b200.csrc.build` "
            "(there is no CPU or PyTorch fallback for the sparse-prefill kernels)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def _check(rc: int, what: str):
    if rc != 0:
        lib = load()
        msg = lib.spf_status_string(rc).decode()
        if rc == -5:
            msg += ": " + lib.spf_last_cuda_error().decode()
        raise SpfError(f"{what} failed ({rc}): {msg}")


def device_timeouts() -> int:
    """Bounded device-side waits that gave up since the last reset (synchronises the device)."""
    return int(load().spf_device_timeouts())


def raise_on_device_timeouts() -> None:
    """Raise if a tcgen05 kernel gave up on a wait since the last check: the rows its CTA owned were
    never written, so whatever was computed since is not to be trusted.  The counter is cleared, so
    the next forward starts clean.  Costs one device synchronisation."""
    if _lib is None:
        return
    n = int(_lib.spf_device_timeouts())
    if n:
        _lib.spf_reset_device_timeouts()
        raise SpfError(f"{n} bounded device-side wait(s) gave up in a tcgen05 kernel since the last check: "
                       "the outputs of that forward are incomplete")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _nhd(t: torch.Tensor):
    """(pointer, token stride, head stride) of a bf16 ``[N,H,D]`` view with contiguous D."""
    if t.dtype != torch.bfloat16:
        raise SpfError("q/k/v must be bfloat16")
    if t.dim() != 3 or t.stride(2) != 1:
        raise SpfError("expected a [N,H,D] view with a contiguous head dimension")
    return t.data_ptr(), t.stride(0), t.stride(1)


def num_blocks(n_tokens: int, block_size: int) -> int:
    return -(-n_tokens // block_size)


def bitmap_words(nb: int) -> int:
    return (nb + 31) // 32


# ---------------------------------------------------------------------------- stage wrappers
# q: [N,H,D] view, k/v: [N,Hkv,D] views (any token/head strides that are multiples of 8).

def pool_qk(q: Optional[torch.Tensor], k: Optional[torch.Tensor], block_size: int):
    lib = load()
    ref = q if q is not None else k
    n, d = ref.shape[0], ref.shape[2]
    nb = num_blocks(n, block_size)
    avg_q = avg_k = None
    qp = kp = (None, 0, 0)
    hq = hk = 0
    if q is not None:
        qp, hq = _nhd(q), q.shape[1]
        avg_q = torch.empty(nb, hq, d, dtype=torch.bfloat16, device=q.device)
    if k is not None:
        kp, hk = _nhd(k), k.shape[1]
        avg_k = torch.empty(nb, hk, d, dtype=torch.bfloat16, device=k.device)
    _check(lib.spf_pool_qk(qp[0], qp[1], qp[2], kp[0], kp[1], kp[2], n, hq, hk, d, block_size,
                           _ptr(avg_q), _ptr(avg_k), _stream()), "spf_pool_qk")
    _launched(1)
    return avg_q, avg_k


def lastblock_profile(q, k, block_size: int, scratch: Optional[torch.Tensor] = None):
    lib = load()
    n, h, d = q.shape
    need = lib.spf_lastblock_scratch_bytes(n, h, block_size)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(need, dtype=torch.uint8, device=q.device)
    vertical = torch.empty(h, n, dtype=torch.float32, device=q.device)
    slash = torch.empty(h, n, dtype=torch.float32, device=q.device)
    qp, kp = _nhd(q), _nhd(k)
    _check(lib.spf_lastblock_profile(qp[0], qp[1], qp[2], kp[0], kp[1], kp[2], n, h, k.shape[1], d,
                                     block_size, vertical.data_ptr(), slash.data_ptr(),
                                     scratch.data_ptr(), scratch.numel(), _stream()),
           "spf_lastblock_profile")
    _launched(3)
    return vertical, slash


def profile_budgets(vertical, slash, block_size, pattern_threshold, min_blocks, max_blocks):
    lib = load()
    h, n = vertical.shape
    nb = num_blocks(n, block_size)
    dev = vertical.device
    nv = torch.empty(h, dtype=torch.int32, device=dev)
    ns = torch.empty(h, dtype=torch.int32, device=dev)
    vpool = torch.empty(h, nb, dtype=torch.float32, device=dev)
    spool = torch.empty(h, nb, dtype=torch.float32, device=dev)
    _check(lib.spf_profile_budgets(vertical.data_ptr(), slash.data_ptr(), h, n, block_size,
                                   float(pattern_threshold), int(min_blocks), int(min(max_blocks, 2**31 - 1)),
                                   nv.data_ptr(), ns.data_ptr(), vpool.data_ptr(), spool.data_ptr(),
                                   _stream()), "spf_profile_budgets")
    _launched(1)
    return nv, ns, vpool, spool


def pooled_last_row(q, avg_k, block_size):
    lib = load()
    n, h, d = q.shape
    nb = avg_k.shape[0]
    out = torch.empty(h, nb, dtype=torch.float32, device=q.device)
    qp = _nhd(q)
    _check(lib.spf_pooled_last_row(qp[0], qp[1], qp[2], avg_k.data_ptr(), n, h, avg_k.shape[1], d,
                                   block_size, out.data_ptr(), _stream()), "spf_pooled_last_row")
    _launched(1)
    return out


class SharingStateBuffer:
    """Device buffer holding the per-forward state of the shared clusters."""

    FIELDS = ["pivot_head", "pivot_layer", "pattern_ready", "vs_ratio", "pivot_nv", "pivot_ns",
              "pivot_vertical", "pivot_slash", "pivot_vlist", "pivot_slist", "pattern", "pivot_attn"]

    def __init__(self, n_slots: int, nb: int, device):
        lib = load()
        self.n_slots, self.nb = n_slots, nb
        self.nbytes = lib.spf_sharing_state_bytes(n_slots, nb)
        if self.nbytes <= 0:
            raise SpfError(f"unsupported sharing state size (slots={n_slots}, blocks={nb})")
        self.buf = torch.zeros(self.nbytes, dtype=torch.uint8, device=device)
        off = (C.c_int64 * 12)()
        _check(lib.spf_sharing_state_layout(n_slots, nb, off), "spf_sharing_state_layout")
        self.offsets = dict(zip(self.FIELDS, list(off)))
        self.reset()

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    def reset(self):
        _check(load().spf_sharing_state_reset(self.ptr, self.n_slots, self.nb, _stream()),
               "spf_sharing_state_reset")
        _launched(1)

    def field(self, name: str) -> torch.Tensor:
        """A typed view of one state array (for tests and cross-GPU exchange)."""
        s, nb, nbw = max(self.n_slots, 1), self.nb, bitmap_words(self.nb)
        shapes = {
            "pivot_head": ((s,), torch.int32), "pivot_layer": ((s,), torch.int32),
            "pattern_ready": ((s,), torch.int32), "vs_ratio": ((s,), torch.float32),
            "pivot_nv": ((s,), torch.int32), "pivot_ns": ((s,), torch.int32),
            "pivot_vertical": ((s, nb), torch.float32), "pivot_slash": ((s, nb), torch.float32),
            "pivot_vlist": ((s, nb), torch.int32), "pivot_slist": ((s, nb), torch.int32),
            "pattern": ((s, nb, nbw), torch.int32), "pivot_attn": ((s, nb, nb), torch.float32),
        }
        shape, dt = shapes[name]
        n = 1
        for x in shape:
            n *= x
        o = self.offsets[name]
        return self.buf[o:o + n * 4].view(dt).view(*shape)


def classify_heads(avg_qk, vpool, spool, slot_of_head, state: SharingStateBuffer):
    lib = load()
    h, nb = vpool.shape
    dev = vpool.device
    out = torch.empty(3, h, dtype=torch.float32, device=dev)
    _check(lib.spf_classify_heads(avg_qk.data_ptr(), vpool.data_ptr(), spool.data_ptr(),
                                  slot_of_head.data_ptr(), state.ptr, state.n_slots, h, nb,
                                  out[0].data_ptr(), out[1].data_ptr(), out[2].data_ptr(), _stream()),
           "spf_classify_heads")
    _launched(1)
    return out[0], out[1], out[2]


def elect_and_share(jsd_qa_all, slot_all, head_offset, jsd_v, jsd_s, vpool, spool, state, layer,
                    queryaware_threshold, similarity_threshold, fallback_threshold, min_blocks, nv, ns):
    lib = load()
    h, nb = vpool.shape
    flags = torch.empty(h, dtype=torch.int32, device=vpool.device)
    _check(lib.spf_elect_and_share(jsd_qa_all.data_ptr(), slot_all.data_ptr(), jsd_qa_all.numel(),
                                   head_offset, h, jsd_v.data_ptr(), jsd_s.data_ptr(), vpool.data_ptr(),
                                   spool.data_ptr(), state.ptr, state.n_slots, nb, int(layer),
                                   float(queryaware_threshold), float(similarity_threshold),
                                   float(fallback_threshold), int(min_blocks), nv.data_ptr(), ns.data_ptr(),
                                   flags.data_ptr(), _stream()), "spf_elect_and_share")
    _launched(1)
    return flags


def build_vs_bitmap(vpool, spool, nv, ns, flags, slot_of_head, state, bitmap=None):
    lib = load()
    h, nb = vpool.shape
    if bitmap is None:
        bitmap = torch.empty(h, nb, bitmap_words(nb), dtype=torch.int32, device=vpool.device)
    _check(lib.spf_build_vs_bitmap(vpool.data_ptr(), spool.data_ptr(), nv.data_ptr(), ns.data_ptr(),
                                   flags.data_ptr(), slot_of_head.data_ptr(), state.ptr, state.n_slots,
                                   h, nb, bitmap.data_ptr(), _stream()), "spf_build_vs_bitmap")
    _launched(1)
    return bitmap


def query_aware_scores(avg_q, avg_k, flags, scores=None):
    lib = load()
    nb, h, d = avg_q.shape
    if scores is None:
        scores = torch.zeros(h, nb, nb, dtype=torch.float32, device=avg_q.device)
    _check(lib.spf_query_aware_scores(avg_q.data_ptr(), avg_k.data_ptr(), _ptr(flags), h, avg_k.shape[1],
                                      d, nb, scores.data_ptr(), _stream()), "spf_query_aware_scores")
    _launched(1)
    return scores


def query_aware_select(scores, flags, pattern_threshold, bitmap):
    lib = load()
    h, nb, _ = scores.shape
    _check(lib.spf_query_aware_select(scores.data_ptr(), _ptr(flags), h, nb, float(pattern_threshold),
                                      bitmap.data_ptr(), _stream()), "spf_query_aware_select")
    _launched(1)
    return bitmap


def bitmap_row_counts(bitmap):
    lib = load()
    h, nb, _ = bitmap.shape
    rows = torch.empty(h, nb, dtype=torch.int32, device=bitmap.device)
    tot = torch.empty(h, dtype=torch.int64, device=bitmap.device)
    _check(lib.spf_bitmap_row_counts(bitmap.data_ptr(), h, nb, rows.data_ptr(), tot.data_ptr(), _stream()),
           "spf_bitmap_row_counts")
    _launched(1)
    return rows, tot


def sparse_attention(q, k, v, bitmap, block_size, softmax_scale, flags=None, slot_of_head=None,
                     state: Optional[SharingStateBuffer] = None, out=None):
    lib = load()
    n, h, d = q.shape
    if out is None:
        out = torch.empty(n, h, d, dtype=torch.bfloat16, device=q.device)
    qp, kp, vp = _nhd(q), _nhd(k), _nhd(v)
    _check(lib.spf_sparse_attention(qp[0], qp[1], qp[2], kp[0], kp[1], kp[2], vp[0], vp[1], vp[2], n, h,
                                    k.shape[1], d, block_size, float(softmax_scale), bitmap.data_ptr(),
                                    _ptr(flags), _ptr(slot_of_head),
                                    None if state is None else state.ptr,
                                    0 if state is None else state.n_slots, out.data_ptr(), _stream()),
           "spf_sparse_attention")
    # the tcgen05 kernel is followed by a pivot-only pass of the generic kernel when state is given
    _launched(2 if (state is not None and state.n_slots > 0 and block_size == 128 and d == 128) else 1)
    return out


_decode_scratch = {}


def decode_attention(q, k, v, softmax_scale, out=None):
    """q ``[H,D]``, k/v ``[Nk,Hkv,D]`` views -> ``[H,D]`` (one decode step, dense attention)."""
    lib = load()
    h, d = q.shape
    nk = k.shape[0]
    if q.dtype != torch.bfloat16 or q.stride(1) != 1:
        raise SpfError("decode query must be a bfloat16 [H,D] view with contiguous D")
    if k.shape != v.shape or k.shape[2] != d or k.dtype != q.dtype or v.dtype != q.dtype:
        raise SpfError(f"decode cache shapes {tuple(k.shape)}/{tuple(v.shape)} do not match query {tuple(q.shape)}")
    if out is None:
        out = torch.empty(h, d, dtype=torch.bfloat16, device=q.device)
    # split-K partials: one buffer per (device, stream), grown on demand and reused by every decode step
    # (calls on one stream are ordered: the merge kernel has consumed the partials before the next call's
    # first kernel starts)
    need = lib.spf_decode_scratch_bytes(nk, h, k.shape[1], d)
    key = (q.device, _stream())
    scratch = _decode_scratch.get(key)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=q.device)
        _decode_scratch[key] = scratch
    kp, vp = _nhd(k), _nhd(v)
    _check(lib.spf_decode_attention(q.data_ptr(), q.stride(0), kp[0], kp[1], kp[2], vp[0], vp[1], vp[2], nk, h,
                                    k.shape[1], d, float(softmax_scale), out.data_ptr(), scratch.data_ptr(),
                                    scratch.numel(), _stream()), "spf_decode_attention")
    _launched(2)
    return out


def update_pivots(flags, slot_of_head, state: SharingStateBuffer, pattern_threshold):
    lib = load()
    _check(lib.spf_update_pivots(flags.data_ptr(), slot_of_head.data_ptr(), state.ptr, state.n_slots,
                                 flags.numel(), state.nb, float(pattern_threshold), _stream()),
           "spf_update_pivots")
    _launched(2)


def pack_pivot_summaries(state: SharingStateBuffer, layer: int, h0: int, h1: int, out=None) -> torch.Tensor:
    """int32 ``[S, width]`` rows of the pivots elected in ``layer`` among heads ``[h0, h1)``."""
    lib = load()
    width = lib.spf_pivot_summary_width(state.nb)
    if out is None:
        out = torch.empty(state.n_slots, width, dtype=torch.int32, device=state.buf.device)
    _check(lib.spf_pack_pivot_summaries(state.ptr, state.n_slots, state.nb, int(layer), int(h0), int(h1),
                                        out.data_ptr(), _stream()), "spf_pack_pivot_summaries")
    _launched(1)
    return out


def merge_pivot_summaries(state: SharingStateBuffer, gathered: torch.Tensor) -> None:
    """Install flagged rows of ``gathered [ranks, S, width]`` into the state."""
    lib = load()
    assert gathered.dtype == torch.int32 and gathered.is_contiguous()
    _check(lib.spf_merge_pivot_summaries(state.ptr, state.n_slots, state.nb, gathered.data_ptr(),
                                         gathered.shape[0], _stream()), "spf_merge_pivot_summaries")
    _launched(1)


# ---------------------------------------------------------------------------- format helpers
def bitmap_to_sets(bitmap: torch.Tensor):
    """Per-head sorted flat block indices ``row*nb+col`` (the reference's list format)."""
    h, nb, nbw = bitmap.shape
    bits = (bitmap.to(torch.int64).unsqueeze(-1) >> torch.arange(32, device=bitmap.device)) & 1
    dense = bits.reshape(h, nb, nbw * 32)[:, :, :nb].bool()
    return [torch.nonzero(dense[i].reshape(-1)).flatten() for i in range(h)]


def sets_to_bitmap(sets, nb: int, device) -> torch.Tensor:
    """Inverse of ``bitmap_to_sets`` (for feeding reference-format index lists to the kernel)."""
    nbw = bitmap_words(nb)
    out = torch.zeros(len(sets), nb, nbw * 32, dtype=torch.bool)
    for i, s in enumerate(sets):
        s = s.to("cpu", torch.int64)
        s = s[s < nb * nb]
        out[i, s // nb, s % nb] = True
    w = (out.view(len(sets), nb, nbw, 32).to(torch.int64) << torch.arange(32)).sum(-1)
    w = torch.where(w >= 2**31, w - 2**32, w).to(torch.int32)
    return w.to(device)
