"""Thin typed wrappers around the kernel library's C interface.

Arguments are CUDA tensors (their ``data_ptr`` is handed over) and plain
numbers; every call runs on torch's current stream, so the calls can be
captured into a CUDA graph.  A non-zero return code raises ``KernelError``:
there is no fallback to another implementation.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

F32, BF16, F16 = 0, 1, 2
HALF_TYPES = (torch.bfloat16, torch.float16)

ERR_TOKEN_RANGE, ERR_WAIT_TIMEOUT, ERR_SLOT_RANGE, ERR_CONTEXT_RANGE = 1, 2, 4, 8

_REFUSALS = {
    -2: "a size that this kernel does not take",
    -3: "an unsupported combination of types or modes",
    -4: "a launch grid beyond the device limits",
    -5: "a bad split count",
    -6: "a pointer that is not 16-byte aligned",
    -10: "cuTensorMapEncodeTiled was not found in the driver",
    -11: "cuTensorMapEncodeTiled refused the tensor",
}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    if dt == torch.float16:
        return F16
    raise KernelError(f"the kernels take float32, bfloat16 and float16 tensors, not {dt}")


_c = ctypes
_vp, _i, _ll, _f, _ull = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float, _c.c_ulonglong
_SIGNATURES = {
    "yalm_embed": [_vp, _vp, _i, _vp, _i, _i, _i, _f, _vp, _vp],
    "yalm_rmsnorm": [_vp, _vp, _i, _ll, _vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "yalm_copy_async": [_vp, _vp, _ll, _i, _vp],
    "yalm_wait_probe": [_ull, _vp, _vp],
    "yalm_stream_wait": [_vp],
    "yalm_silu_mul": [_vp, _i, _ll, _vp, _i, _i, _i, _i, _vp],
    "yalm_rope_store": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                        _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_advance": [_vp, _vp, _vp, _i, _vp],
    "yalm_cache_write": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                       _i, _i, _f, _i, _vp, _i, _i, _vp],
    "yalm_attention_decode": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                              _i, _i, _f, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_prefill_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                   _i, _i, _f, _vp, _i, _i, _vp],
    "yalm_attention_prefill_tc": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp],
    "yalm_attention_prefill_tc_cache": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                                        _i, _f, _vp, _i, _i, _vp, _vp],
    "yalm_attention_decode_mma": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                                  _i, _i, _i, _f, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_decode_mma_fused": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i,
                                        _i, _i, _i, _i, _i, _i, _f, _i, _i, _vp, _i, _i, _vp],
    "yalm_gemm_simt": [_vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "yalm_sample": [_vp, _i, _i, _f, _ull, _vp, _vp, _vp, _vp, _vp, _vp],
    "yalm_gemm_tc": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "yalm_gemm_tc_available": [],
    "yalm_gemm_2sm": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp],
    "yalm_gemm_2sm_token_tile": [_i, _i, _i],
    "yalm_gemm_2sm_rope": [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp],
    "yalm_rope_table": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "yalm_embed_pair": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll,
                        _vp, _vp],
    "yalm_head_gate": [_vp, _i, _vp, _i, _ll, _i, _i, _i, _vp],
    "yalm_softcap": [_vp, _ll, _f, _vp],
    "yalm_element_gate": [_vp, _i, _vp, _i, _ll, _ll, _vp],
    "yalm_residual_add": [_vp, _vp, _vp, _i, _ll, _ll, _vp],
    "yalm_route_topk": [_vp, _i, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp, _vp, _vp, _vp],
    "yalm_route_plan": [_vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "yalm_gather_rows": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "yalm_gemm_grouped": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "yalm_glu_clamp": [_vp, _i, _ll, _vp, _i, _ll, _i, _f, _f, _f, _i, _vp],
    "yalm_gemm_tc_glu": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _f, _f, _vp, _vp],
    "yalm_gemm_2sm_glu": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _f, _f, _vp, _vp],
    "yalm_gemm_2sm_act": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "yalm_gemm_grouped_tc": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _f, _f,
                             _f, _vp, _vp],
    "yalm_routed_combine": [_vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "yalm_attention_pooled": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                              _i, _i, _f, _i, _vp, _i, _i, _vp, _vp, _i, _i, _vp, _i, _i, _vp],
    "yalm_attention_exact_prefill": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i,
                                     _f, _vp, _i, _i, _vp, _vp, _i, _i, _vp, _i, _i, _i, _vp],
    "yalm_qk_norm_rope_store": [_vp, _i, _ll, _vp, _vp, _vp, _i, _i, _f, _vp, _i, _i, _f, _f, _i, _vp, _vp, _vp, _vp,
                                _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp],
    "yalm_pool_blocks": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _i,
                         _i, _vp, _i, _i, _vp, _vp],
    "yalm_sum_norm": [_vp, _f, _i, _vp, _i, _ll, _vp, _f, _vp, _i, _ll, _vp, _f, _f, _vp, _f, _vp, _i, _i,
                      _i, _vp],
    "yalm_cast_rows": [_vp, _vp, _i, _ll, _vp],
    "yalm_head_norm": [_vp, _vp, _vp, _i, _ll, _i, _i, _f, _vp],
    "yalm_gated_recurrence": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "yalm_attention_keep_first": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                                  _i, _i, _i, _f, _i, _vp, _i, _i, _vp],
    "yalm_hc_step": [_vp, _i, _ll, _i, _vp, _i, _ll, _vp, _vp, _f, _vp, _vp, _f, _vp, _i, _vp, _vp],
    "yalm_token_shift": [_vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp],
    "yalm_wkv": [_vp, _i, _ll, _vp, _i, _ll, _vp, _i, _ll, _vp, _i, _ll, _vp, _i, _ll, _vp, _vp, _vp, _vp,
                 _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "yalm_wkv_out": [_vp, _vp, _vp, _vp, _i, _ll, _i, _i, _f, _vp],
    "yalm_latent_store": [_vp, _i, _ll, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                          _i, _vp, _i, _i, _vp],
    "yalm_latent_absorb_q": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp],
    "yalm_latent_expand": [_vp, _vp, _vp, _i, _ll, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "yalm_activation_rows": [_vp, _i, _ll, _vp, _i, _ll, _i, _vp],
    "yalm_norm_step": [_vp, _vp, _i, _ll, _f, _vp, _i, _ll, _f, _i, _vp, _vp, _f, _f, _i, _vp, _vp, _f, _f, _vp,
                       _i, _vp, _i, _i, _vp],
    "yalm_short_conv": [_vp, _i, _ll, _i, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp,
                        _i, _i, _i, _i, _i, _vp],
    "yalm_gated_rows": [_vp, _i, _ll, _vp, _vp, _i, _i, _i, _vp, _i, _i, _i, _vp],
    "yalm_delta_row": [_i, _i, _i, _i],
    "yalm_delta_prep": [_vp, _vp, _i, _ll, _i, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "yalm_delta_scan": [_vp, _vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp],
    "yalm_rglru": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _ll, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                   _f, _vp],
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        l = build.load()
        for name, args in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = _c.c_int
        l.yalm_uniform01.argtypes = [_ull, _c.c_uint, _c.c_uint]
        l.yalm_uniform01.restype = _c.c_float
        _lib = l
    return _lib


def loaded_library_path() -> str:
    lib()
    return build.library_path()


LAUNCHES = 0     # kernels launched through this module (a graph replay adds its captured count)


def _check(rc: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += kernels
        return
    if rc < 0:
        raise KernelError(f"{what}: refused, {_REFUSALS.get(rc, f'code {rc}')}")
    raise KernelError(f"{what}: CUDA error {rc} at launch "
                      f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the direct query is ten times cheaper than building
    a Stream object for every launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


KV_PAGE = 64     # positions per page of a paged cache


def mask_code(window: Optional[int], chunk: Optional[int] = None) -> int:
    """The kernels' ``window`` argument: a sliding window of ``window`` positions as a positive
    number, a chunked mask (a query sees the keys of its own chunk of ``chunk`` positions,
    chunks counted from position 0) as the negative chunk size, 0 for neither."""
    _need(not (window and chunk), "attention: a sliding window and a chunked mask exclude each other")
    return -int(chunk) if chunk else int(window or 0)


def most_visible(max_context: int, window: Optional[int], chunk: Optional[int] = None) -> int:
    """The most keys a query sees when no sequence is longer than ``max_context``."""
    w = int(window or chunk or 0)
    return min(max_context, w) if w else max_context


def _pages(pages, cache: torch.Tensor, G: int, hd: int):
    """(page_table pointer, pages per slot, pages) of a cache argument.  ``pages`` None: the
    cache is contiguous per sequence, [slots, G, capacity, hd].  Else ``pages`` is the int32
    table [slots, pages_per_slot] and the cache is [G, pages, 64, hd]."""
    if pages is None:
        return None, 0, 0
    _need(pages.dtype == torch.int32 and pages.dim() == 2 and pages.is_contiguous(),
          "page table: int32 [slots, pages_per_slot]")
    _need(cache.dim() == 4 and cache.shape[0] == G and tuple(cache.shape[2:]) == (KV_PAGE, hd),
          f"a paged cache is [{G}, pages, {KV_PAGE}, {hd}]")
    return pages.data_ptr(), pages.shape[1], cache.shape[1]


# --------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, x: torch.Tensor, status: torch.Tensor,
          scale: float = 1.0) -> None:
    """x[t] = table[tokens[t]] * scale, float32."""
    n, dim = x.shape
    _need(tokens.dtype == torch.int32 and tokens.numel() >= n, "embed: tokens must be int32 [n]")
    _need(table.shape[1] == dim and x.dtype == torch.float32 and x.is_contiguous()
          and table.is_contiguous(), "embed: shapes")
    _check(lib().yalm_embed(_p(tokens), _p(table), dtype_code(table.dtype), _p(x), n, dim,
                            table.shape[0], float(scale), _p(status), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            partials: Optional[torch.Tensor] = None, n_partials: int = 0,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = norm(x[rows[r]] + sum of partials) * weight; with partials and no
    ``rows`` the sum is written back to x.  partials: float32 [n_partials, N, dim]."""
    dim = x.shape[1]
    n_rows = out.shape[0]
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == dim
          and out.shape[1] == dim and x.is_contiguous() and out.is_contiguous(), "rmsnorm: shapes")
    stride = 0
    if n_partials:
        _need(partials is not None and partials.dtype == torch.float32
              and partials.shape[-1] == dim and partials.shape[-2] == x.shape[0],
              "rmsnorm: partials must be float32 [s, N, dim]")
        stride = x.shape[0] * dim
    if rows is None:
        _need(n_rows == x.shape[0], "rmsnorm: out rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_rows, "rmsnorm: rows int32")
    _check(lib().yalm_rmsnorm(_p(x), _p(partials) if n_partials else None, n_partials, stride,
                              _p(rows), _p(weight), _p(out), dtype_code(out.dtype), n_rows, dim,
                              float(eps), _stream()), "rmsnorm")


def copy_async(dst_ptr: int, src_ptr: int, n_bytes: int, to_device: bool) -> None:
    """A small copy between pinned host memory and the device on the current stream."""
    _check(lib().yalm_copy_async(dst_ptr, src_ptr, n_bytes, 1 if to_device else 0, _stream()),
           "copy_async", kernels=0)


def wait_probe(limit_ns: int, status: torch.Tensor) -> None:
    """Launches a kernel whose bounded barrier wait runs out after ``limit_ns`` and raises
    ERR_WAIT_TIMEOUT in ``status`` (the path a stuck copy or product would take)."""
    _check(lib().yalm_wait_probe(int(limit_ns), _p(status), _stream()), "wait_probe")


def stream_wait() -> None:
    _check(lib().yalm_stream_wait(_stream()), "stream_wait", kernels=0)


def silu_mul(gu: torch.Tensor, out: torch.Tensor, n_partials: int = 1, paired: bool = False) -> None:
    """gu: float32 [(n_partials,) rows, 2F]; out: [rows, F].  Columns of gu are
    (gate | up) or, with ``paired``, 16 gate columns then the 16 up columns of the
    same features, and so on."""
    rows, F = out.shape
    _need(gu.dtype == torch.float32 and gu.shape[-1] == 2 * F and gu.shape[-2] == rows
          and gu.is_contiguous() and out.is_contiguous(), "silu_mul: shapes")
    _check(lib().yalm_silu_mul(_p(gu), n_partials, rows * 2 * F, _p(out), dtype_code(out.dtype),
                               rows, F, 1 if paired else 0, _stream()), "silu_mul")


def rope_store(qkv: torch.Tensor, n_partials: int, inv_freq: torch.Tensor, batch,
               q_out: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
               v_cache: torch.Tensor, slot_pos: torch.Tensor, H: int, G: int, hd: int,
               capacity: int, write_cache: bool = True, pages=None) -> None:
    n = q_out.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(qkv.dtype == torch.float32 and qkv.shape[-1] == (H + 2 * G) * hd
          and qkv.shape[-2] == n and qkv.is_contiguous(), "rope_store: qkv float32 [(s,) N, (H+2G)hd]")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == hd // 2, "rope_store: inv_freq")
    _need(q_out.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype, "rope_store: dtypes")
    _need(q_out.is_contiguous() and kv_step.is_contiguous() and k_cache.is_contiguous()
          and v_cache.is_contiguous(), "rope_store: contiguity")
    _check(lib().yalm_rope_store(_p(qkv), n_partials, n * (H + 2 * G) * hd, _p(inv_freq),
                                 _p(batch.token_seq), _p(batch.q_start), _p(batch.seq_slot),
                                 _p(slot_pos), _p(q_out), _p(kv_step), _p(k_cache), _p(v_cache),
                                 dtype_code(q_out.dtype), n, H, G, hd, capacity,
                                 1 if write_cache else 0, pt, pps, npg, _stream()), "rope_store")


def cache_write(kv_step: torch.Tensor, batch, k_cache: torch.Tensor, v_cache: torch.Tensor,
                slot_pos: torch.Tensor, G: int, hd: int, capacity: int, pages=None) -> None:
    """This step's keys and values (kv_step [N, 2, G, hd]) into the ring rows of the
    positions the ring keeps; positions are those before the step's advance."""
    n = kv_step.shape[0]
    _need(kv_step.dtype == k_cache.dtype == v_cache.dtype and kv_step.is_contiguous()
          and k_cache.is_contiguous() and v_cache.is_contiguous()
          and kv_step.numel() == n * 2 * G * hd, "cache_write: kv_step [N, 2, G, hd] and the cache")
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _check(lib().yalm_cache_write(_p(kv_step), _p(batch.token_seq), _p(batch.q_start),
                                  _p(batch.seq_slot), _p(slot_pos), _p(k_cache), _p(v_cache),
                                  dtype_code(kv_step.dtype), n, G, hd, capacity, pt, pps, npg, _stream()),
           "cache_write")


def advance(batch, slot_pos: torch.Tensor) -> None:
    _check(lib().yalm_advance(_p(batch.q_start), _p(batch.seq_slot), _p(slot_pos), batch.n_seqs,
                              _stream()), "advance")


def attention(q: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              batch, slot_pos: torch.Tensor, out: torch.Tensor, H: int, G: int, hd: int,
              capacity: int, window: Optional[int], nsplit: int = 1,
              part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
              pages=None, chunk: Optional[int] = None, scale: Optional[float] = None,
              pooled=None, keep_first: Optional[int] = None) -> None:
    """``pooled`` = (pool_k, pool_v, pool, pool_capacity, pool_pages): one (mean key, mean value)
    row per block of ``pool`` positions, seen beside the window by the queries it lies wholly
    before (see ``pool_blocks``).  ``keep_first`` = F (with a window): the positions below F stay
    visible, at their own positions, beside the last ``window``; the cache then holds every position
    (``capacity`` is the context, not the window)."""
    n = q.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == out.dtype,
          "attention: dtypes")
    _need(hd % 8 == 0 and 0 < hd <= 256,
          f"attention: head size {hd} is not supported (multiples of 8 up to 256)")
    if nsplit > 1:
        _need(part_o is not None and part_ml is not None
              and part_o.numel() >= n * H * nsplit * hd and part_ml.numel() >= n * H * nsplit * 2
              and part_o.dtype == torch.float32 and part_ml.dtype == torch.float32,
              "attention: split scratch")
    if pooled is not None:
        pool_k, pool_v, pool, pool_cap, pool_pages = pooled
        _need(window and not chunk and pool > 0, "attention: pooled blocks go with a sliding window")
        _need(pool_k.dtype == pool_v.dtype == q.dtype and pool_k.is_contiguous() and pool_v.is_contiguous(),
              "attention: pooled rows in the keys' type")
        ppt, ppps, pnpg = _pages(pool_pages, pool_k, G, hd)
        _check(lib().yalm_attention_pooled(
            _p(q), _p(kv_step), _p(k_cache), _p(v_cache), _p(batch.token_seq), _p(batch.q_start),
            _p(batch.seq_slot), _p(slot_pos), _p(out), _p(part_o), _p(part_ml), dtype_code(q.dtype), n, H,
            G, hd, capacity, int(window), float(scale or 0.0), nsplit, pt, pps, npg, _p(pool_k),
            _p(pool_v), int(pool), int(pool_cap), ppt, ppps, pnpg, _stream()), "attention (pooled)",
            kernels=2 if nsplit > 1 else 1)
        return
    if keep_first:
        _need(window and not chunk, "attention: kept first positions go with a sliding window")
        _check(lib().yalm_attention_keep_first(
            _p(q), _p(kv_step), _p(k_cache), _p(v_cache), _p(batch.token_seq), _p(batch.q_start),
            _p(batch.seq_slot), _p(slot_pos), _p(out), _p(part_o), _p(part_ml), dtype_code(q.dtype), n, H,
            G, hd, capacity, int(window), int(keep_first), float(scale or 0.0), nsplit, pt, pps, npg,
            _stream()), "attention (kept first positions)", kernels=2 if nsplit > 1 else 1)
        return
    _check(lib().yalm_attention(_p(q), _p(kv_step), _p(k_cache), _p(v_cache), _p(batch.token_seq),
                                _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos), _p(out),
                                _p(part_o), _p(part_ml), dtype_code(q.dtype), n, H, G, hd,
                                capacity, mask_code(window, chunk), float(scale or 0.0), nsplit, pt, pps, npg,
                                _stream()), "attention",
           kernels=2 if nsplit > 1 else 1)


def attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     seq_slot: torch.Tensor, slot_pos: torch.Tensor, out: torch.Tensor,
                     part_o: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                     status: torch.Tensor, H: int, G: int, hd: int, capacity: int,
                     window: Optional[int], chunk: int, max_context: int, pages=None,
                     mask_chunk: Optional[int] = None, scale: Optional[float] = None) -> None:
    """One query per sequence over the cache (the query's own row included).  ``chunk`` is the
    kernel's keys per block; ``mask_chunk`` the chunk size of a chunked mask."""
    n = q.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype, "attention_decode: dtypes")
    visible = most_visible(max_context, window, mask_chunk)
    max_chunks = -(-visible // chunk)
    hc = -(-(H // G) // 4)
    _need(part_o.numel() >= n * H * max_chunks * hd and part_ml.numel() >= n * H * max_chunks * 2
          and counters.numel() >= n * G * hc and counters.dtype == torch.int32,
          "attention_decode: workspace")
    _check(lib().yalm_attention_decode(_p(q), _p(k_cache), _p(v_cache), _p(seq_slot), _p(slot_pos),
                                       _p(out), _p(part_o), _p(part_ml), _p(counters), _p(status),
                                       dtype_code(q.dtype), n, H, G, hd, capacity,
                                       mask_code(window, mask_chunk), float(scale or 0.0), chunk,
                                       max_context, pt, pps, npg, _stream()),
           "attention_decode")


def mma_attention_usable(dtype: torch.dtype, hd: int) -> bool:
    """The tensor-core attention kernels take bfloat16 or float16 and head sizes in steps of
    16 up to 128."""
    return dtype in HALF_TYPES and hd % 16 == 0 and 0 < hd <= 128


def attention_prefill_mma(q: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
                          v_cache: torch.Tensor, batch, slot_pos: torch.Tensor, out: torch.Tensor,
                          H: int, G: int, hd: int, capacity: int, window: Optional[int],
                          pages=None, chunk: Optional[int] = None,
                          scale: Optional[float] = None) -> None:
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == out.dtype
          and q.dtype in HALF_TYPES, "attention_prefill_mma: one 16-bit type throughout")
    _check(lib().yalm_attention_prefill_mma(_p(q), _p(kv_step), _p(k_cache), _p(v_cache),
                                            _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos),
                                            _p(out), dtype_code(q.dtype), batch.n_seqs,
                                            max(batch.q_lens), H, G, hd,
                                            capacity, mask_code(window, chunk), float(scale or 0.0),
                                            pt, pps, npg, _stream()),
           "attention_prefill_mma")


def tc_attention_usable(dtype: torch.dtype, hd: int, past, q_lens=None, capacity=None) -> bool:
    """The tcgen05 prefill attention takes bfloat16 or float16 and head size 64 or 128;
    sequences that start at their first token (every key is one of this step's), or, read
    from the cache, sequences that go on without wrapping around their ring in this step."""
    if dtype not in HALF_TYPES or hd not in (64, 128):
        return False
    if all(p == 0 for p in past):
        return True
    return (q_lens is not None and capacity is not None
            and all(p + n <= capacity for p, n in zip(past, q_lens)))


def attention_prefill_tc(q: torch.Tensor, kv_step: torch.Tensor, batch, out: torch.Tensor,
                         H: int, G: int, hd: int, window: Optional[int],
                         status: torch.Tensor, chunk: Optional[int] = None,
                         scale: Optional[float] = None) -> None:
    _need(q.dtype == kv_step.dtype == out.dtype and q.dtype in HALF_TYPES and q.is_contiguous()
          and kv_step.is_contiguous() and out.is_contiguous(),
          "attention_prefill_tc: one 16-bit type throughout")
    _check(lib().yalm_attention_prefill_tc(_p(q), _p(kv_step), _p(batch.q_start), _p(out),
                                           dtype_code(q.dtype), q.shape[0], batch.n_seqs, max(batch.q_lens), H, G, hd,
                                           mask_code(window, chunk), float(scale or 0.0), _p(status),
                                           _stream()),
           "attention_prefill_tc")


def attention_prefill_tc_cache(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch,
                               slot_pos: torch.Tensor, out: torch.Tensor, H: int, G: int, hd: int,
                               capacity: int, window: Optional[int], status: torch.Tensor,
                               pages=None, chunk: Optional[int] = None,
                               scale: Optional[float] = None) -> None:
    """attention_prefill_tc with every key (this step's too) read from the cache, which the
    step wrote before this call; for sequences that go on and do not wrap in this step."""
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype and q.dtype in HALF_TYPES
          and q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
          and out.is_contiguous(), "attention_prefill_tc_cache: one 16-bit type throughout")
    n_slots = slot_pos.numel() if pt is not None else k_cache.shape[0]
    if pt is None:
        _need(tuple(k_cache.shape[1:]) == (G, capacity, hd),
              f"attention_prefill_tc_cache: a cache of one block per sequence is [slots, {G}, {capacity}, {hd}]")
    _check(lib().yalm_attention_prefill_tc_cache(_p(q), _p(k_cache), _p(v_cache), _p(batch.q_start),
                                                 _p(batch.seq_slot), _p(slot_pos), _p(out),
                                                 dtype_code(q.dtype), q.shape[0], batch.n_seqs,
                                                 max(batch.q_lens), n_slots, H, G, hd, capacity,
                                                 mask_code(window, chunk), float(scale or 0.0), pt, pps,
                                                 npg, _p(status), _stream()),
           "attention_prefill_tc_cache")


def decode_mma_parts(max_context: int, window: Optional[int], chunks_per_block: int,
                     mask_chunk: Optional[int] = None) -> int:
    """Blocks (partial results) per query of attention_decode_mma."""
    visible = most_visible(max_context, window, mask_chunk)
    return -(-(-(-visible // 64)) // chunks_per_block)


def attention_decode_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         seq_slot: torch.Tensor, slot_pos: torch.Tensor, out: torch.Tensor,
                         part_o: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                         status: torch.Tensor, H: int, G: int, hd: int, capacity: int,
                         window: Optional[int], max_context: int, chunks_per_block: int,
                         pages=None, warps: int = 4, mask_chunk: Optional[int] = None,
                         scale: Optional[float] = None) -> None:
    """``warps``: 4 (one block to an SM) or 2 (two blocks of two warps to an SM)."""
    n = q.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype and q.dtype in HALF_TYPES,
          "attention_decode_mma: one 16-bit type throughout")
    parts = decode_mma_parts(max_context, window, chunks_per_block, mask_chunk)
    hc = -(-(H // G) // 16)
    _need(part_o.numel() >= n * H * parts * hd and part_ml.numel() >= n * H * parts * 2
          and counters.numel() >= n * G * hc and counters.dtype == torch.int32,
          "attention_decode_mma: workspace")
    _check(lib().yalm_attention_decode_mma(_p(q), _p(k_cache), _p(v_cache), _p(seq_slot),
                                           _p(slot_pos), _p(out), _p(part_o), _p(part_ml),
                                           _p(counters), _p(status), dtype_code(q.dtype), n, H, G,
                                           hd, capacity, mask_code(window, mask_chunk),
                                           float(scale or 0.0), max_context,
                                           chunks_per_block, warps, pt, pps, npg,
                                           _stream()),
           "attention_decode_mma")


def attention_decode_mma_fused(qkv: torch.Tensor, n_partials: int, cos_sin: torch.Tensor,
                               k_cache: torch.Tensor, v_cache: torch.Tensor, seq_slot: torch.Tensor,
                               slot_pos: torch.Tensor, out: torch.Tensor, part_o: torch.Tensor,
                               part_ml: torch.Tensor, counters: torch.Tensor, status: torch.Tensor,
                               H: int, G: int, hd: int, capacity: int, window: Optional[int],
                               max_context: int, chunks_per_block: int, pages=None,
                               mask_chunk: Optional[int] = None,
                               scale: Optional[float] = None) -> None:
    """attention_decode_mma with the rotary kernel's work inside: ``qkv`` is this step's q/k/v
    product as float32 slices [n_partials, n, (H + 2 G) hd] (or [n, ...] for one), ``cos_sin`` the
    step's table of ``rope_table`` [n, hd / 2, 2]; q is rotated in the kernel and the new k and v
    rows are written into the cache by it."""
    n = out.shape[0]
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    row = (H + 2 * G) * hd
    _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.numel() == n_partials * n * row,
          "attention_decode_mma_fused: qkv is float32 [n_partials, n, (H + 2 G) hd]")
    _need(cos_sin.dtype == torch.float32 and cos_sin.is_contiguous()
          and tuple(cos_sin.shape) == (n, hd // 2, 2), "attention_decode_mma_fused: cos_sin [n, hd/2, 2]")
    _need(k_cache.dtype == v_cache.dtype == out.dtype and out.dtype in HALF_TYPES,
          "attention_decode_mma_fused: one 16-bit type throughout")
    parts = decode_mma_parts(max_context, window, chunks_per_block, mask_chunk)
    hc = -(-(H // G) // 16)
    _need(part_o.numel() >= n * H * parts * hd and part_ml.numel() >= n * H * parts * 2
          and counters.numel() >= n * G * hc and counters.dtype == torch.int32,
          "attention_decode_mma_fused: workspace")
    _check(lib().yalm_attention_decode_mma_fused(_p(qkv), n_partials, n * row, _p(cos_sin), _p(k_cache),
                                                 _p(v_cache), _p(seq_slot), _p(slot_pos), _p(out),
                                                 _p(part_o), _p(part_ml), _p(counters), _p(status),
                                                 dtype_code(out.dtype), n, H, G, hd, capacity,
                                                 mask_code(window, mask_chunk), float(scale or 0.0),
                                                 max_context, chunks_per_block, pt, pps, npg, _stream()),
           "attention_decode_mma_fused")


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(out.shape) == (M, N) and a.is_contiguous()
          and w.is_contiguous() and out.is_contiguous(), "gemm_simt: shapes")
    _need(not accumulate or out.dtype == torch.float32, "gemm_simt: accumulate needs float32 out")
    _check(lib().yalm_gemm_simt(_p(a), dtype_code(a.dtype), _p(w), dtype_code(w.dtype), _p(out),
                                dtype_code(out.dtype), M, N, K, 1 if accumulate else 0, _stream()),
           "gemm_simt")


GEMM_STORE, GEMM_ADD, GEMM_SILU_MUL, GEMM_SPLIT, GEMM_SILU_PAIRED = 0, 1, 2, 3, 4


def gemm_tc_usable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == w.dtype and a.dtype in HALF_TYPES and a.shape[1] % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, status: torch.Tensor,
            splits: int = 1, glu: Optional[tuple] = None) -> None:
    """``glu`` = (slope, limit, shift): modes GEMM_SILU_MUL and GEMM_SILU_PAIRED compute
    g' sigmoid(slope g') (u' + shift) under the clamps of ``glu_clamp`` instead of SiLU(g) u."""
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K
          and a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "gemm_tc: operands")
    if mode in (GEMM_SILU_MUL, GEMM_SILU_PAIRED):
        _need(tuple(out.shape) == (M, N // 2), "gemm_tc: silu-mul out is [M, N/2]")
    elif mode == GEMM_SPLIT:
        _need(out.dtype == torch.float32 and out.numel() >= splits * M * N, "gemm_tc: split scratch")
    else:
        _need(tuple(out.shape) == (M, N), "gemm_tc: out is [M, N]")
    if glu is not None:
        _need(mode in (GEMM_SILU_MUL, GEMM_SILU_PAIRED), "gemm_tc: an activation needs a gated mode")
        _check(lib().yalm_gemm_tc_glu(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M,
                                      N, K, mode, float(glu[0]), float(glu[1]), float(glu[2]), _p(status),
                                      _stream()), "gemm_tc")
        return
    _check(lib().yalm_gemm_tc(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M,
                              N, K, mode, splits, _p(status), _stream()), "gemm_tc")


def gemm_2sm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int,
             status: torch.Tensor, splits: int = 1, glu: Optional[tuple] = None) -> None:
    """Two-SM tcgen05 product (pairs of blocks on one 256-feature tile) with a fused epilogue;
    with GEMM_SPLIT, ``splits`` slices of K as 32-bit partial sums in out [splits, M, N]."""
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K
          and a.is_contiguous() and w.is_contiguous() and out.is_contiguous(), "gemm_2sm: operands")
    if mode == GEMM_SPLIT:
        _need(out.dtype == torch.float32 and tuple(out.shape) == (splits, M, N),
              "gemm_2sm: split-K partials are float32 [splits, M, N]")
    else:
        _need(tuple(out.shape) == ((M, N // 2) if mode in (GEMM_SILU_MUL, GEMM_SILU_PAIRED) else (M, N)),
              "gemm_2sm: out shape")
    if glu is not None:
        _need(mode in (GEMM_SILU_MUL, GEMM_SILU_PAIRED), "gemm_2sm: an activation needs a gated mode")
        _check(lib().yalm_gemm_2sm_glu(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M,
                                       N, K, mode, float(glu[0]), float(glu[1]), float(glu[2]), _p(status),
                                       _stream()), "gemm_2sm")
        return
    _check(lib().yalm_gemm_2sm(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M,
                               N, K, mode, splits, _p(status), _stream()), "gemm_2sm")


def gemm_2sm_act(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act: int, status: torch.Tensor) -> None:
    """out = act(a @ w.T) in one launch of the two-SM product: the activation (GELU_TANH or TANH)
    is applied to the 32-bit sums in the epilogue, before they are rounded to out's type."""
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K and a.is_contiguous()
          and w.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (M, N)
          and out.dtype in (a.dtype, torch.float32), "gemm_2sm_act: operands")
    _check(lib().yalm_gemm_2sm_act(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype), M, N, K,
                                   int(act), _p(status), _stream()), "gemm_2sm_act")


def gemm_2sm_token_tile(M: int, N: int, splits: int = 1) -> int:
    """The token tile (256 or 240) that gemm_2sm takes for these sizes."""
    return lib().yalm_gemm_2sm_token_tile(M, N, splits)


class _RopeArgs(ctypes.Structure):
    _fields_ = [("cos_sin", _vp), ("token_seq", _vp), ("q_start", _vp), ("seq_slot", _vp),
                ("slot_pos", _vp), ("q_out", _vp), ("kv_step", _vp), ("k_cache", _vp),
                ("v_cache", _vp), ("page_table", _vp), ("pages_per_slot", _i), ("n_pages", _i),
                ("H", _i), ("G", _i), ("hd", _i), ("capacity", _i), ("write_cache", _i)]


def gemm_2sm_rope_usable(a: torch.Tensor, w: torch.Tensor, hd: int) -> bool:
    """The q/k/v product with the rotary epilogue takes what the tcgen05 product takes and
    head sizes 16, 32, 64 and 128: a block's 128 rows then hold whole heads, and the 16
    features a thread stores lie in one head."""
    return gemm_tc_usable(a, w) and hd % 16 == 0 and 128 % hd == 0


def rope_table(inv_freq: torch.Tensor, batch, slot_pos: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = (cos, sin) of position(t) * inv_freq[i] for the batch's tokens."""
    n, half = batch.n_tokens, inv_freq.numel()
    _need(inv_freq.dtype == torch.float32 and out.dtype == torch.float32 and out.is_contiguous()
          and tuple(out.shape) == (n, half, 2), "rope_table: out is float32 [tokens, hd/2, 2]")
    _check(lib().yalm_rope_table(_p(inv_freq), _p(batch.token_seq), _p(batch.q_start),
                                 _p(batch.seq_slot), _p(slot_pos), _p(out), n, half, _stream()),
           "rope_table")


def gemm_2sm_rope(a: torch.Tensor, w: torch.Tensor, cos_sin: torch.Tensor, batch,
                  q_out: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
                  v_cache: torch.Tensor, slot_pos: torch.Tensor, H: int, G: int, hd: int,
                  capacity: int, status: torch.Tensor, write_cache: bool = True, pages=None) -> None:
    """rope_store(a @ w.T) in one launch: the two-SM product of many tokens whose epilogue
    rotates q and k and writes q_out, kv_step and the cache rows (no 32-bit q/k/v in between).
    ``cos_sin`` is the table of ``rope_table`` for this batch."""
    M, K = a.shape
    N = w.shape[0]
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[1] == K and a.is_contiguous()
          and w.is_contiguous() and N == (H + 2 * G) * hd, "gemm_2sm_rope: operands")
    _need(q_out.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == a.dtype
          and q_out.is_contiguous() and kv_step.is_contiguous() and k_cache.is_contiguous()
          and v_cache.is_contiguous() and q_out.numel() == M * H * hd
          and kv_step.numel() == M * 2 * G * hd and cos_sin.dtype == torch.float32
          and cos_sin.is_contiguous() and tuple(cos_sin.shape) == (M, hd // 2, 2),
          "gemm_2sm_rope: buffers")
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    r = _RopeArgs()
    r.cos_sin, r.token_seq, r.q_start = _p(cos_sin), _p(batch.token_seq), _p(batch.q_start)
    r.seq_slot, r.slot_pos = _p(batch.seq_slot), _p(slot_pos)
    r.q_out, r.kv_step, r.k_cache, r.v_cache = _p(q_out), _p(kv_step), _p(k_cache), _p(v_cache)
    r.page_table, r.pages_per_slot, r.n_pages = pt, pps, npg
    r.H, r.G, r.hd, r.capacity, r.write_cache = H, G, hd, capacity, 1 if write_cache else 0
    _check(lib().yalm_gemm_2sm_rope(_p(a), _p(w), dtype_code(a.dtype), M, N, K, ctypes.byref(r),
                                    _p(status), _stream()), "gemm_2sm_rope")


# ---- small row-wise kernels some architectures add ------------------------------------
def embed_pair(batch, table: torch.Tensor, pair_table: torch.Tensor, prev_token: torch.Tensor,
               slot_pos: torch.Tensor, x: torch.Tensor, x_copy: Optional[torch.Tensor],
               mul_prev: int, mul_cur: int, status: torch.Tensor) -> None:
    """x[t] = table[token] + pair_table[row]; row = buckets (the table's last row) at a
    sequence's position 0, else (previous token * mul_prev + token * mul_cur) mod buckets.
    ``prev_token`` int32 [slots]: each sequence's last token so far, kept up to date here."""
    n, dim = x.shape
    _need(table.dtype == pair_table.dtype and table.shape[1] == dim == pair_table.shape[1]
          and table.is_contiguous() and pair_table.is_contiguous() and x.dtype == torch.float32
          and x.is_contiguous() and pair_table.shape[0] >= 2, "embed_pair: tables and x")
    _need(prev_token.dtype == torch.int32 and prev_token.is_contiguous(), "embed_pair: prev_token int32")
    _need(x_copy is None or (x_copy.dtype == torch.float32 and x_copy.is_contiguous()
                             and x_copy.shape == x.shape), "embed_pair: x_copy like x")
    _check(lib().yalm_embed_pair(_p(batch.tokens), _p(batch.token_seq), _p(batch.q_start),
                                 _p(batch.seq_slot), _p(slot_pos), _p(table), _p(pair_table),
                                 dtype_code(table.dtype), _p(prev_token), _p(x), _p(x_copy), n, dim,
                                 table.shape[0], pair_table.shape[0] - 1, int(mul_prev), int(mul_cur),
                                 _p(status), _stream()), "embed_pair")


def head_gate(o: torch.Tensor, g: torch.Tensor, n_partials: int, H: int, hd: int) -> None:
    """o [n, H * hd] *= sigmoid(g) per head; g float32 [n_partials, n, H] slices that are summed."""
    n = o.shape[0]
    _need(o.is_contiguous() and o.shape[1] == H * hd and g.dtype == torch.float32 and g.is_contiguous()
          and g.numel() >= n_partials * n * H, "head_gate: shapes")
    _check(lib().yalm_head_gate(_p(o), dtype_code(o.dtype), _p(g), n_partials, n * H, n, H, hd, _stream()),
           "head_gate")


def element_gate(o: torch.Tensor, g: torch.Tensor, n_partials: int) -> None:
    """o [n, F] *= sigmoid(g) feature by feature; g float32 [n_partials, n, F] slices that are summed."""
    n = o.numel()
    _need(o.is_contiguous() and g.dtype == torch.float32 and g.is_contiguous()
          and g.numel() >= n_partials * n, "element_gate: shapes")
    if n % 4 or g.data_ptr() % 16:
        head_gate(o, g, n_partials, o.shape[1], 1)       # odd sizes: a "head" per feature
        return
    _check(lib().yalm_element_gate(_p(o), dtype_code(o.dtype), _p(g), n_partials, n, n, _stream()),
           "element_gate")


def softcap(v: torch.Tensor, cap: float) -> None:
    """v <- cap * tanh(v / cap), in place, float32."""
    _need(v.dtype == torch.float32 and v.is_contiguous(), "softcap: float32")
    _check(lib().yalm_softcap(_p(v), v.numel(), float(cap), _stream()), "softcap")


def residual_add(x: torch.Tensor, y: torch.Tensor, partials: Optional[torch.Tensor] = None,
                 n_partials: int = 0) -> None:
    """x += y (+ the sum of ``n_partials`` slices shaped like x), float32."""
    _need(x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
          and x.numel() == y.numel(), "residual_add: float32 tensors of one size")
    if n_partials:
        _need(partials is not None and partials.dtype == torch.float32 and partials.is_contiguous()
              and partials.numel() >= n_partials * x.numel(), "residual_add: partials")
    _check(lib().yalm_residual_add(_p(x), _p(y), _p(partials) if n_partials else None, n_partials,
                                   x.numel(), x.numel(), _stream()), "residual_add")


def exact_attention_usable(dtype: torch.dtype, hd: int, chunk: Optional[int] = None) -> bool:
    """The tensor-core prefill attention that keeps its softmax weights in 32 bits takes bfloat16 or
    float16, head sizes 32, 64, 128 and 256, and a sliding window or none (no chunked mask)."""
    return dtype in HALF_TYPES and hd in (32, 64, 128, 256) and not chunk


def attention_exact_prefill(q: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, batch, slot_pos: torch.Tensor, out: torch.Tensor,
                            H: int, G: int, hd: int, capacity: int, window: Optional[int], pages=None,
                            scale: Optional[float] = None, pooled=None, keep_first: Optional[int] = None) -> None:
    """Prefill attention on tensor cores with the weights split into three 16-bit terms (no
    rounding of the softmax weights); ``pooled`` and ``keep_first`` as in ``attention``."""
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(q.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype == out.dtype and q.dtype in HALF_TYPES
          and q.is_contiguous() and kv_step.is_contiguous() and out.is_contiguous(),
          "attention_exact_prefill: one 16-bit type throughout")
    pk = pv = ppt = None
    pool = pcap = ppps = pnpg = 0
    if pooled is not None:
        pk, pv, pool, pcap, pool_pages = pooled
        _need(bool(window) and pool > 0 and pk.dtype == pv.dtype == q.dtype,
              "attention_exact_prefill: pooled rows go with a sliding window")
        ppt, ppps, pnpg = _pages(pool_pages, pk, G, hd)
    _need(not keep_first or (bool(window) and pooled is None),
          "attention_exact_prefill: kept first positions go with a sliding window and no pooled rows")
    _check(lib().yalm_attention_exact_prefill(
        _p(q), _p(kv_step), _p(k_cache), _p(v_cache), _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos),
        _p(out), dtype_code(q.dtype), batch.n_seqs, max(batch.q_lens), H, G, hd, capacity, int(window or 0),
        float(scale or 0.0), pt, pps, npg, _p(pk), _p(pv), int(pool), int(pcap), ppt, ppps, pnpg,
        int(keep_first or 0), _stream()),
        "attention_exact_prefill")


# ---- whole-projection norms, partial rotation, pooled blocks ----------------------------
def qk_norm_rope_store(qkv: torch.Tensor, n_partials: int, q_norm: Optional[torch.Tensor],
                       k_norm: Optional[torch.Tensor], n_q: int, n_k: int, eps: float,
                       freq: torch.Tensor, dims: int, neighbours: bool, mult: float, batch,
                       q_out: torch.Tensor, kv_step: torch.Tensor, k_cache: torch.Tensor,
                       v_cache: torch.Tensor, slot_pos: torch.Tensor, H: int, G: int, hd: int,
                       has_v: bool, capacity: int, write_cache: bool = True, pages=None,
                       bias: Optional[torch.Tensor] = None, head_norm: Optional[tuple] = None) -> None:
    """qkv float32 [(s,) N, (H + G (+ G)) hd] -> q_out [N, H hd], kv_step [N, 2, G, hd] and the cache
    rows: q and k normed over their whole rows (n_q, n_k true features), the first ``dims``
    features of each head rotated (pairs (i, i + dims/2), or (2i, 2i+1) with ``neighbours``), cos
    and sin times ``mult``; values are the v rows or, without them, the keys as projected.
    ``head_norm`` = (eps, size): after the rotation every head of q and k is divided by its own root
    mean square over ``size`` features (no weight; excludes the whole-row norms)."""
    n = q_out.shape[0]
    head_eps, head_size = (float(head_norm[0]), int(head_norm[1])) if head_norm is not None else (-1.0, hd)
    row = (H + (2 if has_v else 1) * G) * hd
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    _need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[-1] == row
          and qkv.shape[-2] == n, "qk_norm_rope_store: qkv float32 [(s,) N, row]")
    for w, size in ((q_norm, H * hd), (k_norm, G * hd)):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == size and w.is_contiguous()),
              "qk_norm_rope_store: norm weights float32 [heads * hd]")
    _need(freq.dtype == torch.float32 and freq.numel() >= max(1, dims // 2) and dims % 2 == 0
          and 0 <= dims <= hd, "qk_norm_rope_store: freq float32 [dims / 2]")
    _need(q_out.dtype == kv_step.dtype == k_cache.dtype == v_cache.dtype and q_out.is_contiguous()
          and kv_step.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "qk_norm_rope_store: outputs of one type, contiguous")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == row and bias.is_contiguous()),
          "qk_norm_rope_store: bias float32 [row]")
    _check(lib().yalm_qk_norm_rope_store(
        _p(qkv), n_partials, n * row, _p(bias), _p(q_norm), _p(k_norm), int(n_q), int(n_k), float(eps), _p(freq),
        int(dims), 1 if neighbours else 0, float(mult), head_eps, head_size, _p(batch.token_seq),
        _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos), _p(q_out), _p(kv_step), _p(k_cache), _p(v_cache),
        dtype_code(q_out.dtype), n, H, G, hd, 1 if has_v else 0, capacity, 1 if write_cache else 0, pt,
        pps, npg, _stream()), "qk_norm_rope_store")


def pool_blocks(kv_step: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, batch,
                slot_pos: torch.Tensor, pool_k: torch.Tensor, pool_v: torch.Tensor, G: int, hd: int,
                capacity: int, pool: int, pool_capacity: int, status: torch.Tensor, pages=None,
                pool_pages=None) -> None:
    """Mean key and mean value of every block of ``pool`` positions that this step completes,
    into row ``block`` of the pooled cache."""
    pt, pps, npg = _pages(pages, k_cache, G, hd)
    ppt, ppps, pnpg = _pages(pool_pages, pool_k, G, hd)
    _need(kv_step.dtype == k_cache.dtype == v_cache.dtype == pool_k.dtype == pool_v.dtype
          and kv_step.is_contiguous() and pool_k.is_contiguous() and pool_v.is_contiguous(),
          "pool_blocks: one type, contiguous")
    _check(lib().yalm_pool_blocks(_p(kv_step), _p(k_cache), _p(v_cache), _p(batch.q_start),
                                  _p(batch.seq_slot), _p(slot_pos), _p(pool_k), _p(pool_v),
                                  dtype_code(kv_step.dtype), batch.n_seqs, max(batch.q_lens), G, hd,
                                  capacity, int(pool), pt, pps, npg, int(pool_capacity), ppt, ppps, pnpg,
                                  _p(status), _stream()), "pool_blocks")


# ---- layers that norm after the residual sum ------------------------------------------------
def sum_norm(x: torch.Tensor, alpha: float, branches, weight: torch.Tensor, eps: float,
             h: Optional[torch.Tensor] = None, branch_eps: float = 0.0) -> None:
    """x <- n(alpha x + sum_b scale_b B_b, weight) in place (float32), and into ``h`` in h's type.
    ``branches``: up to two (slices float32 [S, N, dim], S, norm weight or None, scale); a branch
    with a weight is itself normed over the row (with ``branch_eps``) before it is added."""
    n, dim = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and weight.dtype == torch.float32
          and weight.numel() == dim, "sum_norm: x float32 [N, dim], weight float32 [dim]")
    _need(len(branches) <= 2, "sum_norm: at most two branches")
    _need(h is None or (h.is_contiguous() and tuple(h.shape) == (n, dim)), "sum_norm: h like x")
    args = []
    for buf, S, w, scale in branches:
        _need(buf.dtype == torch.float32 and buf.is_contiguous() and buf.numel() >= S * n * dim,
              "sum_norm: a branch is float32 [S, N, dim]")
        _need(w is None or (w.dtype == torch.float32 and w.numel() == dim), "sum_norm: branch weight")
        args += [_p(buf), int(S), n * dim, _p(w), float(scale)]
    while len(args) < 10:
        args += [None, 0, 0, None, 0.0]
    _check(lib().yalm_sum_norm(_p(x), float(alpha), len(branches), *args, float(branch_eps), _p(weight),
                               float(eps), _p(h), dtype_code(h.dtype) if h is not None else F32, n, dim,
                               _stream()), "sum_norm")


def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
          and out.numel() == x.numel(), "cast_rows: float32 in, same size out")
    _check(lib().yalm_cast_rows(_p(x), _p(out), dtype_code(out.dtype), x.numel(), _stream()), "cast_rows")


def head_norm(o: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, heads: int, size: int,
              eps: float) -> None:
    """out [N, heads * size] = every head's values of o (float32) normed over ``size`` with weight."""
    n = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape[1] == heads * size
          and weight.dtype == torch.float32 and weight.numel() == size and out.is_contiguous()
          and tuple(out.shape) == (n, heads * size), "head_norm: shapes")
    _check(lib().yalm_head_norm(_p(o), _p(weight), _p(out), dtype_code(out.dtype), n, heads, size,
                                float(eps), _stream()), "head_norm")


def gated_recurrence(proj: torch.Tensor, n_partials: int, f_bias: torch.Tensor, lower: torch.Tensor,
                     batch, state: torch.Tensor, out: torch.Tensor, H: int, dk: int, dv: int,
                     act: torch.Tensor) -> None:
    """S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t per head over a step's tokens, from
    the fused projection (q | f | v) as float32 slices [(s,) N, 2 H dk + H dv]; ``state`` float32
    [slots, H, dk, dv] is read at the step's start and written at its end; out float32 [N, H dv];
    ``act``: float32 scratch [N, 2 H dk + H dv] for the activated projection (two launches)."""
    n = out.shape[0]
    row = 2 * H * dk + H * dv
    _need(proj.dtype == torch.float32 and proj.is_contiguous() and proj.shape[-1] == row
          and proj.shape[-2] == n, "gated_recurrence: projection float32 [(s,) N, 2 H dk + H dv]")
    _need(f_bias.dtype == lower.dtype == torch.float32 and f_bias.numel() == lower.numel() == H * dk,
          "gated_recurrence: bias and lower bound float32 [H dk]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv)
          and out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == H * dv,
          "gated_recurrence: state float32 [slots, H, dk, dv], out float32 [N, H dv]")
    _need(act.dtype == torch.float32 and act.is_contiguous() and act.numel() >= n * row,
          "gated_recurrence: act float32 [N, 2 H dk + H dv]")
    _check(lib().yalm_gated_recurrence(_p(proj), n_partials, n * row, _p(f_bias), _p(lower), _p(act),
                                       _p(batch.q_start), _p(batch.seq_slot), _p(state), _p(out), n,
                                       batch.n_seqs, H, dk, dv, _stream()), "gated_recurrence", kernels=2)


# ---- several residual copies per token --------------------------------------------------------
def hc_step(X: torch.Tensor, write=None, read=None) -> None:
    """X float32 [copies, N, dim].  ``write`` = (slices float32 [S, N, dim], S, mix [copies, copies]
    (from, to), out [copies], mult): X_j <- sum_i mix[i, j] X_i + mult out[j] y.  ``read`` =
    (in [copies], norm weight or None, eps, destination): u = sum_i in[i] X_i of the new X, normed
    into the destination (any storage type), or without a norm weight stored as it is (float32)."""
    s, n, dim = X.shape
    _need(X.dtype == torch.float32 and X.is_contiguous() and 1 <= s <= 8, "hc_step: X float32 [1..8, N, dim]")
    y = mix = out_w = in_w = norm_w = dst = None
    S, mult, eps = 0, 0.0, 0.0
    if write is not None:
        y, S, mix, out_w, mult = write
        _need(y.dtype == torch.float32 and y.is_contiguous() and y.numel() >= S * n * dim
              and mix.dtype == out_w.dtype == torch.float32 and mix.numel() == s * s and out_w.numel() == s
              and mix.is_contiguous(), "hc_step: slices float32 [S, N, dim], mix [s, s], out [s]")
    if read is not None:
        in_w, norm_w, eps, dst = read
        _need(in_w.dtype == torch.float32 and in_w.numel() == s and dst.is_contiguous()
              and dst.numel() == n * dim, "hc_step: in [s], destination [N, dim]")
        _need(norm_w is not None or dst.dtype == torch.float32, "hc_step: an unnormed read is float32")
        _need(norm_w is None or (norm_w.dtype == torch.float32 and norm_w.numel() == dim), "hc_step: norm weight")
    normed = norm_w is not None
    _check(lib().yalm_hc_step(_p(X), s, n, dim, _p(y), int(S), n * dim, _p(mix), _p(out_w), float(mult),
                              _p(in_w), _p(norm_w), float(eps), _p(dst) if normed else None,
                              dtype_code(dst.dtype) if normed else F32,
                              None if (normed or dst is None) else _p(dst), _stream()), "hc_step")


# ---- a recurrence with a decay per channel and a bonus for the current token ---------------------
def token_shift(h: torch.Tensor, prev: torch.Tensor, mu: torch.Tensor, out: torch.Tensor, batch) -> None:
    """out [n_mix, N, dim] = h + (h' - h) mu[s], h' the previous token's row of h; for a step's first
    token the sequence's row of ``prev`` float32 [slots, dim]."""
    n, dim = h.shape
    n_mix = mu.shape[0]
    _need(h.is_contiguous() and out.dtype == h.dtype and out.is_contiguous() and out.numel() == n_mix * n * dim
          and mu.dtype == prev.dtype == torch.float32 and mu.is_contiguous() and mu.shape[1] == dim
          and prev.is_contiguous() and prev.shape[1] == dim, "token_shift: shapes")
    _check(lib().yalm_token_shift(_p(h), _p(prev), _p(mu), _p(out), dtype_code(h.dtype), _p(batch.token_seq),
                                  _p(batch.q_start), _p(batch.seq_slot), n, dim, n_mix, _stream()),
           "token_shift")


def wkv(r, k, v, g, z, w0: torch.Tensor, bonus: torch.Tensor, act: torch.Tensor, gate: torch.Tensor,
        h: torch.Tensor, prev: torch.Tensor, batch, state: torch.Tensor, out: torch.Tensor, H: int, dk: int,
        dv: int) -> None:
    """o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, S_t = diag(w_t) S_(t-1) + k_t v_t^T per head over a
    step's tokens.  r, k, z: (float32 slices [S, N, H dk], S); v, g: (slices [S, N, H dv], S);
    w = exp(-exp(z + w0)); ``gate`` receives silu(g); ``state`` float32 [slots, H, dk, dv]; ``prev``
    float32 [slots, dim] receives every sequence's last row of ``h``; out float32 [N, H dv]."""
    n = out.shape[0]
    row = 3 * H * dk + H * dv
    args = []
    for (buf, S), width in ((r, H * dk), (k, H * dk), (v, H * dv), (g, H * dv), (z, H * dk)):
        _need(buf.dtype == torch.float32 and buf.is_contiguous() and buf.shape[-1] == width
              and buf.shape[-2] == n, "wkv: projections as float32 slices [(s,) N, width]")
        args += [_p(buf), int(S), n * width]
    _need(w0.dtype == bonus.dtype == torch.float32 and w0.numel() == bonus.numel() == H * dk
          and act.dtype == gate.dtype == torch.float32 and act.numel() >= n * row and gate.numel() >= n * H * dv
          and state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv)
          and out.dtype == torch.float32 and out.is_contiguous() and out.shape[1] == H * dv
          and prev.dtype == torch.float32 and prev.is_contiguous() and prev.shape[1] == h.shape[1]
          and h.is_contiguous() and h.shape[0] == n, "wkv: shapes")
    _check(lib().yalm_wkv(*args, _p(w0), _p(bonus), _p(act), _p(gate), _p(h), dtype_code(h.dtype), _p(prev),
                          _p(batch.token_seq), _p(batch.q_start), _p(batch.seq_slot), _p(state), _p(out), n,
                          batch.n_seqs, H, dk, dv, h.shape[1], _stream()), "wkv", kernels=2)


def wkv_out(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, heads: int,
            size: int, eps: float) -> None:
    """out [N, heads * size] = every head of o (float32) over its root mean square, times weight
    [heads * size], times gate (float32 [N, heads * size])."""
    n = o.shape[0]
    _need(o.dtype == gate.dtype == weight.dtype == torch.float32 and o.is_contiguous() and gate.is_contiguous()
          and o.shape[1] == heads * size and weight.numel() == heads * size and gate.numel() >= n * heads * size
          and out.is_contiguous() and tuple(out.shape) == (n, heads * size), "wkv_out: shapes")
    _check(lib().yalm_wkv_out(_p(o), _p(weight), _p(gate), _p(out), dtype_code(out.dtype), n, heads, size,
                              float(eps), _stream()), "wkv_out")


# ---- attention over a cached latent ----------------------------------------------------------------
def latent_store(dkv: torch.Tensor, n_partials: int, c_norm: torch.Tensor, eps: float, freq: torch.Tensor,
                 batch, slot_pos: torch.Tensor, kv_step: torch.Tensor, cache: torch.Tensor, rank: int,
                 rd: int, hd: int, capacity: int, write_cache: bool = True, pages=None) -> None:
    """dkv float32 [(s,) N, rank + rd] -> the row [norm(c) w | rot(kr) | 0] of every token, to
    kv_step [N, 2, 1, hd] (key and value alike) and to the cache."""
    n = kv_step.shape[0]
    pt, pps, npg = _pages(pages, cache, 1, hd)
    _need(dkv.dtype == torch.float32 and dkv.is_contiguous() and dkv.shape[-1] == rank + rd
          and dkv.shape[-2] == n and c_norm.dtype == freq.dtype == torch.float32 and c_norm.numel() == rank
          and freq.numel() >= max(1, rd // 2) and kv_step.dtype == cache.dtype and kv_step.is_contiguous()
          and kv_step.numel() == n * 2 * hd and cache.is_contiguous(), "latent_store: shapes")
    _check(lib().yalm_latent_store(_p(dkv), n_partials, n * (rank + rd), _p(c_norm), float(eps), _p(freq),
                                   _p(batch.token_seq), _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos),
                                   _p(kv_step), _p(cache), dtype_code(cache.dtype), n, rank, rd, hd, capacity,
                                   1 if write_cache else 0, pt, pps, npg, _stream()), "latent_store")


def latent_absorb_q(q: torch.Tensor, n_partials: int, w_uk: torch.Tensor, freq: torch.Tensor, batch,
                    slot_pos: torch.Tensor, q_out: torch.Tensor, H: int, dim: int, rd: int, rank: int,
                    hd: int) -> None:
    """q float32 [(s,) N, H (dim + rd)], w_uk [H, dim, rank] -> q_out [N, H, hd] =
    [Wuk_h^T q_h[:dim] | rot(q_h[dim:]) | 0]."""
    n = q_out.shape[0]
    _need(q.dtype == torch.float32 and q.is_contiguous() and q.shape[-1] == H * (dim + rd) and q.shape[-2] == n
          and w_uk.dtype == q_out.dtype and w_uk.is_contiguous() and w_uk.numel() == H * dim * rank
          and q_out.is_contiguous() and q_out.numel() == n * H * hd and freq.dtype == torch.float32,
          "latent_absorb_q: shapes")
    _check(lib().yalm_latent_absorb_q(_p(q), n_partials, n * H * (dim + rd), _p(w_uk), _p(freq),
                                      _p(batch.token_seq), _p(batch.q_start), _p(batch.seq_slot), _p(slot_pos),
                                      _p(q_out), dtype_code(q_out.dtype), n, H, dim, rd, rank, hd, _stream()),
           "latent_absorb_q")


def latent_expand(o: torch.Tensor, w_uv: torch.Tensor, gate: Optional[torch.Tensor], n_partials: int,
                  out: torch.Tensor, H: int, rank: int, vdim: int, hd: int) -> None:
    """o [N, H, hd], w_uv [H, rank, vdim] -> out [N, H vdim] = (Wuv_h o_h[:rank]) sigmoid(gate)."""
    n = out.shape[0]
    _need(o.dtype == w_uv.dtype == out.dtype and o.is_contiguous() and o.numel() == n * H * hd
          and w_uv.is_contiguous() and w_uv.numel() == H * rank * vdim and out.is_contiguous()
          and out.shape[1] == H * vdim, "latent_expand: shapes")
    _need(gate is None or (gate.dtype == torch.float32 and gate.is_contiguous()
                           and gate.numel() >= n_partials * n * H * vdim), "latent_expand: gate slices")
    _check(lib().yalm_latent_expand(_p(o), _p(w_uv), _p(gate), n_partials, n * H * vdim, _p(out),
                                    dtype_code(out.dtype), n, H, rank, vdim, hd, _stream()), "latent_expand")


GELU_TANH, TANH = 1, 2


def activation_rows(z: torch.Tensor, n_partials: int, out: torch.Tensor, act: int) -> None:
    """out = act(sum of the slices of z float32 [(s,) ...]) in out's type; act GELU_TANH or TANH."""
    n = out.numel()
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.numel() >= n_partials * n and out.is_contiguous(),
          "activation_rows: float32 slices in, contiguous out")
    _check(lib().yalm_activation_rows(_p(z), n_partials, n, _p(out), dtype_code(out.dtype), n, int(act),
                                      _stream()), "activation_rows")


# ---- sublayer outputs normed before they join the residual stream -------------------------------------
NORM_ABSENT, NORM_TANH, NORM_RMS, NORM_NONE = 0, 1, 2, 3


def norm_step(x: torch.Tensor, sets=(), post: Optional[tuple] = None, pre: Optional[tuple] = None,
              h: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
              n_rows: Optional[int] = None) -> None:
    """One pass over the rows of x float32 [N, dim]: x <- x + post(y), then h = pre(x).  y is the sum
    over ``sets`` (up to two (slices float32 [S, N, dim], S, factor)) of factor * sum of slices.  ``post``
    and ``pre`` are (kind, weight, bias, alpha, eps) with kind NORM_TANH (tanh(alpha v) w + b),
    NORM_RMS (v / sqrt(mean v^2 + eps) w) or NORM_NONE, or None for a step without that half.  With
    ``rows`` (int32 row numbers; no post half) only those rows are read: h [n_rows, dim]."""
    n, dim = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "norm_step: x float32 [N, dim]")
    _need(len(sets) <= 2 and (post is None) == (len(sets) == 0), "norm_step: a post step has one or two sets")
    args = []
    for buf, S, factor in sets:
        _need(buf.dtype == torch.float32 and buf.is_contiguous() and buf.numel() >= S * n * dim,
              "norm_step: a set is float32 [S, N, dim]")
        args += [_p(buf), int(S), n * dim, float(factor)]
    while len(args) < 8:
        args += [None, 0, 0, 0.0]
    forms = []
    for f in (post, pre):
        if f is None:
            forms += [NORM_ABSENT, None, None, 0.0, 0.0]
            continue
        kind, w, b, alpha, eps = f
        _need(kind == NORM_NONE or (w is not None and w.dtype == torch.float32 and w.numel() == dim),
              "norm_step: weight float32 [dim]")
        _need(kind != NORM_TANH or (b is not None and b.dtype == torch.float32 and b.numel() == dim),
              "norm_step: bias float32 [dim]")
        forms += [int(kind), _p(w), _p(b), float(alpha), float(eps)]
    count = n if rows is None else int(n_rows)
    _need(pre is None or (h is not None and h.is_contiguous() and h.numel() >= count * dim), "norm_step: h")
    _need(rows is None or (rows.dtype == torch.int32 and post is None), "norm_step: rows int32, no post half")
    _check(lib().yalm_norm_step(_p(x), *args, *forms, _p(h), dtype_code(h.dtype) if h is not None else F32,
                                _p(rows), count, dim, _stream()), "norm_step")


def short_conv(src: torch.Tensor, n_partials: int, col0: int, channels: int, weight: torch.Tensor,
               state: torch.Tensor, batch, out32: Optional[torch.Tensor] = None, out_col0: int = 0,
               out16: Optional[torch.Tensor] = None, block16: Optional[int] = None,
               in_bias: Optional[torch.Tensor] = None, out_bias: Optional[torch.Tensor] = None,
               silu: bool = False) -> None:
    """A causal convolution over time on ``channels`` columns (from ``col0``) of src, float32 slices
    [(s,) N, row]: y_t = sum_j weight[c, j] u_(t - taps + 1 + j) (+ out_bias, then SiLU), u = the summed
    slices (+ in_bias); the inputs before a step's first token come from ``state`` float32
    [slots, taps - 1, channels], which leaves with the step's last ones.  out32: float32 [N, row'] at
    column out_col0; out16: [channels / block16, N, block16] in its own type (block16 None: [N, channels])."""
    n = batch.n_tokens
    row = src.shape[-1]
    taps = weight.shape[1]
    _need(src.dtype == torch.float32 and src.is_contiguous() and src.shape[-2] == n and col0 + channels <= row,
          "short_conv: float32 slices [(s,) N, row]")
    _need(weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == channels
          and state.dtype == torch.float32 and state.is_contiguous()
          and tuple(state.shape[1:]) == (taps - 1, channels), "short_conv: weight [channels, taps], state")
    for b in (in_bias, out_bias):
        _need(b is None or (b.dtype == torch.float32 and b.numel() == channels and b.is_contiguous()),
              "short_conv: bias float32 [channels]")
    _need(out32 is None or (out32.dtype == torch.float32 and out32.is_contiguous() and out32.shape[0] == n
                            and out_col0 + channels <= out32.shape[1]), "short_conv: out32 float32 [N, row']")
    _need(out16 is None or (out16.is_contiguous() and out16.numel() == n * channels), "short_conv: out16")
    _need(out32 is not None or out16 is not None, "short_conv: no output")
    update = not batch.is_decode
    _check(lib().yalm_short_conv(_p(src), int(n_partials), n * row, row, int(col0), _p(in_bias), _p(weight),
                                 _p(out_bias), taps, channels, 1 if silu else 0, _p(state), _p(batch.token_seq),
                                 _p(batch.q_start), _p(batch.seq_slot), _p(out32),
                                 out32.shape[1] if out32 is not None else 0, int(out_col0), _p(out16),
                                 dtype_code(out16.dtype) if out16 is not None else F32,
                                 int(block16 or channels), n, batch.n_seqs, 1 if update else 0, _stream()),
           "short_conv", kernels=2 if update else 1)


def gated_rows(z: torch.Tensor, n_partials: int, tokens: torch.Tensor, table: torch.Tensor, first: int,
               out: torch.Tensor) -> None:
    """out [N, dim] = gelu(sum of the slices of z float32 [(s,) N, dim]) * table[token, first : first + dim]
    (gelu in its tanh form)."""
    n, dim = out.shape
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.shape[-1] == dim and z.shape[-2] == n
          and table.is_contiguous() and table.dim() == 2 and out.is_contiguous() and tokens.dtype == torch.int32,
          "gated_rows: shapes")
    _check(lib().yalm_gated_rows(_p(z), int(n_partials), n * dim, _p(tokens), _p(table), dtype_code(table.dtype),
                                 table.shape[1], int(first), _p(out), dtype_code(out.dtype), n, dim, _stream()),
           "gated_rows")


# ---- the gated delta rule ----------------------------------------------------------------------------
def delta_row(H: int, G: int, dk: int, dv: int) -> int:
    """Floats in a token's activated row [q | k | v | beta (padded to 4) | decay]."""
    return 2 * G * dk + H * dv + ((H + 3) & ~3) + H * dk


def delta_prep(act: torch.Tensor, proj: torch.Tensor, n_partials: int, col_b: int, col_low: int, n_low: int,
               low: torch.Tensor, H: int, G: int, dk: int, dv: int) -> None:
    """act float32 [N, delta_row] holds q | k | v (after convolution and SiLU) in its first columns: q and
    k become unit vectors per head (q also times dk^-1/2), beta = sigmoid of the H columns of ``proj``
    (float32 slices [(s,) N, row]) from col_b, and the n_low columns from col_low go to ``low`` [N, n_low]
    in low's type."""
    n = act.shape[0]
    _need(act.dtype == torch.float32 and act.is_contiguous() and act.shape[1] == delta_row(H, G, dk, dv)
          and proj.dtype == torch.float32 and proj.is_contiguous() and proj.shape[-2] == n
          and low.is_contiguous() and tuple(low.shape) == (n, n_low), "delta_prep: shapes")
    row = proj.shape[-1]
    _check(lib().yalm_delta_prep(_p(act), _p(proj), int(n_partials), n * row, row, int(col_b), int(col_low),
                                 int(n_low), _p(low), dtype_code(low.dtype), n, H, G, dk, dv, _stream()),
           "delta_prep")


def delta_scan(act: torch.Tensor, z: torch.Tensor, n_partials: int, dt_bias: torch.Tensor, a_log: torch.Tensor,
               gate: torch.Tensor, batch, state: torch.Tensor, out: torch.Tensor, H: int, G: int, dk: int,
               dv: int) -> None:
    """The decay exp(-exp(a_log[h]) softplus(z + dt_bias)) (z: float32 slices [(s,) N, H dk + H dv], decay
    logits then gate logits; ``gate`` float32 [N, H dv] receives the gate's sigmoid), then per head
    S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over the step's tokens.  ``state`` float32
    [slots, H, dk, dv]; out float32 [N, H dv]."""
    n = act.shape[0]
    _need(act.dtype == torch.float32 and act.is_contiguous() and act.shape[1] == delta_row(H, G, dk, dv)
          and z.dtype == torch.float32 and z.is_contiguous() and z.shape[-1] == H * dk + H * dv and z.shape[-2] == n
          and dt_bias.dtype == a_log.dtype == torch.float32 and dt_bias.numel() == H * dk and a_log.numel() == H
          and gate.dtype == torch.float32 and gate.numel() >= n * H * dv
          and state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv)
          and out.dtype == torch.float32 and out.is_contiguous() and tuple(out.shape) == (n, H * dv),
          "delta_scan: shapes")
    _check(lib().yalm_delta_scan(_p(act), _p(z), int(n_partials), n * (H * dk + H * dv), _p(dt_bias), _p(a_log),
                                 _p(gate), _p(batch.q_start), _p(batch.seq_slot), _p(state), _p(out), n,
                                 batch.n_seqs, H, G, dk, dv, _stream()), "delta_scan", kernels=2)


# ---- a real-gated linear recurrent unit ----------------------------------------------------------------
def rglru(gates: torch.Tensor, ra_bias: torch.Tensor, ri_bias: torch.Tensor, lam: torch.Tensor, u: torch.Tensor,
          yx: torch.Tensor, n_partials: int, y_bias: Optional[torch.Tensor], coef: torch.Tensor, batch,
          state: torch.Tensor, out: torch.Tensor, width: int, bw: int, c_decay: float) -> None:
    """a = exp(-c r softplus(lam)), S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t, out_t = S_t gelu(y_t + bias)
    per channel over the step's tokens.  gates float32 [width / bw, N, 2 bw] (r logits, then i logits, of
    every block of channels); u float32 [N, width]; yx float32 slices [(s,) N, row] with the y logits in
    the first ``width`` columns; ``state`` float32 [slots, width]; out [N, width]."""
    n = u.shape[0]
    _need(gates.dtype == torch.float32 and gates.is_contiguous() and gates.numel() == 2 * n * width
          and u.dtype == torch.float32 and u.is_contiguous() and u.shape[1] == width
          and yx.dtype == torch.float32 and yx.is_contiguous() and yx.shape[-2] == n and yx.shape[-1] >= width
          and coef.dtype == torch.float32 and coef.numel() >= 3 * n * width
          and state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == width
          and out.is_contiguous() and tuple(out.shape) == (n, width), "rglru: shapes")
    for v in (ra_bias, ri_bias, lam):
        _need(v.dtype == torch.float32 and v.numel() == width and v.is_contiguous(), "rglru: float32 [width]")
    row = yx.shape[-1]
    _check(lib().yalm_rglru(_p(gates), _p(ra_bias), _p(ri_bias), _p(lam), _p(u), _p(yx), int(n_partials), n * row,
                            row, _p(y_bias), _p(coef), _p(batch.q_start), _p(batch.seq_slot), _p(state), _p(out),
                            dtype_code(out.dtype), n, batch.n_seqs, width, bw, float(c_decay), _stream()),
           "rglru", kernels=2)


# ---- a routed feed-forward --------------------------------------------------------------
ROUTED_TILE = 64          # rows per tile of the grouped FMA product


def route_topk(z: torch.Tensor, n_partials: int, n_tokens: int, E: int, n_groups: int, keep: int,
               top: int, renormalise: bool, choice: torch.Tensor, weight: torch.Tensor,
               counts: torch.Tensor, sigmoid: bool = False, correction: Optional[torch.Tensor] = None,
               group_top2: bool = False, norm_eps: float = 0.0, weight_scale: float = 1.0) -> None:
    """Router logits z (float32 slices [n_partials, n_tokens, E]) -> the ``top`` experts of each
    token among the ``keep`` best of ``n_groups`` groups and their scores.  Scores are the softmax
    over all experts, or with ``sigmoid`` each logit's own sigmoid; ``correction`` float32 [E] is added
    to the scores for the choice of groups and experts only; a group's score is its best choice
    score, or with ``group_top2`` the sum of its two best; the weights are the chosen scores, with
    ``renormalise`` divided by (their sum + ``norm_eps``), times ``weight_scale``."""
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.numel() >= n_partials * n_tokens * E,
          "route_topk: logits")
    _need(choice.dtype == torch.int32 and weight.dtype == torch.float32 and counts.dtype == torch.int32
          and choice.numel() >= n_tokens * top and weight.numel() >= n_tokens * top
          and counts.numel() >= E, "route_topk: outputs")
    _need(correction is None or (correction.dtype == torch.float32 and correction.numel() == E
                                 and correction.is_contiguous()), "route_topk: correction float32 [E]")
    _check(lib().yalm_route_topk(_p(z), n_partials, n_tokens * E, n_tokens, E, n_groups, keep, top,
                                 1 if renormalise else 0, 1 if sigmoid else 0, 1 if group_top2 else 0,
                                 float(norm_eps), float(weight_scale), _p(correction), _p(choice), _p(weight),
                                 _p(counts), _stream()), "route_topk")


def routed_max_tiles(n_pairs: int, E: int, tile_rows: int = ROUTED_TILE) -> int:
    """The most tiles a plan can have: every expert may end with a tile that is not full."""
    return min(n_pairs, -(-n_pairs // tile_rows) + E)


def route_plan(counts, choice, n_pairs: int, top: int, E: int, first_row, pair_row, row_token,
               tile_expert, tile_row0, n_tiles, tile_rows: int = ROUTED_TILE) -> None:
    for t in (counts, choice, first_row, pair_row, row_token, tile_expert, tile_row0, n_tiles):
        _need(t.dtype == torch.int32 and t.is_contiguous(), "route_plan: int32 tensors")
    _need(first_row.numel() >= E + 1 and pair_row.numel() >= n_pairs and row_token.numel() >= n_pairs
          and tile_expert.numel() >= routed_max_tiles(n_pairs, E, tile_rows)
          and tile_row0.numel() >= routed_max_tiles(n_pairs, E, tile_rows), "route_plan: sizes")
    _check(lib().yalm_route_plan(_p(counts), _p(choice), n_pairs, top, E, tile_rows, _p(first_row),
                                 _p(pair_row), _p(row_token), _p(tile_expert), _p(tile_row0),
                                 _p(n_tiles), _stream()), "route_plan")


def gather_rows(src: torch.Tensor, row_token: torch.Tensor, dst: torch.Tensor) -> None:
    rows, dim = dst.shape
    _need(src.dtype == dst.dtype and src.shape[1] == dim and src.is_contiguous() and dst.is_contiguous()
          and row_token.dtype == torch.int32 and row_token.numel() >= rows, "gather_rows: shapes")
    _check(lib().yalm_gather_rows(_p(src), _p(row_token), _p(dst), dtype_code(dst.dtype), rows, dim,
                                  _stream()), "gather_rows")


def gemm_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, first_row, tile_expert,
                 tile_row0, n_tiles, max_tiles: int) -> None:
    """out[r] = a[r] @ w[e].T for the rows of every expert e (a in sorted order, w [E, N, K]),
    with 32-bit FMA; the plan's tiles must be ROUTED_TILE rows."""
    rows, K = a.shape
    E, N, _ = w.shape
    _need(w.shape[2] == K and tuple(out.shape) == (rows, N) and a.is_contiguous() and w.is_contiguous()
          and out.is_contiguous(), "gemm_grouped: shapes")
    _check(lib().yalm_gemm_grouped(_p(a), dtype_code(a.dtype), _p(w), dtype_code(w.dtype), _p(out),
                                   dtype_code(out.dtype), _p(first_row), _p(tile_expert),
                                   _p(tile_row0), _p(n_tiles), max_tiles, N, K, _stream()),
           "gemm_grouped")


def routed_tile_rows(n_pairs: int, E: int) -> int:
    """Rows per tile of the tensor-core grouped product for a step's (token, choice) pairs: the
    smallest of 16, 32, 64 that holds an expert's share if the pairs spread evenly, else 128
    (the kernel also takes 256, which was measured and is no faster)."""
    share = -(-n_pairs // E)
    for bt in (16, 32, 64):
        if share <= bt:
            return bt
    return 128


def gemm_grouped_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, first_row, tile_expert,
                    tile_row0, n_tiles, max_tiles: int, tile_rows: int, status: torch.Tensor,
                    glu: Optional[tuple] = None) -> None:
    """The grouped product on tcgen05: out[r] = a[r] @ w[e].T over a plan of ``tile_rows``-row
    tiles; with ``glu`` = (slope, limit, shift) and w = [gate; up] per expert, out [rows, N / 2] is
    the gated activation g' sigmoid(slope g') (u' + shift) under the clamps of ``glu_clamp``."""
    rows, K = a.shape
    E, N, _ = w.shape
    _need(a.dtype == w.dtype and a.dtype in HALF_TYPES and w.shape[2] == K and a.is_contiguous()
          and w.is_contiguous() and out.is_contiguous(), "gemm_grouped_tc: operands")
    _need(tuple(out.shape) == (rows, N // 2 if glu else N), "gemm_grouped_tc: out shape")
    slope, limit, shift = glu if glu else (1.0, 0.0, 0.0)
    _check(lib().yalm_gemm_grouped_tc(_p(a), _p(w), dtype_code(a.dtype), _p(out), dtype_code(out.dtype),
                                      rows, E, N, K, 2 if glu else 0, tile_rows, _p(first_row),
                                      _p(tile_expert), _p(tile_row0), _p(n_tiles), max_tiles,
                                      float(slope), float(limit), float(shift), _p(status), _stream()),
           "gemm_grouped_tc")


def glu_clamp(gu: torch.Tensor, out: torch.Tensor, n_partials: int, alpha: float, limit: float,
              shift: float, paired: bool = False) -> None:
    """out = g' * sigmoid(alpha g') * (u' + shift), g' = min(g, limit), u' = clamp(u, +-limit)
    (no clamps when limit <= 0); gu float32 [(n_partials,) rows, 2F] as (gate | up) or, with
    ``paired``, 16 gate columns then the 16 up columns of the same features, and so on."""
    rows, F = out.shape
    _need(gu.dtype == torch.float32 and gu.shape[-1] == 2 * F and gu.shape[-2] == rows
          and gu.is_contiguous() and out.is_contiguous(), "glu_clamp: shapes")
    _check(lib().yalm_glu_clamp(_p(gu), n_partials, rows * 2 * F, _p(out), dtype_code(out.dtype), rows, F,
                                float(alpha), float(limit), float(shift), 1 if paired else 0, _stream()),
           "glu_clamp")


def routed_combine(x: torch.Tensor, y: torch.Tensor, pair_row: torch.Tensor, weight: torch.Tensor,
                   top: int) -> None:
    """x[t] += sum_j weight[t, j] * y[pair_row[t, j]]."""
    n, dim = x.shape
    _need(x.dtype == y.dtype == weight.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous()
          and y.shape[1] == dim and pair_row.dtype == torch.int32, "routed_combine: shapes")
    _check(lib().yalm_routed_combine(_p(x), _p(y), _p(pair_row), _p(weight), n, top, dim, _stream()),
           "routed_combine")


def sample(logits: torch.Tensor, temperature: float, seed: int, row_key: torch.Tensor,
           seq_slot: torch.Tensor, slot_pos: torch.Tensor, out_tokens: torch.Tensor,
           params: Optional[torch.Tensor] = None) -> None:
    """``params``: int64 [2] on the device holding (seed, temperature bits), which then
    replace the two arguments (see ``sampling_params``)."""
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and out_tokens.dtype == torch.int32
          and row_key.dtype == torch.int32, "sample: types")
    _need(params is None or (params.dtype == torch.int64 and params.numel() >= 2),
          "sample: params is int64 [2]")
    _check(lib().yalm_sample(_p(logits), rows, vocab, float(temperature), int(seed) & (2 ** 64 - 1),
                             _p(params), _p(row_key), _p(seq_slot), _p(slot_pos), _p(out_tokens),
                             _stream()), "sample")


def sampling_params(temperature: float, seed: int):
    """The two 64-bit words ``sample`` reads from ``params`` (as signed Python ints)."""
    import struct
    if temperature < 0:
        raise KernelError("sample: the temperature must not be negative")
    s = int(seed) & (2 ** 64 - 1)
    s = s - 2 ** 64 if s >= 2 ** 63 else s
    return s, struct.unpack("<I", struct.pack("<f", float(temperature)))[0]


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch on (default) or off for all later launches."""
    l = lib()
    l.yalm_set_pdl.argtypes = [_i]
    l.yalm_set_pdl.restype = _c.c_int
    l.yalm_set_pdl(1 if on else 0)


def uniform01(seed: int, key: int, counter: int) -> float:
    return float(lib().yalm_uniform01(int(seed) & (2 ** 64 - 1), int(key) & 0xffffffff,
                                      int(counter) & 0xffffffff))
