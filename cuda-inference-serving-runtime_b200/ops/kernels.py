"""Python face of the CUDA kernels: one function per kernel entry point.

Every function checks shapes, types and contiguity, passes raw device pointers and
the current CUDA stream to the C entry point, and raises `KernelError` on a
non-zero status.  Nothing here falls back to a library or to the CPU: without a
CUDA device or without the compiled kernels these functions fail.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import load_library

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
GEMM_WORKSPACE_BYTES = 64 << 20


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"storage type {dtype} is not supported (float32 and bfloat16 only)") from None


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle.  Every launch asks for it, so it takes the short way where torch has one (a tenth of
    the time of building a Stream object, which showed in steps that launch hundreds of kernels from the host)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_pdl_state = {"on": False}
LAUNCHES = {"own": 0, "library": 0}   # kernels launched so far: this package's own, and vendor-library products


def _check(status: int, what: str, own: int = 1, library: int = 0) -> None:
    LAUNCHES["own"] += own
    LAUNCHES["library"] += library
    if status != 0:
        detail = {-2: "invalid argument", -3: "shared memory need exceeds the device limit"}.get(status, "")
        raise KernelError(f"{what} failed with status {status} {detail}".rstrip())


def _need(t: torch.Tensor, dtype, name: str, dims: Optional[int] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on the CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name} must have {dims} dimensions, got shape {tuple(t.shape)}")


# ------------------------------------------------------------------ elementwise library
def _elementwise():
    lib = load_library("elementwise.cu")
    if not getattr(lib, "_typed", False):
        lib.cisr_embedding.restype = ctypes.c_int
        lib.cisr_add_rmsnorm.restype = ctypes.c_int
        lib.cisr_swiglu.restype = ctypes.c_int
        lib.cisr_rotary_tables.restype = ctypes.c_int
        lib.cisr_rope_store.restype = ctypes.c_int
        lib.cisr_page_copy.restype = ctypes.c_int
        lib.cisr_table_update.restype = ctypes.c_int
        lib._typed = True
    return lib


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] widened to float."""
    _need(table, None, "table", 2); _need(ids, torch.int32, "ids", 1); _need(out, torch.float32, "out", 2)
    tokens, hidden = out.shape
    if ids.numel() != tokens or table.shape[1] != hidden:
        raise KernelError("embedding: shapes of ids, table and out disagree")
    _check(_elementwise().cisr_embedding(_p(table), dtype_code(table.dtype), _p(ids), _p(out), tokens, hidden,
                                         table.shape[0], _stream()), "embedding")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, write_back: bool = True) -> torch.Tensor:
    """x += delta (when given), out = rmsnorm(x) * weight; `rows` selects which rows of x become rows of out."""
    _need(x, torch.float32, "x", 2); _need(weight, None, "weight", 1); _need(out, None, "out", 2)
    hidden = x.shape[1]
    if delta is not None:
        _need(delta, torch.float32, "delta", 2)
        if delta.shape != x.shape:
            raise KernelError("add_rmsnorm: delta and x differ in shape")
    n_rows = out.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows", 1)
        if rows.numel() != n_rows:
            raise KernelError("add_rmsnorm: one row index per output row is needed")
    elif n_rows != x.shape[0]:
        raise KernelError("add_rmsnorm: out and x differ in rows")
    if weight.numel() != hidden or out.shape[1] != hidden:
        raise KernelError("add_rmsnorm: width mismatch")
    _check(_elementwise().cisr_add_rmsnorm(_p(x), _p(delta), _p(weight), dtype_code(weight.dtype), _p(out),
                                           dtype_code(out.dtype), _p(rows), n_rows, hidden, ctypes.c_float(eps),
                                           int(write_back), _stream()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _need(gate_up, torch.float32, "gate_up", 2); _need(out, None, "out", 2)
    tokens, inter = out.shape
    if gate_up.shape != (tokens, 2 * inter):
        raise KernelError("swiglu: gate_up must be [tokens, 2 * intermediate]")
    _check(_elementwise().cisr_swiglu(_p(gate_up), _p(out), dtype_code(out.dtype), tokens, inter, _stream()), "swiglu")
    return out


def rotary_tables(positions: torch.Tensor, inv_freq: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    _need(positions, torch.int32, "positions", 1); _need(inv_freq, torch.float64, "inv_freq", 1)
    _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
    tokens, half = cos.shape
    if positions.numel() != tokens or inv_freq.numel() != half or sin.shape != cos.shape:
        raise KernelError("rotary_tables: shapes disagree")
    _check(_elementwise().cisr_rotary_tables(_p(positions), _p(inv_freq), _p(cos), _p(sin), tokens, half, _stream()),
           "rotary_tables")


def rope_store(proj: torch.Tensor, k_col: int, v_col: int, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               rot_half: int, interleaved: bool, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], token_req: torch.Tensor, positions: torch.Tensor,
               req_slot: torch.Tensor, block_table: torch.Tensor, page_size: int, hq: int, hkv: int, dim: int) -> None:
    """Rotate q (and k), write q to q_out and k, v into their cache pages (k_col < 0: queries only)."""
    _need(proj, torch.float32, "proj", 2); _need(q_out, None, "q_out")
    tokens = proj.shape[0]
    if rot_half:
        _need(cos, torch.float32, "cos", 2); _need(sin, torch.float32, "sin", 2)
        if cos.shape != (tokens, rot_half) or sin.shape != cos.shape:
            raise KernelError("rope_store: rotary tables must be [tokens, rot_half]")
    if q_out.numel() != tokens * hq * dim:
        raise KernelError("rope_store: q_out must hold [tokens, heads, head_dim]")
    cache_code = F32
    if k_col >= 0:
        _need(k_cache, None, "k_cache", 4); _need(v_cache, k_cache.dtype, "v_cache", 4)
        if tuple(k_cache.shape[1:]) != (hkv, page_size, dim) or v_cache.shape != k_cache.shape:
            raise KernelError("rope_store: cache must be [pages, kv_heads, page_size, head_dim]")
        if proj.shape[1] < v_col + hkv * dim or proj.shape[1] < k_col + hkv * dim:
            raise KernelError("rope_store: projection row is too short for its key and value columns")
        cache_code = dtype_code(k_cache.dtype)
    _need(token_req, torch.int32, "token_req", 1); _need(positions, torch.int32, "positions", 1)
    _need(block_table, torch.int32, "block_table", 2); _need(req_slot, torch.int32, "req_slot", 1)
    _check(_elementwise().cisr_rope_store(
        _p(proj), proj.shape[1], k_col, v_col, _p(cos if rot_half else None), _p(sin if rot_half else None), rot_half,
        int(interleaved), _p(q_out), dtype_code(q_out.dtype), _p(k_cache), _p(v_cache), cache_code, _p(token_req),
        _p(positions), _p(req_slot), _p(block_table), block_table.shape[1], page_size, hq, hkv, dim, tokens, _stream()),
        "rope_store")


def page_copy(pool: torch.Tensor, pairs: torch.Tensor, n_planes: int, plane_bytes: int, page_bytes: int) -> None:
    """Copy pages (src, dst) in every plane of a pool laid out [planes, pages, page bytes]."""
    _need(pairs, torch.int32, "pairs", 2)
    _check(_elementwise().cisr_page_copy(_p(pool), _p(pairs), pairs.shape[0], n_planes, ctypes.c_longlong(plane_bytes),
                                         ctypes.c_longlong(page_bytes), _stream()), "page_copy")


def table_update(table: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """table.view(-1)[idx[i]] = val[i] for every i with idx[i] >= 0."""
    _need(table, torch.int32, "table"); _need(idx, torch.int32, "idx", 1); _need(val, torch.int32, "val", 1)
    _check(_elementwise().cisr_table_update(_p(table), _p(idx), _p(val), idx.numel(), _stream()), "table_update")


# ------------------------------------------------------------------ attention (one library per head size and storage)
_attention_libs = {}
TENSOR_CORE_MAX_HEAD_DIM = 128


def _attention_source(head_dim: int, dtype: torch.dtype, kind: str):
    """bfloat16 heads up to 128 wide run on the tensor cores; float, and wider heads, on the CUDA cores."""
    if kind not in ("auto", "simt"):
        raise KernelError(f"unknown attention kernel kind {kind!r}")
    if kind == "auto" and dtype == torch.bfloat16 and head_dim <= TENSOR_CORE_MAX_HEAD_DIM:
        return "attention_mma.cu", {"HEAD_DIM": head_dim}
    return "attention.cu", {"HEAD_DIM": head_dim, "STORAGE_BF16": dtype_code(dtype)}


def attention_library(head_dim: int, dtype: torch.dtype, kind: str = "auto"):
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"attention kernels take head sizes that are multiples of 16 from 16 to 256, not {head_dim}")
    source, defines = _attention_source(head_dim, dtype, kind)
    key = (source, head_dim, dtype)
    lib = _attention_libs.get(key)
    if lib is None:
        lib = load_library(source, defines)
        for name in ("cisr_attn_prefill", "cisr_attn_decode", "cisr_attn_head_dim", "cisr_attn_prefill_tile"):
            getattr(lib, name).restype = ctypes.c_int
        assert lib.cisr_attn_head_dim() == head_dim
        lib._tensor_core = source == "attention_mma.cu"
        lib._tensor_maps = False
        if lib._tensor_core:
            lib.cisr_attn_set_pdl(int(_pdl_state["on"]))
            lib.cisr_attn_decode_tma_ok.restype = ctypes.c_int
            if head_dim % 64 == 0:          # the variant whose tiles arrive by tensor-map copies
                lib.cisr_attn_tma_init.restype = ctypes.c_int
                lib.cisr_attn_decode_tma.restype = ctypes.c_int
                lib.cisr_attn_decode_tma_launches.restype = ctypes.c_int
                lib.cisr_attn_set_clusters(int(_cluster_state["on"]))
                _check(lib.cisr_attn_tma_init(_p(_error_flag())), "attention tensor-map init", own=0)
                lib._tensor_maps = True
        _attention_libs[key] = lib
    return lib


_error_state = {}
_cluster_state = {"on": os.environ.get("CISR_CLUSTERS", "0") not in ("", "0")}


def set_clusters(on: bool) -> None:
    """Whether the decode attention merges the key ranges of a request inside thread-block clusters, or writes every
    range's partial sum for the merge kernel (the default: inside a chain of kernels that start early, clusters of 16
    did not all become resident at once and the step was slower; CISR_CLUSTERS=1 in the environment turns them on)."""
    _cluster_state["on"] = bool(on)
    for lib in _attention_libs.values():
        if lib._tensor_maps:
            lib.cisr_attn_set_clusters(int(on))


def _error_flag() -> torch.Tensor:
    """One int on the device that a kernel sets when one of its bounded waits ran out."""
    flag = _error_state.get("flag")
    if flag is None:
        flag = _error_state["flag"] = torch.zeros(1, dtype=torch.int32, device="cuda")
    return flag


def attention_jobs(head_dim: int, dtype: torch.dtype):
    """The build job of the attention library for this head size and storage type."""
    source, defines = _attention_source(head_dim, dtype, "auto")
    return (source, defines, ())


def attention_tcgen05_jobs(head_dim: int, dtype: torch.dtype):
    """The build jobs of the tcgen05 prompt attention, where this head size and storage type have one."""
    if dtype == torch.bfloat16 and head_dim in TCGEN05_HEAD_DIMS:
        return [("attention_tcgen05.cu", {"HEAD_DIM": head_dim}, ())]
    return []


TCGEN05_HEAD_DIMS = (64, 128)
WIDE_TILE = 128                  # queries per tile of the tcgen05 prompt attention
_attention_tcgen05_libs = {}


def _attention_tcgen05(head_dim: int):
    lib = _attention_tcgen05_libs.get(head_dim)
    if lib is None:
        lib = load_library("attention_tcgen05.cu", {"HEAD_DIM": head_dim})
        for name in ("cisr_attn_prefill_tcgen05", "cisr_attn_tcgen05_init", "cisr_attn_tcgen05_ok", "cisr_attn_tcgen05_tile"):
            getattr(lib, name).restype = ctypes.c_int
        assert lib.cisr_attn_tcgen05_tile() == WIDE_TILE
        _check(lib.cisr_attn_tcgen05_init(_p(_error_flag())), "tcgen05 attention init", own=0)
        lib.cisr_attn_tcgen05_set_pdl(int(_pdl_state["on"]))
        _attention_tcgen05_libs[head_dim] = lib
    return lib


def attn_prefill_wide_ok(q: torch.Tensor, k_cache: torch.Tensor, page_size: int) -> bool:
    """Whether the tcgen05 prompt attention takes these tensors: bfloat16, head size 64 or 128, a page size that is a
    multiple of 8 and divides 128 or is a multiple of it, 16-byte aligned contiguous buffers."""
    dim = k_cache.shape[-1]
    return (k_cache.dtype == torch.bfloat16 and q.dtype == torch.bfloat16 and dim in TCGEN05_HEAD_DIMS
            and page_size % 8 == 0 and (128 % page_size == 0 or page_size % 128 == 0)
            and k_cache.is_contiguous() and q.is_contiguous() and q.data_ptr() % 16 == 0 and k_cache.data_ptr() % 16 == 0
            and k_cache.shape[0] * k_cache.shape[1] * page_size < 2 ** 31)


def attn_prefill_wide(q, out, k_cache, v_cache, req_slot, block_table, wide_req, wide_q0, q_start, q_len, ctx_len, hq, hkv,
                      page_size, scale, window) -> None:
    """Attention of portions on tcgen05: q, out [tokens, hq, D]; tiles of 128 queries as (request, first query)."""
    dim = k_cache.shape[-1]
    _need(q, torch.bfloat16, "q", 3); _need(out, torch.bfloat16, "out", 3); _need(k_cache, torch.bfloat16, "k_cache", 4)
    _need(v_cache, torch.bfloat16, "v_cache", 4)
    for name, t in (("req_slot", req_slot), ("block_table", block_table), ("wide_req", wide_req), ("wide_q0", wide_q0),
                    ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    if not attn_prefill_wide_ok(q, k_cache, page_size):
        raise KernelError("attn_prefill_wide: not a head size, page size or buffer for the tcgen05 attention")
    lib = _attention_tcgen05(dim)
    _check(lib.cisr_attn_prefill_tcgen05(_p(q), _p(out), q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0], _p(req_slot),
                                         _p(block_table), block_table.shape[1], _p(wide_req), _p(wide_q0), wide_req.numel(),
                                         _p(q_start), _p(q_len), _p(ctx_len), hq, hkv, page_size, ctypes.c_float(scale),
                                         int(window or 0), _stream()), "attn_prefill_wide")


PREFILL_TILE = 64


def attn_prefill(q, out, k_cache, v_cache, req_slot, block_table, tile_req, tile_q0, q_start, q_len, ctx_len, hq, hkv,
                 page_size, scale, window, kind: str = "auto") -> None:
    """Attention of portions: q, out [tokens, hq, D]; tiles list (request, first query of the tile)."""
    dim = k_cache.shape[-1]
    _need(q, k_cache.dtype, "q"); _need(out, k_cache.dtype, "out"); _need(k_cache, None, "k_cache", 4)
    _need(v_cache, k_cache.dtype, "v_cache", 4)
    for name, t in (("req_slot", req_slot), ("block_table", block_table), ("tile_req", tile_req), ("tile_q0", tile_q0), ("q_start", q_start),
                    ("q_len", q_len), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    lib = attention_library(dim, k_cache.dtype, kind)
    _check(lib.cisr_attn_prefill(_p(q), _p(out), _p(k_cache), _p(v_cache), _p(req_slot), _p(block_table), block_table.shape[1],
                                 _p(tile_req), _p(tile_q0), tile_req.numel(), _p(q_start), _p(q_len), _p(ctx_len),
                                 hq, hkv, page_size, ctypes.c_float(scale), int(window or 0), _stream()), "attn_prefill")


def attn_decode(q, out, k_cache, v_cache, req_slot, block_table, dec_req, n_dec, q_start, ctx_len, partial, stats, hq, hkv,
                page_size, scale, window, split_size, n_splits, kind: str = "auto", staging: str = "auto", merge: bool = True) -> None:
    """Attention of single new tokens, split over key ranges of `split_size`, merged into out.

    `merge=False` (tensor-core kernels only) leaves the ranges' partial sums in `partial` and `stats` and does not write
    `out`: the caller merges them itself (`merge_out_proj`).

    `staging` picks how the tensor-core kernel brings key and value tiles in: "tensor_map" (one bulk copy per
    page), "gather" (a 16-byte copy per thread), or "auto": tensor maps where the head size (a multiple of 64), the
    page size (a multiple of 8 that divides 64 or is a multiple of it) and the range size allow them."""
    dim = k_cache.shape[-1]
    _need(q, k_cache.dtype, "q"); _need(out, k_cache.dtype, "out"); _need(k_cache, None, "k_cache", 4)
    _need(v_cache, k_cache.dtype, "v_cache", 4); _need(partial, torch.float32, "partial"); _need(stats, torch.float32, "stats")
    for name, t in (("req_slot", req_slot), ("block_table", block_table), ("dec_req", dec_req), ("q_start", q_start), ("ctx_len", ctx_len)):
        _need(t, torch.int32, name)
    if partial.numel() < n_dec * hq * n_splits * dim or stats.numel() < n_dec * hq * n_splits * 2:
        raise KernelError("attn_decode: scratch for partial sums is too small")
    lib = attention_library(dim, k_cache.dtype, kind)
    tail = [_p(req_slot), _p(block_table), block_table.shape[1], _p(dec_req), n_dec, _p(q_start), _p(ctx_len), _p(partial),
            _p(stats), hq, hkv, page_size, ctypes.c_float(scale), int(window or 0), split_size, n_splits]
    if lib._tensor_core:
        tail.append(int(merge))
    elif not merge:
        raise KernelError("attn_decode: only the tensor-core kernels leave the merge to the caller")
    tail.append(_stream())
    if staging not in ("auto", "tensor_map", "gather"):
        raise KernelError(f"unknown staging {staging!r}")
    tensor_maps = (lib._tensor_maps and lib.cisr_attn_decode_tma_ok(page_size, split_size) and k_cache.is_contiguous()
                   and v_cache.is_contiguous() and k_cache.data_ptr() % 16 == 0 and v_cache.data_ptr() % 16 == 0
                   and k_cache.shape[0] * hkv * page_size < 2 ** 31)
    if staging == "tensor_map" and not tensor_maps:
        raise KernelError("attn_decode: tensor-map staging does not take this head size, page size, range size or cache")
    if tensor_maps and staging != "gather":
        status = lib.cisr_attn_decode_tma(_p(q), _p(out), _p(k_cache), _p(v_cache), k_cache.shape[0], *tail)
        _check(status, "attn_decode", own=lib.cisr_attn_decode_tma_launches() if status == 0 else 0)
    else:
        _check(lib.cisr_attn_decode(_p(q), _p(out), _p(k_cache), _p(v_cache), *tail), "attn_decode",
               own=-(-(hq // hkv) // 16) + (1 if merge else 0))


# ------------------------------------------------------------------ merge of the key ranges + output projection (decode steps)
_merge_proj_state = {}


def _merge_proj():
    lib = _merge_proj_state.get("lib")
    if lib is None:
        lib = load_library("merge_proj.cu")
        lib.cisr_merge_proj.restype = ctypes.c_int
        lib.cisr_merge_proj_heads_per_cta.restype = ctypes.c_int
        lib.cisr_merge_proj_set_pdl(int(_pdl_state["on"]))
        _merge_proj_state["lib"] = lib
    return lib


def merge_proj_jobs():
    return [("merge_proj.cu", {}, ())]


MERGE_PROJ_MAX_BYTES = 8 << 20     # larger output projections are bandwidth-bound: the streaming product serves them, and the merge kernel is small beside it


def merge_out_proj_ok(n_dec: int, hq: int, dim: int, w: torch.Tensor) -> bool:
    """Whether `merge_out_proj` takes the shape: bfloat16 weights [N, hq * dim] of a latency-bound size, at most 16 tokens,
    head slices of at most 256 columns in at most 16 CTAs; and thread-block clusters in the attention kernel off."""
    return (0 < n_dec <= 16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[1] == hq * dim and w.numel() * 2 < MERGE_PROJ_MAX_BYTES
            and not _cluster_state["on"] and os.environ.get("CISR_MERGE_PROJ", "1") != "0"
            and _merge_proj().cisr_merge_proj_heads_per_cta(n_dec, hq, dim, w.shape[1]) > 0)


def merge_out_proj(partial: torch.Tensor, stats: torch.Tensor, n_splits: int, dec_req: torch.Tensor, q_start: torch.Tensor,
                   n_dec: int, hq: int, dim: int, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[row of request i] (float [tokens, N]) = (log-sum-exp merge of request i's key ranges, rounded to bfloat16) @ w^T:
    the merge kernel and the output projection of a decode step in one launch of a thread-block cluster.  With
    `accumulate` the product is added to what `out` holds (the residual stream)."""
    _need(partial, torch.float32, "partial"); _need(stats, torch.float32, "stats"); _need(w, torch.bfloat16, "w", 2)
    _need(out, torch.float32, "out", 2); _need(dec_req, torch.int32, "dec_req", 1); _need(q_start, torch.int32, "q_start", 1)
    if partial.numel() < n_dec * hq * n_splits * dim or stats.numel() < n_dec * hq * n_splits * 2 or out.shape[1] != w.shape[0]:
        raise KernelError("merge_out_proj: shapes disagree")
    status = _merge_proj().cisr_merge_proj(_p(partial), _p(stats), n_splits, _p(dec_req), _p(q_start), n_dec, hq, dim, _p(w),
                                           w.shape[0], w.shape[1], _p(out), int(bool(accumulate)), _stream())
    _check(status, "merge_out_proj")
    return out


# ------------------------------------------------------------------ sampling
def _sampling():
    lib = load_library("sampling.cu")
    if not getattr(lib, "_typed", False):
        lib.cisr_sample.restype = ctypes.c_int
        lib.cisr_decode_advance.restype = ctypes.c_int
        lib.cisr_uniform_host.restype = ctypes.c_float
        lib.cisr_uniform_host.argtypes = [ctypes.c_longlong, ctypes.c_longlong]
        lib._typed = True
    return lib


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor], seed: Optional[torch.Tensor],
           counter: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """Token per row: argmax where temperature <= 0 (or None), else inverse-CDF sampling."""
    _need(logits, torch.float32, "logits", 2); _need(out, torch.int32, "out", 1)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, torch.float32, "temperature", 1); _need(seed, torch.int64, "seed", 1)
        _need(counter, torch.int32, "counter", 1)
    _check(_sampling().cisr_sample(_p(logits), rows, vocab, _p(temperature), _p(seed), _p(counter), _p(out), _stream()),
           "sample")
    return out


def decode_advance(token_ids, positions, ctx_len, counter, sampled, live, ring: Optional[torch.Tensor] = None,
                   step_index: Optional[torch.Tensor] = None) -> None:
    """Feed sampled tokens back as the next inputs of live rows and advance their positions, lengths and counters.

    `ring` (int32 [slots, rows + 1]) with `step_index` (one int32): the sampled tokens and the kernels' error flag also
    go to slot step_index % slots, and step_index moves on by one."""
    for name, t in (("token_ids", token_ids), ("positions", positions), ("ctx_len", ctx_len), ("counter", counter),
                    ("sampled", sampled), ("live", live)):
        _need(t, torch.int32, name, 1)
    slots = 0
    if ring is not None:
        _need(ring, torch.int32, "ring", 2); _need(step_index, torch.int32, "step_index", 1)
        if ring.shape[1] != token_ids.numel() + 1:
            raise KernelError("decode_advance: ring must be [slots, rows + 1]")
        slots = ring.shape[0]
    _check(_sampling().cisr_decode_advance(_p(token_ids), _p(positions), _p(ctx_len), _p(counter), _p(sampled), _p(live),
                                           token_ids.numel(), _p(_error_state.get("flag")), _p(ring), slots, _p(step_index),
                                           _stream()), "decode_advance")


def uniform_host(seed: int, counter: int) -> float:
    """The uniform the device sampler draws for (seed, counter), computed on the host by the same code."""
    return float(_sampling().cisr_uniform_host(seed, counter))


# ------------------------------------------------------------------ library matrix product
_gemm_state = {}


def _gemm_library():
    lib = _gemm_state.get("lib")
    if lib is None:
        lib = load_library("gemm_library.cu", extra=("-lcublas",))
        lib.cisr_gemm_library_init.restype = ctypes.c_int
        lib.cisr_gemm_library.restype = ctypes.c_int
        workspace = torch.empty(GEMM_WORKSPACE_BYTES, dtype=torch.uint8, device="cuda")
        _check(lib.cisr_gemm_library_init(_p(workspace), ctypes.c_longlong(GEMM_WORKSPACE_BYTES)), "gemm library init")
        _gemm_state["lib"], _gemm_state["workspace"] = lib, workspace
    return lib


def gemm_library(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (float) = a[M, K] @ w[N, K]^T by the vendor library, float accumulation."""
    _need(a, None, "a", 2); _need(w, a.dtype, "w", 2); _need(out, torch.float32, "out", 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_gemm_library().cisr_gemm_library(_p(a), _p(w), dtype_code(a.dtype), _p(out), m, n, k, _stream()), "gemm",
           own=0, library=1)
    return out


def gemm_jobs(dtype: torch.dtype):
    """Build jobs of the libraries `gemm` may launch for operands of this dtype."""
    jobs = [("gemm_library.cu", {}, ("-lcublas",))]
    if dtype == torch.bfloat16:
        jobs.append(("gemm_tcgen05.cu", {}, ()))
    return jobs


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (float) = a[M, K] @ w[N, K]^T; picks the kernel for the shape and dtype.

    bfloat16 with at least one 128-row tile of tokens: this package's tcgen05 + TMA kernel; float (true 32-bit),
    and shapes that kernel does not take: the vendor library."""
    if tcgen05_ok(a, w):
        return gemm_tcgen05(a, w, out)
    return gemm_library(a, w, out)


# ------------------------------------------------------------------ weight-streaming products for few tokens
SKINNY_MAX_TOKENS = int(os.environ.get("CISR_SKINNY_MAX_TOKENS", "16"))   # most tokens the latency kernels are chosen for (they take up to 64)
SKINNY_NORM_MAX_TOKENS = 16      # beyond this the norm runs once as its own kernel instead of in every CTA
EPI_PLAIN, EPI_SWIGLU, EPI_ROPE = 0, 1, 2


def _skinny():
    lib = load_library("skinny_gemm.cu")
    if not getattr(lib, "_typed", False):
        lib.cisr_skinny_gemm.restype = ctypes.c_int
        lib._typed = True
    return lib


def set_pdl(on: bool) -> None:
    """Launch the decode-path kernels with programmatic dependent launch (a kernel may fetch its weights while the
    kernel before it is still running)."""
    _skinny().cisr_skinny_set_pdl(int(on))
    if "lib" in _stream_state:
        _stream_state["lib"].cisr_stream_set_pdl(int(on))
    for lib in _attention_tcgen05_libs.values():
        lib.cisr_attn_tcgen05_set_pdl(int(on))
    if "lib" in _merge_proj_state:
        _merge_proj_state["lib"].cisr_merge_proj_set_pdl(int(on))
    _elementwise().cisr_elementwise_set_pdl(int(on))
    _sampling().cisr_sampling_set_pdl(int(on))
    if "lib" in _tcgen05_state:
        _tcgen05_state["lib"].cisr_gemm_tcgen05_set_pdl(int(on))
    for (source, _, _), lib in list(_attention_libs.items()):
        if source == "attention_mma.cu":
            lib.cisr_attn_set_pdl(int(on))
    _pdl_state["on"] = bool(on)


def skinny_jobs():
    return [("skinny_gemm.cu", {}, ()), ("stream_gemm.cu", {}, ())]


def stream_takes(tokens: int, w: torch.Tensor) -> bool:
    """Whether skinny_gemm(kind="auto") hands this product to the persistent streaming kernel (stream_gemm.cu): a large
    bfloat16 weight matrix, at most 16 tokens, the tokens and at least three 16 KB stages in shared memory.  (The
    epilogues add their own conditions; where they fail the latency kernels take over.)"""
    if w.dtype != torch.bfloat16 or not 0 < tokens <= STREAM_MAX_TOKENS or w.shape[1] % 8 or w.numel() * 2 < STREAM_MIN_BYTES:
        return False
    padded = 8 if tokens <= 8 else 16
    fixed = 1024 + 64 + 4 * 8 * 16 * padded + tokens * (w.shape[1] + 8) * 2
    return fixed + 3 * (16384 + 16) <= 224 * 1024 - 8192          # 8 KB kept for the rotation tables of the ROPE epilogue


def skinny_ok(tokens: int, w: torch.Tensor) -> bool:
    """Shapes the weight-streaming kernels take: bfloat16 weights, at most 16 tokens, K a multiple of 8."""
    if w.dtype != torch.bfloat16 or not 0 < tokens <= SKINNY_MAX_TOKENS or w.shape[1] % 8:
        return False
    if stream_takes(tokens, w):
        return True
    padded = -(-tokens // 8) * 8
    return padded * (w.shape[1] + 8) * 2 + 64 * padded * 4 * 2 <= 200 * 1024     # the tokens and the partial sums fit in shared memory


def skinny_gemm(w: torch.Tensor, tokens: int, *, act: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None,
                delta: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                x_out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None, epilogue: int = EPI_PLAIN,
                out: Optional[torch.Tensor] = None, rope: Optional[dict] = None, kind: str = "auto",
                accumulate: bool = False) -> None:
    """out = prologue(input) @ w^T with a fused epilogue; see csrc/skinny_gemm.cu and csrc/stream_gemm.cu.

    `kind`: "latency" (skinny_gemm.cu: a CTA per 16 output rows, weights straight to registers), "stream"
    (stream_gemm.cu: persistent CTAs, weights through a ring of tensor-map copies; up to 16 tokens), or "auto": the
    streaming kernel for weight matrices of 8 MB and more where it takes the shape.

    Input is either `act` (bfloat16 [tokens, K]) or the norm prologue (`x`, optional `delta`, `norm_w`, `eps`,
    optional `x_out` receiving x + delta, optional `rows` picking rows of x).  PLAIN writes float `out`
    [tokens, N], or with `accumulate` adds the product to what `out` holds (the residual stream); SWIGLU writes bfloat16 `out` [tokens, N / 2]; ROPE takes the `rope` dict (cos, sin, rot_half,
    interleaved, q_out, k_cache, v_cache, positions, token_req, req_slot, block_table, page_size, hq, hkv, dim).
    """
    _need(w, torch.bfloat16, "w", 2)
    n, k = w.shape
    if act is not None:
        _need(act, torch.bfloat16, "act", 2)
        if act.shape[0] < tokens or act.shape[1] != k:
            raise KernelError("skinny_gemm: act must be [tokens, K]")
    else:
        _need(x, torch.float32, "x", 2); _need(norm_w, None, "norm_w", 1)
        if x.shape[1] != k or norm_w.numel() != k:
            raise KernelError("skinny_gemm: x and norm_w must be K wide")
        if delta is not None:
            _need(delta, torch.float32, "delta", 2)
        if x_out is not None:
            _need(x_out, torch.float32, "x_out", 2)
            if x_out.data_ptr() == x.data_ptr():
                raise KernelError("skinny_gemm: x_out must be another buffer than x")
        if rows is not None:
            _need(rows, torch.int32, "rows", 1)
    r = rope or {}
    out_f32 = out if epilogue == EPI_PLAIN else None
    out_b16 = out if epilogue == EPI_SWIGLU else None
    if epilogue == EPI_PLAIN:
        _need(out, torch.float32, "out", 2)
        if out.shape[0] < tokens or out.shape[1] != n:
            raise KernelError("skinny_gemm: out must be float [tokens, N]")
    elif epilogue == EPI_SWIGLU:
        _need(out, torch.bfloat16, "out", 2)
        if out.shape[0] < tokens or out.shape[1] * 2 != n:
            raise KernelError("skinny_gemm: out must be bfloat16 [tokens, N / 2]")
    else:
        for name in ("q_out", "k_cache", "v_cache"):
            _need(r[name], torch.bfloat16, name)
        for name in ("positions", "token_req", "req_slot", "block_table"):
            _need(r[name], torch.int32, name)
        if r["rot_half"]:
            _need(r["cos"], torch.float32, "cos", 2); _need(r["sin"], torch.float32, "sin", 2)
    args = (_p(w), n, k, _p(act), _p(x), _p(delta), _p(norm_w), dtype_code(norm_w.dtype) if norm_w is not None else 0,
            ctypes.c_float(eps), _p(x_out), _p(rows), tokens, epilogue, _p(out_f32), _p(out_b16),
            n // 2 if epilogue == EPI_SWIGLU else 0, _p(r.get("cos")), _p(r.get("sin")), int(r.get("rot_half", 0)),
            int(bool(r.get("interleaved", False))), _p(r.get("q_out")), _p(r.get("k_cache")), _p(r.get("v_cache")),
            _p(r.get("positions")), _p(r.get("token_req")), _p(r.get("req_slot")), _p(r.get("block_table")),
            r["block_table"].shape[1] if rope else 0, int(r.get("page_size", 0)), int(r.get("hq", 0)), int(r.get("hkv", 0)),
            int(r.get("dim", 0)), int(bool(accumulate)), _stream())
    if accumulate and epilogue != EPI_PLAIN:
        raise KernelError("skinny_gemm: only the plain epilogue adds into its output")
    if kind not in ("auto", "latency", "stream"):
        raise KernelError(f"unknown kind {kind!r}")
    if kind == "stream" or (kind == "auto" and tokens <= STREAM_MAX_TOKENS and w.numel() * 2 >= STREAM_MIN_BYTES):
        status = _stream_lib().cisr_stream_gemm(*args)
        if status != -2:                  # -2: not a shape for the streaming kernel
            _check(status, "stream_gemm")
            return
        if kind == "stream":
            raise KernelError("stream_gemm does not take this shape")
    _check(_skinny().cisr_skinny_gemm(*args), "skinny_gemm")


STREAM_MAX_TOKENS = 16
STREAM_MIN_BYTES = 8 << 20       # smaller weight matrices are latency-bound: the kernels of skinny_gemm.cu serve them better
_stream_state = {}


def _stream_lib():
    lib = _stream_state.get("lib")
    if lib is None:
        lib = load_library("stream_gemm.cu")
        lib.cisr_stream_gemm.restype = ctypes.c_int
        lib.cisr_stream_init.restype = ctypes.c_int
        _check(lib.cisr_stream_init(_p(_error_flag())), "stream gemm init", own=0)
        lib.cisr_stream_set_pdl(int(_pdl_state["on"]))
        _stream_state["lib"] = lib
    return lib


# ------------------------------------------------------------------ tcgen05 + TMA matrix product
_tcgen05_state = {}
TCGEN05_MIN_TOKENS = int(os.environ.get("CISR_TCGEN05_MIN_TOKENS", "128"))   # below one 128-row tile the weight-streaming kernels or the library serve better


def _tcgen05():
    lib = _tcgen05_state.get("lib")
    if lib is None:
        lib = load_library("gemm_tcgen05.cu")
        lib.cisr_gemm_tcgen05_init.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05_swiglu.restype = ctypes.c_int
        lib.cisr_gemm_tcgen05_rope.restype = ctypes.c_int
        _check(lib.cisr_gemm_tcgen05_init(_p(_error_flag())), "tcgen05 gemm init", own=0)
        lib.cisr_gemm_tcgen05_set_pdl(int(_pdl_state["on"]))
        _tcgen05_state["lib"] = lib
    return lib


def tcgen05_jobs():
    return [("gemm_tcgen05.cu", {}, ())]


# The product with rotation and cache write as its epilogue replaces two launches (the library's product and the rotate
# kernel), which pays from far fewer tokens on than the plain product does against the library's.
TCGEN05_FUSED_MIN_TOKENS = int(os.environ.get("CISR_TCGEN05_FUSED_MIN_TOKENS", "17"))


def tcgen05_ok(a: torch.Tensor, w: torch.Tensor, fused: bool = False) -> bool:
    least = min(TCGEN05_MIN_TOKENS, TCGEN05_FUSED_MIN_TOKENS) if fused else TCGEN05_MIN_TOKENS
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[0] >= least
            and a.shape[1] % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[M, N] (float) = a[M, K] @ w[N, K]^T on tcgen05 tensor cores fed by TMA (bfloat16 operands); with
    `accumulate`, out += the product (the residual add as the product's epilogue)."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2); _need(out, torch.float32, "out", 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_tcgen05().cisr_gemm_tcgen05(_p(a), _p(w), _p(out), m, n, k, int(accumulate), _stream()), "gemm_tcgen05")
    return out


def gemm_tcgen05_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out (bfloat16 [M, I]) = silu(a @ w[:I]^T) * (a @ w[I:]^T): the product with SwiGLU as its epilogue."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2); _need(out, torch.bfloat16, "out", 2)
    m, k = a.shape
    inter = out.shape[1]
    if w.shape != (2 * inter, k) or out.shape[0] != m:
        raise KernelError(f"gemm swiglu: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)} disagree")
    _check(_tcgen05().cisr_gemm_tcgen05_swiglu(_p(a), _p(w), _p(out), m, inter, k, _stream()), "gemm_tcgen05_swiglu")
    return out


def tcgen05_rope_ok(dim: int, rot_half: int, interleaved: bool) -> bool:
    """The rotation epilogue takes heads of 64 or 128 rotated over their whole width in split-half pairs."""
    return dim in (64, 128) and 2 * rot_half == dim and not interleaved


def gemm_tcgen05_rope(a: torch.Tensor, w: torch.Tensor, rope: dict) -> None:
    """The stacked q/k/v product with rotation and cache write as its epilogue (`rope` as for skinny_gemm)."""
    _need(a, torch.bfloat16, "a", 2); _need(w, torch.bfloat16, "w", 2)
    m, k = a.shape
    hq, hkv, dim = rope["hq"], rope["hkv"], rope["dim"]
    if w.shape != ((hq + 2 * hkv) * dim, k):
        raise KernelError("gemm rope: w must stack the q, k and v heads")
    for name in ("q_out", "k_cache", "v_cache"):
        _need(rope[name], torch.bfloat16, name)
    for name in ("positions", "token_req", "req_slot", "block_table"):
        _need(rope[name], torch.int32, name)
    _need(rope["cos"], torch.float32, "cos", 2); _need(rope["sin"], torch.float32, "sin", 2)
    if rope["cos"].shape != (m, dim // 2):
        raise KernelError("gemm rope: rotary tables must be [tokens, head_dim / 2]")
    _check(_tcgen05().cisr_gemm_tcgen05_rope(
        _p(a), _p(w), m, k, _p(rope["cos"]), _p(rope["sin"]), _p(rope["q_out"]), _p(rope["k_cache"]), _p(rope["v_cache"]),
        _p(rope["positions"]), _p(rope["token_req"]), _p(rope["req_slot"]), _p(rope["block_table"]),
        rope["block_table"].shape[1], rope["page_size"], hq, hkv, dim, _stream()), "gemm_tcgen05_rope")


_GAVE_UP = {1: "a tcgen05 matrix product gave up waiting on a barrier",
            3: "an attention kernel gave up waiting on a tensor-map copy",
            4: "a weight-streaming product gave up waiting on a tensor-map copy",
            5: "the tcgen05 attention gave up waiting on a barrier"}


def error_flag_tensor() -> Optional[torch.Tensor]:
    """The device flag, for callers that copy it to the host behind a step of their own (None before any kernel that
    can give up was loaded)."""
    return _error_state.get("flag")


def raise_for_code(code: int) -> None:
    """The error for a value read from the flag; clears the flag on the device."""
    if code != 0:
        flag = _error_state.get("flag")
        if flag is not None:
            flag.zero_()
        raise KernelError(f"{_GAVE_UP.get(code, _GAVE_UP[1])}; its output is not valid")


def raise_if_kernel_gave_up() -> None:
    """Reads the flag a kernel sets when one of its bounded waits ran out (synchronises the device)."""
    flag = _error_state.get("flag")
    if flag is not None:
        raise_for_code(int(flag.item()))


# ------------------------------------------------------------------ per-launch timing, for measurement only
_timing = {"records": None}


class timed_launches:
    """Inside this context every kernel function of this module is bracketed by two CUDA events on the current stream;
    `records` collects (function name, shape description, begin event, end event).  Used by bench.py for the
    per-kernel figures (launches run one after the other, outside graphs, so these are isolated kernel times); the
    engine never turns it on.  Read the times with `summary()` after a synchronisation."""

    def __enter__(self):
        self.records = []
        _timing["records"] = self.records
        return self

    def __exit__(self, *exc):
        _timing["records"] = None
        return False

    def summary(self) -> dict:
        """(name, shape) -> {"launches", "us"}: total device time between the two events of each launch."""
        torch.cuda.synchronize()
        out = {}
        for name, shape, begin, end in self.records:
            entry = out.setdefault((name, shape), {"launches": 0, "us": 0.0})
            entry["launches"] += 1
            entry["us"] += begin.elapsed_time(end) * 1e3
        return out


def _describe_gemm(a, w, *rest, **kw):
    return (int(a.shape[0]), int(w.shape[0]), int(w.shape[1]))


_DESCRIBE = {
    "embedding": lambda table, ids, out: (int(out.shape[0]), int(out.shape[1])),
    "add_rmsnorm": lambda x, delta, weight, eps, out, rows=None, write_back=True: (int(out.shape[0]), int(out.shape[1]), delta is not None),
    "swiglu": lambda gate_up, out: (int(out.shape[0]), int(out.shape[1])),
    "rotary_tables": lambda positions, inv_freq, cos, sin: (int(cos.shape[0]), int(cos.shape[1])),
    "rope_store": lambda proj, *rest, **kw: (int(proj.shape[0]), int(proj.shape[1])),
    "page_copy": lambda *a, **kw: (),
    "table_update": lambda *a, **kw: (),
    "attn_prefill_wide": lambda q, out, k_cache, *rest, **kw: (int(q.shape[0]), int(q.shape[1]), int(k_cache.shape[1]), int(q.shape[2])),
    "attn_prefill": lambda q, out, k_cache, *rest, **kw: (int(q.shape[0]), int(q.shape[1]), int(k_cache.shape[1]), int(q.shape[2])),
    "attn_decode": lambda q, out, k_cache, v_cache, req_slot, block_table, dec_req, n_dec, *rest, **kw:
        (int(n_dec), int(q.shape[1]), int(k_cache.shape[1]), int(q.shape[2]), bool(kw.get("merge", True))),
    "merge_out_proj": lambda partial, stats, n_splits, dec_req, q_start, n_dec, hq, dim, w, out, **kw:
        (int(n_dec), int(w.shape[0]), int(w.shape[1]), int(n_splits)),
    "sample": lambda logits, *rest, **kw: (int(logits.shape[0]), int(logits.shape[1])),
    "decode_advance": lambda *a, **kw: (),
    "gemm_library": _describe_gemm,
    "gemm_tcgen05": _describe_gemm,
    "gemm_tcgen05_swiglu": _describe_gemm,
    "gemm_tcgen05_rope": _describe_gemm,
    "skinny_gemm": lambda w, tokens, **kw: (int(tokens), int(w.shape[0]), int(w.shape[1]), int(kw.get("epilogue", EPI_PLAIN)),
                                            kw.get("act") is None),
}


def _instrument() -> None:
    import functools

    def wrap(name, describe):
        fn = globals()[name]

        @functools.wraps(fn)
        def launched(*args, **kwargs):
            records = _timing["records"]
            if records is None:
                return fn(*args, **kwargs)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            result = fn(*args, **kwargs)
            end.record()
            records.append((name, describe(*args, **kwargs), begin, end))
            return result

        globals()[name] = launched

    for name, describe in _DESCRIBE.items():
        wrap(name, describe)


_instrument()
