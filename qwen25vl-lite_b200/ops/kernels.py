"""Python face of the CUDA kernels: each function checks its tensors and launches one kernel
on torch's current stream through ctypes.

There is no fallback: on a machine without the built library, or when a launch fails, the
call raises.  Tensors are torch CUDA tensors used as typed device buffers; nothing here
calls a torch operator on the data.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from .build import build_library

_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float
_LL = ctypes.c_longlong

_SIGNATURES = {
    "q25_embed_gather": [_P, _P, _P, _I, _I, _I, _F, _P],
    "q25_add_rmsnorm": [_P, _P, _P, _F, _P, _P, _I, _I, _P],
    "q25_silu_mul": [_P, _P, _I, _I, _I, _P],
    "q25_rope_store": [_P, _P, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "q25_paged_attention_generic": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P],
    "q25_embed_position_norm": [_P, _P, _P, _P, _P, _F, _P, _I, _I, _I, _I, _I, _F, _P],
    "q25_add_norm_groups": [_P, _P, _P, _F, _I, _P, _F, _I, _P, _P, _I, _I, _P],
    "q25_glu_clamped": [_P, _P, _I, _I, _F, _F, _F, _I, _P],
    "q25_rglru_conv": [_P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "q25_rglru_scan": [_P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, _I, _I, _P],
    "q25_biased_attention_generic": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P, _I, _F, _P, _I, _I, _P],
    "q25_biased_attention_qk_norm_store": [_P, _I, _P, _P, _F, _I, _P, _I, _I, _P, _F, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "q25_add_dyt": [_P, _P, _P, _P, _F, _P, _P, _I, _I, _P],
    "q25_rotary_apply": [_P, _I, _I, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "q25_latent_store": [_P, _I, _I, _I, _P, _F, _P, _I, _I, _P, _P, _I, _P],
    "q25_retention": [_P, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _F, _P, _I, _P, _I, _P, _I, _I, _P],
    "q25_kv_store_mix": [_P, _I, _P, _I, _F, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "q25_moe_route": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "q25_moe_gate_up": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _F, _I, _P, _P],
    "q25_moe_down": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "q25_moe_combine": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    "q25_moe_route_softmax": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P],
    "q25_moe_combine_weighted": [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "q25_activation": [_P, _P, _LL, _I, _P],
    "q25_add_layernorm": [_P, _P, _P, _P, _P, _F, _P, _P, _F, _P, _P, _I, _I, _P],
    "q25_branch_mean_norm": [_P, _P, _I, _P, _I, _I, _F, _P],
    "q25_stream_pair": [_P, _P, _P, _I, _I, _P],
    "q25_memory_gla_decay": [_P, _I, _I, _I, _P, _P, _F, _P, _I, _I, _P],
    "q25_memory_row_dots": [_P, _P, _P, _P, _I, _I, _I, _P],
    "q25_memory_scan": [_P, _I, _I, _I, _I, _P, _P, _F, _F, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "q25_memory_scan_chunked": [_P, _I, _I, _I, _I, _P, _P, _F, _F, _P, _P, _P, _P, _P, _I, _P, _I, _P, _I, _P, _P, _I, _I, _I, _I, _P],
    "q25_memory_output": [_P, _P, _P, _I, _I, _P, _P, _I, _I, _I, _I, _F, _I, _P],
}
_UNTYPED = {
    "q25_attention_decode_bf16": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "q25_attention_prefill_bf16": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P],
    "q25_gemm_f32": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "q25_gemm_tcgen05_bf16": [_P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P, _P],
    "q25_sample_rows": [_P, _LL, _I, _I, _P, _P, _P, _P, _P, _P],
    "q25_apply_penalties": [_P, _LL, _I, _I, _P, _P, _P, _P, _P, _P, _P],
}

_SUFFIX = {torch.float32: "_f32", torch.bfloat16: "_bf16"}
_libs: Dict[str, ctypes.CDLL] = {}
_fns: Dict[str, object] = {}


class KernelError(RuntimeError):
    pass


def load_library(name: str = "core") -> ctypes.CDLL:
    """Builds (first use) and loads a kernel library; raises if that is not possible."""
    lib = _libs.get(name)
    if lib is None:
        path = build_library(name)
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise KernelError(f"cannot load the CUDA kernel library {path}: {exc}") from exc
        _libs[name] = lib
    return lib


# which library holds a symbol, by the symbol's beginning (everything else is in "core"); a
# library is compiled and loaded when one of its kernels is first asked for
_SYMBOL_LIBRARY = (("q25_gemm_chain", "chain"), ("q25_attention_decode", "bf16"), ("q25_attention_prefill", "bf16"),
                   ("q25_gemm_tcgen05", "tcgen05"), ("q25_rope_angles", "bf16"), ("q25_rglru", "recurrent"),
                   ("q25_biased_attention", "biased"), ("q25_kv_store_mix", "biased"), ("q25_moe", "routed"),
                   ("q25_rotary", "rotary"), ("q25_latent", "latent"), ("q25_retention", "retention"), ("q25_memory", "memory"))


def _library_of(symbol: str) -> str:
    for prefix, library in _SYMBOL_LIBRARY:
        if symbol.startswith(prefix):
            return library
    return "core"


def _fn(symbol: str, argtypes, library: Optional[str] = None):
    if _chain and symbol not in _CHAIN_SAFE:
        chain_flush()                       # products that wait in the chain come before this kernel
    f = _fns.get(symbol)
    if f is None:
        lib = load_library(library or _library_of(symbol))
        try:
            f = getattr(lib, symbol)
        except AttributeError as exc:
            raise KernelError(f"the kernel library has no symbol {symbol}") from exc
        f.argtypes = argtypes
        f.restype = _I
        _fns[symbol] = f
    return f


def _typed(base: str, dtype: torch.dtype):
    try:
        return _fn(base + _SUFFIX[dtype], _SIGNATURES[base])
    except KeyError:
        raise KernelError(f"{base}: unsupported dtype {dtype}") from None


_launches = 0
_sm_count: Dict[int, int] = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device, asked once (148 on the B200 the kernels'
    heuristics were measured on); grids and split counts are derived from it."""
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    n = _sm_count.get(dev)
    if n is None:
        n = int(_fn("q25_sm_count", [], "core")()) if dev >= 0 else 148
        if n <= 0:
            raise KernelError("cannot read the device's multiprocessor count")
        _sm_count[dev] = n
    return n


def chain_grid() -> int:
    """CTAs of the chain kernel (one per SM); its barrier counter advances by this per barrier."""
    return int(_fn("q25_gemm_chain_grid", [])())


def launch_count() -> int:
    """How many kernels of this engine have been launched by this process."""
    return _launches


def count_replayed(n: int) -> None:
    """Launches that ran from a captured graph (they do not pass through ``_check``)."""
    global _launches
    _launches += n


def _check(code: int, what: str) -> None:
    global _launches
    _launches += 1
    if code != 0:
        raise KernelError(f"CUDA kernel {what} could not be launched: cudaError {code} "
                          f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


# torch's current stream as a raw handle.  ``torch.cuda.current_stream()`` builds a Python object on every call (3.3 us
# measured, a quarter of a millisecond over the 80 launches of a prompt step); torch's own C entry points hand out the
# same handle in 0.1 us, and are used where this torch has them.
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return _RAW_STREAM(_RAW_DEVICE())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _dev(t: torch.Tensor, dtype: torch.dtype, what: str) -> torch.Tensor:
    if not t.is_cuda or t.dtype != dtype or not t.is_contiguous():
        raise KernelError(f"{what}: needs a contiguous CUDA tensor of {dtype}, got {t.dtype} on {t.device}, "
                          f"contiguous={t.is_contiguous()}")
    return t


# ---------------------------------------------------------------------------------------------


def embed_gather(table: torch.Tensor, ids: torch.Tensor, x_out: torch.Tensor, scale: float = 1.0) -> None:
    """x_out[n, :] (float32) = table[ids[n], :] * scale."""
    n, hidden = x_out.shape
    _dev(ids, torch.int32, "embed_gather ids"); _dev(x_out, torch.float32, "embed_gather out")
    _check(_typed("q25_embed_gather", table.dtype)(table.data_ptr(), ids.data_ptr(), x_out.data_ptr(), n, hidden,
                                                   table.shape[0], float(scale), _stream()), "embed_gather")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (when given); out = rmsnorm(x) * weight.  With ``rows`` only those rows are
    normalised into out[0..len(rows)) and x is left as it is."""
    hidden = x.shape[-1]
    n_out = out.shape[0]
    _dev(x, torch.float32, "add_rmsnorm x"); _dev(weight, torch.float32, "add_rmsnorm weight")
    if delta is not None:
        _dev(delta, out.dtype, "add_rmsnorm delta")
    if rows is not None:
        _dev(rows, torch.int32, "add_rmsnorm rows")
    _check(_typed("q25_add_rmsnorm", out.dtype)(x.data_ptr(), _ptr(delta), weight.data_ptr(), float(eps),
                                                out.data_ptr(), _ptr(rows), n_out, hidden, _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, paired: bool = False) -> None:
    """out = silu(gate) * up.  ``gate_up`` rows hold gate then up (halves), or with ``paired``
    groups of 8 gate features followed by their 8 up features."""
    n, inter = out.shape
    _dev(gate_up, out.dtype, "silu_mul input")
    if paired and inter % 8:
        raise KernelError(f"silu_mul: the paired layout needs a width that is a multiple of 8, got {inter}")
    _check(_typed("q25_silu_mul", out.dtype)(gate_up.data_ptr(), out.data_ptr(), n, inter, int(paired), _stream()),
           "silu_mul")


def rope_store(qkv: torch.Tensor, positions: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
               axis: Optional[torch.Tensor], k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
               kv_slot: Optional[torch.Tensor], nq: int, nkv: int, head_dim: int, page_size: int,
               angles: Optional[torch.Tensor] = None) -> None:
    """Rotates q (in place) and k by the position encoding and writes k, v into the pages at
    ``kv_slot``.  positions None: no rotation; pages None: nothing stored.  ``angles``: what
    ``rope_angles`` made of these positions (float32 [N, D/2, 2]); given, the kernel reads the
    cosines and sines there instead of computing them again in every layer."""
    n = qkv.shape[0]
    rotate = positions is not None
    store = k_pages is not None
    if angles is not None and (angles.dtype != torch.float32 or tuple(angles.shape) != (n, head_dim // 2, 2)
                               or not angles.is_contiguous()):
        raise KernelError(f"rope_store: angles must be float32 [{n}, {head_dim // 2}, 2]")
    _check(_typed("q25_rope_store", qkv.dtype)(
        qkv.data_ptr(), _ptr(positions), n, _ptr(inv_freq), _ptr(axis), _ptr(k_pages), _ptr(v_pages), _ptr(kv_slot),
        nq, nkv, head_dim, page_size, int(rotate), int(store), _ptr(angles), _stream()), "rope_store")


def paged_attention_generic(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                            block_table: torch.Tensor, token_seq: torch.Tensor, cu_q: torch.Tensor,
                            q_start_pos: torch.Tensor, nq: int, nkv: int, head_dim: int, page_size: int,
                            window: int, scale: float) -> None:
    n = qkv.shape[0]
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention: head size {head_dim} is not a multiple of 16 up to 256")
    _check(_typed("q25_paged_attention_generic", qkv.dtype)(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), cu_q.data_ptr(), q_start_pos.data_ptr(), n, nq, nkv, head_dim,
        page_size, int(window or 0), float(scale), _stream()), "paged_attention_generic")


def attention_mma_supports(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Sizes the tensor-core attention kernels take; everything else goes to the general kernel."""
    return (dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 128
            and page_size > 0 and page_size & (page_size - 1) == 0)


def attention_decode(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor, items: torch.Tensor,
                     nq: int, nkv: int, head_dim: int, page_size: int, window: int, scale: float, n_splits: int,
                     scratch: Optional[torch.Tensor]) -> None:
    """Tensor-core attention for the entries listed in ``items`` (int32 entry indices), each
    of which brings exactly one token.  With ``n_splits`` > 1 the keys of an entry are cut
    into that many ranges whose partial results go through ``scratch`` (float32, at least
    ``len(items) * nq * n_splits * (head_dim + 2)`` elements)."""
    n_items = items.shape[0]
    if nq // nkv > 16:
        raise KernelError("attention_decode: more than 16 query heads per kv head; use attention_prefill")
    if n_splits > 1:
        need = n_items * nq * n_splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode: {n_splits} splits need {need} float32 of scratch memory")
    _check(_fn("q25_attention_decode_bf16", _UNTYPED["q25_attention_decode_bf16"])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), items.data_ptr(), n_items, nq, nkv, head_dim,
        page_size, int(window or 0), float(scale), int(n_splits), _ptr(scratch), _stream()), "attention_decode")


def attention_fused_supports(dtype: torch.dtype, head_dim: int, page_size: int, group: int) -> bool:
    return attention_mma_supports(dtype, head_dim, page_size) and head_dim % 32 == 0 and group <= 16


def attention_decode_fused(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                           block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor, items: torch.Tensor,
                           nq: int, nkv: int, head_dim: int, page_size: int, window: int, scale: float, n_splits: int,
                           positions: torch.Tensor, inv_freq: torch.Tensor, axis: torch.Tensor,
                           kv_slot: torch.Tensor, scratch: Optional[torch.Tensor] = None,
                           angles: Optional[torch.Tensor] = None, dense: bool = False) -> None:
    """One kernel for a step of one-token entries: rotary encoding of q and the new k
    (``positions`` int32 [axes, N], ``inv_freq`` float32 [D/2], ``axis`` int32 [D/2]), the write of
    the new k and v at ``kv_slot``, attention, and the merge of the ``n_splits`` key ranges
    (through ``scratch`` as for ``attention_decode``; the CTA that finishes last merges).
    ``qkv`` is read as projected and left unchanged.  ``angles``: the step's table from
    ``rope_angles`` (the kernel computes the angles itself without it).
    ``dense``: ``items`` is 0 .. n-1 and every entry has exactly one token (the kernel then skips two look-ups)."""
    n_items = items.shape[0]
    if angles is not None and (angles.dtype != torch.float32 or tuple(angles.shape) != (positions.shape[1], head_dim // 2, 2)
                               or not angles.is_contiguous()):
        raise KernelError("attention_decode_fused: angles must be float32 [N, D/2, 2]")
    if n_splits > 1:
        need = n_items * nq * n_splits * (head_dim + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode_fused: {n_splits} splits need {need} float32 of scratch memory")
    if not attention_fused_supports(qkv.dtype, head_dim, page_size, nq // nkv) or n_splits < 1:
        raise KernelError(f"attention_decode_fused: unsupported head size {head_dim}, page size {page_size}, "
                          f"group {nq // nkv} or splits {n_splits}")
    if positions.dtype != torch.int32 or positions.dim() != 2 or (angles is None and positions.shape[0] != 3):
        raise KernelError("attention_decode_fused: positions must be int32 [axes, N]; without an angle table the kernel "
                          "computes the angles itself and reads three axes")
    _check(_fn("q25_attention_decode_fused_bf16",
               [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _P])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), items.data_ptr(), items.shape[0], nq, nkv,
        head_dim, page_size, int(window or 0), float(scale), int(n_splits), positions.data_ptr(), positions.shape[1],
        inv_freq.data_ptr(), axis.data_ptr(), kv_slot.data_ptr(), _ptr(scratch),
        _split_counters(qkv.device, n_items * nkv).data_ptr(), _ptr(angles), int(bool(dense)),
        _stream()), "attention_decode_fused")


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor, axis: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of every token's rotary angles, float32 [N, D/2, 2]: ``positions`` int32 [axes, N],
    ``inv_freq`` float32 [D/2], ``axis`` int32 [D/2] (which position axis drives each channel)."""
    n, half = positions.shape[1], inv_freq.shape[0]
    _dev(positions, torch.int32, "rope_angles positions"); _dev(inv_freq, torch.float32, "rope_angles inv_freq")
    _dev(axis, torch.int32, "rope_angles axis")
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(_fn("q25_rope_angles", [_P, _I, _P, _P, _I, _P, _P])(
        positions.data_ptr(), n, inv_freq.data_ptr(), axis.data_ptr(), half, out.data_ptr(), _stream()), "rope_angles")
    return out


_counters: Dict[torch.device, torch.Tensor] = {}


def _split_counters(device, n: int) -> torch.Tensor:
    """Zeroed ints the fused decode attention counts its finished splits in (it leaves them zero)."""
    buf = _counters.get(device)
    if buf is None or buf.numel() < n:
        buf = _counters[device] = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
    return buf


def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor, tiles: torch.Tensor,
                      nq: int, nkv: int, head_dim: int, page_size: int, window: int, scale: float) -> None:
    """Tensor-core attention for runs of tokens.  ``tiles`` is int32 [n, 2]: (entry, row
    tile), a row tile being 64 consecutive rows of the entry's (token, head of the kv group)
    pairs, token-major."""
    _check(_fn("q25_attention_prefill_bf16", _UNTYPED["q25_attention_prefill_bf16"])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0], nq, nkv,
        head_dim, page_size, int(window or 0), float(scale), _stream()), "attention_prefill")


def attention_tcgen05_supports(dtype: torch.dtype, head_dim: int, page_size: int, qkv: Optional[torch.Tensor] = None) -> bool:
    """What the tcgen05 prefill attention takes: bfloat16, head size 128, a page size that is a power
    of two, 16-byte aligned rows."""
    if dtype != torch.bfloat16 or head_dim != 128 or page_size < 1 or page_size & (page_size - 1):
        return False
    return qkv is None or (qkv.data_ptr() % 16 == 0 and qkv.stride(0) % 8 == 0 and qkv.stride(1) == 1)


def attention_prefill_tcgen05(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                              block_table: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor,
                              tiles: torch.Tensor, nq: int, nkv: int, head_dim: int, page_size: int, window: int,
                              scale: float, merges: Optional[torch.Tensor] = None,
                              scratch: Optional[torch.Tensor] = None, pairs: bool = False,
                              sink: Optional[torch.Tensor] = None, gate_off: int = -1,
                              dist_bias: Optional[torch.Tensor] = None) -> None:
    """``attention_prefill`` on the tcgen05 tensor cores (scores, P and the outputs in tensor memory).
    ``tiles`` is int32 [n, 3]: (entry, row tile, code) with row tiles of 128 rows; code 1 is a whole
    tile, else first part << 8 | part << 4 | parts: one of the parts its keys are cut into, which
    leaves unnormalised sums in ``scratch`` (float32, room for n * nkv * 128 * (head_dim + 2)).
    ``merges`` is int32 [m, 4]: (entry, row tile, first part, parts) of the cut tiles, which a second
    kernel adds up.  ``pairs``: every piece of work goes to a cluster of two CTAs instead; code 2 then
    means half of the keys for each, added up through the cluster's shared memory, code 1 the whole
    tile for one of them.  ``sink`` (float32 [nq]) joins each head's denominator; ``gate_off`` >= 0 (a multiple of 8):
    the rows of ``qkv`` hold nq * head_dim gate channels there, whose sigmoid multiplies the result.  ``dist_bias``
    (float32 [rows, nq]): ``dist_bias[min(i - j, rows - 1), head]`` is added to the scaled score."""
    if sink is not None:
        _dev(sink, torch.float32, "attention sink")
    _check_dist_bias(dist_bias, nq)
    if gate_off >= 0 and gate_off % 8:
        raise KernelError("attention_prefill_tcgen05: the gate channels must start on a 16-byte boundary")
    if not attention_tcgen05_supports(qkv.dtype, head_dim, page_size, qkv):
        raise KernelError(f"attention_prefill_tcgen05: unsupported head size {head_dim}, page size {page_size} or layout")
    if tiles.dim() != 2 or tiles.shape[1] != 3:
        raise KernelError("attention_prefill_tcgen05: the work list is (entry, row tile, code) triples")
    n_merge = 0 if merges is None else merges.shape[0]
    if n_merge and (pairs or scratch is None or scratch.dtype != torch.float32
                    or scratch.numel() < tiles.shape[0] * nkv * 128 * (head_dim + 2)):
        raise KernelError("attention_prefill_tcgen05: cut tiles need float32 scratch for every piece of work, and no pairs")
    if pairs and window:
        raise KernelError("attention_prefill_tcgen05: keys behind a window are not cut")
    _check(_fn("q25_attention_prefill_tcgen05_bf16",
               [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _I, _P, _I, _P, _I, _P, _I, _P, _P])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), tiles.data_ptr(), tiles.shape[0], nq, nkv,
        head_dim, page_size, int(window or 0), float(scale), _ptr(merges), n_merge, _ptr(scratch), int(bool(pairs)),
        _ptr(sink), int(gate_off), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0],
        error_flag(qkv.device).data_ptr(), _stream()), "attention_prefill_tcgen05")
    if n_merge:
        count_replayed(1)                      # the merge kernel, launched by the same call


def gemm_f32(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] . w[N,K]^T + bias, plain float32 FMA."""
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype != torch.float32 or not t.is_cuda or t.stride(1) != 1:
            raise KernelError(f"gemm_f32 {what}: needs a float32 CUDA matrix with unit inner stride")
    _check(_fn("q25_gemm_f32", _UNTYPED["q25_gemm_f32"])(
        a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), m, n, k, a.stride(0), w.stride(0), out.stride(0),
        _stream()), "gemm_f32")


SKINNY_STORE, SKINNY_BIAS, SKINNY_F32, SKINNY_SWIGLU, SKINNY_RESIDUAL, SKINNY_GLU, SKINNY_RELU2 = 0, 1, 2, 3, 4, 5, 6
# Rows the weight-streaming kernel takes: the 8 batch columns of one m16n8k16 MMA.  A variant with two
# column tiles ran 9 to 16 rows; measured against the library path on B200 it lost at every size (a
# decode step of 9 / 12 / 16 requests at the 3B sizes 2.64 / 2.66 / 2.65 ms against 2.43 / 2.55 / 2.59,
# 14 layers of the 7B sizes 2.55 / 2.61 / 2.75 against 1.92 / 2.02 / 2.02 ms) and is gone.
SKINNY_MAX_ROWS = 8
_error_flags: Dict[torch.device, torch.Tensor] = {}


def error_flag(device) -> torch.Tensor:
    """One int32 per device that kernels with bounded waits set when a wait gave up."""
    device = torch.device(device)
    flag = _error_flags.get(device)
    if flag is None:
        flag = _error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return flag


def gemm_skinny_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 1 <= x.shape[0] <= SKINNY_MAX_ROWS
            and w.shape[1] % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int) -> None:
    """out = x . w^T for at most 8 rows of x, streaming the weights once (bfloat16).
    ``epilogue``: SKINNY_STORE, SKINNY_BIAS (float32 bias), SKINNY_F32 (float32 out),
    SKINNY_SWIGLU (w rows are groups of 8 gate + 8 up features; out has half as many columns),
    SKINNY_GLU (the same layout with the clamped gated unit; ``bias`` then holds its two constants,
    float32 [limit, alpha]), SKINNY_RELU2 (the square of relu of the product) or SKINNY_RESIDUAL (out is float32 and
    the product is added into it).  Runs as an operation
    of the chain kernel (``csrc/gemm_chain.cu``): at once and alone, or, between ``chain_begin``
    and ``chain_end``, together with the products around it."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_skinny_supports(x, w) or w.shape[1] != k or not w.is_contiguous():
        raise KernelError(f"gemm_skinny: unsupported operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype}")
    _skinny_out(out, m, n, epilogue, "gemm_skinny")
    _chain_add(x, None, 0.0, w, bias, out, epilogue)


def _skinny_out(out: torch.Tensor, m: int, n: int, epilogue: int, what: str) -> None:
    cols = n // 2 if epilogue in (SKINNY_SWIGLU, SKINNY_GLU) else n
    want = torch.float32 if epilogue in (SKINNY_F32, SKINNY_RESIDUAL) else torch.bfloat16
    if out.shape != (m, cols) or out.dtype != want or out.stride(1) != 1:
        raise KernelError(f"{what}: output must be [{m}, {cols}] {want}")
    if epilogue in (SKINNY_SWIGLU, SKINNY_GLU) and n % 16:
        raise KernelError(f"{what}: a gated epilogue needs groups of 8 gate and 8 up rows, got {n} rows")


def gemm_skinny_norm_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_skinny_norm`` takes the float32 rows ``x`` (the residual stream) and ``w``."""
    return (x.dtype == torch.float32 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and 1 <= x.shape[0] <= SKINNY_MAX_ROWS and w.shape[1] % 32 == 0
            and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_skinny_norm(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor,
                     bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int) -> None:
    """out = (rmsnorm(x) * norm_weight) . w^T with the normalisation done inside the kernel;
    x is float32 [M <= 8, K], everything else as for ``gemm_skinny``."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_skinny_norm_supports(x, w) or w.shape[1] != k:
        raise KernelError(f"gemm_skinny_norm: unsupported operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype}")
    _dev(norm_weight, torch.float32, "gemm_skinny_norm norm weight")
    _skinny_out(out, m, n, epilogue, "gemm_skinny_norm")
    _chain_add(x, norm_weight, eps, w, bias, out, epilogue)


# ---- chains of weight-streaming products -------------------------------------------------------
# Every weight-streaming product is an operation of the chain kernel (``csrc/gemm_chain.cu``).  Outside
# ``chain_begin`` / ``chain_end`` each runs at once as a chain of one.  Between them the products are
# not launched one by one: they wait in a list, and the list runs as ONE persistent kernel as soon
# as any other kernel of this module is asked for, so that the order of all kernels is the order of
# the calls.  Only kernels of this module may be launched meanwhile; whoever runs a library operator
# on the stream in between calls ``chain_flush`` first.


class _ChainOpDesc(ctypes.Structure):
    """One product of a chain as ``csrc/gemm_chain.cu`` reads it (``ChainOpDesc``)."""
    _fields_ = [("W", _P), ("X", _P), ("norm_w", _P), ("bias", _P), ("out", _P), ("ldx", _I), ("ldo", _I), ("M", _I),
                ("N", _I), ("K", _I), ("epi", _I), ("norm", _I), ("eps", _F), ("reserved", _I)]


CHAIN_MAX_OPS = 8
_chain_base = 0                           # value of the barrier counter when the next chain kernel begins
_CHAIN_SAFE = {"q25_gemm_chain_bf16", "q25_gemm_chain_scratch_floats", "q25_gemm_chain_available", "q25_gemm_chain_desc_bytes",
               "q25_gemm_chain_grid", "q25_sm_count"}
_chain: Optional[list] = None             # the waiting products: (description, tensors kept alive)
_chain_state: Dict[torch.device, tuple] = {}
_chain_scratch: Dict[torch.device, list] = {}


_chain_ok: Optional[bool] = None


def chain_available() -> bool:
    """Whether the chain kernel can run here: a CUDA device that holds its whole grid at once."""
    global _chain_ok
    if _chain_ok is None:
        if not torch.cuda.is_available():
            return False
        ok = bool(_fn("q25_gemm_chain_available", [])())
        if ok and _fn("q25_gemm_chain_desc_bytes", [])() != ctypes.sizeof(_ChainOpDesc):
            raise KernelError("gemm_chain: the operation description here and in the library differ in layout")
        _chain_ok = ok
    return _chain_ok


def chain_begin() -> bool:
    """Starts gathering.  The counter of the kernels' barrier starts from zero in every gathering
    (a memset on the stream), so the values that a captured graph carries hold in every replay."""
    global _chain, _chain_base
    if _chain is None and chain_available():
        _chain, _chain_base = [], 0
        device = torch.device("cuda", torch.cuda.current_device())
        _chain_buffers(device)[1].zero_()
    return _chain is not None


def _chain_buffers(device: torch.device):
    state = _chain_state.get(device)
    if state is None:
        state = _chain_state[device] = (torch.zeros(65536, dtype=torch.int32, device=device),
                                        torch.zeros(1, dtype=torch.int32, device=device))
    return state


def chain_end() -> None:
    global _chain
    if _chain is not None:
        chain_flush()
        _chain = None


def _chain_add(x, norm_weight, eps, w, bias, out, epilogue) -> None:
    if not chain_available():
        raise KernelError("the weight-streaming kernel needs a device that holds its whole grid at once (one CTA per SM)")
    desc = _ChainOpDesc(W=w.data_ptr(), X=x.data_ptr(), norm_w=_ptr(norm_weight), bias=_ptr(bias), out=out.data_ptr(),
                        ldx=x.stride(0), ldo=out.stride(0), M=x.shape[0], N=w.shape[0], K=w.shape[1], epi=int(epilogue),
                        norm=0 if norm_weight is None else 1, eps=float(eps))
    entry = (desc, (x, norm_weight, w, bias, out))
    if _chain is None:
        _chain_launch([entry])                # nobody is gathering: a chain of one
        return
    _chain.append(entry)
    if len(_chain) == CHAIN_MAX_OPS:
        chain_flush()


def _chain_launch(waiting) -> None:
    global _chain_base
    device = next(t for t in waiting[0][1] if t is not None).device
    ops = (_ChainOpDesc * len(waiting))(*[w_[0] for w_ in waiting])
    need = _fn("q25_gemm_chain_scratch_floats", [_P, _I])
    need.restype = ctypes.c_longlong
    floats = need(ctypes.cast(ops, _P), len(waiting))
    if floats < 0:
        raise KernelError("gemm_chain: a product of the chain cannot be cut")
    held = _chain_scratch.setdefault(device, [])       # never freed or moved: captured graphs keep the addresses
    if not held or held[-1].numel() < max(floats, 1):
        held.append(torch.empty(max(floats, 1), dtype=torch.float32, device=device))
    counters, barrier = _chain_buffers(device)
    _check(_fn("q25_gemm_chain_bf16", [_P, _I, _P, _P, _P, ctypes.c_uint, _P, _P])(
        ctypes.cast(ops, _P), len(waiting), held[-1].data_ptr(), counters.data_ptr(), barrier.data_ptr(),
        _chain_base, error_flag(device).data_ptr(), _stream()), "gemm_chain")
    _chain_base = (_chain_base + (len(waiting) - 1) * chain_grid()) & 0xFFFFFFFF


def chain_flush() -> None:
    """Runs the products that wait, in order, as one kernel."""
    global _chain
    if not _chain:
        return
    waiting, _chain = _chain, None            # the launch below must not gather again
    try:
        _chain_launch(waiting)
    finally:
        _chain = []


def gemm_tcgen05_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Operands the tcgen05 / TMA product takes: bfloat16, K a multiple of 8, 16-byte aligned rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0)


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int) -> None:
    """out = x . w^T on the tcgen05 tensor cores (TMA-fed, accumulators in tensor memory), for
    any number of rows; epilogues as for ``gemm_skinny``."""
    m, k = x.shape
    n = w.shape[0]
    if not gemm_tcgen05_supports(x, w) or w.shape[1] != k:
        raise KernelError(f"gemm_tcgen05: unsupported operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype}")
    _skinny_out(out, m, n, epilogue, "gemm_tcgen05")
    _check(_fn("q25_gemm_tcgen05_bf16", _UNTYPED["q25_gemm_tcgen05_bf16"])(
        w.data_ptr(), x.data_ptr(), x.stride(0), _ptr(bias), out.data_ptr(), out.stride(0), m, n, k, int(epilogue),
        error_flag(x.device).data_ptr(), _stream()), "gemm_tcgen05")


def reset_after_error(device) -> None:
    """After a bounded wait gave up: the error flag, and every flag or counter that kernels leave
    zero when they finish normally, back to zero."""
    device = torch.device(device)
    for table in (_error_flags, _counters):
        if device in table:
            table[device].zero_()
    if device in _chain_state:
        for t in _chain_state[device]:
            t.zero_()


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor], seed: Optional[torch.Tensor],
                token_index: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or temperature is None), else a
    draw from softmax(logits[r] / temperature[r]) keyed by (seed[r], token_index[r])."""
    rows, vocab = logits.shape
    _dev(out, torch.int32, "sample_rows out")
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample_rows: logits must be float32 rows")
    # a large vocabulary is scanned by several blocks per row; their partial winners need scratch
    chunks = _fn("q25_sample_chunks", [_I, _I])(rows, vocab)
    scratch = torch.empty(2 * rows * chunks, dtype=torch.int32, device=logits.device) if chunks > 1 else None
    _check(_fn("q25_sample_rows", _UNTYPED["q25_sample_rows"])(
        logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(seed), _ptr(token_index),
        out.data_ptr(), _ptr(scratch), _stream()), "sample_rows")


def apply_penalties(logits: torch.Tensor, ids: torch.Tensor, counts: torch.Tensor, offsets: torch.Tensor,
                    repetition: torch.Tensor, presence: torch.Tensor, frequency: torch.Tensor) -> None:
    rows, vocab = logits.shape
    _check(_fn("q25_apply_penalties", _UNTYPED["q25_apply_penalties"])(
        logits.data_ptr(), logits.stride(0), rows, vocab, ids.data_ptr(), counts.data_ptr(), offsets.data_ptr(),
        repetition.data_ptr(), presence.data_ptr(), frequency.data_ptr(), _stream()), "apply_penalties")


# ---- a token embedding with learned positions; norms in groups; the clamped gated unit -----------


def embed_position_norm(table: torch.Tensor, pos_table: torch.Tensor, ids: torch.Tensor, positions: torch.Tensor,
                        weight: Optional[torch.Tensor], eps: float, groups: int, x_out: torch.Tensor, scale: float = 1.0) -> None:
    """x_out[n, :] (float32) = norm_in_groups(table[ids[n]] * scale + pos_table[positions[n]]) * weight; without a
    weight there is no norm and the sum starts the stream as it is."""
    n, hidden = x_out.shape
    _dev(ids, torch.int32, "embed_position_norm ids"); _dev(positions, torch.int32, "embed_position_norm positions")
    _dev(x_out, torch.float32, "embed_position_norm out")
    if weight is not None:
        _dev(weight, torch.float32, "embed_position_norm weight")
    if pos_table.dtype != table.dtype or hidden % groups:
        raise KernelError("embed_position_norm: the two tables share a dtype and the groups divide the width")
    _check(_typed("q25_embed_position_norm", table.dtype)(
        table.data_ptr(), pos_table.data_ptr(), ids.data_ptr(), positions.data_ptr(), _ptr(weight), float(eps),
        x_out.data_ptr(), n, hidden, table.shape[0], pos_table.shape[0], int(groups), float(scale), _stream()), "embed_position_norm")


def add_norm_groups(x: torch.Tensor, delta: Optional[torch.Tensor], delta_weight: Optional[torch.Tensor], delta_eps: float,
                    delta_groups: int, weight: Optional[torch.Tensor], eps: float, groups: int,
                    out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = None) -> None:
    """x += d with d = delta, or norm_in_groups(delta) * delta_weight when a weight is given; then
    out = norm_in_groups(x) * weight (out None: only the addition; weight None: out = x as it is, in out's dtype).
    ``rows`` as for ``add_rmsnorm``."""
    hidden = x.shape[-1]
    dtype = out.dtype if out is not None else (delta.dtype if delta is not None else dtype)
    n_out = out.shape[0] if out is not None else (rows.shape[0] if rows is not None else x.shape[0])
    _dev(x, torch.float32, "add_norm_groups x")
    if delta is not None:
        _dev(delta, dtype, "add_norm_groups delta")
    for t in (delta_weight, weight):
        if t is not None:
            _dev(t, torch.float32, "add_norm_groups weight")
    if rows is not None:
        _dev(rows, torch.int32, "add_norm_groups rows")
    _check(_typed("q25_add_norm_groups", dtype)(
        x.data_ptr(), _ptr(delta), _ptr(delta_weight), float(delta_eps), int(delta_groups), _ptr(weight), float(eps), int(groups),
        _ptr(out), _ptr(rows), n_out, hidden, _stream()), "add_norm_groups")


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, paired: bool = False, shift: float = 1.0) -> None:
    """out = g * sigmoid(alpha g) * (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit) (an infinite
    limit, alpha 1 and shift 0: silu(gate) * up);
    ``gate_up`` rows hold the gate features, then the up features, or with ``paired`` groups of 8 gate
    features followed by their 8 up features."""
    n, inter = out.shape
    _dev(gate_up, out.dtype, "glu_clamped input")
    _check(_typed("q25_glu_clamped", out.dtype)(gate_up.data_ptr(), out.data_ptr(), n, inter, float(limit), float(alpha), float(shift), int(paired),
                                                _stream()), "glu_clamped")


# ---- the gated linear recurrence -------------------------------------------------------------------


def rglru_conv(yx: torch.Tensor, x_off: int, conv_w: torch.Tensor, conv_b: torch.Tensor, state: torch.Tensor,
               token_seq: torch.Tensor, cu_q: torch.Tensor, slot_ids: torch.Tensor, u_out: torch.Tensor) -> None:
    """u_out[n, c] (float32) = causal convolution over the request's inputs ``yx[:, x_off + c]``, the
    ``taps - 1`` inputs before the step's first token taken from ``state`` [slots, taps, width]."""
    n, width = u_out.shape
    taps = conv_w.shape[1]
    _dev(u_out, torch.float32, "rglru_conv out"); _dev(state, torch.float32, "rglru_conv state")
    _dev(conv_w, torch.float32, "rglru_conv weight"); _dev(conv_b, torch.float32, "rglru_conv bias")
    if tuple(state.shape[1:]) != (taps, width) or yx.stride(1) != 1:
        raise KernelError(f"rglru_conv: state must be [slots, {taps}, {width}]")
    _check(_typed("q25_rglru_conv", yx.dtype)(yx.data_ptr(), yx.stride(0), int(x_off), conv_w.data_ptr(), conv_b.data_ptr(),
                                              state.data_ptr(), token_seq.data_ptr(), cu_q.data_ptr(), slot_ids.data_ptr(),
                                              u_out.data_ptr(), n, width, taps, _stream()), "rglru_conv")


def rglru_gates(u: torch.Tensor, ra: torch.Tensor, ra_b: torch.Tensor, ri: torch.Tensor, ri_b: torch.Tensor, lam: torch.Tensor,
                gain: float, a_out: torch.Tensor, bx_out: torch.Tensor) -> None:
    """The recurrence's decay a = exp(-gain * sigmoid(Ra u + b) * softplus(lam)) and input term
    sqrt(1 - a^2) * sigmoid(Ri u + b) * u, per block of channels, all float32."""
    n, width = u.shape
    blocks = ra.shape[0]
    for t in (u, ra, ra_b, ri, ri_b, lam, a_out, bx_out):
        _dev(t, torch.float32, "rglru_gates")
    _check(_fn("q25_rglru_gates", [_P, _P, _P, _P, _P, _P, _F, _P, _P, _I, _I, _I, _P])(
        u.data_ptr(), ra.data_ptr(), ra_b.data_ptr(), ri.data_ptr(), ri_b.data_ptr(), lam.data_ptr(), float(gain),
        a_out.data_ptr(), bx_out.data_ptr(), n, width, blocks, _stream()), "rglru_gates")


def rglru_scan(a: torch.Tensor, bx: torch.Tensor, yx: torch.Tensor, y_off: int, x_off: int, state: torch.Tensor,
               cu_q: torch.Tensor, slot_ids: torch.Tensor, out: torch.Tensor, n_seqs: int, max_q_len: int) -> None:
    """S = a S + bx over every entry's tokens from the request's state (row 0 of ``state``), out = S *
    gelu_tanh(yx[:, y_off + c]); the state (S and the last taps - 1 inputs) moves on.  ``max_q_len``:
    the step's longest entry; entries beyond a chunk of tokens are scanned in chunks, in parallel."""
    width = out.shape[1]
    taps = state.shape[1]
    _dev(out, yx.dtype, "rglru_scan out")
    need = _fn("q25_rglru_scan_scratch_floats", [_I, _I, _I])
    need.restype = ctypes.c_longlong
    floats = need(int(n_seqs), int(max_q_len), width)
    sums = torch.empty(floats, dtype=torch.float32, device=out.device) if floats else None
    _check(_typed("q25_rglru_scan", yx.dtype)(a.data_ptr(), bx.data_ptr(), yx.data_ptr(), yx.stride(0), int(y_off), int(x_off),
                                              state.data_ptr(), cu_q.data_ptr(), slot_ids.data_ptr(), out.data_ptr(), int(n_seqs),
                                              int(max_q_len), _ptr(sums), width, taps, _stream()), "rglru_scan")
    if floats:
        count_replayed(1)                      # the chunk summaries' kernel, launched by the same call


# ---- attention with a distance bias, kept first tokens and values of their own size ---------------------


def kv_store_mix(qkv: torch.Tensor, v_other: Optional[torch.Tensor], mix: float, k_pages: torch.Tensor, v_pages: torch.Tensor,
                 kv_slot: torch.Tensor, nq: int, nkv: int, dk: int, dv: int, page_size: int) -> None:
    """Writes the step's keys and values into the pages at ``kv_slot``; with ``v_other`` (rows of
    nkv * dv values of the same tokens) the values become (1 - mix) v + mix v_other first."""
    if v_other is not None and (v_other.dtype != qkv.dtype or v_other.stride(1) != 1 or v_other.shape != (qkv.shape[0], nkv * dv)):
        raise KernelError("kv_store_mix: the other values must be rows of nkv * dv channels of the same tokens")
    _check(_typed("q25_kv_store_mix", qkv.dtype)(
        qkv.data_ptr(), qkv.stride(0), _ptr(v_other), 0 if v_other is None else v_other.stride(0), float(mix), k_pages.data_ptr(),
        v_pages.data_ptr(), kv_slot.data_ptr(), qkv.shape[0], nq, nkv, dk, dv, page_size, _stream()), "kv_store_mix")


def biased_attention_generic(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                             block_table: torch.Tensor, token_seq: torch.Tensor, cu_q: torch.Tensor, q_start_pos: torch.Tensor,
                             nq: int, nkv: int, dk: int, dv: int, page_size: int, window: int, keep_first: int, scale: float,
                             r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], sink: Optional[torch.Tensor] = None,
                             v_row: int = 0, softcap: float = 0.0, dist_bias: Optional[torch.Tensor] = None, gate_off: int = -1) -> None:
    """``sink`` (float32 [nq]): a score per query head that has no key and no value and joins the
    softmax's denominator.  ``v_row``: channels between two value rows of a page when the values lie
    inside the key rows (0: the values have pages of their own, rows of ``dv`` channels).  ``softcap`` c > 0:
    the scaled score becomes ``c * tanh(score / c)`` before anything else is added to it.  ``dist_bias`` (float32
    [rows, nq]): ``dist_bias[min(i - j, rows - 1), head]`` is added to the score.  ``gate_off`` >= 0: the rows of ``qkv``
    hold nq * dv gate channels from that offset on, and the result is multiplied by their sigmoid."""
    if sink is not None:
        _dev(sink, torch.float32, "attention sink")
    _check_dist_bias(dist_bias, nq)
    if dv > 512:
        raise KernelError(f"attention: value size {dv} is beyond 512")
    _check(_typed("q25_biased_attention_generic", qkv.dtype)(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), cu_q.data_ptr(), q_start_pos.data_ptr(), qkv.shape[0], nq, nkv, dk, dv,
        page_size, int(window or 0), int(keep_first or 0), float(scale), _ptr(r1), _ptr(r2), _ptr(sink), int(v_row or 0), float(softcap or 0.0),
        _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], int(gate_off), _stream()), "biased_attention_generic")


def _check_dist_bias(dist_bias: Optional[torch.Tensor], nq: int) -> None:
    if dist_bias is not None:
        _dev(dist_bias, torch.float32, "attention distance table")
        if dist_bias.dim() != 2 or dist_bias.shape[1] != nq or dist_bias.shape[0] < 1 or not dist_bias.is_contiguous():
            raise KernelError(f"attention: the distance table must be [rows, {nq}] float32, got {tuple(dist_bias.shape)}")


# rows of a latent cache the tensor-core kernels are also built for: (rank + rotated channels, rank)
BIASED_LATENT_SIZES = ((48, 32), (80, 64), (96, 64), (160, 128), (192, 128))


def biased_attention_mma_supports(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """Sizes the tensor-core kernels of this attention are built for; the rest goes to the general kernel."""
    return dtype == torch.bfloat16 and ((dk in (32, 64, 128) and dv in (32, 64, 128)) or (dk, dv) in BIASED_LATENT_SIZES)


def biased_attention_mma(qkv: torch.Tensor, out: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                         cu_q: torch.Tensor, q_start_pos: torch.Tensor, tiles: Optional[torch.Tensor], items: Optional[torch.Tensor],
                         nq: int, nkv: int, dk: int, dv: int, page_size: int, window: int, keep_first: int, scale: float,
                         r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], n_splits: int = 1,
                         scratch: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None, v_row: int = 0,
                         softcap: float = 0.0, dist_bias: Optional[torch.Tensor] = None, gate_off: int = -1) -> None:
    """Tensor-core attention (bfloat16): ``tiles`` int32 [n, 2] are (entry, tile of 64 (token, head of
    the group) rows) of the runs, ``items`` the entries that bring one token, whose keys are cut into
    ``n_splits`` ranges (partial results through ``scratch``, float32, len(items) * nq * n_splits * (dv + 2))."""
    n_items = 0 if items is None else items.shape[0]
    n_tiles = 0 if tiles is None else tiles.shape[0]
    _check_dist_bias(dist_bias, nq)
    part_o = part_ml = 0
    if n_items and n_splits > 1:
        need = n_items * nq * n_splits * (dv + 2)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"biased_attention_mma: {n_splits} key ranges need {need} float32 of scratch memory")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * n_items * nq * n_splits * dv
    if not biased_attention_mma_supports(qkv.dtype, dk, dv) or (n_items and nq // nkv > 16):
        raise KernelError(f"biased_attention_mma: unsupported sizes {dk}/{dv} or more than 16 heads per kv head for single tokens")
    _check(_fn("q25_biased_attention_mma_bf16",
               [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P, _I, _I, _P, _P, _F, _P, _I, _I, _P])(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], cu_q.data_ptr(), q_start_pos.data_ptr(), _ptr(tiles), n_tiles, _ptr(items), n_items, nq, nkv, dk, dv,
        page_size, int(window or 0), int(keep_first or 0), float(scale), _ptr(r1), _ptr(r2), _ptr(sink), int(v_row or 0), int(n_splits),
        part_o, part_ml, float(softcap or 0.0), _ptr(dist_bias), 0 if dist_bias is None else dist_bias.shape[0], int(gate_off),
        _stream()), "biased_attention_mma")
    count_replayed((1 if n_tiles and n_items else 0) + (1 if n_items and n_splits > 1 else 0))


# ---- a norm without statistics, a cap on the logits -------------------------------------------------


def add_dyt(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, bias: torch.Tensor, alpha: float,
            out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """x += delta (when given); out = tanh(alpha * x) * weight + bias.  ``rows`` as for ``add_rmsnorm``."""
    hidden = x.shape[-1]
    _dev(x, torch.float32, "add_dyt x"); _dev(weight, torch.float32, "add_dyt weight"); _dev(bias, torch.float32, "add_dyt bias")
    if delta is not None:
        _dev(delta, out.dtype, "add_dyt delta")
    if rows is not None:
        _dev(rows, torch.int32, "add_dyt rows")
    _check(_typed("q25_add_dyt", out.dtype)(x.data_ptr(), _ptr(delta), weight.data_ptr(), bias.data_ptr(), float(alpha),
                                            out.data_ptr(), _ptr(rows), out.shape[0], hidden, _stream()), "add_dyt")


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place (float32)."""
    _dev(logits, torch.float32, "softcap logits")
    _check(_fn("q25_softcap", [_P, _LL, _F, _P])(logits.data_ptr(), logits.numel(), float(cap), _stream()), "softcap")


# ---- rotary positions on one axis, for part of a head, in either pairing -------------------------------

ROTARY_LAYOUTS = {"interleaved": 0, "halves": 1}


def rotary_angles(positions: torch.Tensor, inv_freq: torch.Tensor, magnitude: float) -> torch.Tensor:
    """float32 [N, len(inv_freq), 2]: (cos, sin) of position * frequency, times ``magnitude``."""
    n, half = positions.shape[0], inv_freq.shape[0]
    _dev(positions, torch.int32, "rotary_angles positions"); _dev(inv_freq, torch.float32, "rotary_angles frequencies")
    out = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(_fn("q25_rotary_angles", [_P, _P, _F, _P, _I, _I, _P])(positions.data_ptr(), inv_freq.data_ptr(), float(magnitude),
                                                                 out.data_ptr(), n, half, _stream()), "rotary_angles")
    return out


def rotary_apply(src: torch.Tensor, dst: torch.Tensor, heads: int, width: int, angles: torch.Tensor, layout: str) -> None:
    """For every token and head, ``width`` channels of ``src`` go to ``dst``, the first
    ``2 * angles.shape[1]`` of them rotated.  src and dst are [N, heads, >= width] views (strided; may be the same
    memory) whose channels are contiguous."""
    n = src.shape[0]
    half = angles.shape[1]
    if (src.dtype != dst.dtype or src.dim() != 3 or dst.dim() != 3 or src.shape[1] != heads or dst.shape[1] != heads
            or src.stride(2) != 1 or dst.stride(2) != 1 or dst.shape[0] != n or angles.shape[0] != n or 2 * half > width):
        raise KernelError("rotary_apply: src and dst are [N, heads, width] views of one dtype with contiguous channels")
    _check(_typed("q25_rotary_apply", src.dtype)(
        src.data_ptr(), src.stride(0), src.stride(1), dst.data_ptr(), dst.stride(0), dst.stride(1), n, heads, width, half,
        ROTARY_LAYOUTS[layout], angles.data_ptr(), _stream()), "rotary_apply")


# ---- the latent cache row; retention ----------------------------------------------------------------


def latent_store(x: torch.Tensor, rank: int, rot: int, norm_weight: torch.Tensor, eps: float, angles: Optional[torch.Tensor],
                 layout: str, pages: torch.Tensor, kv_slot: torch.Tensor) -> None:
    """Rows of ``x`` [N, rank + rot] (a strided view) -> cache rows [rank + rot] at ``kv_slot``: the first
    ``rank`` channels RMS-normed with the weight, the last ``rot`` rotated by ``angles``."""
    _dev(norm_weight, torch.float32, "latent_store weight")
    if x.stride(1) != 1 or x.shape[1] != rank + rot or pages.dtype != x.dtype or pages.shape[-1] != rank + rot:
        raise KernelError(f"latent_store: rows and pages must hold {rank} + {rot} channels of one dtype")
    half = 0 if angles is None else angles.shape[1]
    _check(_typed("q25_latent_store", x.dtype)(x.data_ptr(), x.stride(0), rank, rot, norm_weight.data_ptr(), float(eps), _ptr(angles),
                                               half, ROTARY_LAYOUTS[layout], pages.data_ptr(), kv_slot.data_ptr(), x.shape[0],
                                               _stream()), "latent_store")


RETENTION_CHUNK = 64        # tokens of a chunk of a long run; entries up to this many tokens are walked whole


def retention(x: torch.Tensor, q_off: int, k_off: int, v_off: int, g_off: int, angles: Optional[torch.Tensor], layout: str,
              decay: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, slot_ids: torch.Tensor, out: torch.Tensor,
              n_seqs: int, max_q_len: int, heads: int, dim: int, vdim: int, k_scale: float, eps: float,
              chunks: Optional[torch.Tensor] = None, runs: Optional[torch.Tensor] = None, scan_too: bool = True) -> None:
    """Every entry's tokens in order through ``S = decay S + k v^T``, ``o = S^T q`` from the request's
    ``state`` [slots, heads, dim, vdim] (float32), which moves on; out = unit_rms(o) * silu(g) per head.
    ``x`` rows hold the q, k, v and g channels at the given offsets; q and k are rotated by ``angles``.
    ``chunks`` int32 [n, 4] (entry, first token row, tokens, last of its run) and ``runs`` [m, 3] (entry,
    first chunk, chunks): the entries of more than ``RETENTION_CHUNK`` tokens cut into chunks that are
    computed in parallel (two passes and a fold between them); ``scan_too`` False: no other entries."""
    _dev(state, torch.float32, "retention state"); _dev(decay, torch.float32, "retention decay")
    if tuple(state.shape[1:]) != (heads, dim, vdim) or x.stride(1) != 1 or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError(f"retention: state must be [slots, {heads}, {dim}, {vdim}]")
    half = 0 if angles is None else angles.shape[1]
    n_chunks = 0 if chunks is None else chunks.numel() // 4
    n_runs = 0 if runs is None else runs.numel() // 3
    sums = torch.empty(n_chunks * heads * dim * vdim, dtype=torch.float32, device=x.device) if n_chunks else None
    _check(_typed("q25_retention", x.dtype)(
        x.data_ptr(), x.stride(0), q_off, k_off, v_off, g_off, _ptr(angles), half, ROTARY_LAYOUTS[layout], decay.data_ptr(),
        state.data_ptr(), cu_q.data_ptr(), slot_ids.data_ptr(), out.data_ptr(), int(n_seqs), heads, dim, vdim, float(k_scale),
        float(eps), _ptr(chunks), n_chunks, _ptr(runs), n_runs, _ptr(sums), RETENTION_CHUNK, int(scan_too), _stream()), "retention")
    if n_chunks:
        count_replayed(2 + int(scan_too))          # the passes over the chunks, launched by the same call


def plan_retention(q_lens, chunk: int = RETENTION_CHUNK):
    """The chunks of a step's long entries for ``retention``: ``chunks`` (entry, first token row, tokens,
    last of its run), ``runs`` (entry, first chunk, chunks), and whether any entry is left to be walked whole."""
    chunks, runs, row, short = [], [], 0, False
    for entry, n in enumerate(q_lens):
        if n > chunk:
            pieces = -(-n // chunk)
            runs.append((entry, len(chunks), pieces))
            for c in range(pieces):
                chunks.append((entry, row + c * chunk, min(chunk, n - c * chunk), int(c == pieces - 1)))
        else:
            short = True
        row += n
    return chunks, runs, short


# ---- the routed feed-forward ------------------------------------------------------------------------


def moe_max_rows(n_pairs: int, experts: int, tile: int) -> int:
    """Rows the sorted (token, expert) pairs can take: every expert's rows fill whole tiles."""
    return (-(-n_pairs // tile) + experts) * tile


def moe_route(h: torch.Tensor, router: torch.Tensor, shared_gate: Optional[torch.Tensor], top: int, topk_idx: torch.Tensor,
              topk_w: torch.Tensor, sg: Optional[torch.Tensor], counts: torch.Tensor) -> None:
    """Router logits in float32, the ``top`` largest (weights sigmoid(logit)), the shared expert's
    gate sigmoid(shared_gate . h), and how many tokens chose each expert (added into ``counts``)."""
    n, hidden = h.shape
    _dev(router, torch.float32, "moe_route router"); _dev(topk_idx, torch.int32, "moe_route idx")
    _dev(topk_w, torch.float32, "moe_route weights"); _dev(counts, torch.int32, "moe_route counts")
    _check(_typed("q25_moe_route", h.dtype)(h.data_ptr(), router.data_ptr(), _ptr(shared_gate), topk_idx.data_ptr(),
                                            topk_w.data_ptr(), _ptr(sg), counts.data_ptr(), n, hidden, router.shape[0], int(top),
                                            _stream()), "moe_route")


def moe_sort(topk_idx: torch.Tensor, counts: torch.Tensor, cursor: torch.Tensor, plan: torch.Tensor, row_pair: torch.Tensor,
             pair_row: torch.Tensor, experts: int, tile: int) -> None:
    """Lays the pairs out by expert: ``plan`` = [tiles, first row of each expert ..., end, expert of each
    tile ...], ``row_pair`` the pair of every row (-1: empty), ``pair_row`` the row of every pair."""
    n_pairs = topk_idx.numel()
    if plan.numel() < 2 + experts + moe_max_rows(n_pairs, experts, tile) // tile or row_pair.numel() < moe_max_rows(n_pairs, experts, tile):
        raise KernelError("moe_sort: the plan or the row list is too short")
    _check(_fn("q25_moe_sort", [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P])(
        topk_idx.data_ptr(), counts.data_ptr(), cursor.data_ptr(), plan.data_ptr(), row_pair.data_ptr(), pair_row.data_ptr(),
        n_pairs, experts, tile, _stream()), "moe_sort")
    count_replayed(1)                          # two kernels in one call


def moe_gate_up(h: torch.Tensor, w_gate_up: torch.Tensor, act: torch.Tensor, plan: torch.Tensor, row_pair: torch.Tensor,
                topk_w: Optional[torch.Tensor], top: int, limit: float, alpha: float, tile: int, shift: float = 1.0,
                n_pairs: Optional[int] = None) -> None:
    """act[row] = glu(expert of the row's tile applied to weight * h[token of the row]) for the sorted
    rows.  ``w_gate_up``: [experts, 2 * ff, hidden], an expert's gate rows and then its up rows.  Without
    ``topk_w`` the rows go in as they are (``n_pairs`` then says how many pairs the step has); ``shift`` as for
    ``glu_clamped``."""
    n_pairs = topk_w.numel() if n_pairs is None else int(n_pairs)
    experts, ff2, hidden = w_gate_up.shape
    _dev(h, act.dtype, "moe_gate_up input")
    _dev(w_gate_up, h.dtype, "moe_gate_up weights"); _dev(act, h.dtype, "moe_gate_up act")
    # bfloat16: the rows are first written out in the sorted order, weighted, for the tensor-core product
    sorted_rows = torch.empty((act.shape[0], hidden), dtype=h.dtype, device=h.device) if h.dtype == torch.bfloat16 else None
    _check(_typed("q25_moe_gate_up", h.dtype)(h.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), plan.data_ptr(),
                                              row_pair.data_ptr(), _ptr(topk_w), n_pairs, experts, int(top), ff2 // 2, hidden,
                                              float(limit), float(alpha), float(shift), int(tile), _ptr(sorted_rows), _stream()), "moe_gate_up")
    if sorted_rows is not None:
        count_replayed(1)


def moe_gather(h: torch.Tensor, row_pair: torch.Tensor, topk_w: Optional[torch.Tensor], top: int, sorted_rows: torch.Tensor) -> None:
    """sorted_rows[row] = weight of the row's pair * h[token of the pair] (bfloat16), the input of the grouped products."""
    _dev(h, torch.bfloat16, "moe_gather input"); _dev(sorted_rows, torch.bfloat16, "moe_gather rows")
    _check(_fn("q25_moe_gather_bf16", [_P, _P, _P, _P, _I, _I, _I, _P])(
        h.data_ptr(), row_pair.data_ptr(), _ptr(topk_w), sorted_rows.data_ptr(), sorted_rows.shape[0], int(top), h.shape[1],
        _stream()), "moe_gather")


GROUPED_TILE = 128              # rows of a tile of the tcgen05 grouped product


def gemm_tcgen05_grouped_supports(x_dtype: torch.dtype, hidden: int, ff: int) -> bool:
    """What the grouped tcgen05 product takes: bfloat16 rows whose pitch is a multiple of 16 bytes."""
    return x_dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0


def gemm_tcgen05_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, plan: torch.Tensor) -> None:
    """out[row] = x[row] . w[expert of the row's tile]^T on the tcgen05 tensor cores: ``x`` [rows, K] sorted by
    expert in tiles of ``GROUPED_TILE`` rows (rows: the most there can be), ``w`` [experts, N, K], ``plan`` as
    ``moe_sort`` leaves it on the device; ``out`` [rows, N] bfloat16 or float32."""
    rows, k = x.shape
    experts, n, k2 = w.shape
    if (k2 != k or rows % GROUPED_TILE or out.shape != (rows, n) or out.dtype not in (torch.bfloat16, torch.float32)
            or not gemm_tcgen05_supports(x, w.view(experts * n, k))):
        raise KernelError(f"gemm_tcgen05_grouped: unsupported operands {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)}")
    _check(_fn("q25_gemm_tcgen05_grouped_bf16", [_P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _I, _P, _P])(
        w.data_ptr(), x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), rows, n, k, experts, plan.data_ptr(),
        SKINNY_F32 if out.dtype == torch.float32 else SKINNY_STORE, error_flag(x.device).data_ptr(), _stream()), "gemm_tcgen05_grouped")


def moe_down(act: torch.Tensor, w_down: torch.Tensor, y: torch.Tensor, plan: torch.Tensor, row_pair: torch.Tensor, n_pairs: int,
             top: int, tile: int) -> None:
    experts, hidden, ff = w_down.shape
    _dev(w_down, act.dtype, "moe_down weight"); _dev(y, torch.float32, "moe_down out")
    _check(_typed("q25_moe_down", act.dtype)(act.data_ptr(), w_down.data_ptr(), y.data_ptr(), plan.data_ptr(), row_pair.data_ptr(),
                                             int(n_pairs), experts, int(top), hidden, ff, int(tile), _stream()), "moe_down")


def moe_combine(y: torch.Tensor, pair_row: torch.Tensor, sg: Optional[torch.Tensor], shared: Optional[torch.Tensor],
                out: torch.Tensor, top: int) -> None:
    n, hidden = out.shape
    if shared is not None:
        _dev(shared, out.dtype, "moe_combine shared")
    _check(_typed("q25_moe_combine", out.dtype)(y.data_ptr(), pair_row.data_ptr(), _ptr(sg), _ptr(shared), out.data_ptr(), n, hidden,
                                                int(top), _stream()), "moe_combine")


def moe_route_softmax(h: torch.Tensor, router: torch.Tensor, correction: Optional[torch.Tensor], experts: int, top: int, groups: int,
                      keep: int, topk_idx: torch.Tensor, topk_w: torch.Tensor, counts: torch.Tensor, renorm: bool = False,
                      weight_scale: float = 1.0) -> None:
    """Router logits in float32 over all rows of ``router`` (the last ``rows - experts`` stand for experts without
    matrices), scores = softmax; the ``top`` largest of score + correction inside the ``keep`` best of ``groups``
    equal runs of rows are chosen and weigh in with their plain scores (``renorm``: divided by their sum + 1e-20), times
    ``weight_scale``; ``counts`` (one per expert with matrices) takes how many tokens chose each."""
    n, hidden = h.shape
    outputs = router.shape[0]
    _dev(router, torch.float32, "moe_route_softmax router"); _dev(topk_idx, torch.int32, "moe_route_softmax idx")
    _dev(topk_w, torch.float32, "moe_route_softmax weights"); _dev(counts, torch.int32, "moe_route_softmax counts")
    if correction is not None:
        _dev(correction, torch.float32, "moe_route_softmax correction")
    _check(_typed("q25_moe_route_softmax", h.dtype)(h.data_ptr(), router.data_ptr(), _ptr(correction), topk_idx.data_ptr(), topk_w.data_ptr(),
                                                    counts.data_ptr(), n, hidden, int(experts), outputs, int(top), int(groups), int(keep),
                                                    int(bool(renorm)), float(weight_scale), _stream()), "moe_route_softmax")


def moe_combine_weighted(y: torch.Tensor, pair_row: torch.Tensor, topk_w: torch.Tensor, h: torch.Tensor, out: torch.Tensor, top: int,
                         shared: Optional[torch.Tensor] = None) -> None:
    """out[n] = sum over the token's choices of weight * (the row of ``y`` the choice has, or h[n] itself when it has none),
    plus ``shared[n]`` when given (the result of an expert that every token uses)."""
    n, hidden = out.shape
    _dev(y, torch.float32, "moe_combine_weighted rows"); _dev(h, out.dtype, "moe_combine_weighted input")
    if shared is not None:
        _dev(shared, out.dtype, "moe_combine_weighted shared")
        if shared.shape != out.shape or not shared.is_contiguous():
            raise KernelError("moe_combine_weighted: the shared expert's result has the output's shape")
    _check(_typed("q25_moe_combine_weighted", out.dtype)(y.data_ptr(), pair_row.data_ptr(), topk_w.data_ptr(), h.data_ptr(), _ptr(shared),
                                                         out.data_ptr(), n, hidden, int(top), _stream()), "moe_combine_weighted")


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1}


def activation(x: torch.Tensor, out: torch.Tensor, kind: str) -> None:
    """out = act(x) element by element (``out`` may be ``x``): ``relu2`` the square of relu, ``gelu_tanh`` gelu in its
    tanh form."""
    if out.dtype != x.dtype or out.shape != x.shape or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("activation: input and output are contiguous tensors of one shape and dtype")
    _check(_typed("q25_activation", x.dtype)(x.data_ptr(), out.data_ptr(), x.numel(), ACTIVATIONS[kind], _stream()), "activation")


# ---- layer norm around the residual stream, branches into one update, a stream mixed with another ---------


def add_layernorm(x: torch.Tensor, delta: Optional[torch.Tensor], delta_weight: Optional[torch.Tensor], delta_bias: Optional[torch.Tensor],
                  delta_scale: Optional[torch.Tensor], delta_eps: float, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                  eps: float, out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None, dtype: Optional[torch.dtype] = None) -> None:
    """x += post(delta); out = layer_norm(x) * weight + bias.  post(delta) is the layer norm of the update with
    ``delta_weight`` and ``delta_bias``, times ``delta_scale`` per channel when given; without a weight the update
    goes in as it is.  ``out`` None: only the addition.  ``rows`` as for ``add_rmsnorm``."""
    hidden = x.shape[-1]
    dtype = out.dtype if out is not None else (delta.dtype if delta is not None else dtype)
    _dev(x, torch.float32, "add_layernorm x")
    for t in (delta_weight, delta_bias, delta_scale, weight, bias):
        if t is not None:
            _dev(t, torch.float32, "add_layernorm weight")
    if delta is not None:
        _dev(delta, dtype, "add_layernorm delta")
    if rows is not None:
        _dev(rows, torch.int32, "add_layernorm rows")
    n_out = out.shape[0] if out is not None else x.shape[0]
    _check(_typed("q25_add_layernorm", dtype)(x.data_ptr(), _ptr(delta), _ptr(delta_weight), _ptr(delta_bias), _ptr(delta_scale),
                                              float(delta_eps), _ptr(weight), _ptr(bias), float(eps), _ptr(out), _ptr(rows), n_out, hidden,
                                              _stream()), "add_layernorm")


def branch_mean_norm(branches, weights, eps: float, out: torch.Tensor) -> None:
    """out = mean over the branches of branch / rms(branch) * weight (up to 4 branches of out's shape and dtype)."""
    n = len(branches)
    if not 1 <= n <= 4 or len(weights) != n:
        raise KernelError("branch_mean_norm: 1 to 4 branches, each with a weight")
    for b, w in zip(branches, weights):
        _dev(b, out.dtype, "branch_mean_norm branch"); _dev(w, torch.float32, "branch_mean_norm weight")
        if b.shape != out.shape:
            raise KernelError("branch_mean_norm: branches and result have one shape")
    ins = (ctypes.c_void_p * 4)(*[b.data_ptr() for b in branches], *([None] * (4 - n)))
    ws = (ctypes.c_void_p * 4)(*[w.data_ptr() for w in weights], *([None] * (4 - n)))
    _check(_typed("q25_branch_mean_norm", out.dtype)(ctypes.addressof(ins), ctypes.addressof(ws), n, out.data_ptr(), out.shape[0], out.shape[1],
                                                     float(eps), _stream()), "branch_mean_norm")


def stream_pair(x: torch.Tensor, other: torch.Tensor, out: torch.Tensor) -> None:
    """out[n] = [x[n] | other[n]] (two float32 streams side by side) in out's dtype: the input of a product that mixes them."""
    _dev(x, torch.float32, "stream_pair x"); _dev(other, torch.float32, "stream_pair other")
    if out.shape != (x.shape[0], 2 * x.shape[1]) or other.shape != x.shape or not out.is_contiguous():
        raise KernelError("stream_pair: the result holds the two streams side by side")
    _check(_typed("q25_stream_pair", out.dtype)(x.data_ptr(), other.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _stream()), "stream_pair")


def stream_set(x: torch.Tensor, y: torch.Tensor, bias: torch.Tensor) -> None:
    """x = y + bias (float32 rows, a float32 vector), in place of what x held."""
    _dev(x, torch.float32, "stream_set x"); _dev(y, torch.float32, "stream_set y"); _dev(bias, torch.float32, "stream_set bias")
    if y.shape != x.shape:
        raise KernelError("stream_set: shapes differ")
    _check(_fn("q25_stream_set", [_P, _P, _P, _I, _I, _P])(x.data_ptr(), y.data_ptr(), bias.data_ptr(), x.shape[0], x.shape[1], _stream()),
           "stream_set")


# ---- queries and keys normed per head, turned, and cached; keys that serve as values --------------------


def qk_norm_store(qk: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                  angles: Optional[torch.Tensor], layout: str, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                  kv_slot: Optional[torch.Tensor], nq: int, nkv: int, dk: int, page_size: int, keys_as_values: bool,
                  unit_norm: bool = False, positions: Optional[torch.Tensor] = None, temp_coef: float = 0.0, temp_every: int = 0,
                  dv: int = 0) -> None:
    """Rows [nq query heads | nkv key heads] of ``dk`` channels: every head divided by its root mean square and
    multiplied by its weight (dk numbers, shared by the heads; without weights only divided when ``unit_norm``, else
    left alone), then turned by ``angles``; queries are written back, keys go to the pages at ``kv_slot``; with
    ``keys_as_values`` the keys as they came go to the value pages, with ``dv`` > 0 the nkv value heads of ``dv``
    channels that follow the keys in a row.  ``temp_every`` > 0: the queries of a token at position p (``positions``,
    int32 [N]) are multiplied by ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)``."""
    half = 0 if angles is None else angles.shape[1]
    if qk.stride(1) != 1:
        raise KernelError("qk_norm_store: rows must be contiguous")
    if temp_every:
        _dev(positions, torch.int32, "qk_norm_store positions")
    _check(_typed("q25_biased_attention_qk_norm_store", qk.dtype)(
        qk.data_ptr(), qk.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps), int(bool(unit_norm)), _ptr(angles), half,
        ROTARY_LAYOUTS[layout], _ptr(positions) if temp_every else 0, float(temp_coef), int(temp_every or 0), _ptr(k_pages), _ptr(v_pages),
        _ptr(kv_slot), qk.shape[0], int(nq), int(nkv), int(dk), int(dv or 0), int(page_size), int(keys_as_values), _stream()), "qk_norm_store")


# ---- matrix memories with gates that depend on the token -------------------------------------------------


def gla_decay(x: torch.Tensor, low_off: int, rank: int, a2t: torch.Tensor, bias: Optional[torch.Tensor], tau: float, out: torch.Tensor) -> None:
    """out[n, c] (float32) = sigmoid(bias[c] + sum_r a2t[r, c] x[n, low_off + r]) ** (1 / tau)."""
    _dev(a2t, torch.float32, "gla_decay factor"); _dev(out, torch.float32, "gla_decay out")
    if a2t.shape != (rank, out.shape[1]) or x.stride(1) != 1:
        raise KernelError("gla_decay: the second factor comes transposed, [rank, channels]")
    _check(_typed("q25_memory_gla_decay", x.dtype)(x.data_ptr(), x.stride(0), int(low_off), int(rank), a2t.data_ptr(), _ptr(bias), float(tau),
                                                   out.data_ptr(), x.shape[0], out.shape[1], _stream()), "gla_decay")


def row_dots(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """out[n, j] (float32) = bias[j] + w[j] . h[n] for up to 256 float32 rows ``w``, in a fixed order of sums."""
    _dev(h, h.dtype, "row_dots input"); _dev(w, torch.float32, "row_dots rows"); _dev(out, torch.float32, "row_dots out")
    if w.shape[1] != h.shape[1] or out.shape != (h.shape[0], w.shape[0]) or w.shape[0] > 256:
        raise KernelError("row_dots: up to 256 rows of the input's width")
    _check(_typed("q25_memory_row_dots", h.dtype)(h.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), h.shape[0], h.shape[1], w.shape[0],
                                                  _stream()), "row_dots")


def memory_scan(x: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: Optional[torch.Tensor], gates: Optional[torch.Tensor],
                cap: float, q_scale: float, state: torch.Tensor, cu_q: torch.Tensor, slot_ids: torch.Tensor, o_raw: torch.Tensor,
                m_exp: Optional[torch.Tensor], n_seqs: int, heads: int, dim: int, vdim: int) -> None:
    """Every entry's tokens in order through ``S = diag(a) S + b k v^T``, ``o = S^T q`` from the request's state, which
    moves on.  With ``decay`` (float32 [N, heads * dim]) a is that per key channel and b = 1; the state is [slots, heads,
    dim, vdim].  With ``gates`` (float32 [N, 2 * heads]: input gates, then forget gates, before ``cap * tanh(. / cap)``
    and the logarithm of the forget gate's sigmoid) a and b come from the gates and a running maximum m; the state is
    [slots, heads, dim + 1, vdim + 1] (a normaliser column, m in the last row), ``o_raw`` [N, heads, vdim + 1] ends with
    n . q and ``m_exp`` [N, heads] takes exp(-m)."""
    per_head = gates is not None
    extra = 1 if per_head else 0
    _dev(state, torch.float32, "memory_scan state"); _dev(o_raw, torch.float32, "memory_scan out")
    if tuple(state.shape[1:]) != (heads, dim + extra, vdim + extra) or x.stride(1) != 1 or o_raw.numel() != x.shape[0] * heads * (vdim + extra):
        raise KernelError(f"memory_scan: the state must be [slots, {heads}, {dim + extra}, {vdim + extra}]")
    if per_head == (decay is not None):
        raise KernelError("memory_scan: decays per channel or gates per head, one of the two")
    _check(_typed("q25_memory_scan", x.dtype)(
        x.data_ptr(), x.stride(0), int(q_off), int(k_off), int(v_off), _ptr(decay), _ptr(gates), float(cap), float(q_scale), state.data_ptr(),
        cu_q.data_ptr(), slot_ids.data_ptr(), o_raw.data_ptr(), _ptr(m_exp), int(n_seqs), heads, dim, vdim, int(per_head), _stream()),
        "memory_scan")


MEMORY_CHUNK = 64          # tokens of a chunk of a cut run
MEMORY_CUT = 128           # runs of at least this many tokens are cut
MEMORY_FROM_SCRATCH, MEMORY_STATE_NOT_KEPT = 1, 2


def plan_memory(q_lens, chunk: int = MEMORY_CHUNK, cut: int = MEMORY_CUT):
    """The work lists of ``memory_scan_chunked`` for a step whose entries bring ``q_lens`` tokens: ``first`` (a row per
    chunk of a cut run: first token row, end, 0, chunk, 0), ``runs`` (entry, first chunk, chunks) and ``second`` (the
    chunks again, from scratch and without keeping the state, then the entries that are walked whole: first row, end,
    entry, 0, 0).  All empty when no entry is long enough to cut."""
    first, runs, second, whole, row = [], [], [], [], 0
    for entry, n in enumerate(q_lens):
        if n >= cut:
            pieces = -(-n // chunk)
            runs.append((entry, len(first), pieces))
            for c in range(pieces):
                begin, index = row + c * chunk, len(first)
                end = min(begin + chunk, row + n)
                first.append((begin, end, 0, index, 0))
                second.append((begin, end, index, index, MEMORY_FROM_SCRATCH | MEMORY_STATE_NOT_KEPT))
        elif n > 0:
            whole.append((row, row + n, entry, 0, 0))
        row += n
    if not runs:
        return [], [], []
    return first, runs, second + whole


def memory_scan_chunked(x: torch.Tensor, q_off: int, k_off: int, v_off: int, decay: Optional[torch.Tensor], gates: Optional[torch.Tensor],
                        cap: float, q_scale: float, state: torch.Tensor, slot_ids: torch.Tensor, o_raw: torch.Tensor,
                        m_exp: Optional[torch.Tensor], first: torch.Tensor, runs: torch.Tensor, second: torch.Tensor, heads: int, dim: int,
                        vdim: int) -> None:
    """``memory_scan`` for a step with long runs, by the work lists of ``plan_memory`` (flat int32 tensors on the device):
    every chunk's own sum from an empty memory, the sums folded onto the requests' states in order, then every chunk's
    outputs from the state before it, all chunks of a pass in parallel.  Equal to the walk up to rounding."""
    per_head = gates is not None
    extra = 1 if per_head else 0
    _dev(state, torch.float32, "memory_scan_chunked state"); _dev(o_raw, torch.float32, "memory_scan_chunked out")
    for t in (first, runs, second):
        _dev(t, torch.int32, "memory_scan_chunked work list")
    if tuple(state.shape[1:]) != (heads, dim + extra, vdim + extra) or x.stride(1) != 1 or o_raw.numel() != x.shape[0] * heads * (vdim + extra):
        raise KernelError(f"memory_scan_chunked: the state must be [slots, {heads}, {dim + extra}, {vdim + extra}]")
    if per_head == (decay is not None):
        raise KernelError("memory_scan_chunked: decays per channel or gates per head, one of the two")
    n_first = first.numel() // 5
    scratch = torch.empty((n_first, heads, dim + extra, vdim + extra), dtype=torch.float32, device=x.device)
    aux = torch.empty((n_first, heads, 2 if per_head else dim), dtype=torch.float32, device=x.device)
    _check(_typed("q25_memory_scan_chunked", x.dtype)(
        x.data_ptr(), x.stride(0), int(q_off), int(k_off), int(v_off), _ptr(decay), _ptr(gates), float(cap), float(q_scale), state.data_ptr(),
        slot_ids.data_ptr(), o_raw.data_ptr(), _ptr(m_exp), first.data_ptr(), n_first, runs.data_ptr(), runs.numel() // 3, second.data_ptr(),
        second.numel() // 5, scratch.data_ptr(), aux.data_ptr(), heads, dim, vdim, int(per_head), _stream()), "memory_scan_chunked")


MEMORY_GATES = {"silu": 0, "sigmoid": 1}


def memory_output(o_raw: torch.Tensor, m_exp: Optional[torch.Tensor], x: torch.Tensor, g_off: int, weight: torch.Tensor, eps: float,
                  gate: str, out: torch.Tensor, heads: int, vdim: int) -> None:
    """out[n, head] = unit_rms(o / den) * weight * gate(x[n, g_off + head * vdim ...]); den = max(|n . q|, exp(-m)) + 1e-6
    when ``m_exp`` is given (``o_raw`` then has one more column), else 1."""
    extra = 0 if m_exp is None else 1
    _dev(weight, torch.float32, "memory_output weight")
    if weight.numel() != heads * vdim or out.shape != (x.shape[0], heads * vdim) or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError("memory_output: a weight per channel of every head")
    _check(_typed("q25_memory_output", x.dtype)(o_raw.data_ptr(), _ptr(m_exp), x.data_ptr(), x.stride(0), int(g_off), weight.data_ptr(),
                                                out.data_ptr(), x.shape[0], heads, vdim, extra, float(eps), MEMORY_GATES[gate], _stream()),
           "memory_output")
