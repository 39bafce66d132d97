"""Python bindings of the CUDA kernels: one function per exported launcher.

The kernels are plain ``extern "C"`` launchers that take device pointers, sizes and a stream; the
functions here check shapes, dtypes, contiguity and device of the torch tensors they are given,
pass the current torch stream and turn a refusal or launch error into ``KernelError``.  There is
no fallback: without a CUDA device or without the built library every function raises.
"""
from __future__ import annotations

import contextlib
import ctypes
import dataclasses
import threading

import torch

from ..core import KernelError
from . import build as _build

_lib = None
_lock = threading.Lock()
_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float

_CODES = {torch.float32: 0, torch.bfloat16: 1}

_SIGNATURES = {
    "xrt_embedding": [_P, _P, _P, _I, _I, _I, _I, _P, _F, _P],
    "xrt_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _I, _P],
    "xrt_layernorm": [_P, _P, _P, _P, _I, _I, _F, _I, _I, _P],
    "xrt_swiglu": [_P, _P, _I, _I, _I, _I, _I, _P],
    "xrt_rotation_table": [_P, _P, _P, _P, _F, _I, _I, _P],
    "xrt_state_scan": [_P, _P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "xrt_removal_gates": [_P, _I, _P, _P, _I, _P, _P, _I, _P, _I, _I, _I, _I, _F, _F, _P],
    "xrt_rmsnorm_shift": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _F, _I, _I, _I, _P],
    "xrt_add_row": [_P, _P, _I, _I, _I, _P],
    "xrt_act_cast": [_P, _P, _I, _I, _I, _I, _I, _P],
    "xrt_add_scaled_parts": [_P, _P, _P, ctypes.c_longlong, _I, _P],
    "xrt_short_conv": [_P, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "xrt_ssd_scan": [_P, _P, _I, _P, _P, _I, _P, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "xrt_gated_group_norm": [_P, _P, _P, _I, _P, _I, _I, _I, _F, _I, _P],
    "xrt_moe_route": [_P, _P, _P, _P, _I, _I, _I, _P],
    "xrt_moe_experts": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _F, _I, _I, _I, _P],
    "xrt_relu_squared": [_P, _P, _I, _I, _I, _P],
    "xrt_moe_grouped_product": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _F, _I, _P],
    "xrt_moe_group": [_P, _P, _P, _P, _I, _I, _I, _P],
    "xrt_moe_gather": [_P, _P, _P, _I, _I, _I, _P],
    "xrt_moe_activation": [_P, _P, _I, _I, _F, _F, _I, _I, _P],
    "xrt_moe_combine": [_P, _P, _P, _P, _I, _I, _I, _P],
    "xrt_embedding_pair": [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "xrt_layernorm_affine": [_P, _P, _P, _I, ctypes.c_longlong, _P, _P, _P, _I, _I, _F, _I, _P, _P, _P],
    "xrt_qkv_heads_write": [_P, _P, _P, _P, _I, _I, _I, _P, _I, _I, _F, _P, _P, _I, _I, _I, _P, _I, _I,
                            _P, _I, _P, _I, _F, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_rmsnorm_add": [_P, _P, ctypes.c_longlong, _I, _P, _P, _I, _I, _F, _I, _I, _P, _P, _F, _P, _P, _F, _P],
    "xrt_cast_rows": [_P, _P, ctypes.c_longlong, _I, _P],
    "xrt_latent_prepare": [_P, _P, _P, _I, _I, _P, _F, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_head_product": [_P, _I, _I, _I, _P, _I, _I, _I, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_moe_route_scores": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _F, _F, _P],
    "xrt_decay": [_P, _P, _P, _I, _I, _I, _I, _F, _P],
    "xrt_unit_heads": [_P, _I, _I, _I, _I, _F, _I, _F, _P],
    "xrt_head_norm_gate": [_P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _I, _I, _P],
    "xrt_gate_mul": [_P, _P, _I, _I, _I, _I, _I, _I, _P],
    "xrt_rms_scale_add": [_P, _P, _P, _I, _I, _F, _F, _P],
    "xrt_concat_cast": [_P, _P, _P, _I, _I, _I, _P],
    "xrt_scale_softcap": [_P, _I, _I, _F, _F, _P],
    "xrt_rope_table": [_P, _P, _P, _F, _I, _I, _P],
    "xrt_qk_rope_kv_write": [_P, _P, _P, _P, _I, _I, _I, _P, _P, _F, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I,
                             _I, _I, _I, _I, _I, _P],
    "xrt_attention_reference": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _F, _F, _I, _F, _I, _I, _I, _P],
    "xrt_gemm_reference": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_gemm_stream": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "xrt_gemm_stream_norm": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _P],
    "xrt_gemm_stream_normed": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _P, _I, _F, _P],
    "xrt_gemm_tcgen05_normed": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _I, _P, _P, _I, _F, _P],
    "xrt_gemm_decode_tcgen05_normed": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _F, _P],
    "xrt_gemm_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "xrt_gemm_decode_tcgen05": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P],
    "xrt_gemm_decode_tcgen05_norm": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _I, _P, _P],
    "xrt_gemm_decode_tcgen05_norm_parts": [_I, _I, _I, _I],
    "xrt_attention_decode_fused": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _I],
    "xrt_attention_decode": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _I, _P, _P, _P, _I],
    "xrt_attention_decode_qkv": [_P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _I, _F, _P, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I,
                                 _I, _I, _F, _I, _I, _I, _P, _P, _P, _I],
    "xrt_attention_decode_scored": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _F, _F, _I, _F, _I, _I, _P],
    "xrt_attention_prefill": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _F, _F, _I, _F, _P],
    "xrt_attention_prefill_tcgen05": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    "xrt_fill_normal": [_P, ctypes.c_longlong, ctypes.c_ulonglong, ctypes.c_double, ctypes.c_double, _I, _P],
    "xrt_sample": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P, _P, _P],
    "xrt_mark_seen": [_P, _I, _P, _P, _I, _I, _P],
}


def library():
    """The loaded kernel library; builds it first if it is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = _build.build()
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelError(f"cannot load {path}: {exc}") from None
            for name, argtypes in _SIGNATURES.items():
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    raise KernelError(f"{path} does not export {name}") from None
                fn.argtypes = argtypes
                fn.restype = _I
            lib.xrt_attention_decode_fused_max_splits.argtypes = [_I, _I]
            lib.xrt_attention_decode_fused_max_splits.restype = _I
            lib.xrt_gemm_tcgen05_norm_parts.argtypes = [_I]
            lib.xrt_gemm_tcgen05_norm_parts.restype = _I
            lib.xrt_gemm_stream_norm_blocks.argtypes = [_I, _I]
            lib.xrt_gemm_stream_norm_blocks.restype = _I
            lib.xrt_set_tuning.argtypes = [_I, _I]
            lib.xrt_set_tuning.restype = _I
            lib.xrt_gemm_decode_tcgen05_scratch.argtypes = [_I, _I, _I, _I, _I]
            lib.xrt_gemm_decode_tcgen05_scratch.restype = ctypes.c_longlong
            lib.xrt_gemm_decode_tcgen05_plan.argtypes = [_I, _I, _I, _I, _I, ctypes.POINTER(ctypes.c_int)]
            lib.xrt_gemm_decode_tcgen05_plan.restype = _I
            _lib = lib
    return _lib


def _kernels():
    return library()


@dataclasses.dataclass(frozen=True)
class Tuning:
    """Which kernel variant runs where the library has several; the defaults are the measured
    choices.  Set with ``set_tuning`` (process-wide, since the parts call the kernels directly) or
    for a stretch of code with ``tuned(...)``; ``Engine(tuning=...)`` sets it when the engine is made.

    ``graphs``           decode steps are replayed from CUDA graphs
    ``pdl``              kernels of a step are launched with programmatic dependent launch
    ``decode_gemm``      "auto", or "stream" / "tcgen05" to force one of the few-row products
    ``decode_gemm_clusters``  splits of K of the tcgen05 few-row product meet through a cluster
    ``decode_attention`` "auto", "rows" (query heads as MMA rows), "cp" (cp.async tiles), "nocluster"
    ``prefill_attention`` "auto" or "mma" (the mma.sync kernel also where the tcgen05 one applies)
    ``gemm_tile_rows``   0 (auto), 128 or 256: the tile of the prompt product
    ``pending_norm``     "auto": a few-row product that adds into the residual prepares the norm that follows
                         it where the next product runs on the kernel that can finish it; "off": never
                         (a norm kernel runs); "force": wherever the kernels allow, whatever the sizes
    ``decode_cluster_pairs``  decode attention merges a (token, kv head)'s splits as one thread-block
                         cluster up to so many pairs a step; beyond, partials and a second kernel
    """
    graphs: bool = True
    pdl: bool = True
    decode_gemm: str = "auto"
    decode_gemm_clusters: bool = True
    decode_attention: str = "auto"
    prefill_attention: str = "auto"
    gemm_tile_rows: int = 0
    decode_cluster_pairs: int = 128
    pending_norm: str = "auto"


_DECODE_ATTENTION = {"auto": 0, "rows": 1, "cp": 2, "nocluster": 3}
_tuning = Tuning()


def tuning() -> Tuning:
    return _tuning


def set_tuning(new: Tuning) -> None:
    """Makes ``new`` the tuning of every later launch of this process."""
    global _tuning
    if new.decode_gemm not in ("auto", "stream", "tcgen05"):
        raise KernelError(f"tuning: decode_gemm {new.decode_gemm!r} is not auto, stream or tcgen05")
    if new.decode_attention not in _DECODE_ATTENTION:
        raise KernelError(f"tuning: decode_attention {new.decode_attention!r} is not one of {sorted(_DECODE_ATTENTION)}")
    if new.pending_norm not in ("auto", "off", "force"):
        raise KernelError(f"tuning: pending_norm {new.pending_norm!r} is not auto, off or force")
    if new.prefill_attention not in ("auto", "mma"):
        raise KernelError(f"tuning: prefill_attention {new.prefill_attention!r} is not auto or mma")
    lib = library()
    for key, value in ((0, int(new.pdl)), (1, _DECODE_ATTENTION[new.decode_attention]),
                       (2, int(new.gemm_tile_rows)), (3, int(new.decode_gemm_clusters)),
                       (4, int(new.decode_cluster_pairs))):
        if lib.xrt_set_tuning(key, value) != 0:
            raise KernelError(f"tuning: value {value} of setting {key} was refused")
    _tuning = new


@contextlib.contextmanager
def tuned(**changes):
    """``with tuned(prefill_attention="mma"): ...`` runs the body with these settings changed."""
    before = _tuning
    set_tuning(dataclasses.replace(before, **changes))
    try:
        yield
    finally:
        set_tuning(before)


def require_device() -> None:
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: this library runs on the GPU only and has no CPU fallback")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not handled by the kernels (float32, bfloat16)") from None


def _ptr(t, name: str, dtype=None) -> int:
    if t is None:
        return 0
    if not t.is_cuda:
        raise KernelError(f"{name} is not on a CUDA device")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


_launches = 0


def launch_count() -> int:
    """How many kernels of this library were launched so far (a graph replay counts the kernels
    that were captured into it)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status == -1:
        raise KernelError(f"{what}: the kernel refused its arguments")
    if status == -2:
        raise KernelError(f"{what}: sizes or dtypes outside what the kernel handles")
    raise KernelError(f"{what}: CUDA launch error {status}")


def embedding(out, table, ids, error_flag, scale: float = 1.0) -> None:
    """out[t, :] = table[ids[t], :] * scale as float32; raises error_flag[0] on an id outside the table."""
    n, hidden = out.shape
    vocab = table.shape[0]
    if table.shape[1] != hidden or ids.numel() != n:
        raise KernelError("embedding: shapes do not fit")
    _check(_kernels().xrt_embedding(_ptr(out, "out", torch.float32), _ptr(table, "table"),
                                   _ptr(ids, "ids", torch.int32), n, hidden, vocab, _code(table.dtype),
                                   _ptr(error_flag, "error_flag", torch.int32), float(scale), _stream()), "embedding")


def rmsnorm(out, x, weight, eps: float, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r]] if rows is given else x[r]) * weight; x is float32."""
    n_rows, width = out.shape
    if x.shape[1] != width or weight.numel() != width or (rows is None and x.shape[0] != n_rows):
        raise KernelError("rmsnorm: shapes do not fit")
    if rows is not None and rows.numel() != n_rows:
        raise KernelError("rmsnorm: one row index per output row is needed")
    _check(_kernels().xrt_rmsnorm(_ptr(out, "out"), _ptr(x, "x", torch.float32), _ptr(weight, "weight"),
                                 _ptr(rows, "rows", torch.int32), n_rows, width, float(eps),
                                 _code(weight.dtype), _code(out.dtype), _stream()), "rmsnorm")


def layernorm(out, x, weight, eps: float, rows=None) -> None:
    """out[r] = (x[r] - mean) / sqrt(variance + eps) * weight (rows gathered through ``rows`` if given); x is float32."""
    n_rows, width = out.shape
    if x.shape[1] != width or weight.numel() != width or (rows is None and x.shape[0] != n_rows):
        raise KernelError("layernorm: shapes do not fit")
    if rows is not None and rows.numel() != n_rows:
        raise KernelError("layernorm: one row index per output row is needed")
    _check(_kernels().xrt_layernorm(_ptr(out, "out"), _ptr(x, "x", torch.float32), _ptr(weight, "weight"),
                                   _ptr(rows, "rows", torch.int32), n_rows, width, float(eps),
                                   _code(weight.dtype), _code(out.dtype), _stream()), "layernorm")


GATE_ACTS = {"silu": 0, "gelu_tanh": 1}


def _gate_code(act: str, mode: str) -> int:
    """The number of a gated product's activation ("swiglu" mode only: silu, or the tanh form of gelu)."""
    if act not in GATE_ACTS or (act != "silu" and mode != "swiglu"):
        raise KernelError(f"the gate's activation {act!r} is not one of {sorted(GATE_ACTS)}, or the product has no gate")
    return GATE_ACTS[act]


def swiglu(out, gate_up, act: str = "silu") -> None:
    """out[t, f] = act(gate_up[t, f]) * gate_up[t, F + f]; ``act`` "silu" or "gelu_tanh" (the tanh form of gelu)."""
    if act not in GATE_ACTS:
        raise KernelError(f"swiglu: the gate's activation {act!r} is not one of {sorted(GATE_ACTS)}")
    n, width = out.shape
    if gate_up.shape[0] != n or gate_up.shape[1] != 2 * width:
        raise KernelError("swiglu: shapes do not fit")
    _check(_kernels().xrt_swiglu(_ptr(out, "out"), _ptr(gate_up, "gate_up"), n, width, _code(gate_up.dtype),
                                _code(out.dtype), GATE_ACTS[act], _stream()), "swiglu")


def rope_table(cos_sin, positions, freq, scale: float) -> None:
    """cos_sin[t, i] = (cos, sin)(positions[t] * scale / freq[i]); cos_sin is float32 [T, half, 2]."""
    n, half = cos_sin.shape[0], cos_sin.shape[1]
    if positions.numel() != n or freq.numel() != half or cos_sin.shape[2] != 2:
        raise KernelError("rope_table: shapes do not fit")
    _check(_kernels().xrt_rope_table(_ptr(cos_sin, "cos_sin", torch.float32),
                                    _ptr(positions, "positions", torch.int32), _ptr(freq, "freq", torch.float32),
                                    float(scale), n, half, _stream()), "rope_table")


def qk_rope_kv_write(q_out, k_pool, v_pool, qkv, k_offset: int, v_offset: int, q_norm_w, k_norm_w, eps: float,
                     cos_sin, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int, head_dim: int,
                     write_kv: bool = True, pairing: str = "split_half") -> None:
    """Head norms, rotation, q output and cache write in one kernel; see rotary_kv.cu.  ``cos_sin``
    [T, rope_dim / 2, 2] rotates the first rope_dim dims of every head: pairs (i, i + rope_dim / 2)
    with ``pairing`` "split_half", pairs (2i, 2i + 1) with "interleaved"; the rest stays as it is."""
    if pairing not in ("split_half", "interleaved"):
        raise KernelError(f"qk_rope_kv_write: pairing {pairing!r} is not split_half or interleaved")
    n = qkv.shape[0]
    rope_half = 0 if cos_sin is None else cos_sin.shape[1]
    if q_out.shape != (n, n_heads * head_dim) or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("qk_rope_kv_write: shapes do not fit")
    if write_kv:
        for pool in (k_pool, v_pool):
            if pool.dim() != 4 or pool.shape[1] != n_kv_heads or pool.shape[2] != 64 or pool.shape[3] != head_dim:
                raise KernelError("qk_rope_kv_write: the cache pool must be [blocks, kv heads, 64, head_dim]")
        if qkv.shape[1] < v_offset + n_kv_heads * head_dim:
            raise KernelError("qk_rope_kv_write: the q/k/v row is too short")
    norm_dtype = q_norm_w.dtype if q_norm_w is not None else torch.float32
    cache_dtype = k_pool.dtype if write_kv else q_out.dtype
    _check(_kernels().xrt_qk_rope_kv_write(
        _ptr(q_out, "q_out"), _ptr(k_pool if write_kv else None, "k_pool"),
        _ptr(v_pool if write_kv else None, "v_pool"), _ptr(qkv, "qkv", torch.float32), qkv.shape[1], k_offset,
        v_offset, _ptr(q_norm_w, "q_norm_w"), _ptr(k_norm_w, "k_norm_w"), float(eps),
        _ptr(cos_sin, "cos_sin", torch.float32), rope_half, _ptr(tok_slot, "tok_slot", torch.int32),
        _ptr(tok_pos, "tok_pos", torch.int32), _ptr(block_table, "block_table", torch.int32),
        block_table.shape[1], n, n_heads, n_kv_heads, head_dim, 1 if write_kv else 0,
        1 if pairing == "interleaved" else 0, _code(norm_dtype),
        _code(q_out.dtype), _code(cache_dtype), _stream()), "qk_rope_kv_write")


def attention_reference(out, q, k_pool, v_pool, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int,
                        head_dim: int, scale: float, window: int = 0, keep_first: int = 0, softcap: float = 0.0,
                        distance_rate: float = 0.0, sink: float | None = None) -> None:
    """Causal GQA attention over the cache, one warp per (token, head); any dtype.  ``keep_first``: so many first
    keys stay visible behind the window; ``softcap``: s <- cap tanh(s / cap); ``distance_rate`` r: head h's scores
    lose 2^(-r (h + 1) / heads) for every position between query and key (each 0 = off); ``sink`` (None = off): the
    softmax's denominator holds one more term exp(sink) that has no value."""
    n = q.shape[0]
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape:
        raise KernelError("attention_reference: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_reference: the cache pool must be [blocks, kv heads, 64, head_dim]")
    _check(_kernels().xrt_attention_reference(
        _ptr(out, "out"), _ptr(q, "q"), _ptr(k_pool, "k_pool"), _ptr(v_pool, "v_pool", k_pool.dtype),
        _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), int(keep_first), float(softcap), float(distance_rate),
        0 if sink is None else 1, float(sink or 0.0), _code(q.dtype), _code(k_pool.dtype), _code(out.dtype), _stream()),
        "attention_reference")


def gemm_reference(out, x, w, accumulate: bool = False) -> None:
    """out = x . w^T (or out += x . w^T into a float32 out) with 32-bit fused multiply-adds."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError(f"gemm: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: rows must be contiguous")
    if not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm: operands must be on a CUDA device")
    _check(_kernels().xrt_gemm_reference(out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0),
                                        out.stride(0), _code(x.dtype), _code(w.dtype), _code(out.dtype),
                                        1 if accumulate else 0, _stream()), "gemm_reference")


STREAM_MAX_ROWS = 64
_error_flags: dict = {}


def error_flag(device) -> torch.Tensor:
    """The int32 flag of ``device`` that kernels raise when a bounded wait inside them ran out.
    Made when a model is built (never inside a stream capture)."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_flags[key]


def check_error_flag(device) -> None:
    """Reads the flag back (a synchronisation) and raises if a kernel raised it."""
    flag = error_flag(device)
    value = int(flag.item())
    if value != 0:
        flag.zero_()
        key = flag.device.index if flag.device.index is not None else torch.cuda.current_device()
        if key in _counters:  # a block that gave up never brought its tile's counter back to zero
            _counters[key].zero_()
        raise KernelError(f"a kernel reported error {value}: a bounded wait on a copy or a tensor-core operation ran "
                          f"out; results of the last steps are not valid")


DECODE_TCGEN05_MAX_ROWS = 128
_counters: dict = {}
_sm_counts: dict = {}
_COUNTER_SLOTS = 1 << 16


def device_state(device):
    """Per-device state of the kernels, made when a model is built (never inside a stream capture):
    the error flag, the tile counters of the split-K decode product (zero between launches) and
    the number of multiprocessors."""
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _counters:
        _counters[key] = torch.zeros(_COUNTER_SLOTS, dtype=torch.int32, device=device)
        _sm_counts[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return error_flag(device), _counters[key], _sm_counts[key]


_decode_plans: dict = {}


def gemm_decode_tcgen05_fill(sms: int, m: int, n: int, k: int, mode: str):
    """(rounds, share of the multiprocessor-rounds that do work) of ``gemm_decode_tcgen05`` on this
    product on a device of ``sms`` multiprocessors: its items (tiles of 128 weight rows x splits of
    K) run in rounds of one a multiprocessor.  Host arithmetic only: no device is needed."""
    return gemm_decode_tcgen05_plan(sms, m, n, k, mode)[:2]


def gemm_decode_tcgen05_plan(sms: int, m: int, n: int, k: int, mode: str):
    """(rounds, fill, kind of reduction) of ``gemm_decode_tcgen05`` on this product: the kind is "none" (K is not
    split), "cluster" (the splits of a tile meet as a thread-block cluster) or "scratch" (partial sums in
    global memory, merged by the block that brings a tile's last split)."""
    key = (sms, (m + 15) // 16, n, k, mode, tuning().decode_gemm_clusters)
    if key not in _decode_plans:
        plan = (ctypes.c_int * 3)()
        _check(library().xrt_gemm_decode_tcgen05_plan(m, n, k, {"store": 0, "accumulate": 1, "swiglu": 2}[mode], sms, plan),
               "gemm_decode_tcgen05_plan")
        items = plan[0] * plan[1]
        rounds = -(-items // sms)
        kind = "none" if plan[1] == 1 else ("cluster" if plan[2] else "scratch")
        _decode_plans[key] = (rounds, items / (rounds * sms), kind)
    return _decode_plans[key]


_decode_norm_parts: dict = {}


def gemm_decode_tcgen05_norm_parts(m: int, n: int, k: int, device) -> int:
    """How many partial sums of squares a row ``gemm_decode_tcgen05(..., norm=...)`` leaves, or 0 when
    that product cannot prepare a norm on this device (only splits of K that run as clusters do).
    Asks the device once for each class of sizes."""
    sms = device_state(device)[2]
    key = (sms, (m + 15) // 16, n, k, tuning().decode_gemm_clusters)
    if key not in _decode_norm_parts:
        with torch.cuda.device(device):
            _decode_norm_parts[key] = library().xrt_gemm_decode_tcgen05_norm_parts(int(m), int(n), int(k), sms)
    return _decode_norm_parts[key]


def gemm_decode_tcgen05(out, x, w, mode: str = "store", up_rows: int = 0, squares=None, eps: float = 0.0, norm=None,
                        gate_act: str = "silu") -> None:
    """bfloat16 product for at most 128 rows on the tcgen05 tensor cores with swapped operands:
    the weight is streamed once by TMA, K is split across blocks and summed in split order.
    ``squares`` (float32 [parts, rows], from a product with ``norm=...``): ``x`` is a residual times
    its norm weight, and every row's result is multiplied by 1 / sqrt(sum of its parts / K + eps).
    ``norm`` = (scaled, weight, squares) with "accumulate", where ``gemm_decode_tcgen05_norm_parts`` is
    not 0: the product prepares the RMSNorm that follows it, as ``gemm_stream`` does."""
    m, k = x.shape
    n = out.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_decode_tcgen05: operands must be bfloat16")
    rows_needed = n + up_rows if mode == "swiglu" else n
    if w.shape[1] != k or w.shape[0] < rows_needed or out.shape[0] != m or (mode != "swiglu" and w.shape[0] != n):
        raise KernelError(f"gemm_decode_tcgen05: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1 or not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm_decode_tcgen05: rows must be contiguous and on a CUDA device")
    if (n + 127) // 128 > _COUNTER_SLOTS:
        raise KernelError("gemm_decode_tcgen05: more tiles than counters")
    code = {"store": 0, "accumulate": 1, "swiglu": 2}[mode]
    coded = code | (_gate_code(gate_act, mode) << 4)  # the gate's activation rides above the mode's four bits
    flag, counters, sms = device_state(x.device)
    lib = library()
    floats = lib.xrt_gemm_decode_tcgen05_scratch(m, n, k, code, sms)
    partial = torch.empty(floats, dtype=torch.float32, device=x.device) if floats else None
    if squares is not None and (mode == "accumulate" or squares.dim() != 2 or squares.shape[1] != m):
        raise KernelError("gemm_decode_tcgen05: squares must be [parts, rows], and not with accumulate")
    if norm is not None:
        scaled, weight, emitted = norm
        parts = gemm_decode_tcgen05_norm_parts(m, n, k, x.device)
        if (mode != "accumulate" or out.dtype != torch.float32 or parts == 0 or scaled.shape != (m, n) or scaled.stride(1) != 1
                or weight.numel() != n or tuple(emitted.shape) != (parts, m) or not emitted.is_contiguous()):
            raise KernelError("gemm_decode_tcgen05: the buffers of the following norm do not fit the product")
        _check(lib.xrt_gemm_decode_tcgen05_norm(
            out.data_ptr(), x.data_ptr(), _ptr(w, "w"), _ptr(partial, "partial"), counters.data_ptr(), m, n, k, x.stride(0),
            out.stride(0), w.shape[0], sms, flag.data_ptr(), _ptr(scaled, "scaled", torch.bfloat16), scaled.stride(0),
            _ptr(weight, "weight"), _code(weight.dtype), _ptr(emitted, "squares", torch.float32), _stream()),
            "gemm_decode_tcgen05")
        return
    _check(lib.xrt_gemm_decode_tcgen05_normed(
        out.data_ptr(), x.data_ptr(), _ptr(w, "w"), _ptr(partial, "partial"), counters.data_ptr(), m, n, k, x.stride(0),
        out.stride(0), w.shape[0], _code(out.dtype), coded, up_rows, sms, flag.data_ptr(),
        _ptr(squares, "squares", torch.float32), 0 if squares is None else squares.shape[0], float(eps), _stream()),
        "gemm_decode_tcgen05")


def gemm_tcgen05_norm_parts(n: int) -> int:
    """How many partial sums of squares a row ``gemm_tcgen05(..., norm=...)`` leaves (host arithmetic)."""
    return library().xrt_gemm_tcgen05_norm_parts(int(n))


def gemm_tcgen05(out, x, w, mode: str = "store", up_rows: int = 0, norm=None, squares=None, eps: float = 0.0,
                 gate_act: str = "silu") -> None:
    """bfloat16 product for many rows on the tcgen05 tensor cores with TMA-fed operands; modes as
    for ``gemm_stream``.  ``norm`` = (scaled, weight, squares) with "accumulate": the product prepares the
    RMSNorm that follows it (as ``gemm_stream`` does; ``squares`` is float32 [gemm_tcgen05_norm_parts(n), m]).
    ``squares`` (with "store" or "swiglu"): ``x`` is such a prepared input (as for ``gemm_decode_tcgen05``)."""
    m, k = x.shape
    n = out.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05: operands must be bfloat16")
    rows_needed = n + up_rows if mode == "swiglu" else n
    if w.shape[1] != k or w.shape[0] < rows_needed or out.shape[0] != m or (mode != "swiglu" and w.shape[0] != n):
        raise KernelError(f"gemm_tcgen05: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1 or not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm_tcgen05: rows must be contiguous and on a CUDA device")
    code = {"store": 0, "accumulate": 1, "swiglu": 2}[mode]
    coded = code | (_gate_code(gate_act, mode) << 4)  # the gate's activation rides above the mode's four bits
    flag = error_flag(x.device)
    scaled = weight = emitted = None
    if norm is not None:
        scaled, weight, emitted = norm
        if (mode != "accumulate" or scaled.shape != (m, n) or scaled.stride(1) != 1 or weight.numel() != n
                or tuple(emitted.shape) != (gemm_tcgen05_norm_parts(n), m)):
            raise KernelError("gemm_tcgen05: the buffers of the following norm do not fit the product")
    if squares is not None and (mode == "accumulate" or squares.dim() != 2 or squares.shape[1] != m):
        raise KernelError("gemm_tcgen05: squares must be [parts, rows], and not with accumulate")
    _check(_kernels().xrt_gemm_tcgen05_normed(
        out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0), w.shape[0], _code(out.dtype), coded,
        up_rows, flag.data_ptr(), _ptr(scaled, "scaled", torch.bfloat16), 0 if scaled is None else scaled.stride(0),
        _ptr(weight, "weight"), _code(weight.dtype) if weight is not None else 0, _ptr(emitted, "squares", torch.float32),
        _ptr(squares, "squares", torch.float32), 0 if squares is None else squares.shape[0], float(eps), _stream()),
        "gemm_tcgen05")


STREAM_NORM_MAX_ROWS = 16


def gemm_stream_norm_parts(m: int, n: int) -> int:
    """How many partial sums of squares a row ``gemm_stream(..., norm=...)`` leaves (host arithmetic)."""
    parts = library().xrt_gemm_stream_norm_blocks(int(m), int(n))
    if parts <= 0:
        raise KernelError("gemm_stream: a following norm can be prepared for at most 16 rows")
    return parts


def gemm_stream(out, x, w, mode: str = "store", up_rows: int = 0, norm=None, squares=None, eps: float = 0.0,
                gate_act: str = "silu") -> None:
    """bfloat16 product for at most 64 rows that streams the weight once; ``mode`` is "store",
    "accumulate" (into a float32 out) or "swiglu" (out[m, n] = silu(x . w[n]) * (x . w[n + up_rows])).
    ``norm`` = (scaled, weight, squares) with "accumulate" and at most 16 rows: the product also
    prepares the RMSNorm that follows it: ``scaled`` (bfloat16 [m, n]) receives the new residual times
    ``weight`` ([n]), ``squares`` (float32 [gemm_stream_norm_parts(m, n), m]) its sums of squares.
    ``squares`` (float32 [parts, m], with "store" or "swiglu"): ``x`` is such a prepared input, and every
    row's result is multiplied by 1 / sqrt(sum of its parts / k + eps) (as for ``gemm_decode_tcgen05``)."""
    m, k = x.shape
    n = out.shape[1]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_stream: operands must be bfloat16")
    rows_needed = n + up_rows if mode == "swiglu" else n
    if w.shape[1] != k or w.shape[0] < rows_needed or out.shape[0] != m or (mode != "swiglu" and w.shape[0] != n):
        raise KernelError(f"gemm_stream: shapes do not fit: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if x.stride(1) != 1 or out.stride(1) != 1 or not x.is_cuda or not out.is_cuda:
        raise KernelError("gemm_stream: rows must be contiguous and on a CUDA device")
    code = {"store": 0, "accumulate": 1, "swiglu": 2}[mode]
    coded = code | (_gate_code(gate_act, mode) << 4)  # the gate's activation rides above the mode's four bits
    if squares is not None:
        if norm is not None or mode == "accumulate" or squares.dim() != 2 or squares.shape[1] != m or not squares.is_contiguous():
            raise KernelError("gemm_stream: squares must be [parts, rows], and not with accumulate or a following norm")
        _check(_kernels().xrt_gemm_stream_normed(
            out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0), _code(out.dtype), coded, up_rows,
            0, 0, 0, 0, 0, _ptr(squares, "squares", torch.float32), squares.shape[0], float(eps), _stream()), "gemm_stream")
        return
    if norm is None:
        _check(_kernels().xrt_gemm_stream(out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0),
                                         _code(out.dtype), coded, up_rows, _stream()), "gemm_stream")
        return
    scaled, weight, squares = norm
    if (mode != "accumulate" or scaled.shape != (m, n) or scaled.stride(1) != 1 or weight.numel() != n
            or tuple(squares.shape) != (gemm_stream_norm_parts(m, n), m)):
        raise KernelError("gemm_stream: the buffers of the following norm do not fit the product")
    _check(_kernels().xrt_gemm_stream_norm(
        out.data_ptr(), x.data_ptr(), _ptr(w, "w"), m, n, k, x.stride(0), out.stride(0), _code(out.dtype), coded, up_rows,
        _ptr(scaled, "scaled", torch.bfloat16), scaled.stride(0), _ptr(weight, "weight"), _code(weight.dtype),
        _ptr(squares, "squares", torch.float32), _stream()), "gemm_stream")


def attention_decode(out, q, k_pool, v_pool, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int,
                     head_dim: int, scale: float, window: int, chunk: int, n_splits: int, fused: bool = True,
                     clusters: bool = True) -> None:
    """bfloat16 attention of one token a sequence over its cache blocks, split along the keys.
    ``fused``: the splits are merged by the last block of each (token, kv head) instead of by a
    second kernel (needs the device's tile counters; falls back when there are too many).
    ``clusters`` False: the splits never merge as thread-block clusters (for sequences of very unequal
    lengths: a cluster holds its places until its longest block is done)."""
    n = q.shape[0]
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("attention_decode: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_decode: the cache pool must be [blocks, kv heads, 64, head_dim]")
    part_o = part_ml = None
    merged = ctypes.c_int(0)  # set by the launcher when the splits merged themselves as clusters
    flag = error_flag(q.device)
    if n_splits > 1:
        part_o = torch.empty(n * n_heads * n_splits * head_dim, dtype=torch.float32, device=q.device)
        part_ml = torch.empty(n * n_heads * n_splits * 2, dtype=torch.float32, device=q.device)
    if fused and n_splits > 1 and n * n_kv_heads <= _COUNTER_SLOTS:
        _, counters, _ = device_state(q.device)
        _check(_kernels().xrt_attention_decode_fused(
            _ptr(out, "out", torch.bfloat16), _ptr(part_o, "part_o"), _ptr(part_ml, "part_ml"), counters.data_ptr(),
            _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16), _ptr(v_pool, "v_pool", torch.bfloat16),
            k_pool.shape[0], _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
            _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
            float(scale), int(window), int(chunk), int(n_splits), flag.data_ptr(), _stream(), ctypes.byref(merged),
            1 if clusters else 0), "attention_decode")
        if n_splits > 1 and not merged.value and n_splits > attention_decode_fused_max_splits(head_dim, n_heads // n_kv_heads):
            add_launches(1)  # too many splits for the merging block: the combine kernel ran
        return
    _check(_kernels().xrt_attention_decode(
        _ptr(out, "out", torch.bfloat16), _ptr(part_o, "part_o"), _ptr(part_ml, "part_ml"),
        _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16), _ptr(v_pool, "v_pool", torch.bfloat16),
        k_pool.shape[0], _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
        float(scale), int(window), int(chunk), int(n_splits), flag.data_ptr(), _stream(), ctypes.byref(merged),
        1 if clusters else 0), "attention_decode")
    if n_splits > 1 and not merged.value:
        add_launches(1)  # the combine kernel


def attention_decode_takes_qkv(n_heads: int, n_kv_heads: int, head_dim: int, rope_half: int, pairing: str) -> bool:
    """Whether ``attention_decode_qkv`` takes these sizes (the kernel fed by TMA does the step between
    the q/k/v product and attention itself): head size 64, 128 or 256, at most 8 query heads a kv head,
    a split-half rotation over the whole head or none, and no other decode attention kernel forced."""
    return (head_dim in (64, 128, 256) and n_heads // n_kv_heads <= 8 and rope_half in (0, head_dim // 2)
            and (pairing == "split_half" or rope_half == 0) and tuning().decode_attention in ("auto", "nocluster"))


def attention_decode_qkv(out, qkv, k_offset: int, v_offset: int, q_norm_w, k_norm_w, eps: float, cos_sin, k_pool, v_pool,
                         tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                         window: int, chunk: int, n_splits: int, write_kv: bool = True, fused: bool = True,
                         clusters: bool = True) -> None:
    """Decode attention straight from the 32-bit output of the q/k/v product: per-head norms, rotation,
    the newest key and value into the cache (unless ``write_kv`` is False) and attention over the cache
    in ONE kernel (csrc/attention_decode.cu).  ``qkv``: float32 [n, row] with q at 0, k at ``k_offset``,
    v at ``v_offset``.  Check ``attention_decode_takes_qkv`` first; other sizes raise."""
    n = qkv.shape[0]
    if out.shape != (n, n_heads * head_dim) or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("attention_decode_qkv: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_decode_qkv: the cache pool must be [blocks, kv heads, 64, head_dim]")
    if ((write_kv and qkv.shape[1] < v_offset + n_kv_heads * head_dim) or qkv.shape[1] < n_heads * head_dim
            or (cos_sin is not None and cos_sin.shape[1] != head_dim // 2)):
        raise KernelError("attention_decode_qkv: the q/k/v row or the rotation table does not fit the heads")
    part_o = part_ml = None
    merged = ctypes.c_int(0)
    flag, counters, _ = device_state(qkv.device)
    if n_splits > 1:
        part_o = torch.empty(n * n_heads * n_splits * head_dim, dtype=torch.float32, device=qkv.device)
        part_ml = torch.empty(n * n_heads * n_splits * 2, dtype=torch.float32, device=qkv.device)
    use_counters = fused and n_splits > 1 and n * n_kv_heads <= _COUNTER_SLOTS
    norm_dtype = q_norm_w.dtype if q_norm_w is not None else torch.float32
    _check(_kernels().xrt_attention_decode_qkv(
        _ptr(out, "out", torch.bfloat16), _ptr(part_o, "part_o"), _ptr(part_ml, "part_ml"),
        counters.data_ptr() if use_counters else 0, _ptr(qkv, "qkv", torch.float32), qkv.shape[1], int(k_offset),
        int(v_offset), _ptr(q_norm_w, "q_norm_w"), _ptr(k_norm_w, "k_norm_w", norm_dtype), _code(norm_dtype), float(eps),
        _ptr(cos_sin, "cos_sin", torch.float32), 1 if write_kv else 0, _ptr(k_pool, "k_pool", torch.bfloat16),
        _ptr(v_pool, "v_pool", torch.bfloat16), k_pool.shape[0], _ptr(tok_slot, "tok_slot", torch.int32),
        _ptr(tok_pos, "tok_pos", torch.int32), _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n,
        n_heads, n_kv_heads, head_dim, float(scale), int(window), int(chunk), int(n_splits), flag.data_ptr(), _stream(),
        ctypes.byref(merged), 1 if clusters else 0), "attention_decode_qkv")
    if n_splits > 1 and not merged.value and (
            not use_counters or n_splits > attention_decode_fused_max_splits(head_dim, n_heads // n_kv_heads)):
        add_launches(1)  # the combine kernel


def attention_decode_fused_max_splits(head_dim: int, group: int) -> int:
    """The most splits that the last block of a (token, kv head) can merge inside the attention
    kernel (its shared memory holds the splits' maxima and sums); host arithmetic only."""
    n = library().xrt_attention_decode_fused_max_splits(int(head_dim), int(group))
    if n < 0:
        raise KernelError("attention_decode_fused_max_splits: head size or group outside what the kernels take")
    return n


def attention_prefill(out, q, k_pool, v_pool, cu_seqlens, seq_slot, seq_start, block_table, max_new: int,
                      n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int = 0, keep_first: int = 0,
                      softcap: float = 0.0, distance_rate: float = 0.0, sink: float | None = None) -> None:
    """bfloat16 causal attention of sequences laid end to end, each continuing at seq_start.  ``keep_first``,
    ``softcap``, ``distance_rate``: the score options of ``attention_reference``."""
    n = q.shape[0]
    n_seqs = seq_slot.numel()
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or cu_seqlens.numel() != n_seqs + 1:
        raise KernelError("attention_prefill: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_prefill: the cache pool must be [blocks, kv heads, 64, head_dim]")
    _check(_kernels().xrt_attention_prefill(
        _ptr(out, "out", torch.bfloat16), _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16),
        _ptr(v_pool, "v_pool", torch.bfloat16), _ptr(cu_seqlens, "cu_seqlens", torch.int32),
        _ptr(seq_slot, "seq_slot", torch.int32), _ptr(seq_start, "seq_start", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n_seqs, int(max_new), n_heads,
        n_kv_heads, head_dim, float(scale), int(window), int(keep_first), float(softcap), float(distance_rate),
        0 if sink is None else 1, float(sink or 0.0), _stream()), "attention_prefill")


def attention_decode_scored(out, q, k_pool, v_pool, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int,
                            head_dim: int, scale: float, window: int, keep_first: int, softcap: float, distance_rate: float,
                            chunk: int, n_splits: int, sink: float | None = None) -> None:
    """bfloat16 attention of single new tokens with the score options of ``attention_reference``; a token's visible
    keys (kept first keys, then the window) are cut into ``n_splits`` stretches of ``chunk`` keys (a multiple of 32)."""
    n = q.shape[0]
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("attention_decode_scored: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_decode_scored: the cache pool must be [blocks, kv heads, 64, head_dim]")
    partial = None
    if n_splits > 1:
        partial = torch.empty((n, n_heads, n_splits, head_dim + 2), dtype=torch.float32, device=q.device)
        add_launches(1)
    _check(_kernels().xrt_attention_decode_scored(
        _ptr(out, "out", torch.bfloat16), _ptr(partial, "partial"), _ptr(q, "q", torch.bfloat16),
        _ptr(k_pool, "k_pool", torch.bfloat16), _ptr(v_pool, "v_pool", torch.bfloat16),
        _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim, float(scale),
        int(window), int(keep_first), float(softcap), float(distance_rate), 0 if sink is None else 1, float(sink or 0.0),
        int(chunk), int(n_splits), _stream()),
        "attention_decode_scored")


def attention_prefill_tcgen05(out, q, k_pool, v_pool, cu_seqlens, seq_slot, seq_start, block_table, max_new: int,
                              n_heads: int, n_kv_heads: int, head_dim: int, scale: float) -> None:
    """bfloat16 causal attention of sequences laid end to end on the tcgen05 tensor cores (head size 128)."""
    n = q.shape[0]
    n_seqs = seq_slot.numel()
    if q.shape != (n, n_heads * head_dim) or out.shape != q.shape or cu_seqlens.numel() != n_seqs + 1:
        raise KernelError("attention_prefill_tcgen05: shapes do not fit")
    if k_pool.shape != v_pool.shape or k_pool.shape[1:] != (n_kv_heads, 64, head_dim):
        raise KernelError("attention_prefill_tcgen05: the cache pool must be [blocks, kv heads, 64, head_dim]")
    flag = error_flag(q.device)
    _check(_kernels().xrt_attention_prefill_tcgen05(
        _ptr(out, "out", torch.bfloat16), _ptr(q, "q", torch.bfloat16), _ptr(k_pool, "k_pool", torch.bfloat16),
        _ptr(v_pool, "v_pool", torch.bfloat16), _ptr(cu_seqlens, "cu_seqlens", torch.int32),
        _ptr(seq_slot, "seq_slot", torch.int32), _ptr(seq_start, "seq_start", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], k_pool.shape[0], n, n_seqs, int(max_new),
        n_heads, n_kv_heads, head_dim, float(scale), flag.data_ptr(), _stream()), "attention_prefill_tcgen05")


def fill_normal(out, key: int, mean: float, std: float) -> None:
    """Fills ``out`` with the seeded normal stream ``key`` (see weights/random_init.py)."""
    _check(_kernels().xrt_fill_normal(_ptr(out, "out"), out.numel(), key & ((1 << 64) - 1), float(mean),
                                     float(std), _code(out.dtype), _stream()), "fill_normal")


def sample(out_ids, logits, row_slot, temperature, top_k, top_p, penalty, seen, rng_key, rng_counter) -> None:
    """One token id per row of float32 logits; see sampling.cu for the conventions."""
    n, vocab = logits.shape
    seen_words = 0 if seen is None else seen.shape[1]
    _check(_kernels().xrt_sample(
        _ptr(out_ids, "out_ids", torch.int32), _ptr(logits, "logits", torch.float32), n, vocab,
        _ptr(row_slot, "row_slot", torch.int32), _ptr(temperature, "temperature", torch.float32),
        _ptr(top_k, "top_k", torch.int32), _ptr(top_p, "top_p", torch.float32),
        _ptr(penalty, "penalty", torch.float32), _ptr(seen, "seen", torch.int32), seen_words,
        _ptr(rng_key, "rng_key", torch.int64), _ptr(rng_counter, "rng_counter", torch.int32), _stream()), "sample")


def mark_seen(seen, slots, ids, vocab: int) -> None:
    """Sets the bit of ids[i] in the bitmap of slots[i]."""
    n = ids.numel()
    _check(_kernels().xrt_mark_seen(_ptr(seen, "seen", torch.int32), seen.shape[1],
                                   _ptr(slots, "slots", torch.int32), _ptr(ids, "ids", torch.int32), n, vocab,
                                   _stream()), "mark_seen")


# ---------------------------------------------------------------------------------------------------
# Mixers with a matrix state, and the small steps around them (csrc/state_mixers.cu)
_ACTS = {None: 0, "none": 0, "silu": 1, "sigmoid": 2, "tanh": 3}


def _columns(t, name: str, width: int):
    """Pointer and row stride of a float32 tensor [T, >= width] whose rows may be a slice of wider rows."""
    if t.dim() != 2 or t.dtype != torch.float32 or t.stride(1) != 1 or t.shape[1] < width or not t.is_cuda:
        raise KernelError(f"{name} must be float32 rows of at least {width} columns on the device")
    return t.data_ptr(), t.stride(0)


def rotation_table(cos_sin, positions, freq, magnitude: float = 1.0, freq_lo=None) -> None:
    """cos_sin[t, i] = magnitude * (cos, sin)(positions[t] * freq[i]); cos_sin is float32 [T, half, 2].  ``freq_lo``
    (float32 [half]): what ``freq`` lost of its 64-bit value; with it the product's rounding error is carried too, so
    that the angle of a far position is as exact as that of a near one."""
    n, half = cos_sin.shape[0], cos_sin.shape[1]
    if positions.numel() != n or freq.numel() != half or cos_sin.shape[2] != 2:
        raise KernelError("rotation_table: shapes do not fit")
    if freq_lo is not None and freq_lo.numel() != half:
        raise KernelError("rotation_table: freq_lo must have one entry a frequency")
    _check(_kernels().xrt_rotation_table(_ptr(cos_sin, "cos_sin", torch.float32),
                                        _ptr(positions, "positions", torch.int32), _ptr(freq, "freq", torch.float32),
                                        None if freq_lo is None else _ptr(freq_lo, "freq_lo", torch.float32),
                                        float(magnitude), n, half, _stream()), "rotation_table")


def state_scan(out, q, k, v, decay, beta, state, cu_seqlens, seq_slot, n_heads: int, n_qk_heads: int, dim: int,
               vdim: int, q_scale: float = 1.0, delta: bool = False, max_new: int = 0, unit=None, removal=None) -> None:
    """The scan of a matrix state over the step's tokens, a sequence after the other in parallel:
    S <- diag(decay_t) S + k_t u_t^T and out_t = S^T (q_t * q_scale), with u_t = v_t, or with ``delta``
    u_t = sigmoid(beta_t) (v_t - S^T k_t) taken after the decay.  q, k [T, n_qk_heads * dim], v [T, n_heads * vdim],
    decay [T, n_heads * dim] (rows may be slices of wider rows), beta [T, n_heads] before its sigmoid, all
    float32; ``state`` float32 [slots, n_heads, vdim, dim] is read and left as the sequences' last state.
    ``max_new`` (0: not known): the most tokens a sequence brings, from which the kernel sizes its tiles.
    With ``unit`` and ``removal`` (float32 rows of n_heads * dim, n_t and e_t) the state instead loses what it answers
    along n_t: S <- diag(decay_t) S - e_t (n_t^T S) + k_t v_t^T, both corrections from the state as the token found
    it, and out_t = S^T q_t (no ``delta`` then)."""
    if (unit is None) != (removal is None) or (unit is not None and delta):
        raise KernelError("state_scan: unit and removal come together, and without the delta rule")
    n = out.shape[0]
    if out.shape != (n, n_heads * vdim) or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("state_scan: out must be float32 [T, heads * vdim]")
    if state.dim() != 4 or tuple(state.shape[1:]) != (n_heads, vdim, dim) or state.dtype != torch.float32:
        raise KernelError("state_scan: the state must be float32 [slots, heads, vdim, dim]")
    for t in (q, k, v, decay) + ((beta,) if delta else ()):
        if t.shape[0] != n:
            raise KernelError("state_scan: one row a token is needed")
    qp, qs = _columns(q, "q", n_qk_heads * dim)
    kp, ks = _columns(k, "k", n_qk_heads * dim)
    vp, vs = _columns(v, "v", n_heads * vdim)
    dp, ds = _columns(decay, "decay", n_heads * dim)
    bp, bs = _columns(beta, "beta", n_heads) if delta else (0, 0)
    up, us = _columns(unit, "unit", n_heads * dim) if unit is not None else (0, 0)
    rp, rs = _columns(removal, "removal", n_heads * dim) if removal is not None else (0, 0)
    if unit is not None and (unit.shape[0] != n or removal.shape[0] != n):
        raise KernelError("state_scan: one row a token is needed")
    n_seqs = seq_slot.numel()
    if cu_seqlens.numel() != n_seqs + 1:
        raise KernelError("state_scan: cu_seqlens must hold one entry more than seq_slot")
    _check(_kernels().xrt_state_scan(_ptr(out, "out"), qp, qs, kp, ks, vp, vs, dp, ds, bp, bs, up, us, rp, rs, _ptr(state, "state"),
                                    _ptr(cu_seqlens, "cu_seqlens", torch.int32), _ptr(seq_slot, "seq_slot", torch.int32),
                                    n_seqs, n_heads, n_qk_heads, dim, vdim, float(q_scale),
                                    2 if unit is not None else (1 if delta else 0), int(max_new),
                                    _stream()),
           "state_scan")


def short_conv(out, x, weight, state, cu_seqlens, seq_slot, max_new: int, act: str = "silu", bias=None, in_bias=None) -> None:
    """out[t, c] = act(bias[c] + sum_j weight[c, j] * x[t - (taps - 1) + j, c]) inside each sequence (no bias: 0); inputs before the
    step come from ``state`` [slots, taps - 1, channels] (zeros at a sequence's start), which is left holding
    the sequence's last taps - 1 inputs.  x: float32 rows of at least ``channels`` columns; all float32.
    ``in_bias`` (float32 [channels]): every input inside a sequence is x + in_bias (the bias of the product that gave
    x, added here); the state holds such sums, and what stands before a sequence's start stays zero."""
    n, channels = out.shape
    taps = weight.shape[1]
    if weight.shape[0] != channels or x.shape[0] != n or out.dtype != torch.float32:
        raise KernelError("short_conv: shapes do not fit")
    if taps > 1 and (state.dim() != 3 or tuple(state.shape[1:]) != (taps - 1, channels)):
        raise KernelError("short_conv: the state must be [slots, taps - 1, channels]")
    xp, xs = _columns(x, "x", channels)
    n_seqs = seq_slot.numel()
    if any(b is not None and b.numel() != channels for b in (bias, in_bias)):
        raise KernelError("short_conv: one bias a channel is needed")
    _check(_kernels().xrt_short_conv(_ptr(out, "out"), xp, xs, _ptr(weight, "weight", torch.float32),
                                    _ptr(bias, "bias", torch.float32), _ptr(in_bias, "in_bias", torch.float32),
                                    _ptr(state if taps > 1 else None, "state", torch.float32),
                                    _ptr(cu_seqlens, "cu_seqlens", torch.int32), _ptr(seq_slot, "seq_slot", torch.int32),
                                    n_seqs, int(max_new), channels, taps, _ACTS[act], _stream()), "short_conv")
    if taps > 1 and int(max_new) != 1:  # longer portions leave the state in a second launch
        add_launches(1)


def decay_from_gate(a, bias, n_heads: int, dim: int, tau: float) -> None:
    """a <- sigmoid(a + bias)^(1 / tau) in place; a float32 [T, n_heads * dim]."""
    _check(_kernels().xrt_decay(_ptr(a, "a", torch.float32), _ptr(bias, "bias", torch.float32), 0, a.shape[0], n_heads,
                               dim, 0, float(tau), _stream()), "decay_from_gate")


def decay_from_step(a, bias, a_log, n_heads: int, dim: int) -> None:
    """a <- exp(-exp(a_log[head]) * softplus(a + bias)) in place; a float32 [T, n_heads * dim]."""
    if a_log.numel() != n_heads:
        raise KernelError("decay_from_step: one a_log a head is needed")
    _check(_kernels().xrt_decay(_ptr(a, "a", torch.float32), _ptr(bias, "bias", torch.float32),
                               _ptr(a_log, "a_log", torch.float32), a.shape[0], n_heads, dim, 1, 1.0, _stream()),
           "decay_from_step")


def unit_heads(x, n_heads: int, dim: int, eps: float, scaled_heads: int = 0, scale: float = 1.0) -> None:
    """Every head of the first n_heads * dim columns of x (float32 rows) becomes x / sqrt(sum(x^2) + eps), the
    first ``scaled_heads`` of them times ``scale``; in place."""
    xp, xs = _columns(x, "x", n_heads * dim)
    _check(_kernels().xrt_unit_heads(xp, xs, x.shape[0], n_heads, dim, float(eps), int(scaled_heads), float(scale),
                                    _stream()), "unit_heads")


def head_norm_gate(y, o, weight, gate, n_heads: int, vdim: int, eps: float, act: str) -> None:
    """y[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * act(gate[t, h]); o float32 [T, heads * vdim];
    ``weight`` float32 [vdim] (shared by the heads) or [heads * vdim] (one a column of all heads)."""
    n = o.shape[0]
    if y.shape != (n, n_heads * vdim) or o.shape != y.shape or weight.numel() not in (vdim, n_heads * vdim) or gate.shape[0] != n:
        raise KernelError("head_norm_gate: shapes do not fit")
    gp, gs = _columns(gate, "gate", n_heads * vdim)
    _check(_kernels().xrt_head_norm_gate(_ptr(y, "y"), _ptr(o, "o", torch.float32), _ptr(weight, "weight", torch.float32),
                                        gp, gs, n, n_heads, vdim, float(eps), _ACTS[act], _code(y.dtype),
                                        1 if weight.numel() == n_heads * vdim and n_heads > 1 else 0, _stream()),
           "head_norm_gate")


def gate_mul(x, gate, act: str = "sigmoid", group: int = 1) -> None:
    """x[t, c] *= act(gate[t, c // group]) in place; gate: float32 rows of at least x's width / group (``group``
    columns share a gate: a head's, say)."""
    if group < 1 or x.shape[1] % group:
        raise KernelError("gate_mul: the width is no multiple of the group")
    gp, gs = _columns(gate, "gate", x.shape[1] // group)
    if gate.shape[0] != x.shape[0]:
        raise KernelError("gate_mul: shapes do not fit")
    _check(_kernels().xrt_gate_mul(_ptr(x, "x"), gp, gs, x.shape[0], x.shape[1], _ACTS[act], _code(x.dtype), int(group),
                                  _stream()), "gate_mul")


def rms_scale_add(residual, y, weight, eps: float, factor: float = 1.0) -> None:
    """residual += factor * y / sqrt(mean(y^2) + eps) * weight, row by row; all float32."""
    if residual.shape != y.shape or weight.numel() != y.shape[1]:
        raise KernelError("rms_scale_add: shapes do not fit")
    _check(_kernels().xrt_rms_scale_add(_ptr(residual, "residual", torch.float32), _ptr(y, "y", torch.float32),
                                       _ptr(weight, "weight", torch.float32), y.shape[0], y.shape[1], float(eps),
                                       float(factor), _stream()), "rms_scale_add")


def concat_cast(out, a, b) -> None:
    """out[t] = [a[t] | b[t]] in out's dtype; a, b float32 [T, width]."""
    if a.shape != b.shape or out.shape != (a.shape[0], 2 * a.shape[1]):
        raise KernelError("concat_cast: shapes do not fit")
    _check(_kernels().xrt_concat_cast(_ptr(out, "out"), _ptr(a, "a", torch.float32), _ptr(b, "b", torch.float32),
                                     a.shape[0], a.shape[1], _code(out.dtype), _stream()), "concat_cast")


def scale_softcap(x, scale: float, cap: float | None) -> None:
    """x <- cap * tanh(x * scale / cap) in place (x * scale without a cap); x float32 [rows, width]."""
    _check(_kernels().xrt_scale_softcap(_ptr(x, "x", torch.float32), x.shape[0], x.shape[1], float(scale),
                                       float(cap) if cap else 0.0, _stream()), "scale_softcap")


# ---------------------------------------------------------------------------------------------------
# The scalar-decay state-space scan and its group norm (csrc/ssd.cu), routed experts (csrc/moe.cu), and the small
# steps of layers that norm a sublayer's result before adding it
def ssd_scan(out, x, b, c, dt, dt_bias, a_log, d_skip, state, cu_seqlens, seq_slot, n_heads: int, n_groups: int,
             n_state: int, vdim: int, max_new: int = 0) -> None:
    """S <- exp(-exp(a_log) dt) S + dt b x^T, out = S^T c + d_skip x per head, dt = softplus(raw + dt_bias); x rows of
    heads * vdim, b and c rows of groups * n_state (one stride), dt rows of one raw step a head (all float32, rows may
    be slices of wider rows); ``state`` float32 [slots, heads, vdim, n_state] is read and left as the last state."""
    n = out.shape[0]
    if out.shape != (n, n_heads * vdim) or out.dtype != torch.float32 or not out.is_contiguous():
        raise KernelError("ssd_scan: out must be float32 [T, heads * vdim]")
    if state.dim() != 4 or tuple(state.shape[1:]) != (n_heads, vdim, n_state) or state.dtype != torch.float32:
        raise KernelError("ssd_scan: the state must be float32 [slots, heads, vdim, n_state]")
    xp, xs = _columns(x, "x", n_heads * vdim)
    bp, bs = _columns(b, "b", n_groups * n_state)
    cp, cs = _columns(c, "c", n_groups * n_state)
    dp, ds = _columns(dt, "dt", n_heads)
    if bs != cs or any(t.shape[0] != n for t in (x, b, c, dt)):
        raise KernelError("ssd_scan: one row a token, and b and c rows of one stride, are needed")
    for v in (dt_bias, a_log, d_skip):
        if v.numel() != n_heads or v.dtype != torch.float32:
            raise KernelError("ssd_scan: dt_bias, a_log and d_skip are float32 [heads]")
    n_seqs = seq_slot.numel()
    if cu_seqlens.numel() != n_seqs + 1:
        raise KernelError("ssd_scan: cu_seqlens must hold one entry more than seq_slot")
    _check(_kernels().xrt_ssd_scan(_ptr(out, "out"), xp, xs, bp, cp, bs, dp, ds, _ptr(dt_bias, "dt_bias"),
                                  _ptr(a_log, "a_log"), _ptr(d_skip, "d_skip"), _ptr(state, "state"),
                                  _ptr(cu_seqlens, "cu_seqlens", torch.int32), _ptr(seq_slot, "seq_slot", torch.int32),
                                  n_seqs, n_heads, n_groups, n_state, vdim, int(max_new), _stream()), "ssd_scan")


def gated_group_norm(out, y, z, weight, groups: int, eps: float) -> None:
    """out = v / sqrt(mean(v^2 over the group) + eps) * weight with v = y * silu(z), each of ``groups`` equal stretches
    of a row by itself; y float32 [T, width], z float32 rows of at least width, weight float32 [width]."""
    n, width = y.shape
    if out.shape != y.shape or y.dtype != torch.float32 or weight.numel() != width or weight.dtype != torch.float32:
        raise KernelError("gated_group_norm: shapes do not fit")
    zp, zs = _columns(z, "z", width)
    _check(_kernels().xrt_gated_group_norm(_ptr(out, "out"), _ptr(y, "y"), zp, zs, _ptr(weight, "weight"), n, width,
                                          int(groups), float(eps), _code(out.dtype), _stream()), "gated_group_norm")


def moe_route(ids, weights, logits, bias, top: int) -> None:
    """The ``top`` largest of logits + bias a row (ids int32 [T, top]) and the softmax over them (weights float32)."""
    n, experts = logits.shape
    if ids.shape != (n, top) or weights.shape != (n, top) or logits.dtype != torch.float32:
        raise KernelError("moe_route: shapes do not fit")
    _check(_kernels().xrt_moe_route(_ptr(ids, "ids", torch.int32), _ptr(weights, "weights", torch.float32),
                                   _ptr(logits, "logits"), _ptr(bias, "bias", torch.float32), n, experts, int(top),
                                   _stream()), "moe_route")


MOE_ACTS = {"gated_sigmoid": 0, "gelu": 1, "gated_silu": 2}


def _moe_act(act: str) -> int:
    try:
        return MOE_ACTS[act]
    except KeyError:
        raise KernelError(f"experts' activation {act!r} is not one of {sorted(MOE_ACTS)}") from None


def moe_experts(out, h, w_in, w_out, ids, weights, ff: int, limit: float = 0.0, alpha: float = 0.0,
                act: str = "gated_sigmoid") -> None:
    """out[c, t] = weights[t, c] * expert ids[t, c] of h[t]; out float32 [top, T, width]; w_in [experts * 2 * ff,
    width] (an expert's gate rows, then its up rows; with ``act`` "gelu" [experts * ff, width], no gate), w_out
    [experts * width, ff]."""
    top, n, width = out.shape
    blocks = 1 if act == "gelu" else 2
    if h.shape != (n, width) or ids.shape != (n, top) or w_in.shape[1] != width or w_out.shape[1] != ff:
        raise KernelError("moe_experts: shapes do not fit")
    if w_in.shape[0] % (blocks * ff) or w_out.shape[0] != w_in.shape[0] // (blocks * ff) * width or out.dtype != torch.float32:
        raise KernelError("moe_experts: the experts' matrices do not fit")
    hidden = torch.empty((n * top, ff), dtype=torch.float32, device=out.device)  # the hidden units, between the two kernels
    add_launches(1)
    _check(_kernels().xrt_moe_experts(_ptr(out, "out"), _ptr(hidden, "hidden"), _ptr(h, "h"), _ptr(w_in, "w_in"), _ptr(w_out, "w_out", w_in.dtype),
                                     _ptr(ids, "ids", torch.int32), _ptr(weights, "weights", torch.float32), n, width,
                                     int(ff), top, float(limit), float(alpha), _moe_act(act), _code(h.dtype),
                                     _code(w_in.dtype), _stream()), "moe_experts")


def moe_group(offsets, pos, row_token, ids, n_experts: int) -> None:
    """Sorts the (token, choice) pairs of ids [T, top] by expert: offsets int32 [experts + 1] (expert e's rows are
    offsets[e] .. offsets[e + 1]), pos int32 [T * top] the row of every pair, row_token int32 [T * top] the token of
    every row."""
    n, top = ids.shape
    if offsets.numel() != n_experts + 1 or pos.numel() != n * top or row_token.numel() != n * top:
        raise KernelError("moe_group: shapes do not fit")
    _check(_kernels().xrt_moe_group(_ptr(offsets, "offsets", torch.int32), _ptr(pos, "pos", torch.int32),
                                   _ptr(row_token, "row_token", torch.int32), _ptr(ids, "ids", torch.int32), n,
                                   int(n_experts), top, _stream()), "moe_group")


def moe_gather(out, h, row_token) -> None:
    """out[r] = h[row_token[r]]."""
    if out.shape[1] != h.shape[1] or out.dtype != h.dtype or row_token.numel() != out.shape[0]:
        raise KernelError("moe_gather: shapes do not fit")
    _check(_kernels().xrt_moe_gather(_ptr(out, "out"), _ptr(h, "h"), _ptr(row_token, "row_token", torch.int32),
                                    out.shape[0], out.shape[1], _code(h.dtype), _stream()), "moe_gather")


def moe_activation(act, gate_up, limit: float = 0.0, alpha: float = 0.0, kind: str = "gated_sigmoid") -> None:
    """act = g * sigmoid(alpha g) * (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit); gate_up float32
    [rows, 2 * ff] (gate columns, then up columns).  ``kind`` "gelu": act = gelu(gate_up) (exact), gate_up [rows, ff]."""
    rows, ff = act.shape
    if gate_up.shape != (rows, ff if kind == "gelu" else 2 * ff) or gate_up.dtype != torch.float32:
        raise KernelError("moe_activation: shapes do not fit")
    _check(_kernels().xrt_moe_activation(_ptr(act, "act"), _ptr(gate_up, "gate_up"), rows, ff, float(limit), float(alpha),
                                        _moe_act(kind), _code(act.dtype), _stream()), "moe_activation")


def moe_route_scores(ids, weights, logits, top: int, groups: int = 1, keep: int = 1, scores: str = "softmax",
                     correction=None, group_best: int = 1, normalize: bool = False, sum_eps: float = 0.0,
                     scale: float = 1.0) -> None:
    """Routing by scores: softmax of ``logits`` over all experts; of ``groups`` equal groups of neighbouring experts
    only the ``keep`` whose best score is largest may be chosen from; ids int32 [T, top] are the ``top`` largest scores
    among those and weights float32 [T, top] those scores as they are.
    ``scores`` "sigmoid": every score is the sigmoid of its logit.  ``correction`` (float32 [experts]) is added to the
    scores for every choice, of groups and of experts, but not for the weights.  ``group_best``: a group counts by the
    sum of so many of its largest choice scores.  ``normalize``: the weights are divided by their sum + ``sum_eps``;
    ``scale`` multiplies them."""
    n, experts = logits.shape
    if ids.shape != (n, top) or weights.shape != (n, top) or logits.dtype != torch.float32:
        raise KernelError("moe_route_scores: shapes do not fit")
    if scores not in ("softmax", "sigmoid") or (correction is not None and correction.numel() != experts):
        raise KernelError("moe_route_scores: scores are softmax or sigmoid, and a correction has one entry an expert")
    _check(_kernels().xrt_moe_route_scores(_ptr(ids, "ids", torch.int32), _ptr(weights, "weights", torch.float32),
                                          _ptr(logits, "logits"), n, experts, int(top), int(groups), int(keep),
                                          1 if scores == "sigmoid" else 0, _ptr(correction, "correction", torch.float32),
                                          int(group_best), 1 if normalize else 0, float(sum_eps), float(scale), _stream()),
           "moe_route_scores")


def moe_combine(out, y, pos, weights) -> None:
    """out[c, t] = weights[t, c] * y[pos[t * top + c]]; out float32 [top, T, width], y float32 [T * top, width]."""
    top, n, width = out.shape
    if y.shape != (n * top, width) or pos.numel() != n * top or weights.shape != (n, top):
        raise KernelError("moe_combine: shapes do not fit")
    _check(_kernels().xrt_moe_combine(_ptr(out, "out", torch.float32), _ptr(y, "y", torch.float32),
                                     _ptr(pos, "pos", torch.int32), _ptr(weights, "weights", torch.float32), n, width, top,
                                     _stream()), "moe_combine")


def moe_grouped_product(out, a, w, offsets, n_experts: int, ff: int = 0, limit: float = 0.0, alpha: float = 0.0,
                        act: str = "gated_sigmoid") -> None:
    """One launch for all experts' products over rows sorted by expert (bfloat16): with ``ff`` the first product and
    its activation, out bfloat16 [rows, ff] from a [rows, k] and w [experts * 2 * ff, k] (``act`` "gelu": w
    [experts * ff, k], no gate); without, out float32 [rows, n] from a [rows, k] and w [experts * n, k].
    ``offsets`` int32 [experts + 1] on the device."""
    rows, k = a.shape
    first = {"gelu": 2, "gated_silu": 3}.get(act, 1) if ff > 0 else 0
    n = (ff if first == 2 else 2 * ff) if first else out.shape[1]
    _moe_act(act)
    if w.shape != (n_experts * n, k) or out.shape != (rows, ff if first else n) or offsets.numel() != n_experts + 1:
        raise KernelError("moe_grouped_product: shapes do not fit")
    _check(_kernels().xrt_moe_grouped_product(_ptr(out, "out", torch.bfloat16 if first else torch.float32),
                                             _ptr(a, "a", torch.bfloat16), _ptr(w, "w", torch.bfloat16),
                                             _ptr(offsets, "offsets", torch.int32), rows, int(n_experts), n, k, int(ff),
                                             float(limit), float(alpha), first, _stream()),
           "moe_grouped_product")


def relu_squared(out, x) -> None:
    """out = max(x, 0)^2; x float32 [T, width]."""
    if out.shape != x.shape or x.dtype != torch.float32:
        raise KernelError("relu_squared: shapes do not fit")
    _check(_kernels().xrt_relu_squared(_ptr(out, "out"), _ptr(x, "x"), x.shape[0], x.shape[1], _code(out.dtype),
                                      _stream()), "relu_squared")


def embedding_pair(out, table, pairs, ids, tok_slot, tok_pos, last_token, cu_seqlens, seq_slot, mul_prev: int,
                   mul_cur: int, error_flag) -> None:
    """out[t] = table[id] + pairs[(previous * mul_prev + id * mul_cur) mod buckets] (pairs' last row at position 0);
    ``last_token`` int32 [slots] gives a step's first tokens their previous token and is left holding the last."""
    n, hidden = out.shape
    buckets = pairs.shape[0] - 1
    if table.shape[1] != hidden or pairs.shape[1] != hidden or ids.numel() != n or pairs.dtype != table.dtype or buckets < 1:
        raise KernelError("embedding_pair: shapes do not fit")
    n_seqs = seq_slot.numel()
    _check(_kernels().xrt_embedding_pair(_ptr(out, "out", torch.float32), _ptr(table, "table"), _ptr(pairs, "pairs"),
                                        _ptr(ids, "ids", torch.int32), _ptr(tok_slot, "tok_slot", torch.int32),
                                        _ptr(tok_pos, "tok_pos", torch.int32), _ptr(last_token, "last_token", torch.int32),
                                        _ptr(cu_seqlens, "cu_seqlens", torch.int32),
                                        _ptr(seq_slot, "seq_slot", torch.int32), n, n_seqs, hidden, table.shape[0], buckets,
                                        int(mul_prev), int(mul_cur), _code(table.dtype),
                                        _ptr(error_flag, "error_flag", torch.int32), _stream()), "embedding_pair")
    add_launches(1)


def layernorm_affine(x, weight, bias, eps: float, out=None, residual=None, rows=None, n_parts: int = 1, then=None) -> None:
    """y = (x - mean) / sqrt(variance + eps) * weight + bias over float32 rows; written to ``out`` (any dtype), or
    added into ``residual`` (float32) when that is given.  With ``residual``, ``out`` and ``then`` = (weight2, bias2)
    the new residual rows are normed once more, with those, into ``out`` (the norm the next sublayer begins with).
    ``x`` may be [n_parts, T, width]: the parts are added in index order first.  ``rows`` gathers rows of x."""
    width = x.shape[-1]
    target = residual if residual is not None else out
    both = out is not None and residual is not None
    if target is None or target.shape[-1] != width or x.dtype != torch.float32 or both != (then is not None):
        raise KernelError("layernorm_affine: give out or residual of x's width, or both with the second norm")
    if both and (out.shape != residual.shape or rows is not None or then[0].numel() != width):
        raise KernelError("layernorm_affine: the second norm needs rows of the residual's shape")
    if x.dim() != (3 if n_parts > 1 else 2) or (n_parts > 1 and x.shape[0] != n_parts) or not x.is_contiguous():
        raise KernelError("layernorm_affine: x must be [T, width] or [parts, T, width]")
    n_rows = target.shape[0]
    if rows is not None and rows.numel() != n_rows or rows is None and x.shape[-2] != n_rows:
        raise KernelError("layernorm_affine: rows do not fit")
    if weight.numel() != width or (bias is not None and bias.numel() != width):
        raise KernelError("layernorm_affine: weight and bias must be [width]")
    _check(_kernels().xrt_layernorm_affine(_ptr(out, "out"), _ptr(residual, "residual", torch.float32), _ptr(x, "x"),
                                          int(n_parts), x.shape[-2] * width if n_parts > 1 else 0,
                                          _ptr(weight, "weight", torch.float32), _ptr(bias, "bias", torch.float32),
                                          _ptr(rows, "rows", torch.int32), n_rows, width, float(eps),
                                          _code(out.dtype) if out is not None else 0,
                                          _ptr(then[0] if then else None, "weight2", torch.float32),
                                          _ptr(then[1] if then else None, "bias2", torch.float32), _stream()),
           "layernorm_affine")


def qkv_heads_write(q_out, k_pool, v_pool, qkv, k_offset: int, v_offset: int, bias, unit_norm: bool, norm_dim: int,
                    eps: float, tok_slot, tok_pos, block_table, n_heads: int, n_kv_heads: int, head_dim: int,
                    v_keep=None, v_first=None, v_blend: float = 0.0, v_dim: int = 0, write_kv: bool = True,
                    q_norm_w=None, k_norm_w=None, whole_q: int = 0, whole_k: int = 0, cos_sin=None,
                    pairing: str = "split_half", v_unit: bool = False) -> None:
    """``qk_rope_kv_write`` without rotation for layers that add a bias a column of the q/k/v row (float32, laid out as
    the row), divide q and k heads by their root mean square without a weight (over ``norm_dim`` dims where the heads
    are laid out wider), keep the values in 32-bit (``v_keep`` [T, kv heads * v_dim]) and / or cache
    (1 - v_blend) v + v_blend v_first; ``v_dim`` (0: head_dim) is a head's true value size, at which v_keep and
    v_first hold the heads.  ``q_norm_w`` / ``k_norm_w`` with ``whole_q`` / ``whole_k`` > 0: an RMSNorm over the
    whole q (k) projection of a token, all heads at once, one weight a column of the projection as it is laid out, the
    number being the divisor of the mean of squares; ``cos_sin`` and ``pairing`` as in ``qk_rope_kv_write``.
    ``v_unit``: every value head is divided by its root mean square over ``v_dim`` (``eps``, no weight) first."""
    n = qkv.shape[0]
    if pairing not in ("split_half", "interleaved"):
        raise KernelError(f"qkv_heads_write: pairing {pairing!r} is not split_half or interleaved")
    if q_norm_w is not None and q_norm_w.numel() != (n_heads * head_dim if whole_q else head_dim):
        raise KernelError("qkv_heads_write: the q norm's weight does not fit")
    if k_norm_w is not None and k_norm_w.numel() != (n_kv_heads * head_dim if whole_k else head_dim):
        raise KernelError("qkv_heads_write: the k norm's weight does not fit")
    if q_norm_w is not None and k_norm_w is not None and q_norm_w.dtype != k_norm_w.dtype:
        raise KernelError("qkv_heads_write: the norm weights must share a dtype")
    rope_half = 0 if cos_sin is None else cos_sin.shape[1]
    norm_dtype = q_norm_w.dtype if q_norm_w is not None else torch.float32
    if q_out.shape != (n, n_heads * head_dim) or tok_slot.numel() != n or tok_pos.numel() != n:
        raise KernelError("qkv_heads_write: shapes do not fit")
    if write_kv:
        for pool in (k_pool, v_pool):
            if pool.dim() != 4 or pool.shape[1] != n_kv_heads or pool.shape[2] != 64 or pool.shape[3] != head_dim:
                raise KernelError("qkv_heads_write: the cache pool must be [blocks, kv heads, 64, head_dim]")
        if qkv.shape[1] < v_offset + n_kv_heads * head_dim:
            raise KernelError("qkv_heads_write: the q/k/v row is too short")
    if bias is not None and bias.numel() < v_offset + n_kv_heads * head_dim:
        raise KernelError("qkv_heads_write: the bias is shorter than the q/k/v row")
    true_v = int(v_dim) if v_dim else head_dim
    if not 0 < true_v <= head_dim:
        raise KernelError("qkv_heads_write: v_dim must lie in 1 .. head_dim")
    for t in (v_keep, v_first):
        if t is not None and t.shape[0] != n:
            raise KernelError("qkv_heads_write: one row of kept values a token is needed")
    kp, ks = _columns(v_keep, "v_keep", n_kv_heads * true_v) if v_keep is not None else (0, 0)
    fp, fs = _columns(v_first, "v_first", n_kv_heads * true_v) if v_first is not None else (0, 0)
    cache_dtype = k_pool.dtype if write_kv else q_out.dtype
    _check(_kernels().xrt_qkv_heads_write(
        _ptr(q_out, "q_out"), _ptr(k_pool if write_kv else None, "k_pool"), _ptr(v_pool if write_kv else None, "v_pool"),
        _ptr(qkv, "qkv", torch.float32), qkv.shape[1], k_offset, v_offset, _ptr(bias, "bias", torch.float32),
        1 if unit_norm else 0, int(norm_dim), float(eps), _ptr(q_norm_w, "q_norm_w"), _ptr(k_norm_w, "k_norm_w"),
        _code(norm_dtype), int(whole_q), int(whole_k), _ptr(cos_sin, "cos_sin", torch.float32), rope_half,
        1 if pairing == "interleaved" else 0, kp, ks, fp, fs, float(v_blend), true_v, 1 if v_unit else 0,
        _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, n_kv_heads, head_dim,
        1 if write_kv else 0, _code(q_out.dtype), _code(cache_dtype), _stream()), "qkv_heads_write")


def rmsnorm_add(residual, y, weight, eps: float, copy=None, factor: float = 1.0, part_scales=None, bias=None,
                then=None) -> None:
    """residual += factor * RMSNorm(y) * weight, 32-bit; ``y`` float32 [T, width] or [parts, T, width] (added in index
    order first, part p times ``part_scales[p]`` (float32 on the device) where given, plus the row ``bias`` (float32
    [width])); ``copy`` (optional, [T, width] in the compute dtype) receives the new residual as well; ``then`` =
    (weight2, eps2, out2): out2 [T, width] receives RMSNorm(new residual) * weight2 (weight2 of ``weight``'s dtype)."""
    n, width = residual.shape
    parts = y.shape[0] if y.dim() == 3 else 1
    if tuple(y.shape[-2:]) != (n, width) or weight.numel() != width or residual.dtype != torch.float32:
        raise KernelError("rmsnorm_add: shapes do not fit")
    if copy is not None and tuple(copy.shape) != (n, width):
        raise KernelError("rmsnorm_add: the copy does not fit")
    if part_scales is not None and part_scales.numel() != parts or bias is not None and bias.numel() != width:
        raise KernelError("rmsnorm_add: one scale a part and one bias a column are needed")
    then_w = then_out = None
    then_eps = 0.0
    if then is not None:
        then_w, then_eps, then_out = then
        if (tuple(then_out.shape) != (n, width) or then_w.numel() != width or then_w.dtype != weight.dtype
                or (copy is not None and copy.dtype != then_out.dtype)):
            raise KernelError("rmsnorm_add: the second norm does not fit")
    side = copy if copy is not None else then_out
    _check(_kernels().xrt_rmsnorm_add(_ptr(residual, "residual"), _ptr(y, "y", torch.float32), n * width, parts,
                                     _ptr(weight, "weight"), _ptr(copy, "copy"), n, width, float(eps), _code(weight.dtype),
                                     _code(side.dtype if side is not None else torch.float32),
                                     _ptr(part_scales, "part_scales", torch.float32), _ptr(bias, "bias", torch.float32),
                                     float(factor), _ptr(then_w, "then weight"), _ptr(then_out, "then out"),
                                     float(then_eps), _stream()), "rmsnorm_add")


def cast_rows(out, x) -> None:
    """out = x (float32) in out's dtype."""
    if out.shape != x.shape:
        raise KernelError("cast_rows: shapes do not fit")
    _check(_kernels().xrt_cast_rows(_ptr(out, "out"), _ptr(x, "x", torch.float32), x.numel(), _code(out.dtype), _stream()),
           "cast_rows")


def latent_prepare(q_rows, pool, qd, down_offset: int, norm_w, eps: float, cos_sin, tok_slot, tok_pos, block_table,
                   n_heads: int, dim: int, rot: int, rank: int, head_size: int, write_cache: bool = True,
                   pairing: str = "interleaved", first_head: int = 0) -> None:
    """What latent attention does between its first product and attention (csrc/latent.cu): from qd float32
    [T, heads * (dim + rot) ... | rank + rot at down_offset] the cache row [normed latent | rotated shared key part |
    zeros] into ``pool`` [blocks, 1, 64, head_size], and every head's rotated query part (and zeros behind it) into
    columns rank .. head_size of its ``q_rows`` [T, heads * head_size] row.  ``first_head``: the ``n_heads`` heads of
    ``q_rows`` are the heads first_head .. first_head + n_heads - 1 of qd (a part of the heads at a time)."""
    n = qd.shape[0]
    shift = int(first_head) * (dim + rot)
    if (q_rows.shape != (n, n_heads * head_size) or first_head < 0
            or qd.shape[1] < max(shift + n_heads * (dim + rot), down_offset + rank + rot)):
        raise KernelError("latent_prepare: shapes do not fit")
    if write_cache and tuple(pool.shape[1:]) != (1, 64, head_size):
        raise KernelError("latent_prepare: the cache pool must be [blocks, 1, 64, head_size]")
    if norm_w.numel() != rank or (rot and (cos_sin is None or tuple(cos_sin.shape) != (n, rot // 2, 2))):
        raise KernelError("latent_prepare: the norm weight or the rotation table does not fit")
    cache_dtype = pool.dtype if write_cache else q_rows.dtype
    _check(_kernels().xrt_latent_prepare(
        _ptr(q_rows, "q_rows"), _ptr(pool if write_cache else None, "pool"),
        _ptr(qd, "qd", torch.float32) + shift * qd.element_size(), qd.shape[1],
        int(down_offset) - shift, _ptr(norm_w, "norm_w"), float(eps), _ptr(cos_sin, "cos_sin", torch.float32),
        _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
        _ptr(block_table, "block_table", torch.int32), block_table.shape[1], n, n_heads, int(dim), int(rot), int(rank),
        int(head_size), 1 if write_cache else 0, 1 if pairing == "interleaved" else 0, _code(norm_w.dtype),
        _code(q_rows.dtype), _code(cache_dtype), _stream()), "latent_prepare")


def head_product(out, out_head: int, out_off: int, x, x_head: int, x_off: int, w, n_heads: int) -> None:
    """out[t, head * out_head + out_off + n] = sum_k x[t, head * x_head + x_off + k] * w[head, n, k]; w [heads, n, k];
    x and out are rows of any width that hold the heads' pieces at those places.  32-bit sums; a float32 x under a
    bfloat16 w is rounded to bfloat16 first."""
    heads, n, k = w.shape
    t = x.shape[0]
    if heads != n_heads or out.shape[0] != t or x.dim() != 2 or out.dim() != 2 or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("head_product: shapes do not fit")
    if (n_heads - 1) * x_head + x_off + k > x.shape[1] or (n_heads - 1) * out_head + out_off + n > out.shape[1]:
        raise KernelError("head_product: a head's piece lies outside its row")
    _check(_kernels().xrt_head_product(_ptr(out, "out"), out.stride(0), int(out_head), int(out_off), _ptr(x, "x"),
                                      x.stride(0), int(x_head), int(x_off), _ptr(w, "w"), t, n_heads, n, k,
                                      _code(x.dtype), _code(w.dtype), _code(out.dtype), _stream()), "head_product")


# ---------------------------------------------------------------------------------------------------
# Token shift, the row that a pass over a stretch of layers begins with, and the gates of the scan's removal form
def rmsnorm_shift(out, x, weight, shift, state, ctx_arrays, eps: float, single_tokens: bool) -> None:
    """out[t] = n_t + (n_(t-1) - n_t) * shift with n = RMSNorm(x) * weight in 32-bit (csrc/token_shift.cu); n_(t-1) is
    zero at a sequence's start and comes from ``state`` float32 [slots, width] for a step's first token, and the state
    is left holding the n of each sequence's last token.  ``ctx_arrays`` = (tok_slot, tok_pos, cu_seqlens, seq_slot).
    ``single_tokens``: every sequence of the step brings one token (one launch instead of two)."""
    n, width = x.shape
    tok_slot, tok_pos, cu_seqlens, seq_slot = ctx_arrays
    if (out.shape != x.shape or x.dtype != torch.float32 or weight.numel() != width or shift.numel() != width
            or state.dim() != 2 or state.shape[1] != width or tok_slot.numel() != n or tok_pos.numel() != n
            or cu_seqlens.numel() != seq_slot.numel() + 1 or not x.is_contiguous() or not state.is_contiguous()):
        raise KernelError("rmsnorm_shift: shapes do not fit")
    _check(_kernels().xrt_rmsnorm_shift(_ptr(out, "out"), _ptr(x, "x"), _ptr(weight, "weight"),
                                       _ptr(shift, "shift", torch.float32), _ptr(state, "state", torch.float32),
                                       _ptr(tok_slot, "tok_slot", torch.int32), _ptr(tok_pos, "tok_pos", torch.int32),
                                       _ptr(cu_seqlens, "cu_seqlens", torch.int32), _ptr(seq_slot, "seq_slot", torch.int32),
                                       seq_slot.numel(), n, width, float(eps), 1 if single_tokens else 0,
                                       _code(weight.dtype), _code(out.dtype), _stream()), "rmsnorm_shift")
    if not single_tokens:
        add_launches(1)


def add_row(x, row) -> None:
    """x[t] += row in place; x float32 [T, width], row [width]."""
    if x.dim() != 2 or x.dtype != torch.float32 or row.numel() != x.shape[1] or not x.is_contiguous():
        raise KernelError("add_row: shapes do not fit")
    _check(_kernels().xrt_add_row(_ptr(x, "x"), _ptr(row, "row"), x.shape[0], x.shape[1], _code(row.dtype), _stream()),
           "add_row")


def removal_gates(decay, decay_bias, removal, removal_bias, unit, k, n_heads: int, dim: int, rate: float,
                  unit_eps: float) -> None:
    """From raw products, per head of ``dim`` channels: decay <- exp(-rate * sigmoid(decay + decay_bias)) in place;
    unit = k / sqrt(sum(k^2) + unit_eps); removal <- sigmoid(removal + removal_bias) * unit in place.  All float32
    rows of at least n_heads * dim columns (slices of wider rows allowed); the biases float32 [n_heads * dim]."""
    n = k.shape[0]
    width = n_heads * dim
    dp, ds = _columns(decay, "decay", width)
    rp, rs = _columns(removal, "removal", width)
    up, us = _columns(unit, "unit", width)
    kp, ks = _columns(k, "k", width)
    if any(t.shape[0] != n for t in (decay, removal, unit)) or decay_bias.numel() != width or removal_bias.numel() != width:
        raise KernelError("removal_gates: shapes do not fit")
    _check(_kernels().xrt_removal_gates(dp, ds, _ptr(decay_bias, "decay_bias", torch.float32), rp, rs,
                                       _ptr(removal_bias, "removal_bias", torch.float32), up, us, kp, ks, n, n_heads, dim,
                                       float(rate), float(unit_eps), _stream()), "removal_gates")


def act_cast(out, x, act: str) -> None:
    """out = act(x) in out's dtype; x float32 rows of at least out's width (a slice of wider rows allowed); ``act``
    "none", "silu", "sigmoid" or "tanh"."""
    n, width = out.shape
    xp, xs = _columns(x, "x", width)
    if x.shape[0] != n:
        raise KernelError("act_cast: shapes do not fit")
    _check(_kernels().xrt_act_cast(_ptr(out, "out"), xp, xs, n, width, _ACTS[act], _code(out.dtype), _stream()), "act_cast")


def add_scaled_parts(residual, parts, scales) -> None:
    """residual += sum_p scales[p] * parts[p]; residual float32 [T, width], parts float32 [n, T, width], scales float32 [n]."""
    if parts.dim() != 3 or tuple(parts.shape[1:]) != tuple(residual.shape) or scales.numel() != parts.shape[0]:
        raise KernelError("add_scaled_parts: shapes do not fit")
    _check(_kernels().xrt_add_scaled_parts(_ptr(residual, "residual", torch.float32), _ptr(parts, "parts", torch.float32),
                                          _ptr(scales, "scales", torch.float32), residual.numel(), parts.shape[0],
                                          _stream()), "add_scaled_parts")
