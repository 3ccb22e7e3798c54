"""Python binding of the kernel library: thin, checked wrappers over its ``extern "C"`` entry points.

Every wrapper takes torch tensors that live on the GPU, checks dtype, shape and contiguity,
and launches on torch's current stream.  There is no fallback: if the library cannot be built
or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
ABI_VERSION = 24

_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is None:
        path = _build.library_path(build=True)
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        _declare_signatures(handle)
        if handle.llb_abi_version() != ABI_VERSION:
            raise KernelError(f"{path} has ABI version {handle.llb_abi_version()}, expected {ABI_VERSION}")
        _lib = handle
    return _lib


_C_TYPES = {"int": ctypes.c_int, "float": ctypes.c_float, "long long": ctypes.c_longlong,
            "unsigned long long": ctypes.c_ulonglong, "cudaStream_t": ctypes.c_void_p, "const char*": ctypes.c_char_p}


def _declare_signatures(handle: ctypes.CDLL) -> None:
    """Argument and result types of every entry point, read from the ``LLB_EXPORT`` definitions in the
    sources the library was built from: pointers are passed as plain integers, without a ctypes
    object per argument."""
    pattern = re.compile(r"LLB_EXPORT\s+([\w\s\*]+?)\s*\b(llb_\w+)\s*\(([^)]*)\)\s*\{")

    def ctype(decl: str):
        decl = " ".join(decl.split())
        if decl == "void":
            return None
        if decl in _C_TYPES:
            return _C_TYPES[decl]
        if decl.endswith("*"):
            return ctypes.c_void_p
        raise KernelError(f"kernel library: no ctypes type for the C type {decl!r}")

    for name in _build.sources():
        with open(os.path.join(_build.CSRC_DIR, name)) as f:
            text = f.read()
        for ret, fn, args in pattern.findall(text):
            func = getattr(handle, fn)
            func.restype = ctype(ret)
            func.argtypes = [ctype(re.sub(r"\s*\w+$", "", a.strip())) for a in args.split(",") if a.strip() not in ("", "void")]


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().llb_last_error().decode("utf-8", "replace"))


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device address of a tensor (None: a null pointer)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("tensor is not on a CUDA device; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"tensor of shape {tuple(t.shape)} must be contiguous")
    return t.data_ptr()


def _i32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return _ptr(t)


_scoped_stream: Optional[int] = None


def torch_stream() -> "torch.cuda.Stream":
    """torch's current stream on the current device.  The device is named explicitly: asked without one,
    ``torch.cuda.current_stream()`` first looks for an available device type, which counts the devices through the
    driver every time (up to 0.14 ms a call on this machine, several calls a step)."""
    return torch.cuda.current_stream(torch.cuda.current_device())


class stream_scope:
    """Within the scope every launch goes to the stream that was current on entry, without asking torch
    again for each kernel.  The stream must not be switched inside the scope."""

    def __enter__(self):
        global _scoped_stream
        self._outer = _scoped_stream
        _scoped_stream = torch_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._outer
        return False


def _stream() -> int:
    s = _scoped_stream
    return s if s is not None else torch_stream().cuda_stream


def current_stream() -> int:
    """The stream that this module's launches go to right now (see :class:`stream_scope`)."""
    return _stream()


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None,
              scale: float = 1.0, copy: Optional[torch.Tensor] = None) -> None:
    """out[t,:] = table[ids[t],:] * scale as float.  ids int32 [T], table [V,D], out float32 [T,D]; ``copy`` ([T,D] in
    the table's dtype) receives the same rows."""
    T, (V, D) = ids.numel(), table.shape
    if out.dtype != torch.float32 or tuple(out.shape) != (T, D):
        raise KernelError(f"embedding: out must be float32 [{T},{D}], got {out.dtype} {tuple(out.shape)}")
    if scale == 1.0 and copy is None:
        _check(lib().llb_embedding(_i32(ids, "ids"), _ptr(table), _dt(table), _ptr(out), T, D, V,
                                   _i32(err, "err"), _stream()))
        return
    if copy is not None and (copy.dtype != table.dtype or tuple(copy.shape) != (T, D)):
        raise KernelError(f"embedding: copy must be {table.dtype} [{T},{D}]")
    _check(lib().llb_embedding_scaled(_i32(ids, "ids"), _ptr(table), _dt(table), _ptr(out), T, D, V, _i32(err, "err"),
                                      ctypes.c_float(scale), _ptr(copy), _stream()))


def cast_add(src: torch.Tensor, dst: torch.Tensor, accumulate: bool = False) -> None:
    """dst = src (converted to dst's dtype), or dst += src with ``accumulate``; float32 or bfloat16 on either side."""
    if src.numel() != dst.numel():
        raise KernelError(f"cast_add: {tuple(src.shape)} does not fit {tuple(dst.shape)}")
    _check(lib().llb_cast_add(_ptr(src), _dt(src), _ptr(dst), _dt(dst), src.numel(), 1 if accumulate else 0, _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r,:] = rmsnorm(x[rows[r],:]) * weight (rows = None: row r of x)."""
    D = x.shape[-1]
    R = rows.numel() if rows is not None else x.numel() // D
    if weight.numel() != D or out.numel() != R * D:
        raise KernelError(f"rmsnorm: sizes do not fit: x {tuple(x.shape)} weight {tuple(weight.shape)} out {tuple(out.shape)}")
    _check(lib().llb_rmsnorm(_ptr(x), _dt(x), _ptr(weight), _dt(weight), _ptr(out), _dt(out),
                             _i32(rows, "rows"), R, D, ctypes.c_float(eps), _stream()))


def _glu_args(glu):
    """(kind, alpha, limit, up_shift) of a GLU epilogue as C arguments; ``None`` is SiLU."""
    kind, alpha, limit, shift = glu if glu is not None else (0, 1.0, 0.0, 0.0)
    return int(kind), ctypes.c_float(alpha), ctypes.c_float(limit), ctypes.c_float(shift)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
              out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, glu=None) -> None:
    """CUDA-core contraction a[M,K] @ w[N,K]^T with a fused epilogue (see EPI_*).  ``glu = (kind, alpha, limit,
    up_shift)`` names the gated activation of the EPI_SWIGLU epilogue (see :func:`glu_act`; default SiLU)."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: a is {tuple(a.shape)} but w is {tuple(w.shape)}")
    _check_epilogue_args(a, N, M, bias, epilogue, out, residual)
    _check(lib().llb_gemm_simt_glu(_ptr(a), _dt(a), _ptr(w), _ptr(bias), _dt(w), _ptr(out), _ptr(residual),
                                   epilogue, M, N, K, *_glu_args(glu), _stream()))


def _check_epilogue_args(a, N, M, bias, epilogue, out, residual) -> None:
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError(f"gemm: bias must be float32 [{N}], got {bias.dtype} {tuple(bias.shape)}")
    if epilogue == EPI_RESIDUAL:
        if residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError(f"gemm: residual must be float32 [{M},{N}]")
        return
    want_shape = (M, N // 2) if epilogue == EPI_SWIGLU else (M, N)
    want_dtype = torch.float32 if epilogue == EPI_STORE_F32 else a.dtype
    if out is None or tuple(out.shape) != want_shape or out.dtype != want_dtype:
        got = None if out is None else (out.dtype, tuple(out.shape))
        raise KernelError(f"gemm: out must be {want_dtype} {want_shape}, got {got}")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, q_out: torch.Tensor,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate q and k by position and write k, v rows into their cache slots.

    qkv [T, (Hq + 2*Hkv)*hd]; q_out [T, Hq*hd]; caches [slots, Hkv, hd].  Without caches
    (``k_cache is None``) only q is produced and qkv holds Hq heads only."""
    T = qkv.shape[0]
    write_kv = k_cache is not None
    hkv = num_kv_heads if write_kv else 0
    if qkv.shape[1] != (num_heads + 2 * hkv) * head_dim:
        raise KernelError(f"rope_kv_write: qkv has {qkv.shape[1]} columns, expected {(num_heads + 2 * hkv) * head_dim}")
    if q_out.dtype != qkv.dtype or q_out.numel() != T * num_heads * head_dim:
        raise KernelError("rope_kv_write: q_out does not fit")
    if write_kv and (k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype):
        raise KernelError("rope_kv_write: cache dtype differs from the activations'")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_kv_write: inv_freq must be float32 [rotary_dim/2]")
    _check(lib().llb_rope_kv_write(_ptr(qkv), _dt(qkv), _i32(positions, "positions"),
                                   _i32(slot_mapping, "slot_mapping"), _ptr(inv_freq), rotary_dim,
                                   1 if interleaved else 0, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                   T, num_heads, hkv, head_dim, 1 if write_kv else 0, _stream()))


def attention_smem_bytes(bq: int, group: int, head_dim: int, v_head_dim: Optional[int] = None) -> int:
    return int(lib().llb_attention_smem_bytes_v(bq, group, head_dim, head_dim if v_head_dim is None else v_head_dim))


def attention_scratch_floats(num_tiles: int, num_heads: int, head_dim: int, bq: int, nsplit: int) -> int:
    """Floats of scratch for ``nsplit`` pieces; ``head_dim`` is the width of a VALUE row."""
    return int(lib().llb_attention_scratch_floats(num_tiles, num_heads, head_dim, bq, nsplit))


def paged_attention_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         tile_span: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int,
                         span_row: torch.Tensor, span_len: torch.Tensor, span_pos: torch.Tensor,
                         block_table: torch.Tensor, max_pages: int, page_size: int,
                         num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                         bq: int, nsplit: int = 1, scratch: Optional[torch.Tensor] = None,
                         v_head_dim: Optional[int] = None, sinks: Optional[torch.Tensor] = None,
                         v_shared: bool = False, softcap: float = 0.0) -> None:
    """Attention of every query row of the listed tiles over its request's pages.  ``v_head_dim``: width of a value
    row (and of an output row) when it differs from the keys'; ``v_cache`` may be ``k_cache`` itself (values read out
    of the key rows).  ``sinks`` float32 [num_heads]: ``exp(sinks[h])`` joins head h's softmax denominator once.
    ``v_shared``: a slot's value row (``v_head_dim`` wide: all kv heads side by side) is read whole by every query head,
    so ``out`` [T, num_heads, v_head_dim] holds each head's weights applied to the values of every kv head.  ``out`` may
    be float32 under bfloat16 inputs.  ``softcap`` > 0: a score becomes ``softcap * tanh(score / softcap)`` (sinks are
    not capped)."""
    hdv = head_dim if v_head_dim is None else v_head_dim
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or out.dtype not in (q.dtype, torch.float32):
        raise KernelError("attention: q and the caches must share a dtype, out has it or is float32")
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_heads):
        raise KernelError(f"attention: sinks must be float32 [{num_heads}]")
    if out.numel() != q.shape[0] * num_heads * hdv:
        raise KernelError("attention: out does not fit")
    if nsplit > 1:
        need = attention_scratch_floats(num_tiles, num_heads, hdv, bq, nsplit)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: nsplit={nsplit} needs {need} floats of scratch")
    _check(lib().llb_paged_attention_capped(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _dt(q),
        _i32(tile_span, "tile_span"), _i32(tile_q0, "tile_q0"), num_tiles,
        _i32(span_row, "span_row"), _i32(span_len, "span_len"), _i32(span_pos, "span_pos"),
        _i32(block_table, "block_table"), max_pages, page_size, num_heads, num_kv_heads, head_dim, hdv, _ptr(sinks),
        window, ctypes.c_float(scale), ctypes.c_float(softcap or 0.0), bq, nsplit, _ptr(scratch), 1 if v_shared else 0,
        1 if out.dtype == torch.float32 and q.dtype != torch.float32 else 0, _stream()))


def _f32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{what} must be float32, got {t.dtype}")
    return _ptr(t)


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out: torch.Tensor,
              rows: Optional[torch.Tensor] = None, accumulate: bool = False, copy: Optional[torch.Tensor] = None) -> None:
    """out[r,:] = LN(x[rows[r],:]) * weight + bias (rows = None: row r), or out += ... with ``accumulate``.
    x float32; weight and bias share a dtype (``bias`` None: none is added); out float32 or bfloat16.  ``copy`` (bfloat16, out's shape) receives what
    was written to out as well."""
    if copy is not None and (copy.dtype != torch.bfloat16 or copy.numel() != out.numel()):
        raise KernelError("layernorm: copy must be bfloat16 of out's size")
    D = x.shape[-1]
    R = rows.numel() if rows is not None else x.numel() // D
    if x.dtype != torch.float32 or weight.numel() != D or (bias is not None and (bias.numel() != D or weight.dtype != bias.dtype)) \
            or out.numel() != R * D:
        raise KernelError(f"layernorm: x {x.dtype} {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    _check(lib().llb_layernorm(_ptr(x), _ptr(weight), _ptr(bias), _dt(weight), _ptr(out), _dt(out), _i32(rows, "rows"),
                               R, D, ctypes.c_float(eps), 1 if accumulate else 0, _ptr(copy), _stream()))


GLU_SILU, GLU_CLAMPED_SWISH, GLU_GELU_TANH = 0, 1, 2


def glu_act(x: torch.Tensor, out: torch.Tensor, kind: int, alpha: float = 1.0, limit: float = 0.0,
            up_shift: float = 0.0) -> None:
    """out[m, j] = glu(x[m, 2j], x[m, 2j+1]): GLU_SILU ``silu(g) * u``; GLU_CLAMPED_SWISH
    ``g' sigmoid(alpha g') (u' + up_shift)`` with ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``."""
    M, N = x.shape
    if N % 2 or tuple(out.shape) != (M, N // 2) or out.dtype != x.dtype:
        raise KernelError(f"glu_act: x {tuple(x.shape)} does not fit out {tuple(out.shape)}")
    _check(lib().llb_glu_act(_ptr(x), _ptr(out), _dt(x), M, N // 2, kind, ctypes.c_float(alpha), ctypes.c_float(limit),
                             ctypes.c_float(up_shift), _stream()))


def head_gate(x: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, num_heads: int, head_dim: int,
              per_head: bool, act: str, unit_rms: bool = False, eps: float = 0.0,
              norm_weight: Optional[torch.Tensor] = None, denominator: Optional[torch.Tensor] = None) -> None:
    """out[t,h,:] = (x[t,h,:], or x / rms(x) over the head with ``unit_rms``) * act(gate), act ``sigmoid`` or ``silu``;
    ``norm_weight`` (float32, [head_dim] shared by the heads or [num_heads * head_dim]) multiplies the normed head before
    the gate; ``denominator`` (float32 [T, H]) divides every head's x first, before the norm.
    ``gate`` is a [T, H] (``per_head``) or [T, H*head_dim] view whose rows may be strided (columns of a wider tensor).
    x float32 or the dtype of gate and out."""
    T = x.shape[0]
    width = num_heads if per_head else num_heads * head_dim
    if gate.dim() != 2 or tuple(gate.shape) != (T, width) or gate.stride(1) != 1 or gate.dtype != out.dtype:
        raise KernelError(f"head_gate: gate must be {out.dtype} [{T},{width}] with unit inner stride")
    if x.numel() != T * num_heads * head_dim or out.numel() != x.numel():
        raise KernelError("head_gate: sizes do not fit")
    if norm_weight is not None and norm_weight.numel() not in (head_dim, num_heads * head_dim):
        raise KernelError("head_gate: norm_weight must have one weight per dimension of a head, or of every head")
    if denominator is not None and (denominator.dtype != torch.float32 or denominator.numel() != T * num_heads):
        raise KernelError(f"head_gate: the denominator must be float32 [{T},{num_heads}]")
    if not gate.is_cuda:
        raise KernelError("tensor is not on a CUDA device; there is no CPU path")
    per_head_weight = norm_weight is not None and norm_weight.numel() != head_dim
    _check(lib().llb_head_gate_ex(_ptr(x), _dt(x), ctypes.c_void_p(gate.data_ptr()), ctypes.c_longlong(gate.stride(0)),
                                  _ptr(out), _dt(out), T, num_heads, head_dim, 1 if unit_rms else 0, ctypes.c_float(eps),
                                  1 if per_head else 0, {"sigmoid": 0, "silu": 1}[act], _f32(norm_weight, "norm_weight"),
                                  1 if per_head_weight else 0, _f32(denominator, "denominator"), _stream()))


def talk_mix(o: torch.Tensor, talk: Optional[torch.Tensor], gate: Optional[torch.Tensor], out: torch.Tensor,
             num_heads: int, num_kv_heads: int, v_head_dim: int) -> None:
    """out[t, h, :] = sum_g talk[h, g] * o[t, g, kv(h), :], times sigmoid(gate[t, h, :]): ``o`` [T, H, G, vdim] holds every
    query head's softmax weights applied to the values of every kv head (float32 or the activation dtype), ``talk``
    float32 [H, H] mixes the heads (``None``: head h takes ``o[t, h, kv(h)]``), ``gate`` [T, H*vdim] may be columns of a
    wider tensor (``None``: no gate); ``out`` [T, H*vdim] in the activation dtype."""
    T = out.shape[0]
    H, G, vd = num_heads, num_kv_heads, v_head_dim
    if o.numel() != T * H * G * vd or out.numel() != T * H * vd or not o.is_contiguous() or not out.is_contiguous():
        raise KernelError("talk_mix: sizes do not fit")
    if talk is not None and (talk.dtype != torch.float32 or tuple(talk.shape) != (H, H) or not talk.is_contiguous()):
        raise KernelError(f"talk_mix: the mixing matrix must be float32 [{H},{H}]")
    if gate is not None and (gate.dim() != 2 or tuple(gate.shape) != (T, H * vd) or gate.stride(1) != 1 or gate.dtype != out.dtype):
        raise KernelError(f"talk_mix: gate must be {out.dtype} [{T},{H * vd}] with unit inner stride")
    _check(lib().llb_talk_mix(_ptr(o), _dt(o), _ptr(talk), None if gate is None else ctypes.c_void_p(gate.data_ptr()),
                              ctypes.c_longlong(0 if gate is None else gate.stride(0)), _ptr(out), _dt(out), T, H, G, vd,
                              _stream()))


def rmsnorm_add(x: torch.Tensor, weight: torch.Tensor, eps: float, dst: torch.Tensor, scale: float = 1.0) -> None:
    """dst += scale * rmsnorm(x) * weight, x and dst float32 [T, D]: a normed branch joining a float sum."""
    T, D = x.shape
    if x.dtype != torch.float32 or dst.dtype != torch.float32 or tuple(dst.shape) != (T, D) or weight.numel() != D:
        raise KernelError("rmsnorm_add: x and dst must be float32 of one shape, weight one value a column")
    _check(lib().llb_rmsnorm_add(_ptr(x), _ptr(weight), _dt(weight), _ptr(dst), ctypes.c_longlong(T), D,
                                 ctypes.c_float(eps), ctypes.c_float(scale), _stream()))


def axpy(x: torch.Tensor, y: torch.Tensor, a: float, copy: Optional[torch.Tensor] = None) -> None:
    """y += a * x (float32, equal sizes); ``copy`` (bfloat16) receives the new y as well."""
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.numel() != y.numel():
        raise KernelError("axpy: x and y must be float32 of equal size")
    if copy is not None and (copy.dtype != torch.bfloat16 or copy.numel() != y.numel()):
        raise KernelError("axpy: the copy must be bfloat16 of y's size")
    _check(lib().llb_axpy(_ptr(x), _ptr(y), _ptr(copy), ctypes.c_longlong(y.numel()), ctypes.c_float(a), _stream()))


def add_row(x: torch.Tensor, v: torch.Tensor) -> None:
    """x[t, :] += v for every row of the float32 [T, D] tensor x."""
    T, D = x.shape
    if x.dtype != torch.float32 or v.numel() != D or not v.is_contiguous():
        raise KernelError("add_row: x must be float32 [T, D] and v hold D values")
    _check(lib().llb_add_row(_ptr(x), _ptr(v), _dt(v), ctypes.c_longlong(T), D, _stream()))


def softcap(x: torch.Tensor, cap: float) -> None:
    """x = cap * tanh(x / cap) in place (float32)."""
    if x.dtype != torch.float32 or not cap > 0:
        raise KernelError("softcap: x must be float32 and the cap positive")
    _check(lib().llb_softcap(_ptr(x), ctypes.c_longlong(x.numel()), ctypes.c_float(cap), _stream()))


def memory_gates(pre: torch.Tensor, i_off: int, f_off: int, bias_i: Optional[torch.Tensor], bias_f: Optional[torch.Tensor],
                 cap: float, ctx_spans, num_heads: int, state: torch.Tensor, m_off: int, keep: torch.Tensor,
                 take: torch.Tensor, floor: torch.Tensor) -> None:
    """The gates of a matrix memory (csrc/matrix_memory.cu) for every token and head of the step: ``pre`` float32 [T, C]
    holds the pre-activations of the input gates in columns ``i_off ..`` and of the forget gates in ``f_off ..`` (one a
    head; ``bias_*`` float32 [H] are added); ``keep``, ``take``, ``floor`` float32 [T, H] receive ``exp(f + m' - m)``,
    ``exp(i - m)``, ``exp(-m)``; a request's running maximum m [H] lives at ``m_off`` floats into its slot of ``state``."""
    T, C = pre.shape
    H = num_heads
    span_row, span_len, span_pos, span_slot, num_spans = ctx_spans
    base, stride = _state_base(state)
    if pre.dtype != torch.float32 or not pre.is_contiguous() or max(i_off, f_off) + H > C:
        raise KernelError("memory_gates: pre must be contiguous float32 and hold both gates' columns")
    if m_off + H > stride or any(t.dtype != torch.float32 or t.numel() != T * H for t in (keep, take, floor)):
        raise KernelError("memory_gates: outputs must be float32 [T, H] and m must fit in a state slot")
    _check(lib().llb_memory_gates(_ptr(pre), ctypes.c_longlong(T), ctypes.c_longlong(C), i_off, f_off, _f32(bias_i, "bias_i"),
                                  _f32(bias_f, "bias_f"), ctypes.c_float(cap), _i32(span_row, "span_row"),
                                  _i32(span_len, "span_len"), _i32(span_pos, "span_pos"), _i32(span_slot, "span_slot"),
                                  num_spans, H, base, ctypes.c_longlong(stride), ctypes.c_longlong(m_off), _ptr(keep),
                                  _ptr(take), _ptr(floor), _stream()))


def matrix_memory(src: torch.Tensor, q_off: int, k_off: int, v_off: int, q_scale: float, keep: torch.Tensor,
                  take: torch.Tensor, floor: torch.Tensor, ctx_spans, num_heads: int, head_dim: int, v_head_dim: int,
                  state: torch.Tensor, s_off: int, out: torch.Tensor, den: torch.Tensor, pieces=None) -> None:
    """The matrix memory's recurrence over every span of the step (csrc/matrix_memory.cu): q, k [H, dim] and v [H, vdim]
    are column ranges of ``src`` [T, C]; the gates from :func:`memory_gates`; a request's ``[H, dim, vdim + 1]`` floats (S
    with n as its last column) live at ``s_off`` into its slot of ``state``; ``out`` float32 [T, H*vdim] receives the
    numerators ``S^T q`` and ``den`` float32 [T, H] the denominators.  ``pieces`` as :func:`retention` takes them."""
    T, C = src.shape
    H, hd, vd = num_heads, head_dim, v_head_dim
    span_row, span_len, span_pos, span_slot, num_spans = ctx_spans
    base, stride = _state_base(state)
    if max(q_off, k_off) + H * hd > C or v_off + H * vd > C or not src.is_contiguous():
        raise KernelError("matrix_memory: q, k or v lie outside the columns of src")
    if s_off + H * hd * (vd + 1) > stride:
        raise KernelError("matrix_memory: the state does not fit in a slot")
    if out.dtype != torch.float32 or out.numel() != T * H * vd or den.dtype != torch.float32 or den.numel() != T * H:
        raise KernelError("matrix_memory: out must be float32 [T, H*vdim] and den float32 [T, H]")
    scratch = piece_keep = None
    if pieces is None:
        iota = torch.arange(num_spans, dtype=torch.int32, device=src.device)
        item_span, item_c, span_first, num_items, chunk = iota, torch.zeros_like(iota), iota, num_spans, 1 << 30
    else:
        item_span, item_c, span_first, num_items, chunk = pieces
    multi = num_items > num_spans
    if multi:
        scratch = torch.empty((num_items, H, hd, vd + 1), dtype=torch.float32, device=src.device)
        piece_keep = torch.empty((num_items, H), dtype=torch.float32, device=src.device)
    _check(lib().llb_matrix_memory(_ptr(src), _dt(src), ctypes.c_longlong(C), q_off, k_off, v_off, ctypes.c_float(q_scale),
                                   _ptr(keep), _ptr(take), _ptr(floor), _i32(span_row, "span_row"),
                                   _i32(span_len, "span_len"), _i32(span_pos, "span_pos"), _i32(span_slot, "span_slot"),
                                   num_spans, _i32(item_span, "item_span"), _i32(item_c, "item_c"),
                                   _i32(span_first, "span_first"), num_items, chunk, 1 if multi else 0, H, hd, vd, base,
                                   ctypes.c_longlong(stride), ctypes.c_longlong(s_off), _ptr(scratch), _ptr(piece_keep),
                                   _ptr(out), _ptr(den), _stream()))


def qkv_prepare(src: torch.Tensor, q_off: int, k_off: int, v_off: int, num_heads: int, num_kv_heads: int,
                head_dim: int, v_head_dim: int, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                q_out: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, interleaved: bool = False) -> None:
    """From a fused projection ``src`` [T, C] (q at columns ``q_off``, k at ``k_off``, v at ``v_off`` or -1 for none):
    optional RMS norm of q and of k over their whole projection, rotation, q to ``q_out`` [T, Hq*hd], k and v rows to
    their cache slots.  ``num_heads == 0`` writes the cache only."""
    T, C = src.shape
    for off, n in ((q_off, num_heads * head_dim), (k_off, num_kv_heads * head_dim), (v_off, num_kv_heads * v_head_dim)):
        if n and off >= 0 and off + n > C:
            raise KernelError(f"qkv_prepare: columns {off}..{off + n} lie outside the {C} of src")
    if num_heads and (q_out is None or q_out.dtype != src.dtype or q_out.numel() != T * num_heads * head_dim):
        raise KernelError("qkv_prepare: q_out does not fit")
    if slot_mapping is not None and num_kv_heads:
        if k_cache is None or k_cache.dtype != src.dtype or tuple(k_cache.shape[1:]) != (num_kv_heads, head_dim):
            raise KernelError("qkv_prepare: k_cache does not fit")
        if v_off >= 0 and (v_cache is None or v_cache.dtype != src.dtype
                           or tuple(v_cache.shape[1:]) != (num_kv_heads, v_head_dim)):
            raise KernelError("qkv_prepare: v_cache does not fit")
    if q_norm_w is not None and q_norm_w.numel() != num_heads * head_dim:
        raise KernelError("qkv_prepare: q_norm_w must have one weight per column of q")
    if k_norm_w is not None and k_norm_w.numel() != num_kv_heads * head_dim:
        raise KernelError("qkv_prepare: k_norm_w must have one weight per column of k")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("qkv_prepare: inv_freq must be float32 [rotary_dim/2]")
    _check(lib().llb_qkv_prepare(_ptr(src), _dt(src), ctypes.c_longlong(C), q_off, k_off, v_off, T, num_heads, num_kv_heads,
                                 head_dim, v_head_dim, _f32(q_norm_w, "q_norm_w"), _f32(k_norm_w, "k_norm_w"),
                                 ctypes.c_float(eps), _i32(positions, "positions"), _f32(inv_freq, "inv_freq"), rotary_dim,
                                 1 if interleaved else 0, _i32(slot_mapping, "slot_mapping"), _ptr(q_out), _ptr(k_cache),
                                 _ptr(v_cache), _stream()))


def head_prepare(src: torch.Tensor, q_off: int, k_off: int, num_q_heads: int, num_k_heads: int, head_dim: int,
                 positions: torch.Tensor, slot_mapping: Optional[torch.Tensor], q_out: Optional[torch.Tensor],
                 k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], *, q_maps: int = 1,
                 values: Optional[str] = None, v_off: int = -1, v_width: int = 0,
                 q_norm_w: Optional[torch.Tensor] = None, k_norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                 inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0, interleaved: bool = False) -> None:
    """From a fused projection ``src`` [T, C] with ``num_q_heads`` query heads at ``q_off`` and ``num_k_heads`` key heads
    at ``k_off`` (each ``head_dim`` wide): per head an optional RMS norm with a weight [head_dim] shared by the heads
    (float32), then the rotation of the first ``rotary_dim`` dimensions; queries to ``q_out``, keys to the cache rows
    ``slot_mapping`` names (``None``: nothing is cached).  ``q_maps`` = M > 1 writes query head i as a row of
    ``M * head_dim`` numbers with the head at offset ``(i % M) * head_dim`` and zeros elsewhere (attention with M score
    maps a head over key rows that hold a kv head's maps side by side).  ``values``: ``None`` no value rows, ``"columns"``
    the ``v_width`` numbers at ``v_off`` are copied to the slot's value row, ``"keys"`` the value row is the key row as
    projected (before norm and rotation)."""
    T, C = src.shape
    for off, n in ((q_off, num_q_heads * head_dim), (k_off, num_k_heads * head_dim), (v_off, v_width)):
        if n and off >= 0 and off + n > C:
            raise KernelError(f"head_prepare: columns {off}..{off + n} lie outside the {C} of src")
    if src.stride(1) != 1:
        raise KernelError("head_prepare: the rows of src must be dense")
    if num_q_heads and (q_out is None or q_out.dtype != src.dtype or q_out.numel() != T * num_q_heads * q_maps * head_dim):
        raise KernelError("head_prepare: q_out does not fit")
    v_mode = {None: 0, "columns": 1, "keys": 2}[values]
    if slot_mapping is not None and num_k_heads:
        if k_cache is None or k_cache.dtype != src.dtype or k_cache[0].numel() != num_k_heads * head_dim:
            raise KernelError("head_prepare: k_cache does not fit")
        want = {0: None, 1: v_width, 2: num_k_heads * head_dim}[v_mode]
        if want is not None and (v_cache is None or v_cache.dtype != src.dtype or v_cache[0].numel() != want):
            raise KernelError("head_prepare: v_cache does not fit")
    for w_ in (q_norm_w, k_norm_w):
        if w_ is not None and (w_.dtype != torch.float32 or w_.numel() != head_dim):
            raise KernelError("head_prepare: a norm weight is float32 [head_dim], shared by the heads")
    if rotary_dim and (inv_freq is None or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("head_prepare: inv_freq must be float32 [rotary_dim/2]")
    writes = slot_mapping is not None
    _check(lib().llb_head_prepare(_ptr(src), _dt(src), ctypes.c_longlong(src.stride(0)), q_off, k_off, v_off, T, num_q_heads,
                                  num_k_heads if writes else 0, head_dim, q_maps, v_mode if writes else 0, v_width,
                                  _f32(q_norm_w, "q_norm_w"), _f32(k_norm_w, "k_norm_w"), ctypes.c_float(eps),
                                  _i32(positions, "positions"), _f32(inv_freq, "inv_freq"), rotary_dim,
                                  1 if interleaved else 0, _i32(slot_mapping, "slot_mapping"), _ptr(q_out),
                                  _ptr(k_cache) if writes else None, _ptr(v_cache) if writes else None, _stream()))


def diff_combine(a: torch.Tensor, out: torch.Tensor, num_heads: int, v_head_dim: int, lam: float, eps: float,
                 mult: float) -> None:
    """``a`` [T, heads, 2, v_head_dim] (float32 or the dtype of ``out``): the outputs of every head's two attention maps;
    ``out[t, h] = unit_rms(a[t, h, 0] - lam * a[t, h, 1]) * mult`` with the root mean square over the head's values and
    ``eps`` inside the root."""
    T = out.shape[0]
    if a.numel() != T * num_heads * 2 * v_head_dim or out.numel() != T * num_heads * v_head_dim:
        raise KernelError("diff_combine: sizes do not fit")
    if a.dtype not in (torch.float32, out.dtype):
        raise KernelError("diff_combine: a is float32 or has the dtype of out")
    _check(lib().llb_diff_combine(_ptr(a), _dt(a), _ptr(out), _dt(out), T, num_heads, v_head_dim, ctypes.c_float(lam),
                                  ctypes.c_float(eps), ctypes.c_float(mult), _stream()))


def head_linear(x: torch.Tensor, x_off: int, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, h, :] = w[h] @ x[t, x_off + h*in : x_off + (h+1)*in] for w [H, out, in]; x [T, C], out [T, H*out]."""
    T, C = x.shape
    H, on, inn = w.shape
    if x_off < 0 or x_off + H * inn > C or w.dtype != x.dtype or out.dtype != x.dtype or tuple(out.shape) != (T, H * on):
        raise KernelError(f"head_linear: x {tuple(x.shape)} at {x_off}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(lib().llb_head_linear(_ptr(x), ctypes.c_longlong(C), x_off, _ptr(w), _ptr(out), _dt(x), T, H, inn, on, _stream()))


def retention(src: torch.Tensor, q_off: int, k_off: int, v_off: int, span_row: torch.Tensor, span_len: torch.Tensor,
              span_pos: torch.Tensor, span_slot: torch.Tensor, num_spans: int, num_heads: int, head_dim: int,
              v_head_dim: int, decay: torch.Tensor, inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool,
              k_scale: float, state: torch.Tensor, out: torch.Tensor, pieces=None) -> None:
    """The retention recurrence over every span of the step (csrc/retention.cu): ``state`` float32
    [slots, H, dim, vdim] is read where a span continues a request and written at its end; ``out`` float32 [T, H*vdim].

    ``pieces = (item_span, item_c, span_first, num_items, chunk)`` cuts the spans into pieces of ``chunk`` tokens that run
    side by side (int32 arrays on the device: the span and index of every piece, a span's pieces consecutive, and every
    span's first piece); without it every span is one piece."""
    T, C = src.shape
    if max(q_off, k_off) + num_heads * head_dim > C or v_off + num_heads * v_head_dim > C:
        raise KernelError("retention: q, k or v lie outside the columns of src")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (num_heads, head_dim, v_head_dim):
        raise KernelError(f"retention: state must be float32 [slots, {num_heads}, {head_dim}, {v_head_dim}]")
    if out.dtype != torch.float32 or out.numel() != T * num_heads * v_head_dim or decay.numel() != num_heads:
        raise KernelError("retention: out or decay does not fit")
    scratch = None
    if pieces is None:
        iota = torch.arange(num_spans, dtype=torch.int32, device=src.device)
        item_span, item_c, span_first, num_items, chunk = iota, torch.zeros_like(iota), iota, num_spans, 1 << 30
    else:
        item_span, item_c, span_first, num_items, chunk = pieces
    multi = num_items > num_spans
    if multi:
        scratch = torch.empty((num_items, num_heads, head_dim, v_head_dim), dtype=torch.float32, device=src.device)
    _check(lib().llb_retention(_ptr(src), _dt(src), ctypes.c_longlong(C), q_off, k_off, v_off, _i32(span_row, "span_row"),
                               _i32(span_len, "span_len"), _i32(span_pos, "span_pos"), _i32(span_slot, "span_slot"),
                               num_spans, _i32(item_span, "item_span"), _i32(item_c, "item_c"),
                               _i32(span_first, "span_first"), num_items, chunk, 1 if multi else 0, num_heads, head_dim,
                               v_head_dim, _f32(decay, "decay"), _f32(inv_freq, "inv_freq"), rotary_dim,
                               1 if interleaved else 0, ctypes.c_float(k_scale), _ptr(state), _ptr(scratch), _ptr(out),
                               _stream()))


# ---- short convolution, delta rule, routing (csrc/short_conv.cu, csrc/delta_rule.cu, csrc/moe.cu) -------------------------
CONV_NORMS = {None: 0, "rms": 1, "unit": 2}


class ConvSegment:
    """One of the up to three head groups (q, k, v) that :func:`conv_prepare` makes from the convolved channels:
    ``col0`` first channel, ``heads`` x ``head_dim``, ``act`` None or ``"silu"``, ``rotary_dim`` leading dimensions
    rotated, ``norm`` None, ``"rms"`` (unit root mean square) or ``"unit"`` (unit length) with ``eps``, ``scale`` on
    the result, ``out`` a dense [T, heads*head_dim] tensor or (``to_cache``) the cache rows [slots, heads, head_dim].
    ``temperature = (coef, every)``: the result is also multiplied by ``1 + coef * ln(floor((pos + 1) / every) + 1)``."""

    def __init__(self, col0: int, heads: int, head_dim: int, out: torch.Tensor, to_cache: bool = False, act=None,
                 rotary_dim: int = 0, norm=None, eps: float = 0.0, scale: float = 1.0, temperature=None):
        self.col0, self.heads, self.head_dim, self.out, self.to_cache = col0, heads, head_dim, out, to_cache
        self.act, self.rotary_dim, self.norm, self.eps, self.scale = act, rotary_dim, norm, eps, scale
        self.temp_coef, self.temp_every = (float(temperature[0]), int(temperature[1])) if temperature else (0.0, 0)


def _state_base(state: torch.Tensor):
    if state.dtype != torch.float32 or not state.is_contiguous() or not state.is_cuda:
        raise KernelError("the state plane must be contiguous float32 on the device")
    return state.data_ptr(), state.numel() // state.shape[0]


def cast_concat(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """out [T, 2D] = [a | b]: a float32 [T, D] converted to out's dtype, b [T, D] already in it."""
    T, D = a.shape
    if a.dtype != torch.float32 or tuple(b.shape) != (T, D) or b.dtype != out.dtype or tuple(out.shape) != (T, 2 * D):
        raise KernelError("cast_concat: sizes or dtypes do not fit")
    _check(lib().llb_cast_concat(_ptr(a), _ptr(b), _ptr(out), _dt(out), ctypes.c_longlong(T), D, _stream()))


def conv_prepare(src: torch.Tensor, c0: int, channels: int, weight: torch.Tensor, segments, ctx_spans, state,
                 tail_off: int, slot_mapping: Optional[torch.Tensor] = None, freq: Optional[torch.Tensor] = None,
                 rot_scale: float = 1.0, fuse_tail: bool = False) -> None:
    """Short causal convolution (``weight`` float32 [channels, taps]) over columns ``c0 .. c0+channels`` of ``src`` [T, C],
    then per segment activation, rotation of pairs (2i, 2i+1) by ``positions * freq[i]`` (cos and sin times
    ``rot_scale``), head norm and scale.  ``ctx_spans = (span_row, span_len, span_pos, span_slot, num_spans)``;
    ``state`` float32 [slots, ...] holds each request's last ``taps - 1`` inputs at ``tail_off`` floats into its slot
    (``None`` when ``taps == 1``).  ``fuse_tail`` (a step whose spans are all single tokens): the new tails are written by
    this launch and :func:`conv_tail_update` is not needed."""
    T, C = src.shape
    taps = weight.shape[1]
    if weight.dtype != torch.float32 or weight.shape[0] != channels or c0 + channels > C:
        raise KernelError(f"conv_prepare: weight {weight.dtype} {tuple(weight.shape)} for {channels} channels of {C} columns")
    span_row, span_len, span_pos, span_slot, num_spans = ctx_spans
    base, stride = (None, 0) if state is None else _state_base(state)
    if state is not None and tail_off + (taps - 1) * channels > stride:
        raise KernelError("conv_prepare: the tail does not fit in a state slot")
    n = len(segments)
    I, Fl, P = ctypes.c_int * n, ctypes.c_float * n, ctypes.c_void_p * n
    for sg in segments:
        want = (T * sg.heads * sg.head_dim) if not sg.to_cache else None
        if not sg.out.is_cuda or not sg.out.is_contiguous() or (want is not None and sg.out.numel() != want):
            raise KernelError("conv_prepare: a segment's output does not fit")
        if sg.to_cache and tuple(sg.out.shape[1:]) != (sg.heads, sg.head_dim):
            raise KernelError("conv_prepare: a segment's cache plane does not fit")
    _check(lib().llb_conv_prepare_temp(
        _ptr(src), _dt(src), ctypes.c_longlong(C), c0, channels, taps, T, _f32(weight, "weight"),
        _i32(span_row, "span_row"), _i32(span_len, "span_len"), _i32(span_pos, "span_pos"), _i32(span_slot, "span_slot"),
        num_spans, base, ctypes.c_longlong(stride), ctypes.c_longlong(tail_off), _i32(slot_mapping, "slot_mapping"),
        _f32(freq, "freq"), ctypes.c_float(rot_scale), n, I(*[s.col0 for s in segments]), I(*[s.heads for s in segments]),
        I(*[s.head_dim for s in segments]), I(*[{None: 0, "silu": 1}[s.act] for s in segments]),
        I(*[s.rotary_dim for s in segments]), I(*[CONV_NORMS[s.norm] for s in segments]),
        Fl(*[s.eps for s in segments]), Fl(*[s.scale for s in segments]), Fl(*[s.temp_coef for s in segments]),
        I(*[s.temp_every for s in segments]), P(*[s.out.data_ptr() for s in segments]),
        I(*[_dt(s.out) for s in segments]), I(*[1 if s.to_cache else 0 for s in segments]), 1 if fuse_tail else 0,
        _stream()))


def conv_tail_update(src: torch.Tensor, c0: int, channels: int, taps: int, ctx_spans, state: torch.Tensor,
                     tail_off: int) -> None:
    """After :func:`conv_prepare` (and every other reader of the old tails): each span's request keeps the inputs of its
    last ``taps - 1`` positions."""
    if taps <= 1:
        return
    span_row, span_len, span_pos, span_slot, num_spans = ctx_spans
    base, stride = _state_base(state)
    _check(lib().llb_conv_tail_update(_ptr(src), _dt(src), ctypes.c_longlong(src.shape[1]), c0, channels, taps,
                                      _i32(span_row, "span_row"), _i32(span_len, "span_len"), _i32(span_pos, "span_pos"),
                                      _i32(span_slot, "span_slot"), num_spans, base, ctypes.c_longlong(stride),
                                      ctypes.c_longlong(tail_off), _stream()))


def delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, ctx_spans,
               num_heads: int, num_qk_heads: int, head_dim: int, v_head_dim: int, state: torch.Tensor, state_off: int,
               out: torch.Tensor, blocked: bool = False) -> None:
    """The gated delta rule over every span (csrc/delta_rule.cu).  q, k float32 [T, G*dim]; v float32 [T, H*vdim]; g float32
    [T, H*dim] logarithms of the decay factors; ``beta`` a [T, H] view (rows may be strided) of values before the
    sigmoid; the state [H, dim, vdim] of a request lies ``state_off`` floats into its slot of ``state``; out float32
    [T, H*vdim].  ``blocked`` walks the spans in blocks of 16 tokens (for steps with long spans), else token by token."""
    T = q.shape[0]
    H, G, dim, vdim = num_heads, num_qk_heads, head_dim, v_head_dim
    for t, n, what in ((q, G * dim, "q"), (k, G * dim, "k"), (v, H * vdim, "v"), (g, H * dim, "g"), (out, H * vdim, "out")):
        if t.dtype != torch.float32 or t.numel() != T * n:
            raise KernelError(f"delta_rule: {what} must be float32 [{T}, {n}]")
    if beta.dim() != 2 or tuple(beta.shape) != (T, H) or beta.stride(1) != 1 or not beta.is_cuda:
        raise KernelError(f"delta_rule: beta must be [{T}, {H}] with unit inner stride")
    span_row, span_len, span_pos, span_slot, num_spans = ctx_spans
    base, stride = _state_base(state)
    if state_off + H * dim * vdim > stride:
        raise KernelError("delta_rule: the state does not fit in a slot")
    scratch, max_blocks = None, 0
    if blocked:          # what the first kernel leaves for the second: bounded by the step's counts alone
        max_blocks = T // 16 + num_spans
        scratch = torch.empty(int(lib().llb_delta_rule_scratch_floats(max_blocks, H, dim)), dtype=torch.float32, device=q.device)
    _check(lib().llb_delta_rule(_ptr(q), _ptr(k), _ptr(v), _ptr(g), ctypes.c_void_p(beta.data_ptr()),
                                ctypes.c_longlong(beta.stride(0)), _dt(beta), _i32(span_row, "span_row"),
                                _i32(span_len, "span_len"), _i32(span_pos, "span_pos"), _i32(span_slot, "span_slot"),
                                num_spans, H, G, dim, vdim, base, ctypes.c_longlong(stride), ctypes.c_longlong(state_off),
                                _ptr(out), 1 if blocked else 0, _ptr(scratch), max_blocks, _stream()))


LOW_RANK_MODES = {None: 0, "sigmoid": 1, "log_decay": 2}


def low_rank_up(x: torch.Tensor, x_off: int, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                mode=None, rate: Optional[torch.Tensor] = None) -> None:
    """out[t, n] = f(sum_r x[t, x_off + r] * w[n, r] + bias[n]) with float sums: the second half of a low-rank pair,
    read from columns of a fused first projection.  ``mode`` None, ``"sigmoid"`` or ``"log_decay"``:
    ``-rate[h] * softplus(.)`` (the logarithm of a decay factor) with ``rate`` float32 [H] and n = h * (N / H) + ...;
    out float32 or bfloat16 [T, N]."""
    T, C = x.shape
    N, R = w.shape
    if x_off + R > C or tuple(out.shape) != (T, N):
        raise KernelError("low_rank_up: sizes do not fit")
    per = 1
    if mode == "log_decay":
        if rate is None or N % rate.numel():
            raise KernelError("low_rank_up: the decay mode needs one rate per head")
        per = N // rate.numel()
    _check(lib().llb_low_rank_up(_ptr(x), _dt(x), ctypes.c_longlong(C), x_off, T, R, _ptr(w), _dt(w), N, _f32(bias, "bias"),
                                 LOW_RANK_MODES[mode], _f32(rate, "rate"), per, _ptr(out), _dt(out), _stream()))


def moe_route(x: torch.Tensor, w: torch.Tensor, correction: Optional[torch.Tensor], top: int, scale: float,
              ids: torch.Tensor, weights: torch.Tensor, dense: torch.Tensor, softmax: bool = False,
              renormalize: bool = False, *, renorm_eps: float = 0.0, real: Optional[int] = None, groups: int = 0,
              keep: int = 0, identity_weight: Optional[torch.Tensor] = None, gate_rows: int = 0,
              gate_out: Optional[torch.Tensor] = None) -> None:
    """Routing in float (csrc/moe.cu): x [T, D], w float32 [E + gate_rows, D], correction float32 [E] or None (joins the
    choice, not the weights); ids int32 [T, top], weights float32 [T, top], dense float32 [T, real] (zero where not chosen).
    ``real`` < E: the router's outputs from ``real`` on are identity experts; their entries of ``ids`` are -1 and a
    token's weights on them are summed into ``identity_weight`` float32 [T].  ``groups`` > 1: only experts of the ``keep``
    best of ``groups`` equal groups of neighbours can be chosen (a group's score is its largest choice score).
    ``gate_rows``: that many further rows of w give ``gate_out`` float32 [T, gate_rows] = sigmoid(w . x)."""
    T, D = x.shape
    E = w.shape[0] - gate_rows
    real = E if real is None else real
    if w.dtype != torch.float32 or w.shape[1] != D or (correction is not None and correction.numel() != E):
        raise KernelError("moe_route: the router's weights must be float32 [E, D] and the correction [E]")
    if ids.dtype != torch.int32 or ids.numel() != T * top or weights.numel() != T * top or dense.numel() < T * real:
        raise KernelError("moe_route: outputs do not fit")
    if real < E and (identity_weight is None or identity_weight.numel() != T):
        raise KernelError("moe_route: identity experts need identity_weight float32 [T]")
    if gate_rows and (gate_out is None or gate_out.numel() != T * gate_rows):
        raise KernelError("moe_route: gate rows need gate_out float32 [T, gate_rows]")
    _check(lib().llb_moe_route_ex(_ptr(x), _dt(x), _f32(w, "w"), _f32(correction, "correction"), T, D, E, real, top,
                                  1 if softmax else 0, 1 if renormalize else 0, ctypes.c_float(renorm_eps),
                                  ctypes.c_float(scale), groups, keep, gate_rows, _i32(ids, "ids"), _f32(weights, "weights"),
                                  _f32(dense, "dense"), _f32(identity_weight, "identity_weight"), _f32(gate_out, "gate_out"),
                                  _stream()))


def moe_scale(act: torch.Tensor, dense: torch.Tensor, num_experts: int, width: int) -> None:
    """act [T, E*width] *= dense [T, E] expert by expert, in place (exact zeros where an expert was not chosen)."""
    T = act.shape[0]
    if act.numel() != T * num_experts * width or dense.numel() != T * num_experts:
        raise KernelError("moe_scale: sizes do not fit")
    _check(lib().llb_moe_scale(_ptr(act), _dt(act), _f32(dense, "dense"), T, num_experts, width, _stream()))


MOE_TILE_ROWS = 128          # rows of a tile of the grouped contraction: every expert's rows are padded to a multiple


def moe_sorted_tiles(pairs: int, num_experts: int) -> int:
    """Tiles that the (token, expert) pairs take at most once every expert's rows are padded to whole tiles."""
    return -(-pairs // MOE_TILE_ROWS) + num_experts


def moe_sort(ids: torch.Tensor, num_experts: int, slot: torch.Tensor, tile_group: torch.Tensor) -> None:
    """ids int32 [T, top] -> slot int32 [T*top] (each pair's row in expert order, experts padded to whole tiles) and
    tile_group int32 [moe_sorted_tiles(...)] (each tile's expert)."""
    pairs = ids.numel()
    if slot.numel() != pairs or tile_group.numel() < moe_sorted_tiles(pairs, num_experts):
        raise KernelError("moe_sort: outputs do not fit")
    _check(lib().llb_moe_sort(_i32(ids, "ids"), pairs, num_experts, MOE_TILE_ROWS, tile_group.numel(), _i32(slot, "slot"),
                              _i32(tile_group, "tile_group"), _stream()))


def moe_gather(x: torch.Tensor, slot: torch.Tensor, top: int, xs: torch.Tensor) -> None:
    """xs[slot[i]] = x[i // top] for the T*top pairs."""
    T, D = x.shape
    if slot.numel() != T * top or xs.dtype != x.dtype or xs.shape[1] != D:
        raise KernelError("moe_gather: sizes do not fit")
    _check(lib().llb_moe_gather(_ptr(x), _dt(x), _i32(slot, "slot"), T * top, top, D, _ptr(xs), _stream()))


def moe_combine(y: Optional[torch.Tensor], slot: Optional[torch.Tensor], weights: Optional[torch.Tensor],
                residual: torch.Tensor, x: Optional[torch.Tensor] = None,
                identity_weight: Optional[torch.Tensor] = None) -> None:
    """residual[t] += sum_k weights[t, k] * y[slot[t*top + k]] in float (a negative slot is skipped), then
    ``+ identity_weight[t] * x[t]`` when identity experts exist.  ``y`` None: the identity term alone."""
    T, D = residual.shape
    if residual.dtype != torch.float32:
        raise KernelError("moe_combine: the stream is float32")
    top = 0
    if y is not None:
        top = weights.shape[1]
        if y.dtype != torch.float32 or y.shape[1] != D or slot.numel() != T * top:
            raise KernelError("moe_combine: sizes do not fit")
    if (x is None) != (identity_weight is None) or (x is not None and (tuple(x.shape) != (T, D) or identity_weight.numel() != T)):
        raise KernelError("moe_combine: the identity term needs x [T, D] and float32 [T] weights")
    _check(lib().llb_moe_combine_identity(_f32(y, "y"), _i32(slot, "slot"), _f32(weights, "weights"), T, top, D,
                                          _f32(residual, "residual"), _ptr(x), _dt(x) if x is not None else 0,
                                          _f32(identity_weight, "identity_weight"), _stream()))


def moe_pairs(x: torch.Tensor, ids: torch.Tensor, w_gate_up: torch.Tensor, w_down_rows: torch.Tensor, act: torch.Tensor,
              y: torch.Tensor, glu=None) -> None:
    """The chosen experts of a few rows, pair by pair (bfloat16): ``y[t*top + k] = W_down[e] (silu(W_gate[e] x_t) *
    (W_up[e] x_t))`` with e = ids[t, k]; ``w_gate_up`` [E*2F, D] (gate and up rows interleaved), ``w_down_rows`` [E*D, F];
    ``act`` bfloat16 [T*top, F] scratch; ``y`` float32 [T*top, D]."""
    T, D = x.shape
    pairs, top = ids.numel(), ids.shape[1]
    F = w_down_rows.shape[1]
    if x.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16 or w_down_rows.dtype != torch.bfloat16 or \
            w_gate_up.shape[1] != D or tuple(act.shape) != (pairs, F) or act.dtype != torch.bfloat16 or \
            tuple(y.shape) != (pairs, D) or y.dtype != torch.float32 or pairs != T * top:
        raise KernelError("moe_pairs: sizes or dtypes do not fit")
    _check(lib().llb_moe_pairs_glu(_ptr(x), _i32(ids, "ids"), pairs, top, D, F, _ptr(w_gate_up), _ptr(w_down_rows), _ptr(act),
                                   _f32(y, "y"), *_glu_args(glu), _stream()))


def gemm_tcgen05_grouped(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, groups: int,
                         tile_group: torch.Tensor, glu=None) -> None:
    """out[m] = epilogue(a[m] @ w[g(m)]^T): ``w`` is [groups * N, K], the rows of ``a`` are sorted by group with every
    group starting at a multiple of 128 rows, ``tile_group`` int32 names each 128-row tile's group.  bfloat16 operands,
    more than 128 rows; epilogues STORE, STORE_F32, SWIGLU."""
    M, K = a.shape
    if w.shape[1] != K or w.shape[0] % groups or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"gemm_tcgen05_grouped: a {tuple(a.shape)} {a.dtype}, w {tuple(w.shape)} {w.dtype}, {groups} groups")
    N = w.shape[0] // groups
    cols = N // 2 if epilogue == EPI_SWIGLU else N
    want = torch.float32 if epilogue == EPI_STORE_F32 else torch.bfloat16
    if tuple(out.shape) != (M, cols) or out.dtype != want or tile_group.numel() < -(-M // MOE_TILE_ROWS):
        raise KernelError("gemm_tcgen05_grouped: the output or the tiles' groups do not fit")
    _check(lib().llb_gemm_tcgen05_grouped(_ptr(a), _ptr(w), _ptr(out), epilogue, M, N, K, groups, _i32(tile_group, "tile_group"),
                                          _ptr(async_error_flag(a.device)), *_glu_args(glu), _stream()))


DEPI_STORE_F32, DEPI_RESIDUAL, DEPI_SWIGLU, DEPI_ROPE_KV = 1, 2, 3, 4


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, transposed: bool = False) -> torch.Tensor:
    """(cos, sin) of ``positions[t] * inv_freq[i]`` as float32 ``[T, len(inv_freq), 2]``, or pair-major
    ``[len(inv_freq), T, 2]`` with ``transposed``."""
    T, half = positions.numel(), inv_freq.numel()
    shape = (half, T, 2) if transposed else (T, half, 2)
    out = torch.empty(shape, dtype=torch.float32, device=positions.device)
    _check(lib().llb_rope_table(_i32(positions, "positions"), _ptr(inv_freq), _ptr(out), T, half,
                                1 if transposed else 0, _stream()))
    return out


_splitk = {}
_splitk_retired = []     # meeting places that a larger one replaced: CUDA graphs captured earlier still use them


def reserve_splitk_scratch(device: torch.device, floats: int, tiles: int) -> None:
    """Make sure the device has a zeroed meeting place of ``floats`` floats and ``tiles`` counters for
    split-K contractions with fused epilogues.  Call it when a model is bound, never inside a step.
    A meeting place that a larger one replaces is kept alive (and zero, as every launch leaves it): a graph
    captured while it was current goes on adding into it."""
    key = torch.device(device).index or 0
    have = _splitk.get(key)
    if have is None or have[0].numel() < floats or have[1].numel() < tiles:
        floats = max(floats, have[0].numel() if have else 0)
        tiles = max(tiles, have[1].numel() if have else 0)
        if have is not None:
            _splitk_retired.append(have)
        _splitk[key] = (torch.zeros(floats, dtype=torch.float32, device=device),
                        torch.zeros(tiles, dtype=torch.int32, device=device))


def splitk_scratch(device: torch.device):
    return _splitk.get(torch.device(device).index or 0)


def gemm_decode_supports(M: int, N: int, K: int, norm: bool, epilogue: int, head_dim: int = 0) -> bool:
    return bool(lib().llb_gemm_decode_supports(M, N, K, 1 if norm else 0, epilogue, head_dim))


def gemm_decode(w: torch.Tensor, epilogue: int, M: int, *, a: Optional[torch.Tensor] = None,
                x: Optional[torch.Tensor] = None, x_rows: Optional[torch.Tensor] = None,
                norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, split_k: int = 1,
                slot_mapping: Optional[torch.Tensor] = None,
                rope_table: Optional[torch.Tensor] = None, rotary_dim: int = 0, interleaved: bool = False,
                num_heads: int = 0, num_kv_heads: int = 0, head_dim: int = 0, q_out: Optional[torch.Tensor] = None,
                k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None) -> None:
    """The fused contraction of a step with at most 64 rows (see csrc/gemm_decode.cu).

    Operand: ``a`` [M, K] bf16, or the float rows ``x[x_rows]`` (``x[:M]`` without ``x_rows``) to be
    RMS-normalised with ``norm_weight`` and ``eps`` inside the kernel.  Epilogues: DEPI_STORE_F32
    (``out`` float [M, N]), DEPI_RESIDUAL (adds into ``residual``), DEPI_SWIGLU (``out`` bf16 [M, N/2]),
    DEPI_ROPE_KV (rotary by ``rope_table`` from :func:`rope_table`, ``q_out`` and the cache rows ``slot_mapping``)."""
    N, K = w.shape
    if w.dtype != torch.bfloat16:
        raise KernelError("gemm_decode takes bfloat16 weights")
    norm = x is not None
    if norm:
        if x.dtype != torch.float32 or x.shape[-1] != K or norm_weight is None or norm_weight.numel() != K:
            raise KernelError("gemm_decode: the normalised operand must be float32 [*, K] with a weight of K")
    elif a is None or a.dtype != torch.bfloat16 or tuple(a.shape) != (M, K):
        raise KernelError(f"gemm_decode: a must be bfloat16 [{M},{K}]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError(f"gemm_decode: bias must be float32 [{N}]")
    if epilogue == DEPI_RESIDUAL and (residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N)):
        raise KernelError(f"gemm_decode: residual must be float32 [{M},{N}]")
    if epilogue == DEPI_STORE_F32 and (out is None or out.dtype != torch.float32 or tuple(out.shape) != (M, N)):
        raise KernelError(f"gemm_decode: out must be float32 [{M},{N}]")
    if epilogue == DEPI_SWIGLU and (out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N // 2)):
        raise KernelError(f"gemm_decode: out must be bfloat16 [{M},{N // 2}]")
    if epilogue == DEPI_ROPE_KV:
        if q_out is None or q_out.dtype != torch.bfloat16 or q_out.numel() != M * num_heads * head_dim:
            raise KernelError("gemm_decode: q_out does not fit")
        if rotary_dim and (rope_table is None or rope_table.dtype != torch.float32
                           or rope_table.numel() != M * rotary_dim):
            raise KernelError("gemm_decode: rope_table must be float32 [M, rotary_dim/2, 2]")
        if slot_mapping is not None and (k_cache is None or v_cache is None or k_cache.dtype != torch.bfloat16):
            raise KernelError("gemm_decode: the cache must be bfloat16")
    scratch = splitk_scratch(w.device) if (split_k > 1 and epilogue in (DEPI_SWIGLU, DEPI_ROPE_KV)) else None
    if scratch is not None and scratch[1].numel() < -(-N // 128):
        scratch = None
    _check(lib().llb_gemm_decode(
        _ptr(w), _ptr(a), _ptr(x), _i32(x_rows, "x_rows"), _ptr(norm_weight),
        1 if (norm_weight is not None and norm_weight.dtype == torch.bfloat16) else 0, ctypes.c_float(eps),
        1 if norm else 0, _ptr(bias), _ptr(out), _ptr(residual), epilogue, M, N, K, split_k,
        _i32(slot_mapping, "slot_mapping"), _ptr(rope_table), rotary_dim,
        1 if interleaved else 0, num_heads, num_kv_heads, head_dim, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
        _ptr(scratch[0]) if scratch else ctypes.c_void_p(0), ctypes.c_longlong(scratch[0].numel() if scratch else 0),
        _ptr(scratch[1]) if scratch else ctypes.c_void_p(0), _ptr(async_error_flag(w.device)), _stream()))


def gemm_decode_glu(w: torch.Tensor, a: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, split_k: int,
                    glu) -> None:
    """The decode contraction's GLU epilogue with the gated activation ``glu`` (as :func:`gemm_simt`): ``a`` bf16 [M, K],
    ``w`` bf16 [N, K] with (gate, up) rows interleaved, ``out`` bf16 [M, N/2]."""
    N, K = w.shape
    M = a.shape[0]
    if w.dtype != torch.bfloat16 or a.dtype != torch.bfloat16 or tuple(a.shape) != (M, K) \
            or out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N // 2):
        raise KernelError("gemm_decode_glu: bfloat16 a [M,K], w [N,K] and out [M,N/2]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError(f"gemm_decode_glu: bias must be float32 [{N}]")
    scratch = splitk_scratch(w.device) if split_k > 1 else None
    if scratch is not None and (scratch[1].numel() < -(-N // 128) or scratch[0].numel() < 64 * N):
        scratch = None
    if scratch is None:          # no meeting place was reserved for a contraction this wide: one piece
        split_k = 1
    _check(lib().llb_gemm_decode_glu(
        _ptr(w), _ptr(a), _ptr(bias), _ptr(out), M, N, K, split_k,
        _ptr(scratch[0]) if scratch else ctypes.c_void_p(0), ctypes.c_longlong(scratch[0].numel() if scratch else 0),
        _ptr(scratch[1]) if scratch else ctypes.c_void_p(0), _ptr(async_error_flag(w.device)), *_glu_args(glu), _stream()))


def attention_tcgen05_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().llb_attention_tcgen05_supports(head_dim, page_size))


def paged_attention_tcgen05(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                            tile_span: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int,
                            span_row: torch.Tensor, span_len: torch.Tensor, span_pos: torch.Tensor,
                            block_table: torch.Tensor, max_pages: int, page_size: int,
                            num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                            cut=None, sinks: Optional[torch.Tensor] = None, cross: int = 1, softcap: float = 0.0) -> None:
    """Tensor-core attention of the listed tiles (128 query rows each) over the requests' pages; bf16.
    ``sinks`` float32 [num_heads]: ``exp(sinks[h])`` joins head h's softmax denominator once; ``v_cache`` may be
    ``k_cache`` itself (values read out of the key rows).  ``cross`` = ``num_kv_heads`` (> 1): crossed values, ``out``
    is [T, num_heads, cross, head_dim] and holds every query head's weights applied to the values of every kv
    head; ``cut`` must then have been made for ``num_heads * cross`` heads.  ``out`` may be float32.  ``softcap`` > 0: a
    score becomes ``softcap * tanh(score / softcap)`` before the softmax.

    ``cut`` = ``(tile_k0, tile_nk, tile_part, num_parts, merge_span, merge_q0, merge_first, merge_count,
    num_merge)`` cuts long key ranges into items (see ``StepContext.attention_items``); the partial results
    are merged by a second kernel."""
    for t in (q, k_cache, v_cache):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_tcgen05 takes bfloat16 tensors")
    if out.dtype not in (torch.bfloat16, torch.float32) or out.numel() != q.shape[0] * num_heads * cross * head_dim:
        raise KernelError("attention_tcgen05: out is bfloat16 or float32 [T, heads, cross, head_dim]")
    out_float = 1 if out.dtype == torch.float32 else 0
    T = q.shape[0]
    num_slots = k_cache.shape[0]
    k0 = nk = part = scratch = None
    num_parts = 0
    if cut is not None:
        k0, nk, part, num_parts = cut[0], cut[1], cut[2], cut[3]
        if num_parts:
            scratch = torch.empty(num_parts * num_heads * cross * 128 * (head_dim + 2), dtype=torch.float32,
                                  device=q.device)
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_heads):
        raise KernelError(f"attention_tcgen05: sinks must be float32 [{num_heads}]")
    _check(lib().llb_paged_attention_tcgen05_capped(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), T,
        _i32(tile_span, "tile_span"), _i32(tile_q0, "tile_q0"), num_tiles,
        _i32(span_row, "span_row"), _i32(span_len, "span_len"), _i32(span_pos, "span_pos"),
        _i32(block_table, "block_table"), max_pages, page_size, num_slots, num_heads, num_kv_heads, head_dim,
        window, ctypes.c_float(scale), ctypes.c_float(softcap or 0.0), _i32(k0, "tile_k0"), _i32(nk, "tile_nk"), _i32(part, "tile_part"),
        _ptr(scratch), num_parts, _ptr(sinks), cross, out_float, _ptr(async_error_flag(q.device)), _stream()))
    if cut is not None and num_parts:
        _check(lib().llb_attention_tcgen05_merge_cross(
            _ptr(out), _i32(cut[4], "merge_span"), _i32(cut[5], "merge_q0"), _i32(cut[6], "merge_first"),
            _i32(cut[7], "merge_count"), cut[8], _i32(span_row, "span_row"), _i32(span_len, "span_len"),
            _ptr(scratch), num_parts, num_heads, head_dim, _ptr(sinks), cross, out_float, _stream()))


def paged_decode_mma_supports(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return bool(lib().llb_paged_decode_mma_supports(num_heads, num_kv_heads, head_dim))


_cluster_splits: Optional[int] = None


_decode_resident = {}


def decode_mma_resident(head_dim: int) -> int:
    """Blocks of the decode attention kernel that one SM holds at a time for this head size."""
    n = _decode_resident.get(head_dim)
    if n is None:
        n = int(lib().llb_paged_decode_mma_resident(head_dim))
        if n <= 0:
            raise KernelError(lib().llb_last_error().decode("utf-8", "replace"))
        _decode_resident[head_dim] = n
    return n


def decode_mma_cluster_splits() -> int:
    """Up to this many splits the decode attention merges inside the kernel (a thread-block cluster); more
    need scratch and the merge kernel."""
    global _cluster_splits
    if _cluster_splits is None:
        _cluster_splits = int(lib().llb_paged_decode_mma_cluster_splits())
    return _cluster_splits


def paged_decode_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     tile_span: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int, span_row: torch.Tensor,
                     span_pos: torch.Tensor, block_table: torch.Tensor, max_pages: int, page_size: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                     nsplit: int = 1, scratch: Optional[torch.Tensor] = None,
                     sinks: Optional[torch.Tensor] = None, cross: int = 1, softcap: float = 0.0) -> None:
    """Tensor-core decode attention: one query row per tile over its request's pages; bf16.  ``nsplit`` cuts
    each request's keys; up to :func:`decode_mma_cluster_splits` the pieces are merged inside the kernel.
    ``sinks``, ``v_cache is k_cache``, ``cross`` (crossed values), ``softcap`` and a float32 ``out`` as
    :func:`paged_attention_tcgen05`."""
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_heads):
        raise KernelError(f"decode attention: sinks must be float32 [{num_heads}]")
    for t in (q, k_cache, v_cache):
        if t.dtype != torch.bfloat16:
            raise KernelError("paged_decode_mma takes bfloat16 tensors")
    if out.dtype not in (torch.bfloat16, torch.float32) or out.numel() != q.shape[0] * num_heads * cross * head_dim:
        raise KernelError("decode attention: out is bfloat16 or float32 [T, heads, cross, head_dim]")
    if nsplit > decode_mma_cluster_splits():
        need = attention_scratch_floats(num_tiles, num_heads * cross, head_dim, 1, nsplit)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"decode attention: nsplit={nsplit} needs {need} floats of scratch")
    _check(lib().llb_paged_decode_mma_capped(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _i32(tile_span, "tile_span"), _i32(tile_q0, "tile_q0"),
        num_tiles, _i32(span_row, "span_row"), _i32(span_pos, "span_pos"), _i32(block_table, "block_table"),
        max_pages, page_size, num_heads, num_kv_heads, head_dim, window, ctypes.c_float(scale),
        ctypes.c_float(softcap or 0.0), nsplit,
        _ptr(scratch), _ptr(sinks), cross, 1 if out.dtype == torch.float32 else 0, _stream()))


# Where the blocks that share a long row of logits meet (a 64-bit slot and a counter per row), per device.
_ARGMAX_ROWS = 4096
_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the largest logit of row r.  logits float32 [R,V]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with unit inner stride")
    if not logits.is_cuda:
        raise KernelError("argmax: logits are not on a CUDA device; there is no CPU path")
    key = logits.device.index or 0
    scratch = _argmax_scratch.get(key)
    if scratch is None:          # zero once: every launch leaves it zero
        scratch = _argmax_scratch[key] = torch.zeros(3 * _ARGMAX_ROWS, dtype=torch.int32, device=logits.device)
    _check(lib().llb_argmax(ctypes.c_void_p(logits.data_ptr()), R, V, ctypes.c_longlong(logits.stride(0)),
                            _i32(out, "out"), _ptr(scratch), _ARGMAX_ROWS, _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], min_p: Optional[torch.Tensor], uniform: torch.Tensor,
           out: torch.Tensor) -> None:
    """One token per row from softmax(logits / temperature) after the top-k/top-p/min-p filters."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or not logits.is_cuda:
        raise KernelError("sample: logits must be float32 on a CUDA device with unit inner stride")
    for name, t in (("temperature", temperature), ("top_p", top_p), ("min_p", min_p), ("uniform", uniform)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != R):
            raise KernelError(f"sample: {name} must be float32 [{R}]")
    _check(lib().llb_sample(ctypes.c_void_p(logits.data_ptr()), R, V, ctypes.c_longlong(logits.stride(0)),
                            _ptr(temperature), _i32(top_k, "top_k"), _ptr(top_p), _ptr(min_p), _ptr(uniform),
                            _i32(out, "out"), _stream()))


def launch_count() -> int:
    """Kernels this library has launched in this process."""
    return int(lib().llb_launch_count())


def has_tcgen05() -> bool:
    """Whether the library carries the tcgen05 tensor-core contraction."""
    return hasattr(lib(), "llb_gemm_tcgen05")


_async_err = {}


def async_error_flag(device: torch.device) -> torch.Tensor:
    """One int32 on the device that kernels with bounded waits raise when a wait ran out."""
    key = torch.device(device).index or 0
    t = _async_err.get(key)
    if t is None:
        t = _async_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


_reset_on_error = []      # counters that a kernel leaves in an unknown state when it gives up; cleared with the flag


def check_async_errors(device: torch.device) -> None:
    """Synchronises and raises if a kernel gave up on a wait (its output is then invalid)."""
    t = async_error_flag(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        for counters in _reset_on_error:
            if counters.device == t.device:
                counters.zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting on a barrier (code {code}); its results are invalid")


# ---- the layers of a decode step as one persistent kernel (csrc/decode_layers.cu) -----------------------------------
MAX_FUSED_GROUPS = 4
MAX_FUSED_SPLITS = 32


def decode_layers_supports(M: int, D: int, Hq: int, Hkv: int, hd: int, I: int, rotary_dim: int) -> bool:
    return bool(lib().llb_decode_layers_supports(M, D, Hq, Hkv, hd, I, rotary_dim))


def decode_layers_descriptors(layers, D: int, Hq: int, Hkv: int, hd: int, I: int, device) -> torch.Tensor:
    """The device array of layer descriptors for :func:`decode_layers`.  ``layers``: one dict per layer with the
    tensors ``w_qkv``, ``w_o``, ``w_gate_up``, ``w_down``, ``b_qkv`` (or None), ``norm1_w``, ``norm2_w``, ``k_cache``,
    ``v_cache`` and the numbers ``eps1``, ``eps2``, ``window`` (0: none), ``group``.  The tensors must stay alive and
    in place as long as the descriptors are used."""
    import numpy as np
    size = int(lib().llb_decode_layers_desc_bytes())
    host = np.zeros(len(layers) * size, dtype=np.uint8)
    for i, d in enumerate(layers):
        for name in ("w_qkv", "w_o", "w_gate_up", "w_down"):
            if d[name].dtype != torch.bfloat16:
                raise KernelError(f"decode_layers: {name} must be bfloat16")
        if d["norm1_w"].dtype != d["norm2_w"].dtype or d["norm1_w"].dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("decode_layers: the two norm weights must share a dtype (bfloat16 or float32)")
        if d["k_cache"].dtype != torch.bfloat16 or (d["b_qkv"] is not None and d["b_qkv"].dtype != torch.float32):
            raise KernelError("decode_layers: the cache must be bfloat16 and the bias float32")
        _check(lib().llb_decode_layers_describe(
            host.ctypes.data + i * size, _ptr(d["w_qkv"]), _ptr(d["w_o"]), _ptr(d["w_gate_up"]), _ptr(d["w_down"]),
            _ptr(d["b_qkv"]), _ptr(d["norm1_w"]), _ptr(d["norm2_w"]), 1 if d["norm1_w"].dtype == torch.bfloat16 else 0,
            ctypes.c_float(d["eps1"]), ctypes.c_float(d["eps2"]), _ptr(d["k_cache"]), _ptr(d["v_cache"]),
            int(d["window"] or 0), int(d["group"]), D, Hq, Hkv, hd, I))
    return torch.from_numpy(host).to(device)


def decode_layers_scratch_floats(M: int, Hq: int, Hkv: int, hd: int, I: int, nsplit: int) -> int:
    return int(lib().llb_decode_layers_scratch_floats(M, Hq, Hkv, hd, I, nsplit))


def decode_layers_counters(device) -> torch.Tensor:
    """The two counters on which the blocks of :func:`decode_layers` meet (zero between launches)."""
    t = torch.zeros(2, dtype=torch.int32, device=device)
    _reset_on_error.append(t)
    return t


def decode_layers(descriptors: torch.Tensor, num_layers: int, residual: torch.Tensor, D: int, Hq: int, Hkv: int, hd: int,
                  I: int, rotary_dim: int, interleaved: bool, scale: float, rope_table: Optional[torch.Tensor],
                  span_pos: torch.Tensor, block_tables, slot_mappings, max_pages: int, page_size: int, nsplit: int,
                  scratch: torch.Tensor, counters: torch.Tensor, timeline: Optional[torch.Tensor] = None,
                  timeline_block: int = 0) -> None:
    """All layers of a decode step (one token per request, at most 64) in one persistent kernel, in place on the
    float32 ``residual`` [M, D].  ``block_tables`` / ``slot_mappings``: one int32 tensor per cache group (up to 4).
    ``timeline`` (int64, 2 * (2 + 64 * layers) words) receives the milestones of block ``timeline_block`` as (label, SM cycle) pairs."""
    M = residual.shape[0]
    if residual.dtype != torch.float32 or tuple(residual.shape) != (M, D):
        raise KernelError(f"decode_layers: residual must be float32 [{M},{D}]")
    if len(block_tables) > MAX_FUSED_GROUPS or len(block_tables) != len(slot_mappings):
        raise KernelError(f"decode_layers: at most {MAX_FUSED_GROUPS} cache groups")
    bts = [_i32(t, "block_table") for t in block_tables] + [None] * (MAX_FUSED_GROUPS - len(block_tables))
    sms = [_i32(t, "slot_mapping") for t in slot_mappings] + [None] * (MAX_FUSED_GROUPS - len(slot_mappings))
    if scratch.dtype != torch.float32:
        raise KernelError("decode_layers: scratch must be float32")
    _check(lib().llb_decode_layers(
        _ptr(descriptors), num_layers, _ptr(residual), M, D, Hq, Hkv, hd, I, rotary_dim, 1 if interleaved else 0,
        ctypes.c_float(scale), _ptr(rope_table), _i32(span_pos, "span_pos"), *bts, *sms, max_pages, page_size, nsplit,
        _ptr(scratch), scratch.numel(), _ptr(counters), _ptr(async_error_flag(residual.device)), _ptr(timeline),
        timeline_block, _stream()))


def selftest_wait_expires(device: torch.device, limit_cycles: int = 1_000_000) -> torch.Tensor:
    """Run the library's self-test block whose waits nothing ever satisfies (csrc/selftest.cu): afterwards
    :func:`check_async_errors` raises.  Returns the two roles' outcomes (2 = left its wait unsatisfied)."""
    trace = torch.zeros(2, dtype=torch.int32, device=device)
    _check(lib().llb_selftest_wait_expires(_ptr(async_error_flag(device)), _ptr(trace), limit_cycles, _stream()))
    return trace


def selftest_mma_issue(device: torch.device, n: int = 64, a_tmem: bool = False, neighbours: int = 0, kind: int = 1,
                       iters: int = 256) -> dict:
    """The microbenchmark of csrc/selftest.cu: cycles that one thread needs to issue ``4 * iters`` tcgen05.mma of
    128 x n x 16 beside ``neighbours`` busy warps (kind 1: FMA chains, 2: softmax-like), and for the commit."""
    out = torch.zeros(4, dtype=torch.int64, device=device)
    _check(lib().llb_selftest_mma_issue(_ptr(out), n, int(a_tmem), neighbours, kind, iters, _stream()))
    issue, commit, arrive, _ = out.tolist()
    return {"cycles_per_mma": issue / (4 * iters), "commit_cycles": commit, "arrive_cycles": arrive}


_meet_counters = {}
_MEET_COUNTERS = 1 << 16


def meet_counters(device: torch.device) -> torch.Tensor:
    """The device's counters of wide split contractions (zero before and after every launch), made on first use."""
    key = torch.device(device).index or 0
    counters = _meet_counters.get(key)
    if counters is None:
        counters = _meet_counters[key] = torch.zeros(_MEET_COUNTERS, dtype=torch.int32, device=device)
    return counters


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
                 out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 split_k: int = 1, glu=None) -> None:
    """Tensor-core contraction a[M,K] @ w[N,K]^T (bf16, K a multiple of 8) with a fused epilogue (``glu`` as :func:`gemm_simt`).

    ``split_k`` > 1 cuts K into pieces that run as separate work items: up to 128 rows for the residual
    epilogue only (atomic adds); beyond, for every epilogue, through a meeting place in which the piece that
    arrives last adds all pieces in their order (the result does not depend on who arrives last)."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: a is {tuple(a.shape)} but w is {tuple(w.shape)}")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05 takes bfloat16 operands")
    _check_epilogue_args(a, N, M, bias, epilogue, out, residual)
    partials = counters = None
    if split_k > 1 and M > 128:
        need = lib().llb_gemm_tcgen05_counters(M, N, split_k)
        if need > _MEET_COUNTERS:
            split_k = 1
        else:
            counters = meet_counters(a.device)
            partials = torch.empty(lib().llb_gemm_tcgen05_partial_floats(M, N, split_k), dtype=torch.float32,
                                   device=a.device)
    _check(lib().llb_gemm_tcgen05_glu(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), epilogue, M, N, K,
                                      split_k, _ptr(partials), _ptr(counters), _ptr(async_error_flag(a.device)),
                                      *_glu_args(glu), _stream()))


def gemm_tcgen05_rope(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], rope_table: torch.Tensor,
                      slot_mapping: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int = 64) -> None:
    """The q/k/v projection with heads of 64 or 128: a[M,K] @ w[N,K]^T, bias, NeoX rotation of the whole head by
    ``rope_table`` [hd/2, M, 2] (cos, sin; pair-major), q to ``q_out`` [M, Hq*hd], k and v to the cache rows
    ``slot_mapping`` [M] of ``k_cache`` / ``v_cache`` [slots, Hkv, hd] (a negative slot writes nothing)."""
    M, K = a.shape
    N, K2 = w.shape
    hd = head_dim
    if hd not in (64, 128) or K != K2 or N != (num_heads + 2 * num_kv_heads) * hd:
        raise KernelError(f"gemm_tcgen05_rope: a {tuple(a.shape)}, w {tuple(w.shape)}, heads {num_heads}/{num_kv_heads} of {hd}")
    for t, name in ((a, "a"), (w, "w"), (q_out, "q_out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"gemm_tcgen05_rope: {name} must be contiguous bfloat16")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_rope: bias must be float32 of length N")
    if rope_table.dtype != torch.float32 or rope_table.numel() != M * hd or not rope_table.is_contiguous():
        raise KernelError("gemm_tcgen05_rope: rope_table must be float32 [hd/2, M, 2]")
    if slot_mapping.dtype != torch.int32 or slot_mapping.numel() != M:
        raise KernelError("gemm_tcgen05_rope: slot_mapping must be int32 [M]")
    if tuple(q_out.shape) != (M, num_heads * hd) or k_cache.shape[-1] != hd or k_cache.shape[-2] != num_kv_heads \
            or v_cache.shape != k_cache.shape:
        raise KernelError("gemm_tcgen05_rope: q_out must be [M, Hq*hd] and the caches [..., Hkv, hd]")
    _check(lib().llb_gemm_tcgen05_rope(_ptr(a), _ptr(w), _ptr(bias), M, N, K, _ptr(rope_table), _ptr(slot_mapping),
                                       _ptr(q_out), _ptr(k_cache), _ptr(v_cache), num_heads, num_kv_heads, hd,
                                       _ptr(async_error_flag(a.device)), _stream()))


def gemm_tcgen05_rope64(a, w, bias, rope_table, slot_mapping, q_out, k_cache, v_cache, num_heads, num_kv_heads) -> None:
    """:func:`gemm_tcgen05_rope` at heads of 64."""
    gemm_tcgen05_rope(a, w, bias, rope_table, slot_mapping, q_out, k_cache, v_cache, num_heads, num_kv_heads, 64)
