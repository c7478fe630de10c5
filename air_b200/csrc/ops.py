"""Python faces of the CUDA kernels.  Every function checks what it is given (device,
dtype, shape, contiguity), launches on torch's current stream and raises on any error
code.  There is no other implementation behind these functions: if the library cannot be
built or loaded, or a tensor is not on a CUDA device, they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build

_DT = {torch.float32: 0, torch.bfloat16: 1}
c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_SIGNATURES = {
    "air_embedding": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "air_bigram_embedding": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p,
                             c_void_p],
    "air_remember_tokens": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "air_stream_add": [c_void_p, c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    "air_add_parts": [c_void_p, c_void_p, c_int, c_int, c_longlong, c_void_p],
    "air_add_prenorm": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "air_logits_post": [c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p],
    "air_add_rmsnorm": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                        c_longlong, c_float, c_void_p],
    "air_qkv_rope_store": [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "air_silu_mul": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "air_convert": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p],
    "air_gemm_f32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "air_paged_attention_ref": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p,
                                c_int, c_void_p],
    "air_post_norm": [c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int,
                      c_void_p, c_int, c_int, c_int, c_float, c_void_p],
    "air_qk_normed_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_float, c_void_p,
                              c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_void_p, c_void_p, c_int, c_void_p],
    "air_latent_prepare": [c_void_p, c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                           c_void_p, c_void_p],
    "air_grouped_attention": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int, c_int,
                              c_float, c_void_p, c_int, c_void_p],
    "air_gather_keys": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                        c_void_p, c_void_p],
    "air_masked_softmax": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                           c_void_p, c_float, c_void_p],
    "air_moe_route": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                      c_int, c_float, c_float, c_void_p, c_void_p],
    "air_moe_identity": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "air_normed_add_norm": [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_void_p, c_void_p, c_int,
                            c_void_p, c_int, c_int, c_float, c_void_p],
    "air_relu2": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p],
    "air_sigmoid_gate": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    "air_moe_sort": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "air_grouped_gemm": [c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p, c_longlong,
                         c_void_p, c_longlong, c_longlong, c_void_p, c_int, c_longlong, c_int, c_int, c_void_p, c_int,
                         c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "air_rows_by_index": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "air_planes_by_index": [c_void_p, c_int, c_void_p, c_int, c_longlong, c_void_p, c_void_p, c_int, c_int, c_void_p],
    "air_qkv_prepare": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                        c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_void_p, c_void_p],
    "air_short_conv_silu": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_int, c_int, c_void_p],
    "air_linear_scan": [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_float, c_void_p,
                        c_void_p, c_int, c_float, c_void_p],
    "air_gated_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float,
                          c_void_p],
    "air_polynorm": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float,
                     c_float, c_void_p],
    "air_glu": [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p],
    "air_scaled_norm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_int,
                        c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
    "air_table_update": [c_void_p, c_void_p, c_int, c_int, c_void_p],
    "air_decode_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    "air_prefill_attention": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                              c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "air_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float,
                    c_float, c_float, c_void_p],
    "air_gemm_tc_small": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                          c_void_p, c_int, c_float, c_float, c_float, c_float, c_void_p],
    "air_decode_attention_tma": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p,
                                 c_void_p],
    "air_decode_attention_tma_sink": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
                                      c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "air_head_gate": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "air_decode_attention_tma_fresh": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                       c_int, c_int, c_float, c_int, c_void_p, c_void_p],
    "air_prefill_attention_tc": [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,
                                 c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p],
    "air_prefill_attention_tc_sink": [c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                      c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                      c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p],
    "air_sample": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                   c_void_p, c_void_p],
}

_fn = {}
launches = 0   # kernels of this library launched so far (each wrapper launches one)


class KernelError(RuntimeError):
    pass


def _get(name):
    f = _fn.get(name)
    if f is None:
        lib = build.library()
        f = getattr(lib, name)
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _fn[name] = f
    return f


def set_pdl(on: bool) -> None:
    """Whether kernels are launched so that they may overlap the tail of their predecessor."""
    lib = build.library()
    lib.air_set_pdl.argtypes = [c_int]
    lib.air_set_pdl.restype = None
    lib.air_set_pdl(1 if on else 0)


TRACE_NAMES = {1: "embedding", 2: "add_rmsnorm", 3: "qkv_rope_store", 4: "silu_mul", 5: "convert", 6: "table_update",
               7: "attention_ref", 8: "decode_attention", 9: "decode_combine", 10: "prefill_attention", 11: "gemm_f32",
               12: "gemm_tc", 13: "sample", 14: "short_conv", 15: "linear_scan", 16: "gated_rmsnorm",
               17: "qkv_prepare", 18: "glu", 19: "scaled_norm", 20: "post_norm", 21: "qk_normed_prepare",
               22: "latent_prepare", 23: "moe_route", 24: "moe_sort", 25: "grouped_gemm", 26: "gather_keys", 27: "masked_softmax", 28: "grouped_attention", 29: "polynorm", 30: "stream_add", 31: "head_gate",
               32: "normed_add_norm", 33: "relu2"}


def set_trace(buffer: Optional[torch.Tensor]) -> None:
    """buffer: int64 CUDA tensor of 1 + 2 * 16384 elements (zeroed), or None to stop tracing.  While set,
    block 0 of every kernel appends (kernel id, GPU nanosecond timer) after its wait on its predecessor;
    element 0 counts the entries.  Differences of consecutive times are the kernels' spans in a graph."""
    lib = build.library()
    ptr = None if buffer is None else buffer.data_ptr()
    for src in build.sources():
        f = getattr(lib, "air_trace_set_" + src[:-3])
        f.argtypes, f.restype = [c_void_p], c_int
        rc = f(ptr)
        if rc:
            raise KernelError(f"set_trace: CUDA error {rc}")


def _check(code: int, name: str):
    global launches
    launches += 1
    if code != 0:
        if code == 100001:
            raise KernelError(f"{name}: a size or dtype that the kernel does not take")
        raise KernelError(f"{name}: CUDA error {code} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def _stream() -> int:
    """The current stream's handle (the stream that a graph capture or a stream context has made current).
    A step launches hundreds of kernels from Python, so this asks the runtime directly where it can."""
    global _device_index
    if _raw_stream is None:
        return torch.cuda.current_stream().cuda_stream
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return _raw_stream(_device_index)


def _req(t: torch.Tensor, name: str, dtypes=None, shape=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU implementation)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtypes is not None and t.dtype not in dtypes:
        raise KernelError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if shape is not None:
        got = t.shape
        if len(got) != len(shape):
            raise KernelError(f"{name} has shape {tuple(got)}, expected {tuple(shape)}")
        for s, g in zip(shape, got):
            if s is not None and s != g:
                raise KernelError(f"{name} has shape {tuple(got)}, expected {tuple(shape)}")
    return t


_FLOATS = (torch.float32, torch.bfloat16)
_I32 = (torch.int32,)


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def embedding(table, ids, out, status=None, last_token=None, multiplier=1.0):
    """out[t] = table[ids[t]] * multiplier as float32; an id -(s+1) is replaced by last_token[s]."""
    V, E = table.shape
    _req(table, "table", _FLOATS)
    _req(ids, "ids", _I32, (out.shape[0],))
    _req(out, "out", (torch.float32,), (None, E))
    if last_token is not None:
        _req(last_token, "last_token", _I32)
    _check(_get("air_embedding")(table.data_ptr(), _DT[table.dtype], ids.data_ptr(), _ptr(last_token),
                                 out.data_ptr(), out.shape[0], E, V, float(multiplier), _ptr(status), _stream()),
           "embedding")
    return out


def bigram_embedding(table, pairs, ids, positions, token_seq, previous, out, out2, resolved, buckets, mul_prev, mul_cur,
                     status=None, last_token=None):
    """out[t] = table[id] + pairs[(prev * mul_prev + id * mul_cur) % buckets] as float32 (pairs[buckets] at position
    0); prev is the row above where it belongs to the same request, else previous[slot, 0].  out2: a second copy or
    None.  resolved int32 [T] receives the ids used (an id -(s+1) is replaced by last_token[s])."""
    V, E = table.shape
    T = out.shape[0]
    _req(table, "table", _FLOATS)
    _req(pairs, "pairs", (table.dtype,), (buckets + 1, E))
    for name, x in (("ids", ids), ("positions", positions), ("token_seq", token_seq), ("resolved", resolved)):
        _req(x, name, _I32, (T,))
    _req(previous, "previous", _I32)
    _req(out, "out", (torch.float32,), (T, E))
    if out2 is not None:
        _req(out2, "out2", (torch.float32,), (T, E))
    if last_token is not None:
        _req(last_token, "last_token", _I32)
    _check(_get("air_bigram_embedding")(table.data_ptr(), pairs.data_ptr(), _DT[table.dtype], ids.data_ptr(),
                                        positions.data_ptr(), token_seq.data_ptr(), previous.data_ptr(),
                                        _ptr(last_token), out.data_ptr(), _ptr(out2), resolved.data_ptr(), T, E, V,
                                        int(buckets), int(mul_prev), int(mul_cur), _ptr(status), _stream()),
           "bigram_embedding")
    return out


def remember_tokens(resolved, q_start, slots, previous, entries):
    """previous[slots[e], 0] = resolved[q_start[e + 1] - 1] for every entry e of the step."""
    _req(resolved, "resolved", _I32)
    _req(q_start, "q_start", _I32)
    _req(slots, "slots", _I32)
    _req(previous, "previous", _I32)
    if q_start.shape[0] < entries + 1 or slots.shape[0] < entries:
        raise KernelError("remember_tokens: fewer entries than said")
    _check(_get("air_remember_tokens")(resolved.data_ptr(), q_start.data_ptr(), slots.data_ptr(), previous.data_ptr(),
                                       int(entries), _stream()), "remember_tokens")


def stream_add(h, again=None, row=None):
    """h += again + row: again float32 of h's shape or None, row float32 [E] (the same for every row of h) or None."""
    E = h.shape[-1]
    _req(h, "h", (torch.float32,), (None, E))
    if again is not None:
        _req(again, "again", (torch.float32,), tuple(h.shape))
    if row is not None:
        _req(row, "row", (torch.float32,), (E,))
    _check(_get("air_stream_add")(h.data_ptr(), _ptr(again), _ptr(row), E, h.numel(), _stream()), "stream_add")
    return h


def add_parts(h, delta):
    """h += delta in place (float32 h [T, E]); delta [T, E] or partial sums [parts, T, E], added in order."""
    _req(h, "h", (torch.float32,))
    parts = 1 if delta.dim() == h.dim() else delta.shape[0]
    _req(delta, "delta", _FLOATS, tuple(h.shape) if delta.dim() == h.dim() else (parts,) + tuple(h.shape))
    _check(_get("air_add_parts")(h.data_ptr(), delta.data_ptr(), _DT[delta.dtype], parts, h.numel(), _stream()),
           "add_parts")
    return h


PRENORM_CHUNK = 512


def add_prenorm(h, delta, weight, xg, ss):
    """h += delta in place (float32 h [T, E]; delta None, [T, E] or partial sums [parts, T, E]); xg =
    bfloat16(h * weight); ss[chunk, t] = the sum of h[t]^2 over a chunk of 512 columns.  What add_rmsnorm does, short
    of the scale per row (rsqrt(sum of a row's ss / E + eps)), which the product that takes xg applies (gemm_tc's
    row_ss): no block of this kernel waits for another."""
    T, E = h.shape
    _req(h, "h", (torch.float32,))
    parts = 0
    if delta is not None:
        parts = 1 if delta.dim() == 2 else delta.shape[0]
        _req(delta, "delta", _FLOATS, (T, E) if delta.dim() == 2 else (parts, T, E))
    _req(weight, "weight", _FLOATS, (E,))
    _req(xg, "xg", (torch.bfloat16,), (T, E))
    _req(ss, "ss", (torch.float32,), (-(-E // PRENORM_CHUNK), T))
    if E % 4:
        raise KernelError(f"add_prenorm: width {E} is not a multiple of 4")
    _check(_get("air_add_prenorm")(h.data_ptr(), _ptr(delta), _DT[delta.dtype] if delta is not None else 0, parts,
                                   weight.data_ptr(), _DT[weight.dtype], xg.data_ptr(), ss.data_ptr(), T, E,
                                   _stream()), "add_prenorm")
    return xg, ss


def logits_post(logits, bias=None, scale=1.0, softcap=0.0):
    """In place: logits = (logits + bias) * scale, then softcap * tanh(logits / softcap) where softcap > 0."""
    R, V = logits.shape
    _req(logits, "logits", (torch.float32,))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (V,))
    _check(_get("air_logits_post")(logits.data_ptr(), _ptr(bias), float(scale), float(softcap), R, V, _stream()),
           "logits_post")
    return logits


def add_rmsnorm(h, delta, weight, eps, out, rows=None):
    """Without rows: h += delta (in place, float32), out = rmsnorm(h) * weight.
    With rows: out[r] = rmsnorm(h[rows[r]] + delta[rows[r]]) * weight, h unchanged."""
    E = h.shape[-1]
    _req(h, "h", (torch.float32,), (None, E))
    parts = 0
    if delta is not None:
        # [rows, E], or [parts, rows, E]: partial sums that are added in order
        parts = 1 if delta.dim() == 2 else delta.shape[0]
        _req(delta, "delta", _FLOATS, tuple(h.shape) if delta.dim() == 2 else (parts,) + tuple(h.shape))
    _req(weight, "weight", _FLOATS, (E,))
    R = h.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _req(rows, "rows", _I32)
    _req(out, "out", _FLOATS, (R, E))
    _check(_get("air_add_rmsnorm")(h.data_ptr(), _ptr(delta), _DT[delta.dtype] if delta is not None else 0, parts,
                                   weight.data_ptr(), _DT[weight.dtype], out.data_ptr(), _DT[out.dtype],
                                   _ptr(rows), R, E, h.shape[0], float(eps), _stream()), "add_rmsnorm")
    return out


def qkv_rope_store(qkv, bias, table, positions, token_seq, block_table, q_out, cache, heads, kv_heads,
                   head_dim, write_kv=True, status=None):
    """Adds the bias, rotates q and k by the table's cos/sin of each token's position, writes
    q to q_out [T, H, d] and k, v into the pages (cache [page, 2, K, P, d])."""
    T = qkv.shape[-2]
    width = (heads + 2 * kv_heads) * head_dim
    parts = 1 if qkv.dim() == 2 else qkv.shape[0]     # [T, width], or [parts, T, width] partial sums
    _req(qkv, "qkv", _FLOATS, (T, width) if qkv.dim() == 2 else (parts, T, width))
    if bias is not None:
        _req(bias, "bias", _FLOATS, (width,))
    rot = 0
    if table is not None:
        _req(table, "table", (torch.float32,))
        rot = table.shape[1]
        if rot > head_dim or rot % 2:
            raise KernelError(f"rotary width {rot} does not fit head size {head_dim}")
    _req(positions, "positions", _I32, (T,))
    _req(token_seq, "token_seq", _I32, (T,))
    _req(block_table, "block_table", _I32)
    _req(q_out, "q_out", _FLOATS, (T, heads, head_dim))
    _req(cache, "cache", (q_out.dtype,), (None, 2, kv_heads, None, head_dim))
    _check(_get("air_qkv_rope_store")(
        qkv.data_ptr(), _DT[qkv.dtype], parts, _ptr(bias), _DT[bias.dtype] if bias is not None else 0,
        _ptr(table), rot, positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(),
        block_table.shape[1], q_out.data_ptr(), cache.data_ptr(), _DT[q_out.dtype], T, heads, kv_heads,
        head_dim, cache.shape[3], 1 if write_kv else 0, _ptr(status), _stream()), "qkv_rope_store")
    return q_out


def silu_mul(gate_up, out, block=None):
    """out[t, i] = silu(gate[t, i]) * up[t, i], where gate_up [T, 2I] holds blocks of `block` gate
    columns and `block` up columns in turn (default: all gate columns, then all up columns)."""
    T, I = out.shape
    block = I if block is None else block
    if block <= 0 or I % block:
        raise KernelError(f"silu_mul: block {block} does not divide {I}")
    _req(gate_up, "gate_up", _FLOATS, (T, 2 * I))
    _req(out, "out", _FLOATS)
    _check(_get("air_silu_mul")(gate_up.data_ptr(), _DT[gate_up.dtype], out.data_ptr(), _DT[out.dtype], T, I,
                                block, _stream()), "silu_mul")
    return out


def convert(src, out):
    _req(src, "src", _FLOATS)
    _req(out, "out", _FLOATS, tuple(src.shape))
    _check(_get("air_convert")(src.data_ptr(), _DT[src.dtype], out.data_ptr(), _DT[out.dtype], src.numel(),
                               _stream()), "convert")
    return out


def gemm_f32(a, w, bias, out):
    """out[M, N] = a[M, K] @ w[N, K]^T + bias, all float32, on the CUDA cores."""
    M, K = a.shape
    N = w.shape[0]
    _req(a, "a", (torch.float32,))
    _req(w, "w", (torch.float32,), (N, K))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (N,))
    _req(out, "out", (torch.float32,), (M, N))
    _check(_get("air_gemm_f32")(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, _stream()),
           "gemm_f32")
    return out


def paged_attention_ref(q, cache, block_table, token_seq, positions, out, window, scale, softcap=0.0, gate=None,
                        kv_heads=None, page_tokens=None, chunk=None, sink=None, latent=False):
    """Causal attention over the pages with 32-bit arithmetic, for any batch.  q [T, H, d], out [T, H, dv].
    cache [page, 2, K, P, d] where dv == d; where keys and values differ in size a page is flat: the keys
    [K, P, d], then the values [K, P, dv], and kv_heads and page_tokens say what K and P are.  score = scale * q.k,
    then softcap * tanh(score / softcap) where softcap > 0; gate (float32 [T, H]) multiplies a head's output.
    Which keys a query at position p sees: all up to its own; with `window` the last `window` of them; with `chunk`
    those from p - p % chunk on.  sink (float32 [H]): one more term exp(sink[h]) in the softmax's denominator.
    latent: cache [page, P, d] holds one row per token that every head reads as its key and whose first dv elements
    it reads as its value; q may then be float32 whatever the cache's type."""
    T, H, d = q.shape
    dv = out.shape[2]
    _req(q, "q", _FLOATS)
    if latent:
        _req(cache, "cache", (out.dtype,), (None, None, d))
        K, P = 1, cache.shape[1]
        if dv > d:
            raise KernelError("paged_attention_ref: a latent row's value is a part of its key")
    elif cache.dim() == 5:
        _req(cache, "cache", (q.dtype,), (None, 2, None, None, d))
        K, P = cache.shape[2], cache.shape[3]
        if dv != d:
            raise KernelError("paged_attention_ref: pages of the shape [2, K, P, d] hold values of the keys' size")
        if d % 16:
            raise KernelError(f"head size {d}: pages of the shape [2, K, P, d] take multiples of 16 up to 256")
    else:
        K, P = int(kv_heads), int(page_tokens)
        _req(cache, "cache", (q.dtype,), (None, K * P * (d + dv)))
    if q.dtype != out.dtype and q.dtype != torch.float32:
        raise KernelError("paged_attention_ref: q is float32 or of the cache's type")
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (cache.dtype,), (T, H, dv))
    if gate is not None:
        _req(gate, "gate", (torch.float32,), (T, H))
    if sink is not None:
        _req(sink, "sink", (torch.float32,), (H,))
    if window and chunk:
        raise KernelError("paged_attention_ref: a window or a chunk, not both")
    if d > 640 or dv > 640:
        raise KernelError(f"head sizes {d} and {dv}: the 32-bit attention kernel takes up to 640")
    _check(_get("air_paged_attention_ref")(
        q.data_ptr(), 1 if q.dtype == torch.float32 else 0, cache.data_ptr(), _DT[cache.dtype], block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(), _ptr(gate), T, H, K, d, dv, P,
        int(chunk or window or 0), float(scale), float(softcap or 0.0), 1 if chunk else 0, _ptr(sink),
        1 if latent else 0, _stream()), "paged_attention_ref")
    return out


def grouped_attention_ok(cache_dtype, d, dv) -> bool:
    """Whether grouped_attention takes keys of d and values of dv elements: rows of whole 16-byte pieces."""
    size = 4 if cache_dtype == torch.float32 else 2
    return (d * size) % 16 == 0 and (dv * size) % 16 == 0 and dv <= 768


def grouped_attention(q, cache, block_table, token_seq, positions, out, window, scale, kv_heads=1, page_tokens=None,
                      chunk=None, sink=None, latent=False, splits=None, softcap=0.0, gate=None):
    """paged_attention_ref's arithmetic and arguments (32-bit, any batch, window or chunk, sink, latent rows), by the
    kernel in which a block serves all query heads of a key/value head and the keys of a token are split over
    `splits` blocks (default: enough to fill the device); needs grouped_attention_ok(cache.dtype, d, dv).  gate (float32
    [T, H * dv], may be a band of columns): out is multiplied, element by element, by sigmoid(gate)."""
    T, H, d = q.shape
    gp, ldg = (None, 0)
    if gate is not None:
        gp, ldg = _columns(gate, "gate")
        if tuple(gate.shape) != (T, H * out.shape[2]):
            raise KernelError("grouped_attention: the gate does not fit")
    dv = out.shape[2]
    _req(q, "q", _FLOATS)
    G = 1 if latent else int(kv_heads)
    if latent:
        _req(cache, "cache", (out.dtype,), (None, None, d))
        P = cache.shape[1]
    else:
        P = int(page_tokens)
        _req(cache, "cache", (out.dtype,))
        if cache[0].numel() != G * P * (d + dv):
            raise KernelError(f"grouped_attention: a page of {cache[0].numel()} elements, not {G} x {P} x ({d} + {dv})")
    if q.dtype != out.dtype and q.dtype != torch.float32:
        raise KernelError("grouped_attention: q is float32 or of the cache's type")
    if not grouped_attention_ok(cache.dtype, d, dv):
        raise KernelError(f"grouped_attention: head sizes {d} and {dv} are not whole 16-byte pieces")
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (cache.dtype,), (T, H, dv))
    if sink is not None:
        _req(sink, "sink", (torch.float32,), (H,))
    if window and chunk:
        raise KernelError("grouped_attention: a window or a chunk, not both")
    J = H // G
    if splits is None:
        # float32: always the same number, so that a row's sums do not depend on what else is in the batch;
        # bfloat16: as many as fill the device
        blocks = T * G * -(-J // (16 if J > 4 else 4))
        splits = 4 if cache.dtype == torch.float32 else max(1, min(16, 296 // max(1, blocks)))
    part = torch.empty((T, H, splits, dv + 2), dtype=torch.float32, device=q.device)
    _check(_get("air_grouped_attention")(
        q.data_ptr(), 1 if q.dtype == torch.float32 else 0, cache.data_ptr(), _DT[cache.dtype], block_table.data_ptr(),
        block_table.shape[1], token_seq.data_ptr(), positions.data_ptr(), part.data_ptr(), out.data_ptr(), T, H, G, d,
        dv, P, int(chunk or window or 0), float(scale), 1 if chunk else 0, _ptr(sink), 1 if latent else 0, int(splits),
        float(softcap or 0.0), gp, ldg, _stream()), "grouped_attention")
    global launches
    launches += 1
    return out


def gather_keys(cache, table_row, lo, count, keys, values, kv_heads=1, page_tokens=None, latent=False):
    """The keys lo .. lo + count of the request whose block-table row is table_row, from the pages into keys
    [G, Lp, dk] (and values [G, Lp, dv]; latent: cache [pages, P, dk], keys [1, Lp, dk], no values).  Rows count .. Lp
    are zeroed."""
    G, Lp, dk = keys.shape
    _req(keys, "keys", _FLOATS)
    _req(cache, "cache", (keys.dtype,))
    _req(table_row, "table_row", _I32)
    dv = 0
    if latent:
        P = cache.shape[1]
    else:
        _req(values, "values", (keys.dtype,), (G, Lp, None))
        dv, P = values.shape[2], int(page_tokens)
    _check(_get("air_gather_keys")(cache.data_ptr(), _DT[keys.dtype], table_row.data_ptr(), int(lo), int(count), Lp,
                                   int(kv_heads), dk, dv, P, 1 if latent else 0, keys.data_ptr(),
                                   None if latent else values.data_ptr(), _stream()), "gather_keys")


def masked_softmax(scores, weights, heads_per_group, lo, count, pos0, scale, window=None, chunk=None, sink=None,
                   softcap=0.0):
    """scores float32 [G, n * J, Lp] -> weights bfloat16 of the same shape: the softmax of scale * scores over the keys
    that each row's query sees (column c = key lo + c, c < count; row (t, j) = the query at pos0 + t of head g * J + j),
    with exp(sink[h]) in the denominator where sink (float32 [G * J]) is given; with softcap > 0 a score is
    softcap * tanh(scale * score / softcap)."""
    G, rows, Lp = scores.shape
    J = int(heads_per_group)
    _req(scores, "scores", (torch.float32,))
    _req(weights, "weights", (torch.bfloat16,), (G, rows, Lp))
    if sink is not None:
        _req(sink, "sink", (torch.float32,), (G * J,))
    if window and chunk:
        raise KernelError("masked_softmax: a window or a chunk, not both")
    _check(_get("air_masked_softmax")(scores.data_ptr(), weights.data_ptr(), G, rows // J, J, int(count), Lp, int(lo),
                                      int(pos0), int(chunk or window or 0), 1 if chunk else 0, float(scale), _ptr(sink),
                                      float(softcap or 0.0), _stream()), "masked_softmax")


def post_norm(h, alpha, a, b, b_row_scale, weight, eps, out):
    """h <- rms(alpha * h + a + s * b) * weight in place (float32), with a copy in out's type (out may be None).
    a, b: None, float32 [T, E] or partial sums [parts, T, E] added in order; s = b_row_scale (float32 [T]) or 1.
    weight None: only the sum is written back (no norm)."""
    T, E = h.shape
    _req(h, "h", (torch.float32,))
    parts = []
    for name, x in (("a", a), ("b", b)):
        n = 0
        if x is not None:
            n = 1 if x.dim() == 2 else x.shape[0]
            _req(x, name, (torch.float32,), (T, E) if x.dim() == 2 else (n, T, E))
        parts.append(n)
    if b_row_scale is not None:
        _req(b_row_scale, "b_row_scale", (torch.float32,), (T,))
    if weight is not None:
        _req(weight, "weight", _FLOATS, (E,))
    if out is not None:
        _req(out, "out", _FLOATS, (T, E))
    _check(_get("air_post_norm")(h.data_ptr(), float(alpha), _ptr(a), parts[0], _ptr(b), parts[1], _ptr(b_row_scale),
                                 T * E, _ptr(weight), _DT[weight.dtype] if weight is not None else 0, _ptr(out),
                                 _DT[out.dtype] if out is not None else 0, T, E, float(eps), _stream()), "post_norm")
    return out


def qk_normed_prepare(proj, q_weight, k_weight, eps, freq, pairing, magnitude, positions, token_seq, block_table, q_out,
                      cache, kv_heads, v_dim, page_tokens, status=None, bias=None, whole=False):
    """From the fused projection proj (float32 [T, (H + G) dk + G dv]: q, k, v per token) to q_out [T, H, dk] and
    the pages (keys [G, P, dk], then values [G, P, dv]).  q and k heads are normalised (x / sqrt(mean(x^2) + eps) * w,
    w float32 [dk]: q_weight for q, k_weight for k; None: no norm), then their first 2 * len(freq) elements are
    rotated by position * freq[j] (freq float64), pair j = (2j, 2j + 1) where pairing == "neighbours", (j, j + rot/2)
    where "half"; cos and sin are multiplied by magnitude.  bias (float32 [W]) is added to q, k and v first.  whole: the
    norm is taken over all heads of q at once (and over all heads of k), with weights [H * dk] and [G * dk].  proj may be
    a band of columns of a wider matrix."""
    T, H, dk = q_out.shape
    G, dv, P = int(kv_heads), int(v_dim), int(page_tokens)
    W = (H + G) * dk + G * dv
    pp, ld = _columns(proj, "proj")
    if tuple(proj.shape) != (T, W):
        raise KernelError(f"qk_normed_prepare: proj {tuple(proj.shape)}, wanted {(T, W)}")
    for name, w, heads in (("q_weight", q_weight, H), ("k_weight", k_weight, G)):
        if w is not None:
            _req(w, name, (torch.float32,), (heads * dk if whole else dk,))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (W,))
    rot = 0
    if freq is not None:
        _req(freq, "freq", (torch.float64,))
        rot = 2 * freq.numel()
    if pairing not in ("half", "neighbours"):
        raise KernelError(f"qk_normed_prepare: pairing {pairing!r}")
    _req(positions, "positions", _I32, (T,))
    _req(token_seq, "token_seq", _I32, (T,))
    _req(block_table, "block_table", _I32)
    _req(q_out, "q_out", _FLOATS)
    _req(cache, "cache", (q_out.dtype,))
    if cache[0].numel() != G * P * (dk + dv):
        raise KernelError(f"qk_normed_prepare: a page of {cache[0].numel()} elements, not {G} x {P} x ({dk} + {dv})")
    _check(_get("air_qk_normed_prepare")(
        pp, ld, _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(freq), rot,
        1 if pairing == "neighbours" else 0, float(magnitude), positions.data_ptr(), token_seq.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], q_out.data_ptr(), cache.data_ptr(), _DT[q_out.dtype], T, H, G, dk,
        dv, P, _ptr(status), _ptr(bias), 1 if whole else 0, _stream()), "qk_normed_prepare")
    return q_out


def latent_prepare(proj, c_weight, eps, freq, positions, token_seq, block_table, q_plain, q_full, cache, owns,
                   status=None, gate_out=None, gate_column=0):
    """From the first projection of a latent-attention layer (float32 [T, H (d + rot) (+ R + rot where owns) (+ more)])
    to q_plain [T, H, d] (the cache's type), the rotated parts in q_full[:, :, R:] (float32 [T, H, R + rot]) and, where
    owns, the row [rms(c) * c_weight | rotated kr] in the pages (cache [pages, P, R + rot]).  freq None: nothing is
    rotated (rot = 0).  gate_out float32 [T, H] = sigmoid of the H columns of proj from gate_column on."""
    T, H, d = q_plain.shape
    P, width = cache.shape[1], cache.shape[2]
    rot = 2 * freq.numel() if freq is not None else 0
    R = width - rot
    ld = proj.shape[1]
    _req(proj, "proj", (torch.float32,), (T, None))
    if ld < H * (d + rot) + (width if owns else 0):
        raise KernelError(f"latent_prepare: proj has {ld} columns, too few")
    if gate_out is not None:
        _req(gate_out, "gate_out", (torch.float32,), (T, H))
    if freq is not None:
        _req(freq, "freq", (torch.float64,))
    if owns:
        _req(c_weight, "c_weight", (torch.float32,), (R,))
    _req(positions, "positions", _I32, (T,))
    _req(token_seq, "token_seq", _I32, (T,))
    _req(block_table, "block_table", _I32)
    _req(q_plain, "q_plain", _FLOATS)
    _req(q_full, "q_full", (torch.float32,), (T, H, width))
    _req(cache, "cache", (q_plain.dtype,))
    _check(_get("air_latent_prepare")(
        proj.data_ptr(), ld, _ptr(c_weight), float(eps), _ptr(freq), positions.data_ptr(), token_seq.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], q_plain.data_ptr(), q_full.data_ptr(), cache.data_ptr(),
        _DT[q_plain.dtype], 1 if owns else 0, T, H, d, rot, R, P, _ptr(gate_out), int(gate_column), _ptr(status),
        _stream()), "latent_prepare")


def moe_route(z, experts, top, expert_out, weight_out, gate_out=None, has_gate=False, score="sigmoid",
              renormalize=False, groups=0, keep=0, route_scale=1.0, norm_eps=0.0, choice_bias=None):
    """z float32 [T, >= experts (+ 1)]: router logits.  expert_out int32 [T, top], weight_out float32 [T, top]: the
    experts with the largest scores (sigmoid(z), or softmax(z)) and those scores (divided by their sum + norm_eps where
    renormalize), times route_scale; gate_out float32 [T] = sigmoid(z[:, experts]) where has_gate, else 1.  groups > 1:
    the experts are cut into `groups` runs of experts / groups consecutive indices, a run's mark is its best score plus
    its second best, and only experts of the `keep` runs with the highest marks can be chosen.  choice_bias (float32
    [experts]): the experts are chosen by score + choice_bias; the weights stay the scores."""
    T = z.shape[0]
    if choice_bias is not None:
        _req(choice_bias, "choice_bias", (torch.float32,), (experts,))
    _req(z, "z", (torch.float32,))
    _req(expert_out, "expert_out", _I32, (T, top))
    _req(weight_out, "weight_out", (torch.float32,), (T, top))
    if gate_out is not None:
        _req(gate_out, "gate_out", (torch.float32,), (T,))
    if score not in ("sigmoid", "softmax"):
        raise KernelError(f"moe_route: score {score!r}")
    _check(_get("air_moe_route")(z.data_ptr(), z.shape[1], T, int(experts), int(top), 1 if score == "softmax" else 0,
                                 1 if renormalize else 0, 1 if has_gate else 0, expert_out.data_ptr(),
                                 weight_out.data_ptr(), _ptr(gate_out), int(groups), int(keep), float(route_scale),
                                 float(norm_eps), _ptr(choice_bias), _stream()), "moe_route")


def moe_identity(x, expert, weight, real_experts, y):
    """The pairs (token, choice) whose expert has an index of real_experts or more are identity experts: y[choice,
    token] = weight[token, choice] * x[token].  x [T, E]; expert int32 and weight float32 [T, top]; y float32
    [top, T, E]."""
    T, E = x.shape
    top = expert.shape[1]
    _req(x, "x", _FLOATS)
    _req(expert, "expert", _I32, (T, top))
    _req(weight, "weight", (torch.float32,), (T, top))
    _req(y, "y", (torch.float32,), (top, T, E))
    _check(_get("air_moe_identity")(x.data_ptr(), _DT[x.dtype], expert.data_ptr(), weight.data_ptr(), int(real_experts),
                                    top, T, E, y.data_ptr(), _stream()), "moe_identity")
    return y


GROUP_TILE = 64      # rows of a tile of the grouped product


def moe_sort(expert, experts, start, pair_of_slot, tiles, num_tiles):
    """Orders the (token, choice) pairs of expert int32 [T, top] by expert: start int32 [experts + 1], pair_of_slot
    int32 [T * top], the grouped product's row tiles (tiles int32 [max_tiles, 2], num_tiles int32 [1])."""
    pairs = expert.numel()
    _req(expert, "expert", _I32)
    _req(start, "start", _I32, (experts + 1,))
    _req(pair_of_slot, "pair_of_slot", _I32, (pairs,))
    _req(tiles, "tiles", _I32, (None, 2))
    if tiles.shape[0] < pairs // GROUP_TILE + experts:
        raise KernelError("moe_sort: the tile list is too short")
    _req(num_tiles, "num_tiles", _I32, (1,))
    _check(_get("air_moe_sort")(expert.data_ptr(), pairs, int(experts), GROUP_TILE, start.data_ptr(),
                                pair_of_slot.data_ptr(), tiles.data_ptr(), num_tiles.data_ptr(), _stream()), "moe_sort")


def grouped_gemm(a, w, out, n, k, *, lda, ldo, groups, a_group_stride=0, o_group_stride=0, a_index=None, a_div=1,
                 a_scale=None, a_local=False, o_index=None, o_div=1, o_part_stride=0, o_local=False, start=None,
                 rows_per_group=0, tiles=None, num_tiles=None, silu_mul=False, gate_block=0, o_scale=None, o_scale_ld=0,
                 relu2=False):
    """out rows = a rows @ w[g]^T for every group g (w [groups, n (2n with silu_mul), k]); see grouped_gemm.cu for how
    rows are found.  Strides in elements.  out is float32 or of a's type; with silu_mul out = silu(gate) * linear, the
    rows of w[g] being blocks of gate_block gate rows and as many linear rows in turn (0: all gate rows first).
    o_scale float32: the row written for slot s is multiplied, in 32-bit, by o_scale[o_index[s]], or without o_index by
    o_scale[row * o_scale_ld + g] (row: the row of out, inside the group where o_local).  relu2: out = max(product, 0)^2
    in a's type."""
    if relu2 and (silu_mul or out.dtype != a.dtype):
        raise KernelError("grouped_gemm: the squared relu is written in the input's type, and is not gated")
    _req(a, "a", _FLOATS)
    _req(w, "w", (a.dtype,), (groups, 2 * n if silu_mul else n, k))
    _req(out, "out", (torch.float32, a.dtype))
    if silu_mul and out.dtype != a.dtype:
        raise KernelError("grouped_gemm: the activation is written in the input's type")
    for name, x in (("a_index", a_index), ("o_index", o_index), ("start", start), ("tiles", tiles),
                    ("num_tiles", num_tiles)):
        if x is not None:
            _req(x, name, _I32)
    if a_scale is not None:
        _req(a_scale, "a_scale", (torch.float32,))
    if o_scale is not None:
        _req(o_scale, "o_scale", (torch.float32,))
    _check(_get("air_grouped_gemm")(
        a.data_ptr(), int(lda), int(a_group_stride), _ptr(a_index), int(a_div), 1 if a_local else 0, _ptr(a_scale),
        w.data_ptr(), w.shape[1] * w.shape[2], out.data_ptr(), int(ldo), int(o_group_stride), _ptr(o_index), int(o_div),
        int(o_part_stride), 1 if o_local else 0, 1 if out.dtype == torch.float32 else 0, _ptr(start),
        int(rows_per_group), _ptr(tiles), _ptr(num_tiles), tiles.shape[0] if tiles is not None else 0, int(groups),
        int(n), int(k), _DT[a.dtype], 2 if relu2 else (1 if silu_mul else 0), int(gate_block), _ptr(o_scale), int(o_scale_ld), _stream()), "grouped_gemm")
    return out


def rows_by_index(x, index, div, scale, out):
    """out[s] = x[index[s] // div] * scale[index[s]] (scale float32 or None), in x's type."""
    _req(x, "x", _FLOATS)
    _req(index, "index", _I32, (out.shape[0],))
    _req(out, "out", (x.dtype,), (None, x.shape[1]))
    if scale is not None:
        _req(scale, "scale", (torch.float32,))
    _check(_get("air_rows_by_index")(x.data_ptr(), _DT[x.dtype], index.data_ptr(), int(div), _ptr(scale), out.data_ptr(),
                                     out.shape[0], x.shape[1], _stream()), "rows_by_index")
    return out


def planes_by_index(rows, index, div, out, scale=None):
    """out[index[s] % div, index[s] // div] = rows[s] * scale[index[s]] (scale float32 or None); rows [n, E], out
    float32 [div, T, E]."""
    n, E = rows.shape
    _req(rows, "rows", _FLOATS)
    _req(index, "index", _I32, (n,))
    _req(out, "out", (torch.float32,), (div, None, E))
    if scale is not None:
        _req(scale, "scale", (torch.float32,))
    _check(_get("air_planes_by_index")(rows.data_ptr(), _DT[rows.dtype], index.data_ptr(), int(div), out.shape[1] * E,
                                       _ptr(scale), out.data_ptr(), n, E, _stream()), "planes_by_index")
    return out


def qkv_prepare(proj, bias, inv_freq, positions, token_seq, block_table, q_out, cache, kv_heads, v_dim, page_tokens,
                gate_out=None, v_first=None, v_mode=0, v_lambda=None, status=None):
    """From the fused projection of an attention layer to what its attention kernel reads.  proj float32 [T, W]:
    per token q (H heads of dk), k (G heads of dk), v (G heads of dv) and, with gate_out, H gate logits.  Adds the
    bias (float32 [W]), rotates the first 2 * len(inv_freq) elements of each head of q and k (element i with
    i + rot/2, angle position * inv_freq[i] in 32-bit), writes q to q_out [T, H, dk] and k and v into the pages
    (a page: keys [G, P, dk], then values [G, P, dv]) and sigmoid(gate logits) to gate_out (float32 [T, H]).
    v_mode 1 also hands the values on in v_first (float32 [T, G * dv]); v_mode 2 first mixes them with v_first:
    v = (1 - v_lambda) v + v_lambda v_first (v_lambda: a float32 tensor of one element)."""
    T, H, dk = q_out.shape
    G, dv, P = int(kv_heads), int(v_dim), int(page_tokens)
    W = (H + G) * dk + G * dv + (H if gate_out is not None else 0)
    _req(proj, "proj", (torch.float32,), (T, W))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (W,))
    rot = 0
    if inv_freq is not None:
        _req(inv_freq, "inv_freq", (torch.float32,))
        rot = 2 * inv_freq.numel()
        if rot > dk:
            raise KernelError(f"rotary width {rot} does not fit head size {dk}")
    _req(positions, "positions", _I32, (T,))
    _req(token_seq, "token_seq", _I32, (T,))
    _req(block_table, "block_table", _I32)
    _req(q_out, "q_out", _FLOATS)
    _req(cache, "cache", (q_out.dtype,))
    if cache[0].numel() != G * P * (dk + dv):
        raise KernelError(f"qkv_prepare: a page of {cache[0].numel()} elements, not {G} x {P} x ({dk} + {dv})")
    if gate_out is not None:
        _req(gate_out, "gate_out", (torch.float32,), (T, H))
    if v_mode:
        _req(v_first, "v_first", (torch.float32,), (T, G * dv))
    if v_mode == 2:
        _req(v_lambda, "v_lambda", (torch.float32,))
    _check(_get("air_qkv_prepare")(
        proj.data_ptr(), W, _ptr(bias), _ptr(inv_freq), rot, positions.data_ptr(), token_seq.data_ptr(),
        block_table.data_ptr(), block_table.shape[1], q_out.data_ptr(), cache.data_ptr(), _DT[q_out.dtype],
        _ptr(gate_out), _ptr(v_first) if v_mode else None, int(v_mode), _ptr(v_lambda) if v_mode == 2 else None,
        T, H, G, dk, dv, P, _ptr(status), _stream()), "qkv_prepare")
    return q_out


def _columns(t, name):
    """(pointer, row stride) of a float32 matrix whose rows may be a band of columns of a wider one."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a float32 CUDA matrix with contiguous rows")
    return t.data_ptr(), t.stride(0)


def short_conv_silu(x, weight, state, y, q_start, slots, max_tokens, act=True):
    """y[t, c] = silu(sum_j weight[c, j] x[t - (taps - 1 - j), c]) for every entry of the batch (rows q_start[e] ..
    q_start[e + 1], state row slots[e]): a causal convolution over the request's tokens, whose inputs before the
    portion come from state [slots, C, taps - 1] (oldest first; zeros at a request's start) and whose last taps - 1
    inputs are left there.  x: float32 [T, C] (may be a band of columns of a wider matrix); y: float32 [T, C].
    max_tokens: the longest portion of the batch (a host number: it sizes the grid).  act False: the sum itself,
    without the SiLU."""
    C, taps = weight.shape
    xp, ld = _columns(x, "x")
    _req(weight, "weight", (torch.float32,))
    _req(state, "state", (torch.float32,), (None, C, taps - 1))
    _req(y, "y", (torch.float32,), (x.shape[0], C))
    _req(q_start, "q_start", _I32)
    _req(slots, "slots", _I32)
    if x.shape[1] != C:
        raise KernelError(f"short_conv_silu: x has {x.shape[1]} channels, the weight {C}")
    if not (1 <= taps <= 16):
        raise KernelError(f"short_conv_silu: {taps} taps (the kernel takes 1 to 16)")
    _check(_get("air_short_conv_silu")(xp, ld, weight.data_ptr(), state.data_ptr(), y.data_ptr(), q_start.data_ptr(),
                                       slots.data_ptr(), slots.shape[0], C, taps, int(max_tokens), 1 if act else 0,
                                       _stream()),
           "short_conv_silu")
    return y


SCAN_DELTA, SCAN_GLA, SCAN_HGRN, SCAN_RETENTION = 0, 1, 2, 3


def linear_scan(mode, q, k, v, decay, state, out, q_start, slots, token_seq, q_scale=1.0, beta=None, a_log=None,
                dt_bias=None, tau=1.0, unit=False, unit_eps=1e-6, lower=None, gate_bias=None, positions=None, freq=None,
                k_scale=1.0):
    """A state S [d, dv] per head and request, updated token by token in 32-bit and read out after each update.
    q, k float32 [T, G * d], v [T, H * dv] (each may be a band of columns of a wider matrix); head h reads q/k head
    h // (H / G); state [slots, H, d, dv]; out [T, H, dv]; token_seq [T]: the slot of each row's request (negative:
    padding).  Two launches: what the recurrence reads per token (unit lengths, scales, decays) is worked out for all
    tokens side by side, then the scan takes the tokens of each request in order.
    SCAN_DELTA: decay, beta [T, H] logits; g = exp(-exp(a_log[h]) * softplus(decay + dt_bias[h])), b = sigmoid(beta);
      with unit, q and k are first divided by sqrt(sum of squares + unit_eps), q then multiplied by q_scale;
      S = g S; u = b (v - S^T k); S += k u^T; o = S^T q.
    SCAN_GLA: decay [T, H * d] logits; alpha = sigmoid(decay)^(1 / tau); q is multiplied by q_scale;
      S = diag(alpha) S + k v^T; o = S^T q.
    SCAN_HGRN: decay [T, H * d] logits, lower and gate_bias float32 [H * d]; alpha = lower + (1 - lower) *
      sigmoid(decay + gate_bias); k is None (k = 1 - alpha); q = silu(q) * q_scale; the recurrence is SCAN_GLA's.
    SCAN_RETENTION: decay float32 [H], one constant per head; the first 2 * len(freq) elements of every head of q and k
      are rotated (element i with i + rot / 2) by positions[t] * freq[i] (freq float64; the angle and its cos and sin
      in 64-bit), q is multiplied by q_scale, k by k_scale; S = decay[h] S + k v^T; o = S^T q."""
    slots_n, H, d, dv = state.shape
    _req(state, "state", (torch.float32,))
    T = out.shape[0]
    _req(out, "out", (torch.float32,), (T, H, dv))
    qp, ldq = _columns(q, "q")
    kp, ldk = _columns(k, "k") if k is not None else (None, 0)
    vp, ldv = _columns(v, "v")
    if mode == SCAN_RETENTION:
        _req(decay, "decay", (torch.float32,), (H,))
        dp, ldd = decay.data_ptr(), 0
    else:
        dp, ldd = _columns(decay, "decay")
    if (k is None) != (mode == SCAN_HGRN):
        raise KernelError("linear_scan: keys are given except where the gate makes them")
    if q.shape[1] % d or (k is not None and k.shape != q.shape) or v.shape[1] != H * dv:
        raise KernelError("linear_scan: q, k or v do not fit the state's shape")
    G = q.shape[1] // d
    if G == 0 or H % G:
        raise KernelError(f"linear_scan: {H} heads over {G} heads of q and k")
    bp, ldb = (None, 0)
    if mode == SCAN_DELTA:
        bp, ldb = _columns(beta, "beta")
        _req(a_log, "a_log", (torch.float32,), (H,))
        _req(dt_bias, "dt_bias", (torch.float32,), (H,))
        if decay.shape[1] != H or beta.shape[1] != H:
            raise KernelError("linear_scan: the delta rule takes one decay and one beta per head")
    elif mode == SCAN_GLA:
        if decay.shape[1] != H * d or G != H:
            raise KernelError("linear_scan: gated linear attention takes a decay per key channel of every head")
    elif mode == SCAN_HGRN:
        if decay.shape[1] != H * d or G != H:
            raise KernelError("linear_scan: a forget gate per key channel of every head")
        a_log, dt_bias = _req(lower, "lower", (torch.float32,), (H * d,)), _req(gate_bias, "gate_bias",
                                                                                   (torch.float32,), (H * d,))
    elif mode == SCAN_RETENTION:
        if G != H:
            raise KernelError("linear_scan: retention takes a head of q and k per head of v")
        rot = 0
        if freq is not None:
            _req(freq, "freq", (torch.float64,))
            _req(positions, "positions", _I32, (T,))
            rot = 2 * freq.numel()
            if rot > d:
                raise KernelError(f"linear_scan: rotary width {rot} does not fit head size {d}")
    else:
        raise KernelError(f"linear_scan: mode {mode}")
    if d > 1024:
        raise KernelError(f"linear_scan: {d} key channels per head (the kernel takes up to 1,024)")
    _req(q_start, "q_start", _I32)
    _req(slots, "slots", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    rows = 16 if d <= 512 else 32          # of a column of the state per lane; lanes per column: a power of two
    lanes = 1
    while lanes * rows < d:
        lanes *= 2
    kq = torch.empty((T, G, 2, lanes * rows), dtype=torch.float32, device=out.device)
    dec = None if mode == SCAN_RETENTION else \
        torch.empty((T, H, 2 if mode == SCAN_DELTA else lanes * rows), dtype=torch.float32, device=out.device)
    _check(_get("air_linear_scan")(
        int(mode), qp, ldq, kp, ldk, vp, ldv, dp, ldd, bp, ldb, _ptr(a_log), _ptr(dt_bias), state.data_ptr(),
        out.data_ptr(), q_start.data_ptr(), slots.data_ptr(), token_seq.data_ptr(), kq.data_ptr(), _ptr(dec),
        T, slots.shape[0], H, G, d, dv, lanes, float(q_scale), 1.0 / float(tau), 1 if unit else 0, float(unit_eps),
        _ptr(positions), _ptr(freq), 2 * freq.numel() if (mode == SCAN_RETENTION and freq is not None) else 0,
        float(k_scale), _stream()), "linear_scan")
    global launches
    launches += 1
    return out


def gated_rmsnorm(o, gate, weight, eps, out, token_seq):
    """out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * weight * silu(gate[t, h, :]).  o float32 [T, H, dv]; gate
    float32 [T, H * dv] (may be a band of columns) or None (no gate); weight float32 [dv]; out [T, H * dv]."""
    T, H, dv = o.shape
    _req(o, "o", (torch.float32,))
    gp, ldg = _columns(gate, "gate") if gate is not None else (None, 0)
    if gate is not None and gate.shape != (T, H * dv):
        raise KernelError("gated_rmsnorm: the gate does not fit")
    _req(weight, "weight", (torch.float32,), (dv,))
    _req(out, "out", _FLOATS, (T, H * dv))
    _req(token_seq, "token_seq", _I32, (T,))
    _check(_get("air_gated_rmsnorm")(o.data_ptr(), gp, ldg, weight.data_ptr(), out.data_ptr(), _DT[out.dtype],
                                     token_seq.data_ptr(), T, H, dv, float(eps), _stream()), "gated_rmsnorm")
    return out


def head_gate(x, gate, token_seq):
    """x[t, h, :] *= gate[t, h] in place.  x [T, H, d]; gate float32 [T, H]."""
    T, H, d = x.shape
    _req(x, "x", _FLOATS)
    _req(gate, "gate", (torch.float32,), (T, H))
    _req(token_seq, "token_seq", _I32, (T,))
    _check(_get("air_head_gate")(x.data_ptr(), _DT[x.dtype], gate.data_ptr(), token_seq.data_ptr(), T, H, d, _stream()),
           "head_gate")
    return x


def sigmoid_gate(x, gate, token_seq):
    """x[t, c] *= sigmoid(gate[t, c]) in place.  x [T, C]; gate float32 [T, C] (may be a band of columns)."""
    T, C = x.shape
    _req(x, "x", _FLOATS)
    gp, ldg = _columns(gate, "gate")
    if tuple(gate.shape) != (T, C):
        raise KernelError("sigmoid_gate: the gate does not fit")
    _req(token_seq, "token_seq", _I32, (T,))
    _check(_get("air_sigmoid_gate")(x.data_ptr(), _DT[x.dtype], gp, ldg, token_seq.data_ptr(), T, C, _stream()),
           "sigmoid_gate")
    return x


def relu2(x, out):
    """out = max(x, 0)^2 element by element; x and out of one shape, float32 or bfloat16 each."""
    _req(x, "x", _FLOATS)
    _req(out, "out", _FLOATS, tuple(x.shape))
    _check(_get("air_relu2")(x.data_ptr(), _DT[x.dtype], out.data_ptr(), _DT[out.dtype], x.numel(), _stream()), "relu2")
    return out


def normed_add_norm(h, term, term_weight, term_eps, weight, eps, out, rows=None):
    """x = h + term / sqrt(mean(term^2) + term_eps) * term_weight, written into h when rows is None; out = x /
    sqrt(mean(x^2) + eps) * weight.  term float32 [T, E], or [parts, T, E] partial sums that are added in order first;
    term_weight and weight float32 [E].  With rows: out[r] is that of row rows[r], h unchanged.  weight None (and out
    None): only the stream is completed."""
    E = h.shape[-1]
    _req(h, "h", (torch.float32,), (None, E))
    parts = 1 if term.dim() == 2 else term.shape[0]
    _req(term, "term", (torch.float32,), tuple(h.shape) if term.dim() == 2 else (parts,) + tuple(h.shape))
    _req(term_weight, "term_weight", (torch.float32,), (E,))
    R = h.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _req(rows, "rows", _I32)
    if weight is not None:
        _req(weight, "weight", (torch.float32,), (E,))
        _req(out, "out", _FLOATS, (R, E))
    _check(_get("air_normed_add_norm")(h.data_ptr(), term.data_ptr(), parts, h.numel(), term_weight.data_ptr(),
                                       float(term_eps), _ptr(weight), _ptr(out) if weight is not None else None,
                                       _DT[out.dtype] if weight is not None else 0, _ptr(rows), R, E, float(eps),
                                       _stream()), "normed_add_norm")
    return out


def glu(gate_up, out, block=None, alpha=1.0, limit=0.0, shift=0.0):
    """out[t, i] = g * sigmoid(alpha * g) * (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit)
    where limit > 0; gate_up [T, 2I] as silu_mul takes it."""
    T, I = out.shape
    block = I if block is None else block
    if block <= 0 or I % block:
        raise KernelError(f"glu: block {block} does not divide {I}")
    _req(gate_up, "gate_up", _FLOATS, (T, 2 * I))
    _req(out, "out", _FLOATS)
    _check(_get("air_glu")(gate_up.data_ptr(), _DT[gate_up.dtype], out.data_ptr(), _DT[out.dtype], T, I, block,
                           float(alpha), float(limit), float(shift), _stream()), "glu")
    return out


def polynorm(z, bias, coefficients, eps, out, width):
    """out[t, :width] = a N(u) + b N(u^2) + c N(u^3) + e with u = z[t] + bias, powers per element, N(x) = x /
    sqrt(mean(x^2) + eps) over the row, (a, b, c, e) = coefficients; z float32 [T, width]; out [T, >= width] gets 1 in
    column `width` (if it has one) and 0 behind it."""
    T = z.shape[0]
    zp, ld = _columns(z, "z")
    if z.shape[1] != width:
        raise KernelError("polynorm: z does not have `width` columns")
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (width,))
    _req(out, "out", _FLOATS, (T, None))
    a, b, c, e = (float(v) for v in coefficients)
    _check(_get("air_polynorm")(zp, ld, _ptr(bias), out.data_ptr(), _DT[out.dtype], out.shape[1], T, int(width), a, b,
                                c, e, float(eps), _stream()), "polynorm")
    return out


def scaled_norm(h, terms, weight, eps, out, rows=None):
    """x = h + sum of scale * term over up to two terms (term float32 [T, E], or [parts, T, E] partial sums that are
    added in order; scale float32 [E] or None), written into h when rows is None; out = x / sqrt(mean(x^2) + eps) * weight.  With rows: out[r] is that of row rows[r],
    h unchanged.  weight None (and out None): only the stream is completed."""
    E = h.shape[-1]
    _req(h, "h", (torch.float32,), (None, E))
    terms = list(terms)
    if len(terms) > 2:
        raise KernelError("scaled_norm: at most two terms")
    ptrs = []
    for term, scale in terms + [(None, None)] * (2 - len(terms)):
        parts = 1
        if term is not None:
            parts = 1 if term.dim() == 2 else term.shape[0]
            _req(term, "term", (torch.float32,), tuple(h.shape) if term.dim() == 2 else (parts,) + tuple(h.shape))
        if scale is not None:
            _req(scale, "scale", (torch.float32,), (E,))
        ptrs += [_ptr(term), _ptr(scale), parts]
    R = h.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _req(rows, "rows", _I32)
    if weight is not None:
        _req(weight, "weight", _FLOATS, (E,))
        _req(out, "out", _FLOATS, (R, E))
    _check(_get("air_scaled_norm")(h.data_ptr(), *ptrs, h.numel(), _ptr(weight),
                                   _DT[weight.dtype] if weight is not None else 0,
                                   _ptr(out) if weight is not None else None,
                                   _DT[out.dtype] if weight is not None else 0, _ptr(rows), R, E, float(eps),
                                   _stream()), "scaled_norm")
    return out


def sample(logits, temperature, uniform, out, status=None, slots=None, last_token=None, top_k=None, top_p=None):
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or temperature is None), else the
    index drawn from softmax(logits[r] / temperature[r]) with the uniform number uniform[r], after
    keeping the top_k[r] largest logits (0: all) and of those the shortest prefix of the descending order
    that holds the share top_p[r] of the weight (1: all).  With slots and last_token, also
    last_token[slots[r]] = out[r]."""
    R, V = logits.shape
    _req(logits, "logits", (torch.float32,))
    if temperature is not None:
        _req(temperature, "temperature", (torch.float32,), (R,))
        _req(uniform, "uniform", (torch.float32,), (R,))
    if top_k is not None:
        _req(top_k, "top_k", _I32, (R,))
    if top_p is not None:
        _req(top_p, "top_p", (torch.float32,), (R,))
    _req(out, "out", _I32, (R,))
    if slots is not None:
        _req(slots, "slots", _I32, (R,))
        _req(last_token, "last_token", _I32)
    _check(_get("air_sample")(logits.data_ptr(), _ptr(temperature), _ptr(uniform), _ptr(top_k), _ptr(top_p),
                              out.data_ptr(), _ptr(slots), _ptr(last_token), R, V, _ptr(status), _stream()), "sample")
    return out


def table_update(table, updates):
    """table[slot, block] = page for every (slot, block, page) of updates (flat int32 [3n])."""
    _req(table, "table", _I32)
    _req(updates, "updates", _I32)
    _check(_get("air_table_update")(table.data_ptr(), updates.data_ptr(), updates.numel() // 3, table.shape[1],
                                    _stream()), "table_update")
    return table


DECODE_HEAD_DIMS = (64, 128, 256)


def tile_pages(page_tokens: int) -> bool:
    """Whether the kernels that fetch 64 keys at a time with the copy engine take this page size: a tile of
    keys must lie in one page or be made of whole pages."""
    return 64 % page_tokens == 0 if page_tokens < 64 else page_tokens % 64 == 0


def decode_splits(tokens: int, heads: int, kv_heads: int) -> int:
    """How many blocks share the keys of one (token, kv head): so many that about 190 blocks run,
    which keeps every SM busy without a second round (measured on B200: 6 for 8 tokens x 4 kv heads,
    1 for 64 tokens, 32 for one token)."""
    per_split = tokens * kv_heads * (-(-(heads // kv_heads) // 16))
    return max(1, min(32, round(192 / per_split)))


def decode_attention(q, cache, block_table, token_seq, positions, out, window, scale, splits=None, scratch=None,
                     status=None, engine="tma", softcap=0.0, sink=None, gate=None):
    """bfloat16 attention for one query token per request.  softcap > 0: score = softcap * tanh(scale * q.k /
    softcap) (the copy-engine kernel only).  sink (float32 [H]): one more term exp(sink[h]) in the softmax's
    denominator; gate (float32 [T, H * d] logits, may be a band of columns): out is multiplied by sigmoid(gate) element
    by element; both enter where the key splits are merged (the copy-engine kernel only, two splits at least).  scratch: (float32 [T*H*splits*D], float32
    [T*H*splits*2]) or None to allocate.  engine "tma": keys and values by the copy engine into shared
    memory (attention_decode_tma.cu); "ldg": by the warps' own loads (attention_decode.cu)."""
    T, H, d = q.shape
    K, P = cache.shape[2], cache.shape[3]
    _req(q, "q", (torch.bfloat16,))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if d not in DECODE_HEAD_DIMS:
        raise KernelError(f"decode_attention takes head sizes {DECODE_HEAD_DIMS}, not {d}")
    if splits is None:
        splits = decode_splits(T, H, K)
    extra = sink is not None or gate is not None
    if extra:
        splits = max(2, splits)
        if not (engine == "tma" and tile_pages(P)):
            raise KernelError("decode_attention: a sink or gates are taken by the copy-engine kernel only")
    po = pm = None
    if splits > 1:
        if scratch is None:
            scratch = (torch.empty(T * H * splits * d, dtype=torch.float32, device=q.device),
                       torch.empty(T * H * splits * 2, dtype=torch.float32, device=q.device))
        po, pm = scratch
        _req(po, "scratch[0]", (torch.float32,))
        _req(pm, "scratch[1]", (torch.float32,))
        if po.numel() < T * H * splits * d or pm.numel() < T * H * splits * 2:
            raise KernelError("decode_attention: scratch is too small")
    global launches
    if extra:
        gp, ldg = (None, 0)
        if sink is not None:
            _req(sink, "sink", (torch.float32,), (H,))
        if gate is not None:
            gp, ldg = _columns(gate, "gate")
            if tuple(gate.shape) != (T, H * d):
                raise KernelError("decode_attention: the gate does not fit")
        _check(_get("air_decode_attention_tma_sink")(
            q.data_ptr(), cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
            token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(), _ptr(po), _ptr(pm), T, H, K, d, P,
            int(window or 0), float(scale), float(softcap or 0.0), splits, _ptr(status), _ptr(sink), gp, ldg,
            _stream()), "decode_attention_tma")
    elif engine == "tma" and tile_pages(P):
        _check(_get("air_decode_attention_tma")(
            q.data_ptr(), cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
            token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(), _ptr(po), _ptr(pm), T, H, K, d, P,
            int(window or 0), float(scale), float(softcap or 0.0), splits, _ptr(status), _stream()),
            "decode_attention_tma")
    elif softcap:
        raise KernelError("decode_attention: a soft cap is taken by the copy-engine kernel only (pages that divide "
                          "or are multiples of 64 tokens)")
    else:
        _check(_get("air_decode_attention")(
            q.data_ptr(), cache.data_ptr(), block_table.data_ptr(), block_table.shape[1], token_seq.data_ptr(),
            positions.data_ptr(), out.data_ptr(), _ptr(po), _ptr(pm), T, H, K, d, P, int(window or 0), float(scale),
            splits, _stream()), "decode_attention")
    if splits > 1:
        launches += 1
    return out


def decode_attention_fresh_ok(qkv, table, cache, head_dim) -> bool:
    """Whether decode_attention_fresh takes this: float32 product output, a table that rotates all of a head,
    pages that the copy engine's tiles fit."""
    return (qkv.dtype == torch.float32 and head_dim in DECODE_HEAD_DIMS and table is not None
            and table.shape[1] == head_dim and cache.dtype == torch.bfloat16 and tile_pages(cache.shape[3]))


def decode_attention_fresh(qkv, bias, table, cache, block_table, token_seq, positions, out, heads, window, scale,
                           write_kv=True, splits=None, status=None):
    """bfloat16 attention for one query token per request, straight from the q/k/v product: qkv float32
    [T, (H + 2K) d] or [parts, T, (H + 2K) d] partial sums; the kernel adds the bias, rotates q and k by the
    table's row of each token's position, writes k and v to the pages (write_kv) and attends, which
    qkv_rope_store followed by decode_attention do in two launches (attention_decode_tma.cu)."""
    T, H = qkv.shape[-2], heads
    d, K, P = cache.shape[4], cache.shape[2], cache.shape[3]
    width = (H + 2 * K) * d
    parts = 1 if qkv.dim() == 2 else qkv.shape[0]
    _req(qkv, "qkv", (torch.float32,), (T, width) if qkv.dim() == 2 else (parts, T, width))
    if bias is not None:
        _req(bias, "bias", (torch.float32,), (width,))
    _req(table, "table", (torch.float32,), (None, d))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(token_seq, "token_seq", _I32, (T,))
    _req(positions, "positions", _I32, (T,))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if not decode_attention_fresh_ok(qkv, table, cache, d):
        raise KernelError("decode_attention_fresh: head size, rotary width or page size that this kernel does not take")
    if splits is None:
        splits = decode_splits(T, H, K)
    po = pm = None
    if splits > 1:
        po = torch.empty(T * H * splits * d, dtype=torch.float32, device=qkv.device)
        pm = torch.empty(T * H * splits * 2, dtype=torch.float32, device=qkv.device)
    _check(_get("air_decode_attention_tma_fresh")(
        qkv.data_ptr(), parts, _ptr(bias), table.data_ptr(), 1 if write_kv else 0, cache.data_ptr(), cache.shape[0],
        block_table.data_ptr(), block_table.shape[1], token_seq.data_ptr(), positions.data_ptr(), out.data_ptr(),
        _ptr(po), _ptr(pm), T, H, K, d, P, int(window or 0), float(scale), splits, _ptr(status), _stream()),
        "decode_attention_tma")
    if splits > 1:
        global launches
        launches += 1
    return out


TILE_GROUP = 8     # the list of 16-token tiles comes in groups of 8 that belong to one request
TILE_PAIR = 16     # the tcgen05 kernel takes two groups, one after the other in a request, per block


def prefill_attention(q, cache, block_table, tiles, out, window, scale, status=None):
    """bfloat16 causal attention for tiles of up to 16 consecutive tokens of a request (see
    attention_prefill.cu).  tiles [8n, 4] int32: (slot, first token, its position, rows), in groups of
    8 tiles of one request; rows = 0 marks an empty tile."""
    T, H, d = q.shape
    K, P = cache.shape[2], cache.shape[3]
    _req(q, "q", (torch.bfloat16,))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(tiles, "tiles", _I32, (None, 4))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if d not in DECODE_HEAD_DIMS:
        raise KernelError(f"prefill_attention takes head sizes {DECODE_HEAD_DIMS}, not {d}")
    if tiles.shape[0] % TILE_GROUP:
        raise KernelError("prefill_attention: the tile list must come in groups of 8")
    if not tile_pages(P):
        raise KernelError(f"prefill_attention: page size {P} is neither a divisor nor a multiple of 64")
    _check(_get("air_prefill_attention")(
        q.data_ptr(), cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
        tiles.data_ptr(), tiles.shape[0], out.data_ptr(), H, K, d, P, int(window or 0), float(scale), _ptr(status),
        _stream()), "prefill_attention")
    return out


EPI_F32, EPI_BF16, EPI_SILU, EPI_PARTIAL, EPI_RELU2 = 0, 1, 2, 3, 4


SILU = (1.0, 0.0, 0.0)      # the gated activation of EPI_SILU as (alpha, limit, shift): see gemm_tc


def gemm_tc(a, w, out, bn, epi, splits=1, status=None, max_blocks=0, force_rows_as_m=False, row_ss=None, eps=0.0,
            act=SILU):
    """bfloat16 product a[M,K] @ w[N,K]^T on the tcgen05 tensor cores (see gemm_tc.cu).
    row_ss (float32 [tiles, M]) with eps: the accumulators are multiplied per row by
    rsqrt(sum over tiles of row_ss / K + eps) before the epilogue (the kernel for few rows only; see
    add_prenorm).
    epi EPI_F32: out float32 [M,N]; EPI_BF16: out bfloat16 [M,N]; EPI_SILU: w holds gate and up rows
    interleaved in blocks of bn/2, out bfloat16 [M,N/2] = silu(gate)*up, or with act = (alpha, limit, shift)
    g * sigmoid(alpha * g) * (u + shift) where g = min(gate, limit), u = clamp(up, -limit, limit) if limit > 0;
    EPI_RELU2: out bfloat16 [M,N] = max(product, 0)^2; EPI_PARTIAL: out float32
    [splits,M,N] partial sums over parts of k.  With up to 64 rows and bn 128 or 256 the product runs with the
    weights as the M side of the instruction (gemm_tc_small.cu) unless force_rows_as_m."""
    M, K = a.shape
    N = w.shape[0]
    _req(a, "a", (torch.bfloat16,))
    _req(w, "w", (torch.bfloat16,), (N, K))
    if K % 8:
        raise KernelError(f"gemm_tc: K = {K} must be a multiple of 8 (TMA rows are multiples of 16 bytes)")
    if bn not in (32, 64, 128, 256):
        raise KernelError(f"gemm_tc: tile width {bn}")
    if epi == EPI_F32:
        _req(out, "out", (torch.float32,), (M, N))
    elif epi in (EPI_BF16, EPI_RELU2):      # EPI_RELU2: out = max(product, 0)^2
        _req(out, "out", (torch.bfloat16,), (M, N))
    elif epi == EPI_SILU:
        _req(out, "out", (torch.bfloat16,), (M, N // 2))
        if bn < 64 or N % bn:
            raise KernelError(f"gemm_tc: silu epilogue needs N = {N} to be a multiple of the tile width {bn} >= 64")
    elif epi == EPI_PARTIAL:
        _req(out, "out", (torch.float32,), (splits, M, N))
    else:
        raise KernelError(f"gemm_tc: epilogue {epi}")
    if epi != EPI_SILU and N % 4:
        raise KernelError(f"gemm_tc: N = {N} must be a multiple of 4")
    if row_ss is not None:
        _req(row_ss, "row_ss", (torch.float32,), (None, M))
    if small_rows(M, N, bn, epi) and not force_rows_as_m:
        # few tokens: the weights are the M side of the instruction (gemm_tc_small.cu)
        _check(_get("air_gemm_tc_small")(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, bn, epi, splits,
                                         max_blocks, _ptr(status), _ptr(row_ss),
                                         0 if row_ss is None else row_ss.shape[0], float(eps), float(act[0]),
                                         float(act[1]), float(act[2]), _stream()),
               "gemm_tc_small")
        return out
    if row_ss is not None:
        raise KernelError("gemm_tc: a scale per row is taken by the kernel for up to 64 rows only")
    _check(_get("air_gemm_tc")(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, bn, epi, splits, max_blocks,
                               _ptr(status), float(act[0]), float(act[1]), float(act[2]), _stream()), "gemm_tc")
    return out


def small_rows(M: int, N: int, bn: int, epi: int) -> bool:
    """Whether gemm_tc takes the kernel with the weights as the M side: up to 64 tokens, tiles of 128 or
    256 rows of W; with the activation, gate and up rows in blocks of 128."""
    if M > 64 or bn not in (128, 256):
        return False
    return epi != EPI_SILU or (bn == 256 and N % 256 == 0)


TC_ATTENTION_HEAD_DIMS = (64, 128)


def prefill_attention_scratch(slots: int, head_dim: int, device):
    """Where the segments of cut items leave their partial sums: (float32 [slots, 256, d], float32 [slots, 256, 2])."""
    return (torch.empty((slots, 2 * TILE_GROUP * 16, head_dim), dtype=torch.float32, device=device),
            torch.empty((slots, 2 * TILE_GROUP * 16, 2), dtype=torch.float32, device=device))


def prefill_attention_tc(q, cache, block_table, tiles, out, window, scale, status=None, segments=None, items=None,
                         slots=0, scratch=None, softcap=0.0, sink=None):
    """bfloat16 causal attention with both products on the tcgen05 tensor cores (see
    attention_prefill_tc.cu); arguments as prefill_attention; head size 64 or 128.  softcap > 0: score = softcap *
    tanh(scale * q.k / softcap).  sink (float32 [H]): one more term exp(sink[h]) in the softmax's denominator.
    segments [n, 5] int32 (pair of the list, head, first key tile, key tiles, slot or -1): which block takes which
    part of which pair's stream of keys, instead of one block per pair and head; items [m, 4] int32 (pair, head,
    first slot, slots): the (pair, head)s whose segments write partial sums into `slots` slots, merged here.
    scratch: what prefill_attention_scratch gives (or None to allocate): the layers of a step can share it."""
    T, H, d = q.shape
    K, P = cache.shape[2], cache.shape[3]
    _req(q, "q", (torch.bfloat16,))
    _req(cache, "cache", (torch.bfloat16,), (None, 2, None, None, d))
    _req(block_table, "block_table", _I32)
    _req(tiles, "tiles", _I32, (None, 4))
    _req(out, "out", (torch.bfloat16,), (T, H, d))
    if d not in TC_ATTENTION_HEAD_DIMS:
        raise KernelError(f"prefill_attention_tc takes head sizes {TC_ATTENTION_HEAD_DIMS}, not {d}")
    if tiles.shape[0] % TILE_PAIR:
        raise KernelError("prefill_attention_tc: the tile list must come in groups of 16 per request")
    if not tile_pages(P):
        raise KernelError(f"prefill_attention_tc: page size {P} is neither a divisor nor a multiple of 64")
    part_o = part_ml = None
    n_items = 0
    if segments is not None:
        _req(segments, "segments", _I32, (None, 5))
        if segments.shape[0] == 0:
            raise KernelError("prefill_attention_tc: an empty list of segments")
        if slots:
            _req(items, "items", _I32, (None, 4))
            n_items = items.shape[0]
            part_o, part_ml = scratch if scratch is not None else prefill_attention_scratch(slots, d, q.device)
            _req(part_o, "scratch[0]", (torch.float32,), (None, 2 * TILE_GROUP * 16, d))
            _req(part_ml, "scratch[1]", (torch.float32,), (None, 2 * TILE_GROUP * 16, 2))
            if part_o.shape[0] < slots or part_ml.shape[0] < slots:
                raise KernelError("prefill_attention_tc: the scratch tensors hold fewer slots than the segments name")
    args = (q.data_ptr(), T, cache.data_ptr(), cache.shape[0], block_table.data_ptr(), block_table.shape[1],
            tiles.data_ptr(), tiles.shape[0], _ptr(segments), 0 if segments is None else segments.shape[0],
            _ptr(items) if n_items else None, n_items, int(slots) if segments is not None else 0, _ptr(part_o),
            _ptr(part_ml), out.data_ptr(), H, K, d, P, int(window or 0), float(scale), float(softcap or 0.0),
            _ptr(status))
    if sink is not None:
        _req(sink, "sink", (torch.float32,), (H,))
        _check(_get("air_prefill_attention_tc_sink")(*args, sink.data_ptr(), _stream()), "prefill_attention_tc")
    else:
        _check(_get("air_prefill_attention_tc")(*args, _stream()), "prefill_attention_tc")
    return out
