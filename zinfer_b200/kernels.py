"""Python face of the hand-written sm_100a kernels in `csrc/`.

Every function checks its tensors (device, dtype, layout, sizes), launches one kernel on the
current CUDA stream through the library's C entry point and raises `KernelError` if the
launcher refuses the sizes or CUDA reports an error.  There is no other implementation behind
these functions: without a CUDA device, a compiler or a loadable library they raise.
"""
from __future__ import annotations

import ctypes
import functools
from typing import Optional

import torch

from .csrc.build import KernelBuildError, load_library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_C = {"p": ctypes.c_void_p, "i": ctypes.c_int, "f": ctypes.c_float, "l": ctypes.c_longlong}

# library -> function -> argument kinds (p pointer, i int, f float, l long long); the last
# pointer of every launcher is the stream
_SIGNATURES = {
    "elementwise": {
        "zk_embed": "pppiiifip" + "ppi" + "p",
        "zk_rmsnorm": "ppppiifip",
        "zk_silu_mul": "ppiiiip",
        "zk_fill_normal": "pllffip",
        "zk_rmsnorm_add": "pppiiffp",
        "zk_rmsnorm_pair_add": "pppppiiffp",
        "zk_activation": "ppliip",
        "zk_cast_rows": "pplip",
        "zk_softcap": "plfp",
        "zk_scale": "plfp",
        "zk_weighted_sum": "ppilpp",
        "zk_gate_add": "ppppiiip",
        "zk_scale_add": "ppplip",
        "zk_rows_add": "ppplip",
        "zk_norm_shift": "pppplppppiiifiip",
        "zk_clamped_glu": "ppiiiffip",
        "zk_head_gate": "ppiiiiip",
        "zk_layernorm": "pppppiifip",
        "zk_value_gate": "ppiiiiiip",
        "zk_unit_norm_gate": "ppipiiifip",
    },
    "latent": {
        "zk_latent_prepare": "pppi" + "ppppppp" + "iiiiii" + "f" + "iii" + "ppp",
        "zk_latent_pack": "ppipip" + "ppp" + "pppp" + "iiiiiiiiii" + "pppi" + "i" + "p",
        "zk_latent_gather": "pppppp" + "iiiiii" + "p",
        "zk_head_gemm": "piippiipiiiiiip",
    },
    "hgrn2": {
        "zk_hgrn2_scan": "pippplpppiiiiip",
        "zk_hgrn2_max_dim": "",
        "zk_retention_scan": "pippifpplpppiiiiip",
    },
    "seqconv": {
        "zk_seqconv_forward": "ppppppp" + "iiiliiip",
        "zk_seqconv_state_update": "ppppiiilp",
        "zk_seqconv_max_taps": "",
    },
    "moe": {
        "zk_moe_table": "ppppippp" + "iiiiiiiipp",
        "zk_moe_gather": "pppiiip",
        "zk_moe_combine": "pppiiii" + "p" + "pi" + "p",
        "zk_moe_routed": "ppppippp" + "iiiiiii" + "pip",
        "zk_moe_router": "pppp" + "iiiii" + "pp",
        "zk_moe_expert_rows": "piiiiippp" + "ip",
    },
    "gemm_simt": {
        "zk_gemm_simt": "ppppiiiiiiiiip",
    },
    "gemm_skinny": {
        "zk_gemm_skinny": "pppfpppiiiiiiii" + "pippp" + "pi" + "p",
        "zk_gemm_skinny_swiglu": "pppfppiiiiii" + "pi" + "p",
        "zk_gemm_skinny_conv": "pppfppppppp" + "iiiiiiil" + "pi" + "p",
        "zk_gemm_skinny_max_m": "",
        "zk_gemm_skinny_fused_max_m": "",
    },
    "gemm_tc": {
        "zk_gemm_tc": "ppppiiiiiiiiii" + "pifppp" + "p" + "pi" + "ff" + "p",
        "zk_gemm_tc_fuses_epilogue": "iiiii",
        "zk_gemm_tc_force_form": "i",
        "zk_gemm_tc_grouped": "pppiiiiiiiippp",
    },
    "shortconv": {
        "zk_conv_forward": "ppppppppiiiliip",
        "zk_conv_state_update": "ppppiiiliip",
        "zk_conv_decode": "ppppppiiiliip",
    },
    "attention_decode": {
        "zk_attn_decode": "ppppppppp" + "iiiiiiifiip",
        "zk_attn_decode_takes": "iiii",
    },
    "attention_decode_noalloc": {      # for C callers that must not allocate; see csrc/attention_decode_noalloc.h
        "zk_attn_decode_noalloc": "ppppppp" + "iiiiiiifiip",
        "zk_attn_decode_noalloc_bytes": "iiii",
    },
    "attention_prefill": {
        "zk_attn_prefill": "pppppppppp" + "iiiiiiiif" + "pp" + "pp" + "ip" + "f" + "p",
        "zk_attn_prefill_takes": "iiii",
        "zk_attn_prefill_tile_tokens": "ii",
    },
    "attention_prefill_tc5": {
        "zk_attn_prefill_tc5": "pppppppppp" + "iii" + "l" + "iiii" + "f" + "p" + "pp" + "p",
        "zk_attn_prefill_tc5_takes": "iiiii",
        "zk_attn_prefill_tc5_tile_tokens": "ii",
    },
    "attention_decode_latent": {
        "zk_attn_decode_latent": "ppppppppiiiiiifiip",
        "zk_attn_decode_latent_takes": "iiii",
    },
    "attention_decode_tc": {
        "zk_attn_decode_tc": "pppppppppiiiiiiifii" + "pp" + "i" + "ip" + "f" + "p",
        "zk_attn_decode_tc_takes": "iiii",
    },
    "sampling": {
        "zk_apply_penalties": "piipifppip",
        "zk_recent_window": "",
        "zk_penalize_recent": "piipppfp",
        "zk_recent_append": "pipppp",
        "zk_argmax": "piipppp" + "pip" + "p",
        "zk_sample": "piififfffip" + "lpp" + "pp",
    },
    "attention": {
        "zk_qk_prepare": "pppppppppppp" + "iiiiiiifiiip" + "ii" + "fi" + "p",
        "zk_qk_prepare_span": "pipppppppppiiiiiifiiip" + "pi" + "p",
        "zk_attn_fwd": "pppppp" + "pppppp" + "iiiiiiiifiiiii" + "ippi" + "ipi" + "f" + "p",
        "zk_attn_merge_talk": "ppppiiiiiip",
        "zk_attn_merge": "pppiiii" + "pi" + "p",
        "zk_attn_rows_per_block": "",
        "zk_attn_max_head_dim": "",
    },
}


_RESTYPES = {"zk_attn_decode_noalloc_bytes": ctypes.c_longlong}


class KernelError(RuntimeError):
    """A kernel refused its arguments or CUDA reported a failure."""


_funcs: dict[str, object] = {}


def _fn(lib_name: str, fn_name: str):
    f = _funcs.get(fn_name)
    if f is None:
        lib = load_library(lib_name)
        for name, sig in _SIGNATURES[lib_name].items():
            g = getattr(lib, name)
            g.argtypes = [_C[c] for c in sig]
            g.restype = _RESTYPES.get(name, ctypes.c_int)
            _funcs[name] = g
        f = _funcs[fn_name]
    return f


def _error_name(code: int) -> str:
    lib = load_library("elementwise")
    lib.zk_error_name.argtypes = [ctypes.c_int]
    lib.zk_error_name.restype = ctypes.c_char_p
    s = lib.zk_error_name(code)
    return s.decode() if s else f"status {code}"


# Number of kernel launches made through this module since import (the benchmark reports it).
launch_count = 0

_device_state: dict = {}


def _check(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        raise KernelError(f"{what}: {_error_name(code)} (status {code})")
    launch_count += 1


def require_cuda() -> None:
    """Raises unless a CUDA device is usable; the product path has no CPU implementation."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: zinfer_b200 runs on sm_100a GPUs only and has no CPU path")


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device; launch plans size their grids by it."""
    dev = torch.device("cuda" if device is None else device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    n = _device_state.setdefault(("sm_count", idx), None)
    if n is None:
        n = _device_state[("sm_count", idx)] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


# The current stream's handle, asked for at every launch.  torch.cuda.current_stream() builds a Stream
# object each time (some 5 us, a fifth of the host's time per launch of an unrecorded step); the
# raw getter behind it returns the handle itself.  Where a torch build lacks it the public call does.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None, contiguous=True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        if not ok:
            raise KernelError(f"{name}: dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if shape is not None:
        if t.dim() != len(shape) or any(s is not None and s != d for s, d in zip(shape, t.shape)):
            raise KernelError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not a run dtype (float32, bfloat16)") from None


# ------------------------------------------------------------------------------- row kernels

def embed(tokens: torch.Tensor, table: torch.Tensor, status: torch.Tensor, scale: float = 1.0,
          pos_table: Optional[torch.Tensor] = None, tok_pos: Optional[torch.Tensor] = None,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[t] = float32(table[tokens[t]]) * scale; bad ids set status to 1.  With `pos_table`
    [positions, dim] (the table's dtype) the row pos_table[tok_pos[t]] is added, unscaled; a position
    outside it sets status to 3.  `out`: float32 [n, dim] to write into."""
    _need(tokens, "tokens", torch.int32)
    _need(table, "table", (torch.float32, torch.bfloat16), (None, None))
    _need(status, "status", torch.int32)
    n, (vocab, dim) = tokens.numel(), table.shape
    max_pos = 0
    if pos_table is not None:
        _need(pos_table, "pos_table", table.dtype, (None, dim))
        _need(tok_pos, "tok_pos", torch.int32, (n,))
        max_pos = pos_table.shape[0]
    if out is None:
        out = torch.empty((n, dim), dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32, (n, dim))
    _check(_fn("elementwise", "zk_embed")(_ptr(tokens), _ptr(table), _ptr(out), n, dim, vocab, scale,
                                          dtype_code(table.dtype), _ptr(status), _ptr(pos_table), _ptr(tok_pos), max_pos,
                                          _stream()), "embed")
    return out


def rmsnorm_add(m: torch.Tensor, weight: torch.Tensor, eps: float, x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """x += scale * (RMSNorm(m) * weight), row by row, all float32: the norm of a sublayer's output (or a share of
    it) summed into the residual rows."""
    _need(m, "m", torch.float32, (None, None))
    _need(x, "x", torch.float32, tuple(m.shape))
    _need(weight, "weight", torch.float32, (m.shape[1],))
    _check(_fn("elementwise", "zk_rmsnorm_add")(_ptr(m), _ptr(weight), _ptr(x), m.shape[0], m.shape[1], eps, float(scale),
                                                _stream()),
           "rmsnorm_add")
    return x


def rmsnorm_pair_add(a: torch.Tensor, b: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float,
                     x: torch.Tensor, share: float = 0.5) -> torch.Tensor:
    """x += share * (RMSNorm(a) * weight_a + RMSNorm(b) * weight_b), row by row, all float32, in one pass over x."""
    _need(a, "a", torch.float32, (None, None))
    _need(b, "b", torch.float32, tuple(a.shape))
    _need(x, "x", torch.float32, tuple(a.shape))
    _need(weight_a, "weight_a", torch.float32, (a.shape[1],))
    _need(weight_b, "weight_b", torch.float32, (a.shape[1],))
    _check(_fn("elementwise", "zk_rmsnorm_pair_add")(_ptr(a), _ptr(b), _ptr(weight_a), _ptr(weight_b), _ptr(x), a.shape[0],
                                                     a.shape[1], eps, float(share), _stream()), "rmsnorm_pair_add")
    return x


ACTIVATIONS = {"gelu": 0, "gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu": 3, "relu_squared": 4}


def activation(z: torch.Tensor, kind: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(z) elementwise in float32 arithmetic; kind is one of ACTIVATIONS ("gelu" is the erf form)."""
    _need(z, "z", (torch.float32, torch.bfloat16))
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation: unknown kind {kind!r}; known: {sorted(ACTIVATIONS)}")
    if out is None:
        out = torch.empty_like(z)
    _need(out, "out", z.dtype, tuple(z.shape))
    _check(_fn("elementwise", "zk_activation")(_ptr(z), _ptr(out), z.numel(), ACTIVATIONS[kind], dtype_code(z.dtype),
                                               _stream()), "activation")
    return out


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Float32 rows in the run dtype (the rows themselves when that is float32)."""
    _need(x, "x", torch.float32)
    if dtype == torch.float32:
        return x
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(_fn("elementwise", "zk_cast_rows")(_ptr(x), _ptr(y), x.numel(), dtype_code(dtype), _stream()), "cast_rows")
    return y


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """In place: logits <- cap * tanh(logits / cap), float32."""
    _need(logits, "logits", torch.float32)
    _check(_fn("elementwise", "zk_softcap")(_ptr(logits), logits.numel(), float(cap), _stream()), "softcap")
    return logits


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """x *= scale, in place; float32."""
    _need(x, "x", torch.float32)
    _check(_fn("elementwise", "zk_scale")(_ptr(x), x.numel(), float(scale), _stream()), "scale")
    return x


def weighted_sum(planes: torch.Tensor, weights: Optional[torch.Tensor], n_terms: int, out: torch.Tensor) -> torch.Tensor:
    """out = sum_{j < n_terms} weights[j] * planes[j], added in the order of j; planes float32
    [>= n_terms, ...] contiguous, weights float32 [>= n_terms] on the device (None with n_terms 1: a copy)."""
    _need(planes, "planes", torch.float32)
    if planes.dim() < 2 or planes.shape[0] < n_terms or n_terms < 1:
        raise KernelError(f"weighted_sum: {n_terms} terms of planes {tuple(planes.shape)}")
    _need(out, "out", torch.float32, tuple(planes.shape[1:]))
    if weights is not None:
        _need(weights, "weights", torch.float32)
        if weights.numel() < n_terms:
            raise KernelError(f"weighted_sum: {weights.numel()} weights for {n_terms} terms")
    elif n_terms != 1:
        raise KernelError("weighted_sum: several terms need weights")
    _check(_fn("elementwise", "zk_weighted_sum")(_ptr(planes), _ptr(weights), n_terms, out.numel(), _ptr(out), _stream()),
           "weighted_sum")
    return out


def gate_add(x: torch.Tensor, gate: torch.Tensor, branch: torch.Tensor, m: torch.Tensor) -> torch.Tensor:
    """m[t] += sigmoid(x[t] . gate) * branch[t]; x float32 [n, D], gate float32 [D], branch and m float32 [n, O]."""
    _need(x, "x", torch.float32, (None, None))
    n, D = x.shape
    _need(gate, "gate", torch.float32, (D,))
    _need(m, "m", torch.float32, (n, None))
    _need(branch, "branch", torch.float32, tuple(m.shape))
    _check(_fn("elementwise", "zk_gate_add")(_ptr(x), _ptr(gate), _ptr(branch), _ptr(m), n, D, m.shape[1], _stream()),
           "gate_add")
    return m


def scale_add(m: torch.Tensor, scale: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """x[t, c] += scale[c] * m[t, c], all float32: a sublayer's result summed into the residual rows through a
    learned scale per channel."""
    _need(m, "m", torch.float32, (None, None))
    _need(x, "x", torch.float32, tuple(m.shape))
    _need(scale, "scale", torch.float32, (m.shape[1],))
    _check(_fn("elementwise", "zk_scale_add")(_ptr(m), _ptr(scale), _ptr(x), m.numel(), m.shape[1], _stream()), "scale_add")
    return x


def rows_add(x: torch.Tensor, vec: torch.Tensor, base: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[t, :] = (x[t, :] + base[t, :]) + vec[:] in place (without `base`: x[t, :] += vec), float32."""
    _need(x, "x", torch.float32, (None, None))
    _need(vec, "vec", torch.float32, (x.shape[1],))
    if base is not None:
        _need(base, "base", torch.float32, tuple(x.shape))
    _check(_fn("elementwise", "zk_rows_add")(_ptr(x), _ptr(base), _ptr(vec), x.numel(), x.shape[1], _stream()), "rows_add")
    return x


def norm_shift(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, mu: torch.Tensor, state: torch.Tensor,
               tok_seq, cu_q, seq_slot, n_seqs: int, out_dtype: torch.dtype, single_token: bool = False) -> torch.Tensor:
    """Token shift of (optionally RMS-normalised) rows: n_t = rms(x_t) * weight (x_t itself without a weight),
    h_t = n_t + (n_prev - n_t) * mu with n_prev the n of the sequence's token before, taken from the step's own
    rows or, for the first token a sequence brings, from `state` [slots, >= D] (float32, a row per slot,
    rows `state.stride(0)` apart), which afterwards holds the n of each sequence's last token.
    x float32 [n, D] packed; h [n, D] in `out_dtype`."""
    _need(x, "x", torch.float32, (None, None))
    n, D = x.shape
    if weight is not None:
        _need(weight, "weight", torch.float32, (D,))
    _need(mu, "mu", torch.float32, (D,))
    _need(state, "state", torch.float32, contiguous=False)
    if state.dim() != 2 or state.shape[1] < D or state.stride(1) != 1:
        raise KernelError(f"norm_shift: state {tuple(state.shape)} must hold a row of {D} values per slot")
    for t, nm in ((tok_seq, "tok_seq"), (cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    h = torch.empty((n, D), dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "zk_norm_shift")(_ptr(x), _ptr(weight), _ptr(mu), _ptr(state), state.stride(0), _ptr(tok_seq),
                                               _ptr(cu_q), _ptr(seq_slot), _ptr(h), n, n_seqs, D, eps,
                                               1 if single_token else 0, dtype_code(out_dtype), _stream()), "norm_shift")
    return h


# ------------------------------------------------------------------------------- gated linear recurrence

def hgrn2_max_dim() -> int:
    return _constant("hgrn2", "zk_hgrn2_max_dim")


def hgrn2_scan(qfv: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor, state: torch.Tensor, cu_q, seq_slot,
               n_seqs: int, n_heads: int, dim: int, value_dim: int) -> torch.Tensor:
    """Per head S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T, o_t = S_t^T q_t over each sequence's tokens, from the state
    the step before left to the state this one leaves.  qfv float32 [n, 2*H*d + H*e], a row [q | f | v] as the
    projections gave them; its q and f parts are overwritten (q <- silu(q), f <- lower + (1 - lower) *
    sigmoid(f + f_bias), by a kernel of their own before the recurrence); state float32
    [slots, H*d*e] (rows `state.stride(0)` apart), a slot's values ordered [H, d, e]; returns o float32 [n, H*e]."""
    H, d, e = n_heads, dim, value_dim
    _need(qfv, "qfv", torch.float32, (None, 2 * H * d + H * e))
    _need(f_bias, "f_bias", torch.float32, (H * d,))
    _need(lower, "lower", torch.float32, (H * d,))
    _need(state, "state", torch.float32, contiguous=False)
    if state.dim() != 2 or state.shape[1] != H * d * e or state.stride(1) != 1:
        raise KernelError(f"hgrn2_scan: state {tuple(state.shape)} must hold {H * d * e} values per slot")
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    o = torch.empty((qfv.shape[0], H * e), dtype=torch.float32, device=qfv.device)
    _check(_fn("hgrn2", "zk_hgrn2_scan")(_ptr(qfv), qfv.stride(0), _ptr(f_bias), _ptr(lower), _ptr(state), state.stride(0),
                                         _ptr(o), _ptr(cu_q), _ptr(seq_slot), qfv.shape[0], n_seqs, H, d, e, _stream()), "hgrn2_scan")
    return o


def retention_scan(qkv: torch.Tensor, decay: torch.Tensor, inv_freq: Optional[torch.Tensor], n_rot: int, key_scale: float,
                   tok_pos, state: torch.Tensor, cu_q, seq_slot, n_seqs: int, n_heads: int, dim: int,
                   value_dim: int) -> torch.Tensor:
    """Per head S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t over each sequence's tokens, from the state the step
    before left to the state this one leaves.  qkv float32 [n, >= 2*H*d + H*e] (row stride used), a row [q | k | v | ..]
    as the projections gave them; q and k are overwritten: the first `n_rot` entries of every head rotated by the
    token's position (half-split pairs, `inv_freq` float32 [n_rot / 2]; None = no rotation), k then times `key_scale`.
    decay float32 [H]; state float32 [slots, H*d*e]; returns o float32 [n, H*e]."""
    H, d, e = n_heads, dim, value_dim
    _need(qkv, "qkv", torch.float32, (None, None), contiguous=False)
    if qkv.shape[1] < 2 * H * d + H * e or qkv.stride(1) != 1:
        raise KernelError(f"retention_scan: rows of {qkv.shape[1]} values hold no q, k and v of {H} heads")
    _need(decay, "decay", torch.float32, (H,))
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, (n_rot // 2,))
    _need(state, "state", torch.float32, contiguous=False)
    if state.dim() != 2 or state.shape[1] != H * d * e or state.stride(1) != 1:
        raise KernelError(f"retention_scan: state {tuple(state.shape)} must hold {H * d * e} values per slot")
    for t, nm in ((cu_q, "cu_q"), (seq_slot, "seq_slot"), (tok_pos, "tok_pos")):
        _need(t, nm, torch.int32)
    o = torch.empty((qkv.shape[0], H * e), dtype=torch.float32, device=qkv.device)
    _check(_fn("hgrn2", "zk_retention_scan")(_ptr(qkv), qkv.stride(0), _ptr(decay), _ptr(inv_freq), int(n_rot), float(key_scale),
                                             _ptr(tok_pos), _ptr(state), state.stride(0), _ptr(o), _ptr(cu_q), _ptr(seq_slot),
                                             qkv.shape[0], n_seqs, H, d, e, _stream()), "retention_scan")
    return o


# ------------------------------------------------------------------------------- convolution over time on a mixer's input

def seqconv_max_taps() -> int:
    return _constant("seqconv", "zk_seqconv_max_taps")


def seqconv(x: torch.Tensor, state: torch.Tensor, taps: torch.Tensor, tok_seq, cu_q, seq_slot, n_seqs: int,
            out_dtype: torch.dtype, residual: bool = True, single_token: bool = False) -> torch.Tensor:
    """h_t = (x_t +) sum_j taps[j] * x_{t - (K-1) + j} per channel over each sequence's tokens, the
    K-1 inputs before the step taken from `state` [slots, K-1, D], which then moves on to the step's
    last inputs.  x float32 [n, D] packed; taps float32 [K, D]; h [n, D] in `out_dtype`."""
    _need(x, "x", torch.float32, (None, None))
    n, D = x.shape
    _need(taps, "taps", torch.float32, (None, D))
    K = taps.shape[0]
    _need(state, "state", torch.float32, (None, K - 1, D))
    for t, nm in ((tok_seq, "tok_seq"), (cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    h = torch.empty((n, D), dtype=out_dtype, device=x.device)
    _check(_fn("seqconv", "zk_seqconv_forward")(_ptr(x), _ptr(state), _ptr(taps), _ptr(tok_seq), _ptr(cu_q),
                                                _ptr(seq_slot), _ptr(h), n, D, K, state.stride(0),
                                                1 if residual else 0, 1 if single_token else 0, dtype_code(out_dtype),
                                                _stream()), "seqconv")
    if not single_token and K > 1:
        _check(_fn("seqconv", "zk_seqconv_state_update")(_ptr(x), _ptr(state), _ptr(cu_q), _ptr(seq_slot), n_seqs, D, K,
                                                         state.stride(0), _stream()), "seqconv state")
    return h


# ------------------------------------------------------------------------------- experts picked by a table

def moe_table(x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, w_gate_up: torch.Tensor, interleave: int,
              w_down: torch.Tensor, status: torch.Tensor, out: Optional[torch.Tensor] = None,
              accumulate: bool = False) -> torch.Tensor:
    """y[t] = (1/top) sum_k W_down[e] (silu(W_gate[e] x_t) * (W_up[e] x_t)), e = table[tokens[t]][k].
    x [n, D] run dtype; table int32 [vocab, top]; w_gate_up [E, 2F, D], an expert's rows [gate | up] or, with
    `interleave` = g, groups of g gate rows followed by their g up rows; w_down [E, D, F]; y float32 [n, D]."""
    _need(x, "x", (torch.float32, torch.bfloat16), (None, None))
    n, D = x.shape
    _need(tokens, "tokens", torch.int32, (n,))
    _need(table, "table", torch.int32, (None, None))
    vocab, top = table.shape
    _need(w_gate_up, "w_gate_up", x.dtype, (None, None, D))
    E, F = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    _need(w_down, "w_down", x.dtype, (E, D, F))
    if out is None:
        if accumulate:
            raise KernelError("moe_table: accumulate needs an output tensor")
        out = torch.empty((n, D), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, (n, D))
    h = torch.empty((n, top, F), dtype=x.dtype, device=x.device)
    _check(_fn("moe", "zk_moe_table")(_ptr(x), _ptr(tokens), _ptr(table), _ptr(w_gate_up), int(interleave), _ptr(w_down), _ptr(h),
                                      _ptr(out), n, D, F, top, vocab, E, 1 if accumulate else 0, dtype_code(x.dtype),
                                      _ptr(status), _stream()), "moe_table")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows (all, or those listed in `rows`) into `out_dtype`."""
    _need(x, "x", torch.float32, (None, None))
    dim = x.shape[1]
    _need(weight, "weight", torch.float32, (dim,))
    n_out = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    y = torch.empty((n_out, dim), dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "zk_rmsnorm")(_ptr(x), _ptr(rows), _ptr(weight), _ptr(y), n_out, dim, eps,
                                            dtype_code(out_dtype), _stream()), "rmsnorm")
    return y


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Layer norm of float32 rows (all, or those listed in `rows`) into `out_dtype`: (x - mean) / sqrt(var + eps) *
    weight + bias with var the mean of the squared deviations; `bias` None = none."""
    _need(x, "x", torch.float32, (None, None))
    dim = x.shape[1]
    _need(weight, "weight", torch.float32, (dim,))
    if bias is not None:
        _need(bias, "bias", torch.float32, (dim,))
    n_out = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    y = torch.empty((n_out, dim), dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "zk_layernorm")(_ptr(x), _ptr(rows), _ptr(weight), _ptr(bias), _ptr(y), n_out, dim, eps,
                                              dtype_code(out_dtype), _stream()), "layernorm")
    return y


def value_gate(rows: torch.Tensor, gate: torch.Tensor, n_heads: int, valid: int) -> torch.Tensor:
    """rows[t, h, j] *= sigmoid(gate[t, h * valid + j]) for j < valid, in place.  rows [n, H * width] contiguous (run
    dtype; the values of a head behind `valid` are padding and left alone); gate float32 [n, >= H * valid] (a view of
    wider rows is fine: its row stride is used)."""
    _need(rows, "rows", (torch.float32, torch.bfloat16), (None, None))
    n, w = rows.shape
    _need(gate, "gate", torch.float32, (n, None), contiguous=False)
    if w % n_heads or valid > w // n_heads or gate.shape[1] < n_heads * valid or gate.stride(1) != 1:
        raise KernelError(f"value_gate: rows {tuple(rows.shape)} / gate {tuple(gate.shape)} do not fit {n_heads} heads "
                          f"of {valid} values")
    _check(_fn("elementwise", "zk_value_gate")(_ptr(rows), _ptr(gate), gate.stride(0), n, n_heads, w // n_heads, valid,
                                               dtype_code(rows.dtype), _stream()), "value_gate")
    return rows


def unit_norm_gate(o: torch.Tensor, gate: torch.Tensor, n_heads: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """y[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * silu(gate[t, h, :]): every head over its root mean
    square (no weight), gated.  o float32 [n, H * e]; gate float32 [n, >= H * e] (may be a view of wider rows);
    returns [n, H * e] in `out_dtype`."""
    _need(o, "o", torch.float32, (None, None))
    n, w = o.shape
    _need(gate, "gate", torch.float32, (n, None), contiguous=False)
    if w % n_heads or gate.shape[1] < w or gate.stride(1) != 1:
        raise KernelError(f"unit_norm_gate: o {tuple(o.shape)} / gate {tuple(gate.shape)} do not fit {n_heads} heads")
    y = torch.empty((n, w), dtype=out_dtype, device=o.device)
    _check(_fn("elementwise", "zk_unit_norm_gate")(_ptr(o), _ptr(gate), gate.stride(0), _ptr(y), n, n_heads, w // n_heads,
                                                   eps, dtype_code(out_dtype), _stream()), "unit_norm_gate")
    return y


def silu_mul(gu: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """h = silu(gate) * up.  A row of gu is [gate (F) | up (F)], or with `interleave` = g groups of
    g gates followed by their g ups."""
    _need(gu, "gu", (torch.float32, torch.bfloat16), (None, None))
    n, two_f = gu.shape
    if two_f % 2 or (interleave and (two_f // 2) % interleave):
        raise KernelError(f"silu_mul: width {two_f} does not split into gate and up (groups of {interleave})")
    h = torch.empty((n, two_f // 2), dtype=gu.dtype, device=gu.device)
    _check(_fn("elementwise", "zk_silu_mul")(_ptr(gu), _ptr(h), n, two_f // 2, interleave, dtype_code(gu.dtype),
                                             _stream()), "silu_mul")
    return h


def clamped_glu(gu: torch.Tensor, limit: float, alpha: float, interleave: int = 0) -> torch.Tensor:
    """h = g' * sigmoid(alpha * g') * (u' + 1) with g' = min(gate, limit), u' = clamp(up, -limit, limit), in float32
    arithmetic.  Rows of gu as in `silu_mul`."""
    _need(gu, "gu", (torch.float32, torch.bfloat16), (None, None))
    n, two_f = gu.shape
    if two_f % 2 or (interleave and (two_f // 2) % interleave):
        raise KernelError(f"clamped_glu: width {two_f} does not split into gate and up (groups of {interleave})")
    h = torch.empty((n, two_f // 2), dtype=gu.dtype, device=gu.device)
    _check(_fn("elementwise", "zk_clamped_glu")(_ptr(gu), _ptr(h), n, two_f // 2, interleave, float(limit), float(alpha),
                                                dtype_code(gu.dtype), _stream()), "clamped_glu")
    return h


def head_gate(rows: torch.Tensor, gate: torch.Tensor, n_heads: int) -> torch.Tensor:
    """rows[t, h, :] *= sigmoid(gate[t, h]) in place.  rows [n, H * width] contiguous; gate float32 [n, >= H] (a view
    of wider rows is fine: its row stride is used)."""
    _need(rows, "rows", (torch.float32, torch.bfloat16), (None, None))
    n, w = rows.shape
    _need(gate, "gate", torch.float32, (n, None), contiguous=False)
    if w % n_heads or gate.shape[1] < n_heads or gate.stride(1) != 1:
        raise KernelError(f"head_gate: rows {tuple(rows.shape)} / gate {tuple(gate.shape)} do not fit {n_heads} heads")
    _check(_fn("elementwise", "zk_head_gate")(_ptr(rows), _ptr(gate), gate.stride(0), n, n_heads, w // n_heads,
                                              dtype_code(rows.dtype), _stream()), "head_gate")
    return rows


def fill_normal(out: torch.Tensor, seed: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    """Fills `out` with mean + std * N(0, 1), a function of (seed, element index) only."""
    _need(out, "out", (torch.float32, torch.bfloat16))
    _check(_fn("elementwise", "zk_fill_normal")(_ptr(out), out.numel(), seed & 0x7FFFFFFFFFFFFFFF, mean, std,
                                                dtype_code(out.dtype), _stream()), "fill_normal")
    return out


# ------------------------------------------------------------------------------- contractions

def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
              accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) with float32 FMA on the CUDA cores.  a [M, K], w [N, K] share a
    dtype; out is that dtype or float32; accumulate needs a float32 or same-dtype `out`."""
    _need(a, "a", (torch.float32, torch.bfloat16), (None, None))
    _need(w, "w", a.dtype, (None, a.shape[1]))
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    _need(out, "out", (torch.float32, a.dtype), (M, N))
    if a.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("gemm: float32 inputs need a float32 output")
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    _check(_fn("gemm_simt", "zk_gemm_simt")(_ptr(a), _ptr(w), _ptr(out), _ptr(bias), M, N, K, a.stride(0), w.stride(0),
                                            out.stride(0), dtype_code(a.dtype), dtype_code(out.dtype),
                                            1 if accumulate else 0, _stream()), "gemm_simt")
    return out


def status_word(device) -> torch.Tensor:
    """The int32 status word of a device: kernels that can detect a fault of their inputs or give
    up a bounded wait write a code here; `Engine.check_status` reads and clears it."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    st = _device_state.setdefault(dev, {})
    if "status" not in st:
        st["status"] = torch.zeros(1, dtype=torch.int32, device=dev)
    return st["status"]


GEMM_TC_SWAPPED_MAX_M = 64     # up to this many rows the weights take the 128-row side of the tiles


def gemm_tc_takes(a, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> bool:
    """Whether the tcgen05 kernel takes this contraction: bfloat16, K a multiple of 8, rows and
    output 16-byte aligned.  `a` is a bfloat16 tensor, or a ScaledInput of up to 64 rows."""
    if isinstance(a, ScaledInput):
        if a.xw.shape[0] > GEMM_TC_SWAPPED_MAX_M or not a.ssq.is_contiguous():
            return False
        a = a.xw
    ok = (isinstance(a, torch.Tensor) and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2
          and w.dim() == 2 and a.shape[1] == w.shape[1] and a.shape[1] % 8 == 0 and a.stride(1) == 1
          and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
          and w.data_ptr() % 16 == 0 and w.shape[0] <= 4096 * 128)
    if ok and out is not None:
        ok = out.stride(1) == 1 and out.data_ptr() % 16 == 0
    return ok


def gemm_tc_emits(a, out: Optional[torch.Tensor]) -> bool:
    """Whether `gemm_tc` can write a NormEmit beside `out` for this input."""
    return (a.shape[0] <= GEMM_TC_SWAPPED_MAX_M and out is not None and out.dtype == torch.float32
            and out.is_contiguous())


def gemm_tc(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
            accumulate: bool = False, bias: Optional[torch.Tensor] = None, splits: int = 1,
            swiglu: bool = False, emit: Optional["NormEmit"] = None, col_scale: Optional[torch.Tensor] = None,
            act: Optional[str] = None, glu_clamp: Optional[tuple] = None) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) with TMA-fed tcgen05 MMAs and the accumulator in tensor memory.
    `glu_clamp` = (limit, alpha), with `swiglu`: the unit is min(g, limit) * sigmoid(alpha * min(g, limit)) *
    (clamp(u, -limit, limit) + 1) in place of silu(g) * u.
    `act` ("relu_squared") and `col_scale` (float32 [N]) as in `gemm_skinny`, where `gemm_tc_fuses` says so.
    More than 64 rows: persistent blocks on 256-wide tiles when N is a multiple of 256 (pairs of
    blocks with tcgen05.mma.cta_group::2 above 128 rows, TMA stores), else one 128 x 128 tile of
    tokens x weight rows per block.  Up to 64 rows: the weights take
    the 128-row side and K is cut into `splits` (1, 2, 4 or 8) parts, one per block of a cluster,
    that are added in order.  With `swiglu` w holds groups of 16 gate rows and
    their 16 up rows and the result is silu(gate) * up, [M, N/2].  Up to 64 rows `a` may be a
    ScaledInput (the sums are scaled by the rows' 1/rms) and `emit` (see `gemm_tc_emits`) is filled
    for the norm that reads `out` next."""
    if not gemm_tc_takes(a, w, out):
        raise KernelError(f"gemm_tc: a {tuple(a.shape)} / w {tuple(w.shape)} need bfloat16, K a multiple of 8 and "
                          "16-byte aligned rows")
    ssq, ssq_parts, eps = None, 0, 0.0
    if isinstance(a, ScaledInput):
        ssq, ssq_parts, eps, a = _ptr(a.ssq), a.ssq.shape[1], a.eps, a.xw
    M, K = a.shape
    N = w.shape[0]
    if swiglu and (N % 32 or accumulate or bias is not None):
        raise KernelError("gemm_tc: the SwiGLU epilogue needs N a multiple of 32, no bias and no accumulation")
    if glu_clamp is not None and (not swiglu or not glu_clamp[0] > 0):
        raise KernelError("gemm_tc: the clamped unit goes with the gated epilogue and a positive limit")
    n_out = N // 2 if swiglu else N
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
    _need(out, "out", (torch.float32, torch.bfloat16), (M, n_out))
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    if act not in (None, "relu_squared"):
        raise KernelError(f"gemm_tc: no epilogue for the activation {act!r}")
    if col_scale is not None:
        _need(col_scale, "col_scale", torch.float32, (N,))
    if (col_scale is not None or act is not None) and (swiglu or emit is not None or not gemm_tc_fuses(a, w, out, accumulate)):
        raise KernelError("gemm_tc: an activation or a scale per column is taken by the persistent forms only")
    if emit is not None:
        if not gemm_tc_emits(a, out) or swiglu:
            raise KernelError("gemm_tc: the norm's inputs are written for at most 64 rows summed into contiguous "
                              "float32 rows")
        _need(emit.weight, "norm weight", torch.float32, (N,))
        emit.xw = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
        emit.ssq = torch.empty((M, -(-N // 32)), dtype=torch.float32, device=w.device)
    _check(_fn("gemm_tc", "zk_gemm_tc")(_ptr(a), _ptr(w), _ptr(out), _ptr(bias), M, N, K, a.stride(0), w.stride(0),
                                        out.stride(0), dtype_code(out.dtype), 1 if accumulate else 0, splits,
                                        1 if swiglu else 0, ssq, ssq_parts, eps,
                                        _ptr(emit.weight) if emit else None, _ptr(emit.xw) if emit else None,
                                        _ptr(emit.ssq) if emit else None, _ptr(status_word(a.device)), _ptr(col_scale),
                                        1 if act else 0, float(glu_clamp[0]) if glu_clamp else 0.0,
                                        float(glu_clamp[1]) if glu_clamp else 0.0, _stream()),
           "gemm_tc")
    return out


def gemm_tc_fuses(a, w: torch.Tensor, out: Optional[torch.Tensor], accumulate: bool, out_dtype=None) -> bool:
    """Whether `gemm_tc` of these operands runs a form whose epilogue takes `act` and `col_scale`."""
    if isinstance(a, ScaledInput) or not gemm_tc_takes(a, w, out):
        return False
    dt = out.dtype if out is not None else (out_dtype or torch.bfloat16)
    ldc = out.stride(0) if out is not None else w.shape[0]
    return bool(_fn("gemm_tc", "zk_gemm_tc_fuses_epilogue")(a.shape[0], w.shape[0], ldc, dtype_code(dt), 1 if accumulate else 0))


GEMM_TC_GROUP_ROWS = 128       # rows per token tile of a grouped product


def gemm_tc_grouped_takes(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 3 and w.is_contiguous()
            and a.is_contiguous() and a.shape[1] == w.shape[2] and a.shape[1] % 8 == 0 and a.shape[0] % GEMM_TC_GROUP_ROWS == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_grouped(a: torch.Tensor, w: torch.Tensor, tile_group: torch.Tensor, swiglu: bool = False,
                    out_dtype=torch.bfloat16) -> torch.Tensor:
    """out[rows of tile t] = a[rows of tile t] @ w[tile_group[t]].T on the tcgen05 kernel: a [M, K] bfloat16 in
    tiles of 128 rows, w [groups, N, K] bfloat16, tile_group int32 [M / 128] on the device.  With `swiglu`
    every w[g] holds groups of 16 gate rows and their 16 up rows and the result is silu(gate) * up, [M, N/2]."""
    if not gemm_tc_grouped_takes(a, w):
        raise KernelError(f"gemm_tc_grouped: a {tuple(a.shape)} / w {tuple(w.shape)} need bfloat16, whole tiles of "
                          f"{GEMM_TC_GROUP_ROWS} rows, K a multiple of 8")
    M, K = a.shape
    G, N, _ = w.shape
    _need(tile_group, "tile_group", torch.int32, (M // GEMM_TC_GROUP_ROWS,))
    if swiglu and N % 32:
        raise KernelError("gemm_tc_grouped: the SwiGLU epilogue needs N a multiple of 32")
    out = torch.empty((M, N // 2 if swiglu else N), dtype=out_dtype, device=a.device)
    _need(out, "out", (torch.float32, torch.bfloat16))
    _check(_fn("gemm_tc", "zk_gemm_tc_grouped")(_ptr(a), _ptr(w), _ptr(out), M, N, K, G, a.stride(0), out.stride(0),
                                                dtype_code(out.dtype), 1 if swiglu else 0, _ptr(tile_group),
                                                _ptr(status_word(a.device)), _stream()), "gemm_tc_grouped")
    return out


def gemm_tc_force_form(form: int) -> None:
    """For measurements and tests: the form that products of more than 64 rows with N a multiple of
    256 take.  0 = one 128 x 128 tile per block, 256 = persistent blocks with 128 x 256 tiles, 512 =
    persistent pairs of blocks with 256 x 256 tiles (tcgen05.mma.cta_group::2); -1 = the library chooses."""
    _check(_fn("gemm_tc", "zk_gemm_tc_force_form")(int(form)), "gemm_tc_force_form")


_constants: dict[str, int] = {}     # what the libraries say about themselves, asked once


def _constant(lib_name: str, fn_name: str) -> int:
    v = _constants.get(fn_name)
    if v is None:
        v = _constants[fn_name] = _fn(lib_name, fn_name)()
    return v


def gemm_skinny_max_m() -> int:
    return _constant("gemm_skinny", "zk_gemm_skinny_max_m")


def gemm_skinny_fused_max_m() -> int:
    """Most rows for which the skinny kernels fuse RMSNorm, SwiGLU or the short convolution."""
    return _constant("gemm_skinny", "zk_gemm_skinny_fused_max_m")


class NormInput:
    """Rows of the float32 residual stream with an RMSNorm still to be applied: x [M, K], weight
    [K], eps.  The skinny kernels take it in place of a bfloat16 input and normalise themselves."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float):
        _need(x, "x", torch.float32, (None, None))
        _need(weight, "norm weight", torch.float32, (x.shape[1],))
        self.x, self.weight, self.eps = x, weight, float(eps)

    @property
    def shape(self):
        return self.x.shape


class ScaledInput:
    """Rows of the residual stream as the kernel that summed them left them for the next RMSNorm:
    xw [M, K] = bfloat16(x * norm weight) and ssq [M, parts] float32, partial sums of x^2 whose
    sum over `parts` is the row's.  The skinny kernels take it in place of a bfloat16 input and
    scale their sums by 1 / sqrt(sum(ssq) / K + eps)."""

    def __init__(self, xw: torch.Tensor, ssq: torch.Tensor, eps: float):
        _need(xw, "xw", torch.bfloat16, (None, None))
        _need(ssq, "ssq", torch.float32, (xw.shape[0], None))
        self.xw, self.ssq, self.eps = xw, ssq, float(eps)

    @property
    def shape(self):
        return self.xw.shape


class NormEmit:
    """What an accumulating contraction into the residual rows writes for the norm that reads them
    next: `weight` [N] of that norm; after the call `xw` [M, N] = bfloat16(rows * weight) and `ssq`
    [M, parts], partial sums of the rows' squares (how many parts is the kernel's business)."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.xw: Optional[torch.Tensor] = None
        self.ssq: Optional[torch.Tensor] = None


GEMM_SKINNY_EMIT_MAX_M = 16


def _skinny_input(a):
    """(X pointer, Xf pointer, norm weight pointer, eps, M, K, ldx, ssq pointer, ssq parts) of a
    bfloat16 tensor, a NormInput or a ScaledInput."""
    if isinstance(a, NormInput):
        return None, _ptr(a.x), _ptr(a.weight), a.eps, a.x.shape[0], a.x.shape[1], a.x.stride(0), None, 0
    if isinstance(a, ScaledInput):
        return _ptr(a.xw), None, None, a.eps, a.xw.shape[0], a.xw.shape[1], a.xw.stride(0), _ptr(a.ssq), a.ssq.shape[1]
    return _ptr(a), None, None, 0.0, a.shape[0], a.shape[1], a.stride(0), None, 0


def gemm_skinny_takes(a, w: torch.Tensor) -> bool:
    """Whether the skinny kernels take this contraction: bfloat16 weights, few rows, 16-byte
    aligned rows.  `a` is a bfloat16 tensor [M <= 64, K], a NormInput or a ScaledInput [M <= 16, K]."""
    if not (w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0):
        return False
    if isinstance(a, NormInput):
        x = a.x
        return (x.shape[0] <= gemm_skinny_fused_max_m() and x.shape[1] == w.shape[1] and x.stride(1) == 1
                and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0 and a.weight.data_ptr() % 16 == 0)
    if isinstance(a, ScaledInput):
        if a.xw.shape[0] > gemm_skinny_fused_max_m() or not a.ssq.is_contiguous():
            return False
        a = a.xw
    return (a.dtype == torch.bfloat16 and a.dim() == 2 and a.shape[0] <= gemm_skinny_max_m()
            and a.shape[1] == w.shape[1] and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0)


def gemm_skinny_fused_takes(a, w: torch.Tensor) -> bool:
    """Whether the fused SwiGLU / short-convolution variants take this input (at most 16 rows)."""
    return gemm_skinny_takes(a, w) and a.shape[0] <= gemm_skinny_fused_max_m()


def gemm_skinny_emits(a, out: Optional[torch.Tensor]) -> bool:
    """Whether `gemm_skinny` can write a NormEmit beside `out` for this input."""
    return (isinstance(a, torch.Tensor) and a.shape[0] <= GEMM_SKINNY_EMIT_MAX_M and out is not None
            and out.dtype == torch.float32 and out.is_contiguous())


def gemm_skinny(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
                accumulate: bool = False, bias: Optional[torch.Tensor] = None,
                emit: Optional[NormEmit] = None, col_scale: Optional[torch.Tensor] = None,
                act: Optional[str] = None) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) for a [M <= 64, K] on the tensor cores, every weight read once.
    `act` ("relu_squared") is applied to the sums, then `col_scale` (float32 [N], one number per column)
    multiplies them, before they are stored or added to `out`.
    With a NormInput the RMSNorm of the rows is applied inside the kernel; with a ScaledInput the
    sums are scaled by the rows' 1/rms.  `emit` (see `gemm_skinny_emits`) is filled for the norm
    that reads `out` next."""
    if not gemm_skinny_takes(a, w):
        raise KernelError(f"gemm_skinny: a {tuple(a.shape)} / w {tuple(w.shape)} need few rows, "
                          "K a multiple of 8 and 16-byte aligned rows")
    X, Xf, nw, eps, M, K, ldx, ssq, ssq_parts = _skinny_input(a)
    N = w.shape[0]
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=w.device)
    _need(out, "out", (torch.float32, torch.bfloat16), (M, N))
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    if act not in (None, "relu_squared"):
        raise KernelError(f"gemm_skinny: no epilogue for the activation {act!r}")
    if col_scale is not None:
        _need(col_scale, "col_scale", torch.float32, (N,))
    if emit is not None and (col_scale is not None or act is not None):
        raise KernelError("gemm_skinny: the next norm's inputs are not written behind a scale or an activation")
    if emit is not None:
        if not gemm_skinny_emits(a, out):
            raise KernelError("gemm_skinny: the norm's inputs are written for at most 16 bfloat16 rows "
                              "summed into contiguous float32 rows")
        _need(emit.weight, "norm weight", torch.float32, (N,))
        emit.xw = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
        emit.ssq = torch.empty((M, -(-N // 16)), dtype=torch.float32, device=w.device)
    _check(_fn("gemm_skinny", "zk_gemm_skinny")(X, Xf, nw, eps, _ptr(w), _ptr(out), _ptr(bias), M, N, K, ldx,
                                                w.stride(0), out.stride(0), dtype_code(out.dtype),
                                                1 if accumulate else 0, ssq, ssq_parts,
                                                _ptr(emit.weight) if emit else None, _ptr(emit.xw) if emit else None,
                                                _ptr(emit.ssq) if emit else None, _ptr(col_scale), 1 if act else 0,
                                                _stream()), "gemm_skinny")
    return out


def gemm_skinny_swiglu(a, w_gate_up: torch.Tensor) -> torch.Tensor:
    """h = silu(a W_gate^T) * (a W_up^T) in one kernel; w_gate_up [2F, K] holds groups of 16 gate
    rows followed by their 16 up rows."""
    if not gemm_skinny_fused_takes(a, w_gate_up) or w_gate_up.shape[0] % 32:
        raise KernelError("gemm_skinny_swiglu: at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    X, Xf, nw, eps, M, K, ldx, ssq, ssq_parts = _skinny_input(a)
    F = w_gate_up.shape[0] // 2
    h = torch.empty((M, F), dtype=torch.bfloat16, device=w_gate_up.device)
    _check(_fn("gemm_skinny", "zk_gemm_skinny_swiglu")(X, Xf, nw, eps, _ptr(w_gate_up), _ptr(h), M, F, K, ldx,
                                                       w_gate_up.stride(0), h.stride(0), ssq, ssq_parts,
                                                       _stream()),
           "gemm_skinny_swiglu")
    return h


def gemm_skinny_conv(a, w_in: torch.Tensor, in_bias, state: torch.Tensor, taps: torch.Tensor, conv_bias,
                     seq_slot: torch.Tensor) -> torch.Tensor:
    """Single-token step of the gated short convolution fused with its in_proj: row m of `a` is
    sequence m; `state` [slots, K-1, D] is shifted by one; returns y [M, D].  w_in [3D, K] and
    in_bias [3D] hold groups of 16 B rows, 16 C rows, 16 X rows."""
    if not gemm_skinny_fused_takes(a, w_in) or w_in.shape[0] % 48:
        raise KernelError("gemm_skinny_conv: at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    X, Xf, nw, eps, M, K, ldx, ssq, ssq_parts = _skinny_input(a)
    D = w_in.shape[0] // 3
    _need(taps, "conv weight", torch.float32, (None, D))
    n_taps = taps.shape[0]
    _need(state, "conv state", torch.float32, (None, n_taps - 1, D))
    _need(seq_slot, "seq_slot", torch.int32, (M,))
    if in_bias is not None:
        _need(in_bias, "in_proj bias", torch.float32, (3 * D,))
    if conv_bias is not None:
        _need(conv_bias, "conv bias", torch.float32, (D,))
    y = torch.empty((M, D), dtype=torch.bfloat16, device=w_in.device)
    _check(_fn("gemm_skinny", "zk_gemm_skinny_conv")(X, Xf, nw, eps, _ptr(w_in), _ptr(in_bias), _ptr(state), _ptr(taps),
                                                     _ptr(conv_bias), _ptr(seq_slot), _ptr(y), M, D, K, n_taps, ldx,
                                                     w_in.stride(0), y.stride(0), state.stride(0), ssq, ssq_parts,
                                                     _stream()),
           "gemm_skinny_conv")
    return y


# ------------------------------------------------------------------------------- short convolution

def conv_forward(bcx, state, w, bias, tok_seq, cu_q, seq_slot, interleave: int = 0) -> torch.Tensor:
    """y of the gated short convolution for a packed batch; reads `state`, does not change it.
    bcx [n, 3D] = [B | C | X] (or groups of `interleave` channels as [B | C | X]); state
    [slots, K-1, D] float32; w [K, D] float32; bias [D] float32 or None."""
    _need(bcx, "bcx", (torch.float32, torch.bfloat16), (None, None))
    n, three_d = bcx.shape
    D = three_d // 3
    _need(w, "conv weight", torch.float32, (None, D))
    K = w.shape[0]
    _need(state, "conv state", torch.float32, (None, K - 1, D))
    if bias is not None:
        _need(bias, "conv bias", torch.float32, (D,))
    for t, nm in ((tok_seq, "tok_seq"), (cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    y = torch.empty((n, D), dtype=bcx.dtype, device=bcx.device)
    _check(_fn("shortconv", "zk_conv_forward")(_ptr(bcx), _ptr(state), _ptr(w), _ptr(bias), _ptr(tok_seq), _ptr(cu_q),
                                               _ptr(seq_slot), _ptr(y), n, D, K, state.stride(0), interleave,
                                               dtype_code(bcx.dtype), _stream()), "conv_forward")
    return y


def conv_state_update(bcx, state, cu_q, seq_slot, n_seqs: int, K: int, interleave: int = 0) -> None:
    """state[slot] <- the last K-1 values of B*X of each sequence (older rows kept if fewer came)."""
    _need(bcx, "bcx", (torch.float32, torch.bfloat16), (None, None))
    D = bcx.shape[1] // 3
    _need(state, "conv state", torch.float32, (None, K - 1, D))
    _check(_fn("shortconv", "zk_conv_state_update")(_ptr(bcx), _ptr(state), _ptr(cu_q), _ptr(seq_slot), n_seqs, D, K,
                                                    state.stride(0), interleave, dtype_code(bcx.dtype), _stream()),
           "conv_state_update")


def conv_decode(bcx, state, w, bias, seq_slot, interleave: int = 0) -> torch.Tensor:
    """Single-token step: y and the shifted state in one kernel; row b of bcx is sequence b."""
    _need(bcx, "bcx", (torch.float32, torch.bfloat16), (None, None))
    n, three_d = bcx.shape
    D = three_d // 3
    _need(w, "conv weight", torch.float32, (None, D))
    K = w.shape[0]
    _need(state, "conv state", torch.float32, (None, K - 1, D))
    if bias is not None:
        _need(bias, "conv bias", torch.float32, (D,))
    _need(seq_slot, "seq_slot", torch.int32)
    y = torch.empty((n, D), dtype=bcx.dtype, device=bcx.device)
    _check(_fn("shortconv", "zk_conv_decode")(_ptr(bcx), _ptr(state), _ptr(w), _ptr(bias), _ptr(seq_slot), _ptr(y), n,
                                              D, K, state.stride(0), interleave, dtype_code(bcx.dtype), _stream()),
           "conv_decode")
    return y


def moe_gather(x: torch.Tensor, row_token: torch.Tensor) -> torch.Tensor:
    """xg[r] = x[row_token[r]] (zeros where row_token[r] < 0): rows in the order a grouped contraction wants them."""
    _need(x, "x", (torch.float32, torch.bfloat16), (None, None))
    _need(row_token, "row_token", torch.int32)
    xg = torch.empty((row_token.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(_fn("moe", "zk_moe_gather")(_ptr(x), _ptr(row_token), _ptr(xg), row_token.numel(), x.shape[1],
                                       dtype_code(x.dtype), _stream()), "moe_gather")
    return xg


def moe_combine(y: torch.Tensor, pair_row: torch.Tensor, top: int, out: torch.Tensor, accumulate: bool = False,
                weights: Optional[torch.Tensor] = None, identity_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] (+)= sum_k weights[t, k] * y[pair_row[t * top + k]] (weights float32 [n, top]; without them 1/top
    each), float32, added in the order of k.  A pair whose row is negative stands for an identity expert: its term is
    identity_rows[t] (the rows the experts read, [n, D] in a run dtype)."""
    _need(y, "y", torch.float32, (None, None))
    _need(out, "out", torch.float32, (None, y.shape[1]))
    _need(pair_row, "pair_row", torch.int32, (out.shape[0] * top,))
    if weights is not None:
        _need(weights, "weights", torch.float32, (out.shape[0], top))
    if identity_rows is not None:
        _need(identity_rows, "identity_rows", (torch.float32, torch.bfloat16), (out.shape[0], y.shape[1]))
    _check(_fn("moe", "zk_moe_combine")(_ptr(y), _ptr(pair_row), _ptr(out), out.shape[0], y.shape[1], top,
                                        1 if accumulate else 0, _ptr(weights), _ptr(identity_rows),
                                        dtype_code(identity_rows.dtype) if identity_rows is not None else F32, _stream()),
           "moe_combine")
    return out


def moe_router(x: torch.Tensor, w_router: torch.Tensor, top: int,
               correction: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """(experts int32 [n, top], weights float32 [n, top]) of every row of x [n, D] (run dtype): logits W x in
    float32 (w_router float32 [E, D]), softmax over all E experts, the `top` largest scores (of equal ones the
    lower index), each divided by the sum of the chosen (+ 1e-20).  `correction` float32 [E]: the choice goes by
    score + correction, the weights are made of the scores alone."""
    _need(x, "x", (torch.float32, torch.bfloat16), (None, None))
    n, D = x.shape
    _need(w_router, "w_router", torch.float32, (None, D))
    E = w_router.shape[0]
    if correction is not None:
        _need(correction, "correction", torch.float32, (E,))
    if not 0 < top <= E:
        raise KernelError(f"moe_router: {top} experts per token out of {E}")
    ids = torch.empty((n, top), dtype=torch.int32, device=x.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=x.device)
    _check(_fn("moe", "zk_moe_router")(_ptr(x), _ptr(w_router), _ptr(ids), _ptr(wts), n, D, E, top, dtype_code(x.dtype),
                                       _ptr(correction), _stream()), "moe_router")
    return ids, wts


def moe_expert_rows(route_ids: torch.Tensor, n_experts: int, tile: int,
                    n_identity: int = 0) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The (token, k) pairs of route_ids [n, top] (int32, device) sorted by expert on the device, every expert's rows
    padded to whole tiles: (row_token [cap] with -1 for padding rows, pair_row [n * top], tile_group [cap / tile]),
    cap = the most rows any choice can need.  Tiles behind the last expert's hold padding rows only.  Ids n_experts ..
    n_experts + n_identity - 1 name identity experts: such a pair gets no row (pair_row -1)."""
    _need(route_ids, "route_ids", torch.int32, (None, None))
    n, top = route_ids.shape
    P = n * top
    cap = (P // tile + n_experts) * tile
    words = torch.empty(cap + P + cap // tile, dtype=torch.int32, device=route_ids.device)
    row_token, pair_row, tile_group = words[:cap], words[cap:cap + P], words[cap + P:]
    _check(_fn("moe", "zk_moe_expert_rows")(_ptr(route_ids), P, n_experts, top, tile, cap, _ptr(row_token), _ptr(pair_row),
                                            _ptr(tile_group), int(n_identity), _stream()), "moe_expert_rows")
    return row_token, pair_row, tile_group


def moe_routed(x: torch.Tensor, route_ids: torch.Tensor, route_w: torch.Tensor, w_gate_up: torch.Tensor, interleave: int,
               w_down: torch.Tensor, status: torch.Tensor, out: Optional[torch.Tensor] = None,
               accumulate: bool = False, n_identity: int = 0) -> torch.Tensor:
    """y[t] = sum_k route_w[t, k] * W_down[e] (silu(W_gate[e] x_t) * (W_up[e] x_t)), e = route_ids[t, k], added in
    the order of k.  Tensors as in `moe_table`.  Ids E .. E + n_identity - 1 name identity experts, whose term is
    route_w[t, k] * x_t."""
    _need(x, "x", (torch.float32, torch.bfloat16), (None, None))
    n, D = x.shape
    _need(route_ids, "route_ids", torch.int32, (n, None))
    top = route_ids.shape[1]
    _need(route_w, "route_w", torch.float32, (n, top))
    _need(w_gate_up, "w_gate_up", x.dtype, (None, None, D))
    E, F = w_gate_up.shape[0], w_gate_up.shape[1] // 2
    _need(w_down, "w_down", x.dtype, (E, D, F))
    if out is None:
        if accumulate:
            raise KernelError("moe_routed: accumulate needs an output tensor")
        out = torch.empty((n, D), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, (n, D))
    h = torch.empty((n, top, F), dtype=x.dtype, device=x.device)
    _check(_fn("moe", "zk_moe_routed")(_ptr(x), _ptr(route_ids), _ptr(route_w), _ptr(w_gate_up), int(interleave), _ptr(w_down),
                                       _ptr(h), _ptr(out), n, D, F, top, E, 1 if accumulate else 0, dtype_code(x.dtype),
                                       _ptr(status), int(n_identity), _stream()), "moe_routed")
    return out


# ------------------------------------------------------------------------------- one latent vector per token

def latent_prepare(q: torch.Tensor, q_full: torch.Tensor, dkv: torch.Tensor, c_weight: torch.Tensor, inv_freq: torch.Tensor,
                   cache: torch.Tensor, tok_seq, tok_pos, seq_slot, page_table, n_heads: int, dim: int, rot_dim: int,
                   rank: int, eps: float, status, write_kv: bool = True, c_out: Optional[torch.Tensor] = None) -> None:
    """For attention over one latent row per token.  q [n, H * (dim + rot_dim)] (run dtype) as projected; the rotated
    part of every head goes, rotated by the token's position, to q_full[:, h, rank : rank + rot_dim] (q_full
    [n, H * (rank + rot_dim)]).  dkv float32 [n, >= rank + rot_dim] (a view of wider rows is fine): the token's
    cache row becomes [rms(dkv[:rank]) * c_weight | rotated dkv[rank : rank + rot_dim]]; cache is one layer's
    [pages, 1, page_size, rank + rot_dim].  q_full None: the queries are left alone.  c_out [n, rank] (run dtype):
    also receives the normalised latents, packed."""
    _need(q, "q", (torch.float32, torch.bfloat16), (None, n_heads * (dim + rot_dim)))
    n = q.shape[0]
    if q_full is not None:
        _need(q_full, "q_full", q.dtype, (n, n_heads * (rank + rot_dim)))
    if c_out is not None:
        _need(c_out, "c_out", q.dtype, (n, rank))
    _need(dkv, "dkv", torch.float32, (n, None), contiguous=False)
    if dkv.shape[1] < rank + rot_dim or dkv.stride(1) != 1:
        raise KernelError(f"latent_prepare: dkv {tuple(dkv.shape)} holds no {rank} + {rot_dim} values per row")
    _need(c_weight, "latent norm weight", torch.float32, (rank,))
    _need(inv_freq, "inv_freq", torch.float32, (rot_dim // 2,))
    _need(cache, "cache", q.dtype, (None, 1, None, rank + rot_dim))
    _need(page_table, "page_table", torch.int32, (None, None))
    _check(_fn("latent", "zk_latent_prepare")(
        _ptr(q), _ptr(q_full), _ptr(dkv), dkv.stride(0), _ptr(c_weight), _ptr(inv_freq), _ptr(cache), _ptr(tok_seq),
        _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, dim, rot_dim, rank, eps,
        cache.shape[2], 1 if write_kv else 0, dtype_code(q.dtype), _ptr(status), _ptr(c_out), _stream()), "latent_prepare")


def latent_pack(q: torch.Tensor, kvx: torch.Tensor, dkv: Optional[torch.Tensor], inv_freq: torch.Tensor, tok_pos, kv_seq, kv_pos,
                seq_page0: torch.Tensor, n_pages: int, page_size: int, n_heads: int, dim: int, rot_dim: int, value_dim: int,
                rank: int, key_width: int, value_width: int, cache: Optional[torch.Tensor] = None, seq_slot=None,
                page_table=None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Queries, keys and values of a prompt step, for attention over rows that the step lays out itself.
    q [n, H * (dim + rot_dim)] as projected, tok_pos [n] the step tokens' positions; kvx [m, H * dim + H * value_dim]:
    every head's expanded unrotated keys, then every head's values, of the m key/value tokens (kv_seq[j], kv_pos[j]):
    the step's own tokens when its sequences start at position 0 (then dkv float32 [m, >= rank + rot_dim] holds the
    shared key part before rotation in its entries rank..), or every position of the step's sequences (then `cache`
    [pages, 1, page_size, rank + rot_dim] with `seq_slot` and `page_table` holds it, already rotated).  Returns q_pad
    [n, H * key_width] = [q_h[:dim] | rot(q_h[dim:]) | 0], k_rows [n_pages, H, page_size, key_width] = [k_h | rot(k_rot)
    | 0] and v_rows [n_pages, H, page_size, value_width] = [v_h | 0], a token of sequence b at position pos in page
    seq_page0[b] + pos // page_size."""
    _need(q, "q", (torch.float32, torch.bfloat16), (None, n_heads * (dim + rot_dim)))
    n = q.shape[0]
    _need(kvx, "kvx", q.dtype, (None, n_heads * (dim + value_dim)))
    m = kvx.shape[0]
    ld_dkv = 0
    if cache is None:
        _need(dkv, "dkv", torch.float32, (m, None), contiguous=False)
        if dkv.shape[1] < rank + rot_dim or dkv.stride(1) != 1:
            raise KernelError(f"latent_pack: dkv {tuple(dkv.shape)} holds no {rank} + {rot_dim} values per row")
        ld_dkv = dkv.stride(0)
    else:
        _need(cache, "cache", q.dtype, (None, 1, page_size, rank + rot_dim))
        _need(page_table, "page_table", torch.int32, (None, None))
    _need(inv_freq, "inv_freq", torch.float32, (rot_dim // 2,))
    _need(seq_page0, "seq_page0", torch.int32, (None,))
    _need(kv_seq, "kv_seq", torch.int32, (m,))
    _need(kv_pos, "kv_pos", torch.int32, (m,))
    q_pad = torch.empty((n, n_heads * key_width), dtype=q.dtype, device=q.device)
    k_rows = torch.empty((n_pages, n_heads, page_size, key_width), dtype=q.dtype, device=q.device)
    v_rows = torch.empty((n_pages, n_heads, page_size, value_width), dtype=q.dtype, device=q.device)
    _check(_fn("latent", "zk_latent_pack")(
        _ptr(q), _ptr(kvx), kvx.stride(0), _ptr(dkv) if cache is None else None, ld_dkv, _ptr(inv_freq), _ptr(q_pad),
        _ptr(k_rows), _ptr(v_rows), _ptr(tok_pos), _ptr(kv_seq), _ptr(kv_pos), _ptr(seq_page0), n, m, n_heads, dim, rot_dim,
        value_dim, rank, key_width, value_width, page_size, _ptr(cache), _ptr(seq_slot) if cache is not None else None,
        _ptr(page_table) if cache is not None else None, page_table.stride(0) if cache is not None else 0,
        dtype_code(q.dtype), _stream()), "latent_pack")
    return q_pad, k_rows, v_rows


def latent_gather(cache: torch.Tensor, kv_seq, kv_pos, seq_slot, page_table, rank: int) -> torch.Tensor:
    """c_all [m, rank]: the first `rank` entries of the cache rows of the tokens (kv_seq[j], kv_pos[j]); cache
    [pages, 1, page_size, W]."""
    _need(cache, "cache", (torch.float32, torch.bfloat16), (None, 1, None, None))
    _need(kv_seq, "kv_seq", torch.int32, (None,))
    m = kv_seq.numel()
    _need(kv_pos, "kv_pos", torch.int32, (m,))
    _need(page_table, "page_table", torch.int32, (None, None))
    if rank > cache.shape[3]:
        raise KernelError(f"latent_gather: rows of {cache.shape[3]} values hold no {rank}")
    c_all = torch.empty((m, rank), dtype=cache.dtype, device=cache.device)
    _check(_fn("latent", "zk_latent_gather")(_ptr(cache), _ptr(c_all), _ptr(kv_seq), _ptr(kv_pos), _ptr(seq_slot),
                                             _ptr(page_table), page_table.stride(0), m, rank, cache.shape[3], cache.shape[2],
                                             dtype_code(cache.dtype), _stream()), "latent_gather")
    return c_all


def head_gemm(a: torch.Tensor, a_head: int, w: torch.Tensor, out: torch.Tensor, o_head: int,
              gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t, h * o_head + n] = sum_k a[t, h * a_head + k] * w[h, n, k] for every head h, times
    sigmoid(gate[t, h]) if `gate` (float32 [tokens, >= H], may be a view of wider rows) is given.
    a [tokens, >= H * a_head], out [tokens, >= H * o_head] in the run dtype; w [H, N, K] contiguous, K <= a_head,
    N <= o_head."""
    _need(w, "w", (torch.float32, torch.bfloat16), (None, None, None))
    H, N, K = w.shape
    _need(a, "a", w.dtype, (None, None))
    _need(out, "out", w.dtype, (a.shape[0], None))
    if K > a_head or N > o_head or a.shape[1] < H * a_head or out.shape[1] < H * o_head:
        raise KernelError(f"head_gemm: a {tuple(a.shape)} / w {tuple(w.shape)} / out {tuple(out.shape)} do not fit heads "
                          f"of {a_head} inputs and {o_head} outputs")
    ld_gate = 0
    if gate is not None:
        _need(gate, "gate", torch.float32, (a.shape[0], None), contiguous=False)
        if gate.shape[1] < H or gate.stride(1) != 1:
            raise KernelError(f"head_gemm: gate {tuple(gate.shape)} holds no {H} values per row")
        ld_gate = gate.stride(0)
    _check(_fn("latent", "zk_head_gemm")(_ptr(a), a.stride(0), a_head, _ptr(w), _ptr(out), out.stride(0), o_head, _ptr(gate),
                                         ld_gate, a.shape[0], H, N, K, dtype_code(w.dtype), _stream()), "head_gemm")
    return out


# ------------------------------------------------------------------------------- attention

def attn_rows_per_block() -> int:
    return _constant("attention", "zk_attn_rows_per_block")


def attn_max_head_dim() -> int:
    return _constant("attention", "zk_attn_max_head_dim")


def qk_prepare(qkv, k_cache, v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos, seq_slot, page_table, n_heads: int,
               n_kv: int, head_dim: int, n_rot: int, interleaved: bool, eps: float, status, write_kv: bool = True,
               value_dim: Optional[int] = None, unit_norm_after: bool = False,
               query_temperature: Optional[tuple] = None):
    """Per-head RMSNorm of q and k (if weights are given), rotary encoding (if `inv_freq` is
    given), then with `unit_norm_after` q and k heads divided by their root mean square (no weight);
    q out as [n, H*hd], and k, v written to their pages.  k_cache is one layer's
    [pages, Hkv, page_size, hd], v_cache [pages, Hkv, page_size, value_dim (default hd)].
    `query_temperature` = (coef, every): the query at position p is multiplied, last of all, by
    1 + coef * ln(floor((p + 1) / every) + 1)."""
    qt_coef, qt_every = (float(query_temperature[0]), int(query_temperature[1])) if query_temperature else (0.0, 0)
    vd = head_dim if value_dim is None else int(value_dim)
    _need(qkv, "qkv", (torch.float32, torch.bfloat16), (None, (n_heads + n_kv) * head_dim + n_kv * vd))
    n = qkv.shape[0]
    _need(k_cache, "k_cache", qkv.dtype, (None, n_kv, None, head_dim))
    _need(v_cache, "v_cache", qkv.dtype, (None, n_kv, None, vd))
    page_size = k_cache.shape[2]
    if head_dim > attn_max_head_dim() or vd > attn_max_head_dim() or n_rot % 2 or n_rot > head_dim:
        raise KernelError(f"qk_prepare: head_dim {head_dim} and value_dim {vd} must be <= {attn_max_head_dim()}, "
                          f"the rotated width {n_rot} even and <= head_dim")
    for wt, nm in ((q_w, "q norm weight"), (k_w, "k norm weight")):
        if wt is not None:
            _need(wt, nm, torch.float32, (head_dim,))
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, (n_rot // 2,))
    _need(page_table, "page_table", torch.int32, (None, None))
    q = torch.empty((n, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    _check(_fn("attention", "zk_qk_prepare")(
        _ptr(qkv), _ptr(q), None, _ptr(k_cache), _ptr(v_cache), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), _ptr(tok_seq),
        _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, n_rot,
        1 if interleaved else 0, eps, page_size, 1 if write_kv else 0, dtype_code(qkv.dtype), _ptr(status), vd,
        1 if unit_norm_after else 0, qt_coef, qt_every, _stream()),
        "qk_prepare")
    return q


def qk_prepare_span(qkv, k_cache, v_cache, q_w, k_w, tok_seq, tok_pos, seq_slot, page_table, n_heads: int, n_kv: int,
                    head_dim: int, value_dim: int, eps: float, status, write_kv: bool = True,
                    inv_freq: Optional[torch.Tensor] = None, n_rot: int = 0) -> torch.Tensor:
    """RMSNorm of q over all its heads at once (weight [H*hd], or None) and of k likewise ([Hkv*hd]); with
    `inv_freq` [n_rot / 2] the first n_rot entries of every q and k head are then rotated by the token's position
    (entry i paired with entry i + n_rot/2); q out as [n, H*hd]; k and v (value_dim wide) written to their pages.
    A row of qkv holds [q | k | v], or q alone with write_kv False (the caches are then only needed for their sizes)."""
    qd, kd, vd = n_heads * head_dim, n_kv * head_dim, n_kv * value_dim
    _need(qkv, "qkv", (torch.float32, torch.bfloat16), (None, qd + (kd + vd if write_kv else 0)))
    n = qkv.shape[0]
    _need(k_cache, "k_cache", qkv.dtype, (None, n_kv, None, head_dim))
    _need(v_cache, "v_cache", qkv.dtype, (None, n_kv, None, value_dim))
    if q_w is not None:
        _need(q_w, "q norm weight", torch.float32, (qd,))
    if k_w is not None:
        _need(k_w, "k norm weight", torch.float32, (kd,))
    _need(page_table, "page_table", torch.int32, (None, None))
    if inv_freq is not None:
        if n_rot <= 0 or n_rot % 2 or n_rot > head_dim:
            raise KernelError(f"qk_prepare_span: the rotated width {n_rot} must be even and at most head_dim {head_dim}")
        _need(inv_freq, "inv_freq", torch.float32, (n_rot // 2,))
    q = torch.empty((n, qd), dtype=qkv.dtype, device=qkv.device)
    _check(_fn("attention", "zk_qk_prepare_span")(
        _ptr(qkv), qkv.stride(0), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(q_w), _ptr(k_w), _ptr(tok_seq),
        _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, value_dim,
        eps, k_cache.shape[2], 1 if write_kv else 0, dtype_code(qkv.dtype), _ptr(status), _ptr(inv_freq), int(n_rot),
        _stream()), "qk_prepare_span")
    return q


def qk_normed(qkv, q_w, k_w, n_heads: int, n_kv: int, head_dim: int, eps: float, tok_pos, status) -> torch.Tensor:
    """Per-head RMSNorm of the q and k heads of qkv [n, (H + 2 Hkv) * hd] into a new tensor of
    the same shape (v copied); no rotation, no cache write."""
    _need(qkv, "qkv", (torch.float32, torch.bfloat16), (None, (n_heads + 2 * n_kv) * head_dim))
    if head_dim % 2 or head_dim > attn_max_head_dim():
        raise KernelError(f"qk_normed: head_dim {head_dim} must be even and <= {attn_max_head_dim()}")
    for wt, nm in ((q_w, "q norm weight"), (k_w, "k norm weight")):
        if wt is not None:
            _need(wt, nm, torch.float32, (head_dim,))
    dense = torch.empty_like(qkv)
    _check(_fn("attention", "zk_qk_prepare")(
        _ptr(qkv), None, _ptr(dense), None, None, _ptr(q_w), _ptr(k_w), None, None, _ptr(tok_pos), None, None, 0,
        qkv.shape[0], n_heads, n_kv, head_dim, 0, 0, eps, 1, 0, dtype_code(qkv.dtype), _ptr(status), head_dim, 0, 0.0, 0,
        _stream()),
        "qk_normed")
    return dense


def attn_tile_shape(n_heads: int, n_kv: int) -> tuple[int, int]:
    """(tokens per query tile, heads of a KV group per block) for these head counts."""
    rows = attn_rows_per_block()
    gc = min(n_heads // n_kv, rows)
    return max(1, rows // gc), gc


def _may_take(lib: str, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """The sizes a specialised attention library can take at all, known here so that a model it
    cannot serve never has it compiled; the library's own `*_takes` has the last word."""
    group = n_heads // n_kv
    if lib == "attention_decode":
        return head_dim in (32, 64, 96, 128) and group <= 8 and page_size % 32 == 0
    if lib == "attention_decode_tc":
        return head_dim in (64, 128) and group <= 16 and page_size % 64 == 0
    if lib == "attention_prefill":
        return head_dim in (64, 128) and page_size % 64 == 0
    if lib == "attention_prefill_tc5":
        return head_dim == 64 and page_size % 64 == 0
    raise KeyError(lib)


def _takes(lib: str, fn: str, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    return _may_take(lib, n_heads, n_kv, head_dim, page_size) and bool(_fn(lib, fn)(n_heads, n_kv, head_dim, page_size))


@functools.lru_cache(maxsize=None)      # a pure function of sizes, asked for by every attention layer of every step
def attention_plan(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int, page_size: int,
                   single_token: bool, window: int = 0, value_dim: Optional[int] = None,
                   biased: bool = False, talking: bool = False, extras: bool = False,
                   kept_or_sink: bool = False, capped: bool = False) -> tuple[str, int]:
    """Which attention kernel runs for these sizes and how many tokens its query tiles hold:
    ("single_token_tc" | "single_token" | "prompt_tc5" | "prompt_tc" | "general", tokens per tile).
    Values of another width than the keys go to the general kernel; a distance bias on the scores is
    taken by the general kernel and the two mma.sync kernels ("prompt_tc", "single_token_tc"); weights that
    are mixed across the heads after the softmax (`talking`) by those three and the tcgen05 prompt kernel.
    `kept_or_sink`: kept first tokens or a sink in the softmax, which the general kernel and the two mma.sync kernels
    take (without a bias or mixed weights); `extras`: values read from the key rows, the general kernel's; `capped`:
    scores through a tanh cap, which the same three kernels take."""
    same_width = value_dim is None or value_dim == head_dim
    if extras or (kept_or_sink and (biased or talking)):
        return "general", attn_tile_shape(n_heads, n_kv)[0]
    if same_width and dtype == torch.bfloat16 and n_heads % n_kv == 0:
        if (not single_token and window <= 0 and not biased and not kept_or_sink and not capped and _may_take("attention_prefill_tc5", n_heads, n_kv, head_dim, page_size)
                and _fn("attention_prefill_tc5", "zk_attn_prefill_tc5_takes")(n_heads, n_kv, head_dim, page_size, window)):
            return "prompt_tc5", _fn("attention_prefill_tc5", "zk_attn_prefill_tc5_tile_tokens")(n_heads, n_kv)
        if single_token and _takes("attention_decode_tc", "zk_attn_decode_tc_takes", n_heads, n_kv, head_dim, page_size):
            return "single_token_tc", 1
        if (single_token and not biased and not talking and not kept_or_sink and not capped
                and _takes("attention_decode", "zk_attn_decode_takes", n_heads, n_kv, head_dim, page_size)):
            return "single_token", 1
        if not single_token and _takes("attention_prefill", "zk_attn_prefill_takes", n_heads, n_kv, head_dim, page_size):
            return "prompt_tc", _fn("attention_prefill", "zk_attn_prefill_tile_tokens")(n_heads, n_kv)
    return "general", attn_tile_shape(n_heads, n_kv)[0]


def attention(q, k_cache, v_cache, tile_seq, tile_q0, cu_q, seq_start, seq_slot, page_table, n_heads: int, n_kv: int,
              head_dim: int, scale: float, window: int = 0, num_splits: int = 1, split_keys: int = 0,
              single_token: bool = False, kind: Optional[str] = None, value_dim: Optional[int] = None,
              bias: Optional[tuple] = None, talk: Optional[torch.Tensor] = None, keep_first: int = 0,
              sink: Optional[torch.Tensor] = None, values_in_keys: bool = False, softcap: float = 0.0) -> torch.Tensor:
    """Causal grouped-query attention of a packed batch against the paged cache.
    `keep_first`: with a window, the first so many positions of a sequence stay visible to every later query.
    `sink` float32 [H]: exp(sink_h) is one more term of head h's softmax denominator (no key, no value, not scaled).
    `values_in_keys`: there is no value cache; a value row is the first `value_dim` entries of the key row.
    `softcap` > 0: a scaled score s becomes softcap * tanh(s / softcap) (the general kernel's and the two mma.sync kernels').
    The last is the general kernel's; the first two also the two mma.sync kernels' ("prompt_tc", "single_token_tc").  With
    num_splits > 1 the keys are cut at multiples of `split_keys` and merged afterwards.
    `single_token` says that every sequence brings exactly one query (row b = sequence b); the
    bfloat16 kernels for that case are used when they take the sizes.  `kind` names the kernel as
    `attention_plan` chose it (the tile table must then have that plan's tokens per tile);
    without it the general kernel or the single-token kernel runs.  `value_dim`: width of a value
    row if it is not head_dim.  `bias` = (r1, r2), float32 [H] each: r1_h * ln(1 + r2_h * (i - j)) is taken
    off the scaled score of query position i and key position j.  Both are the general kernel's.
    `talk` float32 [H, H]: after the softmax head h's weights become sum_g talk[h, g] * (head g's weights), and
    head h applies them to the values of its own key/value head (every kernel but the one-lane-per-key one:
    every head's weights meet every key/value head's values, and a merge kernel mixes the results)."""
    _need(q, "q", (torch.float32, torch.bfloat16), (None, n_heads * head_dim))
    n = q.shape[0]
    vd = head_dim if value_dim is None else int(value_dim)
    _need(k_cache, "k_cache", q.dtype, (None, n_kv, None, head_dim))
    if values_in_keys:
        if vd > head_dim or talk is not None:
            raise KernelError("attention: values read from the key rows are at most as wide as the keys, and no weights "
                              "are mixed across heads")
        v_cache = k_cache
    else:
        _need(v_cache, "v_cache", q.dtype, (None, n_kv, None, vd))
    kept_or_sink = keep_first > 0 or sink is not None
    if values_in_keys and kind not in (None, "general"):
        raise KernelError(f"attention: the '{kind}' kernel takes no values in the key rows")
    if kept_or_sink and kind not in (None, "general", "prompt_tc", "single_token_tc"):
        raise KernelError(f"attention: the '{kind}' kernel takes no kept first tokens or sink")
    extras = values_in_keys or (kept_or_sink and kind in (None, "general"))
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    if bias is not None:
        for b, nm in zip(bias, ("bias r1", "bias r2")):
            _need(b, nm, torch.float32, (n_heads,))
    if talk is not None:
        _need(talk, "talk", torch.float32, (n_heads, n_heads))
        if kind not in (None, "general", "prompt_tc5", "prompt_tc", "single_token_tc"):
            raise KernelError(f"attention: the '{kind}' kernel mixes no weights across heads")
    softcap = float(softcap or 0.0)
    if softcap > 0 and kind not in (None, "general", "prompt_tc", "single_token_tc"):
        raise KernelError(f"attention: the '{kind}' kernel caps no scores")
    if vd != head_dim and kind not in (None, "general"):
        raise KernelError(f"attention: the '{kind}' kernel takes no value width of its own")
    if bias is not None and kind not in (None, "general", "prompt_tc", "single_token_tc"):
        raise KernelError(f"attention: the '{kind}' kernel takes no distance bias")
    r1, r2 = (_ptr(bias[0]), _ptr(bias[1])) if bias is not None else (None, None)
    page_size = k_cache.shape[2]
    if n_heads % n_kv:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv} KV heads")
    if head_dim > attn_max_head_dim():
        raise KernelError(f"attention: head_dim {head_dim} exceeds {attn_max_head_dim()}")
    if vd > attn_max_head_dim():
        raise KernelError(f"attention: value_dim {vd} exceeds {attn_max_head_dim()}")
    bq, gc = attn_tile_shape(n_heads, n_kv)
    n_tiles = tile_seq.numel()
    out = torch.empty((n, n_heads * vd), dtype=q.dtype, device=q.device)
    if (vd != head_dim or extras or (talk is not None and kind != "single_token_tc")
            or (bias is not None and kind != "single_token_tc")):
        single_token = False        # the general kernel runs single tokens as tiles of one query
    part_o = part_ml = None
    value_heads = n_kv if talk is not None else 1
    if num_splits > 1 or talk is not None:
        part_o = torch.empty((num_splits, n * n_heads * value_heads, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((num_splits, n * n_heads * value_heads, 2), dtype=torch.float32, device=q.device)
    if kind == "prompt_tc5":
        if (q.dtype != torch.bfloat16 or window > 0 or not k_cache.is_contiguous() or not v_cache.is_contiguous()
                or not q.is_contiguous()
                or not _fn("attention_prefill_tc5", "zk_attn_prefill_tc5_takes")(n_heads, n_kv, head_dim, page_size, window)):
            raise KernelError("attention: the tcgen05 prompt kernel does not take these sizes")
        _check(_fn("attention_prefill_tc5", "zk_attn_prefill_tc5")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq), _ptr(tile_q0), _ptr(cu_q),
            _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n_tiles, n, k_cache.shape[0],
            n_heads, n_kv, head_dim, page_size, scale, _ptr(status_word(q.device)),
            _ptr(part_o) if talk is not None else None, _ptr(part_ml) if talk is not None else None, _stream()),
            "attention (prompt, tcgen05)")
        return out if talk is None else _merge_talk(part_o, part_ml, talk, out, n, n_heads, n_kv, vd, 1)
    if kind == "prompt_tc":
        if q.dtype != torch.bfloat16 or not _takes("attention_prefill", "zk_attn_prefill_takes", n_heads, n_kv, head_dim,
                                                   page_size):
            raise KernelError("attention: the tensor-core prompt kernel does not take these sizes")
        _check(_fn("attention_prefill", "zk_attn_prefill")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq), _ptr(tile_q0), _ptr(cu_q),
            _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n_tiles, n_heads, n_kv, head_dim,
            head_dim, page_size, window, scale, r1, r2, _ptr(part_o) if talk is not None else None,
            _ptr(part_ml) if talk is not None else None, int(keep_first), _ptr(sink), softcap, _stream()),
            "attention (prompt, tensor cores)")
        return out if talk is None else _merge_talk(part_o, part_ml, talk, out, n, n_heads, n_kv, vd, 1)
    if (single_token and kind in (None, "single_token_tc") and q.dtype == torch.bfloat16
            and _takes("attention_decode_tc", "zk_attn_decode_tc_takes", n_heads, n_kv, head_dim, page_size)):
        _check(_fn("attention_decode_tc", "zk_attn_decode_tc")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(seq_start),
            _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, page_size, window,
            scale, num_splits, split_keys, r1, r2, 1 if talk is not None else 0, int(keep_first), _ptr(sink), softcap,
            _stream()),
            "attention (single token, tensor cores)")
        if talk is not None:
            return _merge_talk(part_o, part_ml, talk, out, n, n_heads, n_kv, vd, num_splits)
        if num_splits > 1:
            _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, head_dim,
                                                     num_splits, dtype_code(q.dtype), _ptr(sink), n_heads, _stream()), "attention merge")
        return out
    if kind == "single_token_tc":
        raise KernelError("attention: the tensor-core single-token kernel does not take these sizes")
    if (single_token and kind in (None, "single_token") and q.dtype == torch.bfloat16 and softcap <= 0
            and _takes("attention_decode", "zk_attn_decode_takes", n_heads, n_kv, head_dim, page_size)):
        _check(_fn("attention_decode", "zk_attn_decode")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(seq_start),
            _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, page_size, window,
            scale, num_splits, split_keys, _stream()), "attention (single token)")
        if num_splits > 1:
            _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, head_dim,
                                                     num_splits, dtype_code(q.dtype), None, n_heads, _stream()), "attention merge")
        return out
    _check(_fn("attention", "zk_attn_fwd")(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tile_seq), _ptr(tile_q0),
        _ptr(cu_q), _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n_tiles, n, n_heads, n_kv,
        head_dim, page_size, window, scale, bq, gc, num_splits, split_keys, dtype_code(q.dtype), vd, r1, r2,
        1 if talk is not None else 0, int(keep_first), _ptr(sink), 1 if values_in_keys else 0, softcap, _stream()),
        "attention")
    if talk is not None:
        return _merge_talk(part_o, part_ml, talk, out, n, n_heads, n_kv, vd, num_splits)
    if num_splits > 1:
        _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, vd,
                                                 num_splits, dtype_code(q.dtype), _ptr(sink), n_heads, _stream()),
               "attention merge")
    return out


def attention_step_rows_takes(dtype: torch.dtype, head_dim: int, value_dim: int, page_size: int) -> bool:
    """Whether `attention_step_rows` runs for these widths."""
    return (dtype == torch.bfloat16 and (head_dim, value_dim) in ((64, 64), (128, 128), (128, 64))
            and _may_take("attention_prefill", 1, 1, head_dim, page_size))


def attention_step_rows_tile_tokens(n_heads: int) -> int:
    return _fn("attention_prefill", "zk_attn_prefill_tile_tokens")(n_heads, n_heads)


def attention_step_rows(q, k_rows, v_rows, tile_seq, tile_q0, cu_q, seq_start, seq_page0, n_heads: int, scale: float,
                        sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of a prompt step over keys and values that the step itself laid out (no cache): every head
    has keys and values of its own, k_rows [pages, H, page_size, head_dim] and v_rows [pages, H, page_size,
    value_dim], sequence b's position pos at row pos % page_size of page seq_page0[b] + pos // page_size.
    q [n, H * head_dim]; returns [n, H * value_dim].  bfloat16 on the tensor-core prompt kernel; the tiles hold
    `attention_step_rows_tile_tokens` tokens.  `sink` float32 [H]: one more term of every head's softmax denominator."""
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    _need(k_rows, "k_rows", torch.bfloat16, (None, n_heads, None, None))
    hd, page_size = k_rows.shape[3], k_rows.shape[2]
    _need(v_rows, "v_rows", torch.bfloat16, (k_rows.shape[0], n_heads, page_size, None))
    vd = v_rows.shape[3]
    _need(q, "q", torch.bfloat16, (None, n_heads * hd))
    if not attention_step_rows_takes(q.dtype, hd, vd, page_size):
        raise KernelError(f"attention over a step's own rows: no kernel for keys of {hd} and values of {vd}")
    n = q.shape[0]
    out = torch.empty((n, n_heads * vd), dtype=q.dtype, device=q.device)
    _check(_fn("attention_prefill", "zk_attn_prefill")(
        _ptr(q), _ptr(k_rows), _ptr(v_rows), _ptr(out), _ptr(tile_seq), _ptr(tile_q0), _ptr(cu_q), _ptr(seq_start),
        _ptr(seq_page0), None, 0, tile_seq.numel(), n_heads, n_heads, hd, vd, page_size, 0, scale, None, None, None, None,
        0, _ptr(sink), 0.0, _stream()), "attention (prompt, a step's own rows)")
    return out


def attention_latent_single_takes(dtype: torch.dtype, n_heads: int, row_dim: int, value_dim: int, page_size: int) -> bool:
    """Whether `attention_latent_single` runs for these sizes (known here, so that a model it cannot serve never has
    the library compiled)."""
    if (dtype != torch.bfloat16 or row_dim % 16 or value_dim % 16 or value_dim > min(row_dim, 512) or row_dim > 768
            or page_size % 64):
        return False
    return bool(_fn("attention_decode_latent", "zk_attn_decode_latent_takes")(n_heads, row_dim, value_dim, page_size))


def attention_latent_single(q, cache, seq_start, seq_slot, page_table, n_heads: int, value_dim: int, scale: float,
                            num_splits: int = 1, split_keys: int = 0, sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Single-token steps of attention over one cached row per token that is key and value at once: q [n, H * W]
    (sequence b's queries in row b), cache [pages, 1, page_size, W], a value = a row's first `value_dim` entries.
    Returns [n, H * value_dim].  bfloat16, on the tensor cores; with num_splits > 1 the keys are cut at multiples of
    `split_keys` and merged afterwards.  `sink` float32 [H]: one more term of every head's softmax denominator, added
    by the merge (which then runs for a single chunk too)."""
    if sink is not None:
        _need(sink, "sink", torch.float32, (n_heads,))
    _need(cache, "cache", torch.bfloat16, (None, 1, None, None))
    page_size, W = cache.shape[2], cache.shape[3]
    _need(q, "q", torch.bfloat16, (None, n_heads * W))
    n = q.shape[0]
    if not attention_latent_single_takes(q.dtype, n_heads, W, value_dim, page_size):
        raise KernelError(f"attention over latent rows: no kernel for rows of {W} with values of {value_dim}")
    out = torch.empty((n, n_heads * value_dim), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if num_splits > 1 or sink is not None:
        part_o = torch.empty((num_splits, n * n_heads, value_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((num_splits, n * n_heads, 2), dtype=torch.float32, device=q.device)
    _check(_fn("attention_decode_latent", "zk_attn_decode_latent")(
        _ptr(q), _ptr(cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(seq_start), _ptr(seq_slot), _ptr(page_table),
        page_table.stride(0), n, n_heads, W, value_dim, page_size, scale, num_splits, split_keys, _stream()),
        "attention (single token, latent rows)")
    if part_o is not None:
        _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, value_dim, num_splits,
                                                 dtype_code(q.dtype), _ptr(sink), n_heads, _stream()), "attention merge")
    return out


def _merge_talk(part_o, part_ml, talk, out, n: int, n_heads: int, n_kv: int, vd: int, num_splits: int) -> torch.Tensor:
    """out[t, h] = sum_g talk[h, g] * (head g's weights applied to the values of h's key/value head), from the
    unnormalised sums the attention kernels' cross mode left per (split, token, head, value head)."""
    _check(_fn("attention", "zk_attn_merge_talk")(_ptr(part_o), _ptr(part_ml), _ptr(talk), _ptr(out), n, n_heads, n_kv, vd,
                                                  num_splits, dtype_code(out.dtype), _stream()), "attention merge (mixed heads)")
    return out


# ------------------------------------------------------------------------------- sampling

def apply_penalties(logits, rep_tokens, rep_penalty: float, dry_tokens, dry_pen) -> None:
    """In place: repetition penalty on the listed tokens of each row ([n, R] int32, -1 = none),
    then logits[row, tok] -= pen for the DRY pairs ([n, P] int32 / float32)."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    R = P = 0
    if rep_tokens is not None:
        _need(rep_tokens, "rep_tokens", torch.int32, (n, None))
        R = rep_tokens.shape[1]
    if dry_tokens is not None:
        _need(dry_tokens, "dry_tokens", torch.int32, (n, None))
        P = dry_tokens.shape[1]
        _need(dry_pen, "dry_pen", torch.float32, (n, P))
    _check(_fn("sampling", "zk_apply_penalties")(_ptr(logits), n, V, _ptr(rep_tokens), R, rep_penalty,
                                                 _ptr(dry_tokens), _ptr(dry_pen), P, _stream()), "apply_penalties")


def recent_window() -> int:
    """How many of a request's last tokens the device's window for the repetition penalty holds."""
    return _constant("sampling", "zk_recent_window")


def penalize_recent(logits, recent, seen, req_ids, penalty: float) -> None:
    """In place: the repetition penalty (l > 0 ? l / F : l * F) on every distinct token among the last
    tokens of each row's request.  recent int32 [requests, recent_window()] is a ring per request,
    seen int32 [requests] how many tokens each has had, req_ids int32 [n] the request of each row."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    _need(recent, "recent", torch.int32, (None, recent_window()))
    _need(seen, "seen", torch.int32, (recent.shape[0],))
    _need(req_ids, "req_ids", torch.int32, (n,))
    _check(_fn("sampling", "zk_penalize_recent")(_ptr(logits), n, V, _ptr(recent), _ptr(seen), _ptr(req_ids),
                                                 float(penalty), _stream()), "penalize_recent")


def recent_append(tokens, recent, seen, req_ids) -> None:
    """tokens int32 [n], one per row, enter their requests' rings (see penalize_recent)."""
    n = tokens.shape[0]
    _need(tokens, "tokens", torch.int32, (n,))
    _need(recent, "recent", torch.int32, (None, recent_window()))
    _need(seen, "seen", torch.int32, (recent.shape[0],))
    _need(req_ids, "req_ids", torch.int32, (n,))
    _check(_fn("sampling", "zk_recent_append")(_ptr(tokens), n, _ptr(recent), _ptr(seen), _ptr(req_ids), _stream()),
           "recent_append")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, feed: Optional[torch.Tensor] = None,
           status: Optional[torch.Tensor] = None, ring: Optional[torch.Tensor] = None,
           ring_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Lowest index among the largest logits of each row; int32 [n].  `out` may be given (with
    `status` it has n + 1 words and the last receives the status word's value); `feed` [n] receives
    the same indices (the next step's token slots).  `ring` int32 [slots, n + 1]: the kernel also
    writes the tokens and the status word into slot (ring_pos % slots) and adds one to `ring_pos`
    (one int32 word on the device), so that a step's result stays where it is while later steps run."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    ring_slots = 0
    if ring is not None:
        _need(ring, "ring", torch.int32, (None, n + 1))
        _need(ring_pos, "ring_pos", torch.int32, (1,))
        ring_slots = ring.shape[0]
    if out is None:
        out = torch.empty(n + (1 if status is not None else 0), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (n + (1 if status is not None else 0),))
    if feed is not None:
        _need(feed, "feed", torch.int32, (n,))
    if status is not None:
        _need(status, "status", torch.int32)
    scratch = _argmax_scratch(logits.device, n)
    _check(_fn("sampling", "zk_argmax")(_ptr(logits), n, V, _ptr(out), _ptr(feed), _ptr(status), _ptr(scratch),
                                        _ptr(ring), ring_slots, _ptr(ring_pos), _stream()), "argmax")
    return out


def _argmax_scratch(device, n: int) -> torch.Tensor:
    """Zeroed words in which the blocks of an arg-max meet (n 64-bit keys and a counter) and which the
    kernel leaves zero again; one buffer per device, shared by launches that follow one another."""
    dev = torch.device(device)
    key = ("argmax scratch", dev.index if dev.index is not None else torch.cuda.current_device())
    t = _device_state.get(key)
    if t is None or t.numel() < n + 1:
        t = _device_state[key] = torch.zeros(max(n + 1, 4097), dtype=torch.int64, device=dev)
    return t


def sample(logits, uniforms, temp: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
           xtc_probability: float = 0.0, xtc_threshold: float = 0.1, xtc_min_keep: int = 1, seed: int = 0,
           req_ids: Optional[torch.Tensor] = None, draws: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row after top-k, top-p, min-p, temperature and XTC.  The row's two uniforms in
    [0, 1) are uniforms[row] (float32 [n, 2]), or, with uniforms None, computed on the device as
    sampling.sampler.uniform(seed, req_ids[row], draws[req_ids[row]], 0 and 1): req_ids int32 [n]
    names each row's request (distinct), draws int32 [requests] counts each request's draws so far
    and is advanced by one for the rows' requests."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    if uniforms is not None:
        _need(uniforms, "uniforms", torch.float32, (n, 2))
    else:
        _need(req_ids, "req_ids", torch.int32, (n,))
        _need(draws, "draws", torch.int32, (None,))
    if not temp > 0:
        raise KernelError("sample: temperature must be positive (use argmax for greedy)")
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF          # the 64 bits as a signed value for the C side
    if seed >= 1 << 63:
        seed -= 1 << 64
    _check(_fn("sampling", "zk_sample")(_ptr(logits), n, V, temp, top_k, top_p, min_p, xtc_probability, xtc_threshold,
                                        xtc_min_keep, _ptr(uniforms), seed, _ptr(req_ids),
                                        _ptr(draws), _ptr(out), _stream()), "sample")
    return out


__all__ = [n for n in dir() if not n.startswith("_")] + ["KernelBuildError"]
