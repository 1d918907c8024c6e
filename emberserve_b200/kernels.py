"""Python face of the hand-written CUDA kernels (``csrc/*.cu``), through ctypes.

Every function here takes CUDA tensors, checks what the kernel assumes (device,
contiguity, dtypes) and launches on the current torch stream.  There is no CPU path and
no library fallback: a missing or unbuildable extension, a tensor that is not on the
GPU, or a non-zero status from a launcher raises.

The launchers are plain ``extern "C"`` symbols taking raw pointers, so they are
captured by CUDA graphs like any other launch and allocate nothing themselves.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass

import torch

from emberserve_b200 import build

_ERRORS = {
    1: "unknown element type",
    2: "a size this kernel does not take",
    3: "the CUDA launch failed",
    4: "scratch buffer missing or too small",
    5: "pointer or stride not aligned as the kernel needs",
}


class KernelError(RuntimeError):
    pass


_lib_handle: ctypes.CDLL | None = None


def library() -> ctypes.CDLL:
    """The loaded extension; built on first use.  Raises if it cannot be had."""
    global _lib_handle
    if _lib_handle is None:
        path = build.ensure_built()
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:  # pragma: no cover - depends on the machine
            raise KernelError(f"cannot load the emberserve_b200 CUDA extension {path}: {e}") from e
        _declare(lib)
        _lib_handle = lib
    return _lib_handle


def library_path() -> str:
    library()
    return str(build.ensure_built(verbose=False))


def _declare(lib: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "ems_embedding": [P, I, P, P, P, I, I, F, P],
        "ems_add_rmsnorm": [P, P, P, I, P, I, P, I, I, F, I, P],
        "ems_silu_mul": [P, P, I, I, I, P],
        "ems_rope_table": [P, P, I, I, P],
        "ems_rope_kv_write": [P, I, I, I, I, I, P, P, P, I, P, P, P, I, I, I, P],
        "ems_decode_attention_fused": [P, L, P, P, P, P, I, I, P, P, I, I, I, I, I, F, P, I, I, I, P, L, P],
        "ems_paged_attention": [P, L, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, F, I, I, P, L, I, P],
        "ems_argmax": [P, P, I, I, P, P],
        "ems_repetition_penalty": [P, I, I, P, P, P, P],
        "ems_sample": [P, I, I, P, P, P, P, P, P, P],
        "ems_gemm_smallm": [P, P, P, P, I, I, I, I, P, P, P, P, P, I, I, F, I, I, P],
        "ems_gemm_smallm_gated": [P, P, P, I, I, I, P, I, I, F, I, P],
        "ems_gemm_midm": [P, P, P, P, I, I, I, I, I, P],
        "ems_gemm_midm_max_clusters": [I, I],
        "ems_gemm_large_gated": [P, P, P, I, I, I, I, P],
        "ems_stream_inject": [P, P, P, P, P, I, I, I, P],
        "ems_add_norm_grouped": [P, P, I, I, F, P, P, I, I, F, P, I, P, I, I, I, P],
        "ems_glu_act": [P, L, P, I, I, I, I, F, F, I, P],
        "ems_causal_taps": [P, L, P, I, P, I, P, P, P, P, P, I, I, I, I, I, P],
        "ems_paged_attention_masked": [P, L, P, I, P, P, P, I, I, P, P, I, I, I, I, I, I, I, P, P, L, F, I, I,
                                       P, L, I, I, I, P, I, P, F, P],
        "ems_unary_act": [P, P, I, L, I, P],
        "ems_qk_prep": [P, L, I, I, I, I, I, P, P, P, I, I, I, F, P, P, P, I, I, I, I, I, I, F, P, I, P, P, I, I, P],
        "ems_norm_mean2": [P, P, P, P, I, P, I, I, I, F, P],
        "ems_matrix_recurrence": [P, L, P, L, P, L, I, I, F, P, P, P, P, F, P, P, I, I, P, P, I, I, I, I, I, P, I, P],
        "ems_mlstm_gates": [P, P, P, I, F, P, I, I, P, P, I, I, P, P, P, P],
        "ems_group_norm_gate": [P, P, P, I, P, L, P, I, I, I, I, F, P],
        "ems_rglru_scan": [P, P, P, P, P, I, P, L, I, F, P, P, P, P, I, I, I, I, I, P],
        "ems_latent_prep": [P, I, I, I, I, I, I, P, P, I, F, P, P, P, I, I, P, P, I, I, P, I, P],
        "ems_rope_inplace": [P, I, I, I, I, I, I, I, I, P, P, P],
        "ems_latent_attention": [P, P, I, I, I, P, P, I, I, P, P, P, I, I, I, I, F, I, P, L, I, P],
        "ems_heads_gate": [P, P, I, P, I, I, I, I, P],
        "ems_moe_route": [P, I, I, I, I, P, P, P, P, P, I, I, P, I, P, I, P, F, F, I, P],
        "ems_moe_down_grouped_tc05": [P, P, P, I, I, I, I, P, P],
        "ems_moe_combine_rows": [P, P, P, P, I, I, I, P, P, P, I, P],
        "ems_moe_gather": [P, P, I, I, I, P, P],
        "ems_moe_up_grouped_tc05": [P, P, P, I, I, I, I, P, P, P, I, F, F, P],
        "ems_moe_up": [P, P, I, P, P, I, I, I, I, I, P, I, P, F, F, I, P],
        "ems_moe_down": [P, P, I, P, P, I, I, I, P, I, P],
        "ems_moe_combine": [P, P, P, I, I, I, I, P, P, P, I, P],
        "ems_add_cast": [P, P, P, I, I, I, P],
        "ems_token_gate": [P, P, I, L, I, P, P, P, I, I, I, P],
        "ems_depth_mix": [P, P, I, F, P, P, P, I, L, I, I, I, P],
        "ems_add_scaled_norm2": [P, P, P, F, F, F, P, P, P, I, F, F, P, P, I, I, I, P],
        "ems_stream_norm": [P, P, I, F, F, I, I, P],
        "ems_softcap": [P, L, F, P],
        "ems_delta_recurrence": [P, L, P, L, P, L, P, L, I, I, I, F, F, P, P, P, I, P, P, P, I, I, I, I, I, I, P, P, L, P],
        "ems_ssm_gates": [P, L, I, P, P, I, P, P, I, I, P],
        "ems_gate_group_norm": [P, P, L, I, P, P, L, P, I, P, I, I, I, I, I, F, P],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    lib.ems_gemm_large_gated_supported.argtypes = [I, I, I]
    lib.ems_gemm_large_gated_supported.restype = c_int
    lib.ems_gemm_smallm_status.argtypes = []
    lib.ems_gemm_smallm_status.restype = c_int
    lib.ems_tc_status_clear.argtypes = []
    lib.ems_tc_status_clear.restype = None
    lib.ems_argmax_slices.argtypes = [I, I]
    lib.ems_argmax_slices.restype = c_int
    lib.ems_paged_attention_scratch_bytes.argtypes = [I, I, I, I]
    lib.ems_paged_attention_scratch_bytes.restype = c_longlong
    lib.ems_latent_attention_scratch_bytes.argtypes = [I, I, I, I]
    lib.ems_latent_attention_scratch_bytes.restype = c_longlong
    lib.ems_moe_tile_rows.argtypes = []
    lib.ems_moe_tile_rows.restype = c_int
    lib.ems_delta_work_floats.argtypes = [I, I, I, I, I]
    lib.ems_delta_work_floats.restype = c_longlong


_sm_counts: dict[int, int] = {}
# What a helper assumes where there is no device to ask (the host-logic tests): a B200.
B200_SMS = 148


def sm_count(device: "torch.device | str | None" = None) -> int:
    """Streaming multiprocessors of `device` (asked once per device); the grid-shaping helpers
    (how keys or K are split over blocks) take it from here instead of a constant."""
    dev = torch.device(device) if device is not None else None
    if dev is not None and dev.type != "cuda":
        return B200_SMS
    key = dev.index if dev is not None and dev.index is not None else -1
    n = _sm_counts.get(key)
    if n is None:
        # (the driver is asked here only: a question about the device count at every call is slow
        # and can wait behind other users of the driver)
        if not torch.cuda.is_available():
            return B200_SMS
        idx = key if key >= 0 else torch.cuda.current_device()
        n = _sm_counts[key] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process (eager launches; a CUDA
    graph replay adds what its capture recorded)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'status {code}')}")
    _launches += kernels


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: torch.Tensor | None, name: str = "tensor") -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (emberserve_b200 has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t.data_ptr()


def _i32(t: torch.Tensor | None, name: str) -> int | None:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{name} must be int32, got {t.dtype}")
    return _ptr(t, name)


def _stream() -> int:
    # the raw handle of torch's current stream (the capturing stream inside a graph capture);
    # the public torch.cuda.current_stream() costs tens of microseconds per call
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_stream_objects: dict[tuple[int, int], "torch.cuda.Stream"] = {}


def record_event() -> "torch.cuda.Event":
    """A new event recorded on the current stream.  The stream object is looked up by its raw
    handle and kept: ``torch.cuda.current_stream()`` asks the driver for the device count at every
    call, which is slow and can stall behind other users of the driver."""
    key = (torch._C._cuda_getDevice(), _stream())
    stream = _stream_objects.get(key)
    if stream is None:
        stream = _stream_objects[key] = torch.cuda.current_stream()
    event = torch.cuda.Event()
    event.record(stream)
    return event


# ---------------------------------------------------------------------------------------


def embedding(table: torch.Tensor, tokens: torch.Tensor, residual: torch.Tensor,
              deferred: torch.Tensor | None = None, scale: float = 1.0) -> None:
    """residual[n, :] = float32(table[tokens[n], :]) * scale; a token -(k + 1) reads deferred[k] (a token
    sampled on the device by an earlier kernel of the stream)."""
    n, h = residual.shape
    assert table.shape[1] == h and residual.dtype == torch.float32 and tokens.numel() >= n
    _check(library().ems_embedding(_ptr(table, "table"), _dt(table), _i32(tokens, "tokens"),
                                   None if deferred is None else _i32(deferred, "deferred"),
                                   _ptr(residual, "residual"), n, h, float(scale), _stream()), "embedding")


def add_rmsnorm(delta: torch.Tensor | None, residual: torch.Tensor, weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
                num_rows: int | None = None) -> None:
    """residual += delta (32-bit); out = weight * round(residual * rsqrt(mean(residual^2) + eps)).
    With `rows`, only residual rows rows[0..num_rows) are normalised into out[0..num_rows)
    and the residual is not written."""
    h = residual.shape[-1]
    assert residual.dtype == torch.float32 and weight.numel() == h and out.shape[-1] == h
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape[-1] == h
    n_out = residual.shape[0] if rows is None else (rows.numel() if num_rows is None else num_rows)
    if delta is not None and rows is None:
        assert delta.shape[0] >= n_out
    _check(library().ems_add_rmsnorm(_ptr(delta, "delta"), _ptr(residual, "residual"),
                                     _ptr(weight, "weight"), _dt(weight), _ptr(out, "out"), _dt(out),
                                     _i32(rows, "rows"), n_out, h, float(eps),
                                     0 if rows is not None else 1, _stream()), "add_rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]"""
    n, i = out.shape
    assert gate_up.shape == (n, 2 * i) and gate_up.dtype == out.dtype
    _check(library().ems_silu_mul(_ptr(gate_up, "gate_up"), _ptr(out, "out"), _dt(out), n, i,
                                  _stream()), "silu_mul")


def rope_table(inv_freq: torch.Tensor, max_pos: int) -> torch.Tensor:
    """[max_pos, half, 2] float32 table of (cos, sin) of pos * inv_freq[i], both 32-bit."""
    assert inv_freq.dtype == torch.float32
    half = inv_freq.numel()
    table = torch.empty(max_pos, half, 2, dtype=torch.float32, device=inv_freq.device)
    _check(library().ems_rope_table(_ptr(inv_freq, "inv_freq"), _ptr(table), max_pos, half,
                                    _stream()), "rope_table")
    return table


def rope_kv_write(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                  positions: torch.Tensor, row_of_token: torch.Tensor,
                  table: torch.Tensor | None, rotary_dim: int,
                  kcache: torch.Tensor | None, vcache: torch.Tensor | None,
                  block_tables: torch.Tensor | None, page_size: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k by the table rows of `positions`; store k and v of every
    token at its page slot.  qkv: [N, (nh + 2 nkv) D]; caches [pages, nkv, page_size, D]."""
    n = qkv.shape[0]
    assert qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim
    if write_kv:
        assert kcache is not None and vcache is not None and block_tables is not None
        assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype
        assert kcache.shape[1:] == (num_kv_heads, page_size, head_dim)
    bt_stride = block_tables.shape[1] if block_tables is not None else 0
    _check(library().ems_rope_kv_write(
        _ptr(qkv, "qkv"), _dt(qkv), n, num_heads, num_kv_heads, head_dim,
        _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _ptr(table, "table"),
        rotary_dim, _ptr(kcache, "kcache"), _ptr(vcache, "vcache"),
        _i32(block_tables, "block_tables"), bt_stride, page_size, 1 if write_kv else 0, _stream()),
        "rope_kv_write")


def stream_inject(residual: torch.Tensor, tokens: torch.Tensor, embed: torch.Tensor | None,
                  table: torch.Tensor | None, row: int = 0, deferred: torch.Tensor | None = None) -> None:
    """residual[n, :] += embed[tokens[n], :] + table[row, :] in 32 bits (either may be None); a token
    -(k + 1) reads deferred[k], as in `embedding`."""
    n, h = residual.shape
    assert residual.dtype == torch.float32 and (embed is not None or table is not None)
    src = embed if embed is not None else table
    assert embed is None or (embed.shape[1] == h and tokens.numel() >= n)
    assert table is None or (table.shape[1] == h and 0 <= row < table.shape[0] and table.dtype == src.dtype)
    vec = None if table is None else table[row]
    _check(library().ems_stream_inject(_ptr(residual, "residual"), _i32(tokens, "tokens"),
                                       None if deferred is None else _i32(deferred, "deferred"),
                                       _ptr(embed, "embed"), _ptr(vec, "table row"), _dt(src), n, h, _stream()),
           "stream_inject")


def add_norm_grouped(delta: torch.Tensor | None, post_gain: torch.Tensor | None, post_groups: int, post_eps: float,
                     residual: torch.Tensor, gain: torch.Tensor, groups: int, eps: float, out: torch.Tensor,
                     rows: torch.Tensor | None = None) -> None:
    """The grouped RMSNorm of the residual stream, with what joins the stream before it:

        residual += delta                                   (post_gain None)
        residual += grouped_norm(delta; post_groups, post_eps) * post_gain
        out = grouped_norm(residual; groups, eps) * gain

    where grouped_norm divides each of G equal consecutive parts of a row by sqrt(mean(part^2) + eps).
    All 32-bit; only `out` is rounded.  With `rows` only those rows are computed, compactly, and
    the residual is not written."""
    h = residual.shape[-1]
    assert residual.dtype == torch.float32 and gain.numel() == h and out.shape[-1] == h
    n_out = residual.shape[0] if rows is None else rows.numel()
    if delta is not None:
        assert delta.dtype == out.dtype and delta.shape[-1] == h and (rows is not None or delta.shape[0] >= n_out)
    if post_gain is not None:
        assert delta is not None and post_gain.numel() == h and post_gain.dtype == gain.dtype
    _check(library().ems_add_norm_grouped(
        _ptr(delta, "delta"), _ptr(post_gain, "post_gain"), _dt(gain), int(post_groups), float(post_eps),
        _ptr(residual, "residual"), _ptr(gain, "gain"), _dt(gain), int(groups), float(eps), _ptr(out, "out"),
        _dt(out), _i32(rows, "rows"), n_out, h, 0 if rows is not None else 1, _stream()), "add_norm_grouped")


# "swiglu_capped": with g = min(gate, limit) and u = clamp(up, -limit, limit) the result is
# g * sigmoid(alpha * g) * (u + 1); the other three are act(gate) * up.
GLU_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "swiglu_capped": 3}


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, act: str, limit: float = 0.0, alpha: float = 1.0,
            row_gate: bool = False) -> None:
    """out[n, i] = act(gate_up[n, i]) * gate_up[n, I + i] for act in `GLU_ACTIVATIONS` (`limit` and `alpha`
    are the constants of "swiglu_capped").  gate_up may have more columns than 2 I; with `row_gate`,
    column 2 I holds a number z per row and the row of `out` is multiplied by sigmoid(z)."""
    n, i = out.shape
    assert gate_up.shape[0] == n and gate_up.shape[1] >= 2 * i + (1 if row_gate else 0)
    assert gate_up.dtype == out.dtype and gate_up.is_contiguous()
    _check(library().ems_glu_act(_ptr(gate_up, "gate_up"), gate_up.shape[1], _ptr(out, "out"), _dt(out), n, i,
                                 GLU_ACTIVATIONS[act], float(limit), float(alpha), 1 if row_gate else 0, _stream()),
           "glu_act")


def add_cast(delta: torch.Tensor | None, residual: torch.Tensor, out: torch.Tensor) -> None:
    """residual += delta (32-bit; delta may be None); out = residual rounded to out's type: the stream
    itself as the operand of a product."""
    n, h = residual.shape
    assert residual.dtype == torch.float32 and out.shape == (n, h)
    assert delta is None or (delta.dtype == out.dtype and delta.shape[-1] == h and delta.shape[0] >= n)
    _check(library().ems_add_cast(_ptr(delta, "delta"), _ptr(residual, "residual"), _ptr(out, "out"), _dt(out), n, h,
                                  _stream()), "add_cast")


def token_gate(z: torch.Tensor, table: torch.Tensor, col0: int, tokens: torch.Tensor, out: torch.Tensor,
               deferred: torch.Tensor | None = None) -> None:
    """out[n, :] = gelu_tanh(z[n, :]) * table[tokens[n], col0 : col0 + C] (32-bit, rounded once); a token
    -(k + 1) reads deferred[k], as in `embedding`."""
    n, c = z.shape
    assert out.shape == (n, c) and z.dtype == out.dtype and table.dim() == 2 and tokens.numel() >= n
    _check(library().ems_token_gate(_ptr(z, "z"), _ptr(table, "table"), _dt(table), table.shape[1], int(col0),
                                    _i32(tokens, "tokens"), None if deferred is None else _i32(deferred, "deferred"),
                                    _ptr(out, "out"), _dt(out), n, c, _stream()), "token_gate")


def depth_mix(delta: torch.Tensor | None, gain: torch.Tensor | None, eps: float, residual: torch.Tensor,
              hist: torch.Tensor, weights: torch.Tensor | None, count: int) -> None:
    """The newest state of the stream, x = residual + delta (delta / sqrt(mean(delta^2) + eps) * gain when
    a gain is given; delta may be None), is stored as hist[count - 1]; the residual becomes
    sum_j weights[j] * hist[j] over j < count (it stays x when `weights` is None).  hist: [depths, N, H]
    float32; all of it 32-bit."""
    n, h = residual.shape
    assert residual.dtype == hist.dtype == torch.float32 and hist.shape[1:] == (n, h) and 1 <= count <= hist.shape[0]
    assert delta is None or (delta.shape[-1] == h and delta.shape[0] >= n)
    assert weights is None or (weights.dtype == torch.float32 and weights.numel() >= count)
    assert gain is None or (delta is not None and gain.numel() == h)
    dt = _dt(delta) if delta is not None else 0
    _check(library().ems_depth_mix(_ptr(delta, "delta"), _ptr(gain, "gain"), 0 if gain is None else _dt(gain),
                                   float(eps), _ptr(residual, "residual"), _ptr(hist, "hist"),
                                   _ptr(weights, "weights"), count, n * h, dt, n, h, _stream()), "depth_mix")


def causal_taps(x: torch.Tensor, weight: torch.Tensor, state: torch.Tensor | None, slots: torch.Tensor | None,
                cu_q: torch.Tensor, row_of_token: torch.Tensor, out: torch.Tensor, num_rows: int,
                bias: torch.Tensor | None = None, identity: bool = True) -> None:
    """out[t] = (x[t] if identity) + bias + sum_j weight[:, j] * x[t - taps + 1 + j] along each request's
    own tokens, with the inputs before the step's first token taken from `state` ([slots, taps - 1, C]
    float32, the last taps - 1 inputs of each request in time order), which is then brought up to
    date.  `x` may be a column range of a wider buffer."""
    n, c = x.shape
    taps = weight.shape[1]
    assert weight.shape[0] == c and out.shape == x.shape and out.dtype == x.dtype and x.stride(1) == 1
    assert bias is None or (bias.numel() == c and bias.dtype == weight.dtype)
    if taps > 1:
        assert state is not None and state.dtype == torch.float32 and state.shape[1:] == (taps - 1, c)
        assert slots is not None
    if not x.is_cuda:
        raise KernelError("x must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_causal_taps(
        x.data_ptr(), x.stride(0), _ptr(weight, "weight"), _dt(weight), _ptr(bias, "bias"), 1 if identity else 0,
        _ptr(state, "state"), _i32(slots, "slots"),
        _i32(cu_q, "cu_q"), _i32(row_of_token, "row_of_token"), _ptr(out, "out"), _dt(out), n, num_rows, c, taps,
        _stream()), "causal_taps", 2 if taps > 1 else 1)


ROTARY_PAIRINGS = {"half": 0, "interleaved": 1}


def latent_prep(proj: torch.Tensor, q_rank: int, kv_rank: int, rope_dim: int, q_gain: torch.Tensor,
                kv_gain: torch.Tensor, eps: float, positions: torch.Tensor, row_of_token: torch.Tensor,
                table: torch.Tensor | None, rot_dims: int, pairing: str, pages: torch.Tensor,
                block_tables: torch.Tensor, cq: torch.Tensor, write: bool = True) -> None:
    """The tokens of a step for latent attention.  proj: [N, >= q_rank + kv_rank + rope_dim] holds
    [query latent | key/value latent | shared key part | ...] per row.  cq = RMSNorm(query latent)
    * q_gain; the cache vector of the token, at its page slot, becomes [RMSNorm(kv latent) * kv_gain |
    rotate(shared key part)].  pages: [num_pages, page_size, kv_rank + rope_dim]."""
    n = proj.shape[0]
    assert proj.stride(1) == 1 and proj.shape[1] >= q_rank + kv_rank + rope_dim
    assert pages.dtype == proj.dtype == cq.dtype and pages.shape[2] == kv_rank + rope_dim
    assert cq.shape == (n, q_rank) and q_gain.numel() == q_rank and kv_gain.numel() == kv_rank
    assert q_gain.dtype == kv_gain.dtype and (table is None or table.dtype == torch.float32)
    if not proj.is_cuda:
        raise KernelError("proj must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_latent_prep(
        proj.data_ptr(), proj.stride(0), _dt(proj), n, q_rank, kv_rank, rope_dim, _ptr(q_gain, "q_gain"),
        _ptr(kv_gain, "kv_gain"), _dt(q_gain), float(eps), _i32(positions, "positions"),
        _i32(row_of_token, "row_of_token"), _ptr(table, "table"), rot_dims, ROTARY_PAIRINGS[pairing],
        _ptr(pages, "pages"), _i32(block_tables, "block_tables"), block_tables.shape[1], pages.shape[1],
        _ptr(cq, "cq"), 1 if write else 0, _stream()), "latent_prep")


def rope_inplace(x: torch.Tensor, num_heads: int, head_stride: int, offset: int, rot_dims: int, pairing: str,
                 positions: torch.Tensor, table: torch.Tensor) -> None:
    """Rotate, in place, `rot_dims` numbers of every head of x[N, :] that start `offset` into the
    head (head h begins at column h * head_stride), by the table rows of `positions`; pairing "half"
    joins entry i with i + rot_dims/2, "interleaved" joins 2i with 2i + 1."""
    assert x.stride(1) == 1 and table.dtype == torch.float32
    _check(library().ems_rope_inplace(_ptr(x, "x"), _dt(x), x.shape[0], x.stride(0), head_stride, offset, num_heads,
                                      rot_dims, ROTARY_PAIRINGS[pairing], _i32(positions, "positions"),
                                      _ptr(table, "table"), _stream()), "rope_inplace")


def latent_attention_scratch_bytes(num_tokens: int, num_heads: int, kv_rank: int, splits: int) -> int:
    return int(library().ems_latent_attention_scratch_bytes(num_tokens, num_heads, kv_rank, splits))


def latent_attention(qlat: torch.Tensor, q: torch.Tensor, rot_offset: int, head_stride: int, pages: torch.Tensor,
                     block_tables: torch.Tensor, positions: torch.Tensor, row_of_token: torch.Tensor,
                     out: torch.Tensor, num_heads: int, kv_rank: int, rope_dim: int, scale: float,
                     splits: int = 1, scratch: torch.Tensor | None = None, kernel: str = "auto") -> None:
    """Causal attention over cached latent vectors.  qlat: [H, N, kv_rank], the queries folded into
    the latent space; q: [N, H * head_stride] whose `rope_dim` numbers from `rot_offset` on in every
    head are the rotated query part; pages: [num_pages, page_size, kv_rank + rope_dim].
    out[h, n, :] = sum_j softmax_j((qlat[h, n] . c_j + qrot[n, h] . krot_j) * scale) c_j over the
    keys j <= position of token n of its request.  `splits` > 1 cuts every token's keys over
    that many blocks (`scratch` takes the partial sums; a merge kernel follows).  In bfloat16 the
    tensor-core kernel runs where it takes the sizes (kv_rank a multiple of 32 up to 512, rope_dim a
    multiple of 16); kernel="generic" keeps the CUDA-core kernel (tests compare the two)."""
    h, n, r = qlat.shape
    assert h == num_heads and r == kv_rank and out.shape == qlat.shape and pages.shape[2] == kv_rank + rope_dim
    assert qlat.dtype == q.dtype == out.dtype == pages.dtype and q.stride(1) == 1
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_latent_attention(
        _ptr(qlat, "qlat"), q.data_ptr() + rot_offset * q.element_size(), q.stride(0), head_stride, _dt(q),
        _ptr(pages, "pages"), _i32(block_tables, "block_tables"), block_tables.shape[1], pages.shape[1],
        _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _ptr(out, "out"), n, num_heads, kv_rank,
        rope_dim, float(scale), splits, _ptr(scratch, "scratch"),
        0 if scratch is None else scratch.numel() * scratch.element_size(), 1 if kernel == "generic" else 0,
        _stream()), "latent_attention", 2 if splits > 1 else 1)


def heads_gate(ov: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor) -> None:
    """out[n, h * V + i] = ov[h, n, i] * sigmoid(gate[n, h * V + i]); without a gate the plain
    transposition.  `gate` may be a column range of a wider buffer."""
    h, n, v = ov.shape
    assert out.shape == (n, h * v) and out.dtype == ov.dtype
    if gate is not None:
        assert gate.shape == (n, h * v) and gate.stride(1) == 1 and gate.dtype == ov.dtype
    _check(library().ems_heads_gate(_ptr(ov, "ov"), None if gate is None else gate.data_ptr(),
                                    0 if gate is None else gate.stride(0), _ptr(out, "out"), _dt(out), n, h, v,
                                    _stream()), "heads_gate")


def moe_tile_rows() -> int:
    """Rows of one tile of the grouped products of routed experts."""
    return int(library().ems_moe_tile_rows())


def moe_max_tiles(num_pairs: int, num_experts: int, tile_rows: int) -> int:
    """The most tiles that `num_pairs` (token, choice) pairs spread over the experts can make."""
    return num_pairs // tile_rows + min(num_experts, num_pairs)


MOE_BIG_TILE_ROWS = 256  # rows of a tile of the tcgen05 grouped product
MOE_SCORINGS = {"softmax": 0, "sigmoid": 1}
EXPERT_ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "gelu": 4}  # of experts without a gate ("gelu": the erf form)


def moe_route(logits: torch.Tensor, top: int, renormalize: bool, ids: torch.Tensor, weights: torch.Tensor,
              offsets: torch.Tensor, perm: torch.Tensor, plan: torch.Tensor, max_tiles: int,
              align: int = 1, big: torch.Tensor | None = None, inv: torch.Tensor | None = None,
              scoring: str = "softmax", correction: torch.Tensor | None = None, renorm_eps: float = 0.0,
              scale: float = 1.0, plan_experts: int | None = None) -> None:
    """From router logits [N, E] (float32): softmax over all experts (or, with scoring "sigmoid", the
    sigmoid of every logit by itself), the `top` largest per token
    (ids, weights: [N, top]; the weights are the scores, divided by their sum if `renormalize`),
    the first sorted row of every expert (offsets [E + 1], in a buffer of 3 E + 1: counters follow),
    the pairs t * top + k in expert order
    (perm [N * top]) and the tiles of the grouped products (plan: count, then expert / first row /
    rows per tile).  With `align` > 1 (steps of more than 512 tokens) every expert's sorted rows
    start at a multiple of `align`, `perm` (len(big) * align entries) is -1 between them, and `big`
    (int32) receives the expert of every group of `align` rows, -1 where none; `inv` (optional, the
    same steps) receives the sorted row of every pair.  With `correction` (float32 [E]) the experts are
    chosen by score + correction while the weights stay the scores; `renorm_eps` joins the sum that
    `renormalize` divides by; `scale` multiplies the weights; experts at and past `plan_experts` get no
    tiles (they have no weights; `moe_combine` returns their input)."""
    n, e = logits.shape
    assert correction is None or (correction.dtype == torch.float32 and correction.numel() == e)
    assert logits.dtype == torch.float32 and weights.dtype == torch.float32
    assert ids.numel() >= n * top and weights.numel() >= n * top and perm.numel() >= n * top
    assert offsets.numel() >= 3 * e + 1 and plan.numel() >= 1 + 3 * max_tiles
    max_big = 0 if big is None else big.numel()
    assert align == 1 or (big is not None and perm.numel() >= max_big * align)
    _check(library().ems_moe_route(_ptr(logits, "logits"), n, e, top, 1 if renormalize else 0, _i32(ids, "ids"),
                                   _ptr(weights, "weights"), _i32(offsets, "offsets"), _i32(perm, "perm"),
                                   _i32(plan, "plan"), max_tiles, align, _i32(big, "big"), max_big,
                                   _i32(inv, "inv"), MOE_SCORINGS[scoring], _ptr(correction, "correction"),
                                   float(renorm_eps), float(scale), int(plan_experts or 0), _stream()),
           "moe_route", 1 if n <= 512 else 4)


def moe_gather(x: torch.Tensor, perm: torch.Tensor, top: int, xs: torch.Tensor) -> None:
    """xs[i] = x[perm[i] // top] for the sorted rows i with perm[i] >= 0 (bfloat16, K a multiple of 8)."""
    rows, k = xs.shape
    assert x.shape[1] == k and x.dtype == xs.dtype == torch.bfloat16 and perm.numel() >= rows
    _check(library().ems_moe_gather(_ptr(x, "x"), _i32(perm, "perm"), rows, top, k, _ptr(xs, "xs"), _stream()),
           "moe_gather")


def moe_up_grouped_tc05_supported(inter: int, k: int) -> bool:
    """Whether the tcgen05 grouped gate/up product takes the sizes (bfloat16; SiLU or the capped form)."""
    return inter % 128 == 0 and k % 8 == 0


def moe_up_grouped_tc05(xs: torch.Tensor, wgu: torch.Tensor, big: torch.Tensor, out: torch.Tensor,
                        act: str = "silu", perm: torch.Tensor | None = None, in_scale: torch.Tensor | None = None,
                        limit: float = 0.0, alpha: float = 1.0) -> None:
    """out[i, :] = silu(xs[i] Wg[e]^T) * (xs[i] Wu[e]^T) for the rows of every group of 256 sorted rows
    that `big` gives to an expert e (-1: the group is skipped): the two-SM tcgen05 kernel of prompt
    steps in its grouped form.  xs: [len(big) * 256, K]; wgu: [E, 2 * ff, K].  `act` "swiglu_capped" takes
    `limit` and `alpha` as in `moe_up`; with `in_scale` (float32, one number per pair) and `perm` (the pair
    of every sorted row, -1 between experts) both 32-bit sums of a row are multiplied by its pair's number."""
    e, ff2, k = wgu.shape
    rows = xs.shape[0]
    assert rows == big.numel() * MOE_BIG_TILE_ROWS and xs.shape[1] == k and out.shape == (rows, ff2 // 2)
    assert xs.dtype == wgu.dtype == out.dtype == torch.bfloat16 and act in ("silu", "swiglu_capped")
    assert in_scale is None or (perm is not None and perm.numel() >= rows)
    _check(library().ems_moe_up_grouped_tc05(_ptr(xs, "xs"), _ptr(wgu, "wgu"), _ptr(out, "out"), rows, ff2 // 2, k,
                                             e, _i32(big, "big"), None if in_scale is None else _i32(perm, "perm"),
                                             _f32(in_scale, "in_scale"), 1 if act == "swiglu_capped" else 0,
                                             float(limit), float(alpha), _stream()), "moe_up_grouped_tc05")


def moe_up(x: torch.Tensor, wgu: torch.Tensor, perm: torch.Tensor, offsets: torch.Tensor, plan: torch.Tensor,
           max_tiles: int, top: int, act: str, out: torch.Tensor, kernel: str = "auto",
           in_scale: torch.Tensor | None = None, limit: float = 0.0, alpha: float = 1.0, gated: bool = True) -> None:
    """out[i, :] = act(x[t] Wg[e]^T) * (x[t] Wu[e]^T) for sorted pair i (token t = perm[i] // top) of
    expert e; wgu: [E, 2 * ff, K] with the gate rows first.  bfloat16 runs on the tensor cores where K
    is a multiple of 8; kernel="generic" keeps the CUDA-core kernel.  With `in_scale` (float32, one
    number per pair) the expert reads in_scale[pair] * x[t]: both 32-bit sums are multiplied by it.
    `limit` and `alpha` are the constants of the activation "swiglu_capped".  With `gated` False the experts
    have no gate: wgu is [E, ff, K] and out[i, :] = act(x[t] Wu[e]^T), act one of `EXPERT_ACTIVATIONS`."""
    e, ff2, k = wgu.shape
    ff = ff2 // 2 if gated else ff2
    assert x.shape[1] == k and out.shape[1] == ff and x.dtype == wgu.dtype == out.dtype
    code = GLU_ACTIVATIONS[act] if gated else EXPERT_ACTIVATIONS[act]
    _check(library().ems_moe_up(_ptr(x, "x"), _ptr(wgu, "wgu"), _dt(x), _i32(perm, "perm"), _i32(plan, "plan"),
                                max_tiles, top, ff, k, code, _ptr(out, "out"),
                                1 if kernel == "generic" else 0, _f32(in_scale, "in_scale"), float(limit),
                                float(alpha), 1 if gated else 0, _stream()), "moe_up")


def moe_down(act: torch.Tensor, wdown: torch.Tensor, perm: torch.Tensor, offsets: torch.Tensor, plan: torch.Tensor,
             max_tiles: int, y: torch.Tensor, kernel: str = "auto") -> None:
    """y[perm[i], :] = act[i, :] Wd[e]^T (float32, in pair order) for sorted pair i of expert e;
    wdown: [E, H, ff]."""
    e, h, ff = wdown.shape
    assert act.shape[1] == ff and y.shape[1] == h and y.dtype == torch.float32 and act.dtype == wdown.dtype
    _check(library().ems_moe_down(_ptr(act, "act"), _ptr(wdown, "wdown"), _dt(act), _i32(perm, "perm"),
                                  _i32(plan, "plan"), max_tiles, h, ff, _ptr(y, "y"),
                                  1 if kernel == "generic" else 0, _stream()), "moe_down")


def moe_down_grouped_tc05(act: torch.Tensor, wdown: torch.Tensor, big: torch.Tensor, y: torch.Tensor) -> None:
    """y[i, :] = act[i, :] Wd[e]^T (bfloat16) for the rows of every group of 256 sorted rows that `big`
    gives to an expert e: the grouped tcgen05 kernel.  wdown: [E, H, ff]."""
    e, h, ff = wdown.shape
    rows = act.shape[0]
    assert rows == big.numel() * MOE_BIG_TILE_ROWS and act.shape[1] == ff and y.shape == (rows, h)
    assert act.dtype == wdown.dtype == y.dtype == torch.bfloat16
    _check(library().ems_moe_down_grouped_tc05(_ptr(act, "act"), _ptr(wdown, "wdown"), _ptr(y, "y"), rows, h, ff, e,
                                               _i32(big, "big"), _stream()), "moe_down_grouped_tc05")


def moe_combine_rows(y: torch.Tensor, inv: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor, top: int,
                     extra: torch.Tensor | None = None, ids: torch.Tensor | None = None, x: torch.Tensor | None = None,
                     num_real: int = 0) -> None:
    """out[t, :] = sum_k weights[t, k] * y[inv[t * top + k], :] (k ascending; every weight 1 when `weights` is
    None) + extra[t, :] (optional) for bfloat16 rows `y` in the sorted layout.  With `ids`, `x` and `num_real`
    a choice whose expert id is at or past `num_real` contributes x[t] instead (as in `moe_combine`)."""
    n, h = out.shape
    assert y.dtype == out.dtype == torch.bfloat16 and y.shape[1] == h
    assert weights is None or weights.dtype == torch.float32
    assert extra is None or (extra.dtype == out.dtype and extra.shape == out.shape)
    assert x is None or (ids is not None and x.dtype == out.dtype and x.shape == out.shape and x.is_contiguous())
    _check(library().ems_moe_combine_rows(_ptr(y, "y"), _i32(inv, "inv"), _ptr(weights, "weights"), _ptr(out, "out"),
                                          n, top, h, _ptr(extra, "extra"), None if x is None else _i32(ids, "ids"),
                                          _ptr(x, "x"), int(num_real), _stream()), "moe_combine_rows")


def moe_combine(y: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor, top: int,
                extra: torch.Tensor | None = None, ids: torch.Tensor | None = None, x: torch.Tensor | None = None,
                num_real: int = 0) -> None:
    """out[t, :] = sum_k weights[t, k] * y[t * top + k, :] (k ascending; every weight 1 when `weights` is
    None) + extra[t, :] (optional, of out's type).  With `ids` ([N * top] int32), `x` ([N, H], of out's type)
    and `num_real`, a choice whose expert id is at or past `num_real` contributes x[t] instead of its row of y
    (an expert that returns its input)."""
    n, h = out.shape
    assert y.dtype == torch.float32 and y.shape[1] == h and (weights is None or weights.dtype == torch.float32)
    assert extra is None or (extra.dtype == out.dtype and extra.shape == out.shape)
    assert x is None or (ids is not None and x.dtype == out.dtype and x.shape == out.shape and x.is_contiguous())
    _check(library().ems_moe_combine(_ptr(y, "y"), _ptr(weights, "weights"), _ptr(out, "out"), _dt(out), n, top, h,
                                     _ptr(extra, "extra"), None if x is None else _i32(ids, "ids"), _ptr(x, "x"),
                                     int(num_real), _stream()), "moe_combine")


def attention_scratch_bytes(num_tokens: int, num_heads: int, head_dim: int, splits: int) -> int:
    return int(library().ems_paged_attention_scratch_bytes(num_tokens, num_heads, head_dim, splits))


_ATTENTION_IMPL = {"auto": 0, "generic": 1, "tcgen05": 2, "mma": 3}


def paged_attention(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                    block_tables: torch.Tensor, cu_q: torch.Tensor, starts: torch.Tensor,
                    num_rows: int, num_tokens: int, num_heads: int, num_kv_heads: int,
                    head_dim: int, scale: float, max_q_len: int, window: int | None = None,
                    splits: int = 1, scratch: torch.Tensor | None = None, generic: bool = False,
                    tcgen05: bool = False, kernel: str = "auto") -> None:
    """Causal grouped-query attention of every packed query over its request's pages.
    `q` is a [N, stride] tensor whose first nh*D columns are the queries (a view of the
    qkv buffer is fine); `out` is [N, nh*D].  `generic=True` forces the generic kernel where
    a faster one would take the case (tests compare the two); `tcgen05=True` asks for the
    tcgen05 prompt kernel at any length (by default it takes the long portions) and raises if
    that kernel does not take the case.  `kernel` says the same by name: "auto", "generic",
    "tcgen05", or "mma" (the mma.sync kernels where they take the case)."""
    assert q.stride(1) == 1 and out.is_contiguous() and q.dtype == out.dtype == kcache.dtype
    page_size = kcache.shape[2]
    assert kcache.shape[1] == num_kv_heads and kcache.shape[3] == head_dim
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_paged_attention(
        q.data_ptr(), q.stride(0), _ptr(out, "out"), _dt(out), _ptr(kcache, "kcache"),
        _ptr(vcache, "vcache"), _i32(block_tables, "block_tables"), block_tables.shape[1], page_size,
        _i32(cu_q, "cu_q"), _i32(starts, "starts"), num_rows, num_tokens, num_heads, num_kv_heads,
        head_dim, int(window or 0), float(scale), max_q_len, splits,
        _ptr(scratch, "scratch"), 0 if scratch is None else scratch.numel() * scratch.element_size(),
        _ATTENTION_IMPL["generic" if generic else ("tcgen05" if tcgen05 else kernel)], _stream()),
        "paged_attention", 2 if splits > 1 else 1)


def decode_attention_fused_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                                     rotary_dim: int) -> bool:
    """Whether `decode_attention_fused` takes the geometry (the alignment of the tensors is
    checked by the call itself)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and num_heads // num_kv_heads <= 16
            and rotary_dim in (0, head_dim))


def decode_attention_fused(qkv: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                           block_tables: torch.Tensor, cu_q: torch.Tensor, starts: torch.Tensor, num_rows: int,
                           num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                           rope_table: torch.Tensor | None, rotary_dim: int, write_kv: bool,
                           window: int | None = None, splits: int = 1, scratch: torch.Tensor | None = None) -> None:
    """A decode step's attention (every row brings one token) with the rotary encoding of q and
    k and the write of the new key and value done by the attention kernel itself: `qkv` holds
    the raw projections [q | k | v].  With `splits` > 1, `scratch` takes the partials and the merge
    kernel follows."""
    assert qkv.stride(1) == 1 and out.is_contiguous() and qkv.dtype == out.dtype == kcache.dtype == torch.bfloat16
    assert rope_table is None or rope_table.dtype == torch.float32
    _check(library().ems_decode_attention_fused(
        qkv.data_ptr(), qkv.stride(0), _ptr(out, "out"), _ptr(kcache, "kcache"), _ptr(vcache, "vcache"),
        _i32(block_tables, "block_tables"), block_tables.shape[1], kcache.shape[2], _i32(cu_q, "cu_q"),
        _i32(starts, "starts"), num_rows, num_heads, num_kv_heads, head_dim, int(window or 0), float(scale),
        _ptr(rope_table, "rope_table"), rotary_dim, 1 if write_kv else 0, splits, _ptr(scratch, "scratch"),
        0 if scratch is None else scratch.numel() * scratch.element_size(), _stream()),
        "decode_attention_fused", 2 if splits > 1 else 1)


# ---------------------------------------------------------------------------------------
# ungated feed-forward, prepared attention heads, masked attention, recurrent mixers

UNARY_ACTIVATIONS = {"relu": 0, "relu2": 1, "gelu_tanh": 2, "silu": 3, "gelu": 4}  # "gelu": the erf form


def unary_act(x: torch.Tensor, out: torch.Tensor, act: str) -> None:
    """out = act(x) elementwise for act in `UNARY_ACTIVATIONS` (relu2 is the square of relu)."""
    assert x.shape == out.shape and x.dtype == out.dtype
    _check(library().ems_unary_act(_ptr(x, "x"), _ptr(out, "out"), _dt(out), x.numel(), UNARY_ACTIVATIONS[act],
                                   _stream()), "unary_act")


def qk_prep(proj: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, positions: torch.Tensor,
            row_of_token: torch.Tensor, table: torch.Tensor | None, rot_dims: int, pairing: str,
            norm_eps: float | None, kcache: torch.Tensor, vcache: torch.Tensor, block_tables: torch.Tensor,
            values_are_keys: bool, write: bool = True, v_norm_eps: float | None = None,
            v_table: torch.Tensor | None = None, v_pairing: str = "half", q_gain: torch.Tensor | None = None,
            k_gain: torch.Tensor | None = None, norm_first: bool = False) -> None:
    """The tokens of a step for attention over a paged cache.  proj: [N, >= (nh + nkv (+ nkv)) * D]
    holds [q | k | v] per row (no v when `values_are_keys`: the value of a token is then its key as
    projected).  Every head of q and k is rotated by the table rows of `positions` on its first
    `rot_dims` numbers and, with `norm_eps`, divided by its root mean square; q is rewritten in
    place, k and v go to the token's page slot.  caches: [pages, nkv, page_size, D]; the value cache may
    have another last dimension DV (the v columns of `proj` are then nkv * DV wide).  With `v_norm_eps`
    every value head is divided by its root mean square, and with `v_table` ([positions, DV / 2, 2]) it
    is turned by the token's position over its whole length, before it is cached.  With `norm_first`
    the norm of q and k comes BEFORE their rotation; `q_gain` / `k_gain` ([head_dim], shared by the heads, of
    one type) multiply the normed heads."""
    n = proj.shape[0]
    assert (q_gain is None) == (k_gain is None)
    assert q_gain is None or (q_gain.numel() == k_gain.numel() == head_dim and q_gain.dtype == k_gain.dtype
                              and norm_eps is not None)
    dv = vcache.shape[3]
    cols = (num_heads + num_kv_heads) * head_dim + (0 if values_are_keys else num_kv_heads * dv)
    assert proj.stride(1) == 1 and proj.shape[1] >= cols
    assert kcache.dtype == vcache.dtype == proj.dtype and kcache.shape[1] == num_kv_heads and kcache.shape[3] == head_dim
    assert table is None or (table.dtype == torch.float32 and table.shape[1] * 2 == rot_dims)
    assert v_table is None or (v_table.dtype == torch.float32 and v_table.shape[1] * 2 == dv)
    if not proj.is_cuda:
        raise KernelError("proj must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_qk_prep(
        proj.data_ptr(), proj.stride(0), _dt(proj), n, num_heads, num_kv_heads, head_dim,
        _i32(positions, "positions"), _i32(row_of_token, "row_of_token"), _ptr(table, "table"),
        rot_dims if table is not None else 0, ROTARY_PAIRINGS[pairing], 0 if norm_eps is None else 1,
        float(norm_eps or 0.0), _ptr(kcache, "kcache"), _ptr(vcache, "vcache"), _i32(block_tables, "block_tables"),
        block_tables.shape[1], kcache.shape[2], 1 if values_are_keys else 0, 1 if write else 0, dv,
        0 if v_norm_eps is None else 1, float(v_norm_eps or 0.0), _ptr(v_table, "v_table"),
        ROTARY_PAIRINGS[v_pairing], _ptr(q_gain, "q_gain"), _ptr(k_gain, "k_gain"),
        0 if q_gain is None else _dt(q_gain), 1 if norm_first else 0, _stream()), "qk_prep")


def paged_attention_masked(q: torch.Tensor, out: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor,
                           block_tables: torch.Tensor, cu_q: torch.Tensor, starts: torch.Tensor,
                           num_rows: int, num_tokens: int, num_heads: int, num_kv_heads: int,
                           head_dim: int, scale: float, max_q_len: int, window: int | None = None,
                           chunk: int | None = None, sinks: torch.Tensor | None = None,
                           gate: torch.Tensor | None = None, splits: int = 1,
                           scratch: torch.Tensor | None = None, kernel: str = "auto", keep_first: int = 0,
                           out_table: torch.Tensor | None = None, out_pairing: str = "half",
                           positions: torch.Tensor | None = None, softcap: float | None = None) -> None:
    """`paged_attention` with three optional extras: `chunk` (the query at position p sees key j <= p
    only if j // chunk == p // chunk, chunks counted from position 0 of the request), `sinks`
    (float32 [nh]: exp(sinks[h]) is added to head h's softmax denominator; it has no value) and
    `gate` ([N, >= nh], may be a column range of a wider buffer: head h's output is multiplied by
    sigmoid(gate[n, h])).  Further: `keep_first` (keys j < keep_first stay visible to every later query
    beside the window or chunk); a value cache whose last dimension DV differs from head_dim (out is
    then [N, nh * DV]); `out_table` ([positions, DV / 2, 2]: the values were turned by their positions
    when they were cached, and each head's result is turned back by the query's position, positions[n]
    of token n); `softcap` (a scaled score s enters the softmax as softcap * tanh(s / softcap))."""
    assert q.stride(1) == 1 and out.is_contiguous() and q.dtype == out.dtype == kcache.dtype
    page_size = kcache.shape[2]
    dv = vcache.shape[3]
    assert kcache.shape[1] == num_kv_heads and kcache.shape[3] == head_dim and out.shape[1] == num_heads * dv
    assert out_table is None or (out_table.dtype == torch.float32 and out_table.shape[1] * 2 == dv
                                 and positions is not None)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == num_heads)
    assert gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[1] >= num_heads)
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_paged_attention_masked(
        q.data_ptr(), q.stride(0), _ptr(out, "out"), _dt(out), _ptr(kcache, "kcache"),
        _ptr(vcache, "vcache"), _i32(block_tables, "block_tables"), block_tables.shape[1], page_size,
        _i32(cu_q, "cu_q"), _i32(starts, "starts"), num_rows, num_tokens, num_heads, num_kv_heads,
        head_dim, int(window or 0), int(chunk or 0), _ptr(sinks, "sinks"),
        None if gate is None else gate.data_ptr(), 0 if gate is None else gate.stride(0), float(scale), max_q_len,
        splits, _ptr(scratch, "scratch"), 0 if scratch is None else scratch.numel() * scratch.element_size(),
        _ATTENTION_IMPL[kernel], int(keep_first or 0), dv, _ptr(out_table, "out_table"),
        ROTARY_PAIRINGS[out_pairing], None if positions is None else _i32(positions, "positions"),
        float(softcap or 0.0), _stream()),
        "paged_attention_masked", 2 if splits > 1 else 1)


def norm_mean2(a: torch.Tensor, b: torch.Tensor, gain_a: torch.Tensor, gain_b: torch.Tensor, eps: float,
               out: torch.Tensor) -> None:
    """out = (rms(a) * gain_a + rms(b) * gain_b) / 2 over rows of equal width, statistics in 32 bits."""
    n, c = a.shape
    assert b.shape == out.shape == (n, c) and a.dtype == b.dtype == out.dtype
    assert gain_a.numel() == gain_b.numel() == c and gain_a.dtype == gain_b.dtype
    _check(library().ems_norm_mean2(_ptr(a, "a"), _ptr(b, "b"), _ptr(gain_a, "gain_a"), _ptr(gain_b, "gain_b"),
                                    _dt(gain_a), _ptr(out, "out"), _dt(out), n, c, float(eps), _stream()),
           "norm_mean2")


MEMORY_INPUT_ACTIVATIONS = {"none": 0, "silu": 1}


def _f32(t: torch.Tensor | None, name: str) -> int | None:
    if t is not None and t.dtype != torch.float32:
        raise KernelError(f"{name} must be float32, got {t.dtype}")
    return _ptr(t, name)


def matrix_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_heads: int, dim: int, vdim: int,
                      state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, num_rows: int,
                      out: torch.Tensor, act: str = "none", q_scale: float = 1.0,
                      decay_head: torch.Tensor | None = None, a: torch.Tensor | None = None,
                      b: torch.Tensor | None = None, denom_floor: torch.Tensor | None = None,
                      denom: torch.Tensor | None = None, denom_eps: float = 0.0, qk_heads: int | None = None) -> None:
    """A matrix memory per head, run over every request's tokens in order:

        S_t = a_t S_(t-1) + b_t k_t v_t^T,        out_t = S_t^T (q_t * q_scale)

    q, k: [N, >= H * dim], v: [N, >= H * vdim] (column ranges of wider buffers are fine), each passed
    through `act` first; a_t is `decay_head[h]` for every token or `a[t, h]`; b_t is `b[t, h]` or 1.
    state: float32 [slots, H, per_head] holding S ([dim, vdim]) and, when `denom` is given, the
    normaliser n_t = a_t n_(t-1) + b_t k_t ([dim]) behind it; then denom[t, h] = max(|n_t . q_t|,
    denom_floor[t, h]) + denom_eps.  out: float32 [N, H * vdim], not yet divided.  With `qk_heads` (a
    divisor of H) q and k have that many heads and head h reads q / k head h // (H / qk_heads)."""
    n = q.shape[0]
    assert q.stride(1) == k.stride(1) == v.stride(1) == 1 and q.dtype == k.dtype == v.dtype
    assert out.dtype == torch.float32 and out.shape == (n, num_heads * vdim) and state.dtype == torch.float32
    assert state.dim() == 3 and state.shape[1] == num_heads
    assert (decay_head is None) != (a is None)
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_matrix_recurrence(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), _dt(q),
        MEMORY_INPUT_ACTIVATIONS[act], float(q_scale), _f32(decay_head, "decay_head"), _f32(a, "a"), _f32(b, "b"),
        _f32(denom_floor, "denom_floor"), float(denom_eps), _f32(denom, "denom"), _ptr(state, "state"),
        state.shape[2], 0 if denom is None else 1, _i32(slots, "slots"), _i32(cu_q, "cu_q"), num_rows, n,
        num_heads, dim, vdim, _ptr(out, "out"), int(qk_heads or 0), _stream()), "matrix_recurrence")


def mlstm_gates(pre: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float, state: torch.Tensor,
                m_offset: int, slots: torch.Tensor, cu_q: torch.Tensor, num_rows: int, a: torch.Tensor,
                b: torch.Tensor, floor: torch.Tensor) -> None:
    """The stabilised exponential gates of an mLSTM.  pre: float32 [N, 2 H], input-gate then
    forget-gate pre-activations.  i = cap tanh((pre_i + bias_i) / cap), f = logsigmoid(cap tanh((pre_f +
    bias_f) / cap)); the running maximum m_t = max(f + m_(t-1), i) lives at state[slot, h, m_offset]
    (0 in a fresh slot); a = exp(f + m_(t-1) - m_t), b = exp(i - m_t), floor = exp(-m_t), float32 [N, H]."""
    n, h2 = pre.shape
    h = h2 // 2
    assert pre.dtype == torch.float32 and state.dtype == torch.float32 and state.shape[1] == h
    assert bias_i.numel() == bias_f.numel() == h and bias_i.dtype == bias_f.dtype
    assert a.shape == b.shape == floor.shape == (n, h)
    _check(library().ems_mlstm_gates(
        _f32(pre, "pre"), _ptr(bias_i, "bias_i"), _ptr(bias_f, "bias_f"), _dt(bias_i), float(cap),
        _ptr(state, "state"), state.shape[2], m_offset, _i32(slots, "slots"), _i32(cu_q, "cu_q"), num_rows, h,
        _f32(a, "a"), _f32(b, "b"), _f32(floor, "floor"), _stream()), "mlstm_gates")


def group_norm_gate(o: torch.Tensor, groups: int, eps: float, weight: torch.Tensor, gate: torch.Tensor | None,
                    out: torch.Tensor, denom: torch.Tensor | None = None) -> None:
    """out = rms_g(o / denom) * weight * sigmoid(gate): `o` float32 [N, C] is divided per (token, group)
    by `denom` ([N, groups], optional), each of `groups` equal consecutive parts of a row by its
    root mean square; `gate` ([N, >= C], may be a column range) is optional."""
    n, c = o.shape
    assert o.dtype == torch.float32 and out.shape == (n, c) and weight.numel() == c
    assert gate is None or (gate.dtype == out.dtype and gate.stride(1) == 1 and gate.shape[1] >= c)
    assert denom is None or denom.shape == (n, groups)
    if not o.is_cuda:
        raise KernelError("o must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_group_norm_gate(
        _f32(o, "o"), _f32(denom, "denom"), _ptr(weight, "weight"), _dt(weight),
        None if gate is None else gate.data_ptr(), 0 if gate is None else gate.stride(0), _ptr(out, "out"), _dt(out),
        n, c, groups, float(eps), _stream()), "group_norm_gate")


def rglru_scan(u: torch.Tensor, pre: torch.Tensor, bias_r: torch.Tensor, bias_i: torch.Tensor, lam: torch.Tensor,
               y: torch.Tensor, y_act: bool, cmul: float, state: torch.Tensor, slots: torch.Tensor,
               cu_q: torch.Tensor, num_rows: int, out: torch.Tensor, blocks: int) -> None:
    """A gated diagonal recurrence per channel over every request's tokens in order:

        r = sigmoid(pre_r + bias_r), i = sigmoid(pre_i + bias_i), a = exp(-cmul * r * softplus(lam)),
        S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t,      out_t = S_t * (gelu_tanh(y_t) if y_act else y_t)

    u, out: [N, C]; pre: float32 [2, blocks, N, C / blocks] (the r gates, then the i gates, block by block);
    y: [N, >= C], may be a column range; state: float32 [slots, C]."""
    n, c = u.shape
    assert pre.dtype == torch.float32 and pre.numel() == 2 * n * c and state.dtype == torch.float32
    assert state.shape[1:] == (c,) and out.shape == (n, c) and out.dtype == u.dtype == y.dtype and y.stride(1) == 1
    assert bias_r.numel() == bias_i.numel() == lam.numel() == c and bias_r.dtype == bias_i.dtype == lam.dtype
    if not u.is_cuda:
        raise KernelError("u must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_rglru_scan(
        _ptr(u, "u"), _f32(pre, "pre"), _ptr(bias_r, "bias_r"), _ptr(bias_i, "bias_i"), _ptr(lam, "lam"),
        _dt(lam), y.data_ptr(), y.stride(0), 1 if y_act else 0, float(cmul), _ptr(state, "state"),
        _i32(slots, "slots"), _i32(cu_q, "cu_q"), _ptr(out, "out"), _dt(out), num_rows, n, c, blocks, _stream()),
        "rglru_scan")


def add_scaled_norm2(deltas: "list[tuple[torch.Tensor, float]]", residual: torch.Tensor, gain1: torch.Tensor | None,
                     gain2: torch.Tensor | None, gain_offset: float, eps: float, out1: torch.Tensor | None,
                     out2: torch.Tensor | None) -> None:
    """residual += sum_i scale_i * delta_i (up to three pairs (delta, scale); 32-bit sum), then with r =
    rsqrt(mean(residual^2) + eps): out1 = residual r (gain1 + gain_offset), out2 = residual r (gain2 +
    gain_offset); either output may be None (then no norm is computed for it)."""
    n, c = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and len(deltas) <= 3
    outs = [o for o in (out1, out2) if o is not None]
    dt = outs[0].dtype if outs else (deltas[0][0].dtype if deltas else torch.float32)
    for d, _ in deltas:
        assert d.shape == (n, c) and d.dtype == dt and d.is_contiguous()
    for o, g in ((out1, gain1), (out2, gain2)):
        assert o is None or (o.shape == (n, c) and o.dtype == dt and o.is_contiguous() and g is not None and g.numel() == c)
    gains = [g for g in (gain1, gain2) if g is not None]
    assert len({g.dtype for g in gains}) <= 1
    if not residual.is_cuda:
        raise KernelError("residual must be a CUDA tensor (emberserve_b200 has no CPU path)")
    ds = [d for d, _ in deltas] + [None] * (3 - len(deltas))
    sc = [float(x) for _, x in deltas] + [0.0] * (3 - len(deltas))
    _check(library().ems_add_scaled_norm2(
        _ptr(ds[0], "delta"), _ptr(ds[1], "delta"), _ptr(ds[2], "delta"), sc[0], sc[1], sc[2], _ptr(residual, "residual"),
        _ptr(gain1 if out1 is not None else None, "gain1"), _ptr(gain2 if out2 is not None else None, "gain2"),
        _dt(gains[0]) if gains else 0, float(gain_offset), float(eps), _ptr(out1, "out1"), _ptr(out2, "out2"),
        0 if dt == torch.float32 else 1, n, c, _stream()), "add_scaled_norm2")


def stream_norm(residual: torch.Tensor, gain: torch.Tensor, gain_offset: float, eps: float) -> None:
    """residual <- residual / sqrt(mean(residual^2) + eps) * (gain + gain_offset), in place, 32-bit."""
    n, c = residual.shape
    assert residual.dtype == torch.float32 and residual.is_contiguous() and gain.numel() == c
    if not residual.is_cuda:
        raise KernelError("residual must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_stream_norm(_ptr(residual, "residual"), _ptr(gain, "gain"), _dt(gain), float(gain_offset),
                                     float(eps), n, c, _stream()), "stream_norm")


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place (float32)."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    if not x.is_cuda:
        raise KernelError("x must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_softcap(_ptr(x, "x"), x.numel(), float(cap), _stream()), "softcap")


def delta_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, g_raw: torch.Tensor,
                     g_bias: torch.Tensor, a_log: torch.Tensor, num_heads: int, qk_heads: int, dim: int, vdim: int,
                     state: torch.Tensor, slots: torch.Tensor, cu_q: torch.Tensor, num_rows: int, out: torch.Tensor,
                     act: str = "silu", unit_eps: float | None = 1e-6, q_scale: float = 1.0,
                     work: torch.Tensor | None = None) -> None:
    """A matrix memory per head written by the delta rule with a decay per key channel, run over every
    request's tokens in order:

        S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   out_t = S^T q_t

    q, k: [N, >= qk_heads * dim], v: [N, >= H * vdim], beta: [N, >= H] (column ranges of wider buffers are
    fine), each of q, k, v passed through `act`; with `unit_eps` q and k become x / sqrt(sum(x^2) + unit_eps)
    per head; q is multiplied by `q_scale`; beta_t = sigmoid(beta[t, h]); g_t = exp(-exp(a_log[h]) *
    softplus(g_raw[t, h * dim + d] + g_bias[h * dim + d])) with g_raw float32 [N, H * dim].  Head h reads
    q / k head h // (H / qk_heads).  state: float32 [slots, H, dim * vdim]; out: float32 [N, H * vdim].
    `work`: float32, at least `delta_work_floats(N, H, qk_heads, dim, vdim)` elements, where a first kernel leaves
    the prepared q, k, decays, v, k . q and beta of every token (allocated here when None)."""
    n = q.shape[0]
    assert q.stride(1) == k.stride(1) == v.stride(1) == beta.stride(1) == 1 and q.dtype == k.dtype == v.dtype == beta.dtype
    assert out.dtype == torch.float32 and out.shape == (n, num_heads * vdim) and out.is_contiguous()
    assert state.dtype == torch.float32 and state.dim() == 3 and state.shape[1:] == (num_heads, dim * vdim)
    assert g_raw.dtype == torch.float32 and g_raw.shape == (n, num_heads * dim) and g_raw.is_contiguous()
    assert g_bias.numel() == num_heads * dim and a_log.numel() == num_heads and g_bias.dtype == a_log.dtype
    if not q.is_cuda:
        raise KernelError("q must be a CUDA tensor (emberserve_b200 has no CPU path)")
    if work is None:
        work = torch.empty(delta_work_floats(n, num_heads, qk_heads, dim, vdim), dtype=torch.float32, device=q.device)
    _check(library().ems_delta_recurrence(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), beta.data_ptr(),
        beta.stride(0), _dt(q), MEMORY_INPUT_ACTIVATIONS[act], 0 if unit_eps is None else 1, float(unit_eps or 0.0),
        float(q_scale), _f32(g_raw, "g_raw"), _ptr(g_bias, "g_bias"), _ptr(a_log, "a_log"), _dt(a_log),
        _ptr(state, "state"), _i32(slots, "slots"), _i32(cu_q, "cu_q"), num_rows, n, num_heads, qk_heads, dim, vdim,
        _ptr(out, "out"), _f32(work, "work"), work.numel(), _stream()), "delta_recurrence", 2)


def delta_work_floats(num_tokens: int, num_heads: int, qk_heads: int, dim: int, vdim: int) -> int:
    """Elements of the float32 work buffer that `delta_recurrence` needs for `num_tokens` tokens."""
    return int(library().ems_delta_work_floats(num_tokens, num_heads, qk_heads, dim, vdim))


def ssm_gates(x: torch.Tensor, bias: torch.Tensor, a_log: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> None:
    """dt = softplus(x[t, h] + bias[h]); a[t, h] = exp(-exp(a_log[h]) * dt); b[t, h] = dt (float32 [N, H]).
    x: [N, H], may be a column range of a wider buffer."""
    n, h = x.shape
    assert x.stride(1) == 1 and a.shape == b.shape == (n, h) and a.dtype == b.dtype == torch.float32
    assert a.is_contiguous() and b.is_contiguous() and bias.numel() == a_log.numel() == h and bias.dtype == a_log.dtype
    if not x.is_cuda:
        raise KernelError("x must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_ssm_gates(x.data_ptr(), x.stride(0), _dt(x), _ptr(bias, "bias"), _ptr(a_log, "a_log"),
                                   _dt(a_log), _f32(a, "a"), _f32(b, "b"), n, h, _stream()), "ssm_gates")


def gate_group_norm(o: torch.Tensor, groups: int, eps: float, weight: torch.Tensor, out: torch.Tensor,
                    z: torch.Tensor | None = None, skip: torch.Tensor | None = None, x: torch.Tensor | None = None,
                    x_act: str = "none", head_width: int | None = None) -> None:
    """y = (o + skip[h] * act(x)) * silu(z); out = y / rms_g(y) * weight: the gate comes BEFORE the norm.
    o: float32 [N, C]; x, z: [N, >= C] of out's type (column ranges are fine); skip: [C / head_width] of
    weight's type, head h owning the columns [h * head_width, (h + 1) * head_width); each of `groups` equal
    consecutive parts of a row is divided by its own root mean square.  z and skip are optional."""
    n, c = o.shape
    hv = int(head_width or c)
    assert o.dtype == torch.float32 and o.is_contiguous() and out.shape == (n, c) and weight.numel() == c
    assert z is None or (z.dtype == out.dtype and z.stride(1) == 1 and z.shape[1] >= c)
    assert skip is None or (x is not None and x.dtype == out.dtype and x.stride(1) == 1 and x.shape[1] >= c
                            and skip.dtype == weight.dtype and skip.numel() * hv == c)
    if not o.is_cuda:
        raise KernelError("o must be a CUDA tensor (emberserve_b200 has no CPU path)")
    _check(library().ems_gate_group_norm(
        _f32(o, "o"), None if x is None else x.data_ptr(), 0 if x is None else x.stride(0),
        MEMORY_INPUT_ACTIVATIONS[x_act], _ptr(skip, "skip"), None if z is None else z.data_ptr(),
        0 if z is None else z.stride(0), _ptr(weight, "weight"), _dt(weight), _ptr(out, "out"), _dt(out), n, c,
        groups, hv, float(eps), _stream()), "gate_group_norm")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the maximum of logits[r]."""
    r, v = logits.shape
    assert logits.dtype == torch.float32
    slices = library().ems_argmax_slices(r, v)
    tmp = torch.empty(r * slices, dtype=torch.int64, device=logits.device) if slices else None
    _check(library().ems_argmax(_ptr(logits, "logits"), _i32(out, "out"), r, v, _ptr(tmp, "tmp"), _stream()),
           "argmax", 2 if slices else 1)


def repetition_penalty(logits: torch.Tensor, row_ptr: torch.Tensor, token_ids: torch.Tensor,
                       penalty: torch.Tensor) -> None:
    r, v = logits.shape
    assert logits.dtype == torch.float32 and penalty.dtype == torch.float32
    _check(library().ems_repetition_penalty(_ptr(logits, "logits"), r, v, _i32(row_ptr, "row_ptr"),
                                            _i32(token_ids, "token_ids"), _ptr(penalty, "penalty"),
                                            _stream()), "repetition_penalty")


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, seeds: torch.Tensor, counters: torch.Tensor,
           out: torch.Tensor) -> None:
    """One token per row: argmax where temperature == 0, else a seeded draw."""
    r, v = logits.shape
    assert logits.dtype == torch.float32 and temperature.dtype == torch.float32
    assert top_p.dtype == torch.float32 and seeds.dtype == torch.int64 and counters.dtype == torch.int64
    _check(library().ems_sample(_ptr(logits, "logits"), r, v, _ptr(temperature, "temperature"),
                                _i32(top_k, "top_k"), _ptr(top_p, "top_p"), _ptr(seeds, "seeds"),
                                _ptr(counters, "counters"), _i32(out, "out"), _stream()), "sample")


GEMM_SMALLM_MAX_ROWS = 64


# Rows of a step up to which the small-row products can take a norm into their epilogues.
GEMM_NORM_ROWS = 16


@dataclass
class NormBehind:
    """The norm that stands behind a small-row product, begun in the product's epilogue: the
    product is added into `residual` (float32 [m, n], in place) instead of being stored,
    `scaled` (bfloat16 [m, n]) receives residual * gain, and `sumsq` (float32 [parts, 16],
    parts = row tiles * ksplit of the product) every block's share of each row's sum of squares."""

    residual: torch.Tensor
    gain: torch.Tensor
    scaled: torch.Tensor
    sumsq: torch.Tensor


@dataclass
class NormBefore:
    """The norm that stands before a small-row product, finished in its epilogue: the product
    was given residual * gain, and row n of its result is multiplied by
    1 / sqrt(sumsq[:parts, n].sum() / width + eps) before the bias is added."""

    sumsq: torch.Tensor
    parts: int
    width: int
    eps: float


def _norm_before_args(nb: "NormBefore | None", m: int) -> tuple:
    if nb is None:
        return (None, 0, 0, 0.0)
    assert nb.sumsq.dtype == torch.float32 and nb.sumsq.numel() >= nb.parts * GEMM_NORM_ROWS and m <= GEMM_NORM_ROWS
    return (_ptr(nb.sumsq, "sumsq"), nb.parts, nb.width, float(nb.eps))


def tile_weight_shape_ok(weight: torch.Tensor) -> bool:
    """Whether `tile_weight` has a tiled form for this weight."""
    return (weight.dim() == 2 and weight.dtype == torch.bfloat16 and weight.is_cuda and weight.is_contiguous()
            and weight.shape[0] % 128 == 0 and weight.shape[1] % 64 == 0)


def tile_weight(weight: torch.Tensor) -> torch.Tensor | None:
    """The tiled copy of a bfloat16 weight [n, k] that the weight-streaming kernels read faster: the
    128 x 64 tile (row tile r, K tile kt) as 16 KB of contiguous memory at tile index
    r * (k / 64) + kt, so that one TMA load reads whole DRAM pages instead of 128 bytes from each of
    128 rows (7B shape: gate / up product 45.1 -> 43.9 us, down 25.2 -> 24.5, the decode step at
    batch 8 2.90 -> 2.82 ms).  None where n or k is no multiple of 128 / 64.  The copy has the
    shape [n * k / 64, 64]; it is passed as `twin` beside the weight it was made of."""
    if not tile_weight_shape_ok(weight):
        return None
    n, k = weight.shape
    return weight.view(n // 128, 128, k // 64, 64).permute(0, 2, 1, 3).contiguous().view(n * (k // 64), 64)


def _weight_ptr(weight: torch.Tensor, twin: torch.Tensor | None) -> tuple[int | None, int]:
    if twin is None:
        return _ptr(weight, "weight"), 0
    n, k = weight.shape
    assert twin.dtype == weight.dtype and twin.shape == (n * (k // 64), 64) and n % 128 == 0 and k % 64 == 0
    assert twin.is_contiguous()
    return _ptr(twin, "twin"), 1


def gemm_smallm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor | None,
                ksplit: int = 1, norm_behind: NormBehind | None = None,
                norm_before: NormBefore | None = None, twin: torch.Tensor | None = None) -> None:
    """out[m, n] = x[m, :] . weight[n, :] (+ bias[n]) in bfloat16 with float32 accumulation, for
    m <= 64 rows: the weight-streaming tcgen05 kernel.  `ksplit` blocks (up to 8) share K: they
    form a thread-block cluster and add their accumulators on chip, in rank order.  With
    `norm_behind` the product joins the residual stream in the epilogue (`out` is not written and
    may be None); with `norm_before` its rows are scaled there (m <= 16 for both)."""
    m, k = x.shape
    n = weight.shape[0]
    assert weight.shape[1] == k and (out is None or out.shape == (m, n))
    assert x.dtype == weight.dtype == torch.bfloat16
    # (a float32 `out` takes the sums unrounded: only where one block holds the whole sum)
    f32 = out is not None and out.dtype == torch.float32
    assert out is None or out.dtype == torch.bfloat16 or (f32 and ksplit == 1 and norm_behind is None)
    assert bias is None or (bias.dtype == torch.bfloat16 and bias.numel() == n)
    behind = (None, None, None, None)
    if norm_behind is not None:
        nb = norm_behind
        parts = -(-n // 128) * ksplit
        assert m <= GEMM_NORM_ROWS and nb.residual.dtype == torch.float32 and nb.residual.shape == (m, n)
        assert nb.gain.dtype == torch.bfloat16 and nb.gain.numel() == n
        assert nb.scaled.dtype == torch.bfloat16 and nb.scaled.shape == (m, n)
        assert nb.sumsq.dtype == torch.float32 and nb.sumsq.numel() >= parts * GEMM_NORM_ROWS
        behind = (_ptr(nb.residual, "residual"), _ptr(nb.gain, "gain"), _ptr(nb.scaled, "scaled"),
                  _ptr(nb.sumsq, "sumsq"))
    else:
        assert out is not None
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_smallm(
        _ptr(x, "x"), wptr, _ptr(bias, "bias"), _ptr(out, "out"), m, n, k, ksplit,
        *behind, *_norm_before_args(norm_before, m), tiled, 1 if f32 else 0, _stream()), "gemm_smallm")


GEMM_MIDM_ROWS = 128
_midm_clusters: dict[tuple[int, int, int], int] = {}


def gemm_midm_max_clusters(m: int, ksplit: int, device: "torch.device | None" = None) -> int:
    """How many clusters of `ksplit` blocks of the kernel for `m` rows (one block per SM) the device
    holds at once; a cluster lives inside one of the GPU's processing clusters, so this is less than
    SMs // ksplit (a B200 holds 148, 74, 45, 33, 26, 22, 15, 15 for 1..8).  Asked once per size."""
    nt = 32 if m <= 32 else (64 if m <= 64 else 128)
    idx = -1 if device is None or device.index is None else device.index
    key = (idx, nt, ksplit)
    n = _midm_clusters.get(key)
    if n is None:
        n = int(library().ems_gemm_midm_max_clusters(nt, ksplit))
        if n < 0:
            raise KernelError(f"gemm_midm: the occupancy of clusters of {ksplit} could not be asked")
        _midm_clusters[key] = n
    return n


def gemm_midm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, out: torch.Tensor,
              ksplit: int = 1, twin: torch.Tensor | None = None) -> None:
    """out[m, n] = x[m, k] @ weight[n, k].T (+ bias) in bfloat16 for up to 128 rows: the tcgen05
    kernel with one block per SM and a deep ring.  `ksplit` (1..8) blocks share K as a cluster;
    the caller picks it so that all blocks start in one wave."""
    m, k = x.shape
    n = weight.shape[0]
    assert x.dtype == weight.dtype == out.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
    assert x.is_contiguous() and weight.is_contiguous() and out.is_contiguous()
    assert weight.shape[1] == k and out.shape == (m, n)
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_midm(_ptr(x, "x"), wptr, _ptr(bias, "bias"), _ptr(out, "out"),
                                   m, n, k, ksplit, tiled, _stream()), "gemm_midm")


def gemm_smallm_gated(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                      norm_before: NormBefore | None = None, twin: torch.Tensor | None = None) -> None:
    """out[m, i] = silu(x . weight[i]) * (x . weight[I + i]) for weight [2 I, K]: gate and up
    projections of a gated feed-forward and its activation in one tcgen05 kernel, m <= 64.  With
    `norm_before` (m <= 16) both projections' rows are scaled first, as in `gemm_smallm`."""
    m, k = x.shape
    inter = out.shape[1]
    assert weight.shape == (2 * inter, k) and out.shape[0] == m
    assert x.dtype == weight.dtype == out.dtype == torch.bfloat16
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_smallm_gated(_ptr(x, "x"), wptr, _ptr(out, "out"), m, inter, k,
                                           *_norm_before_args(norm_before, m), tiled, _stream()), "gemm_smallm_gated")


def gemm_large_gated_supported(m: int, inter: int, k: int) -> bool:
    """Whether gemm_large_gated takes these sizes (bfloat16 tensors)."""
    return bool(library().ems_gemm_large_gated_supported(m, inter, k))


def gemm_large_gated(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                     twin: torch.Tensor | None = None) -> None:
    """out[m, i] = silu(x . weight[i]) * (x . weight[I + i]) for weight [2 I, K] and any number
    of rows m: the two-SM tcgen05 kernel of prompt steps (256 x 256 tiles, persistent grid), with
    the activation in its epilogue.  I a multiple of 128, K a multiple of 8."""
    m, k = x.shape
    inter = out.shape[1]
    assert weight.shape == (2 * inter, k) and out.shape[0] == m
    assert x.dtype == weight.dtype == out.dtype == torch.bfloat16
    wptr, tiled = _weight_ptr(weight, twin)
    _check(library().ems_gemm_large_gated(_ptr(x, "x"), wptr, _ptr(out, "out"), m, inter, k, tiled,
                                          _stream()), "gemm_large_gated")


def gemm_smallm_status() -> int:
    """0, or the code of the first bounded wait that ran out in the tcgen05 kernel (after a
    synchronisation point): 1 producer, 2 MMA issuer, 3 epilogue, 4 drain, 5 arrival of the split-K
    partials of the small-row kernel;
    11 producer, 12 and 13 MMA issuer, 14 epilogue of the two-SM kernel; 31 producer, 32 MMA issuer,
    33 epilogue, 34 drain, 35 arrival of the partials of the kernel for 17..128 rows; 20 and up: the
    prompt attention."""
    return int(library().ems_gemm_smallm_status())


def clear_status() -> None:
    """Set the status word of the tcgen05 kernels back to 0 (after the device has been waited for)."""
    library().ems_tc_status_clear()


def check_status(clear: bool = True) -> None:
    """Raise if a bounded wait inside a tcgen05 kernel (a GEMM or the prompt attention) ran out
    since the word was last cleared: what that kernel wrote is invalid, and so is everything
    computed from it.  The word lives in host-mapped memory, so the check costs no CUDA call; it
    means something only after a synchronisation point behind the kernels in question.  With
    `clear` the word is reset, so that the next step starts clean."""
    code = gemm_smallm_status()
    if code != 0:
        if clear:
            clear_status()
        raise KernelError(f"a wait inside a tcgen05 kernel ran out (code {code}); the results of the "
                          f"step are invalid")
