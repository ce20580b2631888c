"""Python face of the CUDA kernels: checks tensors, passes pointers and the
current stream to the ``extern "C"`` launchers, and raises on a refusal.

Nothing here computes on the host and nothing falls back: a CPU tensor or a
missing library is an error.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc.build import load_library

IE_F32, IE_BF16 = 0, 1
_CODES = {torch.float32: IE_F32, torch.bfloat16: IE_BF16}
_ERRORS = {-1: "unsupported dtype combination", -2: "unsupported size", -3: "misaligned pointer or stride",
           -4: "size beyond the kernel's static limit"}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 and bfloat16, not {dtype}") from None


LAUNCHES = 0     # launchers called so far (graph replays add what their capture counted)

# Extra -D flags per library ("core", "stream", "tcgen05", "attn_tcgen05", "attn_mma"), read when a library is first
# loaded.  Empty in the product; a measurement or a test that wants a variant (clock notes, no programmatic
# dependent launch, a short spin limit) fills it before the first call or passes ``defines`` to the loader itself.
BUILD_DEFINES: dict[str, dict] = {}


def _check(status: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if status == 0:
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_ERRORS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernels run on CUDA tensors only; there is no CPU path")
    return t.data_ptr()


def _stream() -> int:
    # the raw handle of the current stream of the current device, without building a Stream object: a step makes
    # a hundred launches, and the object cost more host time than everything else around a launch
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_core = None


def core():
    global _core
    if _core is None:
        lib = load_library("core", defines=dict(BUILD_DEFINES.get("core", {})))
        P, I, F, L = c_void_p, c_int, c_float, c_longlong
        lib.ie_embed_gather.argtypes = [P, P, I, P, I, I, I, P]
        lib.ie_patch_tokens.argtypes = [P, P, P, I, P]
        lib.ie_patch_tokens.restype = c_int
        lib.ie_stamp.argtypes = [P, P]
        lib.ie_stamp.restype = c_int
        lib.ie_rmsnorm.argtypes = [P, P, P, I, P, I, P, I, I, F, P]
        lib.ie_residual_add.argtypes = [P, P, I, I, I, P]
        lib.ie_rope_kv_write.argtypes = [P, P, P, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I, P]
        lib.ie_silu_mul.argtypes = [P, P, I, I, I, I, I, P]
        lib.ie_attention_general.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, P, I, I, F, I, I, I, P, P]
        lib.ie_layernorm.argtypes = [P, P, P, P, I, P, I, P, I, I, F, P]
        lib.ie_embed_bigram.argtypes = [P, P, P, P, I, P, P, I, P, P, I, I, I, I, L, L, P]
        lib.ie_add_bias.argtypes = [P, I, P, I, I, I, I, P]
        lib.ie_tanh.argtypes = [P, P, I, I, I, I, P]
        lib.ie_polynorm.argtypes = [P, P, P, I, P, I, I, I, I, F, P]
        lib.ie_headnorm_kv_write.argtypes = [P, P, P, I, I, I, P, P, I, F, P, P, P, I, I, I, I, I, I, I, I, P]
        lib.ie_gemm_simt.argtypes = [P, I, P, I, P, I, I, I, I, I, I, I, P]
        lib.ie_gemm_simt_batched.argtypes = [P, I, P, I, P, I, I, I, I, I, I, I, I, L, L, L, P]
        lib.ie_gemm_rowdot.argtypes = [P, I, P, I, P, I, I, I, I, I, I, P]
        lib.ie_cast_rows.argtypes = [P, P, I, I, I, P]
        lib.ie_outnorm_accumulate.argtypes = [P, P, I, I, P, I, P, I, I, I, F, P]
        lib.ie_outnorm_accumulate_norm.argtypes = [P, P, I, I, P, I, F, P, I, F, P, I, I, I, P]
        lib.ie_outnorm_accumulate_norm.restype = c_int
        lib.ie_causal_conv.argtypes = [P, I, P, P, I, P, L, P, I, P, P, I, I, I, I, I, I, I, P]
        lib.ie_attention_rows.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, I, P, I, P, I, I, F, I, I, I, P, P]
        lib.ie_linear_recurrence.argtypes = [P, I, P, I, P, P, I, P, P, P, I, P, P, I, P, P, I, I, F, F, I, I, P]
        lib.ie_rownorm_rotate_write.argtypes = [P, P, P, I, I, I, P, P, P, P, P, I, F, P, I, P, P, P, P, I, I, I, I, I, I, I, P]
        lib.ie_moe_route.argtypes = [P, I, P, I, P, P, P, I, I, I, I, I, F, F, I, I, P]
        lib.ie_moe_sort.argtypes = [P, I, I, I, P, P, I, P]
        lib.ie_moe_gemm.argtypes = [P, I, P, I, P, I, P, P, I, I, I, I, I, L, I, I, I, I, P]
        lib.ie_moe_combine.argtypes = [P, P, P, P, I, I, P, I, I, I, P]
        lib.ie_moe_tile_rows.restype = c_int
        lib.ie_head_prepare.argtypes = [P, I, I, I, I, I, P, P, I, I, I, I, I, P, I, P, I, I, I, F, P, I, I, F, P, P, P, P, I, I, I, P]
        lib.ie_heads_gemm.argtypes = [P, I, I, I, P, I, P, I, I, I, I, I, I, I, P]
        lib.ie_diff_combine.argtypes = [P, I, P, I, P, I, I, I, I, I, F, F, F, I, P]
        lib.ie_gated_residual_add.argtypes = [P, P, I, P, I, P, I, I, I, I, P]
        lib.ie_scale_rows.argtypes = [P, P, F, I, I, P]
        lib.ie_glu_act.argtypes = [P, P, I, I, I, I, I, F, F, F, I, P]
        lib.ie_mingru_scan.argtypes = [P, P, I, P, I, P, P, I, P, P, I, P, P, I, I, I, I, P]
        lib.ie_mingru_scan_hint.argtypes = [P, P, I, P, I, P, P, I, P, P, I, P, P, I, I, I, I, I, P]
        D = ctypes.c_double
        lib.ie_scale_add_sinusoid.argtypes = [P, P, F, D, I, I, P]
        lib.ie_add_row.argtypes = [P, P, I, I, I, P]
        lib.ie_token_shift.argtypes = [P, P, I, P, I, P, P, P, P, I, I, I, I, P]
        lib.ie_gate_mul.argtypes = [P, I, P, I, I, I, I, I, P]
        lib.ie_qkv_prepare.argtypes = [P, I, I, P, I, P, I, I, P, I, I, P, I, I, I, P, I, I, F, P, P, P, I, I, I, I, P]
        lib.ie_talk_combine.argtypes = [P, I, P, P, I, P, I, I, I, I, I, I, I, I, P]
        lib.ie_mlstm_scan.argtypes = [P, P, P, I, I, I, P, P, I, P, P, I, F, F, P, L, P, I, P, P, I, I, I, I, I, I, P]
        lib.ie_mlstm_finish.argtypes = [P, I, P, I, P, I, P, I, I, I, I, F, I, P]
        lib.ie_mlstm_chunks.argtypes = [I, I]
        lib.ie_mlstm_state_floats.argtypes = [I, I]
        lib.ie_mlstm_state_floats.restype = c_longlong
        lib.ie_argmax.argtypes = [P, P, I, I, L, P]
        lib.ie_repetition_penalty.argtypes = [P, P, P, I, I, L, I, P]
        lib.ie_sample.argtypes = [P, P, P, I, I, L, P]
        for name in ("ie_embed_gather", "ie_rmsnorm", "ie_residual_add", "ie_rope_kv_write", "ie_silu_mul",
                     "ie_attention_general", "ie_gemm_simt", "ie_argmax", "ie_repetition_penalty", "ie_sample",
                     "ie_layernorm", "ie_embed_bigram", "ie_add_bias", "ie_tanh", "ie_polynorm",
                     "ie_headnorm_kv_write", "ie_gemm_simt_batched", "ie_cast_rows", "ie_outnorm_accumulate",
                     "ie_causal_conv", "ie_linear_recurrence", "ie_rownorm_rotate_write", "ie_moe_route", "ie_moe_sort",
                     "ie_moe_gemm", "ie_moe_combine", "ie_attention_rows", "ie_gemm_rowdot", "ie_head_prepare",
                     "ie_heads_gemm", "ie_diff_combine", "ie_gated_residual_add", "ie_scale_rows", "ie_glu_act",
                     "ie_mingru_scan", "ie_mingru_scan_hint", "ie_scale_add_sinusoid", "ie_add_row", "ie_token_shift",
                     "ie_gate_mul", "ie_qkv_prepare", "ie_talk_combine", "ie_mlstm_scan", "ie_mlstm_finish",
                     "ie_mlstm_chunks"):
            getattr(lib, name).restype = c_int
        _core = lib
        _apply_check_limits()
    return _core


# ------------------------------------------------------------------ elementwise
def embed_gather(ids: torch.Tensor, table: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[n] = table[ids[n]] as float32."""
    assert ids.dtype == torch.int32 and residual.dtype == torch.float32 and table.is_contiguous()
    n, d = residual.shape
    _check(core().ie_embed_gather(_ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(residual), n, d,
                                  table.shape[0], _stream()), "embed_gather")


def embed_bigram(ids: torch.Tensor, positions: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor,
                 n_requests: int, table: torch.Tensor, bigram: torch.Tensor, prev_state: torch.Tensor,
                 residual: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int) -> None:
    """residual[n] = table[ids[n]] + bigram[row] as float32, row = (previous token * mul_prev + ids[n] * mul_cur) mod
    buckets, or ``buckets`` (the last row) at position 0.  ``prev_state`` (int32, one word per request slot) holds the
    last token of every request between steps; this call reads and updates it."""
    assert ids.dtype == positions.dtype == q_start.dtype == slots.dtype == prev_state.dtype == torch.int32
    assert residual.dtype == torch.float32 and table.is_contiguous() and bigram.is_contiguous()
    assert table.dtype == bigram.dtype and bigram.shape == (buckets + 1, table.shape[1]) and prev_state.is_contiguous()
    n, d = residual.shape
    _check(core().ie_embed_bigram(_ptr(ids), _ptr(positions), _ptr(q_start), _ptr(slots), n_requests, _ptr(table),
                                  _ptr(bigram), dtype_code(table.dtype), _ptr(prev_state), _ptr(residual), n, d,
                                  table.shape[0], int(buckets), int(mul_prev), int(mul_cur), _stream()), "embed_bigram")


def patch_tokens(ids: torch.Tensor, src: torch.Tensor, prev: torch.Tensor) -> None:
    """ids[i] = prev[src[i]] where src[i] >= 0 (token ids that are still on the device)."""
    assert ids.dtype == src.dtype == prev.dtype == torch.int32 and src.shape[0] >= ids.shape[0]
    _check(core().ie_patch_tokens(_ptr(ids), _ptr(src), _ptr(prev), ids.shape[0], _stream()), "patch_tokens")


def stamp(slots: torch.Tensor, index: int) -> None:
    """slots[index] = the GPU's nanosecond clock once everything enqueued before has finished (int64 tensor);
    for timelines of a step.  Not counted as a launch of the step."""
    global LAUNCHES
    assert slots.dtype is torch.int64 and 0 <= index < slots.numel()
    _check(core().ie_stamp(slots.data_ptr() + 8 * index, _stream()), "stamp")
    LAUNCHES -= 1


def rmsnorm(residual: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, out: torch.Tensor,
            eps: float, row_index: torch.Tensor | None = None) -> None:
    """out = rmsnorm(residual (+ delta)) * gain; residual takes the sum unless rows are gathered."""
    d = residual.shape[-1]
    n_rows = out.shape[0]
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape)
    assert gain.shape == (d,) and out.shape[1] == d
    _check(core().ie_rmsnorm(_ptr(residual), _ptr(delta), _ptr(gain), dtype_code(gain.dtype), _ptr(out),
                             dtype_code(out.dtype), _ptr(row_index), n_rows, d, float(eps), _stream()), "rmsnorm")


def layernorm(residual: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None,
              out: torch.Tensor, eps: float, row_index: torch.Tensor | None = None) -> None:
    """out = (x - mean) / sqrt(var + eps) * weight + bias with x = residual (+ delta); residual takes the sum unless
    rows are gathered."""
    d = residual.shape[-1]
    n_rows = out.shape[0]
    assert residual.dtype == torch.float32 and residual.is_contiguous() and out.is_contiguous()
    assert delta is None or (delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape)
    assert weight.shape == (d,) and out.shape[1] == d and (bias is None or (bias.shape == (d,) and bias.dtype == weight.dtype))
    _check(core().ie_layernorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(bias), dtype_code(weight.dtype),
                               _ptr(out), dtype_code(out.dtype), _ptr(row_index), n_rows, d, float(eps), _stream()),
           "layernorm")


def add_bias(out: torch.Tensor, bias: torch.Tensor) -> None:
    """out[n, :] += bias (out may be a column slice)."""
    n, cols = out.shape
    assert out.stride(1) == 1 and bias.shape == (cols,) and bias.is_contiguous()
    _check(core().ie_add_bias(_ptr(out), dtype_code(out.dtype), _ptr(bias), dtype_code(bias.dtype), n, cols,
                              out.stride(0), _stream()), "add_bias")


def tanh(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = tanh(x); x may be a column slice, out is contiguous."""
    n, cols = x.shape
    assert x.stride(1) == 1 and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype
    _check(core().ie_tanh(_ptr(x), _ptr(out), n, cols, x.stride(0), dtype_code(x.dtype), _stream()), "tanh")


def polynorm(z: torch.Tensor, bias: torch.Tensor | None, coef: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out = c0 N(y) + c1 N(y^2) + c2 N(y^3) + c3 with y = z (+ bias) and N(x) = x / sqrt(mean(x^2) + eps) over a row;
    ``coef`` holds the four numbers on the device."""
    n, cols = z.shape
    assert z.stride(1) == 1 and out.is_contiguous() and out.shape == z.shape and out.dtype == z.dtype
    assert coef.shape == (4,) and (bias is None or (bias.shape == (cols,) and bias.dtype == coef.dtype))
    _check(core().ie_polynorm(_ptr(z), _ptr(bias), _ptr(coef), dtype_code(coef.dtype), _ptr(out), dtype_code(out.dtype),
                              n, cols, z.stride(0), float(eps), _stream()), "polynorm")


def headnorm_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_gain: torch.Tensor | None,
                      k_gain: torch.Tensor | None, eps: float, slot_mapping: torch.Tensor | None,
                      kpool: torch.Tensor | None, vpool: torch.Tensor | None, n_heads: int, n_kv_heads: int,
                      head_dim: int, v_head_dim: int, page_size: int) -> None:
    """RMS norm of every query head (in place) and key head with gains of the head's size shared by all heads
    (None: no norm on that side); the normalised keys and the raw values go to their page slots (if pools are given).
    q, k, v are row-strided views [n, heads * head size]; values have ``v_head_dim`` elements a head."""
    n = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1
    gain = q_gain if q_gain is not None else k_gain
    assert q_gain is None or k_gain is None or q_gain.dtype == k_gain.dtype
    write = kpool is not None
    _check(core().ie_headnorm_kv_write(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(q_gain),
                                       _ptr(k_gain), dtype_code(gain.dtype) if gain is not None else IE_F32, float(eps),
                                       _ptr(slot_mapping), _ptr(kpool), _ptr(vpool), n, n_heads, n_kv_heads, head_dim,
                                       v_head_dim, page_size, 1 if write else 0, dtype_code(q.dtype), _stream()),
           "headnorm_kv_write")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    n, d = residual.shape
    _check(core().ie_residual_add(_ptr(residual), _ptr(delta), dtype_code(delta.dtype), n, d, _stream()),
           "residual_add")


def rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor | None,
                  sin: torch.Tensor | None, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                  kpool: torch.Tensor | None, vpool: torch.Tensor | None, n_heads: int, n_kv_heads: int,
                  head_dim: int, page_size: int, rotate_q: bool = True) -> None:
    """Rotate q in place (unless ``rotate_q`` is off: the attention kernel then rotates it as it reads it);
    write rotated k and raw v into their page slots (if pools are given).

    q, k, v are row-strided views [n, heads*head_dim] (columns of one fused buffer, for instance).
    """
    n = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and k.stride(0) == v.stride(0)
    write = kpool is not None
    _check(core().ie_rope_kv_write(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), _ptr(cos), _ptr(sin),
                                   _ptr(positions), _ptr(slot_mapping), _ptr(kpool), _ptr(vpool), n, n_heads,
                                   n_kv_heads, head_dim, page_size, (1 if write else 0) | (0 if rotate_q else 2),
                                   dtype_code(q.dtype),
                                   _stream()), "rope_kv_write")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out[n, j] = silu(gate_j) * up_j; gate and up are the two halves of a row, or alternate when ``interleaved``."""
    n, inter = out.shape
    assert gate_up.shape == (n, 2 * inter) and gate_up.stride(1) == 1 and out.is_contiguous()
    _check(core().ie_silu_mul(_ptr(gate_up), _ptr(out), n, inter, gate_up.stride(0), 1 if interleaved else 0,
                              dtype_code(out.dtype), _stream()), "silu_mul")


# --------------------------------------------------------------------- attention
def attention_general(q: torch.Tensor, out: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor,
                      block_table: torch.Tensor, q_start: torch.Tensor, ctx_before: torch.Tensor,
                      work_req: torch.Tensor, work_pair0: torch.Tensor, n_work: int, n_heads: int,
                      n_kv_heads: int, head_dim: int, page_size: int, window: int | None, scale: float,
                      score_bias: torch.Tensor | None = None, head_scale: torch.Tensor | None = None,
                      v_head_dim: int | None = None, keep_first: int = 0, out_scale: float = 1.0, chunk: int = 0,
                      n_v_heads: int | None = None, v_row: int | None = None, sink: torch.Tensor | None = None) -> None:
    """Paged causal attention in float32 arithmetic.  ``score_bias`` (float32 [n_heads, D], contiguous) is added to
    the scaled score of a query at position p and a key at position j as ``score_bias[head, min(p - j, D - 1)]``.
    ``head_scale`` (float32 [n_heads]) multiplies the score of its head beside ``scale``.  ``v_head_dim``: head size of
    the values and of ``out`` when it is not ``head_dim``.  ``keep_first``: beside a window, keys at positions below it
    stay visible to every later query.  ``out_scale`` multiplies the output.  ``chunk``: a query sees only the keys of
    its own chunk of that many positions.  ``n_v_heads``: heads of the value pool when several key heads share a value
    head; ``v_row``: elements between value rows when the values are the first dimensions of the key rows (one pool).
    ``sink`` (float32 [n_heads]): the softmax's denominator of head h also holds exp(sink[h]), a term without a key or
    a value that ``scale`` does not touch."""
    assert sink is None or (sink.dtype is torch.float32 and sink.is_contiguous() and sink.shape == (n_heads,))
    assert q.stride(1) == 1 and out.stride(1) == 1 and kpool.dtype == q.dtype == out.dtype
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    if score_bias is not None:
        assert score_bias.dtype is torch.float32 and score_bias.is_contiguous() and score_bias.shape[0] == n_heads
    if head_scale is not None:
        assert head_scale.dtype is torch.float32 and head_scale.is_contiguous() and head_scale.shape == (n_heads,)
    _check(core().ie_attention_general(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table),
                                       _ptr(q_start), _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0),
                                       q.stride(0), out.stride(0), block_table.stride(0), n_work, n_heads,
                                       n_kv_heads, head_dim, page_size, int(window or 0), float(scale),
                                       dtype_code(q.dtype), _ptr(score_bias),
                                       score_bias.shape[1] if score_bias is not None else 0, _ptr(head_scale),
                                       int(v_head_dim or head_dim), int(keep_first or 0), float(out_scale),
                                       int(chunk or 0), int(n_v_heads or 0), int(v_row or 0), _ptr(sink), _stream()),
           f"attention_general(head_dim={head_dim}, heads={n_heads}/{n_kv_heads})")


def attention_rows(q: torch.Tensor, out: torch.Tensor, kpool: torch.Tensor, vpool: torch.Tensor, block_table: torch.Tensor,
                   q_start: torch.Tensor, ctx_before: torch.Tensor, n_requests: int, max_rows: int, n_heads: int,
                   n_kv_heads: int, head_dim: int, page_size: int, window: int | None, scale: float,
                   score_bias: torch.Tensor | None = None, head_scale: torch.Tensor | None = None,
                   v_head_dim: int | None = None, keep_first: int = 0, out_scale: float = 1.0, chunk: int = 0,
                   n_v_heads: int | None = None, v_row: int | None = None, sink: torch.Tensor | None = None) -> None:
    """``attention_general`` for the requests of the step that bring at most ``max_rows`` (token, head-in-group) rows
    (decode tokens, as a rule): a block per (token, query head) whose warps split the visible keys.  Rows of requests
    that bring more are left untouched (the tile kernel's, with a work list of those requests)."""
    assert q.stride(1) == 1 and out.stride(1) == 1 and kpool.dtype == q.dtype == out.dtype
    assert block_table.dtype == torch.int32 and block_table.stride(1) == 1
    if score_bias is not None:
        assert score_bias.dtype is torch.float32 and score_bias.is_contiguous() and score_bias.shape[0] == n_heads
    if head_scale is not None:
        assert head_scale.dtype is torch.float32 and head_scale.is_contiguous() and head_scale.shape == (n_heads,)
    _check(core().ie_attention_rows(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                    _ptr(ctx_before), q.stride(0), out.stride(0), block_table.stride(0), q.shape[0],
                                    n_requests, int(max_rows), n_heads, n_kv_heads, head_dim, page_size, int(window or 0),
                                    float(scale), dtype_code(q.dtype), _ptr(score_bias),
                                    score_bias.shape[1] if score_bias is not None else 0, _ptr(head_scale),
                                    int(v_head_dim or head_dim), int(keep_first or 0), float(out_scale),
                                    int(chunk or 0), int(n_v_heads or 0), int(v_row or 0), _ptr(sink), _stream()),
           f"attention_rows(head_dim={head_dim}, heads={n_heads}/{n_kv_heads})")


# -------------------------------------------------------------------------- gemm
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in float32 arithmetic."""
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().ie_gemm_simt(_ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(out),
                               dtype_code(out.dtype), m, n, k, a.stride(0), w.stride(0), out.stride(0),
                               _stream()), f"gemm_simt({a.dtype},{w.dtype}->{out.dtype})")


def gemm_rowdot(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M,N] = a[M,K] @ w[N,K]^T in float32 arithmetic for a few dozen outputs (a router): a block per row of ``a``, a
    warp per output."""
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n) and out.dtype is torch.float32
    assert a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _check(core().ie_gemm_rowdot(_ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(out), m, n, k, a.stride(0),
                                 w.stride(0), out.stride(0), _stream()), f"gemm_rowdot({a.dtype},{w.dtype})")


def gemm_simt_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """A block-diagonal matrix applied to rows, float32 products and sums: ``w`` is [blocks, n, k] (rows are outputs),
    ``a`` [m, blocks * k] and ``out`` float32 [m, blocks * n]; block b maps columns b*k.. of ``a`` to columns b*n.. of
    ``out``."""
    blocks, n, k = w.shape
    m = a.shape[0]
    assert a.shape[1] == blocks * k and out.shape == (m, blocks * n) and out.dtype is torch.float32
    assert a.stride(1) == 1 and w.is_contiguous() and out.stride(1) == 1
    _check(core().ie_gemm_simt_batched(_ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(out), IE_F32, m, n,
                                       k, a.stride(0), k, out.stride(0), blocks, k, n * k, n, _stream()),
           f"gemm_simt_batched({a.dtype},{w.dtype}, blocks={blocks})")


# ------------------------------------------------------------- norm on a sublayer's output, state along a sequence
def cast_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    """out = x (float32 rows) in out's type."""
    assert x.dtype is torch.float32 and x.is_contiguous() and out.is_contiguous() and out.shape == x.shape
    _check(core().ie_cast_rows(_ptr(x), _ptr(out), dtype_code(out.dtype), x.shape[0], x.shape[1], _stream()), "cast_rows")


def outnorm_accumulate(residual: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float,
                       next_in: torch.Tensor | None = None) -> None:
    """residual += y / sqrt(mean(y^2) + eps) * gain, row by row; ``next_in`` (optional, activation type) takes the new
    residual rows."""
    n, d = residual.shape
    assert residual.dtype is torch.float32 and residual.is_contiguous() and y.shape == (n, d) and y.stride(1) == 1
    assert gain.shape == (d,) and (next_in is None or (next_in.is_contiguous() and next_in.shape == (n, d)))
    _check(core().ie_outnorm_accumulate(_ptr(residual), _ptr(y), dtype_code(y.dtype), y.stride(0), _ptr(gain),
                                        dtype_code(gain.dtype), _ptr(next_in),
                                        dtype_code(next_in.dtype) if next_in is not None else IE_BF16, n, d, float(eps),
                                        _stream()), "outnorm_accumulate")


def outnorm_accumulate_norm(residual: torch.Tensor, y: torch.Tensor, gain: torch.Tensor, eps: float,
                            next_gain: torch.Tensor, next_eps: float, normed: torch.Tensor) -> None:
    """``outnorm_accumulate`` and, in the same kernel, the norm that the residual meets next:
    ``normed = x / sqrt(mean(x^2) + next_eps) * next_gain`` with x the new residual rows, in ``normed``'s type."""
    n, d = residual.shape
    assert residual.dtype is torch.float32 and residual.is_contiguous() and y.shape == (n, d) and y.stride(1) == 1
    assert gain.shape == (d,) and next_gain.shape == (d,) and gain.dtype == next_gain.dtype
    assert normed.is_contiguous() and normed.shape == (n, d)
    _check(core().ie_outnorm_accumulate_norm(_ptr(residual), _ptr(y), dtype_code(y.dtype), y.stride(0), _ptr(gain),
                                             dtype_code(gain.dtype), float(eps), _ptr(next_gain), dtype_code(next_gain.dtype),
                                             float(next_eps), _ptr(normed), dtype_code(normed.dtype), n, d, _stream()),
           "outnorm_accumulate_norm")


CONV_MAX_TAPS = 16


def causal_conv(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, state: torch.Tensor, out: torch.Tensor,
                q_start: torch.Tensor, slots: torch.Tensor, n_requests: int, activation: str | None = None,
                write_state: bool = True, max_q_len: int | None = None) -> None:
    """A causal convolution per channel over each request's tokens of the step: ``out[t, c] = act(bias[c] + sum_j
    weight[c, j] * x[t - (taps - 1 - j), c])``.  ``state`` [slots, taps - 1, channels] (activation type) holds every
    request's last inputs, oldest first, and is moved on by the step's tokens (with ``write_state``).  ``max_q_len``: the
    most tokens one request brings (the launch is cut for it; the step's token count when not given)."""
    n, channels = x.shape
    taps = weight.shape[1]
    assert weight.shape == (channels, taps) and weight.is_contiguous() and x.stride(1) == 1 and out.stride(1) == 1
    assert out.shape == (n, channels) and out.dtype == x.dtype and state.dtype == x.dtype and state.stride(-1) == 1
    assert state.shape[1:] == (max(taps - 1, 0), channels) and (taps == 1 or state.stride(1) == channels)
    assert bias is None or (bias.shape == (channels,) and bias.dtype == weight.dtype)
    assert out.data_ptr() != x.data_ptr(), "the convolution reads earlier rows of its input after writing its output"
    _check(core().ie_causal_conv(_ptr(x), x.stride(0), _ptr(weight), _ptr(bias), dtype_code(weight.dtype), _ptr(state),
                                 state.stride(0), _ptr(out), out.stride(0), _ptr(q_start), _ptr(slots), n_requests,
                                 channels, taps, {None: 0, "silu": 1}[activation], 1 if write_state else 0,
                                 dtype_code(x.dtype), int(max_q_len) if max_q_len else max(n, 1), _stream()),
           f"causal_conv(channels={channels}, taps={taps})")


def linear_recurrence(u: torch.Tensor, y_pre: torch.Tensor, r_pre: torch.Tensor, i_pre: torch.Tensor,
                      r_bias: torch.Tensor, i_bias: torch.Tensor, lam: torch.Tensor, state: torch.Tensor,
                      out: torch.Tensor, q_start: torch.Tensor, slots: torch.Tensor, n_requests: int,
                      decay_scale: float, out_scale: float = 1.0, write_state: bool = True) -> None:
    """The real-gated linear recurrent unit over each request's tokens of the step, per channel: r = sigmoid(r_pre +
    r_bias), i = sigmoid(i_pre + i_bias), a = exp(-decay_scale * r * softplus(lam)), S <- a S + sqrt(1 - a^2) i u,
    out = out_scale * S * gelu_tanh(y_pre).  ``r_pre``/``i_pre`` float32 (columns of one buffer), ``state`` float32
    [slots, width]."""
    n, width = u.shape
    assert u.stride(1) == 1 and y_pre.stride(1) == 1 and y_pre.dtype == u.dtype == out.dtype and out.stride(1) == 1
    assert r_pre.dtype is torch.float32 and i_pre.dtype is torch.float32 and r_pre.stride(0) == i_pre.stride(0)
    assert r_pre.stride(1) == 1 and i_pre.stride(1) == 1 and state.dtype is torch.float32 and state.is_contiguous()
    assert state.shape[1:] == (width,) and r_bias.dtype == i_bias.dtype == lam.dtype
    assert r_bias.shape == i_bias.shape == lam.shape == (width,)
    _check(core().ie_linear_recurrence(_ptr(u), u.stride(0), _ptr(y_pre), y_pre.stride(0), _ptr(r_pre), _ptr(i_pre),
                                       r_pre.stride(0), _ptr(r_bias), _ptr(i_bias), _ptr(lam), dtype_code(lam.dtype),
                                       _ptr(state), _ptr(out), out.stride(0), _ptr(q_start), _ptr(slots), n_requests,
                                       width, float(decay_scale), float(out_scale), 1 if write_state else 0,
                                       dtype_code(u.dtype), _stream()), f"linear_recurrence(width={width})")


def rownorm_rotate_write(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_bias, k_bias, v_bias, q_gain, k_gain,
                         eps: float, inv_freq: torch.Tensor | None, rot_dims: int, positions: torch.Tensor,
                         slot_mapping: torch.Tensor | None, kpool: torch.Tensor | None, vpool: torch.Tensor | None,
                         n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, page_size: int) -> None:
    """For every token: biases added to q, k, v; q and k divided by the root mean square of their WHOLE row and
    multiplied by gains of the row's size; the first ``rot_dims`` dimensions of every head of q and k turned in
    neighbouring pairs by position * inv_freq (float64 [rot_dims / 2]); q written back in place, k and v into their
    page slots (if pools are given).  Any of the biases and gains may be None (all given ones of one type)."""
    n = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and q.dtype == k.dtype == v.dtype
    given = [t for t in (q_bias, k_bias, v_bias, q_gain, k_gain) if t is not None]
    assert all(t.dtype == given[0].dtype and t.is_contiguous() for t in given)
    assert inv_freq is None or (inv_freq.dtype is torch.float64 and inv_freq.is_contiguous() and inv_freq.numel() * 2 >= rot_dims)
    _check(core().ie_rownorm_rotate_write(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(q_bias),
                                          _ptr(k_bias), _ptr(v_bias), _ptr(q_gain), _ptr(k_gain),
                                          dtype_code(given[0].dtype) if given else IE_F32, float(eps), _ptr(inv_freq),
                                          int(rot_dims), _ptr(positions), _ptr(slot_mapping), _ptr(kpool), _ptr(vpool), n,
                                          n_heads, n_kv_heads, head_dim, v_head_dim, page_size, dtype_code(q.dtype),
                                          _stream()), "rownorm_rotate_write")


# ------------------------------------------------------------------ heads before and after attention, gates
def head_prepare(q: torch.Tensor, q_heads: int, q_head_dim: int, k: torch.Tensor, k_heads: int, k_head_dim: int,
                 positions: torch.Tensor, slot_mapping: torch.Tensor | None, kpool: torch.Tensor | None, page_size: int,
                 q_gain: torch.Tensor | None = None, q_norm_dims: int = 0, k_gain: torch.Tensor | None = None,
                 k_norm_dims: int = 0, eps: float = 0.0, inv_freq: torch.Tensor | None = None, rot_dims: int = 0,
                 q_rot_off: int = 0, k_rot_off: int = 0, neighbours: bool = False, mult: float = 1.0,
                 v: torch.Tensor | None = None, vpool: torch.Tensor | None = None, n_v_heads: int = 0,
                 v_head_dim: int = 0) -> None:
    """Per token: an RMS norm over the first ``*_norm_dims`` dimensions of every query head and key head (gains of that
    size; None: no norm), a rotation by position of ``rot_dims`` dimensions that start at ``*_rot_off`` of every head
    (``inv_freq`` float64 [rot_dims / 2]; in halves, or in neighbouring pairs with ``neighbours``; sine and cosine times
    ``mult``); q is written back in place, the keys go to their slots of ``kpool`` [pages, k_heads, page_size,
    k_head_dim] and ``v`` (optional, as it is) to ``vpool`` [pages, n_v_heads, page_size, v_head_dim]."""
    n = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and q.dtype == k.dtype and (v is None or (v.stride(1) == 1 and v.dtype == q.dtype))
    gains = [g for g in (q_gain, k_gain) if g is not None]
    assert all(g.dtype == gains[0].dtype and g.is_contiguous() for g in gains)
    assert q_gain is None or q_gain.numel() >= q_norm_dims
    assert k_gain is None or k_gain.numel() >= k_norm_dims
    assert inv_freq is None or (inv_freq.dtype is torch.float64 and inv_freq.is_contiguous() and inv_freq.numel() * 2 >= rot_dims)
    assert kpool is None or kpool.dtype == q.dtype
    _check(core().ie_head_prepare(_ptr(q), q.stride(0), q_heads, q_head_dim, int(q_norm_dims if q_gain is not None else 0),
                                  int(q_rot_off), _ptr(q_gain), _ptr(k), k.stride(0), k_heads, k_head_dim,
                                  int(k_norm_dims if k_gain is not None else 0), int(k_rot_off), _ptr(k_gain),
                                  dtype_code(gains[0].dtype) if gains else IE_F32, _ptr(v),
                                  v.stride(0) if v is not None else 0, int(n_v_heads), int(v_head_dim), float(eps),
                                  _ptr(inv_freq), int(rot_dims if inv_freq is not None else 0), 1 if neighbours else 0,
                                  float(mult), _ptr(positions), _ptr(slot_mapping), _ptr(kpool), _ptr(vpool), n,
                                  page_size, dtype_code(q.dtype), _stream()), "head_prepare")


def heads_gemm(x: torch.Tensor, x_head: int, w: torch.Tensor, out: torch.Tensor, o_head: int) -> None:
    """A product per head in float32 arithmetic: ``out[m, h * o_head + j] = sum_k x[m, h * x_head + k] * w[h, k, j]`` for
    ``w`` [heads, K, N] (contiguous); ``x`` and ``out`` are rows with a stride, a head every ``x_head`` / ``o_head``
    elements."""
    H, K, N = w.shape
    m = x.shape[0]
    assert w.is_contiguous() and x.stride(1) == 1 and out.stride(1) == 1 and out.shape[0] == m
    assert (H - 1) * x_head + K <= x.shape[1] and (H - 1) * o_head + N <= out.shape[1]
    _check(core().ie_heads_gemm(_ptr(x), dtype_code(x.dtype), x.stride(0), int(x_head), _ptr(w), dtype_code(w.dtype),
                                _ptr(out), dtype_code(out.dtype), out.stride(0), int(o_head), m, H, K, N, _stream()),
           f"heads_gemm({x.dtype},{w.dtype}->{out.dtype}, heads={H}, k={K}, n={N})")


def diff_combine(maps: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                 v_head_dim: int, lam: float, eps: float, out_mult: float) -> None:
    """Two attention maps of every head become one output: ``o = a1 - lam * a2``, divided by its root mean square over
    the head (``eps`` inside the root), times ``out_mult`` and, if given, ``sigmoid(gate)``.  ``maps`` is [n, kv heads,
    2, heads of a group, v_head_dim] flattened; ``gate`` and ``out`` are [n, n_heads * v_head_dim]."""
    n = out.shape[0]
    assert maps.stride(1) == 1 and out.stride(1) == 1 and maps.dtype == out.dtype
    assert maps.shape[1] == 2 * n_heads * v_head_dim and out.shape[1] == n_heads * v_head_dim
    assert gate is None or (gate.stride(1) == 1 and gate.dtype == out.dtype and gate.shape == out.shape)
    _check(core().ie_diff_combine(_ptr(maps), maps.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                  _ptr(out), out.stride(0), n, n_heads, n_kv_heads, v_head_dim, float(lam), float(eps),
                                  float(out_mult), dtype_code(out.dtype), _stream()), "diff_combine")


def gated_residual_add(residual: torch.Tensor, y: torch.Tensor, gate_pre: torch.Tensor, bias: torch.Tensor | None) -> None:
    """residual (float32) += sigmoid(gate_pre + bias) * y, element by element; ``bias`` [d] or None."""
    n, d = residual.shape
    assert residual.dtype is torch.float32 and residual.is_contiguous()
    assert y.shape == (n, d) and gate_pre.shape == (n, d) and y.stride(1) == 1 and gate_pre.stride(1) == 1
    assert y.dtype == gate_pre.dtype and (bias is None or (bias.shape == (d,) and bias.is_contiguous()))
    _check(core().ie_gated_residual_add(_ptr(residual), _ptr(y), y.stride(0), _ptr(gate_pre), gate_pre.stride(0),
                                        _ptr(bias), dtype_code(bias.dtype) if bias is not None else IE_F32, n, d,
                                        dtype_code(y.dtype), _stream()), "gated_residual_add")


def scale_rows(x: torch.Tensor, scale: float, keep: torch.Tensor | None = None) -> None:
    """x (float32) *= scale; ``keep`` (float32, same shape) takes a copy of the result."""
    assert x.dtype is torch.float32 and x.is_contiguous()
    assert keep is None or (keep.dtype is torch.float32 and keep.is_contiguous() and keep.shape == x.shape)
    _check(core().ie_scale_rows(_ptr(x), _ptr(keep), float(scale), x.shape[0], x.shape[1], _stream()), "scale_rows")


GLU_KINDS = {"silu": 0, "clamped_swish": 1}


def glu_act(gate_up: torch.Tensor, out: torch.Tensor, kind: str, interleaved: bool = False, alpha: float = 1.0,
            limit: float = 0.0, up_offset: float = 0.0) -> None:
    """out[n, j] = act(gate_j) * (up_j + up_offset).  ``silu``: g sigmoid(g).  ``clamped_swish``: g' sigmoid(alpha g')
    with g' = min(g, limit), and up clamped to [-limit, limit].  Gate and up are the two halves of a row, or alternate
    when ``interleaved``."""
    n, inter = out.shape
    assert gate_up.shape == (n, 2 * inter) and gate_up.stride(1) == 1 and out.is_contiguous() and gate_up.dtype == out.dtype
    _check(core().ie_glu_act(_ptr(gate_up), _ptr(out), n, inter, gate_up.stride(0), 1 if interleaved else 0,
                             GLU_KINDS[kind], float(alpha), float(limit), float(up_offset), dtype_code(out.dtype),
                             _stream()), f"glu_act({kind})")


def mingru_scan(z_pre: torch.Tensor, u_pre: torch.Tensor, g_pre: torch.Tensor, z_bias: torch.Tensor | None,
                u_bias: torch.Tensor | None, state: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                slots: torch.Tensor, n_requests: int, write_state: bool = True, max_q_len: int = 0) -> None:
    """The minGRU over each request's tokens of the step, per channel: z = sigmoid(z_pre + z_bias), u = u_pre + u_bias,
    candidate = u + 1/2 where u >= 0 and sigmoid(u) where u < 0, S <- (1 - z) S + z candidate, out = S * silu(g_pre).
    ``z_pre`` and ``u_pre`` are columns of one buffer (one row stride); ``state`` float32 [slots, width].  ``max_q_len``:
    the most tokens a request brings, if known; for prompt portions the kernel that cuts a request's tokens into runs
    (the recurrence is linear in the state) stands in for the token-by-token one."""
    n, width = out.shape
    assert z_pre.shape == u_pre.shape == g_pre.shape == (n, width) and z_pre.stride(0) == u_pre.stride(0)
    assert z_pre.stride(1) == 1 and u_pre.stride(1) == 1 and g_pre.stride(1) == 1 and out.stride(1) == 1
    assert z_pre.dtype == u_pre.dtype == g_pre.dtype == out.dtype
    assert state.dtype is torch.float32 and state.is_contiguous() and state.shape[1:] == (width,)
    biases = [b for b in (z_bias, u_bias) if b is not None]
    assert all(b.dtype == biases[0].dtype and b.shape == (width,) and b.is_contiguous() for b in biases)
    _check(core().ie_mingru_scan_hint(_ptr(z_pre), _ptr(u_pre), z_pre.stride(0), _ptr(g_pre), g_pre.stride(0), _ptr(z_bias),
                                      _ptr(u_bias), dtype_code(biases[0].dtype) if biases else IE_F32, _ptr(state), _ptr(out),
                                      out.stride(0), _ptr(q_start), _ptr(slots), n_requests, width, 1 if write_state else 0,
                                      dtype_code(out.dtype), int(max_q_len or 0), _stream()), f"mingru_scan(width={width})")


# ------------------------------------------------- the stream, shifted inputs, mixed heads, the matrix memory
def scale_add_sinusoid(x: torch.Tensor, positions: torch.Tensor, scale: float, base: float) -> None:
    """x (float32 [n, d]) <- x * scale + s(position): s[2i] = sin(p base^(-2i / d)), s[2i + 1] the cosine of the same."""
    assert x.dtype is torch.float32 and x.is_contiguous() and positions.dtype is torch.int32
    _check(core().ie_scale_add_sinusoid(_ptr(x), _ptr(positions), float(scale), float(base), x.shape[0], x.shape[1],
                                        _stream()), "scale_add_sinusoid")


def add_row(x: torch.Tensor, row: torch.Tensor) -> None:
    """x (float32 [n, d]) += row ([d]) for every row of x."""
    assert x.dtype is torch.float32 and x.is_contiguous() and row.is_contiguous() and row.shape == (x.shape[1],)
    _check(core().ie_add_row(_ptr(x), _ptr(row), dtype_code(row.dtype), x.shape[0], x.shape[1], _stream()), "add_row")


def token_shift(h: torch.Tensor, out: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor,
                ctx_before: torch.Tensor, slots: torch.Tensor, n_requests: int, write_state: bool = True) -> None:
    """out = h + (h' - h) * mu with h' the row of the token before (as it was), zeros before a sequence's first token;
    ``state`` [slots, d] (of h's type) carries a request's last row from step to step."""
    n, d = h.shape
    assert h.is_contiguous() and out.is_contiguous() and out.shape == h.shape and out.dtype == h.dtype
    assert out.data_ptr() != h.data_ptr() and mu.shape == (d,) and mu.is_contiguous()
    assert state.dtype == h.dtype and state.is_contiguous() and state.shape[1:] == (d,)
    _check(core().ie_token_shift(_ptr(h), _ptr(out), dtype_code(h.dtype), _ptr(mu), dtype_code(mu.dtype), _ptr(state),
                                 _ptr(q_start), _ptr(ctx_before), _ptr(slots), n_requests, n, d, 1 if write_state else 0,
                                 _stream()), "token_shift")


def gate_mul(x: torch.Tensor, gate_pre: torch.Tensor, group: int = 1) -> None:
    """x[n, j] *= sigmoid(gate_pre[n, j // group]) in place: a gate per coordinate, or per head of ``group`` coordinates."""
    n, d = x.shape
    assert x.stride(1) == 1 and gate_pre.stride(1) == 1 and gate_pre.dtype == x.dtype and gate_pre.shape == (n, d // group)
    _check(core().ie_gate_mul(_ptr(x), x.stride(0), _ptr(gate_pre), gate_pre.stride(0), n, d, int(group),
                              dtype_code(x.dtype), _stream()), "gate_mul")


def qkv_prepare(q: torch.Tensor, q_heads: int, k: torch.Tensor, k_heads: int, head_dim: int, v: torch.Tensor, v_heads: int,
                v_head_dim: int, slot_mapping: torch.Tensor | None, kpool: torch.Tensor | None, vpool: torch.Tensor | None,
                page_size: int, eps: float, q_bias=None, k_bias=None, v_bias=None, q_norm: bool = False,
                k_norm: bool = False, v_norm: bool = False, pool_v_heads: int | None = None) -> None:
    """Per token: biases added to q, k and v, every head of a side whose flag is set divided by its root mean square
    (no gain), q written back in place, k to its slot of ``kpool`` [pages, k_heads, page_size, head_dim] and v to
    ``vpool`` [pages, pool_v_heads, page_size, v_heads * v_head_dim / pool_v_heads]."""
    n = q.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and q.dtype == k.dtype == v.dtype
    biases = [b for b in (q_bias, k_bias, v_bias) if b is not None]
    assert all(b.dtype == biases[0].dtype and b.is_contiguous() for b in biases)
    assert q_bias is None or q_bias.numel() == q_heads * head_dim
    assert k_bias is None or k_bias.numel() == k_heads * head_dim
    assert v_bias is None or v_bias.numel() == v_heads * v_head_dim
    assert (kpool is None or kpool.dtype == q.dtype) and (vpool is None or vpool.dtype == q.dtype)
    _check(core().ie_qkv_prepare(_ptr(q), q.stride(0), q_heads, _ptr(q_bias), 1 if q_norm else 0, _ptr(k), k.stride(0),
                                 k_heads, _ptr(k_bias), 1 if k_norm else 0, head_dim, _ptr(v), v.stride(0), v_heads,
                                 v_head_dim, _ptr(v_bias), 1 if v_norm else 0,
                                 dtype_code(biases[0].dtype) if biases else IE_F32, float(eps), _ptr(slot_mapping),
                                 _ptr(kpool), _ptr(vpool), int(pool_v_heads or v_heads), n, page_size,
                                 dtype_code(q.dtype), _stream()), "qkv_prepare")


def talk_combine(a: torch.Tensor, talk: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, n_heads: int,
                 n_v_heads: int, v_head_dim: int, first_v_head: int = 0, slice_v_heads: int | None = None) -> None:
    """``out[n, h] = sum_g talk[h, g] * a[n, g, value head of h] * sigmoid(gate[n, h])``: ``a`` [n, n_heads *
    slice_v_heads * v_head_dim] holds every query head's softmax weights applied to the value heads first_v_head ..
    first_v_head + slice_v_heads - 1; the heads of ``out`` ([n, n_heads * v_head_dim]) that read those are written."""
    n = out.shape[0]
    nc = int(slice_v_heads or n_v_heads)
    assert a.stride(1) == 1 and out.stride(1) == 1 and a.dtype == out.dtype and a.shape[1] == n_heads * nc * v_head_dim
    assert talk.dtype is torch.float32 and talk.is_contiguous() and talk.shape == (n_heads, n_heads)
    assert gate is None or (gate.stride(1) == 1 and gate.dtype == out.dtype and gate.shape == out.shape)
    _check(core().ie_talk_combine(_ptr(a), a.stride(0), _ptr(talk), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                  _ptr(out), out.stride(0), n, n_heads, n_v_heads, v_head_dim, int(first_v_head), nc,
                                  dtype_code(out.dtype), _stream()), "talk_combine")


def mlstm_state_floats(head_dim: int, v_head_dim: int) -> int:
    """float32 words of a head's state in ``mlstm_scan``: the matrix, and a copy of the normaliser and the maximum for
    every chunk of value columns that a block takes."""
    n = int(core().ie_mlstm_state_floats(int(head_dim), int(v_head_dim)))
    if n <= 0:
        raise KernelError(f"mlstm_scan takes no heads of {head_dim} x {v_head_dim}")
    return n


def mlstm_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gates: torch.Tensor, i_bias: torch.Tensor,
               f_bias: torch.Tensor, cap: float, state: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
               slots: torch.Tensor, n_requests: int, n_heads: int, head_dim: int, v_head_dim: int,
               write_state: bool = True) -> None:
    """The matrix memory with stabilised exponential gates over each request's tokens of the step.  ``gates`` float32
    [n, 2 * n_heads]: the pre-activations of the input gates, then of the forget gates (biases added here); ``state``
    float32 [slots, n_heads, mlstm_state_floats]; ``out`` float32 [n, n_heads * v_head_dim] takes S^T q over its
    denominator, before the head norm."""
    n = out.shape[0]
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and q.dtype == k.dtype == v.dtype
    assert gates.dtype is torch.float32 and gates.stride(1) == 1 and gates.shape == (n, 2 * n_heads)
    assert i_bias.dtype == f_bias.dtype and i_bias.is_contiguous() and f_bias.is_contiguous()
    assert i_bias.shape == f_bias.shape == (n_heads,)
    assert state.dtype is torch.float32 and state.is_contiguous()
    assert state.shape[1:] == (n_heads, mlstm_state_floats(head_dim, v_head_dim))
    assert out.dtype is torch.float32 and out.stride(1) == 1 and out.shape[1] == n_heads * v_head_dim
    _check(core().ie_mlstm_scan(_ptr(q), _ptr(k), _ptr(v), q.stride(0), k.stride(0), v.stride(0), _ptr(gates),
                                gates.data_ptr() + 4 * n_heads, gates.stride(0), _ptr(i_bias), _ptr(f_bias),
                                dtype_code(i_bias.dtype), float(cap), float(head_dim) ** -0.5, _ptr(state),
                                state.stride(0), _ptr(out), out.stride(0), _ptr(q_start), _ptr(slots), n_requests,
                                n_heads, head_dim, v_head_dim, 1 if write_state else 0, dtype_code(q.dtype), _stream()),
           f"mlstm_scan(heads={n_heads}, {head_dim} x {v_head_dim})")


def mlstm_finish(o: torch.Tensor, gain: torch.Tensor, gate_pre: torch.Tensor, out: torch.Tensor, n_heads: int,
                 v_head_dim: int, eps: float) -> None:
    """out = o / rms(o over each head) * gain * sigmoid(gate_pre): ``o`` float32, ``gain`` of all heads' size."""
    n = out.shape[0]
    w = n_heads * v_head_dim
    assert o.dtype is torch.float32 and o.stride(1) == 1 and o.shape == (n, w) and gain.is_contiguous() and gain.shape == (w,)
    assert gate_pre.stride(1) == 1 and out.stride(1) == 1 and gate_pre.dtype == out.dtype and gate_pre.shape == (n, w)
    _check(core().ie_mlstm_finish(_ptr(o), o.stride(0), _ptr(gain), dtype_code(gain.dtype), _ptr(gate_pre),
                                  gate_pre.stride(0), _ptr(out), out.stride(0), n, n_heads, v_head_dim, float(eps),
                                  dtype_code(out.dtype), _stream()), "mlstm_finish")


# ------------------------------------------------------------------ a mixture of experts
def moe_tile_rows() -> int:
    return int(core().ie_moe_tile_rows())


def moe_max_tiles(n_pairs: int, n_experts: int) -> int:
    """An upper bound of the row tiles that ``moe_sort`` makes of ``n_pairs`` pairs (no tile spans two experts)."""
    return -(-n_pairs // moe_tile_rows()) + min(n_experts, n_pairs)


ROUTE_SCORES = {"sigmoid": 0, "softmax_top": 1}


def moe_route(logits: torch.Tensor, correction: torch.Tensor | None, ids: torch.Tensor, weights: torch.Tensor,
              gate: torch.Tensor | None, n_experts: int, top: int, n_groups: int, keep_groups: int, route_scale: float,
              weight_eps: float, gate_col: int = -1, score: str = "sigmoid") -> None:
    """Per token, from float32 router ``logits`` [n, >= n_experts]: the chosen experts ``ids`` int32 [n, top] and their
    ``weights`` float32 [n, top]; ``gate`` float32 [n] = sigmoid(logits[:, gate_col]) (the shared expert's).  ``score``
    "sigmoid": sigmoid scores, ``correction`` added for the choice only, weights the chosen scores over their sum.
    "softmax_top": ``correction`` is a bias of the logits themselves, the largest ``top`` are chosen and their weights
    are the softmax over the chosen logits alone (times ``route_scale``)."""
    n = logits.shape[0]
    assert logits.dtype is torch.float32 and logits.stride(1) == 1 and ids.dtype is torch.int32 and ids.is_contiguous()
    assert weights.dtype is torch.float32 and weights.is_contiguous() and ids.shape == weights.shape == (n, top)
    assert gate is None or (gate.dtype is torch.float32 and gate.shape == (n,))
    _check(core().ie_moe_route(_ptr(logits), logits.stride(0), _ptr(correction),
                               dtype_code(correction.dtype) if correction is not None else IE_F32, _ptr(ids),
                               _ptr(weights), _ptr(gate), n, n_experts, top, n_groups, keep_groups, float(route_scale),
                               float(weight_eps), int(gate_col), ROUTE_SCORES[score], _stream()), f"moe_route(experts={n_experts}, top={top})")


def moe_sort(ids: torch.Tensor, n_experts: int, sorted_pairs: torch.Tensor, tiles: torch.Tensor) -> None:
    """Order the (token, choice) pairs by expert: ``sorted_pairs`` int32 [n_pairs], ``tiles`` int32 [max_tiles, 4] =
    (expert, first position, rows, 0)."""
    n_pairs = ids.numel()
    assert sorted_pairs.dtype is torch.int32 and sorted_pairs.numel() >= n_pairs and tiles.dtype is torch.int32
    assert tiles.is_contiguous() and tiles.shape[1] == 4 and tiles.shape[0] >= moe_max_tiles(n_pairs, n_experts)
    _check(core().ie_moe_sort(_ptr(ids), n_pairs, n_experts, moe_tile_rows(), _ptr(sorted_pairs), _ptr(tiles),
                              tiles.shape[0], _stream()), "moe_sort")


def moe_gemm(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, sorted_pairs: torch.Tensor, tiles: torch.Tensor,
             top: int, gather: bool, scatter: bool, epi: str = "store") -> None:
    """The grouped product over the tiles of ``moe_sort``: ``w`` [experts, N, K]; ``gather``: a pair's row of ``a`` is
    its token's (pair // top), else its sorted position; ``scatter``: its row of ``c`` is the pair's index, else its
    sorted position; ``epi`` "silu_mul": w's rows alternate gate, up and c is N / 2 wide."""
    _, n, k = w.shape
    assert w.is_contiguous() and a.stride(1) == 1 and c.stride(1) == 1 and a.shape[1] == k
    _check(core().ie_moe_gemm(_ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype), _ptr(c), dtype_code(c.dtype),
                              _ptr(sorted_pairs), _ptr(tiles), tiles.shape[0], n, k, a.stride(0), c.stride(0), n * k, top,
                              1 if gather else 0, 1 if scatter else 0, {"store": 0, "silu_mul": 1}[epi], _stream()),
           f"moe_gemm(n={n}, k={k}, {epi})")


def moe_combine(y: torch.Tensor, weights: torch.Tensor, gate: torch.Tensor | None, shared_out: torch.Tensor | None,
                out: torch.Tensor) -> None:
    """out[t] = sum_r weights[t, r] * y[t * top + r] + gate[t] * shared_out[t]; ``y`` and ``out`` float32."""
    n, top = weights.shape
    d = out.shape[1]
    assert y.dtype is torch.float32 and y.is_contiguous() and y.shape == (n * top, d) and out.dtype is torch.float32
    assert out.is_contiguous() and (shared_out is None or shared_out.stride(1) == 1)
    _check(core().ie_moe_combine(_ptr(y), _ptr(weights), _ptr(gate), _ptr(shared_out),
                                 dtype_code(shared_out.dtype) if shared_out is not None else IE_F32,
                                 shared_out.stride(0) if shared_out is not None else 0, _ptr(out), n, d, top, _stream()),
           "moe_combine")


# ---------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and out.dtype == torch.int32
    _check(core().ie_argmax(_ptr(logits), _ptr(out), logits.shape[0], logits.shape[1], logits.stride(0),
                            _stream()), "argmax")


def repetition_penalty(logits: torch.Tensor, context: torch.Tensor, penalty: torch.Tensor) -> None:
    assert logits.dtype == torch.float32 and context.dtype == torch.int32 and penalty.dtype == torch.float32
    assert context.is_contiguous() and context.shape[0] == logits.shape[0]
    _check(core().ie_repetition_penalty(_ptr(logits), _ptr(context), _ptr(penalty), logits.shape[0],
                                        logits.shape[1], logits.stride(0), context.shape[1], _stream()),
           "repetition_penalty")


def sample(logits: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """rows: int32 [n, 7] records (temperature bits, top_p bits, top_k, seed lo/hi, key lo/hi)."""
    assert logits.dtype == torch.float32 and rows.dtype == torch.int32 and rows.shape == (logits.shape[0], 7)
    assert rows.is_contiguous() and out.dtype == torch.int32
    _check(core().ie_sample(_ptr(logits), _ptr(rows), _ptr(out), logits.shape[0], logits.shape[1],
                            logits.stride(0), _stream()), "sample")


# ------------------------------------------------- tensor-core attention (bfloat16)
MMA_HEAD_DIMS = (64, 128)
_mma: dict[tuple, object] = {}
LOG2E = 1.4426950408889634


def _score_extras(score_bias, head_scale, n_heads):
    """Checks of the two optional score inputs of the bias build: ``score_bias`` float32 [n_heads, D] that already
    carries the factor log2(e) (the kernels work in the exponent's units), ``head_scale`` float32 [n_heads]."""
    if score_bias is not None:
        assert score_bias.dtype is torch.float32 and score_bias.is_contiguous() and score_bias.shape[0] == n_heads
    if head_scale is not None:
        assert head_scale.dtype is torch.float32 and head_scale.is_contiguous() and head_scale.shape == (n_heads,)
    return score_bias.shape[1] if score_bias is not None else 0


def attention_mma_library(head_dim: int, biased: bool = False):
    """The tensor-core attention kernels built for one head size; compiled when first asked for.  ``biased``: the
    build that takes a multiplier per head and a bias by distance on the float32 scores and keeps the weights to two
    bfloat16 terms in the product with the values."""
    if head_dim not in MMA_HEAD_DIMS:
        raise KernelError(f"tensor-core attention is built for head sizes {MMA_HEAD_DIMS}, not {head_dim}")
    key = (head_dim, bool(biased))
    lib = _mma.get(key)
    if lib is None:
        defines = {"IE_HD": head_dim, **BUILD_DEFINES.get("attn_mma", {})}
        name = f"attn_mma_hd{head_dim}"
        if biased:
            defines["IE_ATTN_BIAS"] = 1
            name += "_bias"
        lib = load_library(name, ["attention_mma.cu"], defines, ["attention_noalloc.h"])
        P, I, F = c_void_p, c_int, c_float
        lib.ie_attention_prefill_biased.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, P, P]
        lib.ie_attention_prefill_biased.restype = c_int
        lib.ie_attention_prefill_kept.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, P, I, F, P]
        lib.ie_attention_prefill_kept.restype = c_int
        lib.ie_attention_decode_biased.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P, I, P, P]
        lib.ie_attention_decode_biased.restype = c_int
        lib.ie_attention_prefill.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P]
        lib.ie_attention_prefill.restype = c_int
        lib.ie_attention_decode.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, I, P]
        lib.ie_attention_decode.restype = c_int
        lib.ie_attention_decode_fused.argtypes = [P] * 14 + [I] * 10 + [F, I, I, I, P]
        lib.ie_attention_decode_fused.restype = c_int
        lib.ie_attention_decode_scratch_floats.argtypes = [I, I, I]
        lib.ie_attention_decode_scratch_floats.restype = c_longlong
        lib.ie_attention_decode_ticket_words.restype = c_longlong
        lib.ie_attention_decode_warps.restype = c_int
        lib.ie_attention_decode_max_blocks.restype = c_int
        _mma[key] = lib
        _apply_check_limits()
    return lib


def attention_prefill_mma(q, out, kpool, vpool, block_table, q_start, ctx_before, work_req, work_pair0, n_work,
                          n_heads, n_kv_heads, head_dim, page_size, window, scale, rows: int = 64,
                          score_bias_log2e=None, head_scale=None, keep_first: int = 0, out_scale: float = 1.0,
                          float32_scores: bool = False) -> None:
    """Causal paged attention for any mix of portions and single tokens; bfloat16; the work list cuts each
    request's (token, head-in-group) pairs into tiles of ``rows`` (64 or 128).  With ``score_bias_log2e`` (float32
    [n_heads, D]: the bias by distance times log2 e, last column for every larger distance) or ``head_scale``
    (float32 [n_heads]) the bias build of the kernel runs."""
    assert q.dtype is torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    if keep_first or out_scale != 1.0 or float32_scores:
        # the bias build (float32 scores, weights to two bfloat16 terms) also knows kept first keys beside the window
        # and a multiplier of the output
        dists = _score_extras(score_bias_log2e, head_scale, n_heads)
        lib = attention_mma_library(head_dim, biased=True)
        _check(lib.ie_attention_prefill_kept(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table),
                                             _ptr(q_start), _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0),
                                             q.stride(0), out.stride(0), block_table.stride(0), n_work, n_heads,
                                             n_kv_heads, head_dim, page_size, int(window or 0), float(scale), rows,
                                             _ptr(score_bias_log2e), dists, _ptr(head_scale), int(keep_first or 0),
                                             float(out_scale), _stream()), "attention_prefill_mma (bias build, kept keys)")
        return
    if score_bias_log2e is not None or head_scale is not None:
        dists = _score_extras(score_bias_log2e, head_scale, n_heads)
        lib = attention_mma_library(head_dim, biased=True)
        _check(lib.ie_attention_prefill_biased(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table),
                                               _ptr(q_start), _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0),
                                               q.stride(0), out.stride(0), block_table.stride(0), n_work, n_heads,
                                               n_kv_heads, head_dim, page_size, int(window or 0), float(scale), rows,
                                               _ptr(score_bias_log2e), dists, _ptr(head_scale), _stream()),
               "attention_prefill_mma (bias build)")
        return
    lib = attention_mma_library(head_dim)
    _check(lib.ie_attention_prefill(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                    _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0), q.stride(0), out.stride(0),
                                    block_table.stride(0), n_work, n_heads, n_kv_heads, head_dim, page_size,
                                    int(window or 0), float(scale), rows, _stream()), "attention_prefill_mma")


_wide: dict[tuple, object] = {}


def attention_wide_supports(q: torch.Tensor, out: torch.Tensor, head_dim: int, v_head_dim: int, v_row: int | None = None) -> bool:
    """Whether the tensor-core kernel with float32 scores takes these operands: bfloat16, key and value head sizes
    multiples of 16 up to 256, rows that start on 16 bytes."""
    return (q.dtype is torch.bfloat16 and out.dtype is torch.bfloat16 and 0 < head_dim <= 256 and 0 < v_head_dim <= 256
            and head_dim % 16 == 0 and v_head_dim % 16 == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 2 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 4 == 0 and (v_row or v_head_dim) % 8 == 0)


def attention_wide_library(head_dim: int, v_head_dim: int):
    """The tensor-core attention kernel with float32 scores built for one (key, value) head size; compiled when first
    asked for."""
    key = (int(head_dim), int(v_head_dim))
    lib = _wide.get(key)
    if lib is None:
        defines = {"IE_AW_DK": key[0], "IE_AW_DV": key[1], **BUILD_DEFINES.get("attn_wide", {})}
        lib = load_library(f"attn_wide_k{key[0]}_v{key[1]}", ["attention_wide.cu"], defines)
        P, I, F = c_void_p, c_int, c_float
        lib.ie_attention_wide.argtypes = [P] * 9 + [I] * 8 + [F, I, I, I, P, P]
        lib.ie_attention_wide.restype = c_int
        lib.ie_attention_wide_rows.restype = c_int
        lib.ie_attention_wide_keys.restype = c_int
        lib.ie_attention_wide_small.argtypes = [P] * 7 + [I] * 9 + [F] + [I] * 5 + [P, P, P]
        lib.ie_attention_wide_small.restype = c_int
        lib.ie_attention_wide_small_scratch.argtypes = [I, I, I, I]
        lib.ie_attention_wide_small_scratch.restype = c_longlong
        _wide[key] = lib
        _apply_check_limits()
    return lib


ATTENTION_WIDE_ROWS = 64     # (token, head-in-group) pairs of a tile of the kernel below


def attention_wide(q, out, kpool, vpool, block_table, q_start, ctx_before, work_req, work_pair0, n_work, n_heads,
                   n_kv_heads, head_dim, page_size, window, scale, v_head_dim: int | None = None, chunk: int = 0,
                   n_v_heads: int | None = None, v_row: int | None = None, sink: torch.Tensor | None = None) -> None:
    """Causal paged attention of prompt portions on tensor cores with float32 scores, maxima and sums, the weights to
    two bfloat16 terms: ``attention_general``'s options ``v_head_dim``, ``chunk``, ``n_v_heads`` and ``v_row`` and a
    window, for bfloat16 operands whose head sizes are multiples of 16.  The work list cuts each request's (token,
    head-in-group) pairs into tiles of ``ATTENTION_WIDE_ROWS``."""
    dv = int(v_head_dim or head_dim)
    assert attention_wide_supports(q, out, head_dim, dv, v_row) and kpool.dtype is torch.bfloat16 and vpool.dtype is torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and block_table.dtype == torch.int32 and block_table.stride(1) == 1
    lib = attention_wide_library(head_dim, dv)
    _check(lib.ie_attention_wide(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                 _ptr(ctx_before), _ptr(work_req), _ptr(work_pair0), q.stride(0), out.stride(0),
                                 block_table.stride(0), n_work, n_heads, n_kv_heads, page_size, int(window or 0),
                                 float(scale), int(chunk or 0), int(n_v_heads or 0), int(v_row or 0), _ptr(sink), _stream()),
           f"attention_wide(head_dim={head_dim}/{dv}, heads={n_heads}/{n_kv_heads})")


def attention_wide_splits(head_dim: int, v_head_dim: int, keys: int, n_streams: int, n_sms: int | None = None) -> tuple[int, int]:
    """(n_splits, split_keys) for ``attention_wide_small``: ``keys`` is the longest run of keys a request may see,
    counted from the key tile's boundary below its first one; ``n_streams`` the (request tile, key head) pairs that each
    walk such a run.  Enough splits to fill the device about twice, none shorter than two key tiles."""
    tile = int(attention_wide_library(head_dim, v_head_dim).ie_attention_wide_keys())
    n_tiles = max(1, -(-int(keys) // tile))
    want = max(1, -(-2 * (n_sms or sm_count()) // max(1, n_streams)))
    n_splits = max(1, min(want, n_tiles // 2 or 1))
    per = -(-n_tiles // n_splits)
    return -(-n_tiles // per), per * tile


def attention_wide_small_scratch(head_dim: int, v_head_dim: int, n_requests: int, max_rows: int, n_kv_heads: int, n_splits: int) -> int:
    """float32 words of scratch that ``attention_wide_small`` needs."""
    return int(attention_wide_library(head_dim, v_head_dim).ie_attention_wide_small_scratch(n_requests, max_rows, n_kv_heads, n_splits))


def attention_wide_small(q, out, kpool, vpool, block_table, q_start, ctx_before, n_requests: int, max_rows: int, n_heads,
                         n_kv_heads, head_dim, page_size, window, scale, n_splits: int, split_keys: int,
                         scratch: torch.Tensor | None, v_head_dim: int | None = None, chunk: int = 0,
                         n_v_heads: int | None = None, v_row: int | None = None, sink: torch.Tensor | None = None) -> None:
    """``attention_wide`` for the requests of the step that bring at most ``max_rows`` (token, head-in-group) rows (decode
    tokens, as a rule), without a work list: every (request, key head) is cut into ``n_splits`` runs of ``split_keys``
    keys (``attention_wide_splits``), a block each, and a second kernel merges them through ``scratch`` (float32,
    ``attention_wide_small_scratch`` words).  Rows of requests that bring more are left untouched."""
    dv = int(v_head_dim or head_dim)
    assert attention_wide_supports(q, out, head_dim, dv, v_row) and kpool.dtype is torch.bfloat16 and vpool.dtype is torch.bfloat16
    assert q.stride(1) == 1 and out.stride(1) == 1 and block_table.dtype == torch.int32 and block_table.stride(1) == 1
    lib = attention_wide_library(head_dim, dv)
    if n_splits > 1:
        need = int(lib.ie_attention_wide_small_scratch(n_requests, max_rows, n_kv_heads, n_splits))
        assert scratch is not None and scratch.dtype is torch.float32 and scratch.is_contiguous() and scratch.numel() >= need
    _check(lib.ie_attention_wide_small(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                       _ptr(ctx_before), q.stride(0), out.stride(0), block_table.stride(0), n_requests,
                                       int(max_rows), n_heads, n_kv_heads, page_size, int(window or 0), float(scale),
                                       int(chunk or 0), int(n_v_heads or 0), int(v_row or 0), int(n_splits), int(split_keys),
                                       _ptr(scratch), _ptr(sink), _stream()),
           f"attention_wide_small(head_dim={head_dim}/{dv}, heads={n_heads}/{n_kv_heads}, splits={n_splits})")
    if n_splits > 1:
        global LAUNCHES
        LAUNCHES += 1       # the merge kernel


def attention_decode_scratch_floats(n_tokens, n_heads, n_splits, head_dim, biased: bool = False) -> int:
    # the same in both builds of a head size; ``biased`` only says which one to ask (the one the model has loaded)
    return int(attention_mma_library(head_dim, biased).ie_attention_decode_scratch_floats(n_tokens, n_heads, n_splits))


def attention_decode_geometry(head_dim, biased: bool = False) -> tuple[int, int]:
    """(warps, i.e. splits, of a decode block; the most blocks per (request, kv head) a launch takes)."""
    lib = attention_mma_library(head_dim, biased)
    return int(lib.ie_attention_decode_warps()), int(lib.ie_attention_decode_max_blocks())


def attention_decode_ticket_words(head_dim, biased: bool = False) -> int:
    """How many words at the start of the decode scratch hold tickets; they must be zero before the
    first launch on a piece of scratch (every launch leaves them zero)."""
    return int(attention_mma_library(head_dim, biased).ie_attention_decode_ticket_words())


def attention_decode_mma(q, out, kpool, vpool, block_table, q_start, ctx_before, scratch, n_requests, n_tokens,
                         n_heads, n_kv_heads, head_dim, page_size, window, scale, n_splits, split_keys,
                         score_bias_log2e=None, head_scale=None) -> None:
    """Split-key attention for steps where every request brings at most 16 (token, head-in-group) rows.

    ``scratch`` is float32 device memory of ``attention_decode_scratch_floats`` elements: partial
    tickets in its first ``attention_decode_ticket_words`` words, which must be zero when the first
    launch starts and are zero again when a launch ends, then partial outputs, maxima and sums of
    every block, which are written before they are read.  At most warps x blocks of
    ``attention_decode_geometry`` splits, each a multiple of 32 keys."""
    assert q.dtype is torch.bfloat16 and scratch.dtype is torch.float32
    if score_bias_log2e is not None or head_scale is not None:       # as for the prefill kernel: the bias build
        dists = _score_extras(score_bias_log2e, head_scale, n_heads)
        lib = attention_mma_library(head_dim, biased=True)
        _check(lib.ie_attention_decode_biased(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table),
                                              _ptr(q_start), _ptr(ctx_before), _ptr(scratch), q.stride(0),
                                              out.stride(0), block_table.stride(0), n_requests, n_tokens, n_heads,
                                              n_kv_heads, head_dim, page_size, int(window or 0), float(scale), n_splits,
                                              split_keys, _ptr(score_bias_log2e), dists, _ptr(head_scale), _stream()),
               "attention_decode_mma (bias build)")
        return
    lib = attention_mma_library(head_dim)
    _check(lib.ie_attention_decode(_ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start),
                                   _ptr(ctx_before), _ptr(scratch), q.stride(0), out.stride(0),
                                   block_table.stride(0), n_requests, n_tokens, n_heads, n_kv_heads, head_dim,
                                   page_size, int(window or 0), float(scale), n_splits, split_keys, _stream()),
           "attention_decode_mma")


def attention_decode_fused(q, k_new, v_new, out, kpool, vpool, block_table, q_start, ctx_before, scratch, cos, sin,
                           positions, slot_mapping, n_requests, n_heads, n_kv_heads, head_dim, page_size, window,
                           scale, write_kv, n_splits, split_keys) -> None:
    """``attention_decode_mma`` for steps in which every request brings exactly one token, with the rotary
    encoding and the cache write folded in: ``q`` and ``k_new`` arrive unrotated; with ``write_kv`` the
    token's key (rotated) and value join the keys of the step and are stored at ``slot_mapping`` in the
    pools.  ``cos``/``sin`` are float32 tables [positions, head_dim/2], or None for no rotation."""
    assert q.dtype is torch.bfloat16 and scratch.dtype is torch.float32
    assert k_new.stride(0) == v_new.stride(0) and k_new.stride(1) == 1 and v_new.stride(1) == 1
    lib = attention_mma_library(head_dim)
    _check(lib.ie_attention_decode_fused(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(out), _ptr(kpool), _ptr(vpool),
                                         _ptr(block_table), _ptr(q_start), _ptr(ctx_before), _ptr(scratch),
                                         _ptr(cos), _ptr(sin), _ptr(positions), _ptr(slot_mapping), q.stride(0),
                                         k_new.stride(0), out.stride(0), block_table.stride(0), n_requests, n_heads,
                                         n_kv_heads, head_dim, page_size, int(window or 0), float(scale),
                                         1 if write_kv else 0, n_splits, split_keys, _stream()),
           "attention_decode_fused")


# ------------------------------------------------- generalized delta rule (a recurrent mixer)
DELTA_RULE_MAX_DIM = 128
_delta: dict[int, object] = {}


def delta_rule_library(head_dim: int):
    """The delta-rule kernel built for one head size; compiled when first asked for."""
    if not 1 <= head_dim <= DELTA_RULE_MAX_DIM:
        raise KernelError(f"the delta-rule kernel keeps a state column in registers: head sizes up to "
                          f"{DELTA_RULE_MAX_DIM}, not {head_dim}")
    lib = _delta.get(head_dim)
    if lib is None:
        defines = {"IE_DR_DIM": head_dim, **BUILD_DEFINES.get("delta_rule", {})}
        lib = load_library(f"delta_rule_d{head_dim}", ["delta_rule.cu"], defines)
        P, I, F = c_void_p, c_int, c_float
        lib.ie_delta_rule.argtypes = [P, P, P, P, P, I, P, I, P, P, P, I, P, P, I, P, P, I, I, I, F, F, F, I, I, P]
        lib.ie_delta_rule.restype = c_int
        _delta[head_dim] = lib
        _apply_check_limits()
    return lib


def delta_rule(r, k, v, a_pre, g, w_pre, a_bias, w_bias, out_gain, state, out, q_start, slots, n_requests: int,
               n_heads: int, head_dim: int, decay_rate: float, key_eps: float, norm_eps: float,
               write_state: bool = True) -> None:
    """One step of the generalized delta rule for every (request, head) of the batch.

    ``r, k, v, a_pre, g``: [n, heads * head_dim] views with one row stride (columns of one projection buffer) in the
    activation type; ``w_pre`` float32 [n, heads * head_dim]; ``a_bias, w_bias, out_gain`` [heads * head_dim];
    ``state`` float32 [slots, heads, head_dim, head_dim], read and (with ``write_state``) written at ``slots[request]``;
    ``out`` [n, heads * head_dim] in the activation type: the normed, gated result for the output projection."""
    width = n_heads * head_dim
    for t in (r, k, v, a_pre, g):
        assert t.dtype == r.dtype and t.stride(1) == 1 and t.stride(0) == r.stride(0) and t.shape[1] == width
    assert w_pre.dtype is torch.float32 and w_pre.stride(1) == 1 and state.dtype is torch.float32 and state.is_contiguous()
    assert a_bias.dtype == w_bias.dtype == out_gain.dtype and out.dtype == r.dtype and out.stride(1) == 1
    assert state.shape[1:] == (n_heads, head_dim, head_dim)
    _check(delta_rule_library(head_dim).ie_delta_rule(
        _ptr(r), _ptr(k), _ptr(v), _ptr(a_pre), _ptr(g), r.stride(0), _ptr(w_pre), w_pre.stride(0), _ptr(a_bias),
        _ptr(w_bias), _ptr(out_gain), dtype_code(a_bias.dtype), _ptr(state), _ptr(out), out.stride(0), _ptr(q_start),
        _ptr(slots), n_requests, n_heads, head_dim, float(decay_rate), float(key_eps), float(norm_eps),
        1 if write_state else 0, dtype_code(r.dtype), _stream()), f"delta_rule(head_dim={head_dim}, heads={n_heads})")


# ------------------------------------------------- gated delta rule (a recurrent mixer)
_gated_delta: dict[tuple, object] = {}


def gated_delta_library(head_dim: int, v_head_dim: int):
    """The gated delta-rule kernel built for one pair of head sizes; compiled when first asked for."""
    key = (int(head_dim), int(v_head_dim))
    lib = _gated_delta.get(key)
    if lib is None:
        if not (1 <= key[0] <= 512 and 1 <= key[1] <= 1024):
            raise KernelError(f"the gated delta-rule kernel takes key heads up to 512 and value heads up to 1024, not {key}")
        defines = {"IE_GD_DK": key[0], "IE_GD_DV": key[1], **BUILD_DEFINES.get("gated_delta", {})}
        lib = load_library(f"gated_delta_k{key[0]}_v{key[1]}", ["gated_delta.cu"], defines)
        P, I, F = c_void_p, c_int, c_float
        lib.ie_gated_delta.argtypes = [P, P, P, I, I, P, P, I, P, I, P, P, P, I, P, P, I, P, P, I, I, I, I, I, F, F, I, I, P]
        lib.ie_gated_delta.restype = c_int
        _gated_delta[key] = lib
        _apply_check_limits()
    return lib


def gated_delta(q, k, v, b_pre, a_pre, gate, a_log, dt_bias, out_gain, state, out, q_start, slots, n_requests: int,
                n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, key_eps: float, norm_eps: float,
                write_state: bool = True) -> None:
    """One step of the gated delta rule for every (request, head) of the batch.

    ``q, k`` [n, kv_heads * head_dim] and ``v`` [n, heads * v_head_dim] (after their convolutions and SiLU), ``b_pre,
    a_pre`` [n, heads], ``gate`` [n, heads * v_head_dim]: row-strided views in the activation type; ``a_log, dt_bias``
    [heads] and ``out_gain`` [v_head_dim] of one type; ``state`` float32 [slots, heads, head_dim, v_head_dim], read and
    (with ``write_state``) written at ``slots[request]``; ``out`` [n, heads * v_head_dim] in the activation type: the
    normed, gated result for the output projection."""
    for t in (q, k, v, b_pre, a_pre, gate, out):
        assert t.dtype == q.dtype and t.stride(1) == 1
    assert q.stride(0) == k.stride(0) and b_pre.stride(0) == a_pre.stride(0)
    assert q.shape[1] == k.shape[1] == n_kv_heads * head_dim and v.shape[1] == gate.shape[1] == n_heads * v_head_dim
    assert state.dtype is torch.float32 and state.is_contiguous() and state.shape[1:] == (n_heads, head_dim, v_head_dim)
    assert a_log.dtype == dt_bias.dtype == out_gain.dtype and out_gain.shape == (v_head_dim,)
    _check(gated_delta_library(head_dim, v_head_dim).ie_gated_delta(
        _ptr(q), _ptr(k), _ptr(v), q.stride(0), v.stride(0), _ptr(b_pre), _ptr(a_pre), b_pre.stride(0), _ptr(gate),
        gate.stride(0), _ptr(a_log), _ptr(dt_bias), _ptr(out_gain), dtype_code(a_log.dtype), _ptr(state), _ptr(out),
        out.stride(0), _ptr(q_start), _ptr(slots), n_requests, n_heads, n_kv_heads, head_dim, v_head_dim, float(key_eps),
        float(norm_eps), 1 if write_state else 0, dtype_code(q.dtype), _stream()),
        f"gated_delta(head_dim={head_dim}, v_head_dim={v_head_dim}, heads={n_heads}/{n_kv_heads})")


# ----------------------------------------------- weight-streaming product for few rows
STREAM_MAX_ROWS = 64        # what the kernel takes
STREAM_BEST_ROWS = 16       # beyond this the library product is faster (activations are re-read per block)
_EPI = {"bf16": 0, "f32": 1, "residual": 2, "silu_mul": 3, "residual_normout": 4}
SSQ_SLOT = 16               # rows of a sums-of-squares array ([SSQ_SLOT, blocks]: a block's sum for each activation row)
_stream_lib = None
_stream_variants: dict = {}


def _bind_stream(lib):
    P, I, F = c_void_p, c_int, c_float
    lib.ie_gemm_stream.argtypes = [P, P, P, P, I, P, I, I, I, I, I, I, F, I, I, I, P]
    lib.ie_gemm_stream.restype = c_int
    lib.ie_gemm_stream_tma.argtypes = [P, P, P, P, I, P, I, I, I, I, I, I, F, I, I, I, P, I, P, I, P, I, P]
    lib.ie_gemm_stream_tma.restype = c_int
    lib.ie_gemm_stream_tma_supports.argtypes = [I, I, I, I]
    lib.ie_gemm_stream_tma_supports.restype = c_int
    lib.ie_gemm_stream_tma_error.restype = c_int
    return lib


def stream_library(defines: dict | None = None):
    """The streaming products' library.  With ``defines`` a variant compiled with those -D flags (kept apart from the
    product's own; ``gemm_stream(..., lib=...)`` runs it)."""
    global _stream_lib
    if defines:
        key = repr(sorted(defines.items()))
        if key not in _stream_variants:
            _stream_variants[key] = _bind_stream(load_library("stream", ["gemm_stream.cu", "gemm_stream_tma.cu"], dict(defines)))
        return _stream_variants[key]
    if _stream_lib is None:
        _stream_lib = _bind_stream(load_library("stream", ["gemm_stream.cu", "gemm_stream_tma.cu"],
                                                dict(BUILD_DEFINES.get("stream", {}))))
    return _stream_lib


_n_sms: dict[int, int] = {}


def sm_count() -> int:
    dev = torch.cuda.current_device()
    if dev not in _n_sms:
        _n_sms[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _n_sms[dev]


def stream_error(lib=None) -> int:
    """Reads and clears the error word of the bulk-copy streaming kernel (0: no wait ever timed out)."""
    return int((lib or stream_library()).ie_gemm_stream_tma_error())


def gemm_stream_ring_supports(m: int, n: int, k: int, normed: bool) -> bool:
    """Whether the streaming kernel with the shared-memory ring takes m rows of k columns (with a norm in its
    prologue: the rows must then fit in shared memory beside the ring)."""
    return bool(stream_library().ie_gemm_stream_tma_supports(m, n, k, 1 if normed else 0))


def gemm_stream(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, m: int, epi: str = "bf16",
                gain: torch.Tensor | None = None, eps: float = 0.0, row_index: torch.Tensor | None = None,
                nt: int | None = None, prenormed=None, normout=None, lib=None) -> None:
    """c = a @ w^T for m <= 64 rows, bfloat16 weights, reading w once at HBM speed.

    With ``gain`` the input ``a`` is the float32 residual stream (rows gathered by ``row_index`` if given)
    and RMSNorm with that gain and ``eps`` is applied inside the kernel.  ``epi``: "bf16" or "f32" store,
    "residual" adds into the float32 ``c``, "silu_mul" takes w's rows as alternating gate/up and writes
    silu(gate)*up, half as wide.

    Two products can hand a norm over between them.  ``normout=(xg, gain_next, ssq)`` with epi "residual":
    besides adding into ``c`` the kernel writes ``xg`` = bfloat16(new c * gain_next) and, per block, the sums of
    squares of the new rows into ``ssq`` ([SSQ_SLOT rows, SMs] float32).  ``prenormed=(xg, ssq)`` with ``eps``: ``a`` is
    ignored, the input is ``xg`` and the 1/rms comes from ``ssq``: RMSNorm without reading the residual again."""
    n, k = w.shape
    assert w.dtype is torch.bfloat16 and w.stride(1) == 1 and a.stride(-1) == 1 and c.stride(-1) == 1
    lib = lib or stream_library()
    if prenormed is not None or normout is not None:
        pro = 2 if prenormed is not None else 0
        xg, ssq = (prenormed if prenormed is not None else (normout[0], normout[2]))
        gain_next = normout[1] if normout is not None else None
        src = xg if prenormed is not None else a
        assert src.dtype is torch.bfloat16 and xg.dtype is torch.bfloat16 and ssq.dtype is torch.float32
        assert nt is None and lib.ie_gemm_stream_tma_supports(m, n, k, pro)
        code = _EPI["residual_normout"] if normout is not None else _EPI[epi]
        _check(lib.ie_gemm_stream_tma(_ptr(src), _ptr(w), _ptr(c), None, 0, None, m, n, k, src.stride(0), w.stride(0),
                                      c.stride(0), float(eps), pro, code, sm_count(), _ptr(xg), xg.stride(0),
                                      _ptr(gain_next), dtype_code(gain_next.dtype) if gain_next is not None else 0,
                                      _ptr(ssq), ssq.shape[1], _stream()),
               f"gemm_stream_tma(m={m}, n={n}, k={k}, {epi}, handed-over norm)")
        return
    if gain is None:
        assert a.dtype is torch.bfloat16
    else:
        assert a.dtype is torch.float32 and gain.shape == (k,)
    if nt is None and lib.ie_gemm_stream_tma_supports(m, n, k, 0 if gain is None else 1):
        # persistent bulk-copy kernel: one block per SM, weights through a ring of shared memory
        _check(lib.ie_gemm_stream_tma(_ptr(a), _ptr(w), _ptr(c), _ptr(gain),
                                      dtype_code(gain.dtype) if gain is not None else 0, _ptr(row_index), m, n, k,
                                      a.stride(0), w.stride(0), c.stride(0), float(eps),
                                      0 if gain is None else 1, _EPI[epi], sm_count(), None, 0, None, 0, None, 0,
                                      _stream()),
               f"gemm_stream_tma(m={m}, n={n}, k={k}, {epi})")
        return
    if nt is None:
        nt = 4 if n >= 16384 else (2 if n >= 8192 else 1)
        if m > 32:
            nt = min(nt, 2)
    _check(lib.ie_gemm_stream(_ptr(a), _ptr(w), _ptr(c), _ptr(gain),
                                           dtype_code(gain.dtype) if gain is not None else 0, _ptr(row_index), m, n, k,
                                           a.stride(0), w.stride(0), c.stride(0), float(eps),
                                           0 if gain is None else 1, _EPI[epi], nt, _stream()),
           f"gemm_stream(m={m}, n={n}, k={k}, {epi})")


# ------------------------------------------------ tcgen05 product for many rows (prompt portions)
_tc_lib = None


def tcgen05_library():
    global _tc_lib
    if _tc_lib is None:
        lib = load_library("tcgen05", ["gemm_tcgen05.cu"], dict(BUILD_DEFINES.get("tcgen05", {})))
        P, I = c_void_p, c_int
        lib.ie_gemm_tcgen05.argtypes = [P, P, P, I, I, I, I, I, I, I, I, I, P]
        lib.ie_gemm_tcgen05.restype = c_int
        lib.ie_gemm_tcgen05_act.argtypes = [c_void_p] * 3 + [c_int] * 10 + [c_float] * 3 + [c_void_p]
        lib.ie_gemm_tcgen05_act.restype = c_int
        lib.ie_gemm_tcgen05_supports.argtypes = [I, I, I, I, I]
        lib.ie_gemm_tcgen05_supports.restype = c_int
        lib.ie_gemm_tcgen05_error.restype = c_int
        _tc_lib = lib
    return _tc_lib


def gemm_tcgen05_supports(m: int, n: int, k: int, lda: int, ldw: int) -> bool:
    return bool(tcgen05_library().ie_gemm_tcgen05_supports(m, n, k, lda, ldw))


def gemm_tcgen05_error() -> int:
    """Reads and clears the error word that a timed-out wait of the tcgen05 kernel leaves (0: none)."""
    return int(tcgen05_library().ie_gemm_tcgen05_error())


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, epi: str = "bf16", bn: int = 256,
                 act: tuple[float, float, float] | None = None) -> None:
    """c = a @ w^T on the fifth-generation tensor cores (TMA operands, accumulator in tensor memory).

    ``epi``: "bf16" store, "residual" adds into the float32 ``c``, "silu_mul" takes w's rows as alternating
    gate/up and writes silu(gate)*up, half as wide.  ``bn``: tile width, 128 or 256.  ``act`` = (alpha, limit, up_offset)
    with "silu_mul": g' sigmoid(alpha g') (u' + up_offset) with g' = min(g, limit) and u' = clamp(u, -limit, limit)."""
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
    assert act is None or epi == "silu_mul"
    alpha, limit, up_offset = act if act is not None else (1.0, 0.0, 0.0)
    _check(tcgen05_library().ie_gemm_tcgen05_act(_ptr(a), _ptr(w), _ptr(c), m, n, k, a.stride(0), w.stride(0), c.stride(0),
                                                 _EPI[epi], bn, sm_count(), 1 if act is not None else 0, float(alpha),
                                                 float(limit), float(up_offset), _stream()),
           f"gemm_tcgen05(m={m}, n={n}, k={k}, {epi})")


# ------------------------------------------- prompt-portion attention on tcgen05 (head sizes 64 and 128)
_fa5_lib = None


def attention_tcgen05_library():
    global _fa5_lib
    if _fa5_lib is None:
        lib = load_library("attn_tcgen05", ["attention_tcgen05.cu"], dict(BUILD_DEFINES.get("attn_tcgen05", {})))
        P, I = c_void_p, c_int
        lib.ie_attention_tcgen05.argtypes = [P] * 9 + [I] * 9 + [c_float, P, P, P, P]
        lib.ie_attention_tcgen05.restype = c_int
        lib.ie_attention_tcgen05_supports.argtypes = [I, I, I]
        lib.ie_attention_tcgen05_supports.restype = c_int
        lib.ie_attention_tcgen05_error.restype = c_int
        _fa5_lib = lib
        _apply_check_limits()
    return _fa5_lib


def attention_tcgen05_supports(head_dim: int, page_size: int, window) -> bool:
    return bool(attention_tcgen05_library().ie_attention_tcgen05_supports(head_dim, page_size, int(window or 0)))


def attention_tcgen05_error() -> int:
    """Reads and clears the error word that a timed-out wait of the kernel leaves (0: none)."""
    return int(attention_tcgen05_library().ie_attention_tcgen05_error())


def attention_tcgen05(q, out, kpool, vpool, block_table, q_start, ctx_before, work_req, work_pair0, n_work,
                      n_heads, n_kv_heads, head_dim, page_size, scale, cos=None, sin=None, positions=None) -> None:
    """Causal paged attention for prompt portions with tcgen05 tensor cores; bfloat16, head size 64 or 128;
    the work list cuts each request's (token, head-in-group) rows into tiles of 128.  ``kpool``/``vpool``
    are one layer's pages, [pages, kv_heads, page_size, head_dim], contiguous.  With ``cos``/``sin`` (float32
    [positions, head_dim/2]) and ``positions`` (int32 per token) q arrives unrotated and is rotated as read."""
    assert q.dtype is torch.bfloat16 and q.stride(1) == 1 and out.stride(1) == 1
    assert kpool.is_contiguous() and vpool.is_contiguous() and kpool.dim() == 4
    _check(attention_tcgen05_library().ie_attention_tcgen05(
        _ptr(q), _ptr(out), _ptr(kpool), _ptr(vpool), _ptr(block_table), _ptr(q_start), _ptr(ctx_before),
        _ptr(work_req), _ptr(work_pair0), q.stride(0), out.stride(0), block_table.stride(0), n_work, n_heads,
        n_kv_heads, head_dim, page_size, kpool.shape[0], float(scale), _ptr(cos), _ptr(sin), _ptr(positions),
        _stream()), "attention_tcgen05")


# ------------------------------------------------ a checks build: page ids, slots and token ids compared with limits
# (the device has no sanitizer here: this is what stands in for one while debugging a cache manager or a new part)
CHECK_LIBRARIES = ("core", "attn_mma", "attn_tcgen05", "attn_wide", "delta_rule", "gated_delta")
CHECK_UNITS = ("elementwise", "rowwise", "sequence", "attention_general", "attention_mma", "attention_tcgen05",
               "attention_wide", "delta_rule", "gated_delta", "headwise", "gating", "stream_shift", "headmix",
               "matrix_memory")
CHECK_CODES = {1: "page id", 2: "cache slot", 3: "token id"}
_check_limits: tuple[int, int, int] | None = None


def enable_checks() -> None:
    """Build the kernels that read page ids, cache slots and token ids from memory with ``-DIE_CHECKS=1``: a value out
    of range is recorded and replaced by a safe one instead of being used.  Call before the first kernel runs (a
    library that is already loaded stays as it was built); then ``set_check_limits``, and ``check_device_errors`` or
    ``read_check_words`` after the steps in question."""
    for name in CHECK_LIBRARIES:
        BUILD_DEFINES.setdefault(name, {})["IE_CHECKS"] = 1


def checks_enabled() -> bool:
    return any(BUILD_DEFINES.get(name, {}).get("IE_CHECKS") for name in CHECK_LIBRARIES)


def _loaded_check_functions(prefix: str):
    from .csrc import build as _build
    for lib in list(_build._loaded.values()):
        for unit in CHECK_UNITS:
            try:
                fn = getattr(lib, f"{prefix}_{unit}")
            except AttributeError:
                continue
            yield unit, fn


def _apply_check_limits() -> None:
    if _check_limits is None:
        return
    for unit, fn in _loaded_check_functions("ie_check_limits"):
        fn.argtypes = [c_int, c_int, c_int]
        fn.restype = c_int
        _check(fn(*_check_limits), f"ie_check_limits_{unit}")


def set_check_limits(n_pages: int, n_slots: int, vocab: int) -> None:
    """The limits of a checks build: page ids below ``n_pages``, cache slots below ``n_slots``, token ids below
    ``vocab`` (libraries that load later get them when they load)."""
    global _check_limits
    _check_limits = (int(n_pages), int(n_slots), int(vocab))
    _apply_check_limits()


def read_check_words() -> list[tuple[str, str, int, int, int]]:
    """(unit, what, first bad value, its limit, how many) for every unit of a checks build that saw a value out of
    range since the last call; synchronises the device."""
    import ctypes
    out = []
    for unit, fn in _loaded_check_functions("ie_check_read"):
        word = (ctypes.c_int * 4)()
        fn.argtypes = [c_void_p]
        fn.restype = c_int
        _check(fn(ctypes.addressof(word)), f"ie_check_read_{unit}")
        if word[3]:
            out.append((unit, CHECK_CODES.get(word[0], str(word[0])), int(word[1]), int(word[2]), int(word[3])))
    return out


def check_device_errors() -> None:
    """Reads the error words of the kernels that wait on barriers (a wait that ran out records a code and the
    kernel leaves early) and raises if any is set.  It synchronises the device, so it belongs where the
    engine is idle anyway: after a replayed step, at the end of a generation."""
    found = []
    if _stream_lib is not None and (e := stream_error()):
        found.append(f"streaming product: code {e}")
    if _tc_lib is not None and (e := gemm_tcgen05_error()):
        found.append(f"tcgen05 product: code {e}")
    if _fa5_lib is not None and (e := attention_tcgen05_error()):
        found.append(f"tcgen05 attention: code {e}")
    if found:
        raise KernelError("a kernel gave up a bounded wait; its results are not valid (" + "; ".join(found) + ")")
    if checks_enabled():
        bad = read_check_words()
        if bad:
            raise KernelError("checks build: " + "; ".join(
                f"{unit} read {n} value(s) out of range, the first a {what} of {v} (limit {lim})" for unit, what, v, lim, n in bad))
