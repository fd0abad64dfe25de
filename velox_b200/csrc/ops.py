"""Python face of the kernel library: one function per C entry point.

The library is compiled on first use (`build.build`) and loaded with ctypes.
There is no other implementation behind these functions: if the library cannot
be built or loaded, or a kernel refuses a size, the call raises.  Every function
launches on torch's current CUDA stream and takes torch tensors only as holders
of device memory.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build as _build

_LIB = None

VX_F32, VX_BF16 = 0, 1
ACTIVATIONS = {"silu": 0, "gelu": 1, "gelu_pytorch_tanh": 2, "relu": 3}
_ACT_IDENTITY = 4   # (the activation kernel as a plain change of element type)
_ERRORS = {
    -1: "a size the kernel does not take",
    -2: "an element type the kernel does not know",
    -3: "a pointer or stride that is not aligned as the kernel needs",
    -4: "a size beyond the kernel's stated maximum",
    -5: "the device or driver lacks what the kernel needs",
}


class KernelError(RuntimeError):
    pass


def library():
    """The loaded kernel library; built first if needed.  Raises if it cannot be had."""
    global _LIB
    if _LIB is None:
        path = _build.build()
        try:
            _LIB = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError("the kernel library %s could not be loaded: %s" % (path, e))
        _declare(_LIB)
        if os.environ.get("VELOX_B200_PDL", "1") == "0":
            _LIB.vx_set_pdl(0)
        if os.environ.get("VELOX_B200_PDL_MASK"):
            _LIB.vx_set_pdl_mask(int(os.environ["VELOX_B200_PDL_MASK"], 0))
    return _LIB


def set_pdl(enabled: bool) -> None:
    """Programmatic dependent launch on or off for kernels launched from now on
    (on by default; VELOX_B200_PDL=0 in the environment starts with it off)."""
    library().vx_set_pdl(1 if enabled else 0)


def is_loaded() -> bool:
    return _LIB is not None


def _declare(lib) -> None:
    P, I, F = c_void_p, c_int, c_float
    sigs = {
        "vx_embedding": [P, P, P, I, I, I, I, F, P, P],
        "vx_add_rmsnorm": [P, P, P, P, P, P, I, I, F, I, P],
        "vx_rmsnorm": [P, P, P, I, I, F, I, P],
        "vx_gated_act": [P, P, I, I, I, I, I, I, P],
        "vx_add_bias": [P, P, P, I, I, I, F, P],
        "vx_qk_norm_rope_kv": [P, I, P, P, F, P, I, P, P, P, P, I, I, I, I, I, I, I, P],
        "vx_paged_attention_generic": [P, I, P, P, P, I, P, P, P, I, F, I, I, I, I, I, I, I, I, I, F, P, I, P],
        "vx_biased_attention": [P, I, P, P, P, I, P, P, P, P, P, I, F, F, I, I, I, I, I, I, I, I, I, P, I, P, I, P],
        "vx_latent_attention": [P, P, P, I, P, P, P, P, F, I, I, I, I, I, I, I, P],
        "vx_biased_attention_cap": [P, I, P, P, P, I, P, P, P, P, P, I, F, F, I, I, I, I, I, I, I, I, I, P, I, P, I, F, P],
        "vx_embedding_pair": [P, P, P, P, P, P, P, P, P, I, I, I, I, c_longlong, c_longlong, I, P],
        "vx_merge_norm_add_norm": [P, P, P, F, P, P, F, P, F, P, P, I, I, F, I, P],
        "vx_act": [P, I, P, I, I, I, I, I, P],
        "vx_gated_rmsnorm": [P, P, I, P, P, I, I, F, I, P],
        "vx_kv_store": [P, I, I, I, P, P, P, I, I, I, I, I, I, P],
        "vx_linear_attention_recurrent": [P, I, I, I, I, P, P, P, P, P, I, I, I, I, I, I, P],
        "vx_linear_attention_chunked": [P, I, I, I, I, P, P, P, P, P, I, I, I, I, P],
        "vx_linear_attention_parallel": [P, I, I, I, I, P, P, P, P, P, P, I, I, I, I, I, P],
        "vx_moe_route": [P, I, P, P, I, I, I, I, I, P, P, P, P, P, P, P, P, P, I, I, P, I, I, F, I, P, P],
        "vx_moe_gemm": [P, I, P, I, P, P, P, I, P, I, I, I, I, I, I, I, I, I, P],
        "vx_moe_combine": [P, P, P, P, P, I, I, I, I, I, P, I, P, I, P, P],
        "vx_moe_gather_rows": [P, I, P, I, P, I, I, P],
        "vx_moe_gemm_tcgen05": [P, P, P, I, I, I, I, I, I, I, I, P, P, I, P, P],
        "vx_gemm_nt_simt": [P, P, P, P, I, I, I, I, I, I, I, I, P],
        "vx_gemm_tcgen05": [P, P, P, P, I, I, I, I, I, I, I, I, I, P, P],
        "vx_gemm_tcgen05_pair": [P, P, P, P, I, I, I, I, I, I, I, I, P, P],
        "vx_gemm_skinny": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, P],
        "vx_paged_prefill_attention_tc": [P, I, I, P, P, I, P, I, P, P, P, P, I, F, I, I, I, I, I, I, I, P, I, P, P],
        "vx_paged_prefill_attention_tc_ext": [P, I, I, P, P, I, P, I, P, P, P, P, I, F, I, I, I, I, I, I, I, P, I, P, P, I, P],
        "vx_paged_prefill_attention": [P, I, P, P, P, I, P, P, P, P, I, F, I, I, I, I, I, I, I, P],
        "vx_paged_decode_attention": [P, I, P, P, P, I, P, P, P, P, I, P, I, F, I, I, I, I, I, I, I, I, P],
        "vx_sample": [P, I, I, I, P, P, P, P, P],
        "vx_qk_norm_rope_kv_pairs": [P, I, P, P, F, P, I, P, P, P, P, I, I, I, I, I, I, I, I, P],
        "vx_paged_attention_generic_cap": [P, I, P, P, P, I, P, P, P, I, F, I, I, I, I, I, I, I, I, I, F, P, I, F, I, P],
        "vx_gemm_nt_simt_batched": [P, P, P, P, I, I, I, I, I, I, I, c_longlong, c_longlong, c_longlong, I, I, P],
        "vx_linear_attention_walk": [P, I, I, I, I, P, P, I, F, P, I, I, P, F, F, P, P, P, P, I, I, I, I, I, P],
        "vx_linear_attention_walk_parts": [P, I, I, I, I, P, P, I, F, P, I, I, P, F, F, P, P, P, P, I, I, I, I, I, I, P],
        "vx_stretch_log_decay": [P, I, F, P, P, I, I, P],
        "vx_stretch_scan": [P, P, P, P, P, P, P, I, I, I, I, P],
        "vx_latent_gather": [P, P, I, P, P, P, P, I, P, I, I, I, I, I, I, P],
        "vx_biased_attention_rows": [P, I, P, c_longlong, c_longlong, P, c_longlong, c_longlong, P, I, P, P, P, P, I, F, I, I, I, I, I,
                                     I, I, F, P],
        "vx_head_norm_gate": [P, P, I, P, P, I, I, I, F, I, I, P],
        "vx_latent_prep": [P, I, P, I, P, P, F, P, I, P, P, P, I, I, I, I, I, I, P],
        "vx_capped_gated_act": [P, P, P, I, I, F, F, I, P],
        "vx_sum_add_rmsnorm": [P, P, F, P, F, P, F, P, P, P, P, I, I, F, I, P],
        "vx_softcap_rows": [P, P, c_longlong, F, P],
        "vx_qk_norm_rope_kv_shared": [P, I, P, P, F, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P],
        "vx_paged_attention_generic_shared": [P, I, P, P, P, I, P, P, P, I, F, I, I, I, I, I, I, I, I, I, F, P, I, F, I, I, I, P],
        "vx_latent_attention_window": [P, P, P, I, P, P, P, P, F, I, I, I, I, I, I, I, I, P],
        "vx_stream_norm": [P, I, P, P, P, P, F, P, I, P, I, I, I, I, P],
        "vx_stream_update": [P, I, P, P, F, P, P, I, P, P, F, P, I, I, I, I, P],
        "vx_diff_combine": [P, I, P, I, I, P, F, F, F, I, I, I, I, I, P],
        "vx_sigmoid_gate": [P, I, P, I, P, I, I, I, I, P],
        "vx_rmsnorm_rows": [P, I, P, P, I, I, F, I, P],
        "vx_gemm_few_rows_batched": [P, P, P, I, I, I, I, I, I, I, c_longlong, c_longlong, c_longlong, I, P],
        "vx_biased_attention_shared": [P, I, P, P, P, I, P, P, P, P, P, I, F, F, I, I, I, I, I, I, I, I, I, P, I, P, I, F, I, I, P],
        "vx_biased_attention_rows_window": [P, I, P, c_longlong, c_longlong, P, c_longlong, c_longlong, P, I, P, P, P, P, I, F, I, I,
                                            I, I, I, I, I, F, I, P],
        "vx_latent_gather_window": [P, P, I, P, P, P, P, I, P, I, I, I, I, I, I, I, P],
    }
    lib.vx_set_pdl_mask.argtypes = [I]
    lib.vx_set_pdl_mask.restype = None
    lib.vx_set_pdl.argtypes = [I]
    lib.vx_set_pdl.restype = None
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int


_LAUNCHES = 0


def launch_count() -> int:
    """Calls of this library's kernels so far (library matrix products are not counted)."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    """Kernels launched by replaying a captured graph (counted at capture)."""
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, what: str) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if code == 0:
        return
    if code < 0:
        raise KernelError("%s refused: %s (code %d)" % (what, _ERRORS.get(code, "unknown"), code))
    raise KernelError("%s: CUDA error %d at launch" % (what, code))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_GET_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (the capture stream while a graph is recorded).
    Asked of torch's C layer directly: the Python route costs 15 microseconds a call,
    and every kernel launch asks."""
    if _RAW_STREAM is not None and _GET_DEVICE is not None:
        return _RAW_STREAM(_GET_DEVICE())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return VX_F32
    if dtype == torch.bfloat16:
        return VX_BF16
    raise KernelError("element type %s has no kernels (float32 and bfloat16 have)" % dtype)


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _dev(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors; got one on %s" % t.device)


# ----------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0,
              rounded: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 rows of `table` [V,E] at int32 `ids` [T], times `scale`; `rounded` [T,E] (the table's element
    type) takes the same rows rounded."""
    _dev(ids, table, rounded)
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and table.is_contiguous(), "embedding: int32 ids, contiguous")
    t, (v, e) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((t, e), dtype=torch.float32, device=table.device)
    if rounded is not None:
        _need(rounded.dtype == table.dtype and rounded.is_contiguous() and tuple(rounded.shape) == (t, e),
              "embedding: the rounded copy has the table's element type and the result's shape")
    _check(library().vx_embedding(_ptr(ids), _ptr(table), _ptr(out), t, e, v, dtype_code(table.dtype), float(scale),
                                  _ptr(rounded), _stream()), "embedding")
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                residual_out: Optional[torch.Tensor] = None, update_residual: bool = True) -> torch.Tensor:
    """normed = rmsnorm(residual (+ delta)) rounded to `out_dtype`.

    With a delta, the residual must be older than the delta: not something the
    kernel launched just before this one writes (the kernel reads it before it
    waits for that kernel; in a decoder the delta is computed from the residual,
    so this holds by itself).

    Without `rows` the sum is written back into `residual` (if there is a delta
    and `update_residual`).  With `rows` (int32 indices) only those rows are
    read, and the sums go to `residual_out` if given."""
    _dev(residual, delta, weight, rows)
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "add_rmsnorm: float32 contiguous residual")
    _need(weight.dtype == torch.float32, "add_rmsnorm: float32 weight")
    width = residual.shape[-1]
    _need(weight.numel() == width, "add_rmsnorm: weight has %d elements, rows %d" % (weight.numel(), width))
    if delta is not None:
        _need(delta.dtype == out_dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "add_rmsnorm: delta must match the residual's shape and the output's element type")
    n = residual.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, width), dtype=out_dtype, device=residual.device)
    if rows is None:
        res_out = residual if (delta is not None and update_residual) else None
    else:
        _need(rows.dtype == torch.int32, "add_rmsnorm: int32 rows")
        res_out = residual_out
    _check(library().vx_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(rows), _ptr(res_out), _ptr(weight), _ptr(out),
                                    n, width, float(eps), dtype_code(out_dtype), _stream()), "add_rmsnorm")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm of the rows of x times `weight`; a matrix whose rows are contiguous may be a slice of wider rows."""
    _dev(x, weight)
    width = x.shape[-1]
    _need(weight.dtype == torch.float32 and (x.is_contiguous() or (x.dim() == 2 and x.stride(1) == 1)),
          "rmsnorm: contiguous rows, float32 weight")
    _need(weight.numel() == width, "rmsnorm: weight has %d elements, rows %d" % (weight.numel(), width))
    out = torch.empty(tuple(x.shape), dtype=x.dtype, device=x.device)
    ldx = width if x.is_contiguous() else x.stride(0)
    _check(library().vx_rmsnorm_rows(_ptr(x), ldx, _ptr(weight), _ptr(out), x.numel() // width, width, float(eps),
                                     dtype_code(x.dtype), _stream()), "rmsnorm")
    return out


def gated_act(gate_up: torch.Tensor, activation: str, block: int = 0,
              out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(gate) * up.  block == 0: rows are [all gates | all ups]; block > 0: rows
    are tiles of `block` gates followed by their `block` ups.  float32 input may give a
    bfloat16 result (`out_dtype`)."""
    _dev(gate_up)
    _need(gate_up.is_contiguous() and gate_up.shape[-1] % 2 == 0, "gated_act: contiguous rows of even width")
    _need(activation in ACTIVATIONS, "gated_act: activation %r is not one of %s" % (activation, sorted(ACTIVATIONS)))
    rows, inner = gate_up.shape[0], gate_up.shape[-1] // 2
    out = torch.empty((rows, inner), dtype=out_dtype or gate_up.dtype, device=gate_up.device)
    _check(library().vx_gated_act(_ptr(gate_up), _ptr(out), rows, inner, ACTIVATIONS[activation], int(block),
                                  dtype_code(gate_up.dtype), dtype_code(out.dtype), _stream()), "gated_act")
    return out


def qk_norm_rope_kv(qkv: torch.Tensor, q_weight, k_weight, eps: float, inv_freq, rot_dim: int,
                    positions: torch.Tensor, slot_mapping, k_pool, v_pool, num_heads: int, num_kv_heads: int,
                    head_dim: int, v_head_dim: int = 0, interleaved: bool = False, num_v_heads: int = 0,
                    magnitude: float = 1.0) -> None:
    """In place on the packed projections `qkv` [T, (H+Hk)D + Hv Dv (+ more)]; writes new keys
    and values into the pools [pages, Hk, S, D] and [pages, Hv, S, Dv] when a slot mapping is given
    (`v_head_dim` 0: values of the keys' size; `num_v_heads` 0: as many value heads as key heads).  The rotation pairs
    channel i with i + rot_dim/2, or, when `interleaved`, channel 2i with 2i + 1; cosines and sines are multiplied by
    `magnitude`."""
    v_head_dim = int(v_head_dim) or head_dim
    num_v_heads = int(num_v_heads) or num_kv_heads
    _dev(qkv, q_weight, k_weight, inv_freq, positions, slot_mapping, k_pool, v_pool)
    _need(qkv.is_contiguous() and positions.dtype == torch.int32, "qk_norm_rope_kv: contiguous qkv, int32 positions")
    page_size = 1
    if slot_mapping is not None:
        _need(k_pool is not None and v_pool is not None and k_pool.dtype == qkv.dtype and k_pool.is_contiguous()
              and v_pool.is_contiguous(), "qk_norm_rope_kv: pools of the activations' element type")
        _need(tuple(k_pool.shape[1:]) == (num_kv_heads, k_pool.shape[2], head_dim)
              and tuple(v_pool.shape[1:]) == (num_v_heads, k_pool.shape[2], v_head_dim), "qk_norm_rope_kv: pool shape")
        page_size = k_pool.shape[2]
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dim, "qk_norm_rope_kv: inv_freq size")
    for w in (q_weight, k_weight):
        if w is not None:
            _need(w.dtype == torch.float32 and w.numel() == head_dim, "qk_norm_rope_kv: norm weight size")
    _check(library().vx_qk_norm_rope_kv_shared(
        _ptr(qkv), qkv.shape[-1], _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(inv_freq), int(rot_dim),
        _ptr(positions), _ptr(slot_mapping), _ptr(k_pool), _ptr(v_pool), qkv.shape[0], num_heads, num_kv_heads,
        head_dim, page_size, dtype_code(qkv.dtype), v_head_dim, 1 if interleaved else 0, num_v_heads, float(magnitude),
        _stream()), "qk_norm_rope_kv")


ATTENTION_MAX_HEAD_DIM = 256


def attention_head_dim_supported(head_dim: int) -> bool:
    """Head sizes some attention kernel of the library takes: even ones up to 256 (the general
    kernel; the tensor-core kernels take 64 and 128)."""
    return 0 < head_dim <= ATTENTION_MAX_HEAD_DIM and head_dim % 2 == 0


def paged_attention_generic(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                            seq_of_token, positions, scale: float, window: int, num_heads: int,
                            num_kv_heads: int, head_dim: int, tokens: int, v_head_dim: int = 0, keep_first: int = 0,
                            bias_exponent: float = 0.0, sinks: Optional[torch.Tensor] = None,
                            gate_col: int = -1, softcap: float = 0.0, v_stride: int = 0, v_share: int = 1,
                            out_float32: bool = False) -> torch.Tensor:
    """The general kernel.  `v_head_dim`: size of a value (0: a key's); `keep_first`: with a window, the
    first positions that stay visible; `bias_exponent` b > 0: head h's scores lose
    2^(-b (h + 1) / heads) * distance; `sinks` (float32 per head): the softmax's denominator also holds
    exp(sink); `gate_col` >= 0: head h's output times sigmoid of column gate_col + h of the token's row of `q`;
    `softcap` c > 0: a scaled score s becomes c tanh(s / c); `v_stride`: elements from one value row of
    `v_pool` to the next (0: v_head_dim), for a pool whose rows hold the value inside the key's row; `v_share` > 1: that
    many consecutive key heads read one value head (the value pool has num_kv_heads / v_share heads); `out_float32`: the
    result is float32 whatever the queries' element type."""
    _dev(q, k_pool, v_pool, block_table, seq_of_token, positions, sinks)
    _need(v_share >= 1 and num_kv_heads % v_share == 0, "paged_attention: v_share must divide the key heads")
    _check_sinks_gate("paged_attention", sinks, gate_col, num_heads, q_row_stride)
    v_head_dim = int(v_head_dim) or head_dim
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_attention: int32 block table [requests, blocks]")
    _need(k_pool.dtype == q.dtype and v_pool.dtype == q.dtype, "paged_attention: pools of the queries' element type")
    page_size = k_pool.shape[-2]
    _need(0 < head_dim <= ATTENTION_MAX_HEAD_DIM and 0 < v_head_dim <= ATTENTION_MAX_HEAD_DIM,
          "paged_attention: head sizes %d / %d (the general kernel takes sizes up to %d)"
          % (head_dim, v_head_dim, ATTENTION_MAX_HEAD_DIM))
    out = torch.empty((tokens, num_heads * v_head_dim), dtype=torch.float32 if out_float32 else q.dtype, device=q.device)
    _check(library().vx_paged_attention_generic_shared(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(seq_of_token), _ptr(positions), _ptr(out), num_heads * v_head_dim, float(scale), int(window), tokens,
        num_heads, num_kv_heads, head_dim, page_size, dtype_code(q.dtype), v_head_dim, int(keep_first),
        float(bias_exponent), _ptr(sinks), int(gate_col), float(softcap), int(v_stride), int(v_share),
        1 if out_float32 else 0, _stream()), "paged_attention_generic")
    return out


def _check_sinks_gate(what: str, sinks, gate_col: int, num_heads: int, q_row_stride: int) -> None:
    if sinks is not None:
        _need(sinks.dtype == torch.float32 and sinks.is_contiguous() and sinks.numel() == num_heads,
              "%s: one float32 sink per query head" % what)
    _need(gate_col < 0 or gate_col + num_heads <= q_row_stride, "%s: the gates' columns lie outside the row" % what)


BIASED_DECODE_MAX_RUNS = 8


BIASED_ATTENTION_EQUAL_SIZES = (32, 48, 80, 96, 112)


def biased_attention_supported(dtype, head_dim: int, v_head_dim: int, page_size: int) -> bool:
    """What the tensor-core kernels for attention with a bias by distance, a window with kept first positions,
    values of another size than keys, a sink and an output gate take: keys of 64 or 128 with values of 32, 64 or
    128, or keys and values of one size out of 32, 48, 80, 96, 112."""
    sizes = (head_dim in (64, 128) and v_head_dim in (32, 64, 128)) or \
        (head_dim == v_head_dim and head_dim in BIASED_ATTENTION_EQUAL_SIZES)
    return dtype == torch.bfloat16 and sizes and page_size % 16 == 0


def _biased_attention(q, q_row_stride, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, seq_of_token, positions,
                      scale, window, keep_first, bias_exponent, num_heads, num_kv_heads, head_dim, v_head_dim, segments,
                      max_new, tokens, out, max_kv=0, sinks=None, gate_col=-1, softcap=0.0, v_share=1, out_float32=False):
    _dev(q, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, seq_of_token, positions, out, sinks)
    _need(v_share >= 1 and num_kv_heads % v_share == 0 and v_pool.shape[1] * v_share == k_pool.shape[1] == num_kv_heads,
          "biased_attention: value heads times v_share must be the key heads")
    _check_sinks_gate("biased_attention", sinks, gate_col, num_heads, q_row_stride)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "biased_attention: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "biased_attention: int32 block table [requests, blocks]")
    _need(k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.shape[3] == head_dim and v_pool.shape[3] == v_head_dim,
          "biased_attention: pools [pages, kv heads, page size, head size]")
    if out is None:
        out = torch.empty((tokens, num_heads * v_head_dim), dtype=torch.float32 if out_float32 else q.dtype, device=q.device)
    _need(out.dtype == (torch.float32 if out_float32 else q.dtype), "biased_attention: the output's element type")
    # single tokens with many visible keys: the keys cut into runs of at least 16 groups of 16, 8 runs at most
    runs, scratch = 1, None
    if cu_seqlens is None and max_kv > 0:
        keys = max_kv if window <= 0 else min(max_kv, window + keep_first)
        runs = max(1, min(BIASED_DECODE_MAX_RUNS, -(-keys // 16) // 16))
        if runs > 1:
            scratch = workspace(q.device, tokens * num_heads * runs * (v_head_dim + 2), which="biased_decode")
    _check(library().vx_biased_attention_shared(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1], _ptr(cu_seqlens),
        _ptr(kv_offsets), _ptr(seq_of_token), _ptr(positions), _ptr(out), num_heads * v_head_dim, float(scale),
        float(bias_exponent), int(window), int(keep_first), int(segments), int(max_new), num_heads, num_kv_heads, head_dim,
        v_head_dim, k_pool.shape[2], _ptr(scratch), runs, _ptr(sinks), int(gate_col), float(softcap), int(v_share),
        1 if out_float32 else 0, _stream()), "biased_attention")
    return out


def biased_prefill_attention(q, q_row_stride, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, scale: float,
                             window: int, keep_first: int, bias_exponent: float, num_heads: int, num_kv_heads: int,
                             head_dim: int, v_head_dim: int, requests: int, max_new: int, tokens: int, out=None,
                             sinks=None, gate_col: int = -1, softcap: float = 0.0, v_share: int = 1, out_float32: bool = False):
    """Attention of prompt portions (request i: rows cu_seqlens[i] .. at positions kv_offsets[i] ..) with
    score = q.k * scale - 2^(-bias_exponent (h+1) / heads) * distance under a window that keeps the first
    `keep_first` positions; bfloat16, tensor cores, probabilities in two bfloat16 halves.  `sinks`, `gate_col` and
    `softcap`, `v_share` and `out_float32` as in `paged_attention_generic`."""
    return _biased_attention(q, q_row_stride, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, None, None, scale,
                             window, keep_first, bias_exponent, num_heads, num_kv_heads, head_dim, v_head_dim, requests,
                             max_new, tokens, out, sinks=sinks, gate_col=gate_col, softcap=softcap, v_share=v_share,
                             out_float32=out_float32)


def biased_decode_attention(q, q_row_stride, k_pool, v_pool, block_table, seq_of_token, positions, scale: float,
                            window: int, keep_first: int, bias_exponent: float, num_heads: int, num_kv_heads: int,
                            head_dim: int, v_head_dim: int, tokens: int, out=None, max_kv: int = 0, sinks=None,
                            gate_col: int = -1, softcap: float = 0.0, v_share: int = 1, out_float32: bool = False):
    """The same for token rows that each stand alone: row t is request seq_of_token[t] at position positions[t].
    `max_kv` (a bound on any row's position + 1; 0: unknown) lets rows with many visible keys be cut into runs that
    several blocks share."""
    return _biased_attention(q, q_row_stride, k_pool, v_pool, block_table, None, None, seq_of_token, positions, scale,
                             window, keep_first, bias_exponent, num_heads, num_kv_heads, head_dim, v_head_dim, tokens, 1,
                             tokens, out, max_kv=max_kv, sinks=sinks, gate_col=gate_col, softcap=softcap, v_share=v_share,
                             out_float32=out_float32)


def embedding_pair(ids, positions, seq_of_token, cu_seqlens, state_slots, last_token: torch.Tensor,
                   table: torch.Tensor, pair_table: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """float32 rows table[id] + pair_table[(previous id * mul_prev + id * mul_cur) mod buckets] (row `buckets`
    at position 0).  The id before a step's first is read from `last_token` [slots] (int32), which then
    takes the request's last id of this step."""
    _dev(ids, positions, seq_of_token, cu_seqlens, state_slots, last_token, table, pair_table)
    _need(ids.dtype == torch.int32 and last_token.dtype == torch.int32 and last_token.is_contiguous(),
          "embedding_pair: int32 ids and last tokens")
    _need(table.is_contiguous() and pair_table.is_contiguous() and table.dtype == pair_table.dtype
          and pair_table.shape == (buckets + 1, table.shape[1]), "embedding_pair: tables [V,E] and [buckets+1,E]")
    t, (v, e) = ids.numel(), table.shape
    out = torch.empty((t, e), dtype=torch.float32, device=table.device)
    _check(library().vx_embedding_pair(_ptr(ids), _ptr(positions), _ptr(seq_of_token), _ptr(cu_seqlens), _ptr(state_slots),
                                       _ptr(last_token), _ptr(table), _ptr(pair_table), _ptr(out), t, e, v, int(buckets),
                                       int(mul_prev), int(mul_cur), dtype_code(table.dtype), _stream()), "embedding_pair")
    return out


def merge_norm_add_norm(residual: torch.Tensor, y0: torch.Tensor, w_post: torch.Tensor, mult: float, eps: float,
                        w0=None, c0: float = 1.0, y1=None, w1=None, c1: float = 1.0, w_next=None, rounded: bool = False):
    """residual (float32, in place) += mult * rmsnorm(u) * w_post, with u = y0, or with two branches
    u = c0 rmsnorm(y0) w0 + c1 rmsnorm(y1) w1.  Returns rmsnorm(residual) * w_next in y0's element type
    if `w_next` is given; with `rounded` the new residual itself in y0's element type (for a next sublayer
    that reads the stream without a norm before it); else None."""
    _dev(residual, y0, w_post, w0, y1, w1, w_next)
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and y0.is_contiguous()
          and y0.shape == residual.shape, "merge_norm_add_norm: float32 residual, a branch of its shape")
    width = residual.shape[-1]
    for w in (w_post, w0, w1, w_next):
        if w is not None:
            _need(w.dtype == torch.float32 and w.numel() == width, "merge_norm_add_norm: float32 weights of the row's width")
    if y1 is not None:
        _need(y1.is_contiguous() and y1.shape == y0.shape and y1.dtype == y0.dtype and w0 is not None and w1 is not None,
              "merge_norm_add_norm: two branches of one shape, each with its weight")
    _need(not (rounded and w_next is not None), "merge_norm_add_norm: the next norm or the rounded stream, not both")
    out = torch.empty_like(y0) if (w_next is not None or rounded) else None
    _check(library().vx_merge_norm_add_norm(_ptr(residual), _ptr(y0), _ptr(w0), float(c0), _ptr(y1), _ptr(w1), float(c1),
                                            _ptr(w_post), float(mult), _ptr(w_next), _ptr(out), residual.shape[0], width,
                                            float(eps), dtype_code(y0.dtype), _stream()), "merge_norm_add_norm")
    return out


def merge_norms(y0: torch.Tensor, w0: torch.Tensor, c0: float, y1: torch.Tensor, w1: torch.Tensor, c1: float,
                eps: float) -> torch.Tensor:
    """c0 rmsnorm(y0) w0 + c1 rmsnorm(y1) w1, in the branches' element type."""
    _dev(y0, w0, y1, w1)
    width = y0.shape[-1]
    _need(y0.is_contiguous() and y1.is_contiguous() and y0.shape == y1.shape and y0.dtype == y1.dtype
          and w0.dtype == torch.float32 and w1.dtype == torch.float32 and w0.numel() == width and w1.numel() == width,
          "merge_norms: two branches of one shape, float32 weights of the row's width")
    out = torch.empty_like(y0)
    _check(library().vx_merge_norm_add_norm(None, _ptr(y0), _ptr(w0), float(c0), _ptr(y1), _ptr(w1), float(c1), None, 1.0,
                                            None, _ptr(out), y0.shape[0], width, float(eps), dtype_code(y0.dtype), _stream()),
           "merge_norms")
    return out


def act(x: torch.Tensor, activation: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """activation(x), element by element; x [rows, width] with contiguous rows."""
    _dev(x)
    _need(x.dim() == 2 and x.stride(1) == 1, "act: rows must be contiguous")
    _need(activation in ACTIVATIONS, "act: activation %r is not one of %s" % (activation, sorted(ACTIVATIONS)))
    out = torch.empty(x.shape, dtype=out_dtype or x.dtype, device=x.device)
    _check(library().vx_act(_ptr(x), x.stride(0), _ptr(out), x.shape[0], x.shape[1], ACTIVATIONS[activation],
                            dtype_code(x.dtype), dtype_code(out.dtype), _stream()), "act")
    return out


def cast_rows(x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [rows, width] (contiguous rows) in another element type, rounded to nearest."""
    _dev(x)
    _need(x.dim() == 2 and x.stride(1) == 1, "cast_rows: rows must be contiguous")
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _check(library().vx_act(_ptr(x), x.stride(0), _ptr(out), x.shape[0], x.shape[1], _ACT_IDENTITY,
                            dtype_code(x.dtype), dtype_code(out.dtype), _stream()), "cast_rows")
    return out


def scale_rows(x: torch.Tensor, scale: float) -> torch.Tensor:
    """float32 x [rows, n] times a number."""
    _dev(x)
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "scale_rows: float32 rows")
    out = torch.empty_like(x)
    _check(library().vx_add_bias(_ptr(x), None, _ptr(out), x.shape[0], x.shape[1], VX_F32, float(scale), _stream()), "scale_rows")
    return out


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """rmsnorm(o) * weight * sigmoid(gate): o float32 [rows, width]; gate [rows, width] with contiguous rows
    in the element type of the result."""
    _dev(o, gate, weight)
    _need(o.dtype == torch.float32 and o.is_contiguous() and gate.stride(1) == 1 and gate.shape == o.shape
          and weight.dtype == torch.float32 and weight.numel() == o.shape[1], "gated_rmsnorm: shapes and element types")
    out = torch.empty(o.shape, dtype=gate.dtype, device=o.device)
    _check(library().vx_gated_rmsnorm(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), o.shape[0], o.shape[1],
                                      float(eps), dtype_code(gate.dtype), _stream()), "gated_rmsnorm")
    return out


def kv_store(x: torch.Tensor, k_col: int, v_col: int, slot_mapping, k_pool, v_pool) -> None:
    """Keys [Hk, Dk] at column `k_col` and values [Hk, Dv] at column `v_col` of every row of the packed
    projection `x` into the pools [pages, Hk, S, Dk] and [pages, Hk, S, Dv]."""
    _dev(x, slot_mapping, k_pool, v_pool)
    _need(x.stride(1) == 1 and k_pool.dtype == x.dtype and v_pool.dtype == x.dtype and k_pool.is_contiguous()
          and v_pool.is_contiguous() and k_pool.shape[:3] == v_pool.shape[:3], "kv_store: pools of the rows' element type")
    _check(library().vx_kv_store(_ptr(x), x.stride(0), int(k_col), int(v_col), _ptr(slot_mapping), _ptr(k_pool), _ptr(v_pool),
                                 x.shape[0], k_pool.shape[1], k_pool.shape[3], v_pool.shape[3], k_pool.shape[2],
                                 dtype_code(x.dtype), _stream()), "kv_store")


def linear_attention_recurrent(x: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor,
                               state: torch.Tensor, cu_seqlens, state_slots, seqs: int, heads: int, dim: int,
                               vdim: int, silu: bool = True) -> torch.Tensor:
    """Per head S = decay S + k v^T, o = S^T q over every request's tokens in order; q, k [heads, dim] and
    v [heads, vdim] at columns of the packed projection `x`; `state` float32 [slots, heads, dim, vdim] is
    read and written back.  Returns float32 [tokens, heads * vdim]."""
    _dev(x, decay, state, cu_seqlens, state_slots)
    _need(x.stride(1) == 1 and decay.dtype == torch.float32 and decay.numel() == heads, "linear_attention: float32 decay per head")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "linear_attention: float32 state [slots, heads, dim, vdim]")
    out = torch.empty((x.shape[0], heads * vdim), dtype=torch.float32, device=x.device)
    _check(library().vx_linear_attention_recurrent(_ptr(x), x.stride(0), int(q_col), int(k_col), int(v_col), _ptr(decay),
                                                   _ptr(state), _ptr(cu_seqlens), _ptr(state_slots), _ptr(out), int(seqs),
                                                   heads, dim, vdim, 1 if silu else 0, dtype_code(x.dtype), _stream()),
           "linear_attention_recurrent")
    return out


LINEAR_ATTENTION_MAX_DIM = 256


LINEAR_ATTENTION_CHUNKED_MIN_TOKENS = 32   # longest portion of a step from which the chunked kernel is used
LINEAR_ATTENTION_PARALLEL_MIN_TOKENS = 256  # ... from which the chunks are worked on side by side


def linear_attention_chunked_supported(dtype, dim: int, vdim: int) -> bool:
    return dtype == torch.bfloat16 and dim in (32, 64, 128) and vdim % 32 == 0


def linear_attention(x: torch.Tensor, q_col: int, k_col: int, v_col: int, decay: torch.Tensor, state: torch.Tensor,
                     cu_seqlens, state_slots, seqs: int, max_new: int, heads: int, dim: int, vdim: int,
                     silu: bool = True) -> torch.Tensor:
    """Decayed linear attention of a step's tokens against the requests' states (see
    `linear_attention_recurrent`); `max_new` bounds the tokens of any request.  A bfloat16 step with a portion of
    `LINEAR_ATTENTION_CHUNKED_MIN_TOKENS` tokens or more runs in chunks of 64 tokens on the tensor cores (the
    activation first, by a kernel of its own, rounded to bfloat16 as the recurrent kernel rounds it)."""
    width = 2 * heads * dim + heads * vdim
    if (max_new >= LINEAR_ATTENTION_CHUNKED_MIN_TOKENS and linear_attention_chunked_supported(x.dtype, dim, vdim)
            and k_col == q_col + heads * dim and v_col == k_col + heads * dim and q_col + width <= x.shape[1]):
        _dev(x, decay, state, cu_seqlens, state_slots)
        _need(decay.dtype == torch.float32 and decay.numel() == heads, "linear_attention: float32 decay per head")
        _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
              "linear_attention: float32 state [slots, heads, dim, vdim]")
        qkv = act(x[:, q_col:q_col + width], "silu") if silu else x[:, q_col:q_col + width]
        if qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0:
            out = torch.empty((x.shape[0], heads * vdim), dtype=torch.float32, device=x.device)
            if max_new >= LINEAR_ATTENTION_PARALLEL_MIN_TOKENS:
                # long portions: every chunk's own contribution, a scan over the chunks, every chunk's outputs
                max_chunks = x.shape[0] // 64 + int(seqs)
                scratch = workspace(x.device, max_chunks * heads * dim * vdim, which="linear_attention")
                _check(library().vx_linear_attention_parallel(
                    _ptr(qkv), qkv.stride(0), 0, heads * dim, 2 * heads * dim, _ptr(decay), _ptr(state), _ptr(scratch),
                    _ptr(cu_seqlens), _ptr(state_slots), _ptr(out), int(seqs), max_chunks, heads, dim, vdim, _stream()),
                    "linear_attention_parallel")
                return out
            _check(library().vx_linear_attention_chunked(_ptr(qkv), qkv.stride(0), 0, heads * dim, 2 * heads * dim, _ptr(decay),
                                                         _ptr(state), _ptr(cu_seqlens), _ptr(state_slots), _ptr(out),
                                                         int(seqs), heads, dim, vdim, _stream()), "linear_attention_chunked")
            return out
    return linear_attention_recurrent(x, q_col, k_col, v_col, decay, state, cu_seqlens, state_slots, seqs, heads, dim,
                                      vdim, silu)


MOE_TILE_ROWS = 64            # row tiles of the mma.sync grouped product
MOE_SMALL_TILE_ROWS = 16      # ... for steps of few tokens (decode)
MOE_SMALL_MAX_ROWS = 256      # assignments of a step up to which the small tiles are used
MOE_TCGEN05_TILE_ROWS = 128   # ... of the tcgen05 one
MOE_TCGEN05_MIN_ROWS = 1024   # assignments of a step from which the tcgen05 grouped product is used


class MoePlan:
    """What `moe_route` leaves on the device for the grouped products and the combination."""
    __slots__ = ("chosen", "weight", "tiles", "n_tiles", "src_of_row", "row_of", "max_tiles", "top", "assignments",
                 "tile_rows", "experts", "identity", "shared_gate")


_MOE_COUNTS = {}


def moe_route(h: torch.Tensor, w_router: torch.Tensor, bias, experts: int, top: int,
              tile_rows: int = MOE_TILE_ROWS, scores: str = "softmax_chosen", correction=None, groups: int = 1,
              keep_groups: int = 1, route_scale: float = 1.0, identity: int = 0, shared_gate: bool = False) -> MoePlan:
    """Router logits in float32, the `top` largest per token, softmax over the chosen; then every
    assignment's row in expert order and the row tiles (of up to `tile_rows` rows) of the grouped products.

    `experts` counts the router's outputs.  `scores="softmax_all"`: scores s = softmax over all outputs, choice by
    s + `correction` (float32 per output) among the outputs of the `keep_groups` best of `groups` equal groups of
    neighbours, weights s * route_scale (not renormalised).  The last `identity` outputs are identity experts (the
    combination takes the token's own row for them).  With `shared_gate` the router's matrix has one more row, and
    `plan.shared_gate` [tokens] is sigmoid(that row . h)."""
    _dev(h, w_router, bias, correction)
    rows = experts + (1 if shared_gate else 0)
    _need(h.stride(1) == 1 and w_router.dtype == torch.float32 and w_router.is_contiguous()
          and tuple(w_router.shape) == (rows, h.shape[1]), "moe_route: float32 router [outputs (+ 1 for a shared gate), width]")
    _need(scores in ("softmax_chosen", "softmax_all"), "moe_route: scores %r" % (scores,))
    _need(groups >= 1 and experts % groups == 0 and 1 <= keep_groups <= groups and top <= keep_groups * (experts // groups)
          and 0 <= identity < experts, "moe_route: groups, kept groups, top and identity experts do not fit the outputs")
    for b in (bias, correction):
        if b is not None:
            _need(b.dtype == torch.float32 and b.numel() == experts, "moe_route: float32 bias / correction per output")
    t, dev = h.shape[0], h.device
    a = t * top
    plan = MoePlan()
    plan.top, plan.assignments, plan.tile_rows, plan.experts, plan.identity = top, a, int(tile_rows), experts, int(identity)
    plan.shared_gate = torch.empty(t, dtype=torch.float32, device=dev) if shared_gate else None
    plan.max_tiles = -(-a // plan.tile_rows) + experts
    ints = torch.empty(3 * a + (experts + 1) + 3 * plan.max_tiles + 1 + a, dtype=torch.int32, device=dev)
    plan.chosen, pos, plan.src_of_row, plan.row_of = ints[:a], ints[a:2 * a], ints[2 * a:3 * a], ints[3 * a:4 * a]
    rest = ints[4 * a:]
    offsets, plan.tiles, plan.n_tiles = rest[:experts + 1], rest[experts + 1:experts + 1 + 3 * plan.max_tiles], rest[-1:]
    plan.weight = torch.empty((t, top), dtype=torch.float32, device=dev)
    key = (str(dev), experts)
    counts = _MOE_COUNTS.get(key)
    if counts is None or torch.cuda.is_current_stream_capturing():
        counts = torch.zeros(experts, dtype=torch.int32, device=dev)   # (the plan kernel leaves it zero again)
        if not torch.cuda.is_current_stream_capturing():
            _MOE_COUNTS[key] = counts
    _check(library().vx_moe_route(_ptr(h), h.stride(0), _ptr(w_router), _ptr(bias), t, h.shape[1], experts, top,
                                  plan.tile_rows, _ptr(plan.chosen), _ptr(plan.weight), _ptr(counts), _ptr(pos), _ptr(offsets),
                                  _ptr(plan.tiles), _ptr(plan.n_tiles), _ptr(plan.src_of_row), _ptr(plan.row_of),
                                  dtype_code(h.dtype), 1 if scores == "softmax_all" else 0, _ptr(correction), int(groups),
                                  int(keep_groups), float(route_scale), int(identity), _ptr(plan.shared_gate), _stream()),
           "moe_route")
    return plan


def moe_gemm(a: torch.Tensor, w: torch.Tensor, plan: MoePlan, gather: bool, out_dtype: torch.dtype,
             gated_activation: Optional[str] = None) -> torch.Tensor:
    """Grouped product in expert order: row p of the result is a[src(p)] times w[expert of p] transposed, with
    w [experts, N, K]; src(p) is the token of assignment p (`gather`) or p itself.  With `gated_activation`,
    w's rows come in tiles of 8 gate rows followed by their 8 up rows and the result is act(gate) * up."""
    _dev(a, w)
    _need(a.stride(1) == 1 and w.is_contiguous() and w.dim() == 3 and w.shape[2] == a.shape[1] and a.dtype == w.dtype,
          "moe_gemm: a [rows, K], w [experts, N, K] of one element type")
    n, k = w.shape[1], w.shape[2]
    cols = n // 2 if gated_activation else n
    out = torch.empty((plan.assignments, cols), dtype=out_dtype, device=a.device)
    tc = moe_mma_supported(a, k) and w.data_ptr() % 16 == 0
    _need(plan.tile_rows == MOE_TILE_ROWS or (plan.tile_rows == MOE_SMALL_TILE_ROWS and tc),
          "moe_gemm: row tiles of %d, or of %d on the tensor cores" % (MOE_TILE_ROWS, MOE_SMALL_TILE_ROWS))
    _check(library().vx_moe_gemm(_ptr(a), a.stride(0), _ptr(plan.src_of_row) if gather else None, plan.top if gather else 1,
                                 _ptr(w), _ptr(plan.tiles), _ptr(plan.n_tiles), plan.max_tiles, _ptr(out), cols, n, k,
                                 1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0), dtype_code(a.dtype),
                                 dtype_code(out_dtype), 1 if tc else 0, plan.tile_rows, _stream()), "moe_gemm")
    return out


def moe_mma_supported(a: torch.Tensor, k: int) -> bool:
    return a.dtype == torch.bfloat16 and k % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0


def moe_tile_rows(h: torch.Tensor, assignments: int) -> int:
    """Row tiles for the `mma.sync` grouped products of a step: 16 rows for a handful of tokens, else 64."""
    small = assignments <= MOE_SMALL_MAX_ROWS and moe_mma_supported(h, h.shape[1])
    return MOE_SMALL_TILE_ROWS if small else MOE_TILE_ROWS


def moe_tcgen05_supported(h: torch.Tensor, assignments: int, n: int, k: int) -> bool:
    """Whether a step's grouped products run on the tcgen05 tensor cores: bfloat16, enough rows, K a multiple of
    8 and N of 16."""
    return (h.dtype == torch.bfloat16 and assignments >= MOE_TCGEN05_MIN_ROWS and k % 8 == 0 and n % 16 == 0
            and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0)


def moe_gather_rows(x: torch.Tensor, plan: MoePlan) -> torch.Tensor:
    """The tokens' rows of `x` in expert order, one per assignment."""
    _dev(x)
    _need(x.stride(1) == 1 and x.shape[1] % 8 == 0 and x.element_size() == 2, "moe_gather_rows: 16-bit rows of 8 n elements")
    out = torch.empty((plan.assignments, x.shape[1]), dtype=x.dtype, device=x.device)
    _check(library().vx_moe_gather_rows(_ptr(x), x.stride(0), _ptr(plan.src_of_row), plan.top, _ptr(out), plan.assignments,
                                        x.shape[1], _stream()), "moe_gather_rows")
    return out


def moe_gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, plan: MoePlan, gated_activation: Optional[str] = None) -> torch.Tensor:
    """The grouped product on the tcgen05 tensor cores: `a` [assignments, K] bfloat16 IN EXPERT ORDER, w [experts, N, K];
    the plan's row tiles must be of `MOE_TCGEN05_TILE_ROWS` rows.  bfloat16 out."""
    _dev(a, w)
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and w.dim() == 3
          and a.shape == (plan.assignments, w.shape[2]) and plan.tile_rows == MOE_TCGEN05_TILE_ROWS,
          "moe_gemm_tcgen05: bfloat16 a [assignments, K] in expert order, w [experts, N, K], row tiles of 128")
    n, k = w.shape[1], w.shape[2]
    cols = n // 2 if gated_activation else n
    out = torch.empty((plan.assignments, cols), dtype=torch.bfloat16, device=a.device)
    _check(library().vx_moe_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(out), plan.assignments, w.shape[0], n, k, a.stride(0), cols,
                                         1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0), _ptr(plan.tiles),
                                         _ptr(plan.n_tiles), plan.max_tiles, _ptr(_error_word(a.device)), _stream()),
           "moe_gemm_tcgen05")
    note_bounded_wait()
    return out


def moe_combine(y: torch.Tensor, plan: MoePlan, shared_out, out_dtype: torch.dtype, h=None) -> torch.Tensor:
    """Per token the weighted sum of its experts' rows of `y` (expert order; float32, or the result's element
    type), plus `shared_out` (times the plan's shared gate, if it has one).  A plan with identity experts needs
    `h`, the tokens' rows that went into the router: an assignment to one of them adds weight * h[t]."""
    _dev(y, shared_out, h)
    if plan.identity:
        _need(h is not None and h.dtype == out_dtype and h.stride(1) == 1 and h.shape[1] == y.shape[1],
              "moe_combine: identity experts take the tokens' own rows, in the result's element type")
    _need(y.dtype in (torch.float32, out_dtype) and y.is_contiguous(), "moe_combine: float32 rows, or rows of the result's type")
    t = plan.assignments // plan.top
    if shared_out is not None:
        _need(shared_out.dtype == out_dtype and shared_out.is_contiguous() and tuple(shared_out.shape) == (t, y.shape[1]),
              "moe_combine: the shared expert's output in the result's shape and element type")
    out = torch.empty((t, y.shape[1]), dtype=out_dtype, device=y.device)
    _check(library().vx_moe_combine(_ptr(y), _ptr(plan.row_of), _ptr(plan.weight), _ptr(shared_out), _ptr(out), t, y.shape[1],
                                    plan.top, dtype_code(out_dtype), dtype_code(y.dtype),
                                    _ptr(plan.chosen) if plan.identity else None, plan.experts - plan.identity,
                                    _ptr(h) if plan.identity else None, h.stride(0) if plan.identity else 0,
                                    _ptr(plan.shared_gate) if shared_out is not None else None, _stream()), "moe_combine")
    return out


DECODE_CHUNK_TILES = 16  # keys per piece of the split decode kernel: 16 tiles of 16
_WORKSPACE = {}


def workspace(device, nfloats: int, which: str = "decode") -> torch.Tensor:
    """A float32 scratch buffer of at least `nfloats` on `device`, kept between calls
    (one per use: `which`).  While a CUDA graph is being captured the buffer is the
    graph's own."""
    if torch.cuda.is_current_stream_capturing():
        return torch.empty(max(nfloats, 1), dtype=torch.float32, device=device)
    key = (str(device), which)
    buf = _WORKSPACE.get(key)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1 << 16), dtype=torch.float32, device=device)
        _WORKSPACE[key] = buf
    return buf


def decode_attention_supported(dtype, head_dim: int, page_size: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0 and group <= 16


def paged_decode_attention(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                           seq_of_token, positions, scale: float, window: int, num_heads: int, num_kv_heads: int,
                           head_dim: int, requests: int, max_kv: int, token_rows=None,
                           out: Optional[torch.Tensor] = None, out_rows: Optional[int] = None,
                           single_tokens: bool = True) -> torch.Tensor:
    """Attention of one query token per entry over its request's pages (bfloat16), the
    key range split over blocks of DECODE_CHUNK_TILES * 16 keys.  `max_kv` bounds
    every entry's number of keys (it sizes the grid and the scratch).  `token_rows`
    picks the entries' rows; `single_tokens=False` says that some of them are tokens of
    one request's portion (the kernel then waits for the step's cache writes before it
    reads any key)."""
    _dev(q, k_pool, v_pool, block_table, seq_of_token, positions, token_rows)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "paged_decode_attention: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_decode_attention: int32 block table [requests, blocks]")
    if out is None:
        out = torch.empty((out_rows if out_rows is not None else requests, num_heads * head_dim),
                          dtype=q.dtype, device=q.device)
    keys = max_kv if window <= 0 else min(max_kv, window + 15)
    max_splits = max(1, -(-(-(-keys // 16) + (1 if window > 0 else 0)) // DECODE_CHUNK_TILES))
    scratch = None
    if max_splits > 1:
        scratch = workspace(q.device, requests * num_heads * max_splits * (head_dim + 2))
    _check(library().vx_paged_decode_attention(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(token_rows), _ptr(seq_of_token), _ptr(positions), _ptr(scratch), max_splits, _ptr(out),
        num_heads * head_dim, float(scale), int(window), requests, num_heads, num_kv_heads, head_dim,
        k_pool.shape[2], DECODE_CHUNK_TILES, 1 if single_tokens else 0, _stream()), "paged_decode_attention")
    return out


def prefill_attention_supported(dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size % 16 == 0


def paged_prefill_attention(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                            cu_seqlens, kv_offsets, scale: float, window: int, num_heads: int, num_kv_heads: int,
                            head_dim: int, requests: int, max_new: int, tokens: int, seq_list=None,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of prompt portions over the pages (bfloat16, tensor cores):
    request i brings token rows [cu_seqlens[i], cu_seqlens[i+1]) at positions
    kv_offsets[i] onward; `max_new` bounds the tokens of any request.  With `seq_list`
    (int32, on the device) only its first `requests` entries' requests are worked on,
    and only their rows of `out` are written."""
    _dev(q, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, seq_list, out)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "paged_prefill_attention: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_prefill_attention: int32 block table [requests, blocks]")
    if out is None:
        out = torch.empty((tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    _check(library().vx_paged_prefill_attention(
        _ptr(q), q_row_stride, _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(cu_seqlens), _ptr(kv_offsets), _ptr(seq_list), _ptr(out), num_heads * head_dim, float(scale), int(window), requests,
        int(max_new), num_heads, num_kv_heads, head_dim, k_pool.shape[2], _stream()), "paged_prefill_attention")
    return out


PREFILL_MAX_SPLITS = 16


def prefill_attention_tc_supported(dtype, head_dim: int, page_size: int, group: int) -> bool:
    return dtype == torch.bfloat16 and head_dim == 128 and page_size % 16 == 0 and 1 <= group <= 8


def paged_prefill_attention_tc(q: torch.Tensor, q_row_stride: int, k_pool, v_pool, block_table: torch.Tensor,
                               cu_seqlens, kv_offsets, scale: float, window: int, num_heads: int, num_kv_heads: int,
                               head_dim: int, requests: int, max_new: int, tokens: int, seq_list=None,
                               out: Optional[torch.Tensor] = None, max_kv: int = 0, halves: bool = False, sinks=None,
                               gate_col: int = -1) -> torch.Tensor:
    """The same as `paged_prefill_attention` on the tcgen05 tensor cores (head size
    128, accumulators in tensor memory, operands by TMA).  `max_kv` (a bound on any
    request's keys after the step) lets short portions on top of many keys be cut into
    runs of key tiles that several blocks share; 0: never.  `halves`: the probabilities go to the
    tensor core as two bfloat16 halves (32-bit softmax weights in effect; half as many products again);
    with it `sinks` and `gate_col` as in `paged_attention_generic`."""
    _dev(q, k_pool, v_pool, block_table, cu_seqlens, kv_offsets, seq_list, out, sinks)
    _need(halves or (sinks is None and gate_col < 0), "paged_prefill_attention_tc: a sink and a gate go with halves=True")
    _check_sinks_gate("paged_prefill_attention_tc", sinks, gate_col, num_heads, q_row_stride)
    _need(q.dtype == torch.bfloat16 and k_pool.dtype == torch.bfloat16 and v_pool.dtype == torch.bfloat16,
          "paged_prefill_attention_tc: bfloat16 only")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "paged_prefill_attention_tc: int32 block table [requests, blocks]")
    _need(k_pool.is_contiguous() and v_pool.is_contiguous(), "paged_prefill_attention_tc: contiguous pools")
    if out is None:
        out = torch.empty((tokens, num_heads * head_dim), dtype=q.dtype, device=q.device)
    # runs of key tiles: up to a quarter of the longest request's key tiles, 16 at most; only a step whose
    # portions are short can have a request that is cut (a long portion has query tiles enough)
    max_splits, scratch = 1, None
    toks_per_tile = (128 // (num_heads // num_kv_heads)) & ~7   # (as pt_toks_per_tile in the kernel)
    sms = _sm_count(q.device)
    if max_kv >= 8 * 128 and 2 * -(-max_new // (2 * toks_per_tile)) * num_kv_heads <= sms:   # (a block takes two query tiles)
        max_splits = max(1, min(PREFILL_MAX_SPLITS, -(-max_kv // 128) // 4, sms // num_kv_heads))
        scratch = workspace(q.device, tokens * num_heads * max_splits * (head_dim + 2), which="prefill")
    args = (_ptr(q), q_row_stride, tokens, _ptr(k_pool), _ptr(v_pool), k_pool.shape[0], _ptr(block_table),
            block_table.shape[1], _ptr(cu_seqlens), _ptr(kv_offsets), _ptr(seq_list), _ptr(out), num_heads * head_dim, float(scale),
            int(window), requests, int(max_new), num_heads, num_kv_heads, head_dim, k_pool.shape[2],
            _ptr(scratch), max_splits, _ptr(_error_word(q.device)))
    if halves:
        _check(library().vx_paged_prefill_attention_tc_ext(*args, _ptr(sinks), int(gate_col), _stream()),
               "paged_prefill_attention_tc (halves)")
    else:
        _check(library().vx_paged_prefill_attention_tc(*args, _stream()), "paged_prefill_attention_tc")
    note_bounded_wait()
    return out


def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, bias=None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a [M,K] times w [N,K] transposed, float32 multiply-adds on the CUDA cores."""
    _dev(a, w, bias)
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "gemm: a [M,K], w [N,K]")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and a.dtype == w.dtype, "gemm: rows contiguous, one element type")
    out_dtype = out_dtype or a.dtype
    m, k = a.shape
    n = w.shape[0]
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm: float32 bias of N elements")
    out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    _check(library().vx_gemm_nt_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0), n,
                                     dtype_code(a.dtype), dtype_code(out_dtype), _stream()), "gemm_nt_simt")
    return out


GEMM_HEADS_FEW_ROWS = 8   # rows up to which the products per head take the kernel that gives every output column a warp


def gemm_heads(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One product per head: out[:, h, :] = a[:, h, :] w[h]^T with a [M, H, K], w [H, N, K] (contiguous), out [M, H, N];
    `a` and `out` may be views into wider rows (their last dimension contiguous).  float32 multiply-adds (in float32, every
    sum over k in ascending order whatever the number of rows; bfloat16 steps of up to 8 rows take a kernel of their own)."""
    _dev(a, w, out)
    _need(a.dim() == 3 and w.dim() == 3 and out.dim() == 3 and w.is_contiguous() and a.shape[1] == w.shape[0]
          and a.shape[2] == w.shape[2] and out.shape == (a.shape[0], w.shape[0], w.shape[1]), "gemm_heads: a [M,H,K], w [H,N,K], out [M,H,N]")
    _need(a.stride(2) == 1 and out.stride(2) == 1 and a.dtype == w.dtype, "gemm_heads: rows contiguous, one element type")
    m, h, k = a.shape
    n = w.shape[1]
    if a.dtype == torch.bfloat16 and m <= GEMM_HEADS_FEW_ROWS and k % 8 == 0 and k <= 4096 and w.data_ptr() % 16 == 0:
        # a decode step's few rows: a warp per output column, W read once by batch * n / 8 blocks
        _check(library().vx_gemm_few_rows_batched(_ptr(a), _ptr(w), _ptr(out), m, n, k, a.stride(0), k, out.stride(0), h, a.stride(1),
                                                  n * k, out.stride(1), dtype_code(out.dtype), _stream()), "gemm_few_rows_heads")
        return out
    _check(library().vx_gemm_nt_simt_batched(_ptr(a), _ptr(w), None, _ptr(out), m, n, k, a.stride(0), k, out.stride(0), h,
                                             a.stride(1), n * k, out.stride(1), dtype_code(a.dtype), dtype_code(out.dtype),
                                             _stream()), "gemm_nt_simt_heads")
    return out


STRETCH_MIN_TOKENS = 128    # a step's longest portion from which its tokens are walked in stretches side by side
STRETCH_MIN_LENGTH = 64
STRETCH_MOST = 64           # stretches of a step, about: longer steps get longer stretches


class StretchPlan:
    """A step's token rows cut into stretches of at most `length` rows that never cross a request: `cu` [stretches + 1]
    first row of each, `first` [requests + 1] first stretch of each request, `ident` 0 .. stretches - 1 (int32, on the
    device)."""

    def __init__(self, new_lens, device, length: int = 0):
        total = int(sum(new_lens))
        self.length = int(length) or max(STRETCH_MIN_LENGTH, -(-(-(-total // STRETCH_MOST)) // 16) * 16)
        cu, first, row = [0], [0], 0
        for n in new_lens:
            for lo in range(0, int(n), self.length):
                cu.append(row + min(int(n), lo + self.length))
            row += int(n)
            first.append(len(cu) - 1)
        self.count, self.requests = len(cu) - 1, len(new_lens)
        both = torch.tensor(cu + first + list(range(self.count)), dtype=torch.int32).to(device, non_blocking=True)
        self.cu, self.first = both[:len(cu)], both[len(cu):len(cu) + len(first)]
        self.ident = both[len(cu) + len(first):]


def linear_attention_walk(x: torch.Tensor, q_col: int, k_col: int, v_col: int, state: torch.Tensor, cu_seqlens, state_slots,
                          seqs: int, heads: int, dim: int, vdim: int, decay: Optional[torch.Tensor] = None,
                          gate: Optional[torch.Tensor] = None, gate_mul: float = 1.0, inv_freq: Optional[torch.Tensor] = None,
                          rot_dim: int = 0, interleaved: bool = False, positions: Optional[torch.Tensor] = None,
                          q_mul: float = 1.0, k_mul: float = 1.0, stretches: Optional[StretchPlan] = None) -> torch.Tensor:
    """Per head S = a (.) S + k v^T, o = S^T q over every request's tokens in order, a = decay[h] (float32 per head) or
    sigmoid(gate)^gate_mul per key channel and token (`gate` float32 [tokens, heads * dim], contiguous rows).  q and k
    are turned by position * inv_freq on their first `rot_dim` channels, then multiplied by q_mul / k_mul, all in
    float32.  `state` float32 [slots, heads, dim, vdim] is read and written back.  Returns float32 [tokens, heads * vdim].
    With `stretches` (the plan of this step's rows) the stretches are walked side by side: once from zero for what each
    adds to the state, a scan over a request's stretches for the state at the start of each, and once more for the outputs."""
    _dev(x, decay, gate, inv_freq, positions, state, cu_seqlens, state_slots)
    _need(x.stride(1) == 1 and (decay is None) != (gate is None), "linear_attention_walk: a decay per head or a gate per channel")
    if decay is not None:
        _need(decay.dtype == torch.float32 and decay.numel() == heads, "linear_attention_walk: float32 decay per head")
    if gate is not None:
        _need(gate.dtype == torch.float32 and gate.stride(1) == 1 and gate.shape == (x.shape[0], heads * dim),
              "linear_attention_walk: float32 gate [tokens, heads * dim]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dim and positions is not None
              and positions.dtype == torch.int32, "linear_attention_walk: inv_freq of rot_dim / 2 numbers, int32 positions")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "linear_attention_walk: float32 state [slots, heads, dim, vdim]")
    out = torch.empty((x.shape[0], heads * vdim), dtype=torch.float32, device=x.device)
    lib = library()

    def walk(st, cu, slots, n, result, fresh):
        _check(lib.vx_linear_attention_walk_parts(
            _ptr(x), x.stride(0), int(q_col), int(k_col), int(v_col), _ptr(decay), _ptr(gate), gate.stride(0) if gate is not None else 0,
            float(gate_mul), _ptr(inv_freq), int(rot_dim) if inv_freq is not None else 0, 1 if interleaved else 0, _ptr(positions),
            float(q_mul), float(k_mul), _ptr(st), _ptr(cu), _ptr(slots), _ptr(result), int(n), heads, dim, vdim,
            1 if fresh else 0, dtype_code(x.dtype), _stream()), "linear_attention_walk")

    if stretches is None:
        walk(state, cu_seqlens, state_slots, seqs, out, False)
        return out
    _need(stretches.requests == seqs, "linear_attention_walk: the stretches are those of another step")
    per = heads * dim * vdim
    parts = workspace(x.device, stretches.count * per, which="stretch_parts")
    log_a = None
    if gate is not None:
        log_a = workspace(x.device, stretches.count * heads * dim, which="stretch_decay")
        _check(lib.vx_stretch_log_decay(_ptr(gate), gate.stride(0), float(gate_mul), _ptr(stretches.cu), _ptr(log_a),
                                        stretches.count, heads * dim, _stream()), "stretch_log_decay")
    walk(parts, stretches.cu, stretches.ident, stretches.count, None, True)
    _check(lib.vx_stretch_scan(_ptr(parts), _ptr(state), _ptr(log_a), _ptr(decay), _ptr(stretches.cu), _ptr(stretches.first),
                               _ptr(state_slots), seqs, heads, dim, vdim, _stream()), "stretch_scan")
    walk(parts, stretches.cu, stretches.ident, stretches.count, out, False)
    return out


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: Optional[torch.Tensor], heads: int, eps: float,
                   gate_activation: str = "silu") -> torch.Tensor:
    """Every head of o (float32 [rows, heads * vdim]) divided by its root mean square, times `weight` [vdim] if given,
    times silu or sigmoid of `gate` [rows, heads * vdim] (contiguous rows); in the gate's element type."""
    _dev(o, gate, weight)
    vdim = o.shape[1] // heads
    _need(o.dtype == torch.float32 and o.is_contiguous() and gate.stride(1) == 1 and gate.shape == o.shape
          and o.shape[1] == heads * vdim, "head_norm_gate: float32 outputs and a gate of their shape")
    _need(weight is None or (weight.dtype == torch.float32 and weight.numel() == vdim), "head_norm_gate: float32 weight [vdim]")
    _need(gate_activation in ("silu", "sigmoid"), "head_norm_gate: the gate passes through silu or sigmoid")
    out = torch.empty(o.shape, dtype=gate.dtype, device=o.device)
    _check(library().vx_head_norm_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), _ptr(out), o.shape[0], heads, vdim,
                                       float(eps), 1 if gate_activation == "silu" else 0, dtype_code(gate.dtype), _stream()),
           "head_norm_gate")
    return out


def latent_prep(down: torch.Tensor, q: torch.Tensor, qa: Optional[torch.Tensor], weight: torch.Tensor, eps: float, inv_freq: torch.Tensor,
                interleaved: bool, positions: torch.Tensor, slot_mapping, pool, heads: int, dim: int, rot_dim: int,
                rank: int) -> None:
    """`down` [T, rank + rot_dim]: the first `rank` channels RMS-normed with `weight` and, followed by the rotated last
    `rot_dim`, written to `pool` (rows of rank + rot_dim elements) at the step's slots; the last rot_dim channels of every
    head of `q` [T, heads * (dim + rot_dim)] rotated into the last rot_dim channels of `qa` [T, heads, rank + rot_dim], or,
    with `qa` None, where they are."""
    _dev(down, q, qa, weight, inv_freq, positions, slot_mapping, pool)
    _need(qa is None or (qa.is_contiguous() and qa.dtype == q.dtype and tuple(qa.shape) == (q.shape[0], heads, rank + rot_dim)),
          "latent_prep: folded queries [T, heads, rank + rot_dim]")
    _need((down is None or (down.stride(1) == 1 and down.dtype == q.dtype)) and q.stride(1) == 1 and positions.dtype == torch.int32,
          "latent_prep: rows contiguous, one element type, int32 positions")
    _need(down is not None or slot_mapping is None, "latent_prep: a row to write needs the projection that made it")
    _need((weight is None and down is None) or (weight is not None and weight.dtype == torch.float32 and weight.numel() == rank),
          "latent_prep: float32 weight [rank] for the row that the projection made")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() * 2 == rot_dim, "latent_prep: rot_dim / 2 frequencies")
    if slot_mapping is not None:
        _need(pool is not None and pool.dtype == q.dtype and pool.is_contiguous() and pool.shape[-1] == rank + rot_dim,
              "latent_prep: a pool of rows of rank + rot_dim elements")
    _check(library().vx_latent_prep(_ptr(down), down.stride(0) if down is not None else 0, _ptr(q), q.stride(0), _ptr(qa), _ptr(weight), float(eps), _ptr(inv_freq),
                                    1 if interleaved else 0, _ptr(positions), _ptr(slot_mapping), _ptr(pool), q.shape[0],
                                    heads, dim, rot_dim, rank, dtype_code(q.dtype), _stream()), "latent_prep")


LATENT_ATTENTION_MAX_ROW = 1024
LATENT_ATTENTION_MAX_RUNS = 32
LATENT_ATTENTION_BLOCK_HEADS = 16   # query heads that share a staged tile of rows


def latent_attention(qa: torch.Tensor, pool: torch.Tensor, block_table: torch.Tensor, seq_of_token, positions, scale: float,
                     heads: int, rank: int, rot_dim: int, max_kv: int = 0, window: int = 0) -> torch.Tensor:
    """Causal softmax attention of folded queries qa [tokens, heads, rank + rot_dim] over cached latent rows
    (`pool` [pages, 1, page size, rank + rot_dim]; token row t is request seq_of_token[t] at position positions[t]):
    score = qa . row * scale, the value is a row's first `rank` elements.  Returns [tokens, heads, rank] in qa's element
    type.  `max_kv` (a bound on any row's position + 1; 0: unknown) lets a step of few rows cut their keys into runs
    that several blocks share.  With `window` > 0 a row sees only the last `window` positions up to its own."""
    _dev(qa, pool, block_table, seq_of_token, positions)
    tokens, width = qa.shape[0], rank + rot_dim
    if window > 0 and max_kv > 0:
        max_kv = min(max_kv, int(window) + 31)   # (what a row reads at most: its window, from a tile's start)
    _need(qa.is_contiguous() and tuple(qa.shape) == (tokens, heads, width) and pool.dtype == qa.dtype and pool.is_contiguous()
          and pool.dim() == 4 and pool.shape[1] == 1 and pool.shape[3] == width,
          "latent_attention: folded queries [T, heads, rank + rot_dim] and a pool of rows of that width")
    _need(0 < width <= LATENT_ATTENTION_MAX_ROW, "latent_attention: rows of up to %d elements" % LATENT_ATTENTION_MAX_ROW)
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.dim() == 2,
          "latent_attention: int32 block table [requests, blocks]")
    blocks = tokens * (-(-heads // LATENT_ATTENTION_BLOCK_HEADS))
    runs, scratch = 1, None
    if max_kv > 0 and blocks < 2 * _sm_count(qa.device):
        runs = max(1, min(LATENT_ATTENTION_MAX_RUNS, 2 * _sm_count(qa.device) // blocks, -(-max_kv // 64)))
        if runs > 1:
            scratch = workspace(qa.device, tokens * heads * runs * (rank + 2), which="latent_attention")
    out = torch.empty((tokens, heads, rank), dtype=qa.dtype, device=qa.device)
    _check(library().vx_latent_attention_window(_ptr(qa), _ptr(pool), _ptr(block_table), block_table.shape[1], _ptr(seq_of_token),
                                                _ptr(positions), _ptr(out), _ptr(scratch), float(scale), tokens, heads, rank,
                                                rot_dim, pool.shape[2], runs, int(window), dtype_code(qa.dtype), _stream()),
           "latent_attention")
    return out


RAISED_ROWS_BLOCK = 64   # rows of keys and values raised for a step lie in blocks of this many, a request's in a row


class RaisedPlan:
    """Where the raised keys and values of a step's requests lie: request i (holding `kv_lens[i]` positions after the step)
    takes the rows `first[i] * RAISED_ROWS_BLOCK` onward of a matrix of `rows` rows; `table` int32 [requests, blocks] lists,
    by the block of a POSITION, the block of rows that holds it (on the device).  With a `window` (and the positions
    `offsets[i]` cached before the step) a request's rows start at the block of the first position that its first new
    token still sees; earlier positions' entries repeat that block and are never read."""

    def __init__(self, kv_lens, device, offsets=None, window: int = 0):
        self.window = int(window)
        blocks = [-(-int(n) // RAISED_ROWS_BLOCK) for n in kv_lens]
        skipped = [0] * len(blocks)
        if self.window > 0:
            skipped = [max(0, int(o) + 1 - self.window) // RAISED_ROWS_BLOCK for o in offsets]
        self.max_blocks, self.first, at = max(blocks), [], 0
        for b, s in zip(blocks, skipped):
            self.first.append(at)
            at += b - s
        self.rows, self.requests = at * RAISED_ROWS_BLOCK, len(blocks)
        self.max_kv = int(max(int(n) - s * RAISED_ROWS_BLOCK for n, s in zip(kv_lens, skipped)))   # most rows of a request
        table = [[f + min(max(j - s, 0), b - s - 1) for j in range(self.max_blocks)] for f, b, s in zip(self.first, blocks, skipped)]
        self.table = torch.tensor(table, dtype=torch.int32).to(device, non_blocking=True)


def latent_gather(pool: torch.Tensor, block_table: torch.Tensor, cu_seqlens, kv_offsets, plan: RaisedPlan) -> torch.Tensor:
    """The cached rows of every request of a step (positions 0, or the first block that the plan's window still needs, up to
    kv_offsets + new tokens - 1, new ones included) copied out of their pages into one matrix [plan.rows, row width] where
    `plan` says; the rows up to the next block are zeros."""
    _dev(pool, block_table, cu_seqlens, kv_offsets)
    _need(pool.is_contiguous() and pool.dim() == 4 and pool.shape[1] == 1, "latent_gather: a pool [pages, 1, page size, width]")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous() and block_table.shape[0] >= plan.requests,
          "latent_gather: int32 block table [requests, blocks]")
    rows = torch.empty((plan.rows, pool.shape[3]), dtype=pool.dtype, device=pool.device)
    _check(library().vx_latent_gather_window(_ptr(pool), _ptr(block_table), block_table.shape[1], _ptr(cu_seqlens), _ptr(kv_offsets),
                                             None, _ptr(plan.table), plan.max_blocks, _ptr(rows), plan.requests, plan.max_kv,
                                             pool.shape[3], pool.shape[2], RAISED_ROWS_BLOCK, plan.window, dtype_code(pool.dtype),
                                             _stream()), "latent_gather")
    return rows


RAISED_ATTENTION_SIZES = ((64, 32), (64, 64), (64, 128), (128, 32), (128, 64), (128, 128), (32, 32), (48, 48), (80, 80), (96, 96),
                          (112, 112), (192, 128), (192, 64), (96, 64), (96, 32), (256, 128))


def raised_attention_supported(dtype, key_dim: int, v_head_dim: int) -> bool:
    return dtype == torch.bfloat16 and (int(key_dim), int(v_head_dim)) in RAISED_ATTENTION_SIZES


def raised_attention(q: torch.Tensor, q_row_stride: int, kv: torch.Tensor, cu_seqlens, kv_offsets, plan: RaisedPlan, scale: float,
                     num_heads: int, key_dim: int, v_head_dim: int, max_new: int, softcap: float = 0.0) -> torch.Tensor:
    """Causal attention (under the plan's window, if it has one) of prompt portions over keys and values that a matrix product
    left as rows `kv` [plan.rows, num_heads * (key_dim + v_head_dim)], a head's key followed by its value, request i's rows where `plan` says.
    The tensor-core kernel of `biased_prefill_attention` with other strides.  Returns [tokens, num_heads * v_head_dim]."""
    _dev(q, kv, cu_seqlens, kv_offsets)
    per = key_dim + v_head_dim
    _need(q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16 and kv.is_contiguous() and kv.shape[1] == num_heads * per,
          "raised_attention: bfloat16 rows of heads * (key + value) elements")
    out = torch.empty((q.shape[0], num_heads * v_head_dim), dtype=q.dtype, device=q.device)
    _check(library().vx_biased_attention_rows_window(
        _ptr(q), int(q_row_stride), _ptr(kv), kv.shape[1], per, kv.data_ptr() + 2 * key_dim, kv.shape[1], per, _ptr(plan.table),
        plan.max_blocks, _ptr(cu_seqlens), _ptr(kv_offsets), None, _ptr(out), out.shape[1], float(scale), plan.requests,
        int(max_new), num_heads, num_heads, key_dim, v_head_dim, RAISED_ROWS_BLOCK, float(softcap), plan.window, _stream()),
        "raised_attention")
    return out


STREAMS_MAX = 16          # copies of the stream that the stream kernels take
STREAM_MAX_WIDTH = 51200  # ... and the widest row (it lies in a block's shared memory as float32)


def _host_floats(values, n: int, what: str):
    if values is None:
        return None
    vals = [float(v) for v in values]
    _need(len(vals) == n, "%s: expected %d numbers, got %d" % (what, n, len(vals)))
    return (c_float * n)(*vals)


def stream_norm(x: Optional[torch.Tensor], streams: int, in_coef, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None, single: Optional[torch.Tensor] = None,
                copies: Optional[torch.Tensor] = None, rms: bool = False) -> torch.Tensor:
    """The norm of u = sum_s in_coef[s] x_s over the `streams` copies of the stream x float32 [tokens, streams * E]:
    layer norm without bias (`rms`: RMS norm) times `weight`, in `out_dtype`.  `in_coef`: host numbers (None: ones).
    With `rows` (int32 on the device) only those tokens.  With `single` float32 [tokens, E] the copies are all equal to
    it, and are written to `copies` [tokens, streams * E] if given."""
    src = single if single is not None else x
    _dev(x, weight, rows, single, copies)
    tokens = src.shape[0]
    E = weight.numel()
    _need(0 < streams <= STREAMS_MAX, "stream_norm: 1 to %d copies of the stream" % STREAMS_MAX)
    _need(weight.dtype == torch.float32 and src.dtype == torch.float32 and src.is_contiguous()
          and src.shape[1] == (E if single is not None else streams * E), "stream_norm: float32 rows of streams * width elements")
    _need(copies is None or (copies.dtype == torch.float32 and copies.is_contiguous() and tuple(copies.shape) == (tokens, streams * E)),
          "stream_norm: copies [tokens, streams * width] float32")
    _need(rows is None or rows.dtype == torch.int32, "stream_norm: int32 rows")
    n_rows = rows.numel() if rows is not None else tokens
    out = torch.empty((n_rows, E), dtype=out_dtype, device=src.device)
    _check(library().vx_stream_norm(_ptr(x) if single is None else None, int(streams), _host_floats(in_coef, streams, "stream_norm"),
                                    _ptr(single), _ptr(copies), _ptr(weight), float(eps), _ptr(rows), n_rows, _ptr(out), tokens, E,
                                    1 if rms else 0, dtype_code(out_dtype), _stream()), "stream_norm")
    return out


def stream_update(x: torch.Tensor, streams: int, mix, out_coef, mult: float, layer_scale: Optional[torch.Tensor], y: torch.Tensor,
                  in_next=None, weight_next: Optional[torch.Tensor] = None, eps: float = 0.0, rms: bool = False):
    """x float32 [tokens, streams * E] in place: x_t <- sum_s mix[s][t] x_s + mult * out_coef[t] * layer_scale (.) y, all
    copies from the old ones (`mix` rows are "from", host numbers, None: the identity; `out_coef` None: ones; `layer_scale`
    float32 [E] or None).  With `weight_next` also returns the norm of sum_t in_next[t] x_t of the new copies, in y's type."""
    _dev(x, layer_scale, y, weight_next)
    tokens, E = y.shape
    _need(0 < streams <= STREAMS_MAX and x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (tokens, streams * E),
          "stream_update: the stream float32 [tokens, streams * width]")
    _need(y.stride(1) == 1 and (layer_scale is None or (layer_scale.dtype == torch.float32 and layer_scale.numel() == E)),
          "stream_update: rows contiguous, float32 layer scale [width]")
    flat = None if mix is None else [v for row in mix for v in row]
    h = None
    if weight_next is not None:
        _need(weight_next.dtype == torch.float32 and weight_next.numel() == E, "stream_update: float32 norm weight [width]")
        h = torch.empty((tokens, E), dtype=y.dtype, device=y.device)
    _check(library().vx_stream_update(_ptr(x), int(streams), _host_floats(flat, streams * streams, "stream_update"),
                                      _host_floats(out_coef, streams, "stream_update"), float(mult), _ptr(layer_scale), _ptr(y),
                                      y.stride(0), _host_floats(in_next, streams, "stream_update"), _ptr(weight_next), float(eps),
                                      _ptr(h), tokens, E, 1 if rms else 0, dtype_code(y.dtype), _stream()), "stream_update")
    return h


def diff_combine(maps: torch.Tensor, gates: Optional[torch.Tensor], gate_col: int, lam: float, post: float, eps: float,
                 num_heads: int, per_group: int, v_head_dim: int, out_dtype: torch.dtype) -> torch.Tensor:
    """maps [tokens, 2 * num_heads * v_head_dim] (float32 or `out_dtype`), per key/value group the group's `per_group` heads
    of the first softmax map followed by those of the second: o = a1 - lam a2, divided by its root mean square over the head
    (eps inside the root), times `post`, times sigmoid of column gate_col + head of the token's row of `gates` (gate_col < 0:
    no gate).  Returns [tokens, num_heads * v_head_dim] in `out_dtype`, heads in their own order."""
    _dev(maps, gates)
    tokens = maps.shape[0]
    _need(maps.is_contiguous() and maps.shape[1] == 2 * num_heads * v_head_dim and maps.dtype in (torch.float32, out_dtype),
          "diff_combine: maps [tokens, 2 heads * v_head_dim]")
    _need(gate_col < 0 or (gates is not None and gates.dtype == out_dtype and gates.stride(1) == 1), "diff_combine: gates of the output's type")
    out = torch.empty((tokens, num_heads * v_head_dim), dtype=out_dtype, device=maps.device)
    _check(library().vx_diff_combine(_ptr(maps), 1 if maps.dtype == torch.float32 else 0, _ptr(gates),
                                     gates.stride(0) if gates is not None else 0, int(gate_col), _ptr(out), float(lam), float(post),
                                     float(eps), tokens, num_heads, per_group, v_head_dim, dtype_code(out_dtype), _stream()),
           "diff_combine")
    return out


def sigmoid_gate(o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """o * sigmoid(gate), element by element; rows may be strided."""
    _dev(o, gate)
    _need(o.dim() == 2 and o.shape == gate.shape and o.dtype == gate.dtype and o.stride(1) == 1 and gate.stride(1) == 1,
          "sigmoid_gate: two matrices of one shape and type, rows contiguous")
    out = torch.empty(tuple(o.shape), dtype=o.dtype, device=o.device)
    _check(library().vx_sigmoid_gate(_ptr(o), o.stride(0), _ptr(gate), gate.stride(0), _ptr(out), out.stride(0), o.shape[0],
                                     o.shape[1], dtype_code(o.dtype), _stream()), "sigmoid_gate")
    return out


def capped_gated_act(sums: torch.Tensor, bias: Optional[torch.Tensor], limit: float, slope: float,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """sums float32 [rows, 2 inner] (all gates, then all ups), `bias` float32 [2 inner] added first:
    g = min(gate, limit), u = clamp(up, -limit, limit); g sigmoid(slope g) (u + 1), rounded once to `out_dtype`."""
    _dev(sums, bias)
    _need(sums.dtype == torch.float32 and sums.is_contiguous() and sums.dim() == 2 and sums.shape[1] % 2 == 0,
          "capped_gated_act: float32 rows of even width")
    inner = sums.shape[1] // 2
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * inner), "capped_gated_act: float32 bias")
    out = torch.empty((sums.shape[0], inner), dtype=out_dtype, device=sums.device)
    _check(library().vx_capped_gated_act(_ptr(sums), _ptr(bias), _ptr(out), sums.shape[0], inner, float(limit), float(slope),
                                         dtype_code(out_dtype), _stream()), "capped_gated_act")
    return out


def sum_add_rmsnorm(residual: torch.Tensor, branches=(), rows_add: Optional[torch.Tensor] = None,
                    vec: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                    out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """residual (float32, in place) += sum of c * y over up to three `branches` [(y, c)] + rows_add (float32, the
    residual's shape) + vec (float32 [width]); with `weight` returns rmsnorm(residual) * weight in `out_dtype`."""
    branches = [(y, c) for y, c in branches if y is not None]
    _dev(residual, rows_add, vec, weight, *[y for y, _ in branches])
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and len(branches) <= 3, "sum_add_rmsnorm: float32 residual")
    width = residual.shape[-1]
    dt = branches[0][0].dtype if branches else (out_dtype or torch.float32)
    for y, _ in branches:
        _need(y.dtype == dt and y.is_contiguous() and y.shape == residual.shape, "sum_add_rmsnorm: branches of the residual's shape")
    _need(rows_add is None or (rows_add.dtype == torch.float32 and rows_add.is_contiguous() and rows_add.shape == residual.shape),
          "sum_add_rmsnorm: float32 rows of the residual's shape")
    for v in (vec, weight):
        _need(v is None or (v.dtype == torch.float32 and v.numel() == width and v.is_contiguous()), "sum_add_rmsnorm: float32 vectors of the row's width")
    if out_dtype is not None and branches:
        _need(out_dtype == dt, "sum_add_rmsnorm: the normed rows have the branches' element type")
    out = torch.empty(residual.shape, dtype=dt, device=residual.device) if weight is not None else None
    b = branches + [(None, 0.0)] * (3 - len(branches))
    _check(library().vx_sum_add_rmsnorm(_ptr(residual), _ptr(b[0][0]), float(b[0][1]), _ptr(b[1][0]), float(b[1][1]), _ptr(b[2][0]),
                                        float(b[2][1]), _ptr(rows_add), _ptr(vec), _ptr(weight), _ptr(out), residual.shape[0],
                                        width, float(eps), dtype_code(dt), _stream()), "sum_add_rmsnorm")
    return out


def softcap_rows(x: torch.Tensor, cap: float) -> torch.Tensor:
    """cap * tanh(x / cap) on float32 x."""
    _dev(x)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "softcap_rows: float32 rows")
    out = torch.empty_like(x)
    _check(library().vx_softcap_rows(_ptr(x), _ptr(out), x.numel(), float(cap), _stream()), "softcap_rows")
    return out


_SM_COUNTS = {}


def _sm_count(device) -> int:
    key = str(device)
    if key not in _SM_COUNTS:
        _SM_COUNTS[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNTS[key]


_ERROR_WORDS = {}


def _error_word(device) -> torch.Tensor:
    """The device int that kernels with bounded waits report into."""
    key = str(device)
    if key not in _ERROR_WORDS:
        _ERROR_WORDS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _ERROR_WORDS[key]


_BOUNDED_WAIT_LAUNCHES = 0   # launches of kernels with bounded waits, ever
_BOUNDED_WAIT_CHECKED = 0    # ... at the last check of the error word


def bounded_wait_launches() -> int:
    return _BOUNDED_WAIT_LAUNCHES


def note_bounded_wait(n: int = 1) -> None:
    """A kernel whose waits are bounded was launched (by the wrappers below, or by
    the replay of a graph that holds such kernels): the error word has to be read
    before the step's results are trusted."""
    global _BOUNDED_WAIT_LAUNCHES
    _BOUNDED_WAIT_LAUNCHES += n


def bounded_wait_pending() -> bool:
    """True if a kernel with bounded waits was launched since the error word was last read."""
    return _BOUNDED_WAIT_LAUNCHES != _BOUNDED_WAIT_CHECKED


def check_pending_device_errors() -> None:
    """`check_device_errors()` if a kernel with bounded waits ran since the last check,
    else nothing (and no synchronisation).  What steps a model calls this before it
    hands out a step's results; it does not have to know which kernels a part chose."""
    if bounded_wait_pending():
        check_device_errors()


def check_device_errors() -> None:
    """Raises if a kernel has reported that one of its bounded waits ran out since
    the last check (its results are then missing).  Synchronises the device."""
    global _BOUNDED_WAIT_CHECKED
    _BOUNDED_WAIT_CHECKED = _BOUNDED_WAIT_LAUNCHES
    for key, word in _ERROR_WORDS.items():
        code = int(word.item())
        if code:
            word.zero_()
            raise KernelError("a kernel on %s gave up a wait on its asynchronous copies or tensor-core work "
                              "(code %d); its results are missing" % (key, code))


def tcgen05_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and w.shape[0] % 16 == 0
            and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def tcgen05_pair_better(m: int, n: int, device) -> bool:
    """Whether 256 x 256 tiles by pairs of blocks beat 128 x 256 tiles by single blocks for
    an [m, n] result: both kinds of block spend the same time on a tile (a pair a little
    less: each SM reads half of W's tile from its shared memory), so the kind that needs
    fewer rounds of the GPU's SMs wins; padding rows count as work."""
    sms = _sm_count(device)
    cols = -(-n // 256)
    single = -(-(-(-m // 128) * cols) // sms)
    paired = -(-(-(-m // 256) * cols) // max(1, sms // 2))
    return paired * 0.97 < single


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias=None, gated_activation: Optional[str] = None,
                 wide: bool = True, pair: bool = False) -> torch.Tensor:
    """a [M,K] times w [N,K] transposed on the tcgen05 tensor cores (bfloat16 in and
    out, float32 accumulation in tensor memory, operands by TMA).  With
    `gated_activation`, w's rows come in tiles of 8 gate rows followed by their 8 up
    rows and the result is act(gate) * up, [M, N/2].  `wide`: 128 x 256 tiles, else
    128 x 128; `pair`: 256 x 256 tiles, each formed by a pair of blocks."""
    _dev(a, w, bias)
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "gemm_tcgen05: a [M,K], w [N,K]")
    _need(tcgen05_supported(a, w), "gemm_tcgen05: bfloat16, K a multiple of 8, N a multiple of 16, 16-byte aligned rows")
    m, k = a.shape
    n = w.shape[0]
    cols = n // 2 if gated_activation else n
    if gated_activation is not None:
        _need(gated_activation in ACTIVATIONS, "gemm_tcgen05: unknown activation %r" % gated_activation)
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tcgen05: float32 bias of N elements")
    out = torch.empty((m, cols), dtype=torch.bfloat16, device=a.device)
    _need(cols % 8 == 0, "gemm_tcgen05: output rows must be 16-byte aligned")
    if pair:
        _check(library().vx_gemm_tcgen05_pair(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0),
                                              cols, 1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0),
                                              _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05_pair")
    else:
        _check(library().vx_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0), cols,
                                         1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0),
                                         1 if wide else 0, _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05")
    note_bounded_wait()
    return out


SKINNY_MAX_ROWS = 8
_MATMUL_SET = False


def skinny_supported(m: int, k: int, a: torch.Tensor, w: torch.Tensor) -> bool:
    return (0 < m <= SKINNY_MAX_ROWS and k % 32 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias=None, out_dtype: Optional[torch.dtype] = None,
                gated_activation: Optional[str] = None, variant: int = 0) -> torch.Tensor:
    """a [M<=8, K] times w [N,K] transposed, W streamed once (bfloat16).  With
    `gated_activation`, w's rows come in tiles of 8 gate rows followed by their 8 up
    rows and the result is act(gate) * up, [M, N/2]."""
    _dev(a, w, bias)
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
          and a.shape[1] == w.shape[1], "gemm_skinny: bfloat16 a [M,K], w [N,K]")
    out_dtype = out_dtype or torch.bfloat16
    m, k = a.shape
    n = w.shape[0]
    cols = n // 2 if gated_activation else n
    if gated_activation is not None:
        _need(gated_activation in ACTIVATIONS, "gemm_skinny: unknown activation %r" % gated_activation)
    out = torch.empty((m, cols), dtype=out_dtype, device=a.device)
    _check(library().vx_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, a.stride(0), w.stride(0), cols,
                                    1 if gated_activation else 0, ACTIVATIONS.get(gated_activation, 0),
                                    dtype_code(out_dtype), variant, _stream()), "gemm_skinny")
    return out


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, bias=None, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """a [M,K] times w [N,K] transposed on the tensor cores, float32 accumulation."""
    _dev(a, w, bias)
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_bf16: bfloat16 operands")
    out_dtype = out_dtype or torch.bfloat16
    if skinny_supported(a.shape[0], a.shape[1], a, w):
        return gemm_skinny(a, w, bias, out_dtype)
    # library product (cuBLAS through torch); reductions stay in float32
    global _MATMUL_SET
    if not _MATMUL_SET:
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        _MATMUL_SET = True
    if out_dtype == torch.float32 or bias is not None:
        out = torch.mm(a, w.t(), out_dtype=torch.float32)
    else:
        out = torch.mm(a, w.t())
    if bias is not None:
        # added to the float32 sums; the result is rounded once
        _need(bias.dtype == torch.float32 and bias.numel() == w.shape[0], "gemm_bf16: float32 bias of N elements")
        summed = out
        out = torch.empty(summed.shape, dtype=out_dtype, device=a.device)
        _check(library().vx_add_bias(_ptr(summed), _ptr(bias), _ptr(out), summed.shape[0], summed.shape[1],
                                     dtype_code(out_dtype), 1.0, _stream()), "add_bias")
    return out


def sample(logits: torch.Tensor, temperature=None, top_p=None, uniform=None) -> torch.Tensor:
    """int32 token per row of float32 `logits` [R,V]; all greedy without `temperature`."""
    _dev(logits, temperature, top_p, uniform)
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "sample: float32 logits [R,V]")
    r, v = logits.shape
    for t in (temperature, top_p, uniform):
        if t is not None:
            _need(t.dtype == torch.float32 and t.numel() == r, "sample: float32 per-row parameters")
    out = torch.empty((r,), dtype=torch.int32, device=logits.device)
    _check(library().vx_sample(_ptr(logits), logits.stride(0), r, v, _ptr(temperature), _ptr(top_p), _ptr(uniform),
                               _ptr(out), _stream()), "sample")
    return out
