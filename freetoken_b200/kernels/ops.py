"""Python face of the CUDA kernels: argument checks, then one C call per op.

Every function takes device tensors, writes into caller-provided outputs, launches on the
current CUDA stream and allocates nothing.  A tensor that is not on a CUDA device, has the
wrong dtype or is not contiguous raises :class:`KernelError` before anything is launched;
the native side checks sizes again and reports through ``ftk_last_error``.

Kernel inventory (reference kernel each one stands for):

=====================  ==========================================================
embedding_gather       python/freetoken/kernel/csrc/jit/index.cu:31-59
add_rmsnorm            python/freetoken/kernel/triton/norm.py:42-112
norm_rope_store        norm.py:42-75 + python/freetoken/kernel/triton/rope.py:28-91 +
                       python/freetoken/kernel/csrc/jit/store.cu:27-53, in one pass
paged_attention        python/freetoken/kernel/triton/attention.py:147-466,469-880
router_topk            python/freetoken/models/minimax_m3/moe.py:71-81
moe_permute            python/freetoken/kernel/triton/fused_moe.py:5-108
moe_gemm1_act          fused_moe.py:156-302 + python/freetoken/kernel/triton/activation.py:67-112
moe_gemm2              fused_moe.py:156-302 (route weight on the accumulator, :292-296)
moe_combine            fused_moe.py:111-153
act_and_mul            activation.py:67-112
sample                 python/freetoken/engine/sample.py:24-80, python/freetoken/kernel/triton/sampling.py
moe_route              router product + router_topk + moe_permute in one launch (short steps)
add_rmsnorm_routes     moe_combine + add_rmsnorm in one pass
linear                 python/freetoken/layers/linear.py:66-70 (the library product)
copy_tokens            the sampled tokens of the step before, taken on the device
                       (python/freetoken/scheduler/scheduler.py:194-256, overlapped scheduling)
stream_add_norm        no counterpart: several addends into the 32-bit stream and a norm without
                       row statistics (Dynamic Tanh) in one pass
head_gate, table_route, scale  no counterpart: per-head output gate, experts by a table over
                       token ids, logit scale
hyper_step, norm_mean  no counterpart: several residual streams (write, read, norm in one pass), the
                       mean of normed branch outputs
conv_act, ssm_gates,   no counterpart: convolution of projected rows with a per-request state, step sizes
ssm_output, delta_scan and decays, gated group norm of a state-space layer; the gated delta rule
=====================  ==========================================================

``paged_attention`` runs one of five kernels by ``tile_rows``: 16 (float32, or bfloat16 steps of single
tokens where the tcgen05 kernel does not take the sizes), 64 (bfloat16 mma.sync), 128 (bfloat16 tcgen05:
long steps and decode steps), 256 (the same with two query tiles per CTA: very long steps).
"""

from __future__ import annotations

import ctypes
from typing import Any, Optional, Sequence

import torch

from ..errors import KernelError
from . import library

F32, BF16 = 0, 1
ACT_SILU, ACT_SWIGLUOAI = 0, 1
SCORE_SIGMOID, SCORE_SOFTMAX, SCORE_SOFTMAX_OF_CHOSEN = 0, 1, 2
ACT_CODES = {"silu": ACT_SILU, "swigluoai": ACT_SWIGLUOAI}
SCORE_CODES = {"sigmoid": SCORE_SIGMOID, "softmax": SCORE_SOFTMAX, "softmax_of_chosen": SCORE_SOFTMAX_OF_CHOSEN,
               "sigmoid_raw": 3}

_vp = ctypes.c_void_p
_i = ctypes.c_int
_f = ctypes.c_float


class _Section(ctypes.Structure):
    _fields_ = [
        ("first_head", _i), ("n_heads", _i), ("norm_weight", _vp), ("rotate", _i),
        ("dense_out", _vp), ("slab", _vp), ("slot_map", _vp), ("page_size", _i), ("num_pages", _i),
        ("bias", _vp), ("pos_scale", _vp), ("pos_scale_len", _i), ("dst_head_dim", _i),
    ]


class _StreamNorm(ctypes.Structure):
    _fields_ = [
        ("residual", _vp), ("x1", _vp), ("x2", _vp), ("y", _vp), ("route_pos", _vp), ("top_k", _i), ("n_routes", _i),
        ("table", _vp), ("ids", _vp), ("vocab", _i), ("vec", _vp), ("norm", _i), ("weight", _vp), ("bias", _vp),
        ("alpha", _vp), ("out", _vp), ("dtype", _i), ("rows", _vp), ("n_rows", _i), ("hidden", _i),
    ]


class _AttnExtras(ctypes.Structure):
    _fields_ = [("dist_bias", _vp), ("dist_len", _i), ("kv_split", _i), ("has_sink", _i), ("sink_logit", _f),
                ("sink_heads", _vp)]


_SIGNATURES = {
    "ftk_embedding_gather": [_vp, _i, _vp, _i, _i, _i, _vp, _vp],
    "ftk_add_rmsnorm": [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _i, _vp],
    "ftk_add_rmsnorm_routes": [_vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _i, _f, _i, _vp],
    "ftk_norm_rope_store": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _i, _f, _i, _i,
                            ctypes.POINTER(_Section), _vp],
    "ftk_paged_attention": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                            _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ftk_paged_attention_ex": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                               _i, _i, _i, _i, _i, _i, _f, _i, ctypes.POINTER(_AttnExtras), _vp],
    "ftk_stream_add_norm": [ctypes.POINTER(_StreamNorm), _vp],
    "ftk_head_gate": [_vp, _i, _vp, ctypes.c_longlong, _i, _i, _i, _vp],
    "ftk_table_route": [_vp, _vp, _i, _i, _i, _i, _f, _vp, _vp, _vp],
    "ftk_scale_f32": [_vp, ctypes.c_longlong, _f, _vp],
    "ftk_attention_tc_fits": [_i, _i, _i],
    "ftk_paged_attention_tc": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                               _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ftk_paged_attention_tc_ex": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                  _i, _i, _i, _i, _i, _i, _f, _i, ctypes.POINTER(_AttnExtras), _i, _vp],
    "ftk_attention_tc_few_fits": [_i, _i, _i],
    "ftk_paged_attention_tc_few": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                      _i, _i, _i, _i, _i, _i, ctypes.c_float, _i, _vp],
    "ftk_paged_attention_tc_pair": [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                    _i, _i, _i, _i, _i, _i, _f, _i, _vp],
    "ftk_paged_attention_sparse": [_vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp,
                                   _i, _i, _i, _i, _i, _i, _f, _vp, _i, _i, _vp],
    "ftk_sparse_select": [_vp, _vp, _i, _vp, _i, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp],
    "ftk_sparse_score_fits": [_i, _i, _i],
    "ftk_router_topk": [_vp, _i, _vp, _i, _i, _i, _i, _f, _vp, _vp, _vp],
    "ftk_moe_permute": [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "ftk_moe_route_fits": [_i, _i, _i, _i],
    "ftk_moe_route": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp],
    "ftk_small_linear_fits": [_i, _i, _i],
    "ftk_small_linear": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "ftk_moe_small_fits": [_i, _i, _i, _i],
    "ftk_moe_small_gate_up": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp],
    "ftk_moe_small_down": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "ftk_moe_gather": [_vp, _i, _vp, _i, _i, _i, _vp, _vp],
    "ftk_moe_gemm1_act": [_vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "ftk_moe_gemm1_gather_fits": [_i, _i, _i, _i],
    "ftk_moe_gemm1_act_gather": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "ftk_moe_gemm2": [_vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp],
    "ftk_moe_combine": [_vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp],
    "ftk_act_and_mul": [_vp, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "ftk_sample": [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "ftk_cast": [_vp, _i, _vp, _i, ctypes.c_longlong, _vp],
    "ftk_table_update": [_vp, ctypes.c_longlong, _vp, _i, _vp],
    "ftk_copy_tokens": [_vp, _i, _vp, _vp, _i, _i, _i, _vp],
    "ftk_read_status": [ctypes.POINTER(ctypes.c_int)],
    "ftk_set_moe_tensor_cores": [_i],
    "ftk_set_moe_pairs": [_i],
    "ftk_debug_set_status": [_i, _i],
    "ftk_variant_counts": [ctypes.c_char_p, _i, _i],
    "ftk_softcap_f32": [_vp, ctypes.c_longlong, _f, _vp],
    "ftk_postnorm_add_norm": [_vp, _i, _vp, _i, _i, _vp, _vp, _f, _i, _vp, _vp, _f, _i, _vp, _vp, _vp, _i, _i, _vp],
    "ftk_gated_heads": [_vp, _i, _i, _vp, ctypes.c_longlong, _vp, _f, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "ftk_short_conv": [_vp, _vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "ftk_depth_mix": [_vp, ctypes.c_longlong, _i, _vp, _vp, ctypes.c_longlong, _vp],
    "ftk_moe_gather_scaled": [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp],
    "ftk_relu2": [_vp, _i, ctypes.c_longlong, _vp],
    "ftk_latent_store": [_vp, _i, ctypes.c_longlong, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp, _vp, _i, _vp, _vp,
                         ctypes.c_longlong, _vp, _i, _i, _vp],
    "ftk_latent_query_rotate": [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i, _i, _i, _vp],
    "ftk_mlstm_gates": [_vp, _vp, _vp, _f, _vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp],
    "ftk_mlstm_output": [_vp, _vp, _vp, _vp, ctypes.c_longlong, _vp, _f, _vp, _i, _i, _i, _i, _vp],
    "ftk_gla_scan": [_vp, ctypes.c_longlong, _vp, ctypes.c_longlong, _vp, ctypes.c_longlong, _i, _vp, _vp, _f, _f,
                     _vp, _i, _vp, _vp, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _i, _vp, _i, _vp],
    "ftk_hyper_step": [_vp, ctypes.c_longlong, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _f, _vp, _i, _vp, _vp],
    "ftk_conv_act": [_vp, ctypes.c_longlong, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _vp],
    "ftk_delta_scan": [_vp, ctypes.c_longlong, _vp, ctypes.c_longlong, _vp, ctypes.c_longlong, _vp, ctypes.c_longlong,
                       _vp, ctypes.c_longlong, _i, _vp, _vp, _f, _f, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _i, _vp],
    "ftk_ssm_gates": [_vp, ctypes.c_longlong, _i, _vp, _vp, _vp, _vp, _i, _i, _vp],
    "ftk_ssm_output": [_vp, _vp, ctypes.c_longlong, _vp, _vp, ctypes.c_longlong, _i, _vp, _i, _f, _vp, _i, _i, _i, _vp],
    "ftk_norm_mean": [ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i, _i, _f, _vp, _i, _i, _vp],
}
_bound = False
_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (graph replays add their recorded count)."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _lib():
    global _bound
    lib = library.load()
    if not _bound:
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i
        _bound = True
    return lib


def _check(status: int, name: str, launches: int = 1) -> None:
    global _launches
    _launches += launches
    if status != 0:
        msg = library.load().ftk_last_error()
        raise KernelError(f"{name}: {msg.decode() if msg else 'error ' + str(status)}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _code(t: torch.Tensor, what: str) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)")


def _dev(t: Optional[torch.Tensor], what: str, dtype: Optional[torch.dtype] = None) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on '{t.device}', the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    return t.data_ptr()


def read_status() -> int:
    """Code left by a kernel whose bounded wait ran out since the last call (0 = none).  Waits
    for the device.  101-104 come from the tensor-core grouped GEMM (producer, accumulator
    hand-back, operand arrival, accumulator arrival)."""
    out = (ctypes.c_int * 2)()
    status = _lib().ftk_read_status(out)
    if status != 0:
        raise KernelError("read_status: " + library.load().ftk_last_error().decode())
    return int(out[0])


def check_status() -> None:
    code = read_status()
    if code:
        raise KernelError(f"a kernel gave up waiting (status {code}); its results are not valid")


def variant_counts(reset: bool = False) -> dict:
    """Launches so far by the form of kernel they took (``"attention: tcgen05, 128-row query tiles"``,
    ``"expert gate/up product: tcgen05, 64 tokens a tile, deep pipeline"``, ``"route sort: three passes over
    128-route segments"`` ...): what a step really ran, for tests and measurements.  Launches replayed from
    a CUDA graph were counted when the graph was recorded."""
    lib = _lib()
    need = lib.ftk_variant_counts(None, 0, 0)
    buf = ctypes.create_string_buffer(need + 256)
    lib.ftk_variant_counts(buf, len(buf), 1 if reset else 0)
    out = {}
    for line in buf.value.decode().splitlines():
        name, _, n = line.rpartition("\t")
        out[name] = int(n)
    return out


def debug_set_status(unit: int, code: int) -> None:
    """Write ``code`` into a status word from the host (``unit`` 0: grouped GEMM, 1: attention), as a
    kernel whose bounded wait ran out would have.  For tests of the error path; nothing waits."""
    _check(_lib().ftk_debug_set_status(int(unit), int(code)), "debug_set_status", 0)


def set_moe_tensor_cores(enabled: bool) -> None:
    """False sends bfloat16 grouped expert products to the CUDA-core kernels (comparisons only)."""
    _lib().ftk_set_moe_tensor_cores(1 if enabled else 0)


def set_moe_pairs(enabled: bool) -> None:
    """False keeps expert products with 128- and 256-token tiles on the one-CTA form of the tcgen05 kernel instead
    of pairs of CTAs (comparisons only)."""
    _lib().ftk_set_moe_pairs(1 if enabled else 0)


# --------------------------------------------------------------------------- elementwise
def embedding_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, :] = float32(table[ids[t], :])``; ``out`` is the 32-bit residual stream."""
    V, H = table.shape
    T = ids.shape[0]
    if out.shape != (T, H):
        raise KernelError(f"embedding_gather: out shape {tuple(out.shape)} != {(T, H)}")
    _check(_lib().ftk_embedding_gather(_dev(table, "table"), _code(table, "table"),
                                       _dev(ids, "ids", torch.int32), T, H, V,
                                       _dev(out, "out", torch.float32), _stream()),
           "embedding_gather")


def add_rmsnorm(x: Optional[torch.Tensor], residual: Optional[torch.Tensor], weight: torch.Tensor,
                eps: float, gemma: bool, out: torch.Tensor, out_f32: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> None:
    """RMSNorm with the residual sum fused in.

    ``z = x + residual`` in 32-bit (either may be None); without ``rows`` the sum is stored
    back to ``residual``; ``out = z * rsqrt(mean(z^2) + eps) * (1 + w)`` (``w`` when not
    ``gemma``).  With ``rows`` only those rows are read and ``out[i]`` belongs to
    ``rows[i]``; the residual stays as it is.  ``out_f32`` receives ``float32(out)``.
    """
    src = x if x is not None else residual
    if src is None:
        raise KernelError("add_rmsnorm: x and residual are both None")
    H = src.shape[-1]
    n_rows = rows.shape[0] if rows is not None else src.numel() // H
    if weight.shape != (H,):
        raise KernelError(f"add_rmsnorm: weight shape {tuple(weight.shape)} != {(H,)}")
    if out.numel() != n_rows * H:
        raise KernelError(f"add_rmsnorm: out has {out.numel()} elements, expected {n_rows * H}")
    if out_f32 is not None and out_f32.numel() != n_rows * H:
        raise KernelError("add_rmsnorm: out_f32 has the wrong size")
    _check(_lib().ftk_add_rmsnorm(_dev(x, "x"), _code(x, "x") if x is not None else F32,
                                  _dev(residual, "residual", torch.float32),
                                  _dev(weight, "weight", torch.float32),
                                  _dev(out, "out"), _code(out, "out"),
                                  _dev(out_f32, "out_f32", torch.float32),
                                  _dev(rows, "rows", torch.int32), n_rows, H, float(eps),
                                  1 if gemma else 0, _stream()), "add_rmsnorm")


def add_rmsnorm_routes(y: torch.Tensor, route_pos: torch.Tensor, top_k: int, shared: Optional[torch.Tensor],
                       residual: torch.Tensor, weight: torch.Tensor, eps: float, gemma: bool, out: torch.Tensor,
                       out_f32: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """:func:`moe_combine` and :func:`add_rmsnorm` in one pass: the row added to ``residual[t]`` is
    ``sum_j y[route_pos[t*k + j]] (+ shared[t])``, a 32-bit sum in route order rounded to ``y``'s type."""
    R, H = y.shape
    T = residual.numel() // H
    n_rows = rows.shape[0] if rows is not None else T
    if route_pos.numel() != T * top_k or weight.shape != (H,) or out.numel() != n_rows * H:
        raise KernelError("add_rmsnorm_routes: shapes do not agree")
    if shared is not None and (shared.shape != (T, H) or shared.dtype != y.dtype):
        raise KernelError("add_rmsnorm_routes: shared must be [tokens, hidden] of y's dtype")
    if out_f32 is not None and out_f32.numel() != n_rows * H:
        raise KernelError("add_rmsnorm_routes: out_f32 has the wrong size")
    _check(_lib().ftk_add_rmsnorm_routes(_dev(y, "y"), _code(y, "y"), _dev(route_pos, "route_pos", torch.int32), top_k, R,
                                         _dev(shared, "shared"), _dev(residual, "residual", torch.float32),
                                         _dev(weight, "weight", torch.float32), _dev(out, "out"), _code(out, "out"),
                                         _dev(out_f32, "out_f32", torch.float32), _dev(rows, "rows", torch.int32),
                                         n_rows, H, float(eps), 1 if gemma else 0, _stream()), "add_rmsnorm_routes")


def act_and_mul(gate_up: torch.Tensor, out: torch.Tensor, act: str, alpha: float, limit: float) -> None:
    """``out = act(gate_up[:, :I], gate_up[:, I:])`` with ``act`` silu or swigluoai."""
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError("act_and_mul: out must be [rows, I] of the input's dtype")
    _check(_lib().ftk_act_and_mul(_dev(gate_up, "gate_up"), _code(gate_up, "gate_up"), n, two_i // 2,
                                  ACT_CODES[act], float(alpha), float(limit), _dev(out, "out"),
                                  _stream()), "act_and_mul")


def table_update(table: torch.Tensor, updates: torch.Tensor, n_updates: int) -> None:
    """``table.flat[updates[i, 0]] = updates[i, 1]`` for ``i < n_updates``; negative indices are skipped."""
    if updates.numel() < 2 * n_updates:
        raise KernelError("table_update: updates shorter than n_updates")
    _check(_lib().ftk_table_update(_dev(table, "table", torch.int32), table.numel(),
                                   _dev(updates, "updates", torch.int32), n_updates, _stream()),
           "table_update")


def copy_tokens(dst: torch.Tensor, pairs: torch.Tensor, src: torch.Tensor, n: int, vocab: int) -> None:
    """``dst[pairs[i, 0]] = src[pairs[i, 1]]`` for ``i < n`` (negative indices skipped; values outside
    the vocabulary become 0): tokens sampled on the device become the next step's inputs."""
    if pairs.numel() < 2 * n:
        raise KernelError("copy_tokens: pairs shorter than n")
    _check(_lib().ftk_copy_tokens(_dev(dst, "dst", torch.int32), dst.numel(), _dev(pairs, "pairs", torch.int32),
                                  _dev(src, "src", torch.int32), src.numel(), n, vocab, _stream()), "copy_tokens")


def cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """``dst = src`` converted between float32 and bfloat16 (round to nearest even)."""
    if src.numel() != dst.numel():
        raise KernelError("cast: sizes differ")
    _check(_lib().ftk_cast(_dev(src, "src"), _code(src, "src"), _dev(dst, "dst"), _code(dst, "dst"),
                           src.numel(), _stream()), "cast")


# --------------------------------------------------------------------------- attention
def norm_rope_store(x: torch.Tensor, head_dim: int, rotary_dim: int, positions: torch.Tensor,
                    rope_table: Optional[torch.Tensor], eps: float, gemma: bool,
                    sections: Sequence[dict]) -> None:
    """Per-head RMSNorm, partial NeoX rotation and scatter of projected heads, in one pass.

    ``x [T, n_heads_total * head_dim]`` is cut into sections of whole heads.  A section is a
    dict: ``first_head``, ``n_heads``, ``norm_weight`` (float32 ``[head_dim]`` or None),
    ``rotate`` (bool), and one destination: ``dense_out [T, n_heads, head_dim]`` or
    ``slab [pages, n_heads, page_size, head_dim]`` with ``slot_map [T]`` (slot = page *
    page_size + offset, negative = skip).  ``rope_table [max_pos, rotary_dim]`` holds
    cos then sin of ``position * inv_freq`` in float32.

    Optional keys of a section: ``bias`` (float32 ``[n_heads * head_dim]``, added first),
    ``pos_scale`` (float32 ``[positions]``, the heads are multiplied last by the entry of the
    token's position), ``dst_head_dim`` (the destination's rows are that long, zero-filled past
    ``head_dim``).
    """
    T = x.shape[0]
    n_total = x.shape[1] // head_dim
    arr = (_Section * len(sections))()
    keep = []
    for i, s in enumerate(sections):
        if s["first_head"] + s["n_heads"] > n_total:
            raise KernelError("norm_rope_store: section exceeds the heads of x")
        arr[i].first_head = s["first_head"]
        arr[i].n_heads = s["n_heads"]
        arr[i].norm_weight = _dev(s.get("norm_weight"), "norm_weight", torch.float32)
        arr[i].rotate = 1 if s.get("rotate") else 0
        dense, slab = s.get("dense_out"), s.get("slab")
        if (dense is None) == (slab is None):
            raise KernelError("norm_rope_store: a section needs exactly one of dense_out and slab")
        dst_dim = int(s.get("dst_head_dim") or head_dim)
        arr[i].dst_head_dim = dst_dim if dst_dim != head_dim else 0
        bias, pos_scale = s.get("bias"), s.get("pos_scale")
        if bias is not None and bias.numel() != s["n_heads"] * head_dim:
            raise KernelError("norm_rope_store: a section's bias must hold n_heads * head_dim entries")
        arr[i].bias = _dev(bias, "bias", torch.float32)
        arr[i].pos_scale = _dev(pos_scale, "pos_scale", torch.float32)
        arr[i].pos_scale_len = pos_scale.numel() if pos_scale is not None else 0
        if dense is not None:
            if dense.dtype != x.dtype or dense.numel() != T * s["n_heads"] * dst_dim:
                raise KernelError("norm_rope_store: dense_out has the wrong dtype or size")
            arr[i].dense_out = _dev(dense, "dense_out")
        else:
            if slab.dtype != x.dtype or slab.dim() != 4 or slab.shape[1] != s["n_heads"] \
                    or slab.shape[3] != dst_dim:
                raise KernelError("norm_rope_store: slab must be [pages, n_heads, page_size, head_dim]")
            arr[i].slab = _dev(slab, "slab")
            arr[i].slot_map = _dev(s["slot_map"], "slot_map", torch.int32)
            if s["slot_map"].shape[0] < T:
                raise KernelError("norm_rope_store: slot_map shorter than the tokens")
            arr[i].num_pages = slab.shape[0]
            arr[i].page_size = slab.shape[2]
        keep.append(s)
    if rotary_dim:
        if rope_table is None or rope_table.shape[1] != rotary_dim:
            raise KernelError("norm_rope_store: rope_table must be [max_pos, rotary_dim]")
    max_pos = rope_table.shape[0] if rope_table is not None else 0
    _check(_lib().ftk_norm_rope_store(_dev(x, "x"), _code(x, "x"), T, x.shape[1], head_dim, rotary_dim,
                                      _dev(positions, "positions", torch.int32),
                                      _dev(rope_table, "rope_table", torch.float32), max_pos,
                                      float(eps), 1 if gemma else 0, len(sections), arr, _stream()),
           "norm_rope_store")


def paged_attention(q: torch.Tensor, k_slab: torch.Tensor, v_slab: torch.Tensor,
                    block_table: torch.Tensor, seg_info: torch.Tensor, n_segs: int,
                    items: torch.Tensor, n_items: int, part_o: Optional[torch.Tensor],
                    part_ml: Optional[torch.Tensor], out: torch.Tensor, tile_rows: int, scale: float,
                    window: Optional[int], sel: Optional[torch.Tensor] = None, block_size: int = 0,
                    few_rows: bool = False, dist_bias: Optional[torch.Tensor] = None, kv_split: int = 1,
                    sink: Any = None) -> None:
    """Causal softmax attention of the step's queries over the paged keys and values.

    ``q, out [T, Hq, D]``; slabs ``[pages, Hkv, page_size, D]``; ``block_table [rows, width]``
    page ids; ``seg_info [S, 4]`` = q_start, q_len, kv_len, block-table row; ``items [W, 8]``
    from :func:`freetoken_b200.engine.attention_plan.build_plan`; ``part_o [slots, Hkv,
    tile_rows, D]`` and ``part_ml [slots, Hkv, tile_rows, 2]`` float32 scratch for split
    tiles.  Query ``t`` of a segment sits at position ``kv_len - q_len + t`` and reads keys at
    positions ``<=`` its own (and ``>`` its own minus ``window`` when a window is given).

    Block-sparse layers pass ``sel [T, Hkv, topk]`` (chosen key blocks of ``block_size`` positions
    per token and KV head, ascending, -1 padded, from :func:`sparse_select`); a query then reads only
    the keys of its chosen blocks, the work items hold one token each and their key ranges count
    chosen keys.

    ``few_rows`` (with ``tile_rows = 16``, bfloat16) runs the tcgen05 kernel in its form for decode
    steps (one warp takes the softmax of a tile's at most 16 rows); its work list has key pieces that
    are multiples of 128 (``build_plan(..., key_tile=128)``).

    ``dist_bias [Hq, L]`` (float32) adds ``dist_bias[h, min(i - j, L - 1)]`` to the scaled score of query
    position ``i`` and key position ``j`` (a learned bias by distance; not multiplied by ``scale``).
    ``v_slab`` may be ``k_slab`` itself (values that are the keys): each key tile is then brought in once.
    ``kv_split > 1`` (more query heads per KV head than a tile has rows): every KV head is taken as that many
    heads of the same keys with a share of its query heads each; the work list and the scratch are then made for
    ``Hkv * kv_split`` heads.  Not with the tcgen05 kernels.
    Of the tcgen05 kernels the ones with one query tile a piece (128 rows, or at most 16) take the bias; with
    one slab for keys and values their key tile in shared memory serves both products.

    ``sink`` (a logit, a float32 tensor ``[Hq]`` of one logit per query head, or None): the softmax's denominator
    also holds ``e^sink``, a key without a value, so a row's weights are ``e^(s_j) / (e^sink + sum_i e^(s_i))``.  A tile that is split along the keys gets it once,
    in the merge.  Not with block selection.  Of the tcgen05 kernels the one with 128-row tiles takes a window and a
    sink (its work list then starts every piece on a key tile: ``build_plan(..., window, key_tile=128)``), also with
    one slab for keys and values, and a sink together with a bias by distance.
    """
    T, Hq, D = q.shape
    pages, Hkv, P, D2 = k_slab.shape
    if D2 != D or v_slab.shape != k_slab.shape or Hq % Hkv:
        raise KernelError("paged_attention: q / slab shapes do not agree")
    if out.shape != q.shape or out.dtype != q.dtype or k_slab.dtype != q.dtype:
        raise KernelError("paged_attention: dtypes or out shape do not agree")
    n_slots = part_o.shape[0] if part_o is not None else 0
    sink_heads = None
    if isinstance(sink, torch.Tensor):
        if sink.shape != (Hq,):
            raise KernelError("paged_attention: a sink per head must be [Hq]")
        sink_heads, sink = _dev(sink, "sink", torch.float32), 0.0
    kv_split = max(1, int(kv_split))
    Hv = Hkv * kv_split
    if kv_split > 1 and ((Hq // Hkv) % kv_split or sel is not None or tile_rows in (128, 256) or few_rows):
        raise KernelError("paged_attention: kv_split must divide the query heads per KV head (no tcgen05, no selection)")
    if part_o is not None and (part_o.shape[1:] != (Hv, tile_rows, D) or part_ml is None
                               or part_ml.shape != (n_slots, Hv, tile_rows, 2)):
        raise KernelError("paged_attention: scratch shapes do not match tile_rows / heads")
    if few_rows and tile_rows != 16:
        raise KernelError(f"paged_attention: few_rows goes with tiles of 16 rows, got {tile_rows}")
    if tile_rows in (128, 256) or few_rows:
        # bfloat16 steps on the tcgen05 kernels: one query tile per CTA, a pair of them, or tiles of a few rows
        if sel is not None or q.dtype != torch.bfloat16:
            raise KernelError("paged_attention: the tcgen05 kernels take bfloat16 without block selection")
        if window or sink is not None or dist_bias is not None:
            # the form with one 128-row query tile a piece takes a window, a sink and a bias by distance (a bias not
            # together with a window); the form for tiles of at most 16 rows takes the bias alone
            if (window or sink is not None) and (tile_rows != 128 or few_rows):
                raise KernelError("paged_attention: of the tcgen05 kernels the one with 128-row tiles takes a window or a sink")
            if dist_bias is not None and (tile_rows == 256 or window or dist_bias.dim() != 2 or dist_bias.shape[0] != Hq):
                raise KernelError("paged_attention: of the tcgen05 kernels the ones with one query tile a piece take a "
                                  "distance bias [Hq, L] (no window)")
            ex = _AttnExtras(_dev(dist_bias, "dist_bias", torch.float32), dist_bias.shape[1] if dist_bias is not None else 0,
                             1, 0 if sink is None else 1, 0.0 if sink is None else float(sink), sink_heads)
            what = "distance bias" if dist_bias is not None else "window or sink"
            _check(_lib().ftk_paged_attention_tc_ex(
                _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"),
                _dev(block_table, "block_table", torch.int32), block_table.shape[1],
                _dev(seg_info, "seg_info", torch.int32), n_segs,
                _dev(items, "items", torch.int32), n_items,
                _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
                _dev(out, "out"), T, Hq, Hkv, D, P, pages, float(scale), int(window) if window else 0, ctypes.byref(ex),
                1 if few_rows else 0, _stream()),
                f"paged_attention (tcgen05, {what})", 2 if n_slots else 1)
            return
        fn = (_lib().ftk_paged_attention_tc_few if few_rows else
              _lib().ftk_paged_attention_tc_pair if tile_rows == 256 else _lib().ftk_paged_attention_tc)
        _check(fn(
            _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1],
            _dev(seg_info, "seg_info", torch.int32), n_segs,
            _dev(items, "items", torch.int32), n_items,
            _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
            _dev(out, "out"), T, Hq, Hkv, D, P, pages, float(scale), 0, _stream()),
            "paged_attention (tcgen05)", 2 if n_slots else 1)
        return
    if sel is not None:
        if sink is not None:
            raise KernelError("paged_attention: a sink cannot be combined with block selection")
        if sel.dim() != 3 or sel.shape[0] < T or sel.shape[1] != Hkv or block_size < 1:
            raise KernelError("paged_attention: sel must be [T, Hkv, topk] with a positive block_size")
        _check(_lib().ftk_paged_attention_sparse(
            _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"), _code(q, "q"),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1],
            _dev(seg_info, "seg_info", torch.int32), n_segs,
            _dev(items, "items", torch.int32), n_items,
            _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
            _dev(out, "out"), Hq, Hkv, D, P, pages, tile_rows, float(scale),
            _dev(sel, "sel", torch.int32), sel.shape[2], int(block_size), _stream()),
            "paged_attention (block-sparse)", 2 if n_slots else 1)
        return
    if dist_bias is not None or kv_split > 1 or sink is not None:
        if dist_bias is not None and (dist_bias.dim() != 2 or dist_bias.shape[0] != Hq or dist_bias.shape[1] < 1):
            raise KernelError("paged_attention: dist_bias must be [Hq, L]")
        ex = _AttnExtras(_dev(dist_bias, "dist_bias", torch.float32), dist_bias.shape[1] if dist_bias is not None else 0,
                         kv_split, 0 if sink is None else 1, 0.0 if sink is None else float(sink), sink_heads)
        _check(_lib().ftk_paged_attention_ex(
            _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"), _code(q, "q"),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1],
            _dev(seg_info, "seg_info", torch.int32), n_segs,
            _dev(items, "items", torch.int32), n_items,
            _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
            _dev(out, "out"), Hq, Hkv, D, P, pages, tile_rows, float(scale),
            int(window) if window else 0, ctypes.byref(ex), _stream()), "paged_attention (with options)",
            2 if n_slots else 1)
        return
    _check(_lib().ftk_paged_attention(
        _dev(q, "q"), _dev(k_slab, "k_slab"), _dev(v_slab, "v_slab"), _code(q, "q"),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(seg_info, "seg_info", torch.int32), n_segs,
        _dev(items, "items", torch.int32), n_items,
        _dev(part_o, "part_o", torch.float32), _dev(part_ml, "part_ml", torch.float32), n_slots,
        _dev(out, "out"), Hq, Hkv, D, P, pages, tile_rows, float(scale),
        int(window) if window else 0, _stream()), "paged_attention", 2 if n_slots else 1)


def attention_tc_fits(head_dim: int, page_size: int, group: int) -> bool:
    """Whether the tcgen05 attention kernel (tiles of 128 query rows) takes these sizes."""
    return bool(_lib().ftk_attention_tc_fits(head_dim, page_size, group))


def attention_tc_few_fits(head_dim: int, page_size: int, group: int) -> bool:
    """Whether the tcgen05 attention kernel takes these sizes in its form for tiles of at most 16 rows."""
    return bool(_lib().ftk_attention_tc_few_fits(head_dim, page_size, group))


def sparse_score_fits(n_heads: int, dim: int, block_size: int) -> bool:
    """Whether bfloat16 block scores of these sizes are taken on the tensor cores (given a ``scores`` scratch)."""
    return bool(_lib().ftk_sparse_score_fits(n_heads, dim, block_size))


def sparse_select(iq: torch.Tensor, ik_slab: torch.Tensor, block_table: torch.Tensor, seg_info: torch.Tensor,
                  n_segs: int, block_size: int, local_blocks: int, init_blocks: int, max_blocks: int,
                  sel: torch.Tensor, scores: Optional[torch.Tensor] = None, live_blocks: int = 0) -> None:
    """Key blocks each new token of a block-sparse layer attends to.

    ``iq [T, Hi, Di]`` index queries, ``ik_slab [pages, 1, page_size, Di]`` cached index keys.  A
    block's score is the largest ``iq . ik`` over its visible positions; the first ``init_blocks``
    and the newest ``local_blocks`` blocks are always taken; the ``min(topk, visible)`` best go to
    ``sel [T, Hi, topk]`` in ascending order, padded with -1.  ``max_blocks`` bounds the blocks of
    the longest request (sizes the kernel's shared memory).  ``scores [T, Hi, max_blocks]`` float32 scratch lets
    bfloat16 scores be contracted on the tensor cores (:func:`sparse_score_fits`), every key read once per
    tile of tokens; without it a CTA per token and head walks the blocks.  ``live_blocks`` (0 = ``max_blocks``):
    blocks that the longest request of this step can hold, which bounds the launch; a step replayed from a
    CUDA graph must give a bound that holds for every replay."""
    T, Hi, Di = iq.shape
    pages, one, P, Di2 = ik_slab.shape
    if one != 1 or Di2 != Di or ik_slab.dtype != iq.dtype:
        raise KernelError("sparse_select: ik_slab must be [pages, 1, page_size, Di] of iq's dtype")
    if sel.dim() != 3 or sel.shape[0] < T or sel.shape[1] != Hi:
        raise KernelError("sparse_select: sel must be [T, Hi, topk]")
    if scores is not None and (scores.dtype != torch.float32 or scores.numel() < T * Hi * max_blocks):
        raise KernelError("sparse_select: scores must hold [T, Hi, max_blocks] float32")
    _check(_lib().ftk_sparse_select(_dev(iq, "iq"), _dev(ik_slab, "ik_slab"), _code(iq, "iq"),
                                    _dev(block_table, "block_table", torch.int32), block_table.shape[1],
                                    _dev(seg_info, "seg_info", torch.int32), n_segs, T, Hi, Di, P, pages,
                                    int(block_size), sel.shape[2], int(local_blocks), int(init_blocks),
                                    int(max_blocks), int(live_blocks), _dev(sel, "sel", torch.int32),
                                    _dev(scores, "scores", torch.float32), _stream()), "sparse_select",
           2 if scores is not None else 1)


# --------------------------------------------------------------------------- experts
def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, scoring: str,
                scale: float, ids: torch.Tensor, weights: torch.Tensor, n_parts: int = 1) -> None:
    """Expert choice from float32 router logits ``[T, E]``.

    sigmoid: ``s = sigmoid(l)``; choice by ``s + bias``; ``w = s[ids] / (sum + 1e-20) * scale``.
    softmax: ``s = softmax(l)``; choice by ``s (+ bias)``; ``w = s[ids] / sum * scale``.
    softmax_of_chosen: the bias belongs to the logit: choice by ``l + bias``; ``w = softmax((l + bias)[ids]) * scale``.
    The largest goes first; the lower expert index wins a tie.

    With ``n_parts > 1`` the logits come as ``[T, n_parts * E]``: a token's logit of expert ``e`` is the
    32-bit sum of ``logits[t, q * E + e]`` over the parts ``q`` in their order.
    """
    T, PE = logits.shape
    if n_parts < 1 or PE % n_parts or not logits.is_contiguous():
        raise KernelError("router_topk: logits must be contiguous [T, n_parts * E]")
    E = PE // n_parts
    if ids.shape != (T, top_k) or weights.shape != (T, top_k):
        raise KernelError("router_topk: ids / weights must be [T, top_k]")
    if bias is not None and bias.shape != (E,):
        raise KernelError("router_topk: bias must be [E]")
    _check(_lib().ftk_router_topk(_dev(logits, "logits", torch.float32), int(n_parts), _dev(bias, "bias", torch.float32),
                                  T, E, top_k, SCORE_CODES[scoring], float(scale),
                                  _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                                  _stream()), "router_topk")


def moe_permute(topk_ids: torch.Tensor, n_experts: int, expert_counts: torch.Tensor,
                expert_offsets: torch.Tensor, sorted_routes: torch.Tensor, route_pos: torch.Tensor) -> None:
    """Sort the routes ``(t, j)`` by expert, keeping their order within an expert.

    ``expert_counts [E]``: routes per expert;
    ``expert_offsets [E + 1]``: rows of expert ``e`` are ``[offsets[e], offsets[e+1])``;
    ``sorted_routes [T*k]``: route index ``t*k + j`` at each sorted row;
    ``route_pos [T*k]``: sorted row of each route."""
    T, k = topk_ids.shape
    if expert_offsets.shape != (n_experts + 1,) or expert_counts.shape != (n_experts,) \
            or sorted_routes.numel() != T * k \
            or route_pos.numel() != T * k:
        raise KernelError("moe_permute: output shapes are wrong")
    _check(_lib().ftk_moe_permute(_dev(topk_ids, "topk_ids", torch.int32), T, k, n_experts,
                                  _dev(expert_counts, "expert_counts", torch.int32),
                                  _dev(expert_offsets, "expert_offsets", torch.int32),
                                  _dev(sorted_routes, "sorted_routes", torch.int32),
                                  _dev(route_pos, "route_pos", torch.int32), _stream()), "moe_permute", 2)


LINEAR_PAD_ROWS = 16


# Steps of this many tokens stream the weights with this library's own kernel (0 switches it off).  The
# kernel takes up to four rows, but measured on B200 (3072 x 8192 and 6144 x 3072, inside a decode step) it
# wins against the library's 16-row product only for one: 10.2 / 9.3 against 11.2 / 11.1 microseconds; at
# two rows 12.9 / 14.5, at four 17 / 19.6 (the lanes run out of issue slots, not of bandwidth).
SMALL_LINEAR_MAX_TOKENS = 1


def small_linear_fits(n_tokens: int, n_out: int, k: int) -> bool:
    return bool(_lib().ftk_small_linear_fits(n_tokens, n_out, k))


def small_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` in bfloat16 for one to four rows of ``x``: every SM streams its share of the
    weight rows once, 32-bit sums (``csrc/gemv.cu``)."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape != (N, K) or out.shape != (T, N) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 \
            or out.dtype != torch.bfloat16:
        raise KernelError("small_linear: bfloat16 x [T, K], w [N, K], out [T, N] expected")
    _check(_lib().ftk_small_linear(_dev(x, "x"), _dev(w, "w"), _dev(out, "out"), T, N, K, _stream()), "small_linear")


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> None:
    """``out = x @ w^T`` (``x [T, K]``, ``w [N, K]``, ``out [T, N]``): by the library, as in the reference
    (python/freetoken/layers/linear.py:66-70), except for bfloat16 steps of up to four tokens, whose
    product is a stream over the weights that :func:`small_linear` does faster than the library's choice
    of tile (measured on B200, 3072 x 8192 for one token: see the design notes).

    For fewer than 16 rows of bfloat16 and a weight that is at least as long as it is tall, the
    product is taken over 16 rows of the same buffers (the rows past ``T`` hold whatever the
    buffers hold and their results are never read): measured on B200, the library's choice for 16
    rows runs 3072 x 6144 in 10.9 microseconds, its choice for 8 rows in 16.6."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape != (N, K) or out.shape != (T, N):
        raise KernelError("linear: shapes do not agree")
    if bias is not None:  # ``out = x @ w^T + bias``: the bias is added to the 32-bit sums by the library's product
        if bias.shape != (N,) or bias.dtype != x.dtype:
            raise KernelError("linear: bias must be [N] of x's dtype")
        torch.addmm(bias, x, w.t(), out=out)
        return
    if (T <= SMALL_LINEAR_MAX_TOKENS and x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous()
            and w.is_contiguous() and out.is_contiguous() and small_linear_fits(T, N, K)):
        small_linear(x, w, out)
        return
    P = LINEAR_PAD_ROWS
    if (T < P and K >= N and x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous() and out.is_contiguous()
            and _room(x) >= P * K and _room(out) >= P * N):
        torch.matmul(x.as_strided((P, K), (K, 1)), w.t(), out=out.as_strided((P, N), (N, 1)))
    else:
        torch.matmul(x, w.t(), out=out)


def linear_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` kept as the 32-bit sums of the library's product (``out`` float32), for a result
    that enters 32-bit arithmetic (a recurrence's decay logits).  ``x`` may be a view of adjacent columns."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape != (N, K) or out.shape != (T, N) or out.dtype != torch.float32 or x.dtype != w.dtype:
        raise KernelError("linear_f32: shapes or dtypes do not agree")
    if x.dtype == torch.float32:
        torch.matmul(x, w.t(), out=out)
    else:
        torch.mm(x, w.t(), out_dtype=torch.float32, out=out)


def _room(t: torch.Tensor) -> int:
    """Elements from the tensor's first one to the end of its storage."""
    return t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()


def moe_route_fits(n_tokens: int, hidden: int, n_experts: int, top_k: int) -> bool:
    """Whether :func:`moe_route` takes these sizes (small steps only)."""
    return bool(_lib().ftk_moe_route_fits(n_tokens, hidden, n_experts, top_k))


def moe_route(x: torch.Tensor, gate_w: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, scoring: str,
              scale: float, logits: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
              expert_counts: Optional[torch.Tensor] = None, expert_offsets: Optional[torch.Tensor] = None,
              sorted_routes: Optional[torch.Tensor] = None, route_pos: Optional[torch.Tensor] = None) -> None:
    """``logits = x @ gate_w^T`` in float32, then :func:`router_topk` and :func:`moe_permute`, in one launch.
    Without the four outputs of the sort only ids and weights are made (the few-token expert kernels take
    the routes in token order)."""
    T, H = x.shape
    E = gate_w.shape[0]
    if gate_w.shape != (E, H) or logits.shape != (T, E) or ids.shape != (T, top_k) or weights.shape != (T, top_k):
        raise KernelError("moe_route: shapes do not agree")
    sort = expert_counts is not None
    if sort and (expert_offsets is None or sorted_routes is None or route_pos is None):
        raise KernelError("moe_route: give all four outputs of the sort, or none")
    if sort and (expert_offsets.shape != (E + 1,) or expert_counts.shape != (E,) or sorted_routes.numel() != T * top_k
                 or route_pos.numel() != T * top_k):
        raise KernelError("moe_route: output shapes are wrong")
    if bias is not None and bias.shape != (E,):
        raise KernelError("moe_route: bias must be [E]")
    _check(_lib().ftk_moe_route(_dev(x, "x", torch.float32), _dev(gate_w, "gate_w", torch.float32),
                                _dev(bias, "bias", torch.float32), T, H, E, top_k, SCORE_CODES[scoring], float(scale),
                                _dev(logits, "logits", torch.float32), _dev(ids, "ids", torch.int32),
                                _dev(weights, "weights", torch.float32),
                                _dev(expert_counts, "expert_counts", torch.int32),
                                _dev(expert_offsets, "expert_offsets", torch.int32),
                                _dev(sorted_routes, "sorted_routes", torch.int32),
                                _dev(route_pos, "route_pos", torch.int32), 1 if sort else 0, _stream()), "moe_route")


def moe_small_fits(n_tokens: int, hidden: int, inter: int, top_k: int) -> bool:
    """Whether the few-token expert kernels (:func:`moe_small_gate_up`, :func:`moe_small_down`) take a step."""
    return bool(_lib().ftk_moe_small_fits(n_tokens, hidden, inter, top_k))


def moe_small_gate_up(h: torch.Tensor, ids: torch.Tensor, w1: torch.Tensor, act: str, alpha: float, limit: float,
                      out: torch.Tensor) -> None:
    """``out[t*k + j] = act(h[t] W1[ids[t, j]]^T)`` for a step of up to four tokens: routes in token order,
    no sort, no gathered copy; ``w1 [E, 2I, H]`` rows gate then up, bfloat16."""
    T, H = h.shape
    k = ids.shape[1]
    E, two_i, H2 = w1.shape
    if H2 != H or ids.shape != (T, k) or out.shape != (T * k, two_i // 2) or h.dtype != torch.bfloat16 \
            or w1.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("moe_small_gate_up: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_small_gate_up(_dev(h, "h"), _dev(ids, "ids", torch.int32), _dev(w1, "w1"), _dev(out, "out"),
                                        T, k, E, H, two_i // 2, ACT_CODES[act], float(alpha), float(limit), _stream()),
           "moe_small_gate_up")


def moe_small_down(a: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w2: torch.Tensor,
                   out: torch.Tensor) -> None:
    """``out[r] = (a[r] W2[ids.flat[r]]^T) * weights.flat[r]`` for the routes of up to four tokens.
    ``ids`` are read while the launch before this one may still run (they are the routing kernel's, which
    ended before :func:`moe_small_gate_up` began): a caller that writes them just before must do so with an
    ordinary launch."""
    R, I = a.shape
    E, H, I2 = w2.shape
    T, k = ids.shape
    if I2 != I or R != T * k or weights.numel() != R or out.shape != (R, H) or a.dtype != torch.bfloat16 \
            or w2.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("moe_small_down: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_small_down(_dev(a, "a"), _dev(ids, "ids", torch.int32), _dev(weights, "weights", torch.float32),
                                     _dev(w2, "w2"), _dev(out, "out"), T, k, E, H, I, _stream()), "moe_small_down")


def moe_gather(h: torch.Tensor, sorted_routes: torch.Tensor, top_k: int, out: torch.Tensor) -> None:
    """``out[r, :] = h[sorted_routes[r] // top_k, :]``."""
    T, H = h.shape
    R = sorted_routes.numel()
    if out.shape != (R, H) or out.dtype != h.dtype:
        raise KernelError("moe_gather: out must be [routes, hidden] of h's dtype")
    _check(_lib().ftk_moe_gather(_dev(h, "h"), _code(h, "h"), _dev(sorted_routes, "sorted_routes", torch.int32),
                                 R, top_k, H, _dev(out, "out"), _stream()), "moe_gather")


def moe_gemm1_act(x_sorted: torch.Tensor, w1: torch.Tensor, expert_offsets: torch.Tensor,
                  act: str, alpha: float, limit: float, out: torch.Tensor) -> None:
    """``out[r] = act(x[r] W1[e]^T)`` for the rows of each expert; ``w1 [E, 2I, H]`` rows gate then up."""
    R, H = x_sorted.shape
    E, two_i, H2 = w1.shape
    if H2 != H or two_i % 2 or out.shape != (R, two_i // 2) or w1.dtype != x_sorted.dtype \
            or out.dtype != x_sorted.dtype:
        raise KernelError("moe_gemm1_act: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_gemm1_act(_dev(x_sorted, "x_sorted"), _dev(w1, "w1"), _code(w1, "w1"),
                                    _dev(expert_offsets, "expert_offsets", torch.int32), E, R, H,
                                    two_i // 2, ACT_CODES[act], float(alpha), float(limit),
                                    _dev(out, "out"), _stream()), "moe_gemm1_act")


def moe_gemm1_gather_fits(dtype: torch.dtype, hidden: int, inter: int, n_experts: int, n_routes: int) -> bool:
    """Whether :func:`moe_gemm1_act_gather` takes these sizes (bfloat16 on the tensor cores, few enough routes
    per expert for token tiles of at most 32 rows)."""
    return dtype == torch.bfloat16 and bool(_lib().ftk_moe_gemm1_gather_fits(hidden, inter, n_experts, n_routes))


def moe_gemm1_act_gather(h: torch.Tensor, sorted_routes: torch.Tensor, top_k: int, w1: torch.Tensor,
                         expert_offsets: torch.Tensor, act: str, alpha: float, limit: float, out: torch.Tensor) -> None:
    """:func:`moe_gather` and :func:`moe_gemm1_act` in one kernel: ``out[r] = act(h[sorted_routes[r] // top_k]
    W1[e]^T)`` for the rows ``r`` of each expert; ``h [T, H]`` holds the tokens in their own order."""
    T, H = h.shape
    E, two_i, H2 = w1.shape
    R = sorted_routes.numel()
    if H2 != H or two_i % 2 or out.shape != (R, two_i // 2) or w1.dtype != h.dtype or out.dtype != h.dtype \
            or h.dtype != torch.bfloat16 or R != T * top_k or not h.is_contiguous():
        raise KernelError("moe_gemm1_act_gather: shapes or dtypes do not agree")
    _check(_lib().ftk_moe_gemm1_act_gather(_dev(h, "h"), _dev(w1, "w1"),
                                           _dev(expert_offsets, "expert_offsets", torch.int32),
                                           _dev(sorted_routes, "sorted_routes", torch.int32), int(top_k), T, E, R, H,
                                           two_i // 2, ACT_CODES[act], float(alpha), float(limit),
                                           _dev(out, "out"), _stream()), "moe_gemm1_act_gather")


def moe_gemm2(a: torch.Tensor, w2: torch.Tensor, expert_offsets: torch.Tensor,
              sorted_routes: torch.Tensor, topk_weights: torch.Tensor, out: torch.Tensor) -> None:
    """``out[r] = (a[r] W2[e]^T) * topk_weights[sorted_routes[r]]``; ``w2 [E, H, I]``."""
    R, I = a.shape
    E, H, I2 = w2.shape
    if I2 != I or out.shape != (R, H) or w2.dtype != a.dtype or out.dtype != a.dtype:
        raise KernelError("moe_gemm2: shapes or dtypes do not agree")
    if topk_weights.numel() != R or sorted_routes.numel() != R:
        raise KernelError("moe_gemm2: one weight and one route per row expected")
    _check(_lib().ftk_moe_gemm2(_dev(a, "a"), _dev(w2, "w2"), _code(w2, "w2"),
                                _dev(expert_offsets, "expert_offsets", torch.int32),
                                _dev(sorted_routes, "sorted_routes", torch.int32),
                                _dev(topk_weights, "topk_weights", torch.float32), E, R, H, I,
                                _dev(out, "out"), _stream()), "moe_gemm2")


def moe_combine(y: torch.Tensor, route_pos: torch.Tensor, n_tokens: int, top_k: int,
                shared: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out[t] = sum_j y[route_pos[t*k + j]]`` in route order, 32-bit sum, ``+ shared[t]``."""
    R, H = y.shape
    if R != n_tokens * top_k or out.shape != (n_tokens, H) or out.dtype != y.dtype:
        raise KernelError("moe_combine: shapes or dtypes do not agree")
    if shared is not None and (shared.shape != out.shape or shared.dtype != y.dtype):
        raise KernelError("moe_combine: shared must match out")
    _check(_lib().ftk_moe_combine(_dev(y, "y"), _code(y, "y"), _dev(route_pos, "route_pos", torch.int32),
                                  n_tokens, top_k, H, _dev(shared, "shared"), _dev(out, "out"),
                                  _stream()), "moe_combine")


# --------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           u: torch.Tensor, out: torch.Tensor) -> None:
    """One token per row of float32 ``logits [R, V]``.

    ``temperature[r] <= 0``: argmax, lowest index on a tie.  Else ``p = softmax(logits / T)``;
    top-k keeps ``p >=`` the k-th largest value (``top_k <= 0`` keeps all); top-p then keeps
    ``p >= th`` for the largest ``th`` whose kept mass reaches ``top_p`` of the remaining mass;
    the token is the first index whose running kept mass exceeds ``u[r]`` times the kept mass.
    """
    R, V = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("u", u, torch.float32),
                        ("out", out, torch.int32)):
        if t.numel() < R:
            raise KernelError(f"sample: {name} has fewer than {R} entries")
    _check(_lib().ftk_sample(_dev(logits, "logits", torch.float32), R, V,
                             _dev(temperature, "temperature", torch.float32),
                             _dev(top_k, "top_k", torch.int32), _dev(top_p, "top_p", torch.float32),
                             _dev(u, "u", torch.float32), _dev(out, "out", torch.int32), _stream()),
           "sample")


# --------------------------------------------------------------------------- the 32-bit stream
NORM_NONE, NORM_DYNAMIC_TANH = 0, 1


def stream_add_norm(residual: Optional[torch.Tensor], out: Optional[torch.Tensor], x1: Optional[torch.Tensor] = None,
                    x2: Optional[torch.Tensor] = None, routed: Optional[tuple] = None, table: Optional[torch.Tensor] = None,
                    ids: Optional[torch.Tensor] = None, vec: Optional[torch.Tensor] = None,
                    norm: Optional[tuple] = None, rows: Optional[torch.Tensor] = None) -> None:
    """Several addends into the 32-bit stream and a norm without row statistics, in one pass.

    ``z[t] = residual[t] + x1[t] + x2[t] + sum_j y[route_pos[t k + j]] + table[ids[t]] + vec`` with every
    sum in 32 bits (each addend may be None; ``routed = (y, route_pos, top_k)``); without ``rows`` ``z`` is
    stored back to ``residual``.  ``norm = ("dynamic_tanh", weight, bias, alpha)`` (float32 ``[H]``, ``[H]``
    and one element) writes ``out = tanh(alpha z) weight + bias``; ``norm = None`` writes ``out = z`` when
    ``out`` is given.  With ``rows`` only those rows are taken and ``out[i]`` belongs to ``rows[i]``."""
    src = next((t for t in (residual, x1, x2, out) if t is not None), None)
    if src is None:
        raise KernelError("stream_add_norm: nothing to work on")
    H = src.shape[-1]
    total = (residual if residual is not None else src).numel() // H
    n_rows = rows.shape[0] if rows is not None else total
    a = _StreamNorm()
    dense = [t for t in (x1, x2, routed[0] if routed else None, table, out) if t is not None]
    dt = dense[0].dtype if dense else torch.float32
    if any(t.dtype != dt for t in dense):
        raise KernelError("stream_add_norm: addends, table and out must share one dtype")
    a.residual = _dev(residual, "residual", torch.float32)
    for name, t in (("x1", x1), ("x2", x2)):
        if t is not None and t.numel() != total * H:
            raise KernelError(f"stream_add_norm: {name} must be [tokens, hidden]")
        setattr(a, name, _dev(t, name))
    if routed is not None:
        y, pos, top_k = routed
        if y.dim() != 2 or y.shape[1] != H or pos.numel() != total * top_k:
            raise KernelError("stream_add_norm: routed rows / positions have the wrong shape")
        a.y, a.route_pos, a.top_k, a.n_routes = _dev(y, "y"), _dev(pos, "route_pos", torch.int32), int(top_k), y.shape[0]
    if table is not None:
        if ids is None or ids.numel() < total or table.dim() != 2 or table.shape[1] != H:
            raise KernelError("stream_add_norm: a table needs [vocab, hidden] rows and one id per token")
        a.table, a.ids, a.vocab = _dev(table, "table"), _dev(ids, "ids", torch.int32), table.shape[0]
    if vec is not None:
        if vec.numel() != H:
            raise KernelError("stream_add_norm: vec must hold hidden entries")
        a.vec = _dev(vec, "vec", torch.float32)
    if norm is not None:
        kind, w, b, alpha = norm
        if kind != "dynamic_tanh" or w.shape != (H,) or b.shape != (H,) or alpha.numel() != 1 or out is None:
            raise KernelError("stream_add_norm: norm must be ('dynamic_tanh', weight [H], bias [H], alpha [1]) with an out")
        a.norm = NORM_DYNAMIC_TANH
        a.weight, a.bias, a.alpha = (_dev(w, "weight", torch.float32), _dev(b, "bias", torch.float32),
                                     _dev(alpha, "alpha", torch.float32))
    if out is not None and out.numel() != n_rows * H:
        raise KernelError("stream_add_norm: out has the wrong size")
    a.out = _dev(out, "out")
    a.dtype = _code(dense[0], "stream_add_norm") if dense else F32
    a.rows = _dev(rows, "rows", torch.int32)
    a.n_rows, a.hidden = n_rows, H
    _check(_lib().ftk_stream_add_norm(ctypes.byref(a), _stream()), "stream_add_norm")


def head_gate(o: torch.Tensor, gates: torch.Tensor) -> None:
    """``o[t, h, :] *= sigmoid(gates[t, h])`` in place; ``gates`` may be a view of columns of a wider
    row-major tensor (its row stride is taken, its columns must be adjacent)."""
    T, Hq, D = o.shape
    if gates.shape != (T, Hq) or gates.dtype != o.dtype or gates.stride(1) != 1 or not gates.is_cuda:
        raise KernelError("head_gate: gates must be [T, heads] of o's dtype with adjacent columns")
    _check(_lib().ftk_head_gate(_dev(o, "o"), _code(o, "o"), gates.data_ptr(), gates.stride(0) if T > 1 else Hq, T, Hq, D,
                                _stream()), "head_gate")


def table_route(token_ids: torch.Tensor, table: torch.Tensor, n_experts: int, ids: torch.Tensor,
                weights: torch.Tensor) -> None:
    """``ids[t, j] = table[token_ids[t], j]``, ``weights[t, j] = 1 / top``: experts by a table over token ids."""
    V, k = table.shape
    T = ids.shape[0]
    if ids.shape != (T, k) or weights.shape != (T, k) or token_ids.numel() < T:
        raise KernelError("table_route: ids / weights must be [T, top]")
    _check(_lib().ftk_table_route(_dev(token_ids, "token_ids", torch.int32), _dev(table, "table", torch.int32), T, V, k,
                                  int(n_experts), 1.0 / k, _dev(ids, "ids", torch.int32),
                                  _dev(weights, "weights", torch.float32), _stream()), "table_route")


def scale_(x: torch.Tensor, s: float) -> None:
    """``x *= s`` for a float32 tensor."""
    _check(_lib().ftk_scale_f32(_dev(x, "x", torch.float32), x.numel(), float(s), _stream()), "scale")


def softcap_(x: torch.Tensor, cap: float) -> None:
    """``x <- cap * tanh(x / cap)`` for a float32 tensor."""
    if not cap > 0:
        raise KernelError("softcap: the cap must be positive")
    _check(_lib().ftk_softcap_f32(_dev(x, "x", torch.float32), x.numel(), float(cap), _stream()), "softcap")


GATE_CODES = {"sigmoid": 0, "silu": 1}


def postnorm_add_norm(x: torch.Tensor, routed, post_weight: torch.Tensor, post_eps: float, post_gemma: bool,
                      residual: torch.Tensor, pre_weight: Optional[torch.Tensor] = None, pre_eps: float = 0.0,
                      pre_gemma: bool = True, out: Optional[torch.Tensor] = None,
                      out_f32: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> None:
    """A sub-layer's output joins the 32-bit stream through an RMS norm of its own, and the stream is normed
    for the next sub-layer in the same pass:

    ``residual += a * rsqrt(mean(a^2) + post_eps) * w_post``, then (with ``pre_weight``)
    ``out = residual * rsqrt(mean(residual^2) + pre_eps) * w_pre`` (``w = 1 + weight`` in the Gemma form).

    ``a`` is row ``t`` of ``x``, or, with ``routed = (route_pos, top_k, shared or None)``, the 32-bit sum
    ``sum_j x[route_pos[t * top_k + j]] (+ shared[t])`` over a token's expert routes in route order.  With
    ``rows`` only those rows are normed into ``out`` and the stream stays as it is (``out[i]`` belongs to
    ``rows[i]``).  ``out_f32`` receives ``float32(out)``."""
    H = residual.shape[-1]
    n_rows = rows.shape[0] if rows is not None else residual.numel() // H
    if post_weight.shape != (H,) or x.shape[-1] != H or (pre_weight is not None and pre_weight.shape != (H,)):
        raise KernelError("postnorm_add_norm: widths do not agree")
    if pre_weight is None and (out is not None or out_f32 is not None or rows is not None):
        raise KernelError("postnorm_add_norm: an output needs the weight of the stream's norm")
    if pre_weight is not None and out is None:
        raise KernelError("postnorm_add_norm: the stream's norm needs an output")
    if out is not None and (out.numel() != n_rows * H or out.dtype != x.dtype):
        raise KernelError("postnorm_add_norm: out has the wrong size or dtype")
    if out_f32 is not None and out_f32.numel() != n_rows * H:
        raise KernelError("postnorm_add_norm: out_f32 has the wrong size")
    pos, top_k, shared, n_routes = None, 0, None, 0
    if routed is not None:
        pos, top_k, shared = routed
        n_routes = x.shape[0]
        if pos.numel() < residual.numel() // H * top_k or (shared is not None and shared.dtype != x.dtype):
            raise KernelError("postnorm_add_norm: routes do not match the rows")
    elif x.numel() < residual.numel():
        raise KernelError("postnorm_add_norm: x has fewer rows than the stream")
    _check(_lib().ftk_postnorm_add_norm(
        _dev(x, "x"), _code(x, "x"), _dev(pos, "route_pos", torch.int32), int(top_k), int(n_routes),
        _dev(shared, "shared"), _dev(post_weight, "post_weight", torch.float32), float(post_eps),
        1 if post_gemma else 0, _dev(residual, "residual", torch.float32),
        _dev(pre_weight, "pre_weight", torch.float32), float(pre_eps), 1 if pre_gemma else 0, _dev(out, "out"),
        _dev(out_f32, "out_f32", torch.float32), _dev(rows, "rows", torch.int32), n_rows, H, _stream()),
        "postnorm_add_norm")


def gated_heads(x: torch.Tensor, gates: torch.Tensor, out: torch.Tensor, dim: int, act: str = "sigmoid",
                norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0) -> None:
    """``out[t, h, :dim] = norm(x[t, h, :dim]) * act(gates[t, h * dim + :dim])``: a gate taken element by
    element from another projection of the same token, after an optional RMS norm over each head
    (``norm_weight [dim]``, plain weight).  ``x [T, heads, >= dim]`` is float32 or of ``out``'s dtype;
    ``out [T, heads, >= dim]`` may be ``x`` itself; columns past ``dim`` are left alone.  ``gates
    [T, heads * dim]`` may be a view of adjacent columns of a wider row-major tensor."""
    T, H, xs = x.shape
    if out.shape[:2] != (T, H) or out.shape[2] < dim or xs < dim or gates.shape != (T, H * dim):
        raise KernelError("gated_heads: shapes do not agree")
    if gates.dtype != out.dtype or gates.stride(1) != 1 or x.dtype not in (torch.float32, out.dtype):
        raise KernelError("gated_heads: gates must be of out's dtype with adjacent columns, x float32 or out's dtype")
    if norm_weight is not None and norm_weight.shape != (dim,):
        raise KernelError("gated_heads: norm_weight must be [dim]")
    if act not in GATE_CODES:
        raise KernelError(f"gated_heads: unknown gate '{act}'")
    if not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("gated_heads: x and out must be contiguous")
    _check(_lib().ftk_gated_heads(
        _dev(x, "x"), 1 if x.dtype == torch.float32 else 0, xs, gates.data_ptr(),
        gates.stride(0) if T > 1 else H * dim, _dev(norm_weight, "norm_weight", torch.float32), float(eps),
        GATE_CODES[act], _dev(out, "out"), out.shape[2], _code(out, "out"), T, H, dim, _stream()), "gated_heads")


def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, z_bias: Optional[torch.Tensor],
             tau: float, q_scale: float, state: torch.Tensor, state_slots: torch.Tensor, seg_info: torch.Tensor,
             n_segs: int, chunks: torch.Tensor, n_chunks: int, seg_chunks: torch.Tensor, any_single: bool,
             any_multi: bool, carry: Optional[torch.Tensor], decay_prod: Optional[torch.Tensor],
             out: torch.Tensor, k_fac: Optional[torch.Tensor] = None, a_head: Optional[torch.Tensor] = None,
             ones_col: bool = False, out_ones: Optional[torch.Tensor] = None, qk_div: int = 1) -> None:
    """Gated linear attention of the step's tokens, per (request, head):
    ``S <- diag(a_t) S + k_t v_t^T``, ``o_t = S^T (q_t q_scale)``, ``a_t = sigmoid(z_t + z_bias)^(1 / tau)``.

    ``q, k [T, H * D]`` and ``v [T, H * Dv]`` of the engine's dtype (views of adjacent columns of a wider
    tensor are fine); ``z [T, H * D]`` float32 (overwritten with the decays when a segment has several chunks); ``state [slots, H, D, Dv]`` float32, read from and left in
    the slot ``state_slots[segment]`` (a segment with ``kv_len == q_len`` starts from zero);
    ``chunks [n, 4]`` / ``seg_chunks [S, 2]`` from :func:`freetoken_b200.parts.gla.chunk_list`; ``carry
    [n, H, D, Dv]`` and ``decay_prod [n, H, D]`` float32 scratch for segments of several chunks;
    ``out [T, H, Dv]`` float32.

    ``k_fac [T, H]`` float32 multiplies a token's keys of a head (in 32 bits, as they are read); ``a_head [T, H]``
    float32 gives one decay per (token, head) for all key channels, and ``z`` is then ``None``; with ``ones_col``
    the state's last value column belongs to a value that is 1 for every token, and ``v`` is ``[T, H * (Dv - 1)]``
    (the sum of the keys under the same decays: a normaliser); with ``out_ones [T, H]`` that column's outputs go
    there and ``out`` is ``[T, H, Dv - 1]``.

    ``qk_div > 1``: queries and keys are shared by groups of that many heads (head ``h`` reads q/k head
    ``h // qk_div``), and ``q, k`` are ``[T, (H / qk_div) * D]``; with ``a_head`` only."""
    T = out.shape[0]
    H, D, Dv = state.shape[1], state.shape[2], state.shape[3]
    qk_div = int(qk_div)
    if qk_div < 1 or H % qk_div or (qk_div > 1 and a_head is None):
        raise KernelError("gla_scan: qk_div must divide the heads and goes with a decay per head")
    Hqk = H // qk_div
    if q.shape != (T, Hqk * D) or k.shape != (T, Hqk * D) or v.shape != (T, H * (Dv - (1 if ones_col else 0))) \
            or out.shape != (T, H, Dv - (1 if out_ones is not None else 0)) or (z is None) == (a_head is None) or (z is not None and z.shape != (T, H * D)):
        raise KernelError("gla_scan: shapes do not agree")
    if out_ones is not None and not ones_col:
        raise KernelError("gla_scan: out_ones goes with ones_col")
    for name, f in (("k_fac", k_fac), ("a_head", a_head), ("out_ones", out_ones)):
        if f is not None and (f.shape != (T, H) or not f.is_contiguous()):
            raise KernelError(f"gla_scan: {name} must be a contiguous [T, H]")
    if q.dtype != k.dtype or q.dtype != v.dtype or q.stride(1) != 1 or k.stride(1) != 1 or v.stride(1) != 1:
        raise KernelError("gla_scan: q, k, v must share a dtype and have adjacent columns")
    if z_bias is not None and z_bias.numel() != H * D:
        raise KernelError("gla_scan: z_bias must hold H * D entries")
    if any_multi and (carry is None or decay_prod is None or carry.numel() < n_chunks * H * D * Dv
                      or decay_prod.numel() < n_chunks * H * D):
        raise KernelError("gla_scan: scratch for segments of several chunks is missing or too small")
    if chunks.numel() < 4 * n_chunks or seg_chunks.numel() < 2 * n_segs:
        raise KernelError("gla_scan: chunk lists too short")
    launches = (1 if any_single else 0) + ((4 if a_head is None else 3) if any_multi else 0)
    _check(_lib().ftk_gla_scan(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), _code(q, "q"),
        _dev(z, "z", torch.float32), _dev(z_bias, "z_bias", torch.float32), float(tau), float(q_scale),
        _dev(state, "state", torch.float32), state.shape[0], _dev(state_slots, "state_slots", torch.int32),
        _dev(seg_info, "seg_info", torch.int32), n_segs, _dev(chunks, "chunks", torch.int32), n_chunks,
        _dev(seg_chunks, "seg_chunks", torch.int32), 1 if any_single else 0, 1 if any_multi else 0,
        _dev(carry, "carry", torch.float32), _dev(decay_prod, "decay_prod", torch.float32),
        _dev(out, "out", torch.float32), T, H, D, Dv, _dev(k_fac, "k_fac", torch.float32),
        _dev(a_head, "a_head", torch.float32), 1 if ones_col else 0, _dev(out_ones, "out_ones", torch.float32),
        qk_div, _stream()), "gla_scan", max(1, launches))


# --------------------------------------------------------------------------- short convolution, depth mix
def short_conv(x: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], state_slots: torch.Tensor,
               seg_info: torch.Tensor, n_segs: int, out: torch.Tensor) -> None:
    """``out[t] = x[t] + sum_j w[:, j] * in(t - taps + 1 + j)`` over each request's own inputs (a causal
    convolution over time on every channel, plus the input itself): ``x [T, C]`` float32 (the stream),
    ``w [C, taps]`` float32, ``out [T, C]`` of the engine's dtype.  The request's last ``taps - 1`` inputs live in
    ``state [slots, taps - 1, C]`` (float32, oldest first) at ``state_slots[segment]``: read for the step's first
    tokens (zeros for a request whose first tokens these are) and replaced by the step's last inputs."""
    T, C = x.shape
    taps = w.shape[1]
    if w.shape != (C, taps) or out.shape != (T, C) or x.dtype != torch.float32:
        raise KernelError("short_conv: x [T, C] float32, w [C, taps], out [T, C] expected")
    if taps > 1 and (state is None or state.shape[1:] != (taps - 1, C)):
        raise KernelError("short_conv: state must be [slots, taps - 1, C]")
    _check(_lib().ftk_short_conv(
        _dev(x, "x", torch.float32), _dev(w, "w", torch.float32), taps, _dev(state, "state", torch.float32),
        state.shape[0] if state is not None else 0, _dev(state_slots, "state_slots", torch.int32),
        _dev(seg_info, "seg_info", torch.int32), n_segs, _dev(out, "out"), _code(out, "out"), T, C, _stream()),
        "short_conv")


def depth_mix(hist: torch.Tensor, n_prev: int, mix: torch.Tensor, x: torch.Tensor) -> None:
    """``hist[n_prev] = x``, then ``x = sum_{j <= n_prev} mix[j] * hist[j]``: ``hist [layers, cap, C]`` float32 keeps
    every layer's output for the step's tokens (rows ``[:T]`` of each are used), ``x [T, C]`` float32."""
    T, C = x.shape
    if hist.dim() != 3 or hist.shape[2] != C or hist.shape[1] < T or hist.shape[0] <= n_prev or mix.numel() < n_prev + 1:
        raise KernelError("depth_mix: shapes do not agree")
    _check(_lib().ftk_depth_mix(_dev(hist, "hist", torch.float32), hist.stride(0), int(n_prev),
                                _dev(mix, "mix", torch.float32), _dev(x, "x", torch.float32), T * C, _stream()),
           "depth_mix")


def moe_gather_scaled(h: torch.Tensor, sorted_routes: torch.Tensor, weights: torch.Tensor, top_k: int,
                      out: torch.Tensor) -> None:
    """``out[r, :] = weights[sorted_routes[r]] * h[sorted_routes[r] // top_k, :]`` (32-bit product, rounded once):
    expert inputs in expert order, each scaled by its route's weight (``weights [T * top_k]`` float32)."""
    T, H = h.shape
    R = sorted_routes.numel()
    if out.shape != (R, H) or out.dtype != h.dtype or weights.numel() != R:
        raise KernelError("moe_gather_scaled: out must be [routes, hidden] of h's dtype, one weight per route")
    _check(_lib().ftk_moe_gather_scaled(_dev(h, "h"), _code(h, "h"), _dev(sorted_routes, "sorted_routes", torch.int32),
                                        _dev(weights, "weights", torch.float32), R, top_k, H, _dev(out, "out"),
                                        _stream()), "moe_gather_scaled")


def relu2_(x: torch.Tensor) -> None:
    """``x <- max(x, 0)^2`` in place."""
    _check(_lib().ftk_relu2(_dev(x, "x"), _code(x, "x"), x.numel(), _stream()), "relu2")


# --------------------------------------------------------------------------- latent attention
def latent_store(proj: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, n_rot: int, interleaved: bool,
                 wq: torch.Tensor, wkv: torch.Tensor, eps: float, positions: torch.Tensor,
                 rope_table: Optional[torch.Tensor], cq_out: torch.Tensor, slab: torch.Tensor,
                 slot_map: torch.Tensor) -> None:
    """From the rows ``proj [T, q_rank + kv_rank + rot_dim]`` of a latent-attention layer's input projection:
    ``cq_out [T, q_rank]`` gets the RMS-normed query latent (weight ``wq``); the token's cache row of
    ``slab [pages, 1, page_size, pad]`` at ``slot_map[t]`` gets ``[RMS-normed key/value latent (weight wkv) | the
    shared key part turned by the token's position | zeros]``.  The first ``n_rot`` dimensions of the part turn,
    in pairs ``(2i, 2i + 1)`` when ``interleaved`` and ``(i, i + n_rot / 2)`` otherwise, by the angles of
    ``rope_table [positions, n_rot]`` (``cos || sin``).  A token whose slot is negative stores nothing."""
    T = proj.shape[0]
    width = q_rank + kv_rank + rot_dim
    if proj.shape != (T, width) or proj.stride(1) != 1 or not proj.is_cuda or cq_out.shape != (T, q_rank) \
            or not cq_out.is_contiguous():
        raise KernelError("latent_store: proj [T, q_rank + kv_rank + rot_dim], cq_out [T, q_rank] expected")
    if slab.dim() != 4 or slab.shape[1] != 1 or slab.shape[3] < kv_rank + rot_dim or slab.dtype != proj.dtype \
            or cq_out.dtype != proj.dtype or not slab.is_contiguous():
        raise KernelError("latent_store: slab must be [pages, 1, page_size, >= kv_rank + rot_dim] of proj's dtype")
    if n_rot and (rope_table is None or rope_table.shape[1] != n_rot):
        raise KernelError("latent_store: the rotation table must be [positions, n_rot]")
    _check(_lib().ftk_latent_store(
        proj.data_ptr(), _code(proj, "proj"), proj.stride(0) if T > 1 else width, q_rank, kv_rank, rot_dim, n_rot,
        1 if interleaved else 0, _dev(wq, "wq", torch.float32), _dev(wkv, "wkv", torch.float32), float(eps),
        _dev(positions, "positions", torch.int32), _dev(rope_table, "rope_table", torch.float32),
        rope_table.shape[0] if rope_table is not None else 1, _dev(cq_out, "cq_out"), _dev(slab, "slab"),
        slab.shape[0] * slab.shape[2], _dev(slot_map, "slot_map", torch.int32), slab.shape[3], T, _stream()),
        "latent_store")


def latent_query_rotate(q: torch.Tensor, flat_dim: int, rot_dim: int, n_rot: int, interleaved: bool,
                        positions: torch.Tensor, rope_table: Optional[torch.Tensor], q_out: torch.Tensor,
                        kv_rank: int) -> None:
    """``q [T, H, flat_dim + rot_dim]``: every head's last ``rot_dim`` values, turned by the token's position (see
    :func:`latent_store`), go to ``q_out[t, h, kv_rank : kv_rank + rot_dim]``; the columns behind them are zeroed
    (``q_out [T, H, pad]``; its first ``kv_rank`` columns are left alone)."""
    T, H, qd = q.shape
    if qd != flat_dim + rot_dim or q_out.shape[:2] != (T, H) or q_out.shape[2] < kv_rank + rot_dim \
            or q_out.dtype != q.dtype or not q.is_contiguous() or not q_out.is_contiguous():
        raise KernelError("latent_query_rotate: shapes or dtypes do not agree")
    _check(_lib().ftk_latent_query_rotate(
        _dev(q, "q"), _code(q, "q"), H, flat_dim, rot_dim, n_rot, 1 if interleaved else 0,
        _dev(positions, "positions", torch.int32), _dev(rope_table, "rope_table", torch.float32),
        rope_table.shape[0] if rope_table is not None else 1, _dev(q_out, "q_out"), kv_rank, q_out.shape[2], T,
        _stream()), "latent_query_rotate")


def heads_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """A product per head: ``out[t, h, :] = x[t, h, :] @ w[h]`` with ``x [T, H, K]``, ``w [H, K, N]``, ``out [T, H, N]``.
    ``x`` and ``out`` may be views of the leading columns of wider heads (last stride 1): the library's batched
    product reads and writes them where they lie."""
    T, H, K = x.shape
    if w.shape[:2] != (H, K) or out.shape != (T, H, w.shape[2]) or x.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError("heads_linear: shapes do not agree")
    torch.bmm(x.transpose(0, 1), w, out=out.transpose(0, 1))


# --------------------------------------------------------------------------- matrix memory with exponential gates
def mlstm_gates(pre: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float, m_state: torch.Tensor,
                state_slots: torch.Tensor, seg_info: torch.Tensor, n_segs: int, key_fac: torch.Tensor,
                decay: torch.Tensor, m_out: torch.Tensor) -> None:
    """Gates of a matrix-memory layer for the step's tokens, per (request, head), all float32: with
    ``i = cap tanh((pre_i + b_i) / cap)`` and ``f = logsigmoid(cap tanh((pre_f + b_f) / cap))``, the running maximum
    ``m_t = max(f_t + m_(t-1), i_t)``, which starts from ``m_state[slot, head]`` (from 0 for a request's first tokens)
    and is left there, ``key_fac = e^(i_t - m_t)`` and ``decay = e^(f_t + m_(t-1) - m_t)``.  ``pre [T, 2 H]``."""
    T, H2 = pre.shape
    H = H2 // 2
    if key_fac.shape != (T, H) or decay.shape != (T, H) or m_out.shape != (T, H) or m_state.shape[1:] != (H,):
        raise KernelError("mlstm_gates: shapes do not agree")
    _check(_lib().ftk_mlstm_gates(
        _dev(pre, "pre", torch.float32), _dev(bias_i, "bias_i", torch.float32), _dev(bias_f, "bias_f", torch.float32),
        float(cap), _dev(m_state, "m_state", torch.float32), m_state.shape[0],
        _dev(state_slots, "state_slots", torch.int32), _dev(seg_info, "seg_info", torch.int32), n_segs, H, T,
        _dev(key_fac, "key_fac", torch.float32), _dev(decay, "decay", torch.float32),
        _dev(m_out, "m_out", torch.float32), _stream()), "mlstm_gates")


def mlstm_output(o32: torch.Tensor, nq: torch.Tensor, m: torch.Tensor, gates: torch.Tensor, norm_weight: torch.Tensor,
                 eps: float, out: torch.Tensor) -> None:
    """``o32 [T, H, vdim]`` (numerators), ``nq [T, H]`` (``n . q``), ``m [T, H]``: ``o = num / (max(|n . q|, e^-m) +
    1e-6)``, divided by its root mean square over the head, times ``norm_weight [H * vdim]``, times
    ``sigmoid(gates)`` (``gates [T, H * vdim]``, a view of adjacent columns is fine) into ``out [T, H * vdim]``."""
    T, H, Dv = o32.shape
    if out.shape != (T, H * Dv) or gates.shape != (T, H * Dv) or gates.stride(1) != 1 or gates.dtype != out.dtype \
            or norm_weight.numel() != H * Dv or m.shape != (T, H) or nq.shape != (T, H) or not out.is_contiguous():
        raise KernelError("mlstm_output: shapes or dtypes do not agree")
    _check(_lib().ftk_mlstm_output(
        _dev(o32, "o32", torch.float32), _dev(nq, "nq", torch.float32), _dev(m, "m", torch.float32), gates.data_ptr(),
        gates.stride(0) if T > 1 else H * Dv, _dev(norm_weight, "norm_weight", torch.float32), float(eps),
        _dev(out, "out"), _code(out, "out"), T, H, Dv, _stream()), "mlstm_output")


# --------------------------------------------------------------------------- several residual streams
def hyper_step(streams: torch.Tensor, init_from: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
               mix: Optional[torch.Tensor] = None, out_w: Optional[torch.Tensor] = None,
               in_w: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
               h_out: Optional[torch.Tensor] = None, sum_out: Optional[torch.Tensor] = None) -> None:
    """One pass over the ``S`` residual streams ``streams [S, T, C]`` (float32; a view whose streams lie
    ``streams.stride(0)`` apart), every step optional, in this order:

    * ``init_from [T, C]`` (float32): every stream becomes a copy of it;
    * ``y [T, C]`` (a sub-layer's result), ``mix [S, S]`` indexed ``[from, to]``, ``out_w [S]``: all streams at once from
      the old ones, ``x_t <- sum_s mix[s, t] x_s + out_w[t] y``;
    * ``in_w [S]``, ``norm_w [C]``: ``h_out = unit(sum_s in_w[s] x_s) * norm_w`` with ``unit`` the division by the root
      mean square (``eps`` inside the root); ``h_out [T, C]`` is float32 or of the engine's dtype;
    * ``sum_out [T, C]`` (float32) ``= sum_s x_s``.

    All sums are 32-bit; the streams are stored back when the first or second step changed them."""
    S, T, C = streams.shape
    if streams.dtype != torch.float32 or streams.stride(2) != 1 or streams.stride(1) != C or S > 8:
        raise KernelError("hyper_step: streams must be float32 [S <= 8, T, C] with dense rows")
    if (y is None) != (mix is None) or (y is None) != (out_w is None) or (in_w is None) != (norm_w is None) \
            or (in_w is None) != (h_out is None):
        raise KernelError("hyper_step: y goes with mix and out_w; in_w goes with norm_w and h_out")
    for name, t, shape in (("init_from", init_from, (T, C)), ("y", y, (T, C)), ("mix", mix, (S, S)), ("out_w", out_w, (S,)),
                           ("in_w", in_w, (S,)), ("norm_w", norm_w, (C,)), ("h_out", h_out, (T, C)),
                           ("sum_out", sum_out, (T, C))):
        if t is not None and tuple(t.shape) != shape:
            raise KernelError(f"hyper_step: {name} must be {shape}, got {tuple(t.shape)}")
    _check(_lib().ftk_hyper_step(
        streams.data_ptr(), streams.stride(0), S, T, C, _dev(init_from, "init_from", torch.float32), _dev(y, "y"),
        _code(y, "y") if y is not None else F32, _dev(mix, "mix", torch.float32), _dev(out_w, "out_w", torch.float32),
        _dev(in_w, "in_w", torch.float32), _dev(norm_w, "norm_w", torch.float32), float(eps), _dev(h_out, "h_out"),
        _code(h_out, "h_out") if h_out is not None else F32, _dev(sum_out, "sum_out", torch.float32), _stream()),
        "hyper_step")


def norm_mean(xs: Sequence[torch.Tensor], ws: Sequence[torch.Tensor], eps: float, out: torch.Tensor) -> None:
    """``out = (1 / n) sum_i unit(xs[i]) * ws[i]``: up to four ``[T, C]`` tensors of ``out``'s dtype, each divided by
    its rows' root mean square (``eps`` inside the root) and multiplied by a float32 weight ``[C]``; 32-bit sums."""
    n = len(xs)
    T, C = out.shape
    if not 1 <= n <= 4 or len(ws) != n:
        raise KernelError("norm_mean: one to four inputs, a weight each")
    for x, w in zip(xs, ws):
        if x.shape != (T, C) or x.dtype != out.dtype or w.shape != (C,):
            raise KernelError("norm_mean: inputs [T, C] of out's dtype, weights [C]")
    xp = (_vp * 4)(*[_dev(x, "x") for x in xs])
    wp = (_vp * 4)(*[_dev(w, "w", torch.float32) for w in ws])
    _check(_lib().ftk_norm_mean(xp, wp, n, _code(out, "out"), float(eps), _dev(out, "out"), T, C, _stream()), "norm_mean")


CONV_ACT_CODES = {None: 0, "silu": 1}


def conv_act(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act: Optional[str],
             state: Optional[torch.Tensor], state_slots: torch.Tensor, seg_info: torch.Tensor, n_segs: int,
             out: torch.Tensor) -> None:
    """``out[t] = act(bias + sum_j w[:, j] * in(t - taps + 1 + j))`` over each request's own inputs: a causal
    convolution over time on every channel of a projection's rows.  ``x [T, C]`` of the engine's dtype (a view of
    adjacent columns of a wider tensor is fine), ``w [C, taps]`` and ``bias [C]`` float32 (the last tap is the current
    token's), ``act`` None or ``"silu"``, ``out [T, C]`` of ``x``'s dtype.  The request's last ``taps - 1`` inputs live
    in ``state [slots, taps - 1, C]`` (float32, oldest first) at ``state_slots[segment]``: read for the step's first
    tokens (zeros for a request whose first tokens these are) and replaced by the step's last inputs."""
    T, C = x.shape
    taps = w.shape[1]
    if w.shape != (C, taps) or out.shape != (T, C) or out.dtype != x.dtype or x.stride(1) != 1 or not 1 <= taps <= 16:
        raise KernelError("conv_act: x [T, C] with adjacent columns, w [C, taps <= 16], out [T, C] of x's dtype expected")
    if taps > 1 and (state is None or state.shape[1:] != (taps - 1, C)):
        raise KernelError("conv_act: state must be [slots, taps - 1, C]")
    if bias is not None and bias.shape != (C,):
        raise KernelError("conv_act: bias must be [C]")
    if act not in CONV_ACT_CODES:
        raise KernelError(f"conv_act: unknown activation '{act}'")
    _check(_lib().ftk_conv_act(
        x.data_ptr(), x.stride(0) if T > 1 else C, _code(x, "x"), _dev(w, "w", torch.float32),
        _dev(bias, "bias", torch.float32), taps, CONV_ACT_CODES[act], _dev(state, "state", torch.float32),
        state.shape[0] if state is not None else 0, _dev(state_slots, "state_slots", torch.int32),
        _dev(seg_info, "seg_info", torch.int32), n_segs, _dev(out, "out"), T, C, _stream()), "conv_act")


# --------------------------------------------------------------------------- state space, delta rule
def _cols(t: torch.Tensor, what: str, shape, dtype: Optional[torch.dtype] = None) -> int:
    """Row stride of a view of adjacent columns of a row-major tensor."""
    if tuple(t.shape) != tuple(shape) or t.stride(1) != 1 or not t.is_cuda or (dtype is not None and t.dtype != dtype):
        raise KernelError(f"{what} must be {tuple(shape)} with adjacent columns")
    return t.stride(0) if t.shape[0] > 1 else t.shape[1]


def ssm_gates(dt_raw: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, dt_out: torch.Tensor,
              decay_out: torch.Tensor) -> None:
    """Step sizes and decays of a state-space layer, 32-bit: ``dt_out = softplus(dt_raw + dt_bias)`` (no clamp),
    ``decay_out = exp(-exp(a_log) * dt_out)``; ``dt_raw [T, H]`` of the engine's dtype (a view of adjacent columns is
    fine), ``dt_bias, a_log [H]`` and both outputs ``[T, H]`` float32."""
    T, H = dt_out.shape
    stride = _cols(dt_raw, "ssm_gates: dt_raw", (T, H))
    if decay_out.shape != (T, H) or dt_bias.shape != (H,) or a_log.shape != (H,):
        raise KernelError("ssm_gates: shapes do not agree")
    _check(_lib().ftk_ssm_gates(dt_raw.data_ptr(), stride, _code(dt_raw, "dt_raw"), _dev(dt_bias, "dt_bias", torch.float32),
                                _dev(a_log, "a_log", torch.float32), _dev(dt_out, "dt_out", torch.float32),
                                _dev(decay_out, "decay_out", torch.float32), T, H, _stream()), "ssm_gates")


def ssm_output(o32: torch.Tensor, x: torch.Tensor, d_skip: torch.Tensor, z: torch.Tensor, norm_weight: torch.Tensor,
               norm_groups: int, eps: float, out: torch.Tensor) -> None:
    """``y = (o32 + d_skip[head] * x) * silu(z)``, RMS-normed in ``norm_groups`` equal parts of a row (each by its own
    root mean square, ``eps`` inside the root), times ``norm_weight [H * P]``, into ``out [T, H * P]``.  ``o32 [T, H, P]``
    float32; ``x`` and ``z`` ``[T, H * P]`` of ``out``'s dtype (views of adjacent columns are fine); 32-bit arithmetic."""
    T, H, P = o32.shape
    xs = _cols(x, "ssm_output: x", (T, H * P), out.dtype)
    zs = _cols(z, "ssm_output: z", (T, H * P), out.dtype)
    if out.shape != (T, H * P) or d_skip.shape != (H,) or norm_weight.shape != (H * P,) or norm_groups < 1 \
            or (H * P) % norm_groups:
        raise KernelError("ssm_output: shapes do not agree")
    _check(_lib().ftk_ssm_output(_dev(o32, "o32", torch.float32), x.data_ptr(), xs, _dev(d_skip, "d_skip", torch.float32),
                                 z.data_ptr(), zs, _code(out, "out"), _dev(norm_weight, "norm_weight", torch.float32),
                                 int(norm_groups), float(eps), _dev(out, "out"), T, H, P, _stream()), "ssm_output")


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, b_raw: torch.Tensor, a_raw: torch.Tensor,
               a_log: torch.Tensor, dt_bias: torch.Tensor, q_scale: float, unit_eps: float, state: torch.Tensor,
               state_slots: torch.Tensor, seg_info: torch.Tensor, n_segs: int, out: torch.Tensor) -> None:
    """The gated delta rule over the step's tokens, per (request, head), a request's tokens in order:
    ``S <- g S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``, ``o = S^T q``, with ``beta = sigmoid(b_raw)``,
    ``g = exp(-exp(a_log) softplus(a_raw + dt_bias))``, and ``q``, ``k`` first made unit vectors per head
    (``x / sqrt(sum(x^2) + unit_eps)``; ``q`` then times ``q_scale``).

    ``q, k [T, G * D]``, ``v [T, H * Dv]``, ``b_raw, a_raw [T, H]`` of the engine's dtype (views of adjacent columns
    are fine; head ``h`` reads q/k head ``h // (H / G)``); ``a_log, dt_bias [H]`` float32; ``state [slots, H, Dv, D]``
    float32 (``S`` column by column: a value column's key channels are neighbours), read from and left in the slot ``state_slots[segment]`` (a segment with ``kv_len == q_len`` starts from
    zero); ``out [T, H, Dv]`` float32.  Everything but the reading of the rows is 32-bit."""
    T, H, Dv = out.shape
    D = state.shape[3]
    if state.shape[1] != H or state.shape[2] != Dv or q.shape[1] % D or H % (q.shape[1] // D) or D > 256:
        raise KernelError("delta_scan: shapes do not agree (keys of at most 256 channels)")
    G = q.shape[1] // D
    qs, ks = _cols(q, "delta_scan: q", (T, G * D)), _cols(k, "delta_scan: k", (T, G * D), q.dtype)
    vs = _cols(v, "delta_scan: v", (T, H * Dv), q.dtype)
    bs, as_ = _cols(b_raw, "delta_scan: b_raw", (T, H), q.dtype), _cols(a_raw, "delta_scan: a_raw", (T, H), q.dtype)
    if a_log.shape != (H,) or dt_bias.shape != (H,):
        raise KernelError("delta_scan: a_log and dt_bias must be [H]")
    _check(_lib().ftk_delta_scan(
        q.data_ptr(), qs, k.data_ptr(), ks, v.data_ptr(), vs, b_raw.data_ptr(), bs, a_raw.data_ptr(), as_, _code(q, "q"),
        _dev(a_log, "a_log", torch.float32), _dev(dt_bias, "dt_bias", torch.float32), float(q_scale), float(unit_eps),
        _dev(state, "state", torch.float32), state.shape[0], _dev(state_slots, "state_slots", torch.int32),
        _dev(seg_info, "seg_info", torch.int32), n_segs, _dev(out, "out", torch.float32), T, H, G, D, Dv, _stream()),
        "delta_scan")
