"""Python faces of the CUDA kernels.

Each function checks its tensors (device, dtype, layout), passes raw pointers and the
current CUDA stream to an ``extern "C"`` entry point, and raises ``KernelError`` with the
library's message if the arguments were refused or the launch failed.  There is no CPU
path: a tensor that is not on a CUDA device is an error.

``launch_count`` counts the kernels launched through this module (the bench reports it).
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p

import torch

from . import build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

launch_count = 0


class KernelError(RuntimeError):
    pass


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only (got a tensor on %s)" % t.device)


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported dtype {dtype}; kernels take float32 or bfloat16") from None


def _finish(lib: ctypes.CDLL, rc: int, what: str) -> None:
    global launch_count
    if rc != 0:
        msg = lib.mi_error_message().decode("utf-8", "replace")
        raise KernelError(f"{what}: {msg or ('status %d' % rc)}")
    launch_count += 1


class KernelWaitError(KernelError):
    """A kernel gave up one of its bounded waits: what it wrote since is not to be trusted."""


_configured: set[str] = set()

# Libraries whose kernels have bounded waits.  Their give-ups are reported into one int32 word
# per device (``status_word``), which the engine copies to the host with every step's result;
# on their own the libraries would each keep a word that only a synchronising call can read.
_WAITING_LIBRARIES = ("attention_mma", "attention_tc", "gemm_tma")
_status_words: dict[int, torch.Tensor] = {}
_status_shared: set[tuple[str, int]] = set()


def _lib(name: str) -> ctypes.CDLL:
    lib = build.library(name)
    if name not in _configured:
        _SIGNATURES[name](lib)
        _configured.add(name)
    return lib


def _device_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word (on ``device``) that the kernels with bounded waits set to 1 when a wait
    gave up.  Zero means every such kernel launched through this module has waited out its
    copies; the engine reads it with each step's tokens."""
    idx = _device_index(device)
    word = _status_words.get(idx)
    if word is None:
        word = _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return word


def _waiting_lib(name: str, device: torch.device) -> ctypes.CDLL:
    """``_lib`` for a library with bounded waits: the first use on a device points the
    library's give-up reports at that device's shared status word."""
    lib = _lib(name)
    idx = _device_index(device)
    if (name, idx) not in _status_shared:
        with torch.cuda.device(idx):
            rc = lib.mi_set_status_word(_ptr(status_word(device)))
        if rc != 0:
            raise KernelError(f"{name}: cannot share the status word: {lib.mi_error_message().decode()}")
        _status_shared.add((name, idx))
    return lib


def recover_from_wait_failure(device: torch.device) -> None:
    """After a give-up: clear the status word and the arrival counters that the interrupted
    kernels may have left non-zero (they are zero between calls otherwise).  Synchronises."""
    torch.cuda.synchronize(device)
    with torch.inference_mode():      # the buffers were made inside a step, which runs in inference mode
        status_word(device).zero_()
        idx = _device_index(device)
        for buf in _decode_counter_bufs.get(idx, []):
            buf.zero_()
        for _partials, counters in _tma_ws.get(idx, []):
            counters.zero_()
    torch.cuda.synchronize(device)


def _sig_elementwise(lib: ctypes.CDLL) -> None:
    lib.mi_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_add_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_int, c_int, c_float, c_int, c_int, c_void_p]
    lib.mi_rope_write.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_silu_mul.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_silu_mul_pairs.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_table_update.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
    lib.mi_rope_table.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p]


def _sig_gemm_f32(lib: ctypes.CDLL) -> None:
    lib.mi_gemm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_int, c_void_p]


def _sig_attention_generic(lib: ctypes.CDLL) -> None:
    lib.mi_attention_generic.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
        c_float, c_int, c_int, c_void_p]
    lib.mi_attention_generic_tile_tokens.restype = c_int
    lib.mi_attention_generic_kv.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_float, c_int, c_int, c_void_p]
    lib.mi_attention_generic_ext.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.mi_attention_generic_masked.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]


def _sig_sampling(lib: ctypes.CDLL) -> None:
    lib.mi_sample.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]


def _sig_attention_mma(lib: ctypes.CDLL) -> None:
    lib.mi_attention_decode.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p,
        c_void_p, c_void_p]
    lib.mi_attention_decode_sliced.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p,
        c_void_p, c_void_p]
    lib.mi_attention_decode_counters.argtypes = [c_int, c_int, c_int]
    lib.mi_attention_decode_balanced_scratch.argtypes = [c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int),
                                                         ctypes.POINTER(ctypes.c_longlong),
                                                         ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(c_int)]
    lib.mi_attention_decode_balanced.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
        c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
        c_void_p]
    lib.mi_attention_decode_balanced_unit_cost.argtypes = [c_int]
    lib.mi_attention_wait_status.argtypes = [c_int]
    lib.mi_set_status_word.argtypes = [c_void_p]
    lib.mi_attention_prefill.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
        c_float, c_int, c_void_p]
    lib.mi_attention_prefill_tile_tokens.argtypes = [c_int]
    lib.mi_attention_prefill_tile_tokens.restype = c_int


def _sig_gemm_tma(lib: ctypes.CDLL) -> None:
    lib.mi_gemm_tma.argtypes = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
    lib.mi_gemm_tma_fused.argtypes = [c_void_p, ctypes.c_longlong, c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                      c_void_p, c_void_p, c_void_p, c_void_p]
    lib.mi_gemm_tma_workspace.argtypes = [c_int, c_int, c_int, ctypes.POINTER(ctypes.c_longlong),
                                          ctypes.POINTER(c_int)]
    lib.mi_gemm_tma_status.argtypes = [c_int]
    lib.mi_set_status_word.argtypes = [c_void_p]


def _sig_attention_tc(lib: ctypes.CDLL) -> None:
    lib.mi_attention_prefill_tc.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
        c_void_p]
    lib.mi_attention_prefill_tc_ext.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
        c_void_p, c_void_p, c_void_p]
    lib.mi_attention_prefill_tc_masked.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, ctypes.c_longlong, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
        c_void_p, c_void_p, c_void_p]
    lib.mi_attention_prefill_tc_supported.argtypes = [c_int, c_int, c_int, c_int]
    lib.mi_attention_tc_status.argtypes = [c_int]
    lib.mi_set_status_word.argtypes = [c_void_p]


def _sig_layernorm(lib: ctypes.CDLL) -> None:
    lib.mi_embedding_scaled.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p]
    lib.mi_add_layernorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]


def _sig_rope_norm(lib: ctypes.CDLL) -> None:
    lib.mi_rope_norm_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                       c_int, c_int, c_void_p]
    lib.mi_gate_mul.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                c_int, c_int, c_void_p]


def _sig_recurrent(lib: ctypes.CDLL) -> None:
    ll = ctypes.c_longlong
    lib.mi_causal_conv.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, ll, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_rglru_scan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                  c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, ll, c_int,
                                  c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_rglru_scan_chunked.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int,
                                          c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, ll, c_int,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int,
                                          c_int, c_int, c_void_p]
    lib.mi_rglru_chunked_scratch.argtypes = [c_int, c_int, c_int]
    lib.mi_rglru_chunked_scratch.restype = ll
    lib.mi_gla_scan.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_float, c_float,
                                c_void_p, ll, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p]
    lib.mi_mlstm_gates.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, ll, ll, c_void_p,
                                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_delta_scan.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_int, c_float, c_float, c_void_p, ll, ll, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                                  c_void_p]
    lib.mi_gla_chunked_scratch.argtypes = [c_int, c_int, c_int, c_int, c_int]
    lib.mi_gla_chunked_scratch.restype = ll
    lib.mi_headnorm_gate.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                     c_int, c_float, c_int, c_float, c_int, c_void_p, c_float, c_int, c_void_p]


def _sig_moe(lib: ctypes.CDLL) -> None:
    ll = ctypes.c_longlong
    lib.mi_moe_select.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_float, c_void_p, c_int, c_void_p]
    lib.mi_moe_plan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    lib.mi_moe_tile_rows.argtypes = [c_int]
    lib.mi_moe_tile_rows.restype = c_int
    lib.mi_moe_gate_up.argtypes = [c_void_p, c_int, c_void_p, c_void_p, ll, c_void_p, c_int, c_void_p, c_int,
                                   c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_int, c_int, c_void_p]
    lib.mi_moe_down.argtypes = [c_void_p, c_void_p, ll, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                c_void_p]
    lib.mi_moe_combine.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
                                   c_void_p, c_int, c_int, c_void_p]
    lib.mi_moe_gather.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_clamped_glu.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p]


def _sig_stream(lib: ctypes.CDLL) -> None:
    ll = ctypes.c_longlong
    lib.mi_embedding_pair_hash.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, ll, ll, c_int,
                                           c_void_p]
    lib.mi_add_rmsnorm_multi.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p]
    lib.mi_glu_mul_pairs.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    lib.mi_embedding_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int,
                                         c_void_p]
    lib.mi_scaled_norm_add.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_float, c_float, c_void_p, c_int, c_int,
                                       c_int, c_void_p]
    lib.mi_token_gate.argtypes = [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                                  c_int, c_int, c_void_p]
    lib.mi_scale_f32.argtypes = [c_void_p, ll, c_float, c_void_p]


def _sig_qk_prepare(lib: ctypes.CDLL) -> None:
    lib.mi_qk_bias_norm_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p,
                                          c_void_p, c_int, c_int, c_int, c_void_p]
    lib.mi_latent_prepare.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_void_p]


    lib.mi_qk_norm_rope_store.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_float, c_float,
                                          c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_void_p, c_int, c_void_p, c_int, c_void_p]


def _sig_attention_rows(lib: ctypes.CDLL) -> None:
    lib.mi_attention_rows.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
        c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
    lib.mi_attention_rows_tile_tokens.argtypes = [c_int, c_int]
    lib.mi_attention_rows_supported.argtypes = [c_int, c_int, c_int, c_int, c_int]


_SIGNATURES = {
    "attention_rows": _sig_attention_rows,
    "stream": _sig_stream,
    "qk_prepare": _sig_qk_prepare,
    "layernorm": _sig_layernorm,
    "rope_norm": _sig_rope_norm,
    "recurrent": _sig_recurrent,
    "moe": _sig_moe,
    "attention_tc": _sig_attention_tc,
    "gemm_tma": _sig_gemm_tma,
    "attention_mma": _sig_attention_mma,
    "elementwise": _sig_elementwise,
    "gemm_f32": _sig_gemm_f32,
    "attention_generic": _sig_attention_generic,
    "sampling": _sig_sampling,
}


def register_signatures(name: str, fn) -> None:
    _SIGNATURES[name] = fn


# ---------------------------------------------------------------------------------------


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]``; ``ids`` int32 ``[M]``, ``table`` ``[V, H]``."""
    _cuda(table, ids, out)
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("embedding: ids must be a contiguous int32 vector")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embedding: table must be a contiguous [V, H] matrix")
    V, H = table.shape
    M = ids.shape[0]
    if out is None:
        out = torch.empty((M, H), dtype=table.dtype, device=table.device)
    elif out.shape != (M, H) or out.dtype != table.dtype or not out.is_contiguous():
        raise KernelError("embedding: bad output tensor")
    lib = _lib("elementwise")
    rc = lib.mi_embedding(_ptr(table), _ptr(ids), _ptr(out), M, H, V, _code(table.dtype), _stream())
    _finish(lib, rc, "embedding")
    return out


def add_rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float,
    *,
    residual_in: torch.Tensor | None = None,
    residual_out: torch.Tensor | None = None,
    rows: torch.Tensor | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """RMS norm of ``x (+ residual_in)`` with fp32 statistics.

    ``r = float(x[src]) + residual_in[src]`` (``src = rows[i]`` if ``rows`` is given, else
    ``i``); ``residual_out[i] = r`` if given (fp32; may alias ``residual_in`` when no
    ``rows``); returns ``weight * r * rsqrt(mean(r*r) + eps)`` in ``x``'s dtype.
    """
    _cuda(x, weight, residual_in, residual_out, rows, out)
    if x.dim() != 2 or not x.is_contiguous():
        raise KernelError("rmsnorm: x must be a contiguous [M, H] matrix")
    H = x.shape[1]
    M = x.shape[0] if rows is None else rows.shape[0]
    if weight.shape != (H,) or not weight.is_contiguous():
        raise KernelError(f"rmsnorm: weight must have shape ({H},)")
    for name, r in (("residual_in", residual_in), ("residual_out", residual_out)):
        if r is not None and (r.dtype != torch.float32 or r.dim() != 2 or r.shape[1] != H
                              or not r.is_contiguous()):
            raise KernelError(f"rmsnorm: {name} must be a contiguous fp32 [*, {H}] matrix")
    if residual_in is not None and residual_in.shape[0] != x.shape[0]:
        raise KernelError("rmsnorm: residual_in must have x's rows")
    if residual_out is not None and residual_out.shape[0] != M:
        raise KernelError("rmsnorm: residual_out must have one row per output row")
    if rows is not None and (rows.dtype != torch.int32 or rows.dim() != 1 or not rows.is_contiguous()):
        raise KernelError("rmsnorm: rows must be a contiguous int32 vector")
    if out is None:
        out = torch.empty((M, H), dtype=x.dtype, device=x.device)
    elif out.shape != (M, H) or out.dtype != x.dtype or not out.is_contiguous():
        raise KernelError("rmsnorm: bad output tensor")
    lib = _lib("elementwise")
    rc = lib.mi_add_rmsnorm(_ptr(x), _ptr(residual_in), _ptr(residual_out), _ptr(weight), _ptr(out),
                            _ptr(rows), M, H, float(eps), _code(x.dtype), _code(weight.dtype), _stream())
    _finish(lib, rc, "rmsnorm")
    return out


def rope_write(
    qkv: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
    *,
    positions: torch.Tensor | None = None,
    inv_freq: torch.Tensor | None = None,
    rotary_dim: int = 0,
    slots: torch.Tensor | None = None,
    kcache: torch.Tensor | None = None,
    vcache: torch.Tensor | None = None,
) -> None:
    """Rotate q and k inside ``qkv [M, (nq + 2 nkv) * d]`` (half layout, fp32 angles) and
    store k and v at ``slots`` (page * page_size + offset) of ``kcache`` / ``vcache``
    ``[pages, nkv, page_size, d]``."""
    _cuda(qkv, positions, inv_freq, slots, kcache, vcache)
    M = qkv.shape[0]
    if qkv.dim() != 2 or qkv.shape[1] != (nq + 2 * nkv) * head_dim or not qkv.is_contiguous():
        raise KernelError("rope: qkv must be contiguous [M, (nq + 2 nkv) * d]")
    if rotary_dim:
        if positions is None or positions.dtype != torch.int32 or positions.shape != (M,):
            raise KernelError("rope: positions must be int32 [M]")
        if inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.shape != (rotary_dim // 2,):
            raise KernelError("rope: inv_freq must be fp32 [rotary_dim / 2]")
    if kcache is not None:
        if slots is None or slots.dtype != torch.int32 or slots.shape != (M,):
            raise KernelError("rope: slots must be int32 [M]")
        for c in (kcache, vcache):
            if (c is None or c.dtype != qkv.dtype or c.dim() != 4 or c.shape[1] != nkv or c.shape[3] != head_dim
                    or not c.is_contiguous()):
                raise KernelError("rope: caches must be contiguous [pages, nkv, page_size, d] in qkv's dtype")
    page_size = int(kcache.shape[2]) if kcache is not None else 0
    lib = _lib("elementwise")
    rc = lib.mi_rope_write(_ptr(qkv), _ptr(positions), _ptr(inv_freq), _ptr(slots), _ptr(kcache),
                           _ptr(vcache), M, nq, nkv, head_dim, rotary_dim, page_size, _code(qkv.dtype),
                           _stream())
    _finish(lib, rc, "rope")


def table_update(table: torch.Tensor, updates: torch.Tensor, count: torch.Tensor, capacity: int) -> None:
    """Scatter new page ids into a block table: ``table[slot, index] = page`` for the first
    ``count[0]`` (at most ``capacity``) triples ``(slot, index, page)`` of ``updates``; all int32
    on the device.  ``count`` is read when the kernel runs, so a captured step can replay it."""
    _cuda(table, updates, count)
    if table.dtype != torch.int32 or table.dim() != 2 or not table.is_contiguous():
        raise KernelError("table_update: the table must be a contiguous int32 matrix")
    if updates.dtype != torch.int32 or updates.numel() < 3 * capacity or count.dtype != torch.int32 or count.numel() < 1:
        raise KernelError("table_update: updates must hold 3 * capacity int32 values and count one")
    lib = _lib("elementwise")
    rc = lib.mi_table_update(_ptr(table), table.shape[1], table.shape[0], _ptr(updates), _ptr(count),
                             int(capacity), _stream())
    _finish(lib, rc, "table_update")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None, pairs: bool = False) -> torch.Tensor:
    """``silu(gate) * up`` with fp32 arithmetic, for ``gate_up [M, 2 I]`` laid out as halves
    (``gate = gate_up[:, :I]``, ``up = gate_up[:, I:]``) or, with ``pairs``, interleaved
    (``gate = gate_up[:, 0::2]``, ``up = gate_up[:, 1::2]``)."""
    _cuda(gate_up, out)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("silu_mul: input must be contiguous [M, 2 I]")
    M, I2 = gate_up.shape
    I = I2 // 2
    if out is None:
        out = torch.empty((M, I), dtype=gate_up.dtype, device=gate_up.device)
    elif out.shape != (M, I) or out.dtype != gate_up.dtype or not out.is_contiguous():
        raise KernelError("silu_mul: bad output tensor")
    lib = _lib("elementwise")
    fn = lib.mi_silu_mul_pairs if pairs else lib.mi_silu_mul
    rc = fn(_ptr(gate_up), _ptr(out), M, I, _code(gate_up.dtype), _stream())
    _finish(lib, rc, "silu_mul")
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a [M, K] @ w [N, K]^T`` in true fp32 (CUDA cores, fixed summation order)."""
    _cuda(a, w, out)
    if a.dtype != torch.float32 or w.dtype != torch.float32:
        raise KernelError("gemm_f32: operands must be float32")
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1]:
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T do not match")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_f32: operands must be K-contiguous")
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    elif out.shape != (M, N) or out.dtype != torch.float32 or out.stride(1) != 1:
        raise KernelError("gemm_f32: bad output tensor")
    lib = _lib("gemm_f32")
    rc = lib.mi_gemm_f32(_ptr(a), _ptr(w), _ptr(out), M, N, K, a.stride(0) if M > 1 else K,
                         w.stride(0) if N > 1 else K, out.stride(0) if M > 1 else N, _stream())
    _finish(lib, rc, "gemm_f32")
    return out


def cache_swizzle_mask(head_dim: int, dtype: torch.dtype) -> int:
    """The chunk permutation mask of cache rows (``mi_swizzle_mask`` in common.cuh)."""
    row_bytes = head_dim * torch.empty((), dtype=dtype).element_size()
    n = row_bytes // 16
    if row_bytes % 16 or n < 2 or n & (n - 1):      # a row that is no whole number of chunks is stored as it is
        return 0
    return min(n, 8) - 1


def _chunk_permutation(page_size: int, head_dim: int, dtype: torch.dtype) -> torch.Tensor:
    """``perm[t, k]``: where element ``k`` of the row at in-page offset ``t`` is stored."""
    epc = 16 // torch.empty((), dtype=dtype).element_size()
    mask = cache_swizzle_mask(head_dim, dtype)
    t = torch.arange(page_size).view(-1, 1)
    k = torch.arange(head_dim).view(1, -1)
    return ((k // epc) ^ (t & mask)) * epc + k % epc


def pack_cache_pages(by_slot: torch.Tensor, page_size: int) -> torch.Tensor:
    """``[pages * page_size, kv_heads, d]`` (one row per slot) -> the cache layout
    ``[pages, kv_heads, page_size, d]`` with each row's 16-byte chunks permuted by its in-page
    offset.  For tests and tools; the engine writes the cache with the rope/store kernel."""
    n, nkv, d = by_slot.shape
    pages = by_slot.view(n // page_size, page_size, nkv, d).permute(0, 2, 1, 3).contiguous()
    perm = _chunk_permutation(page_size, d, by_slot.dtype).to(by_slot.device)
    out = torch.empty_like(pages)
    out.scatter_(3, perm.view(1, 1, page_size, d).expand_as(pages), pages)
    return out


def unpack_cache_pages(pages: torch.Tensor) -> torch.Tensor:
    """The inverse of ``pack_cache_pages``: ``[pages * page_size, kv_heads, d]`` by slot."""
    n_pages, nkv, page_size, d = pages.shape
    perm = _chunk_permutation(page_size, d, pages.dtype).to(pages.device)
    plain = torch.gather(pages, 3, perm.view(1, 1, page_size, d).expand_as(pages))
    return plain.permute(0, 2, 1, 3).reshape(n_pages * page_size, nkv, d)


# Query tokens per tile of the CUDA-core attention kernel (BQ in attention_generic.cu).
ATTENTION_TILE_TOKENS = 16


def prefill_tile_tokens(group: int) -> int:
    """Tokens per tile of the tensor-core prefill kernel for ``group`` query heads per
    key/value head: 128 rows of (token, head in group) per block (attention_mma.cu)."""
    return 128 // min(group, 128)


PREFILL_TC_TILES = 1      # 128-row tiles per block of the tcgen05 prefill kernel (NTILE in attention_tc.cu)


def prefill_tc_tile_tokens(group: int) -> int:
    """Tokens per block of the tcgen05 prefill kernel: tiles of 128 rows of (token, head in
    group) (attention_tc.cu)."""
    return 128 * PREFILL_TC_TILES // min(group, 128)


def attention_tile_sizes(group: int) -> frozenset[int]:
    """The query tile sizes a step must plan for an attention mixer with this group size."""
    return frozenset({ATTENTION_TILE_TOKENS, prefill_tile_tokens(group), prefill_tc_tile_tokens(group)})


_sm_count: dict[int, int] = {}


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def sm_count(device: torch.device) -> int:
    return _sms(device)


def decode_splits(n_requests: int, nq: int, nkv: int, max_kv_len: int, window: int, device) -> int:
    """For the sliced decode kernel (``attention_decode``), which the engine itself no longer
    uses: how many slices of the keys each (request, key/value head) is cut into: enough blocks
    for about two per SM, but at least four 64-key chunks per slice (a slice costs a fixed
    prologue and a merge, measured at roughly ten chunks' worth of time)."""
    blocks = n_requests * nkv * ((nq // nkv + 7) // 8)
    span = min(max_kv_len, window + 63) if window else max_kv_len
    chunks = max(1, -(-span // 64))
    return max(1, min(2 * _sms(device) // blocks, chunks // 4, 64))


FUSE_DECODE_ROPE = os.environ.get("MINI_INFER_FUSE_ROPE", "1") != "0"
SPLIT_MIXED_STEPS = os.environ.get("MINI_INFER_SPLIT_MIXED", "1") != "0"


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """``[tokens, 2 * len(inv_freq)]`` fp32: per token the sines, then the cosines, of
    ``position * inv_freq``, computed as the rotary kernels compute them (elementwise.cu)."""
    _cuda(positions, inv_freq)
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32:
        raise KernelError("rope_table: int32 positions and fp32 frequencies")
    half = inv_freq.numel()
    out = torch.empty((positions.numel(), 2 * half), dtype=torch.float32, device=positions.device)
    lib = _lib("elementwise")
    rc = lib.mi_rope_table(_ptr(positions), _ptr(inv_freq), _ptr(out), positions.numel(), half, _stream())
    _finish(lib, rc, "rope_table")
    return out


FUSE_DECODE_ROPE_MAX_REQUESTS = 16


def decode_rope_fusable(q_dtype: torch.dtype, head_dim: int, decode_only: bool, n_requests: int) -> bool:
    """Whether ``attention`` should rotate q and store the new key and value itself (the decode
    kernel of bfloat16 steps in which every request brings one token).  Measured inside the
    captured step at Llama 3.1 8B sizes: one kernel boundary less per layer is worth 0.5 % at
    batch 8; at batch 64 the separate kernel is 1 % faster (while it runs, the attention kernel's
    copy warps are already fetching pages), hence the limit."""
    return (FUSE_DECODE_ROPE and decode_only and q_dtype == torch.bfloat16 and head_dim in (64, 128, 256)
            and n_requests <= FUSE_DECODE_ROPE_MAX_REQUESTS)


def attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, cache, ctx, nq: int, nkv: int,
              head_dim: int, scale: float, window: int = 0, rope_table: torch.Tensor | None = None,
              chunk: int = 0) -> None:
    """Attention of this step's queries over one cache layer.

    ``cache`` is a ``LayerCache`` (its ``k``/``v`` pages and group index), ``ctx`` the
    ``StepContext`` (block tables, lengths, query tiles).  float32 runs the CUDA-core kernel;
    bfloat16 runs the tensor-core kernels: the balanced decode kernel when every request brings
    one token, otherwise the tcgen05 prefill kernel where it takes the sizes and the mma.sync
    prefill kernel elsewhere.  ``rope_table`` (only where ``decode_rope_fusable``): q, k, v are
    un-rotated and not yet stored; the decode kernel does both.  ``window`` > 0: a query sees the last
    ``window`` positions only; ``chunk`` > 0: only the keys of its own chunk of positions,
    ``j >= (p // chunk) * chunk`` (one of the two; the mma.sync kernels take a chunk as a negative window).
    """
    group = ctx.groups[cache.group]
    if window and chunk:
        raise KernelError("attention: a window or chunks, not both")
    if chunk < 0 or window < 0:
        raise KernelError("attention: a window and a chunk size are positive")
    if q.dtype == torch.bfloat16:
        mask = -int(chunk) if chunk else int(window)
        if ctx.decode_only:
            attention_decode_balanced(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                                      ctx.q_start, ctx.kv_len, ctx.n_requests, nq, nkv, head_dim, scale, mask,
                                      table_rows=group.table_rows, rope_table=rope_table,
                                      store_kv=bool(cache.writes))
        else:
            if rope_table is not None:
                raise KernelError("attention: only the decode kernel rotates and stores by itself")
            tc = USE_TC_PREFILL and prefill_tc_supported(nq, nkv, head_dim, group.page_size)
            tt = (prefill_tc_tile_tokens if tc else prefill_tile_tokens)(nq // nkv)
            tile_req, tile_tok0, n_tiles = ctx.q_tiles(tt)
            if SPLIT_MIXED_STEPS and ctx.n_single and tt in ctx.tiles_multi:
                # a mixed step: the single tokens through the decode kernel (their keys spread over
                # all blocks), the prompt portions through the prefill kernel; disjoint rows of `out`
                attention_decode_balanced(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                                          ctx.single_q_start, ctx.single_kv_len, ctx.n_single, nq, nkv, head_dim,
                                          scale, mask, table_rows=ctx.single_rows)
                tile_req, tile_tok0, n_tiles = ctx.tiles_multi[tt]
            if tc:
                attention_prefill_tc(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                                     ctx.q_start, ctx.q_len, ctx.kv_len, tile_req, tile_tok0, n_tiles, tt,
                                     nq, nkv, head_dim, scale, window, table_rows=group.table_rows, chunk=chunk)
            else:
                attention_prefill(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                                  ctx.q_start, ctx.q_len, ctx.kv_len, tile_req, tile_tok0, n_tiles, tt,
                                  nq, nkv, head_dim, scale, mask, table_rows=group.table_rows)
        return
    if chunk:
        raise KernelError("attention: float32 chunks go through attention_ext")
    tile_req, tile_tok0, n_tiles = ctx.q_tiles(ATTENTION_TILE_TOKENS)
    attention_generic(q, q_stride, out, cache.k, cache.v, group.block_table, group.page_size,
                      ctx.q_start, ctx.q_len, ctx.kv_len, tile_req, tile_tok0, n_tiles,
                      nq, nkv, head_dim, scale, window, table_rows=group.table_rows)


def _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size, ints):
    for name, t in ints:
        if t is not None and t.dtype != torch.int32:
            raise KernelError(f"attention: {name} must be int32")
    if kcache.dtype != q.dtype or vcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and caches must share a dtype")
    if kcache.dim() != 4 or kcache.shape[1:] != (nkv, page_size, head_dim) or not kcache.is_contiguous() \
            or vcache.shape != kcache.shape or not vcache.is_contiguous():
        raise KernelError("attention: caches must be contiguous [pages, nkv, page_size, d]")
    if out.dim() != 2 or out.shape[1] != nq * head_dim or not out.is_contiguous():
        raise KernelError("attention: out must be contiguous [tokens, nq * d]")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("attention: block_table must be [rows, pages] with unit inner stride")


# Arrival counters of the split-key decode kernel, per device: zero between calls (the kernel
# resets them).  Never freed once handed out: a captured CUDA graph may hold the address.
_decode_counter_bufs: dict[int, list[torch.Tensor]] = {}


def _decode_counters(device: torch.device, n: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    stack = _decode_counter_bufs.setdefault(idx, [])
    if not stack or stack[-1].numel() < n:
        stack.append(torch.zeros(max(n, 16384), dtype=torch.int32, device=device))
    return stack[-1]


def attention_decode(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, kv_len,
                     n_requests, nq, nkv, head_dim, scale, window=0, n_splits=1, slice_chunks=None,
                     table_rows=None) -> None:
    """bfloat16 decode attention: one query token per request, keys cut into ``n_splits``
    slices whose partial results are merged through scratch memory (attention_mma.cu).
    Request ``b`` reads row ``table_rows[b]`` of ``block_table`` (row ``b`` without ``table_rows``).
    ``slice_chunks`` (an int32 tensor of one element on the device, read when the kernel
    runs) makes every slice that many 64-key chunks for all requests; without it every
    request's own keys are cut into ``n_splits`` equal slices."""
    _cuda(q, out, kcache, vcache, block_table, q_start, kv_len, slice_chunks, table_rows)
    if slice_chunks is not None and (slice_chunks.dtype != torch.int32 or slice_chunks.numel() < 1):
        raise KernelError("attention_decode: slice_chunks must be an int32 tensor of one element")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len),
                           ("table_rows", table_rows)))
    part_o = part_ml = counters = None
    lib = _waiting_lib("attention_mma", q.device)
    if n_splits > 1:
        part_o = torch.empty((n_requests * nq * n_splits, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n_requests * nq * n_splits, 2), dtype=torch.float32, device=q.device)
        counters = _decode_counters(q.device, lib.mi_attention_decode_counters(int(n_requests), nq, nkv))
    rc = lib.mi_attention_decode_sliced(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_table),
        block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(kv_len), int(n_requests), nq, nkv,
        head_dim, float(scale), int(window), int(n_splits), _ptr(slice_chunks), _ptr(part_o), _ptr(part_ml),
        _ptr(counters), _stream())
    _finish(lib, rc, "attention_decode")


# Scratch of the balanced decode kernel, per device: partial results, their (max, sum) pairs and
# the per-unit chunk counters (zero between calls).  Never freed once handed out: a captured
# CUDA graph may hold the addresses.
_balanced_ws: dict[int, list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]]] = {}


def _balanced_workspace(device: torch.device, o_floats: int, ml_floats: int, counters: int):
    idx = _device_index(device)
    stack = _balanced_ws.setdefault(idx, [])
    if not stack or stack[-1][0].numel() < o_floats or stack[-1][1].numel() < ml_floats or stack[-1][2].numel() < counters:
        stack.append((torch.empty(max(o_floats, 1 << 20), dtype=torch.float32, device=device),
                      torch.empty(max(ml_floats, 1 << 14), dtype=torch.float32, device=device),
                      torch.zeros(max(counters, 4096), dtype=torch.int32, device=device)))
    return stack[-1]


def attention_decode_balanced(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, kv_len,
                              n_requests, nq, nkv, head_dim, scale, window=0, table_rows=None,
                              rope_table: torch.Tensor | None = None, store_kv: bool = True,
                              sinks: torch.Tensor | None = None) -> None:
    """bfloat16 decode attention with the keys of all requests spread evenly over persistent
    blocks, whatever the requests' lengths (attention_decode_balanced_kernel): no plan from the
    host, the blocks read the lengths themselves.  With ``rope_table`` (``rope_table()`` of the
    step's positions) q, k and v come as the projection left them (one row per token: q heads, k
    heads, v heads): the kernel rotates q itself and, with ``store_kv``, rotates the new key and
    writes it and the new value into their page before it reads them.  ``sinks`` (fp32 ``[nq]``): a score per
    head that joins the softmax's denominator without a key or a value."""
    _cuda(q, out, kcache, vcache, block_table, q_start, kv_len, table_rows, rope_table, sinks)
    _opt_f32(sinks, nq, "attention_decode (sinks)")
    if rope_table is not None and (rope_table.dtype != torch.float32 or not rope_table.is_contiguous()
                                   or rope_table.shape[-1] != head_dim):
        raise KernelError("attention_decode: the rotary table must be contiguous fp32 [tokens, head_dim]")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("kv_len", kv_len),
                           ("table_rows", table_rows)))
    lib = _waiting_lib("attention_mma", q.device)
    grid, o_floats, ml_floats, counters = c_int(0), ctypes.c_longlong(0), ctypes.c_longlong(0), c_int(0)
    rc = lib.mi_attention_decode_balanced_scratch(int(n_requests), nq, nkv, head_dim, _sms(q.device), ctypes.byref(grid),
                                                  ctypes.byref(o_floats), ctypes.byref(ml_floats), ctypes.byref(counters))
    if rc != 0:
        raise KernelError("attention_decode: " + lib.mi_error_message().decode("utf-8", "replace"))
    part_o, part_ml, count = _balanced_workspace(q.device, int(o_floats.value), int(ml_floats.value), int(counters.value))
    rc = lib.mi_attention_decode_balanced(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_table),
        block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(kv_len), int(n_requests), nq, nkv,
        head_dim, float(scale), int(window), int(grid.value), _ptr(part_o), _ptr(part_ml), _ptr(count),
        _ptr(rope_table), 1 if store_kv else 0, _ptr(sinks), _stream())
    _finish(lib, rc, "attention_decode")


def decode_unit_cost(chunks: int | None = None) -> int:
    """What the balanced decode kernel reckons a block pays for taking up one (request, head
    group) unit, in 64-key chunks, when it cuts the requests' keys into equal stretches (so that a
    block with many short requests gets fewer keys than one inside a long request).  Sets it when
    given; returns the value that was in force before."""
    return int(_lib("attention_mma").mi_attention_decode_balanced_unit_cost(-1 if chunks is None else int(chunks)))


def attention_wait_status(reset: bool = True) -> int:
    """1 if a tensor-core attention kernel gave up waiting for a copy since the last reset
    (its output was then invalid); synchronises the device."""
    return int(_lib("attention_mma").mi_attention_wait_status(1 if reset else 0))


def attention_prefill(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, q_len, kv_len,
                      tile_req, tile_tok0, n_tiles, tile_tokens, nq, nkv, head_dim, scale, window=0,
                      table_rows=None) -> None:
    """bfloat16 attention of query portions of any length over the paged cache (attention_mma.cu)."""
    _cuda(q, out, kcache, vcache, block_table, q_start, q_len, kv_len, tile_req, tile_tok0, table_rows)
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("q_len", q_len),
                           ("kv_len", kv_len), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                           ("table_rows", table_rows)))
    lib = _waiting_lib("attention_mma", q.device)
    rc = lib.mi_attention_prefill(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), _ptr(block_table),
        block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(q_len), _ptr(kv_len), _ptr(tile_req),
        _ptr(tile_tok0), int(n_tiles), int(tile_tokens), nq, nkv, head_dim, float(scale), int(window),
        _stream())
    _finish(lib, rc, "attention_prefill")


USE_TC_PREFILL = os.environ.get("MINI_INFER_TC_PREFILL", "1") != "0"


def prefill_tc_supported(nq: int, nkv: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill kernel (attention_tc.cu) takes these sizes: head size 64 or
    128, a power-of-two page of 8 to 64 keys, a group size that divides 128.  (The same test as
    the library's own ``mi_attention_prefill_tc_supported``, made here so that a model the
    kernel does not take never compiles it.)"""
    if head_dim not in (64, 128) or page_size < 8 or page_size > 64 or page_size & (page_size - 1):
        return False
    if nq <= 0 or nkv <= 0 or nq % nkv:
        return False
    return 128 % min(nq // nkv, 128) == 0


def attention_prefill_tc(q, q_stride, out, kcache, vcache, block_table, page_size, q_start, q_len, kv_len,
                         tile_req, tile_tok0, n_tiles, tile_tokens, nq, nkv, head_dim, scale, window=0,
                         table_rows=None, sinks: torch.Tensor | None = None,
                         slopes: torch.Tensor | None = None, chunk: int = 0) -> None:
    """bfloat16 attention of query portions over the paged cache on tcgen05 (attention_tc.cu);
    same arguments as ``attention_prefill``, and optionally ``sinks`` / ``slopes`` (fp32 ``[nq]``: a
    score per head in the softmax's denominator without a key; a distance bias ``slope * (i - j)``
    taken off the scaled scores) and ``chunk`` (> 0: a query at position ``p`` sees only the keys of its
    own chunk of positions, ``j >= (p // chunk) * chunk``)."""
    _cuda(q, out, kcache, vcache, block_table, q_start, q_len, kv_len, tile_req, tile_tok0, table_rows, sinks, slopes)
    for name, t in (("sinks", sinks), ("slopes", slopes)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != nq or not t.is_contiguous()):
            raise KernelError(f"attention_prefill_tc: {name} must be contiguous fp32 [{nq}]")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: bfloat16 only")
    _check_attention_args(q, out, kcache, vcache, block_table, nq, nkv, head_dim, page_size,
                          (("block_table", block_table), ("q_start", q_start), ("q_len", q_len),
                           ("kv_len", kv_len), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                           ("table_rows", table_rows)))
    lib = _waiting_lib("attention_tc", q.device)
    rc = lib.mi_attention_prefill_tc_masked(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache), int(kcache.shape[0]),
        _ptr(block_table), block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(q_len), _ptr(kv_len),
        _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), int(tile_tokens), nq, nkv, head_dim, float(scale),
        int(window), int(chunk), _ptr(sinks), _ptr(slopes), _stream())
    _finish(lib, rc, "attention_prefill_tc")


def attention_tc_status(reset: bool = True) -> int:
    """Non-zero when a block of the tcgen05 prefill kernel gave up a bounded wait since the
    last reset (its output is then wrong).  Synchronises the device."""
    return int(_lib("attention_tc").mi_attention_tc_status(1 if reset else 0))


def attention_generic(
    q: torch.Tensor,
    q_stride: int,
    out: torch.Tensor,
    kcache: torch.Tensor,
    vcache: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    q_start: torch.Tensor,
    q_len: torch.Tensor,
    kv_len: torch.Tensor,
    tile_req: torch.Tensor,
    tile_tok0: torch.Tensor,
    n_tiles: int,
    nq: int,
    nkv: int,
    head_dim: int,
    scale: float,
    window: int = 0,
    table_rows: torch.Tensor | None = None,
) -> None:
    """Causal attention of query portions over the paged cache (see attention_generic.cu).

    ``q`` is any tensor whose element ``(token t, head h, k)`` lies at
    ``t * q_stride + h * head_dim + k`` from its first element.
    """
    _cuda(q, out, kcache, vcache, block_table, q_start, q_len, kv_len, tile_req, tile_tok0, table_rows)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len),
                    ("kv_len", kv_len), ("tile_req", tile_req), ("tile_tok0", tile_tok0),
                    ("table_rows", table_rows)):
        if t is not None and t.dtype != torch.int32:
            raise KernelError(f"attention: {name} must be int32")
    if kcache.dtype != q.dtype or vcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and caches must share a dtype")
    if kcache.dim() != 4 or kcache.shape[1:] != (nkv, page_size, head_dim) or not kcache.is_contiguous() \
            or vcache.shape != kcache.shape or not vcache.is_contiguous():
        raise KernelError("attention: caches must be contiguous [pages, nkv, page_size, d]")
    if out.dim() != 2 or out.shape[1] != nq * head_dim or not out.is_contiguous():
        raise KernelError("attention: out must be contiguous [tokens, nq * d]")
    if block_table.dim() != 2 or block_table.stride(1) != 1:
        raise KernelError("attention: block_table must be [requests, pages] with unit inner stride")
    lib = _lib("attention_generic")
    if lib.mi_attention_generic_tile_tokens() != ATTENTION_TILE_TOKENS:
        raise KernelError("attention: the kernel's tile size differs from ATTENTION_TILE_TOKENS")
    rc = lib.mi_attention_generic(
        _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(kcache), _ptr(vcache),
        _ptr(block_table), block_table.stride(0), _ptr(table_rows), int(page_size), _ptr(q_start), _ptr(q_len),
        _ptr(kv_len), _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), nq, nkv, head_dim,
        float(scale), int(window), _code(q.dtype), _stream())
    _finish(lib, rc, "attention")


def sample(
    logits: torch.Tensor,
    out: torch.Tensor,
    *,
    temperature: torch.Tensor | None = None,
    top_k: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    seed_lo: torch.Tensor | None = None,
    seed_hi: torch.Tensor | None = None,
    draw_index: torch.Tensor | None = None,
) -> torch.Tensor:
    """One token id per row of fp32 ``logits [B, V]`` into int32 ``out [B]`` (see sampling.cu)."""
    _cuda(logits, out, temperature, top_k, top_p, seed_lo, seed_hi, draw_index)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be fp32 [B, V] with unit inner stride")
    B, V = logits.shape
    if out.dtype != torch.int32 or out.shape != (B,) or not out.is_contiguous():
        raise KernelError("sample: out must be int32 [B]")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
                        ("top_p", top_p, torch.float32), ("seed_lo", seed_lo, torch.int32),
                        ("seed_hi", seed_hi, torch.int32), ("draw_index", draw_index, torch.int32)):
        if t is not None and (t.dtype != dt or t.shape != (B,) or not t.is_contiguous()):
            raise KernelError(f"sample: {name} must be {dt} [B]")
    lib = _lib("sampling")
    rc = lib.mi_sample(_ptr(logits), logits.stride(0) if B > 1 else V, B, V, _ptr(temperature),
                       _ptr(top_k), _ptr(top_p), _ptr(seed_lo), _ptr(seed_hi), _ptr(draw_index),
                       _ptr(out), _stream())
    _finish(lib, rc, "sample")
    return out


TMA_GEMM_MAX_ROWS = 128            # what gemm_tma.cu takes
# ``linear`` routes inputs of up to this many rows to gemm_tma.  Measured on a B200 inside a
# captured decode step (Llama 3.1 8B sizes, milliseconds per step, own product against the
# library's): up to 16 rows the own product is ahead, because it marks the weights to leave the
# L2 first and does the block's additions and norms in its epilogues (batch 8: 3.74 vs 4.05;
# batch 16: 4.17 vs 4.42); from 32 rows on the library is (5.23 vs 5.15; 64 rows: 7.34 vs 6.63).
TMA_GEMM_DISPATCH_ROWS = 16
USE_TMA_GEMM = os.environ.get("MINI_INFER_TMA_GEMM", "1") != "0"
_tma_ws: dict[int, list[tuple[torch.Tensor, torch.Tensor]]] = {}


def _tma_workspace(device: torch.device, floats: int, counters: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Partial tiles and per-tile arrival counters (zero between calls) of the streaming
    product, per device; never freed once handed out (a captured graph may hold the address)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    stack = _tma_ws.setdefault(idx, [])
    if not stack or stack[-1][0].numel() < floats or stack[-1][1].numel() < counters:
        stack.append((
            torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device),
            torch.zeros(max(counters, 4096), dtype=torch.int32, device=device),
        ))
    return stack[-1]


def gemm_tma_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_tma`` takes these operands (few rows, 16-byte aligned rows)."""
    return (x.dim() == 2 and w.dim() == 2 and 0 < x.shape[0] <= TMA_GEMM_MAX_ROWS and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.is_contiguous() and (x.shape[0] == 1 or x.stride(0) % 8 == 0)
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


TMA_GEMM_FUSED_ROWS = 16    # the fused epilogues of gemm_tma take one group of 16 token columns
TMA_GEMM_STAT_TOKENS = 16   # columns of a statistics table
TMA_GEMM_TILE_ROWS = 128    # rows of W per tile: one row of a statistics table


class RowStats:
    """Sums of squares of the rows of an fp32 stream ``[M, width]``, 128 features at a time
    (``sums [ceil(width / 128), 16]``, column = row of the stream), as the residual epilogue of
    ``gemm_tma`` leaves them, with the ``eps`` of the norm they are meant for."""

    __slots__ = ("sums", "width", "eps")

    def __init__(self, sums: torch.Tensor, width: int, eps: float) -> None:
        self.sums, self.width, self.eps = sums, int(width), float(eps)


def gemm_tma(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
             swiglu: bool | int = False, row_stats: RowStats | None = None,
             residual: torch.Tensor | None = None, gain: torch.Tensor | None = None,
             eps: float = 0.0):
    """``x [M <= 128, K] @ w [N, K]^T`` for bfloat16 operands on the tcgen05 tensor cores,
    streaming ``w`` once through TMA (gemm_tma.cu); the result is bfloat16 or float32.  With
    ``swiglu`` (True or 1: SiLU; 2: the tanh form of GELU) the rows of ``w`` alternate gate, up and
    the result is ``[M, N / 2]``: ``act(gate) * up`` computed on the fp32 accumulators in the
    product's epilogue.

    Two fused forms for at most 16 rows.  ``row_stats``: every row of the product is first
    scaled by ``rsqrt(sum of its squares / width + eps)`` (the input was multiplied by a norm's
    gain, not yet divided by its root mean square).  ``residual [M, N]`` fp32 with ``gain [N]``
    fp32: the product is added to ``residual`` in place, the result is ``residual * gain`` and a
    second value is returned, the ``RowStats`` of the new residual for a norm with ``eps``."""
    _cuda(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tma: operands must be bfloat16")
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or x.stride(1) != 1 or not w.is_contiguous():
        raise KernelError(f"gemm_tma: shapes {tuple(x.shape)} x {tuple(w.shape)}^T do not match")
    M, K = x.shape
    N = w.shape[0]
    lib = _waiting_lib("gemm_tma", x.device)
    blocks = _sms(x.device)
    floats, counters = ctypes.c_longlong(0), c_int(0)
    lib.mi_gemm_tma_workspace(M, N, blocks, ctypes.byref(floats), ctypes.byref(counters))
    partial, count = _tma_workspace(x.device, int(floats.value), int(counters.value))
    if swiglu and N % 2:
        raise KernelError("gemm_tma: the gate/up epilogue needs an even number of rows")
    n_out = N // 2 if swiglu else N
    out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    sums_in = tiles_in = width = None
    if row_stats is not None:
        sums_in, width = row_stats.sums, row_stats.width
        tiles_in = -(-width // TMA_GEMM_TILE_ROWS)
        if (width != K or sums_in.dtype != torch.float32 or not sums_in.is_contiguous()
                or tuple(sums_in.shape) != (tiles_in, TMA_GEMM_STAT_TOKENS)):
            raise KernelError(f"gemm_tma: row statistics {tuple(sums_in.shape)} of width {width} do not fit K = {K}")
    stats_out = None
    if residual is not None:
        if (gain is None or gain.dtype != torch.float32 or gain.numel() != N or not gain.is_contiguous()
                or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N) or not residual.is_contiguous()):
            raise KernelError("gemm_tma: the residual epilogue needs a contiguous fp32 stream [M, N] and an fp32 gain [N]")
        _cuda(residual, gain)
        stats_out = torch.empty((-(-N // TMA_GEMM_TILE_ROWS), TMA_GEMM_STAT_TOKENS), dtype=torch.float32,
                                device=x.device)
    rc = lib.mi_gemm_tma_fused(_ptr(x), x.stride(0) if M > 1 else K, _ptr(w), _ptr(out), n_out, M, N, K,
                               _code(out_dtype), int(swiglu), blocks, _ptr(partial), _ptr(count),
                               _ptr(sums_in), tiles_in or 0, width or 0, row_stats.eps if row_stats else 0.0,
                               _ptr(residual), _ptr(gain), _ptr(stats_out), _stream())
    _finish(lib, rc, "gemm_tma")
    if residual is not None:
        return out, RowStats(stats_out, N, eps)
    return out


def gemm_tma_status(reset: bool = True) -> int:
    """Non-zero when a block of the streaming product gave up a bounded wait since the last
    reset (its output is then wrong).  Synchronises the device."""
    return int(_lib("gemm_tma").mi_gemm_tma_status(1 if reset else 0))


def fused_norms_enabled() -> bool:
    """Whether additions and norms may ride on the streaming product's epilogues
    (``MINI_INFER_FUSED_NORMS=0`` keeps them as kernels of their own, for comparisons)."""
    return USE_TMA_GEMM and os.environ.get("MINI_INFER_FUSED_NORMS", "1") != "0"


def linear_fusable(n_rows: int, w: torch.Tensor) -> bool:
    """Whether a product of ``n_rows`` rows with ``w`` has the fused forms of ``gemm_tma``
    (``row_stats`` on its input side, ``linear_into_stream`` on its output side)."""
    return (fused_norms_enabled() and 0 < n_rows <= min(TMA_GEMM_DISPATCH_ROWS, TMA_GEMM_FUSED_ROWS)
            and w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
            and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0)


def linear_into_stream(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, gain: torch.Tensor,
                       eps: float) -> tuple[torch.Tensor, "RowStats"]:
    """``residual += x w^T`` in place (fp32); returns ``residual * gain`` in bfloat16 and the row
    statistics a product with ``row_stats`` needs to finish an RMS norm with ``eps``."""
    if not linear_fusable(x.shape[0], w) or not gemm_tma_ok(x, w):
        raise KernelError("linear_into_stream: these operands have no fused form (ask linear_fusable first)")
    return gemm_tma(x, w, torch.bfloat16, residual=residual, gain=gain, eps=eps)


GLU_ACT = {"silu": 1, "gelu_tanh": 2}


def linear_swiglu(x: torch.Tensor, w_pairs: torch.Tensor, row_stats: "RowStats | None" = None,
                  act: str = "silu") -> torch.Tensor:
    """``act(x Wg^T) * (x Wu^T)`` for a merged projection whose rows alternate gate, up
    (``w_pairs [2 I, K]``); ``act`` is ``"silu"`` or ``"gelu_tanh"``.  Decode-sized bfloat16 inputs
    run the product and the activation as one kernel (gemm_tma with its gate/up epilogue);
    everything else runs ``linear`` and an activation-and-multiply kernel on the interleaved
    result.  ``row_stats``: see ``gemm_tma``."""
    if act not in GLU_ACT:
        raise KernelError(f"linear_swiglu: unknown activation {act!r}")
    if (x.dtype == torch.bfloat16 and USE_TMA_GEMM and x.shape[0] <= TMA_GEMM_DISPATCH_ROWS
            and w_pairs.dtype == torch.bfloat16 and gemm_tma_ok(x, w_pairs)):
        return gemm_tma(x, w_pairs, torch.bfloat16, swiglu=GLU_ACT[act], row_stats=row_stats)
    if row_stats is not None:
        raise KernelError("linear_swiglu: row statistics need the streaming product (ask linear_fusable first)")
    if act == "silu":
        return silu_mul(linear(x, w_pairs), pairs=True)
    return glu_mul_pairs(linear(x, w_pairs), act)


_MM_OUT_DTYPE: bool | None = None


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           row_stats: "RowStats | None" = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K]^T``.

    float32 operands run the true-fp32 CUDA-core kernel (never a library product, which
    could pick a reduced-precision mode).  bfloat16 operands with few rows (decode) run the
    weight-streaming tcgen05 kernel of gemm_tma.cu, which starts streaming weights while the
    kernel before it still runs; other bfloat16 operands use the library product with fp32
    accumulation, as the reference does for every linear layer (``distributed/linear.py:167``).
    ``out_dtype=float32`` keeps the accumulator's precision in the result (used for logits).
    ``row_stats`` (streaming product only): see ``gemm_tma``.
    """
    global _MM_OUT_DTYPE, launch_count
    if row_stats is not None:
        if not linear_fusable(x.shape[0], w) or not gemm_tma_ok(x, w):
            raise KernelError("linear: row statistics need the streaming product (ask linear_fusable first)")
        return gemm_tma(x, w, out_dtype or torch.bfloat16, row_stats=row_stats)
    if x.dtype == torch.float32:
        if w.dtype != torch.float32:
            raise KernelError("linear: fp32 activations need fp32 weights")
        return gemm_f32(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"linear: unsupported dtypes {x.dtype} x {w.dtype}")
    _cuda(x, w)
    if out_dtype not in (None, torch.bfloat16, torch.float32):
        raise KernelError(f"linear: unsupported output dtype {out_dtype}")
    if USE_TMA_GEMM and x.shape[0] <= TMA_GEMM_DISPATCH_ROWS and gemm_tma_ok(x, w):
        return gemm_tma(x, w, out_dtype or torch.bfloat16)
    launch_count += 1
    if out_dtype in (None, torch.bfloat16):
        return torch.mm(x, w.t())
    if out_dtype != torch.float32:
        raise KernelError(f"linear: unsupported output dtype {out_dtype}")
    if _MM_OUT_DTYPE is None:
        try:
            torch.mm(x[:1], w[:1].t(), out_dtype=torch.float32)
            _MM_OUT_DTYPE = True
        except (TypeError, RuntimeError):
            _MM_OUT_DTYPE = False
    if _MM_OUT_DTYPE:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t()).float()


# --------------------------------------------------------------------------------------- layer norm


def embedding_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float) -> torch.Tensor:
    """``float(table[ids]) * scale`` as the fp32 residual stream ``[M, H]``."""
    _cuda(table, ids)
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("embedding: ids must be a contiguous int32 vector")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embedding: table must be a contiguous [V, H] matrix")
    V, H = table.shape
    out = torch.empty((ids.shape[0], H), dtype=torch.float32, device=table.device)
    lib = _lib("layernorm")
    rc = lib.mi_embedding_scaled(_ptr(table), _ptr(ids), _ptr(out), ids.shape[0], H, V, float(scale),
                                 _code(table.dtype), _stream())
    _finish(lib, rc, "embedding")
    return out


def add_layernorm(stream: torch.Tensor, adds, norms, eps: float, dtype: torch.dtype, *,
                  rows: torch.Tensor | None = None, update_stream: bool = True):
    """Layer norm(s) of ``r = stream + sum(adds)`` (fp32; ``adds``: up to two ``[M, H]`` tensors
    of ``dtype``).  ``norms``: one or two ``(gain, bias)`` pairs (fp32 ``[H]``); one output in
    ``dtype`` per pair.  Without ``rows`` and with ``update_stream`` the stream is replaced by
    ``r`` in place; with ``rows`` (int32) only those rows are normalised and the stream stays."""
    adds = [a for a in adds if a is not None]
    if len(adds) > 2 or not 1 <= len(norms) <= 2:
        raise KernelError("layernorm: at most two addends and one or two norms")
    _cuda(stream, rows, *adds)
    if stream.dtype != torch.float32 or stream.dim() != 2 or not stream.is_contiguous():
        raise KernelError("layernorm: the stream must be a contiguous fp32 [M, H] matrix")
    H = stream.shape[1]
    for a in adds:
        if a.shape != stream.shape or a.dtype != dtype or not a.is_contiguous():
            raise KernelError("layernorm: addends must be contiguous, shaped like the stream, in the compute dtype")
    for w, b in norms:
        for t in (w, b):
            if t.dtype != torch.float32 or t.shape != (H,) or not t.is_contiguous():
                raise KernelError(f"layernorm: gains and biases must be fp32 [{H}]")
    if rows is not None and (rows.dtype != torch.int32 or rows.dim() != 1 or not rows.is_contiguous()):
        raise KernelError("layernorm: rows must be a contiguous int32 vector")
    M = stream.shape[0] if rows is None else rows.shape[0]
    outs = [torch.empty((M, H), dtype=dtype, device=stream.device) for _ in norms]
    a1 = adds[0] if adds else None
    a2 = adds[1] if len(adds) > 1 else None
    w2, b2 = norms[1] if len(norms) > 1 else (None, None)
    lib = _lib("layernorm")
    rc = lib.mi_add_layernorm(_ptr(stream), _ptr(a1), _ptr(a2),
                              _ptr(stream if (rows is None and update_stream and adds) else None), _ptr(rows),
                              _ptr(norms[0][0]), _ptr(norms[0][1]), _ptr(outs[0]), _ptr(w2), _ptr(b2),
                              _ptr(outs[1] if len(outs) > 1 else None), M, H, float(eps), _code(dtype), _stream())
    _finish(lib, rc, "layernorm")
    return outs


# --------------------------------------------------------------------------------------- rotation, unit norm, gates


def _cols(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: needs a [tokens, columns] tensor (or column range) with unit inner stride")


def rope_norm_store(packed: torch.Tensor, q_off: int, k_off: int, v_off: int, nq: int, nkv: int, d: int, dv: int, *,
                    positions: torch.Tensor | None, inv_freq: torch.Tensor | None, rot: int, unit_norm: bool,
                    eps: float, slots: torch.Tensor | None = None, kcache: torch.Tensor | None = None,
                    vcache: torch.Tensor | None = None) -> None:
    """In the packed projection ``[M, stride]`` (q at columns ``q_off``, ``nq`` heads of ``d``; k at
    ``k_off``, ``nkv`` heads of ``d``; v at ``v_off``, ``nkv`` heads of ``dv``): rotate q and k on their
    first ``rot`` dimensions (interleaved pairs, fp32 angles ``position * inv_freq[i]``), divide
    them by their root mean square over the head (``unit_norm``), write q and k back in place and
    store k and v at ``slots`` of the caches ``[pages, nkv, page_size, d | dv]``."""
    _cuda(packed, positions, inv_freq, slots, kcache, vcache)
    _cols(packed, "rope_norm")
    M, width = packed.shape
    if q_off + nq * d > width or k_off + nkv * d > width or v_off + nkv * dv > width:
        raise KernelError("rope_norm: a column range lies outside the packed projection")
    if rot:
        if positions is None or positions.dtype != torch.int32 or positions.shape != (M,):
            raise KernelError("rope_norm: positions must be int32 [M]")
        if inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.shape != (rot // 2,) or not inv_freq.is_contiguous():
            raise KernelError("rope_norm: inv_freq must be fp32 [rot / 2]")
    writes = kcache is not None
    page_size = 0
    if writes:
        if slots is None or slots.dtype != torch.int32 or slots.shape != (M,):
            raise KernelError("rope_norm: slots must be int32 [M]")
        for c, size in ((kcache, d), (vcache, dv)):
            if (c is None or c.dtype != packed.dtype or c.dim() != 4 or c.shape[1] != nkv or c.shape[3] != size
                    or not c.is_contiguous()):
                raise KernelError("rope_norm: caches must be contiguous [pages, nkv, page_size, size] in the packed dtype")
        page_size = int(kcache.shape[2])
        if vcache.shape[2] != page_size:
            raise KernelError("rope_norm: key and value pages differ in size")
    lib = _lib("rope_norm")
    rc = lib.mi_rope_norm_store(_ptr(packed), packed.stride(0), q_off, k_off, v_off, _ptr(positions), _ptr(inv_freq),
                                _ptr(slots), _ptr(kcache), _ptr(vcache), M, nq, nkv, d, dv, int(rot),
                                1 if unit_norm else 0, float(eps), page_size, 1 if writes else 0,
                                _code(packed.dtype), _stream())
    _finish(lib, rc, "rope_norm")


_ACT = {"sigmoid": 1, "silu": 2, None: 0}


def gate_mul(x: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, act: str | None, scale: float = 1.0,
             per: int = 1) -> None:
    """``out = x * act(gate) * scale`` element by element; ``x`` and ``out`` ``[M, C]`` (column ranges of
    wider tensors are fine), ``act`` ``"sigmoid"`` or ``"silu"``, fp32 arithmetic.  ``per`` > 1: one gate
    for every ``per`` neighbouring columns (a gate per head), ``gate`` being ``[M, C / per]``.  Without a
    gate (``gate`` and ``act`` None): ``out = x * scale``."""
    _cuda(x, gate, out)
    for t in (x, out) + ((gate,) if gate is not None else ()):
        _cols(t, "gate_mul")
    if (gate is None) != (act is None):
        raise KernelError("gate_mul: a gate and its activation come together")
    if (per <= 0 or x.shape[1] % per or x.shape != out.shape or x.dtype != out.dtype
            or (gate is not None and (tuple(gate.shape) != (x.shape[0], x.shape[1] // per) or gate.dtype != x.dtype))):
        raise KernelError("gate_mul: x and out must agree in shape, the gate has a column per group, one dtype")
    lib = _lib("rope_norm")
    rc = lib.mi_gate_mul(_ptr(x), x.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(out),
                         out.stride(0), x.shape[0],
                         x.shape[1], _ACT[act], float(scale), int(per), _code(x.dtype), _stream())
    _finish(lib, rc, "gate_mul")


def attention_kv(q: torch.Tensor, out: torch.Tensor, cache, ctx, nq: int, nkv: int, d: int, dv: int, scale: float,
                 window: int = 0) -> None:
    """Attention of this step's queries over one cache layer whose keys (size ``d``) and values
    (size ``dv``) may differ in size: the CUDA-core kernel with fp32 scores, weights and sums, for
    float32 and bfloat16 alike.  ``q`` and ``out`` are ``[M, nq * d]`` / ``[M, nq * dv]`` column ranges."""
    group = ctx.groups[cache.group]
    _cuda(q, out, cache.k, cache.v)
    _cols(q, "attention")
    _cols(out, "attention")
    if q.shape[1] != nq * d or out.shape[1] != nq * dv or q.dtype != out.dtype:
        raise KernelError("attention: q must be [M, nq * d] and out [M, nq * dv] in one dtype")
    kc, vc = cache.k, cache.v
    if (kc.dtype != q.dtype or vc.dtype != q.dtype or kc.dim() != 4 or vc.dim() != 4
            or kc.shape[1:] != (nkv, group.page_size, d) or vc.shape[1:] != (nkv, group.page_size, dv)
            or not kc.is_contiguous() or not vc.is_contiguous()):
        raise KernelError("attention: caches must be contiguous [pages, nkv, page_size, d | dv] in q's dtype")
    tile_req, tile_tok0, n_tiles = ctx.q_tiles(ATTENTION_TILE_TOKENS)
    lib = _lib("attention_generic")
    if lib.mi_attention_generic_tile_tokens() != ATTENTION_TILE_TOKENS:
        raise KernelError("attention: the kernel's tile size differs from ATTENTION_TILE_TOKENS")
    bt = group.block_table
    rc = lib.mi_attention_generic_kv(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kc), _ptr(vc), _ptr(bt), bt.stride(0),
        _ptr(group.table_rows), int(group.page_size), _ptr(ctx.q_start), _ptr(ctx.q_len), _ptr(ctx.kv_len),
        _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), nq, nkv, d, dv, float(scale), int(window),
        _code(q.dtype), _stream())
    _finish(lib, rc, "attention")


# --------------------------------------------------------------------------------------- recurrences


def _state_rows(state: torch.Tensor, what: str) -> int:
    if state.dtype != torch.float32 or state.dim() < 2 or not state.is_contiguous():
        raise KernelError(f"{what}: the state arena must be contiguous fp32 [slots, ...]")
    return state.stride(0)


def _f32vec(t: torch.Tensor | None, n: int, what: str) -> None:
    if t is not None and (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
        raise KernelError(f"{what}: needs a contiguous fp32 tensor of {n} elements")


def causal_conv(x: torch.Tensor, x_bias: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None,
                state: torch.Tensor, ctx, out: torch.Tensor, act: str | None = None) -> None:
    """Per channel ``out[t] = bias + sum_j weight[:, j] * in[t - (taps - 1 - j)]`` with ``in = x +
    x_bias``; the ``taps - 1`` inputs before a request's portion come from the head of its state
    row (``[taps - 1, C]``, oldest first; zeros at the start of a sequence).  The state is read
    only (the scan behind it moves it on: ``rglru_scan``, ``delta_scan``).  ``act`` ``"silu"``: the SiLU of
    the sum is written."""
    if act not in (None, "silu"):
        raise KernelError(f"causal_conv: unknown activation {act!r}")
    _cuda(x, x_bias, weight, bias, state, out)
    _cols(x, "causal_conv")
    _cols(out, "causal_conv")
    C = x.shape[1]
    if weight.dtype != torch.float32 or weight.dim() != 2 or weight.shape[0] != C or not weight.is_contiguous():
        raise KernelError("causal_conv: the taps must be contiguous fp32 [C, taps]")
    taps = weight.shape[1]
    _f32vec(x_bias, C, "causal_conv")
    _f32vec(bias, C, "causal_conv")
    stride = _state_rows(state, "causal_conv")
    if stride < (taps - 1) * C or out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("causal_conv: state row too short, or out does not match x")
    lib = _lib("recurrent")
    rc = lib.mi_causal_conv(_ptr(x), x.stride(0), _ptr(x_bias), _ptr(weight), _ptr(bias), _ptr(state), stride,
                            _ptr(ctx.q_start), _ptr(ctx.q_len), _ptr(ctx.state_slot), _ptr(out), out.stride(0),
                            ctx.n_requests, _max_q_len(ctx), C, taps, 1 if act == "silu" else 0, _code(x.dtype),
                            _stream())
    _finish(lib, rc, "causal_conv")


def _max_q_len(ctx) -> int:
    return 1 if ctx.decode_only else max(ctx.host_q_len)


RGLRU_CHUNK = 64     # tokens per chunk of the chunked walk; portions up to this long are walked plainly


def rglru_scan(gates: torch.Tensor, gate_bias_r: torch.Tensor, gate_bias_i: torch.Tensor, lam: torch.Tensor,
               decay_scale: float, u: torch.Tensor, y: torch.Tensor, y_bias: torch.Tensor | None,
               x_in: torch.Tensor, x_in_bias: torch.Tensor | None, taps: int, state: torch.Tensor, ctx,
               out: torch.Tensor) -> None:
    """The real-gated linear recurrent unit over each request's portion, from and into its state
    row ``[taps - 1 + 1, C]`` (the convolution's last inputs, then the recurrent state):
    ``r = sigmoid(g_r + b_r)``, ``i = sigmoid(g_i + b_i)``, ``log a = -decay_scale * r * softplus(lam)``,
    ``S = a S + sqrt(1 - a^2) * i * u``, ``out = S * gelu_tanh(y + y_bias)``.  ``gates`` is fp32
    ``[blocks, M, 2 * bw]`` (per block of ``bw`` channels the ``r`` then the ``i`` pre-activations)."""
    _cuda(gates, gate_bias_r, gate_bias_i, lam, u, y, y_bias, x_in, x_in_bias, state, out)
    for t in (u, y, x_in, out):
        _cols(t, "rglru")
    M, C = u.shape
    if gates.dtype != torch.float32 or gates.dim() != 3 or gates.shape[1] != M or not gates.is_contiguous():
        raise KernelError("rglru: gates must be contiguous fp32 [blocks, M, 2 * bw]")
    bw = gates.shape[2] // 2
    if gates.shape[0] * bw != C:
        raise KernelError("rglru: blocks * bw must equal the channel count")
    for t in (gate_bias_r, gate_bias_i, lam):
        _f32vec(t, C, "rglru")
    _f32vec(y_bias, C, "rglru")
    _f32vec(x_in_bias, C, "rglru")
    stride = _state_rows(state, "rglru")
    if stride < taps * C:
        raise KernelError("rglru: state row too short")
    lib = _lib("recurrent")
    longest = _max_q_len(ctx)
    if u.dtype == torch.bfloat16 and longest > RGLRU_CHUNK:
        # long portions: chunks side by side (the float32 path keeps the plain walk, whose sums do not
        # depend on where a portion starts)
        global launch_count
        n_chunks = -(-longest // RGLRU_CHUNK)
        scratch = torch.empty(lib.mi_rglru_chunked_scratch(ctx.n_requests, n_chunks, C), dtype=torch.float32,
                              device=u.device)
        rc = lib.mi_rglru_scan_chunked(_ptr(gates), M, bw, _ptr(gate_bias_r), _ptr(gate_bias_i), _ptr(lam),
                                       float(decay_scale), _ptr(u), u.stride(0), _ptr(y), y.stride(0), _ptr(y_bias),
                                       _ptr(x_in), x_in.stride(0), _ptr(x_in_bias), _ptr(state), stride, int(taps),
                                       _ptr(ctx.q_start), _ptr(ctx.q_len), _ptr(ctx.state_slot), _ptr(out),
                                       out.stride(0), ctx.n_requests, C, _ptr(scratch), n_chunks, RGLRU_CHUNK,
                                       _code(u.dtype), _stream())
        _finish(lib, rc, "rglru")
        launch_count += 1
        return
    rc = lib.mi_rglru_scan(_ptr(gates), M, bw, _ptr(gate_bias_r), _ptr(gate_bias_i), _ptr(lam), float(decay_scale),
                           _ptr(u), u.stride(0), _ptr(y), y.stride(0), _ptr(y_bias), _ptr(x_in), x_in.stride(0),
                           _ptr(x_in_bias), _ptr(state), stride, int(taps), _ptr(ctx.q_start), _ptr(ctx.q_len),
                           _ptr(ctx.state_slot), _ptr(out), out.stride(0), ctx.n_requests, C, _code(u.dtype), _stream())
    _finish(lib, rc, "rglru")


GLA_CHUNK = 128      # tokens per chunk of the chunked walk of gated linear attention


def gla_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor | None, z_bias: torch.Tensor | None,
             tau: float, q_scale: float, heads: int, dk: int, dv: int, state: torch.Tensor, ctx,
             head_decay: torch.Tensor | None = None, tok_gates: torch.Tensor | None = None,
             extra_col: bool = False) -> torch.Tensor:
    """Gated linear attention over each request's portion, from and into its state row
    ``[heads, dk, dv]``: ``S = diag(alpha) S + k v^T``, ``o = S^T (q * q_scale)`` with
    ``alpha = sigmoid(z + z_bias)^(1 / tau)``.  q, k, v: column ranges of one packed projection;
    ``z`` fp32 ``[M, heads * dk]``.  With ``head_decay`` (fp32 ``[heads]``) every head has one fixed
    decay in the place of ``alpha`` and ``z`` is not read (linear attention with a fixed decay, or
    retention).  With ``tok_gates`` (fp32 ``[M, heads, 3]``) the decay, the same for all key channels, and a
    factor on ``k`` come per token and head from its first two numbers.  With ``extra_col`` a head of the
    state and of ``o`` has one more value column, whose values are all ones: the state row is
    ``[heads, dk, dv + 1]`` and ``o [M, heads * (dv + 1)]``, the last column of a head being ``sum(k) . q``.
    Returns fp32 ``o [M, heads * dv]``."""
    _cuda(q, k, v, z, z_bias, state, head_decay, tok_gates)
    for t in (q, k, v) + ((z,) if z is not None else ()):
        _cols(t, "gla")
    M = q.shape[0]
    if q.stride(0) != k.stride(0) or q.dtype != k.dtype:
        raise KernelError("gla: q and k must be column ranges of one matrix")
    if q.dtype != v.dtype and (q.dtype, v.dtype) != (torch.float32, torch.bfloat16):
        raise KernelError("gla: q and k have the values' dtype, or are fp32 beside bfloat16 values")
    if q.shape[1] != heads * dk or k.shape[1] != heads * dk or v.shape[1] != heads * dv:
        raise KernelError("gla: q, k must be [M, heads * dk] and v [M, heads * dv]")
    if head_decay is None and z is None and tok_gates is None:
        raise KernelError("gla: needs z (a decay per channel), head_decay (one per head) or tok_gates (per token and head)")
    if tok_gates is not None and (tok_gates.dtype != torch.float32 or tok_gates.shape != (M, heads, 3)
                                  or not tok_gates.is_contiguous()):
        raise KernelError("gla: tok_gates must be contiguous fp32 [M, heads, 3]")
    dvx = dv + (1 if extra_col else 0)
    if z is not None and (z.dtype != torch.float32 or z.shape != (M, heads * dk)):
        raise KernelError("gla: z must be fp32 [M, heads * dk]")
    _f32vec(head_decay, heads, "gla")
    _f32vec(z_bias, heads * dk, "gla")
    stride = _state_rows(state, "gla")
    if stride < heads * dk * dvx:
        raise KernelError("gla: state row too short")
    o = torch.empty((M, heads * dvx), dtype=torch.float32, device=q.device)
    lib = _lib("recurrent")
    longest = _max_q_len(ctx)
    n_chunks, scratch = 1, None
    if v.dtype == torch.bfloat16 and longest > GLA_CHUNK:
        # long portions: chunks side by side, two launches (the float32 path keeps the plain walk, whose
        # sums do not depend on where a portion starts)
        global launch_count
        n_chunks = -(-longest // GLA_CHUNK)
        scratch = torch.empty(lib.mi_gla_chunked_scratch(ctx.n_requests, n_chunks, heads, dk, dvx), dtype=torch.float32,
                              device=q.device)
        launch_count += 1
    rc = lib.mi_gla_scan(_ptr(q), _ptr(k), q.stride(0), _code(q.dtype), _ptr(v), v.stride(0), _ptr(z),
                         z.stride(0) if z is not None else 0,
                         _ptr(z_bias), 1.0 / float(tau),
                         float(q_scale), _ptr(state), stride, _ptr(ctx.q_start), _ptr(ctx.q_len),
                         _ptr(ctx.state_slot), _ptr(o), o.stride(0), ctx.n_requests, heads, dk, dvx, _ptr(scratch),
                         n_chunks, GLA_CHUNK, _ptr(head_decay), _ptr(tok_gates), 1 if extra_col else 0,
                         _code(v.dtype), _stream())
    _finish(lib, rc, "gla")
    return o


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, dt_bias: torch.Tensor,
               a_log: torch.Tensor, b: torch.Tensor, q_scale: float, unit_eps: float, heads: int, kv_heads: int,
               dk: int, dv: int, state: torch.Tensor, state_offset: int, ctx, *, conv_in: torch.Tensor | None = None,
               taps: int = 1) -> torch.Tensor:
    """The gated delta rule over each request's portion, from and into ``S [heads, dk, dv]`` at
    ``state_offset`` of its state row: ``S <- diag(g) S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``,
    ``o = S^T q`` with ``q`` and ``k`` (``kv_heads`` heads of ``dk``, shared by ``heads / kv_heads`` heads
    each) made unit vectors first (``x / sqrt(sum x^2 + unit_eps)``; ``q`` also times ``q_scale``),
    ``g = exp(-exp(a_log) * softplus(z + dt_bias))`` per head and key channel (``z`` fp32 ``[M, heads *
    dk]``) and ``beta = sigmoid(b)`` (``[M, heads]``).  q, k, v: column ranges of one packed tensor.
    ``conv_in`` (``[M, C]``) with ``taps``: the inputs of the short convolution that produced q, k and
    v; the head of the state row (``[taps - 1, C]``) is moved on to this portion's last inputs.
    Returns fp32 ``o [M, heads * dv]``."""
    _cuda(q, k, v, z, dt_bias, a_log, b, state, conv_in)
    for t in (q, k, v, z, b):
        _cols(t, "delta")
    M = q.shape[0]
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or not (q.dtype == k.dtype == v.dtype == b.dtype):
        raise KernelError("delta: q, k and v must be column ranges of one packed tensor")
    if q.shape[1] != kv_heads * dk or k.shape[1] != kv_heads * dk or v.shape[1] != heads * dv or b.shape != (M, heads):
        raise KernelError("delta: q, k must be [M, kv_heads * dk], v [M, heads * dv] and b [M, heads]")
    if z.dtype != torch.float32 or z.shape != (M, heads * dk):
        raise KernelError("delta: z must be fp32 [M, heads * dk]")
    _f32vec(dt_bias, heads * dk, "delta")
    _f32vec(a_log, heads, "delta")
    stride = _state_rows(state, "delta")
    C = 0
    if conv_in is not None:
        _cols(conv_in, "delta")
        C = conv_in.shape[1]
        if conv_in.dtype != q.dtype or conv_in.shape[0] != M or state_offset < (taps - 1) * C:
            raise KernelError("delta: the convolution's inputs do not fit the state row")
    if stride < state_offset + heads * dk * dv:
        raise KernelError("delta: state row too short")
    o = torch.empty((M, heads * dv), dtype=torch.float32, device=q.device)
    lib = _lib("recurrent")
    rc = lib.mi_delta_scan(_ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(z), z.stride(0), _ptr(dt_bias), _ptr(a_log),
                           _ptr(b), b.stride(0), float(q_scale), float(unit_eps), _ptr(state), stride,
                           int(state_offset), _ptr(ctx.q_start), _ptr(ctx.q_len), _ptr(ctx.state_slot), _ptr(o),
                           o.stride(0), ctx.n_requests, heads, kv_heads, dk, dv, _ptr(conv_in),
                           conv_in.stride(0) if conv_in is not None else 0, C, int(taps) if conv_in is not None else 1,
                           _code(q.dtype), _stream())
    _finish(lib, rc, "delta")
    return o


def headnorm_gate(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor | None, out: torch.Tensor, heads: int,
                  dv: int, eps: float, act: str | None, scale: float = 1.0, *, tok_gates: torch.Tensor | None = None,
                  den_eps: float = 0.0) -> None:
    """``out = o / sqrt(mean_head(o^2) + eps) * weight * act(gate) * scale`` per head of ``dv``
    (``o`` fp32 ``[M, heads * dv]``, ``weight`` fp32 ``[dv]``, shared by the heads, or ``[heads * dv]``, ``gate``
    and ``out`` in the compute dtype).  With ``tok_gates`` (fp32 ``[M, heads, 3]``) a head of ``o`` has
    ``dv + 1`` columns, the last one a normaliser ``n``, and the head is divided by
    ``max(|n|, exp(-m)) + den_eps`` first, ``m`` the third number of the token's and head's gates."""
    _cuda(o, weight, gate, out, tok_gates)
    _cols(o, "headnorm_gate")
    _cols(out, "headnorm_gate")
    dvx = dv + (1 if tok_gates is not None else 0)
    if o.dtype != torch.float32 or o.shape[1] != heads * dvx or out.shape != (o.shape[0], heads * dv):
        raise KernelError("headnorm_gate: o must be fp32 [M, heads * dv] and out shaped like it")
    if tok_gates is not None and (tok_gates.dtype != torch.float32 or tok_gates.shape != (o.shape[0], heads, 3)
                                  or not tok_gates.is_contiguous()):
        raise KernelError("headnorm_gate: tok_gates must be contiguous fp32 [M, heads, 3]")
    per_head = weight.numel() == heads * dv and heads > 1
    _f32vec(weight, heads * dv if per_head else dv, "headnorm_gate")
    if gate is not None:
        _cols(gate, "headnorm_gate")
        if gate.shape != out.shape or gate.dtype != out.dtype:
            raise KernelError("headnorm_gate: the gate must match out")
    lib = _lib("recurrent")
    rc = lib.mi_headnorm_gate(_ptr(o), o.stride(0), _ptr(weight), _ptr(gate), gate.stride(0) if gate is not None else 0,
                              _ptr(out), out.stride(0), o.shape[0], heads, dv, float(eps),
                              _ACT[act if gate is not None else None], float(scale), dv if per_head else 0,
                              _ptr(tok_gates), float(den_eps), _code(out.dtype), _stream())
    _finish(lib, rc, "headnorm_gate")


def mlstm_gates(z: torch.Tensor, bias_i: torch.Tensor | None, bias_f: torch.Tensor | None, cap: float, heads: int,
                state: torch.Tensor, m_offset: int, ctx) -> torch.Tensor:
    """The scalar gates of a matrix memory with a running maximum ``m`` (per request and head at
    ``m_offset`` of its state row, updated): from the pre-activations ``z`` (fp32 ``[M, 2 heads]``: input
    gates, then forget gates), ``i = cap tanh((z_i + b_i) / cap)``, ``f = logsigmoid(cap tanh((z_f + b_f) /
    cap))``, ``m' = max(f + m, i)`` token by token.  Returns fp32 ``[M, heads, 3]``: the state's decay
    ``exp(f + m - m')``, the input's factor ``exp(i - m')``, and ``m'``."""
    _cuda(z, bias_i, bias_f, state)
    _cols(z, "mlstm")
    M = z.shape[0]
    if z.dtype != torch.float32 or z.shape[1] != 2 * heads:
        raise KernelError("mlstm: the gates' pre-activations must be fp32 [M, 2 heads]")
    _f32vec(bias_i, heads, "mlstm")
    _f32vec(bias_f, heads, "mlstm")
    stride = _state_rows(state, "mlstm")
    gates = torch.empty((M, heads, 3), dtype=torch.float32, device=z.device)
    lib = _lib("recurrent")
    rc = lib.mi_mlstm_gates(_ptr(z), _ptr(z[:, heads:]), z.stride(0), _ptr(bias_i), _ptr(bias_f), float(cap),
                            _ptr(state), stride, int(m_offset), _ptr(ctx.q_start), _ptr(ctx.q_len),
                            _ptr(ctx.state_slot), _ptr(gates), ctx.n_requests, heads, _max_q_len(ctx), _stream())
    _finish(lib, rc, "mlstm")
    return gates


# --------------------------------------------------------------------------------------- routed experts


ROUTE_MODES = {"chosen": 0, "all": 1, "sigmoid": 2}


def moe_route(x: torch.Tensor, router: torch.Tensor, top: int, *, all_scores: bool = False, groups: int = 0,
              keep_groups: int = 0, scale: float = 1.0, scores: str | None = None,
              correction: torch.Tensor | None = None, group_top2: bool = False, experts: int | None = None,
              return_logits: bool = False):
    """fp32 router logits ``x router^T``; per token the ``top`` experts with the largest logits
    (int32 ``[M, top]``, largest first) and their weights (fp32): the softmax over those logits alone,
    or, with ``all_scores``, their scores under the softmax over all experts divided by the sum of
    these (+ 1e-20), times ``scale``.  ``groups`` > 1: the experts form that many equal groups of
    neighbours, a group counts as its best expert, and only the ``keep_groups`` best groups give experts.
    ``scores`` names the way outright: ``"chosen"``, ``"all"`` or ``"sigmoid"`` (scores are the logits'
    sigmoids; the choice adds ``correction`` (fp32 ``[experts]``) per expert; the weights are the chosen
    scores times ``scale``, with no division by their sum).  ``group_top2``: a group counts as the sum of its two best
    choice scores.  ``experts``: only the router's first ``experts`` rows are experts; the other rows ride
    along in the product and ``return_logits`` hands all logits back as a third result."""
    _cuda(x, router, correction)
    _cols(x, "moe")
    if router.dim() != 2 or router.shape[1] != x.shape[1] or router.dtype != x.dtype or not router.is_contiguous():
        raise KernelError("moe: the router must be a contiguous [experts, H] matrix in x's dtype")
    M, H = x.shape
    E = router.shape[0] if experts is None else int(experts)
    if not 0 < E <= router.shape[0]:
        raise KernelError(f"moe: {E} experts of a router with {router.shape[0]} rows")
    mode = ROUTE_MODES[scores] if scores is not None else (1 if all_scores else 0)
    _f32vec(correction, E, "moe (correction)")
    logits = linear(x, router, out_dtype=torch.float32)      # exact products, fp32 sums, for either dtype
    ids = torch.empty((M, top), dtype=torch.int32, device=x.device)
    weights = torch.empty((M, top), dtype=torch.float32, device=x.device)
    lib = _lib("moe")
    rc = lib.mi_moe_select(_ptr(logits), logits.stride(0), _ptr(ids), _ptr(weights), M, E, int(top),
                           mode, int(groups), int(keep_groups), float(scale), _ptr(correction),
                           1 if group_top2 else 0, _stream())
    _finish(lib, rc, "moe_select")
    if return_logits:
        return ids, weights, logits
    return ids, weights


MOE_FEW_ROWS_PER_EXPERT = 8     # up to this many rows per expert on average: the streaming products
USE_GROUPED_MM = os.environ.get("MINI_INFER_GROUPED_MM", "1") != "0"


def moe_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                w_down: torch.Tensor, limit: float, alpha: float, shared: torch.Tensor | None = None,
                up_offset: float = 1.0, shared_gate: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = sum_k weights[t, k] * expert_{ids[t, k]}(x[t]) (+ shared[t])`` with
    ``expert(x) = W_down glu(W_gate x, W_up x)``, ``glu(g, u) = g' sigmoid(alpha g') (u' + up_offset)``,
    ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)`` (an infinite ``limit`` with ``alpha`` 1 and
    ``up_offset`` 0 is the plain ``silu(g) * u``).  Weights are stacked per expert:
    ``w_gate_up [E, 2 ff, H]`` (an expert's gate rows, then its up rows), ``w_down [E, H, ff]``.
    ``shared_gate`` (fp32, one number per token, any row stride): its sigmoid multiplies ``shared[t]``.
    Entries are sorted by expert on the device; nothing is read back.  Three routes: a step that
    brings an expert only a few rows streams the weights (bfloat16); large bfloat16 steps gather
    each expert's rows and use the library's grouped product (as the dense layers use the library's
    product for many rows); everything else walks 64-row tiles with this module's own kernels
    (tensor cores for bfloat16, CUDA cores with a fixed summation order for float32)."""
    global launch_count
    _cuda(x, ids, weights, w_gate_up, w_down, shared)
    _cols(x, "moe")
    M, H = x.shape
    E, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    top = ids.shape[1]
    for w, shape in ((w_gate_up, (E, 2 * ff, H)), (w_down, (E, H, ff))):
        if tuple(w.shape) != shape or w.dtype != x.dtype or not w.is_contiguous():
            raise KernelError("moe: expert weights must be contiguous [E, 2 ff, H] and [E, H, ff] in x's dtype")
    if ids.dtype != torch.int32 or weights.dtype != torch.float32 or ids.shape != weights.shape or ids.shape[0] != M \
            or not ids.is_contiguous() or not weights.is_contiguous():
        raise KernelError("moe: ids int32 [M, top] and weights fp32 [M, top]")
    if shared is not None:
        _cols(shared, "moe")
        if shared.shape != (M, H) or shared.dtype != x.dtype:
            raise KernelError("moe: the shared expert's output must be [M, H] in x's dtype")
    n = M * top
    lib = _lib("moe")
    pieces = (x.dtype == torch.bfloat16 and H % 8 == 0 and ff % 8 == 0 and x.stride(0) % 8 == 0
              and x.data_ptr() % 16 == 0)          # rows are whole 16-byte pieces
    few = pieces and n <= MOE_FEW_ROWS_PER_EXPERT * E
    grouped = pieces and not few and USE_GROUPED_MM and hasattr(torch, "_grouped_mm")
    tile = lib.mi_moe_tile_rows(1 if few else 0)
    dev = x.device
    perm = torch.empty(n, dtype=torch.int32, device=dev)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    plan = torch.empty(2 + E + 3 * (-(-n // tile) + E), dtype=torch.int32, device=dev)
    rc = lib.mi_moe_plan(_ptr(ids), n, E, _ptr(perm), _ptr(inv), _ptr(plan), tile, _stream())
    _finish(lib, rc, "moe_plan")
    if grouped:
        xs = torch.empty((n, H), dtype=x.dtype, device=dev)
        rc = lib.mi_moe_gather(_ptr(x), x.stride(0), _ptr(perm), top, _ptr(xs), n, H, _code(x.dtype), _stream())
        _finish(lib, rc, "moe_gather")
        ends = plan[2:2 + E]                       # where each expert's rows end
        act = clamped_glu(torch._grouped_mm(xs, w_gate_up.transpose(-2, -1), offs=ends), limit, alpha, up_offset)
        y = torch._grouped_mm(act, w_down.transpose(-2, -1), offs=ends)
        launch_count += 2
    else:
        act = torch.empty((n, ff), dtype=x.dtype, device=dev)
        rc = lib.mi_moe_gate_up(_ptr(x), x.stride(0), _ptr(w_gate_up), _ptr(w_gate_up[:, ff:]), 2 * ff * H, _ptr(perm),
                                top, _ptr(plan), E, _ptr(act), n, ff, H, float(limit), float(alpha), float(up_offset),
                                tile, _code(x.dtype), _stream())
        _finish(lib, rc, "moe_gate_up")
        y = torch.empty((n, H), dtype=torch.float32, device=dev)
        rc = lib.mi_moe_down(_ptr(act), _ptr(w_down), H * ff, _ptr(plan), E, _ptr(y), n, H, ff, tile, _code(x.dtype),
                             _stream())
        _finish(lib, rc, "moe_down")
    out = torch.empty((M, H), dtype=x.dtype, device=dev)
    if shared_gate is not None and (shared is None or shared_gate.dtype != torch.float32 or shared_gate.shape[0] != M
                                    or shared_gate.dim() > 2 or (shared_gate.dim() == 2 and shared_gate.shape[1] != 1)):
        raise KernelError("moe: the shared expert's gate must be fp32, one number per token, beside a shared expert")
    rc = lib.mi_moe_combine(_ptr(y), _code(y.dtype), _ptr(inv), _ptr(weights), _ptr(shared),
                            shared.stride(0) if shared is not None else 0, _ptr(out), M, H, top, _ptr(shared_gate),
                            shared_gate.stride(0) if shared_gate is not None else 0, _code(x.dtype), _stream())
    _finish(lib, rc, "moe_combine")
    return out


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float, up_offset: float = 1.0) -> torch.Tensor:
    """``glu(gate_up[:, :I], gate_up[:, I:])`` of ``moe_experts`` for a dense expert."""
    _cuda(gate_up)
    _cols(gate_up, "clamped_glu")
    M, I2 = gate_up.shape
    out = torch.empty((M, I2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    lib = _lib("moe")
    rc = lib.mi_clamped_glu(_ptr(gate_up), gate_up.stride(0), _ptr(out), M, I2 // 2, float(limit), float(alpha),
                            float(up_offset), _code(gate_up.dtype), _stream())
    _finish(lib, rc, "clamped_glu")
    return out


def block_diagonal_gates(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``gates[b] = u[:, b * bw:(b + 1) * bw] @ w[b]^T`` in fp32 for ``w [blocks, n, bw]``: float32
    through the true-fp32 product block by block, bfloat16 through the library's batched product
    with fp32 output.  Returns fp32 ``[blocks, M, n]``."""
    global launch_count
    _cuda(u, w)
    _cols(u, "block_diagonal")
    blocks, n, bw = w.shape
    M = u.shape[0]
    if u.shape[1] != blocks * bw or w.dtype != u.dtype or not w.is_contiguous():
        raise KernelError("block_diagonal: u must be [M, blocks * bw] and w contiguous [blocks, n, bw] in u's dtype")
    if u.dtype == torch.float32:
        out = torch.empty((blocks, M, n), dtype=torch.float32, device=u.device)
        for b in range(blocks):
            gemm_f32(u[:, b * bw:(b + 1) * bw], w[b], out[b])
        return out
    launch_count += 1
    ub = u.unflatten(1, (blocks, bw)).transpose(0, 1)           # [blocks, M, bw], a view
    return torch.bmm(ub, w.transpose(1, 2), out_dtype=torch.float32)


# --------------------------------------------------------------------------------------- streams with several addends


def embedding_pair_hash(table: torch.Tensor, pair_table: torch.Tensor, ctx, last_token: torch.Tensor, buckets: int,
                        mul_prev: int, mul_cur: int) -> torch.Tensor:
    """``float(table[id]) + float(pair_table[row])`` as the fp32 residual stream ``[M, H]``, ``row``
    a hash of the token and the one before it, ``(prev * mul_prev + id * mul_cur) mod buckets``,
    and row ``buckets`` for a sequence's first token.  ``last_token`` (int32 ``[request slots]``)
    holds, per request, the last token of its previous portion; the kernel reads it for a
    portion's first token and replaces it by the portion's last one."""
    ids = ctx.token_ids
    _cuda(table, pair_table, ids, last_token)
    if table.dim() != 2 or not table.is_contiguous() or pair_table.dim() != 2 or not pair_table.is_contiguous():
        raise KernelError("embedding: tables must be contiguous [rows, H] matrices")
    V, H = table.shape
    if pair_table.shape != (buckets + 1, H) or pair_table.dtype != table.dtype:
        raise KernelError(f"embedding: the pair table must be [{buckets + 1}, {H}] in the token table's dtype")
    if last_token.dtype != torch.int32 or not last_token.is_contiguous():
        raise KernelError("embedding: the last-token state must be contiguous int32")
    M = ids.shape[0]
    out = torch.empty((M, H), dtype=torch.float32, device=table.device)
    lib = _lib("stream")
    rc = lib.mi_embedding_pair_hash(_ptr(table), _ptr(pair_table), _ptr(ids), _ptr(ctx.positions), _ptr(ctx.q_start),
                                    _ptr(ctx.q_len), _ptr(ctx.state_slot), _ptr(last_token), int(ctx.n_requests),
                                    _ptr(out), M, H, V, int(buckets), int(mul_prev), int(mul_cur), _code(table.dtype),
                                    _stream())
    _finish(lib, rc, "embedding")
    return out


def embedding_rmsnorm(table: torch.Tensor, ids: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * gain`` with ``x = float(table[ids])`` as the fp32 residual stream
    ``[M, H]`` (``gain`` fp32 ``[H]``): an embedding with a norm of its own."""
    _cuda(table, ids, gain)
    if ids.dtype != torch.int32 or ids.dim() != 1 or not ids.is_contiguous():
        raise KernelError("embedding: ids must be a contiguous int32 vector")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embedding: table must be a contiguous [V, H] matrix")
    V, H = table.shape
    _f32vec(gain, H, "embedding")
    out = torch.empty((ids.shape[0], H), dtype=torch.float32, device=table.device)
    lib = _lib("stream")
    rc = lib.mi_embedding_rmsnorm(_ptr(table), _ptr(ids), _ptr(gain), _ptr(out), ids.shape[0], H, V, float(eps),
                                  _code(table.dtype), _stream())
    _finish(lib, rc, "embedding")
    return out


def add_rmsnorm_multi(stream: torch.Tensor | None, adds, gain: torch.Tensor, eps: float, dtype: torch.dtype, *,
                      add32: torch.Tensor | None = None, row_add: torch.Tensor | None = None,
                      rows: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
    """RMS norm of ``r = stream + sum(adds) + add32 + row_add`` in fp32: ``stream`` the fp32 stream
    ``[M, H]``, ``adds`` up to two ``[M, H]`` tensors of ``dtype`` (branch outputs), ``add32`` an fp32
    ``[M, H]`` tensor, ``row_add`` an fp32 ``[H]`` vector added to every row; each may be missing.
    Returns ``(gain * r * rsqrt(mean(r^2) + eps)`` in ``dtype``, the new fp32 stream ``r``)``; with
    ``rows`` (int32) only those rows are normalised and no stream is returned."""
    adds = [a for a in adds if a is not None]
    if len(adds) > 2:
        raise KernelError("rmsnorm: at most two addends in the compute dtype")
    _cuda(stream, add32, row_add, rows, gain, *adds)
    shape = next((tuple(t.shape) for t in (stream, add32, *adds) if t is not None), None)
    if shape is None or len(shape) != 2:
        raise KernelError("rmsnorm: nothing to normalise")
    H = shape[1]
    for t, dt, what in ((stream, torch.float32, "the stream"), (add32, torch.float32, "the fp32 addend"),
                        *((a, dtype, "an addend") for a in adds)):
        if t is not None and (t.dtype != dt or tuple(t.shape) != shape or not t.is_contiguous()):
            raise KernelError(f"rmsnorm: {what} must be contiguous {dt} {shape}")
    if gain.dtype != torch.float32 or gain.shape != (H,) or not gain.is_contiguous():
        raise KernelError(f"rmsnorm: the gain must be fp32 [{H}]")
    if row_add is not None and (row_add.dtype != torch.float32 or row_add.shape != (H,) or not row_add.is_contiguous()):
        raise KernelError(f"rmsnorm: the row addend must be fp32 [{H}]")
    if rows is not None and (rows.dtype != torch.int32 or rows.dim() != 1 or not rows.is_contiguous()):
        raise KernelError("rmsnorm: rows must be a contiguous int32 vector")
    M = shape[0] if rows is None else rows.shape[0]
    out = torch.empty((M, H), dtype=dtype, device=gain.device)
    new_stream = None if rows is not None else torch.empty((M, H), dtype=torch.float32, device=gain.device)
    lib = _lib("stream")
    rc = lib.mi_add_rmsnorm_multi(_ptr(stream), _ptr(adds[0] if adds else None), _ptr(adds[1] if len(adds) > 1 else None),
                                  _ptr(add32), _ptr(row_add), _ptr(new_stream), _ptr(rows), _ptr(gain), _ptr(out),
                                  M, H, float(eps), _code(dtype), _stream())
    _finish(lib, rc, "rmsnorm")
    return out, new_stream


def glu_mul_pairs(gate_up: torch.Tensor, act: str, out: torch.Tensor | None = None) -> torch.Tensor:
    """``act(gate) * up`` with fp32 arithmetic for ``gate_up [M, 2 I]`` whose columns alternate
    gate, up; ``act`` is ``"silu"`` or ``"gelu_tanh"``."""
    _cuda(gate_up, out)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("glu_mul: input must be contiguous [M, 2 I]")
    M, I2 = gate_up.shape
    I = I2 // 2
    if out is None:
        out = torch.empty((M, I), dtype=gate_up.dtype, device=gate_up.device)
    elif out.shape != (M, I) or out.dtype != gate_up.dtype or not out.is_contiguous():
        raise KernelError("glu_mul: bad output tensor")
    lib = _lib("stream")
    rc = lib.mi_glu_mul_pairs(_ptr(gate_up), _ptr(out), M, I, GLU_ACT[act], _code(gate_up.dtype), _stream())
    _finish(lib, rc, "glu_mul")
    return out


def scaled_norm_add(stream: torch.Tensor, branch: torch.Tensor | None, gain: torch.Tensor | None, eps: float,
                    mult: float, dtype: torch.dtype, copy: bool = True) -> torch.Tensor | None:
    """A branch whose norm stands behind it: ``stream += mult * y * rsqrt(mean(y^2) + eps) * gain`` in place
    (``stream`` fp32 ``[M, H]``, ``y`` the branch's rows in ``dtype``, ``gain`` fp32 ``[H]``).  Returns the
    updated stream's copy in ``dtype`` (what the next branch's products read), or, for float32, the
    stream itself.  Without a branch only the copy is made."""
    _cuda(stream, branch, gain)
    if stream.dtype != torch.float32 or stream.dim() != 2 or not stream.is_contiguous():
        raise KernelError("norm_add: the stream must be contiguous fp32 [M, H]")
    M, H = stream.shape
    if branch is not None:
        _cols(branch, "norm_add")
        if branch.shape != (M, H) or branch.dtype != dtype:
            raise KernelError("norm_add: the branch must be [M, H] in the compute dtype")
        _f32vec(gain, H, "norm_add")
    out = None
    if copy and dtype != torch.float32:
        out = torch.empty((M, H), dtype=dtype, device=stream.device)
    if branch is None and out is None:
        return stream
    lib = _lib("stream")
    rc = lib.mi_scaled_norm_add(_ptr(stream), _ptr(branch), branch.stride(0) if branch is not None else 0, _ptr(gain),
                                float(eps), float(mult), _ptr(out), M, H, _code(dtype), _stream())
    _finish(lib, rc, "norm_add")
    return stream if dtype == torch.float32 else out


def token_gate(z: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, col0: int) -> torch.Tensor:
    """``gelu_tanh(z[t, c]) * table[ids[t], col0 + c]`` for ``z [M, n]`` (fp32 or the table's dtype), in the
    table's dtype."""
    _cuda(z, table, ids)
    _cols(z, "token_gate")
    if table.dim() != 2 or not table.is_contiguous() or ids.dtype != torch.int32 or ids.shape != (z.shape[0],):
        raise KernelError("token_gate: a contiguous table [V, columns] and int32 ids [M]")
    M, n = z.shape
    out = torch.empty((M, n), dtype=table.dtype, device=z.device)
    lib = _lib("stream")
    rc = lib.mi_token_gate(_ptr(z), z.stride(0), _code(z.dtype), _ptr(table), table.stride(0), _ptr(ids),
                           table.shape[0], int(col0), _ptr(out), M, n, _code(table.dtype), _stream())
    _finish(lib, rc, "token_gate")
    return out


def scale_(x: torch.Tensor, s: float) -> torch.Tensor:
    """``x *= s`` in place (contiguous fp32)."""
    _cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale: a contiguous fp32 tensor")
    lib = _lib("stream")
    rc = lib.mi_scale_f32(_ptr(x), x.numel(), float(s), _stream())
    _finish(lib, rc, "scale")
    return x


# --------------------------------------------------------------------------------------- between projection and attention


def _opt_f32(t: torch.Tensor | None, n: int, what: str) -> None:
    if t is not None and (not t.is_cuda or t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()):
        raise KernelError(f"{what}: needs a contiguous fp32 CUDA tensor of {n} elements")


def qk_bias_norm_store(packed: torch.Tensor, q_off: int, k_off: int, v_off: int, nq: int, nkv: int, d: int, dv: int, *,
                       q_bias: torch.Tensor | None, k_bias: torch.Tensor | None, q_gain: torch.Tensor | None,
                       k_gain: torch.Tensor | None, eps: float, values_are_keys: bool,
                       slots: torch.Tensor | None = None, kcache: torch.Tensor | None = None,
                       vcache: torch.Tensor | None = None, qk_out: torch.Tensor | None = None) -> None:
    """In the packed projection ``[M, stride]`` (q at columns ``q_off``, ``nq`` heads of ``d``; k at
    ``k_off``, ``nkv`` heads of ``d``): add the biases (fp32 ``[heads * d]``), then give every head an
    RMS norm with the gain shared by the heads (fp32 ``[d]``; None: no norm); q and k are written back
    and k is stored at ``slots`` of ``kcache``.  The values stored in ``vcache`` are the keys with
    their bias before the norm (``values_are_keys``), or the columns at ``v_off`` (``nkv`` heads of ``dv``)."""
    _cuda(packed, slots, kcache, vcache)
    _cols(packed, "qk_prepare")
    M, width = packed.shape
    if q_off + nq * d > width or k_off + nkv * d > width or (not values_are_keys and v_off + nkv * dv > width):
        raise KernelError("qk_prepare: a column range lies outside the packed projection")
    _opt_f32(q_bias, nq * d, "qk_prepare (q bias)")
    _opt_f32(k_bias, nkv * d, "qk_prepare (k bias)")
    _opt_f32(q_gain, d, "qk_prepare (q gain)")
    _opt_f32(k_gain, d, "qk_prepare (k gain)")
    writes = kcache is not None
    page_size = 0
    if writes:
        if slots is None or slots.dtype != torch.int32 or slots.shape != (M,):
            raise KernelError("qk_prepare: slots must be int32 [M]")
        for c, size in ((kcache, d), (vcache, dv)):
            if (c is None or c.dtype != packed.dtype or c.dim() != 4 or c.shape[1] != nkv or c.shape[3] != size
                    or not c.is_contiguous()):
                raise KernelError("qk_prepare: caches must be contiguous [pages, nkv, page_size, size] in the packed dtype")
        page_size = int(kcache.shape[2])
    lib = _lib("qk_prepare")
    rc = lib.mi_qk_bias_norm_store(_ptr(packed), packed.stride(0), q_off, k_off, v_off, M, nq, nkv, d, dv,
                                   _ptr(q_bias), _ptr(k_bias), _ptr(q_gain), _ptr(k_gain), float(eps),
                                   1 if values_are_keys else 0, _ptr(slots), _ptr(kcache), _ptr(vcache), page_size,
                                   1 if writes else 0, _code(packed.dtype), _stream())
    _finish(lib, rc, "qk_prepare")


def qk_norm_rope_store(packed: torch.Tensor, q_off: int, k_off: int, v_off: int | None, nq: int, nkv: int, d: int,
                       dv: int, *, q_gain: torch.Tensor | None = None, k_gain: torch.Tensor | None = None,
                       eps: float = 0.0, rot: int = 0, positions: torch.Tensor | None = None,
                       freq: torch.Tensor | None = None, q_scale: float = 1.0, k_scale: float = 1.0,
                       v_other: torch.Tensor | None = None, blend: torch.Tensor | None = None,
                       slots: torch.Tensor | None = None, kcache: torch.Tensor | None = None,
                       vcache: torch.Tensor | None = None, qk_out: torch.Tensor | None = None,
                       bias: torch.Tensor | None = None) -> None:
    """In the packed projection ``[M, stride]`` (q at columns ``q_off``, ``nq`` heads of ``d``; k at
    ``k_off``, ``nkv`` heads of ``d``; v at ``v_off``, ``nkv`` heads of ``dv``, or ``v_off`` None: no values
    here): q and k get an RMS norm over the head with the gain shared by the heads (fp32 ``[d]``; None:
    no norm), then the rotation of the half layout on their first ``rot`` dimensions (``freq`` float64
    ``[rot / 2]``; the angle in double precision), then the factors ``q_scale`` / ``k_scale``; both are
    written back.  With ``v_other`` (``[M, nkv * dv]``) and ``blend`` (fp32, one element) the values
    become ``(1 - blend) v + blend v_other`` and are written back too.  With caches, k and v are stored
    at ``slots``.  With ``qk_out`` (fp32 ``[M, (nq + nkv) * d]``, queries first) the finished q and k go there
    unrounded and their packed columns stay as they were: for a recurrence that takes them in fp32.
    ``bias`` (fp32, one number per packed column up to the last of q, k and v) is added to q, k and v first."""
    _cuda(packed, q_gain, k_gain, positions, freq, v_other, blend, slots, kcache, vcache, qk_out, bias)
    _cols(packed, "qk_prepare")
    M, width = packed.shape
    has_v = v_off is not None
    if q_off + nq * d > width or k_off + nkv * d > width or (has_v and v_off + nkv * dv > width):
        raise KernelError("qk_prepare: a column range lies outside the packed projection")
    _opt_f32(q_gain, d, "qk_prepare (q gain)")
    _opt_f32(k_gain, d, "qk_prepare (k gain)")
    if rot:
        if positions is None or positions.dtype != torch.int32 or positions.shape != (M,):
            raise KernelError("qk_prepare: positions must be int32 [M]")
        if freq is None or freq.dtype != torch.float64 or freq.shape != (rot // 2,) or not freq.is_contiguous():
            raise KernelError("qk_prepare: freq must be float64 [rot / 2]")
    if v_other is not None:
        _cols(v_other, "qk_prepare")
        if not has_v or v_other.shape != (M, nkv * dv) or v_other.dtype != packed.dtype:
            raise KernelError("qk_prepare: the other values must be [M, nkv * dv] in the packed dtype")
        _opt_f32(blend, 1, "qk_prepare (blend)")
        if blend is None:
            raise KernelError("qk_prepare: blending values needs the blend's weight")
    writes = kcache is not None
    page_size = 0
    if writes:
        if slots is None or slots.dtype != torch.int32 or slots.shape != (M,):
            raise KernelError("qk_prepare: slots must be int32 [M]")
        for c, size in ((kcache, d),) + (((vcache, dv),) if has_v else ()):
            if (c is None or c.dtype != packed.dtype or c.dim() != 4 or c.shape[1] != nkv or c.shape[3] != size
                    or not c.is_contiguous()):
                raise KernelError("qk_prepare: caches must be contiguous [pages, nkv, page_size, size] in the packed dtype")
        page_size = int(kcache.shape[2])
    if qk_out is not None and (qk_out.dtype != torch.float32 or qk_out.shape != (M, (nq + nkv) * d)
                               or qk_out.stride(1) != 1):
        raise KernelError("qk_prepare: qk_out must be fp32 [M, (nq + nkv) * d]")
    if bias is not None:
        need = max(q_off + nq * d, k_off + nkv * d, (v_off + nkv * dv) if has_v else 0)
        if bias.dtype != torch.float32 or bias.dim() != 1 or bias.shape[0] < need or not bias.is_contiguous():
            raise KernelError(f"qk_prepare: the bias must be fp32 with at least {need} numbers")
    lib = _lib("qk_prepare")
    rc = lib.mi_qk_norm_rope_store(_ptr(packed), packed.stride(0), q_off, k_off, v_off if has_v else -1, M, nq, nkv, d,
                                   dv, _ptr(q_gain), _ptr(k_gain), float(eps), int(rot), _ptr(positions), _ptr(freq),
                                   float(q_scale), float(k_scale), _ptr(v_other),
                                   v_other.stride(0) if v_other is not None else 0, _ptr(blend), _ptr(slots),
                                   _ptr(kcache), _ptr(vcache if has_v else None), page_size, 1 if writes else 0,
                                   _ptr(qk_out), qk_out.stride(0) if qk_out is not None else 0, _ptr(bias),
                                   _code(packed.dtype), _stream())
    _finish(lib, rc, "qk_prepare")


def latent_prepare(packed: torch.Tensor, q_off: int, nq: int, q_head: int, q_rot_off: int, c_off: int, rank: int,
                   rot_dim: int, rot: int, *, positions: torch.Tensor, freq: torch.Tensor, c_gain: torch.Tensor,
                   eps: float, qfull: torch.Tensor, slots: torch.Tensor | None = None,
                   kcache: torch.Tensor | None = None) -> None:
    """From the packed projection ``[M, stride]`` of a latent attention: the latent (``rank`` columns
    at ``c_off``) gets an RMS norm with ``c_gain``; the key part behind it (``rot_dim`` columns) and
    every query head's part at ``q_rot_off`` within its ``q_head`` columns are rotated by the
    position (half layout over the first ``rot`` dimensions, ``freq`` float64 ``[rot / 2]``).  The
    cache row ``[latent, rotated key part]`` is stored at ``slots`` of ``kcache``
    ``[pages, 1, page_size, rank + rot_dim]``; the rotated query parts go behind the first ``rank``
    columns of every head of ``qfull [M, nq, rank + rot_dim]``."""
    _cuda(packed, positions, freq, c_gain, qfull, slots, kcache)
    _cols(packed, "latent_prepare")
    M, width = packed.shape
    if q_off + nq * q_head > width or c_off + rank + rot_dim > width:
        raise KernelError("latent_prepare: a column range lies outside the packed projection")
    if positions.dtype != torch.int32 or positions.shape != (M,):
        raise KernelError("latent_prepare: positions must be int32 [M]")
    if rot and (freq.dtype != torch.float64 or freq.shape != (rot // 2,) or not freq.is_contiguous()):
        raise KernelError("latent_prepare: freq must be float64 [rot / 2]")
    _opt_f32(c_gain, rank, "latent_prepare (gain)")
    dk = rank + rot_dim
    if qfull.shape != (M, nq, dk) or qfull.dtype != packed.dtype or not qfull.is_contiguous():
        raise KernelError(f"latent_prepare: qfull must be contiguous [{M}, {nq}, {dk}] in the packed dtype")
    writes = kcache is not None
    page_size = 0
    if writes:
        if slots is None or slots.dtype != torch.int32 or slots.shape != (M,):
            raise KernelError("latent_prepare: slots must be int32 [M]")
        if (kcache.dtype != packed.dtype or kcache.dim() != 4 or kcache.shape[1] != 1 or kcache.shape[3] != dk
                or not kcache.is_contiguous()):
            raise KernelError(f"latent_prepare: the cache must be contiguous [pages, 1, page_size, {dk}] in the packed dtype")
        page_size = int(kcache.shape[2])
    lib = _lib("qk_prepare")
    rc = lib.mi_latent_prepare(_ptr(packed), packed.stride(0), q_off, M, nq, q_head, q_rot_off, c_off, rank, rot_dim,
                               int(rot), _ptr(positions), _ptr(freq), _ptr(c_gain), float(eps), _ptr(qfull),
                               nq * dk, dk, _ptr(slots), _ptr(kcache), page_size, 1 if writes else 0,
                               _code(packed.dtype), _stream())
    _finish(lib, rc, "latent_prepare")


USE_ROWS_ATTENTION = os.environ.get("MINI_INFER_ROWS_ATTENTION", "1") != "0"
ROWS_ATTENTION_ROWS = (16, 32, 64)   # query rows per block of attention_rows.cu: steps of single tokens; prompt portions


def rows_attention_tile_tokens(group: int, rows: int = 16) -> int:
    """Tokens per tile of the tensor-core kernel of ``attention_ext`` for ``group`` query heads per
    key/value head and blocks of ``rows`` rows of (token, head in group), or 0 where it does not take
    the group size.  The same rule as the library's ``mi_attention_rows_tile_tokens``."""
    if group <= 0 or rows not in ROWS_ATTENTION_ROWS:
        return 0
    if group >= rows:
        return 1 if group % rows == 0 else 0
    return rows // group if rows % group == 0 else 0


def rows_attention_tile_sizes(nq: int, nkv: int, d: int, dv: int, values_in_keys: bool) -> frozenset[int]:
    """The query tile sizes a step must plan for a mixer that wants ``attention_ext`` to use the
    tensor-core kernel (empty where the kernel does not take the sizes)."""
    if not rows_attention_supported(nq, nkv, d, dv, values_in_keys):
        return frozenset()
    return frozenset(t for t in (rows_attention_tile_tokens(nq // nkv, r) for r in ROWS_ATTENTION_ROWS) if t)


def rows_attention_supported(nq: int, nkv: int, d: int, dv: int, values_in_keys: bool) -> bool:
    """Whether attention_rows.cu takes these sizes (the library's ``mi_attention_rows_supported``, made
    here so that a model it does not take never compiles it): keys a multiple of 16 up to 1024,
    values a multiple of 32 up to 512, a group size that divides 16 or is a multiple of it."""
    if not USE_ROWS_ATTENTION or nq <= 0 or nkv <= 0 or nq % nkv or not rows_attention_tile_tokens(nq // nkv, 16):
        return False
    if d < 16 or d % 16 or d > 1024 or dv < 32 or dv % 32 or dv > 512:
        return False
    if values_in_keys and dv > d:
        return False
    return _rows_attention_smem(16, d, dv, values_in_keys) <= 227 * 1024


def _rows_attention_smem(rows: int, d: int, dv: int, values_in_keys: bool, stages: int = 1) -> int:
    chunk = 64 * (d + 8) + (0 if values_in_keys else 64 * (dv + 8))
    return (rows * (d + 8) + stages * chunk + rows * 72) * 2 + 32 * rows + stages * 512


def _rows_attention_plan(ctx, nq: int, nkv: int, d: int, dv: int, values_in_keys: bool, device) -> tuple[int, int, int, int]:
    """``(rows per block, tokens per tile, runs of keys per tile, buffers per chunk)`` for this step:
    steps of single tokens take 16 rows and cut every request's keys into runs, so that the blocks
    fill the GPU; prompt portions take 64 rows with two buffers for the chunk's rows (the next chunk
    is copied while this one is multiplied), else 64 rows with one buffer, else 32 rows with two, as
    the group size and shared memory allow."""
    group = nq // nkv
    if not getattr(ctx, "decode_only", False):
        # measured at 2048 tokens: two buffers gain 13 % at 64 rows; 32 rows with two buffers lose 30 % against 64
        # rows with one for rows of 576 (twice the traffic from the L2) and tie for rows of 160 and less
        for rows, stages in ((64, 2), (64, 1), (32, 2)):
            tt = rows_attention_tile_tokens(group, rows)
            if tt and tt in ctx.tiles and _rows_attention_smem(rows, d, dv, values_in_keys, stages) <= 227 * 1024:
                return rows, tt, 1, stages
        return 16, rows_attention_tile_tokens(group, 16), 1, 1
    tt = rows_attention_tile_tokens(group, 16)
    units = ctx.tiles[tt][2] * nkv * max(1, group // 16)
    chunks = max(1, -(-int(getattr(ctx, "max_kv_len", 0) or 64) // 64))
    splits = max(1, min(-(-4 * _sms(device) // units), chunks, 64))
    return 16, tt, splits, 1


def attention_ext(q: torch.Tensor, out: torch.Tensor, cache, ctx, nq: int, nkv: int, d: int, dv: int, scale: float, *,
                  window: int = 0, sinks: torch.Tensor | None = None, slopes: torch.Tensor | None = None,
                  values_in_keys: bool = False, chunk: int = 0) -> None:
    """``attention_kv`` with the extras of the CUDA-core kernel: ``sinks`` (fp32 ``[nq]``: a score per
    head that joins the softmax's denominator without a key or a value), ``slopes`` (fp32 ``[nq]``:
    the scaled score of a key ``dist`` positions back is lowered by ``slope * dist``) and
    ``values_in_keys`` (the cache layer has keys only; a key's value is the first ``dv`` numbers of its
    own row); ``chunk`` > 0: a query at position ``p`` sees only the keys of its own chunk of positions,
    ``j >= (p // chunk) * chunk``.  fp32 scores, weights and sums for float32 and bfloat16 alike.  bfloat16 prompt portions
    with keys and values of one size that attention_tc.cu takes run on tcgen05; other bfloat16 steps with sizes that
    attention_rows.cu takes (``rows_attention_supported``) and tiles planned for it runs on tensor
    cores (weights rounded to bfloat16 for the second product); everything else on CUDA cores."""
    global launch_count
    group = ctx.groups[cache.group]
    _cuda(q, out, cache.k, None if values_in_keys else cache.v, sinks, slopes)
    _cols(q, "attention")
    _cols(out, "attention")
    if q.shape[1] != nq * d or out.shape[1] != nq * dv or q.dtype != out.dtype:
        raise KernelError("attention: q must be [M, nq * d] and out [M, nq * dv] in one dtype")
    _opt_f32(sinks, nq, "attention (sinks)")
    _opt_f32(slopes, nq, "attention (slopes)")
    kc, vc = cache.k, (None if values_in_keys else cache.v)
    if kc.dtype != q.dtype or kc.dim() != 4 or kc.shape[1:] != (nkv, group.page_size, d) or not kc.is_contiguous():
        raise KernelError("attention: the key cache must be contiguous [pages, nkv, page_size, d] in q's dtype")
    if vc is not None and (vc.dtype != q.dtype or vc.dim() != 4 or vc.shape[1:] != (nkv, group.page_size, dv)
                           or not vc.is_contiguous()):
        raise KernelError("attention: the value cache must be contiguous [pages, nkv, page_size, dv] in q's dtype")
    bt = group.block_table
    # prompt portions of heads that the tcgen05 prefill kernel takes (keys and values of 64 or 128) go there
    if (q.dtype == torch.bfloat16 and not values_in_keys and d == dv and not getattr(ctx, "decode_only", False)
            and not chunk and USE_TC_PREFILL and scale > 0 and prefill_tc_supported(nq, nkv, d, group.page_size)
            and prefill_tc_tile_tokens(nq // nkv) in ctx.tiles and out.is_contiguous()
            and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
            and kc.data_ptr() % 128 == 0 and vc.data_ptr() % 128 == 0):
        tt = prefill_tc_tile_tokens(nq // nkv)
        tile_req, tile_tok0, n_tiles = ctx.q_tiles(tt)
        attention_prefill_tc(q, q.stride(0), out, kc, vc, bt, group.page_size, ctx.q_start, ctx.q_len, ctx.kv_len,
                             tile_req, tile_tok0, n_tiles, tt, nq, nkv, d, scale, int(window),
                             table_rows=group.table_rows, sinks=sinks, slopes=slopes)
        return
    if (q.dtype == torch.bfloat16 and not window and not chunk
            and rows_attention_supported(nq, nkv, d, dv, values_in_keys)
            and q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0
            and rows_attention_tile_tokens(nq // nkv, 16) in ctx.tiles):
        rows, tt, splits, stages = _rows_attention_plan(ctx, nq, nkv, d, dv, values_in_keys, q.device)
        tile_req, tile_tok0, n_tiles = ctx.q_tiles(tt)
        part_o = part_ml = None
        if splits > 1:
            units = n_tiles * nkv * max(1, (nq // nkv) // rows)
            part_o = torch.empty(units * splits * rows * dv, dtype=torch.float32, device=q.device)
            part_ml = torch.empty(units * splits * rows * 2, dtype=torch.float32, device=q.device)
        lib = _lib("attention_rows")
        rc = lib.mi_attention_rows(
            _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kc), _ptr(vc), _ptr(bt), bt.stride(0),
            _ptr(group.table_rows), int(group.page_size), _ptr(ctx.q_start), _ptr(ctx.q_len), _ptr(ctx.kv_len),
            _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), tt, rows, nq, nkv, d, dv, float(scale), _ptr(sinks),
            _ptr(slopes), 1 if values_in_keys else 0, splits, _ptr(part_o), _ptr(part_ml), stages, _stream())
        _finish(lib, rc, "attention")
        if splits > 1:
            launch_count += 1        # the merge of the runs
        return
    tile_req, tile_tok0, n_tiles = ctx.q_tiles(ATTENTION_TILE_TOKENS)
    lib = _lib("attention_generic")
    if lib.mi_attention_generic_tile_tokens() != ATTENTION_TILE_TOKENS:
        raise KernelError("attention: the kernel's tile size differs from ATTENTION_TILE_TOKENS")
    rc = lib.mi_attention_generic_masked(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(kc), _ptr(vc), _ptr(bt), bt.stride(0),
        _ptr(group.table_rows), int(group.page_size), _ptr(ctx.q_start), _ptr(ctx.q_len), _ptr(ctx.kv_len),
        _ptr(tile_req), _ptr(tile_tok0), int(n_tiles), nq, nkv, d, dv, float(scale), int(window), int(chunk),
        _ptr(sinks), _ptr(slopes), 1 if values_in_keys else 0, _code(q.dtype), _stream())
    _finish(lib, rc, "attention")


def batched_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """One small product per head: ``out[m, b, :] = w[b] x[m, b, :]`` for ``x [M, B, K]`` and ``out
    [M, B, N]`` (views with unit inner stride are fine) and ``w [B, N, K]`` contiguous.  float32 runs
    the true-fp32 kernel head by head; bfloat16 the library's batched product with fp32 accumulation."""
    global launch_count
    _cuda(x, w, out)
    if x.dim() != 3 or out.dim() != 3 or w.dim() != 3 or not w.is_contiguous():
        raise KernelError("batched_linear: x [M, B, K], w [B, N, K] contiguous, out [M, B, N]")
    M, B, K = x.shape
    N = w.shape[1]
    if w.shape != (B, N, K) or out.shape != (M, B, N) or x.stride(2) != 1 or out.stride(2) != 1:
        raise KernelError(f"batched_linear: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not match")
    if x.dtype == torch.float32:
        for b in range(B):
            gemm_f32(x[:, b], w[b], out=out[:, b])
        return out
    if not (x.dtype == w.dtype == out.dtype == torch.bfloat16):
        raise KernelError("batched_linear: operands must share float32 or bfloat16")
    launch_count += 1
    torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))
    return out
