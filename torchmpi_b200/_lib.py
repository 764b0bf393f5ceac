"""ctypes binding of libtorchmpi_b200.so (the flat C ABI in csrc/include/tmpi_c_api.h).

The reference binds its C symbols through LuaJIT FFI declarations generated per
dtype (torchmpi/ffi.lua:13-219); here dtypes are an enum argument, so one
prototype per operation is enough.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent
_DEBUG_BOUNDS = bool(os.environ.get("TORCHMPI_DEBUG_BOUNDS"))     # the build with recording bounds checks
_LIB_PATH = _PKG / "lib" / ("libtorchmpi_b200_dbg.so" if _DEBUG_BOUNDS else "libtorchmpi_b200.so")


class TorchMPIError(RuntimeError):
    """An entry point of the native runtime returned a non-zero status."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[torchmpi_b200 status {code}] {msg}")
        self.code = code


class TimeoutError_(TorchMPIError):
    """A bounded wait (host or device) ran out (status 3)."""


OK, ERR_INVALID, ERR_CUDA, ERR_TIMEOUT, ERR_STATE, ERR_UNSUPPORTED, ERR_SYS = range(7)

DTYPES = {
    torch.uint8: 0, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4,
    torch.float16: 5, torch.bfloat16: 6, torch.float32: 7, torch.float64: 8,
}


def _load() -> C.CDLL:
    from . import build as _build
    if os.environ.get("TORCHMPI_REBUILD") or not _build.is_current():
        if _build.nvcc() is not None:
            _build.build(force=bool(os.environ.get("TORCHMPI_REBUILD")))
        elif not _LIB_PATH.exists():
            raise ImportError("libtorchmpi_b200.so is missing and nvcc is not available to build it")
    return C.CDLL(str(_LIB_PATH), mode=C.RTLD_GLOBAL)


lib = _load()

_vp, _i, _i64, _u64, _sz, _d, _f, _cp = (C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_size_t,
                                         C.c_double, C.c_float, C.c_char_p)
_ip = C.POINTER(C.c_int)
_i64p = C.POINTER(C.c_int64)


class Group(C.Structure):
    """tmpi_group_t: the ranks of the symmetric heap that take part, my index, the launch lane."""
    _fields_ = [("members", _ip), ("nmembers", _i), ("me", _i), ("lane", _i)]


class SgdBucket(C.Structure):
    """tmpi_sgd_bucket_t."""
    _fields_ = [("grad_off", _sz), ("weight_off", _sz), ("master", _vp), ("momentum", _vp),
                ("n", _sz), ("grad_dtype", _i), ("weight_dtype", _i),
                ("lr", _f), ("momentum_coef", _f), ("dampening", _f), ("weight_decay", _f),
                ("grad_scale", _f), ("nesterov", _i), ("first_step", _i), ("zero_grads", _i)]


_gp = C.POINTER(Group)

_PROTOS = {
    "tmpi_last_error": (_cp, []),
    "tmpi_version": (_i, []),
    "tmpi_has_cuda": (_i, []),
    "tmpi_dtype_size": (_sz, [_i]),
    "tmpi_set_tunable": (_i, [_cp, _i64]),
    "tmpi_get_tunable": (_i, [_cp, _i64p]),
    "tmpi_num_tunables": (_i, []),
    "tmpi_tunable_name": (_cp, [_i]),
    "tmpi_freeze_tunables": (_i, []),
    "tmpi_comm_reset": (_i, [_i, _i]),
    "tmpi_comm_push": (_i, [_cp, _ip, _i, _cp]),
    "tmpi_comm_num_levels": (_i, []),
    "tmpi_comm_set": (_i, [_i]),
    "tmpi_comm_set_typed": (_i, [_i, _i]),
    "tmpi_comm_level": (_i, []),
    "tmpi_comm_is_inter": (_i, []),
    "tmpi_comm_set_span": (_i, [_i, _i]),
    "tmpi_comm_get_span": (_i, [_ip, _ip]),
    "tmpi_comm_is_cartesian": (_i, [_i]),
    "tmpi_comm_members": (_i, [_i, _i, _ip, _i]),
    "tmpi_comm_rank_in": (_i, [_i, _i]),
    "tmpi_comm_key": (_i, [_i, C.c_char_p, _i]),
    "tmpi_comm_current_members": (_i, [_ip, _i]),
    "tmpi_comm_group_of": (_i, [_i, _i, _ip, _i]),
    "tmpi_comm_names": (_i, [C.c_char_p, _i]),
    "tmpi_comm_has_inter_collective": (_i, [_i]),
    "tmpi_comm_has_intra_collective": (_i, [_i]),
    "tmpi_comm_pop_to": (_i, [_i]),
    "tmpi_ring_plan": (_i, [_i, _i, _i, _ip, _i]),
    "tmpi_ring_send_chunk": (_i, [_i, _i, _i, _i]),
    "tmpi_ring_recv_chunk": (_i, [_i, _i, _i, _i]),
    "tmpi_handle_wait": (_i, [_u64, _i64]),
    "tmpi_handle_done": (_i, [_u64]),
    "tmpi_handle_stream_wait": (_i, [_u64, _vp]),
    "tmpi_sync_all": (_i, []),
    "tmpi_handles_in_flight": (_i, []),
    "tmpi_test_lost_handle": (_u64, []),
    "tmpi_test_sleep_task": (_u64, [_i, _i, _i]),
    "tmpi_shm_create": (_i, [_cp, _sz, _i, _i, C.POINTER(_vp)]),
    "tmpi_shm_attach": (_i, [_i, _cp]),
    "tmpi_shm_ready": (_i, []),
    "tmpi_shm_destroy": (_i, []),
    "tmpi_shm_capacity": (_sz, []),
    "tmpi_shm_allreduce": (_i, [_vp, _vp, _sz, _i, _d, _ip, _i, _i, _i]),
    "tmpi_shm_allreduce_async": (_u64, [_vp, _vp, _sz, _i, _d, _ip, _i, _i, _i]),
    "tmpi_shm_broadcast": (_i, [_vp, _sz, _i, _i, _ip, _i, _i]),
    "tmpi_shm_broadcast_async": (_u64, [_vp, _sz, _i, _i, _ip, _i, _i]),
    "tmpi_shm_reduce": (_i, [_vp, _vp, _sz, _i, _i, _ip, _i, _i]),
    "tmpi_shm_allgather": (_i, [_vp, _vp, _sz, _i64p, _i, _ip, _i, _i]),
    "tmpi_shm_barrier": (_i, [_ip, _i, _i, _i64]),
    "tmpi_ps_shard_range": (_i, [_sz, _i, _i, C.POINTER(_sz), C.POINTER(_sz)]),
    "tmpi_shm_ps_init": (_i, [_vp, _sz, _i, _ip, _i, _i]),
    "tmpi_shm_ps_free": (_i, [_i]),
    "tmpi_shm_ps_free_all": (_i, []),
    "tmpi_shm_ps_send": (_u64, [_i, _vp, _i]),
    "tmpi_shm_ps_receive": (_u64, [_i, _vp]),
    "tmpi_trace_enable": (_i, [_i]),
    "tmpi_trace_record": (_i, [_cp, _cp, _u64, _d]),
    "tmpi_trace_dump": (_i, [C.c_char_p, _i]),
    "tmpi_trace_clear": (_i, []),
}

_CUDA_PROTOS = {
    "tmpi_cuda_set_device": (_i, [_i]),
    "tmpi_cuda_heap_create": (_i, [_sz, _i, _i, _i]),
    "tmpi_cuda_heap_create_emulated": (_i, [_sz, _i]),
    "tmpi_cuda_heap_export": (_i, [_vp, _i]),
    "tmpi_cuda_heap_import": (_i, [_i, _vp, _i]),
    "tmpi_cuda_heap_finish": (_i, []),
    "tmpi_cuda_heap_mc_export": (_i, [_vp, _i]),
    "tmpi_cuda_heap_mc_import": (_i, [_vp, _i]),
    "tmpi_cuda_heap_mc_bind": (_i, []),
    "tmpi_cuda_heap_destroy": (_i, []),
    "tmpi_cuda_heap_base": (_vp, [_i]),
    "tmpi_cuda_heap_mc_base": (_vp, []),
    "tmpi_cuda_heap_capacity": (_sz, []),
    "tmpi_cuda_heap_alloc": (_sz, [_sz, _sz]),
    "tmpi_cuda_heap_reset_allocator": (_i, [_sz]),
    "tmpi_cuda_heap_world": (_i, []),
    "tmpi_debug_bounds_build": (_i, []),
    "tmpi_cuda_heap_layout": (_i, [C.POINTER(C.c_size_t), _i]),
    "tmpi_cuda_heap_rank": (_i, []),
    "tmpi_cuda_allreduce": (_i, [_vp, _vp, _sz, _i, _d, _gp, _i, _vp]),
    "tmpi_cuda_allreduce_heap": (_i, [_sz, _sz, _sz, _i, _d, _gp, _i, _vp]),
    "tmpi_cuda_broadcast": (_i, [_vp, _sz, _i, _i, _gp, _vp]),
    "tmpi_cuda_broadcast_heap": (_i, [_sz, _sz, _i, _i, _gp, _i, _vp]),
    "tmpi_cuda_reduce": (_i, [_vp, _vp, _sz, _i, _i, _gp, _vp]),
    "tmpi_cuda_allgather": (_i, [_vp, _vp, _sz, _i, _gp, _vp]),
    "tmpi_cuda_allgatherv": (_i, [_vp, _vp, _sz, _i64p, _i, _gp, _vp]),
    "tmpi_cuda_reduce_scatter": (_i, [_vp, _vp, _sz, _i, _d, _gp, _vp]),
    "tmpi_cuda_barrier": (_i, [_gp, _vp]),
    "tmpi_cuda_allreduce_async": (_u64, [_vp, _vp, _sz, _i, _d, _gp, _i, _vp]),
    "tmpi_cuda_broadcast_async": (_u64, [_vp, _sz, _i, _i, _gp, _vp]),
    "tmpi_cuda_collective_status": (_i, [_i, _ip, _ip, _ip]),
    "tmpi_cuda_test_wait_timeout": (_i, [_i64, _vp]),
    "tmpi_cuda_allreduce_sgd": (_i, [C.POINTER(SgdBucket), _gp, _i, _vp]),
    "tmpi_cuda_ps_push": (_i, [_sz, _vp, _sz, _i, _i, _gp, _vp]),
    "tmpi_cuda_ps_pull": (_i, [_sz, _vp, _sz, _i, _gp, _vp]),
    "tmpi_sgd_momentum": (_i, [_vp, _i, _vp, _i, _vp, _vp, _sz, _f, _f, _f, _f, _f, _i, _i, _i, _vp]),
    "tmpi_xent_fwd_bwd": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp, _f, _vp, _vp]),
    "tmpi_xent_fwd_bwd_ld": (_i, [_vp, _i, _vp, _i, _i, _i, _vp, _vp, _f, _vp, _vp]),
    "tmpi_xent_scratch_bytes": (_sz, [_i]),
    "tmpi_cuda_ps_push_async": (_u64, [_sz, _vp, _sz, _i, _i, _gp, _vp]),
    "tmpi_cuda_ps_pull_async": (_u64, [_sz, _vp, _sz, _i, _gp, _vp]),
    "tmpi_absmean_var": (_i, [_vp, _i, _sz, _vp, _vp, _vp]),
    "tmpi_absmean_var_scratch_bytes": (_sz, []),
    "tmpi_easgd_elastic": (_i, [_vp, _vp, _vp, _sz, _i, _f, _vp]),
    "tmpi_downpour_accum": (_i, [_vp, _vp, _sz, _i, _f, _i, _vp]),
    "tmpi_bias_grad_scratch_bytes": (_sz, [_i]),
    "tmpi_bias_grad": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "tmpi_gelu_fwd": (_i, [_vp, _vp, _sz, _i, _vp]),
    "tmpi_layernorm_supported": (_i, [_i, _i]),
    "tmpi_layernorm_scratch_bytes": (_sz, [_i]),
    "tmpi_layernorm_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "tmpi_layernorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "tmpi_bn_relu_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _f, _f, _i, _i, _i, _vp, _vp, _vp]),
    "tmpi_bn_relu_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp, _vp, _vp]),
    "tmpi_bn_relu_bwd_acc": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "tmpi_bn_scratch_bytes": (_sz, [_i]),
    "tmpi_bn_relu_fwd_partials": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _f, _f, _i, _i, _vp, _vp, _i, _vp]),
    "tmpi_bn_relu_pool_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _i, _i, _vp, _vp]),
    "tmpi_bn_relu_pool_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "tmpi_stem_im2col": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "tmpi_stem_patch_width": (_i, []),
    "tmpi_maxpool_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tmpi_maxpool_bwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tmpi_gemm_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tmpi_gemm_bf16_ex": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i64, _i64, _i64, _i, _vp]),
    "tmpi_gemm_status": (_i, []),
    "tmpi_conv_max_ctas": (_i, []),
    "tmpi_conv_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _ip, _vp]),
    "tmpi_conv_dgrad": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "tmpi_conv_wgrad_workspace_bytes": (_sz, [_i, _i, _i, _i, _i, _i, _i, _i, _i]),
    "tmpi_conv_wgrad": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _i, _vp]),
    "tmpi_conv_status": (_i, []),
    "tmpi_attention_fwd": (_i, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _f, _vp]),
    "tmpi_attention_bwd": (_i, [_vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _f, _vp]),
    "tmpi_attention_bwd_status": (_i, []),
    "tmpi_attention_bwd_set_trace": (None, [_vp]),
    "tmpi_attention_ctas_per_sm": (_i, []),
    "tmpi_attention_set_trace": (None, [_vp]),
    "tmpi_attention_set_v_stages": (None, [_i]),
    "tmpi_attention_status": (_i, []),
    "tmpi_gemm_tn_splitk_workspace_bytes": (_sz, [_i, _i, _i64]),
    "tmpi_gemm_bf16_tn_splitk": (_i, [_vp, _vp, _vp, _i, _i, _i64, _i64, _i64, _vp, _sz, _i, _vp]),
}


def _bind(protos: dict, required: bool) -> None:
    for name, (res, args) in protos.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if required:
                raise
            continue
        fn.restype = res
        fn.argtypes = args


_bind(_PROTOS, True)
_bind(_CUDA_PROTOS, False)


def has_symbol(name: str) -> bool:
    return hasattr(lib, name)


def last_error() -> str:
    return lib.tmpi_last_error().decode(errors="replace")


def check(status: int) -> int:
    """Raises on a non-zero status; negative values are negated statuses."""
    if status == 0:
        return 0
    code = abs(status)
    cls = TimeoutError_ if code == ERR_TIMEOUT else TorchMPIError
    raise cls(code, last_error())


def int_array(values) -> "C.Array[C.c_int]":
    values = list(values)
    return (C.c_int * max(1, len(values)))(*values)


def dtype_code(dt: torch.dtype) -> int:
    try:
        return DTYPES[dt]
    except KeyError:
        raise TypeError(f"torchmpi_b200: unsupported dtype {dt}") from None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(stream=None) -> int:
    """The ``cudaStream_t`` of ``stream`` (default: the current stream of the current device) as an integer.
    The raw accessor avoids building a ``torch.cuda.Stream`` object for every kernel launch."""
    if stream is not None:
        return stream.cuda_stream
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream
