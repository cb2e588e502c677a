"""ctypes binding of ``libpipelink_b200.so`` (declarations: ``include/pipelink_b200.h``).

Loading fails loudly: there is no CPU or library fallback for any stage. The library is
looked for in-tree (``pipelink_b200/_native``) and is produced by ``pipelink_b200.build``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p, POINTER, c_float
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_native" / "libpipelink_b200.so"

STATUS_BYTES = 32
STATUS_NAMES = {
    0: "ok", 1: "full-barrier timeout", 2: "empty-barrier timeout", 3: "accumulator-full timeout",
    4: "accumulator-empty timeout", 5: "readiness-counter timeout", 6: "bad argument on device",
    7: "drain timeout",
}

# name -> (restype, argtypes); must list every symbol include/pipelink_b200.h declares.
PROTOTYPES = {
    "plb_abi_version": (c_int, []),
    "plb_error_string": (c_char_p, [c_int]),
    "plb_last_cuda_error": (c_int, []),
    "plb_moe_set_swiglu_limit": (c_int, [c_float]),
    "plb_moe_swiglu_limit": (c_float, []),
    "plb_moe_tile_rows": (c_int, []),
    "plb_debug_set_profile_buffer": (c_int, [c_void_p]),
    "plb_mxfp8_quantize": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p]),
    "plb_mxfp8_quantize_live": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "plb_mxfp8_dequantize": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "plb_moe_schedule_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "plb_moe_schedule": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "plb_moe_schedule_streams_scratch_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "plb_moe_schedule_streams": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_size_t, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "plb_moe_schedule_noalloc_max_scratch_bytes": (c_size_t, []),
    "plb_moe_schedule_noalloc": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p]),
    "plb_moe_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                 c_void_p, c_void_p, c_void_p]),
    "plb_moe_pack_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p]),
    "plb_moe_gemm_gate_up": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                     c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                     c_void_p]),
    "plb_moe_gemm_down": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p,
                                  c_void_p]),
    "plb_moe_gemm_down_push": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                       c_void_p, c_void_p]),
    "plb_moe_gemm_gate_up_dispatch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p]),
    "plb_moe_gemm_gate_up_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p]),
    "plb_moe_gemm_gate_up_bf16_train": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_int, c_int] + [c_void_p] * 5),
    "plb_moe_gemm_wgrad_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "plb_moe_swiglu_bwd_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "plb_bf16_transpose": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "plb_bf16_transpose_live": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "plb_moe_gemm_down_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                                       c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "plb_ep_pull_rows_bulk": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                      c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "plb_ep_scale_rows": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p]),
    "plb_ep_stream_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int64, c_void_p, c_void_p,
                                   c_void_p]),
    "plb_moe_fwd_epilogue_indexed": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_void_p,
                                             c_void_p]),
    "plb_tp_push_rows": (c_int, [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "plb_tp_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                 c_int, c_void_p, ctypes.c_uint32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "plb_ep_barrier": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "plb_ep_publish": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p]),
    "plb_ep_pull_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                 c_void_p, c_void_p, c_void_p]),
    "plb_sym_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "plb_sym_free": (c_int, [c_void_p]),
    "plb_ipc_export": (c_int, [c_void_p, c_void_p]),
    "plb_ipc_import": (c_int, [c_void_p, POINTER(c_void_p)]),
    "plb_ipc_close": (c_int, [c_void_p]),
    "plb_decode_step": (c_int, [c_void_p, c_int, c_void_p]),
    "plb_decode_attention_partial": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_float, c_void_p]),
    "plb_moe_gemm_gate_up_train": (c_int, [c_void_p] * 6 + [c_int64, c_int, c_int, c_int] + [c_void_p] * 9),
    "plb_moe_gemm_gate_up_train_dispatch": (c_int, [c_void_p] * 10 + [c_int64, c_int, c_int, c_int] + [c_void_p] * 10),
    "plb_moe_bwd_dy": (c_int, [c_void_p] * 7 + [c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "plb_moe_swiglu_bwd": (c_int, [c_void_p] * 6 + [c_int64, c_int, c_void_p, c_void_p]),
    "plb_moe_gather_rows": (c_int, [c_void_p] * 4 + [c_int64, c_int, c_void_p, c_void_p]),
    "plb_moe_gemm_wgrad": (c_int, [c_void_p] * 5 + [c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "plb_ep_bwd_dy": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "plb_moe_router_grad": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "plb_moe_router_grad_indexed": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "plb_ep_gather_rows": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p]),
    "plb_attention_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                  c_int, ctypes.c_uint64, ctypes.c_uint64, c_float, c_int, c_float, c_void_p, ctypes.c_uint32,
                                  c_void_p, c_void_p]),
    "plb_cp_push_kv": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                               c_int, c_void_p]),
    "plb_attention_fwd_cp": (c_int, [c_void_p] * 6 + [c_int, c_int, c_int, c_int, ctypes.c_uint64, ctypes.c_uint64, c_float,
                                     c_void_p, ctypes.c_uint32, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int,
                                     c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "plb_image_load": (c_int, [c_void_p, c_char_p, c_int, POINTER(c_void_p), POINTER(c_void_p)]),
    "plb_image_launch": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "plb_image_launch_cooperative": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "plb_decode_kv_map": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "plb_image_unload": (c_int, [c_void_p]),
    "plb_tensor_map_2d_u8": (c_int, [c_void_p, c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32,
                                     ctypes.c_uint32, c_int]),
    "plb_tensor_map_2d_bf16": (c_int, [c_void_p, c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, c_int]),
    "plb_tensor_map_2d_u32": (c_int, [c_void_p, c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32]),
    "plb_moe_fwd_epilogue": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64,
                                     c_void_p, c_void_p]),
}

_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


class PlbError(RuntimeError):
    def __init__(self, fn: str, code: int, detail: str = ""):
        self.fn, self.code = fn, code
        super().__init__(f"{fn} failed: {code} ({detail})")


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NativeLibraryMissing(
                f"{LIB_PATH} not found: run `python -m pipelink_b200.build` (needs nvcc). "
                "There is no fallback path.")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = restype, argtypes
        if lib.plb_abi_version() != 1:
            raise NativeLibraryMissing("libpipelink_b200.so ABI version mismatch; rebuild")
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise PlbError on a non-zero code."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        detail = lib.plb_error_string(rc).decode()
        if rc == 8:
            detail += f", cudaError {lib.plb_last_cuda_error()}"
        raise PlbError(name, rc, detail)
