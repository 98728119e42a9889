"""ctypes binding to the in-tree native library (`_native/libcuteafd_b200.so`).

The library exposes a plain C ABI (`extern "C" int cuteafd_*(..., cudaStream_t)`), like the reference's
`libcuteafd_native.so` loaded through `libloading` (rust/crates/cuteafd-ffi/src/lib.rs).  On a machine
with a GPU a missing library is an error, never a silent fallback: `lib()` raises with the build hint.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB = None
# CUTEAFD_LIB points at an alternative build of the native library (A/B measurements of kernel variants)
LIB_PATH = Path(os.environ.get("CUTEAFD_LIB") or Path(__file__).resolve().parent.parent / "_native" / "libcuteafd_b200.so")

P, I, F, L, U64 = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_uint64

_PROTOS = {
    "cuteafd_abi_version": [],
    "cuteafd_set_pdl": [I],
    "cuteafd_tc_trace": [P, I],
    "cuteafd_exl3_linear": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, P],
    "cuteafd_fp8_linear": [I, P, P, P, P, P, P, I, I, I, I, I, I, P, P],
    "cuteafd_act_quant_fp8_block128": [P, P, P, I, I, I, P],
    "cuteafd_device_info": [P, P, P, P, P],
    "cuteafd_tmap_encode_kmajor": [P, P, I, U64, U64, U64, U64, U64, C.c_uint32],
    "cuteafd_embed_gather": [P, P, P, I, I, I, P, P],
    "cuteafd_add_rmsnorm": [P, P, P, P, I, I, F, P],
    "cuteafd_qk_norm_rope_kvwrite": [P, P, P, P, P, P, I, I, I, I, F, I, F, I, P, P],
    "cuteafd_quant_fp4_rows": [I, P, P, P, P, P, I, I, I, I, P, P],
    "cuteafd_gather_rows": [P, P, P, P, I, I, P],
    "cuteafd_act_quant_fp8_ue8m0": [P, P, P, P, P, I, I, I, I, P],
    "cuteafd_kv_pages_copy": [P, L, I, I, P, I, P, L, I, P],
    "cuteafd_attn_merge": [P, P, P, P, I, I, I, P],
    "cuteafd_router_logits": [P, P, P, I, I, I, P],
    "cuteafd_attn_partials_only": [],
    "cuteafd_l2_prefetch": [P, L, P],
    "cuteafd_silu_mul": [P, P, P, L, F, P],
    "cuteafd_router_select": [P, P, P, P, I, I, I, I, I, F, I, I, P],
    "cuteafd_add_rmsnorm_quant": [P, P, P, P, I, I, F, P, P, I, P, I, P],
    "cuteafd_moe_combine_norm": [P, P, P, P, P, P, I, I, I, P, F, P, P, P, I, P, I, P, P],
    "cuteafd_router_select_pack": [P, P, P, P, I, I, I, I, I, F, I, I, P, P, P, P, P, P, P, I, I, I, I, P, P, P],
    "cuteafd_route_pack": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, P, P, P, I, P],
    "cuteafd_route_gather": [P, P, P, P, P, P, I, I, I, I, I, I, P, P],
    "cuteafd_tc_cluster_capacity": [I, I, I, P],
    "cuteafd_fp8_cluster_capacity": [I, I, I, P],
    "cuteafd_router_fused": [P, P, P, P, P, P, I, I, I, I, I, I, F, I, I, P, P, P, P, P, P, P, I, I, I, I, P, P, P],
    "cuteafd_router_hash_select": [P, P, P, P, P, I, I, I, I, F, P, P],
    "cuteafd_moe_combine": [P, P, P, P, P, P, I, I, I, P, P],
    "cuteafd_paged_attention": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, P],
    "cuteafd_paged_attention_tc": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P, P, P, I, P, I, P],
    "cuteafd_tmap_encode_kv": [P, P, I, U64],
    "cuteafd_mla_attention": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, P, P],
    "cuteafd_tmap_encode_latent": [P, P, U64],
    "cuteafd_gated_delta_step": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, P, P],
    "cuteafd_linear_prepare": [P, P, P, P, P, P, P, P, P, I, I, I, I, I, P],
    "cuteafd_gated_rmsnorm": [P, P, P, P, I, I, I, I, F, P],
    "cuteafd_short_conv4": [P, P, P, P, P, P, P, I, I, I, I, P, P],
    "cuteafd_short_conv4_peek": [P, P, P, P, P, P, P, I, I, I, I, P, P],
    "cuteafd_mhc_boundary": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, F, P],
    "cuteafd_vision_rgb_patches": [P, P, P, I, I, I, I, I, P],
    "cuteafd_compress_pool": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, F, P],
    "cuteafd_engram_gather": [P, P, P, P, P, I, I, L, P, P],
    "cuteafd_engram_gate": [P, P, I, P, P, P, I, I, I, P],
    "cuteafd_audio_im2col3": [P, P, I, I, I, P],
    "cuteafd_vision_add_norm": [P, P, I, P, P, P, P, I, I, F, I, P],
    "cuteafd_vision_qkv_rope_store": [P, P, P, P, P, P, P, P, I, I, I, F, P, P],
    "cuteafd_vision_bias_act": [P, I, P, P, I, I, I, I, P],
    "cuteafd_dsa_index_scores": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
    "cuteafd_tmap_encode_index_keys": [P, P, U64],
    "cuteafd_dsa_topk": [P, I, P, I, I, I, P, P, P],
    "cuteafd_dsa_gather_rows": [P, P, P, P, P, P, I, I, I, I, L, I, P, P],
    "cuteafd_dsa_scatter_rows": [P, P, P, I, L, I, P, P],
    "cuteafd_gqa_prefill_attention": [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P],
    "cuteafd_mla_gather_ctx": [P, P, P, P, P, I, I, I, L, L, P, P],
    "cuteafd_mla_prefill_attention": [P, P, P, P, L, P, P, P, P, P, I, I, I, I, F, P, P],
    "cuteafd_mla_kv_prepare": [P, P, P, P, P, I, I, F, F, I, P, P],
    "cuteafd_mla_q_split": [P, P, P, P, I, I, F, I, P],
    "cuteafd_head_to_token_major": [P, P, I, I, I, P],
    "cuteafd_head_to_token_major_fp8b": [P, P, P, P, I, I, I, P],
    "cuteafd_silu_mul_quant_fp8b": [P, P, P, P, I, I, I, P],
    "cuteafd_argmax_rows": [P, I, I, I, P, I, P, P, P, P],
    "cuteafd_sample_rows": [P, I, I, I, P, I, P, P, P, P],
    "cuteafd_verify_accept": [P, P, P, P, P, I, I, I, P],
    "cuteafd_ipc_export": [P, P, P],
    "cuteafd_ipc_open": [P, C.c_ulonglong, P],
    "cuteafd_ipc_close": [P, C.c_ulonglong],
    "cuteafd_step_begin": [P, P],
    "cuteafd_wait_flags": [P, I, I, P, C.c_uint, C.c_ulonglong, P, P],
    "cuteafd_push_bytes": [P, P, C.c_size_t, P, P, C.c_uint, P, P],
    "cuteafd_wait_add": [P, P, P, P, C.c_size_t, I, P, P, C.c_uint, C.c_ulonglong, P, P],
    "cuteafd_wait_concat": [P, P, P, I, I, I, I, P, P, C.c_uint, C.c_ulonglong, P, P],
    "cuteafd_dispatch_push": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, C.c_uint, P, P],
    "cuteafd_combine_push": [P, P, P, P, P, P, P, I, I, I, C.c_uint, P],
    "cuteafd_peer_copy": [P, P, C.c_size_t, I, P],
    "cuteafd_copy_engine": [P, P, C.c_size_t, P],
    "cuteafd_flag_pingpong": [P, P, C.c_uint, I, I, C.c_ulonglong, P, P, P],
    "cuteafd_dispatch_tok_push": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, C.c_uint, P, P],
    "cuteafd_combine_push_lanes": [P, P, P, P, P, P, P, I, I, I, I, I, I, C.c_uint, P, P],
    "cuteafd_tc_linear": [I, I, I, P, P, P, P, P, P, I, P, P, P, P, I, P, P, I, I, I, I, I, I, P, P, P, I, P, P],
}


class NativeError(RuntimeError):
    pass


class FlagWaitArg(C.Structure):
    """In-kernel wait handed to a consumer of peer data (`CaFlagWaitArg` of the C ABI): the kernel polls `n` flags,
    `stride` words apart, until each reaches the step number in ctl[1]; a wait that runs out sets `status` and ctl[0]."""
    _fields_ = [("flags", P), ("ctl", P), ("status", P), ("timeout_ns", C.c_ulonglong), ("n", I), ("stride", I)]


class TcExtra(C.Structure):
    """Optional outputs of `cuteafd_tc_linear` (`CaTcExtra` of the C ABI)."""
    _fields_ = [("q_out", P), ("sf_out", P), ("inv_gs_out", P), ("ldsf_out", I), ("n_peer", I), ("peer_y", P * 2), ("peer_flag", P * 2),
                ("peer_row_map", P), ("peer_ctl", P), ("peer_done", P), ("peer_ld", I), ("reserved", I)]


def flag_wait(flags_ptr: int, n: int, stride: int, ctl: torch.Tensor, status: torch.Tensor | None, timeout_ns: int = 2_000_000_000) -> FlagWaitArg:
    return FlagWaitArg(flags_ptr, ctl.data_ptr(), status.data_ptr() if status is not None else None, timeout_ns, n, stride)


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        if not LIB_PATH.exists():
            raise NativeError(f"native library missing at {LIB_PATH}; run `python -m cuteafd_b200.build`")
        _LIB = C.CDLL(str(LIB_PATH))
        _LIB.cuteafd_last_error.restype = C.c_char_p
        for name, args in _PROTOS.items():
            if hasattr(_LIB, name):
                fn = getattr(_LIB, name)
                fn.argtypes = args
                fn.restype = I
    return _LIB


def call(name: str, *args) -> None:
    l = lib()
    rc = getattr(l, name)(*args)
    if rc != 0:
        raise NativeError(f"{name} failed ({rc}): {l.cuteafd_last_error().decode()}")


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def require_gpu_lib():
    """Ops call this first: with a CUDA device present the native library must be loadable."""
    if torch.cuda.is_available():
        lib()


STATUS_CODES = {1: "producer wait timed out", 2: "mma wait timed out", 3: "epilogue wait timed out",
                4: "flag wait timed out", 5: "index out of range"}


def decode_status(word: int) -> str:
    if word == 0:
        return "ok"
    return f"{STATUS_CODES.get(word >> 24, 'unknown')} (detail {word & 0xFFFFFF})"
