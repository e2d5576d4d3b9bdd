"""Loader of libmacseek_b200.so (the C ABI in include/macseek_b200.h).  There is no fallback: if the library has not
been built (python -m macseek_b200.build) importing this module fails."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmacseek_b200.so")


class MsbError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError("libmacseek_b200.so is not built: run `python -m macseek_b200.build` (needs nvcc)")
    return C.CDLL(LIB_PATH)


lib = _load()
lib.msb_last_error.restype = C.c_char_p
lib.msb_version.restype = C.c_char_p
lib.msb_block_bytes.restype = C.c_size_t
lib.msb_row_bytes.restype = C.c_size_t
lib.msb_row_bytes.argtypes = [C.c_int, C.c_int64]
_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float
lib.msb_dequant.argtypes = [_i, _vp, _i64, _vp, _vp]
lib.msb_matvec.argtypes = [_i, _vp, _i, _i, _vp, _vp, _i, _i, _vp]
lib.msb_matvec_n.argtypes = [_i, _vp, _i, _i, _vp, _vp, _i, _i, _i, _vp]


def check(rc):
    if rc != 0:
        raise MsbError("msb error %d: %s" % (rc, lib.msb_last_error().decode()))


def device_status():
    """Synchronise and return (then clear) the device failure word; raises on CUDA errors."""
    rc = lib.msb_device_status()
    if rc < 0:
        check(rc)
    return rc


class ExpertSlotC(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p)]


class MoeDecodeArgsC(C.Structure):
    _fields_ = [("dim", C.c_int), ("inter", C.c_int), ("t_gate_up", C.c_int), ("t_down", C.c_int),
                ("t_shared", C.c_int), ("n_routed", C.c_int), ("has_shared", C.c_int),
                ("slot", ExpertSlotC * 16), ("shared", ExpertSlotC), ("weights", C.c_void_p), ("x", C.c_void_p),
                ("y", C.c_void_p), ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("swiglu_limit", C.c_float)]


class MoePrefillArgsC(C.Structure):
    _fields_ = [("dim", C.c_int), ("inter", C.c_int), ("t_gate_up", C.c_int), ("t_down", C.c_int), ("t_shared", C.c_int),
                ("n_tokens", C.c_int), ("n_exp", C.c_int), ("slots", C.POINTER(ExpertSlotC)), ("offs", C.POINTER(C.c_int)),
                ("tok", C.c_void_p), ("wt", C.c_void_p), ("slot_of", C.c_void_p), ("k_per_token", C.c_int),
                ("has_shared", C.c_int), ("shared", ExpertSlotC), ("X", C.c_void_p), ("Y", C.c_void_p),
                ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("swiglu_limit", C.c_float)]


lib.msb_moe_prefill_scratch_bytes.restype = C.c_size_t
lib.msb_moe_prefill_scratch_bytes.argtypes = [_i, _i, _i, _i, _i]
lib.msb_moe_prefill.argtypes = [C.POINTER(MoePrefillArgsC), _vp]
lib.msb_f32_to_f16.argtypes = [_vp, _vp, C.c_size_t, _vp]
lib.msb_matmul_scratch_bytes.restype = C.c_size_t
lib.msb_matmul_scratch_bytes.argtypes = [_i, _i, _i, _i, _i]
lib.msb_matmul_h.argtypes = [_i, _vp, _i, _i, _vp, _i, _vp, _i, _i, _vp, C.c_size_t, _vp]
lib.msb_matmul.argtypes = [_i, _vp, _i, _i, _vp, _vp, _i, _i, _vp, C.c_size_t, _vp]
lib.msb_moe_decode_scratch_bytes.restype = C.c_size_t
lib.msb_moe_decode_scratch_bytes.argtypes = [_i, _i]
lib.msb_moe_decode.argtypes = [C.POINTER(MoeDecodeArgsC), _vp]
lib.msb_moe_decode_noalloc.argtypes = [C.POINTER(MoeDecodeArgsC), _vp]
lib.msb_moe_decode_table_part.argtypes = [C.POINTER(MoeDecodeArgsC), _vp, _i, _vp]
lib.msb_moe_decode_ids.argtypes = [C.POINTER(MoeDecodeArgsC), _vp, _vp, _i, _i, _i, _vp]
lib.msb_moe_decode_ids_normed.argtypes = [C.POINTER(MoeDecodeArgsC), _vp, _vp, _i, _i, _i, _vp, _vp, C.c_float, _vp]
lib.msb_router_scratch_bytes.restype = C.c_size_t
lib.msb_router_scratch_bytes.argtypes = [_i]
lib.msb_router_fused.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _i, _i, _i, _i, _f, _vp]
lib.msb_router_fused_rmsnorm.argtypes = [_vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _i, _i, _i, _i, _f, _vp]
lib.msb_router_topk.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]
lib.msb_route_lists.argtypes = [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]

lib.msb_index_prep.argtypes = [_vp, _vp, _vp, _i, _i, _vp, _vp, _vp]
lib.msb_index_scores.argtypes = [_i, _vp, _i, _vp, _vp, _i, _vp, _vp, _i, _vp]
lib.msb_topk_scratch_bytes.restype = C.c_size_t
lib.msb_topk_scratch_bytes.argtypes = [_i]
lib.msb_topk.argtypes = [_vp, _i, _i, _vp, _vp, C.c_size_t, _i, _vp]
lib.msb_block_max.argtypes = [_vp, _i, _i, _vp, _vp]
lib.msb_index_decode.argtypes = [_i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _i, _vp]
lib.msb_index_decode_list.argtypes = [_i, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]
lib.msb_sparse_scratch_bytes.restype = C.c_size_t
lib.msb_sparse_scratch_bytes.argtypes = [_i, _i, _i]
lib.msb_sparse_decode.argtypes = [_vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, C.c_size_t, _vp]

lib.msb_rmsnorm.argtypes = [_vp, _vp, _vp, _i, _i, _f, _i, _i, _vp]
lib.msb_kv_window.argtypes = [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]
lib.msb_argmax.argtypes = [_vp, _i, _vp, _vp, _vp]
lib.msb_add.argtypes = [_vp, _vp, _i, _vp]
lib.msb_matvec_rmsnorm.argtypes = [_i, _vp, _i, _i, _vp, _vp, _f, _vp, _vp]
lib.msb_matvec_rmsnorm_shared.argtypes = [_i, _vp, _i, _i, _vp, _vp, _f, _vp, _vp]


class EpCommC(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("base", C.c_void_p * 8)]


lib.msb_moe_decode_ep.argtypes = [C.POINTER(MoeDecodeArgsC), _vp, _vp, _i, _i, _vp, _vp, C.c_float, _i, _i,
                                  C.POINTER(EpCommC), _vp]
lib.msb_ep_exchange_bytes.restype = C.c_size_t
lib.msb_ep_exchange_bytes.argtypes = [_i, _i]
lib.msb_ep_combine.argtypes = [C.POINTER(EpCommC), _vp, _i, _vp]
lib.msb_set_peer_wait_cycles.restype = None
lib.msb_set_peer_wait_cycles.argtypes = [C.c_longlong]
lib.msb_ep_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
lib.msb_ep_free.argtypes = [_vp]
lib.msb_ipc_export.argtypes = [_vp, C.c_char_p]
lib.msb_ipc_import.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
lib.msb_ipc_release.argtypes = [_vp]
lib.msb_hc_scratch_bytes.restype = C.c_size_t
lib.msb_hc_scratch_bytes.argtypes = [_i]
lib.msb_hc_step.argtypes = [_vp] * 10 + [_i, _i, _vp, C.c_size_t, _vp]
lib.msb_compress.argtypes = [_vp] * 7 + [_i] * 6 + [_vp, _i, _vp, _vp]
lib.msb_sample_scratch_bytes.restype = C.c_size_t
lib.msb_sample_scratch_bytes.argtypes = [_i]
lib.msb_argmax_rows.argtypes = [_vp, _i, _i, _vp, _vp, C.c_float, C.c_ulonglong, _vp, C.c_size_t, _vp]
lib.msb_sample_topk.argtypes = [_vp, _i, _i, _i, C.c_float, _vp, _vp, _vp, _vp, C.c_size_t, _vp]
lib.msb_log_softmax.argtypes = [_vp, _vp, _i, _i, _vp]
lib.msb_sample_top_p.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int), _i, C.c_float, C.c_float, C.c_float, C.c_double]
lib.msb_copy_device.argtypes = [_vp, _vp, C.c_size_t, _vp]
