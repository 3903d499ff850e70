"""ctypes binding of libancora_b200.so (the C ABI declared in include/ancora_b200.h).

There is no CPU fallback: if the shared library is missing the import of any compute
class fails with instructions to build it, and if no sm_100 GPU is present the first
context creation fails with the library's own message.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libancora_b200.so")

OK, E_INVALID, E_CUDA, E_NOMEM, E_DEVICE, E_NCCL, E_UNSUPPORTED = 0, -1, -2, -3, -4, -5, -6
GRAD_BF16, GRAD_F32 = 0, 1
ROUND_RNE, ROUND_SR = 0, 1


class AncoraError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"libancora_b200 status {code}: {msg}")
        self.code = code


class AdamWTensor(C.Structure):
    _fields_ = [("g", C.c_void_p), ("p32", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("p16", C.c_void_p), ("numel", C.c_uint64), ("elem_offset", C.c_uint64),
                ("wd", C.c_float), ("_pad", C.c_float)]


class AdamWScalars(C.Structure):
    _fields_ = [(n, C.c_float) for n in
                ("beta1", "one_minus_beta1", "beta2", "one_minus_beta2", "eps", "lr", "ibc1", "ibc2")]


class MuonOutputs(C.Structure):
    _fields_ = [("fp8", C.c_void_p), ("fp8_scale", C.c_void_p), ("p16_t", C.c_void_p),
                ("fp8_t", C.c_void_p), ("fp8_scale_t", C.c_void_p)]


class MuonWeight(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("g", C.c_void_p), ("p32", C.c_void_p), ("p16", C.c_void_p),
                ("K", C.c_int32), ("N", C.c_int32), ("owner", C.c_int32), ("_pad", C.c_int32)]


_vp, _i, _u64, _f, _d, _sz = C.c_void_p, C.c_int, C.c_uint64, C.c_float, C.c_double, C.c_size_t
_pp = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol include/ancora_b200.h declares
SIGNATURES = {
    "anc_version": (_i, []),
    "anc_last_error": (C.c_char_p, []),
    "anc_device_count": (_i, [C.POINTER(_i)]),
    "anc_ctx_create": (_i, [_i, _vp, _pp]),
    "anc_ctx_destroy": (_i, [_vp]),
    "anc_ctx_reserve_sms": (_i, [_vp, _i]),
    "anc_ctx_stream": (_i, [_vp, _pp]),
    "anc_ctx_sync": (_i, [_vp, _vp]),
    "anc_ctx_status": (_i, [_vp, C.POINTER(C.c_uint32)]),
    "anc_malloc": (_i, [_vp, _sz, _pp]),
    "anc_free": (_i, [_vp, _vp]),
    "anc_memset": (_i, [_vp, _vp, _i, _sz, _vp]),
    "anc_h2d": (_i, [_vp, _vp, _vp, _sz, _vp, _i]),
    "anc_d2h": (_i, [_vp, _vp, _vp, _sz, _vp, _i]),
    "anc_d2d": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "anc_host_alloc": (_i, [_sz, _pp]),
    "anc_host_alloc_near": (_i, [_i, _sz, _pp]),
    "anc_host_free": (_i, [_vp]),
    "anc_event_create": (_i, [_pp]),
    "anc_event_record": (_i, [_vp, _vp]),
    "anc_event_sync": (_i, [_vp]),
    "anc_event_elapsed_ms": (_i, [_vp, _vp, C.POINTER(_f)]),
    "anc_event_destroy": (_i, [_vp]),
    "anc_graph_begin": (_i, [_vp, _vp]),
    "anc_graph_end": (_i, [_vp, _vp, _pp]),
    "anc_graph_launch": (_i, [_vp, _vp, _vp]),
    "anc_graph_destroy": (_i, [_vp]),
    "anc_stream_create": (_i, [_vp, _pp]),
    "anc_stream_destroy": (_i, [_vp, _vp]),
    "anc_stream_wait_event": (_i, [_vp, _vp]),
    "anc_flush_l2": (_i, [_vp, _vp]),
    "anc_adamw_plan_create": (_i, [_vp, C.POINTER(AdamWTensor), _i, _i, _pp]),
    "anc_adamw_plan_set_range": (_i, [_vp, _u64, _u64]),
    "anc_adamw_plan_total": (_i, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "anc_adamw_step": (_i, [_vp, C.POINTER(AdamWScalars), _i, _u64, _u64, _vp]),
    "anc_adamw_plan_set_schedule": (_i, [_vp, C.POINTER(AdamWScalars), _i, _u64]),
    "anc_adamw_plan_set_counter": (_i, [_vp, _u64, _vp]),
    "anc_adamw_step_scheduled": (_i, [_vp, _i, _u64, _i, _vp]),
    "anc_adamw_plan_destroy": (_i, [_vp]),
    "anc_muon_plan_create": (_i, [_vp, C.POINTER(MuonWeight), _i, _i, _i, _i, _pp]),
    "anc_muon_plan_create_ex": (_i, [_vp, C.POINTER(MuonWeight), C.POINTER(MuonOutputs), _i, _i, _i, _i, _pp]),
    "anc_muon_step": (_i, [_vp, _d, _f, _i, _i, C.POINTER(_f), _f, _vp]),
    "anc_muon_plan_num_groups": (_i, [_vp, C.POINTER(_i)]),
    "anc_muon_plan_group_info": (_i, [_vp, _i, C.POINTER(C.c_int32)]),
    "anc_muon_step_range": (_i, [_vp, _i, _i, _i, _d, _f, _i, _i, C.POINTER(_f), _f, _vp]),
    "anc_muon_plan_set_timing": (_i, [_vp, _i]),
    "anc_muon_plan_last_timing": (_i, [_vp, C.POINTER(_f), C.POINTER(_d), C.POINTER(_i)]),
    "anc_muon_plan_scratch_bytes": (_i, [_vp, C.POINTER(_u64)]),
    "anc_muon_plan_destroy": (_i, [_vp]),
    "anc_ns_batched": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, C.POINTER(_f), _f, _vp]),
    "anc_ns_gemm_phase": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i, _i, _f, _f, _vp]),
    "anc_muon_momentum": (_i, [_vp, _vp, _vp, _i, _vp, _i, _i, _f, _i, _i, _vp]),
    "anc_muon_update": (_i, [_vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "anc_ns_batched_ex": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, C.POINTER(_f), _f, _i, _vp]),
    "anc_ns_chain_wait_selftest": (_i, [_vp, C.c_uint32]),
    "anc_ring_wait_selftest": (_i, [_vp, C.c_uint32]),
    "anc_fro_normalize": (_i, [_vp, _vp, _vp, _i, _i, _i, _f, _vp]),
    "anc_fro_normalize_static": (_i, [_i, _vp, _vp, _i, _i, _i, _f, _vp]),
    "anc_grad_accumulate": (_i, [_vp, _vp, _vp, _i, _vp, _u64, _u64, _f, _i, _u64, _u64, _i, _vp]),
    "anc_nccl_load": (_i, [C.c_char_p]),
    "anc_nccl_unique_id": (_i, [_vp]),
    "anc_comm_create": (_i, [_vp, _vp, _i, _i, _pp]),
    "anc_comm_destroy": (_i, [_vp]),
    "anc_comm_allgather_bf16": (_i, [_vp, _vp, _u64, _vp]),
    "anc_comm_reduce_scatter_grads": (_i, [_vp, _vp, _u64, _i, _vp]),
    "anc_comm_barrier": (_i, [_vp, _vp]),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ancora_cutile_b200.build` "
                "(needs nvcc).  This package has no CPU or PyTorch fallback.")
        l = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def check(rc):
    if rc != 0:
        msg = lib().anc_last_error()
        raise AncoraError(rc, msg.decode("utf-8", "replace") if msg else "")
    return rc
