"""ctypes declarations of the C ABI in include/liger_b200.h (one-to-one, no logic)."""
import ctypes as C
import os

from .build import LIB_PATH

LIGER_OK = 0
EPI_STORE, EPI_GELU, EPI_GEGLU, EPI_QKV_SPLIT, EPI_RESIDUAL, EPI_SCATTER = 0, 1, 2, 3, 4, 5
DEV_TIMEOUT = 1


class LigerError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"liger error {code}: {msg}")
        self.code = code


class GemmArgs(C.Structure):
    _fields_ = [
        ("a", C.c_void_p), ("wt", C.c_void_p), ("c", C.c_void_p), ("bias", C.c_void_p),
        ("residual", C.c_void_p), ("q_out", C.c_void_p), ("k_out", C.c_void_p), ("v_out", C.c_void_p),
        ("m", C.c_int), ("n", C.c_int), ("k", C.c_int),
        ("lda", C.c_int), ("ldw", C.c_int), ("ldc", C.c_int), ("ldr", C.c_int),
        ("n_begin", C.c_int), ("n_end", C.c_int), ("epilogue", C.c_int),
        ("seq_len", C.c_int), ("heads", C.c_int), ("head_dim", C.c_int),
        ("kv_stride", C.c_int), ("kv_pos", C.c_int),
        ("scatter_comm", C.c_void_p), ("scatter_off", C.c_size_t),
        ("gather_comm", C.c_void_p), ("gather_channel", C.c_int),
    ]


_P, _I, _F, _U32, _SZ = C.c_void_p, C.c_int, C.c_float, C.c_uint32, C.c_size_t


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("max_batch_size", "max_seq_len", "head_num", "size_per_head", "layer_num",
                                       "kernel_num", "factor", "rq_interval", "graph", "act", "ffn_inner", "causal")] + \
               [("seed", C.c_uint32), ("num_requests", C.c_int), ("ignore_num", C.c_int), ("schedule_deep", C.c_int),
                ("contention", C.c_float), ("poisson", C.c_int), ("min_seq_len", C.c_int), ("seq_round", C.c_int),
                ("workspace_slots", C.c_int), ("kv_capacity", C.c_int), ("min_slice_efficiency", C.c_float)]


class ServingMetrics(C.Structure):
    _fields_ = [("records", C.c_int), ("launch_errors", C.c_int), ("total_duration_ms", C.c_double),
                ("throughput_samples_s", C.c_double), ("average_latency_ms", C.c_double), ("tokens_per_s", C.c_double),
                ("p50_latency_ms", C.c_double), ("p99_latency_ms", C.c_double), ("mean_gpu_ms", C.c_double),
                ("tokens", C.c_longlong), ("segments", C.c_longlong), ("secondary_launches", C.c_longlong),
                ("decompositions", C.c_longlong)]


class SimKernel(C.Structure):
    _fields_ = [("type", C.c_int), ("duration_ms", C.c_float)]


class SimLaunch(C.Structure):
    _fields_ = [("request", C.c_int), ("layer", C.c_int), ("name", C.c_int), ("stream", C.c_int),
                ("units_begin", C.c_int), ("units_end", C.c_int), ("duration_ms", C.c_float),
                ("t_start_ms", C.c_double), ("t_end_ms", C.c_double)]


BCAST_INT_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(C.c_int))
BARRIER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p)
MODE_PROFILE, MODE_SCHEDULE, MODE_NO_SCHEDULE = 0, 1, 2
GRAPH_REF, GRAPH_PRELN = 0, 1
ACT_GELU, ACT_GEGLU = 0, 1
COMMUNICATION, COMPUTATION, GEMM = 0, 1, 2

# name -> (restype, argtypes); must list every function declared in include/liger_b200.h
SIGNATURES = {
    "liger_last_error": (C.c_char_p, []),
    "liger_version": (C.c_char_p, []),
    "liger_device_status": (_I, [C.POINTER(C.c_uint * 4)]),
    "liger_device_status_clear": (_I, []),
    "liger_set_wait_budget_ms": (_I, [_I]),
    "liger_fill_normal": (_I, [_P, _I, _I, _I, _I, _I, _I, _U32, _U32, _F, _F, _I, _P]),
    "liger_gemm_fp16": (_I, [C.POINTER(GemmArgs), _P]),
    "liger_transpose_weight": (_I, [_P, _P, _I, _I, _I, _P]),
    "liger_attention_prefill": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P]),
    "liger_attention_decode_scratch_bytes": (_SZ, [_I, _I, _I, _I]),
    "liger_attention_decode": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "liger_attention_decode_noalloc_max_bytes": (_SZ, []),
    "liger_attention_decode_noalloc": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "liger_layernorm": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "liger_add_bias_input_layernorm": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _P]),
    "liger_add_bias_gelu": (_I, [_P, _P, _I, _I, _P]),
    "liger_add_qkv_bias_transpose": (_I, [_P] * 9 + [_I] * 4 + [_P]),
    "liger_transpose_heads": (_I, [_P, _P, _I, _I, _I, _I, _P]),
    "liger_comm_create": (_I, [C.POINTER(_P), _I, _I, _SZ, _I]),
    "liger_comm_export": (_I, [_P, _P]),
    "liger_comm_connect": (_I, [_P, _P]),
    "liger_comm_destroy": (_I, [_P]),
    "liger_comm_data": (_P, [_P]),
    "liger_comm_data_bytes": (_SZ, [_P]),
    "liger_comm_timing": (_I, [_P, _I, _I, C.POINTER(C.c_double * 4)]),
    "liger_comm_rank": (_I, [_P]),
    "liger_comm_world_size": (_I, [_P]),
    "liger_comm_channels": (_I, [_P]),
    "liger_allgather_ce": (_I, [_P, _I, _SZ, _I, _I, _I, _I, _P]),
    "liger_allgather_push": (_I, [_P, _I, _I, _SZ, _I, _I, _P]),
    "liger_allreduce_ce": (_I, [_P, _I, _SZ, _SZ, _SZ, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "liger_gemm_smallm_plan": (_I, [_I, _I, _I, C.POINTER(C.c_int)]),
    "liger_allreduce_fused": (_I, [_P, _I, _SZ, _SZ, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "liger_model_config_init": (None, [C.POINTER(ModelConfig)]),
    "liger_model_comm_bytes": (_SZ, [C.POINTER(ModelConfig), _I]),
    "liger_model_create": (_I, [C.POINTER(_P), C.POINTER(ModelConfig), _I, _I, _P]),
    "liger_model_destroy": (_I, [_P]),
    "liger_model_forward": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "liger_model_forward_host": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "liger_model_set_mask": (_I, [_P, _P]),
    "liger_model_set_micro_batches": (_I, [_P, _I]),
    "liger_model_set_overlap": (_I, [_P, _I]),
    "liger_model_overlap_times": (_I, [_P, C.POINTER(C.c_double * 4)]),
    "liger_model_set_output_sharding": (_I, [_P, _I]),
    "liger_model_decode": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "liger_model_fill_kv_cache": (_I, [_P]),
    "liger_model_timeline": (_I, [_P, _I, _I, C.POINTER(_I), C.POINTER(_I), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "liger_model_set_kernel_timing": (_I, [_P, _I]),
    "liger_model_kernel_times": (_I, [_P, C.POINTER(C.c_double * 9), C.POINTER(C.c_longlong * 9)]),
    "liger_model_kernel_work": (_I, [_P, _I, _I, _I, C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "liger_serve": (_I, [_P, _I, BCAST_INT_FN, BARRIER_FN, _P, C.c_char_p, _I, C.POINTER(ServingMetrics)]),
    "liger_profile_rewrite": (_I, [C.c_char_p, C.c_char_p, _I, C.POINTER(_I), C.POINTER(C.c_double)]),
    "liger_profile_predict": (_I, [C.c_char_p, _I, _I, _I, _I, _I, C.POINTER(C.c_double)]),
    "liger_sim_serve": (_I, [C.POINTER(ModelConfig), C.POINTER(SimKernel), _I, _I, C.c_double, C.c_double,
                             C.POINTER(SimLaunch), _I, C.POINTER(_I), C.POINTER(ServingMetrics)]),
    "liger_sim_serve_rank": (_I, [C.POINTER(ModelConfig), C.POINTER(SimKernel), _I, _I, C.c_double, C.c_double, _I, _I,
                                  BCAST_INT_FN, BARRIER_FN, _P, C.c_double, C.c_double,
                                  C.POINTER(SimLaunch), _I, C.POINTER(_I), C.POINTER(ServingMetrics)]),
}
COMM_HANDLE_BYTES = 128


def default_config(**kw):
    """ModelConfig with the reference's defaults (src/main.cu:14-21), overridden by keyword."""
    cfg = ModelConfig()
    lib().liger_model_config_init(C.byref(cfg))
    for k, v in kw.items():
        if not hasattr(cfg, k):
            raise AttributeError(k)
        setattr(cfg, k, v)
    return cfg

_lib = None


def lib():
    """The loaded CUDA library.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LigerError(-2, f"{LIB_PATH} is missing: build it with build_all() (nvcc, sm_100a); there is no CPU path")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    """Raise LigerError for a negative return code."""
    if rc < 0:
        raise LigerError(rc, lib().liger_last_error().decode())
    return rc
