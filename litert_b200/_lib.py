"""ctypes binding of the C ABI (include/litert_b200.h). Fails loudly when the library is missing."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "liblitert_b200.so")

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i32 = ctypes.c_int32
_sz = ctypes.c_size_t
_f = ctypes.c_float

# name -> (restype, argtypes); mirrors include/litert_b200.h one to one
SIGNATURES = {
    "b200_abi_version": (_i, []),
    "b200_last_error": (ctypes.c_char_p, []),
    "b200_zero_workspace_bytes": (_sz, []),
    "b200_zero_workspace_init": (_i, [_vp, _vp]),
    "b200_fc_scratch_bytes": (_sz, [_i, _i]),
    "b200_read_status": (_i, [_vp, _vp, ctypes.POINTER(_i)]),
    "b200_set_wait_budget": (_i, [_vp, ctypes.c_ulonglong, _vp]),
    "b200_clear_status": (_i, [_vp, _vp]),
    "b200_measure_int8_tensor_peak": (_i, [_i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]),
    "b200_packed_w8_bytes": (_sz, [_i, _i]),
    "b200_pack_w8": (_i, [_vp, _i, _i, _vp, _vp, _vp]),
    "b200_packed_w4_bytes": (_sz, [_i, _i]),
    "b200_pack_w4": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "b200_quantize_rows": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_fc_int8": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp, _i32, _i32, _i32, _vp, _vp, _i, _i32, _i32, _vp, _vp, _vp,
                          _sz, _vp]),
    "b200_fc_hybrid": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "b200_bmm_hybrid": (_i, [_vp, _i, _i, _vp, _i, _vp, _vp, _i, _i, _vp, _vp, _vp, _sz, _vp]),
    "b200_sdpa": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _sz, _vp]),
    "b200_transpose_matrices": (_i, [_vp, _vp, _i, _i, _i, _i, _vp]),
    "b200_fc_w4": (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "b200_sdpa_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "b200_sdpa_rows_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "b200_sdpa_rows": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _sz, _vp]),
    "b200_sdpa_decode": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _sz,
                              _vp]),
    "b200_sdpa_static_workspace_limit": (_sz, []),
    "b200_sdpa_decode_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp]),
    "b200_sdpa_static_last_error": (ctypes.c_char_p, []),
    "b200_glue_last_error": (ctypes.c_char_p, []),
    "b200_tiled_rows_bytes": (_sz, [_i, _i]),
    "b200_untile_rows": (_i, [_vp, _i, _i, _vp, _vp]),
    "b200_embedding_lookup": (_i, [_vp, _i, _vp, _vp, _i, _i, _f, _vp, _vp]),
    "b200_add_rmsnorm_quantize": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp, _vp, _vp, _vp]),
    "b200_geglu_quantize": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_rope_table": (_i, [_vp, _i, _i, _f]),
    "b200_rope_kv_append": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp]),
    "b200_argmax_workspace_bytes": (_sz, [_i]),
    "b200_argmax_rows": (_i, [_vp, _i, _i, _f, _vp, _vp, _sz, _vp]),
    "b200_lm_head_workspace_bytes": (_sz, [_i]),
    "b200_lm_head_greedy": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _f, _vp, _vp, _vp, _sz, _vp, _vp]),
    "b200_attention_step_supported": (_i, [_i, _i, _i, _i]),
    "b200_attention_step": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp]),
    "b200_sdpa_decode_quantized": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp,
                                        _vp, _sz, _vp]),
    "b200_sdpa_decode_quantized_masked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _vp,
                                               _vp, _vp, _vp, _sz, _vp]),
    "b200_fc_hybrid_quantized": (_i, [_vp, _vp, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp]),
    "b200_elementwise_last_error": (ctypes.c_char_p, []),
    "b200_binary_f32": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "b200_gelu_f32": (_i, [_vp, _vp, _sz, _i, _vp]),
    "b200_box_copy": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp]),
    "b200_rms_norm_f32": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "b200_kv_cache_update_f32": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_rope_f32": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "b200_rope_kv_cache_update_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "b200_widen_i32_to_i64": (_i, [_vp, _vp, _i, _vp]),
    "b200_decoder_create": (_i, [_vp, _vp, ctypes.POINTER(_vp)]),
    "b200_decoder_destroy": (None, [_vp]),
    "b200_decoder_set_layer": (_i, [_vp, _i, _vp]),
    "b200_decoder_set_embedding": (_i, [_vp, _vp, _vp, _vp]),
    "b200_decoder_set_allreduce": (_i, [_vp, _vp, _vp]),
    "b200_nccl_unique_id": (_i, [_vp, _sz]),
    "b200_decoder_init_nccl": (_i, [_vp, _vp]),
    "b200_decoder_exchange_handle": (_i, [_vp, _vp, _sz]),
    "b200_decoder_connect_peers": (_i, [_vp, _vp, _sz]),
    "b200_decoder_exchange_bytes": (_sz, [_vp]),
    "b200_decoder_exchange_buffer": (_vp, [_vp]),
    "b200_decoder_connect_peer_pointers": (_i, [_vp, _vp]),
    "b200_decoder_set_wait_budget": (_i, [_vp, ctypes.c_ulonglong]),
    "b200_decoder_clear_fault": (_i, [_vp]),
    "b200_decoder_reset": (_i, [_vp]),
    "b200_decoder_set_logit_soft_cap": (_i, [_vp, _f]),
    "b200_decoder_set_positions": (_i, [_vp, _vp, _i]),
    "b200_decoder_step": (_i, [_vp, _vp, _i, _vp, _vp]),
    "b200_decoder_run": (_i, [_vp, _vp, _i, _i, _vp]),
    "b200_decoder_prefill": (_i, [_vp, _i, _vp, _i, _vp]),
    "b200_decoder_launches_per_step": (_i, [_vp]),
    "b200_decoder_profile_step": (_i, [_vp, _vp, _i, _vp, _vp]),
    "b200_decoder_time_gemv": (_i, [_vp, _i, _i, _vp, _vp]),
    "b200_decoder_last_error": (ctypes.c_char_p, []),
}


class DecoderConfig(ctypes.Structure):
    """b200_decoder_config of include/litert_b200.h."""
    _fields_ = [(n, _i) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "d_ff", "vocab",
                                  "max_seq", "max_batch")] + \
               [(n, _f) for n in ("rms_eps", "rope_base", "embed_scale")] + \
               [(n, _i) for n in ("kv_dtype", "tp_size", "tp_rank")]


class DecoderLayerWeights(ctypes.Structure):
    """b200_decoder_layer_weights of include/litert_b200.h (device pointers)."""
    _fields_ = [(n, _vp) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "sq", "sk", "sv", "so", "sgate",
                                   "sup", "sdown", "norm1", "norm2")]

_lib = None


class B200Error(RuntimeError):
    pass


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200Error(
                f"{LIB_PATH} is missing: build it with `python -m litert_b200.build` "
                "(there is no CPU fallback in this package)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the export is missing
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise B200Error(f"litert_b200 error {rc}: {load().b200_last_error().decode()}")
