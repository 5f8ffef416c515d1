"""ctypes binding of the C ABI in include/qmm.h.  There is no fallback: if
``libqmm.so`` is missing the import of any operator raises."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libqmm.so")

Q8_0, Q8_1, Q4_K, Q6_K = 8, 9, 12, 14
BLOCK_ELEMS = {Q8_0: 32, Q8_1: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q8_1: 36, Q4_K: 144, Q6_K: 210}
TYPE_NAMES = {Q8_0: "q8_0", Q8_1: "q8_1", Q4_K: "q4_k", Q6_K: "q6_k"}

vp, i32, i64 = C.c_void_p, C.c_int, C.c_long

class MatvecJob(C.Structure):
    """qmm_matvec_job of include/qmm.h."""
    _fields_ = [("type", C.c_int), ("n", C.c_int), ("k", C.c_int), ("w", C.c_void_p), ("xq", C.c_void_p), ("y", C.c_void_p),
                ("y_stride", C.c_long), ("select", C.c_void_p), ("select_stride_bytes", C.c_long), ("tp_sum", C.c_int)]


class GgufTensorInfo(C.Structure):
    """qmm_gguf_tensor of include/qmm_gguf.h."""
    _fields_ = [("name", C.c_char * 128), ("type", C.c_int), ("n_dims", C.c_int), ("dims", C.c_long * 4), ("file_offset", C.c_long),
                ("bytes", C.c_long)]


class StoreStats(C.Structure):
    """qmm_store_stats_t of include/qmm_store.h."""
    _fields_ = [(n, C.c_long) for n in ("vram_bytes", "ram_bytes", "disk_bytes", "fetches_vram", "fetches_ram", "fetches_disk", "cache_hits",
                                        "staged_bytes")]


# name -> (restype, argtypes); must list every symbol include/qmm.h declares
SIGNATURES = {
    "qmm_status_string": (C.c_char_p, [i32]),
    "qmm_last_cuda_error": (i32, []),
    "qmm_device_status": (i32, [C.POINTER(i32)]),
    "qmm_row_bytes": (i64, [i32, i64]),
    "qmm_set_overlap": (i32, [i32]),
    "qmm_tune": (i32, [C.c_char_p, i32]),
    "launch_quantize_q8_1": (i32, [vp, vp, i32, i32, vp]),
    "launch_quantize_q8_0": (i32, [vp, vp, i64, i32, vp]),
    "launch_quantize_q4_k": (i32, [vp, vp, i64, i32, vp]),
    "launch_quantize_q6_k": (i32, [vp, vp, i64, i32, vp]),
    "launch_dequantize_q8_0_f32": (i32, [vp, vp, i64, vp]),
    "launch_dequantize_q4_k_f32": (i32, [vp, vp, i64, vp]),
    "launch_dequantize_q6_k_f32": (i32, [vp, vp, i64, vp]),
    "launch_dequantize_q8_0_bf16": (i32, [vp, vp, i64, vp]),
    "launch_dequantize_q4_k_bf16": (i32, [vp, vp, i64, vp]),
    "launch_dequantize_q6_k_bf16": (i32, [vp, vp, i64, vp]),
    "launch_qmatvec_q8_0": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_qmatvec_q4_k": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_qmatvec_q6_k": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_qmatvec": (i32, [i32, vp, vp, vp, i32, i32, i32, vp]),
    "launch_qmatvec_pitched": (i32, [i32, vp, i64, vp, vp, i32, i32, i32, vp]),
    "launch_qmatvec_batch": (i32, [C.POINTER(MatvecJob), i32, i32, vp]),
    "qmm_tp_comm_create": (i32, [i32, i32, i64, C.POINTER(vp)]),
    "qmm_tp_comm_destroy": (i32, [vp]),
    "qmm_tp_comm_export": (i32, [vp, vp]),
    "qmm_tp_comm_import": (i32, [vp, i32, vp]),
    "qmm_tp_comm_ready": (i32, [vp]),
    "launch_qmatvec_tp": (i32, [vp, i32, vp, vp, vp, i32, i32, i32, vp]),
    "launch_qmatvec_batch_tp": (i32, [vp, C.POINTER(MatvecJob), i32, i32, vp]),
    "launch_norm_qmatvec_batch": (i32, [vp, vp, vp, vp, C.c_float, C.POINTER(MatvecJob), i32, i32, vp]),
    "launch_glu_qmatvec_batch": (i32, [vp, i32, C.POINTER(MatvecJob), i32, i32, vp]),
    "launch_qgemm_q4_k_bf16": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_qgemm_q4_k_bf16_f32acc": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "qmm_attn_decode_scratch_bytes": (i64, [i32, i32, i32, i32]),
    "launch_attn_decode": (i32, [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
    "launch_attn_decode_static": (i32, [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]),
    "launch_qblock_dots": (i32, [i32, vp, vp, vp, i32, i32, vp]),
    "launch_add_rmsnorm_q8_1": (i32, [vp, vp, vp, vp, vp, i32, i32, C.c_float, vp]),
    "launch_rope_kv_append": (i32, [vp, vp, vp, i32, i32, i32, i32, i32, i32, C.c_float, vp]),
    "launch_glu_act_q8_1": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_embed_rows": (i32, [i32, vp, vp, vp, i32, i32, i32, vp]),
    "qmm_argmax_scratch_bytes": (i64, [i32]),
    "launch_argmax_rows": (i32, [vp, vp, vp, vp, i32, i32, vp]),
    "launch_scale_f32": (i32, [vp, C.c_float, i64, vp]),
    "launch_gemm_bt_bf16": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_gemm_bt_bf16_f32acc": (i32, [vp, vp, vp, i32, i32, i32, vp]),
    "launch_attn_prefill": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, C.c_float, vp]),
    "launch_attn_prefill_f16kv": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, C.c_float, vp]),
    "launch_attn_prefill_f16kv_at": (i32, [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, C.c_float, vp]),
    "qmm_qdense_scratch_bytes": (i64, [i32, i32, i32]),
    "launch_qdense": (i32, [i32, vp, vp, vp, vp, vp, i32, i32, i32, i32, C.c_float, vp]),
    "launch_moe_router_topk": (i32, [vp, vp, vp, i32, i32, i32, i32, C.c_float, C.c_float, vp, vp, vp, vp]),
    "qmm_moe_scratch_bytes": (i64, [i32, i32, i32, i32]),
    "launch_moe_experts": (i32, [i32, vp, i64, i32, vp, i64, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]),
    "qmm_store_create": (i32, [i64, i64, i64, i32, i64, C.POINTER(vp)]),
    "qmm_store_destroy": (i32, [vp]),
    "qmm_store_place_host": (i32, [vp, C.c_char_p, vp, i64]),
    "qmm_store_place_file": (i32, [vp, C.c_char_p, C.c_char_p, i64, i64]),
    "qmm_store_home": (i32, [vp, C.c_char_p]),
    "qmm_store_stats": (i32, [vp, C.POINTER(StoreStats)]),
    "qmm_store_fetch": (i32, [vp, C.c_char_p, vp, C.POINTER(vp)]),
    "qmm_store_prefetch": (i32, [vp, C.c_char_p, vp]),
    "qmm_store_fetch_cached": (i32, [vp, C.c_char_p, vp, C.POINTER(vp)]),
    "qmm_gguf_open": (i32, [C.c_char_p, C.POINTER(vp)]),
    "qmm_gguf_close": (i32, [vp]),
    "qmm_gguf_tensor_count": (i64, [vp]),
    "qmm_gguf_find": (i64, [vp, C.c_char_p]),
    "qmm_gguf_tensor_info": (i32, [vp, i64, C.POINTER(GgufTensorInfo)]),
    "qmm_gguf_read_tensor": (i32, [vp, i64, vp, i64]),
    "qmm_gguf_upload_tensor": (i32, [vp, i64, vp, i64, vp]),
    "qmm_gguf_meta_u64": (i32, [vp, C.c_char_p, C.POINTER(C.c_ulonglong)]),
    "qmm_gguf_meta_f64": (i32, [vp, C.c_char_p, C.POINTER(C.c_double)]),
    "qmm_gguf_meta_str": (i64, [vp, C.c_char_p, C.c_char_p, i64]),
    "qmm_gguf_writer_create": (i32, [C.c_char_p, C.POINTER(vp)]),
    "qmm_gguf_writer_meta_u32": (i32, [vp, C.c_char_p, C.c_uint]),
    "qmm_gguf_writer_meta_f32": (i32, [vp, C.c_char_p, C.c_float]),
    "qmm_gguf_writer_meta_str": (i32, [vp, C.c_char_p, C.c_char_p]),
    "qmm_gguf_writer_add_tensor": (i32, [vp, C.c_char_p, i32, i32, C.POINTER(C.c_long), vp, i64]),
    "qmm_gguf_writer_finish": (i32, [vp]),
}

_lib = None


class QmmError(RuntimeError):
    def __init__(self, status, what):
        msg = lib().qmm_status_string(status).decode()
        extra = f" (cudaError {lib().qmm_last_cuda_error()})" if status == -6 else ""
        super().__init__(f"{what}: {msg}{extra} [status {status}]")
        self.status = status


def lib():
    """The loaded library.  Raises if it has not been built (python -m nates_recipe_rs_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m nates_recipe_rs_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status, what):
    if status != 0:
        raise QmmError(status, what)
