"""ctypes binding of libferrograd_b200.so (the C ABI declared in include/ferrograd_b200.h).

There is no fallback: if the shared library is missing the import fails with an
explicit error, and every compute call runs a CUDA kernel.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libferrograd_b200.so")

c_ctx = C.c_void_p
c_buf = C.c_void_p
c_plan = C.c_void_p
c_dev = C.c_void_p   # raw device pointer
u32, u64, i32, f32 = C.c_uint32, C.c_uint64, C.c_int32, C.c_float

STATUS = {0: "FG_OK", 1: "FG_ERR_INVALID_ARGUMENT", 2: "FG_ERR_OUT_OF_MEMORY", 3: "FG_ERR_INVALID_DEVICE",
          4: "FG_ERR_LAUNCH_FAILURE", 5: "FG_ERR_SYNC", 6: "FG_ERR_FAILED_BUFFER_COPY",
          7: "FG_ERR_UNSUPPORTED_FEATURE", 8: "FG_ERR_NOT_INITIALIZED", 9: "FG_ERR_INTERNAL",
          10: "FG_ERR_PEER_ACCESS", 11: "FG_ERR_TIMEOUT", 12: "FG_ERR_INCONSISTENT_CAPTURE"}


class AdamWHyper(C.Structure):
    _fields_ = [("lr", f32), ("beta1", f32), ("beta2", f32), ("eps", f32), ("weight_decay", f32)]


class UpdateTensor(C.Structure):
    _fields_ = [("w", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p), ("w_pairs", C.c_void_p),
                ("pairs_stride", C.c_uint64), ("n", C.c_uint64)]


class EwInstr(C.Structure):
    _fields_ = [("op", i32), ("a", i32), ("b", i32), ("imm", f32)]


# name -> (restype, argtypes); the single source of truth for the Python side and for the
# test that checks the library exports everything the header declares.
SIGNATURES = {
    "fg_ctx_create": (i32, [i32, C.POINTER(c_ctx)]),
    "fg_ctx_create_on_stream": (i32, [i32, C.c_void_p, C.POINTER(c_ctx)]),
    "fg_ctx_destroy": (i32, [c_ctx]),
    "fg_sync": (i32, [c_ctx]),
    "fg_is_ready": (i32, [c_ctx, C.POINTER(i32)]),
    "fg_last_error": (C.c_char_p, [c_ctx]),
    "fg_ctx_stream": (C.c_void_p, [c_ctx]),
    "fg_ctx_device": (i32, [c_ctx]),
    "fg_ctx_launch_count": (u64, [c_ctx]),
    "fg_ctx_reserve_workspace": (i32, [c_ctx, u64]),
    "fg_ctx_workspace_bytes": (u64, [c_ctx]),
    "fg_ctx_set_option": (i32, [c_ctx, C.c_char_p, C.c_char_p]),
    "fg_selftest_bounded_wait": (i32, [c_ctx, u32]),
    "fg_ctx_device_status": (i32, [c_ctx, C.POINTER(i32)]),
    "fg_ctx_timing_enable": (i32, [c_ctx, i32]),
    "fg_ctx_timing_read": (i32, [c_ctx, i32, C.POINTER(u64), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "fg_alloc": (i32, [c_ctx, u64, C.POINTER(c_buf)]),
    "fg_alloc_zeroed": (i32, [c_ctx, u64, C.POINTER(c_buf)]),
    "fg_alloc_init": (i32, [c_ctx, C.c_void_p, u64, C.POINTER(c_buf)]),
    "fg_free": (i32, [c_ctx, c_buf]),
    "fg_buf_size_bytes": (u64, [c_buf]),
    "fg_buf_device_ptr": (C.c_void_p, [c_buf]),
    "fg_upload": (i32, [c_ctx, c_buf, C.c_void_p, u64, u64]),
    "fg_download": (i32, [c_ctx, c_buf, C.c_void_p, u64, u64]),
    "fg_copy": (i32, [c_ctx, c_buf, c_buf]),
    "fg_buf_touch": (i32, [c_buf]),
    "fg_upload_async": (i32, [c_ctx, c_dev, C.c_void_p, u64]),
    "fg_download_async": (i32, [c_ctx, C.c_void_p, c_dev, u64]),
    "fg_upload_prefetch": (i32, [c_ctx, c_dev, C.c_void_p, u64]),
    "fg_prefetch_wait": (i32, [c_ctx]),
    "fg_prefetch_mark": (i32, [c_ctx]),
    "fg_copy_dev_async": (i32, [c_ctx, c_dev, c_dev, u64]),
    "fg_host_alloc_pinned": (i32, [u64, C.POINTER(C.c_void_p)]),
    "fg_host_free_pinned": (i32, [C.c_void_p]),
    "fg_memset_zero": (i32, [c_ctx, c_dev, u64]),
    "fg_gemm_f32": (i32, [c_ctx, i32, i32, i32, u32, u32, u32, c_dev, c_dev, c_dev, c_dev, i32, c_dev]),
    "fg_gemm_bwd_f32": (i32, [c_ctx, i32, u32, u32, u32, c_dev, c_dev, c_dev, i32, c_dev, c_dev, c_dev, c_dev, c_dev]),
    "fg_gemm_bwd_exchange_f32": (i32, [c_ctx, i32, u32, u32, u32, c_dev, c_dev, c_dev, i32, c_dev, c_dev, c_dev, c_dev, c_dev,
                                       u64]),
    "fg_pairs_from_f32": (i32, [c_ctx, c_dev, u64, c_dev, u64]),
    "fg_gemm_paired_f32": (i32, [c_ctx, u32, u32, u32, c_dev, c_dev, u64, c_dev, c_dev, u64, c_dev, c_dev, i32, c_dev,
                                 c_dev, u64]),
    "fg_gemm_bwd_paired_f32": (i32, [c_ctx, u32, u32, u32, c_dev, c_dev, u64, c_dev, c_dev, u64, c_dev, c_dev, u64,
                                     c_dev, c_dev, c_dev, i32, c_dev, c_dev, u64, c_dev, c_dev, u64]),
    "fg_gemm_batched_f32": (i32, [c_ctx, i32, u32, u32, u32, u32, c_dev, u64, c_dev, u64, c_dev, u64, c_dev, i32, c_dev]),
    "fg_gemm_batched_bwd_f32": (i32, [c_ctx, i32, u32, u32, u32, u32, c_dev, u64, c_dev, u64, c_dev, u64, i32, c_dev,
                                      c_dev, c_dev]),
    "fg_bias_act_fwd": (i32, [c_ctx, u32, u32, c_dev, c_dev, i32, c_dev]),
    "fg_act_bwd": (i32, [c_ctx, u64, i32, c_dev, c_dev, c_dev]),
    "fg_softmax_fwd": (i32, [c_ctx, u32, u32, c_dev, c_dev]),
    "fg_softmax_bwd": (i32, [c_ctx, u32, u32, c_dev, c_dev, c_dev, i32]),
    "fg_softmax_ce_fwd_bwd": (i32, [c_ctx, c_dev, c_dev, u32, u32, f32, c_dev, c_dev, c_dev, c_dev, c_dev]),
    "fg_ce_loss_grad": (i32, [c_ctx, c_dev, c_dev, u32, u32, c_dev, c_dev]),
    "fg_sum_f32": (i32, [c_ctx, c_dev, u64, c_dev]),
    "fg_mse_loss_grad": (i32, [c_ctx, c_dev, c_dev, u64, f32, c_dev, c_dev, c_dev]),
    "fg_bce_loss_grad": (i32, [c_ctx, c_dev, c_dev, u64, f32, c_dev, c_dev, c_dev]),
    "fg_mse_loss_grad_noalloc": (i32, [c_ctx, c_dev, c_dev, u64, f32, c_dev, c_dev, c_dev]),
    "fg_sgd_step": (i32, [c_ctx, c_dev, c_dev, u64, f32, f32, i32]),
    "fg_adamw_step": (i32, [c_ctx, c_dev, c_dev, c_dev, c_dev, u64, C.POINTER(AdamWHyper), u32, c_dev, f32, i32]),
    "fg_sgd_step_paired": (i32, [c_ctx, c_dev, c_dev, u64, f32, f32, i32, c_dev, u64]),
    "fg_adamw_step_paired": (i32, [c_ctx, c_dev, c_dev, c_dev, c_dev, u64, C.POINTER(AdamWHyper), u32, c_dev, f32, i32,
                                   c_dev, u64]),
    "fg_adamw_step_multi": (i32, [c_ctx, C.POINTER(UpdateTensor), u32, C.POINTER(AdamWHyper), u32, c_dev, f32, i32]),
    "fg_sgd_step_multi": (i32, [c_ctx, C.POINTER(UpdateTensor), u32, f32, f32, i32]),
    "fg_counter_increment": (i32, [c_ctx, c_dev]),
    "fg_eltwise_chain_fwd": (i32, [c_ctx, u64, C.POINTER(EwInstr), i32, C.POINTER(C.c_void_p), i32, c_dev,
                                   C.POINTER(C.c_void_p)]),
    "fg_eltwise_chain_bwd": (i32, [c_ctx, u64, C.POINTER(EwInstr), i32, C.POINTER(C.c_void_p), i32, c_dev,
                                   C.POINTER(C.c_void_p), i32]),
    "fg_eltwise_chain_fwd_dt": (i32, [c_ctx, i32, u64, C.POINTER(EwInstr), i32, C.POINTER(C.c_void_p), i32, c_dev,
                                      C.POINTER(C.c_void_p)]),
    "fg_eltwise_chain_bwd_dt": (i32, [c_ctx, i32, u64, C.POINTER(EwInstr), i32, C.POINTER(C.c_void_p), i32, c_dev,
                                      C.POINTER(C.c_void_p), i32]),
    "fg_gemm_lowp": (i32, [c_ctx, i32, u32, u32, u32, c_dev, c_dev, c_dev, c_dev, i32, c_dev]),
    "fg_gemm_bwd_lowp": (i32, [c_ctx, i32, u32, u32, u32, c_dev, c_dev, c_dev, i32, c_dev, c_dev, c_dev, c_dev]),
    "fg_convert": (i32, [c_ctx, c_dev, i32, c_dev, i32, u64]),
    "fg_graph_create": (i32, [i32, i32, C.POINTER(C.c_void_p)]),
    "fg_graph_destroy": (i32, [C.c_void_p]),
    "fg_graph_node_count": (i32, [C.c_void_p]),
    "fg_graph_input": (i32, [C.c_void_p, C.POINTER(u32), u32, C.POINTER(i32)]),
    "fg_graph_input_dt": (i32, [C.c_void_p, C.POINTER(u32), u32, i32, C.POINTER(i32)]),
    "fg_graph_constant_f32": (i32, [C.c_void_p, f32, C.POINTER(i32)]),
    "fg_graph_op": (i32, [C.c_void_p, i32, i32, i32, C.POINTER(i32)]),
    "fg_exec_create": (i32, [c_ctx, C.c_void_p, C.POINTER(u32), u32, i32, C.POINTER(C.c_void_p)]),
    "fg_exec_destroy": (i32, [C.c_void_p]),
    "fg_exec_set_adamw": (i32, [C.c_void_p, C.POINTER(AdamWHyper)]),
    "fg_exec_bind": (i32, [C.c_void_p, C.POINTER(c_buf), u32, C.c_char_p]),
    "fg_exec_dispatch_forward": (i32, [C.c_void_p]),
    "fg_exec_dispatch_backward": (i32, [C.c_void_p]),
    "fg_exec_dispatch_loss": (i32, [C.c_void_p, c_buf]),
    "fg_exec_dispatch_optim": (i32, [C.c_void_p]),
    "fg_exec_dispatch_single_optim": (i32, [C.c_void_p, c_buf, u32]),
    "fg_exec_forward_out": (c_buf, [C.c_void_p]),
    "fg_exec_seed": (c_buf, [C.c_void_p]),
    "fg_exec_loss_t": (c_buf, [C.c_void_p]),
    "fg_exec_loss_sum": (c_buf, [C.c_void_p]),
    "fg_exec_num_saved": (u32, [C.c_void_p]),
    "fg_exec_saved": (c_buf, [C.c_void_p, u32, C.POINTER(i32)]),
    "fg_exec_num_grads": (u32, [C.c_void_p]),
    "fg_exec_grad": (c_buf, [C.c_void_p, u32, C.POINTER(i32)]),
    "fg_exec_forward_steps": (u32, [C.c_void_p]),
    "fg_exec_plans_active": (i32, [C.c_void_p]),
    "fg_bpat_save": (i32, [c_ctx, C.c_char_p, i32, u32, C.POINTER(c_buf), C.POINTER(u32),
                           C.POINTER(C.POINTER(u32))]),
    "fg_bpat_open": (i32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "fg_bpat_close": (i32, [C.c_void_p]),
    "fg_bpat_format": (i32, [C.c_void_p]),
    "fg_bpat_dtype": (i32, [C.c_void_p]),
    "fg_bpat_count": (u32, [C.c_void_p]),
    "fg_bpat_shape": (i32, [C.c_void_p, u32, C.POINTER(u32), C.POINTER(u32)]),
    "fg_bpat_load_tensor": (i32, [c_ctx, C.c_void_p, u32, C.POINTER(c_buf)]),
    "fg_plan_begin": (i32, [c_ctx]),
    "fg_plan_end": (i32, [c_ctx, C.POINTER(c_plan)]),
    "fg_plan_launch": (i32, [c_ctx, c_plan]),
    "fg_plan_destroy": (i32, [c_plan]),
    "fg_comm_unique_id": (i32, [C.c_void_p]),
    "fg_comm_init": (i32, [c_ctx, i32, i32, C.c_void_p]),
    "fg_allreduce_sum_f32": (i32, [c_ctx, c_dev, u64]),
    "fg_comm_join": (i32, [c_ctx]),
    "fg_comm_sync": (i32, [c_ctx, u32]),
    "fg_comm_abort": (i32, [c_ctx]),
    "fg_comm_checkpoint": (i32, [c_ctx, i32]),
    "fg_comm_wait": (i32, [c_ctx, i32]),
    "fg_comm_destroy": (i32, [c_ctx]),
    "fg_version": (C.c_char_p, []),
}

_lib = None


def load():
    """Loads the shared library and types every entry point.  Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ferrograd_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
