"""ctypes binding of libcinn_b200.so.  There is no fallback: a missing library is an error."""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcinn_b200.so")

CINN_B200_OK = 0
LOWER_FUNC_PTR_G = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p)

_lib = None


class CinnB200Error(RuntimeError):
    """A call into libcinn_b200.so returned a negative status."""

    def __init__(self, code, message):
        super().__init__("cinn_b200 error %d: %s" % (code, message))
        self.code = code
        self.message = message


def lib():
    """The loaded library (loads it on first use).  Raises if it was not built: run `python -m cinn_b200.build`."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                "libcinn_b200.so is missing (%s). Build it with `python -m cinn_b200.build`; "
                "there is no CPU or PyTorch fallback for the fused-group kernels." % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, ci, cs, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_longlong
        L.cinn_b200_last_error.restype = cs
        L.cinn_b200_last_error.argtypes = []
        L.cinn_call_cuda_kernel.restype = None
        L.cinn_call_cuda_kernel.argtypes = [vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]
        L.cinn_b200_call_cuda_kernel_ex.restype = ci
        L.cinn_b200_call_cuda_kernel_ex.argtypes = [vp, vp, ci, ci, ci, ci, ci, ci, ci, ctypes.c_uint,
                                                    ctypes.c_size_t, vp]
        L.cinn_b200_get_kernel.restype = vp
        L.cinn_b200_get_kernel.argtypes = [cs]
        L.cinn_b200_num_kernels.restype = ci
        L.cinn_b200_num_kernels.argtypes = []
        L.cinn_b200_kernel_name.restype = cs
        L.cinn_b200_kernel_name.argtypes = [ci]
        L.cinn_b200_kernel_num_params.restype = ci
        L.cinn_b200_kernel_num_params.argtypes = [cs]
        L.cinn_b200_launch_count.restype = ll
        L.cinn_b200_launch_count.argtypes = []
        L.cinn_b200_compile_group.restype = ci
        L.cinn_b200_compile_group.argtypes = [cs, ctypes.POINTER(vp)]
        L.cinn_b200_lookup.restype = vp
        L.cinn_b200_lookup.argtypes = [cs]
        L.cinn_b200_release_group.restype = ci
        L.cinn_b200_release_group.argtypes = [cs]
        L.cinn_b200_group_run.restype = ci
        L.cinn_b200_group_run.argtypes = [cs, vp, ci, vp]
        L.cinn_b200_group_info.restype = ci
        L.cinn_b200_group_info.argtypes = [cs, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ll),
                                           ctypes.POINTER(ll), ctypes.POINTER(ci), ctypes.POINTER(ll)]
        L.cinn_b200_group_kernel.restype = ci
        L.cinn_b200_group_kernel.argtypes = [cs, ci, ctypes.c_char_p, ctypes.c_size_t]
        L.cinn_b200_group_launch_text.restype = ll
        L.cinn_b200_group_launch_text.argtypes = [cs, ctypes.c_char_p, ctypes.c_size_t]
        L.cinn_b200_num_static_chains.restype = ci
        L.cinn_b200_num_static_chains.argtypes = []
        L.cinn_b200_canonical_expr.restype = ci
        L.cinn_b200_canonical_expr.argtypes = [cs, ctypes.c_char_p, ctypes.c_size_t]
        L.cinn_b200_group_run_host.restype = ci
        L.cinn_b200_group_run_host.argtypes = [cs, vp, ci, ci]
        L.cinn_b200_builder_create.restype = vp
        L.cinn_b200_builder_create.argtypes = [cs]
        L.cinn_b200_builder_destroy.restype = None
        L.cinn_b200_builder_destroy.argtypes = [vp]
        L.cinn_b200_builder_create_input.restype = ci
        L.cinn_b200_builder_create_input.argtypes = [vp, cs, ctypes.POINTER(ll), ci, cs, ctypes.c_char_p,
                                                     ctypes.c_size_t]
        L.cinn_b200_builder_add_op.restype = ci
        L.cinn_b200_builder_add_op.argtypes = [vp, cs, ctypes.POINTER(cs), ci, cs, ctypes.c_char_p, ctypes.c_size_t]
        L.cinn_b200_builder_var_info.restype = ci
        L.cinn_b200_builder_var_info.argtypes = [vp, cs, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ll),
                                                 ctypes.POINTER(ci)]
        L.cinn_b200_computation_build_and_compile.restype = vp
        L.cinn_b200_computation_build_and_compile.argtypes = [vp, ci, ctypes.POINTER(cs), ci]
        L.cinn_b200_computation_destroy.restype = None
        L.cinn_b200_computation_destroy.argtypes = [vp]
        L.cinn_b200_computation_execute.restype = ci
        L.cinn_b200_computation_execute.argtypes = [vp, vp]
        L.cinn_b200_computation_set_tensor_data.restype = ci
        L.cinn_b200_computation_set_tensor_data.argtypes = [vp, cs, vp, ctypes.c_size_t]
        L.cinn_b200_computation_get_tensor_data.restype = ci
        L.cinn_b200_computation_get_tensor_data.argtypes = [vp, cs, vp, ctypes.c_size_t]
        L.cinn_b200_computation_bind_tensor.restype = ci
        L.cinn_b200_computation_bind_tensor.argtypes = [vp, cs, vp]
        L.cinn_b200_computation_num_tensors.restype = ci
        L.cinn_b200_computation_num_tensors.argtypes = [vp]
        L.cinn_b200_computation_tensor_name.restype = cs
        L.cinn_b200_computation_tensor_name.argtypes = [vp, ci]
        L.cinn_b200_computation_tensor_info.restype = ci
        L.cinn_b200_computation_tensor_info.argtypes = [vp, cs, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ll),
                                                        ctypes.POINTER(ci), ctypes.POINTER(vp)]
        L.cinn_b200_computation_num_groups.restype = ci
        L.cinn_b200_computation_num_groups.argtypes = [vp]
        L.cinn_b200_computation_group_desc.restype = ci
        L.cinn_b200_computation_group_desc.argtypes = [vp, ci, ctypes.c_char_p, ctypes.c_size_t]
        L.cinn_b200_computation_group_pattern.restype = ci
        L.cinn_b200_computation_group_pattern.argtypes = [vp, ci, ctypes.c_char_p, ctypes.c_size_t]
        L.cinn_b200_col_reduce_f32_static_scratch.restype = ci
        L.cinn_b200_col_reduce_f32_static_scratch.argtypes = [ci, vp, vp, ll, ll, ll, vp]
        L.cinn_b200_peer_create.restype = ci
        L.cinn_b200_peer_create.argtypes = [ci, ci, ll, ctypes.c_char_p, ctypes.POINTER(vp)]
        L.cinn_b200_peer_connect.restype = ci
        L.cinn_b200_peer_connect.argtypes = [vp, ctypes.c_char_p]
        L.cinn_b200_peer_destroy.restype = ci
        L.cinn_b200_peer_destroy.argtypes = [vp]
        L.cinn_b200_peer_close_imports.restype = ci
        L.cinn_b200_peer_close_imports.argtypes = [vp]
        L.cinn_b200_peer_status.restype = ci
        L.cinn_b200_peer_status.argtypes = [vp, ctypes.POINTER(ci)]
        L.cinn_b200_peer_create_emulated.restype = ci
        L.cinn_b200_peer_create_emulated.argtypes = [ci, ll, ctypes.POINTER(vp)]
        L.cinn_b200_col_reduce_sharded_f32_emulated.restype = ci
        L.cinn_b200_col_reduce_sharded_f32_emulated.argtypes = [vp, ci, ctypes.POINTER(vp), ll, ll,
                                                                ctypes.POINTER(vp), ci, vp]
        L.cinn_b200_col_reduce_sharded_f32_emulated_ranks.restype = ci
        L.cinn_b200_col_reduce_sharded_f32_emulated_ranks.argtypes = [vp, ci, ctypes.POINTER(vp), ll, ll,
                                                                      ctypes.POINTER(vp), ci, ci, ci, vp]
        L.cinn_b200_col_reduce_sharded_f32.restype = ci
        L.cinn_b200_col_reduce_sharded_f32.argtypes = [vp, ci, vp, ll, ll, vp, ci, vp]
        L.cinn_b200_device_status.restype = ci
        L.cinn_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        L.cinn_b200_group_host_chunks.restype = ci
        L.cinn_b200_group_host_chunks.argtypes = [cs]
        L.cinn_b200_set_option.restype = ci
        L.cinn_b200_set_option.argtypes = [cs, ll]
        _lib = L
    return _lib


def check(status):
    """Raise CinnB200Error for a negative status."""
    if status != CINN_B200_OK:
        raise CinnB200Error(status, lib().cinn_b200_last_error().decode())
    return status
