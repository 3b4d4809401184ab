"""ctypes bindings to a polygrad-compatible shared library.

The same binding set drives two libraries:

* ``polygrad_b200/lib/libpolygrad_b200.so`` -- polygrad's own frontend and
  scheduler linked against this repository's sm_100a backend (the product), and
* a stock polygrad build (CPU backend), which tests use as the checker.

Only the calls the execution path needs are declared; signatures follow
polygrad ``src/frontend.h``, ``src/scheduler.h``, ``src/instance.h``,
``src/model_mlp.h``, ``src/modelzoo/modelzoo.h`` and, for the CUDA runtime
symbols, ``src/codegen.h:126-137`` (the way ``py/polygrad/_ffi.py:539-554``
binds them).
"""
import ctypes
import os

_ptr = ctypes.c_void_p
_i64p = ctypes.POINTER(ctypes.c_int64)

# polygrad PolyDeviceId (src/exec_plan.h:28-36)
DEVICE_AUTO, DEVICE_CPU, DEVICE_INTERP, DEVICE_CUDA = 0, 1, 2, 3
OPTIM_NONE, OPTIM_SGD, OPTIM_ADAM, OPTIM_ADAMW = 0, 1, 2, 3      # src/instance.h:39-42

# polygrad instance buffer roles (src/instance.h:33-37)
ROLE_PARAM, ROLE_INPUT, ROLE_TARGET, ROLE_OUTPUT, ROLE_AUX = 0, 1, 2, 3, 4

# dtype ids accepted by poly_buffer_by_id / poly_cast_by_id (src/frontend.c:124-146)
DTYPE_IDS = {'bool': 1, 'int8': 2, 'uint8': 3, 'int16': 4, 'uint16': 5, 'int32': 6,
             'uint32': 7, 'int64': 8, 'uint64': 9, 'float16': 10, 'bfloat16': 11,
             'float32': 12, 'float64': 13}


class PolyBufferHandle(ctypes.Structure):
    _fields_ = [('ptr', _ptr), ('nbytes', ctypes.c_size_t),
                ('domain', ctypes.c_int), ('owned', ctypes.c_bool)]


class PolyBufferBinding(ctypes.Structure):
    _fields_ = [('buffer', _ptr), ('handle', PolyBufferHandle)]


class PolyIOBinding(ctypes.Structure):
    _fields_ = [('name', ctypes.c_char_p), ('data', ctypes.POINTER(ctypes.c_float))]


class GPT2Config(ctypes.Structure):
    _fields_ = [('vocab_size', ctypes.c_int), ('n_embd', ctypes.c_int),
                ('n_head', ctypes.c_int), ('n_layer', ctypes.c_int),
                ('max_seq_len', ctypes.c_int), ('norm_eps', ctypes.c_float)]


class PolyB200Stats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in (
        'launches', 'launches_precompiled', 'launches_generated', 'memsets_elided',
        'memsets_executed', 'bytes_allocated', 'programs_compiled', 'programs_cached', 'bytes_htod', 'bytes_dtoh')]


_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
PRODUCT_LIB = os.path.join(_PKG_DIR, 'lib', 'libpolygrad_b200.so')
KERNEL_LIB = os.path.join(_PKG_DIR, 'lib', 'libpolyb200.so')


def _sig(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def _declare_frontend(lib):
    P, I, D = _ptr, ctypes.c_int, ctypes.c_double
    _sig(lib, 'poly_ctx_new', P, [])
    _sig(lib, 'poly_ctx_destroy', None, [P])
    _sig(lib, 'poly_const_float', P, [P, D])
    _sig(lib, 'poly_alu1', P, [P, I, P])
    _sig(lib, 'poly_alu2', P, [P, I, P, P])
    _sig(lib, 'poly_alu3', P, [P, I, P, P, P])
    _sig(lib, 'poly_op_count', I, [])
    _sig(lib, 'poly_op_name', ctypes.c_char_p, [I])
    _sig(lib, 'poly_store_val', P, [P, P, P])
    _sig(lib, 'poly_sink1', P, [P, P])
    _sig(lib, 'poly_sink_n', P, [P, ctypes.POINTER(P), I])
    _sig(lib, 'poly_buffer_f32', P, [P, ctypes.c_int64])
    _sig(lib, 'poly_buffer_by_id', P, [P, ctypes.c_int64, I])
    _sig(lib, 'poly_cast_by_id', P, [P, P, I])
    _sig(lib, 'poly_realize', I, [P, P, ctypes.POINTER(PolyBufferBinding), I])
    _sig(lib, 'poly_reshape', P, [P, P, _i64p, I])
    _sig(lib, 'poly_expand', P, [P, P, _i64p, I])
    _sig(lib, 'poly_permute', P, [P, P, _i64p, I])
    _sig(lib, 'poly_shrink', P, [P, P, _i64p, I])
    _sig(lib, 'poly_pad', P, [P, P, _i64p, I])
    _sig(lib, 'poly_flip', P, [P, P, _i64p, I])
    for name in ('poly_exp', 'poly_log', 'poly_sin', 'poly_sigmoid', 'poly_tanh_act', 'poly_relu',
                 'poly_gelu', 'poly_abs', 'poly_square', 'poly_rsqrt', 'poly_silu'):
        _sig(lib, name, P, [P, P])
    for name in ('poly_sum_reduce', 'poly_max_reduce', 'poly_mean_reduce'):
        _sig(lib, name, P, [P, P, _i64p, I, I, I, _i64p, ctypes.POINTER(I)])
    _sig(lib, 'poly_var_reduce', P, [P, P, _i64p, I, I, I, I, _i64p, ctypes.POINTER(I)])
    _sig(lib, 'poly_dot', P, [P, P, _i64p, I, P, _i64p, I, _i64p, ctypes.POINTER(I)])
    _sig(lib, 'poly_softmax', P, [P, P, _i64p, I, I])
    _sig(lib, 'poly_layernorm', P, [P, P, _i64p, I, I, D, _i64p, ctypes.POINTER(I)])
    _sig(lib, 'poly_gather', P, [P, P, _i64p, I, P, _i64p, I, _i64p, ctypes.POINTER(I)])
    _sig(lib, 'poly_where_op', P, [P, P, P, P])
    _sig(lib, 'poly_eq', P, [P, P, P])
    _sig(lib, 'poly_maximum', P, [P, P, P])
    # instances
    _sig(lib, 'poly_instance_free', None, [P])
    _sig(lib, 'poly_instance_param_count', I, [P])
    _sig(lib, 'poly_instance_param_name', ctypes.c_char_p, [P, I])
    _sig(lib, 'poly_instance_param_data', ctypes.POINTER(ctypes.c_float), [P, I, _i64p])
    _sig(lib, 'poly_instance_param_shape', I, [P, I, _i64p, I])
    _sig(lib, 'poly_instance_buf_count', I, [P])
    _sig(lib, 'poly_instance_buf_name', ctypes.c_char_p, [P, I])
    _sig(lib, 'poly_instance_buf_role', I, [P, I])
    _sig(lib, 'poly_instance_buf_shape', I, [P, I, _i64p, I])
    _sig(lib, 'poly_instance_buf_data', ctypes.POINTER(ctypes.c_float), [P, I, _i64p])
    _sig(lib, 'poly_instance_set_device', I, [P, I])
    _sig(lib, 'poly_instance_readback_buf', I, [P, I, P, ctypes.c_size_t])
    _sig(lib, 'poly_instance_upload_buf', I, [P, I, P, ctypes.c_size_t])
    _sig(lib, 'poly_instance_upload_param', I, [P, I, P, ctypes.c_size_t])
    _sig(lib, 'poly_instance_forward', I, [P, ctypes.POINTER(PolyIOBinding), I])
    _sig(lib, 'poly_instance_call', I, [P, ctypes.c_char_p, ctypes.POINTER(PolyIOBinding), I])
    _sig(lib, 'poly_instance_readback_param', I, [P, I, P, ctypes.c_size_t])
    _sig(lib, 'poly_instance_set_optimizer', I, [P, I, ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_float])
    _sig(lib, 'poly_instance_train_step', I, [P, ctypes.POINTER(PolyIOBinding), I, ctypes.POINTER(ctypes.c_float)])
    _sig(lib, 'poly_instance_value_and_grad', I, [P, ctypes.c_char_p, ctypes.POINTER(PolyIOBinding), I, ctypes.POINTER(ctypes.c_float)])
    _sig(lib, 'poly_instance_export_weights', ctypes.POINTER(ctypes.c_ubyte), [P, ctypes.POINTER(I)])
    _sig(lib, 'poly_instance_import_weights', I, [P, ctypes.c_char_p, I])
    _sig(lib, 'poly_mlp_instance', P, [ctypes.c_char_p, I])
    _sig(lib, 'poly_gpt2_build', P, [ctypes.POINTER(GPT2Config), I])


def _declare_cuda(lib):
    U, S = ctypes.c_ulonglong, ctypes.c_size_t
    _sig(lib, 'poly_cuda_init', ctypes.c_int, [])
    _sig(lib, 'poly_cuda_available', ctypes.c_bool, [])
    _sig(lib, 'poly_cuda_alloc', U, [S])
    _sig(lib, 'poly_cuda_free', None, [U])
    _sig(lib, 'poly_cuda_copy_htod', ctypes.c_int, [U, _ptr, S])
    _sig(lib, 'poly_cuda_copy_dtoh', ctypes.c_int, [_ptr, U, S])
    _sig(lib, 'poly_cuda_sync', ctypes.c_int, [])
    _sig(lib, 'poly_cuda_memset', ctypes.c_int, [U, ctypes.c_ubyte, S])
    _sig(lib, 'poly_compile_cuda', _ptr, [ctypes.c_char_p, ctypes.c_char_p])
    _sig(lib, 'poly_cuda_launch', ctypes.c_int, [_ptr, ctypes.POINTER(_ptr), ctypes.c_int] + [ctypes.c_int] * 6)
    _sig(lib, 'poly_cuda_program_destroy', None, [_ptr])
    _sig(lib, 'poly_b200_set_device', ctypes.c_int, [ctypes.c_int])
    _sig(lib, 'poly_b200_device', ctypes.c_int, [])
    _sig(lib, 'poly_b200_synchronize', ctypes.c_int, [])
    _sig(lib, 'poly_b200_stream', _ptr, [])
    _sig(lib, 'poly_b200_trim', None, [])
    _sig(lib, 'poly_b200_pool_free_sizes', ctypes.c_int, [ctypes.POINTER(U), ctypes.c_int])
    _sig(lib, 'poly_b200_note_access', ctypes.c_int, [_ptr, ctypes.c_char])
    _sig(lib, 'poly_b200_timing_begin', None, [])
    _sig(lib, 'poly_b200_timing_end', ctypes.c_double, [ctypes.POINTER(ctypes.c_int)])
    _sig(lib, 'poly_b200_timing_active', ctypes.c_int, [])
    LL = ctypes.c_longlong
    _sig(lib, 'poly_b200_gemm', ctypes.c_int, [LL, LL, LL, _ptr, LL, LL, _ptr, LL, LL, _ptr, LL, _ptr,
                                               ctypes.c_int, ctypes.c_int])
    _sig(lib, 'poly_b200_gemm_ex', ctypes.c_int, [LL, LL, LL, _ptr, LL, LL, _ptr, LL, LL, _ptr, LL, _ptr,
                                                  ctypes.c_int, ctypes.c_int])
    _sig(lib, 'poly_b200_gemm_noalloc', ctypes.c_int, [LL, LL, LL, _ptr, LL, LL, _ptr, LL, LL, _ptr, LL, _ptr, ctypes.c_int])
    _sig(lib, 'poly_b200_selftest_bounded_wait', ctypes.c_int, [])
    _sig(lib, 'poly_b200_instance_import_weights', ctypes.c_int,
         [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_longlong, ctypes.POINTER(ctypes.c_longlong)])
    _sig(lib, 'poly_b200_attention', ctypes.c_int, [_ptr, _ptr, _ptr, _ptr, ctypes.c_float, _ptr, ctypes.c_int, ctypes.c_int, ctypes.c_int])
    _sig(lib, 'poly_b200_set_gemm_policy', None, [ctypes.c_int])
    _sig(lib, 'poly_b200_gemm_policy', ctypes.c_int, [])
    _sig(lib, 'poly_b200_host_alloc', _ptr, [S])
    _sig(lib, 'poly_b200_host_free', None, [_ptr])
    _sig(lib, 'poly_b200_last_dtoh_src', U, [])
    _sig(lib, 'poly_b200_copy_rows', ctypes.c_int, [U, U, S, S, S])
    _sig(lib, 'poly_b200_readback_defer', ctypes.c_int, [ctypes.c_int])
    _sig(lib, 'poly_b200_comm_unique_id', ctypes.c_int, [_ptr, S])
    _sig(lib, 'poly_b200_comm_init', ctypes.c_int, [ctypes.c_int, ctypes.c_int, _ptr, S])
    _sig(lib, 'poly_b200_comm_rank', ctypes.c_int, [])
    _sig(lib, 'poly_b200_comm_world', ctypes.c_int, [])
    _sig(lib, 'poly_b200_gather_offset', S, [ctypes.c_int, S])
    _sig(lib, 'poly_b200_gather_async', ctypes.c_int, [_ptr, S, _ptr, ctypes.c_int])
    _sig(lib, 'poly_b200_comm_join', ctypes.c_int, [])
    _sig(lib, 'poly_b200_comm_wait', ctypes.c_int, [])
    _sig(lib, 'poly_b200_comm_max', ctypes.c_int, [ctypes.POINTER(ctypes.c_double)])
    _sig(lib, 'poly_b200_comm_destroy', None, [])
    _sig(lib, 'poly_b200_set_update_averaging', None, [ctypes.c_int])
    _sig(lib, 'poly_b200_update_averaging', ctypes.c_int, [])
    _sig(lib, 'poly_b200_average_enqueue', ctypes.c_int, [_ptr, S])
    _sig(lib, 'poly_b200_average_join', ctypes.c_int, [])
    _sig(lib, 'poly_b200_average_group_bytes', None, [S])
    _sig(lib, 'poly_b200_average_trace', None, [ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong)])
    _sig(lib, 'poly_b200_shard_micro_index', ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int])
    _sig(lib, 'poly_b200_forward_microbatches', ctypes.c_int,
         [_ptr, ctypes.c_char_p, ctypes.POINTER(ctypes.POINTER(ctypes.c_float)), ctypes.c_int, ctypes.c_int, S, _ptr,
          ctypes.c_int, ctypes.c_int])
    _sig(lib, 'poly_b200_readback_wait', ctypes.c_int, [])
    _sig(lib, 'poly_b200_kernels_cut', ctypes.c_longlong, [])
    _sig(lib, 'poly_realize_cuda', ctypes.c_int, [_ptr, _ptr, ctypes.POINTER(PolyBufferBinding), ctypes.c_int])
    _sig(lib, 'poly_cuda_copyback', ctypes.c_int, [ctypes.POINTER(PolyBufferBinding), ctypes.c_int])
    _sig(lib, 'poly_cuda_flush_buffers', None, [])
    _sig(lib, 'poly_cuda_prog_cache_flush', None, [])
    _sig(lib, 'poly_b200_eager_stats', None, [ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_ulonglong),
                                              ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)])
    _sig(lib, 'poly_b200_event_create', _ptr, [])
    _sig(lib, 'poly_b200_event_record', ctypes.c_int, [_ptr])
    _sig(lib, 'poly_b200_event_elapsed_ms', ctypes.c_float, [_ptr, _ptr])
    _sig(lib, 'poly_b200_event_destroy', None, [_ptr])
    _sig(lib, 'poly_b200_stats', None, [ctypes.POINTER(PolyB200Stats)])
    _sig(lib, 'poly_b200_stats_reset', None, [])
    _sig(lib, 'poly_b200_last_error', ctypes.c_char_p, [])


class Library:
    """A loaded polygrad-compatible library with declared signatures."""

    def __init__(self, path, has_cuda):
        if not os.path.isfile(path):
            raise FileNotFoundError(
                f'{path} is missing: build it first (python -c "import __graft_entry__ as g; g.build()")')
        self.path = path
        self.has_cuda = has_cuda
        self.c = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        _declare_frontend(self.c)
        if has_cuda:
            _declare_cuda(self.c)
        self.ops = {}
        for i in range(self.c.poly_op_count() + 8):
            name = self.c.poly_op_name(i)
            if name:
                self.ops[name.decode()] = i

    def __getattr__(self, name):
        return getattr(self.c, name)

    def stats(self):
        st = PolyB200Stats()
        self.c.poly_b200_stats(ctypes.byref(st))
        return {n: getattr(st, n) for n, _ in PolyB200Stats._fields_}

    def eager_stats(self):
        """Counters of the eager entry point: calls that found a kept plan, calls that compiled one,
        plans kept now, results now left on the device."""
        hits, misses = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        kept, resident = ctypes.c_int(), ctypes.c_int()
        self.c.poly_b200_eager_stats(ctypes.byref(hits), ctypes.byref(misses), ctypes.byref(kept), ctypes.byref(resident))
        return dict(hits=hits.value, misses=misses.value, plans_kept=kept.value, buffers_resident=resident.value)

    def last_error(self):
        return self.c.poly_b200_last_error().decode(errors='replace')


_product = None


def product():
    """The product library: polygrad frontend + this repository's sm_100a backend.

    Raises if the library has not been built; there is no fallback."""
    global _product
    if _product is None:
        _product = Library(PRODUCT_LIB, has_cuda=True)
    return _product


def load_reference(path):
    """A stock polygrad build (CPU backend only); used by tests as the checker."""
    return Library(path, has_cuda=False)
