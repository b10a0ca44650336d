"""modelspec_b200: a B200 (sm_100a) CUDA backend for ModelSpec's compiled training step.

The product is the shared library `libmsx.so` beside this file (C ABI in `include/msx.h`). This
module is a thin ctypes binding of that ABI for tests, the benchmark and Python hosts; it holds
no arithmetic. There is no CPU fallback: without the library, or without a B200, every call that
would compute raises.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmsx.so")

OK, BAD_ARGUMENT, NO_DEVICE, OUT_OF_MEMORY, UNSUPPORTED, LAUNCH_FAILED, NON_FINITE, TIMEOUT, BAD_INPUT = range(9)
PLAN_DEFAULT, PLAN_NO_GRAPH, PLAN_EXACT_MATMUL, PLAN_BF16, PLAN_GUARD = 0, 1, 2, 4, 8

STATUS_NAMES = ["MSX_OK", "MSX_BAD_ARGUMENT", "MSX_NO_DEVICE", "MSX_OUT_OF_MEMORY", "MSX_UNSUPPORTED",
                "MSX_LAUNCH_FAILED", "MSX_NON_FINITE", "MSX_TIMEOUT", "MSX_BAD_INPUT"]


class MsxError(RuntimeError):
    def __init__(self, status, message):
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__("%s: %s" % (name, message))
        self.status = status
        self.message = message


class Stats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "launches_per_step", "nodes", "live_nodes", "arena_bytes", "unshared_bytes", "param_bytes",
        "upload_bytes_per_step", "steps_run", "algorithmic_bytes_per_step", "matmul_flop_per_step")]


# Every function include/msx.h declares: name -> (restype, argtypes).
_P = C.c_void_p
SIGNATURES = {
    "msx_open": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "msx_close": (None, [_P]),
    "msx_last_error": (C.c_char_p, [_P]),
    "msx_plan_create": (C.c_int, [_P, C.c_char_p, C.c_uint64, C.c_uint32, _P, C.POINTER(_P)]),
    "msx_plan_destroy": (None, [_P]),
    "msx_plan_input_count": (C.c_uint32, [_P]),
    "msx_plan_input_name": (C.c_char_p, [_P, C.c_uint32]),
    "msx_plan_input_bytes": (C.c_uint64, [_P, C.c_uint32]),
    "msx_plan_input_is_i32": (C.c_int, [_P, C.c_uint32]),
    "msx_plan_param_count": (C.c_uint32, [_P]),
    "msx_plan_param_path": (C.c_char_p, [_P, C.c_uint32]),
    "msx_plan_param_bytes": (C.c_uint64, [_P, C.c_uint32]),
    "msx_param_upload": (C.c_int, [_P, C.c_uint32, _P, C.c_uint64]),
    "msx_param_download": (C.c_int, [_P, C.c_uint32, _P, C.c_uint64]),
    "msx_moment_upload": (C.c_int, [_P, C.c_uint32, C.c_char, _P, C.c_uint64]),
    "msx_moment_download": (C.c_int, [_P, C.c_uint32, C.c_char, _P, C.c_uint64]),
    "msx_set_input": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64]),
    "msx_set_shard": (C.c_int, [_P, C.c_uint64, C.c_uint64]),
    "msx_run": (C.c_int, [_P]),
    "msx_loss": (C.c_int, [_P, C.POINTER(C.c_float), C.c_uint32]),
    "msx_sync": (C.c_int, [_P, C.c_uint32]),
    "msx_loss_of": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_float), C.c_uint32]),
    "msx_steps_submitted": (C.c_uint64, [_P]),
    "msx_step_ms": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_float)]),
    "msx_comm_exposed_ms": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "msx_profile_step": (C.c_int, [_P, C.POINTER(C.c_float), C.c_uint32]),
    "msx_profile_step_repeated": (C.c_int, [_P, C.c_uint32, C.POINTER(C.c_float), C.c_uint32]),
    "msx_launch_kernel": (C.c_char_p, [_P, C.c_uint32]),
    "msx_launch_bytes": (C.c_uint64, [_P, C.c_uint32]),
    "msx_launch_flop": (C.c_uint64, [_P, C.c_uint32]),
    "msx_training_loss_of": (C.c_int, [_P, C.c_uint64, C.POINTER(C.c_float)]),
    "msx_value_download": (C.c_int, [_P, C.c_uint32, _P, C.c_uint64]),
    "msx_plan_stats": (C.c_int, [_P, C.POINTER(Stats)]),
    "msx_plan_check_guards": (C.c_int, [_P]),
    "msx_plan_describe": (C.c_uint64, [_P, C.c_char_p, C.c_uint64]),
    "msx_schedule_describe": (C.c_uint64, [C.c_char_p, C.c_char_p, C.c_uint64]),
    "msx_schedule_describe_with": (C.c_uint64, [C.c_char_p, C.c_uint32, C.c_char_p, C.c_uint64]),
    "msx_elapsed_ms": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "msx_comm_unique_id": (C.c_int, [_P]),
    "msx_comm_init": (C.c_int, [_P, C.c_int, C.c_int, _P]),
    "msx_comm_bucket_count": (C.c_uint32, [_P]),
    "msx_comm_uses_peer_memory": (C.c_uint32, [_P]),
    "msx_peer_reduce_check": (C.c_int, [_P, C.c_uint32, C.c_uint64, _P, C.c_float, C.c_int, C.c_uint32, _P]),
    "msx_comm_share": (C.c_int, [_P, _P]),
    "msx_training_comm_init": (C.c_int, [_P, C.c_int, C.c_int, _P, C.c_uint64]),
    "msx_training_create": (C.c_int, [_P, C.c_char_p, C.c_uint64, C.c_uint32, C.POINTER(_P)]),
    "msx_training_destroy": (None, [_P]),
    "msx_training_step_plan": (_P, [_P]),
    "msx_training_forward_plan": (_P, [_P]),
    "msx_training_steps": (C.c_uint64, [_P]),
    "msx_training_seed": (C.c_uint64, [_P]),
    "msx_training_last_error": (C.c_char_p, [_P]),
    "msx_training_set_input": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64]),
    "msx_training_synthetic": (C.c_int, [_P]),
    "msx_training_get_input": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64]),
    "msx_training_step": (C.c_int, [_P, C.c_uint64, C.c_uint64]),
    "msx_training_loss": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "msx_training_final_loss": (C.c_int, [_P, C.POINTER(C.c_float)]),
    "msx_training_check_finite": (C.c_int, [_P]),
    "msx_training_prediction_count": (C.c_uint64, [_P]),
    "msx_training_infer": (C.c_int, [_P, _P, C.c_uint64, C.POINTER(C.c_float)]),
    "msx_training_infer_report": (C.c_uint64, [_P, C.c_char_p, C.c_uint64]),
    "msx_op_heldout_rows": (C.c_int, [_P, C.c_uint64, _P, _P, C.c_uint64, C.c_uint64, _P, _P, _P]),
    "msx_heldout_create": (C.c_int, [_P, C.c_uint32, C.c_uint32, C.POINTER(_P)]),
    "msx_heldout_destroy": (None, [_P]),
    "msx_heldout_targets": (C.c_int, [_P, C.c_uint32, _P, _P, C.c_uint64]),
    "msx_heldout_begin": (C.c_int, [_P]),
    "msx_heldout_add": (C.c_int, [_P, C.c_uint32]),
    "msx_heldout_sums": (C.c_int, [_P, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.c_uint32]),
    "msx_training_heldout_begin": (C.c_int, [_P, C.c_uint32, C.c_char_p, C.c_char_p]),
    "msx_training_heldout_set": (C.c_int, [_P, C.c_uint32, C.c_char_p, _P, C.c_uint64]),
    "msx_training_heldout_evaluate": (C.c_int, [_P, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "msx_dense_open": (C.c_int, [C.c_char_p, C.c_uint32, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                 C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.c_uint64, C.POINTER(_P)]),
    "msx_dense_close": (None, [_P]),
    "msx_dense_last_error": (C.c_char_p, [_P]),
    "msx_dense_batch": (C.c_uint64, [_P]),
    "msx_dense_samples": (C.c_uint64, [_P]),
    "msx_dense_has_order": (C.c_int, [_P]),
    "msx_dense_tensors": (C.c_uint32, [_P]),
    "msx_dense_batch_bytes": (C.c_uint64, [_P, C.c_uint32]),
    "msx_dense_check_bound": (C.c_int, [_P, C.c_uint32, C.c_uint64, C.c_char_p]),
    "msx_dense_step": (C.c_int, [_P, C.c_uint32, C.c_uint64, C.c_void_p, C.c_uint64]),
    "msx_dense_open_eval": (C.c_int, [C.c_char_p, C.c_uint32, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                      C.POINTER(C.c_uint32), C.POINTER(C.c_uint64), C.POINTER(_P)]),
    "msx_dense_eval_batch": (C.c_int, [_P, C.c_uint32, C.c_uint64, C.c_void_p, C.c_uint64]),
    "msx_training_eval_dense": (C.c_int, [_P, C.c_char_p, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "msx_training_eval_line": (C.c_uint64, [C.c_double, C.c_double, C.c_int, C.c_char_p, C.c_uint64]),
    "msx_training_bind_dense": (C.c_int, [_P, C.c_char_p]),
    "msx_training_feed_dense": (C.c_int, [_P, C.c_uint64]),
    "msx_packed_open": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "msx_packed_close": (None, [_P]),
    "msx_packed_last_error": (C.c_char_p, [_P]),
    "msx_packed_seq_len": (C.c_uint64, [_P]),
    "msx_packed_vocabulary": (C.c_uint64, [_P]),
    "msx_packed_sequences": (C.c_uint64, [_P, C.c_int]),
    "msx_packed_binding_id": (C.c_char_p, [_P]),
    "msx_packed_epoch_order": (C.c_int, [_P, C.c_uint64, C.c_uint64, _P, C.c_uint64]),
    "msx_packed_batch": (C.c_int, [_P, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, _P, _P, _P, _P, _P]),
    "msx_training_bind_packed": (C.c_int, [_P, _P]),
    "msx_training_feed_packed": (C.c_int, [_P, C.c_uint64]),
    "msx_training_heldout_packed": (C.c_int, [_P, C.c_char_p]),
    "msx_training_heldout_batches": (C.c_uint32, [_P]),
    "msx_checkpoint_new": (C.c_int, [C.c_uint64, C.c_uint64, C.c_char_p, C.POINTER(_P)]),
    "msx_checkpoint_destroy": (None, [_P]),
    "msx_checkpoint_last_error": (C.c_char_p, [_P]),
    "msx_checkpoint_set_optimizer": (C.c_int, [_P, C.c_int, C.c_double, C.c_double, C.c_double, C.c_double, C.c_double, C.c_uint64]),
    "msx_checkpoint_add": (C.c_int, [_P, C.c_char_p, C.c_char_p, _P, C.c_uint32, _P]),
    "msx_checkpoint_encode": (C.c_uint64, [_P, _P, C.c_uint64]),
    "msx_checkpoint_write": (C.c_int, [_P, C.c_char_p]),
    "msx_checkpoint_read": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "msx_checkpoint_step": (C.c_uint64, [_P]),
    "msx_checkpoint_seed": (C.c_uint64, [_P]),
    "msx_checkpoint_schema_hash": (C.c_char_p, [_P]),
    "msx_checkpoint_id": (C.c_char_p, [_P]),
    "msx_checkpoint_optimizer": (C.c_int, [_P, C.POINTER(C.c_int)] + [C.POINTER(C.c_double)] * 5 + [C.POINTER(C.c_uint64)]),
    "msx_checkpoint_optimizer_json": (C.c_uint64, [_P, C.c_char_p, C.c_uint64]),
    "msx_checkpoint_count": (C.c_uint32, [_P, C.c_int]),
    "msx_checkpoint_path": (C.c_char_p, [_P, C.c_int, C.c_uint32]),
    "msx_checkpoint_slot": (C.c_char_p, [_P, C.c_int, C.c_uint32]),
    "msx_checkpoint_rank": (C.c_uint32, [_P, C.c_int, C.c_uint32]),
    "msx_checkpoint_shape": (C.POINTER(C.c_uint64), [_P, C.c_int, C.c_uint32]),
    "msx_checkpoint_data": (C.POINTER(C.c_float), [_P, C.c_int, C.c_uint32]),
    "msx_training_checkpoint": (C.c_int, [_P, C.c_uint64, C.POINTER(_P)]),
    "msx_training_resume": (C.c_int, [_P, _P, C.POINTER(C.c_uint64)]),
    "msx_training_schema_hash": (C.c_char_p, [_P]),
    "msx_state_snapshot": (C.c_int, [_P]),
    "msx_state_restore": (C.c_int, [_P]),
    "msx_training_set_replay_window": (C.c_int, [_P, C.c_uint32]),
    "msx_training_rewind": (C.c_int, [_P, C.c_uint64]),
    "msx_packed_data_line": (C.c_uint64, [_P, C.c_char_p, C.c_uint64]),
    "msx_training_run": (C.c_int, [_P, C.c_uint64, C.c_uint64]),
    "msx_training_report": (C.c_uint64, [_P, C.c_char_p, C.c_uint64]),
    "msx_plan_run_stats": (C.c_int, [_P, _P]),
    "msx_stats_report": (C.c_uint64, [_P, C.c_char_p, C.c_uint64]),
    "msx_profile_report": (C.c_uint64, [_P, _P, C.c_uint32, C.c_char_p, C.c_uint64]),
    "msx_op_matmul": (C.c_int, [_P, C.c_int, _P, C.c_int, _P, C.c_uint64, C.c_uint64, C.c_uint64, _P, C.c_uint64, _P, _P, C.c_int]),
    "msx_op_matmul_workspace": (C.c_uint64, [C.c_uint64, C.c_uint64, C.c_uint64]),
    "msx_op_matmul_bf16": (C.c_int, [_P, C.c_int, _P, C.c_int, _P, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, _P, C.c_uint64, _P, _P]),
    "msx_op_matmul_bf16_workspace": (C.c_uint64, [C.c_uint64, C.c_uint64, C.c_uint64]),
    "msx_op_attention_bf16": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _P, _P]),
    "msx_sum_rows_static": (C.c_int, [_P, C.c_uint64, C.c_uint64, _P, _P]),
    "msx_static_last_error": (C.c_char_p, []),
    "msx_compile": (C.c_uint64, [C.c_char_p, C.c_char_p, C.c_uint64, C.c_char_p, C.c_uint64]),
    "msx_compile_function": (C.c_uint64, [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_uint64]),
    "msx_training_create_function": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.c_uint32, C.POINTER(_P)]),
    "msx_training_load_parameters": (C.c_int, [_P, _P, C.POINTER(C.c_uint64)]),
    "msx_training_refuse_out_reading": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p]),
    "msx_training_infer_dense": (C.c_int, [_P, C.c_char_p, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
}

_lib = None


def lib():
    """The loaded library. Raises when it has not been built: there is no other compute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(or `python modelspec_b200/_build.py`); modelspec_b200 has no fallback path" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = L
    return _lib


def _text(call):
    """Calls `call(buffer, capacity)` twice: once for the size, once for the bytes."""
    n = call(None, 0)
    if n == 0:
        raise MsxError(UNSUPPORTED, lib().msx_last_error(None).decode())
    buf = C.create_string_buffer(n)
    call(buf, n)
    return buf.value.decode()


def compile_mspec(source, which="step", masked_rows=0):
    """`.mspec` source to the text of its training step ("step"), its dropout-free forward
    program ("forward") or its lowered tensor program ("tensor")."""
    return _text(lambda buf, cap: lib().msx_compile(source.encode(), which.encode(), masked_rows, buf, cap))


def compile_function(source, name, which="forward"):
    """The model function `name` of `.mspec` source as an inference entry: the text of its
    forward program ("forward") or step ("step"), or its prediction's value id ("prediction").
    A name the model does not declare raises with E-DATA-010 naming the model's functions."""
    return _text(lambda buf, cap: lib().msx_compile_function(source.encode(), name.encode(), which.encode(), buf, cap))


def schedule_describe(ir_text, flags=PLAN_DEFAULT):
    """The kernel launches the backend schedules for a program, one per line; needs no GPU. Under
    PLAN_BF16 the values stored as bf16 carry the suffix `h`."""
    return _text(lambda buf, cap: lib().msx_schedule_describe_with(ir_text.encode(), flags, buf, cap))


def comm_unique_id():
    """128 bytes that name a new data-parallel job; rank 0 makes them, every rank passes them on."""
    buf = C.create_string_buffer(128)
    rc = lib().msx_comm_unique_id(buf)
    if rc != OK:
        raise MsxError(rc, lib().msx_last_error(None).decode())
    return buf.raw


def _host(array):
    a = np.asarray(array)
    if a.dtype.kind in "iu":
        return np.ascontiguousarray(a, dtype=np.int32)
    return np.ascontiguousarray(a, dtype=np.float32)


class Device:
    def __init__(self, ordinal=0):
        h = _P()
        rc = lib().msx_open(ordinal, C.byref(h))
        if rc != OK:
            raise MsxError(rc, lib().msx_last_error(None).decode())
        self.h = h
        self.ordinal = ordinal

    def error(self):
        return lib().msx_last_error(self.h).decode()

    def check(self, rc):
        if rc != OK:
            raise MsxError(rc, self.error())

    def close(self):
        if self.h:
            lib().msx_close(self.h)
            self.h = None

    def peer_reduce_check(self, copies, scale=1.0, peers_present=True, wait_ms=50):
        """msx_peer_reduce_check: the peer-memory all-reduce launches of every rank, run one after
        the other on this device over `copies` (one float32 array per rank). Returns what the
        copies hold afterwards and the status word."""
        import numpy as np
        arrays = [np.ascontiguousarray(c, dtype=np.float32).copy() for c in copies]
        pointers = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
        status = C.c_uint32(0)
        self.check(lib().msx_peer_reduce_check(self.h, len(arrays), arrays[0].size, pointers, scale, 1 if peers_present else 0,
                                               wait_ms, C.byref(status)))
        return arrays, status.value


class Plan:
    """One program's execution plan on one device (msx_plan)."""

    def __init__(self, device, ir_text=None, seed=0, flags=PLAN_DEFAULT, shares=None, handle=None):
        self.device = device
        self.owned = handle is None
        if handle is None:
            h = _P()
            device.check(lib().msx_plan_create(device.h, ir_text.encode(), seed, flags,
                                               shares.h if shares is not None else None, C.byref(h)))
            handle = h
        self.h = handle

    def destroy(self):
        if self.h and self.owned:
            lib().msx_plan_destroy(self.h)
        self.h = None

    def inputs(self):
        L = lib()
        return [(L.msx_plan_input_name(self.h, i).decode(), L.msx_plan_input_bytes(self.h, i),
                 bool(L.msx_plan_input_is_i32(self.h, i))) for i in range(L.msx_plan_input_count(self.h))]

    def params(self):
        L = lib()
        return [(L.msx_plan_param_path(self.h, i).decode(), L.msx_plan_param_bytes(self.h, i))
                for i in range(L.msx_plan_param_count(self.h))]

    def param_upload(self, index, array):
        a = _host(array)
        self.device.check(lib().msx_param_upload(self.h, index, a.ctypes.data, a.nbytes))

    def param_download(self, index):
        out = np.empty(self.params()[index][1] // 4, dtype=np.float32)
        self.device.check(lib().msx_param_download(self.h, index, out.ctypes.data, out.nbytes))
        return out

    def moment_upload(self, index, which, array):
        a = _host(array)
        self.device.check(lib().msx_moment_upload(self.h, index, which.encode(), a.ctypes.data, a.nbytes))

    def moment_download(self, index, which):
        out = np.empty(self.params()[index][1] // 4, dtype=np.float32)
        self.device.check(lib().msx_moment_download(self.h, index, which.encode(), out.ctypes.data, out.nbytes))
        return out

    def set_input(self, name, array):
        a = _host(array)
        self.device.check(lib().msx_set_input(self.h, name.encode(), a.ctypes.data, a.nbytes))

    def set_shard(self, rows_before, global_rows):
        self.device.check(lib().msx_set_shard(self.h, rows_before, global_rows))

    def comm_init(self, rank, world, unique_id):
        """Joins this plan to a data-parallel job; `unique_id` is the 128 bytes of comm_unique_id()."""
        buf = C.create_string_buffer(bytes(unique_id), 128)
        self.device.check(lib().msx_comm_init(self.h, rank, world, buf))

    def run(self):
        self.device.check(lib().msx_run(self.h))

    def sync(self, timeout_ms=0):
        self.device.check(lib().msx_sync(self.h, timeout_ms))

    def loss(self, timeout_ms=0):
        out = C.c_float()
        self.device.check(lib().msx_loss(self.h, C.byref(out), timeout_ms))
        return np.float32(out.value)

    def value(self, value_id, count, dtype=np.float32):
        out = np.empty(count, dtype=dtype)
        self.device.check(lib().msx_value_download(self.h, value_id, out.ctypes.data, out.nbytes))
        return out

    def stats(self):
        s = Stats()
        self.device.check(lib().msx_plan_stats(self.h, C.byref(s)))
        return {n: getattr(s, n) for n, _ in Stats._fields_}

    def describe(self):
        return _text(lambda buf, cap: lib().msx_plan_describe(self.h, buf, cap))

    def stats_report(self):
        """The lines `train --stats` prints for a device run."""
        return _text(lambda buf, cap: lib().msx_stats_report(self.h, buf, cap))

    def profile_report(self, final_plan=None, repeats=1):
        """The lines `train --profile` prints: runs one step launch by launch on each plan."""
        other = final_plan.h if final_plan is not None else None
        n = lib().msx_profile_report(self.h, other, repeats, None, 0)
        if n == 0:
            raise MsxError(LAUNCH_FAILED, self.device.error())
        # The sizing call ran a step too; the lines of the second call (whose times may print with
        # a digit more) are the ones returned.
        buf = C.create_string_buffer(n + 4096)
        lib().msx_profile_report(self.h, other, repeats, buf, n + 4096)
        return buf.value.decode()

    def check_guards(self):
        """For a PLAN_GUARD plan: raises when a kernel wrote past the end of a value."""
        self.device.check(lib().msx_plan_check_guards(self.h))

    def profile_step(self, repeats=1):
        """Runs one step launch by launch (each launch `repeats` times back to back, its time
        divided by `repeats`); returns [(kernel, ms, bytes, flop)] per launch."""
        n = self.stats()["launches_per_step"]
        ms = (C.c_float * n)()
        self.device.check(lib().msx_profile_step_repeated(self.h, repeats, ms, n))
        L = lib()
        return [(L.msx_launch_kernel(self.h, i).decode(), float(ms[i]), L.msx_launch_bytes(self.h, i),
                 L.msx_launch_flop(self.h, i)) for i in range(n)]

    def steps_submitted(self):
        return int(lib().msx_steps_submitted(self.h))

    def step_ms(self, step_number):
        """Device time of one of the last 8 submitted steps, in milliseconds."""
        out = C.c_float()
        self.device.check(lib().msx_step_ms(self.h, step_number, C.byref(out)))
        return float(out.value)

    def loss_of(self, step_number, timeout_ms=0):
        out = C.c_float()
        self.device.check(lib().msx_loss_of(self.h, step_number, C.byref(out), timeout_ms))
        return np.float32(out.value)

    def comm_exposed_ms(self):
        out = C.c_float()
        self.device.check(lib().msx_comm_exposed_ms(self.h, C.byref(out)))
        return float(out.value)

    def elapsed_ms(self):
        total, steps = C.c_double(), C.c_uint64()
        self.device.check(lib().msx_elapsed_ms(self.h, C.byref(total), C.byref(steps)))
        return total.value, steps.value


SPLIT_TRAIN, SPLIT_HELDOUT = 0, 1
OPTIMIZER_SGD, OPTIMIZER_ADAMW, OPTIMIZER_OTHER = 0, 1, 2


class Checkpoint:
    """A `.msckpt` checkpoint in memory (msx_checkpoint): built tensor by tensor or read from a file."""

    def __init__(self, step=0, seed=0, schema_hash="", handle=None):
        if handle is None:
            handle = _P()
            rc = lib().msx_checkpoint_new(step, seed, schema_hash.encode(), C.byref(handle))
            if rc != OK:
                raise MsxError(rc, "msx_checkpoint_new")
        self.h = handle

    @classmethod
    def read(cls, path):
        h = _P()
        rc = lib().msx_checkpoint_read(str(path).encode(), C.byref(h))
        if rc != OK:
            raise MsxError(rc, lib().msx_last_error(None).decode())
        return cls(handle=h)

    def destroy(self):
        if self.h:
            lib().msx_checkpoint_destroy(self.h)
            self.h = None

    def check(self, rc):
        if rc != OK:
            raise MsxError(rc, lib().msx_checkpoint_last_error(self.h).decode())

    def set_optimizer(self, kind, learning_rate, weight_decay=0.0, beta1=0.0, beta2=0.0, epsilon=0.0, warmup_steps=0):
        self.check(lib().msx_checkpoint_set_optimizer(self.h, kind, learning_rate, weight_decay, beta1, beta2, epsilon, warmup_steps))

    def add(self, path, array, slot=None):
        a = np.ascontiguousarray(array, dtype=np.float32)
        shape = (C.c_uint64 * a.ndim)(*a.shape)
        self.check(lib().msx_checkpoint_add(self.h, path.encode(), slot.encode() if slot else None, shape, a.ndim, a.ctypes.data))

    def encode(self):
        n = lib().msx_checkpoint_encode(self.h, None, 0)
        buf = C.create_string_buffer(n)
        lib().msx_checkpoint_encode(self.h, buf, n)
        return buf.raw

    def write(self, path):
        self.check(lib().msx_checkpoint_write(self.h, str(path).encode()))

    step = property(lambda self: int(lib().msx_checkpoint_step(self.h)))
    seed = property(lambda self: int(lib().msx_checkpoint_seed(self.h)))
    schema_hash = property(lambda self: lib().msx_checkpoint_schema_hash(self.h).decode())
    id = property(lambda self: lib().msx_checkpoint_id(self.h).decode())

    def optimizer_json(self):
        return _text(lambda buf, cap: lib().msx_checkpoint_optimizer_json(self.h, buf, cap))

    def tensors(self, slots=False):
        """[(path, slot, array)] of the parameters, or of the optimizer slots."""
        L, which = lib(), 1 if slots else 0
        out = []
        for i in range(L.msx_checkpoint_count(self.h, which)):
            rank = L.msx_checkpoint_rank(self.h, which, i)
            shape = tuple(int(L.msx_checkpoint_shape(self.h, which, i)[d]) for d in range(rank))
            n = int(np.prod(shape)) if rank else 1
            data = np.ctypeslib.as_array(L.msx_checkpoint_data(self.h, which, i), shape=(n,)).copy().reshape(shape)
            out.append((L.msx_checkpoint_path(self.h, which, i).decode(), L.msx_checkpoint_slot(self.h, which, i).decode(), data))
        return out


def eval_line(loss, accuracy=None):
    """The last line of a run with `--eval`: `eval loss=<loss>[ accuracy=<accuracy>]`."""
    return _text(lambda buf, cap: lib().msx_training_eval_line(loss, accuracy if accuracy is not None else 0.0, 0 if accuracy is None else 1, buf, cap))


class Dense:
    """A dense data directory (msx_dense): `<name>.f32` / `<name>.i32` per declaration and an
    optional `order.u32`. `declarations` = [(name, "f32" | "i32", "input" | "target" | "argument",
    shape), ...] in source order ("argument": of a model function run as an inference entry); `steps` = the run's step count (what an order must cover)."""

    def __init__(self, directory, declarations, steps, eval_directory=False):
        n = len(declarations)
        names = (C.c_char_p * n)(*[d[0].encode() for d in declarations])
        is_i32 = (C.c_uint32 * n)(*[1 if d[1] == "i32" else 0 for d in declarations])
        is_target = (C.c_uint32 * n)(*[{"target": 1, "argument": 2}.get(d[2], 0) for d in declarations])
        ranks = (C.c_uint32 * n)(*[len(d[3]) for d in declarations])
        flat = [int(x) for d in declarations for x in d[3]]
        shapes = (C.c_uint64 * max(len(flat), 1))(*flat)
        h = _P()
        if eval_directory:   # `--eval <dir>`: no order, a whole number of batches
            rc = lib().msx_dense_open_eval(str(directory).encode(), n, names, is_i32, is_target, ranks, shapes, C.byref(h))
        else:
            rc = lib().msx_dense_open(str(directory).encode(), n, names, is_i32, is_target, ranks, shapes, steps, C.byref(h))
        if rc != OK:
            raise MsxError(rc, lib().msx_dense_last_error(None).decode())
        self.h = h
        self.declarations = list(declarations)

    def close(self):
        if self.h:
            lib().msx_dense_close(self.h)
            self.h = None

    @property
    def batch(self):
        return int(lib().msx_dense_batch(self.h))

    @property
    def samples(self):
        return int(lib().msx_dense_samples(self.h))

    @property
    def has_order(self):
        return bool(lib().msx_dense_has_order(self.h))

    def check_bound(self, index, bound, what):
        rc = lib().msx_dense_check_bound(self.h, index, bound, what.encode())
        if rc != OK:
            raise MsxError(rc, lib().msx_dense_last_error(self.h).decode())

    def eval_batch(self, index, b):
        """Batch `b` of declaration `index` of an eval directory as a flat array."""
        nbytes = int(lib().msx_dense_batch_bytes(self.h, index))
        out = np.empty(nbytes // 4, dtype=np.int32 if self.declarations[index][1] == "i32" else np.float32)
        rc = lib().msx_dense_eval_batch(self.h, index, b, out.ctypes.data, nbytes)
        if rc != OK:
            raise MsxError(rc, "msx_dense_eval_batch")
        return out

    def step(self, index, k):
        """The batch of step `k` of declaration `index` as a flat array."""
        nbytes = int(lib().msx_dense_batch_bytes(self.h, index))
        out = np.empty(nbytes // 4, dtype=np.int32 if self.declarations[index][1] == "i32" else np.float32)
        rc = lib().msx_dense_step(self.h, index, k, out.ctypes.data, nbytes)
        if rc != OK:
            raise MsxError(rc, "msx_dense_step")
        return out


class Packed:
    """A packed masked-language-model directory (msx_packed): the reference's `--data <packed>`."""

    def __init__(self, directory):
        h = _P()
        rc = lib().msx_packed_open(str(directory).encode(), C.byref(h))
        if rc != OK:
            raise MsxError(rc, lib().msx_last_error(None).decode())
        self.h = h
        self.dir = str(directory)

    def close(self):
        if self.h:
            lib().msx_packed_close(self.h)
            self.h = None

    def check(self, rc):
        if rc != OK:
            raise MsxError(rc, lib().msx_packed_last_error(self.h).decode())

    @property
    def seq_len(self):
        return int(lib().msx_packed_seq_len(self.h))

    @property
    def vocabulary(self):
        return int(lib().msx_packed_vocabulary(self.h))

    @property
    def binding_id(self):
        return lib().msx_packed_binding_id(self.h).decode()

    def sequences(self, split):
        return int(lib().msx_packed_sequences(self.h, split))

    def data_line(self):
        return _text(lambda buf, cap: lib().msx_packed_data_line(self.h, buf, cap))

    def epoch_order(self, seed, epoch):
        out = np.empty(self.sequences(SPLIT_TRAIN), dtype=np.uint32)
        self.check(lib().msx_packed_epoch_order(self.h, seed, epoch, out.ctypes.data, out.size))
        return out

    def batch(self, split, seed, step, batch_size):
        """`mlm_batch`: a dict of ids, positions, key_mask, labels, weights of batch_size * S rows."""
        rows = batch_size * self.seq_len
        out = {"ids": np.empty(rows, np.int32), "positions": np.empty(rows, np.int32), "key_mask": np.empty(rows, np.float32),
               "labels": np.empty(rows, np.int32), "weights": np.empty(rows, np.float32)}
        self.check(lib().msx_packed_batch(self.h, split, seed, step, batch_size, *(out[k].ctypes.data for k in
                                                                                   ("ids", "positions", "key_mask", "labels", "weights"))))
        return out


class HeldOut:
    """The held-out reduction of a plan's logits on the device (msx_heldout): targets once, then
    per evaluation begin(), add(batch) after each batch's run, and sums()."""

    def __init__(self, plan, logits, batches):
        self.plan = plan
        h = _P()
        plan.device.check(lib().msx_heldout_create(plan.h, logits, batches, C.byref(h)))
        self.h = h

    def destroy(self):
        if self.h:
            lib().msx_heldout_destroy(self.h)
            self.h = None

    def targets(self, batch, labels, weights):
        labels = np.ascontiguousarray(labels, dtype=np.int32)
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        self.plan.device.check(lib().msx_heldout_targets(self.h, batch, labels.ctypes.data, weights.ctypes.data, labels.size))

    def begin(self):
        self.plan.device.check(lib().msx_heldout_begin(self.h))

    def add(self, batch):
        self.plan.device.check(lib().msx_heldout_add(self.h, batch))

    def sums(self, timeout_ms=0):
        """(numerator, correct) of the batches added since begin(); the evaluation's one wait."""
        numerator, correct = C.c_double(), C.c_uint64()
        self.plan.device.check(lib().msx_heldout_sums(self.h, C.byref(numerator), C.byref(correct), timeout_ms))
        return float(numerator.value), int(correct.value)


class Training:
    """One training run (msx_training): the host loop of `train --backend cuda`."""

    def __init__(self, device, source, masked_rows=0, flags=PLAN_DEFAULT, function=None):
        """The run of the train block of `source`, or with `function` the model function of that
        name as an inference entry (`infer --data --function`): its arguments the inputs, its
        result the prediction."""
        self.device = device
        h = _P()
        if function is None:
            device.check(lib().msx_training_create(device.h, source.encode(), masked_rows, flags, C.byref(h)))
        else:
            device.check(lib().msx_training_create_function(device.h, source.encode(), function.encode(), flags, C.byref(h)))
        self.h = h
        self.steps = lib().msx_training_steps(h)
        self.seed = lib().msx_training_seed(h)
        self.step_plan = Plan(device, handle=_P(lib().msx_training_step_plan(h)))
        self.forward_plan = Plan(device, handle=_P(lib().msx_training_forward_plan(h)))

    def check(self, rc):
        if rc != OK:
            raise MsxError(rc, lib().msx_training_last_error(self.h).decode())

    def destroy(self):
        if self.h:
            lib().msx_training_destroy(self.h)
            self.h = None

    def comm_init(self, rank, world, unique_id, rows_per_rank):
        buf = C.create_string_buffer(bytes(unique_id), 128)
        self.check(lib().msx_training_comm_init(self.h, rank, world, buf, rows_per_rank))

    def set_input(self, name, array):
        a = _host(array)
        self.check(lib().msx_training_set_input(self.h, name.encode(), a.ctypes.data, a.nbytes))

    def get_input(self, name, count, dtype=np.float32):
        out = np.empty(count, dtype=dtype)
        self.check(lib().msx_training_get_input(self.h, name.encode(), out.ctypes.data, out.nbytes))
        return out

    def synthetic(self):
        self.check(lib().msx_training_synthetic(self.h))

    def step(self, k, end):
        self.check(lib().msx_training_step(self.h, k, end))

    def loss(self):
        out = C.c_float()
        self.check(lib().msx_training_loss(self.h, C.byref(out)))
        return np.float32(out.value)

    def loss_of(self, k):
        out = C.c_float()
        self.check(lib().msx_training_loss_of(self.h, k, C.byref(out)))
        return np.float32(out.value)

    def final_loss(self):
        out = C.c_float()
        self.check(lib().msx_training_final_loss(self.h, C.byref(out)))
        return np.float32(out.value)

    def check_finite(self):
        self.check(lib().msx_training_check_finite(self.h))

    def infer(self):
        """The forward program on the current parameters and batch: (prediction, loss)."""
        n = lib().msx_training_prediction_count(self.h)
        out = np.empty(n, dtype=np.float32)
        loss = C.c_float()
        self.check(lib().msx_training_infer(self.h, out.ctypes.data, out.nbytes, C.byref(loss)))
        return out, np.float32(loss.value)

    def heldout_begin(self, batches, labels, weights):
        """Declares the held-out split of the run: `batches` batches, and the names of the declared
        tensors that hold the rows' labels and weights."""
        self.check(lib().msx_training_heldout_begin(self.h, batches, labels.encode(), weights.encode()))

    def heldout_set(self, batch, name, array):
        a = np.ascontiguousarray(array)
        self.check(lib().msx_training_heldout_set(self.h, batch, name.encode(), a.ctypes.data, a.nbytes))

    def bind_packed(self, packed):
        """Feeds the run from a packed directory; `packed` must stay open while the run lives."""
        self.check(lib().msx_training_bind_packed(self.h, packed.h))
        self._packed = packed

    def bind_dense(self, directory):
        """Feeds the run from a dense directory (`<name>.f32` / `<name>.i32`, optional `order.u32`)."""
        self.check(lib().msx_training_bind_dense(self.h, str(directory).encode()))

    def eval_dense(self, directory):
        """`--eval <dir>`: (mean loss, accuracy or None) of the forward program over an eval directory."""
        loss, accuracy, has = C.c_double(), C.c_double(), C.c_int()
        self.check(lib().msx_training_eval_dense(self.h, str(directory).encode(), C.byref(loss), C.byref(accuracy), C.byref(has)))
        return loss.value, (accuracy.value if has.value else None)

    def feed_dense(self, step):
        """Makes the dense batch of `step` the current batch."""
        self.check(lib().msx_training_feed_dense(self.h, step))

    def feed_packed(self, step):
        """Makes the Train batch of `step` the current batch."""
        self.check(lib().msx_training_feed_packed(self.h, step))

    def heldout_packed(self):
        """Draws the HeldOut batches of the bound directory once; returns how many there are."""
        self.check(lib().msx_training_heldout_packed(self.h, self._packed.dir.encode()))
        return int(lib().msx_training_heldout_batches(self.h))

    def run(self, start=0, eval_every=0):
        """The whole run of the train block from step `start`; returns the text `train` prints for it.
        A run that stops at a loss that is not finite raises, with the text so far in `report()`."""
        rc = lib().msx_training_run(self.h, start, eval_every)
        if rc != OK:
            raise MsxError(rc, lib().msx_training_last_error(self.h).decode())
        return self.report()

    def report(self):
        return _text(lambda buf, cap: lib().msx_training_report(self.h, buf, cap))

    def set_replay_window(self, steps):
        """Takes a device snapshot of the state before every `steps`-th step (0: none)."""
        self.check(lib().msx_training_set_replay_window(self.h, steps))

    def rewind(self, step):
        """Leaves the run as it was after the update of `step` (restore the snapshot, replay)."""
        self.check(lib().msx_training_rewind(self.h, step))

    def checkpoint(self, step):
        """The run's state after `step` updates as a Checkpoint (parameters, and AdamW moments)."""
        h = _P()
        self.check(lib().msx_training_checkpoint(self.h, step, C.byref(h)))
        return Checkpoint(handle=h)

    def resume(self, checkpoint):
        """Loads a checkpoint into the run; returns the step the run continues from."""
        start = C.c_uint64()
        self.check(lib().msx_training_resume(self.h, checkpoint.h, C.byref(start)))
        return int(start.value)

    def load_parameters(self, checkpoint):
        """Loads a checkpoint's parameters, whatever its optimizer (`infer`); returns its step."""
        step = C.c_uint64()
        self.check(lib().msx_training_load_parameters(self.h, checkpoint.h, C.byref(step)))
        return int(step.value)

    def refuse_out_reading(self, directory, out, model=None, checkpoint=None):
        """E-DATA-010 when `out` resolves to a file the function's run reads."""
        enc = lambda v: None if v is None else str(v).encode()
        self.check(lib().msx_training_refuse_out_reading(self.h, str(directory).encode(), str(out).encode(), enc(model), enc(checkpoint)))

    def infer_dense(self, directory, out):
        """Runs the function over every block of a dense directory and writes its results, one
        row per sample, to `out`; returns (blocks, rows)."""
        blocks, rows = C.c_uint64(), C.c_uint64()
        self.check(lib().msx_training_infer_dense(self.h, str(directory).encode(), str(out).encode(), C.byref(blocks), C.byref(rows)))
        return int(blocks.value), int(rows.value)

    def schema_hash(self):
        return lib().msx_training_schema_hash(self.h).decode()

    def heldout_evaluate(self):
        """The held-out (loss, accuracy) of the current parameters, reduced on the device."""
        loss, accuracy = C.c_float(), C.c_float()
        self.check(lib().msx_training_heldout_evaluate(self.h, C.byref(loss), C.byref(accuracy)))
        return np.float32(loss.value), np.float32(accuracy.value)

    def infer_report(self):
        """The two lines `infer` prints: `prediction: <type> = [...]` and `loss <v>`."""
        n = lib().msx_training_infer_report(self.h, None, 0)
        if n == 0:
            raise MsxError(UNSUPPORTED, lib().msx_training_last_error(self.h).decode())
        buf = C.create_string_buffer(n)
        lib().msx_training_infer_report(self.h, buf, n)
        return buf.value.decode()
