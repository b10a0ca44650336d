"""ctypes binding of the CPU oracle (oracle/liboracle.so): test infrastructure only."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_lib = None


def build():
    """Builds oracle/liboracle.so with the recipe beside its source."""
    subprocess.run(["make", "-s", "-C", ORACLE_DIR], check=True)


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.orc_last_error.restype = C.c_char_p
        L.orc_trainer_create.restype = C.c_void_p
        L.orc_trainer_create.argtypes = [C.c_char_p, C.c_uint64]
        L.orc_session_create.restype = C.c_void_p
        L.orc_session_create.argtypes = [C.c_char_p, C.c_int]
        for name in ("orc_trainer_destroy", "orc_session_destroy"):
            getattr(L, name).argtypes = [C.c_void_p]
            getattr(L, name).restype = None
        L.orc_trainer_ir.restype = C.c_uint64
        L.orc_trainer_ir.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_uint64]
        L.orc_trainer_steps.restype = C.c_uint64
        L.orc_trainer_steps.argtypes = [C.c_void_p]
        L.orc_trainer_seed.restype = C.c_uint64
        L.orc_trainer_seed.argtypes = [C.c_void_p]
        L.orc_trainer_synthetic.argtypes = [C.c_void_p]
        L.orc_trainer_set_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]
        L.orc_trainer_set_i32.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]
        L.orc_trainer_get_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]
        L.orc_trainer_step.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.POINTER(C.c_float)]
        L.orc_trainer_final_loss.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
        L.orc_trainer_param_count.restype = C.c_uint64
        L.orc_trainer_param_count.argtypes = [C.c_void_p]
        L.orc_trainer_param_path.restype = C.c_char_p
        L.orc_trainer_param_path.argtypes = [C.c_void_p, C.c_uint64]
        L.orc_trainer_param_len.restype = C.c_uint64
        L.orc_trainer_param_len.argtypes = [C.c_void_p, C.c_uint64]
        L.orc_trainer_read.argtypes = [C.c_void_p, C.c_int, C.c_uint64, C.c_void_p, C.c_uint64]
        L.orc_trainer_write_param.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]
        L.orc_trainer_predict.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64]
        L.orc_tally_create.restype = C.c_void_p
        L.orc_tally_destroy.argtypes = [C.c_void_p]
        L.orc_tally_destroy.restype = None
        L.orc_tally_add.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int]
        L.orc_tally_read.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_void_p, C.c_void_p]
        L.orc_tally_read.restype = None
        L.orc_session_set_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]
        L.orc_session_set_i32.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64]
        L.orc_session_set_param.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]
        L.orc_session_set_seed.argtypes = [C.c_void_p, C.c_uint64]
        L.orc_session_set_seed.restype = None
        L.orc_session_run.argtypes = [C.c_void_p]
        L.orc_session_value.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint64]
        L.orc_canonical_id.restype = C.c_uint64
        L.orc_canonical_id.argtypes = [C.c_char_p]
        L.orc_dropout_id.restype = C.c_uint64
        L.orc_dropout_id.argtypes = [C.c_char_p, C.c_uint64]
        L.orc_dropout_keeps.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, C.c_float]
        L.orc_blake3.argtypes = [C.c_char_p, C.c_uint64, C.c_void_p]
        L.orc_blake3.restype = None
        L.orc_philox.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_philox.restype = None
        L.orc_set_threads.argtypes = [C.c_int]
        L.orc_set_threads.restype = None
        L.orc_set_threads(os.cpu_count() or 1)
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise RuntimeError(lib().orc_last_error().decode())


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return np.ascontiguousarray(a, dtype=np.int32)


class Trainer:
    """One training run on the oracle: the reference's `train --backend cpu` loop."""

    def __init__(self, source, masked_rows=0):
        self.h = lib().orc_trainer_create(source.encode(), masked_rows)
        if not self.h:
            raise RuntimeError(lib().orc_last_error().decode())
        self.steps = lib().orc_trainer_steps(self.h)
        self.seed = lib().orc_trainer_seed(self.h)

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_trainer_destroy(self.h)
            self.h = None

    def ir(self, which="step"):
        n = lib().orc_trainer_ir(self.h, which.encode(), None, 0)
        buf = C.create_string_buffer(n)
        lib().orc_trainer_ir(self.h, which.encode(), buf, n)
        return buf.value.decode()

    def synthetic(self):
        _check(lib().orc_trainer_synthetic(self.h))

    def set_input(self, name, array):
        a = np.asarray(array)
        if a.dtype.kind in "iu":
            a = _i32(a)
            _check(lib().orc_trainer_set_i32(self.h, name.encode(), a.ctypes.data, a.size))
        else:
            a = _f32(a)
            _check(lib().orc_trainer_set_f32(self.h, name.encode(), a.ctypes.data, a.size))

    def get_input(self, name, n):
        out = np.empty(n, dtype=np.float32)
        _check(lib().orc_trainer_get_f32(self.h, name.encode(), out.ctypes.data, n))
        return out

    def step(self, k, end):
        loss = C.c_float()
        _check(lib().orc_trainer_step(self.h, k, end, C.byref(loss)))
        return np.float32(loss.value)

    def final_loss(self):
        loss = C.c_float()
        _check(lib().orc_trainer_final_loss(self.h, C.byref(loss)))
        return np.float32(loss.value)

    def param_paths(self):
        return [lib().orc_trainer_param_path(self.h, i).decode() for i in range(lib().orc_trainer_param_count(self.h))]

    def read(self, which, i):
        """which: 'param', 'm', 'v' or 'grad' of parameter index i."""
        n = lib().orc_trainer_param_len(self.h, i)
        out = np.empty(n, dtype=np.float32)
        _check(lib().orc_trainer_read(self.h, {"param": 0, "m": 1, "v": 2, "grad": 3}[which], i, out.ctypes.data, n))
        return out

    def predict(self, n):
        """The model's prediction for the current batch, from the dropout-free forward program."""
        out = np.empty(n, dtype=np.float32)
        _check(lib().orc_trainer_predict(self.h, out.ctypes.data, n))
        return out

    def write_param(self, i, array):
        a = _f32(array)
        _check(lib().orc_trainer_write_param(self.h, i, a.ctypes.data, a.size))


class Tally:
    """The held-out reduction: batches of logits [rows, classes] in order, then the metrics."""

    def __init__(self, skipping=True):
        self.h = C.c_void_p(lib().orc_tally_create())
        self.skipping = skipping

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_tally_destroy(self.h)
            self.h = None

    def add(self, logits, labels, weights):
        logits, labels, weights = _f32(logits), _i32(labels), _f32(weights)
        rows = labels.size
        _check(lib().orc_tally_add(self.h, logits.ctypes.data, labels.ctypes.data, weights.ctypes.data, rows, logits.size // max(rows, 1),
                                   1 if self.skipping else 0))

    def read(self):
        """(loss, accuracy, numerator, denominator, correct, selected, softmaxes)."""
        loss, accuracy = C.c_float(), C.c_float()
        sums = np.zeros(2, dtype=np.float64)
        counts = np.zeros(3, dtype=np.uint64)
        lib().orc_tally_read(self.h, C.byref(loss), C.byref(accuracy), sums.ctypes.data, counts.ctypes.data)
        return (np.float32(loss.value), np.float32(accuracy.value), float(sums[0]), float(sums[1]), int(counts[0]), int(counts[1]), int(counts[2]))


class Session:
    """One evaluation of a bare Tensor IR program, in f32 or (wide=True) f64."""

    def __init__(self, ir_text, wide=False):
        self.h = lib().orc_session_create(ir_text.encode(), 1 if wide else 0)
        if not self.h:
            raise RuntimeError(lib().orc_last_error().decode())

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_session_destroy(self.h)
            self.h = None

    def set_input(self, name, array):
        a = np.asarray(array)
        if a.dtype.kind in "iu":
            a = _i32(a)
            _check(lib().orc_session_set_i32(self.h, name.encode(), a.ctypes.data, a.size))
        else:
            a = _f32(a)
            _check(lib().orc_session_set_f32(self.h, name.encode(), a.ctypes.data, a.size))

    def set_param(self, i, array):
        a = _f32(array)
        _check(lib().orc_session_set_param(self.h, i, a.ctypes.data, a.size))

    def set_seed(self, seed):
        lib().orc_session_set_seed(self.h, seed)

    def run(self):
        _check(lib().orc_session_run(self.h))

    def value(self, value_id, n):
        out = np.empty(n, dtype=np.float64)
        _check(lib().orc_session_value(self.h, value_id, out.ctypes.data, n))
        return out
