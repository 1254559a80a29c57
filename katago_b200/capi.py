"""ctypes binding of the C ABI declared in include/katab200.h."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

PRECISION_FP32, PRECISION_FP16, PRECISION_BF16 = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkatab200.so")
_lib = None

# Every symbol include/katab200.h declares.
EXPORTED_SYMBOLS = [
    "kb_last_error", "kb_version", "kb_device_count", "kb_device_name", "kb_model_create", "kb_model_destroy",
    "kb_model_info", "kb_model_meta_channels", "kb_forward_host_meta", "kb_upload_inputs_meta", "kb_handle_create", "kb_handle_destroy", "kb_handle_precision", "kb_weight_cache_stats", "kb_selftest_wait_timeout", "kb_tile_plan", "kb_tile_table", "kb_forward_host",
    "kb_upload_inputs", "kb_forward_resident", "kb_download_outputs", "kb_time_forward_resident", "kb_time_forward_steps",
    "kb_profile_enable", "kb_profile_reset", "kb_profile_read", "kb_launches_per_forward", "kb_debug_read_trunk",
    "kb_eval_layer", "kb_host_alloc", "kb_host_free", "kb_conv_noalloc", "kb_conv_noalloc_last_error",
]


class ProfileEntry(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 48), ("launches", ctypes.c_int64), ("ms", ctypes.c_double),
                ("flops", ctypes.c_double), ("bytes", ctypes.c_double)]


def library_path() -> str:
    return _LIB_PATH


def build_library() -> str:
    """Compiles every CUDA source for sm_100a into katago_b200/libkatab200.so (nvcc cross-compiles without a GPU)."""
    subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), "-j8"], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: the CUDA extension has not been built (run __graft_entry__.build()). "
                "There is no CPU fallback.")
        L = ctypes.CDLL(_LIB_PATH)
        vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        L.kb_last_error.restype = ctypes.c_char_p
        L.kb_version.restype = ctypes.c_char_p
        L.kb_device_count.argtypes = [ctypes.POINTER(ci)]
        L.kb_device_name.argtypes = [ci, ctypes.c_char_p, sz]
        L.kb_model_create.argtypes = [vp, sz, ctypes.POINTER(vp)]
        L.kb_model_destroy.argtypes = [vp]
        L.kb_model_info.argtypes = [vp, ctypes.POINTER(ctypes.c_int32)]
        L.kb_model_meta_channels.argtypes = [vp, ctypes.POINTER(ctypes.c_int32)]
        L.kb_forward_host_meta.argtypes = [vp, ci] + [vp] * 9
        L.kb_upload_inputs_meta.argtypes = [vp, ci, vp, vp, vp, vp]
        L.kb_handle_create.argtypes = [vp, ci, ci, ci, ci, ci, ci, ctypes.POINTER(vp)]
        L.kb_handle_destroy.argtypes = [vp]
        L.kb_handle_precision.argtypes = [vp, ctypes.POINTER(ci)]
        L.kb_weight_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_int64)]
        L.kb_selftest_wait_timeout.argtypes = [vp, ctypes.c_ulonglong]
        L.kb_tile_plan.argtypes = [ci, ci, ci, ctypes.POINTER(ctypes.c_int32)]
        L.kb_tile_table.argtypes = [ctypes.POINTER(ctypes.c_int32), ci, ctypes.POINTER(ctypes.c_int32)]
        L.kb_forward_host.argtypes = [vp, ci] + [vp] * 8
        L.kb_upload_inputs.argtypes = [vp, ci, vp, vp, vp]
        L.kb_forward_resident.argtypes = [vp, ci]
        L.kb_download_outputs.argtypes = [vp, ci] + [vp] * 5
        L.kb_time_forward_resident.argtypes = [vp, ci, ci, ctypes.POINTER(ctypes.c_float)]
        L.kb_time_forward_steps.argtypes = [vp, ci, ci, sz, ctypes.POINTER(ctypes.c_float)]
        L.kb_profile_enable.argtypes = [vp, ci]
        L.kb_profile_reset.argtypes = [vp]
        L.kb_profile_read.argtypes = [vp, ctypes.POINTER(ProfileEntry), ci, ctypes.POINTER(ci)]
        L.kb_launches_per_forward.argtypes = [vp, ci, ctypes.POINTER(ci)]
        L.kb_debug_read_trunk.argtypes = [vp, ci, vp]
        L.kb_eval_layer.argtypes = [vp, sz, ci, ci, ci, ci, ci, vp, vp, vp]
        L.kb_host_alloc.argtypes = [sz, ctypes.POINTER(vp)]
        L.kb_host_free.argtypes = [vp]
        L.kb_conv_noalloc.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]
        L.kb_conv_noalloc_last_error.restype = ctypes.c_char_p
        _lib = L
    return _lib


class KBError(RuntimeError):
    pass


def _check(status: int, what: str):
    if status != 0:
        raise KBError(f"{what} failed ({status}): {lib().kb_last_error().decode()}")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def tile_plan(k: int, in_c: int, out_c: int) -> dict:
    """Tile plan of a tensor-core convolution (in_c as the device sees it, a multiple of 64)."""
    a = (ctypes.c_int32 * 6)()
    _check(lib().kb_tile_plan(k, in_c, out_c, a), "kb_tile_plan")
    return dict(bn=int(a[0]), pair=int(a[1]), epi_warps=int(a[2]), epi_warps_res=int(a[3]), chain=int(a[4]), from_table=bool(a[5]))


def tile_table() -> list:
    """Rows of the committed tile table: dicts with k, in_c, out_c and the plan fields."""
    n = ctypes.c_int32()
    _check(lib().kb_tile_table(None, 0, ctypes.byref(n)), "kb_tile_table")
    a = (ctypes.c_int32 * (8 * n.value))()
    _check(lib().kb_tile_table(a, n.value, ctypes.byref(n)), "kb_tile_table")
    keys = ("k", "in_c", "out_c", "bn", "pair", "epi_warps", "epi_warps_res", "chain")
    return [dict(zip(keys, [int(a[i * 8 + j]) for j in range(8)])) for i in range(n.value)]


def weight_cache_stats() -> dict:
    """Counters of the device-side weight cache: live entries, their bytes, uploads made, uploads avoided."""
    a = (ctypes.c_int64 * 4)()
    _check(lib().kb_weight_cache_stats(a), "kb_weight_cache_stats")
    return dict(entries=int(a[0]), bytes=int(a[1]), uploads=int(a[2]), hits=int(a[3]))


def device_count() -> int:
    n = ctypes.c_int(0)
    _check(lib().kb_device_count(ctypes.byref(n)), "kb_device_count")
    return n.value


def device_name(device: int) -> str:
    buf = ctypes.create_string_buffer(256)
    _check(lib().kb_device_name(device, buf, 256), "kb_device_name")
    return buf.value.decode()


class PinnedArray:
    """numpy view over page-locked host memory from kb_host_alloc (freed with the object)."""

    def __init__(self, shape, dtype=np.float32):
        self.nbytes = int(np.prod(shape)) * np.dtype(dtype).itemsize
        self.ptr = ctypes.c_void_p()
        _check(lib().kb_host_alloc(max(self.nbytes, 16), ctypes.byref(self.ptr)), "kb_host_alloc")
        buf = (ctypes.c_uint8 * max(self.nbytes, 16)).from_address(self.ptr.value)
        self.array = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def __del__(self):
        if getattr(self, "ptr", None) and self.ptr.value:
            self.array = None
            lib().kb_host_free(self.ptr)
            self.ptr = ctypes.c_void_p()


class Model:
    def __init__(self, blob: bytes):
        self.h = ctypes.c_void_p()
        self._blob = blob
        _check(lib().kb_model_create(blob, len(blob), ctypes.byref(self.h)), "kb_model_create")
        info = (ctypes.c_int32 * 9)()
        _check(lib().kb_model_info(self.h, info), "kb_model_info")
        (self.version, self.in_c, self.in_global_c, self.policy_c, self.value_c, self.score_c, self.own_c,
         self.trunk_c, self.num_blocks) = list(info)
        mc = ctypes.c_int32(0)
        _check(lib().kb_model_meta_channels(self.h, ctypes.byref(mc)), "kb_model_meta_channels")
        self.meta_c = int(mc.value)

    def __del__(self):
        if getattr(self, "h", None):
            lib().kb_model_destroy(self.h)
            self.h = None


class Handle:
    def __init__(self, model: Model, max_batch: int, nn_x: int = 19, nn_y: int = 19, precision: int = PRECISION_FP16,
                 device: int = -1, require_exact: bool = False):
        self.model, self.max_batch, self.nn_x, self.nn_y = model, max_batch, nn_x, nn_y
        self.h = ctypes.c_void_p()
        _check(lib().kb_handle_create(model.h, device, max_batch, nn_x, nn_y, precision, int(require_exact), ctypes.byref(self.h)),
               "kb_handle_create")

    def close(self):
        if getattr(self, "h", None):
            lib().kb_handle_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def _outputs(self, n, pinned=False):
        m, S = self.model, self.nn_x * self.nn_y
        shapes = dict(policy=(n, S, m.policy_c), policyPass=(n, m.policy_c), value=(n, m.value_c),
                      scoreValue=(n, m.score_c), ownership=(n, S))
        return {k: np.empty(s, np.float32) for k, s in shapes.items()}

    def forward(self, spatial: np.ndarray, glob: np.ndarray, symmetry=None, out=None, meta=None):
        """The call getOutput makes: host buffers in, host buffers out.  meta: [n][meta_c] rows for nets with an SGF
        metadata encoder."""
        n = spatial.shape[0]
        spatial = np.ascontiguousarray(spatial, np.float32)
        glob = np.ascontiguousarray(glob, np.float32)
        sym = None if symmetry is None else np.ascontiguousarray(symmetry, np.int32)
        out = out or self._outputs(n)
        if meta is not None:
            meta = np.ascontiguousarray(meta, np.float32)
            _check(lib().kb_forward_host_meta(self.h, n, _ptr(spatial), _ptr(glob), _ptr(meta), _ptr(sym), _ptr(out["policy"]),
                                              _ptr(out["policyPass"]), _ptr(out["value"]), _ptr(out["scoreValue"]), _ptr(out["ownership"])),
                   "kb_forward_host_meta")
            return out
        _check(lib().kb_forward_host(self.h, n, _ptr(spatial), _ptr(glob), _ptr(sym), _ptr(out["policy"]), _ptr(out["policyPass"]),
                                     _ptr(out["value"]), _ptr(out["scoreValue"]), _ptr(out["ownership"])), "kb_forward_host")
        return out

    def upload(self, spatial, glob, symmetry=None, meta=None):
        n = spatial.shape[0]
        spatial = np.ascontiguousarray(spatial, np.float32)
        glob = np.ascontiguousarray(glob, np.float32)
        sym = None if symmetry is None else np.ascontiguousarray(symmetry, np.int32)
        self._keep = (spatial, glob, sym)
        if meta is not None:
            meta = np.ascontiguousarray(meta, np.float32)
            self._keep = (spatial, glob, sym, meta)
            _check(lib().kb_upload_inputs_meta(self.h, n, _ptr(spatial), _ptr(glob), _ptr(meta), _ptr(sym)), "kb_upload_inputs_meta")
            return
        _check(lib().kb_upload_inputs(self.h, n, _ptr(spatial), _ptr(glob), _ptr(sym)), "kb_upload_inputs")

    def selftest_wait_timeout(self, limit_ns: int):
        """Makes a bounded device-side wait run out on this handle's stream; raises KBError like any such time-out."""
        _check(lib().kb_selftest_wait_timeout(self.h, int(limit_ns)), "kb_selftest_wait_timeout")

    def forward_resident(self, n):
        _check(lib().kb_forward_resident(self.h, n), "kb_forward_resident")

    def download(self, n):
        out = self._outputs(n)
        _check(lib().kb_download_outputs(self.h, n, _ptr(out["policy"]), _ptr(out["policyPass"]), _ptr(out["value"]),
                                         _ptr(out["scoreValue"]), _ptr(out["ownership"])), "kb_download_outputs")
        return out

    def time_forward_resident(self, n, iters) -> float:
        ms = ctypes.c_float(0)
        _check(lib().kb_time_forward_resident(self.h, n, iters, ctypes.byref(ms)), "kb_time_forward_resident")
        return ms.value

    def time_forward_steps(self, n, steps, flush_bytes=0):
        """Per-step device times (ms), each step preceded by an L2 flush of flush_bytes."""
        arr = (ctypes.c_float * steps)()
        _check(lib().kb_time_forward_steps(self.h, n, steps, flush_bytes, arr), "kb_time_forward_steps")
        return [float(x) for x in arr]

    def profile_enable(self, on: bool):
        _check(lib().kb_profile_enable(self.h, int(on)), "kb_profile_enable")

    def profile_reset(self):
        _check(lib().kb_profile_reset(self.h), "kb_profile_reset")

    def profile_read(self):
        cap = 128
        arr = (ProfileEntry * cap)()
        cnt = ctypes.c_int(0)
        _check(lib().kb_profile_read(self.h, arr, cap, ctypes.byref(cnt)), "kb_profile_read")
        return [dict(name=arr[i].name.decode(), launches=arr[i].launches, ms=arr[i].ms, flops=arr[i].flops, bytes=arr[i].bytes)
                for i in range(cnt.value)]

    def launches_per_forward(self, n=None) -> int:
        k = ctypes.c_int(0)
        _check(lib().kb_launches_per_forward(self.h, self.max_batch if n is None else n, ctypes.byref(k)), "kb_launches_per_forward")
        return k.value

    def read_trunk(self, n) -> np.ndarray:
        out = np.empty((n, self.nn_x * self.nn_y, self.model.trunk_c), np.float32)
        _check(lib().kb_debug_read_trunk(self.h, n, _ptr(out)), "kb_debug_read_trunk")
        return out


def conv_noalloc(d_in: int, d_weights: int, d_out: int, n: int, nn_x: int, nn_y: int, in_c: int, out_c: int, ky: int, kx: int,
                 stream: int = 0) -> None:
    """kb_conv_noalloc with raw device addresses (ints).  Enqueues on `stream`; the caller synchronises."""
    status = lib().kb_conv_noalloc(d_in, d_weights, d_out, n, nn_x, nn_y, in_c, out_c, ky, kx, stream or None)
    if status != 0:
        raise KBError(f"kb_conv_noalloc failed ({status}): {lib().kb_conv_noalloc_last_error().decode()}")


def eval_layer(blob: bytes, x: np.ndarray, mask, out_c: int, precision: int = PRECISION_FP32, device: int = -1) -> np.ndarray:
    """x [n,Y,X,C] NHWC fp32, mask [n,Y,X] or None -> [n,Y,X,out_c] (nninterface.h:134-180 testEvaluate*)."""
    n, ylen, xlen, _ = x.shape
    x = np.ascontiguousarray(x, np.float32)
    m = None if mask is None else np.ascontiguousarray(mask, np.float32)
    out = np.empty((n, ylen, xlen, out_c), np.float32)
    _check(lib().kb_eval_layer(blob, len(blob), device, precision, n, xlen, ylen, _ptr(x), _ptr(m), _ptr(out)), "kb_eval_layer")
    return out
