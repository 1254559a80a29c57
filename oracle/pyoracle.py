"""ctypes binding of the CPU oracle (oracle/libkataoracle.so).  TEST INFRASTRUCTURE ONLY:
imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs; never by
the katago_b200 package.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkataoracle.so")
_lib = None


def build() -> str:
    """Compiles the oracle library (g++, no GPU needed)."""
    subprocess.run(["make", "-C", _HERE, "lib"], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.ko_last_error.restype = ctypes.c_char_p
        L.ko_model_create.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p)]
        L.ko_model_destroy.argtypes = [ctypes.c_void_p]
        L.ko_model_info.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        L.ko_forward.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 8
        L.ko_forward_meta.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 9
        L.ko_trunk_streams.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 4
        L.ko_model_meta_channels.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32)]
        L.ko_eval_layer.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int] + [ctypes.c_void_p] * 3
        _lib = L
    return _lib


def _check(status, what):
    if status != 0:
        raise RuntimeError(f"{what}: {lib().ko_last_error().decode()}")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class OracleModel:
    def __init__(self, blob: bytes, nn_x: int = 19, nn_y: int = 19):
        self.h = ctypes.c_void_p()
        self._blob = blob
        _check(lib().ko_model_create(blob, len(blob), nn_x, nn_y, ctypes.byref(self.h)), "ko_model_create")
        info = (ctypes.c_int32 * 9)()
        _check(lib().ko_model_info(self.h, info), "ko_model_info")
        (self.version, self.in_c, self.in_global_c, self.policy_c, self.value_c, self.score_c, self.own_c,
         self.trunk_c, self.num_blocks) = list(info)
        self.nn_x, self.nn_y = nn_x, nn_y

    def __del__(self):
        if getattr(self, "h", None):
            lib().ko_model_destroy(self.h)
            self.h = None

    def forward(self, spatial: np.ndarray, glob: np.ndarray, want_trunk: bool = False, meta: np.ndarray | None = None):
        """meta: [n][metaChannels] rows, required exactly for nets with an SGF metadata encoder."""
        n = spatial.shape[0]
        S = self.nn_x * self.nn_y
        spatial = np.ascontiguousarray(spatial, np.float32).reshape(n, S, self.in_c)
        glob = np.ascontiguousarray(glob, np.float32).reshape(n, self.in_global_c)
        out = dict(
            policy=np.empty((n, S, self.policy_c), np.float32), policyPass=np.empty((n, self.policy_c), np.float32),
            value=np.empty((n, self.value_c), np.float32), scoreValue=np.empty((n, self.score_c), np.float32),
            ownership=np.empty((n, S), np.float32))
        trunk = np.empty((n, S, self.trunk_c), np.float32) if want_trunk else None
        if meta is not None:
            meta = np.ascontiguousarray(meta, np.float32)
        _check(lib().ko_forward_meta(self.h, n, _ptr(spatial), _ptr(glob), _ptr(meta), _ptr(out["policy"]), _ptr(out["policyPass"]),
                                     _ptr(out["value"]), _ptr(out["scoreValue"]), _ptr(out["ownership"]), _ptr(trunk)), "ko_forward_meta")
        if want_trunk:
            out["trunk"] = trunk
        return out


def trunk_streams(model: OracleModel, spatial: np.ndarray, glob: np.ndarray, meta: np.ndarray | None = None) -> np.ndarray:
    """[numBlocks + 1][n][Y][X][trunkC]: the residual stream entering each block of the trunk and leaving the last."""
    n = spatial.shape[0]
    S = model.nn_x * model.nn_y
    spatial = np.ascontiguousarray(spatial, np.float32).reshape(n, S, model.in_c)
    glob = np.ascontiguousarray(glob, np.float32).reshape(n, model.in_global_c)
    if meta is not None:
        meta = np.ascontiguousarray(meta, np.float32)
    out = np.empty((model.num_blocks + 1, n, model.nn_y, model.nn_x, model.trunk_c), np.float32)
    _check(lib().ko_trunk_streams(model.h, n, _ptr(spatial), _ptr(glob), _ptr(meta), _ptr(out)), "ko_trunk_streams")
    return out


def eval_layer(blob: bytes, x: np.ndarray, mask: np.ndarray | None, out_c: int) -> np.ndarray:
    """x [n,Y,X,C] NHWC, mask [n,Y,X] -> [n,Y,X,out_c]."""
    n, ylen, xlen, _ = x.shape
    x = np.ascontiguousarray(x, np.float32)
    m = None if mask is None else np.ascontiguousarray(mask, np.float32)
    out = np.empty((n, ylen, xlen, out_c), np.float32)
    _check(lib().ko_eval_layer(blob, len(blob), n, xlen, ylen, _ptr(x), _ptr(m), _ptr(out)), "ko_eval_layer")
    return out


def num_threads() -> int:
    return int(lib().ko_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of forward passes started by the calling thread from now on."""
    if lib().ko_set_num_threads(int(n)) != 0:
        raise RuntimeError("ko_set_num_threads failed")


def set_storage_emulation(storage: str | None, conv_inputs: bool = True, streams: bool = True) -> None:
    """Rounds the chosen tensors to "fp16" / "bf16" where a reduced-precision backend stores them (None: off).  For
    measuring precision floors only; process-wide."""
    code = {None: 0, "fp16": 1, "bf16": 2}[storage]
    lib().ko_set_storage_emulation(code, (1 if conv_inputs else 0) | (2 if streams else 0))
