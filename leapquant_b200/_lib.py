"""ctypes binding of libleapquant_b200.so (the C ABI declared in include/leapquant_b200.h).

There is no fallback of any kind: if the library is missing, does not load, or a tensor is not on a CUDA device,
the call raises.  The library is built in-tree by `python -m leapquant_b200.csrc.build`.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# LEAPQUANT_B200_LIB points at another build of the same library (e.g. one compiled with different tuning macros)
LIB_PATH = os.environ.get("LEAPQUANT_B200_LIB") or os.path.join(_HERE, "libleapquant_b200.so")

EXPORTS = ("lq_version", "lq_strerror", "lq_last_cuda_error", "lq_device_status", "lq_set_option", "lq_gdn_step", "lq_kda_step",
           "lq_flush", "lq_gdn_decode", "lq_kda_decode", "lq_gdn_decode_conv", "lq_kda_decode_conv", "lq_causal_conv1d_update",
           "lq_decode_work_bytes", "lq_gdn_decode_noalloc",
           "lq_quantize", "lq_dequant", "lq_lowrank")

_P = ctypes.c_void_p
_I = ctypes.c_int32
_F = ctypes.c_float


class LqDims(ctypes.Structure):
    """struct lq_dims of include/leapquant_b200.h."""
    _fields_ = [("NS", _I), ("HV", _I), ("H", _I), ("K", _I), ("V", _I), ("L", _I), ("R", _I), ("SS", ctypes.c_int64)]


class LqConv1d(ctypes.Structure):
    """struct lq_conv1d of include/leapquant_b200.h."""
    _fields_ = [("x", _P), ("x_stride", ctypes.c_int64), ("state", _P), ("stride_slot", ctypes.c_int64), ("stride_dim", ctypes.c_int64),
                ("stride_tap", ctypes.c_int64), ("weight", _P), ("bias", _P), ("width", _I)]


class LeapQuantError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded library (loads on first use; raises if it is absent)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LeapQuantError(f"{LIB_PATH} is missing: build it with `python -m leapquant_b200.csrc.build` "
                                 "(leapquant_b200 has no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        D = ctypes.POINTER(LqDims)
        L.lq_version.restype = _I
        L.lq_strerror.restype = ctypes.c_char_p
        L.lq_strerror.argtypes = [_I]
        L.lq_last_cuda_error.restype = _I
        L.lq_device_status.argtypes = [ctypes.POINTER(_I)]
        L.lq_set_option.argtypes = [ctypes.c_char_p, _I]
        L.lq_set_option.restype = _I
        L.lq_gdn_step.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _F, _P]
        L.lq_kda_step.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _F, _F, _P]
        L.lq_flush.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P]
        I64 = ctypes.c_int64
        L.lq_gdn_decode.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _F, _P, _I, _P, I64, _P]
        L.lq_kda_decode.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _F, _F, _P, _I, _P, I64, _P]
        L.lq_gdn_decode_noalloc.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _F, _P, _I, _P]
        L.lq_decode_work_bytes.argtypes = [_I, _I]
        L.lq_decode_work_bytes.restype = I64
        C = ctypes.POINTER(LqConv1d)
        L.lq_gdn_decode_conv.argtypes = [D, _P, _P, _P, _P, _P, _P, C, _P, _P, _P, _P, _P, _P, _I, _F, _P, _I, _P, I64, _P]
        L.lq_kda_decode_conv.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, C, _P, _P, _P, _P, _P, _P, _I, _F, _F, _P, _I, _P, I64, _P]
        L.lq_causal_conv1d_update.argtypes = [C, _P, _I, _I, _I, _P, ctypes.c_int64, _P]
        L.lq_quantize.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P]
        L.lq_dequant.argtypes = [D, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _P]
        L.lq_lowrank.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P]
        for name in ("lq_device_status", "lq_gdn_step", "lq_kda_step", "lq_flush", "lq_quantize", "lq_dequant", "lq_lowrank",
                     "lq_gdn_decode", "lq_kda_decode", "lq_gdn_decode_conv", "lq_kda_decode_conv", "lq_causal_conv1d_update",
                     "lq_gdn_decode_noalloc"):
            getattr(L, name).restype = _I
        _lib = L
    return _lib


def check(rc, what):
    if rc != 0:
        L = lib()
        msg = L.lq_strerror(rc).decode()
        extra = f" (cudaError {L.lq_last_cuda_error()})" if rc == -5 else ""
        raise LeapQuantError(f"{what}: {msg}{extra}")


def dims(NS, HV, H, K, V, L, R, SS):
    return LqDims(int(NS), int(HV), int(H), int(K), int(V), int(L), int(R), int(SS))


def conv1d(x, conv_state, weight, bias):
    """struct lq_conv1d for one call: x bf16 [N, C'] (row stride free), conv_state bf16 viewed as (slot, channel, tap) with any
    strides (pass the engine's cache transposed if it is stored (slot, tap, channel)), weight bf16 [C, 4], bias bf16 [C] or None."""
    for t in (x, conv_state, weight) + ((bias,) if bias is not None else ()):
        if t.dtype != torch.bfloat16:
            raise LeapQuantError(f"the conv1d update works on bf16 tensors, got {t.dtype}")
    if x.stride(-1) != 1 or not weight.is_contiguous() or (bias is not None and not bias.is_contiguous()):
        raise LeapQuantError("conv1d update: x rows, weight and bias must be contiguous")
    if conv_state.dim() != 3 or conv_state.shape[2] != weight.shape[1] - 1:
        raise LeapQuantError(f"conv state must be (slot, channel, width - 1), got {tuple(conv_state.shape)}")
    return LqConv1d(ptr(x), x.stride(0), ptr(conv_state), conv_state.stride(0), conv_state.stride(1), conv_state.stride(2),
                    ptr(weight), ptr(bias) if bias is not None else None, int(weight.shape[1]))


def ptr(t):
    """Device address of a CUDA tensor's first element; refuses host tensors (no CPU path exists)."""
    if not t.is_cuda:
        raise LeapQuantError("leapquant_b200 kernels take CUDA tensors only (there is no CPU fallback)")
    return t.data_ptr()


def stream_of(t):
    return torch.cuda.current_stream(t.device).cuda_stream


class on_device:
    """Makes the tensor's device current for the duration of a launch when it is not already."""

    def __init__(self, t):
        self.idx = t.device.index
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


def set_option(name, value):
    """Process-wide tuning / debugging switch of the library (see lq_set_option in the header)."""
    check(lib().lq_set_option(name.encode(), int(value)), f"lq_set_option({name})")


def device_status():
    """Device-side status word (0 = clean); synchronises.  Debug / tests."""
    v = _I(0)
    check(lib().lq_device_status(ctypes.byref(v)), "lq_device_status")
    return v.value
