"""ctypes binding of libb2q.so (the C ABI declared in include/b2q.h).

The library is loaded eagerly and loudly: if libb2q.so is missing or a symbol is
absent the import fails; there is no CPU or eager-torch fallback anywhere in this
package.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb2q.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        "libb2q.so not found at %s; build it with `python llm-scaler_b200/build.py` "
        "(needs nvcc; cross-compiles for sm_100a without a GPU)" % LIB_PATH)

lib = C.CDLL(LIB_PATH)

vp, i32, i64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t

_SIGS = {
    "b2q_strerror": (C.c_char_p, [i32]),
    "b2q_version": (i32, []),
    "b2q_device_ok": (i32, []),
    "b2q_dequant_int4": (i32, [vp, i32, vp, i32, vp, i32, i64, i64, i32, vp]),
    "b2q_dequant_fp8": (i32, [vp, i32, vp, i32, i32, vp, i32, i64, i64, vp]),
    "b2q_resadd_rmsnorm": (i32, [vp, vp, vp, vp, i32, i64, i64, C.c_float, vp]),
    "b2q_quantize_fp8": (i32, [vp, i32, i64, vp, vp, i32, i64, i64, vp]),
    "b2q_rmsnorm_fused": (i32, [vp, vp, C.c_float, vp, vp, vp, vp, i32, i64, i64, C.c_float, vp]),
    "b2q_gated_rmsnorm": (i32, [vp, vp, vp, vp, i32, i64, i64, C.c_float, vp]),
    "b2q_quantize_q4_0": (i32, [vp, i32, i64, vp, vp, i64, i64, vp]),
    "b2q_linear_workspace_bytes": (sz, [i64, i64, i64]),
    "b2q_linear_int4": (i32, [vp, i32, i64, vp, i32, vp, i32, i64, i64, vp, i64, i64, i64, i64, i32, vp, sz, vp]),
    "b2q_linear_fp8_workspace_bytes": (sz, [i64, i64, i64]),
    "b2q_linear_fp8": (i32, [vp, i32, i64, vp, i32, vp, i32, i32, vp, i64, i64, i64, i64, vp, sz, vp]),
    "b2q_resadd_norm_linear_fp8": (i32, [vp, vp, vp, vp, C.c_float, C.c_float, i32, vp, i32, vp, i32, i32, vp, i64, i64, i64,
                                         i64, vp, sz, vp]),
    "b2q_act_quant_fp8_1x128": (i32, [vp, i32, i64, vp, vp, i64, i64, vp]),
    "b2q_gemm_fp8_block_w8a8": (i32, [vp, vp, vp, vp, vp, i32, i64, i64, i64, i64, vp]),
    "b2q_moe_topk": (i32, [vp, i32, i64, i32, i32, i32, vp, i32, vp, vp]),
    "b2q_moe_route_workspace_bytes": (sz, [i64, i32]),
    "b2q_moe_route": (i32, [vp, i64, i32, vp, vp, vp, vp, vp, sz, vp]),
    "b2q_moe_route_static": (i32, [vp, i64, i32, vp, vp, vp, vp, vp]),
    "b2q_gather_rows": (i32, [vp, vp, i32, vp, i64, i64, i32, vp]),
    "b2q_silu_mul": (i32, [vp, vp, i32, i64, i64, vp]),
    "b2q_gelu_tanh_mul": (i32, [vp, vp, i32, i64, i64, vp]),
    "b2q_moe_combine": (i32, [vp, vp, i32, vp, vp, i32, i64, i32, i64, i32, vp]),
    "b2q_moe_gemm_workspace_bytes": (sz, [i64, i32, i64, i64, i32, i32]),
    "b2q_moe_shared_gate_add": (i32, [vp, vp, vp, vp, vp, i32, i64, i64, vp]),
    "b2q_device_status": (i32, [vp]),
    "b2q_device_status_reset": (i32, []),
    "b2q_selftest_bounded_wait": (i32, [i32, vp, vp]),
    "b2q_moe_gemm_int4": (i32, [vp, i32, i64, vp, i32, vp, i32, vp, i32, vp, i32, vp, i64, vp,
                                i64, i64, i64, i32, i32, vp, sz, vp]),
    "b2q_moe_gemm_fp8": (i32, [vp, i32, i64, vp, i32, vp, i32, vp, i32, vp, i32, vp, i64, vp,
                               i64, i64, i64, i32, vp, sz, vp]),
    "b2q_comm_create": (i32, [i32, i32, i64, i64, vp, vp]),
    "b2q_comm_create_mode": (i32, [i32, i32, i64, i64, i32, vp, vp]),
    "b2q_comm_connect": (i32, [vp, vp]),
    "b2q_ep_create": (i32, [i32, i32, i64, i64, vp, vp]),
    "b2q_ep_connect": (i32, [vp, vp]),
    "b2q_ep_connect_local": (i32, [vp, i32]),
    "b2q_ep_destroy": (i32, [vp]),
    "b2q_ep_status": (i32, [vp, vp]),
    "b2q_ep_buffers": (i32, [vp, vp, vp, vp]),
    "b2q_ep_dispatch": (i32, [vp, vp, i32, i64, vp, i32, vp, vp, i64, vp]),
    "b2q_ep_return": (i32, [vp, vp, i32, i64, vp]),
    "b2q_ep_wait": (i32, [vp, i32, C.c_double, vp]),
    "b2q_comm_connect_local": (i32, [vp, i32]),
    "b2q_comm_destroy": (i32, [vp]),
    "b2q_comm_status": (i32, [vp, vp]),
    "b2q_comm_result_ptr": (i32, [vp, i32, vp]),
    "b2q_allreduce_sum": (i32, [vp, vp, i32, i64, i64, i64, C.c_double, vp, vp]),
    "b2q_linear_int4_allreduce": (i32, [vp, i32, i64, vp, i32, vp, i32, i64, i64, vp, i64, i64, i64, i64, i32, vp, sz, vp,
                                        C.c_double, vp, vp]),
    "b2q_allreduce_sum_emulated": (i32, [vp, i32, i32, vp, i32, i64, i64, i64, C.c_double, vp, vp]),
    "b2q_set_force_kernel": (None, [i32]),
    "b2q_set_overlap_mode": (None, [i32]),
    "b2q_last_kernel": (C.c_char_p, []),
    "b2q_launch_count": (C.c_uint64, []),
}

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)      # AttributeError here = header / library mismatch
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED = tuple(_SIGS)

BF16, F16, F32 = 0, 1, 2
W4_NMAJOR, W4_KMAJOR, W4_KMAJOR_MARLIN, W4_NMAJOR_S4 = 0, 1, 2, 3
E4M3, E5M2 = 0, 1
SCALE_CHANNEL, SCALE_TENSOR, SCALE_BLOCK128 = 0, 1, 2
ACT_NONE, ACT_SILU_MUL, ACT_SILU_MUL_IN, ACT_GELU_TANH_MUL = 0, 1, 2, 3
COMM_AUTO, COMM_ONE_STEP, COMM_TWO_STEPS = 0, 1, 2

_DT = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32}


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise RuntimeError("b2q: unsupported dtype %s" % t.dtype) from None


def fp8_fmt(t: torch.Tensor) -> int:
    if t.dtype == torch.float8_e5m2:
        return E5M2
    if t.dtype in (torch.float8_e4m3fn, torch.uint8, torch.int8):
        return E4M3
    raise RuntimeError("b2q: fp8 weight must be float8_e4m3fn / float8_e5m2 / uint8, got %s" % t.dtype)


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(lib.b2q_strerror(rc).decode())


def ptr(t):
    return None if t is None else t.data_ptr()


def stream(t: torch.Tensor):
    """Raw cudaStream_t of torch's current stream on the tensor's device."""
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("b2q: tensor must live on a CUDA device (no CPU path exists)")


class on_device:
    """Makes the tensor's device current for the duration of a launch."""

    __slots__ = ("g",)

    def __init__(self, t):
        # the common case (tensor on the current device) costs one integer compare, not a context switch
        idx = t.device.index
        self.g = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(idx)

    def __enter__(self):
        if self.g is not None:
            self.g.__enter__()

    def __exit__(self, *a):
        if self.g is not None:
            self.g.__exit__(*a)


def launch_count() -> int:
    return int(lib.b2q_launch_count())


def last_kernel() -> str:
    return lib.b2q_last_kernel().decode()


def device_status() -> int:
    """Code of the first expired device-side wait (0 = none); synchronises."""
    v = C.c_int(0)
    check(lib.b2q_device_status(C.addressof(v)))
    return int(v.value)


def device_status_reset() -> None:
    check(lib.b2q_device_status_reset())


def selftest_bounded_wait(code: int = 999) -> bool:
    """Runs the bounded-wait self-test on the current device; True when the wait gave up as it must."""
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib.b2q_selftest_bounded_wait(int(code), flag.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return int(flag.item()) == 1


def set_force_kernel(which: int) -> None:
    lib.b2q_set_force_kernel(int(which))


def set_overlap_mode(mode: int) -> None:
    """0 = no kernel overlap, 1 = pre-pass/GEMM overlap (default), 2 = also declare weights static
    (a GEMM may stream weights while earlier kernels of the stream are still draining)."""
    lib.b2q_set_overlap_mode(int(mode))


class DeviceView:
    """Exposes a range of device memory owned by libb2q.so to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int, owner=None):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def view_as_tensor(ptr: int, shape, dtype: torch.dtype, device, owner=None) -> torch.Tensor:
    n = 1
    for d in shape:
        n *= int(d)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return torch.as_tensor(DeviceView(ptr, nbytes, owner), device=device).view(dtype).view(*shape)
