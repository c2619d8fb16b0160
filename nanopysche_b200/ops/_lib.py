"""ctypes binding to the in-tree sm_100a kernel library (``lib/libnpb200.so``).

The library exports plain C entry points that take device pointers and a CUDA stream; the wrappers
in ``ops/`` pass ``tensor.data_ptr()`` and the current torch stream, so every kernel runs in stream
order with the surrounding torch ops and can be captured into CUDA graphs by the caller.

On a box with a GPU the library is mandatory: ``lib()`` raises if it cannot be loaded (there is no
silent eager fallback on CUDA tensors). On a CPU-only box the ops use their PyTorch reference.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB = None
_LIB_ERR: str | None = None
LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libnpb200.so"

c_void_p, c_int, c_ll, c_ull, c_float = C.c_void_p, C.c_int, C.c_longlong, C.c_ulonglong, C.c_float


class GemmArgs(C.Structure):
    """Mirror of ``NpGemmArgs`` in csrc/gemm_sm100.cu (field order matters)."""

    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("B2", c_void_p), ("C", c_void_p), ("C2", c_void_p),
        ("lda", c_ll), ("ldb", c_ll), ("ldc", c_ll), ("ldc2", c_ll),
        ("a_rows", c_ll), ("b_rows", c_ll),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("a_mn", c_int), ("b_mn", c_int), ("out_f32", c_int), ("accumulate", c_int),
        ("epilogue", c_int), ("mode", c_int),
        ("alpha", c_float),
        ("mblk_group", c_void_p), ("mblk_rows", c_void_p), ("group_stride_b", c_ll),
        ("num_groups", c_int), ("blocks_per_group", c_int), ("group_stride_c", c_ll),
        ("ready_flags", c_void_p), ("mblk_flag", c_void_p), ("epoch", c_int), ("flag_limit_ns", c_ull),
        ("row_dst", c_void_p), ("peer_base", c_void_p),
        ("done_counters", c_void_p), ("done_expected", c_void_p), ("done_flag_ptr", c_void_p),
        ("bn", c_int), ("max_ctas", c_int),
        ("Cin", c_void_p), ("ldcin", c_ll), ("epoch_base", c_void_p),
        ("b_ready_flags", c_void_p), ("b_rows_per_flag", c_int),
        ("A_loc", c_void_p), ("lda_loc", c_ll), ("a_loc_lo", c_int), ("a_loc_hi", c_int),
        ("B_loc", c_void_p), ("ldb_loc", c_ll), ("b_loc_lo", c_int), ("b_loc_hi", c_int),
        ("b_local_flag", c_int), ("m_rot", c_int), ("n_rot", c_int),
        ("push_src", c_void_p), ("push_bytes", c_ll), ("push_dst", c_void_p), ("push_flag", c_void_p),
        ("push_n", c_int), ("push_ctr", c_void_p),
        ("bias", c_void_p),
        ("mt", c_int),
    ]


class DispatchArgs(C.Structure):
    """Mirror of ``NpDispatchArgs`` in csrc/moe.cu."""

    _fields_ = [
        ("x", c_void_p), ("indices", c_void_p), ("slot_pos", c_void_p), ("counts_kept", c_void_p),
        ("slot_scale", c_void_p),
        ("T", c_int), ("K", c_int), ("D", c_int), ("E", c_int), ("E_local", c_int), ("n_ranks", c_int),
        ("my_rank", c_int), ("region_rows", c_int), ("quant", c_int),
        ("peer_rows", c_void_p), ("peer_scales", c_void_p), ("peer_row_dst", c_void_p),
        ("peer_mblk_rows", c_void_p), ("peer_src_blocks", c_void_p), ("peer_flags", c_void_p),
        ("done_ctr", c_void_p), ("epoch", c_int), ("write_meta", c_int), ("max_ctas", c_int),
        ("epoch_base", c_void_p),
    ]


class CombineArgs(C.Structure):
    """Mirror of ``NpCombineArgs`` in csrc/moe.cu."""

    _fields_ = [
        ("rows", c_void_p), ("slot_pos", c_void_p), ("weights", c_void_p), ("add1", c_void_p),
        ("add2", c_void_p), ("dl", c_void_p), ("wg", c_void_p), ("out", c_void_p),
        ("T", c_int), ("K", c_int), ("D", c_int), ("E", c_int),
        ("flags", c_void_p), ("sent_to_peer", c_void_p), ("n_ranks", c_int), ("epoch", c_int),
        ("limit_ns", c_ull), ("epoch_base", c_void_p),
    ]


class AttnFwdArgs(C.Structure):
    """Mirror of ``NpAttnFwdArgs`` in csrc/attn_sm100.cu."""

    _fields_ = [
        ("q", c_void_p), ("q_sb", c_ll), ("q_ss", c_ll), ("q_sh", c_ll),
        ("k_ptrs", c_void_p), ("v_ptrs", c_void_p), ("k_sb", c_ll), ("k_ss", c_ll), ("k_sh", c_ll),
        ("o", c_void_p), ("o_sb", c_ll), ("o_ss", c_ll), ("o_sh", c_ll),
        ("lse", c_void_p),
        ("B", c_int), ("Sq", c_int), ("Hq", c_int), ("Hkv", c_int), ("causal", c_int), ("n_src", c_int),
        ("src_len", c_int), ("q_off", c_int),
        ("scale", c_float),
        ("q_blk_pos", c_void_p), ("k_blk_pos", c_void_p),
        ("split", c_int), ("lse_heads", c_int),
        ("src_flags", c_void_p), ("flag_idx", c_void_p), ("flag_epoch", c_int), ("epoch_base", c_void_p),
        ("flag_limit_ns", c_ull), ("flag_own", c_int),
        ("push_k", c_void_p), ("push_v", c_void_p), ("push_bytes", c_ll), ("push_dst", c_void_p),
        ("push_flag", c_void_p), ("push_n", c_int), ("push_ctr", c_void_p),
    ]


class AttnBwdArgs(C.Structure):
    """Mirror of ``NpAttnBwdArgs`` in csrc/attn_sm100.cu."""

    _fields_ = [
        ("q", c_void_p), ("q_sb", c_ll), ("q_ss", c_ll), ("q_sh", c_ll),
        ("k", c_void_p), ("v", c_void_p), ("k_sb", c_ll), ("k_ss", c_ll), ("k_sh", c_ll),
        ("o", c_void_p), ("o_sb", c_ll), ("o_ss", c_ll), ("o_sh", c_ll),
        ("d_o", c_void_p), ("do_sb", c_ll), ("do_ss", c_ll), ("do_sh", c_ll),
        ("lse", c_void_p), ("delta", c_void_p),
        ("dq", c_void_p), ("dq_sb", c_ll), ("dq_ss", c_ll), ("dq_sh", c_ll),
        ("dk", c_void_p), ("dv", c_void_p), ("dk_sb", c_ll), ("dk_ss", c_ll), ("dk_sh", c_ll),
        ("k_src", c_void_p), ("v_src", c_void_p), ("q_src", c_void_p), ("do_src", c_void_p),
        ("lse_src", c_void_p), ("delta_src", c_void_p),
        ("B", c_int), ("Sq", c_int), ("Sk", c_int), ("Hq", c_int), ("Hkv", c_int), ("causal", c_int),
        ("n_src", c_int), ("q_off", c_int), ("phase", c_int),
        ("scale", c_float),
        ("q_blk_pos_local", c_void_p), ("k_blk_pos_all", c_void_p),
        ("k_blk_pos_local", c_void_p), ("q_blk_pos_all", c_void_p),
        ("split", c_int), ("lse_heads", c_int),
        ("src_flags", c_void_p), ("flag_idx", c_void_p), ("flag_epoch", c_int), ("epoch_base", c_void_p),
        ("flag_limit_ns", c_ull), ("flag_which", c_int), ("skip", c_int), ("flag_own", c_int),
        ("push_k", c_void_p), ("push_v", c_void_p), ("push_bytes", c_ll), ("push_dst", c_void_p),
        ("push_flag", c_void_p), ("push_n", c_int), ("push_ctr", c_void_p),
    ]


class Fp8GemmArgs(C.Structure):
    """Mirror of ``NpFp8GemmArgs`` in csrc/gemm_fp8_sm100.cu."""

    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p), ("sa", c_void_p), ("sb", c_void_p),
        ("lda", c_ll), ("ldb", c_ll), ("ldc", c_ll), ("a_rows", c_ll), ("b_rows", c_ll),
        ("M", c_int), ("N", c_int), ("K", c_int), ("out_f32", c_int), ("mode", c_int),
        ("mblk_group", c_void_p), ("mblk_rows", c_void_p), ("group_stride_b", c_ll),
        ("ready_flags", c_void_p), ("mblk_flag", c_void_p), ("epoch", c_int), ("epoch_base", c_void_p),
        ("flag_limit_ns", c_ull),
        ("row_dst", c_void_p), ("peer_base", c_void_p),
        ("done_counters", c_void_p), ("done_expected", c_void_p), ("done_flag_ptr", c_void_p),
        ("max_ctas", c_int),
    ]


class MxGemmArgs(C.Structure):
    """Mirror of ``NpMxGemmArgs`` in csrc/gemm_mxfp8_sm100.cu."""

    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p), ("sfa", c_void_p), ("sfb", c_void_p),
        ("lda", c_ll), ("ldb", c_ll), ("ldc", c_ll), ("a_rows", c_ll), ("b_rows", c_ll),
        ("M", c_int), ("N", c_int), ("K", c_int), ("out_f32", c_int), ("mode", c_int),
        ("mblk_group", c_void_p), ("mblk_rows", c_void_p), ("group_stride_b", c_ll),
        ("max_ctas", c_int),
        ("ready_flags", c_void_p), ("mblk_flag", c_void_p), ("epoch", c_int), ("epoch_base", c_void_p),
        ("flag_limit_ns", c_ull),
        ("row_dst", c_void_p), ("peer_base", c_void_p),
        ("done_counters", c_void_p), ("done_expected", c_void_p), ("done_flag_ptr", c_void_p),
    ]


class KernelError(RuntimeError):
    """A kernel launch failed or a kernel reported a device-side status (timeout, bounds)."""


STATUS_NAMES = {0: "ok", 1: "mbarrier wait timed out", 2: "flag wait timed out", 3: "bad argument",
                4: "bounds check failed"}


def load_error() -> str | None:
    return _LIB_ERR


def lib():
    """Load (building first if the .so is missing and nvcc exists) and return the ctypes library."""
    global _LIB, _LIB_ERR
    if _LIB is not None:
        return _LIB
    if not LIB_PATH.exists():
        try:
            from ..build import build_extension

            build_extension()
        except Exception as e:  # noqa: BLE001
            _LIB_ERR = f"build failed: {e}"
            raise KernelError(f"libnpb200.so missing and could not be built: {e}") from e
    try:
        _LIB = C.CDLL(str(LIB_PATH))
    except OSError as e:
        _LIB_ERR = str(e)
        raise KernelError(f"cannot load {LIB_PATH}: {e}") from e
    _LIB.np_gemm_bf16.argtypes = [C.POINTER(GemmArgs), c_void_p]
    _LIB.np_ep_dispatch.argtypes = [C.POINTER(DispatchArgs), c_void_p]
    _LIB.np_ep_combine.argtypes = [C.POINTER(CombineArgs), c_void_p]
    _LIB.np_gemm_fp8_block.argtypes = [C.POINTER(Fp8GemmArgs), c_void_p]
    _LIB.np_gemm_mxfp8.argtypes = [C.POINTER(MxGemmArgs), c_void_p]
    _LIB.np_mx_quant.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p]
    _LIB.np_flow_quant_act.argtypes = [c_void_p, c_ll, c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_void_p, c_ll,
                                        c_void_p]
    _LIB.np_mx_dequant.argtypes = [c_void_p, c_ll, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]
    _LIB.np_flow_quant_weight.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                           c_void_p]
    _LIB.np_attn_fwd.argtypes = [C.POINTER(AttnFwdArgs), c_void_p]
    _LIB.np_attn_bwd.argtypes = [C.POINTER(AttnBwdArgs), c_void_p]
    _LIB.np_status_read.argtypes = [C.POINTER(c_int)]
    return _LIB


def available() -> bool:
    """True when CUDA tensors should go through the kernels (a GPU is present)."""
    return torch.cuda.is_available()


# True: every op takes its PyTorch statement even on CUDA tensors (the plain library-call arm); NPB200_PLAIN=1 sets it
PLAIN = os.environ.get("NPB200_PLAIN", "0") == "1"


def set_plain(flag: bool) -> None:
    """Route all ops to their PyTorch reference (cuBLAS / SDPA / ATen) regardless of device. Used by the plain
    baseline arm of the benchmarks, which runs the same model through library calls and NCCL collectives."""
    global PLAIN
    PLAIN = bool(flag)


def on(t: torch.Tensor) -> bool:
    """True when ``t`` should go through the sm_100a kernels."""
    return t.is_cuda and not PLAIN


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


NVTX = os.environ.get("NPB200_NVTX", "0") == "1"   # wrap library calls and model blocks in NVTX ranges


class nvtx_range:
    """``with nvtx_range("name"):`` pushes an NVTX range when ``NPB200_NVTX=1`` (profilers show the fused kernels and
    the blocks of the model by name); free otherwise."""

    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if NVTX:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if NVTX:
            torch.cuda.nvtx.range_pop()
        return False


LAUNCHES = 0  # number of successful calls into the kernel library (each launches >= 1 kernel)


def check(rc: int, name: str) -> None:
    global LAUNCHES
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")
    LAUNCHES += 1


def status() -> tuple[int, ...]:
    """Read the device status words (synchronises the device)."""
    buf = (c_int * 8)()
    lib().np_status_read(buf)
    return tuple(buf)


def check_status(where: str = "") -> None:
    st = status()
    if st[0] != 0:
        lib().np_status_clear()
        raise KernelError(
            f"device status {st[0]} ({STATUS_NAMES.get(st[0], '?')}) kernel={st[1]} block={st[2]} "
            f"detail={st[3]} {where}")


def wait_stats(reset: bool = False) -> dict | None:
    """Communication time the kernels accounted since the last reset: ``exposed_ms`` is the mean over the SMs of
    the time an SM spent polling a flag a peer had not raised yet or running a transfer-only kernel (dispatch
    pushes, gradient reduce-scatter loads, weight all-gather stores, barriers). Synchronises the device."""
    if not torch.cuda.is_available():
        return None
    n = lib().np_wait_stats_slots()
    buf = (c_ull * n)()
    if lib().np_wait_stats_read(buf, int(reset)) != 0:
        return None
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    vals = list(buf)[:min(sms, n)]
    return {"exposed_ms": sum(vals) / max(len(vals), 1) / 1e6, "max_sm_ms": max(vals) / 1e6 if vals else 0.0}


def call(name: str, *args) -> None:
    """Call ``np_<name>`` with the current stream appended; scalars are wrapped by type."""
    fn = getattr(lib(), "np_" + name)
    conv = []
    for a in args:
        if isinstance(a, torch.Tensor):
            conv.append(c_void_p(a.data_ptr()))
        elif a is None:
            conv.append(c_void_p(0))
        elif isinstance(a, float):
            conv.append(c_float(a))
        elif isinstance(a, LL):
            conv.append(c_ll(int(a)))
        elif isinstance(a, (bool, int)):
            conv.append(c_int(int(a)))
        else:
            conv.append(a)
    conv.append(c_void_p(stream()))
    if NVTX:
        torch.cuda.nvtx.range_push("np_" + name)
        try:
            check(fn(*conv), name)
        finally:
            torch.cuda.nvtx.range_pop()
        return
    check(fn(*conv), name)


class LL(int):
    """Marks an integer argument that the C side takes as ``long long``."""
