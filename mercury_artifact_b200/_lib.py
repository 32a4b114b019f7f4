"""ctypes binding of libmercury_b200.so (the C ABI declared in include/mercury_b200.h).

The library is the product: there is no Python or CPU fallback.  If the shared
object is missing the import of this module raises, and every op raises when a
call returns a non-zero code.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

MB_MAX_SEGMENTS = 32
MB_MAX_JOBS = 40

MB_SUCCESS = 0
ERROR_NAMES = {
    -1: "MB_E_INVALID (bad argument)",
    -2: "MB_E_UNSUPPORTED (shape or option not implemented by the sm_100a kernels)",
    -3: "MB_E_CUDA (a CUDA runtime call failed)",
    -4: "MB_E_TENSORMAP (TMA descriptor rejected: check 16-byte alignment of pointers and strides)",
    -5: "MB_E_DEVICE (device-side wait timed out)",
    -6: "MB_E_TOO_LARGE (exceeds the fixed scratch of the allocation-free entry point: batch*hq*pad64(sq) > 1048576)",
}

STATUS_NAMES = {
    101: "Q tile never arrived",
    102: "K/V stage never filled",
    103: "K/V stage never released",
    104: "score tile never completed",
    105: "probabilities never written",
    106: "output accumulation never completed",
    107: "staged shard chunk never became ready",
    108: "unspecified wait",
    109: "a K/V shard's arrival flag never reached its value (in-kernel wait)",
}


class KVSegment(C.Structure):
    _fields_ = [
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("stride_b", C.c_int64),
        ("stride_s", C.c_int64),
        ("stride_h", C.c_int64),
        ("sk", C.c_int32),
        ("k_off", C.c_int32),
        ("ready_flag", C.c_void_p),
        ("ready_value", C.c_int32),
        ("reserved", C.c_int32),
    ]


class AttnFwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("q_stride_b", C.c_int64),
        ("q_stride_s", C.c_int64),
        ("q_stride_h", C.c_int64),
        ("o", C.c_void_p),
        ("o_stride_b", C.c_int64),
        ("o_stride_s", C.c_int64),
        ("o_stride_h", C.c_int64),
        ("lse", C.c_void_p),
        ("lse_stride_b", C.c_int64),
        ("lse_stride_h", C.c_int64),
        ("batch", C.c_int32),
        ("sq", C.c_int32),
        ("hq", C.c_int32),
        ("hkv", C.c_int32),
        ("head_dim", C.c_int32),
        ("q_off", C.c_int32),
        ("causal", C.c_int32),
        ("softmax_scale", C.c_float),
        ("nseg", C.c_int32),
        ("seg", KVSegment * MB_MAX_SEGMENTS),
        ("status", C.c_void_p),
    ]


class FwdJob(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("q_stride_b", C.c_int64),
        ("q_stride_s", C.c_int64),
        ("q_stride_h", C.c_int64),
        ("o", C.c_void_p),
        ("o_stride_b", C.c_int64),
        ("o_stride_s", C.c_int64),
        ("o_stride_h", C.c_int64),
        ("lse", C.c_void_p),
        ("lse_stride_b", C.c_int64),
        ("lse_stride_h", C.c_int64),
        ("sq", C.c_int32),
        ("q_off", C.c_int32),
        ("seg_mask", C.c_uint32),
        ("reserved", C.c_int32),
        ("q_ready_flag", C.c_void_p),
        ("q_ready_value", C.c_int32),
        ("done_value", C.c_int32),
        ("done_flag", C.c_void_p),
        ("done_counter", C.c_void_p),
        ("state_o", C.c_void_p),
        ("state_ml", C.c_void_p),
        ("state_in", C.c_int32),
        ("state_out", C.c_int32),
        ("chain", C.c_void_p),
        ("chain_wait", C.c_int32),
        ("chain_set", C.c_int32),
    ]


class AttnFwdMultiArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32),
        ("hq", C.c_int32),
        ("hkv", C.c_int32),
        ("head_dim", C.c_int32),
        ("causal", C.c_int32),
        ("softmax_scale", C.c_float),
        ("njobs", C.c_int32),
        ("nseg", C.c_int32),
        ("job", FwdJob * MB_MAX_JOBS),
        ("seg", KVSegment * MB_MAX_SEGMENTS),
        ("status", C.c_void_p),
    ]


MB_MAX_PULL_RANGES = 8
MB_MAX_PULL_FLAGS = 4


class PullRange(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("bytes", C.c_uint64)]


class PullArgs(C.Structure):
    _fields_ = [
        ("nranges", C.c_int32),
        ("nflags", C.c_int32),
        ("range", PullRange * MB_MAX_PULL_RANGES),
        ("wait_flag", C.c_void_p),
        ("wait_value", C.c_int32),
        ("ctas", C.c_int32),
        ("flag", C.c_void_p * MB_MAX_PULL_FLAGS),
        ("value", C.c_int32 * MB_MAX_PULL_FLAGS),
        ("counter", C.c_void_p),
        ("status", C.c_void_p),
    ]


MB_DTYPE_BF16 = 0
MB_DTYPE_F32 = 1


class MergeArgs(C.Structure):
    _fields_ = [
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("block_out", C.c_void_p),
        ("block_stride_b", C.c_int64),
        ("block_stride_s", C.c_int64),
        ("block_stride_h", C.c_int64),
        ("block_lse", C.c_void_p),
        ("batch", C.c_int32),
        ("seq", C.c_int32),
        ("heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("first", C.c_int32),
        ("block_dtype", C.c_int32),
    ]


MB_BWD_MODE_DKV = 1
MB_BWD_MODE_DQ = 0
MB_BWD_MODE_FUSED = 2
MB_OUT_BF16 = 0
MB_OUT_F32 = 1
MB_OUT_F32_ACCUM = 2


class BwdPreprocessArgs(C.Structure):
    _fields_ = [
        ("dout", C.c_void_p),
        ("dout_stride_b", C.c_int64),
        ("dout_stride_s", C.c_int64),
        ("dout_stride_h", C.c_int64),
        ("out", C.c_void_p),
        ("out_stride_b", C.c_int64),
        ("out_stride_s", C.c_int64),
        ("out_stride_h", C.c_int64),
        ("lse", C.c_void_p),
        ("lse2", C.c_void_p),
        ("delta", C.c_void_p),
        ("batch", C.c_int32),
        ("sq", C.c_int32),
        ("hq", C.c_int32),
        ("head_dim", C.c_int32),
        ("stat_pad", C.c_int32),
    ]


class BwdSegment(C.Structure):
    _fields_ = [
        ("str", C.c_void_p),
        ("str_g", C.c_void_p),
        ("stride_b", C.c_int64),
        ("stride_s", C.c_int64),
        ("stride_h", C.c_int64),
        ("rows", C.c_int32),
        ("pos_off", C.c_int32),
        ("lse2", C.c_void_p),
        ("delta", C.c_void_p),
        ("stat_pad", C.c_int32),
        ("ready_value", C.c_int32),
        ("ready_flag", C.c_void_p),
        ("dq_accum", C.c_void_p),
    ]


class AttnBwdArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int32),
        ("out_mode", C.c_int32),
        ("own", C.c_void_p),
        ("own_g", C.c_void_p),
        ("own_stride_b", C.c_int64),
        ("own_stride_s", C.c_int64),
        ("own_stride_h", C.c_int64),
        ("own_lse2", C.c_void_p),
        ("own_delta", C.c_void_p),
        ("own_stat_pad", C.c_int32),
        ("own_rows", C.c_int32),
        ("own_off", C.c_int32),
        ("batch", C.c_int32),
        ("hq", C.c_int32),
        ("hkv", C.c_int32),
        ("head_dim", C.c_int32),
        ("causal", C.c_int32),
        ("softmax_scale", C.c_float),
        ("out1", C.c_void_p),
        ("out2", C.c_void_p),
        ("out_stride_b", C.c_int64),
        ("out_stride_s", C.c_int64),
        ("out_stride_h", C.c_int64),
        ("nseg", C.c_int32),
        ("reserved", C.c_int32),
        ("seg", BwdSegment * MB_MAX_SEGMENTS),
        ("status", C.c_void_p),
    ]


class AttnBwdBlockArgs(C.Structure):
    _fields_ = [
        ("dout", C.c_void_p),
        ("q", C.c_void_p),
        ("out", C.c_void_p),
        ("q_stride_b", C.c_int64),
        ("q_stride_s", C.c_int64),
        ("q_stride_h", C.c_int64),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("kv_stride_b", C.c_int64),
        ("kv_stride_s", C.c_int64),
        ("kv_stride_h", C.c_int64),
        ("lse", C.c_void_p),
        ("dq", C.c_void_p),
        ("dq_stride_b", C.c_int64),
        ("dq_stride_s", C.c_int64),
        ("dq_stride_h", C.c_int64),
        ("dk", C.c_void_p),
        ("dv", C.c_void_p),
        ("dkv_stride_b", C.c_int64),
        ("dkv_stride_s", C.c_int64),
        ("dkv_stride_h", C.c_int64),
        ("batch", C.c_int32),
        ("sq", C.c_int32),
        ("sk", C.c_int32),
        ("hq", C.c_int32),
        ("hkv", C.c_int32),
        ("head_dim", C.c_int32),
        ("q_off", C.c_int32),
        ("k_off", C.c_int32),
        ("causal", C.c_int32),
        ("out_mode", C.c_int32),
        ("softmax_scale", C.c_float),
        ("status", C.c_void_p),
    ]


import os as _os

# MERCURY_B200_LIB selects another build of the same library (kernel tuning experiments).
LIB_PATH = Path(_os.environ.get("MERCURY_B200_LIB") or (Path(__file__).resolve().parent / "libmercury_b200.so"))


class MercuryB200Error(RuntimeError):
    pass


_SIGNATURES = {
    "mb_version": [],
    "mb_attn_fwd": [C.POINTER(AttnFwdArgs), C.c_void_p],
    "mb_attn_fwd_multi": [C.POINTER(AttnFwdMultiArgs), C.c_void_p],
    "mb_attn_bwd_preprocess": [C.POINTER(BwdPreprocessArgs), C.c_void_p],
    "mb_attn_bwd": [C.POINTER(AttnBwdArgs), C.c_void_p],
    "mb_attn_bwd_dq_convert": [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                               C.c_int32, C.c_int32, C.c_float, C.c_void_p],
    "mb_attn_bwd_block_noalloc": [C.POINTER(AttnBwdBlockArgs), C.c_void_p],
    "mb_merge_out_lse": [C.POINTER(MergeArgs), C.c_void_p],
    "mb_tree_merge": [C.POINTER(C.c_void_p), C.c_int32, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p],
    "mb_flash_reduce": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p],
    "mb_mem_alloc": [C.POINTER(C.c_void_p), C.c_uint64],
    "mb_mem_free": [C.c_void_p],
    "mb_mem_zero": [C.c_void_p, C.c_uint64, C.c_void_p],
    "mb_ipc_export": [C.c_void_p, C.POINTER(C.c_ubyte)],
    "mb_ipc_import": [C.POINTER(C.c_ubyte), C.POINTER(C.c_void_p)],
    "mb_ipc_release": [C.c_void_p],
    "mb_copy_async": [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p],
    "mb_flag_signal": [C.c_void_p, C.c_int32, C.c_void_p],
    "mb_flag_wait": [C.c_void_p, C.c_int32, C.c_uint64, C.c_void_p, C.c_void_p],
    "mb_flags_signal": [C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int32, C.c_void_p],
    "mb_flags_wait": [C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int32, C.c_uint64, C.c_void_p, C.c_void_p],
    "mb_pull_sm": [C.POINTER(PullArgs), C.c_void_p],
    "mb_copy2d_async": [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p],
    "mb_set_peer_wait_ms": [C.c_uint32],
    "mb_status_peek_async": [C.c_void_p, C.c_void_p],
    "mb_status_fetch": [C.POINTER(C.c_int32), C.c_void_p],
    "mb_last_cuda_error": [C.c_char_p, C.c_int32],
}


def _bind(path: Path) -> C.CDLL:
    handle = C.CDLL(str(path))
    try:
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError: the shared object predates this binding
            fn.restype = C.c_int
            fn.argtypes = argtypes
    except AttributeError:
        import _ctypes

        _ctypes.dlclose(handle._handle)  # otherwise a rebuilt file at the same path maps to the old image
        raise
    return handle


def _load() -> C.CDLL:
    """Load libmercury_b200.so; if it is missing, older than this binding, or -- where nvcc and the
    sources are at hand -- built from other sources than the ones on disk, rebuild it once with nvcc
    (under a file lock, so that the ranks of a job do not all compile into the same file).
    There is no other path: without the library the import fails."""
    from . import build as _build

    custom = bool(_os.environ.get("MERCURY_B200_LIB"))
    reason = None
    try:
        if LIB_PATH.exists():
            if custom or _build.find_nvcc() is None or _build.is_current():
                return _bind(LIB_PATH)
            reason = f"{LIB_PATH} was built from other sources than the ones on disk"
        else:
            reason = f"{LIB_PATH} is missing"
    except AttributeError as e:
        reason = f"{LIB_PATH} is stale ({e})"
    if custom or _build.find_nvcc() is None:
        raise ImportError(f"{reason} and nvcc is not available to build it "
                          "(python -m mercury_artifact_b200.build); there is no fallback path")
    _build.build()
    return _bind(LIB_PATH)


lib = _load()


def check(code: int, what: str) -> None:
    if code != MB_SUCCESS:
        detail = ""
        if code == -3:
            buf = C.create_string_buffer(256)
            if lib.mb_last_cuda_error(buf, 256) == MB_SUCCESS and buf.value:
                detail = ": " + buf.value.decode(errors="replace")
        raise MercuryB200Error(f"{what} failed: {ERROR_NAMES.get(code, code)}{detail}")


def status_fetch(stream_ptr: int) -> int:
    """Synchronise the stream and return (then clear) the device status word."""
    out = C.c_int32(0)
    check(lib.mb_status_fetch(C.byref(out), C.c_void_p(stream_ptr)), "mb_status_fetch")
    return int(out.value)


def set_peer_wait_ms(ms: int) -> None:
    """Budget of in-kernel waits for shards that other GPUs deliver (launches made afterwards)."""
    check(lib.mb_set_peer_wait_ms(C.c_uint32(int(ms))), "mb_set_peer_wait_ms")


# MB_PEER_WAIT_MS: how long a kernel (and a stream-level flag wait) waits for another rank before it
# gives up with a status code.  Default 30 s, far above the skew that first-call module loading, data
# loading or a checkpoint on one rank produce.
PEER_WAIT_MS = int(float(_os.environ.get("MB_PEER_WAIT_MS", "30000")))
set_peer_wait_ms(PEER_WAIT_MS)


class StatusMonitor:
    """Notices a timed-out device-side wait of an EARLIER call without synchronising.

    post(stream) enqueues a copy of the device status word into pinned host memory behind the work
    just queued; poll() looks at the copies that have completed and raises if one is non-zero.  Ops
    call poll() when they begin and post() when they have enqueued their work, so a timeout surfaces
    as an exception at the latest at the next call that finds the copy complete, or at check()."""

    def __init__(self):
        import torch

        self._torch = torch
        self._slots = []   # (pinned int32 tensor, event recorded behind the copy into it)
        self._free = []
        self._bad = 0

    def _reap(self) -> None:
        keep = []
        for host, ev in self._slots:
            if ev.query():
                self._bad = self._bad or int(host.item())
                self._free.append(host)
            else:
                keep.append((host, ev))
        self._slots = keep

    def post(self, stream) -> None:
        torch = self._torch
        self._reap()
        host = self._free.pop() if self._free else torch.zeros(1, dtype=torch.int32).pin_memory()
        check(lib.mb_status_peek_async(C.c_void_p(host.data_ptr()), C.c_void_p(stream.cuda_stream)),
              "mb_status_peek_async")
        ev = torch.cuda.Event()
        ev.record(stream)
        self._slots.append((host, ev))

    def poll(self) -> None:
        self._reap()
        if self._bad:
            bad, self._bad = self._bad, 0
            status_fetch(self._torch.cuda.current_stream().cuda_stream)   # synchronise and clear the device word
            raise MercuryB200Error(
                f"a device-side wait of an earlier call timed out: {STATUS_NAMES.get(bad, bad)} (code {bad}); "
                "the results of that call are invalid")


def raise_on_status(stream_ptr: int) -> None:
    st = status_fetch(stream_ptr)
    if st != 0:
        raise MercuryB200Error(f"device-side timeout: {STATUS_NAMES.get(st, st)} (code {st})")
