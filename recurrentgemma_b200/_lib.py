"""ctypes binding of librgk.so (the C ABI declared in include/rgk.h).

There is no CPU implementation behind these calls: if the shared library has not been built, or
the tensors are not on a CUDA device of compute capability 10.x, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# RGK_LIBRARY selects another build of the library, e.g. librgk_checks.so (range-checked indices)
LIB_PATH = os.environ.get("RGK_LIBRARY") or os.path.join(_HERE, "librgk.so")

RGK_F32, RGK_BF16 = 0, 1
# rgk_status codes of include/rgk.h
(RGK_OK, RGK_EINVAL, RGK_ESHAPE, RGK_EALIGN, RGK_EARCH, RGK_ECUDA, RGK_EWORKSPACE,
 RGK_ETIMEOUT, RGK_EBOUNDS) = 0, -1, -2, -3, -4, -5, -6, -7, -8
RGK_I32, RGK_I64 = 0, 1
ACT_NONE, ACT_GELU_TANH, ACT_GEGLU = 0, 1, 2
GATES_AUTO, GATES_SIMT, GATES_TCGEN05, GATES_FUSED, GATES_FUSED_EXACT = 0, 1, 2, 3, 4

_vp, _i64, _int, _sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t


class RgkParams(ctypes.Structure):
  """struct rgk_params of include/rgk.h."""
  _fields_ = [(n, _vp) for n in ("conv_w", "conv_b", "a_param", "gate_x_w", "gate_x_b", "gate_a_w",
                                 "gate_a_b", "gates_packed")]


class RgkBlockParams(ctypes.Structure):
  """struct rgk_block_params of include/rgk.h."""
  _fields_ = [("path", RgkParams)] + [(n, _vp) for n in (
      "linear_y_w", "linear_y_b", "linear_x_w", "linear_x_b", "linear_out_w", "linear_out_b")]


# name -> (restype, argtypes); mirrors include/rgk.h declaration by declaration.
SIGNATURES = {
    "rgk_abi_version": (_int, []),
    "rgk_last_error": (ctypes.c_char_p, []),
    "rgk_device_check": (_int, []),
    "rgk_set_conv_fusion": (_int, [_int]),
    "rgk_conv1d_prefill": (_int, [_vp, _vp, _int, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _vp,
                                  _vp]),
    "rgk_conv1d_decode": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "rgk_blockdiag_linear": (_int, [_vp, _vp, _vp, _i64, _int, _int, _int, _vp, _vp]),
    "rgk_linear_scan": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp, _sz,
                               _vp]),
    "rgk_linear_scan_static": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp,
                                      _vp]),
    "rgk_rglru_forward": (_int, [_vp, _vp, _int, ctypes.POINTER(RgkParams), _vp, _i64, _i64, _i64,
                                 _int, _int, _int, _vp, _vp, _vp, _sz, _vp]),
    "rgk_recurrent_path_prefill": (_int, [_vp, _vp, _vp, _int, ctypes.POINTER(RgkParams), _vp, _i64,
                                          _i64, _i64, _int, _int, _int, _int, _vp, _vp, _vp, _vp,
                                          _sz, _vp]),
    "rgk_recurrent_path_decode": (_int, [_vp, _vp, _vp, _int, ctypes.POINTER(RgkParams), _vp, _vp,
                                         _i64, _i64, _int, _int, _int, _int, _vp, _vp, _vp, _vp,
                                         _sz, _vp]),
    "rgk_gate_pack_bytes": (_sz, [_int]),
    "rgk_gate_pack_bytes_for": (_sz, [_int, _int]),
    "rgk_pack_gate_weights": (_int, [ctypes.POINTER(RgkParams), _int, _int, _int, _vp, _vp]),
    "rgk_dense_linear": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "rgk_block_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _int]),
    "rgk_recurrent_block_prefill": (_int, [_vp, _vp, _int, ctypes.POINTER(RgkBlockParams), _i64,
                                           _i64, _i64, _i64, _int, _int, _int, _vp, _vp, _vp, _vp,
                                           _sz, _vp]),
    "rgk_rmsnorm": (_int, [_vp, _vp, _i64, _i64, ctypes.c_float, _int, _vp, _vp]),
    "rgk_residual_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64, _int]),
    "rgk_residual_block_prefill": (_int, [_vp, _vp, _int, ctypes.POINTER(RgkBlockParams), _vp,
                                          ctypes.c_float, _i64, _i64, _i64, _i64, _int, _int, _int,
                                          _vp, _vp, _vp, _vp, _sz, _vp]),
    "rgk_mlp_pack_bytes": (_sz, [_i64, _i64]),
    "rgk_pack_mlp_up": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp]),
    "rgk_mlp_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "rgk_mlp_block": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _sz, _vp]),
    "rgk_residual_channel": (_int, [_vp, _vp, ctypes.c_float, _vp, _vp, _vp, _i64, _i64, _i64, _int,
                                    _vp, _vp, _sz, _vp]),
    "rgk_rope": (_int, [_vp, _vp, _int, _i64, _int, _int, _int, _vp]),
    "rgk_attention_workspace_bytes": (_sz, [_i64, _i64]),
    "rgk_local_attention_prefill": (_int, [_vp, _vp, _vp, _vp, _int, _i64, _i64, _int, _int, _int,
                                           _int, _vp, _vp, _sz, _vp]),
    "rgk_attention_decode_workspace_bytes": (_sz, [_i64, _int, _int]),
    "rgk_local_attention_decode": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _int, _int, _int, _int,
                                          _int, _vp, _vp, _sz, _vp]),
    "rgk_dense_linear_small": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _vp, _vp]),
    "rgk_dense_linear_small_pair": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _int, _vp,
                                           _vp, _vp, _vp]),
    "rgk_embed": (_int, [_vp, _int, _vp, _i64, _i64, _i64, ctypes.c_float, _int, _vp, _vp]),
    "rgk_logits": (_int, [_vp, _vp, _i64, _i64, _i64, ctypes.c_float, _int, _vp, _vp, _vp]),
    "rgk_argmax": (_int, [_vp, _i64, _i64, _int, _vp, _vp]),
    "rgk_add_rmsnorm": (_int, [_vp, _vp, _vp, _i64, _i64, ctypes.c_float, _int, _vp, _vp, _vp]),
    "rgk_geglu_bias": (_int, [_vp, _vp, _i64, _i64, _int, _vp, _vp]),
    "rgk_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "rgk_workspace_status": (_int, [_vp, _vp]),
    "rgk_selftest_wait_expiry": (_int, [_vp, _sz, _vp]),
}

_lib = None
_lock = threading.Lock()


class RgkError(RuntimeError):
  """A librgk call returned a negative status."""

  def __init__(self, code: int, message: str):
    super().__init__(f"librgk error {code}: {message}")
    self.code = code


def load() -> ctypes.CDLL:
  """Loads librgk.so and declares every entry point; raises if the library is missing."""
  global _lib
  with _lock:
    if _lib is not None:
      return _lib
    if not os.path.exists(LIB_PATH):
      raise RuntimeError(
          f"{LIB_PATH} is missing: build it with `python -m recurrentgemma_b200.build` "
          "(needs nvcc; there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
      fn = getattr(lib, name)
      fn.restype = res
      fn.argtypes = args
    if lib.rgk_abi_version() != 8:
      raise RuntimeError("librgk.so has a different ABI version; rebuild it")
    _lib = lib
    return lib


def check(rc: int) -> None:
  if rc != 0:
    raise RgkError(rc, load().rgk_last_error().decode(errors="replace"))


def dtype_code(dt: torch.dtype) -> int:
  if dt == torch.float32:
    return RGK_F32
  if dt == torch.bfloat16:
    return RGK_BF16
  raise TypeError(f"recurrentgemma_b200 kernels take float32 or bfloat16, got {dt}")


def pos_code(pos: torch.Tensor) -> int:
  if pos.dtype == torch.int64:
    return RGK_I64
  if pos.dtype == torch.int32:
    return RGK_I32
  raise TypeError(f"segment_pos must be int32 or int64, got {pos.dtype}")


def require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
  dev = None
  for t in tensors:
    if t is None:
      continue
    if not t.is_cuda:
      raise RuntimeError(
          "recurrentgemma_b200 has no CPU path: tensors must live on a CUDA (sm_100) device")
    if dev is None:
      dev = t.device
    elif t.device != dev:
      raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
  if dev is None:
    raise RuntimeError("no tensor given")
  return dev


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
  return None if t is None else t.data_ptr()


def stream_ptr(dev: torch.device) -> int:
  return torch.cuda.current_stream(dev).cuda_stream


# One growing scratch buffer per (device, stream): calls on one stream are ordered, so they can
# share it; different streams get different buffers.
_workspaces = {}


def workspace(dev: torch.device, nbytes: int) -> torch.Tensor:
  key = (dev.index if dev.index is not None else torch.cuda.current_device(),
         torch.cuda.current_stream(dev).cuda_stream)
  buf = _workspaces.get(key)
  if buf is None or buf.numel() < nbytes:
    with torch.cuda.device(dev):
      new = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
      # the status word (first int): kernels only ever raise it, nobody but its reader clears it
      if buf is None:
        new[:4].zero_()
      else:
        new[:4].copy_(buf[:4])
    _workspaces[key] = buf = new
  return buf


def workspace_bytes(b: int, t: int, e: int, dt: torch.dtype) -> int:
  return int(load().rgk_workspace_bytes(b, t, e, dtype_code(dt)))


def workspace_status(ws: torch.Tensor, stream: Optional[int] = None) -> None:
  """Raises RgkError(RGK_ETIMEOUT) if a bounded device wait expired in any call on `ws` since the
  word was last read as raised (synchronises the stream; a raised word is cleared as it is reported)."""
  check(load().rgk_workspace_status(ws.data_ptr(),
                                    stream_ptr(ws.device) if stream is None else stream))


def status_ptr(dev: torch.device) -> int:
  """Device address of the status word of the current stream's workspace: what entry points with an
  `int* status` argument are given, so that their timeouts show up in `check_status` too."""
  return workspace(dev, 4).data_ptr()


def check_status(device: Optional[torch.device] = None) -> None:
  """Raises RgkError(RGK_ETIMEOUT) if any kernel launched through this package on `device` (every
  stream that has a workspace) gave up on a bounded wait since the last check.  The kernels finish
  on their own after such an expiry, but what they computed is invalid, and nothing else reports
  it: call this wherever the host synchronises anyway (it synchronises those streams)."""
  index = None
  if device is not None:
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
  for (dev_index, stream), buf in list(_workspaces.items()):
    if index is None or dev_index == index:
      with torch.cuda.device(dev_index):
        workspace_status(buf, stream)
