"""Drop-in counterparts of recurrentgemma.torch.layers for the RG-LRU + Conv1D path.

Same constructor arguments, parameter names and shapes (so reference state_dicts load unchanged),
same forward signatures and cache layout as

  * ``BlockDiagonalLinear``  recurrentgemma/torch/layers.py:76-137
  * ``rnn_scan``             recurrentgemma/torch/layers.py:140-191
  * ``RGLRU``                recurrentgemma/torch/layers.py:233-376
  * ``Conv1D``               recurrentgemma/torch/layers.py:379-650

but every forward runs hand-written sm_100a CUDA through the C ABI of librgk.so.  These are
inference modules: forwards do not record autograd graphs, and there is no CPU implementation
(tensors that are not on a CUDA device raise).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch
from torch import nn

from recurrentgemma_b200 import _lib


def _same_dtype(x: torch.Tensor, *params: torch.Tensor) -> None:
  for p in params:
    if p.dtype != x.dtype:
      raise TypeError(
          f"activations are {x.dtype} but a parameter is {p.dtype}; cast the module with .to()")


def _pos(segment_pos: torch.Tensor, bs: int, l: int) -> torch.Tensor:
  assert segment_pos.shape == (bs, l), (segment_pos.shape, (bs, l))
  if segment_pos.dtype not in (torch.int32, torch.int64):
    segment_pos = segment_pos.to(torch.int64)
  return segment_pos.contiguous()


def rnn_param_init(
    tensor: torch.Tensor, min_rad: float, max_rad: float, transform: str = "softplus",
    eps: float = 1e-8,
) -> torch.Tensor:
  """Ring-uniform init of the RG-LRU's `a_param` (recurrentgemma/torch/layers.py:194-213):
  softplus^-1(-0.5 ln u) with u uniform over [min_rad^2, max_rad^2) + eps.  The draw and every step
  after it happen in place in the tensor's own dtype, as in the reference, so that one seed gives
  the reference's values bit for bit (also in bfloat16, where each step rounds)."""
  if transform != "softplus":
    raise NotImplementedError(transform)
  with torch.no_grad():
    tensor.uniform_(min_rad ** 2 + eps, max_rad ** 2 + eps)      # u
    tensor.log_().mul_(-0.5)                                      # a_real = -0.5 ln u
    tensor.exp_().sub_(1.0).log_()                                # ln(e^a_real - 1)
  return tensor


class RMSNorm(nn.Module):
  """RMS norm over the last dimension (recurrentgemma/torch/layers.py:27-73): same constructor,
  parameter name (`scale`, zero-initialised) and forward."""

  def __init__(self, width: int, eps: float = 1e-6, device=None, dtype=None):
    super().__init__()
    self.width = width
    self.eps = eps
    self.scale = nn.Parameter(torch.empty([self.width], device=device, dtype=dtype))
    self.reset_parameters()

  def reset_parameters(self) -> None:
    torch.nn.init.zeros_(self.scale)

  @torch.no_grad()
  def forward(self, x: torch.Tensor) -> torch.Tensor:
    dev = _lib.require_cuda(x, self.scale)
    _same_dtype(x, self.scale)
    assert x.shape[-1] == self.width
    xc = x.contiguous()
    out = torch.empty_like(xc)
    m = xc.numel() // self.width
    with torch.cuda.device(dev):
      _lib.check(_lib.load().rgk_rmsnorm(
          xc.data_ptr(), self.scale.data_ptr(), m, self.width, float(self.eps),
          _lib.dtype_code(x.dtype), out.data_ptr(), _lib.stream_ptr(dev)))
    return out

  @torch.no_grad()
  def add_norm(self, a: torch.Tensor, b: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(a + b, forward(a + b)) in one kernel: the residual add in front of a block's second norm
    (recurrentgemma/torch/modules.py:902-904)."""
    dev = _lib.require_cuda(a, b, self.scale)
    _same_dtype(a, b, self.scale)
    assert a.shape == b.shape and a.shape[-1] == self.width
    ac, bc = a.contiguous(), b.contiguous()
    total, out = torch.empty_like(ac), torch.empty_like(ac)
    with torch.cuda.device(dev):
      _lib.check(_lib.load().rgk_add_rmsnorm(
          ac.data_ptr(), bc.data_ptr(), self.scale.data_ptr(), ac.numel() // self.width, self.width,
          float(self.eps), _lib.dtype_code(a.dtype), total.data_ptr(), out.data_ptr(),
          _lib.stream_ptr(dev)))
    return total, out


class Einsum(nn.Module):
  """Einsum with a bias (recurrentgemma/torch/layers.py:653-703): same constructor and parameter
  names (`w`, `b`).  Called on its own it is a library contraction; inside `modules.MLPBlock` its
  parameters feed the packed tensor-core GEMM."""

  def __init__(self, w_shape, b_shape, eqn: str, w_init_variance_scale: float = 1.0, device=None,
               dtype=None):
    super().__init__()
    self.w_shape = tuple(w_shape)
    self.b_shape = tuple(b_shape)
    self.eqn = eqn
    self.w_init_variance_scale = w_init_variance_scale
    self.w = nn.Parameter(torch.empty(self.w_shape, device=device, dtype=dtype))
    self.b = nn.Parameter(torch.empty(self.b_shape, device=device, dtype=dtype))
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.w_init_(self.w)
    torch.nn.init.zeros_(self.b)

  def w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0, std=math.sqrt(self.w_init_variance_scale / self.w_shape[1]))

  @torch.no_grad()
  def forward(self, x: torch.Tensor) -> torch.Tensor:
    _lib.require_cuda(x, self.w)
    _same_dtype(x, self.w, self.b)
    return torch.einsum(self.eqn, x, self.w) + self.b


class BlockDiagonalLinear(nn.Module):
  """Block-diagonal linear layer: y[..., h, :] = x[..., h, :] @ w[h] + b[h]."""

  def __init__(self, width: int, num_blocks: int, w_init_variance_scale: float = 1.0,
               device=None, dtype=None):
    super().__init__()
    self.width = width
    self.num_blocks = num_blocks
    self.w_init_variance_scale = w_init_variance_scale
    self.block_width = self.width // self.num_blocks
    self.w = nn.Parameter(torch.empty(
        [self.num_blocks, self.block_width, self.block_width], device=device, dtype=dtype))
    self.b = nn.Parameter(torch.empty([self.num_blocks, self.block_width], device=device,
                                      dtype=dtype))
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.w_init_(self.w)
    torch.nn.init.zeros_(self.b)

  def w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0, std=math.sqrt(self.w_init_variance_scale /
                                                      self.block_width))

  @torch.no_grad()
  def forward(self, x: torch.Tensor) -> torch.Tensor:
    dev = _lib.require_cuda(x, self.w)
    _same_dtype(x, self.w, self.b)
    assert x.shape[-1] == self.width
    xc = x.contiguous()
    out = torch.empty_like(xc)
    m = xc.numel() // self.width
    with torch.cuda.device(dev):
      _lib.check(_lib.load().rgk_blockdiag_linear(
          xc.data_ptr(), self.w.data_ptr(), self.b.data_ptr(), m, self.num_blocks,
          self.block_width, _lib.dtype_code(x.dtype), out.data_ptr(), _lib.stream_ptr(dev)))
    return out


@torch.no_grad()
def rnn_scan(
    x: torch.Tensor, a: torch.Tensor, reset: torch.Tensor, h0: Optional[torch.Tensor],
    acc_dtype: torch.dtype = torch.float32, y_mul: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
  """h_t = (a_t * ~reset_t) * h_{t-1} + x_t; returns (y in x.dtype, last state float32).

  `y_mul`, not part of the reference signature, fuses the recurrent block's join
  y * gelu_tanh(y_mul) into the same pass.
  """
  assert x.ndim == 3
  assert a.shape == x.shape
  assert a.dtype == x.dtype
  assert acc_dtype == torch.float32, "the recurrence accumulates in float32"
  assert h0 is None or h0.dtype == acc_dtype
  dev = _lib.require_cuda(x, a, reset, h0, y_mul)
  bs, l, e = x.shape
  assert reset.shape == (bs, l)
  xc, ac = x.contiguous(), a.contiguous()
  rc = reset.to(torch.uint8).contiguous()
  hc = None if h0 is None else h0.contiguous()
  mc = None if y_mul is None else y_mul.contiguous()
  y = torch.empty_like(xc)
  h_last = torch.empty((bs, e), dtype=torch.float32, device=dev)
  with torch.cuda.device(dev):
    nbytes = _lib.workspace_bytes(bs, l, e, x.dtype)
    ws = _lib.workspace(dev, nbytes)
    _lib.check(_lib.load().rgk_linear_scan(
        xc.data_ptr(), ac.data_ptr(), rc.data_ptr(), _lib.ptr(hc), _lib.ptr(mc), bs, l, e,
        _lib.dtype_code(x.dtype), y.data_ptr(), h_last.data_ptr(), ws.data_ptr(), ws.numel(),
        _lib.stream_ptr(dev)))
  return y, h_last


class RGLRU(nn.Module):
  """A Real-Gated Linear Recurrent Unit (RG-LRU) layer."""

  def __init__(self, width: int, num_heads: int, w_init_variance_scale: float = 1.0,
               device=None, dtype=None):
    super().__init__()
    self.width = width
    self.num_heads = num_heads
    self.w_init_variance_scale = w_init_variance_scale
    self.a_param = nn.Parameter(torch.empty([self.width], device=device, dtype=dtype))
    self.input_gate = BlockDiagonalLinear(width=self.width, num_blocks=self.num_heads,
                                          w_init_variance_scale=w_init_variance_scale,
                                          device=device, dtype=dtype)
    self.a_gate = BlockDiagonalLinear(width=self.width, num_blocks=self.num_heads,
                                      w_init_variance_scale=self.w_init_variance_scale,
                                      device=device, dtype=dtype)
    self.gates_impl = _lib.GATES_AUTO
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.input_gate.reset_parameters()
    self.a_gate.reset_parameters()
    self.a_param_init(self.a_param)

  def a_param_init(self, w: torch.Tensor) -> torch.Tensor:
    return rnn_param_init(w, min_rad=0.9, max_rad=0.999)

  def invalidate_packed(self) -> None:
    """Drops the packed copy of the gate weights; the next forward rebuilds it.  Needed after a
    write that torch does not count (`param.data.copy_(...)`, a raw pointer write): the copy is
    otherwise refreshed when a weight tensor is replaced, modified in place through autograd-visible
    operations, loaded from a state_dict or moved / cast with `.to()` / `.cuda()`."""
    self._pack_key = None

  def _load_from_state_dict(self, *args, **kwargs):
    self.invalidate_packed()
    return super()._load_from_state_dict(*args, **kwargs)

  def _apply(self, fn, *args, **kwargs):
    self.invalidate_packed()
    return super()._apply(fn, *args, **kwargs)

  def _packed_gates(self) -> Optional[int]:
    """Device pointer of the K-major copy of the gate weights the tcgen05 kernels read (bfloat16,
    or the hi / lo halves of the float32 weights for the 3xTF32 kernel), rebuilt
    whenever either weight tensor is replaced or modified in place (a derived, non-persistent
    buffer: it never enters the state_dict).  Writes through `.data` bypass the version counter:
    call `invalidate_packed()` after them."""
    wx, wa = self.input_gate.w, self.a_gate.w
    if (not wx.is_cuda or wx.dtype not in (torch.bfloat16, torch.float32) or wa.dtype != wx.dtype
        or self.width // self.num_heads != 256 or self.gates_impl == _lib.GATES_SIMT):
      return None
    dt = _lib.dtype_code(wx.dtype)
    key = (wx.data_ptr(), wx._version, wa.data_ptr(), wa._version, dt)
    if getattr(self, "_pack_key", None) != key:
      lib = _lib.load()
      buf = torch.empty(lib.rgk_gate_pack_bytes_for(self.num_heads, dt), dtype=torch.uint8,
                        device=wx.device)
      p = _lib.RgkParams(a_param=self.a_param.data_ptr(), gate_x_w=wx.data_ptr(),
                         gate_x_b=self.input_gate.b.data_ptr(), gate_a_w=wa.data_ptr(),
                         gate_a_b=self.a_gate.b.data_ptr())
      with torch.cuda.device(wx.device):
        _lib.check(lib.rgk_pack_gate_weights(ctypes.byref(p), self.num_heads, 256, dt,
                                             buf.data_ptr(), _lib.stream_ptr(wx.device)))
      self._pack_buf, self._pack_key = buf, key
    return self._pack_buf.data_ptr()

  def _params(self, conv: Optional["Conv1D"] = None) -> _lib.RgkParams:
    return _lib.RgkParams(
        gates_packed=self._packed_gates(),
        conv_w=None if conv is None else conv.w.data_ptr(),
        conv_b=None if conv is None else conv.b.data_ptr(),
        a_param=self.a_param.data_ptr(),
        gate_x_w=self.input_gate.w.data_ptr(), gate_x_b=self.input_gate.b.data_ptr(),
        gate_a_w=self.a_gate.w.data_ptr(), gate_a_b=self.a_gate.b.data_ptr())

  @torch.no_grad()
  def forward(
      self, x: torch.Tensor, segment_pos: torch.Tensor, cache: Optional[torch.Tensor] = None,
      return_cache: bool = True,
  ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns (y [B,T,E] in x.dtype, last hidden state [B,E] float32 or None)."""
    bs, l, e = x.shape
    assert e == self.width
    dev = _lib.require_cuda(x, segment_pos, cache, self.a_param)
    _same_dtype(x, self.a_param, self.input_gate.w, self.input_gate.b, self.a_gate.w,
                self.a_gate.b)
    pos = _pos(segment_pos, bs, l)
    assert cache is None or (cache.dtype == torch.float32 and cache.shape == (bs, e))
    xc = x.contiguous()
    hc = None if cache is None else cache.contiguous()
    y = torch.empty_like(xc)
    h_last = torch.empty((bs, e), dtype=torch.float32, device=dev) if return_cache else None
    p = self._params()
    with torch.cuda.device(dev):
      nbytes = _lib.workspace_bytes(bs, l, e, x.dtype)
      ws = _lib.workspace(dev, nbytes)
      _lib.check(_lib.load().rgk_rglru_forward(
          xc.data_ptr(), pos.data_ptr(), _lib.pos_code(pos), ctypes.byref(p), _lib.ptr(hc), bs, l,
          e, self.num_heads, _lib.dtype_code(x.dtype), self.gates_impl, y.data_ptr(),
          _lib.ptr(h_last), ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
    return y, h_last

  @classmethod
  def init_cache(cls, batch_size: int, width: int, device=None) -> torch.Tensor:
    """Empty RG-LRU state; always float32 (recurrentgemma/torch/layers.py:367-376)."""
    return torch.zeros((batch_size, width), dtype=torch.float32, device=device)


class Conv1D(nn.Module):
  """Causal depthwise temporal convolution with document masking and a decode cache."""

  def __init__(self, width: int, temporal_width: int, w_init_variance_scale: float = 0.01,
               device=None, dtype=None):
    super().__init__()
    self.width = width
    self.temporal_width = temporal_width
    self.w_init_variance_scale = w_init_variance_scale
    self.w = nn.Parameter(torch.empty([self.temporal_width, self.width], device=device,
                                      dtype=dtype))
    self.b = nn.Parameter(torch.empty([width], device=device, dtype=dtype))
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.w_init_(self.w)
    torch.nn.init.zeros_(self.b)

  def w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0, std=math.sqrt(self.w_init_variance_scale /
                                                      self.temporal_width))

  @torch.no_grad()
  def forward(
      self, x: torch.Tensor, segment_pos: torch.Tensor, cache: Optional[torch.Tensor] = None,
      return_cache: bool = True,
  ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns (output [B,T,E], new cache [B,temporal_width-1,E] or None).

    Unlike the reference (recurrentgemma/torch/layers.py:497-508) the input is not modified; the
    returned cache holds the same masked rows the reference's in-place masking leaves behind.
    """
    bs, l, e = x.shape
    assert e == self.width
    dev = _lib.require_cuda(x, segment_pos, cache, self.w)
    _same_dtype(x, self.w, self.b)
    if self.temporal_width != 4:
      raise NotImplementedError("the CUDA Conv1D covers temporal_width == 4 only")
    lib = _lib.load()
    dt = _lib.dtype_code(x.dtype)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    with torch.cuda.device(dev):
      if cache is None:
        pos = _pos(segment_pos, bs, l)
        new_cache = (torch.empty((bs, self.temporal_width - 1, e), dtype=x.dtype, device=dev)
                     if return_cache else None)
        _lib.check(lib.rgk_conv1d_prefill(
            xc.data_ptr(), pos.data_ptr(), _lib.pos_code(pos), self.w.data_ptr(),
            self.b.data_ptr(), bs, l, e, self.temporal_width, dt, out.data_ptr(),
            _lib.ptr(new_cache), _lib.stream_ptr(dev)))
        return out, new_cache
      assert cache.shape == (bs, self.temporal_width - 1, e)
      assert l == 1, "decoding takes one token at a time"
      cache_x = cache.to(x.dtype).contiguous()
      new_cache = torch.empty_like(cache_x) if return_cache else None
      _lib.check(lib.rgk_conv1d_decode(
          xc.data_ptr(), cache_x.data_ptr(), self.w.data_ptr(), self.b.data_ptr(), bs, e,
          self.temporal_width, dt, out.data_ptr(), _lib.ptr(new_cache), _lib.stream_ptr(dev)))
      if new_cache is not None and new_cache.dtype != cache.dtype:
        new_cache = new_cache.to(cache.dtype)
      return out, new_cache

  @classmethod
  def init_cache(cls, *, batch_size: int, width: int, dtype: torch.dtype,
                 conv1d_temporal_width: int = 4, device=None) -> torch.Tensor:
    """Empty Conv1D cache (recurrentgemma/torch/layers.py:638-650)."""
    return torch.zeros((batch_size, conv1d_temporal_width - 1, width), dtype=dtype, device=device)
