"""Drop-in counterpart of recurrentgemma.torch.modules.RecurrentBlock (modules.py:496-680).

Same constructor, parameter names (`linear_y`, `linear_x`, `linear_out`, `conv_1d`, `rg_lru`),
forward signature and cache type as the reference, so it slots into the reference `Griffin` model
and `Sampler` unchanged.  The RG-LRU + Conv1D sub-path between the projections runs as one
composed call into librgk.so; the three dense projections are plain library GEMMs.
"""
from __future__ import annotations

import ctypes
import math
from typing import NamedTuple, Optional, Tuple

import torch
from torch import nn

from recurrentgemma_b200 import _lib
from recurrentgemma_b200 import layers


class RecurrentBlockCache(NamedTuple):
  """Field order and dtypes of recurrentgemma/torch/modules.py:32-37."""
  rg_lru_state: torch.Tensor   # [B, lru_width] float32
  conv1d_state: torch.Tensor   # [B, conv1d_temporal_width - 1, lru_width] activation dtype


def recurrent_path(
    xb: torch.Tensor, yb: Optional[torch.Tensor], segment_pos: torch.Tensor,
    conv_1d: layers.Conv1D, rg_lru: layers.RGLRU,
    cache: Optional[RecurrentBlockCache] = None, return_cache: bool = True,
    out: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
  """RGLRU(Conv1D(xb)) * gelu_tanh(yb): the sub-path of RecurrentBlock.forward between the
  input projections and `linear_out` (recurrentgemma/torch/modules.py:631-646)."""
  bs, l, e = xb.shape
  dev = _lib.require_cuda(xb, yb, segment_pos, conv_1d.w, rg_lru.a_param)
  layers._same_dtype(xb, conv_1d.w, conv_1d.b, rg_lru.a_param, rg_lru.input_gate.w,
                     rg_lru.input_gate.b, rg_lru.a_gate.w, rg_lru.a_gate.b)
  if yb is not None:
    assert yb.shape == xb.shape and yb.dtype == xb.dtype
  if conv_1d.temporal_width != 4:
    raise NotImplementedError("the CUDA Conv1D covers temporal_width == 4 only")
  pos = layers._pos(segment_pos, bs, l)
  lib = _lib.load()
  dt = _lib.dtype_code(xb.dtype)
  xc = xb.contiguous()
  yc = None if yb is None else yb.contiguous()
  if out is None:
    out = torch.empty_like(xc)
  p = rg_lru._params(conv_1d)
  with torch.cuda.device(dev):
    ws = _lib.workspace(dev, _lib.workspace_bytes(bs, l, e, xb.dtype))
    if cache is None:
      h_last = torch.empty((bs, e), dtype=torch.float32, device=dev) if return_cache else None
      conv_state = torch.empty((bs, 3, e), dtype=xb.dtype, device=dev) if return_cache else None
      _lib.check(lib.rgk_recurrent_path_prefill(
          xc.data_ptr(), _lib.ptr(yc), pos.data_ptr(), _lib.pos_code(pos), ctypes.byref(p), None,
          bs, l, e, rg_lru.num_heads, 4, dt, rg_lru.gates_impl, out.data_ptr(), _lib.ptr(h_last),
          _lib.ptr(conv_state), ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
    else:
      # Conv1D decoding takes one token at a time (recurrentgemma/torch/layers.py:548-549).
      assert l == 1, "with a cache the recurrent block takes one token at a time"
      assert cache.rg_lru_state.dtype == torch.float32
      assert cache.rg_lru_state.shape == (bs, e) and cache.conv1d_state.shape == (bs, 3, e)
      h_in = cache.rg_lru_state.contiguous()
      conv_in = cache.conv1d_state.to(xb.dtype).contiguous()
      h_last = torch.empty_like(h_in)
      conv_state = torch.empty_like(conv_in)
      _lib.check(lib.rgk_recurrent_path_decode(
          xc.data_ptr(), _lib.ptr(yc), pos.data_ptr(), _lib.pos_code(pos), ctypes.byref(p),
          h_in.data_ptr(), conv_in.data_ptr(), bs, e, rg_lru.num_heads, 4, dt, rg_lru.gates_impl,
          out.data_ptr(), h_last.data_ptr(), conv_state.data_ptr(), ws.data_ptr(), ws.numel(),
          _lib.stream_ptr(dev)))
      if conv_state.dtype != cache.conv1d_state.dtype:
        conv_state = conv_state.to(cache.conv1d_state.dtype)
  if not return_cache:
    return out, None
  return out, RecurrentBlockCache(rg_lru_state=h_last, conv1d_state=conv_state)


@torch.no_grad()
def dense_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                 gelu: bool = False) -> torch.Tensor:
  """x @ weight.T + bias on the tcgen05 GEMM of librgk (bfloat16), optionally followed by
  gelu(approximate="tanh") on the rounded result: `nn.Linear` as the block uses it
  (recurrentgemma/torch/modules.py:531-548, 627-631, 647)."""
  dev = _lib.require_cuda(x, weight, bias)
  layers._same_dtype(x, weight, *([bias] if bias is not None else []))
  n, k = weight.shape
  assert x.shape[-1] == k
  xc, wc = x.contiguous(), weight.contiguous()
  bc = None if bias is None else bias.contiguous()
  out = torch.empty((*x.shape[:-1], n), dtype=x.dtype, device=dev)
  with torch.cuda.device(dev):
    _lib.check(_lib.load().rgk_dense_linear(
        xc.data_ptr(), wc.data_ptr(), _lib.ptr(bc), xc.numel() // k, k, n, _lib.dtype_code(x.dtype),
        1 if gelu else 0, out.data_ptr(), None, _lib.stream_ptr(dev)))
  return out


class RecurrentBlock(nn.Module):
  """Griffin and Hawk's recurrent block."""

  def __init__(self, width: int, num_heads: int, lru_width: Optional[int] = None,
               conv1d_temporal_width: int = 4, final_w_init_variance_scale: float = 1.0,
               device=None, dtype=None):
    super().__init__()
    self.width = width
    self.num_heads = num_heads
    self.lru_width = lru_width or width
    self.conv1d_temporal_width = conv1d_temporal_width
    self.final_w_init_variance_scale = final_w_init_variance_scale

    self.linear_y = nn.Linear(self.width, self.lru_width, device=device, dtype=dtype)
    self.linear_x = nn.Linear(self.width, self.lru_width, device=device, dtype=dtype)
    self.linear_out = nn.Linear(self.lru_width, self.width, device=device, dtype=dtype)
    self.conv_1d = layers.Conv1D(width=self.lru_width, temporal_width=self.conv1d_temporal_width,
                                 device=device, dtype=dtype)
    self.rg_lru = layers.RGLRU(width=self.lru_width, num_heads=self.num_heads, device=device,
                               dtype=dtype)
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.w_init_(self.linear_x.weight)
    torch.nn.init.zeros_(self.linear_x.bias)
    self.w_init_(self.linear_y.weight)
    torch.nn.init.zeros_(self.linear_y.bias)
    self.out_w_init_(self.linear_out.weight)
    torch.nn.init.zeros_(self.linear_out.bias)
    self.conv_1d.reset_parameters()
    self.rg_lru.reset_parameters()

  def w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0, std=math.sqrt(1.0 / self.width))

  def out_w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0,
                          std=math.sqrt(self.final_w_init_variance_scale / self.lru_width))

  @torch.no_grad()
  def forward(
      self, x: torch.Tensor, segment_pos: torch.Tensor,
      cache: Optional[RecurrentBlockCache] = None, return_cache: bool = True,
  ) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
    """Returns (block output [B,T,width], updated cache or None)."""
    dev = _lib.require_cuda(x, segment_pos, self.linear_x.weight)
    if self._fusable(x, cache):
      return self._forward_fused(x, segment_pos, return_cache, dev)
    yb = self.linear_y(x)
    xb = self.linear_x(x)
    z, new_cache = recurrent_path(xb, yb, segment_pos, self.conv_1d, self.rg_lru, cache,
                                  return_cache)
    return self.linear_out(z), new_cache

  def _forward_fused(self, x, segment_pos, return_cache, dev, norm=None):
    """Prefill of the whole block in one library call: the three projections on the tcgen05 GEMM
    (gelu of the y branch in its epilogue), the RG-LRU + Conv1D sub-path in between.  With `norm`
    (an RMSNorm) the call computes block(norm(x)) + x: the norm as its own kernel, the residual in
    the epilogue of linear_out."""
    bs, l, d = x.shape
    e = self.lru_width
    params = [self.linear_y.weight, self.linear_y.bias, self.linear_x.weight, self.linear_x.bias,
              self.linear_out.weight, self.linear_out.bias, self.conv_1d.w, self.conv_1d.b,
              self.rg_lru.a_param, self.rg_lru.input_gate.w, self.rg_lru.input_gate.b,
              self.rg_lru.a_gate.w, self.rg_lru.a_gate.b]
    if norm is not None:
      params.append(norm.scale)
    layers._same_dtype(x, *params)
    pos = layers._pos(segment_pos, bs, l)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    h_last = torch.empty((bs, e), dtype=torch.float32, device=dev) if return_cache else None
    conv_state = torch.empty((bs, 3, e), dtype=x.dtype, device=dev) if return_cache else None
    lib = _lib.load()
    p = _lib.RgkBlockParams(
        path=self.rg_lru._params(self.conv_1d),
        linear_y_w=self.linear_y.weight.data_ptr(), linear_y_b=self.linear_y.bias.data_ptr(),
        linear_x_w=self.linear_x.weight.data_ptr(), linear_x_b=self.linear_x.bias.data_ptr(),
        linear_out_w=self.linear_out.weight.data_ptr(),
        linear_out_b=self.linear_out.bias.data_ptr())
    with torch.cuda.device(dev):
      dt = _lib.dtype_code(x.dtype)
      if norm is None:
        ws = _lib.workspace(dev, int(lib.rgk_block_workspace_bytes(bs, l, d, e, dt)))
        _lib.check(lib.rgk_recurrent_block_prefill(
            xc.data_ptr(), pos.data_ptr(), _lib.pos_code(pos), ctypes.byref(p), bs, l, d, e,
            self.num_heads, 4, dt, out.data_ptr(), _lib.ptr(h_last), _lib.ptr(conv_state),
            ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
      else:
        ws = _lib.workspace(dev, int(lib.rgk_residual_workspace_bytes(bs, l, d, e, dt)))
        _lib.check(lib.rgk_residual_block_prefill(
            xc.data_ptr(), pos.data_ptr(), _lib.pos_code(pos), ctypes.byref(p),
            norm.scale.data_ptr(), float(norm.eps), bs, l, d, e, self.num_heads, 4, dt,
            out.data_ptr(), _lib.ptr(h_last), _lib.ptr(conv_state), ws.data_ptr(), ws.numel(),
            _lib.stream_ptr(dev)))
    if not return_cache:
      return out, None
    return out, RecurrentBlockCache(rg_lru_state=h_last, conv1d_state=conv_state)

  def _fusable(self, x: torch.Tensor, cache) -> bool:
    return (cache is None and x.dtype == torch.bfloat16
            and self.lru_width // self.num_heads == 256 and self.conv1d_temporal_width == 4
            and self.width % 8 == 0 and self.rg_lru.gates_impl != _lib.GATES_SIMT)

  @classmethod
  def init_cache(cls, batch_size: int, lru_width: int, dtype: torch.dtype,
                 conv1d_temporal_width: int = 4, device=None) -> RecurrentBlockCache:
    """Empty cache (recurrentgemma/torch/modules.py:657-680)."""
    return RecurrentBlockCache(
        rg_lru_state=layers.RGLRU.init_cache(batch_size=batch_size, width=lru_width,
                                             device=device),
        conv1d_state=layers.Conv1D.init_cache(batch_size=batch_size, width=lru_width, dtype=dtype,
                                              conv1d_temporal_width=conv1d_temporal_width,
                                              device=device),
    )


@torch.no_grad()
def recurrent_residual(
    x: torch.Tensor, segment_pos: torch.Tensor, temporal_pre_norm: layers.RMSNorm,
    recurrent_block: RecurrentBlock, cache: Optional[RecurrentBlockCache] = None,
    return_cache: bool = True,
) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
  """The temporal half of ResidualBlock.forward for a recurrent block
  (recurrentgemma/torch/modules.py:897-902): recurrent_block(temporal_pre_norm(x)) + x, with the
  updated cache.  bfloat16 prefill with head width 256 runs as one library call (RMSNorm kernel,
  the block's kernels, residual add in the epilogue of linear_out); other cases compose the
  modules."""
  dev = _lib.require_cuda(x, segment_pos, recurrent_block.linear_x.weight)
  if recurrent_block._fusable(x, cache) and temporal_pre_norm.width == recurrent_block.width:
    return recurrent_block._forward_fused(x, segment_pos, return_cache, dev, norm=temporal_pre_norm)
  y, new_cache = recurrent_block(temporal_pre_norm(x), segment_pos, cache, return_cache)
  return y + x, new_cache

class MLPBlock(nn.Module):
  """The gated MLP of a residual block (recurrentgemma/torch/modules.py:683-752): same constructor,
  parameter names (`ffw_up.w [2, width, expanded]`, `ffw_up.b [2, 1, 1, expanded]`,
  `ffw_down.weight/.bias`) and forward."""

  def __init__(self, width: int, expanded_width: int, final_w_init_variance_scale: float = 1.0,
               device=None, dtype=None):
    super().__init__()
    self.width = width
    self.expanded_width = expanded_width
    self.final_w_init_variance_scale = final_w_init_variance_scale
    self.ffw_up = layers.Einsum(w_shape=(2, self.width, self.expanded_width),
                                b_shape=(2, 1, 1, self.expanded_width), eqn="...td,cdD->c...tD",
                                device=device, dtype=dtype)
    self.ffw_down = nn.Linear(self.expanded_width, self.width, device=device, dtype=dtype)
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.ffw_up.reset_parameters()
    self.out_w_init_(self.ffw_down.weight)
    torch.nn.init.zeros_(self.ffw_down.bias)

  def out_w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0,
                          std=math.sqrt(self.final_w_init_variance_scale / self.expanded_width))

  def _fusable(self, x: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and self.width % 8 == 0 and self.expanded_width % 64 == 0)

  def _packed_up(self) -> int:
    """Device pointer of the K-major, gate/value-interleaved copy of ffw_up the GeGLU GEMM reads,
    rebuilt when either parameter is replaced or modified in place (derived, never in the
    state_dict)."""
    w, b = self.ffw_up.w, self.ffw_up.b
    key = (w.data_ptr(), w._version, b.data_ptr(), b._version)
    if getattr(self, "_pack_key", None) != key:
      lib = _lib.load()
      buf = torch.empty(int(lib.rgk_mlp_pack_bytes(self.width, self.expanded_width)),
                        dtype=torch.uint8, device=w.device)
      with torch.cuda.device(w.device):
        _lib.check(lib.rgk_pack_mlp_up(w.data_ptr(), b.data_ptr(), self.width, self.expanded_width,
                                       _lib.RGK_BF16, buf.data_ptr(), _lib.stream_ptr(w.device)))
      self._pack_buf, self._pack_key = buf, key
    return self._pack_buf.data_ptr()

  @torch.no_grad()
  def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None,
              pre_norm: Optional[layers.RMSNorm] = None) -> torch.Tensor:
    """ffw_down(gelu(up_0) * up_1).  The two optional arguments (not in the reference) select the
    channel half of a residual block as one call: with `pre_norm` the MLP reads pre_norm(x) and
    x is added to the result; with `residual` alone that tensor is added."""
    dev = _lib.require_cuda(x, self.ffw_up.w)
    params = [self.ffw_up.w, self.ffw_up.b, self.ffw_down.weight, self.ffw_down.bias]
    if pre_norm is not None:
      params.append(pre_norm.scale)
    layers._same_dtype(x, *params)
    assert x.shape[-1] == self.width
    if not self._fusable(x):
      xin = x if pre_norm is None else pre_norm(x)
      out = self.ffw_up(xin)
      y = self.ffw_down(torch.nn.functional.gelu(out[0], approximate="tanh") * out[1])
      if pre_norm is not None:
        return y + x
      return y if residual is None else y + residual
    xc = x.contiguous()
    m = xc.numel() // self.width
    out = torch.empty_like(xc)
    lib = _lib.load()
    dt = _lib.dtype_code(x.dtype)
    with torch.cuda.device(dev):
      ws = _lib.workspace(dev, int(lib.rgk_mlp_workspace_bytes(m, self.width, self.expanded_width, dt)))
      if pre_norm is not None:
        _lib.check(lib.rgk_residual_channel(
            xc.data_ptr(), pre_norm.scale.data_ptr(), float(pre_norm.eps), self._packed_up(),
            self.ffw_down.weight.data_ptr(), self.ffw_down.bias.data_ptr(), m, self.width,
            self.expanded_width, dt, out.data_ptr(), ws.data_ptr(), ws.numel(),
            _lib.stream_ptr(dev)))
      else:
        rc = None if residual is None else residual.contiguous()
        _lib.check(lib.rgk_mlp_block(
            xc.data_ptr(), self._packed_up(), self.ffw_down.weight.data_ptr(),
            self.ffw_down.bias.data_ptr(), _lib.ptr(rc), m, self.width, self.expanded_width, dt,
            out.data_ptr(), ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
    return out


@torch.no_grad()
def residual_block(
    x: torch.Tensor, segment_pos: torch.Tensor, temporal_pre_norm: layers.RMSNorm,
    recurrent_block: RecurrentBlock, channel_pre_norm: layers.RMSNorm, mlp_block: MLPBlock,
    cache: Optional[RecurrentBlockCache] = None, return_cache: bool = True,
) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
  """ResidualBlock.forward for a recurrent block (recurrentgemma/torch/modules.py:897-911):
  r = recurrent_block(temporal_pre_norm(x)) + x;  out = mlp_block(channel_pre_norm(r)) + r."""
  r, new_cache = recurrent_residual(x, segment_pos, temporal_pre_norm, recurrent_block, cache,
                                    return_cache)
  return mlp_block(r, pre_norm=channel_pre_norm), new_cache
