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


# Fewest rows for which the prefill GEMM of the library is used (see MLPBlock._fusable), and most
# rows for which the few-row (weight-streaming, split-K) kernel is used; torch's contractions in
# between.  The few-row kernel takes up to 256 rows, but the exchange of its K-split partial sums
# grows with the row count: measured on a B200 at 2560 x 2560 it is ahead of the library GEMM up
# to 32 rows (two projections in one launch: 9.7 against 12.6 us at 16 rows) and behind it from 64.
SMALL_M = 1024
SMALL_ROWS = 32
# The MLP's contractions (2560 -> 2 x 7680 -> 2560) stay on the library below SMALL_M: with 120
# feature tiles there is nothing to split, and the library's kernel streams those weights faster
# (15.5 against 21 us).  Raise to SMALL_ROWS to route them through the few-row kernel as well
# (GeGLU and the residual add then run in its epilogues).
SMALL_ROWS_MLP = 0


class RecurrentBlockCache(NamedTuple):
  """Field order and dtypes of recurrentgemma/torch/modules.py:32-37."""
  rg_lru_state: torch.Tensor   # [B, lru_width] float32
  conv1d_state: torch.Tensor   # [B, conv1d_temporal_width - 1, lru_width] activation dtype


def recurrent_path(
    xb: torch.Tensor, yb: Optional[torch.Tensor], segment_pos: torch.Tensor,
    conv_1d: layers.Conv1D, rg_lru: layers.RGLRU,
    cache: Optional[RecurrentBlockCache] = None, return_cache: bool = True,
    out: Optional[torch.Tensor] = None, inplace: bool = False,
) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
  """RGLRU(Conv1D(xb)) * gelu_tanh(yb): the sub-path of RecurrentBlock.forward between the
  input projections and `linear_out` (recurrentgemma/torch/modules.py:631-646).  With `inplace`
  a decode step overwrites the tensors of `cache` and returns that cache (an extension for
  decode loops that run as a CUDA graph; the reference always returns new tensors)."""
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
      if inplace:
        assert h_in is cache.rg_lru_state and conv_in is cache.conv1d_state, (
            "an in-place step needs a contiguous cache in the activation dtype")
        h_last, conv_state = h_in, conv_in
      else:
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
        1 if gelu else 0, out.data_ptr(), _lib.status_ptr(dev), _lib.stream_ptr(dev)))
  return out


@torch.no_grad()
def small_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                 act: int = _lib.ACT_NONE, residual: Optional[torch.Tensor] = None,
                 bias_ptr: Optional[int] = None) -> torch.Tensor:
  """The same projection for at most SMALL_ROWS rows (a decode step) on the weight-streaming
  split-K tcgen05 kernel of librgk.  act: _lib.ACT_NONE, ACT_GELU_TANH (gelu of the rounded result)
  or ACT_GEGLU (weight = the packed up-projection of the MLP block with its bias at `bias_ptr`;
  the result has half as many features as the weight has rows).  `residual` is added to the rounded
  result (its own rounding)."""
  dev = _lib.require_cuda(x, weight, bias, residual)
  n, k = weight.shape
  assert x.shape[-1] == k
  xc = x.contiguous()
  m = xc.numel() // k
  n_out = n // 2 if act == _lib.ACT_GEGLU else n
  out = torch.empty((*x.shape[:-1], n_out), dtype=x.dtype, device=dev)
  rc = None if residual is None else residual.contiguous()
  bc = None if bias is None else bias.contiguous()
  lib = _lib.load()
  with torch.cuda.device(dev):
    _lib.check(lib.rgk_dense_linear_small(
        xc.data_ptr(), weight.data_ptr(), bias_ptr if bias_ptr is not None else _lib.ptr(bc),
        _lib.ptr(rc), m, k, n, _lib.dtype_code(x.dtype), act, out.data_ptr(),
        _lib.status_ptr(dev), _lib.stream_ptr(dev)))
  return out


@torch.no_grad()
def small_linear_pair(x: torch.Tensor, lin_a: nn.Linear, lin_b: nn.Linear
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
  """(lin_a(x), lin_b(x)) for at most SMALL_ROWS rows in ONE launch of the few-row kernel (the two
  projections share the rows of x); lin_a.out_features a multiple of 128."""
  dev = _lib.require_cuda(x, lin_a.weight, lin_b.weight)
  layers._same_dtype(x, lin_a.weight, lin_b.weight,
                     *[l.bias for l in (lin_a, lin_b) if l.bias is not None])
  (na, k), (nb, kb) = lin_a.weight.shape, lin_b.weight.shape
  assert x.shape[-1] == k == kb
  xc = x.contiguous()
  m = xc.numel() // k
  out_a = torch.empty((*x.shape[:-1], na), dtype=x.dtype, device=dev)
  out_b = torch.empty((*x.shape[:-1], nb), dtype=x.dtype, device=dev)
  lib = _lib.load()
  with torch.cuda.device(dev):
    _lib.check(lib.rgk_dense_linear_small_pair(
        xc.data_ptr(), lin_a.weight.data_ptr(), _lib.ptr(lin_a.bias), lin_b.weight.data_ptr(),
        _lib.ptr(lin_b.bias), m, k, na, nb, _lib.dtype_code(x.dtype), out_a.data_ptr(),
        out_b.data_ptr(), _lib.status_ptr(dev), _lib.stream_ptr(dev)))
  return out_a, out_b


def linear_pair(x: torch.Tensor, lin_a: nn.Linear, lin_b: nn.Linear
                ) -> Tuple[torch.Tensor, torch.Tensor]:
  """(lin_a(x), lin_b(x)): one launch of the few-row kernel where it applies, else two `linear`."""
  rows = x.numel() // x.shape[-1]
  if (rows < SMALL_M and _small_ok(x, lin_a.weight) and _small_ok(x, lin_b.weight)
      and lin_a.weight.shape[0] % 128 == 0
      and all(l.bias is None or l.bias.is_contiguous() for l in (lin_a, lin_b))):
    return small_linear_pair(x, lin_a, lin_b)
  return linear(x, lin_a), linear(x, lin_b)


def _small_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
  n, k = weight.shape
  return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()
          and 1 <= x.numel() // x.shape[-1] <= SMALL_ROWS and k % 8 == 0 and n % 8 == 0)


def linear(x: torch.Tensor, lin: nn.Linear, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
  """lin(x) (+ residual): the prefill GEMM from SMALL_M rows on, the few-row kernel up to
  SMALL_ROWS rows, torch in between and for float32."""
  rows = x.numel() // x.shape[-1]
  if x.dtype == torch.bfloat16 and rows >= SMALL_M:
    y = dense_linear(x, lin.weight, lin.bias)
  elif _small_ok(x, lin.weight):
    layers._same_dtype(x, lin.weight, *([lin.bias] if lin.bias is not None else []))
    return small_linear(x, lin.weight, lin.bias, residual=residual)
  else:
    y = lin(x)
  return y if residual is None else y + residual


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
      inplace: bool = False,
  ) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
    """Returns (block output [B,T,width], updated cache or None).  `inplace`: see
    `recurrent_path`."""
    dev = _lib.require_cuda(x, segment_pos, self.linear_x.weight)
    if self._fusable(x, cache):
      return self._forward_fused(x, segment_pos, return_cache, dev)
    yb, xb = linear_pair(x, self.linear_y, self.linear_x)
    z, new_cache = recurrent_path(xb, yb, segment_pos, self.conv_1d, self.rg_lru, cache,
                                  return_cache, inplace=inplace)
    return linear(z, self.linear_out), new_cache

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
    return_cache: bool = True, inplace: bool = False,
) -> Tuple[torch.Tensor, Optional[RecurrentBlockCache]]:
  """The temporal half of ResidualBlock.forward for a recurrent block
  (recurrentgemma/torch/modules.py:897-902): recurrent_block(temporal_pre_norm(x)) + x, with the
  updated cache.  bfloat16 prefill with head width 256 runs as one library call (RMSNorm kernel,
  the block's kernels, residual add in the epilogue of linear_out); other cases compose the
  modules."""
  dev = _lib.require_cuda(x, segment_pos, recurrent_block.linear_x.weight)
  if recurrent_block._fusable(x, cache) and temporal_pre_norm.width == recurrent_block.width:
    return recurrent_block._forward_fused(x, segment_pos, return_cache, dev, norm=temporal_pre_norm)
  y, new_cache = recurrent_block(temporal_pre_norm(x), segment_pos, cache, return_cache,
                                 inplace=inplace)
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
    # below SMALL_M rows the 128 x 256 tiles of the GEMM leave most SMs without a tile (a decode
    # step has M = batch): library contractions, which split K, are used there
    return (x.dtype == torch.bfloat16 and self.width % 8 == 0 and self.expanded_width % 64 == 0
            and x.numel() // x.shape[-1] >= SMALL_M)

  def invalidate_packed(self) -> None:
    """Drops the packed copy of ffw_up; the next forward rebuilds it.  Needed after a write that
    torch does not count (`param.data.copy_(...)`); state_dict loads, `.to()` and counted in-place
    writes refresh it by themselves."""
    self._pack_key = None

  def _load_from_state_dict(self, *args, **kwargs):
    self.invalidate_packed()
    return super()._load_from_state_dict(*args, **kwargs)

  def _apply(self, fn, *args, **kwargs):
    self.invalidate_packed()
    return super()._apply(fn, *args, **kwargs)

  def _packed_up(self) -> int:
    """Device pointer of the K-major, gate/value-interleaved copy of ffw_up the GeGLU GEMM reads,
    rebuilt when either parameter is replaced or modified in place (derived, never in the
    state_dict).  Writes through `.data` bypass the version counter: call `invalidate_packed()`."""
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
    rows = x.numel() // x.shape[-1]
    if (x.dtype == torch.bfloat16 and rows <= SMALL_ROWS_MLP and rows < SMALL_M and self.width % 8 == 0
        and self.expanded_width % 64 == 0 and self.ffw_down.weight.is_contiguous()):
      # a decode step: both contractions on the few-row kernel, GeGLU and the residual add in
      # their epilogues
      xin = x if pre_norm is None else pre_norm(x)
      packed = self._packed_up()
      w_bytes = -(-2 * self.expanded_width * self.width * 2 // 256) * 256
      w_view = self._pack_buf[:2 * self.expanded_width * self.width * 2].view(torch.bfloat16).view(
          2 * self.expanded_width, self.width)
      hidden = small_linear(xin, w_view, None, act=_lib.ACT_GEGLU, bias_ptr=packed + w_bytes)
      res = x if pre_norm is not None else residual
      return small_linear(hidden, self.ffw_down.weight, self.ffw_down.bias, residual=res)
    if not self._fusable(x):
      xin = x if pre_norm is None else pre_norm(x)
      # ffw_up as two plain contractions (the einsum of layers.Einsum would first make a permuted
      # copy of the weights): the contraction and the bias add are two tensor operations
      w, bias = self.ffw_up.w, self.ffw_up.b.reshape(2, -1)
      xw = self.expanded_width
      up = torch.matmul(xin.reshape(1, -1, self.width), w)          # [2, M, X], one batched call
      if (xw * x.element_size()) % 16 == 0:
        hidden = torch.empty((*x.shape[:-1], xw), dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
          _lib.check(_lib.load().rgk_geglu_bias(
              up.data_ptr(), bias.contiguous().data_ptr(), up.shape[1], xw,
              _lib.dtype_code(x.dtype), hidden.data_ptr(), _lib.stream_ptr(dev)))
      else:
        gate, value = up[0] + bias[0], up[1] + bias[1]
        hidden = (torch.nn.functional.gelu(gate, approximate="tanh") * value).reshape(*x.shape[:-1], xw)
      y = self.ffw_down(hidden)
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
    temporal_block: nn.Module, channel_pre_norm: layers.RMSNorm, mlp_block: MLPBlock,
    cache=None, return_cache: bool = True, inplace: bool = False,
):
  """ResidualBlock.forward (recurrentgemma/torch/modules.py:897-911) for either kind of temporal
  block (a `RecurrentBlock` or a `LocalAttentionBlock`):
  r = temporal_block(temporal_pre_norm(x)) + x;  out = mlp_block(channel_pre_norm(r)) + r.
  Returns (out, updated cache of the temporal block or None).  `inplace`: a decode step overwrites
  the tensors of `cache` instead of returning new ones."""
  if (isinstance(temporal_block, RecurrentBlock) and temporal_block._fusable(x, cache)
      and temporal_pre_norm.width == temporal_block.width):
    # bfloat16 prefill of the recurrent kind: each half is one library call
    r, new_cache = recurrent_residual(x, segment_pos, temporal_pre_norm, temporal_block, cache,
                                      return_cache, inplace)
    return mlp_block(r, pre_norm=channel_pre_norm), new_cache
  y, new_cache = temporal_block(temporal_pre_norm(x), segment_pos, cache, return_cache,
                                inplace=inplace)
  r, normed = channel_pre_norm.add_norm(y, x)        # the residual add rides in the norm kernel
  return mlp_block(normed, residual=r), new_cache


class AttentionBlockCache(NamedTuple):
  """Field order and dtypes of recurrentgemma/torch/modules.py:40-46: a ring buffer of the last
  `window` keys and values and the number of tokens seen."""
  keys: torch.Tensor        # [B, window, 1, head_dim]
  values: torch.Tensor      # [B, window, 1, head_dim]
  num_tokens: torch.Tensor  # [B] int32


def _rope(x: torch.Tensor, segment_pos: torch.Tensor) -> torch.Tensor:
  """Rotary embedding of x [B, T, heads, head_dim] in place (torch/modules.py:58-86)."""
  b, t, heads, hd = x.shape
  pos = segment_pos.contiguous()
  dev = x.device
  with torch.cuda.device(dev):
    _lib.check(_lib.load().rgk_rope(x.data_ptr(), pos.data_ptr(), _lib.pos_code(pos), b * t, heads,
                                    hd, _lib.dtype_code(x.dtype), _lib.stream_ptr(dev)))
  return x


def _cache_from_prompt(keys: torch.Tensor, values: torch.Tensor, segment_pos: torch.Tensor,
                       window: int) -> AttentionBlockCache:
  """The last min(window, T) keys / values, rolled by num_tokens mod window so that slot j holds
  the token whose position is j modulo the window, right padded with zeros
  (torch/modules.py:238-258)."""
  b, t = keys.shape[:2]
  w = min(window, t)
  num_tokens = segment_pos[:, -1] + 1
  shift = (num_tokens % window).long()
  src = (torch.arange(w, device=keys.device)[None, :] - shift[:, None]) % w       # [B, w]
  idx = (t - w + src)[:, :, None, None].expand(b, w, 1, keys.shape[-1])
  k = torch.gather(keys, 1, idx)
  v = torch.gather(values, 1, idx)
  if w < window:
    pad = torch.zeros((b, window - w, 1, keys.shape[-1]), dtype=keys.dtype, device=keys.device)
    k, v = torch.cat([k, pad], dim=1), torch.cat([v, pad], dim=1)
  return AttentionBlockCache(keys=k.contiguous(), values=v.contiguous(),
                             num_tokens=num_tokens.to(torch.int32))


class LocalAttentionBlock(nn.Module):
  """Local multi-query attention (recurrentgemma/torch/modules.py:293-493): same constructor,
  parameter names (`proj_q/k/v.weight`, `proj_final.weight/.bias`), forward and cache.  bfloat16
  prefill with head dimension 256 runs on the library (projections on the tcgen05 GEMM, rotary
  kernel, the two-pass tcgen05 attention kernel), and so does the decode step with head dimension
  256 (rotary kernel, the two ring kernels; projections of a handful of rows are library GEMMs);
  other shapes compose the rotary kernel with library contractions."""

  def __init__(self, width: int, num_heads: int, window_size: int,
               final_w_init_variance_scale: float = 1.0, device=None, dtype=None):
    super().__init__()
    self.width = width
    self.num_heads = num_heads
    self.window_size = window_size
    self.final_w_init_variance_scale = final_w_init_variance_scale
    self.proj_q = nn.Linear(self.width, self.width, bias=False, device=device, dtype=dtype)
    self.proj_k = nn.Linear(self.width, self.head_dim, bias=False, device=device, dtype=dtype)
    self.proj_v = nn.Linear(self.width, self.head_dim, bias=False, device=device, dtype=dtype)
    self.proj_final = nn.Linear(self.width, self.width, bias=True, device=device, dtype=dtype)
    self.reset_parameters()

  def reset_parameters(self) -> None:
    self.w_init_(self.proj_q.weight)
    self.w_init_(self.proj_k.weight)
    self.w_init_(self.proj_v.weight)
    self.out_w_init_(self.proj_final.weight)
    torch.nn.init.zeros_(self.proj_final.bias)

  @property
  def head_dim(self) -> int:
    return self.width // self.num_heads

  def w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0, std=math.sqrt(1.0 / self.width))

  def out_w_init_(self, w: torch.Tensor) -> None:
    torch.nn.init.normal_(w, mean=0.0, std=math.sqrt(self.final_w_init_variance_scale / self.width))

  def _linear(self, x: torch.Tensor, lin: nn.Linear) -> torch.Tensor:
    return linear(x, lin)

  @torch.no_grad()
  def forward(
      self, x: torch.Tensor, segment_pos: torch.Tensor,
      cache: Optional[AttentionBlockCache] = None, return_cache: bool = True,
      inplace: bool = False,
  ) -> Tuple[torch.Tensor, Optional[AttentionBlockCache]]:
    """Returns (block output [B,T,width], updated cache or None).  With `inplace` a decode step
    writes the new key and value into their ring slot of `cache` and bumps its `num_tokens`
    (an extension for decode loops that run as a CUDA graph) instead of cloning the ring."""
    dev = _lib.require_cuda(x, segment_pos, self.proj_q.weight)
    layers._same_dtype(x, self.proj_q.weight, self.proj_k.weight, self.proj_v.weight,
                       self.proj_final.weight, self.proj_final.bias)
    b, t, _ = x.shape
    assert segment_pos.shape == (b, t), segment_pos.shape
    n, hd, w = self.num_heads, self.head_dim, self.window_size
    q = self._linear(x, self.proj_q).view(b, t, n, hd)
    k, v = linear_pair(x, self.proj_k, self.proj_v)
    k, v = k.view(b, t, 1, hd), v.view(b, t, 1, hd)
    q, k = _rope(q.contiguous(), segment_pos), _rope(k.contiguous(), segment_pos)
    new_cache = None
    if cache is None:
      if return_cache:
        new_cache = _cache_from_prompt(k, v, segment_pos, w)
      if x.dtype == torch.bfloat16 and hd == 256:
        enc = torch.empty((b, t, n * hd), dtype=x.dtype, device=dev)
        pos = segment_pos.contiguous()
        lib = _lib.load()
        with torch.cuda.device(dev):
          ws = _lib.workspace(dev, int(lib.rgk_attention_workspace_bytes(b, t)))
          _lib.check(lib.rgk_local_attention_prefill(
              q.data_ptr(), k.data_ptr(), v.contiguous().data_ptr(), pos.data_ptr(),
              _lib.pos_code(pos), b, t, n, hd, w, _lib.dtype_code(x.dtype), enc.data_ptr(),
              ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
        return self._linear(enc, self.proj_final), new_cache
      idx = torch.arange(t, device=dev)
      start = torch.where(segment_pos == 0, idx[None, :], torch.zeros_like(segment_pos))
      start = torch.cummax(start, dim=1).values                      # start of each token's document
      lo = torch.maximum(start, idx[None, :] - w)
      visible = (idx[None, None, :] >= lo[:, :, None]) & (idx[None, None, :] <= idx[None, :, None])
      keys, values = k, v
    else:
      assert t == 1, "with a cache the block takes one token at a time"
      lib = _lib.load()
      if (hd == 256 and n in (1, 2, 4, 8, 10)
          and cache.keys.dtype == x.dtype and cache.num_tokens.dtype == torch.int32):
        # the library's decode kernels work on the ring in place; the reference's functional form
        # is the same step on a copy of the cache
        if inplace or not return_cache:
          ring = cache
          assert ring.keys.is_contiguous() and ring.values.is_contiguous()
        else:
          ring = AttentionBlockCache(keys=cache.keys.clone(), values=cache.values.clone(),
                                     num_tokens=cache.num_tokens.clone())
        enc = torch.empty((b, 1, n * hd), dtype=x.dtype, device=dev)
        with torch.cuda.device(dev):
          ws = _lib.workspace(dev, int(lib.rgk_attention_decode_workspace_bytes(b, n, w)))
          _lib.check(lib.rgk_local_attention_decode(
              q.data_ptr(), k.data_ptr(), v.contiguous().data_ptr(), ring.keys.data_ptr(),
              ring.values.data_ptr(), ring.num_tokens.data_ptr(), b, n, hd, w,
              _lib.dtype_code(x.dtype), 1 if return_cache else 0, enc.data_ptr(), ws.data_ptr(),
              ws.numel(), _lib.stream_ptr(dev)))
        return self._linear(enc, self.proj_final), (ring if return_cache else None)
      nt = cache.num_tokens.long()
      kq = nt // w
      j = torch.arange(w, device=dev)[None, :]
      now, prev = j + kq[:, None] * w, j + (kq[:, None] - 1) * w
      kpos = torch.where(now < nt[:, None], now, prev)
      vis = (kpos >= 0) & (kpos <= nt[:, None]) & (nt[:, None] <= kpos + w)
      slot = (nt % w)
      rows = torch.arange(b, device=dev)
      if inplace:
        # the ring is read where it lies (the new token's own logit and value are added beside
        # it), then the slot is overwritten: no copy of the ring
        scale = hd ** -0.5
        lg = torch.einsum("bnh,bsh->bns", q[:, 0], cache.keys[:, :, 0]) * scale
        lg_self = (q[:, 0] * k[:, 0]).sum(-1, dtype=torch.float32).to(x.dtype) * scale
        lg = torch.where(vis[:, None, :], lg, torch.full_like(lg, -2.3819763e38))
        probs = torch.softmax(torch.cat([lg, lg_self[:, :, None]], dim=-1).float(), dim=-1).to(x.dtype)
        enc = (torch.einsum("bns,bsh->bnh", probs[:, :, :w], cache.values[:, :, 0]).float()
               + probs[:, :, w:].float() * v[:, 0].float()).to(x.dtype).reshape(b, 1, n * hd)
        if return_cache:
          cache.keys[rows, slot] = k[:, 0]
          cache.values[rows, slot] = v[:, 0]
          cache.num_tokens.add_(1)
          new_cache = cache
        return self._linear(enc, self.proj_final), new_cache
      visible = torch.cat([vis, torch.ones((b, 1), dtype=torch.bool, device=dev)], dim=1)[:, None, :]
      keys = torch.cat([cache.keys, k], dim=1)
      values = torch.cat([cache.values, v], dim=1)
      if return_cache:
        nk, nv = cache.keys.clone(), cache.values.clone()
        nk[rows, slot] = k[:, 0]
        nv[rows, slot] = v[:, 0]
        new_cache = AttentionBlockCache(keys=nk, values=nv, num_tokens=cache.num_tokens + 1)
    # library contractions with the reference's roundings: logits rounded, scaled, masked, float32
    # softmax, probabilities cast back, second contraction
    logits = torch.einsum("btnh,bsh->bnts", q, keys[:, :, 0]) * (hd ** -0.5)
    masked = torch.where(visible[:, None], logits, torch.full_like(logits, -2.3819763e38))
    probs = torch.softmax(masked.float(), dim=-1).to(x.dtype)
    enc = torch.einsum("bnts,bsh->btnh", probs, values[:, :, 0]).reshape(b, t, n * hd)
    return self._linear(enc, self.proj_final), new_cache

  @classmethod
  def init_cache(cls, batch_size: int, window_size: int, heads_dim: int, dtype: torch.dtype,
                 device=None) -> AttentionBlockCache:
    """Empty cache (recurrentgemma/torch/modules.py:478-493)."""
    shape = (batch_size, window_size, 1, heads_dim)
    return AttentionBlockCache(
        keys=torch.zeros(shape, device=device, dtype=dtype),
        values=torch.zeros(shape, device=device, dtype=dtype),
        num_tokens=torch.zeros([batch_size], dtype=torch.int32, device=device))


class ResidualBlock(nn.Module):
  """Griffin's residual block (recurrentgemma/torch/modules.py:755-945): same constructor
  arguments, attribute and parameter names (`temporal_pre_norm`, `recurrent_block` or
  `attention_block`, `channel_pre_norm`, `mlp_block`), forward and cache.  `temporal_block_type`
  is "recurrent" / "attention" or a member of an enumeration with those names (the reference's
  `common.TemporalBlockType`)."""

  def __init__(self, width: int, mlp_expanded_width: int, num_heads: int,
               attention_window_size: int, temporal_block_type, lru_width: Optional[int] = None,
               conv1d_temporal_width: int = 4, final_w_init_variance_scale: float = 1.0,
               device=None, dtype=None):
    super().__init__()
    self.width = width
    self.mlp_expanded_width = mlp_expanded_width
    self.num_heads = num_heads
    self.attention_window_size = attention_window_size
    self.temporal_block_type = temporal_block_type
    self.lru_width = lru_width
    self.conv1d_temporal_width = conv1d_temporal_width
    self.final_w_init_variance_scale = final_w_init_variance_scale
    self.temporal_pre_norm = layers.RMSNorm(width, device=device, dtype=dtype)
    if block_kind(temporal_block_type) == "recurrent":
      self.recurrent_block = RecurrentBlock(
          width=width, num_heads=num_heads, lru_width=lru_width,
          conv1d_temporal_width=conv1d_temporal_width,
          final_w_init_variance_scale=final_w_init_variance_scale, device=device, dtype=dtype)
    else:
      self.attention_block = LocalAttentionBlock(
          width=width, num_heads=num_heads, window_size=attention_window_size,
          final_w_init_variance_scale=final_w_init_variance_scale, device=device, dtype=dtype)
    self.channel_pre_norm = layers.RMSNorm(width, device=device, dtype=dtype)
    self.mlp_block = MLPBlock(width, mlp_expanded_width, final_w_init_variance_scale,
                              device=device, dtype=dtype)

  def reset_parameters(self) -> None:
    self.temporal_pre_norm.reset_parameters()
    self.temporal_block.reset_parameters()
    self.channel_pre_norm.reset_parameters()
    self.mlp_block.reset_parameters()

  @property
  def temporal_block(self) -> nn.Module:
    if block_kind(self.temporal_block_type) == "recurrent":
      return self.recurrent_block
    return self.attention_block

  def forward(self, x: torch.Tensor, segment_pos: torch.Tensor, cache=None,
              return_cache: bool = True, inplace: bool = False):
    """Returns (block output [B,T,width], updated cache of the temporal block or None)."""
    return residual_block(x, segment_pos, self.temporal_pre_norm, self.temporal_block,
                          self.channel_pre_norm, self.mlp_block, cache, return_cache, inplace)

  @classmethod
  def init_cache(cls, batch_size: int, width: int, num_heads: int, attention_window_size: int,
                 temporal_block_type, dtype: torch.dtype, lru_width: Optional[int] = None,
                 conv1d_temporal_width: int = 4, device=None):
    """Empty cache of the block's kind (recurrentgemma/torch/modules.py:913-945)."""
    if block_kind(temporal_block_type) == "recurrent":
      return RecurrentBlock.init_cache(batch_size=batch_size, lru_width=lru_width or width,
                                       dtype=dtype, conv1d_temporal_width=conv1d_temporal_width,
                                       device=device)
    return LocalAttentionBlock.init_cache(batch_size=batch_size, window_size=attention_window_size,
                                          heads_dim=width // num_heads, dtype=dtype, device=device)


def block_kind(temporal_block_type) -> str:
  """"recurrent" or "attention" from a string or an enumeration member of that name."""
  name = getattr(temporal_block_type, "name", temporal_block_type)
  kind = str(name).lower()
  if kind not in ("recurrent", "attention"):
    raise ValueError(f"unknown temporal block type {temporal_block_type!r}")
  return kind


class Embedder(nn.Module):
  """Token embeddings tied to the output projection (recurrentgemma/torch/modules.py:945-1003):
  `input_embedding` [vocab_size, embed_dim]; `encode` gathers rows (scaled by sqrt(embed_dim)
  rounded to bfloat16 when `scale_by_sqrt_dim`), `decode` multiplies by the transposed table.
  `decode(x, soft_cap)` also applies Griffin's logits soft cap in the same kernel
  (recurrentgemma/torch/griffin.py:183-185)."""

  def __init__(self, vocab_size: int, embed_dim: int, scale_by_sqrt_dim: bool, device=None,
               dtype=None):
    super().__init__()
    self.vocab_size = vocab_size
    self.embed_dim = embed_dim
    self.scale_by_sqrt_dim = scale_by_sqrt_dim
    self.input_embedding = nn.Parameter(
        torch.empty([vocab_size, embed_dim], device=device, dtype=dtype))
    self.reset_parameters()

  def reset_parameters(self) -> None:
    torch.nn.init.normal_(self.input_embedding, mean=0.0, std=math.sqrt(1.0 / self.embed_dim))

  @torch.no_grad()
  def encode(self, x: torch.Tensor) -> torch.Tensor:
    """tokens [...] (int32 / int64) -> activations [..., embed_dim]."""
    table = self.input_embedding
    dev = _lib.require_cuda(x, table)
    if x.dtype not in (torch.int32, torch.int64):
      raise TypeError(f"tokens must be int32 or int64, got {x.dtype}")
    scale = 1.0
    if self.scale_by_sqrt_dim:
      scale = float(torch.tensor(math.sqrt(self.embed_dim)).type(torch.bfloat16))
    tok = x.contiguous()
    out = torch.empty((*x.shape, self.embed_dim), dtype=table.dtype, device=dev)
    with torch.cuda.device(dev):
      _lib.check(_lib.load().rgk_embed(
          tok.data_ptr(), 1 if tok.dtype == torch.int64 else 0, table.data_ptr(), tok.numel(),
          self.vocab_size, self.embed_dim, scale, _lib.dtype_code(table.dtype), out.data_ptr(),
          _lib.stream_ptr(dev)))
    return out

  @torch.no_grad()
  def decode(self, x: torch.Tensor, soft_cap: float = 0.0) -> torch.Tensor:
    """activations [..., embed_dim] -> logits [..., vocab_size] (capped when soft_cap != 0)."""
    table = self.input_embedding
    dev = _lib.require_cuda(x, table)
    layers._same_dtype(x, table)
    assert x.shape[-1] == self.embed_dim
    if x.dtype == torch.bfloat16 and self.embed_dim % 8 == 0 and self.vocab_size % 8 == 0:
      xc = x.contiguous()
      out = torch.empty((*x.shape[:-1], self.vocab_size), dtype=x.dtype, device=dev)
      with torch.cuda.device(dev):
        _lib.check(_lib.load().rgk_logits(
            xc.data_ptr(), table.data_ptr(), xc.numel() // self.embed_dim, self.embed_dim,
            self.vocab_size, float(soft_cap), _lib.dtype_code(x.dtype), out.data_ptr(),
            _lib.status_ptr(dev), _lib.stream_ptr(dev)))
      return out
    logits = x @ table.T                     # float32 and odd shapes: a library contraction
    if soft_cap:
      logits = torch.tanh(logits / soft_cap) * soft_cap
    return logits


@torch.no_grad()
def argmax(logits: torch.Tensor) -> torch.Tensor:
  """torch.argmax(logits, dim=-1) as int32 (greedy sampling,
  recurrentgemma/torch/sampler.py:131-132): the first maximum of every row."""
  dev = _lib.require_cuda(logits)
  v = logits.shape[-1]
  xc = logits.contiguous()
  out = torch.empty(logits.shape[:-1], dtype=torch.int32, device=dev)
  with torch.cuda.device(dev):
    _lib.check(_lib.load().rgk_argmax(xc.data_ptr(), xc.numel() // v, v,
                                      _lib.dtype_code(logits.dtype), out.data_ptr(),
                                      _lib.stream_ptr(dev)))
  return out
