"""ctypes front end of the CPU oracle in oracle/rglru_oracle.c.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU
baseline legs of ``bench.py``.  The shipped package never imports it.

Every function takes CPU torch tensors (float32 or bfloat16), hands float32 copies to the C
restatement with the matching arithmetic mode, and returns tensors in the reference's dtypes
(activations in the input dtype, recurrence state float32).  The reference lines each function
follows are cited in the C file.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "librgo.so")
_lib = None

F32, BF16 = 0, 1


def build(force: bool = False) -> str:
  """Compiles oracle/librgo.so with the Makefile beside it (gcc only)."""
  src = os.path.join(_HERE, "rglru_oracle.c")
  stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
  if force or stale:
    if force and os.path.exists(_LIB_PATH):
      os.remove(_LIB_PATH)
    subprocess.run(["make", "-C", _HERE, "librgo.so"], check=True, capture_output=True)
  return _LIB_PATH


def lib() -> ctypes.CDLL:
  global _lib
  if _lib is None:
    build()
    _lib = ctypes.CDLL(_LIB_PATH)
    _lib.rgo_version.restype = ctypes.c_int
    _lib.rgo_set_threads.restype = ctypes.c_int
    _lib.rgo_max_threads.restype = ctypes.c_int
    _lib.rgo_rglru.restype = ctypes.c_int
    _lib.rgo_recurrent_path.restype = ctypes.c_int
    _lib.rgo_recurrent_block.restype = ctypes.c_int
    _lib.rgo_residual_temporal.restype = ctypes.c_int
    _lib.rgo_mlp.restype = ctypes.c_int
    _lib.rgo_attention_block.restype = ctypes.c_int
    _lib.rgo_residual_channel.restype = ctypes.c_int
  return _lib


def set_threads(n: int) -> int:
  """Sets the OpenMP thread count of the oracle's loops (n <= 0: leave it) and returns the count in
  force.  Timed baselines call this: a launcher may have exported OMP_NUM_THREADS=1."""
  return int(lib().rgo_set_threads(int(n)))


def _mode(t: torch.Tensor) -> int:
  if t.dtype == torch.float32:
    return F32
  if t.dtype == torch.bfloat16:
    return BF16
  raise TypeError(f"oracle handles float32 and bfloat16, got {t.dtype}")


def _f(t: Optional[torch.Tensor]) -> Optional[np.ndarray]:
  if t is None:
    return None
  return np.ascontiguousarray(t.detach().to("cpu", torch.float32).numpy())


def _i64(t: torch.Tensor) -> np.ndarray:
  return np.ascontiguousarray(t.detach().to("cpu", torch.int64).numpy())


def _p(a: Optional[np.ndarray]):
  return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _out(shape, dtype=np.float32) -> np.ndarray:
  return np.empty(shape, dtype=dtype)


def _t(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
  return torch.from_numpy(a).to(dtype)


def blockdiag_linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
  """BlockDiagonalLinear.forward: x [..., H*bw], w [H,bw,bw], b [H,bw]."""
  dt = _mode(x)
  h, bw, _ = w.shape
  xf = _f(x).reshape(-1, h * bw)
  out = _out(xf.shape)
  lib().rgo_blockdiag_linear(_p(xf), _p(_f(w)), _p(_f(b)), ctypes.c_int64(xf.shape[0]), h, bw, dt,
                             _p(out))
  return _t(out.reshape(x.shape), x.dtype)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
  """nn.Linear: weight [N,K]."""
  dt = _mode(x)
  n, k = weight.shape
  xf = _f(x).reshape(-1, k)
  out = _out((xf.shape[0], n))
  lib().rgo_linear(_p(xf), _p(_f(weight)), _p(_f(bias)), ctypes.c_int64(xf.shape[0]), k, n, dt,
                   _p(out))
  return _t(out.reshape(*x.shape[:-1], n), x.dtype)


def conv1d(
    x: torch.Tensor, segment_pos: torch.Tensor, w: torch.Tensor, b: torch.Tensor,
    cache: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
  """Conv1D.forward: prefill when cache is None, else the single-token decode step."""
  dt = _mode(x)
  bsz, t, e = x.shape
  wd = w.shape[0]
  out = _out((bsz, t, e))
  new_cache = _out((bsz, wd - 1, e))
  if cache is None:
    lib().rgo_conv1d_prefill(_p(_f(x)), _p(_i64(segment_pos)), _p(_f(w)), _p(_f(b)), bsz, t, e, wd,
                             dt, _p(out), _p(new_cache))
    return _t(out, x.dtype), _t(new_cache, x.dtype)
  if t != 1:
    raise AssertionError("decode takes exactly one token (layers.py:549)")
  # The cache is first cast to the activation dtype, the new cache back to its own dtype
  # (layers.py:474, 526, 550).
  cache_x = cache.to(x.dtype)
  lib().rgo_conv1d_decode(_p(_f(x)), _p(_f(cache_x)), _p(_f(w)), _p(_f(b)), bsz, e, wd, dt,
                          _p(out), _p(new_cache))
  return _t(out, x.dtype), _t(new_cache, cache.dtype)


def rnn_scan(
    x: torch.Tensor, a: torch.Tensor, reset: torch.Tensor, h0: Optional[torch.Tensor],
) -> Tuple[torch.Tensor, torch.Tensor]:
  """rnn_scan: returns (y in x.dtype, last state float32)."""
  dt = _mode(x)
  bsz, t, e = x.shape
  y = _out((bsz, t, e))
  h = _out((bsz, e))
  r = np.ascontiguousarray(reset.detach().cpu().numpy().astype(np.uint8))
  lib().rgo_rnn_scan(_p(_f(x)), _p(_f(a)), _p(r), _p(_f(h0)), bsz, t, e, dt, _p(y), _p(h))
  return _t(y, x.dtype), _t(h, torch.float32)


def jax_linear_scan(x: torch.Tensor, a: torch.Tensor, h0: Optional[torch.Tensor]):
  """Restatement of recurrentgemma/jax/scan.py lru_linear_scan (a already reset-masked)."""
  dt = _mode(x)
  bsz, t, e = x.shape
  y = _out((bsz, t, e))
  h = _out((bsz, e))
  lib().rgo_jax_linear_scan(_p(_f(x)), _p(_f(a)), _p(_f(h0)), bsz, t, e, dt, _p(y), _p(h))
  return _t(y, x.dtype), _t(h, torch.float32)


def rglru(
    x: torch.Tensor, segment_pos: torch.Tensor, a_param: torch.Tensor,
    wx: torch.Tensor, bx: torch.Tensor, wa: torch.Tensor, ba: torch.Tensor,
    h0: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
  """RGLRU.forward: returns (y, last state float32)."""
  dt = _mode(x)
  bsz, t, e = x.shape
  heads = wx.shape[0]
  y = _out((bsz, t, e))
  h = _out((bsz, e))
  rc = lib().rgo_rglru(_p(_f(x)), _p(_i64(segment_pos)), _p(_f(a_param)), _p(_f(wx)), _p(_f(bx)),
                       _p(_f(wa)), _p(_f(ba)), _p(_f(h0)), bsz, t, e, heads, dt, _p(y), _p(h))
  if rc:
    raise MemoryError("oracle scratch allocation failed")
  return _t(y, x.dtype), _t(h, torch.float32)


def gelu_mul(y: torch.Tensor, y_branch: torch.Tensor) -> torch.Tensor:
  dt = _mode(y)
  out = _out(tuple(y.shape))
  lib().rgo_gelu_mul(_p(_f(y)), _p(_f(y_branch)), ctypes.c_int64(y.numel()), dt, _p(out))
  return _t(out, y.dtype)


def recurrent_path(
    xb: torch.Tensor, yb: torch.Tensor, segment_pos: torch.Tensor, p: dict,
    h0: Optional[torch.Tensor] = None, conv_cache: Optional[torch.Tensor] = None,
):
  """RGLRU(Conv1D(xb)) * gelu(yb) with the parameter dict of ``params_of`` below.

  Returns (out, rg_lru_state float32, conv1d_state).
  """
  dt = _mode(xb)
  bsz, t, e = xb.shape
  heads = p["gate_x_w"].shape[0]
  wd = p["conv_w"].shape[0]
  out = _out((bsz, t, e))
  h = _out((bsz, e))
  cc = _out((bsz, wd - 1, e))
  cache_in = None if conv_cache is None else _f(conv_cache.to(xb.dtype))
  rc = lib().rgo_recurrent_path(
      _p(_f(xb)), _p(_f(yb)), _p(_i64(segment_pos)), _p(_f(p["conv_w"])), _p(_f(p["conv_b"])),
      _p(_f(p["a_param"])), _p(_f(p["gate_x_w"])), _p(_f(p["gate_x_b"])), _p(_f(p["gate_a_w"])),
      _p(_f(p["gate_a_b"])), _p(_f(h0)), _p(cache_in), bsz, t, e, heads, wd, dt, _p(out), _p(h),
      _p(cc))
  if rc:
    raise RuntimeError(f"oracle recurrent_path failed ({rc})")
  cdt = xb.dtype if conv_cache is None else conv_cache.dtype
  return _t(out, xb.dtype), _t(h, torch.float32), _t(cc, cdt)


def recurrent_block(
    x: torch.Tensor, segment_pos: torch.Tensor, p: dict,
    h0: Optional[torch.Tensor] = None, conv_cache: Optional[torch.Tensor] = None,
):
  """RecurrentBlock.forward.  Returns (out, rg_lru_state float32, conv1d_state)."""
  dt = _mode(x)
  bsz, t, d = x.shape
  e = p["linear_x_w"].shape[0]
  heads = p["gate_x_w"].shape[0]
  wd = p["conv_w"].shape[0]
  out = _out((bsz, t, d))
  h = _out((bsz, e))
  cc = _out((bsz, wd - 1, e))
  cache_in = None if conv_cache is None else _f(conv_cache.to(x.dtype))
  rc = lib().rgo_recurrent_block(
      _p(_f(x)), _p(_i64(segment_pos)), _p(_f(p["linear_y_w"])), _p(_f(p["linear_y_b"])),
      _p(_f(p["linear_x_w"])), _p(_f(p["linear_x_b"])), _p(_f(p["linear_out_w"])),
      _p(_f(p["linear_out_b"])), _p(_f(p["conv_w"])), _p(_f(p["conv_b"])), _p(_f(p["a_param"])),
      _p(_f(p["gate_x_w"])), _p(_f(p["gate_x_b"])), _p(_f(p["gate_a_w"])), _p(_f(p["gate_a_b"])),
      _p(_f(h0)), _p(cache_in), bsz, t, d, e, heads, wd, dt, _p(out), _p(h), _p(cc))
  if rc:
    raise RuntimeError(f"oracle recurrent_block failed ({rc})")
  cdt = x.dtype if conv_cache is None else conv_cache.dtype
  return _t(out, x.dtype), _t(h, torch.float32), _t(cc, cdt)


def rmsnorm(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  """RMSNorm.forward over the last dimension."""
  d = x.shape[-1]
  m = x.numel() // d
  out = _out(tuple(x.shape))
  lib().rgo_rmsnorm(_p(_f(x)), _p(_f(scale)), ctypes.c_int64(m), d, ctypes.c_float(eps), _mode(x),
                    _p(out))
  return _t(out, x.dtype)


def residual_temporal(
    x: torch.Tensor, segment_pos: torch.Tensor, norm_scale: torch.Tensor, p: dict,
    h0: Optional[torch.Tensor] = None, conv_cache: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
):
  """recurrent_block(rmsnorm(x)) + x.  Returns (out, rg_lru_state float32, conv1d_state)."""
  dt = _mode(x)
  bsz, t, d = x.shape
  e = p["linear_x_w"].shape[0]
  heads = p["gate_x_w"].shape[0]
  wd = p["conv_w"].shape[0]
  out = _out((bsz, t, d))
  h = _out((bsz, e))
  cc = _out((bsz, wd - 1, e))
  cache_in = None if conv_cache is None else _f(conv_cache.to(x.dtype))
  rc = lib().rgo_residual_temporal(
      _p(_f(x)), _p(_i64(segment_pos)), _p(_f(norm_scale)), ctypes.c_float(eps),
      _p(_f(p["linear_y_w"])), _p(_f(p["linear_y_b"])),
      _p(_f(p["linear_x_w"])), _p(_f(p["linear_x_b"])), _p(_f(p["linear_out_w"])),
      _p(_f(p["linear_out_b"])), _p(_f(p["conv_w"])), _p(_f(p["conv_b"])), _p(_f(p["a_param"])),
      _p(_f(p["gate_x_w"])), _p(_f(p["gate_x_b"])), _p(_f(p["gate_a_w"])), _p(_f(p["gate_a_b"])),
      _p(_f(h0)), _p(cache_in), bsz, t, d, e, heads, wd, dt, _p(out), _p(h), _p(cc))
  if rc:
    raise RuntimeError(f"oracle residual_temporal failed ({rc})")
  cdt = x.dtype if conv_cache is None else conv_cache.dtype
  return _t(out, x.dtype), _t(h, torch.float32), _t(cc, cdt)


def mlp(x: torch.Tensor, w_up: torch.Tensor, b_up: torch.Tensor, w_down: torch.Tensor,
        b_down: torch.Tensor) -> torch.Tensor:
  """MLPBlock.forward: w_up [2, D, X], b_up [2, 1, 1, X] (or [2, X]), w_down [D, X], b_down [D]."""
  d = x.shape[-1]
  m = x.numel() // d
  xw = w_up.shape[-1]
  out = _out(tuple(x.shape))
  rc = lib().rgo_mlp(_p(_f(x)), _p(_f(w_up)), _p(_f(b_up.reshape(2, xw))), _p(_f(w_down)),
                     _p(_f(b_down)), ctypes.c_int64(m), d, xw, _mode(x), _p(out))
  if rc:
    raise RuntimeError(f"oracle mlp failed ({rc})")
  return _t(out, x.dtype)


def residual_channel(residual: torch.Tensor, norm_scale: torch.Tensor, w_up: torch.Tensor,
                     b_up: torch.Tensor, w_down: torch.Tensor, b_down: torch.Tensor,
                     eps: float = 1e-6) -> torch.Tensor:
  """mlp_block(channel_pre_norm(residual)) + residual."""
  d = residual.shape[-1]
  m = residual.numel() // d
  xw = w_up.shape[-1]
  out = _out(tuple(residual.shape))
  rc = lib().rgo_residual_channel(
      _p(_f(residual)), _p(_f(norm_scale)), ctypes.c_float(eps), _p(_f(w_up)),
      _p(_f(b_up.reshape(2, xw))), _p(_f(w_down)), _p(_f(b_down)), ctypes.c_int64(m), d, xw,
      _mode(residual), _p(out))
  if rc:
    raise RuntimeError(f"oracle residual_channel failed ({rc})")
  return _t(out, residual.dtype)


def attention_block(x: torch.Tensor, segment_pos: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor,
                    wv: torch.Tensor, wf: torch.Tensor, bf: torch.Tensor, num_heads: int,
                    window: int, cache=None):
  """LocalAttentionBlock.forward.  cache: None (prefill) or (keys [B,W,1,Hd], values, num_tokens [B]).
  Returns (out, (keys, values, num_tokens int32))."""
  bsz, t, d = x.shape
  hd = d // num_heads
  out = _out((bsz, t, d))
  nk, nv = _out((bsz, window, hd)), _out((bsz, window, hd))
  nn_ = np.zeros((bsz,), dtype=np.int64)
  if cache is None:
    ck = cv = cn = None
  else:
    ck = _f(cache[0].reshape(bsz, window, hd))
    cv = _f(cache[1].reshape(bsz, window, hd))
    cn = _i64(cache[2])
  rc = lib().rgo_attention_block(
      _p(_f(x)), _p(_i64(segment_pos)), _p(_f(wq)), _p(_f(wk)), _p(_f(wv)), _p(_f(wf)), _p(_f(bf)),
      _p(ck), _p(cv), _p(cn), bsz, t, d, num_heads, window, _mode(x), _p(out), _p(nk), _p(nv),
      _p(nn_))
  if rc:
    raise RuntimeError(f"oracle attention_block failed ({rc})")
  return _t(out, x.dtype), (_t(nk, x.dtype).reshape(bsz, window, 1, hd),
                            _t(nv, x.dtype).reshape(bsz, window, 1, hd),
                            torch.from_numpy(nn_).to(torch.int32))


def params_of(state_dict: dict, prefix: str = "") -> dict:
  """Maps a RecurrentBlock (or RGLRU / Conv1D) state_dict to the oracle's parameter names."""
  names = {
      "linear_y_w": "linear_y.weight", "linear_y_b": "linear_y.bias",
      "linear_x_w": "linear_x.weight", "linear_x_b": "linear_x.bias",
      "linear_out_w": "linear_out.weight", "linear_out_b": "linear_out.bias",
      "conv_w": "conv_1d.w", "conv_b": "conv_1d.b",
      "a_param": "rg_lru.a_param",
      "gate_x_w": "rg_lru.input_gate.w", "gate_x_b": "rg_lru.input_gate.b",
      "gate_a_w": "rg_lru.a_gate.w", "gate_a_b": "rg_lru.a_gate.b",
  }
  return {k: state_dict[prefix + v] for k, v in names.items() if prefix + v in state_dict}


def embed(tokens: torch.Tensor, table: torch.Tensor, scale_by_sqrt_dim: bool) -> torch.Tensor:
  """Embedder.encode (modules.py:991-998): rows of the table, times sqrt(width) rounded to bfloat16."""
  x = _f(table)[tokens.numpy().astype(np.int64)]
  if scale_by_sqrt_dim:
    scale = float(torch.tensor(float(np.sqrt(table.shape[1]))).to(torch.bfloat16))
    x = x * np.float32(scale)
  return _t(x, table.dtype)


def logits(x: torch.Tensor, table: torch.Tensor, soft_cap: float) -> torch.Tensor:
  """Embedder.decode and the soft cap (modules.py:1001-1003, griffin.py:180-185): each of the
  contraction, the division, the tanh and the product is one tensor operation of the reference,
  rounded to the activation dtype."""
  out = linear(x, table, None)
  if soft_cap:
    r = lambda a: _f(_t(a, x.dtype))            # round to the activation dtype, back to float32
    q = r(_f(out) / np.float32(soft_cap))
    out = _t(r(np.tanh(q.astype(np.float64)).astype(np.float32)) * np.float32(soft_cap), x.dtype)
  return out


def griffin(sd: dict, block_kinds, num_heads: int, window: int, soft_cap: float,
            tokens: torch.Tensor, segment_pos: torch.Tensor, cache=None):
  """Griffin.forward (griffin.py:136-194) from the pieces above.  sd: the model's state_dict;
  cache: None or {"blocks.i": (h, conv) | (keys, values, num_tokens)}.  Returns (logits, cache)."""
  x = embed(tokens, sd["embedder.input_embedding"], True)
  new_cache = {}
  for i, kind in enumerate(block_kinds):
    pre = f"blocks.{i}."
    p = {k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}
    mlp_p = (p["channel_pre_norm.scale"], p["mlp_block.ffw_up.w"], p["mlp_block.ffw_up.b"],
             p["mlp_block.ffw_down.weight"], p["mlp_block.ffw_down.bias"])
    c = None if cache is None else cache[pre[:-1]]
    if kind == "recurrent":
      op = params_of(p, "recurrent_block.")
      h0, conv = (None, None) if c is None else c
      r, h, conv = residual_temporal(x, segment_pos, p["temporal_pre_norm.scale"], op, h0, conv)
      new_cache[pre[:-1]] = (h, conv)
    else:
      w = tuple(p["attention_block." + k] for k in ("proj_q.weight", "proj_k.weight",
                                                    "proj_v.weight", "proj_final.weight",
                                                    "proj_final.bias"))
      y, ac = attention_block(rmsnorm(x, p["temporal_pre_norm.scale"]), segment_pos, *w, num_heads,
                              window, c)
      r = (y.float() + x.float()).to(x.dtype)
      new_cache[pre[:-1]] = ac
    x = residual_channel(r, *mlp_p)
  return logits(rmsnorm(x, sd["final_norm.scale"]), sd["embedder.input_embedding"], soft_cap), new_cache
