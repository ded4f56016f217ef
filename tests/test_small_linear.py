"""The few-row (M <= 256) weight-streaming split-K GEMM of librgk against a float32 restatement of
torch.nn.Linear with the reference's roundings (recurrentgemma/torch/modules.py:531-548, 626-647,
749-752), through the C ABI.  Needs a B200."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf(t):
  return t.to(torch.bfloat16)


def _ref_linear(x, w, b, gelu=False, residual=None):
  """float32 contraction + bias, ONE rounding; gelu on the rounded value; residual add rounded."""
  y = x.float() @ w.float().t()
  if b is not None:
    y = y + b.float()
  y = _bf(y)
  if gelu:
    y = _bf(torch.nn.functional.gelu(y.float(), approximate="tanh"))
  if residual is not None:
    y = _bf(y.float() + residual.float())
  return y


def _close(got, want, what):
  """Sums are accumulated in another order than the restatement's: an element may land on the
  neighbouring bfloat16 value (a relative step of 2^-7, or 2^-8 of the row scale near zero), and
  few do."""
  g, w = got.float(), want.float()
  scale = w.abs().max().clamp_min(1e-6)
  err = ((g - w).abs() / scale).max().item()
  frac = (g != w).float().mean().item()
  assert err <= 2.0 ** -6, f"{what}: normalised max error {err:.3e}"
  assert frac <= 0.05, f"{what}: {frac:.3%} of the elements differ"


SHAPES = [(1, 2560, 2560), (3, 72, 136), (16, 2560, 2560), (64, 2560, 256), (129, 512, 2560),
          (256, 2560, 2560), (256, 7680, 2560), (5, 8, 8), (200, 4096, 4096)]


@pytest.mark.parametrize("m,k,n", SHAPES, ids=[f"m{m}_k{k}_n{n}" for m, k, n in SHAPES])
@pytest.mark.parametrize("mode", ["bias", "nobias", "gelu", "residual"])
def test_small_linear(m, k, n, mode):
  from recurrentgemma_b200 import _lib, modules
  g = torch.Generator(device="cpu").manual_seed(m * 7 + k * 3 + n)
  x = _bf(torch.randn(m, k, generator=g)).to(DEV)
  w = _bf(torch.randn(n, k, generator=g) / k ** 0.5).to(DEV)
  b = None if mode == "nobias" else _bf(torch.randn(n, generator=g) * 0.1).to(DEV)
  res = _bf(torch.randn(m, n, generator=g)).to(DEV) if mode == "residual" else None
  out = modules.small_linear(x, w, b, act=_lib.ACT_GELU_TANH if mode == "gelu" else _lib.ACT_NONE,
                             residual=res)
  _close(out, _ref_linear(x, w, b, mode == "gelu", res), f"{mode} {m}x{k}x{n}")
  # the K slices are added in a fixed order: a second call gives the same bits
  again = modules.small_linear(x, w, b, act=_lib.ACT_GELU_TANH if mode == "gelu" else _lib.ACT_NONE,
                               residual=res)
  assert torch.equal(again, out)
  _lib.check_status()


@pytest.mark.parametrize("m,k,na,nb", [(1, 2560, 2560, 2560), (16, 512, 128, 264), (256, 2560, 2560, 2560),
                                       (130, 2560, 256, 256), (7, 64, 384, 8)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_small_linear_pair(m, k, na, nb, with_bias):
  """Two projections of the same rows in one launch (linear_y / linear_x, proj_k / proj_v)."""
  from recurrentgemma_b200 import _lib, modules
  torch.manual_seed(m + k + na + nb)
  la = torch.nn.Linear(k, na, bias=with_bias, device=DEV, dtype=torch.bfloat16)
  lb = torch.nn.Linear(k, nb, bias=with_bias, device=DEV, dtype=torch.bfloat16)
  if with_bias:
    la.bias.data.normal_(0, 0.1)
    lb.bias.data.normal_(0, 0.1)
  x = _bf(torch.randn(m, k)).to(DEV)
  ya, yb = modules.small_linear_pair(x, la, lb)
  _close(ya, _ref_linear(x, la.weight, la.bias), "first of the pair")
  _close(yb, _ref_linear(x, lb.weight, lb.bias), "second of the pair")
  _lib.check_status()


@pytest.mark.parametrize("rows", [1, 16, 256])
@pytest.mark.parametrize("with_norm", [False, True])
def test_mlp_block_few_rows(rows, with_norm, monkeypatch):
  """MLPBlock below SMALL_ROWS (GeGLU and residual in the epilogues of the few-row kernel) against
  the prefill kernels of the same library on the same rows."""
  import recurrentgemma_b200 as rg
  from recurrentgemma_b200 import _lib, layers, modules
  torch.manual_seed(rows)
  mlp = rg.MLPBlock(512, 1536, device=DEV, dtype=torch.bfloat16)
  mlp.ffw_up.b.data.normal_(0, 0.1)
  mlp.ffw_down.bias.data.normal_(0, 0.1)
  mlp.invalidate_packed()
  norm = layers.RMSNorm(512, device=DEV, dtype=torch.bfloat16) if with_norm else None
  x = _bf(torch.randn(rows, 1, 512)).to(DEV)
  res = None if with_norm else _bf(torch.randn(rows, 1, 512)).to(DEV)
  monkeypatch.setattr(modules, "SMALL_ROWS_MLP", 256)
  small = mlp(x, residual=res, pre_norm=norm)
  monkeypatch.setattr(modules, "SMALL_M", 1)
  big = mlp(x, residual=res, pre_norm=norm)
  _close(small, big, f"MLP rows={rows}")
  _lib.check_status()


def test_small_linear_rejects():
  from recurrentgemma_b200 import _lib, modules
  x = torch.zeros(257, 64, dtype=torch.bfloat16, device=DEV)
  w = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
  with pytest.raises(_lib.RgkError) as e:
    modules.small_linear(x, w, None)
  assert e.value.code == _lib.RGK_ESHAPE
  with pytest.raises(_lib.RgkError) as e:
    modules.small_linear(x[:4].float(), w.float(), None)
  assert e.value.code == _lib.RGK_ESHAPE
