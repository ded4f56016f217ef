"""B200-native (sm_100a) RG-LRU + Conv1D path for recurrentgemma's torch models.

The public names mirror `recurrentgemma.torch` for the modules on that path; `dropin` swaps them
into a reference `Griffin`.  Importing the package does not load the CUDA library; the first
forward does, and raises if it has not been built.
"""
from recurrentgemma_b200.layers import (BlockDiagonalLinear, Conv1D, Einsum, RGLRU, RMSNorm,
                                        rnn_scan)
from recurrentgemma_b200.modules import (AttentionBlockCache, Embedder, LocalAttentionBlock,
                                         MLPBlock, RecurrentBlock, RecurrentBlockCache,
                                         ResidualBlock, argmax, dense_linear, recurrent_path,
                                         recurrent_residual, residual_block)
from recurrentgemma_b200.griffin import Griffin, GriffinConfig, TemporalBlockType
from recurrentgemma_b200.sampler import GreedySampler
from recurrentgemma_b200._lib import RgkError, check_status

__all__ = [
    "BlockDiagonalLinear", "Conv1D", "Einsum", "RGLRU", "RMSNorm", "rnn_scan", "RecurrentBlock",
    "RecurrentBlockCache", "MLPBlock", "LocalAttentionBlock", "AttentionBlockCache", "ResidualBlock",
    "Embedder", "Griffin", "GriffinConfig", "TemporalBlockType", "GreedySampler", "argmax",
    "recurrent_path", "recurrent_residual", "residual_block", "dense_linear", "check_status",
    "RgkError",
]
