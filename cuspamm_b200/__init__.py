"""B200-native SpAMM (sparse approximate matrix multiply over 32x32 tiles) behind a C ABI.

The compute path is libspamm.so (hand-written sm_100a CUDA, built from csrc/); this package is the host-side
mirror of the reference driver.  Importing the package does not load the library; creating a plan does, and
fails loudly if it cannot be built or loaded.
"""
from .engine import (  # noqa: F401
    BUF_A, BUF_B, BUF_C, BUF_COUNTS, BUF_NORM_A, BUF_NORM_B, MT_COLS, MT_ROWS, TILE,
    ShardedSpamm, SpammGroup, SpammPlan, gen_decay_alg, gen_decay_exp, gen_lattice, gen_ones, gen_signed_exp, gen_uniform,
    gen_uniform_alg, pad_to_tiles, row_blocks, balanced_row_blocks,
)
from ._lib import SpammError, SpammStats  # noqa: F401
