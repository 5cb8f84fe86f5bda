"""Makes tests/golden/rope_anchor.npz from the reference's committed fixtures.

The reference's model code cannot run here (it needs Apple MLX), but three of
its fixture files need no weights: ``reference/fixtures/rope_freqs.npy`` (the
llama3-scaled frequency table of Llama-3.2-1B, 32 float32) and
``q_pre0.npy`` / ``q_rope0.npy`` (queries of layer 0 before and after the
rotation, positions 0..5, float16).  This script copies the table and the first
two heads of the query pair into one small archive.

    python tests/golden/make_rope_golden.py /path/to/mlxforge/reference/fixtures
"""
import sys

import numpy as np

src = sys.argv[1]
freqs = np.load(f"{src}/rope_freqs.npy")
q_pre = np.load(f"{src}/q_pre0.npy")[0, :2]      # [2 heads, 6 positions, 64]
q_rope = np.load(f"{src}/q_rope0.npy")[0, :2]
np.savez("tests/golden/rope_anchor.npz", rope_freqs=freqs, q_pre=q_pre, q_rope=q_rope)
print(freqs.shape, q_pre.shape, q_rope.shape)
