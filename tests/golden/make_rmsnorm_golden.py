"""Makes tests/golden/rmsnorm_anchor.npz from the reference's committed fixtures.

``reference/fixtures/embeddings.npy`` and ``attn_norm0.npy`` are the input and the output of
layer 0's first RMSNorm of Llama-3.2-1B for six positions (float16, [1, 6, 2048]).  The norm's
weight is not among the fixtures, but it is the same vector for every position, so the weight that
position 0 implies must reproduce positions 1..5: that pins the formula (mean over the channel
axis, eps inside the root, the weight multiplying directly) without any checkpoint.

    python tests/golden/make_rmsnorm_golden.py /path/to/mlxforge/reference/fixtures
"""
import sys

import numpy as np

src = sys.argv[1]
x = np.load(f"{src}/embeddings.npy")[0]          # [6, 2048] float16
y = np.load(f"{src}/attn_norm0.npy")[0]
np.savez_compressed("tests/golden/rmsnorm_anchor.npz", x=x, y=y)
print(x.shape, y.shape, x.dtype)
