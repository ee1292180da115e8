"""tileops_b200: B200-native (sm_100a) GQA attention forward behind the TileOPs operator surface.

    from tileops_b200.ops import GroupedQueryAttentionDecodePagedWithKVCacheFwdOp

The operators mirror ``tileops.ops`` (tile-ai/TileOPs); the kernels are hand-written CUDA in
``tileops_b200/csrc`` reached through the C ABI of ``include/tileops_b200.h``.  Importing the
package needs neither a GPU nor the built library; launching a kernel needs both.
"""

from . import backend, manifest, ops, perf  # noqa: F401

__version__ = "0.1.0"
