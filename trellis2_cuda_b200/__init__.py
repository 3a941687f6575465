"""B200-native (sm_100a) sparse convolution for SC-VAE decoders: a drop-in for the sparse-conv operator API
of suvadityamuk/trellis2-cuda (src/spconv.h and the sparse pieces of src/sdec.cu).

The operators live in libt2sc.so (CUDA, C ABI declared in include/t2sc.h); this package is the thin
Python host layer that mirrors the reference's names.  Importing works without a GPU; calling an operator
without one raises.
"""
from ._lib import T2scError  # noqa: F401
from .spconv import (  # noqa: F401
    Level, SpConvCache, SpConvCfg, act_, add_, add_skip, build_neighbors, build_neighbors_range, cache_from_map, context,
    gather_rows, layer_norm, linear, peer_barrier, subm_conv_local, subm_conv_peers, subm_conv_split,
    row_epilogue, spconv_cfg, subdiv_conv, subdivide, subm_conv, subm_conv_host, voxel_lookup,
)
