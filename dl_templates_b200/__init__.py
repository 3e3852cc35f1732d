"""B200-native tiled 2D sliding-window attention with fused 2D RoPE.

Python call surface of the reference's ``src/tiled_swa.py`` and
``src/fused_rope2d.py`` over a C-ABI CUDA library built for sm_100a.
"""
from .fused_rope2d import (FusedInplaceRotaryPositionEncoding2D, FusedRotaryPositionEncodingContext, RotaryPE2D,
                           make_cs_table, rope2d_apply_, rope2d_apply_to)
from .host_pipeline import HostPipeline
from .spatial import (RowShard, SpatialTiledSwaRope2D, embed_rows, exchange_halo, row_range, spatial_backward,
                      spatial_forward)
from .tiled_swa import (TiledSwa, TiledSwaPackedQKV, TiledSwaRope2D, check_status, padded_head_dims, selected_impl,
                        set_rope_mode, swa_backward, swa_backward_noalloc, swa_backward_rot, swa_forward,
                        swa_forward_rot, tiled_swa_fwd)

__all__ = ["HostPipeline", "RowShard", "SpatialTiledSwaRope2D", "embed_rows", "exchange_halo", "row_range", "spatial_forward",
           "spatial_backward", "TiledSwa", "TiledSwaRope2D", "TiledSwaPackedQKV", "tiled_swa_fwd", "swa_forward", "swa_backward",
           "swa_backward_noalloc", "swa_forward_rot", "swa_backward_rot", "selected_impl", "padded_head_dims", "set_rope_mode", "check_status", "RotaryPE2D", "FusedInplaceRotaryPositionEncoding2D",
           "FusedRotaryPositionEncodingContext", "make_cs_table", "rope2d_apply_", "rope2d_apply_to"]
