"""adacode_b200 — the float11 lossless BF16 KV-cache path of AdaCode as sm_100a CUDA kernels
behind the reference's HF-transformers Cache API.

Public surface (same names as the reference package ``kv_compression``):
  ``Float11Cache``, ``float11Layer``              float_cache_utils
  ``MLAFloat11Cache``                             mla_float_cache_utils
  ``compress_tiled_tensor``, ``materialize_tiled_state``, ``TiledCompressedTensor``   codec
  ``export_initial_compress_parameters``          best_bit_analysis_kv_cache
  ``model_config_map``                            model_configs
  ``extract_exp_freq``, ``merge_exp_freq``        export_kvcache_status (exponent statistics only)
  ``CompressorBitMap``                            compress_bitmap_merge (flat codec: 'legacy' layout, weights)
  ``convert_model``                               manager (packed model weights, decoded just in time)
  ``main_lossless_comp``                          the runner (``python -m adacode_b200.main_lossless_comp``)
and, without a reference counterpart, ``decode_attention`` (attention) — one decode step of
attention computed from the packed planes.
"""
from .attention import decode_attention
from .best_bit_analysis_kv_cache import export_initial_compress_parameters
from .codec import TiledCompressedTensor, compress_tiled_tensor, materialize_tiled_state
from .compress_bitmap_merge import CompressorBitMap
from .float_cache_utils import Float11Cache, float11Layer
from .mla_float_cache_utils import MLAFloat11Cache, MLALatentFloat11DenseRopeLayer
from .manager import convert_model
from .model_configs import model_config_map

__all__ = [
    'Float11Cache', 'float11Layer', 'MLAFloat11Cache', 'MLALatentFloat11DenseRopeLayer',
    'TiledCompressedTensor', 'compress_tiled_tensor', 'materialize_tiled_state',
    'export_initial_compress_parameters', 'model_config_map', 'decode_attention', 'CompressorBitMap',
    'convert_model',
]
