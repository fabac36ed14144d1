"""B200-native idxN LUT-palettized linear layer (decode GEMV, prefill GEMM, FHT).

Host side: PyTorch modules mirroring the reference's PalettizedLinear /
SplitQKV / FusedPalettizedMLP; compute: libb200lut.so (hand-written sm_100a CUDA
behind a C ABI, see include/b200_lut.h). Import of this package does not load
the library; the first compute call does, and fails loudly if it is not built.
"""
from . import _lib, fht, idxN, synthetic                                    # noqa: F401
from .palettized_modules import (FusedPalettizedMLP, KGroupedPalettizedLinear,  # noqa: F401
                                 PalettizedEmbedding, PalettizedLinear,
                                 SplitQKV,
                                 reference_dequant, set_programmatic_launch)
from .artifacts import (load_metadata, load_palettized_embedding, load_palettized_weight,  # noqa: F401
                        load_tied_pair, replace_linear_with_palettized)
from .lut_export import export_luts, import_luts, iter_palettized_linears      # noqa: F401
from .loader import load_quant_model                                             # noqa: F401
from . import flute_extended                                                     # noqa: F401

__all__ = ["load_quant_model", "load_palettized_weight", "replace_linear_with_palettized",
           "load_palettized_embedding", "load_tied_pair", "export_luts", "import_luts",
           "iter_palettized_linears", "load_metadata", "PalettizedLinear", "PalettizedEmbedding", "KGroupedPalettizedLinear", "SplitQKV", "FusedPalettizedMLP", "reference_dequant",
           "set_programmatic_launch", "fht", "idxN", "synthetic", "flute_extended"]
